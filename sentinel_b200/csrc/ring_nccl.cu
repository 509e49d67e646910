// Sequence-sharded causal attention over a ring of GPUs, behind the C ABI (sntl_ring_*).
//
// The reference has no sequence-parallel path; this is the long-context schedule of this library for C / C++ hosts.
// It is the schedule sentinel_b200/ring.py documents and its CPU tests pin (zigzag deal of half-shards, W steps with
// two block units per rank per step, log-sum-exp merges forward, travelling fp32 dK/dV accumulators backward whose hop
// runs under the next step's kernels), written against NCCL directly:
//
//   * K/V chunks and the dK/dV accumulators move with grouped ncclSend / ncclRecv on a communication stream of the
//     handle's own, ordered against the compute streams with events; received data lands in local HBM first and is then
//     read by ordinary per-CTA TMA loads (no kernel here ever reads a peer's memory);
//   * the K/V chunks do not wait for anybody's kernels: all world - 1 hops of their journey are posted at the start of a
//     call, each into a receive set of its own, and run back to back at link speed (the Python schedule posts one hop per
//     step instead); the accumulators, which need every rank's contribution on the way, still hop once per step;
//   * the two block pairs of a step run on two compute streams (the caller's and one of the handle's), so that the
//     last, partly filled wave of CTAs of one launch is covered by the other;
//   * nothing is allocated per call: every buffer is carved from the caller's workspace
//     (sntl_ring_attn_workspace_bytes); streams and events are created with the handle.
//
// NCCL is not a link dependency of the library: libnccl.so.2 is opened at run time when the first ring handle is made,
// so hosts that never use the ring need no NCCL at all.
#include "common.cuh"

#include <dlfcn.h>
#include <math.h>
#include <nccl.h>
#include <string.h>

#include <mutex>
#include <new>

namespace sntl {

// ---- small kernels of this file ----
__global__ void fill_f32_kernel(float* __restrict__ p, float value, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = value;
}
namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    bool ok = false;
};

NcclApi& nccl()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // a process that already loaded NCCL (for instance through its deep-learning framework) gets that copy
        api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!api.handle) return;
        auto sym = [&](const char* name) { return dlsym(api.handle, name); };
        api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
        api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
        api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
        api.Send = (decltype(api.Send))sym("ncclSend");
        api.Recv = (decltype(api.Recv))sym("ncclRecv");
        api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
        api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.Send && api.Recv && api.GroupStart && api.GroupEnd;
    });
    return api;
}

inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }
constexpr int kMaxWorld = 64;     // ranks of one ring

}  // namespace
}  // namespace sntl

using namespace sntl;

struct sntl_ring_comm {
    ncclComm_t comm = nullptr;
    bool owns_comm = false;
    int rank = 0, world = 1, device = 0;
    cudaStream_t comm_stream = nullptr, side_stream = nullptr;
    cudaEvent_t ev_main = nullptr, ev_side = nullptr, ev_acc = nullptr, ev_deal = nullptr;
    cudaEvent_t* ev_hop = nullptr;   // [world - 1]: K/V of step h + 1 have arrived
};

namespace sntl {
namespace {

// Everything one call touches, carved from the caller's workspace.  Sizes in elements of one chunk (half a shard).
struct Ring {
    sntl_ring_comm* c;
    bool zigzag;                  // the caller's shards are the two zigzag chunks already (SNTL_FLAG_RING_ZIGZAG)
    int B, Hq, Hkv, Sc, D;        // Sc = tokens per chunk
    float scale;
    size_t n_q, n_kv, n_l;        // elements per chunk of a Q-like tensor, a K-like tensor, an LSE-like tensor
    // zigzag-dealt tensors (two chunks each)
    __nv_bfloat16 *qz[2], *kz[2], *vz[2], *oz[2], *doz[2];
    float* lsez[2];
    // staging for the deal (room for both halves of a tensor: either may leave, and either work chunk may arrive)
    __nv_bfloat16 *st_q, *st_k, *st_v, *st_o, *st_do;
    float* st_l;
    __nv_bfloat16* kvbuf[kMaxWorld][4];   // world - 1 receive sets of (k0, k1, v0, v1): one per hop of the K/V chain
    // forward
    float *o_acc[2], *lse_acc[2];
    __nv_bfloat16* o_part[2];
    float* lse_part[2];
    // backward
    void* pieces[2];
    size_t pieces_bytes;
    float* part[3][2];            // per pair slot: dK, dV partial
    float* acc[3][4];             // travelling accumulators: three rotating sets of (dk0, dk1, dv0, dv1)
    __nv_bfloat16 *dqz[2], *dkz[2], *dvz[2];
    size_t total;
};

size_t pieces_bytes_for(int B, int Hq, int Sc, int D)
{
    const size_t sq_pad = ((size_t)Sc + 127) / 128 * 128;
    const size_t rows = (size_t)B * Hq * sq_pad;
    return up256(kBwdRowAuxBytes * rows) + up256(4 * rows * (size_t)D);
}

// Lays the buffers out from `base` (null: only sizes are wanted).
void lay_out(Ring& r, char* base)
{
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char* p = base ? base + off : nullptr;
        off += up256(bytes);
        return p;
    };
    for (int i = 0; i < 2; ++i) {
        r.qz[i] = (__nv_bfloat16*)take(2 * r.n_q);
        r.oz[i] = (__nv_bfloat16*)take(2 * r.n_q);
        r.doz[i] = (__nv_bfloat16*)take(2 * r.n_q);
        r.kz[i] = (__nv_bfloat16*)take(2 * r.n_kv);
        r.vz[i] = (__nv_bfloat16*)take(2 * r.n_kv);
        r.lsez[i] = (float*)take(4 * r.n_l);
    }
    r.st_q = (__nv_bfloat16*)take(2 * 2 * r.n_q);
    r.st_o = (__nv_bfloat16*)take(2 * 2 * r.n_q);
    r.st_do = (__nv_bfloat16*)take(2 * 2 * r.n_q);
    r.st_k = (__nv_bfloat16*)take(2 * 2 * r.n_kv);
    r.st_v = (__nv_bfloat16*)take(2 * 2 * r.n_kv);
    r.st_l = (float*)take(2 * 4 * r.n_l);
    for (int s = 0; s + 1 < r.c->world; ++s)
        for (int i = 0; i < 4; ++i) r.kvbuf[s][i] = (__nv_bfloat16*)take(2 * r.n_kv);
    // forward-only and backward-only buffers share one region: a call is one or the other
    const size_t shared0 = off;
    for (int i = 0; i < 2; ++i) {
        r.o_acc[i] = (float*)take(4 * r.n_q);
        r.lse_acc[i] = (float*)take(4 * r.n_l);
        r.o_part[i] = (__nv_bfloat16*)take(2 * r.n_q);
        r.lse_part[i] = (float*)take(4 * r.n_l);
    }
    const size_t fwd_end = off;
    off = shared0;
    r.pieces_bytes = pieces_bytes_for(r.B, r.Hq, r.Sc, r.D);
    for (int i = 0; i < 2; ++i) r.pieces[i] = take(r.pieces_bytes);
    for (int s = 0; s < 3; ++s) {
        r.part[s][0] = (float*)take(4 * r.n_kv);
        r.part[s][1] = (float*)take(4 * r.n_kv);
        for (int i = 0; i < 4; ++i) r.acc[s][i] = (float*)take(4 * r.n_kv);
    }
    for (int i = 0; i < 2; ++i) {
        r.dqz[i] = (__nv_bfloat16*)take(2 * r.n_q);
        r.dkz[i] = (__nv_bfloat16*)take(2 * r.n_kv);
        r.dvz[i] = (__nv_bfloat16*)take(2 * r.n_kv);
    }
    r.total = off > fwd_end ? off : fwd_end;
}

int validate_ring(const sntl_ring_comm* c, const sntl_attn_desc* d)
{
    if (!c || !d) return SNTL_ERR_BAD_ARGUMENT;
    if (c->world > kMaxWorld) return SNTL_ERR_UNSUPPORTED;
    if (d->dtype != SNTL_DTYPE_BF16 || d->layout != SNTL_LAYOUT_BHSD) return SNTL_ERR_UNSUPPORTED;
    if (d->batch <= 0 || d->q_heads <= 0 || d->kv_heads <= 0 || d->seq_q <= 0 || d->q_heads % d->kv_heads != 0) return SNTL_ERR_BAD_ARGUMENT;
    if (d->seq_kv != d->seq_q || !d->causal) return SNTL_ERR_BAD_ARGUMENT;     // every rank holds seq_q tokens of one causal sequence
    if (d->seq_q % 2 != 0) return SNTL_ERR_BAD_ARGUMENT;                       // the shard is dealt as two half-shards
    if (d->head_dim != 64 && d->head_dim != 128) return SNTL_ERR_UNSUPPORTED;
    if (d->window_size > 0 || d->global_tokens > 0 || (d->flags & (SNTL_FLAG_FORCE_SIMT | SNTL_FLAG_DETERMINISTIC))) return SNTL_ERR_UNSUPPORTED;
    if (!(d->scale > 0.0f)) return SNTL_ERR_BAD_ARGUMENT;
    return SNTL_OK;
}

void make_ring(Ring& r, sntl_ring_comm* c, const sntl_attn_desc* d, void* workspace)
{
    r.c = c;
    r.zigzag = (d->flags & SNTL_FLAG_RING_ZIGZAG) != 0;
    r.B = d->batch; r.Hq = d->q_heads; r.Hkv = d->kv_heads; r.Sc = d->seq_q / 2; r.D = d->head_dim;
    r.scale = d->scale;
    r.n_q = (size_t)r.B * r.Hq * r.Sc * r.D;
    r.n_kv = (size_t)r.B * r.Hkv * r.Sc * r.D;
    r.n_l = (size_t)r.B * r.Hq * r.Sc;
    lay_out(r, (char*)workspace);
}

struct Fail {
    int status = SNTL_OK;
    void cuda(cudaError_t e) { if (e != cudaSuccess && status == SNTL_OK) status = SNTL_ERR_CUDA; }
    void nccl(ncclResult_t e) { if (e != ncclSuccess && status == SNTL_OK) status = SNTL_ERR_COMM; }
    bool bad() const { return status != SNTL_OK; }
};

inline int owner_zigzag(int chunk, int world) { return chunk < world ? chunk : 2 * world - 1 - chunk; }

// One tensor of the zigzag deal.  x: this rank's contiguous shard, `slabs` slabs of 2*Sc rows of row_bytes.  Chunk
// 2r is the first half of every slab, 2r+1 the second.  This rank works on chunks (r, 2W-1-r) -> z[0], z[1].
struct DealItem {
    const char* x; char* z[2]; char* staging; int slabs; size_t row_bytes;
};

// Posts the copies (on `main`) and the grouped transfers (on the communication stream) of a deal of several tensors,
// and makes `main` wait for them.  reverse = false: contiguous shard -> zigzag chunks; true: the way back
// (then x is the OUTPUT shard, written from z and from what arrives).
void deal(Ring& r, DealItem* items, int n, bool reverse, cudaStream_t main, Fail& f)
{
    sntl_ring_comm* c = r.c;
    const int W = c->world, me = c->rank;
    const int mine[2] = {2 * me, 2 * me + 1};            // chunks of the contiguous shard
    const int work[2] = {me, 2 * W - 1 - me};            // chunks this rank works on
    NcclApi& api = nccl();
    if (r.zigzag) {
        // the shard is the two chunks this rank works on, one after the other inside every slab: a local (un)packing
        for (int t = 0; t < n; ++t) {
            DealItem& it = items[t];
            const size_t chunk_bytes = (size_t)r.Sc * it.row_bytes, pitch = 2 * chunk_bytes;
            for (int h = 0; h < 2; ++h) {
                char* half = const_cast<char*>(it.x) + (size_t)h * chunk_bytes;
                if (!reverse) f.cuda(cudaMemcpy2DAsync(it.z[h], chunk_bytes, half, pitch, chunk_bytes, it.slabs, cudaMemcpyDeviceToDevice, main));
                else f.cuda(cudaMemcpy2DAsync(half, pitch, it.z[h], chunk_bytes, chunk_bytes, it.slabs, cudaMemcpyDeviceToDevice, main));
            }
        }
        return;
    }
    // 1. local copies and packing of what leaves
    for (int t = 0; t < n; ++t) {
        DealItem& it = items[t];
        const size_t chunk_bytes = (size_t)r.Sc * it.row_bytes, pitch = 2 * chunk_bytes;
        for (int h = 0; h < 2; ++h) {                    // half h of the contiguous shard = chunk mine[h]
            int slot = -1;
            for (int s = 0; s < 2; ++s) if (work[s] == mine[h]) slot = s;
            char* half = const_cast<char*>(it.x) + (size_t)h * chunk_bytes;
            if (slot >= 0) {
                if (!reverse) f.cuda(cudaMemcpy2DAsync(it.z[slot], chunk_bytes, half, pitch, chunk_bytes, it.slabs, cudaMemcpyDeviceToDevice, main));
                else f.cuda(cudaMemcpy2DAsync(half, pitch, it.z[slot], chunk_bytes, chunk_bytes, it.slabs, cudaMemcpyDeviceToDevice, main));
            } else if (!reverse) {
                f.cuda(cudaMemcpy2DAsync(it.staging + (size_t)h * chunk_bytes * it.slabs, chunk_bytes, half, pitch, chunk_bytes, it.slabs,
                                         cudaMemcpyDeviceToDevice, main));
            }
        }
    }
    if (W > 1) {
        f.cuda(cudaEventRecord(c->ev_deal, main));
        f.cuda(cudaStreamWaitEvent(c->comm_stream, c->ev_deal, 0));
        f.nccl(api.GroupStart());
        for (int t = 0; t < n; ++t) {
            DealItem& it = items[t];
            const size_t chunk_bytes = (size_t)r.Sc * it.row_bytes * it.slabs;
            if (!reverse) {
                // the half this rank does not work on goes to its zigzag owner; the chunk it lacks comes from its contiguous owner
                for (int h = 0; h < 2; ++h)
                    if (mine[h] != work[0] && mine[h] != work[1])
                        f.nccl(api.Send(it.staging + (size_t)h * chunk_bytes, chunk_bytes, ncclInt8, owner_zigzag(mine[h], W), c->comm, c->comm_stream));
                for (int s = 0; s < 2; ++s)
                    if (work[s] != mine[0] && work[s] != mine[1]) f.nccl(api.Recv(it.z[s], chunk_bytes, ncclInt8, work[s] / 2, c->comm, c->comm_stream));
            } else {
                for (int s = 0; s < 2; ++s)
                    if (work[s] != mine[0] && work[s] != mine[1]) f.nccl(api.Send(it.z[s], chunk_bytes, ncclInt8, work[s] / 2, c->comm, c->comm_stream));
                for (int h = 0; h < 2; ++h)
                    if (mine[h] != work[0] && mine[h] != work[1])
                        f.nccl(api.Recv(it.staging + (size_t)h * chunk_bytes, chunk_bytes, ncclInt8, owner_zigzag(mine[h], W), c->comm, c->comm_stream));
            }
        }
        f.nccl(api.GroupEnd());
        f.cuda(cudaEventRecord(c->ev_deal, c->comm_stream));
        f.cuda(cudaStreamWaitEvent(main, c->ev_deal, 0));
        if (reverse) {
            // unpack what arrived into its half of the output shard
            for (int t = 0; t < n; ++t) {
                DealItem& it = items[t];
                const size_t chunk_bytes = (size_t)r.Sc * it.row_bytes, pitch = 2 * chunk_bytes;
                for (int h = 0; h < 2; ++h)
                    if (mine[h] != work[0] && mine[h] != work[1])
                        f.cuda(cudaMemcpy2DAsync(const_cast<char*>(it.x) + (size_t)h * chunk_bytes, pitch, it.staging + (size_t)h * chunk_bytes * it.slabs,
                                                 chunk_bytes, chunk_bytes, it.slabs, cudaMemcpyDeviceToDevice, main));
            }
        }
    }
}
// (A rank keeps at most one of its halves: chunk 2r or 2r+1 coincides with r or 2W-1-r for at most one of them when
// W > 1, and for most ranks with neither -- hence staging for both halves.)

// Posts the ring shift of `count` buffers of `bytes` each: send[i] to rank+1, recv[i] from rank-1, after `after`.
void rotate(Ring& r, void* const* send, void* const* recv, int count, size_t bytes, cudaEvent_t after, cudaEvent_t done, Fail& f)
{
    sntl_ring_comm* c = r.c;
    NcclApi& api = nccl();
    const int nxt = (c->rank + 1) % c->world, prv = (c->rank + c->world - 1) % c->world;
    f.cuda(cudaStreamWaitEvent(c->comm_stream, after, 0));
    f.nccl(api.GroupStart());
    for (int i = 0; i < count; ++i) f.nccl(api.Send(send[i], bytes, ncclInt8, nxt, c->comm, c->comm_stream));
    for (int i = 0; i < count; ++i) f.nccl(api.Recv(recv[i], bytes, ncclInt8, prv, c->comm, c->comm_stream));
    f.nccl(api.GroupEnd());
    f.cuda(cudaEventRecord(done, c->comm_stream));
}

// Posts the whole journey of the K/V chunks round the ring at once: hop h sends what hop h - 1 received (hop 0: this
// rank's own chunks) to rank + 1 and receives the chunks of step h + 1 from rank - 1 into receive set h.  The hops run
// back to back on the communication stream, at link speed, without waiting for any rank's kernels -- every rank holds a
// buffer per hop -- so a rank that runs late delays nobody's K/V, and only the first steps can ever wait for a hop.
void post_kv_chain(Ring& r, __nv_bfloat16* const own[4], cudaStream_t main, Fail& f)
{
    sntl_ring_comm* c = r.c;
    if (c->world < 2) return;
    f.cuda(cudaEventRecord(c->ev_main, main));
    for (int h = 0; h + 1 < c->world && !f.bad(); ++h) {
        void* s4[4];
        void* r4[4];
        for (int i = 0; i < 4; ++i) {
            s4[i] = h == 0 ? own[i] : r.kvbuf[h - 1][i];
            r4[i] = r.kvbuf[h][i];
        }
        rotate(r, s4, r4, 4, 2 * r.n_kv, c->ev_main, c->ev_hop[h], f);   // (waiting for ev_main again is free)
    }
}

struct Pair { int qi, ki, causal; };
int visible_pairs(const int q_ids[2], const int kv_ids[2], Pair out[4])
{
    int n = 0;
    for (int qi = 0; qi < 2; ++qi)
        for (int ki = 0; ki < 2; ++ki) {
            if (kv_ids[ki] < q_ids[qi]) out[n++] = Pair{qi, ki, 0};
            else if (kv_ids[ki] == q_ids[qi]) out[n++] = Pair{qi, ki, 1};
        }
    return n;
}

AttnShape pair_shape(const Ring& r, int causal)
{
    return AttnShape{r.B, r.Hq, r.Hkv, r.Sc, r.Sc, r.D, r.scale, causal, 0, 0, 0};
}

cudaError_t fill(float* p, float v, size_t n, cudaStream_t st)
{
    fill_f32_kernel<<<1184, 256, 0, st>>>(p, v, n);
    count_launch();
    return cudaGetLastError();
}

}  // namespace
}  // namespace sntl

extern "C" {

int sntl_ring_unique_id(void* id128)
{
    if (!id128) return SNTL_ERR_BAD_ARGUMENT;
    NcclApi& api = nccl();
    if (!api.ok) return SNTL_ERR_COMM;
    ncclUniqueId id;
    if (api.GetUniqueId(&id) != ncclSuccess) return SNTL_ERR_COMM;
    memcpy(id128, &id, sizeof(id));
    return SNTL_OK;
}

static int make_handle(ncclComm_t comm, bool owns, int rank, int world, sntl_ring_comm** out)
{
    sntl_ring_comm* c = new (std::nothrow) sntl_ring_comm;
    if (!c) return SNTL_ERR_CUDA;
    c->comm = comm; c->owns_comm = owns; c->rank = rank; c->world = world;
    bool ok = cudaGetDevice(&c->device) == cudaSuccess;
    // the communication stream gets the highest priority: its few CTAs must get onto an SM as soon as one frees up, not
    // after every CTA of the compute kernels queued before them has been dispatched, or the transfers stop hiding
    int prio_least = 0, prio_greatest = 0;
    ok = ok && cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest) == cudaSuccess;
    ok = ok && cudaStreamCreateWithPriority(&c->comm_stream, cudaStreamNonBlocking, prio_greatest) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking) == cudaSuccess;
    cudaEvent_t* evs[] = {&c->ev_main, &c->ev_side, &c->ev_acc, &c->ev_deal};
    for (cudaEvent_t* e : evs) ok = ok && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess;
    if (world > 1) {
        c->ev_hop = new (std::nothrow) cudaEvent_t[world - 1]();
        ok = ok && c->ev_hop != nullptr;
        for (int i = 0; ok && i + 1 < world; ++i) ok = cudaEventCreateWithFlags(&c->ev_hop[i], cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) { delete c; return SNTL_ERR_CUDA; }
    *out = c;
    return SNTL_OK;
}

int sntl_ring_comm_create(const void* id128, int rank, int world, sntl_ring_comm** out)
{
    if (!id128 || !out || world < 1 || rank < 0 || rank >= world) return SNTL_ERR_BAD_ARGUMENT;
    NcclApi& api = nccl();
    if (!api.ok) return SNTL_ERR_COMM;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t comm = nullptr;
    if (api.CommInitRank(&comm, world, id, rank) != ncclSuccess) return SNTL_ERR_COMM;
    const int rc = make_handle(comm, true, rank, world, out);
    if (rc != SNTL_OK) api.CommDestroy(comm);
    return rc;
}

int sntl_ring_comm_adopt(void* nccl_comm, int rank, int world, sntl_ring_comm** out)
{
    if (!nccl_comm || !out || world < 1 || rank < 0 || rank >= world) return SNTL_ERR_BAD_ARGUMENT;
    if (!nccl().ok) return SNTL_ERR_COMM;
    return make_handle((ncclComm_t)nccl_comm, false, rank, world, out);
}

int sntl_ring_comm_destroy(sntl_ring_comm* c)
{
    if (!c) return SNTL_OK;
    cudaStreamSynchronize(c->comm_stream);
    cudaStreamSynchronize(c->side_stream);
    if (c->owns_comm && c->comm) nccl().CommDestroy(c->comm);
    cudaEvent_t evs[] = {c->ev_main, c->ev_side, c->ev_acc, c->ev_deal};
    for (cudaEvent_t e : evs) if (e) cudaEventDestroy(e);
    if (c->ev_hop) {
        for (int i = 0; i + 1 < c->world; ++i) if (c->ev_hop[i]) cudaEventDestroy(c->ev_hop[i]);
        delete[] c->ev_hop;
    }
    cudaStreamDestroy(c->comm_stream);
    cudaStreamDestroy(c->side_stream);
    delete c;
    return SNTL_OK;
}

size_t sntl_ring_attn_workspace_bytes(const sntl_ring_comm* c, const sntl_attn_desc* d)
{
    if (validate_ring(c, d) != SNTL_OK) return 0;
    Ring r{};
    make_ring(r, const_cast<sntl_ring_comm*>(c), d, nullptr);
    return r.total;
}

int sntl_ring_attn_fwd(sntl_ring_comm* c, const sntl_attn_desc* d, const void* q, const void* k, const void* v, void* o, float* lse,
                       void* workspace, size_t workspace_bytes, void* stream)
{
    int rc = validate_ring(c, d);
    if (rc != SNTL_OK) return rc;
    if (!q || !k || !v || !o || !lse || !workspace) return SNTL_ERR_BAD_ARGUMENT;
    Ring r{};
    make_ring(r, c, d, workspace);
    if (workspace_bytes < r.total) return SNTL_ERR_WORKSPACE;
    cudaStream_t main = (cudaStream_t)stream, side = c->side_stream;
    const int W = c->world, me = c->rank;
    Fail f;
    const size_t row = (size_t)r.D * 2;
    DealItem items[3] = {{(const char*)q, {(char*)r.qz[0], (char*)r.qz[1]}, (char*)r.st_q, r.B * r.Hq, row},
                         {(const char*)k, {(char*)r.kz[0], (char*)r.kz[1]}, (char*)r.st_k, r.B * r.Hkv, row},
                         {(const char*)v, {(char*)r.vz[0], (char*)r.vz[1]}, (char*)r.st_v, r.B * r.Hkv, row}};
    deal(r, items, 3, false, main, f);
    for (int i = 0; i < 2; ++i) {
        f.cuda(cudaMemsetAsync(r.o_acc[i], 0, 4 * r.n_q, main));
        f.cuda(fill(r.lse_acc[i], -INFINITY, r.n_l, main));
    }
    const int q_ids[2] = {me, 2 * W - 1 - me};
    __nv_bfloat16* cur[4] = {r.kz[0], r.kz[1], r.vz[0], r.vz[1]};
    post_kv_chain(r, cur, main, f);
    for (int step = 0; step < W && !f.bad(); ++step) {
        const int src = ((me - step) % W + W) % W;
        const int kv_ids[2] = {src, 2 * W - 1 - src};
        if (step > 0) {
            f.cuda(cudaStreamWaitEvent(main, c->ev_hop[step - 1], 0));
            for (int i = 0; i < 4; ++i) cur[i] = r.kvbuf[step - 1][i];
        }
        f.cuda(cudaEventRecord(c->ev_main, main));
        Pair pairs[4];
        const int n = visible_pairs(q_ids, kv_ids, pairs);
        // the pairs of query chunk 0 on the caller's stream, those of query chunk 1 on the side stream (when both have some)
        bool has[2] = {false, false};
        for (int i = 0; i < n; ++i) has[pairs[i].qi] = true;
        const bool two = has[0] && has[1];
        if (two) f.cuda(cudaStreamWaitEvent(side, c->ev_main, 0));
        for (int i = 0; i < n; ++i) {
            const Pair& p = pairs[i];
            cudaStream_t lane = (two && p.qi == 1) ? side : main;
            TcArgs t{};
            t.s = pair_shape(r, p.causal);
            t.q = r.qz[p.qi]; t.k = cur[p.ki]; t.v = cur[2 + p.ki];
            t.o_out = r.o_part[p.qi]; t.lse_out = r.lse_part[p.qi];
            f.cuda(tc_forward(t, lane));
            f.cuda(merge_partials(SNTL_DTYPE_F32, SNTL_DTYPE_BF16, (long long)r.B * r.Hq * r.Sc, r.D, r.o_acc[p.qi], r.lse_acc[p.qi],
                                  r.o_part[p.qi], r.lse_part[p.qi], lane));
        }
        if (two) {
            f.cuda(cudaEventRecord(c->ev_side, side));
            f.cuda(cudaStreamWaitEvent(main, c->ev_side, 0));
        }
    }
    for (int i = 0; i < 2; ++i) f.cuda(f32_to_bf16(r.o_acc[i], r.oz[i], r.n_q, main));
    // LSE of the zigzag chunks is kept for a backward that reuses this state
    for (int i = 0; i < 2; ++i) f.cuda(cudaMemcpyAsync(r.lsez[i], r.lse_acc[i], 4 * r.n_l, cudaMemcpyDeviceToDevice, main));
    DealItem back[2] = {{(const char*)o, {(char*)r.oz[0], (char*)r.oz[1]}, (char*)r.st_o, r.B * r.Hq, row},
                        {(const char*)lse, {(char*)r.lsez[0], (char*)r.lsez[1]}, (char*)r.st_l, r.B * r.Hq, 4}};
    deal(r, back, 2, true, main, f);
    return f.status;
}

int sntl_ring_attn_bwd(sntl_ring_comm* c, const sntl_attn_desc* d, const void* q, const void* k, const void* v, const void* o,
                       const float* lse, const void* dout, void* dq, void* dk, void* dv, int reuse_forward_state, void* workspace,
                       size_t workspace_bytes, void* stream)
{
    int rc = validate_ring(c, d);
    if (rc != SNTL_OK) return rc;
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv || !workspace) return SNTL_ERR_BAD_ARGUMENT;
    Ring r{};
    make_ring(r, c, d, workspace);
    if (workspace_bytes < r.total) return SNTL_ERR_WORKSPACE;
    cudaStream_t main = (cudaStream_t)stream, side = c->side_stream;
    const int W = c->world, me = c->rank;
    Fail f;
    const size_t row = (size_t)r.D * 2;
    if (reuse_forward_state) {
        DealItem items[1] = {{(const char*)dout, {(char*)r.doz[0], (char*)r.doz[1]}, (char*)r.st_do, r.B * r.Hq, row}};
        deal(r, items, 1, false, main, f);
    } else {
        DealItem items[6] = {{(const char*)q, {(char*)r.qz[0], (char*)r.qz[1]}, (char*)r.st_q, r.B * r.Hq, row},
                             {(const char*)k, {(char*)r.kz[0], (char*)r.kz[1]}, (char*)r.st_k, r.B * r.Hkv, row},
                             {(const char*)v, {(char*)r.vz[0], (char*)r.vz[1]}, (char*)r.st_v, r.B * r.Hkv, row},
                             {(const char*)o, {(char*)r.oz[0], (char*)r.oz[1]}, (char*)r.st_o, r.B * r.Hq, row},
                             {(const char*)dout, {(char*)r.doz[0], (char*)r.doz[1]}, (char*)r.st_do, r.B * r.Hq, row},
                             {(const char*)lse, {(char*)r.lsez[0], (char*)r.lsez[1]}, (char*)r.st_l, r.B * r.Hq, 4}};
        deal(r, items, 6, false, main, f);
    }
    // per query chunk: delta, rescaled LSE, dQ accumulator zeroed
    for (int i = 0; i < 2; ++i) {
        TcArgs t{};
        t.s = pair_shape(r, 0);
        t.delta = (float*)r.pieces[i];
        t.dq_accum = (float*)((char*)r.pieces[i] + up256(kBwdRowAuxBytes * (size_t)r.B * r.Hq * (((size_t)r.Sc + 127) / 128 * 128)));
        t.o = r.oz[i]; t.dout = r.doz[i]; t.lse = r.lsez[i];
        t.phases = kBwdPre;
        f.cuda(tc_backward(t, main));
    }
    const int q_ids[2] = {me, 2 * W - 1 - me};
    __nv_bfloat16* cur[4] = {r.kz[0], r.kz[1], r.vz[0], r.vz[1]};
    int a_cur = 0, a_recv = 1, a_send = 2;         // indices into r.acc: being completed, being received, being sent
    for (int i = 0; i < 4; ++i) f.cuda(cudaMemsetAsync(r.acc[a_cur][i], 0, 4 * r.n_kv, main));
    post_kv_chain(r, cur, main, f);
    for (int step = 0; step < W && !f.bad(); ++step) {
        const int src = ((me - step) % W + W) % W;
        const int kv_ids[2] = {src, 2 * W - 1 - src};
        if (step > 0) {
            f.cuda(cudaStreamWaitEvent(main, c->ev_hop[step - 1], 0));
            for (int i = 0; i < 4; ++i) cur[i] = r.kvbuf[step - 1][i];
        }
        f.cuda(cudaEventRecord(c->ev_main, main));
        Pair pairs[4];
        const int n = visible_pairs(q_ids, kv_ids, pairs);
        const bool two = n > 1;
        if (two) f.cuda(cudaStreamWaitEvent(side, c->ev_main, 0));
        for (int i = 0; i < n; ++i) {
            const Pair& p = pairs[i];
            cudaStream_t lane = (two && (i & 1)) ? side : main;
            f.cuda(cudaMemsetAsync(r.part[i][0], 0, 4 * r.n_kv, lane));
            f.cuda(cudaMemsetAsync(r.part[i][1], 0, 4 * r.n_kv, lane));
            TcArgs t{};
            t.s = pair_shape(r, p.causal);
            t.delta = (float*)r.pieces[p.qi];
            t.dq_accum = (float*)((char*)r.pieces[p.qi] + up256(kBwdRowAuxBytes * (size_t)r.B * r.Hq * (((size_t)r.Sc + 127) / 128 * 128)));
            t.q = r.qz[p.qi]; t.k = cur[p.ki]; t.v = cur[2 + p.ki]; t.dout = r.doz[p.qi];
            t.dk_acc = r.part[i][0]; t.dv_acc = r.part[i][1];
            t.phases = kBwdMain;
            f.cuda(tc_backward(t, lane));
        }
        if (two) {
            f.cuda(cudaEventRecord(c->ev_side, side));
            f.cuda(cudaStreamWaitEvent(main, c->ev_side, 0));
        }
        // the accumulators of this step's key chunks: zeros at step 0, else what the previous rank sent
        if (step > 0) {
            f.cuda(cudaStreamWaitEvent(main, c->ev_acc, 0));
            const int t = a_cur; a_cur = a_recv; a_recv = t;
        }
        for (int i = 0; i < n; ++i) {
            const Pair& p = pairs[i];
            f.cuda(accumulate_f32(SNTL_DTYPE_F32, r.acc[a_cur][p.ki], r.part[i][0], r.n_kv, main));
            f.cuda(accumulate_f32(SNTL_DTYPE_F32, r.acc[a_cur][2 + p.ki], r.part[i][1], r.n_kv, main));
        }
        if (W > 1) {
            // pass them on; the hop runs under the next step's kernels (a_send's previous hop completed with the
            // round this rank has just waited for: a grouped round completes as a whole)
            const int t = a_cur; a_cur = a_send; a_send = t;
            f.cuda(cudaEventRecord(c->ev_main, main));
            void* s4[4] = {r.acc[a_send][0], r.acc[a_send][1], r.acc[a_send][2], r.acc[a_send][3]};
            void* r4[4] = {r.acc[a_recv][0], r.acc[a_recv][1], r.acc[a_recv][2], r.acc[a_recv][3]};
            rotate(r, s4, r4, 4, 4 * r.n_kv, c->ev_main, c->ev_acc, f);
        }
    }
    int home = a_cur;
    if (W > 1) {
        f.cuda(cudaStreamWaitEvent(main, c->ev_acc, 0));   // the last hop brings this rank's own chunks home
        home = a_recv;
    }
    for (int i = 0; i < 2; ++i) {
        TcArgs t{};
        t.s = pair_shape(r, 0);
        t.delta = (float*)r.pieces[i];
        t.dq_accum = (float*)((char*)r.pieces[i] + up256(kBwdRowAuxBytes * (size_t)r.B * r.Hq * (((size_t)r.Sc + 127) / 128 * 128)));
        t.dq = r.dqz[i];
        t.phases = kBwdPost;
        f.cuda(tc_backward(t, main));
        f.cuda(f32_to_bf16(r.acc[home][i], r.dkz[i], r.n_kv, main));
        f.cuda(f32_to_bf16(r.acc[home][2 + i], r.dvz[i], r.n_kv, main));
    }
    DealItem back[3] = {{(const char*)dq, {(char*)r.dqz[0], (char*)r.dqz[1]}, (char*)r.st_q, r.B * r.Hq, row},
                        {(const char*)dk, {(char*)r.dkz[0], (char*)r.dkz[1]}, (char*)r.st_k, r.B * r.Hkv, row},
                        {(const char*)dv, {(char*)r.dvz[0], (char*)r.dvz[1]}, (char*)r.st_v, r.B * r.Hkv, row}};
    deal(r, back, 3, true, main, f);
    return f.status;
}

}  // extern "C"

// Causal attention backward for sm_100a: dQ, dK, dV with P recomputed from the saved log-sum-exp.
//
// Replaces the reference's CudaFlashAttentionDeltaEntry + CudaFlashAttentionBackwardQueryWmma64Entry
// (sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:576-596, :1269-1456).  The reference walks query tiles and
// pushes dK/dV out with global atomics after scalar FMA loops; here all five products run on tcgen05 tensor
// cores and the loop is key-tile-outer:
//
//   * one CTA owns one 128-key tile of one (batch, KV head) and walks every 128-query tile that can see it,
//     for every query head of the group, so dK and dV accumulate in TMEM for the whole CTA lifetime and are
//     written exactly once: deterministic, no atomics, grouped-query sums done in place (the reference
//     materialises repeated K/V and reduces afterwards, CudaCausalSelfAttention.cu:27-44);
//   * everything is computed transposed (rows = keys) so that both P^T and dS^T are consumed by the next MMA
//     straight from TMEM as the A operand:
//         S^T  = K  Q^T  - 1 (LSE/scale)^T    (K, Q  K-major from shared memory)      -> TMEM
//         dP^T = V  dO^T - 1 delta^T          (V, dO K-major from shared memory)      -> TMEM
//           (the rank-one terms ride along as one extra 16-wide contraction step: a constant block of ones on the key
//            side, a 16-byte record per query on the other -- the fp32 value split exactly in three bf16 -- so no
//            per-column operand reaches the compute warps)
//         P^T  = exp2(scale*log2e * that), causal mask on the diagonal tile, bf16 back over S^T
//         dV  += P^T  dO         (A = P^T in TMEM,  B = dO tile MN-major)
//         dS^T = P^T o that, a packed bf16 product, into a shared-memory tile [key][query]
//         dQ_i = dS   K          (A = that tile read MN-major, B = K tile MN-major)
//         dK  += dS^T Q          (A = the same tile read K-major, B = Q tile MN-major)
//     the softmax scale is folded into the final dK store and the dQ conversion pass;
//   * dQ_i lands in TMEM (over the dP^T columns, which are dead by then) and a drain warpgroup adds it into an
//     fp32 accumulator in global memory with coalesced 16-byte vector reductions; the accumulator uses a
//     per-tile [d/4][row][4] order so that the 32 rows of a warp hit consecutive addresses;
//   * warp roles: 2 compute warpgroups (each owns 64 of the 128 query columns, one thread per key row),
//     1 drain warpgroup, 2 MMA-issuing warps, 1 TMA-producer warp; registers are re-allocated per role
//     (setmaxnreg).  Q (with its LSE records) has two stages and dO (with its delta records) one at D=128
//     (shared-memory capacity); three and two at D=64.
//
// A pre-pass computes the per-query records (delta = rowsum(dO o O) and LSE/scale, each split in two bf16; padded rows get a
// huge LSE so they produce P = 0) and zeroes the dQ accumulator; a post-pass converts the accumulator to bf16 dQ (times
// scale).
//
// Long key tiles.  The CTA of key tile 0 visits every query tile of every head of its group; when the grid is small
// (few batch elements x KV heads, as in the chunks of the host-buffer pipeline) or a sliding window leaves only the
// global-token tiles long, that one CTA outlasts the average SM's whole load and bounds the kernel.  Such tiles are
// cut by query head: one CTA per (key tile, KV head, query head of the group), each leaving its dK/dV as an fp32
// partial in scratch, and a small kernel adds the partials in head order (deterministic) and writes bf16.
// TMEM map (512 columns): S^T/P^T [0,128)  dP^T/dQ [128,256)  then dV [256,384) dK [384,512) at head_dim 128, and
// dV [256,320) dK [320,384) plus a second S^T/P^T buffer [384,512) at head_dim 64.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace sntl {

using namespace ptx;

namespace {

constexpr int kT = 128;                 // tile edge: keys per CTA, queries per step
constexpr int kBwdThreads = 512;        // 2 compute WGs + drain WG + 1 WG holding the MMA warp and the producer warp
constexpr uint32_t kTmemCols = 512;

enum BwdSite : uint32_t {
    kSiteKV = 0x21, kSiteQFull, kSiteQEmpty, kSiteDoFull, kSiteDoEmpty, kSiteS, kSiteP, kSiteDP, kSiteDS, kSiteDQ,
    kSiteDrained, kSiteFinal
};

struct BwdParams {
    __nv_bfloat16 *dk, *dv;
    // head_dim 64 (see bwd_folds_row_terms):
    const uint4* qaug;     // [B][Hq][Sq_pad] one 16-byte record per query: bf16 (hi, mid, lo, 0 x 5) of -LSE / scale
    const uint4* doaug;    // the same for -delta = -rowsum(dO o O)
    // head_dim 128:
    const float* lse2;     // [B][Hq][Sq_pad]  -LSE * log2(e), -inf on padded rows
    const float* delta;    // [B][Hq][Sq_pad]  -rowsum(dO o O)
    float* dq_accum;       // [B*Hq][n_qt][D/4][128][4]
    int B, Hq, Hkv, Sq, Skv, Sq_pad;
    int causal;
    int window, global_tokens;   // sliding window and always-visible first keys (0, 0: plain causal)
    int n_qt, n_kt;
    int split_tiles;       // the first split_tiles key tiles are cut into one CTA per query head of the group
    float* dkv_part;       // [split tile][slab][head of group][dV, dK][128][D] fp32
    float *dk_acc, *dv_acc;   // non-null: dK*scale / dV are ADDED into these fp32 [B*Hkv][Skv][D] tensors (no bf16 store)
    float scale, scale_log2;
};

// SMs of the current device (148 on a B200), read once per device ordinal
inline int sm_count()
{
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// Query tiles per head that key tile kt visits (the kernel's own rule)
__host__ __device__ inline int bwd_tiles_per_head(int kt, int n_qt, int causal, int window, int global_tokens)
{
    const int qt_first = causal ? kt : 0;
    const int k0 = kt * kT;
    const int qt_last = (window > 0 && k0 >= global_tokens) ? min(n_qt - 1, (k0 + kT - 1 + window - 1) / kT) : n_qt - 1;
    return max(0, qt_last - qt_first + 1);
}

// How many leading key tiles to cut by query head: those whose CTA would run longer than the average load of an SM.
inline int bwd_split_tiles(const AttnShape& s)
{
    const int group = s.Hq / s.Hkv;
    if (group <= 1 || s.deterministic) return 0;   // (the order-independent dQ form is not instantiated with cut tiles)
    const int n_qt = (s.Sq + kT - 1) / kT, n_kt = (s.Skv + kT - 1) / kT;
    const int window = s.causal ? s.window : 0;
    double total = 0.0;
    for (int kt = 0; kt < n_kt; ++kt) total += bwd_tiles_per_head(kt, n_qt, s.causal, window, s.global_tokens);
    const double avg = total * group * s.B * s.Hkv / sm_count();
    int n = 0;
    while (n < n_kt && (double)bwd_tiles_per_head(n, n_qt, s.causal, window, s.global_tokens) * group > avg) ++n;
    return n;
}

struct BwdBarriers {
    uint64_t kv_full;
    uint64_t q_full[3], q_empty[3], do_full[2], do_empty[2];
    uint64_t s_ready[2], p_ready, dp_ready, ds_ready, dq_ready, dq_drained, final_bar;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// Whether the per-query terms (LSE, delta) are folded into the S^T and dP^T products as one extra contraction step (see
// kAugBytes in the kernel).  That trades shared-memory loads and arithmetic in the compute warps for 2 x 65 tensor-pipe
// cycles per step on the two chains of products: a clear gain at head_dim 64, where the compute warps set the pace
// (-11 % kernel time), a loss at 128, where the chains do (+3 %).
__host__ __device__ constexpr bool bwd_folds_row_terms(int D) { return D == 64; }

// Shared-memory descriptor of an unswizzled K-major operand of ONE contraction step (16 bf16 = two 8-element column
// blocks): a column block is rows of 16 bytes, eight rows forming one 128-byte core matrix (SBO = 128 to the next eight
// rows); LBO is the distance from the first column block to the second.
__device__ __forceinline__ uint64_t make_sdesc_plain(uint32_t smem_addr, uint32_t lbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)(128u >> 4) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version (Blackwell); swizzle field 0 = none
    return d;
}

// One dQ tile (this thread's row in registers) -> staging buffers -> asynchronous bulk add-reductions into the accumulator
// tile, kStageCols columns per piece.  Called by all 128 threads of the drain warpgroup (named barrier 1); `elected` is the
// one thread that owns the bulk groups.  kStagingBytes of staging in all; `piece` counts pieces over the CTA's lifetime, so
// that the rotation carries on from tile to tile (a buffer is rewritten only after the kStages - 1 groups issued since
// its last use are all that may still be reading).
template <int D, bool kDet, int kStageCols, int kStagingBytes>
__device__ __forceinline__ void push_dq_tile(const uint32_t (&r)[D], float* tile, uint8_t* sStage, int row, bool elected, uint32_t& piece)
{
    constexpr int kStageBytes = kStageCols * kT * 4;
    constexpr int kStages = kStagingBytes / kStageBytes;
    static_assert(kStages >= 2 && kStages * kStageBytes == kStagingBytes, "staging must hold whole pieces");
    if constexpr (!kDet) {
#pragma unroll
        for (int c = 0; c < D / kStageCols; ++c) {
            uint8_t* stage = sStage + (piece++ % kStages) * kStageBytes;
            if (elected) bulk_wait_read<kStages - 1>();
            named_barrier_sync(1, 128);
#pragma unroll
            for (int v = 0; v < kStageCols / 4; ++v)
                *reinterpret_cast<uint4*>(stage + ((size_t)v * kT + row) * 16) =
                    make_uint4(r[c * kStageCols + 4 * v], r[c * kStageCols + 4 * v + 1], r[c * kStageCols + 4 * v + 2], r[c * kStageCols + 4 * v + 3]);
            fence_proxy_async_smem();
            named_barrier_sync(1, 128);
            if (elected) {
                bulk_reduce_add_f32(tile + (size_t)c * kStageCols * kT, stage, (uint32_t)kStageBytes);
                bulk_commit();
            }
        }
    } else {
        // Order-independent form: each fp32 value times 2^32 is an integer that fits 64 bits exactly (24-bit
        // mantissa, |value| < 2^31), and integer addition is associative, so the accumulated sum is the same
        // whatever order the key tiles arrive in.  Same staging buffers, half as many columns per piece; the
        // accumulator tile is [d/2][row][2] 64-bit words, so a piece is still one contiguous block.
        constexpr int kDetCols = kStageCols / 2;
        unsigned long long* tile64 = reinterpret_cast<unsigned long long*>(tile);
#pragma unroll
        for (int c = 0; c < D / kDetCols; ++c) {
            uint8_t* stage = sStage + (piece++ % kStages) * kStageBytes;
            if (elected) bulk_wait_read<kStages - 1>();
            named_barrier_sync(1, 128);
#pragma unroll
            for (int v = 0; v < kDetCols / 2; ++v) {
                const long long a = __float2ll_rn(__uint_as_float(r[c * kDetCols + 2 * v]) * 4294967296.0f);
                const long long b2 = __float2ll_rn(__uint_as_float(r[c * kDetCols + 2 * v + 1]) * 4294967296.0f);
                *reinterpret_cast<ulonglong2*>(stage + ((size_t)v * kT + row) * 16) =
                    make_ulonglong2((unsigned long long)a, (unsigned long long)b2);
            }
            fence_proxy_async_smem();
            named_barrier_sync(1, 128);
            if (elected) {
                bulk_reduce_add_u64(tile64 + (size_t)c * kDetCols * kT, stage, (uint32_t)kStageBytes);
                bulk_commit();
            }
        }
    }
}

// Epilogue of a compute warpgroup: its accumulator (dV for warpgroup 0, dK for warpgroup 1; `src` = TMEM address of this
// thread's row) leaves as an fp32 partial (cut tiles), is added into the caller's fp32 accumulators, or is stored as bf16
// through `stage_base` (a shared-memory tile no product reads any more).
template <int D>
__device__ __forceinline__ void write_dkv(const BwdParams& p, bool ok, bool split, int n_iter, int wg, int warp, int lane, int row,
                                          uint32_t src, int kt, int slab, int slabs, int group, int g0, int k0, uint8_t* stage_base)
{
    if (split) {
        // this CTA's share of dV (warpgroup 0) / dK (warpgroup 1) as an fp32 partial; zeros if it saw no query
        float* dst = p.dkv_part + ((((size_t)kt * slabs + slab) * group + g0) * 2 + wg) * (size_t)(kT * D) + (size_t)row * D;
        if (ok) tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            if (ok) {
                tmem_ld32(src + (uint32_t)(c * 32), r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int v = 0; v < 32; ++v) r[v] = 0u;
            }
#pragma unroll
            for (int v = 0; v < 8; ++v)
                *reinterpret_cast<uint4*>(dst + c * 32 + v * 4) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
        }
    } else if (ok && p.dk_acc != nullptr) {
        // accumulate form: this CTA is the only writer of its 128 key rows in this launch
        tc_fence_after();
        const int key = k0 + row;
        const bool store = key < p.Skv;
        const float mul = wg == 0 ? 1.0f : p.scale;
        float* dst = (wg == 0 ? p.dv_acc : p.dk_acc) + ((size_t)slab * p.Skv + (size_t)(store ? key : 0)) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(src + (uint32_t)(c * 32), r);
            tmem_ld_wait();
            if (store) {
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    float4 a = *reinterpret_cast<const float4*>(dst + c * 32 + v * 4);
                    a.x = fmaf(__uint_as_float(r[4 * v + 0]), mul, a.x);
                    a.y = fmaf(__uint_as_float(r[4 * v + 1]), mul, a.y);
                    a.z = fmaf(__uint_as_float(r[4 * v + 2]), mul, a.z);
                    a.w = fmaf(__uint_as_float(r[4 * v + 3]), mul, a.w);
                    *reinterpret_cast<float4*>(dst + c * 32 + v * 4) = a;
                }
            }
        }
    } else if (ok) {
        tc_fence_after();
        const int key = k0 + row;
        const bool store = key < p.Skv;
        const float mul = wg == 0 ? 1.0f : p.scale;
        // Coalesced bf16 store: a thread holds one whole key row, so the warp's 32 rows go through shared memory (the V
        // tile's buffer for dV, the K tile's for dK: every product has retired) and leave with each store instruction
        // covering whole rows; 16-byte units are XOR-swizzled by the row against bank conflicts.
        (void)store;
        __nv_bfloat16* out = (wg == 0 ? p.dv : p.dk) + (size_t)slab * p.Skv * D;
        constexpr int kUnits = D / 8;
        uint8_t* stage = stage_base + (warp & 3) * 32 * (D * 2);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(src + (uint32_t)(c * 32), r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                uint4 w;
                w.x = pack_bf16(__uint_as_float(r[8 * v + 0]) * mul, __uint_as_float(r[8 * v + 1]) * mul);
                w.y = pack_bf16(__uint_as_float(r[8 * v + 2]) * mul, __uint_as_float(r[8 * v + 3]) * mul);
                w.z = pack_bf16(__uint_as_float(r[8 * v + 4]) * mul, __uint_as_float(r[8 * v + 5]) * mul);
                w.w = pack_bf16(__uint_as_float(r[8 * v + 6]) * mul, __uint_as_float(r[8 * v + 7]) * mul);
                const int unit = c * 4 + v;
                *reinterpret_cast<uint4*>(stage + lane * (D * 2) + ((unit ^ (lane & 7)) << 4)) = w;
            }
        }
        __syncwarp();
        {
            constexpr int kRowsPerStore = 32 / kUnits;
            const int sub = lane / kUnits, unit = lane % kUnits;
            const int key_warp0 = key - lane;               // first key row of this warp
#pragma unroll
            for (int i = 0; i < 32 / kRowsPerStore; ++i) {
                const int rr = i * kRowsPerStore + sub;
                const uint4 w = *reinterpret_cast<const uint4*>(stage + rr * (D * 2) + ((unit ^ (rr & 7)) << 4));
                if (key_warp0 + rr < p.Skv) *reinterpret_cast<uint4*>(out + (size_t)(key_warp0 + rr) * D + unit * 8) = w;
            }
        }
    } else if (n_iter == 0 && p.dk_acc == nullptr) {
        // a key tile no query can see (cannot happen for causal with Sq == Skv; kept for safety): zero grads
        const int key = k0 + row;
        if (key < p.Skv) {
            __nv_bfloat16* dst = (wg == 0 ? p.dv : p.dk) + ((size_t)slab * p.Skv + key) * D;
            for (int d = 0; d < D; d += 8) *reinterpret_cast<uint4*>(dst + d) = make_uint4(0, 0, 0, 0);
        }
    }
}

// kSplit: the grid may hold key tiles cut by query head (a separate instantiation, so that the plain kernel carries none
// of that bookkeeping)
// kDet: dQ contributions leave as 64-bit fixed point (see the drain warpgroup)
template <int D, bool kWin, bool kSplit, bool kDet>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do, const BwdParams p)
{
    constexpr int kTileBytes = kT * D * 2;
    constexpr int kChunkBytes = kT * 128;          // 128 rows x 128 B
    constexpr int kChunks = D / 64;
    constexpr int kDoStages = (D == 128) ? 1 : 2;  // shared-memory capacity: 227 KB
    // head_dim 64 leaves 128 TMEM columns and 60 KB of shared memory unused: S^T gets a second buffer there, so that
    // S^T_{i+2} is computed while the compute warps are still busy with step i+1 and they never wait for the dV_i, S^T_{i+1}
    // pair behind their own P^T_i; Q then needs a third stage (Q_{i+2} is loaded while dK_i still reads Q_i)
    constexpr int kSBufs = (D == 128) ? 1 : 2;
    constexpr int kQStages = (D == 128) ? 2 : 3;
    // ... and the dS tile a second buffer, which lets dK_i be issued after the next dP^T instead of before it: the chain
    // dS_i -> dQ_i -> drain -> dP^T_{i+1} -> dS_{i+1} then no longer carries the issue time of dK_i (with one buffer dK_i must
    // have read the tile before dP^T_{i+1} lets the compute warps overwrite it)
    constexpr int kDsBufs = (D == 128) ? 1 : 2;
    constexpr bool kElect14 = D == 64;             // issue form of the dS-side warp (see there)
    // columns of a dQ tile per bulk reduction (kStageCols columns x 128 rows fp32 = one piece): 8 KB pieces at head_dim 128,
    // where the tile loads of Q and dO queue behind the reductions on the SM's path to L2 and shorter pieces let them through
    // sooner (-3 % kernel time); 16 KB pieces at head_dim 64 (there the finer split costs 1 %, and 4 KB pieces cost 10-20 %
    // at either size)
    constexpr int kStageCols = (D == 128) ? 16 : 32;
    constexpr int kStagingBytes = 32 * 1024;       // dQ staging in all
    // The extra contraction step (head_dim 64).  S^T and dP^T each get one more 16-wide k-step whose operands are not tile data: on the
    // key side a constant block (1, 1, 1, 0, ...), on the query side a 16-byte record per query, (hi, mid, lo, 0, ...) with
    // hi + mid + lo = -LSE/scale (for S^T) or -delta (for dP^T): the fp32 value split exactly in three bf16.  The tensor core then delivers
    // S^T - LSE/scale and dP^T - delta, and the compute warps need no per-column operand from shared memory at all:
    // P^T = exp2(scale*log2e * that) and dS^T = P^T o that.  One column block (8 bf16) per operand is real; the second
    // block of the constant operand is zeros, so the second block of the record operand may alias the first (LBO 0).
    constexpr bool kAug = bwd_folds_row_terms(D);
    constexpr int kAugBytes = kT * 16;             // 128 records
    constexpr int kDsBytes = kT * kT * 2;          // dS^T tile: [128 keys][128 queries] bf16 as two 64-query chunks
    // The layout uses every byte of the 227 KB a CTA may have (D = 128), so there is no room for an alignment
    // pad: the kernel has no static shared memory, which puts the dynamic window at the 1024-byte aligned start
    // of the CTA's shared memory; that is verified below instead of assumed.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    uint8_t* sK = smem;
    uint8_t* sV = sK + kTileBytes;
    uint8_t* sQ = sV + kTileBytes;                 // [kQStages]
    uint8_t* sDo = sQ + kQStages * kTileBytes;     // [kDoStages]
    uint8_t* sDs = sDo + kDoStages * kTileBytes;   // [kDsBufs]
    uint8_t* sStage = sDs + kDsBufs * kDsBytes;    // kStagingBytes
    // per-query terms: with the extra contraction step its operands, else -LSE*log2e and -delta as plain fp32 columns
    uint8_t* sTail = sStage + kStagingBytes;
    uint8_t* sOnes = sTail;                        // [2][kAugBytes]: the constant block, then zeros
    uint8_t* sQaug = sOnes + 2 * kAugBytes;        // [kQStages][kAugBytes]
    uint8_t* sDoaug = sQaug + kQStages * kAugBytes;   // [kDoStages][kAugBytes]
    float* sLse = (float*)sTail;                   // [kQStages][128]
    float* sDelta = sLse + kQStages * kT;          // [kQStages][128]
    constexpr int kTailBytes = kAug ? (2 + kQStages + kDoStages) * kAugBytes : 2 * kQStages * kT * 4;
    BwdBarriers* bars = (BwdBarriers*)(sTail + kTailBytes);
    volatile uint32_t* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((smem_u32(smem_raw) & 1023u) != 0u) {      // uniform over the CTA: nothing has been set up yet
        if (threadIdx.x == 0) atomicCAS(&g_device_status, 0u, (0x3fu << 24) | (blockIdx.x & 0xffffffu));
        return;
    }

    // ---- work decode: key tile 0 sees every query tile, so low key tiles go first ----
    const int slabs = p.B * p.Hkv;
    const int group = p.Hq / p.Hkv;
    // the first split_tiles key tiles come as one CTA per (tile, head of the group, slab), the rest as one per (tile, slab)
    const int n_split_ctas = kSplit ? p.split_tiles * group * slabs : 0;
    int kt, slab, g0 = 0, n_heads = group;
    const bool split = kSplit && (int)blockIdx.x < n_split_ctas;
    if (split) {
        kt = blockIdx.x / (group * slabs);
        const int rem = blockIdx.x - kt * group * slabs;
        g0 = rem / slabs;
        slab = rem - g0 * slabs;
        n_heads = 1;
    } else {
        const int idx = blockIdx.x - n_split_ctas;
        kt = p.split_tiles + idx / slabs;
        slab = idx - (idx / slabs) * slabs;             // b * Hkv + hk
    }
    const int b = slab / p.Hkv, hk = slab - b * p.Hkv;
    const int k0 = kt * kT;
    const int qt_first = p.causal ? kt : 0;
    // with a sliding window the last query that sees this tile is (last key + window - 1), unless the tile holds
    // global tokens, which every later query sees
    const int qt_last = (kWin && k0 >= p.global_tokens) ? min(p.n_qt - 1, (k0 + kT - 1 + p.window - 1) / kT) : p.n_qt - 1;
    const int per_head = qt_last - qt_first + 1;        // query tiles per head this CTA visits
    const int n_iter = per_head > 0 ? per_head * n_heads : 0;

    if (warp == 13 && lane == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        prefetch_tensormap(&tmap_do);
        mbar_init(&bars->kv_full, 1);
        for (int i = 0; i < 3; ++i) {
            mbar_init(&bars->q_full[i], 1);
            mbar_init(&bars->q_empty[i], 2);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->do_full[i], 1);
            mbar_init(&bars->do_empty[i], 2);
            mbar_init(&bars->s_ready[i], 1);
        }
        mbar_init(&bars->p_ready, 256);
        mbar_init(&bars->dp_ready, 1);
        mbar_init(&bars->ds_ready, 256);
        mbar_init(&bars->dq_ready, 1);
        mbar_init(&bars->dq_drained, 128);
        mbar_init(&bars->final_bar, 2);
        bars->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 12) {
        tmem_alloc(&bars->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    if (kAug && threadIdx.x < kT) {
        reinterpret_cast<uint4*>(sOnes)[threadIdx.x] = make_uint4(0x3f803f80u, 0x00003f80u, 0u, 0u);   // bf16 (1, 1, 1, 0, 0, 0, 0, 0)
        reinterpret_cast<uint4*>(sOnes + kAugBytes)[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
        fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    // S^T / P^T [0,128)   dP^T / dQ [128,256)   head_dim 128: dV [256,384) dK [384,512)   64: dV [256,320) dK [320,384) 2nd S^T [384,512)
    const uint32_t tm_S = tmem, tm_dP = tmem + 128u, tm_dV = tmem + 256u, tm_dK = tmem + (D == 128 ? 384u : 320u);
    constexpr uint32_t kSBufStride = 384u;         // columns from the first S^T buffer to the second

    // 512 threads start with 128 registers each; the issuing/producer warpgroup needs few, the others get the rest
    // (each role re-allocates registers inside its own branch so that the compiler sees which register count applies where)


    if (warp == 15) {
        setmaxnreg_dec<56>();
        // idle warps of the last warpgroup
    } else if (warp == 13) {
        setmaxnreg_dec<56>();
        // =========================== TMA producer ===========================
        if (lane == 0 && n_iter > 0) {
            mbar_arrive_expect_tx(&bars->kv_full, (uint32_t)(2 * kTileBytes));
            for (int c = 0; c < kChunks; ++c) {
                tma_load_3d(sK + c * kChunkBytes, &tmap_k, &bars->kv_full, c * 64, k0, slab);
                tma_load_3d(sV + c * kChunkBytes, &tmap_v, &bars->kv_full, c * 64, k0, slab);
            }
            for (int i = 0; i < n_iter; ++i) {
                const int g = i / per_head, qt = qt_first + (i - g * per_head);
                const int bh = b * p.Hq + hk * group + g0 + g;
                const int sq = i % kQStages;
                if (i >= kQStages && !mbar_wait(&bars->q_empty[sq], (uint32_t)(((i / kQStages) - 1) & 1), abort_flag, kSiteQEmpty)) break;
                mbar_arrive_expect_tx(&bars->q_full[sq], (uint32_t)(kTileBytes + (kAug ? kAugBytes : 2 * kT * 4)));
                for (int c = 0; c < kChunks; ++c)
                    tma_load_3d(sQ + sq * kTileBytes + c * kChunkBytes, &tmap_q, &bars->q_full[sq], c * 64, qt * kT, bh);
                if constexpr (kAug) {
                    bulk_load_1d(sQaug + sq * kAugBytes, p.qaug + (size_t)bh * p.Sq_pad + (size_t)qt * kT, kAugBytes, &bars->q_full[sq]);
                } else {
                    bulk_load_1d(sLse + sq * kT, p.lse2 + (size_t)bh * p.Sq_pad + (size_t)qt * kT, kT * 4, &bars->q_full[sq]);
                    bulk_load_1d(sDelta + sq * kT, p.delta + (size_t)bh * p.Sq_pad + (size_t)qt * kT, kT * 4, &bars->q_full[sq]);
                }
                const int sd = i % kDoStages;
                if (i >= kDoStages &&
                    !mbar_wait(&bars->do_empty[sd], (uint32_t)(((i / kDoStages) - 1) & 1), abort_flag, kSiteDoEmpty))
                    break;
                mbar_arrive_expect_tx(&bars->do_full[sd], (uint32_t)(kTileBytes + (kAug ? kAugBytes : 0)));
                if constexpr (kAug)
                    bulk_load_1d(sDoaug + sd * kAugBytes, p.doaug + (size_t)bh * p.Sq_pad + (size_t)qt * kT, kAugBytes, &bars->do_full[sd]);
                for (int c = 0; c < kChunks; ++c)
                    tma_load_3d(sDo + sd * kTileBytes + c * kChunkBytes, &tmap_do, &bars->do_full[sd], c * 64, qt * kT, bh);
            }
        }
    } else if (warp == 12 || warp == 14) {
        setmaxnreg_dec<56>();
        // =========================== MMA issuers ===========================
        // Two issuing threads on two different schedulers, because a lone issuing warp shares its scheduler with
        // ALU-dense compute warps and gets too few issue slots to keep the tensor pipe fed:
        //   warp 12 ("P side"):   dV_i += P^T dO_i ,  S^T_{i+1} = K Q_{i+1}^T
        //   warp 14 ("dS side"):  dK_i += dS^T Q_i ,  dQ_i = dS K ,  dP^T_{i+1} = V dO_{i+1}^T
        // Every TMEM region with a write-after-read hazard is touched by one of the two only (S^T/P^T by warp 12,
        // dP^T/dS^T/dQ by warp 14), so the in-order execution of one thread's MMAs still covers those hazards.  The Q
        // and dO stages are read by both and are released when both have committed (barrier count 2).  Each commits its
        // share of a dO stage right after its own product that reads it: with one dO stage (head_dim 128) the next dO tile
        // can only be loaded once both have, and dP^T_{i+1} waits for that load.
        // (Two, not more: MMAs issued by different warps interleave in the tensor pipe k-step by k-step, each on another
        // accumulator, and a third issuing warp for dK measured 7-20 % slower than this split at either head size.)
        if (warp == 12 && n_iter > 0) {
            // P side: all 32 lanes walk the loop (warp-uniform control flow lets descriptors and addresses live in uniform
            // registers) and one elected lane issues each tcgen05 instruction.  dV_i and S^T_{i+1} head the chain the compute
            // warps wait on, and this form issues 8 MMAs in ~720 cycles against ~1100 for a single-lane loop.
            SNTL_TRACE_DECL(tn);
            const bool tl = lane == 0;
            (void)tl;
            constexpr uint32_t idesc_st = make_idesc(kT, kT, false, false);
            constexpr uint32_t idesc_kv = make_idesc(kT, D, false, true);
            auto wait = [&](uint64_t* bar, uint32_t parity, uint32_t site) {
                return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, site));
            };
            const uint64_t d_ones = make_sdesc_plain(smem_u32(sOnes), kAugBytes), d_qaug0 = make_sdesc_plain(smem_u32(sQaug), 0);
            // the D/16 steps over the head dimension, then the extra step that subtracts LSE/scale (see kAugBytes)
            auto issue_kmajor = [&](uint32_t d_tmem, uint64_t a, uint64_t b, uint64_t aug) {
                mma_ss_e<false>(d_tmem, a, b, idesc_st);
#pragma unroll
                for (int ks = 1; ks < D / 16; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * kChunkBytes + (ks & 3) * 32);
                    mma_ss_e<true>(d_tmem, sdesc_advance(a, off), sdesc_advance(b, off), idesc_st);
                }
                if constexpr (kAug) mma_ss_e<true>(d_tmem, d_ones, aug, idesc_st);
            };
            auto issue_from_tmem = [&](uint32_t d_tmem, uint32_t a_tmem, uint64_t b, bool accumulate) {
                if (accumulate) mma_ts_e<true>(d_tmem, a_tmem, b, idesc_kv);
                else mma_ts_e<false>(d_tmem, a_tmem, b, idesc_kv);
#pragma unroll
                for (int ks = 1; ks < kT / 16; ++ks)
                    mma_ts_e<true>(d_tmem, a_tmem + (uint32_t)((ks >> 2) * 64 + (ks & 3) * 8), sdesc_advance(b, ks * 2048), idesc_kv);
            };
            bool ok = wait(&bars->kv_full, 0, kSiteKV);
            const uint64_t dK_k = make_sdesc(smem_u32(sK), 16, 1024);
            const uint64_t dQ_k0 = make_sdesc(smem_u32(sQ), 16, 1024), dDo_mn0 = make_sdesc(smem_u32(sDo), kChunkBytes, 1024);
            // S^T of the first kSBufs steps; after that S^T_{i+kSBufs} follows dV_i into the buffer that P^T_i leaves
            for (int j = 0; ok && j < kSBufs && j < n_iter; ++j) {
                if (!(ok = wait(&bars->q_full[j], 0, kSiteQFull))) break;
                tc_fence_after();
                issue_kmajor(tm_S + (uint32_t)j * kSBufStride, dK_k, sdesc_advance(dQ_k0, j * kTileBytes), sdesc_advance(d_qaug0, j * kAugBytes));
                tc_commit_e(&bars->s_ready[j]);
            }
            for (int i = 0; ok && i < n_iter; ++i) {
                const int sq = i % kQStages, sd = i % kDoStages, sb = i % kSBufs;
                const uint32_t tm_Si = tm_S + (uint32_t)sb * kSBufStride;
                if (!(ok = wait(&bars->p_ready, (uint32_t)(i & 1), kSiteP))) break;
                if (!(ok = wait(&bars->do_full[sd], (uint32_t)((i / kDoStages) & 1), kSiteDoFull))) break;
                SNTL_TRACE_EV(tl, 0, tn, 1);
                tc_fence_after();
                issue_from_tmem(tm_dV, tm_Si, sdesc_advance(dDo_mn0, sd * kTileBytes), i > 0);
                tc_commit_e(&bars->do_empty[sd]);
                tc_commit_e(&bars->q_empty[sq]);
                SNTL_TRACE_EV(tl, 0, tn, 2);
                if (i + kSBufs < n_iter) {
                    const int nq = (i + kSBufs) % kQStages;
                    if (!(ok = wait(&bars->q_full[nq], (uint32_t)(((i + kSBufs) / kQStages) & 1), kSiteQFull))) break;
                    tc_fence_after();
                    issue_kmajor(tm_Si, dK_k, sdesc_advance(dQ_k0, nq * kTileBytes), sdesc_advance(d_qaug0, nq * kAugBytes));
                    tc_commit_e(&bars->s_ready[sb]);
                    SNTL_TRACE_EV(tl, 0, tn, 9);
                }
            }
            tc_commit_e(&bars->final_bar);
            wait(&bars->final_bar, 0, kSiteFinal);
        } else if (warp == 14 && (kElect14 || lane == 0) && n_iter > 0) {
            // dS side.  At head_dim 64 it takes the same warp-uniform form as the P side (-4 % kernel time); at 128 a single
            // lane walks the loop: there the faster form costs 8 % (2.81 vs 2.59 ms) -- these products then get into the
            // tensor pipe ahead of the P side's, whose chain sets the step at that head size.
            const bool tl14 = lane == 0;
            (void)tl14;
            auto wait = [&](uint64_t* bar, uint32_t parity, uint32_t site) {
                if constexpr (kElect14) return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, site));
                else return mbar_wait(bar, parity, abort_flag, site);
            };
            SNTL_TRACE_DECL(tn);
            constexpr uint32_t idesc_st = make_idesc(kT, kT, false, false);   // S^T, dP^T
            constexpr uint32_t idesc_kv = make_idesc(kT, D, false, true);     // dV, dK: A in TMEM, B MN-major
            constexpr uint32_t idesc_dq = make_idesc(kT, D, true, true);      // dQ: both operands MN-major
            // C[128 x 128] = A[128 x D] * B[128 x D]^T, both K-major tiles; one descriptor per tile, advanced per k-step
            // by a 64-bit add (the empty asm keeps the compiler from hoisting every advanced descriptor out of the main
            // loop, which would cost this warp more registers than it is allotted)
            const uint64_t d_ones = make_sdesc_plain(smem_u32(sOnes), kAugBytes), d_doaug0 = make_sdesc_plain(smem_u32(sDoaug), 0);
            // the D/16 steps over the head dimension, then the extra step that subtracts delta (see kAugBytes)
            auto issue_kmajor = [&](uint32_t d_tmem, uint64_t a, uint64_t b, uint64_t aug) {
                asm volatile("" : "+l"(a), "+l"(b), "+l"(aug));
                mma_ss_x<kElect14, false>(d_tmem, a, b, idesc_st);
#pragma unroll
                for (int ks = 1; ks < D / 16; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * kChunkBytes + (ks & 3) * 32);
                    mma_ss_x<kElect14, true>(d_tmem, sdesc_advance(a, off), sdesc_advance(b, off), idesc_st);
                }
                if constexpr (kAug) mma_ss_x<kElect14, true>(d_tmem, d_ones, aug, idesc_st);
            };
            bool ok = wait(&bars->kv_full, 0, kSiteKV);
            {
                const uint64_t dV_k = make_sdesc(smem_u32(sV), 16, 1024), dDo_k0 = make_sdesc(smem_u32(sDo), 16, 1024);
                const uint64_t dK_mn = make_sdesc(smem_u32(sK), kChunkBytes, 1024), dDs_mn = make_sdesc(smem_u32(sDs), kChunkBytes, 1024);
                const uint64_t dDs_k = make_sdesc(smem_u32(sDs), 16, 1024);
                const uint64_t dQ_mn0 = make_sdesc(smem_u32(sQ), kChunkBytes, 1024);
                ok = ok && wait(&bars->do_full[0], 0, kSiteDoFull);
                if (ok) {
                    tc_fence_after();
                    issue_kmajor(tm_dP, dV_k, dDo_k0, d_doaug0);
                    tc_commit_x<kElect14>(&bars->dp_ready);
                    tc_commit_x<kElect14>(&bars->do_empty[0]);   // this warp's share of releasing dO_0: dP^T_0
                }
                for (int i = 0; ok && i < n_iter; ++i) {
                    const uint32_t ph = (uint32_t)(i & 1);
                    const int sq = i % kQStages;
                    if (!(ok = wait(&bars->ds_ready, ph, kSiteDS))) break;
                    SNTL_TRACE_EV(tl14, 4, tn, 3);
                    tc_fence_after();
                    // dQ first: it gates the drain and with it the next dP^T
                    const uint32_t ds_off = (uint32_t)((i % kDsBufs) * kDsBytes);
                    {
                        uint64_t a = sdesc_advance(dDs_mn, ds_off), bq = dK_mn;
                        asm volatile("" : "+l"(a), "+l"(bq));
                        mma_ss_x<kElect14, false>(tm_dP, a, bq, idesc_dq);
#pragma unroll
                        for (int ks = 1; ks < kT / 16; ++ks)
                            mma_ss_x<kElect14, true>(tm_dP, sdesc_advance(a, ks * 2048), sdesc_advance(bq, ks * 2048), idesc_dq);
                    }
                    tc_commit_x<kElect14>(&bars->dq_ready);
                    SNTL_TRACE_EV(tl14, 4, tn, 4);
                    // dK += dS^T Q with dS^T read from its shared-memory tile as a K-major A operand (rows = keys, the 64
                    // contiguous elements run along the queries).  Q_i is ready: ds_ready implies its load was seen.  With
                    // one dS buffer it goes before the next dP^T: by the time the compute warps see that dP^T and rewrite the
                    // tile, this product has read it (one thread's MMAs run in order).  With two it goes after, and the
                    // buffer it reads is rewritten only behind dP^T_{i+2}, which this thread issues later still.
                    auto issue_dk = [&]() {
                        uint64_t a = sdesc_advance(dDs_k, ds_off), bq = sdesc_advance(dQ_mn0, sq * kTileBytes);
                        asm volatile("" : "+l"(a), "+l"(bq));
                        if (i > 0) mma_ss_x<kElect14, true>(tm_dK, a, bq, idesc_kv);
                        else mma_ss_x<kElect14, false>(tm_dK, a, bq, idesc_kv);
#pragma unroll
                        for (int ks = 1; ks < kT / 16; ++ks)
                            mma_ss_x<kElect14, true>(tm_dK, sdesc_advance(a, (ks >> 2) * kChunkBytes + (ks & 3) * 32), sdesc_advance(bq, ks * 2048), idesc_kv);
                        tc_commit_x<kElect14>(&bars->q_empty[sq]);    // this warp's share: dK_i
                    };
                    if constexpr (kDsBufs == 1) issue_dk();
                    if (i + 1 < n_iter) {
                        const int nd = (i + 1) % kDoStages;
                        if (!(ok = wait(&bars->dq_drained, ph, kSiteDrained))) break;
                        SNTL_TRACE_EV(tl14, 4, tn, 5);
                        if (!(ok = wait(&bars->do_full[nd], (uint32_t)(((i + 1) / kDoStages) & 1), kSiteDoFull))) break;
                        tc_fence_after();
                        issue_kmajor(tm_dP, dV_k, sdesc_advance(dDo_k0, nd * kTileBytes), sdesc_advance(d_doaug0, nd * kAugBytes));
                        tc_commit_x<kElect14>(&bars->dp_ready);
                        // this warp's share of releasing dO_{i+1}, committed at once: with a single dO stage the load of the
                        // next tile starts as soon as this product and dV_{i+1} have read the stage
                        tc_commit_x<kElect14>(&bars->do_empty[nd]);
                        SNTL_TRACE_EV(tl14, 4, tn, 6);
                    }
                    if constexpr (kDsBufs == 2) issue_dk();
                }
            }
            // every MMA of this thread has retired once its commit lands; the epilogue waits for both issuers
            tc_commit_x<kElect14>(&bars->final_bar);
            wait(&bars->final_bar, 0, kSiteFinal);
        }
    } else if (warp >= 8) {
        setmaxnreg_inc<152>();
        // =========================== dQ drain warpgroup ===========================
        const int row = (warp & 3) * 32 + lane;                 // query row inside the tile == TMEM lane
        SNTL_TRACE_DECL(tn);
        const bool tw = warp == 8 && lane == 0;
        (void)tw;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const bool elected = warp == 8 && lane == 0;
        bool ok = true;
        uint32_t piece = 0;
        for (int i = 0; i < n_iter; ++i) {
            const int g = i / per_head, qt = qt_first + (i - g * per_head);
            const int bh = b * p.Hq + hk * group + g0 + g;
            // fp32 accumulator: kT*D words per tile; fixed-point accumulator: kT*D 64-bit words per tile
            float* tile = p.dq_accum + ((size_t)bh * p.n_qt + qt) * (size_t)(kT * D) * (kDet ? 2 : 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->dq_ready, (uint32_t)(i & 1), abort_flag, kSiteDQ));
            SNTL_TRACE_EV(tw, 3, tn, 1);
            if (!ok) break;
            tc_fence_after();
            // The whole dQ tile goes to registers first so that the TMEM columns are handed back to the MMA warp at
            // once; pushing 64 KB (D = 128) through the reduction path (~30 bytes/clock per SM) is the slow part and
            // overlaps the next step.  The data leave through the TMA engine, not the load/store unit: reductions
            // issued as instructions queue up in the unit that also carries the compute warps' shared-memory and
            // TMEM traffic and stall them.  kStageCols columns at a time: registers -> staging buffer -> one asynchronous
            // bulk add-reduction (contiguous in the accumulator thanks to its [d/4][row][4] order).  The staging buffers
            // (32 KB in all) rotate; the elected thread makes sure a buffer's previous reduction has finished reading it
            // before it is overwritten.
            uint32_t r[D];
#pragma unroll
            for (int c = 0; c < D / 32; ++c) tmem_ld32(tm_dP + lane_off + (uint32_t)(c * 32), r + c * 32);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&bars->dq_drained);
            SNTL_TRACE_EV(tw, 3, tn, 2);
            push_dq_tile<D, kDet, kStageCols, kStagingBytes>(r, tile, sStage, row, elected, piece);
            SNTL_TRACE_EV(tw, 3, tn, 3);
        }
        if (elected) bulk_wait_all();   // the reductions read shared memory and must land before the CTA retires
    } else {
        setmaxnreg_inc<152>();
        // =========================== compute warpgroups ===========================
        const int wg = warp >> 2;                                // owns query columns [64*wg, 64*wg+64)
        const int row = (warp & 3) * 32 + lane;                  // key row inside the tile == TMEM lane
        SNTL_TRACE_DECL(tn);
        const bool tw = (warp & 3) == 0 && lane == 0;
        (void)tw;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t col0 = (uint32_t)(wg * 64);
        uint8_t* ds_row0 = sDs + wg * kChunkBytes + row * 128;   // this thread's 128-byte row of its 64-query chunk
        bool ok = true;
        for (int i = 0; i < n_iter; ++i) {
            const int qt = qt_first + (i % per_head);
            const uint32_t ph = (uint32_t)(i & 1);
            // ---- P^T ----
            const uint32_t tm_Si = tm_S + (uint32_t)(i % kSBufs) * kSBufStride;
            // (the Q stage's barrier also covers the LSE and delta columns this warp reads when they come as plain columns)
            ok = __all_sync(0xffffffffu, (kAug || mbar_wait(&bars->q_full[i % kQStages], (uint32_t)((i / kQStages) & 1), abort_flag, kSiteQFull)) &&
                                             mbar_wait(&bars->s_ready[i % kSBufs], (uint32_t)((i / kSBufs) & 1), abort_flag, kSiteS));
            SNTL_TRACE_EV(tw, 1 + wg, tn, 1);
            if (!ok) break;
            tc_fence_after();
            uint32_t s[64];
            tmem_ld32(tm_Si + lane_off + col0, s);
            tmem_ld32(tm_Si + lane_off + col0 + 32u, s + 32);
            tmem_ld_wait();
            SNTL_TRACE_EV(tw, 1 + wg, tn, 2);
            // tiles the mask cuts through: the diagonal one and, with a window, those reaching past (first key + window - 1)
            const bool diag = (p.causal && qt == kt) || (kWin && qt * kT + kT - 1 > k0 + p.window - 1);
            uint32_t pk[32];
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            const float4* lse4 = reinterpret_cast<const float4*>(sLse + (i % kQStages) * kT + col0);
            // exponents of four columns: with the extra contraction step the product already holds S^T - LSE/scale and one
            // packed multiply per pair gives them; else x = s*scale*log2(e) - LSE*log2(e) is one packed FMA per pair
            auto exponents = [&](int c, float2& x01, float2& x23) {
                const float2 s01 = make_float2(__uint_as_float(s[4 * c + 0]), __uint_as_float(s[4 * c + 1]));
                const float2 s23 = make_float2(__uint_as_float(s[4 * c + 2]), __uint_as_float(s[4 * c + 3]));
                if constexpr (kAug) {
                    x01 = fmul2(s01, sc2);
                    x23 = fmul2(s23, sc2);
                } else {
                    const float4 l = lse4[c];
                    x01 = ffma2(s01, sc2, make_float2(l.x, l.y));
                    x23 = ffma2(s23, sc2, make_float2(l.z, l.w));
                }
            };
            // branch-free main body (the mask test lives in its own copy of the loop, taken only on the diagonal tile,
            // so that the common copy is one basic block the compiler can software-pipeline)
            if (!diag) {
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    float2 x01, x23;
                    exponents(c, x01, x23);
                    pk[2 * c] = pack_bf16(ex2(x01.x), ex2(x01.y));
                    pk[2 * c + 1] = pack_bf16(ex2(x23.x), ex2(x23.y));
                }
            } else {
                // this thread's key sees the queries from itself (causal) up to key + window - 1 (global keys: all)
                const int key = k0 + row;
                const int first_q = p.causal ? key - qt * kT : -1;
                const int last_q = (kWin && key >= p.global_tokens) ? key + p.window - 1 - qt * kT : kT;
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    float2 x01, x23;
                    exponents(c, x01, x23);
                    const int q = (int)col0 + 4 * c;   // visible: first_q <= query (column) <= last_q
                    const float p0 = (q + 0 < first_q || q + 0 > last_q) ? 0.0f : ex2(x01.x);
                    const float p1 = (q + 1 < first_q || q + 1 > last_q) ? 0.0f : ex2(x01.y);
                    const float p2 = (q + 2 < first_q || q + 2 > last_q) ? 0.0f : ex2(x23.x);
                    const float p3 = (q + 3 < first_q || q + 3 > last_q) ? 0.0f : ex2(x23.y);
                    pk[2 * c] = pack_bf16(p0, p1);
                    pk[2 * c + 1] = pack_bf16(p2, p3);
                }
            }
            SNTL_TRACE_EV(tw, 1 + wg, tn, 3);
            tmem_st32(tm_Si + lane_off + col0, pk);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&bars->p_ready);
            SNTL_TRACE_EV(tw, 1 + wg, tn, 4);
            // ---- dS^T ----
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->dp_ready, ph, abort_flag, kSiteDP));
            SNTL_TRACE_EV(tw, 1 + wg, tn, 5);
            if (!ok) break;
            tc_fence_after();
            tmem_ld32(tm_dP + lane_off + col0, s);
            tmem_ld32(tm_dP + lane_off + col0 + 32u, s + 32);
            tmem_ld_wait();
            SNTL_TRACE_EV(tw, 1 + wg, tn, 6);
            const float4* dl4 = reinterpret_cast<const float4*>(sDelta + (i % kQStages) * kT + col0);
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                if constexpr (kAug) {
                    // the product already holds dP^T - delta, and dS^T = P^T o that is a packed bf16 product: the second
                    // factor is rounded to bf16 first, the product once more (dS^T is a bf16 MMA operand either way)
                    pk[2 * c] = mul_bf16x2(pk[2 * c], pack_bf16(__uint_as_float(s[4 * c + 0]), __uint_as_float(s[4 * c + 1])));
                    pk[2 * c + 1] = mul_bf16x2(pk[2 * c + 1], pack_bf16(__uint_as_float(s[4 * c + 2]), __uint_as_float(s[4 * c + 3])));
                } else {
                    const float4 dl = dl4[c];   // holds -delta
                    const float2 pa = make_float2(__uint_as_float(pk[2 * c] << 16), __uint_as_float(pk[2 * c] & 0xffff0000u));
                    const float2 pb = make_float2(__uint_as_float(pk[2 * c + 1] << 16), __uint_as_float(pk[2 * c + 1] & 0xffff0000u));
                    const float2 da = fmul2(pa, fadd2(make_float2(__uint_as_float(s[4 * c + 0]), __uint_as_float(s[4 * c + 1])), make_float2(dl.x, dl.y)));
                    const float2 db = fmul2(pb, fadd2(make_float2(__uint_as_float(s[4 * c + 2]), __uint_as_float(s[4 * c + 3])), make_float2(dl.z, dl.w)));
                    pk[2 * c] = pack_bf16(da.x, da.y);
                    pk[2 * c + 1] = pack_bf16(db.x, db.y);
                }
            }
            // into shared memory, rows of 128 bytes with the 128-byte swizzle the MMA expects (both the dQ and the dK
            // product read this tile)
            uint8_t* ds_row = ds_row0 + (i % kDsBufs) * kDsBytes;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint4 w = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                *reinterpret_cast<uint4*>(ds_row + ((j ^ (row & 7)) << 4)) = w;
            }
            fence_proxy_async_smem();
            SNTL_TRACE_EV(tw, 1 + wg, tn, 7);
            tc_fence_before();   // orders this thread's TMEM loads of dP^T before the MMA that overwrites those columns
            mbar_arrive(&bars->ds_ready);
            SNTL_TRACE_EV(tw, 1 + wg, tn, 8);
        }
        // ---- epilogue: dV (warpgroup 0) and dK (warpgroup 1) ----
        ok = __all_sync(0xffffffffu, ok && n_iter > 0 && mbar_wait(&bars->final_bar, 0, abort_flag, kSiteFinal));
        write_dkv<D>(p, ok, split, n_iter, wg, warp, lane, row, (wg == 0 ? tm_dV : tm_dK) + lane_off, kt, slab, slabs, group, g0, k0,
                     wg == 0 ? sV : sK);
    }

    // ---- teardown ----
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 12) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// Per padded query row: the two 16-byte records the main kernel feeds to its extra contraction step -- bf16 (hi, mid, lo, 0 x 5)
// with hi + mid + lo = -rowsum(dO o O) (delta) and = -LSE / scale (a large negative number for padded rows and for rows without
// visible keys, so that they produce P = 0) -- and the dQ accumulator zeroed.  D/4 lanes per (b, h, padded row), 8 bytes of O
// and of dO per lane: a warp covers one row at head_dim 128 and two at 64, every lane busy either way.
template <int D>
__global__ void bwd_pre_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                               const float* __restrict__ lse, void* __restrict__ lse_out, void* __restrict__ delta_out,
                               float* __restrict__ dq_accum, int Sq, int Sq_pad, long long rows_padded, int acc_words_per_row,
                               float inv_scale)
{
    constexpr int kLanesPerRow = D / 4, kRowsPerWarp = 32 / kLanesPerRow;
    const int lane = threadIdx.x & 31, sub = lane / kLanesPerRow, l = lane % kLanesPerRow;
    const long long r = (blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5)) * kRowsPerWarp + sub;
    const bool live = r < rows_padded;
    const long long bh = live ? r / Sq_pad : 0;
    const int s = live ? (int)(r - bh * Sq_pad) : 0;
    if (live) {
        // the accumulator is tile-permuted but covers exactly acc_words_per_row 32-bit words per padded row (D, or 2*D
        // when it is 64-bit fixed point): zero it linearly
        float4* z = reinterpret_cast<float4*>(dq_accum + r * acc_words_per_row);
        for (int i = l; i < acc_words_per_row / 4; i += kLanesPerRow) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float acc = 0.0f;
    if (live && s < Sq) {
        const size_t off = ((size_t)bh * Sq + s) * D + l * 4;
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(o + off));
        const uint2 g = __ldg(reinterpret_cast<const uint2*>(dout + off));
        acc = fmaf(__uint_as_float(a.x << 16), __uint_as_float(g.x << 16), acc);
        acc = fmaf(__uint_as_float(a.x & 0xffff0000u), __uint_as_float(g.x & 0xffff0000u), acc);
        acc = fmaf(__uint_as_float(a.y << 16), __uint_as_float(g.y << 16), acc);
        acc = fmaf(__uint_as_float(a.y & 0xffff0000u), __uint_as_float(g.y & 0xffff0000u), acc);
    }
#pragma unroll
    for (int m = kLanesPerRow / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    if (live && l == 0) {
        if constexpr (bwd_folds_row_terms(D)) {
            uint4* qaug = static_cast<uint4*>(lse_out);
            uint4* doaug = static_cast<uint4*>(delta_out);
            // value -> three bf16 (hi, mid, lo) whose sum is the fp32 value exactly (3 x 8 significant bits), as the first
            // three slots of a record
            auto split = [](float x) {
                const __nv_bfloat16 hi = __float2bfloat16_rn(x);
                const float r1 = x - __bfloat162float(hi);
                const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
                const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
                return make_uint4((uint32_t)__bfloat16_as_ushort(hi) | ((uint32_t)__bfloat16_as_ushort(mid) << 16),
                                  (uint32_t)__bfloat16_as_ushort(lo), 0u, 0u);
            };
            constexpr float kMasked = -1.0e30f;   // times scale*log2(e) still far below the exponent range: P = 0, and finite
            if (s >= Sq) { qaug[r] = split(kMasked); doaug[r] = make_uint4(0u, 0u, 0u, 0u); }
            else {
                const float lv = lse[(size_t)bh * Sq + s];
                qaug[r] = split((lv == -INFINITY) ? kMasked : -lv * inv_scale);
                doaug[r] = split(-acc);
            }
        } else {
            float* lse2 = static_cast<float*>(lse_out);
            float* delta = static_cast<float*>(delta_out);
            if (s >= Sq) { lse2[r] = -INFINITY; delta[r] = 0.0f; }
            else {
                const float lv = lse[(size_t)bh * Sq + s];
                lse2[r] = (lv == -INFINITY) ? -INFINITY : -lv * 1.4426950408889634f;
                delta[r] = -acc;
            }
        }
    }
}

// dQ (bf16, [B][Hq][Sq][D]) = scale * accumulator, undoing the per-tile [d/4][row][4] order.
// One CTA per (tile, 32-row group): for a fixed d/4 chunk its 32 rows are 512 contiguous bytes of the accumulator.
template <int D>
__global__ void __launch_bounds__(256) bwd_post_kernel(const float* __restrict__ dq_accum, __nv_bfloat16* __restrict__ dq, int Sq,
                                                       int n_qt, float scale)
{
    constexpr int kRows = 32;
    __shared__ float tile[kRows][D + 4];
    const size_t t = blockIdx.x >> 2;
    const int r0 = (int)(blockIdx.x & 3) * kRows;
    const size_t bh = t / n_qt;
    const int qt = (int)(t - bh * n_qt);
    const float4* src = reinterpret_cast<const float4*>(dq_accum + t * (size_t)(kT * D));
    for (int e = threadIdx.x; e < kRows * D / 4; e += blockDim.x) {
        const int chunk = e / kRows, row = e - chunk * kRows;   // consecutive threads -> consecutive 16-byte units
        const float4 v = src[(size_t)chunk * kT + r0 + row];
        *reinterpret_cast<float4*>(&tile[row][chunk * 4]) = v;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < kRows * D / 8; e += blockDim.x) {
        const int row = e / (D / 8), d8 = (e - row * (D / 8)) * 8;
        const int s = qt * kT + r0 + row;
        if (s >= Sq) continue;
        const float* x = &tile[row][d8];
        uint4 w;
        w.x = pack_bf16(x[0] * scale, x[1] * scale);
        w.y = pack_bf16(x[2] * scale, x[3] * scale);
        w.z = pack_bf16(x[4] * scale, x[5] * scale);
        w.w = pack_bf16(x[6] * scale, x[7] * scale);
        *reinterpret_cast<uint4*>(dq + (bh * Sq + s) * D + d8) = w;
    }
}

// The same for the 64-bit fixed-point accumulator (tiles of [d/2][row][2] words in units of 2^-32): the one rounding
// of the exact integer sum happens here.
template <int D>
__global__ void __launch_bounds__(256) bwd_post_det_kernel(const unsigned long long* __restrict__ dq_accum, __nv_bfloat16* __restrict__ dq,
                                                           int Sq, int n_qt, float scale)
{
    constexpr int kRows = 32;
    __shared__ float tile[kRows][D + 4];
    const size_t t = blockIdx.x >> 2;
    const int r0 = (int)(blockIdx.x & 3) * kRows;
    const size_t bh = t / n_qt;
    const int qt = (int)(t - bh * n_qt);
    const ulonglong2* src = reinterpret_cast<const ulonglong2*>(dq_accum + t * (size_t)(kT * D));
    for (int e = threadIdx.x; e < kRows * D / 2; e += blockDim.x) {
        const int chunk = e / kRows, row = e - chunk * kRows;   // consecutive threads -> consecutive 16-byte units
        const ulonglong2 v = src[(size_t)chunk * kT + r0 + row];
        tile[row][chunk * 2] = (float)((double)(long long)v.x * (1.0 / 4294967296.0));
        tile[row][chunk * 2 + 1] = (float)((double)(long long)v.y * (1.0 / 4294967296.0));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < kRows * D / 8; e += blockDim.x) {
        const int row = e / (D / 8), d8 = (e - row * (D / 8)) * 8;
        const int s = qt * kT + r0 + row;
        if (s >= Sq) continue;
        const float* x = &tile[row][d8];
        uint4 w;
        w.x = pack_bf16(x[0] * scale, x[1] * scale);
        w.y = pack_bf16(x[2] * scale, x[3] * scale);
        w.z = pack_bf16(x[4] * scale, x[5] * scale);
        w.w = pack_bf16(x[6] * scale, x[7] * scale);
        *reinterpret_cast<uint4*>(dq + (bh * Sq + s) * D + d8) = w;
    }
}

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// dV / dK of the key tiles that were cut by query head: the partials of a tile are added in head order and written as
// bf16 (dK times the softmax scale).  One thread per 8 consecutive features of one key row.
template <int D>
__global__ void __launch_bounds__(256) bwd_dkv_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dk,
                                                             __nv_bfloat16* __restrict__ dv, int slabs, int group, int Skv,
                                                             float scale, long long n_units)
{
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= n_units) return;
    constexpr int kPerRow = D / 8;
    const int d8 = (int)(u % kPerRow) * 8;
    long long r = u / kPerRow;
    const int row = (int)(r % kT); r /= kT;
    const int which = (int)(r & 1); r >>= 1;              // 0: dV, 1: dK
    const int slab = (int)(r % slabs);
    const int kt = (int)(r / slabs);
    const int key = kt * kT + row;
    if (key >= Skv) return;
    const float* src = part + (((size_t)kt * slabs + slab) * group * 2 + which) * (size_t)(kT * D) + (size_t)row * D + d8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int g = 0; g < group; ++g) {
        const float4 a = *reinterpret_cast<const float4*>(src + (size_t)g * 2 * kT * D);
        const float4 c = *reinterpret_cast<const float4*>(src + (size_t)g * 2 * kT * D + 4);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += c.x; acc[5] += c.y; acc[6] += c.z; acc[7] += c.w;
    }
    const float mul = which ? scale : 1.0f;
    uint4 w;
    w.x = pack_bf16(acc[0] * mul, acc[1] * mul);
    w.y = pack_bf16(acc[2] * mul, acc[3] * mul);
    w.z = pack_bf16(acc[4] * mul, acc[5] * mul);
    w.w = pack_bf16(acc[6] * mul, acc[7] * mul);
    *reinterpret_cast<uint4*>((which ? dk : dv) + ((size_t)slab * Skv + key) * D + d8) = w;
}

template <int D, bool kWin, bool kSplit, bool kDet>
cudaError_t launch_bwd(const TcArgs& a, cudaStream_t st)
{
    const AttnShape& s = a.s;
    const int n_qt = (s.Sq + kT - 1) / kT, n_kt = (s.Skv + kT - 1) / kT;
    const int Sq_pad = n_qt * kT;
    const long long rows_padded = (long long)s.B * s.Hq * Sq_pad;
    // workspace: [delta records | LSE records] then the accumulator (see tc_backward_workspace_bytes)
    constexpr bool kAug = bwd_folds_row_terms(D);
    uint4* doaug = reinterpret_cast<uint4*>(a.delta);
    uint4* qaug = doaug + rows_padded;
    float* lse2 = a.delta + rows_padded;           // the plain-column form takes the head of the same region
    cudaError_t e;
    const int phases = a.phases ? a.phases : (kBwdPre | kBwdMain | kBwdPost);
    if (phases & kBwdPre) {
        const int warps = 8;
        const long long rows_per_block = (long long)warps * (32 / (D / 4));
        const long long blocks = (rows_padded + rows_per_block - 1) / rows_per_block;
        bwd_pre_kernel<D><<<(unsigned)blocks, warps * 32, 0, st>>>(a.o, a.dout, a.lse, kAug ? (void*)qaug : (void*)lse2,
                                                                    kAug ? (void*)doaug : (void*)a.delta, a.dq_accum, s.Sq, Sq_pad,
                                                                    rows_padded, kDet ? 2 * D : D, 1.0f / s.scale);
        count_launch();
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (phases & kBwdMain) {
    CUtensorMap tq, tk, tv, tdo;
    if ((e = encode_tmap_bf16_3d(&tq, a.q, D, s.Sq, s.B * s.Hq, 128)) != cudaSuccess) return e;
    if ((e = encode_tmap_bf16_3d(&tdo, a.dout, D, s.Sq, s.B * s.Hq, 128)) != cudaSuccess) return e;
    if ((e = encode_tmap_bf16_3d(&tk, a.k, D, s.Skv, s.B * s.Hkv, 128)) != cudaSuccess) return e;
    if ((e = encode_tmap_bf16_3d(&tv, a.v, D, s.Skv, s.B * s.Hkv, 128)) != cudaSuccess) return e;
    BwdParams p{};
    p.dk = a.dk; p.dv = a.dv;
    p.qaug = qaug; p.doaug = doaug; p.lse2 = lse2; p.delta = a.delta; p.dq_accum = a.dq_accum;
    p.B = s.B; p.Hq = s.Hq; p.Hkv = s.Hkv; p.Sq = s.Sq; p.Skv = s.Skv; p.Sq_pad = Sq_pad;
    p.causal = s.causal;
    p.window = s.causal ? s.window : 0;
    p.global_tokens = s.global_tokens;
    p.n_qt = n_qt; p.n_kt = n_kt;
    p.split_tiles = kSplit ? bwd_split_tiles(s) : 0;
    p.dkv_part = reinterpret_cast<float*>(reinterpret_cast<char*>(a.dq_accum) + align256((kDet ? 8 : 4) * (size_t)rows_padded * D));
    p.dk_acc = a.dk_acc; p.dv_acc = a.dv_acc;
    p.scale = s.scale;
    p.scale_log2 = s.scale * 1.4426950408889634f;
    const int group = s.Hq / s.Hkv, slabs = s.B * s.Hkv;
    const long long ctas = (long long)p.split_tiles * group * slabs + (long long)(n_kt - p.split_tiles) * slabs;
    if (ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    static std::atomic<unsigned long long> configured{0};   // per instantiation, one bit per device
    {
        constexpr int kDoStages = (D == 128) ? 1 : 2;
        // K, V, Q stages, dO stages; the dS tile (two at head_dim 64); dQ staging; the per-query terms (see sTail in the kernel)
        constexpr int kQStages = (D == 128) ? 2 : 3;
        const size_t smem = (size_t)(128 * D * 2) * (2 + kQStages + kDoStages) + (D == 128 ? 1 : 2) * 128 * 128 * 2 + 32 * 1024 +
                            (kAug ? (size_t)(2 + kQStages + kDoStages) * 128 * 16 : (size_t)2 * kQStages * 128 * 4) + sizeof(BwdBarriers);
        if ((e = ensure_dynamic_smem(attn_bwd_tc_kernel<D, kWin, kSplit, kDet>, smem, configured)) != cudaSuccess) return e;
        attn_bwd_tc_kernel<D, kWin, kSplit, kDet><<<(unsigned)ctas, kBwdThreads, smem, st>>>(tq, tk, tv, tdo, p);
    }
    count_launch();
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if (p.split_tiles > 0) {
        const long long n_units = (long long)p.split_tiles * slabs * 2 * kT * (D / 8);
        bwd_dkv_reduce_kernel<D><<<(unsigned)((n_units + 255) / 256), 256, 0, st>>>(p.dkv_part, a.dk, a.dv, slabs, group, s.Skv,
                                                                                   s.scale, n_units);
        count_launch();
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    }   // kBwdMain
    if (!(phases & kBwdPost)) return cudaSuccess;
    if (kDet)
        bwd_post_det_kernel<D><<<(unsigned)((long long)s.B * s.Hq * n_qt * 4), 256, 0, st>>>(
            reinterpret_cast<const unsigned long long*>(a.dq_accum), a.dq, s.Sq, n_qt, s.scale);
    else
        bwd_post_kernel<D><<<(unsigned)((long long)s.B * s.Hq * n_qt * 4), 256, 0, st>>>(a.dq_accum, a.dq, s.Sq, n_qt, s.scale);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

bool tc_bwd_supported(const AttnShape& s)
{
    return (s.D == 64 || s.D == 128) && (!s.causal || s.Sq == s.Skv);
}

// [delta records: B*Hq*Sq_pad x 16 bytes][LSE records: same], 256-byte aligned, then the fp32 dQ accumulator B*Hq*Sq_pad*D, then the fp32
// dK/dV partials of the key tiles that are cut by query head (none for most shapes)
size_t tc_backward_workspace_bytes(const AttnShape& s)
{
    const size_t sq_pad = ((size_t)s.Sq + kT - 1) / kT * kT;
    const size_t rows = (size_t)s.B * s.Hq * sq_pad;
    const size_t part = (size_t)bwd_split_tiles(s) * s.B * s.Hq * 2 * kT * (size_t)s.D * 4;   // slabs * group = B * Hq
    return align256(kBwdRowAuxBytes * rows) + align256((s.deterministic ? 8 : 4) * rows * (size_t)s.D) + align256(part);
}

cudaError_t tc_backward(const TcArgs& a, cudaStream_t st)
{
    const bool win = a.s.causal && a.s.window > 0;
    if (a.s.deterministic) {   // (bwd_split_tiles is 0 for this form)
        if (a.s.D == 64) return win ? launch_bwd<64, true, false, true>(a, st) : launch_bwd<64, false, false, true>(a, st);
        return win ? launch_bwd<128, true, false, true>(a, st) : launch_bwd<128, false, false, true>(a, st);
    }
    // the accumulate form has no cut key tiles: their fp32 partials would need a second adding pass
    if (a.dk_acc == nullptr && bwd_split_tiles(a.s) > 0) {
        if (a.s.D == 64) return win ? launch_bwd<64, true, true, false>(a, st) : launch_bwd<64, false, true, false>(a, st);
        return win ? launch_bwd<128, true, true, false>(a, st) : launch_bwd<128, false, true, false>(a, st);
    }
    if (a.s.D == 64) return win ? launch_bwd<64, true, false, false>(a, st) : launch_bwd<64, false, false, false>(a, st);
    return win ? launch_bwd<128, true, false, false>(a, st) : launch_bwd<128, false, false, false>(a, st);
}

#ifdef SNTL_TRACE
// trace build only: choose the CTA that records and read back what the last launch recorded
extern "C" int sntl_debug_trace_bwd(unsigned long long* out, int n_words, int set_cta)
{
    if (out && cudaMemcpyFromSymbol(out, ptx::g_trace, sizeof(unsigned long long) * n_words) != cudaSuccess) return 1;
    static unsigned long long zeros[ptx::kTraceRoles * ptx::kTraceDepth];
    if (cudaMemcpyToSymbol(ptx::g_trace, zeros, sizeof(zeros)) != cudaSuccess) return 2;
    unsigned int c = (unsigned int)set_cta;
    return cudaMemcpyToSymbol(ptx::g_trace_cta, &c, sizeof(c)) == cudaSuccess ? 0 : 3;
}
#endif

cudaError_t read_and_clear_bwd_status(cudaStream_t st, uint32_t* word)
{
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return e;
    unsigned int w = 0, zero = 0;
    if ((e = cudaMemcpyFromSymbol(&w, ptx::g_device_status, sizeof(w))) != cudaSuccess) return e;
    if (w != 0 && (e = cudaMemcpyToSymbol(ptx::g_device_status, &zero, sizeof(zero))) != cudaSuccess) return e;
    *word = w;
    return cudaSuccess;
}

}  // namespace sntl

// C ABI of the attention library: argument validation, path selection, workspace carving.
// Mirrors the host-side duties of CudaFlashAttention::forwardMultiHead / backwardMultiHead
// (sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1543-1609, :1615-1700): validate shapes and the column
// window, pick a kernel, launch on the caller's stream, report launch errors.  Unlike the reference it never
// allocates: scratch comes from the caller.
#include "common.cuh"

#include <atomic>
#include <string.h>

namespace sntl {

static std::atomic<uint64_t> g_launches{0};
static thread_local const char* g_last_path = "none";

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

namespace {

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

int validate(const sntl_attn_desc* d)
{
    if (!d) return SNTL_ERR_BAD_ARGUMENT;
    if (d->dtype != SNTL_DTYPE_BF16 && d->dtype != SNTL_DTYPE_F32) return SNTL_ERR_BAD_ARGUMENT;
    if (d->layout != SNTL_LAYOUT_BHSD && d->layout != SNTL_LAYOUT_SENTINEL) return SNTL_ERR_BAD_ARGUMENT;
    if (d->batch <= 0 || d->q_heads <= 0 || d->kv_heads <= 0 || d->seq_q <= 0 || d->seq_kv <= 0 || d->head_dim <= 0)
        return SNTL_ERR_BAD_ARGUMENT;
    if (d->q_heads % d->kv_heads != 0) return SNTL_ERR_BAD_ARGUMENT;
    if (d->causal && d->seq_q != d->seq_kv) return SNTL_ERR_BAD_ARGUMENT;
    if (!(d->scale > 0.0f)) return SNTL_ERR_BAD_ARGUMENT;
    if (d->global_tokens < 0) return SNTL_ERR_BAD_ARGUMENT;   // CausalSelfAttention.cpp:42
    if ((d->window_size > 0 || d->global_tokens > 0) && !d->causal) return SNTL_ERR_BAD_ARGUMENT;
    if (d->head_dim > 256) return SNTL_ERR_UNSUPPORTED;
    if (d->batch > 65535 || d->q_heads > 65535) return SNTL_ERR_UNSUPPORTED;
    if (d->layout == SNTL_LAYOUT_SENTINEL) {
        if (d->dtype != SNTL_DTYPE_F32) return SNTL_ERR_UNSUPPORTED;
        if (d->seq_q != d->seq_kv) return SNTL_ERR_BAD_ARGUMENT;
        // window [column_start, column_start + batch*seq) must lie inside the matrix (CudaFlashAttention.cu:1533-1539)
        if (d->column_start < 0 || d->stride_columns <= 0) return SNTL_ERR_BAD_ARGUMENT;
        if ((long long)d->column_start + (long long)d->batch * d->seq_q > (long long)d->stride_columns) return SNTL_ERR_BAD_ARGUMENT;
    }
    return SNTL_OK;
}

AttnShape shape_of(const sntl_attn_desc* d)
{
    // a window that already covers the sequence is plain causal attention
    const int window = (d->window_size > 0 && d->window_size < d->seq_kv) ? d->window_size : 0;
    return AttnShape{d->batch, d->q_heads, d->kv_heads, d->seq_q, d->seq_kv, d->head_dim, d->scale, d->causal ? 1 : 0,
                     window, window > 0 ? d->global_tokens : 0, (d->flags & SNTL_FLAG_DETERMINISTIC) ? 1 : 0};
}

// tensor-core path is taken for bf16 tensors, or fp32 tensors when the caller allows bf16 operands
bool wants_tc(const sntl_attn_desc* d, bool backward)
{
    if (d->flags & SNTL_FLAG_FORCE_SIMT) return false;
    if (d->dtype == SNTL_DTYPE_F32 && !(d->flags & SNTL_FLAG_ALLOW_BF16_COMPUTE)) return false;
    return backward ? tc_bwd_supported(shape_of(d)) : tc_fwd_supported(shape_of(d));
}

bool needs_staging(const sntl_attn_desc* d) { return d->dtype == SNTL_DTYPE_F32 || d->layout == SNTL_LAYOUT_SENTINEL; }

void views(const sntl_attn_desc* d, View4& vq, View4& vkv, View3& vlse)
{
    const long long D = d->head_dim;
    if (d->layout == SNTL_LAYOUT_BHSD) {
        vq = View4{(long long)d->q_heads * d->seq_q * D, (long long)d->seq_q * D, D, 1};
        vkv = View4{(long long)d->kv_heads * d->seq_kv * D, (long long)d->seq_kv * D, D, 1};
        vlse = View3{(long long)d->q_heads * d->seq_q, (long long)d->seq_q, 1};
    } else {
        const long long C = d->stride_columns;
        vq = View4{(long long)d->seq_q, D * C, 1, C};
        vkv = View4{(long long)d->seq_kv, D * C, 1, C};
        vlse = View3{(long long)d->seq_q, C, 1};
    }
}

struct Carve {
    char* p;
    size_t left;
    bool ok = true;
    void* take(size_t bytes)
    {
        bytes = align_up(bytes);
        if (bytes > left) { ok = false; return nullptr; }
        void* r = p;
        p += bytes;
        left -= bytes;
        return r;
    }
};

size_t nq_elems(const sntl_attn_desc* d) { return (size_t)d->batch * d->q_heads * d->seq_q * d->head_dim; }
size_t nkv_elems(const sntl_attn_desc* d) { return (size_t)d->batch * d->kv_heads * d->seq_kv * d->head_dim; }
size_t nlse(const sntl_attn_desc* d) { return (size_t)d->batch * d->q_heads * d->seq_q; }

int cuda_status(cudaError_t e) { return e == cudaSuccess ? SNTL_OK : SNTL_ERR_CUDA; }

bool device_ok()
{
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
    return major == 10;
}

// Stage one tensor of `heads` heads into bf16 BHSD.
cudaError_t stage_in(const sntl_attn_desc* d, const void* src, __nv_bfloat16* dst, int heads, int S, cudaStream_t st)
{
    if (d->layout == SNTL_LAYOUT_SENTINEL)
        return sentinel_to_bhsd_bf16((const float*)src, dst, d->batch, heads, S, d->head_dim, d->stride_columns, d->column_start, st);
    return f32_to_bf16((const float*)src, dst, (size_t)d->batch * heads * S * d->head_dim, st);
}
cudaError_t stage_out(const sntl_attn_desc* d, const __nv_bfloat16* src, void* dst, int heads, int S, cudaStream_t st)
{
    if (d->layout == SNTL_LAYOUT_SENTINEL)
        return bhsd_bf16_to_sentinel(src, (float*)dst, d->batch, heads, S, d->head_dim, d->stride_columns, d->column_start, st);
    return bf16_to_f32(src, (float*)dst, (size_t)d->batch * heads * S * d->head_dim, st);
}

}  // namespace
}  // namespace sntl

using namespace sntl;

extern "C" {

int sntl_attn_version(void) { return 100; }

const char* sntl_status_string(int status)
{
    switch (status) {
        case SNTL_OK: return "ok";
        case SNTL_ERR_BAD_ARGUMENT: return "bad argument";
        case SNTL_ERR_UNSUPPORTED: return "unsupported shape, dtype or layout";
        case SNTL_ERR_WORKSPACE: return "workspace missing or too small";
        case SNTL_ERR_CUDA: return "CUDA call or kernel launch failed";
        case SNTL_ERR_NO_DEVICE: return "no compute-capability-10.x device is current";
        case SNTL_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case SNTL_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the library's built-in 32 MiB array";
        case SNTL_ERR_COMM: return "NCCL is not available or an NCCL call failed";
        default: return "unknown status";
    }
}

const char* sntl_attn_last_path(void) { return g_last_path; }

uint64_t sntl_attn_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

size_t sntl_attn_fwd_workspace_bytes(const sntl_attn_desc* d)
{
    if (validate(d) != SNTL_OK) return 0;
    if (!wants_tc(d, false) || !needs_staging(d)) return 0;
    // bf16 copies of Q, K, V, O and a [B][Hq][S] LSE when the caller's LSE is feature-major
    return align_up(2 * nq_elems(d)) * 2 + align_up(2 * nkv_elems(d)) * 2 + align_up(4 * nlse(d));
}

size_t sntl_attn_bwd_workspace_bytes(const sntl_attn_desc* d)
{
    if (validate(d) != SNTL_OK) return 0;
    size_t bytes = align_up(4 * nlse(d));  // delta (exact path) -- the tensor-core path sizes its own below
    if (!wants_tc(d, true)) return bytes;
    bytes = align_up(tc_backward_workspace_bytes(shape_of(d)));
    if (needs_staging(d))  // bf16 Q,O,dO,dQ + K,V,dK,dV + LSE
        bytes += align_up(2 * nq_elems(d)) * 4 + align_up(2 * nkv_elems(d)) * 4 + align_up(4 * nlse(d));
    return bytes;
}

int sntl_attn_fwd(const sntl_attn_desc* d, const void* q, const void* k, const void* v, void* o, float* lse,
                  void* workspace, size_t workspace_bytes, void* stream)
{
    int rc = validate(d);
    if (rc != SNTL_OK) return rc;
    if (!q || !k || !v || !o || !lse) return SNTL_ERR_BAD_ARGUMENT;
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t need = sntl_attn_fwd_workspace_bytes(d);
    if (need && (!workspace || workspace_bytes < need)) return SNTL_ERR_WORKSPACE;

    if (!wants_tc(d, false)) {
        if (d->head_dim % 2 != 0) return SNTL_ERR_UNSUPPORTED;
        SimtArgs a{};
        a.s = shape_of(d);
        a.is_bf16 = d->dtype == SNTL_DTYPE_BF16;
        // feature-major matrices: the window starts column_start elements into every row
        const size_t off = d->layout == SNTL_LAYOUT_SENTINEL ? (size_t)d->column_start * sizeof(float) : 0;
        a.q = (const char*)q + off; a.k = (const char*)k + off; a.v = (const char*)v + off;
        a.o_out = (char*)o + off; a.lse_out = (float*)((char*)lse + off);
        views(d, a.vq, a.vkv, a.vlse);
        g_last_path = a.is_bf16 ? "simt_bf16" : "simt_f32";
        return cuda_status(simt_forward(a, st));
    }

    TcArgs t{};
    t.s = shape_of(d);
    g_last_path = "tcgen05";
    if (!needs_staging(d)) {
        t.q = (const __nv_bfloat16*)q; t.k = (const __nv_bfloat16*)k; t.v = (const __nv_bfloat16*)v;
        t.o_out = (__nv_bfloat16*)o; t.lse_out = lse;
        return cuda_status(tc_forward(t, st));
    }
    g_last_path = "tcgen05_staged";
    Carve c{(char*)workspace, workspace_bytes};
    auto* qb = (__nv_bfloat16*)c.take(2 * nq_elems(d));
    auto* ob = (__nv_bfloat16*)c.take(2 * nq_elems(d));
    auto* kb = (__nv_bfloat16*)c.take(2 * nkv_elems(d));
    auto* vb = (__nv_bfloat16*)c.take(2 * nkv_elems(d));
    auto* lb = (float*)c.take(4 * nlse(d));
    if (!c.ok) return SNTL_ERR_WORKSPACE;
    cudaError_t e;
    if ((e = stage_in(d, q, qb, d->q_heads, d->seq_q, st)) != cudaSuccess) return SNTL_ERR_CUDA;
    if ((e = stage_in(d, k, kb, d->kv_heads, d->seq_kv, st)) != cudaSuccess) return SNTL_ERR_CUDA;
    if ((e = stage_in(d, v, vb, d->kv_heads, d->seq_kv, st)) != cudaSuccess) return SNTL_ERR_CUDA;
    t.q = qb; t.k = kb; t.v = vb; t.o_out = ob;
    t.lse_out = d->layout == SNTL_LAYOUT_SENTINEL ? lb : lse;
    if ((e = tc_forward(t, st)) != cudaSuccess) return SNTL_ERR_CUDA;
    if ((e = stage_out(d, ob, o, d->q_heads, d->seq_q, st)) != cudaSuccess) return SNTL_ERR_CUDA;
    if (d->layout == SNTL_LAYOUT_SENTINEL &&
        (e = lse_bhs_to_sentinel(lb, lse, d->batch, d->q_heads, d->seq_q, d->stride_columns, d->column_start, st)) != cudaSuccess)
        return SNTL_ERR_CUDA;
    return SNTL_OK;
}

namespace sntl {
namespace {

// seq_q new tokens per head against seq_kv cached keys (the new tokens' own keys included, at the end)
int validate_cached(const sntl_attn_desc* d, int32_t capacity)
{
    if (!d) return SNTL_ERR_BAD_ARGUMENT;
    if (d->dtype != SNTL_DTYPE_BF16 && d->dtype != SNTL_DTYPE_F32) return SNTL_ERR_BAD_ARGUMENT;
    if (d->layout != SNTL_LAYOUT_BHSD && d->layout != SNTL_LAYOUT_SENTINEL) return SNTL_ERR_BAD_ARGUMENT;
    if (d->batch <= 0 || d->q_heads <= 0 || d->kv_heads <= 0 || d->seq_q <= 0 || d->seq_kv <= 0 || d->head_dim <= 0)
        return SNTL_ERR_BAD_ARGUMENT;
    if (d->q_heads % d->kv_heads != 0) return SNTL_ERR_BAD_ARGUMENT;
    if (!d->causal) return SNTL_ERR_BAD_ARGUMENT;                 // a cached query never sees later keys
    if (d->seq_q > d->seq_kv) return SNTL_ERR_BAD_ARGUMENT;       // the new tokens are appended before the call
    if (capacity < d->seq_kv) return SNTL_ERR_BAD_ARGUMENT;       // CudaCausalSelfAttention.cu:566 (cache full)
    if (!(d->scale > 0.0f)) return SNTL_ERR_BAD_ARGUMENT;
    if (d->global_tokens < 0) return SNTL_ERR_BAD_ARGUMENT;
    if (d->head_dim > 256 || d->head_dim % 2 != 0) return SNTL_ERR_UNSUPPORTED;
    if (d->batch > 65535 || d->q_heads > 65535) return SNTL_ERR_UNSUPPORTED;
    if (d->layout == SNTL_LAYOUT_SENTINEL) {
        if (d->dtype != SNTL_DTYPE_F32) return SNTL_ERR_UNSUPPORTED;
        if (d->batch != 1) return SNTL_ERR_UNSUPPORTED;           // the reference's cache holds one sequence
        if (d->column_start < 0 || d->stride_columns <= 0) return SNTL_ERR_BAD_ARGUMENT;
        if ((long long)d->column_start + d->seq_q > (long long)d->stride_columns) return SNTL_ERR_BAD_ARGUMENT;
    }
    return SNTL_OK;
}

bool cached_wants_tc(const sntl_attn_desc* d)
{
    if (d->flags & SNTL_FLAG_FORCE_SIMT) return false;
    if (d->dtype != SNTL_DTYPE_BF16 || d->layout != SNTL_LAYOUT_BHSD) return false;
    return tc_cache_supported(shape_of(d));
}

}  // namespace
}  // namespace sntl

size_t sntl_attn_cached_fwd_workspace_bytes(const sntl_attn_desc* d, int32_t cache_capacity)
{
    if (validate_cached(d, cache_capacity) != SNTL_OK || !cached_wants_tc(d)) return 0;
    return tc_cache_workspace_bytes(shape_of(d));
}

int sntl_attn_cached_fwd(const sntl_attn_desc* d, const void* q, const void* k_cache, const void* v_cache,
                         int32_t cache_capacity, void* o, float* lse, void* workspace, size_t workspace_bytes, void* stream)
{
    int rc = validate_cached(d, cache_capacity);
    if (rc != SNTL_OK) return rc;
    if (!q || !k_cache || !v_cache || !o || !lse) return SNTL_ERR_BAD_ARGUMENT;
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    if (cached_wants_tc(d)) {
        const size_t need = tc_cache_workspace_bytes(shape_of(d));
        if (need && (!workspace || workspace_bytes < need)) return SNTL_ERR_WORKSPACE;
        TcArgs t{};
        t.s = shape_of(d);
        t.q = (const __nv_bfloat16*)q; t.k = (const __nv_bfloat16*)k_cache; t.v = (const __nv_bfloat16*)v_cache;
        t.o_out = (__nv_bfloat16*)o; t.lse_out = lse;
        g_last_path = "tcgen05_cache";
        return cuda_status(tc_cache_forward(t, cache_capacity, workspace, st));
    }
    // exact kernels: the same forward kernel, keys addressed with the cache's row pitch
    SimtArgs a{};
    a.s = shape_of(d);
    a.is_bf16 = d->dtype == SNTL_DTYPE_BF16;
    const size_t off = d->layout == SNTL_LAYOUT_SENTINEL ? (size_t)d->column_start * sizeof(float) : 0;
    a.q = (const char*)q + off; a.k = k_cache; a.v = v_cache;
    a.o_out = (char*)o + off; a.lse_out = (float*)((char*)lse + off);
    views(d, a.vq, a.vkv, a.vlse);
    const long long D = d->head_dim, C = cache_capacity;
    a.vkv = d->layout == SNTL_LAYOUT_BHSD ? View4{(long long)d->kv_heads * C * D, C * D, D, 1} : View4{0, D * C, 1, C};
    g_last_path = a.is_bf16 ? "simt_bf16" : "simt_f32";
    return cuda_status(simt_forward(a, st));
}

int sntl_attn_bwd(const sntl_attn_desc* d, const void* q, const void* k, const void* v, const void* o,
                  const float* lse, const void* dout, void* dq, void* dk, void* dv, void* workspace,
                  size_t workspace_bytes, void* stream)
{
    int rc = validate(d);
    if (rc != SNTL_OK) return rc;
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv) return SNTL_ERR_BAD_ARGUMENT;
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t need = sntl_attn_bwd_workspace_bytes(d);
    if (!workspace || workspace_bytes < need) return SNTL_ERR_WORKSPACE;
    Carve c{(char*)workspace, workspace_bytes};

    if (!wants_tc(d, true)) {
        if (d->head_dim % 2 != 0) return SNTL_ERR_UNSUPPORTED;
        SimtArgs a{};
        a.s = shape_of(d);
        a.is_bf16 = d->dtype == SNTL_DTYPE_BF16;
        const size_t off = d->layout == SNTL_LAYOUT_SENTINEL ? (size_t)d->column_start * sizeof(float) : 0;
        a.q = (const char*)q + off; a.k = (const char*)k + off; a.v = (const char*)v + off;
        a.o = (const char*)o + off; a.dout = (const char*)dout + off; a.lse = (const float*)((const char*)lse + off);
        a.dq = (char*)dq + off; a.dk = (char*)dk + off; a.dv = (char*)dv + off;
        a.delta = (float*)c.take(4 * nlse(d));
        if (!c.ok) return SNTL_ERR_WORKSPACE;
        views(d, a.vq, a.vkv, a.vlse);
        a.vdelta = View3{(long long)d->q_heads * d->seq_q, (long long)d->seq_q, 1};
        g_last_path = a.is_bf16 ? "simt_bf16" : "simt_f32";
        return cuda_status(simt_backward(a, st));
    }

    TcArgs t{};
    t.s = shape_of(d);
    char* tcws = (char*)c.take(tc_backward_workspace_bytes(t.s));
    if (!c.ok) return SNTL_ERR_WORKSPACE;
    const size_t sq_pad = ((size_t)d->seq_q + 127) / 128 * 128;
    t.delta = (float*)tcws;
    t.dq_accum = (float*)(tcws + align_up(kBwdRowAuxBytes * (size_t)d->batch * d->q_heads * sq_pad));  // after the per-row records
    g_last_path = "tcgen05";
    if (!needs_staging(d)) {
        t.q = (const __nv_bfloat16*)q; t.k = (const __nv_bfloat16*)k; t.v = (const __nv_bfloat16*)v;
        t.o = (const __nv_bfloat16*)o; t.dout = (const __nv_bfloat16*)dout; t.lse = lse;
        t.dq = (__nv_bfloat16*)dq; t.dk = (__nv_bfloat16*)dk; t.dv = (__nv_bfloat16*)dv;
        return cuda_status(tc_backward(t, st));
    }
    g_last_path = "tcgen05_staged";
    auto* qb = (__nv_bfloat16*)c.take(2 * nq_elems(d));
    auto* ob = (__nv_bfloat16*)c.take(2 * nq_elems(d));
    auto* gb = (__nv_bfloat16*)c.take(2 * nq_elems(d));
    auto* dqb = (__nv_bfloat16*)c.take(2 * nq_elems(d));
    auto* kb = (__nv_bfloat16*)c.take(2 * nkv_elems(d));
    auto* vb = (__nv_bfloat16*)c.take(2 * nkv_elems(d));
    auto* dkb = (__nv_bfloat16*)c.take(2 * nkv_elems(d));
    auto* dvb = (__nv_bfloat16*)c.take(2 * nkv_elems(d));
    auto* lb = (float*)c.take(4 * nlse(d));
    if (!c.ok) return SNTL_ERR_WORKSPACE;
    if (stage_in(d, q, qb, d->q_heads, d->seq_q, st) != cudaSuccess) return SNTL_ERR_CUDA;
    if (stage_in(d, o, ob, d->q_heads, d->seq_q, st) != cudaSuccess) return SNTL_ERR_CUDA;
    if (stage_in(d, dout, gb, d->q_heads, d->seq_q, st) != cudaSuccess) return SNTL_ERR_CUDA;
    if (stage_in(d, k, kb, d->kv_heads, d->seq_kv, st) != cudaSuccess) return SNTL_ERR_CUDA;
    if (stage_in(d, v, vb, d->kv_heads, d->seq_kv, st) != cudaSuccess) return SNTL_ERR_CUDA;
    t.lse = lse;
    if (d->layout == SNTL_LAYOUT_SENTINEL) {
        if (lse_sentinel_to_bhs(lse, lb, d->batch, d->q_heads, d->seq_q, d->stride_columns, d->column_start, st) != cudaSuccess)
            return SNTL_ERR_CUDA;
        t.lse = lb;
    }
    t.q = qb; t.k = kb; t.v = vb; t.o = ob; t.dout = gb; t.dq = dqb; t.dk = dkb; t.dv = dvb;
    if (tc_backward(t, st) != cudaSuccess) return SNTL_ERR_CUDA;
    if (stage_out(d, dqb, dq, d->q_heads, d->seq_q, st) != cudaSuccess) return SNTL_ERR_CUDA;
    if (stage_out(d, dkb, dk, d->kv_heads, d->seq_kv, st) != cudaSuccess) return SNTL_ERR_CUDA;
    if (stage_out(d, dvb, dv, d->kv_heads, d->seq_kv, st) != cudaSuccess) return SNTL_ERR_CUDA;
    return SNTL_OK;
}

// ---- backward in pieces ----
namespace sntl {
namespace {
int validate_pieces(const sntl_attn_desc* d)
{
    const int rc = validate(d);
    if (rc != SNTL_OK) return rc;
    if (d->dtype != SNTL_DTYPE_BF16 || d->layout != SNTL_LAYOUT_BHSD) return SNTL_ERR_UNSUPPORTED;
    if (d->window_size > 0 || d->global_tokens > 0) return SNTL_ERR_UNSUPPORTED;
    if (d->flags & (SNTL_FLAG_FORCE_SIMT | SNTL_FLAG_DETERMINISTIC)) return SNTL_ERR_UNSUPPORTED;
    if (!tc_bwd_supported(shape_of(d))) return SNTL_ERR_UNSUPPORTED;
    return SNTL_OK;
}
size_t pieces_workspace_bytes(const sntl_attn_desc* d)
{
    const size_t sq_pad = ((size_t)d->seq_q + 127) / 128 * 128;
    const size_t rows = (size_t)d->batch * d->q_heads * sq_pad;
    return align_up(kBwdRowAuxBytes * rows) + align_up(4 * rows * (size_t)d->head_dim);
}
void pieces_args(const sntl_attn_desc* d, void* workspace, TcArgs& t)
{
    t.s = shape_of(d);
    const size_t sq_pad = ((size_t)d->seq_q + 127) / 128 * 128;
    t.delta = (float*)workspace;
    t.dq_accum = (float*)((char*)workspace + align_up(kBwdRowAuxBytes * (size_t)d->batch * d->q_heads * sq_pad));
}
}  // namespace
}  // namespace sntl

size_t sntl_attn_bwd_pieces_workspace_bytes(const sntl_attn_desc* d)
{
    return validate_pieces(d) == SNTL_OK ? pieces_workspace_bytes(d) : 0;
}

int sntl_attn_bwd_begin(const sntl_attn_desc* d, const void* o, const float* lse, const void* dout, void* workspace,
                        size_t workspace_bytes, void* stream)
{
    const int rc = validate_pieces(d);
    if (rc != SNTL_OK) return rc;
    if (!o || !lse || !dout) return SNTL_ERR_BAD_ARGUMENT;
    if (!workspace || workspace_bytes < pieces_workspace_bytes(d)) return SNTL_ERR_WORKSPACE;
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    TcArgs t{};
    pieces_args(d, workspace, t);
    t.o = (const __nv_bfloat16*)o; t.dout = (const __nv_bfloat16*)dout; t.lse = lse;
    t.phases = kBwdPre;
    g_last_path = "tcgen05";
    return cuda_status(tc_backward(t, (cudaStream_t)stream));
}

int sntl_attn_bwd_block(const sntl_attn_desc* d, const void* q, const void* k, const void* v, const void* dout, float* dk_acc,
                        float* dv_acc, void* workspace, size_t workspace_bytes, void* stream)
{
    const int rc = validate_pieces(d);
    if (rc != SNTL_OK) return rc;
    if (!q || !k || !v || !dout || !dk_acc || !dv_acc) return SNTL_ERR_BAD_ARGUMENT;
    if (!workspace || workspace_bytes < pieces_workspace_bytes(d)) return SNTL_ERR_WORKSPACE;
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    TcArgs t{};
    pieces_args(d, workspace, t);
    t.q = (const __nv_bfloat16*)q; t.k = (const __nv_bfloat16*)k; t.v = (const __nv_bfloat16*)v;
    t.dout = (const __nv_bfloat16*)dout;
    t.dk_acc = dk_acc; t.dv_acc = dv_acc;
    t.phases = kBwdMain;
    g_last_path = "tcgen05";
    return cuda_status(tc_backward(t, (cudaStream_t)stream));
}

int sntl_attn_bwd_end(const sntl_attn_desc* d, void* dq, void* workspace, size_t workspace_bytes, void* stream)
{
    const int rc = validate_pieces(d);
    if (rc != SNTL_OK) return rc;
    if (!dq) return SNTL_ERR_BAD_ARGUMENT;
    if (!workspace || workspace_bytes < pieces_workspace_bytes(d)) return SNTL_ERR_WORKSPACE;
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    TcArgs t{};
    pieces_args(d, workspace, t);
    t.dq = (__nv_bfloat16*)dq;
    t.phases = kBwdPost;
    g_last_path = "tcgen05";
    return cuda_status(tc_backward(t, (cudaStream_t)stream));
}

int sntl_attn_merge(int32_t acc_dtype, int32_t part_dtype, int64_t rows, int32_t head_dim, void* o_acc, float* lse_acc,
                    const void* o_part, const float* lse_part, void* stream)
{
    if (rows < 0 || head_dim <= 0 || !o_acc || !lse_acc || !o_part || !lse_part) return SNTL_ERR_BAD_ARGUMENT;
    if ((acc_dtype != SNTL_DTYPE_BF16 && acc_dtype != SNTL_DTYPE_F32) ||
        (part_dtype != SNTL_DTYPE_BF16 && part_dtype != SNTL_DTYPE_F32))
        return SNTL_ERR_BAD_ARGUMENT;
    return cuda_status(merge_partials(acc_dtype, part_dtype, rows, head_dim, o_acc, lse_acc, o_part, lse_part, (cudaStream_t)stream));
}

int sntl_attn_accumulate(int32_t part_dtype, int64_t count, float* acc, const void* part, void* stream)
{
    if (count < 0 || !acc || !part) return SNTL_ERR_BAD_ARGUMENT;
    if (part_dtype != SNTL_DTYPE_BF16 && part_dtype != SNTL_DTYPE_F32) return SNTL_ERR_BAD_ARGUMENT;
    return cuda_status(accumulate_f32(part_dtype, acc, part, (size_t)count, (cudaStream_t)stream));
}

namespace sntl {
namespace {
int validate_pack(const void* a, const void* b, int32_t batch, int32_t heads, int32_t seq, int32_t head_dim, int32_t stride_columns,
                  int32_t column_start, const float* cos_table, const float* sin_table, int32_t position_offset,
                  int32_t table_positions)
{
    if (!a || !b) return SNTL_ERR_BAD_ARGUMENT;
    if (batch <= 0 || heads <= 0 || seq <= 0 || head_dim <= 0 || head_dim % 2 != 0) return SNTL_ERR_BAD_ARGUMENT;   // RotaryEmbedding.cpp:11
    if (column_start < 0 || stride_columns <= 0) return SNTL_ERR_BAD_ARGUMENT;
    if ((long long)column_start + (long long)batch * seq > (long long)stride_columns) return SNTL_ERR_BAD_ARGUMENT;
    if ((cos_table == nullptr) != (sin_table == nullptr)) return SNTL_ERR_BAD_ARGUMENT;
    // RotaryEmbedding.cpp:42: a sequence longer than the table is an argument error
    if (cos_table && (position_offset < 0 || (long long)position_offset + seq > (long long)table_positions)) return SNTL_ERR_BAD_ARGUMENT;
    if (batch > 65535 || heads > 65535 || (long long)batch * heads > 65535) return SNTL_ERR_UNSUPPORTED;
    return SNTL_OK;
}
}  // namespace
}  // namespace sntl

int sntl_attn_pack_heads(const float* src, void* dst, int32_t batch, int32_t heads, int32_t seq, int32_t head_dim,
                         int32_t stride_columns, int32_t column_start, const float* cos_table, const float* sin_table,
                         int32_t position_offset, int32_t table_positions, void* stream)
{
    const int rc = validate_pack(src, dst, batch, heads, seq, head_dim, stride_columns, column_start, cos_table, sin_table,
                                 position_offset, table_positions);
    if (rc != SNTL_OK) return rc;
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    return cuda_status(rope_pack_bf16(src, (__nv_bfloat16*)dst, batch, heads, seq, head_dim, stride_columns, column_start, cos_table,
                                      sin_table, position_offset, (cudaStream_t)stream));
}

int sntl_attn_unpack_heads(const void* src, float* dst, int32_t batch, int32_t heads, int32_t seq, int32_t head_dim,
                           int32_t stride_columns, int32_t column_start, const float* cos_table, const float* sin_table,
                           int32_t position_offset, int32_t table_positions, int32_t inverse, void* stream)
{
    const int rc = validate_pack(src, dst, batch, heads, seq, head_dim, stride_columns, column_start, cos_table, sin_table,
                                 position_offset, table_positions);
    if (rc != SNTL_OK) return rc;
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    return cuda_status(rope_unpack_f32((const __nv_bfloat16*)src, dst, batch, heads, seq, head_dim, stride_columns, column_start,
                                       cos_table, sin_table, position_offset, inverse != 0, (cudaStream_t)stream));
}

int sntl_attn_poll_device_status_words(void* stream, uint32_t* forward_word, uint32_t* backward_word)
{
    uint32_t word = 0, word_bwd = 0;
    if (read_and_clear_fwd_status((cudaStream_t)stream, &word) != cudaSuccess) return SNTL_ERR_CUDA;
    if (read_and_clear_bwd_status((cudaStream_t)stream, &word_bwd) != cudaSuccess) return SNTL_ERR_CUDA;
    if (forward_word) *forward_word = word;
    if (backward_word) *backward_word = word_bwd;
    return (word | word_bwd) == 0 ? SNTL_OK : SNTL_ERR_DEVICE_TIMEOUT;
}

int sntl_attn_poll_device_status(void* stream, uint32_t* detail)
{
    uint32_t word = 0, word_bwd = 0;
    const int rc = sntl_attn_poll_device_status_words(stream, &word, &word_bwd);
    if (detail) *detail = word ? word : word_bwd;
    return rc;
}

int sntl_attn_selftest_wait_timeout(uint32_t limit_us, void* stream)
{
    if (limit_us == 0 || limit_us > 100000u) return SNTL_ERR_BAD_ARGUMENT;   // 0.1 s at most: this is a test hook
    if (!device_ok()) return SNTL_ERR_NO_DEVICE;
    return cuda_status(launch_wait_selftest((unsigned long long)limit_us * 1000ull, nullptr, (cudaStream_t)stream));
}

}  // extern "C"

// Shared declarations of the attention library's translation units.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "sntl_attn.h"

namespace sntl {

// Element strides of a [B][H][S][D]-indexed tensor; covers both layouts of the C ABI.
struct View4 {
    long long sb, sh, ss, sd;
};
// Element strides of a [B][H][S]-indexed fp32 tensor (LSE, delta).
struct View3 {
    long long sb, sh, ss;
};

struct AttnShape {
    int B, Hq, Hkv, Sq, Skv, D;
    float scale;
    int causal;
    int window;         // sliding window (keys a query sees counting itself); <= 0: unlimited.  Needs causal.
    int global_tokens;  // the first global_tokens keys stay visible to every later query
    int deterministic;  // backward: dQ summed in 64-bit fixed point, so the result does not depend on the order of arrival
};

// The window part of the reference's CausalSelfAttention::allowsKey (CausalSelfAttention.cpp:95-100); the causal part
// (key <= query) is the caller's.
__host__ __device__ __forceinline__ bool window_allows(const AttnShape& s, int query, int key)
{
    return s.window <= 0 || key < s.global_tokens || key >= query - s.window + 1;
}

// Opt-in to more than 48 KB of dynamic shared memory for `kernel`, once per device: cudaFuncSetAttribute applies to the
// current device only, so a process that drives several GPUs needs it on each.  `done_mask` is the caller's static
// bookkeeping word (one bit per device ordinal below 64; higher ordinals simply set the attribute on every call).
// The first call on a device has to come before any stream capture, like the reference's own lazy configuration
// (CudaFlashAttention.cu:49-66).
template <typename Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, size_t bytes, std::atomic<unsigned long long>& done_mask)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && ((done_mask.load(std::memory_order_acquire) >> dev) & 1ull)) return cudaSuccess;
    if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes)) != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) done_mask.fetch_or(1ull << dev, std::memory_order_release);
    return cudaSuccess;
}

// Exact-fp32 SIMT kernels (attn_simt.cu).  T = float or __nv_bfloat16 element type.
struct SimtArgs {
    AttnShape s;
    int is_bf16;
    const void *q, *k, *v, *o, *dout;
    void *o_out, *dq, *dk, *dv;
    float *lse_out, *delta;
    const float* lse;
    View4 vq, vkv;     // q-like tensors (Q, O, dO, dQ) and kv-like tensors (K, V, dK, dV)
    View3 vlse, vdelta;
};
cudaError_t simt_forward(const SimtArgs& a, cudaStream_t st);
cudaError_t simt_backward(const SimtArgs& a, cudaStream_t st);  // delta pass + dQ kernel + dK/dV kernel

// Tensor-core kernels (attn_fwd_sm100.cu / attn_bwd_sm100.cu): bf16, BHSD contiguous, D in {64,128}.
struct TcArgs {
    AttnShape s;
    const __nv_bfloat16 *q, *k, *v, *o, *dout;
    __nv_bfloat16 *o_out, *dq, *dk, *dv;
    float* lse_out;
    const float* lse;
    float* delta;      // start of the backward workspace: the per-row records (kBwdRowAuxBytes per padded query row)
    float* dq_accum;   // [B][Hq][Sq_pad][D] fp32
    // Backward in pieces (the ring schedule: one query block meets several key blocks).  phases selects which of the
    // three launches run: kBwdPre (per-row records, dQ accumulator zeroed), kBwdMain (the tensor-core kernel, which
    // ADDS this key block's dQ into the accumulator), kBwdPost (accumulator -> bf16 dQ).  0 = all three.
    // dk_acc / dv_acc non-null: the main kernel adds its dK (times scale) / dV into these fp32 [B][Hkv][Skv][D]
    // tensors instead of writing bf16 dk / dv (each element has one owning CTA per launch, so the read-modify-write
    // needs no atomics and stays deterministic).
    int phases = 0;
    float* dk_acc = nullptr;
    float* dv_acc = nullptr;
};
enum : int { kBwdPre = 1, kBwdMain = 2, kBwdPost = 4 };
bool tc_fwd_supported(const AttnShape& s);
bool tc_bwd_supported(const AttnShape& s);
cudaError_t tc_forward(const TcArgs& a, cudaStream_t st);
// New tokens against a KV cache (forward only): s.Sq new tokens per head at positions Skv-Sq .. Skv-1, K/V slabs
// `capacity` rows apart.  The keys are dealt to n_splits CTAs per (KV head, 128-row query block), each running two key
// streams; the 2 * n_splits partial results go through `workspace` (tc_cache_workspace_bytes) and a merge kernel.
struct CachePlan { int n_splits, tiles_per_split; };
CachePlan tc_cache_plan(const AttnShape& s);
size_t tc_cache_workspace_bytes(const AttnShape& s);
bool tc_cache_supported(const AttnShape& s);
cudaError_t tc_cache_forward(const TcArgs& a, int capacity, void* workspace, cudaStream_t st);
cudaError_t tc_backward(const TcArgs& a, cudaStream_t st);
size_t tc_backward_workspace_bytes(const AttnShape& s);
// Bytes per padded query row at the head of the tensor-core backward workspace: two 16-byte records (the extra
// contraction-step operands that carry -delta and -LSE/scale into the dP^T and S^T products)
constexpr size_t kBwdRowAuxBytes = 2 * 16;

// Layout / dtype staging (layout_convert.cu): SENTINEL fp32 feature-major <-> bf16 BHSD.
// The same relayouts with the rotary embedding applied on the way (cos_t == nullptr: plain relayout).
cudaError_t rope_pack_bf16(const float* src, __nv_bfloat16* dst, int B, int H, int S, int D, int stride_columns,
                           int column_start, const float* cos_t, const float* sin_t, int position_offset, cudaStream_t st);
cudaError_t rope_unpack_f32(const __nv_bfloat16* src, float* dst, int B, int H, int S, int D, int stride_columns,
                            int column_start, const float* cos_t, const float* sin_t, int position_offset, bool inverse,
                            cudaStream_t st);
cudaError_t sentinel_to_bhsd_bf16(const float* src, __nv_bfloat16* dst, int B, int H, int S, int D, int stride_columns,
                                  int column_start, cudaStream_t st);
cudaError_t bhsd_bf16_to_sentinel(const __nv_bfloat16* src, float* dst, int B, int H, int S, int D, int stride_columns,
                                  int column_start, cudaStream_t st);
cudaError_t f32_to_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t st);
cudaError_t bf16_to_f32(const __nv_bfloat16* src, float* dst, size_t n, cudaStream_t st);
cudaError_t lse_bhs_to_sentinel(const float* src, float* dst, int B, int H, int S, int stride_columns, int column_start,
                                cudaStream_t st);
cudaError_t lse_sentinel_to_bhs(const float* src, float* dst, int B, int H, int S, int stride_columns, int column_start,
                                cudaStream_t st);
cudaError_t accumulate_f32(int part_dtype, float* acc, const void* part, size_t n, cudaStream_t st);
cudaError_t merge_partials(int acc_dtype, int part_dtype, long long rows, int D, void* o_acc, float* lse_acc,
                           const void* o_part, const float* lse_part, cudaStream_t st);

// Launch accounting (attn_api.cu).
void count_launch(int n = 1);

// A one-warp kernel whose only wait can never complete, limited to limit_ns (attn_fwd_sm100.cu): exercises the
// give-up path of the bounded waits without hanging or faulting anything.  *gave_up (device memory, optional) <- 1.
cudaError_t launch_wait_selftest(unsigned long long limit_ns, unsigned int* gave_up, cudaStream_t st);

// Device status words written by bounded waits (one per tensor-core translation unit).
cudaError_t read_and_clear_fwd_status(cudaStream_t st, uint32_t* word);
cudaError_t read_and_clear_bwd_status(cudaStream_t st, uint32_t* word);

}  // namespace sntl

// Exact-fp32 attention kernels (no tensor cores): forward, delta, dQ, dK/dV.
//
// They cover what the tensor-core kernels do not: fp32 tensors that must match the reference CPU path to
// 1e-4 (the toy fp32 workload, D=16), odd head dimensions, and the reference's feature-major layout
// without a staging copy (all addressing goes through element strides).  They are also the on-device
// cross-check for the tensor-core kernels at full size.
//
// Algorithm (same math as sentinel/NeuralNet/Layers/CausalSelfAttention.cpp:232-254 / :333-352, tiled with
// an online softmax like sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:337-438): one warp owns one query
// row (forward, dQ) or one key row (dK/dV).  Keys (or queries) are visited in tiles of 32 staged in shared
// memory; lane j scores row-vs-tile-row j with a D-long dot product, the warp reduces max/sum, then the
// lanes switch to owning output dimensions d = lane + 32c and accumulate sum_j w_j * tile[j][d] with w_j
// broadcast by shuffle.  dK/dV are owned by exactly one warp each, so the backward is deterministic and
// needs no atomics and no pre-zeroed buffers.
#include "common.cuh"

#include <math.h>

namespace sntl {
namespace {

constexpr int kWarps = 8;          // rows per block
constexpr int kTile = 32;          // tile rows = lanes
constexpr int kMaxC = 8;           // output dims per lane: D <= 256

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float x);
template <> __device__ __forceinline__ void stf<float>(float* p, float x) { *p = x; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_max(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Stage rows [row0, row0+32) of a [S][D] slab (strides ss, sd) into smem[32][ld]; rows >= S become zero.
template <typename T>
__device__ __forceinline__ void stage_tile(float* smem, int ld, const T* base, long long ss, long long sd, int row0, int S,
                                           int D)
{
    const int n = kTile * D;
    if (sd == 1) {
        for (int e = threadIdx.x; e < n; e += blockDim.x) {
            const int r = e / D, d = e - r * D;
            const int row = row0 + r;
            smem[r * ld + d] = row < S ? ldf(base + row * ss + d) : 0.0f;
        }
    } else {  // token-contiguous (feature-major) source: make the row index the fast one
        for (int e = threadIdx.x; e < n; e += blockDim.x) {
            const int d = e / kTile, r = e - d * kTile;
            const int row = row0 + r;
            smem[r * ld + d] = row < S ? ldf(base + row * ss + d * sd) : 0.0f;
        }
    }
}

__device__ __forceinline__ int visible_keys(const AttnShape& s, int query)
{
    if (!s.causal) return s.Skv;
    int n = query + (s.Skv - s.Sq) + 1;
    return n < 0 ? 0 : (n > s.Skv ? s.Skv : n);
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_fwd_kernel(SimtArgs a)
{
    extern __shared__ float smem[];
    const AttnShape& s = a.s;
    const int D = s.D, ld = D + 1;
    float* sq = smem;                       // [kWarps][D]
    float* sk = sq + kWarps * D;            // [32][D+1]
    float* sv = sk + kTile * ld;            // [32][D+1]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, hk = h / (s.Hq / s.Hkv);
    const int row0 = blockIdx.x * kWarps, row = row0 + warp;
    const bool live = row < s.Sq;
    const T* qb = (const T*)a.q + b * a.vq.sb + h * a.vq.sh;
    const T* kb = (const T*)a.k + b * a.vkv.sb + hk * a.vkv.sh;
    const T* vb = (const T*)a.v + b * a.vkv.sb + hk * a.vkv.sh;

    for (int e = threadIdx.x; e < kWarps * D; e += blockDim.x) {
        const int r = e / D, d = e - r * D;
        sq[e] = (row0 + r) < s.Sq ? ldf(qb + (long long)(row0 + r) * a.vq.ss + d * a.vq.sd) : 0.0f;
    }
    const int last_row = min(row0 + kWarps, s.Sq) - 1;
    const int shift = s.causal ? s.Skv - s.Sq : 0;      // query row r sits at position r + shift (new tokens after a KV cache)
    const int n_block = visible_keys(s, last_row);      // keys any row of the block can see
    const int n_mine = live ? visible_keys(s, row) : 0;

    float m = -INFINITY, l = 0.0f, acc[kMaxC];
#pragma unroll
    for (int c = 0; c < kMaxC; ++c) acc[c] = 0.0f;

    for (int k0 = 0; k0 < n_block; k0 += kTile) {
        // tiles between the global tokens and the window of the block's first row are visible to no row of the block
        if (s.window > 0 && k0 >= s.global_tokens && k0 + kTile - 1 < row0 + shift - s.window + 1) continue;
        __syncthreads();
        stage_tile(sk, ld, kb, a.vkv.ss, a.vkv.sd, k0, s.Skv, D);
        stage_tile(sv, ld, vb, a.vkv.ss, a.vkv.sd, k0, s.Skv, D);
        __syncthreads();
        if (k0 >= n_mine) continue;
        float sc = 0.0f;
        const float* qr = sq + warp * D;
        const float* kr = sk + lane * ld;
        for (int d = 0; d < D; ++d) sc = fmaf(qr[d], kr[d], sc);
        sc = (k0 + lane < n_mine && window_allows(s, row + shift, k0 + lane)) ? sc * s.scale : -INFINITY;
        const float m_new = fmaxf(m, warp_max(sc));
        if (m_new == -INFINITY) continue;                 // nothing visible yet (tile below this row's window)
        const float p = expf(sc - m_new);
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < kMaxC; ++c) acc[c] *= corr;
        for (int j = 0; j < kTile; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
            for (int c = 0; c < kMaxC; ++c) {
                const int d = lane + 32 * c;
                if (d < D) acc[c] = fmaf(pj, sv[j * ld + d], acc[c]);
            }
        }
    }
    if (!live) return;
    T* ob = (T*)a.o_out + b * a.vq.sb + h * a.vq.sh + (long long)row * a.vq.ss;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int c = 0; c < kMaxC; ++c) {
        const int d = lane + 32 * c;
        if (d < D) stf(ob + d * a.vq.sd, acc[c] * inv);
    }
    if (lane == 0)
        a.lse_out[b * a.vlse.sb + h * a.vlse.sh + (long long)row * a.vlse.ss] = l > 0.0f ? m + logf(l) : -INFINITY;
}

// delta[b][h][s] = sum_d O * dO   (sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:576-596)
template <typename T>
__global__ void simt_delta_kernel(SimtArgs a)
{
    const AttnShape& s = a.s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= s.Sq) return;
    const long long off = b * a.vq.sb + h * a.vq.sh + (long long)row * a.vq.ss;
    const T* o = (const T*)a.o + off;
    const T* g = (const T*)a.dout + off;
    float x = 0.0f;
    for (int d = lane; d < s.D; d += 32) x = fmaf(ldf(o + d * a.vq.sd), ldf(g + d * a.vq.sd), x);
    x = warp_sum(x);
    if (lane == 0) a.delta[b * a.vdelta.sb + h * a.vdelta.sh + (long long)row * a.vdelta.ss] = x;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_dq_kernel(SimtArgs a)
{
    extern __shared__ float smem[];
    const AttnShape& s = a.s;
    const int D = s.D, ld = D + 1;
    float* sq = smem;                       // [kWarps][D]
    float* sg = sq + kWarps * D;            // [kWarps][D]  dO rows
    float* sk = sg + kWarps * D;            // [32][D+1]
    float* sv = sk + kTile * ld;            // [32][D+1]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, hk = h / (s.Hq / s.Hkv);
    const int row0 = blockIdx.x * kWarps, row = row0 + warp;
    const bool live = row < s.Sq;
    const long long qoff = b * a.vq.sb + h * a.vq.sh;
    const T* kb = (const T*)a.k + b * a.vkv.sb + hk * a.vkv.sh;
    const T* vb = (const T*)a.v + b * a.vkv.sb + hk * a.vkv.sh;
    for (int e = threadIdx.x; e < kWarps * D; e += blockDim.x) {
        const int r = e / D, d = e - r * D;
        const bool ok = (row0 + r) < s.Sq;
        const long long off = qoff + (long long)(row0 + r) * a.vq.ss + d * a.vq.sd;
        sq[e] = ok ? ldf((const T*)a.q + off) : 0.0f;
        sg[e] = ok ? ldf((const T*)a.dout + off) : 0.0f;
    }
    const int last_row = min(row0 + kWarps, s.Sq) - 1;
    const int shift = s.causal ? s.Skv - s.Sq : 0;
    const int n_block = visible_keys(s, last_row);
    const int n_mine = live ? visible_keys(s, row) : 0;
    float lse = 0.0f, delta = 0.0f;
    if (live) {
        lse = a.lse[b * a.vlse.sb + h * a.vlse.sh + (long long)row * a.vlse.ss];
        delta = a.delta[b * a.vdelta.sb + h * a.vdelta.sh + (long long)row * a.vdelta.ss];
    }
    float acc[kMaxC];
#pragma unroll
    for (int c = 0; c < kMaxC; ++c) acc[c] = 0.0f;

    for (int k0 = 0; k0 < n_block; k0 += kTile) {
        // tiles between the global tokens and the window of the block's first row are visible to no row of the block
        if (s.window > 0 && k0 >= s.global_tokens && k0 + kTile - 1 < row0 + shift - s.window + 1) continue;
        __syncthreads();
        stage_tile(sk, ld, kb, a.vkv.ss, a.vkv.sd, k0, s.Skv, D);
        stage_tile(sv, ld, vb, a.vkv.ss, a.vkv.sd, k0, s.Skv, D);
        __syncthreads();
        if (k0 >= n_mine) continue;
        float sc = 0.0f, dp = 0.0f;
        const float* qr = sq + warp * D;
        const float* gr = sg + warp * D;
        const float* kr = sk + lane * ld;
        const float* vr = sv + lane * ld;
        for (int d = 0; d < D; ++d) {
            sc = fmaf(qr[d], kr[d], sc);
            dp = fmaf(gr[d], vr[d], dp);
        }
        const bool vis = (k0 + lane < n_mine) && window_allows(s, row + shift, k0 + lane) && lse > -INFINITY;
        const float p = vis ? expf(sc * s.scale - lse) : 0.0f;
        const float ds = p * (dp - delta) * s.scale;
        for (int j = 0; j < kTile; ++j) {
            const float dsj = __shfl_sync(0xffffffffu, ds, j);
#pragma unroll
            for (int c = 0; c < kMaxC; ++c) {
                const int d = lane + 32 * c;
                if (d < D) acc[c] = fmaf(dsj, sk[j * ld + d], acc[c]);
            }
        }
    }
    if (!live) return;
    T* ob = (T*)a.dq + qoff + (long long)row * a.vq.ss;
#pragma unroll
    for (int c = 0; c < kMaxC; ++c) {
        const int d = lane + 32 * c;
        if (d < D) stf(ob + d * a.vq.sd, acc[c]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_dkv_kernel(SimtArgs a)
{
    extern __shared__ float smem[];
    const AttnShape& s = a.s;
    const int D = s.D, ld = D + 1;
    float* skr = smem;                      // [kWarps][D]  key rows
    float* svr = skr + kWarps * D;          // [kWarps][D]  value rows
    float* sq = svr + kWarps * D;           // [32][D+1]  query tile
    float* sg = sq + kTile * ld;            // [32][D+1]  dO tile
    float* sl = sg + kTile * ld;            // [32] lse
    float* sd = sl + kTile;                 // [32] delta
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, hk = blockIdx.y, group = s.Hq / s.Hkv;
    const int key0 = blockIdx.x * kWarps, key = key0 + warp;
    const bool live = key < s.Skv;
    const long long kvoff = b * a.vkv.sb + hk * a.vkv.sh;
    for (int e = threadIdx.x; e < kWarps * D; e += blockDim.x) {
        const int r = e / D, d = e - r * D;
        const bool ok = (key0 + r) < s.Skv;
        const long long off = kvoff + (long long)(key0 + r) * a.vkv.ss + d * a.vkv.sd;
        skr[e] = ok ? ldf((const T*)a.k + off) : 0.0f;
        svr[e] = ok ? ldf((const T*)a.v + off) : 0.0f;
    }
    // first query that can see key j: i >= j - (Skv - Sq)
    const int shift = s.Skv - s.Sq;
    const int q_first_block = s.causal ? max(0, key0 - shift) : 0;
    const int q_first_mine = s.causal ? max(0, key - shift) : 0;
    float dk[kMaxC], dv[kMaxC];
#pragma unroll
    for (int c = 0; c < kMaxC; ++c) dk[c] = dv[c] = 0.0f;

    for (int g = 0; g < group; ++g) {
        const int h = hk * group + g;
        const long long qoff = b * a.vq.sb + h * a.vq.sh;
        for (int q0 = (q_first_block / kTile) * kTile; q0 < s.Sq; q0 += kTile) {
            // past the window of the block's last key (and no key of the block is global): no later query sees the block
            if (s.window > 0 && key0 >= s.global_tokens && q0 + shift > key0 + kWarps - 1 + s.window - 1) break;
            __syncthreads();
            stage_tile(sq, ld, (const T*)a.q + qoff, a.vq.ss, a.vq.sd, q0, s.Sq, D);
            stage_tile(sg, ld, (const T*)a.dout + qoff, a.vq.ss, a.vq.sd, q0, s.Sq, D);
            if (threadIdx.x < kTile) {
                const int r = q0 + threadIdx.x;
                sl[threadIdx.x] = r < s.Sq ? a.lse[b * a.vlse.sb + h * a.vlse.sh + (long long)r * a.vlse.ss] : -INFINITY;
                sd[threadIdx.x] = r < s.Sq ? a.delta[b * a.vdelta.sb + h * a.vdelta.sh + (long long)r * a.vdelta.ss] : 0.0f;
            }
            __syncthreads();
            if (!live || q0 + kTile <= q_first_mine) continue;
            float sc = 0.0f, dp = 0.0f;
            const float* kr = skr + warp * D;
            const float* vr = svr + warp * D;
            const float* qr = sq + lane * ld;
            const float* gr = sg + lane * ld;
            for (int d = 0; d < D; ++d) {
                sc = fmaf(qr[d], kr[d], sc);
                dp = fmaf(gr[d], vr[d], dp);
            }
            const int qi = q0 + lane;
            const float lse = sl[lane];
            const bool vis = qi < s.Sq && qi >= q_first_mine && window_allows(s, qi + shift, key) && lse > -INFINITY;
            const float p = vis ? expf(sc * s.scale - lse) : 0.0f;
            const float ds = p * (dp - sd[lane]) * s.scale;
            for (int i = 0; i < kTile; ++i) {
                const float pi = __shfl_sync(0xffffffffu, p, i);
                const float dsi = __shfl_sync(0xffffffffu, ds, i);
#pragma unroll
                for (int c = 0; c < kMaxC; ++c) {
                    const int d = lane + 32 * c;
                    if (d < D) {
                        dv[c] = fmaf(pi, sg[i * ld + d], dv[c]);
                        dk[c] = fmaf(dsi, sq[i * ld + d], dk[c]);
                    }
                }
            }
        }
    }
    if (!live) return;
    T* dkb = (T*)a.dk + kvoff + (long long)key * a.vkv.ss;
    T* dvb = (T*)a.dv + kvoff + (long long)key * a.vkv.ss;
#pragma unroll
    for (int c = 0; c < kMaxC; ++c) {
        const int d = lane + 32 * c;
        if (d < D) {
            stf(dkb + d * a.vkv.sd, dk[c]);
            stf(dvb + d * a.vkv.sd, dv[c]);
        }
    }
}

template <typename K>
cudaError_t allow_smem(K kernel, size_t bytes)
{
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <typename T>
cudaError_t fwd_t(const SimtArgs& a, cudaStream_t st)
{
    const int D = a.s.D;
    const size_t smem = sizeof(float) * (kWarps * D + 2 * kTile * (D + 1));
    cudaError_t e = allow_smem(simt_fwd_kernel<T>, smem);
    if (e != cudaSuccess) return e;
    dim3 grid((a.s.Sq + kWarps - 1) / kWarps, a.s.Hq, a.s.B);
    simt_fwd_kernel<T><<<grid, kWarps * 32, smem, st>>>(a);
    count_launch();
    return cudaGetLastError();
}

template <typename T>
cudaError_t bwd_t(const SimtArgs& a, cudaStream_t st)
{
    const int D = a.s.D;
    cudaError_t e;
    {
        dim3 grid((a.s.Sq + 7) / 8, a.s.Hq, a.s.B);
        simt_delta_kernel<T><<<grid, 256, 0, st>>>(a);
        count_launch();
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    {
        const size_t smem = sizeof(float) * (2 * kWarps * D + 2 * kTile * (D + 1));
        if ((e = allow_smem(simt_dq_kernel<T>, smem)) != cudaSuccess) return e;
        dim3 grid((a.s.Sq + kWarps - 1) / kWarps, a.s.Hq, a.s.B);
        simt_dq_kernel<T><<<grid, kWarps * 32, smem, st>>>(a);
        count_launch();
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    {
        const size_t smem = sizeof(float) * (2 * kWarps * D + 2 * kTile * (D + 1) + 2 * kTile);
        if ((e = allow_smem(simt_dkv_kernel<T>, smem)) != cudaSuccess) return e;
        dim3 grid((a.s.Skv + kWarps - 1) / kWarps, a.s.Hkv, a.s.B);
        simt_dkv_kernel<T><<<grid, kWarps * 32, smem, st>>>(a);
        count_launch();
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace

cudaError_t simt_forward(const SimtArgs& a, cudaStream_t st)
{
    return a.is_bf16 ? fwd_t<__nv_bfloat16>(a, st) : fwd_t<float>(a, st);
}

cudaError_t simt_backward(const SimtArgs& a, cudaStream_t st)
{
    return a.is_bf16 ? bwd_t<__nv_bfloat16>(a, st) : bwd_t<float>(a, st);
}

}  // namespace sntl

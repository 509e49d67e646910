// HBM-bound staging kernels: the reference's fp32 feature-major matrices <-> bf16 token-major tensors,
// plain dtype casts, LSE re-indexing, and the log-sum-exp merge of two partial attention results.
//
// Feature-major ("SENTINEL") addressing follows sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:129-131:
// element (b,h,s,d) lives at (h*D + d)*stride_columns + column_start + b*S + s.
#include "common.cuh"

namespace sntl {
namespace {

// 32x32 transposing tile: reads are contiguous along tokens (source rows), writes along d (destination rows).
__global__ void sentinel_to_bhsd_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int H, int S, int D,
                                        int stride_columns, int column_start)
{
    __shared__ float tile[32][33];
    const int bh = blockIdx.z, b = bh / H, h = bh % H;
    const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
    for (int r = ty; r < 32; r += 8) {
        const int d = d0 + r, s = s0 + tx;
        tile[r][tx] = (d < D && s < S) ? src[(long long)(h * D + d) * stride_columns + column_start + (long long)b * S + s] : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int s = s0 + r, d = d0 + tx;
        if (s < S && d < D) dst[((long long)bh * S + s) * D + d] = __float2bfloat16_rn(tile[tx][r]);
    }
}

__global__ void bhsd_to_sentinel_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int H, int S, int D,
                                        int stride_columns, int column_start)
{
    __shared__ float tile[32][33];
    const int bh = blockIdx.z, b = bh / H, h = bh % H;
    const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;
    for (int r = ty; r < 32; r += 8) {
        const int s = s0 + r, d = d0 + tx;
        tile[r][tx] = (s < S && d < D) ? __bfloat162float(src[((long long)bh * S + s) * D + d]) : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int d = d0 + r, s = s0 + tx;
        if (d < D && s < S) dst[(long long)(h * D + d) * stride_columns + column_start + (long long)b * S + s] = tile[tx][r];
    }
}

// Rotary position embedding fused into the two transposes above: what the reference does as separate passes
// (rotaryRotateInPlace / rotaryRotateInverseInPlace over the fp32 matrices, sentinel/NeuralNet/Cuda/CudaOps.cu:362-399,
// then the flash kernel's per-load conversion) becomes part of the one read + one write of the relayout.
// Pairs are interleaved, (2i, 2i+1), angle table entry [position][i] (RotaryEmbedding.cpp:19-27, :38-59); the two members
// of a pair are neighbouring d, i.e. neighbouring lanes of the token-major side, so the partner comes from a shuffle.
// Products and sums are rounded separately (no FMA contraction), which is what the reference's host code computes.
template <bool kInverse>
__device__ __forceinline__ float rotate_lane(float mine, int d, float c, float sn)
{
    const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
    const float even = (d & 1) ? other : mine, odd = (d & 1) ? mine : other;
    if (!kInverse)   // even' = e*cos - o*sin ; odd' = e*sin + o*cos
        return (d & 1) ? __fadd_rn(__fmul_rn(even, sn), __fmul_rn(odd, c)) : __fsub_rn(__fmul_rn(even, c), __fmul_rn(odd, sn));
    // inverse (transpose of the rotation): even' = e*cos + o*sin ; odd' = -e*sin + o*cos
    return (d & 1) ? __fadd_rn(__fmul_rn(-even, sn), __fmul_rn(odd, c)) : __fadd_rn(__fmul_rn(even, c), __fmul_rn(odd, sn));
}

__global__ void rope_pack_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int H, int S, int D,
                                 int stride_columns, int column_start, const float* __restrict__ cos_t,
                                 const float* __restrict__ sin_t, int position_offset)
{
    __shared__ float tile[32][33];
    const int bh = blockIdx.z, b = bh / H, h = bh % H;
    const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
    for (int r = ty; r < 32; r += 8) {
        const int d = d0 + r, s = s0 + tx;
        tile[r][tx] = (d < D && s < S) ? src[(long long)(h * D + d) * stride_columns + column_start + (long long)b * S + s] : 0.0f;
    }
    __syncthreads();
    const int pairs = D >> 1;
    for (int r = ty; r < 32; r += 8) {
        const int s = s0 + r, d = d0 + tx;       // D is even and d0 a multiple of 32: a pair never straddles tiles
        const bool live = s < S && d < D;
        const long long ti = (long long)(position_offset + s) * pairs + (d >> 1);
        const float c = live ? cos_t[ti] : 1.0f, sn = live ? sin_t[ti] : 0.0f;
        const float v = rotate_lane<false>(tile[tx][r], d, c, sn);
        if (live) dst[((long long)bh * S + s) * D + d] = __float2bfloat16_rn(v);
    }
}

template <bool kInverse>
__global__ void rope_unpack_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int H, int S, int D,
                                   int stride_columns, int column_start, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, int position_offset)
{
    __shared__ float tile[32][33];
    const int bh = blockIdx.z, b = bh / H, h = bh % H;
    const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int pairs = D >> 1;
    for (int r = ty; r < 32; r += 8) {
        const int s = s0 + r, d = d0 + tx;
        const bool live = s < S && d < D;
        const float x = live ? __bfloat162float(src[((long long)bh * S + s) * D + d]) : 0.0f;
        const long long ti = (long long)(position_offset + s) * pairs + (d >> 1);
        const float c = live ? cos_t[ti] : 1.0f, sn = live ? sin_t[ti] : 0.0f;
        tile[r][tx] = rotate_lane<kInverse>(x, d, c, sn);
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int d = d0 + r, s = s0 + tx;
        if (d < D && s < S) dst[(long long)(h * D + d) * stride_columns + column_start + (long long)b * S + s] = tile[tx][r];
    }
}

// Head sizes that are multiples of 64 (the tensor-core kernels' sizes) take 64-token x 64-feature tiles: every global
// access is a full 128-byte line per warp (32 tokens of one feature on the fp32 side, the 64 features of one token as
// bf16 pairs on the other), each thread keeps 16 loads in flight, and a rotation pair lives in one thread.
// kRot: 0 no rotation, 1 forward, 2 inverse.
template <int kRot>
__device__ __forceinline__ void rotate_pair(float& even, float& odd, float c, float sn)
{
    if (kRot == 0) return;
    const float e = even, o = odd;
    if (kRot == 1) {
        even = __fsub_rn(__fmul_rn(e, c), __fmul_rn(o, sn));
        odd = __fadd_rn(__fmul_rn(e, sn), __fmul_rn(o, c));
    } else {
        even = __fadd_rn(__fmul_rn(e, c), __fmul_rn(o, sn));
        odd = __fadd_rn(__fmul_rn(-e, sn), __fmul_rn(o, c));
    }
}

// Tiles of kTok tokens x DT = 64 features, every global access 16 bytes wide: on the bf16 side a thread moves eight
// consecutive features of one token, on the fp32 side four consecutive tokens of one feature (runs of kTok * 4 = 512
// contiguous bytes per feature).  (A tile covering a whole 128-feature head makes the bf16 side one contiguous block,
// but its 66 KB of shared memory leave three CTAs per SM and it measured 35 % slower.)  The angle tables come as float4 (four
// pairs).  Lane maps are chosen so that, with the tile's odd row pitch, the 32 lanes of a warp hit 32 different banks in
// both transposing directions: 8 token quads x 4 features on the fp32 side, 8 tokens x 4 eight-feature units on the
// bf16 side.  kVec = false is the same kernel with 4-byte accesses on the fp32 side, for windows whose first column,
// length or row pitch is not a multiple of four elements.
constexpr int kTok = 128;
constexpr int kHeadsPerCta = 4;   // heads one CTA converts in turn: the angle tables then cost a quarter of the L2 traffic

// lane maps (see above): fp32 side -> (first of four tokens, feature); bf16 side -> (token, 8-feature unit)
template <int DT> struct PackMap {
    static constexpr int kQuads = kTok * DT / 4 / 256;        // float4 accesses per thread on the fp32 side
    static constexpr int kUnits = kTok * (DT / 8) / 256;      // 16-byte units per thread on the bf16 side
    static constexpr int kUnitGroups = DT / 32;
    __device__ static void quad(int r, int& s4, int& d)
    {
        const int idx = r * 256 + threadIdx.x, rest = idx >> 5;
        s4 = (rest & 3) * 32 + (idx & 7) * 4;
        d = (rest >> 2) * 4 + ((idx >> 3) & 3);
    }
    __device__ static void unit(int r, int& sl, int& u)
    {
        const int idx = r * 256 + threadIdx.x, rest = idx >> 5;
        sl = (rest / kUnitGroups) * 8 + ((idx >> 2) & 7);
        u = (rest % kUnitGroups) * 4 + (idx & 3);
    }
};

// The angles depend on the token and the feature pair only: a thread fetches those of its (token, unit) slots once
// and keeps them in registers for all the heads its CTA converts.
template <int kRot, int DT>
__device__ __forceinline__ void load_angles(float4* cs, float4* sn, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                            int s0, int d0, int S, int pairs, int position_offset)
{
    if (kRot == 0) return;
#pragma unroll
    for (int r = 0; r < PackMap<DT>::kUnits; ++r) {
        int sl, u;
        PackMap<DT>::unit(r, sl, u);
        const int s = min(s0 + sl, S - 1);
        const long long ti = (long long)(position_offset + s) * pairs + (d0 >> 1) + 4 * u;   // a multiple of 4: 16-byte aligned
        cs[r] = __ldg(reinterpret_cast<const float4*>(cos_t + ti));
        sn[r] = __ldg(reinterpret_cast<const float4*>(sin_t + ti));
    }
}

template <int kRot, bool kVec, int DT>
__global__ void __launch_bounds__(256, 4) pack64_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int H, int S, int D,
                                                     int stride_columns, int column_start, const float* __restrict__ cos_t,
                                                     const float* __restrict__ sin_t, int position_offset)
{
    using M = PackMap<DT>;
    extern __shared__ float tile_raw[];
    float (*tile)[DT + 1] = reinterpret_cast<float (*)[DT + 1]>(tile_raw);   // [token][feature]
    const int groups = (H + kHeadsPerCta - 1) / kHeadsPerCta;
    const int b = blockIdx.z / groups, h_first = (blockIdx.z % groups) * kHeadsPerCta;
    const int s0 = blockIdx.x * kTok, d0 = blockIdx.y * DT;
    float4 cs[M::kUnits], sn[M::kUnits];
    load_angles<kRot, DT>(cs, sn, cos_t, sin_t, s0, d0, S, D >> 1, position_offset);
    for (int h = h_first; h < min(H, h_first + kHeadsPerCta); ++h) {
        const float* base = src + (long long)(h * D + d0) * stride_columns + column_start + (long long)b * S + s0;
        if (kVec) {
            // all of a thread's loads are issued before the first one is used (S is a multiple of four here, so a quad
            // of tokens is inside the sequence or outside it as a whole)
            float4 x[M::kQuads];
#pragma unroll
            for (int r = 0; r < M::kQuads; ++r) {
                int s4, d;
                M::quad(r, s4, d);
                x[r] = (s0 + s4 < S) ? __ldg(reinterpret_cast<const float4*>(base + (long long)d * stride_columns + s4))
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int r = 0; r < M::kQuads; ++r) {
                int s4, d;
                M::quad(r, s4, d);
                tile[s4][d] = x[r].x; tile[s4 + 1][d] = x[r].y; tile[s4 + 2][d] = x[r].z; tile[s4 + 3][d] = x[r].w;
            }
        } else {
#pragma unroll 4
            for (int r = 0; r < kTok * DT / 256; ++r) {
                const int idx = r * 256 + threadIdx.x, d = idx / kTok, sl = idx % kTok;
                tile[sl][d] = (s0 + sl < S) ? base[(long long)d * stride_columns + sl] : 0.0f;
            }
        }
        __syncthreads();
        __nv_bfloat16* out = dst + ((long long)(b * H + h) * S + s0) * D + d0;
#pragma unroll
        for (int r = 0; r < M::kUnits; ++r) {
            int sl, u;
            M::unit(r, sl, u);
            if (s0 + sl >= S) continue;
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = tile[sl][8 * u + i];
            if (kRot != 0) {
                rotate_pair<kRot>(x[0], x[1], cs[r].x, sn[r].x);
                rotate_pair<kRot>(x[2], x[3], cs[r].y, sn[r].y);
                rotate_pair<kRot>(x[4], x[5], cs[r].z, sn[r].z);
                rotate_pair<kRot>(x[6], x[7], cs[r].w, sn[r].w);
            }
            __nv_bfloat162 o0 = __floats2bfloat162_rn(x[0], x[1]), o1 = __floats2bfloat162_rn(x[2], x[3]);
            __nv_bfloat162 o2 = __floats2bfloat162_rn(x[4], x[5]), o3 = __floats2bfloat162_rn(x[6], x[7]);
            uint4 w;
            w.x = *reinterpret_cast<uint32_t*>(&o0); w.y = *reinterpret_cast<uint32_t*>(&o1);
            w.z = *reinterpret_cast<uint32_t*>(&o2); w.w = *reinterpret_cast<uint32_t*>(&o3);
            *reinterpret_cast<uint4*>(out + (long long)sl * D + 8 * u) = w;
        }
        __syncthreads();      // the tile is refilled for the next head
    }
}

template <int kRot, bool kVec, int DT>
__global__ void __launch_bounds__(256, 4) unpack64_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int H, int S, int D,
                                                       int stride_columns, int column_start, const float* __restrict__ cos_t,
                                                       const float* __restrict__ sin_t, int position_offset)
{
    using M = PackMap<DT>;
    extern __shared__ float tile_raw[];
    float (*tile)[DT + 1] = reinterpret_cast<float (*)[DT + 1]>(tile_raw);
    const int groups = (H + kHeadsPerCta - 1) / kHeadsPerCta;
    const int b = blockIdx.z / groups, h_first = (blockIdx.z % groups) * kHeadsPerCta;
    const int s0 = blockIdx.x * kTok, d0 = blockIdx.y * DT;
    float4 cs[M::kUnits], sn[M::kUnits];
    load_angles<kRot, DT>(cs, sn, cos_t, sin_t, s0, d0, S, D >> 1, position_offset);
    for (int h = h_first; h < min(H, h_first + kHeadsPerCta); ++h) {
        const __nv_bfloat16* in = src + ((long long)(b * H + h) * S + s0) * D + d0;
        uint4 win[M::kUnits];
#pragma unroll
        for (int r = 0; r < M::kUnits; ++r) {      // all loads first
            int sl, u;
            M::unit(r, sl, u);
            win[r] = (s0 + sl < S) ? __ldg(reinterpret_cast<const uint4*>(in + (long long)sl * D + 8 * u)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < M::kUnits; ++r) {
            int sl, u;
            M::unit(r, sl, u);
            const uint32_t ws[4] = {win[r].x, win[r].y, win[r].z, win[r].w};
            float x[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                x[2 * i] = __uint_as_float(ws[i] << 16);
                x[2 * i + 1] = __uint_as_float(ws[i] & 0xffff0000u);
            }
            if (kRot != 0) {      // (rows past the end are zeros and stay zeros under the rotation)
                rotate_pair<kRot>(x[0], x[1], cs[r].x, sn[r].x);
                rotate_pair<kRot>(x[2], x[3], cs[r].y, sn[r].y);
                rotate_pair<kRot>(x[4], x[5], cs[r].z, sn[r].z);
                rotate_pair<kRot>(x[6], x[7], cs[r].w, sn[r].w);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) tile[sl][8 * u + i] = x[i];
        }
        __syncthreads();
        float* base = dst + (long long)(h * D + d0) * stride_columns + column_start + (long long)b * S + s0;
        if (kVec) {
#pragma unroll
            for (int r = 0; r < M::kQuads; ++r) {
                int s4, d;
                M::quad(r, s4, d);
                if (s0 + s4 < S)
                    *reinterpret_cast<float4*>(base + (long long)d * stride_columns + s4) =
                        make_float4(tile[s4][d], tile[s4 + 1][d], tile[s4 + 2][d], tile[s4 + 3][d]);
            }
        } else {
#pragma unroll 4
            for (int r = 0; r < kTok * DT / 256; ++r) {
                const int idx = r * 256 + threadIdx.x, d = idx / kTok, sl = idx % kTok;
                if (s0 + sl < S) base[(long long)d * stride_columns + sl] = tile[sl][d];
            }
        }
        __syncthreads();      // the tile is refilled for the next head
    }
}

// launches pack64_kernel / unpack64_kernel (one tile column of 64 features per blockIdx.y)
#define SNTL_PACK_CASE(KERNEL, ROT, VEC, DTV)                                                                                      \
    do {                                                                                                                           \
        constexpr size_t smem = (size_t)kTok * (DTV + 1) * sizeof(float);                                                          \
        static std::atomic<unsigned long long> configured{0};                                                                      \
        if ((e = ensure_dynamic_smem(KERNEL<ROT, VEC, DTV>, smem, configured)) != cudaSuccess) return e;                           \
        dim3 grid((S + kTok - 1) / kTok, D / DTV, B * ((H + kHeadsPerCta - 1) / kHeadsPerCta));                                    \
        KERNEL<ROT, VEC, DTV><<<grid, 256, smem, st>>>(src, dst, H, S, D, stride_columns, column_start, cos_t, sin_t, position_offset); \
    } while (0)
#define SNTL_PACK_ROT(KERNEL, VEC, DTV)                                 \
    do {                                                                \
        if (rot == 0) SNTL_PACK_CASE(KERNEL, 0, VEC, DTV);              \
        else if (rot == 1) SNTL_PACK_CASE(KERNEL, 1, VEC, DTV);         \
        else SNTL_PACK_CASE(KERNEL, 2, VEC, DTV);                       \
    } while (0)
#define SNTL_PACK_ALL(KERNEL)                                                            \
    do {                                                                                 \
        if (vec) SNTL_PACK_ROT(KERNEL, true, 64); else SNTL_PACK_ROT(KERNEL, false, 64);                         \
    } while (0)

cudaError_t launch_pack64(int rot, bool vec, const float* src, __nv_bfloat16* dst, int B, int H, int S, int D, int stride_columns,
                          int column_start, const float* cos_t, const float* sin_t, int position_offset, cudaStream_t st)
{
    cudaError_t e;
    SNTL_PACK_ALL(pack64_kernel);
    count_launch();
    return cudaGetLastError();
}
cudaError_t launch_unpack64(int rot, bool vec, const __nv_bfloat16* src, float* dst, int B, int H, int S, int D, int stride_columns,
                            int column_start, const float* cos_t, const float* sin_t, int position_offset, cudaStream_t st)
{
    cudaError_t e;
    SNTL_PACK_ALL(unpack64_kernel);
    count_launch();
    return cudaGetLastError();
}
#undef SNTL_PACK_ALL
#undef SNTL_PACK_ROT
#undef SNTL_PACK_CASE

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __float2bfloat16_rn(src[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __bfloat162float(src[i]);
}

// dir 0: [B][H][S] -> H x stride_columns ; dir 1: the reverse
__global__ void lse_reindex_kernel(const float* __restrict__ src, float* __restrict__ dst, int B, int H, int S,
                                   int stride_columns, int column_start, int dir)
{
    const long long n = (long long)B * H * S;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int s = (int)(i % S);
        const int h = (int)((i / S) % H);
        const int b = (int)(i / ((long long)S * H));
        const long long j = (long long)h * stride_columns + column_start + (long long)b * S + s;
        if (dir == 0) dst[j] = src[i];
        else dst[i] = src[j];
    }
}

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float x);
template <> __device__ __forceinline__ void stf<float>(float* p, float x) { *p = x; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

// One warp per row: (o_acc, lse_acc) <- the softmax-weighted combination with (o_part, lse_part).
template <typename T, typename P>
__global__ void merge_kernel(long long rows, int D, T* __restrict__ o_acc, float* __restrict__ lse_acc,
                             const P* __restrict__ o_part, const float* __restrict__ lse_part)
{
    const int lane = threadIdx.x & 31;
    const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float la = lse_acc[row], lb = lse_part[row];
    const float m = fmaxf(la, lb);
    if (m == -INFINITY) return;  // both empty: keep zeros / -inf
    const float wa = expf(la - m), wb = expf(lb - m);
    const float inv = 1.0f / (wa + wb);
    for (int d = lane; d < D; d += 32) {
        const float x = ldf(o_acc + row * D + d) * wa + ldf(o_part + row * D + d) * wb;
        stf(o_acc + row * D + d, x * inv);
    }
    if (lane == 0) lse_acc[row] = m + logf(wa + wb);
}

template <typename P>
__global__ void accumulate_kernel(float* __restrict__ acc, const P* __restrict__ part, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        acc[i] += ldf(part + i);
}

inline int blocks_for(size_t n, int threads)
{
    size_t b = (n + threads - 1) / threads;
    return (int)(b > 148 * 16 ? 148 * 16 : (b ? b : 1));
}

}  // namespace

cudaError_t sentinel_to_bhsd_bf16(const float* src, __nv_bfloat16* dst, int B, int H, int S, int D, int stride_columns,
                                  int column_start, cudaStream_t st)
{
    if (D % 64 == 0 && (long long)B * H <= 65535) return rope_pack_bf16(src, dst, B, H, S, D, stride_columns, column_start, nullptr, nullptr, 0, st);
    dim3 grid((S + 31) / 32, (D + 31) / 32, B * H), block(32, 8);
    sentinel_to_bhsd_kernel<<<grid, block, 0, st>>>(src, dst, H, S, D, stride_columns, column_start);
    count_launch();
    return cudaGetLastError();
}

cudaError_t bhsd_bf16_to_sentinel(const __nv_bfloat16* src, float* dst, int B, int H, int S, int D, int stride_columns,
                                  int column_start, cudaStream_t st)
{
    if (D % 64 == 0 && (long long)B * H <= 65535)
        return rope_unpack_f32(src, dst, B, H, S, D, stride_columns, column_start, nullptr, nullptr, 0, false, st);
    dim3 grid((S + 31) / 32, (D + 31) / 32, B * H), block(32, 8);
    bhsd_to_sentinel_kernel<<<grid, block, 0, st>>>(src, dst, H, S, D, stride_columns, column_start);
    count_launch();
    return cudaGetLastError();
}

// the fp32 side can be accessed 16 bytes at a time when every row of the window starts on a 16-byte boundary
static bool f32_rows_aligned(const void* p, int S, int stride_columns, int column_start)
{
    return ((uintptr_t)p & 15u) == 0 && stride_columns % 4 == 0 && column_start % 4 == 0 && S % 4 == 0;
}
static bool tables_aligned(const float* cos_t, const float* sin_t) { return (((uintptr_t)cos_t | (uintptr_t)sin_t) & 15u) == 0; }

cudaError_t rope_pack_bf16(const float* src, __nv_bfloat16* dst, int B, int H, int S, int D, int stride_columns,
                           int column_start, const float* cos_t, const float* sin_t, int position_offset, cudaStream_t st)
{
    if (D % 64 == 0) {
        // the bf16 side and the angle tables are accessed 16 bytes at a time (as are all bf16 tensors of the tensor-core kernels)
        if (((uintptr_t)dst & 15u) != 0 || (cos_t && !tables_aligned(cos_t, sin_t))) return cudaErrorMisalignedAddress;
        return launch_pack64(cos_t ? 1 : 0, f32_rows_aligned(src, S, stride_columns, column_start), src, dst, B, H, S, D, stride_columns,
                             column_start, cos_t, sin_t, position_offset, st);
    }
    if (!cos_t) return sentinel_to_bhsd_bf16(src, dst, B, H, S, D, stride_columns, column_start, st);
    dim3 grid((S + 31) / 32, (D + 31) / 32, B * H), block(32, 8);
    rope_pack_kernel<<<grid, block, 0, st>>>(src, dst, H, S, D, stride_columns, column_start, cos_t, sin_t, position_offset);
    count_launch();
    return cudaGetLastError();
}

cudaError_t rope_unpack_f32(const __nv_bfloat16* src, float* dst, int B, int H, int S, int D, int stride_columns,
                            int column_start, const float* cos_t, const float* sin_t, int position_offset, bool inverse,
                            cudaStream_t st)
{
    if (D % 64 == 0) {
        if (((uintptr_t)src & 15u) != 0 || (cos_t && !tables_aligned(cos_t, sin_t))) return cudaErrorMisalignedAddress;
        return launch_unpack64(!cos_t ? 0 : (inverse ? 2 : 1), f32_rows_aligned(dst, S, stride_columns, column_start), src, dst, B, H, S, D,
                               stride_columns, column_start, cos_t, sin_t, position_offset, st);
    }
    if (!cos_t) return bhsd_bf16_to_sentinel(src, dst, B, H, S, D, stride_columns, column_start, st);
    dim3 grid((S + 31) / 32, (D + 31) / 32, B * H), block(32, 8);
    if (inverse)
        rope_unpack_kernel<true><<<grid, block, 0, st>>>(src, dst, H, S, D, stride_columns, column_start, cos_t, sin_t, position_offset);
    else
        rope_unpack_kernel<false><<<grid, block, 0, st>>>(src, dst, H, S, D, stride_columns, column_start, cos_t, sin_t, position_offset);
    count_launch();
    return cudaGetLastError();
}

cudaError_t f32_to_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t st)
{
    f32_to_bf16_kernel<<<blocks_for(n, 256), 256, 0, st>>>(src, dst, n);
    count_launch();
    return cudaGetLastError();
}

cudaError_t bf16_to_f32(const __nv_bfloat16* src, float* dst, size_t n, cudaStream_t st)
{
    bf16_to_f32_kernel<<<blocks_for(n, 256), 256, 0, st>>>(src, dst, n);
    count_launch();
    return cudaGetLastError();
}

cudaError_t lse_bhs_to_sentinel(const float* src, float* dst, int B, int H, int S, int stride_columns, int column_start,
                                cudaStream_t st)
{
    lse_reindex_kernel<<<blocks_for((size_t)B * H * S, 256), 256, 0, st>>>(src, dst, B, H, S, stride_columns, column_start, 0);
    count_launch();
    return cudaGetLastError();
}

cudaError_t lse_sentinel_to_bhs(const float* src, float* dst, int B, int H, int S, int stride_columns, int column_start,
                                cudaStream_t st)
{
    lse_reindex_kernel<<<blocks_for((size_t)B * H * S, 256), 256, 0, st>>>(src, dst, B, H, S, stride_columns, column_start, 1);
    count_launch();
    return cudaGetLastError();
}

cudaError_t accumulate_f32(int part_dtype, float* acc, const void* part, size_t n, cudaStream_t st)
{
    if (n == 0) return cudaSuccess;
    if (part_dtype == SNTL_DTYPE_BF16)
        accumulate_kernel<<<blocks_for(n, 256), 256, 0, st>>>(acc, (const __nv_bfloat16*)part, n);
    else
        accumulate_kernel<<<blocks_for(n, 256), 256, 0, st>>>(acc, (const float*)part, n);
    count_launch();
    return cudaGetLastError();
}

cudaError_t merge_partials(int acc_dtype, int part_dtype, long long rows, int D, void* o_acc, float* lse_acc,
                           const void* o_part, const float* lse_part, cudaStream_t st)
{
    const int warps = 8;
    const long long blocks = (rows + warps - 1) / warps;
    if (blocks <= 0) return cudaSuccess;
    const unsigned g = (unsigned)blocks;
    const bool ab = acc_dtype == SNTL_DTYPE_BF16, pb = part_dtype == SNTL_DTYPE_BF16;
    if (ab && pb)
        merge_kernel<<<g, warps * 32, 0, st>>>(rows, D, (__nv_bfloat16*)o_acc, lse_acc, (const __nv_bfloat16*)o_part, lse_part);
    else if (!ab && pb)
        merge_kernel<<<g, warps * 32, 0, st>>>(rows, D, (float*)o_acc, lse_acc, (const __nv_bfloat16*)o_part, lse_part);
    else if (ab && !pb)
        merge_kernel<<<g, warps * 32, 0, st>>>(rows, D, (__nv_bfloat16*)o_acc, lse_acc, (const float*)o_part, lse_part);
    else
        merge_kernel<<<g, warps * 32, 0, st>>>(rows, D, (float*)o_acc, lse_acc, (const float*)o_part, lse_part);
    count_launch();
    return cudaGetLastError();
}

}  // namespace sntl

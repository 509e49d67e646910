// Thin inline-PTX wrappers for the Blackwell (sm_100a) primitives the attention kernels use:
// mbarrier, TMA tensor loads, tcgen05 MMA / TMEM load-store / alloc, and the UMMA descriptors.
// Every wait is bounded: it gives up after ~1 s of wall time (or at once when another wait on this GPU gave
// up less than a second ago), records where in a device status word, and returns false so the caller can unwind.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sntl {
namespace ptx {

// ---------------------------------------------------------------------------------------------------
// device status word: 0 = fine; otherwise (site << 24) | (blockIdx.x & 0xffffff) of the first wait that gave up.
// It is a sticky REPORT: only the host clears it (sntl_attn_poll_device_status).  It never makes a kernel give up.
// What lets the remaining CTAs of a stuck grid leave without each spending its own full limit is g_abort_until_ns:
// a give-up writes (now + its wait limit) there; a wait that has spun for a while and finds that time still in the
// future gives up too (and renews it, so the later waves of the same grid follow).  One limit after the last
// give-up the word is stale and launches behave normally again, whether or not the host has polled.
// ---------------------------------------------------------------------------------------------------
static __device__ unsigned int g_device_status;          // one copy per translation unit; each exposes its own reader
static __device__ unsigned long long g_abort_until_ns;   // 0 = no wait has ever given up

// Optional phase tracing (compile with -DSNTL_TRACE): one chosen CTA records (SM clock << 8 | event) per role, so
// the length of each pipeline phase and each hand-off can be read back.  Compiles to nothing otherwise.
#ifdef SNTL_TRACE
constexpr int kTraceRoles = 8, kTraceDepth = 2048;
static __device__ unsigned long long g_trace[kTraceRoles * kTraceDepth];
static __device__ unsigned int g_trace_cta;
__device__ __forceinline__ void trace_event(bool who, int role, int& n, uint32_t ev)
{
    if (who && blockIdx.x == g_trace_cta && n < kTraceDepth) g_trace[role * kTraceDepth + n++] = ((unsigned long long)clock64() << 8) | ev;
}
#define SNTL_TRACE_DECL(n) int n = 0
#define SNTL_TRACE_EV(who, role, n, ev) ::sntl::ptx::trace_event(who, role, n, ev)
#else
#define SNTL_TRACE_DECL(n)
#define SNTL_TRACE_EV(who, role, n, ev)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s

// Bounded wait for the phase with the given parity.  `abort_flag` is a CTA-shared word any waiter sets when
// it gives up; all later waits of the CTA then return false at once.  Returns true when the phase completed.
__device__ __forceinline__ bool mbar_wait_for(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t site,
                                              uint64_t limit_ns)
{
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 0x3ffu) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = global_timer_ns();
            if (now < *(volatile unsigned long long*)&g_abort_until_ns || now - t0 > limit_ns) {
                atomicCAS(&g_device_status, 0u, (site << 24) | (blockIdx.x & 0xffffffu));
                *(volatile unsigned long long*)&g_abort_until_ns = now + limit_ns;
                *abort_flag = 1u;
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t site)
{
    return mbar_wait_for(bar, parity, abort_flag, site, kWaitLimitNs);
}

// ---------------------------------------------------------------------------------------------------
// TMA (per-CTA tensor loads, no multicast)
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tiled load: coordinates (c0 = innermost element, c1 = row, c2 = slab); c0*elemsize must be a multiple of 16 B.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// fire-and-forget fp32 vector reduction into global memory (16-byte aligned)
__device__ __forceinline__ void red_add_v4(float* gptr, float a, float b, float c, float d)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(gptr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// asynchronous fp32 add-reduction of a contiguous shared-memory block into global memory (both 16-byte aligned,
// bytes a multiple of 16); tracked by bulk groups
__device__ __forceinline__ void bulk_reduce_add_f32(float* gmem_dst, const void* smem_src, uint32_t bytes)
{
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
}
// the same with 64-bit integer adds (two's complement: serves signed fixed-point sums)
__device__ __forceinline__ void bulk_reduce_add_u64(unsigned long long* gmem_dst, const void* smem_src, uint32_t bytes)
{
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.u64 [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// returns once at most N of this thread's bulk groups are still reading their shared-memory source
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// barrier among a subset of the CTA's warps (id 1..15; `threads` a multiple of 32)
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// per-warpgroup register re-allocation (all four warps of the warpgroup must execute it)
template <int N> __device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// packed fp32x2 arithmetic (two independent fp32 lanes in one 64-bit register)
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c)
{
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
          "l"(reinterpret_cast<unsigned long long&>(c)));
    return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b)
{
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b)
{
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}

// ---------------------------------------------------------------------------------------------------
// tcgen05: TMEM allocation, fences, commit
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols)  // one full warp
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)  // one full warp
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// mbarrier arrives once every MMA issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---------------------------------------------------------------------------------------------------
// UMMA descriptors (bf16 operands, fp32 accumulate)
// ---------------------------------------------------------------------------------------------------
// Instruction descriptor for kind::f16: D fp32 (bit 4), A/B bf16 (bits 7, 10), major-ness bits 15/16
// (0 = K-major, 1 = MN-major), N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, bool a_mn_major, bool b_mn_major)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.  Tiles are stored as rows of 128 bytes (64 bf16), the
// layout a TMA box with a 64-element inner extent and CU_TENSOR_MAP_SWIZZLE_128B produces; eight rows form
// one 1024-byte swizzle atom, tile bases are 1024-byte aligned.
//   K-major operand  (rows = M/N index, the 64 contiguous elements run along K): SBO = 1024 (next 8 rows),
//                    LBO unused; a K step of 16 elements advances the start address by 32 bytes.
//   MN-major operand (rows = K index, the 64 contiguous elements run along M/N): SBO = 1024 (next 8 K rows),
//                    LBO = byte distance between consecutive 64-element chunks along M/N; a K step of 16
//                    advances the start address by 16 rows = 2048 bytes.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A holds bf16 pairs packed in 32-bit TMEM columns (K/2 columns per row)
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Lean issue forms.  The single issuing thread shares its scheduler with busy softmax warps, so every instruction
// it spends per MMA shows up as tensor-pipe idle time: descriptors are built once per tile and advanced with one
// 64-bit add (the start-address field is in 16-byte units and never carries out of its 14 bits for addresses below
// 256 KB), and the accumulate flag is a compile-time constant wherever the k-step is known.
__device__ __forceinline__ uint64_t sdesc_advance(uint64_t desc, uint32_t bytes) { return desc + (uint64_t)(bytes >> 4); }
template <bool kAccumulate>
__device__ __forceinline__ void mma_ss_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc)
{
    if (kAccumulate)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                     "l"(a_desc), "l"(b_desc), "r"(idesc)
                     : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                     "l"(a_desc), "l"(b_desc), "r"(idesc)
                     : "memory");
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc)
{
    if (kAccumulate)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
                     "r"(a_tmem), "l"(b_desc), "r"(idesc)
                     : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
                     "r"(a_tmem), "l"(b_desc), "r"(idesc)
                     : "memory");
}

// One lane of a fully active warp (always the same one): lets an MMA-issuing warp run its loop with all 32 lanes --
// warp-uniform control flow, so descriptors and addresses can live in uniform registers -- with only the tcgen05
// instruction itself behind the election.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_ss_e(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc)
{
    if (elect_one()) mma_ss_c<kAccumulate>(d_tmem, a_desc, b_desc, idesc);
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_ts_e(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc)
{
    if (elect_one()) mma_ts_c<kAccumulate>(d_tmem, a_tmem, b_desc, idesc);
}
__device__ __forceinline__ void tc_commit_e(uint64_t* bar)
{
    if (elect_one()) tc_commit(bar);
}
// either form, chosen at compile time: kElect = a fully active warp with an elected lane, else the calling thread itself
template <bool kElect, bool kAccumulate>
__device__ __forceinline__ void mma_ss_x(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc)
{
    if constexpr (kElect) mma_ss_e<kAccumulate>(d_tmem, a_desc, b_desc, idesc);
    else mma_ss_c<kAccumulate>(d_tmem, a_desc, b_desc, idesc);
}
template <bool kElect, bool kAccumulate>
__device__ __forceinline__ void mma_ts_x(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc)
{
    if constexpr (kElect) mma_ts_e<kAccumulate>(d_tmem, a_tmem, b_desc, idesc);
    else mma_ts_c<kAccumulate>(d_tmem, a_tmem, b_desc, idesc);
}
template <bool kElect>
__device__ __forceinline__ void tc_commit_x(uint64_t* bar)
{
    if constexpr (kElect) tc_commit_e(bar);
    else tc_commit(bar);
}

// ---------------------------------------------------------------------------------------------------
// TMEM <-> registers.  32x32b shape: thread `lane` of warp w touches TMEM lane 32*(w%4)+lane and 32 (or 16)
// consecutive 32-bit columns starting at the column in taddr.  taddr = (lane << 16) | column.
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(
            taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// three-input maximum in one instruction (NaN operands are ignored, like fmaxf)
__device__ __forceinline__ float fmax3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// element-wise product of two bf16 pairs, rounded to nearest even
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

}  // namespace ptx

// Host side: encode a 3-D tiled tensor map over a bf16 [slabs][rows][D] tensor with a {64, box_rows, 1} box and
// 128-byte swizzle.  The driver entry point is looked up at run time, so the library does not link libcuda.
cudaError_t encode_tmap_bf16_3d(CUtensorMap* out, const void* base, int D, int rows, int slabs, int box_rows, int slab_rows = 0);
cudaError_t encode_tmap_bf16_3d_uncached(CUtensorMap* out, const void* base, int D, int rows, int slabs, int box_rows, int slab_rows);

}  // namespace sntl

// Causal attention forward for sm_100a: tcgen05 MMA with accumulators in TMEM, TMA-staged operands,
// warp-specialised producer / MMA / softmax roles.
//
// Replaces the reference's CudaFlashAttentionForwardWmma64Entry
// (sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1105-1266): same math -- S = scale*Q K^T, causal mask,
// online softmax, O = P V, LSE = m + ln(l) -- re-designed for Blackwell:
//
//   * one CTA owns 256 consecutive query rows of one (batch, head) as two 128-row tiles; each tile has its
//     own softmax warpgroup (one thread per query row: tcgen05.ld's 32x32b shape hands thread i row i, so the
//     row max / row sum need no shuffles) while a single MMA-issuing warp (one elected lane) feeds the tensor core for both,
//     so one tile's softmax overlaps the other tile's MMAs;
//   * S (fp32, 128 columns) and O (fp32, D columns) live in TMEM; P is written back as packed bf16 -- over S at
//     head_dim 128, into 64 columns of its own at head_dim 64, where the next S of the tile is then issued as soon as
//     the softmax warps have read the current one -- and consumed by the PV MMA straight from TMEM (A operand in
//     TMEM), V is consumed from shared memory as an MN-major operand, so nothing is transposed and P never touches
//     shared memory;
//   * Q/K/V tiles arrive by per-CTA TMA (128-byte swizzle, no multicast) into two-stage K and V rings
//     guarded by mbarriers; stages are released by tcgen05.commit;
//   * the softmax works in the exp2 domain with scale*log2(e) folded into one FMA, and rescales O lazily:
//     only when a row's running max grew by more than 2^8 since the last rescale;
//   * grouped-query heads index their shared K/V head directly (no repeated K/V as at
//     sentinel/NeuralNet/Cuda/CudaCausalSelfAttention.cu:27-34); CTAs are ordered heaviest-first and the query
//     heads of one group are adjacent in launch order so they share K/V tiles in L2.
//
// Layout: bf16 token-major [B][H][S][D], D in {64,128}; LSE [B][Hq][Sq] fp32 (natural log).
// TMEM map (512 columns): head_dim 128 and KV-cache mode S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D);
// head_dim 64 S0 [0,128) P0 [128,192) S1 [192,320) P1 [320,384) O0 [384,448) O1 [448,512).
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <algorithm>
#include <mutex>

namespace sntl {

using namespace ptx;

namespace {

constexpr int kM = 128;          // query rows per tile
constexpr int kN = 128;          // keys per tile
constexpr int kFwdThreads = 384; // 2 softmax warpgroups + 1 warpgroup holding the MMA warp and the TMA warp
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum WaitSite : uint32_t {
    kSiteQ = 1, kSiteKFull, kSiteVFull, kSiteKEmpty, kSiteVEmpty, kSiteSReady, kSitePReady, kSiteOReady, kSiteFinal, kSiteIssue
};

struct FwdParams {
    __nv_bfloat16* o;
    float* lse;
    int B, Hq, Hkv, Sq, Skv;
    int causal;
    int window, global_tokens;   // sliding window and always-visible first keys (0, 0: plain causal)
    // KV-cache mode: the rows of one slab are the (query head of the group, new token) pairs of one KV head, row r
    // sits at position Skv - new_tokens + r % new_tokens, and the key tiles are dealt to n_splits CTAs whose partial
    // (O, LSE) land in o / lse as [split][slab][row]
    int new_tokens, n_splits, tiles_per_split;
    int n_qblk;       // 256-row query blocks per (b, h)
    float scale_log2; // scale * log2(e)
};

struct FwdBarriers {
    uint64_t q_full;
    uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
    uint64_t s_ready[2], p_ready[2], o_ready[2];
    uint64_t p_half[2];      // the first 64 columns of P_t are written
    uint64_t final_bar;
    uint32_t tmem_base;
    uint32_t abort_flag;
    uint64_t s_free[2];      // head_dim 64 (plain / window): the softmax warps have read S_j of tile t
};

// kMode: kPlain = causal / full attention of a whole sequence; kWindow adds the sliding window (separate so that the
// plain kernel carries none of its bookkeeping); kCache = new tokens against a KV cache, grouped-query heads packed into
// the rows of one tile, keys split over CTAs.
enum FwdMode : int { kPlain = 0, kWindow = 1, kCache = 2 };

template <int D, int kMode>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const FwdParams p)
{
    constexpr int kTileBytes = 128 * D * 2;          // one 128-row tile of Q, K or V
    constexpr int kChunkBytes = 128 * 128;           // one 64-element-wide TMA box (128 rows x 128 B)
    constexpr int kChunks = D / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;                               // [2][kTileBytes]
    uint8_t* sK = sQ + 2 * kTileBytes;                // [2][kTileBytes]
    uint8_t* sV = sK + 2 * kTileBytes;                // [2][kTileBytes]
    FwdBarriers* bars = (FwdBarriers*)(sV + 2 * kTileBytes);
    volatile uint32_t* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- work decode: heaviest query blocks first; the heads of one KV group are adjacent ----
    constexpr bool kWin = kMode != kPlain;
    const int bh_count = kMode == kCache ? p.B * p.Hkv : p.B * p.Hq;
    int qblk_rank = blockIdx.x / bh_count;
    const int bh = blockIdx.x - qblk_rank * bh_count;
    int split = 0;
    if (kMode == kCache) {
        split = qblk_rank / p.n_qblk;
        qblk_rank -= split * p.n_qblk;
    }
    const int qblk = (p.causal && kMode != kCache) ? (p.n_qblk - 1 - qblk_rank) : qblk_rank;
    int bh_kv = bh;
    if (kMode != kCache) {
        const int b = bh / p.Hq, h = bh - b * p.Hq;
        bh_kv = b * p.Hkv + h / (p.Hq / p.Hkv);
    }
    // plain / window: the CTA owns two consecutive 128-row tiles.  Cache mode: it owns ONE 128-row tile and its two
    // softmax warpgroups take alternate key tiles of the CTA's piece (two independent streams, each with its own K/V
    // stage, S and O columns and running max / sum), so one stream's softmax overlaps the other's MMAs.
    const int q0 = kMode == kCache ? qblk * kM : qblk * 2 * kM;
    const int n_ktiles_all = (p.Skv + kN - 1) / kN;
    // position of a row in its sequence (what the causal and window masks compare keys with)
    auto row_pos = [&](int r) { return kMode == kCache ? p.Skv - p.new_tokens + r % p.new_tokens : r; };
    // Key tiles this CTA visits, in ascending order: the tiles holding global tokens, then the tiles from the window
    // of the block's first query row up to the diagonal.  Without a window that is simply 0 .. diagonal.
    // In cache mode every row of the slab sees keys up to (almost) the end of the cache; the list is cut into
    // tiles_per_split pieces and this CTA takes piece `split`.
    const int first_pos = kMode == kCache ? p.Skv - p.new_tokens : q0;   // lowest position among the CTA's rows
    const bool windowed = kWin && p.window > 0;
    const int g_tiles = windowed ? (p.global_tokens + kN - 1) / kN : 0;
    const int w_first = windowed ? max(g_tiles, max(0, first_pos - p.window + 1) / kN) : 0;
    const int list0 = kMode == kCache ? split * p.tiles_per_split : 0;
    auto key_tile = [&](int j) { j += list0; return j < g_tiles ? j : w_first + (j - g_tiles); };   // j-th load of the CTA
    int n_t[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int row0 = kMode == kCache ? q0 : q0 + t * kM;
        if (row0 >= p.Sq) n_t[t] = 0;
        else if (kMode == kCache) {
            const int n_list = min(g_tiles, n_ktiles_all) + max(0, n_ktiles_all - w_first);
            const int mine = max(0, min(p.tiles_per_split, n_list - list0));
            n_t[t] = (mine + 1 - t) / 2;       // stream t takes loads t, t + 2, ...
        } else if (p.causal) {
            const int diag = min(n_ktiles_all - 1, row0 / kN);
            n_t[t] = min(g_tiles, diag + 1) + max(0, diag - w_first + 1);
        } else n_t[t] = n_ktiles_all;
    }
    const int n_max = max(n_t[0], n_t[1]);
    const int n_loads = kMode == kCache ? n_t[0] + n_t[1] : n_max;   // K/V tiles the producer brings in

    // ---- setup ----
    if (warp == 9 && lane == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        mbar_init(&bars->q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->k_full[i], 1);
            mbar_init(&bars->k_empty[i], 1);
            mbar_init(&bars->v_full[i], 1);
            mbar_init(&bars->v_empty[i], 1);
            mbar_init(&bars->s_ready[i], 1);
            if (D == 64 && kMode != kCache) mbar_init(&bars->s_free[i], 128);
            mbar_init(&bars->p_ready[i], 128);
            mbar_init(&bars->p_half[i], 128);
            mbar_init(&bars->o_ready[i], 1);
        }
        mbar_init(&bars->final_bar, 1);
        bars->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(&bars->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    // head_dim 64 (plain / window kernels) leaves room for P in columns of its own: S_t [192t, 192t+128), P_t the next 64,
    // O_t [384+64t, +64).  The next S of a tile is then issued as soon as the softmax warps have READ the current one
    // instead of behind the P V product that consumes P, which takes a tile's two products out of the chain between two of
    // its softmax passes.  Otherwise (512 columns full at head_dim 128): S_t [128t, +128) with P written over it,
    // O_t [256+128t, +128).
    constexpr bool kOwnP = D == 64 && kMode != kCache;
    // (computed, not looked up: a two-element array indexed by the warp's tile would live in local memory)
    auto tmem_S = [&](int t) { return tmem + (uint32_t)t * (kOwnP ? 192u : 128u); };
    constexpr uint32_t kPOff = kOwnP ? 128u : 0u;   // P relative to the S of its tile
    // head_dim 128 (plain / window): P is written over S, so a tile's P V product and next S stay in the chain between two of
    // its softmax passes; there the first half of P V is issued as soon as the first 64 columns of P are written (-6 %)
    constexpr bool kHalfP = !kOwnP && kMode != kCache;
    auto tmem_O = [&](int t) { return tmem + (kOwnP ? 384u : 256u) + (uint32_t)t * (kOwnP ? 64u : 128u); };

    // 384 threads start with 168 registers each; each role re-allocates inside its own branch
    if (warp >= 10) {
        setmaxnreg_dec<72>();   // idle warps of the last warpgroup
    } else if (warp == 9) {
        setmaxnreg_dec<72>();
        // =========================== TMA producer ===========================
        if (lane == 0) {
            if (kMode == kCache) {      // one query tile, shared by both streams
                if (n_loads > 0) mbar_arrive_expect_tx(&bars->q_full, (uint32_t)kTileBytes);
                for (int c = 0; c < kChunks && n_loads > 0; ++c) tma_load_3d(sQ + c * kChunkBytes, &tmap_q, &bars->q_full, c * 64, q0, bh);
            } else {
                int n_valid = (n_t[0] > 0) + (n_t[1] > 0);
                mbar_arrive_expect_tx(&bars->q_full, (uint32_t)(n_valid * kTileBytes));
                for (int t = 0; t < 2; ++t)
                    if (n_t[t] > 0)
                        for (int c = 0; c < kChunks; ++c)
                            tma_load_3d(sQ + t * kTileBytes + c * kChunkBytes, &tmap_q, &bars->q_full, c * 64, q0 + t * kM, bh);
            }
            for (int j = 0; j < n_loads; ++j) {
                const int st = j & 1;
                if (j >= 2 && !mbar_wait(&bars->k_empty[st], ((j >> 1) - 1) & 1, abort_flag, kSiteKEmpty)) break;
                mbar_arrive_expect_tx(&bars->k_full[st], (uint32_t)kTileBytes);
                for (int c = 0; c < kChunks; ++c)
                    tma_load_3d(sK + st * kTileBytes + c * kChunkBytes, &tmap_k, &bars->k_full[st], c * 64, key_tile(j) * kN, bh_kv);
                if (j >= 2 && !mbar_wait(&bars->v_empty[st], ((j >> 1) - 1) & 1, abort_flag, kSiteVEmpty)) break;
                mbar_arrive_expect_tx(&bars->v_full[st], (uint32_t)kTileBytes);
                for (int c = 0; c < kChunks; ++c)
                    tma_load_3d(sV + st * kTileBytes + c * kChunkBytes, &tmap_v, &bars->v_full[st], c * 64, key_tile(j) * kN, bh_kv);
            }
        }
    } else if (warp == 8) {
        setmaxnreg_dec<72>();
        // =========================== MMA issuer ===========================
        // All 32 lanes walk the loops (warp-uniform control flow keeps descriptors and addresses in uniform registers) and
        // one elected lane issues each tcgen05 instruction: the warp shares its scheduler with two softmax warps and this
        // form needs fewer of the issue slots it is given per MMA than a single-lane loop (-3.7 % at head_dim 64, where
        // the issue order below makes this warp's pace count; no change at 128).  The KV-cache kernel, which is bound by
        // HBM, keeps a single lane.
        constexpr bool kElectF = kMode != kCache;
        if (kElectF || lane == 0) {
            auto wait = [&](uint64_t* bar, uint32_t parity, uint32_t site) {
                if constexpr (kElectF) return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, site));
                else return mbar_wait(bar, parity, abort_flag, site);
            };
            const bool tl8 = lane == 0;
            (void)tl8;
            SNTL_TRACE_DECL(tn);
            constexpr uint32_t idesc_s = make_idesc(kM, kN, false, false);
            constexpr uint32_t idesc_pv = make_idesc(kM, D, false, true);
            // one descriptor per tile, advanced per k-step by a 64-bit add
            const uint64_t dq0 = make_sdesc(smem_u32(sQ), 16, 1024), dq1 = sdesc_advance(dq0, kTileBytes);
            const uint64_t dk0 = make_sdesc(smem_u32(sK), 16, 1024), dk1 = sdesc_advance(dk0, kTileBytes);
            const uint64_t dv0 = make_sdesc(smem_u32(sV), kChunkBytes, 1024), dv1 = sdesc_advance(dv0, kTileBytes);
            auto issue_s = [&](int t, int st) {
                uint64_t a = (t && kMode != kCache) ? dq1 : dq0, b = st ? dk1 : dk0;
                asm volatile("" : "+l"(a), "+l"(b));   // keeps the advanced descriptors from being hoisted into registers
                const uint32_t d = tmem_S(t);
                mma_ss_x<kElectF, false>(d, a, b, idesc_s);
#pragma unroll
                for (int ks = 1; ks < D / 16; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * kChunkBytes + (ks & 3) * 32);
                    mma_ss_x<kElectF, true>(d, sdesc_advance(a, off), sdesc_advance(b, off), idesc_s);
                }
                tc_commit_x<kElectF>(&bars->s_ready[t]);
            };
            // With kHalfP, P V in two halves of the contraction: the first four k-steps need only the first 64 columns of P
            // (p_half, which the caller has waited for), the rest the whole of it (p_ready) -- so half the product is issued
            // while the softmax warps still compute the second half of their exponentials.  Otherwise the caller has waited
            // for the whole of P.  Returns false when a wait gave up.
            auto issue_pv = [&](int t, int st, bool accumulate, uint32_t parity) {
                uint64_t b = st ? dv1 : dv0;
                asm volatile("" : "+l"(b));
                const uint32_t d = tmem_O(t), a = tmem_S(t) + kPOff;
                if (accumulate) mma_ts_x<kElectF, true>(d, a, b, idesc_pv);
                else mma_ts_x<kElectF, false>(d, a, b, idesc_pv);
#pragma unroll
                for (int ks = 1; ks < kN / 32; ++ks) mma_ts_x<kElectF, true>(d, a + (uint32_t)(ks * 8), sdesc_advance(b, ks * 2048), idesc_pv);
                if constexpr (kHalfP) {
                    if (!wait(&bars->p_ready[t], parity, kSitePReady)) return false;
                    tc_fence_after();
                }
#pragma unroll
                for (int ks = kN / 32; ks < kN / 16; ++ks) mma_ts_x<kElectF, true>(d, a + (uint32_t)(ks * 8), sdesc_advance(b, ks * 2048), idesc_pv);
                tc_commit_x<kElectF>(&bars->o_ready[t]);
                return true;
            };
            if constexpr (kMode == kCache) {
                // two independent streams: stream t owns K/V stage t, S_t and O_t; its jj-th key tile is load 2*jj + t
                bool ok = n_max > 0 && wait(&bars->q_full, 0, kSiteQ);
                for (int t = 0; t < 2 && ok; ++t) {
                    if (n_t[t] == 0) continue;
                    if (!(ok = wait(&bars->k_full[t], 0, kSiteKFull))) break;
                    tc_fence_after();
                    issue_s(t, t);
                    tc_commit_x<kElectF>(&bars->k_empty[t]);
                }
                for (int jj = 0; ok && jj < n_max; ++jj) {
                    const uint32_t ph = (uint32_t)(jj & 1), nph = ph ^ 1u;
                    for (int t = 0; t < 2 && ok; ++t) {
                        if (jj >= n_t[t]) continue;
                        if (!(ok = wait(&bars->v_full[t], ph, kSiteVFull))) break;
                        if (!(ok = wait(kHalfP ? &bars->p_half[t] : &bars->p_ready[t], ph, kSitePReady))) break;
                        tc_fence_after();
                        if (!(ok = issue_pv(t, t, jj > 0, ph))) break;
                        tc_commit_x<kElectF>(&bars->v_empty[t]);
                        if (jj + 1 < n_t[t]) {
                            if (!(ok = wait(&bars->k_full[t], nph, kSiteKFull))) break;
                            tc_fence_after();
                            issue_s(t, t);
                            tc_commit_x<kElectF>(&bars->k_empty[t]);
                        }
                    }
                }
            } else if constexpr (kOwnP) {
                // With P in columns of its own the next S of a tile no longer waits for the P V product that consumes P:
                // per key tile j the thread first issues S_{j+1} of both query tiles, each as soon as its softmax warps have
                // READ S_j (s_free, early in their pass), then the two P V products of step j as their P arrive.
                bool ok = n_max > 0 && wait(&bars->q_full, 0, kSiteQ) &&
                          wait(&bars->k_full[0], 0, kSiteKFull);
                if (ok) {
                    tc_fence_after();
                    if (n_t[0] > 0) issue_s(0, 0);
                    if (n_t[1] > 0) issue_s(1, 0);
                    tc_commit_x<kElectF>(&bars->k_empty[0]);
                }
                for (int j = 0; ok && j < n_max; ++j) {
                    const int st = j & 1, nst = st ^ 1;
                    if (j + 1 < n_max) {
                        if (!(ok = wait(&bars->k_full[nst], (uint32_t)(((j + 1) >> 1) & 1), kSiteKFull))) break;
                        for (int t = 0; t < 2 && ok; ++t) {
                            if (j + 1 >= n_t[t]) continue;
                            if (!(ok = wait(&bars->s_free[t], (uint32_t)(j & 1), kSiteIssue))) break;
                            tc_fence_after();
                            issue_s(t, nst);
                        }
                        if (!ok) break;
                        tc_commit_x<kElectF>(&bars->k_empty[nst]);
                    }
                    if (!(ok = wait(&bars->v_full[st], (uint32_t)((j >> 1) & 1), kSiteVFull))) break;
                    for (int t = 0; t < 2 && ok; ++t) {
                        if (j >= n_t[t]) continue;
                        if (!(ok = wait(kHalfP ? &bars->p_half[t] : &bars->p_ready[t], (uint32_t)(j & 1), kSitePReady))) break;
                        tc_fence_after();
                        if (!(ok = issue_pv(t, st, j > 0, (uint32_t)(j & 1)))) break;
                    }
                    if (!ok) break;
                    tc_commit_x<kElectF>(&bars->v_empty[st]);
                }
            } else {
            bool ok = n_max > 0 && wait(&bars->q_full, 0, kSiteQ) &&
                      wait(&bars->k_full[0], 0, kSiteKFull);
            if (ok) {
                tc_fence_after();
                if (n_t[0] > 0) issue_s(0, 0);
                if (n_t[1] > 0) issue_s(1, 0);
                tc_commit_x<kElectF>(&bars->k_empty[0]);
            }
            for (int j = 0; ok && j < n_max; ++j) {
                const int st = j & 1, nst = st ^ 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1), nph = (uint32_t)(((j + 1) >> 1) & 1);
                if (!(ok = wait(&bars->v_full[st], ph, kSiteVFull))) break;
                bool next_k_ready = false;
                for (int t = 0; t < 2 && ok; ++t) {
                    if (j >= n_t[t]) continue;
                    if (!(ok = wait(kHalfP ? &bars->p_half[t] : &bars->p_ready[t], (uint32_t)(j & 1), kSitePReady))) break;
                    SNTL_TRACE_EV(tl8, 0, tn, 10 + t);
                    tc_fence_after();
                    if (!(ok = issue_pv(t, st, j > 0, (uint32_t)(j & 1)))) break;
                    SNTL_TRACE_EV(tl8, 0, tn, 20 + t);
                    if (j + 1 < n_t[t]) {
                        if (!next_k_ready) {
                            SNTL_TRACE_EV(tl8, 0, tn, 40);
                            if (!(ok = wait(&bars->k_full[nst], nph, kSiteKFull))) break;
                            tc_fence_after();
                            SNTL_TRACE_EV(tl8, 0, tn, 41);
                            next_k_ready = true;
                        }
                        issue_s(t, nst);
                        SNTL_TRACE_EV(tl8, 0, tn, 30 + t);
                    }
                }
                if (!ok) break;
                if (j + 1 < n_max) tc_commit_x<kElectF>(&bars->k_empty[nst]);
                tc_commit_x<kElectF>(&bars->v_empty[st]);
            }
            }
            // every MMA issued above must have retired before shared memory / TMEM are given up
            tc_commit_x<kElectF>(&bars->final_bar);
            wait(&bars->final_bar, 0, kSiteFinal);
        }
    } else {
        // =========================== softmax + epilogue warpgroups ===========================
        setmaxnreg_inc<216>();
        const int t = warp >> 2;                       // tile 0 or 1
        const int row = (warp & 3) * 32 + lane;        // row inside the tile == TMEM lane
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const int grow = kMode == kCache ? q0 + row : q0 + t * kM + row;   // query row inside the (batch, head) slab
        const int n_mine = n_t[t];
        SNTL_TRACE_DECL(tn);
        const bool tw = (warp & 3) == 0 && lane == 0;
        (void)tw;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_mine; ++j) {
            if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_ready[t], (uint32_t)(j & 1), abort_flag, kSiteSReady)))) break;
            SNTL_TRACE_EV(tw, 1 + t, tn, 1);
            tc_fence_after();
            uint32_t s[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(tmem_S(t) + lane_off + (uint32_t)(c * 32), s + c * 32);
            tmem_ld_wait();
            if constexpr (kOwnP) {      // S_j is in registers: the next S of this tile may overwrite it
                tc_fence_before();
                mbar_arrive(&bars->s_free[t]);
            }
            SNTL_TRACE_EV(tw, 1 + t, tn, 2);
            // number of visible keys of this row inside this tile
            const int key0 = key_tile(kMode == kCache ? 2 * j + t : j) * kN;
            const int qpos = row_pos(grow);
            int limit = (p.causal ? min(p.Skv, qpos + 1) : p.Skv) - key0;
            if (limit < kN) {
#pragma unroll
                for (int c = 0; c < kN; ++c)
                    if (c >= limit) s[c] = 0xff800000u;  // -inf
            }
            if (kWin && (kMode != kCache || p.window > 0)) {
                // keys below the row's window are hidden unless they are global tokens
                const int lo = qpos - p.window + 1 - key0, glim = p.global_tokens - key0;
                if (lo > 0 && glim < min(lo, kN)) {
#pragma unroll
                    for (int c = 0; c < kN; ++c)
                        if (c < lo && c >= glim) s[c] = 0xff800000u;
                }
            }
            // row max with eight independent chains (a single 128-long dependent chain costs ~600 cycles) of
            // three-input maxima: half the instructions of a two-input reduction
            float mx8[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) mx8[c] = __uint_as_float(s[c]);
#pragma unroll
            for (int c = 8; c + 16 <= kN; c += 16)
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmax3(mx8[i], __uint_as_float(s[c + i]), __uint_as_float(s[c + 8 + i]));
#pragma unroll
            for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(mx8[i], __uint_as_float(s[kN - 8 + i]));
            const float mx = fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
            const float m_new = fmaxf(m_ref, mx * p.scale_log2);
            SNTL_TRACE_EV(tw, 1 + t, tn, 3);
            const bool need = (m_new - m_ref) > kRescaleThreshold;   // false when both are -inf (NaN compare)
            if constexpr (kOwnP) {      // P_{j-1} has been consumed (and O holds its product): P_j may be written
                if (j > 0) {
                    if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_ready[t], (uint32_t)((j - 1) & 1), abort_flag, kSiteOReady)))) break;
                    tc_fence_after();
                }
            }
            if (j == 0) {
                m_ref = m_new;
            } else if (__any_sync(0xffffffffu, need)) {
                if (!kOwnP && !(ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_ready[t], (uint32_t)((j - 1) & 1), abort_flag, kSiteOReady)))) break;
                tc_fence_after();
                const float factor = need ? ex2(m_ref - m_new) : 1.0f;
                if (need) m_ref = m_new;
                l *= factor;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld32(tmem_O(t) + lane_off + (uint32_t)(c * 32), o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                    tmem_st32(tmem_O(t) + lane_off + (uint32_t)(c * 32), o);
                }
                tmem_st_wait();
            }
            SNTL_TRACE_EV(tw, 1 + t, tn, 4);
            const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref;
            // exp2, row sum (four independent partial sums) and bf16 packing, 64 columns at a time so the packed half
            // can be stored while the other half is computed
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(neg_m, neg_m);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t pk[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float2 x = ffma2(make_float2(__uint_as_float(s[h * 64 + 2 * c]), __uint_as_float(s[h * 64 + 2 * c + 1])), sc2, nm2);
                    const float p0 = ex2(x.x), p1 = ex2(x.y);
                    l4[c & 3] += p0 + p1;
                    pk[c] = pack_bf16(p0, p1);
                }
                tmem_st32(tmem_S(t) + kPOff + lane_off + (uint32_t)(h * 32), pk);
                if (kHalfP && h == 0) {   // the P V product may start on the first 64 keys while the rest is computed
                    tmem_st_wait();
                    tc_fence_before();
                    mbar_arrive(&bars->p_half[t]);
                }
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            SNTL_TRACE_EV(tw, 1 + t, tn, 5);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&bars->p_ready[t]);
            SNTL_TRACE_EV(tw, 1 + t, tn, 6);
        }
        if (__all_sync(0xffffffffu, ok && n_mine > 0 && mbar_wait(&bars->o_ready[t], (uint32_t)((n_mine - 1) & 1), abort_flag, kSiteOReady))) {
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const bool store = grow < p.Sq;
            // cache mode: each stream of each split writes its own partial result, [2 * split + t][slab][row]
            const size_t part = kMode == kCache ? (size_t)(2 * split + t) : 0;
            const size_t out_row = (part * bh_count + bh) * p.Sq + (size_t)(store ? grow : 0);
            // Coalesced store of O.  A thread holds one whole row (2*D bytes); written straight from there a warp's store
            // instruction would touch 32 rows, 16 bytes each.  So the warp's 32 rows go through shared memory -- this tile's
            // Q buffer, free since the last S product of this tile retired (o_ready of the last step implies it) -- and
            // come back out with each store instruction covering whole
            // rows: 16 lanes x 16 bytes = one 256-byte row at head_dim 128, 8 lanes per 128-byte row at 64.  Only the rows of
            // this warp are exchanged, so a warp-level sync is all it takes; 16-byte units are XOR-swizzled by the row so
            // that both the row-wise writes and the row-wise reads spread over the banks.
            // (Cache mode: the two streams share ONE query tile, which the other stream may still be reading, but each owns
            // K stage t, and that stage gets no further load once the stream's last tile is done.)
            constexpr int kUnits = D / 8;                       // 16-byte units per row
            uint8_t* stage = (kMode == kCache ? sK : sQ) + t * kTileBytes + (warp & 3) * 32 * (D * 2);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(tmem_O(t) + lane_off + (uint32_t)(c * 32), o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 w;
                    w.x = pack_bf16(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
                    w.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
                    w.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
                    w.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
                    const int unit = c * 4 + i;
                    *reinterpret_cast<uint4*>(stage + lane * (D * 2) + ((unit ^ (lane & (kUnits - 1) & 7)) << 4)) = w;
                }
            }
            __syncwarp();
            {
                constexpr int kRowsPerStore = 32 / kUnits;       // rows one store instruction of the warp covers
                const int sub = lane / kUnits, unit = lane % kUnits;
                const int warp_row0 = grow - lane;                // first row of this warp inside the slab
                const size_t part_base = (part * bh_count + bh) * (size_t)p.Sq;
#pragma unroll
                for (int i = 0; i < 32 / kRowsPerStore; ++i) {
                    const int r = i * kRowsPerStore + sub;        // row inside the warp's 32
                    const uint4 w = *reinterpret_cast<const uint4*>(stage + r * (D * 2) + ((unit ^ (r & (kUnits - 1) & 7)) << 4));
                    if (warp_row0 + r < p.Sq)
                        *reinterpret_cast<uint4*>(p.o + (part_base + (size_t)(warp_row0 + r)) * D + unit * 8) = w;
                }
            }
            if (store)
                p.lse[out_row] = l > 0.0f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
        } else if (kMode == kCache && ok && n_mine == 0 && grow < p.Sq) {
            // a stream that got no key tile (a piece of one tile): its partial result weighs nothing in the merge
            p.lse[((size_t)(2 * split + t) * bh_count + bh) * p.Sq + grow] = -INFINITY;
        }
    }

    // ---- teardown ----
    if (*abort_flag) {
        // a wait gave up: let TMA copies that may still be in flight land before the CTA's memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    });
    return fn;
}

template <int D, int kMode>
cudaError_t launch_fwd(const TcArgs& a, cudaStream_t st)
{
    const AttnShape& s = a.s;
    CUtensorMap tq, tk, tv;
    cudaError_t e;
    if ((e = encode_tmap_bf16_3d(&tq, a.q, D, s.Sq, s.B * s.Hq, 128)) != cudaSuccess) return e;
    if ((e = encode_tmap_bf16_3d(&tk, a.k, D, s.Skv, s.B * s.Hkv, 128)) != cudaSuccess) return e;
    if ((e = encode_tmap_bf16_3d(&tv, a.v, D, s.Skv, s.B * s.Hkv, 128)) != cudaSuccess) return e;
    FwdParams p{};
    p.o = a.o_out;
    p.lse = a.lse_out;
    p.B = s.B; p.Hq = s.Hq; p.Hkv = s.Hkv; p.Sq = s.Sq; p.Skv = s.Skv;
    p.causal = s.causal;
    p.window = s.causal ? s.window : 0;
    p.global_tokens = s.global_tokens;
    p.n_qblk = (s.Sq + 2 * kM - 1) / (2 * kM);
    p.scale_log2 = s.scale * 1.4426950408889634f;
    const long long ctas = (long long)p.n_qblk * s.B * s.Hq;
    if (ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const size_t smem = 6 * (size_t)(128 * D * 2) + sizeof(FwdBarriers) + 1024;
    static std::atomic<unsigned long long> configured{0};   // per instantiation, one bit per device
    if ((e = ensure_dynamic_smem(attn_fwd_tc_kernel<D, kMode>, smem, configured)) != cudaSuccess) return e;
    attn_fwd_tc_kernel<D, kMode><<<(unsigned)ctas, kFwdThreads, smem, st>>>(tq, tk, tv, p);
    count_launch();
    return cudaGetLastError();
}

// ---- KV-cache mode ----------------------------------------------------------------------------------------------
// Combines the per-split partial results: LSE = log sum_s exp(lse_s), O = sum_s exp(lse_s - LSE) * O_s.  One warp per
// row; a split that saw no visible key for the row carries LSE = -inf and weighs nothing.
template <int D>
__global__ void __launch_bounds__(256) cache_merge_kernel(const __nv_bfloat16* __restrict__ o_part, const float* __restrict__ lse_part,
                                                          int n_splits, long long rows, __nv_bfloat16* __restrict__ o,
                                                          float* __restrict__ lse)
{
    const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    float m = -INFINITY;
    for (int sp = lane; sp < n_splits; sp += 32) m = fmaxf(m, lse_part[(size_t)sp * rows + r]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float sum = 0.0f;
    if (m > -INFINITY)
        for (int sp = lane; sp < n_splits; sp += 32) sum += __expf(lse_part[(size_t)sp * rows + r] - m);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float total = m > -INFINITY ? m + __logf(sum) : -INFINITY;
    constexpr int kPer = D / 32;   // consecutive elements per lane
    float acc[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) acc[i] = 0.0f;
    for (int sp = 0; sp < n_splits; ++sp) {
        const float l = lse_part[(size_t)sp * rows + r];
        if (!(l > -INFINITY)) continue;
        const float w = __expf(l - total);
        const __nv_bfloat16* src = o_part + ((size_t)sp * rows + r) * D + lane * kPer;
#pragma unroll
        for (int i = 0; i < kPer; ++i) acc[i] = fmaf(w, __bfloat162float(src[i]), acc[i]);
    }
    __nv_bfloat16* dst = o + (size_t)r * D + lane * kPer;
#pragma unroll
    for (int i = 0; i < kPer; ++i) dst[i] = __float2bfloat16(acc[i]);
    if (lane == 0) lse[r] = total;
}

template <int D>
cudaError_t launch_cache(const TcArgs& a, int capacity, void* workspace, cudaStream_t st)
{
    const AttnShape& s = a.s;
    const CachePlan plan = tc_cache_plan(s);
    const int group = s.Hq / s.Hkv, rows_per_slab = group * s.Sq, slabs = s.B * s.Hkv;
    const long long rows = (long long)slabs * rows_per_slab;
    CUtensorMap tq, tk, tv;
    cudaError_t e;
    // Q [B][Hq][new][D] read as [B*Hkv][group*new][D]: the query heads of a group are consecutive heads
    if ((e = encode_tmap_bf16_3d(&tq, a.q, D, rows_per_slab, slabs, 128)) != cudaSuccess) return e;
    if ((e = encode_tmap_bf16_3d(&tk, a.k, D, s.Skv, slabs, 128, capacity)) != cudaSuccess) return e;
    if ((e = encode_tmap_bf16_3d(&tv, a.v, D, s.Skv, slabs, 128, capacity)) != cudaSuccess) return e;
    const int n_parts = 2 * plan.n_splits;   // two key streams per CTA
    float* lse_part = reinterpret_cast<float*>(workspace);
    __nv_bfloat16* o_part = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(workspace) +
                                                             (((size_t)n_parts * rows * sizeof(float) + 255) / 256) * 256);
    FwdParams p{};
    p.o = o_part;
    p.lse = lse_part;
    p.B = s.B; p.Hq = s.Hq; p.Hkv = s.Hkv; p.Sq = rows_per_slab; p.Skv = s.Skv;
    p.causal = 1;
    p.window = s.window;
    p.global_tokens = s.global_tokens;
    p.new_tokens = s.Sq;
    p.n_splits = plan.n_splits;
    p.tiles_per_split = plan.tiles_per_split;
    p.n_qblk = (rows_per_slab + kM - 1) / kM;
    p.scale_log2 = s.scale * 1.4426950408889634f;
    const size_t smem = 6 * (size_t)(128 * D * 2) + sizeof(FwdBarriers) + 1024;
    static std::atomic<unsigned long long> configured{0};   // one bit per device
    if ((e = ensure_dynamic_smem(attn_fwd_tc_kernel<D, kCache>, smem, configured)) != cudaSuccess) return e;
    const long long ctas = (long long)plan.n_splits * p.n_qblk * slabs;
    if (ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    attn_fwd_tc_kernel<D, kCache><<<(unsigned)ctas, kFwdThreads, smem, st>>>(tq, tk, tv, p);
    count_launch();
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    cache_merge_kernel<D><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(o_part, lse_part, n_parts, rows, a.o_out, a.lse_out);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

// Key tiles the cache-mode kernel visits (global-token tiles, then the window of the oldest new token up to the end of
// the cache) and how they are dealt to CTAs: about one CTA per SM in total.
CachePlan tc_cache_plan(const AttnShape& s)
{
    const int n_tiles = (s.Skv + kN - 1) / kN;
    int n_list = n_tiles;
    if (s.window > 0) {
        const int g_tiles = (s.global_tokens + kN - 1) / kN;
        const int first_pos = s.Skv - s.Sq;
        const int w_first = std::max(g_tiles, std::max(0, first_pos - s.window + 1) / kN);
        n_list = std::min(g_tiles, n_tiles) + std::max(0, n_tiles - w_first);
    }
    const int group = s.Hq / s.Hkv;
    const long long base = (long long)s.B * s.Hkv * ((group * s.Sq + kM - 1) / kM);
    // pieces of at least two tiles (one per stream of a CTA), about one CTA per SM in total
    int want = (int)std::max(1LL, std::min<long long>((n_list + 1) / 2, 148 / std::max(1LL, base)));
    CachePlan plan;
    plan.tiles_per_split = (n_list + want - 1) / want;
    plan.n_splits = (n_list + plan.tiles_per_split - 1) / plan.tiles_per_split;
    return plan;
}

size_t tc_cache_workspace_bytes(const AttnShape& s)
{
    const size_t n_parts = 2 * (size_t)tc_cache_plan(s).n_splits;
    const size_t rows = (size_t)s.B * s.Hq * s.Sq;
    return ((n_parts * rows * sizeof(float) + 255) / 256) * 256 + n_parts * rows * s.D * 2;
}

bool tc_cache_supported(const AttnShape& s)
{
    return (s.D == 64 || s.D == 128) && s.causal && s.Sq <= s.Skv;
}

cudaError_t tc_cache_forward(const TcArgs& a, int capacity, void* workspace, cudaStream_t st)
{
    return a.s.D == 64 ? launch_cache<64>(a, capacity, workspace, st) : launch_cache<128>(a, capacity, workspace, st);
}

// A training loop calls with the same tensors step after step (the reference's trainer even replays a captured graph
// with identical pointers, CudaLanguageModel.cu:2176-2209), and on small problems the seven driver calls that encode
// the tensor maps of one forward + backward are a visible part of the launch path.  So the last few encodings are
// kept, keyed by everything that goes into one; a tensor map holds no data, only the address and the geometry, so a
// hit is exact whatever has happened to the memory since.
namespace {
struct TmapKey {
    const void* base; int D, rows, slabs, box_rows, slab_rows;
    bool operator==(const TmapKey& o) const
    {
        return base == o.base && D == o.D && rows == o.rows && slabs == o.slabs && box_rows == o.box_rows && slab_rows == o.slab_rows;
    }
};
constexpr int kTmapCacheSize = 32;
struct TmapCache {
    std::mutex guard;
    TmapKey keys[kTmapCacheSize];
    CUtensorMap maps[kTmapCacheSize];
    int used = 0, next = 0;
};
TmapCache& tmap_cache()
{
    static TmapCache* c = new TmapCache;
    return *c;
}
}  // namespace

cudaError_t encode_tmap_bf16_3d(CUtensorMap* out, const void* base, int D, int rows, int slabs, int box_rows, int slab_rows)
{
    if (slab_rows <= 0) slab_rows = rows;   // rows of storage per slab (a KV cache holds more rows than are in use)
    const TmapKey key{base, D, rows, slabs, box_rows, slab_rows};
    TmapCache& cache = tmap_cache();
    {
        std::lock_guard<std::mutex> lock(cache.guard);
        for (int i = 0; i < cache.used; ++i)
            if (cache.keys[i] == key) { *out = cache.maps[i]; return cudaSuccess; }
    }
    const cudaError_t e = encode_tmap_bf16_3d_uncached(out, base, D, rows, slabs, box_rows, slab_rows);
    if (e == cudaSuccess) {
        std::lock_guard<std::mutex> lock(cache.guard);
        const int slot = cache.next;
        cache.keys[slot] = key;
        cache.maps[slot] = *out;
        cache.next = (slot + 1) % kTmapCacheSize;
        if (cache.used < kTmapCacheSize) ++cache.used;
    }
    return e;
}

cudaError_t encode_tmap_bf16_3d_uncached(CUtensorMap* out, const void* base, int D, int rows, int slabs, int box_rows, int slab_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cudaErrorNotSupported;
    if (((uintptr_t)base & 15u) != 0) return cudaErrorMisalignedAddress;
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)slabs};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)slab_rows * D * 2};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

bool tc_fwd_supported(const AttnShape& s)
{
    return (s.D == 64 || s.D == 128) && (!s.causal || s.Sq == s.Skv);
}

cudaError_t tc_forward(const TcArgs& a, cudaStream_t st)
{
    const bool win = a.s.causal && a.s.window > 0;
    if (a.s.D == 64) return win ? launch_fwd<64, kWindow>(a, st) : launch_fwd<64, kPlain>(a, st);
    return win ? launch_fwd<128, kWindow>(a, st) : launch_fwd<128, kPlain>(a, st);
}

#ifdef SNTL_TRACE
// trace build only: choose the CTA that records and read back what the last launch recorded
extern "C" int sntl_debug_trace_fwd(unsigned long long* out, int n_words, int set_cta)
{
    if (out && cudaMemcpyFromSymbol(out, ptx::g_trace, sizeof(unsigned long long) * n_words) != cudaSuccess) return 1;
    static unsigned long long zeros[ptx::kTraceRoles * ptx::kTraceDepth];
    if (cudaMemcpyToSymbol(ptx::g_trace, zeros, sizeof(zeros)) != cudaSuccess) return 2;
    unsigned int c = (unsigned int)set_cta;
    return cudaMemcpyToSymbol(ptx::g_trace_cta, &c, sizeof(c)) == cudaSuccess ? 0 : 3;
}
#endif

// Self-test of the bounded wait: one warp waits on a barrier that by construction never receives its arrival, with a
// limit of `limit_ns` instead of the kernels' one second.  The wait runs out, records kSiteSelfTest in the status word
// exactly as a stuck production wait would, and the kernel returns normally (no trap, the context stays usable).
constexpr uint32_t kSiteSelfTest = 0x7e;
__global__ void wait_selftest_kernel(unsigned long long limit_ns, unsigned int* gave_up)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_word;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        abort_word = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    const bool done = ptx::mbar_wait_for(&bar, 0, &abort_word, kSiteSelfTest, limit_ns);
    if (threadIdx.x == 0 && gave_up) *gave_up = done ? 0u : 1u;
}

cudaError_t launch_wait_selftest(unsigned long long limit_ns, unsigned int* gave_up, cudaStream_t st)
{
    wait_selftest_kernel<<<1, 32, 0, st>>>(limit_ns, gave_up);
    count_launch();
    return cudaGetLastError();
}

cudaError_t read_and_clear_fwd_status(cudaStream_t st, uint32_t* word)
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

/*
 * sntl_attn.h -- C ABI of the B200 (sm_100a) causal self-attention library.
 *
 * This is the boundary a Sentinel build binds instead of its flash-attention launch sites.  Every entry
 * point takes plain pointers and sizes; the caller owns all tensors and all scratch memory, and names the
 * CUDA stream.  No entry point allocates, frees or synchronises, so calls may sit inside a stream capture
 * once the first (eager) call of each kind on a device has been made (that first call sets kernel
 * attributes and encodes nothing that depends on data).
 *
 * Reference interfaces replaced (paths relative to the reference project root):
 *   sntl_attn_fwd   <- CudaFlashAttention::forwardMultiHead
 *                      sentinel/NeuralNet/Cuda/CudaFlashAttention.hpp:30, .cu:1543-1609
 *                      (call site sentinel/NeuralNet/Cuda/CudaCausalSelfAttention.cu:237-249)
 *   sntl_attn_bwd   <- CudaFlashAttention::backwardMultiHead
 *                      sentinel/NeuralNet/Cuda/CudaFlashAttention.hpp:40, .cu:1615-1700
 *                      (call site sentinel/NeuralNet/Cuda/CudaCausalSelfAttention.cu:421-438)
 *   sntl_attn_bwd_workspace_bytes / sntl_attn_fwd_workspace_bytes
 *                   <- the callee-side ensureSize of deltaWorkspace, CudaFlashAttention.cu:1638
 *   shape checks    <- validateMultiHeadShape / resolveColumnWindow,
 *                      sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1458-1471, :1533-1539
 *
 * Differences from the reference that a binding must know:
 *   - grouped-query attention is native: K/V carry kv_heads heads (the reference needs them repeated to
 *     q_heads rows, CudaFlashAttention.cu:1467); kv_heads == q_heads reproduces the reference call.
 *   - dK/dV are overwritten deterministically (the reference accumulates with atomics into buffers the
 *     caller zeroes first, CudaCausalSelfAttention.cu:391-394 -- zeroing first stays harmless).
 *   - head_dim 128 is supported (reference: maxHeadDimension = 64, CudaFlashAttention.hpp:16).
 */
#ifndef SNTL_ATTN_H
#define SNTL_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  0 is success; the C++ compat layer maps BAD_ARGUMENT/UNSUPPORTED to std::invalid_argument
 * and the rest to std::runtime_error, the reference's convention (CudaFlashAttention.cu:1459-1470, :1608). */
enum {
    SNTL_OK = 0,
    SNTL_ERR_BAD_ARGUMENT = 1,   /* null pointer, non-positive extent, q_heads % kv_heads != 0, bad window */
    SNTL_ERR_UNSUPPORTED = 2,    /* shape/dtype/layout combination no kernel covers */
    SNTL_ERR_WORKSPACE = 3,      /* workspace missing or smaller than *_workspace_bytes() */
    SNTL_ERR_CUDA = 4,           /* a CUDA runtime/driver call or a launch failed */
    SNTL_ERR_NO_DEVICE = 5,      /* current device is not compute capability 10.x */
    SNTL_ERR_DEVICE_TIMEOUT = 6, /* a bounded device-side wait ran out (reported by sntl_attn_poll_device_status) */
    SNTL_ERR_SCRATCH_LIMIT = 7,  /* sntl_attn_bwd_static_scratch: the problem needs more than the built-in scratch */
    SNTL_ERR_COMM = 8            /* sntl_ring_*: NCCL is not available, or an NCCL call failed */
};

enum { SNTL_DTYPE_BF16 = 0, SNTL_DTYPE_F32 = 1 };

/* Tensor layouts.
 *   BHSD      token-major: element (b,h,s,d) at ((b*H + h)*S + s)*D + d; LSE/delta are [B][Hq][S] fp32.
 *   SENTINEL  the reference's feature-major matrix, (H*D) rows x stride_columns columns, fp32 only:
 *             element (b,h,s,d) at (h*D + d)*stride_columns + column_start + b*S + s, i.e. "packs" are
 *             consecutive column windows of S tokens (CudaFlashAttention.cu:129-131, :358-361);
 *             LSE is q_heads x stride_columns with the same column rule. */
enum { SNTL_LAYOUT_BHSD = 0, SNTL_LAYOUT_SENTINEL = 1 };

/* Flags. */
enum {
    /* fp32 tensors may be computed with bf16 tensor-core operands (fp32 accumulate).  Without it fp32
     * tensors take the exact-fp32 kernel.  The reference rounds operands to fp16 on its flash path
     * (CudaFlashAttention.cu:209-214), so this is the analogous trade. */
    SNTL_FLAG_ALLOW_BF16_COMPUTE = 1,
    /* never use the tensor-core kernels (diagnostics / cross-checks) */
    SNTL_FLAG_FORCE_SIMT = 2,
    /* Backward: make dQ bit-reproducible from run to run.  The tensor-core kernel sums the dQ contributions of the
     * key tiles in global memory in their order of arrival; fp32 addition is not associative, so without this flag
     * the last bits of dQ vary between runs (dK, dV and the forward are always reproducible: each of their elements
     * has one owner).  With it every contribution is converted exactly to 64-bit fixed point (2^-32 units) and
     * summed as integers, which no order can change; the sum is rounded once at the end, so it is also slightly
     * more accurate.  Cost: the dQ accumulator in the workspace and its reduction traffic double
     * (sntl_attn_bwd_workspace_bytes accounts for it).  |dQ / scale| must stay below 2^31.  The reference's
     * head_dim-64 backward has an exclusive dQ store (sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1434-1455);
     * a caller that relies on bit-stable input gradients sets this flag.  Ignored by the exact kernels, whose
     * dQ is reproducible already. */
    SNTL_FLAG_DETERMINISTIC = 4,
    /* sntl_ring_attn_fwd / _bwd only: the shard a rank passes is already its two zigzag chunks.  The sequence is cut in
     * 2*world equal chunks; tokens [0, S/2W) of rank r's shard are chunk r and tokens [S/2W, S/W) are chunk
     * 2*world-1-r (results come back in the same order).  A host that keeps its activations in this order for the whole
     * model -- the usual arrangement of causal sequence parallelism -- saves the redistribution round before and after
     * every call: the deal becomes a local copy. */
    SNTL_FLAG_RING_ZIGZAG = 8
};

typedef struct sntl_attn_desc {
    int32_t dtype;           /* SNTL_DTYPE_*  (element type of Q,K,V,O,dO,dQ,dK,dV) */
    int32_t layout;          /* SNTL_LAYOUT_* */
    int32_t batch;           /* independent sequences (the reference's packCount) */
    int32_t q_heads;
    int32_t kv_heads;        /* divides q_heads */
    int32_t seq_q;           /* query tokens per sequence (the reference's columnCount) */
    int32_t seq_kv;          /* key tokens per sequence; must equal seq_q when causal */
    int32_t head_dim;        /* tensor-core kernels: 64 or 128; exact kernel: any even value <= 256 */
    float scale;             /* softmax scale, normally 1/sqrt(head_dim) */
    int32_t causal;          /* 1: key j visible to query i iff j <= i.  0: all keys visible */
    int32_t stride_columns;  /* SENTINEL layout: columns of the matrices (q.cols); ignored for BHSD */
    int32_t column_start;    /* SENTINEL layout: first column of the window; ignored for BHSD */
    int32_t flags;           /* SNTL_FLAG_* */
    /* Sliding window with global tokens, the reference's CausalSelfAttention::allowsKey
     * (sentinel/NeuralNet/Layers/CausalSelfAttention.cpp:95-100; its CUDA flash path refuses such layers,
     * sentinel/NeuralNet/Cuda/CudaCausalSelfAttention.cu:50):
     * key j is visible to query i iff j <= i and (j < global_tokens or window_size <= 0 or j >= i - window_size + 1).
     * Both need causal = 1; 0 / 0 is plain causal attention. */
    int32_t window_size;     /* keys a query sees counting itself; <= 0: unlimited */
    int32_t global_tokens;   /* the first global_tokens keys stay visible to every later query; >= 0 */
} sntl_attn_desc;

/* Library version (major*10000 + minor*100 + patch). */
int sntl_attn_version(void);

/* Static text for a status code. */
const char* sntl_status_string(int status);

/* Scratch bytes sntl_attn_fwd needs for this descriptor (0 unless a layout/dtype staging copy is needed). */
size_t sntl_attn_fwd_workspace_bytes(const sntl_attn_desc* desc);

/* Scratch bytes sntl_attn_bwd needs: delta [B][Hq][Sq] fp32, the fp32 dQ accumulator of the tensor-core
 * kernel, and staging copies when the layout/dtype is converted. */
size_t sntl_attn_bwd_workspace_bytes(const sntl_attn_desc* desc);

/* O = softmax(scale * Q K^T + mask) V and LSE = m + ln(sum exp(s - m)) (natural log) per (b, head, query).
 * q,o: q_heads heads; k,v: kv_heads heads.  A query row with no visible key gets O = 0, LSE = -inf.
 * workspace may be null when sntl_attn_fwd_workspace_bytes() is 0.  Asynchronous on `stream`
 * (a cudaStream_t passed as void*; null = the legacy default stream). */
int sntl_attn_fwd(const sntl_attn_desc* desc, const void* q, const void* k, const void* v, void* o, float* lse,
                  void* workspace, size_t workspace_bytes, void* stream);

/* New tokens against a KV cache, forward only: the reference's attendCachedQuery / decode
 * (sentinel/NeuralNet/Cuda/CudaCausalSelfAttention.cu:318-341, :557-571) and, with seq_q > 1, a prefill continued from a cache.
 *   desc->seq_q   new tokens per head (1 for decode); desc->seq_kv  keys in use, the new tokens' own keys included
 *   (append before calling, as the reference does); query i sits at position seq_kv - seq_q + i and sees keys
 *   j <= that position, subject to window_size / global_tokens; desc->causal must be 1.
 *   BHSD:     q, o [B][Hq][seq_q][D]; k_cache, v_cache [B][Hkv][cache_capacity][D]; lse [B][Hq][seq_q].
 *   SENTINEL: q, o (Hq*D) x stride_columns with the new tokens at columns [column_start, column_start + seq_q);
 *             k_cache, v_cache (Hkv*D) x cache_capacity, key j in column j (CudaKvCache); batch must be 1.
 * bf16 BHSD tensors with head_dim 64 / 128 run on the tensor-core kernel: the query heads of one KV group are the
 * rows of one tile (K/V are read once per group) and the keys are split over about one CTA per SM, merged by a
 * second kernel.  Everything else runs on the exact kernel.  Scratch: sntl_attn_cached_fwd_workspace_bytes(). */
size_t sntl_attn_cached_fwd_workspace_bytes(const sntl_attn_desc* desc, int32_t cache_capacity);
int sntl_attn_cached_fwd(const sntl_attn_desc* desc, const void* q, const void* k_cache, const void* v_cache,
                         int32_t cache_capacity, void* o, float* lse, void* workspace, size_t workspace_bytes, void* stream);

/* dQ, dK, dV from dO with P recomputed as exp(scale*q.k - LSE) and delta = rowsum(dO o O).
 * dq: q_heads heads, overwritten.  dk, dv: kv_heads heads, overwritten with the sum over the query heads
 * of each group.  Asynchronous on `stream`. */
int sntl_attn_bwd(const sntl_attn_desc* desc, const void* q, const void* k, const void* v, const void* o,
                  const float* lse, const void* dout, void* dq, void* dk, void* dv, void* workspace,
                  size_t workspace_bytes, void* stream);

/* Backward in pieces, for schedules in which one block of queries meets several blocks of keys in turn (the
 * sequence-sharded ring): what sntl_attn_bwd does in one call, split at its three launches so that the parts that
 * depend only on the query block run once per block instead of once per pair.
 *   sntl_attn_bwd_begin   delta = rowsum(dO o O) and the rescaled LSE of the query block; its fp32 dQ accumulator
 *                         (inside `workspace`) zeroed.  desc: the query block (seq_kv / causal are not used).
 *   sntl_attn_bwd_block   one (query block, key block) pair with the query block's FINAL lse / delta: adds the
 *                         pair's dQ into the accumulator, and adds dK * scale and dV into the caller's fp32
 *                         dk_acc, dv_acc [B][kv_heads][seq_kv][D] (read-modify-write by one owner per element: no
 *                         atomics, deterministic given the call order).  desc: seq_q as in begin; seq_kv = the key
 *                         block; causal = 1 only for the diagonal pair (seq_q == seq_kv, same positions).
 *   sntl_attn_bwd_end     dq (bf16) = scale * accumulator.
 * `workspace` (sntl_attn_bwd_pieces_workspace_bytes, a function of batch, q_heads, seq_q, head_dim only) carries
 * delta, LSE and the accumulator from begin to end and belongs to that one query block meanwhile.  bf16 BHSD
 * tensors with head_dim 64 / 128 only (SNTL_ERR_UNSUPPORTED otherwise), no sliding window.  Asynchronous on
 * `stream`.  No counterpart in the reference (it has no sequence-parallel path; its backward is one call,
 * sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1615-1700). */
size_t sntl_attn_bwd_pieces_workspace_bytes(const sntl_attn_desc* desc);
int sntl_attn_bwd_begin(const sntl_attn_desc* desc, const void* o, const float* lse, const void* dout, void* workspace,
                        size_t workspace_bytes, void* stream);
int sntl_attn_bwd_block(const sntl_attn_desc* desc, const void* q, const void* k, const void* v, const void* dout,
                        float* dk_acc, float* dv_acc, void* workspace, size_t workspace_bytes, void* stream);
int sntl_attn_bwd_end(const sntl_attn_desc* desc, void* dq, void* workspace, size_t workspace_bytes, void* stream);

/* The same backward for callers that cannot allocate device memory and so cannot bring a workspace (a plugin
 * running inside another component's stream capture, a host that bans cudaMalloc in its hot loop, a binding with
 * no allocator to lend).  The scratch is a fixed array inside the library image, sntl_attn_static_scratch_capacity()
 * bytes (32 MiB) on every GPU that loads the library; a problem whose sntl_attn_bwd_workspace_bytes() exceeds it
 * returns SNTL_ERR_SCRATCH_LIMIT and launches nothing.  The first call on a device resolves the array's device
 * address and should be made before any stream capture.  All calls on a device share the array (each call rewrites
 * what it reads, so nothing needs clearing), hence calls that can overlap on one GPU race and must be ordered by
 * the caller.  Allocates nothing.  This entry point has no counterpart in the reference. */
int sntl_attn_bwd_static_scratch(const sntl_attn_desc* desc, const void* q, const void* k, const void* v, const void* o,
                                 const float* lse, const void* dout, void* dq, void* dk, void* dv, void* stream);

/* Size in bytes of the built-in scratch used by sntl_attn_bwd_static_scratch.  No counterpart in the reference. */
size_t sntl_attn_static_scratch_capacity(void);

/* Boundary conversions fused with the rotary embedding: one read and one write per element where the reference
 * makes separate passes (rotaryRotateInPlace / rotaryRotateInverseInPlace over fp32 matrices,
 * sentinel/NeuralNet/Cuda/CudaOps.cu:362-399, called
 * at CudaCausalSelfAttention.cu:206-207, :508-509) before its flash kernel converts operands on every load.
 *   pack:   src fp32 feature-major (heads*head_dim) x stride_columns, tokens of pack b at columns
 *           column_start + b*seq + s  ->  dst bf16 [batch][heads][seq][head_dim], rotated by the angle tables.
 *   unpack: the reverse relayout to fp32; inverse != 0 applies the inverse rotation (the gradients dQ, dK),
 *           inverse == 0 the forward one.
 * cos_table / sin_table: [table_positions][head_dim/2] fp32, entry [position][i] for the pair (2i, 2i+1)
 * (sentinel/NeuralNet/Layers/RotaryEmbedding.cpp:19-27); both null = no rotation (V, O, dV).  Token s of every pack sits at position
 * position_offset + s (packs restart at 0: CudaOps.cu:366).  Products and sums are rounded separately, as the
 * reference's host code computes them, so the result is the bf16 rounding of exactly that fp32 value.
 * Asynchronous on `stream`. */
int sntl_attn_pack_heads(const float* src, void* dst, int32_t batch, int32_t heads, int32_t seq, int32_t head_dim,
                         int32_t stride_columns, int32_t column_start, const float* cos_table, const float* sin_table,
                         int32_t position_offset, int32_t table_positions, void* stream);
int sntl_attn_unpack_heads(const void* src, float* dst, int32_t batch, int32_t heads, int32_t seq, int32_t head_dim,
                           int32_t stride_columns, int32_t column_start, const float* cos_table, const float* sin_table,
                           int32_t position_offset, int32_t table_positions, int32_t inverse, void* stream);

/* Log-sum-exp merge of two partial attention results over disjoint key sets (the ring schedule's
 * combine step): o_acc,lse_acc <- merge((o_acc,lse_acc),(o_part,lse_part)).  BHSD layout, `rows` =
 * B*Hq*Sq rows of head_dim elements; the accumulator and the partial may have different element types
 * (an fp32 accumulator keeps repeated merges from compounding bf16 rounding).  A side whose LSE is -inf
 * contributes nothing.  Asynchronous on `stream`.  No counterpart in the reference (it has no
 * sequence-parallel path). */
int sntl_attn_merge(int32_t acc_dtype, int32_t part_dtype, int64_t rows, int32_t head_dim, void* o_acc, float* lse_acc,
                    const void* o_part, const float* lse_part, void* stream);

/* acc[i] += part[i] for `count` elements, acc fp32, part bf16 or fp32: the ring schedule's running sums of the
 * dQ / dK / dV partials of successive key blocks.  Asynchronous on `stream`.  No counterpart in the reference. */
int sntl_attn_accumulate(int32_t part_dtype, int64_t count, float* acc, const void* part, void* stream);

/* ---- Sequence-sharded attention over a ring of GPUs (the long-context workload) ----
 * One process per GPU; rank r of `world` holds tokens [r*S/W, (r+1)*S/W) of ONE causal sequence: q, o, dout, dq
 * [B][q_heads][S/W][D], k, v, dk, dv [B][kv_heads][S/W][D], lse [B][q_heads][S/W], all bf16 BHSD (lse fp32),
 * head_dim 64 or 128, desc->seq_q = desc->seq_kv = S/W (even), desc->causal = 1.  The shards are dealt as half-shards in
 * a zigzag so that every rank has the same work under the causal mask; K/V half-shards travel round the ring with
 * grouped ncclSend / ncclRecv on the handle's own stream while the kernels of the current step run, and in the backward
 * fp32 dK/dV accumulators travel with them.  Results come back in the contiguous layout (with SNTL_FLAG_RING_ZIGZAG the
 * shards are taken and returned in the zigzag order itself and nothing is redistributed).  Every rank makes the same
 * calls in the same order.  All scratch comes from `workspace` (sntl_ring_attn_workspace_bytes; it must not be touched
 * between a forward and a backward that reuses its state); streams and events belong to the handle.
 *   sntl_ring_unique_id      rank 0 fills 128 bytes (an ncclUniqueId) that the host distributes to all ranks.
 *   sntl_ring_comm_create    collective: makes the rank's handle (ncclCommInitRank on the current device).
 *   sntl_ring_comm_adopt     the same around a communicator the host already has (an ncclComm_t; not destroyed with
 *                            the handle).
 *   sntl_ring_attn_bwd       reuse_forward_state != 0: q, k, v, o, lse are the tensors of the last sntl_ring_attn_fwd
 *                            through this workspace, whose dealt copies are still there (only dout is dealt).
 * NCCL is opened at run time (libnccl.so.2); SNTL_ERR_COMM when it is missing or a call fails.  A peer that stops
 * answering is NCCL's to detect (its own time-outs / ncclCommAbort by the host); the device-side waits of the kernels
 * stay bounded as everywhere.  No counterpart in the reference (it has no multi-GPU path at all). */
typedef struct sntl_ring_comm sntl_ring_comm;
int sntl_ring_unique_id(void* id128);
int sntl_ring_comm_create(const void* id128, int rank, int world, sntl_ring_comm** out);
int sntl_ring_comm_adopt(void* nccl_comm, int rank, int world, sntl_ring_comm** out);
int sntl_ring_comm_destroy(sntl_ring_comm* comm);
size_t sntl_ring_attn_workspace_bytes(const sntl_ring_comm* comm, const sntl_attn_desc* desc);
int sntl_ring_attn_fwd(sntl_ring_comm* comm, const sntl_attn_desc* desc, const void* q, const void* k, const void* v, void* o,
                       float* lse, void* workspace, size_t workspace_bytes, void* stream);
int sntl_ring_attn_bwd(sntl_ring_comm* comm, const sntl_attn_desc* desc, const void* q, const void* k, const void* v,
                       const void* o, const float* lse, const void* dout, void* dq, void* dk, void* dv,
                       int reuse_forward_state, void* workspace, size_t workspace_bytes, void* stream);

/* Name of the kernel family the most recent sntl_attn_fwd / sntl_attn_bwd call on this thread dispatched to
 * ("simt_f32", "tcgen05", ...), so a test can assert the path taken, like the reference's
 * usedFlashAttention flag (CudaCausalSelfAttention.hpp:36). */
const char* sntl_attn_last_path(void);

/* Number of kernels this library has launched from this process so far (all entry points). */
uint64_t sntl_attn_launch_count(void);

/* Reads (and clears) the device-side status word the tensor-core kernels write when one of their bounded
 * waits runs out.  Synchronises `stream`.  Returns SNTL_OK or SNTL_ERR_DEVICE_TIMEOUT; *detail (optional)
 * receives the raw word (which wait, which CTA). */
int sntl_attn_poll_device_status(void* stream, uint32_t* detail);

/* The same poll with the two words kept apart: the forward kernels (and the self-test below) report in one, the
 * backward kernels in the other.  Either pointer may be null.  No counterpart in the reference. */
int sntl_attn_poll_device_status_words(void* stream, uint32_t* forward_word, uint32_t* backward_word);

/* What a timeout means for the caller.  Every device-side wait of the tensor-core kernels is bounded (about one
 * second).  A wait that runs out records its site in the status word, the kernel unwinds and returns normally (no
 * trap; the context stays usable), and the tensors that call was writing hold garbage.  sntl_attn_fwd / _bwd have
 * long returned SNTL_OK by then: they are asynchronous.  The status word stays set until it is polled, and for one
 * wait limit after a give-up other waits on that GPU give up early too, so calls launched in that interval may be
 * cut short as well.  A caller therefore polls at the points where it synchronises anyway (end of a training step,
 * before reading results back) and discards the step on SNTL_ERR_DEVICE_TIMEOUT. */

/* Self-test of that path, for test suites: launches one warp whose only wait can never complete, limited to
 * limit_us microseconds (1..100000).  The wait runs out, the kernel returns, and the next poll reports
 * SNTL_ERR_DEVICE_TIMEOUT with site code 0x7e in the top byte of the forward word.  Nothing hangs or faults.
 * Asynchronous on `stream`.  No counterpart in the reference. */
int sntl_attn_selftest_wait_timeout(uint32_t limit_us, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* SNTL_ATTN_H */

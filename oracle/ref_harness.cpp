// ref_harness.cpp -- drives the UNMODIFIED reference CPU attention (compiled from the
// reference project's own sources, see oracle/Makefile) on caller-supplied Q/K/V/dO.
//
// THIS FILE IS TEST INFRASTRUCTURE (checker + timed CPU baseline); the shipped CUDA
// library never links or calls it.  It contains no reference code: it only includes the
// reference headers and calls public members.
//
// Two routes are exported:
//
//  ref_layer_fwd_bwd   goes through the reference's public layer API
//      CausalSelfAttention::forward / ::backward
//      (sentinel/NeuralNet/Layers/CausalSelfAttention.cpp:212-258, :260-368).
//      The layer is built with selector weights Wq=[I 0 0], Wk=[0 I 0], Wv=[0 0 I], Wo=I
//      over the stacked input [Q;K;V] and a RotaryEmbedding whose public cos/sin tables
//      are overwritten with 1/0, so the layer computes exactly the attention core.  dQ/dK/dV
//      are read from the public cache members queryGradient/keyGradient/valueGradient.
//      This is the parity pin for the fp64 restatement and for the fp32 CUDA path.
//
//  ref_core_fwd_bwd    issues the same per-head sequence of the reference's public
//      primitives (Matrix::gemm Matrix.cpp:106-148, Matrix::scaleInPlace,
//      Softmax::applyInto Softmax.cpp:10-44) that the layer's dense branch issues
//      (CausalSelfAttention.cpp:122-126, :150-152, :333-347), without the selector
//      projections.  Used for timing the CPU baseline (attention core only); a test checks
//      that it is bit-identical to the layer route.
//
// Layout at this boundary: token-major [B][H][S][D] fp32; the reference's own layout is
// feature-major (H*D) x S per sequence (row = h*D + d, column = token), one sequence per
// call, so the harness loops over B.
#include "NeuralNet/Activations/Softmax.hpp"
#include "NeuralNet/Layers/CausalSelfAttention.hpp"
#include "NeuralNet/Layers/RotaryEmbedding.hpp"
#include "NeuralNet/Math/Matrix.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstddef>
#include <cstring>
#include <limits>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

namespace {

double now_s()
{
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// [H][S][D] slab (one batch element) -> feature-major rows [rowOffset + h*D + d][s]
void gather_rows(const float* bhsd, int H, int S, int D, Matrix& dst, size_t rowOffset)
{
    for (int h = 0; h < H; ++h)
        for (int s = 0; s < S; ++s)
            for (int d = 0; d < D; ++d)
                dst.at(rowOffset + (size_t)h * D + d, (size_t)s) = bhsd[((size_t)h * S + s) * D + d];
}

void scatter_rows(const Matrix& src, size_t rowOffset, int H, int S, int D, float* bhsd)
{
    for (int h = 0; h < H; ++h)
        for (int s = 0; s < S; ++s)
            for (int d = 0; d < D; ++d)
                bhsd[((size_t)h * S + s) * D + d] = src.data[(rowOffset + (size_t)h * D + d) * src.cols + s];
}

// lse[query] = m + ln(sum_k exp(s_k - m)) over the masked, scaled scores[key][query] the layer
// cached; the definition follows sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1258-1265.
void lse_from_scores(const Matrix& scores, float* lse)
{
    const size_t n = scores.cols;
    for (size_t qi = 0; qi < n; ++qi) {
        float m = -std::numeric_limits<float>::infinity();
        for (size_t k = 0; k < scores.rows; ++k) m = std::max(m, scores.data[k * n + qi]);
        double l = 0.0;
        for (size_t k = 0; k < scores.rows; ++k) l += std::exp((double)scores.data[k * n + qi] - (double)m);
        lse[qi] = (float)((double)m + std::log(l));
    }
}

}  // namespace

extern "C" {

int ref_threads()
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Public-API route.  q,o,dout,dq: [B][Hq][S][D]; k,v,dk,dv: [B][Hkv][S][D]; lse: [B][Hq][S].
// dout/dq/dk/dv may be null (forward only).  Returns 0, or 1 when the reference threw.
// window <= 0: the whole sequence (plain causal).  With 0 < window < S the reference layer takes its sparse
// branch (CausalSelfAttention.cpp:102-107, :128-148, :154-168, :296-331), the same mask computed pairwise.
int ref_layer_fwd_bwd_windowed(int B, int Hq, int Hkv, int S, int D, int window, int global_tokens, const float* q,
                               const float* k, const float* v, const float* dout, float* o, float* lse, float* dq,
                               float* dk, float* dv)
{
    try {
        const size_t qRows = (size_t)Hq * D, kvRows = (size_t)Hkv * D, inRows = qRows + 2 * kvRows;
        Matrix wq(qRows, inRows, 0.0f), wk(kvRows, inRows, 0.0f), wv(kvRows, inRows, 0.0f), wo(qRows, qRows, 0.0f);
        for (size_t r = 0; r < qRows; ++r) { wq.at(r, r) = 1.0f; wo.at(r, r) = 1.0f; }
        for (size_t r = 0; r < kvRows; ++r) { wk.at(r, qRows + r) = 1.0f; wv.at(r, qRows + kvRows + r) = 1.0f; }
        RotaryEmbedding rope(D, S, RotaryEmbedding::DefaultBase);
        std::fill(rope.cosTable.begin(), rope.cosTable.end(), 1.0f);  // inputs arrive with RoPE already applied
        std::fill(rope.sinTable.begin(), rope.sinTable.end(), 0.0f);
        CausalSelfAttention layer(wq, wk, wv, wo, rope, Hq, /*windowSize=*/window > 0 ? window : S,
                                  /*globalTokenCount=*/global_tokens, Hkv);

        for (int b = 0; b < B; ++b) {
            Matrix input(inRows, (size_t)S, 0.0f);
            gather_rows(q + (size_t)b * Hq * S * D, Hq, S, D, input, 0);
            gather_rows(k + (size_t)b * Hkv * S * D, Hkv, S, D, input, qRows);
            gather_rows(v + (size_t)b * Hkv * S * D, Hkv, S, D, input, qRows + kvRows);
            CausalSelfAttentionCache cache;
            Matrix out = layer.forward(input, cache);
            scatter_rows(out, 0, Hq, S, D, o + (size_t)b * Hq * S * D);
            if (lse)
                for (int h = 0; h < Hq; ++h) lse_from_scores(cache.scores[(size_t)h], lse + ((size_t)b * Hq + h) * S);
            if (dout && dq && dk && dv) {
                Matrix grad(qRows, (size_t)S, 0.0f);
                gather_rows(dout + (size_t)b * Hq * S * D, Hq, S, D, grad, 0);
                Matrix gwq, gwk, gwv, gwo;
                layer.backward(grad, cache, gwq, gwk, gwv, gwo);
                scatter_rows(cache.queryGradient, 0, Hq, S, D, dq + (size_t)b * Hq * S * D);
                scatter_rows(cache.keyGradient, 0, Hkv, S, D, dk + (size_t)b * Hkv * S * D);
                scatter_rows(cache.valueGradient, 0, Hkv, S, D, dv + (size_t)b * Hkv * S * D);
            }
        }
        return 0;
    } catch (...) {
        return 1;
    }
}

int ref_layer_fwd_bwd(int B, int Hq, int Hkv, int S, int D, const float* q, const float* k, const float* v,
                      const float* dout, float* o, float* lse, float* dq, float* dk, float* dv)
{
    return ref_layer_fwd_bwd_windowed(B, Hq, Hkv, S, D, 0, 0, q, k, v, dout, o, lse, dq, dk, dv);
}

// The reference's RotaryEmbedding on a feature-major (heads*D) x cols matrix, in place (forward or inverse rotation),
// and its angle tables ([positions][D/2]; pass null to skip).  Returns 0, or 1 when the reference threw.
int ref_rope(int D, int positions, float base, int heads, int cols, float* tensor, int inverse, float* cos_out, float* sin_out)
{
    try {
        RotaryEmbedding rope(D, positions, base);
        if (cos_out) std::memcpy(cos_out, rope.cosTable.data(), rope.cosTable.size() * sizeof(float));
        if (sin_out) std::memcpy(sin_out, rope.sinTable.data(), rope.sinTable.size() * sizeof(float));
        if (tensor) {
            Matrix m((size_t)heads * D, (size_t)cols, 0.0f);
            std::memcpy(m.data.data(), tensor, m.data.size() * sizeof(float));
            if (inverse) rope.rotateInverseInPlace(m, heads);
            else rope.rotateInPlace(m, heads);
            std::memcpy(tensor, m.data.data(), m.data.size() * sizeof(float));
        }
        return 0;
    } catch (...) {
        return 1;
    }
}

// The public layer route with the layer's own rotary embedding left in place (rope_base > 0): inputs are the
// un-rotated Q and K, the layer rotates them (CausalSelfAttention.cpp:232-236) and its backward applies the inverse
// rotation to dQ and dK (:355-356), so dq / dk come back with respect to the un-rotated inputs.
int ref_layer_fwd_bwd_rope(int B, int Hq, int Hkv, int S, int D, float rope_base, int window, int global_tokens, const float* q,
                           const float* k, const float* v, const float* dout, float* o, float* dq, float* dk, float* dv)
{
    try {
        const size_t qRows = (size_t)Hq * D, kvRows = (size_t)Hkv * D, inRows = qRows + 2 * kvRows;
        Matrix wq(qRows, inRows, 0.0f), wk(kvRows, inRows, 0.0f), wv(kvRows, inRows, 0.0f), wo(qRows, qRows, 0.0f);
        for (size_t r = 0; r < qRows; ++r) { wq.at(r, r) = 1.0f; wo.at(r, r) = 1.0f; }
        for (size_t r = 0; r < kvRows; ++r) { wk.at(r, qRows + r) = 1.0f; wv.at(r, qRows + kvRows + r) = 1.0f; }
        RotaryEmbedding rope(D, S, rope_base);
        CausalSelfAttention layer(wq, wk, wv, wo, rope, Hq, window > 0 ? window : S, global_tokens, Hkv);
        for (int b = 0; b < B; ++b) {
            Matrix input(inRows, (size_t)S, 0.0f);
            gather_rows(q + (size_t)b * Hq * S * D, Hq, S, D, input, 0);
            gather_rows(k + (size_t)b * Hkv * S * D, Hkv, S, D, input, qRows);
            gather_rows(v + (size_t)b * Hkv * S * D, Hkv, S, D, input, qRows + kvRows);
            CausalSelfAttentionCache cache;
            Matrix out = layer.forward(input, cache);
            scatter_rows(out, 0, Hq, S, D, o + (size_t)b * Hq * S * D);
            if (dout && dq && dk && dv) {
                Matrix grad(qRows, (size_t)S, 0.0f);
                gather_rows(dout + (size_t)b * Hq * S * D, Hq, S, D, grad, 0);
                Matrix gwq, gwk, gwv, gwo;
                Matrix inGrad = layer.backward(grad, cache, gwq, gwk, gwv, gwo);
                // with selector weights the input gradient is [dQ; dK; dV] with respect to the un-rotated inputs
                scatter_rows(inGrad, 0, Hq, S, D, dq + (size_t)b * Hq * S * D);
                scatter_rows(inGrad, qRows, Hkv, S, D, dk + (size_t)b * Hkv * S * D);
                scatter_rows(inGrad, qRows + kvRows, Hkv, S, D, dv + (size_t)b * Hkv * S * D);
            }
        }
        return 0;
    } catch (...) {
        return 1;
    }
}

// Primitive route (timed baseline).  Same tensors as above; all outputs optional except none --
// pass null to skip a store.  seconds[0] = forward time, seconds[1] = backward time (attention core only,
// layout gathers excluded).  head_limit > 0 restricts the run to the first head_limit query heads of
// each batch element (bounded sample for the bench); dk/dv then hold only those heads' contributions.
int ref_core_fwd_bwd(int B, int Hq, int Hkv, int S, int D, int head_limit, const float* q, const float* k,
                     const float* v, const float* dout, float* o, float* dq, float* dk, float* dv,
                     double* seconds)
{
    try {
        const int group = Hq / Hkv;
        const int heads = (head_limit > 0 && head_limit < Hq) ? head_limit : Hq;
        const float scale = 1.0f / std::sqrt((float)D);
        double tf = 0.0, tb = 0.0;
        Matrix qh((size_t)D, (size_t)S), kh((size_t)D, (size_t)S), vh((size_t)D, (size_t)S), gh((size_t)D, (size_t)S);
        Matrix scores, probs, attended, dvh, dprob, dscore, dqh, dkh;
        std::vector<float> dkAcc, dvAcc;
        for (int b = 0; b < B; ++b) {
            dkAcc.assign((size_t)Hkv * S * D, 0.0f);
            dvAcc.assign((size_t)Hkv * S * D, 0.0f);
            for (int h = 0; h < heads; ++h) {
                const int hk = h / group;
                gather_rows(q + ((size_t)b * Hq + h) * S * D, 1, S, D, qh, 0);
                gather_rows(k + ((size_t)b * Hkv + hk) * S * D, 1, S, D, kh, 0);
                gather_rows(v + ((size_t)b * Hkv + hk) * S * D, 1, S, D, vh, 0);
                double t0 = now_s();
                Matrix::gemm(kh, qh, scores, true, false);
                Matrix::scaleInPlace(scores, scale);
                for (int key = 0; key < S; ++key)
                    for (int query = 0; query < key; ++query) scores.at((size_t)key, (size_t)query) = -1e9f;
                Softmax::applyInto(scores, probs);
                Matrix::gemm(vh, probs, attended);
                tf += now_s() - t0;
                if (o) scatter_rows(attended, 0, 1, S, D, o + ((size_t)b * Hq + h) * S * D);
                if (!dout) continue;
                gather_rows(dout + ((size_t)b * Hq + h) * S * D, 1, S, D, gh, 0);
                t0 = now_s();
                Matrix::gemm(gh, probs, dvh, false, true);
                Matrix::gemm(vh, gh, dprob, true, false);
                dscore.ensureSize((size_t)S, (size_t)S);
                for (int query = 0; query < S; ++query) {
                    float dot = 0.0f;
                    for (int key = 0; key < S; ++key) dot += dprob.at((size_t)key, (size_t)query) * probs.at((size_t)key, (size_t)query);
                    for (int key = 0; key < S; ++key)
                        dscore.at((size_t)key, (size_t)query) =
                            probs.at((size_t)key, (size_t)query) * (dprob.at((size_t)key, (size_t)query) - dot);
                }
                for (int key = 0; key < S; ++key)
                    for (int query = 0; query < key; ++query) dscore.at((size_t)key, (size_t)query) = 0.0f;
                Matrix::scaleInPlace(dscore, scale);
                Matrix::gemm(kh, dscore, dqh);
                Matrix::gemm(qh, dscore, dkh, false, true);
                tb += now_s() - t0;
                if (dq) scatter_rows(dqh, 0, 1, S, D, dq + ((size_t)b * Hq + h) * S * D);
                for (int s = 0; s < S; ++s)
                    for (int d = 0; d < D; ++d) {
                        dkAcc[((size_t)hk * S + s) * D + d] += dkh.data[(size_t)d * S + s];
                        dvAcc[((size_t)hk * S + s) * D + d] += dvh.data[(size_t)d * S + s];
                    }
            }
            if (dk) std::memcpy(dk + (size_t)b * Hkv * S * D, dkAcc.data(), dkAcc.size() * sizeof(float));
            if (dv) std::memcpy(dv + (size_t)b * Hkv * S * D, dvAcc.data(), dvAcc.size() * sizeof(float));
        }
        if (seconds) { seconds[0] = tf; seconds[1] = tb; }
        return 0;
    } catch (...) {
        return 1;
    }
}

}  // extern "C"

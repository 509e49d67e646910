// ref_cuda_harness.cu -- drives the UNMODIFIED reference CUDA flash-attention kernels (compiled from the reference
// project's own sources for sm_100a, see oracle/Makefile) on caller-supplied tensors.
//
// THIS FILE IS TEST INFRASTRUCTURE: a GPU baseline and a second parity subject held to the same oracle as the
// product kernels.  It contains no reference code; it includes the reference headers and calls
// CudaFlashAttention::forwardMultiHead / backwardMultiHead (sentinel/NeuralNet/Cuda/CudaFlashAttention.hpp:30, :40)
// the way the reference's own call sites do (sentinel/NeuralNet/Cuda/CudaCausalSelfAttention.cu:237-249, :391-438):
// K/V repeated to the query head count by the caller, dK/dV zeroed before the backward call.
//
// Layout at this boundary is the reference's own: fp32 feature-major (H*D) x columns host arrays, packCount
// segments of `segment` columns starting at column 0.
#include "NeuralNet/Cuda/CudaFlashAttention.hpp"
#include "NeuralNet/Cuda/CudaMatmul.hpp"
#include "NeuralNet/Cuda/CudaOps.hpp"
#include "NeuralNet/Math/Matrix.hpp"

#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <exception>

namespace {
Matrix to_matrix(const float* data, size_t rows, size_t cols)
{
    Matrix m(rows, cols, 0.0f);
    std::memcpy(m.data.data(), data, rows * cols * sizeof(float));
    return m;
}
}  // namespace

extern "C" {

// Returns 0 on success, 1 when the reference threw (message in err).  ms[0] = forward, ms[1] = backward (delta + main
// kernel, dK/dV zeroing included as at the reference call site), each the mean of `reps` timed runs after one warm-up.
int ref_cuda_flash_fwd_bwd(int headCount, int headDimension, int columns, int segment, int packCount, const float* q,
                           const float* k, const float* v, const float* dout, float* out, float* lse, float* dq, float* dk,
                           float* dv, int reps, float* ms, char* err, int err_len)
{
    try {
        const size_t rows = (size_t)headCount * headDimension;
        const float scale = 1.0f / sqrtf((float)headDimension);
        CudaMatrix mq, mk, mv, mo, ml, mg, mdq, mdk, mdv, mdelta;
        mq.upload(to_matrix(q, rows, columns));
        mk.upload(to_matrix(k, rows, columns));
        mv.upload(to_matrix(v, rows, columns));
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        float t_fwd = 0.0f, t_bwd = 0.0f;
        for (int r = 0; r <= reps; ++r) {
            cudaEventRecord(e0, CudaMatmul::activeStream());
            CudaFlashAttention::forwardMultiHead(mq, mk, mv, mo, ml, headCount, headDimension, scale, true, 0, segment, packCount);
            cudaEventRecord(e1, CudaMatmul::activeStream());
            cudaEventSynchronize(e1);
            float t = 0.0f;
            cudaEventElapsedTime(&t, e0, e1);
            if (r > 0) t_fwd += t;
        }
        {
            Matrix h = mo.download();
            std::memcpy(out, h.data.data(), rows * columns * sizeof(float));
            Matrix hl = ml.download();
            std::memcpy(lse, hl.data.data(), (size_t)headCount * columns * sizeof(float));
        }
        if (dout) {
            mg.upload(to_matrix(dout, rows, columns));
            mdq.ensureSize(rows, columns);
            mdk.ensureSize(rows, columns);
            mdv.ensureSize(rows, columns);
            for (int r = 0; r <= reps; ++r) {
                cudaEventRecord(e0, CudaMatmul::activeStream());
                CudaOps::zeroInPlace(mdk);
                CudaOps::zeroInPlace(mdv);
                CudaFlashAttention::backwardMultiHead(mq, mk, mv, mo, ml, mg, mdq, mdk, mdv, mdelta, headCount, headDimension, scale,
                                                      true, 0, segment, packCount);
                cudaEventRecord(e1, CudaMatmul::activeStream());
                cudaEventSynchronize(e1);
                float t = 0.0f;
                cudaEventElapsedTime(&t, e0, e1);
                if (r > 0) t_bwd += t;
            }
            Matrix a = mdq.download(), b = mdk.download(), c = mdv.download();
            std::memcpy(dq, a.data.data(), rows * columns * sizeof(float));
            std::memcpy(dk, b.data.data(), rows * columns * sizeof(float));
            std::memcpy(dv, c.data.data(), rows * columns * sizeof(float));
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        if (ms) { ms[0] = t_fwd / (reps > 0 ? reps : 1); ms[1] = t_bwd / (reps > 0 ? reps : 1); }
        return 0;
    } catch (const std::exception& e) {
        if (err && err_len > 0) { strncpy(err, e.what(), (size_t)err_len - 1); err[err_len - 1] = 0; }
        return 1;
    }
}

}  // extern "C"

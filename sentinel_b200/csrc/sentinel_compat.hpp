// Host-side mirror of the reference's flash-attention operator interface, implemented on the C ABI.
//
// A Sentinel build links this translation unit in place of its own
// sentinel/NeuralNet/Cuda/CudaFlashAttention.cu: the class name, the four static methods, their argument
// order, defaults and meaning, and the exception types are those of
// sentinel/NeuralNet/Cuda/CudaFlashAttention.hpp:10-41, so CudaCausalSelfAttention.cu:237-249 and :421-438
// compile and behave unchanged and LanguageModel::enableCuda() / setCudaPreferFlashAttention keep working.
//
// Standing alone (as built here) the class needs a device matrix type; `CudaMatrix` below is a minimal
// stand-in with the members the operator touches (rows, cols, device pointer, grow-only ensureSize, upload /
// download), shaped after sentinel/NeuralNet/Cuda/CudaMatmul.hpp:100-171.  Inside a Sentinel build the real
// CudaMatrix is used instead (define SNTL_COMPAT_USE_SENTINEL_TYPES and include CudaMatmul.hpp first).
#pragma once

#include <cstddef>
#include <vector>

#include <cuda_runtime.h>

namespace sentinel_b200 {

#ifndef SNTL_COMPAT_USE_SENTINEL_TYPES
/// row-major fp32 device matrix, data[row * cols + col]; storage grows but never shrinks
class CudaMatrix {
public:
    size_t rows = 0;
    size_t cols = 0;

    CudaMatrix() = default;
    CudaMatrix(size_t rowCount, size_t columnCount);
    ~CudaMatrix();
    CudaMatrix(const CudaMatrix&) = delete;
    CudaMatrix& operator=(const CudaMatrix&) = delete;

    /// reshape; reallocates only when the element count exceeds the capacity (never inside a stream capture)
    void ensureSize(size_t rowCount, size_t columnCount);
    void upload(const float* host, size_t rowCount, size_t columnCount);
    void download(float* host) const;
    float* deviceData() { return this->data; }
    const float* deviceData() const { return this->data; }

private:
    float* data = nullptr;
    size_t capacity = 0;
};
#endif

/// tiled causal attention with online softmax on sm_100a; forward stores per-query log-sum-exp for backward.
/// multi-head tensors are (headCount * headDim) x strideColumns, logSumExp is headCount x strideColumns
class CudaFlashAttention {
public:
    static constexpr int queryTileSize = 128;
    static constexpr int keyTileSize = 128;
    static constexpr int maxHeadDimension = 128;   // reference: 64 (CudaFlashAttention.hpp:16)

    static void forward(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                        CudaMatrix& logSumExp, float scale, bool causal = true);

    /// columns [columnStart, columnStart + packCount*columnCount) of strideColumns-wide matrices; every pack is an
    /// independent sequence.  key/value may carry fewer heads than query (rows = kvHeads*headDimension, kvHeads
    /// dividing headCount): grouped-query attention without repeating K/V.
    /// windowSize / globalTokenCount (after the reference's arguments, default off) are the layer's sliding window and
    /// global tokens (CausalSelfAttention::allowsKey, CausalSelfAttention.cpp:95-100), which the reference's flash path
    /// refuses (CudaCausalSelfAttention.cu:50) and this one computes.
    static void forwardMultiHead(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                                 CudaMatrix& logSumExp, int headCount, int headDimension, float scale, bool causal = true,
                                 int columnStart = 0, int columnCount = 0, int packCount = 1, int windowSize = 0,
                                 int globalTokenCount = 0);

    static void backward(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, const CudaMatrix& out,
                         const CudaMatrix& logSumExp, const CudaMatrix& outGradient, CudaMatrix& queryGradient,
                         CudaMatrix& keyGradient, CudaMatrix& valueGradient, float scale, bool causal = true);

    /// deltaWorkspace is kept for signature compatibility and sized like the reference does
    /// (headCount x packCount*columnCount); the library's own scratch is a grow-only internal buffer.
    static void backwardMultiHead(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, const CudaMatrix& out,
                                  const CudaMatrix& logSumExp, const CudaMatrix& outGradient, CudaMatrix& queryGradient,
                                  CudaMatrix& keyGradient, CudaMatrix& valueGradient, CudaMatrix& deltaWorkspace, int headCount,
                                  int headDimension, float scale, bool causal = true, int columnStart = 0, int columnCount = 0,
                                  int packCount = 1, int windowSize = 0, int globalTokenCount = 0);

    /// stream all launches go to (the reference reads CudaMatmul::activeStream(), CudaMatmul.cu:498-500)
    static void setActiveStream(cudaStream_t stream);
    static cudaStream_t activeStream();

    /// fp32 matrices are computed exactly in fp32 unless this is set; then head dimensions 64/128 run on the
    /// tensor cores with bf16 operands (the reference's own flash kernel rounds operands to fp16)
    static void setAllowReducedPrecision(bool allow);

    /// "tcgen05", "tcgen05_staged", "simt_f32" ...: which kernel family the last call used
    static const char* lastPath();
};

}  // namespace sentinel_b200

// Host-side mirror of the reference's flash-attention operator interface, implemented on the C ABI.
//
// Two ways to build the accompanying sentinel_compat.cu:
//
//  * Inside a Sentinel build (-DSNTL_COMPAT_USE_SENTINEL_TYPES, include path = the reference's `sentinel/` folder):
//    the translation unit includes the reference's OWN header sentinel/NeuralNet/Cuda/CudaFlashAttention.hpp and
//    defines the four static methods that header declares (class `CudaFlashAttention` in the global namespace,
//    CudaFlashAttention.hpp:12-41) on the reference's own CudaMatrix (device pointer = buffer.deviceData,
//    CudaMatmul.hpp:10-13, :100-104) and launch stream (CudaMatmul::activeStream(), CudaMatmul.hpp:221).  It is
//    linked IN PLACE OF sentinel/NeuralNet/Cuda/CudaFlashAttention.cu; no other file of the reference changes, so
//    CudaCausalSelfAttention.cu:237-249 and :421-438 compile and behave unchanged and LanguageModel::enableCuda() /
//    setCudaPreferFlashAttention keep working.  The extras of this library that the reference's header has no slot
//    for are the free functions of namespace sentinel_b200 declared below.
//
//  * Standing alone (as built into libsntl_attn.so): the class lives in namespace sentinel_b200 and works on a
//    minimal stand-in `CudaMatrix` with the members the operator touches (rows, cols, device pointer, grow-only
//    ensureSize, upload / download), shaped after sentinel/NeuralNet/Cuda/CudaMatmul.hpp:100-171.  This is what the
//    unit tests drive through the extern "C" hooks at the end of sentinel_compat.cu.
#pragma once

#include <cstddef>
#include <vector>

#include <cuda_runtime.h>

#ifdef SNTL_COMPAT_USE_SENTINEL_TYPES

#include "NeuralNet/Cuda/CudaFlashAttention.hpp"

namespace sentinel_b200 {

/// fp32 matrices are computed exactly in fp32 unless this is set; then head dimensions 64/128 run on the tensor
/// cores with bf16 operands (the reference's own flash kernel rounds operands to fp16, CudaFlashAttention.cu:209-214).
/// The environment variable SNTL_ATTN_REDUCED_PRECISION=1 sets the initial value.
void setAllowReducedPrecision(bool allow);

/// "tcgen05_staged", "simt_f32" ...: which kernel family the last call on this thread used
const char* lastPath();

/// Synchronises the active stream and throws std::runtime_error if a bounded device-side wait ran out since the
/// last poll (see sntl_attn_poll_device_status); call it where the training step synchronises anyway.
void throwIfDeviceWaitTimedOut();

/// The same operators with the layer's sliding window and global tokens (CausalSelfAttention::allowsKey,
/// sentinel/NeuralNet/Layers/CausalSelfAttention.cpp:95-100), which the reference's flash path refuses
/// (CudaCausalSelfAttention.cu:50), and with grouped-query K/V (rows = kvHeads*headDimension).
void forwardMultiHeadWindowed(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                              CudaMatrix& logSumExp, int headCount, int headDimension, float scale, bool causal, int columnStart,
                              int columnCount, int packCount, int windowSize, int globalTokenCount);
void backwardMultiHeadWindowed(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, const CudaMatrix& out,
                               const CudaMatrix& logSumExp, const CudaMatrix& outGradient, CudaMatrix& queryGradient,
                               CudaMatrix& keyGradient, CudaMatrix& valueGradient, CudaMatrix& deltaWorkspace, int headCount,
                               int headDimension, float scale, bool causal, int columnStart, int columnCount, int packCount,
                               int windowSize, int globalTokenCount);

}  // namespace sentinel_b200

#else  // stand-alone build

namespace sentinel_b200 {

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
    /// copies to the host, then throws std::runtime_error if a device-side wait ran out since the last check
    void download(float* host) const;
    float* deviceData() { return this->data; }
    const float* deviceData() const { return this->data; }

private:
    float* data = nullptr;
    size_t capacity = 0;
};

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
    /// (headCount x packCount*columnCount); the library's own scratch is a grow-only internal buffer per
    /// (device, stream).
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

#endif

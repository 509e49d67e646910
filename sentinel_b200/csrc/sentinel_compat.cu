// Implementation of the reference-shaped operator class on top of the C ABI (see sentinel_compat.hpp), plus a
// few extern "C" hooks that let a test harness drive the C++ class with host arrays.
//
// Argument checks and their exception types follow validateMultiHeadShape / resolveColumnWindow and the two
// entry functions of the reference (sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1458-1471, :1533-1539,
// :1543-1556, :1615-1638): std::invalid_argument for shape and window errors, std::runtime_error for a
// missing device or a failed launch.
#include "sentinel_compat.hpp"

#include <stdexcept>
#include <string>

#include "sntl_attn.h"

namespace sentinel_b200 {

namespace {

cudaStream_t g_stream = nullptr;
bool g_allow_reduced = false;
void* g_workspace = nullptr;   // grow-only, like the reference's CudaDeviceBuffer::ensureCapacity (CudaMatmul.cu:119-136)
size_t g_workspace_bytes = 0;

void cuda_or_throw(cudaError_t e, const char* what)
{
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

void status_or_throw(int status, const char* op)
{
    if (status == SNTL_OK) return;
    const std::string msg = std::string(op) + " " + sntl_status_string(status);
    if (status == SNTL_ERR_BAD_ARGUMENT || status == SNTL_ERR_UNSUPPORTED) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

void* workspace(size_t bytes)
{
    if (bytes > g_workspace_bytes) {
        if (g_workspace) cuda_or_throw(cudaFree(g_workspace), "CudaFlashAttention workspace free");
        g_workspace = nullptr;
        g_workspace_bytes = 0;
        cuda_or_throw(cudaMalloc(&g_workspace, bytes), "CudaFlashAttention workspace alloc");
        g_workspace_bytes = bytes;
    }
    return g_workspace;
}

bool empty(const CudaMatrix& m) { return m.rows == 0 || m.cols == 0; }

// returns kv head count
int validate_shape(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, int headCount, int headDimension,
                   const char* op)
{
    if (empty(query) || empty(key) || empty(value)) throw std::invalid_argument(std::string(op) + " empty input");
    if (headCount <= 0 || headDimension <= 0) throw std::invalid_argument(std::string(op) + " invalid head geometry");
    if (query.rows != (size_t)headCount * (size_t)headDimension)
        throw std::invalid_argument(std::string(op) + " query rows mismatch headCount*headDim");
    if (key.rows != value.rows || key.rows == 0 || key.rows % (size_t)headDimension != 0)
        throw std::invalid_argument(std::string(op) + " key/value rows mismatch");
    const int kvHeads = (int)(key.rows / (size_t)headDimension);
    if (kvHeads > headCount || headCount % kvHeads != 0)
        throw std::invalid_argument(std::string(op) + " key/value rows mismatch");
    if (query.cols != key.cols || query.cols != value.cols) throw std::invalid_argument(std::string(op) + " sequenceLength mismatch");
    return kvHeads;
}

void resolve_window(const CudaMatrix& query, int& columnStart, int& columnCount)
{
    const int strideColumns = (int)query.cols;
    if (columnCount <= 0) columnCount = strideColumns - columnStart;
    if (columnStart < 0 || columnCount <= 0 || columnStart + columnCount > strideColumns)
        throw std::invalid_argument("CudaFlashAttention invalid column window");
}

bool device_available()
{
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
}

sntl_attn_desc make_desc(const CudaMatrix& query, int headCount, int kvHeads, int headDimension, float scale, bool causal,
                         int columnStart, int columnCount, int packCount, int windowSize, int globalTokenCount)
{
    sntl_attn_desc d{};
    d.window_size = windowSize;
    d.global_tokens = globalTokenCount;
    d.dtype = SNTL_DTYPE_F32;
    d.layout = SNTL_LAYOUT_SENTINEL;
    d.batch = packCount;
    d.q_heads = headCount;
    d.kv_heads = kvHeads;
    d.seq_q = columnCount;
    d.seq_kv = columnCount;
    d.head_dim = headDimension;
    d.scale = scale;
    d.causal = causal ? 1 : 0;
    d.stride_columns = (int)query.cols;
    d.column_start = columnStart;
    d.flags = g_allow_reduced ? SNTL_FLAG_ALLOW_BF16_COMPUTE : 0;
    return d;
}

}  // namespace

#ifndef SNTL_COMPAT_USE_SENTINEL_TYPES
CudaMatrix::CudaMatrix(size_t rowCount, size_t columnCount) { this->ensureSize(rowCount, columnCount); }

CudaMatrix::~CudaMatrix()
{
    if (this->data) cudaFree(this->data);
}

void CudaMatrix::ensureSize(size_t rowCount, size_t columnCount)
{
    const size_t n = rowCount * columnCount;
    if (n > this->capacity) {
        if (this->data) cuda_or_throw(cudaFree(this->data), "CudaMatrix free");
        this->data = nullptr;
        this->capacity = 0;
        cuda_or_throw(cudaMalloc((void**)&this->data, n * sizeof(float)), "CudaMatrix alloc");
        this->capacity = n;
    }
    this->rows = rowCount;
    this->cols = columnCount;
}

void CudaMatrix::upload(const float* host, size_t rowCount, size_t columnCount)
{
    this->ensureSize(rowCount, columnCount);
    cuda_or_throw(cudaMemcpyAsync(this->data, host, rowCount * columnCount * sizeof(float), cudaMemcpyHostToDevice, g_stream),
                  "CudaMatrix upload");
    cuda_or_throw(cudaStreamSynchronize(g_stream), "CudaMatrix upload sync");
}

void CudaMatrix::download(float* host) const
{
    cuda_or_throw(cudaMemcpyAsync(host, this->data, this->rows * this->cols * sizeof(float), cudaMemcpyDeviceToHost, g_stream),
                  "CudaMatrix download");
    cuda_or_throw(cudaStreamSynchronize(g_stream), "CudaMatrix download sync");
}
#endif

void CudaFlashAttention::setActiveStream(cudaStream_t stream) { g_stream = stream; }
cudaStream_t CudaFlashAttention::activeStream() { return g_stream; }
void CudaFlashAttention::setAllowReducedPrecision(bool allow) { g_allow_reduced = allow; }
const char* CudaFlashAttention::lastPath() { return sntl_attn_last_path(); }

void CudaFlashAttention::forwardMultiHead(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                                          CudaMatrix& logSumExp, int headCount, int headDimension, float scale, bool causal,
                                          int columnStart, int columnCount, int packCount, int windowSize, int globalTokenCount)
{
    const char* op = "CudaFlashAttention::forwardMultiHead";
    const int kvHeads = validate_shape(query, key, value, headCount, headDimension, op);
    if (headDimension > 256)  // tensor-core kernels stop at maxHeadDimension; the exact-fp32 kernels at 256
        throw std::invalid_argument(std::string(op) + " headDim exceeds maxHeadDimension");
    if (!device_available()) throw std::runtime_error(std::string(op) + " no CUDA device");
    if (packCount <= 0) packCount = 1;
    if (globalTokenCount < 0) throw std::invalid_argument(std::string(op) + " globalTokenCount must be >= 0");
    if ((windowSize > 0 || globalTokenCount > 0) && !causal)
        throw std::invalid_argument(std::string(op) + " a sliding window needs the causal mask");
    resolve_window(query, columnStart, columnCount);
    if (columnStart + packCount * columnCount > (int)query.cols) throw std::invalid_argument(std::string(op) + " pack window exceeds columns");

    out.ensureSize(query.rows, query.cols);
    logSumExp.ensureSize((size_t)headCount, query.cols);
    const sntl_attn_desc d = make_desc(query, headCount, kvHeads, headDimension, scale, causal, columnStart, columnCount, packCount,
                                       windowSize, globalTokenCount);
    const size_t ws = sntl_attn_fwd_workspace_bytes(&d);
    void* wsp = ws ? workspace(ws) : nullptr;
    status_or_throw(sntl_attn_fwd(&d, query.deviceData(), key.deviceData(), value.deviceData(), out.deviceData(),
                                  logSumExp.deviceData(), wsp, ws, g_stream),
                    op);
}

void CudaFlashAttention::forward(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                                 CudaMatrix& logSumExp, float scale, bool causal)
{
    forwardMultiHead(query, key, value, out, logSumExp, 1, (int)query.rows, scale, causal, 0, (int)query.cols);
}

void CudaFlashAttention::backwardMultiHead(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value,
                                           const CudaMatrix& out, const CudaMatrix& logSumExp, const CudaMatrix& outGradient,
                                           CudaMatrix& queryGradient, CudaMatrix& keyGradient, CudaMatrix& valueGradient,
                                           CudaMatrix& deltaWorkspace, int headCount, int headDimension, float scale, bool causal,
                                           int columnStart, int columnCount, int packCount, int windowSize,
                                           int globalTokenCount)
{
    const char* op = "CudaFlashAttention::backwardMultiHead";
    const int kvHeads = validate_shape(query, key, value, headCount, headDimension, op);
    if (out.rows != query.rows || out.cols != query.cols) throw std::invalid_argument(std::string(op) + " out shape mismatch");
    if (outGradient.rows != query.rows || outGradient.cols != query.cols)
        throw std::invalid_argument(std::string(op) + " outGradient shape mismatch");
    if (logSumExp.rows != (size_t)headCount || logSumExp.cols != query.cols)
        throw std::invalid_argument(std::string(op) + " logSumExp shape mismatch");
    if (!device_available()) throw std::runtime_error(std::string(op) + " no CUDA device");
    if (packCount <= 0) packCount = 1;
    if (globalTokenCount < 0) throw std::invalid_argument(std::string(op) + " globalTokenCount must be >= 0");
    if ((windowSize > 0 || globalTokenCount > 0) && !causal)
        throw std::invalid_argument(std::string(op) + " a sliding window needs the causal mask");
    resolve_window(query, columnStart, columnCount);
    if (columnStart + packCount * columnCount > (int)query.cols) throw std::invalid_argument(std::string(op) + " pack window exceeds columns");

    queryGradient.ensureSize(query.rows, query.cols);
    keyGradient.ensureSize(key.rows, key.cols);
    valueGradient.ensureSize(value.rows, value.cols);
    deltaWorkspace.ensureSize((size_t)headCount, (size_t)packCount * (size_t)columnCount);
    const sntl_attn_desc d = make_desc(query, headCount, kvHeads, headDimension, scale, causal, columnStart, columnCount, packCount,
                                       windowSize, globalTokenCount);
    const size_t ws = sntl_attn_bwd_workspace_bytes(&d);
    status_or_throw(sntl_attn_bwd(&d, query.deviceData(), key.deviceData(), value.deviceData(), out.deviceData(),
                                  logSumExp.deviceData(), outGradient.deviceData(), queryGradient.deviceData(),
                                  keyGradient.deviceData(), valueGradient.deviceData(), workspace(ws), ws, g_stream),
                    op);
}

void CudaFlashAttention::backward(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, const CudaMatrix& out,
                                  const CudaMatrix& logSumExp, const CudaMatrix& outGradient, CudaMatrix& queryGradient,
                                  CudaMatrix& keyGradient, CudaMatrix& valueGradient, float scale, bool causal)
{
    CudaMatrix deltaWorkspace;
    backwardMultiHead(query, key, value, out, logSumExp, outGradient, queryGradient, keyGradient, valueGradient, deltaWorkspace, 1,
                      (int)query.rows, scale, causal, 0, (int)query.cols);
}

}  // namespace sentinel_b200

// ---- test hooks: drive the C++ operator class with host arrays in the reference's feature-major layout ----
// Return 0 on success, 1 for std::invalid_argument, 2 for any other exception (message copied to err).
using sentinel_b200::CudaFlashAttention;
using sentinel_b200::CudaMatrix;

namespace {
void copy_err(char* err, size_t n, const char* what)
{
    if (!err || n == 0) return;
    size_t i = 0;
    for (; i + 1 < n && what[i]; ++i) err[i] = what[i];
    err[i] = 0;
}
}  // namespace

extern "C" {

int sntl_compat_forward_backward_windowed(const float* q, const float* k, const float* v, const float* dout, int headCount,
                                          int kvHeads, int headDimension, int strideColumns, float scale, int causal,
                                          int columnStart, int columnCount, int packCount, int windowSize, int globalTokenCount,
                                          int allowReduced, float* out, float* lse, float* dq, float* dk, float* dv, char* path,
                                          size_t path_len, char* err, size_t err_len)
{
    try {
        CudaFlashAttention::setAllowReducedPrecision(allowReduced != 0);
        CudaMatrix mq, mk, mv, mo, ml, mg, mdq, mdk, mdv, mdelta;
        const size_t qRows = (size_t)headCount * headDimension, kvRows = (size_t)kvHeads * headDimension;
        mq.upload(q, qRows, (size_t)strideColumns);
        mk.upload(k, kvRows, (size_t)strideColumns);
        mv.upload(v, kvRows, (size_t)strideColumns);
        // outputs start from a recognisable fill so columns outside the window can be checked for being untouched
        std::vector<float> fill(qRows * (size_t)strideColumns, -777.0f);
        mo.upload(fill.data(), qRows, (size_t)strideColumns);
        ml.upload(fill.data(), (size_t)headCount, (size_t)strideColumns);
        CudaFlashAttention::forwardMultiHead(mq, mk, mv, mo, ml, headCount, headDimension, scale, causal != 0, columnStart, columnCount,
                                             packCount, windowSize, globalTokenCount);
        copy_err(path, path_len, CudaFlashAttention::lastPath());
        mo.download(out);
        ml.download(lse);
        if (dout) {
            mg.upload(dout, qRows, (size_t)strideColumns);
            mdq.upload(fill.data(), qRows, (size_t)strideColumns);
            mdk.upload(fill.data(), kvRows, (size_t)strideColumns);
            mdv.upload(fill.data(), kvRows, (size_t)strideColumns);
            CudaFlashAttention::backwardMultiHead(mq, mk, mv, mo, ml, mg, mdq, mdk, mdv, mdelta, headCount, headDimension, scale,
                                                  causal != 0, columnStart, columnCount, packCount, windowSize, globalTokenCount);
            mdq.download(dq);
            mdk.download(dk);
            mdv.download(dv);
        }
        return 0;
    } catch (const std::invalid_argument& e) {
        copy_err(err, err_len, e.what());
        return 1;
    } catch (const std::exception& e) {
        copy_err(err, err_len, e.what());
        return 2;
    }
}

int sntl_compat_forward_backward(const float* q, const float* k, const float* v, const float* dout, int headCount, int kvHeads,
                                 int headDimension, int strideColumns, float scale, int causal, int columnStart, int columnCount,
                                 int packCount, int allowReduced, float* out, float* lse, float* dq, float* dk, float* dv,
                                 char* path, size_t path_len, char* err, size_t err_len)
{
    return sntl_compat_forward_backward_windowed(q, k, v, dout, headCount, kvHeads, headDimension, strideColumns, scale, causal,
                                                 columnStart, columnCount, packCount, 0, 0, allowReduced, out, lse, dq, dk, dv, path,
                                                 path_len, err, err_len);
}

// argument-check probe that needs no device work: runs the shape/window validation only
int sntl_compat_validate(int qRows, int kvRows, int cols, int headCount, int headDimension, int columnStart, int columnCount,
                         int packCount, char* err, size_t err_len)
{
    try {
        if (qRows <= 0 || kvRows <= 0 || cols <= 0) throw std::invalid_argument("CudaFlashAttention::forwardMultiHead empty input");
        if (headCount <= 0 || headDimension <= 0) throw std::invalid_argument("CudaFlashAttention::forwardMultiHead invalid head geometry");
        if (qRows != headCount * headDimension) throw std::invalid_argument("CudaFlashAttention::forwardMultiHead query rows mismatch headCount*headDim");
        if (kvRows % headDimension != 0 || headCount % (kvRows / headDimension) != 0)
            throw std::invalid_argument("CudaFlashAttention::forwardMultiHead key/value rows mismatch");
        if (packCount <= 0) packCount = 1;
        if (columnCount <= 0) columnCount = cols - columnStart;
        if (columnStart < 0 || columnCount <= 0 || columnStart + columnCount > cols)
            throw std::invalid_argument("CudaFlashAttention invalid column window");
        if (columnStart + packCount * columnCount > cols)
            throw std::invalid_argument("CudaFlashAttention::forwardMultiHead pack window exceeds columns");
        return 0;
    } catch (const std::invalid_argument& e) {
        copy_err(err, err_len, e.what());
        return 1;
    }
}

}  // extern "C"

// Implementation of the reference-shaped operator class on top of the C ABI (see sentinel_compat.hpp), plus a
// few extern "C" hooks that let a test harness drive the C++ class with host arrays.
//
// Argument checks and their exception types follow validateMultiHeadShape / resolveColumnWindow and the two
// entry functions of the reference (sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1458-1471, :1533-1539,
// :1543-1556, :1615-1638): std::invalid_argument for shape and window errors, std::runtime_error for a
// missing device or a failed launch.
#include "sentinel_compat.hpp"

#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>

#include "sntl_attn.h"

namespace sentinel_b200 {

namespace {

#ifdef SNTL_COMPAT_USE_SENTINEL_TYPES
// inside a Sentinel build: the reference's own matrix type and its process-global launch stream
using Matrix_t = ::CudaMatrix;
inline const float* dev(const Matrix_t& m) { return m.buffer.deviceData; }
inline float* dev(Matrix_t& m) { return m.buffer.deviceData; }
inline cudaStream_t launch_stream() { return CudaMatmul::activeStream(); }
bool g_allow_reduced = [] {
    const char* e = std::getenv("SNTL_ATTN_REDUCED_PRECISION");
    return e && e[0] == '1';
}();
#else
using Matrix_t = CudaMatrix;
cudaStream_t g_stream = nullptr;
inline const float* dev(const Matrix_t& m) { return m.deviceData(); }
inline float* dev(Matrix_t& m) { return m.deviceData(); }
inline cudaStream_t launch_stream() { return g_stream; }
bool g_allow_reduced = false;
#endif

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

// Scratch for the C ABI calls: one grow-only buffer per (device ordinal, stream), like the reference's
// CudaDeviceBuffer::ensureCapacity (CudaMatmul.cu:119-136).  Calls on different devices or streams never share a
// buffer, so they neither race on it nor hand one GPU another GPU's memory; the map itself is guarded by a mutex.
// A buffer is only ever replaced by a larger one when its own (device, stream) asks for more, which -- as with
// every grow-only buffer of the reference -- must not happen while earlier work of that stream still uses it or
// inside a stream capture: sizes are stable after the first step, which the trainer runs eagerly
// (CudaLanguageModel.cu:761-793).  The map is never destroyed: at process exit the context is already gone.
struct Scratch {
#ifdef SNTL_COMPAT_USE_SENTINEL_TYPES
    CudaDeviceBuffer buffer;   // the reference's buffer type: its free() keeps CudaAmp's half caches coherent (CudaMatmul.cu:169)
    void* grow(size_t bytes)
    {
        this->buffer.ensureCapacity(bytes);
        return this->buffer.deviceData;
    }
#else
    void* data = nullptr;
    size_t capacity = 0;
    void* grow(size_t bytes)
    {
        if (bytes > this->capacity) {
            if (this->data) cuda_or_throw(cudaFree(this->data), "CudaFlashAttention workspace free");
            this->data = nullptr;
            this->capacity = 0;
            cuda_or_throw(cudaMalloc(&this->data, bytes), "CudaFlashAttention workspace alloc");
            this->capacity = bytes;
        }
        return this->data;
    }
#endif
};

void* workspace(size_t bytes, cudaStream_t stream)
{
    static std::mutex* guard = new std::mutex;
    static auto* buffers = new std::map<std::pair<int, cudaStream_t>, Scratch>;
    int device = 0;
    cuda_or_throw(cudaGetDevice(&device), "CudaFlashAttention workspace device");
    std::lock_guard<std::mutex> lock(*guard);
    return (*buffers)[std::make_pair(device, stream)].grow(bytes);
}

bool empty(const Matrix_t& m) { return m.rows == 0 || m.cols == 0; }

// returns kv head count
int validate_shape(const Matrix_t& query, const Matrix_t& key, const Matrix_t& value, int headCount, int headDimension,
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

void resolve_window(const Matrix_t& query, int& columnStart, int& columnCount)
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

sntl_attn_desc make_desc(const Matrix_t& query, int headCount, int kvHeads, int headDimension, float scale, bool causal,
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

void forward_impl(const Matrix_t& query, const Matrix_t& key, const Matrix_t& value, Matrix_t& out, Matrix_t& logSumExp,
                  int headCount, int headDimension, float scale, bool causal, int columnStart, int columnCount, int packCount,
                  int windowSize, int globalTokenCount)
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
    const cudaStream_t stream = launch_stream();
    const size_t ws = sntl_attn_fwd_workspace_bytes(&d);
    void* wsp = ws ? workspace(ws, stream) : nullptr;
    status_or_throw(sntl_attn_fwd(&d, dev(query), dev(key), dev(value), dev(out), dev(logSumExp), wsp, ws, stream), op);
}

void backward_impl(const Matrix_t& query, const Matrix_t& key, const Matrix_t& value, const Matrix_t& out, const Matrix_t& logSumExp,
                   const Matrix_t& outGradient, Matrix_t& queryGradient, Matrix_t& keyGradient, Matrix_t& valueGradient,
                   Matrix_t& deltaWorkspace, int headCount, int headDimension, float scale, bool causal, int columnStart,
                   int columnCount, int packCount, int windowSize, int globalTokenCount)
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
    const cudaStream_t stream = launch_stream();
    const size_t ws = sntl_attn_bwd_workspace_bytes(&d);
    status_or_throw(sntl_attn_bwd(&d, dev(query), dev(key), dev(value), dev(out), dev(logSumExp), dev(outGradient), dev(queryGradient),
                                  dev(keyGradient), dev(valueGradient), workspace(ws, stream), ws, stream),
                    op);
}

void throw_if_device_wait_timed_out(cudaStream_t stream)
{
    uint32_t fwd = 0, bwd = 0;
    const int rc = sntl_attn_poll_device_status_words(stream, &fwd, &bwd);
    if (rc == SNTL_OK) return;
    char words[64];
    snprintf(words, sizeof(words), " (forward 0x%08x, backward 0x%08x)", fwd, bwd);
    throw std::runtime_error(std::string("CudaFlashAttention ") + sntl_status_string(rc) + words);
}

}  // namespace

#ifdef SNTL_COMPAT_USE_SENTINEL_TYPES

void setAllowReducedPrecision(bool allow) { g_allow_reduced = allow; }
const char* lastPath() { return sntl_attn_last_path(); }
void throwIfDeviceWaitTimedOut() { throw_if_device_wait_timed_out(launch_stream()); }

void forwardMultiHeadWindowed(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                              CudaMatrix& logSumExp, int headCount, int headDimension, float scale, bool causal, int columnStart,
                              int columnCount, int packCount, int windowSize, int globalTokenCount)
{
    forward_impl(query, key, value, out, logSumExp, headCount, headDimension, scale, causal, columnStart, columnCount, packCount,
                 windowSize, globalTokenCount);
}

void backwardMultiHeadWindowed(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, const CudaMatrix& out,
                               const CudaMatrix& logSumExp, const CudaMatrix& outGradient, CudaMatrix& queryGradient,
                               CudaMatrix& keyGradient, CudaMatrix& valueGradient, CudaMatrix& deltaWorkspace, int headCount,
                               int headDimension, float scale, bool causal, int columnStart, int columnCount, int packCount,
                               int windowSize, int globalTokenCount)
{
    backward_impl(query, key, value, out, logSumExp, outGradient, queryGradient, keyGradient, valueGradient, deltaWorkspace, headCount,
                  headDimension, scale, causal, columnStart, columnCount, packCount, windowSize, globalTokenCount);
}

}  // namespace sentinel_b200

// ---- the reference's class, as declared by its own header (sentinel/NeuralNet/Cuda/CudaFlashAttention.hpp:12-41) ----

void CudaFlashAttention::forwardMultiHead(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                                          CudaMatrix& logSumExp, int headCount, int headDimension, float scale, bool causal,
                                          int columnStart, int columnCount, int packCount)
{
    sentinel_b200::forwardMultiHeadWindowed(query, key, value, out, logSumExp, headCount, headDimension, scale, causal, columnStart,
                                            columnCount, packCount, 0, 0);
}

void CudaFlashAttention::forward(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                                 CudaMatrix& logSumExp, float scale, bool causal)
{
    CudaFlashAttention::forwardMultiHead(query, key, value, out, logSumExp, 1, (int)query.rows, scale, causal, 0, (int)query.cols);
}

void CudaFlashAttention::backwardMultiHead(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value,
                                           const CudaMatrix& out, const CudaMatrix& logSumExp, const CudaMatrix& outGradient,
                                           CudaMatrix& queryGradient, CudaMatrix& keyGradient, CudaMatrix& valueGradient,
                                           CudaMatrix& deltaWorkspace, int headCount, int headDimension, float scale, bool causal,
                                           int columnStart, int columnCount, int packCount)
{
    sentinel_b200::backwardMultiHeadWindowed(query, key, value, out, logSumExp, outGradient, queryGradient, keyGradient, valueGradient,
                                             deltaWorkspace, headCount, headDimension, scale, causal, columnStart, columnCount,
                                             packCount, 0, 0);
}

void CudaFlashAttention::backward(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, const CudaMatrix& out,
                                  const CudaMatrix& logSumExp, const CudaMatrix& outGradient, CudaMatrix& queryGradient,
                                  CudaMatrix& keyGradient, CudaMatrix& valueGradient, float scale, bool causal)
{
    CudaMatrix deltaWorkspace;
    CudaFlashAttention::backwardMultiHead(query, key, value, out, logSumExp, outGradient, queryGradient, keyGradient, valueGradient,
                                          deltaWorkspace, 1, (int)query.rows, scale, causal, 0, (int)query.cols);
}

#else  // stand-alone build: own matrix type, class in namespace sentinel_b200, test hooks

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
    throw_if_device_wait_timed_out(g_stream);   // this is a synchronisation point: a timed-out wait surfaces here
}

void CudaFlashAttention::setActiveStream(cudaStream_t stream) { g_stream = stream; }
cudaStream_t CudaFlashAttention::activeStream() { return g_stream; }
void CudaFlashAttention::setAllowReducedPrecision(bool allow) { g_allow_reduced = allow; }
const char* CudaFlashAttention::lastPath() { return sntl_attn_last_path(); }

void CudaFlashAttention::forwardMultiHead(const CudaMatrix& query, const CudaMatrix& key, const CudaMatrix& value, CudaMatrix& out,
                                          CudaMatrix& logSumExp, int headCount, int headDimension, float scale, bool causal,
                                          int columnStart, int columnCount, int packCount, int windowSize, int globalTokenCount)
{
    forward_impl(query, key, value, out, logSumExp, headCount, headDimension, scale, causal, columnStart, columnCount, packCount,
                 windowSize, globalTokenCount);
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
    backward_impl(query, key, value, out, logSumExp, outGradient, queryGradient, keyGradient, valueGradient, deltaWorkspace, headCount,
                  headDimension, scale, causal, columnStart, columnCount, packCount, windowSize, globalTokenCount);
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

#endif  // stand-alone build

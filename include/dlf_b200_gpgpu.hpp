// dlf_b200_gpgpu.hpp - C++ host side of the backend: the reference's template API for this path,
// implemented over the C ABI of dlf_b200.h.
//
// Namespace dlf_b200::gpgpu holds
//   * a small CUDA-runtime rendition of the plumbing types the reference's API is written
//     against - Buffer<T> (gpgpu/include/gpgpu.h:639-698), Queue (:593-623), Event (:625-637),
//     TemporaryBuffer<T> (:710-746) - so that this header can be built and tested on its own, and
//   * blas::gemm / blas::gemmBatched / blas::gemmStridedBatched and dnn::conv2d with the
//     reference's exact signatures (gpgpu/include/gblas.h:496-504, 661-683; gdnn.h:201-213).
// Inside dlf itself the same four function bodies go where the CUBLAS(...) lambdas and cudnnConv
// sit today; only the two `unwrap` helpers change.
//
// Error behaviour follows the reference: argument errors throw BLASError carrying the StatusCode
// (gpgpu/src/utilities/exceptions.hpp:24-35), CUDA failures throw APIError (gpgpu.h:21-121).
// Buffer sizes are validated here (TestMatrixA/B/C, gpgpu/src/utilities/buffer_test.hpp:24-55)
// because only the Buffer knows its size.
#ifndef DLF_B200_GPGPU_HPP_
#define DLF_B200_GPGPU_HPP_

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "dlf_b200.h"

namespace dlf_b200 {
namespace gpgpu {

class APIError : public std::runtime_error {
public:
    APIError(int status, const std::string& where)
        : std::runtime_error(where + ": " + dlf_b200_status_string(status)), status_(status) {}
    int status() const noexcept { return status_; }
private:
    int status_;
};

inline void check_cuda(cudaError_t e, const char* where) {
    if (e != cudaSuccess) throw APIError(static_cast<int>(e), where);
}

// ---------------------------------------------------------------------------- Queue / Event
class Event {
public:
    Event() {
        check_cuda(cudaEventCreate(&start_), "cudaEventCreate");
        check_cuda(cudaEventCreate(&end_), "cudaEventCreate");
    }
    ~Event() { cudaEventDestroy(start_); cudaEventDestroy(end_); }
    Event(const Event&) = delete;
    Event& operator=(const Event&) = delete;
    void waitForCompletion() const { check_cuda(cudaEventSynchronize(end_), "cudaEventSynchronize"); }
    float getElapsedTime() const {
        waitForCompletion();
        float ms = 0;
        check_cuda(cudaEventElapsedTime(&ms, start_, end_), "cudaEventElapsedTime");
        return ms;
    }
    cudaEvent_t start() const { return start_; }
    cudaEvent_t end() const { return end_; }
private:
    cudaEvent_t start_{}, end_{};
};

class Queue {
public:
    Queue() {
        auto s = new cudaStream_t;
        check_cuda(cudaStreamCreateWithFlags(s, cudaStreamNonBlocking), "cudaStreamCreate");
        stream_ = std::shared_ptr<cudaStream_t>(s, [](cudaStream_t* p) { cudaStreamDestroy(*p); delete p; });
    }
    void finish() const { check_cuda(cudaStreamSynchronize(*stream_), "cudaStreamSynchronize"); }
    cudaStream_t unwrap() const { return *stream_; }
private:
    std::shared_ptr<cudaStream_t> stream_;
};

namespace current {
inline const Queue& queue() {
    thread_local Queue q;  // one queue per host thread (gpgpu/src/gpgpu.cpp:155-168)
    return q;
}
}  // namespace current

// ---------------------------------------------------------------------------- Buffer<T>
template <typename T>
class Buffer {
public:
    Buffer() = default;
    explicit Buffer(size_t size) : size_(size) {
        void* p = nullptr;
        check_cuda(cudaMalloc(&p, (size ? size : 1) * sizeof(T)), "cudaMalloc");
        mem_ = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
    }
    size_t size() const noexcept { return size_; }
    size_t data_size() const noexcept { return size_ * sizeof(T); }
    void write(const Queue& q, const T* host, size_t n, size_t offset = 0) {
        check_cuda(cudaMemcpyAsync(unwrap() + offset, host, n * sizeof(T), cudaMemcpyHostToDevice, q.unwrap()),
                   "cudaMemcpyAsync");
        q.finish();
    }
    void read(const Queue& q, T* host, size_t n, size_t offset = 0) const {
        check_cuda(cudaMemcpyAsync(host, unwrap() + offset, n * sizeof(T), cudaMemcpyDeviceToHost, q.unwrap()),
                   "cudaMemcpyAsync");
        q.finish();
    }
    T* unwrap() const noexcept { return static_cast<T*>(mem_.get()); }
private:
    std::shared_ptr<void> mem_;
    size_t size_ = 0;
};

// Scratch that lives as long as one call: a LIFO slab like the reference's per-context pool
// (rawContext::getTemporaryBuffer / releaseTemporaryBuffer, gpgpu/src/gpgpu.cpp:189-214): a
// buffer is carved off the end of the slab, buffers are released in reverse order of their
// creation (anything else throws, as in the reference), and the slab only grows. One pool per
// host thread and device, next to that thread's queue: work that uses the scratch is ordered by
// the queue, so the next call may overwrite it without waiting - which is what lets the calls
// below stay asynchronous. Like the reference's pool it must not be shared between queues whose
// work overlaps.
class TemporaryPool {
public:
    static TemporaryPool& current() {
        thread_local TemporaryPool pools[16];
        int dev = 0;
        check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
        if (dev < 0 || dev >= 16) throw APIError(static_cast<int>(cudaErrorInvalidDevice), "TemporaryPool");
        return pools[dev];
    }
    // returns the byte offset of `bytes` bytes of scratch, aligned to `align`
    size_t acquire(size_t bytes, size_t align, void** base) {
        size_t off = top_;
        if (off % align) off += align - off % align;
        const size_t end = off + bytes;
        if (end > size_) {
            // earlier work may still use the old slab: it is freed only after the device drained
            // (cudaFree waits), and nothing carved from it may be alive
            if (top_ != 0) throw std::runtime_error("temporary buffer pool cannot grow while in use");
            if (slab_) check_cuda(cudaFree(slab_), "cudaFree");
            slab_ = nullptr;
            size_t want = end < (size_t(1) << 20) ? (size_t(1) << 20) : end;
            check_cuda(cudaMalloc(&slab_, want), "cudaMalloc");
            size_ = want;
        }
        *base = slab_;
        marks_.push_back(top_);
        top_ = end;
        return off;
    }
    void release(size_t end) {
        if (end != top_ || marks_.empty()) throw std::runtime_error("temporary buffer allocation violation");
        top_ = marks_.back();
        marks_.pop_back();
    }
    ~TemporaryPool() { if (slab_) cudaFree(slab_); }
private:
    void* slab_ = nullptr;
    size_t size_ = 0, top_ = 0;
    std::vector<size_t> marks_;
};

template <typename T>
class TemporaryBuffer {
public:
    TemporaryBuffer() = default;
    explicit TemporaryBuffer(size_t size) : pool_(&TemporaryPool::current()), size_(size) {
        void* base = nullptr;
        const size_t align = sizeof(T) > 256 ? sizeof(T) : 256;
        offset_bytes_ = pool_->acquire(size * sizeof(T), align, &base);
        ptr_ = reinterpret_cast<T*>(static_cast<char*>(base) + offset_bytes_);
    }
    ~TemporaryBuffer() noexcept(false) { if (pool_) pool_->release(offset_bytes_ + size_ * sizeof(T)); }
    TemporaryBuffer(const TemporaryBuffer&) = delete;
    TemporaryBuffer& operator=(const TemporaryBuffer&) = delete;
    size_t size() const noexcept { return size_; }
    size_t data_size() const noexcept { return size_ * sizeof(T); }
    size_t offset() const noexcept { return offset_bytes_ / sizeof(T); }
    T* unwrap() const noexcept { return ptr_; }
private:
    TemporaryPool* pool_ = nullptr;
    size_t size_ = 0, offset_bytes_ = 0;
    T* ptr_ = nullptr;
};

// ---------------------------------------------------------------------------- blas
namespace blas {

enum class StatusCode {
    kSuccess = 0, kInvalidValue = -30, kNotImplemented = -1024, kInvalidMatrixA = -1022,
    kInvalidMatrixB = -1021, kInvalidMatrixC = -1020, kInvalidDimension = -1017,
    kInvalidLeadDimA = -1016, kInvalidLeadDimB = -1015, kInvalidLeadDimC = -1014,
    kInsufficientMemoryA = -1011, kInsufficientMemoryB = -1010, kInsufficientMemoryC = -1009,
    kInsufficientMemoryTemp = -2050, kInvalidBatchCount = -2049, kUnexpectedError = -2039,
};
enum class Layout { RowMajor = 101, ColMajor = 102 };
enum class Transpose { NoTrans = 111, Trans = 112, ConjTrans = 113 };
enum class Triangle { Upper = 121, Lower = 122 };
enum class Diagonal { NonUnit = 131, Unit = 132 };
enum class Side { Left = 141, Right = 142 };

class BLASError : public std::runtime_error {
public:
    explicit BLASError(StatusCode status)
        : std::runtime_error(std::string("BLAS error: ") + dlf_b200_status_string(static_cast<int>(status))),
          status_(status) {}
    StatusCode status() const noexcept { return status_; }
private:
    StatusCode status_;
};

using half = __half;
using bfloat16 = __nv_bfloat16;

template <typename T> struct PrecisionOf;
template <> struct PrecisionOf<float> { static constexpr int value = DLF_B200_SINGLE; };
template <> struct PrecisionOf<half> { static constexpr int value = DLF_B200_HALF; };
template <> struct PrecisionOf<bfloat16> { static constexpr int value = DLF_B200_BFLOAT16; };

namespace detail {

inline void raise(int rc, const char* where) {
    if (rc == 0) return;
    if (rc < 0) throw BLASError(static_cast<StatusCode>(rc));
    throw APIError(rc, where);
}

struct Dims { size_t a_one, a_two, b_one, b_two, c_one, c_two; };

// Xgemm<T>::ProcessArguments (gpgpu/src/routines/level3/xgemm.hpp:54-91)
inline Dims process_arguments(Layout layout, Transpose ta, Transpose tb, size_t m, size_t n, size_t k) {
    if (m == 0 || n == 0 || k == 0) throw BLASError(StatusCode::kInvalidDimension);
    const bool row = layout == Layout::RowMajor;
    const bool a_rot = (!row && ta != Transpose::NoTrans) || (row && ta == Transpose::NoTrans);
    const bool b_rot = (!row && tb != Transpose::NoTrans) || (row && tb == Transpose::NoTrans);
    return Dims{a_rot ? k : m, a_rot ? m : k, b_rot ? n : k, b_rot ? k : n, row ? n : m, row ? m : n};
}

// TestMatrixA/B/C (gpgpu/src/utilities/buffer_test.hpp:24-55)
template <typename T>
void test_matrix(size_t one, size_t two, const Buffer<T>& buf, size_t offset, size_t ld,
                 StatusCode lead, StatusCode mem) {
    if (ld < one) throw BLASError(lead);
    if (buf.data_size() < (ld * (two - 1) + one + offset) * sizeof(T)) throw BLASError(mem);
}

struct EventScope {  // start/end events around the launch, like cuKernel::launch (gpgpu_cu.cpp:389-398)
    EventScope(const Queue& q, Event* e) : q_(q), e_(e) { if (e_) cudaEventRecord(e_->start(), q_.unwrap()); }
    ~EventScope() { if (e_) cudaEventRecord(e_->end(), q_.unwrap()); }
    const Queue& q_;
    Event* e_;
};

}  // namespace detail

template <typename T>
void gemm(const Layout layout, const Transpose a_transpose, const Transpose b_transpose,
          const size_t m, const size_t n, const size_t k,
          const T alpha,
          const Buffer<T>& a_buffer, const size_t a_offset, const size_t a_ld,
          const Buffer<T>& b_buffer, const size_t b_offset, const size_t b_ld,
          const T beta,
          Buffer<T>& c_buffer, const size_t c_offset, const size_t c_ld,
          const Queue& queue = current::queue(), Event* event = nullptr) {
    const auto d = detail::process_arguments(layout, a_transpose, b_transpose, m, n, k);
    detail::test_matrix(d.a_one, d.a_two, a_buffer, a_offset, a_ld, StatusCode::kInvalidLeadDimA, StatusCode::kInsufficientMemoryA);
    detail::test_matrix(d.b_one, d.b_two, b_buffer, b_offset, b_ld, StatusCode::kInvalidLeadDimB, StatusCode::kInsufficientMemoryB);
    detail::test_matrix(d.c_one, d.c_two, c_buffer, c_offset, c_ld, StatusCode::kInvalidLeadDimC, StatusCode::kInsufficientMemoryC);
    // scratch for a K-split of products with few output tiles, from the temporary-buffer pool as
    // Xgemm takes its temporaries (gpgpu/src/routines/level3/xgemm.cpp:107-223); 0 bytes = no use
    TemporaryBuffer<unsigned char> work(dlf_b200_gemm_workspace_bytes(PrecisionOf<T>::value, m, n, k));
    detail::EventScope scope(queue, event);
    detail::raise(dlf_b200_gemm_ex(PrecisionOf<T>::value, static_cast<int>(layout), static_cast<int>(a_transpose),
                                   static_cast<int>(b_transpose), m, n, k, &alpha,
                                   a_buffer.unwrap() + a_offset, a_ld, b_buffer.unwrap() + b_offset, b_ld, &beta,
                                   c_buffer.unwrap() + c_offset, c_ld, work.size() ? work.unwrap() : nullptr,
                                   work.data_size(), queue.unwrap()),
                  "dlf_b200_gemm_ex");
}

template <typename T>
void gemmStridedBatched(const Layout layout, const Transpose a_transpose, const Transpose b_transpose,
                        const size_t m, const size_t n, const size_t k,
                        const T alpha,
                        const Buffer<T>& a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride,
                        const Buffer<T>& b_buffer, const size_t b_offset, const size_t b_ld, const size_t b_stride,
                        const T beta,
                        Buffer<T>& c_buffer, const size_t c_offset, const size_t c_ld, const size_t c_stride,
                        const size_t batch_count,
                        const Queue& queue = current::queue(), Event* event = nullptr) {
    if (batch_count < 1) throw BLASError(StatusCode::kInvalidBatchCount);
    const auto d = detail::process_arguments(layout, a_transpose, b_transpose, m, n, k);
    const size_t last = batch_count - 1;
    detail::test_matrix(d.a_one, d.a_two, a_buffer, a_offset + last * a_stride, a_ld, StatusCode::kInvalidLeadDimA, StatusCode::kInsufficientMemoryA);
    detail::test_matrix(d.b_one, d.b_two, b_buffer, b_offset + last * b_stride, b_ld, StatusCode::kInvalidLeadDimB, StatusCode::kInsufficientMemoryB);
    detail::test_matrix(d.c_one, d.c_two, c_buffer, c_offset + last * c_stride, c_ld, StatusCode::kInvalidLeadDimC, StatusCode::kInsufficientMemoryC);
    detail::EventScope scope(queue, event);
    detail::raise(dlf_b200_gemm_strided_batched(
                      PrecisionOf<T>::value, static_cast<int>(layout), static_cast<int>(a_transpose),
                      static_cast<int>(b_transpose), m, n, k, &alpha, a_buffer.unwrap() + a_offset, a_ld, a_stride,
                      b_buffer.unwrap() + b_offset, b_ld, b_stride, &beta, c_buffer.unwrap() + c_offset, c_ld,
                      c_stride, batch_count, queue.unwrap()),
                  "dlf_b200_gemm_strided_batched");
}

template <typename T>
void gemmBatched(const Layout layout, const Transpose a_transpose, const Transpose b_transpose,
                 const size_t m, const size_t n, const size_t k,
                 const T* alphas,
                 const Buffer<T>& a_buffer, const size_t* a_offsets, const size_t a_ld,
                 const Buffer<T>& b_buffer, const size_t* b_offsets, const size_t b_ld,
                 const T* betas,
                 Buffer<T>& c_buffer, const size_t* c_offsets, const size_t c_ld,
                 const size_t batch_count,
                 const Queue& queue = current::queue(), Event* event = nullptr) {
    if (batch_count < 1) throw BLASError(StatusCode::kInvalidBatchCount);
    const auto d = detail::process_arguments(layout, a_transpose, b_transpose, m, n, k);
    for (size_t i = 0; i < batch_count; ++i) {
        detail::test_matrix(d.a_one, d.a_two, a_buffer, a_offsets[i], a_ld, StatusCode::kInvalidLeadDimA, StatusCode::kInsufficientMemoryA);
        detail::test_matrix(d.b_one, d.b_two, b_buffer, b_offsets[i], b_ld, StatusCode::kInvalidLeadDimB, StatusCode::kInsufficientMemoryB);
        detail::test_matrix(d.c_one, d.c_two, c_buffer, c_offsets[i], c_ld, StatusCode::kInvalidLeadDimC, StatusCode::kInsufficientMemoryC);
    }
    // scratch for the per-batch tables: the reference takes its equivalents from the context's
    // temporary-buffer pool (gpgpu/src/gblas.cpp:2972-2988). The pool's slab outlives the call and
    // later users of it are ordered behind this call's kernel by the queue, so nothing waits here.
    TemporaryBuffer<unsigned char> work(dlf_b200_gemm_batched_workspace_bytes(batch_count));
    detail::EventScope scope(queue, event);
    detail::raise(dlf_b200_gemm_batched(
                      PrecisionOf<T>::value, static_cast<int>(layout), static_cast<int>(a_transpose),
                      static_cast<int>(b_transpose), m, n, k, alphas, a_buffer.unwrap(), a_offsets, a_ld,
                      b_buffer.unwrap(), b_offsets, b_ld, betas, c_buffer.unwrap(), c_offsets, c_ld, batch_count,
                      work.unwrap(), work.data_size(), queue.unwrap()),
                  "dlf_b200_gemm_batched");
}

// ---- level-3 routines on the GEMM main loop (gpgpu/include/gblas.h:506-586) ----

// Symmetric matrix-matrix multiplication (gblas.h:506-515)
template <typename T>
void symm(const Layout layout, const Side side, const Triangle triangle,
          const size_t m, const size_t n,
          const T alpha,
          const Buffer<T>& a_buffer, const size_t a_offset, const size_t a_ld,
          const Buffer<T>& b_buffer, const size_t b_offset, const size_t b_ld,
          const T beta,
          Buffer<T>& c_buffer, const size_t c_offset, const size_t c_ld,
          const Queue& queue = current::queue(), Event* event = nullptr) {
    if (m == 0 || n == 0) throw BLASError(StatusCode::kInvalidDimension);
    const size_t ka = side == Side::Left ? m : n;
    const bool row = layout == Layout::RowMajor;
    detail::test_matrix(ka, ka, a_buffer, a_offset, a_ld, StatusCode::kInvalidLeadDimA, StatusCode::kInsufficientMemoryA);
    detail::test_matrix(row ? n : m, row ? m : n, b_buffer, b_offset, b_ld, StatusCode::kInvalidLeadDimB, StatusCode::kInsufficientMemoryB);
    detail::test_matrix(row ? n : m, row ? m : n, c_buffer, c_offset, c_ld, StatusCode::kInvalidLeadDimC, StatusCode::kInsufficientMemoryC);
    TemporaryBuffer<unsigned char> work(dlf_b200_level3_workspace_bytes(DLF_B200_SYMM, PrecisionOf<T>::value, m, n));
    detail::EventScope scope(queue, event);
    detail::raise(dlf_b200_symm(PrecisionOf<T>::value, static_cast<int>(layout), static_cast<int>(side),
                                static_cast<int>(triangle), m, n, &alpha, a_buffer.unwrap() + a_offset, a_ld,
                                b_buffer.unwrap() + b_offset, b_ld, &beta, c_buffer.unwrap() + c_offset, c_ld,
                                work.unwrap(), work.data_size(), queue.unwrap()),
                  "dlf_b200_symm");
}

// Rank-K update of a symmetric matrix (gblas.h:528-536)
template <typename T>
void syrk(const Layout layout, const Triangle triangle, const Transpose a_transpose,
          const size_t n, const size_t k,
          const T alpha,
          const Buffer<T>& a_buffer, const size_t a_offset, const size_t a_ld,
          const T beta,
          Buffer<T>& c_buffer, const size_t c_offset, const size_t c_ld,
          const Queue& queue = current::queue(), Event* event = nullptr) {
    if (n == 0 || k == 0) throw BLASError(StatusCode::kInvalidDimension);
    const bool row = layout == Layout::RowMajor;
    const bool a_rot = (row && a_transpose == Transpose::NoTrans) || (!row && a_transpose != Transpose::NoTrans);
    detail::test_matrix(a_rot ? k : n, a_rot ? n : k, a_buffer, a_offset, a_ld, StatusCode::kInvalidLeadDimA, StatusCode::kInsufficientMemoryA);
    detail::test_matrix(n, n, c_buffer, c_offset, c_ld, StatusCode::kInvalidLeadDimC, StatusCode::kInsufficientMemoryC);
    TemporaryBuffer<unsigned char> work(dlf_b200_level3_workspace_bytes(DLF_B200_SYRK, PrecisionOf<T>::value, n, n));
    detail::EventScope scope(queue, event);
    detail::raise(dlf_b200_syrk(PrecisionOf<T>::value, static_cast<int>(layout), static_cast<int>(triangle),
                                static_cast<int>(a_transpose), n, k, &alpha, a_buffer.unwrap() + a_offset, a_ld, &beta,
                                c_buffer.unwrap() + c_offset, c_ld, work.unwrap(), work.data_size(), queue.unwrap()),
                  "dlf_b200_syrk");
}

namespace detail {
template <typename T, typename Fn>
void triangular(Fn fn, const char* name, int routine, const Layout layout, const Side side, const Triangle triangle,
                const Transpose a_transpose, const Diagonal diagonal, const size_t m, const size_t n, const T alpha,
                const Buffer<T>& a_buffer, const size_t a_offset, const size_t a_ld, Buffer<T>& b_buffer,
                const size_t b_offset, const size_t b_ld, const Queue& queue, Event* event) {
    if (m == 0 || n == 0) throw BLASError(StatusCode::kInvalidDimension);
    const size_t ka = side == Side::Left ? m : n;
    const bool row = layout == Layout::RowMajor;
    test_matrix(ka, ka, a_buffer, a_offset, a_ld, StatusCode::kInvalidLeadDimA, StatusCode::kInsufficientMemoryA);
    test_matrix(row ? n : m, row ? m : n, b_buffer, b_offset, b_ld, StatusCode::kInvalidLeadDimB, StatusCode::kInsufficientMemoryB);
    TemporaryBuffer<unsigned char> work(dlf_b200_level3_workspace_bytes(routine, PrecisionOf<T>::value, m, n) + 16);
    EventScope scope(queue, event);
    raise(fn(PrecisionOf<T>::value, static_cast<int>(layout), static_cast<int>(side), static_cast<int>(triangle),
             static_cast<int>(a_transpose), static_cast<int>(diagonal), m, n, &alpha, a_buffer.unwrap() + a_offset, a_ld,
             b_buffer.unwrap() + b_offset, b_ld, work.unwrap(), work.data_size(), queue.unwrap()),
          name);
}
}  // namespace detail

// Triangular matrix-matrix multiplication (gblas.h:570-577)
template <typename T>
void trmm(const Layout layout, const Side side, const Triangle triangle, const Transpose a_transpose, const Diagonal diagonal,
          const size_t m, const size_t n,
          const T alpha,
          const Buffer<T>& a_buffer, const size_t a_offset, const size_t a_ld,
          Buffer<T>& b_buffer, const size_t b_offset, const size_t b_ld,
          const Queue& queue = current::queue(), Event* event = nullptr) {
    detail::triangular<T>(dlf_b200_trmm, "dlf_b200_trmm", DLF_B200_TRMM, layout, side, triangle, a_transpose, diagonal, m, n,
                          alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, queue, event);
}

// Solves a triangular system of equations (gblas.h:579-586)
template <typename T>
void trsm(const Layout layout, const Side side, const Triangle triangle, const Transpose a_transpose, const Diagonal diagonal,
          const size_t m, const size_t n,
          const T alpha,
          const Buffer<T>& a_buffer, const size_t a_offset, const size_t a_ld,
          Buffer<T>& b_buffer, const size_t b_offset, const size_t b_ld,
          const Queue& queue = current::queue(), Event* event = nullptr) {
    detail::triangular<T>(dlf_b200_trsm, "dlf_b200_trsm", DLF_B200_TRSM, layout, side, triangle, a_transpose, diagonal, m, n,
                          alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, queue, event);
}

}  // namespace blas

// ---------------------------------------------------------------------------- dnn
namespace dnn {

// gpgpu::dnn::conv2d (gpgpu/include/gdnn.h:201-213). `bias`, `residual` and `activation` are
// additions (default: none): the reference adds the bias in a separate pass
// (dlf/include/predict.h:1272-1281) and runs the residual Add (predict.h:928-960) and the Relu
// (predict.h:776-784) as operators of their own; here they are fused into the epilogue.
template <typename T>
void conv2d(const size_t batches, const size_t channels,
            const size_t height, const size_t width,
            const size_t output_h, const size_t output_w,
            const size_t num_kernels, const size_t group,
            const size_t kernel_h, const size_t kernel_w,
            const size_t pad_top, const size_t pad_left,
            const size_t pad_bottom, const size_t pad_right,
            const size_t stride_h, const size_t stride_w,
            const size_t dilation_h, const size_t dilation_w,
            const Buffer<T>& im_buffer, const Buffer<T>& kernel_buffer,
            Buffer<T>& result_buffer,
            const Queue& queue = current::queue(), Event* event = nullptr,
            const Buffer<T>* bias = nullptr, const Buffer<T>* residual = nullptr,
            const int activation = DLF_B200_ACT_NONE) {
    using blas::BLASError;
    using blas::StatusCode;
    if (group == 0 || channels % group != 0 || num_kernels % group != 0) throw BLASError(StatusCode::kInvalidDimension);
    if (im_buffer.size() < batches * channels * height * width) throw BLASError(StatusCode::kInsufficientMemoryA);
    if (kernel_buffer.size() < num_kernels * (channels / group) * kernel_h * kernel_w) throw BLASError(StatusCode::kInsufficientMemoryB);
    if (result_buffer.size() < batches * num_kernels * output_h * output_w) throw BLASError(StatusCode::kInsufficientMemoryC);
    if (bias && bias->size() < num_kernels) throw BLASError(StatusCode::kInvalidValue);
    if (residual && residual->size() < batches * num_kernels * output_h * output_w) throw BLASError(StatusCode::kInvalidValue);
    // scratch for the filter bank in the kernel's shared-memory layout, from the temporary-buffer
    // pool as cudnnConv takes its workspace (gpgpu/src/gdnn.cpp:1452-1508). Without it the kernel
    // gathers the filter bank inside its main loop, at well under half the speed.
    TemporaryBuffer<unsigned char> work(dlf_b200_conv2d_workspace_bytes(
        blas::PrecisionOf<T>::value, batches, channels, height, width, output_h, output_w, num_kernels, group,
        kernel_h, kernel_w));
    blas::detail::EventScope scope(queue, event);
    blas::detail::raise(dlf_b200_conv2d_fused(blas::PrecisionOf<T>::value, batches, channels, height, width,
                                              output_h, output_w, num_kernels, group, kernel_h, kernel_w, pad_top,
                                              pad_left, pad_bottom, pad_right, stride_h, stride_w, dilation_h,
                                              dilation_w, im_buffer.unwrap(), kernel_buffer.unwrap(),
                                              bias ? bias->unwrap() : nullptr,
                                              residual ? residual->unwrap() : nullptr, activation,
                                              result_buffer.unwrap(), work.unwrap(), work.data_size(),
                                              queue.unwrap()),
                        "dlf_b200_conv2d_fused");
}

// gpgpu::dnn::maxpool / avgpool in the argument order of their definitions
// (gpgpu/src/gdnn.cpp:1667-1676, 1728-1738).
template <typename T>
void maxpool(const size_t batches, const size_t channels,
             const size_t height, const size_t width,
             const size_t output_h, const size_t output_w,
             const size_t kernel_h, const size_t kernel_w,
             const size_t pad_top, const size_t pad_left,
             const size_t pad_bottom, const size_t pad_right,
             const size_t stride_h, const size_t stride_w,
             const size_t dilation_h, const size_t dilation_w,
             const Buffer<T>& x_buffer, Buffer<T>& y_buffer,
             const Queue& queue = current::queue(), Event* event = nullptr) {
    using blas::BLASError;
    using blas::StatusCode;
    if (x_buffer.size() < batches * channels * height * width) throw BLASError(StatusCode::kInsufficientMemoryA);
    if (y_buffer.size() < batches * channels * output_h * output_w) throw BLASError(StatusCode::kInsufficientMemoryC);
    blas::detail::EventScope scope(queue, event);
    blas::detail::raise(dlf_b200_maxpool(blas::PrecisionOf<T>::value, batches, channels, height, width, output_h,
                                         output_w, kernel_h, kernel_w, pad_top, pad_left, pad_bottom, pad_right,
                                         stride_h, stride_w, dilation_h, dilation_w, x_buffer.unwrap(),
                                         y_buffer.unwrap(), queue.unwrap()),
                        "dlf_b200_maxpool");
}

template <typename T>
void avgpool(const size_t batches, const size_t channels,
             const size_t height, const size_t width,
             const size_t output_h, const size_t output_w,
             const size_t kernel_h, const size_t kernel_w,
             const size_t pad_top, const size_t pad_left,
             const size_t pad_bottom, const size_t pad_right,
             const size_t stride_h, const size_t stride_w,
             const size_t dilation_h, const size_t dilation_w,
             const bool count_include_pad,
             const Buffer<T>& x_buffer, Buffer<T>& y_buffer,
             const Queue& queue = current::queue(), Event* event = nullptr) {
    using blas::BLASError;
    using blas::StatusCode;
    if (x_buffer.size() < batches * channels * height * width) throw BLASError(StatusCode::kInsufficientMemoryA);
    if (y_buffer.size() < batches * channels * output_h * output_w) throw BLASError(StatusCode::kInsufficientMemoryC);
    blas::detail::EventScope scope(queue, event);
    blas::detail::raise(dlf_b200_avgpool(blas::PrecisionOf<T>::value, batches, channels, height, width, output_h,
                                         output_w, kernel_h, kernel_w, pad_top, pad_left, pad_bottom, pad_right,
                                         stride_h, stride_w, dilation_h, dilation_w, count_include_pad ? 1 : 0,
                                         x_buffer.unwrap(), y_buffer.unwrap(), queue.unwrap()),
                        "dlf_b200_avgpool");
}

// Channels-last operators for an operator-list runtime that owns the tensors between its operators
// (no counterpart in gpgpu::dnn, whose operators are NCHW): the same argument order as the NCHW
// functions above, buffers (N, H, W, C), 16-bit T.
enum class Layout4D { NHWC = DLF_B200_LAYOUT_NHWC, NCHW = DLF_B200_LAYOUT_NCHW };

template <typename T>
void nchw_to_nhwc(const size_t batches, const size_t channels, const size_t height, const size_t width,
                  const Buffer<T>& x_buffer, Buffer<T>& y_buffer,
                  const Queue& queue = current::queue(), Event* event = nullptr) {
    using blas::BLASError;
    using blas::StatusCode;
    if (x_buffer.size() < batches * channels * height * width) throw BLASError(StatusCode::kInsufficientMemoryA);
    if (y_buffer.size() < batches * height * width * ((channels + 7) / 8 * 8)) throw BLASError(StatusCode::kInsufficientMemoryC);
    blas::detail::EventScope scope(queue, event);
    blas::detail::raise(dlf_b200_nchw_to_nhwc(blas::PrecisionOf<T>::value, batches, channels, height, width,
                                              x_buffer.unwrap(), y_buffer.unwrap(), queue.unwrap()),
                        "dlf_b200_nchw_to_nhwc");
}

// OIHW filter bank -> the K-major operand conv2d_nhwc reads; `packed` holds at least
// dlf_b200_nhwc_filter_elems(channels, num_kernels, kernel_h, kernel_w) elements. Done once per layer.
template <typename T>
void pack_filters_nhwc(const size_t channels, const size_t num_kernels, const size_t kernel_h, const size_t kernel_w,
                       const Buffer<T>& kernel_buffer, Buffer<T>& packed,
                       const Queue& queue = current::queue(), Event* event = nullptr) {
    using blas::BLASError;
    using blas::StatusCode;
    if (kernel_buffer.size() < num_kernels * channels * kernel_h * kernel_w) throw BLASError(StatusCode::kInsufficientMemoryB);
    if (packed.size() < dlf_b200_nhwc_filter_elems(channels, num_kernels, kernel_h, kernel_w))
        throw BLASError(StatusCode::kInsufficientMemoryC);
    blas::detail::EventScope scope(queue, event);
    blas::detail::raise(dlf_b200_pack_filters_nhwc(blas::PrecisionOf<T>::value, channels, num_kernels, kernel_h, kernel_w,
                                                   kernel_buffer.unwrap(), packed.unwrap(), queue.unwrap()),
                        "dlf_b200_pack_filters_nhwc");
}

template <typename T>
void conv2d_nhwc(const size_t batches, const size_t channels,
                 const size_t height, const size_t width,
                 const size_t output_h, const size_t output_w,
                 const size_t num_kernels,
                 const size_t kernel_h, const size_t kernel_w,
                 const size_t pad_top, const size_t pad_left,
                 const size_t pad_bottom, const size_t pad_right,
                 const size_t stride_h, const size_t stride_w,
                 const size_t dilation_h, const size_t dilation_w,
                 const Buffer<T>& im_buffer, const Buffer<T>& packed_kernel_buffer,
                 Buffer<T>& result_buffer,
                 const Queue& queue = current::queue(), Event* event = nullptr,
                 const Buffer<T>* bias = nullptr, const Buffer<T>* residual = nullptr,
                 const int activation = DLF_B200_ACT_NONE, const Layout4D result_layout = Layout4D::NHWC) {
    using blas::BLASError;
    using blas::StatusCode;
    if (im_buffer.size() < batches * channels * height * width) throw BLASError(StatusCode::kInsufficientMemoryA);
    if (packed_kernel_buffer.size() < dlf_b200_nhwc_filter_elems(channels, num_kernels, kernel_h, kernel_w))
        throw BLASError(StatusCode::kInsufficientMemoryB);
    if (result_buffer.size() < batches * num_kernels * output_h * output_w) throw BLASError(StatusCode::kInsufficientMemoryC);
    if (bias && bias->size() < num_kernels) throw BLASError(StatusCode::kInvalidValue);
    if (residual && residual->size() < batches * num_kernels * output_h * output_w) throw BLASError(StatusCode::kInvalidValue);
    blas::detail::EventScope scope(queue, event);
    blas::detail::raise(dlf_b200_conv2d_nhwc(blas::PrecisionOf<T>::value, batches, channels, height, width, output_h,
                                             output_w, num_kernels, kernel_h, kernel_w, pad_top, pad_left, pad_bottom,
                                             pad_right, stride_h, stride_w, dilation_h, dilation_w, im_buffer.unwrap(),
                                             packed_kernel_buffer.unwrap(), bias ? bias->unwrap() : nullptr,
                                             residual ? residual->unwrap() : nullptr, activation, result_buffer.unwrap(),
                                             static_cast<int>(result_layout), queue.unwrap()),
                        "dlf_b200_conv2d_nhwc");
}

// max (average == false) or average pooling between channels-last buffers
template <typename T>
void pool_nhwc(const bool average, const bool count_include_pad,
               const size_t batches, const size_t channels,
               const size_t height, const size_t width,
               const size_t output_h, const size_t output_w,
               const size_t kernel_h, const size_t kernel_w,
               const size_t pad_top, const size_t pad_left,
               const size_t stride_h, const size_t stride_w,
               const Buffer<T>& x_buffer, Buffer<T>& y_buffer,
               const Queue& queue = current::queue(), Event* event = nullptr) {
    using blas::BLASError;
    using blas::StatusCode;
    if (x_buffer.size() < batches * channels * height * width) throw BLASError(StatusCode::kInsufficientMemoryA);
    if (y_buffer.size() < batches * channels * output_h * output_w) throw BLASError(StatusCode::kInsufficientMemoryC);
    blas::detail::EventScope scope(queue, event);
    blas::detail::raise(dlf_b200_pool_nhwc(blas::PrecisionOf<T>::value, average ? 1 : 0, count_include_pad ? 1 : 0, batches,
                                           channels, height, width, output_h, output_w, kernel_h, kernel_w, pad_top,
                                           pad_left, stride_h, stride_w, x_buffer.unwrap(), y_buffer.unwrap(),
                                           queue.unwrap()),
                        "dlf_b200_pool_nhwc");
}

}  // namespace dnn
}  // namespace gpgpu
}  // namespace dlf_b200

#endif  // DLF_B200_GPGPU_HPP_

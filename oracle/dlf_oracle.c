/* dlf_oracle.c - CPU restatement of dlf's CPU implementation of the dense-contraction path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA path is compared against; it is
 * never linked into, imported by or called from the product library. Only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark may use it.
 *
 * Parity pin: the functions below reproduce, bit for bit, every golden vector the reference's
 * own unit tests hold for this path (small-integer inputs, exact in fp32): TensorTest.Gemm,
 * GPGPUTest.GEMM, MatMulTest.*, Conv2D.* and PredictTest.Gemm/Conv (see tests/golden/). For
 * float GEMM the reference's arithmetic lives in a third-party BLAS that is not vendored:
 * Intel MKL 2019.4-070 (Dockerfile:23; ILP64 + TBB threading, cmake/FindMKL.cmake:42-44),
 * reached through cblas_sgemm (dlf/include/cxxblas.h:727-740). Its blocking and summation
 * order are not observable, so for random inputs parity is defined by the tolerances of the
 * tests (1e-5 relative Frobenius for fp32), not bit equality: beyond the small goldens parity
 * is unpinned. dlf_oracle_sgemm restates the published definition of SGEMM.
 *
 * Each function cites the reference lines it follows (paths relative to the dlf tree).
 */
#include <float.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DLF_ROW_MAJOR 101
#define DLF_COL_MAJOR 102
#define DLF_NO_TRANS 111
#define DLF_TRANS 112
#define DLF_CONJ_TRANS 113

/* ------------------------------------------------------------------------------------------
 * gemm_serial: dlf/include/tensor/linalg_detail.h:241-268. The generic (non-BLAS) kernel that
 * defines the exact evaluation order for integer types: if incB < ldb, C is scaled by beta and
 * then updated row by row with axpys (k outer, j inner); otherwise each C[i][j] is a dot
 * product followed by alpha*acc + beta*C. alpha == 0 only scales C. The scaling (mscal,
 * linalg_detail.h:78-89) writes zeros without reading C when beta == 0.
 * ------------------------------------------------------------------------------------------ */
#define DEFINE_GEMM_SERIAL(NAME, T)                                                              \
    void NAME(int m, int n, int p, T alpha, const T* A, int lda, int incA, const T* B, int ldb,  \
              int incB, T beta, T* C, int ldc) {                                                 \
        int i, j, k;                                                                             \
        if (alpha == (T)0) {                                                                     \
            for (i = 0; i < m; ++i)                                                              \
                for (j = 0; j < n; ++j)                                                          \
                    C[(size_t)i * ldc + j] = beta == (T)0 ? (T)0 : beta * C[(size_t)i * ldc + j];    \
            return;                                                                              \
        }                                                                                        \
        if (incB < ldb) {                                                                        \
            for (i = 0; i < m; ++i)                                                              \
                for (j = 0; j < n; ++j)                                                          \
                    C[(size_t)i * ldc + j] = beta == (T)0 ? (T)0 : beta * C[(size_t)i * ldc + j];    \
            for (i = 0; i < m; ++i) {                                                            \
                const T* Ai = A + (size_t)i * lda;                                               \
                T* Ci = C + (size_t)i * ldc;                                                     \
                for (k = 0; k < p; ++k) {                                                        \
                    const T s = alpha * Ai[(size_t)k * incA];                                    \
                    const T* Bk = B + (size_t)k * ldb;                                           \
                    for (j = 0; j < n; ++j) Ci[j] += s * Bk[(size_t)j * incB];                   \
                }                                                                                \
            }                                                                                    \
        } else {                                                                                 \
            for (i = 0; i < m; ++i) {                                                            \
                const T* Ai = A + (size_t)i * lda;                                               \
                T* Ci = C + (size_t)i * ldc;                                                     \
                for (j = 0; j < n; ++j) {                                                        \
                    T acc = (T)0;                                                                \
                    const T* Bj = B + (size_t)j * incB;                                          \
                    for (k = 0; k < p; ++k) acc += Ai[(size_t)k * incA] * Bj[(size_t)k * ldb];   \
                    Ci[j] = alpha * acc + beta * Ci[j];                                          \
                }                                                                                \
            }                                                                                    \
        }                                                                                        \
    }

DEFINE_GEMM_SERIAL(dlf_oracle_gemm_serial_f32, float)
DEFINE_GEMM_SERIAL(dlf_oracle_gemm_serial_f64, double)
DEFINE_GEMM_SERIAL(dlf_oracle_gemm_serial_i32, int32_t)
DEFINE_GEMM_SERIAL(dlf_oracle_gemm_serial_i64, int64_t)

/* detail::gemm for non-BLAS types: dlf/include/tensor/linalg_detail.h:314-329. A transposed
 * operand is expressed by swapping (ld, inc). Row-major throughout, as dlf::gemm passes
 * stride(0) as the leading dimension (dlf/include/tensor/linalg.h:42-101). */
#define DEFINE_GEMM_GENERIC(NAME, SERIAL, T)                                                     \
    void NAME(int trans_a, int trans_b, int m, int n, int p, T alpha, const T* A, int lda,       \
              const T* B, int ldb, T beta, T* C, int ldc) {                                      \
        int incA = 1, incB = 1, t;                                                               \
        if (trans_a != DLF_NO_TRANS) { t = lda; lda = incA; incA = t; }                          \
        if (trans_b != DLF_NO_TRANS) { t = ldb; ldb = incB; incB = t; }                          \
        SERIAL(m, n, p, alpha, A, lda, incA, B, ldb, incB, beta, C, ldc);                        \
    }

DEFINE_GEMM_GENERIC(dlf_oracle_gemm_generic_f32, dlf_oracle_gemm_serial_f32, float)
DEFINE_GEMM_GENERIC(dlf_oracle_gemm_generic_f64, dlf_oracle_gemm_serial_f64, double)
DEFINE_GEMM_GENERIC(dlf_oracle_gemm_generic_i32, dlf_oracle_gemm_serial_i32, int32_t)
DEFINE_GEMM_GENERIC(dlf_oracle_gemm_generic_i64, dlf_oracle_gemm_serial_i64, int64_t)

/* ------------------------------------------------------------------------------------------
 * cblas::gemm -> cblas_sgemm(layout, transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, C,
 * ldc): dlf/include/cxxblas.h:727-740, called with RowMajor from
 * dlf/include/tensor/linalg_detail.h:332-344. Restated from the BLAS definition
 * C = alpha*op(A)*op(B) + beta*C; beta == 0 overwrites C without reading it. Rows of C are
 * spread over OpenMP threads (standing in for MKL's TBB threading layer). `wide` selects the
 * accumulator: 0 = float (what an fp32 BLAS does), 1 = double (error reference).
 * ------------------------------------------------------------------------------------------ */
static void sgemm_rowmajor(int ta, int tb, int m, int n, int k, float alpha, const float* A,
                           int lda, const float* B, int ldb, float beta, float* C, int ldc,
                           int wide) {
    /* element (i,kk) of op(A) = A[i*sa_i + kk*sa_k] */
    const size_t sa_i = ta == DLF_NO_TRANS ? (size_t)lda : 1, sa_k = ta == DLF_NO_TRANS ? 1 : (size_t)lda;
    const size_t sb_k = tb == DLF_NO_TRANS ? (size_t)ldb : 1, sb_j = tb == DLF_NO_TRANS ? 1 : (size_t)ldb;
    int i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < m; ++i) {
        int j, kk;
        float* Ci = C + (size_t)i * ldc;
        if (wide) {
            double* acc = (double*)calloc((size_t)n, sizeof(double));
            for (kk = 0; kk < k; ++kk) {
                const double a = (double)A[i * sa_i + kk * sa_k];
                const float* Bk = B + kk * sb_k;
                for (j = 0; j < n; ++j) acc[j] += a * (double)Bk[j * sb_j];
            }
            for (j = 0; j < n; ++j)
                Ci[j] = (float)((double)alpha * acc[j] + (beta == 0.0f ? 0.0 : (double)beta * (double)Ci[j]));
            free(acc);
        } else {
            float* acc = (float*)calloc((size_t)n, sizeof(float));
            for (kk = 0; kk < k; ++kk) {
                const float a = A[i * sa_i + kk * sa_k];
                const float* Bk = B + kk * sb_k;
                for (j = 0; j < n; ++j) acc[j] += a * Bk[j * sb_j];
            }
            for (j = 0; j < n; ++j) Ci[j] = alpha * acc[j] + (beta == 0.0f ? 0.0f : beta * Ci[j]);
            free(acc);
        }
    }
}

void dlf_oracle_sgemm(int layout, int trans_a, int trans_b, int m, int n, int k, float alpha,
                      const float* A, int lda, const float* B, int ldb, float beta, float* C,
                      int ldc, int wide) {
    if (layout == DLF_ROW_MAJOR) {
        sgemm_rowmajor(trans_a, trans_b, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, wide);
    } else {
        /* a column-major product is the row-major product of the swapped operands:
         * C^T = op(B)^T op(A)^T  (the identity the reference itself relies on at
         * gpgpu/src/gblas.cpp:1932-1940) */
        sgemm_rowmajor(trans_b, trans_a, n, m, k, alpha, B, ldb, A, lda, beta, C, ldc, wide);
    }
}

/* gpgpu::blas::gemm semantics (gpgpu/include/gblas.h:496-504): element offsets into the three
 * buffers, then the same product. Index truth table: routines/level3/xgemm.hpp:54-91. */
void dlf_oracle_gblas_sgemm(int layout, int trans_a, int trans_b, size_t m, size_t n, size_t k,
                            float alpha, const float* A, size_t a_offset, size_t a_ld,
                            const float* B, size_t b_offset, size_t b_ld, float beta, float* C,
                            size_t c_offset, size_t c_ld, int wide) {
    dlf_oracle_sgemm(layout, trans_a, trans_b, (int)m, (int)n, (int)k, alpha, A + a_offset,
                     (int)a_ld, B + b_offset, (int)b_ld, beta, C + c_offset, (int)c_ld, wide);
}

/* gemmStridedBatched (gblas.h:673-683): batch i uses offsets a_offset + i*a_stride etc; CPU
 * counterpart = the per-batch cblas::gemm loop of detail::matmul
 * (dlf/include/tensor/linalg_detail.h:1480-1571). */
void dlf_oracle_gblas_sgemm_strided_batched(int layout, int trans_a, int trans_b, size_t m,
                                            size_t n, size_t k, float alpha, const float* A,
                                            size_t a_offset, size_t a_ld, size_t a_stride,
                                            const float* B, size_t b_offset, size_t b_ld,
                                            size_t b_stride, float beta, float* C, size_t c_offset,
                                            size_t c_ld, size_t c_stride, size_t batch, int wide) {
    size_t i;
    for (i = 0; i < batch; ++i)
        dlf_oracle_sgemm(layout, trans_a, trans_b, (int)m, (int)n, (int)k, alpha,
                         A + a_offset + i * a_stride, (int)a_ld, B + b_offset + i * b_stride,
                         (int)b_ld, beta, C + c_offset + i * c_stride, (int)c_ld, wide);
}

/* gemmBatched (gblas.h:661-671): per-batch alpha, beta and offsets. */
void dlf_oracle_gblas_sgemm_batched(int layout, int trans_a, int trans_b, size_t m, size_t n,
                                    size_t k, const float* alphas, const float* A,
                                    const size_t* a_offsets, size_t a_ld, const float* B,
                                    const size_t* b_offsets, size_t b_ld, const float* betas,
                                    float* C, const size_t* c_offsets, size_t c_ld, size_t batch,
                                    int wide) {
    size_t i;
    for (i = 0; i < batch; ++i)
        dlf_oracle_sgemm(layout, trans_a, trans_b, (int)m, (int)n, (int)k, alphas[i],
                         A + a_offsets[i], (int)a_ld, B + b_offsets[i], (int)b_ld, betas[i],
                         C + c_offsets[i], (int)c_ld, wide);
}

/* ------------------------------------------------------------------------------------------
 * Filter2D::output_h / output_w: dlf/include/tensor/dnn.h:99-109.
 * ------------------------------------------------------------------------------------------ */
size_t dlf_oracle_output_dim(size_t in, size_t pad_lo, size_t pad_hi, size_t kernel,
                             size_t stride, size_t dilation) {
    const size_t size = in + pad_lo + pad_hi;
    const size_t ext = dilation * (kernel - 1) + 1;
    return size >= ext ? (size - ext) / stride + 1 : 1;
}

/* detail::im2col: dlf/include/tensor/dnn_detail.h:77-121. One image, `channels` (= C/group)
 * channels; col[(c*kh*kw + kh_id*kw + kw_id)][h_id][w_id] = padded input or 0. */
void dlf_oracle_im2col_f32(const float* x, float* col, int channels, int input_h, int input_w,
                           int output_h, int output_w, int kernel_h, int kernel_w, int pad_h,
                           int pad_w, int stride_h, int stride_w, int dilation_h,
                           int dilation_w) {
    int hc;
#pragma omp parallel for schedule(static)
    for (hc = 0; hc < output_h * channels; ++hc) {
        const int c_id = hc / output_h;
        const int h_id = hc - c_id * output_h;
        int w_id, kh_id, kw_id;
        for (w_id = 0; w_id < output_w; ++w_id)
            for (kh_id = 0; kh_id < kernel_h; ++kh_id)
                for (kw_id = 0; kw_id < kernel_w; ++kw_id) {
                    const int h_index = kh_id * dilation_h + stride_h * h_id - pad_h;
                    const int w_index = kw_id * dilation_w + stride_w * w_id - pad_w;
                    float val = 0.0f;
                    if (h_index >= 0 && h_index < input_h && w_index >= 0 && w_index < input_w)
                        val = x[((size_t)c_id * input_h + h_index) * input_w + w_index];
                    const int kernel_index = kw_id + kernel_w * kh_id;
                    col[(((size_t)c_id * kernel_h * kernel_w + kernel_index) * output_h + h_id) *
                            output_w + w_id] = val;
                }
    }
}

/* detail::conv2d (CPU): dlf/include/tensor/dnn_detail.h:123-152. For each image, for each
 * group: im2col into a {k, n} work matrix, then Y_b,g = W_g (m x k) * work (k x n) with
 * alpha = 1, beta = 0. Cross-correlation; (pad_top, pad_left) shift the origin. `gemm_fn` is
 * the row-major NoTrans/NoTrans sgemm to use (NULL = dlf_oracle_sgemm with a float accumulator),
 * so the timed CPU baseline can plug in a tuned cblas_sgemm exactly where the reference does. */
typedef void (*dlf_oracle_sgemm_nn_fn)(int m, int n, int k, const float* A, int lda,
                                       const float* B, int ldb, float* C, int ldc);

void dlf_oracle_conv2d_f32(const float* X, const float* W, float* Y, size_t batches,
                           size_t channels, size_t height, size_t width, size_t num_kernels,
                           size_t group, size_t kernel_h, size_t kernel_w, size_t pad_top,
                           size_t pad_left, size_t pad_bottom, size_t pad_right, size_t stride_h,
                           size_t stride_w, size_t dilation_h, size_t dilation_w, int wide,
                           dlf_oracle_sgemm_nn_fn gemm_fn) {
    const size_t oh = dlf_oracle_output_dim(height, pad_top, pad_bottom, kernel_h, stride_h, dilation_h);
    const size_t ow = dlf_oracle_output_dim(width, pad_left, pad_right, kernel_w, stride_w, dilation_w);
    const size_t m = num_kernels / group;
    const size_t k = channels * kernel_h * kernel_w / group;
    const size_t n = oh * ow;
    float* work = (float*)malloc(k * n * sizeof(float));
    const float* xb = X;
    float* yb = Y;
    size_t b, c;
    for (b = 0; b < batches; ++b) {
        const float* wb = W;
        for (c = 0; c < group; ++c) {
            dlf_oracle_im2col_f32(xb, work, (int)(channels / group), (int)height, (int)width,
                                  (int)oh, (int)ow, (int)kernel_h, (int)kernel_w, (int)pad_top,
                                  (int)pad_left, (int)stride_h, (int)stride_w, (int)dilation_h,
                                  (int)dilation_w);
            if (gemm_fn)
                gemm_fn((int)m, (int)n, (int)k, wb, (int)k, work, (int)n, yb, (int)n);
            else
                dlf_oracle_sgemm(DLF_ROW_MAJOR, DLF_NO_TRANS, DLF_NO_TRANS, (int)m, (int)n, (int)k,
                                 1.0f, wb, (int)k, work, (int)n, 0.0f, yb, (int)n, wide);
            xb += channels * height * width / group;
            yb += num_kernels * n / group;
            wb += num_kernels * k / group;
        }
    }
    free(work);
}

/* Bias add of ConvOp::evaluate: dlf/include/predict.h:1272-1281 -> transformChannel(out, B,
 * out, axis 1, plus), CPU form dlf/include/tensor/transform.h:155-182: Y[b][c][:] += B[c]. */
void dlf_oracle_bias_f32(float* Y, const float* bias, size_t batches, size_t channels,
                         size_t plane) {
    size_t bc;
    for (bc = 0; bc < batches * channels; ++bc) {
        const float v = bias[bc % channels];
        float* y = Y + bc * plane;
        size_t i;
        for (i = 0; i < plane; ++i) y[i] = y[i] + v;
    }
}

/* Pooling: dlf/include/tensor/dnn_detail.h:172-227 (detail::pooling) with the accumulators of
 * dlf/include/tensor/dnn.h:207-247: max_pooling starts from numeric_limits<T>::lowest() and keeps
 * std::max; average_pooling starts from T{} (0), adds in (kh, kw) order and divides by the
 * number of taps inside the image, or by kernel_h*kernel_w with count_include_pad. mode: 0 max,
 * 1 average. The origin shift is (pad_top, pad_left) (pad_h() / pad_w(), dnn.h:92-93). */
void dlf_oracle_pool2d_f32(const float* X, float* Y, int mode, int count_include_pad, size_t batches,
                           size_t channels, size_t height, size_t width, size_t output_h,
                           size_t output_w, size_t kernel_h, size_t kernel_w, size_t pad_top,
                           size_t pad_left, size_t stride_h, size_t stride_w, size_t dilation_h,
                           size_t dilation_w) {
    long b, c, h, w, kh, kw;
    for (b = 0; b < (long)batches; ++b)
        for (c = 0; c < (long)channels; ++c)
            for (h = 0; h < (long)output_h; ++h)
                for (w = 0; w < (long)output_w; ++w) {
                    float acc = mode == 0 ? -FLT_MAX : 0.0f;
                    int count = 0;
                    for (kh = 0; kh < (long)kernel_h; ++kh) {
                        const long hi = kh * (long)dilation_h + (long)stride_h * h - (long)pad_top;
                        if (hi < 0 || hi >= (long)height) continue;
                        for (kw = 0; kw < (long)kernel_w; ++kw) {
                            const long wi = kw * (long)dilation_w + (long)stride_w * w - (long)pad_left;
                            float x;
                            if (wi < 0 || wi >= (long)width) continue;
                            x = X[((b * (long)channels + c) * (long)height + hi) * (long)width + wi];
                            if (mode == 0) acc = acc < x ? x : acc; /* std::max(acc, x) */
                            else acc = acc + x;
                            ++count;
                        }
                    }
                    if (count_include_pad) count = (int)(kernel_h * kernel_w);
                    Y[((b * (long)channels + c) * (long)output_h + h) * (long)output_w + w] =
                        mode == 0 ? acc : acc / count;
                }
}

/* Global pooling: dlf/include/tensor/dnn_detail.h:229-260 (detail::global_pooling) with the
 * accumulators of dlf/include/tensor/dnn.h:337-375: one value per (batch, channel) plane, the
 * maximum or sum / N. The reference combines partial results of a parallel reduction in an
 * unspecified order; this restatement adds sequentially (with a double accumulator when `wide`,
 * the error reference for tolerance tests). */
void dlf_oracle_global_pool_f32(const float* X, float* Y, int mode, size_t planes, size_t n, int wide) {
    size_t p, i;
    for (p = 0; p < planes; ++p) {
        const float* x = X + p * n;
        if (mode == 0) {
            float acc = -FLT_MAX;
            for (i = 0; i < n; ++i) acc = acc < x[i] ? x[i] : acc;
            Y[p] = acc;
        } else if (wide) {
            double acc = 0.0;
            for (i = 0; i < n; ++i) acc += x[i];
            Y[p] = (float)(acc / (double)n);
        } else {
            float acc = 0.0f;
            for (i = 0; i < n; ++i) acc = acc + x[i];
            Y[p] = acc / n;
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Level-3 routines that sit on GEMM: symm, syrk, trmm, trsm, row-major, float.
 *
 * dlf's CPU path hands float operands to cblas_ssymm / cblas_ssyrk / cblas_strmm / cblas_strsm
 * (dlf/include/tensor/linalg_detail.h:463-470, 546-552, 1265-1272, 1318-1323 over
 * dlf/include/cxxblas.h); for element types without a BLAS it evaluates the definitions below
 * itself (symv_up / symv_lo :365-399, syrk_serial :486-523, trmm_serial :720-812, trsm_serial).
 * Only the named triangle of A (symm, trmm, trsm) or of C (syrk) is read or written; with
 * Diagonal::Unit the diagonal of A is not read and counts as 1. `wide` = double accumulators.
 * Enumerators are gblas.h:110-114: Upper 121, Lower 122; NonUnit 131, Unit 132; Left 141, Right 142.
 * ------------------------------------------------------------------------------------------ */
enum { DLF_UPPER = 121, DLF_LOWER = 122, DLF_NON_UNIT = 131, DLF_UNIT = 132, DLF_LEFT = 141, DLF_RIGHT = 142 };

/* element (i, j) of the symmetric matrix whose `uplo` triangle is stored in A */
static float sym_at(const float* A, size_t lda, int uplo, size_t i, size_t j) {
    const int stored = uplo == DLF_UPPER ? (i <= j) : (i >= j);
    return stored ? A[i * lda + j] : A[j * lda + i];
}

/* element (i, j) of op(T), T the triangular matrix stored in the `uplo` triangle of A */
static float tri_at(const float* A, size_t lda, int uplo, int trans, int diag, size_t i, size_t j) {
    const size_t r = trans == DLF_NO_TRANS ? i : j, c = trans == DLF_NO_TRANS ? j : i;
    if (r == c) return diag == DLF_UNIT ? 1.0f : A[r * lda + c];
    if (uplo == DLF_UPPER ? (r < c) : (r > c)) return A[r * lda + c];
    return 0.0f;
}

void dlf_oracle_symm_f32(int side, int uplo, size_t m, size_t n, float alpha, const float* A, size_t lda,
                         const float* B, size_t ldb, float beta, float* C, size_t ldc, int wide) {
    long i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (long)m; ++i) {
        size_t j, l;
        for (j = 0; j < n; ++j) {
            double accd = 0.0;
            float accf = 0.0f;
            if (side == DLF_LEFT) {  /* C = alpha * S(m x m) * B + beta * C */
                for (l = 0; l < m; ++l) {
                    const float a = sym_at(A, lda, uplo, (size_t)i, l), b = B[l * ldb + j];
                    if (wide) accd += (double)a * (double)b; else accf += a * b;
                }
            } else {                 /* C = alpha * B * S(n x n) + beta * C */
                for (l = 0; l < n; ++l) {
                    const float b = B[(size_t)i * ldb + l], a = sym_at(A, lda, uplo, l, j);
                    if (wide) accd += (double)b * (double)a; else accf += b * a;
                }
            }
            float* c = C + (size_t)i * ldc + j;
            if (wide) *c = (float)((double)alpha * accd + (beta == 0.0f ? 0.0 : (double)beta * (double)*c));
            else *c = alpha * accf + (beta == 0.0f ? 0.0f : beta * *c);
        }
    }
}

/* C(uplo triangle) = alpha * op(A) * op(A)^T + beta * C; op(A) is n x k (A is n x k for NoTrans, k x n for Trans) */
void dlf_oracle_syrk_f32(int uplo, int trans, size_t n, size_t k, float alpha, const float* A, size_t lda,
                         float beta, float* C, size_t ldc, int wide) {
    long i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (long)n; ++i) {
        size_t j, l;
        for (j = 0; j < n; ++j) {
            if (!(uplo == DLF_UPPER ? ((size_t)i <= j) : ((size_t)i >= j))) continue;
            double accd = 0.0;
            float accf = 0.0f;
            for (l = 0; l < k; ++l) {
                const float a = trans == DLF_NO_TRANS ? A[(size_t)i * lda + l] : A[l * lda + (size_t)i];
                const float b = trans == DLF_NO_TRANS ? A[j * lda + l] : A[l * lda + j];
                if (wide) accd += (double)a * (double)b; else accf += a * b;
            }
            float* c = C + (size_t)i * ldc + j;
            if (wide) *c = (float)((double)alpha * accd + (beta == 0.0f ? 0.0 : (double)beta * (double)*c));
            else *c = alpha * accf + (beta == 0.0f ? 0.0f : beta * *c);
        }
    }
}

/* B = alpha * op(T) * B (Left, T is m x m) or alpha * B * op(T) (Right, T is n x n), in place */
void dlf_oracle_trmm_f32(int side, int uplo, int trans, int diag, size_t m, size_t n, float alpha,
                         const float* A, size_t lda, float* B, size_t ldb, int wide) {
    float* out = (float*)malloc(m * n * sizeof(float));
    long i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (long)m; ++i) {
        size_t j, l;
        for (j = 0; j < n; ++j) {
            double accd = 0.0;
            float accf = 0.0f;
            if (side == DLF_LEFT) {
                for (l = 0; l < m; ++l) {
                    const float t = tri_at(A, lda, uplo, trans, diag, (size_t)i, l), b = B[l * ldb + j];
                    if (wide) accd += (double)t * (double)b; else accf += t * b;
                }
            } else {
                for (l = 0; l < n; ++l) {
                    const float b = B[(size_t)i * ldb + l], t = tri_at(A, lda, uplo, trans, diag, l, j);
                    if (wide) accd += (double)b * (double)t; else accf += b * t;
                }
            }
            out[(size_t)i * n + j] = wide ? (float)((double)alpha * accd) : alpha * accf;
        }
    }
    {
        size_t r, c;
        for (r = 0; r < m; ++r)
            for (c = 0; c < n; ++c) B[r * ldb + c] = out[r * n + c];
    }
    free(out);
}

/* Solves op(T) * X = alpha * B (Left) or X * op(T) = alpha * B (Right) by substitution; X overwrites B. */
void dlf_oracle_trsm_f32(int side, int uplo, int trans, int diag, size_t m, size_t n, float alpha,
                         const float* A, size_t lda, float* B, size_t ldb, int wide) {
    /* op(T) is lower triangular when (Lower, NoTrans) or (Upper, Trans) */
    const int eff_lower = (uplo == DLF_LOWER) == (trans == DLF_NO_TRANS);
    if (side == DLF_LEFT) {
        long j;
#pragma omp parallel for schedule(static)
        for (j = 0; j < (long)n; ++j) {  /* columns of B are independent systems */
            size_t s, l;
            double* x = (double*)malloc(m * sizeof(double));
            for (s = 0; s < m; ++s) {
                const size_t i = eff_lower ? s : m - 1 - s;
                double acc = (double)alpha * (double)B[i * ldb + (size_t)j];
                float accf = alpha * B[i * ldb + (size_t)j];
                for (l = 0; l < s; ++l) {
                    const size_t c = eff_lower ? l : m - 1 - l;
                    const float t = tri_at(A, lda, uplo, trans, diag, i, c);
                    acc -= (double)t * x[c];
                    accf -= t * (float)x[c];
                }
                {
                    const float d = tri_at(A, lda, uplo, trans, diag, i, i);
                    x[i] = wide ? acc / (double)d : (double)(accf / d);
                }
            }
            for (s = 0; s < m; ++s) B[s * ldb + (size_t)j] = (float)x[s];
            free(x);
        }
    } else {
        long i;
#pragma omp parallel for schedule(static)
        for (i = 0; i < (long)m; ++i) {  /* rows of B are independent systems: x * op(T) = alpha * b */
            size_t s, l;
            double* x = (double*)malloc(n * sizeof(double));
            float* b = B + (size_t)i * ldb;
            for (s = 0; s < n; ++s) {
                /* x_j needs x_l for the l with op(T)(l, j) != 0, l != j: l < j when op(T) is upper */
                const size_t j = eff_lower ? n - 1 - s : s;
                double acc = (double)alpha * (double)b[j];
                float accf = alpha * b[j];
                for (l = 0; l < s; ++l) {
                    const size_t r = eff_lower ? n - 1 - l : l;
                    const float t = tri_at(A, lda, uplo, trans, diag, r, j);
                    acc -= x[r] * (double)t;
                    accf -= (float)x[r] * t;
                }
                {
                    const float d = tri_at(A, lda, uplo, trans, diag, j, j);
                    x[j] = wide ? acc / (double)d : (double)(accf / d);
                }
            }
            for (s = 0; s < n; ++s) b[s] = (float)x[s];
            free(x);
        }
    }
}

// Helper kernels of the level-3 routines that sit on the GEMM main loop (symm, syrk, trmm, trsm).
//
// The reference's GPU versions of these routines (CLBlast-derived Xsymm / Xsyrk / Xtrmm / Xtrsm
// behind gpgpu/include/gblas.h:506-586) do the same thing this file does: the triangular or
// symmetric operand is first written out as a general square matrix, the product then runs on
// the GEMM kernel, and trsm is a blocked substitution whose off-diagonal updates are GEMMs. The
// kernels here are the memory-bound pieces of that scheme; all of them take row-major operands
// (element (i, j) at i*ld + j) - a column-major call is the row-major call with the side, the
// triangle and (syrk) the transposition flipped, which the host code does.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace dlfb200 {

template <typename T> __device__ __forceinline__ float l3_load(const T* p) { return static_cast<float>(*p); }
template <> __device__ __forceinline__ float l3_load<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float l3_load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ T l3_make(float v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __half l3_make<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 l3_make<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// dst (n x n, ld = n) = the full matrix that the `upper`/lower triangle of src stands for:
// symmetric (mirror the stored triangle) or triangular (zero elsewhere; `unit`: diagonal = 1).
template <typename T>
__global__ void l3_expand_square_kernel(T* __restrict__ dst, const T* __restrict__ src, long long ld, int n,
                                        int symmetric, int upper, int unit) {
    const long long total = static_cast<long long>(n) * n;
    for (long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; id < total;
         id += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int i = static_cast<int>(id / n);
        const int j = static_cast<int>(id - static_cast<long long>(i) * n);
        const bool stored = upper ? (i <= j) : (i >= j);
        T v;
        if (i == j && unit) v = l3_make<T>(1.0f);
        else if (stored) v = src[i * ld + j];
        else if (symmetric) v = src[j * ld + i];
        else v = l3_make<T>(0.0f);
        dst[id] = v;
    }
}

// syrk: the named triangle of C = S + beta * C, S (n x n, ld = n) holding alpha * op(A) op(A)^T;
// the other triangle of C is not touched. beta == 0 does not read C.
template <typename T>
__global__ void l3_triangle_merge_kernel(T* __restrict__ c, long long ldc, const T* __restrict__ s, int n, int upper,
                                         float beta) {
    const long long total = static_cast<long long>(n) * n;
    for (long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; id < total;
         id += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int i = static_cast<int>(id / n);
        const int j = static_cast<int>(id - static_cast<long long>(i) * n);
        if (!(upper ? (i <= j) : (i >= j))) continue;
        float v = l3_load(s + id);
        if (beta != 0.0f) v += beta * l3_load(c + i * ldc + j);
        c[i * ldc + j] = l3_make<T>(v);
    }
}

// B (m x n) *= alpha
template <typename T>
__global__ void l3_scale_kernel(T* __restrict__ b, long long ldb, int m, int n, float alpha) {
    const long long total = static_cast<long long>(m) * n;
    for (long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; id < total;
         id += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int i = static_cast<int>(id / n);
        const int j = static_cast<int>(id - static_cast<long long>(i) * n);
        b[i * ldb + j] = l3_make<T>(alpha * l3_load(b + i * ldb + j));
    }
}

// K-split GEMM: D[i + j*ldd] = alpha * sum_s part[s][i + j*M] + beta * D[i + j*ldd] over the M x N
// window (i contiguous); `part` holds `slices` fp32 products of M*N elements each.
template <typename T>
__global__ void splitk_reduce_kernel(T* __restrict__ d, long long ldd, const float* __restrict__ part, int M, int N,
                                     int slices, float alpha, float beta) {
    const long long total = static_cast<long long>(M) * N;
    for (long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; id < total;
         id += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int j = static_cast<int>(id / M);
        const int i = static_cast<int>(id - static_cast<long long>(j) * M);
        float acc = 0.0f;
        for (int s = 0; s < slices; ++s) acc += part[s * total + id];
        float v = alpha * acc;
        T* o = d + j * ldd + i;
        if (beta != 0.0f) v += beta * l3_load(o);
        *o = l3_make<T>(v);
    }
}

constexpr int kTrsmBlock = 64;     // order of a diagonal block
constexpr int kTrsmThreads = 128;  // independent systems per CTA

// Diagonal block of the blocked substitution: nb <= 64 unknowns per system, one thread per system.
// Left  (right_side = 0): op(T)(nb x nb) * X = B, the systems are the `nsys` columns of the nb x nsys block at b
//                         (unknown r of system t at b[r*ldb + t]);
// Right (right_side = 1): X * op(T) = B, the systems are the `nsys` rows of the nsys x nb block at b
//                         (unknown r of system t at b[t*ldb + r]).
// `a` addresses T's diagonal block (row-major, lda); `trans` applies op; `lower` / `unit` describe T as stored.
template <typename T>
__global__ void __launch_bounds__(kTrsmThreads)
    l3_trsm_diag_kernel(const T* __restrict__ a, long long lda, int trans, int lower, int unit, int right_side, int nb,
                        T* __restrict__ b, long long ldb, int nsys) {
    __shared__ float coef[kTrsmBlock][kTrsmBlock];  // coef[eq][var]; read as a broadcast, so no padding
    __shared__ float xs[kTrsmBlock][kTrsmThreads];
    // coefficient of unknown `var` in equation `eq`: Left op(T)(eq, var); Right op(T)(var, eq)
    for (int id = threadIdx.x; id < nb * nb; id += blockDim.x) {
        const int eq = id / nb, var = id - eq * nb;
        int r = right_side ? var : eq, c = right_side ? eq : var;  // element (r, c) of op(T)
        if (trans) {
            const int t = r;
            r = c;
            c = t;
        }
        float v;
        if (r == c) v = unit ? 1.0f : l3_load(a + r * lda + c);
        else if (lower ? (r > c) : (r < c)) v = l3_load(a + r * lda + c);
        else v = 0.0f;
        coef[eq][var] = v;
    }
    __syncthreads();
    // the coefficient matrix is lower triangular (forward substitution) when op(T) is lower for
    // the left side, upper for the right side
    const bool op_lower = (lower != 0) != (trans != 0);
    const bool forward = right_side ? !op_lower : op_lower;
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nsys) return;
    T* bt = right_side ? b + static_cast<long long>(t) * ldb : b + t;
    const long long step = right_side ? 1 : ldb;
    for (int s = 0; s < nb; ++s) {
        const int eq = forward ? s : nb - 1 - s;
        float acc = l3_load(bt + eq * step);
        for (int l = 0; l < s; ++l) {
            const int var = forward ? l : nb - 1 - l;
            acc -= coef[eq][var] * xs[var][threadIdx.x];
        }
        xs[eq][threadIdx.x] = acc / coef[eq][eq];
    }
    for (int r = 0; r < nb; ++r) bt[r * step] = l3_make<T>(xs[r][threadIdx.x]);
}

}  // namespace dlfb200

// Epilogue shared by the contraction kernels: one warp owns 32 TMEM lanes (32 consecutive
// values of the output's contiguous index i) and walks the tile's columns 32 at a time.
// For every column j the warp writes 32 consecutive output elements, so stores and the
// optional reads of C (beta != 0) are fully coalesced without staging.
//
// The per-element work is kept to a multiply-add, a conversion and a store: alpha / beta /
// bias / output-format decisions are taken once per tile (template parameters), addresses
// advance by a constant stride, and interior chunks run without bounds checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace dlfb200 {

enum : int { OUT_F32 = 0, OUT_F16 = 1, OUT_BF16 = 2 };

template <int OUT>
__device__ __forceinline__ void out_store(char* ptr, float v) {
    if constexpr (OUT == OUT_F32) {
        *reinterpret_cast<float*>(ptr) = v;
    } else if constexpr (OUT == OUT_F16) {
        *reinterpret_cast<__half*>(ptr) = __float2half_rn(v);
    } else {
        *reinterpret_cast<__nv_bfloat16*>(ptr) = __float2bfloat16_rn(v);
    }
}
template <int OUT>
__device__ __forceinline__ float out_load(const char* ptr) {
    if constexpr (OUT == OUT_F32) {
        return *reinterpret_cast<const float*>(ptr);
    } else if constexpr (OUT == OUT_F16) {
        return __half2float(*reinterpret_cast<const __half*>(ptr));
    } else {
        return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(ptr));
    }
}

// Fused extras of the convolution epilogue: `rdelta` is the byte distance from an element of D to
// the element of the residual tensor added to it (0: the beta term reads D itself), `relu` clamps
// the result at zero before it is stored.
struct EpiExtra {
    long long rdelta = 0;
    bool relu = false;
};

// One 32-column chunk. `ptr` addresses D(i, j0) for this lane's row i; consecutive columns are
// `stride` bytes apart. `ncols` (1..32) columns of the chunk exist; `row_ok` says whether this
// lane's row exists. `bias` addresses bias[j0] (storage type) and is only read when HAS_BIAS.
// `pair_ok` (16-bit outputs, beta == 0): this lane and its neighbour (lane ^ 1) hold rows that are
// adjacent in memory, both exist, and the even lane's element is 4-byte aligned in every column.
// Then the two lanes trade one value per column pair and each writes one 32-bit word (two rows of
// one column) instead of two 16-bit values: half the store instructions, 128 bytes per warp store.
template <int OUT, bool HAS_BETA, bool HAS_BIAS>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&v)[32], char* ptr, long long stride,
                                               int ncols, bool row_ok, float alpha, float beta,
                                               const char* bias, int lane, bool pair_ok = false,
                                               EpiExtra ex = EpiExtra()) {
    constexpr int OES = OUT == OUT_F32 ? 4 : 2;
    const char* cptr = ptr + ex.rdelta;  // where the beta term is read
    float bv = 0.0f;
    if constexpr (HAS_BIAS) {
        if (lane < ncols) bv = out_load<OUT>(bias + lane * OES);
    }
    if constexpr (OUT != OUT_F32 && !HAS_BETA) {
        if (ncols == 32 && __all_sync(0xffffffffu, pair_ok || !row_ok)) {
            const bool odd = lane & 1;
#pragma unroll
            for (int jj = 0; jj < 32; jj += 2) {
                float r0 = alpha * __uint_as_float(v[jj]);
                float r1 = alpha * __uint_as_float(v[jj + 1]);
                if constexpr (HAS_BIAS) {
                    r0 += __shfl_sync(0xffffffffu, bv, jj);
                    r1 += __shfl_sync(0xffffffffu, bv, jj + 1);
                }
                if (ex.relu) {
                    r0 = fmaxf(r0, 0.0f);
                    r1 = fmaxf(r1, 0.0f);
                }
                const float got = __shfl_xor_sync(0xffffffffu, odd ? r0 : r1, 1);
                // even lane: rows (i, i+1) of column jj; odd lane: rows (i-1, i) of column jj+1
                const float lo = odd ? got : r0;
                const float hi = odd ? r1 : got;
                uint32_t word;
                if constexpr (OUT == OUT_F16) {
                    const __half2 h = __floats2half2_rn(lo, hi);
                    word = *reinterpret_cast<const uint32_t*>(&h);
                } else {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                    word = *reinterpret_cast<const uint32_t*>(&h);
                }
                char* dst = odd ? ptr - 2 + (jj + 1) * stride : ptr + jj * stride;
                if (row_ok) *reinterpret_cast<uint32_t*>(dst) = word;
            }
            return;
        }
    }
    if (ncols == 32) {
        float c[HAS_BETA ? 32 : 1];
        if constexpr (HAS_BETA) {
            if (row_ok) {
#pragma unroll
                for (int jj = 0; jj < 32; ++jj) c[jj] = out_load<OUT>(cptr + jj * stride);
            } else {
#pragma unroll
                for (int jj = 0; jj < 32; ++jj) c[jj] = 0.0f;
            }
        }
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
            float r = alpha * __uint_as_float(v[jj]);
            if constexpr (HAS_BETA) r += beta * c[jj];
            if constexpr (HAS_BIAS) r += __shfl_sync(0xffffffffu, bv, jj);
            if (ex.relu) r = fmaxf(r, 0.0f);
            if (row_ok) out_store<OUT>(ptr + jj * stride, r);
        }
    } else {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
            float r = alpha * __uint_as_float(v[jj]);
            const bool ok = row_ok && jj < ncols;
            if constexpr (HAS_BETA) {
                if (ok) r += beta * out_load<OUT>(cptr + jj * stride);
            }
            if constexpr (HAS_BIAS) r += __shfl_sync(0xffffffffu, bv, jj);
            if (ex.relu) r = fmaxf(r, 0.0f);
            if (ok) out_store<OUT>(ptr + jj * stride, r);
        }
    }
}

// Epilogue of a convolution computed with the roles swapped: the lanes hold output channels and
// the columns are consecutive output pixels j = img * P + pp of an NCHW tensor, so one lane's
// columns are consecutive in memory and leave as vectors of G elements (G = 8, 4, 2 or 1: the
// largest that divides P and keeps every vector aligned; the caller guarantees that the chunk's
// first pixel and its column count are multiples of G, so a vector never crosses an image).
// `v`: 32 accumulator columns; `ncols` of them exist; (img, pp): image and pixel of column 0
// (warp-uniform); `rowoff` = channel * P for this lane; `img_stride` = channels * P (elements).
// The residual may be addressed differently from the destination (a destination staged in shared
// memory): element (img_r + images passed, rrowoff, pp) with image stride rimg_stride.
template <int OUT, int G>
__device__ __forceinline__ void epilogue_swapped_chunk(const uint32_t (&v)[32], int ncols, char* d, const char* resid,
                                                       long long rowoff, long long img_stride, int P, int img, int pp,
                                                       float alpha, float bv, bool relu, bool row_ok,
                                                       long long rrowoff, long long rimg_stride, int img_r) {
    static_assert(OUT == OUT_F16 || OUT == OUT_BF16, "16-bit outputs");
#pragma unroll
    for (int k = 0; k < 32 / G; ++k) {
        if (G * k < ncols) {
            while (pp >= P) {  // next image (warp-uniform)
                pp -= P;
                ++img;
                ++img_r;
            }
            const long long e = static_cast<long long>(img) * img_stride + rowoff + pp;
            const long long er = static_cast<long long>(img_r) * rimg_stride + rrowoff + pp;
            float r[G];
#pragma unroll
            for (int g = 0; g < G; ++g) r[g] = alpha * __uint_as_float(v[G * k + g]) + bv;
            if (resid != nullptr && row_ok) {
                if constexpr (G == 1) {
                    r[0] += out_load<OUT>(resid + er * 2);
                } else {
                    uint32_t w[G / 2];
                    if constexpr (G == 8) {
                        const uint4 u = *reinterpret_cast<const uint4*>(resid + er * 2);
                        w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w;
                    } else if constexpr (G == 4) {
                        const uint2 u = *reinterpret_cast<const uint2*>(resid + er * 2);
                        w[0] = u.x; w[1] = u.y;
                    } else {
                        w[0] = *reinterpret_cast<const uint32_t*>(resid + er * 2);
                    }
#pragma unroll
                    for (int g = 0; g < G / 2; ++g) {
                        if constexpr (OUT == OUT_F16) {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[g]));
                            r[2 * g] += f.x;
                            r[2 * g + 1] += f.y;
                        } else {
                            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[g]));
                            r[2 * g] += f.x;
                            r[2 * g + 1] += f.y;
                        }
                    }
                }
            }
            if (relu) {
#pragma unroll
                for (int g = 0; g < G; ++g) r[g] = fmaxf(r[g], 0.0f);
            }
            if (row_ok) {
                if constexpr (G == 1) {
                    out_store<OUT>(d + e * 2, r[0]);
                } else {
                    uint32_t w[G / 2];
#pragma unroll
                    for (int g = 0; g < G / 2; ++g) {
                        if constexpr (OUT == OUT_F16) {
                            const __half2 h = __floats2half2_rn(r[2 * g], r[2 * g + 1]);
                            w[g] = *reinterpret_cast<const uint32_t*>(&h);
                        } else {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * g], r[2 * g + 1]);
                            w[g] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    }
                    if constexpr (G == 8)
                        *reinterpret_cast<uint4*>(d + e * 2) = make_uint4(w[0], w[1], w[2], w[3]);
                    else if constexpr (G == 4)
                        *reinterpret_cast<uint2*>(d + e * 2) = make_uint2(w[0], w[1]);
                    else
                        *reinterpret_cast<uint32_t*>(d + e * 2) = w[0];
                }
            }
            pp += G;
        }
    }
}

// The same for planes of at least 32 pixels, where a chunk of 32 columns crosses at most one
// image boundary: no loop-carried state between the vectors, so the unrolled body is one
// independent multiply-add / convert / store group per vector. `d0` / `r0` address the element of
// column 0 in the destination / residual; columns from `split` on (a multiple of G, 32 or more when
// the chunk stays inside one image) belong to the next image, `d_jump` / `r_jump` bytes further.
template <int OUT, int G>
__device__ __forceinline__ void epilogue_swapped_chunk_fast(const uint32_t (&v)[32], int ncols, char* d0, const char* r0,
                                                            int split, long long d_jump, long long r_jump, float alpha,
                                                            float bv, bool relu, bool row_ok) {
    static_assert(OUT == OUT_F16 || OUT == OUT_BF16, "16-bit outputs");
    static_assert(G == 8 || G == 4 || G == 2, "vector stores");
#pragma unroll
    for (int k = 0; k < 32 / G; ++k) {
        const int c = G * k;
        if (c < ncols) {
            const bool next = c >= split;
            float r[G];
#pragma unroll
            for (int g = 0; g < G; ++g) r[g] = fmaf(alpha, __uint_as_float(v[c + g]), bv);
            if (r0 != nullptr && row_ok) {
                const char* rp = r0 + c * 2 + (next ? r_jump : 0);
                uint32_t w[G / 2];
                if constexpr (G == 8) {
                    const uint4 u = *reinterpret_cast<const uint4*>(rp);
                    w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w;
                } else if constexpr (G == 4) {
                    const uint2 u = *reinterpret_cast<const uint2*>(rp);
                    w[0] = u.x; w[1] = u.y;
                } else {
                    w[0] = *reinterpret_cast<const uint32_t*>(rp);
                }
#pragma unroll
                for (int g = 0; g < G / 2; ++g) {
                    if constexpr (OUT == OUT_F16) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[g]));
                        r[2 * g] += f.x;
                        r[2 * g + 1] += f.y;
                    } else {
                        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[g]));
                        r[2 * g] += f.x;
                        r[2 * g + 1] += f.y;
                    }
                }
            }
            uint32_t w[G / 2];
#pragma unroll
            for (int g = 0; g < G / 2; ++g) {
                const float a = relu ? fmaxf(r[2 * g], 0.0f) : r[2 * g];
                const float b = relu ? fmaxf(r[2 * g + 1], 0.0f) : r[2 * g + 1];
                if constexpr (OUT == OUT_F16) {
                    const __half2 h = __floats2half2_rn(a, b);
                    w[g] = *reinterpret_cast<const uint32_t*>(&h);
                } else {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                    w[g] = *reinterpret_cast<const uint32_t*>(&h);
                }
            }
            if (row_ok) {
                char* dp = d0 + c * 2 + (next ? d_jump : 0);
                if constexpr (G == 8)
                    *reinterpret_cast<uint4*>(dp) = make_uint4(w[0], w[1], w[2], w[3]);
                else if constexpr (G == 4)
                    *reinterpret_cast<uint2*>(dp) = make_uint2(w[0], w[1]);
                else
                    *reinterpret_cast<uint32_t*>(dp) = w[0];
            }
        }
    }
}

// Whether this lane and lane ^ 1 can share 32-bit stores (see epilogue_chunk): rows adjacent in
// memory, both present, column stride even and the even lane's first element 4-byte aligned.
__device__ __forceinline__ bool pair_store_ok(const char* ptr, long long rowbase, long long colstride,
                                              bool row_ok, int lane) {
    const long long other = __shfl_xor_sync(0xffffffffu, rowbase, 1);
    const bool other_ok = __shfl_xor_sync(0xffffffffu, row_ok ? 1 : 0, 1) != 0;
    const bool odd = lane & 1;
    const bool adjacent = odd ? (other == rowbase - 1) : (other == rowbase + 1);
    const uintptr_t even_addr = reinterpret_cast<uintptr_t>(ptr) - (odd ? 2 : 0);
    return row_ok && other_ok && adjacent && (colstride & 1) == 0 && (even_addr & 3u) == 0;
}

// All columns of one accumulator tile held in TMEM at `trow` (lane base and column base already
// applied). ncols_total = number of valid columns of this tile (<= BN).
// `part` (optional): this thread's row of fp32 partial sums of earlier K-chunks in shared memory,
// element of column j at part[j*128]; added to the accumulator before alpha is applied.
template <int OUT, bool HAS_BETA, bool HAS_BIAS>
__device__ __forceinline__ void epilogue_tile(uint32_t trow, int ncols_total, char* ptr,
                                              long long stride, bool row_ok, float alpha,
                                              float beta, const char* bias, int lane,
                                              const float* part = nullptr, bool pair_ok = false,
                                              EpiExtra ex = EpiExtra()) {
    constexpr int OES = OUT == OUT_F32 ? 4 : 2;
    for (int c0 = 0; c0 < ncols_total; c0 += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(trow + c0, v);
        ptx::tmem_ld_wait();
        if (part != nullptr) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
                if (c0 + jj < ncols_total) v[jj] = __float_as_uint(__uint_as_float(v[jj]) + part[(c0 + jj) * 128]);
        }
        const int nc = min(32, ncols_total - c0);
        epilogue_chunk<OUT, HAS_BETA, HAS_BIAS>(v, ptr + c0 * stride, stride, nc, row_ok, alpha,
                                                beta, HAS_BIAS ? bias + c0 * OES : nullptr, lane, pair_ok, ex);
    }
}

template <int OUT>
__device__ __forceinline__ void epilogue_dispatch(uint32_t trow, int ncols_total, char* ptr,
                                                  long long stride, bool row_ok, float alpha,
                                                  float beta, const char* bias, int lane,
                                                  const float* part = nullptr, bool pair_ok = false,
                                                  EpiExtra ex = EpiExtra()) {
    if (beta != 0.0f) {
        if (bias)
            epilogue_tile<OUT, true, true>(trow, ncols_total, ptr, stride, row_ok, alpha, beta, bias, lane, part, pair_ok, ex);
        else
            epilogue_tile<OUT, true, false>(trow, ncols_total, ptr, stride, row_ok, alpha, beta, bias, lane, part, pair_ok, ex);
    } else {
        if (bias)
            epilogue_tile<OUT, false, true>(trow, ncols_total, ptr, stride, row_ok, alpha, beta, bias, lane, part, pair_ok, ex);
        else
            epilogue_tile<OUT, false, false>(trow, ncols_total, ptr, stride, row_ok, alpha, beta, bias, lane, part, pair_ok, ex);
    }
}

// The four epilogue warps (threads 0-127 of the CTA) meet here; barrier 0 belongs to __syncthreads.
// Used where the warps hand a block of results to one thread that issues TMA stores for it.
__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int OUT>
__device__ __forceinline__ unsigned short to_bits16(float v) {
    if constexpr (OUT == OUT_F16) return __half_as_ushort(__float2half_rn(v));
    else return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// Adds (or, for the first chunk, stores) one finished K-chunk accumulator to the running fp32
// sums in shared memory. The tensor core truncates when it adds into its fp32 accumulator, a
// bias that grows linearly with the number of accumulation steps (about 6e-9 * K relative for
// 3xTF32); summing short chunks with round-to-nearest adds on the CUDA cores keeps it bounded.
__device__ __forceinline__ void drain_chunk(uint32_t trow, int ncols, float* part, bool first) {
    for (int c0 = 0; c0 < ncols; c0 += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(trow + c0, v);
        ptx::tmem_ld_wait();
        // ncols need not be a multiple of 32 (row form: taps x channels, e.g. 7 x 16 = 112): the
        // sum array has exactly ncols rows
        if (first) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
                if (c0 + jj < ncols) part[(c0 + jj) * 128] = __uint_as_float(v[jj]);
        } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
                if (c0 + jj < ncols) part[(c0 + jj) * 128] += __uint_as_float(v[jj]);
        }
    }
}

}  // namespace dlfb200

// NCHW pooling (max / average) and the plane reduction used for global pooling.
//
// These are HBM-bound: every input element is needed once (windows overlap only inside a few
// rows, which the L1/L2 absorb) and every output element is written once. One thread produces
// `VEC` horizontally adjacent outputs of one plane row so that 16-bit outputs leave as one
// 32-bit store; threads of a warp cover consecutive outputs, so loads of a tap are consecutive
// (stride_w apart) addresses. Arithmetic follows dlf's CPU pooling
// (dlf/include/tensor/dnn_detail.h:172-227): max starts from the type's lowest value, the average
// divides the sum of the taps inside the image by their count, or by kernel_h*kernel_w with
// count_include_pad; a window that lies entirely in the padding gives lowest / 0/0 as there.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cfloat>
#include <cstdint>
#include <type_traits>

#include "epilogue.cuh"

namespace dlfb200 {

struct PoolParams {
    long long planes;  // batches * channels
    int toh;           // pool2d_rows_kernel: output rows per block
    int ih_rows;       // ... and input rows staged for them
    int group;         // pool_planes_kernel: threads per plane (power of two)
    int ablate;        // measurement aid: 1 skip the staging loads, 2 skip the window evaluation
    int H, W, OH, OW, KH, KW, pad_t, pad_l, sh, sw, dh, dw;
    int mode;               // 0 max, 1 average
    int count_include_pad;  // average only
    const char* x;
    char* y;
};

template <typename T>
struct PoolType;
template <>
struct PoolType<float> {
    static __device__ __forceinline__ float load(const char* p, long long i) { return reinterpret_cast<const float*>(p)[i]; }
    static __device__ __forceinline__ void store(char* p, long long i, float v) { reinterpret_cast<float*>(p)[i] = v; }
    static __device__ __forceinline__ float lowest() { return -FLT_MAX; }
    static __device__ __forceinline__ float round(float v) { return v; }
};
template <>
struct PoolType<__half> {
    static __device__ __forceinline__ float load(const char* p, long long i) { return __half2float(reinterpret_cast<const __half*>(p)[i]); }
    static __device__ __forceinline__ void store(char* p, long long i, float v) { reinterpret_cast<__half*>(p)[i] = __float2half_rn(v); }
    static __device__ __forceinline__ float lowest() { return -65504.0f; }
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};
template <>
struct PoolType<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const char* p, long long i) { return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]); }
    static __device__ __forceinline__ void store(char* p, long long i, float v) { reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float lowest() { return -3.38953139e38f; }
    static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// One thread = one output element; consecutive threads = consecutive ow, then oh, then plane.
template <typename T>
__global__ void __launch_bounds__(256) pool2d_kernel(const PoolParams p) {
    const long long per_plane = static_cast<long long>(p.OH) * p.OW;
    const long long total = p.planes * per_plane;
    for (long long o = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; o < total;
         o += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long plane = o / per_plane;
        const int rem = static_cast<int>(o - plane * per_plane);
        const int oh = rem / p.OW;
        const int ow = rem - oh * p.OW;
        const long long xbase = plane * p.H * p.W;
        const int ih0 = oh * p.sh - p.pad_t;
        const int iw0 = ow * p.sw - p.pad_l;
        float acc = p.mode == 0 ? PoolType<T>::lowest() : 0.0f;
        int count = 0;
        for (int kh = 0; kh < p.KH; ++kh) {
            const int ih = ih0 + kh * p.dh;
            if (static_cast<unsigned>(ih) >= static_cast<unsigned>(p.H)) continue;
            const long long row = xbase + static_cast<long long>(ih) * p.W;
            for (int kw = 0; kw < p.KW; ++kw) {
                const int iw = iw0 + kw * p.dw;
                if (static_cast<unsigned>(iw) >= static_cast<unsigned>(p.W)) continue;
                const float v = PoolType<T>::load(p.x, row + iw);
                acc = p.mode == 0 ? fmaxf(acc, v) : acc + v;  // fp32 sum, taps in (kh, kw) order
                ++count;
            }
        }
        if (p.mode == 1) {
            if (p.count_include_pad) count = p.KH * p.KW;
            acc = acc / static_cast<float>(count);
        }
        PoolType<T>::store(p.y, o, acc);
    }
}

// Windowed pooling through shared memory. A block owns `toh` consecutive output rows of one
// plane: the input rows they need are copied in once, with 16-byte loads when the rows are
// 16-byte multiples (every row then starts aligned), and all taps are read from shared memory.
// HBM sees each input row once per block (rows shared by two neighbouring blocks twice).
template <typename T, int K>
__global__ void __launch_bounds__(256) pool2d_rows_kernel(const PoolParams p) {
    extern __shared__ __align__(16) unsigned char pool_smem[];
    constexpr int ES = sizeof(T);
    const int tiles = (p.OH + p.toh - 1) / p.toh;
    const long long nblocks = p.planes * tiles;
    const int row_bytes = p.W * ES;
    const bool vec = (row_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0;
    for (long long blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
        const long long plane = blk / tiles;
        const int oh0 = static_cast<int>(blk - plane * tiles) * p.toh;
        const int ih_lo = oh0 * p.sh - p.pad_t;
        const char* xp = p.x + plane * p.H * static_cast<long long>(row_bytes);
        __syncthreads();  // the previous tile's readers are done
        if (p.ablate & 1) {
        } else if (vec) {
            const int cpr = row_bytes >> 4;  // 16-byte chunks per row
            for (int id = threadIdx.x; id < p.ih_rows * cpr; id += blockDim.x) {
                const int r = id / cpr;
                const int c = id - r * cpr;
                const int ih = ih_lo + r;
                if (static_cast<unsigned>(ih) < static_cast<unsigned>(p.H))
                    reinterpret_cast<uint4*>(pool_smem)[id] =
                        reinterpret_cast<const uint4*>(xp + static_cast<long long>(ih) * row_bytes)[c];
            }
        } else {
            for (int id = threadIdx.x; id < p.ih_rows * p.W; id += blockDim.x) {
                const int r = id / p.W;
                const int ih = ih_lo + r;
                if (static_cast<unsigned>(ih) < static_cast<unsigned>(p.H))
                    reinterpret_cast<T*>(pool_smem)[id] =
                        reinterpret_cast<const T*>(xp)[static_cast<long long>(ih) * p.W + (id - r * p.W)];
            }
        }
        __syncthreads();
        // Each thread produces two horizontally adjacent outputs (one 32-bit store for 16-bit
        // types when the pair is aligned). Windows that lie inside the image - all but the border
        // ones - run without bounds tests, fully unrolled when the window is the compile-time K x K.
        const int rows = min(p.toh, p.OH - oh0);
        const int pairs_per_row = (p.OW + 1) >> 1;
        const int kh_n = K ? K : p.KH, kw_n = K ? K : p.KW;
        for (int id = threadIdx.x; id < ((p.ablate & 2) ? 0 : rows * pairs_per_row); id += blockDim.x) {
            const int ohl = id / pairs_per_row;
            const int ow0 = (id - ohl * pairs_per_row) * 2;
            const int r0 = ohl * p.sh;  // first staged row of the window
            const bool rows_in = ih_lo + r0 >= 0 && ih_lo + r0 + (kh_n - 1) * p.dh < p.H;
            float res[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int ow = ow0 + e;
                const int iw0 = ow * p.sw - p.pad_l;
                float acc = p.mode == 0 ? PoolType<T>::lowest() : 0.0f;
                int count = 0;
                if (ow >= p.OW) {
                    res[e] = 0.0f;
                    continue;
                }
                if (rows_in && iw0 >= 0 && iw0 + (kw_n - 1) * p.dw < p.W) {
                    const char* s0 = reinterpret_cast<const char*>(pool_smem) + static_cast<long long>(r0) * row_bytes;
                    if (K) {
                        // K x K window, no dilation: constant offsets from one pointer
                        const char* b0 = s0 + iw0 * ES;
#pragma unroll
                        for (int kh = 0; kh < (K ? K : 1); ++kh) {
                            const char* rp = b0 + kh * row_bytes;
#pragma unroll
                            for (int kw = 0; kw < (K ? K : 1); ++kw) {
                                const float v = PoolType<T>::load(rp, kw);
                                acc = p.mode == 0 ? fmaxf(acc, v) : acc + v;
                            }
                        }
                    } else {
                        for (int kh = 0; kh < kh_n; ++kh)
                            for (int kw = 0; kw < kw_n; ++kw) {
                                const float v = PoolType<T>::load(s0 + static_cast<long long>(kh * p.dh) * row_bytes, iw0 + kw * p.dw);
                                acc = p.mode == 0 ? fmaxf(acc, v) : acc + v;
                            }
                    }
                    count = kh_n * kw_n;
                } else {
                    for (int kh = 0; kh < kh_n; ++kh) {
                        const int r = r0 + kh * p.dh;
                        if (static_cast<unsigned>(ih_lo + r) >= static_cast<unsigned>(p.H)) continue;
                        const char* srow = reinterpret_cast<const char*>(pool_smem) + static_cast<long long>(r) * row_bytes;
                        for (int kw = 0; kw < kw_n; ++kw) {
                            const int iw = iw0 + kw * p.dw;
                            if (static_cast<unsigned>(iw) >= static_cast<unsigned>(p.W)) continue;
                            const float v = PoolType<T>::load(srow, iw);
                            acc = p.mode == 0 ? fmaxf(acc, v) : acc + v;
                            ++count;
                        }
                    }
                }
                if (p.mode == 1) {
                    if (p.count_include_pad) count = kh_n * kw_n;
                    acc = acc / static_cast<float>(count);
                }
                res[e] = acc;
            }
            const long long o = (plane * p.OH + oh0 + ohl) * p.OW + ow0;
            if (sizeof(T) == 2 && ow0 + 1 < p.OW && ((o & 1) == 0) && (reinterpret_cast<uintptr_t>(p.y) & 3u) == 0) {
                T pair[2];
                PoolType<T>::store(reinterpret_cast<char*>(pair), 0, res[0]);
                PoolType<T>::store(reinterpret_cast<char*>(pair), 1, res[1]);
                reinterpret_cast<uint32_t*>(p.y)[o >> 1] = *reinterpret_cast<const uint32_t*>(pair);
            } else {
                PoolType<T>::store(p.y, o, res[0]);
                if (ow0 + 1 < p.OW) PoolType<T>::store(p.y, o + 1, res[1]);
            }
        }
    }
}

__device__ __forceinline__ __half __high2half_or_bf16(__half2 v) { return __high2half(v); }
__device__ __forceinline__ __half __low2half_or_bf16(__half2 v) { return __low2half(v); }
__device__ __forceinline__ __nv_bfloat16 __high2half_or_bf16(__nv_bfloat162 v) { return __high2bfloat16(v); }
__device__ __forceinline__ __nv_bfloat16 __low2half_or_bf16(__nv_bfloat162 v) { return __low2bfloat16(v); }
template <typename T, typename T2>
__device__ __forceinline__ T2 pool_make2(T lo, T hi);
template <>
__device__ __forceinline__ __half2 pool_make2<__half, __half2>(__half lo, __half hi) { return __halves2half2(lo, hi); }
template <>
__device__ __forceinline__ __nv_bfloat162 pool_make2<__nv_bfloat16, __nv_bfloat162>(__nv_bfloat16 lo, __nv_bfloat16 hi) {
    return __halves2bfloat162(lo, hi);
}

// The pooling layer of ResNet-style stems - max, 3 x 3, stride 2, one column of left padding,
// 16-bit storage, rows that are multiples of eight elements - without per-tap work: a thread owns
// eight consecutive outputs of one row. Per input row it loads the three 16-byte vectors that
// hold columns 16j-8 .. 16j+15, takes the vertical maximum on packed pairs (two values per
// instruction), and forms each output from one odd column and one packed pair:
//     out[t] = max(x[16j-1+2t], x[16j+2t], x[16j+1+2t]),   t = 0..7.
// About ten instructions per output instead of about two hundred in the generic kernel.
// Vectors outside the image (first strip of a row, rows of the vertical padding) count as the
// type's lowest value, exactly as taps outside the image do in the reference.
template <typename T2>
__device__ __forceinline__ T2 pool_bits_as(uint32_t v) {
    return *reinterpret_cast<const T2*>(&v);
}
template <typename T2>
__device__ __forceinline__ uint32_t pool_as_bits(T2 v) {
    return *reinterpret_cast<const uint32_t*>(&v);
}
template <typename T, typename T2>
__global__ void __launch_bounds__(256) maxpool3s2_strip_kernel(const PoolParams p, const uint32_t lowest2) {
    const int spr = p.OW >> 3;  // strips per output row
    const long long rows_total = p.planes * p.OH;
    const long long total = rows_total * spr;
    const int vpr = p.W >> 3;  // 16-byte vectors per input row
    for (long long sid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; sid < total;
         sid += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long orow = sid / spr;  // plane * OH + oh
        const int j = static_cast<int>(sid - orow * spr);
        const long long plane = orow / p.OH;
        const int oh = static_cast<int>(orow - plane * p.OH);
        const uint4* xrow0 = reinterpret_cast<const uint4*>(p.x) + plane * p.H * vpr;
        // packed vertical maxima of columns 16j-8 .. 16j+15 (12 pairs)
        uint32_t v[12];
#pragma unroll
        for (int k = 0; k < 12; ++k) v[k] = lowest2;
#pragma unroll
        for (int kh = 0; kh < 3; ++kh) {
            const int ih = oh * 2 - p.pad_t + kh;
            if (static_cast<unsigned>(ih) >= static_cast<unsigned>(p.H)) continue;
            const uint4* xr = xrow0 + static_cast<long long>(ih) * vpr;
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const int vi = 2 * j - 1 + q;  // vector index inside the row
                if (static_cast<unsigned>(vi) >= static_cast<unsigned>(vpr)) continue;
                const uint4 w = xr[vi];
                v[4 * q + 0] = pool_as_bits(__hmax2(pool_bits_as<T2>(v[4 * q + 0]), pool_bits_as<T2>(w.x)));
                v[4 * q + 1] = pool_as_bits(__hmax2(pool_bits_as<T2>(v[4 * q + 1]), pool_bits_as<T2>(w.y)));
                v[4 * q + 2] = pool_as_bits(__hmax2(pool_bits_as<T2>(v[4 * q + 2]), pool_bits_as<T2>(w.z)));
                v[4 * q + 3] = pool_as_bits(__hmax2(pool_bits_as<T2>(v[4 * q + 3]), pool_bits_as<T2>(w.w)));
            }
        }
        // pair k holds columns 16j-8+2k, 16j-8+2k+1; output t needs the high half of pair 3+t
        // (column 16j-1+2t) and both halves of pair 4+t
        uint32_t out[4];
#pragma unroll
        for (int t = 0; t < 8; t += 2) {
            T r[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const T2 left = pool_bits_as<T2>(v[3 + t + e]);
                const T2 mid = pool_bits_as<T2>(v[4 + t + e]);
                r[e] = __hmax(__high2half_or_bf16(left), __hmax(__low2half_or_bf16(mid), __high2half_or_bf16(mid)));
            }
            out[t >> 1] = pool_as_bits(pool_make2<T, T2>(r[0], r[1]));
        }
        reinterpret_cast<uint4*>(p.y)[sid] = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// Global pooling of small planes (7 x 7, 14 x 14): a block copies the contiguous memory of
// 256 / group planes into shared memory with coalesced loads, then `group` neighbouring lanes
// reduce each plane and the block writes its results as one contiguous run.
template <typename T>
__global__ void __launch_bounds__(256) pool_planes_kernel(const PoolParams p) {
    extern __shared__ __align__(16) unsigned char pool_smem[];
    constexpr int ES = sizeof(T);
    const int n = p.H * p.W;
    const int ppb = 256 / p.group;  // planes per block
    const long long nblocks = (p.planes + ppb - 1) / ppb;
    for (long long blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
        const long long plane0 = blk * ppb;
        const int np = static_cast<int>(min(static_cast<long long>(ppb), p.planes - plane0));
        const long long bytes = static_cast<long long>(np) * n * ES;
        const char* src = p.x + plane0 * n * ES;
        __syncthreads();
        // the block's range starts at a multiple of ppb*n*ES bytes: 16-byte aligned whenever
        // that product is (checked on the host); the tail is copied element by element
        const long long vbytes = ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) ? (bytes & ~15ll) : 0;
        for (long long o = threadIdx.x * 16ll; o < vbytes; o += 256 * 16)
            *reinterpret_cast<uint4*>(pool_smem + o) = *reinterpret_cast<const uint4*>(src + o);
        for (long long o = vbytes + threadIdx.x * ES; o < bytes; o += 256 * ES)
            *reinterpret_cast<T*>(pool_smem + o) = *reinterpret_cast<const T*>(src + o);
        __syncthreads();
        const int pl = threadIdx.x / p.group;
        const int sub = threadIdx.x - pl * p.group;
        float acc = p.mode == 0 ? PoolType<T>::lowest() : 0.0f;
        if (pl < np) {
            const char* sp = reinterpret_cast<const char*>(pool_smem) + static_cast<long long>(pl) * n * ES;
            for (int i = sub; i < n; i += p.group) {
                const float v = PoolType<T>::load(sp, i);
                acc = p.mode == 0 ? fmaxf(acc, v) : acc + v;
            }
        }
        for (int d = p.group >> 1; d > 0; d >>= 1) {
            const float o = __shfl_xor_sync(0xffffffffu, acc, d);
            acc = p.mode == 0 ? fmaxf(acc, o) : acc + o;
        }
        if (pl < np && sub == 0) PoolType<T>::store(p.y, plane0 + pl, p.mode == 0 ? acc : acc / static_cast<float>(n));
    }
}

// Global pooling: the window is the whole plane (no padding). One warp per plane, lanes stride
// through it (coalesced), fp32 partial results combined with shuffles.
template <typename T>
__global__ void __launch_bounds__(256) pool_plane_kernel(const PoolParams p) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    const int n = p.H * p.W;
    for (long long plane = warp; plane < p.planes; plane += warps) {
        const long long base = plane * n;
        float acc = p.mode == 0 ? PoolType<T>::lowest() : 0.0f;
        for (int i = lane; i < n; i += 32) {
            const float v = PoolType<T>::load(p.x, base + i);
            acc = p.mode == 0 ? fmaxf(acc, v) : acc + v;
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const float o = __shfl_xor_sync(0xffffffffu, acc, d);
            acc = p.mode == 0 ? fmaxf(acc, o) : acc + o;
        }
        if (lane == 0) PoolType<T>::store(p.y, plane, p.mode == 0 ? acc : acc / static_cast<float>(n));
    }
}

// Channels-last pooling: x (N, H, W, C), y (N, OH, OW, C), C a multiple of 8. One thread produces 8
// channels of one output pixel: every tap is one 16-byte load, consecutive threads take consecutive
// channel groups and then consecutive pixels, so a warp's loads of a tap are contiguous runs. Same
// arithmetic as the NCHW kernels above: fp32 accumulation in (kh, kw) order, max from the type's
// lowest value, the average divided by the taps inside the image or by KH * KW. A global pool is the
// window KH = H, KW = W.
struct PoolNhwc {
    int C8, H, W, OH, OW, KH, KW, pad_t, pad_l, sh, sw;
    int average, count_include_pad;
    long long total;  // N * OH * OW * C8
};

template <int OUT>
__global__ void __launch_bounds__(256) pool_nhwc_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, const PoolNhwc p) {
    static_assert(OUT == OUT_F16 || OUT == OUT_BF16, "16-bit types");
    using T = typename std::conditional<OUT == OUT_F16, __half, __nv_bfloat16>::type;
    for (long long o = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; o < p.total;
         o += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int cg = static_cast<int>(o % p.C8);
        long long r = o / p.C8;
        const int ow = static_cast<int>(r % p.OW);
        r /= p.OW;
        const int oh = static_cast<int>(r % p.OH);
        const long long img = r / p.OH;
        const int ih0 = oh * p.sh - p.pad_t;
        const int iw0 = ow * p.sw - p.pad_l;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = p.average ? 0.0f : PoolType<T>::lowest();
        int count = 0;
        for (int kh = 0; kh < p.KH; ++kh) {
            const int ih = ih0 + kh;
            if (static_cast<unsigned>(ih) >= static_cast<unsigned>(p.H)) continue;
            for (int kw = 0; kw < p.KW; ++kw) {
                const int iw = iw0 + kw;
                if (static_cast<unsigned>(iw) >= static_cast<unsigned>(p.W)) continue;
                const uint4 u = x[((img * p.H + ih) * p.W + iw) * p.C8 + cg];
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float2 f;
                    if constexpr (OUT == OUT_F16) f = __half22float2(*reinterpret_cast<const __half2*>(&w[g]));
                    else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[g]));
                    acc[2 * g] = p.average ? acc[2 * g] + f.x : fmaxf(acc[2 * g], f.x);
                    acc[2 * g + 1] = p.average ? acc[2 * g + 1] + f.y : fmaxf(acc[2 * g + 1], f.y);
                }
                ++count;
            }
        }
        if (p.average) {
            if (p.count_include_pad) count = p.KH * p.KW;
            const float d = static_cast<float>(count);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = acc[e] / d;
        }
        uint4 out;
        uint32_t* ow4 = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            if constexpr (OUT == OUT_F16) {
                const __half2 h = __floats2half2_rn(acc[2 * g], acc[2 * g + 1]);
                ow4[g] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * g], acc[2 * g + 1]);
                ow4[g] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        y[o] = out;
    }
}

}  // namespace dlfb200

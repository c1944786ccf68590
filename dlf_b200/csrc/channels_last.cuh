// Helper kernels of the channels-last route of a 16-bit convolution.
//
// The tensor-map unit can fetch the operand of an implicit-GEMM convolution by itself (im2col
// mode: one instruction brings the tile's 128 filter windows x 64 channels for one filter tap,
// zero-filled outside the image, already in the swizzled K-major layout tcgen05.mma reads), but
// only from a channels-last tensor. dlf's tensors are NCHW (gpgpu/include/gdnn.h:201-213), so the
// route starts with a transposing copy of the activations into caller scratch:
//
//   cl_pack_activations_kernel   X (N, C, H, W)  ->  X' (N, OH', OW', Cp)
//       general filters: OH' = H, OW' = W (the copy is the whole input);
//       1x1 filters without padding: OH' = OH, OW' = OW, only the pixels a stride > 1 keeps,
//       after which the convolution is a plain GEMM over X' (M = N*OH*OW rows of Cp channels).
//       Cp >= C is the channel count rounded up to a 16-byte multiple; the tail is zero.
//   cl_pack_filters_kernel       W (Cout, C, KH, KW) -> W' (Cout, KH*KW, Ck)
//       the filter bank with k ordered (tap, channel), Ck = C rounded up to the 64-channel
//       k-block, zero-padded, so that one k-block is one tap's channel block.
//
// Both are bound by memory traffic: |X| read + |X'| written, a few MB for the filters.
// X' must be 16-byte aligned (it is the base of a tensor map and written with 16-byte stores).
#pragma once
#include <cstdint>

namespace dlfb200 {

constexpr int kClTile = 64;  // pixels and channels per block of the transposing copy

// How a thread of the transposing copy fetches its 8 consecutive output pixels of one channel:
enum : int {
    CL_VEC8 = 8,     // kept pixels are contiguous and 16-byte aligned: one 16-byte load
    CL_VEC4 = 4,     // ... 8-byte aligned: two 8-byte loads
    CL_VEC2 = 2,     // ... 4-byte aligned: four 4-byte loads
    CL_FUNNEL = 1,   // contiguous, any alignment: aligned 4-byte loads and a 16-bit funnel shift
    CL_S2_VEC4 = 42, // every second pixel of a row, groups of 4 kept pixels from 16 aligned bytes
    CL_S2_VEC2 = 22, // ... groups of 2 kept pixels from 8 aligned bytes
    CL_ANY = 0,      // any strides: one 2-byte load per pixel
};

__device__ __forceinline__ uint32_t ld_u32(const uint16_t* p) { return *reinterpret_cast<const uint32_t*>(p); }

// grid: (pixel blocks of 64 over OH*OW, channel blocks of 64 over Cp, images); block: 256 threads.
// Output pixel p = oh*OW + ow of image img and channel c is x[(img*C + c)*plane + oh*sh*W + ow*sw]
// (a copy of the whole plane is passed as OH = 1, OW = plane, strides 1). `total` = elements of x.
// The 64 x 64 tile goes through shared memory as [channel][pixel] rows; ldmatrix with .trans hands
// each thread 8 consecutive channels of one pixel (four 8x8 matrices whose rows are picked so that
// a thread's four registers are channels 8j .. 8j+7), which leave as one 16-byte store.
template <int MODE>
__global__ void __launch_bounds__(256)
    cl_pack_activations_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ xp, int C, long long plane,
                               int W, int OH, int OW, int sh, int sw, int Cp, long long total) {
    __shared__ __align__(16) uint16_t tile[kClTile][kClTile + 8];  // 144-byte rows: ldmatrix rows fall in distinct banks
    const int t = threadIdx.x;
    const int p0 = blockIdx.x * kClTile;
    const int c0 = blockIdx.y * kClTile;
    const long long img = blockIdx.z;
    const int P = OH * OW;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int id = t + 256 * i;
        const int pc = id & 7;  // chunk of 8 pixels
        const int c = id >> 3;
        const int p = p0 + pc * 8;
        uint32_t v[4] = {0u, 0u, 0u, 0u};
        if (c0 + c < C && p < P) {
            const long long cbase = (img * C + c0 + c) * plane;
            const uint16_t* src = x + cbase;
            bool done = false;
            if constexpr (MODE == CL_VEC8 || MODE == CL_VEC4 || MODE == CL_VEC2 || MODE == CL_FUNNEL) {
                // dense copy: OH == 1, pixels p .. p+7 are consecutive elements
                if (p + 8 <= P) {
                    const uint16_t* q = src + p;
                    if constexpr (MODE == CL_VEC8) {
                        const uint4 u = *reinterpret_cast<const uint4*>(q);
                        v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
                        done = true;
                    } else if constexpr (MODE == CL_VEC4) {
                        const uint2 u0 = *reinterpret_cast<const uint2*>(q);
                        const uint2 u1 = *reinterpret_cast<const uint2*>(q + 4);
                        v[0] = u0.x; v[1] = u0.y; v[2] = u1.x; v[3] = u1.y;
                        done = true;
                    } else if constexpr (MODE == CL_VEC2) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) v[j] = ld_u32(q + 2 * j);
                        done = true;
                    } else {
                        if ((reinterpret_cast<uintptr_t>(q) & 3u) == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) v[j] = ld_u32(q + 2 * j);
                            done = true;
                        } else if (cbase + p >= 1 && cbase + p + 9 <= total) {  // both end words lie inside x
                            uint32_t w[5];
#pragma unroll
                            for (int j = 0; j < 5; ++j) w[j] = ld_u32(q - 1 + 2 * j);
#pragma unroll
                            for (int j = 0; j < 4; ++j) v[j] = __funnelshift_r(w[j], w[j + 1], 16);
                            done = true;
                        }
                    }
                }
            } else if constexpr (MODE == CL_S2_VEC4) {
                // OW % 4 == 0: groups of four kept pixels never cross a row
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int pg = p + 4 * g;
                    if (pg < P) {
                        const int oh = pg / OW;
                        const int ow = pg - oh * OW;
                        const uint4 u = *reinterpret_cast<const uint4*>(src + static_cast<long long>(oh) * sh * W + ow * 2);
                        v[2 * g] = __byte_perm(u.x, u.y, 0x5410);
                        v[2 * g + 1] = __byte_perm(u.z, u.w, 0x5410);
                    }
                }
                done = true;
            } else if constexpr (MODE == CL_S2_VEC2) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int pg = p + 2 * g;
                    if (pg < P) {
                        const int oh = pg / OW;
                        const int ow = pg - oh * OW;
                        const uint2 u = *reinterpret_cast<const uint2*>(src + static_cast<long long>(oh) * sh * W + ow * 2);
                        v[g] = __byte_perm(u.x, u.y, 0x5410);
                    }
                }
                done = true;
            }
            if (!done) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int pj = p + j;
                    uint32_t e = 0u;
                    if (pj < P) {
                        const int oh = pj / OW;
                        const int ow = pj - oh * OW;
                        e = src[static_cast<long long>(oh) * sh * W + static_cast<long long>(ow) * sw];
                    }
                    v[j >> 1] |= e << ((j & 1) * 16);
                }
            }
        }
        *reinterpret_cast<uint4*>(&tile[c][pc * 8]) = make_uint4(v[0], v[1], v[2], v[3]);
    }
    __syncthreads();
    const int warp = t >> 5, lane = t & 31;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int item = warp + 8 * i;
        const int pg8 = item & 7;  // group of 8 pixels
        const int ch = item >> 3;  // channels 0-31 or 32-63 of the tile
        const int m = lane >> 3, rr = lane & 7;  // this lane supplies row rr of matrix m
        const int crow = ch * 32 + 8 * (rr >> 1) + 2 * m + (rr & 1);
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(&tile[crow][pg8 * 8]));
        uint32_t d0, d1, d2, d3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
                     : "r"(addr));
        const int p = p0 + pg8 * 8 + (lane >> 2);
        const int c = c0 + ch * 32 + 8 * (lane & 3);
        if (p < P && c < Cp)  // Cp is a multiple of 8: a group of 8 channels is inside or outside as a whole
            *reinterpret_cast<uint4*>(xp + (img * P + p) * Cp + c) = make_uint4(d0, d1, d2, d3);
    }
}

// one thread per (output channel, input channel): its taps are adjacent in W (read once, through
// L1) and land in W' one tap plane apart, consecutive threads writing consecutive channels
__global__ void cl_pack_filters_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ wp, int Cout, int C,
                                       int taps, int Ck) {
    const long long total = static_cast<long long>(Cout) * Ck;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % Ck);
        const long long co = i / Ck;
        const uint16_t* src = w + (co * C + c) * taps;
        uint16_t* dst = wp + co * taps * Ck + c;
        for (int tap = 0; tap < taps; ++tap)
            dst[static_cast<long long>(tap) * Ck] = c < C ? src[tap] : static_cast<uint16_t>(0);
    }
}

// Filters over at most 4 input channels (an RGB stem). With so few channels a filter tap is 8
// bytes and the tap-by-tap loads above would spend a 64-channel k-block on 4 of them. Instead the
// copy interleaves two image rows, carries a zero border wide enough for every filter window and
// splits the pixels of a row into sw phases:
//     X'' (N, sw, J, OWp, 2, 4),
//     X''[n][ph][j][i][rr][c] = X[n][c][j*rstep + rr - pad_top][i*sw + ph - pad_left]
// (zero outside the image or for c >= C): 16 bytes per pixel, the pixels i*sw + ph that
// consecutive outputs i need for one filter tap are consecutive in memory, and so are the row
// pairs of one phase that a tile of output rows needs (OWp pixels per row, the tile's column count
// per output row). conv_small.cuh reads the overlapping filter windows straight out of a copy of
// such rows. Row pairs start at rows j*rstep:
// every row when the vertical stride is odd, every second row when it is even (only those are
// ever read). The filters are laid out to match: k-block kb covers filter rows 2*kb, 2*kb+1; its
// four 16-element k-steps are taps (m, m+1) of phase ph in the order ph = 0: m = 0, 2, ..; ph = 1:
// ..., i.e. filter columns kw = sw*(m + c) + ph for the step's chunk c, each chunk holding
// (kh & 1) * 4 + channel (zero for kw >= KW, channel >= C, kh >= KH).
__global__ void __launch_bounds__(256)
    cl_pack_small_activations_kernel(const uint16_t* __restrict__ x, uint4* __restrict__ xp, int C, int H, int W,
                                     int J, int OWp, int sw, int rstep, int pad_t, int pad_l, long long total) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int ii = static_cast<int>(i % OWp);
        long long r0 = i / OWp;
        const int j = static_cast<int>(r0 % J);
        r0 /= J;
        const int ph = static_cast<int>(r0 % sw);
        const long long n = r0 / sw;
        const int iw = ii * sw + ph - pad_l;
        uint32_t v[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (static_cast<unsigned>(iw) < static_cast<unsigned>(W)) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int ih = j * rstep + rr - pad_t;
                if (static_cast<unsigned>(ih) < static_cast<unsigned>(H)) {
                    const uint16_t* src = x + (n * C * H + ih) * W + iw;
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (c < C) v[rr * 4 + c] = src[static_cast<long long>(c) * H * W];
                }
            }
        }
        xp[i] = make_uint4(v[0] | (v[1] << 16), v[2] | (v[3] << 16), v[4] | (v[5] << 16), v[6] | (v[7] << 16));
    }
}

// one thread per element of W'' (Cout, KB, 64)
__global__ void cl_pack_small_filters_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ wp, int Cout,
                                             int C, int KH, int KW, int KB, int sw) {
    const long long total = static_cast<long long>(Cout) * KB * 64;
    const int tpp = 8 / sw;  // taps per phase
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int k = static_cast<int>(i & 63);
        const long long r = i >> 6;
        const int kb = static_cast<int>(r % KB);
        const long long co = r / KB;
        const int ks = k >> 4, c = (k >> 3) & 1, e = k & 7;
        const int ph = (2 * ks) / tpp, m = (2 * ks) % tpp;
        const int kw = sw * (m + c) + ph, kh = 2 * kb + (e >> 2), ch = e & 3;
        uint16_t v = 0;
        if (kh < KH && kw < KW && ch < C) v = w[((co * C + ch) * KH + kh) * KW + kw];
        wp[i] = v;
    }
}

}  // namespace dlfb200

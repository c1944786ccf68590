// Stride-1 convolution (16-bit, one group, channels a multiple of 64) as an implicit GEMM in which
// the activations are fetched ONCE per tile and every filter tap is a descriptor offset.
//
// Roles are swapped as in conv_small.cuh: the 128 tensor-memory lanes are output channels, the
// columns are R output rows of one image, Wp = OW + KW - 1 columns per row (the last KW - 1 columns
// of a row are not outputs). The activations come from a bordered copy in channel-group-major order,
//     X^ (N, C/8, Hp, Wp, 8),  X^[n][g][r][q][e] = X[n][8g + e][r - pad_top][q - pad_left]  (zero outside),
// Hp = OH + KH - 1: 16 bytes per pixel and channel group, the pixels of a row - and the rows - of a
// group consecutive. A tile needs rows oh0 .. oh0 + R + KH - 2 of every group: one bulk copy per
// group lands them in shared memory as they are. In the unswizzled K-major operand layout row n of
// a core matrix lies 16 bytes after row n - 1, so with the halo positions as rows, column
// n = r * Wp + ow of the tile and filter tap (kh, kw) is halo position n + kh * Wp + kw: the operand
// of a tap is the same shared memory read from a start address (kh * Wp + kw) * 16 bytes further,
// and the two 8-channel k-chunks of a UMMA lie one group (the descriptor's leading-dimension offset)
// apart. Against the im2col-mode route (every activation fetched KH * KW times from L2) the
// operand traffic of a 3x3 layer drops ninefold; what remains per tile is the filter bank
// (KH * KW * C/64 tiles of 16 KB through a ring) and the halo (R + KH - 1 rows).
//
// Warp roles: 0-3 and 6-17 epilogue (four sets, as in conv_small.cuh), 4 UMMA issuer and TMEM
// owner, 5 copy producer. All waits are bounded as in contraction.cuh.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "contraction.cuh"
#include "conv_small.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"

namespace dlfb200 {

constexpr int kHaloEpiSets = 4;
constexpr int kHaloThreads = (2 + 4 * kHaloEpiSets) * 32;
constexpr int kHaloStageOut = kHaloEpiSets * 4 * 2 * 2048;
constexpr int kHaloMaxA = 8;   // filter-bank ring
constexpr int kHaloMaxH = 3;   // halo stages

struct HaloParams {
    const char* xh;     // X^ (bytes)
    char* y;
    const char* bias;
    const char* resid;
    int relu, fmt;
    int Cout, CB;              // output channels, 64-channel blocks of the input
    int OH, OW, P, Hp, Wp, KH, KW;
    int images;
    int R, BN;                 // output rows per tile, tile width (R * Wp rounded up to 16, <= 240)
    int tiles_per_image, co_tiles, total_tiles;
    long long out_img_stride;  // Cout * P
    int a_stages, h_stages;
    unsigned group_units;      // 16-byte units per channel group of a halo stage
    unsigned stage_bytes;      // 8 groups
    int d_tma;    // TMA stores of [32 channels][32 pixels] boxes possible (planes and rows of a multiple of 8 pixels)
    int out_vec;  // elements per store of a lane where it stores itself: 8, 4, 2 or 1
    long long wait_limit;
    int* status;
};

// one thread per pixel and channel group of X^
__global__ void __launch_bounds__(256)
    halo_pack_activations_kernel(const uint16_t* __restrict__ x, uint4* __restrict__ xh, int C, int H, int W, int Hp,
                                 int Wp, int pad_t, int pad_l, long long total) {
    const long long plane = static_cast<long long>(H) * W;
    const int CG = C / 8;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int q = static_cast<int>(i % Wp);
        long long r0 = i / Wp;
        const int r = static_cast<int>(r0 % Hp);
        r0 /= Hp;
        const int g = static_cast<int>(r0 % CG);
        const long long n = r0 / CG;
        const int ih = r - pad_t, iw = q - pad_l;
        uint32_t v[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (static_cast<unsigned>(ih) < static_cast<unsigned>(H) && static_cast<unsigned>(iw) < static_cast<unsigned>(W)) {
            const uint16_t* src = x + (n * C + 8 * g) * plane + static_cast<long long>(ih) * W + iw;
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = src[e * plane];
        }
        xh[i] = make_uint4(v[0] | (v[1] << 16), v[2] | (v[3] << 16), v[4] | (v[5] << 16), v[6] | (v[7] << 16));
    }
}

__global__ void __launch_bounds__(kHaloThreads, 1)
    conv_halo_kernel(const __grid_constant__ HaloParams p, const __grid_constant__ CUtensorMap tmW,
                     const __grid_constant__ CUtensorMap tmD) {
    constexpr uint32_t A_TILE = kBM * 128;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t a_full[kHaloMaxA];
    __shared__ __align__(8) uint64_t a_empty[kHaloMaxA];
    __shared__ __align__(8) uint64_t h_full[kHaloMaxH];
    __shared__ __align__(8) uint64_t h_empty[kHaloMaxH];
    __shared__ __align__(8) uint64_t tfull_bar[2];
    __shared__ __align__(8) uint64_t tempty_bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    // (through a shuffle: the compiler then knows that the warp index is uniform)
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int BN = p.BN;
    const int SA = p.a_stages, SH = p.h_stages;
    const int taps = p.KH * p.KW;
    const uint32_t smem0 = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = smem0;                                         // filter-bank ring
    const uint32_t sOut = sA + static_cast<uint32_t>(SA) * A_TILE;     // output staging blocks
    const uint32_t sHalo = sOut + kHaloStageOut;                       // halo stages: [group][row][Wp] x 16 bytes
    const uint32_t tmem_cols = 2 * BN > 256 ? 512u : (2 * BN > 128 ? 256u : 128u);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < SA; ++s) {
            ptx::mbar_init(ptx::smem_u32(&a_full[s]), 1u);
            ptx::mbar_init(ptx::smem_u32(&a_empty[s]), 1u);
        }
        for (int s = 0; s < SH; ++s) {
            ptx::mbar_init(ptx::smem_u32(&h_full[s]), 1u);
            ptx::mbar_init(ptx::smem_u32(&h_empty[s]), 1u);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(ptx::smem_u32(&tfull_bar[i]), 1u);
            ptx::mbar_init(ptx::smem_u32(&tempty_bar[i]), kHaloEpiSets * 4u);  // one arrival per epilogue warp
        }
        ptx::fence_mbar_init();
    }
    if (warp == 4) {
        __syncwarp();
        ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), tmem_cols);
        ptx::tmem_relinquish();
    }
    if (warp == 5 && lane == 0) ptx::tma_prefetch_desc(&tmW);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
    volatile int* abort_p = &abort_flag;
    const long long wait_limit = p.wait_limit;
    const int per_image = p.tiles_per_image * p.co_tiles;  // tile t: co tile fastest, then row block, then image

    if (warp < 4 || warp >= 6) {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;
        const int ewarp = warp < 4 ? warp : warp - 2;
        const int eset = ewarp >> 2;
        const bool relu = p.relu != 0;
        const int cpr = (p.OW + 31) / 32;  // blocks of 32 columns per output row
        uint32_t it = 0, chunk_no = 0;
        for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x, ++it) {
            const int img = t / per_image;
            const int rem = t - img * per_image;
            const int co0 = (rem % p.co_tiles) * kBM;
            const int oh0 = (rem / p.co_tiles) * p.R;
            const int rows = min(p.R, p.OH - oh0);
            const int co = co0 + q * 32 + lane;
            const bool co_ok = co < p.Cout;
            float bv = 0.0f;
            if (p.bias != nullptr && co_ok)
                bv = p.fmt == FMT_F16 ? out_load<OUT_F16>(p.bias + co * 2) : out_load<OUT_BF16>(p.bias + co * 2);
            const uint32_t buf = it & 1u;
            const uint32_t tphase = (it >> 1) & 1u;
            const bool w = ptx::mbar_wait_bounded(ptx::smem_u32(&tfull_bar[buf]), tphase, abort_p, wait_limit);
            if (!__all_sync(0xffffffffu, w)) break;
            ptx::tc_fence_after();
            const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
            const long long e_img = static_cast<long long>(img) * p.out_img_stride + static_cast<long long>(co) * p.P;
            // blocks (row r, columns c0 .. c0+31 of that row): the warp sets take them in turn
            // (a lane quadrant whose 32 channels all lie beyond Cout has nothing to write)
            const int nblocks = co0 + q * 32 < p.Cout ? rows * cpr : 0;
            for (int idx = eset; idx < nblocks; idx += kHaloEpiSets) {
                const int r = idx / cpr;
                const int c0 = (idx - r * cpr) * 32;
                uint32_t v[32];
                ptx::tmem_ld_32x32(tacc + r * p.Wp + c0, v);
                ptx::tmem_ld_wait();
                const int nc = min(32, p.OW - c0);
                const int pp0 = (oh0 + r) * p.OW + c0;  // first pixel of the block in its channel plane
                const long long e0 = e_img + pp0;
                if (p.d_tma && nc == 32) {
                    const uint32_t half = chunk_no & 1u;
                    if (chunk_no >= 2) {
                        if (lane == 0) ptx::bulk_wait_group_read<1>();
                        __syncwarp();
                    }
                    const uint32_t sblk = sOut + (ewarp * 2 + half) * 2048u;
                    const char* rp = p.resid ? p.resid + e0 * 2 : nullptr;
                    if (p.fmt == FMT_F16)
                        small_stage_block<OUT_F16>(v, sblk + lane * 64u, rp, co_ok, bv, relu);
                    else
                        small_stage_block<OUT_BF16>(v, sblk + lane * 64u, rp, co_ok, bv, relu);
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_3d(&tmD, sblk, pp0, co0 + q * 32, img);
                        ptx::bulk_commit_group();
                    }
                    ++chunk_no;
                } else {
                    // a partial block, or planes without 16-byte alignment: the lanes store themselves,
                    // in the widest vectors the row length allows (the tile lies inside one image: no
                    // wrap, the "plane" passed is unbounded)
#define DLF_HALO_DIRECT(OUT, G) \
    epilogue_swapped_chunk<OUT, G>(v, nc, p.y, p.resid, e0, 0, 1 << 30, 0, 0, 1.0f, bv, relu, co_ok, e0, 0, 0)
                    if (p.fmt == FMT_F16) {
                        if (p.out_vec == 8) DLF_HALO_DIRECT(OUT_F16, 8);
                        else if (p.out_vec == 4) DLF_HALO_DIRECT(OUT_F16, 4);
                        else if (p.out_vec == 2) DLF_HALO_DIRECT(OUT_F16, 2);
                        else DLF_HALO_DIRECT(OUT_F16, 1);
                    } else {
                        if (p.out_vec == 8) DLF_HALO_DIRECT(OUT_BF16, 8);
                        else if (p.out_vec == 4) DLF_HALO_DIRECT(OUT_BF16, 4);
                        else if (p.out_vec == 2) DLF_HALO_DIRECT(OUT_BF16, 2);
                        else DLF_HALO_DIRECT(OUT_BF16, 1);
                    }
#undef DLF_HALO_DIRECT
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[buf]));
        }
        if (p.d_tma && lane == 0) ptx::bulk_wait_group<0>();
    } else if (warp == 4) {
        // ------------------------------------------------------------ UMMA issuer
        // (the whole warp runs the loop, converged, and one elected lane issues: loop state and
        // descriptors stay in uniform registers)
        {
            const uint32_t idesc = ptx::make_idesc(static_cast<uint32_t>(p.fmt), 0u, 0u, kBM, BN);
            const uint64_t da0 = ptx::make_smem_desc(sA, 16u, 1024u, 2u);
            // operand B: unswizzled K-major; rows (halo positions) 16 bytes apart, the two 8-channel
            // k-chunks of a UMMA one channel group apart
            const uint64_t db0 = ptx::make_smem_desc(sHalo, p.group_units * 16u, 128u, 0u);
            uint32_t as = 0, aph = 0, hs = 0, hph = 0, it = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x, ++it) {
                const uint32_t buf = it & 1u;
                const uint32_t tphase = (it >> 1) & 1u;
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&tempty_bar[buf]), tphase ^ 1u, abort_p, wait_limit))) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int cb = 0; ok && cb < p.CB; ++cb) {
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&h_full[hs]), hph, abort_p, wait_limit))) {
                        ok = false;
                        break;
                    }
                    const uint32_t h_units = (hs * p.stage_bytes) >> 4;
                    int kh = 0, kw = 0;
                    for (int tap = 0; tap < taps; ++tap) {
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&a_full[as]), aph, abort_p, wait_limit))) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint32_t a_units = (as * A_TILE) >> 4;
                        const uint32_t shift = static_cast<uint32_t>(kh * p.Wp + kw);
                        if (ptx::elect_one()) {
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks)
                                ptx::umma_f16(d_tmem, da0 + (a_units + ks * 2), db0 + (h_units + 2 * ks * p.group_units + shift),
                                              idesc, (cb | tap | ks) ? 1u : 0u);
                            ptx::umma_commit(ptx::smem_u32(&a_empty[as]));
                        }
                        __syncwarp();
                        if (++as == static_cast<uint32_t>(SA)) {
                            as = 0;
                            aph ^= 1u;
                        }
                        if (++kw == p.KW) {
                            kw = 0;
                            ++kh;
                        }
                    }
                    if (!ok) break;
                    if (ptx::elect_one()) ptx::umma_commit(ptx::smem_u32(&h_empty[hs]));
                    __syncwarp();
                    if (++hs == static_cast<uint32_t>(SH)) {
                        hs = 0;
                        hph ^= 1u;
                    }
                }
                if (ok && ptx::elect_one()) ptx::umma_commit(ptx::smem_u32(&tfull_bar[buf]));
                __syncwarp();
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ copy producer
        // (converged warp, one issuing lane, as the UMMA issuer)
        {
            const bool leader = ptx::elect_one();
            uint32_t as = 0, aph = 0, hs = 0, hph = 0;
            bool ok = true;
            const int CG = p.CB * 8;
            for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                const int img = t / per_image;
                const int rem = t - img * per_image;
                const int co0 = (rem % p.co_tiles) * kBM;
                const int oh0 = (rem / p.co_tiles) * p.R;
                const int nrows = min(p.R + p.KH - 1, p.Hp - oh0);  // halo rows that exist
                for (int cb = 0; ok && cb < p.CB; ++cb) {
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&h_empty[hs]), hph ^ 1u, abort_p, wait_limit))) {
                        ok = false;
                        break;
                    }
                    // one bulk copy per channel group brings the tile's rows of that group as they lie
                    // (fewer at the bottom of the bordered image: the rows left out feed no output). A
                    // single 4-D tiled copy of all 8 groups - 16-byte inner boxes - was slower
                    // (64 -> 64 at 56x56: 207 vs 186 us)
                    const uint32_t hbar = ptx::smem_u32(&h_full[hs]);
                    const uint32_t bytes = static_cast<uint32_t>(nrows * p.Wp) * 16u;
                    if (leader) ptx::mbar_arrive_expect_tx(hbar, 8u * bytes);
                    const uint32_t dst0 = sHalo + hs * p.stage_bytes;
                    for (int g = 0; g < 8; ++g)
                        if (leader) ptx::bulk_load(dst0 + g * p.group_units * 16u,
                                       p.xh + ((static_cast<long long>(img) * CG + cb * 8 + g) * p.Hp + oh0) * p.Wp * 16, bytes, hbar);
                    if (++hs == static_cast<uint32_t>(SH)) {
                        hs = 0;
                        hph ^= 1u;
                    }
                    for (int tap = 0; tap < taps; ++tap) {
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&a_empty[as]), aph ^ 1u, abort_p, wait_limit))) {
                            ok = false;
                            break;
                        }
                        const uint32_t abar = ptx::smem_u32(&a_full[as]);
                        if (leader) ptx::mbar_arrive_expect_tx(abar, A_TILE);
                        if (leader) ptx::tma_load_3d(sA + as * A_TILE, &tmW, abar, (tap * p.CB + cb) * 64, co0, 0);
                        if (++as == static_cast<uint32_t>(SA)) {
                            as = 0;
                            aph ^= 1u;
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_p) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        if (threadIdx.x == 0) atomicOr(p.status, DEV_STATUS_WAIT_TIMEOUT);
        __syncthreads();
    }
    if (warp == 4) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, tmem_cols);
    }
}

}  // namespace dlfb200

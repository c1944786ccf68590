// Convolution of an input with at most 4 channels (an RGB stem: 7x7, stride 2) as an implicit GEMM
// with the roles swapped: the 128 tensor-memory lanes are output channels (at most 128; a filter
// bank of 64 fills half), the columns are R whole output rows of one image, OWp = OW + 3 rounded
// up to 8 columns per row (R * OWp <= 256; the extra columns of a row are not outputs).
//
// The activations come from the bordered row-pair copy X'' (N, sw, J, OWp, 2, 4) made by
// cl_pack_small_activations_kernel (channels_last.cuh): 16 bytes per pixel (two image rows x 4
// channels), the pixels of a row pair split into sw phases (pixel q in phase q % sw at q / sw), so
// that the pixels sw*i + ph that consecutive outputs i need for a filter tap are consecutive, and
// the row pairs of one phase consecutive as well.
// Windows of neighbouring outputs overlap, and a tensor-map load of the [output][window] operand
// would fetch every byte 8 / sw times from L2 in requests that are not line-aligned (measured:
// that load alone set the pace of the 224x224 stem, 458 us at batch 256). Instead all row pairs a
// tile needs (its R output rows and the filter rows above and below: one contiguous range per
// phase) arrive with one bulk copy per phase and tile - copies cost the copy engine about 150
// clocks apiece whatever their size, so few large ones matter - and the tensor core reads the
// overlapping windows in place: with the K-major *unswizzled* operand layout row n
// of a core matrix lies 16 bytes after row n-1, and the descriptor's leading-dimension offset
// (the distance between the two 8-element k-chunks of one UMMA) is set to the same 16 bytes, so
// operand row n, chunk c is pixel n + c of the phase - exactly the window; the row pair of a
// k-block (filter rows 2*kb, 2*kb+1) is a whole number of rows further on. One UMMA k-step is two
// taps of one phase; the filter bank (packed to match, swizzled K-major, K = ceil(KH/2) * 64) stays
// resident in shared memory for the whole launch.
//
// Warp roles: 0-3 and 6-17 epilogue (TMEM lane quadrant = warp & 3; the four sets take the tile's
// blocks of 32 columns in turn: measured, the conversions of eight epilogue warps were the longest
// stage of the 224x224 stem), 4 UMMA issuer and TMEM owner, 5 copy producer.
// All waits are bounded as in contraction.cuh.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "contraction.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"

namespace dlfb200 {

constexpr int kSmallEpiSets = 4;                            // sets of four epilogue warps (one per lane quadrant)
constexpr int kSmallThreads = (2 + 4 * kSmallEpiSets) * 32;  // + UMMA issuer + copy producer
constexpr int kSmallStageOut = kSmallEpiSets * 4 * 2 * 2048;  // two staging blocks per epilogue warp
constexpr int kSmallMaxStages = 8;

struct SmallParams {
    const char* xp;    // X'' (bytes)
    char* y;           // NCHW output
    const char* bias;  // per output channel, storage type, or null
    const char* resid; // tensor laid out like y, or null
    int relu, fmt;
    int Cout, OH, OW, P;       // P = OH * OW
    int J, sh, sw, rstep;  // row pairs per image, strides, image rows between row pairs (sh / rstep must be 1)
    int kb_rows;           // row pairs between consecutive k-blocks (2 / rstep)
    int span;              // row pairs a tile needs: R + kb_rows * (KB - 1)
    int KB;                     // k-blocks = ceil(KH / 2)
    int images;
    int R, OWp, BN;             // output rows per tile, columns per row, tile width R * OWp (a multiple of 16)
    int tiles_per_image;        // ceil(OH / R)
    int total_tiles;
    long long out_img_stride;   // Cout * P
    int stages;
    unsigned phase_bytes;  // one phase of a stage: (span * OWp + 8) pixels x 16 bytes
    unsigned stage_bytes;  // sw phases, rounded up to 128
    int d_tma;             // TMA stores of [32 channels][32 pixels] boxes possible
    long long wait_limit;
    int* status;
};

// One lane's 32 consecutive output pixels: bias, residual, ReLU, conversion, and 64 bytes into the
// staging block of a TMA store (row = this lane's channel; `srow` = its 64 bytes in a block aligned
// to 512 bytes).
template <int OUT>
__device__ __forceinline__ void small_stage_block(const uint32_t (&v)[32], uint32_t srow, const char* rp, bool row_ok,
                                                  float bv, bool relu) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float r[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) r[g] = __uint_as_float(v[8 * k + g]) + bv;
        if (rp != nullptr && row_ok) {
            const uint4 u = *reinterpret_cast<const uint4*>(rp + 16 * k);
            const uint32_t wds[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float2 f;
                if constexpr (OUT == OUT_F16) f = __half22float2(*reinterpret_cast<const __half2*>(&wds[g]));
                else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wds[g]));
                r[2 * g] += f.x;
                r[2 * g + 1] += f.y;
            }
        }
        if (relu) {
#pragma unroll
            for (int g = 0; g < 8; ++g) r[g] = fmaxf(r[g], 0.0f);
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            if constexpr (OUT == OUT_F16) {
                const __half2 h = __floats2half2_rn(r[2 * g], r[2 * g + 1]);
                ow[g] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * g], r[2 * g + 1]);
                ow[g] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        // the staging block is 64-byte swizzled (the box of the TMA store says so): 16-byte unit k of
        // row r lies at unit k ^ ((r >> 1) & 3), which spreads the lanes' stores over all bank groups
        st_shared_v4(srow + ((static_cast<uint32_t>(k) ^ ((srow >> 7) & 3u)) << 4), o);
    }
}

__global__ void __launch_bounds__(kSmallThreads, 1)
    conv_small_kernel(const __grid_constant__ SmallParams p, const __grid_constant__ CUtensorMap tmW,
                      const __grid_constant__ CUtensorMap tmD) {
    constexpr uint32_t A_KB = kBM * 128;  // one k-block of the filter bank
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t raw_full[kSmallMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kSmallMaxStages];
    __shared__ __align__(8) uint64_t a_full;
    __shared__ __align__(8) uint64_t tfull_bar[2];
    __shared__ __align__(8) uint64_t tempty_bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    // (through a shuffle: the compiler then knows that the warp index is uniform)
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int BN = p.BN;
    const int S = p.stages;
    const uint32_t smem0 = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = smem0;                                         // resident filter bank
    const uint32_t sOut = smem0 + static_cast<uint32_t>(p.KB) * A_KB;  // output staging blocks of the epilogue warps
    const uint32_t sStage = sOut + kSmallStageOut;                     // stages: [phase][row pair][OWp pixels]
    const uint32_t tmem_cols = 2 * BN > 256 ? 512u : (2 * BN > 128 ? 256u : 128u);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < S; ++s) {
            ptx::mbar_init(ptx::smem_u32(&raw_full[s]), 1u);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1u);
        }
        ptx::mbar_init(ptx::smem_u32(&a_full), 1u);
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(ptx::smem_u32(&tfull_bar[i]), 1u);
            ptx::mbar_init(ptx::smem_u32(&tempty_bar[i]), kSmallEpiSets * 4u);  // one arrival per epilogue warp
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

    if (warp < 4 || warp >= 6) {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;
        const int ewarp = warp < 4 ? warp : warp - 2;  // 0 .. 4 * kSmallEpiSets - 1
        const int eset = ewarp >> 2;                     // which of the sets this warp belongs to
        const int co = q * 32 + lane;
        const bool co_ok = co < p.Cout;
        float bv = 0.0f;
        if (p.bias != nullptr && co_ok)
            bv = p.fmt == FMT_F16 ? out_load<OUT_F16>(p.bias + co * 2) : out_load<OUT_BF16>(p.bias + co * 2);
        const bool relu = p.relu != 0;
        const int cpr = (p.OW + 31) / 32;  // blocks of 32 columns per output row
        uint32_t it = 0, chunk_no = 0;
        for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x, ++it) {
            const int img = t / p.tiles_per_image;
            const int oh0 = (t - img * p.tiles_per_image) * p.R;
            const int rows = min(p.R, p.OH - oh0);
            const uint32_t buf = it & 1u;
            const uint32_t tphase = (it >> 1) & 1u;
            const bool w = ptx::mbar_wait_bounded(ptx::smem_u32(&tfull_bar[buf]), tphase, abort_p, wait_limit);
            if (!__all_sync(0xffffffffu, w)) break;
            ptx::tc_fence_after();
            const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
            const long long e_img = static_cast<long long>(img) * p.out_img_stride + static_cast<long long>(co) * p.P;
            // blocks (row r, columns c0 .. c0+31 of that row): the warp sets take them in turn
            // (a lane quadrant whose 32 channels all lie beyond Cout - two of the four with 64 output
            // channels - has nothing to write: its blocks would only occupy the copy unit)
            const int nblocks = q * 32 < p.Cout ? rows * cpr : 0;
            for (int idx = eset; idx < nblocks; idx += kSmallEpiSets) {
                const int r = idx / cpr;
                const int c0 = (idx - r * cpr) * 32;
                uint32_t v[32];
                ptx::tmem_ld_32x32(tacc + r * p.OWp + c0, v);
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
                        ptx::tma_store_3d(&tmD, sblk, pp0, q * 32, img);
                        ptx::bulk_commit_group();
                    }
                    ++chunk_no;
                } else {
                    // a partial block, or planes without 16-byte alignment: the lanes store themselves
                    // (the tile lies inside one image: no wrap, the "plane" passed is unbounded)
                    if (p.d_tma) {
                        if (p.fmt == FMT_F16)
                            epilogue_swapped_chunk<OUT_F16, 8>(v, nc, p.y, p.resid, e0, 0, 1 << 30, 0, 0, 1.0f, bv, relu,
                                                               co_ok, e0, 0, 0);
                        else
                            epilogue_swapped_chunk<OUT_BF16, 8>(v, nc, p.y, p.resid, e0, 0, 1 << 30, 0, 0, 1.0f, bv, relu,
                                                                co_ok, e0, 0, 0);
                    } else {
                        if (p.fmt == FMT_F16)
                            epilogue_swapped_chunk<OUT_F16, 1>(v, nc, p.y, p.resid, e0, 0, 1 << 30, 0, 0, 1.0f, bv, relu,
                                                               co_ok, e0, 0, 0);
                        else
                            epilogue_swapped_chunk<OUT_BF16, 1>(v, nc, p.y, p.resid, e0, 0, 1 << 30, 0, 0, 1.0f, bv, relu,
                                                                co_ok, e0, 0, 0);
                    }
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
            // operand B: unswizzled K-major, rows 16 bytes apart, the two k-chunks of a UMMA 16 bytes apart too
            const uint64_t db0 = ptx::make_smem_desc(sStage, 16u, 128u, 0u);
            const int taps_per_phase = 8 / p.sw;                 // 16-byte pixels of a window in one phase
            const uint32_t phase_units = p.phase_bytes >> 4;     // 16-byte units between the phases of a stage
            const uint32_t kb_units = static_cast<uint32_t>(p.kb_rows * p.OWp);  // ... between the row pairs of k-blocks
            bool ok = __all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&a_full), 0u, abort_p, wait_limit));
            uint32_t stage = 0, phase = 0, it = 0;
            for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x, ++it) {
                const uint32_t buf = it & 1u;
                const uint32_t tphase = (it >> 1) & 1u;
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&tempty_bar[buf]), tphase ^ 1u, abort_p, wait_limit) &&
                                                 ptx::mbar_wait_bounded(ptx::smem_u32(&raw_full[stage]), phase, abort_p, wait_limit))) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const uint32_t b_units = (stage * p.stage_bytes) >> 4;
                if (ptx::elect_one()) {
                for (int kb = 0; kb < p.KB; ++kb) {
                    const uint32_t a_units = (static_cast<uint32_t>(kb) * A_KB) >> 4;
                    // k-step ks = taps (m, m+1) of phase ph: ks = ph * taps_per_phase / 2 + m / 2
                    int ph = 0, m = 0;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        ptx::umma_f16(d_tmem, da0 + (a_units + ks * 2),
                                      db0 + (b_units + ph * phase_units + kb * kb_units + m), idesc, (kb | ks) ? 1u : 0u);
                        m += 2;
                        if (m >= taps_per_phase) {
                            m = 0;
                            ++ph;
                        }
                    }
                }
                ptx::umma_commit(ptx::smem_u32(&empty_bar[stage]));
                ptx::umma_commit(ptx::smem_u32(&tfull_bar[buf]));
                }
                __syncwarp();
                if (++stage == static_cast<uint32_t>(S)) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ copy producer
        // (converged warp, one issuing lane, as the UMMA issuer)
        {
            const bool leader = ptx::elect_one();
            if (leader) ptx::mbar_arrive_expect_tx(ptx::smem_u32(&a_full), static_cast<uint32_t>(p.KB) * A_KB);
            for (int kb = 0; kb < p.KB; ++kb) if (leader) ptx::tma_load_3d(sA + kb * A_KB, &tmW, ptx::smem_u32(&a_full), kb * 64, 0, 0);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                const int img = t / p.tiles_per_image;
                const int oh0 = (t - img * p.tiles_per_image) * p.R;
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_p, wait_limit))) break;
                // row pairs j0 .. j0 + span - 1 of every phase (fewer at the bottom of the image: the
                // rows left out only feed output rows that do not exist)
                const int j0 = (oh0 * p.sh) / p.rstep;
                const int nrows = min(p.span, p.J - j0);
                const uint32_t bytes = static_cast<uint32_t>(nrows * p.OWp) * 16u;
                const uint32_t bar = ptx::smem_u32(&raw_full[stage]);
                if (leader) ptx::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(p.sw) * bytes);
                const uint32_t dst0 = sStage + stage * p.stage_bytes;
                for (int ph = 0; ph < p.sw; ++ph)
                    if (leader) ptx::bulk_load(dst0 + ph * p.phase_bytes,
                                   p.xp + ((static_cast<long long>(img) * p.sw + ph) * p.J + j0) * p.OWp * 16, bytes, bar);
                if (++stage == static_cast<uint32_t>(S)) {
                    stage = 0;
                    phase ^= 1u;
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

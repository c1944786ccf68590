// Persistent, warp-specialised tcgen05 contraction kernel.
//
// One kernel body serves gemm / gemmStridedBatched / gemmBatched and conv2d. Every call is
// first brought to one canonical problem on the host:
//
//     D[i + j*ldd] = alpha * sum_k Au(i,k) * Bu(j,k) + beta * D[i + j*ldd] (+ bias[j])
//
// with i the memory-contiguous index of the output. i maps to the 128 TMEM lanes of a
// UMMA tile, so a warp of the epilogue stores 32 consecutive output elements per
// instruction. Au (M x K) and Bu (N x K) are each either "K-major" (k contiguous in
// memory) or "MN-major" (i resp. j contiguous); tcgen05.mma accepts both for f16, bf16
// and tf32, which is why no transposition or padding pass exists.
//
// Shared-memory operand tiles use the 128-byte-swizzled canonical UMMA layouts. A tile
// of R rows by BK = 128/sizeof(T) k-values is R "lines" of 128 bytes; 16-byte chunk c of
// line L sits at  L*128 + ((c ^ (L & 7)) << 4).
//   K-major : line L = row L, the 128 bytes run along k.
//             descriptor: SBO = 1024 (8 rows), one UMMA k-step = +32 bytes.
//   MN-major: line L = (row group g = L / BK, k = L % BK), the 128 bytes run along rows
//             g*E .. g*E+E-1 (E = BK). descriptor: LBO = BK*128 (next row group),
//             SBO = 1024 (next 8 k), one UMMA k-step = +(UMMA_K/8)*1024 bytes.
//             32-bit (tf32) MN-major operands must use the 32-byte-atom form of the swizzle
//             instead: 32-byte chunk c2 of line L sits at L*128 + ((c2 ^ (L & 3)) << 5),
//             SBO = 512 (next 4 k).
// TMA boxes with CU_TENSOR_MAP_SWIZZLE_128B produce exactly these layouts; the generic
// loader warps reproduce them with plain stores.
//
// Roles (warp index): 0-3 epilogue (TMEM lane quadrant = warp index), 4 UMMA issuer and
// TMEM owner, 5 TMA producer, 6-13 generic loader warps (only launched for the generic
// variant). fp32 inputs run as 3xTF32: the loader writes hi = tf32(x) and lo = tf32(x - hi)
// tiles and the issuer accumulates lo*hi + hi*lo + hi*hi into one fp32 TMEM accumulator.
//
// All mbarrier waits are bounded (ptx::mbar_wait_bounded); a timeout raises a per-CTA
// abort flag, every role drains, TMEM is freed and a status word in global memory is set.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "epilogue.cuh"
#include "ptx.cuh"

namespace dlfb200 {

// Measurement build (-DDLF_ROLE_CLOCKS): one thread per role and CTA adds the SM clocks it spent
// waiting and working to a global table; compiled out otherwise.
#ifdef DLF_ROLE_CLOCKS
__device__ unsigned long long g_role_clocks[16];
#define DLF_CLK_DECL(cond) const bool clk_on = (cond); long long clk_t = clock64();
#define DLF_CLK_ADD(slot)                                                                         \
    do {                                                                                          \
        if (clk_on) {                                                                             \
            const long long now__ = clock64();                                                    \
            atomicAdd(&g_role_clocks[slot], static_cast<unsigned long long>(now__ - clk_t));      \
            clk_t = now__;                                                                        \
        }                                                                                         \
    } while (0)
#else
#define DLF_CLK_DECL(cond)
#define DLF_CLK_ADD(slot)
#endif

constexpr int kBM = 128;
constexpr int kMmaWarp = 4;
constexpr int kTmaWarp = 5;
constexpr int kFirstLoaderWarp = 6;
constexpr int kLoaderWarps = 8;
constexpr int kLoaderThreads = kLoaderWarps * 32;
// TMA variant: ESETS sets of four epilogue warps (warps 0-3, then 6 upwards), each set taking a share
// of the tile's columns. Two sets leave the registers and the shared memory a long main loop wants
// (168 registers, four 48 KB stages); four sets (96 registers, three stages) halve the time of the
// epilogue, which is what bounds tiles with a short K.
constexpr int tma_threads(int esets) { return (2 + 4 * esets) * 32; }
constexpr int epi_stage_bytes(int esets) { return esets * 4 * 2 * 2048; }  // two 2 KB output staging blocks per warp (dynamic)
constexpr int kThreadsTma = tma_threads(2);
constexpr int kThreadsPair = tma_threads(2);
constexpr int kThreadsGen = (kFirstLoaderWarp + kLoaderWarps) * 32;
constexpr int kMaxStages = 8;
constexpr int kGroupM = 8;  // tile rasterisation: kGroupM row-tiles share their column sweep

enum : int { FMT_F16 = 0, FMT_BF16 = 1, FMT_F32 = 2 };

enum : int {
    DEV_STATUS_OK = 0,
    DEV_STATUS_WAIT_TIMEOUT = 1,  // a bounded mbarrier wait gave up
};

struct GenOperand {
    const char* base;        // element (0,0) of batch 0
    long long ld;            // elements between consecutive 128-byte lines' origins
    long long batch_stride;  // elements between batches (0 = shared by every batch)
    int k_major;             // 1: k contiguous in memory; 0: row index contiguous
    int im2col;              // operand is an implicit im2col view of an NCHW tensor (A only)
};

// Geometry of the implicit im2col operand. Row index i of the canonical problem is the
// global output pixel  img * P + oh * OW + ow ; k = (c * KH + kh) * KW + kw.
struct Im2colGeom {
    int H, W, OH, OW, KH, KW, pad_t, pad_l, sh, sw, dh, dw;
    int P;                     // OH*OW
    long long img_stride;      // elements between images of X (C*H*W)
    long long out_img_stride;  // elements between images of Y (Cout*P)
};

// Division of a non-negative 32-bit int (< 2^31) by a divisor fixed for the launch, as a multiply
// and a shift: q = (mulhi(n, mul) + n) >> shift with shift = ceil(log2 d) and
// mul = floor(2^32 * (2^shift - d) / d) + 1, exact for n < 2^31 (the sum stays below 2^32). The role
// warps decode a tile index and an image / row position once per tile; the compiler's division
// sequences were a visible part of the per-tile cost. mul == 0: not prepared, divide plainly.
struct FastDiv {
    uint32_t mul, shift;
};
__device__ __forceinline__ int fast_div(int n, FastDiv f, int d) {
    return f.mul ? static_cast<int>((__umulhi(static_cast<uint32_t>(n), f.mul) + static_cast<uint32_t>(n)) >> f.shift) : n / d;
}

struct Params {
    int M, N, K, batch;
    int BN, stages, fmt;
    int tiles_m, tiles_n;
    int total_tiles;
    FastDiv fd_per, fd_group, fd_P, fd_OW;  // tiles_m * tiles_n, kGroupM * tiles_n, g.P, g.OW
    float alpha, beta;
    GenOperand a, b;
    char* d;
    long long ldd, d_batch_stride;
    // Batched products whose matrices lie at offsets off_b = base + idx_b * stride (the offset tables of
    // gemmBatched, when they have that form): per operand the index of batch entry b, or null for
    // idx_b = b. The index is the batch coordinate of the tensor maps.
    const int* a_idx;
    const int* b_idx;
    const int* d_idx;
    // gemmBatched tables (device memory, entries per batch); null for the other calls
    const long long* a_offs;
    const long long* b_offs;
    const long long* d_offs;
    const float* alphas;
    const float* betas;
    const char* bias;  // bias[batch*bias_stride + j] in the storage type, or null
    long long bias_stride;
    int bias_rows;     // the bias belongs to the rows of D (bias[i], one value per lane) instead of the columns:
                       // a channels-last convolution computed with the filter bank as operand A
    // fused convolution epilogue: resid (null or a tensor laid out like D) is added to the result,
    // relu clamps it at zero before the store
    const char* resid;
    int relu;
    Im2colGeom g;
    int* status;
    int d_tma;   // 0, or the column count (32 / 64) of the TMA store box. 16-bit outputs with
                 // beta == 0 and TMA-compatible strides: the epilogue stages
                 // 32 x 32 blocks in shared memory and writes them with TMA stores
    int d_f32;   // 16-bit operands, but D is written as fp32 (partial products of a K-split GEMM)
    int r_tma;   // the launch uses the RES instantiation: the residual's 32 x 32 boxes are fetched by TMA
                 // loads (map tmR, laid out like tmD) into the staging block their results leave from,
                 // one block ahead of the accumulator
    // Channels-last route of a convolution: operand A is a channels-last (N, H, W, C) copy of the
    // activations. a_cl == 1: tmA is an im2col-mode tensor map; k-block kb is channel block
    // kb % cl_cblocks of filter tap kb / cl_cblocks and one load brings the tile's 128 windows.
    // out_nchw: row i of the problem is output pixel img * P + pp and lands in an NCHW tensor
    // (the output mapping of the implicit-im2col operand, whatever A is).
    int a_cl, cl_cblocks, out_nchw;
    // cl_swap: the roles are swapped - operand A (rows, tensor-memory lanes) is the filter bank,
    // operand B (columns) the channels-last activations (tmB is then the im2col-mode map when
    // a_cl == 1), and the output mapping is out_nchw == 3: row = output channel, column = output
    // pixel img * P + pp, written as vectors of out_vec elements per lane (see epilogue.cuh).
    int cl_swap, out_vec;
    long long wait_limit;  // SM clocks a bounded wait may take (see ptx::mbar_wait_bounded)
    int skip_tile_commit;  // test aid: the UMMA issuer leaves out the commit that hands a finished
                           // accumulator to the epilogue, so that the epilogue's wait runs out
    int ablate;  // measurement aid (tuning flags >> 16; results are then meaningless):
                 // 1 A producer skips its loads, 2 B loaders skip theirs, 4 producers skip the TMEM
                 // stores, 8 / 16 row-form epilogue skips its body / its stores, 32 the plain
                 // epilogue of the TMEM-operand kernel is skipped, 0x100 pooling always takes the
                 // plain one-thread-per-output kernel (results stay valid), 0x4000 no programmatic
                 // dependent launch after the filter-packing grid (results stay valid)
};

struct PixelEntry {  // one output pixel of the current tile (implicit im2col operand)
    long long base;  // img*img_stride + ih0*W + iw0 (may point before the image: guarded)
    int ih0, iw0;    // oh*sh - pad_t, ow*sw - pad_l ; ih0 = INT_MIN/2 marks "no such pixel"
};

// total_tiles < 2^31 is checked on the host, so tile arithmetic stays in 32 bits.
__device__ __forceinline__ void decode_tile(const Params& p, int t, int& b, int& m0, int& n0,
                                            int rows_per_tile = kBM) {
    const int per = p.tiles_m * p.tiles_n;
    b = fast_div(t, p.fd_per, per);
    const int r = t - b * per;
    const int group = kGroupM * p.tiles_n;
    const int gi = fast_div(r, p.fd_group, group);
    const int first = gi * kGroupM;
    const int gm = min(p.tiles_m - first, kGroupM);
    const int rr = r - gi * group;
    const int cq = gm == kGroupM ? rr / kGroupM : rr / gm;  // (a full group: a shift)
    m0 = (first + rr - cq * gm) * rows_per_tile;
    n0 = cq * p.BN;
}

template <int ES>
__device__ __forceinline__ uint4 load_chunk_dense(const GenOperand& op, long long boff,
                                                  int line_coord, int line_lim, int cont0,
                                                  int cont_lim) {
    constexpr int CPE = 16 / ES;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (line_coord >= line_lim || cont0 >= cont_lim) return v;
    const char* ptr =
        op.base + (boff + static_cast<long long>(line_coord) * op.ld + cont0) * ES;
    if (cont0 + CPE <= cont_lim) {
        // a whole chunk inside the operand: the widest loads its address allows
        const uint32_t mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(ptr)) & 15u;
        if (mis == 0u) return *reinterpret_cast<const uint4*>(ptr);
        if ((mis & 7u) == 0u) {
            const uint2 lo = *reinterpret_cast<const uint2*>(ptr);
            const uint2 hi = *reinterpret_cast<const uint2*>(ptr + 8);
            return make_uint4(lo.x, lo.y, hi.x, hi.y);
        }
        if ((mis & 3u) == 0u) {
            const uint32_t* q = reinterpret_cast<const uint32_t*>(ptr);
            return make_uint4(q[0], q[1], q[2], q[3]);
        }
    }
    if constexpr (ES == 2) {
        unsigned short e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            e[i] = (cont0 + i < cont_lim) ? reinterpret_cast<const unsigned short*>(ptr)[i]
                                          : static_cast<unsigned short>(0);
        v.x = e[0] | (static_cast<uint32_t>(e[1]) << 16);
        v.y = e[2] | (static_cast<uint32_t>(e[3]) << 16);
        v.z = e[4] | (static_cast<uint32_t>(e[5]) << 16);
        v.w = e[6] | (static_cast<uint32_t>(e[7]) << 16);
    } else {
        uint32_t e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            e[i] = (cont0 + i < cont_lim) ? reinterpret_cast<const uint32_t*>(ptr)[i] : 0u;
        v = make_uint4(e[0], e[1], e[2], e[3]);
    }
    return v;
}

template <int ES>
__device__ __forceinline__ uint4 load_chunk_im2col(const Params& p, const PixelEntry* table,
                                                   long long boff, int k, int pix0) {
    constexpr int CPE = 16 / ES;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (k >= p.K) return v;
    const int khw = p.g.KH * p.g.KW;
    const int ch = k / khw;
    const int rem = k - ch * khw;
    const int kh = rem / p.g.KW;
    const int kw = rem - kh * p.g.KW;
    const int dy = kh * p.g.dh, dx = kw * p.g.dw;
    const long long koff =
        boff + (static_cast<long long>(ch) * p.g.H + dy) * p.g.W + dx;
    if constexpr (ES == 2) {
        unsigned short e[8];
#pragma unroll
        for (int i = 0; i < CPE; ++i) {
            const PixelEntry pe = table[pix0 + i];
            const bool ok = static_cast<unsigned>(pe.ih0 + dy) < static_cast<unsigned>(p.g.H) &&
                            static_cast<unsigned>(pe.iw0 + dx) < static_cast<unsigned>(p.g.W);
            e[i] = ok ? reinterpret_cast<const unsigned short*>(p.a.base)[pe.base + koff]
                      : static_cast<unsigned short>(0);
        }
        v.x = e[0] | (static_cast<uint32_t>(e[1]) << 16);
        v.y = e[2] | (static_cast<uint32_t>(e[3]) << 16);
        v.z = e[4] | (static_cast<uint32_t>(e[5]) << 16);
        v.w = e[6] | (static_cast<uint32_t>(e[7]) << 16);
    } else {
        uint32_t e[4];
#pragma unroll
        for (int i = 0; i < CPE; ++i) {
            const PixelEntry pe = table[pix0 + i];
            const bool ok = static_cast<unsigned>(pe.ih0 + dy) < static_cast<unsigned>(p.g.H) &&
                            static_cast<unsigned>(pe.iw0 + dx) < static_cast<unsigned>(p.g.W);
            e[i] = ok ? reinterpret_cast<const uint32_t*>(p.a.base)[pe.base + koff] : 0u;
        }
        v = make_uint4(e[0], e[1], e[2], e[3]);
    }
    return v;
}

// x = hi + lo with hi, lo both exactly representable in tf32 (10 explicit mantissa bits).
__device__ __forceinline__ void split_tf32(uint32_t x, uint32_t& hi, uint32_t& lo) {
    const float xf = __uint_as_float(x);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(xf));
    const float rest = xf - __uint_as_float(hi);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(rest));
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

template <int ES>
__device__ __forceinline__ void store_chunk(uint32_t tile, uint32_t lo_tile, int L, int c,
                                            const uint4& v, bool atom32) {
    const uint32_t cs = atom32 ? static_cast<uint32_t>((((c >> 1) ^ (L & 3)) << 1) | (c & 1))
                               : static_cast<uint32_t>(c ^ (L & 7));
    const uint32_t off = static_cast<uint32_t>(L) * 128u + (cs << 4);
    if constexpr (ES == 2) {
        st_shared_v4(tile + off, v);
    } else {
        uint4 hi, lo;
        split_tf32(v.x, hi.x, lo.x);
        split_tf32(v.y, hi.y, lo.y);
        split_tf32(v.z, hi.z, lo.z);
        split_tf32(v.w, hi.w, lo.w);
        st_shared_v4(tile + off, hi);
        st_shared_v4(lo_tile + off, lo);
    }
}

// PAIR: the CTA is one of a cluster of two that share 256 x BN tiles through cta_group::2 UMMAs
// (only with USE_TMA). Each CTA loads its own 128 rows of A and BN/2 rows of B with plain
// per-CTA TMA loads. Rank 0 issues the UMMAs and signals both CTAs' barriers.
template <int ES, bool USE_TMA, bool PAIR = false, int ESETS = 2, bool RES = false>
__global__ void __launch_bounds__(PAIR ? kThreadsPair : (USE_TMA ? tma_threads(ESETS) : kThreadsGen), 1)
    contraction_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmD,
                       const __grid_constant__ CUtensorMap tmR) {
    static_assert(!(USE_TMA && ES == 4), "fp32 operands need the split done by loader warps");
    static_assert(!PAIR || USE_TMA, "CTA pairs are fed by TMA");
    static_assert(!RES || (USE_TMA && !PAIR && ES == 2), "residual boxes belong to the TMA-store epilogue");
    constexpr int BK = 128 / ES;               // k-values per stage (one 128-byte line)
    constexpr int E = BK;                      // rows per MN-major row group
    constexpr int CPE = 16 / ES;               // elements per 16-byte chunk
    constexpr int UMMA_K = 32 / ES;            // 16 (f16/bf16) or 8 (tf32)
    constexpr uint32_t KSTEP_K = 32;           // bytes per UMMA k-step, K-major
    constexpr uint32_t KSTEP_MN = (UMMA_K / 8) * 1024;  // bytes per UMMA k-step, MN-major
    constexpr uint32_t A_TILE = kBM * 128;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ __align__(8) uint64_t tfull_bar[2];
    __shared__ __align__(8) uint64_t tempty_bar[2];
    __shared__ __align__(8) uint64_t res_bar[RES ? 4 * ESETS : 1][2];  // residual boxes, per epilogue warp and staging block
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ __align__(16) PixelEntry pix_table[USE_TMA ? 1 : kLoaderWarps * kBM];
    // output staging of the TMA-store epilogue: per epilogue warp two 32 x 32 blocks of 16-bit
    // values, [column][row] with rows contiguous (64-byte lines)
    __shared__ __align__(128) uint8_t d_stage_pair[PAIR ? 8 * 2 * 2048 : 16];  // CTA pairs keep their staging static

    // the warp index through a shuffle: the compiler then knows that it is the same in every lane,
    // keeps the role branches and what they compute on the uniform datapath, and the descriptors of
    // the UMMA issuer never pass through per-lane registers
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int BN = p.BN;
    const int S = p.stages;
    const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;  // position in the CTA pair
    const int b_rows = PAIR ? BN / 2 : BN;                     // rows of Bu this CTA stages
    const uint32_t b_tile = static_cast<uint32_t>(b_rows) * 128u;
    const uint32_t stage_bytes = (A_TILE + b_tile) * (ES == 4 ? 2u : 1u);
    const uint32_t smem0 = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const int num_kb = (p.K + BK - 1) / BK;
    const uint32_t tmem_cols = (PAIR || 2 * BN > 256) ? 512u : (2 * BN <= 128 ? 128u : 256u);
    const int tile0 = PAIR ? blockIdx.x / 2 : blockIdx.x;
    const int tile_step = PAIR ? gridDim.x / 2 : gridDim.x;
    const int tile_rows = PAIR ? 2 * kBM : kBM;
    const int row_off = PAIR ? static_cast<int>(rank) * kBM : 0;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < S; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), USE_TMA ? 1u : kLoaderThreads);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1u);
        }
        if constexpr (RES) {
            for (int i = 0; i < 4 * ESETS; ++i) {
                ptx::mbar_init(ptx::smem_u32(&res_bar[i][0]), 1u);
                ptx::mbar_init(ptx::smem_u32(&res_bar[i][1]), 1u);
            }
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(ptx::smem_u32(&tfull_bar[i]), 1u);
            // one arrival per epilogue warp (256 per-thread arrivals on one barrier serialise in shared
            // memory); PAIR: the warps of both CTAs (8 + 8), all on rank 0's barrier
            ptx::mbar_init(ptx::smem_u32(&tempty_bar[i]), PAIR ? 16u : (USE_TMA ? ESETS * 4u : 4u));
        }
        ptx::fence_mbar_init();
    }
    if (warp == kMmaWarp) {
        __syncwarp();
        if constexpr (PAIR) {
            ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_slot), tmem_cols);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), tmem_cols);
            ptx::tmem_relinquish();
        }
    }
    if (USE_TMA && warp == kTmaWarp && lane == 0) {
        ptx::tma_prefetch_desc(&tmA);
        ptx::tma_prefetch_desc(&tmB);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) ptx::cluster_sync();  // the peer's barriers exist before anything remote happens
    ptx::tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
    volatile int* abort_p = &abort_flag;
    const long long wait_limit = p.wait_limit;  // clocks a bounded wait may take before it gives up

    if (warp < 4 || (USE_TMA && warp >= 6)) {
        // ------------------------------------------------------------ epilogue
        // TMA variant: warps 0-3 take the first half of the tile's columns, warps 6-9 the second
        const int q = warp & 3;                       // TMEM lane quadrant (warp index mod 4)
        const int ewarp = warp < 4 ? warp : warp - 2;  // 0..7: staging buffer index
        // column sets: the tile's columns are shared out among min(sets, BN / 32) sets of four warps
        const int cset = (USE_TMA && warp >= 6) ? (warp - 6) / 4 + 1 : 0;
        const int nset = USE_TMA ? min(PAIR ? 2 : ESETS, BN / 32) : 1;
        const int cols_per = ((BN / 32 + nset - 1) / nset) * 32;  // whole blocks of 32 columns; the last set may get fewer
        const int cbase = cset < nset ? min(cset * cols_per, BN) : BN;  // idle sets start past the tile
        const uint32_t d_stage = PAIR ? ptx::smem_u32(d_stage_pair) : smem0 + static_cast<uint32_t>(S) * stage_bytes;
        uint32_t it = 0;
        uint32_t chunk_no = 0;  // TMA-store epilogue: 32-column blocks written so far by this warp
        // Residual boxes (p.r_tma): a block's residual is the box of the residual tensor that its
        // result is the box of in D, so one TMA load lands it in the block's own staging buffer, at
        // the addresses each lane is going to overwrite with its results. The load is issued when
        // the previous block's store has been handed over - a block ahead of the accumulator, across
        // tile boundaries too - because loads issued after the accumulator has arrived would add
        // their whole latency to every block (64 -> 256 channels at 56x56: 128 -> 414 us that way).
        uint32_t res_pending = 0;  // bit h: a residual load into staging block h is in flight or has landed
        uint32_t res_parity = 0;   // bit h: phase of res_bar[.][h] to wait for
        // box coordinates of block c0 of tile tt for this warp; false when that block does not leave
        // through a TMA store (the conditions of the store paths below)
        auto res_box = [&](int tt, int c0, int& x, int& y, int& z) -> bool {
            if (tt >= p.total_tiles) return false;
            int bb, mm, nn;
            decode_tile(p, tt, bb, mm, nn, tile_rows);
            mm += row_off;
            const int ncols_t = max(0, min(cols_per, min(BN, p.N - nn) - cbase));
            if (p.out_nchw == 3) {
                if (c0 + 32 > ncols_t || mm + q * 32 >= p.M) return false;
                const int j0 = nn + cbase + c0;
                const int img = fast_div(j0, p.fd_P, p.g.P);
                const int pp = j0 - img * p.g.P;
                if (pp + 32 > p.g.P && p.batch == 1) return false;
                x = pp;
                y = mm + q * 32;
                z = p.batch > 1 ? bb : img;
                return true;
            }
            const int i0 = mm + q * 32;
            if (i0 >= p.M || c0 >= ncols_t) return false;
            if (p.out_nchw == 5) {  // channels-last: {channels, pixels}
                x = nn + cbase + c0;
                y = i0;
                z = p.d_batch_stride ? bb : 0;
                return true;
            }
            const int img0 = p.out_nchw == 1 ? fast_div(i0, p.fd_P, p.g.P) : 0;
            const int pp0 = p.out_nchw == 1 ? i0 - img0 * p.g.P : i0;
            if (p.out_nchw == 1 && pp0 + 32 > p.g.P) return false;
            x = pp0;
            y = nn + cbase + c0;
            z = p.out_nchw == 1 ? img0 : (p.d_batch_stride ? bb : 0);
            return true;
        };
        auto res_fetch = [&](int tt, int c0, uint32_t h) {
            int x = 0, y = 0, z = 0;
            if (!res_box(tt, c0, x, y, z)) return;
            if (lane == 0) {
                const uint32_t bar = ptx::smem_u32(&res_bar[RES ? ewarp : 0][h]);
                ptx::mbar_arrive_expect_tx(bar, 2048u);
                ptx::tma_load_3d(d_stage + (ewarp * 2 + h) * 2048u, &tmR, bar, x, y, z);
            }
            res_pending |= 1u << h;
        };
        // the residual of block (tt, c0) is in staging block h (waits for it), or was never fetched
        auto res_landed = [&](uint32_t h) -> bool {
            if (!((res_pending >> h) & 1u)) return false;
            (void)ptx::mbar_wait_bounded(ptx::smem_u32(&res_bar[RES ? ewarp : 0][h]), (res_parity >> h) & 1u,
                                         abort_p, wait_limit);
            res_parity ^= 1u << h;
            res_pending &= ~(1u << h);
            return true;
        };
        // after block c0 of tile tt (ncols_t columns for this warp) has been handed to its store: the
        // other staging block is free once the store before that one has read it
        auto res_ahead = [&](int tt, int c0, int ncols_t, uint32_t h) {
            if (lane == 0) ptx::bulk_wait_group_read<1>();
            if (c0 + 32 < ncols_t) res_fetch(tt, c0 + 32, h);
            else res_fetch(tt + tile_step, 0, h);
        };
        // A block of 64 accumulator columns of this warp's 32 rows as ONE box of 64 x 32 elements (4 KB,
        // rows of 128 bytes, 128-byte swizzle) - p.d_tma == 64 in the forms whose boxes are [row][column]
        // images of the accumulator (out_nchw 3 and 5). TMA copies cost the SM's copy unit ~150 clocks
        // apiece whatever their size, and a layer that writes 411 MB in 2 KB boxes (plus as many residual
        // boxes) is bound by exactly that (64 -> 256 at 56x56: 102 us, 210 us with a residual; the bytes
        // alone would take 80 and 140). The warp's two 2 KB staging blocks form the one 4 KB block, so
        // there is no second buffer: the block's previous store must have read it before it is refilled,
        // and the residual box is fetched into it at the start of the block rather than a block ahead.
        // `trow`: tensor-memory address of column 0; (x, y, z): box coordinates; bias: per lane (`brow`)
        // or per column (`bias_cols` != null: entry of column 0). Warp-uniform arguments throughout.
        auto wide_block = [&](uint32_t trow, int x, int y, int z, int ncols_valid, float brow, const char* bias_cols,
                              int cols_left_in_tensor, bool relu_on) {
            if (chunk_no >= 1) {
                if (lane == 0) ptx::bulk_wait_group_read<0>();
                __syncwarp();
            }
            const uint32_t sblk = d_stage + ewarp * 4096u;
            bool res_smem = false;
            if constexpr (RES) {
                if (!(res_pending & 1u)) {  // not fetched ahead (see the channels-last call site)
                    if (lane == 0) {
                        const uint32_t bar = ptx::smem_u32(&res_bar[RES ? ewarp : 0][0]);
                        ptx::mbar_arrive_expect_tx(bar, 4096u);
                        ptx::tma_load_3d(sblk, &tmR, bar, x, y, z);
                    }
                    res_pending |= 1u;
                }
            }
            const uint32_t srow = sblk + lane * 128u;
            const uint32_t sx = static_cast<uint32_t>(lane) & 7u;
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                if (32 * h >= ncols_valid) break;
                uint32_t v[32];
                ptx::tmem_ld_32x32(trow + 32 * h, v);
                ptx::tmem_ld_wait();
                float bcol = 0.0f;
                if (bias_cols != nullptr && 32 * h + lane < cols_left_in_tensor)
                    bcol = p.fmt == FMT_F16 ? out_load<OUT_F16>(bias_cols + (32 * h + lane) * 2)
                                            : out_load<OUT_BF16>(bias_cols + (32 * h + lane) * 2);
                if constexpr (RES) {
                    if (h == 0) res_smem = res_landed(0u);
                }
                // alpha and the bias in a pass of their own: a select between the two kinds of bias
                // around the shuffle inside the loop below costs far more than it looks
                if (bias_cols != nullptr) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        v[j] = __float_as_uint(fmaf(p.alpha, __uint_as_float(v[j]), __shfl_sync(0xffffffffu, bcol, j)));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(fmaf(p.alpha, __uint_as_float(v[j]), brow));
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float r[8];
#pragma unroll
                    for (int g = 0; g < 8; ++g) r[g] = __uint_as_float(v[8 * k + g]);
                    const uint32_t saddr = srow + ((static_cast<uint32_t>(4 * h + k) ^ sx) << 4);
                    if (res_smem) {
                        const uint4 u = ld_shared_v4(saddr);
                        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const float2 f = p.fmt == FMT_F16
                                                 ? __half22float2(*reinterpret_cast<const __half2*>(&w[g]))
                                                 : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[g]));
                            r[2 * g] += f.x;
                            r[2 * g + 1] += f.y;
                        }
                    }
                    uint4 o;
                    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float a = relu_on ? fmaxf(r[2 * g], 0.0f) : r[2 * g];
                        const float c = relu_on ? fmaxf(r[2 * g + 1], 0.0f) : r[2 * g + 1];
                        if (p.fmt == FMT_F16) {
                            const __half2 hh = __floats2half2_rn(a, c);
                            ow[g] = *reinterpret_cast<const uint32_t*>(&hh);
                        } else {
                            const __nv_bfloat162 hh = __floats2bfloat162_rn(a, c);
                            ow[g] = *reinterpret_cast<const uint32_t*>(&hh);
                        }
                    }
                    st_shared_v4(saddr, o);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                ptx::tma_store_3d(&tmD, sblk, x, y, z);
                ptx::bulk_commit_group();
            }
            ++chunk_no;
        };
        DLF_CLK_DECL(warp == 0 && lane == 0)
        for (int t = tile0; t < p.total_tiles; t += tile_step, ++it) {
            int b, m0, n0;
            decode_tile(p, t, b, m0, n0, tile_rows);
            m0 += row_off;
            const int bd = p.d_idx ? p.d_idx[b] : b;  // where batch entry b of D lies
            const uint32_t buf = it & 1u;
            const uint32_t tphase = (it >> 1) & 1u;
            DLF_CLK_ADD(1);  // epilogue work of the previous tile
            // tcgen05.ld is warp-collective: the warp leaves together or not at all
            const bool w = ptx::mbar_wait_bounded(ptx::smem_u32(&tfull_bar[buf]), tphase, abort_p, wait_limit);
            if (!__all_sync(0xffffffffu, w)) break;
            ptx::tc_fence_after();
            DLF_CLK_ADD(0);  // waiting for an accumulator

            if constexpr (USE_TMA && !PAIR && ES == 2) {
                if (p.out_nchw == 3) {
                    // swapped roles: lanes are output channels, columns are output pixels
                    const int co = m0 + q * 32 + lane;
                    const bool co_ok = co < p.M;
                    const int cb3 = cbase;
                    // a quadrant whose 32 channels all lie beyond M (64 output channels on 128 lanes) has nothing to write
                    const int ncols3 = m0 + q * 32 < p.M ? max(0, min(cols_per, min(BN, p.N - n0) - cb3)) : 0;
                    float bv3 = 0.0f;
                    if (p.bias != nullptr && co_ok)
                        bv3 = p.fmt == FMT_F16 ? out_load<OUT_F16>(p.bias + co * 2) : out_load<OUT_BF16>(p.bias + co * 2);
                    const uint32_t trow3 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + cb3;
                    const long long rowoff = static_cast<long long>(co) * p.g.P;
                    const long long boff3 = static_cast<long long>(b) * p.d_batch_stride * 2;  // batched form: one image per batch entry
                    const bool relu3 = p.relu != 0;
                    for (int c0 = 0; c0 < ncols3; c0 += 32) {
                        const int j0 = n0 + cb3 + c0;
                        const int img = fast_div(j0, p.fd_P, p.g.P);
                        const int pp = j0 - img * p.g.P;
                        const int nc = min(32, ncols3 - c0);
                        if (p.d_tma == 64 && (c0 & 63) == 0 && ncols3 - c0 >= 64 && (pp + 64 <= p.g.P || p.batch > 1)) {
                            // 64 pixels x 32 channels in one box (clipped at the plane's end in the batched form)
                            wide_block(trow3 + c0, pp, m0 + q * 32, p.batch > 1 ? b : img, 64, bv3, nullptr, 0, relu3);
                            c0 += 32;
                            continue;
                        }
                        uint32_t v[32];
                        DLF_CLK_ADD(1);
                        ptx::tmem_ld_32x32(trow3 + c0, v);
                        ptx::tmem_ld_wait();
                        DLF_CLK_ADD(12);  // accumulator columns in registers
                        if (p.d_tma == 32 && nc == 32 && (pp + 32 <= p.g.P || p.batch > 1)) {
                            // the warp's 32 channels x 32 pixels are one box of the {pixels, channels,
                            // images} map: each lane lays its 32 pixels (64 bytes) into the staging
                            // block, which is then the box's own [channel][pixel] image. In the batched
                            // form a box that overhangs the plane is clipped by the hardware.
                            const uint32_t half = chunk_no & 1u;
                            if (chunk_no >= 2) {
                                if (lane == 0) ptx::bulk_wait_group_read<1>();
                                __syncwarp();
                            }
                            const uint32_t sblk = d_stage + (ewarp * 2 + half) * 2048u;
                            bool res_smem = false;
                            if constexpr (RES) {
                                if (!((res_pending >> half) & 1u)) res_fetch(t, c0, half);  // nothing was fetched ahead
                                res_smem = res_landed(half);
                            }
                            const char* rp = (p.resid && !res_smem)
                                                 ? p.resid + boff3 +
                                                       (static_cast<long long>(img) * p.g.out_img_stride + rowoff + pp) * 2
                                                 : nullptr;
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                float r[8];
#pragma unroll
                                for (int g = 0; g < 8; ++g) r[g] = fmaf(p.alpha, __uint_as_float(v[8 * k + g]), bv3);
                                if (res_smem || (rp != nullptr && co_ok)) {
                                    const uint4 u = res_smem ? ld_shared_v4(sblk + lane * 64u + ((static_cast<uint32_t>(k) ^ ((lane >> 1) & 3u)) << 4))
                                                             : *reinterpret_cast<const uint4*>(rp + 16 * k);
                                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                                    for (int g = 0; g < 4; ++g) {
                                        const float2 f = p.fmt == FMT_F16
                                                             ? __half22float2(*reinterpret_cast<const __half2*>(&w[g]))
                                                             : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[g]));
                                        r[2 * g] += f.x;
                                        r[2 * g + 1] += f.y;
                                    }
                                }
                                uint4 o;
                                uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                                for (int g = 0; g < 4; ++g) {
                                    const float a = relu3 ? fmaxf(r[2 * g], 0.0f) : r[2 * g];
                                    const float c = relu3 ? fmaxf(r[2 * g + 1], 0.0f) : r[2 * g + 1];
                                    if (p.fmt == FMT_F16) {
                                        const __half2 h = __floats2half2_rn(a, c);
                                        ow[g] = *reinterpret_cast<const uint32_t*>(&h);
                                    } else {
                                        const __nv_bfloat162 h = __floats2bfloat162_rn(a, c);
                                        ow[g] = *reinterpret_cast<const uint32_t*>(&h);
                                    }
                                }
                                // 64-byte swizzle of the box: 16-byte unit k of row r lies at unit k ^ ((r >> 1) & 3)
                                st_shared_v4(sblk + lane * 64u + ((static_cast<uint32_t>(k) ^ ((lane >> 1) & 3u)) << 4), o);
                            }
                            ptx::fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                ptx::tma_store_3d(&tmD, sblk, pp, m0 + q * 32, p.batch > 1 ? b : img);
                                ptx::bulk_commit_group();
                            }
                            ++chunk_no;
                            if constexpr (RES) res_ahead(t, c0, ncols3, half ^ 1u);
                            continue;
                        }
#define DLF_SWAPPED(OUT, G)                                                                                   \
    epilogue_swapped_chunk<OUT, G>(v, nc, p.d + boff3, p.resid ? p.resid + boff3 : nullptr, rowoff, p.g.out_img_stride, \
                                   p.g.P, img, pp, p.alpha, bv3, relu3, co_ok, rowoff, p.g.out_img_stride, img)
#define DLF_SWAPPED_FAST(OUT, G)                                                                              \
    epilogue_swapped_chunk_fast<OUT, G>(v, nc, p.d + boff3 + e0 * 2, p.resid ? p.resid + boff3 + e0 * 2 : nullptr, \
                                        p.g.P - pp, jump, jump, p.alpha, bv3, relu3, co_ok)
                        if (p.g.P >= 32 && p.out_vec > 1) {
                            const long long e0 = static_cast<long long>(img) * p.g.out_img_stride + rowoff + pp;
                            const long long jump = (p.g.out_img_stride - p.g.P) * 2;
                            if (p.fmt == FMT_F16) {
                                if (p.out_vec == 8) DLF_SWAPPED_FAST(OUT_F16, 8);
                                else if (p.out_vec == 4) DLF_SWAPPED_FAST(OUT_F16, 4);
                                else DLF_SWAPPED_FAST(OUT_F16, 2);
                            } else {
                                if (p.out_vec == 8) DLF_SWAPPED_FAST(OUT_BF16, 8);
                                else if (p.out_vec == 4) DLF_SWAPPED_FAST(OUT_BF16, 4);
                                else DLF_SWAPPED_FAST(OUT_BF16, 2);
                            }
                        } else if (p.fmt == FMT_F16) {
                            if (p.out_vec == 8) DLF_SWAPPED(OUT_F16, 8);
                            else if (p.out_vec == 4) DLF_SWAPPED(OUT_F16, 4);
                            else if (p.out_vec == 2) DLF_SWAPPED(OUT_F16, 2);
                            else DLF_SWAPPED(OUT_F16, 1);
                        } else {
                            if (p.out_vec == 8) DLF_SWAPPED(OUT_BF16, 8);
                            else if (p.out_vec == 4) DLF_SWAPPED(OUT_BF16, 4);
                            else if (p.out_vec == 2) DLF_SWAPPED(OUT_BF16, 2);
                            else DLF_SWAPPED(OUT_BF16, 1);
                        }
#undef DLF_SWAPPED
#undef DLF_SWAPPED_FAST
                    }
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[buf]));
                    continue;
                }
                if (p.out_nchw == 5) {
                    // Channels-last output D[pixel][channel]: the lanes are pixels, the columns output
                    // channels, so a lane's 32 columns are 64 consecutive bytes of D and the warp's
                    // block is one [32 pixels][32 channels] box of the {channels, pixels} map (clipped
                    // by the hardware at the last channel and the last pixel). Staging, swizzle,
                    // residual boxes and the store are those of the swapped NCHW form above.
                    const int i0 = m0 + q * 32;
                    const int ncols5 = i0 < p.M ? max(0, min(cols_per, min(BN, p.N - n0) - cbase)) : 0;
                    const uint32_t trow5 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + cbase;
                    const bool relu5 = p.relu != 0;
                    const uint32_t sw5 = (static_cast<uint32_t>(lane) >> 1) & 3u;
                    for (int c0 = 0; c0 < ncols5; c0 += 32) {
                        if (p.d_tma == 64) {
                            // 64 channels x 32 pixels in one box (clipped at the last channel and pixel)
                            const int colw = n0 + cbase + c0;
                            wide_block(trow5 + c0, colw, i0, p.d_batch_stride ? bd : 0, ncols5 - c0, 0.0f, p.bias ? p.bias + colw * 2 : nullptr,
                                       p.N - colw, relu5);
                            if constexpr (RES) {
                                // The block's store has been handed over: once it has read the staging block,
                                // the residual box of this warp's block of the NEXT tile is fetched into it, so
                                // that its latency runs beside the wait for that tile's accumulator.
                                if (c0 + 64 >= ncols5) {
                                    int rx = 0, ry = 0, rz = 0;
                                    if (res_box(t + tile_step, 0, rx, ry, rz)) {
                                        if (lane == 0) {
                                            ptx::bulk_wait_group_read<0>();
                                            const uint32_t bar = ptx::smem_u32(&res_bar[RES ? ewarp : 0][0]);
                                            ptx::mbar_arrive_expect_tx(bar, 4096u);
                                            ptx::tma_load_3d(d_stage + ewarp * 4096u, &tmR, bar, rx, ry, rz);
                                        }
                                        res_pending |= 1u;
                                    }
                                }
                            }
                            c0 += 32;
                            continue;
                        }
                        uint32_t v[32];
                        ptx::tmem_ld_32x32(trow5 + c0, v);
                        ptx::tmem_ld_wait();
                        const int col = n0 + cbase + c0;
                        float bv = 0.0f;
                        if (p.bias != nullptr && col + lane < p.N)
                            bv = p.fmt == FMT_F16 ? out_load<OUT_F16>(p.bias + (col + lane) * 2)
                                                  : out_load<OUT_BF16>(p.bias + (col + lane) * 2);
                        const uint32_t half = chunk_no & 1u;
                        if (chunk_no >= 2) {
                            if (lane == 0) ptx::bulk_wait_group_read<1>();
                            __syncwarp();
                        }
                        const uint32_t sblk = d_stage + (ewarp * 2 + half) * 2048u;
                        bool res_smem = false;
                        if constexpr (RES) {
                            if (!((res_pending >> half) & 1u)) res_fetch(t, c0, half);
                            res_smem = res_landed(half);
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float r[8];
#pragma unroll
                            for (int g = 0; g < 8; ++g)
                                r[g] = fmaf(p.alpha, __uint_as_float(v[8 * k + g]), __shfl_sync(0xffffffffu, bv, 8 * k + g));
                            const uint32_t saddr = sblk + lane * 64u + ((static_cast<uint32_t>(k) ^ sw5) << 4);
                            if (res_smem) {
                                const uint4 u = ld_shared_v4(saddr);
                                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                                for (int g = 0; g < 4; ++g) {
                                    const float2 f = p.fmt == FMT_F16
                                                         ? __half22float2(*reinterpret_cast<const __half2*>(&w[g]))
                                                         : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[g]));
                                    r[2 * g] += f.x;
                                    r[2 * g + 1] += f.y;
                                }
                            }
                            uint4 o;
                            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                const float a = relu5 ? fmaxf(r[2 * g], 0.0f) : r[2 * g];
                                const float c = relu5 ? fmaxf(r[2 * g + 1], 0.0f) : r[2 * g + 1];
                                if (p.fmt == FMT_F16) {
                                    const __half2 h = __floats2half2_rn(a, c);
                                    ow[g] = *reinterpret_cast<const uint32_t*>(&h);
                                } else {
                                    const __nv_bfloat162 h = __floats2bfloat162_rn(a, c);
                                    ow[g] = *reinterpret_cast<const uint32_t*>(&h);
                                }
                            }
                            st_shared_v4(saddr, o);
                        }
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            ptx::tma_store_3d(&tmD, sblk, col, i0, p.d_batch_stride ? bd : 0);
                            ptx::bulk_commit_group();
                        }
                        ++chunk_no;
                        if constexpr (RES) res_ahead(t, c0, ncols5, half ^ 1u);
                    }
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[buf]));
                    continue;
                }
            }
            const int i = m0 + q * 32 + lane;
            const bool row_ok = i < p.M;
            long long rowbase;
            long long colstride;
            if (p.a.im2col || p.out_nchw) {
                const int img = fast_div(i, p.fd_P, p.g.P);
                const int pp = i - img * p.g.P;
                rowbase = static_cast<long long>(img) * p.g.out_img_stride +
                          static_cast<long long>(b) * p.d_batch_stride + pp;
                colstride = p.g.P;
            } else {
                rowbase = (p.d_offs ? p.d_offs[b] : static_cast<long long>(bd) * p.d_batch_stride) + i;
                colstride = p.ldd;
            }
            const float alpha = p.alphas ? p.alphas[b] : p.alpha;
            const float beta = p.betas ? p.betas[b] : p.beta;
            const char* bias =
                p.bias ? p.bias + (static_cast<long long>(b) * p.bias_stride + n0 + (USE_TMA ? cbase : 0)) * ES : nullptr;
            const int cb = USE_TMA ? cbase : 0;  // first column of this warp's share
            const uint32_t trow = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + cb;
            char* optr = p.d + (rowbase + static_cast<long long>(n0 + cb) * colstride) * ES;
            const int ncols = max(0, min(USE_TMA ? cols_per : BN, min(BN, p.N - n0) - cb));
            if constexpr (USE_TMA) {
                if (p.d_tma) {
                    const int i0 = m0 + q * 32;
                    // NCHW output: a block of 32 pixels is one box of the {P, channels, images} map
                    // unless it runs over the end of its image; such a block (and only it) is
                    // written by the lanes themselves
                    const int img0 = p.out_nchw == 1 ? fast_div(i0, p.fd_P, p.g.P) : 0;
                    const int pp0 = p.out_nchw == 1 ? i0 - img0 * p.g.P : i0;
                    const bool direct = p.out_nchw == 1 && pp0 + 32 > p.g.P;
                    const bool blk_ok = i0 < p.M;
                    // Blocks of 32 rows x 32 columns go to one of the warp's two staging buffers
                    // (2 KB each, adjacent). With 32-column boxes the buffers alternate and every
                    // block is one TMA store; with 64-column boxes (tiles of 128 columns or more)
                    // two consecutive blocks fill both buffers and leave as one 4 KB store: TMA
                    // stores this small are bound by their number, not their bytes.
                    const bool wide = p.d_tma == 64;
                    for (int c0 = 0; c0 < ncols && blk_ok; c0 += 32, ++chunk_no) {
                        uint32_t v[32];
                        DLF_CLK_ADD(1);
                        ptx::tmem_ld_32x32(trow + c0, v);
                        ptx::tmem_ld_wait();
                        DLF_CLK_ADD(12);
                        float bv = 0.0f;  // this lane's entry of the columns' bias (stays 0 with a bias per row)
                        if (!p.bias_rows && bias != nullptr && c0 + lane < ncols)
                            bv = p.fmt == FMT_F16 ? out_load<OUT_F16>(bias + (c0 + lane) * 2)
                                                  : out_load<OUT_BF16>(bias + (c0 + lane) * 2);
                        const uint32_t half = wide ? static_cast<uint32_t>((c0 >> 5) & 1) : (chunk_no & 1u);
                        // the store that last read this buffer must have drained it
                        if (wide ? (half == 0 && chunk_no >= 1) : (chunk_no >= 2)) {
                            if (lane == 0) {
                                if (wide) ptx::bulk_wait_group_read<0>();
                                else ptx::bulk_wait_group_read<1>();
                            }
                            __syncwarp();
                        }
                        const uint32_t sbuf = d_stage + (ewarp * 2 + half) * 2048u + lane * 2u;
                        bool res_smem = false;
                        if constexpr (RES) {
                            if (!direct) {
                                if (!((res_pending >> half) & 1u)) res_fetch(t, c0, half);
                                res_smem = res_landed(half);
                            }
                        }
                        if (res_smem) {
                            // the block's residual lies in the staging block, [column][row] like the results
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) {
                                unsigned short h16;
                                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h16) : "r"(sbuf + jj * 64u) : "memory");
                                const float rv = p.fmt == FMT_F16 ? __half2float(__ushort_as_half(h16))
                                                                  : __bfloat162float(__ushort_as_bfloat16(h16));
                                v[jj] = __float_as_uint(alpha * __uint_as_float(v[jj]) + rv);
                            }
                        } else if (p.resid != nullptr) {
                            // residual values first (loads must not sit between the stores)
                            const char* rp = p.resid + (optr - p.d) + static_cast<long long>(c0) * colstride * 2;
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) {
                                float rv = 0.0f;
                                if (row_ok && c0 + jj < ncols)
                                    rv = p.fmt == FMT_F16 ? out_load<OUT_F16>(rp + jj * colstride * 2)
                                                          : out_load<OUT_BF16>(rp + jj * colstride * 2);
                                v[jj] = __float_as_uint(alpha * __uint_as_float(v[jj]) + rv);
                            }
                        } else {
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) v[jj] = __float_as_uint(alpha * __uint_as_float(v[jj]));
                        }
                        if (p.bias_rows && p.bias != nullptr) {
                            // a bias per row is one value per lane: added here, in a pass of its own, so that
                            // the loops below stay as they are without it (a select around their shuffle
                            // doubled the time of the batched product 1024 x (512 x 512 x 64))
                            const float brow = !row_ok ? 0.0f
                                               : (p.fmt == FMT_F16 ? out_load<OUT_F16>(p.bias + i * 2) : out_load<OUT_BF16>(p.bias + i * 2));
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) v[jj] = __float_as_uint(__uint_as_float(v[jj]) + brow);
                        }
                        // the clamp only exists under ReLU: fmaxf drops a NaN operand, so an
                        // unconditional fmaxf(r, -inf) would turn NaN results into -inf
                        const bool relu = p.relu != 0;
                        if (direct) {
                            char* op = optr + static_cast<long long>(c0) * colstride * 2;
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) {
                                float r = __uint_as_float(v[jj]) + __shfl_sync(0xffffffffu, bv, jj);
                                r = relu ? fmaxf(r, 0.0f) : r;
                                if (row_ok && c0 + jj < ncols) {
                                    if (p.fmt == FMT_F16) out_store<OUT_F16>(op + jj * colstride * 2, r);
                                    else out_store<OUT_BF16>(op + jj * colstride * 2, r);
                                }
                            }
                            continue;
                        }
                        if (p.fmt == FMT_F16) {
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) {
                                float r = __uint_as_float(v[jj]) + __shfl_sync(0xffffffffu, bv, jj);
                                r = relu ? fmaxf(r, 0.0f) : r;
                                const unsigned short h = __half_as_ushort(__float2half_rn(r));
                                asm volatile("st.shared.u16 [%0], %1;" ::"r"(sbuf + jj * 64u), "h"(h) : "memory");
                            }
                        } else {
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) {
                                float r = __uint_as_float(v[jj]) + __shfl_sync(0xffffffffu, bv, jj);
                                r = relu ? fmaxf(r, 0.0f) : r;
                                const unsigned short h = __bfloat16_as_ushort(__float2bfloat16_rn(r));
                                asm volatile("st.shared.u16 [%0], %1;" ::"r"(sbuf + jj * 64u), "h"(h) : "memory");
                            }
                        }
                        // a wide store leaves after its second block, or after the first when no
                        // second one exists (the box is then clipped at column N by the hardware)
                        if (wide && half == 0 && c0 + 32 < ncols) continue;
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const uint32_t ssrc = d_stage + (ewarp * 2 + (wide ? 0u : half)) * 2048u;
                            const int col = n0 + cb + (wide ? (c0 & ~63) : c0);
                            ptx::tma_store_3d(&tmD, ssrc, pp0, col, p.out_nchw == 1 ? img0 : (p.d_batch_stride ? bd : 0));
                            ptx::bulk_commit_group();
                        }
                        if constexpr (RES) res_ahead(t, c0, ncols, half ^ 1u);
                    }
                    ptx::tc_fence_before();
                    if constexpr (PAIR) {
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&tempty_bar[buf]), 0u));
                    } else {
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[buf]));
                    }
                    continue;
                }
            }
            EpiExtra ex;
            ex.relu = p.relu != 0;
            ex.rdelta = p.resid ? p.resid - p.d : 0;
            const float beta_e = p.resid ? 1.0f : beta;  // a residual takes the place of the beta term
            if constexpr (ES == 4) {
                epilogue_dispatch<OUT_F32>(trow, ncols, optr, colstride * ES, row_ok, alpha, beta_e,
                                           bias, lane, nullptr, false, ex);
            } else if (p.d_f32) {
                char* o32 = p.d + (rowbase + static_cast<long long>(n0 + cb) * colstride) * 4;
                epilogue_dispatch<OUT_F32>(trow, ncols, o32, colstride * 4, row_ok, alpha, beta_e, nullptr, lane,
                                           nullptr, false, ex);
            } else {
                const bool pair_ok = pair_store_ok(optr, rowbase, colstride, row_ok, lane);
                if (p.fmt == FMT_F16)
                    epilogue_dispatch<OUT_F16>(trow, ncols, optr, colstride * ES, row_ok, alpha,
                                               beta_e, bias, lane, nullptr, pair_ok, ex);
                else
                    epilogue_dispatch<OUT_BF16>(trow, ncols, optr, colstride * ES, row_ok, alpha,
                                                beta_e, bias, lane, nullptr, pair_ok, ex);
            }
            ptx::tc_fence_before();
            if constexpr (PAIR) {
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&tempty_bar[buf]), 0u));
            } else {
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[buf]));
            }
        }
        if constexpr (USE_TMA) {
            // a residual box fetched ahead of a block that never came (the loop was left early): its
            // bytes must have landed before the CTA's shared memory is given back
            if constexpr (RES) {
                if (res_pending & 1u) (void)res_landed(0u);
                if (res_pending & 2u) (void)res_landed(1u);
            }
            if (p.d_tma && lane == 0) ptx::bulk_wait_group<0>();  // all staged blocks are in global memory
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ UMMA issuer
        // The whole warp runs the loop, converged, and one elected lane issues: loop state and
        // descriptors then live in uniform registers. (Issued from inside an `if (lane == 0)` region
        // every UMMA paid for moving its operands over from per-lane registers: a 64-column UMMA
        // cost as much issue time as a 256-column one.)
        if (rank == 0) {
            const uint32_t idesc =
                ptx::make_idesc(p.fmt == FMT_F32 ? 2u : static_cast<uint32_t>(p.fmt),
                                p.a.k_major ? 0u : 1u, p.b.k_major ? 0u : 1u, PAIR ? 2 * kBM : kBM, BN);
            const uint32_t a_step = p.a.k_major ? KSTEP_K : KSTEP_MN;
            const uint32_t b_step = p.b.k_major ? KSTEP_K : KSTEP_MN;
            const uint32_t a_lbo = p.a.k_major ? 16u : static_cast<uint32_t>(BK) * 128u;
            const uint32_t b_lbo = p.b.k_major ? 16u : static_cast<uint32_t>(BK) * 128u;
            const uint32_t a_mode = (ES == 4 && !p.a.k_major) ? 1u : 2u;
            const uint32_t b_mode = (ES == 4 && !p.b.k_major) ? 1u : 2u;
            const uint32_t a_sbo = a_mode == 1u ? 512u : 1024u;
            const uint32_t b_sbo = b_mode == 1u ? 512u : 1024u;
            // descriptors differ only in the 14-bit start-address field (address >> 4): build
            // them once and advance by plain adds
            const uint64_t da0 = ptx::make_smem_desc(smem0, a_lbo, a_sbo, a_mode);
            const uint64_t db0 = ptx::make_smem_desc(smem0 + A_TILE, b_lbo, b_sbo, b_mode);
            const uint32_t lo_units = (A_TILE + b_tile) >> 4;
            uint32_t stage = 0, phase = 0;
            uint32_t it = 0;
            bool ok = true;
            DLF_CLK_DECL(lane == 0)
            for (int t = tile0; ok && t < p.total_tiles; t += tile_step, ++it) {
                const uint32_t buf = it & 1u;
                const uint32_t tphase = (it >> 1) & 1u;
                DLF_CLK_ADD(4);  // issue
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&tempty_bar[buf]), tphase ^ 1u, abort_p, wait_limit))) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                DLF_CLK_ADD(2);  // waiting for the epilogue to free an accumulator
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    DLF_CLK_ADD(4);
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&full_bar[stage]), phase, abort_p, wait_limit))) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    DLF_CLK_ADD(3);  // waiting for operands
                    const uint32_t st_units = (stage * stage_bytes) >> 4;
                    if (ptx::elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < BK / UMMA_K; ++ks) {
                        const uint64_t da = da0 + (st_units + ((ks * a_step) >> 4));
                        const uint64_t db = db0 + (st_units + ((ks * b_step) >> 4));
                        const uint32_t acc = (kb | ks) ? 1u : 0u;
                        if constexpr (PAIR) {
                            ptx::umma_f16_pair(d_tmem, da, db, idesc, acc);
                        } else if constexpr (ES == 2) {
                            ptx::umma_f16(d_tmem, da, db, idesc, acc);
                        } else {
                            ptx::umma_tf32(d_tmem, da + lo_units, db, idesc, acc);
                            ptx::umma_tf32(d_tmem, da, db + lo_units, idesc, 1u);
                            ptx::umma_tf32(d_tmem, da, db, idesc, 1u);
                        }
                    }
                    if constexpr (PAIR) {  // free the stage in both CTAs
                        ptx::umma_commit_pair(ptx::smem_u32(&empty_bar[stage]));
                        ptx::umma_commit_pair(ptx::map_to_cta(ptx::smem_u32(&empty_bar[stage]), 1u));
                    } else {
                        ptx::umma_commit(ptx::smem_u32(&empty_bar[stage]));
                    }
                    }
                    __syncwarp();
                    if (++stage == static_cast<uint32_t>(S)) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok && !p.skip_tile_commit && ptx::elect_one()) {
                    if constexpr (PAIR) {  // both CTAs' epilogue warps read their half of the tile
                        ptx::umma_commit_pair(ptx::smem_u32(&tfull_bar[buf]));
                        ptx::umma_commit_pair(ptx::map_to_cta(ptx::smem_u32(&tfull_bar[buf]), 1u));
                    } else {
                        ptx::umma_commit(ptx::smem_u32(&tfull_bar[buf]));
                    }
                }
            }
        }
    } else if (USE_TMA && warp == kTmaWarp) {
        // ------------------------------------------------------------ TMA producer
        // The whole warp runs the loop, converged, and one lane issues the copies: coordinates,
        // addresses and loop state then stay in uniform registers, which is where the copy
        // instructions take them from (see the UMMA issuer).
        {
            const bool leader = ptx::elect_one();
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            DLF_CLK_DECL(lane == 0)
            for (int t = tile0; ok && t < p.total_tiles; t += tile_step) {
                int b, m0, n0;
                decode_tile(p, t, b, m0, n0, tile_rows);
                m0 += row_off;
                n0 += PAIR ? static_cast<int>(rank) * b_rows : 0;  // this CTA's share of the Bu rows
                // (table entries come from memory: the shuffle tells the compiler that they are uniform)
                const int ba = p.a.batch_stride ? (p.a_idx ? __shfl_sync(0xffffffffu, p.a_idx[b], 0) : b) : 0;
                const int bb = p.b.batch_stride ? (p.b_idx ? __shfl_sync(0xffffffffu, p.b_idx[b], 0) : b) : 0;
                // im2col-mode loads: base pixel of the tile's first filter window
                int cl_n = 0, cl_h = 0, cl_w = 0;
                if (!PAIR && p.a_cl == 1) {
                    const int first = p.cl_swap ? n0 : m0;  // first output pixel of the tile
                    cl_n = fast_div(first, p.fd_P, p.g.P);
                    const int pp = first - cl_n * p.g.P;
                    const int oh = fast_div(pp, p.fd_OW, p.g.OW);
                    cl_h = oh * p.g.sh - p.g.pad_t;
                    cl_w = (pp - oh * p.g.OW) * p.g.sw - p.g.pad_l;
                }
                int cl_cb = 0, cl_kh = 0, cl_kw = 0;  // channel block and filter tap of kb
                for (int kb = 0; kb < num_kb; ++kb) {
                    DLF_CLK_ADD(6);  // issue
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u,
                                                                        abort_p, wait_limit))) {
                        ok = false;
                        break;
                    }
                    DLF_CLK_ADD(5);  // waiting for a free stage
                    const uint32_t sA = smem0 + stage * stage_bytes;
                    const uint32_t sB = sA + A_TILE;
                    if (!PAIR && p.cl_swap && p.a_cl == 1) {
                        // swapped roles: A = filter bank (tiled), B = activations (im2col mode, BN windows)
                        const uint32_t bar = ptx::smem_u32(&full_bar[stage]);
                        if (leader) {  // one divergent region per k-block
                            ptx::mbar_arrive_expect_tx(bar, A_TILE + b_tile);
                            ptx::tma_load_3d(sA, &tmA, bar, kb * BK, m0, 0);
                            ptx::tma_load_im2col_4d(sB, &tmB, bar, cl_cb * BK, cl_w, cl_h, cl_n,
                                                    static_cast<unsigned short>(cl_kw * p.g.dw),
                                                    static_cast<unsigned short>(cl_kh * p.g.dh));
                        }
                        DLF_CLK_ADD(8);  // copies handed over
                        if (++cl_cb == p.cl_cblocks) {
                            cl_cb = 0;
                            if (++cl_kw == p.g.KW) {
                                cl_kw = 0;
                                ++cl_kh;
                            }
                        }
                        if (++stage == static_cast<uint32_t>(S)) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    if (!PAIR && p.a_cl == 1) {
                        const uint32_t bar = ptx::smem_u32(&full_bar[stage]);
                        if (leader) {  // one divergent region per k-block
                            ptx::mbar_arrive_expect_tx(bar, A_TILE + b_tile);
                            ptx::tma_load_im2col_4d(sA, &tmA, bar, cl_cb * BK, cl_w, cl_h, cl_n,
                                                    static_cast<unsigned short>(cl_kw * p.g.dw),
                                                    static_cast<unsigned short>(cl_kh * p.g.dh));
                            ptx::tma_load_3d(sB, &tmB, bar, kb * BK, n0, bb);
                        }
                        DLF_CLK_ADD(8);
                        if (++cl_cb == p.cl_cblocks) {
                            cl_cb = 0;
                            if (++cl_kw == p.g.KW) {
                                cl_kw = 0;
                                ++cl_kh;
                            }
                        }
                        if (++stage == static_cast<uint32_t>(S)) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    if constexpr (PAIR) {
                        // both CTAs' copies are counted on rank 0's barrier, which rank 0 arms
                        // with the bytes of the two CTAs together
                        const uint32_t bar = ptx::map_to_cta(ptx::smem_u32(&full_bar[stage]), 0u);
                        if (leader && rank == 0) ptx::mbar_arrive_expect_tx(ptx::smem_u32(&full_bar[stage]), 2u * (A_TILE + b_tile));
                        if (p.a.k_major) {
                            if (leader) ptx::tma_load_3d_pair(sA, &tmA, bar, kb * BK, m0, ba);
                        } else {
                            for (int g = 0; g < kBM / E; ++g)
                                if (leader) ptx::tma_load_3d_pair(sA + g * BK * 128, &tmA, bar, m0 + g * E, kb * BK, ba);
                        }
                        if (p.b.k_major) {
                            if (leader) ptx::tma_load_3d_pair(sB, &tmB, bar, kb * BK, n0, bb);
                        } else {
                            for (int g = 0; g < b_rows / E; ++g)
                                if (leader) ptx::tma_load_3d_pair(sB + g * BK * 128, &tmB, bar, n0 + g * E, kb * BK, bb);
                        }
                    } else {
                        const uint32_t bar = ptx::smem_u32(&full_bar[stage]);
                        if (leader) {  // one divergent region per k-block
                            ptx::mbar_arrive_expect_tx(bar, A_TILE + b_tile);
                            if (p.a.k_major) {
                                ptx::tma_load_3d(sA, &tmA, bar, kb * BK, m0, ba);
                            } else {
                                for (int g = 0; g < kBM / E; ++g)
                                    ptx::tma_load_3d(sA + g * BK * 128, &tmA, bar, m0 + g * E, kb * BK, ba);
                            }
                            if (p.b.k_major) {
                                ptx::tma_load_3d(sB, &tmB, bar, kb * BK, n0, bb);
                            } else {
                                for (int g = 0; g < BN / E; ++g)
                                    ptx::tma_load_3d(sB + g * BK * 128, &tmB, bar, n0 + g * E, kb * BK, bb);
                            }
                        }
                        DLF_CLK_ADD(8);
                    }
                    if (++stage == static_cast<uint32_t>(S)) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (!USE_TMA && warp >= kFirstLoaderWarp) {
        // ------------------------------------------------------------ generic loader warps
        const int lt = threadIdx.x - kFirstLoaderWarp * 32;
        const int c = lt & 7;
        const int l0 = lt >> 3;
        const bool a_atom32 = ES == 4 && !p.a.k_major;
        const bool b_atom32 = ES == 4 && !p.b.k_major;
        uint32_t stage = 0, phase = 0;
        uint32_t it = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x, ++it) {
            int b, m0, n0;
            decode_tile(p, t, b, m0, n0);
            const long long a_boff =
                p.a_offs ? p.a_offs[b] : static_cast<long long>(b) * p.a.batch_stride;
            const long long b_boff =
                p.b_offs ? p.b_offs[b] : static_cast<long long>(b) * p.b.batch_stride;
            // Each loader warp keeps its own table of the tile's 128 output pixels, so no
            // cross-warp barrier is needed when warps run ahead of one another.
            PixelEntry* table = pix_table + (warp - kFirstLoaderWarp) * kBM;
            if (p.a.im2col) {
                __syncwarp();
#pragma unroll
                for (int q = 0; q < kBM / 32; ++q) {
                    PixelEntry pe;
                    const int gp = m0 + lane + 32 * q;
                    if (gp < p.M) {
                        const int img = gp / p.g.P;
                        const int pp = gp - img * p.g.P;
                        const int oh = pp / p.g.OW;
                        const int ow = pp - oh * p.g.OW;
                        pe.ih0 = oh * p.g.sh - p.g.pad_t;
                        pe.iw0 = ow * p.g.sw - p.g.pad_l;
                        pe.base = static_cast<long long>(img) * p.g.img_stride +
                                  static_cast<long long>(pe.ih0) * p.g.W + pe.iw0;
                    } else {
                        pe.ih0 = -(1 << 30);
                        pe.iw0 = -(1 << 30);
                        pe.base = 0;
                    }
                    table[lane + 32 * q] = pe;
                }
                __syncwarp();
            }
            for (int kb = 0; kb < num_kb; ++kb) {
                // the whole warp leaves together: later __syncwarp()s need every lane
                const bool w =
                    ptx::mbar_wait_bounded(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_p, wait_limit);
                if (!__all_sync(0xffffffffu, w)) {
                    ok = false;
                    break;
                }
                const uint32_t sA = smem0 + stage * stage_bytes;
                const uint32_t sB = sA + A_TILE;
                const uint32_t lo_off = A_TILE + b_tile;
                // A tile: kBM lines
                {
                    uint4 v[kBM / 32];
#pragma unroll
                    for (int q = 0; q < kBM / 32; ++q) {
                        const int L = l0 + 32 * q;
                        if (p.a.im2col) {
                            v[q] = load_chunk_im2col<ES>(p, table, a_boff, kb * BK + (L % BK),
                                                         (L / BK) * E + c * CPE);
                        } else if (p.a.k_major) {
                            v[q] = load_chunk_dense<ES>(p.a, a_boff, m0 + L, p.M, kb * BK + c * CPE,
                                                        p.K);
                        } else {
                            v[q] = load_chunk_dense<ES>(p.a, a_boff, kb * BK + (L % BK), p.K,
                                                        m0 + (L / BK) * E + c * CPE, p.M);
                        }
                    }
#pragma unroll
                    for (int q = 0; q < kBM / 32; ++q)
                        store_chunk<ES>(sA, sA + lo_off, l0 + 32 * q, c, v[q], a_atom32);
                }
                // B tile: BN lines, four at a time
                for (int q0 = 0; q0 < BN / 32; q0 += 4) {
                    uint4 v[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int L = l0 + 32 * (q0 + q);
                        if (q0 + q >= BN / 32) {
                            v[q] = make_uint4(0u, 0u, 0u, 0u);
                        } else if (p.b.k_major) {
                            v[q] = load_chunk_dense<ES>(p.b, b_boff, n0 + L, p.N, kb * BK + c * CPE,
                                                        p.K);
                        } else {
                            v[q] = load_chunk_dense<ES>(p.b, b_boff, kb * BK + (L % BK), p.K,
                                                        n0 + (L / BK) * E + c * CPE, p.N);
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (q0 + q < BN / 32)
                            store_chunk<ES>(sB, sB + lo_off, l0 + 32 * (q0 + q), c, v[q], b_atom32);
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(ptx::smem_u32(&full_bar[stage]));
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
        // Give copies and UMMAs still in flight time to land before shared memory and
        // TMEM are released.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        if (threadIdx.x == 0) atomicOr(p.status, DEV_STATUS_WAIT_TIMEOUT);
        __syncthreads();
    }
    if constexpr (PAIR) ptx::cluster_sync();  // the peer may still signal this CTA's barriers until here
    if (warp == kMmaWarp) {
        __syncwarp();
        ptx::tc_fence_after();
        if constexpr (PAIR)
            ptx::tmem_dealloc_pair(tmem_base, tmem_cols);
        else
            ptx::tmem_dealloc(tmem_base, tmem_cols);
    }
}

}  // namespace dlfb200

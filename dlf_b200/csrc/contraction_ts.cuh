// Contraction kernel whose A operand lives in tensor memory ("TS" form of tcgen05.mma).
//
// Same canonical problem as contraction.cuh:
//     D[i + j*ldd] = alpha * sum_k Au(i,k) * Bu(j,k) + beta * D (+ bias[j])
// but the 128 x BK tile of Au never touches shared memory. Eight producer warps own the 128
// TMEM lanes (two warps per 32-lane quadrant, alternating k-blocks); thread <-> row i of the
// tile. Each thread loads its row's BK values straight from global memory into registers -
// for an MN-major Au and for the implicit im2col view of an NCHW tensor the 32 lanes of a warp
// read 32 consecutive addresses - splits fp32 values into tf32 (hi, lo) in registers, and writes
// them to TMEM with tcgen05.st. The UMMA issuer then runs tcgen05.mma with A = [tmem] and
// B = shared-memory descriptor. Only Bu (for convolutions: the filter bank) is staged in
// swizzled shared memory, by four loader warps.
//
// Why: with both operands in shared memory a 3xTF32 tile reads each operand three times and
// writes hi and lo copies of both; for the 128 x 64 tiles of a 64-channel convolution that is
// more shared-memory traffic than the tensor pipe can be fed with. Moving A to TMEM removes
// two thirds of it and all the address swizzling from the gather.
//
// Convolution (im2col) gather: k = (c*KH + kh)*KW + kw. A per-CTA table in shared memory holds,
// for every k, the element offset c*H*W + kh*dh*W + kw*dw and (kh*dh, kw*dw); a thread keeps
// its pixel's (ih0, iw0, base offset) in registers and a tap is valid when
// 0 <= ih0 + kh*dh < H and 0 <= iw0 + kw*dw < W (zero otherwise: the padding).
//
// Row form of the convolution (A_ROWCONV; stride_w = dilation_w = 1, KW >= 2). A UMMA costs the
// same ~115 clocks for any N <= 128, so a 64-channel layer wastes most of the tensor pipe when N is
// the channel count. Here the horizontal taps move from K into N:
//     D'[(img,oh,u), (kw,co)] = sum_{kh,c} X[img][c][oh*sh-pt+kh*dh][u] * W[co][c][kh][kw]
//     Y[img][co][oh][ow]      = sum_kw D'[(img,oh,ow+kw-pl), (kw,co)]
// K shrinks to C*KH and N grows to KW*cpt (192 for 3x3 with 64 channels per tile): a third of the
// MMAs and a third of the gathered elements. Rows of D' are input columns u; the sum over kw is
// done in the epilogue with warp shuffles between neighbouring lanes, so every warp owns a window
// of 32 consecutive positions of which the inner T = 32 - (KW-1) produce outputs (windows of
// consecutive warps overlap by KW-1 positions).
//
// With a horizontal stride sw > 1 (and dilation_w = 1) the same form applies after splitting the
// input columns into sw phases: u = sw*ow + kw - pl = sw*(ow + d) + r with r = (kw - pl) mod sw,
// d = floor((kw - pl) / sw). Positions are (img, oh, w') over a virtual row of w' values, the
// column phases join the channels in K (k' = (kh*C + c)*sw + r reads X[..][sw*w' + r]) and the taps
// become the shifts d = dmin..dmax: Y[ow] = sum_d D'[(ow + d), (d, co)]. The 7x7 stride-2 stem of
// ResNet becomes K' = 42 (one k-block), N = 4 x 64.
//
// TMEM columns: [0, acc_bufs*BN) accumulators, then `stages` A slots of 32 (16-bit types: 64 k
// packed two per column) or 64 (fp32: 32 hi + 32 lo) columns.
// Warp roles: 0-3 epilogue, 4-11 A producers (quadrant = warp % 4), 12-14 B loaders, 15 UMMA
// issuer and TMEM owner.
#pragma once
#include "contraction.cuh"

namespace dlfb200 {

constexpr int kTsProducerWarp0 = 4;
constexpr int kTsLoaderWarp0 = 12;
constexpr int kTsMmaWarp = 15;
constexpr int kTsThreads = 16 * 32;  // 512 threads: 128 registers each
constexpr int kTsLoaderThreads = 3 * 32;
constexpr int kTsLoaderLines = kTsLoaderThreads / 8;  // lines covered per pass of the B loaders

enum : int { A_DENSE_MN = 0, A_DENSE_K = 1, A_IM2COL = 2, A_ROWCONV = 3 };

struct KEntry {  // one k of the implicit im2col operand
    int off;     // c*H*W + kh*dh*W + kw*dw
    short dy;    // kh*dh
    short dx;    // kw*dw
};

struct TsParams {
    Params base;
    int a_kind;
    int acc_bufs;      // 1 or 2 accumulator buffers in TMEM
    int ktable_bytes;  // bytes reserved at the start of dynamic shared memory for KEntry[k]
    // A_ROWCONV only (see the header comment): taps per row, output channels per tile, output
    // positions per warp, lanes of left halo
    int rc_kw, rc_cpt, rc_T, rc_lo;
    // Row form with a horizontal stride (see the header comment): rc_sw = stride_w (number of
    // column phases folded into K), rc_wv = positions per row, rc_dmin = smallest tap shift
    // (rc_lo = -rc_dmin); with stride_w = 1 these are 1, W and -pad_left.
    int rc_sw, rc_wv, rc_dmin;
    // Filter bank already laid out as the kernel's shared-memory stage images (pack_weights_kernel):
    // [batch][n-tile][k-block][stage_bytes]; null = the loader warps gather from the OIHW tensor
    const unsigned char* b_packed;
    // fp32 with long K: the accumulator is restarted every kc_blocks k-blocks and the finished
    // chunks are summed in shared memory at byte offset sums_off of the dynamic segment
    // (float[BN][128]); 0 = one chunk (see drain_chunk in epilogue.cuh)
    int kc_blocks, sums_off;
    // fp32 dense products whose B operand satisfies the TMA rules: TMA delivers the raw fp32 tiles
    // (which double as the hi image), the loader warps derive the lo image from them. (The same
    // scheme for the packed filter bank of a convolution - raw images only, half the bytes from
    // L2 - was measured slower, 123 vs 90 us on the 64-channel 3x3 layer: with two operand stages
    // the extra hop through the converter warps is not hidden.)
    int b_tma;
    // A_IM2COL with a 1x1 filter and no padding (any stride): addresses are affine in k
    int a_pointwise;
    // byte offset, in the dynamic segment, of the blocks that rc_tma stages its results in
    int stage_off;
    // Row form with image-aligned tiles (rc_tpi = tiles per image, 0 = tiles run across images): a
    // tile then is one contiguous range of one image's pixels for every channel, and 16-bit
    // results leave as TMA stores (rc_tma; two blocks of rc_tma_buf bytes at stage_off).
    int rc_tpi, rc_tma, rc_tma_buf;
    int b_stages;  // depth of the B ring in shared memory (Params::stages is the depth of the A ring)
    int rc_pair;   // row form, stride_w = 2, 16-bit: gather with one 32-bit load per pair of k
    // The packed filter bank of the (only) column tile fits in the B ring as a whole (b_stages =
    // number of k-blocks): every CTA loads it once, for its first tile, and keeps it - the bank is
    // then not streamed from L2 again for every tile.
    int b_resident;
};

// First position of row-form tile `tm`, and (image-aligned tiles) the image it belongs to.
__device__ __forceinline__ int rowconv_pos0(const TsParams& tp, int tm, int OHW, int& tile_img) {
    if (tp.rc_tpi) {
        tile_img = tm / tp.rc_tpi;
        return tile_img * OHW + (tm - tile_img * tp.rc_tpi) * 4 * tp.rc_T;
    }
    tile_img = -1;
    return tm * 4 * tp.rc_T;
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :
        : "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]),
          "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
          "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
          "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Element k' = (kh*C + c)*sw + r of the row-form filter operand for output channel `co_off`
// (element offset of W[co][0][0][0]) and tap j: W[co][c][kh][kw] with kw = sw*(j + dmin) + r + pl,
// zero where that kw does not exist or k' >= k_lim.
struct RowTaps {
    int KH, KW, cg;  // real filter height and width, channels per group
    int sw, dmin, pl;
};
template <int ES>
__device__ __forceinline__ uint32_t rowconv_weight(const char* base, long long co_off, const RowTaps& rt,
                                                   int j, int k, int k_lim) {
    if (k >= k_lim) return 0u;
    const int cgv = rt.cg * rt.sw;
    const int kh = k / cgv;
    const int rem = k - kh * cgv;
    const int c = rem / rt.sw;
    const int r = rem - c * rt.sw;
    const int kw = rt.sw * (j + rt.dmin) + r + rt.pl;
    if (kw < 0 || kw >= rt.KW) return 0u;
    const long long idx = co_off + static_cast<long long>(c * rt.KH + kh) * rt.KW + kw;
    if constexpr (ES == 4) return reinterpret_cast<const uint32_t*>(base)[idx];
    else return reinterpret_cast<const unsigned short*>(base)[idx];
}
template <int ES>
__device__ __forceinline__ uint4 load_chunk_rowconv(const char* base, long long co_off, const RowTaps& rt,
                                                    int j, bool row_ok, int k0, int k_lim) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (!row_ok || k0 >= k_lim) return v;
    if constexpr (ES == 4) {
        v.x = rowconv_weight<ES>(base, co_off, rt, j, k0, k_lim);
        v.y = rowconv_weight<ES>(base, co_off, rt, j, k0 + 1, k_lim);
        v.z = rowconv_weight<ES>(base, co_off, rt, j, k0 + 2, k_lim);
        v.w = rowconv_weight<ES>(base, co_off, rt, j, k0 + 3, k_lim);
    } else {
        uint32_t e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = rowconv_weight<ES>(base, co_off, rt, j, k0 + i, k_lim);
        v = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
    }
    return v;
}
__device__ __forceinline__ RowTaps row_taps(const TsParams& tp) {
    RowTaps rt;
    rt.KH = tp.base.g.KH;
    rt.KW = tp.base.g.KW;
    rt.sw = tp.rc_sw;
    rt.cg = tp.base.K / (tp.base.g.KH * tp.rc_sw);
    rt.dmin = tp.rc_dmin;
    rt.pl = tp.base.g.pad_l;
    return rt;
}

// Lays the filter bank of a convolution out as the stage images the kernel above consumes, once
// per call: for every (batch entry = group, n-tile, k-block) BN lines of 128 bytes in the swizzled
// K-major layout (hi image, then lo image for fp32). One thread per 16-byte chunk.
template <int ES>
__global__ void pack_weights_kernel(const TsParams tp, unsigned char* out, long long total_chunks) {
    const Params& p = tp.base;
    constexpr int BK = 128 / ES;
    constexpr int CPE = 16 / ES;
    const int BN = p.BN;
    const int num_kb = (p.K + BK - 1) / BK;
    const long long stage_bytes = static_cast<long long>(BN) * 128 * (ES == 4 ? 2 : 1);
    // the contraction kernel is launched as a programmatic dependent of this grid: let it start
    // (prologue, activation gather) while the filter bank is still being packed; its filter
    // loader waits for this grid's completion (griddepcontrol.wait) before it reads `out`
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; id < total_chunks;
         id += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(id & 7);
        long long r = id >> 3;
        const int L = static_cast<int>(r % BN);
        r /= BN;
        const int kb = static_cast<int>(r % num_kb);
        r /= num_kb;
        const int tn = static_cast<int>(r % p.tiles_n);
        const int b = static_cast<int>(r / p.tiles_n);
        const long long b_boff = static_cast<long long>(b) * p.b.batch_stride;
        uint4 v;
        if (tp.a_kind == A_ROWCONV) {
            const int kw = L / tp.rc_cpt;
            const int co = tn * tp.rc_cpt + (L - kw * tp.rc_cpt);
            const RowTaps rt = row_taps(tp);
            v = load_chunk_rowconv<ES>(p.b.base, b_boff + static_cast<long long>(co) * rt.cg * rt.KH * rt.KW, rt,
                                       kw, co < p.N, kb * BK + c * CPE, p.K);
        } else {
            v = load_chunk_dense<ES>(p.b, b_boff, tn * BN + L, p.N, kb * BK + c * CPE, p.K);
        }
        unsigned char* img = out + (((static_cast<long long>(b) * p.tiles_n + tn) * num_kb) + kb) * stage_bytes;
        const long long o = static_cast<long long>(L) * 128 + ((c ^ (L & 7)) << 4);
        if constexpr (ES == 2) {
            *reinterpret_cast<uint4*>(img + o) = v;
        } else {
            uint4 hi, lo;
            split_tf32(v.x, hi.x, lo.x);
            split_tf32(v.y, hi.y, lo.y);
            split_tf32(v.z, hi.z, lo.z);
            split_tf32(v.w, hi.w, lo.w);
            *reinterpret_cast<uint4*>(img + o) = hi;
            *reinterpret_cast<uint4*>(img + static_cast<long long>(BN) * 128 + o) = lo;
        }
    }
}

// AK: the kind of the A operand the instantiation serves - A_ROWCONV, A_IM2COL, or A_DENSE_MN for
// both dense kinds (told apart at run time). One instantiation per kind keeps the code of the
// other kinds' gathers and epilogues out of the kernel: fewer registers and a smaller footprint
// in the instruction cache for every role.
template <int ES, int AK>
__global__ void __launch_bounds__(kTsThreads, 1)
    contraction_ts_kernel(const __grid_constant__ TsParams tp, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmD) {
    const Params& p = tp.base;
    const int a_kind = (AK == A_ROWCONV || AK == A_IM2COL) ? AK : tp.a_kind;
    constexpr int BK = 128 / ES;             // k per stage: 32 (fp32) or 64 (16-bit)
    constexpr int CPE = 16 / ES;
    constexpr int UMMA_K = 32 / ES;
    constexpr int A_COLS = ES == 4 ? 64 : 32;  // TMEM columns per A slot
    constexpr int A_KSTEP_COLS = 8;            // columns one UMMA k-step consumes
    constexpr uint32_t KSTEP_K = 32;
    constexpr uint32_t KSTEP_MN = (UMMA_K / 8) * 1024;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_a[kMaxStages];
    __shared__ __align__(8) uint64_t full_b[kMaxStages];
    __shared__ __align__(8) uint64_t raw_b[kMaxStages];  // b_tma: raw tile landed
    __shared__ __align__(8) uint64_t empty_a[kMaxStages];  // A slot (tensor memory) consumed
    __shared__ __align__(8) uint64_t empty_b[kMaxStages];  // B stage (shared memory) consumed
    __shared__ __align__(8) uint64_t tfull_bar[2];
    __shared__ __align__(8) uint64_t tempty_bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int epi_ok[2][4];  // TMA-store epilogue: outcome of each epilogue warp's wait for the tile

    // (through a shuffle: the compiler then knows that the warp index is uniform)
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int BN = p.BN;
    // The A slots live in tensor memory and the B stages in shared memory: the two rings have their
    // own depths (a wide fp32 tile leaves room for only two A slots but for four B stages, whose
    // bulk copies take longer than the tensor core needs for a k-block).
    const int SA = p.stages;
    const int SB = tp.b_stages;
    const int nbuf = tp.acc_bufs;
    const uint32_t b_tile = static_cast<uint32_t>(BN) * 128u;
    const uint32_t stage_bytes = b_tile * (ES == 4 ? 2u : 1u);
    const KEntry* ktable = reinterpret_cast<const KEntry*>(smem_raw);
    const uint32_t smem0 =
        (ptx::smem_u32(smem_raw) + static_cast<uint32_t>(tp.ktable_bytes) + 1023u) & ~1023u;
    const int num_kb = (p.K + BK - 1) / BK;
    const uint32_t a_col0 = static_cast<uint32_t>(nbuf * BN);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < kMaxStages; ++s) {
            // (one arrival per warp: per-thread arrivals on one barrier serialise in shared memory)
            ptx::mbar_init(ptx::smem_u32(&full_a[s]), 4u);
            ptx::mbar_init(ptx::smem_u32(&full_b[s]), tp.b_packed ? 1u : (tp.b_tma ? 2u : kTsLoaderThreads / 32u));
            ptx::mbar_init(ptx::smem_u32(&raw_b[s]), 1u);
            ptx::mbar_init(ptx::smem_u32(&empty_a[s]), 1u);
            ptx::mbar_init(ptx::smem_u32(&empty_b[s]), 1u);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(ptx::smem_u32(&tfull_bar[i]), 1u);
            ptx::mbar_init(ptx::smem_u32(&tempty_bar[i]), 4u);  // one arrival per epilogue warp
        }
        ptx::fence_mbar_init();
    }
    if (a_kind == A_ROWCONV) {
        // k' = (kh*C + c)*sw + r -> (offset of the input row + column phase r, kh*dh, r); the
        // column is the thread's own (times sw). With sw = 1 a k-block usually lies inside one kh:
        // one validity test and a constant address stride (H*W) for the whole block. With sw = 2
        // the two phases of a (kh, c) are neighbours in k and in memory: one 32-bit load fills a
        // packed register of 16-bit values (rc_pair).
        KEntry* kt = reinterpret_cast<KEntry*>(smem_raw);
        const int cgv = p.K / p.g.KH;     // channels per group x column phases
        for (int k = threadIdx.x; k < num_kb * BK; k += blockDim.x) {
            KEntry e;
            const int kk = k < p.K ? k : 0;
            const int kh = kk / cgv;
            const int rem = kk - kh * cgv;
            const int ch = rem / tp.rc_sw;
            const int r = rem - ch * tp.rc_sw;
            e.off = (ch * p.g.H + kh * p.g.dh) * p.g.W + r;
            e.dy = static_cast<short>(kh * p.g.dh);
            e.dx = static_cast<short>(r);
            kt[k] = e;
        }
    }
    if (a_kind == A_IM2COL && !tp.a_pointwise) {
        // k -> (offset, dy, dx) table, filled cooperatively; k beyond K is never read as valid
        KEntry* kt = reinterpret_cast<KEntry*>(smem_raw);
        const int khw = p.g.KH * p.g.KW;
        for (int k = threadIdx.x; k < num_kb * BK; k += blockDim.x) {
            KEntry e;
            const int kk = k < p.K ? k : 0;
            const int ch = kk / khw;
            const int rem = kk - ch * khw;
            const int kh = rem / p.g.KW;
            const int kw = rem - kh * p.g.KW;
            e.off = (ch * p.g.H + kh * p.g.dh) * p.g.W + kw * p.g.dw;
            e.dy = static_cast<short>(kh * p.g.dh);
            e.dx = static_cast<short>(kw * p.g.dw);
            kt[k] = e;
        }
    }
    if (warp == kTsMmaWarp) {
        __syncwarp();
        ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), 512u);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
    volatile int* abort_p = &abort_flag;
    const long long wait_limit = p.wait_limit;  // clocks a bounded wait may take before it gives up

    // Register reallocation between the four warpgroups (the CTA starts with 512 x 128 = the
    // whole register file): loaders and the UMMA issuer need few, the epilogue and the producers
    // hold 32-64 values per thread in flight. 3 x 152 + 56 = 4 x 128, so every increase is
    // covered by the decrease; all warps pass here exactly once.
    if (warp >= kTsLoaderWarp0) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");

    if (warp < 4) {
        // ------------------------------------------------------------ epilogue
        uint32_t buf = 0, tphase = 0;
        uint32_t stage_buf = 0;  // which of the two staging blocks the next block of columns takes
        uint32_t tile_par = 0;   // alternates between consecutive tiles of this CTA
        // staging blocks of the output (TMA stores want their source on a 128-byte boundary)
        const uint32_t stage_base = (ptx::smem_u32(smem_raw) + static_cast<uint32_t>(tp.stage_off) + 127u) & ~127u;
        const int kc = tp.kc_blocks > 0 ? tp.kc_blocks : num_kb;
        float* part_row = reinterpret_cast<float*>(smem_raw + tp.sums_off) + warp * 32 + lane;
        bool alive = true;
        for (int t = blockIdx.x; alive && t < p.total_tiles; t += gridDim.x, tile_par ^= 1u) {
            int b, m0, n0;
            decode_tile(p, t, b, m0, n0);
            // Row form: where this tile's positions start. With image-aligned tiles (rc_tpi > 0,
            // see TsParams) a tile never crosses into the next image.
            const int OHW = p.g.OH * tp.rc_wv;
            int tile_img = -1, pos0 = 0;
            if (a_kind == A_ROWCONV) pos0 = rowconv_pos0(tp, m0 / kBM, OHW, tile_img);
            // all K-chunks but the last only feed the running sums
            for (int kb0 = 0; kb0 + kc < num_kb; kb0 += kc) {
                const bool wc = ptx::mbar_wait_bounded(ptx::smem_u32(&tfull_bar[buf]), tphase, abort_p, wait_limit);
                if (!__all_sync(0xffffffffu, wc)) {
                    alive = false;
                    break;
                }
                ptx::tc_fence_after();
                drain_chunk(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + buf * BN, BN, part_row, kb0 == 0);
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[buf]));
                if (++buf == static_cast<uint32_t>(nbuf)) {
                    buf = 0;
                    tphase ^= 1u;
                }
            }
            if (!alive) break;
            const float* part = kc < num_kb ? part_row : nullptr;
            const bool w = ptx::mbar_wait_bounded(ptx::smem_u32(&tfull_bar[buf]), tphase, abort_p, wait_limit);
            if constexpr (ES == 2) {
                if (tp.rc_tma) {
                    // The TMA-store epilogue below synchronises the four epilogue warps with a named
                    // barrier, which has no time limit: the warps must agree on whether this tile
                    // is processed. Every warp gets here (its wait is bounded), votes, and all
                    // leave together if any wait gave up.
                    const bool warp_ok = __all_sync(0xffffffffu, w);
                    if (lane == 0) epi_ok[tile_par][warp] = warp_ok ? 1 : 0;
                    epilogue_bar();
                    if (!(epi_ok[tile_par][0] && epi_ok[tile_par][1] && epi_ok[tile_par][2] && epi_ok[tile_par][3])) break;
                } else if (!__all_sync(0xffffffffu, w)) {
                    break;
                }
            } else {
                if (!__all_sync(0xffffffffu, w)) break;
            }
            ptx::tc_fence_after();
            if (a_kind == A_ROWCONV) {
                const int tn = n0 / BN;
                const int pos = pos0 + warp * tp.rc_T - tp.rc_lo + lane;
                const bool pos_ok = pos >= 0 && pos < p.M;
                const int img = pos_ok ? pos / OHW : 0;
                const int rem = pos_ok ? pos - img * OHW : 0;
                const int oh = rem / tp.rc_wv;
                const int u = rem - oh * tp.rc_wv;
                const bool produce = pos_ok && lane >= tp.rc_lo && lane < tp.rc_lo + tp.rc_T && u < p.g.OW &&
                                     (tile_img < 0 || img == tile_img);
                const int c0 = tn * tp.rc_cpt;
                const long long obase = static_cast<long long>(img) * p.g.out_img_stride +
                                        static_cast<long long>(b) * p.d_batch_stride +
                                        static_cast<long long>(oh) * p.g.OW + u;
                const uint32_t trow = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + buf * BN;
                const int nco = min(tp.rc_cpt, p.N - c0);
                const char* bias_g =
                    p.bias ? p.bias + (static_cast<long long>(b) * p.bias_stride + c0) * ES : nullptr;
                // how this tile's results leave: 0 one element per lane, 2 TMA stores of whole blocks
                // (image-aligned tiles)
                int mode = 0;
                int tile_slot = 0;
                uint32_t sbuf = 0;
                if constexpr (ES == 2) {
                    if (tp.rc_tma) {
                        mode = 2;
                        sbuf = stage_base + stage_buf * static_cast<uint32_t>(tp.rc_tma_buf);
                        tile_slot = warp * tp.rc_T + (lane - tp.rc_lo);  // position inside the tile
                    }
                }
                for (int co0 = 0; co0 < ((p.ablate & 8) ? 0 : nco); co0 += 16) {
                    // bias first (one value per lane, broadcast later): keeps loads out of the
                    // store loop, where they would serialise behind each store
                    float bv = 0.0f;
                    if (bias_g != nullptr && lane < 16 && co0 + lane < nco) {
                        const char* bp = bias_g + static_cast<long long>(co0 + lane) * ES;
                        if constexpr (ES == 4) bv = out_load<OUT_F32>(bp);
                        else bv = p.fmt == FMT_F16 ? out_load<OUT_F16>(bp) : out_load<OUT_BF16>(bp);
                    }
                    float acc[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) acc[e] = __shfl_sync(0xffffffffu, bv, e);
                    if (p.resid != nullptr && produce) {
                        // residual values, loaded before the taps so that their latency is hidden
                        const char* rp = p.resid + (obase + static_cast<long long>(c0 + co0) * p.g.P) * ES;
                        const long long cstride = static_cast<long long>(p.g.P) * ES;
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            if (co0 + e < nco) {
                                if constexpr (ES == 4) acc[e] += out_load<OUT_F32>(rp + e * cstride);
                                else acc[e] += p.fmt == FMT_F16 ? out_load<OUT_F16>(rp + e * cstride)
                                                                : out_load<OUT_BF16>(rp + e * cstride);
                            }
                        }
                    }
                    for (int kw = 0; kw < tp.rc_kw; ++kw) {
                        uint32_t d[16];
                        ptx::tmem_ld_32x16(trow + kw * tp.rc_cpt + co0, d);
                        ptx::tmem_ld_wait();
                        if (part != nullptr) {
#pragma unroll
                            for (int e = 0; e < 16; ++e)
                                d[e] = __float_as_uint(__uint_as_float(d[e]) + part[(kw * tp.rc_cpt + co0 + e) * 128]);
                        }
                        const int src = lane + kw - tp.rc_lo;
                        const bool in = static_cast<unsigned>(u + kw - tp.rc_lo) < static_cast<unsigned>(tp.rc_wv);
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const float tv = __uint_as_float(__shfl_sync(0xffffffffu, d[e], src & 31));
                            acc[e] += in ? tv : 0.0f;
                        }
                    }
                    if (p.relu) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) acc[e] = fmaxf(acc[e], 0.0f);
                    }
                    if constexpr (ES == 2) {
                        if (mode == 2) {
                            // block [channel][position of the tile]: one TMA store per 16 channels below
                            if (produce) {
                                const uint32_t sa = sbuf + static_cast<uint32_t>(co0 * 4 * tp.rc_T + tile_slot) * 2u;
#pragma unroll
                                for (int e = 0; e < 16; ++e) {
                                    const unsigned short h = p.fmt == FMT_F16 ? to_bits16<OUT_F16>(acc[e]) : to_bits16<OUT_BF16>(acc[e]);
                                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(sa + static_cast<uint32_t>(e * 4 * tp.rc_T) * 2u), "h"(h) : "memory");
                                }
                            }
                            continue;
                        }
                    }
                    if (produce && !((p.ablate & 16) && acc[0] != 123.456f)) {
                        char* optr = p.d + (obase + static_cast<long long>(c0 + co0) * p.g.P) * ES;
                        const long long cstride = static_cast<long long>(p.g.P) * ES;
                        if (co0 + 16 <= nco) {
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                if constexpr (ES == 4) out_store<OUT_F32>(optr + e * cstride, acc[e]);
                                else if (p.fmt == FMT_F16) out_store<OUT_F16>(optr + e * cstride, acc[e]);
                                else out_store<OUT_BF16>(optr + e * cstride, acc[e]);
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                if (co0 + e < nco) {
                                    if constexpr (ES == 4) out_store<OUT_F32>(optr + e * cstride, acc[e]);
                                    else if (p.fmt == FMT_F16) out_store<OUT_F16>(optr + e * cstride, acc[e]);
                                    else out_store<OUT_BF16>(optr + e * cstride, acc[e]);
                                }
                            }
                        }
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[buf]));
                if constexpr (ES == 2) {
                    if (mode == 2) {
                        // every staging thread makes its writes visible to the async proxy, then
                        // one thread hands the block to the TMA unit, 16 channels per store; rows
                        // beyond the image's last pixel are clipped by the hardware
                        ptx::fence_proxy_async_smem();
                        epilogue_bar();
                        if (threadIdx.x == 0 && !(p.ablate & 8)) {
                            const int x = pos0 - tile_img * OHW;
                            for (int co0 = 0; co0 < nco; co0 += 16)
                                ptx::tma_store_3d(&tmD, sbuf + static_cast<uint32_t>(co0 * 4 * tp.rc_T) * 2u, x,
                                                  b * p.N + c0 + co0, tile_img);
                            ptx::bulk_commit_group();
                            // the block written two tiles ago is reused next: its store must have read it
                            ptx::bulk_wait_group_read<1>();
                        }
                        stage_buf ^= 1u;
                    }
                }
                if (++buf == static_cast<uint32_t>(nbuf)) {
                    buf = 0;
                    tphase ^= 1u;
                }
                continue;
            }
            const int i = m0 + warp * 32 + lane;
            const bool row_ok = i < p.M;
            long long rowbase, colstride;
            if (a_kind == A_IM2COL) {
                const int img = i / p.g.P;
                const int pp = i - img * p.g.P;
                rowbase = static_cast<long long>(img) * p.g.out_img_stride +
                          static_cast<long long>(b) * p.d_batch_stride + pp;
                colstride = p.g.P;
            } else {
                rowbase = (p.d_offs ? p.d_offs[b] : static_cast<long long>(b) * p.d_batch_stride) + i;
                colstride = p.ldd;
            }
            const float alpha = p.alphas ? p.alphas[b] : p.alpha;
            const float beta = p.betas ? p.betas[b] : p.beta;
            const char* bias =
                p.bias ? p.bias + (static_cast<long long>(b) * p.bias_stride + n0) * ES : nullptr;
            const uint32_t trow = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + buf * BN;
            char* optr = p.d + (rowbase + static_cast<long long>(n0) * colstride) * ES;
            const int ncols = min(BN, p.N - n0);
            EpiExtra ex;
            ex.relu = p.relu != 0;
            ex.rdelta = p.resid ? p.resid - p.d : 0;
            const float beta_e = p.resid ? 1.0f : beta;  // a residual takes the place of the beta term
            if (p.ablate & 32) {
            } else if constexpr (ES == 4) {
                epilogue_dispatch<OUT_F32>(trow, ncols, optr, colstride * ES, row_ok, alpha, beta_e,
                                           bias, lane, part, false, ex);
            } else {
                const bool pair_ok = pair_store_ok(optr, rowbase, colstride, row_ok, lane);
                if (p.fmt == FMT_F16)
                    epilogue_dispatch<OUT_F16>(trow, ncols, optr, colstride * ES, row_ok, alpha,
                                               beta_e, bias, lane, part, pair_ok, ex);
                else
                    epilogue_dispatch<OUT_BF16>(trow, ncols, optr, colstride * ES, row_ok, alpha,
                                                beta_e, bias, lane, part, pair_ok, ex);
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[buf]));
            if (++buf == static_cast<uint32_t>(nbuf)) {
                buf = 0;
                tphase ^= 1u;
            }
        }
        if constexpr (ES == 2) {
            // TMA stores of the last blocks must have left shared memory before the CTA ends
            if (tp.rc_tma && threadIdx.x == 0) ptx::bulk_wait_group<0>();
        }
    } else if (warp >= kTsProducerWarp0 && warp < kTsLoaderWarp0) {
        // ------------------------------------------------------------ A producers (-> TMEM)
        const int q = warp & 3;                          // TMEM lane quadrant this warp may access
        const int par = (warp - kTsProducerWarp0) >> 2;  // which k-blocks (global parity) it takes
        const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
        uint32_t s = 0, ph = 0, gpar = 0;  // stage, its phase, parity of the running k-block count
        bool ok = true;
        for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
            int b, m0, n0;
            decode_tile(p, t, b, m0, n0);
            const long long a_boff =
                p.a_offs ? p.a_offs[b] : static_cast<long long>(b) * p.a.batch_stride;
            const int i = m0 + q * 32 + lane;
            const bool row_ok = i < p.M;
            long long pbase = 0;
            int ih0 = -(1 << 30), iw0 = -(1 << 30);
            if (a_kind == A_ROWCONV) {
                const int OHW = p.g.OH * tp.rc_wv;
                int tile_img;
                const int pos = rowconv_pos0(tp, m0 / kBM, OHW, tile_img) + q * tp.rc_T - tp.rc_lo + lane;
                if (pos >= 0 && pos < p.M) {
                    const int img = pos / OHW;
                    const int rem = pos - img * OHW;
                    const int oh = rem / tp.rc_wv;
                    iw0 = (rem - oh * tp.rc_wv) * tp.rc_sw;  // sw = 1: the input column itself, always inside the row
                    ih0 = oh * p.g.sh - p.g.pad_t;
                    pbase = a_boff + static_cast<long long>(img) * p.g.img_stride +
                            static_cast<long long>(ih0) * p.g.W + iw0;
                }
            } else if (a_kind == A_IM2COL) {
                if (row_ok) {
                    const int img = i / p.g.P;
                    const int pp = i - img * p.g.P;
                    const int oh = pp / p.g.OW;
                    const int ow = pp - oh * p.g.OW;
                    ih0 = oh * p.g.sh - p.g.pad_t;
                    iw0 = ow * p.g.sw - p.g.pad_l;
                    pbase = a_boff + static_cast<long long>(img) * p.g.img_stride +
                            static_cast<long long>(ih0) * p.g.W + iw0;
                }
            } else if (a_kind == A_DENSE_MN) {
                pbase = a_boff + i;
            } else {
                pbase = a_boff + static_cast<long long>(i) * p.a.ld;
            }
            for (int kb = 0; kb < num_kb; ++kb) {
                if (gpar != static_cast<uint32_t>(par)) {  // the other warp of this quadrant takes it
                    gpar ^= 1u;
                    if (++s == static_cast<uint32_t>(SA)) {
                        s = 0;
                        ph ^= 1u;
                    }
                    continue;
                }
                const int k0 = kb * BK;
                const int kcount = min(BK, p.K - k0);
                uint32_t v[32];  // fp32: raw values; 16-bit: two k per register (low half first)
                if (p.ablate & 1) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0x3f800000u + j;
                } else if (a_kind == A_ROWCONV && tp.rc_sw == 1 && kcount == BK && ktable[k0].dy == ktable[k0 + BK - 1].dy) {
                    // whole k-block inside one kh: consecutive k are consecutive channels
                    const KEntry e0 = ktable[k0];
                    const bool in = static_cast<unsigned>(ih0 + e0.dy) < static_cast<unsigned>(p.g.H);
                    const long long hw = static_cast<long long>(p.g.H) * p.g.W;
                    if constexpr (ES == 4) {
                        const uint32_t* x = reinterpret_cast<const uint32_t*>(p.a.base) + (in ? pbase + e0.off : 0);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = in ? x[j * hw] : 0u;
                    } else {
                        const unsigned short* x = reinterpret_cast<const unsigned short*>(p.a.base) + (in ? pbase + e0.off : 0);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t lo = in ? x[(2 * j) * hw] : 0u;
                            const uint32_t hi = in ? x[(2 * j + 1) * hw] : 0u;
                            v[j] = lo | (hi << 16);
                        }
                    }
                } else if (ES == 2 && a_kind == A_ROWCONV && tp.rc_pair) {
                    // stride_w = 2, 16-bit: k = 2j and 2j+1 are the two column phases of one
                    // (kh, channel): neighbours in memory, 4-byte aligned, both inside the row
                    const KEntry* te = ktable + k0;
                    const uint32_t* x32 = reinterpret_cast<const uint32_t*>(p.a.base);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const KEntry e = te[2 * j];
                        const bool in = 2 * j < kcount && static_cast<unsigned>(ih0 + e.dy) < static_cast<unsigned>(p.g.H);
                        v[j] = in ? x32[(pbase + e.off) >> 1] : 0u;
                    }
                } else if (a_kind == A_IM2COL && tp.a_pointwise) {
                    // 1x1 filter without padding: k is the channel, every tap lies inside the
                    // image, consecutive k are H*W elements apart (no table, no bounds tests)
                    const long long hw = static_cast<long long>(p.g.H) * p.g.W;
                    if constexpr (ES == 4) {
                        const uint32_t* x = reinterpret_cast<const uint32_t*>(p.a.base) + pbase + k0 * hw;
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = (row_ok && j < kcount) ? x[j * hw] : 0u;
                    } else {
                        const unsigned short* x =
                            reinterpret_cast<const unsigned short*>(p.a.base) + pbase + k0 * hw;
                        if (row_ok && kcount == BK) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const uint32_t lo = x[(2 * j) * hw];
                                const uint32_t hi = x[(2 * j + 1) * hw];
                                v[j] = lo | (hi << 16);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const uint32_t lo = (row_ok && 2 * j < kcount) ? x[(2 * j) * hw] : 0u;
                                const uint32_t hi = (row_ok && 2 * j + 1 < kcount) ? x[(2 * j + 1) * hw] : 0u;
                                v[j] = lo | (hi << 16);
                            }
                        }
                    }
                } else if (a_kind == A_IM2COL || a_kind == A_ROWCONV) {
                    const KEntry* te = ktable + k0;
                    if constexpr (ES == 4) {
                        const uint32_t* x = reinterpret_cast<const uint32_t*>(p.a.base);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const KEntry e = te[j];
                            const bool in = j < kcount &&
                                            static_cast<unsigned>(ih0 + e.dy) < static_cast<unsigned>(p.g.H) &&
                                            static_cast<unsigned>(iw0 + e.dx) < static_cast<unsigned>(p.g.W);
                            v[j] = in ? x[pbase + e.off] : 0u;
                        }
                    } else {
                        const unsigned short* x = reinterpret_cast<const unsigned short*>(p.a.base);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const KEntry e0 = te[2 * j], e1 = te[2 * j + 1];
                            const bool in0 = 2 * j < kcount &&
                                             static_cast<unsigned>(ih0 + e0.dy) < static_cast<unsigned>(p.g.H) &&
                                             static_cast<unsigned>(iw0 + e0.dx) < static_cast<unsigned>(p.g.W);
                            const bool in1 = 2 * j + 1 < kcount &&
                                             static_cast<unsigned>(ih0 + e1.dy) < static_cast<unsigned>(p.g.H) &&
                                             static_cast<unsigned>(iw0 + e1.dx) < static_cast<unsigned>(p.g.W);
                            const uint32_t lo = in0 ? x[pbase + e0.off] : 0u;
                            const uint32_t hi = in1 ? x[pbase + e1.off] : 0u;
                            v[j] = lo | (hi << 16);
                        }
                    }
                } else if (a_kind == A_DENSE_MN) {
                    if constexpr (ES == 4) {
                        const uint32_t* x = reinterpret_cast<const uint32_t*>(p.a.base) + pbase;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = (row_ok && j < kcount) ? x[static_cast<long long>(k0 + j) * p.a.ld] : 0u;
                    } else {
                        const unsigned short* x = reinterpret_cast<const unsigned short*>(p.a.base) + pbase;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t lo = (row_ok && 2 * j < kcount)
                                                    ? x[static_cast<long long>(k0 + 2 * j) * p.a.ld] : 0u;
                            const uint32_t hi = (row_ok && 2 * j + 1 < kcount)
                                                    ? x[static_cast<long long>(k0 + 2 * j + 1) * p.a.ld] : 0u;
                            v[j] = lo | (hi << 16);
                        }
                    }
                } else {  // A_DENSE_K: this thread's row is contiguous along k
                    const char* x = p.a.base + (pbase + k0) * ES;
                    const bool vec = row_ok && kcount == BK && (reinterpret_cast<uintptr_t>(x) & 15u) == 0u;
                    if (vec) {
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint4 u = reinterpret_cast<const uint4*>(x)[c];
                            v[4 * c + 0] = u.x;
                            v[4 * c + 1] = u.y;
                            v[4 * c + 2] = u.z;
                            v[4 * c + 3] = u.w;
                        }
                    } else if constexpr (ES == 4) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = (row_ok && j < kcount) ? reinterpret_cast<const uint32_t*>(x)[j] : 0u;
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t lo = (row_ok && 2 * j < kcount)
                                                    ? reinterpret_cast<const unsigned short*>(x)[2 * j] : 0u;
                            const uint32_t hi = (row_ok && 2 * j + 1 < kcount)
                                                    ? reinterpret_cast<const unsigned short*>(x)[2 * j + 1] : 0u;
                            v[j] = lo | (hi << 16);
                        }
                    }
                }
                const bool w = ptx::mbar_wait_bounded(ptx::smem_u32(&empty_a[s]), ph ^ 1u, abort_p, wait_limit);
                if (!__all_sync(0xffffffffu, w)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t slot = tmem_base + lane_base + a_col0 + s * A_COLS;
                if (!(p.ablate & 4)) {
                    if constexpr (ES == 4) {
                        uint32_t lo[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) split_tf32(v[j], v[j], lo[j]);
                        tmem_st_32x32(slot, v);
                        tmem_st_32x32(slot + 32, lo);
                    } else {
                        tmem_st_32x32(slot, v);
                    }
                    tmem_st_wait();
                } else {
                    uint32_t acc = 0;
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc ^= v[j];
                    if (acc == 0x12345678u) p.status[1] = 1;  // keeps the loads alive
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&full_a[s]));
                gpar ^= 1u;
                if (++s == static_cast<uint32_t>(SA)) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp >= kTsLoaderWarp0 && warp < kTsMmaWarp) {
        // ------------------------------------------------------------ B loaders (-> swizzled smem)
        const int lt = threadIdx.x - kTsLoaderWarp0 * 32;
        const int c = lt & 7;
        const int l0 = lt >> 3;  // 0..kTsLoaderLines-1
        const bool b_atom32 = ES == 4 && !p.b.k_major;
        uint32_t s = 0, ph = 0;
        bool ok = true;
        if (tp.b_tma) {
            if (warp == kTsLoaderWarp0) {
                // TMA producer: raw fp32 tile of Bu into the hi image of the stage
                // (the whole warp runs the loop, converged; one lane issues: see the UMMA issuer)
                {
                    const bool leader = ptx::elect_one();
                    if (leader) ptx::tma_prefetch_desc(&tmB);
                    for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                        int b, m0, n0;
                        decode_tile(p, t, b, m0, n0);
                        const int bb = p.b.batch_stride ? b : 0;
                        for (int kb = 0; kb < num_kb; ++kb) {
                            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&empty_b[s]), ph ^ 1u, abort_p, wait_limit))) {
                                ok = false;
                                break;
                            }
                            const uint32_t bar = ptx::smem_u32(&raw_b[s]);
                            const uint32_t sB = smem0 + s * stage_bytes;
                            if (leader) ptx::mbar_arrive_expect_tx(bar, b_tile);
                            if (p.b.k_major) {
                                if (leader) ptx::tma_load_3d(sB, &tmB, bar, kb * BK, n0, bb);
                            } else {
                                for (int g = 0; g < BN / BK; ++g)
                                    if (leader) ptx::tma_load_3d(sB + g * BK * 128, &tmB, bar, n0 + g * BK, kb * BK, bb);
                            }
                            if (++s == static_cast<uint32_t>(SB)) {
                                s = 0;
                                ph ^= 1u;
                            }
                        }
                    }
                }
            } else {
                // Converters (warps 13-14). The tensor core reads a raw fp32 word as its tf32
                // truncation, so the tile TMA delivered already is the hi image; only
                // lo = x - trunc(x) is written, chunk by chunk where the data lies (the operation
                // is element-wise, so the swizzle does not matter).
                const int ct = threadIdx.x - (kTsLoaderWarp0 + 1) * 32;  // 0..63
                for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                    for (int kb = 0; kb < num_kb; ++kb) {
                        const bool w = ptx::mbar_wait_bounded(ptx::smem_u32(&raw_b[s]), ph, abort_p, wait_limit);
                        if (!__all_sync(0xffffffffu, w)) {
                            ok = false;
                            break;
                        }
                        const uint32_t sB = smem0 + s * stage_bytes;
                        for (uint32_t o = ct * 16u; o < b_tile; o += 64u * 16u) {
                            uint4 v;
                            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                                         : "r"(sB + o)
                                         : "memory");
                            uint4 lo;
                            lo.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(v.x & 0xffffe000u));
                            lo.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(v.y & 0xffffe000u));
                            lo.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(v.z & 0xffffe000u));
                            lo.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(v.w & 0xffffe000u));
                            st_shared_v4(sB + b_tile + o, lo);
                        }
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&full_b[s]));
                        if (++s == static_cast<uint32_t>(SB)) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                }
            }
            ok = false;  // skip the gather loop below
        }
        if (tp.b_packed != nullptr) {
            // stage images were prepared in global memory: the first loader warp streams them in with
            // bulk copies (converged, one lane issuing: see the UMMA issuer), the other loader
            // threads have nothing to do
            if (warp == kTsLoaderWarp0) {
                const bool leader = ptx::elect_one();
                // the packing grid launched just before this one must have completed
                asm volatile("griddepcontrol.wait;" ::: "memory");
                for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                    if (tp.b_resident && t != static_cast<int>(blockIdx.x)) break;  // loaded once, kept
                    int b, m0, n0;
                    decode_tile(p, t, b, m0, n0);
                    const unsigned char* src =
                        tp.b_packed + (static_cast<long long>(b) * p.tiles_n + n0 / BN) * num_kb * stage_bytes;
                    for (int kb = 0; kb < num_kb; ++kb) {
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&empty_b[s]), ph ^ 1u, abort_p, wait_limit))) {
                            ok = false;
                            break;
                        }
                        const uint32_t bar = ptx::smem_u32(&full_b[s]);
                        const uint32_t sB = smem0 + s * stage_bytes;
                        if (leader) ptx::mbar_arrive_expect_tx(bar, stage_bytes);
                        for (uint32_t o = 0; o < stage_bytes; o += 8192u)
                            if (leader) ptx::bulk_load(sB + o, src + static_cast<long long>(kb) * stage_bytes + o,
                                           min(8192u, stage_bytes - o), bar);
                        if (++s == static_cast<uint32_t>(SB)) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                }
            }
            ok = false;  // skip the gather loop below
        }
        for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
            int b, m0, n0;
            decode_tile(p, t, b, m0, n0);
            const long long b_boff =
                p.b_offs ? p.b_offs[b] : static_cast<long long>(b) * p.b.batch_stride;
            for (int kb = 0; kb < num_kb; ++kb) {
                const bool w = ptx::mbar_wait_bounded(ptx::smem_u32(&empty_b[s]), ph ^ 1u, abort_p, wait_limit);
                if (!__all_sync(0xffffffffu, w)) {
                    ok = false;
                    break;
                }
                const uint32_t sB = smem0 + s * stage_bytes;
                for (int L0 = l0; L0 < BN; L0 += 4 * kTsLoaderLines) {
                    uint4 v[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int L = L0 + q * kTsLoaderLines;
                        if (L >= BN || (p.ablate & 2)) {
                            v[q] = make_uint4(0u, 0u, 0u, 0u);
                        } else if (a_kind == A_ROWCONV) {
                            // column L = (kw, co): W[c0+co][c][kh][kw] for k' = kh*C + c
                            const int kw = L / tp.rc_cpt;
                            const int co = (n0 / BN) * tp.rc_cpt + (L - kw * tp.rc_cpt);
                            const RowTaps rt = row_taps(tp);
                            v[q] = load_chunk_rowconv<ES>(p.b.base, b_boff + static_cast<long long>(co) * rt.cg * rt.KH * rt.KW,
                                                          rt, kw, co < p.N, kb * BK + c * CPE, p.K);
                        } else if (p.b.k_major) {
                            v[q] = load_chunk_dense<ES>(p.b, b_boff, n0 + L, p.N, kb * BK + c * CPE, p.K);
                        } else {
                            v[q] = load_chunk_dense<ES>(p.b, b_boff, kb * BK + (L % BK), p.K,
                                                        n0 + (L / BK) * BK + c * CPE, p.N);
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int L = L0 + q * kTsLoaderLines;
                        if (L < BN) store_chunk<ES>(sB, sB + b_tile, L, c, v[q], b_atom32);
                    }
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&full_b[s]));
                if (++s == static_cast<uint32_t>(SB)) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp == kTsMmaWarp) {
        // ------------------------------------------------------------ UMMA issuer
        // The whole warp runs the loop, converged, and one elected lane issues, so that loop state
        // and descriptors stay in uniform registers (see contraction.cuh).
        {
            const uint32_t idesc =
                ptx::make_idesc(p.fmt == FMT_F32 ? 2u : static_cast<uint32_t>(p.fmt), 0u,
                                p.b.k_major ? 0u : 1u, kBM, BN);
            const uint32_t b_step = p.b.k_major ? KSTEP_K : KSTEP_MN;
            const uint32_t b_lbo = p.b.k_major ? 16u : static_cast<uint32_t>(BK) * 128u;
            const uint32_t b_mode = (ES == 4 && !p.b.k_major) ? 1u : 2u;
            const uint32_t b_sbo = b_mode == 1u ? 512u : 1024u;
            const uint64_t db0 = ptx::make_smem_desc(smem0, b_lbo, b_sbo, b_mode);
            const uint32_t lo_units = b_tile >> 4;
            uint32_t s = 0, ph = 0, sb = 0, phb = 0, buf = 0, tphase = 0;  // A slot / B stage and their phases
            bool ok = true;
            const int kc = tp.kc_blocks > 0 ? tp.kc_blocks : num_kb;
            for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                for (int kb0 = 0; ok && kb0 < num_kb; kb0 += kc) {  // one accumulator per K-chunk
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&tempty_bar[buf]), tphase ^ 1u, abort_p, wait_limit))) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    const int kb1 = min(kb0 + kc, num_kb);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        // (a resident filter bank arrives once: only the first tile waits for it)
                        const bool wait_b = !tp.b_resident || t == static_cast<int>(blockIdx.x);
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(&full_a[s]), ph, abort_p, wait_limit) &&
                                                         (!wait_b || ptx::mbar_wait_bounded(ptx::smem_u32(&full_b[sb]), phb, abort_p, wait_limit)))) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint32_t st_units = (sb * stage_bytes) >> 4;
                        const uint32_t a_slot = tmem_base + a_col0 + s * A_COLS;
                        if (ptx::elect_one()) {
#pragma unroll
                        for (int ks = 0; ks < BK / UMMA_K; ++ks) {
                            const uint64_t db = db0 + (st_units + ((ks * b_step) >> 4));
                            const uint32_t acc = ((kb - kb0) | ks) ? 1u : 0u;
                            const uint32_t a_hi = a_slot + ks * A_KSTEP_COLS;
                            if constexpr (ES == 2) {
                                umma_ts_f16(d_tmem, a_hi, db, idesc, acc);
                            } else {
                                umma_ts_tf32(d_tmem, a_hi + 32, db, idesc, acc);
                                umma_ts_tf32(d_tmem, a_hi, db + lo_units, idesc, 1u);
                                umma_ts_tf32(d_tmem, a_hi, db, idesc, 1u);
                            }
                        }
                        ptx::umma_commit(ptx::smem_u32(&empty_a[s]));
                        if (!tp.b_resident) ptx::umma_commit(ptx::smem_u32(&empty_b[sb]));
                        }
                        __syncwarp();
                        if (++s == static_cast<uint32_t>(SA)) {
                            s = 0;
                            ph ^= 1u;
                        }
                        if (++sb == static_cast<uint32_t>(SB)) {
                            sb = 0;
                            phb ^= 1u;
                        }
                    }
                    if (ok && !p.skip_tile_commit && ptx::elect_one()) ptx::umma_commit(ptx::smem_u32(&tfull_bar[buf]));
                    __syncwarp();
                    if (++buf == static_cast<uint32_t>(nbuf)) {
                        buf = 0;
                        tphase ^= 1u;
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
    if (warp == kTsMmaWarp) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, 512u);
    }
}

}  // namespace dlfb200

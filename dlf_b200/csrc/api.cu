// extern "C" boundary of the library (declared in include/dlf_b200.h): argument checks in the
// reference's order, reduction of every call to the canonical problem of contraction.cuh,
// tile / loader selection, TMA descriptor encoding and the launch. No call here allocates
// device memory except the one-off 4-byte status word per device.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <climits>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/dlf_b200.h"
#include "channels_last.cuh"
#include "contraction.cuh"
#include "contraction_ts.cuh"
#include "conv_small.cuh"
#include "conv_halo.cuh"
#include "level3.cuh"
#include "pooling.cuh"

using namespace dlfb200;

namespace {

// gpgpu::blas::StatusCode values used here (gpgpu/include/gblas.h:43-107)
enum : int {
    kSuccess = 0,
    kInvalidValue = -30,
    kNotImplemented = -1024,
    kInvalidMatrixA = -1022,
    kInvalidMatrixB = -1021,
    kInvalidMatrixC = -1020,
    kInvalidDimension = -1017,
    kInvalidLeadDimA = -1016,
    kInvalidLeadDimB = -1015,
    kInvalidLeadDimC = -1014,
    kInsufficientMemoryTemp = -2050,
    kInvalidBatchCount = -2049,
    kNoHalfPrecision = -2045,
    kUnexpectedError = -2039,
};

constexpr int kMaxDevices = 64;
constexpr int kSmemPerBlockOptin = 232448;  // 227 KB

struct DeviceState {
    bool ready = false;
    int num_sms = 0;
    int* status = nullptr;
    int static_smem_tma = 0;
    int static_smem_tma4 = 0;  // the instantiation with four sets of epilogue warps
    int static_smem_tma3 = 0;  // ... with three
    int static_smem_gen2 = 0;
    int static_smem_gen4 = 0;
    int static_smem_ts2 = 0;
    int static_smem_ts4 = 0;
    int static_smem_pair = 0;
    int static_smem_small = 0;
    int static_smem_halo = 0;
    int max_pair_clusters = 0;  // co-resident CTA pairs of the pair kernel (0 = not usable)
    PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    PFN_cuTensorMapEncodeIm2col_v12000 encode_im2col = nullptr;  // null: the driver has none
};

DeviceState g_dev[kMaxDevices];
std::mutex g_mu;
std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_force_bn{0};
std::atomic<int> g_force_generic{0};

#define CUDA_TRY(expr)                                   \
    do {                                                 \
        cudaError_t e__ = (expr);                        \
        if (e__ != cudaSuccess) return static_cast<int>(e__); \
    } while (0)

// The device a call works on is the one its stream belongs to (the reference binds a queue to its
// context's device, gpgpu/src/gpgpu_cu.cpp:174-204), not whatever device happens to be current on
// the calling thread. The guard makes that device current for the duration of the call and puts
// the previous one back; the legacy default stream (null) means the current device.
struct StreamDevice {
    int dev = 0;
    int prev = -1;
    int rc = kSuccess;
    explicit StreamDevice(cudaStream_t s) {
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) {
            rc = static_cast<int>(e);
            return;
        }
        if (s != nullptr && s != cudaStreamLegacy && s != cudaStreamPerThread) {
            // a stream that is being captured into a CUDA graph may not be queried (the query fails and
            // invalidates the capture): such a call works on the current device, which a capture
            // requires to be the stream's anyway
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) {
                (void)cudaGetLastError();
                cap = cudaStreamCaptureStatusNone;
            }
            if (cap != cudaStreamCaptureStatusNone) return;
            int sd = dev;
            e = cudaStreamGetDevice(s, &sd);
            if (e != cudaSuccess) {
                rc = static_cast<int>(e);
                return;
            }
            if (sd != dev) {
                e = cudaSetDevice(sd);
                if (e != cudaSuccess) {
                    rc = static_cast<int>(e);
                    return;
                }
                prev = dev;
                dev = sd;
            }
        }
    }
    ~StreamDevice() {
        if (prev >= 0) (void)cudaSetDevice(prev);
    }
    StreamDevice(const StreamDevice&) = delete;
    StreamDevice& operator=(const StreamDevice&) = delete;
};

// The tensor-memory-operand kernel exists once per element size and operand kind (see
// contraction_ts.cuh): attributes are set on all of them, the largest static shared-memory use is
// what the launch arithmetic counts with.
template <int ES>
int setup_ts_kernels(int* static_smem) {
    cudaFuncAttributes fa;
    int worst = 0;
#define DLF_TS_SETUP(AK)                                                                              \
    CUDA_TRY(cudaFuncGetAttributes(&fa, contraction_ts_kernel<ES, AK>));                              \
    worst = std::max(worst, static_cast<int>(fa.sharedSizeBytes));
    DLF_TS_SETUP(A_DENSE_MN)
    DLF_TS_SETUP(A_IM2COL)
    DLF_TS_SETUP(A_ROWCONV)
#undef DLF_TS_SETUP
#define DLF_TS_ATTR(AK)                                                                               \
    CUDA_TRY(cudaFuncSetAttribute(contraction_ts_kernel<ES, AK>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  kSmemPerBlockOptin - worst));
    DLF_TS_ATTR(A_DENSE_MN)
    DLF_TS_ATTR(A_IM2COL)
    DLF_TS_ATTR(A_ROWCONV)
#undef DLF_TS_ATTR
    *static_smem = worst;
    return kSuccess;
}

template <int ES>
cudaError_t launch_ts_kernel(const cudaLaunchConfig_t* cfg, const TsParams& tp, const CUtensorMap& tm_b,
                             const CUtensorMap& tm_d) {
    if (tp.a_kind == A_ROWCONV) return cudaLaunchKernelEx(cfg, contraction_ts_kernel<ES, A_ROWCONV>, tp, tm_b, tm_d);
    if (tp.a_kind == A_IM2COL) return cudaLaunchKernelEx(cfg, contraction_ts_kernel<ES, A_IM2COL>, tp, tm_b, tm_d);
    return cudaLaunchKernelEx(cfg, contraction_ts_kernel<ES, A_DENSE_MN>, tp, tm_b, tm_d);
}

int ensure_device(DeviceState** out) {
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return kInvalidValue;
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        CUDA_TRY(cudaDeviceGetAttribute(&st.num_sms, cudaDevAttrMultiProcessorCount, dev));
        int major = 0;
        CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return kNotImplemented;  // tcgen05 kernels: sm_100a only
        cudaFuncAttributes fa;
        // the TMA-fed kernel exists with two, three and four sets of epilogue warps, each with and
        // without residual boxes fetched by TMA; a pair shares the launch arithmetic, which counts
        // with the larger static shared-memory use of the two
#define DLF_TMA_SETUP(ESETS, FIELD)                                                                       \
        {                                                                                                 \
            auto k0 = contraction_kernel<2, true, false, ESETS, false>;                                   \
            auto k1 = contraction_kernel<2, true, false, ESETS, true>;                                    \
            CUDA_TRY(cudaFuncGetAttributes(&fa, k0));                                                     \
            int worst = static_cast<int>(fa.sharedSizeBytes);                                             \
            CUDA_TRY(cudaFuncGetAttributes(&fa, k1));                                                     \
            worst = std::max(worst, static_cast<int>(fa.sharedSizeBytes));                                \
            st.FIELD = worst;                                                                             \
            if (ESETS != 2) {                                                                             \
                CUDA_TRY(cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPerBlockOptin - worst)); \
            }                                                                                             \
            CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPerBlockOptin - worst));     \
        }
        DLF_TMA_SETUP(2, static_smem_tma)
        DLF_TMA_SETUP(4, static_smem_tma4)
        DLF_TMA_SETUP(3, static_smem_tma3)
#undef DLF_TMA_SETUP
        CUDA_TRY(cudaFuncGetAttributes(&fa, contraction_kernel<2, false>));
        st.static_smem_gen2 = static_cast<int>(fa.sharedSizeBytes);
        CUDA_TRY(cudaFuncGetAttributes(&fa, contraction_kernel<4, false>));
        st.static_smem_gen4 = static_cast<int>(fa.sharedSizeBytes);
        CUDA_TRY(cudaFuncSetAttribute(contraction_kernel<2, true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemPerBlockOptin - st.static_smem_tma));
        CUDA_TRY(cudaFuncSetAttribute(contraction_kernel<2, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemPerBlockOptin - st.static_smem_gen2));
        CUDA_TRY(cudaFuncSetAttribute(contraction_kernel<4, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemPerBlockOptin - st.static_smem_gen4));
        CUDA_TRY(cudaFuncGetAttributes(&fa, conv_halo_kernel));
        st.static_smem_halo = static_cast<int>(fa.sharedSizeBytes);
        CUDA_TRY(cudaFuncSetAttribute(conv_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemPerBlockOptin - st.static_smem_halo));
        CUDA_TRY(cudaFuncGetAttributes(&fa, conv_small_kernel));
        st.static_smem_small = static_cast<int>(fa.sharedSizeBytes);
        CUDA_TRY(cudaFuncSetAttribute(conv_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemPerBlockOptin - st.static_smem_small));
        {
            int rc2 = setup_ts_kernels<2>(&st.static_smem_ts2);
            if (rc2 != kSuccess) return rc2;
            rc2 = setup_ts_kernels<4>(&st.static_smem_ts4);
            if (rc2 != kSuccess) return rc2;
        }
        {
            auto pair_kernel = contraction_kernel<2, true, true>;
            CUDA_TRY(cudaFuncGetAttributes(&fa, pair_kernel));
            st.static_smem_pair = static_cast<int>(fa.sharedSizeBytes);
            const int dyn = kSmemPerBlockOptin - st.static_smem_pair;
            CUDA_TRY(cudaFuncSetAttribute(pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * st.num_sms, 1, 1);
            cfg.blockDim = dim3(kThreadsPair, 1, 1);
            cfg.dynamicSmemBytes = static_cast<size_t>(dyn);
            cudaLaunchAttribute attr;
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = 2;
            attr.val.clusterDim.y = 1;
            attr.val.clusterDim.z = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            int n = 0;
            const cudaError_t oe = cudaOccupancyMaxActiveClusters(&n, pair_kernel, &cfg);
            if (oe == cudaSuccess) st.max_pair_clusters = n;
            if (std::getenv("DLF_B200_DEBUG"))
                std::fprintf(stderr, "dlf_b200: pair kernel static smem %d, dyn %d, max clusters %d (%s)\n",
                             st.static_smem_pair, dyn, n, cudaGetErrorString(oe));
            (void)cudaGetLastError();
        }
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return kUnexpectedError;
        st.encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
        fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            st.encode_im2col = reinterpret_cast<PFN_cuTensorMapEncodeIm2col_v12000>(fn);
        (void)cudaGetLastError();
        CUDA_TRY(cudaMalloc(&st.status, 2 * sizeof(int)));
        CUDA_TRY(cudaMemset(st.status, 0, 2 * sizeof(int)));
        st.ready = true;
    }
    *out = &st;
    return kSuccess;
}

bool dtype_info(int dtype, int& fmt, int& es) {
    switch (dtype) {
        case DLF_B200_HALF: fmt = FMT_F16; es = 2; return true;
        case DLF_B200_BFLOAT16: fmt = FMT_BF16; es = 2; return true;
        case DLF_B200_SINGLE: fmt = FMT_F32; es = 4; return true;
        default: return false;
    }
}

float scalar_to_float(int fmt, const void* p) {
    if (fmt == FMT_F16) {
        __half h;
        std::memcpy(&h, p, 2);
        return __half2float(h);
    }
    if (fmt == FMT_BF16) {
        __nv_bfloat16 h;
        std::memcpy(&h, p, 2);
        return __bfloat162float(h);
    }
    float f;
    std::memcpy(&f, p, 4);
    return f;
}

struct Problem {
    int fmt = 0, es = 0;
    long long M = 0, N = 0, K = 0, batch = 1;
    GenOperand a{}, b{};
    char* d = nullptr;
    long long ldd = 0, d_batch_stride = 0;
    float alpha = 1.f, beta = 0.f;
    const long long* a_offs = nullptr;
    const long long* b_offs = nullptr;
    const long long* d_offs = nullptr;
    const float* alphas = nullptr;
    const float* betas = nullptr;
    const char* bias = nullptr;
    long long bias_stride = 0;
    int bias_rows = 0;  // bias per row of D (channels-last convolution with the filter bank as operand A)
    const int* a_idx = nullptr;  // per batch entry: index into the strided sequence of A / B / D matrices (device)
    const int* b_idx = nullptr;
    const int* d_idx = nullptr;
    long long a_count = 0, b_count = 0, d_count = 0;  // matrices the index tables reach (batch extents of the tensor maps)
    bool narrow_boxes = false;  // row-staged epilogue with 32-column boxes even where 64-column ones are possible
    const char* resid = nullptr;
    int relu = 0;
    Im2colGeom g{};
    // row form of a convolution (contraction_ts.cuh, A_ROWCONV); rc_kw == 0: not used
    int rc_kw = 0, rc_cpt = 0, rc_T = 0, rc_lo = 0, rc_sw = 1, rc_wv = 0, rc_dmin = 0;
    int rc_tpi = 0;  // row form with image-aligned tiles and TMA stores: tiles per image (0: off)
    // caller-provided scratch for the packed filter bank of a convolution (may be null)
    unsigned char* pack_ws = nullptr;
    size_t pack_ws_bytes = 0;
    // channels-last route of a convolution (channels_last.cuh): a.base is the channels-last copy.
    // a_cl == 1: operand A comes through an im2col-mode tensor map over (cl_n, cl_h, cl_w, cl_cp);
    // out_nchw: rows are output pixels of an NCHW tensor (g.P, g.out_img_stride)
    int a_cl = 0, cl_cblocks = 0;
    // cl_swap: rows of the problem are output channels (a = filter bank), columns are output pixels
    // (b = the channels-last copy; with a_cl == 1 through the im2col-mode map); out_nchw == 3 and
    // out_vec = elements per store of one lane
    int cl_swap = 0, out_vec = 1;
    int out_nchw = 0;
    long long cl_n = 0, cl_h = 0, cl_w = 0, cl_cp = 0;
    bool d_f32 = false;  // 16-bit operands with fp32 output (partial products of a K-split GEMM)
    bool no_ts = false;  // convolution whose taps overflow the k table's 16/32-bit fields
};

bool tma_ok(const GenOperand& op, int es, long long rows, long long K, long long batch) {
    if (op.im2col) return false;
    if (reinterpret_cast<uintptr_t>(op.base) & 15u) return false;
    const long long lines = op.k_major ? rows : K;
    if (lines > 1 && (op.ld * es) % 16 != 0) return false;
    if (batch > 1 && op.batch_stride != 0 && (op.batch_stride * es) % 16 != 0) return false;
    if (op.ld * es >= (1ll << 40) || op.batch_stride * es >= (1ll << 40)) return false;
    return true;
}

// 3-D tiled tensor map {contiguous dim, line dim, batch} with 128-byte swizzle and zero fill.
int encode_map(const DeviceState& st, CUtensorMap* map, const GenOperand& op, int es,
               long long rows, long long K, long long batch, int box_rows) {
    const int BK = 128 / es;
    cuuint64_t dims[3];
    cuuint64_t strides[2];
    cuuint32_t box[3];
    cuuint32_t estr[3] = {1, 1, 1};
    const long long ld_bytes = (op.ld * es) % 16 == 0 && op.ld > 0 ? op.ld * es : 16;
    if (op.k_major) {
        dims[0] = static_cast<cuuint64_t>(K);
        dims[1] = static_cast<cuuint64_t>(rows);
        box[0] = BK;
        box[1] = box_rows;
    } else {
        dims[0] = static_cast<cuuint64_t>(rows);
        dims[1] = static_cast<cuuint64_t>(K);
        box[0] = BK;  // E rows of the MN-major operand
        box[1] = BK;
    }
    const bool batched = batch > 1 && op.batch_stride != 0;
    dims[2] = batched ? static_cast<cuuint64_t>(batch) : 1;
    strides[0] = static_cast<cuuint64_t>(ld_bytes);
    strides[1] = batched ? static_cast<cuuint64_t>(op.batch_stride * es)
                         : static_cast<cuuint64_t>(ld_bytes) * dims[1];
    if (strides[1] >= (1ull << 40)) strides[1] = static_cast<cuuint64_t>(ld_bytes);
    box[2] = 1;
    const CUtensorMapDataType dt =
        es == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    // MN-major fp32 tiles use the 32-byte-atom form of the 128-byte swizzle (see contraction.cuh)
    const CUtensorMapSwizzle swz =
        (es == 4 && !op.k_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    CUresult r = st.encode(map, dt, 3, const_cast<char*>(op.base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? kSuccess : kUnexpectedError;
}

// im2col-mode tensor map over the channels-last copy (C', W, H, N) of a convolution's input: one
// load fetches 128 filter windows x 64 channels. The bounding box of window origins starts at
// (-pad_left, -pad_top) and is as wide as the outputs need, (OW-1)*stride_w + 1 origins per row
// (whatever the caller's right / bottom padding says: the tensor-map unit zero-fills what lies
// outside the image); the traversal strides are the convolution's strides. Corners are limited to
// [-128, 127] by the 4-D form of the map.
int encode_im2col_map(const DeviceState& st, CUtensorMap* map, const Problem& q, const char* base, int windows) {
    if (st.encode_im2col == nullptr) return kNotImplemented;
    const Im2colGeom& g = q.g;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(q.cl_cp), static_cast<cuuint64_t>(q.cl_w),
                          static_cast<cuuint64_t>(q.cl_h), static_cast<cuuint64_t>(q.cl_n)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(q.cl_cp * 2), static_cast<cuuint64_t>(q.cl_w * q.cl_cp * 2),
                             static_cast<cuuint64_t>(q.cl_h * q.cl_w * q.cl_cp * 2)};
    int lower[2] = {-g.pad_l, -g.pad_t};
    int upper[2] = {(g.OW - 1) * g.sw + 1 - g.W - g.pad_l, (g.OH - 1) * g.sh + 1 - g.H - g.pad_t};
    for (int i = 0; i < 2; ++i)
        if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) return kNotImplemented;
    cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(g.sw), static_cast<cuuint32_t>(g.sh), 1};
    CUresult r = st.encode_im2col(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<char*>(base), dims, strides,
                                  lower, upper, 64, static_cast<cuuint32_t>(windows), estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? kSuccess : kNotImplemented;
}

// Tensor map for TMA stores of the output (blocks of 32 rows x 32 or 64 columns, no swizzle): only when nothing of C has
// to be read (beta == 0, no per-batch tables) and D's base and strides are 16-byte multiples.
bool encode_output_map(const DeviceState& st, CUtensorMap* map, const Problem& q, unsigned box_cols) {
    if (q.out_nchw == 3) {
        // swapped roles (rows = channels, columns = pixels): boxes of 32 pixels x 32 channels of the
        // NCHW output {pixels of a plane, channels, images}; images are the batch entries in the
        // batched form (N = P), else N / P. The staging block is 64-byte swizzled: its rows are 64
        // bytes, and lanes that write 16 bytes each at a 64-byte stride would otherwise use two of
        // the eight 16-byte bank groups (four times the shared-memory wavefronts)
        const long long P = q.g.P;
        const bool ok = q.es == 2 && q.beta == 0.0f && (reinterpret_cast<uintptr_t>(q.d) & 15u) == 0 &&
                        (P * q.es) % 16 == 0 && P * q.M * q.es < (1ll << 40) && !(g_force_generic.load() & 0x4000);
        if (!ok) return false;
        const long long images = q.batch > 1 ? q.batch : q.N / P;
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(P), static_cast<cuuint64_t>(q.M), static_cast<cuuint64_t>(images)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(P * q.es), static_cast<cuuint64_t>(P * q.M * q.es)};
        cuuint32_t box[3] = {box_cols, 32, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = st.encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, q.d, dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS;
    }
    if (q.out_nchw == 5) {
        // channels-last output D[pixel][channel] (rows = pixels of all images): boxes of 32 channels x 32
        // pixels of {channels, pixels}, 64-byte swizzled like the swapped form's
        const long long dcount = q.d_idx ? q.d_count : q.batch;
        const bool batched = dcount > 1 && q.d_batch_stride != 0;
        const bool ok = q.es == 2 && q.beta == 0.0f && (reinterpret_cast<uintptr_t>(q.d) & 15u) == 0 &&
                        (q.N * q.es) % 16 == 0 && (q.ldd * q.es) % 16 == 0 && q.ldd * q.es < (1ll << 40) &&
                        (!batched || ((q.d_batch_stride * q.es) % 16 == 0 && q.d_batch_stride * q.es < (1ll << 40))) &&
                        !(g_force_generic.load() & 0x4000);
        if (!ok) return false;
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(q.N), static_cast<cuuint64_t>(q.M),
                              static_cast<cuuint64_t>(batched ? dcount : 1)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(q.ldd * q.es),
                                 static_cast<cuuint64_t>(batched ? q.d_batch_stride * q.es : q.ldd * q.es * (q.M > 0 ? q.M : 1))};
        if (strides[1] >= (1ull << 40)) strides[1] = strides[0];
        cuuint32_t box[3] = {box_cols, 32, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = st.encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, q.d, dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS;
    }
    if (q.out_nchw) {
        // NCHW output of a convolution: {pixels of a plane, channels, images}
        const long long P = q.g.P;
        const bool ok = q.es == 2 && q.beta == 0.0f && (reinterpret_cast<uintptr_t>(q.d) & 15u) == 0 &&
                        (P * q.es) % 16 == 0 && P * q.N * q.es < (1ll << 40) && !(g_force_generic.load() & 0x4000);
        if (!ok) return false;
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(P), static_cast<cuuint64_t>(q.N),
                              static_cast<cuuint64_t>(q.M / P)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(P * q.es), static_cast<cuuint64_t>(P * q.N * q.es)};
        cuuint32_t box[3] = {32, box_cols, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = st.encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, q.d, dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS;
    }
    const bool d_ok = q.es == 2 && q.beta == 0.0f && q.betas == nullptr && q.d_offs == nullptr &&
                      (reinterpret_cast<uintptr_t>(q.d) & 15u) == 0 && (q.ldd * q.es) % 16 == 0 &&
                      // measured: a TMA store is clipped at the next 16-byte boundary after the
                      // tensor's contiguous extent, not at the extent itself, so with a padded
                      // leading dimension it would overwrite up to 7 elements of the padding
                      (q.M * q.es) % 16 == 0 &&
                      (q.batch == 1 || (q.d_batch_stride * q.es) % 16 == 0) &&
                      q.ldd * q.es < (1ll << 40) && q.d_batch_stride * q.es < (1ll << 40) &&
                      !(g_force_generic.load() & 0x4000);
    if (!d_ok) return false;
    const long long dcount = q.d_idx ? q.d_count : q.batch;
    const bool batched = dcount > 1 && q.d_batch_stride != 0;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(q.M), static_cast<cuuint64_t>(q.N),
                          static_cast<cuuint64_t>(batched ? dcount : 1)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(q.ldd * q.es),
                             static_cast<cuuint64_t>(batched ? q.d_batch_stride * q.es
                                                             : q.ldd * q.es * (q.N > 0 ? q.N : 1))};
    if (strides[1] >= (1ull << 40)) strides[1] = strides[0];
    cuuint32_t box[3] = {32, box_cols, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = st.encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, q.d, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Tile width. tcgen05.mma with M = 128 was measured (back-to-back issue, on a B200) at about
// 112-116 clocks for any N <= 128, 171 clocks for N = 256 with both operands in shared memory and
// 138 clocks for N = 256 with A in tensor memory: narrow tiles waste most of the tensor pipe.
// Pick the width that minimises (waves of tiles) x (clocks per UMMA of that width).
int choose_bn(long long M, long long N, long long batch, int num_sms, bool a_in_tmem, int max_bn) {
    const long long tiles_m = (M + kBM - 1) / kBM;
    int best = 64;
    double best_cost = 0;
    for (int w = 64; w <= max_bn; w *= 2) {
        const long long tiles = batch * tiles_m * ((N + w - 1) / w);
        const double waves = static_cast<double>((tiles + num_sms - 1) / num_sms);
        const double clk = w == 256 ? (a_in_tmem ? 138.0 : 171.0) : 114.0;
        const double cost = waves * clk;
        if (w == 64 || cost < best_cost) {
            best = w;
            best_cost = cost;
        }
        if (N <= w) break;
    }
    return best;
}

// Tile width for the kernel that keeps operand A in tensor memory. Per tile the main loop costs
// num_kb x max(tensor-core issue time, time the producer warps need for one k-block) and the
// epilogue about 30 clocks per column; the two overlap only with two accumulators in tensor
// memory, which 512 columns allow up to 192 (fp16) or 192 (fp32, two A slots) columns per tile.
// Constants are measurements on B200: issue clocks per UMMA 114 (N <= 128), 126 (192), 138 (256);
// a gathered 16-bit k-block (64 two-byte loads per thread) takes the producers about 2600 clocks.
int choose_bn_ts(const Problem& q, int num_sms, int max_bn, int a_cols, long long num_kb) {
    const long long tiles_m = (q.M + kBM - 1) / kBM;
    const bool gathered = q.es == 2 && (q.a.im2col || !q.a.k_major);
    const double mmas = q.es == 4 ? 12.0 : 4.0;  // per k-block
    int best = 64;
    double best_cost = 0;
    for (int w : {64, 128, 192, 256}) {
        if (w > max_bn) break;
        const long long tiles = q.batch * tiles_m * ((q.N + w - 1) / w);
        const double waves = static_cast<double>((tiles + num_sms - 1) / num_sms);
        const double clk = w <= 128 ? 114.0 : (w == 192 ? 126.0 : 138.0);
        double kb_clk = mmas * clk;
        if (gathered && kb_clk < 2600.0) kb_clk = 2600.0;
        const double main_clk = static_cast<double>(num_kb) * kb_clk;
        const double epi_clk = 30.0 * w;
        const bool dual = (512 - 2 * w) / a_cols >= 2;
        const double tile_clk = dual ? (main_clk > epi_clk ? main_clk : epi_clk) : main_clk + epi_clk + 600.0;
        const double cost = waves * tile_clk;
        if (w == 64 || cost < best_cost) {
            best = w;
            best_cost = cost;
        }
        if (q.N <= w) break;
    }
    return best;
}

// Wait limit of a launch, and the one host-made failure the device-side time-out path can be
// exercised with: tuning bit 0x10000000 makes a launch that consists of a single tile leave out the
// commit that hands the finished accumulator to the epilogue, with a wait limit of 2^21 clocks
// (about a millisecond) instead of 2^32. The epilogue's wait then runs out, every role drains,
// tensor memory is freed and the status word reports the time-out; nothing traps or faults, and
// the next launch runs normally.
// multiply-shift constants for a divisor (see FastDiv in contraction.cuh); {0, 0} = divide plainly
FastDiv make_fastdiv(long long d) {
    FastDiv f{0u, 0u};
    if (d <= 0 || d >= (1ll << 31)) return f;
    unsigned shift = 0;
    while ((1ull << shift) < static_cast<unsigned long long>(d)) ++shift;
    f.shift = shift;
    f.mul = static_cast<uint32_t>((((1ull << shift) - static_cast<unsigned long long>(d)) << 32) / static_cast<unsigned long long>(d)) + 1u;
    return f;
}

// (also prepares the divisions of the tile decode: tiles_m, tiles_n and g are set by now)
void set_wait_policy(Params& p, long long total_tiles) {
    p.fd_per = make_fastdiv(static_cast<long long>(p.tiles_m) * p.tiles_n);
    p.fd_group = make_fastdiv(static_cast<long long>(kGroupM) * p.tiles_n);
    p.fd_P = make_fastdiv(p.g.P);
    p.fd_OW = make_fastdiv(p.g.OW);
    const bool inject = (g_force_generic.load() & 0x10000000) != 0 && total_tiles == 1;
    p.wait_limit = inject ? (1ll << 21) : (1ll << 32);
    p.skip_tile_commit = inject ? 1 : 0;
}

// A launch below is checked with cudaGetLastError(), which also returns an error that an earlier,
// unrelated runtime call of this host thread left behind (non-sticky errors stay until read).
// Such a leftover is not this call's failure: it is read away before the first launch.
inline void clear_stale_error() { (void)cudaGetLastError(); }

int launch_ts(const DeviceState& st, const Problem& q, cudaStream_t stream) {
    clear_stale_error();
    const int a_cols = q.es == 4 ? 64 : 32;
    const int BK = 128 / q.es;
    long long tiles_m = (q.M + kBM - 1) / kBM;
    // fp32 with more than 16 k-blocks (K > 512): accumulate in chunks of 8 k-blocks and sum the
    // chunks in shared memory (the tensor core's accumulate truncates; see drain_chunk). The
    // float[BN][128] sum array (96 KB at 192 columns) and two operand stages of 48 KB limit such
    // tiles to 192 columns, which is also the widest tile that leaves room for two accumulators.
    const long long num_kb_all = (q.K + BK - 1) / BK;
    const int kc_blocks = (q.es == 4 && num_kb_all > 16 && !(g_force_generic.load() & 0x1000)) ? 8 : 0;
    int bn = choose_bn_ts(q, st.num_sms, kc_blocks ? 192 : 256, a_cols, num_kb_all);
    const int forced = g_force_bn.load() & 0xffff;
    if (forced >= 64 && forced <= (kc_blocks ? 192 : 256) && forced % 32 == 0) bn = forced;
    // an MN-major B tile is made of whole groups of BK columns (the UMMA reads all k-rows of the
    // last group it touches): a width that ends inside a group would make it read past the stage
    if (!q.b.k_major && bn % BK != 0) bn = bn / BK * BK;
    long long tiles_n = (q.N + bn - 1) / bn;
    if (q.rc_kw) {  // tile = 4 warps x rc_T output positions by rc_cpt channels (x rc_kw columns)
        bn = q.rc_cpt * q.rc_kw;
        tiles_m = (q.M + 4 * q.rc_T - 1) / (4 * q.rc_T);
        if (q.rc_tpi) tiles_m = q.M / (static_cast<long long>(q.g.OH) * q.rc_wv) * q.rc_tpi;  // images x tiles per image
        tiles_n = (q.N + q.rc_cpt - 1) / q.rc_cpt;
    }
    const long long total = q.batch * tiles_m * tiles_n;
    if (total >= INT_MAX) return kInvalidDimension;

    // two accumulator buffers (epilogue overlaps the next main loop) unless that would leave
    // fewer than two A slots in tensor memory. Two slots are enough: each producer warp holds one
    // more k-block in registers while it waits for its slot. (0x400: demand three slots.)
    const int min_slots = (g_force_generic.load() & 0x400) ? 3 : 2;
    const int acc_bufs = ((512 - 2 * bn) / a_cols >= min_slots) ? 2 : 1;
    const long long num_kb = (q.K + BK - 1) / BK;
    int ktable_bytes = 0;
    // 1x1 filters without padding address X affinely in k and need no k table
    const bool pointwise = q.a.im2col && !q.rc_kw && q.g.KH == 1 && q.g.KW == 1 && q.g.pad_t == 0 &&
                           q.g.pad_l == 0 && (q.g.OH - 1) * q.g.sh < q.g.H && (q.g.OW - 1) * q.g.sw < q.g.W &&
                           !(g_force_generic.load() & 0x2000);
    if ((q.a.im2col || q.rc_kw) && !pointwise) {
        const long long need = num_kb * BK * static_cast<long long>(sizeof(KEntry));
        if (need > 96 * 1024) return kNotImplemented;  // caller falls back to the smem-A kernel
        ktable_bytes = static_cast<int>((need + 15) & ~15ll);
    }
    const int static_smem = q.es == 2 ? st.static_smem_ts2 : st.static_smem_ts4;
    const int stage_bytes = bn * 128 * (q.es == 4 ? 2 : 1);
    const int sums_bytes = kc_blocks ? bn * 128 * 4 : 0;
    if (kc_blocks && bn > 192) return kUnexpectedError;
    // row form with image-aligned tiles: two blocks of [channels of the tile][positions of the tile]
    const int rc_tma_buf = q.rc_tpi ? (q.rc_cpt * 4 * q.rc_T * 2 + 127) / 128 * 128 : 0;
    const int out_stage_bytes = q.rc_tpi ? 2 * rc_tma_buf + 128 : 0;  // + alignment slack
    if (q.rc_tpi && (q.es != 2 || q.beta != 0.0f)) return kUnexpectedError;
    // the k table is padded to a multiple of 1024 in the layout below: count it that way here too
    // B stages in shared memory and A slots in tensor memory are separate rings in the kernel, but
    // a B ring deeper than the A ring was measured as no gain or a loss (64-channel 3x3 layer in
    // fp16 245 -> 265 us, fp32 80.3 -> 81.1 us), so both get the depth of the shallower one unless
    // measurement bit 0x200 << 16 asks for the deeper B ring
    int b_stages = (kSmemPerBlockOptin - static_smem - 1024 - ((ktable_bytes + 1023) / 1024 * 1024) - sums_bytes - out_stage_bytes) / stage_bytes;
    int stages = (512 - acc_bufs * bn) / a_cols;
    if (b_stages > kMaxStages) b_stages = kMaxStages;
    if (stages > kMaxStages) stages = kMaxStages;
    const int b_room = b_stages;  // B stages that shared memory has room for
    if (!((g_force_generic.load() >> 16) & 0x200)) b_stages = stages = std::min(b_stages, stages);
    if (stages < 2 || b_stages < 2) return kUnexpectedError;
    // One column tile, one batch entry, and the whole packed filter bank fits in the B ring: it is
    // loaded once per CTA and stays (decided here, used where the bank is packed below).
    const bool b_resident_ok = tiles_n == 1 && q.batch == 1 && num_kb <= b_room && num_kb <= kMaxStages &&
                               !((static_cast<unsigned>(g_force_generic.load()) >> 16) & 0x8000u);
    // (whether the bank will be packed: the caller's scratch must hold it)
    bool will_pack = false;
    if (q.pack_ws != nullptr && (q.a.im2col || q.rc_kw) && q.b.k_major && !(g_force_generic.load() & 0x8000)) {
        const size_t slack = static_cast<size_t>(((reinterpret_cast<uintptr_t>(q.pack_ws) + 127) & ~uintptr_t(127)) -
                                                 reinterpret_cast<uintptr_t>(q.pack_ws));
        will_pack = q.pack_ws_bytes >= slack &&
                    static_cast<long long>(q.pack_ws_bytes - slack) >= q.batch * tiles_n * num_kb * stage_bytes;
    }
    const bool b_resident = b_resident_ok && will_pack;
    if (b_resident) b_stages = static_cast<int>(num_kb);  // ring index = k-block index
    // dynamic segment: [k table][pad to 1024][B stages][partial sums]
    const int sums_off = ((ktable_bytes + 1023) / 1024 * 1024) + 1024 + b_stages * stage_bytes;
    size_t dyn_smem = static_cast<size_t>(sums_off) + sums_bytes + out_stage_bytes;
    // more than half of the SM's shared memory: never two CTAs (and two 512-column TMEM
    // allocations) on one SM
    if (dyn_smem < 120 * 1024) dyn_smem = 120 * 1024;

    TsParams tp{};
    Params& p = tp.base;
    p.M = static_cast<int>(q.M);
    p.N = static_cast<int>(q.N);
    p.K = static_cast<int>(q.K);
    p.batch = static_cast<int>(q.batch);
    p.BN = bn;
    p.stages = stages;
    p.fmt = q.fmt;
    p.tiles_m = static_cast<int>(tiles_m);
    p.tiles_n = static_cast<int>(tiles_n);
    p.total_tiles = static_cast<int>(total);
    p.alpha = q.alpha;
    p.beta = q.beta;
    p.a = q.a;
    p.b = q.b;
    p.d = q.d;
    p.ldd = q.ldd;
    p.d_batch_stride = q.d_batch_stride;
    p.a_offs = q.a_offs;
    p.b_offs = q.b_offs;
    p.d_offs = q.d_offs;
    p.alphas = q.alphas;
    p.betas = q.betas;
    p.bias = q.bias;
    p.bias_stride = q.bias_stride;
    p.resid = q.resid;
    p.relu = q.relu;
    p.g = q.g;
    p.status = st.status;
    p.ablate = g_force_generic.load() >> 16;
    set_wait_policy(p, total);
    tp.a_kind = q.rc_kw ? A_ROWCONV : (q.a.im2col ? A_IM2COL : (q.a.k_major ? A_DENSE_K : A_DENSE_MN));
    tp.a_pointwise = pointwise ? 1 : 0;
    tp.rc_kw = q.rc_kw;
    tp.rc_cpt = q.rc_cpt;
    tp.rc_T = q.rc_T;
    tp.rc_lo = q.rc_lo;
    tp.rc_sw = q.rc_sw;
    tp.rc_wv = q.rc_wv;
    tp.rc_dmin = q.rc_dmin;
    tp.kc_blocks = kc_blocks;
    tp.sums_off = sums_off;
    tp.stage_off = sums_off + sums_bytes;
    tp.rc_tpi = q.rc_tpi;
    tp.rc_tma = q.rc_tpi ? 1 : 0;
    tp.rc_tma_buf = rc_tma_buf;
    tp.b_stages = b_stages;
    // row form with stride_w = 2 on 16-bit data: the two column phases of a tap are adjacent in
    // memory; one aligned 32-bit load serves both when the rows and the tensor start on 4 bytes
    tp.rc_pair = (q.rc_kw && q.rc_sw == 2 && q.es == 2 && q.g.W % 2 == 0 && 2 * q.rc_wv <= q.g.W &&
                  (reinterpret_cast<uintptr_t>(q.a.base) & 3u) == 0 && !((g_force_generic.load() >> 16) & 64))
                     ? 1 : 0;
    tp.acc_bufs = acc_bufs;
    tp.ktable_bytes = ktable_bytes;

    tp.b_packed = nullptr;
    tp.b_tma = 0;
    if (q.pack_ws != nullptr && (q.a.im2col || q.rc_kw) && p.b.k_major && !(g_force_generic.load() & 0x8000)) {
        // lay the filter bank out as stage images first (same stream), then stream them with bulk copies
        unsigned char* ws = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(q.pack_ws) + 127) & ~uintptr_t(127));
        const size_t slack = static_cast<size_t>(ws - q.pack_ws);
        const long long need = q.batch * tiles_n * num_kb * stage_bytes;
        if (q.pack_ws_bytes >= slack && static_cast<long long>(q.pack_ws_bytes - slack) >= need) {
            const long long chunks = q.batch * tiles_n * num_kb * bn * 8;
            const unsigned pgrid = static_cast<unsigned>(chunks / 256 + 1 < 148 * 16 ? chunks / 256 + 1 : 148 * 16);
            if (q.es == 2)
                pack_weights_kernel<2><<<pgrid, 256, 0, stream>>>(tp, ws, chunks);
            else
                pack_weights_kernel<4><<<pgrid, 256, 0, stream>>>(tp, ws, chunks);
            g_launches.fetch_add(1);
            tp.b_packed = ws;
            tp.b_resident = b_resident ? 1 : 0;
        }
    }

    CUtensorMap tm_b;
    std::memset(&tm_b, 0, sizeof(tm_b));
    if (q.es == 4 && !q.a.im2col && !q.rc_kw && q.b_offs == nullptr && !(g_force_generic.load() & 0x800) &&
        tma_ok(q.b, q.es, q.N, q.K, q.batch)) {
        if (encode_map(st, &tm_b, q.b, q.es, q.N, q.K, q.batch, bn) == kSuccess) tp.b_tma = 1;
    }

    CUtensorMap tm_d;
    std::memset(&tm_d, 0, sizeof(tm_d));
    if (q.rc_tpi) {
        // Y as {pixels of a plane, all channels, images}; a box is one tile's positions x 16 channels
        const long long ctot = q.batch * q.N;
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(q.g.P), static_cast<cuuint64_t>(ctot),
                              static_cast<cuuint64_t>(q.M / (static_cast<long long>(q.g.OH) * q.rc_wv))};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(q.g.P) * 2u, static_cast<cuuint64_t>(q.g.out_img_stride) * 2u};
        cuuint32_t box[3] = {static_cast<cuuint32_t>(4 * q.rc_T), 16u, 1u};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = st.encode(&tm_d, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, q.d, dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return kUnexpectedError;
    }

    const unsigned grid = static_cast<unsigned>(total < st.num_sms ? total : st.num_sms);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kTsThreads, 1, 1);
    cfg.dynamicSmemBytes = dyn_smem;
    cfg.stream = stream;
    // after a packing launch: programmatic dependent launch, so that this kernel's prologue and
    // activation gather overlap the packing grid (only its filter loader waits for that grid)
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = (tp.b_packed != nullptr && !(g_force_generic.load() & 0x40000000)) ? 1 : 0;
    if (std::getenv("DLF_B200_DEBUG"))
        std::fprintf(stderr, "dlf_b200: ts launch es=%d bn=%d a_slots=%d acc_bufs=%d grid=%u dyn_smem=%zu ktable=%d sums=%d packed=%d pending=%s\n",
                     q.es, bn, stages, acc_bufs, grid, dyn_smem, ktable_bytes, sums_bytes, tp.b_packed != nullptr,
                     cudaGetErrorString(cudaPeekAtLastError()));
    if (q.es == 2)
        CUDA_TRY(launch_ts_kernel<2>(&cfg, tp, tm_b, tm_d));
    else
        CUDA_TRY(launch_ts_kernel<4>(&cfg, tp, tm_b, tm_d));
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}

int launch(const Problem& q_in, cudaStream_t stream, DeviceState* preset = nullptr) {
    DeviceState* st = preset;
    int rc = kSuccess;
    if (st == nullptr) {
        rc = ensure_device(&st);
        if (rc != kSuccess) return rc;
    }
    clear_stale_error();
    if (q_in.M > INT_MAX - 512 || q_in.N > INT_MAX - 512 || q_in.K > INT_MAX - 512 || q_in.batch > INT_MAX)
        return kInvalidDimension;

    // A plain 16-bit product whose result can leave through TMA stores is computed transposed: with
    // the operands exchanged the lanes hold the columns j of D and the accumulator columns run along
    // i, the contiguous index of D, so a lane's 32 columns are 64 consecutive bytes - four 16-byte
    // shared-memory stores into the [row][column] staging block of the channels-last convolution
    // (out_nchw == 5) instead of 32 two-byte ones, and no shuffles. The product itself is the same
    // (D^T = Bu * Au^T; both operands are K-major or MN-major either way). Only for products whose
    // epilogue sets the pace - a short K - and whose N fills the 128 lanes. Measured: the batched
    // product 1024 x (512 x 512 x 64) 187 -> 125 us (a library bmm: 105 us); 1024 x (512 x 64 x 512)
    // would lose (106 -> 111 us, half of the lanes idle) and so would 4096^3 (118 -> 137 us: twice the
    // TMA stores beside a main loop that needs the copy unit itself). Bit 30 of the tile-width word: never.
    Problem q = q_in;
    if (q.es == 2 && q.out_nchw == 0 && q.a_cl == 0 && !q.a.im2col && q.beta == 0.0f && q.betas == nullptr &&
        q.alphas == nullptr && q.a_offs == nullptr && q.b_offs == nullptr && q.d_offs == nullptr && q.bias == nullptr &&
        q.resid == nullptr && !q.d_f32 && !(g_force_generic.load() & (0xff | 0x4000 | 0x200)) && q.K <= 256 && q.N >= 128 &&
        (reinterpret_cast<uintptr_t>(q.d) & 15u) == 0 && (q.ldd * q.es) % 16 == 0 && (q.M * q.es) % 16 == 0 &&
        (q.batch == 1 || q.d_batch_stride == 0 || (q.d_batch_stride * q.es) % 16 == 0) &&
        tma_ok(q.a, q.es, q.M, q.K, q.batch) && tma_ok(q.b, q.es, q.N, q.K, q.batch) &&
        !((g_force_bn.load() >> 16) & 16384)) {
        std::swap(q.a, q.b);
        std::swap(q.M, q.N);
        std::swap(q.a_idx, q.b_idx);
        std::swap(q.a_count, q.b_count);
        q.out_nchw = 5;
        q.narrow_boxes = true;  // measured on the batched product above: 125-128 us with 2 KB boxes, 136 us with 4 KB ones
    }

    const bool use_tma = q.es == 2 && !(g_force_generic.load() & 0xff) && q.a_offs == nullptr &&
                         ((q.a_cl != 0 && !q.cl_swap) || tma_ok(q.a, q.es, q.M, q.K, q.batch)) &&
                         ((q.a_cl != 0 && q.cl_swap) || tma_ok(q.b, q.es, q.N, q.K, q.batch));
    if (q.a_cl != 0 && !use_tma) return kNotImplemented;
    // A through tensor memory: every convolution and every fp32 product (see contraction_ts.cuh)
    const int force_path = g_force_generic.load() & 0xff;
    if (force_path != 2 && !q.no_ts && !use_tma && (q.a.im2col || q.es == 4 || force_path == 3)) {
        rc = launch_ts(*st, q, stream);
        if (rc != kNotImplemented) return rc;  // else: im2col table too large, use the smem-A kernel
    }

    const long long tiles_m = (q.M + kBM - 1) / kBM;
    // fp32 here keeps hi and lo copies of both operands per stage: 128 columns leave >= 3 stages
    int bn = choose_bn(q.M, q.N, q.batch, st->num_sms, false, q.es == 4 ? 128 : 256);
    const int forced = g_force_bn.load() & 0xffff;
    if (forced == 64 || forced == 128 || (forced == 256 && q.es == 2)) bn = forced;

    // CTA pairs (cta_group::2): 256 x 256 tiles, each CTA stages 128 rows of A and 128 of B, so
    // a third less shared-memory fill per flop than a lone 128 x 256 tile.
    if (use_tma && bn == 256 && q.M > kBM && st->max_pair_clusters > 0 && (g_force_generic.load() & 0x200) &&
        q.a_cl == 0 && q.out_nchw == 0 && q.a_idx == nullptr && q.b_idx == nullptr && q.d_idx == nullptr) {
        const long long ptiles_m = (q.M + 2 * kBM - 1) / (2 * kBM);
        const long long ptiles_n = (q.N + bn - 1) / bn;
        const long long ptotal = q.batch * ptiles_m * ptiles_n;
        if (ptotal >= INT_MAX) return kInvalidDimension;
        const int pstage = (kBM + bn / 2) * 128;
        int pstages = (kSmemPerBlockOptin - st->static_smem_pair - 1024) / pstage;
        if (pstages > kMaxStages) pstages = kMaxStages;
        Params p{};
        p.M = static_cast<int>(q.M);
        p.N = static_cast<int>(q.N);
        p.K = static_cast<int>(q.K);
        p.batch = static_cast<int>(q.batch);
        p.BN = bn;
        p.stages = pstages;
        p.fmt = q.fmt;
        p.tiles_m = static_cast<int>(ptiles_m);
        p.tiles_n = static_cast<int>(ptiles_n);
        p.total_tiles = static_cast<int>(ptotal);
        p.alpha = q.alpha;
        p.beta = q.beta;
        p.a = q.a;
        p.b = q.b;
        p.d = q.d;
        p.ldd = q.ldd;
        p.d_batch_stride = q.d_batch_stride;
        p.bias = q.bias;
        p.bias_stride = q.bias_stride;
        p.resid = q.resid;
        p.relu = q.relu;
        p.g = q.g;
        p.status = st->status;
        set_wait_policy(p, ptotal);
        CUtensorMap tm_a, tm_b, tm_d;
        std::memset(&tm_d, 0, sizeof(tm_d));
        rc = encode_map(*st, &tm_a, q.a, q.es, q.M, q.K, q.batch, kBM);
        if (rc != kSuccess) return rc;
        rc = encode_map(*st, &tm_b, q.b, q.es, q.N, q.K, q.batch, bn / 2);
        if (rc != kSuccess) return rc;
        p.d_tma = encode_output_map(*st, &tm_d, q, 64) ? 64 : 0;
        const long long clusters = ptotal < st->max_pair_clusters ? ptotal : st->max_pair_clusters;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters), 1, 1);
        cfg.blockDim = dim3(kThreadsPair, 1, 1);
        cfg.dynamicSmemBytes = static_cast<size_t>(pstages) * pstage + 1024;
        cfg.stream = stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        CUDA_TRY(cudaLaunchKernelEx(&cfg, contraction_kernel<2, true, true>, p, tm_a, tm_b, tm_d, tm_d));
        g_launches.fetch_add(1);
        CUDA_TRY(cudaGetLastError());
        return kSuccess;
    }
    const long long tiles_n = (q.N + bn - 1) / bn;
    const long long total = q.batch * tiles_m * tiles_n;
    if (total >= INT_MAX) return kInvalidDimension;

    // Epilogue warps of the TMA variant: four sets for convolutions whose main loop is short against
    // the epilogue (K <= 512 and K <= twice the output channels, tiles of 128 columns or more), where the
    // epilogue is the longest stage (64 -> 256 1x1 at 56x56, batch 256: 149 -> 127 us; 128 -> 512 at
    // 28x28: 87 -> 77 us; 512 -> 2048 at 7x7: 79 -> 62 us); two sets otherwise - a long main loop
    // wants the registers and the fourth 48 KB stage (512 -> 128 at 28x28: 49 vs 54 us), and so does
    // the paired-store epilogue of even planes that cannot have TMA stores (256 -> 1024 at 14x14).
    // Plain GEMM calls keep two sets (1024 x 512x64x512, bound by its reads: 105 vs 111 us).
    const long long num_kb_l = (q.K + 63) / 64;
    const bool paired_plain = q.out_nchw == 1 && q.g.P % 2 == 0 && q.g.P % 8 != 0;
    const long long out_ch = q.cl_swap ? q.M : q.N;
    const bool four_sets = use_tma && (q.out_nchw != 0 || q.bias_rows) && num_kb_l <= 8 && q.K <= 2 * out_ch && bn >= 128 && !paired_plain &&
                           !((g_force_bn.load() >> 16) & 32);
    // Three sets (448 threads, 128 registers, no spills) for the widening pixel-per-lane layers the
    // four-set form leaves out (256 -> 1024 at 14x14: 77 -> 73 us; 1024 -> 2048 stride 2: 110 -> 98 us;
    // 3x3 layers lose 4-6 % with it). Bit 22 of the tile-width word: never.
    const bool three_sets = use_tma && !four_sets && (q.out_nchw == 1 || q.out_nchw == 5) && bn >= 128 && q.N >= 2 * q.K &&
                            !((g_force_bn.load() >> 16) & 64);
    const int esets = four_sets ? 4 : (three_sets ? 3 : 2);
    const int static_smem = use_tma ? (four_sets ? st->static_smem_tma4 : three_sets ? st->static_smem_tma3 : st->static_smem_tma)
                                    : (q.es == 2 ? st->static_smem_gen2 : st->static_smem_gen4);
    const int stage_bytes = (kBM + bn) * 128 * (q.es == 4 ? 2 : 1);
    const int epi_stage = use_tma ? epi_stage_bytes(esets) : 0;  // output staging blocks of the epilogue warps
    int stages = (kSmemPerBlockOptin - static_smem - 1024 - epi_stage) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return kUnexpectedError;
    const size_t dyn_smem = static_cast<size_t>(stages) * stage_bytes + 1024 + epi_stage;

    Params p{};
    p.M = static_cast<int>(q.M);
    p.N = static_cast<int>(q.N);
    p.K = static_cast<int>(q.K);
    p.batch = static_cast<int>(q.batch);
    p.BN = bn;
    p.stages = stages;
    p.fmt = q.fmt;
    p.tiles_m = static_cast<int>(tiles_m);
    p.tiles_n = static_cast<int>(tiles_n);
    p.total_tiles = static_cast<int>(total);
    p.alpha = q.alpha;
    p.beta = q.beta;
    p.a = q.a;
    p.b = q.b;
    p.d = q.d;
    p.ldd = q.ldd;
    p.d_batch_stride = q.d_batch_stride;
    p.a_offs = q.a_offs;
    p.b_offs = q.b_offs;
    p.d_offs = q.d_offs;
    p.alphas = q.alphas;
    p.betas = q.betas;
    p.bias = q.bias;
    p.bias_stride = q.bias_stride;
    p.bias_rows = q.bias_rows;
    p.a_idx = q.a_idx;
    p.b_idx = q.b_idx;
    p.d_idx = q.d_idx;
    p.resid = q.resid;
    p.relu = q.relu;
    p.g = q.g;
    p.status = st->status;
    p.d_f32 = q.d_f32 ? 1 : 0;
    p.a_cl = q.a_cl;
    p.cl_cblocks = q.cl_cblocks;
    p.out_nchw = q.out_nchw;
    p.cl_swap = q.cl_swap;
    p.out_vec = q.out_vec;
    set_wait_policy(p, total);

    CUtensorMap tm_a, tm_b, tm_d, tm_r;
    std::memset(&tm_a, 0, sizeof(tm_a));
    std::memset(&tm_b, 0, sizeof(tm_b));
    std::memset(&tm_d, 0, sizeof(tm_d));
    std::memset(&tm_r, 0, sizeof(tm_r));
    p.d_tma = 0;
    p.r_tma = 0;
    if (use_tma) {
        if (q.cl_swap) {
            rc = encode_map(*st, &tm_a, q.a, q.es, q.M, q.K, q.a_idx ? q.a_count : q.batch, kBM);
            if (rc != kSuccess) return rc;
            rc = q.a_cl == 1 ? encode_im2col_map(*st, &tm_b, q, q.b.base, bn)
                             : encode_map(*st, &tm_b, q.b, q.es, q.N, q.K, q.b_idx ? q.b_count : q.batch, bn);
        } else {
            rc = q.a_cl == 1 ? encode_im2col_map(*st, &tm_a, q, q.a.base, kBM)
                             : encode_map(*st, &tm_a, q.a, q.es, q.M, q.K, q.a_idx ? q.a_count : q.batch, kBM);
            if (rc != kSuccess) return rc;
            rc = encode_map(*st, &tm_b, q.b, q.es, q.N, q.K, q.b_idx ? q.b_count : q.batch, bn);
        }
        if (rc != kSuccess) return rc;
        // 64-column boxes need 64 columns per epilogue warp
        // (a residual is fetched box by box into single staging blocks: 32-column boxes then)
        // (the forms that prefetch a residual box a block ahead need the two single staging blocks:
        // 32-column boxes; the row-staged forms fetch it into the wide box itself. Measured at batch
        // 256, NCHW swapped form: 64 -> 256 at 56x56 120 -> 92 us, with a residual 220 -> 185 us;
        // 128 -> 512 at 28x28 with a residual 135 -> 105 us. Channels-last form: 105 -> 97 us and
        // 199 -> 180 us on the first layer, 108 -> 99 us on the second.)
        const bool boxes_are_rows = q.out_nchw == 3 || q.out_nchw == 5;
        const unsigned box_cols = (esets == 2 ? bn >= 128 : (esets == 4 && bn >= 256)) && !(g_force_generic.load() & 0x100) &&
                                          (q.resid == nullptr || boxes_are_rows) && !q.narrow_boxes &&
                                          !(boxes_are_rows && ((g_force_bn.load() >> 16) & 2048)) ? 64 : 32;
        p.d_tma = (!q.d_f32 && encode_output_map(*st, &tm_d, q, box_cols)) ? static_cast<int>(box_cols) : 0;
        if ((q.out_nchw == 5 || q.bias_rows) && !p.d_tma) return kNotImplemented;  // the channels-last forms only leave through TMA stores
        // the residual tensor is laid out like D: the same boxes of it, fetched by TMA loads
        if (p.d_tma && q.resid != nullptr && (reinterpret_cast<uintptr_t>(q.resid) & 15u) == 0 && !((g_force_bn.load() >> 16) & 512)) {
            Problem qr = q;
            qr.d = const_cast<char*>(q.resid);
            p.r_tma = encode_output_map(*st, &tm_r, qr, box_cols) ? 1 : 0;
        }
        if ((q.out_nchw == 5 || q.bias_rows) && q.resid != nullptr && !p.r_tma) return kNotImplemented;
    }

    const unsigned grid = static_cast<unsigned>(total < st->num_sms ? total : st->num_sms);
    if (use_tma) {
#define DLF_TMA_LAUNCH(ESETS)                                                                                      \
        if (p.r_tma)                                                                                               \
            contraction_kernel<2, true, false, ESETS, true><<<grid, tma_threads(ESETS), dyn_smem, stream>>>(p, tm_a, tm_b, tm_d, tm_r); \
        else                                                                                                       \
            contraction_kernel<2, true, false, ESETS, false><<<grid, tma_threads(ESETS), dyn_smem, stream>>>(p, tm_a, tm_b, tm_d, tm_r)
        if (four_sets) {
            DLF_TMA_LAUNCH(4);
        } else if (three_sets) {
            DLF_TMA_LAUNCH(3);
        } else {
            DLF_TMA_LAUNCH(2);
        }
#undef DLF_TMA_LAUNCH
    } else if (q.es == 2) {
        contraction_kernel<2, false><<<grid, kThreadsGen, dyn_smem, stream>>>(p, tm_a, tm_b, tm_d, tm_r);
    } else {
        contraction_kernel<4, false><<<grid, kThreadsGen, dyn_smem, stream>>>(p, tm_a, tm_b, tm_d, tm_r);
    }
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}

// ---------------------------------------------------------------------------------------------
// Scratch that lives in the library image instead of in allocated memory.
//
// dlf_b200_gemm_batched needs its per-batch tables (three offset tables, alpha, beta) in device
// memory and takes that scratch from the caller. Some callers have no scratch to give and may not
// create any: a dlf routine that runs while the context's temporary-buffer pool is in use by an
// enclosing routine (the pool is a LIFO slab that throws on out-of-order release and is not
// thread-safe), or a serving process whose device memory was handed in full to another owner at
// start-up. For them the tables - and the status word the kernels report to - sit in these
// file-scope device arrays, which every GPU that loads the library holds until the process exits.
// The names below are host-side stand-ins, not device addresses: the device address is looked up
// once per device with cudaGetSymbolAddress (noalloc_device) and that pointer goes to the kernel.
constexpr size_t kNoAllocMaxBatch = 4096;
constexpr size_t kNoAllocTableBytes = kNoAllocMaxBatch * (3 * sizeof(long long) + 2 * sizeof(float));
static __device__ __align__(256) unsigned char g_noalloc_tables[kNoAllocTableBytes];
static __device__ __align__(256) int g_noalloc_status[2];

struct NoAllocDevice {
    bool ready = false;
    DeviceState st;          // same per-device facts as the allocating path, status -> static word
    unsigned char* tables = nullptr;
};
NoAllocDevice g_noalloc_dev[kMaxDevices];

// Per-device set-up of the no-allocation path, with that device current: kernel attributes, the
// tensor-map encoder and the device addresses of the two static arrays. Allocates nothing.
int noalloc_device(NoAllocDevice** out) {
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return kInvalidValue;
    std::lock_guard<std::mutex> lock(g_mu);
    NoAllocDevice& nd = g_noalloc_dev[dev];
    if (!nd.ready) {
        DeviceState& st = nd.st;
        CUDA_TRY(cudaDeviceGetAttribute(&st.num_sms, cudaDevAttrMultiProcessorCount, dev));
        int major = 0;
        CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return kNotImplemented;
        cudaFuncAttributes fa;
        CUDA_TRY(cudaFuncGetAttributes(&fa, contraction_kernel<2, true>));
        st.static_smem_tma = static_cast<int>(fa.sharedSizeBytes);
        CUDA_TRY(cudaFuncGetAttributes(&fa, contraction_kernel<2, false>));
        st.static_smem_gen2 = static_cast<int>(fa.sharedSizeBytes);
        CUDA_TRY(cudaFuncGetAttributes(&fa, contraction_kernel<4, false>));
        st.static_smem_gen4 = static_cast<int>(fa.sharedSizeBytes);
        {
            int rc2 = setup_ts_kernels<2>(&st.static_smem_ts2);
            if (rc2 != kSuccess) return rc2;
            rc2 = setup_ts_kernels<4>(&st.static_smem_ts4);
            if (rc2 != kSuccess) return rc2;
        }
        CUDA_TRY(cudaFuncSetAttribute(contraction_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemPerBlockOptin - st.static_smem_tma));
        CUDA_TRY(cudaFuncSetAttribute(contraction_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemPerBlockOptin - st.static_smem_gen2));
        CUDA_TRY(cudaFuncSetAttribute(contraction_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemPerBlockOptin - st.static_smem_gen4));
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return kUnexpectedError;
        st.encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
        void* p_tables = nullptr;
        void* p_status = nullptr;
        CUDA_TRY(cudaGetSymbolAddress(&p_tables, g_noalloc_tables));
        CUDA_TRY(cudaGetSymbolAddress(&p_status, g_noalloc_status));
        nd.tables = static_cast<unsigned char*>(p_tables);
        st.status = static_cast<int*>(p_status);
        st.ready = true;
        nd.ready = true;
    }
    *out = &nd;
    return kSuccess;
}

// Argument rules of Xgemm<T>::ProcessArguments (gpgpu/src/routines/level3/xgemm.hpp:54-91)
// and TestMatrixA/B/C (gpgpu/src/utilities/buffer_test.hpp:24-55), then the mapping of the
// user's (layout, transposes) onto the canonical problem whose output index i is contiguous.
int setup_gemm(Problem& q, int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k,
               const void* a, size_t a_ld, const void* b, size_t b_ld, void* c, size_t c_ld) {
    if (!dtype_info(dtype, q.fmt, q.es)) return kNotImplemented;
    if (layout != DLF_B200_ROW_MAJOR && layout != DLF_B200_COL_MAJOR) return kInvalidValue;
    if (ta < DLF_B200_NO_TRANS || ta > DLF_B200_CONJ_TRANS) return kInvalidValue;
    if (tb < DLF_B200_NO_TRANS || tb > DLF_B200_CONJ_TRANS) return kInvalidValue;
    if (m == 0 || n == 0 || k == 0) return kInvalidDimension;
    const bool row = layout == DLF_B200_ROW_MAJOR;
    const bool a_rot = (!row && ta != DLF_B200_NO_TRANS) || (row && ta == DLF_B200_NO_TRANS);
    const bool b_rot = (!row && tb != DLF_B200_NO_TRANS) || (row && tb == DLF_B200_NO_TRANS);
    const size_t a_one = a_rot ? k : m;
    const size_t b_one = b_rot ? n : k;
    const size_t c_one = row ? n : m;
    if (a_ld < a_one) return kInvalidLeadDimA;
    if (b_ld < b_one) return kInvalidLeadDimB;
    if (c_ld < c_one) return kInvalidLeadDimC;
    if (a == nullptr) return kInvalidMatrixA;
    if (b == nullptr) return kInvalidMatrixB;
    if (c == nullptr) return kInvalidMatrixC;

    GenOperand ua{}, ub{};
    ua.base = static_cast<const char*>(a);
    ua.ld = static_cast<long long>(a_ld);
    ua.k_major = a_rot ? 1 : 0;  // a_rot: k is the contiguous index of A
    ub.base = static_cast<const char*>(b);
    ub.ld = static_cast<long long>(b_ld);
    ub.k_major = b_rot ? 0 : 1;  // b_rot: n is the contiguous index of B
    q.K = static_cast<long long>(k);
    if (!row) {  // C(m x n) column-major: i = row of C
        q.M = static_cast<long long>(m);
        q.N = static_cast<long long>(n);
        q.a = ua;
        q.b = ub;
    } else {  // C row-major: i = column of C, so B supplies the "A" side
        q.M = static_cast<long long>(n);
        q.N = static_cast<long long>(m);
        q.a = ub;
        q.b = ua;
    }
    q.d = static_cast<char*>(c);
    q.ldd = static_cast<long long>(c_ld);
    return kSuccess;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// K-split GEMM. A product with few output tiles and a long K leaves most SMs idle (the fully
// connected layer 256 x 1000 x 2048: 16 tiles on 148 SMs). With scratch from the caller the K range
// is cut into slices that run as the batch entries of one launch, each writing an fp32 partial
// product, and a second kernel adds the slices and applies alpha / beta.
// ---------------------------------------------------------------------------------------------
size_t splitk_slices(const Problem& q, int num_sms) {
    if (q.batch != 1 || q.a_offs != nullptr || q.a.im2col) return 1;
    const long long BK = 128 / q.es;
    const long long tiles = ((q.M + kBM - 1) / kBM) * ((q.N + 127) / 128);
    if (tiles * 2 > num_sms || q.K < 8 * BK) return 1;
    // the fewest slices that fill about three quarters of the SMs, each at least four k-blocks long
    size_t best = 1;
    for (size_t s : {2, 4, 8}) {
        if (q.K % (static_cast<long long>(s) * BK) != 0 || q.K / static_cast<long long>(s) < 4 * BK) break;
        best = s;
        if (tiles * static_cast<long long>(s) * 4 >= 3ll * num_sms) break;
    }
    return best;
}

int launch_splitk(const Problem& q, size_t slices, void* workspace, cudaStream_t stream, DeviceState* st) {
    Problem r = q;
    const long long ks = q.K / static_cast<long long>(slices);
    r.K = ks;
    r.batch = static_cast<long long>(slices);
    r.a.batch_stride = q.a.k_major ? ks : ks * q.a.ld;
    r.b.batch_stride = q.b.k_major ? ks : ks * q.b.ld;
    r.d = static_cast<char*>(workspace);
    r.ldd = q.M;
    r.d_batch_stride = q.M * q.N;
    r.alpha = 1.0f;
    r.beta = 0.0f;
    r.bias = nullptr;
    r.d_f32 = q.es == 2;
    int rc = launch(r, stream, st);
    if (rc != kSuccess) return rc;
    const long long total = q.M * q.N;
    const unsigned grid = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 148 * 8));
    const float* part = static_cast<const float*>(workspace);
    if (q.fmt == FMT_F32)
        splitk_reduce_kernel<float><<<grid, 256, 0, stream>>>(reinterpret_cast<float*>(q.d), q.ldd, part, static_cast<int>(q.M), static_cast<int>(q.N), static_cast<int>(slices), q.alpha, q.beta);
    else if (q.fmt == FMT_F16)
        splitk_reduce_kernel<__half><<<grid, 256, 0, stream>>>(reinterpret_cast<__half*>(q.d), q.ldd, part, static_cast<int>(q.M), static_cast<int>(q.N), static_cast<int>(slices), q.alpha, q.beta);
    else
        splitk_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(q.d), q.ldd, part, static_cast<int>(q.M), static_cast<int>(q.N), static_cast<int>(slices), q.alpha, q.beta);
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}

// ---------------------------------------------------------------------------------------------
// helpers of the level-3 routines (symm, syrk, trmm, trsm) further down
// ---------------------------------------------------------------------------------------------
namespace {

enum : int { kUpper = 121, kLower = 122, kNonUnit = 131, kUnit = 132, kLeft = 141, kRight = 142 };

void float_to_scalar(int fmt, float v, void* out) {
    if (fmt == FMT_F16) {
        const __half h = __float2half_rn(v);
        std::memcpy(out, &h, 2);
    } else if (fmt == FMT_BF16) {
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        std::memcpy(out, &h, 2);
    } else {
        std::memcpy(out, &v, 4);
    }
}

int dtype_of(int fmt) { return fmt == FMT_F16 ? DLF_B200_HALF : (fmt == FMT_BF16 ? DLF_B200_BFLOAT16 : DLF_B200_SINGLE); }

// row-major GEMM on device pointers with float scalars, through the public entry point
int rm_gemm(int fmt, int ta, int tb, size_t m, size_t n, size_t k, float alpha, const void* a, size_t lda,
            const void* b, size_t ldb, float beta, void* c, size_t ldc, void* stream) {
    unsigned char al[4], be[4];
    float_to_scalar(fmt, alpha, al);
    float_to_scalar(fmt, beta, be);
    return dlf_b200_gemm(dtype_of(fmt), DLF_B200_ROW_MAJOR, ta, tb, m, n, k, al, a, lda, b, ldb, be, c, ldc, stream);
}

unsigned l3_grid(long long total) {
    const long long blocks = (total + 255) / 256;
    return static_cast<unsigned>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

char* align256(void* p) { return reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(p) + 255) & ~uintptr_t(255)); }

template <typename T>
int l3_expand(T* dst, const void* src, size_t ld, size_t n, bool symmetric, bool upper, bool unit, cudaStream_t s) {
    l3_expand_square_kernel<T><<<l3_grid(static_cast<long long>(n) * n), 256, 0, s>>>(
        dst, static_cast<const T*>(src), static_cast<long long>(ld), static_cast<int>(n), symmetric ? 1 : 0,
        upper ? 1 : 0, unit ? 1 : 0);
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}

int l3_expand_any(int fmt, void* dst, const void* src, size_t ld, size_t n, bool symmetric, bool upper, bool unit,
                  cudaStream_t s) {
    if (fmt == FMT_F32) return l3_expand(static_cast<float*>(dst), src, ld, n, symmetric, upper, unit, s);
    if (fmt == FMT_F16) return l3_expand(static_cast<__half*>(dst), src, ld, n, symmetric, upper, unit, s);
    return l3_expand(static_cast<__nv_bfloat16*>(dst), src, ld, n, symmetric, upper, unit, s);
}

}  // namespace

namespace {

// common argument rules of trmm / trsm; on success the call is in row-major form
int tri_args(int dtype, int& fmt, int& es, int layout, int& side, int& triangle, int a_transpose, int diagonal,
             size_t& m, size_t& n, const void* alpha, const void* a, size_t a_ld, const void* b, size_t b_ld) {
    if (!dtype_info(dtype, fmt, es)) return kNotImplemented;
    if (layout != DLF_B200_ROW_MAJOR && layout != DLF_B200_COL_MAJOR) return kInvalidValue;
    if ((side != kLeft && side != kRight) || (triangle != kUpper && triangle != kLower)) return kInvalidValue;
    if (a_transpose < DLF_B200_NO_TRANS || a_transpose > DLF_B200_CONJ_TRANS) return kInvalidValue;
    if (diagonal != kNonUnit && diagonal != kUnit) return kInvalidValue;
    if (m == 0 || n == 0) return kInvalidDimension;
    const bool row = layout == DLF_B200_ROW_MAJOR;
    if (a_ld < (side == kLeft ? m : n)) return kInvalidLeadDimA;
    if (b_ld < (row ? n : m)) return kInvalidLeadDimB;
    if (a == nullptr) return kInvalidMatrixA;
    if (b == nullptr) return kInvalidMatrixB;
    if (alpha == nullptr) return kInvalidValue;
    // column-major: B^T (n x m, row-major) = B^T op(T)^T: the other side, and the stored
    // triangle of the row-major view of A is the other one; op stays as given
    if (!row) {
        side = side == kLeft ? kRight : kLeft;
        triangle = triangle == kUpper ? kLower : kUpper;
        const size_t t = m;
        m = n;
        n = t;
    }
    return kSuccess;
}

}  // namespace

extern "C" {

int dlf_b200_gemm(int dtype, int layout, int trans_a, int trans_b, size_t m, size_t n, size_t k,
                  const void* alpha, const void* a, size_t a_ld, const void* b, size_t b_ld,
                  const void* beta, void* c, size_t c_ld, void* stream) {
    Problem q;
    int rc = setup_gemm(q, dtype, layout, trans_a, trans_b, m, n, k, a, a_ld, b, b_ld, c, c_ld);
    if (rc != kSuccess) return rc;
    if (alpha == nullptr || beta == nullptr) return kInvalidValue;
    q.alpha = scalar_to_float(q.fmt, alpha);
    q.beta = scalar_to_float(q.fmt, beta);
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;
    return launch(q, static_cast<cudaStream_t>(stream));
}

size_t dlf_b200_gemm_workspace_bytes(int dtype, size_t m, size_t n, size_t k) {
    // optional scratch of dlf_b200_gemm_ex: up to 8 fp32 partial products of m x n elements, only
    // for products small enough to profit from a K-split (an upper bound; 0 = never used)
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es) || m == 0 || n == 0 || k == 0) return 0;
    const size_t tiles = ((m + 127) / 128) * ((n + 127) / 128);
    if (tiles > 148 || k < 8 * static_cast<size_t>(128 / es)) return 0;
    return 8 * m * n * sizeof(float) + 256;
}

int dlf_b200_gemm_ex(int dtype, int layout, int trans_a, int trans_b, size_t m, size_t n, size_t k,
                     const void* alpha, const void* a, size_t a_ld, const void* b, size_t b_ld,
                     const void* beta, void* c, size_t c_ld, void* workspace, size_t workspace_bytes,
                     void* stream) {
    Problem q;
    int rc = setup_gemm(q, dtype, layout, trans_a, trans_b, m, n, k, a, a_ld, b, b_ld, c, c_ld);
    if (rc != kSuccess) return rc;
    if (alpha == nullptr || beta == nullptr) return kInvalidValue;
    q.alpha = scalar_to_float(q.fmt, alpha);
    q.beta = scalar_to_float(q.fmt, beta);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamDevice sd(s);
    if (sd.rc != kSuccess) return sd.rc;
    DeviceState* st = nullptr;
    rc = ensure_device(&st);
    if (rc != kSuccess) return rc;
    if (workspace != nullptr && !(g_force_generic.load() & 0x20000000)) {
        char* ws = align256(workspace);
        const size_t slack = static_cast<size_t>(ws - static_cast<char*>(workspace));
        size_t slices = splitk_slices(q, st->num_sms);
        // the partial products are plain dense products: they need the TMA-fed kernel (16-bit) or
        // the tensor-memory-operand kernel (fp32); other operand layouts run unsplit
        const bool fast = q.es == 4 || (!(g_force_generic.load() & 0xff) && tma_ok(q.a, q.es, q.M, q.K, 1) &&
                                        tma_ok(q.b, q.es, q.N, q.K, 1) &&
                                        (q.K / static_cast<long long>(slices) * (q.a.k_major ? 1 : q.a.ld) * q.es) % 16 == 0 &&
                                        (q.K / static_cast<long long>(slices) * (q.b.k_major ? 1 : q.b.ld) * q.es) % 16 == 0);
        while (slices > 1 && workspace_bytes < slack + slices * q.M * q.N * sizeof(float)) slices /= 2;
        if (slices > 1 && fast) return launch_splitk(q, slices, ws, s, st);
    }
    return launch(q, s, st);
}

int dlf_b200_gemm_strided_batched(int dtype, int layout, int trans_a, int trans_b, size_t m,
                                  size_t n, size_t k, const void* alpha, const void* a,
                                  size_t a_ld, size_t a_stride, const void* b, size_t b_ld,
                                  size_t b_stride, const void* beta, void* c, size_t c_ld,
                                  size_t c_stride, size_t batch_count, void* stream) {
    if (batch_count < 1) return kInvalidBatchCount;
    Problem q;
    int rc = setup_gemm(q, dtype, layout, trans_a, trans_b, m, n, k, a, a_ld, b, b_ld, c, c_ld);
    if (rc != kSuccess) return rc;
    if (alpha == nullptr || beta == nullptr) return kInvalidValue;
    q.alpha = scalar_to_float(q.fmt, alpha);
    q.beta = scalar_to_float(q.fmt, beta);
    q.batch = static_cast<long long>(batch_count);
    const bool row = layout == DLF_B200_ROW_MAJOR;
    (row ? q.b : q.a).batch_stride = static_cast<long long>(a_stride);
    (row ? q.a : q.b).batch_stride = static_cast<long long>(b_stride);
    q.d_batch_stride = static_cast<long long>(c_stride);
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;
    return launch(q, static_cast<cudaStream_t>(stream));
}

size_t dlf_b200_gemm_batched_workspace_bytes(size_t batch_count) {
    // three int64 offset tables + two float scalar tables + three int32 index tables
    return batch_count * (3 * sizeof(long long) + 2 * sizeof(float) + 3 * sizeof(int));
}

int dlf_b200_gemm_batched(int dtype, int layout, int trans_a, int trans_b, size_t m, size_t n,
                          size_t k, const void* alphas, const void* a, const size_t* a_offsets,
                          size_t a_ld, const void* b, const size_t* b_offsets, size_t b_ld,
                          const void* betas, void* c, const size_t* c_offsets, size_t c_ld,
                          size_t batch_count, void* workspace, size_t workspace_bytes,
                          void* stream) {
    if (batch_count < 1 || alphas == nullptr || betas == nullptr || a_offsets == nullptr ||
        b_offsets == nullptr || c_offsets == nullptr)
        return kInvalidBatchCount;
    Problem q;
    int rc = setup_gemm(q, dtype, layout, trans_a, trans_b, m, n, k, a, a_ld, b, b_ld, c, c_ld);
    if (rc != kSuccess) return rc;
    const size_t need = dlf_b200_gemm_batched_workspace_bytes(batch_count);
    if (workspace == nullptr || workspace_bytes < need) return kInsufficientMemoryTemp;
    if (reinterpret_cast<uintptr_t>(workspace) & 7u) return kInvalidValue;

    const bool row = layout == DLF_B200_ROW_MAJOR;
    std::vector<unsigned char> host(need);
    long long* h_a = reinterpret_cast<long long*>(host.data());
    long long* h_b = h_a + batch_count;
    long long* h_d = h_b + batch_count;
    float* h_alpha = reinterpret_cast<float*>(h_d + batch_count);
    float* h_beta = h_alpha + batch_count;
    for (size_t i = 0; i < batch_count; ++i) {
        // the canonical "A" side is the user's B for row-major calls
        h_a[i] = static_cast<long long>(row ? b_offsets[i] : a_offsets[i]);
        h_b[i] = static_cast<long long>(row ? a_offsets[i] : b_offsets[i]);
        h_d[i] = static_cast<long long>(c_offsets[i]);
        h_alpha[i] = scalar_to_float(q.fmt, static_cast<const char*>(alphas) + i * q.es);
        h_beta[i] = scalar_to_float(q.fmt, static_cast<const char*>(betas) + i * q.es);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamDevice sd(s);
    if (sd.rc != kSuccess) return sd.rc;
    // Tables that are affine in the batch index (offset_i = offset_0 + i * stride with stride >= 0
    // for all three matrices, one alpha and one beta) describe a strided batch: the product then
    // takes the strided path - tensor-map-fed operands, no tables on the device, nothing copied
    // from the host. (dlf's matmul reaches gemmBatched with such tables whenever its operands
    // broadcast in a way its own stride test, linalg_detail.h:1430-1478, does not recognise.)
    {
        bool affine = true;
        const long long sa = batch_count > 1 ? h_a[1] - h_a[0] : 0, sb = batch_count > 1 ? h_b[1] - h_b[0] : 0,
                        sd_ = batch_count > 1 ? h_d[1] - h_d[0] : 0;
        if (sa < 0 || sb < 0 || sd_ < 0) affine = false;
        for (size_t i = 1; affine && i < batch_count; ++i)
            affine = h_a[i] - h_a[0] == static_cast<long long>(i) * sa && h_b[i] - h_b[0] == static_cast<long long>(i) * sb &&
                     h_d[i] - h_d[0] == static_cast<long long>(i) * sd_ && h_alpha[i] == h_alpha[0] && h_beta[i] == h_beta[0];
        if (affine && !((g_force_bn.load() >> 16) & 4)) {  // bit 18 of the tile-width word: always through the tables
            q.a.base += h_a[0] * q.es;
            q.b.base += h_b[0] * q.es;
            q.d += h_d[0] * q.es;
            q.a.batch_stride = sa;
            q.b.batch_stride = sb;
            q.d_batch_stride = sd_;
            q.alpha = h_alpha[0];
            q.beta = h_beta[0];
            q.batch = static_cast<long long>(batch_count);
            return launch(q, s);
        }
    }
    // Tables whose offsets are base + idx * stride with 16-byte aligned base and stride (matrices of a
    // packed array visited in any order, an operand shared by several products, ...) keep the
    // tensor-map-fed kernel: idx becomes the batch coordinate of the operand's tensor map, read from
    // a small table. Needs 16-bit operands that satisfy the TMA rules and, for D, beta == 0 everywhere.
    int* h_ai = reinterpret_cast<int*>(h_beta + batch_count);
    int* h_bi = h_ai + batch_count;
    int* h_di = h_bi + batch_count;
    bool indexed = q.es == 2 && !(g_force_generic.load() & 0xff) && !((g_force_bn.load() >> 16) & 4);
    long long base3[3] = {0, 0, 0}, stride3[3] = {0, 0, 0}, count3[3] = {1, 1, 1};
    {
        const long long* tabs[3] = {h_a, h_b, h_d};
        int* idxs[3] = {h_ai, h_bi, h_di};
        for (int t = 0; indexed && t < 3; ++t) {
            long long lo = tabs[t][0], g = 0;
            for (size_t i = 1; i < batch_count; ++i) lo = std::min(lo, tabs[t][i]);
            for (size_t i = 0; i < batch_count; ++i) {
                long long d = tabs[t][i] - lo;
                while (d != 0) {  // g = gcd(g, d)
                    const long long r = g % d;
                    g = d;
                    d = r;
                }
            }
            long long hi = 0;
            for (size_t i = 0; i < batch_count; ++i) {
                const long long v = g ? (tabs[t][i] - lo) / g : 0;
                hi = std::max(hi, v);
                idxs[t][i] = static_cast<int>(v);
            }
            indexed = (lo * q.es) % 16 == 0 && (g * q.es) % 16 == 0 && g * q.es < (1ll << 40) && hi < INT_MAX - 1;
            base3[t] = lo;
            stride3[t] = g;
            count3[t] = hi + 1;
        }
        for (size_t i = 0; indexed && i < batch_count; ++i) indexed = h_beta[i] == 0.0f;
    }
    if (indexed) {
        Problem r = q;
        r.a.base += base3[0] * q.es;
        r.b.base += base3[1] * q.es;
        r.d += base3[2] * q.es;
        r.a.batch_stride = stride3[0];
        r.b.batch_stride = stride3[1];
        r.d_batch_stride = stride3[2];
        r.batch = static_cast<long long>(batch_count);
        indexed = tma_ok(r.a, r.es, r.M, r.K, count3[0]) && tma_ok(r.b, r.es, r.N, r.K, count3[1]) &&
                  (reinterpret_cast<uintptr_t>(r.d) & 15u) == 0 && (r.ldd * r.es) % 16 == 0 && (r.M * r.es) % 16 == 0;
        if (indexed) {
            CUDA_TRY(cudaMemcpyAsync(workspace, host.data(), need, cudaMemcpyHostToDevice, s));
            char* w = static_cast<char*>(workspace);
            const float* d_alpha = reinterpret_cast<const float*>(w + 3 * sizeof(long long) * batch_count);
            const int* d_idx0 = reinterpret_cast<const int*>(d_alpha + 2 * batch_count);
            r.a_idx = d_idx0;
            r.b_idx = d_idx0 + batch_count;
            r.d_idx = d_idx0 + 2 * batch_count;
            r.a_count = count3[0];
            r.b_count = count3[1];
            r.d_count = count3[2];
            bool one_alpha = true;
            for (size_t i = 1; i < batch_count; ++i) one_alpha = one_alpha && h_alpha[i] == h_alpha[0];
            if (one_alpha) r.alpha = h_alpha[0];
            else r.alphas = d_alpha;
            r.beta = 0.0f;
            return launch(r, s);
        }
    }
    // pageable source: the runtime stages it before returning, so `host` may go out of scope
    CUDA_TRY(cudaMemcpyAsync(workspace, host.data(), need, cudaMemcpyHostToDevice, s));
    char* w = static_cast<char*>(workspace);
    q.a_offs = reinterpret_cast<const long long*>(w);
    q.b_offs = q.a_offs + batch_count;
    q.d_offs = q.b_offs + batch_count;
    q.alphas = reinterpret_cast<const float*>(q.d_offs + batch_count);
    q.betas = q.alphas + batch_count;
    q.batch = static_cast<long long>(batch_count);
    return launch(q, s);
}

int dlf_b200_gemm_batched_noalloc(int dtype, int layout, int trans_a, int trans_b, size_t m,
                                  size_t n, size_t k, const void* alphas, const void* a,
                                  const size_t* a_offsets, size_t a_ld, const void* b,
                                  const size_t* b_offsets, size_t b_ld, const void* betas, void* c,
                                  const size_t* c_offsets, size_t c_ld, size_t batch_count,
                                  void* stream) {
    if (batch_count < 1 || alphas == nullptr || betas == nullptr || a_offsets == nullptr ||
        b_offsets == nullptr || c_offsets == nullptr)
        return kInvalidBatchCount;
    if (batch_count > kNoAllocMaxBatch) return kInsufficientMemoryTemp;  // static scratch is fixed
    Problem q;
    int rc = setup_gemm(q, dtype, layout, trans_a, trans_b, m, n, k, a, a_ld, b, b_ld, c, c_ld);
    if (rc != kSuccess) return rc;
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;
    NoAllocDevice* nd = nullptr;
    rc = noalloc_device(&nd);  // first call on a device: looks up the static arrays' addresses
    if (rc != kSuccess) return rc;

    // host staging for the tables is per-thread static storage as well
    thread_local static unsigned char host[kNoAllocTableBytes];
    const bool row = layout == DLF_B200_ROW_MAJOR;
    long long* h_a = reinterpret_cast<long long*>(host);
    long long* h_b = h_a + batch_count;
    long long* h_d = h_b + batch_count;
    float* h_alpha = reinterpret_cast<float*>(h_d + batch_count);
    float* h_beta = h_alpha + batch_count;
    for (size_t i = 0; i < batch_count; ++i) {
        h_a[i] = static_cast<long long>(row ? b_offsets[i] : a_offsets[i]);
        h_b[i] = static_cast<long long>(row ? a_offsets[i] : b_offsets[i]);
        h_d[i] = static_cast<long long>(c_offsets[i]);
        h_alpha[i] = scalar_to_float(q.fmt, static_cast<const char*>(alphas) + i * q.es);
        h_beta[i] = scalar_to_float(q.fmt, static_cast<const char*>(betas) + i * q.es);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t need = batch_count * (3 * sizeof(long long) + 2 * sizeof(float));
    // every byte the kernel reads is rewritten here, so nothing of an earlier call survives
    CUDA_TRY(cudaMemcpyAsync(nd->tables, host, need, cudaMemcpyHostToDevice, s));
    q.a_offs = reinterpret_cast<const long long*>(nd->tables);
    q.b_offs = q.a_offs + batch_count;
    q.d_offs = q.b_offs + batch_count;
    q.alphas = reinterpret_cast<const float*>(q.d_offs + batch_count);
    q.betas = q.alphas + batch_count;
    q.batch = static_cast<long long>(batch_count);
    return launch(q, s, &nd->st);
}

size_t dlf_b200_conv2d_workspace_bytes(int dtype, size_t batches, size_t channels, size_t height, size_t width,
                                       size_t, size_t, size_t num_kernels, size_t group, size_t kernel_h,
                                       size_t kernel_w) {
    // Optional scratch: the filter bank re-laid as the kernel's shared-memory stage images (a few
    // hundred KB to a few MB). The im2col matrix itself is never materialised. An upper bound over
    // the tilings the library may choose is returned; with less (or none) the kernel gathers the
    // filter bank itself, more slowly.
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es) || group == 0 || kernel_w == 0) return 0;
    const size_t cg = channels / group, ng = num_kernels / group;
    const size_t bk = 128 / es, dup = es == 4 ? 2 : 1;
    const size_t plain = group * ((ng + 255) / 256 * 256 + 256) * 128 * dup * ((cg * kernel_h * kernel_w + bk - 1) / bk);
    // row form: taps x K' <= (KW + 2*sw) x C*KH for strides sw <= 4 (column phases join K, taps
    // become ceil-ish KW/sw shifts), output channels padded to the tile's channel count
    const size_t row = group * ((ng + 255) / 256 * 256 + 256) * 128 * dup *
                       ((cg * kernel_h * (kernel_w + 8) + bk - 1) / bk + 8);
    size_t need = (plain > row ? plain : row) + 256;
    // channels-last route (16-bit, one group): channels-last copy of the activations plus the
    // filter bank in (tap, channel) order
    if (es == 2 && group == 1) {
        const size_t cp = (channels + 7) / 8 * 8, ck = (channels + 63) / 64 * 64;
        const size_t cl = batches * height * width * cp * 2 + num_kernels * kernel_h * kernel_w * ck * 2 + 4096;
        if (cl > need) need = cl;
        // halo-tile kernel: bordered channel-group-major copy (at most (H + KH) x (W + KW) pixels per plane)
        const size_t halo = batches * ((channels + 7) / 8) * (height + kernel_h) * (width + kernel_w) * 16 +
                            num_kernels * kernel_h * kernel_w * ck * 2 + 4096;
        if (halo > need) need = halo;
        if (channels <= 4) {
            // bordered row-pair copy: at most (H + 2*KH + 2) row pairs of (W + 2*KW + 80) pixels of 16 bytes per image
            // (all phases of a row together; every phase rounded up to the tile's columns per row)
            const size_t small = batches * (height + 2 * kernel_h + 2) * (width + 2 * kernel_w + 80) * 16 +
                                 num_kernels * (kernel_h + 1) / 2 * 128 + 4096;
            if (small > need) need = small;
        }
    }
    return need;
}

int dlf_b200_conv2d_fused(int dtype, size_t batches, size_t channels, size_t height, size_t width,
                          size_t output_h, size_t output_w, size_t num_kernels, size_t group,
                          size_t kernel_h, size_t kernel_w, size_t pad_top, size_t pad_left,
                          size_t pad_bottom, size_t pad_right, size_t stride_h, size_t stride_w,
                          size_t dilation_h, size_t dilation_w, const void* x, const void* w,
                          const void* bias, const void* residual, int activation, void* y,
                          void* workspace, size_t workspace_bytes, void* stream) {
    (void)pad_bottom;
    (void)pad_right;
    Problem q;
    if (activation != DLF_B200_ACT_NONE && activation != DLF_B200_ACT_RELU) return kInvalidValue;
    q.resid = static_cast<const char*>(residual);
    q.relu = activation == DLF_B200_ACT_RELU ? 1 : 0;
    q.pack_ws = static_cast<unsigned char*>(workspace);
    q.pack_ws_bytes = workspace_bytes;
    if (!dtype_info(dtype, q.fmt, q.es)) return kNotImplemented;
    if (batches == 0 || channels == 0 || height == 0 || width == 0 || output_h == 0 ||
        output_w == 0 || num_kernels == 0 || kernel_h == 0 || kernel_w == 0)
        return kInvalidDimension;
    if (group == 0 || channels % group != 0 || num_kernels % group != 0) return kInvalidDimension;
    if (stride_h == 0 || stride_w == 0 || dilation_h == 0 || dilation_w == 0) return kInvalidValue;
    if (x == nullptr) return kInvalidMatrixA;
    if (w == nullptr) return kInvalidMatrixB;
    if (y == nullptr) return kInvalidMatrixC;
    const long long P = static_cast<long long>(output_h) * output_w;
    const long long cg = static_cast<long long>(channels / group);
    const long long ng = static_cast<long long>(num_kernels / group);
    const long long K = cg * kernel_h * kernel_w;
    const size_t lim = 1u << 30;
    if (height >= lim || width >= lim || kernel_h >= lim || kernel_w >= lim || pad_top >= lim ||
        pad_left >= lim || stride_h >= lim || stride_w >= lim || dilation_h >= lim ||
        dilation_w >= lim || static_cast<long long>(height) * width >= INT_MAX)
        return kInvalidDimension;

    // The k table of the tensor-memory-operand kernel keeps kh*dilation_h and kw*dilation_w as
    // 16-bit values and the offset of a tap inside one image's channel group as a 32-bit one;
    // a convolution beyond either takes the shared-memory-operand kernel, which uses wide indices.
    const bool ktable_fits = (kernel_h - 1) * dilation_h <= 32767 && (kernel_w - 1) * dilation_w <= 32767 &&
                             cg * static_cast<long long>(height) * width < INT_MAX;
    q.no_ts = !ktable_fits;
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;

    // A 1x1, stride-1, unpadded convolution is a batched GEMM over the images,
    //     Y[b] (Cout x P) = W (Cout x Cin) * X[b] (Cin x P),
    // exactly the reference's convWithIm2Col shortcut (gpgpu/src/gdnn.cpp:1512-1559: weights
    // shared with stride 0). With TMA-compatible strides it takes the TMA-fed kernel.
    if (kernel_h == 1 && kernel_w == 1 && stride_h == 1 && stride_w == 1 && pad_top == 0 &&
        pad_left == 0 && output_h == height && output_w == width && group == 1 && q.es == 2 &&
        (P * q.es) % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && (channels * q.es) % 16 == 0 &&
        !(g_force_generic.load() & 0xff)) {
        q.M = P;
        q.N = static_cast<long long>(num_kernels);
        q.K = static_cast<long long>(channels);
        q.batch = static_cast<long long>(batches);
        q.a.base = static_cast<const char*>(x);
        q.a.k_major = 0;
        q.a.ld = P;
        q.a.batch_stride = static_cast<long long>(channels) * P;
        q.b.base = static_cast<const char*>(w);
        q.b.k_major = 1;
        q.b.ld = static_cast<long long>(channels);
        q.b.batch_stride = 0;
        q.d = static_cast<char*>(y);
        q.ldd = P;
        q.d_batch_stride = static_cast<long long>(num_kernels) * P;
        q.bias = static_cast<const char*>(bias);
        q.bias_stride = 0;
        // With the roles swapped (rows = output channels = lanes, columns = pixels) a lane's 32
        // columns are 64 consecutive bytes of Y: four 16-byte shared-memory stores fill the staging
        // block of a TMA store, where the pixel-per-lane form needs 32 two-byte ones. Measured on the
        // ResNet-50 shapes (batch 256): 128 -> 512 at 28x28 94 -> 86 us, 256 -> 64 at 56x56 98 -> 90 us,
        // 512 -> 128 at 28x28 56 -> 49 us. With 64 output channels half of the 128 lanes idle, but the
        // epilogue warps of the idle quadrants skip their blocks and the staged stores are still the
        // cheaper ones (64 -> 64 at 56x56: 69 -> 63 us; 256 -> 64: 93 -> 92 us). Bit 19 of the
        // tile-width word: never swap.
        const uintptr_t ya = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(residual);
        if (P % 8 == 0 && P >= 32 && ya % 16 == 0 && num_kernels >= 64 && !((g_force_bn.load() >> 16) & 8)) {
            std::swap(q.a, q.b);
            q.M = static_cast<long long>(num_kernels);
            q.N = P;
            q.cl_swap = 1;
            q.out_nchw = 3;
            q.out_vec = 8;
            q.g.P = static_cast<int>(P);
            q.g.out_img_stride = static_cast<long long>(num_kernels) * P;
        }
        return launch(q, static_cast<cudaStream_t>(stream));
    }

    q.M = static_cast<long long>(batches) * P;  // global output pixel index
    q.N = ng;
    q.K = K;
    q.batch = static_cast<long long>(group);
    q.a.base = static_cast<const char*>(x);
    q.a.im2col = 1;
    q.a.k_major = 0;
    q.a.ld = 0;
    q.a.batch_stride = cg * static_cast<long long>(height) * width;
    q.b.base = static_cast<const char*>(w);
    q.b.k_major = 1;
    q.b.ld = K;
    q.b.batch_stride = ng * K;
    q.d = static_cast<char*>(y);
    q.ldd = P;
    q.d_batch_stride = ng * P;
    q.alpha = 1.f;
    q.beta = 0.f;
    q.bias = static_cast<const char*>(bias);
    q.bias_stride = ng;
    q.g.H = static_cast<int>(height);
    q.g.W = static_cast<int>(width);
    q.g.OH = static_cast<int>(output_h);
    q.g.OW = static_cast<int>(output_w);
    q.g.KH = static_cast<int>(kernel_h);
    q.g.KW = static_cast<int>(kernel_w);
    q.g.pad_t = static_cast<int>(pad_top);
    q.g.pad_l = static_cast<int>(pad_left);
    q.g.sh = static_cast<int>(stride_h);
    q.g.sw = static_cast<int>(stride_w);
    q.g.dh = static_cast<int>(dilation_h);
    q.g.dw = static_cast<int>(dilation_w);
    q.g.P = static_cast<int>(P);
    q.g.img_stride = static_cast<long long>(channels) * height * width;
    q.g.out_img_stride = static_cast<long long>(num_kernels) * P;
    if (P > INT_MAX) return kInvalidDimension;

    // Filters over at most 4 input channels, at most 8 taps per row, horizontal stride 1, 2 or 4 and
    // at most 128 output channels (the 7x7 stride-2 RGB stem of a ResNet): bordered, phase-split
    // row-pair copy (channels_last.cuh) + the dedicated kernel of conv_small.cuh.
    {
        const int tune = g_force_generic.load();
        const int cl_neutral = 0x100 | 0x4000 | 0x10000000 | 0x20000000;
        const int route = g_force_bn.load() >> 16;
        const long long kb2 = (static_cast<long long>(kernel_h) + 1) / 2;
        const long long rstep = stride_h % 2 == 0 ? 2 : 1;
        const long long jn = ((static_cast<long long>(output_h) - 1) * stride_h + 2 * (kb2 - 1)) / rstep + 1;  // row pairs
        const bool sw_ok = stride_w == 1 || stride_w == 2 || stride_w == 4;
        const long long swl = sw_ok ? static_cast<long long>(stride_w) : 1;
        const long long wph = static_cast<long long>(output_w) - 1 + 8 / swl;  // pixels per phase of a bordered row
        const long long owp = (wph + 7) / 8 * 8;                               // tile columns per output row
        const size_t w_bytes = (static_cast<size_t>(num_kernels) * kb2 * 128 + 1023) / 1024 * 1024;
        const size_t x_bytes = static_cast<size_t>(batches) * jn * swl * (owp + 8) * 16;  // rows of up to owp + 8 pixels
        unsigned char* ws = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 255u) & ~uintptr_t(255));
        const size_t slack = static_cast<size_t>(ws - static_cast<unsigned char*>(workspace));
        if (q.es == 2 && group == 1 && channels <= 4 && (tune & ~cl_neutral) == 0 && !(route & 1) && workspace != nullptr &&
            workspace_bytes >= slack + w_bytes + x_bytes && kernel_w <= 8 && sw_ok && stride_h <= 2 &&
            dilation_h == 1 && dilation_w == 1 && num_kernels <= 128 && owp <= 240 && jn < (1 << 28) &&
            pad_top < (1u << 28) && pad_left < (1u << 28) && P * static_cast<long long>(num_kernels) < (1ll << 38)) {
            DeviceState* st = nullptr;
            int rc = ensure_device(&st);
            if (rc != kSuccess) return rc;
            SmallParams sp{};
            // rows per tile: as many as 240 columns hold (two accumulators and the 32-column loads of
            // the epilogue must stay inside the 512 columns of tensor memory), an even count when the
            // width per row is an odd multiple of 8, so that the tile width is a multiple of 16
            int rr = static_cast<int>(240 / owp);
            if (rr > static_cast<int>(output_h)) rr = static_cast<int>(output_h);
            long long owp_t = owp;
            if ((rr * owp_t) % 16 != 0) {
                if (rr > 1) --rr;
                else owp_t += 8;
            }
            sp.R = rr;
            sp.OWp = static_cast<int>(owp_t);
            sp.BN = static_cast<int>(rr * owp_t);
            sp.kb_rows = static_cast<int>(2 / rstep);
            sp.span = rr + sp.kb_rows * static_cast<int>(kb2 - 1);
            sp.phase_bytes = static_cast<unsigned>((sp.span * owp_t + 8) * 16);
            sp.stage_bytes = static_cast<unsigned>((swl * sp.phase_bytes + 127) / 128 * 128);
            const long long a_bytes = kb2 * kBM * 128;
            long long stages = (kSmemPerBlockOptin - st->static_smem_small - 1024 - a_bytes - kSmallStageOut) / sp.stage_bytes;
            if (stages > kSmallMaxStages) stages = kSmallMaxStages;
            const long long tiles_per_image = (static_cast<long long>(output_h) + rr - 1) / rr;
            const long long total_tiles = static_cast<long long>(batches) * tiles_per_image;
            if (stages >= 2 && total_tiles < INT_MAX && sp.BN <= 240 && sp.BN % 16 == 0) {
                clear_stale_error();
                cudaStream_t cs = static_cast<cudaStream_t>(stream);
                uint16_t* wpk = reinterpret_cast<uint16_t*>(ws);
                uint4* xp = reinterpret_cast<uint4*>(ws + w_bytes);
                const long long total = static_cast<long long>(batches) * swl * jn * owp_t;
                const unsigned xblocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 32ll * st->num_sms));
                cl_pack_small_activations_kernel<<<xblocks, 256, 0, cs>>>(
                    static_cast<const uint16_t*>(x), xp, static_cast<int>(channels), static_cast<int>(height),
                    static_cast<int>(width), static_cast<int>(jn), static_cast<int>(owp_t), static_cast<int>(swl),
                    static_cast<int>(rstep), static_cast<int>(pad_top), static_cast<int>(pad_left), total);
                g_launches.fetch_add(1);
                CUDA_TRY(cudaGetLastError());
                const long long wtotal = static_cast<long long>(num_kernels) * kb2 * 64;
                cl_pack_small_filters_kernel<<<static_cast<unsigned>(std::min<long long>((wtotal + 255) / 256, 8ll * st->num_sms)), 256, 0, cs>>>(
                    static_cast<const uint16_t*>(w), wpk, static_cast<int>(num_kernels), static_cast<int>(channels),
                    static_cast<int>(kernel_h), static_cast<int>(kernel_w), static_cast<int>(kb2), static_cast<int>(swl));
                g_launches.fetch_add(1);
                CUDA_TRY(cudaGetLastError());
                sp.xp = reinterpret_cast<const char*>(xp);
                sp.y = static_cast<char*>(y);
                sp.bias = static_cast<const char*>(bias);
                sp.resid = q.resid;
                sp.relu = q.relu;
                sp.fmt = q.fmt;
                sp.Cout = static_cast<int>(num_kernels);
                sp.OH = static_cast<int>(output_h);
                sp.OW = static_cast<int>(output_w);
                sp.P = static_cast<int>(P);
                sp.J = static_cast<int>(jn);
                sp.sh = static_cast<int>(stride_h);
                sp.sw = static_cast<int>(swl);
                sp.rstep = static_cast<int>(rstep);
                sp.KB = static_cast<int>(kb2);
                sp.images = static_cast<int>(batches);
                sp.tiles_per_image = static_cast<int>(tiles_per_image);
                sp.total_tiles = static_cast<int>(total_tiles);
                sp.out_img_stride = static_cast<long long>(num_kernels) * P;
                sp.stages = static_cast<int>(stages);
                sp.status = st->status;
                sp.wait_limit = 1ll << 32;
                CUtensorMap tm_w, tm_d;
                std::memset(&tm_d, 0, sizeof(tm_d));
                GenOperand wop{};
                wop.base = reinterpret_cast<const char*>(wpk);
                wop.ld = kb2 * 64;
                wop.k_major = 1;
                rc = encode_map(*st, &tm_w, wop, 2, static_cast<long long>(num_kernels), kb2 * 64, 1, kBM);
                if (rc != kSuccess) return rc;
                const uintptr_t ya = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(residual);
                if (P % 8 == 0 && output_w % 8 == 0 && ya % 16 == 0 && !(tune & 0x4000)) {
                    cuuint64_t dims[3] = {static_cast<cuuint64_t>(P), static_cast<cuuint64_t>(num_kernels),
                                          static_cast<cuuint64_t>(batches)};
                    cuuint64_t strides[2] = {static_cast<cuuint64_t>(P * 2), static_cast<cuuint64_t>(P * num_kernels * 2)};
                    cuuint32_t box[3] = {32, 32, 1};
                    cuuint32_t estr[3] = {1, 1, 1};
                    sp.d_tma = st->encode(&tm_d, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, y, dims, strides, box, estr,
                                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
                                   ? 1
                                   : 0;
                }
                const unsigned grid = static_cast<unsigned>(total_tiles < st->num_sms ? total_tiles : st->num_sms);
                const size_t dyn = static_cast<size_t>(a_bytes) + kSmallStageOut + static_cast<size_t>(stages) * sp.stage_bytes + 1024;
                conv_small_kernel<<<grid, kSmallThreads, dyn, cs>>>(sp, tm_w, tm_d);
                g_launches.fetch_add(1);
                CUDA_TRY(cudaGetLastError());
                return kSuccess;
            }
        }
    }

    // Stride-1 filters larger than 1x1 over a multiple of 64 channels with at most 64 output channels
    // and rows of a multiple of 8 outputs (64 -> 64 3x3 at 56x56): the halo-tile kernel (conv_halo.cuh)
    // - bordered channel-group-major copy, every tile's activations fetched once, filter taps as
    // descriptor offsets. With few output channels the activations are most of the operand traffic
    // (210 -> 186 us at batch 256, main kernel 165 -> 126 us); with 128 and more the filter bank is,
    // and the im2col-mode route with its 256-pixel tiles is faster (128 -> 128 at 28x28: 87 vs 105 us).
    // Bit 24 of the tile-width word takes this kernel for every layer it can serve, bit 23 for none.
    {
        const int tune = g_force_generic.load();
        const int cl_neutral = 0x100 | 0x4000 | 0x10000000 | 0x20000000;
        const int route = g_force_bn.load() >> 16;
        const long long taps = static_cast<long long>(kernel_h) * kernel_w;
        const long long hp = static_cast<long long>(output_h) + kernel_h - 1;
        const long long wp = static_cast<long long>(output_w) + kernel_w - 1;
        const long long cg = static_cast<long long>(channels) / 8;
        const size_t w_bytes = (static_cast<size_t>(num_kernels) * taps * channels * 2 + 1023) / 1024 * 1024;
        const size_t x_bytes = static_cast<size_t>(batches) * cg * hp * wp * 16;
        unsigned char* ws = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 255u) & ~uintptr_t(255));
        const size_t slack = static_cast<size_t>(ws - static_cast<unsigned char*>(workspace));
        if (q.es == 2 && group == 1 && channels % 64 == 0 && taps > 1 && stride_h == 1 && stride_w == 1 &&
            dilation_h == 1 && dilation_w == 1 && (tune & ~cl_neutral) == 0 && !(route & 1) && !(route & 128) &&
            workspace != nullptr && workspace_bytes >= slack + w_bytes + x_bytes && wp <= 240 && output_w % 2 == 0 &&
            ((num_kernels <= 64 && output_w % 8 == 0) || (route & 256)) &&
            kernel_h <= 16 && kernel_w <= 16 && pad_top < (1u << 20) && pad_left < (1u << 20) &&
            P * static_cast<long long>(num_kernels) < (1ll << 38) && taps * static_cast<long long>(channels) < INT_MAX - 512) {
            DeviceState* st = nullptr;
            int rc = ensure_device(&st);
            if (rc != kSuccess) return rc;
            HaloParams hp_{};
            int rr = static_cast<int>(240 / wp);
            if (rr > static_cast<int>(output_h)) rr = static_cast<int>(output_h);
            hp_.R = rr;
            hp_.BN = static_cast<int>((rr * wp + 15) / 16 * 16);
            hp_.group_units = static_cast<unsigned>((hp_.BN + (kernel_h - 1) * wp + kernel_w + 7) / 8 * 8);
            hp_.stage_bytes = 8u * hp_.group_units * 16u;
            const long long budget = kSmemPerBlockOptin - st->static_smem_halo - 1024 - kHaloStageOut;
            int hs = 2;
            long long sa = (budget - static_cast<long long>(hs) * hp_.stage_bytes) / (kBM * 128);
            if (sa > kHaloMaxA) sa = kHaloMaxA;
            const long long tiles_per_image = (static_cast<long long>(output_h) + rr - 1) / rr;
            const long long co_tiles = (static_cast<long long>(num_kernels) + kBM - 1) / kBM;
            const long long total_tiles = static_cast<long long>(batches) * tiles_per_image * co_tiles;
            if (sa >= 3 && total_tiles < INT_MAX) {
                clear_stale_error();
                cudaStream_t cs = static_cast<cudaStream_t>(stream);
                uint16_t* wpk = reinterpret_cast<uint16_t*>(ws);
                uint4* xh = reinterpret_cast<uint4*>(ws + w_bytes);
                const long long total = static_cast<long long>(batches) * cg * hp * wp;
                halo_pack_activations_kernel<<<static_cast<unsigned>(std::min<long long>((total + 255) / 256, 32ll * st->num_sms)), 256, 0, cs>>>(
                    static_cast<const uint16_t*>(x), xh, static_cast<int>(channels), static_cast<int>(height),
                    static_cast<int>(width), static_cast<int>(hp), static_cast<int>(wp), static_cast<int>(pad_top),
                    static_cast<int>(pad_left), total);
                g_launches.fetch_add(1);
                CUDA_TRY(cudaGetLastError());
                const long long wtotal = static_cast<long long>(num_kernels) * channels;
                cl_pack_filters_kernel<<<static_cast<unsigned>(std::min<long long>((wtotal + 255) / 256, 8ll * st->num_sms)), 256, 0, cs>>>(
                    static_cast<const uint16_t*>(w), wpk, static_cast<int>(num_kernels), static_cast<int>(channels),
                    static_cast<int>(taps), static_cast<int>(channels));
                g_launches.fetch_add(1);
                CUDA_TRY(cudaGetLastError());
                hp_.xh = reinterpret_cast<const char*>(xh);
                hp_.y = static_cast<char*>(y);
                hp_.bias = static_cast<const char*>(bias);
                hp_.resid = q.resid;
                hp_.relu = q.relu;
                hp_.fmt = q.fmt;
                hp_.Cout = static_cast<int>(num_kernels);
                hp_.CB = static_cast<int>(channels / 64);
                hp_.OH = static_cast<int>(output_h);
                hp_.OW = static_cast<int>(output_w);
                hp_.P = static_cast<int>(P);
                hp_.Hp = static_cast<int>(hp);
                hp_.Wp = static_cast<int>(wp);
                hp_.KH = static_cast<int>(kernel_h);
                hp_.KW = static_cast<int>(kernel_w);
                hp_.images = static_cast<int>(batches);
                hp_.tiles_per_image = static_cast<int>(tiles_per_image);
                hp_.co_tiles = static_cast<int>(co_tiles);
                hp_.total_tiles = static_cast<int>(total_tiles);
                hp_.out_img_stride = static_cast<long long>(num_kernels) * P;
                hp_.a_stages = static_cast<int>(sa);
                hp_.h_stages = hs;
                hp_.status = st->status;
                hp_.wait_limit = 1ll << 32;
                const uintptr_t ya = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(residual);
                hp_.out_vec = (output_w % 8 == 0 && ya % 16 == 0) ? 8 : (output_w % 4 == 0 && ya % 8 == 0) ? 4 : (ya % 4 == 0 ? 2 : 1);
                CUtensorMap tm_w, tm_d;
                std::memset(&tm_d, 0, sizeof(tm_d));
                GenOperand wop{};
                wop.base = reinterpret_cast<const char*>(wpk);
                wop.ld = taps * static_cast<long long>(channels);
                wop.k_major = 1;
                rc = encode_map(*st, &tm_w, wop, 2, static_cast<long long>(num_kernels), taps * static_cast<long long>(channels), 1, kBM);
                if (rc != kSuccess) return rc;
                if (hp_.out_vec == 8 && !(tune & 0x4000)) {
                    cuuint64_t dims[3] = {static_cast<cuuint64_t>(P), static_cast<cuuint64_t>(num_kernels),
                                          static_cast<cuuint64_t>(batches)};
                    cuuint64_t strides[2] = {static_cast<cuuint64_t>(P * 2), static_cast<cuuint64_t>(P * num_kernels * 2)};
                    cuuint32_t box[3] = {32, 32, 1};
                    cuuint32_t estr[3] = {1, 1, 1};
                    hp_.d_tma = st->encode(&tm_d, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, y, dims, strides, box, estr,
                                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
                                    ? 1
                                    : 0;
                }
                const unsigned grid = static_cast<unsigned>(total_tiles < st->num_sms ? total_tiles : st->num_sms);
                const size_t dyn = static_cast<size_t>(sa) * kBM * 128 + kHaloStageOut + static_cast<size_t>(hs) * hp_.stage_bytes + 1024;
                conv_halo_kernel<<<grid, kHaloThreads, dyn, cs>>>(hp_, tm_w, tm_d);
                g_launches.fetch_add(1);
                CUDA_TRY(cudaGetLastError());
                return kSuccess;
            }
        }
    }

    // Channels-last route (channels_last.cuh): 16-bit, one group, enough scratch. The activations are
    // copied into scratch as (N, H, W, C'), after which the tensor-map unit feeds the operand by
    // itself: im2col-mode loads for general filters (one load = 128 filter windows x 64 channels of
    // one tap), plain tiled loads for 1x1 filters (the copy then keeps only the pixels the strides
    // select, and the convolution is one GEMM over all images). The reference's Xconvgemm gathers
    // the same operand element by element (kernels/levelx/xconvgemm_part1.cl:26-117).
    {
        const int tune = g_force_generic.load();
        const bool pointwise = kernel_h == 1 && kernel_w == 1 && pad_top == 0 && pad_left == 0 &&
                               (output_h - 1) * stride_h < height && (output_w - 1) * stride_w < width;
        const long long taps = static_cast<long long>(kernel_h) * kernel_w;
        const long long cp = (static_cast<long long>(channels) + 7) / 8 * 8;
        const bool w_direct = pointwise && channels % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0;
        const long long ck = pointwise ? cp : (static_cast<long long>(channels) + 63) / 64 * 64;
        const long long xh = pointwise ? static_cast<long long>(output_h) : static_cast<long long>(height);
        const long long xw = pointwise ? static_cast<long long>(output_w) : static_cast<long long>(width);
        const size_t w_bytes = w_direct ? 0 : (static_cast<size_t>(num_kernels) * taps * ck * 2 + 1023) / 1024 * 1024;
        const size_t x_bytes = static_cast<size_t>(batches) * xh * xw * cp * 2;
        unsigned char* ws = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 255u) & ~uintptr_t(255));
        const size_t slack = static_cast<size_t>(ws - static_cast<unsigned char*>(workspace));
        // a filter with few channels would spend most of each 64-channel k-block on zeros
        const bool dense_k = pointwise || channels * 2 >= static_cast<size_t>(ck);
        // 1x1 filters: the transposing copy costs a pass over the input, repaid by the output side
        // (tensor-map stores, no per-element gather) only when the layer widens (measured on the
        // ResNet-50 shapes: 256->1024 at 14x14 99 -> 74 us, 1024->256 70 -> 90 us)
        const bool widens = !pointwise || num_kernels >= 2 * channels;
        // every measurement / forcing bit that addresses the other convolution kernels (and the
        // route's own off switch, bit 16 of the tile-width word) keeps the call on those kernels
        const int cl_neutral = 0x100 | 0x4000 | 0x10000000 | 0x20000000;
        const int route = g_force_bn.load() >> 16;
        if (q.es == 2 && group == 1 && (tune & ~cl_neutral) == 0 && !(route & 1) && workspace != nullptr &&
            workspace_bytes >= slack + w_bytes + x_bytes && dense_k && widens && batches < 65536 && cp < 65536ll * 64 &&
            (pointwise || (dilation_h * (kernel_h - 1) < 256 && dilation_w * (kernel_w - 1) < 256 && stride_h <= 8 &&
                           stride_w <= 8)) &&
            q.M < INT_MAX - 512 && taps * ck < INT_MAX - 512) {
            DeviceState* st = nullptr;
            int rc = ensure_device(&st);
            if (rc != kSuccess) return rc;
            if (pointwise || st->encode_im2col != nullptr) {
                clear_stale_error();
                cudaStream_t cs = static_cast<cudaStream_t>(stream);
                uint16_t* wp = reinterpret_cast<uint16_t*>(ws);
                uint16_t* xp = reinterpret_cast<uint16_t*>(ws + w_bytes);
                const long long xpix = xh * xw;
                dim3 grid(static_cast<unsigned>((xpix + kClTile - 1) / kClTile), static_cast<unsigned>((cp + kClTile - 1) / kClTile),
                          static_cast<unsigned>(batches));
                const uint16_t* xs = static_cast<const uint16_t*>(x);
                const long long plane = static_cast<long long>(height) * width;
                const long long total = static_cast<long long>(batches) * channels * plane;
                const uintptr_t xa = reinterpret_cast<uintptr_t>(x);
                const int ci = static_cast<int>(channels), cpi = static_cast<int>(cp);
                if (!pointwise || (stride_h == 1 && stride_w == 1)) {
                    // whole planes (a 1x1 filter with unit strides keeps every pixel): one row of `plane` pixels
                    const int pl = static_cast<int>(plane);
                    if (plane % 8 == 0 && xa % 16 == 0)
                        cl_pack_activations_kernel<CL_VEC8><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, pl, 1, pl, 1, 1, cpi, total);
                    else if (plane % 4 == 0 && xa % 8 == 0)
                        cl_pack_activations_kernel<CL_VEC4><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, pl, 1, pl, 1, 1, cpi, total);
                    else if (plane % 2 == 0 && xa % 4 == 0)
                        cl_pack_activations_kernel<CL_VEC2><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, pl, 1, pl, 1, 1, cpi, total);
                    else
                        cl_pack_activations_kernel<CL_FUNNEL><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, pl, 1, pl, 1, 1, cpi, total);
                } else {
                    const int wi = static_cast<int>(width), ohi = static_cast<int>(output_h), owi = static_cast<int>(output_w);
                    const int shi = static_cast<int>(stride_h), swi = static_cast<int>(stride_w);
                    const long long row_bytes = static_cast<long long>(stride_h) * width * 2;
                    const bool s2 = stride_w == 2 && 2 * output_w <= width;
                    if (s2 && output_w % 4 == 0 && row_bytes % 16 == 0 && (plane * 2) % 16 == 0 && xa % 16 == 0)
                        cl_pack_activations_kernel<CL_S2_VEC4><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, wi, ohi, owi, shi, swi, cpi, total);
                    else if (s2 && output_w % 2 == 0 && row_bytes % 8 == 0 && (plane * 2) % 8 == 0 && xa % 8 == 0)
                        cl_pack_activations_kernel<CL_S2_VEC2><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, wi, ohi, owi, shi, swi, cpi, total);
                    else
                        cl_pack_activations_kernel<CL_ANY><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, wi, ohi, owi, shi, swi, cpi, total);
                }
                g_launches.fetch_add(1);
                CUDA_TRY(cudaGetLastError());
                if (!w_direct) {
                    const long long total = static_cast<long long>(num_kernels) * ck;
                    const unsigned blocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 8ll * st->num_sms));
                    cl_pack_filters_kernel<<<blocks, 256, 0, cs>>>(static_cast<const uint16_t*>(w), wp,
                                                                  static_cast<int>(num_kernels), static_cast<int>(channels),
                                                                  static_cast<int>(taps), static_cast<int>(ck));
                    g_launches.fetch_add(1);
                    CUDA_TRY(cudaGetLastError());
                }
                Problem r = q;
                r.batch = 1;
                r.N = static_cast<long long>(num_kernels);
                r.K = w_direct ? static_cast<long long>(channels) : taps * ck;
                r.a.base = reinterpret_cast<const char*>(xp);
                r.a.im2col = 0;
                r.a.k_major = 1;
                r.a.ld = cp;
                r.a.batch_stride = 0;
                r.b.base = w_direct ? static_cast<const char*>(w) : reinterpret_cast<const char*>(wp);
                r.b.k_major = 1;
                r.b.ld = r.K;
                r.b.batch_stride = 0;
                r.d_batch_stride = 0;
                r.bias_stride = 0;
                r.out_nchw = 1;
                r.a_cl = pointwise ? 0 : 1;
                r.cl_cblocks = static_cast<int>(ck / 64);
                r.cl_n = static_cast<long long>(batches);
                r.cl_h = xh;
                r.cl_w = xw;
                r.cl_cp = cp;
                r.pack_ws = nullptr;
                r.pack_ws_bytes = 0;
                // Swapped roles when the planes allow 16-byte stores: the lanes then hold output
                // channels and each writes runs of consecutive pixels (an NCHW tensor is contiguous
                // along pixels), and a tile is 256 pixels wide whatever the channel count, which
                // halves the filter-bank traffic of layers with 64 or 128 output channels (128 -> 128
                // 3x3 at 28x28: 93 -> 67 us). With smaller vectors the scattered stores of the 32
                // lanes cost more than the paired stores of the pixel-per-lane form (256 -> 1024
                // 1x1 at 14x14: 67 -> 92 us), so those planes stay unswapped.
                {
                    const uintptr_t ya = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(residual);
                    int vec = 1;
                    if (P % 8 == 0 && ya % 16 == 0) vec = 8;
                    else if (P % 4 == 0 && ya % 8 == 0) vec = 4;
                    else if (P % 2 == 0 && ya % 4 == 0) vec = 2;
                    const bool want = (route & 2) ? vec > 1 : vec == 8;  // route bit 1: measurement, swap with any vector
                    if (want && P >= 32) {
                        std::swap(r.a, r.b);
                        r.M = static_cast<long long>(num_kernels);
                        r.N = q.M;  // output pixels of all images
                        r.cl_swap = 1;
                        r.out_nchw = 3;
                        r.out_vec = vec;
                    }
                }
                rc = launch(r, cs, st);
                if (rc != kNotImplemented) return rc;
            }
        }
    }

    // Row form (see contraction_ts.cuh): horizontal taps become output columns of the GEMM. With
    // stride_w = sw the input columns split into sw phases that join the channels in K, and the
    // taps become the shifts d = floor((kw - pad_left) / sw).
    const int path = ktable_fits ? (g_force_generic.load() & 0xff) : 2;
    const long long sw = static_cast<long long>(stride_w);
    const long long pl = static_cast<long long>(pad_left);
    auto floor_div = [](long long a, long long b) { return a >= 0 ? a / b : -((-a + b - 1) / b); };
    const long long dmin = floor_div(-pl, sw);
    const long long dmax = floor_div(static_cast<long long>(kernel_w) - 1 - pl, sw);
    const long long taps = dmax - dmin + 1;
    const long long lo = -dmin;
    const long long hi = dmax > 0 ? dmax : 0;
    // positions per row: every input column for sw = 1; for sw > 1 the w' that some output needs
    // and whose columns sw*w' + r are not all beyond the row
    const long long wv = sw == 1 ? static_cast<long long>(width)
                                 : std::min<long long>(static_cast<long long>(output_w) + hi,
                                                       (static_cast<long long>(width) + sw - 1) / sw);
    if (path != 2 && path != 4 && sw >= 1 && sw <= 4 && dilation_w == 1 && dmax >= 0 && taps >= 2 && taps <= 8 &&
        static_cast<long long>(output_w) <= wv && lo + hi <= 16 && !(sw > 1 && path == 5) &&
        static_cast<long long>(batches) * output_h * wv < INT_MAX - 4096) {
        // fp32 with K' = C*KH*sw > 512 sums K-chunks in a float[N][128] shared array: N <= 192 then
        const bool chunked = q.es == 4 && cg * static_cast<long long>(kernel_h) * sw > 512;
        const int cpt_max = static_cast<int>(((chunked ? 192 : 256) / taps) / 16 * 16);
        const int n_tiles = static_cast<int>((ng + cpt_max - 1) / cpt_max);
        int cpt = static_cast<int>(((ng + n_tiles - 1) / n_tiles + 15) / 16 * 16);
        if (cpt > cpt_max) cpt = cpt_max;
        const int forced_bn = g_force_bn.load() & 0xffff;  // experiments: tile width -> channels per tile
        if (forced_bn >= 16 * taps && forced_bn / taps / 16 * 16 <= cpt_max) cpt = static_cast<int>(forced_bn / taps / 16 * 16);
        Problem r = q;
        r.rc_kw = static_cast<int>(taps);
        r.rc_cpt = cpt;
        r.rc_lo = static_cast<int>(lo);
        r.rc_T = 32 - static_cast<int>(lo + hi);
        // 16-bit results of large planes leave as TMA stores: tiles are then aligned to images (a
        // tile is one contiguous range of pixels of one image) and start on 16-byte boundaries
        // (even rc_T). Needs every position to be an output (wv == OW), planes of a 16-byte
        // multiple, channel blocks of 16 that stay inside their group, and a plane large enough
        // that the partly filled last tile of an image is a small loss.
        {
            const int t_even = r.rc_T & ~1;
            const long long ohw = static_cast<long long>(output_h) * wv;
            // (measured: a gain for the strided row form - the 7x7 stride-2 stem, 1183 -> 1102 us -
            // and a small loss for stride 1, where the partly filled last tile of every image
            // costs more than the stores save; measurement bit 128 << 16 forces it on for stride 1)
            const bool want = sw > 1 || ((g_force_generic.load() >> 16) & 128);
            if (want && q.es == 2 && wv == static_cast<long long>(output_w) && (P * 2) % 16 == 0 && t_even >= 16 &&
                ohw >= 4ll * 4 * t_even && (group == 1 || ng % 16 == 0) &&
                (reinterpret_cast<uintptr_t>(y) & 15u) == 0) {
                r.rc_T = t_even;
                r.rc_tpi = static_cast<int>((ohw + 4 * t_even - 1) / (4 * t_even));
            }
        }
        r.rc_sw = static_cast<int>(sw);
        r.rc_wv = static_cast<int>(wv);
        r.rc_dmin = static_cast<int>(dmin);
        r.M = static_cast<long long>(batches) * output_h * wv;  // positions (img, oh, w')
        r.K = cg * static_cast<long long>(kernel_h) * sw;         // (kh, column phase, c)
        r.a.im2col = 1;
        DeviceState* st = nullptr;
        int rc = ensure_device(&st);
        if (rc != kSuccess) return rc;
        rc = launch_ts(*st, r, static_cast<cudaStream_t>(stream));
        if (rc != kNotImplemented) return rc;
    }
    // fp32 with a k table that would not fit (K = C*KH*KW > 12288, not row form, not 1x1): the
    // loader-warp fallback accumulates all of K in one tensor-core accumulator, whose truncation
    // error grows with K beyond the fp32 tolerance. Split the channels into ranges that fit the
    // table instead and accumulate the ranges through beta = 1 (bias and residual enter with
    // the first range, the ReLU leaves with the last).
    const long long khw = static_cast<long long>(kernel_h) * kernel_w;
    const bool affine_1x1 = kernel_h == 1 && kernel_w == 1 && pad_top == 0 && pad_left == 0 &&
                            (output_h - 1) * stride_h < height && (output_w - 1) * stride_w < width &&
                            !(g_force_generic.load() & 0x2000);  // needs no k table: one launch serves any K
    if (q.es == 4 && K > 12288 && khw <= 12288 && path != 2 && !affine_1x1) {
        DeviceState* st = nullptr;
        int rc = ensure_device(&st);
        if (rc != kSuccess) return rc;
        const long long cpc = 12288 / khw;  // channels per range
        for (long long c0 = 0; c0 < cg; c0 += cpc) {
            const long long cc = std::min<long long>(cpc, cg - c0);
            Problem r = q;
            r.K = cc * khw;
            r.a.base = q.a.base + c0 * static_cast<long long>(height) * width * q.es;
            r.b.base = q.b.base + c0 * khw * q.es;
            if (c0 > 0) {
                r.beta = 1.f;
                r.bias = nullptr;
                r.resid = nullptr;
            }
            r.relu = (c0 + cc >= cg) ? q.relu : 0;
            rc = launch_ts(*st, r, static_cast<cudaStream_t>(stream));
            if (rc != kSuccess) return rc == kNotImplemented ? launch(q, static_cast<cudaStream_t>(stream)) : rc;
        }
        return kSuccess;
    }
    return launch(q, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
// Level-3 routines on the GEMM main loop: symm, syrk, trmm, trsm
// (gpgpu/include/gblas.h:506-586). Scheme as in level3.cuh.
// ---------------------------------------------------------------------------------------------

size_t dlf_b200_level3_workspace_bytes(int routine, int dtype, size_t m, size_t n) {
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es)) return 0;
    switch (routine) {
        case DLF_B200_SYMM: { const size_t ka = m > n ? m : n; return ka * ka * es + 512; }           // the expanded A
        case DLF_B200_SYRK: return n * n * es + 512;                                                 // alpha*op(A)*op(A)^T
        case DLF_B200_TRMM: { const size_t ka = m > n ? m : n; return ka * ka * es + m * n * es + 1024; }  // expanded A + copy of B
        case DLF_B200_TRSM: return 0;
        default: return 0;
    }
}

int dlf_b200_symm(int dtype, int layout, int side, int triangle, size_t m, size_t n, const void* alpha,
                  const void* a, size_t a_ld, const void* b, size_t b_ld, const void* beta, void* c, size_t c_ld,
                  void* workspace, size_t workspace_bytes, void* stream) {
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es)) return kNotImplemented;
    if (layout != DLF_B200_ROW_MAJOR && layout != DLF_B200_COL_MAJOR) return kInvalidValue;
    if ((side != kLeft && side != kRight) || (triangle != kUpper && triangle != kLower)) return kInvalidValue;
    if (m == 0 || n == 0) return kInvalidDimension;
    const size_t ka = side == kLeft ? m : n;  // order of A
    const bool row = layout == DLF_B200_ROW_MAJOR;
    if (a_ld < ka) return kInvalidLeadDimA;
    if (b_ld < (row ? n : m)) return kInvalidLeadDimB;
    if (c_ld < (row ? n : m)) return kInvalidLeadDimC;
    if (a == nullptr) return kInvalidMatrixA;
    if (b == nullptr) return kInvalidMatrixB;
    if (c == nullptr) return kInvalidMatrixC;
    if (alpha == nullptr || beta == nullptr) return kInvalidValue;
    // column-major: C^T (n x m, row-major) = B^T S (Left) resp. S B^T (Right), and the stored
    // triangle of A^T is the other one
    if (!row) {
        side = side == kLeft ? kRight : kLeft;
        triangle = triangle == kUpper ? kLower : kUpper;
        const size_t t = m;
        m = n;
        n = t;
    }
    const size_t need = ka * ka * es;
    char* full = align256(workspace);
    if (workspace == nullptr || workspace_bytes < need + static_cast<size_t>(full - static_cast<char*>(workspace)))
        return kInsufficientMemoryTemp;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamDevice sd(s);
    if (sd.rc != kSuccess) return sd.rc;
    int rc = l3_expand_any(fmt, full, a, a_ld, ka, true, triangle == kUpper, false, s);
    if (rc != kSuccess) return rc;
    const float al = scalar_to_float(fmt, alpha), be = scalar_to_float(fmt, beta);
    if (side == kLeft)
        return rm_gemm(fmt, DLF_B200_NO_TRANS, DLF_B200_NO_TRANS, m, n, m, al, full, m, b, b_ld, be, c, c_ld, stream);
    return rm_gemm(fmt, DLF_B200_NO_TRANS, DLF_B200_NO_TRANS, m, n, n, al, b, b_ld, full, n, be, c, c_ld, stream);
}

int dlf_b200_syrk(int dtype, int layout, int triangle, int a_transpose, size_t n, size_t k, const void* alpha,
                  const void* a, size_t a_ld, const void* beta, void* c, size_t c_ld, void* workspace,
                  size_t workspace_bytes, void* stream) {
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es)) return kNotImplemented;
    if (layout != DLF_B200_ROW_MAJOR && layout != DLF_B200_COL_MAJOR) return kInvalidValue;
    if (triangle != kUpper && triangle != kLower) return kInvalidValue;
    if (a_transpose < DLF_B200_NO_TRANS || a_transpose > DLF_B200_CONJ_TRANS) return kInvalidValue;
    if (n == 0 || k == 0) return kInvalidDimension;
    const bool row = layout == DLF_B200_ROW_MAJOR;
    bool trans = a_transpose != DLF_B200_NO_TRANS;
    // column-major: the stored A is the row-major transpose, C^T = C
    if (!row) {
        trans = !trans;
        triangle = triangle == kUpper ? kLower : kUpper;
    }
    if (a_ld < (trans ? n : k)) return kInvalidLeadDimA;
    if (c_ld < n) return kInvalidLeadDimC;
    if (a == nullptr) return kInvalidMatrixA;
    if (c == nullptr) return kInvalidMatrixC;
    if (alpha == nullptr || beta == nullptr) return kInvalidValue;
    const size_t need = n * n * es;
    char* prod = align256(workspace);
    if (workspace == nullptr || workspace_bytes < need + static_cast<size_t>(prod - static_cast<char*>(workspace)))
        return kInsufficientMemoryTemp;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamDevice sd(s);
    if (sd.rc != kSuccess) return sd.rc;
    const float al = scalar_to_float(fmt, alpha), be = scalar_to_float(fmt, beta);
    const int ta = trans ? DLF_B200_TRANS : DLF_B200_NO_TRANS, tb = trans ? DLF_B200_NO_TRANS : DLF_B200_TRANS;
    int rc = rm_gemm(fmt, ta, tb, n, n, k, al, a, a_ld, a, a_ld, 0.0f, prod, n, stream);
    if (rc != kSuccess) return rc;
    const unsigned grid = l3_grid(static_cast<long long>(n) * n);
    const int up = triangle == kUpper ? 1 : 0;
    if (fmt == FMT_F32)
        l3_triangle_merge_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(c), static_cast<long long>(c_ld), reinterpret_cast<const float*>(prod), static_cast<int>(n), up, be);
    else if (fmt == FMT_F16)
        l3_triangle_merge_kernel<__half><<<grid, 256, 0, s>>>(static_cast<__half*>(c), static_cast<long long>(c_ld), reinterpret_cast<const __half*>(prod), static_cast<int>(n), up, be);
    else
        l3_triangle_merge_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(c), static_cast<long long>(c_ld), reinterpret_cast<const __nv_bfloat16*>(prod), static_cast<int>(n), up, be);
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}


int dlf_b200_trmm(int dtype, int layout, int side, int triangle, int a_transpose, int diagonal, size_t m, size_t n,
                  const void* alpha, const void* a, size_t a_ld, void* b, size_t b_ld, void* workspace,
                  size_t workspace_bytes, void* stream) {
    int fmt = 0, es = 0;
    int rc = tri_args(dtype, fmt, es, layout, side, triangle, a_transpose, diagonal, m, n, alpha, a, a_ld, b, b_ld);
    if (rc != kSuccess) return rc;
    const size_t ka = side == kLeft ? m : n;
    char* full = align256(workspace);
    char* copy = align256(full + ka * ka * es);
    const size_t need = static_cast<size_t>(copy - static_cast<char*>(workspace)) + m * n * es;
    if (workspace == nullptr || workspace_bytes < need) return kInsufficientMemoryTemp;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamDevice sd(s);
    if (sd.rc != kSuccess) return sd.rc;
    rc = l3_expand_any(fmt, full, a, a_ld, ka, false, triangle == kUpper, diagonal == kUnit, s);
    if (rc != kSuccess) return rc;
    // the product reads all of B while it writes B: work from a copy
    CUDA_TRY(cudaMemcpy2DAsync(copy, n * es, b, b_ld * es, n * es, m, cudaMemcpyDeviceToDevice, s));
    const float al = scalar_to_float(fmt, alpha);
    const int ta = a_transpose == DLF_B200_NO_TRANS ? DLF_B200_NO_TRANS : DLF_B200_TRANS;
    if (side == kLeft)
        return rm_gemm(fmt, ta, DLF_B200_NO_TRANS, m, n, m, al, full, m, copy, n, 0.0f, b, b_ld, stream);
    return rm_gemm(fmt, DLF_B200_NO_TRANS, ta, m, n, n, al, copy, n, full, n, 0.0f, b, b_ld, stream);
}

int dlf_b200_trsm(int dtype, int layout, int side, int triangle, int a_transpose, int diagonal, size_t m, size_t n,
                  const void* alpha, const void* a, size_t a_ld, void* b, size_t b_ld, void* workspace,
                  size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    int fmt = 0, es = 0;
    int rc = tri_args(dtype, fmt, es, layout, side, triangle, a_transpose, diagonal, m, n, alpha, a, a_ld, b, b_ld);
    if (rc != kSuccess) return rc;
    if (m > INT_MAX || n > INT_MAX) return kInvalidDimension;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamDevice sd(s);
    if (sd.rc != kSuccess) return sd.rc;
    clear_stale_error();
    const bool trans = a_transpose != DLF_B200_NO_TRANS;
    const bool lower = triangle == kLower;
    const bool op_lower = lower != trans;
    const float al = scalar_to_float(fmt, alpha);
    const char* A = static_cast<const char*>(a);
    char* B = static_cast<char*>(b);
    auto a_at = [&](size_t r, size_t c) { return A + (r * a_ld + c) * es; };
    auto b_at = [&](size_t r, size_t c) { return B + (r * b_ld + c) * es; };
    if (al != 1.0f) {
        const unsigned grid = l3_grid(static_cast<long long>(m) * n);
        if (fmt == FMT_F32) l3_scale_kernel<float><<<grid, 256, 0, s>>>(reinterpret_cast<float*>(B), static_cast<long long>(b_ld), static_cast<int>(m), static_cast<int>(n), al);
        else if (fmt == FMT_F16) l3_scale_kernel<__half><<<grid, 256, 0, s>>>(reinterpret_cast<__half*>(B), static_cast<long long>(b_ld), static_cast<int>(m), static_cast<int>(n), al);
        else l3_scale_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(B), static_cast<long long>(b_ld), static_cast<int>(m), static_cast<int>(n), al);
        g_launches.fetch_add(1);
        CUDA_TRY(cudaGetLastError());
    }
    auto diag_solve = [&](size_t d0, size_t nb, char* bblk, size_t nsys) -> int {
        const unsigned grid = static_cast<unsigned>((nsys + kTrsmThreads - 1) / kTrsmThreads);
        const int rs = side == kRight ? 1 : 0;
        if (fmt == FMT_F32)
            l3_trsm_diag_kernel<float><<<grid, kTrsmThreads, 0, s>>>(reinterpret_cast<const float*>(a_at(d0, d0)), static_cast<long long>(a_ld), trans, lower, diagonal == kUnit, rs, static_cast<int>(nb), reinterpret_cast<float*>(bblk), static_cast<long long>(b_ld), static_cast<int>(nsys));
        else if (fmt == FMT_F16)
            l3_trsm_diag_kernel<__half><<<grid, kTrsmThreads, 0, s>>>(reinterpret_cast<const __half*>(a_at(d0, d0)), static_cast<long long>(a_ld), trans, lower, diagonal == kUnit, rs, static_cast<int>(nb), reinterpret_cast<__half*>(bblk), static_cast<long long>(b_ld), static_cast<int>(nsys));
        else
            l3_trsm_diag_kernel<__nv_bfloat16><<<grid, kTrsmThreads, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(a_at(d0, d0)), static_cast<long long>(a_ld), trans, lower, diagonal == kUnit, rs, static_cast<int>(nb), reinterpret_cast<__nv_bfloat16*>(bblk), static_cast<long long>(b_ld), static_cast<int>(nsys));
        g_launches.fetch_add(1);
        CUDA_TRY(cudaGetLastError());
        return kSuccess;
    };
    const int N = DLF_B200_NO_TRANS, T = DLF_B200_TRANS;
    if (side == kLeft) {
        // op(T) X = B: row blocks of B, top to bottom when op(T) is lower, else bottom to top;
        // every block first loses the contribution of the rows already solved (a GEMM)
        const size_t blocks = (m + kTrsmBlock - 1) / kTrsmBlock;
        for (size_t bi = 0; bi < blocks; ++bi) {
            const size_t blk = op_lower ? bi : blocks - 1 - bi;
            const size_t i0 = blk * kTrsmBlock, i1 = std::min<size_t>(m, i0 + kTrsmBlock), ib = i1 - i0;
            if (op_lower && i0 > 0) {
                rc = trans ? rm_gemm(fmt, T, N, ib, n, i0, -1.0f, a_at(0, i0), a_ld, b_at(0, 0), b_ld, 1.0f, b_at(i0, 0), b_ld, stream)
                           : rm_gemm(fmt, N, N, ib, n, i0, -1.0f, a_at(i0, 0), a_ld, b_at(0, 0), b_ld, 1.0f, b_at(i0, 0), b_ld, stream);
            } else if (!op_lower && i1 < m) {
                rc = trans ? rm_gemm(fmt, T, N, ib, n, m - i1, -1.0f, a_at(i1, i0), a_ld, b_at(i1, 0), b_ld, 1.0f, b_at(i0, 0), b_ld, stream)
                           : rm_gemm(fmt, N, N, ib, n, m - i1, -1.0f, a_at(i0, i1), a_ld, b_at(i1, 0), b_ld, 1.0f, b_at(i0, 0), b_ld, stream);
            }
            if (rc != kSuccess) return rc;
            rc = diag_solve(i0, ib, b_at(i0, 0), n);
            if (rc != kSuccess) return rc;
        }
    } else {
        // X op(T) = B: column blocks of B, left to right when op(T) is upper, else right to left
        const size_t blocks = (n + kTrsmBlock - 1) / kTrsmBlock;
        for (size_t bi = 0; bi < blocks; ++bi) {
            const size_t blk = op_lower ? blocks - 1 - bi : bi;
            const size_t j0 = blk * kTrsmBlock, j1 = std::min<size_t>(n, j0 + kTrsmBlock), jb = j1 - j0;
            if (!op_lower && j0 > 0) {
                rc = trans ? rm_gemm(fmt, N, T, m, jb, j0, -1.0f, b_at(0, 0), b_ld, a_at(j0, 0), a_ld, 1.0f, b_at(0, j0), b_ld, stream)
                           : rm_gemm(fmt, N, N, m, jb, j0, -1.0f, b_at(0, 0), b_ld, a_at(0, j0), a_ld, 1.0f, b_at(0, j0), b_ld, stream);
            } else if (op_lower && j1 < n) {
                rc = trans ? rm_gemm(fmt, N, T, m, jb, n - j1, -1.0f, b_at(0, j1), b_ld, a_at(j0, j1), a_ld, 1.0f, b_at(0, j0), b_ld, stream)
                           : rm_gemm(fmt, N, N, m, jb, n - j1, -1.0f, b_at(0, j1), b_ld, a_at(j1, j0), a_ld, 1.0f, b_at(0, j0), b_ld, stream);
            }
            if (rc != kSuccess) return rc;
            rc = diag_solve(j0, jb, b_at(0, j0), m);
            if (rc != kSuccess) return rc;
        }
    }
    return kSuccess;
}

int dlf_b200_conv2d(int dtype, size_t batches, size_t channels, size_t height, size_t width,
                    size_t output_h, size_t output_w, size_t num_kernels, size_t group,
                    size_t kernel_h, size_t kernel_w, size_t pad_top, size_t pad_left,
                    size_t pad_bottom, size_t pad_right, size_t stride_h, size_t stride_w,
                    size_t dilation_h, size_t dilation_w, const void* x, const void* w,
                    const void* bias, void* y, void* workspace, size_t workspace_bytes,
                    void* stream) {
    return dlf_b200_conv2d_fused(dtype, batches, channels, height, width, output_h, output_w, num_kernels,
                                 group, kernel_h, kernel_w, pad_top, pad_left, pad_bottom, pad_right,
                                 stride_h, stride_w, dilation_h, dilation_w, x, w, bias, nullptr,
                                 DLF_B200_ACT_NONE, y, workspace, workspace_bytes, stream);
}

namespace {

int launch_pool(int dtype, int mode, int count_include_pad, size_t batches, size_t channels, size_t height,
                size_t width, size_t output_h, size_t output_w, size_t kernel_h, size_t kernel_w, size_t pad_top,
                size_t pad_left, size_t stride_h, size_t stride_w, size_t dilation_h, size_t dilation_w,
                const void* x, void* y, void* stream) {
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es)) return kNotImplemented;
    if (batches == 0 || channels == 0 || height == 0 || width == 0 || output_h == 0 || output_w == 0 ||
        kernel_h == 0 || kernel_w == 0 || stride_h == 0 || stride_w == 0 || dilation_h == 0 || dilation_w == 0)
        return kInvalidDimension;
    if (x == nullptr || y == nullptr) return kInvalidValue;
    const size_t lim = 1u << 30;
    if (height >= lim || width >= lim || output_h >= lim || output_w >= lim || kernel_h >= lim || kernel_w >= lim ||
        pad_top >= lim || pad_left >= lim || stride_h >= lim || stride_w >= lim || dilation_h >= lim ||
        dilation_w >= lim || static_cast<long long>(height) * width >= INT_MAX ||
        static_cast<long long>(output_h) * output_w >= INT_MAX)
        return kInvalidDimension;
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;
    DeviceState* st = nullptr;
    int rc = ensure_device(&st);
    if (rc != kSuccess) return rc;
    PoolParams p{};
    p.planes = static_cast<long long>(batches) * static_cast<long long>(channels);
    p.H = static_cast<int>(height);
    p.W = static_cast<int>(width);
    p.OH = static_cast<int>(output_h);
    p.OW = static_cast<int>(output_w);
    p.KH = static_cast<int>(kernel_h);
    p.KW = static_cast<int>(kernel_w);
    p.pad_t = static_cast<int>(pad_top);
    p.pad_l = static_cast<int>(pad_left);
    p.sh = static_cast<int>(stride_h);
    p.sw = static_cast<int>(stride_w);
    p.dh = static_cast<int>(dilation_h);
    p.dw = static_cast<int>(dilation_w);
    p.mode = mode;
    p.ablate = (g_force_generic.load() >> 26) & 3;
    p.count_include_pad = count_include_pad;
    p.x = static_cast<const char*>(x);
    p.y = static_cast<char*>(y);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    clear_stale_error();
    // the whole plane as one unpadded, undilated window: global pooling, one warp per plane
    const bool whole_plane = output_h == 1 && output_w == 1 && kernel_h == height && kernel_w == width &&
                             pad_top == 0 && pad_left == 0 && dilation_h == 1 && dilation_w == 1 &&
                             !((g_force_generic.load() >> 16) & 0x100);
    constexpr int kPoolSmem = 48 * 1024;  // static limit: no opt-in needed
    const long long plane_bytes = static_cast<long long>(height) * width * es;
    if (whole_plane && plane_bytes * 8 + 16 <= kPoolSmem) {
        // small planes: 256 / group planes per block staged through shared memory (+16 bytes of
        // alignment slack, counted against the 48 KB limit)
        int group = 1;
        while ((256 / group) * plane_bytes + 16 > kPoolSmem) group *= 2;
        p.group = group;
        const long long ppb = 256 / group;
        const long long blocks = (p.planes + ppb - 1) / ppb;
        const unsigned grid = static_cast<unsigned>(std::min<long long>(blocks, static_cast<long long>(st->num_sms) * 8));
        const size_t smem = static_cast<size_t>(ppb * plane_bytes + 16);
        if (fmt == FMT_F32) pool_planes_kernel<float><<<grid, 256, smem, s>>>(p);
        else if (fmt == FMT_F16) pool_planes_kernel<__half><<<grid, 256, smem, s>>>(p);
        else pool_planes_kernel<__nv_bfloat16><<<grid, 256, smem, s>>>(p);
    } else if (whole_plane) {
        const long long blocks = (p.planes + 7) / 8;  // eight warps per block
        const unsigned grid = static_cast<unsigned>(std::min<long long>(blocks, static_cast<long long>(st->num_sms) * 16));
        if (fmt == FMT_F32) pool_plane_kernel<float><<<grid, 256, 0, s>>>(p);
        else if (fmt == FMT_F16) pool_plane_kernel<__half><<<grid, 256, 0, s>>>(p);
        else pool_plane_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(p);
    } else {
        // rows of the window of one output row, and how many output rows a block can take
        const long long row_bytes = static_cast<long long>(width) * es;
        const long long win_rows = static_cast<long long>(kernel_h - 1) * dilation_h + 1;
        long long toh = 0;
        if (win_rows * row_bytes <= kPoolSmem && !((g_force_generic.load() >> 16) & 0x100)) {
            toh = (kPoolSmem / row_bytes - win_rows) / static_cast<long long>(stride_h) + 1;
            // about 24 KB per block: eight blocks per SM keep ~200 KB of loads in flight
            toh = std::min<long long>(toh, std::max<long long>(1, (24 * 1024 / row_bytes - win_rows) / static_cast<long long>(stride_h) + 1));
            toh = std::min<long long>(toh, static_cast<long long>(output_h));
        }
        const bool strip = mode == 0 && es == 2 && kernel_h == 3 && kernel_w == 3 && stride_h == 2 && stride_w == 2 &&
                           dilation_h == 1 && dilation_w == 1 && pad_left == 1 && width % 8 == 0 &&
                           output_w % 8 == 0 && output_w * 2 <= width + 1 &&
                           (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0 &&
                           !((g_force_generic.load() >> 16) & 0x100);
        if (strip) {
            const long long strips = p.planes * output_h * (static_cast<long long>(output_w) / 8);
            const unsigned grid = static_cast<unsigned>(
                std::min<long long>((strips + 255) / 256, static_cast<long long>(st->num_sms) * 32));
            if (fmt == FMT_F16) maxpool3s2_strip_kernel<__half, __half2><<<grid, 256, 0, s>>>(p, 0xFBFFFBFFu);
            else maxpool3s2_strip_kernel<__nv_bfloat16, __nv_bfloat162><<<grid, 256, 0, s>>>(p, 0xFF7FFF7Fu);
        } else if (toh >= 1) {
            p.toh = static_cast<int>(toh);
            p.ih_rows = static_cast<int>((toh - 1) * stride_h + win_rows);
            const long long blocks = p.planes * ((static_cast<long long>(output_h) + toh - 1) / toh);
            const unsigned grid = static_cast<unsigned>(std::min<long long>(blocks, static_cast<long long>(st->num_sms) * 32));
            const size_t smem = static_cast<size_t>(p.ih_rows * row_bytes);
            const int k = (kernel_h == kernel_w && (kernel_h == 2 || kernel_h == 3) && dilation_h == 1 && dilation_w == 1)
                              ? static_cast<int>(kernel_h) : 0;
#define DLF_POOL_ROWS(T)                                                              \
    do {                                                                              \
        if (k == 3) pool2d_rows_kernel<T, 3><<<grid, 256, smem, s>>>(p);              \
        else if (k == 2) pool2d_rows_kernel<T, 2><<<grid, 256, smem, s>>>(p);         \
        else pool2d_rows_kernel<T, 0><<<grid, 256, smem, s>>>(p);                     \
    } while (0)
            if (fmt == FMT_F32) DLF_POOL_ROWS(float);
            else if (fmt == FMT_F16) DLF_POOL_ROWS(__half);
            else DLF_POOL_ROWS(__nv_bfloat16);
#undef DLF_POOL_ROWS
        } else {
            const long long total = p.planes * output_h * output_w;
            const long long blocks = (total + 255) / 256;
            const unsigned grid = static_cast<unsigned>(std::min<long long>(blocks, static_cast<long long>(st->num_sms) * 32));
            if (fmt == FMT_F32) pool2d_kernel<float><<<grid, 256, 0, s>>>(p);
            else if (fmt == FMT_F16) pool2d_kernel<__half><<<grid, 256, 0, s>>>(p);
            else pool2d_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(p);
        }
    }
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}

}  // namespace

size_t dlf_b200_nhwc_filter_elems(size_t channels, size_t num_kernels, size_t kernel_h, size_t kernel_w) {
    return num_kernels * kernel_h * kernel_w * ((channels + 63) / 64 * 64);
}

int dlf_b200_pack_filters_nhwc(int dtype, size_t channels, size_t num_kernels, size_t kernel_h, size_t kernel_w,
                               const void* w, void* w_packed, void* stream) {
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es) || es != 2) return kNotImplemented;
    if (channels == 0 || num_kernels == 0 || kernel_h == 0 || kernel_w == 0) return kInvalidDimension;
    if (w == nullptr) return kInvalidMatrixB;
    if (w_packed == nullptr || (reinterpret_cast<uintptr_t>(w_packed) & 15u)) return kInvalidMatrixC;
    const long long taps = static_cast<long long>(kernel_h) * kernel_w;
    const long long ck = (static_cast<long long>(channels) + 63) / 64 * 64;
    if (taps * ck >= INT_MAX - 512 || static_cast<long long>(num_kernels) * ck >= (1ll << 40)) return kInvalidDimension;
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;
    DeviceState* st = nullptr;
    int rc = ensure_device(&st);
    if (rc != kSuccess) return rc;
    clear_stale_error();
    const long long total = static_cast<long long>(num_kernels) * ck;
    const unsigned blocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 8ll * st->num_sms));
    cl_pack_filters_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(w), static_cast<uint16_t*>(w_packed), static_cast<int>(num_kernels),
        static_cast<int>(channels), static_cast<int>(taps), static_cast<int>(ck));
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}

int dlf_b200_nchw_to_nhwc(int dtype, size_t batches, size_t channels, size_t height, size_t width, const void* x,
                          void* y, void* stream) {
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es) || es != 2) return kNotImplemented;
    if (batches == 0 || channels == 0 || height == 0 || width == 0) return kInvalidDimension;
    if (x == nullptr) return kInvalidMatrixA;
    if (y == nullptr || (reinterpret_cast<uintptr_t>(y) & 15u)) return kInvalidMatrixC;
    const long long plane = static_cast<long long>(height) * width;
    const long long cp = (static_cast<long long>(channels) + 7) / 8 * 8;
    if (plane >= INT_MAX || batches >= 65536 || cp >= 65536ll * 64) return kInvalidDimension;
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;
    DeviceState* st = nullptr;
    int rc = ensure_device(&st);
    if (rc != kSuccess) return rc;
    clear_stale_error();
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    dim3 grid(static_cast<unsigned>((plane + kClTile - 1) / kClTile), static_cast<unsigned>((cp + kClTile - 1) / kClTile),
              static_cast<unsigned>(batches));
    const uint16_t* xs = static_cast<const uint16_t*>(x);
    uint16_t* xp = static_cast<uint16_t*>(y);
    const long long total = static_cast<long long>(batches) * channels * plane;
    const uintptr_t xa = reinterpret_cast<uintptr_t>(x);
    const int ci = static_cast<int>(channels), cpi = static_cast<int>(cp), pl = static_cast<int>(plane);
    if (plane % 8 == 0 && xa % 16 == 0)
        cl_pack_activations_kernel<CL_VEC8><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, pl, 1, pl, 1, 1, cpi, total);
    else if (plane % 4 == 0 && xa % 8 == 0)
        cl_pack_activations_kernel<CL_VEC4><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, pl, 1, pl, 1, 1, cpi, total);
    else if (plane % 2 == 0 && xa % 4 == 0)
        cl_pack_activations_kernel<CL_VEC2><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, pl, 1, pl, 1, 1, cpi, total);
    else
        cl_pack_activations_kernel<CL_FUNNEL><<<grid, 256, 0, cs>>>(xs, xp, ci, plane, pl, 1, pl, 1, 1, cpi, total);
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}

int dlf_b200_conv2d_nhwc(int dtype, size_t batches, size_t channels, size_t height, size_t width, size_t output_h,
                         size_t output_w, size_t num_kernels, size_t kernel_h, size_t kernel_w, size_t pad_top,
                         size_t pad_left, size_t pad_bottom, size_t pad_right, size_t stride_h, size_t stride_w,
                         size_t dilation_h, size_t dilation_w, const void* x, const void* w_packed, const void* bias,
                         const void* residual, int activation, void* y, int y_layout, void* stream) {
    (void)pad_bottom;
    (void)pad_right;
    Problem q;
    if (activation != DLF_B200_ACT_NONE && activation != DLF_B200_ACT_RELU) return kInvalidValue;
    if (y_layout != DLF_B200_LAYOUT_NHWC && y_layout != DLF_B200_LAYOUT_NCHW) return kInvalidValue;
    if (!dtype_info(dtype, q.fmt, q.es)) return kNotImplemented;
    if (q.es != 2) return kNotImplemented;
    if (batches == 0 || channels == 0 || height == 0 || width == 0 || output_h == 0 || output_w == 0 ||
        num_kernels == 0 || kernel_h == 0 || kernel_w == 0)
        return kInvalidDimension;
    if (stride_h == 0 || stride_w == 0 || dilation_h == 0 || dilation_w == 0) return kInvalidValue;
    if (x == nullptr) return kInvalidMatrixA;
    if (w_packed == nullptr) return kInvalidMatrixB;
    if (y == nullptr) return kInvalidMatrixC;
    const size_t lim = 1u << 20;
    if (height >= lim || width >= lim || kernel_h > 16 || kernel_w > 16 || pad_top >= 128 || pad_left >= 128 ||
        stride_h > 8 || stride_w > 8 || dilation_h * (kernel_h - 1) >= 256 || dilation_w * (kernel_w - 1) >= 256 ||
        batches >= 65536)
        return kNotImplemented;
    // the tensor-map unit wants 16-byte pixels and rows; the stores 16-byte rows of D
    if (channels % 8 != 0 || (y_layout == DLF_B200_LAYOUT_NHWC && num_kernels % 8 != 0)) return kNotImplemented;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_packed) | reinterpret_cast<uintptr_t>(y) |
         reinterpret_cast<uintptr_t>(residual)) & 15u)
        return kNotImplemented;
    const long long P = static_cast<long long>(output_h) * output_w;
    const long long taps = static_cast<long long>(kernel_h) * kernel_w;
    const long long ck = (static_cast<long long>(channels) + 63) / 64 * 64;
    if (P >= INT_MAX || static_cast<long long>(batches) * P >= INT_MAX - 512 || taps * ck >= INT_MAX - 512)
        return kInvalidDimension;
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;
    DeviceState* st = nullptr;
    int rc = ensure_device(&st);
    if (rc != kSuccess) return rc;
    if (st->encode_im2col == nullptr) return kNotImplemented;
    clear_stale_error();
    q.resid = static_cast<const char*>(residual);
    q.relu = activation == DLF_B200_ACT_RELU ? 1 : 0;
    q.alpha = 1.f;
    q.beta = 0.f;
    q.bias = static_cast<const char*>(bias);
    q.bias_stride = 0;
    q.batch = 1;
    q.M = static_cast<long long>(batches) * P;  // output pixels of all images
    q.N = static_cast<long long>(num_kernels);
    q.K = taps * ck;
    q.g.H = static_cast<int>(height);
    q.g.W = static_cast<int>(width);
    q.g.OH = static_cast<int>(output_h);
    q.g.OW = static_cast<int>(output_w);
    q.g.KH = static_cast<int>(kernel_h);
    q.g.KW = static_cast<int>(kernel_w);
    q.g.pad_t = static_cast<int>(pad_top);
    q.g.pad_l = static_cast<int>(pad_left);
    q.g.sh = static_cast<int>(stride_h);
    q.g.sw = static_cast<int>(stride_w);
    q.g.dh = static_cast<int>(dilation_h);
    q.g.dw = static_cast<int>(dilation_w);
    q.g.P = static_cast<int>(P);
    q.g.img_stride = static_cast<long long>(channels) * height * width;
    q.g.out_img_stride = static_cast<long long>(num_kernels) * P;
    // operand A: filter windows of the channels-last activations, fetched by im2col-mode loads (one
    // load = 128 windows x 64 channels of one tap); operand B: the packed filter bank (Cout, tap, Ck)
    q.a.base = static_cast<const char*>(x);
    q.a.im2col = 0;
    q.a.k_major = 1;
    q.a.ld = static_cast<long long>(channels);
    q.a.batch_stride = 0;
    q.b.base = static_cast<const char*>(w_packed);
    q.b.k_major = 1;
    q.b.ld = q.K;
    q.b.batch_stride = 0;
    q.d = static_cast<char*>(y);
    q.d_batch_stride = 0;
    q.a_cl = 1;
    q.cl_cblocks = static_cast<int>(ck / 64);
    q.cl_n = static_cast<long long>(batches);
    q.cl_h = static_cast<long long>(height);
    q.cl_w = static_cast<long long>(width);
    q.cl_cp = static_cast<long long>(channels);
    q.pack_ws = nullptr;
    q.pack_ws_bytes = 0;
    if (y_layout == DLF_B200_LAYOUT_NHWC) {
        q.ldd = static_cast<long long>(num_kernels);
        q.out_nchw = 5;
        // With 65 to 128 output channels and a filter larger than 1x1 the pixel-per-lane form runs UMMAs
        // of 128 columns and fetches the filter bank once per 128 pixels. With the filter bank as
        // operand A (lanes = output channels) a tile is 256 pixels wide: D[pixel][channel] is then the
        // plain column-major output of that product, written through the GEMM epilogue's boxes with
        // the bias taken per row. Measured at batch 256: 128 -> 128 3x3 at 28x28 77 -> 61 us; not for
        // 64 output channels, where half of the lanes idle (64 -> 64 3x3 at 56x56: 146 -> 156 us;
        // 256 -> 64 1x1: 81 -> 108 us), nor for 1x1 filters (512 -> 128 at 28x28: 48 -> 50 us).
        // Bit 28 of the tile-width word: never.
        if (num_kernels > 64 && num_kernels <= 128 && taps > 1 && !((g_force_bn.load() >> 16) & 4096)) {
            std::swap(q.a, q.b);
            q.M = static_cast<long long>(num_kernels);
            q.N = static_cast<long long>(batches) * P;
            q.cl_swap = 1;
            q.out_nchw = 0;
            q.bias_rows = 1;
        }
    } else {
        // NCHW output: the forms of the channels-last route of dlf_b200_conv2d_fused
        q.ldd = P;
        q.out_nchw = 1;
        if (P % 8 == 0 && P >= 32) {
            std::swap(q.a, q.b);
            q.M = static_cast<long long>(num_kernels);
            q.N = static_cast<long long>(batches) * P;
            q.cl_swap = 1;
            q.out_nchw = 3;
            q.out_vec = 8;
        } else {
            q.out_vec = P % 4 == 0 ? 4 : (P % 2 == 0 ? 2 : 1);
        }
    }
    return launch(q, static_cast<cudaStream_t>(stream), st);
}

int dlf_b200_pool_nhwc(int dtype, int average, int count_include_pad, size_t batches, size_t channels, size_t height,
                       size_t width, size_t output_h, size_t output_w, size_t kernel_h, size_t kernel_w, size_t pad_top,
                       size_t pad_left, size_t stride_h, size_t stride_w, const void* x, void* y, void* stream) {
    int fmt = 0, es = 0;
    if (!dtype_info(dtype, fmt, es) || es != 2) return kNotImplemented;
    if (batches == 0 || channels == 0 || height == 0 || width == 0 || output_h == 0 || output_w == 0 || kernel_h == 0 ||
        kernel_w == 0)
        return kInvalidDimension;
    if (stride_h == 0 || stride_w == 0) return kInvalidValue;
    if (x == nullptr) return kInvalidMatrixA;
    if (y == nullptr) return kInvalidMatrixC;
    if (channels % 8 != 0 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u)) return kNotImplemented;
    const size_t lim = 1u << 20;
    if (height >= lim || width >= lim || kernel_h >= lim || kernel_w >= lim || pad_top >= lim || pad_left >= lim ||
        stride_h >= lim || stride_w >= lim)
        return kInvalidDimension;
    const long long total = static_cast<long long>(batches) * output_h * output_w * (channels / 8);
    if (total >= (1ll << 40)) return kInvalidDimension;
    StreamDevice sd(static_cast<cudaStream_t>(stream));
    if (sd.rc != kSuccess) return sd.rc;
    DeviceState* st = nullptr;
    int rc = ensure_device(&st);
    if (rc != kSuccess) return rc;
    clear_stale_error();
    const unsigned blocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 32ll * st->num_sms));
    PoolNhwc g;
    g.C8 = static_cast<int>(channels / 8);
    g.H = static_cast<int>(height);
    g.W = static_cast<int>(width);
    g.OH = static_cast<int>(output_h);
    g.OW = static_cast<int>(output_w);
    g.KH = static_cast<int>(kernel_h);
    g.KW = static_cast<int>(kernel_w);
    g.pad_t = static_cast<int>(pad_top);
    g.pad_l = static_cast<int>(pad_left);
    g.sh = static_cast<int>(stride_h);
    g.sw = static_cast<int>(stride_w);
    g.average = average ? 1 : 0;
    g.count_include_pad = count_include_pad ? 1 : 0;
    g.total = total;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (fmt == FMT_F16)
        pool_nhwc_kernel<OUT_F16><<<blocks, 256, 0, cs>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y), g);
    else
        pool_nhwc_kernel<OUT_BF16><<<blocks, 256, 0, cs>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y), g);
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    return kSuccess;
}

int dlf_b200_maxpool(int dtype, size_t batches, size_t channels, size_t height, size_t width, size_t output_h,
                     size_t output_w, size_t kernel_h, size_t kernel_w, size_t pad_top, size_t pad_left,
                     size_t, size_t, size_t stride_h, size_t stride_w, size_t dilation_h, size_t dilation_w,
                     const void* x, void* y, void* stream) {
    return launch_pool(dtype, 0, 0, batches, channels, height, width, output_h, output_w, kernel_h, kernel_w,
                       pad_top, pad_left, stride_h, stride_w, dilation_h, dilation_w, x, y, stream);
}

int dlf_b200_avgpool(int dtype, size_t batches, size_t channels, size_t height, size_t width, size_t output_h,
                     size_t output_w, size_t kernel_h, size_t kernel_w, size_t pad_top, size_t pad_left,
                     size_t, size_t, size_t stride_h, size_t stride_w, size_t dilation_h, size_t dilation_w,
                     int count_include_pad, const void* x, void* y, void* stream) {
    return launch_pool(dtype, 1, count_include_pad ? 1 : 0, batches, channels, height, width, output_h, output_w,
                       kernel_h, kernel_w, pad_top, pad_left, stride_h, stride_w, dilation_h, dilation_w, x, y,
                       stream);
}

const char* dlf_b200_status_string(int status) {
    switch (status) {
        case kSuccess: return "kSuccess";
        case kInvalidValue: return "kInvalidValue";
        case kNotImplemented: return "kNotImplemented";
        case kInvalidMatrixA: return "kInvalidMatrixA";
        case kInvalidMatrixB: return "kInvalidMatrixB";
        case kInvalidMatrixC: return "kInvalidMatrixC";
        case kInvalidDimension: return "kInvalidDimension";
        case kInvalidLeadDimA: return "kInvalidLeadDimA";
        case kInvalidLeadDimB: return "kInvalidLeadDimB";
        case kInvalidLeadDimC: return "kInvalidLeadDimC";
        case kInsufficientMemoryTemp: return "kInsufficientMemoryTemp";
        case kInvalidBatchCount: return "kInvalidBatchCount";
        case kNoHalfPrecision: return "kNoHalfPrecision";
        case kUnexpectedError: return "kUnexpectedError";
        default: break;
    }
    if (status > 0) return cudaGetErrorName(static_cast<cudaError_t>(status));
    return "unknown status";
}

int dlf_b200_device_status(int* device_status) {
    // Reads (and clears) the status words of the current device that exist already; it sets
    // nothing up and allocates nothing, so it also works for a process that only ever uses
    // dlf_b200_gemm_batched_noalloc and has no device memory to spare.
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return kInvalidValue;
    int* words[2] = {nullptr, nullptr};
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (g_dev[dev].ready) words[0] = g_dev[dev].status;
        if (g_noalloc_dev[dev].ready) words[1] = g_noalloc_dev[dev].st.status;
    }
    int v = 0;
    if (words[0] != nullptr || words[1] != nullptr) CUDA_TRY(cudaDeviceSynchronize());
    for (int* w : words) {
        if (w == nullptr) continue;
        int x = 0;
        CUDA_TRY(cudaMemcpy(&x, w, sizeof(int), cudaMemcpyDeviceToHost));
        if (x != 0) CUDA_TRY(cudaMemset(w, 0, sizeof(int)));
        v |= x;
    }
    if (device_status) *device_status = v;
    return kSuccess;
}

#ifdef DLF_ROLE_CLOCKS
// measurement build only: reads (and clears) the role clock table of contraction.cuh
int dlf_b200_debug_role_clocks(unsigned long long* out16) {
    CUDA_TRY(cudaDeviceSynchronize());
    CUDA_TRY(cudaMemcpyFromSymbol(out16, g_role_clocks, 16 * sizeof(unsigned long long)));
    unsigned long long zero[16] = {};
    CUDA_TRY(cudaMemcpyToSymbol(g_role_clocks, zero, sizeof(zero)));
    return 0;
}
#endif

void dlf_b200_set_tuning(int force_bn, int force_generic_loader) {
    g_force_bn.store(force_bn);
    g_force_generic.store(force_generic_loader);
}

unsigned long long dlf_b200_launch_count(void) { return g_launches.load(); }

}  // extern "C"

/* dlf_b200.h - C ABI of the B200 (sm_100a) dense-contraction backend for dlf's gpgpu layer.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*), launches
 * asynchronously on that stream and returns an int:
 *     0                      success (gpgpu::blas::StatusCode::kSuccess)
 *     negative               a gpgpu::blas::StatusCode value (gpgpu/include/gblas.h:43-107)
 *     positive               a cudaError_t from the CUDA runtime
 * Nothing throws. The C++ shim in dlf_b200_gpgpu.hpp turns a non-zero return into the
 * exception the reference raises for the same mistake.
 *
 * Enumerations reuse the reference's integer values:
 *     layout     101 RowMajor, 102 ColMajor              (gblas.h:110)
 *     transpose  111 NoTrans, 112 Trans, 113 ConjTrans   (gblas.h:111)
 *     dtype      16 Half, 32 Single                      (Precision, gblas.h:118-123)
 *                1600 bfloat16 (an addition: the reference has no bf16 type)
 * Matrix pointers are "buffer + offset" already resolved by the caller, exactly what the
 * reference passes to its cuBLAS calls (gpgpu/src/gblas.cpp:1928-1930). Leading dimensions,
 * strides and offsets are counted in elements. alpha / beta are passed by pointer in the
 * storage type of the matrices (host memory).
 */
#ifndef DLF_B200_H_
#define DLF_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    DLF_B200_ROW_MAJOR = 101,
    DLF_B200_COL_MAJOR = 102,
    DLF_B200_NO_TRANS = 111,
    DLF_B200_TRANS = 112,
    DLF_B200_CONJ_TRANS = 113,
    DLF_B200_UPPER = 121,     /* Triangle, Diagonal, Side: gpgpu/include/gblas.h:112-114 */
    DLF_B200_LOWER = 122,
    DLF_B200_NON_UNIT = 131,
    DLF_B200_UNIT = 132,
    DLF_B200_LEFT = 141,
    DLF_B200_RIGHT = 142,
    DLF_B200_HALF = 16,
    DLF_B200_SINGLE = 32,
    DLF_B200_BFLOAT16 = 1600
};

/* C = alpha * op(A) * op(B) + beta * C.
 * Replaces gpgpu::blas::gemm<T> (gpgpu/include/gblas.h:496-504; cuBLAS call site
 * gpgpu/src/gblas.cpp:1926-1951; OpenCL routine gpgpu/src/routines/level3/xgemm.cpp:53-99).
 * beta == 0 never reads C. */
int dlf_b200_gemm(int dtype, int layout, int trans_a, int trans_b, size_t m, size_t n, size_t k,
                  const void* alpha, const void* a, size_t a_ld, const void* b, size_t b_ld,
                  const void* beta, void* c, size_t c_ld, void* stream);

/* dlf_b200_gemm with optional scratch (may be NULL: then exactly dlf_b200_gemm). With at least
 * dlf_b200_gemm_workspace_bytes(...) bytes of caller-owned device memory, products that have few
 * output tiles and a long K (a fully connected layer 256 x 1000 x 2048, a 1024^3 product) are cut
 * along K into slices that run side by side, followed by a reduction kernel; other products run
 * as before. The reference takes such temporaries from its context's pool
 * (Xgemm's temp buffer, gpgpu/src/routines/level3/xgemm.cpp:107-223). Results of a split product
 * differ from the unsplit one by fp32 rounding of the slice sums only. */
int dlf_b200_gemm_ex(int dtype, int layout, int trans_a, int trans_b, size_t m, size_t n, size_t k,
                     const void* alpha, const void* a, size_t a_ld, const void* b, size_t b_ld,
                     const void* beta, void* c, size_t c_ld, void* workspace, size_t workspace_bytes,
                     void* stream);
size_t dlf_b200_gemm_workspace_bytes(int dtype, size_t m, size_t n, size_t k);

/* Same product for batch_count matrices spaced by fixed strides; a stride of 0 shares one
 * operand between all batches. Replaces gpgpu::blas::gemmStridedBatched<T>
 * (gblas.h:673-683; gblas.cpp:3090-3141; routines/levelx/xgemmstridedbatched.cpp:53-95). */
int dlf_b200_gemm_strided_batched(int dtype, int layout, int trans_a, int trans_b, size_t m,
                                  size_t n, size_t k, const void* alpha, const void* a,
                                  size_t a_ld, size_t a_stride, const void* b, size_t b_ld,
                                  size_t b_stride, const void* beta, void* c, size_t c_ld,
                                  size_t c_stride, size_t batch_count, void* stream);

/* Batched product with per-batch alpha / beta and per-batch element offsets, all given as host
 * arrays of batch_count entries, as in gpgpu::blas::gemmBatched<T> (gblas.h:661-671;
 * gblas.cpp:2928-3012; routines/levelx/xgemmbatched.cpp:51-118). a, b, c are the buffer bases.
 * The tables are copied into `workspace` (device memory, at least
 * dlf_b200_gemm_batched_workspace_bytes(batch_count) bytes, owned by the caller, e.g. taken from
 * gpgpu's TemporaryBuffer pool) on the given stream before the kernel runs. Tables that are affine
 * in the batch index (offset_i = offset_0 + i * stride, stride >= 0, one alpha and one beta) are
 * recognised on the host and run as dlf_b200_gemm_strided_batched: nothing is copied then. */
int dlf_b200_gemm_batched(int dtype, int layout, int trans_a, int trans_b, size_t m, size_t n,
                          size_t k, const void* alphas, const void* a, const size_t* a_offsets,
                          size_t a_ld, const void* b, const size_t* b_offsets, size_t b_ld,
                          const void* betas, void* c, const size_t* c_offsets, size_t c_ld,
                          size_t batch_count, void* workspace, size_t workspace_bytes,
                          void* stream);
size_t dlf_b200_gemm_batched_workspace_bytes(size_t batch_count);

/* dlf_b200_gemm_batched without the workspace argument, for callers that have no device scratch
 * to hand over and must not create any at call time - for instance a dlf routine that is invoked
 * while its context's temporary-buffer pool (a LIFO slab, not thread-safe) is already in use
 * further up the call stack, or a process whose device memory was given away in full at start-up.
 * This entry point has no counterpart in the reference. It allocates nothing: the per-batch
 * tables go into a fixed array inside the library's device image (128 KiB on every GPU that loads
 * the library, kept until the process exits), so batch_count is limited to
 * DLF_B200_NOALLOC_MAX_BATCH; a larger count returns kInsufficientMemoryTemp (-2050) and does
 * nothing. The first call on each device looks up the array's device address and sets kernel
 * attributes; make that first call outside any stream capture. All calls share the one array:
 * each call rewrites the part it uses before its kernel reads it, in stream order, so calls on
 * the same stream are safe, but two calls whose work overlaps on the GPU (different streams or
 * host threads without ordering between them) race on the tables. Results are identical to
 * dlf_b200_gemm_batched. */
#define DLF_B200_NOALLOC_MAX_BATCH 4096
int dlf_b200_gemm_batched_noalloc(int dtype, int layout, int trans_a, int trans_b, size_t m,
                                  size_t n, size_t k, const void* alphas, const void* a,
                                  const size_t* a_offsets, size_t a_ld, const void* b,
                                  const size_t* b_offsets, size_t b_ld, const void* betas, void* c,
                                  const size_t* c_offsets, size_t c_ld, size_t batch_count,
                                  void* stream);

/* NCHW cross-correlation Y = conv2d(X, W) (+ bias), computed as an implicit GEMM: no im2col
 * buffer is materialised. X is {batches, channels, height, width}, W is
 * {num_kernels, channels/group, kernel_h, kernel_w}, Y is {batches, num_kernels, output_h,
 * output_w}; (pad_top, pad_left) is the origin shift, pad_bottom / pad_right only enter through
 * output_h / output_w, as in dlf (dlf/include/tensor/dnn.h:92-109).
 * Replaces gpgpu::dnn::conv2d<T> (gpgpu/include/gdnn.h:201-213; gpgpu/src/gdnn.cpp:1577-1630).
 * `bias` (num_kernels entries, storage type) may be NULL; when given it is added in the
 * epilogue, replacing the separate transformChannel pass of ConvOp
 * (dlf/include/predict.h:1272-1281). `workspace` is optional caller-owned device scratch
 * (dlf_b200_conv2d_workspace_bytes: about the size of X for 16-bit convolutions of one group,
 * whose activations are copied there channels-last and then fetched by tensor-map loads; a few MB
 * for the packed filter bank otherwise). With NULL the kernels gather their operands themselves:
 * same results within the tolerance, slower. */
int dlf_b200_conv2d(int dtype, size_t batches, size_t channels, size_t height, size_t width,
                    size_t output_h, size_t output_w, size_t num_kernels, size_t group,
                    size_t kernel_h, size_t kernel_w, size_t pad_top, size_t pad_left,
                    size_t pad_bottom, size_t pad_right, size_t stride_h, size_t stride_w,
                    size_t dilation_h, size_t dilation_w, const void* x, const void* w,
                    const void* bias, void* y, void* workspace, size_t workspace_bytes,
                    void* stream);
/* Convolution with the operator-level fusion dlf's graph runtime applies around it: ConvOp is
 * conv + bias (dlf/include/predict.h:1258-1286) and in ResNet-style graphs is followed by an Add
 * of the block's input and a Relu, each a separate full pass over Y in the reference. Here
 *     Y = act(conv2d(X, W) + bias + residual)
 * in the convolution's epilogue. `residual` (NULL, or a tensor with Y's shape and layout; it may
 * be Y itself) is read once per element before Y is written; `activation` is one of the values
 * below. With residual == NULL and DLF_B200_ACT_NONE this is dlf_b200_conv2d. */
#define DLF_B200_ACT_NONE 0
#define DLF_B200_ACT_RELU 1
int dlf_b200_conv2d_fused(int dtype, size_t batches, size_t channels, size_t height, size_t width,
                          size_t output_h, size_t output_w, size_t num_kernels, size_t group,
                          size_t kernel_h, size_t kernel_w, size_t pad_top, size_t pad_left,
                          size_t pad_bottom, size_t pad_right, size_t stride_h, size_t stride_w,
                          size_t dilation_h, size_t dilation_w, const void* x, const void* w,
                          const void* bias, const void* residual, int activation, void* y,
                          void* workspace, size_t workspace_bytes, void* stream);

size_t dlf_b200_conv2d_workspace_bytes(int dtype, size_t batches, size_t channels, size_t height,
                                       size_t width, size_t output_h, size_t output_w,
                                       size_t num_kernels, size_t group, size_t kernel_h,
                                       size_t kernel_w);

/* Channels-last operators for an operator-list runtime (dlf's Predictor, dlf/include/predict.h:
 * 2048-2070) that owns the tensors between its operators and may therefore keep them in the
 * layout the tensor-map unit reads: (N, H, W, C), 16-bit, C a multiple of 8, 16-byte aligned.
 * The reference's own operators are NCHW (gpgpu/include/gdnn.h:201-251); these entries compute
 * the same functions on the permuted tensors.
 *
 * dlf_b200_conv2d_nhwc: Y = act(conv2d(X, W) + bias + residual), one group. X is (N, H, W, C);
 * `w_packed` is the filter bank as dlf_b200_pack_filters_nhwc writes it - (Cout, KH*KW, Ck), Ck = C
 * rounded up to 64, dlf_b200_nhwc_filter_elems elements; for a 1x1 filter over a multiple of 64
 * channels that is the OIHW bank itself. `y_layout` says how Y (and `residual`, which has Y's shape
 * and layout) is stored: DLF_B200_LAYOUT_NHWC (Cout a multiple of 8) or DLF_B200_LAYOUT_NCHW. The
 * activations are fetched by im2col-mode tensor-map loads straight from X: no scratch, no copy, one
 * launch. kNotImplemented (nothing launched) for what the tensor-map unit cannot address: channel
 * counts that are not a multiple of 8, unaligned bases, pads of 128 or more, strides above 8,
 * filters above 16 x 16, (k - 1) * dilation of 256 or more.
 * dlf_b200_nchw_to_nhwc: (N, C, H, W) -> (N, H, W, C') with C' = C rounded up to 8, the added
 * channels zero. dlf_b200_pool_nhwc: max (average == 0) or average pooling on (N, H, W, C), C a
 * multiple of 8, with the arithmetic of dlf_b200_maxpool / dlf_b200_avgpool; a global pool is the
 * window kernel = (H, W). */
#define DLF_B200_LAYOUT_NHWC 0
#define DLF_B200_LAYOUT_NCHW 1
size_t dlf_b200_nhwc_filter_elems(size_t channels, size_t num_kernels, size_t kernel_h, size_t kernel_w);
int dlf_b200_pack_filters_nhwc(int dtype, size_t channels, size_t num_kernels, size_t kernel_h, size_t kernel_w,
                               const void* w, void* w_packed, void* stream);
int dlf_b200_nchw_to_nhwc(int dtype, size_t batches, size_t channels, size_t height, size_t width, const void* x,
                          void* y, void* stream);
int dlf_b200_conv2d_nhwc(int dtype, size_t batches, size_t channels, size_t height, size_t width, size_t output_h,
                         size_t output_w, size_t num_kernels, size_t kernel_h, size_t kernel_w, size_t pad_top,
                         size_t pad_left, size_t pad_bottom, size_t pad_right, size_t stride_h, size_t stride_w,
                         size_t dilation_h, size_t dilation_w, const void* x, const void* w_packed, const void* bias,
                         const void* residual, int activation, void* y, int y_layout, void* stream);
int dlf_b200_pool_nhwc(int dtype, int average, int count_include_pad, size_t batches, size_t channels, size_t height,
                       size_t width, size_t output_h, size_t output_w, size_t kernel_h, size_t kernel_w, size_t pad_top,
                       size_t pad_left, size_t stride_h, size_t stride_w, const void* x, void* y, void* stream);

/* Level-3 routines that run on the GEMM main loop. Each replaces the gpgpu::blas template of the
 * same name (gpgpu/include/gblas.h:506-586; instantiations gpgpu/src/gblas.cpp; the OpenCL
 * routines expand the symmetric / triangular operand into a general square and call Xgemm, which
 * is the scheme used here too) with the semantics of the CPU path
 * (dlf/include/tensor/linalg_detail.h:362-560, 720-1334):
 *   symm  C = alpha*S*B + beta*C (Left, S is m x m) or alpha*B*S + beta*C (Right, S is n x n);
 *         only the named triangle of A is read;
 *   syrk  the named triangle of C = alpha*op(A)*op(A)^T + beta*C, op(A) is n x k; the other
 *         triangle of C is left untouched;
 *   trmm  B = alpha*op(T)*B (Left) or alpha*B*op(T) (Right), T triangular in the named triangle
 *         of A, with an implicit unit diagonal when diagonal == DLF_B200_UNIT;
 *   trsm  solves op(T)*X = alpha*B (Left) or X*op(T) = alpha*B (Right); X overwrites B.
 * `workspace` is caller-owned device scratch of at least dlf_b200_level3_workspace_bytes(...)
 * bytes (the reference takes its temporaries from the context's pool); trsm needs none.
 * Argument errors return the StatusCode of the matching gblas routine. */
enum { DLF_B200_SYMM = 1, DLF_B200_SYRK = 2, DLF_B200_TRMM = 3, DLF_B200_TRSM = 4 };
size_t dlf_b200_level3_workspace_bytes(int routine, int dtype, size_t m, size_t n);
int dlf_b200_symm(int dtype, int layout, int side, int triangle, size_t m, size_t n, const void* alpha,
                  const void* a, size_t a_ld, const void* b, size_t b_ld, const void* beta, void* c,
                  size_t c_ld, void* workspace, size_t workspace_bytes, void* stream);
int dlf_b200_syrk(int dtype, int layout, int triangle, int a_transpose, size_t n, size_t k,
                  const void* alpha, const void* a, size_t a_ld, const void* beta, void* c, size_t c_ld,
                  void* workspace, size_t workspace_bytes, void* stream);
int dlf_b200_trmm(int dtype, int layout, int side, int triangle, int a_transpose, int diagonal, size_t m,
                  size_t n, const void* alpha, const void* a, size_t a_ld, void* b, size_t b_ld,
                  void* workspace, size_t workspace_bytes, void* stream);
int dlf_b200_trsm(int dtype, int layout, int side, int triangle, int a_transpose, int diagonal, size_t m,
                  size_t n, const void* alpha, const void* a, size_t a_ld, void* b, size_t b_ld,
                  void* workspace, size_t workspace_bytes, void* stream);

/* NCHW pooling, the second "next" step around the convolution path (a ResNet forward is
 * conv -> maxpool -> ... -> global average pool -> FC). Replace gpgpu::dnn::maxpool / avgpool
 * (gpgpu/include/gdnn.h:215-238; definitions and the argument order that callers use - output
 * size before kernel size - gpgpu/src/gdnn.cpp:1667-1676, 1728-1738), which run cuDNN pooling or
 * an OpenCL kernel. Semantics are those of dlf's CPU pooling
 * (dlf/include/tensor/dnn_detail.h:172-227): X is {batches, channels, height, width}, Y is
 * {batches, channels, output_h, output_w}; (pad_top, pad_left) is the origin shift, pad_bottom /
 * pad_right only enter through the output size; max starts from the type's lowest value; the
 * average divides by the number of taps inside the image, or by kernel_h*kernel_w when
 * count_include_pad is non-zero. Global pooling (dlf/include/tensor/dnn.h:337-375) is the case
 * kernel = {height, width}, output 1 x 1, which takes a one-warp-per-plane reduction. */
int dlf_b200_maxpool(int dtype, size_t batches, size_t channels, size_t height, size_t width,
                     size_t output_h, size_t output_w, size_t kernel_h, size_t kernel_w,
                     size_t pad_top, size_t pad_left, size_t pad_bottom, size_t pad_right,
                     size_t stride_h, size_t stride_w, size_t dilation_h, size_t dilation_w,
                     const void* x, void* y, void* stream);
int dlf_b200_avgpool(int dtype, size_t batches, size_t channels, size_t height, size_t width,
                     size_t output_h, size_t output_w, size_t kernel_h, size_t kernel_w,
                     size_t pad_top, size_t pad_left, size_t pad_bottom, size_t pad_right,
                     size_t stride_h, size_t stride_w, size_t dilation_h, size_t dilation_w,
                     int count_include_pad, const void* x, void* y, void* stream);

/* Name of a status code returned by the functions above (static storage). Mirrors the
 * StatusCode enumerators of gblas.h:43-107. */
const char* dlf_b200_status_string(int status);

/* Synchronises the current device and reads-and-clears its kernel status word: 0 when every
 * kernel since the last call ran to completion, non-zero when a bounded device-side wait gave
 * up (bit 0). Kernels never trap or spin forever; this is how such a failure is reported. */
int dlf_b200_device_status(int* device_status);

/* Tuning overrides for experiments, for every following call of this process: force the N-tile
 * width (64, 128 or 256; the kernel that keeps operand A in tensor memory takes any multiple of
 * 32 in that range; 0 = automatic) and the operand path: 0 = automatic, 1 = never the TMA
 * producer, 2 = always the loader-warp kernel with both operands in shared memory, 3 = the
 * kernel that keeps operand A in tensor memory whenever the TMA producer is not used, 4 = as 0
 * but convolutions never use the row form (horizontal taps as GEMM columns), 5 = as 0 but the
 * row form only for stride_w = 1. Higher bits switch
 * single features for measurements: 0x100 TMA stores of 32-column blocks only (default: 64
 * columns for tiles of 128 columns or more), 0x200 use CTA pairs (cta_group::2) for 256-column fp16 tiles,
 * 0x400 a second accumulator only when three operand slots remain in tensor memory (default:
 * two), 0x800 no TMA for the fp32 B operand, 0x1000 no K-chunked fp32 accumulation, 0x2000 no
 * affine addressing for 1x1 filters, 0x4000 no TMA stores, 0x8000 never pack the filter bank of
 * a convolution. Bits 16 and up are measurement aids: most switch a part of a kernel off to time the
 * rest (results are then meaningless); 0x100 << 16 (pooling always through the generic
 * one-thread-per-output kernel) and 0x4000 << 16 (no programmatic dependent launch after the
 * filter-packing grid) keep results valid. 0x10000000 is a test aid for the device-side time-out
 * path: a launch that consists of one tile leaves out the commit that hands its accumulator to the
 * epilogue and waits at most 2^21 clocks (about a millisecond): the call returns, the output is
 * not written and dlf_b200_device_status() reports bit 0 once.
 * Bits 16 and up of force_bn steer the channels-last route of 16-bit convolutions (transposing
 * copy into the caller's scratch + tensor-map-fed operand): 0x10000 never take it (the kernels
 * that gather the activations themselves serve the call, as they do for callers without scratch),
 * 0x40000 dlf_b200_gemm_batched always through its offset tables (default: tables that are affine in
 * the batch index take the strided path), 0x20000 swap the operand roles (lanes = output channels) for every even plane size, not only
 * for planes of a multiple of 8 pixels, 0x80000 never swap the roles of a 1x1 stride-1 convolution
 * that runs as a batched GEMM, 0x200000 never use the instantiation of the TMA-fed kernel with four
 * sets of epilogue warps (default for tiles of 128 or more columns with K <= 512), 0x400000 never
 * the one with three sets, 0x800000 never the halo-tile kernel (stride-1 filters larger than 1x1
 * over a multiple of 64 channels; default with at most 64 output channels and rows of a multiple
 * of 8 outputs), 0x1000000 that kernel for every convolution it can serve, 0x8000000 32-column
 * boxes only in the swapped NCHW epilogue (default: 64-column boxes where a warp owns 64 columns),
 * 0x10000000 never compute a channels-last convolution with the filter bank as operand A (default
 * for filters larger than 1x1 with 65 to 128 output channels), 0x40000000 never compute a plain
 * 16-bit product transposed (default for K <= 256 and N >= 128 when the result can leave through
 * TMA stores: the epilogue then writes 16-byte pieces of D's contiguous direction). */
void dlf_b200_set_tuning(int force_bn, int force_generic_loader);

/* Counts kernel launches made by this library in this process (all threads). */
unsigned long long dlf_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* DLF_B200_H_ */

// Exercises the C++ host side (include/dlf_b200_gpgpu.hpp) the way dlf's own GPU tests exercise
// gpgpu::blas / gpgpu::dnn: the gemm golden of dlf/test/GPGPUTest.cpp:236-304 through all four
// transpose combinations, the conv + bias golden of dlf/test/model/PredictTest.cpp:92-117, a
// strided-batched and an offset-table batched product against a host loop, and the reference's
// exceptions for bad arguments. Prints "ok" and exits 0 on success.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "dlf_b200_gpgpu.hpp"

using namespace dlf_b200::gpgpu;
using blas::Layout;
using blas::Transpose;

static int failures = 0;
#define CHECK(cond)                                                      \
    do {                                                                 \
        if (!(cond)) {                                                   \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            ++failures;                                                  \
        }                                                                \
    } while (0)

template <typename T>
static Buffer<T> dev(const std::vector<T>& h) {
    Buffer<T> b(h.size());
    b.write(current::queue(), h.data(), h.size());
    return b;
}
template <typename T>
static std::vector<T> host(const Buffer<T>& b) {
    std::vector<T> h(b.size());
    b.read(current::queue(), h.data(), h.size());
    return h;
}

static void gemm_golden() {
    const std::vector<float> A = {5, 10, 9, 1, 10, 3, 7, 6, 6, 6, 1, 1, 6, 2, 6, 10, 9, 3};
    const std::vector<float> At = {5, 7, 6, 10, 6, 2, 9, 6, 6, 1, 6, 10, 10, 1, 9, 3, 1, 3};
    const std::vector<float> B = {7, 1, 8, 7, 9, 5, 2, 6, 7, 8, 5, 7, 6, 9, 1, 1, 4, 10, 1, 10, 3, 8, 8, 5};
    const std::vector<float> Bt = {7, 9, 7, 6, 4, 3, 1, 5, 8, 9, 10, 8, 8, 2, 5, 1, 1, 8, 7, 6, 7, 1, 10, 5};
    const std::vector<float> C = {230, 254, 116, 199, 219, 236, 201, 252, 173, 148, 155, 167};
    const std::vector<float> R = {1176, 1282, 628, 1145, 1033, 1022, 829, 1052, 933, 980, 715, 923};
    auto dA = dev(A), dAt = dev(At), dB = dev(B), dBt = dev(Bt);
    struct Case { Transpose ta, tb; Buffer<float>* a; size_t lda; Buffer<float>* b; size_t ldb; };
    const Case cases[] = {{Transpose::NoTrans, Transpose::NoTrans, &dA, 6, &dB, 4},
                          {Transpose::Trans, Transpose::NoTrans, &dAt, 3, &dB, 4},
                          {Transpose::NoTrans, Transpose::Trans, &dA, 6, &dBt, 6},
                          {Transpose::Trans, Transpose::Trans, &dAt, 3, &dBt, 6}};
    for (const auto& c : cases) {
        auto dC = dev(C);
        Event ev;
        blas::gemm<float>(Layout::RowMajor, c.ta, c.tb, 3, 4, 6, 2.0f, *c.a, 0, c.lda, *c.b, 0, c.ldb, 3.0f, dC, 0,
                          4, current::queue(), &ev);
        CHECK(host(dC) == R);
        CHECK(ev.getElapsedTime() >= 0.0f);
    }
    // half precision: all values are exactly representable
    std::vector<__half> hA(A.size()), hB(B.size()), hC(C.size());
    for (size_t i = 0; i < A.size(); ++i) hA[i] = __float2half(A[i]);
    for (size_t i = 0; i < B.size(); ++i) hB[i] = __float2half(B[i]);
    for (size_t i = 0; i < C.size(); ++i) hC[i] = __float2half(C[i]);
    auto dhA = dev(hA), dhB = dev(hB), dhC = dev(hC);
    blas::gemm<__half>(Layout::RowMajor, Transpose::NoTrans, Transpose::NoTrans, 3, 4, 6, __float2half(2.0f), dhA, 0,
                       6, dhB, 0, 4, __float2half(3.0f), dhC, 0, 4);
    auto out = host(dhC);
    for (size_t i = 0; i < R.size(); ++i) CHECK(__half2float(out[i]) == R[i]);
}

static void conv_bias_golden() {
    std::vector<float> X(25), W(9, 1.0f), bias = {1.0f};
    for (int i = 0; i < 25; ++i) X[i] = static_cast<float>(i);
    const std::vector<float> Y = {13, 22, 28, 34, 25, 34, 55, 64, 73, 52, 64, 100, 109,
                                  118, 82, 94, 145, 154, 163, 112, 73, 112, 118, 124, 85};
    auto dX = dev(X), dW = dev(W), dBias = dev(bias);
    Buffer<float> dY(25);
    // the binding hands the library scratch from the temporary-buffer pool, so the filter bank is
    // packed by a launch of its own before the main kernel: two launches per convolution
    const unsigned long long launches0 = dlf_b200_launch_count();
    dnn::conv2d<float>(1, 1, 5, 5, 5, 5, 1, 1, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, dX, dW, dY, current::queue(), nullptr,
                       &dBias);
    CHECK(dlf_b200_launch_count() - launches0 == 2);
    CHECK(host(dY) == Y);

    // fused: relu(conv + bias + residual) with residual = -60 everywhere
    std::vector<float> R(25, -60.0f), Yf(25);
    for (int i = 0; i < 25; ++i) Yf[i] = Y[i] - 60.0f > 0.0f ? Y[i] - 60.0f : 0.0f;
    auto dR = dev(R);
    Buffer<float> dY2(25);
    dnn::conv2d<float>(1, 1, 5, 5, 5, 5, 1, 1, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, dX, dW, dY2, current::queue(), nullptr,
                       &dBias, &dR, DLF_B200_ACT_RELU);
    CHECK(host(dY2) == Yf);
}

static void channels_last_chain() {
    // 8 channels of ones, 3x3 filter bank of ones over 8 channels, pad 1 on a 4 x 4 image: every output
    // is 8 x (taps inside the image) + bias, exactly representable in fp16. Through the channels-last
    // entries: copy, packed filters, convolution with both output layouts, then a 2 x 2 max pool.
    const size_t N = 1, C = 8, H = 4, W = 4, Co = 8;
    std::vector<__half> X(N * C * H * W, __float2half(1.0f)), Wt(Co * C * 9, __float2half(1.0f)), b(Co);
    for (size_t i = 0; i < Co; ++i) b[i] = __float2half(static_cast<float>(i));
    auto dX = dev(X), dW = dev(Wt), dB = dev(b);
    Buffer<__half> dXn(N * H * W * C), dWp(dlf_b200_nhwc_filter_elems(C, Co, 3, 3)), dYn(N * H * W * Co), dYc(N * Co * H * W);
    dnn::nchw_to_nhwc<__half>(N, C, H, W, dX, dXn);
    dnn::pack_filters_nhwc<__half>(C, Co, 3, 3, dW, dWp);
    const unsigned long long launches0 = dlf_b200_launch_count();
    dnn::conv2d_nhwc<__half>(N, C, H, W, H, W, Co, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, dXn, dWp, dYn, current::queue(), nullptr, &dB);
    CHECK(dlf_b200_launch_count() - launches0 == 1);  // no scratch, no copy: one launch
    dnn::conv2d_nhwc<__half>(N, C, H, W, H, W, Co, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, dXn, dWp, dYc, current::queue(), nullptr, &dB,
                             nullptr, DLF_B200_ACT_NONE, dnn::Layout4D::NCHW);
    const auto yn = host(dYn), yc = host(dYc);
    for (size_t h = 0; h < H; ++h)
        for (size_t w = 0; w < W; ++w) {
            const int th = 3 - (h == 0) - (h == H - 1), tw = 3 - (w == 0) - (w == W - 1);
            for (size_t co = 0; co < Co; ++co) {
                const float want = 8.0f * th * tw + static_cast<float>(co);
                CHECK(__half2float(yn[(h * W + w) * Co + co]) == want);
                CHECK(__half2float(yc[(co * H + h) * W + w]) == want);
            }
        }
    Buffer<__half> dP(N * 2 * 2 * Co);
    dnn::pool_nhwc<__half>(false, false, N, Co, H, W, 2, 2, 2, 2, 0, 0, 2, 2, dYn, dP);
    const auto pooled = host(dP);
    for (size_t co = 0; co < Co; ++co) CHECK(__half2float(pooled[co]) == 72.0f + static_cast<float>(co));  // max of the top-left 2 x 2: the interior 9-tap pixel
}

static void maxpool_golden() {
    // TEST(MaxPool, basic_2d_with_padding), dlf/test/DNNTest.cpp:625-644
    std::vector<float> X(25);
    for (int i = 0; i < 25; ++i) X[i] = static_cast<float>(i + 1);
    const std::vector<float> R = {7,  8,  9,  10, 10, 12, 13, 14, 15, 15, 17, 18, 19,
                                  20, 20, 22, 23, 24, 25, 25, 22, 23, 24, 25, 25};
    auto dX = dev(X);
    Buffer<float> dY(25);
    dnn::maxpool<float>(1, 1, 5, 5, 5, 5, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, dX, dY);
    CHECK(host(dY) == R);
    // global average of the same plane through avgpool with the plane as the window
    Buffer<float> dG(1);
    dnn::avgpool<float>(1, 1, 5, 5, 1, 1, 5, 5, 0, 0, 0, 0, 5, 5, 1, 1, false, dX, dG);
    CHECK(host(dG) == std::vector<float>{13.0f});
}

static void batched() {
    const size_t m = 5, n = 7, k = 9, batch = 3;
    std::vector<float> A(batch * m * k), B(k * n), C(batch * m * n, 0.0f);
    for (size_t i = 0; i < A.size(); ++i) A[i] = static_cast<float>((i * 7) % 11) - 5.0f;
    for (size_t i = 0; i < B.size(); ++i) B[i] = static_cast<float>((i * 5) % 13) - 6.0f;
    std::vector<float> ref(C.size());
    for (size_t b = 0; b < batch; ++b)
        for (size_t i = 0; i < m; ++i)
            for (size_t j = 0; j < n; ++j) {
                float acc = 0;
                for (size_t kk = 0; kk < k; ++kk) acc += A[(b * m + i) * k + kk] * B[kk * n + j];
                ref[(b * m + i) * n + j] = acc;
            }
    auto dA = dev(A), dB = dev(B), dC = dev(C);
    // shared B: stride 0, as the reference's convolution passes its weights
    blas::gemmStridedBatched<float>(Layout::RowMajor, Transpose::NoTrans, Transpose::NoTrans, m, n, k, 1.0f, dA, 0, k,
                                    m * k, dB, 0, n, 0, 0.0f, dC, 0, n, m * n, batch);
    CHECK(host(dC) == ref);
    auto dC2 = dev(C);
    const std::vector<float> alphas(batch, 1.0f), betas(batch, 0.0f);
    const std::vector<size_t> ao = {0, m * k, 2 * m * k}, bo = {0, 0, 0}, co = {2 * m * n, 0, m * n};
    blas::gemmBatched<float>(Layout::RowMajor, Transpose::NoTrans, Transpose::NoTrans, m, n, k, alphas.data(), dA,
                             ao.data(), k, dB, bo.data(), n, betas.data(), dC2, co.data(), n, batch);
    // a second offset-table call right behind the first, without waiting: both take their tables
    // from the same pool slab, ordered by the queue
    auto dC3 = dev(C);
    const std::vector<size_t> co3 = {m * n, 2 * m * n, 0};
    blas::gemmBatched<float>(Layout::RowMajor, Transpose::NoTrans, Transpose::NoTrans, m, n, k, alphas.data(), dA,
                             ao.data(), k, dB, bo.data(), n, betas.data(), dC3, co3.data(), n, batch);
    auto got = host(dC2);
    auto got3 = host(dC3);
    for (size_t b = 0; b < batch; ++b)
        for (size_t e = 0; e < m * n; ++e) {
            CHECK(got[co[b] + e] == ref[b * m * n + e]);
            CHECK(got3[co3[b] + e] == ref[b * m * n + e]);
        }
}

static void temporary_pool_is_lifo() {
    // releaseTemporaryBuffer (gpgpu/src/gpgpu.cpp:207-214): out-of-order release is an error
    TemporaryBuffer<float> outer(100);
    {
        TemporaryBuffer<unsigned char> inner(33);
        CHECK(inner.offset() >= 400);
        CHECK(reinterpret_cast<uintptr_t>(inner.unwrap()) % 256 == 0);
    }
    TemporaryBuffer<float> again(10);
    CHECK(again.offset() * sizeof(float) >= 400 && again.offset() * sizeof(float) < 1024);
}

static void level3_goldens() {
    // symm_test / trmm_test of dlf/test/GPGPUTest.cpp:307-470: A = {6,5}.range(1), B = {4,3}.range(1) / identity
    std::vector<float> A(30), B(12);
    for (int i = 0; i < 30; ++i) A[i] = static_cast<float>(i + 1);
    for (int i = 0; i < 12; ++i) B[i] = static_cast<float>(i + 1);
    auto dA = dev(A), dB = dev(B);
    Buffer<float> dC(12);
    blas::symm<float>(Layout::RowMajor, blas::Side::Left, blas::Triangle::Lower, 4, 3, 1.0f, dA, 0, 5, dB, 0, 3, 0.0f, dC, 0, 3);
    CHECK(host(dC) == (std::vector<float>{262, 296, 330, 288, 330, 372, 330, 384, 438, 400, 470, 540}));
    blas::symm<float>(Layout::RowMajor, blas::Side::Right, blas::Triangle::Upper, 4, 3, 1.0f, dA, 0, 5, dB, 0, 3, 0.0f, dC, 0, 3);
    CHECK(host(dC) == (std::vector<float>{14, 40, 58, 32, 91, 130, 50, 142, 202, 68, 193, 274}));
    std::vector<float> I(16, 0.0f);
    for (int i = 0; i < 4; ++i) I[i * 5] = 1.0f;
    auto dI = dev(I);
    blas::trmm<float>(Layout::RowMajor, blas::Side::Left, blas::Triangle::Upper, Transpose::NoTrans, blas::Diagonal::Unit, 4, 4,
                      1.0f, dA, 0, 5, dI, 0, 4);
    CHECK(host(dI) == (std::vector<float>{1, 2, 3, 4, 0, 1, 8, 9, 0, 0, 1, 14, 0, 0, 0, 1}));
    // trsm undoes it
    blas::trsm<float>(Layout::RowMajor, blas::Side::Left, blas::Triangle::Upper, Transpose::NoTrans, blas::Diagonal::Unit, 4, 4,
                      1.0f, dA, 0, 5, dI, 0, 4);
    CHECK(host(dI) == I);
    // syrk: lower triangle of C = A A^T for the leading 3 x 5 block of A; the strict upper triangle keeps its 7s
    std::vector<float> C(9, 7.0f);
    auto dS = dev(C);
    blas::syrk<float>(Layout::RowMajor, blas::Triangle::Lower, Transpose::NoTrans, 3, 5, 1.0f, dA, 0, 5, 0.0f, dS, 0, 3);
    CHECK(host(dS) == (std::vector<float>{55, 7, 7, 130, 330, 7, 205, 530, 855}));
}

static void errors() {
    Buffer<float> a(16), c(15);
    auto status_of = [&](auto&& fn) {
        try {
            fn();
        } catch (const blas::BLASError& e) {
            return static_cast<int>(e.status());
        }
        return 0;
    };
    CHECK(status_of([&] { blas::gemm<float>(Layout::RowMajor, Transpose::NoTrans, Transpose::NoTrans, 0, 4, 4, 1.f, a,
                                            0, 4, a, 0, 4, 0.f, a, 0, 4); }) == -1017);
    CHECK(status_of([&] { blas::gemm<float>(Layout::RowMajor, Transpose::NoTrans, Transpose::NoTrans, 4, 4, 4, 1.f, a,
                                            0, 3, a, 0, 4, 0.f, a, 0, 4); }) == -1016);
    CHECK(status_of([&] { blas::gemm<float>(Layout::RowMajor, Transpose::NoTrans, Transpose::NoTrans, 4, 4, 4, 1.f, a,
                                            0, 4, a, 0, 4, 0.f, c, 0, 4); }) == -1009);
    CHECK(status_of([&] { blas::gemmStridedBatched<float>(Layout::RowMajor, Transpose::NoTrans, Transpose::NoTrans, 4,
                                                          4, 4, 1.f, a, 0, 4, 0, a, 0, 4, 0, 0.f, a, 0, 4, 0, 0); }) ==
          -2049);
}

int main() {
    gemm_golden();
    conv_bias_golden();
    channels_last_chain();
    maxpool_golden();
    batched();
    temporary_pool_is_lifo();
    level3_goldens();
    errors();
    int dev_status = -1;
    CHECK(dlf_b200_device_status(&dev_status) == 0 && dev_status == 0);
    if (failures) return 1;
    std::printf("ok\n");
    return 0;
}

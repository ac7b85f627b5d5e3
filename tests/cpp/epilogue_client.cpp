// The C ABI used the way the reference would use it: plain C++ and the CUDA runtime, no Python, no torch.
// Mirrors the patched ConvLayer<Device::CUDA>::forward (include/cuda/ConvLayer.h:284-307): the layer owns
// its output and parameter buffers, the call fills one descriptor.  Checks the result against a host loop of
// the reference's formulas and prints "ok"; any mismatch or error status is a non-zero exit code.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime.h>

#include "pxe.h"

#define CUDA_OK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
    std::printf("%s: %s\n", #call, cudaGetErrorString(e_)); return 10; } } while (0)
#define PXE_OK_OR_FAIL(call) do { int rc_ = (call); if (rc_ != PXE_OK) { \
    std::printf("%s: %s (%s)\n", #call, pxe_status_string(rc_), pxe_last_error_string()); return 11; } } while (0)

static float* upload(const std::vector<float>& h)
{
    float* d = nullptr;
    if (cudaMalloc(&d, h.size() * sizeof(float)) != cudaSuccess) return nullptr;
    cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice);
    return d;
}

int main()
{
    const int B = 3, C = 24, H = 26, W = 26;
    const size_t n = (size_t)B * C * H * W;
    std::vector<float> x(n), gamma(C), beta(C), mean(C), var(C), from(n);
    unsigned s = 12345u;
    auto rnd = [&s]() { s = s * 1664525u + 1013904223u; return (float)(s >> 8) / 16777216.0f; };
    for (auto& v : x) v = rnd() * 4.0f - 2.0f;
    for (auto& v : from) v = rnd() * 2.0f - 1.0f;
    for (int c = 0; c < C; ++c) { gamma[c] = 0.5f + rnd(); beta[c] = rnd() * 0.2f - 0.1f; mean[c] = rnd() * 0.2f - 0.1f; var[c] = 0.5f + rnd(); }

    float *dx = upload(x), *dg = upload(gamma), *db = upload(beta), *dm = upload(mean), *dv = upload(var), *df = upload(from);
    float *dpool = nullptr, *dwide = nullptr;
    const int OH = pxe_maxpool_out_dim(H, 2, 2, 1), OW = pxe_maxpool_out_dim(W, 2, 2, 1);
    CUDA_OK(cudaMalloc(&dpool, (size_t)B * C * OH * OW * sizeof(float)));
    CUDA_OK(cudaMalloc(&dwide, (size_t)B * (C + 8) * H * W * sizeof(float)));       // a route's concat buffer
    if (!dx || !dg || !db || !dm || !dv || !df) return 12;
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));

    // 1. BN + leaky + shortcut add, stored twice: in place and into channels 8.. of the concat buffer
    pxe_epilogue_desc d{};
    d.x = dx; d.y = dx; d.y2 = dwide + (size_t)8 * H * W; d.y2_batch_stride = (long long)(C + 8) * H * W;
    d.batch = B; d.channels = C; d.height = H; d.width = W;
    d.gamma = dg; d.beta = db; d.mean = dm; d.var = dv; d.eps = 1e-5f; d.eps_mode = PXE_BN_EPS_CUDNN;
    d.act = PXE_ACT_LEAKY;
    d.residual = df; d.res_alpha = 1.0f; d.res_beta = 1.0f; d.res_act = PXE_ACT_LINEAR;
    PXE_OK_OR_FAIL(pxe_conv_epilogue(stream, &d));
    // 2. a second layer's epilogue with the 2x2 max pool folded in, pooled output only
    pxe_epilogue_desc e{};
    e.x = dx; e.y = nullptr; e.batch = B; e.channels = C; e.height = H; e.width = W;
    e.act = PXE_ACT_LINEAR;
    e.pool_kernel = 2; e.pool_stride = 2; e.pool_padding = 1; e.y_pool = dpool;
    PXE_OK_OR_FAIL(pxe_conv_epilogue(stream, &e));
    CUDA_OK(cudaStreamSynchronize(stream));

    std::vector<float> y(n), wide((size_t)B * (C + 8) * H * W), pool((size_t)B * C * OH * OW);
    CUDA_OK(cudaMemcpy(y.data(), dx, n * sizeof(float), cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(wide.data(), dwide, wide.size() * sizeof(float), cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(pool.data(), dpool, pool.size() * sizeof(float), cudaMemcpyDeviceToHost));

    double worst = 0.0;
    for (int b = 0; b < B; ++b)
        for (int c = 0; c < C; ++c)
            for (int i = 0; i < H * W; ++i) {
                const size_t at = ((size_t)b * C + c) * H * W + i;
                const double norm = ((double)x[at] - mean[c]) / std::sqrt((double)var[c] + 1e-5) * gamma[c] + beta[c];
                const double ref = (norm > 0 ? norm : 0.1 * norm) + from[at];
                const double err = std::fabs(y[at] - ref) / (1e-6 + 1e-5 * std::fabs(ref));
                if (err > worst) worst = err;
                if (wide[((size_t)b * (C + 8) + 8 + c) * H * W + i] != y[at]) { std::printf("slot store differs\n"); return 2; }
            }
    if (worst > 1.0) { std::printf("epilogue outside tolerance: %.2f x\n", worst); return 3; }
    for (int b = 0; b < B; ++b)
        for (int c = 0; c < C; ++c)
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    float m = -INFINITY;
                    for (int ky = 0; ky < 2; ++ky)
                        for (int kx = 0; kx < 2; ++kx) {
                            const int iy = 2 * oh + ky, ix = 2 * ow + kx;
                            if (iy < H && ix < W) { const float v = y[((size_t)b * C + c) * H * W + (size_t)iy * W + ix]; if (v > m) m = v; }
                        }
                    if (pool[(((size_t)b * C + c) * OH + oh) * OW + ow] != m) { std::printf("pooled value differs\n"); return 4; }
                }
    // 3. errors come back as status codes, never as exceptions or aborts
    pxe_epilogue_desc bad = d;
    bad.act = 77;
    if (pxe_conv_epilogue(stream, &bad) != PXE_ERR_BAD_ARG) return 5;
    std::printf("ok: epilogue + shortcut + slot store within %.2f of the tolerance, folded pool exact\n", worst);
    return 0;
}

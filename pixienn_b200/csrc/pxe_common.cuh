// Shared helpers for the epilogue kernels: error reporting, launch sizing, exact integer
// division by launch-time constants, and the activation functions.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <cfloat>
#include <cmath>
#include <cstdarg>
#include <cstdio>

#include "pxe.h"

namespace pxe {

// ---------------------------------------------------------------- errors
int set_error(int status, const char* fmt, ...);

#define PXE_REQUIRE(cond, ...)                                            \
    do {                                                                  \
        if (!(cond)) return ::pxe::set_error(PXE_ERR_BAD_ARG, __VA_ARGS__); \
    } while (0)

#define PXE_CUDA_OK(expr)                                                             \
    do {                                                                              \
        cudaError_t e_ = (expr);                                                      \
        if (e_ != cudaSuccess)                                                        \
            return ::pxe::set_error(PXE_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

// Checks that the launch just issued was accepted (does not synchronise).
#define PXE_LAUNCH_OK(name)                                                           \
    do {                                                                              \
        cudaError_t e_ = cudaPeekAtLastError();                                       \
        if (e_ != cudaSuccess)                                                        \
            return ::pxe::set_error(PXE_ERR_CUDA, "launch %s: %s", name, cudaGetErrorString(e_)); \
    } while (0)

// ---------------------------------------------------------------- device info
struct DeviceInfo {
    int sm_count;
    int max_smem_optin;
};
// Immutable properties of the current device (cached per device).
int device_info(DeviceInfo* out);

// Grid size for a grid-stride kernel: enough blocks for `work_items` at
// `items_per_block`, capped at `waves` resident blocks per SM.
inline unsigned grid_for(long long work_items, int items_per_block, int sm_count, int blocks_per_sm)
{
    long long need = (work_items + items_per_block - 1) / items_per_block;
    long long cap = (long long)sm_count * blocks_per_sm;
    if (need < 1) need = 1;
    return (unsigned)(need < cap ? need : cap);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }

// ---------------------------------------------------------------- exact division
// Division of a 32-bit unsigned value by a constant fixed at launch time, as a
// multiply-high and a shift (round-up method; exact for every n < 2^32).
struct FastDiv {
    uint32_t d, mul, shift;
    FastDiv() : d(1), mul(0), shift(0) {}
    explicit FastDiv(uint32_t divisor) : d(divisor)
    {
        if (d <= 1) { d = 1; mul = 0; shift = 0; return; }
        uint32_t l = 0;
        while ((1ull << l) < d) ++l;            // l = ceil(log2 d)
        mul = (uint32_t)(((1ull << 32) * ((1ull << l) - d)) / d + 1);
        shift = l;
    }
    __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const
    {
#ifdef __CUDA_ARCH__
        if (d == 1) return n;
        uint32_t t = __umulhi(n, mul);
        return (uint32_t)(((uint64_t)t + n) >> shift);
#else
        return n / d;
#endif
    }
    __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const
    {
        q = div(n);
        r = n - q * d;
    }
};

// ---------------------------------------------------------------- activations
// Each function evaluates the same expression as the functor of the same name in the
// reference's include/Activation.h (precise math library, no fast-math), except mish, which
// uses an algebraically equal single-exponential form (see act_mish).

__device__ __forceinline__ float act_logistic(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ float act_softplus(float x)
{
    if (x > 20.0f) return x;
    if (x < -20.0f) return expf(x);
    return logf(expf(x) + 1.0f);
}

// mish(x) = x * tanh(softplus(x)) with one exponential instead of exp + log + tanh.
// With e = exp(x): tanh(log(1 + e)) = ((1+e)^2 - 1) / ((1+e)^2 + 1) = n / (n + 2), n = e*(e + 2),
// which has no cancellation.  The |x| > 20 branches are the reference's softplus branches: above
// 20 tanh(x) rounds to 1, below -20 tanh(exp(x)) rounds to exp(x).
//
// Distance from the reference's expression x * tanhf(logf(expf(x) + 1)): the reference rounds
// exp(x) + 1 to fp32 before the log, an absolute error of up to 2^-24 in softplus, i.e. up to
// |x| * 5.96e-8 in the result (the sum even rounds to exactly 1, giving mish = 0, for
// -20 <= x < -16.64).  That error is the reference's, not this form's; the two differ by at most
// 16.64 * 5.96e-8 = 9.9e-7 < 1e-6, attained near x = -16.64, and by a few ulp elsewhere.
__device__ __forceinline__ float act_mish(float x)
{
    if (x > 20.0f) return x;
    const float e = expf(x);
    if (x < -20.0f) return x * e;
    const float n = e * (e + 2.0f);
    return x * (n / (n + 2.0f));
}

// ---- hardware-approximate forms for the three transcendental activations the model presets use.
// exp(x) = ex2.approx(x * log2 e): relative error at most (2 + 1.17|x|) ulp; rcp.approx: 1 ulp.
// The .ftz forms are single MUFU instructions (the non-ftz ones carry denormal fix-up code): a
// subnormal exp() result or reciprocal flushes to zero, which only happens where the activation's
// value is below 1e-36 anyway.
// In the units of the parity tolerance (|err| <= 1e-6 + 1e-5 |ref|) the worst case over the whole
// input range is about 4 % of the tolerance: where |x| is large enough for the exponent's error to
// grow, the affected term is either negligible against 1 or the result is far below 1e-6.
__device__ __forceinline__ float fast_ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_rcp(float x)
{
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_exp(float x) { return fast_ex2(x * 1.4426950408889634f); }

__device__ __forceinline__ float act_logistic_fast(float x) { return fast_rcp(1.0f + fast_exp(-x)); }
__device__ __forceinline__ float act_swish_fast(float x) { return x * fast_rcp(1.0f + fast_exp(-x)); }
// Same n/(n+2) form as act_mish.  Below -20 it needs no branch (n/(n+2) -> e to within e/2
// relative); above 20 the select keeps exp() overflow (inf * 0) out of the result.
__device__ __forceinline__ float act_mish_fast(float x)
{
    const float e = fast_exp(x);
    const float n = e * (e + 2.0f);
    const float t = n * fast_rcp(n + 2.0f);
    return x > 20.0f ? x : x * t;
}

// FAST selects the hardware-approximate forms for logistic / swish / mish (the streaming
// epilogue kernels, where the precise forms are instruction-bound); everything else, and every
// decode that compares scores against a threshold, evaluates the reference's expressions with
// the precise math library.
template <int ACT, bool FAST = false>
__device__ __forceinline__ float activate(float x)
{
    if (ACT == PXE_ACT_LEAKY) return fmaxf(x, 0.1f * x);      // == (x > 0 ? x : 0.1f * x) for every x, NaN and -0 included
    if (ACT == PXE_ACT_LINEAR) return x;
    if (ACT == PXE_ACT_LOGGY) return 2.0f / (1.0f + expf(-x)) - 1.0f;
    if (ACT == PXE_ACT_LOGISTIC) return FAST ? act_logistic_fast(x) : act_logistic(x);
    if (ACT == PXE_ACT_MISH) return FAST ? act_mish_fast(x) : act_mish(x);
    if (ACT == PXE_ACT_RELU) return x > 0.0f ? x : 0.0f;
    if (ACT == PXE_ACT_SOFTPLUS) return act_softplus(x);
    if (ACT == PXE_ACT_SWISH) return FAST ? act_swish_fast(x) : x / (1.0f + expf(-x));
    if (ACT == PXE_ACT_TANH) return tanhf(x);
    return x;
}

__device__ __forceinline__ float activate_dyn(int act, float x)
{
    switch (act) {
    case PXE_ACT_LEAKY: return activate<PXE_ACT_LEAKY>(x);
    case PXE_ACT_LOGGY: return activate<PXE_ACT_LOGGY>(x);
    case PXE_ACT_LOGISTIC: return activate<PXE_ACT_LOGISTIC>(x);
    case PXE_ACT_MISH: return activate<PXE_ACT_MISH>(x);
    case PXE_ACT_RELU: return activate<PXE_ACT_RELU>(x);
    case PXE_ACT_SOFTPLUS: return activate<PXE_ACT_SOFTPLUS>(x);
    case PXE_ACT_SWISH: return activate<PXE_ACT_SWISH>(x);
    case PXE_ACT_TANH: return activate<PXE_ACT_TANH>(x);
    default: return x;
    }
}

inline bool valid_activation(int act)
{
    return act >= PXE_ACT_LEAKY && act <= PXE_ACT_TANH;
}

}  // namespace pxe

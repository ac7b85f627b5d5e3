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

// ---------------------------------------------------------------- global-memory accessors
// Every access of a kernel to global memory is written with one of these: gld / gst for an element of the pointer's
// own type, gldv<V> / gstv for a wider vector at an element pointer, gldg / gldgv<V> for the read-only path, and
// gcheck around an atomic.  In the ordinary build they are the plain dereference.  With -DPXE_BOUNDS_CHECK each
// one first looks the address up in the table of the caller's allocations (include/pxe_debug.h): an access
// outside every allocation, across the end of one, or misaligned for its width is skipped (loads give zeros) and
// recorded with the file and line of the access; the kernel runs to its end, nothing traps.
#ifdef PXE_BOUNDS_CHECK
constexpr int kBoundsMaxSpans = 4096;
struct BoundsTable {
    unsigned long long start[kBoundsMaxSpans];     // sorted
    unsigned long long end[kBoundsMaxSpans];
    int n;                                         // 0 = disarmed
    unsigned int violations;
    unsigned long long bad_address;
    int bad_bytes, bad_line, bad_store, bad_misaligned;
    char bad_file[48];
};
// One pointer per translation unit (the library is linked without relocatable device code); pxe_api.cu calls every
// unit's attach function when a table is installed.
static __device__ BoundsTable* tu_bounds_table = nullptr;
void bounds_register_unit(void (*attach)(BoundsTable*));
int bounds_add_internal(const void* p, size_t bytes);      // memory the library owns and its kernels reach through a pointer
namespace {
inline void bounds_attach_this_unit(BoundsTable* t) { cudaMemcpyToSymbol(tu_bounds_table, &t, sizeof(t)); }
struct BoundsRegistrar {
    BoundsRegistrar() { bounds_register_unit(&bounds_attach_this_unit); }
};
static BoundsRegistrar bounds_registrar;
}  // namespace

static __device__ __noinline__ bool bounds_ok(const void* p, unsigned bytes, unsigned align, bool store, int line, const char* file)
{
    BoundsTable* t = tu_bounds_table;
    if (t == nullptr || t->n <= 0 || !__isGlobal(p)) return true;
    const unsigned long long a = (unsigned long long)p;
    int lo = 0, hi = t->n;                         // first span that starts after a
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (t->start[mid] <= a) lo = mid + 1; else hi = mid;
    }
    const bool inside = lo > 0 && a + bytes <= t->end[lo - 1];
    const bool aligned = (a % align) == 0;
    if (inside && aligned) return true;
    if (atomicAdd(&t->violations, 1u) == 0) {
        t->bad_address = a; t->bad_bytes = (int)bytes; t->bad_line = line; t->bad_store = store; t->bad_misaligned = inside && !aligned;
        const char* base = file;
        for (const char* c = file; *c; ++c) if (*c == '/') base = c + 1;
        int k = 0;
        for (; k < 47 && base[k]; ++k) t->bad_file[k] = base[k];
        t->bad_file[k] = 0;
    }
    return false;
}
#define PXE_SITE , int line_ = __builtin_LINE(), const char* file_ = __builtin_FILE()
#define PXE_OK_LD(V) bounds_ok(p, sizeof(V), alignof(V), false, line_, file_)
#define PXE_OK_ST(V) bounds_ok(p, sizeof(V), alignof(V), true, line_, file_)
#else
#define PXE_SITE
#define PXE_OK_LD(V) true
#define PXE_OK_ST(V) true
#endif

template <typename T>
__device__ __forceinline__ T gld(const T* p PXE_SITE) { return PXE_OK_LD(T) ? *p : T{}; }
template <typename V, typename T>
__device__ __forceinline__ V gldv(const T* p PXE_SITE) { return PXE_OK_LD(V) ? *reinterpret_cast<const V*>(p) : V{}; }
template <typename T>
__device__ __forceinline__ T gldg(const T* p PXE_SITE) { return PXE_OK_LD(T) ? __ldg(p) : T{}; }
template <typename V, typename T>
__device__ __forceinline__ V gldgv(const T* p PXE_SITE) { return PXE_OK_LD(V) ? __ldg(reinterpret_cast<const V*>(p)) : V{}; }
template <typename T> struct same_type { using type = T; };
template <typename T>
__device__ __forceinline__ void gst(T* p, typename same_type<T>::type v PXE_SITE) { if (PXE_OK_ST(T)) *p = v; }
template <typename V, typename T>
__device__ __forceinline__ void gstv(T* p, const V& v PXE_SITE) { if (PXE_OK_ST(V)) *reinterpret_cast<V*>(p) = v; }
// Around an atomic or any other access the helpers above do not cover: true when `bytes` at p may be touched.
template <typename T>
__device__ __forceinline__ bool gcheck(T* p PXE_SITE) { return PXE_OK_ST(T); }
template <typename T>
__device__ __forceinline__ T gatomic_add(T* p, typename same_type<T>::type v PXE_SITE) { return PXE_OK_ST(T) ? atomicAdd(p, v) : T{}; }

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

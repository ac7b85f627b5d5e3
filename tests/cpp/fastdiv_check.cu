// Host program (compiled by nvcc, runs without a GPU): the multiply-high division every kernel indexes with
// (FastDiv in csrc/pxe_common.cuh) against the hardware division, with the constants the struct's own
// constructor computes and the device formula restated -- q = (umulhi(n, mul) + n) >> shift in 64 bits.
#include <cstdint>
#include <cstdio>
#include <random>
#include <vector>

#include "pxe_common.cuh"

static inline uint32_t device_formula(const pxe::FastDiv& f, uint32_t n)
{
    if (f.d == 1) return n;
    const uint32_t t = (uint32_t)(((uint64_t)n * f.mul) >> 32);
    return (uint32_t)(((uint64_t)t + n) >> f.shift);
}

int main()
{
    std::vector<uint32_t> divisors;
    for (uint32_t d = 1; d <= 5000; ++d) divisors.push_back(d);                 // every size a layer has
    for (int b = 12; b < 32; ++b)
        for (int k = -2; k <= 2; ++k) divisors.push_back((uint32_t)((1ull << b) + k));
    for (uint32_t d : {10816u, 43264u, 173056u, 369664u, 1478656u, 2147483647u, 4294967295u, 4294967291u, 3000000007u})
        divisors.push_back(d);
    std::mt19937 rng(12345);
    for (int i = 0; i < 2000; ++i) divisors.push_back(rng() | 1u);
    unsigned long long checked = 0;
    for (uint32_t d : divisors) {
        const pxe::FastDiv f(d);
        auto check = [&](uint32_t n) {
            ++checked;
            if (device_formula(f, n) != n / d) {
                std::printf("MISMATCH d=%u n=%u: %u != %u\n", d, n, device_formula(f, n), n / d);
                return false;
            }
            return true;
        };
        for (uint32_t n = 0; n < 3000; ++n) if (!check(n)) return 1;
        for (uint32_t n : {0xffffffffu, 0xfffffffeu, 0x80000000u, 0x7fffffffu, 0x80000001u}) if (!check(n)) return 1;
        for (int i = 0; i < 400; ++i) {                                          // around multiples of d
            const uint64_t k = (uint64_t)rng() % (0xffffffffull / d + 1);
            for (int e = -1; e <= 1; ++e) {
                const int64_t n = (int64_t)(k * d) + e;
                if (n >= 0 && n <= 0xffffffffll && !check((uint32_t)n)) return 1;
            }
        }
        for (int i = 0; i < 300; ++i) if (!check(rng())) return 1;
    }
    std::printf("ok: %zu divisors, %llu quotients\n", divisors.size(), checked);
    return 0;
}

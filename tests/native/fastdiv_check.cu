// Host-side check of the invariant division the kernels decode tile numbers with
// (reference_model_b200/csrc/rescale_math.cuh: fastdiv_make / fastdiv_apply) against the / operator: every divisor up to
// 70 000 with its boundary dividends, and seeded random (divisor, dividend) pairs over the whole 32-bit range.
// Compiled and run by tests/test_rescale_rec_cpu.py.
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "../../reference_model_b200/csrc/rescale_math.cuh"

using namespace tb200;

int main()
{
    long long bad = 0, checked = 0;
    uint64_t st = 12345;
    auto next = [&]() {
        st = st * 6364136223846793005ULL + 1442695040888963407ULL;
        return (uint32_t)(st >> 32);
    };
    for (uint32_t d = 1; d <= 70000; d++)
    {
        uint32_t md[2];
        fastdiv_make(d, md);
        const uint32_t probes[] = { 0u, 1u, d - 1, d, d + 1, 2 * d - 1, 2 * d, 3 * d + 7, 0x7fffffffu, 0xffffffffu };
        for (uint32_t n : probes)
        {
            bad += fastdiv_apply(n, md) != n / d;
            checked++;
        }
        for (int i = 0; i < 100; i++)
        {
            const uint32_t n = next();
            bad += fastdiv_apply(n, md) != n / d;
            checked++;
        }
    }
    for (int i = 0; i < 2000000; i++)
    {
        uint32_t d = next();
        if (d == 0)
            d = 1;
        if (i & 1)
            d >>= (next() & 31);
        if (d == 0)
            d = 1;
        const uint32_t n = next();
        uint32_t md[2];
        fastdiv_make(d, md);
        bad += fastdiv_apply(n, md) != n / d;
        checked++;
    }
    printf("checked=%lld mismatches=%lld\n", checked, bad);
    return bad != 0;
}

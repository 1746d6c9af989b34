// Host-side check of the lean RESCALE form (reference_model_b200/csrc/rescale_math.cuh: rescale_rec_build /
// rescale_rec_apply) against QuantUtil::apply_scale_32 restated in 64-bit arithmetic
// (reference_model/src/quant_util.h:45-84), plus the output zero point: seeded random and corner values over every
// shift, both rounding modes, and records that must come out unusable.  Compiled and run by tests/test_rescale_rec_cpu.py.
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "../../reference_model_b200/csrc/rescale_math.cuh"

using namespace tb200;

static int64_t apply_scale_32_ref(int32_t v, int32_t m, int32_t s, bool dr)
{
    int64_t round = (int64_t)1 << (s - 1);
    if (dr && s > 31)
        round += (v >= 0) ? ((int64_t)1 << 30) : -((int64_t)1 << 30);
    return ((int64_t)v * m + round) >> s;
}

static uint64_t state = 88172645463325252ULL;
static uint64_t rnd()
{
    state ^= state << 13;
    state ^= state >> 7;
    state ^= state << 17;
    return state;
}

int main(int argc, char** argv)
{
    const long iterations = argc > 1 ? atol(argv[1]) : 400000;
    long long bad = 0, checked = 0, unusable = 0;
    for (long it = 0; it < iterations; it++)
    {
        int32_t s = 2 + (int)(rnd() % 54);    // 2..55: 54 and 55 must be refused
        if (it % 3 == 0)
            s = 30 + (int)(rnd() % 11);       // the range quantized graphs use
        int32_t m = (int32_t)(rnd() & 0x7fffffff);
        if (it % 5 == 0)
            m = (int32_t)((1u << 30) + (rnd() % (1u << 30)));
        const bool dr      = rnd() & 1;
        const int32_t zp   = (int32_t)(rnd() % 256) - 128;
        const int32_t corr = (int32_t)(rnd() % (1u << 26)) - (1 << 25);
        // what the form can prove: |t| < 2^30 above shift 31; below, apply_scale_32's own limit 2^(shift-1), one bit less
        // when the layer rounds twice (the sign term is applied to every column and such a column is kept non-negative)
        const int bits     = (s <= 31) ? (dr ? s - 2 : s - 1) : 30;
        int64_t vmax       = ((int64_t)1 << bits) - 1;
        if (it % 7 == 0)
            vmax = (int64_t)1 << bits;    // one more than the form can prove: must be refused
        int32_t r8[8];
        rescale_rec_build(m, s, dr, zp, corr, vmax, r8);
        const bool expect_ok = s <= 53 && vmax < ((int64_t)1 << bits);
        if ((r8[7] != 0) != expect_ok)
        {
            bad++;
            if (bad < 10)
                printf("usable flag wrong: shift %d vmax %lld\n", s, (long long)vmax);
        }
        if (!r8[7])
        {
            unusable++;
            continue;
        }
        for (int j = 0; j < 8; j++)
        {
            int64_t t;
            switch (j)
            {
                case 0: t = vmax; break;
                case 1: t = -vmax; break;
                case 2: t = 0; break;
                case 3: t = -1; break;
                case 4: t = 1; break;
                default: t = (int64_t)(rnd() % (2 * (uint64_t)vmax + 1)) - vmax;
            }
            if (t > vmax || t < -vmax)
                continue;    // +-1 when the provable range is {0}
            // the kernel sees the raw accumulator; the correction rides on the record
            const int32_t acc = (int32_t)((uint32_t)(int32_t)t - (uint32_t)corr);
            const int32_t z   = rescale_rec_apply(acc, r8[0], r8[1], r8[2], r8[3], r8[4], r8[5], dr);
            const int64_t e   = apply_scale_32_ref((int32_t)t, m, s, dr) + zp;
            checked++;
            if ((int64_t)z != e)
            {
                bad++;
                if (bad < 10)
                    printf("MISMATCH t=%lld m=%d shift=%d dr=%d zp=%d corr=%d: got %d, want %lld\n", (long long)t, m, s, (int)dr, zp,
                           corr, z, (long long)e);
            }
        }
    }
    printf("checked=%lld unusable=%lld mismatches=%lld\n", checked, unusable, bad);
    return bad != 0;
}

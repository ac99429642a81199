// ref_inputs.cpp -- the input family of the reference's accuracy test, regenerated from its seeds.
//
// TEST INFRASTRUCTURE ONLY (see ozaki2_oracle.c). The reference's accuracy table (bench/ozaki_test.cu:27-32,41) fills
// A and B with normal(0,1) * 2^uniform(-spread, spread) from std::mt19937_64 seeded 1+K and 2+K, using libstdc++'s
// distributions; there are no stored vectors, so the published errors can only be reproduced by drawing the same
// numbers from the same library. This translation unit does exactly that and nothing else.
#include <cmath>
#include <cstddef>
#include <random>

extern "C" void oz_ref_fill(double *v, size_t n, double spread, unsigned seed) {
    std::mt19937_64 g(seed);
    std::normal_distribution<double> nd;
    std::uniform_real_distribution<double> u(-spread, spread);
    for (size_t i = 0; i < n; i++) v[i] = nd(g) * exp2(u(g));
}

// bench/dd_test.cu:25-34 of the reference: one generator seeded K + spread fills A then B, each value a full 106-bit
// double-double: hi = normal * 2^uniform(-spread, spread), lo = hi * 2^-54 * (2 u - 1) with u a 53-bit uniform.
extern "C" void oz_ref_fill_dd(double *Ah, double *Al, size_t na, double *Bh, double *Bl, size_t nb, double spread, unsigned seed) {
    std::mt19937_64 g(seed);
    std::normal_distribution<double> nd;
    std::uniform_real_distribution<double> u(-spread, spread);
    double *hi[2] = {Ah, Bh}, *lo[2] = {Al, Bl};
    const size_t n[2] = {na, nb};
    for (int t = 0; t < 2; t++)
        for (size_t i = 0; i < n[t]; i++) {
            hi[t][i] = nd(g) * exp2(u(g));
            lo[t][i] = hi[t][i] * 0x1p-54 * (2 * (g() >> 11) * 0x1p-53 - 1);
        }
}

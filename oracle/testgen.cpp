// testgen.cpp -- regenerates the seeded inputs of the reference's exact-equality GEMV
// tests (tests/test_sparse_ternary.cu:252-402): std::mt19937(seed), ternary weights from
// uniform_int_distribution(-1,1) drawn four at a time, a 2-of-4 mask from std::shuffle of
// {0,1,2,3} per group, then x from uniform_int_distribution(lo,hi).  The sequences depend
// on libstdc++'s distribution and shuffle algorithms, so the golden outputs under
// tests/golden/ were produced with the same toolchain.  TEST INFRASTRUCTURE ONLY.
#include <algorithm>
#include <cstdint>
#include <random>

extern "C" void testgen_gemv_case(unsigned seed, int rows, int cols, int xlo, int xhi,
                                  int8_t* weights, uint8_t* mask, int8_t* x) {
    const int total = rows * cols;
    std::mt19937 rng(seed);
    std::uniform_int_distribution<int> wdist(-1, 1);
    for (int i = 0; i < total; ++i) mask[i] = 0;
    for (int i = 0; i < total; i += 4) {
        for (int j = 0; j < 4; ++j) weights[i + j] = static_cast<int8_t>(wdist(rng));
        int idx[4] = {0, 1, 2, 3};
        std::shuffle(idx, idx + 4, rng);
        mask[i + idx[0]] = 1;
        mask[i + idx[1]] = 1;
    }
    std::uniform_int_distribution<int> xdist(xlo, xhi);
    for (int c = 0; c < cols; ++c) x[c] = static_cast<int8_t>(xdist(rng));
}

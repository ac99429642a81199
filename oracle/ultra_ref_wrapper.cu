// ultra_ref_wrapper.cu -- TEST INFRASTRUCTURE ONLY: exposes the reference's own host superaccumulator to the tests.
//
// The reference checks its exact BF16 x block-scaled FP8 products against a 2560-bit host accumulator that adds every
// product exactly and rounds once (llm/ultra.cu:336-369: Big, big_round, exact_dot; operand decoding llm/ultra.cu:45-62;
// activations llm/ultra.cu:165-174). This wrapper compiles that file where it lies (REF, never copied), with its main()
// renamed, and exports one C function around exact_dot for a single output. Built by oracle/Makefile into oracle/_ref/.
// Only host code of the reference runs through it: it needs no GPU.
#define main ozref_ultra_main_unused
#include "llm/ultra.cu"
#undef main

// One output of Y = X (W o S): w holds the K FP8 E4M3 codes of one weight row, s the K/128 BF16 block scales of that row
// (bit patterns), x the K activations as floats (BF16 values are floats); returns the exact sum rounded once to p bits.
extern "C" __attribute__((visibility("default"))) float ozref_exact_dot_e4m3b(const uint8_t *w, const uint16_t *s, int K, const float *x, int p) {
    DevW W{};
    W.fmt = F_E4M3B; W.M = 1; W.K = K; W.w = w; W.sw = reinterpret_cast<const uint8_t *>(s); W.Gm = 1; W.Ge = 0; W.Gf = 1.f;
    const std::vector<float> xv(x, x + K);
    const Act a = act_plain(xv);
    return exact_dot(W, 0, a, p);
}

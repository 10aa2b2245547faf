// C entry points around the reference demo's host-side sampling helpers -- TEST INFRASTRUCTURE ONLY.
//
// row_logsumexp and sample_row live in apps/04_gpt2_grpo.cu:61-80 of the reference, one
// translation unit with model code that is not in the tree, so that file cannot be compiled.  The
// two helpers themselves need only <algorithm>, <cmath> and <random>: oracle/Makefile (target
// ref-sample) cuts those lines out of the reference file at build time into
// _ref/sample_cut.inc, which is included below unmodified.  Nothing of the reference is stored in
// this repository; the object code exists only under oracle/_ref/.
#include <algorithm>
#include <cmath>
#include <random>

namespace {
#include "sample_cut.inc"
}  // namespace

extern "C" {

double grpo_ref_row_logsumexp(const float* row, int V) { return row_logsumexp(row, V); }

// n draws in a row from one std::mt19937 seeded with `seed`, as the demo draws its samples
// (apps/04_gpt2_grpo.cu:138-161: one generator, one sample_row call per response): rows[i] is a
// row index into logits[.][P].  tokens_out[i] is the drawn token.
void grpo_ref_sample_rows(const float* logits, int P, int V, const int* rows, int n, unsigned seed, int* tokens_out) {
    std::mt19937 rng(seed);
    for (int i = 0; i < n; i++) tokens_out[i] = sample_row(logits + static_cast<size_t>(rows[i]) * P, V, rng);
}

// The uniform numbers those n draws consume, in order: what a caller of the CUDA path passes as
// `coins` to reproduce the demo's tokens (the same distribution object type and generator).
void grpo_ref_coins(unsigned seed, int n, double* coins_out) {
    std::mt19937 rng(seed);
    for (int i = 0; i < n; i++) {
        std::uniform_real_distribution<double> uniform(0.0, 1.0);
        coins_out[i] = uniform(rng);
    }
}

}  // extern "C"

// Host-side validation shared by the reference-facing calls (host_api.cu) and the token-sharded
// host call (sharded_host.cu): the reference's messages, in the reference's order
// (src/cuda/grpo_loss_cuda.cu:584-618, 662-724; include/grpo/grpo_loss.hpp:51-67).
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

#include "grpo_b200.h"

namespace grpo_b200 {
namespace host {

struct Shape {
    size_t sequences = 0, tokens = 0;
};
struct Options {
    float clip_eps, beta, alpha;
    int reduction;
};

int invalid(const std::string& msg);
int nonfinite(const char* msg);
int checked_shape(int B, int G, int T, Shape& out);
int expect_size(const char* name, size_t got, size_t want);
int check_options(const Options& o);
// options, then the sizes of the token arrays, in the reference's order (the first part of validate_inputs)
int validate_sizes(bool has_new, size_t n_new, size_t n_old, size_t n_ref, size_t n_adv, size_t n_mask,
                   const Shape& shape, const Options& opt);
// token-array checks; logp_new may be null (the logits calls have none)
int validate_inputs(const float* lp_new, size_t n_new, const float* lp_old, size_t n_old, const float* lp_ref,
                    size_t n_ref, const float* adv, size_t n_adv, const int32_t* mask, size_t n_mask,
                    const Shape& shape, const Options& opt);
// 1 and the index of the first active row whose selected id lies outside [0, V), else 0
int check_selected(const int32_t* selected, const int32_t* mask, size_t n, int V, size_t& first_bad);
// loss/pg/kl of a device record into floats; negative bad_inputs and non-finite sums become errors
int fill_stats(const grpo_b200_result_t& r, float* stats, const char* what);


// ---- one-pass copy-and-check loops of the host entries (each vectorises: restrict pointers, no branches)
// copy n words and report whether any of them is an infinity or a NaN (one vectorised loop)
inline unsigned copy_and_check_finite(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, size_t n) {
    unsigned bad = 0;
    for (size_t i = 0; i < n; i++) {
        const uint32_t b = src[i];
        bad |= (b & 0x7f800000u) == 0x7f800000u;
        dst[i] = b;
    }
    return bad;
}
// copy the selected ids and report whether an active row's id lies outside [0, V)
inline unsigned copy_and_check_selected(const int32_t* __restrict__ sel, const int32_t* __restrict__ mask,
                                 int32_t* __restrict__ dst, size_t n, uint32_t vocab) {
    unsigned bad = 0;
    for (size_t i = 0; i < n; i++) {
        const int32_t v = sel[i];
        bad |= (mask[i] != 0) & (static_cast<uint32_t>(v) >= vocab);
        dst[i] = v;
    }
    return bad;
}
// copy one response's mask, count its valid tokens and report values outside {0, 1}
inline unsigned copy_and_count_mask(const int32_t* __restrict__ src, int32_t* __restrict__ dst, int T, int& count) {
    unsigned bad = 0;
    int c = 0;
    for (int t = 0; t < T; t++) {
        const int32_t v = src[t];
        bad |= static_cast<uint32_t>(v) > 1u;
        c += v != 0;
        dst[t] = v;
    }
    count = c;
    return bad;
}

}  // namespace host
}  // namespace grpo_b200

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

}  // namespace host
}  // namespace grpo_b200

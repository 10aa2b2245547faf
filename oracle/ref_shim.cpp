// C entry points around the reference's own CPU functions -- TEST INFRASTRUCTURE ONLY.
//
// This file is compiled together with the reference's src/cpu/grpo_loss.cpp,
// taken from the reference tree where it lies, into oracle/_ref/libgrpo_ref.so
// (see the Makefile beside it).  The shim adds no arithmetic: it builds the
// std::vector arguments, calls grpo::group_advantages_cpu / grpo_loss_cpu /
// grpo_logits_cpu (include/grpo/grpo_loss.hpp:78-110 of the reference) and
// turns a std::runtime_error into return code -1 plus a retrievable message.
// The library is used to validate the C restatement in grpo_oracle.c, to
// generate the golden vectors under tests/golden/, and as the timed CPU
// baseline of the benchmark.
#include "grpo/grpo_loss.hpp"

#include <cstring>
#include <exception>
#include <string>
#include <vector>

namespace {
thread_local std::string g_last_error;

grpo::LossConfig make_config(float clip_eps, float beta, int reduction, float alpha) {
    grpo::LossConfig cfg;
    cfg.clip_eps = clip_eps;
    cfg.beta = beta;
    cfg.reduction = static_cast<grpo::ReductionMode>(reduction);
    cfg.length_alpha = alpha;
    return cfg;
}

// Element counts to copy from the caller's arrays; 0 when the dims are ones the reference
// rejects before it looks at any array (non-positive, or a product beyond INT_MAX).
void counts(int B, int G, int T, size_t& n_seq, size_t& n_tok) {
    n_seq = n_tok = 0;
    if (B <= 0 || G <= 0 || T <= 0) return;
    size_t s = static_cast<size_t>(B) * static_cast<size_t>(G);
    if (s > 2147483647u || s * static_cast<size_t>(T) > 2147483647u) return;
    n_seq = s;
    n_tok = s * static_cast<size_t>(T);
}

template <class F>
int guarded(F&& body) {
    try {
        body();
        g_last_error.clear();
        return 0;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return -1;
    }
}
}  // namespace

extern "C" {

const char* grpo_ref_last_error() { return g_last_error.c_str(); }

int grpo_ref_group_advantages(const float* rewards, int B, int G, int mode, float eps,
                              float* advantages_out) {
    return guarded([&] {
        size_t n, unused;
        counts(B, G, 1, n, unused);
        std::vector<float> r(rewards, rewards + n);
        auto a = grpo::group_advantages_cpu(r, B, G, static_cast<grpo::AdvantageMode>(mode), eps);
        std::memcpy(advantages_out, a.data(), a.size() * sizeof(float));
    });
}

int grpo_ref_loss(const float* logp_new, const float* logp_old, const float* logp_ref,
                  const float* advantages, const int* mask, int B, int G, int T,
                  float clip_eps, float beta, int reduction, float alpha,
                  float* dlogp_out, float* stats_out, int* valid_tokens_out) {
    return guarded([&] {
        size_t s, n;
        counts(B, G, T, s, n);
        std::vector<float> a(logp_new, logp_new + n), b(logp_old, logp_old + n),
            c(logp_ref, logp_ref + n), adv(advantages, advantages + s);
        std::vector<int> m(mask, mask + n);
        auto r = grpo::grpo_loss_cpu(a, b, c, adv, m, B, G, T,
                                     make_config(clip_eps, beta, reduction, alpha));
        std::memcpy(dlogp_out, r.dlogp_new.data(), r.dlogp_new.size() * sizeof(float));
        stats_out[0] = r.stats.loss;
        stats_out[1] = r.stats.pg_loss;
        stats_out[2] = r.stats.kl;
        *valid_tokens_out = r.stats.valid_tokens;
    });
}

int grpo_ref_logits(const float* logits, const float* logp_old, const float* logp_ref,
                    const int* selected, const float* advantages, const int* mask,
                    int B, int G, int T, int V,
                    float clip_eps, float beta, int reduction, float alpha,
                    float* dlogits_out, float* stats_out, int* valid_tokens_out) {
    return guarded([&] {
        size_t s, n;
        counts(B, G, T, s, n);
        size_t nv = V > 0 ? n * V : 0;
        std::vector<float> x(logits, logits + nv), b(logp_old, logp_old + n),
            c(logp_ref, logp_ref + n), adv(advantages, advantages + s);
        std::vector<int> sel(selected, selected + n), m(mask, mask + n);
        auto r = grpo::grpo_logits_cpu(x, b, c, sel, adv, m, B, G, T, V,
                                       make_config(clip_eps, beta, reduction, alpha));
        std::memcpy(dlogits_out, r.dlogits.data(), r.dlogits.size() * sizeof(float));
        stats_out[0] = r.stats.loss;
        stats_out[1] = r.stats.pg_loss;
        stats_out[2] = r.stats.kl;
        *valid_tokens_out = r.stats.valid_tokens;
    });
}

}  // extern "C"

// Public option and result types of the GRPO loss boundary, source-compatible with the
// reference's include/grpo/grpo_loss.hpp (types at :10-43, shape guard at :46-67, index helpers at
// :70-76, CPU entry points at :78-117) so that code written against the reference compiles unchanged
// against this header.
//
// The three CPU functions at the bottom are DECLARED here, with the reference's signatures, and
// defined by the reference's own grpo_cpu library (src/cpu/grpo_loss.cpp), which a caller that uses
// them keeps linking exactly as the reference's build does (CMakeLists.txt:46-48 links grpo_cpu into
// grpo_cuda's users).  This library defines none of them: it has no CPU compute path.
#pragma once

#include <climits>
#include <cstddef>
#include <stdexcept>
#include <vector>

namespace grpo {

// How rewards inside one prompt's group become advantages.
enum class AdvantageMode { standardized, centered };

// How per-token terms are weighted into the scalar loss:
//   sequence_mean    each response weighs 1/S, its tokens share that equally
//   token_mean       every valid token of the batch weighs 1/(number of valid tokens)
//   length_weighted  a response of L valid tokens weighs L^alpha / S, shared equally by its tokens
enum class ReductionMode { sequence_mean, token_mean, length_weighted };

struct LossConfig {
    float clip_eps = 0.2f;  // PPO clip half-width, in [0, 1)
    float beta = 0.0f;      // weight of the KL term against the fixed reference policy, >= 0
    ReductionMode reduction = ReductionMode::sequence_mean;
    float length_alpha = 0.0f;  // exponent of length_weighted, in [0, 1]
};

struct LossStats {
    float loss = 0.0f;     // pg_loss + beta * kl
    float pg_loss = 0.0f;  // clipped policy-gradient surrogate
    float kl = 0.0f;       // k3 estimate of KL(new || reference) on the sampled tokens
    int valid_tokens = 0;  // number of mask == 1 tokens
};

struct LossResult {
    LossStats stats;
    std::vector<float> dlogp_new;  // dL/dlogp per token slot, 0 where masked
};

struct LogitsLossResult {
    LossStats stats;
    std::vector<float> dlogits;  // dL/dlogits, [B*G*T][V]
};

namespace detail {
struct Shape {
    std::size_t sequences;
    std::size_t tokens;
};

// B*G responses and B*G*T token slots, both of which must fit an int.
inline Shape checked_shape(int B, int G, int T) {
    if (B <= 0 || G <= 0 || T <= 0) throw std::runtime_error("B, G and T must be positive");
    const std::size_t limit = static_cast<std::size_t>(INT_MAX);
    const std::size_t sequences = static_cast<std::size_t>(B) * static_cast<std::size_t>(G);
    if (sequences > limit) throw std::runtime_error("sequence count exceeds INT_MAX");
    const std::size_t tokens = sequences * static_cast<std::size_t>(T);
    if (tokens > limit) throw std::runtime_error("token count exceeds INT_MAX");
    return {sequences, tokens};
}
}  // namespace detail

// Row-major positions in the [B][G] and [B][G][T] layouts.
inline std::size_t idx2(int b, int g, int G) { return static_cast<std::size_t>(b) * G + g; }
inline std::size_t idx3(int b, int g, int t, int G, int T) { return idx2(b, g, G) * T + t; }

// Defined by the reference's grpo_cpu library, not by this one (see the note at the top).
std::vector<float> group_advantages_cpu(const std::vector<float>& rewards, int B, int G,
                                        AdvantageMode mode = AdvantageMode::standardized, float eps = 1e-8f);
LossResult grpo_loss_cpu(const std::vector<float>& logp_new, const std::vector<float>& logp_old,
                         const std::vector<float>& logp_ref, const std::vector<float>& advantages,
                         const std::vector<int>& mask, int B, int G, int T, LossConfig config = {});
LogitsLossResult grpo_logits_cpu(const std::vector<float>& logits_new, const std::vector<float>& logp_old,
                                 const std::vector<float>& logp_ref, const std::vector<int>& selected_tokens,
                                 const std::vector<float>& advantages, const std::vector<int>& mask, int B, int G,
                                 int T, int V, LossConfig config = {});

}  // namespace grpo

// Times the REFERENCE's own CUDA library (src/cuda/grpo_loss_cuda.cu, compiled where it lies for
// sm_100a) on the benchmark configurations, through its own timing entry points and protocol
// (benchmark_grpo_loss_cuda: median of 7 repeats; benchmark_grpo_logits_cuda: medians of 15
// alternating samples, separate input and output buffers) -- TEST/BASELINE INFRASTRUCTURE ONLY.
// This file is a driver over the reference's public API; it contains none of the reference's code.
//
//   ref_cuda_timer v32k | v128k_a0.5 | v128k_a1.0 | cfg2_1M | cfg2_4M | cfg2_1M_ragged | cfg2_4M_ragged
//
// Prints one JSON object per run.  Inputs are seeded and have the configurations' shapes and
// value ranges; their exact values do not matter for a timing.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "grpo/grpo_loss_cuda.cuh"

namespace {

struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ULL + 1) {}
    uint64_t next() {
        s += 0x9E3779B97F4A7C15ULL;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
        return z ^ (z >> 31);
    }
    double uniform() { return (next() >> 11) * (1.0 / 9007199254740992.0); }
    // sum of four 16-bit fields, centred and scaled to unit variance: close enough to normal here
    float normalish() {
        const uint64_t h = next();
        const int k = int(h & 0xffff) + int((h >> 16) & 0xffff) + int((h >> 32) & 0xffff) + int(h >> 48) - 131070;
        return float(k * (1.0 / 37837.23));
    }
    int below(int n) { return int(next() % uint64_t(n)); }
};

std::vector<int> prefix_mask(const std::vector<int>& lengths, int T) {
    std::vector<int> mask(lengths.size() * size_t(T), 0);
    for (size_t s = 0; s < lengths.size(); s++)
        for (int t = 0; t < lengths[s]; t++) mask[s * T + t] = 1;
    return mask;
}

int run_logits(const char* name, int B, int G, int T, int V, bool ragged, grpo::ReductionMode reduction, float alpha) {
    Rng rng(42);
    const int S = B * G;
    const size_t N = size_t(S) * T;
    std::vector<int> lengths(S, T);
    if (ragged)
        for (auto& L : lengths) L = 16 + rng.below(T - 16 + 1);
    std::vector<int> mask = prefix_mask(lengths, T);
    std::vector<float> logits(N * V);
    for (auto& x : logits) x = 2.0f * rng.normalish();
    std::vector<int> selected(N);
    std::vector<float> old(N), ref(N), adv(S);
    const float typical = -std::log(float(V)) - 2.0f;  // about what a random token's log-probability is
    for (size_t i = 0; i < N; i++) {
        selected[i] = mask[i] ? rng.below(V) : -1;
        old[i] = mask[i] ? typical + 0.05f * rng.normalish() : 0.0f;
        ref[i] = mask[i] ? typical + 0.05f * rng.normalish() : 0.0f;
    }
    for (auto& a : adv) a = rng.uniform() < 0.5 ? 1.0f : -1.0f;
    grpo::LossConfig config;
    config.clip_eps = 0.2f;
    config.beta = 0.01f;
    config.reduction = reduction;
    config.length_alpha = alpha;
    const auto t = grpo::benchmark_grpo_logits_cuda(logits, old, ref, selected, adv, mask, B, G, T, V, config, 3, 10);
    size_t active = 0;
    for (int m : mask) active += m != 0;
    std::printf("{\"config\": \"%s\", \"rows\": %zu, \"V\": %d, \"active_rows\": %zu, \"separate_ms\": %.6f, "
                "\"fused_ms\": %.6f, \"protocol\": \"reference benchmark_grpo_logits_cuda: separate in/out buffers, "
                "10 back-to-back passes per sample, median of 15 alternating samples\"}\n",
                name, N, V, active, t.separate_ms, t.fused_ms);
    return 0;
}

int run_loss(const char* name, int B, int G, int T, bool ragged) {
    Rng rng(42);
    const int S = B * G;
    const size_t N = size_t(S) * T;
    std::vector<int> lengths(S, T);
    if (ragged)
        for (auto& L : lengths) L = 1 + rng.below(T);
    std::vector<int> mask = prefix_mask(lengths, T);
    std::vector<float> now(N), old(N), ref(N), adv(S);
    for (size_t i = 0; i < N; i++) {
        now[i] = float(std::log(0.01 + 0.99 * rng.uniform()));
        old[i] = now[i] + 0.02f * rng.normalish();
        ref[i] = now[i] + 0.05f * rng.normalish();
    }
    for (auto& a : adv) a = rng.normalish();
    grpo::LossConfig config;
    config.clip_eps = 0.2f;
    config.beta = 0.01f;
    config.reduction = grpo::ReductionMode::sequence_mean;
    const auto t = grpo::benchmark_grpo_loss_cuda(now, old, ref, adv, mask, B, G, T, config, 5, 20);
    size_t active = 0;
    for (int m : mask) active += m != 0;
    std::printf("{\"config\": \"%s\", \"tokens\": %zu, \"active_tokens\": %zu, \"atomic_ms\": %.6f, \"block_ms\": %.6f, "
                "\"protocol\": \"reference benchmark_grpo_loss_cuda: 20 back-to-back passes per repeat, median of 7\"}\n",
                name, N, active, t.atomic_ms, t.block_ms);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    int rc = 0;
    for (int i = 1; i < argc; i++) {
        const std::string c = argv[i];
        if (c == "v32k") rc |= run_logits("v32k", 2, 8, 64, 32768, false, grpo::ReductionMode::token_mean, 0.0f);
        else if (c == "v128k_a0.5") rc |= run_logits("v128k_a0.5", 2, 8, 64, 131072, true, grpo::ReductionMode::length_weighted, 0.5f);
        else if (c == "v128k_a1.0") rc |= run_logits("v128k_a1.0", 2, 8, 64, 131072, true, grpo::ReductionMode::length_weighted, 1.0f);
        else if (c == "cfg2_1M") rc |= run_loss("cfg2_1M", 512, 8, 256, false);
        else if (c == "cfg2_1M_ragged") rc |= run_loss("cfg2_1M_ragged", 512, 8, 256, true);
        else if (c == "cfg2_4M") rc |= run_loss("cfg2_4M", 512, 8, 1024, false);
        else if (c == "cfg2_4M_ragged") rc |= run_loss("cfg2_4M_ragged", 512, 8, 1024, true);
        else {
            std::fprintf(stderr, "unknown configuration %s\n", c.c_str());
            return 2;
        }
    }
    return rc;
}

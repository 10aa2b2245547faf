// namespace grpo entry points: std::vector in, structs out, exceptions for the reference's throw
// sites.  Pure forwarding to the host layer of the C ABI; no arithmetic happens here.
#include <cstdio>
#include <cstdlib>
#include <stdexcept>

#include "grpo/grpo_loss_cuda.cuh"
#include "grpo_b200.h"

namespace grpo {
namespace {

// Reference behaviour per failure class: throw for its throw sites, print-and-exit for CUDA
// runtime failures (include/grpo/cuda_utils.cuh:8-16 of the reference).
void raise(int status) {
    if (status == GRPO_B200_OK) return;
    if (status == GRPO_B200_E_CUDA) {
        std::fprintf(stderr, "%s\n", grpo_b200_last_error());
        std::exit(1);
    }
    throw std::runtime_error(grpo_b200_last_error());
}

static_assert(sizeof(int) == sizeof(int32_t), "mask and token ids are passed as int32");

}  // namespace

LossResult grpo_loss_cuda(const std::vector<float>& logp_new, const std::vector<float>& logp_old,
                          const std::vector<float>& logp_ref, const std::vector<float>& advantages,
                          const std::vector<int>& mask, int B, int G, int T, LossConfig config,
                          CudaLossKernel kernel) {
    LossResult out;
    // Size the output only for shapes the call will accept; anything else throws below.
    if (B > 0 && G > 0 && T > 0 && logp_new.size() == static_cast<size_t>(B) * G * T)
        out.dlogp_new.assign(logp_new.size(), 0.0f);
    float stats[3] = {0.0f, 0.0f, 0.0f};
    raise(grpo_b200_loss_host(logp_new.data(), logp_new.size(), logp_old.data(), logp_old.size(), logp_ref.data(),
                              logp_ref.size(), advantages.data(), advantages.size(), mask.data(), mask.size(), B, G,
                              T, config.clip_eps, config.beta, static_cast<int>(config.reduction),
                              config.length_alpha, static_cast<int>(kernel), out.dlogp_new.data(), stats,
                              &out.stats.valid_tokens));
    out.stats.loss = stats[0];
    out.stats.pg_loss = stats[1];
    out.stats.kl = stats[2];
    return out;
}

CudaTiming benchmark_grpo_loss_cuda(const std::vector<float>& logp_new, const std::vector<float>& logp_old,
                                    const std::vector<float>& logp_ref, const std::vector<float>& advantages,
                                    const std::vector<int>& mask, int B, int G, int T, LossConfig config,
                                    int warmup, int iterations) {
    CudaTiming t;
    raise(grpo_b200_benchmark_loss_host(logp_new.data(), logp_new.size(), logp_old.data(), logp_old.size(),
                                        logp_ref.data(), logp_ref.size(), advantages.data(), advantages.size(),
                                        mask.data(), mask.size(), B, G, T, config.clip_eps, config.beta,
                                        static_cast<int>(config.reduction), config.length_alpha, warmup, iterations,
                                        &t.atomic_ms, &t.block_ms));
    return t;
}

LogitsLossResult grpo_logits_cuda(const std::vector<float>& logits_new, const std::vector<float>& logp_old,
                                  const std::vector<float>& logp_ref, const std::vector<int>& selected_tokens,
                                  const std::vector<float>& advantages, const std::vector<int>& mask, int B, int G,
                                  int T, int V, LossConfig config, CudaLogitsKernel kernel) {
    LogitsLossResult out;
    if (B > 0 && G > 0 && T > 0 && V > 0 && logits_new.size() == static_cast<size_t>(B) * G * T * V)
        out.dlogits.resize(logits_new.size());
    float stats[3] = {0.0f, 0.0f, 0.0f};
    raise(grpo_b200_logits_host(logits_new.data(), logits_new.size(), logp_old.data(), logp_old.size(),
                                logp_ref.data(), logp_ref.size(), selected_tokens.data(), selected_tokens.size(),
                                advantages.data(), advantages.size(), mask.data(), mask.size(), B, G, T, V,
                                config.clip_eps, config.beta, static_cast<int>(config.reduction),
                                config.length_alpha, static_cast<int>(kernel), out.dlogits.data(), stats,
                                &out.stats.valid_tokens));
    out.stats.loss = stats[0];
    out.stats.pg_loss = stats[1];
    out.stats.kl = stats[2];
    return out;
}

LossStats grpo_logits_cuda_device_inplace(float* logits_and_dlogits, const std::vector<float>& logp_old,
                                          const std::vector<float>& logp_ref,
                                          const std::vector<int>& selected_tokens,
                                          const std::vector<float>& advantages, const std::vector<int>& mask,
                                          int B, int G, int T, int V, int P, LossConfig config,
                                          CudaLogitsKernel kernel) {
    LossStats out;
    float stats[3] = {0.0f, 0.0f, 0.0f};
    raise(grpo_b200_logits_device_inplace_host(
        logits_and_dlogits, logp_old.data(), logp_old.size(), logp_ref.data(), logp_ref.size(),
        selected_tokens.data(), selected_tokens.size(), advantages.data(), advantages.size(), mask.data(),
        mask.size(), B, G, T, V, P, config.clip_eps, config.beta, static_cast<int>(config.reduction),
        config.length_alpha, static_cast<int>(kernel), stats, &out.valid_tokens));
    out.loss = stats[0];
    out.pg_loss = stats[1];
    out.kl = stats[2];
    return out;
}

CudaLogitsTiming benchmark_grpo_logits_cuda(const std::vector<float>& logits_new,
                                            const std::vector<float>& logp_old,
                                            const std::vector<float>& logp_ref,
                                            const std::vector<int>& selected_tokens,
                                            const std::vector<float>& advantages, const std::vector<int>& mask,
                                            int B, int G, int T, int V, LossConfig config, int warmup,
                                            int iterations) {
    CudaLogitsTiming t;
    raise(grpo_b200_benchmark_logits_host(logits_new.data(), logits_new.size(), logp_old.data(), logp_old.size(),
                                          logp_ref.data(), logp_ref.size(), selected_tokens.data(),
                                          selected_tokens.size(), advantages.data(), advantages.size(), mask.data(),
                                          mask.size(), B, G, T, V, config.clip_eps, config.beta,
                                          static_cast<int>(config.reduction), config.length_alpha, warmup,
                                          iterations, &t.separate_ms, &t.fused_ms));
    return t;
}

}  // namespace grpo

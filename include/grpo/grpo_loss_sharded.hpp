// C++ face of the token-sharded logits boundary: one object per rank, the reference's types and
// exceptions.  Header-only over the C ABI of grpo_b200.h.
//
// The reference has no sharded loss call: its two-GPU demos shard whole responses and average on
// the host (apps/03_two_gpu_train.cu:200-215, 247-281) or keep replicas (apps/05_two_gpu_gpt2_grpo.cu).
// ShardedLogitsBoundary::run has the argument meaning and error behaviour of
// grpo::grpo_logits_cuda_device_inplace (include/grpo/grpo_loss_cuda.cuh:68-86) for one rank's rows
// of the batch, and returns the GLOBAL statistics.  Usable from one host thread per device of one
// process (connect) and from one process per device (handle / connect_ipc).
#pragma once

#include <array>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <vector>

#include "grpo/grpo_loss_cuda.cuh"
#include "grpo_b200.h"

namespace grpo {

class ShardedLogitsBoundary {
public:
    using Handle = std::array<unsigned char, 64>;

    // Rows [row_offset, row_offset + n_rows) of a batch of B*G responses of T token slots each, on the
    // current device.  Every rank of `world` makes one.
    ShardedLogitsBoundary(int rank, int world, int B, int G, int T, int V, int P, long long row_offset, long long n_rows)
        : world_(world), n_rows_(n_rows), sequences_(static_cast<long long>(B) * G) {
        if (B <= 0 || G <= 0 || T <= 0) throw std::runtime_error("B, G and T must be positive");
        raise(grpo_b200_shard_create(rank, world, sequences_, T, V, P, row_offset, n_rows, &shard_));
    }
    ~ShardedLogitsBoundary() { grpo_b200_shard_destroy(shard_); }
    ShardedLogitsBoundary(const ShardedLogitsBoundary&) = delete;
    ShardedLogitsBoundary& operator=(const ShardedLogitsBoundary&) = delete;

    // one process per device: trade these 64 bytes, then pass all ranks' handles in rank order
    Handle handle() const {
        Handle h{};
        raise(grpo_b200_shard_export(shard_, h.data()));
        return h;
    }
    void connect_ipc(const std::vector<Handle>& handles) {
        if (static_cast<int>(handles.size()) != world_) throw std::runtime_error("one handle per rank, in rank order");
        std::vector<unsigned char> flat;
        for (const Handle& h : handles) flat.insert(flat.end(), h.begin(), h.end());
        raise(grpo_b200_shard_connect_ipc(shard_, flat.data()));
    }
    // one host thread per device in one process: every rank's object, in rank order, after all were made
    void connect(const std::vector<ShardedLogitsBoundary*>& all) {
        if (static_cast<int>(all.size()) != world_) throw std::runtime_error("one boundary per rank, in rank order");
        std::vector<grpo_b200_shard_t> shards;
        for (const ShardedLogitsBoundary* b : all) shards.push_back(b ? b->shard_ : nullptr);
        raise(grpo_b200_shard_connect_local(shard_, shards.data()));
    }

    // This rank's metadata (n_rows entries; advantages: one per response of the whole batch) and its
    // device logits [n_rows][P], replaced in place by dL/dlogits.  Returns the global statistics.
    LossStats run(float* logits_and_dlogits, const std::vector<float>& logp_old, const std::vector<float>& logp_ref,
                  const std::vector<int>& selected_tokens, const std::vector<float>& advantages,
                  const std::vector<int>& mask, LossConfig config = {},
                  CudaLogitsKernel kernel = CudaLogitsKernel::fused) {
        float stats[3] = {0.0f, 0.0f, 0.0f};
        LossStats out;
        raise(grpo_b200_logits_sharded_host(shard_, logits_and_dlogits, logp_old.data(), logp_old.size(), logp_ref.data(),
                                            logp_ref.size(), selected_tokens.data(), selected_tokens.size(),
                                            advantages.data(), advantages.size(), mask.data(), mask.size(),
                                            config.clip_eps, config.beta, static_cast<int>(config.reduction),
                                            config.length_alpha, static_cast<int>(kernel), stats, &out.valid_tokens));
        out.loss = stats[0];
        out.pg_loss = stats[1];
        out.kl = stats[2];
        return out;
    }

private:
    // the reference's behaviour per failure class: throw for its throw sites, print and exit for CUDA
    // runtime failures (include/grpo/cuda_utils.cuh:8-16) -- except a timed-out exchange, which a
    // caller may want to survive and which therefore throws too
    static void raise(int status) {
        if (status == GRPO_B200_OK) return;
        throw std::runtime_error(grpo_b200_last_error());
    }

    grpo_b200_shard_t shard_ = nullptr;
    int world_;
    long long n_rows_;
    long long sequences_;
};

}  // namespace grpo

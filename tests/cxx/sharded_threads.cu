// One host thread per device, each with its own cudaSetDevice, calling the token-sharded logits
// boundary on its rows of one batch -- the reference's thread-per-device pattern
// (apps/03_two_gpu_train.cu:200-215) -- checked against the single-device call on the whole batch.
//
//   sharded_threads <world>      exit 0: ok, 77: fewer devices than ranks (skipped), 1: failed
//
// Kernels of different ranks wait on one another, so every rank needs a device of its own.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "grpo/grpo_loss_sharded.hpp"

namespace {

struct Batch {
    int B = 2, G = 4, T = 16, V = 8191, P = 8192;
    std::vector<float> logits, old, ref, adv;
    std::vector<int> sel, mask;
    int S() const { return B * G; }
    int N() const { return B * G * T; }
};

float unit(unsigned long long& s) {  // in [0, 1)
    s = s * 6364136223846793005ULL + 1442695040888963407ULL;
    return static_cast<float>((s >> 40) * (1.0 / 16777216.0));
}

Batch make_batch(unsigned long long seed, bool empty_response) {
    Batch b;
    unsigned long long s = seed;
    b.logits.assign(static_cast<size_t>(b.N()) * b.P, 123.0f);  // the padded tail holds a sentinel
    b.old.resize(b.N());
    b.ref.resize(b.N());
    b.sel.resize(b.N());
    b.mask.assign(b.N(), 0);
    b.adv.resize(b.S());
    for (int q = 0; q < b.S(); q++) {
        b.adv[q] = q % 3 == 0 ? 0.0f : (q % 2 ? 0.7f : -0.4f);
        int len = 1 + static_cast<int>(unit(s) * b.T);
        if (len > b.T) len = b.T;
        if (empty_response && q == 3) len = 0;
        for (int t = 0; t < len; t++) b.mask[q * b.T + t] = 1;
    }
    const float typical = -std::log(static_cast<float>(b.V)) - 1.0f;
    for (int i = 0; i < b.N(); i++) {
        for (int v = 0; v < b.V; v++) b.logits[static_cast<size_t>(i) * b.P + v] = 6.0f * unit(s) - 3.0f;
        b.sel[i] = b.mask[i] ? static_cast<int>(unit(s) * b.V) % b.V : -1;
        b.old[i] = b.mask[i] ? typical + 0.1f * unit(s) : 0.0f;
        b.ref[i] = b.mask[i] ? typical + 0.1f * unit(s) : 0.0f;
    }
    return b;
}

#define CK(x)                                                                        \
    do {                                                                             \
        cudaError_t e__ = (x);                                                       \
        if (e__ != cudaSuccess) {                                                    \
            std::fprintf(stderr, "CUDA: %s (%s)\n", cudaGetErrorString(e__), #x);    \
            std::exit(1);                                                            \
        }                                                                            \
    } while (0)

struct SpinBarrier {  // host threads line up here (between steps, nothing in flight on the devices that waits)
    std::atomic<int> count{0}, generation{0};
    int n;
    explicit SpinBarrier(int n_) : n(n_) {}
    void wait() {
        const int gen = generation.load();
        if (count.fetch_add(1) + 1 == n) {
            count.store(0);
            generation.fetch_add(1);
        } else {
            while (generation.load() == gen) std::this_thread::yield();
        }
    }
};

}  // namespace

int main(int argc, char** argv) {
    const int world = argc > 1 ? std::atoi(argv[1]) : 2;
    int n_dev = 0;
    CK(cudaGetDeviceCount(&n_dev));
    if (world < 1 || world > 8) return 2;
    if (n_dev < world) {
        std::printf("skipped: %d devices for %d ranks\n", n_dev, world);
        return 77;
    }
    grpo::LossConfig config;
    config.clip_eps = 0.2f;
    config.beta = 0.01f;
    config.reduction = grpo::ReductionMode::token_mean;
    int failures = 0;
    for (int round = 0; round < 3; round++) {
        const bool empty = round == 2;  // the last round has a response without a valid token: every rank must throw
        const Batch b = make_batch(1000 + round, empty);
        const size_t row_bytes = static_cast<size_t>(b.P) * sizeof(float);

        // the whole batch on device 0 through the reference-facing call
        grpo::LossStats want{};
        std::vector<float> want_d(b.logits.size());
        std::string want_error;
        CK(cudaSetDevice(0));
        {
            float* d = nullptr;
            CK(cudaMalloc(&d, b.logits.size() * sizeof(float)));
            CK(cudaMemcpy(d, b.logits.data(), b.logits.size() * sizeof(float), cudaMemcpyHostToDevice));
            try {
                want = grpo::grpo_logits_cuda_device_inplace(d, b.old, b.ref, b.sel, b.adv, b.mask, b.B, b.G, b.T, b.V, b.P, config);
            } catch (const std::runtime_error& e) {
                want_error = e.what();
            }
            CK(cudaMemcpy(want_d.data(), d, want_d.size() * sizeof(float), cudaMemcpyDeviceToHost));
            CK(cudaFree(d));
        }

        std::vector<grpo::ShardedLogitsBoundary*> all(world, nullptr);
        std::vector<grpo::LossStats> got(world);
        std::vector<std::string> errors(world);
        std::vector<double> worst(world, 0.0);
        std::vector<int> identical(world, 1);
        SpinBarrier barrier(world);
        auto rank_main = [&](int r) {
            CK(cudaSetDevice(r));
            const int n = b.N();
            const int lo = static_cast<int>(static_cast<long long>(n) * r / world), hi = static_cast<int>(static_cast<long long>(n) * (r + 1) / world);
            grpo::ShardedLogitsBoundary mine(r, world, b.B, b.G, b.T, b.V, b.P, lo, hi - lo);
            all[r] = &mine;
            barrier.wait();  // every rank's boundary exists
            mine.connect(all);
            float* d = nullptr;
            CK(cudaMalloc(&d, (hi - lo) * row_bytes));
            CK(cudaMemcpy(d, b.logits.data() + static_cast<size_t>(lo) * b.P, (hi - lo) * row_bytes, cudaMemcpyHostToDevice));
            const std::vector<float> old(b.old.begin() + lo, b.old.begin() + hi), ref(b.ref.begin() + lo, b.ref.begin() + hi);
            const std::vector<int> sel(b.sel.begin() + lo, b.sel.begin() + hi), mask(b.mask.begin() + lo, b.mask.begin() + hi);
            barrier.wait();  // every rank is connected: line up before the batch's first exchange
            try {
                got[r] = mine.run(d, old, ref, sel, b.adv, mask, config);
            } catch (const std::runtime_error& e) {
                errors[r] = e.what();
            }
            std::vector<float> out(static_cast<size_t>(hi - lo) * b.P);
            CK(cudaMemcpy(out.data(), d, out.size() * sizeof(float), cudaMemcpyDeviceToHost));
            if (errors[r].empty()) {
                for (size_t i = 0; i < out.size(); i++) {
                    const float w = want_d[static_cast<size_t>(lo) * b.P + i];
                    const double err = std::fabs(static_cast<double>(out[i]) - w), tol = 1e-7 + 1e-5 * std::fabs(w);
                    if (err / tol > worst[r]) worst[r] = err / tol;
                    if (std::memcmp(&out[i], &w, 4) != 0) identical[r] = 0;
                }
            }
            CK(cudaFree(d));
            barrier.wait();  // nobody destroys a region a peer's kernel may still write to
        };
        std::vector<std::thread> threads;
        for (int r = 0; r < world; r++) threads.emplace_back(rank_main, r);
        for (auto& t : threads) t.join();

        for (int r = 0; r < world; r++) {
            if (empty) {
                const bool ok = errors[r] == "every sequence needs at least one valid token" && want_error == errors[r];
                if (!ok) failures++;
                std::printf("round %d rank %d: error \"%s\" (single device: \"%s\") %s\n", round, r, errors[r].c_str(),
                            want_error.c_str(), ok ? "ok" : "FAILED");
                continue;
            }
            const bool same_as_rank0 = std::memcmp(&got[r], &got[0], sizeof(grpo::LossStats)) == 0;
            auto close = [](float a, float w) { return std::fabs(a - w) <= 1e-5f * std::fabs(w) + 1e-9f; };
            const bool ok = errors[r].empty() && same_as_rank0 && got[r].valid_tokens == want.valid_tokens &&
                            close(got[r].loss, want.loss) && close(got[r].pg_loss, want.pg_loss) && close(got[r].kl, want.kl) &&
                            worst[r] <= 1.0;
            if (!ok) failures++;
            std::printf("round %d rank %d: loss %.9g (single device %.9g) valid %d  max err/tol %.3g  gradient bits %s  %s %s\n",
                        round, r, got[r].loss, want.loss, got[r].valid_tokens, worst[r], identical[r] ? "identical" : "differ",
                        errors[r].c_str(), ok ? "ok" : "FAILED");
        }
    }
    std::printf(failures ? "FAILED (%d)\n" : "all ok\n", failures);
    return failures ? 1 : 0;
}

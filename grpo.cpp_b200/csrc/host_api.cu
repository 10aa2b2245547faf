// Host layer of the C ABI: the reference-facing calls.
//
// Same contract as the reference's host wrappers (src/cuda/grpo_loss_cuda.cu:584-817): validate
// with the same messages in the same order, build the per-response weights on the host with the
// same fp32 expressions (make_weights, :21-57), move data, run, wait, check for non-finite
// results.  What differs is the plumbing around the kernels:
//   * no per-call cudaMalloc/cudaFree: device arenas and pinned staging are cached per device
//     and leased to one caller at a time (thread-safe; concurrent callers get separate arenas);
//   * the small per-token metadata travel as ONE pinned host-to-device copy, not six;
//   * the dense-logits variant runs in place on its upload buffer (one device copy of the logits
//     instead of two) and checks logits and gradients for non-finite values on the device
//     instead of scanning N*V floats twice on the host.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "host_util.hpp"

namespace grpo_b200 {
namespace host {

constexpr size_t kIntMaxSz = 2147483647u;

int invalid(const std::string& msg) {
    set_error("%s", msg.c_str());
    return GRPO_B200_E_INVALID;
}

int nonfinite(const char* msg) {
    set_error("%s", msg);
    return GRPO_B200_E_NONFINITE;
}

}  // namespace host
namespace {
using namespace host;

// ---- leased per-device buffers --------------------------------------------------------------
struct Arena {
    int device = -1;
    char* dev = nullptr;
    size_t dev_cap = 0;
    char* pinned = nullptr;
    size_t pinned_cap = 0;
    cudaEvent_t ev[2] = {nullptr, nullptr};
    unsigned* ticket = nullptr;  // zero between calls: the selected-token kernel's ticket counter

    // On failure everything the arena holds is released, so the pool never keeps a half-built one.
    cudaError_t reserve(size_t dev_bytes, size_t pinned_bytes) {
        const cudaError_t err = reserve_parts(dev_bytes, pinned_bytes);
        if (err != cudaSuccess) release_memory();
        return err;
    }
    cudaError_t reserve_parts(size_t dev_bytes, size_t pinned_bytes) {
        if (!ticket) {
            cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&ticket), 256);
            if (err != cudaSuccess) return err;
            err = cudaMemset(ticket, 0, 256);
            if (err != cudaSuccess) return err;
        }
        if (dev_bytes > dev_cap) {
            if (dev) cudaFree(dev);
            dev = nullptr;
            dev_cap = 0;
            const size_t want = dev_bytes + dev_bytes / 8 + (1u << 20);
            cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&dev), want);
            if (err != cudaSuccess) return err;
            dev_cap = want;
        }
        if (pinned_bytes > pinned_cap) {
            if (pinned) cudaFreeHost(pinned);
            pinned = nullptr;
            pinned_cap = 0;
            const size_t want = pinned_bytes + pinned_bytes / 8 + (64u << 10);
            cudaError_t err = cudaMallocHost(reinterpret_cast<void**>(&pinned), want);
            if (err != cudaSuccess) return err;
            pinned_cap = want;
        }
        if (!ev[0]) {
            cudaError_t err = cudaEventCreate(&ev[0]);
            if (err != cudaSuccess) return err;
            err = cudaEventCreate(&ev[1]);
            if (err != cudaSuccess) return err;
        }
        return cudaSuccess;
    }
    void release_memory() {
        if (dev) cudaFree(dev);
        if (pinned) cudaFreeHost(pinned);
        if (ticket) cudaFree(ticket);
        for (cudaEvent_t& e : ev) {
            if (e) cudaEventDestroy(e);
            e = nullptr;
        }
        ticket = nullptr;
        dev = pinned = nullptr;
        dev_cap = pinned_cap = 0;
    }
};

std::mutex g_pool_mutex;
std::unordered_map<int, std::vector<Arena*>> g_pool;

struct Lease {
    Arena* arena = nullptr;
    cudaError_t acquire() {
        int device = 0;
        cudaError_t err = cudaGetDevice(&device);
        if (err != cudaSuccess) return err;
        std::lock_guard<std::mutex> lock(g_pool_mutex);
        auto& idle = g_pool[device];
        if (idle.empty()) {
            arena = new Arena();
            arena->device = device;
        } else {
            arena = idle.back();
            idle.pop_back();
        }
        return cudaSuccess;
    }
    ~Lease() {
        if (!arena) return;
        std::lock_guard<std::mutex> lock(g_pool_mutex);
        g_pool[arena->device].push_back(arena);
    }
};

// bump allocator over an arena, 256-byte aligned slices
struct Bump {
    char* base;
    size_t off = 0;
    explicit Bump(char* b) : base(b) {}
    template <class T>
    T* take(size_t count) {
        T* p = reinterpret_cast<T*>(base + off);
        off += (count * sizeof(T) + 255) & ~static_cast<size_t>(255);
        return p;
    }
};
size_t slice(size_t bytes) { return (bytes + 255) & ~static_cast<size_t>(255); }

}  // namespace
namespace host {
// ---- validation (messages and order of src/cuda/grpo_loss_cuda.cu:584-618, 662-724) ----------

int checked_shape(int B, int G, int T, Shape& out) {
    // include/grpo/grpo_loss.hpp:51-67 of the reference
    if (B <= 0 || G <= 0 || T <= 0) return invalid("B, G and T must be positive");
    const size_t s = static_cast<size_t>(B) * static_cast<size_t>(G);
    if (s > kIntMaxSz) return invalid("sequence count exceeds INT_MAX");
    const size_t n = s * static_cast<size_t>(T);
    if (n > kIntMaxSz) return invalid("token count exceeds INT_MAX");
    out.sequences = s;
    out.tokens = n;
    return GRPO_B200_OK;
}

int expect_size(const char* name, size_t got, size_t want) {
    if (got == want) return GRPO_B200_OK;
    return invalid(std::string(name) + " has size " + std::to_string(got) + ", expected " + std::to_string(want));
}


int check_options(const Options& o) {
    if (o.clip_eps < 0.0f || o.clip_eps >= 1.0f || !std::isfinite(o.clip_eps))
        return invalid("clip_eps must be finite and in [0, 1)");
    if (o.beta < 0.0f || !std::isfinite(o.beta)) return invalid("beta must be finite and non-negative");
    if (!std::isfinite(o.alpha) || o.alpha < 0.0f || o.alpha > 1.0f)
        return invalid("length_alpha must be finite and in [0, 1]");
    return GRPO_B200_OK;
}

// Token-array checks shared by all three calls.  logp_new is null for the logits calls, whose
// reference validators pass a zero vector of the right size in its place.
int validate_sizes(bool has_new, size_t n_new, size_t n_old, size_t n_ref, size_t n_adv, size_t n_mask,
                   const Shape& shape, const Options& opt) {
    if (int rc = check_options(opt)) return rc;
    if (has_new)
        if (int rc = expect_size("logp_new", n_new, shape.tokens)) return rc;
    if (int rc = expect_size("logp_old", n_old, shape.tokens)) return rc;
    if (int rc = expect_size("logp_ref", n_ref, shape.tokens)) return rc;
    if (int rc = expect_size("advantages", n_adv, shape.sequences)) return rc;
    return expect_size("mask", n_mask, shape.tokens);
}

int validate_inputs(const float* lp_new, size_t n_new, const float* lp_old, size_t n_old, const float* lp_ref,
                    size_t n_ref, const float* adv, size_t n_adv, const int32_t* mask, size_t n_mask,
                    const Shape& shape, const Options& opt) {
    if (int rc = validate_sizes(lp_new != nullptr, n_new, n_old, n_ref, n_adv, n_mask, shape, opt)) return rc;
    // one branch-free sweep first (it vectorises); only a batch that has a bad value is walked again in the
    // reference's order to find which complaint comes first
    unsigned bad = 0;
    const uint32_t* old_bits = reinterpret_cast<const uint32_t*>(lp_old);
    const uint32_t* ref_bits = reinterpret_cast<const uint32_t*>(lp_ref);
    for (size_t i = 0; i < shape.tokens; i++) {
        bad |= ((old_bits[i] & 0x7f800000u) == 0x7f800000u) | ((ref_bits[i] & 0x7f800000u) == 0x7f800000u) |
               (static_cast<uint32_t>(mask[i]) > 1u);
    }
    if (lp_new) {
        const uint32_t* new_bits = reinterpret_cast<const uint32_t*>(lp_new);
        for (size_t i = 0; i < shape.tokens; i++) bad |= (new_bits[i] & 0x7f800000u) == 0x7f800000u;
    }
    if (bad) {
        for (size_t i = 0; i < shape.tokens; i++) {
            if ((lp_new && !std::isfinite(lp_new[i])) || !std::isfinite(lp_old[i]) || !std::isfinite(lp_ref[i]))
                return invalid("log probabilities must be finite");
            if (mask[i] != 0 && mask[i] != 1) return invalid("mask values must be 0 or 1");
        }
    }
    for (size_t s = 0; s < shape.sequences; s++)
        if (!std::isfinite(adv[s])) return invalid("advantages must be finite");
    return GRPO_B200_OK;
}

}  // namespace host
namespace {
// Host twin of make_weights (src/cuda/grpo_loss_cuda.cu:21-57): same fp32 expressions.
int weights_from_lengths(const int* lengths, int valid_tokens, const Shape& shape, const Options& opt, float* weights);

int make_weights(const int32_t* mask, const Shape& shape, int T, const Options& opt, float* weights,
                 int& valid_tokens) {
    std::vector<int> lengths(shape.sequences, 0);
    valid_tokens = 0;
    for (size_t s = 0; s < shape.sequences; s++) {
        const int32_t* m = mask + s * static_cast<size_t>(T);
        int count = 0;
        for (int t = 0; t < T; t++) count += m[t] != 0;
        lengths[s] = count;
        valid_tokens += count;
    }
    return weights_from_lengths(lengths.data(), valid_tokens, shape, opt, weights);
}

int weights_from_lengths(const int* lengths, int valid_tokens, const Shape& shape, const Options& opt, float* weights) {
    const float n_seq = static_cast<float>(shape.sequences);
    for (size_t s = 0; s < shape.sequences; s++) {
        if (lengths[s] == 0) return invalid("every sequence needs at least one valid token");
        if (opt.reduction == GRPO_B200_SEQUENCE_MEAN)
            weights[s] = 1.0f / (n_seq * lengths[s]);
        else if (opt.reduction == GRPO_B200_TOKEN_MEAN)
            weights[s] = 1.0f / static_cast<float>(valid_tokens);
        else
            weights[s] = std::pow(static_cast<float>(lengths[s]), opt.alpha - 1.0f) / n_seq;
    }
    return GRPO_B200_OK;
}

}  // namespace
namespace host {
int check_selected(const int32_t* selected, const int32_t* mask, size_t n, int V, size_t& first_bad) {
    first_bad = n;
    unsigned any = 0;  // branch-free sweep first; the index is only looked for when there is one
    for (size_t i = 0; i < n; i++) any |= (mask[i] != 0) & (static_cast<uint32_t>(selected[i]) >= static_cast<uint32_t>(V));
    if (!any) return 0;
    for (size_t i = 0; i < n; i++)
        if (mask[i] != 0 && (selected[i] < 0 || selected[i] >= V)) {
            first_bad = i;
            return 1;
        }
    return 0;
}

int fill_stats(const grpo_b200_result_t& r, float* stats, const char* what) {
    if (r.bad_inputs < 0.0) {  // the pass itself failed (include/grpo_b200.h, grpo_b200_result_t)
        if (r.bad_inputs == kBadInputsRowOrder)
            set_error("CUDA error: the row order handed to the logits kernel does not belong to the mask");
        else if (r.bad_inputs == kBadInputsExchangeTimeout)
            set_error("CUDA error: the exchange between ranks timed out");
        else
            set_error("CUDA error: logits kernel abandoned a stalled copy pipeline");
        return GRPO_B200_E_CUDA;
    }
    stats[0] = static_cast<float>(r.loss);
    stats[1] = static_cast<float>(r.pg_loss);
    stats[2] = static_cast<float>(r.kl);
    if (!std::isfinite(stats[0]) || !std::isfinite(stats[1]) || !std::isfinite(stats[2])) return nonfinite(what);
    return GRPO_B200_OK;
}

}  // namespace host
namespace {
// Device image of the per-token metadata of a logits call, staged through one pinned block.
struct LogitsMeta {
    float* old_d;
    float* ref_d;
    int32_t* sel_d;
    int32_t* mask_d;
    float* adv_d;
    float* w_d;
    int32_t* order_d;  // {n_active, n_masked, active rows, masked rows}: balanced row order for the row kernel
    grpo_b200_result_t* result_d;
    void* work_d;
    size_t work_bytes;
    grpo_b200_result_t* result_h;  // pinned
};

size_t logits_meta_bytes(const Shape& shape) {
    return 4 * slice(shape.tokens * 4) + 2 * slice(shape.sequences * 4) +
           slice(grpo_b200_row_order_bytes(static_cast<int64_t>(shape.tokens))) +
           slice(sizeof(grpo_b200_result_t)) +
           slice(grpo_b200_logits_workspace_bytes(static_cast<int64_t>(shape.tokens)));
}

// Packs old/ref/selected/mask/advantages/weights and the row order (the mask is on the host here,
// so the partition into active and masked rows costs one pass over it) into pinned memory in the
// device layout and issues the single upload.
cudaError_t stage_logits_meta(Arena& arena, Bump& bump, const Shape& shape, const float* lp_old,
                              const float* lp_ref, const int32_t* selected, const float* adv,
                              const float* weights, const int32_t* mask, LogitsMeta& m, bool order_on_device = false) {
    const size_t n = shape.tokens, s = shape.sequences;
    char* dev_start = bump.base + bump.off;
    m.old_d = bump.take<float>(n);
    m.ref_d = bump.take<float>(n);
    m.sel_d = bump.take<int32_t>(n);
    m.mask_d = bump.take<int32_t>(n);
    m.adv_d = bump.take<float>(s);
    m.w_d = bump.take<float>(s);
    size_t packed = static_cast<size_t>(bump.base + bump.off - dev_start);  // what travels in the one upload
    m.order_d = bump.take<int32_t>(grpo_b200_row_order_bytes(static_cast<int64_t>(n)) / sizeof(int32_t));
    if (!order_on_device) packed = static_cast<size_t>(reinterpret_cast<char*>(m.order_d + n + 2) - dev_start);
    m.result_d = bump.take<grpo_b200_result_t>(1);
    m.work_bytes = grpo_b200_logits_workspace_bytes(static_cast<int64_t>(n));
    m.work_d = bump.take<char>(m.work_bytes);

    char* h = arena.pinned;
    auto put = [&](const void* src, size_t bytes, const void* dev_ptr) {
        std::memcpy(h + (static_cast<const char*>(dev_ptr) - dev_start), src, bytes);
    };
    put(lp_old, n * 4, m.old_d);
    put(lp_ref, n * 4, m.ref_d);
    put(selected, n * 4, m.sel_d);
    put(mask, n * 4, m.mask_d);
    put(adv, s * 4, m.adv_d);
    put(weights, s * 4, m.w_d);
    if (!order_on_device) {
        int32_t* order_h = reinterpret_cast<int32_t*>(h + (reinterpret_cast<char*>(m.order_d) - dev_start));
        size_t n_active = 0;
        for (size_t i = 0; i < n; i++) n_active += mask[i] != 0;
        order_h[0] = static_cast<int32_t>(n_active);
        order_h[1] = static_cast<int32_t>(n - n_active);
        int32_t* active = order_h + 2;
        int32_t* masked = active + n_active;
        for (size_t i = 0; i < n; i++) *(mask[i] != 0 ? active : masked)++ = static_cast<int32_t>(i);
    }
    m.result_h = reinterpret_cast<grpo_b200_result_t*>(arena.pinned + slice(packed));
    cudaError_t err = cudaMemcpyAsync(dev_start, h, packed, cudaMemcpyHostToDevice, nullptr);
    // the partition of the rows by mask: two small launches behind the upload instead of two host passes and 4 bytes
    // per row more to upload
    if (err == cudaSuccess && order_on_device) err = launch_row_order(m.mask_d, static_cast<long long>(n), m.order_d, nullptr);
    return err;
}

// The in-place call's checks and staging in two sweeps over the host arrays instead of five, with
// the uploads in flight while the host is still sweeping:
//   sweep 1  the mask: values in {0, 1}, the responses' valid-token counts, its pinned image; the
//            mask is uploaded and the row order is built on the device behind it;
//   sweep 2  log-probabilities finite, selected ids in range on active rows, their pinned images;
//            then advantages and weights, and the second upload.
// Whenever a sweep finds something wrong the ordered validators are asked which complaint the
// reference would raise first (src/cuda/grpo_loss_cuda.cu:584-618, 676-697).  Nothing that was
// enqueued by then touches the caller's logits.
int check_and_stage_logits_meta(Arena& arena, Bump& bump, const Shape& shape, int T, int V, int kernel,
                                const Options& opt, const float* lp_old, size_t n_old, const float* lp_ref,
                                size_t n_ref, const int32_t* selected, const float* adv, size_t n_adv,
                                const int32_t* mask, size_t n_mask, LogitsMeta& m, int& valid_tokens) {
    if (int rc = validate_sizes(false, 0, n_old, n_ref, n_adv, n_mask, shape, opt)) return rc;
    const size_t n = shape.tokens, s = shape.sequences;
    char* dev_start = bump.base + bump.off;
    m.mask_d = bump.take<int32_t>(n);  // first: it travels alone, ahead of the rest
    char* rest_start = bump.base + bump.off;
    m.old_d = bump.take<float>(n);
    m.ref_d = bump.take<float>(n);
    m.sel_d = bump.take<int32_t>(n);
    m.adv_d = bump.take<float>(s);
    m.w_d = bump.take<float>(s);
    const size_t packed = static_cast<size_t>(bump.base + bump.off - dev_start);
    const size_t mask_bytes = static_cast<size_t>(rest_start - dev_start);
    m.order_d = bump.take<int32_t>(grpo_b200_row_order_bytes(static_cast<int64_t>(n)) / sizeof(int32_t));
    m.result_d = bump.take<grpo_b200_result_t>(1);
    m.work_bytes = grpo_b200_logits_workspace_bytes(static_cast<int64_t>(n));
    m.work_d = bump.take<char>(m.work_bytes);
    char* h = arena.pinned;
    m.result_h = reinterpret_cast<grpo_b200_result_t*>(h + slice(packed));
    auto host_of = [&](const void* dev_ptr) { return h + (static_cast<const char*>(dev_ptr) - dev_start); };

    // ---- sweep 1: the mask
    std::vector<int> lengths(s);
    int32_t* mask_h = reinterpret_cast<int32_t*>(host_of(m.mask_d));
    unsigned bad = 0;
    valid_tokens = 0;
    for (size_t q = 0; q < s; q++) {
        int count = 0;
        bad |= copy_and_count_mask(mask + q * static_cast<size_t>(T), mask_h + q * static_cast<size_t>(T), T, count);
        lengths[q] = count;
        valid_tokens += count;
    }
    GRPO_CUDA_TRY(cudaMemcpyAsync(dev_start, h, mask_bytes, cudaMemcpyHostToDevice, nullptr));
    GRPO_CUDA_TRY(launch_row_order(m.mask_d, static_cast<long long>(n), m.order_d, nullptr));

    // ---- sweep 2: log-probabilities, selected ids, advantages (one vectorised copy-and-check loop per array)
    bad |= copy_and_check_finite(reinterpret_cast<const uint32_t*>(lp_old), reinterpret_cast<uint32_t*>(host_of(m.old_d)), n);
    bad |= copy_and_check_finite(reinterpret_cast<const uint32_t*>(lp_ref), reinterpret_cast<uint32_t*>(host_of(m.ref_d)), n);
    bad |= copy_and_check_selected(selected, mask, reinterpret_cast<int32_t*>(host_of(m.sel_d)), n, static_cast<uint32_t>(V));
    bad |= copy_and_check_finite(reinterpret_cast<const uint32_t*>(adv), reinterpret_cast<uint32_t*>(host_of(m.adv_d)), s);
    if (bad) {  // which complaint comes first
        if (int rc = validate_inputs(nullptr, 0, lp_old, n_old, lp_ref, n_ref, adv, n_adv, mask, n_mask, shape, opt))
            return rc;
        size_t first_bad;
        if (check_selected(selected, mask, n, V, first_bad)) return invalid("selected token is outside the vocabulary");
    }
    if (kernel != GRPO_B200_LOGITS_SEPARATE && kernel != GRPO_B200_LOGITS_FUSED)
        return invalid("unknown logits kernel selector");
    if (int rc = weights_from_lengths(lengths.data(), valid_tokens, shape, opt, reinterpret_cast<float*>(host_of(m.w_d))))
        return rc;
    GRPO_CUDA_TRY(cudaMemcpyAsync(rest_start, h + mask_bytes, packed - mask_bytes, cudaMemcpyHostToDevice, nullptr));
    return GRPO_B200_OK;
}

}  // namespace
}  // namespace grpo_b200

using namespace grpo_b200;

extern "C" {

int grpo_b200_loss_host(const float* logp_new, size_t n_logp_new, const float* logp_old, size_t n_logp_old,
                        const float* logp_ref, size_t n_logp_ref, const float* advantages, size_t n_advantages,
                        const int32_t* mask, size_t n_mask, int B, int G, int T, float clip_eps, float beta,
                        int reduction, float length_alpha, int kernel, float* dlogp_out, float* stats_out,
                        int* valid_tokens_out) {
    (void)kernel;  // both selectors run the one deterministic kernel
    Shape shape;
    if (int rc = checked_shape(B, G, T, shape)) return rc;
    const Options opt{clip_eps, beta, length_alpha, reduction};
    if (int rc = validate_inputs(logp_new, n_logp_new, logp_old, n_logp_old, logp_ref, n_logp_ref, advantages,
                                 n_advantages, mask, n_mask, shape, opt))
        return rc;
    std::vector<float> weights(shape.sequences);
    int valid = 0;
    if (int rc = make_weights(mask, shape, T, opt, weights.data(), valid)) return rc;

    const size_t n = shape.tokens, s = shape.sequences;
    Lease lease;
    GRPO_CUDA_TRY(lease.acquire());
    Arena& arena = *lease.arena;
    const size_t work_bytes = grpo_b200_loss_workspace_bytes(static_cast<int64_t>(n));
    GRPO_CUDA_TRY(arena.reserve(5 * slice(n * 4) + 2 * slice(s * 4) + slice(sizeof(grpo_b200_result_t)) +
                                    slice(work_bytes),
                                2 * slice(s * 4) + slice(sizeof(grpo_b200_result_t))));
    Bump bump(arena.dev);
    float* new_d = bump.take<float>(n);
    float* old_d = bump.take<float>(n);
    float* ref_d = bump.take<float>(n);
    int32_t* mask_d = bump.take<int32_t>(n);
    float* dlogp_d = bump.take<float>(n);
    float* adv_d = bump.take<float>(s);  // advantages and weights are adjacent: one copy
    float* w_d = bump.take<float>(s);
    auto* result_d = bump.take<grpo_b200_result_t>(1);
    void* work_d = bump.take<char>(work_bytes);

    const size_t small = static_cast<size_t>(reinterpret_cast<char*>(w_d) - reinterpret_cast<char*>(adv_d)) + s * 4;
    std::memcpy(arena.pinned, advantages, s * 4);
    std::memcpy(arena.pinned + (reinterpret_cast<char*>(w_d) - reinterpret_cast<char*>(adv_d)), weights.data(), s * 4);
    auto* result_h = reinterpret_cast<grpo_b200_result_t*>(arena.pinned + 2 * slice(s * 4));

    GRPO_CUDA_TRY(cudaMemcpyAsync(adv_d, arena.pinned, small, cudaMemcpyHostToDevice, nullptr));
    GRPO_CUDA_TRY(cudaMemcpyAsync(new_d, logp_new, n * 4, cudaMemcpyHostToDevice, nullptr));
    GRPO_CUDA_TRY(cudaMemcpyAsync(old_d, logp_old, n * 4, cudaMemcpyHostToDevice, nullptr));
    GRPO_CUDA_TRY(cudaMemcpyAsync(ref_d, logp_ref, n * 4, cudaMemcpyHostToDevice, nullptr));
    GRPO_CUDA_TRY(cudaMemcpyAsync(mask_d, mask, n * 4, cudaMemcpyHostToDevice, nullptr));
    if (int rc = loss_pass(new_d, old_d, ref_d, adv_d, w_d, mask_d, static_cast<int64_t>(n), 0, T, clip_eps, beta,
                           dlogp_d, result_d, work_d, work_bytes, arena.ticket, nullptr))
        return rc;
    GRPO_CUDA_TRY(cudaMemcpyAsync(result_h, result_d, sizeof(*result_h), cudaMemcpyDeviceToHost, nullptr));
    GRPO_CUDA_TRY(cudaMemcpyAsync(dlogp_out, dlogp_d, n * 4, cudaMemcpyDeviceToHost, nullptr));
    GRPO_CUDA_TRY(cudaStreamSynchronize(nullptr));

    *valid_tokens_out = valid;
    if (int rc = fill_stats(*result_h, stats_out, "CUDA loss became non-finite")) return rc;
    if (result_h->bad_grads != 0.0) return nonfinite("CUDA gradient became non-finite");
    return GRPO_B200_OK;
}

int grpo_b200_logits_device_inplace_host(float* logits_and_dlogits, const float* logp_old, size_t n_logp_old,
                                         const float* logp_ref, size_t n_logp_ref, const int32_t* selected,
                                         size_t n_selected, const float* advantages, size_t n_advantages,
                                         const int32_t* mask, size_t n_mask, int B, int G, int T, int V, int P,
                                         float clip_eps, float beta, int reduction, float length_alpha,
                                         int kernel, float* stats_out, int* valid_tokens_out) {
    if (logits_and_dlogits == nullptr) return invalid("logits_and_dlogits must not be null");
    if (P < V) return invalid("P must be at least V");
    Shape shape;
    if (int rc = checked_shape(B, G, T, shape)) return rc;
    if (V <= 0) return invalid("V must be positive");
    if (int rc = expect_size("selected_tokens", n_selected, shape.tokens)) return rc;
    const Options opt{clip_eps, beta, length_alpha, reduction};
    if (int rc = check_options(opt)) return rc;  // before any memory is leased, as the other entries do

    Lease lease;
    GRPO_CUDA_TRY(lease.acquire());
    Arena& arena = *lease.arena;
    const size_t meta = logits_meta_bytes(shape);
    GRPO_CUDA_TRY(arena.reserve(meta, meta));
    Bump bump(arena.dev);
    LogitsMeta m;
    int valid = 0;
    if (int rc = check_and_stage_logits_meta(arena, bump, shape, T, V, kernel, opt, logp_old, n_logp_old, logp_ref,
                                             n_logp_ref, selected, advantages, n_advantages, mask, n_mask, m, valid))
        return rc;
    if (int rc = grpo_b200_logits(logits_and_dlogits, logits_and_dlogits, m.old_d, m.ref_d, m.sel_d, m.adv_d,
                                  m.w_d, m.mask_d, static_cast<int64_t>(shape.tokens), 0, T, V, P, clip_eps, beta,
                                  kernel, 0, nullptr, m.order_d, m.result_d, m.work_d, m.work_bytes, nullptr))
        return rc;
    GRPO_CUDA_TRY(cudaMemcpyAsync(m.result_h, m.result_d, sizeof(*m.result_h), cudaMemcpyDeviceToHost, nullptr));
    GRPO_CUDA_TRY(cudaStreamSynchronize(nullptr));
    *valid_tokens_out = valid;
    return fill_stats(*m.result_h, stats_out, "CUDA logits loss became non-finite");
}

int grpo_b200_logits_host(const float* logits, size_t n_logits, const float* logp_old, size_t n_logp_old,
                          const float* logp_ref, size_t n_logp_ref, const int32_t* selected, size_t n_selected,
                          const float* advantages, size_t n_advantages, const int32_t* mask, size_t n_mask, int B,
                          int G, int T, int V, float clip_eps, float beta, int reduction, float length_alpha,
                          int kernel, float* dlogits_out, float* stats_out, int* valid_tokens_out) {
    Shape shape;
    if (int rc = checked_shape(B, G, T, shape)) return rc;
    if (V <= 0) return invalid("V must be positive");
    const size_t vocab = static_cast<size_t>(V);
    if (shape.tokens > static_cast<size_t>(-1) / vocab) return invalid("logits count is too large");
    const size_t total = shape.tokens * vocab;
    if (int rc = expect_size("logits_new", n_logits, total)) return rc;
    if (int rc = expect_size("selected_tokens", n_selected, shape.tokens)) return rc;
    const Options opt{clip_eps, beta, length_alpha, reduction};
    if (int rc = validate_inputs(nullptr, 0, logp_old, n_logp_old, logp_ref, n_logp_ref, advantages,
                                 n_advantages, mask, n_mask, shape, opt))
        return rc;
    // The reference walks the active rows in order, checking the selected id and then the row's
    // logits.  The logits are checked on the device here; only when an id is out of range do the
    // rows before it have to be scanned on the host to decide which complaint comes first.
    size_t first_bad;
    if (check_selected(selected, mask, shape.tokens, V, first_bad)) {
        for (size_t i = 0; i < first_bad; i++) {
            if (mask[i] == 0) continue;
            for (size_t v = 0; v < vocab; v++)
                if (!std::isfinite(logits[i * vocab + v])) return invalid("logits must be finite");
        }
        return invalid("selected token is outside the vocabulary");
    }
    if (kernel != GRPO_B200_LOGITS_SEPARATE && kernel != GRPO_B200_LOGITS_FUSED)
        return invalid("unknown logits kernel selector");
    std::vector<float> weights(shape.sequences);
    int valid = 0;
    if (int rc = make_weights(mask, shape, T, opt, weights.data(), valid)) return rc;

    Lease lease;
    GRPO_CUDA_TRY(lease.acquire());
    Arena& arena = *lease.arena;
    const size_t meta = logits_meta_bytes(shape);
    GRPO_CUDA_TRY(arena.reserve(meta + slice(total * 4), meta));
    Bump bump(arena.dev);
    LogitsMeta m;
    GRPO_CUDA_TRY(stage_logits_meta(arena, bump, shape, logp_old, logp_ref, selected, advantages, weights.data(),
                                    mask, m));
    float* logits_d = bump.take<float>(total);
    GRPO_CUDA_TRY(cudaMemcpyAsync(logits_d, logits, total * 4, cudaMemcpyHostToDevice, nullptr));
    if (int rc = grpo_b200_logits(logits_d, logits_d, m.old_d, m.ref_d, m.sel_d, m.adv_d, m.w_d, m.mask_d,
                                  static_cast<int64_t>(shape.tokens), 0, T, V, V, clip_eps, beta, kernel, 1,
                                  nullptr, m.order_d, m.result_d, m.work_d, m.work_bytes, nullptr))
        return rc;
    GRPO_CUDA_TRY(cudaMemcpyAsync(m.result_h, m.result_d, sizeof(*m.result_h), cudaMemcpyDeviceToHost, nullptr));
    GRPO_CUDA_TRY(cudaMemcpyAsync(dlogits_out, logits_d, total * 4, cudaMemcpyDeviceToHost, nullptr));
    GRPO_CUDA_TRY(cudaStreamSynchronize(nullptr));
    if (m.result_h->bad_inputs > 0.0) return invalid("logits must be finite");
    *valid_tokens_out = valid;
    if (int rc = fill_stats(*m.result_h, stats_out, "CUDA logits loss became non-finite")) return rc;
    if (m.result_h->bad_grads != 0.0) return nonfinite("CUDA logits gradient became non-finite");
    return GRPO_B200_OK;
}

// ---- timers (protocol of src/cuda/grpo_loss_cuda.cu:819-975) ------------------------------------

int grpo_b200_benchmark_loss_host(const float* logp_new, size_t n_logp_new, const float* logp_old,
                                  size_t n_logp_old, const float* logp_ref, size_t n_logp_ref,
                                  const float* advantages, size_t n_advantages, const int32_t* mask, size_t n_mask,
                                  int B, int G, int T, float clip_eps, float beta, int reduction,
                                  float length_alpha, int warmup, int iterations, float* atomic_ms,
                                  float* block_ms) {
    Shape shape;
    if (int rc = checked_shape(B, G, T, shape)) return rc;
    const Options opt{clip_eps, beta, length_alpha, reduction};
    if (int rc = validate_inputs(logp_new, n_logp_new, logp_old, n_logp_old, logp_ref, n_logp_ref, advantages,
                                 n_advantages, mask, n_mask, shape, opt))
        return rc;
    if (warmup < 0 || iterations <= 0) return invalid("invalid benchmark iteration count");
    std::vector<float> weights(shape.sequences);
    int valid = 0;
    if (int rc = make_weights(mask, shape, T, opt, weights.data(), valid)) return rc;

    const size_t n = shape.tokens, s = shape.sequences;
    Lease lease;
    GRPO_CUDA_TRY(lease.acquire());
    Arena& arena = *lease.arena;
    const size_t work_bytes = grpo_b200_loss_workspace_bytes(static_cast<int64_t>(n));
    GRPO_CUDA_TRY(arena.reserve(5 * slice(n * 4) + 2 * slice(s * 4) + slice(sizeof(grpo_b200_result_t)) +
                                    slice(work_bytes),
                                64));
    Bump bump(arena.dev);
    float* new_d = bump.take<float>(n);
    float* old_d = bump.take<float>(n);
    float* ref_d = bump.take<float>(n);
    int32_t* mask_d = bump.take<int32_t>(n);
    float* dlogp_d = bump.take<float>(n);
    float* adv_d = bump.take<float>(s);
    float* w_d = bump.take<float>(s);
    auto* result_d = bump.take<grpo_b200_result_t>(1);
    void* work_d = bump.take<char>(work_bytes);
    GRPO_CUDA_TRY(cudaMemcpy(new_d, logp_new, n * 4, cudaMemcpyHostToDevice));
    GRPO_CUDA_TRY(cudaMemcpy(old_d, logp_old, n * 4, cudaMemcpyHostToDevice));
    GRPO_CUDA_TRY(cudaMemcpy(ref_d, logp_ref, n * 4, cudaMemcpyHostToDevice));
    GRPO_CUDA_TRY(cudaMemcpy(mask_d, mask, n * 4, cudaMemcpyHostToDevice));
    GRPO_CUDA_TRY(cudaMemcpy(adv_d, advantages, s * 4, cudaMemcpyHostToDevice));
    GRPO_CUDA_TRY(cudaMemcpy(w_d, weights.data(), s * 4, cudaMemcpyHostToDevice));

    auto pass = [&]() {
        return loss_pass(new_d, old_d, ref_d, adv_d, w_d, mask_d, static_cast<int64_t>(n), 0, T, clip_eps, beta,
                         dlogp_d, result_d, work_d, work_bytes, arena.ticket, nullptr);
    };
    for (int i = 0; i < 2 * warmup; i++)
        if (int rc = pass()) return rc;
    GRPO_CUDA_TRY(cudaDeviceSynchronize());
    float medians[2] = {0.0f, 0.0f};
    for (int which = 0; which < 2; which++) {  // "atomic" then "block": the same kernel, timed twice
        std::vector<float> samples;
        for (int repeat = 0; repeat < 7; repeat++) {
            GRPO_CUDA_TRY(cudaEventRecord(arena.ev[0], nullptr));
            for (int i = 0; i < iterations; i++)
                if (int rc = pass()) return rc;
            GRPO_CUDA_TRY(cudaEventRecord(arena.ev[1], nullptr));
            GRPO_CUDA_TRY(cudaEventSynchronize(arena.ev[1]));
            float ms = 0.0f;
            GRPO_CUDA_TRY(cudaEventElapsedTime(&ms, arena.ev[0], arena.ev[1]));
            samples.push_back(ms / static_cast<float>(iterations));
        }
        std::sort(samples.begin(), samples.end());
        medians[which] = samples[samples.size() / 2];
    }
    *atomic_ms = medians[0];
    *block_ms = medians[1];
    return GRPO_B200_OK;
}

int grpo_b200_benchmark_logits_host(const float* logits, size_t n_logits, const float* logp_old, size_t n_logp_old,
                                    const float* logp_ref, size_t n_logp_ref, const int32_t* selected,
                                    size_t n_selected, const float* advantages, size_t n_advantages,
                                    const int32_t* mask, size_t n_mask, int B, int G, int T, int V, float clip_eps,
                                    float beta, int reduction, float length_alpha, int warmup, int iterations,
                                    float* separate_ms, float* fused_ms) {
    Shape shape;
    if (int rc = checked_shape(B, G, T, shape)) return rc;
    if (V <= 0) return invalid("V must be positive");
    const size_t vocab = static_cast<size_t>(V);
    if (shape.tokens > static_cast<size_t>(-1) / vocab) return invalid("logits count is too large");
    const size_t total = shape.tokens * vocab;
    if (int rc = expect_size("logits_new", n_logits, total)) return rc;
    if (int rc = expect_size("selected_tokens", n_selected, shape.tokens)) return rc;
    const Options opt{clip_eps, beta, length_alpha, reduction};
    if (int rc = validate_inputs(nullptr, 0, logp_old, n_logp_old, logp_ref, n_logp_ref, advantages,
                                 n_advantages, mask, n_mask, shape, opt))
        return rc;
    for (size_t i = 0; i < shape.tokens; i++) {
        if (mask[i] == 0) continue;
        if (selected[i] < 0 || selected[i] >= V) return invalid("selected token is outside the vocabulary");
        for (size_t v = 0; v < vocab; v++)
            if (!std::isfinite(logits[i * vocab + v])) return invalid("logits must be finite");
    }
    if (warmup < 0 || iterations <= 0) return invalid("invalid benchmark iteration count");
    std::vector<float> weights(shape.sequences);
    int valid = 0;
    if (int rc = make_weights(mask, shape, T, opt, weights.data(), valid)) return rc;

    Lease lease;
    GRPO_CUDA_TRY(lease.acquire());
    Arena& arena = *lease.arena;
    const size_t meta = logits_meta_bytes(shape);
    GRPO_CUDA_TRY(arena.reserve(meta + 2 * slice(total * 4), meta));
    Bump bump(arena.dev);
    LogitsMeta m;
    GRPO_CUDA_TRY(stage_logits_meta(arena, bump, shape, logp_old, logp_ref, selected, advantages, weights.data(),
                                    mask, m));
    float* in_d = bump.take<float>(total);
    float* out_d = bump.take<float>(total);
    GRPO_CUDA_TRY(cudaMemcpy(in_d, logits, total * 4, cudaMemcpyHostToDevice));

    auto pass = [&](int kernel) {
        return grpo_b200_logits(in_d, out_d, m.old_d, m.ref_d, m.sel_d, m.adv_d, m.w_d, m.mask_d,
                                static_cast<int64_t>(shape.tokens), 0, T, V, V, clip_eps, beta, kernel, 0, nullptr,
                                m.order_d, m.result_d, m.work_d, m.work_bytes, nullptr);
    };
    auto time_once = [&](int kernel, float& ms_per_pass) -> int {
        GRPO_CUDA_TRY(cudaEventRecord(arena.ev[0], nullptr));
        for (int i = 0; i < iterations; i++)
            if (int rc = pass(kernel)) return rc;
        GRPO_CUDA_TRY(cudaEventRecord(arena.ev[1], nullptr));
        GRPO_CUDA_TRY(cudaEventSynchronize(arena.ev[1]));
        float ms = 0.0f;
        GRPO_CUDA_TRY(cudaEventElapsedTime(&ms, arena.ev[0], arena.ev[1]));
        ms_per_pass = ms / static_cast<float>(iterations);
        return GRPO_B200_OK;
    };
    for (int i = 0; i < warmup; i++) {
        if (int rc = pass(GRPO_B200_LOGITS_SEPARATE)) return rc;
        if (int rc = pass(GRPO_B200_LOGITS_FUSED)) return rc;
    }
    GRPO_CUDA_TRY(cudaDeviceSynchronize());
    std::vector<float> sep, fus;
    for (int sample = 0; sample < 15; sample++) {
        float a = 0.0f, b = 0.0f;
        const int first = sample % 2 == 0 ? GRPO_B200_LOGITS_SEPARATE : GRPO_B200_LOGITS_FUSED;
        const int second = first == GRPO_B200_LOGITS_SEPARATE ? GRPO_B200_LOGITS_FUSED : GRPO_B200_LOGITS_SEPARATE;
        if (int rc = time_once(first, a)) return rc;
        if (int rc = time_once(second, b)) return rc;
        (first == GRPO_B200_LOGITS_SEPARATE ? sep : fus).push_back(a);
        (second == GRPO_B200_LOGITS_SEPARATE ? sep : fus).push_back(b);
    }
    std::sort(sep.begin(), sep.end());
    std::sort(fus.begin(), fus.end());
    *separate_ms = sep[sep.size() / 2];
    *fused_ms = fus[fus.size() / 2];
    return GRPO_B200_OK;
}

int grpo_b200_release_cache(void) {
    int device = 0;
    GRPO_CUDA_TRY(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    for (Arena* a : g_pool[device]) {  // idle arenas only: a leased one is not in the pool
        a->release_memory();
        delete a;
    }
    g_pool[device].clear();
    return GRPO_B200_OK;
}

}  // extern "C"

// Device layer of the C ABI: argument checks and kernel dispatch.  The compute entry points neither
// allocate nor synchronise nor exit, and every pointer they take is a device pointer on the current
// device; only the exchange-region calls (create / export / open / close / destroy) manage memory.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>

#include "common.cuh"

#define GRPO_STR2(x) #x
#define GRPO_STR(x) GRPO_STR2(x)

namespace grpo_b200 {

namespace {
thread_local std::string g_error;
}

void set_error(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_error = buf;
}

int cuda_fail(cudaError_t err, const char* what) {
    set_error("CUDA error: %s (%s)", cudaGetErrorString(err), what);
    return GRPO_B200_E_CUDA;
}

namespace {

int invalid(const char* msg) {
    set_error("%s", msg);
    return GRPO_B200_E_INVALID;
}

// Option ranges, with the reference's messages (src/cuda/grpo_loss_cuda.cu:596-601).
int check_options(float clip_eps, float beta) {
    if (!(clip_eps >= 0.0f && clip_eps < 1.0f)) return invalid("clip_eps must be finite and in [0, 1)");
    if (!(beta >= 0.0f && beta <= 3.402823466e+38f)) return invalid("beta must be finite and non-negative");
    return GRPO_B200_OK;
}

constexpr long long kIntMax = 2147483647LL;

// Exchange regions created by this process, with the response count each was sized for: a sharded
// call whose n_seq differs from its own region's would write past the end of every rank's region.
std::mutex g_regions_mutex;
std::unordered_map<const void*, long long> g_regions;
std::atomic<long long> g_exchange_timeout_cycles{kDefaultExchangeTimeoutCycles};

// 0: the own region is unknown to this process (mapped from elsewhere) or matches; else an error code
int check_own_region(void* const* regions, int rank, int64_t n_seq) {
    std::lock_guard<std::mutex> lock(g_regions_mutex);
    auto it = g_regions.find(regions[rank]);
    if (it != g_regions.end() && it->second != n_seq) {
        set_error("n_seq is %lld but this rank's exchange region was created for %lld responses",
                  static_cast<long long>(n_seq), it->second);
        return GRPO_B200_E_INVALID;
    }
    return GRPO_B200_OK;
}

}  // namespace

// The selected-token pass.  `kept_counter` is a ticket counter that is zero now and that the kernel
// leaves at zero (the library's own per-device buffers keep one); without it the counter at the end
// of the caller's workspace is used and cleared first, which costs one more stream operation.
int loss_pass(const float* logp_new, const float* logp_old, const float* logp_ref, const float* advantages,
              const float* weights, const int32_t* mask, int64_t n_tokens, int64_t token_offset, int tokens_per_seq,
              float clip_eps, float beta, float* dlogp, grpo_b200_result_t* result, void* workspace,
              size_t workspace_bytes, unsigned* kept_counter, grpo_b200_stream_t stream) {
    if (!logp_new || !logp_old || !logp_ref || !advantages || !weights || !mask || !dlogp || !result)
        return invalid("device pointers must not be null");
    if (n_tokens <= 0 || tokens_per_seq <= 0 || token_offset < 0) return invalid("B, G and T must be positive");
    if (token_offset + n_tokens > kIntMax) return invalid("token count exceeds INT_MAX");
    if (int rc = check_options(clip_eps, beta)) return rc;
    if (!workspace || workspace_bytes < grpo_b200_loss_workspace_bytes(n_tokens) ||
        (reinterpret_cast<uintptr_t>(workspace) & 7u)) {
        set_error("workspace must be 8-byte aligned and hold grpo_b200_loss_workspace_bytes() bytes");
        return GRPO_B200_E_WORKSPACE;
    }
    LossArgs a;
    a.logp_new = logp_new;
    a.logp_old = logp_old;
    a.logp_ref = logp_ref;
    a.advantages = advantages;
    a.weights = weights;
    a.mask = mask;
    a.n_tokens = n_tokens;
    a.token_offset = token_offset;
    a.tokens_per_seq = tokens_per_seq;
    a.clip_eps = clip_eps;
    a.beta = beta;
    a.dlogp = dlogp;
    a.result = result;
    a.partials = static_cast<double*>(workspace);
    a.counter = kept_counter ? kept_counter : reinterpret_cast<unsigned*>(a.partials + 2048 * 5);
    GRPO_CUDA_TRY(launch_loss(a, kept_counter == nullptr, reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

}  // namespace grpo_b200

using namespace grpo_b200;

extern "C" {

const char* grpo_b200_last_error(void) { return g_error.c_str(); }

const char* grpo_b200_build_info(void) { return "grpo_b200 0.1 (sm_100a, CUDA " GRPO_STR(CUDART_VERSION) ")"; }

int grpo_b200_count_lengths(const int32_t* mask, int64_t n_rows, int64_t row_offset, int tokens_per_seq,
                            int64_t n_seq, int32_t* lengths, grpo_b200_stream_t stream) {
    if (!mask || !lengths) return invalid("mask and lengths must not be null");
    if (n_rows <= 0 || n_seq <= 0 || tokens_per_seq <= 0 || row_offset < 0)
        return invalid("B, G and T must be positive");
    if (n_seq > kIntMax) return invalid("sequence count exceeds INT_MAX");
    if (row_offset + n_rows > n_seq * static_cast<int64_t>(tokens_per_seq))
        return invalid("local rows reach past the end of the batch");
    GRPO_CUDA_TRY(launch_count_lengths(mask, n_rows, row_offset, tokens_per_seq, n_seq, lengths,
                                       reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

int grpo_b200_weights_from_lengths(const int32_t* lengths, int64_t n_seq, int reduction, float length_alpha,
                                   float* weights, int32_t* meta, grpo_b200_stream_t stream) {
    if (!lengths || !weights || !meta) return invalid("lengths, weights and meta must not be null");
    if (n_seq <= 0) return invalid("B, G and T must be positive");
    if (n_seq > kIntMax) return invalid("sequence count exceeds INT_MAX");
    if (reduction < 0 || reduction > 2) return invalid("unknown reduction mode");
    if (!(length_alpha >= 0.0f && length_alpha <= 1.0f)) return invalid("length_alpha must be finite and in [0, 1]");
    GRPO_CUDA_TRY(launch_weights(lengths, n_seq, reduction, length_alpha, weights, meta,
                                 reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

int grpo_b200_count_lengths_f64(const int32_t* mask, int64_t n_rows, int64_t row_offset, int tokens_per_seq,
                                int64_t n_seq, double* lengths, grpo_b200_stream_t stream) {
    if (!mask || !lengths) return invalid("mask and lengths must not be null");
    if (n_rows <= 0 || n_seq <= 0 || tokens_per_seq <= 0 || row_offset < 0)
        return invalid("B, G and T must be positive");
    if (n_seq > kIntMax) return invalid("sequence count exceeds INT_MAX");
    if (row_offset + n_rows > n_seq * static_cast<int64_t>(tokens_per_seq))
        return invalid("local rows reach past the end of the batch");
    GRPO_CUDA_TRY(launch_count_lengths_f64(mask, n_rows, row_offset, tokens_per_seq, n_seq, lengths,
                                           reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

int grpo_b200_weights_from_lengths_f64(const double* lengths, int64_t n_seq, int reduction, float length_alpha,
                                       float* weights, int32_t* meta, grpo_b200_stream_t stream) {
    if (!lengths || !weights || !meta) return invalid("lengths, weights and meta must not be null");
    if (n_seq <= 0) return invalid("B, G and T must be positive");
    if (n_seq > kIntMax) return invalid("sequence count exceeds INT_MAX");
    if (reduction < 0 || reduction > 2) return invalid("unknown reduction mode");
    if (!(length_alpha >= 0.0f && length_alpha <= 1.0f)) return invalid("length_alpha must be finite and in [0, 1]");
    GRPO_CUDA_TRY(launch_weights_f64(lengths, n_seq, reduction, length_alpha, weights, meta,
                                     reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

int grpo_b200_group_advantages(const float* rewards, int B, int G, int mode, float eps, float* advantages,
                               int32_t* meta, grpo_b200_stream_t stream) {
    if (!rewards || !advantages || !meta) return invalid("rewards, advantages and meta must not be null");
    if (B <= 0 || G <= 0) return invalid("B, G and T must be positive");
    if (static_cast<long long>(B) * G > kIntMax) return invalid("sequence count exceeds INT_MAX");
    if (!(eps >= 0.0f && eps <= 3.402823466e+38f)) return invalid("eps must be finite and non-negative");
    if (mode != GRPO_B200_ADV_STANDARDIZED && mode != GRPO_B200_ADV_CENTERED) return invalid("unknown advantage mode");
    GRPO_CUDA_TRY(launch_group_advantages(rewards, B, G, mode, eps, advantages, meta,
                                          reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

size_t grpo_b200_loss_workspace_bytes(int64_t n_tokens) {
    (void)n_tokens;
    return static_cast<size_t>(2048) * 5 * sizeof(double) + 8;  // per-block partials (fixed upper bound) + ticket counter
}

int grpo_b200_loss(const float* logp_new, const float* logp_old, const float* logp_ref, const float* advantages,
                   const float* weights, const int32_t* mask, int64_t n_tokens, int64_t token_offset,
                   int tokens_per_seq, float clip_eps, float beta, float* dlogp, grpo_b200_result_t* result,
                   void* workspace, size_t workspace_bytes, grpo_b200_stream_t stream) {
    return loss_pass(logp_new, logp_old, logp_ref, advantages, weights, mask, n_tokens, token_offset, tokens_per_seq,
                     clip_eps, beta, dlogp, result, workspace, workspace_bytes, nullptr, stream);
}

size_t grpo_b200_logits_workspace_bytes(int64_t n_rows) {
    // one 32-byte record per row, one 32-byte slot for the status word and the ticket counter,
    // then room for five doubles per 256 rows for the reduce kernel (it uses one slot per block of 1,024 rows)
    if (n_rows <= 0) return 0;
    const size_t blocks = (static_cast<size_t>(n_rows) + 255) / 256;
    return static_cast<size_t>(n_rows) * sizeof(RowRecord) + 32 + blocks * 5 * sizeof(double);
}

}  // extern "C"

namespace {

// The whole device-side pass: row kernel, then the reduce kernel (with or without the exchange).
int logits_pass(const float* logits, float* dlogits, const float* logp_old, const float* logp_ref,
                const int32_t* selected, const float* advantages, const float* weights, const int32_t* mask,
                int64_t n_rows, int64_t row_offset, int tokens_per_seq, int V, int P, float clip_eps, float beta,
                int kernel, int check_inputs, float* selected_logp, const int32_t* row_order,
                grpo_b200_result_t* result, void* workspace, size_t workspace_bytes, const ExchangeArgs& x,
                grpo_b200_stream_t stream) {
    if (!logits || !dlogits) return invalid("logits_and_dlogits must not be null");
    if (!logp_old || !logp_ref || !selected || !advantages || !weights || !mask || !result)
        return invalid("device pointers must not be null");
    if (n_rows <= 0 || tokens_per_seq <= 0 || row_offset < 0) return invalid("B, G and T must be positive");
    if (row_offset + n_rows > kIntMax) return invalid("token count exceeds INT_MAX");
    if (V <= 0) return invalid("V must be positive");
    if (P < V) return invalid("P must be at least V");
    if (kernel != GRPO_B200_LOGITS_SEPARATE && kernel != GRPO_B200_LOGITS_FUSED)
        return invalid("unknown logits kernel selector");
    if (int rc = check_options(clip_eps, beta)) return rc;
    if (!workspace || workspace_bytes < grpo_b200_logits_workspace_bytes(n_rows) ||
        (reinterpret_cast<uintptr_t>(workspace) & 31u)) {
        set_error("workspace must be 32-byte aligned and hold grpo_b200_logits_workspace_bytes() bytes");
        return GRPO_B200_E_WORKSPACE;
    }
    LogitsArgs a;
    a.logits = logits;
    a.dlogits = dlogits;
    a.logp_old = logp_old;
    a.logp_ref = logp_ref;
    a.selected = selected;
    a.advantages = advantages;
    a.weights = weights;
    a.mask = mask;
    a.n_rows = n_rows;
    a.row_offset = row_offset;
    a.tokens_per_seq = tokens_per_seq;
    a.V = V;
    a.P = P;
    a.clip_eps = clip_eps;
    a.beta = beta;
    a.row_order = row_order;
    a.rows = static_cast<RowRecord*>(workspace);
    a.selected_logp = selected_logp;
    a.result = result;
    a.status = reinterpret_cast<int*>(a.rows + n_rows);
    a.counter = reinterpret_cast<unsigned*>(a.status) + 1;
    a.partials = reinterpret_cast<double*>(reinterpret_cast<unsigned char*>(a.status) + 32);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int variant = kernel == GRPO_B200_LOGITS_FUSED ? pick_resident_variant(logits, dlogits, V, P, n_rows) : -1;
    if (variant >= 0)
        GRPO_CUDA_TRY(launch_logits_resident(variant, check_inputs != 0, a, s));
    else
        GRPO_CUDA_TRY(launch_logits_streaming(check_inputs != 0, a, s));
    GRPO_CUDA_TRY(launch_logits_reduce(a, x, s));
    return GRPO_B200_OK;
}

}  // namespace

extern "C" {

int grpo_b200_logits(const float* logits, float* dlogits, const float* logp_old, const float* logp_ref,
                     const int32_t* selected, const float* advantages, const float* weights, const int32_t* mask,
                     int64_t n_rows, int64_t row_offset, int tokens_per_seq, int V, int P, float clip_eps,
                     float beta, int kernel, int check_inputs, float* selected_logp, const int32_t* row_order,
                     grpo_b200_result_t* result, void* workspace, size_t workspace_bytes,
                     grpo_b200_stream_t stream) {
    ExchangeArgs x = {};
    return logits_pass(logits, dlogits, logp_old, logp_ref, selected, advantages, weights, mask, n_rows, row_offset,
                       tokens_per_seq, V, P, clip_eps, beta, kernel, check_inputs, selected_logp, row_order, result,
                       workspace, workspace_bytes, x, stream);
}

size_t grpo_b200_row_order_bytes(int64_t n_rows) {
    // the order itself, then one scratch count per tile of 1024 rows
    return n_rows > 0 ? (static_cast<size_t>(n_rows) + 2 + (static_cast<size_t>(n_rows) + 1023) / 1024) * sizeof(int32_t)
                      : 0;
}

int grpo_b200_row_order(const int32_t* mask, int64_t n_rows, int32_t* order, grpo_b200_stream_t stream) {
    if (!mask || !order) return invalid("device pointers must not be null");
    if (n_rows <= 0 || n_rows > kIntMax) return invalid("n_rows must lie in [1, INT_MAX]");
    GRPO_CUDA_TRY(launch_row_order(mask, n_rows, order, reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

size_t grpo_b200_exchange_bytes(int64_t n_seq) {
    if (n_seq <= 0) return 0;
    return exchange_lengths_offset(n_seq) + static_cast<size_t>(n_seq) * sizeof(double);
}

int grpo_b200_exchange_create(int64_t n_seq, void** region) {
    if (!region || n_seq <= 0) return invalid("region must not be null and n_seq must be positive");
    void* p = nullptr;
    GRPO_CUDA_TRY(cudaMalloc(&p, grpo_b200_exchange_bytes(n_seq)));
    cudaError_t err = cudaMemset(p, 0, grpo_b200_exchange_bytes(n_seq));
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (err != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(err, "clearing the exchange region");
    }
    {
        std::lock_guard<std::mutex> lock(g_regions_mutex);
        g_regions[p] = n_seq;
    }
    *region = p;
    return GRPO_B200_OK;
}

int grpo_b200_exchange_set_timeout_cycles(int64_t cycles) {
    if (cycles <= 0) return invalid("the exchange timeout must be a positive number of SM clock cycles");
    g_exchange_timeout_cycles.store(cycles, std::memory_order_relaxed);
    return GRPO_B200_OK;
}

int grpo_b200_exchange_export(void* region, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed around as 64 bytes");
    if (!region || !handle) return invalid("region and handle must not be null");
    cudaIpcMemHandle_t h;
    GRPO_CUDA_TRY(cudaIpcGetMemHandle(&h, region));
    memcpy(handle, &h, sizeof(h));
    return GRPO_B200_OK;
}

int grpo_b200_exchange_open(const unsigned char handle[64], void** peer_region) {
    if (!handle || !peer_region) return invalid("handle and peer_region must not be null");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    GRPO_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *peer_region = p;
    return GRPO_B200_OK;
}

int grpo_b200_exchange_close(void* peer_region) {
    if (!peer_region) return GRPO_B200_OK;
    GRPO_CUDA_TRY(cudaIpcCloseMemHandle(peer_region));
    return GRPO_B200_OK;
}

int grpo_b200_exchange_destroy(void* region) {
    if (!region) return GRPO_B200_OK;
    {
        std::lock_guard<std::mutex> lock(g_regions_mutex);
        g_regions.erase(region);
    }
    GRPO_CUDA_TRY(cudaFree(region));
    return GRPO_B200_OK;
}

int grpo_b200_logits_sharded(const float* logits, float* dlogits, const float* logp_old, const float* logp_ref,
                             const int32_t* selected, const float* advantages, const float* weights,
                             const int32_t* mask, int64_t n_rows, int64_t row_offset, int tokens_per_seq, int V, int P,
                             float clip_eps, float beta, int kernel, int check_inputs, float* selected_logp,
                             const int32_t* row_order, grpo_b200_result_t* result, void* workspace,
                             size_t workspace_bytes, void* const* regions, int rank, int world, int64_t n_seq, const int32_t* next_mask,
                             int reduction, float length_alpha, float* next_weights, int32_t* next_meta,
                             double* next_lengths, grpo_b200_stream_t stream) {
    if (world < 1 || world > kExchangeMaxWorld) return invalid("world must lie in [1, 8]");
    if (rank < 0 || rank >= world) return invalid("rank must lie in [0, world)");
    if (!regions || !next_mask || !next_weights || !next_meta || n_seq <= 0)
        return invalid("regions, next_mask, next_weights and next_meta must not be null and n_seq must be positive");
    if (reduction < GRPO_B200_SEQUENCE_MEAN || reduction > GRPO_B200_LENGTH_WEIGHTED)
        return invalid("unknown reduction mode");
    if (!(length_alpha >= 0.0f && length_alpha <= 1.0f)) return invalid("length_alpha must be finite and in [0, 1]");
    if (tokens_per_seq > 0 && n_rows > 0 && row_offset >= 0 &&
        (row_offset + n_rows + tokens_per_seq - 1) / tokens_per_seq > n_seq)
        return invalid("rows reach beyond the last response");
    ExchangeArgs x = {};
    for (int r = 0; r < world; r++) {
        if (!regions[r]) return invalid("every rank's exchange region must be mapped");
        x.peers[r] = static_cast<unsigned char*>(regions[r]);
    }
    if (int rc = check_own_region(regions, rank, n_seq)) return rc;
    x.timeout_cycles = g_exchange_timeout_cycles.load(std::memory_order_relaxed);
    x.rank = rank;
    x.world = world;
    x.n_seq = n_seq;
    x.next_mask = next_mask;
    x.reduction = reduction;
    x.length_alpha = length_alpha;
    x.weights_out = next_weights;
    x.meta_out = next_meta;
    x.lengths_out = next_lengths;
    return logits_pass(logits, dlogits, logp_old, logp_ref, selected, advantages, weights, mask, n_rows, row_offset,
                       tokens_per_seq, V, P, clip_eps, beta, kernel, check_inputs, selected_logp, row_order, result,
                       workspace, workspace_bytes, x, stream);
}

int grpo_b200_lengths_sharded(const int32_t* mask, int64_t n_rows, int64_t row_offset, int tokens_per_seq,
                              int64_t n_seq, void* const* regions, int rank, int world, int reduction,
                              float length_alpha, float* weights, int32_t* meta, double* lengths,
                              grpo_b200_result_t* status, void* workspace, size_t workspace_bytes,
                              grpo_b200_stream_t stream) {
    if (world < 1 || world > kExchangeMaxWorld) return invalid("world must lie in [1, 8]");
    if (rank < 0 || rank >= world) return invalid("rank must lie in [0, world)");
    if (!mask || !regions || !weights || !meta || !status || n_seq <= 0)
        return invalid("mask, regions, weights, meta and status must not be null and n_seq must be positive");
    if (n_rows <= 0 || tokens_per_seq <= 0 || row_offset < 0) return invalid("B, G and T must be positive");
    if (row_offset + n_rows > kIntMax) return invalid("token count exceeds INT_MAX");
    if ((row_offset + n_rows + tokens_per_seq - 1) / tokens_per_seq > n_seq)
        return invalid("rows reach beyond the last response");
    if (reduction < GRPO_B200_SEQUENCE_MEAN || reduction > GRPO_B200_LENGTH_WEIGHTED)
        return invalid("unknown reduction mode");
    if (!(length_alpha >= 0.0f && length_alpha <= 1.0f)) return invalid("length_alpha must be finite and in [0, 1]");
    if (!workspace || workspace_bytes < grpo_b200_logits_workspace_bytes(n_rows) ||
        (reinterpret_cast<uintptr_t>(workspace) & 31u)) {
        set_error("workspace must be 32-byte aligned and hold grpo_b200_logits_workspace_bytes() bytes");
        return GRPO_B200_E_WORKSPACE;
    }
    ExchangeArgs x = {};
    for (int r = 0; r < world; r++) {
        if (!regions[r]) return invalid("every rank's exchange region must be mapped");
        x.peers[r] = static_cast<unsigned char*>(regions[r]);
    }
    if (int rc = check_own_region(regions, rank, n_seq)) return rc;
    x.timeout_cycles = g_exchange_timeout_cycles.load(std::memory_order_relaxed);
    x.rank = rank;
    x.world = world;
    x.n_seq = n_seq;
    x.next_mask = mask;
    x.reduction = reduction;
    x.length_alpha = length_alpha;
    x.weights_out = weights;
    x.meta_out = meta;
    x.lengths_out = lengths;
    // the reduce kernel with no rows to reduce: it counts, exchanges (an all-zero record rides along) and
    // derives the weights; the exchanged record (bad_inputs = -2 when a rank did not answer) goes to `status`
    LogitsArgs a = {};
    a.n_rows = n_rows;
    a.row_offset = row_offset;
    a.tokens_per_seq = tokens_per_seq;
    a.rows = static_cast<RowRecord*>(workspace);
    a.result = status;
    a.status = reinterpret_cast<int*>(a.rows + n_rows);
    a.counter = reinterpret_cast<unsigned*>(a.status) + 1;
    a.partials = reinterpret_cast<double*>(reinterpret_cast<unsigned char*>(a.status) + 32);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    GRPO_CUDA_TRY(cudaMemsetAsync(a.status, 0, 32, s));
    GRPO_CUDA_TRY(launch_logits_reduce(a, x, s));
    return GRPO_B200_OK;
}

int grpo_b200_sample_rows(const float* logits, int64_t n_rows, int V, int P, const int32_t* rows, int n_selected,
                          const double* coins, const int32_t* given_tokens, int32_t* tokens_out, float* logp_out,
                          double* lse_out, grpo_b200_stream_t stream) {
    if (!logits || !rows) return invalid("device pointers must not be null");
    if (n_rows <= 0 || n_rows > kIntMax) return invalid("n_rows must lie in [1, INT_MAX]");
    if (V <= 0) return invalid("V must be positive");
    if (P < V) return invalid("P must be at least V");
    if (n_selected <= 0) return invalid("n_selected must be positive");
    if ((coins == nullptr) == (given_tokens == nullptr)) return invalid("pass either coins or given_tokens");
    if (coins && !tokens_out) return invalid("tokens_out must not be null when tokens are drawn");
    GRPO_CUDA_TRY(launch_sample_rows(logits, n_rows, V, P, rows, n_selected, coins, given_tokens, tokens_out, logp_out,
                                     lse_out, reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

int grpo_b200_logits_set_variant(int variant) {
    if (set_forced_variant(variant) != 0) return invalid("no such kernel variant");
    return GRPO_B200_OK;
}

int grpo_b200_synthetic_logits(float* logits, int64_t n_rows, int64_t row_offset, int V, int P, float scale,
                               uint64_t seed, float tail_fill, grpo_b200_stream_t stream) {
    if (!logits) return invalid("device pointers must not be null");
    if (n_rows <= 0 || row_offset < 0 || row_offset + n_rows > kIntMax) return invalid("n_rows must lie in [1, INT_MAX]");
    if (V <= 0) return invalid("V must be positive");
    if (P < V) return invalid("P must be at least V");
    GRPO_CUDA_TRY(launch_synthetic_logits(logits, n_rows, row_offset, V, P, scale, seed, tail_fill,
                                          reinterpret_cast<cudaStream_t>(stream)));
    return GRPO_B200_OK;
}

const char* grpo_b200_logits_variant_name(int variant) { return resident_variant_name(variant); }

const char* grpo_b200_logits_plan(const void* logits, const void* dlogits, int V, int P, int64_t n_rows, int kernel) {
    if (kernel != GRPO_B200_LOGITS_FUSED) return "streaming";
    const int v = pick_resident_variant(logits, dlogits, V, P, n_rows);
    return v >= 0 ? resident_variant_name(v) : "streaming";
}

}  // extern "C"

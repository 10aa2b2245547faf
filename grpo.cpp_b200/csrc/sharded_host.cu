// Host side of token-sharded execution: one rank's resources and the reference-shaped call on them.
//
// The reference's multi-GPU callers are C++: one std::thread per device, each with its own
// cudaSetDevice, calling the library (apps/03_two_gpu_train.cu:200-215), and forked per-rank
// processes (apps/05_two_gpu_gpt2_grpo.cu:309-328).  A shard serves both: its exchange region is
// reached by the other ranks either through a CUDA IPC handle (processes) or directly, with peer
// access enabled (threads of one process).
//
// grpo_b200_logits_sharded_host is grpo_logits_cuda_device_inplace (src/cuda/grpo_loss_cuda.cu:774-817)
// for one rank's rows of a batch: host metadata in, device logits replaced in place, the GLOBAL
// loss terms out.  Per call: one packed pinned host-to-device copy, the row order, the lengths
// exchange, the row kernel and the reduce kernel (with the record exchange) enqueued back to back
// without an intermediate synchronisation, one pinned read-back, and the reference's error
// contract applied to the global quantities.
#include <cmath>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"
#include "host_util.hpp"

using namespace grpo_b200;
using namespace grpo_b200::host;

struct grpo_b200_shard {
    int device = -1;
    int rank = 0, world = 1;
    int64_t n_seq = 0;
    int tokens_per_seq = 0;
    int V = 0, P = 0;
    int64_t row_offset = 0, n_rows = 0;
    void* region = nullptr;                      // own exchange region
    void* regions[kExchangeMaxWorld] = {};       // every rank's region as reachable from this rank
    bool opened_ipc[kExchangeMaxWorld] = {};     // regions[r] came from grpo_b200_exchange_open
    bool connected = false;
    char* dev = nullptr;                         // packed device metadata, then results, workspace, row order
    char* pinned = nullptr;                      // host image of the packed metadata, then the read-back block
    size_t packed_bytes = 0;
    // device views
    float* old_d = nullptr;
    float* ref_d = nullptr;
    int32_t* sel_d = nullptr;
    int32_t* mask_d = nullptr;
    float* adv_d = nullptr;
    float* weights_d = nullptr;
    char* readback_d = nullptr;                  // {record[5], lengths status[5], meta[2]} contiguous
    void* work_d = nullptr;
    size_t work_bytes = 0;
    int32_t* order_d = nullptr;
    cudaStream_t stream = nullptr;               // the legacy default stream, like the reference's calls
};

namespace {

size_t slice256(size_t bytes) { return (bytes + 255) & ~static_cast<size_t>(255); }

struct Readback {
    grpo_b200_result_t record;
    grpo_b200_result_t lengths_status;
    int32_t meta[2];
    int32_t pad[2];
};

int cuda_error(cudaError_t err, const char* what) { return cuda_fail(err, what); }

struct DeviceGuard {
    int previous = -1;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&previous) != cudaSuccess) previous = -1;
        if (previous != device) cudaSetDevice(device);
    }
    ~DeviceGuard() {
        if (previous >= 0) cudaSetDevice(previous);
    }
};

}  // namespace

extern "C" {

int grpo_b200_shard_create(int rank, int world, int64_t n_seq, int tokens_per_seq, int V, int P, int64_t row_offset,
                           int64_t n_rows, grpo_b200_shard_t* out) {
    if (!out) return invalid("out must not be null");
    *out = nullptr;
    if (world < 1 || world > kExchangeMaxWorld) return invalid("world must lie in [1, 8]");
    if (rank < 0 || rank >= world) return invalid("rank must lie in [0, world)");
    if (n_seq <= 0 || tokens_per_seq <= 0 || n_rows <= 0 || row_offset < 0) return invalid("B, G and T must be positive");
    if (n_seq > 2147483647LL) return invalid("sequence count exceeds INT_MAX");
    if (n_seq * static_cast<int64_t>(tokens_per_seq) > 2147483647LL) return invalid("token count exceeds INT_MAX");
    if (row_offset + n_rows > n_seq * static_cast<int64_t>(tokens_per_seq))
        return invalid("local rows reach past the end of the batch");
    if (V <= 0) return invalid("V must be positive");
    if (P < V) return invalid("P must be at least V");
    grpo_b200_shard* s = new (std::nothrow) grpo_b200_shard();
    if (!s) return invalid("out of host memory");
    s->rank = rank;
    s->world = world;
    s->n_seq = n_seq;
    s->tokens_per_seq = tokens_per_seq;
    s->V = V;
    s->P = P;
    s->row_offset = row_offset;
    s->n_rows = n_rows;
    cudaError_t err = cudaGetDevice(&s->device);
    int rc = GRPO_B200_OK;
    const size_t n = static_cast<size_t>(n_rows), S = static_cast<size_t>(n_seq);
    // packed metadata (one upload): old, ref, selected, mask, advantages
    s->packed_bytes = 4 * slice256(n * 4) + slice256(S * 4);
    s->work_bytes = grpo_b200_logits_workspace_bytes(n_rows);
    const size_t order_bytes = grpo_b200_row_order_bytes(n_rows);
    const size_t total = s->packed_bytes + slice256(S * 4) + slice256(sizeof(Readback)) + slice256(s->work_bytes) +
                         slice256(order_bytes);
    if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&s->dev), total);
    if (err == cudaSuccess) err = cudaMemset(s->dev, 0, total);
    if (err == cudaSuccess) err = cudaMallocHost(reinterpret_cast<void**>(&s->pinned), s->packed_bytes + slice256(sizeof(Readback)));
    if (err != cudaSuccess) {
        rc = cuda_error(err, "allocating a shard's buffers");
    } else {
        rc = grpo_b200_exchange_create(n_seq, &s->region);
    }
    if (rc != GRPO_B200_OK) {
        grpo_b200_shard_destroy(s);
        return rc;
    }
    char* p = s->dev;
    s->old_d = reinterpret_cast<float*>(p);
    p += slice256(n * 4);
    s->ref_d = reinterpret_cast<float*>(p);
    p += slice256(n * 4);
    s->sel_d = reinterpret_cast<int32_t*>(p);
    p += slice256(n * 4);
    s->mask_d = reinterpret_cast<int32_t*>(p);
    p += slice256(n * 4);
    s->adv_d = reinterpret_cast<float*>(p);
    p += slice256(S * 4);
    s->weights_d = reinterpret_cast<float*>(p);
    p += slice256(S * 4);
    s->readback_d = p;
    p += slice256(sizeof(Readback));
    s->work_d = p;
    p += slice256(s->work_bytes);
    s->order_d = reinterpret_cast<int32_t*>(p);
    s->regions[rank] = s->region;
    s->connected = world == 1;
    *out = s;
    return GRPO_B200_OK;
}

int grpo_b200_shard_export(grpo_b200_shard_t s, unsigned char handle[64]) {
    if (!s || !handle) return invalid("shard and handle must not be null");
    DeviceGuard guard(s->device);
    return grpo_b200_exchange_export(s->region, handle);
}

int grpo_b200_shard_connect_ipc(grpo_b200_shard_t s, const unsigned char* handles) {
    if (!s || !handles) return invalid("shard and handles must not be null");
    DeviceGuard guard(s->device);
    for (int r = 0; r < s->world; r++) {
        if (r == s->rank || s->regions[r]) continue;
        void* peer = nullptr;
        if (int rc = grpo_b200_exchange_open(handles + 64 * static_cast<size_t>(r), &peer)) return rc;
        s->regions[r] = peer;
        s->opened_ipc[r] = true;
    }
    s->connected = true;
    return GRPO_B200_OK;
}

int grpo_b200_shard_connect_local(grpo_b200_shard_t s, grpo_b200_shard_t const* all) {
    if (!s || !all) return invalid("shard and the list of shards must not be null");
    DeviceGuard guard(s->device);
    for (int r = 0; r < s->world; r++) {
        if (r == s->rank) continue;
        const grpo_b200_shard* peer = all[r];
        if (!peer || peer->rank != r || peer->world != s->world || peer->n_seq != s->n_seq)
            return invalid("the list must hold every rank's shard of the same batch, in rank order");
        if (peer->device != s->device) {
            int can = 0;
            GRPO_CUDA_TRY(cudaDeviceCanAccessPeer(&can, s->device, peer->device));
            if (!can) return invalid("this rank's device cannot reach a peer's memory");
            const cudaError_t err = cudaDeviceEnablePeerAccess(peer->device, 0);
            if (err != cudaSuccess && err != cudaErrorPeerAccessAlreadyEnabled) return cuda_error(err, "enabling peer access");
            if (err == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        }
        s->regions[r] = peer->region;
    }
    s->connected = true;
    return GRPO_B200_OK;
}

int grpo_b200_shard_destroy(grpo_b200_shard_t s) {
    if (!s) return GRPO_B200_OK;
    if (s->device >= 0) {
        DeviceGuard guard(s->device);
        cudaStreamSynchronize(s->stream);
        for (int r = 0; r < kExchangeMaxWorld; r++)
            if (s->opened_ipc[r] && s->regions[r]) grpo_b200_exchange_close(s->regions[r]);
        if (s->region) grpo_b200_exchange_destroy(s->region);
        if (s->dev) cudaFree(s->dev);
        if (s->pinned) cudaFreeHost(s->pinned);
    }
    delete s;
    return GRPO_B200_OK;
}

int grpo_b200_logits_sharded_host(grpo_b200_shard_t s, float* logits_and_dlogits, const float* logp_old,
                                  size_t n_logp_old, const float* logp_ref, size_t n_logp_ref, const int32_t* selected,
                                  size_t n_selected, const float* advantages, size_t n_advantages, const int32_t* mask,
                                  size_t n_mask, float clip_eps, float beta, int reduction, float length_alpha,
                                  int kernel, float* stats_out, int* valid_tokens_out) {
    if (!s) return invalid("shard must not be null");
    if (logits_and_dlogits == nullptr) return invalid("logits_and_dlogits must not be null");
    if (!stats_out || !valid_tokens_out) return invalid("stats_out and valid_tokens_out must not be null");
    if (!s->connected) return invalid("the shard is not connected to the other ranks' exchange regions");
    int current = -1;
    GRPO_CUDA_TRY(cudaGetDevice(&current));
    if (current != s->device) return invalid("the shard belongs to another device than the current one");
    const size_t n = static_cast<size_t>(s->n_rows), S = static_cast<size_t>(s->n_seq);
    // the reference's checks, on this rank's slice (src/cuda/grpo_loss_cuda.cu:584-618, 676-697)
    if (int rc = expect_size("selected_tokens", n_selected, n)) return rc;
    Shape shape;
    shape.sequences = S;
    shape.tokens = n;
    const Options opt{clip_eps, beta, length_alpha, reduction};
    if (reduction < GRPO_B200_SEQUENCE_MEAN || reduction > GRPO_B200_LENGTH_WEIGHTED) return invalid("unknown reduction mode");
    if (int rc = validate_sizes(false, 0, n_logp_old, n_logp_ref, n_advantages, n_mask, shape, opt)) return rc;
    // the checks and the pinned image of the one packed upload in a single vectorised pass per array; when a
    // pass finds something wrong the ordered validators say which complaint the reference would raise first
    char* h = s->pinned;
    auto host_of = [&](const void* dev_ptr) { return h + (static_cast<const char*>(dev_ptr) - s->dev); };
    unsigned bad = 0;
    int local_valid = 0;
    bad |= copy_and_count_mask(mask, reinterpret_cast<int32_t*>(host_of(s->mask_d)), static_cast<int>(n), local_valid);
    bad |= copy_and_check_finite(reinterpret_cast<const uint32_t*>(logp_old), reinterpret_cast<uint32_t*>(host_of(s->old_d)), n);
    bad |= copy_and_check_finite(reinterpret_cast<const uint32_t*>(logp_ref), reinterpret_cast<uint32_t*>(host_of(s->ref_d)), n);
    bad |= copy_and_check_selected(selected, mask, reinterpret_cast<int32_t*>(host_of(s->sel_d)), n, static_cast<uint32_t>(s->V));
    bad |= copy_and_check_finite(reinterpret_cast<const uint32_t*>(advantages), reinterpret_cast<uint32_t*>(host_of(s->adv_d)), S);
    if (bad) {
        if (int rc = validate_inputs(nullptr, 0, logp_old, n_logp_old, logp_ref, n_logp_ref, advantages, n_advantages, mask,
                                     n_mask, shape, opt))
            return rc;
        size_t first_bad;
        if (check_selected(selected, mask, n, s->V, first_bad)) return invalid("selected token is outside the vocabulary");
    }
    if (kernel != GRPO_B200_LOGITS_SEPARATE && kernel != GRPO_B200_LOGITS_FUSED)
        return invalid("unknown logits kernel selector");
    GRPO_CUDA_TRY(cudaMemcpyAsync(s->dev, h, s->packed_bytes, cudaMemcpyHostToDevice, s->stream));

    auto* rb_d = reinterpret_cast<Readback*>(s->readback_d);
    grpo_b200_stream_t st = reinterpret_cast<grpo_b200_stream_t>(s->stream);
    // row order (local work first: the ranks reach the exchange a little closer together), global lengths ->
    // weights (exchange 1), row kernel + reduce kernel with the record exchange (exchange 2; it also recounts
    // the same mask for a next pass, which costs nothing and keeps one kernel)
    if (int rc = grpo_b200_row_order(s->mask_d, s->n_rows, s->order_d, st)) return rc;
    if (int rc = grpo_b200_lengths_sharded(s->mask_d, s->n_rows, s->row_offset, s->tokens_per_seq, s->n_seq, s->regions,
                                           s->rank, s->world, reduction, length_alpha, s->weights_d, rb_d->meta, nullptr,
                                           &rb_d->lengths_status, s->work_d, s->work_bytes, st))
        return rc;
    if (int rc = grpo_b200_logits_sharded(logits_and_dlogits, logits_and_dlogits, s->old_d, s->ref_d, s->sel_d, s->adv_d,
                                          s->weights_d, s->mask_d, s->n_rows, s->row_offset, s->tokens_per_seq, s->V, s->P,
                                          clip_eps, beta, kernel, 0, nullptr, s->order_d, &rb_d->record, s->work_d,
                                          s->work_bytes, s->regions, s->rank, s->world, s->n_seq, s->mask_d, reduction,
                                          length_alpha, s->weights_d, rb_d->meta, nullptr, st))
        return rc;
    auto* rb_h = reinterpret_cast<Readback*>(s->pinned + s->packed_bytes);
    GRPO_CUDA_TRY(cudaMemcpyAsync(rb_h, rb_d, sizeof(Readback), cudaMemcpyDeviceToHost, s->stream));
    GRPO_CUDA_TRY(cudaStreamSynchronize(s->stream));

    // the reference's error contract, on the global quantities (src/cuda/grpo_loss_cuda.cu:44-46, 814-815)
    if (rb_h->lengths_status.bad_inputs < 0.0) {
        set_error("CUDA error: the exchange between ranks timed out");
        return GRPO_B200_E_CUDA;
    }
    if (rb_h->record.bad_inputs < 0.0) return fill_stats(rb_h->record, stats_out, "");
    if (rb_h->meta[1] != 0) return invalid("every sequence needs at least one valid token");
    *valid_tokens_out = rb_h->meta[0];
    return fill_stats(rb_h->record, stats_out, "CUDA logits loss became non-finite");
}

}  // extern "C"

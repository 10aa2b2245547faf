// Selected-token GRPO loss (K1), valid-token counting, response weights and group advantages.
//
// K1 replaces the reference's grpo_loss_block_kernel / grpo_loss_atomic_kernel
// (src/cuda/grpo_loss_cuda.cu:97-179).  Differences by design:
//   * 128-bit loads: one thread owns four consecutive tokens per step, so the three
//     log-probability streams, the mask and dlogp move as float4/int4 (20 B per active token,
//     8 B per fully masked group of the input streams is never fetched);
//   * the three sums are carried in double from fp32 per-token products -- the same recipe as
//     the CPU path (src/cpu/grpo_loss.cpp:114-116,157-159) -- through a fixed shuffle tree, a
//     fixed warp-order tree per block and a fixed-order pass over per-block partials by the block
//     that takes the last ticket: no floating-point atomics, bit-identical results from run to
//     run, one kernel per pass;
//   * no accumulator memset: the last block overwrites the result record (the only word cleared
//     is the integer ticket counter, and not even that when the library owns the buffers).
#include <mutex>

#include "common.cuh"

namespace grpo_b200 {

namespace {

constexpr int kLossThreads = 256;
constexpr int kLossMaxBlocks = 2048;  // bounds the per-block partials the last block reads
constexpr int kPartialWidth = 5;      // loss, pg, kl, bad gradients, bad inputs

struct Acc {
    double v[kPartialWidth];
};

__device__ __forceinline__ float one_token(const LossArgs& a, float lp_new, float lp_old, float lp_ref,
                                           int m, long long seq, Acc& acc) {
    if (m == 0) return 0.0f;
    const float adv = __ldg(a.advantages + seq);
    const float w = __ldg(a.weights + seq);
    const TokenTerms t = token_terms<false>(lp_new, lp_old, lp_ref, adv, w, a.clip_eps, a.beta);
    acc.v[0] += static_cast<double>(t.loss);
    acc.v[1] += static_cast<double>(t.pg);
    acc.v[2] += static_cast<double>(t.kl);
    if (!finite_f(t.grad)) acc.v[3] += 1.0;
    if (m != 1 || !finite_f(lp_new) || !finite_f(lp_old) || !finite_f(lp_ref)) acc.v[4] += 1.0;
    return t.grad;
}

// TICKET: the block that takes the last ticket also adds the per-block partials in index order and
// writes the result record, so the pass is one kernel launch (after a 4-byte clear of the counter).
template <bool VEC, int THREADS, bool TICKET>
__global__ void __launch_bounds__(THREADS) token_loss_kernel(const LossArgs a) {
    __shared__ double scratch[kPartialWidth * THREADS / 32];
    __shared__ int is_last;
    Acc acc;
#pragma unroll
    for (int k = 0; k < kPartialWidth; k++) acc.v[k] = 0.0;

    const long long tid = static_cast<long long>(blockIdx.x) * THREADS + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * THREADS;
    const long long T = a.tokens_per_seq;

    if (VEC) {
        const long long groups = a.n_tokens >> 2;
        for (long long g = tid; g < groups; g += stride) {
            const int4 m = __ldg(reinterpret_cast<const int4*>(a.mask) + g);
            float4 grad = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if ((m.x | m.y | m.z | m.w) != 0) {
                const float4 ln = __ldcs(reinterpret_cast<const float4*>(a.logp_new) + g);
                const float4 lo = __ldcs(reinterpret_cast<const float4*>(a.logp_old) + g);
                const float4 lr = __ldcs(reinterpret_cast<const float4*>(a.logp_ref) + g);
                const long long i0 = a.token_offset + 4 * g;
                long long seq = i0 / T;
                long long rem = i0 - seq * T;
                grad.x = one_token(a, ln.x, lo.x, lr.x, m.x, seq, acc);
                if (++rem == T) { rem = 0; ++seq; }
                grad.y = one_token(a, ln.y, lo.y, lr.y, m.y, seq, acc);
                if (++rem == T) { rem = 0; ++seq; }
                grad.z = one_token(a, ln.z, lo.z, lr.z, m.z, seq, acc);
                if (++rem == T) { rem = 0; ++seq; }
                grad.w = one_token(a, ln.w, lo.w, lr.w, m.w, seq, acc);
            }
            __stcs(reinterpret_cast<float4*>(a.dlogp) + g, grad);
        }
        // the up-to-three tokens past the last full group
        const long long i = (groups << 2) + tid;
        if (i < a.n_tokens) {
            const int m = a.mask[i];
            float g1 = 0.0f;
            if (m != 0)
                g1 = one_token(a, a.logp_new[i], a.logp_old[i], a.logp_ref[i], m,
                               (a.token_offset + i) / T, acc);
            a.dlogp[i] = g1;
        }
    } else {
        for (long long i = tid; i < a.n_tokens; i += stride) {
            const int m = a.mask[i];
            float g1 = 0.0f;
            if (m != 0)
                g1 = one_token(a, a.logp_new[i], a.logp_old[i], a.logp_ref[i], m,
                               (a.token_offset + i) / T, acc);
            a.dlogp[i] = g1;
        }
    }

    block_sum<THREADS, kPartialWidth>(acc.v, scratch);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int k = 0; k < kPartialWidth; k++) a.partials[blockIdx.x * kPartialWidth + k] = acc.v[k];
        if (TICKET) {
            __threadfence();
            is_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
        }
    }
    if (!TICKET) return;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x == 0) *a.counter = 0u;  // every ticket is taken: the counter is left as it was found
    double v[kPartialWidth];
#pragma unroll
    for (int k = 0; k < kPartialWidth; k++) v[k] = 0.0;
    for (unsigned b = threadIdx.x; b < gridDim.x; b += THREADS) {
#pragma unroll
        for (int k = 0; k < kPartialWidth; k++) v[k] += __ldcg(a.partials + b * kPartialWidth + k);
    }
    block_sum<THREADS, kPartialWidth>(v, scratch);
    if (threadIdx.x == 0) {
        a.result->loss = v[0];
        a.result->pg_loss = v[1];
        a.result->kl = v[2];
        a.result->bad_grads = v[3];
        a.result->bad_inputs = v[4];
    }
}

// One block walks the per-block partials in index order and overwrites the result record.
__global__ void __launch_bounds__(256) loss_finalize_kernel(const double* __restrict__ partials, int n,
                                                            grpo_b200_result_t* result) {
    __shared__ double scratch[kPartialWidth * 256 / 32];
    double v[kPartialWidth];
#pragma unroll
    for (int k = 0; k < kPartialWidth; k++) v[k] = 0.0;
    for (int b = threadIdx.x; b < n; b += 256) {
#pragma unroll
        for (int k = 0; k < kPartialWidth; k++) v[k] += partials[b * kPartialWidth + k];
    }
    block_sum<256, kPartialWidth>(v, scratch);
    if (threadIdx.x == 0) {
        result->loss = v[0];
        result->pg_loss = v[1];
        result->kl = v[2];
        result->bad_grads = v[3];
        result->bad_inputs = v[4];
    }
}

// One warp per response: counts the non-zero mask entries of its local token range.
// LEN is int32_t, or double for the packed exchange buffer of the token-sharded path.
template <class LEN>
__global__ void __launch_bounds__(256) count_lengths_kernel(const int32_t* __restrict__ mask, long long n_rows,
                                                            long long row_offset, long long T, long long n_seq,
                                                            LEN* __restrict__ lengths) {
    const long long seq = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) >> 5;
    if (seq >= n_seq) return;
    const int lane = threadIdx.x & 31;
    long long lo = seq * T, hi = lo + T;
    if (lo < row_offset) lo = row_offset;
    if (hi > row_offset + n_rows) hi = row_offset + n_rows;
    int count = 0;
    for (long long i = lo + lane; i < hi; i += 32) count += __ldg(mask + (i - row_offset)) != 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) count += __shfl_down_sync(0xffffffffu, count, o);
    if (lane == 0) lengths[seq] = static_cast<LEN>(count);
}

// Single block: total of the lengths, number of empty responses, then the weights with the
// reference's fp32 expressions (src/cuda/grpo_loss_cuda.cu:43-55).  The power is evaluated in
// double and rounded, which reproduces a correctly rounded powf.
template <class LEN>
__global__ void __launch_bounds__(1024) weights_kernel(const LEN* __restrict__ lengths, long long n_seq,
                                                       int reduction, float alpha, float* __restrict__ weights,
                                                       int32_t* __restrict__ meta) {
    __shared__ double scratch[2 * 1024 / 32 + 1];
    block_weights<1024>(lengths, n_seq, reduction, alpha, weights, meta, scratch);
}

// Stable partition of the row indices by mask: order = {n_active, n_masked, active rows ascending,
// masked rows ascending}, in two launches over tiles of 1024 rows.  The first counts each tile's
// active rows into a scratch tail of `order`; the second gives every tile its offsets (sum of the
// counts before it) and scatters its rows, warp ballots providing the positions inside the tile.
constexpr int kOrderTile = 1024;

__global__ void __launch_bounds__(kOrderTile) row_order_count_kernel(const int32_t* __restrict__ mask,
                                                                     long long n_rows, int32_t* __restrict__ counts) {
    __shared__ int warp_count[kOrderTile / 32];
    const long long i = static_cast<long long>(blockIdx.x) * kOrderTile + threadIdx.x;
    const bool active = i < n_rows && mask[i] != 0;
    const unsigned bits = __ballot_sync(0xffffffffu, active);
    if ((threadIdx.x & 31) == 0) warp_count[threadIdx.x >> 5] = __popc(bits);
    __syncthreads();
    if (threadIdx.x < 32) {
        int c = warp_count[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
        if (threadIdx.x == 0) counts[blockIdx.x] = c;
    }
}

__global__ void __launch_bounds__(kOrderTile) row_order_scatter_kernel(const int32_t* __restrict__ mask,
                                                                       long long n_rows,
                                                                       const int32_t* __restrict__ counts,
                                                                       int32_t* __restrict__ order) {
    __shared__ int warp_count[kOrderTile / 32];
    __shared__ long long sums[2];  // active rows before this tile; active rows in all
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // every block adds up the tile counts (a few hundred at most for the batches this serves)
    long long before = 0, all = 0;
    for (unsigned b = tid; b < gridDim.x; b += kOrderTile) {
        const int c = counts[b];
        all += c;
        if (b < blockIdx.x) before += c;
    }
    __shared__ long long red[2][kOrderTile / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        before += __shfl_down_sync(0xffffffffu, before, o);
        all += __shfl_down_sync(0xffffffffu, all, o);
    }
    if (lane == 0) {
        red[0][warp] = before;
        red[1][warp] = all;
    }
    const long long i = static_cast<long long>(blockIdx.x) * kOrderTile + tid;
    const bool in_range = i < n_rows;
    const bool active = in_range && mask[i] != 0;
    const unsigned bits = __ballot_sync(0xffffffffu, active);
    if (lane == 0) warp_count[warp] = __popc(bits);
    __syncthreads();
    if (tid == 0) {
        long long s0 = 0, s1 = 0;
        for (int w = 0; w < kOrderTile / 32; w++) {
            s0 += red[0][w];
            s1 += red[1][w];
        }
        sums[0] = s0;
        sums[1] = s1;
    }
    int in_tile = __popc(bits & ((1u << lane) - 1u));  // active rows before this one: in its warp ...
    for (int w = 0; w < warp; w++) in_tile += warp_count[w];  // ... and in the tile's earlier warps
    __syncthreads();
    const long long active_before = sums[0] + in_tile;
    if (in_range) {
        if (active)
            order[2 + active_before] = static_cast<int32_t>(i);
        else
            order[2 + sums[1] + (i - active_before)] = static_cast<int32_t>(i);
    }
    if (blockIdx.x == 0 && tid == 0) {
        order[0] = static_cast<int32_t>(sums[1]);
        order[1] = static_cast<int32_t>(n_rows - sums[1]);
    }
}

// One thread per prompt walks its G rewards in order: Welford mean / M2 in double with
// unfused IEEE operations, exactly the CPU sequence (src/cpu/grpo_loss.cpp:31-52).
__global__ void __launch_bounds__(256) group_advantages_kernel(const float* __restrict__ rewards, int B, int G,
                                                               int mode, float eps, float* __restrict__ adv,
                                                               int32_t* __restrict__ meta) {
    __shared__ double scratch[256 / 32];
    double bad[1] = {0.0};
    for (int b = threadIdx.x; b < B; b += 256) {
        const float* r = rewards + static_cast<long long>(b) * G;
        float* a = adv + static_cast<long long>(b) * G;
        const float first = r[0];
        bool same = true;
        for (int g = 0; g < G; g++) {
            const float x = r[g];
            same = same && (x == first);
            if (!finite_f(x)) bad[0] += 1.0;
        }
        if (same) {
            for (int g = 0; g < G; g++) a[g] = 0.0f;
            continue;
        }
        double mean = 0.0, m2 = 0.0;
        for (int g = 0; g < G; g++) {
            const double x = r[g];
            const double delta = __dsub_rn(x, mean);
            mean = __dadd_rn(mean, __ddiv_rn(delta, static_cast<double>(g + 1)));
            m2 = __dadd_rn(m2, __dmul_rn(delta, __dsub_rn(x, mean)));
        }
        const double var = __ddiv_rn(m2, static_cast<double>(G));
        const double denom = mode == GRPO_B200_ADV_STANDARDIZED ? __dsqrt_rn(__dadd_rn(var, static_cast<double>(eps))) : 1.0;
        for (int g = 0; g < G; g++) {
            const float out = static_cast<float>(__ddiv_rn(__dsub_rn(static_cast<double>(r[g]), mean), denom));
            if (!finite_f(out)) bad[0] += 1.0;
            a[g] = out;
        }
    }
    block_sum<256, 1>(bad, scratch);
    if (threadIdx.x == 0) meta[0] = static_cast<int32_t>(bad[0]);
}

int sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
    return sms;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int loss_grid_blocks(long long n_tokens) {
    const long long groups = (n_tokens + 3) / 4;
    long long blocks = (groups + kLossThreads - 1) / kLossThreads;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks > kLossMaxBlocks) blocks = kLossMaxBlocks;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

cudaError_t launch_loss(const LossArgs& a, bool clear_counter, cudaStream_t stream) {
    const bool vec = aligned16(a.logp_new) && aligned16(a.logp_old) && aligned16(a.logp_ref) &&
                     aligned16(a.mask) && aligned16(a.dlogp);
    const int blocks = loss_grid_blocks(a.n_tokens);
    if (clear_counter) {
        cudaError_t err = cudaMemsetAsync(a.counter, 0, sizeof(unsigned), stream);
        if (err != cudaSuccess) return err;
    }
    if (vec)
        token_loss_kernel<true, kLossThreads, true><<<blocks, kLossThreads, 0, stream>>>(a);
    else
        token_loss_kernel<false, kLossThreads, true><<<blocks, kLossThreads, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_count_lengths(const int32_t* mask, long long n_rows, long long row_offset, int tokens_per_seq,
                                 long long n_seq, int32_t* lengths, cudaStream_t stream) {
    const long long threads = n_seq * 32;
    const long long blocks = (threads + 255) / 256;
    count_lengths_kernel<int32_t><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(mask, n_rows, row_offset, tokens_per_seq,
                                                                            n_seq, lengths);
    return cudaGetLastError();
}

cudaError_t launch_weights(const int32_t* lengths, long long n_seq, int reduction, float alpha, float* weights,
                           int32_t* meta, cudaStream_t stream) {
    weights_kernel<int32_t><<<1, 1024, 0, stream>>>(lengths, n_seq, reduction, alpha, weights, meta);
    return cudaGetLastError();
}

cudaError_t launch_count_lengths_f64(const int32_t* mask, long long n_rows, long long row_offset, int tokens_per_seq,
                                     long long n_seq, double* lengths, cudaStream_t stream) {
    const long long blocks = (n_seq * 32 + 255) / 256;
    count_lengths_kernel<double><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(mask, n_rows, row_offset,
                                                                                   tokens_per_seq, n_seq, lengths);
    return cudaGetLastError();
}

cudaError_t launch_weights_f64(const double* lengths, long long n_seq, int reduction, float alpha, float* weights,
                               int32_t* meta, cudaStream_t stream) {
    weights_kernel<double><<<1, 1024, 0, stream>>>(lengths, n_seq, reduction, alpha, weights, meta);
    return cudaGetLastError();
}

cudaError_t launch_row_order(const int32_t* mask, long long n_rows, int32_t* order, cudaStream_t stream) {
    const unsigned tiles = static_cast<unsigned>((n_rows + kOrderTile - 1) / kOrderTile);
    int32_t* counts = order + 2 + n_rows;  // scratch tail of the order buffer
    row_order_count_kernel<<<tiles, kOrderTile, 0, stream>>>(mask, n_rows, counts);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    row_order_scatter_kernel<<<tiles, kOrderTile, 0, stream>>>(mask, n_rows, counts, order);
    return cudaGetLastError();
}

cudaError_t launch_group_advantages(const float* rewards, int B, int G, int mode, float eps, float* advantages,
                                    int32_t* meta, cudaStream_t stream) {
    group_advantages_kernel<<<1, 256, 0, stream>>>(rewards, B, G, mode, eps, advantages, meta);
    return cudaGetLastError();
}

}  // namespace grpo_b200

// ---------------------------------------------------------------------------------------------
// Selected-token loss for callers that have no device memory to lend and may not allocate any.
// ---------------------------------------------------------------------------------------------
namespace grpo_b200 {
namespace {

constexpr long long kNoAllocMaxTokens = 1LL << 24;  // 16,777,216 tokens per call
constexpr int kNoAllocBlocks = kLossMaxBlocks;      // as many partial slots as the ordinary entry point's grid can have

// The scratch the ordinary entry point takes from its caller lives here instead: 2048 x 5 doubles
// (80 KB) of per-block partial sums -- the same number of slots, so both entry points cut a batch
// into the same blocks and add the same partials in the same order.  Every GPU that loads this
// library keeps the array until the process exits.  In host code this name is only a handle for
// the runtime, not a device address.
static __device__ __align__(256) double g_noalloc_partials[kNoAllocBlocks * kPartialWidth];

std::mutex g_noalloc_mutex;
double* g_noalloc_ptr[64] = {nullptr};  // per device: the array's device address, looked up once

}  // namespace
}  // namespace grpo_b200

extern "C" int grpo_b200_loss_noalloc(const float* logp_new, const float* logp_old, const float* logp_ref,
                                      const float* advantages, const float* weights, const int32_t* mask,
                                      int64_t n_tokens, int64_t token_offset, int tokens_per_seq, float clip_eps,
                                      float beta, float* dlogp, grpo_b200_result_t* result,
                                      grpo_b200_stream_t stream) {
    using namespace grpo_b200;
    if (!logp_new || !logp_old || !logp_ref || !advantages || !weights || !mask || !dlogp || !result) {
        set_error("device pointers must not be null");
        return GRPO_B200_E_INVALID;
    }
    if (n_tokens <= 0 || tokens_per_seq <= 0 || token_offset < 0) {
        set_error("B, G and T must be positive");
        return GRPO_B200_E_INVALID;
    }
    if (n_tokens > kNoAllocMaxTokens) {
        set_error("grpo_b200_loss_noalloc takes at most %lld tokens per call (got %lld); use grpo_b200_loss with a "
                  "caller-provided workspace for larger batches",
                  kNoAllocMaxTokens, static_cast<long long>(n_tokens));
        return GRPO_B200_E_INVALID;
    }
    if (token_offset + n_tokens > 2147483647LL) {
        set_error("token count exceeds INT_MAX");
        return GRPO_B200_E_INVALID;
    }
    if (!(clip_eps >= 0.0f && clip_eps < 1.0f)) {
        set_error("clip_eps must be finite and in [0, 1)");
        return GRPO_B200_E_INVALID;
    }
    if (!(beta >= 0.0f && beta <= 3.402823466e+38f)) {
        set_error("beta must be finite and non-negative");
        return GRPO_B200_E_INVALID;
    }

    // Set-up, once per device and with that device current: ask the runtime where the array lives
    // on THIS device.  Passing the symbol itself to a kernel would hand it a host-side address.
    // The address is kept for the life of the process: a cudaDeviceReset in between would leave it
    // stale (the header says so).
    int dev = 0;
    GRPO_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("device index %d is outside the range this entry point tracks", dev);
        return GRPO_B200_E_INVALID;
    }
    double* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_ptr[dev] == nullptr) {
            void* ptr = nullptr;
            GRPO_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_partials));
            g_noalloc_ptr[dev] = static_cast<double*>(ptr);
        }
        scratch = g_noalloc_ptr[dev];
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
    a.partials = scratch;
    a.counter = nullptr;  // two-launch form: no ticket

    // Same kernels as grpo_b200_loss, with the grid capped at the number of partial slots held here.
    // Every block overwrites its own slot and the finalize pass reads exactly `blocks` slots, so
    // nothing left over from an earlier call is ever read and nothing needs clearing.
    int blocks = loss_grid_blocks(n_tokens);
    if (blocks > kNoAllocBlocks) blocks = kNoAllocBlocks;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bool vec = aligned16(logp_new) && aligned16(logp_old) && aligned16(logp_ref) && aligned16(mask) &&
                     aligned16(dlogp);
    if (vec)
        token_loss_kernel<true, kLossThreads, false><<<blocks, kLossThreads, 0, s>>>(a);
    else
        token_loss_kernel<false, kLossThreads, false><<<blocks, kLossThreads, 0, s>>>(a);
    GRPO_CUDA_TRY(cudaGetLastError());
    loss_finalize_kernel<<<1, 256, 0, s>>>(scratch, blocks, result);
    GRPO_CUDA_TRY(cudaGetLastError());
    return GRPO_B200_OK;
}

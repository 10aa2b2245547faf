// Row log-sum-exp, log-probability extraction and inverse-CDF sampling on logits that stay on the
// device.
//
// The reference copies all N*P logits to the host after every forward pass to draw one token per
// response and to read log p(token) under the policy and under the frozen reference model
// (apps/04_gpt2_grpo.cu:61-88 row_logsumexp / sample_row / copy_logits, :138-161 draw_sample).
// Here one CTA per requested row does the same arithmetic next to the logits and only the few
// results cross the bus: per row, the log-sum-exp (double), the drawn or given token, and its
// fp32 log-probability.
//
//   lse    = max + log( sum_v exp( (double)(x_v - max) ) )            (float subtraction, double exp)
//   sample = first v with coin < sum_{u<=v} exp( (double)x_u - lse ), else V-1
//   logp   = (float)( (double)x_token - lse )
//
// The sums are formed tile by tile (256 consecutive columns, ordered scan inside the tile, running
// total across tiles), so they differ from a purely sequential sum in the last bits only; a drawn
// token can differ from the host's only if the coin lies within ~1e-15 of a boundary of the
// cumulative distribution.  The work is a few rows per step: latency-bound, not a bandwidth kernel.
#include "common.cuh"

namespace grpo_b200 {
namespace {

constexpr int kSampleThreads = 256;

// inclusive scan of one double per thread over the block, in thread order; returns the thread's
// inclusive value and leaves the block total in *total_sh (valid after the call's last barrier)
__device__ __forceinline__ double block_inclusive_scan(double v, double* warp_sums, double* total_sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += up;
    }
    if (lane == 31) warp_sums[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double w = lane < kSampleThreads / 32 ? warp_sums[lane] : 0.0;
        const double own = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
        if (lane < kSampleThreads / 32) warp_sums[lane] = w - own;  // exclusive prefix of the warps
        if (lane == kSampleThreads / 32 - 1) *total_sh = w;
    }
    __syncthreads();
    return v + warp_sums[warp];
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(const float* __restrict__ logits,
                                                                     long long n_rows, int V, int P,
                                                                     const int32_t* __restrict__ rows, int n_sel,
                                                                     const double* __restrict__ coins,
                                                                     const int32_t* __restrict__ given,
                                                                     int32_t* __restrict__ tokens_out,
                                                                     float* __restrict__ logp_out,
                                                                     double* __restrict__ lse_out) {
    __shared__ double warp_sums[kSampleThreads / 32];
    __shared__ double total_sh;
    __shared__ float red_f[kSampleThreads / 32];
    __shared__ int found_sh;
    const int i = blockIdx.x;
    if (i >= n_sel) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long row = rows[i];
    if (row < 0 || row >= n_rows) {  // never read outside the logits: the caller sees token -1 and a NaN lse
        if (tid == 0) {
            if (tokens_out) tokens_out[i] = -1;
            if (lse_out) lse_out[i] = __longlong_as_double(0x7ff8000000000000LL);
            if (logp_out) logp_out[i] = 0.0f;
        }
        return;
    }
    const float* x = logits + static_cast<size_t>(row) * static_cast<size_t>(P);

    // ---- maximum
    float m = -CUDART_INF_F;
    for (int v = tid; v < V; v += kSampleThreads) m = fmaxf(m, x[v]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red_f[warp] = m;
    __syncthreads();
    m = red_f[0];
#pragma unroll
    for (int w = 1; w < kSampleThreads / 32; w++) m = fmaxf(m, red_f[w]);

    // ---- normaliser: tiles of 256 columns in order, ordered scan inside a tile
    double running = 0.0;
    for (int base = 0; base < V; base += kSampleThreads) {
        const int v = base + tid;
        const double e = v < V ? exp(static_cast<double>(__fsub_rn(x[v], m))) : 0.0;
        block_inclusive_scan(e, warp_sums, &total_sh);
        running += total_sh;
        __syncthreads();  // total_sh and warp_sums are rewritten by the next tile
    }
    const double lse = static_cast<double>(m) + log(running);

    // ---- the token: given, or drawn by walking the cumulative distribution
    int token;
    if (coins == nullptr) {
        token = given[i];
    } else {
        const double coin = coins[i];
        if (tid == 0) found_sh = V - 1;
        __syncthreads();
        double before = 0.0;
        for (int base = 0; base < V; base += kSampleThreads) {
            const int v = base + tid;
            const double p = v < V ? exp(static_cast<double>(x[v]) - lse) : 0.0;
            const double cumulative = before + block_inclusive_scan(p, warp_sums, &total_sh);
            if (v < V && coin < cumulative) atomicMin(&found_sh, v);  // the first such column wins
            before += total_sh;
            __syncthreads();
            if (found_sh != V - 1 || coin < before) break;  // uniform: every thread reads the same shared value
        }
        __syncthreads();
        token = found_sh;
    }
    if (tid == 0) {
        if (tokens_out) tokens_out[i] = token;
        if (lse_out) lse_out[i] = lse;
        if (logp_out) {
            float lp = 0.0f;
            if (token >= 0 && token < V) lp = static_cast<float>(static_cast<double>(x[token]) - lse);
            logp_out[i] = lp;
        }
    }
}

}  // namespace

cudaError_t launch_sample_rows(const float* logits, long long n_rows, int V, int P, const int32_t* rows, int n_sel,
                               const double* coins, const int32_t* given, int32_t* tokens_out, float* logp_out,
                               double* lse_out, cudaStream_t stream) {
    sample_rows_kernel<<<n_sel, kSampleThreads, 0, stream>>>(logits, n_rows, V, P, rows, n_sel, coins, given,
                                                             tokens_out, logp_out, lse_out);
    return cudaGetLastError();
}

}  // namespace grpo_b200

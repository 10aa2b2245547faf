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
// The normaliser is a sum of per-thread partial sums (columns t, t + 512, ...; fixed tree), so it
// differs from a purely sequential sum in the last bits only.  The draw walks the cumulative
// distribution in index order in two levels: every thread adds up its own contiguous segment of
// the row, one block scan gives each segment its starting value, and the one segment that holds
// the crossing is walked again, one column per thread.  A drawn token can differ from the host's
// only if the coin lies within ~1e-15 of a boundary of the cumulative distribution.  Three sweeps
// over a row (maximum, normaliser, segments), the second and third from L2; two block scans per
// row.  The work is a few rows per step: latency-bound, not a bandwidth kernel.
#include "common.cuh"

namespace grpo_b200 {
namespace {

constexpr int kSampleThreads = 512;
constexpr int kSampleWarps = kSampleThreads / 32;

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
        double w = lane < kSampleWarps ? warp_sums[lane] : 0.0;
        const double own = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
        if (lane < kSampleWarps) warp_sums[lane] = w - own;  // exclusive prefix of the warps
        if (lane == kSampleWarps - 1) *total_sh = w;
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
    __shared__ double warp_sums[kSampleWarps];
    __shared__ double total_sh;
    __shared__ double before_sh;
    __shared__ float red_f[kSampleWarps];
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
    // 128-bit loads over the columns [0, V4*4) when the row starts on a 16-byte boundary
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    const int V4 = aligned ? V >> 2 : 0;
    const float4* x4 = reinterpret_cast<const float4*>(x);

    // ---- maximum
    float m = -CUDART_INF_F;
    for (int c = tid; c < V4; c += kSampleThreads) {
        const float4 q = x4[c];
        m = fmaxf(fmaxf(m, fmaxf(q.x, q.y)), fmaxf(q.z, q.w));
    }
    for (int v = 4 * V4 + tid; v < V; v += kSampleThreads) m = fmaxf(m, x[v]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red_f[warp] = m;
    __syncthreads();
    m = red_f[0];
#pragma unroll
    for (int w = 1; w < kSampleWarps; w++) m = fmaxf(m, red_f[w]);

    // ---- normaliser: per-thread partial sums in double, then one fixed tree
    double part = 0.0;
    for (int c = tid; c < V4; c += kSampleThreads) {
        const float4 q = x4[c];
        part += (exp(static_cast<double>(__fsub_rn(q.x, m))) + exp(static_cast<double>(__fsub_rn(q.y, m)))) +
                (exp(static_cast<double>(__fsub_rn(q.z, m))) + exp(static_cast<double>(__fsub_rn(q.w, m))));
    }
    for (int v = 4 * V4 + tid; v < V; v += kSampleThreads) part += exp(static_cast<double>(__fsub_rn(x[v], m)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    __syncthreads();  // red_f has been read by everyone; warp_sums is free
    if (lane == 0) warp_sums[warp] = part;
    __syncthreads();
    double running = 0.0;
#pragma unroll
    for (int w = 0; w < kSampleWarps; w++) running += warp_sums[w];
    const double lse = static_cast<double>(m) + log(running);
    __syncthreads();  // warp_sums is rewritten by the scans below

    // ---- the token: given, or drawn by walking the cumulative distribution
    int token;
    if (coins == nullptr) {
        token = given[i];
    } else {
        const double coin = coins[i];
        // level 1: thread t owns columns [t*seg, (t+1)*seg), added up in index order
        const int seg = (V + kSampleThreads - 1) / kSampleThreads;
        const int v0 = min(tid * seg, V), v1 = min(v0 + seg, V);
        double mine = 0.0;
        for (int v = v0; v < v1; v++) mine += exp(static_cast<double>(x[v]) - lse);
        const double inclusive = block_inclusive_scan(mine, warp_sums, &total_sh);
        if (tid == 0) {
            found_sh = kSampleThreads;  // the segment that holds the crossing: the first whose end value exceeds the coin
            before_sh = 0.0;
        }
        __syncthreads();
        if (v0 < v1 && coin < inclusive) atomicMin(&found_sh, tid);
        __syncthreads();
        const int owner = found_sh;
        if (tid == owner) before_sh = inclusive - mine;
        __syncthreads();  // also separates this scan's shared scratch from the next one's
        token = V - 1;    // the coin is at or beyond the last cumulative value
        if (owner < kSampleThreads) {
            // level 2: the owner's segment again, one column per thread (seg <= kSampleThreads whenever V <= 2^18;
            // longer segments take several rounds)
            const int s0 = owner * seg, s1 = min(s0 + seg, V);
            double before = before_sh;
            if (tid == 0) found_sh = s1 - 1;  // rounding between the two levels may hide the crossing: then the segment's last column
            __syncthreads();
            for (int base = s0; base < s1; base += kSampleThreads) {
                const int v = base + tid;
                const double pv = v < s1 ? exp(static_cast<double>(x[v]) - lse) : 0.0;
                const double cumulative = before + block_inclusive_scan(pv, warp_sums, &total_sh);
                if (v < s1 && coin < cumulative) atomicMin(&found_sh, v);
                before += total_sh;
                __syncthreads();
                if (coin < before) break;  // uniform: every thread holds the same value
            }
            __syncthreads();
            token = found_sh;
        }
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

// Shared device helpers of the GRPO loss-boundary kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "grpo_b200.h"

namespace grpo_b200 {

// ---- error text (thread-local, read back through grpo_b200_last_error) ---------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t err, const char* what);

#define GRPO_CUDA_TRY(expr)                                             \
    do {                                                                \
        cudaError_t err__ = (expr);                                     \
        if (err__ != cudaSuccess) return ::grpo_b200::cuda_fail(err__, #expr); \
    } while (0)

// ---- per-token loss ------------------------------------------------------------------------
// The four weighted terms of one active token.  Arithmetic mirrors the reference's CPU path
// (src/cpu/grpo_loss.cpp:137-160; its CUDA twin token_loss, src/cuda/grpo_loss_cuda.cu:59-95)
// one fp32 operation at a time: explicit round-to-nearest intrinsics keep the compiler from
// fusing a multiply into an add, because the CPU build has no fused multiply-add.
struct TokenTerms {
    float loss, pg, kl, grad;
};

// Everything after the two transcendental calls: rho = exp(lp_new - lp_old) (read only when the
// advantage is non-zero), em1 = expm1(d), d = lp_ref - lp_new.
__device__ __forceinline__ TokenTerms token_assemble(float rho, float em1, float d, float adv, float w,
                                                     float clip_eps, float beta) {
    const float lo = __fsub_rn(1.0f, clip_eps);
    const float hi = __fadd_rn(1.0f, clip_eps);
    float pg = 0.0f, pg_grad = 0.0f;
    if (adv != 0.0f) {  // a zero advantage never looks at the ratio (overflow-safe)
        const float rho_c = rho < lo ? lo : (hi < rho ? hi : rho);
        const float u = __fmul_rn(rho, adv);
        const float c = __fmul_rn(rho_c, adv);
        pg = -(c < u ? c : u);
        // strictly outside the window on the side the advantage pushes towards: no gradient;
        // exactly on the boundary the unclipped branch is kept
        const bool cut = (adv > 0.0f && rho > hi) || (adv < 0.0f && rho < lo);
        pg_grad = cut ? 0.0f : __fmul_rn(-adv, rho);
    }
    const float kl = __fsub_rn(em1, d);  // k3 estimator: e^d - 1 - d >= 0
    const float loss = __fadd_rn(pg, __fmul_rn(beta, kl));
    const float kl_grad = __fmul_rn(-beta, em1);
    TokenTerms t;
    t.loss = __fmul_rn(w, loss);
    t.pg = __fmul_rn(w, pg);
    t.kl = __fmul_rn(w, kl);
    t.grad = __fmul_rn(w, __fadd_rn(pg_grad, kl_grad));
    return t;
}

// PRECISE = true evaluates exp / expm1 in double and rounds to fp32 (matches a correctly
// rounded libm expf in all but the rarest cases; used where there is one token per row of
// logits).  PRECISE = false uses the fp32 device functions (<= 2 ulp), for the path that runs
// millions of tokens per launch.
template <bool PRECISE>
__device__ __forceinline__ TokenTerms token_terms(float lp_new, float lp_old, float lp_ref,
                                                  float adv, float w, float clip_eps, float beta) {
    float rho = 1.0f;
    if (adv != 0.0f) {
        const float a = __fsub_rn(lp_new, lp_old);
        rho = PRECISE ? static_cast<float>(exp(static_cast<double>(a))) : expf(a);
    }
    const float d = __fsub_rn(lp_ref, lp_new);
    const float em1 = PRECISE ? static_cast<float>(expm1(static_cast<double>(d))) : expm1f(d);
    return token_assemble(rho, em1, d, adv, w, clip_eps, beta);
}

__device__ __forceinline__ bool finite_f(float x) { return fabsf(x) <= 3.402823466e+38f; }

// ---- deterministic reductions ----------------------------------------------------------------
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;  // lane 0 holds the sum; the tree shape is fixed
}

// Sums NV doubles per thread over a block of THREADS threads (fixed tree: lanes, then warps in
// index order).  Thread 0 returns the totals in v[]; `scratch` needs NV * THREADS/32 doubles.
template <int THREADS, int NV>
__device__ __forceinline__ void block_sum(double (&v)[NV], double* scratch) {
    constexpr int WARPS = THREADS / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < NV; k++) {
        v[k] = warp_sum(v[k]);
        if (lane == 0) scratch[k * WARPS + warp] = v[k];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int k = 0; k < NV; k++) {
            double x = lane < WARPS ? scratch[k * WARPS + lane] : 0.0;
            v[k] = warp_sum(x);
        }
    }
}

// Per-response weights and the two counters {valid tokens, empty responses} from global lengths, by
// one block of THREADS threads: the reference's fp32 expressions (src/cuda/grpo_loss_cuda.cu:43-55).
// The power is evaluated in double and rounded, which reproduces a correctly rounded powf.
// `scratch` needs 2 * THREADS/32 + 1 doubles.  Ends with every thread past its last store.
template <int THREADS, class LEN>
__device__ __forceinline__ void block_weights(const LEN* lengths, long long n_seq, int reduction, float alpha,
                                              float* weights, int32_t* meta, double* scratch) {
    double v[2] = {0.0, 0.0};
    for (long long s = threadIdx.x; s < n_seq; s += THREADS) {
        const int L = static_cast<int>(lengths[s]);
        v[0] += static_cast<double>(L);
        v[1] += L == 0 ? 1.0 : 0.0;
    }
    block_sum<THREADS, 2>(v, scratch);
    double* total_sh = scratch + 2 * THREADS / 32;
    if (threadIdx.x == 0) {
        *total_sh = v[0];
        meta[0] = static_cast<int32_t>(v[0]);
        meta[1] = static_cast<int32_t>(v[1]);
    }
    __syncthreads();
    const float n_valid = static_cast<float>(static_cast<int32_t>(*total_sh));
    const float n_seq_f = static_cast<float>(n_seq);
    const float expo = __fsub_rn(alpha, 1.0f);
    for (long long s = threadIdx.x; s < n_seq; s += THREADS) {
        const int L = static_cast<int>(lengths[s]);
        float w = 0.0f;
        if (L > 0) {
            const float Lf = static_cast<float>(L);
            if (reduction == GRPO_B200_SEQUENCE_MEAN) {
                w = __fdiv_rn(1.0f, __fmul_rn(n_seq_f, Lf));
            } else if (reduction == GRPO_B200_TOKEN_MEAN) {
                w = __fdiv_rn(1.0f, n_valid);
            } else {
                const float p = static_cast<float>(pow(static_cast<double>(Lf), static_cast<double>(expo)));
                w = __fdiv_rn(p, n_seq_f);
            }
        }
        weights[s] = w;
    }
}

// base-2 exponential on the special-function unit (max relative error about 2^-22)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr double kLn2 = 0.693147180559945309417232121458;

// streaming (evict-first) 128-bit accesses: every logit is touched exactly once
__device__ __forceinline__ float4 load_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void store_stream(float4* p, float4 v) { __stcs(p, v); }

// ---- kernel launchers (device layer back end) -------------------------------------------------
struct LossArgs {
    const float* logp_new;
    const float* logp_old;
    const float* logp_ref;
    const float* advantages;
    const float* weights;
    const int32_t* mask;
    long long n_tokens;
    long long token_offset;
    int tokens_per_seq;
    float clip_eps, beta;
    float* dlogp;
    grpo_b200_result_t* result;
    double* partials;   // [blocks][5]
    unsigned* counter;  // ticket counter of the blocks (cleared before the launch); unused by the two-launch form
};
int loss_grid_blocks(long long n_tokens);
cudaError_t launch_loss(const LossArgs& a, bool clear_counter, cudaStream_t stream);
int loss_pass(const float* logp_new, const float* logp_old, const float* logp_ref, const float* advantages,
              const float* weights, const int32_t* mask, int64_t n_tokens, int64_t token_offset, int tokens_per_seq,
              float clip_eps, float beta, float* dlogp, grpo_b200_result_t* result, void* workspace,
              size_t workspace_bytes, unsigned* kept_counter, grpo_b200_stream_t stream);

// What the row kernels leave per active row for the reduce kernel: the normaliser (relative to
// e^m, double), the row maximum, the gathered selected logit and the input-error flags.  The
// reduce kernel turns it into the row's loss terms.
struct __align__(32) RowRecord {
    double z;
    float m;
    float x_sel;
    float flags;
    float pad[3];
};

struct LogitsArgs {
    const float* logits;
    float* dlogits;
    const float* logp_old;
    const float* logp_ref;
    const int32_t* selected;
    const float* advantages;
    const float* weights;
    const int32_t* mask;
    long long n_rows;
    long long row_offset;
    int tokens_per_seq;
    int V, P;
    float clip_eps, beta;
    const int32_t* row_order;  // nullable: {n_active, n_masked, active rows ascending, masked rows ascending}
    RowRecord* rows;    // [n_rows] per-row hand-over between the row kernel and the reduce kernel
    float* selected_logp;
    grpo_b200_result_t* result;
    int* status;        // bit 0: a bounded pipeline wait gave up; bit 1: row_order does not match the mask
    unsigned* counter;  // ticket counter of the reduce kernel's blocks (zeroed with the status word)
    double* partials;   // [ceil(n_rows / 256)][5] per-block sums of the reduce kernel
};

// The exchange region of one rank (device memory that every rank of the box maps): a header with
// the region's own pass counter; slots[2][8][stride][2] 8-byte words ([buffer = pass & 1][source
// rank][element][half]), each word = 32 bits of a double in the low half and the pass number in
// the high half; counts[n_seq] int32, this rank's valid-token counts for the next pass (zero
// between passes: the kernel that reads them clears them); lengths[n_seq] doubles, the global
// counts of the last exchange.
constexpr int kExchangeMaxWorld = 8;
constexpr int kExchangePassOffset = 128;
constexpr int kExchangeHeaderBytes = 256;
__host__ __device__ inline long long exchange_stride(long long n_seq) { return (5 + n_seq + 1) & ~1LL; }
__host__ __device__ inline size_t exchange_counts_offset(long long n_seq) {
    return kExchangeHeaderBytes + static_cast<size_t>(2 * kExchangeMaxWorld) * exchange_stride(n_seq) * 16;
}
__host__ __device__ inline size_t exchange_lengths_offset(long long n_seq) {
    return exchange_counts_offset(n_seq) + ((static_cast<size_t>(n_seq) * sizeof(int32_t) + 15) & ~static_cast<size_t>(15));
}

struct ExchangeArgs {
    unsigned char* peers[kExchangeMaxWorld];  // every rank's region as mapped into this process; [rank] is this GPU's own
    int rank;
    int world;  // 0: no exchange, the record goes straight to `result`
    long long n_seq;
    const int32_t* next_mask;  // [n_rows] the next pass's mask over the same rows (may be this pass's)
    int reduction;
    float length_alpha;
    float* weights_out;  // [n_seq] the next pass's weights
    int32_t* meta_out;   // {valid tokens, empty responses} of the next pass's mask
    double* lengths_out; // [n_seq] global valid-token counts of the next pass's mask (nullable)
    long long timeout_cycles;  // SM clock cycles the exchange poll may wait for the peers before it gives up
};
constexpr long long kDefaultExchangeTimeoutCycles = 1LL << 32;  // about two seconds
// status word of a pass and the negative bad_inputs values the reduce kernel derives from it
constexpr int kStatusPipelineTimeout = 1;
constexpr int kStatusRowOrderMismatch = 2;
constexpr double kBadInputsPipelineTimeout = -1.0;
constexpr double kBadInputsExchangeTimeout = -2.0;
constexpr double kBadInputsRowOrder = -3.0;
// flags stored in row_terms.w (small integers, exact in fp32)
constexpr float kRowBadGrad = 1.0f;
constexpr float kRowBadInput = 2.0f;

int pick_resident_variant(const void* logits, const void* dlogits, int V, int P, long long n_rows);
int set_forced_variant(int variant);
const char* resident_variant_name(int variant);
int resident_variant_count();
cudaError_t launch_logits_resident(int variant, bool check, const LogitsArgs& a, cudaStream_t stream);
cudaError_t launch_logits_streaming(bool check, const LogitsArgs& a, cudaStream_t stream);
cudaError_t launch_logits_reduce(const LogitsArgs& a, const ExchangeArgs& x, cudaStream_t stream);

cudaError_t launch_count_lengths(const int32_t* mask, long long n_rows, long long row_offset,
                                 int tokens_per_seq, long long n_seq, int32_t* lengths,
                                 cudaStream_t stream);
cudaError_t launch_weights(const int32_t* lengths, long long n_seq, int reduction, float alpha,
                           float* weights, int32_t* meta, cudaStream_t stream);
cudaError_t launch_count_lengths_f64(const int32_t* mask, long long n_rows, long long row_offset,
                                     int tokens_per_seq, long long n_seq, double* lengths, cudaStream_t stream);
cudaError_t launch_weights_f64(const double* lengths, long long n_seq, int reduction, float alpha,
                               float* weights, int32_t* meta, cudaStream_t stream);
cudaError_t launch_sample_rows(const float* logits, long long n_rows, int V, int P, const int32_t* rows, int n_sel,
                               const double* coins, const int32_t* given, int32_t* tokens_out, float* logp_out,
                               double* lse_out, cudaStream_t stream);
cudaError_t launch_synthetic_logits(float* out, long long n_rows, long long row_offset, int V, int P, float scale,
                                    unsigned long long seed, float tail_fill, cudaStream_t stream);
cudaError_t launch_row_order(const int32_t* mask, long long n_rows, int32_t* order, cudaStream_t stream);
cudaError_t launch_group_advantages(const float* rewards, int B, int G, int mode, float eps,
                                    float* advantages, int32_t* meta, cudaStream_t stream);

}  // namespace grpo_b200

/*
 * grpo_b200.h -- C ABI of the B200-native GRPO loss boundary (libgrpo_b200.so).
 *
 * Two layers, both plain C (pointers and sizes, no C++ or framework types):
 *
 *   1. DEVICE layer  (grpo_b200_loss, grpo_b200_logits, ...): every pointer is a
 *      device pointer on the current device.  These calls allocate nothing, never
 *      synchronise and never exit the process: they validate their scalar
 *      arguments, enqueue hand-written sm_100a kernels on the given stream and
 *      return.  Results land in a small device record (grpo_b200_result_t) so a
 *      caller can keep everything on the device, all-reduce it, or read it back.
 *
 *   2. HOST layer  (grpo_b200_*_host): the reference-facing calls.  They take the
 *      same host arrays the reference's C++ API takes (as pointers + counts),
 *      perform the reference's validation, copy to the device, run layer 1,
 *      synchronise and copy back -- the exact contract of grpo::grpo_loss_cuda,
 *      grpo::grpo_logits_cuda and grpo::grpo_logits_cuda_device_inplace.  The C++
 *      functions in include/grpo/grpo_loss_cuda.cuh are thin wrappers over them.
 *
 * Each declaration cites the interface of the reference (KartikVashishta/grpo.cpp,
 * paths relative to its root) that it replaces.
 *
 * There is no CPU fallback anywhere in this library: without a CUDA device every
 * compute call fails with GRPO_B200_E_CUDA.
 *
 * Data layout shared by all calls (reference include/grpo/grpo_loss.hpp:70-76):
 *   S = B*G responses, each padded to T token slots; N = S*T token rows, row i
 *   belongs to response i / T.  mask[N] is int32 0/1 at arbitrary positions.
 *   advantages[S], weights[S] are fp32.  Logits are N rows of P fp32 columns, of
 *   which the first V are the vocabulary.
 *
 * Thread safety: all calls may be made concurrently from several host threads,
 * each with its own current device (reference apps/03_two_gpu_train.cu:201-215).
 */
#ifndef GRPO_B200_H
#define GRPO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A CUDA stream handle (cudaStream_t); NULL is the legacy default stream. */
typedef struct CUstream_st* grpo_b200_stream_t;

/* Return codes.  On a non-zero return grpo_b200_last_error() holds the text; for
 * GRPO_B200_E_INVALID and GRPO_B200_E_NONFINITE it is, word for word, the message
 * of the std::runtime_error the reference throws for the same condition. */
enum {
    GRPO_B200_OK = 0,
    GRPO_B200_E_INVALID = 1,   /* argument / shape / value rejected (reference: throw) */
    GRPO_B200_E_NONFINITE = 2, /* a result became non-finite (reference: throw) */
    GRPO_B200_E_CUDA = 3,      /* CUDA runtime failure (reference: print + exit(1),
                                  include/grpo/cuda_utils.cuh:8-16) */
    GRPO_B200_E_WORKSPACE = 4  /* workspace pointer null or too small */
};

/* reference include/grpo/grpo_loss.hpp:15-19 */
enum { GRPO_B200_SEQUENCE_MEAN = 0, GRPO_B200_TOKEN_MEAN = 1, GRPO_B200_LENGTH_WEIGHTED = 2 };
/* reference include/grpo/grpo_loss_cuda.cuh:6-14.  Both values of each selector are accepted.
 * The selected-token path has ONE kernel here (a deterministic shuffle/block/partials
 * reduction with no global atomics), so ATOMIC and BLOCK_REDUCE run the same code.
 * For the logits path FUSED picks the row-resident kernel (row held on chip, one read and one
 * write of the logits) whenever the row layout allows it, SEPARATE forces the generic
 * streaming kernel that also serves rows the resident kernel cannot take. */
enum { GRPO_B200_LOSS_ATOMIC = 0, GRPO_B200_LOSS_BLOCK_REDUCE = 1 };
enum { GRPO_B200_LOGITS_SEPARATE = 0, GRPO_B200_LOGITS_FUSED = 1 };
/* reference include/grpo/grpo_loss.hpp:10-13 */
enum { GRPO_B200_ADV_STANDARDIZED = 0, GRPO_B200_ADV_CENTERED = 1 };

/* Device-side result record, written by the last block of each device call's final kernel.
 * Sums are accumulated in double from fp32 per-token products, in a fixed order:
 * repeated runs on the same inputs give bit-identical records. */
typedef struct {
    double loss;      /* sum of weight * (pg + beta * kl) over active tokens   */
    double pg_loss;   /* sum of weight * pg                                    */
    double kl;        /* sum of weight * kl                                    */
    double bad_grads; /* number of active tokens whose gradient is non-finite  */
    double bad_inputs;/* selected-token path: active tokens with a non-finite log-probability or
                         a mask value other than 0/1; logits path: active rows with an
                         out-of-vocabulary selected id or (when checked) a non-finite logit.
                         Logits path, negative values: the pass itself failed and the other fields
                         mean nothing -- -1 a bounded wait of the copy pipeline gave up, -2 a rank
                         did not answer the exchange in time, -3 row_order does not belong to mask */
} grpo_b200_result_t;

const char* grpo_b200_last_error(void);
/* Library version and the architecture the kernels were compiled for ("sm_100a"). */
const char* grpo_b200_build_info(void);

/* ------------------------------------------------------------------------------------
 * DEVICE LAYER
 * ------------------------------------------------------------------------------------ */

/* Per-response valid-token counts from the mask.
 * Replaces the counting half of the reference's host-side make_weights
 * (src/cuda/grpo_loss_cuda.cu:33-41; CPU twin src/cpu/grpo_loss.cpp:97-104).
 * Counts the local rows [row_offset, row_offset + n_rows) of a batch of n_seq responses of
 * tokens_per_seq slots each; lengths[n_seq] is fully written (0 for responses with no local
 * row), so that per-rank partial counts of a token-sharded batch can be summed.  Any non-zero
 * mask value counts as valid here, as in the reference's kernels; values other than 0/1 are
 * reported by the loss calls through result->bad_inputs. */
int grpo_b200_count_lengths(const int32_t* mask, int64_t n_rows, int64_t row_offset,
                            int tokens_per_seq, int64_t n_seq, int32_t* lengths,
                            grpo_b200_stream_t stream);

/* Per-response token weights from (global) lengths.
 * Replaces the weighting half of make_weights (src/cuda/grpo_loss_cuda.cu:43-55):
 *   sequence_mean   1.0f / (float(S) * L_i)
 *   token_mean      1.0f / float(sum L_i)
 *   length_weighted powf(float(L_i), alpha - 1.0f) / float(S)
 * meta[0] = sum of lengths (the reference's valid_tokens), meta[1] = number of responses with
 * L_i == 0 (the reference throws "every sequence needs at least one valid token" for any). */
int grpo_b200_weights_from_lengths(const int32_t* lengths, int64_t n_seq, int reduction,
                                   float length_alpha, float* weights, int32_t* meta,
                                   grpo_b200_stream_t stream);

/* The same two steps with the lengths held as doubles, so that a token-sharded caller can put the
 * partial lengths next to the five-double result record and sum both across ranks with ONE
 * all-reduce per pass (counts are exact in a double).  Replace the same reference code as the
 * int32 forms above (src/cuda/grpo_loss_cuda.cu:33-41 and :43-55). */
int grpo_b200_count_lengths_f64(const int32_t* mask, int64_t n_rows, int64_t row_offset,
                                int tokens_per_seq, int64_t n_seq, double* lengths,
                                grpo_b200_stream_t stream);
int grpo_b200_weights_from_lengths_f64(const double* lengths, int64_t n_seq, int reduction,
                                       float length_alpha, float* weights, int32_t* meta,
                                       grpo_b200_stream_t stream);

/* Group-relative advantages on the device.
 * Replaces grpo::group_advantages_cpu (src/cpu/grpo_loss.cpp:16-58): per prompt, Welford mean
 * and population variance in double, all-equal groups give exact zeros.  rewards[B*G] ->
 * advantages[B*G]; meta[0] counts non-finite rewards or advantages. */
int grpo_b200_group_advantages(const float* rewards, int B, int G, int mode, float eps,
                               float* advantages, int32_t* meta, grpo_b200_stream_t stream);

/* Selected-token path: masked per-token clipped policy-gradient + KL loss, dlogp and the three
 * weighted sums.
 * Replaces grpo_loss_block_kernel / grpo_loss_atomic_kernel and launch_loss
 * (src/cuda/grpo_loss_cuda.cu:97-179, 527-549) including the accumulator reset the reference
 * times with it (:834).  dlogp[n_tokens] is fully written (0 where masked).  The local tokens
 * are [token_offset, token_offset + n_tokens) of the batch: token i belongs to response
 * (token_offset + i) / tokens_per_seq, which indexes advantages[] and weights[].
 * Uses workspace (grpo_b200_loss_workspace_bytes) for per-block partial sums. */
size_t grpo_b200_loss_workspace_bytes(int64_t n_tokens);
int grpo_b200_loss(const float* logp_new, const float* logp_old, const float* logp_ref,
                   const float* advantages, const float* weights, const int32_t* mask,
                   int64_t n_tokens, int64_t token_offset, int tokens_per_seq,
                   float clip_eps, float beta, float* dlogp, grpo_b200_result_t* result,
                   void* workspace, size_t workspace_bytes, grpo_b200_stream_t stream);

/* Selected-token path without any memory from the caller beyond inputs and outputs.
 * This entry point has no counterpart in the reference.  It exists for callers that cannot call
 * cudaMalloc and have no spare device buffer to pass as workspace: a trainer that carves all of
 * its device memory out of one slab at start-up and has accounted for every byte of it, or code
 * running where an allocation would stall the whole device (cudaMalloc synchronises with every
 * stream) or is simply forbidden by the host framework's memory policy.
 * Same arithmetic, kernels, grid and summation order as grpo_b200_loss, so the same bits in dlogp
 * and in the result record at every size it accepts; the per-block partial sums go to an 80 KB
 * array that the library itself holds on every GPU it is loaded on (until the process exits)
 * instead of a caller workspace.  Limits and rules:
 *   - at most 16,777,216 tokens per call; larger calls are refused with GRPO_B200_E_INVALID and a
 *     message naming the limit (use grpo_b200_loss for those);
 *   - the first call on each device looks up the array's device address (no allocation, but a
 *     runtime query): make that first call before starting any stream capture on that device;
 *   - the address found by that first call is kept until the process exits: after a
 *     cudaDeviceReset of that device it is stale and this entry point must not be used again in
 *     the process;
 *   - all calls on one device share the array, so two calls that can overlap on the GPU (different
 *     streams, no dependency between them) race on it and must be serialised by the caller; calls
 *     in the same stream are safe, and nothing needs clearing between calls;
 *   - it never calls cudaMalloc, cudaFree or any allocating library routine. */
int grpo_b200_loss_noalloc(const float* logp_new, const float* logp_old, const float* logp_ref,
                           const float* advantages, const float* weights, const int32_t* mask,
                           int64_t n_tokens, int64_t token_offset, int tokens_per_seq,
                           float clip_eps, float beta, float* dlogp, grpo_b200_result_t* result,
                           grpo_b200_stream_t stream);

/* Logits path: per active row log-softmax (max + normaliser), gather of the selected logit,
 * token loss, and the log-softmax backward dL/dlogits = dlogp * (onehot - softmax); columns
 * [V, P) and every masked row are written as zeros; masked rows and their selected id are
 * never read.
 * Replaces grpo_logits_fused_kernel, selected_logp_kernel + logits_backward_kernel and
 * launch_logits (src/cuda/grpo_loss_cuda.cu:181-349, 551-582).  dlogits may equal logits
 * (in place, the contract of grpo_logits_cuda_device_inplace, :774-817) or be a separate
 * buffer of the same row stride P.  Rows are the local rows [row_offset, row_offset + n_rows).
 * kernel: GRPO_B200_LOGITS_FUSED or _SEPARATE.  check_inputs != 0 additionally records rows
 * with a non-finite logit or an out-of-range selected id in result->bad_inputs.
 * selected_logp (nullable) receives log p(selected) per row (0 for masked rows).
 * row_order (nullable) is the output of grpo_b200_row_order for this mask: with it the row
 * kernel deals every cluster the same number of active and of masked rows, evenly interleaved,
 * instead of every n-th row whatever its mask; results do not depend on it.  A row order made
 * from another mask is detected (counts that do not add up, row indices outside the batch, a
 * listed row whose mask value disagrees) and reported as bad_inputs = -3; no access leaves the
 * batch because of it. */
size_t grpo_b200_logits_workspace_bytes(int64_t n_rows);
int grpo_b200_logits(const float* logits, float* dlogits, const float* logp_old,
                     const float* logp_ref, const int32_t* selected, const float* advantages,
                     const float* weights, const int32_t* mask, int64_t n_rows, int64_t row_offset,
                     int tokens_per_seq, int V, int P, float clip_eps, float beta, int kernel,
                     int check_inputs, float* selected_logp, const int32_t* row_order,
                     grpo_b200_result_t* result, void* workspace, size_t workspace_bytes,
                     grpo_b200_stream_t stream);

/* Stable partition of the local row indices by mask, for the row_order argument above:
 * order = {n_active, n_masked, active rows ascending, masked rows ascending}, n_rows + 2
 * entries, in a buffer of grpo_b200_row_order_bytes(n_rows) (the tail is scratch).
 * No counterpart in the reference (its kernels take one row per block, in index order,
 * src/cuda/grpo_loss_cuda.cu:551-582).  Depends on the mask only: computed once per batch. */
size_t grpo_b200_row_order_bytes(int64_t n_rows);
int grpo_b200_row_order(const int32_t* mask, int64_t n_rows, int32_t* order,
                        grpo_b200_stream_t stream);

/* Token-sharded logits path with the pass's exchange done by the library's own kernel over
 * NVLink peer memory.  No counterpart in the reference, whose two-GPU demo shards whole
 * responses and averages on the host (apps/03_two_gpu_train.cu:200-215, 247-281).
 *
 * Every rank (one process per GPU of one box, at most 8) owns an exchange region, created here
 * with cudaMalloc and cleared; it exports a 64-byte inter-process handle, the ranks trade
 * handles by any means they have, and each opens the others' regions.  regions[world] is a
 * HOST array of the regions as mapped into this process, regions[rank] being the own one.
 *
 * grpo_b200_logits_sharded is grpo_b200_logits on this rank's rows followed, inside the same
 * last kernel, by everything the ranks must agree on: it counts next_mask's valid tokens per
 * response among this rank's rows (next_mask may be mask itself), sums {the result record, the
 * counts} over the ranks, and derives the next pass's weights from the global counts.  On
 * return (in stream order) result holds the global record, next_weights[n_seq] and
 * next_meta[2] what grpo_b200_weights_from_lengths would give for the whole batch's next_mask
 * (next_weights may be the buffer `weights` points to), and next_lengths[n_seq] (nullable) the
 * global counts as doubles.  The sums are taken in rank order, so every rank gets the same
 * bits.  The region counts its own passes on the device; the ranks must make the same sequence
 * of calls on their regions, with the n_seq their regions were created for (checked against the
 * own region).  A rank whose peers do not answer within the exchange timeout (about two seconds
 * of SM clock unless grpo_b200_exchange_set_timeout_cycles changed it) stops waiting and reports
 * bad_inputs = -2; nothing blocks forever.  The timeout treats a late peer like a lost one, and a
 * rank that gave up runs ahead of the others: line the ranks up on the host (a barrier of whatever
 * process group they share) before the first call on a batch and after any host-side stall such
 * as a checkpoint, and treat -2 as fatal for the regions involved.  world = 1 runs the same code
 * against the own region alone. */
size_t grpo_b200_exchange_bytes(int64_t n_seq);
int grpo_b200_exchange_create(int64_t n_seq, void** region);
/* Process-wide limit of the exchange's wait for the other ranks, in SM clock cycles (default 2^32,
 * about two seconds; no counterpart in the reference).  Read when a sharded call is enqueued. */
int grpo_b200_exchange_set_timeout_cycles(int64_t cycles);
int grpo_b200_exchange_export(void* region, unsigned char handle[64]);
int grpo_b200_exchange_open(const unsigned char handle[64], void** peer_region);
int grpo_b200_exchange_close(void* peer_region);
int grpo_b200_exchange_destroy(void* region);
int grpo_b200_logits_sharded(const float* logits, float* dlogits, const float* logp_old,
                             const float* logp_ref, const int32_t* selected,
                             const float* advantages, const float* weights, const int32_t* mask,
                             int64_t n_rows, int64_t row_offset, int tokens_per_seq, int V, int P,
                             float clip_eps, float beta, int kernel, int check_inputs,
                             float* selected_logp, const int32_t* row_order,
                             grpo_b200_result_t* result, void* workspace, size_t workspace_bytes,
                             void* const* regions, int rank, int world,
                             int64_t n_seq, const int32_t* next_mask, int reduction,
                             float length_alpha, float* next_weights, int32_t* next_meta,
                             double* next_lengths, grpo_b200_stream_t stream);

/* The first pass's weights without a collective call: counts mask's valid tokens per response
 * among this rank's rows, sums the counts over the ranks through their exchange regions (the
 * exchange of grpo_b200_logits_sharded, with an all-zero record) and derives the weights.
 * Replaces make_weights (src/cuda/grpo_loss_cuda.cu:21-57) for a batch whose rows are spread
 * over ranks.  weights[n_seq], meta[2] and lengths[n_seq] (nullable) as in
 * grpo_b200_logits_sharded; workspace as for grpo_b200_logits on n_rows rows.  status (a device
 * record, required) receives the exchanged record: all zeros, or bad_inputs = -2 when a rank did
 * not answer in time -- the weights then come from partial counts and must not be used.  Counts as
 * one pass of the region: every rank makes the call. */
int grpo_b200_lengths_sharded(const int32_t* mask, int64_t n_rows, int64_t row_offset,
                              int tokens_per_seq, int64_t n_seq, void* const* regions, int rank,
                              int world, int reduction, float length_alpha, float* weights,
                              int32_t* meta, double* lengths, grpo_b200_result_t* status,
                              void* workspace, size_t workspace_bytes, grpo_b200_stream_t stream);

/* Sampling and log-probability extraction on logits that stay on the device.  Replaces, for
 * the rows named in rows[n_selected] (indices into the [n_rows][P] logits), the host-side
 * row_logsumexp / sample_row / draw_sample of apps/04_gpt2_grpo.cu:61-80,138-161, which need
 * the whole logits array copied to the host (copy_logits, :82-90):
 *   lse   = max + log(sum_v exp((double)(x_v - max)))
 *   token = coins ? first v with coins[i] < sum_{u<=v} exp((double)x_u - lse), else V-1
 *                 : given_tokens[i]
 *   logp  = (float)((double)x_token - lse)        (0 when a given token is outside [0, V))
 * Exactly one of coins (uniform numbers in [0,1), drawn by the caller's generator) and
 * given_tokens is non-null: draw under the policy's logits with coins, then read the same tokens'
 * log-probabilities under the reference model's logits with given_tokens.  tokens_out, logp_out
 * and lse_out are device arrays of n_selected entries (logp_out, lse_out, and tokens_out when
 * tokens are given, may be null).  A row index outside [0, n_rows) yields token -1, a NaN lse. */
int grpo_b200_sample_rows(const float* logits, int64_t n_rows, int V, int P, const int32_t* rows,
                          int n_selected, const double* coins, const int32_t* given_tokens,
                          int32_t* tokens_out, float* logp_out, double* lse_out,
                          grpo_b200_stream_t stream);

/* Counter-based synthetic logits for benchmarks and tests: element (row_offset + r, v) of a batch
 * with row stride P is a pure function of (seed, global row, column) -- the sum of eight 16-bit
 * fields of two splitmix64 outputs, centred, times `scale` (one fp32 multiply) -- so any split of
 * the batch over ranks builds the same rows and a host can rebuild any row bit for bit.  Columns
 * [V, P) receive tail_fill.  Stands where the reference builds its arithmetic fixtures on the
 * host and copies them over (bench/bench_grpo_loss_cuda.cu:60-102). */
int grpo_b200_synthetic_logits(float* logits, int64_t n_rows, int64_t row_offset, int V, int P,
                               float scale, uint64_t seed, float tail_fill,
                               grpo_b200_stream_t stream);

/* Test and tuning hook (no counterpart in the reference): force the row-resident kernel variant (index into the table printed by
 * grpo_b200_logits_variant_name), or -1 for the built-in choice.  Process-wide; not for use while
 * other threads are inside the library. */
int grpo_b200_logits_set_variant(int variant);
/* Name ("cluster x threads x vec") of variant i, NULL past the end of the table. */
const char* grpo_b200_logits_variant_name(int variant);
/* Name of the kernel the dispatcher would run for this row layout, row count and selector. */
const char* grpo_b200_logits_plan(const void* logits, const void* dlogits, int V, int P,
                                  int64_t n_rows, int kernel);

/* ------------------------------------------------------------------------------------
 * HOST LAYER (reference-facing; host arrays in, host results out, synchronous)
 * ------------------------------------------------------------------------------------ */

/* Replaces grpo::grpo_loss_cuda (include/grpo/grpo_loss_cuda.cuh:26-37,
 * src/cuda/grpo_loss_cuda.cu:620-660).  n_* are the element counts of the caller's arrays
 * (the reference's std::vector sizes, checked the same way).  stats_out = {loss, pg_loss, kl}. */
int grpo_b200_loss_host(const float* logp_new, size_t n_logp_new, const float* logp_old,
                        size_t n_logp_old, const float* logp_ref, size_t n_logp_ref,
                        const float* advantages, size_t n_advantages, const int32_t* mask,
                        size_t n_mask, int B, int G, int T, float clip_eps, float beta,
                        int reduction, float length_alpha, int kernel, float* dlogp_out,
                        float* stats_out, int* valid_tokens_out);

/* Replaces grpo::grpo_logits_cuda (include/grpo/grpo_loss_cuda.cuh:53-66,
 * src/cuda/grpo_loss_cuda.cu:726-772): dense host logits [N][V] in, host dlogits [N][V] out. */
int grpo_b200_logits_host(const float* logits, size_t n_logits, const float* logp_old,
                          size_t n_logp_old, const float* logp_ref, size_t n_logp_ref,
                          const int32_t* selected, size_t n_selected, const float* advantages,
                          size_t n_advantages, const int32_t* mask, size_t n_mask, int B, int G,
                          int T, int V, float clip_eps, float beta, int reduction,
                          float length_alpha, int kernel, float* dlogits_out, float* stats_out,
                          int* valid_tokens_out);

/* Replaces grpo::grpo_logits_cuda_device_inplace (include/grpo/grpo_loss_cuda.cuh:68-86,
 * src/cuda/grpo_loss_cuda.cu:774-817): logits_and_dlogits is a caller-owned DEVICE pointer to
 * N rows of P floats on the current device, replaced in place by dL/dlogits; the per-token
 * metadata are host arrays.  Returns after the device work is complete. */
int grpo_b200_logits_device_inplace_host(float* logits_and_dlogits, const float* logp_old,
                                         size_t n_logp_old, const float* logp_ref,
                                         size_t n_logp_ref, const int32_t* selected,
                                         size_t n_selected, const float* advantages,
                                         size_t n_advantages, const int32_t* mask, size_t n_mask,
                                         int B, int G, int T, int V, int P, float clip_eps,
                                         float beta, int reduction, float length_alpha, int kernel,
                                         float* stats_out, int* valid_tokens_out);

/* Replaces grpo::benchmark_grpo_loss_cuda (include/grpo/grpo_loss_cuda.cuh:39-51,
 * src/cuda/grpo_loss_cuda.cu:819-886): resident arrays, `warmup` passes, then the median of 7
 * repeats of `iterations` back-to-back passes per selector, in ms per pass. */
int grpo_b200_benchmark_loss_host(const float* logp_new, size_t n_logp_new, const float* logp_old,
                                  size_t n_logp_old, const float* logp_ref, size_t n_logp_ref,
                                  const float* advantages, size_t n_advantages,
                                  const int32_t* mask, size_t n_mask, int B, int G, int T,
                                  float clip_eps, float beta, int reduction, float length_alpha,
                                  int warmup, int iterations, float* atomic_ms, float* block_ms);

/* Replaces grpo::benchmark_grpo_logits_cuda (include/grpo/grpo_loss_cuda.cuh:88-102,
 * src/cuda/grpo_loss_cuda.cu:888-975): separate input and output logits buffers with P = V,
 * 15 samples in alternating order, medians in ms per pass. */
int grpo_b200_benchmark_logits_host(const float* logits, size_t n_logits, const float* logp_old,
                                    size_t n_logp_old, const float* logp_ref, size_t n_logp_ref,
                                    const int32_t* selected, size_t n_selected,
                                    const float* advantages, size_t n_advantages,
                                    const int32_t* mask, size_t n_mask, int B, int G, int T, int V,
                                    float clip_eps, float beta, int reduction, float length_alpha,
                                    int warmup, int iterations, float* separate_ms, float* fused_ms);

/* Token-sharded run, host side: grpo_logits_cuda_device_inplace (include/grpo/grpo_loss_cuda.cuh:68-86,
 * src/cuda/grpo_loss_cuda.cu:774-817) for ONE RANK'S ROWS of a batch whose rows are spread over up to
 * eight GPUs of one box, for the reference's two kinds of multi-GPU caller: one host thread per device
 * in one process (apps/03_two_gpu_train.cu:200-215) and one process per device
 * (apps/05_two_gpu_gpt2_grpo.cu:309-328).
 *
 * A shard owns what one rank needs between calls: its exchange region, device copies of the per-token
 * metadata, pinned staging, workspace.  grpo_b200_shard_create is called with the rank's device current
 * (rows [row_offset, row_offset + n_rows) of a batch of n_seq responses of tokens_per_seq slots).  Then
 * the ranks connect, either way:
 *   processes: every rank exports 64 bytes (grpo_b200_shard_export), the ranks trade them by whatever
 *              channel they have, and each calls grpo_b200_shard_connect_ipc with all world handles
 *              concatenated in rank order (its own entry is ignored);
 *   threads:   every rank calls grpo_b200_shard_connect_local with the array of all world shards in rank
 *              order (peer access between the devices is enabled as needed), after all were created.
 * The ranks line up on the host (a barrier) after connecting and before every call on a new batch.
 *
 * grpo_b200_logits_sharded_host: this rank's host metadata in (logp_old, logp_ref, selected, mask:
 * n_rows entries each; advantages: all n_seq), this rank's device logits (n_rows x P) replaced in place
 * by dL/dlogits, and the GLOBAL loss, pg_loss, kl and valid-token count out -- the same on every rank,
 * bit for bit.  One packed pinned upload, the row order, the lengths exchange, the row kernel and the
 * reduce kernel (with the record exchange over NVLink peer memory) enqueued on the legacy default stream
 * without an intermediate synchronisation, one pinned read-back; returns after the device work is
 * complete.  Errors as the reference's call, applied to the global quantities ("every sequence needs at
 * least one valid token" looks at the whole batch); a rank whose peers do not answer within the exchange
 * timeout gets GRPO_B200_E_CUDA "the exchange between ranks timed out".  Every rank makes the same
 * sequence of calls; a rank that returns early on an argument error leaves its peers to that timeout. */
typedef struct grpo_b200_shard* grpo_b200_shard_t;
int grpo_b200_shard_create(int rank, int world, int64_t n_seq, int tokens_per_seq, int V, int P,
                           int64_t row_offset, int64_t n_rows, grpo_b200_shard_t* shard);
int grpo_b200_shard_export(grpo_b200_shard_t shard, unsigned char handle[64]);
int grpo_b200_shard_connect_ipc(grpo_b200_shard_t shard, const unsigned char* handles);
int grpo_b200_shard_connect_local(grpo_b200_shard_t shard, grpo_b200_shard_t const* all_shards);
int grpo_b200_shard_destroy(grpo_b200_shard_t shard);
int grpo_b200_logits_sharded_host(grpo_b200_shard_t shard, float* logits_and_dlogits,
                                  const float* logp_old, size_t n_logp_old, const float* logp_ref,
                                  size_t n_logp_ref, const int32_t* selected, size_t n_selected,
                                  const float* advantages, size_t n_advantages, const int32_t* mask,
                                  size_t n_mask, float clip_eps, float beta, int reduction,
                                  float length_alpha, int kernel, float* stats_out,
                                  int* valid_tokens_out);

/* Gradient all-reduce fused with the 1/world scale, in place, by ONE kernel per rank over NVLink peer
 * memory.  Replaces ncclAllReduce(grads) followed by scale_kernel(grads, 1/world) of the reference's
 * two-GPU GPT-2 demo (apps/05_two_gpu_gpt2_grpo.cu:216-219, 260-268), which moves the data through a
 * collective and then reads and writes all of it again.  Rank r loads slice r of every rank's buffer
 * (peer loads), adds the terms in rank order, multiplies by `scale`, and stores the result into slice r
 * of every rank's buffer (peer stores): every replica ends with the same bits, as the demo's replica
 * hash check requires (:330-342).
 *
 * A handle registers this rank's buffer (device memory, 16-byte aligned, n floats; it may lie inside a
 * larger allocation) with the rank's device current.  Ranks connect like shards do: processes trade the
 * 192-byte blocks of grpo_b200_gradsync_export and call _connect_ipc with all of them concatenated in
 * rank order; threads of one process call _connect_local with all handles in rank order.  After that,
 * every rank calls grpo_b200_allreduce_scale the same number of times; the call only enqueues the
 * kernel.  The ranks' kernels wait for one another through flag words (bounded: about four seconds of SM
 * clock unless grpo_b200_gradsync_set_timeout_cycles changed it); grpo_b200_gradsync_status reads back
 * whether a wait on this rank ever gave up (it synchronises the device).
 * grpo_b200_gradsync_slice is the slice arithmetic itself (pure host code): floats
 * [first, first + count) are what rank `rank` reduces; whole float4s, the last rank taking the tail. */
typedef struct grpo_b200_gradsync* grpo_b200_gradsync_t;
void grpo_b200_gradsync_slice(int64_t n, int world, int rank, int64_t* first, int64_t* count);
int grpo_b200_gradsync_create(int rank, int world, float* grads, int64_t n, grpo_b200_gradsync_t* handle);
int grpo_b200_gradsync_export(grpo_b200_gradsync_t handle, unsigned char block[192]);
int grpo_b200_gradsync_connect_ipc(grpo_b200_gradsync_t handle, const unsigned char* blocks);
int grpo_b200_gradsync_connect_local(grpo_b200_gradsync_t handle, grpo_b200_gradsync_t const* all_handles);
int grpo_b200_gradsync_set_timeout_cycles(int64_t cycles);
int grpo_b200_allreduce_scale(grpo_b200_gradsync_t handle, float scale, grpo_b200_stream_t stream);
int grpo_b200_gradsync_status(grpo_b200_gradsync_t handle, int* timed_out);
int grpo_b200_gradsync_destroy(grpo_b200_gradsync_t handle);

/* LM-head projection fused with the loss statistics (forward): logits = hidden[n_rows][C] x
 * lm_head[P][C]^T are formed tile by tile on the tensor cores (tcgen05.mma, TF32 inputs, fp32
 * accumulation in tensor memory) and reduced at once to the row maximum, the normaliser and the selected
 * logit; the [n_rows][P] logits are never written.  Then the logits path's reduce kernel turns the row
 * records into the three weighted sums.  Stands where the reference runs gpt2_forward's last matmul into
 * model.acts.output and hands the N x P logits to the loss (apps/04_gpt2_grpo.cu:322-331); it gives the
 * loss terms and log p(selected), not the gradient (that half would recompute the tiles).
 * hidden and lm_head: device, fp32, row-major, 16-byte aligned, C a multiple of 32; rows [V, P) of
 * lm_head are never used.  The tensor cores read fp32 words as TF32 (the low 13 mantissa bits are
 * ignored), the precision of the TF32 matmul llm.c uses for this projection.  selected_logp[n_rows]
 * (nullable) receives log p(selected) (0 for masked rows), lse_out[n_rows] (nullable) the row
 * log-sum-exp.  Everything else as grpo_b200_logits; the workspace is larger
 * (grpo_b200_lmhead_workspace_bytes).  Single-GPU code: one CTA per SM, no cluster, no multicast. */
size_t grpo_b200_lmhead_workspace_bytes(int64_t n_rows, int P);
int grpo_b200_lmhead_loss(const float* hidden, const float* lm_head, int64_t n_rows, int C, int V, int P,
                          const float* logp_old, const float* logp_ref, const int32_t* selected,
                          const float* advantages, const float* weights, const int32_t* mask,
                          int64_t row_offset, int tokens_per_seq, float clip_eps, float beta,
                          float* selected_logp, double* lse_out, grpo_b200_result_t* result,
                          void* workspace, size_t workspace_bytes, grpo_b200_stream_t stream);

/* Frees the calling thread's current device's cached workspace and staging buffers. */
int grpo_b200_release_cache(void);

#ifdef __cplusplus
}
#endif
#endif /* GRPO_B200_H */

/*
 * CPU oracle for the GRPO loss boundary -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's single-threaded CPU path
 * (src/cpu/grpo_loss.cpp in KartikVashishta/grpo.cpp).  It exists so that the
 * CUDA path can be checked against it; nothing that ships may call it.  Only
 * tests, the smoke check and the benchmark's CPU-baseline leg link or load it.
 *
 * Parity status: PINNED.  The restatement is checked (a) against every
 * known-answer case the reference's own unit tests hold for this path
 * (tests/test_grpo_loss.cpp), (b) bit-for-bit against the reference's own
 * object code compiled into oracle/_ref/ when the reference tree is present,
 * and (c) against committed golden vectors generated from (b).
 *
 * Every function returns 0 on success or one of the GRPO_ORACLE_E_* codes;
 * grpo_oracle_strerror() gives the reference's exception text for that code.
 */
#ifndef GRPO_ORACLE_H
#define GRPO_ORACLE_H

#ifdef __cplusplus
extern "C" {
#endif

enum {
    GRPO_ORACLE_OK = 0,
    GRPO_ORACLE_E_DIMS = 1,          /* "B, G and T must be positive" */
    GRPO_ORACLE_E_SEQ_OVERFLOW = 2,  /* "sequence count exceeds INT_MAX" */
    GRPO_ORACLE_E_TOK_OVERFLOW = 3,  /* "token count exceeds INT_MAX" */
    GRPO_ORACLE_E_CLIP = 4,          /* "clip_eps must be finite and in [0, 1)" */
    GRPO_ORACLE_E_BETA = 5,          /* "beta must be finite and non-negative" */
    GRPO_ORACLE_E_ALPHA = 6,         /* "length_alpha must be finite and in [0, 1]" */
    GRPO_ORACLE_E_LOGP = 7,          /* "log probabilities must be finite" */
    GRPO_ORACLE_E_MASK = 8,          /* "mask values must be 0 or 1" */
    GRPO_ORACLE_E_ADV = 9,           /* "advantages must be finite" */
    GRPO_ORACLE_E_EMPTY_SEQ = 10,    /* "every sequence needs at least one valid token" */
    GRPO_ORACLE_E_LOSS_NONFINITE = 11, /* "loss became non-finite" */
    GRPO_ORACLE_E_GRAD_NONFINITE = 12, /* "gradient became non-finite" */
    GRPO_ORACLE_E_VOCAB = 13,        /* "V must be positive" */
    GRPO_ORACLE_E_LOGITS_OVERFLOW = 14, /* "logits count is too large" */
    GRPO_ORACLE_E_SELECTED = 15,     /* "selected token is outside the vocabulary" */
    GRPO_ORACLE_E_LOGITS = 16,       /* "logits must be finite" */
    GRPO_ORACLE_E_EPS = 17,          /* "eps must be finite and non-negative" */
    GRPO_ORACLE_E_REWARDS = 18,      /* "rewards must be finite" */
    GRPO_ORACLE_E_ADV_NONFINITE = 19 /* "advantages became non-finite" */
};

/* reduction: 0 sequence_mean, 1 token_mean, 2 length_weighted
 * (include/grpo/grpo_loss.hpp:15-19 of the reference). */
enum { GRPO_ORACLE_SEQUENCE_MEAN = 0, GRPO_ORACLE_TOKEN_MEAN = 1, GRPO_ORACLE_LENGTH_WEIGHTED = 2 };
/* advantage mode: 0 standardized, 1 centered (include/grpo/grpo_loss.hpp:10-13). */
enum { GRPO_ORACLE_STANDARDIZED = 0, GRPO_ORACLE_CENTERED = 1 };

const char* grpo_oracle_strerror(int code);

/* src/cpu/grpo_loss.cpp:16-58.  rewards[B*G] -> advantages[B*G]. */
int grpo_oracle_group_advantages(const float* rewards, int B, int G, int mode, float eps,
                                 float* advantages_out);

/* src/cpu/grpo_loss.cpp:60-174.  All token arrays are [B*G*T], advantages [B*G].
 * stats_out = {loss, pg_loss, kl}; dlogp_out[B*G*T] is fully written. */
int grpo_oracle_loss(const float* logp_new, const float* logp_old, const float* logp_ref,
                     const float* advantages, const int* mask, int B, int G, int T,
                     float clip_eps, float beta, int reduction, float length_alpha,
                     float* dlogp_out, float* stats_out, int* valid_tokens_out);

/* src/cpu/grpo_loss.cpp:176-239.  logits [B*G*T][V] dense rows; dlogits_out same
 * shape, fully written (rows whose dlogp is 0 stay all-zero).  selected_logp_out
 * (nullable) receives the fp32 log-probability of the selected token per row
 * (0 for masked rows), the intermediate the reference feeds to the token loss. */
int grpo_oracle_logits(const float* logits, const float* logp_old, const float* logp_ref,
                       const int* selected, const float* advantages, const int* mask,
                       int B, int G, int T, int V,
                       float clip_eps, float beta, int reduction, float length_alpha,
                       float* dlogits_out, float* stats_out, int* valid_tokens_out,
                       float* selected_logp_out);

/* The same per-row steps as grpo_oracle_logits (forward :200-216, token loss :137-160, backward
 * :223-237) for n rows taken out of a larger batch, with each row's advantage and weight given
 * by the caller.  rows [n][V]; dlogits_out [n][V]; sel_logp_out [n] (nullable); terms_out [n][3]
 * = the fp32 products {w*loss, w*pg, w*kl} the reference adds to its double totals.  Checked in
 * tests against grpo_oracle_logits on whole small batches (same bits). */
int grpo_oracle_logits_rows(const float* rows, int n, int V, const float* logp_old,
                            const float* logp_ref, const int* selected, const float* adv,
                            const float* w, float clip_eps, float beta, float* dlogits_out,
                            float* sel_logp_out, float* terms_out);

/* Sampling helpers of the reference's GPT-2 demo, restated: apps/04_gpt2_grpo.cu:61-66
 * (row_logsumexp) and :68-78 (sample_row, with the uniform number passed in instead of drawn
 * from std::mt19937 inside).  Parity of these two: PINNED -- oracle/Makefile cuts the two helpers
 * out of the reference file at build time and compiles them behind ref_sample_shim.cpp; the
 * committed vectors (tests/golden/sampling_cases.npz: log-sum-exp bits, the generator's coins,
 * drawn tokens) come from that object code, and the restatement reproduces them exactly. */
double grpo_oracle_row_logsumexp(const float* row, int V);
int grpo_oracle_sample_row(const float* row, int V, double coin);

#ifdef __cplusplus
}
#endif
#endif

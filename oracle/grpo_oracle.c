/*
 * CPU oracle for the GRPO loss boundary -- TEST INFRASTRUCTURE ONLY.
 * See grpo_oracle.h for what may use it and how its parity is pinned.
 *
 * The arithmetic follows the reference's CPU path operation for operation:
 * fp32 per-token math through libm's expf/expm1f/powf, fp32 products of
 * weight and per-token terms, double accumulation of those products, double
 * log-sum-exp for the logits rows.  Build with -ffp-contract=off so that no
 * multiply-add is fused (the reference builds for baseline x86-64, which has
 * no FMA instruction).
 */
#include "grpo_oracle.h"

#include <limits.h>
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

const char* grpo_oracle_strerror(int code) {
    switch (code) {
        case GRPO_ORACLE_OK: return "ok";
        case GRPO_ORACLE_E_DIMS: return "B, G and T must be positive";
        case GRPO_ORACLE_E_SEQ_OVERFLOW: return "sequence count exceeds INT_MAX";
        case GRPO_ORACLE_E_TOK_OVERFLOW: return "token count exceeds INT_MAX";
        case GRPO_ORACLE_E_CLIP: return "clip_eps must be finite and in [0, 1)";
        case GRPO_ORACLE_E_BETA: return "beta must be finite and non-negative";
        case GRPO_ORACLE_E_ALPHA: return "length_alpha must be finite and in [0, 1]";
        case GRPO_ORACLE_E_LOGP: return "log probabilities must be finite";
        case GRPO_ORACLE_E_MASK: return "mask values must be 0 or 1";
        case GRPO_ORACLE_E_ADV: return "advantages must be finite";
        case GRPO_ORACLE_E_EMPTY_SEQ: return "every sequence needs at least one valid token";
        case GRPO_ORACLE_E_LOSS_NONFINITE: return "loss became non-finite";
        case GRPO_ORACLE_E_GRAD_NONFINITE: return "gradient became non-finite";
        case GRPO_ORACLE_E_VOCAB: return "V must be positive";
        case GRPO_ORACLE_E_LOGITS_OVERFLOW: return "logits count is too large";
        case GRPO_ORACLE_E_SELECTED: return "selected token is outside the vocabulary";
        case GRPO_ORACLE_E_LOGITS: return "logits must be finite";
        case GRPO_ORACLE_E_EPS: return "eps must be finite and non-negative";
        case GRPO_ORACLE_E_REWARDS: return "rewards must be finite";
        case GRPO_ORACLE_E_ADV_NONFINITE: return "advantages became non-finite";
        default: return "unknown oracle error";
    }
}

/* include/grpo/grpo_loss.hpp:51-67: positive dims, S = B*G <= INT_MAX,
 * N = S*T <= INT_MAX.  (The size_t overflow branches of the reference cannot
 * trigger for int inputs on a 64-bit host.) */
static int shape_of(int B, int G, int T, size_t* n_seq, size_t* n_tok) {
    if (B <= 0 || G <= 0 || T <= 0) return GRPO_ORACLE_E_DIMS;
    size_t s = (size_t)B * (size_t)G;
    if (s > (size_t)INT_MAX) return GRPO_ORACLE_E_SEQ_OVERFLOW;
    size_t n = s * (size_t)T;
    if (n > (size_t)INT_MAX) return GRPO_ORACLE_E_TOK_OVERFLOW;
    *n_seq = s;
    *n_tok = n;
    return GRPO_ORACLE_OK;
}

/* src/cpu/grpo_loss.cpp:16-58 */
int grpo_oracle_group_advantages(const float* rewards, int B, int G, int mode, float eps,
                                 float* adv) {
    size_t n_seq, n_tok;
    int rc = shape_of(B, G, 1, &n_seq, &n_tok);
    if (rc) return rc;
    if (eps < 0.0f || !isfinite(eps)) return GRPO_ORACLE_E_EPS;
    for (size_t i = 0; i < n_seq; i++)
        if (!isfinite(rewards[i])) return GRPO_ORACLE_E_REWARDS;
    for (size_t i = 0; i < n_seq; i++) adv[i] = 0.0f;

    for (int b = 0; b < B; b++) {
        const float* r = rewards + (size_t)b * G;
        float* a = adv + (size_t)b * G;
        int same = 1;
        for (int g = 1; g < G; g++) same = same && (r[g] == r[0]);
        if (same) continue; /* a constant group carries no signal: exact zeros (:32-37) */

        /* Welford running mean / sum of squared deviations in double (:39-46) */
        double mean = 0.0, m2 = 0.0;
        for (int g = 0; g < G; g++) {
            double x = r[g];
            double delta = x - mean;
            mean += delta / (double)(g + 1);
            m2 += delta * (x - mean);
        }
        double var = m2 / (double)G; /* population variance (:47) */
        double denom = mode == GRPO_ORACLE_STANDARDIZED ? sqrt(var + eps) : 1.0;
        for (int g = 0; g < G; g++) a[g] = (float)(((double)r[g] - mean) / denom);
    }
    for (size_t i = 0; i < n_seq; i++)
        if (!isfinite(adv[i])) return GRPO_ORACLE_E_ADV_NONFINITE;
    return GRPO_ORACLE_OK;
}

/* One active token (src/cpu/grpo_loss.cpp:137-160): terms = {w*loss, w*pg, w*kl} as fp32 products,
 * returns w * dL/dlogp. */
static float one_token(float lp_new, float lp_old, float lp_ref, float A, float w, float lo, float hi,
                       float beta, float terms[3]) {
    float pg = 0.0f, pg_grad = 0.0f;
    if (A != 0.0f) { /* zero advantage never evaluates the ratio (:139) */
        float rho = expf(lp_new - lp_old);
        float rho_c = rho < lo ? lo : (hi < rho ? hi : rho);
        float u = rho * A, c = rho_c * A;
        pg = -(c < u ? c : u);
        /* strictly outside the clip window on the side the advantage pushes to:
         * no gradient; the boundary itself keeps the ratio branch (:144-147) */
        int cut_hi = A > 0.0f && rho > hi;
        int cut_lo = A < 0.0f && rho < lo;
        pg_grad = (cut_hi || cut_lo) ? 0.0f : -A * rho;
    }

    /* k3 estimator of KL(new || ref) on the sampled token (:150-155) */
    float d = lp_ref - lp_new;
    float em1 = expm1f(d);
    float kl = em1 - d;
    float loss = pg + beta * kl;
    float kl_grad = -beta * em1;

    terms[0] = w * loss;
    terms[1] = w * pg;
    terms[2] = w * kl;
    return w * (pg_grad + kl_grad);
}

/* src/cpu/grpo_loss.cpp:60-174 */
int grpo_oracle_loss(const float* lp_new, const float* lp_old, const float* lp_ref,
                     const float* adv, const int* mask, int B, int G, int T,
                     float clip_eps, float beta, int reduction, float alpha,
                     float* dlogp, float* stats, int* valid_out) {
    size_t n_seq, n_tok;
    int rc = shape_of(B, G, T, &n_seq, &n_tok);
    if (rc) return rc;
    /* option ranges (:72-77) */
    if (clip_eps < 0.0f || clip_eps >= 1.0f || !isfinite(clip_eps)) return GRPO_ORACLE_E_CLIP;
    if (beta < 0.0f || !isfinite(beta)) return GRPO_ORACLE_E_BETA;
    if (!isfinite(alpha) || alpha < 0.0f || alpha > 1.0f) return GRPO_ORACLE_E_ALPHA;

    /* input values (:88-95) */
    for (size_t i = 0; i < n_tok; i++) {
        if (!isfinite(lp_new[i]) || !isfinite(lp_old[i]) || !isfinite(lp_ref[i]))
            return GRPO_ORACLE_E_LOGP;
        if (mask[i] != 0 && mask[i] != 1) return GRPO_ORACLE_E_MASK;
    }
    for (size_t s = 0; s < n_seq; s++)
        if (!isfinite(adv[s])) return GRPO_ORACLE_E_ADV;

    /* valid-token count per response and overall (:97-108) */
    int* len = (int*)calloc(n_seq, sizeof(int));
    if (!len) abort();
    int valid = 0;
    for (size_t i = 0; i < n_tok; i++) {
        if (mask[i] == 0) continue;
        len[i / (size_t)T]++;
        valid++;
    }
    for (size_t s = 0; s < n_seq; s++) {
        if (len[s] == 0) { free(len); return GRPO_ORACLE_E_EMPTY_SEQ; }
    }

    *valid_out = valid;
    for (size_t i = 0; i < n_tok; i++) dlogp[i] = 0.0f;

    double sum_loss = 0.0, sum_pg = 0.0, sum_kl = 0.0;
    const float lo = 1.0f - clip_eps;
    const float hi = 1.0f + clip_eps;

    for (size_t s = 0; s < n_seq; s++) {
        const float A = adv[s];
        /* per-response weight of each of its tokens (:124-131) */
        float w;
        if (reduction == GRPO_ORACLE_SEQUENCE_MEAN) {
            w = 1.0f / ((float)n_seq * (float)len[s]);
        } else if (reduction == GRPO_ORACLE_TOKEN_MEAN) {
            w = 1.0f / (float)valid;
        } else {
            w = powf((float)len[s], alpha - 1.0f) / (float)n_seq;
        }

        for (int t = 0; t < T; t++) {
            size_t i = s * (size_t)T + (size_t)t;
            if (mask[i] == 0) continue;

            float terms[3];
            dlogp[i] = one_token(lp_new[i], lp_old[i], lp_ref[i], A, w, lo, hi, beta, terms);
            /* fp32 products, double running totals (:157-160) */
            sum_loss += terms[0];
            sum_pg += terms[1];
            sum_kl += terms[2];
        }
    }
    free(len);

    stats[0] = (float)sum_loss;
    stats[1] = (float)sum_pg;
    stats[2] = (float)sum_kl;
    if (!isfinite(stats[0]) || !isfinite(stats[1]) || !isfinite(stats[2]))
        return GRPO_ORACLE_E_LOSS_NONFINITE;
    for (size_t i = 0; i < n_tok; i++)
        if (!isfinite(dlogp[i])) return GRPO_ORACLE_E_GRAD_NONFINITE;
    return GRPO_ORACLE_OK;
}

/* src/cpu/grpo_loss.cpp:176-239 */
int grpo_oracle_logits(const float* logits, const float* lp_old, const float* lp_ref,
                       const int* selected, const float* adv, const int* mask,
                       int B, int G, int T, int V,
                       float clip_eps, float beta, int reduction, float alpha,
                       float* dlogits, float* stats, int* valid_out, float* sel_logp_out) {
    size_t n_seq, n_tok;
    int rc = shape_of(B, G, T, &n_seq, &n_tok);
    if (rc) return rc;
    if (V <= 0) return GRPO_ORACLE_E_VOCAB;
    const size_t vocab = (size_t)V;
    if (n_tok > ((size_t)-1) / vocab) return GRPO_ORACLE_E_LOGITS_OVERFLOW;

    float* sel_logp = (float*)calloc(n_tok, sizeof(float));
    float* dlogp = (float*)malloc(n_tok * sizeof(float));
    if (!sel_logp || !dlogp) abort();

    /* forward: log-softmax of the selected token, in double, active rows only (:200-216) */
    for (size_t i = 0; i < n_tok; i++) {
        if (mask[i] == 0) continue;
        int sel = selected[i];
        if (sel < 0 || sel >= V) { rc = GRPO_ORACLE_E_SELECTED; goto done; }
        const float* row = logits + i * vocab;
        double top = row[0];
        for (int v = 0; v < V; v++) {
            if (!isfinite(row[v])) { rc = GRPO_ORACLE_E_LOGITS; goto done; }
            double x = (double)row[v];
            top = top < x ? x : top;
        }
        double z = 0.0;
        for (int v = 0; v < V; v++) z += exp((double)row[v] - top);
        double lse = top + log(z);
        sel_logp[i] = (float)((double)row[sel] - lse);
    }

    /* token loss on the gathered log-probabilities (:218-220) */
    rc = grpo_oracle_loss(sel_logp, lp_old, lp_ref, adv, mask, B, G, T,
                          clip_eps, beta, reduction, alpha, dlogp, stats, valid_out);
    if (rc) goto done;

    /* backward through log-softmax (:223-237): rows with a zero dlogp stay zero */
    memset(dlogits, 0, n_tok * vocab * sizeof(float));
    for (size_t i = 0; i < n_tok; i++) {
        float g = dlogp[i];
        if (g == 0.0f) continue;
        int sel = selected[i];
        const float* row = logits + i * vocab;
        float* out = dlogits + i * vocab;
        double x_sel = row[sel];
        for (int v = 0; v < V; v++) {
            double p = exp((double)row[v] - x_sel + sel_logp[i]);
            out[v] = g * ((v == sel ? 1.0f : 0.0f) - (float)p);
        }
    }
    if (sel_logp_out) memcpy(sel_logp_out, sel_logp, n_tok * sizeof(float));

done:
    free(sel_logp);
    free(dlogp);
    return rc;
}

/* The per-row steps of grpo_oracle_logits for rows taken out of a batch that is too large to hold
 * on the host: forward (src/cpu/grpo_loss.cpp:200-216), token loss (:137-160) and backward
 * (:223-237) of each given row, with its response's advantage and weight passed in (the caller
 * derives the weight from the whole batch's mask with the expressions of :124-131). */
int grpo_oracle_logits_rows(const float* rows, int n, int V, const float* lp_old, const float* lp_ref,
                            const int* selected, const float* adv, const float* w, float clip_eps,
                            float beta, float* dlogits, float* sel_logp_out, float* terms_out) {
    if (n <= 0) return GRPO_ORACLE_E_DIMS;
    if (V <= 0) return GRPO_ORACLE_E_VOCAB;
    if (clip_eps < 0.0f || clip_eps >= 1.0f || !isfinite(clip_eps)) return GRPO_ORACLE_E_CLIP;
    if (beta < 0.0f || !isfinite(beta)) return GRPO_ORACLE_E_BETA;
    const size_t vocab = (size_t)V;
    const float lo = 1.0f - clip_eps;
    const float hi = 1.0f + clip_eps;
    for (int i = 0; i < n; i++) {
        int sel = selected[i];
        if (sel < 0 || sel >= V) return GRPO_ORACLE_E_SELECTED;
        const float* row = rows + (size_t)i * vocab;
        float* out = dlogits + (size_t)i * vocab;
        double top = row[0];
        for (int v = 0; v < V; v++) {
            if (!isfinite(row[v])) return GRPO_ORACLE_E_LOGITS;
            double x = (double)row[v];
            top = top < x ? x : top;
        }
        double z = 0.0;
        for (int v = 0; v < V; v++) z += exp((double)row[v] - top);
        double lse = top + log(z);
        float sel_logp = (float)((double)row[sel] - lse);
        if (sel_logp_out) sel_logp_out[i] = sel_logp;
        float g = one_token(sel_logp, lp_old[i], lp_ref[i], adv[i], w[i], lo, hi, beta, terms_out + 3 * (size_t)i);
        memset(out, 0, vocab * sizeof(float));
        if (g == 0.0f) continue;
        double x_sel = row[sel];
        for (int v = 0; v < V; v++) {
            double p = exp((double)row[v] - x_sel + sel_logp);
            out[v] = g * ((v == sel ? 1.0f : 0.0f) - (float)p);
        }
    }
    return GRPO_ORACLE_OK;
}

/* apps/04_gpt2_grpo.cu:61-66 */
double grpo_oracle_row_logsumexp(const float* row, int V) {
    float top = row[0];
    for (int v = 1; v < V; v++)
        if (row[v] > top) top = row[v];
    double sum = 0.0;
    for (int v = 0; v < V; v++) sum += exp((double)(row[v] - top));
    return (double)top + log(sum);
}

/* apps/04_gpt2_grpo.cu:68-80 */
int grpo_oracle_sample_row(const float* row, int V, double coin) {
    double lse = grpo_oracle_row_logsumexp(row, V);
    double cumulative = 0.0;
    for (int v = 0; v < V; v++) {
        cumulative += exp((double)row[v] - lse);
        if (coin < cumulative) return v;
    }
    return V - 1;
}

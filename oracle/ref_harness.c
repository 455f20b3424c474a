/*
 * oracle/ref_harness.c — TEST INFRASTRUCTURE, never linked into the product.
 *
 * A thin driver around the UNMODIFIED reference sampler. It textually includes
 * the reference translation unit (src/engine/sampler.c, found through -I at
 * build time; no reference source is copied into this repository) so that the
 * file-local helpers softmax_into / inv_cdf_sample / cmp_desc_logit are
 * reachable, and exposes plain-C entry points that ctypes can bind:
 *
 *   ref_rng_*            reference xorshift64* stream      (sampler.c:27-48)
 *   ref_sample           per-row 4-way dispatch            (head.c:172-183, :289-303)
 *   ref_softmax          softmax_into + normalise          (sampler.c:68-85, :253-255)
 *   ref_topk_detail      kept set + probabilities of top-k (sampler.c:178-228)
 *   ref_topp_detail      nucleus + probabilities of top-p  (sampler.c:232-305)
 *   ref_softcap          the output head's final-logit soft cap, the reference's expression with this
 *                        host's tanhf (src/archs/transformer/forward/head.c:148-159, :279-288; the head
 *                        itself does not compile outside its engine, so the one-line loop is restated)
 *
 * Everything numeric below is executed by the reference's own code; this file
 * only loops, dispatches and copies results out.
 */
#include "src/engine/sampler.c" /* the reference TU itself */

#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

uint64_t ref_rng_seed_state(uint64_t seed) {
    struct geist_rng r;
    geist_rng_seed(&r, seed);
    return r.state;
}

/* n raw draws and n unit draws from two fresh generators with the same seed. */
void ref_rng_vectors(uint64_t seed, size_t n, uint64_t *out_u64, float *out_unit) {
    struct geist_rng a, b;
    geist_rng_seed(&a, seed);
    geist_rng_seed(&b, seed);
    for (size_t i = 0; i < n; i++) {
        out_u64[i]  = geist_rng_next_u64(&a);
        out_unit[i] = geist_rng_next_unit(&b);
    }
}

/* Advance a raw state by n draws (what a session's rng looks like after n rows). */
uint64_t ref_rng_advance(uint64_t state, size_t n) {
    struct geist_rng r = {.state = state};
    for (size_t i = 0; i < n; i++) {
        (void) geist_rng_next_u64(&r);
    }
    return r.state;
}

static geist_token_t dispatch_row(struct geist_sampler_workspace *ws,
                                  size_t                          V,
                                  const float                    *row,
                                  float                           T,
                                  int                             top_k,
                                  float                           top_p,
                                  struct geist_rng               *rng) {
    /* Same exclusive precedence as finalize_logits_one_row. */
    if (T == 0.0f) {
        return geist_sampler_argmax(V, row);
    } else if (top_k > 1) {
        return geist_sampler_top_k_ws(ws, row, top_k, T, rng);
    } else if (top_p > 0.0f && top_p < 1.0f) {
        return geist_sampler_top_p_ws(ws, row, top_p, T, rng);
    }
    return geist_sampler_temperature(V, row, T, rng);
}

/*
 * S sequences of R rows each, logits [S, R, V] (row stride `stride` floats).
 * Sequence s owns one generator (rng_state[s], in/out) and samples its R rows
 * in order, exactly like finalize_logits_batch does for one session. R == 1 is
 * the plain batched case. Parameters are per sequence. Returns 0, or -1 on OOM.
 */
int ref_sample(const float *logits,
               size_t       S,
               size_t       R,
               size_t       V,
               size_t       stride,
               const float *temperature,
               const int   *top_k,
               const float *top_p,
               uint64_t    *rng_state,
               int32_t     *tokens,
               int          nthreads) {
    int failed = 0;
#ifdef _OPENMP
    if (nthreads > 0) {
        omp_set_num_threads(nthreads);
    }
#else
    (void) nthreads;
#endif
#pragma omp parallel
    {
        struct geist_sampler_workspace ws = {0};
        if (geist_sampler_workspace_init(&ws, V) != GEIST_OK) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(dynamic, 1)
            for (size_t s = 0; s < S; s++) {
                struct geist_rng rng = {.state = rng_state[s]};
                for (size_t r = 0; r < R; r++) {
                    const float *row   = logits + (s * R + r) * stride;
                    tokens[s * R + r] = dispatch_row(&ws, V, row, temperature[s], top_k[s], top_p[s], &rng);
                }
                rng_state[s] = rng.state;
            }
        }
        geist_sampler_workspace_destroy(&ws);
    }
    return failed ? -1 : 0;
}

/* Direct single calls, for the literal arrays of tests/test_sampler_unit.c. */
int32_t ref_argmax(size_t V, const float *row) { return geist_sampler_argmax(V, row); }

int32_t ref_temperature(size_t V, const float *row, float T, uint64_t *state) {
    struct geist_rng rng = {.state = *state};
    geist_token_t    t   = geist_sampler_temperature(V, row, T, &rng);
    *state               = rng.state;
    return t;
}

int32_t ref_top_k(size_t V, const float *row, int top_k, float T, uint64_t *state) {
    struct geist_sampler_workspace ws = {0};
    if (geist_sampler_workspace_init(&ws, V) != GEIST_OK) {
        return -1;
    }
    struct geist_rng rng = {.state = *state};
    geist_token_t    t   = geist_sampler_top_k_ws(&ws, row, top_k, T, &rng);
    *state               = rng.state;
    geist_sampler_workspace_destroy(&ws);
    return t;
}

int32_t ref_top_p(size_t V, const float *row, float top_p, float T, uint64_t *state) {
    struct geist_sampler_workspace ws = {0};
    if (geist_sampler_workspace_init(&ws, V) != GEIST_OK) {
        return -1;
    }
    struct geist_rng rng = {.state = *state};
    geist_token_t    t   = geist_sampler_top_p_ws(&ws, row, top_p, T, &rng);
    *state               = rng.state;
    geist_sampler_workspace_destroy(&ws);
    return t;
}

/* probs[i] = (float)((double) e_i / sum) — the vector top-p sorts. Returns sum. */
double ref_softmax(size_t V, const float *row, float T, float *probs) {
    double sum = softmax_into(V, row, T, probs);
    for (size_t i = 0; i < V; i++) {
        probs[i] = (float) ((double) probs[i] / sum);
    }
    return sum;
}

/*
 * The k entries the top-k path keeps, in the order it walks them, with
 * q_i / sum as float. Returns k (after the 8192 clamp), or 0 when the call
 * would have left the top-k path (top_k <= 1, T <= 0, top_k >= V).
 */
int ref_topk_detail(size_t V, const float *row, int top_k, float T, int32_t *idx, float *prob, float *unnorm, double *sum_out) {
    if (top_k <= 1 || T <= 0.0f || (size_t) top_k >= V) {
        return 0;
    }
    struct kv_pair *pairs = malloc(V * sizeof *pairs);
    if (pairs == nullptr) {
        return -1;
    }
    for (size_t i = 0; i < V; i++) {
        pairs[i].logit = row[i];
        pairs[i].idx   = (uint32_t) i;
    }
    qsort(pairs, V, sizeof *pairs, cmp_desc_logit);
    int k = top_k > 8192 ? 8192 : top_k;
    float *tl = malloc((size_t) k * sizeof *tl);
    float *tp = malloc((size_t) k * sizeof *tp);
    for (int i = 0; i < k; i++) {
        tl[i] = pairs[i].logit;
    }
    double sum = softmax_into((size_t) k, tl, T, tp);
    for (int i = 0; i < k; i++) {
        idx[i]  = (int32_t) pairs[i].idx;
        prob[i] = (float) ((double) tp[i] / sum);
        if (unnorm != nullptr) {
            unnorm[i] = tp[i];
        }
    }
    if (sum_out != nullptr) {
        *sum_out = sum;
    }
    free(tl);
    free(tp);
    free(pairs);
    return k;
}

/*
 * The nucleus of the top-p path in walk order. Writes at most `cap` entries
 * of (index, normalised prob p_i, p_i / nucleus_sum) and returns the cutoff
 * (nucleus size); 0 when the call would have left the top-p path.
 */
long ref_topp_detail(size_t V, const float *row, float top_p, float T, size_t cap, int32_t *idx, float *p_norm, float *p_nucleus, double *nucleus_sum_out) {
    if (top_p <= 0.0f || T <= 0.0f || top_p >= 1.0f) {
        return 0;
    }
    float          *probs = malloc(V * sizeof *probs);
    struct kv_pair *pairs = malloc(V * sizeof *pairs);
    if (probs == nullptr || pairs == nullptr) {
        free(probs);
        free(pairs);
        return -1;
    }
    double sum = softmax_into(V, row, T, probs);
    for (size_t i = 0; i < V; i++) {
        pairs[i].logit = (float) ((double) probs[i] / sum);
        pairs[i].idx   = (uint32_t) i;
    }
    qsort(pairs, V, sizeof *pairs, cmp_desc_logit);
    double cum    = 0.0;
    size_t cutoff = 0;
    for (cutoff = 0; cutoff < V; cutoff++) {
        cum += (double) pairs[cutoff].logit;
        if (cum >= (double) top_p) {
            cutoff++;
            break;
        }
    }
    if (cutoff < 1) {
        cutoff = 1;
    }
    double nsum = 0.0;
    for (size_t i = 0; i < cutoff; i++) {
        nsum += (double) pairs[i].logit;
    }
    for (size_t i = 0; i < cutoff && i < cap; i++) {
        idx[i]       = (int32_t) pairs[i].idx;
        p_norm[i]    = pairs[i].logit;
        p_nucleus[i] = (float) ((double) pairs[i].logit / nsum);
    }
    if (nucleus_sum_out != nullptr) {
        *nucleus_sum_out = nsum;
    }
    free(probs);
    free(pairs);
    return (long) cutoff;
}

/* head.c:152-155 / :284-287: p[i] = tanhf(p[i] / c) * c, in place. */
void ref_softcap(size_t n, float *p, float c) {
    for (size_t i = 0; i < n; i++) {
        p[i] = tanhf(p[i] / c) * c;
    }
}

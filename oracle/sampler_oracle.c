/*
 * oracle/sampler_oracle.c — TEST INFRASTRUCTURE: a CPU restatement of the
 * logits -> token path of geistlib, used only as the checker for the CUDA
 * kernels (tests, the smoke check, the bench's CPU leg). The product never
 * calls into this file and has no CPU fallback.
 *
 * What it restates (reference file:line, paths inside the geistlib tree):
 *   xorshift64* generator ................ src/engine/sampler.c:27-48
 *   greedy argmax ........................ src/engine/sampler.c:52-62
 *   softmax with temperature ............. src/engine/sampler.c:68-85
 *   inverse-CDF draw ..................... src/engine/sampler.c:90-102
 *   temperature / top-k / top-p samplers . src/engine/sampler.c:106-132, :178-228, :232-305
 *   4-way exclusive mode dispatch ........ src/archs/transformer/forward/head.c:172-183
 *   one generator per session, rows in order  head.c:274-306
 *   session option normalisation ......... src/archs/transformer/forward/step.c:385-411
 *   speculative prefix-accept rule ....... src/engine/session.c:599-625
 *
 * Pinning: every function here is compared with the reference's own compiled
 * sampler (oracle/_ref) on random and adversarial inputs by the CPU test
 * suite, and with golden vectors that were produced by that reference build.
 *
 * Two parts have no counterpart in geistlib and are therefore "parity
 * unpinned" (this file is their specification):
 *   - repetition / frequency / presence penalties (orc_apply_penalties);
 *   - the merge of per-shard top-k candidates (orc_merge_candidates).
 *
 * The sort order the reference gets from glibc's stable qsort is made
 * explicit here: (key descending, index ascending).
 *
 * Build with -ffp-contract=off and without -ffast-math (oracle/Makefile does):
 * the penalty arithmetic and (x - max) * inv_t are meant as separately
 * rounded binary32 operations.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_TOPK_CLAMP 8192 /* sampler.c:212-215 */

/* ------------------------------------------------------------------ rng -- */

uint64_t orc_rng_seed(uint64_t seed) { /* sampler.c:27-33: zero is remapped */
    return seed ? seed : 0x9E3779B97F4A7C15ULL;
}

uint64_t orc_rng_next(uint64_t *state) { /* sampler.c:35-42 */
    uint64_t s = *state;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    *state = s;
    return s * 0x2545F4914F6CDD1DULL;
}

float orc_rng_unit(uint64_t *state) { /* sampler.c:44-48: top 24 bits / 2^24 */
    return (float) (uint32_t) (orc_rng_next(state) >> 40) * (1.0f / 16777216.0f);
}

uint64_t orc_rng_advance(uint64_t state, size_t n) {
    while (n--) {
        (void) orc_rng_next(&state);
    }
    return state;
}

/* -------------------------------------------------------------- penalties -- */

/*
 * EXTENSION (no geistlib counterpart; this is the specification).
 * For every distinct id t in hist[0..H) with 0 <= t < V and multiplicity c:
 *     x = row[t]
 *     x = x > 0 ? x / rep : x * rep          (rep <= 0 is read as 1)
 *     x = x - (float)c * freq                (product rounded, then difference)
 *     x = x - pres
 * each step one IEEE-754 binary32 operation, no fused multiply-add. With
 * rep == 1 and freq == pres == 0 every step is the identity, so the row is
 * bit-identical to the input. Ids outside [0, V) are ignored.
 */
void orc_apply_penalties(float *row, size_t V, const int32_t *hist, size_t H, float rep, float freq, float pres) {
    if (H == 0) {
        return;
    }
    if (!(rep > 0.0f)) {
        rep = 1.0f;
    }
    uint32_t *count = calloc(V, sizeof *count);
    for (size_t j = 0; j < H; j++) {
        if (hist[j] >= 0 && (size_t) hist[j] < V) {
            count[hist[j]]++;
        }
    }
    for (size_t j = 0; j < H; j++) {
        int32_t t = hist[j];
        if (t < 0 || (size_t) t >= V || count[t] == 0) {
            continue;
        }
        float x  = row[t];
        x        = x > 0.0f ? x / rep : x * rep;
        float d  = (float) count[t] * freq;
        x        = x - d;
        x        = x - pres;
        row[t]   = x;
        count[t] = 0; /* each distinct id once */
    }
    free(count);
}

/* ----------------------------------------------------------------- argmax -- */

int32_t orc_argmax(const float *row, size_t V) { /* sampler.c:52-62: strict >, first wins */
    size_t best = 0;
    for (size_t i = 1; i < V; i++) {
        if (row[i] > row[best]) {
            best = i;
        }
    }
    return (int32_t) best;
}

/* ---------------------------------------------------------- ordered pairs -- */

struct orc_pair {
    float    key;
    uint32_t idx;
};

/* a goes before b: larger key first; equal (or unordered) keys by lower index. */
static int pair_before(const struct orc_pair *a, const struct orc_pair *b) {
    if (a->key > b->key) {
        return 1;
    }
    if (a->key < b->key) {
        return 0;
    }
    return a->idx < b->idx;
}

/* Bottom-up merge sort into (key desc, idx asc); `tmp` has n entries. */
static void sort_pairs(struct orc_pair *a, struct orc_pair *tmp, size_t n) {
    struct orc_pair *src = a, *dst = tmp;
    for (size_t w = 1; w < n; w *= 2) {
        for (size_t lo = 0; lo < n; lo += 2 * w) {
            size_t mid = lo + w < n ? lo + w : n;
            size_t hi  = lo + 2 * w < n ? lo + 2 * w : n;
            size_t i = lo, j = mid, o = lo;
            while (i < mid && j < hi) {
                dst[o++] = pair_before(&src[j], &src[i]) ? src[j++] : src[i++];
            }
            while (i < mid) {
                dst[o++] = src[i++];
            }
            while (j < hi) {
                dst[o++] = src[j++];
            }
        }
        struct orc_pair *t = src;
        src                = dst;
        dst                = t;
    }
    if (src != a) {
        memcpy(a, src, n * sizeof *a);
    }
}

/* ---------------------------------------------------------------- softmax -- */

/* e_i = expf((x_i - max) * inv_t), returns sum of e_i as double, index order
 * (sampler.c:68-85). inv_t = 1/T for T > 0 else 1. */
static double exp_weights(const float *x, size_t n, float T, float *e) {
    float m = x[0];
    for (size_t i = 1; i < n; i++) {
        if (x[i] > m) {
            m = x[i];
        }
    }
    const float inv_t = T > 0.0f ? 1.0f / T : 1.0f;
    double      sum   = 0.0;
    for (size_t i = 0; i < n; i++) {
        e[i] = expf((x[i] - m) * inv_t); /* built with -ffp-contract=off: two roundings */
        sum += (double) e[i];
    }
    return sum;
}

/* First i with u*sum < running double prefix; n-1 if never (sampler.c:90-102). */
static size_t inverse_cdf(const float *w, size_t n, double sum, uint64_t *rng) {
    const double u   = (double) orc_rng_unit(rng) * sum;
    double       acc = 0.0;
    for (size_t i = 0; i < n; i++) {
        acc += (double) w[i];
        if (u < acc) {
            return i;
        }
    }
    return n - 1;
}

/* Normalised softmax probabilities as the top-p path forms them
 * (sampler.c:248-255): p_i = (float)((double)e_i / sum). Returns the sum. */
double orc_softmax(const float *row, size_t V, float T, float *probs) {
    double sum = exp_weights(row, V, T, probs);
    for (size_t i = 0; i < V; i++) {
        probs[i] = (float) ((double) probs[i] / sum);
    }
    return sum;
}

/* ------------------------------------------------------------ the samplers -- */

struct orc_scratch {
    float           *w;     /* V floats */
    struct orc_pair *pairs; /* V */
    struct orc_pair *tmp;   /* V */
    size_t           V;
};

static int scratch_init(struct orc_scratch *s, size_t V) {
    s->V     = V;
    s->w     = malloc(V * sizeof *s->w);
    s->pairs = malloc(V * sizeof *s->pairs);
    s->tmp   = malloc(V * sizeof *s->tmp);
    return (s->w && s->pairs && s->tmp) ? 0 : -1;
}

static void scratch_free(struct orc_scratch *s) {
    free(s->w);
    free(s->pairs);
    free(s->tmp);
}

/* Compact description of the kept set of one row (optional output). */
struct orc_detail {
    int32_t  n;       /* kept entries (k, nucleus size; 0 for argmax/temperature) */
    int32_t  cap;     /* capacity of idx/prob */
    int32_t *idx;     /* vocabulary ids in walk order */
    float   *prob;    /* kept-set probabilities, renormalised inside the kept set */
};

static int32_t sample_temperature(struct orc_scratch *s, const float *row, size_t V, float T, uint64_t *rng) {
    if (T <= 0.0f) { /* sampler.c:110-112 */
        return orc_argmax(row, V);
    }
    double sum = exp_weights(row, V, T, s->w);
    return (int32_t) inverse_cdf(s->w, V, sum, rng);
}

static int32_t sample_top_k(struct orc_scratch *s, const float *row, size_t V, int top_k, float T, uint64_t *rng, struct orc_detail *d) {
    if (top_k <= 1 || T <= 0.0f) { /* sampler.c:184-186 */
        return orc_argmax(row, V);
    }
    if ((size_t) top_k >= V) { /* sampler.c:187-189 */
        return sample_temperature(s, row, V, T, rng);
    }
    for (size_t i = 0; i < V; i++) {
        s->pairs[i].key = row[i];
        s->pairs[i].idx = (uint32_t) i;
    }
    sort_pairs(s->pairs, s->tmp, V);
    const size_t k = top_k > ORC_TOPK_CLAMP ? ORC_TOPK_CLAMP : (size_t) top_k;
    float        kept[ORC_TOPK_CLAMP], q[ORC_TOPK_CLAMP];
    for (size_t i = 0; i < k; i++) {
        kept[i] = s->pairs[i].key;
    }
    double sum  = exp_weights(kept, k, T, q); /* max of the kept set = its first entry */
    size_t pick = inverse_cdf(q, k, sum, rng);
    if (d != NULL) {
        d->n = (int32_t) k;
        for (size_t i = 0; i < k && (int32_t) i < d->cap; i++) {
            d->idx[i]  = (int32_t) s->pairs[i].idx;
            d->prob[i] = (float) ((double) q[i] / sum);
        }
    }
    return (int32_t) s->pairs[pick].idx;
}

static int32_t sample_top_p(struct orc_scratch *s, const float *row, size_t V, float top_p, float T, uint64_t *rng, struct orc_detail *d) {
    if (top_p <= 0.0f || T <= 0.0f) { /* sampler.c:238-240 */
        return orc_argmax(row, V);
    }
    if (top_p >= 1.0f) { /* sampler.c:241-243 */
        return sample_temperature(s, row, V, T, rng);
    }
    double sum = exp_weights(row, V, T, s->w);
    if (sum <= 0.0) { /* sampler.c:249-251 */
        return orc_argmax(row, V);
    }
    for (size_t i = 0; i < V; i++) {
        s->pairs[i].key = (float) ((double) s->w[i] / sum);
        s->pairs[i].idx = (uint32_t) i;
    }
    sort_pairs(s->pairs, s->tmp, V);
    /* smallest prefix whose double running sum reaches top_p, inclusive (sampler.c:273-283) */
    double cum = 0.0;
    size_t cut = V;
    for (size_t i = 0; i < V; i++) {
        cum += (double) s->pairs[i].key;
        if (cum >= (double) top_p) {
            cut = i + 1;
            break;
        }
    }
    if (cut < 1) {
        cut = 1;
    }
    double nsum = 0.0;
    for (size_t i = 0; i < cut; i++) {
        nsum += (double) s->pairs[i].key;
    }
    const double u    = (double) orc_rng_unit(rng) * nsum;
    double       acc  = 0.0;
    size_t       pick = cut - 1; /* default: last nucleus entry (sampler.c:292) */
    for (size_t i = 0; i < cut; i++) {
        acc += (double) s->pairs[i].key;
        if (u < acc) {
            pick = i;
            break;
        }
    }
    if (d != NULL) {
        d->n = (int32_t) cut;
        for (size_t i = 0; i < cut && (int32_t) i < d->cap; i++) {
            d->idx[i]  = (int32_t) s->pairs[i].idx;
            d->prob[i] = (float) ((double) s->pairs[i].key / nsum);
        }
    }
    return (int32_t) s->pairs[pick].idx;
}

/* head.c:172-183: T == 0 -> greedy; top_k > 1 -> top-k (top_p ignored);
 * 0 < top_p < 1 -> top-p; else plain temperature. */
static int32_t sample_dispatch(struct orc_scratch *s, const float *row, size_t V, float T, int top_k, float top_p, uint64_t *rng, struct orc_detail *d) {
    if (d != NULL) {
        d->n = 0;
    }
    if (T == 0.0f) {
        return orc_argmax(row, V);
    }
    if (top_k > 1) {
        return sample_top_k(s, row, V, top_k, T, rng, d);
    }
    if (top_p > 0.0f && top_p < 1.0f) {
        return sample_top_p(s, row, V, top_p, T, rng, d);
    }
    return sample_temperature(s, row, V, T, rng);
}

/* One row, for direct comparison with the reference entry points. */
int32_t orc_sample_row(const float *row, size_t V, float T, int top_k, float top_p, uint64_t *rng_state, int32_t detail_cap, int32_t *detail_n, int32_t *detail_idx, float *detail_prob) {
    struct orc_scratch s;
    if (scratch_init(&s, V) != 0) {
        scratch_free(&s);
        return -1;
    }
    struct orc_detail d   = {0, detail_cap, detail_idx, detail_prob};
    int32_t           tok = sample_dispatch(&s, row, V, T, top_k, top_p, rng_state, detail_cap > 0 ? &d : NULL);
    if (detail_n != NULL) {
        *detail_n = d.n;
    }
    scratch_free(&s);
    return tok;
}

/* Direct calls of the three sampler entry points (not through the dispatch),
 * for the cases tests/test_sampler_unit.c drives that way. which: 0 temperature,
 * 1 top-k, 2 top-p. */
int32_t orc_sampler_call(int which, const float *row, size_t V, float T, int top_k, float top_p, uint64_t *rng_state) {
    struct orc_scratch s;
    if (scratch_init(&s, V) != 0) {
        scratch_free(&s);
        return -1;
    }
    int32_t tok;
    if (which == 1) {
        tok = sample_top_k(&s, row, V, top_k, T, rng_state, NULL);
    } else if (which == 2) {
        tok = sample_top_p(&s, row, V, top_p, T, rng_state, NULL);
    } else {
        tok = sample_temperature(&s, row, V, T, rng_state);
    }
    scratch_free(&s);
    return tok;
}

/*
 * Batched sampling: S sequences x R rows, logits [S, R, V] with `stride`
 * floats between rows. Sequence s has one generator (rng_state[s], in/out)
 * that its R rows consume in order (head.c:282-303), one parameter set, and
 * an optional id history hist[s*hist_stride .. +hist_len[s]) for the penalty
 * extension. `extra`, when given, holds the tokens fed through a verify pass
 * (extra[s][0] = the pending token, already part of the history; the rest are
 * proposals): row r additionally sees extra[s][1..r] as history. Optional outputs: the penalised rows, and the kept set
 * (detail_cap entries per row).
 */
int orc_sample_batch(const float   *logits,
                     size_t         S,
                     size_t         R,
                     size_t         V,
                     size_t         stride,
                     const float   *temperature,
                     const int32_t *top_k,
                     const float   *top_p,
                     const float   *rep,
                     const float   *freq,
                     const float   *pres,
                     const int32_t *hist,
                     size_t         hist_stride,
                     const int32_t *hist_len,
                     const int32_t *extra,
                     size_t         extra_stride,
                     uint64_t      *rng_state,
                     int32_t       *tokens,
                     float         *out_logits,
                     int32_t        detail_cap,
                     int32_t       *detail_n,
                     int32_t       *detail_idx,
                     float         *detail_prob,
                     int            nthreads) {
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
        struct orc_scratch sc;
        float             *work = malloc(V * sizeof *work);
        if (scratch_init(&sc, V) != 0 || work == NULL) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(dynamic, 1)
            for (size_t s = 0; s < S; s++) {
                uint64_t rng = rng_state[s];
                for (size_t r = 0; r < R; r++) {
                    const size_t row_id = s * R + r;
                    const float *row    = logits + row_id * stride;
                    const int    pen    = hist != NULL && hist_len != NULL && (hist_len[s] > 0 || extra != NULL);
                    if (pen) {
                        memcpy(work, row, V * sizeof *work);
                        /* history and the fed tokens form ONE multiset */
                        size_t   H   = (size_t) (hist_len[s] > 0 ? hist_len[s] : 0);
                        size_t   E   = extra != NULL ? r : 0;
                        int32_t *all = malloc((H + E + 1) * sizeof *all);
                        memcpy(all, hist + s * hist_stride, H * sizeof *all);
                        if (E) {
                            memcpy(all + H, extra + s * extra_stride + 1, E * sizeof *all);
                        }
                        orc_apply_penalties(work, V, all, H + E, rep ? rep[s] : 1.0f, freq ? freq[s] : 0.0f, pres ? pres[s] : 0.0f);
                        free(all);
                        row = work;
                    }
                    if (out_logits != NULL) {
                        memcpy(out_logits + row_id * V, row, V * sizeof *row);
                    }
                    struct orc_detail d = {0, detail_cap, detail_idx ? detail_idx + row_id * (size_t) detail_cap : NULL, detail_prob ? detail_prob + row_id * (size_t) detail_cap : NULL};
                    tokens[row_id]      = sample_dispatch(&sc, row, V, temperature[s], top_k[s], top_p[s], &rng, detail_cap > 0 ? &d : NULL);
                    if (detail_n != NULL) {
                        detail_n[row_id] = d.n;
                    }
                }
                rng_state[s] = rng;
            }
        }
        scratch_free(&sc);
        free(work);
    }
    return failed ? -1 : 0;
}

/* ------------------------------------------------------------- speculative -- */

/*
 * session.c:599-625. fed[0..k) are the tokens pushed through the verify pass
 * (fed[0] = the already pending token, fed[1..k) = proposals); verify_out[i] is
 * the token sampled from row i. accepted = longest run of i < k-1 with
 * verify_out[i] == fed[i+1]. Emits fed[0..accepted] followed by
 * verify_out[accepted] (which is the bonus token when everything matched).
 * Returns the number of emitted tokens (accepted + 2).
 */
size_t orc_spec_accept(size_t k, const int32_t *fed, const int32_t *verify_out, int32_t *emitted, int32_t *accepted_out) {
    size_t a = 0;
    while (a + 1 < k && verify_out[a] == fed[a + 1]) {
        a++;
    }
    for (size_t i = 0; i <= a; i++) {
        emitted[i] = fed[i];
    }
    emitted[a + 1] = verify_out[a];
    if (accepted_out != NULL) {
        *accepted_out = (int32_t) a;
    }
    return a + 2;
}

/* ------------------------------------------------------------ vocab shards -- */

/*
 * EXTENSION (no geistlib counterpart). n candidates (value, global id) gathered
 * from all vocabulary shards of one row; keeps the k best in (value desc,
 * id asc) order. With per-shard lists that each hold their shard's best
 * min(k, shard size) entries the result equals the top-k of the whole row.
 */
void orc_merge_candidates(size_t n, const float *val, const int32_t *gid, size_t k, float *out_val, int32_t *out_gid) {
    struct orc_pair *p = malloc(n * sizeof *p), *t = malloc(n * sizeof *t);
    for (size_t i = 0; i < n; i++) {
        p[i].key = val[i];
        p[i].idx = (uint32_t) gid[i];
    }
    sort_pairs(p, t, n);
    for (size_t i = 0; i < k && i < n; i++) {
        out_val[i] = p[i].key;
        out_gid[i] = (int32_t) p[i].idx;
    }
    free(p);
    free(t);
}

/* Top-k draw over an already ordered candidate list (sampler.c:217-222):
 * softmax of the k values with temperature, one draw. */
int32_t orc_sample_ordered(size_t k, const float *val, const int32_t *gid, float T, uint64_t *rng_state) {
    float q[ORC_TOPK_CLAMP];
    if (k > ORC_TOPK_CLAMP) {
        k = ORC_TOPK_CLAMP;
    }
    double sum = exp_weights(val, k, T, q);
    return gid[inverse_cdf(q, k, sum, rng_state)];
}

/* -------------------------------------------------------------- soft cap -- */

/* The output head's final-logit soft cap, in place: p[i] = tanhf(p[i] / c) * c
 * (src/archs/transformer/forward/head.c:152-155, :284-287). Division, tanhf and
 * product are three separately rounded binary32 steps. */
void orc_softcap(size_t n, float *p, float c) {
    for (size_t i = 0; i < n; i++) {
        float q = p[i] / c;
        q       = tanhf(q);
        p[i]    = q * c;
    }
}

/* ---------------------------------------------------------- n-gram drafter -- */

/*
 * Restates propose_drafts_ngram (src/engine/session.c:437-513). The context is
 * history + [seed]; for L = min(max_suffix, 8) down to 1 its last L tokens (L - 1
 * history tokens and the seed) are looked for at every earlier position p of the
 * history, newest first. A position counts only if at least one token follows the
 * match inside the history; among those the one with the most following tokens
 * (capped at k_max - 1) wins, the newest on ties, and the search of this L stops
 * as soon as a position offers k_max - 1 of them. The first L with a match ends
 * the search. out[0] = seed, out[1..] = the tokens that followed; returns their
 * number including the seed; *match_L = L, or 0 without a match.
 */
size_t orc_propose_drafts_ngram(const int32_t *history, size_t history_n, int32_t seed, size_t k_max, size_t max_suffix, int32_t *out, size_t *match_L) {
    out[0] = seed;
    if (match_L) {
        *match_L = 0;
    }
    if (k_max <= 1 || history_n == 0) {
        return 1;
    }
    if (max_suffix > 8) {
        max_suffix = 8;
    }
    const size_t want = k_max - 1;
    for (size_t L = max_suffix; L >= 1; L--) {
        if (L - 1 > history_n) {
            continue;
        }
        const size_t tail  = history_n - (L - 1); /* where the context's history part starts; also the number of start positions */
        size_t       best  = 0, best_follow = 0;
        int          found = 0;
        for (size_t p = tail; p-- > 0;) {
            if (history[p + L - 1] != seed || p + L >= history_n) {
                continue;
            }
            size_t i = 0;
            while (i + 1 < L && history[p + i] == history[tail + i]) {
                i++;
            }
            if (i + 1 < L) {
                continue;
            }
            size_t follow = history_n - (p + L);
            if (follow > want) {
                follow = want;
            }
            if (!found || follow > best_follow) {
                best        = p;
                best_follow = follow;
                found       = 1;
                if (follow >= want) {
                    break;
                }
            }
        }
        if (found) {
            for (size_t i = 0; i < best_follow; i++) {
                out[1 + i] = history[best + L + i];
            }
            if (match_L) {
                *match_L = L;
            }
            return 1 + best_follow;
        }
    }
    return 1;
}

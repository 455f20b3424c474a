/*
 * geist_b200.h — C ABI of the B200 (sm_100a) token-sampling path for geistlib.
 *
 * libgeist_b200.so replaces ONE path of the geistlib engine: logits -> token
 * (sampler, speculative verify/accept, multi-session batching). Three layers,
 * innermost first; each entry cites the geistlib interface it stands in for
 * (paths inside the geistlib tree):
 *
 *   1. sampler.h surface, host pointers ........ src/engine/sampler.h:27-69
 *   2. batched device entries + plugin slot ..... include/geist_backend.h:414-421,
 *                                                 src/archs/transformer/forward/head.c:131-186, :267-306
 *   3. per-session state, verify/accept, batcher  include/geist.h:209-247,
 *                                                 src/archs/transformer/arch_state.h:287-294,
 *                                                 src/archs/transformer/forward/step.c:385-411,
 *                                                 src/engine/session.c:593-636
 *
 * Conventions kept from geistlib: every fallible call returns enum geist_status
 * (0 = OK); no exceptions or errno cross this boundary; detail text through
 * geist_b200_errmsg(); per-session calls may run concurrently on different
 * sessions, never on the same one (include/geist_arch.h:43-51).
 *
 * There is no CPU fallback anywhere in this library: a call that cannot reach
 * the GPU fails with GEIST_E_BACKEND.
 *
 * EXTENSIONS (no geistlib counterpart, zero-initialised = off):
 *   Penalties. For every distinct id t of a row's history (multiplicity c),
 *   before temperature and before any filter:
 *       x = logits[t];  x = x > 0 ? x / r : x * r;   (r = repetition_penalty, r <= 0 reads as 1)
 *       x = x - (float)c * frequency_penalty;  x = x - presence_penalty;
 *   each step one binary32 operation (no fused multiply-add). Ids outside the
 *   vocabulary are ignored. In a verify pass the pending token fed[0] is taken
 *   to be part of the history already (it joined when it was sampled); row i
 *   additionally counts the proposals fed[1..i].
 *   Vocabulary shards. A shard emits its best k (value, global id); the union
 *   over shards, ordered by (value desc, id asc) and cut to k, is the row's
 *   top-k, which then goes through the ordinary top-k draw.
 */
#ifndef GEIST_B200_H
#define GEIST_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- status -- */
/* Same enumerators, same values as include/geist.h:46-67. */
#ifndef GEIST_H
enum geist_status {
    GEIST_OK = 0,
    GEIST_E_OOM,
    GEIST_E_INVALID_ARG,
    GEIST_E_INTERNAL,
    GEIST_E_FILE_NOT_FOUND,
    GEIST_E_IO,
    GEIST_E_FORMAT,
    GEIST_E_UNSUPPORTED,
    GEIST_E_NOT_FOUND,
    GEIST_E_BACKEND,
    GEIST_E_INVALID_STATE,
    GEIST_E_TOO_MANY_TOKENS,
};
typedef int32_t geist_token_t; /* include/geist.h:190 */
#endif

/* Text of the last failure on the calling thread ("" when none). Replaces the
 * per-backend error slot of include/geist_backend.h:599-626 for this path. */
const char *geist_b200_errmsg(void);

/* ------------------------------------------------- 1. sampler.h surface -- */
/* Same names, argument meaning and early-outs as src/engine/sampler.h:27-69.
 * `logits` are HOST pointers: the row is staged to the device, one kernel
 * runs, four bytes come back. On a device failure the token is -1 and
 * geist_b200_errmsg() says why (the reference's "degrade to argmax on OOM"
 * has no equivalent here: nothing is computed on the CPU). */

struct geist_rng {
    uint64_t state; /* src/engine/sampler.h:28-30 */
};

void     geist_rng_seed(struct geist_rng *rng, uint64_t seed);      /* sampler.c:27-33 */
uint64_t geist_rng_next_u64(struct geist_rng *rng);                 /* sampler.c:35-42 */
float    geist_rng_next_unit(struct geist_rng *rng);                /* sampler.c:44-48 */

geist_token_t geist_sampler_argmax(size_t n_vocab, const float *logits); /* sampler.c:52-62 */
geist_token_t geist_sampler_temperature(size_t n_vocab, const float *logits, float temperature,
                                        struct geist_rng *rng);     /* sampler.c:106-132 */

struct geist_sampler_workspace {
    float *probs;   /* here: pinned host staging for one row (sampler.h:50-53 keeps V floats of scratch) */
    size_t n_vocab;
};

enum geist_status geist_sampler_workspace_init(struct geist_sampler_workspace *ws, size_t n_vocab); /* sampler.c:136-149 */
void              geist_sampler_workspace_destroy(struct geist_sampler_workspace *ws);              /* sampler.c:151-157 */

geist_token_t geist_sampler_top_k_ws(struct geist_sampler_workspace *ws, const float *logits, int top_k,
                                     float temperature, struct geist_rng *rng); /* sampler.c:178-228 */
geist_token_t geist_sampler_top_p_ws(struct geist_sampler_workspace *ws, const float *logits, float top_p,
                                     float temperature, struct geist_rng *rng); /* sampler.c:232-305 */

/* ------------------------------------------ 2. batched device entries -- */

/* One per (device, caller). Owns the kernels' scratch memory (slice records,
 * candidate lists, row counters), which grows on demand: the first call with a
 * larger batch allocates. At most four launches of one context may be in
 * flight on the GPU at a time (they rotate over four scratch sets); callers
 * that need more overlap create more contexts. */
struct geist_b200_ctx;

enum geist_status geist_b200_ctx_create(int device, struct geist_b200_ctx **out);
void              geist_b200_ctx_destroy(struct geist_b200_ctx *ctx);

/* Row status bits written by the kernels (int32 per row). */
#define GEIST_B200_ROW_LOAD_TIMEOUT  (1 << 0) /* result invalid */
#define GEIST_B200_ROW_SLOW_PATH     (1 << 1) /* informational */
#define GEIST_B200_ROW_HIST_OVERFLOW (1 << 2) /* result invalid */
#define GEIST_B200_ROW_KEPT_PARTIAL  (1 << 3) /* kept_idx / kept_val not filled, kept_n is */
#define GEIST_B200_ROW_INTERNAL      (1 << 4) /* result invalid */
#define GEIST_B200_ROW_RETRY         (1 << 5) /* finish_hint GREEDY_TOPK / GREEDY only: not sampled (token -1), see there */

/*
 * One launch over n_seq * rows_per_seq logits rows. All pointers are DEVICE
 * pointers. A "sequence" is what geistlib calls a session's sampler state
 * (arch_state.h:287-294): one parameter set, one generator, one history. Its
 * rows_per_seq rows are sampled "in order with the same generator" exactly as
 * finalize_logits_batch does (head.c:282-303): row r starts from the state
 * left by r draws. rows_per_seq == 1 is plain batched decode (head.c:165-186).
 *
 * Mode per sequence, head.c:172-183 folded with the early-outs of the three
 * sampler functions: temperature <= 0 -> argmax, 0 draws; top_k > 1 -> top-k
 * (top_k >= n_vocab -> temperature; top_k clamps to 8192); 0 < top_p < 1 ->
 * top-p; else plain temperature. top_p is used as given: callers wanting the
 * session rule "top_p <= 0 means 1.0" (step.c:391) apply it first, as the
 * session layer below does.
 */
struct geist_b200_batch {
    const float *logits;    /* [n_seq * rows_per_seq, n_vocab] fp32 */
    size_t       row_stride; /* floats between rows (>= n_vocab) */
    size_t       n_seq;
    size_t       rows_per_seq;
    size_t       n_vocab;

    const int32_t *slot; /* optional [n_seq]: index of sequence s in every per-sequence array; NULL = s */

    const float   *temperature; /* per sequence */
    const int32_t *top_k;       /* per sequence */
    const float   *top_p;       /* per sequence */

    const float   *repetition_penalty; /* per sequence or NULL   (EXTENSION) */
    const float   *frequency_penalty;  /* per sequence or NULL   (EXTENSION) */
    const float   *presence_penalty;   /* per sequence or NULL   (EXTENSION) */
    const int32_t *history;            /* [*, history_stride] or NULL */
    size_t         history_stride;     /* also the longest history a row can have: at most 8192 ids per row (history plus
                                        * fed tokens), else GEIST_E_UNSUPPORTED. A batch whose rows can bring more than 256 ids
                                        * costs one more kernel launch (the rows' distinct ids are counted ahead of the stream
                                        * kernel). */
    const int32_t *history_len;        /* per sequence */
    const int32_t *fed_tokens;         /* optional [n_seq, fed_stride]: row r also counts fed[1..r] */
    size_t         fed_stride;

    const uint64_t *rng_in;  /* per sequence: xorshift64* state (sampler.h:28-30) */
    uint64_t       *rng_out; /* per sequence: state after the sequence's draws; may equal rng_in only if rows_per_seq == 1 */

    int32_t *tokens;     /* [n_seq * rows_per_seq] */
    int32_t *row_status; /* [n_seq * rows_per_seq] */

    float *out_logits; /* optional [rows, n_vocab]: rows after penalties */

    int32_t  kept_cap; /* 0 = off; else entries per row below */
    int32_t *kept_n;   /* [rows] size of the kept set (k, nucleus size, 0 for argmax/temperature) */
    int32_t *kept_idx; /* [rows, kept_cap] ids in walk order */
    float   *kept_prob; /* [rows, kept_cap] probability renormalised inside the kept set */

    int32_t vocab_offset; /* id of column 0; added to every id written, subtracted from history ids */

    /* Final-logit soft cap (head.c:145-159, :279-288): per sequence or NULL. A row whose sequence has c > 0 and
     * T > 0 is sampled from tanhf(x / c) * c; greedy rows skip it, as the reference does (monotone). Applied to
     * the logits as they stream in, before mask and penalties; out_logits shows the capped values. */
    const float *softcap;

    /* Constrained decoding (EXTENSION): optional [n_seq, logit_mask_stride] 32-bit words in call order; bit i of
     * a sequence's row set = column i may be sampled, clear = the column reads as -inf (after the soft cap,
     * before the penalties). All rows of a sequence share its mask row. */
    const uint32_t *logit_mask;
    size_t          logit_mask_stride; /* words per mask row, >= ceil(n_vocab / 32) */

    /* Which finishing kernel the launch carries: see GEIST_B200_FINISH_* below. 0 = the general one. */
    int32_t finish_hint;
};

/* finish_hint. The stream kernel is followed by ONE finishing kernel: the general one, which carries the code
 * for every kind of row, or a small one for greedy rows and top-k rows with k <= 256 (a tenth of the code,
 * 7 - 8 us less per launch). A caller that knows its sessions' sampler settings says which:
 *   AUTO         the general kernel; any mix of rows.
 *   GREEDY_TOPK  the small kernel; or none at all: where the launch deals whole rows to its thread blocks
 *                (batches of about half the device's thread-block slots and more, no kept-set output) the
 *                stream kernel finishes the rows itself. A row that is neither greedy nor top-k <= 256 is not
 *                sampled: its row_status carries GEIST_B200_ROW_INTERNAL and its token is -1. A top-k row whose
 *                candidates do not fit the lists of this path (thousands of equal values at the top of the
 *                row) is not sampled either and says GEIST_B200_ROW_RETRY: launch its sequence again without
 *                the hint, from the same rng_in (geist_b200_batcher_* do that themselves).
 *   GENERAL      the general kernel, as AUTO; tells the launch that its rows are temperature / top-p rows,
 *                for which another way of dealing the rows out to the thread blocks is faster.
 *   GREEDY       every row is greedy (T <= 0): the stream kernel writes the tokens itself (the thread block that
 *                streamed the whole row, or the last of the row's parts to publish its record) and no finishing
 *                kernel is launched. A row with T > 0 is not sampled: GEIST_B200_ROW_INTERNAL, token -1. */
enum {
    GEIST_B200_FINISH_AUTO        = 0,
    GEIST_B200_FINISH_GREEDY_TOPK = 1,
    GEIST_B200_FINISH_GENERAL     = 2,
    GEIST_B200_FINISH_GREEDY      = 3,
};

/* Replaces the sampler dispatch of finalize_logits_one_row / _batch
 * (head.c:165-186, :289-303) for any number of sessions at once. `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream, as in CUDA). Asynchronous. */
enum geist_status geist_b200_sample_batch(struct geist_b200_ctx *ctx, const struct geist_b200_batch *b, void *stream);

/* Backend operator slot argmax_f32 (include/geist_backend.h:414-421): greedy
 * argmax of one [1, n] F32 row that lives on this device; ties -> lowest index.
 * Synchronous: returns after the 4-byte index is on the host. The glue that
 * unpacks struct geist_tensor is a few lines in the backend that registers the slot. */
enum geist_status geist_b200_argmax_f32(struct geist_b200_ctx *ctx, const float *logits_dev, size_t n, int32_t *out_index);
/* The matching probe (geist_backend.h:276-326): true for q->op == ARGMAX_F32, m == 1, 1 <= d_model <= supported max. */
int geist_b200_argmax_f32_supported(size_t m, size_t n_vocab);

/* Speculative accept rule, session.c:599-625, batched: for each sequence,
 * accepted = longest run of i < k-1 with verify_out[i] == fed[i+1]; emitted =
 * fed[0..accepted] + verify_out[accepted] (accepted + 2 tokens, the last one is
 * the bonus token when everything matched). Device pointers; emitted is
 * [n_seq, k+1], unused tail = -1. */
enum geist_status geist_b200_accept_batch(struct geist_b200_ctx *ctx, size_t n_seq, size_t k, const int32_t *fed,
                                          const int32_t *verify_out, int32_t *accepted, int32_t *n_emitted,
                                          int32_t *emitted, void *stream);

/* Dense inspection outputs (device pointers). */
/* probs[r, :] = softmax(logits[r, :] / T_r) as the top-p path forms it (sampler.c:68-85, :253-255). */
enum geist_status geist_b200_softmax(struct geist_b200_ctx *ctx, const float *logits, size_t row_stride, size_t n_rows,
                                     size_t n_vocab, const float *temperature, float *probs, double *sums, void *stream);
/* dense[r, :] = 0 except the kept entries: the "post-filter probability vector". */
enum geist_status geist_b200_scatter_kept(struct geist_b200_ctx *ctx, size_t n_rows, size_t n_vocab, int32_t kept_cap,
                                          const int32_t *kept_n, const int32_t *kept_idx, const float *kept_prob,
                                          int32_t vocab_offset, float *dense, void *stream);

/* Vocabulary shards (EXTENSION). Phase 1 on every rank: the shard's best
 * min(top_k, n_vocab) candidates per row as (raw value, global id) into
 * kept_prob / kept_idx (any order), kept_n = their number; penalties apply to
 * the ids of this shard. The caller all-gathers the three arrays (NCCL) into
 * [n_shards, n_rows, kept_cap] buffers. Phase 2: merge + top-k draw. */
enum geist_status geist_b200_shard_select(struct geist_b200_ctx *ctx, const struct geist_b200_batch *b, void *stream);

struct geist_b200_merge {
    const float   *cand_val; /* [n_shards, n_rows, cand_stride] */
    const int32_t *cand_gid; /* [n_shards, n_rows, cand_stride] */
    const int32_t *cand_n;   /* [n_shards, n_rows] */
    size_t         n_shards, n_rows, cand_stride;
    const float   *temperature; /* [n_rows] */
    const int32_t *top_k;       /* [n_rows] */
    const uint64_t *rng_in;     /* [n_rows] */
    uint64_t       *rng_out;    /* [n_rows] */
    int32_t        *tokens;     /* [n_rows] */
    int32_t        *row_status; /* [n_rows] */
    int32_t         kept_cap;
    int32_t        *kept_n, *kept_idx;
    float          *kept_prob;
};
enum geist_status geist_b200_shard_merge_sample(struct geist_b200_ctx *ctx, const struct geist_b200_merge *m, void *stream);

/* ----------------------------- 3. sessions, verify/accept, the batcher -- */

#ifndef GEIST_H
enum geist_kv_mode { GEIST_KV_AUTO = 0, GEIST_KV_FP32, GEIST_KV_INT8, GEIST_KV_KIVI, GEIST_KV_F16, GEIST_KV_INT4 };
/* Field for field include/geist.h:209-247; only the four sampler fields are read here. */
struct geist_session_opts {
    size_t             max_seq_len;
    float              temperature;
    float              top_p;
    int                top_k;
    uint64_t           random_seed;
    const char        *awq_scales_path;
    enum geist_kv_mode kv_mode;
    size_t             m_max;
};
#endif

/* EXTENSION, separate from geist_session_opts so that struct keeps its layout; all zero = off. */
struct geist_b200_penalty_opts {
    float repetition_penalty; /* <= 0 reads as 1 */
    float frequency_penalty;
    float presence_penalty;
};

#define GEIST_B200_SPEC_KMAX 16 /* GEIST_SPEC_KMAX_HARDCAP, session.c:515 */

struct geist_b200_batcher; /* N sessions -> one launch */

/* max_history: ids kept per session for the penalties (0 = none kept). */
enum geist_status geist_b200_batcher_create(struct geist_b200_ctx *ctx, size_t n_vocab, size_t max_sessions,
                                            size_t max_history, struct geist_b200_batcher **out);
void              geist_b200_batcher_destroy(struct geist_b200_batcher *b);

/* Sampler half of geist_session_create (geist.h:252-255): defaults T=0, top_p=1,
 * top_k=0, seed 0xCAFEBABE1234 (arch_state.c:1168-1173); then opts applied as
 * transformer_session_apply_opts does: top_p <= 0 -> 1.0, random_seed 0 keeps
 * the default stream (step.c:385-411). opts / pen may be NULL. */
enum geist_status geist_b200_session_open(struct geist_b200_batcher *b, const struct geist_session_opts *opts,
                                          const struct geist_b200_penalty_opts *pen, int32_t *out_session);
enum geist_status geist_b200_session_close(struct geist_b200_batcher *b, int32_t session);
/* geist_session_reset (geist.h:262): forget the history, keep sampler config and generator. */
enum geist_status geist_b200_session_reset(struct geist_b200_batcher *b, int32_t session);
/* Tokens committed to the context (prompt, or tokens emitted elsewhere). */
enum geist_status geist_b200_session_push_history(struct geist_b200_batcher *b, int32_t session, size_t n,
                                                  const geist_token_t *ids);
/* The generator word (checkpoint / resume of a sampled stream). */
enum geist_status geist_b200_session_get_rng(struct geist_b200_batcher *b, int32_t session, uint64_t *state);
enum geist_status geist_b200_session_set_rng(struct geist_b200_batcher *b, int32_t session, uint64_t state);

/* Sampler half of one decode step for n sessions at once (finalize_logits_one_row,
 * head.c:165-186, for each). logits [n, n_vocab] is a DEVICE pointer unless
 * logits_on_host != 0, in which case it is a host buffer that is copied in
 * inside the call. out_tokens is a HOST array. Each session's generator
 * advances and, when append_history != 0, its sampled token joins its history.
 * Synchronous. */
enum geist_status geist_b200_batcher_step(struct geist_b200_batcher *b, size_t n, const int32_t *sessions,
                                          const float *logits, size_t row_stride, int logits_on_host,
                                          int append_history, geist_token_t *out_tokens);

/* Sampler + accept half of geist_session_decode_speculative (session.c:593-636)
 * for n sessions: logits [n, k, n_vocab] are the verify pass's rows, fed [n, k]
 * the tokens pushed through it (fed[.][0] = pending token, the rest proposals;
 * HOST array). All k rows are sampled in order with the session's generator,
 * then the prefix-accept rule runs. Outputs (HOST): accepted [n], n_out [n],
 * out_tokens [n, k+1]. 1 <= k <= GEIST_B200_SPEC_KMAX. The emitted tokens join
 * the history when append_history != 0. The caller then feeds the last emitted
 * token back (the "correction prefill" of session.c:627-634) and calls
 * geist_b200_batcher_step for its logits. */
enum geist_status geist_b200_batcher_verify(struct geist_b200_batcher *b, size_t n, const int32_t *sessions, size_t k,
                                            const geist_token_t *fed, const float *logits, size_t row_stride,
                                            int logits_on_host, int append_history, int32_t *accepted,
                                            int32_t *n_out, geist_token_t *out_tokens);

/* ---- pending token (arch.c:133-161) ------------------------------------------
 * A session holds the token its last sampled row predicted until somebody hands it out:
 * geist_b200_batcher_step samples a row and makes the token pending (and returns it);
 * geist_b200_batcher_decode_step is op_decode_step's cadence, batched: it returns each session's
 * pending token and makes the token sampled from `logits` (the model's output for that pending
 * token) the new pending one; GEIST_E_INVALID_STATE, with nothing changed, when a session has
 * none pending. geist_b200_batcher_verify takes fed[i][0] from the session when the caller
 * writes a negative id there (same error when nothing is pending) and leaves the session without
 * a pending token: the last emitted one still has to go through the model. */
enum geist_status geist_b200_batcher_decode_step(struct geist_b200_batcher *b, size_t n, const int32_t *sessions,
                                                 const float *logits, size_t row_stride, int logits_on_host,
                                                 int append_history, geist_token_t *out_tokens);
/* op_peek_next_token (arch.c:155-160): the pending token, -1 when there is none. */
geist_token_t geist_b200_session_peek_next_token(struct geist_b200_batcher *b, int32_t session);

/* geist_session_peek_logits (geist_util.h:195-211; arch.c:163-195): the logits row the pending token
 * was sampled from, as a HOST copy that belongs to the session and stays valid until the session's
 * next sampling call; the model's soft cap (below) is applied, penalties and mask are not. NULL and
 * *n_logits = 0 when nothing is pending. The row is read where it lay when it was sampled: device
 * logits passed to the batcher must still be alive and unchanged; host logits are read from the
 * batcher's own staging copy, which lives until its next call with host logits. */
const float *geist_b200_session_peek_logits(struct geist_b200_batcher *b, int32_t session, size_t *n_logits);

/* The final-logit soft cap of the session's model (config.logit_softcap, head.c:145-159); 0 = none. */
enum geist_status geist_b200_session_set_softcap(struct geist_b200_batcher *b, int32_t session, float softcap);
/* Constrained decoding (EXTENSION): bit i of `allowed` set = column i may be sampled; n_words >=
 * ceil(n_vocab / 32); NULL lifts the mask. HOST array, copied. Holds until it is replaced or lifted. */
enum geist_status geist_b200_session_set_logit_mask(struct geist_b200_batcher *b, int32_t session, const uint32_t *allowed,
                                                    size_t n_words);

/* ---- n-gram drafter (session.c:437-513) -----------------------------------------
 * propose_drafts_ngram for n_seq sequences at once, searched on the device: the longest suffix
 * (<= max_suffix, at most 8) of history + [seed] that occurs earlier in the history, the place with
 * the most following tokens, the most recent on ties. HOST arrays: histories [n_seq, history_stride],
 * history_len [n_seq], seeds [n_seq]; out_drafts [n_seq, out_capacity] (drafts[0] = seed, unused
 * tail -1), n_drafts [n_seq] (>= 1), match_L [n_seq] or NULL (0 = no match). As in
 * geist_session_decode_speculative (session.c:540-549): 1 <= k_max <= GEIST_B200_SPEC_KMAX and
 * out_capacity >= k_max + 1, else GEIST_E_INVALID_ARG. Synchronous. */
enum geist_status geist_b200_draft_ngram(struct geist_b200_ctx *ctx, size_t n_seq, const geist_token_t *histories,
                                         size_t history_stride, const int32_t *history_len, const geist_token_t *seeds,
                                         size_t k_max, size_t max_suffix, size_t out_capacity, geist_token_t *out_drafts,
                                         int32_t *n_drafts, int32_t *match_L);
/* The drafting half of geist_session_decode_speculative (session.c:553-591) for n sessions: seed = the
 * session's pending token (GEIST_E_INVALID_STATE when none), context = the session's history ring on
 * the device (its last max_history tokens), max_suffix 4, then the lazy gate: a session whose match is
 * shorter than GEIST_SPEC_MIN_L (environment, default 2, read once) or that found nothing comes back
 * with n_drafts = 1 and decodes one token the plain way. The rows with n_drafts > 1 go through the
 * model's verify pass and geist_b200_batcher_verify. */
enum geist_status geist_b200_batcher_propose_drafts(struct geist_b200_batcher *b, size_t n, const int32_t *sessions,
                                                    size_t k_max, size_t out_capacity, geist_token_t *out_drafts,
                                                    int32_t *n_drafts, int32_t *match_L);

/* Launch-shape report for one vocabulary size on the current device: slices a
 * row is cut into, floats per slice, shared memory per thread block, stages of
 * each warp's bulk-copy ring. GEIST_E_UNSUPPORTED when the row cannot be served. */
enum geist_status geist_b200_plan(size_t n_vocab, size_t max_history, int32_t *slices_per_row, int32_t *slice,
                                  int32_t *smem_bytes, int32_t *ring_stages);

/* How one launch over n_rows rows of this vocabulary is spread over the current device: the number of thread
 * blocks (each takes a contiguous run of (row, slice) items) and how many of them one SM holds at a time. */
enum geist_status geist_b200_grid(size_t n_vocab, size_t max_history, size_t n_rows, int32_t *thread_blocks,
                                  int32_t *blocks_per_sm);

/* Greedy argmax of n_rows rows [n_rows, n_vocab] (device memory, row_stride floats apart)
 * into out_index [n_rows] (device memory), ties -> lowest index, WITHOUT allocating: no
 * context, no cudaMalloc, no growth on larger batches. No counterpart in the reference; it
 * exists for callers that cannot allocate while they decode (an engine whose arena owns
 * the whole device, a loop with a fixed per-token footprint, a thread that must stay off
 * the driver's allocation lock). The scratch is an array built into this library
 * (528 KB per device), so one call takes at most 4096 rows and at most 65536 slices of
 * 8192 floats (rows * ceil(n_vocab / 8192)); beyond that it returns GEIST_E_INVALID_ARG
 * and geist_b200_errmsg() says what would fit. Every call on a device shares that
 * array: calls that overlap in time (different streams or threads) race and must be
 * serialised by the caller. The first call on a device looks the array's address up
 * (set-up; make that call before any stream capture begins) and keeps it for the life of
 * the process: after cudaDeviceReset on that device the entry must not be called again.
 * Asynchronous on `stream` (cudaStream_t as void*, NULL = the legacy default stream): the
 * indices are in DEVICE memory once the stream reaches that point, so a caller that needs
 * one on the host (the synchronous argmax_f32 backend slot does) adds a 4-byte copy and a
 * stream synchronise of its own. The calling thread's current device is the same after the
 * call as before it. */
enum geist_status geist_b200_argmax_rows_static(int device, const float *logits, size_t row_stride, size_t n_rows,
                                                size_t n_vocab, int32_t *out_index, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GEIST_B200_H */

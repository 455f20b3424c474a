/*
 * geist_b200_abi.cu — the C ABI declared in include/geist_b200.h: argument
 * checks, launch planning, the sampler.h host-pointer surface, sessions and
 * the multi-session batcher. All numeric work happens in the kernels of
 * sampler_stream.cu, sampler_aux.cu and sampler_static.cu; nothing here
 * computes a token on the CPU.
 */
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/geist_b200.h"
#include "sampler_params.h"

namespace gb {
size_t      sample_stream_smem(int n_slices, int long_ids);
cudaError_t sample_stream_ctas_per_sm(size_t smem_bytes, int *out);
cudaError_t finish_rows_max_ctas(int sms, int *out);
cudaError_t launch_sample_stream(const SampleParams &p, int grid, size_t smem_bytes, int finish_grid, cudaStream_t stream);
cudaError_t launch_merge_sample(const MergeParams &p, cudaStream_t stream);
cudaError_t launch_accept(const AcceptParams &p, cudaStream_t stream);
cudaError_t launch_scatter_kept(const int *kept_n, const int *kept_idx, const float *kept_val, int kept_cap, int n_rows, int V, int vocab_offset, float *dense, cudaStream_t stream);
cudaError_t launch_softmax_rows(const float *logits, long long row_stride, int n_rows, int V, const float *temperature, float *probs, double *sums, cudaStream_t stream);
int         argmax_rows_static_max_rows(long long n_vocab);
cudaError_t launch_argmax_rows_static(int device, const float *logits, long long row_stride, int n_rows, int V, int *out, cudaStream_t stream, const char **what);
cudaError_t launch_post_step(const int *slot, int n_seq, int per_seq, int first, const int *tokens, const int *counts, int *hist, int hist_cap, int *hist_len, long long *hist_total, const unsigned long long *rng_tmp, unsigned long long *rng, cudaStream_t stream);
cudaError_t launch_draft_ngram(const int *slot, int n_seq, const int *hist, long long stride, const int *hist_len, const long long *hist_total, const int *seeds, const int *skip_last,
                               int k_max, int max_suffix, int min_L, int out_stride, int *drafts, int *n_drafts, int *match_L, cudaStream_t stream);
cudaError_t launch_softcap_row(float *row, int n, float c, cudaStream_t stream);
} /* namespace gb */

/* ------------------------------------------------------------- errors -- */

static thread_local std::string g_err;

static enum geist_status fail(enum geist_status s, const char *fmt, ...) {
    char    buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return s;
}

#define CUDA_TRY(expr)                                                                                   \
    do {                                                                                                 \
        cudaError_t e_ = (expr);                                                                         \
        if (e_ != cudaSuccess) {                                                                         \
            return fail(e_ == cudaErrorMemoryAllocation ? GEIST_E_OOM : GEIST_E_BACKEND, "%s: %s", #expr, \
                        cudaGetErrorString(e_));                                                         \
        }                                                                                                \
    } while (0)

extern "C" const char *geist_b200_errmsg(void) { return g_err.c_str(); }

/* ------------------------------------------------------- launch planning -- */

namespace {

constexpr size_t kSmemMax = 227 * 1024; /* opt-in shared memory per CTA on sm_100 */
constexpr int    kLanes   = 4;          /* launches of one context that may overlap on the GPU */

struct Plan {
    int    n_slices     = 0;
    int    slice        = 0;
    int    row_cap      = 0;
    int    bucket_cap   = 0;
    int    id_slots     = 0;
    int    hist_cap     = 0;
    size_t smem         = 0;
    int    ctas         = 0; /* thread blocks of the stream kernel the device holds at once (its grid never exceeds this) */
    int    fin_ctas     = 0; /* ... and of the finishing kernel */
};

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

/* hist_max = 0: no history pointer will be given. Rows are cut into the fewest slices of at
 * most kSliceMax floats. */
bool make_plan(size_t V, size_t hist_max, Plan &pl) {
    int            dev = 0;
    cudaDeviceProp prop;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
        return false;
    }
    const size_t n_slices = (V + gb::kSliceMax - 1) / gb::kSliceMax;
    const size_t slice    = round_up((V + n_slices - 1) / n_slices, 4);
    if (n_slices > (size_t) gb::kMaxSlices || (n_slices > 1 && (n_slices - 1) * slice >= V)) {
        return false;
    }
    pl.n_slices     = (int) n_slices;
    pl.slice        = (int) slice;
    /* histories of more than kRowIds ids are counted by a kernel of their own, in a shared-memory table with at
     * least two slots per id */
    pl.id_slots     = 0;
    pl.row_cap      = 0;
    pl.bucket_cap   = 0;
    if (hist_max > (size_t) gb::kRowIds) {
        size_t slots = 1024;
        while (slots < 2 * hist_max) {
            slots *= 2;
        }
        if (slots > 16384) {
            return false; /* 128 KB of table */
        }
        pl.id_slots   = (int) slots;
        pl.row_cap    = (int) round_up(hist_max, 4);
        pl.bucket_cap = (int) round_up(n_slices + 1, 4);
    }
    pl.hist_cap = hist_max ? (int) round_up(std::min<size_t>(hist_max, 1024), 4) : 0; /* the finisher walks segments of at most 1024 ids */
    pl.smem     = gb::sample_stream_smem(pl.n_slices, pl.id_slots > 0 ? 1 : 0);
    if (pl.smem > kSmemMax) {
        return false;
    }
    int per_sm = 0;
    if (gb::sample_stream_ctas_per_sm(pl.smem, &per_sm) != cudaSuccess || per_sm < 1) {
        return false;
    }
    pl.ctas = per_sm * prop.multiProcessorCount;
    if (gb::finish_rows_max_ctas(prop.multiProcessorCount, &pl.fin_ctas) != cudaSuccess || pl.fin_ctas < 1) {
        return false;
    }
    return true;
}

/* How a launch's (row, slice) items are dealt out to the stream kernel's thread blocks (gb::RunMap), the grid that
 * goes with it, and over how many thread blocks a row can be spread. A thread block's cost is taken as its items
 * plus kPartCost items' worth for every part of a row it touches (set-up, the first slice's threshold, the
 * record): five where rows may be top-k rows (measured: 256 whole rows beat 296 equal runs by 5 us of 51), one
 * where the caller said they are temperature / top-p rows (their parts set no threshold; equal runs measured
 * 6 - 10 % faster there), eight where the caller said they are greedy (whole rows need no finishing kernel). */
struct Deal {
    gb::RunMap map;
    int        grid;
    int        parts_max;
};
Deal deal_items(size_t n_rows, int n_slices, int ctas, size_t kPartCost = 5) {
    const size_t S = (size_t) n_slices, n_items = n_rows * S;
    /* equal runs of items */
    Deal         a;
    a.grid                = (int) std::min<size_t>((size_t) ctas, n_items);
    const size_t q        = n_items / (size_t) a.grid, rem = n_items % (size_t) a.grid;
    a.map                 = gb::RunMap{gb::RUN_ITEMS, (int) q, (int) rem, 1};
    a.parts_max           = (int) std::min<size_t>(S, (S - 1 + q - 1) / q + 1);
    const size_t a_items  = q + (rem ? 1 : 0);
    const size_t a_cost   = a_items + kPartCost * std::min<size_t>((a_items - 1 + S - 1) / S + 1, a_items);
    /* rows kept whole, or cut into equal parts */
    Deal   b;
    size_t b_cost;
    const size_t P = n_rows < (size_t) ctas ? std::min<size_t>((size_t) ctas / n_rows, S) : 1;
    if (P <= 1) {
        b.grid               = (int) std::min<size_t>((size_t) ctas, n_rows);
        const size_t qr      = n_rows / (size_t) b.grid, rr = n_rows % (size_t) b.grid;
        b.map                = gb::RunMap{gb::RUN_ROWS, (int) qr, (int) rr, 1};
        b.parts_max          = 1;
        const size_t rows_mx = qr + (rr ? 1 : 0);
        b_cost               = rows_mx * (S + kPartCost);
    } else {
        b.grid      = (int) (n_rows * P);
        b.map       = gb::RunMap{gb::RUN_PARTS, (int) (S / P), (int) (S % P), (int) P};
        b.parts_max = (int) P;
        b_cost      = S / P + (S % P ? 1 : 0) + kPartCost;
    }
    return b_cost <= a_cost ? b : a;
}

struct PlanCache {
    std::mutex mu;
    struct Key {
        int    dev;
        size_t V, H;
    };
    std::vector<std::pair<Key, Plan>> items;

    bool get(size_t V, size_t H, Plan &pl) {
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lk(mu);
        for (auto &it : items) {
            if (it.first.dev == dev && it.first.V == V && it.first.H == H) {
                pl = it.second;
                return pl.n_slices > 0;
            }
        }
        Plan p;
        bool ok = make_plan(V, H, p);
        if (!ok) {
            p = Plan();
        }
        items.push_back({{dev, V, H}, p});
        pl = p;
        return ok;
    }
} g_plans;

cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

} /* namespace */

/* ------------------------------------------------------------- context -- */

struct geist_b200_ctx {
    int          device = 0;
    cudaStream_t stream = nullptr;
    /* scratch of the host-pointer surface: one row + a handful of words */
    float *d_row     = nullptr;
    size_t d_row_cap = 0;
    struct Small {
        float              T;
        int                top_k;
        float              top_p;
        int                token;
        int                status;
        int                pad;
        unsigned long long rng_in;
        unsigned long long rng_out;
    };
    Small *d_small = nullptr;
    Small *h_small = nullptr; /* pinned */
    std::mutex small_mu;      /* one synchronous host-pointer call at a time stages through the two words above */

    /* kernel scratch: part records, candidate groups, segment sums, row counters, multi-pass row copies. kLanes
     * independent sets, used round-robin, so that up to kLanes launches may overlap on the GPU. */
    struct Lane {
        unsigned char *buf         = nullptr;
        size_t         bytes       = 0;
        int           *counters    = nullptr; /* one flag per row copy of the multi-pass path */
        int           *arrive      = nullptr; /* one counter per row: parts that have published (greedy launches); zero between launches */
        size_t         arrive_cap  = 0;
        size_t         counter_cap = 0;
    } lane[kLanes];
    unsigned   next_lane = 0;
    std::mutex lane_mu;
};

extern "C" enum geist_status geist_b200_ctx_create(int device, struct geist_b200_ctx **out) {
    if (out == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "ctx_create: out is NULL");
    }
    *out = nullptr;
    int n = 0;
    CUDA_TRY(cudaGetDeviceCount(&n));
    if (device < 0 || device >= n) {
        return fail(GEIST_E_INVALID_ARG, "ctx_create: device %d of %d", device, n);
    }
    CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        return fail(GEIST_E_UNSUPPORTED, "ctx_create: device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    }
    geist_b200_ctx *c = new (std::nothrow) geist_b200_ctx();
    if (c == nullptr) {
        return fail(GEIST_E_OOM, "ctx_create: host allocation");
    }
    c->device = device;
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) {
        e = cudaMalloc(&c->d_small, sizeof(geist_b200_ctx::Small));
    }
    if (e == cudaSuccess) {
        e = cudaHostAlloc(&c->h_small, sizeof(geist_b200_ctx::Small), cudaHostAllocDefault);
    }
    if (e != cudaSuccess) {
        geist_b200_ctx_destroy(c);
        return fail(GEIST_E_BACKEND, "ctx_create: %s", cudaGetErrorString(e));
    }
    *out = c;
    return GEIST_OK;
}

extern "C" void geist_b200_ctx_destroy(struct geist_b200_ctx *c) {
    if (c == nullptr) {
        return;
    }
    cudaSetDevice(c->device);
    if (c->stream) {
        cudaStreamSynchronize(c->stream);
    }
    for (auto &ln : c->lane) {
        cudaFree(ln.buf);
        cudaFree(ln.counters);
        cudaFree(ln.arrive);
    }
    cudaFree(c->d_row);
    cudaFree(c->d_small);
    cudaFreeHost(c->h_small);
    if (c->stream) {
        cudaStreamDestroy(c->stream);
    }
    delete c;
}

/* ------------------------------------------------------- batched entries -- */

static enum geist_status launch_batch(struct geist_b200_ctx *ctx, const struct geist_b200_batch *b, void *stream, unsigned flags) {
    if (ctx == nullptr || b == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: NULL context or batch");
    }
    if (b->logits == nullptr || b->tokens == nullptr || b->row_status == nullptr || b->temperature == nullptr || b->top_k == nullptr || b->top_p == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: logits, tokens, row_status, temperature, top_k, top_p are required");
    }
    if (b->n_seq == 0 || b->rows_per_seq == 0 || b->n_vocab == 0) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: n_seq, rows_per_seq and n_vocab must be positive");
    }
    if (b->n_vocab > 0x7fffffffu || b->n_seq * b->rows_per_seq > (size_t) 0x7fffffff / gb::kMaxSlices) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: sizes exceed int32 ids / grid limits");
    }
    if (b->row_stride < b->n_vocab) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: row_stride %zu < n_vocab %zu", b->row_stride, b->n_vocab);
    }
    if (b->rows_per_seq > 1 && b->rng_out != nullptr && (const void *) b->rng_out == (const void *) b->rng_in) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: rng_out may alias rng_in only when rows_per_seq == 1");
    }
    if (b->history != nullptr && (b->history_len == nullptr || b->history_stride == 0)) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: history needs history_len and history_stride");
    }
    if (b->fed_tokens != nullptr && b->fed_stride < b->rows_per_seq) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: fed_stride %zu < rows_per_seq %zu", b->fed_stride, b->rows_per_seq);
    }
    if (b->kept_cap < 0 || (b->kept_cap > 0 && (b->kept_n == nullptr || b->kept_idx == nullptr || b->kept_prob == nullptr))) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: kept_cap > 0 needs kept_n, kept_idx and kept_prob");
    }
    if (b->logit_mask != nullptr && b->logit_mask_stride * 32 < b->n_vocab) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: logit_mask_stride %zu words hold fewer than n_vocab %zu bits", b->logit_mask_stride, b->n_vocab);
    }
    if (b->finish_hint < GEIST_B200_FINISH_AUTO || b->finish_hint > GEIST_B200_FINISH_GREEDY) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: finish_hint %d is not one of GEIST_B200_FINISH_*", b->finish_hint);
    }
    if ((flags & gb::F_SELECT_ONLY) && b->kept_cap <= 0) {
        return fail(GEIST_E_INVALID_ARG, "shard_select: kept_cap must hold the shard's candidates");
    }
    CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t hist_max = (b->history || b->fed_tokens) ? (b->history ? b->history_stride : 0) + (b->fed_tokens ? b->rows_per_seq : 0) : 0;
    Plan         pl;
    if (!g_plans.get(b->n_vocab, hist_max, pl)) {
        return fail(GEIST_E_UNSUPPORTED, "sample_batch: no launch shape for n_vocab=%zu with %zu history ids per row (shared memory)", b->n_vocab, hist_max);
    }
    gb::SampleParams p{};
    p.logits       = b->logits;
    p.row_stride   = (long long) b->row_stride;
    p.V            = (int) b->n_vocab;
    p.n_rows       = (int) (b->n_seq * b->rows_per_seq);
    p.rows_per_seq = (int) b->rows_per_seq;
    p.vocab_offset = b->vocab_offset;
    p.slot         = b->slot;
    p.temperature  = b->temperature;
    p.top_k        = b->top_k;
    p.top_p        = b->top_p;
    p.rep          = b->repetition_penalty;
    p.freq         = b->frequency_penalty;
    p.pres         = b->presence_penalty;
    p.softcap      = b->softcap;
    p.mask         = b->logit_mask;
    p.mask_stride  = (long long) b->logit_mask_stride;
    p.hist         = b->history;
    p.hist_stride  = (long long) b->history_stride;
    p.hist_len     = b->history_len;
    p.extra        = b->fed_tokens;
    p.extra_stride = (long long) b->fed_stride;
    p.rng_in       = reinterpret_cast<const unsigned long long *>(b->rng_in);
    p.rng_out      = reinterpret_cast<unsigned long long *>(b->rng_out);
    p.tokens       = b->tokens;
    p.status       = b->row_status;
    p.out_logits   = b->out_logits;
    p.kept_cap     = b->kept_cap;
    p.kept_n       = b->kept_n;
    p.kept_idx     = b->kept_idx;
    p.kept_val     = b->kept_prob;
    p.n_slices     = pl.n_slices;
    p.slice        = pl.slice;
    p.row_cap      = pl.row_cap;
    p.bucket_cap   = pl.bucket_cap;
    p.id_slots     = pl.id_slots;
    p.hist_cap     = pl.hist_cap;
    p.aligned      = ((reinterpret_cast<uintptr_t>(b->logits) & 15u) == 0 && (b->row_stride & 3u) == 0) ? 1 : 0;
    p.flags        = flags;
    if ((flags & gb::F_SELECT_ONLY) == 0u) { /* a shard's select is a top-k row whatever its parameters say: the small kernel takes k <= kFastKMax, the general one the rest */
        p.flags |= b->finish_hint == GEIST_B200_FINISH_GREEDY_TOPK ? gb::F_FAST_ONLY : 0u;
        if (b->finish_hint == GEIST_B200_FINISH_GREEDY) {
            p.flags |= gb::F_FAST_ONLY | gb::F_GREEDY_ONLY; /* where rows are split over thread blocks the small finishing kernel still merges them */
        }
    }
    cudaStream_t st = as_stream(stream);

    /* scratch of this launch */
    const size_t n_rows   = (size_t) p.n_rows;
    const size_t n_items  = n_rows * (size_t) pl.n_slices;
    const size_t part_cost = (flags & gb::F_SELECT_ONLY) ? 5 : (b->finish_hint == GEIST_B200_FINISH_GENERAL ? 1 : (b->finish_hint == GEIST_B200_FINISH_GREEDY ? 8 : 5));
    const Deal   deal     = deal_items(n_rows, pl.n_slices, pl.ctas, part_cost);
    const int    grid     = deal.grid;
    const size_t parts    = (size_t) deal.parts_max;
    p.parts_max           = deal.parts_max;
    p.map                 = deal.map;
    if ((p.flags & gb::F_FAST_ONLY) != 0u && (p.flags & gb::F_GREEDY_ONLY) == 0u && deal.map.mode == gb::RUN_ROWS && b->kept_cap == 0) {
        p.flags |= gb::F_INLINE_TOPK; /* whole rows per thread block: the stream kernel finishes them itself */
    }
    const size_t gen_str  = round_up(b->n_vocab, 4);
    const size_t gen_bmw  = (b->n_vocab + 31) / 32;
    const size_t gen_hcap = hist_max ? std::min(hist_max, b->n_vocab) : 0;
    const size_t off_gv   = 0;
    const size_t off_gb   = round_up(off_gv + n_rows * parts * (size_t) gb::kPartSlots * 16, 256);
    const size_t off_seg  = round_up(off_gb + n_rows * parts * (size_t) gb::kPartSlots * 4, 256);
    const int    fin_grid = (int) std::min<size_t>((size_t) pl.fin_ctas, n_rows);
    const size_t slots    = (size_t) fin_grid; /* row copies of the multi-pass path: one per finishing thread block that can run at a time */
    const size_t off_rows = round_up(off_seg + n_items * (size_t) gb::kWarps * sizeof(gb::SegRec), 256);
    const size_t off_bm   = round_up(off_rows + slots * gen_str * 4, 256);
    const size_t off_dl   = round_up(off_bm + slots * gen_bmw * 4, 256);
    const size_t gen_lcap = std::min<size_t>(b->n_vocab, 16384); /* entries of one histogram bin that the multi-pass path picks out of a row */
    const size_t off_ls   = round_up(off_dl + slots * gen_hcap * sizeof(gb::Pair), 256);
    const size_t off_pl   = round_up(off_ls + slots * gen_lcap * sizeof(gb::Pair), 256);
    const size_t off_po   = round_up(off_pl + (pl.id_slots ? n_rows * (size_t) pl.row_cap * 4 : 0), 256);
    const size_t need     = round_up(off_po + (pl.id_slots ? n_rows * (size_t) (pl.n_slices + 1) * 4 : 0), 256) + 256;
    geist_b200_ctx::Lane *ln;
    {
        std::lock_guard<std::mutex> lk(ctx->lane_mu);
        ln = &ctx->lane[ctx->next_lane++ % kLanes];
        if (ln->bytes < need) {
            cudaFree(ln->buf); /* waits for work that may still use it */
            ln->buf   = nullptr;
            ln->bytes = 0;
            CUDA_TRY(cudaMalloc((void **) &ln->buf, need));
            ln->bytes = need;
        }
        if (ln->counter_cap < slots) {
            cudaFree(ln->counters);
            ln->counters    = nullptr;
            ln->counter_cap = 0;
            const size_t cap = round_up(slots, 1024);
            /* one flag per row copy of the multi-pass path, zero between launches (whoever takes a copy gives it
             * back). Zeroed on the launch's own stream, so the first kernel that uses them comes behind it. */
            CUDA_TRY(cudaMalloc((void **) &ln->counters, cap * sizeof(int)));
            CUDA_TRY(cudaMemsetAsync(ln->counters, 0, cap * sizeof(int), st));
            ln->counter_cap = cap;
        }
        if ((p.flags & gb::F_GREEDY_ONLY) != 0u && ln->arrive_cap < n_rows) {
            cudaFree(ln->arrive);
            ln->arrive     = nullptr;
            ln->arrive_cap = 0;
            const size_t cap = round_up(n_rows, 1024);
            /* zeroed on the launch's own stream; whoever completes a row puts its counter back */
            CUDA_TRY(cudaMalloc((void **) &ln->arrive, cap * sizeof(int)));
            CUDA_TRY(cudaMemsetAsync(ln->arrive, 0, cap * sizeof(int), st));
            ln->arrive_cap = cap;
        }
    }
    p.pool             = ln->counters;
    p.arrive           = ln->arrive;
    p.pool_slots       = (int) slots;
    p.grp_v            = reinterpret_cast<float4 *>(ln->buf + off_gv);
    p.grp_b            = reinterpret_cast<int *>(ln->buf + off_gb);
    p.segs             = reinterpret_cast<gb::SegRec *>(ln->buf + off_seg);
    p.gen_rows         = reinterpret_cast<float *>(ln->buf + off_rows);
    p.gen_stride       = (long long) gen_str;
    p.gen_bitmap       = reinterpret_cast<unsigned *>(ln->buf + off_bm);
    p.gen_bitmap_words = (int) gen_bmw;
    p.gen_dlist        = reinterpret_cast<gb::Pair *>(ln->buf + off_dl);
    p.gen_hist_cap     = (int) gen_hcap;
    p.gen_list         = reinterpret_cast<gb::Pair *>(ln->buf + off_ls);
    p.gen_list_cap     = (int) gen_lcap;
    p.pre_list         = reinterpret_cast<unsigned *>(ln->buf + off_pl);
    p.pre_off          = reinterpret_cast<int *>(ln->buf + off_po);
    CUDA_TRY(gb::launch_sample_stream(p, grid, pl.smem, fin_grid, st));
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_sample_batch(struct geist_b200_ctx *ctx, const struct geist_b200_batch *b, void *stream) {
    if (b != nullptr && (b->rng_in == nullptr || b->rng_out == nullptr)) {
        return fail(GEIST_E_INVALID_ARG, "sample_batch: rng_in and rng_out are required");
    }
    return launch_batch(ctx, b, stream, 0u);
}

extern "C" enum geist_status geist_b200_shard_select(struct geist_b200_ctx *ctx, const struct geist_b200_batch *b, void *stream) {
    if (b != nullptr && b->rows_per_seq != 1) {
        return fail(GEIST_E_INVALID_ARG, "shard_select: rows_per_seq must be 1");
    }
    return launch_batch(ctx, b, stream, gb::F_SELECT_ONLY);
}

extern "C" enum geist_status geist_b200_shard_merge_sample(struct geist_b200_ctx *ctx, const struct geist_b200_merge *m, void *stream) {
    if (ctx == nullptr || m == nullptr || m->cand_val == nullptr || m->cand_gid == nullptr || m->cand_n == nullptr || m->temperature == nullptr || m->top_k == nullptr ||
        m->rng_in == nullptr || m->tokens == nullptr || m->row_status == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "shard_merge_sample: missing pointer");
    }
    if (m->n_shards == 0 || m->n_rows == 0 || m->cand_stride == 0 || m->n_shards * m->cand_stride > 8192) {
        return fail(GEIST_E_INVALID_ARG, "shard_merge_sample: n_shards * cand_stride must be in [1, 8192]");
    }
    if (m->kept_cap > 0 && (m->kept_n == nullptr || m->kept_idx == nullptr || m->kept_prob == nullptr)) {
        return fail(GEIST_E_INVALID_ARG, "shard_merge_sample: kept_cap > 0 needs the kept arrays");
    }
    CUDA_TRY(cudaSetDevice(ctx->device));
    gb::MergeParams p{};
    p.cand_val    = m->cand_val;
    p.cand_gid    = m->cand_gid;
    p.cand_n      = m->cand_n;
    p.n_shards    = (int) m->n_shards;
    p.n_rows      = (int) m->n_rows;
    p.k_stride    = (int) m->cand_stride;
    p.temperature = m->temperature;
    p.top_k       = m->top_k;
    p.rng_in      = reinterpret_cast<const unsigned long long *>(m->rng_in);
    p.rng_out     = reinterpret_cast<unsigned long long *>(m->rng_out);
    p.tokens      = m->tokens;
    p.status      = m->row_status;
    p.kept_cap    = m->kept_cap;
    p.kept_n      = m->kept_n;
    p.kept_idx    = m->kept_idx;
    p.kept_val    = m->kept_prob;
    CUDA_TRY(gb::launch_merge_sample(p, as_stream(stream)));
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_accept_batch(struct geist_b200_ctx *ctx, size_t n_seq, size_t k, const int32_t *fed, const int32_t *verify_out, int32_t *accepted,
                                                     int32_t *n_emitted, int32_t *emitted, void *stream) {
    if (ctx == nullptr || fed == nullptr || verify_out == nullptr || accepted == nullptr || n_emitted == nullptr || emitted == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "accept_batch: missing pointer");
    }
    if (n_seq == 0 || k == 0 || k > GEIST_B200_SPEC_KMAX) {
        return fail(GEIST_E_INVALID_ARG, "accept_batch: need n_seq > 0 and 1 <= k <= %d", GEIST_B200_SPEC_KMAX);
    }
    CUDA_TRY(cudaSetDevice(ctx->device));
    gb::AcceptParams p{fed, verify_out, (int) n_seq, (int) k, accepted, n_emitted, emitted};
    CUDA_TRY(gb::launch_accept(p, as_stream(stream)));
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_softmax(struct geist_b200_ctx *ctx, const float *logits, size_t row_stride, size_t n_rows, size_t n_vocab, const float *temperature,
                                                float *probs, double *sums, void *stream) {
    if (ctx == nullptr || logits == nullptr || temperature == nullptr || probs == nullptr || n_rows == 0 || n_vocab == 0 || n_vocab > 0x7fffffffu || row_stride < n_vocab) {
        return fail(GEIST_E_INVALID_ARG, "softmax: bad argument");
    }
    CUDA_TRY(cudaSetDevice(ctx->device));
    CUDA_TRY(gb::launch_softmax_rows(logits, (long long) row_stride, (int) n_rows, (int) n_vocab, temperature, probs, sums, as_stream(stream)));
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_scatter_kept(struct geist_b200_ctx *ctx, size_t n_rows, size_t n_vocab, int32_t kept_cap, const int32_t *kept_n, const int32_t *kept_idx,
                                                     const float *kept_prob, int32_t vocab_offset, float *dense, void *stream) {
    if (ctx == nullptr || kept_n == nullptr || kept_idx == nullptr || kept_prob == nullptr || dense == nullptr || n_rows == 0 || n_vocab == 0 || kept_cap <= 0) {
        return fail(GEIST_E_INVALID_ARG, "scatter_kept: bad argument");
    }
    CUDA_TRY(cudaSetDevice(ctx->device));
    CUDA_TRY(gb::launch_scatter_kept(kept_n, kept_idx, kept_prob, kept_cap, (int) n_rows, (int) n_vocab, vocab_offset, dense, as_stream(stream)));
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_plan(size_t n_vocab, size_t max_history, int32_t *slices_per_row, int32_t *slice, int32_t *smem_bytes, int32_t *ring_stages) {
    Plan pl;
    if (n_vocab == 0 || !g_plans.get(n_vocab, max_history, pl)) {
        if (slices_per_row) {
            *slices_per_row = 0;
        }
        return fail(GEIST_E_UNSUPPORTED, "plan: no launch shape for n_vocab=%zu, history=%zu", n_vocab, max_history);
    }
    if (slices_per_row) {
        *slices_per_row = pl.n_slices;
    }
    if (slice) {
        *slice = pl.slice;
    }
    if (smem_bytes) {
        *smem_bytes = (int32_t) pl.smem;
    }
    if (ring_stages) {
        *ring_stages = gb::kStages;
    }
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_grid(size_t n_vocab, size_t max_history, size_t n_rows, int32_t *thread_blocks, int32_t *blocks_per_sm) {
    Plan pl;
    if (n_vocab == 0 || n_rows == 0 || !g_plans.get(n_vocab, max_history, pl)) {
        return fail(GEIST_E_UNSUPPORTED, "grid: no launch shape for n_vocab=%zu, history=%zu", n_vocab, max_history);
    }
    int            dev = 0;
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
    if (thread_blocks) {
        *thread_blocks = (int32_t) deal_items(n_rows, pl.n_slices, pl.ctas).grid;
    }
    if (blocks_per_sm) {
        *blocks_per_sm = pl.ctas / prop.multiProcessorCount;
    }
    return GEIST_OK;
}

/* -------------------------------------------- sampler.h host-pointer surface -- */

extern "C" void geist_rng_seed(struct geist_rng *rng, uint64_t seed) {
    if (rng != nullptr) {
        rng->state = seed != 0 ? seed : 0x9E3779B97F4A7C15ULL; /* the all-zero state is a fixed point */
    }
}

extern "C" uint64_t geist_rng_next_u64(struct geist_rng *rng) {
    uint64_t s = rng->state;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    rng->state = s;
    return s * 0x2545F4914F6CDD1DULL;
}

extern "C" float geist_rng_next_unit(struct geist_rng *rng) { return (float) (uint32_t) (geist_rng_next_u64(rng) >> 40) * (1.0f / 16777216.0f); }

namespace {

std::mutex      g_default_mu;
geist_b200_ctx *g_default_ctx[64] = {nullptr};

geist_b200_ctx *default_ctx() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        fail(GEIST_E_BACKEND, "no CUDA device is current");
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_default_mu);
    if (g_default_ctx[dev] == nullptr) {
        if (geist_b200_ctx_create(dev, &g_default_ctx[dev]) != GEIST_OK) {
            return nullptr;
        }
    }
    return g_default_ctx[dev];
}

/* One host row through the batched kernel. staging: optional pinned buffer of n floats. */
geist_token_t sample_host_row(size_t n, const float *logits, float *staging, float T, int top_k, float top_p, struct geist_rng *rng) {
    if (n == 0 || logits == nullptr) {
        fail(GEIST_E_INVALID_ARG, "sampler: empty row");
        return -1;
    }
    geist_b200_ctx *c = default_ctx();
    if (c == nullptr) {
        return -1;
    }
    static std::mutex           mu; /* the default context's scratch is shared */
    std::lock_guard<std::mutex> lk(mu);
    cudaError_t                 e = cudaSetDevice(c->device);
    if (e == cudaSuccess && c->d_row_cap < n) {
        cudaFree(c->d_row);
        c->d_row     = nullptr;
        c->d_row_cap = 0;
        e            = cudaMalloc(&c->d_row, n * sizeof(float));
        if (e == cudaSuccess) {
            c->d_row_cap = n;
        }
    }
    if (e == cudaSuccess) {
        const float *src = logits;
        if (staging != nullptr) {
            memcpy(staging, logits, n * sizeof(float));
            src = staging;
        }
        e = cudaMemcpyAsync(c->d_row, src, n * sizeof(float), cudaMemcpyHostToDevice, c->stream);
    }
    if (e != cudaSuccess) {
        fail(GEIST_E_BACKEND, "sampler: staging the row: %s", cudaGetErrorString(e));
        return -1;
    }
    geist_b200_ctx::Small *h = c->h_small;
    h->T                     = T;
    h->top_k                 = top_k;
    h->top_p                 = top_p;
    h->token                 = -1;
    h->status                = 0;
    h->rng_in                = rng ? rng->state : 1ull;
    h->rng_out               = h->rng_in;
    e                        = cudaMemcpyAsync(c->d_small, h, sizeof *h, cudaMemcpyHostToDevice, c->stream);
    if (e != cudaSuccess) {
        fail(GEIST_E_BACKEND, "sampler: %s", cudaGetErrorString(e));
        return -1;
    }
    geist_b200_batch b{};
    b.logits       = c->d_row;
    b.row_stride   = n;
    b.n_seq        = 1;
    b.rows_per_seq = 1;
    b.n_vocab      = n;
    b.temperature  = &c->d_small->T;
    b.top_k        = &c->d_small->top_k;
    b.top_p        = &c->d_small->top_p;
    b.rng_in       = reinterpret_cast<const uint64_t *>(&c->d_small->rng_in);
    b.rng_out      = reinterpret_cast<uint64_t *>(&c->d_small->rng_out);
    b.tokens       = &c->d_small->token;
    b.row_status   = &c->d_small->status;
    if (geist_b200_sample_batch(c, &b, c->stream) != GEIST_OK) {
        return -1;
    }
    e = cudaMemcpyAsync(h, c->d_small, sizeof *h, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(c->stream);
    }
    if (e != cudaSuccess) {
        fail(GEIST_E_BACKEND, "sampler: %s", cudaGetErrorString(e));
        return -1;
    }
    if (h->status & (GEIST_B200_ROW_LOAD_TIMEOUT | GEIST_B200_ROW_HIST_OVERFLOW | GEIST_B200_ROW_INTERNAL)) {
        fail(GEIST_E_BACKEND, "sampler: kernel reported row status 0x%x", h->status);
        return -1;
    }
    if (rng != nullptr) {
        rng->state = h->rng_out;
    }
    return h->token;
}

} /* namespace */

extern "C" geist_token_t geist_sampler_argmax(size_t n_vocab, const float *logits) { return sample_host_row(n_vocab, logits, nullptr, 0.0f, 0, 1.0f, nullptr); }

extern "C" geist_token_t geist_sampler_temperature(size_t n_vocab, const float *logits, float temperature, struct geist_rng *rng) {
    return sample_host_row(n_vocab, logits, nullptr, temperature, 0, 1.0f, rng); /* T <= 0 -> argmax inside */
}

extern "C" enum geist_status geist_sampler_workspace_init(struct geist_sampler_workspace *ws, size_t n_vocab) {
    if (ws == nullptr || n_vocab == 0) {
        return fail(GEIST_E_INVALID_ARG, "workspace_init: NULL workspace or n_vocab == 0");
    }
    ws->probs   = nullptr;
    ws->n_vocab = 0;
    if (default_ctx() == nullptr) {
        return GEIST_E_BACKEND;
    }
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void **>(&ws->probs), n_vocab * sizeof(float), cudaHostAllocDefault);
    if (e != cudaSuccess) {
        ws->probs = nullptr;
        return fail(GEIST_E_OOM, "workspace_init: pinned staging: %s", cudaGetErrorString(e));
    }
    ws->n_vocab = n_vocab;
    return GEIST_OK;
}

extern "C" void geist_sampler_workspace_destroy(struct geist_sampler_workspace *ws) {
    if (ws == nullptr) {
        return;
    }
    if (ws->probs != nullptr) {
        cudaFreeHost(ws->probs);
        ws->probs = nullptr;
    }
    ws->n_vocab = 0;
}

extern "C" geist_token_t geist_sampler_top_k_ws(struct geist_sampler_workspace *ws, const float *logits, int top_k, float temperature, struct geist_rng *rng) {
    if (ws == nullptr || ws->n_vocab == 0) {
        fail(GEIST_E_INVALID_ARG, "top_k_ws: workspace not initialised");
        return -1;
    }
    if (top_k <= 1 || !(temperature > 0.0f)) { /* sampler.c:184-186: greedy, no draw */
        return sample_host_row(ws->n_vocab, logits, ws->probs, 0.0f, 0, 1.0f, nullptr);
    }
    return sample_host_row(ws->n_vocab, logits, ws->probs, temperature, top_k, 1.0f, rng);
}

extern "C" geist_token_t geist_sampler_top_p_ws(struct geist_sampler_workspace *ws, const float *logits, float top_p, float temperature, struct geist_rng *rng) {
    if (ws == nullptr || ws->n_vocab == 0) {
        fail(GEIST_E_INVALID_ARG, "top_p_ws: workspace not initialised");
        return -1;
    }
    if (!(top_p > 0.0f) || !(temperature > 0.0f)) { /* sampler.c:238-240: greedy, no draw */
        return sample_host_row(ws->n_vocab, logits, ws->probs, 0.0f, 0, 1.0f, nullptr);
    }
    return sample_host_row(ws->n_vocab, logits, ws->probs, temperature, 0, top_p, rng); /* top_p >= 1 -> temperature inside */
}

extern "C" int geist_b200_argmax_f32_supported(size_t m, size_t n_vocab) {
    if (m != 1 || n_vocab == 0 || n_vocab > 0x7fffffffu) {
        return 0;
    }
    Plan pl;
    return g_plans.get(n_vocab, 0, pl) ? 1 : 0;
}

extern "C" enum geist_status geist_b200_argmax_f32(struct geist_b200_ctx *ctx, const float *logits_dev, size_t n, int32_t *out_index) {
    if (ctx == nullptr || logits_dev == nullptr || out_index == nullptr || n == 0) {
        return fail(GEIST_E_INVALID_ARG, "argmax_f32: bad argument");
    }
    std::lock_guard<std::mutex> lk(ctx->small_mu); /* callers on several threads share the context's staging words */
    CUDA_TRY(cudaSetDevice(ctx->device));
    geist_b200_ctx::Small *h = ctx->h_small;
    memset(h, 0, sizeof *h);
    h->top_p  = 1.0f;
    h->token  = -1;
    h->rng_in = 1;
    CUDA_TRY(cudaMemcpyAsync(ctx->d_small, h, sizeof *h, cudaMemcpyHostToDevice, ctx->stream));
    geist_b200_batch b{};
    b.logits       = logits_dev;
    b.row_stride   = n;
    b.n_seq        = 1;
    b.rows_per_seq = 1;
    b.n_vocab      = n;
    b.temperature  = &ctx->d_small->T;
    b.top_k        = &ctx->d_small->top_k;
    b.top_p        = &ctx->d_small->top_p;
    b.rng_in       = reinterpret_cast<const uint64_t *>(&ctx->d_small->rng_in);
    b.rng_out      = reinterpret_cast<uint64_t *>(&ctx->d_small->rng_out);
    b.tokens       = &ctx->d_small->token;
    b.row_status   = &ctx->d_small->status;
    enum geist_status s = geist_b200_sample_batch(ctx, &b, ctx->stream);
    if (s != GEIST_OK) {
        return s;
    }
    CUDA_TRY(cudaMemcpyAsync(h, ctx->d_small, sizeof *h, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if ((h->status & ~(GEIST_B200_ROW_SLOW_PATH | GEIST_B200_ROW_KEPT_PARTIAL)) != 0 || h->token < 0 || (size_t) h->token >= n) {
        return fail(GEIST_E_BACKEND, "argmax_f32: row status 0x%x, index %d", h->status, h->token);
    }
    *out_index = h->token;
    return GEIST_OK;
}

/* ------------------------------------------------- sessions and the batcher -- */

struct geist_b200_batcher {
    geist_b200_ctx *ctx          = nullptr;
    size_t          V            = 0;
    size_t          max_sessions = 0;
    size_t          max_history  = 0;
    std::mutex      mu; /* open/close/push/get/set are setup-time calls; step/verify take it too */

    /* per-slot device state (what arch_state.h:287-294 keeps per session) */
    float              *d_T = nullptr, *d_P = nullptr, *d_rep = nullptr, *d_freq = nullptr, *d_pres = nullptr;
    int                *d_K        = nullptr;
    unsigned long long *d_rng      = nullptr;
    unsigned long long *d_rng_tmp  = nullptr;
    int                *d_hist     = nullptr; /* [max_sessions, max_history] ring */
    int                *d_hist_len = nullptr;
    long long          *d_hist_tot = nullptr;

    /* per-call device scratch, sized for max_sessions * GEIST_B200_SPEC_KMAX rows */
    int   *d_slot = nullptr, *d_tokens = nullptr, *d_status = nullptr, *d_fed = nullptr;
    int   *d_accepted = nullptr, *d_nemit = nullptr, *d_emitted = nullptr, *d_ones = nullptr;
    float *d_logits     = nullptr; /* staging for host logits, grown on demand */
    size_t d_logits_cap = 0;
    int   *h_pin        = nullptr; /* pinned: slots | fed | tokens | status | accepted | nemit | emitted */
    size_t h_pin_ints   = 0;

    cudaStream_t copy_stream[2] = {nullptr, nullptr};
    cudaEvent_t  ev[2]          = {nullptr, nullptr};

    std::vector<char> used;
    std::vector<char> pen_active;
    size_t            n_pen_active = 0;

    /* host mirrors of what the slots hold, for decisions that need no device round trip */
    std::vector<float> h_T, h_P, h_cap;
    std::vector<int>   h_K;
    size_t             n_cap_active = 0;
    /* the pending token of a session (arch.c:133-161): what its last sampled row predicted, not yet handed out */
    std::vector<int>  pending;          /* -1: none */
    std::vector<char> pending_in_hist;  /* the sampler appended it to the history ring when it was drawn */
    int              *d_pending = nullptr;
    float            *d_cap     = nullptr;
    /* allowed-column masks, one row per slot, all ones until a session sets one */
    uint32_t         *d_mask       = nullptr;
    size_t            mask_words   = 0;
    std::vector<char> mask_active;
    size_t            n_mask_active = 0;
    /* where the logits row that a session was last sampled from lies (peek_logits) */
    struct LastRow {
        const float *ptr     = nullptr; /* device pointer of the row */
        bool         valid   = false;
    };
    std::vector<LastRow>            last_row;
    std::vector<std::vector<float>> peek_stage; /* session-owned host copies, filled on demand */
    float                          *d_peek = nullptr;
    /* drafter scratch */
    int *d_drafts = nullptr, *d_ndrafts = nullptr, *d_matchL = nullptr, *d_skip = nullptr;
};

extern "C" void geist_b200_batcher_destroy(struct geist_b200_batcher *b) {
    if (b == nullptr) {
        return;
    }
    cudaSetDevice(b->ctx->device);
    cudaDeviceSynchronize();
    void *dev[] = {b->d_T, b->d_P, b->d_rep, b->d_freq, b->d_pres, b->d_K, b->d_rng, b->d_rng_tmp, b->d_hist, b->d_hist_len, b->d_hist_tot, b->d_slot, b->d_tokens,
                   b->d_status, b->d_fed, b->d_accepted, b->d_nemit, b->d_emitted, b->d_ones, b->d_logits, b->d_pending, b->d_cap, b->d_mask, b->d_peek,
                   b->d_drafts, b->d_ndrafts, b->d_matchL, b->d_skip};
    for (void *p : dev) {
        cudaFree(p);
    }
    cudaFreeHost(b->h_pin);
    for (int i = 0; i < 2; i++) {
        if (b->copy_stream[i]) {
            cudaStreamDestroy(b->copy_stream[i]);
        }
        if (b->ev[i]) {
            cudaEventDestroy(b->ev[i]);
        }
    }
    delete b;
}

extern "C" enum geist_status geist_b200_batcher_create(struct geist_b200_ctx *ctx, size_t n_vocab, size_t max_sessions, size_t max_history, struct geist_b200_batcher **out) {
    if (out == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "batcher_create: out is NULL");
    }
    *out = nullptr;
    if (ctx == nullptr || n_vocab == 0 || n_vocab > 0x7fffffffu || max_sessions == 0 || max_sessions > (1u << 20)) {
        return fail(GEIST_E_INVALID_ARG, "batcher_create: bad argument");
    }
    CUDA_TRY(cudaSetDevice(ctx->device));
    Plan pl;
    if (!g_plans.get(n_vocab, max_history ? max_history + GEIST_B200_SPEC_KMAX : 0, pl)) {
        return fail(GEIST_E_UNSUPPORTED, "batcher_create: no launch shape for n_vocab=%zu with max_history=%zu", n_vocab, max_history);
    }
    geist_b200_batcher *b = new (std::nothrow) geist_b200_batcher();
    if (b == nullptr) {
        return fail(GEIST_E_OOM, "batcher_create: host allocation");
    }
    b->ctx          = ctx;
    b->V            = n_vocab;
    b->max_sessions = max_sessions;
    b->max_history  = max_history;
    b->used.assign(max_sessions, 0);
    b->pen_active.assign(max_sessions, 0);
    b->h_T.assign(max_sessions, 0.0f);
    b->h_P.assign(max_sessions, 1.0f);
    b->h_K.assign(max_sessions, 0);
    b->h_cap.assign(max_sessions, 0.0f);
    b->pending.assign(max_sessions, -1);
    b->pending_in_hist.assign(max_sessions, 0);
    b->mask_active.assign(max_sessions, 0);
    b->last_row.assign(max_sessions, geist_b200_batcher::LastRow{});
    b->peek_stage.resize(max_sessions);
    b->mask_words = (n_vocab + 31) / 32;
    const size_t S = max_sessions, R = S * GEIST_B200_SPEC_KMAX;
    cudaError_t  e = cudaSuccess;
    auto         A = [&](void **p, size_t bytes) {
        if (e == cudaSuccess) {
            e = cudaMalloc(p, std::max<size_t>(bytes, 16));
            if (e == cudaSuccess) {
                e = cudaMemset(*p, 0, std::max<size_t>(bytes, 16));
            }
        }
    };
    A((void **) &b->d_T, S * 4);
    A((void **) &b->d_P, S * 4);
    A((void **) &b->d_rep, S * 4);
    A((void **) &b->d_freq, S * 4);
    A((void **) &b->d_pres, S * 4);
    A((void **) &b->d_K, S * 4);
    A((void **) &b->d_rng, S * 8);
    A((void **) &b->d_rng_tmp, S * 8);
    A((void **) &b->d_hist, S * std::max<size_t>(max_history, 1) * 4);
    A((void **) &b->d_hist_len, S * 4);
    A((void **) &b->d_hist_tot, S * 8);
    A((void **) &b->d_slot, S * 4);
    A((void **) &b->d_tokens, R * 4);
    A((void **) &b->d_status, R * 4);
    A((void **) &b->d_fed, R * 4);
    A((void **) &b->d_accepted, S * 4);
    A((void **) &b->d_nemit, S * 4);
    A((void **) &b->d_emitted, S * (GEIST_B200_SPEC_KMAX + 1) * 4);
    A((void **) &b->d_ones, S * 4);
    A((void **) &b->d_pending, S * 4);
    A((void **) &b->d_cap, S * 4);
    A((void **) &b->d_peek, n_vocab * 4);
    A((void **) &b->d_drafts, S * (GEIST_B200_SPEC_KMAX + 1) * 4);
    A((void **) &b->d_ndrafts, S * 4);
    A((void **) &b->d_matchL, S * 4);
    A((void **) &b->d_skip, S * 4);
    b->h_pin_ints = S * (1 + 2 + 2 * GEIST_B200_SPEC_KMAX + GEIST_B200_SPEC_KMAX + GEIST_B200_SPEC_KMAX + 1) + 64;
    if (e == cudaSuccess) {
        e = cudaHostAlloc((void **) &b->h_pin, b->h_pin_ints * 4, cudaHostAllocDefault);
    }
    for (int i = 0; i < 2 && e == cudaSuccess; i++) {
        e = cudaStreamCreateWithFlags(&b->copy_stream[i], cudaStreamNonBlocking);
        if (e == cudaSuccess) {
            e = cudaEventCreateWithFlags(&b->ev[i], cudaEventDisableTiming);
        }
    }
    if (e == cudaSuccess) {
        std::vector<int> ones(S, 1);
        e = cudaMemcpy(b->d_ones, ones.data(), S * 4, cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess) {
        e = cudaMemset(b->d_pending, 0xff, S * 4); /* -1: nothing pending */
    }
    if (e != cudaSuccess) {
        geist_b200_batcher_destroy(b);
        return fail(e == cudaErrorMemoryAllocation ? GEIST_E_OOM : GEIST_E_BACKEND, "batcher_create: %s", cudaGetErrorString(e));
    }
    *out = b;
    return GEIST_OK;
}

static bool slot_ok(const geist_b200_batcher *b, int32_t s) { return b != nullptr && s >= 0 && (size_t) s < b->max_sessions && b->used[(size_t) s]; }

extern "C" enum geist_status geist_b200_session_open(struct geist_b200_batcher *b, const struct geist_session_opts *opts, const struct geist_b200_penalty_opts *pen,
                                                     int32_t *out_session) {
    if (b == nullptr || out_session == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "session_open: NULL batcher or out_session");
    }
    *out_session = -1;
    std::lock_guard<std::mutex> lk(b->mu);
    size_t                      s = 0;
    while (s < b->max_sessions && b->used[s]) {
        s++;
    }
    if (s == b->max_sessions) {
        return fail(GEIST_E_OOM, "session_open: all %zu session slots are in use", b->max_sessions);
    }
    /* arch_state.c:1168-1173 defaults, then step.c:385-411 */
    float    T = 0.0f, P = 1.0f;
    int      K    = 0;
    uint64_t seed = 0xCAFEBABE1234ULL;
    if (opts != nullptr) {
        T = opts->temperature;
        P = opts->top_p > 0.0f ? opts->top_p : 1.0f;
        K = opts->top_k;
        if (opts->random_seed != 0) {
            seed = opts->random_seed;
        }
        if (T != T || P != P) {
            return fail(GEIST_E_INVALID_ARG, "session_open: NaN sampler option");
        }
    }
    float rep = 1.0f, freq = 0.0f, pres = 0.0f;
    if (pen != nullptr) {
        rep  = pen->repetition_penalty > 0.0f ? pen->repetition_penalty : 1.0f;
        freq = pen->frequency_penalty;
        pres = pen->presence_penalty;
        if (rep != rep || freq != freq || pres != pres) {
            return fail(GEIST_E_INVALID_ARG, "session_open: NaN penalty option");
        }
    }
    const bool active = rep != 1.0f || freq != 0.0f || pres != 0.0f;
    if (active && b->max_history == 0) {
        return fail(GEIST_E_INVALID_ARG, "session_open: penalties need a batcher created with max_history > 0");
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    struct geist_rng r;
    geist_rng_seed(&r, seed);
    const long long zero64 = 0;
    const int       zero   = 0;
    CUDA_TRY(cudaMemcpy(b->d_T + s, &T, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_P + s, &P, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_K + s, &K, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_rep + s, &rep, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_freq + s, &freq, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_pres + s, &pres, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_rng + s, &r.state, 8, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_hist_len + s, &zero, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_hist_tot + s, &zero64, 8, cudaMemcpyHostToDevice));
    const int   none = -1;
    const float nocap = 0.0f;
    CUDA_TRY(cudaMemcpy(b->d_pending + s, &none, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_cap + s, &nocap, 4, cudaMemcpyHostToDevice));
    b->used[s]       = 1;
    b->pen_active[s] = active ? 1 : 0;
    b->n_pen_active += active ? 1 : 0;
    b->h_T[s]        = T;
    b->h_P[s]        = P;
    b->h_K[s]        = K;
    b->h_cap[s]      = 0.0f;
    b->pending[s]    = -1;
    b->pending_in_hist[s] = 0;
    b->last_row[s]   = geist_b200_batcher::LastRow{};
    *out_session = (int32_t) s;
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_session_close(struct geist_b200_batcher *b, int32_t session) {
    if (b == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "session_close: NULL batcher");
    }
    std::lock_guard<std::mutex> lk(b->mu);
    if (!slot_ok(b, session)) {
        return fail(GEIST_E_INVALID_ARG, "session_close: session %d is not open", session);
    }
    b->n_pen_active -= b->pen_active[(size_t) session] ? 1 : 0;
    b->pen_active[(size_t) session] = 0;
    b->n_cap_active -= b->h_cap[(size_t) session] > 0.0f ? 1 : 0;
    b->h_cap[(size_t) session] = 0.0f;
    if (b->mask_active[(size_t) session]) { /* the slot's mask row goes back to all ones for whoever opens it next */
        cudaSetDevice(b->ctx->device);
        cudaMemset(b->d_mask + (size_t) session * b->mask_words, 0xff, b->mask_words * 4);
        b->mask_active[(size_t) session] = 0;
        b->n_mask_active--;
    }
    b->pending[(size_t) session]  = -1;
    b->last_row[(size_t) session] = geist_b200_batcher::LastRow{};
    b->used[(size_t) session]     = 0;
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_session_reset(struct geist_b200_batcher *b, int32_t session) {
    if (b == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "session_reset: NULL batcher");
    }
    std::lock_guard<std::mutex> lk(b->mu);
    if (!slot_ok(b, session)) {
        return fail(GEIST_E_INVALID_ARG, "session_reset: session %d is not open", session);
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    const long long zero64 = 0;
    const int       zero   = 0;
    CUDA_TRY(cudaMemcpy(b->d_hist_len + session, &zero, 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_hist_tot + session, &zero64, 8, cudaMemcpyHostToDevice));
    const int none = -1;
    CUDA_TRY(cudaMemcpy(b->d_pending + session, &none, 4, cudaMemcpyHostToDevice));
    b->pending[(size_t) session]         = -1;
    b->pending_in_hist[(size_t) session] = 0;
    b->last_row[(size_t) session]        = geist_b200_batcher::LastRow{};
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_session_get_rng(struct geist_b200_batcher *b, int32_t session, uint64_t *state) {
    if (b == nullptr || state == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "session_get_rng: NULL argument");
    }
    std::lock_guard<std::mutex> lk(b->mu);
    if (!slot_ok(b, session)) {
        return fail(GEIST_E_INVALID_ARG, "session_get_rng: session %d is not open", session);
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    CUDA_TRY(cudaMemcpy(state, b->d_rng + session, 8, cudaMemcpyDeviceToHost));
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_session_set_rng(struct geist_b200_batcher *b, int32_t session, uint64_t state) {
    if (b == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "session_set_rng: NULL batcher");
    }
    std::lock_guard<std::mutex> lk(b->mu);
    if (!slot_ok(b, session)) {
        return fail(GEIST_E_INVALID_ARG, "session_set_rng: session %d is not open", session);
    }
    if (state == 0) {
        return fail(GEIST_E_INVALID_ARG, "session_set_rng: 0 is not a valid xorshift state");
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    CUDA_TRY(cudaMemcpy(b->d_rng + session, &state, 8, cudaMemcpyHostToDevice));
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_session_push_history(struct geist_b200_batcher *b, int32_t session, size_t n, const geist_token_t *ids) {
    if (b == nullptr || (n > 0 && ids == nullptr)) {
        return fail(GEIST_E_INVALID_ARG, "session_push_history: NULL argument");
    }
    std::lock_guard<std::mutex> lk(b->mu);
    if (!slot_ok(b, session)) {
        return fail(GEIST_E_INVALID_ARG, "session_push_history: session %d is not open", session);
    }
    if (b->max_history == 0 || n == 0) {
        return GEIST_OK; /* nothing is kept */
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    long long tot = 0;
    CUDA_TRY(cudaMemcpy(&tot, b->d_hist_tot + session, 8, cudaMemcpyDeviceToHost));
    /* ring: only the last max_history ids can matter */
    const size_t H     = b->max_history;
    const size_t first = n > H ? n - H : 0;
    int         *row   = b->d_hist + (size_t) session * H;
    for (size_t i = first; i < n;) {
        const size_t pos = (size_t) ((tot + (long long) i) % (long long) H);
        const size_t run = std::min(n - i, H - pos);
        CUDA_TRY(cudaMemcpy(row + pos, ids + i, run * 4, cudaMemcpyHostToDevice));
        i += run;
    }
    tot += (long long) n;
    const int len = (int) std::min<long long>(tot, (long long) H);
    CUDA_TRY(cudaMemcpy(b->d_hist_tot + session, &tot, 8, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMemcpy(b->d_hist_len + session, &len, 4, cudaMemcpyHostToDevice));
    return GEIST_OK;
}

namespace {

/* Shared by step and verify: k rows per session, optional accept. */
enum geist_status batcher_run(geist_b200_batcher *b, size_t n, const int32_t *sessions, size_t k, const geist_token_t *fed, const float *logits, size_t row_stride,
                              int logits_on_host, int append_history, bool verify, int32_t *accepted, int32_t *n_out, geist_token_t *out_tokens, bool hand_out_pending = false) {
    if (b == nullptr || sessions == nullptr || logits == nullptr || out_tokens == nullptr || n == 0) {
        return fail(GEIST_E_INVALID_ARG, "batcher: missing argument");
    }
    if (n > b->max_sessions) {
        return fail(GEIST_E_INVALID_ARG, "batcher: %zu sessions in one call, batcher holds %zu", n, b->max_sessions);
    }
    if (k == 0 || k > GEIST_B200_SPEC_KMAX) {
        return fail(GEIST_E_INVALID_ARG, "batcher: k must be in [1, %d]", GEIST_B200_SPEC_KMAX);
    }
    if (verify && (fed == nullptr || accepted == nullptr || n_out == nullptr)) {
        return fail(GEIST_E_INVALID_ARG, "batcher_verify: fed, accepted and n_out are required");
    }
    if (row_stride < b->V) {
        return fail(GEIST_E_INVALID_ARG, "batcher: row_stride %zu < n_vocab %zu", row_stride, b->V);
    }
    std::lock_guard<std::mutex> lk(b->mu);
    std::vector<char>           seen(b->max_sessions, 0);
    for (size_t i = 0; i < n; i++) {
        if (!slot_ok(b, sessions[i])) {
            return fail(GEIST_E_INVALID_ARG, "batcher: session %d is not open", sessions[i]);
        }
        if (seen[(size_t) sessions[i]]) {
            return fail(GEIST_E_INVALID_ARG, "batcher: session %d appears twice in one call", sessions[i]);
        }
        seen[(size_t) sessions[i]] = 1;
        /* arch.c:138-140: nothing pending, nothing to hand out or to verify from */
        if ((hand_out_pending || (verify && fed[i * k] < 0)) && b->pending[(size_t) sessions[i]] < 0) {
            return fail(GEIST_E_INVALID_STATE, "batcher: session %d has no pending token (sample a row for it first)", sessions[i]);
        }
    }
    /* which finishing kernels the launch needs: the sessions' sampler settings are known here */
    bool any_fast = false, any_rest = false, all_greedy = true;
    for (size_t i = 0; i < n; i++) {
        const size_t sl   = (size_t) sessions[i];
        const float  T    = b->h_T[sl];
        const int    K    = b->h_K[sl];
        const bool   fast = !(T > 0.0f) || (K > 1 && (size_t) K < b->V && K <= gb::kFastKMax);
        any_fast |= fast;
        any_rest |= !fast;
        all_greedy &= !(T > 0.0f);
    }
    int32_t hint = !any_rest ? GEIST_B200_FINISH_GREEDY_TOPK : (!any_fast ? GEIST_B200_FINISH_GENERAL : GEIST_B200_FINISH_AUTO);
    if (all_greedy) {
        hint = GEIST_B200_FINISH_GREEDY;
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    cudaStream_t st   = b->ctx->stream;
    const size_t rows = n * k;
    /* pinned layout */
    int *h_slot = b->h_pin;
    int *h_fed  = h_slot + b->max_sessions;
    int *h_tok  = h_fed + b->max_sessions * GEIST_B200_SPEC_KMAX;
    int *h_stat = h_tok + b->max_sessions * GEIST_B200_SPEC_KMAX;
    int *h_acc  = h_stat + b->max_sessions * GEIST_B200_SPEC_KMAX;
    int *h_nem  = h_acc + b->max_sessions;
    int *h_emit = h_nem + b->max_sessions; /* [n, k+1] */
    memcpy(h_slot, sessions, n * 4);
    CUDA_TRY(cudaMemcpyAsync(b->d_slot, h_slot, n * 4, cudaMemcpyHostToDevice, st));
    if (verify) {
        memcpy(h_fed, fed, rows * 4);
        for (size_t i = 0; i < n; i++) {
            if (h_fed[i * k] < 0) { /* the caller left the first fed token to the session: its pending token */
                h_fed[i * k] = b->pending[(size_t) sessions[i]];
            }
        }
        CUDA_TRY(cudaMemcpyAsync(b->d_fed, h_fed, rows * 4, cudaMemcpyHostToDevice, st));
    }
    const bool pen = b->n_pen_active > 0 && b->max_history > 0;
    if (logits_on_host) { /* the staging block is about to be overwritten: rows remembered in it are gone */
        for (auto &lr : b->last_row) {
            if (lr.valid && b->d_logits != nullptr && lr.ptr >= b->d_logits && lr.ptr < b->d_logits + b->d_logits_cap) {
                lr.valid = false;
            }
        }
    }

    geist_b200_batch d{};
    d.n_vocab            = b->V;
    d.rows_per_seq       = k;
    d.temperature        = b->d_T;
    d.top_k              = b->d_K;
    d.top_p              = b->d_P;
    d.repetition_penalty = pen ? b->d_rep : nullptr;
    d.frequency_penalty  = pen ? b->d_freq : nullptr;
    d.presence_penalty   = pen ? b->d_pres : nullptr;
    d.history            = pen ? b->d_hist : nullptr;
    d.history_stride     = b->max_history;
    d.history_len        = pen ? b->d_hist_len : nullptr;
    d.fed_stride         = k;
    d.rng_in             = reinterpret_cast<const uint64_t *>(b->d_rng);
    d.rng_out            = reinterpret_cast<uint64_t *>(b->d_rng_tmp);
    d.softcap            = b->n_cap_active > 0 ? b->d_cap : nullptr;
    d.logit_mask         = b->n_mask_active > 0 ? b->d_mask : nullptr;
    d.logit_mask_stride  = b->mask_words;
    d.finish_hint        = hint;

    /* the sampling launch(es); run a second time without the hint when a row asked for that */
    auto launch_sampling = [&](bool copy_in) -> enum geist_status {
        if (!logits_on_host) {
            d.logits     = logits;
            d.row_stride = row_stride;
            d.n_seq      = n;
            d.slot       = b->d_slot;
            d.fed_tokens = (pen && verify) ? b->d_fed : nullptr;
            d.tokens     = b->d_tokens;
            d.row_status = b->d_status;
            enum geist_status s = geist_b200_sample_batch(b->ctx, &d, st);
            if (s != GEIST_OK) {
                return s;
            }
        } else {
            /* host logits: copy in chunks of sequences on two streams so that one chunk's kernel
             * runs under the next chunk's copy */
            if (b->d_logits_cap < rows * b->V) {
                cudaFree(b->d_logits);
                b->d_logits     = nullptr;
                b->d_logits_cap = 0;
                CUDA_TRY(cudaMalloc((void **) &b->d_logits, rows * b->V * sizeof(float)));
                b->d_logits_cap = rows * b->V;
            }
            CUDA_TRY(cudaEventRecord(b->ev[0], st)); /* slots / fed are on the way */
            const size_t seq_chunk = std::max<size_t>(1, (32 + k - 1) / k);
            int          which     = 0;
            for (size_t s0 = 0; s0 < n; s0 += seq_chunk, which ^= 1) {
                const size_t ns = std::min(seq_chunk, n - s0);
                cudaStream_t cs = b->copy_stream[which];
                if (s0 < 2 * seq_chunk) {
                    CUDA_TRY(cudaStreamWaitEvent(cs, b->ev[0], 0));
                }
                if (!copy_in) {
                /* second time round: the rows are on the device already */
            } else if (row_stride == b->V) { /* dense rows: one linear copy per chunk */
                    CUDA_TRY(cudaMemcpyAsync(b->d_logits + s0 * k * b->V, logits + s0 * k * row_stride, ns * k * b->V * 4, cudaMemcpyHostToDevice, cs));
                } else {
                    CUDA_TRY(cudaMemcpy2DAsync(b->d_logits + s0 * k * b->V, b->V * 4, logits + s0 * k * row_stride, row_stride * 4, b->V * 4, ns * k, cudaMemcpyHostToDevice, cs));
                }
                d.logits     = b->d_logits + s0 * k * b->V;
                d.row_stride = b->V;
                d.n_seq      = ns;
                d.slot       = b->d_slot + s0;
                d.fed_tokens = (pen && verify) ? b->d_fed + s0 * k : nullptr;
                d.tokens     = b->d_tokens + s0 * k;
                d.row_status = b->d_status + s0 * k;
                enum geist_status s = geist_b200_sample_batch(b->ctx, &d, cs);
                if (s != GEIST_OK) {
                    return s;
                }
            }
            for (int i = 0; i < 2; i++) {
                CUDA_TRY(cudaEventRecord(b->ev[1], b->copy_stream[i]));
                CUDA_TRY(cudaStreamWaitEvent(st, b->ev[1], 0));
            }
        }
        return GEIST_OK;
    };
    const int *append_tok = b->d_tokens;
    const int *append_cnt = b->d_ones;
    int        per_seq    = 1;
    int        first      = 0;
    if (verify) {
        append_tok = b->d_emitted;
        append_cnt = b->d_nemit;
        per_seq    = (int) k + 1;
        first      = 1; /* emitted[0] is the pending token, which joined the history when it was sampled */
    }
    for (int attempt = 0; attempt < 2; attempt++) {
        const enum geist_status ls = launch_sampling(attempt == 0);
        if (ls != GEIST_OK) {
            return ls;
        }
        if (verify) {
            gb::AcceptParams ap{b->d_fed, b->d_tokens, (int) n, (int) k, b->d_accepted, b->d_nemit, b->d_emitted};
            CUDA_TRY(gb::launch_accept(ap, st));
        }
        CUDA_TRY(cudaMemcpyAsync(h_stat, b->d_status, rows * 4, cudaMemcpyDeviceToHost, st));
        if (verify) {
            CUDA_TRY(cudaMemcpyAsync(h_acc, b->d_accepted, n * 4, cudaMemcpyDeviceToHost, st));
            CUDA_TRY(cudaMemcpyAsync(h_nem, b->d_nemit, n * 4, cudaMemcpyDeviceToHost, st));
            CUDA_TRY(cudaMemcpyAsync(h_emit, b->d_emitted, n * (k + 1) * 4, cudaMemcpyDeviceToHost, st));
        } else {
            CUDA_TRY(cudaMemcpyAsync(h_tok, b->d_tokens, rows * 4, cudaMemcpyDeviceToHost, st));
        }
        CUDA_TRY(cudaStreamSynchronize(st));
        bool retry = false;
        for (size_t i = 0; i < rows; i++) {
            if (h_stat[i] & (GEIST_B200_ROW_LOAD_TIMEOUT | GEIST_B200_ROW_HIST_OVERFLOW | GEIST_B200_ROW_INTERNAL)) {
                return fail(GEIST_E_BACKEND, "batcher: row %zu reported status 0x%x", i, h_stat[i]);
            }
            retry |= (h_stat[i] & GEIST_B200_ROW_RETRY) != 0;
        }
        if (!retry) {
            break;
        }
        if (attempt == 1) {
            return fail(GEIST_E_BACKEND, "batcher: a row asked to be launched again twice");
        }
        /* a top-k row with more candidates than the small finishing kernel holds (rare: thousands of equal values
         * at the top): the whole call again with the general kernel; nothing of the first attempt was committed */
        d.finish_hint = GEIST_B200_FINISH_AUTO;
    }
    /* committed behind the host's look at the status: generator words and history ring (asynchronous: the next call
     * is ordered behind it on the same stream) */
    CUDA_TRY(gb::launch_post_step(b->d_slot, (int) n, per_seq, first, (append_history && b->max_history) ? append_tok : nullptr, append_cnt, b->d_hist, (int) b->max_history,
                                  b->d_hist_len, b->d_hist_tot, b->d_rng_tmp, b->d_rng, st));
    const float *dev_rows = logits_on_host ? b->d_logits : logits;
    const size_t dev_stride = logits_on_host ? b->V : row_stride;
    if (verify) {
        memcpy(accepted, h_acc, n * 4);
        memcpy(n_out, h_nem, n * 4);
        memcpy(out_tokens, h_emit, n * (k + 1) * 4);
        for (size_t i = 0; i < n; i++) { /* session.c:627-634: the last emitted token still has to go through the model */
            b->pending[(size_t) sessions[i]]  = -1;
            b->last_row[(size_t) sessions[i]] = geist_b200_batcher::LastRow{};
        }
    } else {
        for (size_t i = 0; i < n; i++) {
            const size_t sl = (size_t) sessions[i];
            out_tokens[i]   = hand_out_pending ? b->pending[sl] : h_tok[i]; /* arch.c:141-147: return, then advance */
            b->pending[sl]  = h_tok[i];
            b->pending_in_hist[sl] = (append_history && b->max_history) ? 1 : 0;
            b->last_row[sl].ptr    = dev_rows + i * dev_stride;
            b->last_row[sl].valid  = true;
        }
    }
    return GEIST_OK;
}

} /* namespace */

extern "C" enum geist_status geist_b200_batcher_step(struct geist_b200_batcher *b, size_t n, const int32_t *sessions, const float *logits, size_t row_stride, int logits_on_host,
                                                     int append_history, geist_token_t *out_tokens) {
    return batcher_run(b, n, sessions, 1, nullptr, logits, row_stride, logits_on_host, append_history, false, nullptr, nullptr, out_tokens);
}

extern "C" enum geist_status geist_b200_batcher_verify(struct geist_b200_batcher *b, size_t n, const int32_t *sessions, size_t k, const geist_token_t *fed, const float *logits,
                                                       size_t row_stride, int logits_on_host, int append_history, int32_t *accepted, int32_t *n_out, geist_token_t *out_tokens) {
    return batcher_run(b, n, sessions, k, fed, logits, row_stride, logits_on_host, append_history, true, accepted, n_out, out_tokens);
}

/* arch.c:133-147, batched: hands out each session's pending token and makes the token sampled from `logits`
 * (the model's output for that pending token) the new pending one. */
extern "C" enum geist_status geist_b200_batcher_decode_step(struct geist_b200_batcher *b, size_t n, const int32_t *sessions, const float *logits, size_t row_stride,
                                                            int logits_on_host, int append_history, geist_token_t *out_tokens) {
    return batcher_run(b, n, sessions, 1, nullptr, logits, row_stride, logits_on_host, append_history, false, nullptr, nullptr, out_tokens, true);
}

extern "C" geist_token_t geist_b200_session_peek_next_token(struct geist_b200_batcher *b, int32_t session) {
    if (b == nullptr) {
        return -1;
    }
    std::lock_guard<std::mutex> lk(b->mu);
    return slot_ok(b, session) ? b->pending[(size_t) session] : -1;
}

extern "C" enum geist_status geist_b200_session_set_softcap(struct geist_b200_batcher *b, int32_t session, float softcap) {
    if (b == nullptr || softcap != softcap || softcap < 0.0f) {
        return fail(GEIST_E_INVALID_ARG, "session_set_softcap: NULL batcher or a cap that is negative or NaN");
    }
    std::lock_guard<std::mutex> lk(b->mu);
    if (!slot_ok(b, session)) {
        return fail(GEIST_E_INVALID_ARG, "session_set_softcap: session %d is not open", session);
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    CUDA_TRY(cudaMemcpy(b->d_cap + session, &softcap, 4, cudaMemcpyHostToDevice));
    b->n_cap_active += (softcap > 0.0f ? 1 : 0) - (b->h_cap[(size_t) session] > 0.0f ? 1 : 0);
    b->h_cap[(size_t) session] = softcap;
    return GEIST_OK;
}

extern "C" enum geist_status geist_b200_session_set_logit_mask(struct geist_b200_batcher *b, int32_t session, const uint32_t *allowed, size_t n_words) {
    if (b == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "session_set_logit_mask: NULL batcher");
    }
    std::lock_guard<std::mutex> lk(b->mu);
    if (!slot_ok(b, session)) {
        return fail(GEIST_E_INVALID_ARG, "session_set_logit_mask: session %d is not open", session);
    }
    if (allowed != nullptr && n_words < b->mask_words) {
        return fail(GEIST_E_INVALID_ARG, "session_set_logit_mask: %zu words hold fewer than n_vocab %zu bits", n_words, b->V);
    }
    if (allowed == nullptr && !b->mask_active[(size_t) session]) {
        return GEIST_OK;
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    if (b->d_mask == nullptr) { /* first mask of this batcher: one row per slot, every column allowed */
        CUDA_TRY(cudaMalloc((void **) &b->d_mask, b->max_sessions * b->mask_words * 4));
        CUDA_TRY(cudaMemset(b->d_mask, 0xff, b->max_sessions * b->mask_words * 4));
    }
    uint32_t *row = b->d_mask + (size_t) session * b->mask_words;
    if (allowed != nullptr) {
        CUDA_TRY(cudaMemcpy(row, allowed, b->mask_words * 4, cudaMemcpyHostToDevice));
    } else {
        CUDA_TRY(cudaMemset(row, 0xff, b->mask_words * 4));
    }
    const char now = allowed != nullptr ? 1 : 0;
    b->n_mask_active += (size_t) now - (size_t) b->mask_active[(size_t) session];
    b->mask_active[(size_t) session] = now;
    return GEIST_OK;
}

/* geist_session_peek_logits (geist_util.h:195-211, arch.c:163-195): the row the session's pending token was
 * sampled from, copied into storage that belongs to the session, with the model's soft cap applied. */
extern "C" const float *geist_b200_session_peek_logits(struct geist_b200_batcher *b, int32_t session, size_t *n_logits) {
    if (n_logits == nullptr) {
        return nullptr;
    }
    *n_logits = 0;
    if (b == nullptr) {
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(b->mu);
    if (!slot_ok(b, session) || !b->last_row[(size_t) session].valid || b->pending[(size_t) session] < 0) {
        return nullptr; /* nothing pending */
    }
    if (cudaSetDevice(b->ctx->device) != cudaSuccess) {
        return nullptr;
    }
    cudaStream_t        st    = b->ctx->stream;
    std::vector<float> &stage = b->peek_stage[(size_t) session];
    try {
        stage.resize(b->V);
    } catch (const std::bad_alloc &) {
        fail(GEIST_E_OOM, "session_peek_logits: no host memory for %zu floats", b->V);
        return nullptr;
    }
    const float c  = b->h_cap[(size_t) session];
    cudaError_t e  = cudaMemcpyAsync(b->d_peek, b->last_row[(size_t) session].ptr, b->V * 4, cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess && c > 0.0f) {
        e = gb::launch_softcap_row(b->d_peek, (int) b->V, c, st);
    }
    if (e == cudaSuccess) {
        e = cudaMemcpyAsync(stage.data(), b->d_peek, b->V * 4, cudaMemcpyDeviceToHost, st);
    }
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(st);
    }
    if (e != cudaSuccess) {
        fail(GEIST_E_BACKEND, "session_peek_logits: %s", cudaGetErrorString(e));
        return nullptr;
    }
    *n_logits = b->V;
    return stage.data();
}

namespace {
int spec_min_L() { /* session.c:583-591: GEIST_SPEC_MIN_L, default 2, read once */
    static const int v = [] {
        const char *env = getenv("GEIST_SPEC_MIN_L");
        const long  x   = env != nullptr ? atol(env) : 2;
        return x <= 0 ? 1 : (x > 8 ? 8 : (int) x);
    }();
    return v;
}
} /* namespace */

/* The n-gram drafter over caller-held histories (session.c:437-513): host arrays in, host arrays out, the search
 * itself on the device. No lazy gate here: n_drafts is what the search found. */
extern "C" enum geist_status geist_b200_draft_ngram(struct geist_b200_ctx *ctx, size_t n_seq, const geist_token_t *histories, size_t history_stride, const int32_t *history_len,
                                                    const geist_token_t *seeds, size_t k_max, size_t max_suffix, size_t out_capacity, geist_token_t *out_drafts, int32_t *n_drafts,
                                                    int32_t *match_L) {
    if (ctx == nullptr || n_seq == 0 || history_len == nullptr || seeds == nullptr || out_drafts == nullptr || n_drafts == nullptr || (histories == nullptr && history_stride > 0)) {
        return fail(GEIST_E_INVALID_ARG, "draft_ngram: missing argument");
    }
    if (k_max == 0 || k_max > GEIST_B200_SPEC_KMAX || out_capacity < k_max + 1 || max_suffix == 0) { /* session.c:540-549 */
        return fail(GEIST_E_INVALID_ARG, "draft_ngram: k_max must be in [1, %d], out_capacity >= k_max + 1, max_suffix >= 1", GEIST_B200_SPEC_KMAX);
    }
    if (n_seq > (1u << 20) || history_stride > 0x7fffffffu) {
        return fail(GEIST_E_INVALID_ARG, "draft_ngram: sizes out of range");
    }
    for (size_t i = 0; i < n_seq; i++) {
        if (history_len[i] < 0 || (size_t) history_len[i] > history_stride) {
            return fail(GEIST_E_INVALID_ARG, "draft_ngram: history_len[%zu] = %d outside [0, history_stride]", i, history_len[i]);
        }
    }
    CUDA_TRY(cudaSetDevice(ctx->device));
    std::lock_guard<std::mutex> lk(ctx->small_mu);
    const size_t hs = std::max<size_t>(history_stride, 1);
    int         *d  = nullptr;
    /* one allocation: histories | lens | seeds | drafts | n | L */
    const size_t ints = n_seq * (hs + 2 + out_capacity + 2);
    CUDA_TRY(cudaMalloc((void **) &d, ints * 4));
    int *d_h = d, *d_len = d_h + n_seq * hs, *d_seed = d_len + n_seq, *d_out = d_seed + n_seq, *d_n = d_out + n_seq * out_capacity, *d_L = d_n + n_seq;
    cudaStream_t st = ctx->stream;
    cudaError_t  e  = cudaSuccess;
    if (history_stride > 0) {
        e = cudaMemcpyAsync(d_h, histories, n_seq * hs * 4, cudaMemcpyHostToDevice, st);
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_len, history_len, n_seq * 4, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_seed, seeds, n_seq * 4, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_out, 0xff, n_seq * out_capacity * 4, st);
    if (e == cudaSuccess) {
        e = gb::launch_draft_ngram(nullptr, (int) n_seq, d_h, (long long) hs, d_len, nullptr, d_seed, nullptr, (int) k_max, (int) std::min<size_t>(max_suffix, 8), 1, (int) out_capacity, d_out,
                                   d_n, d_L, st);
    }
    std::vector<int> hL(n_seq);
    if (e == cudaSuccess) e = cudaMemcpyAsync(out_drafts, d_out, n_seq * out_capacity * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(n_drafts, d_n, n_seq * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(hL.data(), d_L, n_seq * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d);
    if (e != cudaSuccess) {
        return fail(GEIST_E_BACKEND, "draft_ngram: %s", cudaGetErrorString(e));
    }
    if (match_L != nullptr) {
        memcpy(match_L, hL.data(), n_seq * 4);
    }
    return GEIST_OK;
}

/* The drafting half of geist_session_decode_speculative (session.c:532-591) for n sessions at once: seed = the
 * session's pending token, context = the session's history ring on the device, max_suffix 4, then the lazy gate.
 * A session that should decode one token the plain way comes back with n_drafts = 1. */
extern "C" enum geist_status geist_b200_batcher_propose_drafts(struct geist_b200_batcher *b, size_t n, const int32_t *sessions, size_t k_max, size_t out_capacity,
                                                               geist_token_t *out_drafts, int32_t *n_drafts, int32_t *match_L) {
    if (b == nullptr || sessions == nullptr || n == 0 || out_drafts == nullptr || n_drafts == nullptr) {
        return fail(GEIST_E_INVALID_ARG, "batcher_propose_drafts: missing argument");
    }
    if (k_max == 0 || k_max > GEIST_B200_SPEC_KMAX || out_capacity < k_max + 1) { /* session.c:540-549 */
        return fail(GEIST_E_INVALID_ARG, "batcher_propose_drafts: k_max must be in [1, %d] and out_capacity >= k_max + 1", GEIST_B200_SPEC_KMAX);
    }
    if (n > b->max_sessions) {
        return fail(GEIST_E_INVALID_ARG, "batcher_propose_drafts: %zu sessions in one call, batcher holds %zu", n, b->max_sessions);
    }
    std::lock_guard<std::mutex> lk(b->mu);
    int *h_slot = b->h_pin, *h_seed = h_slot + b->max_sessions, *h_skip = h_seed + b->max_sessions; /* the pinned block is larger than 3 * max_sessions ints */
    int *h_out  = h_skip + b->max_sessions;
    for (size_t i = 0; i < n; i++) {
        if (!slot_ok(b, sessions[i])) {
            return fail(GEIST_E_INVALID_ARG, "batcher_propose_drafts: session %d is not open", sessions[i]);
        }
        const size_t sl = (size_t) sessions[i];
        if (b->pending[sl] < 0) {
            return fail(GEIST_E_INVALID_STATE, "batcher_propose_drafts: session %d has no pending token", sessions[i]);
        }
        h_slot[i] = sessions[i];
        h_seed[i] = b->pending[sl];
        h_skip[i] = b->pending_in_hist[sl] ? 1 : 0;
    }
    CUDA_TRY(cudaSetDevice(b->ctx->device));
    cudaStream_t st = b->ctx->stream;
    const int    oc = GEIST_B200_SPEC_KMAX + 1; /* row length of the device-side draft table */
    CUDA_TRY(cudaMemcpyAsync(b->d_slot, h_slot, n * 4, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaMemcpyAsync(b->d_pending, h_seed, n * 4, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaMemcpyAsync(b->d_skip, h_skip, n * 4, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaMemsetAsync(b->d_drafts, 0xff, n * oc * 4, st));
    CUDA_TRY(gb::launch_draft_ngram(b->d_slot, (int) n, b->d_hist, (long long) std::max<size_t>(b->max_history, 1), b->d_hist_len, b->d_hist_tot, b->d_pending, b->d_skip, (int) k_max, 4,
                                    spec_min_L(), oc, b->d_drafts, b->d_ndrafts, b->d_matchL, st));
    int *h_n = h_out + n * oc, *h_L = h_n + n;
    CUDA_TRY(cudaMemcpyAsync(h_out, b->d_drafts, n * oc * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaMemcpyAsync(h_n, b->d_ndrafts, n * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaMemcpyAsync(h_L, b->d_matchL, n * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    for (size_t i = 0; i < n; i++) {
        for (size_t j = 0; j < out_capacity; j++) {
            out_drafts[i * out_capacity + j] = (j < (size_t) oc && (int) j < h_n[i]) ? h_out[i * oc + j] : -1;
        }
        n_drafts[i] = h_n[i];
        if (match_L != nullptr) {
            match_L[i] = h_L[i];
        }
    }
    return GEIST_OK;
}


/* ------------------------------------------------ no-allocation entry -- */

extern "C" enum geist_status geist_b200_argmax_rows_static(int device, const float *logits, size_t row_stride, size_t n_rows, size_t n_vocab, int32_t *out_index, void *stream) {
    if (logits == nullptr || out_index == nullptr || n_rows == 0 || n_vocab == 0) {
        return fail(GEIST_E_INVALID_ARG, "argmax_rows_static: logits, out_index, n_rows and n_vocab are required");
    }
    if (row_stride < n_vocab) {
        return fail(GEIST_E_INVALID_ARG, "argmax_rows_static: row_stride %zu < n_vocab %zu", row_stride, n_vocab);
    }
    if (n_vocab > (size_t) 0x7fffffff) {
        return fail(GEIST_E_INVALID_ARG, "argmax_rows_static: n_vocab %zu does not fit int32 ids", n_vocab);
    }
    const int max_rows = gb::argmax_rows_static_max_rows((long long) n_vocab);
    if (n_rows > (size_t) max_rows) {
        return fail(GEIST_E_INVALID_ARG,
                    "argmax_rows_static: %zu rows of %zu exceed the built-in scratch (at most %d rows at this vocabulary: 4096 rows and 65536 slices of 8192 floats per call); "
                    "split the batch or use geist_b200_sample_batch",
                    n_rows, n_vocab, max_rows);
    }
    const char *what = "";
    cudaError_t e    = gb::launch_argmax_rows_static(device, logits, (long long) row_stride, (int) n_rows, (int) n_vocab, out_index, static_cast<cudaStream_t>(stream), &what);
    if (e != cudaSuccess) {
        return fail(e == cudaErrorInvalidDevice ? GEIST_E_INVALID_ARG : GEIST_E_BACKEND, "argmax_rows_static: %s: %s", what, cudaGetErrorString(e));
    }
    return GEIST_OK;
}

/*
 * sampler_stream.cu — the logits -> token kernel (sm_100a).
 *
 * A persistent grid (one CTA per SM) streams every logits row through the chip
 * exactly once. A row is cut into slices of at most 14336 floats; the work
 * item is (row, slice); every CTA owns a contiguous run of items, so that
 * consecutive items mostly belong to one row. Inside a CTA the warps are
 * specialised and nobody waits for another CTA:
 *
 *   The LOADER warp keeps a ring of shared-memory stages full with bulk
 *   asynchronous copies (global -> this CTA's shared memory, signalled on
 *   mbarriers) and prepares each item a few items ahead: its configuration and
 *   the list of the history ids that fall into the slice, each with its count.
 *
 *   14 WORKER warps walk the slices at their own pace. Each owns a fixed share
 *   of every slice: it waits for the copy, applies the penalties that fall
 *   into its share, reads the share once (maximum per lane), looks only at
 *   the lanes that hold something that matters (the maximum's first id, the
 *   entries above the row's select threshold), gives the stage back and adds
 *   what it found to the slice's accumulators. Candidates go straight to
 *   global scratch. The warps meet once per row, to set the row's select
 *   threshold; every later slice of the row reuses it.
 *
 *   The PUBLISHER warp folds a slice as soon as its last worker warp is done:
 *   record to global scratch, the row's counter, and a higher select threshold
 *   for the slices to come (from a histogram of the candidates seen so far).
 *
 *   4 FINISHER warps finish the rows this CTA completed: they merge the row's
 *   slice records, order the few surviving candidates, evaluate their
 *   probabilities exactly and make the draw, while the workers stream on.
 *
 * Rows whose kept set is too large for this (top-k beyond the candidate room,
 * wide top-p nuclei) are served by the finisher warps alone with a multi-pass
 * bisection over a private copy of the row in global scratch.
 *
 * Semantics follow geistlib's CPU sampler:
 *   mode dispatch ............ src/archs/transformer/forward/head.c:172-183
 *   argmax ................... src/engine/sampler.c:52-62
 *   softmax / inverse CDF .... src/engine/sampler.c:68-102
 *   temperature / top-k / top-p  src/engine/sampler.c:106-132, :178-228, :232-305
 *   xorshift64* .............. src/engine/sampler.c:27-48
 *   rows of one session share one generator, in order  head.c:282-303
 * Penalties and vocabulary shards have no counterpart there; they are defined
 * in the header of include/geist_b200.h.
 */
#include "sampler_device.cuh"

namespace gb {

#ifndef GB_FIN_PAUSE
#define GB_FIN_PAUSE 60
#endif

struct PenEntry {
    int   li;
    float orig;
};

/* A short, bounded pause between two polls of a flag (the sleep instruction's granularity is far
 * coarser than the waits here). */
__device__ __forceinline__ void pause_cycles(int cycles) {
    const long long t0 = clock64();
    while (clock64() - t0 < cycles) {
    }
}

/* A load that is served by the L2, where the other SMs' atomics and stores land (a cached load can
 * keep returning an old line of this SM's L1). */
__device__ __forceinline__ unsigned load_l2(const unsigned *p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int load_l2(const int *p) { return (int) load_l2(reinterpret_cast<const unsigned *>(p)); }

#ifdef GB_PROFILE
__device__ long long g_prof3[256][16]; /* finisher thread 0: cycles per phase, summed over its rows */
#define FPROF_INIT() long long fprof_t = clock64()
#define FPROF(i)                                              \
    if (g.tid == 0 && blockIdx.x < 256) {                     \
        const long long t_ = clock64();                       \
        g_prof3[blockIdx.x][i] += t_ - fprof_t;               \
        fprof_t = t_;                                         \
    }
#else
#define FPROF_INIT()
#define FPROF(i)
#endif

__device__ __forceinline__ float key_to_float(unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k); }

/* A set of warps that synchronise on their own named barrier. */
struct Grp {
    int tid, lane, warp; /* position inside the group */
    int n, nw;           /* threads, warps */
    int bar;             /* hardware barrier id (0 is left to __syncthreads) */
    __device__ __forceinline__ void sync() const { asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(n) : "memory"); }
};

/* Reduction scratch, one instance per group. */
struct __align__(16) GroupShared {
    float     wred_f[32];
    int       wred_a[32];
    double    wred_d[32];
    long long wred_l[32];
    int       bins[kHistBins];
    double    S;
    float     tau;
    float     blk_max;
    int       blk_arg;
    int       n_cand;
    int       n_dlist;
    int       n_sel;
    int       n_border;
    int       b_star;
    int       n_hi;
    int       flag;
    int       pick;
    unsigned  tau_key;       /* ordered key of the select threshold */
    int       cur_row;
    float     hmax[kHistBins]; /* finisher: slice maxima of the row */
    int       harg[kHistBins]; /* finisher: their first ids */
};

/* float4 of a slice that one worker warp owns: an equal share, rounded up to whole warp steps */
__host__ __device__ __forceinline__ int share_len(int nv4) { return ((nv4 + kWorkWarps - 1) / kWorkWarps + 31) & ~31; }

/* A work item's configuration, decoded once by the loader warp. */
struct __align__(16) ItemCfg {
    int   row, item, s0, n;         /* what the worker warps read, four words at a time */
    int   mode, kq, flags, pad0;    /* flags: bit 0 = penalties on */
    float inv_t, rep, freq, pres;
    int   L, nv4, c, st0;           /* float4 per warp, float4 in the slice, slice number, status bits of the id list */
    int   H, E, seq, seq0;          /* loader only */
};

/* What the worker warps of one slice add up, each at its own pace. */
struct __align__(8) SliceAcc {
    unsigned long long best;    /* (ordered key of the maximum, ~first id): larger word wins */
    int                n_cand;  /* candidates placed so far */
    int                arrived; /* worker warps that are done with the slice */
    int                st;      /* status bits */
    int                pad;
    float              wmax[32]; /* per warp: maximum of its part ... */
    double             wsum[32]; /* ... and its sum of expf((x - that maximum) * inv_t) */
};

constexpr int kIdSlotBits = 8;
constexpr int kIdSlots    = 1 << kIdSlotBits; /* open-addressing table for at most kLoaderIds ids */
constexpr int kLoaderIds  = 128;              /* ids of a row (history + fed tokens) that the loader warp keeps in registers */
constexpr int kFinQueue = 64; /* completed rows waiting for this CTA's finisher warps */
constexpr int kCfgRing  = 8; /* decoded configurations kept */
constexpr int kListRing = kMaxStages + 1; /* per-slice id lists / accumulators kept: a warp can run at most `stages` slices ahead of another */
constexpr int kLiBits   = 14; /* an id list entry is (position in the slice) | (count << kLiBits) */
static_assert(kSliceMax <= (1 << kLiBits), "slice positions must fit the id list entry");

struct __align__(16) StreamShared {
    unsigned long long full[kMaxStages];  /* the slice has landed (bulk copy -> workers) */
    unsigned long long empty[kMaxStages]; /* every worker warp has lifted its part (workers -> loader) */
    GroupShared        wk; /* workers */
    GroupShared        fn; /* finishers */
    ItemCfg            cfg[kCfgRing];
    SliceAcc           acc[kListRing];
    int                n_dl[kListRing]; /* entries of the slice's id list */
    unsigned           tau_key[2];      /* select threshold of a row's first slice, alternating */
    unsigned           top_key[2];      /* largest group maximum of that slice, alternating */
    unsigned           low_key[2];      /* smallest group maximum of that slice, alternating */
    int                boot_n[2];       /* groups (threads with a share) of that slice, alternating */
    __align__(16) int  bhist[kHistBins]; /* group maxima of that slice, binned by key */
    unsigned long long tau_pub;         /* (row, ordered key of the best threshold known for it): only grows */
    int                id_key[kIdSlots]; /* loader: the distinct ids of the row in preparation ... */
    int                id_cnt[kIdSlots]; /* ... and how often each occurs */
    __align__(16) int  thist[kHistBins]; /* the row's candidates so far, binned by value between threshold and maximum */
    volatile int slice_done[kListRing]; /* j + 1 once every worker warp is done with slice j (workers -> publisher) */
    float        t_lo, t_scale;         /* the candidate histogram's map from value to bin ... */
    int          t_row;                 /* ... and the row it belongs to */
    volatile int q_done;    /* the worker loop has ended */
    volatile int q_error;
    volatile int p_done;    /* the publisher has ended */
    volatile int fin_q[kFinQueue]; /* rows this CTA completed, publisher -> finisher warps */
    volatile int fin_head;  /* rows queued so far */
    volatile int fin_tail;  /* rows taken so far */
    volatile int l_decoded; /* items whose configuration and id list are ready (loader -> workers) */
    int          w_done;    /* slices every worker warp is done with (workers -> loader) */
    int          done_warps;
    int          n_slow;    /* rows left to the multi-pass path at the kernel's end */
};

enum Mode { M_ARGMAX, M_TOPK, M_TOPP, M_TEMP };

constexpr int ST_DEFERRED = 1 << 30; /* inside the kernel only: the row waits for the multi-pass path at the kernel's end */

/* Everything a row needs that does not depend on the slice. */
struct RowCfg {
    int                row, seq0, seq, rr;
    float              T, top_p, inv_t;
    int                top_k, k, kq;
    Mode               mode;
    bool               select_only, pen_on;
    int                H, E;
    float              rep, freq, pres;
    const int         *hrow, *erow;
    unsigned long long rng; /* generator state this row starts from */
    int                draws_per_row;
};

/* The part of a row's configuration that costs memory round trips; workers
 * fetch it one item ahead. */
struct RawCfg {
    int   seq;
    float T, top_p;
    int   top_k, hist_len;
    float rep, freq, pres;
    unsigned long long rng; /* the sequence's generator word (only when asked for) */
};

__device__ __forceinline__ RawCfg raw_config(const SampleParams &p, int row, bool want_rng = false) {
    RawCfg    c;
    const int seq0 = p.rows_per_seq == 1 ? row : row / p.rows_per_seq;
    c.seq          = p.slot ? p.slot[seq0] : seq0;
    c.T            = p.temperature[c.seq];
    c.top_k        = p.top_k[c.seq];
    c.top_p        = p.top_p[c.seq];
    c.hist_len     = p.hist ? p.hist_len[c.seq] : 0;
    c.rep          = p.rep ? p.rep[c.seq] : 1.0f;
    c.freq         = p.freq ? p.freq[c.seq] : 0.0f;
    c.pres         = p.pres ? p.pres[c.seq] : 0.0f;
    c.rng          = (want_rng && p.rng_in) ? p.rng_in[c.seq] : 1ull; /* travels with the other parameters */
    return c;
}

__device__ __forceinline__ RowCfg row_config(const SampleParams &p, int row, const RawCfg &c, bool want_rng) {
    RowCfg r;
    r.row   = row;
    r.seq0  = p.rows_per_seq == 1 ? row : row / p.rows_per_seq;
    r.rr    = row - r.seq0 * p.rows_per_seq;
    r.seq   = c.seq;
    r.T     = c.T;
    r.top_k = c.top_k;
    r.top_p = c.top_p;
    /* head.c:172-183 folded with the early-outs of the three sampler functions */
    if (!(r.T > 0.0f)) {
        r.mode = M_ARGMAX;
    } else if (r.top_k > 1) {
        r.mode = r.top_k >= p.V ? M_TEMP : M_TOPK;
    } else if (r.top_p > 0.0f && r.top_p < 1.0f) {
        r.mode = M_TOPP;
    } else {
        r.mode = M_TEMP;
    }
    r.select_only = (p.flags & F_SELECT_ONLY) != 0;
    r.k           = min(r.top_k, kTopKClamp);
    if (r.select_only) {
        r.mode = M_TOPK;
        r.k    = min(max(r.top_k, 1), min(p.V, kTopKClamp));
    }
    r.kq            = r.mode == M_TOPK ? r.k : (r.mode == M_TOPP ? min(kNucleusProbe, p.V) : 0);
    r.inv_t         = r.T > 0.0f ? __fdiv_rn(1.0f, r.T) : 1.0f;
    r.draws_per_row = (r.T > 0.0f && !r.select_only) ? 1 : 0;
    r.rng           = 1ull;
    if (want_rng) {
        r.rng = c.rng;
        for (int i = 0; i < r.rr * r.draws_per_row; i++) {
            (void) xorshift_next(r.rng);
        }
    }
    r.pen_on = p.hist != nullptr || p.extra != nullptr;
    r.H      = p.hist ? (int) min((long long) max(c.hist_len, 0), p.hist_stride) : 0;
    r.E      = p.extra ? r.rr : 0; /* proposals fed before this row: extra[1..rr] */
    r.rep    = c.rep > 0.0f ? c.rep : 1.0f;
    r.freq   = c.freq;
    r.pres   = c.pres;
    r.hrow   = p.hist ? p.hist + (size_t) r.seq * (size_t) p.hist_stride : nullptr;
    r.erow   = p.extra ? p.extra + (size_t) r.seq0 * (size_t) p.extra_stride : nullptr; /* per call, not per slot */
    return r;
}

__device__ __forceinline__ int hist_id(const RowCfg &r, int j, int vocab_offset) {
    return (j < r.H ? r.hrow[j] : r.erow[1 + j - r.H]) - vocab_offset;
}

__device__ __forceinline__ float penalise(float x, int cnt, float rep, float freq, float pres) {
    x = x > 0.0f ? __fdiv_rn(x, rep) : __fmul_rn(x, rep);
    x = __fsub_rn(x, __fmul_rn((float) cnt, freq));
    return __fsub_rn(x, pres);
}

/*
 * Penalties on a run of n values that hold the global ids [s0, s0 + n). `buf`
 * may be shared or global memory; `bitmap` has (n + 31) / 32 zeroed words;
 * `dlist` has room for `cap` distinct ids; *n_dlist is zero. `first_id` is the
 * caller's pre-fetched history id for j = g.tid (or any value when the caller
 * did not prefetch: have_first = false). All threads of the group call this.
 * Returns status bits.
 */
__device__ int apply_penalties(const Grp &g, float *buf, int s0, int n, const RowCfg &r, int V, int vocab_offset, unsigned *bitmap, PenEntry *dlist, int cap, int *n_dlist,
                               bool have_first, int first_id) {
    int       st    = 0;
    const int total = r.H + r.E;
    auto      id_at = [&](int j) { return (have_first && j == g.tid) ? first_id : hist_id(r, j, vocab_offset); };
    if (r.freq == 0.0f) {
        /* multiplicities do not matter: the first thread to mark an id rewrites it, one pass */
        for (int j = g.tid; j < total; j += g.n) {
            const int id = id_at(j);
            const int li = id - s0;
            if (id >= 0 && id < V && li >= 0 && li < n) {
                const unsigned bit = 1u << (li & 31);
                if (!(atomicOr(&bitmap[li >> 5], bit) & bit)) {
                    buf[li] = penalise(buf[li], 1, r.rep, 0.0f, r.pres);
                }
            }
        }
        g.sync();
        return st;
    }
    /* (a) the first thread to mark an id owns it and saves the original value */
    for (int j = g.tid; j < total; j += g.n) {
        const int id = id_at(j);
        const int li = id - s0;
        if (id >= 0 && id < V && li >= 0 && li < n) {
            const unsigned bit = 1u << (li & 31);
            if (!(atomicOr(&bitmap[li >> 5], bit) & bit)) {
                const int pos = atomicAdd(n_dlist, 1);
                if (pos < cap) {
                    dlist[pos].li   = li;
                    dlist[pos].orig = buf[li];
                }
            }
        }
    }
    g.sync();
    int nd = *n_dlist;
    if (nd > cap) { /* cannot happen when the launcher sized the room; keep the run consistent anyway */
        st |= ST_HIST_OVERFLOW;
        nd = 0;
    }
    /* (b) the slot becomes an integer counter */
    for (int i = g.tid; i < nd; i += g.n) {
        reinterpret_cast<int *>(buf)[dlist[i].li] = 0;
    }
    g.sync();
    if (nd > 0) {
        for (int j = g.tid; j < total; j += g.n) {
            const int id = id_at(j);
            const int li = id - s0;
            if (id >= 0 && id < V && li >= 0 && li < n) {
                atomicAdd(reinterpret_cast<int *>(buf) + li, 1);
            }
        }
    }
    g.sync();
    /* (c) one thread per distinct id writes the penalised value */
    for (int i = g.tid; i < nd; i += g.n) {
        const int li = dlist[i].li;
        buf[li]      = penalise(dlist[i].orig, reinterpret_cast<int *>(buf)[li], r.rep, r.freq, r.pres);
    }
    g.sync();
    return st;
}

/* ------------------------------------------------------- group reductions -- */

/* (max, first id) over the group; every thread gets the result. */
__device__ __forceinline__ void group_argmax(const Grp &g, GroupShared *sh, float &v, int &a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int   oa = __shfl_xor_sync(0xffffffffu, a, o);
        if (pair_before(ov, oa, v, a)) {
            v = ov;
            a = oa;
        }
    }
    g.sync(); /* earlier readers of the scratch are done */
    if (g.lane == 0) {
        sh->wred_f[g.warp] = v;
        sh->wred_a[g.warp] = a;
    }
    g.sync();
    if (g.warp == 0) {
        v = g.lane < g.nw ? sh->wred_f[g.lane] : -CUDART_INF_F;
        a = g.lane < g.nw ? sh->wred_a[g.lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int   oa = __shfl_xor_sync(0xffffffffu, a, o);
            if (pair_before(ov, oa, v, a)) {
                v = ov;
                a = oa;
            }
        }
        if (g.lane == 0) {
            sh->blk_max = v;
            sh->blk_arg = a;
        }
    }
    g.sync();
    v = sh->blk_max;
    a = sh->blk_arg;
}

/* Maximum over the group (values only); one barrier less than group_argmax. */
__device__ __forceinline__ float group_max(const Grp &g, GroupShared *sh, float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    }
    g.sync();
    if (g.lane == 0) {
        sh->wred_f[g.warp] = v;
    }
    g.sync();
    float m = sh->wred_f[0];
    for (int w = 1; w < g.nw; w++) {
        m = fmaxf(m, sh->wred_f[w]);
    }
    return m;
}

/* Every thread gets the same total (fixed order of additions). */
__device__ __forceinline__ double group_sum_d(const Grp &g, GroupShared *sh, double v) {
    v = warp_sum_d(v);
    g.sync(); /* the previous result has been read */
    if (g.lane == 0) {
        sh->wred_d[g.warp] = v;
    }
    g.sync();
    double t = 0.0;
    for (int w = 0; w < g.nw; w++) {
        t += sh->wred_d[w];
    }
    return t;
}

__device__ __forceinline__ long long group_sum_ll(const Grp &g, GroupShared *sh, long long v) {
    v = warp_sum_ll(v);
    g.sync();
    if (g.lane == 0) {
        sh->wred_l[g.warp] = v;
    }
    g.sync();
    long long t = 0;
    for (int w = 0; w < g.nw; w++) {
        t += sh->wred_l[w];
    }
    return t;
}

/* ------------------------------------------- finisher: ordered select of kq -- */

/*
 * cand[0..total) hold distinct ids, total >= kq >= 1. Writes the kq best in
 * (value desc, id asc) order to sorted[0..kq). A histogram over the
 * candidates' key range finds the bin that holds the kq-th entry; entries in
 * higher bins are in, only that one bin is ranked exactly. tmp has room for
 * `total` pairs. Called by the whole group.
 */
__device__ void select_sorted(const Grp &g, GroupShared *sh, const Pair *cand, int total, int kq, Pair *tmp, Pair *sorted) {
    unsigned lo = 0xffffffffu, hi = 0u;
    for (int i = g.tid; i < total; i += g.n) {
        const unsigned key = order_key(cand[i].v);
        lo                 = min(lo, key);
        hi                 = max(hi, key);
    }
    lo = __reduce_min_sync(0xffffffffu, lo);
    hi = __reduce_max_sync(0xffffffffu, hi);
    g.sync();
    if (g.lane == 0) {
        sh->wred_a[g.warp]                               = (int) lo;
        reinterpret_cast<unsigned *>(sh->wred_f)[g.warp] = hi;
    }
    for (int i = g.tid; i < kHistBins; i += g.n) {
        sh->bins[i] = 0;
    }
    if (g.tid == 0) {
        sh->n_sel    = 0;
        sh->n_border = 0;
        sh->b_star   = 0;
        sh->n_hi     = 0;
    }
    g.sync();
    lo = 0xffffffffu;
    hi = 0u;
    for (int w = 0; w < g.nw; w++) {
        lo = min(lo, (unsigned) sh->wred_a[w]);
        hi = max(hi, reinterpret_cast<unsigned *>(sh->wred_f)[w]);
    }
    const unsigned range = hi >= lo ? hi - lo : 0u;
    const int      shift = max(0, (32 - __clz(range)) - 8); /* (range >> shift) < 256 */
    for (int i = g.tid; i < total; i += g.n) {
        atomicAdd(&sh->bins[(order_key(cand[i].v) - lo) >> shift], 1);
    }
    g.sync();
    if (g.warp == 0) {
        /* b* = largest bin with count(bins >= b*) >= kq; lane l owns bins [8l, 8l+8) */
        int mine = 0;
#pragma unroll
        for (int q = 0; q < 8; q++) {
            mine += sh->bins[8 * g.lane + q];
        }
        int suffix = mine; /* entries owned by this lane and all higher ones */
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int dn = __shfl_down_sync(0xffffffffu, suffix, o);
            if (g.lane + o < 32) {
                suffix += dn;
            }
        }
        const int above = suffix - mine; /* entries owned by higher lanes */
        if (above < kq && above + mine >= kq) {
            int acc = above;
            for (int q = 7; q >= 0; q--) {
                const int c = sh->bins[8 * g.lane + q];
                if (acc + c >= kq) {
                    sh->b_star = 8 * g.lane + q;
                    sh->n_hi   = acc;
                    break;
                }
                acc += c;
            }
        }
    }
    g.sync();
    const int b_star = sh->b_star, n_hi = sh->n_hi;
    /* entries above the bin fill tmp from the front, the bin's entries from the back */
    for (int i = g.tid; i < total; i += g.n) {
        const int bin = (int) ((order_key(cand[i].v) - lo) >> shift);
        if (bin > b_star) {
            tmp[atomicAdd(&sh->n_sel, 1)] = cand[i];
        } else if (bin == b_star) {
            tmp[total - 1 - atomicAdd(&sh->n_border, 1)] = cand[i];
        }
    }
    g.sync();
    const int nb   = sh->n_border;
    const int need = kq - n_hi;
    for (int i = g.tid; i < nb; i += g.n) {
        const Pair me   = tmp[total - 1 - i];
        int        rank = 0;
        for (int j = 0; j < nb; j++) {
            const Pair o = tmp[total - 1 - j];
            rank += pair_before(o.v, o.idx, me.v, me.idx) ? 1 : 0;
        }
        if (rank < need) {
            sorted[n_hi + rank] = me;
        }
    }
    for (int i = g.tid; i < n_hi; i += g.n) {
        const Pair me   = tmp[i];
        int        rank = 0;
        for (int j = 0; j < n_hi; j++) {
            rank += pair_before(tmp[j].v, tmp[j].idx, me.v, me.idx) ? 1 : 0;
        }
        sorted[rank] = me;
    }
    g.sync();
}

/* ------------------------------------------------- multi-pass path (finisher) -- */

template <class F>
__device__ __forceinline__ void row_sweep(const Grp &g, const float *row, int V, F &&f) {
    const int     V4 = V >> 2;
    const float4 *p4 = reinterpret_cast<const float4 *>(row);
    int           j  = g.tid;
    for (; j + 3 * g.n < V4; j += 4 * g.n) { /* four loads in flight per thread */
        const float4 a = p4[j], b = p4[j + g.n], c = p4[j + 2 * g.n], d = p4[j + 3 * g.n];
        f(a.x, 4 * j), f(a.y, 4 * j + 1), f(a.z, 4 * j + 2), f(a.w, 4 * j + 3);
        f(b.x, 4 * (j + g.n)), f(b.y, 4 * (j + g.n) + 1), f(b.z, 4 * (j + g.n) + 2), f(b.w, 4 * (j + g.n) + 3);
        f(c.x, 4 * (j + 2 * g.n)), f(c.y, 4 * (j + 2 * g.n) + 1), f(c.z, 4 * (j + 2 * g.n) + 2), f(c.w, 4 * (j + 2 * g.n) + 3);
        f(d.x, 4 * (j + 3 * g.n)), f(d.y, 4 * (j + 3 * g.n) + 1), f(d.z, 4 * (j + 3 * g.n) + 2), f(d.w, 4 * (j + 3 * g.n) + 3);
    }
    for (; j < V4; j += g.n) {
        const float4 x = p4[j];
        f(x.x, 4 * j);
        f(x.y, 4 * j + 1);
        f(x.z, 4 * j + 2);
        f(x.w, 4 * j + 3);
    }
    for (int i = (V4 << 2) + g.tid; i < V; i += g.n) {
        f(row[i], i);
    }
}

template <class F>
__device__ __forceinline__ void row_rewrite(const Grp &g, float *row, int V, F &&f) {
    for (int i = g.tid; i < V; i += g.n) {
        row[i] = f(row[i], i);
    }
}

/* Largest composite word t such that at least `want` entries are >= t. */
__device__ unsigned long long bisect_rank(const Grp &g, GroupShared *sh, const float *row, int V, int idx_bits, long long want) {
    unsigned long long prefix = 0;
    for (int bit = 31 + idx_bits; bit >= 0; bit--) {
        const unsigned long long t   = prefix | (1ull << bit);
        long long                cnt = 0;
        row_sweep(g, row, V, [&](float x, int i) { cnt += composite(order_key(x), i, idx_bits) >= t ? 1 : 0; });
        if (group_sum_ll(g, sh, cnt) >= want) {
            prefix = t;
        }
    }
    return prefix;
}

/* Largest composite word t with mass{word >= t} >= target (inclusive) or > target. The search may
 * start from a known prefix of the word: the bits above top_bit are taken from `prefix`. */
template <class KeyF, class MassF>
__device__ unsigned long long bisect_mass(const Grp &g, GroupShared *sh, const float *row, int V, int idx_bits, double target, bool inclusive, KeyF &&key, MassF &&mass,
                                          unsigned long long prefix = 0ull, int top_bit = -1) {
    for (int bit = top_bit >= 0 ? top_bit : 31 + idx_bits; bit >= 0; bit--) {
        const unsigned long long t = prefix | (1ull << bit);
        double                   m = 0.0;
        row_sweep(g, row, V, [&](float x, int i) {
            if (composite(key(x), i, idx_bits) >= t) {
                m += mass(x, i);
            }
        });
        const double tot = group_sum_d(g, sh, m);
        if (inclusive ? (tot >= target) : (tot > target)) {
            prefix = t;
        }
    }
    return prefix;
}

/* Where a walk over the row in descending key order first reaches a target mass. */
struct RadixOut {
    bool      found;  /* false: the whole row stays below the target */
    unsigned  key;    /* the key at which the running mass crosses */
    double    above;  /* mass of the entries with a larger key */
    long long n_above; /* how many those are */
    long long ties;   /* entries with exactly this key (and mass > 0) */
};

/*
 * The same answer as the top 32 bits of bisect_mass, in four sweeps instead of thirty-two: one
 * byte of the key per sweep, masses and counts per byte value in shared memory (`copies` private
 * histograms, one per warp where the room allows), then a scan from the top value down. hm / hc
 * hold copies * 256 doubles / ints.
 */
template <bool kUnit = false, class KeyF, class MassF>
__device__ RadixOut radix_mass(const Grp &g, GroupShared *sh, double *hm, int *hc, int copies, const float *row, int V, double target, bool inclusive, KeyF &&key,
                               MassF &&mass) {
    RadixOut out;
    out.found   = true;
    out.key     = 0u;
    out.above   = 0.0;
    out.n_above = 0;
    out.ties    = 0;
    for (int level = 3; level >= 0; level--) {
        const int shift = 8 * level;
        for (int i = g.tid; i < copies * 256; i += g.n) {
            hm[i] = 0.0;
            hc[i] = 0;
        }
        g.sync();
        double        *mym = hm + (g.warp % copies) * 256;
        int           *myc = hc + (g.warp % copies) * 256;
        const unsigned pre = out.key;
        row_sweep(g, row, V, [&](float x, int i) {
            const unsigned k = key(x);
            if (level == 3 || (k >> (shift + 8)) == (pre >> (shift + 8))) {
                const unsigned d = (k >> shift) & 255u;
                if (kUnit) { /* every entry weighs one: the counts are the masses */
                    atomicAdd(&myc[d], 1);
                } else {
                    const double m = mass(x, i);
                    if (m > 0.0) {
                        atomicAdd(&mym[d], m);
                        atomicAdd(&myc[d], 1);
                    }
                }
            }
        });
        g.sync();
        if (g.warp == 0) {
            /* lane l owns the byte values 255 - 8 l down to 248 - 8 l: the walk order */
            double m8[8];
            int    c8[8];
            double lane_m = 0.0;
            int    lane_c = 0;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const int b = 255 - (8 * g.lane + q);
                m8[q]       = 0.0;
                c8[q]       = 0;
                for (int w = 0; w < copies; w++) {
                    m8[q] += hm[w * 256 + b];
                    c8[q] += hc[w * 256 + b];
                }
                if (kUnit) {
                    m8[q] = (double) c8[q];
                }
                lane_m += m8[q];
                lane_c += c8[q];
            }
            double incl_m = lane_m;
            int    incl_c = lane_c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double um = __shfl_up_sync(0xffffffffu, incl_m, o);
                const int    uc = __shfl_up_sync(0xffffffffu, incl_c, o);
                if (g.lane >= o) {
                    incl_m += um;
                    incl_c += uc;
                }
            }
            const double   before = out.above + (incl_m - lane_m);
            const bool     cross  = inclusive ? (before + lane_m >= target) : (before + lane_m > target);
            const unsigned ball   = __ballot_sync(0xffffffffu, cross);
            if (ball == 0u) {
                if (g.lane == 0) {
                    sh->b_star = -1;
                }
            } else if (g.lane == __ffs(ball) - 1) {
                double run = before;
                int    cnt = incl_c - lane_c;
                int    b   = 255 - 8 * g.lane - 7;
                int    tc  = c8[7];
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const bool hit = inclusive ? (run + m8[q] >= target) : (run + m8[q] > target);
                    if (hit) {
                        b  = 255 - (8 * g.lane + q);
                        tc = c8[q];
                        break;
                    }
                    run += m8[q];
                    cnt += c8[q];
                }
                sh->b_star = b;
                sh->S      = run;
                sh->n_hi   = cnt;
                sh->n_sel  = tc;
            }
        }
        g.sync();
        if (sh->b_star < 0) {
            out.found = false;
            g.sync();
            return out;
        }
        out.key |= (unsigned) sh->b_star << shift;
        out.above = sh->S;
        out.n_above += (long long) sh->n_hi;
        out.ties = (long long) sh->n_sel;
        g.sync();
    }
    return out;
}

/*
 * From the key at which a walk crosses to the composite word of the crossing entry: entries with
 * equal keys are walked by ascending id, and `j` of them (1-based) are needed. One of a kind: one
 * sweep finds its id. Several: the low bits of the word are bisected as before.
 */
template <class KeyF, class MassF>
__device__ unsigned long long resolve_ties(const Grp &g, GroupShared *sh, const float *row, int V, int idx_bits, const RadixOut &ro, double target, bool inclusive, KeyF &&key,
                                           MassF &&mass) {
    if (ro.ties <= 1) {
        if (g.tid == 0) {
            sh->pick = 0x7fffffff;
        }
        g.sync();
        row_sweep(g, row, V, [&](float x, int i) {
            if (key(x) == ro.key && mass(x, i) > 0.0) {
                atomicMin(&sh->pick, i);
            }
        });
        g.sync();
        const int id = sh->pick;
        g.sync();
        return composite(ro.key, id == 0x7fffffff ? 0 : id, idx_bits);
    }
    return bisect_mass(g, sh, row, V, idx_bits, target, inclusive, key, mass, (unsigned long long) ro.key << idx_bits, idx_bits - 1);
}

/* All threads of the CTA serve a row whose kept set does not fit the one-pass path. */
__device__ int multipass_row(const Grp &g, const SampleParams &p, GroupShared *sh, RowCfg &r, float row_max, int row_arg, void *hist_mem, int hist_bytes) {
    /* room for the byte histograms of the radix walks: per warp where it fits, else one for all */
    const int copies = hist_bytes >= g.nw * 256 * 12 ? g.nw : 1;
    double   *hm     = reinterpret_cast<double *>(hist_mem);
    int      *hc     = reinterpret_cast<int *>(hm + copies * 256);
    const int    V        = p.V;
    const int    idx_bits = 32 - __clz(max(V - 1, 1));
    int          st       = ST_SLOW_PATH;
    float       *gr       = p.gen_rows + (size_t) blockIdx.x * (size_t) p.gen_stride;
    const float *src      = p.logits + (size_t) r.row * (size_t) p.row_stride;
    int         *kept_i   = p.kept_cap > 0 ? p.kept_idx + (size_t) r.row * (size_t) p.kept_cap : nullptr;
    float       *kept_v   = p.kept_cap > 0 ? p.kept_val + (size_t) r.row * (size_t) p.kept_cap : nullptr;
    /* private copy of the row, penalties applied once */
    if (p.aligned) { /* rows start on 16-byte boundaries: four values per load */
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        float4       *d4 = reinterpret_cast<float4 *>(gr);
        for (int i = g.tid; i < (V >> 2); i += g.n) {
            d4[i] = s4[i];
        }
        for (int i = (V & ~3) + g.tid; i < V; i += g.n) {
            gr[i] = src[i];
        }
    } else {
        for (int i = g.tid; i < V; i += g.n) {
            gr[i] = src[i];
        }
    }
    if (r.pen_on) {
        unsigned *bm = p.gen_bitmap + (size_t) blockIdx.x * (size_t) p.gen_bitmap_words;
        for (int i = g.tid; i < p.gen_bitmap_words; i += g.n) {
            bm[i] = 0u;
        }
        if (g.tid == 0) {
            sh->n_dlist = 0;
        }
        g.sync();
        st |= apply_penalties(g, gr, 0, V, r, V, p.vocab_offset, bm, reinterpret_cast<PenEntry *>(p.gen_dlist + (size_t) blockIdx.x * (size_t) p.gen_hist_cap), p.gen_hist_cap,
                              &sh->n_dlist, false, 0);
    } else {
        g.sync();
    }
    /* the fast path's slice records need not carry the maximum: take it from the copy */
    row_max = -CUDART_INF_F;
    row_arg = 0x7fffffff;
    row_sweep(g, gr, V, [&](float x, int i) {
        if (row_arg == 0x7fffffff || pair_before(x, i, row_max, row_arg)) {
            row_max = x;
            row_arg = i;
        }
    });
    group_argmax(g, sh, row_max, row_arg);
    if (r.mode == M_TOPK) {
        /* the k-th entry in (value desc, id asc) order: a radix walk on counts, then the ids of its ties */
        auto                     okey   = [](float x) { return order_key(x); };
        auto                     one    = [](float, int) { return 1.0; };
        const RadixOut           rs     = radix_mass<true>(g, sh, hm, hc, copies, gr, V, (double) r.k, true, okey, one);
        const unsigned long long t_set  = rs.found ? resolve_ties(g, sh, gr, V, idx_bits, rs, (double) r.k, true, okey, one) : 0ull;
        auto                     in_set = [&](float x, int i) { return composite(order_key(x), i, idx_bits) >= t_set; };
        if (r.select_only) {
            if (g.tid == 0) {
                sh->n_sel = 0;
            }
            g.sync();
            row_sweep(g, gr, V, [&](float x, int i) {
                if (in_set(x, i)) {
                    const int pos = atomicAdd(&sh->n_sel, 1);
                    if (pos < p.kept_cap) {
                        kept_i[pos] = i + p.vocab_offset;
                        kept_v[pos] = x;
                    }
                }
            });
            if (g.tid == 0) {
                p.kept_n[r.row] = r.k;
                p.tokens[r.row] = row_arg + p.vocab_offset;
            }
        } else {
            auto   qof = [&](float x) { return (double) exp_exact(scaled_arg(x, row_max, r.inv_t)); };
            double m   = 0.0;
            row_sweep(g, gr, V, [&](float x, int i) {
                if (in_set(x, i)) {
                    m += qof(x);
                }
            });
            const double S = group_sum_d(g, sh, m);
            const double u = (double) unit_from(xorshift_next(r.rng)) * S;
            /* the pick is the earliest walk position whose running sum exceeds u: the largest
             * word t with mass{word >= t} > u */
            auto                     qmass  = [&](float x, int i) { return in_set(x, i) ? qof(x) : 0.0; };
            const RadixOut           rp     = radix_mass(g, sh, hm, hc, copies, gr, V, u, false, okey, qmass);
            unsigned long long       t_pick = rp.found ? resolve_ties(g, sh, gr, V, idx_bits, rp, u, false, okey, qmass) : 0ull;
            if (t_pick < t_set) {
                t_pick = t_set;
            }
            row_sweep(g, gr, V, [&](float x, int i) {
                if (composite(order_key(x), i, idx_bits) == t_pick) {
                    p.tokens[r.row] = i + p.vocab_offset;
                }
            });
            if (g.tid == 0 && p.kept_cap > 0) {
                p.kept_n[r.row] = r.k;
            }
            if (p.kept_cap > 0) {
                st |= ST_KEPT_PARTIAL;
            }
        }
    } else {
        /* top-p with any nucleus size: the copy becomes e_i, then p_i (sampler.c:245-255) */
        double acc = 0.0;
        /* e_i as a correctly rounded expf gives it: with a nucleus of tens of thousands of ids an
         * exponential that is off by a fraction of an ulp on average moves the running sum by more than
         * the distance between two neighbours of the walk */
        row_rewrite(g, gr, V, [&](float x, int) {
            const float e = exp_exact(scaled_arg(x, row_max, r.inv_t));
            acc += (double) e;
            return e;
        });
        const double S = group_sum_d(g, sh, acc);
        row_rewrite(g, gr, V, [&](float e, int) { return __double2float_rn((double) e / S); });
        g.sync();
        auto keyf  = [](float pv) { return __float_as_uint(pv); }; /* p >= 0: the bits are ordered */
        auto massf = [](float pv, int) { return (double) pv; };
        /* cutoff: first walk position whose running sum reaches top_p, inclusive */
        /* The radix walks look at a window of keys stretched over all 32 bits, so that the entries
         * spread over the byte values instead of piling up in a few. Cutoff: entries with
         * p < (1 - top_p) / V add up to less than 1 - top_p, so the walk crosses above them. */
        auto windowed = [&](unsigned k_lo, unsigned k_hi, double target, bool inclusive, auto &&mass_in) {
            const unsigned span = k_hi > k_lo ? k_hi - k_lo : 0u;
            const int      ls   = span > 0u ? __clz(span) : 0;
            auto           kw   = [&](float pv) {
                const unsigned k = keyf(pv);
                return k >= k_lo ? (min(k, k_hi) - k_lo) << ls : 0u;
            };
            auto mw = [&](float pv, int i) { return keyf(pv) >= k_lo ? mass_in(pv, i) : 0.0; };
            RadixOut ro = radix_mass(g, sh, hm, hc, copies, gr, V, target, inclusive, kw, mw);
            ro.key      = (ro.key >> ls) + k_lo; /* back to the key itself */
            return ro;
        };
        const unsigned k_top   = keyf(__double2float_rn(1.0 / S)); /* the largest p: e = 1 at the row maximum */
        const float    p_floor = __double2float_rn(0.5 * (1.0 - (double) r.top_p) / (double) V);
        const unsigned k_floor = (p_floor > 0.0f && keyf(p_floor) < k_top) ? keyf(p_floor) : 0u;
        RadixOut       rc      = windowed(k_floor, k_top, (double) r.top_p, true, massf);
        if (!rc.found && k_floor != 0u) {
            rc = windowed(0u, k_top, (double) r.top_p, true, massf); /* rounding kept the window short of top_p */
        }
        const unsigned long long t_cut = rc.found ? resolve_ties(g, sh, gr, V, idx_bits, rc, (double) r.top_p, true, keyf, massf) : 0ull;
        double                   nm    = 0.0;
        long long                ncnt  = 0;
        row_sweep(g, gr, V, [&](float pv, int i) {
            if (composite(keyf(pv), i, idx_bits) >= t_cut) {
                nm += (double) pv;
                ncnt++;
            }
        });
        const double       N      = group_sum_d(g, sh, nm);
        const long long    cut    = group_sum_ll(g, sh, ncnt);
        const double       u      = (double) unit_from(xorshift_next(r.rng)) * N;
        auto               nmass  = [&](float pv, int i) { return composite(keyf(pv), i, idx_bits) >= t_cut ? (double) pv : 0.0; };
        const RadixOut     rk     = windowed((unsigned) (t_cut >> idx_bits), k_top, u, false, nmass);
        unsigned long long t_pick = rk.found ? resolve_ties(g, sh, gr, V, idx_bits, rk, u, false, keyf, nmass) : 0ull;
        if (t_pick < t_cut) {
            t_pick = t_cut; /* default: the last nucleus entry (sampler.c:292) */
        }
        row_sweep(g, gr, V, [&](float pv, int i) {
            if (composite(keyf(pv), i, idx_bits) == t_pick) {
                p.tokens[r.row] = i + p.vocab_offset;
            }
        });
        if (g.tid == 0 && p.kept_cap > 0) {
            p.kept_n[r.row] = (int) cut;
        }
        if (p.kept_cap > 0) {
            st |= ST_KEPT_PARTIAL;
        }
    }
    g.sync();
    return st;
}

/* ---------------------------------------------------------------- finisher -- */

struct FinBuffers {
    Pair     *fcand, *ftmp, *fsort;
    float    *fq;
    unsigned *bitmap; /* 16 words: ids of one walked segment */
    PenEntry *dlist;
    int       dlist_cap;
};

/* What the finisher warps request from global scratch the moment a row is theirs, so that it
 * travels while the row's configuration is still being read. */
static_assert(kFinThreads * 8 >= 1024, "the finisher threads walk a crossing segment of up to 1024 entries, 8 each");
constexpr int kSpecSlots = 8; /* per finisher thread: candidates fetched before the slices' counts are known */
/* how many of each slice's candidates that is (0: the row has too many slices) */
__device__ __forceinline__ int spec_per_slice(const SampleParams &p) {
    return p.n_slices * 64 <= kFinThreads * kSpecSlots ? 64 : (p.n_slices * 48 <= kFinThreads * kSpecSlots ? 48 : 0);
}
/* flat index of the request -> (slice, position) */
__device__ __forceinline__ void spec_split(int f, int k_spec, int &cc, int &i) {
    if (k_spec == 64) {
        cc = f >> 6;
        i  = f & 63;
    } else {
        cc = f / 48;
        i  = f - cc * 48;
    }
}
struct Prefetch {
    int4      hdr;              /* slice record header {max, arg, n_cand, st} of slice g.tid */
    long long c[kSpecSlots];    /* candidate (value, id) pairs, flat index g.tid + kFinThreads * m */
    double    seg;              /* temperature rows: segment sum number g.tid of the row */
};

__device__ __forceinline__ Prefetch prefetch_row(const Grp &g, const SampleParams &p, int row) {
    Prefetch        pf;
    const SliceRec *recs = p.recs + (size_t) row * (size_t) p.n_slices;
    pf.hdr               = make_int4(0, 0, 0, 0);
    if (g.tid < p.n_slices) {
        pf.hdr = __ldcg(reinterpret_cast<const int4 *>(&recs[g.tid]));
    }
    pf.seg = 0.0;
    if (g.tid < p.n_slices * kWorkWarps) {
        pf.seg = __ldcg(&recs[g.tid / kWorkWarps].seg[g.tid % kWorkWarps]);
    }
    const int   kSpec = spec_per_slice(p);
    const int   flat  = p.n_slices * kSpec;
    const Pair *base = p.cands + (size_t) row * (size_t) p.n_slices * (size_t) p.cand_cap;
#pragma unroll
    for (int m = 0; m < kSpecSlots; m++) {
        const int f = g.tid + kFinThreads * m;
        pf.c[m]     = 0;
        if (f < flat) {
            int cc, i;
            spec_split(f, kSpec, cc, i);
            pf.c[m] = __ldcg(reinterpret_cast<const long long *>(base + (size_t) cc * (size_t) p.cand_cap + i));
        }
    }
    return pf;
}

/* Warp 0 of the group: S = sum of w[0..n) and the first i with u(S) < w[0] + .. + w[i] (n - 1 if
 * none), for n <= 256. u01 is the unit draw; the comparison is made against u01 * S like the
 * reference's inverse CDF (sampler.c:90-102). Sums are formed lane-wise and scanned across the
 * warp in double precision. Returns through *S_out and the return value (valid in every lane). */
__device__ __forceinline__ int warp_inverse_cdf(int lane, const float *w, int n, float u01, double *S_out) {
    const int per = (n + 31) / 32; /* <= 8 consecutive weights per lane */
    const int b   = lane * per;
    double    mine = 0.0;
    for (int i = b; i < min(b + per, n); i++) {
        mine += (double) w[i];
    }
    double incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) {
            incl += up;
        }
    }
    const double   S    = __shfl_sync(0xffffffffu, incl, 31);
    const double   u    = (double) u01 * S;
    const unsigned ball = __ballot_sync(0xffffffffu, b < n && u < incl);
    int            pick = n - 1;
    if (ball != 0u) {
        const int src = __ffs(ball) - 1;
        int       f   = n - 1;
        if (lane == src) {
            double a = incl - mine;
            f        = min(b + per, n) - 1;
            for (int i = b; i < min(b + per, n); i++) {
                a += (double) w[i];
                if (u < a) {
                    f = i;
                    break;
                }
            }
        }
        pick = __shfl_sync(0xffffffffu, f, src);
    }
    *S_out = S;
    return pick;
}

/* Runs in the finisher warps of the CTA that completed the row. Returns the row's status bits. */
__device__ int finish_row(const Grp &g, const SampleParams &p, GroupShared *sh, RowCfg &r, const FinBuffers &fb, const Prefetch &pf) {
    const int       row    = r.row;
    const SliceRec *recs   = p.recs + (size_t) row * (size_t) p.n_slices;
    int            *kept_i = p.kept_cap > 0 ? p.kept_idx + (size_t) row * (size_t) p.kept_cap : nullptr;
    float          *kept_v = p.kept_cap > 0 ? p.kept_val + (size_t) row * (size_t) p.kept_cap : nullptr;
    int             st     = 0;
    FPROF_INIT();

    /* slice headers into shared memory; every thread then derives the row's maximum, its first id,
     * the status bits and the candidate totals from them */
    const bool small_row = p.n_slices <= kHistBins;
    g.sync();
    if (small_row) {
        for (int cc = g.tid; cc < p.n_slices; cc += g.n) {
            const int4 h = cc == g.tid ? pf.hdr : __ldcg(reinterpret_cast<const int4 *>(&recs[cc]));
            sh->hmax[cc] = __int_as_float(h.x);
            sh->harg[cc] = h.y;
            sh->bins[cc] = h.z;
            st |= h.w;
        }
    }
    st = __reduce_or_sync(0xffffffffu, st);
    if (g.lane == 0) {
        sh->wred_a[g.warp] = st;
    }
    g.sync();
    for (int w = 0; w < g.nw; w++) {
        st |= sh->wred_a[w];
    }
    float row_max  = -CUDART_INF_F;
    int   row_arg  = 0x7fffffff;
    int   total    = 0;
    bool  overflow = false;
    if (small_row) {
        for (int cc = 0; cc < p.n_slices; cc++) {
            const float m = sh->hmax[cc];
            const int   a = sh->harg[cc];
            if (row_arg == 0x7fffffff || pair_before(m, a, row_max, row_arg)) {
                row_max = m;
                row_arg = a;
            }
            const int nc = sh->bins[cc];
            overflow |= nc > p.cand_cap;
            total += nc;
        }
    } else {
        /* very long rows: the records are read straight from global memory */
        int rst = 0;
        for (int cc = g.tid; cc < p.n_slices; cc += g.n) {
            const int4  h = __ldcg(reinterpret_cast<const int4 *>(&recs[cc]));
            const float m = __int_as_float(h.x);
            rst |= h.w;
            if (row_arg == 0x7fffffff || pair_before(m, h.y, row_max, row_arg)) {
                row_max = m;
                row_arg = h.y;
            }
        }
        rst = __reduce_or_sync(0xffffffffu, rst);
        g.sync();
        if (g.lane == 0) {
            sh->wred_l[g.warp] = rst;
        }
        group_argmax(g, sh, row_max, row_arg);
        for (int w = 0; w < g.nw; w++) {
            st |= (int) sh->wred_l[w];
        }
    }
    auto slice_max = [&](int cc) { return small_row ? sh->hmax[cc] : __ldcg(&recs[cc].max); };

    if (r.mode == M_ARGMAX) {
        if (g.tid == 0) {
            p.tokens[row] = row_arg + p.vocab_offset;
            if (p.kept_cap > 0) {
                p.kept_n[row] = 0;
            }
        }
        return st;
    }

    if (r.mode == M_TEMP) {
        /* segment sums, rescaled from their slice maximum to the row maximum, in id order */
        const int nseg   = p.n_slices * kWorkWarps;
        auto      seg_at = [&](int t) {
            const int   cc = t / kWorkWarps;
            const float m  = slice_max(cc);
            const double sc = m == -CUDART_INF_F ? 0.0 : exp(((double) m - (double) row_max) * (double) r.inv_t);
            return sc * (t == g.tid ? pf.seg : __ldcg(&recs[cc].seg[t % kWorkWarps]));
        };
        double part = 0.0;
        for (int t = g.tid; t < nseg; t += g.n) {
            part += seg_at(t);
        }
        const double S     = group_sum_d(g, sh, part);
        FPROF(2); /* temperature: headers + segment sums */
        const double u     = (double) unit_from(xorshift_next(r.rng)) * S;
        double       carry = 0.0;
        int          found = -1;
        double       fbase = -CUDART_INF; /* nothing crosses: the walk ends on its last id */
        for (int t0 = 0; t0 < nseg; t0 += g.n) {
            const int    t    = t0 + g.tid;
            const double val  = t < nseg ? seg_at(t) : 0.0;
            double       incl = val;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, incl, o);
                if (g.lane >= o) {
                    incl += up;
                }
            }
            g.sync();
            if (g.lane == 31) {
                sh->wred_d[g.warp] = incl;
            }
            if (g.tid == 0) {
                sh->pick = 0x7fffffff;
            }
            g.sync();
            double woff = carry;
            for (int w = 0; w < g.warp; w++) {
                woff += sh->wred_d[w];
            }
            incl += woff;
            if (t < nseg && u < incl) {
                atomicMin(&sh->pick, t);
            }
            g.sync();
            const int pk = sh->pick;
            if (pk != 0x7fffffff) {
                if (t == pk) {
                    sh->S = incl - val;
                }
                g.sync();
                found = pk;
                fbase = sh->S;
                break;
            }
            for (int w = 0; w < g.nw; w++) {
                carry += sh->wred_d[w];
            }
        }
        if (found < 0) {
            found = nseg - 1;
        }
        FPROF(3); /* temperature: scan to the crossing segment */
        /* the crossing segment, re-read from the row (L2), penalised, walked with the row maximum */
        const int    cc    = found / kWorkWarps, w = found % kWorkWarps;
        const int    s0c   = cc * p.slice;
        const int    nc    = max(0, min(p.slice, p.V - s0c));
        const int    nv4c  = (nc + 3) >> 2;
        const int    Lc    = share_len(nv4c);
        const int    e0    = min(4 * w * Lc, nc);
        const int    e1    = min(4 * min((w + 1) * Lc, nv4c), nc);
        const int    seg_n = max(e1 - e0, 0);
        float       *wbuf  = reinterpret_cast<float *>(fb.fcand); /* >= 512 floats */
        const float *src   = p.logits + (size_t) row * (size_t) p.row_stride + s0c + e0;
        g.sync();
        for (int i = g.tid; i < seg_n; i += g.n) {
            wbuf[i] = src[i];
        }
        if (r.pen_on) {
            for (int i = g.tid; i < kFinBitmapWords; i += g.n) {
                fb.bitmap[i] = 0u;
            }
            if (g.tid == 0) {
                sh->n_dlist = 0;
            }
        }
        g.sync();
        if (r.pen_on && seg_n > 0) {
            st |= apply_penalties(g, wbuf, s0c + e0, seg_n, r, p.V, p.vocab_offset, fb.bitmap, fb.dlist, fb.dlist_cap, &sh->n_dlist, false, 0);
        }
        FPROF(4); /* temperature: segment loaded and penalised */
        {
            /* every thread takes a run of consecutive entries; the runs' sums are scanned over the
             * group and the thread whose run crosses u walks it */
            const int per = (seg_n + g.n - 1) / g.n; /* <= 8 for 128 threads */
            const int i0  = g.tid * per;
            float     ev[8];
            double    mine = 0.0;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const int i = i0 + q;
                ev[q]       = (q < per && i < seg_n) ? expf(scaled_arg(wbuf[i], row_max, r.inv_t)) : 0.0f;
                mine += (double) ev[q];
            }
            double incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, incl, o);
                if (g.lane >= o) {
                    incl += up;
                }
            }
            g.sync();
            if (g.lane == 31) {
                sh->wred_d[g.warp] = incl;
            }
            if (g.tid == 0) {
                sh->pick = 0x7fffffff;
            }
            g.sync();
            double base = fbase;
            for (int w = 0; w < g.warp; w++) {
                base += sh->wred_d[w];
            }
            if (u < base + incl && i0 < seg_n) {
                atomicMin(&sh->pick, g.tid);
            }
            g.sync();
            const int pk = sh->pick;
            if (pk == 0x7fffffff) {
                if (g.tid == 0) { /* regrouped sums can end a hair below the segment's share */
                    p.tokens[row] = s0c + e0 + max(seg_n - 1, 0) + p.vocab_offset;
                }
            } else if (g.tid == pk) {
                double a   = base + (incl - mine);
                int    hit = min(i0 + per - 1, seg_n - 1);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    a += (double) ev[q];
                    if (q < per && u < a) {
                        hit = i0 + q;
                        break;
                    }
                }
                p.tokens[row] = s0c + e0 + min(hit, seg_n - 1) + p.vocab_offset;
            }
            if (g.tid == 0 && p.kept_cap > 0) {
                p.kept_n[row] = 0;
            }
        }
        g.sync();
        FPROF(5); /* temperature: walk */
        return st;
    }

    FPROF(2); /* headers, row maximum */
    /* ---- top-k and top-p: merge the slices' candidates ---- */
    bool need_multipass = !(r.kq > 0 && r.kq <= kFastKMax) || !small_row || overflow || total > p.fin_cap || total < r.kq;
    if (!need_multipass) {
        /* place the pre-fetched candidates, then fetch what the pre-fetch did not cover */
        const int  kSpec = spec_per_slice(p);
        const bool spec  = kSpec > 0;
        if (spec) {
#pragma unroll
            for (int m = 0; m < kSpecSlots; m++) {
                const int f = g.tid + kFinThreads * m;
                if (f < p.n_slices * kSpec) {
                    int cc, i;
                    spec_split(f, kSpec, cc, i);
                    if (i < sh->bins[cc]) {
                        int off = 0;
                        for (int q = 0; q < cc; q++) {
                            off += sh->bins[q];
                        }
                        Pair v;
                        v.v               = __int_as_float((int) (pf.c[m] & 0xffffffffll));
                        v.idx             = (int) (pf.c[m] >> 32);
                        fb.fcand[off + i] = v;
                    }
                }
            }
        }
        const int first = spec ? kSpec : 0;
        for (int cc = g.warp; cc < p.n_slices; cc += g.nw) {
            const int nc = sh->bins[cc];
            if (nc > first) {
                int off = 0;
                for (int i = 0; i < cc; i++) {
                    off += sh->bins[i];
                }
                const long long *src = reinterpret_cast<const long long *>(p.cands + ((size_t) row * (size_t) p.n_slices + (size_t) cc) * (size_t) p.cand_cap);
                for (int i = first + g.lane; i < nc; i += 32) {
                    const long long w = __ldcg(src + i);
                    Pair            v;
                    v.v               = __int_as_float((int) (w & 0xffffffffll));
                    v.idx             = (int) (w >> 32);
                    fb.fcand[off + i] = v;
                }
            }
        }
        g.sync();
        FPROF(3); /* candidates into shared memory */
        if (r.mode == M_TOPK) {
            const int k = r.k;
            select_sorted(g, sh, fb.fcand, total, k, fb.ftmp, fb.fsort);
            FPROF(4); /* select + order */
            if (r.select_only) {
                for (int i = g.tid; i < min(k, p.kept_cap); i += g.n) {
                    kept_i[i] = fb.fsort[i].idx + p.vocab_offset;
                    kept_v[i] = fb.fsort[i].v;
                }
                if (g.tid == 0) {
                    p.kept_n[row] = k;
                    p.tokens[row] = fb.fsort[0].idx + p.vocab_offset;
                }
                g.sync();
                return st;
            }
            /* sampler.c:217-222: softmax over the k kept logits (max = the first), one draw */
            const float m = fb.fsort[0].v;
            for (int i = g.tid; i < k; i += g.n) {
                fb.fq[i] = exp_exact(scaled_arg(fb.fsort[i].v, m, r.inv_t));
            }
            g.sync();
            if (g.warp == 0) {
                double    S;
                const int pick = warp_inverse_cdf(g.lane, fb.fq, k, unit_from(xorshift_next(r.rng)), &S);
                if (g.lane == 0) {
                    p.tokens[row] = fb.fsort[pick].idx + p.vocab_offset;
                    sh->S         = S;
                    if (p.kept_cap > 0) {
                        p.kept_n[row] = k;
                    }
                }
            }
            if (p.kept_cap > 0) {
                g.sync();
                const double S = sh->S;
                for (int i = g.tid; i < min(k, p.kept_cap); i += g.n) {
                    kept_i[i] = fb.fsort[i].idx + p.vocab_offset;
                    kept_v[i] = __double2float_rn((double) fb.fq[i] / S);
                }
            }
            g.sync();
            FPROF(5); /* weights, draw, outputs */
            return st;
        }

        /* top-p over a small nucleus (sampler.c:245-300). Candidates get their exact e_i relative
         * to the row maximum; the rest of the row was summed per slice with expf relative to the
         * slice maximum and is rescaled here. */
        double part = 0.0;
        for (int i = g.tid; i < total; i += g.n) {
            const float e = exp_exact(scaled_arg(fb.fcand[i].v, row_max, r.inv_t));
            fb.fcand[i].v = e;
            part += (double) e;
        }
        for (int cc = g.tid; cc < p.n_slices; cc += g.n) {
            const float  m  = slice_max(cc);
            const double sc = m == -CUDART_INF_F ? 0.0 : exp(((double) m - (double) row_max) * (double) r.inv_t);
            part += sc * __ldcg(&recs[cc].bulk);
        }
        const double S = group_sum_d(g, sh, part);
        for (int i = g.tid; i < total; i += g.n) {
            fb.fcand[i].v = __double2float_rn((double) fb.fcand[i].v / S); /* p_i as the reference normalises it */
        }
        g.sync();
        /* the walk order is (p desc, id asc); the row's kq most probable ids are all candidates */
        const int kq = min(r.kq, total);
        select_sorted(g, sh, fb.fcand, total, kq, fb.ftmp, fb.fsort);
        if (g.tid == 0) {
            const float p_floor = fb.fsort[kq - 1].v; /* nothing outside fsort has a larger p */
            double      cum     = 0.0;
            int         cut     = -1;
            for (int i = 0; i < kq; i++) {
                cum += (double) fb.fsort[i].v;
                if (cum >= (double) r.top_p) {
                    cut = i + 1;
                    break;
                }
            }
            const bool all_in = kq >= p.V;
            bool       ok     = cut > 0 && (fb.fsort[cut - 1].v > p_floor || all_in);
            if (cut < 0 && all_in) { /* never reached top_p: the nucleus is the whole row */
                cut = kq;
                ok  = true;
            }
            if (ok) {
                double N = 0.0;
                for (int i = 0; i < cut; i++) {
                    N += (double) fb.fsort[i].v;
                }
                const double u    = (double) unit_from(xorshift_next(r.rng)) * N;
                double       a    = 0.0;
                int          pick = cut - 1;
                for (int i = 0; i < cut; i++) {
                    a += (double) fb.fsort[i].v;
                    if (u < a) {
                        pick = i;
                        break;
                    }
                }
                p.tokens[row] = fb.fsort[pick].idx + p.vocab_offset;
                if (p.kept_cap > 0) {
                    p.kept_n[row] = cut;
                    for (int i = 0; i < min(cut, p.kept_cap); i++) {
                        kept_i[i] = fb.fsort[i].idx + p.vocab_offset;
                        kept_v[i] = __double2float_rn((double) fb.fsort[i].v / N);
                    }
                }
            }
            sh->flag = ok ? 1 : 0;
        }
        g.sync();
        if (sh->flag) {
            return st;
        }
    }
    g.sync();
    /* the multi-pass path sweeps the whole row several times: it is left to the end of the kernel,
     * when all threads of the CTA are free to share it */
    if (g.tid == 0) {
        sh->blk_max = row_max;
        sh->blk_arg = row_arg;
    }
    g.sync();
    return st | ST_DEFERRED;
}

/* Optional cycle accounting of worker thread 0 (build with -DGB_PROFILE): where one CTA's time goes. */
#ifdef GB_PROFILE
__device__ long long g_prof[512][8]; /* [0,256) workers, [256,512) finishers */
__device__ __forceinline__ long long gtime() { long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define PROF_INIT()              \
    long long prof_acc[8] = {0}; \
    long long prof_t      = clock64()
#define PROF(i)                         \
    if (g.tid == 0) {                   \
        const long long t_ = clock64(); \
        prof_acc[i] += t_ - prof_t;     \
        prof_t = t_;                    \
    }
#define PROF_DONE()                                \
    prof_acc[7] = gtime();                         \
    if (g.tid == 0 && blockIdx.x < 256) {          \
        for (int i_ = 0; i_ < 8; i_++) {           \
            g_prof[blockIdx.x][i_] = prof_acc[i_]; \
        }                                          \
    }
/* finer accounting of one worker warp (warp 5) */
__device__ long long g_prof2[256][16];
#define PROF2_INIT()              \
    long long prof2_acc[16] = {0}; \
    long long prof2_t       = clock64()
#define PROF2(i)                         \
    if (g.tid == 160) {                  \
        const long long t_ = clock64();  \
        prof2_acc[i] += t_ - prof2_t;    \
        prof2_t = t_;                    \
    }
#define PROF2_DONE()                                  \
    if (g.tid == 160 && blockIdx.x < 256) {           \
        for (int i_ = 0; i_ < 12; i_++) {             \
            g_prof2[blockIdx.x][i_] = prof2_acc[i_];  \
        }                                             \
    }
#else
#define PROF_INIT()
#define PROF(i)
#define PROF_DONE()
#define PROF2_INIT()
#define PROF2(i)
#define PROF2_DONE()
#endif

/*
 * The publisher warp takes the CTA's slices in order, each as soon as the last worker warp is done
 * with it: it folds the warps' results into the slice's record (global scratch), frees the
 * slice's accumulators, raises the row's select threshold from the histogram of the candidates
 * seen so far, and counts the slice at its row. The CTA whose slice completes a row finishes that
 * row: every CTA owns a contiguous run of items, so it completes the rows that end inside its run
 * (the CTA that holds a row's first part is through with it long before), and the finishing work
 * spreads evenly by itself.
 */
__device__ void publisher_loop(int lane, const SampleParams &p, StreamShared *sh, int my_count) {
    int  next      = 0; /* the slice to take next */
    bool done_seen = false;
    while (next < my_count) {
        /* ---- fold every slice that is ready (shared memory only); lane b keeps the b-th one's record ---- */
        int    n_new = 0;
        int    my_row = -1, my_item = 0;
        int4   my_h   = make_int4(0, 0, 0, 0);
        double my_bulk = 0.0;
        while (n_new < 32 && next < my_count && sh->slice_done[next % kListRing] == next + 1) {
            const int j = next;
            __threadfence_block(); /* what the worker warps left before they arrived is readable */
            const ItemCfg *cf   = &sh->cfg[j % kCfgRing]; /* stays until w_done moves past j */
            SliceAcc      *acc  = &sh->acc[j % kListRing];
            const int      row  = cf->row, item = cf->item, mode = cf->mode, kq = cf->kq;
            const float    inv_t = cf->inv_t;
            const bool     sel  = (mode == M_TOPK || mode == M_TOPP) && kq > 0 && kq <= kFastKMax;
            const unsigned long long bw   = acc->best;
            const float              smax = key_to_float((unsigned) (bw >> 32));
            double                   bulk = 0.0;
            if (mode == M_TEMP || (mode == M_TOPP && sel)) {
                /* per-warp sums move from their own maximum to the slice maximum */
                double f = 0.0;
                if (lane < kWorkWarps) {
                    const float wm = acc->wmax[lane];
                    f              = wm == -CUDART_INF_F ? 0.0 : acc->wsum[lane] * exp(((double) wm - (double) smax) * (double) inv_t);
                }
                if (mode == M_TEMP) {
                    if (lane < kWorkWarps) {
                        p.recs[item].seg[lane] = f;
                    }
                } else {
                    bulk = warp_sum_d(f);
                }
            }
            if (lane == n_new) {
                my_row  = row;
                my_item = item;
                my_h.x  = __float_as_int(smax);
                my_h.y  = (int) (0xffffffffu - (unsigned) (bw & 0xffffffffull));
                my_h.z  = acc->n_cand;
                my_h.w  = acc->st;
                my_bulk = bulk;
            }
            __syncwarp();
            if (lane == 0) {
                /* the accumulators serve slice j + kListRing next */
                acc->best    = 0ull;
                acc->n_cand  = 0;
                acc->st      = 0;
                acc->arrived = 0;
                __threadfence_block();
                *reinterpret_cast<volatile int *>(&sh->w_done) = j + 1; /* the loader may prepare item j + kListRing */
            }
            /* the row's threshold: the lowest bin edge above which at least kq candidates lie, one bin
             * lower to be safe against rounding at the edge. Lane l holds bins 8 l .. 8 l + 7. */
            if (sel && sh->t_row == row && sh->t_scale > 0.0f) {
                const float t_lo = sh->t_lo, t_scale = sh->t_scale;
                int         c[8];
                const int4  lo4 = *reinterpret_cast<const int4 *>(&sh->thist[8 * lane]);
                const int4  hi4 = *reinterpret_cast<const int4 *>(&sh->thist[8 * lane + 4]);
                c[0] = lo4.x, c[1] = lo4.y, c[2] = lo4.z, c[3] = lo4.w, c[4] = hi4.x, c[5] = hi4.y, c[6] = hi4.z, c[7] = hi4.w;
                int mine = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    mine += c[i];
                }
                int suffix = mine; /* candidates in this lane's bins and all higher ones */
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int dn = __shfl_down_sync(0xffffffffu, suffix, o);
                    if (lane + o < 32) {
                        suffix += dn;
                    }
                }
                const unsigned ball = __ballot_sync(0xffffffffu, suffix >= kq);
                if (ball != 0u && lane == 31 - __clz(ball)) {
                    int run = suffix - mine, b = 8 * lane;
#pragma unroll
                    for (int i = 7; i >= 0; i--) {
                        run += c[i];
                        if (run >= kq) {
                            b = 8 * lane + i;
                            break;
                        }
                    }
                    if (b >= 2 && sh->t_row == row) {
                        const float t_new = t_lo + (float) (b - 1) / t_scale;
                        if (t_new > t_lo) {
                            atomicMax(&sh->tau_pub, ((unsigned long long) (unsigned) row << 32) | order_key(t_new));
                        }
                    }
                }
            }
            __syncwarp();
            n_new++;
            next++;
        }
        if (n_new == 0) {
            /* bounded wait for the next slice, or for the end of the worker loop */
            bool ready = false;
            for (long long spin = 0; spin < (1ll << 31); spin++) {
                ready = sh->slice_done[next % kListRing] == next + 1;
                if (ready || done_seen) {
                    break;
                }
                done_seen = sh->q_done != 0; /* look once more after the workers have left */
                pause_cycles(40);
            }
            if (!ready) {
                if (lane == 0 && !done_seen) {
                    sh->q_error = 1; /* gave up waiting */
                }
                break;
            }
            continue;
        }
        /* ---- publish the folded slices, one per lane, so that their round trips overlap ---- */
        bool last = false;
        if (lane < n_new) {
            SliceRec *rec                  = p.recs + my_item;
            *reinterpret_cast<int4 *>(rec) = my_h;
            rec->bulk                      = my_bulk;
            __threadfence(); /* the slice's record and candidates are visible before the counter moves */
            last = atomicAdd(&p.row_counter[my_row], 1) == p.n_slices - 1;
            if (last) {
                __threadfence(); /* and the other slices' records are visible to whoever saw the last count */
            }
        }
        for (unsigned lasts = __ballot_sync(0xffffffffu, last); lasts != 0u; lasts &= lasts - 1u) {
            const int done_row = __shfl_sync(0xffffffffu, my_row, __ffs(lasts) - 1);
            if (lane == 0) {
                const int hq = sh->fin_head;
                for (long long spin = 0; spin < (1ll << 31) && hq - sh->fin_tail >= kFinQueue; spin++) {
                    pause_cycles(100);
                }
                sh->fin_q[hq % kFinQueue] = done_row;
                __threadfence_block();
                sh->fin_head = hq + 1;
            }
        }
    }
    if (lane == 0) {
        __threadfence_block();
        sh->p_done = 1;
#ifdef GB_PROFILE
        if (blockIdx.x < 256) {
            g_prof[256 + blockIdx.x][3] = gtime();
        }
#endif
    }
}

/* Status of a finished row and, behind a sequence's last row, its generator. One thread. */
__device__ __forceinline__ void row_epilogue(const SampleParams &p, const RowCfg &r, int row, int st) {
    p.status[row] = st;
    if (p.rng_out != nullptr && r.rr == p.rows_per_seq - 1) {
        /* the sequence's generator after all of its rows drew */
        unsigned long long s = p.rng_in ? p.rng_in[r.seq] : 1ull;
        for (int i = 0; i < p.rows_per_seq * r.draws_per_row; i++) {
            (void) xorshift_next(s);
        }
        p.rng_out[r.seq] = s;
    }
}

/* The rows that the finisher warps left to the multi-pass path, served by all threads of the CTA
 * once its slices are done. The ring's memory holds the radix walks' histograms. */
__device__ __noinline__ void slow_rows(const SampleParams p, StreamShared *sh, unsigned char *ring) {
    Grp g;
    g.tid  = (int) threadIdx.x;
    g.lane = g.tid & 31;
    g.warp = g.tid >> 5;
    g.n    = kThreads;
    g.nw   = kThreads / 32;
    g.bar  = 0;
    const int n_slow = sh->n_slow;
    for (int i = 0; i < n_slow; i++) {
        const int4   e   = __ldcg(&p.slow_list[(size_t) blockIdx.x * (size_t) p.slow_cap + i]);
        const RawCfg rc  = raw_config(p, e.x, true);
        RowCfg       r   = row_config(p, e.x, rc, true);
        const int    st  = e.w | multipass_row(g, p, &sh->fn, r, __int_as_float(e.z), e.y, ring, p.stages * p.stage_bytes);
        if (g.tid == 0) {
            row_epilogue(p, r, e.x, st);
        }
        g.sync();
    }
}

/* The finisher warps' loop: they finish the rows this CTA completed, in the order they completed. */
__device__ void finisher_loop(const Grp &g, const SampleParams &p, StreamShared *sh, const FinBuffers &fb) {
    GroupShared *fs = &sh->fn;
    FPROF_INIT();
#ifdef GB_PROFILE
    long long facc[8] = {0};
    facc[6]           = gtime();
#endif
    for (;;) {
        if (g.tid == 0) {
            /* bounded wait for the next row this CTA completed, or for the end of the publisher */
            int row = -1;
            for (long long spin = 0; spin < (1ll << 31); spin++) {
                const int t = sh->fin_tail;
                if (sh->fin_head > t) {
                    __threadfence_block();
                    row          = sh->fin_q[t % kFinQueue];
                    sh->fin_tail = t + 1;
                    break;
                }
                if (sh->p_done) {
                    if (sh->fin_head > t) {
                        continue; /* queued just before the publisher left */
                    }
                    row = -2;
                    break;
                }
                pause_cycles(GB_FIN_PAUSE);
            }
            if (row == -1) {
                sh->q_error = 1; /* gave up waiting: leave */
                row         = -2;
            }
            __threadfence(); /* the row's records, some published by another CTA, are visible from here on */
            fs->cur_row = row;
        }
        g.sync();
        FPROF(0); /* waiting for a ticket */
        const int row = fs->cur_row;
        if (row < 0) {
#ifdef GB_PROFILE
            facc[7] = gtime();
            if (g.tid == 0 && blockIdx.x < 256) {
                for (int i_ = 0; i_ < 8; i_++) {
                    if (i_ != 3) {
                        g_prof[256 + blockIdx.x][i_] = facc[i_];
                    }
                }
            }
#endif
            return;
        }
#ifdef GB_PROFILE
        const long long ft0 = clock64();
#endif
        const RawCfg   rc  = raw_config(p, row, true); /* in flight together with ... */
        const Prefetch pf  = prefetch_row(g, p, row); /* ... the row's slice headers and first candidates */
        RowCfg         r   = row_config(p, row, rc, true);
        FPROF(1); /* configuration and prefetch requested */
        const int      fst = finish_row(g, p, fs, r, fb, pf);
#ifdef GB_PROFILE
        fprof_t = clock64();
#endif
#ifdef GB_PROFILE
        facc[4] += clock64() - ft0;
        facc[5] += 1;
        facc[2] = gtime();
#endif
        if (g.tid == 0) {
            if (fst & ST_DEFERRED) {
                const int n = sh->n_slow; /* a CTA completes at most slow_cap rows */
                if (n < p.slow_cap) {
                    p.slow_list[(size_t) blockIdx.x * (size_t) p.slow_cap + n] = make_int4(row, fs->blk_arg, __float_as_int(fs->blk_max), fst & ~ST_DEFERRED);
                    sh->n_slow = n + 1;
                } else {
                    p.status[row] = ST_INTERNAL;
                }
            } else {
                row_epilogue(p, r, row, fst);
            }
        }
        g.sync();
        FPROF(6); /* status, generator */
    }
}

/* ------------------------------------------------- worker warps: helpers -- */

/* Registers of one worker thread that outlive a slice: the select threshold of the row in work. */
struct TauState {
    float tau;     /* a lower bound of the row's kq-th largest value */
    int   row;     /* the row it belongs to (-1: none) */
    float lo;      /* candidate histogram: bin = (v - lo) * scale */
    float scale;   /* 0: no histogram for this row */
    int   boots;   /* thresholds set so far (selects the alternating words) */
};

/*
 * Sets the select threshold of a row on the first slice this CTA sees of it. Called by all
 * worker threads (three group barriers). bv = the thread's maximum over its share (`own`: it has
 * one), wkey = the ordered key of the warp's maximum. Every owning thread is a group of up to
 * 32 entries; the group maxima are binned by their ordered keys into 256 bins below the largest,
 * and tau = the lower edge of the highest bin above which at least kq group maxima lie: at least
 * kq entries of this slice alone are >= tau, so tau cannot exceed the row's kq-th largest value.
 * Fewer than kq groups: everything passes.
 */
__device__ __noinline__ TauState set_row_threshold(int tid, StreamShared *sh, float bv, bool own, unsigned wkey, int kq, int row, int boots) {
    Grp g;
    g.tid  = tid;
    g.lane = tid & 31;
    g.warp = tid >> 5;
    g.n    = kWorkThreads;
    g.nw   = kWorkWarps;
    g.bar  = 1;
    TauState ts;
    ts.boots       = boots + 1;
    const int bsel = boots & 1;
    const unsigned bkey = order_key(bv + 0.0f);
    {
        const unsigned wlo  = __reduce_min_sync(0xffffffffu, own ? bkey : 0xffffffffu);
        const int      wown = __popc(__ballot_sync(0xffffffffu, own));
        if (g.lane == 0 && wown > 0) {
            atomicMax(&sh->top_key[bsel], wkey);
            atomicMin(&sh->low_key[bsel], wlo);
            atomicAdd(&sh->boot_n[bsel], wown);
        }
    }
    for (int i = g.tid; i < kHistBins; i += g.n) {
        sh->bhist[i] = 0; /* the previous use's readers passed its last barrier long ago */
    }
    g.sync();
    if (g.tid == 0) {
        sh->tau_key[bsel ^ 1] = 0xffffffffu; /* their readers have all passed the barrier above */
        sh->top_key[bsel ^ 1] = 0u;
        sh->low_key[bsel ^ 1] = 0xffffffffu;
        sh->boot_n[bsel ^ 1]  = 0;
        sh->t_row             = -1;
    }
    for (int i = g.tid; i < kHistBins; i += g.n) {
        sh->thist[i] = 0;
    }
    const unsigned khi = sh->top_key[bsel];
    /* values far below the largest all go to bin 0: the walk comes from the top */
    const unsigned klo   = max(sh->low_key[bsel], khi > (1u << 27) ? khi - (1u << 27) : 0u);
    const int      n_own = sh->boot_n[bsel];
    const unsigned span  = khi - klo;
    const int      shift = max(0, (32 - __clz(span)) - 8); /* (span >> shift) < 256 */
    if (own && n_own >= kq) {
        atomicAdd(&sh->bhist[(max(bkey, klo) - klo) >> shift], 1);
    }
    g.sync();
    if (g.warp == 0) {
        unsigned tkey = 0u; /* below everything: all entries pass */
        if (n_own >= kq) {
            /* lane l holds bins 8 l .. 8 l + 7; the highest bin with at least kq group maxima in it and above */
            int        c[8];
            const int4 lo4 = *reinterpret_cast<const int4 *>(&sh->bhist[8 * g.lane]);
            const int4 hi4 = *reinterpret_cast<const int4 *>(&sh->bhist[8 * g.lane + 4]);
            c[0] = lo4.x, c[1] = lo4.y, c[2] = lo4.z, c[3] = lo4.w, c[4] = hi4.x, c[5] = hi4.y, c[6] = hi4.z, c[7] = hi4.w;
            int mine = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                mine += c[i];
            }
            int suffix = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int dn = __shfl_down_sync(0xffffffffu, suffix, o);
                if (g.lane + o < 32) {
                    suffix += dn;
                }
            }
            const unsigned ball = __ballot_sync(0xffffffffu, suffix >= kq);
            int            b    = 0;
            if (ball != 0u && g.lane == 31 - __clz(ball)) {
                int run = suffix - mine;
                b       = 8 * g.lane;
#pragma unroll
                for (int i = 7; i >= 0; i--) {
                    run += c[i];
                    if (run >= kq) {
                        b = 8 * g.lane + i;
                        break;
                    }
                }
            }
            b    = __shfl_sync(0xffffffffu, b, ball != 0u ? 31 - __clz(ball) : 0);
            tkey = b == 0 ? sh->low_key[bsel] : klo + ((unsigned) b << shift); /* bin 0 also holds what was clamped */
        }
        if (g.lane == 0) {
            sh->tau_key[bsel] = tkey;
        }
    }
    g.sync();
    const unsigned tkey = sh->tau_key[bsel];
    ts.tau = tkey == 0u ? -CUDART_INF_F : key_to_float(tkey);
    ts.row = row;
    /* the row's candidates are binned between tau and this slice's maximum; the publisher reads the
     * bins from the top and raises the threshold for the slices to come (each thread computes the
     * same map from value to bin) */
    const float top = key_to_float(khi);
    ts.lo           = ts.tau;
    ts.scale        = (n_own >= kq && top > ts.tau && top - ts.tau < CUDART_INF_F) ? (float) kHistBins / (top - ts.tau) : 0.0f;
    if (g.tid == 0) {
        sh->t_lo    = ts.lo;
        sh->t_scale = ts.scale;
        __threadfence_block();
        sh->t_row = row; /* the publisher raises the threshold of this row from now on */
    }
    return ts;
}

/* ------------------------------------------------------------------ kernel -- */

__global__ void __launch_bounds__(kThreads, 1) sample_stream_kernel(const __grid_constant__ SampleParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];

    unsigned char  *ring = smem_raw;
    StreamShared   *sh   = reinterpret_cast<StreamShared *>(smem_raw + (size_t) p.stages * (size_t) p.stage_bytes);
    unsigned       *dlr  = reinterpret_cast<unsigned *>(sh + 1);                             /* id lists of the slices in flight */
    FinBuffers      fb;
    fb.dlist_cap = min(p.hist_cap, 512);
    fb.bitmap    = reinterpret_cast<unsigned *>(dlr + kListRing * p.hist_cap);
    fb.dlist     = reinterpret_cast<PenEntry *>(fb.bitmap + kFinBitmapWords);
    fb.fcand     = reinterpret_cast<Pair *>(fb.dlist + fb.dlist_cap); /* merged candidates of one row */
    fb.ftmp      = fb.fcand + p.fin_cap;
    fb.fsort     = fb.ftmp + p.fin_cap;                             /* kFastKMax entries */
    fb.fq        = reinterpret_cast<float *>(fb.fsort + kFastKMax); /* kFastKMax entries */

    /* every CTA takes a contiguous run of the (row, slice) items, so that consecutive items mostly
     * belong to one row and what a slice learns about its row serves the next ones */
    const int n_items  = p.n_rows * p.n_slices;
    const int G        = (int) gridDim.x;
    const int q_items  = n_items / G, r_items = n_items - q_items * G;
    const int my_first = (int) blockIdx.x * q_items + min((int) blockIdx.x, r_items);
    const int my_count = q_items + ((int) blockIdx.x < r_items ? 1 : 0);
    const int row0     = my_first / p.n_slices;
    const int c0       = my_first - row0 * p.n_slices;

    if (p.chained) {
        /* Launched as a programmatic dependent of the kernel before it in the stream: the thread block may
         * have been placed while that kernel's last blocks were still at work. Everything it touches in
         * global memory waits here for that kernel to be complete and visible, so the stream's order is
         * kept; what is saved is the gap between two grids. The kernel behind this one may be placed
         * likewise. */
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;");
    }
    /* the control words (row counters, queue slots, tickets) of this scratch set exist twice; this
     * launch uses one copy, which was zeroed during the set's previous use, and zeroes the other */
    for (int i = (int) blockIdx.x * kThreads + (int) threadIdx.x; i < p.clear_words; i += G * kThreads) {
        p.clear_ptr[i] = 0;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], kWorkWarps);
        }
        for (int i = 0; i < kListRing; i++) {
            sh->acc[i].best    = 0ull;
            sh->acc[i].n_cand  = 0;
            sh->acc[i].arrived = 0;
            sh->acc[i].st      = 0;
            sh->n_dl[i]        = 0;
        }
        for (int i = 0; i < kListRing; i++) {
            sh->slice_done[i] = 0;
        }
        sh->t_row = -1;
        sh->tau_key[0] = 0xffffffffu;
        sh->tau_key[1] = 0xffffffffu;
        sh->top_key[0] = 0u;
        sh->top_key[1] = 0u;
        sh->low_key[0] = 0xffffffffu;
        sh->low_key[1] = 0xffffffffu;
        sh->boot_n[0]  = 0;
        sh->boot_n[1]  = 0;
        sh->tau_pub    = 0ull;
        sh->q_done     = 0;
        sh->q_error    = 0;
        sh->p_done     = 0;
        sh->fin_head   = 0;
        sh->fin_tail   = 0;
        sh->l_decoded  = 0;
        sh->w_done     = 0;
        sh->done_warps = 0;
        sh->n_slow     = 0;
    }
    __syncthreads();

    auto advance = [&](int &row, int &c) {
        c++;
        if (c == p.n_slices) {
            c = 0;
            row++;
        }
    };

    /* the loader keeps the ring full: the jj-th item of this CTA goes to stage jj % stages */
    auto issue = [&](int row, int c, int stage) {
        const int      s0    = c * p.slice;
        const int      n     = max(0, min(p.slice, p.V - s0));
        const unsigned bytes = (unsigned) (n & ~3) * 4u;
        if (bytes == 0u) {
            return;
        }
        unsigned char       *dst = ring + (size_t) stage * (size_t) p.stage_bytes;
        const unsigned char *src = reinterpret_cast<const unsigned char *>(p.logits + (size_t) row * (size_t) p.row_stride + s0);
        mbar_expect_tx(&sh->full[stage], bytes);
        for (unsigned off = 0; off < bytes; off += 32768u) {
            bulk_g2s(dst + off, src + off, min(32768u, bytes - off), &sh->full[stage]);
        }
    };
    /* an item's configuration is decoded into shared memory a few items ahead, so that the worker
     * warps spend no instructions and no memory round trips on it */
    auto decode = [&](int row, int c, const RowCfg &r, ItemCfg *o) {
        const int s0 = c * p.slice;
        const int n  = max(0, min(p.slice, p.V - s0));
        const int n4 = (n + 3) >> 2;
        int4     *w  = reinterpret_cast<int4 *>(o); /* five stores of four words */
        w[0]         = make_int4(row, row * p.n_slices + c, s0, n);
        w[1]         = make_int4((int) r.mode, r.kq, r.pen_on ? 1 : 0, 0);
        w[2]         = make_int4(__float_as_int(r.inv_t), __float_as_int(r.rep), __float_as_int(r.freq), __float_as_int(r.pres));
        w[3]         = make_int4(share_len(n4), n4, c, 0);
        w[4]         = make_int4(r.H, r.E, r.seq, r.seq0);
    };
    static_assert(sizeof(ItemCfg) == 80, "decode() writes the item configuration as five int4");

    if (threadIdx.x >= kWorkThreads && threadIdx.x < kWorkThreads + 32) {
        /* ============================================================== loader == */
        /* Lane 0 issues the bulk copies as stages come free; the whole warp prepares each item up to
         * kListRing items ahead of the slowest worker warp: its configuration and the list of the
         * history ids that fall into the slice, without repeats, each with its count. Every wait is
         * bounded. */
        const int lane = (int) threadIdx.x - kWorkThreads;
        int       irow = row0, ic = c0; /* next item to load */
        int       drow = row0, dcs = c0; /* next item to decode */
        int       issued = 0, decoded = 0, istage = 0;
        RawCfg    raw{};
        if (lane == 0 && my_count > 0) {
            raw = raw_config(p, drow);
        }
        RowCfg rcur{};
        int    rcur_row = -1;
        int hc[4]   = {-1, -1, -1, -1}; /* this lane's share of the history ids of row hc_row ... */
        int hcnt[4] = {0, 0, 0, 0};     /* ... and how often each occurs, kept by its first occurrence only */
        int hc_row = -1;
        int hn[4]  = {-1, -1, -1, -1}; /* the next row's ids, fetched ahead (raw, before the shard offset) */
        int hn_row = -1, hn_asked = -1, prev_item_row = -1;
        int offr = 0, off_row = -1; /* lane i: where slice i's run starts in the prepared id list of row off_row */
        bool lists_ready = false;   /* the kernel that prepares the lists has been waited for */
        int my_issued = 0; /* lane 0: copies issued, the warp's count follows at the next turn */
        /* one copy if a stage is free; never blocks: the items' preparation must go on */
        auto try_issue = [&]() {
            if (p.aligned && my_issued < my_count) {
                bool ok = my_issued < p.stages;
                if (!ok) { /* the stage's previous slice must have been lifted by all worker warps */
                    ok = mbar_test(&sh->empty[istage], (unsigned) ((my_issued / p.stages - 1) & 1));
                }
                if (ok) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    issue(irow, ic, istage);
                    advance(irow, ic);
                    istage = istage + 1 == p.stages ? 0 : istage + 1;
                    my_issued++;
                }
            }
        };
#ifdef GB_PROFILE
        long long lp_busy = 0, lp_idle = 0, lp_t = clock64();
#endif
        long long idle = 0;
        while ((p.aligned && issued < my_count) || decoded < my_count) {
            int act = 0;
            if (lane == 0) {
                try_issue();
                act |= (my_issued - issued) << 2;
                if (decoded < my_count && decoded < *reinterpret_cast<volatile int *>(&sh->w_done) + kListRing) {
                    act |= 2;
                }
            }
            act = __shfl_sync(0xffffffffu, act, 0);
            issued += act >> 2;
            if (act & 2) {
                ItemCfg *o = &sh->cfg[decoded % kCfgRing];
                if (lane == 0) {
                    if (rcur_row != drow) {
                        /* a new row: its parameters were requested when the previous row began */
                        rcur     = row_config(p, drow, raw, false);
                        rcur_row = drow;
                        if (drow + 1 < p.n_rows) {
                            raw = raw_config(p, drow + 1); /* requested now, used when the next row begins */
                        }
                    }
                    decode(drow, dcs, rcur, o);
                    advance(drow, dcs);
                }
                __syncwarp();
                int nd = 0, ovf = 0;
                if (o->flags & 1) {
                    const int  H = o->H, total = o->H + o->E, s0 = o->s0, n = o->n;
                    const int *hrow = p.hist ? p.hist + (size_t) o->seq * (size_t) p.hist_stride : nullptr;
                    const int *erow = p.extra ? p.extra + (size_t) o->seq0 * (size_t) p.extra_stride : nullptr;
                    unsigned  *dl   = dlr + (size_t) (decoded % kListRing) * (size_t) p.hist_cap;
                    if (total <= kLoaderIds) {
                        /* The usual case. A row's ids are the same for all of its slices: once per row
                         * they are read into registers (four per lane) and each is marked as the first
                         * of its value with that value's count; a slice then only picks its own. */
                        if (hc_row != o->row) {
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const int j  = 32 * k + lane;
                                int       id = -1;
                                if (j < total) { /* fetched ahead while the previous row was in work, where that was possible */
                                    id = (hn_row == o->row ? hn[k] : (j < H ? hrow[j] : erow[1 + j - H])) - p.vocab_offset;
                                }
                                id    = (id >= 0 && id < p.V) ? id : -1 - j; /* unusable ids match nothing */
                                hc[k] = id;
                            }
                            /* counts by a small open-addressing table in shared memory: the lane whose id
                             * opened a slot speaks for that id and reads the slot's final count */
                            for (int i = lane; i < kIdSlots; i += 32) {
                                sh->id_key[i] = -1;
                                sh->id_cnt[i] = 0;
                            }
                            __syncwarp();
                            int slot_of[4];
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                slot_of[k] = -1;
                                if (hc[k] >= 0) {
                                    unsigned hsh = ((unsigned) hc[k] * 2654435761u) >> (32 - kIdSlotBits);
                                    for (int probe = 0; probe < kIdSlots; probe++) {
                                        const int old = atomicCAS(&sh->id_key[hsh], -1, hc[k]);
                                        if (old == -1 || old == hc[k]) {
                                            atomicAdd(&sh->id_cnt[hsh], 1);
                                            slot_of[k] = old == -1 ? (int) hsh : -1; /* only the opener keeps the slot */
                                            break;
                                        }
                                        hsh = (hsh + 1) & (kIdSlots - 1);
                                    }
                                }
                            }
                            __syncwarp();
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                hcnt[k] = slot_of[k] >= 0 ? sh->id_cnt[slot_of[k]] : 0; /* 0: another lane speaks for this id */
                            }
                            __syncwarp();
                            hc_row = o->row;
                        }
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            if (32 * k < total) {
                                const bool     in   = hcnt[k] > 0 && hc[k] >= s0 && hc[k] - s0 < n;
                                const unsigned ball = __ballot_sync(0xffffffffu, in);
                                if (in) {
                                    const int pos = nd + __popc(ball & ((1u << lane) - 1u));
                                    if (pos < p.hist_cap) {
                                        dl[pos] = (unsigned) (hc[k] - s0) | ((unsigned) hcnt[k] << kLiBits);
                                    }
                                }
                                nd += __popc(ball);
                            }
                        }
                    } else {
                        /* Long histories: a kernel that ran before this one left the row's distinct ids with
                         * their counts in global memory, grouped by slice; a slice copies its run. */
                        if (!lists_ready) {
                            /* this kernel may have been started while that one was still running
                             * (programmatic dependent launch): its lists are complete and visible from here on */
                            if (lane == 0) { /* the ring fills meanwhile */
                                for (int i = 1; i < p.stages; i++) {
                                    try_issue();
                                }
                            }
                            __syncwarp();
                            asm volatile("griddepcontrol.wait;" ::: "memory");
                            lists_ready = true;
                        }
                        if (off_row != o->row) {
                            offr    = lane <= p.n_slices ? p.pre_off[(size_t) o->row * (size_t) (p.n_slices + 1) + lane] : 0;
                            off_row = o->row;
                        }
                        int lo, hi;
                        if (p.n_slices < 32) {
                            lo = __shfl_sync(0xffffffffu, offr, o->c);
                            hi = __shfl_sync(0xffffffffu, offr, o->c + 1);
                        } else {
                            lo = p.pre_off[(size_t) o->row * (size_t) (p.n_slices + 1) + o->c];
                            hi = p.pre_off[(size_t) o->row * (size_t) (p.n_slices + 1) + o->c + 1];
                        }
                        const unsigned *src = p.pre_list + (size_t) o->row * (size_t) p.row_cap;
                        for (int i = lo + lane; i < hi && i - lo < p.hist_cap; i += 32) {
                            copy_word_async(&dl[i - lo], &src[i]);
                        }
                        async_copies_wait();
                        nd = hi - lo;
                    }
                    if (nd > p.hist_cap) { /* cannot happen when the launcher sized the room */
                        ovf = 1;
                        nd  = 0;
                    }
                    /* the next row's ids are requested one item after this row began (its parameters have
                     * arrived by then), so that the row change does not wait for global memory */
                    const int nrow = o->row + 1;
                    if (hn_row != nrow && hn_asked != nrow && nrow < p.n_rows && o->row == prev_item_row) {
                        int seq_n = 0, H_n = 0;
                        if (lane == 0) { /* lane 0 holds the next row's raw parameters */
                            seq_n = raw.seq;
                            H_n   = p.hist ? (int) min((long long) max(raw.hist_len, 0), p.hist_stride) : 0;
                        }
                        seq_n            = __shfl_sync(0xffffffffu, seq_n, 0);
                        H_n              = __shfl_sync(0xffffffffu, H_n, 0);
                        const int seq0_n = p.rows_per_seq == 1 ? nrow : nrow / p.rows_per_seq;
                        const int E_n    = p.extra ? nrow - seq0_n * p.rows_per_seq : 0;
                        if (H_n + E_n <= kLoaderIds) {
                            const int *hr = p.hist ? p.hist + (size_t) seq_n * (size_t) p.hist_stride : nullptr;
                            const int *er = p.extra ? p.extra + (size_t) seq0_n * (size_t) p.extra_stride : nullptr;
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const int j = 32 * k + lane;
                                hn[k]       = j < H_n + E_n ? (j < H_n ? hr[j] : er[1 + j - H_n]) : -1;
                            }
                            hn_row = nrow;
                        }
                        hn_asked = nrow;
                    }
                    prev_item_row = o->row;
                }
                __syncwarp();
                if (lane == 0) {
                    sh->n_dl[decoded % kListRing] = nd;
                    o->st0                        = ovf ? ST_HIST_OVERFLOW : 0;
                    __threadfence_block();
                    sh->l_decoded = decoded + 1;
                }
                decoded++;
            }
#ifdef GB_PROFILE
            {
                const long long t_ = clock64();
                if (act & 2) {
                    lp_busy += t_ - lp_t;
                } else {
                    lp_idle += t_ - lp_t;
                }
                lp_t = t_;
            }
#endif
            if (act == 0) {
                if (++idle > (1ll << 26)) {
                    if (lane == 0) {
                        sh->q_error = 4; /* the workers stopped releasing stages: leave */
                    }
                    break;
                }
                pause_cycles(40);
            } else {
                idle = 0;
            }
        }
#ifdef GB_PROFILE
        if (lane == 0 && blockIdx.x < 256) {
            g_prof2[blockIdx.x][12] = lp_busy;
            g_prof2[blockIdx.x][13] = lp_idle;
        }
#endif
    } else if (threadIdx.x >= kWorkThreads + 32 && threadIdx.x < kWorkThreads + 64) {
        publisher_loop((int) threadIdx.x - kWorkThreads - 32, p, sh, my_count);
    } else if (threadIdx.x >= kWorkThreads + 64) {
        Grp g;
        g.tid  = (int) threadIdx.x - kWorkThreads - 64;
        g.lane = g.tid & 31;
        g.warp = g.tid >> 5;
        g.n    = kFinThreads;
        g.nw   = kFinWarps;
        g.bar  = 2;
        finisher_loop(g, p, sh, fb);
    } else {
    /* ================================================================ workers == */
    /* Every worker warp walks the CTA's slices at its own pace: it owns a fixed share of each slice
     * (float4 [warp * L, (warp + 1) * L), lanes interleaved), waits for the slice's copy, applies the
     * penalties that fall into its share, lifts the share into registers, gives the stage back and
     * runs its passes on registers. Warps meet only in the slice's accumulators (shared-memory
     * atomics) and, once per row, in the barrier that sets the row's select threshold. The warp
     * that arrives last at a slice's accumulators writes the slice's mail. */
    Grp g;
    g.tid  = (int) threadIdx.x;
    g.lane = g.tid & 31;
    g.warp = g.tid >> 5;
    g.n    = kWorkThreads;
    g.nw   = kWorkWarps;
    g.bar  = 1;

    /* bounded wait until the loader has prepared item jj */
    auto wait_decoded = [&](int jj) {
        for (long long spin = 0; spin < (1ll << 26) && sh->l_decoded <= jj; spin++) {
            pause_cycles(20);
        }
        return sh->l_decoded > jj;
    };
    unsigned phase_bits = 0u; /* parity of the next wait for a copy, one bit per stage */
    int      stage      = 0;
    TauState ts;
    ts.tau   = 0.0f;
    ts.row   = -1;
    ts.lo    = 0.0f;
    ts.scale = 0.0f;
    ts.boots = 0;

    PROF_INIT();
    PROF2_INIT();
#ifdef GB_PROFILE
    prof_acc[3] = gtime();
#endif
    for (int j = 0; j < my_count; j++) {
        PROF(0); /* loop overhead */
        PROF2(0);
        if (!wait_decoded(j)) {
            break; /* the loader gave up (it has flagged the error); every warp stops at the same item */
        }
        const ItemCfg *cf = &sh->cfg[j % kCfgRing];
        const int4     c0 = *reinterpret_cast<const int4 *>(&cf->row);   /* row, item, s0, n */
        const int4     c1 = *reinterpret_cast<const int4 *>(&cf->mode);  /* mode, kq, flags, - */
        const int4     c3 = *reinterpret_cast<const int4 *>(&cf->L);     /* L, nv4, c, st0 */
        const int      row = c0.x, item = c0.y, s0 = c0.z, n = c0.w;
        const int      mode = c1.x, kq = c1.y;
        const bool     pen_on = (c1.z & 1) != 0;
        const int      L = c3.x, nv4 = c3.y;
        SliceAcc      *acc   = &sh->acc[j % kListRing];
        float         *sl    = reinterpret_cast<float *>(ring + (size_t) stage * (size_t) p.stage_bytes);
        const int      body  = p.aligned ? (n & ~3) : 0;
        const int      w4lo  = min(g.warp * L, nv4);
        const int      mine4 = min(L, nv4 - w4lo); /* float4 this warp owns (L is a multiple of 32) */
        const float   *grow  = p.logits + (size_t) row * (size_t) p.row_stride + s0;
        int            st    = g.warp == 0 ? c3.w : ST_OK;
        if (g.tid == 96 && c3.z == 0) {
            p.status[row] = ST_INTERNAL; /* stands until the row's finisher writes the real status */
        }
        PROF2(1); /* decoded + cfg */

        /* ---- 1. the warp's share of the slice is in the stage; the slice's tail is padded with -inf ---- */
        if (p.aligned) {
            const unsigned parity = (phase_bits >> stage) & 1u;
            phase_bits ^= 1u << stage;
            if (body > 0 && !mbar_wait_bounded(&sh->full[stage], parity)) {
                st |= ST_LOAD_TIMEOUT;
                (void) mbar_wait_bounded(&sh->full[stage], parity); /* a second bounded chance for the copy in flight */
            }
            if (nv4 * 4 > body && w4lo + mine4 == nv4 && mine4 > 0 && g.lane < 4) {
                const int i = body + g.lane; /* the last float4 is not part of the bulk copy */
                sl[i]       = i < n ? grow[i] : -CUDART_INF_F;
            }
        } else {
            /* rows off the 16-byte grid: plain loads; before the stage is written again every warp must
             * have lifted the slice that used it last */
            if (j >= p.stages && !mbar_wait_bounded(&sh->empty[stage], (unsigned) ((j / p.stages - 1) & 1))) {
                st |= ST_LOAD_TIMEOUT;
            }
            for (int i = 4 * w4lo + g.lane; i < 4 * (w4lo + mine4); i += 32) {
                sl[i] = i < n ? grow[i] : -CUDART_INF_F;
            }
        }
        __syncwarp();
        PROF(1); /* waiting for the slice */
        PROF2(2);

        /* ---- 2. penalties on the share (the loader left the slice's distinct ids with their counts) ---- */
        if (pen_on) {
            const int       nd = sh->n_dl[j % kListRing];
            const unsigned *dl = dlr + (size_t) (j % kListRing) * (size_t) p.hist_cap;
            for (int i = g.lane; i < nd; i += 32) {
                const unsigned e  = dl[i];
                const int      li = (int) (e & ((1u << kLiBits) - 1u));
                if ((li >> 2) >= w4lo && (li >> 2) < w4lo + mine4) {
                    sl[li] = penalise(sl[li], (int) (e >> kLiBits), cf->rep, cf->freq, cf->pres);
                }
            }
            __syncwarp();
        }
        if (p.out_logits != nullptr) {
            float *orow = p.out_logits + (size_t) row * (size_t) p.V + s0;
            for (int i = 4 * w4lo + g.lane; i < min(4 * (w4lo + mine4), n); i += 32) {
                orow[i] = sl[i];
            }
        }
        /* what a thread does not own reads as -inf, so the passes below need no bounds checks */
        const int     first4 = w4lo + g.lane; /* this thread's float4 are first4 + 32 i */
        const float4 *s4     = reinterpret_cast<const float4 *>(sl) + first4;
        float4        x[8];
        if (mine4 == 256) { /* the usual case: a full share */
#pragma unroll
            for (int i = 0; i < 8; i++) {
                x[i] = s4[32 * i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                x[i] = g.lane + 32 * i < mine4 ? s4[32 * i] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
            }
        }
        PROF(2); /* penalties, registers */
        PROF2(3);

        /* ---- 3. the share's maximum; the few entries that matter are then picked from the stage ---- */
        float bv = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            bv = fmaxf(bv, fmaxf(fmaxf(x[i].x, x[i].y), fmaxf(x[i].z, x[i].w)));
        }
        PROF2(4); /* lane max (waits for the loads) */
        const unsigned bkey = order_key(bv + 0.0f); /* -0 and +0 are one value, as the comparison of floats has it */
        const unsigned wkey = __reduce_max_sync(0xffffffffu, bkey);
        const float    wmax = key_to_float(wkey);
        /* The 32 entries of lane L, one per lane of the warp: lane l looks at element l & 3 of L's
         * float4 number l >> 2. `look` says whether that entry exists, is L's own and is no padding. */
        const int  e4   = g.lane >> 2, eq = g.lane & 3;
        auto       look = [&](int L_, int &li, float &v) {
            li            = 4 * (w4lo + L_ + 32 * e4) + eq;
            const bool ok = L_ + 32 * e4 < mine4 && li < n;
            v             = ok ? sl[li] : -CUDART_INF_F;
            return ok;
        };
        if (mode == M_ARGMAX) {
            /* the first id of the warp's maximum, if it can still be the slice's; only the lanes that hold
             * the maximum are searched */
            unsigned best = 0x7fffffffu;
            if (wkey >= (unsigned) (*reinterpret_cast<volatile unsigned long long *>(&acc->best) >> 32)) {
                for (unsigned hits = __ballot_sync(0xffffffffu, bkey == wkey && g.lane < mine4); hits != 0u; hits &= hits - 1u) {
                    int            li;
                    float          v;
                    const bool     ok = look(__ffs(hits) - 1, li, v);
                    const unsigned eb = __ballot_sync(0xffffffffu, ok && v == wmax);
                    if (eb != 0u) {
                        best = min(best, (unsigned) (s0 + __shfl_sync(0xffffffffu, li, __ffs(eb) - 1)));
                    }
                }
            }
            if (g.lane == 0 && best != 0x7fffffffu) {
                atomicMax(&acc->best, ((unsigned long long) wkey << 32) | (unsigned long long) (0xffffffffu - best));
            }
        } else if (g.lane == 0 && mine4 > 0) {
            atomicMax(&acc->best, (unsigned long long) wkey << 32); /* the maximum alone: no other mode asks where it is */
        }
        PROF2(5); /* key reduce + first id */
        PROF2(6);

        const bool  sel   = (mode == M_TOPK || mode == M_TOPP) && kq > 0 && kq <= kFastKMax;
        const float inv_t = cf->inv_t;
        float       tau   = CUDART_INF_F;
        if (sel) {
            /* top-k / top-p fast path. The select threshold tau is a lower bound of the row's kq-th
             * largest value, so every entry of the row's kq best passes it wherever it lies. It is set
             * once per row and CTA, on the first slice the CTA sees of the row (all warps meet there);
             * the other slices of the row reuse it, raised by what the mail writers publish, and need no
             * barrier. */
#ifdef GB_FAKE_TAU
            if (ts.row != row) { /* experiment only: a constant that suits the synthetic rows */
                ts.tau = 7.0f; ts.row = row; ts.lo = 7.0f; ts.scale = 0.0f;
            } else if (false) {
#else
            if (ts.row != row) {
#endif
                ts = set_row_threshold(g.tid, sh, bv, g.lane < mine4, wkey, kq, row, ts.boots);
                PROF(6);
            } else {
                const unsigned long long pub = *reinterpret_cast<volatile unsigned long long *>(&sh->tau_pub);
                if ((int) (pub >> 32) == row && (unsigned) pub > order_key(ts.tau)) {
                    ts.tau = key_to_float((unsigned) pub);
                }
            }
            tau      = ts.tau;
            Pair *gc = p.cands + (size_t) item * (size_t) p.cand_cap;
            /* the lanes whose maximum passes hold all the candidates: their entries are looked at by the
             * whole warp, one lane after the other (about three per slice and warp) */
            for (unsigned hits = __ballot_sync(0xffffffffu, bv >= tau && g.lane < mine4); hits != 0u; hits &= hits - 1u) {
                int            li;
                float          v;
                const bool     ok = look(__ffs(hits) - 1, li, v) && v >= tau;
                const unsigned pb = __ballot_sync(0xffffffffu, ok);
                int            base = 0;
                if (g.lane == 0) {
                    base = atomicAdd(&acc->n_cand, __popc(pb));
                }
                base = __shfl_sync(0xffffffffu, base, 0);
                if (ok) {
                    const int pos = base + __popc(pb & ((1u << g.lane) - 1u));
                    if (pos < p.cand_cap) {
                        Pair c2;
                        c2.v    = v;
                        c2.idx  = s0 + li;
                        gc[pos] = c2; /* straight to the row's scratch */
                    }
                    if (ts.scale > 0.0f) {
                        atomicAdd(&sh->thist[min(kHistBins - 1, max(0, __float2int_rz((v - ts.lo) * ts.scale)))], 1);
                    }
                }
            }
        }
        __syncwarp();
        if (g.lane == 0) {
            mbar_arrive(&sh->empty[stage]); /* this warp is done with the stage */
        }
        PROF2(10); /* threshold + candidates */
        if (mode == M_TEMP || (mode == M_TOPP && sel)) {
            /* sum of e_i relative to the WARP's maximum (top-p: of what stays below the threshold); the
             * mail writer rescales to the slice maximum and the finisher to the row maximum. -inf
             * padding gives exp(-inf) = 0. */
            const float ref = wmax == -CUDART_INF_F ? 0.0f : wmax;
            double      sum = 0.0;
            if (mode == M_TEMP) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float e0 = expf(scaled_arg(x[i].x, ref, inv_t));
                    const float e1 = expf(scaled_arg(x[i].y, ref, inv_t));
                    const float e2 = expf(scaled_arg(x[i].z, ref, inv_t));
                    const float e3 = expf(scaled_arg(x[i].w, ref, inv_t));
                    sum += (double) ((e0 + e1) + (e2 + e3));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    /* what passed the threshold is a candidate and counts there: its argument becomes -inf
                     * (exp gives 0), so that the 32 evaluations stay one straight line and overlap */
                    const float e0 = expf(x[i].x >= tau ? -CUDART_INF_F : scaled_arg(x[i].x, ref, inv_t));
                    const float e1 = expf(x[i].y >= tau ? -CUDART_INF_F : scaled_arg(x[i].y, ref, inv_t));
                    const float e2 = expf(x[i].z >= tau ? -CUDART_INF_F : scaled_arg(x[i].z, ref, inv_t));
                    const float e3 = expf(x[i].w >= tau ? -CUDART_INF_F : scaled_arg(x[i].w, ref, inv_t));
                    sum += (double) ((e0 + e1) + (e2 + e3));
                }
            }
            sum = warp_sum_d(sum);
            if (g.lane == 0) {
                acc->wmax[g.warp] = wmax;
                acc->wsum[g.warp] = sum;
            }
        }
        PROF(4); /* the passes */
        PROF2(7);

        /* ---- 4. arrive at the slice; the last warp hands the slice's result to the publisher ---- */
        st = __reduce_or_sync(0xffffffffu, (unsigned) st);
        int last = 0;
        if (g.lane == 0) {
            if (st != 0) {
                atomicOr(&acc->st, st);
            }
            __threadfence_block(); /* this warp's candidates and sums are ordered before its arrival */
            last = atomicAdd(&acc->arrived, 1) == kWorkWarps - 1 ? 1 : 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        PROF2(8); /* arrive */
        if (last && g.lane == 0) {
            sh->slice_done[j % kListRing] = j + 1; /* the publisher takes it from here */
        }
        PROF(5); /* mail */
        PROF2(9);
        stage = stage + 1 == p.stages ? 0 : stage + 1;
    }
    PROF_DONE();
    PROF2_DONE();
    if (g.lane == 0) {
        __threadfence_block();
        if (atomicAdd(&sh->done_warps, 1) == kWorkWarps - 1) {
            sh->q_done = 1;
        }
    }
    } /* workers */

    /* every role has ended (all of their waits are bounded): what is left are the rows that need the
     * multi-pass path, shared by all threads */
    __syncthreads();
    if (sh->n_slow > 0) {
        slow_rows(p, sh, ring);
    }
}

/* ------------------------------------------------ long histories, prepared -- */

constexpr int kRowIdThreads = 256;

/* One CTA per row whose history (plus fed tokens) is longer than the stream kernel's loader keeps
 * in registers: the row's distinct ids with their counts, grouped by the slice they fall into.
 * pre_off[row][c] .. pre_off[row][c + 1] is slice c's run in pre_list[row]; an entry is
 * (position in the slice) | (count << kLiBits). Shorter rows are left to the loader. */
__global__ void __launch_bounds__(kRowIdThreads) row_ids_kernel(const __grid_constant__ SampleParams p) {
    extern __shared__ __align__(16) int row_ids_smem[];
    int *tkey = row_ids_smem;          /* open-addressing table: the id ... */
    int *tcnt = tkey + p.id_slots;     /* ... and how often it occurs */
    int *bcnt = tcnt + p.id_slots;     /* entry c + 1: distinct ids in slice c; after the scan, entry c: ids in slices < c */
    int *bpos = bcnt + p.bucket_cap;   /* next free place of each slice's run */

    /* the stream kernel behind this one may start now: it copies logits and sets itself up while the
     * lists are made, and waits for them where it first needs one */
    asm volatile("griddepcontrol.launch_dependents;");
    const int row  = (int) blockIdx.x, tid = (int) threadIdx.x;
    const int seq0 = p.rows_per_seq == 1 ? row : row / p.rows_per_seq;
    const int seq  = p.slot ? p.slot[seq0] : seq0;
    const int H    = p.hist ? (int) min((long long) max(p.hist_len[seq], 0), p.hist_stride) : 0;
    const int E    = p.extra ? row - seq0 * p.rows_per_seq : 0;
    if (H + E <= kLoaderIds) {
        return;
    }
    const int *hrow = p.hist ? p.hist + (size_t) seq * (size_t) p.hist_stride : nullptr;
    const int *erow = p.extra ? p.extra + (size_t) seq0 * (size_t) p.extra_stride : nullptr;
    for (int i = tid; i < p.id_slots; i += kRowIdThreads) {
        tkey[i] = -1;
        tcnt[i] = 0;
    }
    for (int i = tid; i <= p.n_slices; i += kRowIdThreads) {
        bcnt[i] = 0;
    }
    __syncthreads();
    const unsigned smask = (unsigned) p.id_slots - 1u;
    for (int j = tid; j < H + E; j += kRowIdThreads) {
        const int id = (j < H ? hrow[j] : erow[1 + j - H]) - p.vocab_offset;
        if (id >= 0 && id < p.V) {
            unsigned hsh = ((unsigned) id * 2654435761u) & smask;
            for (int probe = 0; probe < p.id_slots; probe++) { /* at most half of the slots are ever taken */
                const int old = atomicCAS(&tkey[hsh], -1, id);
                if (old == -1 || old == id) {
                    atomicAdd(&tcnt[hsh], 1);
                    if (old == -1) {
                        atomicAdd(&bcnt[id / p.slice + 1], 1);
                    }
                    break;
                }
                hsh = (hsh + 1u) & smask;
            }
        }
    }
    __syncthreads();
    if (tid < 32) {
        int *off   = p.pre_off + (size_t) row * (size_t) (p.n_slices + 1);
        int  carry = 0;
        for (int base = 0; base <= p.n_slices; base += 32) {
            const int i    = base + tid;
            int       incl = i <= p.n_slices ? bcnt[i] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                if (tid >= d) {
                    incl += up;
                }
            }
            if (i <= p.n_slices) {
                bcnt[i] = carry + incl;
                bpos[i] = carry + incl;
                off[i]  = carry + incl;
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();
    unsigned *list = p.pre_list + (size_t) row * (size_t) p.row_cap;
    for (int i = tid; i < p.id_slots; i += kRowIdThreads) {
        const int id = tkey[i];
        if (id >= 0) {
            const int c   = id / p.slice;
            const int pos = atomicAdd(&bpos[c], 1);
            list[pos]     = (unsigned) (id - c * p.slice) | ((unsigned) tcnt[i] << kLiBits);
        }
    }
}

/* ----------------------------------------------------------------- launchers -- */

size_t sample_stream_fixed_smem() { return sizeof(StreamShared); }

static cudaError_t ensure_attributes(size_t smem_bytes) {
    static int  configured_smem[64] = {0};
    int         dev                 = 0;
    cudaError_t e                   = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    if (dev < 0 || dev >= 64) {
        return cudaErrorInvalidDevice;
    }
    if ((int) smem_bytes > configured_smem[dev]) {
        e = cudaFuncSetAttribute(sample_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) {
            return e;
        }
        configured_smem[dev] = (int) smem_bytes;
    }
    return cudaSuccess;
}

static cudaError_t ensure_row_ids_attributes(size_t smem_bytes) {
    static int  configured_smem[64] = {0};
    int         dev                 = 0;
    cudaError_t e                   = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    if (dev < 0 || dev >= 64) {
        return cudaErrorInvalidDevice;
    }
    if (smem_bytes > 48 * 1024 && (int) smem_bytes > configured_smem[dev]) {
        e = cudaFuncSetAttribute(row_ids_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) {
            return e;
        }
        configured_smem[dev] = (int) smem_bytes;
    }
    return cudaSuccess;
}

#ifdef GB_PROFILE
extern "C" int geist_b200_debug_prof3(long long *out, int clear) {
    if (clear) {
        static long long zero[256 * 16];
        return (int) cudaMemcpyToSymbol(g_prof3, zero, sizeof(zero));
    }
    return (int) cudaMemcpyFromSymbol(out, g_prof3, sizeof(long long) * 256 * 16);
}
extern "C" int geist_b200_debug_prof2(long long *out) { return (int) cudaMemcpyFromSymbol(out, g_prof2, sizeof(long long) * 256 * 16); }
extern "C" int geist_b200_debug_prof(long long *out) { return (int) cudaMemcpyFromSymbol(out, g_prof, sizeof(long long) * 512 * 8); }
#endif

cudaError_t launch_sample_stream(const SampleParams &p, int grid, size_t smem_bytes, cudaStream_t stream) {
    cudaError_t e = ensure_attributes(smem_bytes);
    if (e != cudaSuccess) {
        return e;
    }
    if (p.id_slots > 0) { /* rows may bring more ids than the loader keeps in registers: prepare their lists first */
        const size_t ids_smem = ((size_t) p.id_slots * 2 + (size_t) p.bucket_cap * 2) * sizeof(int);
        e                     = ensure_row_ids_attributes(ids_smem);
        if (e != cudaSuccess) {
            return e;
        }
        row_ids_kernel<<<dim3((unsigned) p.n_rows), dim3(kRowIdThreads), ids_smem, stream>>>(p);
        e = cudaGetLastError();
        if (e != cudaSuccess) {
            return e;
        }
#ifndef GB_COOP
        /* programmatic dependent launch: the stream kernel's thread blocks start as soon as that kernel
         * lets them, and its loader waits for the lists (griddepcontrol.wait) before it reads one.
         * Worth it for small batches, where start-up is a good part of the launch (64 rows: 27.0 -> 23.3 us);
         * with several waves of list blocks the early start only gets in their way (4096 rows: +4 %). */
        if (p.n_rows > 4 * grid) {
            sample_stream_kernel<<<dim3((unsigned) grid), dim3(kThreads), smem_bytes, stream>>>(p);
            return cudaGetLastError();
        }
        cudaLaunchConfig_t   cfg{};
        cudaLaunchAttribute attr[1];
        cfg.gridDim          = dim3((unsigned) grid);
        cfg.blockDim         = dim3(kThreads);
        cfg.dynamicSmemBytes = smem_bytes;
        cfg.stream           = stream;
        attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs                                          = attr;
        cfg.numAttrs                                       = 1;
        return cudaLaunchKernelEx(&cfg, sample_stream_kernel, p);
#endif
    }
    /* no CTA ever waits for another one, so the grid needs no co-residency */
#ifdef GB_COOP
    void *args[] = {const_cast<SampleParams *>(&p)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(sample_stream_kernel), dim3((unsigned) grid), dim3(kThreads), args, smem_bytes, stream);
#else
    {
        SampleParams        pc = p;
        cudaLaunchConfig_t  cfg{};
        cudaLaunchAttribute attr[1];
        pc.chained           = 1;
        cfg.gridDim          = dim3((unsigned) grid);
        cfg.blockDim         = dim3(kThreads);
        cfg.dynamicSmemBytes = smem_bytes;
        cfg.stream           = stream;
        attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs                                          = attr;
        cfg.numAttrs                                       = 1;
        return cudaLaunchKernelEx(&cfg, sample_stream_kernel, pc);
    }
#endif
}

} /* namespace gb */

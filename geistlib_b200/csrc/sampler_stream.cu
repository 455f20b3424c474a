/*
 * sampler_stream.cu — the logits -> token kernel (sm_100a).
 *
 * Every logits row crosses the chip exactly once. A row is cut into slices of at most 8192 floats; the work item
 * is (row, slice); the grid is two thread blocks of 8 warps per SM, and every thread block owns a contiguous run
 * of the row-major item list. The consecutive slices of one row inside a run are a PART of that row.
 *
 *   Streaming. Every warp owns a fixed share of each slice (256 float4) and keeps its own ring of two stages
 *   full with bulk asynchronous copies (global -> this thread block's shared memory, signalled on the warp's own
 *   mbarriers): it waits for its share, applies the penalties that fall into it, lifts it into registers, asks
 *   for the share two items ahead and works on the registers. Inside a part no warp waits for another one.
 *
 *   Greedy rows keep (maximum, first id) per warp. Top-k / top-p rows pick candidates against a select
 *   threshold tau, a lower bound of the row's kq-th largest value: the part's first slice sets it (the thread
 *   maxima of all warps are binned by key; the only barriers inside a part), a histogram of the candidates
 *   raises it as the part streams. What is kept is the float4 GROUP that holds a candidate (four values and the
 *   id of the first): the lanes that hold any place them into the warp's own list themselves, one pass per
 *   slice, the places counted in shared memory. Temperature and top-p rows also sum
 *   expf((x - warp maximum) * inv_t) per warp and slice.
 *
 *   Before any of this a row's share may pass the soft cap tanhf(x / c) * c and the mask of allowed columns,
 *   in place in the stage (head.c:145-159; only launches that carry one pay for it).
 *
 *   Part boundaries. The thread block meets and writes the part's record (maximum, first id, threshold, sums;
 *   two 16-byte slots) followed by its candidate groups to the part's place in global scratch. Nothing else is
 *   shared between thread blocks: no counters, no thread block waits for another one.
 *
 *   Finishing is left to a kernel of its own behind the stream kernel, launched as a programmatic dependent so
 *   that its thread blocks are placed while the stream kernel drains: one thread block per row merges the parts'
 *   records; greedy rows end there; top-k rows (k <= 256) get their surviving candidates ordered, their
 *   probabilities evaluated exactly (double exp rounded once) and the draw made; temperature rows walk the
 *   per-warp segment sums and re-read the one segment that the draw falls into; top-p rows with a small nucleus
 *   are served from the candidates and the sums of the rest; rows whose kept set is too large for one pass
 *   (top-k beyond 256, wide nuclei) are worked on a private copy of the row in global scratch (the multi-pass
 *   path, ROW_SLOW_PATH). finish_rows_kernel<false> carries all of that; finish_rows_kernel<true> carries greedy
 *   and top-k alone and is launched instead when the caller vouched for such rows (F_FAST_ONLY); with
 *   F_GREEDY_ONLY, and with F_INLINE_TOPK (whole rows per thread block, greedy and top-k rows), the stream kernel
 *   writes the tokens itself and no finishing kernel runs.
 *   Histories of more than kRowIds ids are counted per row by row_ids_kernel ahead of all this.
 *
 *   The stream kernel is a template over what a launch can meet (kinds of rows vouched for, penalties at all,
 *   plain input, short histories), chosen by the host at the launch: an instantiation carries no code for the
 *   rest, and no call to an out-of-line function is left inside its slice loop.
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

/* Optional instrumentation, compiled in with -DGB_PROFILE (and -DGB_PROFILE_CYC): PROF(i) stamps %globaltimer
 * at fixed points of a thread block's life (stream kernel 0-4, finishing kernels 5-13), MP(i) at the stages of
 * the multi-pass path, CYC(i) adds up a warp's cycles per section of the stream kernel's slice loop (0 wait for
 * data, 1 load + maxima + refill, 2 argmax / capture / raise, 4 loop top, 5 part set-up, 6 part end, 7 first
 * slice's threshold). The arrays are read back through geist_b200_debug_*. All of it is empty otherwise. */
#ifdef GB_PROFILE
__device__ long long g_prof[1024][16];
__device__ __forceinline__ long long gtime() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define PROF(i)                                        \
    if (threadIdx.x == 0 && blockIdx.x < 1024) {       \
        g_prof[blockIdx.x][i] = gtime();               \
    }
#define PROF_ONCE(i)                                                       \
    if (threadIdx.x == 0 && blockIdx.x < 1024 && g_prof[blockIdx.x][i] == 0) { \
        g_prof[blockIdx.x][i] = gtime();                                   \
    }
__device__ long long g_mp[1024][24];
#define MP(i)                                          \
    if (threadIdx.x == 0 && blockIdx.x < 1024) {       \
        g_mp[blockIdx.x][i] = gtime();                 \
    }
#ifdef GB_PROFILE_CYC
__device__ long long g_cyc[1024][kWarps][8];
#define CYC_INIT()              \
    long long cyc_acc[8] = {0}; \
    long long cyc_t      = clock64()
#define CYC(i)                          \
    {                                   \
        const long long t_ = clock64(); \
        cyc_acc[i] += t_ - cyc_t;       \
        cyc_t = t_;                     \
    }
#define CYC_DONE()                                                  \
    if ((threadIdx.x & 31) == 0 && blockIdx.x < 1024) {             \
        for (int i_ = 0; i_ < 8; i_++) {                            \
            g_cyc[blockIdx.x][threadIdx.x >> 5][i_] = cyc_acc[i_];  \
        }                                                           \
    }
#else
#define CYC_INIT()
#define CYC(i)
#define CYC_DONE()
#endif
#else
#define MP(i)
#define PROF(i)
#define PROF_ONCE(i)
#define CYC_INIT()
#define CYC(i)
#define CYC_DONE()
#endif

struct PenEntry {
    int   li;
    float orig;
};

__device__ __forceinline__ float key_to_float(unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k); }


/* The threads that share a reduction: here always the whole thread block. */
struct Grp {
    int tid, lane, warp; /* position inside the group */
    int n, nw;           /* threads, warps */
    int bar;             /* unused: the group is the thread block */
    __device__ __forceinline__ void sync() const { __syncthreads(); }
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

/* float4 of a slice that one warp owns: an equal share, rounded up to whole warp steps */
__host__ __device__ __forceinline__ int share_len(int nv4) { return ((nv4 + kWarps - 1) / kWarps + 31) & ~31; }

constexpr int kLiBits = 14; /* an id list entry is (position in the slice) | (count << kLiBits) */
static_assert(kSliceMax <= (1 << kLiBits), "slice positions must fit the id list entry");
static_assert((long long) kMaxSlices * kSliceMax <= (1ll << 28), "a candidate group keeps four flag bits above the id of its first value");

enum Mode { M_ARGMAX, M_TOPK, M_TOPP, M_TEMP };

constexpr int ST_DEFERRED = 1 << 30; /* inside the kernel only: the one-pass finish could not serve the row (the multi-pass path has to, or the kernel lacks the code) */

/* Everything a row needs that does not depend on the slice. */
struct RowCfg {
    int                row, seq0, seq, rr;
    float              T, top_p, inv_t;
    int                top_k, k, kq;
    Mode               mode;
    bool               select_only, pen_on;
    int                H, E;
    float              rep, freq, pres;
    float              cap;  /* > 0: the row is sampled from tanhf(x / cap) * cap */
    const unsigned    *mrow; /* the sequence's mask of allowed columns, or null */
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
    float cap;
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
    c.cap          = p.softcap ? p.softcap[c.seq] : 0.0f;
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
    /* head.c:145-159: the cap is skipped for greedy rows (monotone, the argmax is the same) */
    r.cap    = (c.cap > 0.0f && r.T > 0.0f) ? c.cap : 0.0f;
    r.mrow   = p.mask ? p.mask + (size_t) r.seq * (size_t) p.mask_stride : nullptr;
    r.hrow   = p.hist ? p.hist + (size_t) r.seq * (size_t) p.hist_stride : nullptr;
    r.erow   = p.extra ? p.extra + (size_t) r.seq0 * (size_t) p.extra_stride : nullptr; /* per call, not per slot */
    return r;
}

__device__ __forceinline__ int hist_id(const RowCfg &r, int j, int vocab_offset) {
    return (j < r.H ? r.hrow[j] : r.erow[1 + j - r.H]) - vocab_offset;
}

/* What happens to a logit before the penalties: the final-logit soft cap in the reference's own expression
 * (head.c:154, :286), then the mask of allowed columns (bit i of the sequence's mask row: column i may be
 * sampled; a masked column reads as -inf). `i` is the column inside this call's logits. */
__device__ __forceinline__ float soft_cap(float x, float c) {
    return __fmul_rn(tanhf(__fdiv_rn(x, c)), c);
}
__device__ __forceinline__ float prologue_one(float x, int i, float cap, const unsigned *mrow) {
    if (cap > 0.0f) {
        x = soft_cap(x, cap);
    }
    if (mrow != nullptr && ((mrow[i >> 5] >> (i & 31)) & 1u) == 0u) {
        x = -CUDART_INF_F;
    }
    return x;
}

/* The same over a warp's share of a slice in its stage (sl: the share's first float; e0: its index inside the
 * slice; mine4 float4 groups, lane-strided; n: the slice's length, what lies behind it stays -inf). Kept out of
 * line: the stream kernel's loop stays short for the launches that have neither cap nor mask. */
__device__ __noinline__ void prologue_share(float *sl, int lane, int mine4, int e0, int n, int s0, float cap, const unsigned *mrow) {
    float4 *w4 = reinterpret_cast<float4 *>(sl) + lane;
    for (int i = 0; lane + 32 * i < mine4; i++) {
        const int e = e0 + 4 * (lane + 32 * i);
        float4    v = w4[32 * i];
        if (e + 0 < n) v.x = prologue_one(v.x, s0 + e + 0, cap, mrow);
        if (e + 1 < n) v.y = prologue_one(v.y, s0 + e + 1, cap, mrow);
        if (e + 2 < n) v.z = prologue_one(v.z, s0 + e + 2, cap, mrow);
        if (e + 3 < n) v.w = prologue_one(v.w, s0 + e + 3, cap, mrow);
        w4[32 * i] = v;
    }
    __syncwarp();
}

/* The same with the division by rep done as a double product with 1 / rep (rounded to double once per part): the
 * float nearest to x * rcp is the correctly rounded x / rep for every pair of floats (a quotient of two 24-bit
 * numbers is at least 2^-49 of itself away from every midpoint of two floats, the product's error is below 2^-52),
 * and the slice loop keeps clear of the division's out-of-line slow path: a call inside that loop costs every
 * slice. */
__device__ __forceinline__ float penalise_rcp(float x, int cnt, double rcp, float rep, float freq, float pres) {
    x = x > 0.0f ? __double2float_rn(__dmul_rn((double) x, rcp)) : __fmul_rn(x, rep);
    x = __fsub_rn(x, __fmul_rn((float) cnt, freq));
    return __fsub_rn(x, pres);
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

/* ------------------------------------------------------------ multi-pass path -- */

template <class F>
__device__ __forceinline__ void row_sweep(const Grp &g, const float *row, int V, F &&f) {
    const int     V4 = V >> 2;
    const float4 *p4 = reinterpret_cast<const float4 *>(row);
    int           j  = g.tid;
    for (; j + 7 * g.n < V4; j += 8 * g.n) { /* eight loads in flight per thread */
        float4 v[8];
#pragma unroll
        for (int q = 0; q < 8; q++) {
            v[q] = p4[j + q * g.n];
        }
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const int b = 4 * (j + q * g.n);
            f(v[q].x, b), f(v[q].y, b + 1), f(v[q].z, b + 2), f(v[q].w, b + 3);
        }
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
    /* private copies start on 16-byte boundaries: four values per access, four accesses in flight per thread */
    const int V4 = V >> 2;
    float4   *p4 = reinterpret_cast<float4 *>(row);
    int       j  = g.tid;
    for (; j + 3 * g.n < V4; j += 4 * g.n) {
        float4 a = p4[j], b = p4[j + g.n], c = p4[j + 2 * g.n], d = p4[j + 3 * g.n];
        a.x = f(a.x, 4 * j), a.y = f(a.y, 4 * j + 1), a.z = f(a.z, 4 * j + 2), a.w = f(a.w, 4 * j + 3);
        p4[j] = a;
        b.x = f(b.x, 4 * (j + g.n)), b.y = f(b.y, 4 * (j + g.n) + 1), b.z = f(b.z, 4 * (j + g.n) + 2), b.w = f(b.w, 4 * (j + g.n) + 3);
        p4[j + g.n] = b;
        c.x = f(c.x, 4 * (j + 2 * g.n)), c.y = f(c.y, 4 * (j + 2 * g.n) + 1), c.z = f(c.z, 4 * (j + 2 * g.n) + 2), c.w = f(c.w, 4 * (j + 2 * g.n) + 3);
        p4[j + 2 * g.n] = c;
        d.x = f(d.x, 4 * (j + 3 * g.n)), d.y = f(d.y, 4 * (j + 3 * g.n) + 1), d.z = f(d.z, 4 * (j + 3 * g.n) + 2), d.w = f(d.w, 4 * (j + 3 * g.n) + 3);
        p4[j + 3 * g.n] = d;
    }
    for (; j < V4; j += g.n) {
        float4 x = p4[j];
        x.x = f(x.x, 4 * j), x.y = f(x.y, 4 * j + 1), x.z = f(x.z, 4 * j + 2), x.w = f(x.w, 4 * j + 3);
        p4[j] = x;
    }
    for (int i = (V4 << 2) + g.tid; i < V; i += g.n) {
        row[i] = f(row[i], i);
    }
}

/* out[i] = f(in[i], i): both rows on 16-byte boundaries (in may be out). */
template <class F>
__device__ __forceinline__ void row_map(const Grp &g, const float *in, float *out, int V, F &&f) {
    const int     V4 = V >> 2;
    const float4 *i4 = reinterpret_cast<const float4 *>(in);
    float4       *o4 = reinterpret_cast<float4 *>(out);
    int           j  = g.tid;
    for (; j + 3 * g.n < V4; j += 4 * g.n) {
        float4 v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            v[q] = i4[j + q * g.n];
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int b = 4 * (j + q * g.n);
            v[q].x = f(v[q].x, b), v[q].y = f(v[q].y, b + 1), v[q].z = f(v[q].z, b + 2), v[q].w = f(v[q].w, b + 3);
            o4[j + q * g.n] = v[q];
        }
    }
    for (; j < V4; j += g.n) {
        float4 x = i4[j];
        x.x = f(x.x, 4 * j), x.y = f(x.y, 4 * j + 1), x.z = f(x.z, 4 * j + 2), x.w = f(x.w, 4 * j + 3);
        o4[j] = x;
    }
    for (int i = (V4 << 2) + g.tid; i < V; i += g.n) {
        out[i] = f(in[i], i);
    }
}

/* A walk is written against "something that calls f(value, id) for every entry": the whole private copy of a
 * row, or a short list of (value, id) pairs picked out of it. */
template <class F>
__device__ __forceinline__ void list_sweep(const Grp &g, const Pair *list, int n, F &&f) {
    int j = g.tid;
    for (; j + 3 * g.n < n; j += 4 * g.n) {
        const Pair a = list[j], b = list[j + g.n], c = list[j + 2 * g.n], d = list[j + 3 * g.n];
        f(a.v, a.idx), f(b.v, b.idx), f(c.v, c.idx), f(d.v, d.idx);
    }
    for (; j < n; j += g.n) {
        const Pair a = list[j];
        f(a.v, a.idx);
    }
}

/* Largest composite word t with mass{word >= t} >= target (inclusive) or > target. The search may
 * start from a known prefix of the word: the bits above top_bit are taken from `prefix`. */
template <class Sweep, class KeyF, class MassF>
__device__ unsigned long long bisect_mass(const Grp &g, GroupShared *sh, Sweep &&sweep, int idx_bits, double target, bool inclusive, KeyF &&key, MassF &&mass,
                                          unsigned long long prefix = 0ull, int top_bit = -1) {
    for (int bit = top_bit >= 0 ? top_bit : 31 + idx_bits; bit >= 0; bit--) {
        const unsigned long long t = prefix | (1ull << bit);
        double                   m = 0.0;
        sweep([&](float x, int i) {
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
template <bool kUnit = false, class Sweep, class KeyF, class MassF>
__device__ RadixOut radix_mass(const Grp &g, GroupShared *sh, double *hm, int *hc, int copies, double scale, Sweep &&sweep, double target, bool inclusive, KeyF &&key,
                               MassF &&mass, int last_level = 0, bool top_filled = false) {
    /* masses are summed as 64-bit fixed point (mass * scale, truncated): integer adds in shared memory are one
     * instruction whatever the conflicts, and the sums do not depend on the order. The caller picks a scale that
     * keeps the row's total below 2^63. */
    unsigned long long *hq = reinterpret_cast<unsigned long long *>(hm);
    RadixOut out;
    out.found   = true;
    out.key     = 0u;
    out.above   = 0.0;
    out.n_above = 0;
    out.ties    = 0;
    for (int level = 3; level >= last_level; level--) { /* last_level 3: the top byte alone; the histograms then stay as they are for the caller */
        const int shift = 8 * level;
        if (!(top_filled && level == 3)) { /* top_filled: the caller binned the top byte itself while it had the entries in hand */
        for (int i = g.tid; i < copies * 256; i += g.n) {
            hq[i] = 0ull;
            hc[i] = 0;
        }
        g.sync();
        unsigned long long *mym = hq + (g.warp % copies) * 256;
        int           *myc = hc + (g.warp % copies) * 256;
        const unsigned pre = out.key;
        sweep([&](float x, int i) {
            const unsigned k = key(x);
            if (level == 3 || (k >> (shift + 8)) == (pre >> (shift + 8))) {
                const unsigned d = (k >> shift) & 255u;
                if (kUnit) { /* every entry weighs one: the counts are the masses */
                    atomicAdd(&myc[d], 1);
                } else {
                    const double m = mass(x, i);
                    if (m > 0.0) {
                        atomicAdd(&mym[d], __double2ull_rz(m * scale));
                        atomicAdd(&myc[d], 1);
                    }
                }
            }
        });
        }
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
                unsigned long long q8 = 0ull;
                c8[q]                 = 0;
                for (int w = 0; w < copies; w++) {
                    q8 += hq[w * 256 + b];
                    c8[q] += hc[w * 256 + b];
                }
                m8[q] = kUnit ? (double) c8[q] : (double) q8 / scale;
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
template <class Sweep, class KeyF, class MassF>
__device__ unsigned long long resolve_ties(const Grp &g, GroupShared *sh, Sweep &&sweep, int idx_bits, const RadixOut &ro, double target, bool inclusive, KeyF &&key,
                                           MassF &&mass) {
    if (ro.ties <= 1) {
        if (g.tid == 0) {
            sh->pick = 0x7fffffff;
        }
        g.sync();
        sweep([&](float x, int i) {
            if (key(x) == ro.key && mass(x, i) > 0.0) {
                atomicMin(&sh->pick, i);
            }
        });
        g.sync();
        const int id = sh->pick;
        g.sync();
        return composite(ro.key, id == 0x7fffffff ? 0 : id, idx_bits);
    }
    return bisect_mass(g, sh, sweep, idx_bits, target, inclusive, key, mass, (unsigned long long) ro.key << idx_bits, idx_bits - 1);
}

/* All threads of the thread block serve a row whose kept set does not fit the one-pass path. */
__device__ __noinline__ int multipass_row(const Grp &g, const SampleParams &p, GroupShared *sh, RowCfg &r, float row_max, int row_arg, void *hist_mem, int hist_bytes, int slot, void *save_mem) {
    /* room for the byte histograms of the radix walks: per warp where it fits, else one for all */
    const int copies = hist_bytes >= g.nw * 256 * 12 ? g.nw : 1;
    double   *hm     = reinterpret_cast<double *>(hist_mem);
    int      *hc     = reinterpret_cast<int *>(hm + copies * 256);
    const int    V        = p.V;
    const int    idx_bits = 32 - __clz(max(V - 1, 1));
    int          st       = ST_SLOW_PATH;
    float       *gr       = p.gen_rows + (size_t) slot * (size_t) p.gen_stride;
    const float *src      = p.logits + (size_t) r.row * (size_t) p.row_stride;
    int         *kept_i   = p.kept_cap > 0 ? p.kept_idx + (size_t) r.row * (size_t) p.kept_cap : nullptr;
    float       *kept_v   = p.kept_cap > 0 ? p.kept_val + (size_t) r.row * (size_t) p.kept_cap : nullptr;
    /* Nothing changes the row's values (no penalties, cap or mask) and it lies on a 16-byte boundary: it is read
     * where it is, and the private copy only takes what a top-p row is rewritten into. */
    const bool   in_place = !r.pen_on && !(r.cap > 0.0f) && r.mrow == nullptr && p.aligned != 0;
    const float *cur      = in_place ? src : gr; /* what the sweeps read */
    auto         row_sw   = [&](auto &&f) { row_sweep(g, cur, V, f); };
    /* the entries that pred(value, id) names, picked out of the row into this thread block's list (any order);
     * every thread gets their number, which may exceed the list's room: the caller checks */
    Pair *list     = p.gen_list + (size_t) slot * (size_t) p.gen_list_cap;
    auto  pick_out = [&](auto &&pred) {
        if (g.tid == 0) {
            sh->n_sel = 0;
        }
        g.sync();
        row_sweep(g, cur, V, [&](float x, int i) {
            if (pred(x, i)) {
                const int pos = atomicAdd(&sh->n_sel, 1);
                if (pos < p.gen_list_cap) {
                    list[pos].v   = x;
                    list[pos].idx = i;
                }
            }
        });
        __threadfence_block();
        g.sync();
        const int n = sh->n_sel;
        g.sync();
        return n;
    };
    MP(0);
    /* private copy of the row, penalties applied once */
    if (in_place) {
    } else if (p.aligned) { /* rows start on 16-byte boundaries: four values per load */
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
    if (r.cap > 0.0f || r.mrow != nullptr) {
        g.sync();
        const float     cap  = r.cap;
        const unsigned *mrow = r.mrow;
        row_rewrite(g, gr, V, [&](float x, int i) { return prologue_one(x, i, cap, mrow); });
    }
    if (r.pen_on) {
        unsigned *bm = p.gen_bitmap + (size_t) slot * (size_t) p.gen_bitmap_words;
        for (int i = g.tid; i < p.gen_bitmap_words; i += g.n) {
            bm[i] = 0u;
        }
        if (g.tid == 0) {
            sh->n_dlist = 0;
        }
        g.sync();
        st |= apply_penalties(g, gr, 0, V, r, V, p.vocab_offset, bm, reinterpret_cast<PenEntry *>(p.gen_dlist + (size_t) slot * (size_t) p.gen_hist_cap), p.gen_hist_cap,
                              &sh->n_dlist, false, 0);
    } else {
        g.sync();
    }
    MP(1);
    /* the fast path's slice records need not carry the maximum: take it from the copy */
    row_max = -CUDART_INF_F;
    row_arg = 0x7fffffff;
    row_sweep(g, cur, V, [&](float x, int i) {
        if (row_arg == 0x7fffffff || pair_before(x, i, row_max, row_arg)) {
            row_max = x;
            row_arg = i;
        }
    });
    group_argmax(g, sh, row_max, row_arg);
    MP(2);
    if (r.mode == M_TOPK) {
        /* the k-th entry in (value desc, id asc) order: a radix walk on counts, then the ids of its ties */
        auto                     okey   = [](float x) { return order_key(x); };
        auto                     one    = [](float, int) { return 1.0; };
        /* The set's last entry, the short way: one sweep counts the entries per top byte of the key, the byte value
         * in which the k-th falls is picked out into the list and the k-th is found there. The long way (four
         * sweeps, ties by bisection) stays for what does not fit the list. */
        unsigned long long t_set    = 0ull;
        bool               have_set = false;
        int                n_list   = 0;
        auto               lst_sw   = [&](auto &&f) { list_sweep(g, list, n_list, f); };
        if (p.gen_list_cap > 0) {
            const RadixOut r3 = radix_mass<true>(g, sh, hm, hc, copies, 1.0, row_sw, (double) r.k, true, okey, one, 3);
            if (r3.found && r3.ties <= (long long) p.gen_list_cap) {
                const unsigned top = r3.key >> 24;
                n_list             = pick_out([&](float x, int) { return (order_key(x) >> 24) == top; });
                if (n_list <= p.gen_list_cap) {
                    const double   tgt = (double) r.k - r3.above;
                    const RadixOut rc  = radix_mass<true>(g, sh, hm, hc, copies, 1.0, lst_sw, tgt, true, okey, one);
                    if (rc.found) {
                        t_set    = resolve_ties(g, sh, lst_sw, idx_bits, rc, tgt, true, okey, one);
                        have_set = true;
                    }
                }
            }
        }
        if (!have_set) {
            const RadixOut rs = radix_mass<true>(g, sh, hm, hc, copies, 1.0, row_sw, (double) r.k, true, okey, one);
            t_set             = rs.found ? resolve_ties(g, sh, row_sw, idx_bits, rs, (double) r.k, true, okey, one) : 0ull;
        }
        auto in_set = [&](float x, int i) { return composite(order_key(x), i, idx_bits) >= t_set; };
        /* the kept set itself (at most 8192 entries) goes into the list: its sum and the draw are found there */
        n_list            = p.gen_list_cap > 0 ? pick_out(in_set) : p.gen_list_cap + 1;
        const bool listed = n_list <= p.gen_list_cap;
        if (r.select_only) {
            if (listed) {
                for (int j = g.tid; j < min(n_list, p.kept_cap); j += g.n) {
                    kept_i[j] = list[j].idx + p.vocab_offset;
                    kept_v[j] = list[j].v;
                }
            } else {
                if (g.tid == 0) {
                    sh->n_sel = 0;
                }
                g.sync();
                row_sweep(g, cur, V, [&](float x, int i) {
                    if (in_set(x, i)) {
                        const int pos = atomicAdd(&sh->n_sel, 1);
                        if (pos < p.kept_cap) {
                            kept_i[pos] = i + p.vocab_offset;
                            kept_v[pos] = x;
                        }
                    }
                });
            }
            if (g.tid == 0) {
                p.kept_n[r.row] = r.k;
                p.tokens[r.row] = row_arg + p.vocab_offset;
            }
        } else {
            auto   qof = [&](float x) { return (double) exp_exact(scaled_arg(x, row_max, r.inv_t)); };
            double m   = 0.0;
            auto   set_sw = [&](auto &&f) { /* the kept set: from the list, else filtered out of the row */
                if (listed) {
                    list_sweep(g, list, n_list, f);
                } else {
                    row_sweep(g, cur, V, [&](float x, int i) {
                        if (in_set(x, i)) {
                            f(x, i);
                        }
                    });
                }
            };
            set_sw([&](float x, int) { m += qof(x); });
            const double S = group_sum_d(g, sh, m);
            const double u = (double) unit_from(xorshift_next(r.rng)) * S;
            /* the pick is the earliest walk position whose running sum exceeds u: the largest
             * word t with mass{word >= t} > u */
            auto                     qmass  = [&](float x, int) { return qof(x); };
            const RadixOut           rp     = radix_mass(g, sh, hm, hc, copies, 0x1p49, set_sw, u, false, okey, qmass); /* weights <= 1, at most 8192 of them */
            unsigned long long       t_pick = rp.found ? resolve_ties(g, sh, set_sw, idx_bits, rp, u, false, okey, qmass) : 0ull;
            if (t_pick < t_set) {
                t_pick = t_set;
            }
            if (g.tid == 0) { /* the word names its entry */
                const unsigned long long id_mask = (1ull << idx_bits) - 1ull;
                p.tokens[r.row]                  = min((int) (id_mask - (t_pick & id_mask)), V - 1) + p.vocab_offset;
            }
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
        row_map(g, cur, gr, V, [&](float x, int) {
            const float e = exp_exact(scaled_arg(x, row_max, r.inv_t));
            acc += (double) e;
            return e;
        });
        cur            = gr; /* from here on the sweeps read the rewritten copy */
        const double S = group_sum_d(g, sh, acc);
        MP(3);
        /* p_i; and while every p_i is in hand it is binned by the top byte of the window's key (what the short way
         * below starts from) */
        const unsigned k_top_w   = __float_as_uint(__double2float_rn(1.0 / S));
        const float    p_floor_w = __double2float_rn(0.5 * (1.0 - (double) r.top_p) / (double) V);
        const unsigned k_floor_w = (p_floor_w > 0.0f && __float_as_uint(p_floor_w) < k_top_w) ? __float_as_uint(p_floor_w) : 0u;
        const unsigned span_w    = k_top_w > k_floor_w ? k_top_w - k_floor_w : 0u;
        const int      ls_w      = span_w > 0u ? __clz(span_w) : 0;
        {
            unsigned long long *hq = reinterpret_cast<unsigned long long *>(hm);
            for (int i = g.tid; i < copies * 256; i += g.n) {
                hq[i] = 0ull;
                hc[i] = 0;
            }
            g.sync();
            unsigned long long *mym = hq + (g.warp % copies) * 256;
            int                *myc = hc + (g.warp % copies) * 256;
            row_rewrite(g, gr, V, [&](float e, int) {
                const float    pv = __double2float_rn((double) e / S);
                const unsigned k  = __float_as_uint(pv);
                if (k >= k_floor_w && pv > 0.0f) {
                    const unsigned d = ((min(k, k_top_w) - k_floor_w) << ls_w) >> 24;
                    atomicAdd(&mym[d], __double2ull_rz((double) pv * 0x1p62));
                    atomicAdd(&myc[d], 1);
                }
                return pv;
            });
        }
        g.sync();
        MP(4);
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
            RadixOut ro = radix_mass(g, sh, hm, hc, copies, 0x1p62, row_sw, target, inclusive, kw, mw); /* probabilities: the row adds up to 1 */
            ro.key      = (ro.key >> ls) + k_lo; /* back to the key itself */
            return ro;
        };
        const unsigned k_top   = keyf(__double2float_rn(1.0 / S)); /* the largest p: e = 1 at the row maximum */
        const float    p_floor = __double2float_rn(0.5 * (1.0 - (double) r.top_p) / (double) V);
        const unsigned k_floor = (p_floor > 0.0f && keyf(p_floor) < k_top) ? keyf(p_floor) : 0u;
        const unsigned long long id_mask = (1ull << idx_bits) - 1ull;
        unsigned long long t_cut = 0ull, t_pick = 0ull;
        long long          cut   = 0;
        bool               have_cut = false, have_pick = false;
        double             N = 0.0, u = 0.0;
        /*
         * Short way. One sweep bins the row by the top byte of the window's key (mass and count per bin). The
         * walk crosses top_p inside one bin: its entries (a few hundred on rows of this kind) are picked out into
         * a list, and the crossing entry is found on the list, target reduced by the mass of the bins above. The
         * draw is walked the same way: the bins' masses are known already (the crossing bin's is what of it lies
         * in the nucleus), the bin it falls into is picked out if it is another one, and the entry is found on
         * that list. Three sweeps of the row instead of a dozen and more. Whatever does not fit (a bin with more
         * entries than the list holds, sums that round apart) takes the long way below.
         */
        {
            const unsigned span = k_top > k_floor ? k_top - k_floor : 0u;
            const int      ls   = span > 0u ? __clz(span) : 0;
            auto           kw   = [&](float pv) {
                const unsigned k = keyf(pv);
                return k >= k_floor ? (min(k, k_top) - k_floor) << ls : 0u;
            };
            auto mwin = [&](float pv, int) { return keyf(pv) >= k_floor ? (double) pv : 0.0; };
            unsigned long long *sq   = reinterpret_cast<unsigned long long *>(save_mem); /* the bins' masses and counts, kept */
            int                *sc   = reinterpret_cast<int *>(sq + 256);
            auto in_bin_of = [&](int bin) { return [&, bin](float pv, int) { return keyf(pv) >= k_floor && (int) (kw(pv) >> 24) == bin && pv > 0.0f; }; };
            const RadixOut r3 = radix_mass(g, sh, hm, hc, copies, 0x1p62, row_sw, (double) r.top_p, true, kw, mwin, 3, true);
            MP(11);
            if (r3.found && r3.ties <= (long long) p.gen_list_cap && p.gen_list_cap > 0) {
                const int b_cut = (int) (r3.key >> 24);
                if (g.tid < 256) { /* the histograms of the sweep are still there: their sums are kept for the draw */
                    unsigned long long q = 0ull;
                    int                c = 0;
                    for (int w = 0; w < copies; w++) {
                        q += reinterpret_cast<unsigned long long *>(hm)[w * 256 + g.tid];
                        c += hc[w * 256 + g.tid];
                    }
                    sq[g.tid] = q;
                    sc[g.tid] = c;
                }
                g.sync();
                int  n_list = pick_out(in_bin_of(b_cut));
                MP(12);
                auto lst_sw = [&](auto &&f) { list_sweep(g, list, n_list, f); };
                if (n_list <= p.gen_list_cap) {
                    const double   tgt = (double) r.top_p - r3.above;
                    const RadixOut rc  = radix_mass(g, sh, hm, hc, copies, 0x1p62, lst_sw, tgt, true, keyf, massf);
                    if (rc.found) {
                        MP(13);
                        t_cut      = resolve_ties(g, sh, lst_sw, idx_bits, rc, tgt, true, keyf, massf);
                        MP(14);
                        double nm  = 0.0;
                        long long ncnt = 0;
                        lst_sw([&](float pv, int i) {
                            if (composite(keyf(pv), i, idx_bits) >= t_cut) {
                                nm += (double) pv;
                                ncnt++;
                            }
                        });
                        const double in_bin = group_sum_d(g, sh, nm);
                        N                   = r3.above + in_bin;
                        cut                 = r3.n_above + group_sum_ll(g, sh, ncnt);
                        have_cut            = true;
                        u                   = (double) unit_from(xorshift_next(r.rng)) * N;
                        /* the bin the draw falls into: a walk over the kept bins from the top, the crossing bin with
                         * its share of the nucleus */
                        if (g.tid == 0) {
                            double run = 0.0;
                            int    bp  = -1;
                            for (int bin = 255; bin >= b_cut && bp < 0; bin--) {
                                const double mb = bin == b_cut ? in_bin : (double) sq[bin] / 0x1p62;
                                if (u < run + mb) {
                                    bp = bin;
                                } else {
                                    run += mb;
                                }
                            }
                            sh->b_star = bp;
                            sh->S      = run;
                        }
                        g.sync();
                        MP(15);
                        const int    b_pick  = sh->b_star;
                        const double above_p = sh->S;
                        g.sync();
                        if (b_pick < 0) {
                            have_pick = true; /* rounding left u at the very end: the last nucleus entry (sampler.c:292) */
                        } else if (b_pick == b_cut) {
                            auto           nml = [&](float pv, int i) { return composite(keyf(pv), i, idx_bits) >= t_cut ? (double) pv : 0.0; };
                            const double   ut  = u - above_p;
                            const RadixOut rk  = radix_mass(g, sh, hm, hc, copies, 0x1p62, lst_sw, ut, false, keyf, nml);
                            t_pick             = rk.found ? resolve_ties(g, sh, lst_sw, idx_bits, rk, ut, false, keyf, nml) : 0ull;
                            have_pick          = true;
                        } else if (sc[b_pick] <= p.gen_list_cap) {
                            n_list = pick_out(in_bin_of(b_pick));
                            MP(16);
                            if (n_list <= p.gen_list_cap) {
                                const double   ut = u - above_p;
                                const RadixOut rk = radix_mass(g, sh, hm, hc, copies, 0x1p62, lst_sw, ut, false, keyf, massf);
                                t_pick            = rk.found ? resolve_ties(g, sh, lst_sw, idx_bits, rk, ut, false, keyf, massf) : 0ull;
                                have_pick         = true;
                            }
                        }
                    }
                }
            }
        }
        if (!have_cut) { /* the long way: radix walks over the whole row */
            RadixOut rc = windowed(k_floor, k_top, (double) r.top_p, true, massf);
            if (!rc.found && k_floor != 0u) {
                rc = windowed(0u, k_top, (double) r.top_p, true, massf); /* rounding kept the window short of top_p */
            }
            MP(5);
            t_cut = rc.found ? resolve_ties(g, sh, row_sw, idx_bits, rc, (double) r.top_p, true, keyf, massf) : 0ull;
            MP(6);
            double    nm   = 0.0;
            long long ncnt = 0;
            row_sweep(g, gr, V, [&](float pv, int i) {
                if (composite(keyf(pv), i, idx_bits) >= t_cut) {
                    nm += (double) pv;
                    ncnt++;
                }
            });
            N   = group_sum_d(g, sh, nm);
            MP(7);
            cut = group_sum_ll(g, sh, ncnt);
            u   = (double) unit_from(xorshift_next(r.rng)) * N;
        }
        if (!have_pick) {
            auto           nmass = [&](float pv, int i) { return composite(keyf(pv), i, idx_bits) >= t_cut ? (double) pv : 0.0; };
            const RadixOut rk    = windowed((unsigned) (t_cut >> idx_bits), k_top, u, false, nmass);
            MP(8);
            t_pick = rk.found ? resolve_ties(g, sh, row_sw, idx_bits, rk, u, false, keyf, nmass) : 0ull;
            MP(9);
        }
        if (t_pick < t_cut) {
            t_pick = t_cut; /* default: the last nucleus entry (sampler.c:292) */
        }
        if (g.tid == 0) { /* the word names its entry: the id is in its low bits */
            p.tokens[r.row] = min((int) (id_mask - (t_pick & id_mask)), V - 1) + p.vocab_offset;
        }
        if (g.tid == 0 && p.kept_cap > 0) {
            p.kept_n[r.row] = (int) cut;
        }
        if (p.kept_cap > 0) {
            st |= ST_KEPT_PARTIAL;
        }
    }
    g.sync();
    MP(10);
    return st;
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

/* Status of a finished row and, behind a sequence's last row, its generator. One thread. */
__device__ __forceinline__ void row_epilogue(const SampleParams &p, const RowCfg &r, int row, int st, unsigned long long rng0) {
    p.status[row] = st;
    if (p.rng_out != nullptr && r.rr == p.rows_per_seq - 1) {
        /* the sequence's generator (rng0: the word it came with) after all of its rows drew */
        unsigned long long s = rng0;
        for (int i = 0; i < p.rows_per_seq * r.draws_per_row; i++) {
            (void) xorshift_next(s);
        }
        p.rng_out[r.seq] = s;
    }
}

/* ------------------------------------------------------------ shared state -- */

/* What the warps of one thread block share. The ring (every warp's two stages) lies in front of it in dynamic
 * shared memory, the candidate groups of the part in work behind it. */
constexpr int kInlineCap = 1024; /* candidates of a row that the stream kernel can order by itself */
struct __align__(16) StreamShared {
    unsigned long long full[kWarps][kStages]; /* warp w's share of item j has landed in its stage j % kStages */
    /* the part in work */
    unsigned           tau_key;   /* ordered key of the raised select threshold (0: not raised yet) */
    int                tau_lock;  /* one warp at a time reads the candidate histogram */
    int                st;        /* status bits of the part */
    unsigned           wkey[kWarps], wlow[kWarps]; /* first slice: largest / smallest group maximum per warp */
    int                wown[kWarps];               /* ... and how many groups the warp holds */
    int                wn[kWarps], wn_all[kWarps]; /* candidate groups per warp: held / found */
    unsigned long long best[kWarps];               /* (key of the maximum, ~first id) per warp */
    float              wb_ref[kWarps];             /* top-p: per warp, sum of expf((x - ref) * inv_t) over what is no candidate */
    double             wb_sum[kWarps];
    int                bhist[kHistBins];           /* first slice: group maxima binned by key */
    int                thist[kHistBins];           /* candidates binned by value between threshold and maximum */
    int                rl_id[kRowIds], rl_cnt[kRowIds + 4]; /* the row's distinct history ids as (offset in the share | count << 10 | tag << 20),
                                                             * grouped by the (slice, warp) share they fall into, and where each group's run starts */
    /* finishing inside the stream kernel (F_INLINE_TOPK): the row's candidates, its k best in order, their weights */
    int                fin_n, cur_rr;
    alignas(8) Pair    fin_c[kInlineCap]; /* also holds the draw's running sums (doubles) once the ranking is done */
    Pair               fin_s[kFastKMax];
    float              fin_q[kFastKMax];
    int                wcur[kWarps];    /* groups in each warp's list (the lanes count themselves in) */
    float              wsq[kWarps];     /* top-k: the threshold at which each warp last cleared its candidate list of what had fallen below */
    unsigned long long cur_rng;         /* the generator word the part's sequence came with, its sequence, and whether the row is the sequence's last */
    int                cur_seq, cur_last;
    float              cap;             /* the part's soft cap and mask row (0 / null: none) */
    const unsigned    *mrow;
    RawCfg             raw_nxt;         /* parameters of the next row of this run, copied in while the part streams */
    int                nxt_ids[kRowIds]; /* that row's history ids (raw): the first words of its history row ... */
    int                nxt_ext[kRowIds]; /* ... and the tokens fed before it */
};

constexpr int kStagedParts = 4;

/* What the threads of one finishing thread block share; the merged candidate list lies behind it. */
struct __align__(16) FinishShared {
    GroupShared gs; /* reductions of the whole thread block */
    float       pmax[kMaxParts], ptau[kMaxParts], pbref[kMaxParts];
    int         parg[kMaxParts], pn[kMaxParts], poff[kMaxParts];
    double      pbsum[kMaxParts];
    int         bhist[kHistBins]; /* select histogram */
    int         n_sel, n_border, n_ent, slot;
    unsigned    fin_bitmap[kFinBitmapWords];
    Pair        fsort[kFastKMax];
    float       fq[kFastKMax];
    PenEntry    fdlist[512];
    float4      st_v[kStagedParts][kThreads]; /* the first 256 slots of the row's first parts, as they came in ... */
    int         st_b[kStagedParts][kThreads]; /* ... in one round trip */
};

constexpr int kGroupBytes = kPartGroups * 20; /* float4 + first id per group */
constexpr int kSqueezeAt  = 64;               /* a warp holding more candidate groups than this looks whether the threshold has left some behind */
constexpr int kListSmem   = 1024;             /* prepared id-list entries of a part that are kept in shared memory */
constexpr int kFinCap     = 2048;             /* candidates the finisher can order per row (8 per thread) */
constexpr int kFinPer     = kFinCap / kThreads;
constexpr int kRankAll    = 384;              /* up to this many candidates are ranked one against all */
constexpr int kFinBytes   = kWarps * 256 * 12;    /* finisher: the merged candidate list; the multi-pass path keeps one byte histogram per warp there */
static_assert(kFinCap * (int) sizeof(Pair) <= kFinBytes, "the merged list fits");
static_assert(kGroupBytes >= 4 * kRowIds * 4, "the id table of a part's set-up lies in the groups' memory");

/* n things dealt out in runs of q + 1 (the first r runs) and q: which run holds thing i */
__device__ __forceinline__ int run_of(int i, int q, int r) { return i < r * (q + 1) ? i / (q + 1) : r + (i - r * (q + 1)) / q; }

/* The thread block that streams item i, and the run [first, first + count) of thread block b (RunMap). */
__device__ __forceinline__ int cta_of_item(const SampleParams &p, int i) {
    const RunMap &m = p.map;
    if (m.mode == RUN_ITEMS) {
        return run_of(i, m.q, m.r);
    }
    const int row = i / p.n_slices;
    if (m.mode == RUN_ROWS) {
        return run_of(row, m.q, m.r);
    }
    return row * m.P + run_of(i - row * p.n_slices, m.q, m.r);
}
__device__ __forceinline__ void run_of_cta(const SampleParams &p, int b, int &first, int &count) {
    const RunMap &m = p.map;
    if (m.mode == RUN_ITEMS) {
        first = b * m.q + min(b, m.r);
        count = m.q + (b < m.r ? 1 : 0);
    } else if (m.mode == RUN_ROWS) {
        first = (b * m.q + min(b, m.r)) * p.n_slices;
        count = (m.q + (b < m.r ? 1 : 0)) * p.n_slices;
    } else {
        const int row = b / m.P, j = b - row * m.P;
        first         = row * p.n_slices + j * m.q + min(j, m.r);
        count         = m.q + (j < m.r ? 1 : 0);
    }
}

/* Highest bin b with at least kq entries in bins >= b (0 when there is none); the whole warp calls, every lane gets it. */
__device__ __forceinline__ int top_bin(const int *hist, int lane, int kq) {
    int cc[8], mine = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        cc[i] = *reinterpret_cast<const volatile int *>(&hist[8 * lane + i]);
        mine += cc[i];
    }
    int suffix = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int dn = __shfl_down_sync(0xffffffffu, suffix, o);
        if (lane + o < 32) {
            suffix += dn;
        }
    }
    const unsigned ball = __ballot_sync(0xffffffffu, suffix >= kq);
    int            b    = 0;
    if (ball != 0u && lane == 31 - __clz(ball)) {
        int run = suffix - mine;
        b       = 8 * lane;
#pragma unroll
        for (int i = 7; i >= 0; i--) {
            run += cc[i];
            if (run >= kq) {
                b = 8 * lane + i;
                break;
            }
        }
    }
    return __shfl_sync(0xffffffffu, b, ball != 0u ? 31 - __clz(ball) : 0);
}

/* Group f of this thread block's own candidates: the warps' lists one after the other. */
__device__ __forceinline__ int own_slot(const StreamShared *sh, int f) {
    int w = 0;
#pragma unroll
    for (int i = 0; i < kWarps - 1; i++) {
        const int n = sh->wn[i];
        if (w == i && f >= n) {
            f -= n;
            w = i + 1;
        }
    }
    return w * kGroupCapWarp + f;
}

/* ------------------------------------------- finisher: ordered select of kq -- */

/*
 * cand[0..total) hold distinct ids, total >= kq >= 1, total <= kFinCap. Writes the kq best in (value desc, id asc)
 * order to sorted[0..kq). Every thread lifts its entries into registers; a histogram over their key range finds
 * the bin that holds the kq-th entry; entries in higher bins are in, only that one bin is ranked exactly. cand is
 * overwritten. Called by the whole thread block.
 */
__device__ void select_sorted(const Grp &g, FinishShared *sh, Pair *cand, int total, int kq, Pair *sorted) {
    Pair     e[kFinPer];
    unsigned lo = 0xffffffffu, hi = 0u;
#pragma unroll
    for (int i = 0; i < kFinPer; i++) {
        const int f = g.tid + kThreads * i;
        if (f < total) {
            e[i]             = cand[f];
            const unsigned k = order_key(e[i].v);
            lo               = min(lo, k);
            hi               = max(hi, k);
        }
    }
    lo = __reduce_min_sync(0xffffffffu, lo);
    hi = __reduce_max_sync(0xffffffffu, hi);
    g.sync(); /* earlier readers of the scratch are done; every entry is in a register */
    if (g.lane == 0) {
        sh->gs.wred_a[g.warp]                               = (int) lo;
        reinterpret_cast<unsigned *>(sh->gs.wred_f)[g.warp] = hi;
    }
    if (g.tid < kHistBins) {
        sh->bhist[g.tid] = 0;
    }
    if (g.tid == 0) {
        sh->n_sel    = 0;
        sh->n_border = 0;
    }
    g.sync();
#pragma unroll
    for (int w = 0; w < kWarps; w++) {
        lo = min(lo, (unsigned) sh->gs.wred_a[w]);
        hi = max(hi, reinterpret_cast<unsigned *>(sh->gs.wred_f)[w]);
    }
    const unsigned range = hi >= lo ? hi - lo : 0u;
    const int      shift = max(0, (32 - __clz(range)) - 8); /* (range >> shift) < 256 */
#pragma unroll
    for (int i = 0; i < kFinPer; i++) {
        if (g.tid + kThreads * i < total) {
            atomicAdd(&sh->bhist[(order_key(e[i].v) - lo) >> shift], 1);
        }
    }
    g.sync();
    /* b* = largest bin with count(bins >= b*) >= kq; every warp finds it for itself */
    const int b_star = top_bin(sh->bhist, g.lane, kq);
    int       n_hi   = 0;
    for (int b = b_star + 1 + g.lane; b < kHistBins; b += 32) {
        n_hi += sh->bhist[b];
    }
    n_hi = __reduce_add_sync(0xffffffffu, n_hi);
    /* entries above the bin fill cand from the front, the bin's entries follow */
#pragma unroll
    for (int i = 0; i < kFinPer; i++) {
        if (g.tid + kThreads * i < total) {
            const int bin = (int) ((order_key(e[i].v) - lo) >> shift);
            if (bin > b_star) {
                cand[atomicAdd(&sh->n_sel, 1)] = e[i];
            } else if (bin == b_star) {
                cand[n_hi + atomicAdd(&sh->n_border, 1)] = e[i];
            }
        }
    }
    g.sync();
    const int nb   = sh->n_border;
    const int need = kq - n_hi;
    for (int i = g.tid; i < n_hi + nb; i += g.n) {
        const Pair me   = cand[i];
        int        rank = 0;
        if (i < n_hi) {
            for (int j = 0; j < n_hi; j++) {
                rank += pair_before(cand[j].v, cand[j].idx, me.v, me.idx) ? 1 : 0;
            }
            sorted[rank] = me;
        } else {
            for (int j = n_hi; j < n_hi + nb; j++) {
                rank += pair_before(cand[j].v, cand[j].idx, me.v, me.idx) ? 1 : 0;
            }
            if (rank < need) {
                sorted[n_hi + rank] = me;
            }
        }
    }
    g.sync();
}

/* ---------------------------------------------------------------- finisher -- */

/*
 * One row, all threads of a finishing thread block. Merges the parts' records, then by mode: argmax; temperature
 * (segment sums, then the crossing segment re-read and walked); top-k / top-p over the merged candidates. cmem:
 * room for the merged list. Returns the row's status bits (ST_DEFERRED: the multi-pass path has to serve it).
 */
template <bool kFast>
__device__ __forceinline__ int finish_row(const Grp &g, const SampleParams &p, FinishShared *sh, RowCfg &r, unsigned char *cmem) {
    const int  row     = r.row;
    int       *kept_i  = p.kept_cap > 0 ? p.kept_idx + (size_t) row * (size_t) p.kept_cap : nullptr;
    float     *kept_v  = p.kept_cap > 0 ? p.kept_val + (size_t) row * (size_t) p.kept_cap : nullptr;
    Pair      *cbuf    = reinterpret_cast<Pair *>(cmem);
    GroupShared *gs    = &sh->gs;
    const int  b_first = cta_of_item(p, row * p.n_slices);
    const int  b_last  = cta_of_item(p, row * p.n_slices + p.n_slices - 1);
    const int  n_parts = b_last - b_first + 1;
    int        st      = 0;

    g.sync(); /* the staging of the row before is no longer read */
    {
        /* one round trip: the first 256 slots (record + 254 groups) of up to four parts, whatever their counts are */
        float4 tv[kStagedParts];
        int    tb[kStagedParts];
#pragma unroll
        for (int k = 0; k < kStagedParts; k++) {
            tv[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            tb[k] = 0;
            if (k < n_parts) {
                const size_t at = ((size_t) row * (size_t) p.parts_max + (size_t) k) * (size_t) kPartSlots + (size_t) g.tid;
                tv[k]           = __ldcg(p.grp_v + at);
                tb[k]           = __ldcg(p.grp_b + at);
            }
        }
#pragma unroll
        for (int k = 0; k < kStagedParts; k++) {
            sh->st_v[k][g.tid] = tv[k];
            sh->st_b[k][g.tid] = tb[k];
        }
    }
    g.sync();
    if (n_parts > kMaxParts) {
        /* a row spread over that many thread blocks (a handful of rows on the whole chip): its maximum is
         * taken from the records one by one, everything else is left to the multi-pass path */
        float m = -CUDART_INF_F;
        int   a = 0x7fffffff;
        for (int i = g.tid; i < n_parts; i += g.n) {
            const int4  h  = __ldcg(reinterpret_cast<const int4 *>(p.grp_v + ((size_t) row * (size_t) p.parts_max + (size_t) i) * (size_t) kPartSlots));
            const float pm = __int_as_float(h.x);
            st |= h.w;
            if (pair_before(pm, h.y, m, a)) {
                m = pm;
                a = h.y;
            }
        }
        st = __reduce_or_sync(0xffffffffu, st);
        if (g.lane == 0) {
            gs->wred_l[g.warp] = st;
        }
        group_argmax(g, gs, m, a);
        for (int w = 0; w < g.nw; w++) {
            st |= (int) gs->wred_l[w];
        }
        if (r.mode == M_ARGMAX) {
            if (g.tid == 0) {
                p.tokens[row] = a + p.vocab_offset;
                if (p.kept_cap > 0) {
                    p.kept_n[row] = 0;
                }
            }
            return st;
        }
        if (g.tid == 0) {
            gs->blk_max = m;
            gs->blk_arg = a;
        }
        g.sync();
        return st | ST_DEFERRED;
    }
    if (g.tid < n_parts) {
        int4 h, h2;
        if (g.tid < kStagedParts) { /* the record came in with the part's first slots */
            h  = *reinterpret_cast<const int4 *>(&sh->st_v[g.tid][0]);
            h2 = *reinterpret_cast<const int4 *>(&sh->st_v[g.tid][1]);
        } else {
            const int4 *rec = reinterpret_cast<const int4 *>(p.grp_v + ((size_t) row * (size_t) p.parts_max + (size_t) g.tid) * (size_t) kPartSlots);
            h               = __ldcg(rec);
            h2              = __ldcg(rec + 1);
        }
        sh->pmax[g.tid]  = __int_as_float(h.x);
        sh->parg[g.tid]  = h.y;
        sh->pn[g.tid]    = h.z;
        sh->ptau[g.tid]  = __int_as_float(h2.x);
        sh->pbref[g.tid] = __int_as_float(h2.y);
        sh->pbsum[g.tid] = __hiloint2double(h2.w, h2.z);
        st |= h.w;
    }
    st = __reduce_or_sync(0xffffffffu, st);
    if (g.lane == 0) {
        gs->wred_a[g.warp] = st;
    }
    g.sync();
    PROF(9);
    for (int w = 0; w < g.nw; w++) {
        st |= gs->wred_a[w];
    }
    float row_max  = -CUDART_INF_F, tau_row = -CUDART_INF_F;
    int   row_arg  = 0x7fffffff;
    int   others   = 0;
    bool  overflow = false;
    for (int i = 0; i < n_parts; i++) {
        const float m = sh->pmax[i];
        const int   a = sh->parg[i];
        if (pair_before(m, a, row_max, row_arg)) { /* rows that are not greedy carry no id: the plain maximum */
            row_max = m;
            row_arg = a;
        }
        tau_row = fmaxf(tau_row, sh->ptau[i]);
        overflow |= sh->pn[i] > kPartGroups;
        if (g.tid == 0) {
            sh->poff[i] = others;
        }
        others += sh->pn[i];
    }

    if (r.mode == M_ARGMAX) {
        if (g.tid == 0) {
            p.tokens[row] = row_arg + p.vocab_offset;
            if (p.kept_cap > 0) {
                p.kept_n[row] = 0;
            }
        }
        return st;
    }

    if (kFast && r.mode != M_TOPK) {
        return st | ST_DEFERRED; /* temperature and top-p rows: the general finishing kernel's */
    }
    if constexpr (!kFast) {
    if (r.mode == M_TEMP) {
        /* segment sums (one per warp and slice, ids in order), moved from their own maximum to the row maximum */
        const int     nseg   = p.n_slices * kWarps;
        const SegRec *segs   = p.segs + (size_t) row * (size_t) nseg;
        auto          seg_at = [&](int t) {
            const float  ref = __ldcg(&segs[t].ref);
            const double sm  = __ldcg(&segs[t].sum);
            return ref == -CUDART_INF_F ? 0.0 : sm * exp(((double) ref - (double) row_max) * (double) r.inv_t);
        };
        double part = 0.0;
        for (int t = g.tid; t < nseg; t += g.n) {
            part += seg_at(t);
        }
        const double S     = group_sum_d(g, gs, part);
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
                gs->wred_d[g.warp] = incl;
            }
            if (g.tid == 0) {
                gs->pick = 0x7fffffff;
            }
            g.sync();
            double woff = carry;
            for (int w = 0; w < g.warp; w++) {
                woff += gs->wred_d[w];
            }
            incl += woff;
            if (t < nseg && u < incl) {
                atomicMin(&gs->pick, t);
            }
            g.sync();
            const int pk = gs->pick;
            if (pk != 0x7fffffff) {
                if (t == pk) {
                    gs->S = incl - val;
                }
                g.sync();
                found = pk;
                fbase = gs->S;
                break;
            }
            for (int w = 0; w < g.nw; w++) {
                carry += gs->wred_d[w];
            }
        }
        if (found < 0) {
            found = nseg - 1;
        }
        /* the crossing segment, re-read from the row (L2), penalised, walked with the row maximum */
        const int    cc    = found / kWarps, w = found % kWarps;
        const int    s0c   = cc * p.slice;
        const int    nc    = max(0, min(p.slice, p.V - s0c));
        const int    nv4c  = (nc + 3) >> 2;
        const int    Lc    = share_len(nv4c);
        const int    e0    = min(4 * w * Lc, nc);
        const int    e1    = min(4 * min((w + 1) * Lc, nv4c), nc);
        const int    seg_n = max(e1 - e0, 0);
        float       *wbuf  = reinterpret_cast<float *>(cmem); /* >= 1024 floats */
        const float *src   = p.logits + (size_t) row * (size_t) p.row_stride + s0c + e0;
        g.sync();
        for (int i = g.tid; i < seg_n; i += g.n) {
            wbuf[i] = prologue_one(src[i], s0c + e0 + i, r.cap, r.mrow);
        }
        if (r.pen_on) {
            for (int i = g.tid; i < kFinBitmapWords; i += g.n) {
                sh->fin_bitmap[i] = 0u;
            }
            if (g.tid == 0) {
                gs->n_dlist = 0;
            }
        }
        g.sync();
        if (r.pen_on && seg_n > 0) {
            st |= apply_penalties(g, wbuf, s0c + e0, seg_n, r, p.V, p.vocab_offset, sh->fin_bitmap, sh->fdlist, min(p.hist_cap, 512), &gs->n_dlist, false, 0);
        }
        {
            /* every thread takes a run of consecutive entries; the runs' sums are scanned over the
             * group and the thread whose run crosses u walks it */
            const int per = (seg_n + g.n - 1) / g.n; /* <= 4 */
            const int i0  = g.tid * per;
            float     ev[4];
            double    mine = 0.0;
#pragma unroll
            for (int q = 0; q < 4; q++) {
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
                gs->wred_d[g.warp] = incl;
            }
            if (g.tid == 0) {
                gs->pick = 0x7fffffff;
            }
            g.sync();
            double base = fbase;
            for (int ww = 0; ww < g.warp; ww++) {
                base += gs->wred_d[ww];
            }
            if (u < base + incl && i0 < seg_n) {
                atomicMin(&gs->pick, g.tid);
            }
            g.sync();
            const int pk = gs->pick;
            if (pk == 0x7fffffff) {
                if (g.tid == 0) { /* regrouped sums can end a hair below the segment's share */
                    p.tokens[row] = s0c + e0 + max(seg_n - 1, 0) + p.vocab_offset;
                }
            } else if (g.tid == pk) {
                double a   = base + (incl - mine);
                int    hit = min(i0 + per - 1, seg_n - 1);
#pragma unroll
                for (int q = 0; q < 4; q++) {
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
        return st;
    }

    }
    /* ---- top-k and top-p: merge the parts' candidate groups ---- */
    const int n_groups       = others;
    bool      need_multipass = !(r.kq > 0 && r.kq <= kFastKMax) || overflow || n_groups > 8 * kFinCap; /* what counts is how many stay above the row's threshold: checked below */
    if (!need_multipass) {
        const bool keep_all = r.mode == M_TOPP; /* every marked entry was left out of the bulk sums */
        /* The candidates of all parts are merged in up to three passes of one rolled loop. The first keeps what
         * passes the row's threshold (the largest of the parts' thresholds). A row cut into many parts can have far
         * more of those than k (every part kept at least k of its own): if they do not fit, a second pass bins them
         * by value between the threshold and the row's maximum, and a third keeps the bins from the top down to the
         * one in which the kq-th falls. */
        float bin_scale = 0.0f;
        int   bin_min   = 0;
        auto  bin_of    = [&](float v) { return min(kHistBins - 1, max(0, __float2int_rz((v - tau_row) * bin_scale))); };
        int   pass      = 0; /* 0 keep by threshold, 1 bin, 2 keep by bin */
        /* A group is four consecutive values, the id of the first and, in the id's top four bits, which of them
         * passed. The whole warp calls: the entries that stay are counted over the warp and get their places
         * with one atomic per warp. */
        auto place_group = [&](bool valid, const float4 &v, int raw) {
            const int      b  = raw & 0x0fffffff;
            const unsigned cm = valid ? (unsigned) raw >> 28 : 0u;
            bool           k0 = (cm & 1u) && b < p.V && (keep_all || v.x >= tau_row);
            bool           k1 = (cm & 2u) && b + 1 < p.V && (keep_all || v.y >= tau_row);
            bool           k2 = (cm & 4u) && b + 2 < p.V && (keep_all || v.z >= tau_row);
            bool           k3 = (cm & 8u) && b + 3 < p.V && (keep_all || v.w >= tau_row);
            if (pass == 1) {
                if (k0) atomicAdd(&sh->bhist[bin_of(v.x)], 1);
                if (k1) atomicAdd(&sh->bhist[bin_of(v.y)], 1);
                if (k2) atomicAdd(&sh->bhist[bin_of(v.z)], 1);
                if (k3) atomicAdd(&sh->bhist[bin_of(v.w)], 1);
                return;
            }
            if (pass == 2) {
                k0 = k0 && bin_of(v.x) >= bin_min;
                k1 = k1 && bin_of(v.y) >= bin_min;
                k2 = k2 && bin_of(v.z) >= bin_min;
                k3 = k3 && bin_of(v.w) >= bin_min;
            }
            const int      cnt = (int) k0 + (int) k1 + (int) k2 + (int) k3;
            if (__ballot_sync(0xffffffffu, cnt > 0) == 0u) {
                return;
            }
            int incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (g.lane >= o) {
                    incl += up;
                }
            }
            int base = 0;
            if (g.lane == 31) {
                base = atomicAdd(&sh->n_ent, incl);
            }
            base    = __shfl_sync(0xffffffffu, base, 31);
            int pos = base + incl - cnt;
            if (k0) { if (pos < kFinCap) { cbuf[pos].v = v.x; cbuf[pos].idx = b; } pos++; }
            if (k1) { if (pos < kFinCap) { cbuf[pos].v = v.y; cbuf[pos].idx = b + 1; } pos++; }
            if (k2) { if (pos < kFinCap) { cbuf[pos].v = v.z; cbuf[pos].idx = b + 2; } pos++; }
            if (k3) { if (pos < kFinCap) { cbuf[pos].v = v.w; cbuf[pos].idx = b + 3; } pos++; }
        };
        int total = 0;
#pragma unroll 1
        for (pass = 0; pass < 3; pass++) {
            if (g.tid == 0) {
                sh->n_ent = 0;
            }
            if (pass == 1 && g.tid < kHistBins) {
                sh->bhist[g.tid] = 0;
            }
            g.sync();
            /* one loop over the groups of all parts (rolled: code that runs once per row costs what it weighs) */
#pragma unroll 1
            for (int f0 = 0; f0 < others; f0 += g.n) {
                const int  f  = f0 + g.tid;
                const bool ok = f < others;
                int        pi = 0;
                for (int q = 1; q < n_parts; q++) {
                    if (f >= sh->poff[q]) {
                        pi = q; /* offsets ascend */
                    }
                }
                const int slot = f - sh->poff[pi] + 2; /* behind the part's record */
                float4    v    = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                int       b    = 0;
                if (ok) {
                    if (pi < kStagedParts && slot < kThreads) {
                        v = sh->st_v[pi][slot];
                        b = sh->st_b[pi][slot];
                    } else {
                        const size_t at = ((size_t) row * (size_t) p.parts_max + (size_t) pi) * (size_t) kPartSlots + (size_t) slot;
                        v               = __ldcg(p.grp_v + at);
                        b               = __ldcg(p.grp_b + at);
                    }
                }
                place_group(ok, v, b);
            }
            g.sync();
            if (pass == 1) { /* the bin in which the kq-th candidate from the top falls */
                if (g.warp == 0) {
                    const int bb = top_bin(sh->bhist, g.lane, r.kq);
                    if (g.lane == 0) {
                        gs->b_star = bb;
                    }
                }
                g.sync();
                bin_min = gs->b_star;
                g.sync();
                if (bin_min <= 0) {
                    break; /* nothing to gain: the candidates sit in the lowest bin (many equal values) */
                }
                continue;
            }
            total = sh->n_ent;
            if (pass == 2 || total <= kFinCap || keep_all || !(row_max > tau_row) || !(row_max - tau_row < CUDART_INF_F)) {
                break;
            }
            bin_scale = (float) kHistBins / (row_max - tau_row);
        }
        PROF(10);
        if (total > kFinCap || total < r.kq) {
            need_multipass = true;
        }
        if (!need_multipass && r.mode == M_TOPK) {
            const int k = r.k;
            if (total <= kRankAll) {
                /* few candidates: every entry is ranked against all others (a short loop that stays in the
                 * instruction cache, instead of the histogram select's long straight-line code) */
#pragma unroll 1
                for (int i = g.tid; i < total; i += g.n) {
                    const Pair me   = cbuf[i];
                    int        rank = 0;
#pragma unroll 4
                    for (int j = 0; j < total; j++) {
                        rank += pair_before(cbuf[j].v, cbuf[j].idx, me.v, me.idx) ? 1 : 0;
                    }
                    if (rank < k) {
                        sh->fsort[rank] = me;
                    }
                }
                g.sync();
            } else {
                select_sorted(g, sh, cbuf, total, k, sh->fsort);
            }
            PROF(11);
            if (r.select_only) {
                for (int i = g.tid; i < min(k, p.kept_cap); i += g.n) {
                    kept_i[i] = sh->fsort[i].idx + p.vocab_offset;
                    kept_v[i] = sh->fsort[i].v;
                }
                if (g.tid == 0) {
                    p.kept_n[row] = k;
                    p.tokens[row] = sh->fsort[0].idx + p.vocab_offset;
                }
                g.sync();
                return st;
            }
            /* sampler.c:217-222: softmax over the k kept logits (max = the first), one draw */
            const float m = sh->fsort[0].v;
            for (int i = g.tid; i < k; i += g.n) {
                sh->fq[i] = exp_exact(scaled_arg(sh->fsort[i].v, m, r.inv_t));
            }
            g.sync();
            PROF(12);
            if (k <= 64) {
                if (g.tid == 0) { /* sampler.c:90-102 as it stands: the sum and the walk in the reference's order, by one thread */
                    double S = 0.0;
#pragma unroll 1
                    for (int i0 = 0; i0 < k; i0 += 8) { /* eight weights per round: their loads overlap, the sum keeps its order */
                        float w8[8];
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            w8[q] = i0 + q < k ? sh->fq[i0 + q] : 0.0f;
                        }
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            S += (double) w8[q]; /* adding +0 behind the last weight changes nothing */
                        }
                    }
                    const double u    = (double) unit_from(xorshift_next(r.rng)) * S;
                    double       a    = 0.0;
                    int          pick = k - 1;
#pragma unroll 1
                    for (int i0 = 0; i0 < k; i0 += 8) {
                        float w8[8];
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            w8[q] = i0 + q < k ? sh->fq[i0 + q] : 0.0f;
                        }
                        double pre[8]; /* the running sums behind each of the eight, in walk order */
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            a += (double) w8[q];
                            pre[q] = a;
                        }
                        int first = 8;
#pragma unroll
                        for (int q = 7; q >= 0; q--) {
                            if (u < pre[q] && i0 + q < k) {
                                first = q;
                            }
                        }
                        if (first < 8) {
                            pick = i0 + first;
                            break;
                        }
                    }
                    p.tokens[row] = sh->fsort[pick].idx + p.vocab_offset;
                    gs->S         = S;
                    if (p.kept_cap > 0) {
                        p.kept_n[row] = k;
                    }
                }
            } else if (g.warp == 0) {
                double    S;
                const int pick = warp_inverse_cdf(g.lane, sh->fq, k, unit_from(xorshift_next(r.rng)), &S);
                if (g.lane == 0) {
                    p.tokens[row] = sh->fsort[pick].idx + p.vocab_offset;
                    gs->S         = S;
                    if (p.kept_cap > 0) {
                        p.kept_n[row] = k;
                    }
                }
            }
            if (p.kept_cap > 0) {
                g.sync();
                const double S = gs->S;
                for (int i = g.tid; i < min(k, p.kept_cap); i += g.n) {
                    kept_i[i] = sh->fsort[i].idx + p.vocab_offset;
                    kept_v[i] = __double2float_rn((double) sh->fq[i] / S);
                }
            }
            g.sync();
            return st;
        }
        if constexpr (!kFast) {
        if (!need_multipass) {
            /* top-p over a small nucleus (sampler.c:245-300). Candidates get their exact e_i relative to the row
             * maximum; the rest of the row was summed per part with expf relative to a maximum of its own and is
             * rescaled here. */
            double part = 0.0;
            for (int i = g.tid; i < total; i += g.n) {
                const float e = exp_exact(scaled_arg(cbuf[i].v, row_max, r.inv_t));
                cbuf[i].v     = e;
                part += (double) e;
            }
            if (g.tid < n_parts) {
                const float  ref = sh->pbref[g.tid];
                const double sc  = ref == -CUDART_INF_F ? 0.0 : exp(((double) ref - (double) row_max) * (double) r.inv_t);
                part += sc * sh->pbsum[g.tid];
            }
            const double S = group_sum_d(g, gs, part);
            for (int i = g.tid; i < total; i += g.n) {
                cbuf[i].v = __double2float_rn((double) cbuf[i].v / S); /* p_i as the reference normalises it */
            }
            g.sync();
            /* the walk order is (p desc, id asc); the row's kq most probable ids are all candidates */
            const int kq = min(r.kq, total);
            select_sorted(g, sh, cbuf, total, kq, sh->fsort);
            if (g.tid == 0) {
                const float p_floor = sh->fsort[kq - 1].v; /* nothing outside fsort has a larger p */
                double      cum     = 0.0;
                int         cut     = -1;
                for (int i = 0; i < kq; i++) {
                    cum += (double) sh->fsort[i].v;
                    if (cum >= (double) r.top_p) {
                        cut = i + 1;
                        break;
                    }
                }
                const bool all_in = kq >= p.V;
                bool       ok     = cut > 0 && (sh->fsort[cut - 1].v > p_floor || all_in);
                if (cut < 0 && all_in) { /* never reached top_p: the nucleus is the whole row */
                    cut = kq;
                    ok  = true;
                }
                if (ok) {
                    double N = 0.0;
                    for (int i = 0; i < cut; i++) {
                        N += (double) sh->fsort[i].v;
                    }
                    const double u    = (double) unit_from(xorshift_next(r.rng)) * N;
                    double       a    = 0.0;
                    int          pick = cut - 1;
                    for (int i = 0; i < cut; i++) {
                        a += (double) sh->fsort[i].v;
                        if (u < a) {
                            pick = i;
                            break;
                        }
                    }
                    p.tokens[row] = sh->fsort[pick].idx + p.vocab_offset;
                    if (p.kept_cap > 0) {
                        p.kept_n[row] = cut;
                        for (int i = 0; i < min(cut, p.kept_cap); i++) {
                            kept_i[i] = sh->fsort[i].idx + p.vocab_offset;
                            kept_v[i] = __double2float_rn((double) sh->fsort[i].v / N);
                        }
                    }
                }
                gs->flag = ok ? 1 : 0;
            }
            g.sync();
            if (gs->flag) {
                return st;
            }
        }
        }
    }
    g.sync();
    if (g.tid == 0) {
        gs->blk_max = row_max;
        gs->blk_arg = row_arg;
    }
    g.sync();
    return st | ST_DEFERRED;
}

/* ------------------------------------------------------------------ kernel -- */

/* How many ids (history + tokens fed before this row) a row brings. */
__device__ __forceinline__ int row_id_count(const SampleParams &p, int hist_len, int row) {
    const int seq0 = p.rows_per_seq == 1 ? row : row / p.rows_per_seq;
    const int H    = p.hist ? (int) min((long long) max(hist_len, 0), p.hist_stride) : 0;
    const int E    = p.extra ? row - seq0 * p.rows_per_seq : 0;
    return H + E;
}

/*
 * A top-k row that went through one thread block as a whole, finished by that thread block from its own candidate
 * lists (all threads call): the candidates above the part's final threshold are gathered, ranked one against all,
 * the k best get their exact weights and the draw is made as in finish_row. What does not fit here (a warp's list
 * ran over, more than kInlineCap candidates, fewer than k) is handed back with ST_RETRY.
 */
__device__ __forceinline__ void inline_finish_topk(const SampleParams &p, StreamShared *sh, const float4 *grp_v, const int *grp_b, int row, int held, bool complete, float tau_fin,
                                                int k, float inv_t, int st_bits) {
    const int tid = (int) threadIdx.x;
    if (tid == 0) {
        sh->fin_n = 0;
    }
    __syncthreads();
    for (int f = tid; f < held; f += kThreads) {
        const int      slot = own_slot(sh, f);
        const float4   v    = grp_v[slot];
        const int      raw  = grp_b[slot];
        const int      b    = raw & 0x0fffffff;
        const unsigned cm   = (unsigned) raw >> 28;
        const float    c4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            if (((cm >> c) & 1u) != 0u && b + c < p.V && c4[c] >= tau_fin) {
                const int pos = atomicAdd(&sh->fin_n, 1);
                if (pos < kInlineCap) {
                    sh->fin_c[pos].v   = c4[c];
                    sh->fin_c[pos].idx = b + c;
                }
            }
        }
    }
    __syncthreads();
    const int  total = sh->fin_n;
    const bool ok    = complete && total <= kInlineCap && total >= k && k <= kFastKMax;
    if (ok) {
#pragma unroll 1
        for (int i = tid; i < total; i += kThreads) {
            const Pair me   = sh->fin_c[i];
            int        rank = 0;
#pragma unroll 4
            for (int j = 0; j < total; j++) {
                rank += pair_before(sh->fin_c[j].v, sh->fin_c[j].idx, me.v, me.idx) ? 1 : 0;
            }
            if (rank < k) {
                sh->fin_s[rank] = me;
            }
        }
        __syncthreads();
        const float m = sh->fin_s[0].v;
        for (int i = tid; i < k; i += kThreads) {
            sh->fin_q[i] = exp_exact(scaled_arg(sh->fin_s[i].v, m, inv_t));
        }
        __syncthreads();
    }
    if (tid == 0) {
        unsigned long long rng = sh->cur_rng; /* the sequence's word; this row starts cur_rr draws behind it */
        for (int i = 0; i < sh->cur_rr; i++) {
            (void) xorshift_next(rng);
        }
        int tok = -1;
        if (ok) {
            /* sampler.c:90-102: the sum and the walk in the reference's order, eight weights per step (their loads overlap) */
            double S = 0.0;
#pragma unroll 1
            for (int i0 = 0; i0 < k; i0 += 8) {
                float w8[8];
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    w8[q] = i0 + q < k ? sh->fin_q[i0 + q] : 0.0f;
                }
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    S += (double) w8[q];
                }
            }
            const double u    = (double) unit_from(xorshift_next(rng)) * S;
            double       a    = 0.0;
            int          pick = k - 1;
#pragma unroll 1
            for (int i0 = 0; i0 < k; i0 += 8) {
                float w8[8];
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    w8[q] = i0 + q < k ? sh->fin_q[i0 + q] : 0.0f;
                }
                double pre[8];
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    a += (double) w8[q];
                    pre[q] = a;
                }
                int first = 8;
#pragma unroll
                for (int q = 7; q >= 0; q--) {
                    if (u < pre[q] && i0 + q < k) {
                        first = q;
                    }
                }
                if (first < 8) {
                    pick = i0 + first;
                    break;
                }
            }
            tok = sh->fin_s[pick].idx + p.vocab_offset;
        } else {
            (void) xorshift_next(rng);
            st_bits |= ST_RETRY;
        }
        p.tokens[row] = tok;
        p.status[row] = st_bits;
        if (p.rng_out != nullptr && sh->cur_last) {
            p.rng_out[sh->cur_seq] = rng; /* the word after the sequence's last row */
        }
    }
    __syncthreads();
}

/*
 * A row's parameters cost up to two dependent memory round trips (slot -> parameters and history ids). Warp 0
 * fetches them for the NEXT row of the run with 4-byte asynchronous copies into shared memory, one step per
 * slice of the part in work, so that nothing waits for them when that row begins. The history ids are asked for
 * before the row's history length is known: the first kRowIds words of the session's history row (they exist,
 * whatever the length is), and the tokens fed before this row into a list of their own. `stage`: 0 nothing asked
 * yet, 1 the slot, 2 everything. Called by all lanes of warp 0.
 */
constexpr int kPrefetchDone = 2;
__device__ __forceinline__ void prefetch_step(const SampleParams &p, StreamShared *sh, int row, int lane, int &stage) {
    const int seq0 = p.rows_per_seq == 1 ? row : row / p.rows_per_seq;
    if (stage == 0) {
        if (lane == 0) {
            if (p.slot) {
                copy_word_async(&sh->raw_nxt.seq, &p.slot[seq0]);
            } else {
                sh->raw_nxt.seq = seq0;
            }
        }
        stage = 1;
        if (p.slot) {
            return; /* the slot must arrive first */
        }
    }
    async_copies_wait();
    __syncwarp();
    const int seq = *reinterpret_cast<volatile int *>(&sh->raw_nxt.seq);
    if (lane == 0) copy_word_async(&sh->raw_nxt.T, &p.temperature[seq]);
    if (lane == 1) copy_word_async(&sh->raw_nxt.top_k, &p.top_k[seq]);
    if (lane == 2) copy_word_async(&sh->raw_nxt.top_p, &p.top_p[seq]);
    if (lane == 3) { if (p.hist) copy_word_async(&sh->raw_nxt.hist_len, &p.hist_len[seq]); else sh->raw_nxt.hist_len = 0; }
    if (lane == 4) { if (p.rep) copy_word_async(&sh->raw_nxt.rep, &p.rep[seq]); else sh->raw_nxt.rep = 1.0f; }
    if (lane == 5) { if (p.freq) copy_word_async(&sh->raw_nxt.freq, &p.freq[seq]); else sh->raw_nxt.freq = 0.0f; }
    if (lane == 6) { if (p.pres) copy_word_async(&sh->raw_nxt.pres, &p.pres[seq]); else sh->raw_nxt.pres = 0.0f; }
    if (lane == 9) { if (p.softcap) copy_word_async(&sh->raw_nxt.cap, &p.softcap[seq]); else sh->raw_nxt.cap = 0.0f; }
    if (lane == 7 || lane == 8) {
        unsigned *dst = reinterpret_cast<unsigned *>(&sh->raw_nxt.rng) + (lane - 7);
        if (p.rng_in) copy_word_async(dst, reinterpret_cast<const unsigned *>(&p.rng_in[seq]) + (lane - 7)); else *dst = lane == 7 ? 1u : 0u;
    }
    if (p.hist) {
        const int hs = (int) min((long long) kRowIds, p.hist_stride);
        for (int t = lane; t < hs; t += 32) {
            copy_word_async(&sh->nxt_ids[t], &p.hist[(size_t) seq * (size_t) p.hist_stride + t]);
        }
    }
    if (p.extra) {
        const int E = min(row - seq0 * p.rows_per_seq, kRowIds);
        for (int t = lane; t < E; t += 32) {
            copy_word_async(&sh->nxt_ext[t], &p.extra[(size_t) seq0 * (size_t) p.extra_stride + 1 + t]);
        }
    }
    stage = kPrefetchDone;
}

/* Which kinds of rows an instantiation of the stream kernel carries the code for: every one carries greedy rows;
 * K_SEL adds the candidate select of top-k rows, K_SUMS the sums of temperature and top-p rows (and top-p's select).
 * A launch whose caller vouched for its rows' kinds (finish_hint) runs the instantiation without the rest: less
 * code to fetch, fewer live registers in the slice loop; likewise a launch without histories runs one without the
 * penalties' code. A row of a kind that is not carried is streamed as a
 * greedy row and reported (ROW_INTERNAL) where the launch's rows are finished. */
constexpr int K_SEL = 1, K_SUMS = 2, K_PEN = 4, K_PLAIN = 8, K_SHORT = 16; /* K_PEN: the launch brings history ids or fed tokens (penalties) */
template <int kKinds>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) sample_stream_kernel(const __grid_constant__ SampleParams p) {
    /* K_PLAIN: rows on the 16-byte grid, no soft cap, mask or logits output; K_SHORT: no row with more ids than the
     * thread block counts by itself. The launch's host side has checked it, the code for the rest is left out. */
    constexpr bool kPlain  = (kKinds & K_PLAIN) != 0;
    const bool     aligned = kPlain || p.aligned != 0;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char *ring    = smem_raw;
    StreamShared  *sh      = reinterpret_cast<StreamShared *>(smem_raw + (size_t) kWarps * kStages * kWarpStageBytes);
    unsigned char *gmem    = reinterpret_cast<unsigned char *>(sh + 1); /* candidate groups of the part in work */
    float4        *grp_v   = reinterpret_cast<float4 *>(gmem);
    int           *grp_b   = reinterpret_cast<int *>(gmem + (size_t) kPartGroups * 16);
    int           *sl_off  = reinterpret_cast<int *>(gmem + kGroupBytes); /* long histories: where each slice's run of the prepared list starts */
    unsigned      *sl_list = reinterpret_cast<unsigned *>(gmem + kGroupBytes + ((((size_t) p.n_slices + 1) * 4 + 15) & ~(size_t) 15)); /* ... and the part's entries, when they fit */

    Grp g;
    g.tid  = (int) threadIdx.x;
    g.lane = g.tid & 31;
    g.warp = g.tid >> 5;
    g.n    = kThreads;
    g.nw   = kWarps;
    g.bar  = 0;
    const int      tid = g.tid, lane = g.lane, warp = g.warp;
    const unsigned lt  = (1u << lane) - 1u;

    /* every thread block takes a contiguous run of the (row, slice) items */
    int my_first, my_count;
    run_of_cta(p, (int) blockIdx.x, my_first, my_count);

    if (tid == 0) {
        for (int w = 0; w < kWarps; w++) {
            for (int s = 0; s < kStages; s++) {
                mbar_init_only(&sh->full[w][s], 1);
            }
        }
        mbar_init_fence();
    }
    __syncthreads();
    /* Launched as a programmatic dependent of the kernel before it in the stream: the thread block may have
     * been placed while that kernel's last blocks were still at work. Everything it touches in global memory
     * waits here for that kernel to be complete and visible, so the stream's order is kept; what is saved is
     * the gap between two grids. The kernel behind this one may be placed likewise. */
    if (lane == 0 && aligned) {
        /* While it waits, the thread block asks L2 for what its ring will copy first (the warp's shares of the run's
         * first kStages items). Nothing is read: a line that the kernel before this one is still writing arrives in
         * L2 with its stores either way. Back to back this is worth 0.5 us per launch: the last thread blocks of the
         * grid before leave DRAM idle. */
        const int n_full_ = min(p.slice, p.V), n_last_ = p.V - (p.n_slices - 1) * p.slice;
        for (int jj = 0; jj < min(kStages, my_count); jj++) {
            const int item = my_first + jj, r_ = item / p.n_slices, c_ = item - r_ * p.n_slices;
            const int n_   = c_ == p.n_slices - 1 ? n_last_ : n_full_;
            const int nv4_ = (n_ + 3) >> 2, L_ = share_len(nv4_);
            const int lo_  = min(warp * L_, nv4_);
            const int b4_  = max(0, min(min(L_, nv4_ - lo_), (n_ >> 2) - lo_));
            if (b4_ > 0) {
                bulk_prefetch_l2(p.logits + (size_t) r_ * (size_t) p.row_stride + (size_t) c_ * (size_t) p.slice + 4 * lo_, (unsigned) b4_ * 16u);
            }
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
#ifdef GB_PROFILE
    if (tid == 0 && blockIdx.x < 1024) {
        for (int i = 1; i < 16; i++) {
            g_prof[blockIdx.x][i] = 0;
        }
    }
#endif
    PROF(0);

    /* ---- the warp's own ring: lane 0 asks for the warp's share of the item kStages ahead ---- */
    unsigned char *wring = ring + (size_t) warp * kStages * kWarpStageBytes;
    /* a row's slices have one of two shapes: the full one and the row's last one; what the warp owns of each */
    const int n_full = min(p.slice, p.V), n_last = p.V - (p.n_slices - 1) * p.slice;
    int       w4lo_f, mine4_f, w4lo_l, mine4_l;
    {
        const int nv4f = (n_full + 3) >> 2, Lf = share_len(nv4f);
        w4lo_f         = min(warp * Lf, nv4f);
        mine4_f        = min(Lf, nv4f - w4lo_f);
        const int nv4l = (n_last + 3) >> 2, Ll = share_len(nv4l);
        w4lo_l         = min(warp * Ll, nv4l);
        mine4_l        = min(Ll, nv4l - w4lo_l);
    }
    const int    bulk4_f = max(0, min(mine4_f, (n_full >> 2) - w4lo_f)); /* float4 of the share that a bulk copy brings */
    const int    bulk4_l = max(0, min(mine4_l, (n_last >> 2) - w4lo_l));
    int          irow = my_first / p.n_slices, ic = my_first - irow * p.n_slices, ijj = 0; /* the next item to request */
    const float *isrc = p.logits + (size_t) irow * (size_t) p.row_stride + (size_t) ic * (size_t) p.slice; /* ... and where its slice starts */
    auto issue_next = [&]() {
        const bool last  = ic == p.n_slices - 1;
        const int  b4    = last ? bulk4_l : bulk4_f;
        const int  stage = ijj % kStages;
        if (b4 > 0) {
            mbar_expect_tx(&sh->full[warp][stage], (unsigned) b4 * 16u);
            bulk_g2s(wring + (size_t) stage * kWarpStageBytes, isrc + 4 * (last ? w4lo_l : w4lo_f), (unsigned) b4 * 16u, &sh->full[warp][stage]);
        }
        ijj++;
        ic++;
        isrc += p.slice;
        if (last) {
            ic = 0;
            isrc += p.row_stride - (long long) p.n_slices * p.slice; /* on to the next row */
        }
    };
    if (lane == 0 && aligned) {
        for (int jj = 0; jj < min(kStages, my_count); jj++) {
            issue_next();
        }
    }

    CYC_INIT();
    int j         = 0;
    int ring_dead = -1; /* the item at which a copy of this warp failed to arrive in time (-1: none) */
    int pf        = 0; /* warp 0: how far the parameters of the row that begins next have been fetched */
    while (j < my_count) {
        const int  item0 = my_first + j, row = item0 / p.n_slices, c0 = item0 - row * p.n_slices;
        const int  part_len   = min(p.n_slices - c0, my_count - j);
        const bool final_part = j + part_len == my_count;
        CYC(6);
        if (warp == 0) { /* what has not been fetched while the previous part streamed (first part, short parts) */
            while (pf < kPrefetchDone) {
                prefetch_step(p, sh, row, lane, pf);
            }
            async_copies_wait();
            pf = 0;
        }
        __syncthreads();
        PROF_ONCE(1);
        int   mode, kq, n_ids, my_id = -1;
        float inv_t, rep, freq, pres;
        bool  pen_on, pro_on;
        {
            const RawCfg raw = sh->raw_nxt;
            const RowCfg r   = row_config(p, row, raw, false); /* what the finisher needs more of is derived again when the row is complete */
            mode   = (int) r.mode;
            kq     = r.kq;
            inv_t  = r.inv_t;
            n_ids  = r.H + r.E;
            pen_on = (kKinds & K_PEN) != 0 && r.pen_on && n_ids > 0;
            rep    = r.rep;
            freq   = r.freq;
            pres   = r.pres;
            pro_on = !kPlain && (r.cap > 0.0f || r.mrow != nullptr);
            if (tid == 0) { /* read again by the warps only if pro_on; the barriers of the part set-up lie between */
                sh->cap      = r.cap;
                sh->mrow     = r.mrow;
                sh->cur_rng  = raw.rng;
                sh->cur_seq  = r.seq;
                sh->cur_last = r.rr == p.rows_per_seq - 1 ? 1 : 0;
                sh->cur_rr   = r.rr;
            }
            if (tid < n_ids && n_ids <= kRowIds) {
                my_id = tid < r.H ? sh->nxt_ids[tid] : sh->nxt_ext[tid - r.H];
            }
        }
        /* the kind the row is streamed as */
        const int   smode   = ((kKinds & K_SUMS) == 0 && (mode == M_TEMP || mode == M_TOPP)) || ((kKinds & K_SEL) == 0 && mode == M_TOPK) ? (int) M_ARGMAX : mode;
        const bool  sel     = (kKinds & K_SEL) != 0 && (smode == M_TOPK || ((kKinds & K_SUMS) != 0 && smode == M_TOPP)) && kq > 0 && kq <= kFastKMax;
        const bool  sums    = (kKinds & K_SUMS) != 0 && (smode == M_TEMP || (smode == M_TOPP && sel));
        const bool  long_ids = (kKinds & K_SHORT) == 0 && n_ids > kRowIds;
        const int   b_first = cta_of_item(p, row * p.n_slices);
        const int   part_idx = (int) blockIdx.x - b_first;
        const int   n_parts = cta_of_item(p, row * p.n_slices + p.n_slices - 1) - b_first + 1;

        /* ---- part set-up ---- */
        if (tid == 0) {
            sh->st       = 0;
            sh->tau_key  = 0u;
            sh->tau_lock = 0;
            sh->fin_n    = 0;
        }
        if (tid < kHistBins) {
            sh->thist[tid] = 0;
            sh->bhist[tid] = 0;
        }
        if (tid < kWarps) {
            sh->wcur[tid] = 0;
            sh->wsq[tid] = -CUDART_INF_F;
        }
        if (pen_on && !long_ids) {
            /* The row's distinct ids with their counts: an open-addressing table in the groups' memory (free
             * between two parts), one id per thread; the thread whose id opened a slot speaks for that id. The ids
             * are then grouped by the (slice, warp) share of the part that they fall into, so that a warp looks at
             * its own share's run alone (most shares hold none): kRowIds groups, slice c of the part and slice
             * c + 32 share one and tell their ids apart by a tag. Entry: offset in the share | count << 10 | tag << 20. */
            int *id_key = reinterpret_cast<int *>(gmem);
            int *id_cnt = id_key + 2 * kRowIds;
            for (int i = tid; i < 2 * kRowIds; i += kThreads) {
                id_key[i] = -1;
                id_cnt[i] = 0;
            }
            for (int i = tid; i <= kRowIds; i += kThreads) {
                sh->rl_cnt[i] = 0; /* entry g + 1: ids in group g; after the scan, entry g: ids in the groups before g */
            }
            int id = my_id;
            if (tid < n_ids) {
                id -= p.vocab_offset;
                if (id < 0 || id >= p.V) {
                    id = -1;
                }
            } else {
                id = -1;
            }
            /* which group holds the id (-1: a slice of another part of the row), and the rest of its entry */
            auto group_of = [&](int gid, int &rest) {
                const int c = gid / p.slice;
                if (c < c0 || c >= c0 + part_len) {
                    return -1;
                }
                const int local = gid - c * p.slice;
                const int L     = share_len(((c == p.n_slices - 1 ? n_last : n_full) + 3) >> 2); /* float4 per warp */
                const int w     = (local >> 2) / L;
                rest            = (local - 4 * w * L) | (((c - c0) >> 5) << 20);
                return ((c - c0) & 31) * kWarps + w;
            };
            __syncthreads();
            int slot = -1, place = -1;
            if (id >= 0) {
                unsigned h = ((unsigned) id * 2654435761u) >> (32 - 9);
                for (int probe = 0; probe < 2 * kRowIds; probe++) {
                    const int old = atomicCAS(&id_key[h], -1, id);
                    if (old == -1 || old == id) {
                        atomicAdd(&id_cnt[h], 1);
                        slot = old == -1 ? (int) h : -1;
                        break;
                    }
                    h = (h + 1) & (2 * kRowIds - 1);
                }
                if (slot >= 0) {
                    int       rest;
                    const int grp = group_of(id, rest);
                    if (grp >= 0) {
                        place = atomicAdd(&sh->rl_cnt[grp + 1], 1);
                    }
                }
            }
            __syncthreads();
            if (warp == 0) { /* running sums over the kRowIds counters, eight per lane */
                int v[8], run = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    run += sh->rl_cnt[1 + 8 * lane + i];
                    v[i] = run;
                }
                int before = run;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int o = __shfl_up_sync(0xffffffffu, before, d);
                    if (lane >= d) {
                        before += o;
                    }
                }
                before -= run;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    sh->rl_cnt[1 + 8 * lane + i] = before + v[i];
                }
            }
            __syncthreads();
            if (place >= 0) {
                int       rest;
                const int grp = group_of(id, rest);
                sh->rl_id[sh->rl_cnt[grp] + place] = rest | (id_cnt[slot] << 10);
            }
        } else if (pen_on) {
            /* long histories: a kernel that ran before this one left the row's distinct ids with their counts
             * in global memory, grouped by slice; the part copies where its slices' runs start */
            const int *off = p.pre_off + (size_t) row * (size_t) (p.n_slices + 1) + c0;
            for (int i = tid; i <= part_len; i += kThreads) {
                sl_off[i] = off[i];
            }
            /* the part's entries themselves come along when there are at most kListSmem of them: the slices then
             * read them from shared memory instead of paying a round trip to L2 each */
            const int e_lo = off[0], e_n = off[part_len] - e_lo;
            if (e_n <= kListSmem) {
                const unsigned *src = p.pre_list + (size_t) row * (size_t) p.row_cap + e_lo;
                for (int i = tid; i < e_n; i += kThreads) {
                    sl_list[i] = src[i];
                }
            }
        }
        __syncthreads();
        static_assert(2 * kRowIds == 512, "the id table's hash keeps 9 bits");

        PROF_ONCE(3);
        CYC(5);
        const double rep_rcp = pen_on ? 1.0 / (double) rep : 1.0;
        unsigned run_key = 0u; /* this warp's maximum of the part so far (key) and its first id */
        int      run_arg = 0x7fffffff;
        float    tau_reg = -CUDART_INF_F, t_lo = 0.0f, t_scale = 0.0f;
        int      wcnt = 0, since = 0; /* this warp's candidate groups of the part; those since it last looked at the threshold */
        float    b_ref = -CUDART_INF_F; /* top-p: running sum of what is no candidate, relative to b_ref */
        double   b_sum = 0.0;
        int      wst   = 0;
        float4  *seg_v = grp_v + warp * kGroupCapWarp;
        int     *seg_b = grp_b + warp * kGroupCapWarp;

        /* ---- the part's slices, every warp on its own ---- */
        for (int s = 0; s < part_len; s++, j++) {
            const int      stage  = j % kStages;
            const unsigned parity = (unsigned) (j / kStages) & 1u;
            const int      c      = c0 + s, s0 = c * p.slice;
            const bool     last_c = c == p.n_slices - 1;
            const int      n = last_c ? n_last : n_full, nv4 = (n + 3) >> 2, body = n & ~3;
            const int      w4lo = last_c ? w4lo_l : w4lo_f, mine4 = last_c ? mine4_l : mine4_f;
            float         *sl   = reinterpret_cast<float *>(wring + (size_t) stage * kWarpStageBytes); /* local index = slice index - 4 * w4lo */
            const float   *grow = p.logits + (size_t) row * (size_t) p.row_stride + s0;
            bool           wrote = !aligned; /* the warp wrote into its stage with ordinary stores */
            if (warp == 0 && !final_part && pf < kPrefetchDone) {
                prefetch_step(p, sh, row + 1, lane, pf); /* one step per slice: the step before has long arrived */
            }
            CYC(4);
            /* ---- 1. the warp's share of the slice is in its stage; the slice's tail is padded with -inf ---- */
            if (aligned) {
                const int full4 = last_c ? bulk4_l : bulk4_f;
                if (ring_dead >= 0) {
                    wst |= ST_LOAD_TIMEOUT; /* every row the warp still touches is reported as not loaded */
                } else if (full4 > 0 && !mbar_wait_bounded(&sh->full[warp][stage], parity)) {
                    wst |= ST_LOAD_TIMEOUT;
                    ring_dead = j; /* the warp asks for no further copy and waits for none; see the kernel's end */
                }
                if (nv4 * 4 > body && w4lo + mine4 == nv4 && mine4 > 0) {
                    wrote = true;
                    if (lane < 4) {
                        const int i      = body + lane; /* the last float4 is not part of the bulk copy */
                        sl[i - 4 * w4lo] = i < n ? grow[i] : -CUDART_INF_F;
                    }
                }
            } else {
                /* rows off the 16-byte grid: plain loads into the warp's own stage */
                for (int i = lane; i < 4 * mine4; i += 32) {
                    const int gi = 4 * w4lo + i;
                    sl[i]        = gi < n ? grow[gi] : -CUDART_INF_F;
                }
            }
            __syncwarp();
            CYC(0);

            /* ---- 1b. soft cap and mask, in place ---- */
            if (pro_on) {
                wrote = true;
                prologue_share(sl, lane, mine4, 4 * w4lo, n, s0, sh->cap, sh->mrow);
            }

            /* ---- 2. penalties on the share ---- */
            if (pen_on) {
                bool touched = false; /* most shares hold none of the row's ids: those need no fence before the refill */
                if (!long_ids) {
                    const int grp = (s & 31) * kWarps + warp;
                    const int lo = sh->rl_cnt[grp], hi = sh->rl_cnt[grp + 1];
                    for (int e = lo + lane; e < hi; e += 32) {
                        const unsigned en = (unsigned) sh->rl_id[e];
                        if ((int) (en >> 20) == (s >> 5)) {
                            float *q = sl + (en & 0x3ffu);
                            *q       = penalise_rcp(*q, (int) ((en >> 10) & 0x3ffu), rep_rcp, rep, freq, pres);
                            touched  = true;
                        }
                    }
                } else {
                    const unsigned *src = p.pre_list + (size_t) row * (size_t) p.row_cap;
                    const int       lo = sl_off[s], hi = sl_off[s + 1], e_lo = sl_off[0];
                    const bool      in_smem = sl_off[part_len] - e_lo <= kListSmem;
                    for (int i = lo + lane; i < hi; i += 32) {
                        const unsigned e  = in_smem ? sl_list[i - e_lo] : src[i];
                        const int      li = (int) (e & ((1u << kLiBits) - 1u));
                        if (li >= 4 * w4lo && li < 4 * (w4lo + mine4) && li < n) {
                            sl[li - 4 * w4lo] = penalise_rcp(sl[li - 4 * w4lo], (int) (e >> kLiBits), rep_rcp, rep, freq, pres);
                            touched           = true;
                        }
                    }
                }
                wrote |= __any_sync(0xffffffffu, touched); /* also orders the stores before the loads below */
            }
            if (!kPlain && p.out_logits != nullptr) {
                float *orow = p.out_logits + (size_t) row * (size_t) p.V + s0;
                for (int i = 4 * w4lo + lane; i < min(4 * (w4lo + mine4), n); i += 32) {
                    orow[i] = sl[i - 4 * w4lo];
                }
            }

            /* ---- 3. the share in registers; what a thread does not own reads as -inf ---- */
            const float4 *s4 = reinterpret_cast<const float4 *>(sl) + lane;
            float4        x[kNV4];
            float         gm[kNV4]; /* maximum of each float4 group */
            float         bv = -CUDART_INF_F;
#pragma unroll
            for (int i = 0; i < kNV4; i++) {
                x[i]  = lane + 32 * i < mine4 ? s4[32 * i] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
                gm[i] = fmaxf(fmaxf(x[i].x, x[i].y), fmaxf(x[i].z, x[i].w));
                bv    = fmaxf(bv, gm[i]);
            }
            CYC(1);
            const unsigned bkey = order_key(bv + 0.0f); /* -0 and +0 are one value, as the comparison of floats has it */
            const bool     own  = lane < mine4;
            const unsigned wkey = __reduce_max_sync(0xffffffffu, own ? bkey : 0u);
            const float    wmax = wkey == 0u ? -CUDART_INF_F : key_to_float(wkey);

            if (smode == M_ARGMAX) {
                if (wkey > run_key) { /* rare: the warp's running maximum moves; its first id in this slice */
                    int best = 0x7fffffff;
                    if (own && bkey == wkey) {
#pragma unroll
                        for (int i = kNV4 - 1; i >= 0; i--) {
                            const int b = 4 * (w4lo + lane + 32 * i);
                            if (x[i].w == wmax) best = b + 3;
                            if (x[i].z == wmax) best = b + 2;
                            if (x[i].y == wmax) best = b + 1;
                            if (x[i].x == wmax) best = b;
                        }
                    }
                    best    = __reduce_min_sync(0xffffffffu, best);
                    run_key = wkey;
                    run_arg = s0 + best;
                }
            } else if (wkey > run_key) {
                run_key = wkey; /* the maximum alone: no other mode asks where it is */
            }

            float tau = CUDART_INF_F;
            if (sel) {
                if (s == 0) {
                    /* The part's first slice sets the threshold; all warps meet here (the only barriers inside a
                     * part). The thread maxima (wide k: the float4 maxima) are binned by their ordered keys into 256
                     * bins below the largest, and tau = the lower edge of the highest bin above which at least kq of
                     * them lie: at least kq entries of this slice alone are >= tau, so tau cannot exceed the row's
                     * kq-th largest value. Fewer than kq groups: everything passes. */
                    const bool fine = kq > 64;
                    float      gmin = bv;
                    int        ng   = own ? 1 : 0;
                    if (fine) {
                        gmin = CUDART_INF_F;
                        ng   = 0;
#pragma unroll
                        for (int i = 0; i < kNV4; i++) {
                            if (lane + 32 * i < mine4) {
                                gmin = fminf(gmin, gm[i]);
                                ng++;
                            }
                        }
                    }
                    const unsigned wlow = __reduce_min_sync(0xffffffffu, own ? order_key(gmin + 0.0f) : 0xffffffffu);
                    ng                  = __reduce_add_sync(0xffffffffu, ng);
                    if (lane == 0) {
                        sh->wkey[warp] = wkey;
                        sh->wlow[warp] = wlow;
                        sh->wown[warp] = ng;
                    }
                    __syncthreads();
                    unsigned khi = 0u, klo = 0xffffffffu;
                    int      n_own = 0;
#pragma unroll
                    for (int w = 0; w < kWarps; w++) {
                        khi = max(khi, sh->wkey[w]);
                        klo = min(klo, sh->wlow[w]);
                        n_own += sh->wown[w];
                    }
                    /* values far below the largest all go to bin 0: the walk comes from the top */
                    const unsigned klo2  = max(klo, khi > (1u << 27) ? khi - (1u << 27) : 0u);
                    const unsigned span  = khi - klo2;
                    const int      shift = max(0, (32 - __clz(span)) - 8); /* (span >> shift) < 256 */
                    if (n_own >= kq) {
                        if (fine) {
#pragma unroll
                            for (int i = 0; i < kNV4; i++) {
                                if (lane + 32 * i < mine4) {
                                    atomicAdd(&sh->bhist[(max(order_key(gm[i] + 0.0f), klo2) - klo2) >> shift], 1);
                                }
                            }
                        } else {
                            /* most thread maxima fall into a few low bins: the lanes of a warp that share a bin
                             * add once for all of them */
                            const int      bin   = own ? (int) ((max(bkey, klo2) - klo2) >> shift) : -1;
                            const unsigned peers = __match_any_sync(0xffffffffu, bin);
                            if (own && lane == __ffs(peers) - 1) {
                                atomicAdd(&sh->bhist[bin], __popc(peers));
                            }
                        }
                    }
                    __syncthreads();
                    unsigned tkey = 0u; /* below everything: all entries pass */
                    if (n_own >= kq) { /* every warp reads the bins for itself */
                        const int b = top_bin(sh->bhist, lane, kq);
                        tkey        = b == 0 ? klo : klo2 + ((unsigned) b << shift); /* bin 0 also holds what was clamped */
                    }
                    tau_reg = tkey == 0u ? -CUDART_INF_F : key_to_float(tkey);
                    /* the part's candidates are binned between tau and this slice's maximum; the bins are read from
                     * the top to raise the threshold for the slices to come */
                    const float top = key_to_float(khi);
                    t_lo            = tau_reg;
                    t_scale         = (n_own >= kq && top > tau_reg && top - tau_reg < CUDART_INF_F) ? (float) kHistBins / (top - tau_reg) : 0.0f;
                }
                CYC(7);
                PROF_ONCE(7);
                const unsigned pkey = *reinterpret_cast<volatile unsigned *>(&sh->tau_key);
                tau                 = pkey == 0u ? tau_reg : fmaxf(tau_reg, key_to_float(pkey));
                /* Candidates: the float4 groups whose maximum passes. Which of a thread's eight groups do is one bit
                 * each; a lane that holds any takes them one after the other in ONE rolled loop (rarely run code
                 * inside the hot loop is kept in one copy: it has to come from the instruction cache each time), the
                 * values re-read from the stage. */
                unsigned mybits = 0u;
#pragma unroll
                for (int i = 0; i < kNV4; i++) {
                    mybits |= (gm[i] >= tau && lane + 32 * i < mine4) ? (1u << i) : 0u;
                }
                if (__any_sync(0xffffffffu, mybits != 0u)) {
                    /* every lane that holds candidates places its groups itself, the places counted in shared memory:
                     * one pass whatever the number of lanes and groups (the order inside the list means nothing) */
                    unsigned mb = mybits;
                    while (mb != 0u) {
                        const int i = __ffs(mb) - 1;
                        mb &= mb - 1u;
                        const float4 v   = s4[32 * i];
                        const int    pos = atomicAdd(&sh->wcur[warp], 1);
                        if (pos < kGroupCapWarp) {
                            /* which of the four pass: the finisher takes those, the sums below leave those out */
                            const unsigned cm = (v.x >= tau ? 1u : 0u) | (v.y >= tau ? 2u : 0u) | (v.z >= tau ? 4u : 0u) | (v.w >= tau ? 8u : 0u);
                            seg_v[pos]        = v;
                            seg_b[pos]        = (s0 + 4 * (w4lo + lane + 32 * i)) | (int) (cm << 28);
                        }
                        if (t_scale > 0.0f) {
                            const float gmax = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
                            atomicAdd(&sh->thist[min(kHistBins - 1, max(0, __float2int_rz((gmax - t_lo) * t_scale)))], 1);
                        }
                    }
                    __syncwarp();
                    const int now = *reinterpret_cast<volatile int *>(&sh->wcur[warp]);
                    since += now - wcnt;
                    wcnt = now;
                }
            }
            CYC(2);
            /* the stage is free again: the warp refills it itself */
            __syncwarp();
            if (lane == 0 && aligned && j + kStages < my_count && ring_dead < 0) {
                if (wrote) { /* ordinary stores of this warp come before the copy engine's */
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                issue_next();
            }
            CYC(1);
            if (sums) {
                /* sum of e_i relative to the WARP's maximum of this slice (top-p: of what is in no candidate
                 * group); -inf padding gives exp(-inf) = 0 */
                const float ref = wmax == -CUDART_INF_F ? 0.0f : wmax;
                const float k2  = inv_t * 1.4426950408889634f; /* e^(a / T) = 2^(a * log2(e) / T) */
                double      sum = 0.0;
#pragma unroll
                for (int i = 0; i < kNV4; i++) {
                    /* a candidate's argument becomes -inf (exp gives 0), so that the evaluations stay one straight
                     * line and overlap */
                    const float e0 = exp2_fast(x[i].x >= tau ? -CUDART_INF_F : (x[i].x - ref) * k2);
                    const float e1 = exp2_fast(x[i].y >= tau ? -CUDART_INF_F : (x[i].y - ref) * k2);
                    const float e2 = exp2_fast(x[i].z >= tau ? -CUDART_INF_F : (x[i].z - ref) * k2);
                    const float e3 = exp2_fast(x[i].w >= tau ? -CUDART_INF_F : (x[i].w - ref) * k2);
                    sum += (double) ((e0 + e1) + (e2 + e3));
                }
                sum = warp_sum_d(sum);
                if (smode == M_TEMP) {
                    if (lane == 0) {
                        SegRec sr;
                        sr.ref = wmax;
                        sr.pad = 0.0f;
                        sr.sum = sum;
                        p.segs[((size_t) row * (size_t) p.n_slices + (size_t) c) * kWarps + warp] = sr;
                    }
                } else if (wmax != -CUDART_INF_F) {
                    if (wmax > b_ref) {
                        b_sum = b_ref == -CUDART_INF_F ? 0.0 : b_sum * exp(((double) b_ref - (double) wmax) * (double) inv_t);
                        b_ref = wmax;
                    }
                    b_sum += sum * exp(((double) wmax - (double) b_ref) * (double) inv_t);
                }
            }
            if (sel && since >= 8 && t_scale > 0.0f) {
                /* after a few new candidates of its own the warp looks whether the threshold can go up: the lowest
                 * bin edge above which at least kq candidates lie, one bin lower to be safe against rounding */
                since  = 0;
                int go = 0;
                if (lane == 0) {
                    go = atomicCAS(&sh->tau_lock, 0, 1) == 0 ? 1 : 0;
                }
                go = __shfl_sync(0xffffffffu, go, 0);
                if (go) {
                    const int b = top_bin(sh->thist, lane, kq);
                    if (lane == 0) {
                        if (b >= 2) {
                            const float t_new = t_lo + (float) (b - 1) / t_scale;
                            if (t_new > t_lo) {
                                atomicMax(&sh->tau_key, order_key(t_new));
                            }
                        }
                        __threadfence_block();
                        sh->tau_lock = 0;
                    }
                }
            }
            if ((kKinds & K_SEL) != 0 && smode == M_TOPK && wcnt > kSqueezeAt && wcnt <= kGroupCapWarp) {
                /* The threshold has gone up since most of the warp's groups were taken: those whose maximum has
                 * fallen below it cannot hold one of the row's kq largest any more and leave the list (top-k rows
                 * only: a top-p row's candidates were left out of its sums and must all arrive). Without this a
                 * wide k fills a warp's list before the row is through. */
                const unsigned pk    = *reinterpret_cast<volatile unsigned *>(&sh->tau_key);
                const float    tau_c = pk == 0u ? tau_reg : fmaxf(tau_reg, key_to_float(pk));
                if (tau_c > sh->wsq[warp]) {
                    int kept = 0;
                    for (int base = 0; base < wcnt; base += 32) {
                        const int j    = base + lane;
                        float4    v    = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        int       bb   = 0;
                        bool      keep = false;
                        if (j < wcnt) {
                            v    = seg_v[j];
                            bb   = seg_b[j];
                            keep = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)) >= tau_c;
                        }
                        const unsigned m = __ballot_sync(0xffffffffu, keep); /* every lane has read its entry before any is overwritten */
                        if (keep) {
                            const int pos = kept + __popc(m & lt);
                            seg_v[pos]    = v;
                            seg_b[pos]    = bb;
                        }
                        kept += __popc(m);
                        __syncwarp();
                    }
                    wcnt = kept;
                    if (lane == 0) {
                        sh->wcur[warp] = kept;
                        sh->wsq[warp] = tau_c;
                    }
                    __syncwarp();
                }
            }
            CYC(2);
        }

        PROF(2);
        /* ---- the part is through: one record and the candidate groups go to global scratch ---- */
        wst = __reduce_or_sync(0xffffffffu, (unsigned) wst);
        if (lane == 0) {
            sh->best[warp]   = ((unsigned long long) run_key << 32) | (unsigned long long) (0xffffffffu - (unsigned) run_arg);
            sh->wn[warp]     = min(wcnt, kGroupCapWarp);
            sh->wn_all[warp] = wcnt;
            sh->wb_ref[warp] = b_ref;
            sh->wb_sum[warp] = b_sum;
            if (wst != 0) {
                atomicOr(&sh->st, wst);
            }
        }
        __syncthreads();
        int held = 0;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            held += sh->wn[w];
        }
        if ((p.flags & F_INLINE_TOPK) != 0u && mode != M_ARGMAX) {
            /* whole rows, top-k: finished here, nothing goes to global scratch (every row of such a launch is one
             * part); a row of another kind is reported as the small finishing kernel would */
            if (mode == M_TOPK) {
                int n_all = 0;
#pragma unroll
                for (int w = 0; w < kWarps; w++) {
                    n_all += sh->wn_all[w];
                }
                const unsigned pkey = sh->tau_key;
                inline_finish_topk(p, sh, grp_v, grp_b, row, held, held == n_all, pkey == 0u ? tau_reg : fmaxf(tau_reg, key_to_float(pkey)), kq, inv_t, sh->st);
            } else {
                if (tid == 0) {
                    p.tokens[row] = -1;
                    p.status[row] = sh->st | ST_INTERNAL;
                }
                __syncthreads();
            }
            CYC(6);
            continue;
        }
        if (tid == 0) {
            unsigned long long bw    = 0ull;
            int                n_all = 0;
            float              bref  = -CUDART_INF_F;
#pragma unroll
            for (int w = 0; w < kWarps; w++) {
                bw = max(bw, sh->best[w]);
                n_all += sh->wn_all[w];
                bref = fmaxf(bref, sh->wb_ref[w]);
            }
            double bsum = 0.0;
            if (mode == M_TOPP && sel) {
#pragma unroll
                for (int w = 0; w < kWarps; w++) {
                    const float wr = sh->wb_ref[w];
                    if (wr != -CUDART_INF_F) {
                        bsum += sh->wb_sum[w] * exp(((double) wr - (double) bref) * (double) inv_t);
                    }
                }
            }
            const unsigned pkey = sh->tau_key;
            int4           h, h2;
            h.x  = __float_as_int((unsigned) (bw >> 32) == 0u ? -CUDART_INF_F : key_to_float((unsigned) (bw >> 32)));
            h.y  = (int) (0xffffffffu - (unsigned) (bw & 0xffffffffull));
            h.z  = held == n_all ? n_all : kPartGroups + 1; /* a warp ran out of room for its groups */
            h.w  = sh->st;
            h2.x = __float_as_int(pkey == 0u ? tau_reg : fmaxf(tau_reg, key_to_float(pkey)));
            h2.y = __float_as_int(bref);
            h2.z = __double2loint(bsum);
            h2.w = __double2hiint(bsum);
            int4 *rec = reinterpret_cast<int4 *>(p.grp_v + ((size_t) row * (size_t) p.parts_max + (size_t) part_idx) * (size_t) kPartSlots);
            rec[0]    = h; /* the part's record takes the first two slots of its group list */
            rec[1]    = h2;
            if ((p.flags & (F_GREEDY_ONLY | F_INLINE_TOPK)) != 0u) { /* in a launch that finishes its top-k rows here, the greedy ones are finished here as well */
                /* The caller said that every row is greedy: no finishing kernel follows. A row that went through
                 * this thread block as a whole is known here. A row cut into parts is finished by whichever of its
                 * parts arrives last: every part publishes its record, then counts itself in; the one that finds
                 * all the others counted reads their records and puts the counter back to zero for the next launch.
                 * Nobody waits for anybody. A row that is not greedy after all is reported. */
                int  best_arg = h.y, stq = h.w;
                bool mine     = n_parts == 1;
                if (!mine) {
                    __threadfence();
                    if (atomicAdd(&p.arrive[row], 1) == n_parts - 1) {
                        __threadfence();
                        p.arrive[row] = 0;
                        float m       = -CUDART_INF_F;
                        best_arg      = 0x7fffffff;
                        for (int q = 0; q < n_parts; q++) {
                            const int4 o = __ldcg(reinterpret_cast<const int4 *>(p.grp_v + ((size_t) row * (size_t) p.parts_max + (size_t) q) * (size_t) kPartSlots));
                            stq |= o.w;
                            if (pair_before(__int_as_float(o.x), o.y, m, best_arg)) {
                                m        = __int_as_float(o.x);
                                best_arg = o.y;
                            }
                        }
                        mine = true;
                    }
                }
                if (mine) {
                    if (mode == M_ARGMAX) {
                        p.tokens[row] = best_arg + p.vocab_offset;
                    } else { /* only with F_GREEDY_ONLY: the other flag's rows of other kinds never come here */
                        p.tokens[row] = -1;
                        stq |= ST_INTERNAL;
                    }
                    if (p.kept_cap > 0) {
                        p.kept_n[row] = 0;
                    }
                    p.status[row] = stq;
                    if (p.rng_out != nullptr && sh->cur_last) {
                        p.rng_out[sh->cur_seq] = sh->cur_rng; /* greedy rows draw nothing (sampler.c:106-112) */
                    }
                }
            }
        }
        const size_t at = ((size_t) row * (size_t) p.parts_max + (size_t) part_idx) * (size_t) kPartSlots + 2;
        for (int f = tid; f < held; f += kThreads) {
            const int slot  = own_slot(sh, f);
            p.grp_v[at + f] = grp_v[slot];
            p.grp_b[at + f] = grp_b[slot];
        }
        __syncthreads(); /* the lists are free for the next part */
        CYC(6);
    }
    if (ring_dead >= 0 && aligned) {
        /* copies that were asked for before the warp gave up (the item it gave up on and the one behind it) may
         * still be on their way into this thread block's shared memory: one more bounded wait for each before the
         * thread block may end */
        for (int jj = ring_dead; jj < min(ring_dead + kStages, my_count); jj++) {
            (void) mbar_wait_bounded(&sh->full[warp][jj % kStages], (unsigned) (jj / kStages) & 1u);
        }
    }
    CYC_DONE();
    PROF(4);
}

/* ----------------------------------------------------------- finishing kernel -- */

/*
 * Run behind the stream kernel, one thread block per row at a time (rows blockIdx.x, blockIdx.x + gridDim.x, ...):
 * it merges the records that the row's parts left and finishes the row. finish_rows_kernel<false> carries the
 * code for every kind of row: greedy, top-k, temperature (segment walks), top-p (nucleus sums), and the
 * multi-pass path over a private copy of the row (the copies come from a small pool that the thread blocks claim
 * slots of). finish_rows_kernel<true> carries greedy and top-k (k <= 256) alone: a tenth of the code, 7 - 8 us
 * less per launch; it is launched instead when the caller vouched for such rows, and reports any other row as
 * ROW_INTERNAL. Both write the row's status and, behind a sequence's last row, its generator.
 */
template <bool kFast>
__global__ void __launch_bounds__(kThreads, 2) finish_rows_kernel(const __grid_constant__ SampleParams p) {
    extern __shared__ __align__(128) unsigned char fsmem[];
    FinishShared  *sh   = reinterpret_cast<FinishShared *>(fsmem);
    unsigned char *cmem = reinterpret_cast<unsigned char *>(sh + 1);

    Grp g;
    g.tid  = (int) threadIdx.x;
    g.lane = g.tid & 31;
    g.warp = g.tid >> 5;
    g.n    = kThreads;
    g.nw   = kWarps;
    g.bar  = 0;
    /* The first row's parameters are inputs of the launch, written before the stream kernel began: they may be
     * read while that kernel's last thread blocks are still at work. Everything it wrote waits for the line below. */
    RawCfg rc0{};
    if ((int) blockIdx.x < p.n_rows) {
        rc0 = raw_config(p, (int) blockIdx.x, true);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory"); /* the records of the kernel before this one are complete and visible */
    asm volatile("griddepcontrol.launch_dependents;");
    PROF(kFast ? 5 : 7);
    for (int row = (int) blockIdx.x; row < p.n_rows; row += (int) gridDim.x) {
        const RawCfg rc = row == (int) blockIdx.x ? rc0 : raw_config(p, row, true);
        RowCfg       r  = row_config(p, row, rc, true);
        PROF(8);
        int          st = finish_row<kFast>(g, p, sh, r, cmem);
        PROF(13);
        if (st & ST_DEFERRED) {
            if constexpr (kFast) {
                /* This kernel does not carry the code for the row. A top-k row whose candidates did not fit (many
                 * equal values at the top) is the caller's to launch again without the hint; any other kind of
                 * row the caller said would not come. */
                st = (st & ~ST_DEFERRED) | (r.mode == M_TOPK ? ST_RETRY : ST_INTERNAL);
                if (g.tid == 0) {
                    p.tokens[row] = -1;
                }
            } else {
                /* the multi-pass path: all threads of this thread block, over a private copy of the row */
                __syncthreads();
                const float bm = sh->gs.blk_max;
                const int   ba = sh->gs.blk_arg;
                if (g.tid == 0) {
                    /* claim a row copy: bounded search, the holders always make progress */
                    int got = -1;
                    for (long long t = 0; t < (1ll << 24) && got < 0; t++) {
                        const int c = (int) ((blockIdx.x + t) % (unsigned) p.pool_slots);
                        if (atomicCAS(&p.pool[c], 0, 1) == 0) {
                            got = c;
                        }
                    }
                    __threadfence();
                    sh->slot = got;
                }
                __syncthreads();
                const int slot = sh->slot;
                if (slot < 0) {
                    st = (st & ~ST_DEFERRED) | ST_INTERNAL;
                } else {
                    st = (st & ~ST_DEFERRED) | multipass_row(g, p, &sh->gs, r, bm, ba, cmem, kFinBytes, slot, &sh->st_v[0][0]); /* the staging of the parts' first slots is free by now: 3 KB of it keep a histogram */
                    __syncthreads();
                    if (g.tid == 0) {
                        __threadfence();
                        atomicExch(&p.pool[slot], 0);
                    }
                }
            }
        }
        if (g.tid == 0) {
            row_epilogue(p, r, row, st, rc.rng);
        }
        __syncthreads();
    }
    PROF(kFast ? 6 : 7);
}

/* ------------------------------------------------ long histories, prepared -- */

constexpr int kRowIdThreads = 256;

/* One CTA per row whose history (plus fed tokens) is longer than the stream kernel counts
 * by itself: the row's distinct ids with their counts, grouped by the slice they fall into.
 * pre_off[row][c] .. pre_off[row][c + 1] is slice c's run in pre_list[row]; an entry is
 * (position in the slice) | (count << kLiBits). Shorter rows are left to the stream kernel. */
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
    if (H + E <= kRowIds) {
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

#ifdef GB_PROFILE
extern "C" int geist_b200_debug_mp(long long *out) { return (int) cudaMemcpyFromSymbol(out, g_mp, sizeof(long long) * 1024 * 24); }
extern "C" int geist_b200_debug_prof(long long *out) { return (int) cudaMemcpyFromSymbol(out, g_prof, sizeof(long long) * 1024 * 16); }
#ifdef GB_PROFILE_CYC
extern "C" int geist_b200_debug_cyc(long long *out) { return (int) cudaMemcpyFromSymbol(out, g_cyc, sizeof(long long) * 1024 * kWarps * 8); }
#endif
#endif

size_t sample_stream_smem(int n_slices, int long_ids) {
    size_t b = (size_t) kWarps * kStages * kWarpStageBytes + sizeof(StreamShared) + (size_t) kGroupBytes;
    if (long_ids) {
        b += (((size_t) n_slices + 1) * 4 + 15) & ~(size_t) 15;
        b += (size_t) kListSmem * 4;
    }
    return b;
}

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
        /* two thread blocks per SM need nearly all of its shared memory: ask for the largest carve-out */
#define GB_STREAM_ALL(X)                                                                                                                     \
    X(K_SEL | K_SUMS | K_PEN) X(K_SEL | K_PEN) X(K_PEN) X(K_SEL | K_SUMS | K_PEN | K_SHORT) X(K_SEL | K_PEN | K_SHORT) X(K_PEN | K_SHORT)      \
    X(K_SEL | K_SUMS | K_SHORT) X(K_SEL | K_SHORT) X(K_SHORT)                                                                                  \
    X(K_PLAIN | K_SEL | K_SUMS | K_PEN) X(K_PLAIN | K_SEL | K_PEN) X(K_PLAIN | K_PEN)                                                         \
    X(K_PLAIN | K_SEL | K_SUMS | K_PEN | K_SHORT) X(K_PLAIN | K_SEL | K_PEN | K_SHORT) X(K_PLAIN | K_PEN | K_SHORT)                            \
    X(K_PLAIN | K_SEL | K_SUMS | K_SHORT) X(K_PLAIN | K_SEL | K_SHORT) X(K_PLAIN | K_SHORT)
#define GB_STREAM_PTR(K) reinterpret_cast<const void *>(sample_stream_kernel<(K)>),
        const void *kernels[] = {GB_STREAM_ALL(GB_STREAM_PTR)};
#undef GB_STREAM_PTR
        for (const void *k : kernels) {
            e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
            if (e == cudaSuccess) {
                e = cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, (int) cudaSharedmemCarveoutMaxShared);
            }
            if (e != cudaSuccess) {
                return e;
            }
        }
        configured_smem[dev] = (int) smem_bytes;
    }
    return cudaSuccess;
}

/* Thread blocks of the stream kernel that one SM of the current device holds at this much shared memory. */
cudaError_t sample_stream_ctas_per_sm(size_t smem_bytes, int *out) {
    cudaError_t e = ensure_attributes(smem_bytes);
    if (e != cudaSuccess) {
        return e;
    }
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(out, sample_stream_kernel<K_SEL | K_SUMS | K_PEN>, kThreads, smem_bytes);
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

size_t finish_rows_smem() { return sizeof(FinishShared) + (size_t) kFinBytes; }

static cudaError_t ensure_finish_attributes() {
    static int  configured[64] = {0};
    int         dev            = 0;
    cudaError_t e              = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    if (dev < 0 || dev >= 64) {
        return cudaErrorInvalidDevice;
    }
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(finish_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) finish_rows_smem());
        if (e == cudaSuccess) {
            e = cudaFuncSetAttribute(finish_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) finish_rows_smem());
        }
        if (e != cudaSuccess) {
            return e;
        }
        configured[dev] = 1;
    }
    return cudaSuccess;
}

/* Thread blocks of the finishing kernel that the current device holds at once. */
cudaError_t finish_rows_max_ctas(int sms, int *out) {
    cudaError_t e = ensure_finish_attributes();
    if (e != cudaSuccess) {
        return e;
    }
    int per_sm = 0;
    e          = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, finish_rows_kernel<false>, kThreads, finish_rows_smem());
    *out       = per_sm * sms;
    return e;
}

cudaError_t launch_sample_stream(const SampleParams &p, int grid, size_t smem_bytes, int finish_grid, cudaStream_t stream) {
    cudaError_t e = ensure_attributes(smem_bytes);
    if (e == cudaSuccess) {
        e = ensure_finish_attributes();
    }
    if (e != cudaSuccess) {
        return e;
    }
    if (p.id_slots > 0) { /* rows may bring more ids than the stream kernel counts by itself: prepare their lists first */
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
    }
    /* Programmatic dependent launch, both kernels: the thread blocks are placed while the kernel before them
     * in the stream drains, and wait (griddepcontrol.wait) until that kernel is complete and visible before they
     * touch global memory. No thread block ever waits for another one of its grid, so neither grid needs
     * co-residency. */
    cudaLaunchConfig_t  cfg{};
    cudaLaunchAttribute attr[1];
    cfg.gridDim          = dim3((unsigned) grid);
    cfg.blockDim         = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream           = stream;
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = 1;
    /* the instantiation that carries no more than the kinds of rows the caller vouched for, and the penalties' code
     * only where the launch brings ids */
    const bool pen   = p.hist != nullptr || p.extra != nullptr;
    const int  kinds = (p.flags & F_SELECT_ONLY) != 0u ? (K_SEL | K_SUMS) : (p.flags & F_GREEDY_ONLY) != 0u ? 0 : (p.flags & F_FAST_ONLY) != 0u ? K_SEL : (K_SEL | K_SUMS);
    const bool plain     = p.aligned != 0 && p.softcap == nullptr && p.mask == nullptr && p.out_logits == nullptr;
    const bool short_ids = !pen || p.id_slots == 0; /* no row brings more ids than a thread block counts by itself */
#define GB_STREAM_CASE(K)                                                  \
    case (K):                                                              \
        e = cudaLaunchKernelEx(&cfg, sample_stream_kernel<(K)>, p);        \
        break;
    switch (kinds | (pen ? K_PEN : 0) | (plain ? K_PLAIN : 0) | (short_ids ? K_SHORT : 0)) {
        GB_STREAM_ALL(GB_STREAM_CASE)
    default:
        e = cudaErrorInvalidValue;
        break;
    }
#undef GB_STREAM_CASE
    if (e != cudaSuccess) {
        return e;
    }
    cfg.gridDim          = dim3((unsigned) finish_grid);
    cfg.dynamicSmemBytes = finish_rows_smem();
    if ((p.flags & (F_GREEDY_ONLY | F_INLINE_TOPK)) != 0u) {
        return cudaSuccess; /* the stream kernel writes the tokens itself */
    }
    /* one finishing kernel per launch: the small one when the caller vouched for greedy / top-k rows, else the
     * general one (it finishes every kind of row; a third kernel in the chain of dependent launches cost 7 - 8 us
     * even when it had no row to take, as much as the general kernel costs more than the small one) */
    if ((p.flags & F_FAST_ONLY) != 0u) {
        return cudaLaunchKernelEx(&cfg, finish_rows_kernel<true>, p);
    }
    return cudaLaunchKernelEx(&cfg, finish_rows_kernel<false>, p);
}

} /* namespace gb */

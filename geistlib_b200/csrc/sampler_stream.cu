/*
 * sampler_stream.cu — the logits -> token kernel (sm_100a).
 *
 * A persistent grid (one CTA per SM) streams every logits row through the chip
 * exactly once. A row is cut into slices of at most 16384 floats; the work
 * item is (row, slice). Each CTA keeps a ring of shared-memory stages that a
 * single thread fills with bulk asynchronous copies (mbarrier-signalled, no
 * cluster multicast) a few items ahead, so HBM stays busy while the CTA
 * computes. A slice is lifted from its stage into registers (4 float4 per
 * thread) and the stage is handed back to the copy engine at once; the passes
 * over the slice (maximum, select threshold, collect / exp-sum) then run on
 * registers.
 *
 * What a slice finds goes to a small record in global scratch. The CTA that
 * completes a row (a per-row counter tells it) is the row's finisher: it
 * merges the slice records, orders the few surviving candidates, evaluates
 * their probabilities exactly and makes the draw. Nothing ever waits on
 * another CTA.
 *
 * Rows whose kept set is too large for this (top-k beyond the candidate room,
 * wide top-p nuclei) are served by the finisher alone with a multi-pass
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

struct PenEntry {
    int   li;
    float orig;
};

struct __align__(16) StreamShared {
    unsigned long long full[kMaxStages];
    float              gmax[kGroupCap];
    float              wred_f[kWarps];
    int                wred_a[kWarps];
    double             wred_d[kWarps];
    long long          wred_l[kWarps];
    int                bins[kHistBins];
    double             S;
    float              tau;
    float              blk_max;
    int                blk_arg;
    int                n_cand;
    int                n_dlist;
    int                is_last;
    int                n_sel;
    int                n_border;
    int                b_star;
    int                n_hi;
    int                flag;
    int                pick;
};

enum Mode { M_ARGMAX, M_TOPK, M_TOPP, M_TEMP };

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

__device__ __forceinline__ RowCfg row_config(const SampleParams &p, int row) {
    RowCfg r;
    r.row   = row;
    r.seq0  = row / p.rows_per_seq;
    r.rr    = row - r.seq0 * p.rows_per_seq;
    r.seq   = p.slot ? p.slot[r.seq0] : r.seq0;
    r.T     = p.temperature[r.seq];
    r.top_k = p.top_k[r.seq];
    r.top_p = p.top_p[r.seq];
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
    r.kq = r.mode == M_TOPK ? r.k : (r.mode == M_TOPP ? min(kNucleusProbe, p.V) : 0);
    r.inv_t         = r.T > 0.0f ? __fdiv_rn(1.0f, r.T) : 1.0f;
    r.draws_per_row = (r.T > 0.0f && !r.select_only) ? 1 : 0;
    r.rng           = p.rng_in ? p.rng_in[r.seq] : 1ull;
    for (int i = 0; i < r.rr * r.draws_per_row; i++) {
        (void) xorshift_next(r.rng);
    }
    r.pen_on = p.hist != nullptr || p.extra != nullptr;
    r.H      = p.hist ? (int) min((long long) max(p.hist_len[r.seq], 0), p.hist_stride) : 0;
    r.E      = p.extra ? r.rr : 0; /* proposals fed before this row: extra[1..rr] */
    r.rep    = p.rep ? p.rep[r.seq] : 1.0f;
    if (!(r.rep > 0.0f)) {
        r.rep = 1.0f;
    }
    r.freq = p.freq ? p.freq[r.seq] : 0.0f;
    r.pres = p.pres ? p.pres[r.seq] : 0.0f;
    r.hrow = p.hist ? p.hist + (size_t) r.seq * (size_t) p.hist_stride : nullptr;
    r.erow = p.extra ? p.extra + (size_t) r.seq0 * (size_t) p.extra_stride : nullptr; /* per call, not per slot */
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
 * `dlist` has room for `cap` distinct ids. All threads of the CTA call this.
 * Returns status bits.
 */
template <class Entry>
__device__ int apply_penalties(float *buf, int s0, int n, const RowCfg &r, int V, int vocab_offset, unsigned *bitmap, Entry *dlist, int cap, int *n_dlist) {
    const int tid = threadIdx.x;
    int       st  = 0;
    /* (a) the first thread to mark an id owns it and saves the original value */
    for (int j = tid; j < r.H + r.E; j += kThreads) {
        const int id = hist_id(r, j, vocab_offset);
        const int li = id - s0;
        if (id >= 0 && id < V && li >= 0 && li < n) {
            const unsigned bit = 1u << (li & 31);
            const unsigned old = atomicOr(&bitmap[li >> 5], bit);
            if (!(old & bit)) {
                const int pos = atomicAdd(n_dlist, 1);
                if (pos < cap) {
                    dlist[pos] = Entry{li, buf[li]};
                }
            }
        }
    }
    __syncthreads();
    int nd = *n_dlist;
    if (nd > cap) { /* cannot happen when the launcher sized the room; keep the run consistent anyway */
        st |= ST_HIST_OVERFLOW;
        nd = 0;
    }
    /* (b) the slot becomes an integer counter */
    for (int i = tid; i < nd; i += kThreads) {
        reinterpret_cast<int *>(buf)[dlist[i].li] = 0;
    }
    __syncthreads();
    if (nd > 0) {
        for (int j = tid; j < r.H + r.E; j += kThreads) {
            const int id = hist_id(r, j, vocab_offset);
            const int li = id - s0;
            if (id >= 0 && id < V && li >= 0 && li < n) {
                atomicAdd(reinterpret_cast<int *>(buf) + li, 1);
            }
        }
    }
    __syncthreads();
    /* (c) one thread per distinct id writes the penalised value */
    for (int i = tid; i < nd; i += kThreads) {
        const int li = dlist[i].li;
        buf[li]      = penalise(dlist[i].orig, reinterpret_cast<int *>(buf)[li], r.rep, r.freq, r.pres);
    }
    __syncthreads();
    return st;
}

/* ------------------------------------------------------- block reductions -- */

__device__ __forceinline__ void block_argmax(StreamShared *sh, float &v, int &a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int   oa = __shfl_xor_sync(0xffffffffu, a, o);
        if (pair_before(ov, oa, v, a)) {
            v = ov;
            a = oa;
        }
    }
    if (lane == 0) {
        sh->wred_f[warp] = v;
        sh->wred_a[warp] = a;
    }
    __syncthreads();
    if (warp == 0) {
        v = sh->wred_f[lane];
        a = sh->wred_a[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int   oa = __shfl_xor_sync(0xffffffffu, a, o);
            if (pair_before(ov, oa, v, a)) {
                v = ov;
                a = oa;
            }
        }
        if (lane == 0) {
            sh->blk_max = v;
            sh->blk_arg = a;
        }
    }
    __syncthreads();
    v = sh->blk_max;
    a = sh->blk_arg;
}

/* Every thread gets the same total (fixed order of additions). */
__device__ __forceinline__ double block_sum_d(StreamShared *sh, double v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum_d(v);
    __syncthreads(); /* the previous result has been read */
    if (lane == 0) {
        sh->wred_d[warp] = v;
    }
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < kWarps; w++) {
        t += sh->wred_d[w];
    }
    return t;
}

__device__ __forceinline__ long long block_sum_ll(StreamShared *sh, long long v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum_ll(v);
    __syncthreads();
    if (lane == 0) {
        sh->wred_l[warp] = v;
    }
    __syncthreads();
    long long t = 0;
#pragma unroll
    for (int w = 0; w < kWarps; w++) {
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
 * `total` pairs. Called by the whole CTA.
 */
__device__ void select_sorted(StreamShared *sh, const Pair *cand, int total, int kq, Pair *tmp, Pair *sorted) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned  lo = 0xffffffffu, hi = 0u;
    for (int i = tid; i < total; i += kThreads) {
        const unsigned key = order_key(cand[i].v);
        lo                 = min(lo, key);
        hi                 = max(hi, key);
    }
    lo = __reduce_min_sync(0xffffffffu, lo);
    hi = __reduce_max_sync(0xffffffffu, hi);
    __syncthreads();
    if (lane == 0) {
        sh->wred_a[warp]                               = (int) lo;
        reinterpret_cast<unsigned *>(sh->wred_f)[warp] = hi;
    }
    for (int i = tid; i < kHistBins; i += kThreads) {
        sh->bins[i] = 0;
    }
    if (tid == 0) {
        sh->n_sel    = 0;
        sh->n_border = 0;
        sh->b_star   = 0;
        sh->n_hi     = 0;
    }
    __syncthreads();
    lo = 0xffffffffu;
    hi = 0u;
    for (int w = 0; w < kWarps; w++) {
        lo = min(lo, (unsigned) sh->wred_a[w]);
        hi = max(hi, reinterpret_cast<unsigned *>(sh->wred_f)[w]);
    }
    const unsigned range = hi >= lo ? hi - lo : 0u;
    const int      shift = max(0, (32 - __clz(range)) - 8); /* (range >> shift) < 256 */
    for (int i = tid; i < total; i += kThreads) {
        atomicAdd(&sh->bins[(order_key(cand[i].v) - lo) >> shift], 1);
    }
    __syncthreads();
    if (warp == 0) {
        /* b* = largest bin with count(bins >= b*) >= kq; lane l owns bins [8l, 8l+8) */
        int mine = 0;
#pragma unroll
        for (int q = 0; q < 8; q++) {
            mine += sh->bins[8 * lane + q];
        }
        int above = 0; /* entries owned by higher lanes */
        for (int l = 31; l >= 1; l--) {
            const int c = __shfl_sync(0xffffffffu, mine, l);
            if (lane < l) {
                above += c;
            }
        }
        if (above < kq && above + mine >= kq) {
            int acc = above;
            for (int q = 7; q >= 0; q--) {
                const int c = sh->bins[8 * lane + q];
                if (acc + c >= kq) {
                    sh->b_star = 8 * lane + q;
                    sh->n_hi   = acc;
                    break;
                }
                acc += c;
            }
        }
    }
    __syncthreads();
    const int b_star = sh->b_star, n_hi = sh->n_hi;
    /* entries above the bin fill tmp from the front, the bin's entries from the back */
    for (int i = tid; i < total; i += kThreads) {
        const int bin = (int) ((order_key(cand[i].v) - lo) >> shift);
        if (bin > b_star) {
            tmp[atomicAdd(&sh->n_sel, 1)] = cand[i];
        } else if (bin == b_star) {
            tmp[total - 1 - atomicAdd(&sh->n_border, 1)] = cand[i];
        }
    }
    __syncthreads();
    const int nb   = sh->n_border;
    const int need = kq - n_hi;
    for (int i = tid; i < nb; i += kThreads) {
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
    for (int i = tid; i < n_hi; i += kThreads) {
        const Pair me   = tmp[i];
        int        rank = 0;
        for (int j = 0; j < n_hi; j++) {
            rank += pair_before(tmp[j].v, tmp[j].idx, me.v, me.idx) ? 1 : 0;
        }
        sorted[rank] = me;
    }
    __syncthreads();
}

/* ------------------------------------------------- multi-pass path (finisher) -- */

template <class F>
__device__ __forceinline__ void row_sweep(const float *row, int V, F &&f) {
    const int     V4 = V >> 2;
    const float4 *p4 = reinterpret_cast<const float4 *>(row);
    for (int j = threadIdx.x; j < V4; j += kThreads) {
        const float4 x = p4[j];
        f(x.x, 4 * j);
        f(x.y, 4 * j + 1);
        f(x.z, 4 * j + 2);
        f(x.w, 4 * j + 3);
    }
    for (int i = (V4 << 2) + threadIdx.x; i < V; i += kThreads) {
        f(row[i], i);
    }
}

template <class F>
__device__ __forceinline__ void row_rewrite(float *row, int V, F &&f) {
    for (int i = threadIdx.x; i < V; i += kThreads) {
        row[i] = f(row[i], i);
    }
}

/* Largest composite word t such that at least `want` entries are >= t. */
__device__ unsigned long long bisect_rank(StreamShared *sh, const float *row, int V, int idx_bits, long long want) {
    unsigned long long prefix = 0;
    for (int bit = 31 + idx_bits; bit >= 0; bit--) {
        const unsigned long long t   = prefix | (1ull << bit);
        long long                cnt = 0;
        row_sweep(row, V, [&](float x, int i) { cnt += composite(order_key(x), i, idx_bits) >= t ? 1 : 0; });
        if (block_sum_ll(sh, cnt) >= want) {
            prefix = t;
        }
    }
    return prefix;
}

/* Largest composite word t with mass{word >= t} >= target (inclusive) or > target. */
template <class KeyF, class MassF>
__device__ unsigned long long bisect_mass(StreamShared *sh, const float *row, int V, int idx_bits, double target, bool inclusive, KeyF &&key, MassF &&mass) {
    unsigned long long prefix = 0;
    for (int bit = 31 + idx_bits; bit >= 0; bit--) {
        const unsigned long long t = prefix | (1ull << bit);
        double                   m = 0.0;
        row_sweep(row, V, [&](float x, int i) {
            if (composite(key(x), i, idx_bits) >= t) {
                m += mass(x, i);
            }
        });
        const double tot = block_sum_d(sh, m);
        if (inclusive ? (tot >= target) : (tot > target)) {
            prefix = t;
        }
    }
    return prefix;
}

/* The finisher alone serves a row whose kept set does not fit the fast path. */
__device__ int multipass_row(const SampleParams &p, StreamShared *sh, RowCfg &r, float row_max, int row_arg) {
    const int   tid      = threadIdx.x;
    const int   V        = p.V;
    const int   idx_bits = 32 - __clz(max(V - 1, 1));
    int         st       = ST_SLOW_PATH;
    float      *g        = p.gen_rows + (size_t) blockIdx.x * (size_t) p.gen_stride;
    const float *src     = p.logits + (size_t) r.row * (size_t) p.row_stride;
    int        *kept_i   = p.kept_cap > 0 ? p.kept_idx + (size_t) r.row * (size_t) p.kept_cap : nullptr;
    float      *kept_v   = p.kept_cap > 0 ? p.kept_val + (size_t) r.row * (size_t) p.kept_cap : nullptr;
    /* private copy of the row, penalties applied once */
    for (int i = tid; i < V; i += kThreads) {
        g[i] = src[i];
    }
    if (r.pen_on) {
        unsigned *bm = p.gen_bitmap + (size_t) blockIdx.x * (size_t) p.gen_bitmap_words;
        for (int i = tid; i < p.gen_bitmap_words; i += kThreads) {
            bm[i] = 0u;
        }
        if (tid == 0) {
            sh->n_dlist = 0;
        }
        __syncthreads();
        st |= apply_penalties(g, 0, V, r, V, p.vocab_offset, bm, reinterpret_cast<PenEntry *>(p.gen_dlist + (size_t) blockIdx.x * (size_t) p.gen_hist_cap), p.gen_hist_cap,
                              &sh->n_dlist);
    } else {
        __syncthreads();
    }
    if (r.mode == M_TOPK) {
        const unsigned long long t_set  = bisect_rank(sh, g, V, idx_bits, (long long) r.k);
        auto                     in_set = [&](float x, int i) { return composite(order_key(x), i, idx_bits) >= t_set; };
        if (r.select_only) {
            if (tid == 0) {
                sh->n_sel = 0;
            }
            __syncthreads();
            row_sweep(g, V, [&](float x, int i) {
                if (in_set(x, i)) {
                    const int pos = atomicAdd(&sh->n_sel, 1);
                    if (pos < p.kept_cap) {
                        kept_i[pos] = i + p.vocab_offset;
                        kept_v[pos] = x;
                    }
                }
            });
            if (tid == 0) {
                p.kept_n[r.row] = r.k;
                p.tokens[r.row] = row_arg + p.vocab_offset;
            }
        } else {
            auto   qof = [&](float x) { return (double) exp_exact(scaled_arg(x, row_max, r.inv_t)); };
            double m   = 0.0;
            row_sweep(g, V, [&](float x, int i) {
                if (in_set(x, i)) {
                    m += qof(x);
                }
            });
            const double S = block_sum_d(sh, m);
            const double u = (double) unit_from(xorshift_next(r.rng)) * S;
            /* the pick is the earliest walk position whose running sum exceeds u: the largest
             * word t with mass{word >= t} > u */
            unsigned long long t_pick = bisect_mass(
                    sh, g, V, idx_bits, u, false, [&](float x) { return order_key(x); }, [&](float x, int i) { return in_set(x, i) ? qof(x) : 0.0; });
            if (t_pick < t_set) {
                t_pick = t_set;
            }
            row_sweep(g, V, [&](float x, int i) {
                if (composite(order_key(x), i, idx_bits) == t_pick) {
                    p.tokens[r.row] = i + p.vocab_offset;
                }
            });
            if (tid == 0 && p.kept_cap > 0) {
                p.kept_n[r.row] = r.k;
            }
            if (p.kept_cap > 0) {
                st |= ST_KEPT_PARTIAL;
            }
        }
    } else {
        /* top-p with any nucleus size: the copy becomes e_i, then p_i (sampler.c:245-255) */
        double acc = 0.0;
        row_rewrite(g, V, [&](float x, int) {
            const float e = expf(scaled_arg(x, row_max, r.inv_t));
            acc += (double) e;
            return e;
        });
        const double S = block_sum_d(sh, acc);
        row_rewrite(g, V, [&](float e, int) { return __double2float_rn((double) e / S); });
        __syncthreads();
        auto keyf  = [](float pv) { return __float_as_uint(pv); }; /* p >= 0: the bits are ordered */
        auto massf = [](float pv, int) { return (double) pv; };
        /* cutoff: first walk position whose running sum reaches top_p, inclusive */
        const unsigned long long t_cut = bisect_mass(sh, g, V, idx_bits, (double) r.top_p, true, keyf, massf);
        double                   nm    = 0.0;
        long long                ncnt  = 0;
        row_sweep(g, V, [&](float pv, int i) {
            if (composite(keyf(pv), i, idx_bits) >= t_cut) {
                nm += (double) pv;
                ncnt++;
            }
        });
        const double       N      = block_sum_d(sh, nm);
        const long long    cut    = block_sum_ll(sh, ncnt);
        const double       u      = (double) unit_from(xorshift_next(r.rng)) * N;
        unsigned long long t_pick = bisect_mass(sh, g, V, idx_bits, u, false, keyf, massf);
        if (t_pick < t_cut) {
            t_pick = t_cut; /* default: the last nucleus entry (sampler.c:292) */
        }
        row_sweep(g, V, [&](float pv, int i) {
            if (composite(keyf(pv), i, idx_bits) == t_pick) {
                p.tokens[r.row] = i + p.vocab_offset;
            }
        });
        if (tid == 0 && p.kept_cap > 0) {
            p.kept_n[r.row] = (int) cut;
        }
        if (p.kept_cap > 0) {
            st |= ST_KEPT_PARTIAL;
        }
    }
    __syncthreads();
    return st;
}


/* ---------------------------------------------------------------- finisher -- */

struct FinBuffers {
    Pair     *fcand, *ftmp, *fsort;
    float    *fq;
    unsigned *bitmap;
    PenEntry *dlist;
};

/* Runs in the CTA that completed the row. Returns status bits for the row. */
__device__ int finish_row(const SampleParams &p, StreamShared *sh, RowCfg &r, const FinBuffers &fb) {
    const int       tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int       row    = r.row;
    const SliceRec *recs   = p.recs + (size_t) row * (size_t) p.n_slices;
    int            *kept_i = p.kept_cap > 0 ? p.kept_idx + (size_t) row * (size_t) p.kept_cap : nullptr;
    float          *kept_v = p.kept_cap > 0 ? p.kept_val + (size_t) row * (size_t) p.kept_cap : nullptr;
    int             st     = 0;

    /* row maximum, its first id, and the slices' status bits */
    float row_max = -CUDART_INF_F;
    int   row_arg = 0x7fffffff;
    int   rst     = 0;
    for (int cc = tid; cc < p.n_slices; cc += kThreads) {
        const float m = __ldcg(&recs[cc].max);
        const int   a = __ldcg(&recs[cc].arg);
        rst |= __ldcg(&recs[cc].st);
        if (row_arg == 0x7fffffff || pair_before(m, a, row_max, row_arg)) {
            row_max = m;
            row_arg = a;
        }
    }
    rst = __reduce_or_sync(0xffffffffu, rst);
    __syncthreads();
    if (lane == 0) {
        sh->wred_l[warp] = rst;
    }
    block_argmax(sh, row_max, row_arg);
    for (int w = 0; w < kWarps; w++) {
        st |= (int) sh->wred_l[w];
    }

    if (r.mode == M_ARGMAX) {
        if (tid == 0) {
            p.tokens[row] = row_arg + p.vocab_offset;
            if (p.kept_cap > 0) {
                p.kept_n[row] = 0;
            }
        }
        return st;
    }

    if (r.mode == M_TEMP) {
        /* segment sums, rescaled from their slice maximum to the row maximum, in id order */
        const int nseg   = p.n_slices * kWarps;
        auto      seg_at = [&](int t) {
            const int cc = t / kWarps;
            return exp(((double) __ldcg(&recs[cc].max) - (double) row_max) * (double) r.inv_t) * __ldcg(&recs[cc].seg[t % kWarps]);
        };
        double part = 0.0;
        for (int t = tid; t < nseg; t += kThreads) {
            part += seg_at(t);
        }
        const double S     = block_sum_d(sh, part);
        const double u     = (double) unit_from(xorshift_next(r.rng)) * S;
        double       carry = 0.0;
        int          found = -1;
        double       fbase = -CUDART_INF; /* nothing crosses: the walk ends on its last id */
        for (int t0 = 0; t0 < nseg; t0 += kThreads) {
            const int    t    = t0 + tid;
            const double val  = t < nseg ? seg_at(t) : 0.0;
            double       incl = val;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) {
                    incl += up;
                }
            }
            __syncthreads();
            if (lane == 31) {
                sh->wred_d[warp] = incl;
            }
            if (tid == 0) {
                sh->pick = 0x7fffffff;
            }
            __syncthreads();
            double woff = carry;
            for (int w = 0; w < warp; w++) {
                woff += sh->wred_d[w];
            }
            incl += woff;
            if (t < nseg && u < incl) {
                atomicMin(&sh->pick, t);
            }
            __syncthreads();
            const int pk = sh->pick;
            if (pk != 0x7fffffff) {
                if (t == pk) {
                    sh->S = incl - val;
                }
                __syncthreads();
                found = pk;
                fbase = sh->S;
                break;
            }
            for (int w = 0; w < kWarps; w++) {
                carry += sh->wred_d[w];
            }
        }
        if (found < 0) {
            found = nseg - 1;
        }
        /* the crossing segment, re-read from the row (L2), penalised, walked with the row maximum */
        const int    cc     = found / kWarps, w = found % kWarps;
        const int    s0c    = cc * p.slice;
        const int    nc     = max(0, min(p.slice, p.V - s0c));
        const int    nv4c   = (nc + 3) >> 2;
        const int    Lc     = (nv4c + kWarps - 1) / kWarps;
        const int    e0     = min(4 * w * Lc, nc);
        const int    e1     = min(4 * min((w + 1) * Lc, nv4c), nc);
        const int    seg_n  = max(e1 - e0, 0);
        float       *wbuf   = reinterpret_cast<float *>(fb.fcand); /* >= 512 floats */
        const float *src    = p.logits + (size_t) row * (size_t) p.row_stride + s0c + e0;
        __syncthreads();
        for (int i = tid; i < seg_n; i += kThreads) {
            wbuf[i] = src[i];
        }
        if (r.pen_on) {
            for (int i = tid; i < (seg_n + 31) / 32; i += kThreads) {
                fb.bitmap[i] = 0u;
            }
            if (tid == 0) {
                sh->n_dlist = 0;
            }
        }
        __syncthreads();
        if (r.pen_on && seg_n > 0) {
            st |= apply_penalties(wbuf, s0c + e0, seg_n, r, p.V, p.vocab_offset, fb.bitmap, fb.dlist, p.hist_cap, &sh->n_dlist);
        }
        if (warp == 0) {
            int    hit  = -1;
            double base = fbase;
            for (int c0 = 0; c0 < seg_n && hit < 0; c0 += 128) {
                float ev[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int i = c0 + 4 * lane + q;
                    ev[q]       = i < seg_n ? expf(scaled_arg(wbuf[i], row_max, r.inv_t)) : 0.0f;
                }
                const double mine = ((double) ev[0] + (double) ev[1]) + ((double) ev[2] + (double) ev[3]);
                double       incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const double up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) {
                        incl += up;
                    }
                }
                const unsigned ball = __ballot_sync(0xffffffffu, u < base + incl);
                if (ball != 0u) {
                    const int srcl = __ffs(ball) - 1;
                    int       f    = -1;
                    if (lane == srcl) {
                        double a = base + (incl - mine);
                        f        = c0 + 4 * lane + 3;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            a += (double) ev[q];
                            if (u < a) {
                                f = c0 + 4 * lane + q;
                                break;
                            }
                        }
                    }
                    hit = min(__shfl_sync(0xffffffffu, f, srcl), seg_n - 1);
                }
                base += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (hit < 0) {
                hit = max(seg_n - 1, 0); /* regrouped sums can end a hair below the segment's share */
            }
            if (lane == 0) {
                p.tokens[row] = s0c + e0 + hit + p.vocab_offset;
                if (p.kept_cap > 0) {
                    p.kept_n[row] = 0;
                }
            }
        }
        __syncthreads();
        return st;
    }

    /* ---- top-k and top-p: merge the slices' candidates ---- */
    bool need_multipass = !(r.kq > 0 && r.kq <= kFastKMax) || p.n_slices > kHistBins;
    int  total          = 0;
    if (!need_multipass) {
        __syncthreads();
        for (int cc = tid; cc < p.n_slices; cc += kThreads) {
            sh->bins[cc] = __ldcg(&recs[cc].n_cand);
        }
        __syncthreads();
        for (int cc = 0; cc < p.n_slices; cc++) {
            const int nc = sh->bins[cc];
            if (nc > p.cand_cap) {
                need_multipass = true;
            }
            total += nc;
        }
        if (total > p.fin_cap || total < r.kq) {
            need_multipass = true; /* too many ties / clustered maxima, or NaN rows */
        }
    }
    if (!need_multipass) {
        for (int cc = warp; cc < p.n_slices; cc += kWarps) {
            int off = 0;
            for (int i = 0; i < cc; i++) {
                off += sh->bins[i];
            }
            const Pair *src = p.cands + ((size_t) row * (size_t) p.n_slices + (size_t) cc) * (size_t) p.cand_cap;
            const int   nc  = sh->bins[cc];
            for (int i = lane; i < nc; i += 32) {
                Pair v;
                v.v              = __ldcg(&src[i].v);
                v.idx            = __ldcg(&src[i].idx);
                fb.fcand[off + i] = v;
            }
        }
        __syncthreads();
        if (r.mode == M_TOPK) {
            const int k = r.k;
            select_sorted(sh, fb.fcand, total, k, fb.ftmp, fb.fsort);
            if (r.select_only) {
                for (int i = tid; i < min(k, p.kept_cap); i += kThreads) {
                    kept_i[i] = fb.fsort[i].idx + p.vocab_offset;
                    kept_v[i] = fb.fsort[i].v;
                }
                if (tid == 0) {
                    p.kept_n[row] = k;
                    p.tokens[row] = fb.fsort[0].idx + p.vocab_offset;
                }
                return st;
            }
            /* sampler.c:217-222: softmax over the k kept logits (max = the first), one draw */
            const float m = fb.fsort[0].v;
            for (int i = tid; i < k; i += kThreads) {
                fb.fq[i] = exp_exact(scaled_arg(fb.fsort[i].v, m, r.inv_t));
            }
            __syncthreads();
            if (tid == 0) {
                double S = 0.0;
                for (int i = 0; i < k; i++) {
                    S += (double) fb.fq[i];
                }
                const double u    = (double) unit_from(xorshift_next(r.rng)) * S;
                double       a    = 0.0;
                int          pick = k - 1;
                for (int i = 0; i < k; i++) {
                    a += (double) fb.fq[i];
                    if (u < a) {
                        pick = i;
                        break;
                    }
                }
                p.tokens[row] = fb.fsort[pick].idx + p.vocab_offset;
                sh->S         = S;
                if (p.kept_cap > 0) {
                    p.kept_n[row] = k;
                }
            }
            __syncthreads();
            if (p.kept_cap > 0) {
                const double S = sh->S;
                for (int i = tid; i < min(k, p.kept_cap); i += kThreads) {
                    kept_i[i] = fb.fsort[i].idx + p.vocab_offset;
                    kept_v[i] = __double2float_rn((double) fb.fq[i] / S);
                }
            }
            __syncthreads();
            return st;
        }

        /* top-p over a small nucleus (sampler.c:245-300). Candidates get their exact e_i relative
         * to the row maximum; the rest of the row was summed per slice with expf relative to the
         * slice maximum and is rescaled here. */
        double part = 0.0;
        for (int i = tid; i < total; i += kThreads) {
            const float e = exp_exact(scaled_arg(fb.fcand[i].v, row_max, r.inv_t));
            fb.fcand[i].v = e;
            part += (double) e;
        }
        for (int cc = tid; cc < p.n_slices; cc += kThreads) {
            part += exp(((double) __ldcg(&recs[cc].max) - (double) row_max) * (double) r.inv_t) * __ldcg(&recs[cc].bulk);
        }
        const double S = block_sum_d(sh, part);
        for (int i = tid; i < total; i += kThreads) {
            fb.fcand[i].v = __double2float_rn((double) fb.fcand[i].v / S); /* p_i as the reference normalises it */
        }
        __syncthreads();
        /* the walk order is (p desc, id asc); the row's kq most probable ids are all candidates */
        const int kq = min(r.kq, total);
        select_sorted(sh, fb.fcand, total, kq, fb.ftmp, fb.fsort);
        if (tid == 0) {
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
        __syncthreads();
        if (sh->flag) {
            return st;
        }
        need_multipass = true;
    }
    __syncthreads();
    return st | multipass_row(p, sh, r, row_max, row_arg);
}

/* ------------------------------------------------------------------ kernel -- */

__global__ void __launch_bounds__(kThreads, 1) sample_stream_kernel(const __grid_constant__ SampleParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    unsigned char *ring   = smem_raw;
    StreamShared  *sh     = reinterpret_cast<StreamShared *>(smem_raw + (size_t) p.stages * (size_t) p.stage_bytes);
    Pair          *cstage = reinterpret_cast<Pair *>(sh + 1); /* this slice's candidates */
    FinBuffers     fb;
    fb.bitmap = reinterpret_cast<unsigned *>(cstage + p.cand_cap);
    fb.dlist  = reinterpret_cast<PenEntry *>(fb.bitmap + p.bitmap_words);
    fb.fcand  = reinterpret_cast<Pair *>(fb.dlist + p.hist_cap); /* finisher: merged candidates */
    fb.ftmp   = fb.fcand + p.fin_cap;
    fb.fsort  = fb.ftmp + p.fin_cap;                              /* kFastKMax entries */
    fb.fq     = reinterpret_cast<float *>(fb.fsort + kFastKMax);  /* kFastKMax entries */

    const int n_items  = p.n_rows * p.n_slices;
    const int G        = (int) gridDim.x;
    const int my_count = (int) blockIdx.x < n_items ? (n_items - (int) blockIdx.x + G - 1) / G : 0;

    if (tid == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&sh->full[s], 1);
        }
    }
    __syncthreads();

    /* one thread keeps the ring full: item jj of this CTA goes to stage jj % stages */
    auto issue = [&](int jj) {
        const int      item  = (int) blockIdx.x + jj * G;
        const int      row   = item / p.n_slices;
        const int      c     = item - row * p.n_slices;
        const int      s0    = c * p.slice;
        const int      n     = max(0, min(p.slice, p.V - s0));
        const unsigned bytes = (unsigned) (n & ~3) * 4u;
        if (bytes == 0u) {
            return;
        }
        const int            stage = jj % p.stages;
        unsigned char       *dst   = ring + (size_t) stage * (size_t) p.stage_bytes;
        const unsigned char *src   = reinterpret_cast<const unsigned char *>(p.logits + (size_t) row * (size_t) p.row_stride + s0);
        mbar_expect_tx(&sh->full[stage], bytes);
        for (unsigned off = 0; off < bytes; off += 32768u) {
            bulk_g2s(dst + off, src + off, min(32768u, bytes - off), &sh->full[stage]);
        }
    };
    if (tid == 0 && p.aligned) {
        for (int jj = 0; jj < min(p.stages, my_count); jj++) {
            issue(jj);
        }
    }
    unsigned phase_bits = 0u; /* parity of the next wait, one bit per stage */

    for (int j = 0; j < my_count; j++) {
        const int item  = (int) blockIdx.x + j * G;
        const int row   = item / p.n_slices;
        const int c     = item - row * p.n_slices;
        const int stage = j % p.stages;
        float    *sl    = reinterpret_cast<float *>(ring + (size_t) stage * (size_t) p.stage_bytes);
        const int s0    = c * p.slice;
        const int n     = max(0, min(p.slice, p.V - s0));
        const int nv4   = (n + 3) >> 2;
        const int body  = p.aligned ? (n & ~3) : 0;
        int       st    = ST_OK;
        RowCfg    r     = row_config(p, row);

        /* ---- 1. the slice arrives in its stage ---- */
        {
            const float *grow = p.logits + (size_t) row * (size_t) p.row_stride + s0;
            for (int i = body + tid; i < nv4 * 4; i += kThreads) {
                sl[i] = i < n ? grow[i] : -CUDART_INF_F;
            }
            if (tid == 0) {
                sh->n_cand  = 0;
                sh->n_dlist = 0;
                sh->tau     = -CUDART_INF_F;
            }
            if (r.pen_on) {
                for (int i = tid; i < p.bitmap_words; i += kThreads) {
                    fb.bitmap[i] = 0u;
                }
            }
            if (body > 0) {
                const unsigned parity = (phase_bits >> stage) & 1u;
                phase_bits ^= 1u << stage;
                if (!mbar_wait_bounded(&sh->full[stage], parity)) {
                    st |= ST_LOAD_TIMEOUT;
                    (void) mbar_wait_bounded(&sh->full[stage], parity); /* a second bounded chance for the copy in flight */
                }
            }
            __syncthreads();
        }

        /* ---- 2. penalties in shared memory, then the slice moves to registers ---- */
        if (r.pen_on) {
            st |= apply_penalties(sl, s0, n, r, p.V, p.vocab_offset, fb.bitmap, fb.dlist, p.hist_cap, &sh->n_dlist);
        }
        if (p.out_logits != nullptr) {
            float *orow = p.out_logits + (size_t) row * (size_t) p.V + s0;
            for (int i = tid; i < n; i += kThreads) {
                orow[i] = sl[i];
            }
        }
        /* warp w owns float4 [w*L, (w+1)*L) of the slice, lanes interleave: 128 consecutive ids per step */
        const int L = (nv4 + kWarps - 1) / kWarps; /* <= 128 */
        float4    x[4];
        int       base4[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int  o  = lane + 32 * i;
            const int  j4 = warp * L + o;
            const bool ok = o < L && j4 < nv4;
            base4[i]      = ok ? 4 * j4 : -1;
            x[i]          = ok ? reinterpret_cast<const float4 *>(sl)[j4] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        }
        __syncthreads(); /* the stage is free again */
        if (tid == 0 && p.aligned && j + p.stages < my_count) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(j + p.stages);
        }

        /* ---- 3. pass 1 on registers: maximum, its first id, group maxima ---- */
        float bv = -CUDART_INF_F;
        int   bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float xs[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int li = base4[i] + q;
                if (base4[i] >= 0 && li < n && (bi == 0x7fffffff || xs[q] > bv)) {
                    bv = xs[q];
                    bi = s0 + li;
                }
            }
        }
        /* groups for the select threshold: 128 / 256 / 512 per slice (8 / 4 / 2 lanes each) */
        const int  lpg      = r.kq <= 64 ? 8 : (r.kq <= 128 ? 4 : 2);
        const int  Gs       = kThreads / lpg;
        const bool fast_sel = r.kq > 0 && r.kq <= kFastKMax;
        if (fast_sel) {
            float gv = bv;
            for (int o = 1; o < lpg; o <<= 1) {
                gv = fmaxf(gv, __shfl_xor_sync(0xffffffffu, gv, o));
            }
            if ((lane % lpg) == 0) {
                sh->gmax[tid / lpg] = gv;
            }
        }
        float smax = bv;
        int   sarg = bi;
        block_argmax(sh, smax, sarg); /* its barriers also publish gmax */

        SliceRec *rec = p.recs + item;
        if (r.mode == M_TEMP) {
            /* per-warp sums of e_i relative to the SLICE maximum; the finisher rescales to the row maximum */
            double acc = 0.0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (base4[i] >= 0) {
                    const float e0 = base4[i] + 0 < n ? expf(scaled_arg(x[i].x, smax, r.inv_t)) : 0.0f;
                    const float e1 = base4[i] + 1 < n ? expf(scaled_arg(x[i].y, smax, r.inv_t)) : 0.0f;
                    const float e2 = base4[i] + 2 < n ? expf(scaled_arg(x[i].z, smax, r.inv_t)) : 0.0f;
                    const float e3 = base4[i] + 3 < n ? expf(scaled_arg(x[i].w, smax, r.inv_t)) : 0.0f;
                    acc += ((double) e0 + (double) e1) + ((double) e2 + (double) e3);
                }
            }
            acc = warp_sum_d(acc);
            if (lane == 0) {
                rec->seg[warp] = acc;
            }
        } else if (fast_sel) {
            /* tau = kq-th largest group maximum of this slice: at least kq entries are >= tau, so the
             * slice's share of the row's kq best is among them */
            for (int t = tid; t < Gs; t += kThreads) {
                const float v    = sh->gmax[t];
                int         rank = 0;
                for (int g4 = 0; g4 < Gs / 4; g4++) {
                    const float4 o = reinterpret_cast<const float4 *>(sh->gmax)[g4];
                    rank += (o.x > v || (o.x == v && 4 * g4 + 0 < t)) ? 1 : 0;
                    rank += (o.y > v || (o.y == v && 4 * g4 + 1 < t)) ? 1 : 0;
                    rank += (o.z > v || (o.z == v && 4 * g4 + 2 < t)) ? 1 : 0;
                    rank += (o.w > v || (o.w == v && 4 * g4 + 3 < t)) ? 1 : 0;
                }
                if (rank == min(r.kq, Gs) - 1) {
                    sh->tau = v;
                }
            }
            __syncthreads();
            const float tau  = sh->tau;
            double      bulk = 0.0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float xs[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
                float       part  = 0.0f;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int li = base4[i] + q;
                    if (base4[i] >= 0 && li < n) {
                        if (xs[q] >= tau) {
                            const int pos = atomicAdd(&sh->n_cand, 1);
                            if (pos < p.cand_cap) {
                                cstage[pos].v   = xs[q];
                                cstage[pos].idx = s0 + li;
                            }
                        } else if (r.mode == M_TOPP) {
                            part += expf(scaled_arg(xs[q], smax, r.inv_t));
                        }
                    }
                }
                bulk += (double) part;
            }
            if (r.mode == M_TOPP) {
                bulk = block_sum_d(sh, bulk);
            } else {
                __syncthreads();
            }
            const int nc = sh->n_cand;
            Pair     *gc = p.cands + (size_t) item * (size_t) p.cand_cap;
            for (int i = tid; i < min(nc, p.cand_cap); i += kThreads) {
                gc[i] = cstage[i];
            }
            if (tid == 0) {
                rec->n_cand = nc;
                rec->bulk   = bulk;
            }
        }
        if (tid == 0) {
            rec->max = smax;
            rec->arg = sarg;
            rec->st  = st;
        }

        /* ---- 4. the CTA that completes the row finishes it ---- */
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int old = atomicAdd(&p.row_counter[row], 1);
            sh->is_last   = old == p.n_slices - 1 ? 1 : 0;
        }
        __syncthreads();
        if (!sh->is_last) {
            continue;
        }
        __threadfence();
        const int fst = finish_row(p, sh, r, fb);
        if (tid == 0) {
            p.status[row]      = fst;
            p.row_counter[row] = 0; /* ready for the next launch */
            if (p.rng_out != nullptr && r.rr == p.rows_per_seq - 1) {
                /* the sequence's generator after all of its rows drew */
                unsigned long long s = p.rng_in ? p.rng_in[r.seq] : 1ull;
                for (int i = 0; i < p.rows_per_seq * r.draws_per_row; i++) {
                    (void) xorshift_next(s);
                }
                p.rng_out[r.seq] = s;
            }
        }
        __syncthreads();
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

cudaError_t launch_sample_stream(const SampleParams &p, int grid, size_t smem_bytes, cudaStream_t stream) {
    cudaError_t e = ensure_attributes(smem_bytes);
    if (e != cudaSuccess) {
        return e;
    }
    sample_stream_kernel<<<grid, kThreads, smem_bytes, stream>>>(p);
    return cudaGetLastError();
}

} /* namespace gb */

/*
 * sampler_kernels.cu — the logits -> token kernels (sm_100a).
 *
 * One thread-block CLUSTER owns one logits row. Each CTA of the cluster pulls
 * its contiguous slice of the row from HBM into shared memory exactly once
 * (bulk asynchronous copy signalled on an mbarrier) and every later pass —
 * penalties, max, threshold select, exp/sum, bisection — re-reads shared
 * memory, never HBM. CTAs of a cluster talk through distributed shared memory
 * (small pushes of maxima / counts / sums) and cluster barriers. Several CTAs
 * of different clusters are resident per SM, so one cluster's compute overlaps
 * another's load.
 *
 * Semantics follow geistlib's CPU sampler:
 *   mode dispatch ............ src/archs/transformer/forward/head.c:172-183
 *   argmax ................... src/engine/sampler.c:52-62
 *   softmax / inverse CDF .... src/engine/sampler.c:68-102
 *   temperature / top-k / top-p  src/engine/sampler.c:106-132, :178-228, :232-305
 *   xorshift64* .............. src/engine/sampler.c:27-48
 *   rows of one session share one generator, in order  head.c:282-303
 * Penalties and vocabulary shards have no counterpart there; their definition
 * is in the header of include/geist_b200.h.
 *
 * No bulk copy here uses cluster multicast; every CTA fetches its own slice.
 */
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "sampler_params.h"

namespace cg = cooperative_groups;

namespace gb {

struct Pair {
    float v;
    int   idx;
};

struct PenEntry {
    int   li;
    float orig;
};

struct __align__(16) RowShared {
    unsigned long long mbar;
    float              cta_max[kMaxCluster]; /* pushed by every CTA of the cluster */
    int                cta_arg[kMaxCluster];
    union {
        float  gmax[kGroupCap];               /* group maxima of the whole row (pushed) */
        double seg_sum[kMaxCluster * kWarps]; /* per-warp segment sums of the whole row (pushed) */
        struct {                              /* top-p finisher scratch (after the maxima are dead) */
            Pair  ml[kNucleusCap];
            Pair  srt[kNucleusCap];
            Pair  byp[kNucleusCap];
            float q[kNucleusCap];
        } fin;
    } u;
    double    cta_dsum[2][kMaxCluster];
    long long cta_cnt[2][kMaxCluster];
    int       cta_ncand[kMaxCluster];
    int       cta_st[kMaxCluster];
    double    cta_bulk[kMaxCluster];
    double    wred_d[2][kWarps];
    long long wred_i[2][kWarps];
    float     wred_f[kWarps];
    int       wred_a[kWarps];
    int       n_cand_local;
    int       n_dlist;
    int       decision;
    int       found_flag;
    float     tau;
};

/* ------------------------------------------------------------ small helpers -- */

__device__ __forceinline__ unsigned order_key(float x) {
    /* monotone map float -> uint32 (larger float, larger key) */
    unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long xorshift_next(unsigned long long &s) {
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return s * 0x2545F4914F6CDD1DULL;
}

__device__ __forceinline__ float unit_from(unsigned long long r) {
    return (float) (unsigned) (r >> 40) * (1.0f / 16777216.0f);
}

/* expf of the reference, for the few entries that decide a draw: the double
 * exponential rounded once to binary32 (what a correctly rounded expf gives). */
__device__ __forceinline__ float exp_exact(float a) { return __double2float_rn(exp((double) a)); }

__device__ __forceinline__ float scaled_arg(float x, float m, float inv_t) {
    return __fmul_rn(__fsub_rn(x, m), inv_t); /* two roundings, never fused */
}

__device__ __forceinline__ bool pair_before(float av, int ai, float bv, int bi) {
    return av > bv || (av == bv && ai < bi);
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

__device__ __forceinline__ long long warp_sum_ll(long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

/* mbarrier + bulk copy (global -> this CTA's shared memory, no multicast) */
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, unsigned bytes, unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
    return ok != 0;
}

/* Bounded wait. Returns false when the copy never signalled. */
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long *bar, unsigned parity) {
    for (int i = 0; i < (1 << 20); i++) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
    }
    return false;
}

/* ------------------------------------------------------------ row context -- */

struct Ctx {
    RowShared        *sh;
    float            *sl;  /* slice buffer */
    int               C, crank, tid, lane, warp;
    int               V, s0, n, nv4; /* slice = global ids [s0, s0+n); nv4 float4 incl. -inf padding */
    int               idx_bits;
    unsigned          par; /* parity of the next cluster reduction */
};

/* Visit every element of the slice: f(value, local index). Warp w owns a
 * contiguous run of float4, lanes interleave inside it, so one warp iteration
 * covers 128 consecutive vocabulary ids. */
template <class F>
__device__ __forceinline__ void sweep(const Ctx &c, F &&f) {
    const int     L = (c.nv4 + kWarps - 1) / kWarps;
    const int     b = c.warp * L;
    const int     e = min(b + L, c.nv4);
    const float4 *p = reinterpret_cast<const float4 *>(c.sl);
    for (int j = b + c.lane; j < e; j += 32) {
        const float4 x = p[j];
        f(x.x, 4 * j);
        f(x.y, 4 * j + 1);
        f(x.z, 4 * j + 2);
        f(x.w, 4 * j + 3);
    }
}

/* Same traversal, rewriting each element in place. */
template <class F>
__device__ __forceinline__ void sweep_rw(const Ctx &c, F &&f) {
    const int L = (c.nv4 + kWarps - 1) / kWarps;
    const int b = c.warp * L;
    const int e = min(b + L, c.nv4);
    float4   *p = reinterpret_cast<float4 *>(c.sl);
    for (int j = b + c.lane; j < e; j += 32) {
        float4 x = p[j];
        x.x      = f(x.x, 4 * j);
        x.y      = f(x.y, 4 * j + 1);
        x.z      = f(x.z, 4 * j + 2);
        x.w      = f(x.w, 4 * j + 3);
        p[j]     = x;
    }
}

/* Sum a per-thread value over the whole cluster; every thread of every CTA
 * gets the same total (same values added in the same order everywhere). */
__device__ double cluster_sum_d(Ctx &c, double v) {
    const unsigned par = c.par & 1u;
    c.par++;
    v = warp_sum_d(v);
    if (c.lane == 0) {
        c.sh->wred_d[par][c.warp] = v;
    }
    __syncthreads();
    if (c.tid < c.C) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            t += c.sh->wred_d[par][w];
        }
        *cg::this_cluster().map_shared_rank(&c.sh->cta_dsum[par][c.crank], c.tid) = t;
    }
    cg::this_cluster().sync();
    double tot = 0.0;
    for (int i = 0; i < c.C; i++) {
        tot += c.sh->cta_dsum[par][i];
    }
    return tot;
}

__device__ long long cluster_sum_ll(Ctx &c, long long v) {
    const unsigned par = c.par & 1u;
    c.par++;
    v = warp_sum_ll(v);
    if (c.lane == 0) {
        c.sh->wred_i[par][c.warp] = v;
    }
    __syncthreads();
    if (c.tid < c.C) {
        long long t = 0;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            t += c.sh->wred_i[par][w];
        }
        *cg::this_cluster().map_shared_rank(&c.sh->cta_cnt[par][c.crank], c.tid) = t;
    }
    cg::this_cluster().sync();
    long long tot = 0;
    for (int i = 0; i < c.C; i++) {
        tot += c.sh->cta_cnt[par][i];
    }
    return tot;
}

/* (key, id) packed so that a larger word comes earlier in (key desc, id asc). */
__device__ __forceinline__ unsigned long long composite(unsigned key, int gid, int idx_bits) {
    const unsigned long long mask = (1ull << idx_bits) - 1ull;
    return ((unsigned long long) key << idx_bits) | (mask - (unsigned long long) gid);
}

/* ------------------------------------------------ generic (bisection) paths -- */

/* Largest composite word t such that at least `want` elements are >= t. */
__device__ unsigned long long bisect_rank(Ctx &c, long long want) {
    unsigned long long prefix = 0;
    for (int bit = 31 + c.idx_bits; bit >= 0; bit--) {
        const unsigned long long t   = prefix | (1ull << bit);
        long long                cnt = 0;
        sweep(c, [&](float x, int li) {
            if (li < c.n && composite(order_key(x), c.s0 + li, c.idx_bits) >= t) {
                cnt++;
            }
        });
        if (cluster_sum_ll(c, cnt) >= want) {
            prefix = t;
        }
    }
    return prefix;
}

/* Largest composite word t with mass{word >= t} REL target, where REL is >= (inclusive)
 * or > (strict). weight(x, li) gives the element's mass (0 for elements outside the set);
 * key(x) its ordering key. */
template <class KeyF, class MassF>
__device__ unsigned long long bisect_mass(Ctx &c, double target, bool inclusive, KeyF &&key, MassF &&mass) {
    unsigned long long prefix = 0;
    for (int bit = 31 + c.idx_bits; bit >= 0; bit--) {
        const unsigned long long t = prefix | (1ull << bit);
        double                   m = 0.0;
        sweep(c, [&](float x, int li) {
            if (li < c.n && composite(key(x), c.s0 + li, c.idx_bits) >= t) {
                m += mass(x, li);
            }
        });
        const double tot = cluster_sum_d(c, m);
        if (inclusive ? (tot >= target) : (tot > target)) {
            prefix = t;
        }
    }
    return prefix;
}

/* ------------------------------------------------------------------ kernel -- */

__global__ void __launch_bounds__(kThreads) sample_rows_kernel(const __grid_constant__ SampleParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];

    Ctx c;
    c.C     = (int) cg::this_cluster().num_blocks();
    c.crank = (int) cg::this_cluster().block_rank();
    c.tid   = threadIdx.x;
    c.lane  = c.tid & 31;
    c.warp  = c.tid >> 5;
    c.par   = 0;
    c.sl    = reinterpret_cast<float *>(smem_raw);
    c.sh    = reinterpret_cast<RowShared *>(smem_raw + p.slice_bytes);
    Pair     *cand   = reinterpret_cast<Pair *>(c.sh + 1); /* this CTA's candidates for the row's finisher */
    unsigned *bitmap = reinterpret_cast<unsigned *>(cand + p.cand_cap);
    PenEntry *dlist  = reinterpret_cast<PenEntry *>(bitmap + p.bitmap_words);
    RowShared *sh    = c.sh;

    const int row  = blockIdx.x / c.C;
    const int seq0 = row / p.rows_per_seq;
    const int rr   = row - seq0 * p.rows_per_seq;
    const int seq  = p.slot ? p.slot[seq0] : seq0; /* where this sequence's parameters, history and generator live */
    c.V           = p.V;
    c.s0          = c.crank * p.slice;
    c.n           = max(0, min(p.slice, p.V - c.s0));
    c.nv4         = (c.n + 3) >> 2;
    c.idx_bits    = 32 - __clz(max(p.V - 1, 1));

    const float T     = p.temperature[seq];
    const int   top_k = p.top_k[seq];
    const float top_p = p.top_p[seq];
    /* head.c:172-183 folded with the early-outs of the three sampler functions */
    enum { M_ARGMAX, M_TOPK, M_TOPP, M_TEMP } mode;
    if (!(T > 0.0f)) {
        mode = M_ARGMAX;
    } else if (top_k > 1) {
        mode = top_k >= p.V ? M_TEMP : M_TOPK;
    } else if (top_p > 0.0f && top_p < 1.0f) {
        mode = M_TOPP;
    } else {
        mode = M_TEMP;
    }
    const bool select_only = (p.flags & F_SELECT_ONLY) != 0;
    int        k           = min(top_k, kTopKClamp);
    if (select_only) {
        mode = M_TOPK;
        k    = min(max(top_k, 1), min(p.V, kTopKClamp));
    }
    const float inv_t = T > 0.0f ? __fdiv_rn(1.0f, T) : 1.0f;
    int         st    = ST_OK;

    /* generator state this row starts from: the sequence's state after the draws of rows 0..rr-1 */
    const int          draws_per_row = (T > 0.0f && !select_only) ? 1 : 0;
    unsigned long long rng           = p.rng_in ? p.rng_in[seq] : 1ull;
    for (int i = 0; i < rr * draws_per_row; i++) {
        (void) xorshift_next(rng);
    }

    /* ---- 1. the slice: HBM -> shared memory, once ---- */
    const float *grow = p.logits + (size_t) row * (size_t) p.row_stride + c.s0;
    if (c.tid == 0) {
        sh->n_cand_local = 0;
        sh->n_dlist      = 0;
        sh->decision     = 0;
        sh->found_flag   = 0;
        sh->tau          = -CUDART_INF_F;
        mbar_init(&sh->mbar, 1);
    }
    __syncthreads();
    const int body = p.aligned ? (c.n & ~3) : 0; /* floats moved by bulk copies */
    if (c.tid == 0 && body > 0) {
        const unsigned bytes = (unsigned) body * 4u;
        mbar_expect_tx(&sh->mbar, bytes);
        for (unsigned off = 0; off < bytes; off += 32768u) {
            const unsigned len = min(32768u, bytes - off);
            bulk_g2s(reinterpret_cast<unsigned char *>(c.sl) + off, reinterpret_cast<const unsigned char *>(grow) + off, len, &sh->mbar);
        }
    }
    for (int i = body + c.tid; i < c.nv4 * 4; i += kThreads) {
        c.sl[i] = i < c.n ? grow[i] : -CUDART_INF_F;
    }
    const bool pen_on = p.hist != nullptr || p.extra != nullptr;
    if (pen_on) {
        for (int i = c.tid; i < p.bitmap_words; i += kThreads) {
            bitmap[i] = 0u;
        }
    }
    if (body > 0 && !mbar_wait_bounded(&sh->mbar, 0)) {
        st |= ST_LOAD_TIMEOUT;
        (void) mbar_wait_bounded(&sh->mbar, 0); /* give the copy in flight a second bounded chance to land */
    }
    __syncthreads();

    /* ---- 2. penalties, in shared memory ---- */
    if (pen_on) {
        const int H   = p.hist ? (int) min((long long) max(p.hist_len[seq], 0), p.hist_stride) : 0;
        const int E   = p.extra ? rr : 0; /* proposals fed before this row: extra[1..rr] */
        float     rep = p.rep ? p.rep[seq] : 1.0f;
        if (!(rep > 0.0f)) {
            rep = 1.0f;
        }
        const float freq = p.freq ? p.freq[seq] : 0.0f;
        const float pres = p.pres ? p.pres[seq] : 0.0f;
        const int  *hrow = p.hist ? p.hist + (size_t) seq * (size_t) p.hist_stride : nullptr;
        const int  *erow = p.extra ? p.extra + (size_t) seq0 * (size_t) p.extra_stride : nullptr; /* per call, not per slot */
        /* (a) first thread to mark an id owns it: it saves the original value */
        for (int j = c.tid; j < H + E; j += kThreads) {
            const int id = (j < H ? hrow[j] : erow[1 + j - H]) - p.vocab_offset;
            const int li = id - c.s0;
            if (id >= 0 && id < p.V && li >= 0 && li < c.n) {
                const unsigned bit = 1u << (li & 31);
                const unsigned old = atomicOr(&bitmap[li >> 5], bit);
                if (!(old & bit)) {
                    const int pos = atomicAdd(&sh->n_dlist, 1);
                    if (pos < p.hist_cap) {
                        dlist[pos].li   = li;
                        dlist[pos].orig = c.sl[li];
                    }
                }
            }
        }
        __syncthreads();
        int nd = sh->n_dlist;
        if (nd > p.hist_cap) { /* cannot happen when the launcher sized hist_cap; keep the row consistent anyway */
            st |= ST_HIST_OVERFLOW;
            nd = 0;
        }
        /* (b) the slot becomes an integer counter */
        for (int i = c.tid; i < nd; i += kThreads) {
            reinterpret_cast<int *>(c.sl)[dlist[i].li] = 0;
        }
        __syncthreads();
        if (nd > 0) {
            for (int j = c.tid; j < H + E; j += kThreads) {
                const int id = (j < H ? hrow[j] : erow[1 + j - H]) - p.vocab_offset;
                const int li = id - c.s0;
                if (id >= 0 && id < p.V && li >= 0 && li < c.n) {
                    atomicAdd(reinterpret_cast<int *>(c.sl) + li, 1);
                }
            }
        }
        __syncthreads();
        /* (c) one thread per distinct id writes the penalised value */
        for (int i = c.tid; i < nd; i += kThreads) {
            const int   li  = dlist[i].li;
            const int   cnt = reinterpret_cast<int *>(c.sl)[li];
            float       x   = dlist[i].orig;
            x               = x > 0.0f ? __fdiv_rn(x, rep) : __fmul_rn(x, rep);
            x               = __fsub_rn(x, __fmul_rn((float) cnt, freq));
            x               = __fsub_rn(x, pres);
            c.sl[li]        = x;
        }
        __syncthreads();
    }
    if (p.out_logits != nullptr) {
        float *orow = p.out_logits + (size_t) row * (size_t) p.V + c.s0;
        for (int i = c.tid; i < c.n; i += kThreads) {
            orow[i] = c.sl[i];
        }
    }

    /* ---- 3. pass 1: maximum, first index of the maximum, group maxima ---- */
    float bv = -CUDART_INF_F;
    int   bi = 0x7fffffff;
    sweep(c, [&](float x, int li) {
        if (li < c.n && (bi == 0x7fffffff || x > bv)) {
            bv = x;
            bi = c.s0 + li;
        }
    });
    /* group layout for the select threshold: gpc groups per CTA, lpg lanes per group */
    int kq = 0; /* how many candidates the threshold must let through */
    if (mode == M_TOPK) {
        kq = k;
    } else if (mode == M_TOPP) {
        kq = min(kNucleusProbe, p.V);
    }
    int gpc = kWarps;
    while (gpc * c.C < 2 * kq && gpc * 2 * c.C <= kGroupCap && gpc < kThreads) {
        gpc *= 2;
    }
    const int  lpg       = kThreads / gpc; /* 32 .. 1 */
    const int  G         = gpc * c.C;
    const bool fast_sel  = kq > 0 && kq <= kFastKMax && G >= kq;
    {
        float gv = bv;
        for (int o = 1; o < lpg; o <<= 1) {
            gv = fmaxf(gv, __shfl_xor_sync(0xffffffffu, gv, o));
        }
        if (fast_sel && (c.lane % lpg) == 0) {
            const int g = c.tid / lpg;
            for (int peer = 0; peer < c.C; peer++) {
                cg::this_cluster().map_shared_rank(sh->u.gmax, peer)[c.crank * gpc + g] = gv;
            }
        }
        float wv = bv;
        int   wi = bi;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
            const int   oi = __shfl_xor_sync(0xffffffffu, wi, o);
            if (pair_before(ov, oi, wv, wi)) {
                wv = ov;
                wi = oi;
            }
        }
        if (c.lane == 0) {
            sh->wred_f[c.warp] = wv;
            sh->wred_a[c.warp] = wi;
        }
        __syncthreads();
        if (c.tid < c.C) {
            float mv = sh->wred_f[0];
            int   mi = sh->wred_a[0];
            for (int w = 1; w < kWarps; w++) {
                if (pair_before(sh->wred_f[w], sh->wred_a[w], mv, mi)) {
                    mv = sh->wred_f[w];
                    mi = sh->wred_a[w];
                }
            }
            RowShared *peer         = cg::this_cluster().map_shared_rank(sh, c.tid);
            peer->cta_max[c.crank] = mv;
            peer->cta_arg[c.crank] = mi;
            peer->cta_st[c.crank]  = st; /* load / history problems of any slice reach the writer */
        }
    }
    cg::this_cluster().sync();
    float row_max = sh->cta_max[0];
    int   row_arg = sh->cta_arg[0];
    for (int i = 1; i < c.C; i++) {
        if (pair_before(sh->cta_max[i], sh->cta_arg[i], row_max, row_arg)) {
            row_max = sh->cta_max[i];
            row_arg = sh->cta_arg[i];
        }
    }
    for (int i = 0; i < c.C; i++) {
        st |= sh->cta_st[i];
    }

    const bool writer = c.crank == 0 && c.tid == 0;
    int       *kept_i = p.kept_cap > 0 ? p.kept_idx + (size_t) row * (size_t) p.kept_cap : nullptr;
    float     *kept_v = p.kept_cap > 0 ? p.kept_val + (size_t) row * (size_t) p.kept_cap : nullptr;

    /* ================================================================ greedy == */
    if (mode == M_ARGMAX) {
        if (writer) {
            p.tokens[row] = row_arg + p.vocab_offset;
            if (p.kept_cap > 0) {
                p.kept_n[row] = 0;
            }
        }
    }

    /* ========================================================== temperature == */
    else if (mode == M_TEMP) {
        /* per-warp segment sums of e_i = expf((x - max) * inv_t), pushed to every CTA */
        double acc = 0.0;
        sweep(c, [&](float x, int li) {
            if (li < c.n) {
                acc += (double) expf(scaled_arg(x, row_max, inv_t));
            }
        });
        acc = warp_sum_d(acc);
        if (c.lane < c.C) {
            cg::this_cluster().map_shared_rank(sh->u.seg_sum, c.lane)[c.crank * kWarps + c.warp] = acc;
        }
        cg::this_cluster().sync();
        /* every CTA walks the same kWarps*C numbers in id order */
        const int    nseg = c.C * kWarps;
        double       S    = 0.0;
        for (int i = 0; i < nseg; i++) {
            S += sh->u.seg_sum[i];
        }
        const float  unit = unit_from(xorshift_next(rng));
        const double u    = (double) unit * S;
        double       run  = 0.0;
        int          hit  = -1;
        double       base = 0.0;
        for (int i = 0; i < nseg; i++) {
            const double nxt = run + sh->u.seg_sum[i];
            if (hit < 0 && u < nxt) {
                hit  = i;
                base = run;
            }
            run = nxt;
        }
        if (hit < 0) { /* u >= S cannot happen for unit < 1, but stay defined */
            hit  = nseg - 1;
            base = run - sh->u.seg_sum[nseg - 1];
        }
        if (hit / kWarps == c.crank && hit % kWarps == c.warp) {
            /* this warp owns the segment with the crossing: walk it 128 ids at a time */
            const int     L     = (c.nv4 + kWarps - 1) / kWarps;
            const int     b     = c.warp * L;
            const int     e     = min(b + L, c.nv4);
            const float4 *pv    = reinterpret_cast<const float4 *>(c.sl);
            int           found = -1;
            int           last  = -1; /* last real id of the segment */
            for (int j0 = b; j0 < e && found < 0; j0 += 32) {
                const int j = j0 + c.lane;
                float     ev[4] = {0.f, 0.f, 0.f, 0.f};
                if (j < e) {
                    const float4 x  = pv[j];
                    const float  xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        ev[q] = (4 * j + q) < c.n ? expf(scaled_arg(xs[q], row_max, inv_t)) : 0.0f;
                    }
                }
                double mine = ((double) ev[0] + (double) ev[1]) + ((double) ev[2] + (double) ev[3]);
                double incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const double t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (c.lane >= o) {
                        incl += t;
                    }
                }
                const double   excl = base + (incl - mine);
                const unsigned ball = __ballot_sync(0xffffffffu, j < e && u < base + incl);
                if (ball != 0u) {
                    const int src = __ffs(ball) - 1;
                    if (c.lane == src) {
                        double a = excl;
                        int    f = 4 * j + 3;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            a += (double) ev[q];
                            if (u < a) {
                                f = 4 * j + q;
                                break;
                            }
                        }
                        found = min(f, c.n - 1);
                    }
                    found = __shfl_sync(0xffffffffu, found, src);
                }
                base += __shfl_sync(0xffffffffu, incl, 31);
                last = min(4 * min(j0 + 31, e - 1) + 3, c.n - 1);
            }
            if (found < 0) {
                found = last; /* regrouped double sums may end a hair below the segment total */
            }
            if (c.lane == 0) {
                p.tokens[row] = c.s0 + found + p.vocab_offset;
            }
        }
        if (writer && p.kept_cap > 0) {
            p.kept_n[row] = 0;
        }
    }

    /* ====================================================== top-k and top-p == */
    else {
        bool  need_generic = !fast_sel;
        float tau          = -CUDART_INF_F;
        if (fast_sel) {
            /* tau = kq-th largest group maximum: a lower bound of the kq-th largest element */
            for (int t = c.tid; t < G; t += kThreads) {
                const float v    = sh->u.gmax[t];
                int         rank = 0;
                for (int j = 0; j < G; j++) {
                    const float o = sh->u.gmax[j];
                    rank += (o > v || (o == v && j < t)) ? 1 : 0;
                }
                if (rank == kq - 1) {
                    sh->tau = v;
                }
            }
            __syncthreads();
            tau = sh->tau;
        }

        /* pass 2: collect everything >= tau; top-p also sums the rest of the row */
        double bulk = 0.0;
        if (fast_sel) {
            sweep(c, [&](float x, int li) {
                if (li < c.n) {
                    if (x >= tau) {
                        const int pos = atomicAdd(&sh->n_cand_local, 1);
                        if (pos < p.cand_cap) {
                            cand[pos].v   = x;
                            cand[pos].idx = c.s0 + li;
                        }
                    } else if (mode == M_TOPP) {
                        bulk += (double) expf(scaled_arg(x, row_max, inv_t));
                    }
                }
            });
            if (mode == M_TOPP) {
                bulk = warp_sum_d(bulk);
                if (c.lane == 0) {
                    sh->wred_d[0][c.warp] = bulk;
                }
            }
            __syncthreads();
            if (c.tid < c.C) {
                RowShared *peer          = cg::this_cluster().map_shared_rank(sh, c.tid);
                peer->cta_ncand[c.crank] = sh->n_cand_local;
                if (mode == M_TOPP) {
                    double t = 0.0;
                    for (int w = 0; w < kWarps; w++) {
                        t += sh->wred_d[0][w];
                    }
                    peer->cta_bulk[c.crank] = t;
                }
            }
            cg::this_cluster().sync(); /* barrier A: candidate lists are complete and nobody reads its slice any more */
            int total = 0;
            for (int i = 0; i < c.C; i++) {
                const int nc = sh->cta_ncand[i];
                if (nc > p.cand_cap) {
                    need_generic = true;
                }
                total += nc;
            }
            if (total < kq) {
                need_generic = true; /* only with NaN rows */
            }
            if (mode == M_TOPP && total > kNucleusCap) {
                need_generic = true;
            }

            if (!need_generic && c.crank == 0) {
                /* the finisher pulls all candidate lists into its (now idle) slice buffer */
                /* top-k: scratch in the (now idle) slice buffer, which the launcher sizes for it.
                 * top-p: scratch in the dead group-maxima area, because a failed probe must leave
                 * the slice intact for the bisection path. */
                const bool in_slice = mode == M_TOPK;
                const int  fcap     = c.C * p.cand_cap;
                Pair      *ml       = in_slice ? reinterpret_cast<Pair *>(c.sl) : sh->u.fin.ml; /* merged, unsorted */
                Pair      *sorted   = in_slice ? ml + fcap : sh->u.fin.srt;                     /* walk order */
                float     *q        = in_slice ? reinterpret_cast<float *>(sorted + fcap) : sh->u.fin.q;
                if (c.warp < c.C) {
                    int off = 0;
                    for (int i = 0; i < c.warp; i++) {
                        off += sh->cta_ncand[i];
                    }
                    const Pair *src = cg::this_cluster().map_shared_rank(cand, c.warp);
                    const int   nc  = sh->cta_ncand[c.warp];
                    for (int i = c.lane; i < nc; i += 32) {
                        ml[off + i] = src[i];
                    }
                }
                __syncthreads();
                /* rank sort by (value desc, id asc): all ids are distinct, ranks are a permutation */
                for (int t = c.tid; t < total; t += kThreads) {
                    const Pair me   = ml[t];
                    int        rank = 0;
                    for (int j = 0; j < total; j++) {
                        rank += pair_before(ml[j].v, ml[j].idx, me.v, me.idx) ? 1 : 0;
                    }
                    sorted[rank] = me;
                }
                __syncthreads();

                if (mode == M_TOPK && select_only) {
                    for (int i = c.tid; i < min(k, p.kept_cap); i += kThreads) {
                        kept_i[i] = sorted[i].idx + p.vocab_offset;
                        kept_v[i] = sorted[i].v;
                    }
                    if (c.tid == 0) {
                        p.kept_n[row] = k;
                        p.tokens[row] = sorted[0].idx + p.vocab_offset;
                    }
                } else if (mode == M_TOPK) {
                    /* sampler.c:217-222: softmax over the k kept logits (max = the first), one draw */
                    const float m = sorted[0].v;
                    for (int i = c.tid; i < k; i += kThreads) {
                        q[i] = exp_exact(scaled_arg(sorted[i].v, m, inv_t));
                    }
                    __syncthreads();
                    if (c.tid == 0) {
                        double S = 0.0;
                        for (int i = 0; i < k; i++) {
                            S += (double) q[i];
                        }
                        const double u    = (double) unit_from(xorshift_next(rng)) * S;
                        double       a    = 0.0;
                        int          pick = k - 1;
                        for (int i = 0; i < k; i++) {
                            a += (double) q[i];
                            if (u < a) {
                                pick = i;
                                break;
                            }
                        }
                        p.tokens[row]       = sorted[pick].idx + p.vocab_offset;
                        sh->cta_dsum[0][0]  = S;
                        if (p.kept_cap > 0) {
                            p.kept_n[row] = k;
                        }
                    }
                    __syncthreads();
                    if (p.kept_cap > 0) {
                        const double S = sh->cta_dsum[0][0];
                        for (int i = c.tid; i < min(k, p.kept_cap); i += kThreads) {
                            kept_i[i] = sorted[i].idx + p.vocab_offset;
                            kept_v[i] = __double2float_rn((double) q[i] / S);
                        }
                    }
                } else {
                    /* top-p over a small nucleus (sampler.c:245-300). Candidates carry their exact
                     * e_i; everything else was summed with expf. */
                    for (int i = c.tid; i < total; i += kThreads) {
                        q[i] = exp_exact(scaled_arg(sorted[i].v, row_max, inv_t));
                    }
                    __syncthreads();
                    if (c.tid == 0) {
                        double S = 0.0;
                        for (int i = 0; i < c.C; i++) {
                            S += sh->cta_bulk[i];
                        }
                        for (int i = total - 1; i >= 0; i--) {
                            S += (double) q[i]; /* small terms first */
                        }
                        sh->cta_dsum[0][0] = S;
                    }
                    __syncthreads();
                    const double S = sh->cta_dsum[0][0];
                    for (int i = c.tid; i < total; i += kThreads) {
                        q[i] = __double2float_rn((double) q[i] / S); /* p_i as the reference normalises it */
                    }
                    __syncthreads();
                    /* walk order is (p desc, id asc); p is monotone in the logit, so only runs of
                     * equal p can be out of place: re-rank on (p, id) */
                    Pair *byp = sh->u.fin.byp;
                    for (int t = c.tid; t < total; t += kThreads) {
                        const float pv = q[t];
                        const int   id = sorted[t].idx;
                        int         rank = 0;
                        for (int j = 0; j < total; j++) {
                            rank += pair_before(q[j], sorted[j].idx, pv, id) ? 1 : 0;
                        }
                        byp[rank].v   = pv;
                        byp[rank].idx = id;
                    }
                    __syncthreads();
                    if (c.tid == 0) {
                        const float  p_floor = byp[total - 1].v; /* nothing outside the candidates has a larger p */
                        double       cum     = 0.0;
                        int          cut     = -1;
                        for (int i = 0; i < total; i++) {
                            cum += (double) byp[i].v;
                            if (cum >= (double) top_p) {
                                cut = i + 1;
                                break;
                            }
                        }
                        const bool all_in = total >= p.V;
                        bool       ok     = cut > 0 && (byp[cut - 1].v > p_floor || all_in);
                        if (cut < 0 && all_in) { /* never reached top_p: the nucleus is the whole row */
                            cut = total;
                            ok  = true;
                        }
                        if (ok) {
                            double N = 0.0;
                            for (int i = 0; i < cut; i++) {
                                N += (double) byp[i].v;
                            }
                            const double u    = (double) unit_from(xorshift_next(rng)) * N;
                            double       a    = 0.0;
                            int          pick = cut - 1;
                            for (int i = 0; i < cut; i++) {
                                a += (double) byp[i].v;
                                if (u < a) {
                                    pick = i;
                                    break;
                                }
                            }
                            p.tokens[row] = byp[pick].idx + p.vocab_offset;
                            if (p.kept_cap > 0) {
                                p.kept_n[row] = cut;
                                for (int i = 0; i < min(cut, p.kept_cap); i++) {
                                    kept_i[i] = byp[i].idx + p.vocab_offset;
                                    kept_v[i] = __double2float_rn((double) byp[i].v / N);
                                }
                            }
                        }
                        /* tell the whole cluster whether the bisection path must redo this row */
                        for (int peer = 0; peer < c.C; peer++) {
                            cg::this_cluster().map_shared_rank(sh, peer)->decision = ok ? 1 : 2;
                        }
                    }
                }
            }
            cg::this_cluster().sync(); /* barrier B: the finisher is done reading its peers' lists */
            if (mode == M_TOPP && !need_generic) {
                need_generic = sh->decision != 1;
            }
        }

        if (need_generic) {
            st |= ST_SLOW_PATH;
            if (mode == M_TOPK) {
                /* exact set: the k largest (value, id) words */
                const unsigned long long t_set = bisect_rank(c, (long long) k);
                auto                     in_set = [&](float x, int li) { return composite(order_key(x), c.s0 + li, c.idx_bits) >= t_set; };
                if (select_only) {
                    /* hand the set out unsorted; the merge step orders candidates anyway */
                    long long mine = 0;
                    sweep(c, [&](float x, int li) {
                        if (li < c.n && in_set(x, li)) {
                            mine++;
                        }
                    });
                    mine = warp_sum_ll(mine);
                    if (c.lane == 0) {
                        sh->wred_i[0][c.warp] = mine;
                    }
                    __syncthreads();
                    if (c.tid < c.C) {
                        long long t = 0;
                        for (int w = 0; w < kWarps; w++) {
                            t += sh->wred_i[0][w];
                        }
                        cg::this_cluster().map_shared_rank(sh, c.tid)->cta_ncand[c.crank] = (int) t;
                    }
                    if (c.tid == 0) {
                        sh->n_cand_local = 0;
                    }
                    cg::this_cluster().sync();
                    int off = 0;
                    for (int i = 0; i < c.crank; i++) {
                        off += sh->cta_ncand[i];
                    }
                    sweep(c, [&](float x, int li) {
                        if (li < c.n && in_set(x, li)) {
                            const int pos = off + atomicAdd(&sh->n_cand_local, 1);
                            if (pos < p.kept_cap) {
                                kept_i[pos] = c.s0 + li + p.vocab_offset;
                                kept_v[pos] = x;
                            }
                        }
                    });
                    if (writer) {
                        p.kept_n[row] = k;
                        p.tokens[row] = row_arg + p.vocab_offset;
                    }
                } else {
                    auto   qof = [&](float x) { return (double) exp_exact(scaled_arg(x, row_max, inv_t)); };
                    double m   = 0.0;
                    sweep(c, [&](float x, int li) {
                        if (li < c.n && in_set(x, li)) {
                            m += qof(x);
                        }
                    });
                    const double S = cluster_sum_d(c, m);
                    const double u = (double) unit_from(xorshift_next(rng)) * S;
                    /* the pick is the earliest walk position whose running sum exceeds u, i.e. the
                     * largest word t with mass{word >= t} > u */
                    unsigned long long t_pick = bisect_mass(
                            c, u, false, [&](float x) { return order_key(x); },
                            [&](float x, int li) { return in_set(x, li) ? qof(x) : 0.0; });
                    if (t_pick < t_set) {
                        t_pick = t_set;
                    }
                    sweep(c, [&](float x, int li) {
                        if (li < c.n && composite(order_key(x), c.s0 + li, c.idx_bits) == t_pick) {
                            p.tokens[row] = c.s0 + li + p.vocab_offset;
                        }
                    });
                    if (writer && p.kept_cap > 0) {
                        p.kept_n[row] = k;
                        st |= ST_KEPT_PARTIAL;
                    }
                }
            } else {
                /* top-p, any nucleus size. The slice is rewritten in place: e_i, then p_i. */
                double acc = 0.0;
                sweep_rw(c, [&](float x, int li) {
                    if (li >= c.n) {
                        return 0.0f;
                    }
                    const float e = expf(scaled_arg(x, row_max, inv_t));
                    acc += (double) e;
                    return e;
                });
                const double S = cluster_sum_d(c, acc);
                sweep_rw(c, [&](float e, int li) { return li < c.n ? __double2float_rn((double) e / S) : 0.0f; });
                __syncthreads();
                auto keyf  = [](float pv) { return __float_as_uint(pv); }; /* p >= 0: bits are ordered */
                auto massf = [](float pv, int) { return (double) pv; };
                /* cutoff: first walk position whose running sum reaches top_p (inclusive) */
                const unsigned long long t_cut = bisect_mass(c, (double) top_p, true, keyf, massf);
                double                   nm    = 0.0;
                long long                ncnt  = 0;
                sweep(c, [&](float pv, int li) {
                    if (li < c.n && composite(keyf(pv), c.s0 + li, c.idx_bits) >= t_cut) {
                        nm += (double) pv;
                        ncnt++;
                    }
                });
                const double    N   = cluster_sum_d(c, nm);
                const long long cut = cluster_sum_ll(c, ncnt);
                const double    u   = (double) unit_from(xorshift_next(rng)) * N;
                unsigned long long t_pick = bisect_mass(c, u, false, keyf, massf);
                if (t_pick < t_cut) {
                    t_pick = t_cut; /* default: the last nucleus entry (sampler.c:292) */
                }
                sweep(c, [&](float pv, int li) {
                    if (li < c.n && composite(keyf(pv), c.s0 + li, c.idx_bits) == t_pick) {
                        p.tokens[row] = c.s0 + li + p.vocab_offset;
                    }
                });
                if (writer && p.kept_cap > 0) {
                    p.kept_n[row] = (int) cut;
                    st |= ST_KEPT_PARTIAL;
                }
            }
        }
    }

    if (writer) {
        p.status[row] = st;
        if (p.rng_out != nullptr && rr == p.rows_per_seq - 1) {
            /* the sequence's generator after all of its rows drew */
            unsigned long long s = p.rng_in ? p.rng_in[seq] : 1ull;
            for (int i = 0; i < p.rows_per_seq * draws_per_row; i++) {
                (void) xorshift_next(s);
            }
            p.rng_out[seq] = s;
        }
    }
}

/* ------------------------------------------------- merge of shard candidates -- */

/* One CTA per row: the union of the per-shard lists, ordered by (value desc,
 * global id asc), cut to k, then the top-k draw of sampler.c:217-222. */
__global__ void __launch_bounds__(256) merge_sample_kernel(const __grid_constant__ MergeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int row   = blockIdx.x;
    const int cap   = p.n_shards * p.k_stride;
    Pair     *ml    = reinterpret_cast<Pair *>(smem_raw);
    Pair     *srt   = ml + cap;
    float    *q     = reinterpret_cast<float *>(srt + cap);
    __shared__ int    n_total;
    __shared__ double S_sh;
    if (threadIdx.x == 0) {
        n_total = 0;
    }
    __syncthreads();
    for (int s = 0; s < p.n_shards; s++) {
        const int    nc  = min(p.cand_n[(size_t) s * p.n_rows + row], p.k_stride);
        const size_t off = ((size_t) s * p.n_rows + row) * (size_t) p.k_stride;
        __shared__ int base;
        if (threadIdx.x == 0) {
            base = n_total;
            n_total += nc;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nc; i += blockDim.x) {
            ml[base + i].v   = p.cand_val[off + i];
            ml[base + i].idx = p.cand_gid[off + i];
        }
        __syncthreads();
    }
    const int total = n_total;
    for (int t = threadIdx.x; t < total; t += blockDim.x) {
        const Pair me   = ml[t];
        int        rank = 0;
        for (int j = 0; j < total; j++) {
            rank += pair_before(ml[j].v, ml[j].idx, me.v, me.idx) ? 1 : 0;
        }
        srt[rank] = me;
    }
    __syncthreads();
    const float T     = p.temperature[row];
    int         k     = min(min(p.top_k[row], kTopKClamp), total);
    const float inv_t = T > 0.0f ? __fdiv_rn(1.0f, T) : 1.0f;
    if (!(T > 0.0f) || k <= 1) {
        /* greedy: best candidate, no draw (sampler.c:184-186) */
        if (threadIdx.x == 0) {
            p.tokens[row] = total > 0 ? srt[0].idx : -1;
            p.status[row] = total > 0 ? ST_OK : ST_INTERNAL;
            if (p.rng_out) {
                p.rng_out[row] = p.rng_in[row];
            }
            if (p.kept_cap > 0) {
                p.kept_n[row] = 0;
            }
        }
        return;
    }
    const float m = srt[0].v;
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        q[i] = exp_exact(scaled_arg(srt[i].v, m, inv_t));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double S = 0.0;
        for (int i = 0; i < k; i++) {
            S += (double) q[i];
        }
        unsigned long long rng  = p.rng_in[row];
        const double       u    = (double) unit_from(xorshift_next(rng)) * S;
        double             a    = 0.0;
        int                pick = k - 1;
        for (int i = 0; i < k; i++) {
            a += (double) q[i];
            if (u < a) {
                pick = i;
                break;
            }
        }
        p.tokens[row] = srt[pick].idx;
        p.status[row] = ST_OK;
        if (p.rng_out) {
            p.rng_out[row] = rng;
        }
        if (p.kept_cap > 0) {
            p.kept_n[row] = k;
        }
        S_sh = S;
    }
    __syncthreads();
    if (p.kept_cap > 0) {
        for (int i = threadIdx.x; i < min(k, p.kept_cap); i += blockDim.x) {
            p.kept_idx[(size_t) row * p.kept_cap + i] = srt[i].idx;
            p.kept_val[(size_t) row * p.kept_cap + i] = __double2float_rn((double) q[i] / S_sh);
        }
    }
}

/* ------------------------------------------------------ speculative accept -- */

/* session.c:599-625, one thread per sequence. */
__global__ void accept_kernel(const AcceptParams p) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= p.n_seq) {
        return;
    }
    const int *fed = p.fed + (size_t) s * p.k;
    const int *vo  = p.verify_out + (size_t) s * p.k;
    int        a   = 0;
    while (a + 1 < p.k && vo[a] == fed[a + 1]) {
        a++;
    }
    int *em = p.emitted + (size_t) s * (p.k + 1);
    for (int i = 0; i <= a; i++) {
        em[i] = fed[i];
    }
    em[a + 1] = vo[a];
    for (int i = a + 2; i <= p.k; i++) {
        em[i] = -1;
    }
    p.accepted[s]  = a;
    p.n_emitted[s] = a + 2;
}

/* ------------------------------------------------------ batcher bookkeeping -- */

/* After a batcher call, one thread per participating session: the generator
 * word computed by the sampling kernel becomes the session's state, and the
 * tokens that were committed join its history ring. */
__global__ void post_step_kernel(const int *slot, int n_seq, int per_seq, int first, const int *tokens, const int *counts, int *hist, int hist_cap, int *hist_len,
                                 long long *hist_total, const unsigned long long *rng_tmp, unsigned long long *rng) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_seq) {
        return;
    }
    const int s = slot[i];
    rng[s]      = rng_tmp[s];
    if (tokens != nullptr && hist_cap > 0) {
        long long tot = hist_total[s];
        const int cnt = counts[i];
        for (int j = first; j < cnt; j++) {
            hist[(size_t) s * hist_cap + (size_t) (tot % hist_cap)] = tokens[(size_t) i * per_seq + j];
            tot++;
        }
        hist_total[s] = tot;
        hist_len[s]   = (int) (tot < hist_cap ? tot : hist_cap);
    }
}

/* ------------------------------------------------------------- dense helpers -- */

/* probs[row, :] = 0, then kept entries scattered: the post-filter probability vector. */
__global__ void scatter_kept_kernel(const int *kept_n, const int *kept_idx, const float *kept_val, int kept_cap, int V, int vocab_offset, float *dense) {
    const int row = blockIdx.x;
    const int n   = min(kept_n[row], kept_cap);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int id = kept_idx[(size_t) row * kept_cap + i] - vocab_offset;
        if (id >= 0 && id < V) {
            dense[(size_t) row * V + id] = kept_val[(size_t) row * kept_cap + i];
        }
    }
}

/* Dense softmax with temperature, p_i = (float)((double)expf((x_i - max) * inv_t) / sum)
 * (sampler.c:68-85 and :253-255). One CTA per row, three passes; an inspection
 * kernel, not part of the sampling hot path. */
__global__ void __launch_bounds__(1024) softmax_rows_kernel(const float *logits, long long row_stride, int V, const float *temperature, float *probs, double *sums) {
    const int    row = blockIdx.x;
    const float *x   = logits + (size_t) row * (size_t) row_stride;
    float       *y   = probs + (size_t) row * (size_t) V;
    const float  T   = temperature[row];
    const float  inv_t = T > 0.0f ? __fdiv_rn(1.0f, T) : 1.0f;
    __shared__ float  red_f[32];
    __shared__ double red_d[32];
    float m = -CUDART_INF_F;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        m = fmaxf(m, x[i]);
    }
    for (int o = 16; o > 0; o >>= 1) {
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    if ((threadIdx.x & 31) == 0) {
        red_f[threadIdx.x >> 5] = m;
    }
    __syncthreads();
    m = red_f[0];
    for (int w = 1; w < (int) (blockDim.x >> 5); w++) {
        m = fmaxf(m, red_f[w]);
    }
    double acc = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float e = expf(scaled_arg(x[i], m, inv_t));
        y[i]          = e;
        acc += (double) e;
    }
    acc = warp_sum_d(acc);
    if ((threadIdx.x & 31) == 0) {
        red_d[threadIdx.x >> 5] = acc;
    }
    __syncthreads();
    double S = 0.0;
    for (int w = 0; w < (int) (blockDim.x >> 5); w++) {
        S += red_d[w];
    }
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        y[i] = __double2float_rn((double) y[i] / S);
    }
    if (threadIdx.x == 0 && sums != nullptr) {
        sums[row] = S;
    }
}

/* ----------------------------------------------------------------- launchers -- */

size_t sample_rows_fixed_smem() { return sizeof(RowShared); }

/* Function attributes are per device and only ever raised. */
static cudaError_t ensure_attributes(size_t smem_bytes) {
    static int configured_smem[64] = {0};
    static bool cluster_ok[64]     = {false};
    int         dev                = 0;
    cudaError_t e                  = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    if (dev < 0 || dev >= 64) {
        return cudaErrorInvalidDevice;
    }
    if (!cluster_ok[dev]) {
        e = cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) {
            return e;
        }
        cluster_ok[dev] = true;
    }
    if ((int) smem_bytes > configured_smem[dev]) {
        e = cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) {
            return e;
        }
        configured_smem[dev] = (int) smem_bytes;
    }
    return cudaSuccess;
}

static void cluster_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, unsigned grid, int cluster, size_t smem_bytes, cudaStream_t stream) {
    cfg                      = {};
    cfg.gridDim              = dim3(grid, 1, 1);
    cfg.blockDim             = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes     = smem_bytes;
    cfg.stream               = stream;
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned) cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = 1;
}

cudaError_t launch_sample_rows(const SampleParams &p, int cluster, size_t smem_bytes, cudaStream_t stream) {
    cudaError_t e = ensure_attributes(smem_bytes);
    if (e != cudaSuccess) {
        return e;
    }
    cudaLaunchConfig_t  cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(cfg, attr, (unsigned) (p.n_rows * cluster), cluster, smem_bytes, stream);
    return cudaLaunchKernelEx(&cfg, sample_rows_kernel, p);
}

/* How many clusters of this shape the device can keep resident (0 = shape not launchable). */
int sample_rows_max_clusters(int cluster, size_t smem_bytes) {
    if (ensure_attributes(smem_bytes) != cudaSuccess) {
        (void) cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t  cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(cfg, attr, (unsigned) cluster, cluster, smem_bytes, nullptr);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, sample_rows_kernel, &cfg) != cudaSuccess) {
        (void) cudaGetLastError();
        return 0;
    }
    return n;
}

cudaError_t launch_merge_sample(const MergeParams &p, cudaStream_t stream) {
    const size_t cap  = (size_t) p.n_shards * (size_t) p.k_stride;
    const size_t smem = cap * (2 * sizeof(Pair) + sizeof(float));
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(merge_sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) {
            return e;
        }
    }
    merge_sample_kernel<<<p.n_rows, 256, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_accept(const AcceptParams &p, cudaStream_t stream) {
    accept_kernel<<<(p.n_seq + 127) / 128, 128, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_post_step(const int *slot, int n_seq, int per_seq, int first, const int *tokens, const int *counts, int *hist, int hist_cap, int *hist_len, long long *hist_total,
                             const unsigned long long *rng_tmp, unsigned long long *rng, cudaStream_t stream) {
    post_step_kernel<<<(n_seq + 127) / 128, 128, 0, stream>>>(slot, n_seq, per_seq, first, tokens, counts, hist, hist_cap, hist_len, hist_total, rng_tmp, rng);
    return cudaGetLastError();
}

cudaError_t launch_scatter_kept(const int *kept_n, const int *kept_idx, const float *kept_val, int kept_cap, int n_rows, int V, int vocab_offset, float *dense, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(dense, 0, (size_t) n_rows * (size_t) V * sizeof(float), stream);
    if (e != cudaSuccess) {
        return e;
    }
    scatter_kept_kernel<<<n_rows, 128, 0, stream>>>(kept_n, kept_idx, kept_val, kept_cap, V, vocab_offset, dense);
    return cudaGetLastError();
}

cudaError_t launch_softmax_rows(const float *logits, long long row_stride, int n_rows, int V, const float *temperature, float *probs, double *sums, cudaStream_t stream) {
    softmax_rows_kernel<<<n_rows, 1024, 0, stream>>>(logits, row_stride, V, temperature, probs, sums);
    return cudaGetLastError();
}

} /* namespace gb */

/*
 * sampler_aux.cu — the small kernels around the streaming sampler: merge of
 * vocabulary-shard candidates, the speculative prefix-accept rule, batcher
 * bookkeeping, and the dense inspection outputs.
 */
#include "sampler_device.cuh"

namespace gb {

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
    constexpr int kFlatShards = 64;
    __shared__ int s_off[kFlatShards + 1]; /* where each shard's list starts in ml (up to kFlatShards shards) */
    if (p.n_shards <= kFlatShards) {
        /* counts first, all at once; then every entry of every list in one flat loop: two round trips to memory
         * for the whole row instead of two per shard */
        if (threadIdx.x < p.n_shards) {
            s_off[threadIdx.x + 1] = min(p.cand_n[(size_t) threadIdx.x * p.n_rows + row], p.k_stride);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            s_off[0] = 0;
            for (int s = 0; s < p.n_shards; s++) {
                s_off[s + 1] += s_off[s];
            }
            n_total = s_off[p.n_shards];
        }
        __syncthreads();
        const int all = n_total;
        for (int j = threadIdx.x; j < all; j += blockDim.x) {
            int sh = 0;
            while (j >= s_off[sh + 1]) {
                sh++;
            }
            const size_t at = ((size_t) sh * p.n_rows + row) * (size_t) p.k_stride + (size_t) (j - s_off[sh]);
            ml[j].v         = p.cand_val[at];
            ml[j].idx       = p.cand_gid[at];
        }
        __syncthreads();
    } else {
        /* every thread walks the shards' counts itself: no meeting per shard */
        int lo = 0;
        for (int s = 0; s < p.n_shards; s++) {
            const int    nc  = min(p.cand_n[(size_t) s * p.n_rows + row], p.k_stride);
            const size_t off = ((size_t) s * p.n_rows + row) * (size_t) p.k_stride;
            for (int i = threadIdx.x; i < nc; i += blockDim.x) {
                ml[lo + i].v   = p.cand_val[off + i];
                ml[lo + i].idx = p.cand_gid[off + i];
            }
            lo += nc;
        }
        if (threadIdx.x == 0) {
            n_total = lo;
        }
        __syncthreads();
    }
    /* The key of the row's k-th largest candidate, by a radix select over the merged list (one byte of the ordered
     * key per step, counts in shared memory); what lies below it is dropped before the ordering, which ranks every
     * entry against all others (with eight shards of fifty: 400 x 400 comparisons against about 50 x 50). */
    {
        const int kk = min(min(max(p.top_k[row], 1), kTopKClamp), n_total);
        __shared__ int      hist[256];
        __shared__ unsigned pre_key;
        __shared__ int      need_sh, n_keep;
        if (threadIdx.x == 0) {
            pre_key = 0u;
            need_sh = kk;
            n_keep  = 0;
        }
        const int all = n_total;
        for (int level = 3; level >= 0 && all > kk; level--) {
            const int shift = 8 * level;
            hist[threadIdx.x & 255] = 0; /* blockDim.x == 256 */
            __syncthreads();
            const unsigned pre = pre_key;
            for (int t = threadIdx.x; t < all; t += blockDim.x) {
                const unsigned key = order_key(ml[t].v + 0.0f);
                if (level == 3 || (key >> (shift + 8)) == (pre >> (shift + 8))) {
                    atomicAdd(&hist[(key >> shift) & 255u], 1);
                }
            }
            __syncthreads();
            if (threadIdx.x < 32) { /* lane l owns the byte values 255 - 8 l down to 248 - 8 l: from the top */
                const int lane = threadIdx.x, need = need_sh;
                int       c8[8], mine = 0;
#pragma unroll
                for (int q8 = 0; q8 < 8; q8++) {
                    c8[q8] = hist[255 - (8 * lane + q8)];
                    mine += c8[q8];
                }
                int incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) {
                        incl += up;
                    }
                }
                const unsigned ball = __ballot_sync(0xffffffffu, incl >= need);
                if (ball != 0u && lane == __ffs(ball) - 1) {
                    int run = incl - mine;
                    for (int q8 = 0; q8 < 8; q8++) {
                        if (run + c8[q8] >= need) {
                            pre_key = pre | ((unsigned) (255 - (8 * lane + q8)) << shift);
                            need_sh = need - run;
                            break;
                        }
                        run += c8[q8];
                    }
                }
            }
            __syncthreads();
        }
        if (all > kk) {
            const unsigned tk = pre_key;
            for (int t0 = 0; t0 < all; t0 += blockDim.x) { /* compact into srt, then back */
                const int  t    = t0 + threadIdx.x;
                const bool keep = t < all && order_key(ml[t].v + 0.0f) >= tk;
                if (keep) {
                    srt[atomicAdd(&n_keep, 1)] = ml[t];
                }
            }
            __syncthreads();
            const int nk = n_keep;
            for (int t = threadIdx.x; t < nk; t += blockDim.x) {
                ml[t] = srt[t];
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                n_total = nk;
            }
            __syncthreads();
        }
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
        /* sampler.c:90-102: the sum and the walk in the reference's order, eight weights per step so that their
         * loads overlap */
        double S = 0.0;
        for (int i0 = 0; i0 < k; i0 += 8) {
            float w8[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                w8[j] = i0 + j < k ? q[i0 + j] : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                S += (double) w8[j];
            }
        }
        unsigned long long rng  = p.rng_in[row];
        const double       u    = (double) unit_from(xorshift_next(rng)) * S;
        double             a    = 0.0;
        int                pick = k - 1;
        for (int i0 = 0; i0 < k; i0 += 8) {
            float w8[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                w8[j] = i0 + j < k ? q[i0 + j] : 0.0f;
            }
            double pre[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                a += (double) w8[j];
                pre[j] = a;
            }
            int first = 8;
#pragma unroll
            for (int j = 7; j >= 0; j--) {
                if (u < pre[j] && i0 + j < k) {
                    first = j;
                }
            }
            if (first < 8) {
                pick = i0 + first;
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

/* ---------------------------------------------------------- n-gram drafter -- */

/*
 * propose_drafts_ngram of session.c:437-513, one thread block per sequence. The context is the sequence's
 * history plus the seed (the token its model predicts next). For L = min(max_suffix, 8) down to 1 the last L
 * context tokens are looked for at every earlier place p of the history; a place counts if something follows
 * it inside the history. The reference walks the places newest first, keeps the one with the most following
 * tokens (capped at k_max - 1) and the newer one on ties: since the capped number can only fall as p grows,
 * that is the largest (follow, p) pair, which is what the threads reduce with one 64-bit maximum. The first L
 * with a match ends the search. drafts[b][0] = seed, [1..] the tokens that followed; n_drafts[b] their number;
 * match_L[b] = L or 0. Below min_L (the lazy gate of session.c:583-591) the sequence is told to decode one
 * token the plain way: n_drafts[b] = 1, match_L stays what was found.
 *
 * The history of sequence b is hist[seq * stride + ((base[seq] + i) % stride)], i < len: a ring when base is
 * given, a flat row when it is null. skip_last[b] = 1 leaves the newest entry out (the seed itself, when the
 * sampler already appended it).
 */
constexpr int kDraftThreads = 128;
__global__ void __launch_bounds__(kDraftThreads) draft_ngram_kernel(const int *slot, const int *hist, long long stride, const int *hist_len, const long long *hist_total,
                                                                     const int *seeds, const int *skip_last, int k_max, int max_suffix, int min_L, int out_stride,
                                                                     int *drafts, int *n_drafts, int *match_L) {
    const int       b    = (int) blockIdx.x;
    const int       seq  = slot ? slot[b] : b;
    const int       full = hist_len[seq];
    const int       len  = max(0, full - (skip_last ? skip_last[b] : 0));
    const long long base = hist_total ? hist_total[seq] - (long long) full : 0ll;
    const int      *row  = hist + (size_t) seq * (size_t) stride;
    const int       seed = seeds[seq];
    auto            H    = [&](int i) { return row[(size_t) ((base + (long long) i) % stride)]; };
    __shared__ unsigned long long best;
    int *out = drafts + (size_t) b * (size_t) out_stride;
    if (threadIdx.x == 0) {
        out[0]     = seed;
        n_drafts[b] = 1;
        match_L[b]  = 0;
    }
    if (k_max <= 1 || len == 0) {
        return;
    }
    const int want = k_max - 1;
    for (int L = min(max_suffix, 8); L >= 1; L--) {
        if (L - 1 > len) {
            continue;
        }
        const int tail = len - (L - 1); /* the context's history part starts here; also the number of places */
        __syncthreads();
        if (threadIdx.x == 0) {
            best = 0ull;
        }
        __syncthreads();
        unsigned long long mine = 0ull;
        for (int p = (int) threadIdx.x; p < tail; p += kDraftThreads) {
            if (p + L >= len || H(p + L - 1) != seed) {
                continue;
            }
            bool ok = true;
            for (int i = 0; i + 1 < L && ok; i++) {
                ok = H(p + i) == H(tail + i);
            }
            if (ok) {
                const int follow = min(len - (p + L), want);
                mine             = max(mine, ((unsigned long long) follow << 32) | (unsigned long long) (unsigned) (p + 1));
            }
        }
        if (mine != 0ull) {
            atomicMax(&best, mine);
        }
        __syncthreads();
        const unsigned long long got = best;
        if (got != 0ull) {
            const int follow = (int) (got >> 32), p = (int) (got & 0xffffffffull) - 1;
            for (int i = (int) threadIdx.x; i < follow; i += kDraftThreads) {
                out[1 + i] = H(p + L + i);
            }
            if (threadIdx.x == 0) {
                match_L[b]  = L;
                n_drafts[b] = (1 + follow > 1 && L >= min_L) ? 1 + follow : 1;
            }
            return;
        }
    }
}

cudaError_t launch_draft_ngram(const int *slot, int n_seq, const int *hist, long long stride, const int *hist_len, const long long *hist_total, const int *seeds, const int *skip_last,
                               int k_max, int max_suffix, int min_L, int out_stride, int *drafts, int *n_drafts, int *match_L, cudaStream_t stream) {
    draft_ngram_kernel<<<n_seq, kDraftThreads, 0, stream>>>(slot, hist, stride, hist_len, hist_total, seeds, skip_last, k_max, max_suffix, min_L, out_stride, drafts, n_drafts, match_L);
    return cudaGetLastError();
}

/* The output head's soft cap on one dense row, in place: what peek_logits hands to value consumers
 * (arch.c:185-195; the expression of head.c:154). */
__global__ void softcap_row_kernel(float *row, int n, float c) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        row[i] = __fmul_rn(tanhf(__fdiv_rn(row[i], c)), c);
    }
}

cudaError_t launch_softcap_row(float *row, int n, float c, cudaStream_t stream) {
    softcap_row_kernel<<<(n + 1023) / 1024, 256, 0, stream>>>(row, n, c);
    return cudaGetLastError();
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

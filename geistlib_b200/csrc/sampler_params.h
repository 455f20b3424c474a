/*
 * Launch parameters shared by the sampling kernels and their host launchers.
 * Device pointers only; one struct is passed by value (__grid_constant__).
 */
#pragma once
#include <stdint.h>

namespace gb {

#ifndef GB_WORK_WARPS
#define GB_WORK_WARPS 14
#endif
#ifndef GB_FIN_WARPS
#define GB_FIN_WARPS 4
#endif
constexpr int kWorkWarps    = GB_WORK_WARPS;  /* warps that stream slices */
constexpr int kWorkThreads  = kWorkWarps * 32;
constexpr int kFinWarps     = GB_FIN_WARPS;   /* warps that finish completed rows */
constexpr int kFinThreads   = kFinWarps * 32;
constexpr int kQueue        = 32;             /* finished slices waiting for the publisher warp */
constexpr int kThreads      = kWorkThreads + 64 + kFinThreads; /* workers, loader warp, publisher warp, finishers: 640 */
constexpr int kWarps        = 32;             /* room for per-warp values in the slice record */
constexpr int kSliceMax     = 14336;          /* floats of one row slice: at most 8 float4 per worker thread */
static_assert(kSliceMax <= 32 * kWorkThreads, "a worker thread holds at most 8 float4 of a slice");
constexpr int kTopKClamp    = 8192;           /* sampler.c:212-215 */
constexpr int kFastKMax     = 256;            /* largest k served by the threshold fast path */
#ifndef GB_NUCLEUS_PROBE
#define GB_NUCLEUS_PROBE 32
#endif
constexpr int kNucleusProbe = GB_NUCLEUS_PROBE; /* entries the top-p fast path looks at */
constexpr int kMaxSlices    = 1024;           /* slices per row the finisher can merge */
constexpr int kMaxStages    = 4;              /* depth of the bulk-copy ring */
constexpr int kFinBitmapWords = 32;           /* finisher: one bit per entry of a crossing segment (at most 1024) */
constexpr int kHistBins     = 256;            /* value histogram of the finisher's select */

/* status word, one per row (bit set) */
enum : int {
    ST_OK            = 0,
    ST_LOAD_TIMEOUT  = 1 << 0, /* a bulk copy did not signal in time; row result is invalid */
    ST_SLOW_PATH     = 1 << 1, /* informational: the multi-pass path served this row */
    ST_HIST_OVERFLOW = 1 << 2, /* more distinct history ids than the launch reserved */
    ST_KEPT_PARTIAL  = 1 << 3, /* kept-set list not materialised (only kept_n is valid) */
    ST_INTERNAL      = 1 << 4, /* an invariant of the select failed; row result is invalid */
};

enum : unsigned {
    F_SELECT_ONLY = 1u << 0, /* vocabulary shard: emit the row's best k (value, global id), no draw */
};

struct Pair {
    float v;
    int   idx;
};

/* What one CTA leaves behind for one (row, slice) work item. */
struct __align__(16) SliceRec {
    float  max;         /* slice maximum after penalties */
    int    arg;         /* first global id of that maximum */
    int    n_cand;      /* candidates this slice found (may exceed the reserved room) */
    int    st;          /* status bits raised while processing the slice */
    double bulk;        /* top-p: sum of expf((x - max) * inv_t) over the non-candidates */
    double pad;
    double seg[kWarps]; /* temperature: per-warp sums of expf((x - max) * inv_t), id order */
};

struct SampleParams {
    const float *logits;      /* [n_rows, V], row_stride floats apart */
    long long    row_stride;
    int          V;
    int          n_rows;
    int          rows_per_seq; /* rows that share one generator and one parameter set */
    int          vocab_offset; /* global id of column 0 (vocabulary shards) */

    const int *slot; /* optional [n_seq]: index into every per-sequence array below (null = identity) */

    const float *temperature; /* [n_seq] */
    const int   *top_k;       /* [n_seq] */
    const float *top_p;       /* [n_seq] */
    const float *rep;         /* [n_seq] or null */
    const float *freq;        /* [n_seq] or null */
    const float *pres;        /* [n_seq] or null */

    const int *hist;          /* [n_seq, hist_stride] or null */
    long long  hist_stride;
    const int *hist_len;      /* [n_seq] */
    const int *extra;         /* [n_seq, extra_stride] or null: tokens fed through a verify pass */
    long long  extra_stride;

    const unsigned long long *rng_in;  /* [n_seq] */
    unsigned long long       *rng_out; /* [n_seq]; may alias rng_in only when rows_per_seq == 1 */

    int   *tokens;     /* [n_rows] */
    int   *status;     /* [n_rows] */
    float *out_logits; /* optional [n_rows, V]: rows after penalties */

    int    kept_cap;  /* entries per row in the kept_* arrays (0 = off) */
    int   *kept_n;    /* [n_rows] */
    int   *kept_idx;  /* [n_rows, kept_cap] */
    float *kept_val;  /* [n_rows, kept_cap]: probability inside the kept set (or raw value for F_SELECT_ONLY) */

    /* launch shape */
    int      n_slices;     /* work items per row */
    int      slice;        /* floats per slice, multiple of 4, <= kSliceMax */
    int      stage_bytes;  /* bytes of one ring stage (multiple of 128, >= 4 * slice) */
    int      stages;       /* ring depth, 1..kMaxStages */
    /* rows with more than 128 ids: their distinct ids are prepared by a kernel of their own */
    int       id_slots;    /* slots of that kernel's id table (a power of two, at least twice the ids a row can bring); 0: no such rows */
    int       row_cap;     /* entries of one row's prepared list */
    int       bucket_cap;  /* n_slices + 1 rounded up to a multiple of 4 */
    unsigned *pre_list;    /* [n_rows][row_cap] (position in the slice) | (count << 14), grouped by slice */
    int      *pre_off;     /* [n_rows][n_slices + 1] where each slice's run starts */
    /* rows left to the multi-pass path: (row, first id of the maximum, maximum, status bits), per CTA */
    int4     *slow_list;   /* [grid][slow_cap] */
    int       slow_cap;    /* rows one CTA can complete */
    int       chained;     /* 1: launched as a programmatic dependent of the kernel before it; waits for it before any global access */
    int      hist_cap;     /* distinct-id entries reserved per slice */
    int      cand_cap;     /* candidates reserved per slice */
    int      fin_cap;      /* candidates the finisher can merge per row */
    int      aligned;      /* rows start on 16-byte boundaries: bulk copies allowed */
    unsigned flags;

    /* scratch in global memory (one lane of the context's scratch) */
    int       *row_counter; /* [n_rows] slices published per row; zero when the launch starts */
    int       *ready_rows;  /* [n_rows] grid-wide queue of completed rows: row + 1, 0 = empty */
    unsigned  *q_ctr;       /* {tickets reserved, tickets claimed}, zero when the launch starts */
    int       *clear_ptr;   /* the other copy of these control words, zeroed by this launch */
    int        clear_words;
    SliceRec  *recs;        /* [n_rows * n_slices] */
    Pair      *cands;       /* [n_rows * n_slices, cand_cap] */
    float     *gen_rows;    /* [grid, gen_stride]: a CTA's private copy of one row for the multi-pass path */
    long long  gen_stride;  /* floats */
    unsigned  *gen_bitmap;  /* [grid, gen_bitmap_words] */
    int        gen_bitmap_words;
    Pair      *gen_dlist;   /* [grid, gen_hist_cap] (id, original value) */
    int        gen_hist_cap;
};

struct MergeParams {
    const float *cand_val; /* [n_shards, n_rows, k] */
    const int   *cand_gid; /* [n_shards, n_rows, k] */
    const int   *cand_n;   /* [n_shards, n_rows] valid entries per list */
    int          n_shards;
    int          n_rows;
    int          k_stride; /* entries reserved per list */

    const float *temperature; /* [n_rows] */
    const int   *top_k;       /* [n_rows] */
    const unsigned long long *rng_in;
    unsigned long long       *rng_out;
    int   *tokens;
    int   *status;
    int    kept_cap;
    int   *kept_n;
    int   *kept_idx;
    float *kept_val;
};

struct AcceptParams {
    const int *fed;        /* [n_seq, k]: fed[0] pending token, fed[1..k) proposals */
    const int *verify_out; /* [n_seq, k] */
    int        n_seq;
    int        k;
    int       *accepted;   /* [n_seq] */
    int       *n_emitted;  /* [n_seq] */
    int       *emitted;    /* [n_seq, k+1] */
};

} /* namespace gb */

/*
 * Launch parameters shared by the sampling kernels and their host launchers.
 * Device pointers only; one struct is passed by value (__grid_constant__).
 */
#pragma once
#include <stdint.h>
#include <vector_types.h>

namespace gb {

constexpr int kWarps        = 8;              /* warps of one thread block; each streams its own share of every slice */
constexpr int kThreads      = kWarps * 32;
constexpr int kNV4          = 8;              /* float4 one thread holds of a slice */
constexpr int kSliceMax     = kThreads * kNV4 * 4; /* floats of one row slice: 8192 */
constexpr int kStages       = 2;              /* depth of each warp's bulk-copy ring */
constexpr int kWarpStageBytes = kSliceMax * 4 / kWarps; /* one warp's share of a slice: 4 KB */
constexpr int kCtasPerSm    = 2;              /* thread blocks the launch bounds ask for per SM */
constexpr int kTopKClamp    = 8192;           /* sampler.c:212-215 */
constexpr int kFastKMax     = 256;            /* largest k served by the threshold fast path */
#ifndef GB_NUCLEUS_PROBE
#define GB_NUCLEUS_PROBE 32
#endif
constexpr int kNucleusProbe = GB_NUCLEUS_PROBE; /* entries the top-p fast path looks at */
constexpr int kMaxSlices    = 1024;           /* slices per row */
constexpr int kMaxParts     = 64;             /* thread blocks a row may be spread over before the finisher gives the row to the multi-pass path */
constexpr int kFinBitmapWords = 32;           /* finisher: one bit per entry of a crossing segment (at most 1024) */
constexpr int kHistBins     = 256;            /* value histograms (threshold, select) */
constexpr int kGroupCapWarp = 160;            /* candidate groups (one float4 each) a warp can hold of one row part */
constexpr int kPartGroups   = kWarps * kGroupCapWarp; /* ... and a whole thread block: 1280 */
constexpr int kPartSlots    = kPartGroups + 2;        /* a part in global scratch: its record in the first two 16-byte slots, then its groups */
constexpr int kRowIds       = 256;            /* ids of a row (history + fed tokens) counted inside the stream kernel, one per thread */

/* status word, one per row (bit set) */
enum : int {
    ST_OK            = 0,
    ST_LOAD_TIMEOUT  = 1 << 0, /* a bulk copy did not signal in time; row result is invalid */
    ST_SLOW_PATH     = 1 << 1, /* informational: the multi-pass path served this row */
    ST_HIST_OVERFLOW = 1 << 2, /* more distinct history ids than the launch reserved */
    ST_KEPT_PARTIAL  = 1 << 3, /* kept-set list not materialised (only kept_n is valid) */
    ST_INTERNAL      = 1 << 4, /* an invariant of the select failed; row result is invalid */
    ST_RETRY         = 1 << 5, /* the small finishing kernel met a top-k row whose candidates did not fit its lists: not sampled, to be launched again without the hint */
};

enum : unsigned {
    F_SELECT_ONLY = 1u << 0, /* vocabulary shard: emit the row's best k (value, global id), no draw */
    F_FAST_ONLY   = 1u << 1, /* the caller vouches that every row is greedy or top-k <= kFastKMax: the small finishing kernel runs instead of the general one */
    F_INLINE_TOPK = 1u << 2, /* with F_FAST_ONLY, whole rows per thread block and no kept-set output: the stream kernel finishes top-k rows itself from its own candidate lists; no finishing kernel runs; what does not fit asks for ST_RETRY */
    F_GREEDY_ONLY = 1u << 3, /* the caller vouches that every row is greedy: the stream kernel writes the tokens itself (the thread block that streamed the whole row, or the last of its parts to arrive) and no finishing kernel runs */
};

struct Pair {
    float v;
    int   idx;
};

/* What one thread block leaves behind for its part of a row (a run of consecutive slices). */
struct __align__(16) PartRec {
    float  max;      /* maximum of the part after penalties */
    int    arg;      /* first global id of that maximum */
    int    n_groups; /* candidate groups this part found (more than kPartGroups: some were dropped) */
    int    st;       /* status bits raised while the part streamed */
    float  tau;      /* the part's final select threshold: a lower bound of the row's kq-th largest value */
    float  bulk_ref; /* top-p: the sum below is relative to this value ... */
    double bulk_sum; /* ... sum of expf((x - bulk_ref) * inv_t) over everything outside the candidate groups */
};

/* Temperature rows: one warp's share of one slice, ids in order. */
struct __align__(16) SegRec {
    float  ref;  /* maximum of the segment */
    float  pad;
    double sum;  /* sum of expf((x - ref) * inv_t) over the segment */
};

/* Which (row, slice) items a thread block of the stream kernel takes: always one contiguous run of the row-major
 * item list. The host picks the cheaper of two ways to cut the list (a part of a row costs a thread block
 * about as much as five slices):
 *   RUN_ITEMS  runs of equal length (q or q + 1 items, the first r blocks the longer ones); runs may begin and
 *              end inside a row;
 *   RUN_ROWS   whole rows (q or q + 1 rows per block), when there are at least as many rows as blocks or one
 *              block per row comes out cheaper;
 *   RUN_PARTS  every row cut into P runs of q or q + 1 slices, when there are fewer rows than blocks. */
enum RunMode { RUN_ITEMS = 0, RUN_ROWS = 1, RUN_PARTS = 2 };
struct RunMap {
    int mode;
    int q, r;
    int P; /* RUN_PARTS: thread blocks per row */
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
    const float *softcap;     /* [n_seq] or null: final-logit soft cap of the sequence's model (0 = none) */
    const unsigned *mask;     /* [n_seq, mask_stride] or null: bit i set = column i may be sampled */
    long long       mask_stride; /* 32-bit words per mask row */

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
    int      parts_max;    /* thread blocks one row can be spread over */
    RunMap   map;          /* how the items are dealt out to the stream kernel's thread blocks */
    /* rows with more than kRowIds ids: their distinct ids are prepared by a kernel of their own */
    int       id_slots;    /* slots of that kernel's id table (a power of two, at least twice the ids a row can bring); 0: no such rows */
    int       row_cap;     /* entries of one row's prepared list */
    int       bucket_cap;  /* n_slices + 1 rounded up to a multiple of 4 */
    unsigned *pre_list;    /* [n_rows][row_cap] (position in the slice) | (count << 14), grouped by slice */
    int      *pre_off;     /* [n_rows][n_slices + 1] where each slice's run starts */
    int      hist_cap;     /* distinct-id entries the finisher reserves for one walked segment */
    int      aligned;      /* rows start on 16-byte boundaries: bulk copies allowed */
    unsigned flags;

    /* scratch in global memory (one lane of the context's scratch) */
    int       *arrive;      /* [n_rows] greedy launches: how many parts of the row have published their record; zero between launches */
    int       *pool;        /* [pool_slots] 1: the row copy of this number is taken; zero between launches */
    int        pool_slots;
    float4    *grp_v;       /* [n_rows, parts_max, kPartSlots] per part: its PartRec (two slots), then its candidate groups: four consecutive values ... */
    int       *grp_b;       /* ... and the global id of the first */
    SegRec    *segs;        /* [n_rows, n_slices, kWarps] temperature rows */
    float     *gen_rows;    /* [pool_slots, gen_stride]: private copies of one row for the multi-pass path */
    long long  gen_stride;  /* floats */
    unsigned  *gen_bitmap;  /* [pool_slots, gen_bitmap_words] */
    int        gen_bitmap_words;
    Pair      *gen_dlist;   /* [pool_slots, gen_hist_cap] (id, original value) */
    Pair      *gen_list;    /* [pool_slots, gen_list_cap] (probability, id): the entries of one histogram bin, picked out of the row */
    int        gen_list_cap;
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

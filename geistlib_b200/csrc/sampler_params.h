/*
 * Launch parameters shared by the sampling kernels and their host launchers.
 * Device pointers only; one struct is passed by value (__grid_constant__).
 */
#pragma once
#include <stdint.h>

namespace gb {

constexpr int kThreads      = 512;            /* threads per CTA */
constexpr int kWarps        = kThreads / 32;  /* 16 */
constexpr int kMaxCluster   = 16;             /* CTAs that share one row */
constexpr int kLocalCand    = 128;            /* candidates one CTA may hand to the row's finisher */
constexpr int kGroupCap     = 512;            /* group maxima per row used for the select threshold */
constexpr int kTopKClamp    = 8192;           /* sampler.c:212-215 */
constexpr int kFastKMax     = 256;            /* largest k served by the threshold fast path */
constexpr int kNucleusProbe = 32;             /* candidates the top-p fast path asks the threshold for */
constexpr int kNucleusCap   = 64;             /* candidates the top-p fast path can hold */

/* status word, one per row (bit set) */
enum : int {
    ST_OK            = 0,
    ST_LOAD_TIMEOUT  = 1 << 0, /* bulk copy did not signal in time; row result is invalid */
    ST_SLOW_PATH     = 1 << 1, /* informational: the bisection path served this row */
    ST_HIST_OVERFLOW = 1 << 2, /* more distinct history ids in a slice than the launch reserved */
    ST_KEPT_PARTIAL  = 1 << 3, /* kept-set list not materialised (only kept_n is valid) */
    ST_INTERNAL      = 1 << 4, /* an invariant of the select failed; row result is invalid */
};

enum : unsigned {
    F_SELECT_ONLY = 1u << 0, /* vocabulary shard: emit the row's best k (value, global id), no draw */
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
    const int *extra;         /* [n_seq, extra_stride] or null: tokens fed before row r (r+1 of them) */
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

    int      slice;        /* floats per CTA, multiple of 4 */
    int      slice_bytes;  /* bytes reserved for the slice buffer (multiple of 128) */
    int      bitmap_words; /* 0 when no history is given */
    int      hist_cap;     /* distinct-id entries reserved per CTA */
    int      cand_cap;     /* candidate entries reserved per CTA (>= kLocalCand) */
    int      aligned;      /* rows start on 16-byte boundaries: bulk copies allowed */
    unsigned flags;
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

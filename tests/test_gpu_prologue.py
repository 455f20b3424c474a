"""GPU parity of what happens to a row before it is sampled — the final-logit soft cap
(head.c:145-159, :279-288), the mask of allowed columns — of the finishing hints, and one
penalty-free case per sampler mode straight against the reference's own sampler.c."""
import numpy as np
import pytest

import oracle
from geistlib_b200 import api
from helpers import gumbel_logits, histories, independent_states, normal_logits, rel_err, seq_states, to_dev
from test_gpu_parity import check_tokens, run_gpu

pytestmark = pytest.mark.gpu
CAP_RTOL = 1e-5  # device tanhf against the host's: both within a few ulp of the true value

needs_ref = pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built")


def cap_dev(n_seq, c):
    return to_dev(np.broadcast_to(np.asarray(c, np.float32), (n_seq,)))


def mask_words(allowed):
    """bool [rows, V] -> int32 words [rows, ceil(V / 32)], bit i of a row = column i allowed."""
    rows, V = allowed.shape
    W = (V + 31) // 32
    pad = np.zeros((rows, W * 32), bool)
    pad[:, :V] = allowed
    w = np.packbits(pad.reshape(rows, W, 32), axis=2, bitorder="little").view(np.uint32).reshape(rows, W)
    return np.ascontiguousarray(w.view(np.int32))


@needs_ref
@pytest.mark.parametrize("shape", ["c1", "c3"])
def test_softcap_logits_and_tokens(ctx, shape):
    """c = 30 on rows shaped like the single-row case (temperature 0.8, top-k 40) and like the
    nucleus case (Gumbel rows, top-p): capped logits within 1e-5 of the host's tanhf, tokens equal."""
    c = 30.0
    if shape == "c1":
        rows, V = 24, 128256
        x = normal_logits(rows, V, 12.0, 41)  # wide enough for the cap to bend the top of the row
        T, K, P = 0.8, 40, 0.95
        st = independent_states(oracle.port, 41, rows)
    else:
        rows, V = 24, 262144
        x = gumbel_logits(rows, V, 4.0, 43)
        T, K, P = 0.9, 0, 0.9
        st = seq_states(oracle.port, 43, rows)
    capped = oracle.ref.softcap(x, c)
    g = run_gpu(ctx, x, T, K, P, st, softcap=cap_dev(rows, c), want_logits=True)
    assert rel_err(g["logits"], capped) <= CAP_RTOL
    assert np.abs(g["logits"]).max() <= c
    o = oracle.ref.sample(capped, T, K, P, st)
    check_tokens(g, o)


def test_softcap_skipped_for_greedy_and_zero(ctx):
    """T == 0 rows skip the cap (head.c:145-149) and c == 0 means none: both bit-identical to no cap at all."""
    rows, V = 8, 50257
    x = normal_logits(rows, V, 20.0, 3)
    st = independent_states(oracle.port, 3, rows)
    T = np.array([0.0, 0.7] * 4, np.float32)
    caps = np.array([30.0, 0.0] * 4, np.float32)
    g = run_gpu(ctx, x, T, 40, 1.0, st, softcap=to_dev(caps), want_logits=True)
    assert np.array_equal(g["logits"].view(np.uint32), x.view(np.uint32))
    check_tokens(g, oracle.port.sample_batch(x, T, 40, 1.0, st))


def test_softcap_then_penalties_temperature_and_verify_rows(ctx):
    """The cap comes before the penalties; temperature rows re-read a segment of the row in the finisher,
    and the rows of one sequence share its cap."""
    S, R, V, H = 6, 3, 32000, 48
    x = normal_logits(S * R, V, 9.0, 77)
    h = histories(S, H, V, 78)
    st = independent_states(oracle.port, 77, S)
    c = 25.0
    g = run_gpu(ctx, x, 1.0, 0, 1.0, st, rows_per_seq=R, softcap=cap_dev(S, c), rep=1.2, history=h, want_logits=True)
    capped = oracle.port.softcap(x, c)
    o = oracle.port.sample_batch(capped, 1.0, 0, 1.0, st, rows_per_seq=R, rep=1.2, hist=h, want_logits=True)
    assert rel_err(g["logits"], o["logits"]) <= CAP_RTOL
    check_tokens(g, o)


def test_softcap_wide_nucleus_path(ctx):
    """Rows whose nucleus is too wide for one pass take the multi-pass path, which caps its own copy of the row."""
    rows, V = 4, 40000
    x = normal_logits(rows, V, 2.0, 9)
    st = independent_states(oracle.port, 9, rows)
    g = run_gpu(ctx, x, 1.0, 0, 0.95, st, softcap=cap_dev(rows, 30.0))
    assert (g["status"] & api.ROW_SLOW_PATH).any(), "expected the multi-pass path"
    o = oracle.port.sample_batch(oracle.port.softcap(x, 30.0), 1.0, 0, 0.95, st)
    check_tokens(g, o)


@pytest.mark.parametrize("mode", ["greedy", "topk", "topp", "temp"])
def test_logit_mask(ctx, mode):
    """Masked columns read as -inf: the sampled ids are those of the CPU sampler on rows with -inf written in."""
    rows, V = 12, 50257
    x = normal_logits(rows, V, 2.5, 500)
    rng = np.random.default_rng(501)
    allowed = rng.random((rows, V)) < 0.3
    allowed[0, :] = False
    allowed[0, 4097] = True          # a single allowed column
    allowed[1, :] = True             # nothing masked
    allowed[2, x[2].argmax()] = False  # the winner is masked
    T, K, P = {"greedy": (0.0, 0, 1.0), "topk": (0.8, 40, 1.0), "topp": (0.8, 0, 0.6), "temp": (1.0, 0, 1.0)}[mode]
    st = independent_states(oracle.port, 500, rows)
    g = run_gpu(ctx, x, T, K, P, st, logit_mask=to_dev(mask_words(allowed)), want_logits=True)
    xm = np.where(allowed, x, -np.inf).astype(np.float32)
    assert np.array_equal(g["logits"].view(np.uint32), xm.view(np.uint32))
    check_tokens(g, oracle.port.sample_batch(xm, T, K, P, st))
    assert allowed[np.arange(rows), g["tokens"]].all()
    assert g["tokens"][0] == 4097


def test_logit_mask_with_softcap_and_penalties(ctx):
    rows, V, H = 8, 128256, 64
    x = normal_logits(rows, V, 10.0, 600)
    h = histories(rows, H, V, 601)
    allowed = np.random.default_rng(602).random((rows, V)) < 0.5
    st = independent_states(oracle.port, 600, rows)
    g = run_gpu(ctx, x, 0.8, 40, 1.0, st, softcap=cap_dev(rows, 30.0), logit_mask=to_dev(mask_words(allowed)), rep=1.1, history=h)
    xm = np.where(allowed, oracle.port.softcap(x, 30.0), -np.inf).astype(np.float32)
    check_tokens(g, oracle.port.sample_batch(xm, 0.8, 40, 1.0, st, rep=1.1, hist=h))


def test_logit_mask_stride_too_short(ctx):
    rows, V = 2, 1000
    x = to_dev(normal_logits(rows, V, 1.0, 1))
    import torch
    m = torch.zeros(rows, 8, dtype=torch.int32, device="cuda")  # 256 bits < V
    dT, dK, dP = to_dev(np.zeros(rows, np.float32)), to_dev(np.zeros(rows, np.int32)), to_dev(np.ones(rows, np.float32))
    with pytest.raises(api.GeistError, match="GEIST_E_INVALID_ARG"):
        ctx.sample_batch(x, dT, dK, dP, to_dev(np.ones(rows, np.int64)), logit_mask=m)


# ------------------------------------------------------------- finishing hints --

def test_finish_hint_same_tokens(ctx):
    """A correct hint changes which kernels run, never a token."""
    rows, V = 64, 128256
    x = normal_logits(rows, V, 2.5, 900)
    st = independent_states(oracle.port, 900, rows)
    T = np.where(np.arange(rows) % 2 == 0, 0.0, 0.8).astype(np.float32)
    auto = run_gpu(ctx, x, T, 40, 1.0, st)
    fast = run_gpu(ctx, x, T, 40, 1.0, st, finish_hint=api.FINISH_GREEDY_TOPK)
    gen = run_gpu(ctx, x, T, 40, 1.0, st, finish_hint=api.FINISH_GENERAL)
    check_tokens(fast, auto)
    check_tokens(gen, auto)
    check_tokens(auto, oracle.port.sample_batch(x, T, 40, 1.0, st))
    # rows of the other modes through the general kernel alone
    Tm = np.full(rows, 0.9, np.float32)
    Pm = np.where(np.arange(rows) % 2 == 0, 1.0, 0.5).astype(np.float32)
    check_tokens(run_gpu(ctx, x, Tm, 0, Pm, st, finish_hint=api.FINISH_GENERAL), oracle.port.sample_batch(x, Tm, 0, Pm, st))


@pytest.mark.parametrize("rows,V,R", [(256, 5000, 1), (200, 40000, 1), (64, 128256, 1), (300, 9000, 1), (240, 3000, 3)])
def test_finish_hint_greedy(ctx, rows, V, R):
    """All rows greedy and the caller says so: whole-row launches write the tokens from the stream kernel alone
    (no finishing kernel), split-row launches merge as usual; ids, status and generator words as without the hint."""
    x = normal_logits(rows, V, 3.0, 77 + rows)
    x[3, :] = 1.5           # all equal: lowest index
    x[5, V // 3:] = x[5].max() + 2.0
    S = rows // R
    st = independent_states(oracle.port, 5, S)
    h = histories(S, 40, V, 6)
    g = run_gpu(ctx, x, 0.0, 0, 1.0, st, rows_per_seq=R, finish_hint=api.FINISH_GREEDY, freq=0.4, history=h)
    o = oracle.port.sample_batch(x, 0.0, 0, 1.0, st, rows_per_seq=R, freq=0.4, hist=h)
    check_tokens(g, o)
    assert np.array_equal(g["rng_state"], st), "greedy rows draw nothing"


def test_finish_hint_greedy_wrong_is_loud(ctx):
    from helpers import u64_to_dev
    rows, V = 256, 4000
    x = normal_logits(rows, V, 3.0, 9)
    T = np.zeros(rows, np.float32)
    T[17] = 0.7
    dT, dK, dP = to_dev(T), to_dev(np.zeros(rows, np.int32)), to_dev(np.ones(rows, np.float32))
    out = ctx.sample_batch(to_dev(x), dT, dK, dP, u64_to_dev(independent_states(oracle.port, 1, rows)), finish_hint=api.FINISH_GREEDY)
    status, tok = out["status"].cpu().numpy(), out["tokens"].cpu().numpy()
    assert status[17] & api.ROW_INTERNAL and tok[17] == -1
    ok = np.arange(rows) != 17
    assert (status[ok] & api.ROW_INVALID == 0).all() and np.array_equal(tok[ok], x[ok].argmax(axis=1))


def test_finish_hint_wrong_is_loud(ctx):
    """GREEDY_TOPK with a temperature row in the batch: that row reports ROW_INTERNAL and token -1, the others are sampled."""
    import torch
    rows, V = 8, 32000
    x = normal_logits(rows, V, 2.5, 901)
    st = independent_states(oracle.port, 901, rows)
    T = np.full(rows, 0.8, np.float32)
    K = np.full(rows, 40, np.int32)
    K[3] = 0  # plain temperature sampling
    dT, dK, dP = to_dev(T), to_dev(K), to_dev(np.ones(rows, np.float32))
    from helpers import u64_to_dev
    out = ctx.sample_batch(to_dev(x), dT, dK, dP, u64_to_dev(st), finish_hint=api.FINISH_GREEDY_TOPK)
    status, tok = out["status"].cpu().numpy(), out["tokens"].cpu().numpy()
    assert status[3] & api.ROW_INTERNAL and tok[3] == -1
    ok = np.arange(rows) != 3
    assert (status[ok] & api.ROW_INVALID == 0).all()
    o = oracle.port.sample_batch(x, T, K, 1.0, st)
    assert np.array_equal(tok[ok], o["tokens"][ok])
    with pytest.raises(api.GeistError, match="GEIST_E_INVALID_ARG"):
        ctx.sample_batch(to_dev(x), dT, dK, dP, u64_to_dev(st), finish_hint=9)


# ------------------------------------- every mode against the reference's own code --

@needs_ref
@pytest.mark.parametrize("mode,T,K,P", [("argmax", 0.0, 0, 1.0), ("top_k", 0.8, 40, 0.95), ("top_k_wide", 1.0, 300, 1.0),
                                        ("top_p", 0.8, 0, 0.9), ("temperature", 1.1, 0, 1.0)])
def test_mode_against_reference_sampler(ctx, mode, T, K, P):
    """No penalties, no extension in play: the CUDA path against src/engine/sampler.c itself (oracle/_ref)."""
    rows, V = 48, 128256
    x = gumbel_logits(rows, V, 3.0, 1000) if mode == "top_p" else normal_logits(rows, V, 2.5, 1000)
    x[:, :4] += 9.0
    st = seq_states(oracle.port, 1000, rows)
    g = run_gpu(ctx, x, T, K, P, st)
    check_tokens(g, oracle.ref.sample(x, T, K, P, st))


# ------------------------------------------------------ how the items are dealt out --

@pytest.mark.parametrize("V", [700, 9000, 20000])  # 1, 2 and 3 slices per row
def test_run_maps_over_row_counts(ctx, V):
    """Row counts on both sides of every switch between the three ways of cutting the item list (whole rows,
    rows cut into equal parts, equal runs of items), with each hint's weighting: the tokens never depend on it."""
    sm2 = 2 * 148
    counts = sorted({1, 2, 3, 37, 73, 74, 75, 147, 148, 149, 150, 200, 255, 256, 257, sm2 - 1, sm2, sm2 + 1, 300, 2 * sm2 - 1, 2 * sm2, 2 * sm2 + 1, 640})
    rows_max = max(counts)
    x = normal_logits(rows_max, V, 2.5, 4000 + V)
    x[:, :3] += 6.0
    st = independent_states(oracle.port, 4000, rows_max)
    h = histories(rows_max, 24, V, 4001)
    for mode, (T, K, P), hints in [("greedy", (0.0, 0, 1.0), (api.FINISH_AUTO, api.FINISH_GREEDY_TOPK, api.FINISH_GREEDY)),
                                   ("topk", (0.8, 40, 1.0), (api.FINISH_AUTO, api.FINISH_GREEDY_TOPK)),
                                   ("temp", (1.0, 0, 1.0), (api.FINISH_AUTO, api.FINISH_GENERAL))]:
        o = oracle.port.sample_batch(x, T, K, P, st, rep=1.1, hist=h)
        for n in counts:
            for hint in hints:
                g = run_gpu(ctx, x[:n], T, K, P, st[:n], rep=1.1, history=h[:n], finish_hint=hint)
                bad = np.nonzero(g["tokens"] != o["tokens"][:n])[0]
                assert bad.size == 0, (mode, n, hint, bad[:5])
                assert np.array_equal(g["rng_state"], o["rng_state"][:n]), (mode, n, hint)


def test_small_finisher_hands_back_rows_whose_candidates_overflow(ctx):
    """GREEDY_TOPK promises greedy / top-k rows, not easy ones. A top-k row with thousands of equal values at the
    top (more candidates than the small kernel's lists hold) comes back unsampled with ROW_RETRY; launched again
    without the hint it is sampled. The batcher does that second launch itself."""
    from helpers import u64_to_dev
    rows, V = 6, 128256
    x = normal_logits(rows, V, 2.5, 4242)
    x[0, 1000:9000] = 30.0          # 8000 ties at the top: the k kept are the lowest ids among them
    x[1, :] = 1.0                   # a flat row
    x[2, ::3] = x[2].max() + 1.0    # every third entry tied
    st = independent_states(oracle.port, 4242, rows)
    for K in (40, 200):
        o = oracle.port.sample_batch(x, 0.9, K, 1.0, st)
        dT, dK, dP = to_dev(np.full(rows, 0.9, np.float32)), to_dev(np.full(rows, K, np.int32)), to_dev(np.ones(rows, np.float32))
        out = ctx.sample_batch(to_dev(x), dT, dK, dP, u64_to_dev(st), finish_hint=api.FINISH_GREEDY_TOPK)
        status, tok = out["status"].cpu().numpy(), out["tokens"].cpu().numpy()
        assert (status[:3] & api.ROW_RETRY).all() and (tok[:3] == -1).all()
        assert (status[3:] & (api.ROW_RETRY | api.ROW_INVALID) == 0).all() and np.array_equal(tok[3:], o["tokens"][3:])
        check_tokens(run_gpu(ctx, x, 0.9, K, 1.0, st), o)  # the same rows without the hint
    bt = api.Batcher(ctx, V, 8)
    sess = [bt.open(temperature=0.9, top_k=40, top_p=1.0, seed=4242 + i) for i in range(rows)]  # all top-k: the batcher gives the hint
    got = bt.step(sess, to_dev(x))
    assert np.array_equal(got, oracle.port.sample_batch(x, 0.9, 40, 1.0, st)["tokens"])
    for i, s_ in enumerate(sess):
        assert bt.get_rng(s_) == oracle.port.rng_advance(int(st[i]), 1)
    bt.close()


def test_stream_kernel_finishes_whole_rows_itself(ctx):
    """GREEDY_TOPK on a launch that deals whole rows: no finishing kernel runs, the stream kernel's thread blocks
    finish greedy and top-k rows from their own lists. Same tokens and generator words as without the hint; rows
    whose candidates do not fit come back with ROW_RETRY."""
    from helpers import u64_to_dev
    rows, V = 200, 128256
    x = normal_logits(rows, V, 2.5, 777)
    x[:, :5] += 7.0
    x[3, 2000:9000] = 40.0   # thousands of ties at the top
    x[4, :] = 0.5            # flat
    st = independent_states(oracle.port, 777, rows)
    h = histories(rows, 64, V, 778)
    T = np.where(np.arange(rows) % 5 == 0, 0.0, 0.8).astype(np.float32)
    K = np.where(np.arange(rows) % 3 == 0, 200, 40).astype(np.int32)
    o = oracle.port.sample_batch(x, T, K, 1.0, st, rep=1.1, hist=h)
    assert api.grid(V, rows, 64)["thread_blocks"] == rows  # whole rows
    dT, dK, dP = to_dev(T), to_dev(K), to_dev(np.ones(rows, np.float32))
    out = ctx.sample_batch(to_dev(x), dT, dK, dP, u64_to_dev(st), rep=to_dev(np.full(rows, 1.1, np.float32)), history=to_dev(h),
                           history_len=to_dev(np.full(rows, 64, np.int32)), finish_hint=api.FINISH_GREEDY_TOPK)
    status, tok = out["status"].cpu().numpy(), out["tokens"].cpu().numpy()
    retry = (status & api.ROW_RETRY) != 0
    assert retry[3] and retry[4] and retry.sum() == 2 and (tok[retry] == -1).all()
    assert (status[~retry] & api.ROW_INVALID == 0).all()
    assert np.array_equal(tok[~retry], o["tokens"][~retry])
    from helpers import u64_from_dev
    assert np.array_equal(u64_from_dev(out["rng_state"]), o["rng_state"])
    # verify rows (three per sequence) through the same path
    S, R = 66, 3
    xv = normal_logits(S * R, V, 2.5, 779)
    sv = independent_states(oracle.port, 779, S)
    g = run_gpu(ctx, xv, 0.9, 50, 1.0, sv, rows_per_seq=R, finish_hint=api.FINISH_GREEDY_TOPK)
    check_tokens(g, oracle.port.sample_batch(xv, 0.9, 50, 1.0, sv, rows_per_seq=R))

"""GPU parity: the CUDA path through the C ABI against the CPU checker on the
same seeded inputs. Token ids, kept-set ids and generator states must be
bit-exact; probabilities within 1e-5 relative (fp32)."""
import numpy as np
import pytest

import oracle
from helpers import (gumbel_logits, histories, independent_states, normal_logits, per_seq, rel_err, seq_states,
                     to_dev, u64_from_dev, u64_to_dev)

pytestmark = pytest.mark.gpu
PROB_RTOL = 1e-5
INVALID = 1 | 4 | 16


def run_gpu(ctx, logits, T, K, P, states, **kw):
    n_seq = logits.shape[0] // kw.get("rows_per_seq", 1)
    dT, dK, dP = per_seq(n_seq, T, K, P)
    dl = to_dev(logits)
    extra = {}
    for name in ("rep", "freq", "pres"):
        if kw.get(name) is not None:
            extra[name] = to_dev(np.broadcast_to(np.asarray(kw.pop(name), np.float32), (n_seq,)))
        else:
            kw.pop(name, None)
    if kw.get("history") is not None:
        h = kw.pop("history")
        hl = kw.pop("history_len", None)
        extra["history"] = to_dev(h)
        extra["history_len"] = to_dev(np.full(n_seq, h.shape[1], np.int32) if hl is None else np.asarray(hl, np.int32))
    if kw.get("fed") is not None:
        extra["fed"] = to_dev(kw.pop("fed"))
    out = ctx.sample_batch(dl, dT, dK, dP, u64_to_dev(states), **extra, **kw)
    res = {k: (v.cpu().numpy() if v is not None else None) for k, v in out.items() if not k.startswith("_")}
    res["rng_state"] = u64_from_dev(out["rng_state"])
    assert (res["status"] & INVALID == 0).all(), res["status"]
    return res


def check_tokens(g, o):
    bad = np.nonzero(g["tokens"] != o["tokens"])[0]
    assert bad.size == 0, f"{bad.size} of {g['tokens'].size} tokens differ, first rows {bad[:8]}: gpu {g['tokens'][bad[:8]]} cpu {o['tokens'][bad[:8]]}"
    assert (g["rng_state"] == o["rng_state"]).all()


@pytest.mark.parametrize("V", [1, 2, 3, 31, 32, 33, 127, 1023, 1024, 1025, 4099, 16384, 16385, 50257])
def test_greedy_edge_sizes(ctx, V):
    x = normal_logits(5, V, 3.0, 100 + V)
    x[1, :] = 0.25          # all equal: lowest index wins
    x[2, V // 2:] = x[2].max() + 1.0   # tie of the maximum
    x[3, :] = -np.inf       # sampler.c:52-62 keeps index 0
    st = independent_states(oracle.port, 5, 5)
    g = run_gpu(ctx, x, 0.0, 0, 1.0, st)
    o = oracle.port.sample_batch(x, 0.0, 0, 1.0, st)
    check_tokens(g, o)


def test_greedy_batched_with_penalties(ctx):
    """Batched greedy + frequency/presence penalties, 256-token histories (scaled-down rows)."""
    V, rows, H = 151936, 16, 256
    x = normal_logits(rows, V, 3.0, 7)
    h = histories(rows, H, V, 8)
    h[:, :32] = h[:, 32:64]  # repeated ids so that counts > 1 matter
    arg = x.argmax(axis=1)
    h[:, 0] = arg            # the unpenalised winner is in the history
    st = independent_states(oracle.port, 7, rows)
    g = run_gpu(ctx, x, 0.0, 0, 1.0, st, freq=0.2, pres=0.3, history=h, want_logits=True)
    o = oracle.port.sample_batch(x, 0.0, 0, 1.0, st, freq=0.2, pres=0.3, hist=h, want_logits=True)
    check_tokens(g, o)
    assert np.array_equal(g["logits"].view(np.uint32), o["logits"].view(np.uint32)), "post-penalty logits must be bit-equal"
    assert (g["tokens"] != arg).any()


@pytest.mark.parametrize("rep,freq,pres", [(1.1, 0.0, 0.0), (1.15, 0.2, 0.3), (0.0, 0.0, 0.0)])
def test_topk_with_repetition_penalty(ctx, rep, freq, pres):
    V, rows, H = 128256, 16, 64
    x = normal_logits(rows, V, 2.5, 1234)
    rng = np.random.default_rng(5)
    for r in range(rows):
        x[r, rng.integers(0, V, 8)] += 12.0
    h = histories(rows, H, V, 9)
    h[:, :8] = np.argsort(-x, axis=1)[:, :8]  # penalise the boosted ids
    hl = rng.integers(0, H + 1, rows).astype(np.int32)
    st = seq_states(oracle.port, 1234, rows)
    g = run_gpu(ctx, x, 0.8, 40, 0.95, st, rep=rep, freq=freq, pres=pres, history=h, history_len=hl, kept_cap=40, want_logits=True)
    o = oracle.port.sample_batch(x, 0.8, 40, 0.95, st, rep=rep, freq=freq, pres=pres, hist=h, hist_len=hl, detail_cap=40, want_logits=True)
    check_tokens(g, o)
    assert np.array_equal(g["logits"].view(np.uint32), o["logits"].view(np.uint32))
    assert np.array_equal(g["kept_n"], o["detail_n"])
    assert np.array_equal(g["kept_idx"], o["detail_idx"])
    assert rel_err(g["kept_prob"], o["detail_prob"]) <= PROB_RTOL


@pytest.mark.parametrize("V,k", [(128256, 40), (128256, 2), (128256, 50), (128256, 128), (128256, 256), (32000, 40), (5000, 40), (300, 40), (41, 40), (262144, 64)])
def test_topk_sizes(ctx, V, k):
    rows = 8
    x = normal_logits(rows, V, 2.5, 31 + V + k)
    st = independent_states(oracle.port, 77, rows)
    g = run_gpu(ctx, x, 0.7, k, 0.9, st, kept_cap=k)
    o = oracle.port.sample_batch(x, 0.7, k, 0.9, st, detail_cap=k)
    check_tokens(g, o)
    assert np.array_equal(g["kept_n"], o["detail_n"])
    full = (g["status"] & 8) == 0  # rows whose kept list was materialised (not the multi-pass path)
    if k <= 128:
        assert full.all(), "k <= 128 must be served by the single-pass path with its kept list"
    assert np.array_equal(g["kept_idx"][full], o["detail_idx"][full])
    assert rel_err(g["kept_prob"][full], o["detail_prob"][full]) <= PROB_RTOL


def test_topk_ties_and_slow_path(ctx):
    """Rows made of a few distinct values: the k-th entry sits inside a run of ties, which
    must resolve by ascending id; also k beyond the fast path."""
    V, rows = 20000, 6
    rng = np.random.default_rng(3)
    x = rng.integers(-3, 4, size=(rows, V)).astype(np.float32)
    x[0, :] = 0.0
    st = independent_states(oracle.port, 11, rows)
    for k in (3, 40, 1000, 9000):
        g = run_gpu(ctx, x, 1.0, k, 1.0, st)
        o = oracle.port.sample_batch(x, 1.0, k, 1.0, st)
        check_tokens(g, o)
    x2 = normal_logits(4, 128256, 2.5, 4)
    for k in (1000, 8192, 20000):
        g = run_gpu(ctx, x2, 0.9, k, 1.0, st[:4])
        o = oracle.port.sample_batch(x2, 0.9, k, 1.0, st[:4])
        check_tokens(g, o)


def test_topp_heavy_tail(ctx):
    """Gumbel*4 rows, per-row temperature and top_p: tiny nuclei (fast path)."""
    V, rows = 262144, 32
    x = gumbel_logits(rows, V, 4.0, 99)
    rng = np.random.default_rng(99)
    T = rng.uniform(0.5, 1.2, rows).astype(np.float32)
    P = rng.uniform(0.8, 0.98, rows).astype(np.float32)
    st = seq_states(oracle.port, 99, rows)
    g = run_gpu(ctx, x, T, 0, P, st, kept_cap=16)
    o = oracle.port.sample_batch(x, T, 0, P, st, detail_cap=16)
    check_tokens(g, o)
    assert np.array_equal(g["kept_n"], o["detail_n"])
    full = (g["status"] & 8) == 0
    assert full.any()
    assert np.array_equal(g["kept_idx"][full], o["detail_idx"][full])
    assert rel_err(g["kept_prob"][full], o["detail_prob"][full]) <= PROB_RTOL


@pytest.mark.parametrize("V,sigma,p", [(128256, 2.5, 0.95), (128256, 2.5, 0.5), (5000, 1.0, 0.9), (1000, 0.0, 0.9), (33, 2.0, 0.3)])
def test_topp_wide_nucleus(ctx, V, sigma, p):
    """Gaussian rows give nuclei of thousands of ids: the bisection path."""
    rows = 6
    x = normal_logits(rows, V, sigma, 17 + V)
    st = independent_states(oracle.port, 21, rows)
    g = run_gpu(ctx, x, 0.8, 0, p, st, kept_cap=8)
    o = oracle.port.sample_batch(x, 0.8, 0, p, st, detail_cap=8)
    check_tokens(g, o)
    assert np.array_equal(g["kept_n"], o["detail_n"])


@pytest.mark.parametrize("V", [5, 1000, 32000, 128256, 262144])
def test_temperature_only(ctx, V):
    rows = 16
    x = normal_logits(rows, V, 2.5, 5 + V)
    x[0, :] = 0.0  # uniform row: every id equally likely
    st = independent_states(oracle.port, 42, rows)
    T = np.linspace(0.3, 1.5, rows).astype(np.float32)
    g = run_gpu(ctx, x, T, 0, 1.0, st)
    o = oracle.port.sample_batch(x, T, 0, 1.0, st)
    check_tokens(g, o)
    # top_k >= V and top_p >= 1 also end in the temperature path (sampler.c:187-189, :241-243)
    g = run_gpu(ctx, x, T, V + 5, 1.0, st)
    check_tokens(g, o)


def test_softmax_probabilities(ctx):
    V, rows = 128256, 4
    x = normal_logits(rows, V, 2.5, 2)
    T = np.array([0.5, 0.8, 1.0, 1.3], np.float32)
    probs, sums = ctx.softmax(to_dev(x), to_dev(T))
    probs = probs.cpu().numpy()
    for r in range(rows):
        ref, s = oracle.port.softmax(x[r], float(T[r]))
        big = ref > 1e-30
        assert rel_err(probs[r][big], ref[big]) <= PROB_RTOL
        assert abs(float(sums[r]) - s) / s < 1e-6


def test_verify_rows_share_one_generator(ctx):
    """K+1 rows per sequence sampled in order with one generator, then the prefix-accept rule."""
    V, S, K = 128256, 6, 6
    R = K + 1
    rng = np.random.default_rng(2024)
    draft = normal_logits(S * K, V, 2.5, 2024).reshape(S, K, V)
    target = np.empty((S, R, V), np.float32)
    target[:, :K] = draft + normal_logits(S * K, V, 0.5, 2025).reshape(S, K, V)
    target[:, K] = normal_logits(S, V, 2.5, 2026)
    target = target.reshape(S * R, V)
    for (T, k, p) in [(0.0, 0, 1.0), (1.0, 0, 1.0), (0.8, 40, 1.0)]:
        st = independent_states(oracle.port, 2024, S)
        dst = independent_states(oracle.port, 3024, S)
        drafts = oracle.port.sample_batch(draft.reshape(S * K, V), T, k, p, dst, rows_per_seq=K)["tokens"].reshape(S, K)
        fed = np.concatenate([rng.integers(0, V, (S, 1)).astype(np.int32), drafts], axis=1)
        # make some proposals certainly right: replace them by what the target will say
        o = oracle.port.sample_batch(target, T, k, p, st, rows_per_seq=R)
        vo = o["tokens"].reshape(S, R)
        fed[0, 1:] = vo[0, :K]        # everything accepted
        fed[1, 1:3] = vo[1, :2]       # at least two accepted
        g = run_gpu(ctx, target, T, k, p, st, rows_per_seq=R)
        check_tokens(g, o)
        acc, nem, em = ctx.accept_batch(to_dev(fed), to_dev(g["tokens"].reshape(S, R)))
        acc, nem, em = acc.cpu().numpy(), nem.cpu().numpy(), em.cpu().numpy()
        for s in range(S):
            a, emitted = oracle.port.spec_accept(fed[s], vo[s])
            assert acc[s] == a and nem[s] == a + 2
            assert np.array_equal(em[s, :a + 2], emitted)
        assert acc[0] == K and acc[1] >= 2


def test_verify_penalties_count_fed_tokens(ctx):
    V, S, R, H = 32000, 4, 5, 32
    x = normal_logits(S * R, V, 2.5, 8)
    h = histories(S, H, V, 9)
    fed = np.argsort(-x.reshape(S, R, V)[:, -1], axis=1)[:, :R].astype(np.int32)  # ids that matter in the last row
    st = independent_states(oracle.port, 1, S)
    g = run_gpu(ctx, x, 0.0, 0, 1.0, st, rows_per_seq=R, rep=1.3, freq=0.5, pres=0.4, history=h, fed=fed, want_logits=True)
    o = oracle.port.sample_batch(x, 0.0, 0, 1.0, st, rows_per_seq=R, rep=1.3, freq=0.5, pres=0.4, hist=h, extra=fed, want_logits=True)
    check_tokens(g, o)
    assert np.array_equal(g["logits"].view(np.uint32), o["logits"].view(np.uint32))


def test_unaligned_rows(ctx):
    """Rows that do not start on 16-byte boundaries take the plain-load path."""
    import torch
    V, rows = 10007, 8
    x = normal_logits(rows, V, 2.5, 6)
    buf = torch.zeros(rows * (V + 3) + 1, dtype=torch.float32, device="cuda")
    view = buf[1:1 + rows * (V + 3)].view(rows, V + 3)[:, :V]
    view.copy_(torch.from_numpy(x))
    st = independent_states(oracle.port, 3, rows)
    dT, dK, dP = per_seq(rows, 0.8, 40, 1.0)
    out = ctx.sample_batch(view, dT, dK, dP, u64_to_dev(st))
    o = oracle.port.sample_batch(x, 0.8, 40, 1.0, st)
    assert np.array_equal(out["tokens"].cpu().numpy(), o["tokens"])


def test_mixed_modes_in_one_launch(ctx):
    V, rows = 128256, 12
    x = normal_logits(rows, V, 2.5, 12)
    x[:, :4] += 14.0
    T = np.array([0.0, 0.8, 0.8, 1.0] * 3, np.float32)
    K = np.array([0, 40, 0, 0] * 3, np.int32)
    P = np.array([1.0, 1.0, 0.9, 1.0] * 3, np.float32)
    st = independent_states(oracle.port, 8, rows)
    g = run_gpu(ctx, x, T, K, P, st)
    o = oracle.port.sample_batch(x, T, K, P, st)
    check_tokens(g, o)


def test_mixed_modes_large_batch_with_penalties(ctx):
    """Several hundred rows, all four modes interleaved row by row, two rows per generator, histories
    of different lengths: every CTA meets rows of every kind back to back."""
    V, S, R, H = 32000, 150, 2, 48
    rows = S * R
    x = normal_logits(rows, V, 2.5, 4242)
    x[:, :6] += 11.0
    rng = np.random.default_rng(4242)
    modes = [(0.0, 0, 1.0), (0.8, 40, 1.0), (0.9, 0, 0.9), (1.1, 0, 1.0), (0.7, 100, 1.0), (0.8, 300, 1.0)]
    pick = rng.integers(0, len(modes), S)
    T = np.array([modes[i][0] for i in pick], np.float32)
    K = np.array([modes[i][1] for i in pick], np.int32)
    P = np.array([modes[i][2] for i in pick], np.float32)
    h = histories(S, H, V, 4243)
    h[:, :4] = np.arange(4)
    hl = rng.integers(0, H + 1, S).astype(np.int32)
    fed = rng.integers(0, V, (S, R)).astype(np.int32)
    st = independent_states(oracle.port, 4242, S)
    g = run_gpu(ctx, x, T, K, P, st, rows_per_seq=R, rep=1.2, freq=0.1, pres=0.05, history=h, history_len=hl, fed=fed)
    o = oracle.port.sample_batch(x, T, K, P, st, rows_per_seq=R, rep=1.2, freq=0.1, pres=0.05, hist=h, hist_len=hl, extra=fed)
    check_tokens(g, o)


def test_unaligned_rows_with_penalties(ctx):
    import torch
    V, rows, H = 20011, 10, 32
    x = normal_logits(rows, V, 2.5, 66)
    h = histories(rows, H, V, 67)
    h[:, 0] = x.argmax(axis=1)
    buf = torch.zeros(rows * (V + 1) + 3, dtype=torch.float32, device="cuda")
    view = buf[3:3 + rows * (V + 1)].view(rows, V + 1)[:, :V]
    view.copy_(torch.from_numpy(x))
    st = independent_states(oracle.port, 9, rows)
    for (T, K, P) in [(0.0, 0, 1.0), (0.8, 40, 1.0), (1.0, 0, 1.0)]:
        dT, dK, dP = per_seq(rows, T, K, P)
        out = ctx.sample_batch(view, dT, dK, dP, u64_to_dev(st), rep=to_dev(np.full(rows, 1.3, np.float32)),
                               freq=to_dev(np.full(rows, 0.2, np.float32)), history=to_dev(h),
                               history_len=to_dev(np.full(rows, H, np.int32)))
        o = oracle.port.sample_batch(x, T, K, P, st, rep=1.3, freq=0.2, hist=h)
        assert np.array_equal(out["tokens"].cpu().numpy(), o["tokens"]), (T, K, P)


def test_temperature_penalised_ids_late_in_the_crossing_segment(ctx):
    """The draw lands among a few heavy ids that sit in the second half of one 1024-id segment and are
    partly penalised: the finisher has to re-penalise that segment correctly at any offset."""
    V, rows = 128256, 24
    x = np.full((rows, V), -30.0, np.float32)
    x += normal_logits(rows, V, 0.1, 5150)
    rng = np.random.default_rng(5150)
    h = histories(rows, 64, V, 5151)
    for r in range(rows):
        seg0 = int(rng.integers(0, V // 1024 - 1)) * 1024
        ids = seg0 + 600 + rng.choice(400, 8, replace=False)
        x[r, ids] = 6.0 + rng.random(8).astype(np.float32)
        h[r, :4] = ids[:4]
        h[r, 4:8] = ids[:4]  # twice: the frequency term counts
    st = independent_states(oracle.port, 5150, rows)
    g = run_gpu(ctx, x, 1.0, 0, 1.0, st, rep=1.5, freq=0.7, pres=0.3, history=h)
    o = oracle.port.sample_batch(x, 1.0, 0, 1.0, st, rep=1.5, freq=0.7, pres=0.3, hist=h)
    check_tokens(g, o)


def _long_history_case(rows, V, stride, seed):
    """Histories of mixed lengths around the 128-id limit of the loader's register path, ids drawn
    from small pools so that most repeat, some rows with every id in one slice."""
    rng = np.random.default_rng(seed)
    h = np.zeros((rows, stride), np.int32)
    lens = np.array([(0, 5, 128, 129, 130, 200, 333, stride)[r % 8] for r in range(rows)], np.int32)
    for r in range(rows):
        if r % 3 == 0:
            pool = rng.integers(0, min(V, 14000), size=90)  # all in the first slice, heavy repeats
        elif r % 3 == 1:
            pool = rng.integers(0, V, size=40 + 10 * r)
        else:
            pool = np.arange(V - 300, V)  # the last ids of the row, the ragged tail of the last slice
        h[r] = rng.choice(pool, size=stride)
    return h, lens


@pytest.mark.parametrize("T,K,P", [(0.0, 0, 1.0), (0.8, 40, 1.0), (1.0, 0, 1.0), (0.9, 0, 0.9)])
def test_long_histories_of_mixed_lengths(ctx, T, K, P):
    V, rows, stride = 128256, 48, 700
    x = normal_logits(rows, V, 2.5, 7001)
    h, lens = _long_history_case(rows, V, stride, 7002)
    for r in range(rows):  # the ids that decide the row are among the penalised ones
        top = np.argsort(-x[r])[:6]
        h[r, :min(6, lens[r])] = top[:min(6, lens[r])]
    st = independent_states(oracle.port, 7003, rows)
    rep = np.where(np.arange(rows) % 2 == 0, 1.3, 1.0).astype(np.float32)
    freq = np.where(np.arange(rows) % 4 < 2, 0.25, 0.0).astype(np.float32)
    pres = np.full(rows, 0.1, np.float32)
    g = run_gpu(ctx, x, T, K, P, st, rep=rep, freq=freq, pres=pres, history=h, history_len=lens, want_logits=True)
    o = oracle.port.sample_batch(x, T, K, P, st, rep=rep, freq=freq, pres=pres, hist=h, hist_len=lens, want_logits=True)
    assert np.array_equal(g["logits"].view(np.uint32), o["logits"].view(np.uint32))
    check_tokens(g, o)
    assert np.array_equal(g["rng_state"], o["rng_state"])


def test_long_histories_with_fed_tokens_of_verify_rows(ctx):
    V, S, R, H = 50257, 5, 6, 300
    x = normal_logits(S * R, V, 2.5, 7101)
    rng = np.random.default_rng(7102)
    h = rng.choice(rng.integers(0, V, size=70), size=(S, H)).astype(np.int32)
    lens = np.array([H, 127, 128, 126, 250], np.int32)  # 127 + up to 5 fed tokens crosses the limit inside a sequence
    fed = np.argsort(-x.reshape(S, R, V)[:, -1], axis=1)[:, :R].astype(np.int32)
    fed[:, 2] = fed[:, 1]  # a fed token twice: counted twice
    st = independent_states(oracle.port, 7103, S)
    for T in (0.0, 0.8):
        g = run_gpu(ctx, x, T, 0, 1.0, st, rows_per_seq=R, rep=1.2, freq=0.5, pres=0.4, history=h, history_len=lens, fed=fed, want_logits=True)
        o = oracle.port.sample_batch(x, T, 0, 1.0, st, rows_per_seq=R, rep=1.2, freq=0.5, pres=0.4, hist=h, hist_len=lens, extra=fed, want_logits=True)
        assert np.array_equal(g["logits"].view(np.uint32), o["logits"].view(np.uint32))
        check_tokens(g, o)


def test_long_histories_on_a_vocabulary_shard(ctx):
    """A shard sees only the ids of its own range; the others are skipped, not wrapped."""
    V, rows, stride, off = 128256, 12, 512, 40000
    vs = 32064
    x = normal_logits(rows, V, 2.5, 7201)
    h, lens = _long_history_case(rows, V, stride, 7202)
    lens[:] = stride
    shard = np.ascontiguousarray(x[:, off:off + vs])
    dT, dK, dP = per_seq(rows, 0.0, 0, 1.0)
    st = independent_states(oracle.port, 7203, rows)
    out = ctx.sample_batch(to_dev(shard), dT, dK, dP, u64_to_dev(st), rep=to_dev(np.full(rows, 1.4, np.float32)),
                           freq=to_dev(np.full(rows, 0.3, np.float32)), history=to_dev(h), history_len=to_dev(lens),
                           vocab_offset=off, want_logits=True)
    o = oracle.port.sample_batch(x, 0.0, 0, 1.0, st, rep=1.4, freq=0.3, hist=h, want_logits=True)
    assert np.array_equal(out["logits"].cpu().numpy().view(np.uint32), o["logits"][:, off:off + vs].view(np.uint32))


def test_many_multi_pass_rows_per_block(ctx):
    """Every row needs the multi-pass path (top-k beyond the one-pass limit, wide nuclei), several per
    thread block: they are queued while the block streams and served at its end."""
    V, rows = 32000, 480
    x = normal_logits(rows, V, 2.5, 8101)
    T = np.where(np.arange(rows) % 2 == 0, 0.8, 1.0).astype(np.float32)
    K = np.where(np.arange(rows) % 2 == 0, 300, 0).astype(np.int32)
    P = np.where(np.arange(rows) % 2 == 0, 1.0, 0.97).astype(np.float32)
    st = independent_states(oracle.port, 8102, rows)
    g = run_gpu(ctx, x, T, K, P, st)
    o = oracle.port.sample_batch(x, T, K, P, st)
    check_tokens(g, o)
    assert np.array_equal(g["rng_state"], o["rng_state"])
    assert (g["status"] & 2).all()  # informational bit: the multi-pass path served the row


def test_wide_topk_with_long_histories(ctx):
    """Top-k 200 with 600-id histories: less shared-memory room for a row's merged candidates, so some
    rows change to the multi-pass path; the tokens do not depend on which path served a row."""
    V, rows, H = 128256, 64, 600
    x = normal_logits(rows, V, 2.5, 8201)
    h = histories(rows, H, V, 8202)
    for r in range(rows):
        h[r, :20] = np.argsort(-x[r])[:20]
    st = independent_states(oracle.port, 8203, rows)
    g = run_gpu(ctx, x, 0.9, 200, 1.0, st, rep=1.2, freq=0.1, history=h)
    o = oracle.port.sample_batch(x, 0.9, 200, 1.0, st, rep=1.2, freq=0.1, hist=h)
    check_tokens(g, o)


def test_signed_zeros_are_one_value(ctx):
    """-0.0 and +0.0 compare equal in the reference's sort and argmax, so ties between them go to the
    lower id; a key built from the bit pattern alone would put every +0.0 first."""
    V, rows = 1582, 96
    rng = np.random.default_rng(8301)
    x = (np.round(rng.standard_normal((rows, V)).astype(np.float32) * 0.02) / 2).astype(np.float32)  # only +0.0 and -0.0
    assert np.signbit(x).any() and not np.signbit(x).all()
    x[::3, 7] = 0.5  # some rows with one clear maximum
    st = independent_states(oracle.port, 8302, rows)
    for (T, K, P) in [(0.0, 0, 1.0), (0.3, 40, 1.0), (1.5, 200, 1.0), (1.0, 300, 1.0), (1.0, 0, 0.3)]:
        g = run_gpu(ctx, x, T, K, P, st, kept_cap=40)
        o = oracle.port.sample_batch(x, T, K, P, st, detail_cap=40)
        check_tokens(g, o)
        if K == 40:
            listed = (g["status"] & 8) == 0  # rows of nothing but ties take the multi-pass path, which lists no kept set
            assert np.array_equal(g["kept_idx"][listed], o["detail_idx"][listed])


def test_topp_nucleus_of_most_of_the_vocabulary(ctx):
    """Nearly flat rows: the nucleus holds over a hundred thousand ids a few 1e-6 apart, so the draw
    lands on the reference's id only if every e_i is the correctly rounded one."""
    V, rows = 151936, 256
    x = normal_logits(rows, V, 0.01, 8401)
    st = independent_states(oracle.port, 8402, rows)
    P = np.where(np.arange(rows) % 2 == 0, 0.9, 0.99).astype(np.float32)
    g = run_gpu(ctx, x, 1.0, 0, P, st)
    o = oracle.port.sample_batch(x, 1.0, 0, P, st)
    check_tokens(g, o)


def test_history_sizes_up_to_the_limit(ctx):
    """4000 ids per row still run (one ring stage less), 9000 are refused with a message."""
    from geistlib_b200 import api
    V, rows = 128256, 6
    x = normal_logits(rows, V, 2.5, 8501)
    h = histories(rows, 4000, V, 8502)
    h[:, :8] = np.argsort(-x, axis=1)[:, :8]
    st = independent_states(oracle.port, 8503, rows)
    for (T, K) in [(0.0, 0), (0.8, 40)]:
        g = run_gpu(ctx, x, T, K, 1.0, st, rep=1.3, freq=0.05, history=h)
        o = oracle.port.sample_batch(x, T, K, 1.0, st, rep=1.3, freq=0.05, hist=h)
        check_tokens(g, o)
    with pytest.raises(api.GeistError):
        run_gpu(ctx, x, 0.0, 0, 1.0, st, rep=1.3, history=histories(rows, 9000, V, 8504))

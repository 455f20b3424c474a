"""CPU checks (no GPU): the C restatement (oracle/sampler_oracle.c) against
  (1) golden vectors produced by the reference's own sampler.c (tests/golden),
  (2) the reference compiled here (oracle/_ref), live, on random and adversarial rows,
  (3) the properties the reference's unit test asserts (tests/test_sampler_unit.c)."""
import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from helpers import gumbel_logits, histories, independent_states, normal_logits

G = np.load(Path(__file__).parent / "golden" / "sampler_golden.npz")
META = json.loads((Path(__file__).parent / "golden" / "sampler_golden.json").read_text())
port = oracle.port
needs_ref = pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built (reference tree absent)")

# first raw draw per seed as hex, from a recorded run of the reference's own generator
KNOWN_RNG = {0: "0d83b3e29a21487a", 1: "47e4ce4b896cdd1d", 7: "d1fbaf7f728d2eae", 99: "4c0ab4d5974e3cef",
              1234: "bc5614c61020390e", 2024: "fa90026eb2d63a0a", 31337: "93801fc0758ef0c1",
              0xCAFEBABE1234: "3620af4c8a44b89a", 0xC0FFEE: "fec579340d9c0ad5"}


def test_rng_matches_golden_streams():
    for i, seed in enumerate(G["rng_seeds"]):
        u, f = port.rng_stream(int(seed), 16)
        assert np.array_equal(u, G["rng_u64"][i])
        assert np.array_equal(f.view(np.uint32), G["rng_unit"][i].view(np.uint32))
        if int(seed) in KNOWN_RNG:
            assert f"{int(u[0]):016x}" == KNOWN_RNG[int(seed)]
    assert port.rng_seed(0) == 0x9E3779B97F4A7C15
    assert ((G["rng_unit"] >= 0) & (G["rng_unit"] < 1)).all()


def _stream(which, row, n, seed, **kw):
    st = port.rng_seed(seed)
    toks = []
    for _ in range(n):
        t, st = port.sampler_call(which, row, state=st, **kw)
        toks.append(t)
    return np.array(toks, np.int32)


def test_reference_unit_test_cases():
    """The eight checks of tests/test_sampler_unit.c, token for token against the reference's output."""
    assert port.argmax(G["lit_argmax_ties"]) == int(G["lit_argmax_ties_tok"][0]) == 3
    t = _stream("temperature", G["lit_peaked"], 1000, 42, T=0.1)
    assert np.array_equal(t, G["lit_peaked_T0.1_seed42"]) and (t == 3).sum() > 990
    assert _stream("temperature", G["lit_small4"], 1, 1, T=0.0)[0] == 2
    t = _stream("temperature", G["lit_uniform5"], 5000, 7, T=1.0)
    assert np.array_equal(t, G["lit_uniform5_T1_seed7"])
    assert np.bincount(t, minlength=5).tolist() == [997, 1055, 979, 999, 970]
    t = _stream("top_k", G["lit_topk8"], 1000, 11, top_k=2, T=1.0)
    assert np.array_equal(t, G["lit_topk8_k2_T1_seed11"]) and set(t.tolist()) == {2, 4}
    t = _stream("top_p", G["lit_topp5"], 1000, 13, top_p=0.5, T=1.0)
    assert np.array_equal(t, G["lit_topp5_p0.5_T1_seed13"]) and (t == 0).sum() > 990
    assert np.array_equal(_stream("top_k", G["lit_ws8"], 100, 17, top_k=3, T=1.0), G["lit_ws8_k3_T1_seed17"])


@pytest.mark.parametrize("case", META["cases"], ids=lambda c: c["name"])
def test_dispatch_matches_golden(case):
    n = case["name"]
    x = G[f"case_{n}_logits"]
    o = port.sample_batch(x, case["T"], case["top_k"], case["top_p"], G[f"case_{n}_state_in"],
                          rows_per_seq=case["rows_per_seq"], detail_cap=2048)
    assert np.array_equal(o["tokens"], G[f"case_{n}_tokens"])
    assert np.array_equal(o["rng_state"], G[f"case_{n}_state_out"])
    if f"case_{n}_kept_idx" in G.files:
        k = G[f"case_{n}_kept_idx"].size
        assert o["detail_n"][0] == k
        assert np.array_equal(o["detail_idx"][0, :k], G[f"case_{n}_kept_idx"])
        assert np.array_equal(o["detail_prob"][0, :k].view(np.uint32), G[f"case_{n}_kept_prob"].view(np.uint32))


def test_softmax_matches_golden():
    p, s = port.softmax(G["softmax_logits"], 0.7)
    assert np.array_equal(p.view(np.uint32), G["softmax_T0.7"].view(np.uint32))
    assert s == float(G["softmax_T0.7_sum"][0])


@needs_ref
@pytest.mark.parametrize("V", [1, 2, 5, 100, 1023, 1025, 8192, 8193, 40000])
def test_port_equals_reference_live(V):
    rows = 6
    rng = np.random.default_rng(V)
    for kind in ("normal", "ties", "gumbel"):
        if kind == "normal":
            x = normal_logits(rows, V, 2.5, V + 1)
        elif kind == "ties":
            x = rng.integers(-2, 3, (rows, V)).astype(np.float32)
        else:
            x = gumbel_logits(rows, V, 4.0, V + 2)
        x[0, :] = 1.5
        if V > 3:
            x[1, 1] = -np.inf
            x[1, 2] = np.inf
        st = independent_states(port, 9, rows)
        for (T, K, P) in [(0.0, 0, 1.0), (0.8, 40, 0.95), (1.0, 2, 1.0), (0.8, 0, 0.9), (0.5, 0, 0.3),
                          (1.3, 0, 1.0), (0.8, 9000, 1.0), (-0.5, 5, 0.5), (0.8, 1, 0.0), (0.8, 0, 1.5)]:
            a = oracle.ref.sample(x, T, K, P, st)
            b = port.sample_batch(x, T, K, P, st)
            assert np.array_equal(a["tokens"], b["tokens"]), (kind, T, K, P)
            assert np.array_equal(a["rng_state"], b["rng_state"]), (kind, T, K, P)


@needs_ref
def test_port_equals_reference_rows_in_sequence():
    V, S, R = 5000, 5, 7
    x = normal_logits(S * R, V, 2.5, 3)
    st = independent_states(port, 2024, S)
    for (T, K, P) in [(0.9, 30, 1.0), (0.7, 0, 0.8), (1.0, 0, 1.0), (0.0, 0, 1.0)]:
        a = oracle.ref.sample(x, T, K, P, st, rows_per_seq=R)
        b = port.sample_batch(x, T, K, P, st, rows_per_seq=R)
        assert np.array_equal(a["tokens"], b["tokens"])
        assert np.array_equal(a["rng_state"], b["rng_state"])
        draws = R if T > 0 else 0
        assert all(int(b["rng_state"][s]) == port.rng_advance(int(st[s]), draws) for s in range(S))


@needs_ref
def test_release_flag_build_agrees_with_strict_build():
    """The timed CPU baseline is the reference built with its release flags; its tokens are
    cross-checked against the strict build that serves as parity checker."""
    x = normal_logits(16, 128256, 2.5, 11)
    st = independent_states(port, 4, 16)
    for (T, K, P) in [(0.0, 0, 1.0), (0.8, 40, 1.0), (0.8, 0, 0.95), (0.8, 0, 1.0)]:
        a = oracle.ref.sample(x, T, K, P, st)
        b = oracle.ref_release.sample(x, T, K, P, st)
        assert np.array_equal(a["tokens"], b["tokens"])


@needs_ref
def test_kept_sets_equal_reference():
    x = normal_logits(3, 3000, 2.5, 5)
    x[2] = np.round(x[2])  # many ties
    for r in range(3):
        o = port.sample_batch(x[r:r + 1], 0.8, 40, 1.0, [7], detail_cap=64)
        idx, prob, _ = oracle.ref.topk_detail(x[r], 40, 0.8)
        assert np.array_equal(o["detail_idx"][0, :40], idx)
        assert np.array_equal(o["detail_prob"][0, :40].view(np.uint32), prob.view(np.uint32))
        o = port.sample_batch(x[r:r + 1], 0.8, 0, 0.9, [7], detail_cap=3000)
        n, idx, pn, pq, _ = oracle.ref.topp_detail(x[r], 0.9, 0.8)
        assert o["detail_n"][0] == n
        assert np.array_equal(o["detail_idx"][0, :n], idx)
        assert np.array_equal(o["detail_prob"][0, :n].view(np.uint32), pq.view(np.uint32))


def test_penalties_off_is_bit_identical_and_on_follows_the_definition():
    V = 4000
    x = normal_logits(1, V, 2.5, 1)[0]
    h = histories(1, 200, V, 2)[0]
    h[:50] = h[50:100]
    h[0] = -5
    h[1] = V + 7  # ids outside the vocabulary are ignored
    assert np.array_equal(port.apply_penalties(x, h, 1.0, 0.0, 0.0).view(np.uint32), x.view(np.uint32))
    assert np.array_equal(port.apply_penalties(x, h, 0.0, 0.0, 0.0).view(np.uint32), x.view(np.uint32))
    y = port.apply_penalties(x, h, 1.2, 0.25, 0.5)
    cnt = np.bincount(h[(h >= 0) & (h < V)], minlength=V)
    exp = x.copy()
    hit = cnt > 0
    rep = np.float32(1.2)
    exp[hit] = np.where(x[hit] > 0, x[hit] / rep, x[hit] * rep)
    exp[hit] = exp[hit] - cnt[hit].astype(np.float32) * np.float32(0.25)
    exp[hit] = exp[hit] - np.float32(0.5)
    assert np.array_equal(y.view(np.uint32), exp.astype(np.float32).view(np.uint32))
    assert np.array_equal(y[~hit].view(np.uint32), x[~hit].view(np.uint32))


def test_spec_accept_rule():
    """session.c:599-625: longest matching prefix, then the target's token at the first mismatch."""
    fed = np.array([10, 11, 12, 13], np.int32)
    a, em = port.spec_accept(fed, np.array([11, 12, 13, 99], np.int32))
    assert a == 3 and em.tolist() == [10, 11, 12, 13, 99]          # all accepted + bonus
    a, em = port.spec_accept(fed, np.array([11, 77, 13, 99], np.int32))
    assert a == 1 and em.tolist() == [10, 11, 77]                  # correction at the first mismatch
    a, em = port.spec_accept(fed, np.array([5, 12, 13, 99], np.int32))
    assert a == 0 and em.tolist() == [10, 5]
    a, em = port.spec_accept(fed[:1], np.array([42], np.int32))
    assert a == 0 and em.tolist() == [10, 42]                      # k == 1: plain decode


def test_shard_merge_equals_unsharded_topk():
    V, G_, k = 4096, 8, 50
    x = np.round(normal_logits(1, V, 2.5, 9)[0] * 4) / 4  # ties across shards
    vs = V // G_
    vals, gids = [], []
    for g in range(G_):
        shard = x[g * vs:(g + 1) * vs]
        order = np.lexsort((np.arange(vs), -shard))[:k]
        vals.append(shard[order])
        gids.append(order + g * vs)
    mv, mg = port.merge_candidates(np.concatenate(vals), np.concatenate(gids), k)
    order = np.lexsort((np.arange(V), -x))[:k]
    assert np.array_equal(mg, order) and np.array_equal(mv, x[order])
    tok, st = port.sample_ordered(mv, mg, 0.7, port.rng_seed(31337))
    ref = port.sample_batch(x[None, :], 0.7, k, 0.9, [port.rng_seed(31337)])
    assert tok == ref["tokens"][0] and st == int(ref["rng_state"][0])


# ------------------------------------------------------------ soft cap, drafter --

def test_softcap_port_equals_reference_expression():
    """head.c:152-155: p = tanhf(p / c) * c; the port and the harness around the reference agree bit for bit."""
    x = (np.random.default_rng(11).standard_normal(200000) * 40).astype(np.float32)
    x[:4] = [0.0, -0.0, np.inf, -np.inf]
    y = port.softcap(x, 30.0)
    assert y[2] == 30.0 and y[3] == -30.0 and np.abs(y).max() <= 30.0
    assert np.all(np.diff(y[np.argsort(x, kind="stable")]) >= 0), "monotone"
    if oracle.ref is not None:
        assert np.array_equal(y.view(np.uint32), oracle.ref.softcap(x, 30.0).view(np.uint32))


def test_drafter_known_answers():
    """session.c:437-513 by hand: longest suffix first, most following context, newest on ties."""
    d = port.propose_drafts
    assert d([], 5, 8)[0].tolist() == [5] and d([], 5, 8)[1] == 0
    assert d([1, 2, 3], 9, 8)[0].tolist() == [9] and d([1, 2, 3], 9, 8)[1] == 0      # seed never seen
    out, L = d([1, 2, 3, 4, 1, 2], 3, 4)          # context ...1 2 [3]: matches position 0..2, then 4 1 2 follow
    assert L == 3 and out.tolist() == [3, 4, 1, 2]
    out, L = d([7, 3, 8, 9, 7, 3, 5], 3, 3, 1)    # L = 1: two places; the older one offers 2 tokens, the newer 1
    assert L == 1 and out.tolist() == [3, 8, 9]
    out, L = d([3, 8, 9, 3, 8, 9, 4], 3, 3, 1)    # tie on following context: the newest place wins
    assert L == 1 and out.tolist() == [3, 8, 9]
    out, L = d([1, 2, 3], 3, 4)                   # the only match sits at the tail: nothing follows
    assert L == 0 and out.tolist() == [3]
    out, L = d([1, 2, 3, 4], 2, 1)                # k_max 1: the seed alone
    assert L == 0 and out.tolist() == [2]
    out, L = d(list(range(10)) * 2, 0, 16, 20)    # max_suffix is clamped to 8
    assert L == 8 and out.tolist() == list(range(10))


@pytest.mark.skipif(oracle.ref_drafter is None, reason="oracle/_ref not built")
def test_drafter_port_equals_reference_function():
    """The restatement against the reference's own propose_drafts_ngram on random small-alphabet histories."""
    rng = np.random.default_rng(2026)
    for _ in range(4000):
        n, voc = int(rng.integers(0, 64)), int(rng.integers(1, 7))
        h = rng.integers(0, voc, n).astype(np.int32)
        seed, k, ms = int(rng.integers(0, voc)), int(rng.integers(1, 17)), int(rng.integers(1, 12))
        a, b = port.propose_drafts(h, seed, k, ms), oracle.ref_drafter.propose_drafts(h, seed, k, ms)
        assert np.array_equal(a[0], b[0]) and a[1] == b[1], (h, seed, k, ms, a, b)

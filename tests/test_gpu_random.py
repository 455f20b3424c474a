"""Randomised parity: batches drawn from a seeded generator (vocabulary, rows, modes per sequence, logit
shapes, histories with repeats, verify rows with fed tokens) through the C-ABI library against the oracle.
Every case is reproducible from its seed."""
import numpy as np
import pytest

import oracle
from helpers import independent_states, per_seq, to_dev, u64_from_dev, u64_to_dev

pytestmark = pytest.mark.gpu

INVALID = 1 | 4 | 16  # load timeout, history overflow, internal: never expected
KEPT_PARTIAL = 8


@pytest.fixture(scope="module")
def ctx():
    from geistlib_b200 import api
    return api.Context(0)


def make_case(seed):
    rg = np.random.default_rng(seed)
    V = int(rg.choice([rg.integers(2, 2000), rg.integers(2000, 40000), rg.integers(40000, 300000), 128256, 151936]))
    R = int(rg.choice([1, 1, 1, 3, 7]))
    S = int(rg.integers(1, max(2, min(200, 12_000_000 // (V * R)))))
    rows = S * R
    kind = str(rg.choice(["normal", "gumbel", "ties", "masked", "peaked"]))
    x = rg.standard_normal((rows, V), dtype=np.float32) * np.float32(rg.choice([0.01, 1.0, 2.5, 6.0]))
    if kind == "gumbel":
        x = (-4.0 * np.log(-np.log(rg.uniform(1e-12, 1 - 1e-7, (rows, V))))).astype(np.float32)
    elif kind == "ties":
        x = (np.round(x * 2) / 2).astype(np.float32)
    elif kind == "masked":
        m = rg.uniform(size=(rows, V)) < rg.choice([0.1, 0.9, 0.99])
        m[:, rg.integers(0, V)] = False
        x[m] = -np.inf
    elif kind == "peaked":
        x[np.arange(rows), rg.integers(0, V, rows)] += 15.0
    T = rg.choice([0.0, 0.3, 0.7, 1.0, 1.5], size=S).astype(np.float32)
    K = rg.choice([0, 1, 2, 5, 40, 100, 200, 256, 300, 1000, 9000], size=S).astype(np.int32)
    P = rg.choice([1.0, 0.3, 0.8, 0.9, 0.95, 0.99], size=S).astype(np.float32)
    gpu_kw, ref_kw = {}, {}
    H = int(rg.choice([0, 0, 5, 64, 128, 129, 300, 700]))
    if H:
        pool = rg.integers(0, V, size=max(1, int(rg.choice([H // 4 + 1, 4 * H]))))
        h = rg.choice(pool, size=(S, H)).astype(np.int32)
        hl = rg.integers(0, H + 1, S).astype(np.int32)
        rep = rg.choice([1.0, 1.1, 1.5, 0.8], size=S).astype(np.float32)
        freq = rg.choice([0.0, 0.2, -0.1], size=S).astype(np.float32)
        pres = rg.choice([0.0, 0.3], size=S).astype(np.float32)
        gpu_kw = dict(history=h, history_len=hl, rep=rep, freq=freq, pres=pres)
        ref_kw = dict(hist=h, hist_len=hl, rep=rep, freq=freq, pres=pres)
        if R > 1:
            fed = rg.integers(0, V, size=(S, R)).astype(np.int32)
            gpu_kw["fed"] = fed
            ref_kw["extra"] = fed
    return dict(x=x, T=T, K=K, P=P, R=R, S=S, gpu_kw=gpu_kw, ref_kw=ref_kw, what=f"V={V} S={S} R={R} {kind} H={H}")


@pytest.mark.parametrize("seed", [4200 + i for i in range(32)])
def test_random_batch_matches_the_oracle(ctx, seed):
    c = make_case(seed)
    x, T, K, P, R, S = c["x"], c["T"], c["K"], c["P"], c["R"], c["S"]
    st = independent_states(oracle.port, seed, S)
    dT, dK, dP = per_seq(S, T, K, P)
    cap = 64
    out = ctx.sample_batch(to_dev(x), dT, dK, dP, u64_to_dev(st), rows_per_seq=R, kept_cap=cap, want_logits=True,
                           **{k: to_dev(v) for k, v in c["gpu_kw"].items()})
    ref = oracle.port.sample_batch(x, T, K, P, st, rows_per_seq=R, detail_cap=cap, want_logits=True, **c["ref_kw"])
    status = out["status"].cpu().numpy()
    assert (status & INVALID == 0).all(), c["what"]
    assert np.array_equal(out["logits"].cpu().numpy().view(np.uint32), ref["logits"].view(np.uint32)), c["what"]
    tok = out["tokens"].cpu().numpy()
    assert np.array_equal(tok, ref["tokens"]), (c["what"], np.nonzero(tok != ref["tokens"])[0][:5])
    assert np.array_equal(u64_from_dev(out["rng_state"]), ref["rng_state"]), c["what"]
    # kept sets of the rows that filter (top-k or top-p) and list their set
    Tr, Kr, Pr = np.repeat(T, R), np.repeat(K, R), np.repeat(P, R)
    listed = (Tr > 0) & ((Kr > 1) | ((Pr > 0) & (Pr < 1))) & ((status & KEPT_PARTIAL) == 0)
    kn, ki, kp = out["kept_n"].cpu().numpy(), out["kept_idx"].cpu().numpy(), out["kept_prob"].cpu().numpy()
    for r in np.nonzero(listed)[0]:
        m = min(int(kn[r]), cap)
        assert kn[r] == ref["detail_n"][r], (c["what"], r)
        assert np.array_equal(ki[r, :m], ref["detail_idx"][r, :m]), (c["what"], r)
        if m:
            rel = np.abs(kp[r, :m] - ref["detail_prob"][r, :m]) / np.maximum(ref["detail_prob"][r, :m], 1e-30)
            assert rel.max() <= 1e-5, (c["what"], r)  # fp32 probabilities: 1e-5 relative

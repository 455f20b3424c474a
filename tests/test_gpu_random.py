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


@pytest.mark.parametrize("seed,HM", [(9100, 24), (9101, 24), (9102, 200), (9103, 200)])
def test_random_session_traffic_through_the_batcher(ctx, seed, HM):
    """Sessions open and close, decode steps and verify passes take random subsets of them in random
    order; every session must behave like a reference session of its own (generator word, history
    ring of HM ids, sampler options)."""
    from geistlib_b200 import api
    port = oracle.port
    V, MAXS = 6000, 12
    rg = np.random.default_rng(seed)
    bt = api.Batcher(ctx, V, MAXS, max_history=HM)
    live = {}  # session id -> dict(cfg, state, hist)

    def open_one():
        T = float(rg.choice([0.0, 0.6, 1.0])); K = int(rg.choice([0, 1, 20, 300])); P = float(rg.choice([1.0, 0.9, 0.5]))
        rep = float(rg.choice([1.0, 1.2])); freq = float(rg.choice([0.0, 0.3])); pres = float(rg.choice([0.0, 0.2]))
        sd = int(rg.integers(1, 1 << 30))
        s = bt.open(temperature=T, top_p=P, top_k=K, seed=sd, rep=rep, freq=freq, pres=pres)
        h = rg.integers(0, V, int(rg.integers(0, HM + 1))).astype(np.int32)
        if len(h):
            bt.push_history(s, h)
        live[s] = dict(cfg=(T, K, P, rep, freq, pres), state=port.rng_seed(sd), hist=list(h))

    def ref_rows(s, x, rows_per_seq=1, fed=None):
        T, K, P, rep, freq, pres = live[s]["cfg"]
        hh = np.array(live[s]["hist"][-HM:], np.int32)[None, :]
        kw = dict(rep=rep, freq=freq, pres=pres)
        if hh.shape[1]:
            kw["hist"] = hh
        if fed is not None:
            kw["extra"] = fed[None, :]
        return port.sample_batch(x, T, K, P, [live[s]["state"]], rows_per_seq=rows_per_seq, **kw)

    for _ in range(3):
        open_one()
    for op in range(40):
        what = rg.choice(["open", "close", "step", "step", "step", "verify"])
        if what == "open" and len(live) < MAXS:
            open_one()
        elif what == "close" and len(live) > 1:
            s = int(rg.choice(list(live)))
            bt.close_session(s)
            del live[s]
        elif what == "step":
            ss = [int(s) for s in rg.permutation(list(live))[:int(rg.integers(1, len(live) + 1))]]
            x = (rg.standard_normal((len(ss), V)) * 2.5).astype(np.float32)
            got = bt.step(ss, to_dev(x) if op % 2 else x)
            for i, s in enumerate(ss):
                o = ref_rows(s, x[i:i + 1])
                assert got[i] == o["tokens"][0], (op, s, live[s]["cfg"])
                live[s]["state"] = int(o["rng_state"][0])
                live[s]["hist"].append(int(got[i]))
                assert bt.get_rng(s) == live[s]["state"]
        elif what == "verify":
            ss = [int(s) for s in rg.permutation(list(live))[:int(rg.integers(1, len(live) + 1))]]
            k = int(rg.integers(1, 7))
            x = (rg.standard_normal((len(ss) * k, V)) * 2.5).astype(np.float32)
            x[:, :3] += 9.0  # a few likely tokens, so that some proposals are accepted
            fed = rg.integers(0, 3, (len(ss), k)).astype(np.int32)
            acc, nout, toks = bt.verify(ss, fed, to_dev(x))
            for i, s in enumerate(ss):
                o = ref_rows(s, x[i * k:(i + 1) * k], rows_per_seq=k, fed=fed[i])
                a, em = port.spec_accept(fed[i], o["tokens"])
                assert acc[i] == a and nout[i] == len(em) and np.array_equal(toks[i, :nout[i]], em), (op, s, k)
                live[s]["state"] = int(o["rng_state"][0])
                live[s]["hist"].extend(int(t) for t in em[1:])  # em[0] is the pending token: it joined the history when it was sampled
                assert bt.get_rng(s) == live[s]["state"]
    bt.close()

"""GPU tests of the reference-facing layers of the C ABI: the sampler.h host-pointer
surface, the argmax_f32 operator slot, the session batcher (decode step and speculative
verify), vocabulary shards, and the dense inspection outputs."""
import ctypes as C

import numpy as np
import pytest

import oracle
from geistlib_b200 import api
from helpers import histories, independent_states, normal_logits, per_seq, rel_err, to_dev, u64_from_dev, u64_to_dev

pytestmark = pytest.mark.gpu
port = oracle.port


def test_sampler_h_surface_matches_reference_unit_cases(ctx):
    """tests/test_sampler_unit.c, driven through the same-named entry points with host arrays."""
    assert api.sampler_argmax(np.array([-1.0, 2.0, 0.5, 3.0, 3.0, -0.5], np.float32)) == 3
    rng = api.rng_seed(1)
    assert api.sampler_temperature(np.array([1.0, 2.0, 3.0, 0.5], np.float32), 0.0, rng) == 2
    assert rng.state == 1  # greedy draws nothing
    # fixed-seed streams against the CPU checker, token for token
    x = normal_logits(1, 128256, 2.5, 77)[0]
    ws = api.SamplerWorkspace(x.size)
    for which, kw in [("top_k", dict(top_k=40, T=0.8)), ("top_p", dict(top_p=0.9, T=0.8)), ("temperature", dict(T=1.1))]:
        rng = api.rng_seed(1234)
        st = port.rng_seed(1234)
        for _ in range(6):
            if which == "top_k":
                t = ws.top_k(x, kw["top_k"], kw["T"], rng)
            elif which == "top_p":
                t = ws.top_p(x, kw["top_p"], kw["T"], rng)
            else:
                t = api.sampler_temperature(x, kw["T"], rng)
            e, st = port.sampler_call(which, x, state=st, **kw)
            assert t == e and rng.state == st
    # early-outs of the reference functions: no draw is consumed
    rng = api.rng_seed(5)
    assert ws.top_k(x, 1, 0.8, rng) == int(x.argmax()) and rng.state == 5
    assert ws.top_p(x, 0.0, 0.8, rng) == int(x.argmax()) and rng.state == 5
    assert ws.top_k(x, 40, 0.0, rng) == int(x.argmax()) and rng.state == 5
    ws.close()
    small = np.array([0.0, 1.0, 4.0, 2.0, 5.0, 1.5, 0.0, 0.5], np.float32)
    ws = api.SamplerWorkspace(8)
    rng = api.rng_seed(11)
    assert {ws.top_k(small, 2, 1.0, rng) for _ in range(200)} == {2, 4}
    ws.close()


def test_argmax_f32_slot(ctx):
    """test_fused_probe_agreement_unit.c:139-160: if the probe says yes the op must return OK and 77."""
    import torch
    assert api.lib.geist_b200_argmax_f32_supported(1, 256) == 1
    assert api.lib.geist_b200_argmax_f32_supported(2, 256) == 0
    row = torch.zeros(256, device="cuda")
    row[77] = 9.0
    assert ctx.argmax_f32(row) == 77
    x = normal_logits(1, 151936, 3.0, 3)[0]
    x[1000] = x[90000] = x.max() + 1.0  # tie: lowest index
    assert ctx.argmax_f32(to_dev(x)) == 1000


@pytest.mark.parametrize("H0,HM", [(20, 24), (294, 300)])  # short histories; histories prepared by the kernel of their own
def test_batcher_decode_steps_equal_independent_reference_sessions(ctx, H0, HM):
    V, N, steps = 32000, 12, 6  # the history ring wraps during the run
    rng = np.random.default_rng(0)
    bt = api.Batcher(ctx, V, 16, max_history=HM)
    cfgs = [(0.0, 0, 1.0), (0.8, 40, 0.95), (0.7, 0, 0.9), (1.0, 0, 0.0)] * 3
    pens = [(1.0, 0.0, 0.0), (1.2, 0.0, 0.0), (1.1, 0.3, 0.2), (0.0, 0.0, 0.4)] * 3
    sess, state, hist = [], [], []
    for i, ((T, K, P), (r, f, pr)) in enumerate(zip(cfgs, pens)):
        seed = 0 if i == 1 else 100 + i
        sess.append(bt.open(temperature=T, top_p=P, top_k=K, seed=seed, rep=r, freq=f, pres=pr))
        state.append(port.rng_seed(seed if seed else 0xCAFEBABE1234))  # arch_state.c:1168-1173
        h = rng.integers(0, V, H0).astype(np.int32)
        bt.push_history(sess[-1], h)
        hist.append(list(h))
    for step in range(steps):
        x = normal_logits(N, V, 2.5, 50 + step)
        x[:, :5] += 9.0
        got = bt.step(sess, to_dev(x)) if step % 2 == 0 else bt.step(sess, x)  # device and host logits
        for i, ((T, K, P), (r, f, pr)) in enumerate(zip(cfgs, pens)):
            Pn = P if P > 0 else 1.0  # step.c:391
            hh = np.array(hist[i][-HM:], np.int32)[None, :]
            o = port.sample_batch(x[i:i + 1], T, K, Pn, [state[i]], rep=r if r > 0 else 1.0, freq=f, pres=pr, hist=hh)
            assert got[i] == o["tokens"][0], (step, i)
            state[i] = int(o["rng_state"][0])
            hist[i].append(int(got[i]))
            assert bt.get_rng(sess[i]) == state[i]
    # checkpoint / resume of a sampled stream = restoring the generator word
    saved = bt.get_rng(sess[1])
    x = normal_logits(N, V, 2.5, 999)
    a = bt.step(sess, to_dev(x), append_history=False)
    bt.set_rng(sess[1], saved)
    b = bt.step(sess[1:2], to_dev(x[1:2]), append_history=False)
    assert a[1] == b[0]
    with pytest.raises(api.GeistError):
        bt.step([sess[0], sess[0]], to_dev(x[:2]))
    bt.close()


def test_batcher_verify_applies_the_prefix_accept_rule(ctx):
    V, N, k = 32000, 6, 5
    bt = api.Batcher(ctx, V, 8, max_history=32)
    rng = np.random.default_rng(1)
    for (T, K, P) in [(0.0, 0, 1.0), (0.9, 30, 1.0)]:
        sess = [bt.open(temperature=T, top_k=K, top_p=P, seed=7 + i, rep=1.2, freq=0.1) for i in range(N)]
        h = histories(N, 16, V, 4)
        for s, hh in zip(sess, h):
            bt.push_history(s, hh)
        x = normal_logits(N * k, V, 2.5, 6)
        x[:, :4] += 8.0
        st = np.array([port.rng_seed(7 + i) for i in range(N)], np.uint64)
        fed = rng.integers(0, V, (N, k)).astype(np.int32)
        o = port.sample_batch(x, T, K, P, st, rows_per_seq=k, rep=1.2, freq=0.1, hist=h, extra=fed)
        vo = o["tokens"].reshape(N, k)
        fed[0, 1:] = vo[0, :k - 1]  # every proposal right -> bonus token
        fed[1, 1:3] = vo[1, :2]
        o = port.sample_batch(x, T, K, P, st, rows_per_seq=k, rep=1.2, freq=0.1, hist=h, extra=fed)
        vo = o["tokens"].reshape(N, k)
        acc, nout, toks = bt.verify(sess, fed, to_dev(x))
        for i in range(N):
            a, em = port.spec_accept(fed[i], vo[i])
            assert acc[i] == a and nout[i] == a + 2 and np.array_equal(toks[i, :a + 2], em)
            assert bt.get_rng(sess[i]) == int(o["rng_state"][i])
        assert acc[0] == k - 1
        for s in sess:
            bt.close_session(s)
    with pytest.raises(api.GeistError):
        bt.verify([0], np.zeros((1, 17), np.int32), to_dev(np.zeros((17, V), np.float32)))  # k_max is 16
    bt.close()


def test_vocab_shards_equal_the_unsharded_row(ctx):
    """8 shards of V/8 with per-shard top-50 (global ids), merged, then the top-k draw."""
    import torch
    V, G, B, k, T = 128256, 8, 16, 50, 0.7
    x = normal_logits(B, V, 2.5, 31337)
    x[:, ::4001] = np.round(x[:, ::4001])  # ties across shards
    h = histories(B, 128, V, 3)
    st = independent_states(port, 31337, B)
    ref = port.sample_batch(x, T, k, 0.9, st, rep=1.15, hist=h, detail_cap=k)
    vs = V // G
    dT, dK, dP = per_seq(B, T, k, 0.9)
    vals, gids, ns = [], [], []
    for g in range(G):
        shard = to_dev(np.ascontiguousarray(x[:, g * vs:(g + 1) * vs]))
        out = ctx.sample_batch(shard, dT, dK, dP, u64_to_dev(st), rep=to_dev(np.full(B, 1.15, np.float32)),
                               history=to_dev(h), history_len=to_dev(np.full(B, 128, np.int32)),
                               kept_cap=k, vocab_offset=g * vs, select_only=True)
        vals.append(out["kept_prob"]), gids.append(out["kept_idx"]), ns.append(out["kept_n"])
    m = ctx.shard_merge_sample(torch.stack(vals), torch.stack(gids), torch.stack(ns), dT, dK, u64_to_dev(st), kept_cap=k)
    assert np.array_equal(m["tokens"].cpu().numpy(), ref["tokens"])
    assert np.array_equal(u64_from_dev(m["rng_state"]), ref["rng_state"])
    assert np.array_equal(m["kept_idx"].cpu().numpy(), ref["detail_idx"])
    assert rel_err(m["kept_prob"].cpu().numpy(), ref["detail_prob"]) <= 1e-5


def test_post_filter_probability_vector(ctx):
    """Single-row case: token plus the dense post-filter probability vector."""
    V = 128256
    rng = np.random.default_rng(1234)
    x = normal_logits(1, V, 2.5, 1234)
    x[0, rng.integers(0, V, 8)] += 12.0
    h = histories(1, 64, V, 1234)
    st = np.array([port.rng_seed(1234)], np.uint64)
    dT, dK, dP = per_seq(1, 0.8, 40, 0.95)
    out = ctx.sample_batch(to_dev(x), dT, dK, dP, u64_to_dev(st), rep=to_dev(np.array([1.1], np.float32)),
                           history=to_dev(h), history_len=to_dev(np.array([64], np.int32)), kept_cap=40)
    dense = ctx.scatter_kept(out, V).cpu().numpy()[0]
    o = port.sample_batch(x, 0.8, 40, 0.95, st, rep=1.1, hist=h, detail_cap=40)
    exp = np.zeros(V, np.float32)
    exp[o["detail_idx"][0]] = o["detail_prob"][0]
    assert int(out["tokens"][0]) == int(o["tokens"][0])
    assert np.array_equal(np.nonzero(dense)[0], np.nonzero(exp)[0])
    assert rel_err(dense[exp > 0], exp[exp > 0]) <= 1e-5 and abs(dense.sum() - 1.0) < 1e-5


def test_invalid_arguments_are_refused(ctx):
    import torch
    x = torch.zeros(4, 100, device="cuda")
    dT, dK, dP = per_seq(2, 0.5, 3, 1.0)
    st = u64_to_dev(np.ones(2, np.uint64))
    with pytest.raises(api.GeistError) as e:
        b = api.Batch()
        api._check(api.lib.geist_b200_sample_batch(ctx.handle, C.byref(b), None))
    assert e.value.status == 2  # GEIST_E_INVALID_ARG
    out = ctx.sample_batch(x, dT, dK, dP, st, rows_per_seq=2)  # fine: separate rng_out
    with pytest.raises(api.GeistError):
        out["_desc"].rng_out = st.data_ptr()  # aliasing rng with rows_per_seq > 1
        ctx.relaunch(out, torch.cuda.current_stream().cuda_stream)

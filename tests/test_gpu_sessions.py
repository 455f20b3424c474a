"""GPU tests of the session layer around the sampler: the pending-token protocol
(arch.c:133-161), peek_logits staging (geist_util.h:195-211), per-session soft cap and
mask, and the n-gram drafter with its lazy gate (session.c:437-513, :540-591)."""
import numpy as np
import pytest

import oracle
from geistlib_b200 import api
from helpers import normal_logits, rel_err, to_dev
from test_gpu_prologue import mask_words

pytestmark = pytest.mark.gpu
port = oracle.port


def test_pending_token_protocol(ctx):
    V, N = 32000, 5
    bt = api.Batcher(ctx, V, 8, max_history=16)
    sess = [bt.open(temperature=0.8, top_k=40, top_p=1.0, seed=10 + i) for i in range(N)]
    state = [port.rng_seed(10 + i) for i in range(N)]
    x0, x1, x2 = (normal_logits(N, V, 2.5, 70 + j) for j in range(3))
    assert all(bt.peek_next_token(s) == -1 for s in sess)
    assert bt.peek_logits(sess[0]) is None
    with pytest.raises(api.GeistError, match="GEIST_E_INVALID_STATE"):
        bt.decode_step(sess, to_dev(x1))
    # the row behind the prompt: sampled, pending, returned
    t0 = bt.step(sess, to_dev(x0))
    o0 = port.sample_batch(x0, 0.8, 40, 1.0, state)
    assert np.array_equal(t0, o0["tokens"])
    assert [bt.peek_next_token(s) for s in sess] == t0.tolist()
    # decode_step: return, then advance
    prev = bt.decode_step(sess, x1)  # host logits
    assert np.array_equal(prev, t0)
    o1 = port.sample_batch(x1, 0.8, 40, 1.0, o0["rng_state"])
    assert [bt.peek_next_token(s) for s in sess] == o1["tokens"].tolist()
    # a failed call changes nothing: one session of the call has nothing pending
    extra = bt.open(temperature=0.0)
    with pytest.raises(api.GeistError, match="GEIST_E_INVALID_STATE"):
        bt.decode_step(sess[:2] + [extra], to_dev(x2[:3]))
    assert [bt.peek_next_token(s) for s in sess] == o1["tokens"].tolist()
    assert bt.get_rng(sess[0]) == int(o1["rng_state"][0])
    prev = bt.decode_step(sess, to_dev(x2))
    assert np.array_equal(prev, o1["tokens"])
    bt.reset(sess[0])
    assert bt.peek_next_token(sess[0]) == -1 and bt.peek_next_token(sess[1]) >= 0
    assert bt.peek_next_token(99) == -1
    bt.close()


def test_verify_takes_the_pending_token_as_first_fed(ctx):
    V, N, k = 32000, 4, 4
    x0 = normal_logits(N, V, 2.5, 5)
    xv = normal_logits(N * k, V, 2.5, 6)
    xv[:, :3] += 8.0
    drafts = np.random.default_rng(3).integers(0, V, (N, k)).astype(np.int32)
    res = []
    for explicit in (True, False):
        bt = api.Batcher(ctx, V, 8, max_history=32)
        sess = [bt.open(temperature=0.9, top_k=30, top_p=1.0, seed=40 + i, rep=1.2) for i in range(N)]
        pend = bt.step(sess, to_dev(x0))
        fed = drafts.copy()
        fed[:, 0] = pend if explicit else -1
        res.append(bt.verify(sess, fed, to_dev(xv)))
        assert all(bt.peek_next_token(s) == -1 for s in sess), "the last emitted token still has to go through the model"
        if not explicit:
            assert np.array_equal(res[-1][2][:, 0], pend)
            with pytest.raises(api.GeistError, match="GEIST_E_INVALID_STATE"):
                bt.verify(sess, fed, to_dev(xv))  # nothing pending any more
        bt.close()
    for a, b in zip(*res):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("on_host", [False, True])
def test_peek_logits_staging(ctx, on_host):
    V, N = 50257, 3
    bt = api.Batcher(ctx, V, 4)
    sess = [bt.open(temperature=0.0), bt.open(temperature=0.7, top_k=20), bt.open(temperature=1.0)]
    bt.set_softcap(sess[1], 30.0)
    x = normal_logits(N, V, 15.0, 8)
    dx = to_dev(x)
    tok = bt.step(sess, x if on_host else dx)
    rows = [bt.peek_logits(s).copy() for s in sess]
    assert np.array_equal(rows[0].view(np.uint32), x[0].view(np.uint32))
    assert np.array_equal(rows[2].view(np.uint32), x[2].view(np.uint32))
    capped = port.softcap(x[1], 30.0)
    assert rel_err(rows[1], capped) <= 1e-5 and np.abs(rows[1]).max() <= 30.0
    # the sampler saw the same capped row
    o = port.sample_batch(capped[None, :], 0.7, 20, 1.0, [port.rng_seed(0xCAFEBABE1234)])
    assert tok[1] == o["tokens"][0]
    assert tok[0] == int(x[0].argmax())
    # a greedy session with a cap: the sampler skips it (monotone), value consumers get it (arch.c:185-195)
    bt.set_softcap(sess[0], 20.0)
    assert rel_err(bt.peek_logits(sess[0]), port.softcap(x[0], 20.0)) <= 1e-5
    bt.reset(sess[2])
    assert bt.peek_logits(sess[2]) is None
    with pytest.raises(api.GeistError):
        bt.set_softcap(sess[0], -1.0)
    bt.close()


def test_session_mask_and_softcap_through_the_batcher(ctx):
    V, N = 32000, 6
    bt = api.Batcher(ctx, V, 8, max_history=8)
    cfg = [(0.0, 0, 1.0), (0.8, 40, 1.0), (0.9, 0, 0.7), (1.0, 0, 1.0), (0.8, 40, 1.0), (0.0, 0, 1.0)]
    sess = [bt.open(temperature=T, top_k=K, top_p=P, seed=60 + i) for i, (T, K, P) in enumerate(cfg)]
    allowed = np.random.default_rng(9).random((N, V)) < 0.2
    words = mask_words(allowed)
    for i in (0, 1, 2, 3):
        bt.set_logit_mask(sess[i], words[i])
    bt.set_softcap(sess[1], 30.0)
    bt.set_softcap(sess[4], 30.0)
    x = normal_logits(N, V, 10.0, 61)
    got = bt.step(sess, to_dev(x))
    for i, (T, K, P) in enumerate(cfg):
        row = x[i].copy()
        if i in (1, 4):
            row = port.softcap(row, 30.0)
        if i < 4:
            row = np.where(allowed[i], row, -np.inf).astype(np.float32)
            assert allowed[i, got[i]]
        o = port.sample_batch(row[None, :], T, K, P, [port.rng_seed(60 + i)])
        assert got[i] == o["tokens"][0], i
    # lifting the mask
    bt.set_logit_mask(sess[0], None)
    got = bt.step(sess[:1], to_dev(x[:1]))
    assert got[0] == int(x[0].argmax())
    with pytest.raises(api.GeistError):
        bt.set_logit_mask(sess[1], words[1][:10])
    bt.close()


# ------------------------------------------------------------------ drafter --

def test_draft_ngram_equals_the_checker(ctx):
    rng = np.random.default_rng(77)
    n, stride = 300, 96
    h = np.zeros((n, stride), np.int32)
    hl = rng.integers(0, stride + 1, n).astype(np.int32)
    hl[:4] = [0, 1, 2, stride]
    seeds = np.empty(n, np.int32)
    for i in range(n):
        voc = int(rng.integers(1, 7))
        h[i, :hl[i]] = rng.integers(0, voc, hl[i])
        seeds[i] = rng.integers(0, voc)
    for k_max, ms in [(1, 4), (2, 4), (8, 4), (16, 4), (16, 8), (5, 1), (7, 20)]:
        d, nd, L = api.draft_ngram(ctx, h, hl, seeds, k_max, ms)
        for i in range(n):
            od, oL = port.propose_drafts(h[i, :hl[i]], int(seeds[i]), k_max, ms)
            assert nd[i] == od.size and L[i] == oL and np.array_equal(d[i, :nd[i]], od), (k_max, ms, i)
            assert (d[i, nd[i]:] == -1).all()


def test_draft_ngram_long_history(ctx):
    """A history of thousands of tokens over a small alphabet: many places match, the reduction must pick
    the one the reference's newest-first walk picks."""
    rng = np.random.default_rng(5)
    h = rng.integers(0, 3, (4, 6000)).astype(np.int32)
    hl = np.array([6000, 5999, 4097, 33], np.int32)
    seeds = np.array([0, 1, 2, 0], np.int32)
    d, nd, L = api.draft_ngram(ctx, h, hl, seeds, 16, 8)
    for i in range(4):
        od, oL = port.propose_drafts(h[i, :hl[i]], int(seeds[i]), 16, 8)
        assert nd[i] == od.size and L[i] == oL and np.array_equal(d[i, :nd[i]], od)


def test_draft_ngram_argument_checks(ctx):
    h = np.zeros((1, 8), np.int32)
    one = np.array([4], np.int32)
    for k_max, cap in [(0, 4), (17, 18), (4, 4)]:  # session.c:540-549
        with pytest.raises(api.GeistError, match="GEIST_E_INVALID_ARG"):
            api.draft_ngram(ctx, h, one, one, k_max, 4, out_capacity=cap)
    with pytest.raises(api.GeistError, match="GEIST_E_INVALID_ARG"):
        api.draft_ngram(ctx, h, np.array([9], np.int32), one, 4)


def test_batcher_propose_drafts_over_the_history_ring(ctx):
    V, HM = 1000, 40
    bt = api.Batcher(ctx, V, 8, max_history=HM)
    rng = np.random.default_rng(12)
    # session 0: a repeating pattern, so the context recurs with L = 4; session 1: only the seed recurs (L = 1: gated);
    # session 2: a prompt longer than the ring (its last HM tokens count); session 3: nothing pending
    pat = [7, 8, 9, 10, 11, 12]
    prompts = [np.array(pat * 4 + [7, 8, 9], np.int32),
               np.array([500, 3, 4, 5, 6, 501, 502, 503], np.int32),
               rng.integers(0, 3, 100).astype(np.int32),
               np.array([1, 2, 3], np.int32)]
    nxt = [10, 3, int(rng.integers(0, 3)), 0]  # what the model "predicts" for each
    sess = [bt.open(temperature=0.0) for _ in prompts]
    for s, p in zip(sess, prompts):
        bt.push_history(s, p)
    x = np.full((3, V), -5.0, np.float32)
    for i in range(3):
        x[i, nxt[i]] = 5.0
    for append in (True, False):  # the sampler may or may not have appended the pending token to the ring
        if append is False:
            for s, p in zip(sess, prompts):
                bt.reset(s)
                bt.push_history(s, p)
        tok = bt.step(sess[:3], to_dev(x), append_history=append)
        assert tok.tolist() == nxt[:3]
        with pytest.raises(api.GeistError, match="GEIST_E_INVALID_STATE"):
            bt.propose_drafts(sess, 8)
        d, nd, L = bt.propose_drafts(sess[:3], 8)
        for i in range(3):
            # with the pending token in the ring the window holds one prompt token less
            hist = prompts[i][-(HM - 1 if append else HM):]
            od, oL = port.propose_drafts(hist, nxt[i], 8, 4)
            gated = oL < 2 or od.size <= 1
            assert L[i] == oL
            assert nd[i] == (1 if gated else od.size)
            assert np.array_equal(d[i, :nd[i]], od[:nd[i]]) and (d[i, nd[i]:] == -1).all()
        assert L[0] == 4 and nd[0] == 8 and d[0].tolist()[:8] == [10, 11, 12, 7, 8, 9, 10, 11]
        assert L[1] == 1 and nd[1] == 1
    with pytest.raises(api.GeistError, match="GEIST_E_INVALID_ARG"):
        bt.propose_drafts(sess[:3], 17)
    with pytest.raises(api.GeistError, match="GEIST_E_INVALID_ARG"):
        bt.propose_drafts(sess[:3], 8, out_capacity=8)
    bt.close()

"""The entry point that allocates nothing (greedy argmax with the scratch built into the
library), called through the C ABI and compared with the context-based entry point.
Collected last on purpose: it must pass alone and after every other test has used the
device, and two calls in a row must both be right (the scratch is shared by all calls)."""
import ctypes as C

import numpy as np
import pytest

from geistlib_b200 import api
from helpers import normal_logits, per_seq, to_dev, u64_to_dev

pytestmark = pytest.mark.gpu


def static_argmax(x_dev, n_vocab=None, stride=None, out=None):
    import torch
    rows = x_dev.shape[0]
    if out is None:
        out = torch.full((rows,), -7, dtype=torch.int32, device=x_dev.device)
    st = torch.cuda.current_stream(x_dev.device).cuda_stream
    api._check(api.lib.geist_b200_argmax_rows_static(x_dev.device.index or 0, x_dev.data_ptr(), stride or x_dev.stride(0), rows,
                                                     n_vocab or x_dev.shape[1], out.data_ptr(), C.c_void_p(st)))
    torch.cuda.synchronize(x_dev.device)
    return out.cpu().numpy()


def context_argmax(ctx, x_dev):
    rows = x_dev.shape[0]
    dT, dK, dP = per_seq(rows, 0.0, 0, 1.0)
    out = ctx.sample_batch(x_dev, dT, dK, dP, u64_to_dev(np.ones(rows, np.uint64)))
    assert int(out["status"].max()) == 0
    return out["tokens"].cpu().numpy()


def test_two_calls_in_a_row_equal_the_context_entry_point(ctx):
    import torch
    V = 128256
    xa = normal_logits(256, V, 2.5, 1)
    xa[3, 100] = xa[3, 90000] = xa[3].max() + 1.0  # tie across slices: lowest id
    xa[4, :] = -np.inf                              # sampler.c:52-62 keeps index 0
    xa[5, :] = 0.5
    xb = normal_logits(64, 151936, 3.0, 2)
    da, db = to_dev(xa), to_dev(xb)
    oa = torch.empty(256, dtype=torch.int32, device="cuda")
    ob = torch.empty(64, dtype=torch.int32, device="cuda")
    first = static_argmax(da, out=oa)   # the first call on a device also does the set-up
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    second = static_argmax(db, out=ob)  # other shape, same scratch, directly after
    third = static_argmax(da, out=oa)
    assert torch.cuda.mem_get_info()[0] == free_before, "the calls took device memory"
    assert np.array_equal(first, context_argmax(ctx, da))
    assert np.array_equal(second, context_argmax(ctx, db))
    assert np.array_equal(third, first)
    assert first[3] == 100 and first[4] == 0 and first[5] == 0
    assert np.array_equal(first, xa.argmax(axis=1)) and np.array_equal(second, xb.argmax(axis=1))


@pytest.mark.parametrize("V", [1, 3, 33, 4099, 8192, 8193, 50257])
def test_edge_sizes_and_unaligned_rows(ctx, V):
    import torch
    rows = 7
    x = normal_logits(rows, V, 3.0, 40 + V)
    x[1, V // 2:] = x[1].max() + 2.0
    d = to_dev(x)
    assert np.array_equal(static_argmax(d), context_argmax(ctx, d))
    # rows that start off a 16-byte boundary take the scalar loads
    buf = torch.zeros(rows * (V + 3) + 1, dtype=torch.float32, device="cuda")
    view = buf[1:1 + rows * (V + 3)].view(rows, V + 3)[:, :V]
    view.copy_(d)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    api._check(api.lib.geist_b200_argmax_rows_static(0, view.data_ptr(), V + 3, rows, V, out.data_ptr(), None))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), x.argmax(axis=1))


def test_sizes_beyond_the_built_in_scratch_are_refused(ctx):
    import torch
    x = torch.zeros(8, 16, device="cuda")
    out = torch.empty(8, dtype=torch.int32, device="cuda")
    lib = api.lib
    # 4097 rows, and 4096 rows of a vocabulary that needs 17 slices per row
    for rows, V in [(4097, 16), (4096, 8192 * 16 + 1)]:
        rc = lib.geist_b200_argmax_rows_static(0, x.data_ptr(), V, rows, V, out.data_ptr(), None)
        assert rc == 2 and b"exceed the built-in scratch" in lib.geist_b200_errmsg()
    assert lib.geist_b200_argmax_rows_static(0, None, 16, 8, 16, out.data_ptr(), None) == 2
    assert lib.geist_b200_argmax_rows_static(0, x.data_ptr(), 8, 8, 16, out.data_ptr(), None) == 2  # stride < n_vocab
    # the largest batch that fits at V = 128256 (16 slices per row)
    big = torch.randn(4096, 128256, device="cuda")
    got = static_argmax(big)
    assert np.array_equal(got, big.argmax(dim=1).cpu().numpy())

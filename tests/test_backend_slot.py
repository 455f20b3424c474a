"""The backend operator slot `argmax_f32` with the reference's own signature
(include/geist_backend.h:414-421) and its load-time probe (:276-326).

libgeist_b200_backend.so is geistlib_b200/csrc/geist_b200_backend.c compiled against the geistlib
headers; its geist_b200_slot_contract_check() runs the reference's contract test
(tests/test_fused_probe_agreement_unit.c:139-160: a [1, 256] row with a spike at 77 must give
GEIST_OK and 77 once the probe said yes) through the function pointers of a `struct
geist_backend_fused`, plus offset views, ties and the refusals that send the arch to its host scan."""
import ctypes as C
import threading

import numpy as np
import pytest

from geistlib_b200 import PKG_DIR, api

BACKEND_LIB = PKG_DIR / "libgeist_b200_backend.so"
needs_glue = pytest.mark.skipif(not BACKEND_LIB.exists(), reason="the glue is built where the geistlib headers are (make -C geistlib_b200/csrc backend)")


@needs_glue
def test_glue_exports_the_slot_functions():
    lib = C.CDLL(str(BACKEND_LIB))
    for name in ("geist_b200_fused_supported", "geist_b200_fused_argmax_f32", "geist_b200_fused", "geist_b200_slot_contract_check",
                 "geist_b200_buffer_create", "geist_b200_buffer_map", "geist_b200_buffer_unmap", "geist_b200_buffer_destroy"):
        assert hasattr(lib, name), name


@needs_glue
@pytest.mark.gpu
def test_slot_contract_through_the_fused_table():
    lib = C.CDLL(str(BACKEND_LIB))
    lib.geist_b200_slot_contract_check.restype = C.c_int
    lib.geist_b200_slot_contract_check.argtypes = [C.c_int, C.c_char_p, C.c_size_t]
    detail = C.create_string_buffer(4096)
    fails = lib.geist_b200_slot_contract_check(0, detail, len(detail))
    assert fails == 0, detail.value.decode()


@pytest.mark.gpu
def test_argmax_f32_from_two_threads_on_one_context():
    """Calls on one context may come from several threads: each gets its own row's index."""
    import torch
    ctx = api.Context(0)
    n = 50000
    rows, want = [], []
    rng = np.random.default_rng(3)
    for t in range(2):
        x = rng.standard_normal(n).astype(np.float32)
        w = int(rng.integers(0, n))
        x[w] = 50.0 + t
        rows.append(torch.from_numpy(x).cuda())
        want.append(w)
    torch.cuda.synchronize()
    bad = []

    def work(t):
        out = C.c_int32(-1)
        for _ in range(200):
            s = api.lib.geist_b200_argmax_f32(ctx.handle, C.c_void_p(rows[t].data_ptr()), n, C.byref(out))
            if s != api.GEIST_OK or out.value != want[t]:
                bad.append((t, s, out.value))
                return

    th = [threading.Thread(target=work, args=(t,)) for t in range(2)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not bad, bad
    ctx.close()

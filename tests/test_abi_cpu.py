"""No-GPU checks of the drop-in boundary: the shared library loads, exports every
symbol include/geist_b200.h declares, its struct layouts match the ctypes view,
and the pure-host entry points behave like the reference's."""
import ctypes as C
import re
from pathlib import Path

import numpy as np

import oracle
from geistlib_b200 import HEADER_PATH, LIB_PATH, api


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER_PATH.read_text(), flags=re.S)
    names = set(re.findall(r"\b(geist_[a-z0-9_]+)\s*\(", text))
    return {n for n in names if not n.endswith("_t")}


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(str(LIB_PATH))
    names = declared_functions()
    assert len(names) >= 30
    for n in sorted(names):
        assert hasattr(lib, n), f"{n} is declared in include/geist_b200.h but not exported"
    assert names == set(api.PROTOTYPES), names ^ set(api.PROTOTYPES)


def test_host_generator_is_the_reference_stream():
    for seed in (0, 1, 7, 1234, 0xCAFEBABE1234):
        r = api.rng_seed(seed)
        assert r.state == oracle.port.rng_seed(seed)
        u64, unit = oracle.port.rng_stream(seed, 8)
        got = [api.lib.geist_rng_next_u64(C.byref(r)) for _ in range(8)]
        assert got == [int(v) for v in u64]
        r = api.rng_seed(seed)
        gotf = np.array([api.lib.geist_rng_next_unit(C.byref(r)) for _ in range(8)], np.float32)
        assert np.array_equal(gotf.view(np.uint32), unit.view(np.uint32))


def test_session_opts_layout_matches_reference_header():
    # include/geist.h:209-247 on LP64: size_t, float, float, int, (pad), uint64, ptr, enum, (pad), size_t
    assert C.sizeof(api.SessionOpts) == 56
    assert api.SessionOpts.temperature.offset == 8
    assert api.SessionOpts.top_p.offset == 12
    assert api.SessionOpts.top_k.offset == 16
    assert api.SessionOpts.random_seed.offset == 24
    assert C.sizeof(api.Rng) == 8 and C.sizeof(api.Workspace) == 16


def test_calls_without_a_device_fail_loudly_not_silently():
    """No GPU here: entry points must report an error status, never compute on the CPU."""
    import torch
    if torch.cuda.is_available():
        return
    h = C.c_void_p()
    st = api.lib.geist_b200_ctx_create(0, C.byref(h))
    assert st != api.GEIST_OK and not h.value
    assert len(api.lib.geist_b200_errmsg()) > 0
    row = np.zeros(16, np.float32)
    assert api.sampler_argmax(row) == -1

"""ctypes bindings of the two CPU checkers. Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")


def build(quiet: bool = True) -> None:
    """Compile liboracle.so and, when the reference tree is present, oracle/_ref."""
    subprocess.run(["make", "-C", str(HERE)], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _opt(a, dtype):
    if a is None:
        return None
    a = np.ascontiguousarray(a, dtype=dtype)
    return a.ctypes.data_as(C.c_void_p)


class Port:
    """The C restatement (oracle/sampler_oracle.c)."""

    def __init__(self, path: Path):
        L = self.lib = C.CDLL(str(path))
        L.orc_rng_seed.restype = C.c_uint64
        L.orc_rng_seed.argtypes = [C.c_uint64]
        L.orc_rng_next.restype = C.c_uint64
        L.orc_rng_next.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_rng_unit.restype = C.c_float
        L.orc_rng_unit.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_rng_advance.restype = C.c_uint64
        L.orc_rng_advance.argtypes = [C.c_uint64, C.c_size_t]
        L.orc_argmax.restype = C.c_int32
        L.orc_argmax.argtypes = [_f32p, C.c_size_t]
        L.orc_apply_penalties.restype = None
        L.orc_apply_penalties.argtypes = [_f32p, C.c_size_t, _i32p, C.c_size_t, C.c_float, C.c_float, C.c_float]
        L.orc_softmax.restype = C.c_double
        L.orc_softmax.argtypes = [_f32p, C.c_size_t, C.c_float, _f32p]
        L.orc_sampler_call.restype = C.c_int32
        L.orc_sampler_call.argtypes = [C.c_int, _f32p, C.c_size_t, C.c_float, C.c_int, C.c_float, C.POINTER(C.c_uint64)]
        L.orc_sample_batch.restype = C.c_int
        L.orc_sample_batch.argtypes = [
            _f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
            _f32p, _i32p, _f32p,
            C.c_void_p, C.c_void_p, C.c_void_p,
            C.c_void_p, C.c_size_t, C.c_void_p,
            C.c_void_p, C.c_size_t,
            _u64p, _i32p, C.c_void_p,
            C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_spec_accept.restype = C.c_size_t
        L.orc_spec_accept.argtypes = [C.c_size_t, _i32p, _i32p, _i32p, C.POINTER(C.c_int32)]
        L.orc_merge_candidates.restype = None
        L.orc_merge_candidates.argtypes = [C.c_size_t, _f32p, _i32p, C.c_size_t, _f32p, _i32p]
        L.orc_sample_ordered.restype = C.c_int32
        L.orc_sample_ordered.argtypes = [C.c_size_t, _f32p, _i32p, C.c_float, C.POINTER(C.c_uint64)]
        L.orc_softcap.restype = None
        L.orc_softcap.argtypes = [C.c_size_t, _f32p, C.c_float]
        L.orc_propose_drafts_ngram.restype = C.c_size_t
        L.orc_propose_drafts_ngram.argtypes = [_i32p, C.c_size_t, C.c_int32, C.c_size_t, C.c_size_t, _i32p, C.POINTER(C.c_size_t)]

    def softcap(self, logits, c: float):
        """tanhf(x / c) * c of every entry (a copy)."""
        out = np.array(logits, dtype=np.float32, copy=True, order="C")
        self.lib.orc_softcap(out.size, out.reshape(-1), c)
        return out

    def propose_drafts(self, history, seed: int, k_max: int, max_suffix: int = 4):
        """(drafts incl. the seed, match length) of the n-gram drafter."""
        return _drafts(self.lib.orc_propose_drafts_ngram, history, seed, k_max, max_suffix)

    # -- generator
    def rng_seed(self, seed: int) -> int:
        return int(self.lib.orc_rng_seed(seed))

    def rng_stream(self, seed: int, n: int):
        s = C.c_uint64(self.rng_seed(seed))
        u64 = np.array([self.lib.orc_rng_next(C.byref(s)) for _ in range(n)], dtype=np.uint64)
        s = C.c_uint64(self.rng_seed(seed))
        unit = np.array([self.lib.orc_rng_unit(C.byref(s)) for _ in range(n)], dtype=np.float32)
        return u64, unit

    def rng_advance(self, state: int, n: int) -> int:
        return int(self.lib.orc_rng_advance(state, n))

    # -- pieces
    def argmax(self, row) -> int:
        row = np.ascontiguousarray(row, np.float32)
        return int(self.lib.orc_argmax(row, row.size))

    def apply_penalties(self, row, hist, rep=1.0, freq=0.0, pres=0.0):
        out = np.array(row, dtype=np.float32, copy=True)
        hist = np.ascontiguousarray(hist, np.int32)
        if hist.size:
            self.lib.orc_apply_penalties(out, out.size, hist, hist.size, rep, freq, pres)
        return out

    def softmax(self, row, T):
        row = np.ascontiguousarray(row, np.float32)
        probs = np.empty_like(row)
        s = self.lib.orc_softmax(row, row.size, T, probs)
        return probs, float(s)

    def sampler_call(self, which: str, row, T=1.0, top_k=0, top_p=1.0, state=1):
        row = np.ascontiguousarray(row, np.float32)
        s = C.c_uint64(state)
        w = {"temperature": 0, "top_k": 1, "top_p": 2}[which]
        tok = self.lib.orc_sampler_call(w, row, row.size, T, top_k, top_p, C.byref(s))
        return int(tok), int(s.value)

    def sample_batch(self, logits, temperature, top_k, top_p, rng_state, rows_per_seq=1,
                     rep=None, freq=None, pres=None, hist=None, hist_len=None, extra=None,
                     want_logits=False, detail_cap=0, nthreads=0):
        """logits [S*R, V]; per-sequence parameters of length S. Returns a dict."""
        logits = np.ascontiguousarray(logits, np.float32)
        n_rows, V = logits.shape
        R = rows_per_seq
        S = n_rows // R
        assert S * R == n_rows
        T = np.ascontiguousarray(np.broadcast_to(np.asarray(temperature, np.float32), (S,)))
        K = np.ascontiguousarray(np.broadcast_to(np.asarray(top_k, np.int32), (S,)))
        P = np.ascontiguousarray(np.broadcast_to(np.asarray(top_p, np.float32), (S,)))
        st = np.array(np.broadcast_to(np.asarray(rng_state, np.uint64), (S,)), dtype=np.uint64, copy=True)
        tokens = np.empty(n_rows, np.int32)
        keep = []

        def opt(a, dt, shape=None):
            if a is None:
                return None
            a = np.ascontiguousarray(np.broadcast_to(np.asarray(a, dt), shape) if shape else np.asarray(a, dt))
            keep.append(a)
            return a.ctypes.data_as(C.c_void_p)

        hist_stride = 0
        if hist is not None:
            hist = np.ascontiguousarray(hist, np.int32)
            hist_stride = hist.shape[1]
            if hist_len is None:
                hist_len = np.full(S, hist.shape[1], np.int32)
        extra_stride = 0
        if extra is not None:
            extra = np.ascontiguousarray(extra, np.int32)
            extra_stride = extra.shape[1]
            if hist is None:
                hist = np.zeros((S, 1), np.int32)
                hist_stride = 1
                hist_len = np.zeros(S, np.int32)
        out_logits = np.empty((n_rows, V), np.float32) if want_logits else None
        dn = np.zeros(n_rows, np.int32) if detail_cap else None
        di = np.full((n_rows, detail_cap), -1, np.int32) if detail_cap else None
        dp = np.zeros((n_rows, detail_cap), np.float32) if detail_cap else None
        rc = self.lib.orc_sample_batch(
            logits, S, R, V, V, T, K, P,
            opt(rep, np.float32, (S,)), opt(freq, np.float32, (S,)), opt(pres, np.float32, (S,)),
            opt(hist, np.int32), hist_stride, opt(hist_len, np.int32, (S,)),
            opt(extra, np.int32), extra_stride,
            st, tokens,
            out_logits.ctypes.data_as(C.c_void_p) if want_logits else None,
            detail_cap,
            dn.ctypes.data_as(C.c_void_p) if detail_cap else None,
            di.ctypes.data_as(C.c_void_p) if detail_cap else None,
            dp.ctypes.data_as(C.c_void_p) if detail_cap else None,
            nthreads)
        if rc != 0:
            raise MemoryError("oracle allocation failed")
        return {"tokens": tokens, "rng_state": st, "logits": out_logits,
                "detail_n": dn, "detail_idx": di, "detail_prob": dp}

    def spec_accept(self, fed, verify_out):
        fed = np.ascontiguousarray(fed, np.int32)
        vo = np.ascontiguousarray(verify_out, np.int32)
        k = fed.size
        em = np.empty(k + 1, np.int32)
        a = C.c_int32(0)
        n = self.lib.orc_spec_accept(k, fed, vo, em, C.byref(a))
        return int(a.value), em[:n].copy()

    def merge_candidates(self, val, gid, k):
        val = np.ascontiguousarray(val, np.float32).ravel()
        gid = np.ascontiguousarray(gid, np.int32).ravel()
        k = min(k, val.size)
        ov = np.empty(k, np.float32)
        og = np.empty(k, np.int32)
        self.lib.orc_merge_candidates(val.size, val, gid, k, ov, og)
        return ov, og

    def sample_ordered(self, val, gid, T, state):
        val = np.ascontiguousarray(val, np.float32)
        gid = np.ascontiguousarray(gid, np.int32)
        s = C.c_uint64(state)
        tok = self.lib.orc_sample_ordered(val.size, val, gid, T, C.byref(s))
        return int(tok), int(s.value)


class Ref:
    """The reference's own sampler.c behind oracle/ref_harness.c."""

    def __init__(self, path: Path):
        L = self.lib = C.CDLL(str(path))
        L.ref_rng_seed_state.restype = C.c_uint64
        L.ref_rng_seed_state.argtypes = [C.c_uint64]
        L.ref_rng_vectors.restype = None
        L.ref_rng_vectors.argtypes = [C.c_uint64, C.c_size_t, _u64p, _f32p]
        L.ref_rng_advance.restype = C.c_uint64
        L.ref_rng_advance.argtypes = [C.c_uint64, C.c_size_t]
        L.ref_sample.restype = C.c_int
        L.ref_sample.argtypes = [_f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                 _f32p, _i32p, _f32p, _u64p, _i32p, C.c_int]
        L.ref_argmax.restype = C.c_int32
        L.ref_argmax.argtypes = [C.c_size_t, _f32p]
        L.ref_temperature.restype = C.c_int32
        L.ref_temperature.argtypes = [C.c_size_t, _f32p, C.c_float, C.POINTER(C.c_uint64)]
        L.ref_top_k.restype = C.c_int32
        L.ref_top_k.argtypes = [C.c_size_t, _f32p, C.c_int, C.c_float, C.POINTER(C.c_uint64)]
        L.ref_top_p.restype = C.c_int32
        L.ref_top_p.argtypes = [C.c_size_t, _f32p, C.c_float, C.c_float, C.POINTER(C.c_uint64)]
        L.ref_softmax.restype = C.c_double
        L.ref_softmax.argtypes = [C.c_size_t, _f32p, C.c_float, _f32p]
        L.ref_topk_detail.restype = C.c_int
        L.ref_topk_detail.argtypes = [C.c_size_t, _f32p, C.c_int, C.c_float, _i32p, _f32p, C.c_void_p, C.POINTER(C.c_double)]
        L.ref_topp_detail.restype = C.c_long
        L.ref_topp_detail.argtypes = [C.c_size_t, _f32p, C.c_float, C.c_float, C.c_size_t, _i32p, _f32p, _f32p, C.POINTER(C.c_double)]
        if hasattr(L, "ref_softcap"):
            L.ref_softcap.restype = None
            L.ref_softcap.argtypes = [C.c_size_t, _f32p, C.c_float]

    def softcap(self, logits, c: float):
        out = np.array(logits, dtype=np.float32, copy=True, order="C")
        self.lib.ref_softcap(out.size, out.reshape(-1), c)
        return out

    def rng_seed(self, seed: int) -> int:
        return int(self.lib.ref_rng_seed_state(seed))

    def rng_stream(self, seed: int, n: int):
        u = np.empty(n, np.uint64)
        f = np.empty(n, np.float32)
        self.lib.ref_rng_vectors(seed, n, u, f)
        return u, f

    def rng_advance(self, state: int, n: int) -> int:
        return int(self.lib.ref_rng_advance(state, n))

    def argmax(self, row) -> int:
        row = np.ascontiguousarray(row, np.float32)
        return int(self.lib.ref_argmax(row.size, row))

    def sampler_call(self, which: str, row, T=1.0, top_k=0, top_p=1.0, state=1):
        row = np.ascontiguousarray(row, np.float32)
        s = C.c_uint64(state)
        if which == "temperature":
            tok = self.lib.ref_temperature(row.size, row, T, C.byref(s))
        elif which == "top_k":
            tok = self.lib.ref_top_k(row.size, row, top_k, T, C.byref(s))
        else:
            tok = self.lib.ref_top_p(row.size, row, top_p, T, C.byref(s))
        return int(tok), int(s.value)

    def softmax(self, row, T):
        row = np.ascontiguousarray(row, np.float32)
        probs = np.empty_like(row)
        s = self.lib.ref_softmax(row.size, row, T, probs)
        return probs, float(s)

    def sample(self, logits, temperature, top_k, top_p, rng_state, rows_per_seq=1, nthreads=0):
        logits = np.ascontiguousarray(logits, np.float32)
        n_rows, V = logits.shape
        R = rows_per_seq
        S = n_rows // R
        T = np.ascontiguousarray(np.broadcast_to(np.asarray(temperature, np.float32), (S,)))
        K = np.ascontiguousarray(np.broadcast_to(np.asarray(top_k, np.int32), (S,)))
        P = np.ascontiguousarray(np.broadcast_to(np.asarray(top_p, np.float32), (S,)))
        st = np.array(np.broadcast_to(np.asarray(rng_state, np.uint64), (S,)), dtype=np.uint64, copy=True)
        tokens = np.empty(n_rows, np.int32)
        rc = self.lib.ref_sample(logits, S, R, V, V, T, K, P, st, tokens, nthreads)
        if rc != 0:
            raise MemoryError("reference workspace allocation failed")
        return {"tokens": tokens, "rng_state": st}

    def topk_detail(self, row, top_k, T):
        row = np.ascontiguousarray(row, np.float32)
        k = min(top_k, 8192)
        idx = np.empty(max(k, 1), np.int32)
        prob = np.empty(max(k, 1), np.float32)
        s = C.c_double(0)
        n = self.lib.ref_topk_detail(row.size, row, top_k, T, idx, prob, None, C.byref(s))
        return idx[:n].copy(), prob[:n].copy(), float(s.value)

    def topp_detail(self, row, top_p, T, cap=None):
        row = np.ascontiguousarray(row, np.float32)
        cap = cap or row.size
        idx = np.empty(cap, np.int32)
        pn = np.empty(cap, np.float32)
        pq = np.empty(cap, np.float32)
        s = C.c_double(0)
        n = self.lib.ref_topp_detail(row.size, row, top_p, T, cap, idx, pn, pq, C.byref(s))
        m = min(n, cap)
        return int(n), idx[:m].copy(), pn[:m].copy(), pq[:m].copy(), float(s.value)


def _drafts(fn, history, seed, k_max, max_suffix):
    h = np.ascontiguousarray(history, np.int32)
    out = np.full(max(int(k_max), 1), -1, np.int32)
    L = C.c_size_t(0)
    hp = h if h.size else np.zeros(1, np.int32)
    n = int(fn(hp, h.size, int(seed), int(k_max), int(max_suffix), out, C.byref(L)))
    return out[:n].copy(), int(L.value)


class RefDrafter:
    """The reference's own propose_drafts_ngram (session.c:437-513) behind oracle/ref_drafter_harness.c."""

    def __init__(self, path: Path):
        L = self.lib = C.CDLL(str(path))
        L.ref_propose_drafts_ngram.restype = C.c_size_t
        L.ref_propose_drafts_ngram.argtypes = [_i32p, C.c_size_t, C.c_int32, C.c_size_t, C.c_size_t, _i32p, C.POINTER(C.c_size_t)]

    def propose_drafts(self, history, seed: int, k_max: int, max_suffix: int = 4):
        return _drafts(self.lib.ref_propose_drafts_ngram, history, seed, k_max, max_suffix)


def _load(cls, path: Path):
    return cls(path) if path.exists() else None


if not (HERE / "liboracle.so").exists():
    build()
port: Port = Port(HERE / "liboracle.so")
ref = _load(Ref, HERE / "_ref" / "libgeist_ref.so")
ref_release = _load(Ref, HERE / "_ref" / "libgeist_ref_release.so")
ref_drafter = _load(RefDrafter, HERE / "_ref" / "libgeist_ref_drafter.so")

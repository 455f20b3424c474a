"""ctypes view of include/geist_b200.h for torch callers (tests, bench).

Every function below forwards to one C entry point; device buffers are torch
CUDA tensors passed by ``data_ptr()``. Nothing is computed in Python.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import LIB_PATH

if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
        "or `make -C geistlib_b200/csrc` (there is no CPU or PyTorch fallback)")

lib = C.CDLL(str(LIB_PATH))

GEIST_OK = 0
STATUS_NAMES = ["GEIST_OK", "GEIST_E_OOM", "GEIST_E_INVALID_ARG", "GEIST_E_INTERNAL", "GEIST_E_FILE_NOT_FOUND",
                "GEIST_E_IO", "GEIST_E_FORMAT", "GEIST_E_UNSUPPORTED", "GEIST_E_NOT_FOUND", "GEIST_E_BACKEND",
                "GEIST_E_INVALID_STATE", "GEIST_E_TOO_MANY_TOKENS"]
ROW_LOAD_TIMEOUT, ROW_SLOW_PATH, ROW_HIST_OVERFLOW, ROW_KEPT_PARTIAL, ROW_INTERNAL, ROW_RETRY = 1, 2, 4, 8, 16, 32
FINISH_AUTO, FINISH_GREEDY_TOPK, FINISH_GENERAL, FINISH_GREEDY = 0, 1, 2, 3
ROW_INVALID = ROW_LOAD_TIMEOUT | ROW_HIST_OVERFLOW | ROW_INTERNAL
SPEC_KMAX = 16

c_void_p, c_size_t, c_int32, c_float = C.c_void_p, C.c_size_t, C.c_int32, C.c_float


class GeistError(RuntimeError):
    def __init__(self, status: int):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{name}: {lib.geist_b200_errmsg().decode()}")


def _check(status: int) -> None:
    if status != GEIST_OK:
        raise GeistError(status)


class Batch(C.Structure):
    _fields_ = [
        ("logits", c_void_p), ("row_stride", c_size_t), ("n_seq", c_size_t), ("rows_per_seq", c_size_t),
        ("n_vocab", c_size_t),
        ("slot", c_void_p),
        ("temperature", c_void_p), ("top_k", c_void_p), ("top_p", c_void_p),
        ("repetition_penalty", c_void_p), ("frequency_penalty", c_void_p), ("presence_penalty", c_void_p),
        ("history", c_void_p), ("history_stride", c_size_t), ("history_len", c_void_p),
        ("fed_tokens", c_void_p), ("fed_stride", c_size_t),
        ("rng_in", c_void_p), ("rng_out", c_void_p),
        ("tokens", c_void_p), ("row_status", c_void_p),
        ("out_logits", c_void_p),
        ("kept_cap", c_int32), ("kept_n", c_void_p), ("kept_idx", c_void_p), ("kept_prob", c_void_p),
        ("vocab_offset", c_int32),
        ("softcap", c_void_p),
        ("logit_mask", c_void_p), ("logit_mask_stride", c_size_t),
        ("finish_hint", c_int32),
    ]


class Merge(C.Structure):
    _fields_ = [
        ("cand_val", c_void_p), ("cand_gid", c_void_p), ("cand_n", c_void_p),
        ("n_shards", c_size_t), ("n_rows", c_size_t), ("cand_stride", c_size_t),
        ("temperature", c_void_p), ("top_k", c_void_p),
        ("rng_in", c_void_p), ("rng_out", c_void_p),
        ("tokens", c_void_p), ("row_status", c_void_p),
        ("kept_cap", c_int32), ("kept_n", c_void_p), ("kept_idx", c_void_p), ("kept_prob", c_void_p),
    ]


class SessionOpts(C.Structure):
    """struct geist_session_opts, field for field."""
    _fields_ = [("max_seq_len", c_size_t), ("temperature", c_float), ("top_p", c_float), ("top_k", C.c_int),
                ("random_seed", C.c_uint64), ("awq_scales_path", C.c_char_p), ("kv_mode", C.c_int),
                ("m_max", c_size_t)]


class PenaltyOpts(C.Structure):
    _fields_ = [("repetition_penalty", c_float), ("frequency_penalty", c_float), ("presence_penalty", c_float)]


class Rng(C.Structure):
    _fields_ = [("state", C.c_uint64)]


class Workspace(C.Structure):
    _fields_ = [("probs", C.POINTER(c_float)), ("n_vocab", c_size_t)]


# every symbol include/geist_b200.h declares, with its signature
PROTOTYPES = {
    "geist_b200_errmsg": (C.c_char_p, []),
    "geist_rng_seed": (None, [C.POINTER(Rng), C.c_uint64]),
    "geist_rng_next_u64": (C.c_uint64, [C.POINTER(Rng)]),
    "geist_rng_next_unit": (c_float, [C.POINTER(Rng)]),
    "geist_sampler_argmax": (c_int32, [c_size_t, c_void_p]),
    "geist_sampler_temperature": (c_int32, [c_size_t, c_void_p, c_float, C.POINTER(Rng)]),
    "geist_sampler_workspace_init": (C.c_int, [C.POINTER(Workspace), c_size_t]),
    "geist_sampler_workspace_destroy": (None, [C.POINTER(Workspace)]),
    "geist_sampler_top_k_ws": (c_int32, [C.POINTER(Workspace), c_void_p, C.c_int, c_float, C.POINTER(Rng)]),
    "geist_sampler_top_p_ws": (c_int32, [C.POINTER(Workspace), c_void_p, c_float, c_float, C.POINTER(Rng)]),
    "geist_b200_ctx_create": (C.c_int, [C.c_int, C.POINTER(c_void_p)]),
    "geist_b200_ctx_destroy": (None, [c_void_p]),
    "geist_b200_sample_batch": (C.c_int, [c_void_p, C.POINTER(Batch), c_void_p]),
    "geist_b200_argmax_f32": (C.c_int, [c_void_p, c_void_p, c_size_t, C.POINTER(c_int32)]),
    "geist_b200_argmax_f32_supported": (C.c_int, [c_size_t, c_size_t]),
    "geist_b200_accept_batch": (C.c_int, [c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p]),
    "geist_b200_softmax": (C.c_int, [c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_void_p,
                                     c_void_p, c_void_p]),
    "geist_b200_scatter_kept": (C.c_int, [c_void_p, c_size_t, c_size_t, c_int32, c_void_p, c_void_p, c_void_p,
                                          c_int32, c_void_p, c_void_p]),
    "geist_b200_shard_select": (C.c_int, [c_void_p, C.POINTER(Batch), c_void_p]),
    "geist_b200_shard_merge_sample": (C.c_int, [c_void_p, C.POINTER(Merge), c_void_p]),
    "geist_b200_batcher_create": (C.c_int, [c_void_p, c_size_t, c_size_t, c_size_t, C.POINTER(c_void_p)]),
    "geist_b200_batcher_destroy": (None, [c_void_p]),
    "geist_b200_session_open": (C.c_int, [c_void_p, C.POINTER(SessionOpts), C.POINTER(PenaltyOpts),
                                          C.POINTER(c_int32)]),
    "geist_b200_session_close": (C.c_int, [c_void_p, c_int32]),
    "geist_b200_session_reset": (C.c_int, [c_void_p, c_int32]),
    "geist_b200_session_push_history": (C.c_int, [c_void_p, c_int32, c_size_t, c_void_p]),
    "geist_b200_session_get_rng": (C.c_int, [c_void_p, c_int32, C.POINTER(C.c_uint64)]),
    "geist_b200_session_set_rng": (C.c_int, [c_void_p, c_int32, C.c_uint64]),
    "geist_b200_batcher_step": (C.c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_size_t, C.c_int, C.c_int,
                                          c_void_p]),
    "geist_b200_batcher_verify": (C.c_int, [c_void_p, c_size_t, c_void_p, c_size_t, c_void_p, c_void_p, c_size_t,
                                            C.c_int, C.c_int, c_void_p, c_void_p, c_void_p]),
    "geist_b200_batcher_decode_step": (C.c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_size_t, C.c_int, C.c_int,
                                                 c_void_p]),
    "geist_b200_session_peek_next_token": (c_int32, [c_void_p, c_int32]),
    "geist_b200_session_peek_logits": (c_void_p, [c_void_p, c_int32, C.POINTER(c_size_t)]),
    "geist_b200_session_set_softcap": (C.c_int, [c_void_p, c_int32, C.c_float]),
    "geist_b200_session_set_logit_mask": (C.c_int, [c_void_p, c_int32, c_void_p, c_size_t]),
    "geist_b200_draft_ngram": (C.c_int, [c_void_p, c_size_t, c_void_p, c_size_t, c_void_p, c_void_p, c_size_t, c_size_t,
                                         c_size_t, c_void_p, c_void_p, c_void_p]),
    "geist_b200_batcher_propose_drafts": (C.c_int, [c_void_p, c_size_t, c_void_p, c_size_t, c_size_t, c_void_p, c_void_p,
                                                    c_void_p]),
    "geist_b200_argmax_rows_static": (C.c_int, [C.c_int, c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_void_p]),
    "geist_b200_grid": (C.c_int, [c_size_t, c_size_t, c_size_t, C.POINTER(c_int32), C.POINTER(c_int32)]),
    "geist_b200_plan": (C.c_int, [c_size_t, c_size_t, C.POINTER(c_int32), C.POINTER(c_int32), C.POINTER(c_int32),
                                  C.POINTER(c_int32)]),
}
for _name, (_res, _args) in PROTOTYPES.items():
    _f = getattr(lib, _name)
    _f.restype = _res
    _f.argtypes = _args


def _ptr(t) -> Optional[int]:
    return None if t is None else t.data_ptr()


class Context:
    """struct geist_b200_ctx for one device."""

    def __init__(self, device: int = 0):
        h = c_void_p()
        _check(lib.geist_b200_ctx_create(device, C.byref(h)))
        self.handle = h
        self.device = device

    def close(self):
        if self.handle:
            lib.geist_b200_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------ batched --
    def sample_batch(self, logits, temperature, top_k, top_p, rng_state, rows_per_seq: int = 1,
                     rep=None, freq=None, pres=None, history=None, history_len=None, fed=None,
                     slot=None, kept_cap: int = 0, want_logits: bool = False, vocab_offset: int = 0,
                     select_only: bool = False, stream=None, out=None, sync: bool = True, launch: bool = True,
                     softcap=None, logit_mask=None, finish_hint: int = 0):
        """logits: CUDA float32 [rows, V] (rows = n_seq * rows_per_seq). Per-sequence
        arguments are CUDA tensors of length n_seq (or of the slot table's size).
        Returns a dict of CUDA tensors; ``out`` lets a caller reuse a previous dict."""
        import torch

        assert logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2
        rows, V = logits.shape
        n_seq = rows // rows_per_seq
        assert n_seq * rows_per_seq == rows
        dev = logits.device
        if out is None:
            out = {
                "tokens": torch.empty(rows, dtype=torch.int32, device=dev),
                "status": torch.empty(rows, dtype=torch.int32, device=dev),
                "rng_state": torch.empty_like(rng_state),
                "logits": torch.empty(rows, V, dtype=torch.float32, device=dev) if want_logits else None,
                "kept_n": torch.zeros(rows, dtype=torch.int32, device=dev) if kept_cap else None,
                "kept_idx": torch.full((rows, kept_cap), -1, dtype=torch.int32, device=dev) if kept_cap else None,
                "kept_prob": torch.zeros(rows, kept_cap, dtype=torch.float32, device=dev) if kept_cap else None,
            }
        b = Batch()
        b.logits = logits.data_ptr()
        b.row_stride = logits.stride(0)
        b.n_seq = n_seq
        b.rows_per_seq = rows_per_seq
        b.n_vocab = V
        b.slot = _ptr(slot)
        b.temperature = temperature.data_ptr()
        b.top_k = top_k.data_ptr()
        b.top_p = top_p.data_ptr()
        b.repetition_penalty = _ptr(rep)
        b.frequency_penalty = _ptr(freq)
        b.presence_penalty = _ptr(pres)
        if history is not None:
            b.history = history.data_ptr()
            b.history_stride = history.stride(0)
            b.history_len = history_len.data_ptr()
        if fed is not None:
            b.fed_tokens = fed.data_ptr()
            b.fed_stride = fed.stride(0)
        b.rng_in = rng_state.data_ptr()
        b.rng_out = out["rng_state"].data_ptr()
        b.tokens = out["tokens"].data_ptr()
        b.row_status = out["status"].data_ptr()
        b.out_logits = _ptr(out["logits"])
        b.kept_cap = kept_cap
        b.kept_n = _ptr(out["kept_n"])
        b.kept_idx = _ptr(out["kept_idx"])
        b.kept_prob = _ptr(out["kept_prob"])
        b.vocab_offset = vocab_offset
        b.softcap = _ptr(softcap)
        if logit_mask is not None:  # CUDA int32 [n_seq, words]: bit i set = column i may be sampled
            b.logit_mask = logit_mask.data_ptr()
            b.logit_mask_stride = logit_mask.stride(0)
        b.finish_hint = finish_hint
        if stream is None:
            stream = torch.cuda.current_stream(dev).cuda_stream
        fn = lib.geist_b200_shard_select if select_only else lib.geist_b200_sample_batch
        if launch:
            _check(fn(self.handle, C.byref(b), c_void_p(stream)))
            if sync:
                torch.cuda.synchronize(dev)
        out["_desc"] = b  # the filled struct geist_b200_batch, for callers that relaunch it themselves
        out["_select"] = select_only
        return out

    def relaunch(self, out, stream: int) -> None:
        """Launch a descriptor prepared by sample_batch(..., launch=False) again (asynchronous)."""
        fn = lib.geist_b200_shard_select if out.get("_select") else lib.geist_b200_sample_batch
        _check(fn(self.handle, C.byref(out["_desc"]), c_void_p(stream)))

    def argmax_f32(self, row) -> int:
        idx = c_int32(-1)
        _check(lib.geist_b200_argmax_f32(self.handle, row.data_ptr(), row.numel(), C.byref(idx)))
        return int(idx.value)

    def accept_batch(self, fed, verify_out):
        import torch

        n, k = fed.shape
        acc = torch.empty(n, dtype=torch.int32, device=fed.device)
        nem = torch.empty(n, dtype=torch.int32, device=fed.device)
        em = torch.empty(n, k + 1, dtype=torch.int32, device=fed.device)
        st = torch.cuda.current_stream(fed.device).cuda_stream
        _check(lib.geist_b200_accept_batch(self.handle, n, k, fed.data_ptr(), verify_out.data_ptr(), acc.data_ptr(),
                                           nem.data_ptr(), em.data_ptr(), c_void_p(st)))
        torch.cuda.synchronize(fed.device)
        return acc, nem, em

    def softmax(self, logits, temperature):
        import torch

        rows, V = logits.shape
        probs = torch.empty(rows, V, dtype=torch.float32, device=logits.device)
        sums = torch.empty(rows, dtype=torch.float64, device=logits.device)
        st = torch.cuda.current_stream(logits.device).cuda_stream
        _check(lib.geist_b200_softmax(self.handle, logits.data_ptr(), logits.stride(0), rows, V, temperature.data_ptr(),
                                      probs.data_ptr(), sums.data_ptr(), c_void_p(st)))
        torch.cuda.synchronize(logits.device)
        return probs, sums

    def scatter_kept(self, out, V: int, vocab_offset: int = 0):
        import torch

        rows, cap = out["kept_idx"].shape
        dense = torch.empty(rows, V, dtype=torch.float32, device=out["kept_idx"].device)
        st = torch.cuda.current_stream(dense.device).cuda_stream
        _check(lib.geist_b200_scatter_kept(self.handle, rows, V, cap, out["kept_n"].data_ptr(), out["kept_idx"].data_ptr(),
                                           out["kept_prob"].data_ptr(), vocab_offset, dense.data_ptr(), c_void_p(st)))
        torch.cuda.synchronize(dense.device)
        return dense

    def shard_merge_sample(self, cand_val, cand_gid, cand_n, temperature, top_k, rng_state, kept_cap: int = 0, out=None, sync: bool = True):
        """cand_*: [n_shards, n_rows, stride] / [n_shards, n_rows] CUDA tensors (after the all-gather)."""
        import torch

        G, rows, stride = cand_val.shape
        dev = cand_val.device
        out = out or {
            "tokens": torch.empty(rows, dtype=torch.int32, device=dev),
            "status": torch.empty(rows, dtype=torch.int32, device=dev),
            "rng_state": torch.empty_like(rng_state),
            "kept_n": torch.zeros(rows, dtype=torch.int32, device=dev) if kept_cap else None,
            "kept_idx": torch.full((rows, kept_cap), -1, dtype=torch.int32, device=dev) if kept_cap else None,
            "kept_prob": torch.zeros(rows, kept_cap, dtype=torch.float32, device=dev) if kept_cap else None,
        }
        m = Merge()
        m.cand_val, m.cand_gid, m.cand_n = cand_val.data_ptr(), cand_gid.data_ptr(), cand_n.data_ptr()
        m.n_shards, m.n_rows, m.cand_stride = G, rows, stride
        m.temperature, m.top_k = temperature.data_ptr(), top_k.data_ptr()
        m.rng_in, m.rng_out = rng_state.data_ptr(), out["rng_state"].data_ptr()
        m.tokens, m.row_status = out["tokens"].data_ptr(), out["status"].data_ptr()
        m.kept_cap = kept_cap
        m.kept_n, m.kept_idx, m.kept_prob = _ptr(out["kept_n"]), _ptr(out["kept_idx"]), _ptr(out["kept_prob"])
        st = torch.cuda.current_stream(dev).cuda_stream
        _check(lib.geist_b200_shard_merge_sample(self.handle, C.byref(m), c_void_p(st)))
        if sync:
            torch.cuda.synchronize(dev)
        return out


def draft_ngram(ctx: Context, histories, history_len, seeds, k_max: int, max_suffix: int = 4, out_capacity: Optional[int] = None):
    """histories: host int32 [n, stride]. Returns (drafts [n, out_capacity], n_drafts [n], match_L [n])."""
    h = np.ascontiguousarray(histories, np.int32)
    n, stride = h.shape
    hl = np.ascontiguousarray(history_len, np.int32)
    sd = np.ascontiguousarray(seeds, np.int32)
    cap = k_max + 1 if out_capacity is None else out_capacity
    d = np.empty((n, max(cap, 1)), np.int32)
    nd = np.empty(n, np.int32)
    L = np.empty(n, np.int32)
    _check(lib.geist_b200_draft_ngram(ctx.handle, n, h.ctypes.data_as(c_void_p), stride, hl.ctypes.data_as(c_void_p), sd.ctypes.data_as(c_void_p),
                                      k_max, max_suffix, cap, d.ctypes.data_as(c_void_p), nd.ctypes.data_as(c_void_p), L.ctypes.data_as(c_void_p)))
    return d, nd, L


def plan(n_vocab: int, max_history: int = 0):
    c, s, m, r = c_int32(), c_int32(), c_int32(), c_int32()
    _check(lib.geist_b200_plan(n_vocab, max_history, C.byref(c), C.byref(s), C.byref(m), C.byref(r)))
    return {"slices_per_row": c.value, "slice": s.value, "smem_bytes": m.value, "ring_stages": r.value}


def grid(n_vocab: int, n_rows: int, max_history: int = 0):
    """Thread blocks of one launch over n_rows rows, and how many of them an SM holds at a time."""
    g, per = c_int32(), c_int32()
    _check(lib.geist_b200_grid(n_vocab, max_history, n_rows, C.byref(g), C.byref(per)))
    return {"thread_blocks": g.value, "blocks_per_sm": per.value}


class Batcher:
    """struct geist_b200_batcher: N sessions -> one launch."""

    def __init__(self, ctx: Context, n_vocab: int, max_sessions: int, max_history: int = 0):
        h = c_void_p()
        _check(lib.geist_b200_batcher_create(ctx.handle, n_vocab, max_sessions, max_history, C.byref(h)))
        self.handle, self.ctx, self.V = h, ctx, n_vocab

    def close(self):
        if self.handle:
            lib.geist_b200_batcher_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def open(self, temperature=0.0, top_p=0.0, top_k=0, seed=0, rep=0.0, freq=0.0, pres=0.0) -> int:
        o = SessionOpts(0, temperature, top_p, top_k, seed, None, 0, 0)
        p = PenaltyOpts(rep, freq, pres)
        s = c_int32(-1)
        _check(lib.geist_b200_session_open(self.handle, C.byref(o), C.byref(p), C.byref(s)))
        return int(s.value)

    def close_session(self, s: int):
        _check(lib.geist_b200_session_close(self.handle, s))

    def reset(self, s: int):
        _check(lib.geist_b200_session_reset(self.handle, s))

    def push_history(self, s: int, ids: Sequence[int]):
        a = np.ascontiguousarray(ids, np.int32)
        _check(lib.geist_b200_session_push_history(self.handle, s, a.size, a.ctypes.data_as(c_void_p)))

    def get_rng(self, s: int) -> int:
        v = C.c_uint64()
        _check(lib.geist_b200_session_get_rng(self.handle, s, C.byref(v)))
        return int(v.value)

    def set_rng(self, s: int, state: int):
        _check(lib.geist_b200_session_set_rng(self.handle, s, state))

    def step(self, sessions: Sequence[int], logits, append_history: bool = True) -> np.ndarray:
        """logits: CUDA tensor [n, V] or a host numpy / pinned torch CPU tensor [n, V]."""
        ss = np.ascontiguousarray(sessions, np.int32)
        out = np.empty(ss.size, np.int32)
        ptr, stride, on_host = _logits_arg(logits)
        _check(lib.geist_b200_batcher_step(self.handle, ss.size, ss.ctypes.data_as(c_void_p), c_void_p(ptr), stride,
                                           on_host, int(append_history), out.ctypes.data_as(c_void_p)))
        return out

    def decode_step(self, sessions: Sequence[int], logits, append_history: bool = True) -> np.ndarray:
        """Returns each session's pending token; the token sampled from `logits` becomes pending."""
        ss = np.ascontiguousarray(sessions, np.int32)
        out = np.empty(ss.size, np.int32)
        ptr, stride, on_host = _logits_arg(logits)
        _check(lib.geist_b200_batcher_decode_step(self.handle, ss.size, ss.ctypes.data_as(c_void_p), c_void_p(ptr), stride,
                                                  on_host, int(append_history), out.ctypes.data_as(c_void_p)))
        return out

    def peek_next_token(self, s: int) -> int:
        return int(lib.geist_b200_session_peek_next_token(self.handle, s))

    def peek_logits(self, s: int):
        """numpy view of the session's staging row (valid until its next sampling call), or None."""
        n = c_size_t(0)
        p = lib.geist_b200_session_peek_logits(self.handle, s, C.byref(n))
        if not p:
            return None
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n.value,))

    def set_softcap(self, s: int, c: float):
        _check(lib.geist_b200_session_set_softcap(self.handle, s, c))

    def set_logit_mask(self, s: int, allowed_words):
        if allowed_words is None:
            _check(lib.geist_b200_session_set_logit_mask(self.handle, s, None, 0))
            return
        w = np.ascontiguousarray(allowed_words).view(np.uint32)
        _check(lib.geist_b200_session_set_logit_mask(self.handle, s, w.ctypes.data_as(c_void_p), w.size))

    def propose_drafts(self, sessions: Sequence[int], k_max: int, out_capacity: Optional[int] = None):
        """(drafts [n, out_capacity], n_drafts [n], match_L [n]) from the sessions' pending tokens and history rings."""
        ss = np.ascontiguousarray(sessions, np.int32)
        cap = k_max + 1 if out_capacity is None else out_capacity
        d = np.empty((ss.size, max(cap, 1)), np.int32)
        nd = np.empty(ss.size, np.int32)
        L = np.empty(ss.size, np.int32)
        _check(lib.geist_b200_batcher_propose_drafts(self.handle, ss.size, ss.ctypes.data_as(c_void_p), k_max, cap,
                                                     d.ctypes.data_as(c_void_p), nd.ctypes.data_as(c_void_p), L.ctypes.data_as(c_void_p)))
        return d, nd, L

    def verify(self, sessions: Sequence[int], fed, logits, append_history: bool = True):
        """fed: host int32 [n, k]; logits [n*k, V]. Returns (accepted[n], n_out[n], out_tokens[n, k+1])."""
        ss = np.ascontiguousarray(sessions, np.int32)
        fed = np.ascontiguousarray(fed, np.int32)
        n, k = fed.shape
        acc = np.empty(n, np.int32)
        nout = np.empty(n, np.int32)
        toks = np.empty((n, k + 1), np.int32)
        ptr, stride, on_host = _logits_arg(logits)
        _check(lib.geist_b200_batcher_verify(self.handle, n, ss.ctypes.data_as(c_void_p), k, fed.ctypes.data_as(c_void_p),
                                             c_void_p(ptr), stride, on_host, int(append_history),
                                             acc.ctypes.data_as(c_void_p), nout.ctypes.data_as(c_void_p),
                                             toks.ctypes.data_as(c_void_p)))
        return acc, nout, toks


def _logits_arg(logits):
    if isinstance(logits, np.ndarray):
        assert logits.dtype == np.float32 and logits.flags.c_contiguous
        return logits.ctypes.data, logits.shape[1], 1
    assert str(logits.dtype) == "torch.float32"
    return logits.data_ptr(), logits.stride(0), 0 if logits.is_cuda else 1


# ---------------------------------------------------- sampler.h host surface --

def rng_seed(seed: int) -> Rng:
    r = Rng()
    lib.geist_rng_seed(C.byref(r), seed)
    return r


def sampler_argmax(row: np.ndarray) -> int:
    row = np.ascontiguousarray(row, np.float32)
    return int(lib.geist_sampler_argmax(row.size, row.ctypes.data_as(c_void_p)))


def sampler_temperature(row: np.ndarray, T: float, rng: Rng) -> int:
    row = np.ascontiguousarray(row, np.float32)
    return int(lib.geist_sampler_temperature(row.size, row.ctypes.data_as(c_void_p), T, C.byref(rng)))


class SamplerWorkspace:
    def __init__(self, n_vocab: int):
        self.ws = Workspace()
        _check(lib.geist_sampler_workspace_init(C.byref(self.ws), n_vocab))

    def top_k(self, row: np.ndarray, top_k: int, T: float, rng: Rng) -> int:
        row = np.ascontiguousarray(row, np.float32)
        return int(lib.geist_sampler_top_k_ws(C.byref(self.ws), row.ctypes.data_as(c_void_p), top_k, T, C.byref(rng)))

    def top_p(self, row: np.ndarray, top_p: float, T: float, rng: Rng) -> int:
        row = np.ascontiguousarray(row, np.float32)
        return int(lib.geist_sampler_top_p_ws(C.byref(self.ws), row.ctypes.data_as(c_void_p), top_p, T, C.byref(rng)))

    def close(self):
        lib.geist_sampler_workspace_destroy(C.byref(self.ws))

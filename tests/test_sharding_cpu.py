"""World-size-2 gloo runs of the two multi-GPU schemes, on CPU with the CPU checker
standing in for the kernels: rows split across ranks (no collective on the data path)
and the vocabulary split across ranks with one all-gather of per-shard candidates."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle
    from helpers import normal_logits, independent_states
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, V, k, T = 12, 4096, 50, 0.7
    x = np.round(normal_logits(B, V, 2.5, 31337) * 8) / 8   # every rank builds the same rows; ties included
    st = independent_states(oracle.port, 31337, B)
    full = oracle.port.sample_batch(x, T, k, 0.9, st)

    # (1) rows sharded: contiguous B/world rows per rank, tokens gathered afterwards
    lo, hi = rank * B // world, (rank + 1) * B // world
    mine = oracle.port.sample_batch(x[lo:hi], T, k, 0.9, st[lo:hi])
    toks = [torch.zeros(hi - lo, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(toks, torch.from_numpy(mine["tokens"]))
    ok_rows = np.array_equal(torch.cat(toks).numpy(), full["tokens"])

    # (2) vocabulary sharded: local top-k with global ids -> all-gather -> merge -> draw
    vs = V // world
    shard = x[:, rank * vs:(rank + 1) * vs]
    val = np.empty((B, k), np.float32)
    gid = np.empty((B, k), np.int32)
    for r in range(B):
        order = np.lexsort((np.arange(vs), -shard[r]))[:k]
        val[r], gid[r] = shard[r][order], order + rank * vs
    gv = [torch.zeros(B, k) for _ in range(world)]
    gg = [torch.zeros(B, k, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gv, torch.from_numpy(val))
    dist.all_gather(gg, torch.from_numpy(gid))
    gv, gg = torch.stack(gv).numpy(), torch.stack(gg).numpy()
    ok_vocab = True
    for r in range(B):
        mv, mg = oracle.port.merge_candidates(gv[:, r].ravel(), gg[:, r].ravel(), k)
        tok, s2 = oracle.port.sample_ordered(mv, mg, T, int(st[r]))
        ok_vocab &= tok == full["tokens"][r] and s2 == int(full["rng_state"][r])
    q.put((rank, bool(ok_rows), bool(ok_vocab)))
    dist.barrier()
    dist.destroy_process_group()


def test_row_and_vocab_sharding_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == [(0, True, True), (1, True, True)]

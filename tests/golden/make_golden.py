"""Regenerates tests/golden/sampler_golden.npz from the reference's own sampler.

Run where the reference tree is mounted (oracle/_ref must be buildable):

    python tests/golden/make_golden.py

Every array is an OUTPUT OF THE REFERENCE CODE (src/engine/sampler.c compiled
unmodified, strict IEEE flags, through oracle/ref_harness.c) on the inputs
stored next to it. The literal logit arrays are the ones the reference's unit
test uses (tests/test_sampler_unit.c:34, :43, :57, :66, :96, :120, :141).
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402

assert oracle.ref is not None, "build oracle/_ref first (make -C oracle)"
ref = oracle.ref
out = {}
meta = {"cases": []}

# --- generator streams (sampler.c:27-48)
seeds = [0, 1, 7, 42, 99, 1234, 2024, 31337, 0xCAFEBABE1234, 0xC0FFEE]
out["rng_seeds"] = np.array(seeds, np.uint64)
out["rng_u64"] = np.stack([ref.rng_stream(s, 16)[0] for s in seeds])
out["rng_unit"] = np.stack([ref.rng_stream(s, 16)[1] for s in seeds])

# --- the literal arrays of the reference's unit test, with what the reference returns
lit = {
    "argmax_ties": np.array([-1.0, 2.0, 0.5, 3.0, 3.0, -0.5], np.float32),
    "peaked": np.array([0.0, 0.0, 0.0, 10.0, 0.0], np.float32),
    "small4": np.array([1.0, 2.0, 3.0, 0.5], np.float32),
    "uniform5": np.zeros(5, np.float32),
    "topk8": np.array([0.0, 1.0, 4.0, 2.0, 5.0, 1.5, 0.0, 0.5], np.float32),
    "topp5": np.array([10.0, 0.0, 0.0, 0.0, 0.0], np.float32),
    "ws8": np.array([0.1, 0.2, 0.3, 5.0, 0.1, 0.0, 0.0, 0.0], np.float32),
}
for k, v in lit.items():
    out["lit_" + k] = v
out["lit_argmax_ties_tok"] = np.array([ref.argmax(lit["argmax_ties"])], np.int32)


def stream(which, row, n, seed, **kw):
    st = ref.rng_seed(seed)
    toks = []
    for _ in range(n):
        t, st = ref.sampler_call(which, row, state=st, **kw)
        toks.append(t)
    return np.array(toks, np.int32), np.uint64(st)


out["lit_peaked_T0.1_seed42"], _ = stream("temperature", lit["peaked"], 1000, 42, T=0.1)
out["lit_small4_T0_seed1"], _ = stream("temperature", lit["small4"], 1, 1, T=0.0)
out["lit_uniform5_T1_seed7"], _ = stream("temperature", lit["uniform5"], 5000, 7, T=1.0)
out["lit_topk8_k2_T1_seed11"], _ = stream("top_k", lit["topk8"], 1000, 11, top_k=2, T=1.0)
out["lit_topp5_p0.5_T1_seed13"], _ = stream("top_p", lit["topp5"], 1000, 13, top_p=0.5, T=1.0)
out["lit_ws8_k3_T1_seed17"], _ = stream("top_k", lit["ws8"], 100, 17, top_k=3, T=1.0)

# --- synthetic rows through the 4-way dispatch, one generator per sequence
rng = np.random.default_rng(20240)
cases = [
    # name, rows, V, rows_per_seq, T, top_k, top_p, kind
    ("greedy", 6, 1500, 1, 0.0, 0, 1.0, "normal"),
    ("topk40", 6, 1500, 1, 0.8, 40, 0.95, "normal"),
    ("topk_ties", 6, 700, 1, 1.0, 5, 1.0, "ties"),
    ("topk_ge_V", 4, 64, 1, 0.7, 64, 1.0, "normal"),
    ("topp", 6, 1500, 1, 0.8, 0, 0.9, "normal"),
    ("topp_gumbel", 6, 2000, 1, 0.9, 0, 0.95, "gumbel"),
    ("topp_flat", 4, 300, 1, 1.0, 0, 0.5, "ties"),
    ("temperature", 6, 1500, 1, 1.1, 0, 1.0, "normal"),
    ("verify_rows", 8, 1000, 4, 0.9, 20, 1.0, "normal"),
    ("neg_temperature", 3, 200, 1, -1.0, 10, 0.5, "normal"),
    ("topk1", 3, 200, 1, 0.8, 1, 0.5, "normal"),
]
for name, rows, V, R, T, K, P, kind in cases:
    if kind == "normal":
        x = (rng.standard_normal((rows, V)) * 2.5).astype(np.float32)
    elif kind == "gumbel":
        x = (4.0 * -np.log(-np.log(rng.random((rows, V))))).astype(np.float32)
    else:
        x = rng.integers(-2, 3, (rows, V)).astype(np.float32)
    S = rows // R
    st = np.array([ref.rng_seed(1000 + i) for i in range(S)], np.uint64)
    r = ref.sample(x, T, K, P, st, rows_per_seq=R)
    out[f"case_{name}_logits"] = x
    out[f"case_{name}_state_in"] = st
    out[f"case_{name}_tokens"] = r["tokens"]
    out[f"case_{name}_state_out"] = r["rng_state"]
    meta["cases"].append({"name": name, "rows": rows, "V": V, "rows_per_seq": R, "T": T, "top_k": K, "top_p": P})
    if K > 1 and T > 0 and K < V:
        idx, prob, s = ref.topk_detail(x[0], K, T)
        out[f"case_{name}_kept_idx"], out[f"case_{name}_kept_prob"] = idx, prob
    elif 0 < P < 1 and T > 0 and K <= 1:
        n, idx, pn, pq, s = ref.topp_detail(x[0], P, T)
        out[f"case_{name}_kept_idx"], out[f"case_{name}_kept_prob"] = idx, pq
        out[f"case_{name}_kept_pnorm"] = pn

# --- softmax as the top-p path normalises it
x = (rng.standard_normal(1200) * 3.0).astype(np.float32)
out["softmax_logits"] = x
out["softmax_T0.7"], s = ref.softmax(x, 0.7)
out["softmax_T0.7_sum"] = np.array([s])

np.savez_compressed(Path(__file__).with_name("sampler_golden.npz"), **out)
Path(__file__).with_name("sampler_golden.json").write_text(json.dumps(meta, indent=1))
print("wrote", len(out), "arrays")

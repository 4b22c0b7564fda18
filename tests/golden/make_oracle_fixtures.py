"""Writes tests/golden/oracle_small.npz (and q8k_small.npz, the Q8_K activation quantiser): small seeded
inputs and the CPU oracle's outputs for every op of the hot path.  The fixtures pin the oracle itself (a rebuilt oracle, another
libm or another compiler must reproduce them) and give the GPU tests a committed target
that does not depend on the oracle being rebuilt on the GPU box.
Run from the repository root: python tests/golden/make_oracle_fixtures.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from agention_infer_b200 import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402

out = {}
T, H, hd, nq, nkv, I = 12, 512, 64, 4, 2, 768

x = synth.activations(1, "x", (T, H)); w = synth.norm_weight(1, "w", H); d = synth.activations(1, "delta", (T, H))
out.update(rms_x=x, rms_w=w, rms_out=orc.rms_norm_rows(x, w, 1e-5))
nx, nm = orc.add_residual_rms_norm_rows(x, d, w, 1e-5)
out.update(res_delta=d, res_new_x=nx, res_normed=nm)

q = synth.activations(1, "q", (T, nq * hd)); k = synth.activations(1, "k", (T, nkv * hd))
pos = np.array([0, 1, 2, 3, 17, 100, 511, 1000, 4095, 8191, 20000, 32767], dtype=np.int32)
wq = synth.norm_weight(1, "wq", hd)
out.update(rope_q=q, rope_k=k, rope_pos=pos,
           rope_q_neox=orc.rope_rows(q, nq, hd, hd, pos, 500000.0, 1.0, orc.NEOX),
           rope_k_neox=orc.rope_rows(k, nkv, hd, hd, pos, 500000.0, 1.0, orc.NEOX),
           rope_q_normal=orc.rope_rows(q, nq, hd, hd, pos, 500000.0, 1.0, orc.NORMAL),
           rope_q_partial=orc.rope_rows(q, nq, hd, 32, pos, 10000.0, 0.5, orc.NEOX),
           qknorm_w=wq, qknorm_rope_q=orc.qk_norm_rope_rows(q, wq, nq, hd, 1e-6, hd, pos, 1e6))

g = synth.activations(1, "gate", (T, I)); u = synth.activations(1, "up", (T, I))
out.update(silu_gate=g, silu_up=u, silu_out=orc.silu_mul(g, u))

s = synth.causal_scores(1, 2, 32)
nv = np.tile(np.arange(1, 33, dtype=np.int32), 2)
out.update(softmax_in=s, softmax_nv=nv, softmax_out=orc.softmax_rows(s, nv))

for name, dt, rl in (("q8_0", orc.Q8_0, 96), ("q4_k", orc.Q4_K, 512), ("q6_k", orc.Q6_K, 512)):
    table = synth.quant_table(dt, 24, rl, cfg_index=1)
    ids = np.array([0, 23, 5, 5, 11, 7], dtype=np.uint32)
    st, rows = orc.get_rows(dt, table, 24, rl, ids)
    assert st == orc.OK
    out.update({f"{name}_table": table, f"{name}_ids": ids, f"{name}_rows": rows})

logits = synth.activations(5, "logits", (16, 8))
idx, wts = orc.router_top2(logits)
xg = synth.activations(5, "x", (16, 64))
go, goff, gtok, gslot = orc.gather_rows_by_expert(xg, idx, 8)
out.update(router_logits=logits, router_idx=idx, router_w=wts, gather_x=xg, gather_out=go, gather_offsets=goff,
           gather_token=gtok, gather_slot=gslot)

path = Path(__file__).with_name("oracle_small.npz")
np.savez_compressed(path, **out)
print("wrote", path, path.stat().st_size, "bytes")

# Q8_K activation rows (quantize_row_q8_k, src/quant/q8_k.rs:49-92): ragged rows with a tie of +a / -a, an all-zero
# block, exact .5 products, a NaN and an infinity; integer outputs, so the fixture is exact
xq = (synth.activations(1, "x", (8, 600)) * np.float32(3.0)).astype(np.float32)
xq[1, :256] = 0.0
xq[2, 7], xq[2, 300] = 9.5, -9.5
xq[3, :6] = [-127.0, 0.5, 1.5, -2.5, 126.5, -0.5]; xq[3, 6:256] = 0.25
xq[4, 11] = np.nan
xq[5, 13] = np.inf
with np.errstate(all="ignore"):
    qd, qq, qb = orc.quantize_rows_q8_k(xq)
qpath = Path(__file__).with_name("q8k_small.npz")
np.savez_compressed(qpath, x=xq, d=qd, qs=qq, bsums=qb)
print("wrote", qpath, qpath.stat().st_size, "bytes")

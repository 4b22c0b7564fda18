#!/usr/bin/env python
"""Layer-op hot-path benchmark: tokens/s and HBM GB/s of the CUDA backend, one JSON line.

  python bench.py --gpus N --steps K --warmup W            # our CUDA arm (default)
  python bench.py --impl reference --gpus N --steps K ...  # the CPU restatement of the reference
  torchrun --nproc-per-node N bench.py --gpus N ...        # one rank per GPU

A step is one pass of the hot path over one batch of token rows of the Qwen2.5-7B-shaped
prefill configuration (T=4096 rows per GPU): quantised-embedding get_rows (Q4_K), RMSNorm,
NeoX RoPE on Q and K, the fused per-head norm->RoPE, and the fused SiLU*mul.  Rows shard
across ranks with no data-path collective (weak scaling: T rows per GPU).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "layer_op_tokens_per_s"
UNIT = "tokens/s"
NSETS = 4  # rotating buffer sets: every timed launch reads inputs that are not in L2


# --------------------------------------------------------------------------- helpers

def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def silu_traffic_bytes(n_elements):
    """DRAM bytes of one silu_mul launch (dram__bytes_read.sum + dram__bytes_write.sum), from one-pass ncu
    captures of this kernel summarised under profiles/: at the headline size (4096 rows, 77,594,624 elements)
    620.8 MB read = 8.00 B per element, i.e. no re-reads, and 262.4 MB of the 310.4 MB written, the other 48 MB
    still dirty in L2 when the kernel ends (43.5 MB at 2048 rows).  Other sizes: reads and writes scale with the
    element count, the dirty remainder does not."""
    dirty_left = 48.0e6
    return 8.0 * n_elements + max(4.0 * n_elements - dirty_left, 0.0)


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the GPU is under load."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(device_index), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.f,
                                      stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def mark_load(self, begin: bool):
        """Wall-clock bounds of the phase whose samples count (the GPU is under load)."""
        import datetime
        if begin:
            self.t0 = datetime.datetime.now()
        else:
            self.t1 = datetime.datetime.now()

    def stop(self):
        import datetime
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [l.strip().split(", ") for l in open(self.f.name) if l.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons, power = [], [], set(), []
        t0, t1 = getattr(self, "t0", None), getattr(self, "t1", None)
        for r in rows:
            if len(r) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(r[0].strip(), "%Y/%m/%d %H:%M:%S.%f")
                if t0 and t1 and not (t0 <= ts <= t1):
                    continue
                r = r[1:]
                sm.append(float(r[0])); mx.append(float(r[1])); power.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": float(max(power))}


# ---------------------------------------------------------------------------- workloads

WORKLOADS = {
    # name: (config key, ops of one step, scaling)
    "c2": ("c2", ["get_rows", "rms_norm", "rope_qk", "qk_norm_rope_qk", "silu_mul"], "weak"),
    "c1": ("c1", ["get_rows", "rms_norm", "rope_qk", "silu_mul", "softmax"], "weak"),
    "c4": ("c4", ["get_rows", "rms_norm", "rope_qk", "qk_norm_rope_qk", "silu_mul"], "strong"),
    "c5": ("c5", ["get_rows", "rms_norm", "rope_qk", "router_top2", "gather_rows_by_expert", "silu_mul"], "strong"),
}
DTYPE_NAMES = {8: "Q8_0", 12: "Q4_K", 14: "Q6_K"}


def op_bytes(cfg, T, ops, act_bytes=4):
    """Algorithmic bytes of each op of a step for T token rows (activations of act_bytes each, read + write)."""
    from agention_infer_b200 import CudaBackend
    H, hd, nq, nkv, I = cfg.hidden, cfg.head_dim, cfg.n_q_heads, cfg.n_kv_heads, cfg.ffn
    a = act_bytes
    rope = 2 * a * T * (nq + nkv) * hd + 4 * T + 2 * cfg.n_rot
    L = T  # c1: causal scores [nq, T, T]
    table = {
        "get_rows": T * CudaBackend.type_size(cfg.embd_dtype, H) + a * T * H + 4 * T,
        "rms_norm": 2 * a * T * H + 4 * H,
        "rope_qk": rope,
        "qk_norm_rope_qk": rope + 8 * hd,
        "silu_mul": 3 * a * T * I * (2 if cfg.n_experts else 1),  # MoE: 2T routed rows
        "softmax": 4 * (nq * L * (L + 1) // 2 + nq * L * L),
        "router_top2": 4 * T * max(cfg.n_experts, 1) + 16 * T,
        "gather_rows_by_expert": 2 * 2 * T * H * 4,
    }
    return {k: table[k] for k in ops}


def workload_config(cfg, tokens_per_gpu, tokens_total, ops, world):
    """The `config` object of the JSON line: what the workload is, the same keys and values in both arms."""
    return {"workload": cfg.name, "tokens_per_gpu": tokens_per_gpu, "tokens_total": tokens_total, "hidden": cfg.hidden,
            "head_dim": cfg.head_dim, "q_heads": cfg.n_q_heads, "kv_heads": cfg.n_kv_heads, "ffn": cfg.ffn,
            "embedding": f"{DTYPE_NAMES[cfg.embd_dtype]} {cfg.vocab}x{cfg.hidden}", "ops": list(ops),
            "parallelism": f"token rows sharded over {world} rank(s), no data-path collective"}


# ------------------------------------------------------------------- CPU (reference) arm

def host_threads():
    """All host threads this process may use (torchrun exports OMP_NUM_THREADS=1, so the OpenMP
    default is not it)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def host_data(cfg, T, ops, vocab_rows=None):
    """Seeded host inputs of one batch.  A reduced number of table rows keeps the CPU arm's
    set-up short; ids are drawn inside it."""
    from agention_infer_b200 import synth
    vocab = cfg.vocab if vocab_rows is None else vocab_rows
    i = cfg.index
    R = 2 * T if cfg.n_experts else T
    d = {
        "table": synth.quant_table(cfg.embd_dtype, vocab, cfg.hidden, cfg_index=i),
        "ids": synth.token_ids(i, T, vocab),
        "x": synth.activations(i, "x", (T, cfg.hidden)),
        "w": synth.norm_weight(i, "w", cfg.hidden),
        "q": synth.activations(i, "q", (T, cfg.n_q_heads * cfg.head_dim)),
        "k": synth.activations(i, "k", (T, cfg.n_kv_heads * cfg.head_dim)),
        "wq": synth.norm_weight(i, "wq", cfg.head_dim),
        "wk": synth.norm_weight(i, "wk", cfg.head_dim),
        "pos": synth.positions(i, T, cfg.random_pos),
        "gate": synth.activations(i, "gate", (R, cfg.ffn)),
        "up": synth.activations(i, "up", (R, cfg.ffn)),
    }
    if "softmax" in ops:
        d["scores"] = synth.causal_scores(i, cfg.n_q_heads, T)
        d["nv"] = np.tile(np.arange(1, T + 1, dtype=np.int32), cfg.n_q_heads)
    if cfg.n_experts:
        d["logits"] = synth.activations(i, "logits", (T, cfg.n_experts))
    return d, vocab


def cpu_step(orc, cfg, d, T, ops, threads):
    """One pass of the hot path over T token rows on the host, oracle code."""
    for op in ops:
        if op == "get_rows":
            orc.get_rows(cfg.embd_dtype, d["table"], cfg.vocab, cfg.hidden, d["ids"][:T], threads)
        elif op == "rms_norm":
            orc.rms_norm_rows(d["x"][:T], d["w"], cfg.eps, threads)
        elif op == "rope_qk":
            orc.rope_rows(d["q"][:T], cfg.n_q_heads, cfg.head_dim, cfg.n_rot, d["pos"][:T], cfg.theta, 1.0, 0, threads)
            orc.rope_rows(d["k"][:T], cfg.n_kv_heads, cfg.head_dim, cfg.n_rot, d["pos"][:T], cfg.theta, 1.0, 0, threads)
        elif op == "qk_norm_rope_qk":
            orc.qk_norm_rope_rows(d["q"][:T], d["wq"], cfg.n_q_heads, cfg.head_dim, cfg.eps, cfg.n_rot, d["pos"][:T],
                                  cfg.theta, 1.0, 0, threads)
            orc.qk_norm_rope_rows(d["k"][:T], d["wk"], cfg.n_kv_heads, cfg.head_dim, cfg.eps, cfg.n_rot, d["pos"][:T],
                                  cfg.theta, 1.0, 0, threads)
        elif op == "silu_mul":
            R = 2 * T if cfg.n_experts else T
            orc.silu_mul(d["gate"][:R], d["up"][:R], threads)
        elif op == "softmax":
            orc.softmax_rows(d["scores"], d["nv"], threads)
        elif op == "router_top2":
            d["idx"], _ = orc.router_top2(d["logits"][:T])
        elif op == "gather_rows_by_expert":
            orc.gather_rows_by_expert(d["x"][:T], d["idx"], cfg.n_experts)


def time_cpu(orc, cfg, data, rows, ops, threads, reps):
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        cpu_step(orc, cfg, data, rows, ops, threads)
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_sample(cfg, ops):
    """Bounded sample of the workload for the host arm: at most 4096 token rows (the whole batch of
    the headline configuration; all 512 for the causal-softmax configuration, whose scores need
    whole heads), ids drawn over the configuration's whole embedding table."""
    from oracle import oracle as orc
    rows = cfg.T if "softmax" in ops else min(cfg.T, 4096)
    data, vocab = host_data(cfg, rows, ops)
    return orc, rows, data, dataclasses.replace(cfg, T=rows), vocab


def run_reference(args, cfg, ops, wl):
    """The reference's CPU implementation of the path (C restatement; the Rust original cannot
    be built here), all host threads, on a bounded row sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    orc, rows, data, c, vocab = cpu_sample(cfg, ops)
    threads = host_threads()
    t1 = time_cpu(orc, c, data, rows, ops, threads, 1)
    limit_s = 120.0
    while rows > 64 and "softmax" not in ops and t1 * (args.steps + args.warmup) > limit_s:
        rows //= 2
        t1 = time_cpu(orc, c, data, rows, ops, threads, 1)
    for _ in range(args.warmup):
        cpu_step(orc, c, data, rows, ops, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(orc, c, data, rows, ops, threads)
    dt = (time.perf_counter() - t0) / args.steps
    value = rows / dt
    sample = f"{rows} of {cfg.T} token rows per step, table of {vocab} rows, OpenMP over rows"
    world = max(1, args.gpus)
    scaling = WORKLOADS[wl][2]
    per_gpu = cfg.T // world if scaling == "strong" else cfg.T
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, per_gpu, cfg.T if scaling == "strong" else world * cfg.T, ops, world),
        "sample_rows_per_step": rows,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def cpu_baseline(cfg, ops):
    """The oracle timed on this box's host cores on a bounded sample of the workload."""
    orc, rows, data, c, vocab = cpu_sample(cfg, ops)
    threads = host_threads()
    cpu_step(orc, c, data, rows, ops, threads)
    t_all = time_cpu(orc, c, data, rows, ops, threads, 20)
    t_one = time_cpu(orc, c, data, rows, ops, 1, 3)
    return {"value": rows / t_all, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{rows} of {cfg.T} token rows, table of {vocab} rows, best of 20, OpenMP over rows",
            "single_thread_value": rows / t_one}


# ------------------------------------------------------------------------- CUDA arm

def setup_cuda(args):
    import torch
    import torch.distributed as dist

    from agention_infer_b200 import CudaBackend
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # the version banner goes to stdout, which carries the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    sampler = ClockSampler(local) if rank == 0 else None  # started early: nvidia-smi takes a second to come up
    be = CudaBackend(local)
    # One explicit (non-default) stream for everything: torch's allocations and events and our
    # kernels.  (A null handle would select the backend's own stream, which torch events on
    # the default stream do not see.)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    assert stream.cuda_stream != 0
    be.set_stream(stream.cuda_stream)
    assert be.stream() == stream.cuda_stream
    if args.no_pdl:
        be.set_option("pdl", 0)
    for kv in args.set_option or []:  # tuning knobs of agn_ctx_set_option, e.g. --set-option rms_ring=3
        name, _, val = kv.partition("=")
        be.set_option(name, int(val))
    return torch, dist, be, dev, stream, sampler, rank, world, local


def run_ours(args, cfg, ops_list, wl):
    from agention_infer_b200 import sharding, synth
    torch, dist, be, dev, stream, sampler, rank, world, local = setup_cuda(args)
    scaling = WORKLOADS[wl][2]
    if scaling == "strong":  # the configuration's rows are split over the ranks
        r0, r1 = sharding.shard_rows(cfg.T, rank, world)
        T = r1 - r0
    else:                    # every rank runs the configuration's rows
        T = cfg.T
    T_total = cfg.T if scaling == "strong" else world * cfg.T
    H, hd, nq, nkv, I, E = cfg.hidden, cfg.head_dim, cfg.n_q_heads, cfg.n_kv_heads, cfg.ffn, cfg.n_experts
    R = 2 * T if E else T  # rows of the SwiGLU operands (MoE: routed rows)
    f16 = args.act == "f16"
    if f16 and any(o in ops_list for o in ("softmax", "router_top2", "gather_rows_by_expert")):
        raise SystemExit("--act f16 covers get_rows, rms_norm, rope, fused norm->rope and silu_mul (workloads c2, c4)")
    adt = torch.float16 if f16 else torch.float32
    ab = op_bytes(cfg, T, ops_list, 2 if f16 else 4)
    step_bytes = sum(ab.values())
    nsets = NSETS if step_bytes < 4e9 else 2
    table_h = synth.quant_table(cfg.embd_dtype, cfg.vocab, H, cfg_index=cfg.index)
    table = torch.from_numpy(table_h).to(dev)
    table_bytes = table_h.nbytes
    w = torch.from_numpy(synth.norm_weight(cfg.index, "w", H)).to(dev)
    wq = torch.from_numpy(synth.norm_weight(cfg.index, "wq", hd)).to(dev)
    wk = torch.from_numpy(synth.norm_weight(cfg.index, "wk", hd)).to(dev)
    pos = torch.from_numpy(synth.positions(cfg.index, T, cfg.random_pos)).to(dev)
    gen = torch.Generator(device=dev)
    rn = lambda *shape: torch.randn(*shape, device=dev, generator=gen).to(adt)
    # Buffer set 0 holds seeded host bytes (the same arrays the CPU arm and the oracle read) and is what the
    # outputs are checked on after the timed region; the other sets hold device-generated values that differ
    # per rank.  (The 16 GB configuration generates set 0 on the device too: its host copy would be 17 GB.)
    host0 = None
    if step_bytes < 4e9:
        ci = cfg.index
        host0 = {"x": synth.activations(ci, "x", (T, H)), "q": synth.activations(ci, "q", (T, nq * hd)),
                 "k": synth.activations(ci, "k", (T, nkv * hd)), "gate": synth.activations(ci, "gate", (R, I)),
                 "up": synth.activations(ci, "up", (R, I))}
        if "softmax" in ops_list:
            host0["scores"] = synth.causal_scores(ci, nq, T)
        if E:
            host0["logits"] = synth.activations(ci, "logits", (T, E))
    up0 = lambda name: torch.from_numpy(host0[name]).to(dev).to(adt)
    sets = []
    for s in range(nsets):
        salt = 0 if s == 0 else 1 + rank * NSETS + s
        gen.manual_seed(synth.BASE_SEED + 1000 * cfg.index + 7919 * salt)
        ids = torch.from_numpy(synth.token_ids(cfg.index, T, cfg.vocab, salt=salt).astype(np.int32)).to(dev)
        from_host = s == 0 and host0 is not None
        mk = (lambda name, *shape: up0(name)) if from_host else (lambda name, *shape: rn(*shape))
        b = {"ids": ids, "emb": torch.empty(T, H, device=dev, dtype=adt), "x": mk("x", T, H),
             "xn": torch.empty(T, H, device=dev, dtype=adt), "q": mk("q", T, nq * hd), "k": mk("k", T, nkv * hd),
             "gate": mk("gate", R, I), "up": mk("up", R, I), "act": torch.empty(R, I, device=dev, dtype=adt)}
        if "qk_norm_rope_qk" in ops_list:
            b.update(q2=mk("q", T, nq * hd), k2=mk("k", T, nkv * hd))
        if "softmax" in ops_list:
            b.update(scores=up0("scores") if from_host else rn(nq, T, T) * 2.0, probs=torch.empty(nq, T, T, device=dev))
        if E:
            b.update(logits=mk("logits", T, E), ridx=torch.empty(T, 2, dtype=torch.int32, device=dev),
                     rw=torch.empty(T, 2, device=dev), gx=torch.empty(2 * T, H, device=dev),
                     goff=torch.empty(E + 1, dtype=torch.int32, device=dev),
                     gtok=torch.empty(2 * T, dtype=torch.int32, device=dev),
                     gslot=torch.empty(2 * T, dtype=torch.int32, device=dev))
        sets.append(b)

    all_ops = {
        "get_rows": lambda b: be.get_rows(cfg.embd_dtype, table, table_bytes, cfg.vocab, H, b["ids"], T, out=b["emb"]),
        "rms_norm": lambda b: be.launch_rms_norm(b["x"], w, T, H, cfg.eps, out=b["xn"]),
        "rope_qk": lambda b: be.launch_rope_qk(b["q"], b["k"], T, nq, nkv, hd, cfg.n_rot, pos, cfg.theta),
        "qk_norm_rope_qk": lambda b: be.launch_qk_norm_rope_qk(b["q2"], b["k2"], wq, wk, T, nq, nkv, hd, cfg.eps,
                                                               cfg.n_rot, pos, cfg.theta),
        "silu_mul": lambda b: be.launch_silu_mul(b["gate"], b["up"], R * I, out=b["act"]),
        "softmax": lambda b: be.launch_softmax_rows(b["scores"], nq * T, T, out=b["probs"], causal_period=T),
        "router_top2": lambda b: be.router_top2(b["logits"], T, E, idx=b["ridx"], w=b["rw"]),
        "gather_rows_by_expert": lambda b: be.gather_rows_by_expert(b["x"], b["ridx"], T, H, E, out=b["gx"],
                                                                    offsets=b["goff"], src_token=b["gtok"],
                                                                    src_slot=b["gslot"]),
    }
    if f16:  # the same ops on f16 activation buffers (the reference's default `Act`)
        all_ops.update({
            "get_rows": lambda b: be.get_rows_f16(cfg.embd_dtype, table, table_bytes, cfg.vocab, H, b["ids"], T, out=b["emb"]),
            "rms_norm": lambda b: be.launch_rms_norm_f16(b["x"], w, T, H, cfg.eps, out=b["xn"]),
            "rope_qk": lambda b: be.launch_qk_norm_rope_qk_f16(b["q"], b["k"], None, None, T, nq, nkv, hd, 0.0, cfg.n_rot, pos,
                                                               cfg.theta),
            "qk_norm_rope_qk": lambda b: be.launch_qk_norm_rope_qk_f16(b["q2"], b["k2"], wq, wk, T, nq, nkv, hd, cfg.eps,
                                                                       cfg.n_rot, pos, cfg.theta),
            "silu_mul": lambda b: be.launch_silu_mul_f16(b["gate"], b["up"], R * I, out=b["act"]),
        })
    ops = {k: all_ops[k] for k in ops_list}
    order = list(ops)

    def step(i, silu_events=None):
        b = sets[i % nsets]
        for name in order:
            # events around the dominant kernel on every 4th step only: an event between two
            # kernels breaks their programmatic overlap, so sampling keeps the timed region honest
            if silu_events is not None and name == "silu_mul" and i % 4 == 0:
                e0, e1 = silu_events
                e0.record(stream); ops[name](b); e1.record(stream)
            else:
                ops[name](b)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up: at least W (>= 3) steps and at least 0.6 s, so that clocks settle and the
    # clock sampler has the GPU under load for a while before the timed region
    if sampler:
        sampler.mark_load(True)
    t_w = time.perf_counter()
    n_warm = 0
    while n_warm < max(args.warmup, 3) or time.perf_counter() - t_w < args.warm_seconds:
        for _ in range(5):
            step(n_warm); n_warm += 1
        torch.cuda.synchronize()
    barrier()

    # ---- timed regions: exactly K steps each, device time, max over ranks; the K-step region is repeated
    #      `repeats` times back to back (each bracketed by barrier + synchronize) and the median region is the
    #      reported one, so that the headline does not rest on a few milliseconds
    use_graph = args.graph == "on" or (args.graph == "auto" and step_bytes < 2e8)  # launch-bound steps: one graph replay each
    silu_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graphs = []
    if use_graph:
        for s_ in range(nsets):
            be.graph_begin(); step(s_); graphs.append(be.graph_end())
        for s_ in range(nsets):
            be.graph_launch(graphs[s_])
    region_ms, silu_samples, launches = [], [], 0
    for rep in range(max(1, args.repeats)):
        barrier()
        n0 = be.launch_count
        start.record(stream)
        if use_graph:
            for i in range(args.steps):
                be.graph_launch(graphs[i % nsets])
        else:
            for i in range(args.steps):
                step(i, silu_ev[i])
        stop.record(stream)
        barrier()
        launches = be.launch_count - n0
        region_ms.append(sharding.max_over_ranks(start.elapsed_time(stop)))
        if not use_graph:
            silu_samples += [a.elapsed_time(b) for i, (a, b) in enumerate(silu_ev) if i % 4 == 0]
    for g_ in graphs:
        be.graph_destroy(g_)
    silu_ms = float(np.mean(silu_samples)) if silu_samples else None
    elapsed_ms = float(np.median(region_ms))
    ms_per_step = elapsed_ms / args.steps
    value = T_total / (ms_per_step * 1e-3)

    # ---- per-op device time, each op alone, rotating buffer sets (inputs never L2-resident)
    per_op = {}
    reps = 40 if step_bytes < 4e9 else 10
    for name in order:
        for i in range(4):
            ops[name](sets[i % nsets])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for i in range(reps):
            ops[name](sets[i % nsets])
        b.record(stream)
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / reps
        per_op[name] = {"us": round(us, 2), "gbs": round(ab[name] / (us * 1e-6) / 1e9, 1)}
        # calibration: a plain device copy (torch copy_, what the measured peak was taken with)
        # moving the same number of bytes, timed the same way: the speed of light at this size
        n_el = max(ab[name] // 8, 1)
        srcs = [torch.empty(n_el, device=dev) for _ in range(nsets)]
        dsts = [torch.empty(n_el, device=dev) for _ in range(nsets)]
        for i in range(4):
            dsts[i % nsets].copy_(srcs[i % nsets])
        torch.cuda.synchronize()
        a.record(stream)
        for i in range(reps):
            dsts[i % nsets].copy_(srcs[i % nsets])
        b.record(stream)
        torch.cuda.synchronize()
        cus = a.elapsed_time(b) * 1e3 / reps
        per_op[name]["copy_same_bytes_us"] = round(cus, 2)
        per_op[name]["frac_of_copy_same_bytes"] = round(cus / us, 3)
        del srcs, dsts
    # ---- ops of the path that are not part of this configuration's step, each alone (f32 only):
    #      fused residual-add + norm, KV-cache packing, and a causal softmax at prefill size
    extra_ops = {}
    q8k_report = None
    if not f16 and not args.no_extras and step_bytes < 8e9:
        from agention_infer_b200 import AGN_BF16, AGN_F16 as KV_F16, AGN_KV_Q8_0_WORDS as KV_Q8_0_WORDS, AGN_Q8_0 as KV_Q8_0
        hd_kv = nkv * hd
        Ls = min(T, 2048)
        ex_sets = []
        for s_ in range(nsets):
            ex_sets.append({"x": rn(T, H), "d": rn(T, H), "nx": torch.empty(T, H, device=dev), "nm": torch.empty(T, H, device=dev),
                            "nb": torch.empty(T, H, dtype=torch.bfloat16, device=dev),
                            "k": rn(T, hd_kv), "v": rn(T, hd_kv),
                            "kc": torch.empty(T * be.kv_bytes_per_token(KV_Q8_0, hd_kv), dtype=torch.uint8, device=dev),
                            "vc": torch.empty(T * be.kv_bytes_per_token(KV_Q8_0, hd_kv), dtype=torch.uint8, device=dev),
                            "kw": torch.empty(T * be.kv_bytes_per_token(KV_Q8_0_WORDS, hd_kv), dtype=torch.uint8, device=dev),
                            "vw": torch.empty(T * be.kv_bytes_per_token(KV_Q8_0_WORDS, hd_kv), dtype=torch.uint8, device=dev),
                            "kh": torch.empty(T * hd_kv, dtype=torch.float16, device=dev),
                            "vh": torch.empty(T * hd_kv, dtype=torch.float16, device=dev),
                            "sc": rn(nq, Ls, Ls) * 2.0, "pr": torch.empty(nq, Ls, Ls, device=dev),
                            "pb": torch.empty(nq, Ls, Ls, dtype=torch.bfloat16, device=dev),
                            "ab": torch.empty(R, I, dtype=torch.bfloat16, device=dev),
                            "g": sets[s_]["gate"], "u": sets[s_]["up"], "q2": sets[s_].get("q2"), "k2": sets[s_].get("k2")})
        extras = {
            "add_residual_rms_norm": (lambda b: be.launch_add_residual_rms_norm(b["x"], b["d"], w, T, H, cfg.eps, new_x=b["nx"], normed=b["nm"]),
                                      16 * T * H + 4 * H),
            "silu_mul_out_bf16": (lambda b: be.launch_silu_mul_out16(b["g"], b["u"], R * I, AGN_BF16, out=b["ab"]), 10 * R * I),
            "rms_norm_out_bf16": (lambda b: be.launch_rms_norm_out16(b["x"], w, T, H, cfg.eps, AGN_BF16, out=b["nb"]), 6 * T * H + 4 * H),
            "add_residual_rms_norm_out_bf16": (lambda b: be.launch_add_residual_rms_norm_out16(b["x"], b["d"], w, T, H, cfg.eps, AGN_BF16,
                                                                                                new_x=b["nx"], normed=b["nb"]),
                                               14 * T * H + 4 * H),
            "kv_write_q8_0": (lambda b: be.kv_write(KV_Q8_0, b["k"], b["v"], b["kc"], b["vc"], T, hd_kv, None, T),
                              2 * T * (4 * hd_kv + be.kv_bytes_per_token(KV_Q8_0, hd_kv))),
            "kv_write_q8_0_words": (lambda b: be.kv_write(KV_Q8_0_WORDS, b["k"], b["v"], b["kw"], b["vw"], T, hd_kv, None, T),
                                    2 * T * (4 * hd_kv + be.kv_bytes_per_token(KV_Q8_0_WORDS, hd_kv))),
            "kv_write_f16": (lambda b: be.kv_write(KV_F16, b["k"], b["v"], b["kh"], b["vh"], T, hd_kv, None, T),
                             2 * T * (4 * hd_kv + 2 * hd_kv)),
            f"softmax_causal_{nq}x{Ls}x{Ls}": (lambda b: be.launch_softmax_rows(b["sc"], nq * Ls, Ls, out=b["pr"], causal_period=Ls),
                                               4 * (nq * Ls * (Ls + 1) // 2 + nq * Ls * Ls)),
            f"softmax_causal_scaled_out_bf16_{nq}x{Ls}x{Ls}": (
                lambda b: be.launch_softmax_rows_scaled_out16(b["sc"], nq * Ls, Ls, float(hd) ** -0.5, AGN_BF16, out=b["pb"],
                                                              causal_period=Ls),
                4 * (nq * Ls * (Ls + 1) // 2) + 2 * nq * Ls * Ls),
        }
        if "qk_norm_rope_qk" in ops_list:
            # QK-norm -> RoPE of q and k and the f16 cache write of the rotated k and of v, one launch
            extras["qk_norm_rope_kv_write_f16"] = (
                lambda b: be.launch_qk_norm_rope_kv_write(b["q2"], b["k2"], b["v"], wq, wk, T, nq, nkv, hd, cfg.eps, cfg.n_rot,
                                                          pos, cfg.theta, KV_F16, b["kh"], b["vh"], T),
                ab["qk_norm_rope_qk"] + T * (4 * hd_kv + 2 * 2 * hd_kv))
        # the reference's form: entries past the valid length are not written
        extras[f"softmax_causal_leave_tail_{nq}x{Ls}x{Ls}"] = (
            lambda b: be.launch_softmax_rows_valid(b["sc"], nq * Ls, Ls, b["pr"], causal_period=Ls),
            8 * (nq * Ls * (Ls + 1) // 2))
        if H % 256 == 0 and I % 256 == 0:
            # Q8_K activation rows (the input of a Q5_K matmul): 4 B read, 1 B + 36 B / 256 written per value
            nq8 = max(T * H, R * I)
            for b_ in ex_sets:
                b_["q8"] = (torch.empty(nq8 // 256, device=dev), torch.empty(nq8, dtype=torch.int8, device=dev),
                            torch.empty(nq8 // 16, dtype=torch.int16, device=dev))
            q8_out = lambda n: n + 36 * (n // 256)
            extras["quantize_rows_q8_k"] = (lambda b: be.launch_quantize_rows_q8_k(b["x"], T, H, out=b["q8"]), 4 * T * H + q8_out(T * H))
            extras["rms_norm_q8_k"] = (lambda b: be.launch_rms_norm_q8_k(b["x"], w, T, H, cfg.eps, out=b["q8"]),
                                       4 * T * H + 4 * H + q8_out(T * H))
            extras["add_residual_rms_norm_q8_k"] = (
                lambda b: be.launch_add_residual_rms_norm_q8_k(b["x"], b["d"], w, T, H, cfg.eps, new_x=b["nx"], out=b["q8"]),
                12 * T * H + 4 * H + q8_out(T * H))
            extras["silu_mul_q8_k"] = (lambda b: be.launch_silu_mul_q8_k(b["g"], b["u"], R, I, out=b["q8"]), 8 * R * I + q8_out(R * I))
        for name, (fn, nbytes) in extras.items():
            for i in range(4):
                fn(ex_sets[i % nsets])
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for i in range(reps):
                fn(ex_sets[i % nsets])
            b.record(stream)
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / reps
            extra_ops[name] = {"us": round(us, 2), "gbs": round(nbytes / (us * 1e-6) / 1e9, 1), "bytes": nbytes}
        if "quantize_rows_q8_k" in extras and not args.no_verify:
            # The Q8_K rows against the oracle, on 64 strided rows of buffer set 0: the quantiser alone must give the
            # oracle's bytes for the same f32 rows; the fused norm is held to the oracle's norm -> quantise chain
            # (scales to 1e-5 relative, a quantised value at most one step off, group sums exact).
            from oracle import oracle as orc
            b_ = ex_sets[0]
            rows = torch.from_numpy(np.unique(np.linspace(0, T - 1, min(T, args.check_rows)).astype(np.int64))).to(dev)
            nbk = H // 256
            xs = b_["x"].index_select(0, rows).contiguous()
            sub = (torch.empty(rows.numel() * nbk, device=dev), torch.empty(rows.numel() * H, dtype=torch.int8, device=dev),
                   torch.empty(rows.numel() * nbk * 16, dtype=torch.int16, device=dev))
            host = lambda t3: (t3[0].cpu().numpy().reshape(-1, nbk), t3[1].cpu().numpy().reshape(-1, H),
                               t3[2].cpu().numpy().reshape(-1, nbk * 16))
            be.launch_quantize_rows_q8_k(xs, rows.numel(), H, out=sub)
            be.sync(); torch.cuda.synchronize()
            got = host(sub)
            x_h = xs.cpu().numpy()
            ref = orc.quantize_rows_q8_k(x_h)
            exact = bool(np.array_equal(got[0].view(np.uint32), ref[0].view(np.uint32)) and np.array_equal(got[1], ref[1])
                         and np.array_equal(got[2], ref[2]))
            be.launch_rms_norm_q8_k(xs, w, rows.numel(), H, cfg.eps, out=sub)
            be.sync(); torch.cuda.synchronize()
            got = host(sub)
            ref = orc.quantize_rows_q8_k(orc.rms_norm_rows(x_h, synth.norm_weight(cfg.index, "w", H), cfg.eps))
            dq = np.abs(got[1].astype(np.int32) - ref[1].astype(np.int32))
            d_rel = float(np.max(np.abs(got[0] - ref[0]) / np.maximum(np.abs(ref[0]), 1e-30)))
            sums_ok = bool(np.array_equal(got[2], got[1].reshape(got[1].shape[0], -1, 16).astype(np.int16).sum(axis=2)))
            q8k_report = {"rows_checked": int(rows.numel()), "quantize_rows_bit_exact": exact,
                          "rms_norm_q8_k": {"max_rel_err_d": float(f"{d_rel:.3g}"), "max_step_err_q": int(dq.max()),
                                            "fraction_of_q_off_by_one": float(f"{float((dq != 0).mean()):.3g}"),
                                            "bsums_are_group_sums": sums_ok},
                          "ok": exact and d_rel <= 1e-5 and int(dq.max()) <= 1 and float((dq != 0).mean()) < 2e-3 and sums_ok}
        del ex_sets
    if sampler:
        sampler.mark_load(False)
    clocks = sampler.stop() if sampler else None

    # ---- end to end through the public host-slice API: pinned host arrays in, pinned host
    #      arrays out, every step, copies inside the timed region
    e2e = None
    e2e_ops = [o for o in order if o in ("get_rows", "rms_norm", "rope_qk", "qk_norm_rope_qk", "silu_mul", "softmax")]
    if not args.no_e2e and not f16 and e2e_ops == order and step_bytes < 4e9:  # (the 16 GB configuration would pin 17 GB of host memory)
        b0 = sets[0]
        needs = {"get_rows": (["ids"], ["emb"]), "rms_norm": (["x"], ["xn"]), "rope_qk": (["q", "k"], []),
                 "qk_norm_rope_qk": (["q2", "k2"], []), "silu_mul": (["gate", "up"], ["act"]),
                 "softmax": (["scores"], ["probs"])}
        names_in = [n for o in order for n in needs[o][0]]
        names_out = [n for o in order for n in needs[o][1]]
        inplace = [n for n in names_in if n in ("q", "k", "q2", "k2")]  # rotated in place in their host arrays
        host_in = {n: b0[n].cpu().pin_memory() for n in names_in}
        host_out = {n: torch.empty_like(b0[n], device="cpu").pin_memory() for n in names_out}
        h2d = sum(t.numel() * t.element_size() for t in host_in.values())
        d2h = sum(t.numel() * t.element_size() for t in host_out.values()) + sum(host_in[n].numel() * 4 for n in inplace)
        hin = {n: t.numpy() for n, t in host_in.items()}
        hout = {n: t.numpy() for n, t in host_out.items()}
        if "ids" in hin:
            hin["ids"] = hin["ids"].view(np.uint32)
        pos_h = None if not cfg.random_pos else synth.positions(cfg.index, T, True)
        host_ops = {
            "get_rows": lambda: be.get_rows_into(cfg.embd_dtype, table, table_bytes, cfg.vocab, H, hin["ids"], hout["emb"]),
            "rms_norm": lambda: be.rms_norm_into(hin["x"], w, hout["xn"], cfg.eps),
            "rope_qk": lambda: be.rope_host(hin["q"], hin["k"], nq, nkv, hd, cfg.n_rot, pos_h, cfg.theta),
            "qk_norm_rope_qk": lambda: be.rope_host(hin["q2"], hin["k2"], nq, nkv, hd, cfg.n_rot, pos_h, cfg.theta,
                                                    wq_dev=wq, wk_dev=wk, eps=cfg.eps),
            "silu_mul": lambda: be.silu_mul_into(hin["gate"], hin["up"], hout["act"]),
            "softmax": lambda: be.softmax_rows_into(hin["scores"], hout["probs"], causal_period=T),
        }

        def e2e_step():
            for o in order:
                host_ops[o]()
            be.sync()  # the step's results are read on the host

        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        # the link is shared with the other tenants of the host: the K-step region is repeated and the median taken
        e2e_regions = []
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(max(1, min(args.repeats, 5))):
            barrier()
            a.record(stream)
            for _ in range(e2e_steps):
                e2e_step()
            b.record(stream)
            barrier()
            e2e_regions.append(sharding.max_over_ranks(a.elapsed_time(b)) / e2e_steps)
        e2e_ms = float(np.median(e2e_regions))
        e2e = {"value": T_total / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms, "ms_per_step_min": min(e2e_regions), "ms_per_step_max": max(e2e_regions),
               "steps": e2e_steps, "repeats": len(e2e_regions),
               "api": "host-slice entry points (agn_host_*), pinned host arrays, staging ring over three streams"}

    # ---- the two other configurations a driver run should see: the decode chain (one GPU) and the large batch
    #      split over the ranks (every N).  The headline buffers make room first.
    decode_rec = split_rec = None
    if world == 1 and not args.no_decode and not f16:
        sw, fl, c3 = decode_sweep(torch, be, dev, stream, 20)
        decode_rec = {"workload": c3.name, "chain": "28 x (qk_norm_rope_qk + silu_mul), random positions", "sweep": sw,
                      "launch_floor": fl, "us_graph_T1": sw[0]["us_graph"]}
    if not args.no_split and not f16 and wl == "c2":
        for b in sets[1:]:
            b.clear()
        torch.cuda.empty_cache()
        split_rec = strong_split_record(torch, be, dev, stream, rank, world, barrier, sharding.max_over_ranks)

    # ---- verification.  (1) Against the CPU oracle, outside every timed region: the inputs of buffer set 0 are
    #      restored (the timed steps rotated q and k in place), every op runs once more, and a strided sample of
    #      rows of every output is compared with the oracle's result for the same input rows, which are read
    #      back from the device — bit-exact for the embedding rows and the routing, 1e-5 of the row scale for the
    #      float ops.  (2) Across ranks: per-rank checksums of the same outputs (set 0 is identical on every
    #      rank), gathered over the process group — the only collective.
    b0 = sets[0]
    if host0 is not None:
        for n in ("x", "q", "k", "gate", "up"):
            b0[n].copy_(up0(n))
        if "qk_norm_rope_qk" in order:
            b0["q2"].copy_(up0("q")); b0["k2"].copy_(up0("k"))
    else:
        gen.manual_seed(synth.BASE_SEED + 1000 * cfg.index)
        fresh = {n: rn(*b0[n].shape) for n in ("x", "q", "k", "gate", "up")}
        for n, t in fresh.items():
            b0[n].copy_(t)
        if "qk_norm_rope_qk" in order:
            b0["q2"].copy_(fresh["q"]); b0["k2"].copy_(fresh["k"])
        del fresh
    n_chk = min(T, args.check_rows)
    rows = np.unique(np.linspace(0, T - 1, n_chk).astype(np.int64))
    rows_t = torch.from_numpy(rows).to(dev)
    take = lambda t, idx=None: t.index_select(0, rows_t if idx is None else idx).float().cpu().numpy()
    ins = {n: take(b0[n]) for n in ("x", "q", "k")}
    rrows = np.unique(np.linspace(0, R - 1, n_chk).astype(np.int64)); rrows_t = torch.from_numpy(rrows).to(dev)
    ins["gate"], ins["up"] = take(b0["gate"], rrows_t), take(b0["up"], rrows_t)
    for name in order:
        ops[name](b0)
    be.sync()
    torch.cuda.synchronize()
    oracle_report = None
    if not f16 and not args.no_verify:
        from oracle import oracle as orc
        pos_h = synth.positions(cfg.index, T, cfg.random_pos)[rows]
        w_h, wq_h, wk_h = (synth.norm_weight(cfg.index, n, m) for n, m in (("w", H), ("wq", hd), ("wk", hd)))
        p999 = {}

        def rel(got, ref, key=None):  # max error relative to the row scale; its 99.9th percentile on the side
            if key is not None:
                p999[key] = max(p999.get(key, 0.0), synth.p999_rel_to_row_scale(got, ref))
            return synth.max_rel_to_row_scale(got, ref)

        err = {}
        for name in order:
            if name == "get_rows":
                ids_h = b0["ids"].cpu().numpy().view(np.uint32)[rows]
                _, ref = orc.get_rows(cfg.embd_dtype, table_h, cfg.vocab, H, ids_h)
                err[name] = 0.0 if np.array_equal(take(b0["emb"]).view(np.uint32), ref.view(np.uint32)) else float("inf")
            elif name == "rms_norm":
                err[name] = rel(take(b0["xn"]), orc.rms_norm_rows(ins["x"], w_h, cfg.eps), name)
            elif name == "rope_qk":
                err[name] = max(rel(take(b0["q"]), orc.rope_rows(ins["q"], nq, hd, cfg.n_rot, pos_h, cfg.theta), name),
                                rel(take(b0["k"]), orc.rope_rows(ins["k"], nkv, hd, cfg.n_rot, pos_h, cfg.theta), name))
            elif name == "qk_norm_rope_qk":
                err[name] = max(
                    rel(take(b0["q2"]), orc.qk_norm_rope_rows(ins["q"], wq_h, nq, hd, cfg.eps, cfg.n_rot, pos_h, cfg.theta), name),
                    rel(take(b0["k2"]), orc.qk_norm_rope_rows(ins["k"], wk_h, nkv, hd, cfg.eps, cfg.n_rot, pos_h, cfg.theta), name))
            elif name == "silu_mul":
                err[name] = rel(take(b0["act"], rrows_t), orc.silu_mul(ins["gate"], ins["up"]), name)
            elif name == "softmax":  # rows `rows` of every head; row i of a head has i + 1 valid entries
                sc = b0["scores"].index_select(1, rows_t).cpu().numpy().reshape(-1, T)
                pr = b0["probs"].index_select(1, rows_t).cpu().numpy().reshape(-1, T)
                err[name] = rel(pr, orc.softmax_rows(sc, np.tile(rows + 1, nq).astype(np.int32)), name)
            elif name == "router_top2":
                ridx_ref, rw_ref = orc.router_top2(take(b0["logits"]))
                same = np.array_equal(take(b0["ridx"]).astype(np.int32), ridx_ref)
                err[name] = float(np.max(np.abs(take(b0["rw"]) - rw_ref))) * 10.0 if same else float("inf")  # weights within 1e-6
            elif name == "gather_rows_by_expert":  # a global sort: the whole batch
                ref = orc.gather_rows_by_expert(b0["x"].cpu().numpy(), b0["ridx"].cpu().numpy(), E)
                got = (b0["gx"].cpu().numpy(), b0["goff"].cpu().numpy(), b0["gtok"].cpu().numpy(), b0["gslot"].cpu().numpy())
                err[name] = 0.0 if all(np.array_equal(g.view(np.uint32), r.view(np.uint32)) for g, r in zip(got, ref)) else float("inf")
        oracle_report = {"max_rel_err": {k: float(f"{v:.3g}") for k, v in err.items()},
                         "p999_rel_err": {k: float(f"{v:.3g}") for k, v in p999.items()}, "rows_checked": int(rows.size),
                         "tolerance": 1e-5, "bit_exact_ops": [o for o in order if o in ("get_rows", "gather_rows_by_expert")],
                         "ok": all(v <= 1e-5 for v in err.values()),
                         "how": "rows of buffer set 0 re-run after the timed regions, oracle fed the same input rows"}
    outs = ["emb", "xn", "q", "k", "act"] + (["q2", "k2"] if "qk_norm_rope_qk" in order else []) + \
           (["probs"] if "softmax" in order else []) + (["ridx", "gx"] if E else [])
    mine = [sharding.checksum(b0[n][: min(T, 512)].contiguous().cpu().numpy()) for n in outs]
    chk = sharding.gather_objects(mine)
    agree = all(c == chk[0] for c in chk)
    verified = agree and (oracle_report is None or oracle_report["ok"]) and (q8k_report is None or q8k_report["ok"])

    if rank == 0:
        peak, peak_src = measured_peaks()
        for rec in list(per_op.values()) + list(extra_ops.values()):
            rec["frac_of_peak"] = round(rec["gbs"] / peak, 3)
            rec["frac_of_nominal_8tbs"] = round(rec["gbs"] / 8000.0, 3)
        if silu_ms is None:  # the step ran as a graph replay: no events inside it; use the kernel-alone time
            silu_ms = per_op["silu_mul"]["us"] * 1e-3
        achieved = ab["silu_mul"] / (silu_ms * 1e-3) / 1e9
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "f32" if not f16 else "f16 storage, f32 arithmetic", "data": "synthetic",
            "config": workload_config(cfg, T, T_total, order, world),
            "timing": {"l2": f"inputs larger than L2: {nsets} rotating buffer sets, {step_bytes / 1e9:.2f} GB per step",
                       "launch": "one CUDA graph replay per step" if use_graph else "stream launches",
                       "preheat_steps": n_warm, "repeats": len(region_ms),
                       "ms_per_step_median": ms_per_step, "ms_per_step_min": min(region_ms) / args.steps,
                       "ms_per_step_max": max(region_ms) / args.steps,
                       "what": "K steps per region, regions back to back, each bracketed by barrier + synchronize; "
                               "value and ms_per_step are the median region"},
            "hbm_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9 * world,
            "hbm_frac_of_measured_peak": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
            "hbm_frac_of_nominal_8tbs": step_bytes / (ms_per_step * 1e-3) / 1e9 / 8000.0,
            "roofline": {"kernel": "silu_mul_vec4_kernel", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": "of measured (copy bandwidth, MEASURED_PEAKS.json)" if peak_src == "measured"
                         else "of fallback", "traffic": silu_traffic_bytes(R * I) if not f16 else None,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel at this "
                                           "size (profiles/dram_traffic_qwen7b_prefill_rows4096.md), scaled with the element "
                                           "count; not measured by this run",
                         "algorithmic_bytes_per_launch": ab["silu_mul"], "avg_launch_ms": silu_ms},
            "ops": per_op, "extra_ops": extra_ops, "clocks": clocks, "gpu_launches": launches, "e2e": e2e,
            "verification": {"ranks": len(chk), "outputs_checked": outs, "identical_across_ranks": agree,
                             "how": "checksums of every op's output for identical inputs, gathered over the process group",
                             "oracle": oracle_report, "q8_k_rows": q8k_report},
            "strong_c4": split_rec, "decode_c3": decode_rec,
        }
        if world == 1 and not args.no_cpu and not f16:
            out["cpu_baseline"] = cpu_baseline(cfg, order)
        if world == 1 and args.workload == "c2" and not args.no_others and not f16:
            out["other_workloads"] = other_workloads()
            if any(r.get("oracle_ok") is False for r in out["other_workloads"].values()):
                verified = False
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    be.close()
    if not verified:
        raise SystemExit("bench: outputs differ from the CPU oracle (or between ranks); see `verification` in the JSON line")


def other_workloads():
    """The two configurations the default line does not otherwise touch, each as a short run of this
    file in a child process on the same GPU (one GPU only): c1 (Llama-3.2-1B shapes with the causal
    softmax, launch-bound, one graph replay per step) and c5 (Mixtral-shaped MoE routing: router top-2, gather
    by expert, SiLU over the routed rows).  Device time per step, every op alone, and the comparison of the
    outputs with the CPU oracle."""
    recs = {}
    for w in ("c1", "c5"):
        cmd = [sys.executable, os.path.abspath(__file__), "--workload", w, "--no-e2e", "--no-cpu", "--no-split", "--no-decode",
               "--no-extras", "--no-others", "--repeats", "5", "--warm-seconds", "0.2"]
        try:
            p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
            lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
            if not lines:
                recs[w] = {"unavailable": f"child exited {p.returncode}: {p.stderr.strip()[-200:]}"}
                continue
            d = json.loads(lines[-1])
            orc_rep = (d.get("verification") or {}).get("oracle") or {}
            recs[w] = {"workload": d["config"]["workload"], "tokens": d["config"].get("tokens_per_gpu"), "steps": d["steps"],
                       "ms_per_step": d["ms_per_step"], "tokens_per_s": d["value"], "launch": d["timing"]["launch"],
                       "hbm_gbs": d["hbm_gbs"], "hbm_frac_of_measured_peak": d["hbm_frac_of_measured_peak"],
                       "ops": {k: {"us": v["us"], "gbs": v["gbs"]} for k, v in d["ops"].items()},
                       "oracle_ok": orc_rep.get("ok"), "oracle_max_rel_err": orc_rep.get("max_rel_err"),
                       "gpu_launches": d.get("gpu_launches")}
        except Exception as e:  # a child that hangs or prints something else: say so, keep the headline
            recs[w] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    return recs


def decode_sweep(torch, be, dev, stream, steps, seed_salt=0):
    """Decode-shaped latency sweep (Qwen2.5-7B shapes): for T in {1, 8, 32, 64} tokens per step with
    random positions, the fused norm->rope and SiLU*mul kernels run back to back for 28 layers.
    Timed as plain stream launches and as one CUDA graph replay.  Returns (sweep, launch floor)."""
    from agention_infer_b200 import synth
    cfg = synth.CONFIGS["c3"]
    H, hd, nq, nkv, I, layers = cfg.hidden, cfg.head_dim, cfg.n_q_heads, cfg.n_kv_heads, cfg.ffn, 28
    wq = torch.from_numpy(synth.norm_weight(cfg.index, "wq", hd)).to(dev)
    wk = torch.from_numpy(synth.norm_weight(cfg.index, "wk", hd)).to(dev)
    gen = torch.Generator(device=dev); gen.manual_seed(synth.BASE_SEED + 3000 + seed_salt)
    sweep = []

    def timed(fn, reps):
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            fn()
        b_.record(stream); torch.cuda.synchronize()
        return a.elapsed_time(b_) * 1e3 / reps

    # the floor: the same number of empty kernels, as plain launches and as a graph
    def noops():
        for _ in range(2 * layers):
            be.launch_noop()
    for _ in range(3):
        noops()
    torch.cuda.synchronize()
    floor_plain = timed(noops, 20)
    be.graph_begin(); noops(); g0 = be.graph_end()
    for _ in range(3):
        be.graph_launch(g0)
    floor_graph = timed(lambda: be.graph_launch(g0), 50)
    be.graph_destroy(g0)
    reps = max(steps, 20)
    for T in (1, 8, 32, 64):
        pos = torch.from_numpy(synth.positions(cfg.index, T, True)).to(dev)
        # one buffer set per layer: 28 layers of activations are distinct memory, as in the engine
        L = [{"q": torch.randn(T, nq * hd, device=dev, generator=gen), "k": torch.randn(T, nkv * hd, device=dev, generator=gen),
              "gate": torch.randn(T, I, device=dev, generator=gen), "up": torch.randn(T, I, device=dev, generator=gen),
              "act": torch.empty(T, I, device=dev)} for _ in range(layers)]

        def chain():
            for b in L:
                be.launch_qk_norm_rope_qk(b["q"], b["k"], wq, wk, T, nq, nkv, hd, cfg.eps, cfg.n_rot, pos, cfg.theta)
                be.launch_silu_mul(b["gate"], b["up"], T * I, out=b["act"])

        for _ in range(5):
            chain()
        torch.cuda.synchronize()
        us_plain = timed(chain, reps)
        be.graph_begin(); chain(); g = be.graph_end()  # recorded through the library's own graph entry points
        for _ in range(5):
            be.graph_launch(g)
        torch.cuda.synchronize()
        us_graph = timed(lambda: be.graph_launch(g), reps)
        be.graph_destroy(g)
        bytes_chain = layers * (8 * T * (nq + nkv) * hd + 12 * T * I)
        sweep.append({"T": T, "layers": layers, "launches": 2 * layers, "us_plain": round(us_plain, 2),
                      "us_graph": round(us_graph, 2), "us_per_layer_graph": round(us_graph / layers, 3),
                      "gbs_graph": round(bytes_chain / (us_graph * 1e-6) / 1e9, 1),
                      "tokens_per_s_graph": round(T / (us_graph * 1e-6), 1)})
    floor = {"kernels": 2 * layers, "us_plain": round(floor_plain, 2), "us_graph": round(floor_graph, 2),
             "what": "the same number of empty kernels"}
    return sweep, floor, cfg


def run_decode_sweep(args):
    """`--workload c3`: the decode sweep as the run's own JSON line."""
    torch, dist, be, dev, stream, sampler, rank, world, local = setup_cuda(args)
    if sampler:
        sampler.mark_load(True)
    sweep, floor, cfg = decode_sweep(torch, be, dev, stream, args.steps, seed_salt=rank)
    if sampler:
        sampler.mark_load(False)
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        best = sweep[-1]
        print(json.dumps({
            "metric": "decode_layer_chain_tokens_per_s", "value": best["tokens_per_s_graph"], "unit": UNIT, "n_gpus": world,
            "steps": max(args.steps, 20), "warmup": 5, "ms_per_step": best["us_graph"] / 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg.name, "chain": "28 x (qk_norm_rope_qk + silu_mul)", "hidden": cfg.hidden, "ffn": cfg.ffn,
                       "positions": "random in [0, 32768)", "timing": "CUDA graph replay vs plain launches"},
            "launch_floor": floor,
            "sweep": sweep, "clocks": clocks, "gpu_launches": 2 * 28 * max(args.steps, 20), "e2e": None}))
    if world > 1:
        dist.destroy_process_group()
    be.close()


def strong_split_record(torch, be, dev, stream, rank, world, barrier, max_over_ranks, steps=10):
    """The large prefill batch (Llama-3-8B shapes, T = 65536 token rows, Q6_K embedding 128256 x 4096) with its rows
    SPLIT over the ranks: T / world rows per GPU, no data-path collective.  Device time of K steps (max over ranks)
    and of every op alone.  With more than one rank, rank 0 then runs the whole batch by itself, so that the
    efficiency against one GPU comes from the same invocation."""
    from agention_infer_b200 import sharding, synth
    cfg = synth.CONFIGS["c4"]
    ops_list = WORKLOADS["c4"][1]
    H, hd, nq, nkv, I = cfg.hidden, cfg.head_dim, cfg.n_q_heads, cfg.n_kv_heads, cfg.ffn
    table_h = synth.quant_table(cfg.embd_dtype, cfg.vocab, H, cfg_index=cfg.index)
    table = torch.from_numpy(table_h).to(dev)
    w = torch.from_numpy(synth.norm_weight(cfg.index, "w", H)).to(dev)
    wq = torch.from_numpy(synth.norm_weight(cfg.index, "wq", hd)).to(dev)
    wk = torch.from_numpy(synth.norm_weight(cfg.index, "wk", hd)).to(dev)
    gen = torch.Generator(device=dev)

    def measure(T, row0, collective):
        nsets = 2 if T > 16384 else 4  # every launch reads inputs that are not in L2 (>= 2 GB per set)
        pos = torch.arange(row0, row0 + T, dtype=torch.int32, device=dev)
        sets = []
        for s_ in range(nsets):
            gen.manual_seed(synth.BASE_SEED + 4000 + 7919 * (1 + rank * NSETS + s_))
            rn = lambda *shape: torch.randn(*shape, device=dev, generator=gen)
            ids = torch.from_numpy(synth.token_ids(cfg.index, T, cfg.vocab, salt=1 + rank * NSETS + s_).astype(np.int32)).to(dev)
            sets.append({"ids": ids, "emb": torch.empty(T, H, device=dev), "x": rn(T, H), "xn": torch.empty(T, H, device=dev),
                         "q": rn(T, nq * hd), "k": rn(T, nkv * hd), "q2": rn(T, nq * hd), "k2": rn(T, nkv * hd),
                         "gate": rn(T, I), "up": rn(T, I), "act": torch.empty(T, I, device=dev)})
        ops = {
            "get_rows": lambda b: be.get_rows(cfg.embd_dtype, table, table_h.nbytes, cfg.vocab, H, b["ids"], T, out=b["emb"]),
            "rms_norm": lambda b: be.launch_rms_norm(b["x"], w, T, H, cfg.eps, out=b["xn"]),
            "rope_qk": lambda b: be.launch_rope_qk(b["q"], b["k"], T, nq, nkv, hd, cfg.n_rot, pos, cfg.theta),
            "qk_norm_rope_qk": lambda b: be.launch_qk_norm_rope_qk(b["q2"], b["k2"], wq, wk, T, nq, nkv, hd, cfg.eps, cfg.n_rot,
                                                                   pos, cfg.theta),
            "silu_mul": lambda b: be.launch_silu_mul(b["gate"], b["up"], T * I, out=b["act"]),
        }
        ab = op_bytes(cfg, T, ops_list)

        def step(i):
            for name in ops_list:
                ops[name](sets[i % nsets])

        sync = barrier if collective else torch.cuda.synchronize
        for i in range(3):
            step(i)
        sync()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for i in range(steps):
            step(i)
        b_.record(stream)
        sync()
        ms = a.elapsed_time(b_)
        if collective:
            ms = max_over_ranks(ms)
        per_op = {}
        for name in ops_list:
            for i in range(2):
                ops[name](sets[i % nsets])
            torch.cuda.synchronize()
            a.record(stream)
            for i in range(steps):
                ops[name](sets[i % nsets])
            b_.record(stream)
            torch.cuda.synchronize()
            us = a.elapsed_time(b_) * 1e3 / steps
            per_op[name] = {"us": round(us, 2), "gbs": round(ab[name] / (us * 1e-6) / 1e9, 1)}
        del sets
        torch.cuda.empty_cache()
        return ms / steps, per_op, sum(ab.values())

    r0, r1 = sharding.shard_rows(cfg.T, rank, world)
    ms_split, per_op, bytes_rank = measure(r1 - r0, r0, world > 1)
    rec = {"workload": cfg.name, "scaling": "strong", "tokens_total": cfg.T, "tokens_per_gpu": r1 - r0, "n_gpus": world,
           "steps": steps, "ms_per_step": ms_split, "tokens_per_s": cfg.T / (ms_split * 1e-3),
           "hbm_gbs_per_gpu": bytes_rank / (ms_split * 1e-3) / 1e9, "ops_rank0": per_op,
           "embedding": f"{DTYPE_NAMES[cfg.embd_dtype]} {cfg.vocab}x{H}"}
    if world == 1:
        rec.update(ms_per_step_n1=ms_split, efficiency_vs_n1=1.0)
    else:
        ms_n1 = None
        if rank == 0:  # the other ranks wait at the barrier below
            ms_n1, _, _ = measure(cfg.T, 0, False)
        barrier()
        rec.update(ms_per_step_n1=ms_n1, efficiency_vs_n1=(ms_n1 / world / ms_split) if ms_n1 else None,
                   n1_how="rank 0 ran all 65536 rows by itself in the same invocation, the other ranks idle")
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 200; 5 for --impl reference)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=list(WORKLOADS) + ["c3"], default="c2",
                    help="c2 (default, the headline): Qwen2.5-7B-shaped prefill, T=4096 rows per GPU; c1: Llama-3.2-1B "
                         "shapes incl. causal softmax; c3: decode latency sweep; c4: T=65536 Llama-3-8B-shaped rows "
                         "split over the GPUs; c5: Mixtral-shaped MoE routing ops")
    ap.add_argument("--act", choices=["f32", "f16"], default="f32",
                    help="activation storage: f32 (the benchmark's contract) or f16 (the reference GPU path's default)")
    ap.add_argument("--graph", choices=["auto", "on", "off"], default="auto",
                    help="run each step as one CUDA graph replay (auto: for launch-bound steps under 200 MB)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the ops measured outside the step")
    ap.add_argument("--no-pdl", action="store_true", help="plain stream-ordered launches (for comparison)")
    ap.add_argument("--set-option", action="append", metavar="NAME=INT",
                    help="a tuning knob passed to agn_ctx_set_option before the run (repeatable)")
    ap.add_argument("--no-verify", action="store_true", help="skip the comparison of the outputs with the CPU oracle")
    ap.add_argument("--no-split", action="store_true", help="skip the strong_c4 record (the large batch split over the ranks)")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode_c3 record (one GPU)")
    ap.add_argument("--no-others", action="store_true", help="skip the other_workloads record (c1 and c5 as child runs, one GPU); implied by --no-split with --no-decode "
                         "(the headline workload alone)")
    ap.add_argument("--repeats", type=int, default=25, help="how many times the K-step timed region is repeated (median reported)")
    ap.add_argument("--check-rows", type=int, default=64, help="rows of every output compared with the oracle")
    ap.add_argument("--warm-seconds", type=float, default=0.6,
                    help="minimum duration of the warm-up (0 for profiling runs)")
    ap.add_argument("--tokens", type=int, default=None,
                    help="token rows (default: the configuration's); smaller values are for profiling")
    args = ap.parse_args()
    from agention_infer_b200 import synth
    if args.no_split and args.no_decode:
        args.no_others = True
    if args.steps is None:
        args.steps = 5 if args.impl == "reference" else (200 if args.workload in ("c1", "c2", "c3") else 20)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "ours" and world == 1 and args.gpus > 1:
        # not under torchrun: relaunch one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29517", __file__, *sys.argv[1:]]
        sys.exit(subprocess.call(cmd))
    if args.workload == "c3":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the decode latency sweep has no host arm"}))
            return
        return run_decode_sweep(args)
    key, ops, _ = WORKLOADS[args.workload]
    cfg = synth.CONFIGS[key]
    if args.tokens:
        cfg = dataclasses.replace(cfg, T=args.tokens, name=f"{cfg.name} (rows overridden to {args.tokens})")
    if args.impl == "reference":
        run_reference(args, cfg, ops, args.workload)
    else:
        run_ours(args, cfg, ops, args.workload)


if __name__ == "__main__":
    main()

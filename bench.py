#!/usr/bin/env python
"""Benchmark of the W4A16 decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one pass of the Llama-3-8B-shape W4A16 decode layer chain (rms_norm -> QKV int4
GEMM -> RoPE + kv append -> GQA decode attention -> o_proj -> add+rms_norm -> gate_up int4
-> silu_mul -> down int4 -> add) over one batch of 64 sequences with 4096 tokens of context
each, on synthetic seeded data.  Prints ONE JSON line.  With N > 1 (under torchrun) the
layer is tensor-parallel over N ranks (column-parallel QKV / gate_up, row-parallel o / down
with an all-reduce, attention by KV head); the batch is fixed, so scaling is strong.

`--impl reference` times the CPU restatement of the same chain (the reference has no CPU
implementation and cannot be built here) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes
import importlib
import json
import os
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BATCH, CTX = 64, 4096
N_SETS = 4                    # distinct weight + KV sets rotated step by step (4 x 1.2 GB >> L2)
METRIC = "layer tok/s (Llama-3-8B-shape W4A16 decode layer, batch 64, ctx 4096)"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


# --------------------------------------------------------------------------------------
# CPU legs (the only place the oracle is executed by this file)
# --------------------------------------------------------------------------------------
def load_oracle_c():
    so = ROOT / "oracle" / "liboracle_c.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True)
    oc = ctypes.CDLL(str(so))
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    oc.oc_set_num_threads(cores)        # all host cores, whatever OMP_NUM_THREADS the launcher exported
    return oc


def cpu_layer_case(rng, batch, ctx):
    """Seeded inputs of the layer chain at the benchmark's extents, `batch` sequences."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle as o
    H, hq, hkv, d, I, G = 4096, 32, 8, 128, 14336, 128
    ml = ctx + 1

    def gptq(k, n):
        # nibbles 1..15 around the zero-point 8 (stored 7, +1 in the GEMM): weights without a DC component, so the
        # 14336-deep down projection stays inside fp16 and the result can be compared (same cost as any nibbles)
        qw = np.zeros((k // 8, n), dtype=np.uint32)
        for i in range(8):
            qw |= rng.integers(1, 16, (k // 8, n), dtype=np.uint32) << np.uint32(4 * i)
        return (qw.view(np.int32), rng.uniform(0.002, 0.02, (k // G, n)).astype(np.float16),
                np.full((k // G, n // 8), 0x77777777, dtype=np.int32))
    cos, sin = o.rope_tables(ml, d, 500000.0)
    case = dict(H=H, hq=hq, hkv=hkv, d=d, I=I, G=G, ml=ml, cos=cos, sin=sin,
                ln1=rng.uniform(0.5, 1.5, H).astype(np.float16), ln2=rng.uniform(0.5, 1.5, H).astype(np.float16),
                qkv=gptq(H, (hq + 2 * hkv) * d), o=gptq(hq * d, H), gate_up=gptq(H, 2 * I), down=gptq(I, H),
                hidden=rng.standard_normal((batch, H)).astype(np.float16),
                pos=np.full(batch, ctx, dtype=np.int32))
    # the cache of 4 sequences, repeated: same arithmetic cost, a quarter of the set-up time
    base_k = rng.standard_normal((min(batch, 4), hkv, ml, d), dtype=np.float32).astype(np.float16)
    base_v = rng.standard_normal((min(batch, 4), hkv, ml, d), dtype=np.float32).astype(np.float16)
    reps = -(-batch // base_k.shape[0])
    case["kc"] = np.ascontiguousarray(np.tile(base_k, (reps, 1, 1, 1))[:batch])
    case["vc"] = np.ascontiguousarray(np.tile(base_v, (reps, 1, 1, 1))[:batch])
    return case


def cpu_layer_run(oc, c):
    batch = c["hidden"].shape[0]
    out = np.zeros((batch, c["H"]), np.float32)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    args = [ptr(c["hidden"]), ptr(out), batch, c["H"], c["hq"], c["hkv"], c["d"], c["I"], c["G"], 1,
            ctypes.c_float(1e-5), ptr(c["ln1"]), ptr(c["ln2"])]
    for name in ("qkv", "o", "gate_up", "down"):
        args += [ptr(x) for x in c[name]]
    args += [ptr(c["cos"]), ptr(c["sin"]), ptr(c["pos"]), ptr(c["kc"]), ptr(c["vc"]), c["ml"]]
    t0 = time.perf_counter()
    oc.oc_decode_layer(*args)
    return time.perf_counter() - t0, out


def cpu_baseline(sample_batch=BATCH, reps=3, gate=None):
    """Times the CPU restatement on the benchmark's extents; `gate(case, cpu_out)` (optional) then checks the
    library's result on the very same inputs against it."""
    oc = load_oracle_c()
    oc.oc_num_threads.restype = ctypes.c_int
    cores = oc.oc_num_threads()
    case = cpu_layer_case(np.random.default_rng(4), sample_batch, CTX)
    _, out = cpu_layer_run(oc, case)             # warm-up (page in, thread pool); every run appends the same K/V row
    ts = [cpu_layer_run(oc, case)[0] for _ in range(reps)]
    best = min(ts)
    line = {"value": sample_batch / best, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{sample_batch} of {BATCH} sequences, ctx {CTX}, full layer chain, best of {reps}"}
    return line, (gate(case, out) if gate else None)


def parity_gate(pkg, torch, dev, case, cpu_out):
    """The whole config-4 layer through the C ABI on the CPU leg's inputs, against the CPU result."""
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    shape = pkg.LayerShape()
    w = {k: tuple(t(x) for x in case[k]) for k in ("qkv", "o", "gate_up", "down")}
    layer = pkg.DecodeLayer(shape, w, t(case["ln1"]), t(case["ln2"]), t(case["cos"]), t(case["sin"]),
                            max_batch=case["hidden"].shape[0], max_len=case["ml"], use_graph=False,
                            k_cache=t(case["kc"]), v_cache=t(case["vc"]))
    got = layer.forward(t(case["hidden"]), t(case["pos"])).float().cpu().numpy()
    layer.close()
    # Outputs of this layer are O(30) (unit-variance input through a 14336-deep projection), so the absolute part of
    # the tolerance (2e-2, as in the layer tests) scales with the output's RMS: |got - ref| <= 2e-2 |ref| + 2e-2 rms(ref);
    # the relative RMS error must also stay below 5e-3 (fp16 storage between the ten kernels gives about 2e-3)
    err = np.abs(got.astype(np.float64) - cpu_out)
    rms_ref = float(np.sqrt(np.mean(np.square(cpu_out, dtype=np.float64))))
    bound = 2e-2 * np.abs(cpu_out) + 2e-2 * rms_ref
    finite = bool(np.isfinite(got).all() and np.isfinite(cpu_out).all())
    rms_err = float(np.sqrt(np.nanmean(err * err)))
    ok = finite and bool((err <= bound).all()) and rms_err <= 5e-3 * rms_ref
    return {"what": "config-4 layer (batch 64, ctx 4096) through the C ABI vs the CPU restatement, same inputs",
            "tolerance": "|got - ref| <= 2e-2 |ref| + 2e-2 rms(ref) and rms(err) <= 5e-3 rms(ref)",
            "max_abs_err": float(np.nanmax(err)), "rms_err": rms_err, "rms_ref": rms_ref,
            "max_abs_ref": float(np.nanmax(np.abs(cpu_out))),
            "worst_err_over_bound": float(np.nanmax(err / bound)), "ok": ok}


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons of one GPU, read (never set) through NVML every few milliseconds by a
    background thread while the timed regions run."""
    BITS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, torch, index):
        self.samples, self.reasons, self.max_mhz, self._stop, self._thr = [], set(), None, False, None
        self.err = None
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self._thr = threading.Thread(target=self._run, daemon=True)
        except Exception as e:      # no NVML: the line says so instead of inventing numbers
            self.err = f"{type(e).__name__}: {e}"

    def _run(self):
        nv = self.nv
        while not self._stop:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for name, bit in self.BITS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception as e:
                self.err = f"{type(e).__name__}: {e}"
                return
            time.sleep(0.004)

    def start(self):
        if self._thr:
            self._thr.start()

    def stop(self):
        self._stop = True
        if self._thr:
            self._thr.join(timeout=2)
        sm = sorted(self.samples)
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
               "samples": len(sm)}
        if self.err:
            out["note"] = self.err
        return out


def component_metrics(pkg, torch, dev, gen):
    """The other parts of the compound metric: W4A16 GEMM TFLOP/s and GB/s (configs 0 and 2), decode
    attention GB/s (config 1), fused MoE (config 3).  Small kernels are replayed from a CUDA graph over
    rotating weight buffers (> 400 MB in total) so that every launch streams from HBM."""
    P = pkg.prelude
    hbm_peak, tf_peak, _ = peaks()

    def graph_time(fn, calls, reps=5):
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            for _ in range(calls):
                fn()
        gr.replay()
        torch.cuda.synchronize()
        best = 1e30
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); gr.replay(); b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b) / calls)
        return best   # ms per call

    def ri(*s):
        return torch.randint(-2 ** 31, 2 ** 31 - 1, s, device=dev, dtype=torch.int32, generator=gen)

    out = {}
    G = 128
    for fmt, m, k, n in [("gptq", 16, 4096, 4096), ("gptq", 1, 4096, 4096), ("awq", 1, 4096, 28672),
                         ("awq", 16, 4096, 28672), ("awq", 128, 4096, 6144), ("awq", 1024, 4096, 6144),
                         ("awq", 1024, 14336, 4096)]:
        nbuf = max(2, int(400e6 // (k * n // 2)))
        qws = [ri(k // 8, n) if fmt == "gptq" else ri(k, n // 8) for _ in range(nbuf)]
        sc = (torch.rand((k // G, n), device=dev, generator=gen) * 0.018 + 0.002).half()
        qz = ri(k // G, n // 8)
        a = torch.randn((m, k), device=dev, generator=gen, dtype=torch.float16)
        c = torch.empty((m, n), device=dev, dtype=torch.float16)
        i = [0]

        def fn():
            i[0] = (i[0] + 1) % nbuf
            (P.gptq_gemm if fmt == "gptq" else P.awq_gemm)(a, qws[i[0]], sc, qz, G, out=c)
        ms = graph_time(fn, 2 * nbuf)
        byts = k * n // 2 + (k // G) * n * 2 + (k // G) * n // 2 + 2 * m * k + 2 * m * n
        out[f"{fmt}_gemm_m{m}_k{k}_n{n}"] = {
            "us": ms * 1e3, "GB/s": byts / ms / 1e6, "TFLOP/s": 2 * m * k * n / ms / 1e9,
            "frac_hbm": byts / ms / 1e6 / hbm_peak, "frac_tensor": 2 * m * k * n / ms / 1e9 / tf_peak,
            "timing": "cold (rotating weight buffers), CUDA-graph replay of back-to-back launches (the set-up of a launch overlaps the tail of the one before: programmatic dependent launch)"}
        del qws
    # config 1: decode attention, batch 32, lengths U[512, 8192]
    b, hq, hkv, d, ml = 32, 32, 8, 128, 8192
    q = torch.randn((b, hq, d), device=dev, generator=gen, dtype=torch.float16)
    kc = torch.randn((b, hkv, ml, d), device=dev, generator=gen, dtype=torch.float16)
    vc = torch.randn((b, hkv, ml, d), device=dev, generator=gen, dtype=torch.float16)
    lens = torch.randint(512, ml + 1, (b,), device=dev, dtype=torch.int32, generator=gen)
    ao = torch.empty_like(q)
    ms = graph_time(lambda: P.batched_decode_attention_hm_f16(q, kc, vc, lens, ao, b, hq, hkv, d, ml, 1.0 / float(np.sqrt(d))), 4)
    byts = 4096 * int(lens.sum()) + 2 * b * hq * d * 2
    out["decode_attention_c1"] = {"us": ms * 1e3, "GB/s": byts / ms / 1e6, "frac_hbm": byts / ms / 1e6 / hbm_peak,
                                  "sum_len": int(lens.sum()), "timing": "inputs (537 MB) larger than L2"}
    del kc, vc
    # config 3: fused MoE, Mixtral-8x7B shape
    T, E, kk, H, I = 512, 8, 2, 4096, 14336
    w13q, w2q = ri(E, H // 8, 2 * I), ri(E, I // 8, H)
    w13s = (torch.rand((E, H // G, 2 * I), device=dev, generator=gen) * 0.018 + 0.002).half()
    w2s = (torch.rand((E, I // G, H), device=dev, generator=gen) * 0.018 + 0.002).half()
    x = torch.randn((T, H), device=dev, generator=gen, dtype=torch.float16)
    lg = torch.randn((T, E), device=dev, generator=gen)
    mo = torch.empty((T, H), dtype=torch.float16, device=dev)
    ms = graph_time(lambda: P.fused_moe_gptq_f16(x, lg, w13q, w13s, None, w2q, w2s, None, mo, T, H, E, kk, I, G, None, 0), 2)
    flops = T * kk * (2 * H * 2 * I + 2 * I * H)
    out["fused_moe_c3"] = {"us": ms * 1e3, "TFLOP/s": flops / ms / 1e9, "frac_tensor": flops / ms / 1e9 / tf_peak,
                           "weight_GB/s": 726663168 / ms / 1e6,
                           "timing": "weights (727 MB) larger than L2"}
    return out


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    pkg = importlib.import_module("triton-rs_b200")
    P = pkg.prelude
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N > 1 through torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    def note(msg):
        if os.environ.get("BENCH_VERBOSE"):
            print(f"[rank {rank}] {time.strftime('%H:%M:%S')} {msg}", file=sys.stderr, flush=True)

    if world > 1:
        import datetime
        # a collective that cannot complete ends with an error after 5 minutes instead of waiting for ever
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
        note("process group up")
    pkg.lib().call("b200k_device_check")

    shape = pkg.LayerShape()
    ls = shape.local(world)
    H, d, G = shape.hidden, shape.head_dim, shape.group_size
    ml = CTX + 1
    gen = torch.Generator(device=dev).manual_seed(1234)      # same seed on every rank: identical full weights

    def rand_i32(*s):
        return torch.randint(-2 ** 31, 2 ** 31 - 1, s, device=dev, dtype=torch.int32, generator=gen)

    def gptq(k, n):
        # nibbles uniform 0..15; symmetric zero-point 8 = stored nibble 7 under the GPTQ GEMM's +1 rule
        return (rand_i32(k // 8, n), (torch.rand((k // G, n), device=dev, generator=gen) * 0.018 + 0.002).half(),
                torch.full((k // G, n // 8), 0x77777777, device=dev, dtype=torch.int32))

    sys.path.insert(0, str(ROOT / "oracle"))
    half = d // 2
    inv_freq = 1.0 / (shape.rope_theta ** (torch.arange(half, dtype=torch.float64) * 2.0 / d))
    ang = torch.arange(ml, dtype=torch.float64)[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)

    # N > 1: the library's own peer-to-peer all-reduce inside its captured layer chain;
    # BENCH_TP_COMM=nccl runs the staged chain with NCCL all-reduces between the stages instead
    own_comm = world > 1 and os.environ.get("BENCH_TP_COMM", "p2p") == "p2p"
    comm = pkg.Comm.from_process_group(BATCH * H * 2) if own_comm else None
    layers = []
    for _ in range(N_SETS):
        full = {"qkv": gptq(H, (shape.num_q_heads + 2 * shape.num_kv_heads) * d), "o": gptq(shape.num_q_heads * d, H),
                "gate_up": gptq(H, 2 * shape.intermediate), "down": gptq(shape.intermediate, H)}
        w = pkg.shard_layer_weights(full, shape, rank, world) if world > 1 else full
        del full
        ln1 = (torch.rand(H, device=dev, generator=gen) + 0.5).half()
        ln2 = (torch.rand(H, device=dev, generator=gen) + 0.5).half()
        kc = torch.randn((BATCH, ls.num_kv_heads, ml, d), device=dev, generator=gen, dtype=torch.float16)
        vc = torch.randn((BATCH, ls.num_kv_heads, ml, d), device=dev, generator=gen, dtype=torch.float16)
        layers.append(pkg.DecodeLayer(ls, w, ln1, ln2, cos, sin, max_batch=BATCH, max_len=ml,
                                      use_graph=(world == 1 or own_comm), k_cache=kc, v_cache=vc))
        if comm is not None:
            layers[-1].set_comm(comm)
    hidden = torch.randn((BATCH, H), device=dev, generator=gen, dtype=torch.float16)
    positions = torch.full((BATCH,), CTX, device=dev, dtype=torch.int32)
    out = torch.empty_like(hidden)
    stream = torch.cuda.current_stream()

    # ---- one step -----------------------------------------------------------------------
    part = torch.empty_like(hidden)
    part2 = torch.empty_like(hidden)

    def step_single(i):
        layers[i % N_SETS].forward(hidden, positions, out=out)

    def step_tp_eager(i):
        L = layers[i % N_SETS]
        L.forward_stage(0, hidden=hidden, positions=positions, partial=part, batch=BATCH)
        dist.all_reduce(part)
        L.forward_stage(1, hidden=hidden, reduced=part, partial=part2, batch=BATCH)
        dist.all_reduce(part2)
        L.forward_stage(2, reduced=part2, out=out, batch=BATCH)

    tp_graphs = []
    if world > 1 and not own_comm:
        note("layers built")
        for i in range(N_SETS):           # first-use set-up outside any capture
            step_tp_eager(i)
        torch.cuda.synchronize()
        note("eager steps done")
    if world > 1 and not own_comm and not os.environ.get("BENCH_NO_TP_GRAPH"):
        try:
            for i in range(N_SETS):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    step_tp_eager(i)
                tp_graphs.append(g)
        except Exception:                 # capture of the collective not possible: stay eager
            tp_graphs = []
            torch.cuda.synchronize()

    def step(i):
        if world == 1 or own_comm:
            step_single(i)
        elif tp_graphs:
            tp_graphs[i % N_SETS].replay()
        else:
            step_tp_eager(i)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()                        # ranks enter the first exchange together (its wait is bounded to about a second)
    note(f"tp graphs: {len(tp_graphs)}")
    sampler = ClockSampler(torch, local)
    if rank == 0:
        sampler.start()              # samples every 25 ms from warm-up to the last timed kernel
    for i in range(max(args.warmup, 3) + N_SETS):    # graph capture happens on first use of each set
        step(i)
    barrier()
    note("warm-up done")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    note(f"timed region done: {ms_total / args.steps:.3f} ms/step")
    if world > 1:
        tt = torch.tensor([ms_total], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total = float(tt.item())
    ms_step = ms_total / args.steps

    # ---- end to end through the C ABI with host buffers (N = 1: one call; N > 1: staged) ----
    hh = hidden.cpu().pin_memory()
    hp = positions.cpu().pin_memory()
    ho = torch.empty((BATCH, H), dtype=torch.float16).pin_memory()

    def e2e_step(i):
        if world == 1 or own_comm:
            layers[i % N_SETS].forward_host(hh, hp, ho)
        else:
            hidden.copy_(hh, non_blocking=True)
            positions.copy_(hp, non_blocking=True)
            step(i)
            ho.copy_(out, non_blocking=True)
        stream.synchronize()              # the caller reads the result before the next decode step

    note("e2e warm-up")
    for i in range(3):
        e2e_step(i)
    note("e2e warm-up steps issued")
    barrier()
    note("e2e timed")
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    if world > 1:
        tt = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item())

    note(f"e2e done: {e2e_ms:.3f} ms/step")
    # ---- the dominant kernel (decode attention) timed alone on the same rotating caches ----
    q = torch.randn((BATCH, ls.num_q_heads, d), device=dev, generator=gen, dtype=torch.float16)
    lens = torch.full((BATCH,), ml, device=dev, dtype=torch.int32)
    ao = torch.empty_like(q)
    scale = 1.0 / float(np.sqrt(d))

    def attn(i):
        L = layers[i % N_SETS]
        P.batched_decode_attention_hm_f16(q, L.k_cache, L.v_cache, lens, ao, BATCH, ls.num_q_heads, ls.num_kv_heads, d,
                                          ml, scale)
    for i in range(N_SETS):
        attn(i)
    torch.cuda.synchronize()
    n_at = max(args.steps, 8)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_at)]
    for i, (a, b) in enumerate(evs):
        a.record(); attn(i); b.record()
    torch.cuda.synchronize()
    attn_ms = sum(a.elapsed_time(b) for a, b in evs) / n_at
    note("attention timed")
    clocks = sampler.stop() if rank == 0 else None
    note("sampler stopped")

    components = component_metrics(pkg, torch, dev, gen) if world == 1 and not args.no_components else None

    status = ctypes.c_int(-1)
    pkg.lib().call("b200k_device_status", ctypes.addressof(status), stream.cuda_stream)

    if rank == 0:
        hbm_peak, tf_peak, peak_kind = peaks()
        attn_bytes = 2 * BATCH * ls.num_kv_heads * ml * d * 2 + 2 * BATCH * ls.num_q_heads * d * 2
        achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": BATCH / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage, int4 weights, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": "C4: Llama-3-8B-shape W4A16 (GPTQ) decode layer chain, batch 64, ctx 4096",
                       "parallelism": f"tp{world}" if world > 1 else "single GPU",
                       "l2": f"inputs larger than L2: {N_SETS} weight+KV sets rotated, "
                             f"{(2 * BATCH * ls.num_kv_heads * ml * d * 2) / 1e9:.2f} GB of KV per step",
                       "all_reduce": None if world == 1 else ("own one-shot kernel over NVLink peer memory" if own_comm else "NCCL"),
                       "graph": bool(world == 1 or own_comm or tp_graphs), "device_status": status.value,
                       "comm_status": comm.status() if comm is not None else None},
            "e2e": {"value": BATCH / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": BATCH * H * 2 + BATCH * 4, "d2h_bytes_per_step": BATCH * H * 2},
            "gpu_launches": (layers[0].launches_per_forward) * args.steps,
            "roofline": {"kernel": "attn_split_f16_kernel", "bound": "hbm", "achieved": achieved, "peak": hbm_peak,
                         "unit": "GB/s", "frac": achieved / hbm_peak, "peak_kind": peak_kind,
                         # dram bytes per launch: ncu capture of a smaller launch of this kernel (profiles/
                         # attn_split_f16_b8_ctx4096.md: 1.033 x algorithmic), scaled to this launch
                         "traffic": int(attn_bytes * 1.033),
                         "algorithmic_bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms},
            "clocks": clocks,
        }
        if components is not None:
            line["components"] = components
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"], line["parity"] = cpu_baseline(gate=lambda c, o: parity_gate(pkg, torch, dev, c, o))
            if not line["parity"]["ok"]:          # a run that fails the gate publishes no throughput
                line["value"] = None
                line["e2e"]["value"] = None
        print(json.dumps(line))
    if world > 1:
        # Tearing the process group down while CUDA graphs that captured its collectives are alive
        # can block for ever; every rank is done, so leave without the teardown.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_reference_arm(args):
    """The reference has no CPU implementation of these kernels and its Rust / Triton toolchain is absent, so the
    reference arm is the CPU restatement of the same layer chain (oracle/oracle_c.c, OpenMP on all host cores) on
    the benchmark's own extents: each step = the whole batch of 64 sequences at context 4096.  Rank 0 alone runs
    and prints; other ranks return at once."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    oc = load_oracle_c()
    oc.oc_num_threads.restype = ctypes.c_int
    cores = oc.oc_num_threads()
    sample = BATCH
    case = cpu_layer_case(np.random.default_rng(4), sample, CTX)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_layer_run(oc, case)
    ts = [cpu_layer_run(oc, case)[0] for _ in range(max(1, args.steps))]
    ms = 1e3 * sum(ts) / len(ts)
    value = sample / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage, int4 weights, f32 accumulate", "data": "synthetic",
        "config": {"workload": "C4: Llama-3-8B-shape W4A16 (GPTQ) decode layer chain, batch 64, ctx 4096",
                   "note": "CPU restatement of the reference kernels' arithmetic (oracle/oracle_c.c, OpenMP); "
                           "the reference has no CPU path and its Rust/Triton toolchain is absent"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} of {BATCH} sequences per step, ctx {CTX}, full layer chain"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-components", action="store_true", help="skip the per-kernel figures (configs 0-3)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()

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
    oc.oc_num_threads.restype = ctypes.c_int
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    oc.oc_set_num_threads(cores)        # all host cores, whatever OMP_NUM_THREADS the launcher exported
    return oc


def cpu_layer_case(rng, batch, ctx):
    """Seeded inputs of the layer chain at the benchmark's extents, `batch` sequences: nibbles uniform 0..15 around the
    symmetric zero-point 8 (stored 7, +1 in the GEMM), scales U(0.002, 0.02), activations N(0, 1) -- config 4."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle as o
    H, hq, hkv, d, I, G = 4096, 32, 8, 128, 14336, 128
    ml = ctx + 1

    def gptq(k, n):
        qw = rng.integers(0, 2 ** 32, (k // 8, n), dtype=np.uint32)
        return (qw.view(np.int32), rng.uniform(0.002, 0.02, (k // G, n)).astype(np.float16),
                np.full((k // G, n // 8), 0x77777777, dtype=np.int32))
    cos, sin = o.rope_tables(ml, d, 500000.0)
    case = dict(H=H, hq=hq, hkv=hkv, d=d, I=I, G=G, ml=ml, eps=1e-5, cos=cos, sin=sin,
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


def oracle_tools():
    """The checker (oracle/layer_check.py): CPU restatement of the chain + the comparison rules."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import layer_check
    return layer_check


def cpu_layer_time(oc, lc, case, reps):
    """Best-of-`reps` seconds of the reference-faithful CPU chain on `case` (every run appends the same K/V row)."""
    lc.oracle_layer(oc, case, want_stages=False)                       # warm-up: page in, thread pool
    return min(lc.oracle_layer(oc, case, want_stages=False)[2] for _ in range(reps))


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


def _median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


class ReferenceCubins:
    """The reference's own CUDA fixtures (tools/reference_cu/*.cu compiled unmodified into oracle/_ref/*.cubin by
    `make -C oracle ref`), launched through the driver API as the reference-owned comparator of three glue kernels.
    Comparator only: nothing of the product path goes through here."""

    def __init__(self, torch):
        self.torch, self.fns = torch, {}
        try:
            from cuda.bindings import driver
            self.driver = driver
        except Exception:
            self.driver = None

    def get(self, cubin, name):
        path = ROOT / "oracle" / "_ref" / cubin
        if self.driver is None or not path.exists():
            return None
        if (cubin, name) not in self.fns:
            d = self.driver
            err, mod = d.cuModuleLoadData(path.read_bytes())
            if err != d.CUresult.CUDA_SUCCESS:
                return None
            err, fn = d.cuModuleGetFunction(mod, name.encode())
            if err != d.CUresult.CUDA_SUCCESS:
                return None
            self.fns[(cubin, name)] = (mod, fn)
        fn = self.fns[(cubin, name)][1]

        def launch(grid, block, values, types):
            st = self.torch.cuda.current_stream().cuda_stream
            (e,) = self.driver.cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, 0, st, (tuple(values), tuple(types)), 0)
            if e != self.driver.CUresult.CUDA_SUCCESS:
                raise RuntimeError(f"reference fixture {name}: {e}")
        return launch


def component_metrics(pkg, torch, dev, gen):
    """The other parts of the compound metric: W4A16 GEMM TFLOP/s and GB/s (config 0 and all 16 cells of config 2), decode
    attention GB/s (config 1), fused MoE (config 3), and the glue kernels at the sizes the reference published.  Every
    figure is given two ways: `us` = CUDA-graph replay of back-to-back launches over rotating buffers (every launch
    streams from HBM; under programmatic dependent launch the set-up of a launch overlaps the tail of the one before,
    so this is a throughput figure), and `us_isolated` = median of single launches bracketed by events."""
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

    def isolated_time(fn, n=12):
        # one launch between two events, nothing in flight before it and nothing queued behind it; a spin kernel ahead
        # of the first event keeps the GPU busy while the host enqueues, so host-side launch preparation is not timed
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in evs:
            torch.cuda._sleep(400000)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
        return _median([a.elapsed_time(b) for a, b in evs])

    def ri(*s):
        return torch.randint(-2 ** 31, 2 ** 31 - 1, s, device=dev, dtype=torch.int32, generator=gen)

    out = {}
    G = 128
    cells = [("gptq", 16, 4096, 4096), ("gptq", 1, 4096, 4096)]
    cells += [("awq", m, k, n) for (k, n) in [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)] for m in (1, 16, 128, 1024)]
    for fmt, m, k, n in cells:
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
        iso = isolated_time(fn)
        byts = k * n // 2 + (k // G) * n * 2 + (k // G) * n // 2 + 2 * m * k + 2 * m * n
        out[f"{fmt}_gemm_m{m}_k{k}_n{n}"] = {
            "us": ms * 1e3, "us_isolated": iso * 1e3, "GB/s": byts / ms / 1e6, "TFLOP/s": 2 * m * k * n / ms / 1e9,
            "frac_hbm": byts / ms / 1e6 / hbm_peak, "frac_tensor": 2 * m * k * n / ms / 1e9 / tf_peak,
            "timing": "cold (rotating weight buffers)"}
        del qws
    # the same 16 cells with the weight pre-packed once into the K-packed layout (b200k_prepack_awq, an optional loader step)
    for (k, n) in [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)]:
        nbuf = max(2, int(400e6 // (k * n // 2)))
        sc = (torch.rand((k // G, n), device=dev, generator=gen) * 0.018 + 0.002).half()
        qz = ri(k // G, n // 8)
        qzp = torch.empty_like(qz)
        qwps = []
        for _ in range(nbuf):
            qw = ri(k, n // 8)
            qwp = torch.empty((k // 8, n), device=dev, dtype=torch.int32)
            P.b200k_prepack_awq(qw, qz, qwp, qzp, k, n, G)
            qwps.append(qwp)
            del qw
        for m in (1, 16, 128, 1024):
            a = torch.randn((m, k), device=dev, generator=gen, dtype=torch.float16)
            c = torch.empty((m, n), device=dev, dtype=torch.float16)
            i = [0]

            def fn():
                i[0] = (i[0] + 1) % nbuf
                P.awq_gemm_int4_prepacked_f16(a, qwps[i[0]], sc, qzp, c, m, n, k, G)
            ms = graph_time(fn, 2 * nbuf)
            byts = k * n // 2 + (k // G) * n * 2 + (k // G) * n // 2 + 2 * m * k + 2 * m * n
            out[f"awq_prepacked_gemm_m{m}_k{k}_n{n}"] = {
                "us": ms * 1e3, "GB/s": byts / ms / 1e6, "TFLOP/s": 2 * m * k * n / ms / 1e9,
                "frac_hbm": byts / ms / 1e6 / hbm_peak, "frac_tensor": 2 * m * k * n / ms / 1e9 / tf_peak,
                "timing": "cold (rotating weight buffers); weight rewritten once by b200k_prepack_awq, outside the timed region"}
        del qwps
    # config 1: decode attention, batch 32, lengths U[512, 8192]
    b, hq, hkv, d, ml = 32, 32, 8, 128, 8192
    q = torch.randn((b, hq, d), device=dev, generator=gen, dtype=torch.float16)
    kc = torch.randn((b, hkv, ml, d), device=dev, generator=gen, dtype=torch.float16)
    vc = torch.randn((b, hkv, ml, d), device=dev, generator=gen, dtype=torch.float16)
    lens = torch.randint(512, ml + 1, (b,), device=dev, dtype=torch.int32, generator=gen)
    ao = torch.empty_like(q)
    fn = lambda: P.batched_decode_attention_hm_f16(q, kc, vc, lens, ao, b, hq, hkv, d, ml, 1.0 / float(np.sqrt(d)))
    ms, iso = graph_time(fn, 4), isolated_time(fn)
    byts = 4096 * int(lens.sum()) + 2 * b * hq * d * 2
    out["decode_attention_c1"] = {"us": ms * 1e3, "us_isolated": iso * 1e3, "GB/s": byts / ms / 1e6,
                                  "frac_hbm": byts / ms / 1e6 / hbm_peak, "sum_len": int(lens.sum()),
                                  "timing": "inputs (537 MB) larger than L2"}
    del kc, vc
    # causal prefill (flash_attn_full_f16), Llama-3-8B head layout: one 2048-token and one 8192-token sequence.  The
    # contraction is counted causally (each query against the positions it sees: 4 * Hq * D * L (L + 1) / 2 flops)
    for L in (2048, 8192):
        pq = torch.randn((1, hq, L, d), device=dev, generator=gen, dtype=torch.float16)
        pk = torch.randn((1, hkv, L, d), device=dev, generator=gen, dtype=torch.float16)
        pv = torch.randn((1, hkv, L, d), device=dev, generator=gen, dtype=torch.float16)
        po = torch.empty_like(pq)
        fn = lambda: P.flash_attn_full_f16(pq, pk, pv, po, 1, hq, hkv, L, L, d, 0, 1.0 / float(np.sqrt(d)))
        ms, iso = graph_time(fn, 4), isolated_time(fn, 8)
        flops = 4.0 * hq * d * L * (L + 1) / 2
        out[f"prefill_attention_l{L}"] = {"us": ms * 1e3, "us_isolated": iso * 1e3, "TFLOP/s": flops / ms / 1e9,
                                          "frac_tensor": flops / ms / 1e9 / tf_peak,
                                          "timing": "tensor-bound: K/V (%d MB) are re-read from L2 by design" % (4 * hkv * L * d // 2 ** 20)}
        del pq, pk, pv, po
    # unified prefill + decode over a paged fp32 pool (unified_attention_f32): 4 sequences prefilling 256 tokens each and
    # 28 decoding one token at context 2048, blocks of 16 positions; a CUDA-core kernel (fp32 arithmetic throughout)
    useq = [(256, 256)] * 4 + [(1, 2048)] * 28
    ubs = 16
    bps = max(-(-sl // ubs) for _, sl in useq)
    nblk = len(useq) * bps
    uq = torch.randn((sum(ql for ql, _ in useq), hq, d), device=dev, generator=gen)
    ukp = torch.randn((nblk, ubs, hkv, d), device=dev, generator=gen)
    uvp = torch.randn((nblk, ubs, hkv, d), device=dev, generator=gen)
    utab = torch.randperm(nblk, device=dev, generator=gen).to(torch.int32).reshape(len(useq), bps).contiguous()
    usl = torch.tensor([sl for _, sl in useq], device=dev, dtype=torch.int32)
    uqs = torch.tensor(np.concatenate([[0], np.cumsum([ql for ql, _ in useq])]), device=dev, dtype=torch.int32)
    uo = torch.empty_like(uq)
    fn = lambda: P.unified_attention_f32(uq, ukp, uvp, uo, utab, usl, uqs, hq, hkv, d, ubs, bps, 1.0 / float(np.sqrt(d)), len(useq))
    ms, iso = graph_time(fn, 2), isolated_time(fn, 6)
    kv_bytes = sum(sl for _, sl in useq) * hkv * d * 4 * 2
    uflops = sum(4.0 * hq * d * (ql * (sl - ql) + ql * (ql + 1) / 2) for ql, sl in useq)
    out["unified_attention_f32_mixed"] = {"us": ms * 1e3, "us_isolated": iso * 1e3, "GB/s_kv_once": kv_bytes / ms / 1e6,
                                          "TFLOP/s": uflops / ms / 1e9, "batch": "4 x 256-token prefill + 28 x decode at ctx 2048",
                                          "timing": "KV pool 0.5 GB, larger than L2"}
    del ukp, uvp
    # config 3: fused MoE, Mixtral-8x7B shape
    T, E, kk, H, I = 512, 8, 2, 4096, 14336
    w13q, w2q = ri(E, H // 8, 2 * I), ri(E, I // 8, H)
    w13s = (torch.rand((E, H // G, 2 * I), device=dev, generator=gen) * 0.018 + 0.002).half()
    w2s = (torch.rand((E, I // G, H), device=dev, generator=gen) * 0.018 + 0.002).half()
    x = torch.randn((T, H), device=dev, generator=gen, dtype=torch.float16)
    lg = torch.randn((T, E), device=dev, generator=gen)
    mo = torch.empty((T, H), dtype=torch.float16, device=dev)
    fn = lambda: P.fused_moe_gptq_f16(x, lg, w13q, w13s, None, w2q, w2s, None, mo, T, H, E, kk, I, G, None, 0)
    ms, iso = graph_time(fn, 2), isolated_time(fn, 6)
    flops = T * kk * (2 * H * 2 * I + 2 * I * H)
    out["fused_moe_c3"] = {"us": ms * 1e3, "us_isolated": iso * 1e3, "TFLOP/s": flops / ms / 1e9,
                           "frac_tensor": flops / ms / 1e9 / tf_peak, "weight_GB/s": 726663168 / ms / 1e6,
                           "timing": "weights (727 MB) larger than L2"}
    del w13q, w2q, w13s, w2s
    # glue at the sizes the reference published (BENCH_RESULTS.md of the reference: residual_add_f32 and
    # fused_silu_mul_f32 at N = 33,554,432, rms_norm_f32 at 32768 x 1024), f32 and f16, with the reference's own CUDA
    # fixtures timed on the same buffers.  Bytes = reads + writes, the weight vector ignored, as the reference counts.
    ref = ReferenceCubins(torch)
    import ctypes as C
    n_el, rows, row = 33554432, 32768, 1024
    for tname, tdt, esz in (("f32", torch.float32, 4), ("f16", torch.float16, 2)):
        nb = 2 if esz == 4 else 3                                    # rotate so that f16 sets (> 126 MB in all) miss L2
        a_ = [torch.randn(n_el, device=dev, generator=gen, dtype=tdt) for _ in range(nb)]
        b_ = [torch.randn(n_el, device=dev, generator=gen, dtype=tdt) for _ in range(nb)]
        o_ = torch.empty(n_el, device=dev, dtype=tdt)
        w_ = (torch.rand(row, device=dev, generator=gen) + 0.5).to(tdt)
        i = [0]

        def rot():
            i[0] = (i[0] + 1) % nb
            return i[0]
        jobs = {
            f"residual_add_{tname}": (3 * n_el * esz, lambda: getattr(P, f"residual_add_{tname}")(a_[rot()], b_[i[0]], o_, n_el),
                                      ("residual_add.cubin", lambda L: L((n_el + 255) // 256, 256, (a_[rot()].data_ptr(), b_[i[0]].data_ptr(), o_.data_ptr(), n_el), (C.c_void_p, C.c_void_p, C.c_void_p, C.c_int)))),
            f"fused_silu_mul_{tname}": (3 * n_el * esz, lambda: getattr(P, f"fused_silu_mul_{tname}")(a_[rot()], b_[i[0]], o_, n_el),
                                        ("fused_silu_mul.cubin", lambda L: L((n_el + 255) // 256, 256, (a_[rot()].data_ptr(), b_[i[0]].data_ptr(), o_.data_ptr(), n_el), (C.c_void_p, C.c_void_p, C.c_void_p, C.c_int)))),
            f"rms_norm_{tname}": (2 * rows * row * esz, lambda: getattr(P, f"rms_norm_{tname}")(a_[rot()], w_, o_, row, 1.0 / row, 1e-6, rows),
                                  ("rms_norm.cubin", lambda L: L(rows, row, (a_[rot()].data_ptr(), w_.data_ptr(), o_.data_ptr(), row, 1e-6), (C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_float)))),
        }
        for name, (byts, fn, (cubin, ref_call)) in jobs.items():
            ms, iso = graph_time(fn, 2 * nb), isolated_time(fn, 8)
            ent = {"us": ms * 1e3, "us_isolated": iso * 1e3, "GB/s": byts / ms / 1e6, "frac_hbm": byts / ms / 1e6 / hbm_peak,
                   "bytes": byts, "timing": "inputs larger than L2" if esz == 4 else "rotating inputs larger than L2"}
            L = ref.get(cubin, name)
            if L is not None:
                rms_ = graph_time(lambda: ref_call(L), 2 * nb)
                ent["reference_cu"] = {"us": rms_ * 1e3, "GB/s": byts / rms_ / 1e6, "frac_hbm": byts / rms_ / 1e6 / hbm_peak,
                                       "what": f"the reference's tools/reference_cu kernel {name}, compiled unmodified for sm_100a, same buffers"}
            out[name] = ent
        del a_, b_, o_
    return out


def tp_component_metrics(pkg, torch, dist, dev, rank, world, gen, shape, comm):
    """N > 1: what one rank runs, kernel by kernel (CUDA-graph replay over rotating weights, max over ranks): the four
    GEMMs of the layer at their rank-local extents, the all-reduce alone, and the expert-parallel fused MoE of config 3
    (E / N experts per rank, replicated tokens, one all-reduce of the partial outputs)."""
    P = pkg.prelude
    hbm_peak, tf_peak, _ = peaks()
    ls = shape.local(world)
    H, d, G = shape.hidden, shape.head_dim, shape.group_size

    def ri(*s):
        return torch.randint(-2 ** 31, 2 ** 31 - 1, s, device=dev, dtype=torch.int32, generator=gen)

    def replay_ms(fn, calls, reps=5):
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            for _ in range(calls):
                fn()
        best = 1e30
        for _ in range(reps + 1):
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); gr.replay(); b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b) / calls)
        t = torch.tensor([best], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {}
    cells = {"qkv": (H, (ls.num_q_heads + 2 * ls.num_kv_heads) * d), "o": (ls.num_q_heads * d, H),
             "gate_up": (H, 2 * ls.intermediate), "down": (ls.intermediate, H)}
    for name, (k, n) in cells.items():
        nbuf = max(2, int(300e6 // (k * n // 2)))
        qws = [ri(k // 8, n) for _ in range(nbuf)]
        sc = (torch.rand((k // G, n), device=dev, generator=gen) * 0.018 + 0.002).half()
        qz = torch.full((k // G, n // 8), 0x77777777, device=dev, dtype=torch.int32)
        a = torch.randn((BATCH, k), device=dev, generator=gen, dtype=torch.float16)
        c = torch.empty((BATCH, n), device=dev, dtype=torch.float16)
        i = [0]

        def fn():
            i[0] = (i[0] + 1) % nbuf
            P.gptq_gemm(a, qws[i[0]], sc, qz, G, out=c)
        ms = replay_ms(fn, 2 * nbuf)
        byts = k * n // 2 + (k // G) * n * 2 + (k // G) * n // 2 + 2 * BATCH * k + 2 * BATCH * n
        out[f"gemm_{name}_m{BATCH}_k{k}_n{n}"] = {"us": ms * 1e3, "GB/s": byts / ms / 1e6, "frac_hbm": byts / ms / 1e6 / hbm_peak}
        del qws
    # config 2 under tensor parallelism: the AWQ GEMM of every (K, N) cell at its rank-local extents (qkv and gate_up
    # column-parallel: N / world; o and down row-parallel: K / world, their partial sums completed by the all-reduce
    # timed below), M = 1, 16, 128, 1024
    for (k, n, split) in [(4096, 6144, "n"), (4096, 4096, "k"), (4096, 28672, "n"), (14336, 4096, "k")]:
        kl, nl = (k // world, n) if split == "k" else (k, n // world)
        if kl % G or nl % 64:
            continue
        nbuf = max(2, int(200e6 // (kl * nl // 2)))
        qws = [ri(kl, nl // 8) for _ in range(nbuf)]
        sc = (torch.rand((kl // G, nl), device=dev, generator=gen) * 0.018 + 0.002).half()
        qz = ri(kl // G, nl // 8)
        for m in (1, 16, 128, 1024):
            a = torch.randn((m, kl), device=dev, generator=gen, dtype=torch.float16)
            c = torch.empty((m, nl), device=dev, dtype=torch.float16)
            i = [0]

            def fn():
                i[0] = (i[0] + 1) % nbuf
                P.awq_gemm(a, qws[i[0]], sc, qz, G, out=c)
            ms = replay_ms(fn, 2 * nbuf, reps=3)
            byts = kl * nl // 2 + (kl // G) * nl * 2 + (kl // G) * nl // 2 + 2 * m * kl + 2 * m * nl
            out[f"awq_gemm_tp_m{m}_k{kl}_n{nl}"] = {"us": ms * 1e3, "GB/s": byts / ms / 1e6, "frac_hbm": byts / ms / 1e6 / hbm_peak,
                                                   "TFLOP/s": 2 * m * kl * nl / ms / 1e9, "frac_tensor": 2 * m * kl * nl / ms / 1e9 / tf_peak,
                                                   "full_cell": f"K {k}, N {n}, {'row' if split == 'k' else 'column'}-parallel"}
        del qws
    # the exchange alone: one all-reduce of the layer's [64, H] fp16 partial sums, slots alternating
    x = torch.randn((BATCH, H), device=dev, generator=gen, dtype=torch.float16)
    y = torch.empty_like(x)
    sl = [0]

    def ar():
        sl[0] ^= 1
        comm.all_reduce(sl[0], y, BATCH * H, input=x)
    ms = replay_ms(ar, 8)
    out["all_reduce_64x4096_f16"] = {"us": ms * 1e3, "bytes_in_per_rank": (world - 1) * BATCH * H * 2}
    # config 3 expert-parallel
    T, E, kk, Hm, I = 512, 8, 2, 4096, 14336
    if E % world == 0:
        per = E // world
        big = pkg.Comm.from_process_group(T * Hm * 2)
        mgen = torch.Generator(device=dev).manual_seed(99)                  # same tokens and logits on every rank
        xm = torch.randn((T, Hm), device=dev, generator=mgen, dtype=torch.float16)
        lg = torch.randn((T, E), device=dev, generator=mgen)
        w13q, w2q = ri(per, Hm // 8, 2 * I), ri(per, I // 8, Hm)
        w13s = (torch.rand((per, Hm // G, 2 * I), device=dev, generator=gen) * 0.018 + 0.002).half()
        w2s = (torch.rand((per, I // G, Hm), device=dev, generator=gen) * 0.018 + 0.002).half()
        part = torch.empty((T, Hm), dtype=torch.float16, device=dev)
        full = torch.empty_like(part)
        sl2 = [0]

        def moe():
            sl2[0] ^= 1
            P.fused_moe_gptq_ep_f16(xm, lg, w13q, w13s, None, w2q, w2s, None, part, T, Hm, E, rank * per, per, kk, I, G, None, 0)
            big.all_reduce(sl2[0], full, T * Hm, input=part)
        ms = replay_ms(moe, 2)
        flops = T * kk * (2 * Hm * 2 * I + 2 * I * Hm)
        out["fused_moe_c3_expert_parallel"] = {"us": ms * 1e3, "TFLOP/s_all_ranks": flops / ms / 1e9,
                                               "experts_per_rank": per, "all_reduce_bytes": T * Hm * 2,
                                               "comm_status": big.status()}
        torch.cuda.synchronize()
        dist.barrier()
        big.close()
        # the same MoE by token exchange: every rank holds T / N of the tokens and E / N experts
        if T % world == 0:
            L = pkg.lib()
            t_loc = T // world
            xc = pkg.Comm.from_process_group(L.call("fused_moe_a2a_slot_bytes", t_loc, Hm, kk, world))
            x_loc = xm[rank * t_loc:(rank + 1) * t_loc].contiguous()
            lg_loc = lg[rank * t_loc:(rank + 1) * t_loc].contiguous()
            o_loc = torch.empty((t_loc, Hm), dtype=torch.float16, device=dev)

            def moe_x():
                L.call("fused_moe_gptq_a2a_f16", xc.handle, x_loc, lg_loc, w13q, w13s, None, w2q, w2s, None, o_loc, t_loc, Hm, E, kk, I, G,
                       7, None, 0, torch.cuda.current_stream().cuda_stream)
            ms = replay_ms(moe_x, 2)
            # the two forms must agree on this rank's tokens (same pairs, same experts, same weights): checked against the
            # all-reduce form computed above
            # all-reduce form computed above.  That form rounds every rank's partial sum to fp16 before adding them, and the
            # partial sums cancel, so the yardstick is the magnitude of the outputs, not of each element
            want = full[rank * t_loc:(rank + 1) * t_loc].float()
            diff, top = float((o_loc.float() - want).abs().max()), float(want.abs().max())
            out["fused_moe_c3_token_exchange"] = {"us": ms * 1e3, "TFLOP/s_all_ranks": flops / ms / 1e9, "experts_per_rank": per,
                                                  "rows_out_per_rank": t_loc * kk, "max_abs_diff_vs_all_reduce_form": diff,
                                                  "max_abs_output": top, "agrees_with_all_reduce_form": bool(diff <= 5e-3 * top),
                                                  "comm_status": xc.status()}
            torch.cuda.synchronize()
            dist.barrier()
            xc.close()
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

    half = d // 2
    inv_freq = 1.0 / (shape.rope_theta ** (torch.arange(half, dtype=torch.float64) * 2.0 / d))
    ang = torch.arange(ml, dtype=torch.float64)[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)

    # N > 1: the library's own peer-to-peer all-reduce inside its captured layer chain;
    # BENCH_TP_COMM=nccl runs the staged chain with NCCL all-reduces between the stages instead
    own_comm = world > 1 and os.environ.get("BENCH_TP_COMM", "p2p") == "p2p"
    comm = pkg.Comm.from_process_group(BATCH * H * 2) if own_comm else None
    layers = []
    gate_case = None          # rank 0: host copy of set 0's FULL (unsharded) tensors for the parity gate
    for si in range(N_SETS):
        full = {"qkv": gptq(H, (shape.num_q_heads + 2 * shape.num_kv_heads) * d), "o": gptq(shape.num_q_heads * d, H),
                "gate_up": gptq(H, 2 * shape.intermediate), "down": gptq(shape.intermediate, H)}
        w = pkg.shard_layer_weights(full, shape, rank, world) if world > 1 else full
        ln1 = (torch.rand(H, device=dev, generator=gen) + 0.5).half()
        ln2 = (torch.rand(H, device=dev, generator=gen) + 0.5).half()
        # every rank draws the same numbers, so the full cache of the unsharded layer is this tensor repeated over the
        # rank axis: kv head h of the full layer = local head h % (heads per rank)
        kc = torch.randn((BATCH, ls.num_kv_heads, ml, d), device=dev, generator=gen, dtype=torch.float16)
        vc = torch.randn((BATCH, ls.num_kv_heads, ml, d), device=dev, generator=gen, dtype=torch.float16)
        if si == 0 and rank == 0 and not args.no_cpu:
            hn = lambda x: np.ascontiguousarray(x.cpu().numpy())
            gate_case = dict(H=H, hq=shape.num_q_heads, hkv=shape.num_kv_heads, d=d, I=shape.intermediate, G=G, ml=ml, eps=shape.rms_eps,
                             cos=hn(cos), sin=hn(sin), ln1=hn(ln1), ln2=hn(ln2),
                             kc=np.ascontiguousarray(np.tile(hn(kc), (1, world, 1, 1))), vc=np.ascontiguousarray(np.tile(hn(vc), (1, world, 1, 1))),
                             **{k_: tuple(hn(x) for x in full[k_]) for k_ in full})
        del full
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
        sampler.start()              # samples every few ms from warm-up to the last timed kernel
    for i in range(max(args.warmup, 3) + N_SETS):    # graph capture happens on first use of each set
        step(i)
    barrier()
    note("warm-up done")

    # ---- the tensors that are timed are the tensors that are gated: set 0's output, kept for the parity gate ----
    step(0)
    barrier()
    gate_out = out.clone()
    same_bits = True
    if world > 1:                    # every rank must hold the same bits (the all-reduce sums in rank order everywhere)
        outs = [torch.empty_like(gate_out) for _ in range(world)]
        dist.all_gather(outs, gate_out)
        same_bits = all(bool(torch.equal(o_, outs[0])) for o_ in outs)

    # ---- timed region: `loops` loops of exactly `steps` steps; the line carries the median loop ----
    loop_ms = []
    for _ in range(max(1, args.loops)):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for i in range(args.steps):
            step(i)
        ev1.record()
        barrier()
        ms_total = ev0.elapsed_time(ev1)
        if world > 1:
            tt = torch.tensor([ms_total], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms_total = float(tt.item())
        loop_ms.append(ms_total / args.steps)
    ms_step = _median(loop_ms)
    note(f"timed region done: {ms_step:.3f} ms/step")

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

    for i in range(3 + N_SETS):
        e2e_step(i)
    e2e_loops = []
    for _ in range(max(1, args.loops)):
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        if world > 1:
            tt = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e_ms = float(tt.item())
        e2e_loops.append(e2e_ms)
    e2e_ms = _median(e2e_loops)
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

    components = component_metrics(pkg, torch, dev, gen) if world == 1 and not args.no_components else None
    if world > 1 and own_comm and not args.no_components:
        components = tp_component_metrics(pkg, torch, dist, dev, rank, world, gen, shape, comm)
        components["decode_attention_rank_local"] = {"us": attn_ms * 1e3, "kv_heads": ls.num_kv_heads,
                                                     "GB/s": (2 * BATCH * ls.num_kv_heads * ml * d * 2) / attn_ms / 1e6}
        note("tensor-parallel components timed")

    # device-side failure channels: any bounded wait that gave up, any clamped index, on any rank, voids the number
    status = ctypes.c_int(-1)
    pkg.lib().call("b200k_device_status", ctypes.addressof(status), stream.cuda_stream)
    comm_status = comm.status() if comm is not None else 0
    worst = torch.tensor([status.value, comm_status], device=dev, dtype=torch.int32)
    if world > 1:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    dev_status, comm_status = int(worst[0].item()), int(worst[1].item())

    if rank == 0:
        hbm_peak, tf_peak, peak_kind = peaks()
        attn_bytes = 2 * BATCH * ls.num_kv_heads * ml * d * 2 + 2 * BATCH * ls.num_q_heads * d * 2
        achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": BATCH / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "ms_per_step_min": min(loop_ms), "ms_per_step_loops": loop_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage, int4 weights, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": "C4: Llama-3-8B-shape W4A16 (GPTQ) decode layer chain, batch 64, ctx 4096",
                       "parallelism": f"tp{world}" if world > 1 else "single GPU",
                       "l2": f"inputs larger than L2: {N_SETS} weight+KV sets rotated, "
                             f"{(2 * BATCH * ls.num_kv_heads * ml * d * 2) / 1e9:.2f} GB of KV per step",
                       "all_reduce": None if world == 1 else ("own one-shot kernel over NVLink peer memory" if own_comm else "NCCL"),
                       "graph": bool(world == 1 or own_comm or tp_graphs), "device_status": dev_status,
                       "comm_status": comm_status if comm is not None else None,
                       "timing": f"{len(loop_ms)} loops of {args.steps} steps, CUDA events, max over ranks per loop; value = median loop"},
            "e2e": {"value": BATCH / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms, "ms_per_step_min": min(e2e_loops),
                    "h2d_bytes_per_step": BATCH * H * 2 + BATCH * 4, "d2h_bytes_per_step": BATCH * H * 2},
            "gpu_launches": (layers[0].launches_per_forward) * args.steps,
            "roofline": {"kernel": "attn_split_f16_kernel", "bound": "hbm", "achieved": achieved, "peak": hbm_peak,
                         "unit": "GB/s", "frac": achieved / hbm_peak, "peak_kind": peak_kind,
                         # dram bytes per launch: from an ncu capture of a smaller launch of this kernel (measured
                         # 1.033 x algorithmic bytes), scaled to this launch by the bytes processed
                         "traffic": int(attn_bytes * 1.033),
                         "algorithmic_bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms},
            "clocks": clocks,
        }
        if components is not None:
            line["components"] = components
        ok = dev_status == 0 and comm_status == 0 and same_bits
        if gate_case is not None:
            # The parity gate runs on the tensors that were timed: set 0's weights, caches, hidden state and positions,
            # and the output the timed chain produced from them (at N > 1: the tensor-parallel output, identical bits on
            # every rank, against the CPU restatement of the UNSHARDED layer).
            lc = oracle_tools()
            oc = load_oracle_c()
            gate_case["hidden"] = np.ascontiguousarray(hidden.cpu().numpy())
            gate_case["pos"] = np.ascontiguousarray(positions.cpu().numpy())
            # (the drift yardstick runs first: both restatements append a K/V row, and the caches must end up holding the
            # reference-faithful one)
            ref_alt = lc.oracle_layer(oc, gate_case, faithful=0, want_stages=False)[0]     # fp32 weight products
            ref, st, _ = lc.oracle_layer(oc, gate_case)
            rep = lc.check_layer(pkg, torch, dev, gate_case, ref, st, got_out=gate_out.float().cpu().numpy(), ref_alt=ref_alt)
            rep["what"] = ("the timed tensors (weight + KV set 0, batch 64, ctx 4096) through the C ABI vs the CPU restatement "
                           "of the unsharded layer" + (f"; tensor-parallel output of {world} ranks, bit-identical on all: {same_bits}" if world > 1 else ""))
            rep["ranks_bit_identical"] = same_bits
            line["parity"] = rep
            ok = ok and rep["ok"]
            if world == 1:
                best = cpu_layer_time(oc, lc, gate_case, 2)
                line["cpu_baseline"] = {"value": BATCH / best, "unit": "tok/s", "cores": oc.oc_num_threads(), "kind": "port",
                                        "sample": f"{BATCH} of {BATCH} sequences, ctx {CTX}, full layer chain on the timed tensors, best of 2"}
        else:
            line["parity"] = {"ok": None, "what": "skipped (--no-cpu)", "ranks_bit_identical": same_bits}
        if not ok:                   # a run that fails the gate, or saw a device-side give-up, publishes no throughput
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
    lc = oracle_tools()
    cores = oc.oc_num_threads()
    sample = BATCH
    case = cpu_layer_case(np.random.default_rng(4), sample, CTX)
    for _ in range(max(1, min(args.warmup, 2))):
        lc.oracle_layer(oc, case, want_stages=False)
    ts = [lc.oracle_layer(oc, case, want_stages=False)[2] for _ in range(max(1, args.steps))]
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
    ap.add_argument("--loops", type=int, default=7, help="timed loops of --steps steps each; the line carries the median loop")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU legs (parity gate and CPU baseline)")
    ap.add_argument("--no-components", action="store_true", help="skip the per-kernel figures (configs 0-3, glue)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()

"""Peer-to-peer all-reduce and the tensor-parallel layer chain on real GPUs.

One process per GPU (children of the test), rendezvous on 127.0.0.1.  The two-rank cases
need two visible GPUs and are skipped otherwise; the one-rank case runs everywhere.
The all-reduce must be bit-exact: fp32 sum of the ranks' fp16 values in rank order, one rounding."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _expected(parts):
    acc = np.zeros(parts[0].shape, dtype=np.float32)
    for p in parts:                       # rank order, fp32 accumulate, one rounding to fp16
        acc = acc + p.astype(np.float32)
    return acc.astype(np.float16)


def test_allreduce_single_rank(pkg):
    dev = "cuda:0"
    n = 4096 + 8
    comm = pkg.Comm(0, 1, n * 2, exchange=None)
    x = torch.randn(n, device=dev, dtype=torch.float16)
    out = torch.zeros_like(x)
    for slot in (0, 1, 0):
        comm.all_reduce(slot, out, n, input=x)
        torch.cuda.synchronize()
        assert torch.equal(out, x)
    assert comm.status() == 0
    # the fused forms give the bits of the plain all-reduce followed by the separate kernel
    L, st = pkg.lib(), torch.cuda.current_stream().cuda_stream
    rows, h = 4, 1024
    part = torch.randn(rows * h, device=dev, dtype=torch.float16)
    res = torch.randn(rows * h, device=dev, dtype=torch.float16)
    w = (torch.rand(h, device=dev) + 0.5).half()
    red = torch.empty_like(part)
    comm.all_reduce(1, red, rows * h, input=part)
    want = torch.empty_like(part)
    pkg.prelude.residual_add_f16(res, red, want, rows * h)
    got = torch.empty_like(part)
    L.call("b200k_comm_allreduce_add_f16", comm.handle, 0, part, res, got, rows * h, st)
    assert torch.equal(got, want)
    y0, r0, y1, r1 = (torch.empty_like(part) for _ in range(4))
    pkg.prelude.fused_add_rms_norm_f16(red, res, w, y0, r0, h, 1.0 / h, 1e-5, rows)
    L.call("b200k_comm_allreduce_add_rms_norm_f16", comm.handle, 1, part, res, w, y1, r1, h, 1.0 / h, 1e-5, rows, st)
    torch.cuda.synchronize()
    assert torch.equal(r1, r0) and torch.equal(y1, y0)
    assert comm.status() == 0
    with pytest.raises(pkg.B200KError):
        comm.all_reduce(0, torch.zeros(n + 512, device=dev, dtype=torch.float16), n + 512, input=None)   # larger than a slot
    with pytest.raises(pkg.B200KError):
        comm.all_reduce(2, out, n, input=x)              # no such slot
    comm.close()


def _rank_main(rank, world, port, q):
    try:
        sys.path.insert(0, str(ROOT))
        sys.path.insert(0, str(ROOT / "oracle"))
        sys.path.insert(0, str(ROOT / "tests"))
        import importlib
        import torch.distributed as dist
        import oracle as o
        from test_layer_gpu import make_layer
        pkg = importlib.import_module("triton-rs_b200")
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)

        def t(a):
            return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

        # ---- all-reduce alone: several sizes, both slots, staged input and in-place slot ----
        n_max = 64 * 4096
        comm = pkg.Comm.from_process_group(n_max * 2)
        rng = np.random.default_rng(7)
        for it, n in enumerate([8, 4096, 64 * 4096, 1000 * 8, 64 * 4096]):
            parts = [rng.standard_normal(n).astype(np.float16) for _ in range(world)]   # same stream of numbers on every rank
            out = torch.zeros(n, device=dev, dtype=torch.float16)
            dist.barrier()                # the kernel waits for its peers for about a second only
            comm.all_reduce(it & 1, out, n, input=t(parts[rank]))
            torch.cuda.synchronize()
            got = out.cpu().numpy()
            assert np.array_equal(got.view(np.uint16), _expected(parts).view(np.uint16)), f"all-reduce n={n}"
        assert comm.status() == 0

        # ---- tensor-parallel layer (own all-reduce inside the captured chain) against the oracle ----
        rng = np.random.default_rng(17)
        B, H, hq, hkv, d, I, G, ml = 3, 256, 4, 2, 128, 512, 128, 40
        p = make_layer(o, rng, H, hq, hkv, d, I, G, ml)
        shape = pkg.LayerShape(H, hq, hkv, d, I, G, 1e-5)
        ls = shape.local(world)
        full = {k: tuple(None if x is None else t(x) for x in p[k]) for k in ("qkv", "o", "gate_up", "down")}
        w = pkg.shard_layer_weights(full, shape, rank, world)
        kc = rng.standard_normal((B, hkv, ml, d)).astype(np.float16)
        vc = rng.standard_normal((B, hkv, ml, d)).astype(np.float16)
        per = hkv // world
        layer = pkg.DecodeLayer(ls, w, t(p["ln1"]), t(p["ln2"]), t(p["cos"]), t(p["sin"]), max_batch=4, max_len=ml,
                                use_graph=True, k_cache=t(kc[:, rank * per:(rank + 1) * per]),
                                v_cache=t(vc[:, rank * per:(rank + 1) * per]))
        layer.set_comm(comm)
        assert layer.launches_per_forward == 10      # the two all-reduces are fused with the steps that consume them
        for step, pos in enumerate([[5, 0, 38], [6, 1, 39], [7, 2, 3]]):     # later steps replay the captured graph
            pos = np.array(pos, dtype=np.int32)
            hidden = rng.standard_normal((B, H)).astype(np.float16)
            stg = {}
            ref = o.decode_layer(hidden, p, kc, vc, pos, stages=stg)
            dist.barrier()
            out = layer.forward(t(hidden), t(pos))
            torch.cuda.synchronize()
            got = out.float().cpu().numpy()
            from conftest import assert_close_sum, assert_close_terms
            assert_close_sum(got, ref, (stg["h1"], stg["down"]), what=f"tp layer step {step}")   # sum of two fp16 tensors
            gathered = [None] * world
            dist.all_gather_object(gathered, got.tobytes())
            assert all(g == gathered[0] for g in gathered), "ranks disagree"
        assert comm.status() == 0

        # ---- expert-parallel MoE: every rank computes the share of its experts, one all-reduce adds them ----
        rng = np.random.default_rng(29)
        T, E, k, H, I, G = 33, 8, 2, 256, 384, 128
        x = rng.standard_normal((T, H)).astype(np.float16)
        logits = rng.standard_normal((T, E)).astype(np.float32)
        w13q = np.stack([o.pack_gptq_qweight(rng.integers(1, 16, (H, 2 * I), dtype=np.int32)) for _ in range(E)])
        w13s = rng.uniform(0.002, 0.02, (E, H // G, 2 * I)).astype(np.float16)
        w2q = np.stack([o.pack_gptq_qweight(rng.integers(1, 16, (I, H), dtype=np.int32)) for _ in range(E)])
        w2s = rng.uniform(0.002, 0.02, (E, I // G, H)).astype(np.float16)
        ref, mag = o.fused_moe_gptq(x, logits, w13q, w13s, w2q, w2s, k, G, faithful=True, with_mag=True)
        per = E // world
        lo, hi = rank * per, (rank + 1) * per
        share = torch.empty((T, H), dtype=torch.float16, device=dev)
        full = torch.empty_like(share)
        st = torch.cuda.current_stream().cuda_stream
        pkg.prelude.fused_moe_gptq_ep_f16(t(x), t(logits), t(w13q[lo:hi]), t(w13s[lo:hi]), None, t(w2q[lo:hi]), t(w2s[lo:hi]),
                                          None, share, T, H, E, lo, per, k, I, G, None, 0, st)
        dist.barrier()
        comm.all_reduce(0, full, T * H, input=share)
        comm.all_reduce(1, share, T * H, input=full)       # keeps the slots alternating for whoever comes next
        torch.cuda.synchronize()
        got = full.float().cpu().numpy()
        assert_close_terms(got, ref, mag, k, what="ep moe")
        assert comm.status() == 0

        # ---- expert-parallel MoE by token exchange: every rank holds a slice of the tokens and of the experts ----
        T_loc = 20
        T = world * T_loc
        x = rng.standard_normal((T, H)).astype(np.float16)
        logits = rng.standard_normal((T, E)).astype(np.float32)
        ref, mag = o.fused_moe_gptq(x, logits, w13q, w13s, w2q, w2s, k, G, faithful=True, with_mag=True)
        L = pkg.lib()
        big = pkg.Comm.from_process_group(L.call("fused_moe_a2a_slot_bytes", T_loc, H, k, world))
        mine = torch.empty((T_loc, H), dtype=torch.float16, device=dev)
        wl = (t(w13q[lo:hi]), t(w13s[lo:hi]), t(w2q[lo:hi]), t(w2s[lo:hi]))
        for rnd in range(3):                     # later rounds reuse every region of the exchange buffers
            dist.barrier()
            L.call("fused_moe_gptq_a2a_f16", big.handle, t(x[rank * T_loc:(rank + 1) * T_loc]), t(logits[rank * T_loc:(rank + 1) * T_loc]),
                   wl[0], wl[1], None, wl[2], wl[3], None, mine, T_loc, H, E, k, I, G, 7, None, 0, st)
            torch.cuda.synchronize()
            assert big.status() == 0
            got = mine.float().cpu().numpy()
            sl = slice(rank * T_loc, (rank + 1) * T_loc)
            assert_close_terms(got, ref[sl], mag[sl], k, what=f"token-exchange moe, round {rnd}")
        dist.barrier()
        big.close()
        dist.barrier()
        layer.close()
        comm.close()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))


@pytest.mark.timeout(300)
def test_two_ranks_allreduce_and_tp_layer():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, 29731
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            r, msg = q.get(timeout=240)
            results[r] = msg
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert all(v == "ok" for v in results.values()), results


# ---- the two-shot form (large tensors on three or more ranks), forced on smaller groups through its override ----
_ONE_RANK_TWOSHOT = r"""
import importlib, sys
import torch
sys.path.insert(0, sys.argv[1])
pkg = importlib.import_module("triton-rs_b200")
dev = "cuda:0"
n = 64 * 4096 + 8
comm = pkg.Comm(0, 1, n * 2, exchange=None)
x = torch.randn(n, device=dev, dtype=torch.float16)
res = torch.randn(n, device=dev, dtype=torch.float16)
out = torch.zeros_like(x)
for slot in (0, 1, 0, 1):
    comm.all_reduce(slot, out, n, input=x)
    torch.cuda.synchronize()
    assert torch.equal(out, x), slot
got = torch.empty_like(x)
pkg.lib().call("b200k_comm_allreduce_add_f16", comm.handle, 0, x, res, got, n, torch.cuda.current_stream().cuda_stream)
torch.cuda.synchronize()
assert torch.equal(got, res + x)
assert comm.status() == 0
comm.close()
print("ok")
"""


def test_twoshot_allreduce_single_rank():
    import subprocess
    env = dict(os.environ, B200K_COMM_TWOSHOT="1")
    r = subprocess.run([sys.executable, "-c", _ONE_RANK_TWOSHOT, str(ROOT)], env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr


def _rank_twoshot(rank, world, port, q):
    try:
        sys.path.insert(0, str(ROOT))
        import importlib
        import torch.distributed as dist
        pkg = importlib.import_module("triton-rs_b200")
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        n_max = 512 * 4096
        comm = pkg.Comm.from_process_group(n_max * 2)
        rng = np.random.default_rng(11)
        for it, n in enumerate([8, 64 * 4096, 1000 * 8, 512 * 4096, 512 * 4096, 4096 + 8]):
            parts = [rng.standard_normal(n).astype(np.float16) for _ in range(world)]   # same stream of numbers on every rank
            out = torch.zeros(n, device=dev, dtype=torch.float16)
            dist.barrier()                # the kernel waits for its peers for about a second only
            comm.all_reduce(it & 1, out, n, input=torch.from_numpy(parts[rank]).to(dev))
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy().view(np.uint16), _expected(parts).view(np.uint16)), f"two-shot all-reduce n={n}"
        assert comm.status() == 0
        dist.barrier()
        comm.close()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))


@pytest.mark.timeout(300)
def test_two_ranks_twoshot_allreduce(monkeypatch):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    monkeypatch.setenv("B200K_COMM_TWOSHOT", "1")      # inherited by the ranks; read once per process by the library
    world, port = 2, 29741
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_twoshot, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            r, msg = q.get(timeout=240)
            results[r] = msg
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert all(v == "ok" for v in results.values()), results

"""Tensor-parallel sharding of the layer's int4 weights, checked on CPU with two gloo
ranks: every rank runs the oracle on its shard, partial sums meet in an all-reduce,
and the result must equal the unsharded oracle."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _rank_main(rank, world, port, fmt, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "oracle"))
    import importlib
    import oracle as o
    pkg = importlib.import_module("triton-rs_b200")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(123)                       # same weights on every rank
        H, hq, hkv, d, I, G, B = 256, 4, 2, 128, 512, 128, 3
        shape = pkg.LayerShape(H, hq, hkv, d, I, G)

        def quant(k, n):
            nib = rng.integers(0, 16, (k, n), dtype=np.int32)
            zer = rng.integers(0, 16, (k // G, n), dtype=np.int32)
            sc = rng.uniform(0.002, 0.02, (k // G, n)).astype(np.float16)
            if fmt == "gptq":
                return o.pack_gptq_qweight(nib), sc, o.pack_rowpacked_straight(zer)
            return o.pack_awq(nib), sc, o.pack_awq(zer)
        full = {"qkv": quant(H, (hq + 2 * hkv) * d), "o": quant(hq * d, H), "gate_up": quant(H, 2 * I),
                "down": quant(I, H)}
        gemm = (lambda a, w: o.w4a16_gptq_gemm(a, *w, G)) if fmt == "gptq" else (lambda a, w: o.awq_gemm_int4(a, *w, G))
        x = rng.standard_normal((B, H)).astype(np.float16)
        att = rng.standard_normal((B, hq * d)).astype(np.float16)

        # unsharded reference
        qkv_ref = gemm(x, full["qkv"])
        o_ref = gemm(att, full["o"])
        gu_ref = gemm(x, full["gate_up"])
        act_ref = o.fused_silu_mul_interleaved(gu_ref, I).astype(np.float16)
        dn_ref = gemm(act_ref, full["down"])

        tw = {k: tuple(None if t is None else torch.from_numpy(t) for t in v) for k, v in full.items()}
        loc = pkg.shard_layer_weights(tw, shape, rank, world, fmt)
        loc = {k: tuple(None if t is None else t.numpy() for t in v) for k, v in loc.items()}
        ls = shape.local(world)

        # column-parallel QKV: this rank's q heads, k heads, v heads
        qkv = gemm(x, loc["qkv"])
        hq_l, hkv_l = ls.num_q_heads, ls.num_kv_heads
        want = np.concatenate([
            qkv_ref[:, rank * hq_l * d:(rank + 1) * hq_l * d],
            qkv_ref[:, hq * d + rank * hkv_l * d: hq * d + (rank + 1) * hkv_l * d],
            qkv_ref[:, (hq + hkv) * d + rank * hkv_l * d:(hq + hkv) * d + (rank + 1) * hkv_l * d]], axis=1)
        assert np.allclose(qkv, want, rtol=1e-5, atol=1e-5)
        # row-parallel o_proj: local heads' slice of the attention output, then all-reduce
        att_l = att[:, rank * hq_l * d:(rank + 1) * hq_l * d]
        part = torch.from_numpy(gemm(att_l, loc["o"]).astype(np.float32))
        dist.all_reduce(part)
        assert np.allclose(part.numpy(), o_ref, rtol=1e-4, atol=1e-4)
        # column-parallel gate_up keeps gate/up pairs together; row-parallel down + all-reduce
        gu = gemm(x, loc["gate_up"])
        act = o.fused_silu_mul_interleaved(gu, ls.intermediate).astype(np.float16)
        assert np.array_equal(act, act_ref[:, rank * ls.intermediate:(rank + 1) * ls.intermediate])
        part = torch.from_numpy(gemm(act, loc["down"]).astype(np.float32))
        dist.all_reduce(part)
        assert np.allclose(part.numpy(), dn_ref, rtol=1e-4, atol=1e-4)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt", ["gptq", "awq"])
def test_tp2_sharding_matches_unsharded(fmt):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 1000) + (0 if fmt == "gptq" else 1)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, fmt, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res


def _ep_rank_main(rank, world, port, q):
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle as o
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(77)                       # same inputs on every rank
        T, E, k, H, I, G = 19, 4, 2, 128, 128, 128
        x = rng.standard_normal((T, H)).astype(np.float16)
        logits = rng.standard_normal((T, E)).astype(np.float32)
        w13q = np.stack([o.pack_gptq_qweight(rng.integers(1, 16, (H, 2 * I), dtype=np.int32)) for _ in range(E)])
        w13s = rng.uniform(0.002, 0.02, (E, H // G, 2 * I)).astype(np.float16)
        w2q = np.stack([o.pack_gptq_qweight(rng.integers(1, 16, (I, H), dtype=np.int32)) for _ in range(E)])
        w2s = rng.uniform(0.002, 0.02, (E, I // G, H)).astype(np.float16)
        full = o.fused_moe_gptq(x, logits, w13q, w13s, w2q, w2s, k, G)
        per = E // world
        lo, hi = rank * per, (rank + 1) * per
        share = o.fused_moe_gptq(x, logits, w13q[lo:hi], w13s[lo:hi], w2q[lo:hi], w2s[lo:hi], k, G, expert_first=lo)
        total = torch.from_numpy(share.copy())
        dist.all_reduce(total)                                # the one exchange of the expert-parallel scheme
        assert np.allclose(total.numpy(), full, rtol=1e-5, atol=1e-5), np.abs(total.numpy() - full).max()
        # every (token, slot) pair is owned by exactly one rank
        ids, _ = o.moe_route(logits, k)
        owned = torch.from_numpy(((ids >= lo) & (ids < hi)).astype(np.int64))
        dist.all_reduce(owned)
        assert (owned.numpy() == 1).all()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_shares_all_reduce_to_the_full_moe():
    """Expert-parallel MoE on two gloo CPU ranks: replicated tokens, routing recomputed on every rank, each rank
    adds the share of its experts, one all-reduce completes the output."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 1000) + 7
    procs = [ctx.Process(target=_ep_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res

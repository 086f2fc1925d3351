"""The decode-layer chain through the C ABI against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def make_layer(oracle, rng, H, hq, hkv, d, I, G, ml, sym=False, zero_mean=False):
    def gptq(k, n):
        if zero_mean:
            # nibbles 1..15 around the zero-point 8 (stored 7, +1 in the GEMM): weights with no DC
            # component, so that a deep K (14336) cannot push fp16 activations to overflow
            qw = oracle.pack_gptq_qweight(rng.integers(1, 16, (k, n), dtype=np.int32))
            qz = np.full((k // G, n // 8), 0x77777777, dtype=np.int32)
        else:
            qw = oracle.pack_gptq_qweight(rng.integers(0, 16, (k, n), dtype=np.int32))
            qz = None if sym else oracle.pack_rowpacked_straight(rng.integers(0, 16, (k // G, n), dtype=np.int32))
        sc = rng.uniform(0.002, 0.02, (k // G, n)).astype(np.float16)
        return qw, sc, qz
    cos, sin = oracle.rope_tables(ml, d, 500000.0)
    return dict(hq=hq, hkv=hkv, d=d, group=G, zero_offset=1, eps=1e-5, cos=cos, sin=sin,
                ln1=rng.uniform(0.5, 1.5, H).astype(np.float16), ln2=rng.uniform(0.5, 1.5, H).astype(np.float16),
                qkv=gptq(H, (hq + 2 * hkv) * d), o=gptq(hq * d, H), gate_up=gptq(H, 2 * I), down=gptq(I, H))


def to_dev(p):
    w = {k: tuple(None if x is None else t(x) for x in p[k]) for k in ("qkv", "o", "gate_up", "down")}
    return w, t(p["ln1"]), t(p["ln2"]), t(p["cos"]), t(p["sin"])


@pytest.mark.parametrize("use_graph", [False, True])
@pytest.mark.parametrize("sym", [False, True])
def test_layer_small_vs_numpy_oracle(pkg, oracle, use_graph, sym):
    rng = np.random.default_rng(17)
    B, H, hq, hkv, d, I, G, ml = 3, 256, 4, 2, 128, 384, 128, 40
    p = make_layer(oracle, rng, H, hq, hkv, d, I, G, ml, sym)
    shape = pkg.LayerShape(H, hq, hkv, d, I, G, 1e-5)
    w, ln1, ln2, cos, sin = to_dev(p)
    kc = rng.standard_normal((B, hkv, ml, d)).astype(np.float16)
    vc = rng.standard_normal((B, hkv, ml, d)).astype(np.float16)
    layer = pkg.DecodeLayer(shape, w, ln1, ln2, cos, sin, max_batch=4, max_len=ml, use_graph=use_graph,
                            k_cache=t(kc), v_cache=t(vc))
    if sym:
        p = dict(p, zero_offset=0, **{k: (p[k][0], p[k][1], None) for k in ("qkv", "o", "gate_up", "down")})
    for step, pos in enumerate([[5, 0, 38], [6, 1, 39]]):       # second step replays the captured graph
        pos = np.array(pos, dtype=np.int32)
        hidden = rng.standard_normal((B, H)).astype(np.float16)
        ref = oracle.decode_layer(hidden, p, kc, vc, pos)       # appends into kc, vc
        out = layer.forward(t(hidden), t(pos))
        assert_close(out.float().cpu().numpy(), ref, 2e-2, 2e-2, f"layer step {step}")
        assert_close(layer.k_cache.float().cpu().numpy(), kc.astype(np.float32), 2e-3, 2e-3, "k cache")
        assert_close(layer.v_cache.float().cpu().numpy(), vc.astype(np.float32), 2e-3, 2e-3, "v cache")
    # host-buffer entry point
    hidden = rng.standard_normal((B, H)).astype(np.float16)
    pos = np.array([7, 2, 3], dtype=np.int32)
    ref = oracle.decode_layer(hidden, p, kc, vc, pos)
    hh = torch.from_numpy(hidden).pin_memory()
    hp = torch.from_numpy(pos).pin_memory()
    ho = torch.empty((B, H), dtype=torch.float16).pin_memory()
    layer.forward_host(hh, hp, ho)
    torch.cuda.synchronize()
    assert_close(ho.float().numpy(), ref, 2e-2, 2e-2, "layer via host buffers")
    # staged form == fused form
    part = torch.empty((B, H), dtype=torch.float16, device=DEV)
    part2 = torch.empty_like(part)
    o2 = torch.empty_like(part)
    hd, pd = t(hidden), t(np.array([8, 3, 4], dtype=np.int32))
    kc0, vc0 = layer.k_cache.clone(), layer.v_cache.clone()
    full = layer.forward(hd, pd)
    layer.set_kv_cache(kc0, vc0)
    layer.forward_stage(0, hidden=hd, positions=pd, partial=part, batch=B)
    layer.forward_stage(1, hidden=hd, reduced=part, partial=part2, batch=B)
    layer.forward_stage(2, reduced=part2, out=o2, batch=B)
    assert torch.equal(full, o2)
    layer.close()


def test_layer_llama_shape_vs_c_oracle(pkg, oracle, oracle_c):
    """BASELINE config 4 extents with a short context (the C oracle handles it in seconds)."""
    import ctypes
    rng = np.random.default_rng(4)
    B, H, hq, hkv, d, I, G, ml = 8, 4096, 32, 8, 128, 14336, 128, 300
    p = make_layer(oracle, rng, H, hq, hkv, d, I, G, ml, zero_mean=True)
    w, ln1, ln2, cos, sin = to_dev(p)
    kc = rng.standard_normal((B, hkv, ml, d)).astype(np.float16)
    vc = rng.standard_normal((B, hkv, ml, d)).astype(np.float16)
    layer = pkg.DecodeLayer(pkg.LayerShape(), w, ln1, ln2, cos, sin, max_batch=B, max_len=ml, k_cache=t(kc), v_cache=t(vc))
    hidden = rng.standard_normal((B, H)).astype(np.float16)
    pos = rng.integers(100, ml - 1, B).astype(np.int32)
    out = layer.forward(t(hidden), t(pos))
    ref = np.zeros((B, H), np.float32)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    args = [ptr(hidden), ptr(ref), B, H, hq, hkv, d, I, G, 1, ctypes.c_float(1e-5), ptr(p["ln1"]), ptr(p["ln2"])]
    for name in ("qkv", "o", "gate_up", "down"):
        args += [ptr(x) for x in p[name]]
    args += [ptr(p["cos"]), ptr(p["sin"]), ptr(pos), ptr(kc), ptr(vc), ml]
    oracle_c.oc_decode_layer(*args)
    assert np.isfinite(ref).all()
    # ten fp16 roundings deep, values up to a few hundred: tolerance relative to the row scale
    scale = np.abs(ref).max(axis=1, keepdims=True)
    err = np.abs(out.float().cpu().numpy() - ref)
    assert (err <= 2e-2 * scale + 2e-2).all(), float((err / scale).max())
    layer.close()

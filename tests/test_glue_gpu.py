"""CUDA glue kernels (through the C ABI) against the CPU oracle and the golden vectors."""
import numpy as np
import pytest
import torch

from conftest import assert_close, golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def padded(shape, dtype, fill):
    """A tensor view inside a poison-filled buffer, to catch out-of-bounds writes."""
    n = int(np.prod(shape))
    buf = torch.full((n + 64,), fill, dtype=dtype, device=DEV)
    return buf, buf[32:32 + n].view(*shape)


def check_padding(buf, n, fill):
    assert (buf[:32] == fill).all() and (buf[32 + n:] == fill).all(), "write outside the output"


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("rows,n", [(1, 8), (3, 100), (16, 1024), (64, 4096), (5, 4104), (2, 40000), (7, 33)])
def test_rms_norm(P, oracle, dtype, rows, n):
    rng = np.random.default_rng(rows * 1000 + n)
    x = rng.standard_normal((rows, n)).astype(dtype)
    w = rng.uniform(0.5, 1.5, n).astype(dtype)
    td = torch.float16 if dtype == np.float16 else torch.float32
    buf, y = padded((rows, n), td, 777.0)
    fn = P.rms_norm_f16 if dtype == np.float16 else P.rms_norm_f32
    fn(t(x), t(w), y, n, 1.0 / n, 1e-5, rows)
    ref = oracle.rms_norm(x, w, 1e-5)
    tol = (1e-2, 1e-2) if dtype == np.float16 else (1e-4, 1e-4)   # f32: run_rms_norm.rs:71-87
    assert_close(y.float().cpu().numpy(), ref, *tol, what="rms_norm")
    check_padding(buf, rows * n, 777.0)


def test_rms_norm_reference_example_inputs(P):
    # crates/triton-runtime/examples/run_rms_norm.rs:23-37,71-87
    rows, n, eps = 16, 1024, 1e-6
    x = np.sin(np.arange(rows * n, dtype=np.float32) * np.float32(0.01)).reshape(rows, n)
    w = (1.0 + np.arange(n, dtype=np.float32) * np.float32(0.001))
    y = torch.empty((rows, n), device=DEV)
    P.rms_norm_f32(t(x), t(w), y, n, 1.0 / n, eps, rows)
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + eps) * w
    got = y.cpu().numpy()
    assert (np.abs(got - want) <= np.maximum(1e-4, np.abs(want) * 1e-4)).all()


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("rows,n", [(16, 1024), (64, 4096), (3, 1001), (1, 16)])
def test_fused_add_rms_norm(P, oracle, dtype, rows, n):
    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, n)).astype(dtype)
    r = rng.standard_normal((rows, n)).astype(dtype)
    w = rng.uniform(0.5, 1.5, n).astype(dtype)
    td = torch.float16 if dtype == np.float16 else torch.float32
    y = torch.empty((rows, n), dtype=td, device=DEV)
    ro = torch.empty((rows, n), dtype=td, device=DEV)
    fn = P.fused_add_rms_norm_f16 if dtype == np.float16 else P.fused_add_rms_norm_f32
    fn(t(x), t(r), t(w), y, ro, n, 1.0 / n, 1e-5, rows)
    ref, rref = oracle.fused_add_rms_norm(x, r, w, 1e-5)
    if dtype == np.float16:
        # residual_out is the fp16 rounding of the exact fp32 sum: bit-exact
        assert (ro.cpu().numpy() == rref.astype(np.float16)).all()
        assert_close(y.float().cpu().numpy(), ref, what="fused_add_rms_norm")
    else:
        assert (ro.cpu().numpy() == rref).all()
        assert_close(y.cpu().numpy(), ref, 5e-3, 2e-3)     # run_fused_add_rms_norm.rs:86


@pytest.mark.parametrize("n", [0, 1, 7, 4096, 262144, 1000003])
def test_residual_add_and_silu(P, oracle, n):
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float16)
    b = rng.standard_normal(n).astype(np.float16)
    buf, out = padded((n,), torch.float16, 555.0)
    P.residual_add_f16(t(a), t(b), out, n)
    # one add, one rounding: bit-exact against fp16(a + b)
    assert (out.cpu().numpy() == (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16)).all()
    check_padding(buf, n, 555.0)
    ai = t(a)
    P.residual_add_inplace_f16(ai, t(b), n)
    assert (ai.cpu().numpy() == out.cpu().numpy()).all()
    P.fused_silu_mul_f16(t(a), t(b), out, n)
    assert_close(out.float().cpu().numpy(), oracle.fused_silu_mul(a, b), what="silu_mul f16")
    a32, b32 = a.astype(np.float32) * 3, b.astype(np.float32)
    o32 = torch.empty(n, device=DEV)
    P.fused_silu_mul_f32(t(a32), t(b32), o32, n)
    assert_close(o32.cpu().numpy(), oracle.fused_silu_mul(a32, b32), 1e-5, 1e-5)   # run_vec_add.rs:140
    P.residual_add_f32(t(a32), t(b32), o32, n)
    assert (o32.cpu().numpy() == a32 + b32).all()
    a3 = t(a32)
    P.residual_add_inplace_f32(a3, t(b32), n)
    assert (a3.cpu().numpy() == a32 + b32).all()


def test_unaligned_views(P):
    # pointers off a 16-byte boundary take the scalar path
    a = torch.randn(1001, device=DEV).half()
    b = torch.randn(1001, device=DEV).half()
    out = torch.zeros(1001, dtype=torch.float16, device=DEV)
    P.residual_add_f16(a[1:], b[1:], out[1:], 1000)
    assert (out[1:] == (a[1:].float() + b[1:].float()).half()).all() and out[0] == 0


@pytest.mark.parametrize("rows,inter", [(64, 14336), (3, 96), (5, 7), (1, 8)])
def test_silu_mul_interleaved(P, oracle, rows, inter):
    rng = np.random.default_rng(inter)
    gu = rng.standard_normal((rows, 2 * inter)).astype(np.float16)
    out = torch.empty((rows, inter), dtype=torch.float16, device=DEV)
    P.fused_silu_mul_interleaved_f16(t(gu), out, inter, rows * inter)
    assert_close(out.float().cpu().numpy(), oracle.fused_silu_mul_interleaved(gu, inter))
    gu32 = gu.astype(np.float32)
    o32 = torch.empty((rows, inter), device=DEV)
    P.fused_silu_mul_interleaved_f32(t(gu32), o32, inter, rows * inter)
    assert_close(o32.cpu().numpy(), oracle.fused_silu_mul_interleaved(gu32, inter), 1e-5, 1e-5)


def test_rope(P, oracle):
    rng = np.random.default_rng(5)
    cos, sin = oracle.rope_tables(4200, 128, 500000.0)
    for tokens, heads in [(64, 32), (64, 8), (1, 1), (5, 3)]:
        x = rng.standard_normal((tokens, heads, 128)).astype(np.float32)
        pos = rng.integers(0, 4200, tokens).astype(np.int32)
        out = torch.empty((tokens, heads, 128), device=DEV)
        P.rope_full_f32(t(x), t(cos), t(sin), t(pos), out, heads, 128, tokens)
        assert_close(out.cpu().numpy(), oracle.rope_full(x, cos, sin, pos), 1e-6, 1e-6)
        xh = x.astype(np.float16)
        oh = torch.empty((tokens, heads, 128), dtype=torch.float16, device=DEV)
        P.rope_full_f16(t(xh), t(cos), t(sin), t(pos), oh, heads, 128, tokens)
        ref = oracle.rope_full(xh, cos, sin, pos).astype(np.float16)
        assert (np.abs(oh.cpu().numpy().astype(np.float32) - ref.astype(np.float32)) <= 2e-3 + 1e-3 * np.abs(ref)).all()
    # single-position variants
    q = rng.standard_normal((32, 128)).astype(np.float32)
    out = torch.empty((32, 128), device=DEV)
    P.rope_q_f32(t(q), t(cos[17]), t(sin[17]), out, 128, 32)
    assert_close(out.cpu().numpy(), oracle.rope_single(q, cos[17], sin[17]), 1e-6, 1e-6)
    P.rope_k_f32(t(q[:8]), t(cos[3]), t(sin[3]), out[:8], 128, 8)
    assert_close(out[:8].cpu().numpy(), oracle.rope_single(q[:8], cos[3], sin[3]), 1e-6, 1e-6)


def test_kv_cache_append(P, oracle):
    rng = np.random.default_rng(6)
    b, h, d, ms = 5, 8, 128, 40
    nk = rng.standard_normal((b, h, d)).astype(np.float32)
    nv = rng.standard_normal((b, h, d)).astype(np.float32)
    kc = rng.standard_normal((ms, h, d)).astype(np.float32)
    vc = rng.standard_normal((ms, h, d)).astype(np.float32)
    idx = np.array([0, 39, 7, 8, 20], dtype=np.int32)
    kg, vg = t(kc), t(vc)
    P.kv_cache_append_f32(t(nk), t(nv), kg, vg, t(idx), h, d, b)
    oracle.kv_cache_append(nk, nv, kc, vc, idx)
    assert (kg.cpu().numpy() == kc).all() and (vg.cpu().numpy() == vc).all()
    # batched head-major fp16
    nk16, nv16 = nk.astype(np.float16), nv.astype(np.float16)
    kc = rng.standard_normal((b, h, ms, d)).astype(np.float16)
    vc = rng.standard_normal((b, h, ms, d)).astype(np.float16)
    kg, vg = t(kc), t(vc)
    P.kv_cache_append_hm_f16(t(nk16), t(nv16), kg, vg, t(idx), h, d, ms, b)
    oracle.kv_cache_append_hm(nk16, nv16, kc, vc, idx)
    assert (kg.cpu().numpy() == kc).all() and (vg.cpu().numpy() == vc).all()


def test_rope_kv_append_fused(P, oracle):
    rng = np.random.default_rng(8)
    b, hq, hkv, d, ml = 6, 8, 2, 128, 50
    cos, sin = oracle.rope_tables(ml, d, 500000.0)
    qkv = rng.standard_normal((b, (hq + 2 * hkv) * d)).astype(np.float16)
    pos = rng.integers(0, ml, b).astype(np.int32)
    kc = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
    vc = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
    kg, vg = t(kc), t(vc)
    qo = torch.empty((b, hq, d), dtype=torch.float16, device=DEV)
    P.rope_kv_append_hm_f16(t(qkv), t(cos), t(sin), t(pos), qo, kg, vg, hq, hkv, d, ml, b)
    q = qkv[:, :hq * d].reshape(b, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].reshape(b, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(b, hkv, d)
    qr = oracle.rope_full(q, cos, sin, pos).astype(np.float16)
    kr = oracle.rope_full(k, cos, sin, pos).astype(np.float16)
    oracle.kv_cache_append_hm(kr, v, kc, vc, pos)
    assert_close(qo.float().cpu().numpy(), qr.astype(np.float32), 2e-3, 2e-3)
    assert_close(kg.float().cpu().numpy(), kc.astype(np.float32), 2e-3, 2e-3)
    assert (vg.cpu().numpy() == vc).all()


def test_golden_glue(P):
    g = golden("glue")
    rows, n = g["x"].shape
    y = torch.empty((rows, n), dtype=torch.float16, device=DEV)
    P.rms_norm_f16(t(g["x"]), t(g["w"]), y, n, 1.0 / n, 1e-5, rows)
    assert_close(y.float().cpu().numpy(), g["rms"])
    out = torch.empty((rows, 96), dtype=torch.float16, device=DEV)
    P.fused_silu_mul_interleaved_f16(t(g["x"]), out, 96, rows * 96)
    assert_close(out.float().cpu().numpy(), g["silu_il"])
    tok, heads, d = g["xr"].shape
    o = torch.empty((tok, heads, d), dtype=torch.float16, device=DEV)
    P.rope_full_f16(t(g["xr"]), t(g["cos"]), t(g["sin"]), t(g["pos"]), o, heads, d, tok)
    assert_close(o.float().cpu().numpy(), g["rope"], 2e-3, 2e-3)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_rms_norm_at_the_reference_benchmark_size(P, oracle, dtype):
    """32768 rows of 1024: the size the reference publishes its rms_norm timing at (bench_rms_norm.rs); short rows take
    the warp-per-row kernel."""
    rows, n = 32768, 1024
    g = torch.Generator(device=DEV).manual_seed(9)
    tdt = torch.float32 if dtype == np.float32 else torch.float16
    x = torch.randn((rows, n), device=DEV, generator=g, dtype=tdt)
    w = (torch.rand(n, device=DEV, generator=g) + 0.5).to(tdt)
    y = torch.empty_like(x)
    (P.rms_norm_f32 if dtype == np.float32 else P.rms_norm_f16)(x, w, y, n, 1.0 / n, 1e-6, rows)
    sample = np.r_[0:64, rows - 64:rows]
    ref = oracle.rms_norm(x[sample].cpu().numpy(), w.cpu().numpy(), 1e-6)
    tol = (1e-4, 1e-4) if dtype == np.float32 else (1e-2, 1e-2)
    assert_close(y[sample].float().cpu().numpy(), ref, *tol, "rms_norm 32768 x 1024")
    assert torch.isfinite(y).all()

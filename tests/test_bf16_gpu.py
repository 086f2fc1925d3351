"""bf16 editions of the `_typed` kernels (the reference's kernels are generic over T = f32 / f16 / bf16): same oracle,
inputs rounded to bf16 first, outputs within 1e-2 + 1e-2 |ref| (bf16 keeps 8 significant bits: one output rounding is
up to 0.4 % of the value)."""
import numpy as np
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bf(a):
    """numpy fp32 -> torch bf16 on the device, and the same values back as fp32 numpy (what the oracle gets)."""
    tt = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).bfloat16()
    return tt, tt.float().cpu().numpy()


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def rb(w):
    """fp32 -> nearest bf16 -> fp32: the rounding of the dequantised weight before the product
    (the reference's as_t::<T> with T = bf16, `w4a16_gptq_gemm_typed.rs:256-260`)."""
    return torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32)).bfloat16().float().numpy()


@pytest.mark.parametrize("fmt", ["gptq", "awq"])
@pytest.mark.parametrize("m,k,n", [(1, 4096, 512), (16, 1024, 256), (64, 512, 384), (130, 256, 264), (300, 1024, 256)])
def test_gemm_bf16(P, oracle, fmt, m, k, n):
    rng = np.random.default_rng(m + k + n)
    g = 128
    a, a32 = bf(rng.standard_normal((m, k)))
    sc, sc32 = bf(rng.uniform(0.002, 0.02, (k // g, n)))
    nib = rng.integers(0, 16, (k, n), dtype=np.int32)
    zn = rng.integers(0, 16, (k // g, n), dtype=np.int32)
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    if fmt == "gptq":
        qw, qz = oracle.pack_gptq_qweight(nib), oracle.pack_rowpacked_straight(zn)
        ref = a32 @ rb((nib - (zn + 1)[np.arange(k) // g]).astype(np.float32) * sc32[np.arange(k) // g])
        qwd, qzd = t(qw), t(qz)
        P.w4a16_gptq_gemm_bf16(a, qwd, sc, qzd, c, m, n, k, g, k, 1, n, 1, n, 1, n // 8, 1, n, 1)
    else:
        qw, qz = oracle.pack_awq(nib), oracle.pack_awq(zn)
        ref = a32 @ rb((nib - zn[np.arange(k) // g]).astype(np.float32) * sc32[np.arange(k) // g])
        qwd, qzd = t(qw), t(qz)
        P.awq_gemm_int4_bf16(a, qwd, sc, qzd, c, m, n, k, g, k, 1, n // 8, 1, n, 1, n // 8, 1, n, 1)
    assert_close(c.float().cpu().numpy(), ref, what=f"{fmt} bf16 {m}x{k}x{n}")


def test_gptq_gemm_bf16_symmetric_and_strided(P, oracle):
    rng = np.random.default_rng(3)
    m, k, n, g = 6, 256, 72, 128
    a, a32 = bf(rng.standard_normal((m, k)))
    sc, sc32 = bf(rng.uniform(0.002, 0.02, (k // g, n)))
    nib = rng.integers(0, 16, (k, n), dtype=np.int32)
    qw = t(oracle.pack_gptq_qweight(nib))
    ref = a32 @ rb((nib - 8).astype(np.float32) * sc32[np.arange(k) // g])
    c = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    P.w4a16_gptq_gemm_bf16(a, qw, sc, None, c, m, n, k, g, k, 1, n, 1, n, 1, 0, 1, n, 1)      # qzeros NULL: zero-point 8
    assert_close(c.float().cpu().numpy(), ref, what="gptq bf16 symmetric")
    at = a.t().contiguous().t()                                  # transposed activations: the strided family
    P.w4a16_gptq_gemm_bf16(at, qw, sc, None, c, m, n, k, g, at.stride(0), at.stride(1), n, 1, n, 1, 0, 1, n, 1)
    assert_close(c.float().cpu().numpy(), ref, what="gptq bf16 strided")


def test_glue_bf16(P, oracle):
    rng = np.random.default_rng(5)
    rows, h, inter = 7, 4096, 1536
    x, x32 = bf(rng.standard_normal((rows, h)))
    r, r32 = bf(rng.standard_normal((rows, h)))
    w, w32 = bf(rng.uniform(0.5, 1.5, h))
    y = torch.empty_like(x)
    P.rms_norm_bf16(x, w, y, h, 1.0 / h, 1e-5, rows)
    assert_close(y.float().cpu().numpy(), oracle.rms_norm(x32, w32, 1e-5), what="rms_norm bf16")
    ro = torch.empty_like(x)
    P.fused_add_rms_norm_bf16(x, r, w, y, ro, h, 1.0 / h, 1e-5, rows)
    yo, rr = oracle.fused_add_rms_norm(x32, r32, w32, 1e-5)
    assert_close(y.float().cpu().numpy(), yo, what="fused_add_rms_norm bf16")
    assert_close(ro.float().cpu().numpy(), rr, what="fused_add_rms_norm bf16 residual")
    P.residual_add_bf16(x, r, y, rows * h)
    assert torch.equal(y, (x.float() + r.float()).bfloat16())
    z = x.clone()
    P.residual_add_inplace_bf16(z, r, rows * h)
    assert torch.equal(z, y)
    gu, gu32 = bf(rng.standard_normal((rows, 2 * inter)) * 2)
    act = torch.empty((rows, inter), dtype=torch.bfloat16, device=DEV)
    P.fused_silu_mul_interleaved_bf16(gu, act, inter, rows * inter)
    assert_close(act.float().cpu().numpy(), oracle.fused_silu_mul_interleaved(gu32, inter), what="silu_mul_interleaved bf16")
    ga, ga32 = bf(rng.standard_normal(5000) * 2)
    ub, ub32 = bf(rng.standard_normal(5000))
    so = torch.empty_like(ga)
    P.fused_silu_mul_bf16(ga, ub, so, 5000)
    assert_close(so.float().cpu().numpy(), oracle.fused_silu_mul(ga32, ub32), what="silu_mul bf16")
    # rope, kv append, embedding, softmax
    tok, heads, d = 5, 3, 128
    q, q32 = bf(rng.standard_normal((tok, heads, d)))
    cos, sin = oracle.rope_tables(50, d, 10000.0)
    pos = rng.integers(0, 50, tok).astype(np.int32)
    qo = torch.empty_like(q)
    P.rope_full_bf16(q, t(cos), t(sin), t(pos), qo, heads, d, tok)
    assert_close(qo.float().cpu().numpy(), oracle.rope_full(q32, cos, sin, pos), what="rope bf16")
    b, hk, ml = 3, 2, 9
    nk, _ = bf(rng.standard_normal((b, hk, d)))
    nv, _ = bf(rng.standard_normal((b, hk, d)))
    kc = torch.zeros((b, hk, ml, d), dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    idx = torch.tensor([0, 8, 4], dtype=torch.int32, device=DEV)
    P.kv_cache_append_hm_bf16(nk, nv, kc, vc, idx, hk, d, ml, b)
    for i, p_ in enumerate([0, 8, 4]):
        assert torch.equal(kc[i, :, p_], nk[i]) and torch.equal(vc[i, :, p_], nv[i])
    assert int((kc != 0).sum()) == int((nk != 0).sum())
    table, _ = bf(rng.standard_normal((40, 100)))
    ids = t(rng.integers(0, 40, 11).astype(np.int32))
    eo = torch.empty((11, 100), dtype=torch.bfloat16, device=DEV)
    P.embedding_lookup_bf16(table, ids, eo, 100, 11)
    assert torch.equal(eo, table[ids.long()])
    sx, sx32 = bf(rng.standard_normal((4, 1000)) * 3)
    so2 = torch.empty_like(sx)
    P.softmax_bf16(sx, so2, 4, 1000)
    assert_close(so2.float().cpu().numpy(), oracle.softmax(sx32), 1e-2, 1e-4, what="softmax bf16")


def test_decode_attention_bf16(P, oracle):
    rng = np.random.default_rng(8)
    hq, hkv, d, n = 8, 2, 128, 300
    q, q32 = bf(rng.standard_normal((hq, d)))
    scale = 1.0 / np.sqrt(d)
    k, k32 = bf(rng.standard_normal((n, hkv, d)))
    v, v32 = bf(rng.standard_normal((n, hkv, d)))
    out = torch.empty_like(q)
    P.decode_attention_bf16(q, k, v, out, hq, hkv, d, n, scale)
    assert_close(out.float().cpu().numpy(), oracle.decode_attention(q32, k32, v32, hkv, n, scale), what="decode attention bf16")
    cap = 320
    kh, kh32 = bf(rng.standard_normal((hkv, cap, d)))
    vh, vh32 = bf(rng.standard_normal((hkv, cap, d)))
    P.decode_attention_hm_bf16(q, kh, vh, out, hq, hkv, d, cap, n, scale)
    assert_close(out.float().cpu().numpy(), oracle.decode_attention_hm(q32, kh32, vh32, n, scale), what="decode attention hm bf16")
    bs, nblocks = 16, 24
    kp, kp32 = bf(rng.standard_normal((nblocks, bs, hkv, d)))
    vp, vp32 = bf(rng.standard_normal((nblocks, bs, hkv, d)))
    table = rng.permutation(nblocks)[: (n + bs - 1) // bs].astype(np.int32)
    P.paged_decode_attention_bf16(q, kp, vp, t(table), out, hq, hkv, d, n, bs, scale)
    assert_close(out.float().cpu().numpy(), oracle.paged_decode_attention(q32, kp32, vp32, table, n, bs, scale), what="paged bf16")


@pytest.mark.parametrize("b,hq,hkv,q_len,kv_len,off", [(1, 4, 2, 300, 300, 0), (2, 4, 1, 200, 500, 300), (1, 2, 2, 70, 70, 0)])
@pytest.mark.parametrize("d", [128, 64])
def test_flash_attn_full_bf16(P, oracle, b, hq, hkv, q_len, kv_len, off, d):
    """head_dim 128 takes the tensor-core kernel, 64 the general one."""
    rng = np.random.default_rng(q_len + d)
    q, q32 = bf(rng.standard_normal((b, hq, q_len, d)))
    k, k32 = bf(rng.standard_normal((b, hkv, kv_len, d)))
    v, v32 = bf(rng.standard_normal((b, hkv, kv_len, d)))
    scale = 1.0 / np.sqrt(d)
    out = torch.full(q.shape, float("nan"), device=DEV, dtype=torch.bfloat16)
    P.flash_attn_full_bf16(q, k, v, out, b, hq, hkv, q_len, kv_len, d, off, scale)
    assert_close(out.float().cpu().numpy(), oracle.flash_attn_full(q32, k32, v32, off, scale), what=f"prefill attention bf16 d={d}")

"""W4A16 GEMM (GPTQ, symmetric GPTQ, AWQ), dequant and unpack through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import assert_close, golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def make_case(oracle, fmt, m, k, n, g, seed, sym=False):
    rng = np.random.default_rng(seed)
    nib = rng.integers(0, 16, (k, n), dtype=np.int32)
    zer = rng.integers(0, 16, (k // g, n), dtype=np.int32)
    sc = rng.uniform(0.002, 0.02, (k // g, n)).astype(np.float16)
    a = rng.standard_normal((m, k)).astype(np.float16)
    if fmt == "gptq":
        qw = oracle.pack_gptq_qweight(nib)
        qz = None if sym else oracle.pack_rowpacked_straight(zer)
    else:
        qw, qz = oracle.pack_awq(nib), oracle.pack_awq(zer)
    return a, qw, sc, qz


def ref_gemm(oracle, fmt, a, qw, sc, qz, g):
    if fmt == "gptq":
        return oracle.w4a16_gptq_gemm(a, qw, sc, qz, g, zero_offset=1)
    return oracle.awq_gemm_int4(a, qw, sc, qz, g)


def run_gemm(P, fmt, a, qw, sc, qz, g):
    if fmt == "gptq":
        return P.gptq_gemm(t(a), t(qw), t(sc), None if qz is None else t(qz), g)
    return P.awq_gemm(t(a), t(qw), t(sc), t(qz), g)


def test_unpack_bit_exact(P, oracle):
    rng = np.random.default_rng(11)
    for words in (rng.integers(0, 2 ** 32, (64, 48), dtype=np.uint64).astype(np.uint32),
                  np.full((16, 8), 0x76543210, dtype=np.uint32),
                  np.full((8, 8), 0xF0000000, dtype=np.uint32)):
        w = words.view(np.int32)
        r, c = w.shape
        out = torch.empty((r * 8, c), dtype=torch.int8, device=DEV)
        P.b200k_unpack_gptq_qweight(t(w), out, r * 8, c)
        assert (out.cpu().numpy() == oracle.unpack_gptq_qweight(w)).all()
        out = torch.empty((r, c * 8), dtype=torch.int8, device=DEV)
        P.b200k_unpack_gptq_qzeros(t(w), out, r, c * 8, 1)
        assert (out.cpu().numpy() == oracle.unpack_rowpacked_straight(w) + 1).all()
        P.b200k_unpack_awq(t(w), out, r, c * 8)
        assert (out.cpu().numpy() == oracle.unpack_awq(w)).all()


def test_dequant_kernels(P, oracle):
    a, qw, sc, qz = make_case(oracle, "gptq", 1, 256, 72, 128, 12)
    out = torch.empty((72, 256), dtype=torch.float16, device=DEV)
    P.dequant_int4_to_fp16(t(qw), t(sc), t(qz), out, 256, 72, 128, 9)
    assert (out.cpu().numpy() == oracle.dequant_int4_to_fp16(qw, sc, qz, 128)).all()
    P.dequant_int4_sym_to_fp16(t(qw), t(sc), out, 256, 72, 128)
    assert (out.cpu().numpy() == oracle.dequant_int4_sym_to_fp16(qw, sc, 128)).all()


SHAPES = [
    # (m, k, n, g)
    (1, 128, 8, 128), (1, 4096, 4096, 128), (1, 512, 264, 64), (1, 14336, 512, 128),
    (2, 256, 72, 128), (3, 512, 136, 128), (16, 4096, 512, 128), (17, 1024, 256, 128),
    (64, 1024, 384, 128), (128, 512, 256, 128), (130, 256, 264, 32), (300, 1024, 256, 128), (1024, 512, 128, 128),
]


@pytest.mark.parametrize("fmt", ["gptq", "awq"])
@pytest.mark.parametrize("m,k,n,g", SHAPES)
def test_gemm_vs_oracle(P, oracle, fmt, m, k, n, g):
    a, qw, sc, qz = make_case(oracle, fmt, m, k, n, g, seed=m * 7 + k + n)
    c = run_gemm(P, fmt, a, qw, sc, qz, g)
    assert_close(c.float().cpu().numpy(), ref_gemm(oracle, fmt, a, qw, sc, qz, g), what=f"{fmt} {m}x{k}x{n}")
    c2 = run_gemm(P, fmt, a, qw, sc, qz, g)
    assert torch.equal(c, c2), "two runs differ"


@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (16, 4096, 512), (5, 256, 72)])
def test_gptq_sym_equals_stored_seven(P, oracle, m, k, n):
    a, qw, sc, _ = make_case(oracle, "gptq", m, k, n, 128, seed=99, sym=True)
    qz7 = np.full((k // 128, n // 8), 0x77777777, dtype=np.int32)
    c_sym = run_gemm(P, "gptq", a, qw, sc, None, 128)
    c_7 = run_gemm(P, "gptq", a, qw, sc, qz7, 128)
    if n % 32 == 0:
        assert torch.equal(c_sym, c_7)       # same kernel family, same arithmetic
    else:
        # a qzeros row pitch that is not a multiple of 16 bytes takes the strided family
        assert_close(c_7.float().cpu().numpy(), c_sym.float().cpu().numpy(), 2e-3, 2e-3)
    assert_close(c_sym.float().cpu().numpy(), oracle.w4a16_gptq_gemm(a, qw, sc, None, 128))


def test_gemm_strided_operands(P, oracle):
    # transposed A and a C with a row pitch: the strided family
    a, qw, sc, qz = make_case(oracle, "gptq", 6, 256, 72, 128, seed=5)
    at = t(np.ascontiguousarray(a.T)).t()            # [6,256] view with strides (1, 6)
    cbuf = torch.full((6, 100), 9.0, dtype=torch.float16, device=DEV)
    c = cbuf[:, :72]
    qwg, scg, qzg = t(qw), t(sc), t(qz)
    P.w4a16_gptq_gemm_f16(at, qwg, scg, qzg, c, 6, 72, 256, 128, at.stride(0), at.stride(1), qwg.stride(0),
                          qwg.stride(1), scg.stride(0), scg.stride(1), qzg.stride(0), qzg.stride(1), c.stride(0),
                          c.stride(1))
    assert_close(c.float().cpu().numpy(), oracle.w4a16_gptq_gemm(a, qw, sc, qz, 128))
    assert (cbuf[:, 72:] == 9.0).all()


def test_gemm_linearity_full_size(P, oracle):
    # size-independent property at a Llama shape: C(a1 + a2) == C(a1) + C(a2) within fp16 rounding
    rng = np.random.default_rng(21)
    k, n, g = 4096, 6144, 128
    qw = t(rng.integers(-2 ** 31, 2 ** 31, (k // 8, n), dtype=np.int64).astype(np.int32))
    sc = t(rng.uniform(0.002, 0.02, (k // g, n)).astype(np.float16))
    qz = t(rng.integers(-2 ** 31, 2 ** 31, (k // g, n // 8), dtype=np.int64).astype(np.int32))
    for m in (1, 16):
        a1 = torch.randn((m, k), device=DEV).half()
        a2 = torch.randn((m, k), device=DEV).half()
        s = (a1.float() + a2.float()).half()
        c1 = P.gptq_gemm(a1, qw, sc, qz, g).float()
        c2 = P.gptq_gemm(a2, qw, sc, qz, g).float()
        cs = P.gptq_gemm(s, qw, sc, qz, g).float()
        err = (cs - (c1 + c2)).abs()
        assert (err <= 3e-2 + 1e-2 * (c1 + c2).abs()).all(), float(err.max())


def test_golden_gemm(P):
    g = golden("gptq_gemm")
    c = P.gptq_gemm(t(g["a"]), t(g["qweight"]), t(g["scales"]), t(g["qzeros"]), 128)
    assert_close(c.float().cpu().numpy(), g["c"])
    c = P.gptq_gemm(t(g["a"]), t(g["qweight"]), t(g["scales"]), None, 128)
    assert_close(c.float().cpu().numpy(), g["c_sym"])
    w = golden("awq_gemm")
    c = P.awq_gemm(t(w["a"]), t(w["qweight"]), t(w["scales"]), t(w["qzeros"]), 128)
    assert_close(c.float().cpu().numpy(), w["c"])


@pytest.mark.parametrize("M,K,N,G,sym", [(64, 4096, 6144, 128, True), (16, 512, 256, 128, False), (1, 1024, 512, 128, False),
                                         (300, 1024, 256, 64, False), (7, 256, 128, 128, True)])
def test_prepermuted_activations_give_identical_bits(P, M, K, N, G, sym):
    """w4a16_gptq_gemm_kperm_f16 on permute_k8_f16(a) == the plain entry point on a, bit for bit."""
    gen = torch.Generator(device=DEV).manual_seed(M + K)
    a = torch.randn((M, K), device=DEV, generator=gen).half()
    qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 8, N), device=DEV, dtype=torch.int32, generator=gen)
    sc = (torch.rand((K // G, N), device=DEV, generator=gen) * 0.018 + 0.002).half()
    qz = None if sym else torch.randint(-2 ** 31, 2 ** 31 - 1, (K // G, N // 8), device=DEV, dtype=torch.int32, generator=gen)
    ref = P.gptq_gemm(a, qw, sc, qz, G)
    ap = torch.empty_like(a)
    st = torch.cuda.current_stream().cuda_stream
    P.permute_k8_f16(a, ap, M, K, st)
    chunk = a.view(M, K // 8, 8)[:, :, [0, 4, 1, 5, 2, 6, 3, 7]].reshape(M, K)
    assert torch.equal(ap, chunk)
    out = torch.empty_like(ref)
    P.w4a16_gptq_gemm_kperm_f16(ap, qw, sc, qz, out, M, N, K, G, st)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("m,k,inter,sym", [(64, 1024, 512, False), (5, 512, 192, True), (1, 256, 64, False), (200, 512, 128, False)])
def test_gate_up_gemm_with_fused_silu_mul(P, oracle, m, k, inter, sym):
    """w4a16_gptq_gemm_silu_mul_f16 = silu(a Wgate) * (a Wup), gate columns first, against the two-step oracle
    (GEMM in fp32, then fused_silu_mul_interleaved)."""
    a, qw, sc, qz = make_case(oracle, "gptq", m, k, 2 * inter, 128, seed=m + inter, sym=sym)
    gu = oracle.w4a16_gptq_gemm(a, qw, sc, qz, 128, zero_offset=1, faithful=True)
    ref = oracle.fused_silu_mul_interleaved(gu, inter)
    out = torch.full((m, inter), float("nan"), dtype=torch.float16, device=DEV)
    P.w4a16_gptq_gemm_silu_mul_f16(t(a), t(qw), t(sc), None if qz is None else t(qz), out, m, inter, k, 128)
    # the product of two GEMM outputs: each within 1e-2 of its value, so the bound is propagated through silu(g) * u
    g_, u_ = gu[:, :inter], gu[:, inter:]
    sil = g_ / (1.0 + np.exp(-g_))
    bound = 1e-2 + 1e-2 * np.abs(ref) + (1e-2 + 1e-2 * np.abs(g_)) * 1.1 * np.abs(u_) + (1e-2 + 1e-2 * np.abs(u_)) * np.abs(sil)
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert (np.abs(got - ref) <= bound).all(), float(np.abs(got - ref).max())
    # and plainly close: the fused form skips one fp16 rounding, it does not add error
    assert_close(got, ref, 2e-2, 2e-2, "fused gate_up + silu")


@pytest.mark.parametrize("m,k,n", [(1, 4096, 512), (1, 256, 264), (16, 1024, 256), (130, 512, 384)])
def test_awq_prepacked_into_the_k_packed_layout(P, oracle, m, k, n):
    """b200k_prepack_awq: the rewritten tensor holds the same nibbles (compared with == through the unpack probes), and
    awq_gemm_int4_prepacked_f16 on it gives the product of the original AWQ tensor."""
    g = 128
    a, qw, sc, qz = make_case(oracle, "awq", m, k, n, g, seed=k + n)
    qwd, qzd = t(qw), t(qz)
    qwp = torch.empty((k // 8, n), dtype=torch.int32, device=DEV)
    qzp = torch.empty((k // g, n // 8), dtype=torch.int32, device=DEV)
    P.b200k_prepack_awq(qwd, qzd, qwp, qzp, k, n, g)
    u0 = torch.empty((k, n), dtype=torch.int8, device=DEV)
    u1 = torch.empty_like(u0)
    P.b200k_unpack_awq(qwd, u0, k, n)
    P.b200k_unpack_gptq_qweight(qwp, u1, k, n)
    assert torch.equal(u0, u1)
    z0 = torch.empty((k // g, n), dtype=torch.int8, device=DEV)
    z1 = torch.empty_like(z0)
    P.b200k_unpack_awq(qzd, z0, k // g, n)
    P.b200k_unpack_gptq_qzeros(qzp, z1, k // g, n, 0)
    assert torch.equal(z0, z1)
    c = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    P.awq_gemm_int4_prepacked_f16(t(a), qwp, t(sc), qzp, c, m, n, k, g)
    assert_close(c.float().cpu().numpy(), oracle.awq_gemm_int4(a, qw, sc, qz, g), what="prepacked awq gemm")


@pytest.mark.parametrize("fmt", ["gptq", "awq"])
@pytest.mark.parametrize("k,n", [(4096, 512), (14336, 256)])
def test_gemv_with_massive_activations(P, oracle, fmt, k, n):
    """M = 1 with activation outliers (a few channels a thousand times the rest, as the massive activations of LLMs): the
    integer GEMV quantises activations per group of 128, which cannot hold both scales, and must fall back to fp32 for
    the groups that contain an outlier.  Also an all-zero group and an all-zero vector."""
    g = 128
    a, qw, sc, qz = make_case(oracle, fmt, 1, k, n, g, seed=k + n + 1)
    a = a.astype(np.float32)
    a[0, 5] = 2000.0                     # outlier in group 0
    a[0, 3 * g + 77] = -900.0            # and one in group 3
    a[0, g:2 * g] = 0.0                  # group 1: all zero
    a[0, 2 * g:3 * g] *= 1e-3            # group 2: tiny values only
    a = a.astype(np.float16)
    got = run_gemm(P, fmt, a, qw, sc, qz, g).float().cpu().numpy()
    ref = ref_gemm(oracle, fmt, a, qw, sc, qz, g)
    assert_close(got, ref, what=f"{fmt} gemv with outliers")
    # without the outliers' own terms the rest of the sum must still be right: compare the difference of two runs that
    # differ only in the outlier values (their groups stay on the fp32 path in both)
    a2 = a.copy()
    a2[0, 5] = 1000.0
    got2 = run_gemm(P, fmt, a2, qw, sc, qz, g).float().cpu().numpy()
    ref2 = ref_gemm(oracle, fmt, a2, qw, sc, qz, g)
    assert_close(got2, ref2, what=f"{fmt} gemv with outliers, second vector")
    z = np.zeros_like(a)
    assert not run_gemm(P, fmt, z, qw, sc, qz, g).float().cpu().numpy().any()

"""The benchmark's own configurations at their full sizes, through the C ABI, against the C/OpenMP oracle.

C0  GPTQ W4A16 GEMM, M = 16, K = N = 4096
C1  GQA decode attention, batch 32, 32 q / 8 kv heads, head_dim 128, lengths uniform in [512, 8192]
C2  AWQ W4A16 GEMM, M in {1, 16, 128, 1024} x the four Llama-3-8B projection shapes (16 cells)
C3  fused MoE, Mixtral-8x7B shape: 512 tokens, 8 experts, top-2
(C4, the layer chain, is in test_layer_gpu.py and in the benchmark's own parity gate.)
Inputs have the configs' distributions; fp16 outputs must satisfy |got - ref| <= 1e-2 + 1e-2 |ref|."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import assert_close, assert_close_terms

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
G = 128


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _gen(seed):
    return torch.Generator(device=DEV).manual_seed(seed)


def _ri(gen, *s):
    return torch.randint(-2 ** 31, 2 ** 31 - 1, s, device=DEV, dtype=torch.int32, generator=gen)


def _scales(gen, *s):
    return (torch.rand(s, device=DEV, generator=gen) * 0.018 + 0.002).half()


def test_c0_gptq_gemm_m16_4096x4096(P, oracle_c):
    gen = _gen(0)
    m, k, n = 16, 4096, 4096
    a = torch.randn((m, k), device=DEV, generator=gen).half()
    qw, sc = _ri(gen, k // 8, n), _scales(gen, k // G, n)
    qz = torch.full((k // G, n // 8), 0x77777777, device=DEV, dtype=torch.int32)      # zero-point 8 under the +1 rule
    got = P.gptq_gemm(a, qw, sc, qz, G).float().cpu().numpy()
    a32 = np.ascontiguousarray(a.float().cpu().numpy())
    ref = np.zeros((m, n), np.float32)
    oracle_c.oc_gptq_gemm(_p(a32), _p(qw.cpu().numpy()), _p(sc.cpu().numpy()), _p(qz.cpu().numpy()), _p(ref), m, n, k, G, 1)
    assert_close(got, ref, what="C0")
    # the symmetric entry point gives the same bits
    assert torch.equal(P.gptq_gemm(a, qw, sc, None, G), P.gptq_gemm(a, qw, sc, qz, G))


def test_c1_decode_attention_batch32_ragged(P, oracle_c):
    gen = _gen(1)
    b, hq, hkv, d, ml = 32, 32, 8, 128, 8192
    q = torch.randn((b, hq, d), device=DEV, generator=gen).half()
    kc = torch.randn((b, hkv, ml, d), device=DEV, generator=gen).half()
    vc = torch.randn((b, hkv, ml, d), device=DEV, generator=gen).half()
    lens = torch.randint(512, ml + 1, (b,), device=DEV, dtype=torch.int32, generator=gen)
    lens[0], lens[1] = 512, ml
    out = torch.empty_like(q)
    P.batched_decode_attention_hm_f16(q, kc, vc, lens, out, b, hq, hkv, d, ml, 1.0 / float(np.sqrt(d)))
    got = out.float().cpu().numpy()
    q32 = np.ascontiguousarray(q.float().cpu().numpy())
    kh, vh, lh = kc.cpu().numpy(), vc.cpu().numpy(), lens.cpu().numpy()
    ref = np.zeros((b, hq, d), np.float32)
    oracle_c.oc_batched_decode_attention_hm(_p(q32), _p(kh), _p(vh), _p(lh), _p(ref), b, hq, hkv, d, ml,
                                            ctypes.c_float(1.0 / np.sqrt(d)))
    assert_close(got, ref, what="C1")


@pytest.mark.parametrize("k,n", [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)])
@pytest.mark.parametrize("m", [1, 16, 128, 1024])
def test_c2_awq_gemm_cell(P, oracle_c, m, k, n):
    gen = _gen(2 + m + k + n)
    a = torch.randn((m, k), device=DEV, generator=gen).half()
    qw, qz, sc = _ri(gen, k, n // 8), _ri(gen, k // G, n // 8), _scales(gen, k // G, n)
    got = P.awq_gemm(a, qw, sc, qz, G).float().cpu().numpy()
    # the oracle checks every row up to M = 128 and every 8th row (128 rows across all token tiles) at M = 1024
    rows = np.arange(m) if m <= 128 else np.arange(3, m, 8)
    a32 = np.ascontiguousarray(a.float().cpu().numpy()[rows])
    ref = np.zeros((len(rows), n), np.float32)
    oracle_c.oc_awq_gemm(_p(a32), _p(qw.cpu().numpy()), _p(sc.cpu().numpy()), _p(qz.cpu().numpy()), _p(ref), len(rows), n, k, G)
    assert_close(got[rows], ref, what=f"C2 m={m} k={k} n={n}")


def test_c3_fused_moe_mixtral_shape(P, oracle_c):
    gen = _gen(3)
    T, E, k, H, I = 512, 8, 2, 4096, 14336
    w13q, w2q = _ri(gen, E, H // 8, 2 * I), _ri(gen, E, I // 8, H)
    w13s, w2s = _scales(gen, E, H // G, 2 * I), _scales(gen, E, I // G, H)
    x = torch.randn((T, H), device=DEV, generator=gen).half()
    logits = torch.randn((T, E), device=DEV, generator=gen)
    out = torch.empty((T, H), dtype=torch.float16, device=DEV)
    P.fused_moe_gptq_f16(x, logits, w13q, w13s, None, w2q, w2s, None, out, T, H, E, k, I, G, None, 0)
    got = out.float().cpu().numpy()
    ref, mag = np.zeros((T, H), np.float32), np.zeros((T, H), np.float32)
    ids = np.zeros((T, k), np.int32)
    oracle_c.oc_fused_moe_gptq(_p(x.cpu().numpy()), _p(np.ascontiguousarray(logits.cpu().numpy())), _p(w13q.cpu().numpy()),
                               _p(w13s.cpu().numpy()), _p(w2q.cpu().numpy()), _p(w2s.cpu().numpy()), _p(ref), T, H, E, k, I, G,
                               1, _p(ids), None, _p(mag))
    assert np.isfinite(ref).all()
    # routing must be identical (bit-exact item), the output a weighted sum of k expert outputs
    gids = torch.empty((T, k), dtype=torch.int32, device=DEV)
    gw = torch.empty((T, k), dtype=torch.float32, device=DEV)
    P.moe_route_topk_f32(logits, gids, gw, T, E, k)
    assert np.array_equal(gids.cpu().numpy(), ids)
    assert_close_terms(got, ref, mag, k, what="C3")

"""Projection helpers (split_qkv, head/token transposes, RoPE / QK-norm + RoPE fused with the transpose)
through the C ABI against the CPU oracle.  The pure moves are compared bit for bit."""
import numpy as np
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def S():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("batch,heads,d", [(64, 32, 128), (3, 5, 6), (1, 1, 1)])
def test_split_qkv(P, oracle, batch, heads, d):
    rng = np.random.default_rng(1)
    qkv = rng.standard_normal((batch, 3, heads, d)).astype(np.float32)
    outs = [torch.full((batch, heads, d), float("nan"), device=DEV) for _ in range(3)]
    P.split_qkv_f32(t(qkv), *outs, heads, d, batch, S())
    for got, ref in zip(outs, oracle.split_qkv(qkv, heads, d)):
        assert np.array_equal(got.cpu().numpy(), ref)


@pytest.mark.parametrize("tokens,heads,d", [(64, 32, 128), (7, 3, 10), (1, 4, 64)])
def test_transposes_are_exact_and_inverse(P, oracle, tokens, heads, d):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((tokens, heads, d)).astype(np.float32)
    hm = torch.full((heads, tokens, d), float("nan"), device=DEV)
    P.transpose_token_to_head_f32(t(x), hm, tokens, heads, d, S())
    assert np.array_equal(hm.cpu().numpy(), oracle.transpose_token_to_head(x))
    back = torch.full((tokens, heads, d), float("nan"), device=DEV)
    P.transpose_head_to_token_f32(hm, back, tokens, heads, d, S())
    assert np.array_equal(back.cpu().numpy(), x)
    assert np.array_equal(back.cpu().numpy(), oracle.transpose_head_to_token(hm.cpu().numpy()))


@pytest.mark.parametrize("tokens,heads,d,off", [(64, 32, 128, 4096), (5, 3, 64, 0), (2, 2, 6, 9)])
def test_rope_transpose(P, oracle, tokens, heads, d, off):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((tokens, heads, d)).astype(np.float32)
    cos, sin = oracle.rope_tables(off + tokens, d, 500000.0)
    out = torch.full((heads, tokens, d), float("nan"), device=DEV)
    P.rope_transpose_f32(t(x), t(cos), t(sin), out, tokens, heads, d, off, S())
    assert_close(out.cpu().numpy(), oracle.rope_transpose(x, cos, sin, off), 1e-5, 1e-5, "rope_transpose")


@pytest.mark.parametrize("tokens,heads,d,off", [(64, 32, 128, 4096), (5, 3, 64, 0), (2, 2, 6, 9)])
def test_qk_norm_rope_transpose(P, oracle, tokens, heads, d, off):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((tokens, heads, d)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    cos, sin = oracle.rope_tables(off + tokens, d, 1000000.0)
    out = torch.full((heads, tokens, d), float("nan"), device=DEV)
    P.qk_norm_rope_transpose_f32(t(x), t(w), t(cos), t(sin), out, tokens, heads, d, off, 1.0 / d, 1e-6, S())
    assert_close(out.cpu().numpy(), oracle.qk_norm_rope_transpose(x, w, cos, sin, off, 1e-6), 1e-4, 1e-5, "qk_norm_rope_transpose")


def test_empty_and_bad_arguments(P):
    z = torch.zeros(8, device=DEV)
    P.split_qkv_f32(None, None, None, None, 4, 8, 0, S())                  # empty batch: nothing to do
    P.rope_transpose_f32(None, None, None, None, 0, 4, 8, 0, S())
    with pytest.raises(Exception):
        P.rope_transpose_f32(z, z, z, z, 1, 1, 7, 0, S())                     # odd head_dim
    with pytest.raises(Exception):
        P.transpose_token_to_head_f32(None, z, 1, 1, 8, S())                  # NULL input

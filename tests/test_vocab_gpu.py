"""Embedding gather and row softmax (the two ends of a decode step) against the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def test_softmax_f32_reference_example(P, oracle):
    """crates/triton-runtime/examples/run_softmax.rs: 8 x 1024, its inputs and its tolerance."""
    rows, cols = 8, 1024
    i = np.arange(rows * cols)
    x = (((i % cols).astype(np.float32) - np.float32(512.0)) * np.float32(0.01) * (i // cols + 1).astype(np.float32)).reshape(rows, cols)
    out = torch.empty((rows, cols), dtype=torch.float32, device=DEV)
    P.softmax_f32(t(x), out, rows, cols)
    got, want = out.cpu().numpy(), oracle.softmax(x)
    assert (np.abs(got - want) <= np.maximum(1e-5, np.abs(want) * 1e-4)).all()
    assert (np.abs(got.sum(axis=1) - 1.0) <= 1e-4).all()


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (5, 1000), (2, 128256), (64, 4096)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_softmax_shapes(P, oracle, rows, cols, dtype):
    rng = np.random.default_rng(rows * 131 + cols)
    x = (rng.standard_normal((rows, cols)) * 3).astype(dtype)
    if cols > 2:
        x[0, 1] = 11.0                      # a dominant element and a far-away minimum
        x[0, 2] = -60.0
    out = torch.full((rows, cols), float("nan"), dtype=torch.float32 if dtype == np.float32 else torch.float16, device=DEV)
    (P.softmax_f32 if dtype == np.float32 else P.softmax_f16)(t(x), out, rows, cols)
    got, want = out.float().cpu().numpy(), oracle.softmax(x)
    tol = (1e-6, 1e-4) if dtype == np.float32 else (1e-4, 2e-3)      # f16: one rounding at the store
    assert np.isfinite(got).all()
    assert (np.abs(got - want) <= tol[0] + tol[1] * np.abs(want)).all()


@pytest.mark.parametrize("hidden", [4096, 100, 3])      # 16-byte rows and rows that are not
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_embedding_lookup_is_bit_exact(P, oracle, hidden, dtype):
    rng = np.random.default_rng(hidden)
    vocab, tokens = 300, 77
    table = rng.standard_normal((vocab, hidden)).astype(dtype)
    idx = rng.integers(0, vocab, tokens).astype(np.int32)
    idx[:3] = [0, vocab - 1, vocab - 1]
    out = torch.zeros((tokens, hidden), dtype=torch.float32 if dtype == np.float32 else torch.float16, device=DEV)
    (P.embedding_lookup_f32 if dtype == np.float32 else P.embedding_lookup_f16)(t(table), t(idx), out, hidden, tokens)
    assert np.array_equal(out.cpu().numpy(), oracle.embedding_lookup(table, idx))


def test_empty_calls_launch_nothing(P):
    z = torch.zeros(8, device=DEV)
    P.softmax_f32(z, z, 0, 8)
    P.embedding_lookup_f32(z, torch.zeros(1, dtype=torch.int32, device=DEV), z, 8, 0)

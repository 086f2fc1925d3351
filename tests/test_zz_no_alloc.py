"""The allocation-free attention entry point gives the same answer as the ordinary one.

Some callers of this library own every byte of GPU memory themselves and cannot let a library
call cudaMalloc behind their back; `batched_decode_attention_hm_f16_noalloc` serves them from a
scratch array built into the library.  This file is collected last on purpose: if it fails, every
other test has already run."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, b, hq, hkv, ml):
    g = torch.Generator(device=DEV).manual_seed(seed)
    d = 128
    q = torch.randn((b, hq, d), device=DEV, generator=g).half()
    k = torch.randn((b, hkv, ml, d), device=DEV, generator=g).half()
    v = torch.randn((b, hkv, ml, d), device=DEV, generator=g).half()
    lens = torch.randint(1, ml + 1, (b,), device=DEV, dtype=torch.int32, generator=g)
    return q, k, v, lens, d


def test_noalloc_matches_regular_entry_twice_in_a_row(P):
    for seed, (b, hq, hkv, ml) in enumerate([(4, 32, 8, 3000), (6, 16, 4, 1500)]):   # two calls in a row, different shapes
        q, k, v, lens, d = _case(seed, b, hq, hkv, ml)
        want = torch.empty((b, hq, d), dtype=torch.float16, device=DEV)
        got = torch.full_like(want, float("nan"))
        scale = 1.0 / float(np.sqrt(d))
        P.batched_decode_attention_hm_f16(q, k, v, lens, want, b, hq, hkv, d, ml, scale)
        before = torch.cuda.memory_allocated()
        P.batched_decode_attention_hm_f16_noalloc(q, k, v, lens, got, b, hq, hkv, d, ml, scale)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        err = (got.float() - want.float()).abs()
        assert torch.isfinite(got).all()
        assert (err <= 1e-2 + 1e-2 * want.float().abs()).all(), float(err.max())
        assert torch.equal(got, want)          # same kernel, same partial order: the bits agree too


def test_noalloc_rejects_oversized_shapes(pkg, P):
    b, hq, hkv, ml, d = 512, 64, 64, 65536, 128     # scratch need far beyond the built-in array
    need = pkg.lib().call("b200k_attention_workspace_bytes", b, hq, hkv, d, ml)
    assert need > 8 << 20
    t = torch.zeros(16, dtype=torch.float16, device=DEV)
    lens = torch.zeros(b, dtype=torch.int32, device=DEV)
    with pytest.raises(pkg.B200KError) as e:
        P.batched_decode_attention_hm_f16_noalloc(t, t, t, lens, t, b, hq, hkv, d, ml, 0.1)
    assert e.value.code == -4 and "bytes of scratch" in e.value.message

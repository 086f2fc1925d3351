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
        P.batched_decode_attention_hm_f16_noalloc(q, k, v, lens, got, b, hq, hkv, d, ml, scale)
        torch.cuda.synchronize()
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


_FRESH = r"""
import ctypes, importlib, sys
import numpy as np, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/oracle")
import oracle
pkg = importlib.import_module("triton-rs_b200")
P = pkg.prelude
dev = "cuda:0"
rng = np.random.default_rng(5)
b, hq, hkv, d, ml = 3, 16, 4, 128, 900
q = rng.standard_normal((b, hq, d)).astype(np.float16)
k = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
v = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
lens = np.array([900, 1, 333], np.int32)
t = lambda a: torch.from_numpy(a).to(dev)
qd, kd, vd, ld = t(q), t(k), t(v), t(lens)
out = torch.empty((b, hq, d), dtype=torch.float16, device=dev)
scale = 1.0 / float(np.sqrt(d))
# set-up call: batch 0 launches nothing but makes the library's static array resident
P.batched_decode_attention_hm_f16_noalloc(qd, kd, vd, ld, out, 0, hq, hkv, d, ml, scale)
P.batched_decode_attention_hm_f16_noalloc(qd, kd, vd, ld, out, b, hq, hkv, d, ml, scale)     # first real call
out.fill_(float("nan"))                        # (before the measurement: torch loads its fill kernel on first use)
torch.cuda.synchronize()
free0 = torch.cuda.mem_get_info()[0]           # device-wide free bytes (cudaMemGetInfo): sees any cudaMalloc
P.batched_decode_attention_hm_f16_noalloc(qd, kd, vd, ld, out, b, hq, hkv, d, ml, scale)     # second call
torch.cuda.synchronize()
free1 = torch.cuda.mem_get_info()[0]
assert free1 == free0, (free0, free1)
ref = oracle.batched_decode_attention_hm(q, k, v, lens, scale)
got = out.float().cpu().numpy()
assert np.isfinite(got).all() and (np.abs(got - ref) <= 1e-2 + 1e-2 * np.abs(ref)).all()
st = ctypes.c_int(-1)
pkg.lib().call("b200k_noalloc_status", ctypes.addressof(st), torch.cuda.current_stream().cuda_stream)
assert st.value == 0
assert torch.cuda.mem_get_info()[0] == free0
print("fresh-process noalloc ok")
"""


def test_noalloc_in_a_fresh_process_allocates_nothing_and_matches_the_oracle():
    """A process that never touches the ordinary entry point (so the library's default workspace is never created):
    device-wide free memory is the same before and after a call, the result agrees with the CPU oracle, and the status
    word of the built-in array reads 0 through b200k_noalloc_status."""
    import subprocess
    import sys
    from conftest import ROOT
    r = subprocess.run([sys.executable, "-c", _FRESH.format(root=str(ROOT))], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "fresh-process noalloc ok" in r.stdout, r.stdout + r.stderr

"""The library's glue kernels against the REFERENCE's own CUDA fixtures.

`oracle/Makefile` (`make ref`) compiles the reference's tools/reference_cu/{rms_norm, residual_add,
fused_silu_mul}.cu, unmodified and where they lie, into oracle/_ref/*.cubin (built files, not tracked).
Here those kernels are launched through the CUDA driver API on the same inputs as the library's entry
points.  Skipped when the cubins have not been built."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import ROOT, assert_close

pytestmark = pytest.mark.gpu
REF = ROOT / "oracle" / "_ref"
DEV = "cuda:0"


def _kernel(cubin: str, name: str):
    path = REF / cubin
    if not path.exists():
        pytest.skip(f"{path} not built (make -C oracle ref)")
    from cuda.bindings import driver
    torch.zeros(1, device=DEV)                       # torch's primary context becomes current
    err, mod = driver.cuModuleLoadData(path.read_bytes())
    assert err == driver.CUresult.CUDA_SUCCESS, err
    err, fn = driver.cuModuleGetFunction(mod, name.encode())
    assert err == driver.CUresult.CUDA_SUCCESS, err

    def launch(grid, block, values, types):
        st = torch.cuda.current_stream().cuda_stream
        (e,) = driver.cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, 0, st, (tuple(values), tuple(types)), 0)
        assert e == driver.CUresult.CUDA_SUCCESS, e
        torch.cuda.synchronize()
    launch.module = mod
    return launch


P_, I_, F_ = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


@pytest.mark.parametrize("rows,n", [(64, 4096), (7, 3008), (1, 128)])   # the fixture wants whole warps per block
def test_rms_norm_f16_matches_reference_fixture(pkg, rows, n):
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn((rows, n), device=DEV, generator=g, dtype=torch.float16)
    w = (torch.rand(n, device=DEV, generator=g) + 0.5).half()
    ref, out = torch.empty_like(x), torch.empty_like(x)
    _kernel("rms_norm.cubin", "rms_norm_f16")(rows, min(n, 1024), (x.data_ptr(), w.data_ptr(), ref.data_ptr(), n, 1e-5),
                                               (P_, P_, P_, I_, F_))
    pkg.prelude.rms_norm_f16(x, w, out, n, 1.0 / n, 1e-5, rows, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    # the fixture is built with --use_fast_math (approximate rsqrt); one fp16 ulp is the most that can differ
    assert_close(out.float().cpu().numpy(), ref.float().cpu().numpy(), 2e-3, 2e-3, "rms_norm vs reference fixture")


@pytest.mark.parametrize("n", [64 * 4096, 1001])
def test_residual_add_f16_matches_reference_fixture_bit_for_bit(pkg, n):
    g = torch.Generator(device=DEV).manual_seed(4)
    a = torch.randn(n, device=DEV, generator=g, dtype=torch.float16)
    b = torch.randn(n, device=DEV, generator=g, dtype=torch.float16)
    ref, out = torch.empty_like(a), torch.empty_like(a)
    _kernel("residual_add.cubin", "residual_add_f16")((n + 255) // 256, 256, (a.data_ptr(), b.data_ptr(), ref.data_ptr(), n),
                                                       (P_, P_, P_, I_))
    pkg.prelude.residual_add_f16(a, b, out, n, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("batch,inter", [(64, 14336), (3, 520)])
def test_silu_mul_interleaved_f16_matches_reference_fixture(pkg, batch, inter):
    g = torch.Generator(device=DEV).manual_seed(5)
    gu = torch.randn((batch, 2 * inter), device=DEV, generator=g, dtype=torch.float16) * 2
    total = batch * inter
    ref = torch.empty((batch, inter), device=DEV, dtype=torch.float16)
    out = torch.empty_like(ref)
    _kernel("fused_silu_mul.cubin", "fused_silu_mul_interleaved_f16")((total + 255) // 256, 256,
                                                                      (gu.data_ptr(), ref.data_ptr(), inter, total), (P_, P_, I_, I_))
    pkg.prelude.fused_silu_mul_interleaved_f16(gu, out, inter, total, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    # fast-math exp / division in the fixture: allow an fp16 ulp or two
    assert_close(out.float().cpu().numpy(), ref.float().cpu().numpy(), 3e-3, 3e-3, "silu_mul vs reference fixture")


def test_silu_mul_f16_matches_reference_fixture(pkg):
    g = torch.Generator(device=DEV).manual_seed(6)
    n = 5000
    a = torch.randn(n, device=DEV, generator=g, dtype=torch.float16) * 2
    b = torch.randn(n, device=DEV, generator=g, dtype=torch.float16)
    ref, out = torch.empty_like(a), torch.empty_like(a)
    _kernel("fused_silu_mul.cubin", "fused_silu_mul_f16")((n + 255) // 256, 256, (a.data_ptr(), b.data_ptr(), ref.data_ptr(), n),
                                                          (P_, P_, P_, I_))
    pkg.prelude.fused_silu_mul_f16(a, b, out, n, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert_close(out.float().cpu().numpy(), ref.float().cpu().numpy(), 3e-3, 3e-3, "silu_mul vs reference fixture")

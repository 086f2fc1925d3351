"""Host-side mirror of `triton_kernels::prelude` (crates/triton-kernels/src/lib.rs:45-76)
plus the two int4 GEMMs of `triton-dsl/examples`.

Every function has the reference kernel's name and takes the reference kernel's
arguments in the reference's order, followed by the extents the reference took from
its launch grid; tensors are torch CUDA tensors (used only as owners of device
memory), and the call goes straight to the C ABI on torch's current stream unless
`stream=` says otherwise.  Example, next to the reference's launch in
crates/triton-runtime/examples/run_rms_norm.rs:52-66:

    prelude.rms_norm_f32(x, w, y, row_size, 1.0 / row_size, eps, rows)
"""
from __future__ import annotations

import torch

from ._lib import lib


def _make(name, nargs):
    def fn(*args, stream=None):
        if len(args) == nargs - 1:  # stream omitted
            st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
            return lib().call(name, *args, st)
        return lib().call(name, *args)
    fn.__name__ = name
    fn.__doc__ = f"C ABI `{name}`; see include/b200_kernels.h for the argument list."
    return fn


def __getattr__(name):
    protos = lib().protos
    if name in protos:
        ret, args = protos[name]
        if args and args[-1][0] == "b200k_stream":
            f = _make(name, len(args))
        else:
            def f(*a, _n=name):
                return lib().call(_n, *a)
        globals()[name] = f
        return f
    raise AttributeError(name)


# ---- conveniences for contiguous tensors (fill in the stride arguments) -----------
def gptq_gemm(a, qweight, scales, qzeros, group_size, out=None):
    """w4a16_gptq_gemm_f16 (or the _sym edition when qzeros is None) on contiguous tensors."""
    m, k = a.shape
    n = qweight.shape[1]
    c = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=a.device)
    if qzeros is None:
        __getattr__("w4a16_gptq_gemm_sym_f16")(a, qweight, scales, c, m, n, k, group_size, a.stride(0), a.stride(1),
                                               qweight.stride(0), qweight.stride(1), scales.stride(0),
                                               scales.stride(1), c.stride(0), c.stride(1))
    else:
        __getattr__("w4a16_gptq_gemm_f16")(a, qweight, scales, qzeros, c, m, n, k, group_size, a.stride(0),
                                           a.stride(1), qweight.stride(0), qweight.stride(1), scales.stride(0),
                                           scales.stride(1), qzeros.stride(0), qzeros.stride(1), c.stride(0),
                                           c.stride(1))
    return c


def awq_gemm(a, qweight, scales, qzeros, group_size, out=None):
    """awq_gemm_int4_f16 on contiguous tensors."""
    m, k = a.shape
    n = qweight.shape[1] * 8
    c = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=a.device)
    __getattr__("awq_gemm_int4_f16")(a, qweight, scales, qzeros, c, m, n, k, group_size, a.stride(0), a.stride(1),
                                     qweight.stride(0), qweight.stride(1), scales.stride(0), scales.stride(1),
                                     qzeros.stride(0), qzeros.stride(1), c.stride(0), c.stride(1))
    return c

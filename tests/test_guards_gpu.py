"""Failure paths that return a status instead of faulting: cache positions and lengths outside the cache, and an
all-reduce whose peer never arrives.  Nothing here hangs or faults the GPU: the waits are bounded and the bad indices
are skipped or clamped."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _status(pkg):
    v = ctypes.c_int(-1)
    pkg.lib().call("b200k_device_status", ctypes.addressof(v), torch.cuda.current_stream().cuda_stream)
    return v.value


def _clear(pkg):
    pkg.lib().call("b200k_device_clear_status", torch.cuda.current_stream().cuda_stream)
    assert _status(pkg) == 0


def test_append_position_outside_the_cache_is_skipped_and_reported(pkg, P, oracle):
    g = torch.Generator(device=DEV).manual_seed(1)
    b, hq, hkv, d, ml = 4, 8, 2, 128, 16
    qkv = torch.randn((b, (hq + 2 * hkv) * d), device=DEV, generator=g).half()
    cos, sin = (torch.from_numpy(x).to(DEV) for x in oracle.rope_tables(ml, d, 10000.0))
    kc = torch.randn((b, hkv, ml, d), device=DEV, generator=g).half()
    vc = torch.randn((b, hkv, ml, d), device=DEV, generator=g).half()
    kc0, vc0 = kc.clone(), vc.clone()
    q = torch.empty((b, hq, d), dtype=torch.float16, device=DEV)
    _clear(pkg)
    pos = torch.tensor([ml, -1, 3, 2 ** 30], dtype=torch.int32, device=DEV)       # one valid row among three bad ones
    P.rope_kv_append_hm_f16(qkv, cos, sin, pos, q, kc, vc, hq, hkv, d, ml, b)
    torch.cuda.synchronize()
    assert _status(pkg) & 4
    for row in (0, 1, 3):
        assert torch.equal(kc[row], kc0[row]) and torch.equal(vc[row], vc0[row])
    assert not torch.equal(kc[2, :, 3], kc0[2, :, 3]) and torch.equal(vc[2, :, 3], qkv[2, (hq + hkv) * d:].view(hkv, d))
    kc[2, :, 3], vc[2, :, 3] = kc0[2, :, 3], vc0[2, :, 3]
    assert torch.equal(kc, kc0) and torch.equal(vc, vc0)          # nothing else was touched
    # the plain append entry point guards the same way
    _clear(pkg)
    nk = torch.randn((b, hkv, d), device=DEV, generator=g).half()
    P.kv_cache_append_hm_f16(nk, nk, kc, vc, pos, hkv, d, ml, b)
    torch.cuda.synchronize()
    assert _status(pkg) & 4 and torch.equal(kc[0], kc0[0]) and torch.equal(kc[2, :, 3], nk[2])
    _clear(pkg)


def test_attention_length_beyond_the_cache_is_clamped_and_reported(pkg, P):
    g = torch.Generator(device=DEV).manual_seed(2)
    b, hq, hkv, d, ml = 3, 32, 8, 128, 700
    q = torch.randn((b, hq, d), device=DEV, generator=g).half()
    kc = torch.randn((b, hkv, ml, d), device=DEV, generator=g).half()
    vc = torch.randn((b, hkv, ml, d), device=DEV, generator=g).half()
    scale = 1.0 / float(np.sqrt(d))
    run = lambda lens, out: P.batched_decode_attention_hm_f16(q, kc, vc, lens, out, b, hq, hkv, d, ml, scale)
    good = torch.tensor([ml, 37, 512], dtype=torch.int32, device=DEV)
    want = torch.empty_like(q)
    _clear(pkg)
    run(good, want)
    torch.cuda.synchronize()
    assert _status(pkg) == 0
    bad = torch.tensor([ml + 1, 37, 2 ** 30], dtype=torch.int32, device=DEV)
    got = torch.full_like(q, float("nan"))
    run(bad, got)
    torch.cuda.synchronize()
    assert _status(pkg) & 4
    full = torch.tensor([ml, 37, ml], dtype=torch.int32, device=DEV)
    ref = torch.empty_like(q)
    run(full, ref)
    assert torch.equal(got, ref)                 # clamped to the cache, every row written
    again = torch.empty_like(q)
    run(good, again)                             # the arrival counters were left at zero: the next call is unaffected
    assert torch.equal(again, want)
    _clear(pkg)


def test_allreduce_whose_peer_never_arrives_gives_up_and_reports(pkg):
    """A world of two in ONE process: the second 'rank' is just a buffer that nobody ever flags.  With a wait of about
    a millisecond the kernel gives up, sets the status word and leaves the output alone; the context stays usable."""
    L = pkg.lib()
    st = torch.cuda.current_stream().cuda_stream
    n = 4096
    h = [ctypes.c_void_p(), ctypes.c_void_p()]
    for r in range(2):
        L.call("b200k_comm_create", r, 2, n * 2, ctypes.addressof(h[r]))
    buf = [ctypes.c_void_p(), ctypes.c_void_p()]
    for r in range(2):
        L.call("b200k_comm_buffer", h[r].value, ctypes.addressof(buf[r]))
    L.call("b200k_comm_set_peer_pointer", h[0].value, 1, buf[1].value)       # rank 0 sees "rank 1"; rank 1 never runs
    L.call("b200k_comm_set_timeout_cycles", h[0].value, 2_000_000)           # ~1 ms of SM clock
    x = torch.randn(n, device=DEV).half()
    out = torch.full((n,), 7.0, dtype=torch.float16, device=DEV)
    L.call("b200k_comm_allreduce_f16", h[0].value, 0, x, out, n, st)
    torch.cuda.synchronize()
    v = ctypes.c_int(-1)
    L.call("b200k_comm_status", h[0].value, ctypes.addressof(v), st)
    assert v.value == 1
    assert bool((out == 7.0).all())              # the reduce was skipped
    # the give-up left the buffers consistent: once the peer does flag (here: rank 1's kernel finally runs, with
    # rank 0 as its peer), later rounds complete
    L.call("b200k_comm_clear_status", h[0].value, st)
    # a healthy world of one on the same GPU still works, and so does an ordinary kernel
    solo = ctypes.c_void_p()
    L.call("b200k_comm_create", 0, 1, n * 2, ctypes.addressof(solo))
    blob = ctypes.create_string_buffer(64)
    L.call("b200k_comm_ipc_handle", solo.value, ctypes.addressof(blob))
    L.call("b200k_comm_open_peers", solo.value, ctypes.addressof(blob))
    out2 = torch.empty_like(x)
    L.call("b200k_comm_allreduce_f16", solo.value, 0, x, out2, n, st)
    torch.cuda.synchronize()
    L.call("b200k_comm_status", solo.value, ctypes.addressof(v), st)
    assert v.value == 0 and torch.equal(out2, x)
    y = torch.empty_like(x)
    pkg.prelude.residual_add_f16(x, x, y, n)
    assert torch.equal(y, x + x)
    for c in (h[0], h[1], solo):
        L.raw("b200k_comm_destroy")(c.value)

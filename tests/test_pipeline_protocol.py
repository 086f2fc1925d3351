"""Host-side model of the tensor-core GEMM's barrier protocol (three rings, NG dequant groups, one or two
MMA issuers that take the K blocks alternately), run for the exact ring depths the library would launch with.  A ring-depth combination that
can deadlock shows up here, on the CPU, as agents left waiting."""
import ctypes

import pytest


def simulate(NG, SD, SA, R, nkb, NMMA=1):
    done = {}

    def completed(b):
        return done.get(b, 0)

    def wprod():
        for i in range(nkb):
            if i >= R:
                yield ("wait", ("RAWE", i % R), i // R - 1)
            yield ("arrive", ("RAWF", i % R))

    def aprod():
        for i in range(nkb):
            if i >= SA:
                yield ("wait", ("ACTE", i % SA), i // SA - 1)
            yield ("arrive", ("ACTF", i % SA))

    def mma(w):
        for i in range(w, nkb, NMMA):
            yield ("wait", ("DQF", i % SD), i // SD)
            yield ("arrive", ("DQE", i % SD))

    def group(g):
        old = ((g - SD) % NG + NG) % NG
        for i in range(g, nkb, NG):
            yield ("wait", ("RAWF", i % R), i // R)
            yield ("arrive", ("RAWE", i % R))
            if i >= SD:
                yield ("wait", ("DQE", i % SD), i // SD - 1)
                assert old == i - SD
                yield ("arrive", ("ACTE", old % SA))      # block i - SD retired: its activation slot is free
                old += NG
            yield ("wait", ("ACTF", i % SA), i // SA)      # published only once the activation tile has landed
            yield ("arrive", ("DQF", i % SD))

    agents = [wprod(), aprod()] + [mma(w) for w in range(NMMA)] + [group(g) for g in range(NG)]
    pending = [next(a, None) for a in agents]
    progress = True
    while progress:
        progress = False
        for k, a in enumerate(agents):
            while pending[k] is not None:
                op = pending[k]
                if op[0] == "wait":
                    if completed(op[1]) <= op[2]:
                        break
                else:
                    done[op[1]] = completed(op[1]) + 1
                pending[k] = next(a, None)
                progress = True
    return [p for p in pending if p is not None]


def test_model_detects_a_known_bad_configuration():
    assert simulate(4, 5, 3, 10, 64)            # activation ring shallower than the operand ring: stuck at the tail
    assert not simulate(4, 5, 5, 13, 64)


@pytest.mark.parametrize("awq", [0, 1])
@pytest.mark.parametrize("m", [2, 16, 17, 33, 64, 100, 128, 300, 1024, 4096])
@pytest.mark.parametrize("k,n", [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096), (256, 128), (64, 64)])
def test_launch_plans_cannot_deadlock(pkg, m, k, n, awq):
    plan = (ctypes.c_int * 10)()
    pkg.lib().call("b200k_gemm_tc_plan", m, n, k, 64 if k == 64 else 128, awq, ctypes.addressof(plan))
    tt, ng, sd, sa, r, ksplit, kb_per_split, tiles, nmma, in_tmem = list(plan)
    assert tt in (16, 32, 64, 128, 256) and ng in (2, 4) and 1 <= ksplit <= 8
    assert sd >= ng and sa >= sd and r >= 2 and nmma in (1, 2) and in_tmem in (0, 1)
    if in_tmem:       # tensor memory: 256 columns per CTA when two CTAs share an SM, 512 otherwise
        assert max(32, nmma * tt) + 32 * sd <= (256 if tt <= 64 else 512)
    for nkb in {kb_per_split, max(1, (k // 64) - kb_per_split * (ksplit - 1)), 1, 2, 3, 7}:
        assert not simulate(ng, sd, sa, r, nkb, nmma), (plan[:], nkb)


def _plan(pkg, m, n, k, awq=0, group=128):
    plan = (ctypes.c_int * 10)()
    pkg.lib().call("b200k_gemm_tc_plan", m, n, k, group, awq, ctypes.addressof(plan))
    names = ("tt", "ng", "sd", "sa", "r", "ksplit", "steps", "tiles", "nmma", "flags")
    return dict(zip(names, plan))


def test_launch_plans_fill_whole_waves(pkg):
    """Above 64 tokens form and K split are planned together: the grids of the Llama-3-8B projections stay within the
    resident slots of 148 SMs (two CTAs per SM in the two-group forms, one in the four-group form) wherever one wave can
    hold them, and a grid that already fills the machine is not split."""
    sms = 148
    for awq in (0, 1):
        for m, n, k in [(128, 6144, 4096), (128, 4096, 4096), (128, 28672, 4096), (128, 4096, 14336),
                        (1024, 4096, 4096), (1024, 4096, 14336), (512, 6144, 4096)]:
            p = _plan(pkg, m, n, k, awq)
            ctas = p["tiles"] * p["ksplit"]
            slots = sms * (2 if p["ng"] == 2 else 1)
            assert ctas <= slots, (m, n, k, awq, p)
    assert _plan(pkg, 128, 28672, 4096)["ng"] == 2          # 224 tiles: one wave as two CTAs per SM, two waves otherwise
    assert _plan(pkg, 1024, 4096, 4096)["ksplit"] == 1      # 128 tiles of 256 tokens: one wave, nothing to split
    assert _plan(pkg, 1024, 6144, 4096)["ksplit"] == 1      # 192 tiles fill the machine


def test_pipeline_steps_of_128_k_where_tensor_memory_allows(pkg):
    """GPTQ layouts with group 128: token tiles up to 64 and the paired 128-token form take steps of 128 k (K / 128 steps
    per CTA and split); group 64, AWQ layouts and 256-token tiles keep 64-k steps."""
    assert _plan(pkg, 64, 4096, 4096)["steps"] * _plan(pkg, 64, 4096, 4096)["ksplit"] == 4096 // 128
    assert _plan(pkg, 128, 28672, 4096)["steps"] == 4096 // 128
    assert _plan(pkg, 64, 4096, 4096, group=64)["steps"] * _plan(pkg, 64, 4096, 4096, group=64)["ksplit"] == 4096 // 64
    assert _plan(pkg, 64, 4096, 4096, awq=1)["steps"] * _plan(pkg, 64, 4096, 4096, awq=1)["ksplit"] == 4096 // 64
    assert _plan(pkg, 1024, 4096, 4096)["steps"] == 4096 // 64
    for m, n, k in [(16, 4096, 4096), (64, 28672, 4096), (128, 4096, 14336)]:
        p = _plan(pkg, m, n, k)
        assert p["sd"] == 2 and p["sd"] >= p["ng"]           # two sub-tiles x ring of two beside the accumulators: 256 TMEM columns
        assert max(32, p["nmma"] * p["tt"]) + 2 * 32 * p["sd"] <= 256

"""Decode attention through the C ABI against the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import assert_close, golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def test_golden_attention(P):
    g = golden("attention_hm")
    b, hq, d = g["q"].shape
    hkv, ml = g["k"].shape[1], g["k"].shape[2]
    out = torch.empty((b, hq, d), dtype=torch.float16, device=DEV)
    P.batched_decode_attention_hm_f16(t(g["q"]), t(g["k"]), t(g["v"]), t(g["lens"]), out, b, hq, hkv, d, ml,
                                      1.0 / np.sqrt(d))
    assert_close(out.float().cpu().numpy(), g["out"])


@pytest.mark.parametrize("b,hq,hkv,ml,lens", [
    (4, 32, 8, 1500, [1, 511, 513, 1500]),
    (2, 8, 8, 300, [64, 300]),            # no grouping
    (3, 16, 2, 2100, [2100, 1024, 1025]), # group of 8
    (2, 4, 2, 96, [0, 96]),               # an empty sequence -> zero row
])
def test_batched_hm_ragged_with_poisoned_tail(P, oracle, b, hq, hkv, ml, lens):
    rng = np.random.default_rng(sum(lens))
    d = 128
    q = rng.standard_normal((b, hq, d)).astype(np.float16)
    k = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
    v = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
    lens = np.array(lens, dtype=np.int32)
    for i in range(b):                       # positions >= len must never be read
        k[i, :, lens[i]:] = np.nan
        v[i, :, lens[i]:] = np.nan
    out = torch.empty((b, hq, d), dtype=torch.float16, device=DEV)
    args = (t(q), t(k), t(v), t(lens), out, b, hq, hkv, d, ml, 1.0 / np.sqrt(d))
    P.batched_decode_attention_hm_f16(*args)
    got = out.float().cpu().numpy()
    for i in range(b):
        if lens[i] == 0:
            assert (got[i] == 0).all()
        else:
            ref = oracle.decode_attention_hm(q[i], k[i], v[i], int(lens[i]), 1.0 / np.sqrt(d))
            assert_close(got[i], ref, what=f"seq {i} len {lens[i]}")
    out2 = torch.empty_like(out)
    P.batched_decode_attention_hm_f16(*args[:4], out2, *args[5:])
    assert torch.equal(out, out2), "two runs differ"


def test_batched_hm_oracle_c_mid_size(P, oracle_c):
    # a size numpy would crawl through: checked with the C oracle
    rng = np.random.default_rng(77)
    b, hq, hkv, d, ml = 8, 32, 8, 128, 4096
    q = rng.standard_normal((b, hq, d)).astype(np.float16)
    k = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
    v = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
    lens = rng.integers(512, ml + 1, b).astype(np.int32)
    out = torch.empty((b, hq, d), dtype=torch.float16, device=DEV)
    P.batched_decode_attention_hm_f16(t(q), t(k), t(v), t(lens), out, b, hq, hkv, d, ml, 1.0 / np.sqrt(d))
    ref = np.zeros((b, hq, d), np.float32)
    q32 = np.ascontiguousarray(q.astype(np.float32))
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    oracle_c.oc_batched_decode_attention_hm(p(q32), p(k), p(v), p(lens), p(ref), b, hq, hkv, d, ml,
                                            ctypes.c_float(1.0 / np.sqrt(d)))
    assert_close(out.float().cpu().numpy(), ref)


def test_full_size_property_constant_values(P):
    # BASELINE config 1 extents. Size-independent property: if every V row of a sequence is
    # the same vector, the output is that vector for every head, whatever the scores are.
    b, hq, hkv, d, ml = 32, 32, 8, 128, 8192
    gen = torch.Generator(device=DEV).manual_seed(1)
    q = torch.randn((b, hq, d), device=DEV, generator=gen).half()
    k = torch.randn((b, hkv, ml, d), device=DEV, generator=gen).half()
    vrow = torch.randn((b, hkv, 1, d), device=DEV, generator=gen).half()
    v = vrow.expand(b, hkv, ml, d).contiguous()
    lens = torch.randint(512, ml + 1, (b,), device=DEV, dtype=torch.int32, generator=gen)
    out = torch.empty((b, hq, d), dtype=torch.float16, device=DEV)
    P.batched_decode_attention_hm_f16(q, k, v, lens, out, b, hq, hkv, d, ml, 1.0 / np.sqrt(d))
    want = vrow.expand(b, hkv, hq // hkv, d).reshape(b, hq, d).float()
    assert ((out.float() - want).abs() <= 1e-2 + 1e-2 * want.abs()).all()


def test_single_sequence_layouts(P, oracle):
    rng = np.random.default_rng(31)
    hq, hkv, d, L, cap = 32, 8, 128, 777, 800
    q = rng.standard_normal((hq, d)).astype(np.float16)
    ks = rng.standard_normal((cap, hkv, d)).astype(np.float16)
    vs = rng.standard_normal((cap, hkv, d)).astype(np.float16)
    ks[L:] = np.nan
    vs[L:] = np.nan
    scale = 1.0 / np.sqrt(d)
    ref = oracle.decode_attention(q, ks, vs, hkv, L, scale)
    out = torch.empty((hq, d), dtype=torch.float16, device=DEV)
    P.decode_attention_f16(t(q), t(ks), t(vs), out, hq, hkv, d, L, scale)
    assert_close(out.float().cpu().numpy(), ref, what="seq-major")
    khm, vhm = ks.transpose(1, 0, 2).copy(), vs.transpose(1, 0, 2).copy()
    P.decode_attention_hm_f16(t(q), t(khm), t(vhm), out, hq, hkv, d, cap, L, scale)
    assert_close(out.float().cpu().numpy(), ref, what="head-major")
    # f32 editions
    o32 = torch.empty((hq, d), device=DEV)
    P.decode_attention_f32(t(q.astype(np.float32)), t(ks.astype(np.float32)), t(vs.astype(np.float32)), o32, hq, hkv,
                           d, L, scale)
    assert_close(o32.cpu().numpy(), ref, 1e-4, 1e-5, what="seq-major f32")
    P.decode_attention_hm_f32(t(q.astype(np.float32)), t(khm.astype(np.float32)), t(vhm.astype(np.float32)), o32, hq,
                              hkv, d, cap, L, scale)
    assert_close(o32.cpu().numpy(), ref, 1e-4, 1e-5, what="head-major f32")
    # head_dim 64 takes the generic family
    q64 = q[:, :64].copy()
    k64, v64 = ks[:L, :, :64].copy(), vs[:L, :, :64].copy()
    o64 = torch.empty((hq, 64), dtype=torch.float16, device=DEV)
    P.decode_attention_f16(t(q64), t(k64), t(v64), o64, hq, hkv, 64, L, 0.125)
    assert_close(o64.float().cpu().numpy(), oracle.decode_attention(q64, k64, v64, hkv, L, 0.125), what="d64")


def test_paged(P, oracle):
    rng = np.random.default_rng(41)
    hq, hkv, d, bs, nblk, L = 16, 4, 128, 16, 40, 16 * 23
    q = rng.standard_normal((hq, d)).astype(np.float16)
    kp = rng.standard_normal((nblk, bs, hkv, d)).astype(np.float16)
    vp = rng.standard_normal((nblk, bs, hkv, d)).astype(np.float16)
    table = rng.permutation(nblk)[: L // bs].astype(np.int32)
    out = torch.empty((hq, d), dtype=torch.float16, device=DEV)
    P.paged_decode_attention_f16(t(q), t(kp), t(vp), t(table), out, hq, hkv, d, L, bs, 1 / np.sqrt(d))
    assert_close(out.float().cpu().numpy(), oracle.paged_decode_attention(q, kp, vp, table, L, bs, 1 / np.sqrt(d)))


def test_f32_batched_and_split_phases(P, oracle):
    rng = np.random.default_rng(51)
    b, hq, hkv, d, S, L = 3, 8, 2, 64, 200, 192
    q = rng.standard_normal((b, hq, d)).astype(np.float32)
    k = rng.standard_normal((b, S, hkv, d)).astype(np.float32)
    v = rng.standard_normal((b, S, hkv, d)).astype(np.float32)
    scale = 0.125
    out = torch.empty((b, hq, d), device=DEV)
    P.batched_decode_attention_f32(t(q), t(k), t(v), out, b, hq, hkv, d, S, L, scale)
    ref = oracle.batched_decode_attention(q, k, v, L, scale)
    assert_close(out.cpu().numpy(), ref, 1e-4, 1e-5)
    splits, bkv = 3, 32
    pa = torch.empty((b, hq, splits, d), device=DEV)
    pm = torch.empty((b, hq, splits), device=DEV)
    ps = torch.empty((b, hq, splits), device=DEV)
    P.batched_flash_decode_attn_phase1_f32(t(q), t(k), t(v), pa, pm, ps, b, hq, hkv, d, S, L, splits, scale, bkv)
    for i in range(b):
        ra, rm, rs = oracle.flash_decode_phase1(q[i], k[i], v[i], hkv, L, splits, scale, bkv)
        # the partials are un-normalised against each split's own max: compare after the merge
        assert_close((pa[i].cpu().numpy() * np.exp(pm[i].cpu().numpy())[..., None]),
                     ra * np.exp(rm)[..., None], 1e-3, 1e-4)
    o2 = torch.empty((b, hq, d), device=DEV)
    P.flash_decode_attn_phase2_f32(pa, pm, ps, o2, b * hq, d, splits)
    assert_close(o2.cpu().numpy(), ref, 1e-4, 1e-5)
    # single-sequence phase 1 + the oracle's phase 2
    P.flash_decode_attn_phase1_f32(t(q[0]), t(k[0]), t(v[0]), pa[0], pm[0], ps[0], hq, hkv, d, L, splits, scale, bkv)
    comb = oracle.flash_decode_phase2(pa[0].cpu().numpy(), pm[0].cpu().numpy(), ps[0].cpu().numpy())
    assert_close(comb, ref[0], 1e-4, 1e-5)


def _unified_case(rng, q_lens, seq_lens, hq, hkv, d, bs):
    nseq = len(q_lens)
    qsl = np.zeros(nseq + 1, dtype=np.int32)
    qsl[1:] = np.cumsum(q_lens)
    blocks_per_seq = max(-(-int(s) // bs) for s in seq_lens)
    nblocks = nseq * blocks_per_seq + 3
    table = rng.permutation(nblocks)[:nseq * blocks_per_seq].reshape(nseq, blocks_per_seq).astype(np.int32)
    q = rng.standard_normal((int(qsl[-1]), hq, d)).astype(np.float32)
    kp = rng.standard_normal((nblocks, bs, hkv, d)).astype(np.float32)
    vp = rng.standard_normal((nblocks, bs, hkv, d)).astype(np.float32)
    return q, kp, vp, table, np.asarray(seq_lens, dtype=np.int32), qsl, blocks_per_seq


@pytest.mark.parametrize("q_lens,seq_lens,hq,hkv,d,bs", [
    ([1, 1, 1], [17, 64, 5], 8, 2, 128, 16),            # pure decode
    ([7, 12], [7, 12], 4, 4, 64, 8),                    # pure prefill (context 0): the standard causal mask
    ([1, 9, 3, 1], [40, 9, 30, 1], 8, 2, 128, 16),      # mixed batch, one sequence of a single token
    ([5], [21], 2, 1, 96, 4),                           # head_dim not a power of two
])
def test_unified_attention_vs_oracle(P, oracle, q_lens, seq_lens, hq, hkv, d, bs):
    rng = np.random.default_rng(sum(seq_lens) + d)
    q, kp, vp, table, sl, qsl, bps = _unified_case(rng, q_lens, seq_lens, hq, hkv, d, bs)
    scale = 1.0 / np.sqrt(d)
    ref = oracle.unified_attention(q, kp, vp, table, sl, qsl, hkv, bs, scale)
    out = torch.full(q.shape, float("nan"), device=DEV)
    P.unified_attention_f32(t(q), t(kp), t(vp), out, t(table), t(sl), t(qsl), hq, hkv, d, bs, bps, scale, len(q_lens),
                            torch.cuda.current_stream().cuda_stream)
    assert_close(out.cpu().numpy(), ref, 1e-4, 1e-5, "unified attention")



@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("b,hq,hkv,q_len,kv_len,d,off", [
    (2, 8, 2, 64, 64, 128, 0),        # plain causal prefill, the reference's tile-aligned case
    (1, 4, 4, 37, 100, 64, 63),       # chunked prefill: 63 cached positions, ragged lengths
    (1, 2, 1, 5, 3, 96, 0),           # queries past the end of the KV stream see all of it; head_dim not a power of two
    (3, 4, 2, 1, 9, 128, 8),          # a single query row per sequence (decode through the prefill entry point)
])
def test_flash_attn_full_vs_oracle(P, oracle, dtype, b, hq, hkv, q_len, kv_len, d, off):
    rng = np.random.default_rng(q_len * 7 + kv_len)
    np_t, th_t = (np.float32, torch.float32) if dtype == "f32" else (np.float16, torch.float16)
    q = rng.standard_normal((b, hq, q_len, d)).astype(np_t)
    k = rng.standard_normal((b, hkv, kv_len, d)).astype(np_t)
    v = rng.standard_normal((b, hkv, kv_len, d)).astype(np_t)
    scale = 1.0 / np.sqrt(d)
    ref = oracle.flash_attn_full(q, k, v, off, scale)
    out = torch.full(q.shape, float("nan"), device=DEV, dtype=th_t)
    fn = P.flash_attn_full_f32 if dtype == "f32" else P.flash_attn_full_f16
    fn(t(q), t(k), t(v), out, b, hq, hkv, q_len, kv_len, d, off, scale, torch.cuda.current_stream().cuda_stream)
    if dtype == "f32":
        assert_close(out.cpu().numpy(), ref, 1e-4, 1e-5, "prefill attention f32")
    else:
        assert_close(out.float().cpu().numpy(), ref, 1e-2, 1e-2, "prefill attention f16")


@pytest.mark.parametrize("b,hq,hkv,q_len,kv_len,off", [
    (1, 4, 2, 300, 300, 0),           # three query tiles, three KV tiles, ragged last tile of both
    (2, 8, 2, 200, 500, 300),         # chunked prefill over 300 cached positions
    (1, 2, 2, 260, 150, 0),           # queries past the end of the KV stream
    (1, 8, 1, 128, 128, 0),           # exactly one tile; GQA group of 8
    (2, 4, 4, 129, 1, 0),             # a single KV position
    (1, 2, 1, 640, 640, 0),           # five tiles: both ring slots wrap twice; the last pair of query tiles is half empty
    (1, 2, 2, 300, 1000, 700),        # chunked prefill: the queries start at position 700 of a longer KV stream
    (1, 32, 8, 2048, 2048, 0),        # one 2048-token sequence of the Llama-3-8B head layout (the timed size)
])
def test_flash_attn_full_f16_head_dim_128_tensor_core_path(P, oracle, b, hq, hkv, q_len, kv_len, off):
    """head_dim 128 in fp16 runs on the tcgen05 kernel (128 x 128 tiles): tile boundaries, the causal diagonal inside a
    tile, KV streams shorter and longer than the queries, and outputs beyond q_len untouched."""
    d = 128
    rng = np.random.default_rng(q_len * 3 + kv_len)
    q = rng.standard_normal((b, hq, q_len, d)).astype(np.float16)
    k = rng.standard_normal((b, hkv, kv_len, d)).astype(np.float16)
    v = rng.standard_normal((b, hkv, kv_len, d)).astype(np.float16)
    scale = 1.0 / np.sqrt(d)
    ref = oracle.flash_attn_full(q, k, v, off, scale)
    out = torch.full(q.shape, float("nan"), device=DEV, dtype=torch.float16)
    st = torch.cuda.current_stream().cuda_stream
    P.flash_attn_full_f16(t(q), t(k), t(v), out, b, hq, hkv, q_len, kv_len, d, off, scale, st)
    assert_close(out.float().cpu().numpy(), ref, 1e-2, 1e-2, "prefill attention f16 (tensor core)")
    out2 = torch.empty_like(out)
    P.flash_attn_full_f16(t(q), t(k), t(v), out2, b, hq, hkv, q_len, kv_len, d, off, scale, st)
    assert torch.equal(out, out2), "two runs differ"


def test_flash_attn_full_rejects_bad_shapes(P, pkg):
    z = torch.zeros(16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    with pytest.raises(pkg.B200KError):
        P.flash_attn_full_f32(z, z, z, z, 1, 3, 2, 1, 1, 16, 0, 1.0, st)       # q heads not a multiple of kv heads
    with pytest.raises(pkg.B200KError):
        P.flash_attn_full_f32(z, z, z, z, 1, 2, 2, 1, 1, 512, 0, 1.0, st)      # head_dim too large
    P.flash_attn_full_f32(z, z, z, z, 0, 2, 2, 1, 1, 16, 0, 1.0, st)           # empty batch: nothing to do

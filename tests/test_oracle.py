"""Pins the CPU oracle: against the inputs, host formulas and tolerances of the
reference's own numeric checks (f32 glue), against hand-computable known answers for
the bit-exact nibble orders, against the committed golden vectors, and the numpy and C
editions against each other."""
import ctypes

import numpy as np
import pytest

from conftest import assert_close, assert_close_sum, golden


# ---- reference's e2e example inputs (crates/triton-runtime/examples/run_*.rs) ------
def test_rms_norm_matches_reference_example(oracle):
    # run_rms_norm.rs:23-37 inputs, :71-87 host formula and tolerance max(1e-4, 1e-4*|want|)
    rows, n, eps = 16, 1024, 1e-6
    x = np.sin(np.arange(rows * n, dtype=np.float32) * np.float32(0.01)).reshape(rows, n)
    w = (1.0 + np.arange(n, dtype=np.float32) * np.float32(0.001))
    got = oracle.rms_norm(x, w, eps)
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + eps) * w
    tol = np.maximum(1e-4, np.abs(want) * 1e-4)
    assert (np.abs(got - want) <= tol).all()


def test_fused_add_rms_norm_matches_reference_example(oracle):
    # run_fused_add_rms_norm.rs:21-34 inputs, :73-94 formula, tol max(2e-3, 5e-3*|want|), residual 1e-5
    rows, n, eps = 16, 1024, 1e-6
    i = np.arange(rows * n, dtype=np.float32)
    x = np.sin(i * np.float32(0.013)).reshape(rows, n)
    r = np.cos(i * np.float32(0.027)).reshape(rows, n)
    w = (1.0 + np.arange(n, dtype=np.float32) * np.float32(0.001))
    out, res = oracle.fused_add_rms_norm(x, r, w, eps)
    s = x.astype(np.float64) + r
    want = s / np.sqrt((s ** 2).mean(axis=1, keepdims=True) + eps) * w
    assert (np.abs(res - s) <= 1e-5).all()
    assert (np.abs(out - want) <= np.maximum(2e-3, np.abs(want) * 5e-3)).all()


def test_silu_mul_and_add_match_reference_example(oracle):
    # run_vec_add.rs:63-80 inputs (x = i, y = 2i, N = 4096), :125-150 formulas, tol max(1e-5, 1e-5*|want|)
    n = 4096
    x = np.arange(n, dtype=np.float32)
    y = (np.arange(n) * 2).astype(np.float32)
    assert (oracle.residual_add(x, y) == x + y).all()
    got = oracle.fused_silu_mul(x, y)
    want = x.astype(np.float64) / (1.0 + np.exp(-x.astype(np.float64))) * y
    assert (np.abs(got - want) <= np.maximum(1e-5, np.abs(want) * 1e-5)).all()


# ---- bit-exact nibble orders -------------------------------------------------------
def test_unpack_walking_nibbles(oracle):
    w = np.array([[0x76543210]], dtype=np.uint32).view(np.int32)
    # GPTQ qweight: nibble i of the word is row 8r+i (w4a16_gptq_gemm_typed.rs:167-173)
    assert oracle.unpack_gptq_qweight(w)[:, 0].tolist() == [0, 1, 2, 3, 4, 5, 6, 7]
    # GPTQ qzeros: column n at nibble n%8 (:155-162)
    assert oracle.unpack_rowpacked_straight(w)[0].tolist() == [0, 1, 2, 3, 4, 5, 6, 7]
    # AWQ: column n at nibble [0,4,1,5,2,6,3,7][n%8] (awq_gemm_int4_typed.rs:137-151)
    assert oracle.unpack_awq(w)[0].tolist() == [0, 4, 1, 5, 2, 6, 3, 7]
    top = np.array([[0xF0000000]], dtype=np.uint32).view(np.int32)   # sign bit set: shifts are logical
    assert oracle.unpack_gptq_qweight(top)[:, 0].tolist() == [0] * 7 + [15]
    assert oracle.unpack_awq(top)[0].tolist() == [0, 0, 0, 0, 0, 0, 0, 15]


def test_pack_unpack_roundtrip(oracle):
    rng = np.random.default_rng(1)
    nib = rng.integers(0, 16, (64, 40), dtype=np.int32)
    assert (oracle.unpack_gptq_qweight(oracle.pack_gptq_qweight(nib)) == nib).all()
    assert (oracle.unpack_awq(oracle.pack_awq(nib)) == nib).all()
    assert (oracle.unpack_rowpacked_straight(oracle.pack_rowpacked_straight(nib)) == nib).all()


def test_gptq_zero_offset_and_sym(oracle):
    # stored zero nibble 7 with the GEMM's +1 == symmetric zero-point 8
    rng = np.random.default_rng(2)
    nib = rng.integers(0, 16, (128, 16), dtype=np.int32)
    qw = oracle.pack_gptq_qweight(nib)
    sc = rng.uniform(0.002, 0.02, (1, 16)).astype(np.float16)
    qz7 = np.full((1, 2), 0x77777777, dtype=np.int32)
    a = rng.standard_normal((3, 128)).astype(np.float16)
    c1 = oracle.w4a16_gptq_gemm(a, qw, sc, qz7, 128, zero_offset=1)
    c2 = oracle.w4a16_gptq_gemm(a, qw, sc, None, 128)
    assert (c1 == c2).all()
    want = a.astype(np.float64) @ ((nib - 8) * sc.astype(np.float64))
    assert_close(c1, want, rtol=1e-5, atol=1e-5)
    # dequant kernels: column-major output, no +1 (ferrum_dequant_int4.rs:76,80-89)
    d = oracle.dequant_int4_to_fp16(qw, sc, qz7, 128)
    assert d.shape == (16, 128)
    assert (d.astype(np.float32) == ((nib - 7).T * sc.astype(np.float32).T).astype(np.float16).astype(np.float32)).all()
    ds = oracle.dequant_int4_sym_to_fp16(qw, sc, 128)
    assert (ds.astype(np.float32) == ((nib - 8).T * sc.astype(np.float32).T).astype(np.float16).astype(np.float32)).all()


# ---- attention variants agree with each other ---------------------------------------
def test_attention_layouts_and_split_combine(oracle):
    rng = np.random.default_rng(3)
    hq, hkv, d, L = 8, 2, 32, 96
    q = rng.standard_normal((hq, d)).astype(np.float32)
    k = rng.standard_normal((L, hkv, d)).astype(np.float32)
    v = rng.standard_normal((L, hkv, d)).astype(np.float32)
    scale = 1 / np.sqrt(d)
    ref = oracle.decode_attention(q, k, v, hkv, L, scale)
    hm = oracle.decode_attention_hm(q, k.transpose(1, 0, 2).copy(), v.transpose(1, 0, 2).copy(), L, scale)
    assert_close(hm, ref, rtol=1e-5, atol=1e-6)
    acc, mx, sm = oracle.flash_decode_phase1(q, k, v, hkv, L, 3, scale, 16)
    comb = oracle.flash_decode_phase2(acc, mx, sm)
    assert_close(comb, ref, rtol=1e-5, atol=1e-6)
    # paged: scatter the sequence into shuffled physical blocks
    bs = 16
    table = rng.permutation(10)[: L // bs].astype(np.int32)
    kp = np.zeros((10, bs, hkv, d), np.float32)
    vp = np.zeros_like(kp)
    for lb, pb in enumerate(table):
        kp[pb] = k[lb * bs:(lb + 1) * bs]
        vp[pb] = v[lb * bs:(lb + 1) * bs]
    pg = oracle.paged_decode_attention(q, kp, vp, table, L, bs, scale)
    assert_close(pg, ref, rtol=1e-5, atol=1e-6)
    # explicit double-precision softmax as an independent check
    grp = hq // hkv
    for h in range(hq):
        s = (k[:, h // grp].astype(np.float64) @ q[h]) * scale
        p = np.exp(s - s.max())
        want = (p / p.sum()) @ v[:, h // grp]
        assert_close(ref[h], want, rtol=1e-4, atol=1e-5)


def test_moe_routing_tiebreak_and_permutation(oracle):
    logits = np.array([[0.25, 0.25, 0.25, 0.25], [0.0, 2.0, 2.0, -1.0], [3.0, 0.0, 1.0, 2.0]], np.float32)
    ids, w = oracle.moe_route(logits, 2)
    assert ids.tolist() == [[0, 1], [1, 2], [0, 3]]
    assert np.allclose(w.sum(axis=1), 1.0)
    assert np.allclose(w[0], [0.5, 0.5])
    counts, offsets, sorted_pairs, inv = oracle.moe_permute(ids, 4)
    assert counts.tolist() == [2, 2, 1, 1]
    assert offsets.tolist() == [0, 2, 4, 5, 6]
    assert sorted_pairs.tolist() == [0, 4, 1, 2, 3, 5]      # expert-major, pair index ascending inside
    assert (sorted_pairs[inv] == np.arange(6)).all()


# ---- golden vectors --------------------------------------------------------------------
def test_golden_vectors_reproduce(oracle):
    g = golden("gptq_gemm")
    assert (oracle.unpack_gptq_qweight(g["qweight"]) == g["nib"]).all()
    assert (oracle.unpack_rowpacked_straight(g["qzeros"]) + 1 == g["zeros"]).all()
    assert_close(oracle.w4a16_gptq_gemm(g["a"], g["qweight"], g["scales"], g["qzeros"], 128), g["c"], 1e-6, 1e-6)
    assert_close(oracle.w4a16_gptq_gemm(g["a"], g["qweight"], g["scales"], None, 128), g["c_sym"], 1e-6, 1e-6)
    a = golden("awq_gemm")
    assert (oracle.unpack_awq(a["qweight"]) == a["nib"]).all()
    assert_close(oracle.awq_gemm_int4(a["a"], a["qweight"], a["scales"], a["qzeros"], 128), a["c"], 1e-6, 1e-6)
    t = golden("attention_hm")
    assert_close(oracle.batched_decode_attention_hm(t["q"], t["k"], t["v"], t["lens"], 1 / np.sqrt(128)), t["out"], 1e-6, 1e-6)
    m = golden("moe")
    ids, wts = oracle.moe_route(m["logits"], 2)
    assert (ids == m["ids"]).all() and (ids[3] == [0, 1]).all()
    c, off, sp, inv = oracle.moe_permute(ids, 4)
    assert (c == m["counts"]).all() and (sp == m["sorted_pairs"]).all() and (inv == m["inv"]).all()


# ---- numpy oracle vs C oracle ------------------------------------------------------------
def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_c_oracle_matches_numpy(oracle, oracle_c):
    g = golden("gptq_gemm")
    a32 = np.ascontiguousarray(g["a"].astype(np.float32))
    m, k = a32.shape
    n = g["qweight"].shape[1]
    c = np.zeros((m, n), np.float32)
    oracle_c.oc_gptq_gemm(_p(a32), _p(g["qweight"]), _p(g["scales"]), _p(g["qzeros"]), _p(c), m, n, k, 128, 1)
    assert_close(c, g["c"], 1e-5, 1e-5, "C gptq")
    oracle_c.oc_gptq_gemm(_p(a32), _p(g["qweight"]), _p(g["scales"]), None, _p(c), m, n, k, 128, 0)
    assert_close(c, g["c_sym"], 1e-5, 1e-5, "C gptq sym")
    w = golden("awq_gemm")
    oracle_c.oc_awq_gemm(_p(a32 * 0 + w["a"].astype(np.float32)), _p(w["qweight"]), _p(w["scales"]), _p(w["qzeros"]),
                         _p(c), m, n, k, 128)
    assert_close(c, w["c"], 1e-5, 1e-5, "C awq")
    t = golden("attention_hm")
    q32 = np.ascontiguousarray(t["q"].astype(np.float32))
    b, hq, d = q32.shape
    hkv, ml = t["k"].shape[1], t["k"].shape[2]
    out = np.zeros((b, hq, d), np.float32)
    oracle_c.oc_batched_decode_attention_hm(_p(q32), _p(t["k"]), _p(t["v"]), _p(t["lens"]), _p(out), b, hq, hkv, d,
                                            ml, ctypes.c_float(1 / np.sqrt(d)))
    assert_close(out, t["out"], 1e-4, 1e-5, "C attention")


def test_c_layer_matches_numpy_layer(oracle, oracle_c):
    rng = np.random.default_rng(7)
    B, H, hq, hkv, d, I, G, ml = 3, 256, 4, 2, 64, 384, 128, 24

    def gptq(k, n):
        return (oracle.pack_gptq_qweight(rng.integers(0, 16, (k, n), dtype=np.int32)),
                rng.uniform(0.002, 0.02, (k // G, n)).astype(np.float16),
                oracle.pack_rowpacked_straight(rng.integers(0, 16, (k // G, n), dtype=np.int32)))
    cos, sin = oracle.rope_tables(ml, d, 500000.0)
    p = dict(hq=hq, hkv=hkv, d=d, group=G, zero_offset=1, eps=1e-5, cos=cos, sin=sin,
             ln1=rng.uniform(0.5, 1.5, H).astype(np.float16), ln2=rng.uniform(0.5, 1.5, H).astype(np.float16),
             qkv=gptq(H, (hq + 2 * hkv) * d), o=gptq(hq * d, H), gate_up=gptq(H, 2 * I), down=gptq(I, H))
    hidden = rng.standard_normal((B, H)).astype(np.float16)
    kc = rng.standard_normal((B, hkv, ml, d)).astype(np.float16)
    vc = rng.standard_normal((B, hkv, ml, d)).astype(np.float16)
    pos = np.array([5, 0, 23], dtype=np.int32)
    kc2, vc2 = kc.copy(), vc.copy()
    st = {}
    ref = oracle.decode_layer(hidden, p, kc, vc, pos, stages=st)
    out = np.zeros((B, H), np.float32)
    names = ("n1", "qkv", "q", "att", "o", "h1", "n2", "gate_up", "act", "down")
    bufs = [np.zeros(st[n].size, np.float32) for n in names]
    stage_ptrs = (ctypes.c_void_p * 10)(*[b.ctypes.data for b in bufs])
    args = [_p(hidden), _p(out), B, H, hq, hkv, d, I, G, 1, ctypes.c_float(1e-5), _p(p["ln1"]), _p(p["ln2"])]
    for name in ("qkv", "o", "gate_up", "down"):
        args += [_p(x) for x in p[name]]
    args += [_p(cos), _p(sin), _p(pos), _p(kc2), _p(vc2), ml]
    oracle_c.oc_decode_layer_ex(*args, 1, stage_ptrs)
    # every intermediate of the two restatements agrees to an fp16 ulp or two; the closing residual add is a sum of
    # two fp16 tensors (h1 + down), so its tolerance is the sum of the summands' tolerances
    for n, b in zip(names, bufs):
        assert_close(b.reshape(st[n].shape), st[n], 5e-3, 5e-3, f"C layer stage {n}")   # half the product's tolerance
    assert_close_sum(out, ref, (st["h1"], st["down"]), 5e-3, 5e-3, "C layer")
    assert (kc2 == kc).all() and (vc2 == vc).all()
    # the non-faithful mode (fp32 weight product, norm of the rounded residual) is the numpy oracle's faithful=False
    ref0 = oracle.decode_layer(hidden, p, kc.copy(), vc.copy(), pos, faithful=False, stages=st)
    oracle_c.oc_decode_layer_ex(*args, 0, None)
    assert_close_sum(out, ref0, (st["h1"], st["down"]), 5e-3, 5e-3, "C layer, fp32 weight product")


def test_projection_helpers_compose(oracle):
    """The fused helpers equal the composition of the plain ones; the transposes invert each other."""
    rng = np.random.default_rng(11)
    tokens, heads, d, off = 5, 3, 8, 2
    x = rng.standard_normal((tokens, heads, d)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    cos, sin = oracle.rope_tables(off + tokens, d, 10000.0)
    assert np.array_equal(oracle.transpose_head_to_token(oracle.transpose_token_to_head(x)), x)
    pos = off + np.arange(tokens)
    ref = oracle.rope_full(oracle.rms_norm(x, w, 1e-6), cos, sin, pos).transpose(1, 0, 2)
    assert np.allclose(oracle.qk_norm_rope_transpose(x, w, cos, sin, off, 1e-6), ref, rtol=0, atol=0)
    # hand-checkable case: one token, one head, D = 2, angle with cos = 0.6, sin = 0.8
    out = oracle.rope_transpose(np.array([[[1.0, 2.0]]], np.float32), np.array([[0.6]], np.float32),
                                np.array([[0.8]], np.float32), 0)
    assert np.allclose(out, [[[1.0 * 0.6 - 2.0 * 0.8, 2.0 * 0.6 + 1.0 * 0.8]]])
    qkv = np.arange(2 * 3 * 2 * 4, dtype=np.float32).reshape(2, 3, 2, 4)
    q, k, v = oracle.split_qkv(qkv, 2, 4)
    assert q[1, 1, 0] == qkv[1, 0, 1, 0] and k[0, 1, 3] == qkv[0, 1, 1, 3] and v[1, 0, 2] == qkv[1, 2, 0, 2]


def test_unified_attention_decode_equals_paged_decode(oracle):
    """With one query token per sequence the unified oracle computes what the paged decode oracle computes; with
    context 0 it is plain causal attention."""
    rng = np.random.default_rng(5)
    hq, hkv, d, bs, n = 8, 2, 16, 4, 13
    nblocks = 6
    table = rng.permutation(nblocks)[:4].reshape(1, 4).astype(np.int32)
    q = rng.standard_normal((1, hq, d)).astype(np.float32)
    kp = rng.standard_normal((nblocks, bs, hkv, d)).astype(np.float32)
    vp = rng.standard_normal((nblocks, bs, hkv, d)).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    got = oracle.unified_attention(q, kp, vp, table, np.array([n], np.int32), np.array([0, 1], np.int32), hkv, bs, scale)[0]
    ref = oracle.paged_decode_attention(q[0], kp, vp, table[0], n, bs, scale)
    assert np.allclose(got, ref, rtol=1e-5, atol=1e-6)
    # prefill of 3 tokens, one head: token j attends to positions 0..j
    q3 = rng.standard_normal((3, 1, d)).astype(np.float32)
    out = oracle.unified_attention(q3, kp[:, :, :1], vp[:, :, :1], table, np.array([3], np.int32), np.array([0, 3], np.int32), 1, bs, scale)
    k = kp[table[0][0], :3, 0]
    v = vp[table[0][0], :3, 0]
    for j in range(3):
        sc = (k[:j + 1] @ q3[j, 0]) * scale
        p = np.exp(sc - sc.max())
        assert np.allclose(out[j, 0], (p[:, None] * v[:j + 1]).sum(0) / p.sum(), rtol=1e-5, atol=1e-6)


def test_flash_attn_full_matches_the_reference_mask_formulation(oracle):
    """The prefill oracle against a literal restatement of the reference's tile loop: additive -1e30 mask on every
    KV tile, online softmax with running max (`attention.rs:836-890`); and, with context = pos_offset, against the
    unified oracle on the same tokens."""
    rng = np.random.default_rng(11)
    b, hq, hkv, ql, kl, d, off = 2, 4, 2, 8, 16, 16, 8
    q = rng.standard_normal((b, hq, ql, d)).astype(np.float32)
    k = rng.standard_normal((b, hkv, kl, d)).astype(np.float32)
    v = rng.standard_normal((b, hkv, kl, d)).astype(np.float32)
    scale = np.float32(1.0 / np.sqrt(d))
    got = oracle.flash_attn_full(q, k, v, off, scale)
    bkv = 4
    for bi in range(b):
        for h in range(hq):
            kvh = h // (hq // hkv)
            m = np.full(ql, -1e30, np.float32); l = np.zeros(ql, np.float32); acc = np.zeros((ql, d), np.float32)
            for kb in range(kl // bkv):
                kt, vt = k[bi, kvh, kb * bkv:(kb + 1) * bkv], v[bi, kvh, kb * bkv:(kb + 1) * bkv]
                sc = (q[bi, h] @ kt.T) * scale
                mask = (np.arange(kb * bkv, (kb + 1) * bkv)[None, :] <= (np.arange(ql)[:, None] + off)).astype(np.float32)
                sc = sc + (mask - 1.0) * np.float32(1e30)
                m_new = np.maximum(m, sc.max(axis=1))
                alpha = np.exp(m - m_new)
                p = np.exp(sc - m_new[:, None])
                acc = acc * alpha[:, None] + p @ vt
                l = l * alpha + p.sum(axis=1)
                m = m_new
            assert np.allclose(got[bi, h], acc / l[:, None], rtol=1e-5, atol=1e-6)
    # the same tokens through the unified (paged) oracle: one block per sequence, query = the last q_len positions
    kp = np.ascontiguousarray(k.transpose(0, 2, 1, 3))          # [b, kl, hkv, d] = pool of b blocks of size kl
    vp = np.ascontiguousarray(v.transpose(0, 2, 1, 3))
    qt = np.ascontiguousarray(q.transpose(0, 2, 1, 3)).reshape(b * ql, hq, d)
    uni = oracle.unified_attention(qt, kp, vp, np.arange(b, dtype=np.int32).reshape(b, 1), np.full(b, off + ql, np.int32),
                                   np.arange(0, (b + 1) * ql, ql, dtype=np.int32), hkv, kl, scale)
    assert np.allclose(uni.reshape(b, ql, hq, d).transpose(0, 2, 1, 3), got, rtol=1e-5, atol=1e-6)


def test_softmax_reference_example_inputs(oracle):
    """Inputs, host formula and tolerance of the reference's own numeric check
    (crates/triton-runtime/examples/run_softmax.rs:20-21,31-33,62-86)."""
    rows, cols = 8, 1024
    i = np.arange(rows * cols)
    x = (((i % cols).astype(np.float32) - np.float32(512.0)) * np.float32(0.01) * (i // cols + 1).astype(np.float32)).reshape(rows, cols)
    got = oracle.softmax(x)
    for r in range(rows):          # the example's sequential fp32 host loop
        row_max = np.float32(-np.inf)
        for v in x[r]:
            row_max = max(row_max, v)
        exps = np.exp(x[r] - row_max, dtype=np.float32)
        s = np.float32(0.0)
        for e in exps:
            s = np.float32(s + e)
        want = exps / s
        assert (np.abs(got[r] - want) <= np.maximum(1e-5, np.abs(want) * 1e-4)).all()
        assert abs(float(got[r].sum()) - 1.0) <= 1e-4


def test_embedding_is_a_gather(oracle):
    table = np.arange(5 * 3, dtype=np.float32).reshape(5, 3)
    out = oracle.embedding_lookup(table, np.array([4, 0, 4, 2], np.int32))
    assert np.array_equal(out, table[[4, 0, 4, 2]])

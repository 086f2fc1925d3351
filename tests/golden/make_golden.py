"""Writes the committed golden vectors (tests/golden/*.npz) from the CPU oracle.

    python tests/golden/make_golden.py

Each file holds the seeded inputs and the fp32 oracle outputs of one small case.  The
reference itself has no runnable build and no numeric fixtures for these kernels, so
the vectors pin the oracle's behaviour (and, through it, the CUDA path) across changes;
they are not outputs of the reference.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent / "oracle"))
import oracle as o  # noqa: E402


def quant_case(rng, k, n, g, fmt):
    nib = rng.integers(0, 16, (k, n), dtype=np.int32)
    zer = rng.integers(0, 16, (k // g, n), dtype=np.int32)
    sc = rng.uniform(0.002, 0.02, (k // g, n)).astype(np.float16)
    if fmt == "gptq":
        return o.pack_gptq_qweight(nib), sc, o.pack_rowpacked_straight(zer)
    return o.pack_awq(nib), sc, o.pack_awq(zer)


def main():
    rng = np.random.default_rng(20240)
    # GPTQ / AWQ GEMM, M = 5 (ragged), K = 256, N = 72, G = 128
    for fmt in ("gptq", "awq"):
        qw, sc, qz = quant_case(rng, 256, 72, 128, fmt)
        a = rng.standard_normal((5, 256)).astype(np.float16)
        if fmt == "gptq":
            c = o.w4a16_gptq_gemm(a, qw, sc, qz, 128, zero_offset=1)
            c_sym = o.w4a16_gptq_gemm(a, qw, sc, None, 128)
            cf = o.w4a16_gptq_gemm(a, qw, sc, qz, 128, zero_offset=1, faithful=True)
            np.savez_compressed(HERE / "gptq_gemm.npz", a=a, qweight=qw, scales=sc, qzeros=qz, c=c, c_sym=c_sym,
                                c_faithful=cf, nib=o.unpack_gptq_qweight(qw),
                                zeros=o.unpack_rowpacked_straight(qz) + 1)
        else:
            c = o.awq_gemm_int4(a, qw, sc, qz, 128)
            np.savez_compressed(HERE / "awq_gemm.npz", a=a, qweight=qw, scales=sc, qzeros=qz, c=c,
                                nib=o.unpack_awq(qw), zeros=o.unpack_awq(qz))
    # batched head-major attention with ragged lengths (incl. 1 and a non-multiple of any tile)
    b, hq, hkv, d, ml = 2, 8, 2, 128, 136
    q = rng.standard_normal((b, hq, d)).astype(np.float16)
    k = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
    v = rng.standard_normal((b, hkv, ml, d)).astype(np.float16)
    lens = np.array([1, 131], dtype=np.int32)
    out = o.batched_decode_attention_hm(q, k, v, lens, 1.0 / np.sqrt(d))
    np.savez_compressed(HERE / "attention_hm.npz", q=q, k=k, v=v, lens=lens, out=out)
    # glue
    x = rng.standard_normal((6, 192)).astype(np.float16)
    r = rng.standard_normal((6, 192)).astype(np.float16)
    w = rng.uniform(0.5, 1.5, 192).astype(np.float16)
    y = o.rms_norm(x, w, 1e-5)
    fy, fr = o.fused_add_rms_norm(x, r, w, 1e-5)
    cos, sin = o.rope_tables(64, 128, 500000.0)
    xr = rng.standard_normal((4, 3, 128)).astype(np.float16)
    pos = np.array([0, 7, 63, 31], dtype=np.int32)
    np.savez_compressed(HERE / "glue.npz", x=x, r=r, w=w, rms=y, fused_out=fy, fused_res=fr,
                        add=o.residual_add(x, r), silu=o.fused_silu_mul(x, r),
                        silu_il=o.fused_silu_mul_interleaved(x, 96), cos=cos, sin=sin, xr=xr, pos=pos,
                        rope=o.rope_full(xr, cos, sin, pos))
    # MoE routing + permutation (bit-exact items) and a tiny fused MoE
    t, e, h, inter, g = 24, 4, 128, 128, 128
    logits = rng.standard_normal((t, e)).astype(np.float32)
    logits[3, :] = 0.25          # a full tie: lowest expert indices must win
    ids, wts = o.moe_route(logits, 2)
    counts, offsets, sorted_pairs, inv = o.moe_permute(ids, e)
    xm = rng.standard_normal((t, h)).astype(np.float16)
    w13q = np.stack([o.pack_gptq_qweight(rng.integers(0, 16, (h, 2 * inter), dtype=np.int32)) for _ in range(e)])
    w13s = rng.uniform(0.002, 0.02, (e, h // g, 2 * inter)).astype(np.float16)
    w2q = np.stack([o.pack_gptq_qweight(rng.integers(0, 16, (inter, h), dtype=np.int32)) for _ in range(e)])
    w2s = rng.uniform(0.002, 0.02, (e, inter // g, h)).astype(np.float16)
    out = o.fused_moe_gptq(xm, logits, w13q, w13s, w2q, w2s, 2, g)
    np.savez_compressed(HERE / "moe.npz", logits=logits, ids=ids, wts=wts, counts=counts, offsets=offsets,
                        sorted_pairs=sorted_pairs, inv=inv, x=xm, w13q=w13q, w13s=w13s, w2q=w2q, w2s=w2s, out=out)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()

"""CPU oracle for the LLM-decode kernel hot path (TEST INFRASTRUCTURE ONLY).

This module is a numpy restatement, in fp32, of the arithmetic the reference
kernels (sizzlecar/triton-rs, `triton-kernels` crate and the two int4 GEMM
examples of `triton-dsl`) define.  It is the checker for the CUDA path: only
the test-suite, the smoke check and the benchmark's CPU-baseline leg may import
it.  Nothing in the shipped package may call into it.

Parity status
-------------
* f32 glue (rms_norm, fused_add_rms_norm, silu_mul, add): pinned by the inputs,
  host formulas and tolerances of the reference's own numeric checks
  (`crates/triton-runtime/examples/run_rms_norm.rs:34-37,71-87`,
  `run_fused_add_rms_norm.rs:32-34,73-94`, `run_vec_add.rs:79-80,125-150`).
* int4 GEMM (GPTQ/AWQ), attention, RoPE, kv-cache append, fused MoE:
  **parity unpinned** -- the reference holds no numeric test, golden vector or
  runnable build of these kernels (its tests assert MLIR text only), so the
  oracle follows the kernel source line by line and nothing else.
* The masked attention kernels of the reference turn an i1 mask into f32 with a
  signed cast (`attention.rs:134-136`, `triton-ir/src/module.rs:722-723`), which
  gives -1.0 for "valid".  The oracle implements the documented intent (masked
  positions are excluded, `attention.rs:90-92,131-133`), not that defect.

Conventions: every function takes numpy arrays; fp16 tensors are given as
np.float16 and are widened to fp32 before any arithmetic; results are fp32
unless the name says otherwise (callers round to fp16 when they compare with a
fp16 kernel output).  Integer division and remainder follow the reference's
signed semantics, which coincide with numpy's on the non-negative indices used.
"""
from __future__ import annotations

import numpy as np

# AWQ nibble order: column j of a packed group of 8 sits at nibble AWQ_ORDER[j]
# (`crates/triton-dsl/examples/awq_gemm_int4_typed.rs:137-151`).
AWQ_ORDER = np.array([0, 4, 1, 5, 2, 6, 3, 7], dtype=np.int64)


# ---------------------------------------------------------------------------
# int4 pack / unpack  (bit-exact items)
# ---------------------------------------------------------------------------
def unpack_gptq_qweight(qweight: np.ndarray) -> np.ndarray:
    """[K/8, N] int32 -> [K, N] int32 in 0..15; nibble i of a word is row 8*r+i.

    `w4a16_gptq_gemm_typed.rs:167-173,246-247` (shift = (k % 8) * 4, logical
    shift right, mask 0xF); same order as `ferrum_dequant_int4.rs:95-138`.
    """
    q = qweight.astype(np.int64) & 0xFFFFFFFF
    k8, n = q.shape
    shifts = (np.arange(8, dtype=np.int64) * 4)[None, :, None]
    out = (q[:, None, :] >> shifts) & 0xF
    return out.reshape(k8 * 8, n).astype(np.int32)


def pack_gptq_qweight(nib: np.ndarray) -> np.ndarray:
    """Inverse of :func:`unpack_gptq_qweight` ([K, N] values 0..15 -> [K/8, N] int32)."""
    k, n = nib.shape
    assert k % 8 == 0
    v = nib.astype(np.int64).reshape(k // 8, 8, n)
    shifts = (np.arange(8, dtype=np.int64) * 4)[None, :, None]
    w = (v << shifts).sum(axis=1) & 0xFFFFFFFF
    return w.astype(np.uint32).view(np.int32)


def unpack_rowpacked_straight(packed: np.ndarray) -> np.ndarray:
    """[R, N/8] int32 -> [R, N]; column n at bits 4*(n%8) (GPTQ qzeros order).

    `w4a16_gptq_gemm_typed.rs:155-162,233-234`.
    """
    q = packed.astype(np.int64) & 0xFFFFFFFF
    r, n8 = q.shape
    shifts = (np.arange(8, dtype=np.int64) * 4)[None, None, :]
    out = (q[:, :, None] >> shifts) & 0xF
    return out.reshape(r, n8 * 8).astype(np.int32)


def pack_rowpacked_straight(nib: np.ndarray) -> np.ndarray:
    r, n = nib.shape
    assert n % 8 == 0
    v = nib.astype(np.int64).reshape(r, n // 8, 8)
    shifts = (np.arange(8, dtype=np.int64) * 4)[None, None, :]
    w = (v << shifts).sum(axis=2) & 0xFFFFFFFF
    return w.astype(np.uint32).view(np.int32)


def unpack_awq(packed: np.ndarray) -> np.ndarray:
    """[R, N/8] int32 -> [R, N]; column n at bits 4*AWQ_ORDER[n%8].

    `awq_gemm_int4_typed.rs:137-151,196-197`; used for qweight and qzeros alike
    (`:202-205`).
    """
    q = packed.astype(np.int64) & 0xFFFFFFFF
    r, n8 = q.shape
    shifts = (AWQ_ORDER * 4)[None, None, :]
    out = (q[:, :, None] >> shifts) & 0xF
    return out.reshape(r, n8 * 8).astype(np.int32)


def pack_awq(nib: np.ndarray) -> np.ndarray:
    r, n = nib.shape
    assert n % 8 == 0
    v = nib.astype(np.int64).reshape(r, n // 8, 8)
    shifts = (AWQ_ORDER * 4)[None, None, :]
    w = (v << shifts).sum(axis=2) & 0xFFFFFFFF
    return w.astype(np.uint32).view(np.int32)


# ---------------------------------------------------------------------------
# int4 dequant + W4A16 GEMM
# ---------------------------------------------------------------------------
def _dequant(nib, zeros, scales, group_size, faithful):
    """(nib[K,N] - zeros[K/G,N]) * scales[K/G,N] in fp32; optionally rounded to
    fp16 as the reference does before its MMA (`w4a16_gptq_gemm_typed.rs:256-260`)."""
    k = nib.shape[0]
    g = np.arange(k) // group_size
    w = (nib - zeros[g]).astype(np.float32) * scales.astype(np.float32)[g]
    if faithful:
        w = w.astype(np.float16).astype(np.float32)
    return w


def gptq_dequant(qweight, scales, qzeros, group_size, zero_offset=1, faithful=False):
    """Dense [K, N] fp32 weight of a GPTQ tensor.  `zero_offset` is the +1 the
    reference GEMM adds to the stored zero nibble
    (`w4a16_gptq_gemm_typed.rs:223-236`); `qzeros=None` means symmetric zero 8
    (`ferrum_dequant_int4_sym.rs:60`)."""
    nib = unpack_gptq_qweight(qweight)
    if qzeros is None:
        zeros = np.full((nib.shape[0] // group_size, nib.shape[1]), 8, dtype=np.int32)
    else:
        zeros = unpack_rowpacked_straight(qzeros) + zero_offset
    return _dequant(nib, zeros, scales, group_size, faithful)


def awq_dequant(qweight, scales, qzeros, group_size, faithful=False):
    """Dense [K, N] fp32 weight of an AWQ tensor (no +1 on zeros,
    `awq_gemm_int4_typed.rs:202-205`)."""
    nib = unpack_awq(qweight)
    zeros = unpack_awq(qzeros)
    return _dequant(nib, zeros, scales, group_size, faithful)


def w4a16_gptq_gemm(a, qweight, scales, qzeros, group_size, zero_offset=1, faithful=False):
    """C[m,n] = sum_k A[m,k] * ((q[k,n] - zero[k/G,n]) * s[k/G,n]), fp32 accumulate
    (`w4a16_gptq_gemm_typed.rs:131-273`).  Returns fp32 [M, N]."""
    w = gptq_dequant(qweight, scales, qzeros, group_size, zero_offset, faithful)
    return a.astype(np.float32) @ w


def awq_gemm_int4(a, qweight, scales, qzeros, group_size, faithful=False):
    """`awq_gemm_int4_typed.rs:117-241`.  Returns fp32 [M, N]."""
    w = awq_dequant(qweight, scales, qzeros, group_size, faithful)
    return a.astype(np.float32) @ w


def dequant_int4_to_fp16(qweight, scales, qzeros, group_size):
    """Full-matrix GPTQ dequant, output COLUMN-major fp16 `out[col*K + k]`, zero =
    stored nibble with no +1 (`ferrum_dequant_int4.rs:59-138`).  Returns fp16 [N, K]."""
    w = gptq_dequant(qweight, scales, qzeros, group_size, zero_offset=0)
    return np.ascontiguousarray(w.T).astype(np.float16)


def dequant_int4_sym_to_fp16(qweight, scales, group_size):
    """Symmetric variant, zero = 8 (`ferrum_dequant_int4_sym.rs:58-130`).  fp16 [N, K]."""
    w = gptq_dequant(qweight, scales, None, group_size)
    return np.ascontiguousarray(w.T).astype(np.float16)


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def _attend(q, k, v, scale):
    """q [G, D], k/v [L, D] fp32 -> [G, D]; softmax over L in fp32.  Equal, up to
    fp32 rounding, to the reference's tile loop with m=-1e30, l=0 initial state
    (`attention.rs:81-82,139-153`)."""
    s = (q @ k.T) * np.float32(scale)
    m = s.max(axis=1, keepdims=True)
    p = np.exp(s - m)
    l = p.sum(axis=1, keepdims=True)
    return (p @ v) / l


def decode_attention(q, k_cache, v_cache, num_kv_heads, valid_kv_len, scale):
    """Seq-major cache [seq, Hkv, D]; q [Hq, D] (`attention.rs:66-163`)."""
    q = q.astype(np.float32)
    hq, d = q.shape
    grp = hq // num_kv_heads
    out = np.empty((hq, d), np.float32)
    for h in range(num_kv_heads):
        k = k_cache[:valid_kv_len, h].astype(np.float32)
        v = v_cache[:valid_kv_len, h].astype(np.float32)
        out[h * grp:(h + 1) * grp] = _attend(q[h * grp:(h + 1) * grp], k, v, scale)
    return out


def decode_attention_hm(q, k_cache, v_cache, valid_kv_len, scale):
    """Head-major cache [Hkv, capacity, D] (`attention.rs:198-272`)."""
    q = q.astype(np.float32)
    hq, d = q.shape
    hkv = k_cache.shape[0]
    grp = hq // hkv
    out = np.empty((hq, d), np.float32)
    for h in range(hkv):
        k = k_cache[h, :valid_kv_len].astype(np.float32)
        v = v_cache[h, :valid_kv_len].astype(np.float32)
        out[h * grp:(h + 1) * grp] = _attend(q[h * grp:(h + 1) * grp], k, v, scale)
    return out


def batched_decode_attention(q, k_cache, v_cache, valid_kv_len, scale):
    """q [B, Hq, D]; cache [B, seq, Hkv, D] seq-major; one shared length
    (`attention.rs:304-367`)."""
    return np.stack([
        decode_attention(q[b], k_cache[b], v_cache[b], k_cache.shape[2], valid_kv_len, scale)
        for b in range(q.shape[0])])


def batched_decode_attention_hm(q, k_cache, v_cache, context_lens, scale):
    """Extension named by the reference as its follow-up (`attention.rs:287-289`):
    q [B, Hq, D]; cache [B, Hkv, max_len, D] head-major; per-sequence lengths."""
    return np.stack([
        decode_attention_hm(q[b], k_cache[b], v_cache[b], int(context_lens[b]), scale)
        for b in range(q.shape[0])])


def flash_decode_phase1(q, k_cache, v_cache, num_kv_heads, valid_kv_len, num_splits, scale, block_kv):
    """Split-KV partials, seq-major cache (`attention.rs:522-584`).  Returns
    (partial_acc [Hq,S,D], partial_max [Hq,S], partial_sum [Hq,S]); each split
    covers chunk_blocks*block_kv positions with chunk_blocks = (len/S)/block_kv."""
    q = q.astype(np.float32)
    hq, d = q.shape
    grp = hq // num_kv_heads
    chunk = ((valid_kv_len // num_splits) // block_kv) * block_kv
    acc = np.zeros((hq, num_splits, d), np.float32)
    mx = np.full((hq, num_splits), -1e30, np.float32)
    sm = np.zeros((hq, num_splits), np.float32)
    for s in range(num_splits):
        lo, hi = s * chunk, (s + 1) * chunk
        if hi == lo:
            continue
        for h in range(hq):
            k = k_cache[lo:hi, h // grp].astype(np.float32)
            v = v_cache[lo:hi, h // grp].astype(np.float32)
            sc = (k @ q[h]) * np.float32(scale)
            m = sc.max()
            p = np.exp(sc - m)
            acc[h, s] = p @ v
            mx[h, s] = m
            sm[h, s] = p.sum()
    return acc, mx, sm


def flash_decode_phase2(partial_acc, partial_max, partial_sum):
    """Log-sum-exp combine (`attention.rs:611-641`): out [Hq, D]."""
    m = partial_max.max(axis=1, keepdims=True)
    alpha = np.exp(partial_max - m)
    l = (partial_sum * alpha).sum(axis=1, keepdims=True)
    w = alpha / l
    return (w[:, :, None] * partial_acc).sum(axis=1)


def paged_decode_attention(q, k_pool, v_pool, block_table, valid_kv_len, block_size, scale):
    """Block-table gather (`attention.rs:416-489`): pool [max_blocks, bs, Hkv, D]."""
    pos = np.arange(valid_kv_len)
    phys = block_table[pos // block_size]
    slot = pos % block_size
    k = k_pool[phys, slot]            # [L, Hkv, D]
    v = v_pool[phys, slot]
    return decode_attention(q, k, v, k_pool.shape[2], valid_kv_len, scale)


# ---------------------------------------------------------------------------
# glue
# ---------------------------------------------------------------------------
def rms_norm(x, w, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w, reduce in fp32 (`norms.rs:16-41,125-150`)."""
    x = x.astype(np.float32)
    inv_n = np.float32(1.0 / x.shape[-1])
    ms = (x * x).sum(axis=-1, keepdims=True, dtype=np.float32) * inv_n
    inv = (1.0 / np.sqrt(ms + np.float32(eps))).astype(np.float32)
    return x * inv * w.astype(np.float32)


def fused_add_rms_norm(x, res, w, eps):
    """r = x + res (fp32); norm computed from the unrounded sum; returns (out,
    residual_out) both fp32 (`norms.rs:85-115,189-220`)."""
    r = x.astype(np.float32) + res.astype(np.float32)
    return rms_norm(r, w, eps), r


def rope_tables(max_pos, head_dim, theta):
    """cos/sin [max_pos, D/2] fp32, the caller-side table `rope_full_f32` indexes
    (`positional.rs:94-129`); inv_freq_i = theta^(-2i/D)."""
    half = head_dim // 2
    inv_freq = (1.0 / (np.float64(theta) ** (np.arange(half, dtype=np.float64) * 2.0 / head_dim)))
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv_freq[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rope_single(x, cos_row, sin_row):
    """rope_q / rope_k: x [heads, D], tables [D/2] for one position; half-split
    pairs (i, i+D/2) (`positional.rs:24-80`)."""
    x = x.astype(np.float32)
    half = x.shape[-1] // 2
    x0, x1 = x[..., :half], x[..., half:]
    c, s = cos_row.astype(np.float32), sin_row.astype(np.float32)
    return np.concatenate([x0 * c - x1 * s, x1 * c + x0 * s], axis=-1)


def rope_full(x, cos_table, sin_table, positions):
    """x [tokens, heads, D]; tables [max_pos, D/2]; positions [tokens] i32
    (`positional.rs:94-129`)."""
    x = x.astype(np.float32)
    half = x.shape[-1] // 2
    c = cos_table[positions][:, None, :].astype(np.float32)
    s = sin_table[positions][:, None, :].astype(np.float32)
    x0, x1 = x[..., :half], x[..., half:]
    return np.concatenate([x0 * c - x1 * s, x1 * c + x0 * s], axis=-1)


def unified_attention(q, k_pool, v_pool, block_table, seq_lens, query_start_loc, num_kv_heads, block_size, scale):
    """Prefill + decode over a paged pool (`attention.rs:988-1187`): q [tokens, Hq, D]; pools
    [blocks, block_size, Hkv, D]; the query tokens of a sequence are the last q_len positions of its KV
    stream, causal mask kv_pos <= context_len + q_pos (`:1137-1153`), paged address arithmetic as `:1093-1101`."""
    q = np.asarray(q, dtype=np.float32)
    tokens, hq, d = q.shape
    out = np.zeros_like(q)
    groups = hq // num_kv_heads
    for s in range(len(seq_lens)):
        q0, q1 = int(query_start_loc[s]), int(query_start_loc[s + 1])
        seq_len = int(seq_lens[s])
        ctx = seq_len - (q1 - q0)
        pos = np.arange(seq_len)
        phys = np.asarray(block_table[s])[pos // block_size]
        k = np.asarray(k_pool, dtype=np.float32)[phys, pos % block_size]        # [seq_len, Hkv, D]
        v = np.asarray(v_pool, dtype=np.float32)[phys, pos % block_size]
        for j in range(q1 - q0):
            vis = ctx + j + 1
            for h in range(hq):
                kvh = h // groups
                sc = (k[:vis, kvh] @ q[q0 + j, h]) * np.float32(scale)
                p = np.exp(sc - sc.max())
                out[q0 + j, h] = (p[:, None] * v[:vis, kvh]).sum(axis=0) / p.sum()
    return out


def flash_attn_full(q, k, v, pos_offset, scale):
    """Causal prefill attention (`attention.rs:780-909`): q [B, Hq, q_len, D], k / v [B, Hkv, kv_len, D];
    query row i sees kv positions <= pos_offset + i (`:864-870`); fp32 throughout (`:773-779`)."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    b, hq, q_len, d = q.shape
    hkv, kv_len = k.shape[1], k.shape[2]
    groups = hq // hkv
    out = np.zeros_like(q)
    for bi in range(b):
        for h in range(hq):
            kvh = h // groups
            sc = (q[bi, h] @ k[bi, kvh].T) * np.float32(scale)                       # [q_len, kv_len]
            allowed = np.arange(kv_len)[None, :] <= (np.arange(q_len)[:, None] + pos_offset)
            sc = np.where(allowed, sc, -np.inf)
            mx = sc.max(axis=1, keepdims=True)
            p = np.exp(sc - np.where(np.isfinite(mx), mx, 0.0))
            den = p.sum(axis=1, keepdims=True)
            out[bi, h] = np.where(den > 0, (p @ v[bi, kvh]) / np.where(den > 0, den, 1.0), 0.0)
    return out


def split_qkv(qkv, num_heads, head_dim):
    """qkv [batch, 3, heads, D] -> (q, k, v) each [batch, heads, D] (`projection.rs:18-51`)."""
    x = np.asarray(qkv, dtype=np.float32).reshape(-1, 3, num_heads, head_dim)
    return x[:, 0].copy(), x[:, 1].copy(), x[:, 2].copy()


def transpose_head_to_token(x):
    """[heads, tokens, D] -> [tokens, heads, D] (`projection.rs:60-79`)."""
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32).transpose(1, 0, 2))


def transpose_token_to_head(x):
    """[tokens, heads, D] -> [heads, tokens, D] (`projection.rs:87-105`)."""
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32).transpose(1, 0, 2))


def rope_transpose(x, cos_table, sin_table, pos_offset):
    """x [tokens, heads, D] -> RoPE with table row pos_offset + token on the pairs (i, i + D/2), stored
    head-major [heads, tokens, D] (`projection.rs:182-215`)."""
    x = np.asarray(x, dtype=np.float32)
    pos = pos_offset + np.arange(x.shape[0])
    return transpose_token_to_head(rope_full(x, cos_table, sin_table, pos))


def qk_norm_rope_transpose(x, norm_w, cos_table, sin_table, pos_offset, eps):
    """Per (token, head): x * rsqrt(mean(x^2) + eps) * norm_w, then RoPE, then head-major store
    (`projection.rs:119-175`; the scaled halves feed the rotation, `:164-168`)."""
    x = np.asarray(x, dtype=np.float32)
    return rope_transpose(rms_norm(x, np.asarray(norm_w, dtype=np.float32), eps), cos_table, sin_table, pos_offset)


def kv_cache_append(new_k, new_v, k_cache, v_cache, cache_idx):
    """Seq-major shared cache [max_seq, H, D]; row b goes to cache[cache_idx[b]]
    (`cache.rs:21-47`).  In place."""
    for b in range(new_k.shape[0]):
        k_cache[cache_idx[b]] = new_k[b]
        v_cache[cache_idx[b]] = new_v[b]


def kv_cache_append_hm(new_k, new_v, k_cache, v_cache, cache_idx):
    """Batched head-major extension: cache [B, H, max_len, D]; row (b, h) goes to
    cache[b, h, cache_idx[b]].  Same gather/scatter as `cache.rs:21-47` with the
    head-major addressing of `attention.rs:216-230`.  In place."""
    for b in range(new_k.shape[0]):
        k_cache[b, :, cache_idx[b]] = new_k[b]
        v_cache[b, :, cache_idx[b]] = new_v[b]


def residual_add(a, b):
    """fp32 add (`elementwise.rs:46-58`).  For fp16 inputs the reference adds in
    fp16 (`:62-74`), which rounds identically to an fp32 add rounded once."""
    return a.astype(np.float32) + b.astype(np.float32)


def fused_silu_mul(gate, up):
    """silu(g) * u with silu(g) = g / (1 + exp(-g)), all fp32 (`elementwise.rs:148-184`)."""
    g = gate.astype(np.float32)
    u = up.astype(np.float32)
    return g / (np.exp(-g) + np.float32(1.0)) * u


def fused_silu_mul_interleaved(gate_up, inter):
    """Row b of gate_up [B, 2*inter]: gate = first `inter`, up = second `inter`
    (`elementwise.rs:188-212,225-250`)."""
    gu = gate_up.reshape(-1, 2 * inter)
    return fused_silu_mul(gu[:, :inter], gu[:, inter:])


# ---------------------------------------------------------------------------
# the two ends of a decode step: embedding gather, row softmax
# ---------------------------------------------------------------------------
def embedding_lookup(embeddings, indices):
    """output[tok, :] = embeddings[indices[tok], :] (`embedding.rs:17-55`); a pure move."""
    return embeddings[np.asarray(indices, dtype=np.int64)]


def softmax(x):
    """Row softmax in fp32: exp(x - max) / sum(exp(x - max)) (`reduction.rs:11-68`; host formula of
    `crates/triton-runtime/examples/run_softmax.rs:62-68`).  Returns fp32."""
    x = x.astype(np.float32)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True, dtype=np.float32)


# ---------------------------------------------------------------------------
# fused MoE (absent from the reference; specified by the benchmark config and
# the reference's conventions for its parts: GPTQ layout, half-split gate|up)
# ---------------------------------------------------------------------------
def moe_route(logits, top_k):
    """fp32 softmax over experts, top-k (ties: lowest expert index first), weights
    renormalised to sum 1.  Experts are ranked by logit: softmax is monotonic, so this
    is the top-k of the softmax, and the ranking does not depend on how exp rounds.
    Returns (topk_ids [T,k] int32, topk_w [T,k] fp32)."""
    x = logits.astype(np.float32)
    m = x.max(axis=1, keepdims=True)
    # stable argsort on -x keeps the lowest index first among equals
    order = np.argsort(-x, axis=1, kind="stable")[:, :top_k]
    w = np.exp(np.take_along_axis(x, order, axis=1) - m)     # softmax numerators; the denominator cancels
    w = w / w.sum(axis=1, keepdims=True, dtype=np.float32)
    return order.astype(np.int32), w.astype(np.float32)


def moe_permute(topk_ids, num_experts):
    """Segmented token list.  Pair index p = t*k + j.  Returns
    (counts [E], offsets [E+1], sorted_pairs [T*k] int32 = pair indices ordered by
    expert then by pair index (stable), inv [T*k] int32 = position of each pair)."""
    flat = topk_ids.reshape(-1)
    sorted_pairs = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=num_experts).astype(np.int32)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    inv = np.empty_like(sorted_pairs)
    inv[sorted_pairs] = np.arange(sorted_pairs.size, dtype=np.int32)
    return counts, offsets, sorted_pairs, inv


def fused_moe_gptq(x, logits, w13_q, w13_s, w2_q, w2_s, top_k, group_size, round_intermediate=True, expert_first=0,
                   faithful=False, with_mag=False):
    """x [T, H] fp16; per-expert symmetric GPTQ w13 [E, H/8, 2I] (gate | up halves),
    w2 [E, I/8, H]; out[t] = sum_j w[t,j] * (silu(g)*u) @ W2_e.  The intermediate
    activation is rounded to fp16 between the GEMMs when `round_intermediate`
    (the CUDA path stores it as fp16).  Returns fp32 [T, H].
    Expert-parallel share: pass the weight stacks of experts [expert_first, expert_first + len(w13_q)) only;
    routing still runs over all of `logits`' experts and pairs routed elsewhere contribute nothing.
    `faithful` rounds the dequantised weights to fp16 first, as the reference's GEMM does
    (`w4a16_gptq_gemm_typed.rs:256-260`).  `with_mag` also returns sum_j |w[t,j] * y_j|, the magnitude of the
    summands of every output element (a sum of k terms is only as exact as its terms, whatever it comes to)."""
    t, h = x.shape
    e = logits.shape[1]
    ids, wts = moe_route(logits, top_k)
    out = np.zeros((t, h), np.float32)
    mag = np.zeros((t, h), np.float32)
    xf = x.astype(np.float32)
    for ex in range(expert_first, min(e, expert_first + len(w13_q))):
        tok, slot = np.nonzero(ids == ex)
        if tok.size == 0:
            continue
        w13 = gptq_dequant(w13_q[ex - expert_first], w13_s[ex - expert_first], None, group_size, faithful=faithful)
        w2 = gptq_dequant(w2_q[ex - expert_first], w2_s[ex - expert_first], None, group_size, faithful=faithful)
        gu = xf[tok] @ w13
        inter = w13.shape[1] // 2
        act = fused_silu_mul(gu[:, :inter], gu[:, inter:])
        if round_intermediate:
            act = act.astype(np.float16).astype(np.float32)
        y = act @ w2
        np.add.at(out, tok, y * wts[tok, slot][:, None])
        np.add.at(mag, tok, np.abs(y * wts[tok, slot][:, None]))
    return (out, mag) if with_mag else out


# ---------------------------------------------------------------------------
# decode layer chain (Llama shape): the consumer's per-layer call sequence
# ---------------------------------------------------------------------------
def decode_layer(hidden, p, k_cache, v_cache, positions, round_fp16=True, faithful=True, stages=None):
    """rms_norm -> QKV int4 GEMM -> RoPE -> kv_cache_append -> decode attention ->
    o_proj -> residual_add -> rms_norm -> gate_up int4 -> silu_mul -> down int4 ->
    residual_add, on hidden [B, H].  `p` holds GPTQ tensors (qweight, scales,
    qzeros) for "qkv", "o", "gate_up", "down", norm weights "ln1", "ln2", the RoPE
    tables "cos", "sin", and ints "hq", "hkv", "d", "group", "zero_offset", "eps".
    Caches are [B, Hkv, max_len, D] head-major and are appended in place at
    `positions`; attention then runs over positions+1 entries.  With `round_fp16`
    each tensor that the CUDA path materialises in fp16 is rounded at that point.
    `faithful` adds the reference's own extra roundings: the dequantised weight rounded
    to fp16 before the product (`w4a16_gptq_gemm_typed.rs:256-260`) and the second norm
    taken from the unrounded fp32 sum while the stored residual is that sum rounded to
    fp16 (`norms.rs:208-219`).  A dict passed as `stages` receives the intermediates
    (n1, qkv, q, att, o, h1, n2, gate_up, act, down).  Returns fp32 [B, H]."""
    r16 = (lambda a: a.astype(np.float16).astype(np.float32)) if round_fp16 else (lambda a: a)
    hq, hkv, d, g, zo = p["hq"], p["hkv"], p["d"], p["group"], p["zero_offset"]
    b = hidden.shape[0]
    x = hidden.astype(np.float32)
    n1 = r16(rms_norm(x, p["ln1"], p["eps"]))
    qkv = r16(w4a16_gptq_gemm(n1, *p["qkv"], g, zo, faithful))
    q = qkv[:, :hq * d].reshape(b, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].reshape(b, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(b, hkv, d)
    q = r16(rope_full(q, p["cos"], p["sin"], positions))
    k = r16(rope_full(k, p["cos"], p["sin"], positions))
    kv_cache_append_hm(k.astype(k_cache.dtype), v.astype(v_cache.dtype), k_cache, v_cache, positions)
    scale = 1.0 / np.sqrt(d)
    attn = r16(batched_decode_attention_hm(q, k_cache, v_cache, positions + 1, scale))
    o = r16(w4a16_gptq_gemm(attn.reshape(b, hq * d), *p["o"], g, zo, faithful))
    h1 = r16(residual_add(x, o))
    n2 = r16(rms_norm(residual_add(x, o) if faithful else h1, p["ln2"], p["eps"]))
    gu = r16(w4a16_gptq_gemm(n2, *p["gate_up"], g, zo, faithful))
    act = r16(fused_silu_mul_interleaved(gu, gu.shape[1] // 2))
    dn = r16(w4a16_gptq_gemm(act, *p["down"], g, zo, faithful))
    if stages is not None:
        stages.update(n1=n1, qkv=qkv, q=q, att=attn, o=o, h1=h1, n2=n2, gate_up=gu, act=act, down=dn)
    return residual_add(h1, dn)

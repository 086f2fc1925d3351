// Generated from include/b200_kernels.h by triton-rs_b200/rust_sys.py; do not edit by hand.
// One declaration per prototype of the header.  Device pointers are raw pointers into CUDA
// memory (a cudarc `CudaSlice<T>`'s `device_ptr` cast to the pointer type); `b200k_stream` is
// the `CUstream` of a cudarc `CudaStream`.
#![allow(non_camel_case_types, non_upper_case_globals, clippy::too_many_arguments)]

use std::os::raw::{c_char, c_int, c_void};

/// IEEE binary16 bits (`half::f16::to_bits`).
pub type b200k_half = u16;
/// bfloat16 bits (`half::bf16::to_bits`).
pub type b200k_bf16 = u16;
/// `cudaStream_t` / `CUstream`; null is the legacy default stream.
pub type b200k_stream = *mut c_void;

#[repr(C)]
pub struct b200k_layer {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct b200k_comm {
    _opaque: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct b200k_layer_config {
    pub hidden: c_int,
    pub num_q_heads: c_int,
    pub num_kv_heads: c_int,
    pub head_dim: c_int,
    pub intermediate: c_int,
    pub group_size: c_int,
    pub weight_format: c_int,
    pub max_batch: c_int,
    pub max_len: c_int,
    pub rms_eps: f32,
    pub use_graph: c_int,
    pub reserved: [c_int; 5],
}

pub const B200K_OK: c_int = 0;
pub const B200K_E_NULL: c_int = -1;
pub const B200K_E_SHAPE: c_int = -2;
pub const B200K_E_ALIGN: c_int = -3;
pub const B200K_E_WORKSPACE: c_int = -4;
pub const B200K_E_DEVICE: c_int = -5;
pub const B200K_E_STATE: c_int = -6;
pub const B200K_DEFAULT_WORKSPACE_BYTES: usize = (256 << 20);
pub const B200K_NOALLOC_SCRATCH_BYTES: usize = (8 << 20);

#[link(name = "b200_kernels")]
extern "C" {
    pub fn b200k_last_error() -> *const c_char;
    pub fn b200k_version() -> *const c_char;
    pub fn b200k_device_check() -> c_int;
    pub fn b200k_set_workspace(workspace: *mut c_void, bytes: usize) -> c_int;
    pub fn b200k_gemm_workspace_bytes(m: c_int, n: c_int, k: c_int) -> usize;
    pub fn b200k_attention_workspace_bytes(
        batch: c_int, num_q_heads: c_int, num_kv_heads: c_int, head_dim: c_int, max_len: c_int
    ) -> usize;
    pub fn b200k_workspace_status(
        workspace: *const c_void, host_status_out: *mut c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_workspace_clear_status(workspace: *mut c_void, stream: b200k_stream) -> c_int;
    pub fn w4a16_gptq_gemm_f16(
        a: *const b200k_half, qweight: *const i32, scales: *const b200k_half, qzeros: *const i32,
        c: *mut b200k_half, m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int, stride_am: c_int,
        stride_ak: c_int, stride_qwk: c_int, stride_qwn: c_int, stride_sk: c_int, stride_sn: c_int,
        stride_qzk: c_int, stride_qzn: c_int, stride_cm: c_int, stride_cn: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn w4a16_gptq_gemm_sym_f16(
        a: *const b200k_half, qweight: *const i32, scales: *const b200k_half, c: *mut b200k_half,
        m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int, stride_am: c_int, stride_ak: c_int,
        stride_qwk: c_int, stride_qwn: c_int, stride_sk: c_int, stride_sn: c_int, stride_cm: c_int,
        stride_cn: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn awq_gemm_int4_f16(
        a: *const b200k_half, qweight: *const i32, scales: *const b200k_half, qzeros: *const i32,
        c: *mut b200k_half, m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int, stride_am: c_int,
        stride_ak: c_int, stride_qwk: c_int, stride_qwn: c_int, stride_sk: c_int, stride_sn: c_int,
        stride_qzk: c_int, stride_qzn: c_int, stride_cm: c_int, stride_cn: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn w4a16_gptq_gemm_f16_ws(
        a: *const b200k_half, qweight: *const i32, scales: *const b200k_half, qzeros: *const i32,
        c: *mut b200k_half, m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int, stride_am: c_int,
        stride_ak: c_int, stride_qwk: c_int, stride_qwn: c_int, stride_sk: c_int, stride_sn: c_int,
        stride_qzk: c_int, stride_qzn: c_int, stride_cm: c_int, stride_cn: c_int, workspace: *mut c_void,
        workspace_bytes: usize, stream: b200k_stream
    ) -> c_int;
    pub fn awq_gemm_int4_f16_ws(
        a: *const b200k_half, qweight: *const i32, scales: *const b200k_half, qzeros: *const i32,
        c: *mut b200k_half, m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int, stride_am: c_int,
        stride_ak: c_int, stride_qwk: c_int, stride_qwn: c_int, stride_sk: c_int, stride_sn: c_int,
        stride_qzk: c_int, stride_qzn: c_int, stride_cm: c_int, stride_cn: c_int, workspace: *mut c_void,
        workspace_bytes: usize, stream: b200k_stream
    ) -> c_int;
    pub fn w4a16_gptq_gemm_silu_mul_f16(
        a: *const b200k_half, qweight: *const i32, scales: *const b200k_half, qzeros: *const i32,
        c: *mut b200k_half, m_size: c_int, inter_size: c_int, k_size: c_int, group_size: c_int,
        stream: b200k_stream
    ) -> c_int;
    pub fn permute_k8_f16(
        input: *const b200k_half, output: *mut b200k_half, rows: c_int, k_size: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn w4a16_gptq_gemm_kperm_f16(
        a_permuted: *const b200k_half, qweight: *const i32, scales: *const b200k_half, qzeros: *const i32,
        c: *mut b200k_half, m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int,
        stream: b200k_stream
    ) -> c_int;
    pub fn b200k_gemm_tc_plan(
        m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int, awq: c_int, host_plan_out: *mut c_int
    ) -> c_int;
    pub fn dequant_int4_to_fp16(
        qweight: *const i32, scales: *const b200k_half, qzeros: *const i32, output: *mut b200k_half,
        k_dim: c_int, n_dim: c_int, group_size: c_int, n_div_8: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn dequant_int4_sym_to_fp16(
        qweight: *const i32, scales: *const b200k_half, output: *mut b200k_half, k_dim: c_int, n_dim: c_int,
        group_size: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_prepack_awq(
        qweight: *const i32, qzeros: *const i32, qweight_packed: *mut i32, qzeros_packed: *mut i32,
        k_size: c_int, n_size: c_int, group_size: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn awq_gemm_int4_prepacked_f16(
        a: *const b200k_half, qweight_packed: *const i32, scales: *const b200k_half,
        qzeros_packed: *const i32, c: *mut b200k_half, m_size: c_int, n_size: c_int, k_size: c_int,
        group_size: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_unpack_gptq_qweight(
        qweight: *const i32, out: *mut i8, k_dim: c_int, n_dim: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_unpack_gptq_qzeros(
        qzeros: *const i32, out: *mut i8, groups: c_int, n_dim: c_int, zero_offset: c_int,
        stream: b200k_stream
    ) -> c_int;
    pub fn b200k_unpack_awq(
        packed: *const i32, out: *mut i8, rows: c_int, n_dim: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn decode_attention_f16(
        q: *const b200k_half, k_cache: *const b200k_half, v_cache: *const b200k_half, output: *mut b200k_half,
        num_q_heads: c_int, num_kv_heads: c_int, head_dim: c_int, valid_kv_len: c_int, scale: f32,
        stream: b200k_stream
    ) -> c_int;
    pub fn decode_attention_f32(
        q: *const f32, k_cache: *const f32, v_cache: *const f32, output: *mut f32, num_q_heads: c_int,
        num_kv_heads: c_int, head_dim: c_int, valid_kv_len: c_int, scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn decode_attention_hm_f16(
        q: *const b200k_half, k_cache: *const b200k_half, v_cache: *const b200k_half, output: *mut b200k_half,
        num_q_heads: c_int, num_kv_heads: c_int, head_dim: c_int, capacity: c_int, valid_kv_len: c_int,
        scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn decode_attention_hm_f32(
        q: *const f32, k_cache: *const f32, v_cache: *const f32, output: *mut f32, num_q_heads: c_int,
        num_kv_heads: c_int, head_dim: c_int, capacity: c_int, valid_kv_len: c_int, scale: f32,
        stream: b200k_stream
    ) -> c_int;
    pub fn batched_decode_attention_f32(
        q: *const f32, k_cache: *const f32, v_cache: *const f32, output: *mut f32, batch_size: c_int,
        num_q_heads: c_int, num_kv_heads: c_int, head_dim: c_int, seq_len: c_int, valid_kv_len: c_int,
        scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn batched_decode_attention_hm_f16(
        q: *const b200k_half, k_cache: *const b200k_half, v_cache: *const b200k_half,
        context_lens: *const i32, output: *mut b200k_half, batch_size: c_int, num_q_heads: c_int,
        num_kv_heads: c_int, head_dim: c_int, max_len: c_int, scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn batched_decode_attention_hm_f16_ws(
        q: *const b200k_half, k_cache: *const b200k_half, v_cache: *const b200k_half,
        context_lens: *const i32, output: *mut b200k_half, batch_size: c_int, num_q_heads: c_int,
        num_kv_heads: c_int, head_dim: c_int, max_len: c_int, scale: f32, workspace: *mut c_void,
        workspace_bytes: usize, stream: b200k_stream
    ) -> c_int;
    pub fn batched_decode_attention_hm_f16_noalloc(
        q: *const b200k_half, k_cache: *const b200k_half, v_cache: *const b200k_half,
        context_lens: *const i32, output: *mut b200k_half, batch_size: c_int, num_q_heads: c_int,
        num_kv_heads: c_int, head_dim: c_int, max_len: c_int, scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_noalloc_status(host_status_out: *mut c_int, stream: b200k_stream) -> c_int;
    pub fn flash_decode_attn_phase1_f32(
        q: *const f32, k_cache: *const f32, v_cache: *const f32, partial_acc: *mut f32, partial_max: *mut f32,
        partial_sum: *mut f32, num_q_heads: c_int, num_kv_heads: c_int, head_dim: c_int, valid_kv_len: c_int,
        num_splits: c_int, scale: f32, block_kv: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn batched_flash_decode_attn_phase1_f32(
        q: *const f32, k_cache: *const f32, v_cache: *const f32, partial_acc: *mut f32, partial_max: *mut f32,
        partial_sum: *mut f32, batch_size: c_int, num_q_heads: c_int, num_kv_heads: c_int, head_dim: c_int,
        seq_len: c_int, valid_kv_len: c_int, num_splits: c_int, scale: f32, block_kv: c_int,
        stream: b200k_stream
    ) -> c_int;
    pub fn flash_decode_attn_phase2_f32(
        partial_acc: *const f32, partial_max: *const f32, partial_sum: *const f32, output: *mut f32,
        num_q_heads: c_int, head_dim: c_int, num_splits: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn paged_decode_attention_f16(
        q: *const b200k_half, k_block_pool: *const b200k_half, v_block_pool: *const b200k_half,
        block_table: *const i32, output: *mut b200k_half, num_q_heads: c_int, num_kv_heads: c_int,
        head_dim: c_int, valid_kv_len: c_int, block_size: c_int, scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn unified_attention_f32(
        q: *const f32, k_cache: *const f32, v_cache: *const f32, output: *mut f32, block_table: *const i32,
        seq_lens: *const i32, query_start_loc: *const i32, num_q_heads: c_int, num_kv_heads: c_int,
        head_dim: c_int, block_size: c_int, max_blocks_per_seq: c_int, sm_scale: f32, num_seqs: c_int,
        stream: b200k_stream
    ) -> c_int;
    pub fn flash_attn_full_f32(
        q: *const f32, k: *const f32, v: *const f32, output: *mut f32, batch: c_int, num_heads: c_int,
        num_kv_heads: c_int, q_len: c_int, kv_len: c_int, head_dim: c_int, pos_offset: c_int, scale: f32,
        stream: b200k_stream
    ) -> c_int;
    pub fn flash_attn_full_f16(
        q: *const b200k_half, k: *const b200k_half, v: *const b200k_half, output: *mut b200k_half,
        batch: c_int, num_heads: c_int, num_kv_heads: c_int, q_len: c_int, kv_len: c_int, head_dim: c_int,
        pos_offset: c_int, scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn split_qkv_f32(
        qkv: *const f32, q_out: *mut f32, k_out: *mut f32, v_out: *mut f32, num_heads: c_int, head_dim: c_int,
        batch: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn transpose_head_to_token_f32(
        input: *const f32, output: *mut f32, tokens: c_int, heads: c_int, head_dim: c_int,
        stream: b200k_stream
    ) -> c_int;
    pub fn transpose_token_to_head_f32(
        input: *const f32, output: *mut f32, tokens: c_int, heads: c_int, head_dim: c_int,
        stream: b200k_stream
    ) -> c_int;
    pub fn qk_norm_rope_transpose_f32(
        input: *const f32, norm_w: *const f32, cos_tab: *const f32, sin_tab: *const f32, output: *mut f32,
        tokens: c_int, heads: c_int, head_dim: c_int, pos_offset: c_int, inv_n: f32, eps: f32,
        stream: b200k_stream
    ) -> c_int;
    pub fn rope_transpose_f32(
        input: *const f32, cos_tab: *const f32, sin_tab: *const f32, output: *mut f32, tokens: c_int,
        heads: c_int, head_dim: c_int, pos_offset: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn moe_route_topk_f32(
        router_logits: *const f32, topk_ids: *mut i32, topk_weights: *mut f32, num_tokens: c_int,
        num_experts: c_int, top_k: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn moe_permute(
        topk_ids: *const i32, counts: *mut i32, offsets: *mut i32, sorted_pairs: *mut i32, inverse: *mut i32,
        num_pairs: c_int, num_experts: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_moe_workspace_bytes(
        num_tokens: c_int, hidden: c_int, num_experts: c_int, top_k: c_int, intermediate: c_int
    ) -> usize;
    pub fn fused_moe_gptq_f16(
        x: *const b200k_half, router_logits: *const f32, w13_qweight: *const i32,
        w13_scales: *const b200k_half, w13_qzeros: *const i32, w2_qweight: *const i32,
        w2_scales: *const b200k_half, w2_qzeros: *const i32, out: *mut b200k_half, num_tokens: c_int,
        hidden: c_int, num_experts: c_int, top_k: c_int, intermediate: c_int, group_size: c_int,
        workspace: *mut c_void, workspace_bytes: usize, stream: b200k_stream
    ) -> c_int;
    pub fn fused_moe_gptq_ep_f16(
        x: *const b200k_half, router_logits: *const f32, w13_qweight: *const i32,
        w13_scales: *const b200k_half, w13_qzeros: *const i32, w2_qweight: *const i32,
        w2_scales: *const b200k_half, w2_qzeros: *const i32, partial_out: *mut b200k_half, num_tokens: c_int,
        hidden: c_int, num_experts: c_int, expert_first: c_int, num_local_experts: c_int, top_k: c_int,
        intermediate: c_int, group_size: c_int, workspace: *mut c_void, workspace_bytes: usize,
        stream: b200k_stream
    ) -> c_int;
    pub fn rms_norm_f16(
        input: *const b200k_half, weight: *const b200k_half, output: *mut b200k_half, row_size: c_int,
        inv_n: f32, eps: f32, num_rows: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn rms_norm_f32(
        input: *const f32, weight: *const f32, output: *mut f32, row_size: c_int, inv_n: f32, eps: f32,
        num_rows: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_add_rms_norm_f16(
        input: *const b200k_half, residual: *const b200k_half, weight: *const b200k_half,
        output: *mut b200k_half, residual_out: *mut b200k_half, hidden_size: c_int, inv_n: f32, eps: f32,
        num_rows: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_add_rms_norm_f32(
        input: *const f32, residual: *const f32, weight: *const f32, output: *mut f32, residual_out: *mut f32,
        hidden_size: c_int, inv_n: f32, eps: f32, num_rows: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn residual_add_f16(
        a: *const b200k_half, b: *const b200k_half, out: *mut b200k_half, n: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn residual_add_f32(
        a: *const f32, b: *const f32, out: *mut f32, n: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn residual_add_inplace_f16(
        a: *mut b200k_half, b: *const b200k_half, n: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn residual_add_inplace_f32(a: *mut f32, b: *const f32, n: c_int, stream: b200k_stream) -> c_int;
    pub fn fused_silu_mul_f16(
        gate: *const b200k_half, up: *const b200k_half, out: *mut b200k_half, n: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_silu_mul_f32(
        gate: *const f32, up: *const f32, out: *mut f32, n: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_silu_mul_interleaved_f16(
        gate_up: *const b200k_half, out: *mut b200k_half, inter: c_int, total: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_silu_mul_interleaved_f32(
        gate_up: *const f32, out: *mut f32, inter: c_int, total: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn rope_q_f32(
        q: *const f32, cos_table: *const f32, sin_table: *const f32, q_out: *mut f32, head_dim: c_int,
        num_heads: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn rope_k_f32(
        k: *const f32, cos_table: *const f32, sin_table: *const f32, k_out: *mut f32, head_dim: c_int,
        num_heads: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn rope_full_f32(
        q: *const f32, cos_table: *const f32, sin_table: *const f32, positions: *const i32, q_out: *mut f32,
        num_heads: c_int, head_dim: c_int, num_tokens: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn rope_full_f16(
        q: *const b200k_half, cos_table: *const f32, sin_table: *const f32, positions: *const i32,
        q_out: *mut b200k_half, num_heads: c_int, head_dim: c_int, num_tokens: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn kv_cache_append_f32(
        new_keys: *const f32, new_values: *const f32, k_cache: *mut f32, v_cache: *mut f32,
        cache_idx: *const i32, num_heads: c_int, head_dim: c_int, batch: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn kv_cache_append_hm_f16(
        new_keys: *const b200k_half, new_values: *const b200k_half, k_cache: *mut b200k_half,
        v_cache: *mut b200k_half, cache_idx: *const i32, num_heads: c_int, head_dim: c_int, max_len: c_int,
        batch: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn rope_kv_append_hm_f16(
        qkv: *const b200k_half, cos_table: *const f32, sin_table: *const f32, positions: *const i32,
        q_out: *mut b200k_half, k_cache: *mut b200k_half, v_cache: *mut b200k_half, num_q_heads: c_int,
        num_kv_heads: c_int, head_dim: c_int, max_len: c_int, batch: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn w4a16_gptq_gemm_bf16(
        a: *const b200k_bf16, qweight: *const i32, scales: *const b200k_bf16, qzeros: *const i32,
        c: *mut b200k_bf16, m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int, stride_am: c_int,
        stride_ak: c_int, stride_qwk: c_int, stride_qwn: c_int, stride_sk: c_int, stride_sn: c_int,
        stride_qzk: c_int, stride_qzn: c_int, stride_cm: c_int, stride_cn: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn awq_gemm_int4_bf16(
        a: *const b200k_bf16, qweight: *const i32, scales: *const b200k_bf16, qzeros: *const i32,
        c: *mut b200k_bf16, m_size: c_int, n_size: c_int, k_size: c_int, group_size: c_int, stride_am: c_int,
        stride_ak: c_int, stride_qwk: c_int, stride_qwn: c_int, stride_sk: c_int, stride_sn: c_int,
        stride_qzk: c_int, stride_qzn: c_int, stride_cm: c_int, stride_cn: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn decode_attention_bf16(
        q: *const b200k_bf16, k_cache: *const b200k_bf16, v_cache: *const b200k_bf16, output: *mut b200k_bf16,
        num_q_heads: c_int, num_kv_heads: c_int, head_dim: c_int, valid_kv_len: c_int, scale: f32,
        stream: b200k_stream
    ) -> c_int;
    pub fn decode_attention_hm_bf16(
        q: *const b200k_bf16, k_cache: *const b200k_bf16, v_cache: *const b200k_bf16, output: *mut b200k_bf16,
        num_q_heads: c_int, num_kv_heads: c_int, head_dim: c_int, capacity: c_int, valid_kv_len: c_int,
        scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn paged_decode_attention_bf16(
        q: *const b200k_bf16, k_block_pool: *const b200k_bf16, v_block_pool: *const b200k_bf16,
        block_table: *const i32, output: *mut b200k_bf16, num_q_heads: c_int, num_kv_heads: c_int,
        head_dim: c_int, valid_kv_len: c_int, block_size: c_int, scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn rms_norm_bf16(
        input: *const b200k_bf16, weight: *const b200k_bf16, output: *mut b200k_bf16, row_size: c_int,
        inv_n: f32, eps: f32, num_rows: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_add_rms_norm_bf16(
        input: *const b200k_bf16, residual: *const b200k_bf16, weight: *const b200k_bf16,
        output: *mut b200k_bf16, residual_out: *mut b200k_bf16, hidden_size: c_int, inv_n: f32, eps: f32,
        num_rows: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn residual_add_bf16(
        a: *const b200k_bf16, b: *const b200k_bf16, out: *mut b200k_bf16, n: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn residual_add_inplace_bf16(
        a: *mut b200k_bf16, b: *const b200k_bf16, n: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_silu_mul_bf16(
        gate: *const b200k_bf16, up: *const b200k_bf16, out: *mut b200k_bf16, n: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn fused_silu_mul_interleaved_bf16(
        gate_up: *const b200k_bf16, out: *mut b200k_bf16, inter: c_int, total: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn rope_full_bf16(
        q: *const b200k_bf16, cos_table: *const f32, sin_table: *const f32, positions: *const i32,
        q_out: *mut b200k_bf16, num_heads: c_int, head_dim: c_int, num_tokens: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn kv_cache_append_hm_bf16(
        new_keys: *const b200k_bf16, new_values: *const b200k_bf16, k_cache: *mut b200k_bf16,
        v_cache: *mut b200k_bf16, cache_idx: *const i32, num_heads: c_int, head_dim: c_int, max_len: c_int,
        batch: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn embedding_lookup_bf16(
        embeddings: *const b200k_bf16, indices: *const i32, output: *mut b200k_bf16, hidden_size: c_int,
        num_tokens: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn softmax_bf16(
        input: *const b200k_bf16, output: *mut b200k_bf16, rows: c_int, cols: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn flash_attn_full_bf16(
        q: *const b200k_bf16, k: *const b200k_bf16, v: *const b200k_bf16, output: *mut b200k_bf16,
        batch: c_int, num_heads: c_int, num_kv_heads: c_int, q_len: c_int, kv_len: c_int, head_dim: c_int,
        pos_offset: c_int, scale: f32, stream: b200k_stream
    ) -> c_int;
    pub fn embedding_lookup_f32(
        embeddings: *const f32, indices: *const i32, output: *mut f32, hidden_size: c_int, num_tokens: c_int,
        stream: b200k_stream
    ) -> c_int;
    pub fn embedding_lookup_f16(
        embeddings: *const b200k_half, indices: *const i32, output: *mut b200k_half, hidden_size: c_int,
        num_tokens: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn softmax_f32(
        input: *const f32, output: *mut f32, rows: c_int, cols: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn softmax_f16(
        input: *const b200k_half, output: *mut b200k_half, rows: c_int, cols: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_layer_create(config: *const b200k_layer_config, out_layer: *mut *mut b200k_layer) -> c_int;
    pub fn b200k_layer_destroy(layer: *mut b200k_layer);
    pub fn b200k_layer_set_weight(
        layer: *mut b200k_layer, which: c_int, qweight: *const i32, scales: *const b200k_half,
        qzeros: *const i32
    ) -> c_int;
    pub fn b200k_layer_set_norms_rope(
        layer: *mut b200k_layer, ln1: *const b200k_half, ln2: *const b200k_half, cos_table: *const f32,
        sin_table: *const f32
    ) -> c_int;
    pub fn b200k_layer_set_kv_cache(
        layer: *mut b200k_layer, k_cache: *mut b200k_half, v_cache: *mut b200k_half
    ) -> c_int;
    pub fn b200k_comm_create(
        rank: c_int, world: c_int, slot_bytes: usize, out_comm: *mut *mut b200k_comm
    ) -> c_int;
    pub fn b200k_comm_ipc_handle(comm: *mut b200k_comm, host_handle_64_bytes: *mut c_void) -> c_int;
    pub fn b200k_comm_open_peers(comm: *mut b200k_comm, host_all_handles: *const c_void) -> c_int;
    pub fn b200k_comm_slot(comm: *mut b200k_comm, slot: c_int, host_out_ptr: *mut *mut b200k_half) -> c_int;
    pub fn b200k_comm_allreduce_f16(
        comm: *mut b200k_comm, slot: c_int, input: *const b200k_half, output: *mut b200k_half, count: usize,
        stream: b200k_stream
    ) -> c_int;
    pub fn b200k_comm_allreduce_add_f16(
        comm: *mut b200k_comm, slot: c_int, input: *const b200k_half, addend: *const b200k_half,
        output: *mut b200k_half, count: usize, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_comm_allreduce_add_rms_norm_f16(
        comm: *mut b200k_comm, slot: c_int, input: *const b200k_half, residual: *const b200k_half,
        weight: *const b200k_half, output: *mut b200k_half, residual_out: *mut b200k_half, hidden_size: c_int,
        inv_n: f32, eps: f32, num_rows: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_comm_status(
        comm: *mut b200k_comm, host_status_out: *mut c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_comm_clear_status(comm: *mut b200k_comm, stream: b200k_stream) -> c_int;
    pub fn b200k_comm_set_timeout_cycles(comm: *mut b200k_comm, cycles: i64) -> c_int;
    pub fn b200k_comm_buffer(comm: *mut b200k_comm, host_out_ptr: *mut *mut c_void) -> c_int;
    pub fn b200k_comm_set_peer_pointer(
        comm: *mut b200k_comm, peer_rank: c_int, peer_buffer: *mut c_void
    ) -> c_int;
    pub fn b200k_comm_destroy(comm: *mut b200k_comm);
    pub fn fused_moe_a2a_slot_bytes(tokens_local: c_int, hidden: c_int, top_k: c_int, world: c_int) -> usize;
    pub fn fused_moe_gptq_a2a_f16(
        comm: *mut b200k_comm, x_local: *const b200k_half, router_logits_local: *const f32,
        w13_qweight: *const i32, w13_scales: *const b200k_half, w13_qzeros: *const i32,
        w2_qweight: *const i32, w2_scales: *const b200k_half, w2_qzeros: *const i32,
        out_local: *mut b200k_half, tokens_local: c_int, hidden: c_int, num_experts: c_int, top_k: c_int,
        intermediate: c_int, group_size: c_int, phases: c_int, workspace: *mut c_void, workspace_bytes: usize,
        stream: b200k_stream
    ) -> c_int;
    pub fn b200k_layer_set_comm(layer: *mut b200k_layer, comm: *mut b200k_comm) -> c_int;
    pub fn b200k_layer_forward(
        layer: *mut b200k_layer, hidden_in: *const b200k_half, positions: *const i32,
        hidden_out: *mut b200k_half, batch: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_layer_forward_host(
        layer: *mut b200k_layer, host_hidden_in: *const b200k_half, host_positions: *const i32,
        host_hidden_out: *mut b200k_half, batch: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_layer_forward_stage(
        layer: *mut b200k_layer, stage: c_int, hidden_in: *const b200k_half, positions: *const i32,
        reduced_in: *const b200k_half, partial_out: *mut b200k_half, hidden_out: *mut b200k_half,
        batch: c_int, stream: b200k_stream
    ) -> c_int;
    pub fn b200k_layer_launches_per_forward(layer: *const b200k_layer) -> c_int;
    pub fn b200k_device_status(host_status_out: *mut c_int, stream: b200k_stream) -> c_int;
    pub fn b200k_device_clear_status(stream: b200k_stream) -> c_int;
}

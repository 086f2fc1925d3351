/* b200_kernels.h -- C ABI of libb200_kernels.so: the LLM-decode kernel hot path of
 * sizzlecar/triton-rs (`triton-kernels` crate + the two int4 GEMM examples of
 * `triton-dsl`) as pre-built sm_100a code.
 *
 * What a caller of the reference does today, per kernel:
 *     K::<CONSTS>::mlir()                      crates/triton-dsl/src/codegen.rs:89-113
 *     -> triton_sys::Context::compile          crates/triton-sys/src/lib.rs:139
 *     -> cudarc launch_builder().arg(..)       crates/triton-runtime/examples/run_vec_add.rs:105-118
 * with the arguments in signature order, a caller-chosen grid, and two trailing
 * scratch pointers.  Here each kernel is ONE function with the same name (dtype
 * generics spelled as _f16/_f32 suffixes, the scheme the reference prelude already
 * uses, crates/triton-kernels/src/lib.rs:45-76), the same arguments in the same
 * order and the same tensor layouts, followed by
 *     - the extents the reference took from its launch grid (rows, tokens, batch),
 *     - a CUDA stream.
 * Grid, block, shared memory, tile sizes and scratch arguments are chosen inside.
 *
 * Conventions (modelled on crates/triton-sys/shim/triton_c.h:25-45,62-77: plain C
 * types, no exceptions, status + message):
 *   - every pointer is a raw device pointer (what cudarc's CudaSlice::device_ptr
 *     yields) unless the name says `host`;
 *   - return value: 0 = launched; < 0 = argument rejected on the host before any
 *     launch (B200K_E_*); > 0 = the cudaError_t of a failed launch;
 *   - b200k_last_error() returns a thread-local message for the last non-zero return;
 *   - calls are asynchronous and stream-ordered; nothing synchronises the device;
 *   - no kernel traps or asserts: device-side waits are bounded and report through
 *     a status word;
 *   - the library never falls back to host arithmetic.
 *
 * `half` below means IEEE binary16 stored as uint16_t.
 */
#ifndef B200_KERNELS_H
#define B200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint16_t b200k_half;
typedef uint16_t b200k_bf16; /* bfloat16 stored as uint16_t */
typedef void *b200k_stream; /* cudaStream_t */

enum {
    B200K_OK = 0,
    B200K_E_NULL = -1,        /* a required pointer is NULL */
    B200K_E_SHAPE = -2,       /* extent not supported (e.g. K % 8 != 0, head_dim) */
    B200K_E_ALIGN = -3,       /* pointer or stride alignment not supported */
    B200K_E_WORKSPACE = -4,   /* workspace missing or too small */
    B200K_E_DEVICE = -5,      /* current device is not sm_100 */
    B200K_E_STATE = -6        /* handle misuse */
};

const char *b200k_last_error(void);
const char *b200k_version(void);
/* 0 when the current CUDA device can run this library (compute capability 10.x). */
int b200k_device_check(void);

/* ------------------------------------------------------------------------- */
/* Workspace.  Split-K GEMM partials, split-KV attention partials and the MoE  */
/* permutation buffers live in scratch memory.  The drop-in entry points below */
/* draw it from one per-device default workspace that the library allocates on */
/* first use (cudaMalloc, B200K_DEFAULT_WORKSPACE_BYTES) or that the caller     */
/* installs with b200k_set_workspace (then the library allocates nothing).     */
/* Calls that use the default workspace must not overlap on the device: issue  */
/* them on one stream, or use the *_ws variants with a workspace per stream.   */
/* ------------------------------------------------------------------------- */
#define B200K_DEFAULT_WORKSPACE_BYTES ((size_t)256 << 20)
int b200k_set_workspace(void *workspace, size_t bytes);
size_t b200k_gemm_workspace_bytes(int m, int n, int k);
size_t b200k_attention_workspace_bytes(int batch, int num_q_heads, int num_kv_heads,
                                       int head_dim, int max_len);
/* The first word of every workspace is a status word that kernels OR bits into and never clear:
 *   bit 0 (1)  a bounded device-side wait gave up (attention pipeline);
 *   bit 1 (2)  a bounded wait of the tensor-core GEMM pipeline gave up;
 *   bit 2 (4)  a sequence length or cache position outside [0, max_len) was clamped / its row skipped.
 * b200k_workspace_status copies it to the host for a caller-owned workspace (the `_ws` entry points;
 * synchronises the stream; allocates nothing); b200k_device_status (below) does the same for the
 * default workspace; b200k_workspace_clear_status sets it back to 0. */
int b200k_workspace_status(const void *workspace, int *host_status_out, b200k_stream stream);
int b200k_workspace_clear_status(void *workspace, b200k_stream stream);

/* ------------------------------------------------------------------------- */
/* int4 W4A16 GEMM                                                             */
/* ------------------------------------------------------------------------- */

/* Replaces w4a16_gptq_gemm_typed<f16,BM,BN,BK>
 * (crates/triton-dsl/examples/w4a16_gptq_gemm_typed.rs:104-274; argument list :110-128).
 *   C[m,n] = sum_k A[m,k] * (((qweight[k/8,n] >> 4(k%8)) & 15)
 *                            - (((qzeros[k/G,n/8] >> 4(n%8)) & 15) + 1)) * scales[k/G,n]
 * fp32 accumulate, dequantised weight rounded to fp16 before the product (:256-260),
 * fp16 output.  Requires K % 8 == 0, N % 8 == 0, group_size % 8 == 0, K % group_size == 0.
 * Any element strides are accepted; the tensor-core and GEMV paths are taken when
 * stride_ak = stride_qwn = stride_sn = stride_qzn = stride_cn = 1 and the row
 * strides keep 16-byte alignment, otherwise a strided CUDA-core path runs. */
int w4a16_gptq_gemm_f16(const b200k_half *a, const int32_t *qweight, const b200k_half *scales,
                        const int32_t *qzeros, b200k_half *c, int m_size, int n_size,
                        int k_size, int group_size, int stride_am, int stride_ak,
                        int stride_qwk, int stride_qwn, int stride_sk, int stride_sn,
                        int stride_qzk, int stride_qzn, int stride_cm, int stride_cn,
                        b200k_stream stream);

/* Same contraction with the symmetric zero-point 8 and no qzeros tensor: the GEMM
 * counterpart of dequant_int4_sym_to_fp16
 * (crates/triton-dsl/examples/ferrum_dequant_int4_sym.rs:25-131, zero at :60).
 * Argument list = the GPTQ one without qzeros and its two strides. */
int w4a16_gptq_gemm_sym_f16(const b200k_half *a, const int32_t *qweight,
                            const b200k_half *scales, b200k_half *c, int m_size, int n_size,
                            int k_size, int group_size, int stride_am, int stride_ak,
                            int stride_qwk, int stride_qwn, int stride_sk, int stride_sn,
                            int stride_cm, int stride_cn, b200k_stream stream);

/* Replaces awq_gemm_int4_typed<f16,BM,BN,BK>
 * (crates/triton-dsl/examples/awq_gemm_int4_typed.rs:95-242; argument list :96-114).
 * qweight [K, N/8], qzeros [K/G, N/8]; column n sits at nibble [0,4,1,5,2,6,3,7][n%8]
 * (:137-151) in both; zeros are used as stored, no +1 (:202-205). */
int awq_gemm_int4_f16(const b200k_half *a, const int32_t *qweight, const b200k_half *scales,
                      const int32_t *qzeros, b200k_half *c, int m_size, int n_size, int k_size,
                      int group_size, int stride_am, int stride_ak, int stride_qwk,
                      int stride_qwn, int stride_sk, int stride_sn, int stride_qzk,
                      int stride_qzn, int stride_cm, int stride_cn, b200k_stream stream);

/* The same three GEMMs with an explicit workspace (b200k_gemm_workspace_bytes). */
int w4a16_gptq_gemm_f16_ws(const b200k_half *a, const int32_t *qweight,
                           const b200k_half *scales, const int32_t *qzeros, b200k_half *c,
                           int m_size, int n_size, int k_size, int group_size, int stride_am,
                           int stride_ak, int stride_qwk, int stride_qwn, int stride_sk,
                           int stride_sn, int stride_qzk, int stride_qzn, int stride_cm,
                           int stride_cn, void *workspace, size_t workspace_bytes,
                           b200k_stream stream);
int awq_gemm_int4_f16_ws(const b200k_half *a, const int32_t *qweight, const b200k_half *scales,
                         const int32_t *qzeros, b200k_half *c, int m_size, int n_size,
                         int k_size, int group_size, int stride_am, int stride_ak,
                         int stride_qwk, int stride_qwn, int stride_sk, int stride_sn,
                         int stride_qzk, int stride_qzn, int stride_cm, int stride_cn,
                         void *workspace, size_t workspace_bytes, b200k_stream stream);

/* Gate/up projection with the activation fused (no counterpart in the reference, whose consumer runs the GEMM and
 * fused_silu_mul_interleaved as two kernels): c [M, inter] = silu(a Wgate) * (a Wup) for one GPTQ weight [K, 2 inter]
 * whose first `inter` columns are the gate projection (the half-split layout of fused_silu_mul_interleaved,
 * crates/triton-kernels/src/elementwise.rs:199-206).  Contiguous tensors; tensor-core family only (K % 64,
 * inter % 64, group a power of two >= 64), other shapes are refused with B200K_E_SHAPE.  The products are not
 * rounded to fp16 before the activation, so the result is at least as close to the fp32 value as the two-kernel
 * sequence. */
int w4a16_gptq_gemm_silu_mul_f16(const b200k_half *a, const int32_t *qweight, const b200k_half *scales,
                                 const int32_t *qzeros, b200k_half *c, int m_size, int inter_size,
                                 int k_size, int group_size, b200k_stream stream);
/* GPTQ GEMM on activations whose every 8 consecutive k are stored as (k0,k4,k1,k5,k2,k6,k3,k7) -- the order in
 * which the nibble arithmetic yields a packed word's values, so the kernel skips the byte-permutes that would
 * restore k order (a contraction may visit k in any order when both operands agree).  Contiguous tensors only
 * (a [M, K], qweight [K/8, N], scales [K/G, N], qzeros [K/G, N/8] or NULL for the symmetric zero-point 8,
 * c [M, N]); same result, bit for bit, as w4a16_gptq_gemm_f16 / _sym_f16 on the unpermuted activations.
 * permute_k8_f16 produces that order from a plain [rows, K] tensor (a producer kernel that writes it directly
 * pays nothing: b200k_layer does so internally).  No counterpart in the reference. */
int permute_k8_f16(const b200k_half *input, b200k_half *output, int rows, int k_size,
                   b200k_stream stream);
int w4a16_gptq_gemm_kperm_f16(const b200k_half *a_permuted, const int32_t *qweight,
                              const b200k_half *scales, const int32_t *qzeros, b200k_half *c,
                              int m_size, int n_size, int k_size, int group_size,
                              b200k_stream stream);

/* Launch plan of the tensor-core GEMM family for a shape, without launching anything (usable without a
 * GPU): host_plan_out[10] = {token tile, dequant groups, operand-ring depth, activation-ring depth,
 * weight-ring depth, K split, K blocks per split, output tiles, MMA-issuing warps, 1 if the dequantised
 * operand tile lives in tensor memory (0: shared memory)}.  Lets host-side tests check the kernel's
 * barrier protocol for the exact ring depths that would be used.  No counterpart in the reference. */
int b200k_gemm_tc_plan(int m_size, int n_size, int k_size, int group_size, int awq,
                       int *host_plan_out);

/* Replaces dequant_int4_to_fp16<BLOCK>
 * (crates/triton-dsl/examples/ferrum_dequant_int4.rs:28-139): GPTQ full-matrix
 * dequant, output COLUMN-major out[col*K + k] (:80-89), zero = stored nibble with
 * no +1 (:76). */
int dequant_int4_to_fp16(const int32_t *qweight, const b200k_half *scales,
                         const int32_t *qzeros, b200k_half *output, int k_dim, int n_dim,
                         int group_size, int n_div_8, b200k_stream stream);
/* Replaces dequant_int4_sym_to_fp16<BLOCK>
 * (crates/triton-dsl/examples/ferrum_dequant_int4_sym.rs:25-131). */
int dequant_int4_sym_to_fp16(const int32_t *qweight, const b200k_half *scales,
                             b200k_half *output, int k_dim, int n_dim, int group_size,
                             b200k_stream stream);

/* Optional loader step for AWQ checkpoints (no counterpart in the reference, which reads the on-disk layout in every
 * call): b200k_prepack_awq rewrites qweight [K, N/8] (AWQ nibble order) once as [K/8, N] -- a word = 8 consecutive k of one
 * column, the layout of w4a16_gptq_gemm_f16 -- and qzeros [K/G, N/8] into straight nibble order; scales are used as they
 * are.  awq_gemm_int4_prepacked_f16 multiplies by such a tensor (contiguous operands) with AWQ's zero-point rule (no + 1).
 * Same values as awq_gemm_int4_f16 on the original tensor; the K-packed layout is the faster one here (16-byte loads and no
 * byte transposes in the M = 1 kernel, the dequantised operand written straight to tensor memory in the tensor-core one). */
int b200k_prepack_awq(const int32_t *qweight, const int32_t *qzeros, int32_t *qweight_packed,
                      int32_t *qzeros_packed, int k_size, int n_size, int group_size, b200k_stream stream);
int awq_gemm_int4_prepacked_f16(const b200k_half *a, const int32_t *qweight_packed, const b200k_half *scales,
                                const int32_t *qzeros_packed, b200k_half *c, int m_size, int n_size,
                                int k_size, int group_size, b200k_stream stream);

/* Bit-exact unpack probes (no counterpart kernel in the reference; they expose the
 * nibble orders its GEMMs use so that tests can compare them with ==):
 *   gptq_qweight: [K/8,N] -> int8 [K,N]          (w4a16_gptq_gemm_typed.rs:167-173)
 *   gptq_qzeros : [groups,N/8] -> int8 [groups,N], value + zero_offset   (:155-162,236)
 *   awq         : [rows,N/8] -> int8 [rows,N]     (awq_gemm_int4_typed.rs:137-151) */
int b200k_unpack_gptq_qweight(const int32_t *qweight, int8_t *out, int k_dim, int n_dim,
                              b200k_stream stream);
int b200k_unpack_gptq_qzeros(const int32_t *qzeros, int8_t *out, int groups, int n_dim,
                             int zero_offset, b200k_stream stream);
int b200k_unpack_awq(const int32_t *packed, int8_t *out, int rows, int n_dim,
                     b200k_stream stream);

/* ------------------------------------------------------------------------- */
/* decode attention                                                            */
/* ------------------------------------------------------------------------- */

/* Replaces decode_attention_typed<T,HEAD_DIM,BLOCK_KV>
 * (crates/triton-kernels/src/attention.rs:51-164): q [Hq,D], caches [seq,Hkv,D]
 * seq-major, output [Hq,D]; kv_head = q_head / (Hq/Hkv) (:68-69); fp32 softmax.
 * Positions >= valid_kv_len are excluded (the documented intent, :90-92,131-133). */
int decode_attention_f16(const b200k_half *q, const b200k_half *k_cache,
                         const b200k_half *v_cache, b200k_half *output, int num_q_heads,
                         int num_kv_heads, int head_dim, int valid_kv_len, float scale,
                         b200k_stream stream);
int decode_attention_f32(const float *q, const float *k_cache, const float *v_cache,
                         float *output, int num_q_heads, int num_kv_heads, int head_dim,
                         int valid_kv_len, float scale, b200k_stream stream);

/* Replaces decode_attention_hm_typed (attention.rs:182-273): head-major caches
 * [Hkv,capacity,D], off = kv_head*capacity*D + pos*D + d (:216-230). */
int decode_attention_hm_f16(const b200k_half *q, const b200k_half *k_cache,
                            const b200k_half *v_cache, b200k_half *output, int num_q_heads,
                            int num_kv_heads, int head_dim, int capacity, int valid_kv_len,
                            float scale, b200k_stream stream);
int decode_attention_hm_f32(const float *q, const float *k_cache, const float *v_cache,
                            float *output, int num_q_heads, int num_kv_heads, int head_dim,
                            int capacity, int valid_kv_len, float scale, b200k_stream stream);

/* Replaces batched_decode_attention_f32 (attention.rs:291-368): q [B,Hq,D], caches
 * [B,seq_len,Hkv,D] seq-major, one shared valid_kv_len.  The reference walks
 * valid_kv_len / BLOCK_KV whole tiles (:324) and asks callers to pad; this entry
 * covers all valid_kv_len positions, which is the same thing for padded callers. */
int batched_decode_attention_f32(const float *q, const float *k_cache, const float *v_cache,
                                 float *output, int batch_size, int num_q_heads,
                                 int num_kv_heads, int head_dim, int seq_len,
                                 int valid_kv_len, float scale, b200k_stream stream);

/* The follow-up the reference names at attention.rs:287-289 (per-sequence lengths),
 * on the head-major layout of decode_attention_hm: q [B,Hq,D], caches
 * [B,Hkv,max_len,D], context_lens [B] int32, output [B,Hq,D].  No counterpart
 * kernel in the reference.  Split-KV over a work list of fixed-size chunks, all q
 * heads of a GQA group per KV read, then a combine pass. */
int batched_decode_attention_hm_f16(const b200k_half *q, const b200k_half *k_cache,
                                    const b200k_half *v_cache, const int32_t *context_lens,
                                    b200k_half *output, int batch_size, int num_q_heads,
                                    int num_kv_heads, int head_dim, int max_len, float scale,
                                    b200k_stream stream);
int batched_decode_attention_hm_f16_ws(const b200k_half *q, const b200k_half *k_cache,
                                       const b200k_half *v_cache, const int32_t *context_lens,
                                       b200k_half *output, int batch_size, int num_q_heads,
                                       int num_kv_heads, int head_dim, int max_len,
                                       float scale, void *workspace, size_t workspace_bytes,
                                       b200k_stream stream);

/* batched_decode_attention_hm_f16 for callers that must not allocate device memory: an engine
 * that has handed the whole GPU to its own arena, a plugin running inside someone else's
 * allocator, or a host that may not call cudaMalloc once serving has started.  It has no
 * counterpart in the reference.  The split-KV partials go to a fixed array that is part of the
 * library image (B200K_NOALLOC_SCRATCH_BYTES per GPU) instead of the workspace; the call performs
 * no cudaMalloc, cudaFree or other allocating call.  The array becomes resident when the CUDA
 * runtime loads the module that holds it, which with lazy module loading (the default) is the
 * first use of this part of the library on that GPU, and stays until the process exits: an engine
 * that is about to claim the rest of the GPU for its own arena should make one call first (a call
 * with batch_size 0 is enough: it looks the array up and launches nothing).
 *   - Shapes whose scratch need (b200k_attention_workspace_bytes) exceeds the array are rejected
 *     with B200K_E_WORKSPACE and a message naming both sizes; nothing is launched.
 *   - The first call on each device looks the array's address up (that device must be current):
 *     make that call before any stream capture begins.
 *   - All calls on a device share the one array.  Its arrival counters are left at zero by every
 *     call, so back-to-back calls on one stream are fine; calls that may run at the same time
 *     on the same GPU (different streams) race on it and must not be made.
 *   - b200k_noalloc_status reads the array's status word (same bits as b200k_workspace_status; a
 *     bounded wait that gave up on this path reports there); it allocates nothing either. */
#define B200K_NOALLOC_SCRATCH_BYTES (8u << 20)
int batched_decode_attention_hm_f16_noalloc(const b200k_half *q, const b200k_half *k_cache,
                                            const b200k_half *v_cache, const int32_t *context_lens,
                                            b200k_half *output, int batch_size, int num_q_heads,
                                            int num_kv_heads, int head_dim, int max_len, float scale,
                                            b200k_stream stream);

int b200k_noalloc_status(int *host_status_out, b200k_stream stream);

/* Replaces flash_decode_attn_phase1_f32<HEAD_DIM,BLOCK_KV> (attention.rs:508-585):
 * split s of q head h covers chunk_blocks*block_kv positions from
 * s*chunk_blocks*block_kv, chunk_blocks = (valid_kv_len/num_splits)/block_kv (:538);
 * writes un-normalised partial_acc [Hq,S,D], partial_max [Hq,S], partial_sum [Hq,S]
 * (:579-584).  block_kv is the reference's BLOCK_KV const generic. */
int flash_decode_attn_phase1_f32(const float *q, const float *k_cache, const float *v_cache,
                                 float *partial_acc, float *partial_max, float *partial_sum,
                                 int num_q_heads, int num_kv_heads, int head_dim,
                                 int valid_kv_len, int num_splits, float scale, int block_kv,
                                 b200k_stream stream);
/* Replaces batched_flash_decode_attn_phase1_f32 (attention.rs:663-747). */
int batched_flash_decode_attn_phase1_f32(const float *q, const float *k_cache,
                                         const float *v_cache, float *partial_acc,
                                         float *partial_max, float *partial_sum,
                                         int batch_size, int num_q_heads, int num_kv_heads,
                                         int head_dim, int seq_len, int valid_kv_len,
                                         int num_splits, float scale, int block_kv,
                                         b200k_stream stream);
/* Replaces flash_decode_attn_phase2_f32<HEAD_DIM,NUM_SPLITS_TILE> (attention.rs:599-642):
 * M = max m_s; L = sum l_s e^(m_s-M); out = sum acc_s e^(m_s-M) / L.  The batched
 * caller flattens batch into num_q_heads (:659-661). */
int flash_decode_attn_phase2_f32(const float *partial_acc, const float *partial_max,
                                 const float *partial_sum, float *output, int num_q_heads,
                                 int head_dim, int num_splits, b200k_stream stream);

/* Replaces paged_decode_attention_typed (attention.rs:399-490): pools
 * [max_blocks,block_size,Hkv,D]; phys = block_table[pos/block_size] (:450-455). */
int paged_decode_attention_f16(const b200k_half *q, const b200k_half *k_block_pool,
                               const b200k_half *v_block_pool, const int32_t *block_table,
                               b200k_half *output, int num_q_heads, int num_kv_heads,
                               int head_dim, int valid_kv_len, int block_size, float scale,
                               b200k_stream stream);

/* Replaces unified_attention_f32 (crates/triton-kernels/src/attention.rs:988-1187): prefill and decode in one
 * call over a paged KV pool.  q / output [total_tokens, num_q_heads, D] token-major; k/v_cache
 * [num_blocks, block_size, num_kv_heads, D]; block_table [num_seqs, max_blocks_per_seq]; seq_lens [num_seqs];
 * query_start_loc [num_seqs + 1] (CSR offsets of each sequence's query tokens, which are the last q_len
 * positions of its KV stream).  Causal: query token j of a sequence sees kv positions
 * 0 .. seq_len - q_len + j.  The reference walks the KV stream in BLOCK_KV tiles and drops a ragged tail
 * (seq_len / BLOCK_KV tiles, :1069); here every position below seq_len is used, which is the same
 * thing whenever the caller keeps seq_len a multiple of its tile as that kernel asks.  num_seqs (the
 * reference's grid extent) is the trailing argument; D <= 256. */
int unified_attention_f32(const float *q, const float *k_cache, const float *v_cache,
                          float *output, const int32_t *block_table, const int32_t *seq_lens,
                          const int32_t *query_start_loc, int num_q_heads, int num_kv_heads,
                          int head_dim, int block_size, int max_blocks_per_seq, float sm_scale,
                          int num_seqs, b200k_stream stream);

/* Replaces flash_attn_full<T, HEAD_DIM, BLOCK_Q, BLOCK_KV> (crates/triton-kernels/src/attention.rs:780-909): causal
 * prefill attention.  q / output [batch, num_heads, q_len, D]; k / v [batch, num_kv_heads, kv_len, D] (all
 * contiguous); query row i sees kv positions 0 .. pos_offset + i.  Arguments in the reference's order, with the
 * grid's batch extent made an explicit argument after `output`.  All arithmetic in fp32 for either element type
 * (:773-779).  The reference asks for q_len and kv_len to be multiples of its tiles; any length is accepted
 * here, and masked positions contribute exactly 0 (its -1e30 additive mask underflows to the same).  D <= 256.
 * The 16-bit editions at head_dim 128 (pos_offset >= 0, scale > 0) run on the tensor cores: scores and output
 * accumulate in fp32, the probabilities enter the second product rounded to the element type. */
int flash_attn_full_f32(const float *q, const float *k, const float *v, float *output, int batch,
                        int num_heads, int num_kv_heads, int q_len, int kv_len, int head_dim,
                        int pos_offset, float scale, b200k_stream stream);
int flash_attn_full_f16(const b200k_half *q, const b200k_half *k, const b200k_half *v,
                        b200k_half *output, int batch, int num_heads, int num_kv_heads, int q_len,
                        int kv_len, int head_dim, int pos_offset, float scale, b200k_stream stream);

/* ------------------------------------------------------------------------- */
/* Projection helpers either side of attention (crates/triton-kernels/src/projection.rs), fp32 as in */
/* the reference.  Its const generics (BLOCK, HEAD_DIM, HALF_DIM) are tile limits there and runtime    */
/* extents here: HALF_DIM = head_dim / 2 (the tables are [positions, head_dim / 2]); the launch grid   */
/* of the reference becomes the trailing extent argument where the signature does not already have it. */
/* ------------------------------------------------------------------------- */
/* Replaces split_qkv_f32 (projection.rs:18-51): qkv [batch, 3, heads, D] -> q, k, v [batch, heads, D]. */
int split_qkv_f32(const float *qkv, float *q_out, float *k_out, float *v_out, int num_heads,
                  int head_dim, int batch, b200k_stream stream);
/* Replace transpose_head_to_token_f32 (:60-79): [heads, tokens, D] -> [tokens, heads, D], and
 * transpose_token_to_head_f32 (:87-105): the inverse. */
int transpose_head_to_token_f32(const float *input, float *output, int tokens, int heads,
                                int head_dim, b200k_stream stream);
int transpose_token_to_head_f32(const float *input, float *output, int tokens, int heads,
                                int head_dim, b200k_stream stream);
/* Replaces qk_norm_rope_transpose_f32 (:119-175): per (token, head) RMS norm with norm_w [D] (caller passes
 * inv_n = 1 / D), RoPE on the pairs (i, i + D/2) with tables row pos_offset + token, stored head-major
 * [heads, tokens, D]. */
int qk_norm_rope_transpose_f32(const float *input, const float *norm_w, const float *cos_tab,
                               const float *sin_tab, float *output, int tokens, int heads,
                               int head_dim, int pos_offset, float inv_n, float eps,
                               b200k_stream stream);
/* Replaces rope_transpose_f32 (:182-215): the same without the norm. */
int rope_transpose_f32(const float *input, const float *cos_tab, const float *sin_tab,
                       float *output, int tokens, int heads, int head_dim, int pos_offset,
                       b200k_stream stream);

/* ------------------------------------------------------------------------- */
/* fused MoE                                                                   */
/* ------------------------------------------------------------------------- */
/* The reference has no MoE kernel (a search of its tree finds two comment mentions,
 * crates/triton-dsl/examples/awq_gemm_int4_typed.rs:63 and
 * crates/triton-kernels/src/elementwise.rs:222); these entry points follow its conventions for
 * the parts: GPTQ layout and +1 zero rule of w4a16_gptq_gemm_typed, half-split gate|up rows of
 * fused_silu_mul_interleaved (elementwise.rs:199-206).
 *
 * moe_route_topk_f32: fp32 softmax over experts, top-k (ties: lowest expert index), weights
 * renormalised to sum 1.  topk_ids [T,k] int32, topk_weights [T,k] fp32.
 * moe_permute: pair p = t*k + j.  counts [E], offsets [E+1], sorted_pairs [T*k] = pair indices by
 * expert then by pair index, inverse [T*k] = position of each pair in that order.
 * fused_moe_gptq_f16: x [T,H] fp16, router_logits [T,E] fp32, stacked expert weights
 * w13_qweight [E, H/8, 2I] (gate columns then up columns), w13_scales [E, H/G, 2I],
 * w2_qweight [E, I/8, H], w2_scales [E, I/G, H]; qzeros [E, K/G, N/8] or NULL for the symmetric
 * zero-point 8; out[t] = sum_j w[t,j] * (silu(g) * u) W2_e.  workspace NULL = default workspace
 * (fused_moe_workspace_bytes says how much is used). */
int moe_route_topk_f32(const float *router_logits, int32_t *topk_ids, float *topk_weights,
                       int num_tokens, int num_experts, int top_k, b200k_stream stream);
int moe_permute(const int32_t *topk_ids, int32_t *counts, int32_t *offsets, int32_t *sorted_pairs,
                int32_t *inverse, int num_pairs, int num_experts, b200k_stream stream);
size_t fused_moe_workspace_bytes(int num_tokens, int hidden, int num_experts, int top_k,
                                 int intermediate);
int fused_moe_gptq_f16(const b200k_half *x, const float *router_logits, const int32_t *w13_qweight,
                       const b200k_half *w13_scales, const int32_t *w13_qzeros,
                       const int32_t *w2_qweight, const b200k_half *w2_scales,
                       const int32_t *w2_qzeros, b200k_half *out, int num_tokens, int hidden,
                       int num_experts, int top_k, int intermediate, int group_size,
                       void *workspace, size_t workspace_bytes, b200k_stream stream);

/* Expert-parallel share of the same computation: this call holds the weights of experts
 * [expert_first, expert_first + num_local_experts) only (stacks of num_local_experts matrices).  Tokens
 * and router logits are the full, replicated ones; routing is computed over all num_experts (identically
 * on every rank), pairs routed to other ranks' experts are dropped, and partial_out [num_tokens, hidden]
 * receives the weighted sum over the local experts (zero rows for tokens with none).  The sum of
 * partial_out over the ranks is the MoE output: one all-reduce (b200k_comm_allreduce_f16), no all-to-all
 * and no size exchange.  No counterpart in the reference. */
int fused_moe_gptq_ep_f16(const b200k_half *x, const float *router_logits,
                          const int32_t *w13_qweight, const b200k_half *w13_scales,
                          const int32_t *w13_qzeros, const int32_t *w2_qweight,
                          const b200k_half *w2_scales, const int32_t *w2_qzeros,
                          b200k_half *partial_out, int num_tokens, int hidden, int num_experts,
                          int expert_first, int num_local_experts, int top_k, int intermediate,
                          int group_size, void *workspace, size_t workspace_bytes,
                          b200k_stream stream);

/* ------------------------------------------------------------------------- */
/* bandwidth-bound glue                                                        */
/* ------------------------------------------------------------------------- */

/* Replace rms_norm_f16 / rms_norm_f32 (crates/triton-kernels/src/norms.rs:125-150,
 * 16-41): y = x * rsqrt(sum(x^2)*inv_n + eps) * w, reduction in fp32.  num_rows is
 * the reference's launch grid. */
int rms_norm_f16(const b200k_half *input, const b200k_half *weight, b200k_half *output,
                 int row_size, float inv_n, float eps, int num_rows, b200k_stream stream);
int rms_norm_f32(const float *input, const float *weight, float *output, int row_size,
                 float inv_n, float eps, int num_rows, b200k_stream stream);

/* Replace fused_add_rms_norm_f16 / _f32 (norms.rs:189-220, 85-115): r = x + res;
 * residual_out = r; output = rms_norm(r) from the unrounded fp32 sum (:208-219). */
int fused_add_rms_norm_f16(const b200k_half *input, const b200k_half *residual,
                           const b200k_half *weight, b200k_half *output,
                           b200k_half *residual_out, int hidden_size, float inv_n, float eps,
                           int num_rows, b200k_stream stream);
int fused_add_rms_norm_f32(const float *input, const float *residual, const float *weight,
                           float *output, float *residual_out, int hidden_size, float inv_n,
                           float eps, int num_rows, b200k_stream stream);

/* Replace residual_add_f16/_f32 and residual_add_inplace_f16/_f32
 * (crates/triton-kernels/src/elementwise.rs:62-74, 46-58, 95-107, 79-91). */
int residual_add_f16(const b200k_half *a, const b200k_half *b, b200k_half *out, int n,
                     b200k_stream stream);
int residual_add_f32(const float *a, const float *b, float *out, int n, b200k_stream stream);
int residual_add_inplace_f16(b200k_half *a, const b200k_half *b, int n, b200k_stream stream);
int residual_add_inplace_f32(float *a, const float *b, int n, b200k_stream stream);

/* Replace fused_silu_mul_f16/_f32 (elementwise.rs:169-184, 148-164) and
 * fused_silu_mul_interleaved_f16/_f32 (:188-212, 225-250): silu(g) = g/(1+e^-g) in
 * fp32; interleaved = row b of gate_up [B, 2*inter] holds gate then up (:199-206). */
int fused_silu_mul_f16(const b200k_half *gate, const b200k_half *up, b200k_half *out, int n,
                       b200k_stream stream);
int fused_silu_mul_f32(const float *gate, const float *up, float *out, int n,
                       b200k_stream stream);
int fused_silu_mul_interleaved_f16(const b200k_half *gate_up, b200k_half *out, int inter,
                                   int total, b200k_stream stream);
int fused_silu_mul_interleaved_f32(const float *gate_up, float *out, int inter, int total,
                                   b200k_stream stream);

/* Replace rope_q_f32 / rope_k_f32 (crates/triton-kernels/src/positional.rs:24-80):
 * one position, tables [D/2] already sliced; pairs (i, i+D/2) (:45-46).  num_heads is
 * the reference's launch grid. */
int rope_q_f32(const float *q, const float *cos_table, const float *sin_table, float *q_out,
               int head_dim, int num_heads, b200k_stream stream);
int rope_k_f32(const float *k, const float *cos_table, const float *sin_table, float *k_out,
               int head_dim, int num_heads, b200k_stream stream);
/* Replaces rope_full_f32 (positional.rs:94-129): x [tokens,heads,D], tables
 * [max_pos,D/2], positions [tokens] int32.  num_tokens is grid / num_heads. */
int rope_full_f32(const float *q, const float *cos_table, const float *sin_table,
                  const int32_t *positions, float *q_out, int num_heads, int head_dim,
                  int num_tokens, b200k_stream stream);
/* fp16 edition of rope_full (tables stay fp32, arithmetic fp32, one rounding at the
 * store); the reference ships f32 only. */
int rope_full_f16(const b200k_half *q, const float *cos_table, const float *sin_table,
                  const int32_t *positions, b200k_half *q_out, int num_heads, int head_dim,
                  int num_tokens, b200k_stream stream);

/* Replaces kv_cache_append_f32<BLOCK> (crates/triton-kernels/src/cache.rs:21-47):
 * new_keys/values [B,H,D] -> caches [max_seq,H,D] at row cache_idx[b] (:38-46).
 * batch is grid / num_heads. */
int kv_cache_append_f32(const float *new_keys, const float *new_values, float *k_cache,
                        float *v_cache, const int32_t *cache_idx, int num_heads, int head_dim,
                        int batch, b200k_stream stream);
/* Batched head-major fp16 edition for the cache layout of
 * batched_decode_attention_hm_f16: caches [B,H,max_len,D], row (b,h) goes to
 * [b,h,cache_idx[b],:].  No counterpart kernel in the reference. */
int kv_cache_append_hm_f16(const b200k_half *new_keys, const b200k_half *new_values,
                           b200k_half *k_cache, b200k_half *v_cache, const int32_t *cache_idx,
                           int num_heads, int head_dim, int max_len, int batch,
                           b200k_stream stream);
/* rope_full on q and k + kv_cache_append_hm in one pass over a fused QKV row
 * [B, (Hq+2Hkv)*D] (q heads, then k heads, then v heads): q_out [B,Hq,D] rotated,
 * k rotated and v copied into the caches at positions[b].  Fusion of
 * positional.rs:94-129 and cache.rs:21-47; no counterpart kernel in the reference. */
int rope_kv_append_hm_f16(const b200k_half *qkv, const float *cos_table,
                          const float *sin_table, const int32_t *positions,
                          b200k_half *q_out, b200k_half *k_cache, b200k_half *v_cache,
                          int num_q_heads, int num_kv_heads, int head_dim, int max_len,
                          int batch, b200k_stream stream);

/* ------------------------------------------------------------------------- */
/* bf16 editions                                                               */
/* ------------------------------------------------------------------------- */
/* The reference's `_typed` kernels are generic over T = f32 / f16 / bf16
 * (crates/triton-dsl/examples/w4a16_gptq_gemm_typed.rs:65-67,
 * crates/triton-dsl/tests/proc_macro_ferrum_typed.rs:6-19).  Same arguments as the _f16 entry points
 * with bf16 tensors; arithmetic in fp32 inside, one rounding to bf16 at the store. */
/* The two int4 GEMMs with bf16 activations, scales and output (dequantised weight rounded to bf16 before the
 * product, as the reference's as_t::<T> does); qzeros NULL in the GPTQ edition = symmetric zero-point 8. */
int w4a16_gptq_gemm_bf16(const b200k_bf16 *a, const int32_t *qweight, const b200k_bf16 *scales,
                         const int32_t *qzeros, b200k_bf16 *c, int m_size, int n_size, int k_size,
                         int group_size, int stride_am, int stride_ak, int stride_qwk,
                         int stride_qwn, int stride_sk, int stride_sn, int stride_qzk,
                         int stride_qzn, int stride_cm, int stride_cn, b200k_stream stream);
int awq_gemm_int4_bf16(const b200k_bf16 *a, const int32_t *qweight, const b200k_bf16 *scales,
                       const int32_t *qzeros, b200k_bf16 *c, int m_size, int n_size, int k_size,
                       int group_size, int stride_am, int stride_ak, int stride_qwk,
                       int stride_qwn, int stride_sk, int stride_sn, int stride_qzk,
                       int stride_qzn, int stride_cm, int stride_cn, b200k_stream stream);
/* decode_attention_typed / _hm_typed / paged_decode_attention_typed with T = bf16 (fp32 arithmetic inside). */
int decode_attention_bf16(const b200k_bf16 *q, const b200k_bf16 *k_cache, const b200k_bf16 *v_cache,
                          b200k_bf16 *output, int num_q_heads, int num_kv_heads, int head_dim,
                          int valid_kv_len, float scale, b200k_stream stream);
int decode_attention_hm_bf16(const b200k_bf16 *q, const b200k_bf16 *k_cache,
                             const b200k_bf16 *v_cache, b200k_bf16 *output, int num_q_heads,
                             int num_kv_heads, int head_dim, int capacity, int valid_kv_len,
                             float scale, b200k_stream stream);
int paged_decode_attention_bf16(const b200k_bf16 *q, const b200k_bf16 *k_block_pool,
                                const b200k_bf16 *v_block_pool, const int32_t *block_table,
                                b200k_bf16 *output, int num_q_heads, int num_kv_heads,
                                int head_dim, int valid_kv_len, int block_size, float scale,
                                b200k_stream stream);
int rms_norm_bf16(const b200k_bf16 *input, const b200k_bf16 *weight, b200k_bf16 *output,
                  int row_size, float inv_n, float eps, int num_rows, b200k_stream stream);
int fused_add_rms_norm_bf16(const b200k_bf16 *input, const b200k_bf16 *residual,
                            const b200k_bf16 *weight, b200k_bf16 *output,
                            b200k_bf16 *residual_out, int hidden_size, float inv_n, float eps,
                            int num_rows, b200k_stream stream);
int residual_add_bf16(const b200k_bf16 *a, const b200k_bf16 *b, b200k_bf16 *out, int n,
                      b200k_stream stream);
int residual_add_inplace_bf16(b200k_bf16 *a, const b200k_bf16 *b, int n, b200k_stream stream);
int fused_silu_mul_bf16(const b200k_bf16 *gate, const b200k_bf16 *up, b200k_bf16 *out, int n,
                        b200k_stream stream);
int fused_silu_mul_interleaved_bf16(const b200k_bf16 *gate_up, b200k_bf16 *out, int inter,
                                    int total, b200k_stream stream);
int rope_full_bf16(const b200k_bf16 *q, const float *cos_table, const float *sin_table,
                   const int32_t *positions, b200k_bf16 *q_out, int num_heads, int head_dim,
                   int num_tokens, b200k_stream stream);
int kv_cache_append_hm_bf16(const b200k_bf16 *new_keys, const b200k_bf16 *new_values,
                            b200k_bf16 *k_cache, b200k_bf16 *v_cache, const int32_t *cache_idx,
                            int num_heads, int head_dim, int max_len, int batch,
                            b200k_stream stream);
int embedding_lookup_bf16(const b200k_bf16 *embeddings, const int32_t *indices,
                          b200k_bf16 *output, int hidden_size, int num_tokens,
                          b200k_stream stream);
int softmax_bf16(const b200k_bf16 *input, b200k_bf16 *output, int rows, int cols,
                 b200k_stream stream);
/* flash_attn_full with T = bf16 (tensor-core path at head_dim 128, as for fp16). */
int flash_attn_full_bf16(const b200k_bf16 *q, const b200k_bf16 *k, const b200k_bf16 *v,
                         b200k_bf16 *output, int batch, int num_heads, int num_kv_heads, int q_len,
                         int kv_len, int head_dim, int pos_offset, float scale,
                         b200k_stream stream);

/* ------------------------------------------------------------------------- */
/* the two ends of a decode step                                               */
/* ------------------------------------------------------------------------- */
/* Replace embedding_lookup_f32 / _f16 (crates/triton-kernels/src/embedding.rs:17-55):
 * output[tok, :] = embeddings[indices[tok], :], rows of hidden_size elements.  num_tokens is the
 * reference's launch grid; its BLOCK >= hidden_size limit is gone.  The table's row count is not an
 * argument (it is not one in the reference either), so indices are the caller's responsibility. */
int embedding_lookup_f32(const float *embeddings, const int32_t *indices, float *output,
                         int hidden_size, int num_tokens, b200k_stream stream);
int embedding_lookup_f16(const b200k_half *embeddings, const int32_t *indices, b200k_half *output,
                         int hidden_size, int num_tokens, b200k_stream stream);
/* Replace softmax_f32 / _f16 (crates/triton-kernels/src/reduction.rs:11-68): row softmax,
 * out[r,c] = exp(x[r,c] - max_r) / sum_c exp(x[r,c] - max_r), fp32 arithmetic for either element
 * type, any cols (the reference needs cols <= BLOCK and, through its zero-filled masked loads, counts
 * the BLOCK - cols padding lanes in the sum when cols < BLOCK; this entry sums over cols only, which is
 * the documented formula and what the reference computes whenever cols == BLOCK, as in its own check,
 * crates/triton-runtime/examples/run_softmax.rs:20-21). */
int softmax_f32(const float *input, float *output, int rows, int cols, b200k_stream stream);
int softmax_f16(const b200k_half *input, b200k_half *output, int rows, int cols,
                b200k_stream stream);

/* ------------------------------------------------------------------------- */
/* decode layer chain                                                          */
/* ------------------------------------------------------------------------- */
/* The reference holds the kernels but not the loop that strings them together: its
 * consumer calls about a dozen launches per layer in the order shown by
 * crates/triton-core/examples/ferrum_integration_demo.rs:52-108.  This handle is that
 * call sequence for one Llama-shape decode layer, kept inside the library so that it
 * can be captured once in a CUDA graph and replayed:
 *   rms_norm -> QKV int4 GEMM -> RoPE + kv_cache_append -> decode attention -> o_proj
 *   -> [all-reduce] -> residual add + rms_norm -> gate_up int4 GEMM -> silu_mul ->
 *   down int4 GEMM -> [all-reduce] -> residual add
 * All extents are the LOCAL ones of a tensor-parallel rank (q heads, kv heads and
 * intermediate columns already divided by the world size); weights are GPTQ
 * (qzeros NULL = symmetric zero-point 8) or AWQ, caller-owned and not copied.
 * No counterpart in the reference. */
typedef struct b200k_layer b200k_layer;
typedef struct b200k_layer_config {
    int hidden;          /* model width H */
    int num_q_heads;     /* local */
    int num_kv_heads;    /* local */
    int head_dim;        /* 128 */
    int intermediate;    /* local */
    int group_size;
    int weight_format;   /* 0 = GPTQ, 1 = AWQ */
    int max_batch;
    int max_len;         /* KV cache rows per (sequence, kv head) */
    float rms_eps;
    int use_graph;       /* capture the call in a CUDA graph on first use per (batch size, buffer addresses):
                          * a decode loop that reuses its buffers replays one graph, copies included */
    int reserved[5];     /* zero */
} b200k_layer_config;

int b200k_layer_create(const b200k_layer_config *config, b200k_layer **out_layer);
void b200k_layer_destroy(b200k_layer *layer);
/* which: 0 = qkv [H, (Hq+2Hkv)*D], 1 = o [Hq*D, H], 2 = gate_up [H, 2*I] (gate columns then
 * up columns), 3 = down [I, H].  Packed layouts as in the GEMM entry points. */
int b200k_layer_set_weight(b200k_layer *layer, int which, const int32_t *qweight,
                           const b200k_half *scales, const int32_t *qzeros);
/* ln1/ln2 [H] fp16; cos/sin [max_pos, D/2] fp32 (rope_full_f32's tables). */
int b200k_layer_set_norms_rope(b200k_layer *layer, const b200k_half *ln1, const b200k_half *ln2,
                               const float *cos_table, const float *sin_table);
/* caches [max_batch, num_kv_heads, max_len, D] fp16 head-major, caller-owned. */
int b200k_layer_set_kv_cache(b200k_layer *layer, b200k_half *k_cache, b200k_half *v_cache);
/* ---- tensor-parallel exchange: one-shot all-reduce over NVLink peer memory -----------------------
 * No counterpart in the reference, which is single-GPU (its consumer would call NCCL).  One process
 * per GPU.  Each rank creates an exchange buffer (flags + two slots of slot_bytes), publishes its
 * 64-byte CUDA IPC handle, and maps the handles of all ranks (host_all_handles = world x 64 bytes in
 * rank order; how they travel between processes is the caller's business, e.g. an all-gather over
 * the process group).  world <= 8, one node.
 * b200k_comm_allreduce_f16 sums `count` fp16 values (multiple of 8) held in slot `slot` of every
 * rank, fp32 accumulation in rank order, every rank gets identical bits in `output` (local memory).
 * `input` non-NULL is first copied into the slot; NULL means the producer wrote the slot directly
 * (b200k_comm_slot).  Every rank must make the same sequence of calls; use slots alternately (a slot
 * may be rewritten once a LATER all-reduce has been enqueued behind the one that read it).  The
 * kernel waits for its peers at most about a second, then sets the status word (b200k_comm_status
 * != 0) and leaves `output` unwritten.  Plain peer loads and stores only.
 * Large tensors on three or more ranks (b200k_comm_allreduce_f16 and _add_f16) take a two-shot form:
 * every rank reduces one share and stores it into the OTHER slot of all ranks, a second round of
 * flags, then a local copy; same bits, a fraction of the NVLink traffic.  The other slot's content
 * is therefore lost during such a call -- which the alternation rule already allows. */
struct b200k_comm;
int b200k_comm_create(int rank, int world, size_t slot_bytes, struct b200k_comm **out_comm);
int b200k_comm_ipc_handle(struct b200k_comm *comm, void *host_handle_64_bytes);
int b200k_comm_open_peers(struct b200k_comm *comm, const void *host_all_handles);
int b200k_comm_slot(struct b200k_comm *comm, int slot, b200k_half **host_out_ptr);
int b200k_comm_allreduce_f16(struct b200k_comm *comm, int slot, const b200k_half *input, b200k_half *output,
                             size_t count, b200k_stream stream);
/* The all-reduce fused with the step that consumes it in a tensor-parallel layer (same protocol, same slot rules):
 *   _add_f16           output = addend + fp16(sum over ranks)              (the closing residual add)
 *   _add_rms_norm_f16  r = residual + fp16(sum over ranks); residual_out = fp16(r);
 *                      output = rms_norm(r) from the unrounded r: the arithmetic of fused_add_rms_norm_f16
 *                      (crates/triton-kernels/src/norms.rs:189-220) on the reduced tensor; one CTA per row,
 *                      hidden_size a multiple of 8 up to 32768.
 * Bit-identical to the plain all-reduce followed by residual_add_f16 / fused_add_rms_norm_f16. */
int b200k_comm_allreduce_add_f16(struct b200k_comm *comm, int slot, const b200k_half *input,
                                 const b200k_half *addend, b200k_half *output, size_t count,
                                 b200k_stream stream);
int b200k_comm_allreduce_add_rms_norm_f16(struct b200k_comm *comm, int slot, const b200k_half *input,
                                          const b200k_half *residual, const b200k_half *weight,
                                          b200k_half *output, b200k_half *residual_out, int hidden_size,
                                          float inv_n, float eps, int num_rows, b200k_stream stream);
int b200k_comm_status(struct b200k_comm *comm, int *host_status_out, b200k_stream stream);
int b200k_comm_clear_status(struct b200k_comm *comm, b200k_stream stream);
/* How long a kernel waits for its peers, in SM clock cycles (default 2e9, about a second; <= 0 restores it). */
int b200k_comm_set_timeout_cycles(struct b200k_comm *comm, int64_t cycles);
/* For ranks that live in ONE process (several GPUs with peer access enabled by the caller, or a test that
 * stands a second buffer in for a peer): b200k_comm_buffer yields this rank's exchange buffer,
 * b200k_comm_set_peer_pointer installs a peer's buffer directly instead of an IPC mapping. */
int b200k_comm_buffer(struct b200k_comm *comm, void **host_out_ptr);
int b200k_comm_set_peer_pointer(struct b200k_comm *comm, int peer_rank, void *peer_buffer);
void b200k_comm_destroy(struct b200k_comm *comm);
/* Expert parallelism by token exchange (dispatch / combine): rank r of the group holds tokens_local tokens and the
 * experts [r E/N, (r + 1) E/N) (w13 / w2 stacks of E/N matrices, layouts as fused_moe_gptq_f16).  Every rank makes the
 * same call; a call routes the local tokens, writes each (token, choice) row into the exchange buffer of the rank that
 * owns the expert (peer stores), runs the local experts on what it received, and gathers the k result rows of each
 * local token from their owners (peer loads) with the routing weights: out_local [tokens_local, H].  Per rank
 * tokens_local * top_k rows travel each way, against the (N - 1) * N * tokens_local rows read by the all-reduce of
 * fused_moe_gptq_ep_f16 partial outputs.  The exchange buffer's slots must hold fused_moe_a2a_slot_bytes(...) bytes
 * (b200k_comm_create); num_experts % N == 0.  Waits for peers are bounded (b200k_comm_set_timeout_cycles) and report
 * through b200k_comm_status.  `phases`: 7 in a real group (one process per GPU).  The bits run the three phases
 * separately -- 1 dispatch, 2 experts, 4 combine, each waiting only for what earlier phases of the other ranks
 * published -- so that a harness holding every rank's buffers on one GPU can run phase by phase over the ranks;
 * kernels that wait for one another must never be queued in the other order on one GPU.  workspace: as
 * fused_moe_gptq_f16, sized by fused_moe_workspace_bytes(N * tokens_local, ...); ranks that share a GPU need one each.
 * No counterpart in the reference. */
size_t fused_moe_a2a_slot_bytes(int tokens_local, int hidden, int top_k, int world);
int fused_moe_gptq_a2a_f16(struct b200k_comm *comm, const b200k_half *x_local, const float *router_logits_local,
                           const int32_t *w13_qweight, const b200k_half *w13_scales, const int32_t *w13_qzeros,
                           const int32_t *w2_qweight, const b200k_half *w2_scales, const int32_t *w2_qzeros,
                           b200k_half *out_local, int tokens_local, int hidden, int num_experts, int top_k,
                           int intermediate, int group_size, int phases, void *workspace,
                           size_t workspace_bytes, b200k_stream stream);
/* Attach to a layer: the o and down GEMMs then write into slots 0 and 1 and the layer chain runs the
 * two all-reduces itself, each fused with the step that consumes it (10 launches, as on one GPU).
 * NULL detaches (single GPU). */
int b200k_layer_set_comm(b200k_layer *layer, struct b200k_comm *comm);

/* Whole layer on device buffers: hidden_in/out [batch, H] fp16, positions [batch] int32
 * (the row each sequence appends at; attention then covers positions[b]+1 rows). */
int b200k_layer_forward(b200k_layer *layer, const b200k_half *hidden_in, const int32_t *positions,
                        b200k_half *hidden_out, int batch, b200k_stream stream);
/* The same through HOST buffers (pinned memory for full copy speed): copies the inputs
 * in, runs the layer, copies the result out, all on `stream`; returns after enqueueing. */
int b200k_layer_forward_host(b200k_layer *layer, const b200k_half *host_hidden_in,
                             const int32_t *host_positions, b200k_half *host_hidden_out,
                             int batch, b200k_stream stream);
/* The chain in three pieces, for callers that run their own collective (e.g. NCCL)
 * between them.  stage 0: up to and including o_proj, partial sums into partial_out
 * [batch,H]; stage 1: takes the reduced o_proj output in reduced_in, up to and including
 * the down GEMM, partial sums into partial_out; stage 2: final residual add of
 * reduced_in into hidden_out. */
int b200k_layer_forward_stage(b200k_layer *layer, int stage, const b200k_half *hidden_in,
                              const int32_t *positions, const b200k_half *reduced_in,
                              b200k_half *partial_out, b200k_half *hidden_out, int batch,
                              b200k_stream stream);
/* Number of kernel launches one forward call issues (for launch accounting). */
int b200k_layer_launches_per_forward(const b200k_layer *layer);
/* Reads the device status word of the default workspace (0 = nothing to report; bits as listed at
 * b200k_workspace_status).  Synchronises the stream. */
int b200k_device_status(int *host_status_out, b200k_stream stream);
/* Sets that word back to 0 (stream-ordered). */
int b200k_device_clear_status(b200k_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_KERNELS_H */

// Unified (prefill + decode) attention over a paged KV pool, fp32, causal
// (crates/triton-kernels/src/attention.rs:988-1187).  Query tokens of all sequences are packed token-major
// (query_start_loc is the CSR offset array); a sequence's query tokens are the LAST q_len positions of its KV
// stream, so query token j of a sequence sees kv positions 0 .. (seq_len - q_len) + j.
//
// A straightforward kernel: one warp per (query token, q head), online softmax in fp32, one KV row per
// step with a warp reduction.  The decode-only paged case has its own bandwidth-oriented kernel
// (paged_decode_attention); this entry point is for the mixed batches a serving engine forms.
#include "common.cuh"

namespace b200k {

constexpr int UA_MAX_D = 256;

__global__ void __launch_bounds__(256)
unified_attention_kernel(const float *__restrict__ q, const float *__restrict__ kc, const float *__restrict__ vc,
                         float *__restrict__ out, const int32_t *__restrict__ block_table,
                         const int32_t *__restrict__ seq_lens, const int32_t *__restrict__ query_start_loc, int hq, int hkv,
                         int d, int block_size, int max_blocks_per_seq, float sm_scale) {
    const int seq = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int kvh = head / (hq / hkv);
    const int q_start = query_start_loc[seq], q_len = query_start_loc[seq + 1] - q_start;
    const int seq_len = seq_lens[seq];
    const int context_len = seq_len - q_len;
    const long kv_inner = (long)hkv * d, block_stride = (long)block_size * kv_inner;
    const int32_t *bt = block_table + (long)seq * max_blocks_per_seq;
    constexpr int PER = UA_MAX_D / 32;
    for (int j = warp; j < q_len; j += nwarps) {
        const long row = ((long)(q_start + j) * hq + head) * d;
        float qv[PER], acc[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            qv[i] = x < d ? q[row + x] * sm_scale : 0.f;
            acc[i] = 0.f;
        }
        float m = -1.0e30f, l = 0.f;
        const int limit = min(seq_len, context_len + j + 1);     // causal and in-bounds
        for (int p = 0; p < limit; ++p) {
            const long base = (long)bt[p / block_size] * block_stride + (long)(p % block_size) * kv_inner + (long)kvh * d;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int x = lane + 32 * i;
                if (x < d) s += qv[i] * kc[base + x];
            }
            s = warp_sum(s);
            const float m_new = fmaxf(m, s);
            const float alpha = expf(m - m_new), pexp = expf(s - m_new);
            l = l * alpha + pexp;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int x = lane + 32 * i;
                if (x < d) acc[i] = acc[i] * alpha + pexp * vc[base + x];
            }
            m = m_new;
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            if (x < d) out[row + x] = acc[i] / l;
        }
    }
}

}  // namespace b200k

using namespace b200k;

extern "C" int unified_attention_f32(const float *q, const float *k_cache, const float *v_cache, float *output,
                                     const int32_t *block_table, const int32_t *seq_lens, const int32_t *query_start_loc,
                                     int num_q_heads, int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                                     float sm_scale, int num_seqs, b200k_stream stream) {
    B200K_REQUIRE(num_seqs >= 0 && num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0 && head_dim > 0 &&
                      head_dim <= UA_MAX_D && block_size > 0 && max_blocks_per_seq > 0,
                  B200K_E_SHAPE, "unified_attention_f32: seqs %d, heads %d/%d, head_dim %d (<= %d), block_size %d, blocks per seq %d",
                  num_seqs, num_q_heads, num_kv_heads, head_dim, UA_MAX_D, block_size, max_blocks_per_seq);
    if (num_seqs == 0) return 0;
    B200K_REQUIRE(q && k_cache && v_cache && output && block_table && seq_lens && query_start_loc, B200K_E_NULL,
                  "unified_attention_f32: NULL pointer");
    B200K_REQUIRE(num_q_heads <= 65535, B200K_E_SHAPE, "unified_attention_f32: %d q heads", num_q_heads);
    unified_attention_kernel<<<dim3(num_seqs, num_q_heads), 256, 0, to_stream(stream)>>>(
        q, k_cache, v_cache, output, block_table, seq_lens, query_start_loc, num_q_heads, num_kv_heads, head_dim, block_size,
        max_blocks_per_seq, sm_scale);
    return launch_status("unified_attention_f32");
}

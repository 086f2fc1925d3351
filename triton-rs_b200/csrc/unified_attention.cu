// Unified (prefill + decode) attention over a paged KV pool, fp32, causal
// (crates/triton-kernels/src/attention.rs:988-1187).  Query tokens of all sequences are packed token-major
// (query_start_loc is the CSR offset array); a sequence's query tokens are the LAST q_len positions of its KV
// stream, so query token j of a sequence sees kv positions 0 .. (seq_len - q_len) + j.
//
// A CUDA-core kernel, fp32 throughout (the entry point is fp32; its tolerance leaves no room for tf32 tensor cores):
// one CTA per (sequence, q head, slice of the sequence's query tokens), online softmax in fp32, four KV rows per step so
// that the four dot-product reductions and the dependent block-table / K / V loads of a step overlap.
//   * sequences with many query tokens (prefill): warp w of slice z takes tokens 8 z + w, + 8 UA_SLICES, ...
//   * sequences with at most UA_SPLIT_MAX query tokens (decode): slice 0 alone works; its eight warps split the KV
//     positions of each token (warp w takes the groups of four w, w + 8, ...) and merge their partial softmax states
//     through shared memory in warp order.
// Registers are kept low on purpose: the kernel lives on occupancy (a variant that held the next group's K rows and the
// current V rows in registers to overlap their latency needed 157 registers and ran 1.5x slower).
// The decode-only paged case has its own bandwidth-oriented kernel (paged_decode_attention); this entry point is for the
// mixed batches a serving engine forms.
#include "common.cuh"

namespace b200k {

constexpr int UA_MAX_D = 256;
constexpr int UA_WARPS = 8;
constexpr int UA_SLICES = 16;        // grid.z: token slices per (sequence, head); slices beyond q_len leave at once
constexpr int UA_SPLIT_MAX = 4;      // at most this many query tokens: the warps split the KV range instead of the tokens

// one warp: the groups of four positions first_group, first_group + group_step, ... of [0, limit), online softmax state
template <int PER>
__device__ __forceinline__ void ua_scan(const float *__restrict__ kc, const float *__restrict__ vc, const int32_t *__restrict__ bt,
                                        const float (&qv)[PER], float (&acc)[PER], float &m, float &l, int first_group,
                                        int group_step, int limit, int block_size, long block_stride, long kv_inner, long head_off,
                                        int d, int lane) {
    for (int p = 4 * first_group; p < limit; p += 4 * group_step) {
        long base[4];
        float s[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int pp = min(p + u, limit - 1);       // the tail group re-reads the last row; its weight is zeroed below
            base[u] = (long)bt[pp / block_size] * block_stride + (long)(pp % block_size) * kv_inner + head_off;
            s[u] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            if (x < d) {
#pragma unroll
                for (int u = 0; u < 4; ++u) s[u] += qv[i] * kc[base[u] + x];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) s[u] = warp_sum(s[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (p + u >= limit) s[u] = -1.0e30f;
        const float m_new = fmaxf(fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3])), m);
        const float alpha = expf(m - m_new);
        float pe[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) pe[u] = p + u < limit ? expf(s[u] - m_new) : 0.f;
        l = l * alpha + ((pe[0] + pe[1]) + (pe[2] + pe[3]));
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            if (x < d) {
                float a = acc[i] * alpha;
#pragma unroll
                for (int u = 0; u < 4; ++u) a += pe[u] * vc[base[u] + x];
                acc[i] = a;
            }
        }
        m = m_new;
    }
}

__global__ void __launch_bounds__(UA_WARPS * 32)
unified_attention_kernel(const float *__restrict__ q, const float *__restrict__ kc, const float *__restrict__ vc,
                         float *__restrict__ out, const int32_t *__restrict__ block_table,
                         const int32_t *__restrict__ seq_lens, const int32_t *__restrict__ query_start_loc, int hq, int hkv,
                         int d, int block_size, int max_blocks_per_seq, float sm_scale) {
    constexpr int PER = UA_MAX_D / 32;
    __shared__ float sm_acc[UA_WARPS][UA_MAX_D];
    __shared__ float sm_m[UA_WARPS], sm_l[UA_WARPS];
    const int seq = blockIdx.x, head = blockIdx.y, slice = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = head / (hq / hkv);
    const int q_start = query_start_loc[seq], q_len = query_start_loc[seq + 1] - q_start;
    const int seq_len = seq_lens[seq];
    const int context_len = seq_len - q_len;
    const long kv_inner = (long)hkv * d, block_stride = (long)block_size * kv_inner, head_off = (long)kvh * d;
    const int32_t *bt = block_table + (long)seq * max_blocks_per_seq;
    const bool split = q_len <= UA_SPLIT_MAX;
    if (split ? slice > 0 : slice * UA_WARPS >= q_len) return;      // uniform per CTA, before any barrier

    auto load_q = [&](long row, float (&qv)[PER], float (&acc)[PER]) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            qv[i] = x < d ? q[row + x] * sm_scale : 0.f;
            acc[i] = 0.f;
        }
    };
    if (!split) {
        for (int j = slice * UA_WARPS + warp; j < q_len; j += UA_SLICES * UA_WARPS) {
            const long row = ((long)(q_start + j) * hq + head) * d;
            float qv[PER], acc[PER];
            load_q(row, qv, acc);
            float m = -1.0e30f, l = 0.f;
            const int limit = min(seq_len, context_len + j + 1);     // causal and in-bounds
            ua_scan<PER>(kc, vc, bt, qv, acc, m, l, 0, 1, limit, block_size, block_stride, kv_inner, head_off, d, lane);
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int x = lane + 32 * i;
                if (x < d) out[row + x] = acc[i] / l;
            }
        }
        return;
    }
    for (int j = 0; j < q_len; ++j) {
        const long row = ((long)(q_start + j) * hq + head) * d;
        float qv[PER], acc[PER];
        load_q(row, qv, acc);
        float m = -1.0e30f, l = 0.f;
        const int limit = min(seq_len, context_len + j + 1);
        ua_scan<PER>(kc, vc, bt, qv, acc, m, l, warp, UA_WARPS, limit, block_size, block_stride, kv_inner, head_off, d, lane);
        // merge the warps' states in warp order: out = sum_w acc_w e^(m_w - M) / sum_w l_w e^(m_w - M)
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            if (x < d) sm_acc[warp][x] = acc[i];
        }
        if (lane == 0) {
            sm_m[warp] = m;
            sm_l[warp] = l;
        }
        __syncthreads();
        float M = sm_m[0];
#pragma unroll
        for (int w = 1; w < UA_WARPS; ++w) M = fmaxf(M, sm_m[w]);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < UA_WARPS; ++w) L += sm_l[w] * expf(sm_m[w] - M);       // a warp without positions has l = 0
        for (int x = threadIdx.x; x < d; x += UA_WARPS * 32) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < UA_WARPS; ++w) o += sm_acc[w][x] * expf(sm_m[w] - M);
            out[row + x] = o / L;
        }
        __syncthreads();      // before the next token overwrites the staging rows
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
    unified_attention_kernel<<<dim3(num_seqs, num_q_heads, UA_SLICES), UA_WARPS * 32, 0, to_stream(stream)>>>(
        q, k_cache, v_cache, output, block_table, seq_lens, query_start_loc, num_q_heads, num_kv_heads, head_dim, block_size,
        max_blocks_per_seq, sm_scale);
    return launch_status("unified_attention_f32");
}

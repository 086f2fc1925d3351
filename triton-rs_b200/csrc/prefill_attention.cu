// Causal prefill attention over contiguous head-major tensors, fp32 arithmetic for every element type
// (crates/triton-kernels/src/attention.rs:780-909, flash_attn_full): Q, O [batch, Hq, q_len, D];
// K, V [batch, Hkv, kv_len, D]; query row i sees kv positions 0 .. pos_offset + i (and never past kv_len).
// The reference adds -1e30 to masked scores and walks every KV tile; since exp underflows to exactly 0 there,
// the result is the softmax over the visible positions, which is what is computed here (masked tiles are skipped).
//
// First, plain version of this entry point: one warp per query row, the eight rows of a CTA are consecutive
// rows of one head so that their K / V rows are shared through L1; four KV positions per step so that the
// four warp reductions overlap.  The decode kernels are the bandwidth-tuned ones; a tensor-core prefill
// (tcgen05, the pipeline of the int4 GEMM) is the follow-up.
#include <cuda_bf16.h>

#include "common.cuh"

namespace b200k {

constexpr int PF_MAX_D = 256;
constexpr int PF_WARPS = 8;

__device__ __forceinline__ float ldf(const float *p) { return __ldg(p); }
__device__ __forceinline__ float ldf(const __half *p) { return __half2float(__ldg(p)); }
__device__ __forceinline__ void stf(float *p, float v) { *p = v; }
__device__ __forceinline__ void stf(__half *p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ float ldf(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(PF_WARPS * 32)
prefill_attention_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ out, int hq,
                         int hkv, int q_len, int kv_len, int d, int pos_offset, float scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * PF_WARPS + warp, head = blockIdx.y, batch = blockIdx.z;
    if (row >= q_len) return;
    const int kvh = head / (hq / hkv);
    const long q_base = (((long)batch * hq + head) * q_len + row) * d;
    const long kv_base = ((long)batch * hkv + kvh) * (long)kv_len * d;
    constexpr int PER = PF_MAX_D / 32;
    float qv[PER], acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int x = lane + 32 * i;
        qv[i] = x < d ? ldf(q + q_base + x) * scale : 0.f;
        acc[i] = 0.f;
    }
    float m = -1.0e30f, l = 0.f;
    const long vis = (long)pos_offset + row + 1;
    const int limit = (int)(vis < 0 ? 0 : (vis < kv_len ? vis : kv_len));
    int p = 0;
    for (; p + 4 <= limit; p += 4) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            if (x < d) {
#pragma unroll
                for (int u = 0; u < 4; ++u) s[u] += qv[i] * ldf(k + kv_base + (long)(p + u) * d + x);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) s[u] = warp_sum(s[u]);
        const float m_new = fmaxf(fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3])), m);
        const float alpha = expf(m - m_new);
        float pe[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) pe[u] = expf(s[u] - m_new);
        l = l * alpha + ((pe[0] + pe[1]) + (pe[2] + pe[3]));
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            if (x < d) {
                float a = acc[i] * alpha;
#pragma unroll
                for (int u = 0; u < 4; ++u) a += pe[u] * ldf(v + kv_base + (long)(p + u) * d + x);
                acc[i] = a;
            }
        }
        m = m_new;
    }
    for (; p < limit; ++p) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            if (x < d) s += qv[i] * ldf(k + kv_base + (long)p * d + x);
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new), pe = expf(s - m_new);
        l = l * alpha + pe;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int x = lane + 32 * i;
            if (x < d) acc[i] = acc[i] * alpha + pe * ldf(v + kv_base + (long)p * d + x);
        }
        m = m_new;
    }
    // a row that sees nothing (negative pos_offset) writes zeros
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int x = lane + 32 * i;
        if (x < d) stf(out + q_base + x, acc[i] * inv);
    }
}

template <typename T>
static int prefill_launch(const char *name, const T *q, const T *k, const T *v, T *out, int batch, int hq, int hkv, int q_len,
                          int kv_len, int d, int pos_offset, float scale, b200k_stream stream) {
    B200K_REQUIRE(batch >= 0 && hq > 0 && hkv > 0 && hq % hkv == 0 && q_len >= 0 && kv_len >= 0 && d > 0 && d <= PF_MAX_D,
                  B200K_E_SHAPE, "%s: batch %d, heads %d/%d, q_len %d, kv_len %d, head_dim %d (<= %d)", name, batch, hq, hkv, q_len,
                  kv_len, d, PF_MAX_D);
    if (batch == 0 || q_len == 0) return 0;
    B200K_REQUIRE(q && k && v && out, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(hq <= 65535 && batch <= 65535, B200K_E_SHAPE, "%s: %d heads, batch %d (grid limits)", name, hq, batch);
    const dim3 grid((q_len + PF_WARPS - 1) / PF_WARPS, hq, batch);
    prefill_attention_kernel<T><<<grid, PF_WARPS * 32, 0, to_stream(stream)>>>(q, k, v, out, hq, hkv, q_len, kv_len, d, pos_offset,
                                                                            scale);
    return launch_status(name);
}

}  // namespace b200k

using namespace b200k;

extern "C" int flash_attn_full_f32(const float *q, const float *k, const float *v, float *output, int batch, int num_heads,
                                   int num_kv_heads, int q_len, int kv_len, int head_dim, int pos_offset, float scale,
                                   b200k_stream stream) {
    return prefill_launch<float>("flash_attn_full_f32", q, k, v, output, batch, num_heads, num_kv_heads, q_len, kv_len, head_dim,
                                 pos_offset, scale, stream);
}

namespace b200k {
// tensor-core kernel (prefill_tc.cu): head_dim 128, pos_offset >= 0; -1000 when the call is outside what it covers
int prefill_tc_launch(const __half *q, const __half *k, const __half *v, __half *out, int batch, int hq, int hkv, int q_len,
                      int kv_len, int d, int pos_offset, float scale, bool bf16, cudaStream_t st);
}  // namespace b200k

extern "C" int flash_attn_full_f16(const b200k_half *q, const b200k_half *k, const b200k_half *v, b200k_half *output, int batch,
                                   int num_heads, int num_kv_heads, int q_len, int kv_len, int head_dim, int pos_offset,
                                   float scale, b200k_stream stream) {
    if (q && k && v && output && batch > 0 && num_heads > 0 && num_kv_heads > 0 && env_char("B200K_PREFILL") != 'g') {
        const int rc = prefill_tc_launch(reinterpret_cast<const __half *>(q), reinterpret_cast<const __half *>(k),
                                         reinterpret_cast<const __half *>(v), reinterpret_cast<__half *>(output), batch, num_heads,
                                         num_kv_heads, q_len, kv_len, head_dim, pos_offset, scale, false, to_stream(stream));
        if (rc != -1000) return rc;
    }
    return prefill_launch<__half>("flash_attn_full_f16", reinterpret_cast<const __half *>(q), reinterpret_cast<const __half *>(k),
                                  reinterpret_cast<const __half *>(v), reinterpret_cast<__half *>(output), batch, num_heads,
                                  num_kv_heads, q_len, kv_len, head_dim, pos_offset, scale, stream);
}

extern "C" int flash_attn_full_bf16(const b200k_bf16 *q, const b200k_bf16 *k, const b200k_bf16 *v, b200k_bf16 *output, int batch,
                                    int num_heads, int num_kv_heads, int q_len, int kv_len, int head_dim, int pos_offset,
                                    float scale, b200k_stream stream) {
    if (q && k && v && output && batch > 0 && num_heads > 0 && num_kv_heads > 0 && env_char("B200K_PREFILL") != 'g') {
        const int rc = prefill_tc_launch(reinterpret_cast<const __half *>(q), reinterpret_cast<const __half *>(k),
                                         reinterpret_cast<const __half *>(v), reinterpret_cast<__half *>(output), batch, num_heads,
                                         num_kv_heads, q_len, kv_len, head_dim, pos_offset, scale, true, to_stream(stream));
        if (rc != -1000) return rc;
    }
    return prefill_launch<__nv_bfloat16>("flash_attn_full_bf16", reinterpret_cast<const __nv_bfloat16 *>(q),
                                         reinterpret_cast<const __nv_bfloat16 *>(k), reinterpret_cast<const __nv_bfloat16 *>(v),
                                         reinterpret_cast<__nv_bfloat16 *>(output), batch, num_heads, num_kv_heads, q_len, kv_len,
                                         head_dim, pos_offset, scale, stream);
}

// Projection helpers around attention in the reference's consumer: split of a combined QKV tensor, the
// two head/token transposes, and RoPE (optionally with a per-head RMS norm first) fused with the
// transpose to head-major.  fp32, as in the reference (crates/triton-kernels/src/projection.rs).  All are
// one pass over a few hundred KiB: 128-bit accesses where the row length allows, no shared memory.
#include "common.cuh"

namespace b200k {

// Copies `rows` rows of `d` floats between two row orders.  Row index r counts (outer, head) pairs, head fastest:
//   mode 0  split of [batch, 3, heads, d]: part `which` of batch r / heads, head r % heads  ->  row r
//   mode 1  head-major [heads, tokens, d] row (r % heads, r / heads)                        ->  token-major row r
//   mode 2  token-major row r                                                               ->  head-major row (r % heads, r / heads)
__global__ void __launch_bounds__(256)
row_move_kernel(const float *__restrict__ in, float *__restrict__ out, long rows, int d, bool vec, int mode, int heads,
                int outer, int which) {
    const int per = vec ? d / 4 : d;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per; i += (long)gridDim.x * blockDim.x) {
        const long r = i / per;
        const int c = (int)(i - r * per);
        const long o = r / heads, h = r - o * heads;
        long src = r * d, dst = r * d;
        if (mode == 0) src = ((o * 3 + which) * heads + h) * d;
        else if (mode == 1) src = (h * outer + o) * d;
        else dst = (h * outer + o) * d;
        if (vec) reinterpret_cast<float4 *>(out + dst)[c] = reinterpret_cast<const float4 *>(in + src)[c];
        else out[dst + c] = in[src + c];
    }
}

static int move_grid(long work) {
    long blocks = (work + 255) / 256;
    const long cap = (long)sm_count() * 8;
    return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}
static bool vec_ok(int d, const void *a, const void *b) { return d % 4 == 0 && aligned16(a) && aligned16(b); }

// One warp per (token, head): optional RMS norm of the head vector, RoPE on the (i, i + D/2) pairs,
// store at the head-major position.
template <bool NORM>
__global__ void __launch_bounds__(256)
rope_transpose_kernel(const float *__restrict__ in, const float *__restrict__ norm_w, const float *__restrict__ cos_t,
                      const float *__restrict__ sin_t, float *__restrict__ out, int tokens, int heads, int d,
                      int pos_offset, float inv_n, float eps) {
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (warp >= (long)tokens * heads) return;
    const int tok = (int)(warp / heads), head = (int)(warp - (long)tok * heads);
    const int half = d / 2;
    const float *src = in + ((long)tok * heads + head) * d;
    float inv_rms = 1.f;
    if (NORM) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss += src[i] * src[i];
        ss = warp_sum(ss);
        inv_rms = rsqrtf(ss * inv_n + eps);
    }
    const long cs = (long)(pos_offset + tok) * half;
    float *dst = out + ((long)head * tokens + tok) * d;
    for (int i = lane; i < half; i += 32) {
        const float c = cos_t[cs + i], s = sin_t[cs + i];
        float x0 = src[i], x1 = src[i + half];
        if (NORM) {
            x0 = x0 * inv_rms * norm_w[i];
            x1 = x1 * inv_rms * norm_w[i + half];
        }
        dst[i] = x0 * c - x1 * s;
        dst[i + half] = x1 * c + x0 * s;
    }
}

}  // namespace b200k

using namespace b200k;

extern "C" int split_qkv_f32(const float *qkv, float *q_out, float *k_out, float *v_out, int num_heads, int head_dim,
                             int batch, b200k_stream stream) {
    B200K_REQUIRE(num_heads > 0 && head_dim > 0 && batch >= 0, B200K_E_SHAPE, "split_qkv_f32: heads %d, head_dim %d, batch %d",
                  num_heads, head_dim, batch);
    if (batch == 0) return 0;
    B200K_REQUIRE(qkv && q_out && k_out && v_out, B200K_E_NULL, "split_qkv_f32: NULL pointer");
    float *outs[3] = {q_out, k_out, v_out};
    const long rows = (long)batch * num_heads;
    for (int which = 0; which < 3; ++which) {
        const bool vec = vec_ok(head_dim, qkv, outs[which]);
        row_move_kernel<<<move_grid(rows * head_dim / (vec ? 4 : 1)), 256, 0, to_stream(stream)>>>(qkv, outs[which], rows, head_dim,
                                                                                                   vec, 0, num_heads, batch, which);
    }
    return launch_status("split_qkv_f32");
}

extern "C" int transpose_head_to_token_f32(const float *input, float *output, int tokens, int heads, int head_dim,
                                           b200k_stream stream) {
    B200K_REQUIRE(tokens >= 0 && heads > 0 && head_dim > 0, B200K_E_SHAPE, "transpose_head_to_token_f32: tokens %d, heads %d, head_dim %d",
                  tokens, heads, head_dim);
    if (tokens == 0) return 0;
    B200K_REQUIRE(input && output, B200K_E_NULL, "transpose_head_to_token_f32: NULL pointer");
    const long rows = (long)tokens * heads;
    const bool vec = vec_ok(head_dim, input, output);
    row_move_kernel<<<move_grid(rows * head_dim / (vec ? 4 : 1)), 256, 0, to_stream(stream)>>>(input, output, rows, head_dim, vec, 1,
                                                                                               heads, tokens, 0);
    return launch_status("transpose_head_to_token_f32");
}

extern "C" int transpose_token_to_head_f32(const float *input, float *output, int tokens, int heads, int head_dim,
                                           b200k_stream stream) {
    B200K_REQUIRE(tokens >= 0 && heads > 0 && head_dim > 0, B200K_E_SHAPE, "transpose_token_to_head_f32: tokens %d, heads %d, head_dim %d",
                  tokens, heads, head_dim);
    if (tokens == 0) return 0;
    B200K_REQUIRE(input && output, B200K_E_NULL, "transpose_token_to_head_f32: NULL pointer");
    const long rows = (long)tokens * heads;
    const bool vec = vec_ok(head_dim, input, output);
    row_move_kernel<<<move_grid(rows * head_dim / (vec ? 4 : 1)), 256, 0, to_stream(stream)>>>(input, output, rows, head_dim, vec, 2,
                                                                                               heads, tokens, 0);
    return launch_status("transpose_token_to_head_f32");
}

static int rope_transpose_check(const char *name, int tokens, int heads, int head_dim, int pos_offset) {
    B200K_REQUIRE(tokens >= 0 && heads > 0 && head_dim > 0 && head_dim % 2 == 0 && pos_offset >= 0, B200K_E_SHAPE,
                  "%s: tokens %d, heads %d, head_dim %d (even), pos_offset %d", name, tokens, heads, head_dim, pos_offset);
    return 0;
}

extern "C" int qk_norm_rope_transpose_f32(const float *input, const float *norm_w, const float *cos_tab, const float *sin_tab,
                                          float *output, int tokens, int heads, int head_dim, int pos_offset, float inv_n,
                                          float eps, b200k_stream stream) {
    int rc = rope_transpose_check("qk_norm_rope_transpose_f32", tokens, heads, head_dim, pos_offset);
    if (rc) return rc;
    if (tokens == 0) return 0;
    B200K_REQUIRE(input && norm_w && cos_tab && sin_tab && output, B200K_E_NULL, "qk_norm_rope_transpose_f32: NULL pointer");
    const long warps = (long)tokens * heads;
    rope_transpose_kernel<true><<<(unsigned)((warps + 7) / 8), 256, 0, to_stream(stream)>>>(input, norm_w, cos_tab, sin_tab, output, tokens,
                                                                                           heads, head_dim, pos_offset, inv_n, eps);
    return launch_status("qk_norm_rope_transpose_f32");
}

extern "C" int rope_transpose_f32(const float *input, const float *cos_tab, const float *sin_tab, float *output, int tokens,
                                  int heads, int head_dim, int pos_offset, b200k_stream stream) {
    int rc = rope_transpose_check("rope_transpose_f32", tokens, heads, head_dim, pos_offset);
    if (rc) return rc;
    if (tokens == 0) return 0;
    B200K_REQUIRE(input && cos_tab && sin_tab && output, B200K_E_NULL, "rope_transpose_f32: NULL pointer");
    const long warps = (long)tokens * heads;
    rope_transpose_kernel<false><<<(unsigned)((warps + 7) / 8), 256, 0, to_stream(stream)>>>(input, nullptr, cos_tab, sin_tab, output, tokens,
                                                                                            heads, head_dim, pos_offset, 0.f, 0.f);
    return launch_status("rope_transpose_f32");
}

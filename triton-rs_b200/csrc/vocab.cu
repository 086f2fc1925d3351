// The two ends of a decode step around the layer stack: the embedding gather before the first
// layer and the row softmax over the logits after the last (embedding.rs, reduction.rs of the
// reference's kernel crate).  Both are bandwidth-bound single passes.
#include <cuda_bf16.h>

#include "common.cuh"

namespace b200k {

// output[tok, :] = embeddings[indices[tok], :]; CHUNK-byte accesses when the row pitch allows.
template <typename V>
__global__ void __launch_bounds__(256)
embedding_kernel(const V *__restrict__ table, const int32_t *__restrict__ indices, V *__restrict__ out, long row_vecs,
                 long total_vecs) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vecs; i += (long)gridDim.x * blockDim.x) {
        const long tok = i / row_vecs, c = i - tok * row_vecs;
        out[i] = table[(long)indices[tok] * row_vecs + c];
    }
}

template <typename T>
static int embedding_launch(const char *name, const T *table, const int32_t *indices, T *out, int hidden, int tokens,
                            cudaStream_t st) {
    B200K_REQUIRE(hidden > 0 && tokens >= 0, B200K_E_SHAPE, "%s: hidden_size %d, tokens %d", name, hidden, tokens);
    if (tokens == 0) return 0;
    B200K_REQUIRE(table && indices && out, B200K_E_NULL, "%s: NULL pointer", name);
    const size_t row_bytes = (size_t)hidden * sizeof(T);
    auto grid = [](long work) {
        long blocks = (work + 255) / 256;
        const long cap = (long)sm_count() * 16;
        return (int)(blocks > cap ? cap : blocks);
    };
    if (row_bytes % 16 == 0 && aligned16(table) && aligned16(out)) {
        const long rv = (long)(row_bytes / 16), total = rv * tokens;
        embedding_kernel<uint4><<<grid(total), 256, 0, st>>>((const uint4 *)table, indices, (uint4 *)out, rv, total);
    } else {
        const long total = (long)hidden * tokens;
        embedding_kernel<T><<<grid(total), 256, 0, st>>>(table, indices, out, hidden, total);
    }
    return launch_status(name);
}

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// One CTA per row.  Pass 1 keeps a running (max, sum of exp) pair per thread and merges the pairs across the
// CTA; pass 2 re-reads the row (from L2 at any practical width) and writes exp(x - max) / sum.
template <typename T>
__global__ void __launch_bounds__(256)
softmax_kernel(const T *__restrict__ in, T *__restrict__ out, int cols) {
    __shared__ float red[32];
    __shared__ float s_max, s_sum;
    const T *x = in + (long)blockIdx.x * cols;
    T *y = out + (long)blockIdx.x * cols;
    float m = -INFINITY, l = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = to_f(x[c]);
        if (v > m) {
            l = l * expf(m - v) + 1.f;    // expf(-inf) = 0 on the first element
            m = v;
        } else {
            l += expf(v - m);
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float wm = warp_max(m);
    l = (m == -INFINITY) ? 0.f : l * expf(m - wm);
    l = warp_sum(l);
    if (lane == 0) { red[warp] = wm; red[16 + warp] = l; }
    __syncthreads();
    if (warp == 0) {
        const float bm0 = lane < nw ? red[lane] : -INFINITY;
        const float bm = warp_max(bm0);
        float bl = (lane < nw && bm0 != -INFINITY) ? red[16 + lane] * expf(bm0 - bm) : 0.f;
        bl = warp_sum(bl);
        if (lane == 0) { s_max = bm; s_sum = bl; }
    }
    __syncthreads();
    const float rm = s_max, rs = s_sum;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) y[c] = from_f<T>(expf(to_f(x[c]) - rm) / rs);
}

template <typename T>
static int softmax_launch(const char *name, const T *in, T *out, int rows, int cols, cudaStream_t st) {
    B200K_REQUIRE(rows >= 0 && cols > 0, B200K_E_SHAPE, "%s: rows %d, cols %d", name, rows, cols);
    if (rows == 0) return 0;
    B200K_REQUIRE(in && out, B200K_E_NULL, "%s: NULL pointer", name);
    softmax_kernel<T><<<rows, 256, 0, st>>>(in, out, cols);
    return launch_status(name);
}

}  // namespace b200k

using namespace b200k;

extern "C" int embedding_lookup_f32(const float *embeddings, const int32_t *indices, float *output, int hidden_size,
                                    int num_tokens, b200k_stream stream) {
    return embedding_launch<float>("embedding_lookup_f32", embeddings, indices, output, hidden_size, num_tokens, to_stream(stream));
}
extern "C" int embedding_lookup_f16(const b200k_half *embeddings, const int32_t *indices, b200k_half *output,
                                    int hidden_size, int num_tokens, b200k_stream stream) {
    return embedding_launch<__half>("embedding_lookup_f16", (const __half *)embeddings, indices, (__half *)output, hidden_size,
                                    num_tokens, to_stream(stream));
}
extern "C" int softmax_f32(const float *input, float *output, int rows, int cols, b200k_stream stream) {
    return softmax_launch<float>("softmax_f32", input, output, rows, cols, to_stream(stream));
}
extern "C" int softmax_f16(const b200k_half *input, b200k_half *output, int rows, int cols, b200k_stream stream) {
    return softmax_launch<__half>("softmax_f16", (const __half *)input, (__half *)output, rows, cols, to_stream(stream));
}
extern "C" int embedding_lookup_bf16(const b200k_bf16 *embeddings, const int32_t *indices, b200k_bf16 *output, int hidden_size,
                                     int num_tokens, b200k_stream stream) {
    // a gather of 16-bit elements: the fp16 kernel
    return embedding_launch<__half>("embedding_lookup_bf16", (const __half *)embeddings, indices, (__half *)output, hidden_size,
                                    num_tokens, to_stream(stream));
}
extern "C" int softmax_bf16(const b200k_bf16 *input, b200k_bf16 *output, int rows, int cols, b200k_stream stream) {
    return softmax_launch<__nv_bfloat16>("softmax_bf16", (const __nv_bfloat16 *)input, (__nv_bfloat16 *)output, rows, cols, to_stream(stream));
}

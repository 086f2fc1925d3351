// GQA decode attention over a KV cache.
//
// Two kernel families:
//  * attn_split_f16 (head_dim 128, fp16): split-KV flash-decode.  One CTA per
//    (sequence, kv head, chunk of CH positions) handles ALL q heads of the GQA group,
//    so every K/V element is read from HBM once.  K/V rows are staged into shared
//    memory by bulk asynchronous copies (cp.async.bulk, one 256-byte row per copy,
//    mbarrier transaction counts) in a 4-deep ring; scores are computed one position
//    per thread pair, the softmax statistics once per chunk, and the P.V product with
//    16 lanes per row; partial (acc, max, sum) triples go to scratch and the last CTA
//    of a (sequence, kv head) to arrive merges them (log-sum-exp).  Every mbarrier
//    wait is bounded and reports through a status word.
//  * attn_generic (any head_dim <= 256, fp16 or fp32): one CTA per (sequence, q head,
//    split); backs the f32 entry points and the explicit phase-1 / phase-2 API.
#include "common.cuh"

namespace b200k {

// ---------------------------------------------------------------------------
// addressing of one K/V row, shared by both families
// ---------------------------------------------------------------------------
struct KvLayout {
    long stride_b, stride_h, stride_p;  // elements; contiguous head_dim rows
    const int32_t *block_table;         // paged pools when non-null
    int block_size;
    long block_stride;                  // elements per physical block
};
__device__ __forceinline__ long kv_row_offset(const KvLayout &L, int b, int kvh, int pos) {
    if (L.block_table) {
        const int phys = L.block_table[pos / L.block_size];
        return (long)phys * L.block_stride + (long)(pos % L.block_size) * L.stride_p + (long)kvh * L.stride_h;
    }
    return (long)b * L.stride_b + (long)kvh * L.stride_h + (long)pos * L.stride_p;
}

// ---------------------------------------------------------------------------
// mbarrier + bulk-copy primitives (shared::cta addresses as 32-bit)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~1 s of SM clock and returns false.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > 2000000000LL) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---------------------------------------------------------------------------
// split-KV fp16 family
// ---------------------------------------------------------------------------
constexpr int AT_D = 128;               // head_dim
constexpr int AT_THREADS = 128;
constexpr int AT_TILE = 64;             // positions per stage
constexpr int AT_STAGES = 4;
constexpr int AT_ROW = AT_D * 2 + 16;   // padded row stride in shared memory (bytes)
constexpr int AT_MAX_CH = 1024;         // largest chunk (positions)

struct AttnSplitArgs {
    const __half *q;        // [B, Hq, D]
    const __half *k, *v;
    __half *out;            // [B, Hq, D]
    const int32_t *lens;    // per sequence, or nullptr -> len_scalar
    int len_scalar;
    int hq, hkv;
    int chunk;              // positions per CTA, multiple of AT_TILE, <= AT_MAX_CH
    float scale_log2e;      // softmax scale * log2(e)
    KvLayout L;
    float *ws_acc;          // [B*Hkv*max_chunks, G, D]
    float *ws_ml;           // [B*Hkv*max_chunks, G, 2]  (max, sum)
    int *counters;          // [B*Hkv], zero between launches
    int *status;            // device status word (0 = ok)
};

template <int G>
struct AttnSmem {
    __align__(16) unsigned char stage[AT_STAGES][AT_TILE * AT_ROW];
    __align__(16) float sp[AT_MAX_CH * G];    // scores, then probabilities, [pos][G]
    __align__(16) float q[G * AT_D];          // q * scale * log2(e)
    float red[AT_THREADS / 32][2 * G];
    float m[G], l[G];
    __align__(8) unsigned long long full[AT_STAGES];
    int abort_flag;
    int is_last;
};

template <int G>
__global__ void __launch_bounds__(AT_THREADS)
attn_split_f16_kernel(AttnSplitArgs A) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    AttnSmem<G> &S = *reinterpret_cast<AttnSmem<G> *>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk_id = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int len = A.lens ? A.lens[b] : A.len_scalar;
    const int nchunks = (len + A.chunk - 1) / A.chunk;
    if (len <= 0) {
        // no keys: defined as a zero output row (the reference would divide 0 by 0)
        if (chunk_id == 0)
            for (int i = tid; i < G * AT_D; i += AT_THREADS)
                A.out[((long)b * A.hq + kvh * G) * AT_D + i] = __float2half_rn(0.f);
        return;
    }
    if (chunk_id >= nchunks) return;
    const int p0 = chunk_id * A.chunk;
    const int npos = min(A.chunk, len - p0);
    const int ntiles = (npos + AT_TILE - 1) / AT_TILE;
    const int total_tiles = 2 * ntiles;  // K tiles then V tiles

    if (tid == 0) {
        for (int s = 0; s < AT_STAGES; ++s) mbar_init(smem_u32(&S.full[s]), 1);
        S.abort_flag = 0;
        S.is_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < G * AT_D; i += AT_THREADS)
        S.q[i] = __half2float(A.q[((long)b * A.hq + kvh * G) * AT_D + i]) * A.scale_log2e;
    __syncthreads();

    // producer: warp 0 issues the row copies of tile t into stage t % STAGES
    auto issue_tile = [&](int t) {
        const bool is_v = t >= ntiles;
        const int tt = is_v ? t - ntiles : t;
        const int rows = min(AT_TILE, npos - tt * AT_TILE);
        const uint32_t bar = smem_u32(&S.full[t % AT_STAGES]);
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows * AT_D * 2);
        __syncwarp();
        const __half *base = is_v ? A.v : A.k;
        for (int r = lane; r < rows; r += 32) {
            const long off = kv_row_offset(A.L, b, kvh, p0 + tt * AT_TILE + r);
            bulk_g2s(smem_u32(&S.stage[t % AT_STAGES][r * AT_ROW]), base + off, AT_D * 2, bar);
        }
    };
    if (warp == 0)
        for (int t = 0; t < min(AT_STAGES, total_tiles); ++t) issue_tile(t);

    // ---- K phase: thread (h = lane / 16, position = warp * 16 + lane % 16) ----
    const int kp = warp * 16 + (lane & 15), kh = lane >> 4;
    int t = 0;
    for (; t < ntiles; ++t) {
        const int st = t % AT_STAGES;
        if (!S.abort_flag && !mbar_wait_bounded(smem_u32(&S.full[st]), (t / AT_STAGES) & 1)) {
            S.abort_flag = 1;
            atomicExch(A.status, 1);
        }
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.f;
        const unsigned char *row = &S.stage[st][kp * AT_ROW];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int j = 2 * i + kh;  // 16-byte column of the row
            const uint4 kv = *reinterpret_cast<const uint4 *>(row + j * 16);
            const float2 k0 = h2_to_f2(kv.x), k1 = h2_to_f2(kv.y), k2 = h2_to_f2(kv.z), k3 = h2_to_f2(kv.w);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 qa = *reinterpret_cast<const float4 *>(&S.q[g * AT_D + j * 8]);
                const float4 qb = *reinterpret_cast<const float4 *>(&S.q[g * AT_D + j * 8 + 4]);
                s[g] += qa.x * k0.x + qa.y * k0.y + qa.z * k1.x + qa.w * k1.y + qb.x * k2.x + qb.y * k2.y +
                        qb.z * k3.x + qb.w * k3.y;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], 16);
        const int pos = t * AT_TILE + kp;  // within the chunk
        if (kh == 0 && pos < npos) {
#pragma unroll
            for (int g = 0; g < G; ++g) S.sp[pos * G + g] = s[g];
        }
        __syncthreads();  // stage st is free again
        if (warp == 0 && t + AT_STAGES < total_tiles) issue_tile(t + AT_STAGES);
    }

    // ---- softmax statistics of the chunk ----
    {
        float mx[G], sum[G];
#pragma unroll
        for (int g = 0; g < G; ++g) mx[g] = -1e30f;
        for (int p = tid; p < npos; p += AT_THREADS)
#pragma unroll
            for (int g = 0; g < G; ++g) mx[g] = fmaxf(mx[g], S.sp[p * G + g]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            mx[g] = warp_max(mx[g]);
            if (lane == 0) S.red[warp][g] = mx[g];
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float m = S.red[0][g];
            for (int w = 1; w < AT_THREADS / 32; ++w) m = fmaxf(m, S.red[w][g]);
            mx[g] = m;
            sum[g] = 0.f;
        }
        for (int p = tid; p < npos; p += AT_THREADS)
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float e = exp2f(S.sp[p * G + g] - mx[g]);
                S.sp[p * G + g] = e;
                sum[g] += e;
            }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            sum[g] = warp_sum(sum[g]);
            if (lane == 0) S.red[warp][G + g] = sum[g];
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; ++g)
            if (tid == g) {  // mx[] is identical in every thread
                float l = 0.f;
                for (int w = 0; w < AT_THREADS / 32; ++w) l += S.red[w][G + g];
                S.m[g] = mx[g];
                S.l[g] = l;
            }
    }

    // ---- V phase: thread (group = tid / 16 takes positions = group mod 8, lane16 -> 8 dims) ----
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[g][d] = 0.f;
    const int vg = tid >> 4, vl = tid & 15;
    for (; t < total_tiles; ++t) {
        const int st = t % AT_STAGES, tt = t - ntiles;
        if (!S.abort_flag && !mbar_wait_bounded(smem_u32(&S.full[st]), (t / AT_STAGES) & 1)) {
            S.abort_flag = 1;
            atomicExch(A.status, 1);
        }
        const int rows = min(AT_TILE, npos - tt * AT_TILE);
#pragma unroll 2
        for (int r = vg; r < rows; r += 8) {
            const uint4 vv = *reinterpret_cast<const uint4 *>(&S.stage[st][r * AT_ROW + vl * 16]);
            const float2 v0 = h2_to_f2(vv.x), v1 = h2_to_f2(vv.y), v2 = h2_to_f2(vv.z), v3 = h2_to_f2(vv.w);
            const float *pp = &S.sp[(tt * AT_TILE + r) * G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float p = pp[g];
                acc[g][0] += p * v0.x; acc[g][1] += p * v0.y; acc[g][2] += p * v1.x; acc[g][3] += p * v1.y;
                acc[g][4] += p * v2.x; acc[g][5] += p * v2.y; acc[g][6] += p * v3.x; acc[g][7] += p * v3.y;
            }
        }
        __syncthreads();
        if (warp == 0 && t + AT_STAGES < total_tiles) issue_tile(t + AT_STAGES);
    }

    // ---- reduce the 8 position groups through shared memory (reuses the stage ring) ----
    float *red = reinterpret_cast<float *>(&S.stage[0][0]);  // [8][G][D]
#pragma unroll
    for (int g = 0; g < G; ++g) {
        *reinterpret_cast<float4 *>(&red[(vg * G + g) * AT_D + vl * 8]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        *reinterpret_cast<float4 *>(&red[(vg * G + g) * AT_D + vl * 8 + 4]) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    }
    __syncthreads();
    const long item = ((long)b * A.hkv + kvh) * gridDim.x + chunk_id;
    for (int i = tid; i < G * AT_D; i += AT_THREADS) {
        float o = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) o += red[j * G * AT_D + i];
        if (nchunks == 1) {
            A.out[((long)b * A.hq + kvh * G) * AT_D + i] = __float2half_rn(o / S.l[i / AT_D]);
        } else {
            A.ws_acc[item * G * AT_D + i] = o;
        }
    }
    if (nchunks == 1) return;
    if (tid < G) {
        A.ws_ml[(item * G + tid) * 2 + 0] = S.m[tid];
        A.ws_ml[(item * G + tid) * 2 + 1] = S.l[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int done = atomicAdd(&A.counters[b * A.hkv + kvh], 1);
        S.is_last = (done == nchunks - 1);
    }
    __syncthreads();
    if (!S.is_last) return;
    __threadfence();
    // ---- merge: out = sum_c acc_c 2^(m_c - M) / sum_c l_c 2^(m_c - M) ----
    const long item0 = ((long)b * A.hkv + kvh) * gridDim.x;
    for (int i = tid; i < G * AT_D; i += AT_THREADS) {
        const int g = i / AT_D;
        float M = -1e30f;
        for (int c = 0; c < nchunks; ++c) M = fmaxf(M, __ldcg(&A.ws_ml[((item0 + c) * G + g) * 2]));
        float L = 0.f, o = 0.f;
        for (int c = 0; c < nchunks; ++c) {
            const float w = exp2f(__ldcg(&A.ws_ml[((item0 + c) * G + g) * 2]) - M);
            L += __ldcg(&A.ws_ml[((item0 + c) * G + g) * 2 + 1]) * w;
            o += __ldcg(&A.ws_acc[(item0 + c) * G * AT_D + i]) * w;
        }
        A.out[((long)b * A.hq + kvh * G) * AT_D + i] = __float2half_rn(o / L);
    }
    if (tid == 0) A.counters[b * A.hkv + kvh] = 0;  // ready for the next launch
}

// Scratch layout: [status 256 B][counters B*Hkv ints, padded to 256 B][ml][acc]
struct AttnWs {
    int *status;
    int *counters;
    float *ml;
    float *acc;
    size_t bytes;
};
static AttnWs attn_ws_layout(void *base, int batch, int hkv, int g, int max_chunks) {
    AttnWs w;
    unsigned char *p = (unsigned char *)base;
    size_t off = 0;
    w.status = (int *)(p + off);
    off += 256;
    w.counters = (int *)(p + off);
    off += (((size_t)batch * hkv * sizeof(int)) + 255) / 256 * 256;
    const size_t items = (size_t)batch * hkv * max_chunks;
    w.ml = (float *)(p + off);
    off += ((items * g * 2 * sizeof(float)) + 255) / 256 * 256;
    w.acc = (float *)(p + off);
    off += items * g * AT_D * sizeof(float);
    w.bytes = off;
    return w;
}

static int pick_chunk(int batch, int hkv, int max_len) {
    // Largest chunk that still gives every SM ~4 CTAs when all sequences are full length.
    const long want = 4L * sm_count();
    int chunk = AT_MAX_CH;
    while (chunk > 256 && (long)batch * hkv * ceil_div(max_len, chunk) < want) chunk /= 2;
    return chunk;
}

struct AttnCall {
    const __half *q, *k, *v;
    __half *out;
    const int32_t *lens;
    int len_scalar;
    int batch, hq, hkv, d, max_len;
    float scale;
    KvLayout L;
    void *ws;
    size_t ws_bytes;
    bool own_ws;
    cudaStream_t stream;
};

template <int G>
static int attn_split_launch_g(const AttnSplitArgs &A, dim3 grid, cudaStream_t st) {
    const size_t smem = sizeof(AttnSmem<G>);
    static bool attr_set[16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_split_f16_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
        attr_set[dev] = true;
    }
    attn_split_f16_kernel<G><<<grid, AT_THREADS, smem, st>>>(A);
    return launch_status("decode attention (split-KV)");
}

static int attn_split_launch(const char *name, AttnCall c) {
    const int g = c.hq / c.hkv;
    const int chunk = pick_chunk(c.batch, c.hkv, c.max_len);
    const int max_chunks = ceil_div(c.max_len, chunk);
    if (!c.ws && c.own_ws) {
        int rc = default_workspace(&c.ws, &c.ws_bytes);
        if (rc) return rc;
    }
    B200K_REQUIRE(c.ws, B200K_E_WORKSPACE, "%s: workspace is NULL", name);
    AttnWs w = attn_ws_layout(c.ws, c.batch, c.hkv, g, max_chunks);
    B200K_REQUIRE(w.bytes <= c.ws_bytes, B200K_E_WORKSPACE, "%s: workspace %zu bytes, need %zu", name, c.ws_bytes, w.bytes);
    AttnSplitArgs A;
    A.q = c.q; A.k = c.k; A.v = c.v; A.out = c.out; A.lens = c.lens; A.len_scalar = c.len_scalar;
    A.hq = c.hq; A.hkv = c.hkv; A.chunk = chunk;
    A.scale_log2e = c.scale * 1.4426950408889634f;
    A.L = c.L;
    A.ws_acc = w.acc; A.ws_ml = w.ml; A.counters = w.counters; A.status = w.status;
    dim3 grid(max_chunks, c.hkv, c.batch);
    switch (g) {
        case 1: return attn_split_launch_g<1>(A, grid, c.stream);
        case 2: return attn_split_launch_g<2>(A, grid, c.stream);
        case 4: return attn_split_launch_g<4>(A, grid, c.stream);
        case 8: return attn_split_launch_g<8>(A, grid, c.stream);
    }
    return 1;
}

// ---------------------------------------------------------------------------
// generic family: one CTA (128 threads) per (sequence, q head, split).  Warp w takes
// positions w, w+4, ... of the split; lanes stride over head_dim.  Online softmax per
// warp, merged across the 4 warps at the end.  Output either normalised (MODE 0) or
// as un-normalised phase-1 partials (MODE 1).
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float ldf(const T *p);
template <> __device__ __forceinline__ float ldf<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float ldf<__half>(const __half *p) { return __half2float(*p); }
template <typename T> __device__ __forceinline__ void stf(T *p, float v);
template <> __device__ __forceinline__ void stf<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__half>(__half *p, float v) { *p = __float2half_rn(v); }

struct AttnGenericArgs {
    const void *q, *k, *v;
    void *out;                 // MODE 0: [B,Hq,D] of T
    float *pacc, *pmax, *psum; // MODE 1: [B*Hq, S, D], [B*Hq, S], [B*Hq, S]
    int hq, hkv, d;
    int valid_len;
    int num_splits, split_len; // split s covers [s*split_len, min((s+1)*split_len, valid_len))
    float scale;
    KvLayout L;
};

template <typename T, int MODE>
__global__ void __launch_bounds__(128)
attn_generic_kernel(AttnGenericArgs A) {
    constexpr int MAXD = 256, PER = MAXD / 32;
    __shared__ float sm_acc[4][MAXD];
    __shared__ float sm_m[4], sm_l[4];
    const int bh = blockIdx.x, split = blockIdx.y;
    const int b = bh / A.hq, h = bh % A.hq;
    const int kvh = h / (A.hq / A.hkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T *q = (const T *)A.q + (long)bh * A.d;
    const T *kc = (const T *)A.k, *vc = (const T *)A.v;
    float qr[PER], acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < A.d ? ldf<T>(q + d) : 0.f;
        acc[i] = 0.f;
    }
    float m = -1e30f, l = 0.f;
    const int lo = split * A.split_len;
    const int hi = min(lo + A.split_len, A.valid_len);
    for (int pos = lo + warp; pos < hi; pos += 4) {
        const long off = kv_row_offset(A.L, b, kvh, pos);
        float kvv[PER], dot = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (d < A.d) {
                dot += qr[i] * ldf<T>(kc + off + d);
                kvv[i] = ldf<T>(vc + off + d);
            } else {
                kvv[i] = 0.f;
            }
        }
        const float s = warp_sum(dot) * A.scale;
        const float mn = fmaxf(m, s);
        const float alpha = expf(m - mn), p = expf(s - mn);
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] = acc[i] * alpha + p * kvv[i];
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) sm_acc[warp][lane + 32 * i] = acc[i];
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
    __syncthreads();
    const float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    float w[4], Lsum = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        w[j] = expf(sm_m[j] - M);
        Lsum += sm_l[j] * w[j];
    }
    for (int d = threadIdx.x; d < A.d; d += 128) {
        const float o = sm_acc[0][d] * w[0] + sm_acc[1][d] * w[1] + sm_acc[2][d] * w[2] + sm_acc[3][d] * w[3];
        if (MODE == 0)
            stf<T>((T *)A.out + (long)bh * A.d + d, o / Lsum);
        else
            A.pacc[((long)bh * A.num_splits + split) * A.d + d] = o;
    }
    if (MODE == 1 && threadIdx.x == 0) {
        A.pmax[(long)bh * A.num_splits + split] = M;
        A.psum[(long)bh * A.num_splits + split] = Lsum;
    }
}

// phase 2: one warp per (flattened) q head
__global__ void __launch_bounds__(128)
attn_combine_kernel(const float *__restrict__ pacc, const float *__restrict__ pmax, const float *__restrict__ psum,
                    float *__restrict__ out, int heads, int d, int splits) {
    const int h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= heads) return;
    float M = -1e30f;
    for (int s = lane; s < splits; s += 32) M = fmaxf(M, pmax[(long)h * splits + s]);
    M = warp_max(M);
    float L = 0.f;
    for (int s = lane; s < splits; s += 32) L += psum[(long)h * splits + s] * expf(pmax[(long)h * splits + s] - M);
    L = warp_sum(L);
    for (int dd = lane; dd < d; dd += 32) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s)
            o += pacc[((long)h * splits + s) * d + dd] * (expf(pmax[(long)h * splits + s] - M) / L);
        out[(long)h * d + dd] = o;
    }
}

template <typename T>
static int attn_generic_launch(const char *name, const void *q, const void *k, const void *v, void *out, int batch,
                               int hq, int hkv, int d, int valid_len, float scale, const KvLayout &L,
                               cudaStream_t st) {
    AttnGenericArgs A = {};
    A.q = q; A.k = k; A.v = v; A.out = out;
    A.hq = hq; A.hkv = hkv; A.d = d; A.valid_len = valid_len; A.num_splits = 1;
    A.split_len = valid_len > 0 ? valid_len : 1;
    A.scale = scale; A.L = L;
    attn_generic_kernel<T, 0><<<dim3(batch * hq, 1), 128, 0, st>>>(A);
    return launch_status(name);
}

static int attn_common_checks(const char *name, const void *q, const void *k, const void *v, const void *out, int hq,
                              int hkv, int d, int len) {
    B200K_REQUIRE(q && k && v && out, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, B200K_E_SHAPE, "%s: num_q_heads %d, num_kv_heads %d", name, hq, hkv);
    B200K_REQUIRE(d > 0 && d <= 256, B200K_E_SHAPE, "%s: head_dim %d (1..256 supported)", name, d);
    B200K_REQUIRE(len > 0, B200K_E_SHAPE, "%s: valid_kv_len %d", name, len);
    return 0;
}

static bool split_ok(int hq, int hkv, int d, const void *q, const void *k, const void *v, const void *out,
                     const KvLayout &L) {
    const int g = hq / hkv;
    if (d != AT_D || !(g == 1 || g == 2 || g == 4 || g == 8)) return false;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return false;
    if (L.stride_b % 8 || L.stride_h % 8 || L.stride_p % 8 || L.block_stride % 8) return false;
    return true;
}

}  // namespace b200k

using namespace b200k;

// ---- fp16 single-sequence entry points ---------------------------------------
static int decode_f16_common(const char *name, const b200k_half *q, const b200k_half *k, const b200k_half *v,
                             b200k_half *out, int hq, int hkv, int d, int len, float scale, const KvLayout &L,
                             int cap_for_chunks, b200k_stream stream) {
    int rc = attn_common_checks(name, q, k, v, out, hq, hkv, d, len);
    if (rc) return rc;
    if (split_ok(hq, hkv, d, q, k, v, out, L)) {
        AttnCall c = {};
        c.q = (const __half *)q; c.k = (const __half *)k; c.v = (const __half *)v; c.out = (__half *)out;
        c.lens = nullptr; c.len_scalar = len; c.batch = 1; c.hq = hq; c.hkv = hkv; c.d = d;
        c.max_len = cap_for_chunks; c.scale = scale; c.L = L; c.ws = nullptr; c.own_ws = true;
        c.stream = to_stream(stream);
        rc = attn_split_launch(name, c);
        if (rc != 1) return rc;
    }
    return attn_generic_launch<__half>(name, q, k, v, out, 1, hq, hkv, d, len, scale, L, to_stream(stream));
}

extern "C" int decode_attention_f16(const b200k_half *q, const b200k_half *k_cache, const b200k_half *v_cache,
                                    b200k_half *output, int num_q_heads, int num_kv_heads, int head_dim,
                                    int valid_kv_len, float scale, b200k_stream stream) {
    KvLayout L = {0, head_dim, (long)num_kv_heads * head_dim, nullptr, 0, 0};
    return decode_f16_common("decode_attention_f16", q, k_cache, v_cache, output, num_q_heads, num_kv_heads, head_dim,
                             valid_kv_len, scale, L, valid_kv_len, stream);
}
extern "C" int decode_attention_hm_f16(const b200k_half *q, const b200k_half *k_cache, const b200k_half *v_cache,
                                       b200k_half *output, int num_q_heads, int num_kv_heads, int head_dim,
                                       int capacity, int valid_kv_len, float scale, b200k_stream stream) {
    B200K_REQUIRE(capacity >= valid_kv_len, B200K_E_SHAPE, "decode_attention_hm_f16: capacity %d < valid_kv_len %d",
                  capacity, valid_kv_len);
    KvLayout L = {0, (long)capacity * head_dim, head_dim, nullptr, 0, 0};
    return decode_f16_common("decode_attention_hm_f16", q, k_cache, v_cache, output, num_q_heads, num_kv_heads,
                             head_dim, valid_kv_len, scale, L, valid_kv_len, stream);
}
extern "C" int paged_decode_attention_f16(const b200k_half *q, const b200k_half *k_block_pool,
                                          const b200k_half *v_block_pool, const int32_t *block_table,
                                          b200k_half *output, int num_q_heads, int num_kv_heads, int head_dim,
                                          int valid_kv_len, int block_size, float scale, b200k_stream stream) {
    B200K_REQUIRE(block_table, B200K_E_NULL, "paged_decode_attention_f16: block_table is NULL");
    B200K_REQUIRE(block_size > 0, B200K_E_SHAPE, "paged_decode_attention_f16: block_size %d", block_size);
    KvLayout L = {0, head_dim, (long)num_kv_heads * head_dim, block_table, block_size,
                  (long)block_size * num_kv_heads * head_dim};
    return decode_f16_common("paged_decode_attention_f16", q, k_block_pool, v_block_pool, output, num_q_heads,
                             num_kv_heads, head_dim, valid_kv_len, scale, L, valid_kv_len, stream);
}

// ---- fp16 batched, per-sequence lengths ---------------------------------------
extern "C" int batched_decode_attention_hm_f16_ws(const b200k_half *q, const b200k_half *k_cache,
                                                  const b200k_half *v_cache, const int32_t *context_lens,
                                                  b200k_half *output, int batch_size, int num_q_heads,
                                                  int num_kv_heads, int head_dim, int max_len, float scale,
                                                  void *workspace, size_t workspace_bytes, b200k_stream stream) {
    const char *name = "batched_decode_attention_hm_f16";
    B200K_REQUIRE(q && k_cache && v_cache && context_lens && output, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, B200K_E_SHAPE,
                  "%s: num_q_heads %d, num_kv_heads %d", name, num_q_heads, num_kv_heads);
    B200K_REQUIRE(batch_size >= 0 && max_len > 0, B200K_E_SHAPE, "%s: batch %d, max_len %d", name, batch_size, max_len);
    if (batch_size == 0) return 0;
    KvLayout L = {(long)num_kv_heads * max_len * head_dim, (long)max_len * head_dim, head_dim, nullptr, 0, 0};
    B200K_REQUIRE(split_ok(num_q_heads, num_kv_heads, head_dim, q, k_cache, v_cache, output, L), B200K_E_SHAPE,
                  "%s: needs head_dim 128, group size 1/2/4/8 and 16-byte aligned tensors", name);
    AttnCall c = {};
    c.q = (const __half *)q; c.k = (const __half *)k_cache; c.v = (const __half *)v_cache; c.out = (__half *)output;
    c.lens = context_lens; c.len_scalar = 0; c.batch = batch_size; c.hq = num_q_heads; c.hkv = num_kv_heads;
    c.d = head_dim; c.max_len = max_len; c.scale = scale; c.L = L;
    c.ws = workspace; c.ws_bytes = workspace_bytes; c.own_ws = workspace == nullptr;
    c.stream = to_stream(stream);
    return attn_split_launch(name, c);
}
extern "C" int batched_decode_attention_hm_f16(const b200k_half *q, const b200k_half *k_cache,
                                               const b200k_half *v_cache, const int32_t *context_lens,
                                               b200k_half *output, int batch_size, int num_q_heads, int num_kv_heads,
                                               int head_dim, int max_len, float scale, b200k_stream stream) {
    return batched_decode_attention_hm_f16_ws(q, k_cache, v_cache, context_lens, output, batch_size, num_q_heads,
                                              num_kv_heads, head_dim, max_len, scale, nullptr, 0, stream);
}
extern "C" size_t b200k_attention_workspace_bytes(int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                                  int max_len) {
    if (batch <= 0 || num_kv_heads <= 0 || num_q_heads <= 0 || max_len <= 0 || head_dim != AT_D) return 0;
    const int chunk = pick_chunk(batch, num_kv_heads, max_len);
    return attn_ws_layout(nullptr, batch, num_kv_heads, num_q_heads / num_kv_heads, ceil_div(max_len, chunk)).bytes;
}

// ---- f32 entry points ------------------------------------------------------------
extern "C" int decode_attention_f32(const float *q, const float *k_cache, const float *v_cache, float *output,
                                    int num_q_heads, int num_kv_heads, int head_dim, int valid_kv_len, float scale,
                                    b200k_stream stream) {
    const char *name = "decode_attention_f32";
    int rc = attn_common_checks(name, q, k_cache, v_cache, output, num_q_heads, num_kv_heads, head_dim, valid_kv_len);
    if (rc) return rc;
    KvLayout L = {0, head_dim, (long)num_kv_heads * head_dim, nullptr, 0, 0};
    return attn_generic_launch<float>(name, q, k_cache, v_cache, output, 1, num_q_heads, num_kv_heads, head_dim,
                                      valid_kv_len, scale, L, to_stream(stream));
}
extern "C" int decode_attention_hm_f32(const float *q, const float *k_cache, const float *v_cache, float *output,
                                       int num_q_heads, int num_kv_heads, int head_dim, int capacity,
                                       int valid_kv_len, float scale, b200k_stream stream) {
    const char *name = "decode_attention_hm_f32";
    int rc = attn_common_checks(name, q, k_cache, v_cache, output, num_q_heads, num_kv_heads, head_dim, valid_kv_len);
    if (rc) return rc;
    B200K_REQUIRE(capacity >= valid_kv_len, B200K_E_SHAPE, "%s: capacity %d < valid_kv_len %d", name, capacity, valid_kv_len);
    KvLayout L = {0, (long)capacity * head_dim, head_dim, nullptr, 0, 0};
    return attn_generic_launch<float>(name, q, k_cache, v_cache, output, 1, num_q_heads, num_kv_heads, head_dim,
                                      valid_kv_len, scale, L, to_stream(stream));
}
extern "C" int batched_decode_attention_f32(const float *q, const float *k_cache, const float *v_cache, float *output,
                                            int batch_size, int num_q_heads, int num_kv_heads, int head_dim,
                                            int seq_len, int valid_kv_len, float scale, b200k_stream stream) {
    const char *name = "batched_decode_attention_f32";
    int rc = attn_common_checks(name, q, k_cache, v_cache, output, num_q_heads, num_kv_heads, head_dim, valid_kv_len);
    if (rc) return rc;
    B200K_REQUIRE(batch_size >= 0 && seq_len >= valid_kv_len, B200K_E_SHAPE, "%s: batch %d, seq_len %d, valid_kv_len %d",
                  name, batch_size, seq_len, valid_kv_len);
    if (batch_size == 0) return 0;
    KvLayout L = {(long)seq_len * num_kv_heads * head_dim, head_dim, (long)num_kv_heads * head_dim, nullptr, 0, 0};
    return attn_generic_launch<float>(name, q, k_cache, v_cache, output, batch_size, num_q_heads, num_kv_heads,
                                      head_dim, valid_kv_len, scale, L, to_stream(stream));
}

static int phase1_common(const char *name, const float *q, const float *k, const float *v, float *pacc, float *pmax,
                         float *psum, int batch, int hq, int hkv, int d, int seq_len, int valid_len, int splits,
                         float scale, int block_kv, b200k_stream stream) {
    int rc = attn_common_checks(name, q, k, v, pacc, hq, hkv, d, valid_len);
    if (rc) return rc;
    B200K_REQUIRE(pmax && psum, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(splits > 0 && block_kv > 0 && batch >= 0, B200K_E_SHAPE, "%s: num_splits %d, block_kv %d", name, splits, block_kv);
    if (batch == 0) return 0;
    AttnGenericArgs A = {};
    A.q = q; A.k = k; A.v = v; A.pacc = pacc; A.pmax = pmax; A.psum = psum;
    A.hq = hq; A.hkv = hkv; A.d = d; A.num_splits = splits;
    // chunk_blocks = (valid_kv_len / num_splits) / BLOCK_KV whole tiles per split (attention.rs:538)
    A.split_len = ((valid_len / splits) / block_kv) * block_kv;
    A.valid_len = A.split_len * splits;
    A.scale = scale;
    A.L = KvLayout{(long)seq_len * hkv * d, d, (long)hkv * d, nullptr, 0, 0};
    attn_generic_kernel<float, 1><<<dim3(batch * hq, splits), 128, 0, to_stream(stream)>>>(A);
    return launch_status(name);
}
extern "C" int flash_decode_attn_phase1_f32(const float *q, const float *k_cache, const float *v_cache,
                                            float *partial_acc, float *partial_max, float *partial_sum,
                                            int num_q_heads, int num_kv_heads, int head_dim, int valid_kv_len,
                                            int num_splits, float scale, int block_kv, b200k_stream stream) {
    return phase1_common("flash_decode_attn_phase1_f32", q, k_cache, v_cache, partial_acc, partial_max, partial_sum, 1,
                         num_q_heads, num_kv_heads, head_dim, 0, valid_kv_len, num_splits, scale, block_kv, stream);
}
extern "C" int batched_flash_decode_attn_phase1_f32(const float *q, const float *k_cache, const float *v_cache,
                                                    float *partial_acc, float *partial_max, float *partial_sum,
                                                    int batch_size, int num_q_heads, int num_kv_heads, int head_dim,
                                                    int seq_len, int valid_kv_len, int num_splits, float scale,
                                                    int block_kv, b200k_stream stream) {
    return phase1_common("batched_flash_decode_attn_phase1_f32", q, k_cache, v_cache, partial_acc, partial_max,
                         partial_sum, batch_size, num_q_heads, num_kv_heads, head_dim, seq_len, valid_kv_len,
                         num_splits, scale, block_kv, stream);
}
extern "C" int flash_decode_attn_phase2_f32(const float *partial_acc, const float *partial_max,
                                            const float *partial_sum, float *output, int num_q_heads, int head_dim,
                                            int num_splits, b200k_stream stream) {
    const char *name = "flash_decode_attn_phase2_f32";
    B200K_REQUIRE(partial_acc && partial_max && partial_sum && output, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(num_q_heads >= 0 && head_dim > 0 && num_splits > 0, B200K_E_SHAPE, "%s: heads %d, head_dim %d, splits %d",
                  name, num_q_heads, head_dim, num_splits);
    if (num_q_heads == 0) return 0;
    attn_combine_kernel<<<ceil_div(num_q_heads, 4), 128, 0, to_stream(stream)>>>(partial_acc, partial_max, partial_sum,
                                                                                output, num_q_heads, head_dim, num_splits);
    return launch_status(name);
}

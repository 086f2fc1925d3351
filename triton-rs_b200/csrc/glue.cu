// Bandwidth-bound glue kernels: rms_norm, fused_add_rms_norm, residual_add,
// fused_silu_mul (+interleaved), RoPE, kv-cache append.  All are one pass over
// their operands with 128-bit accesses where the extents and pointers allow it
// and a scalar path otherwise; reductions and transcendental math are fp32.
#include <cuda_bf16.h>

#include "common.cuh"

namespace b200k {

// ---------------------------------------------------------------------------
// element traits: VEC elements per 16 bytes
// ---------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
    static constexpr int VEC = 8;
    __device__ static void load(const __half *p, float (&f)[8]) {
        uint4 u = *reinterpret_cast<const uint4 *>(p);
        float2 a = h2_to_f2(u.x), b = h2_to_f2(u.y), c = h2_to_f2(u.z), d = h2_to_f2(u.w);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    }
    __device__ static void store(__half *p, const float (&f)[8]) {
        uint4 u;
        u.x = f2_to_h2(f[0], f[1]); u.y = f2_to_h2(f[2], f[3]);
        u.z = f2_to_h2(f[4], f[5]); u.w = f2_to_h2(f[6], f[7]);
        *reinterpret_cast<uint4 *>(p) = u;
    }
    // the same 8 values stored as (f0,f4,f1,f5,f2,f6,f3,f7): the order the int4 GEMM's nibble arithmetic yields a
    // packed word's values in, so a GEMM fed with such activations skips its byte-permutes
    __device__ static void store_kperm(__half *p, const float (&f)[8]) {
        uint4 u;
        u.x = f2_to_h2(f[0], f[4]); u.y = f2_to_h2(f[1], f[5]);
        u.z = f2_to_h2(f[2], f[6]); u.w = f2_to_h2(f[3], f[7]);
        *reinterpret_cast<uint4 *>(p) = u;
    }
    __device__ static float ld1(const __half *p) { return __half2float(*p); }
    __device__ static void st1(__half *p, float v) { *p = __float2half_rn(v); }
};
// bf16: the upper 16 bits of an fp32; widened exactly, rounded to nearest even on the way back
template <> struct Elem<__nv_bfloat16> {
    static constexpr int VEC = 8;
    __device__ static void load(const __nv_bfloat16 *p, float (&f)[8]) {
        const uint4 u = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    __device__ static uint32_t pack(float a, float b) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    __device__ static void store(__nv_bfloat16 *p, const float (&f)[8]) {
        *reinterpret_cast<uint4 *>(p) = make_uint4(pack(f[0], f[1]), pack(f[2], f[3]), pack(f[4], f[5]), pack(f[6], f[7]));
    }
    __device__ static void store_kperm(__nv_bfloat16 *p, const float (&f)[8]) {
        *reinterpret_cast<uint4 *>(p) = make_uint4(pack(f[0], f[4]), pack(f[1], f[5]), pack(f[2], f[6]), pack(f[3], f[7]));
    }
    __device__ static float ld1(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
    __device__ static void st1(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Elem<float> {
    static constexpr int VEC = 4;
    __device__ static void load(const float *p, float (&f)[4]) {
        float4 u = *reinterpret_cast<const float4 *>(p);
        f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
    }
    __device__ static void store(float *p, const float (&f)[4]) {
        *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
    }
    __device__ static void store_kperm(float *p, const float (&f)[4]) { store(p, f); }   // fp16 only; never selected
    __device__ static float ld1(const float *p) { return *p; }
    __device__ static void st1(float *p, float v) { *p = v; }
};

// ---------------------------------------------------------------------------
// rms_norm / fused_add_rms_norm: one CTA per row, row kept in registers
// (up to ITERS vectors per thread), one read and one write per element.
// ---------------------------------------------------------------------------
template <typename T, bool FUSED_ADD, bool VECTOR, int ITERS>
__global__ void __launch_bounds__(1024)
rms_norm_kernel(const T *__restrict__ x, const T *__restrict__ res, const T *__restrict__ w,
                T *__restrict__ y, T *__restrict__ res_out, int n, float inv_n, float eps, bool kperm) {
    constexpr int VEC = Elem<T>::VEC;
    __shared__ float red[32];
    pdl_wait();
    pdl_launch_dependents();
    const size_t row_off = (size_t)blockIdx.x * n;
    const T *xr = x + row_off;
    float ss = 0.f;
    if (VECTOR) {
        float v[ITERS][VEC];
        const int nv = n / VEC;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int i = threadIdx.x + it * blockDim.x;
            if (i < nv) {
                Elem<T>::load(xr + i * VEC, v[it]);
                if (FUSED_ADD) {
                    float r[VEC];
                    Elem<T>::load(res + row_off + i * VEC, r);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) v[it][j] += r[j];
                    Elem<T>::store(res_out + row_off + i * VEC, v[it]);
                }
#pragma unroll
                for (int j = 0; j < VEC; ++j) ss += v[it][j] * v[it][j];
            }
        }
        const float inv = rsqrtf(block_sum(ss, red) * inv_n + eps);
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int i = threadIdx.x + it * blockDim.x;
            if (i < nv) {
                float wv[VEC], o[VEC];
                Elem<T>::load(w + i * VEC, wv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) o[j] = v[it][j] * inv * wv[j];
                if (kperm) Elem<T>::store_kperm(y + row_off + i * VEC, o);
                else Elem<T>::store(y + row_off + i * VEC, o);
            }
        }
    } else {
        // any row length / alignment: two passes, the second served by L1/L2
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            float v = Elem<T>::ld1(xr + i);
            if (FUSED_ADD) {
                v += Elem<T>::ld1(res + row_off + i);
                Elem<T>::st1(res_out + row_off + i, v);
            }
            ss += v * v;
        }
        const float inv = rsqrtf(block_sum(ss, red) * inv_n + eps);
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            float v = Elem<T>::ld1(xr + i);
            if (FUSED_ADD) v += Elem<T>::ld1(res + row_off + i);
            Elem<T>::st1(y + row_off + i, v * inv * Elem<T>::ld1(w + i));
        }
    }
}

// Short rows (up to 32 * ITERS vectors of 16 bytes): one WARP per row, eight rows per CTA, shuffle reduction only.  A CTA per
// 2 KiB row is bound by CTA launch rate, not by memory.
template <typename T, bool FUSED_ADD, int ITERS>
__global__ void __launch_bounds__(256)
rms_norm_warp_kernel(const T *__restrict__ x, const T *__restrict__ res, const T *__restrict__ w,
                     T *__restrict__ y, T *__restrict__ res_out, int n, float inv_n, float eps, int rows, bool kperm) {
    constexpr int VEC = Elem<T>::VEC;
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const size_t row_off = (size_t)row * n;
    const int nv = n / VEC;
    float v[ITERS][VEC];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int i = lane + it * 32;
        if (i < nv) {
            Elem<T>::load(x + row_off + i * VEC, v[it]);
            if (FUSED_ADD) {
                float r[VEC];
                Elem<T>::load(res + row_off + i * VEC, r);
#pragma unroll
                for (int j = 0; j < VEC; ++j) v[it][j] += r[j];
                Elem<T>::store(res_out + row_off + i * VEC, v[it]);
            }
#pragma unroll
            for (int j = 0; j < VEC; ++j) ss += v[it][j] * v[it][j];
        }
    }
    const float inv = rsqrtf(warp_sum(ss) * inv_n + eps);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int i = lane + it * 32;
        if (i < nv) {
            float wv[VEC], o[VEC];
            Elem<T>::load(w + i * VEC, wv);
#pragma unroll
            for (int j = 0; j < VEC; ++j) o[j] = v[it][j] * inv * wv[j];
            if (kperm) Elem<T>::store_kperm(y + row_off + i * VEC, o);
            else Elem<T>::store(y + row_off + i * VEC, o);
        }
    }
}

template <typename T, bool FUSED_ADD>
static int rms_norm_launch(const char *name, const T *x, const T *res, const T *w, T *y, T *res_out,
                           int n, float inv_n, float eps, int rows, cudaStream_t st, bool kperm = false) {
    B200K_REQUIRE(x && w && y && (!FUSED_ADD || (res && res_out)), B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(n > 0 && rows >= 0, B200K_E_SHAPE, "%s: row_size %d, rows %d", name, n, rows);
    if (rows == 0) return 0;
    constexpr int VEC = Elem<T>::VEC;
    bool vec = (n % VEC == 0) && aligned16(x) && aligned16(w) && aligned16(y) &&
               (!FUSED_ADD || (aligned16(res) && aligned16(res_out)));
    const int nv = n / VEC;
    // In the fused kernel the in-place form (residual_out == residual) is allowed: each
    // element is read and written by the same thread.
    B200K_REQUIRE(!kperm || (vec && nv <= 4 * 1024 && VEC == 8), B200K_E_SHAPE, "%s: the permuted output needs fp16 rows of a multiple of 8, 16-byte aligned", name);
    if (vec && nv <= 256 && rows >= 8 * 148) {
        // many short rows: a warp per row
        const dim3 grid(ceil_div(rows, 8)), block(256);
        if (nv <= 128)
            launch_kernel(rms_norm_warp_kernel<T, FUSED_ADD, 4>, grid, block, 0, st, x, res, w, y, res_out, n, inv_n, eps, rows, kperm);
        else
            launch_kernel(rms_norm_warp_kernel<T, FUSED_ADD, 8>, grid, block, 0, st, x, res, w, y, res_out, n, inv_n, eps, rows, kperm);
    } else if (vec && nv <= 4 * 1024) {
        int threads = nv <= 128 ? 128 : (nv <= 256 ? 256 : (nv <= 512 ? 512 : 1024));
        int iters = ceil_div(nv, threads);
        if (iters == 1)
            launch_kernel(rms_norm_kernel<T, FUSED_ADD, true, 1>, dim3(rows), dim3(threads), 0, st, x, res, w, y, res_out, n, inv_n, eps, kperm);
        else if (iters == 2)
            launch_kernel(rms_norm_kernel<T, FUSED_ADD, true, 2>, dim3(rows), dim3(threads), 0, st, x, res, w, y, res_out, n, inv_n, eps, kperm);
        else
            launch_kernel(rms_norm_kernel<T, FUSED_ADD, true, 4>, dim3(rows), dim3(threads), 0, st, x, res, w, y, res_out, n, inv_n, eps, kperm);
    } else {
        int threads = n >= 1024 ? 1024 : ((n + 31) / 32) * 32;
        launch_kernel(rms_norm_kernel<T, FUSED_ADD, false, 1>, dim3(rows), dim3(threads), 0, st, x, res, w, y, res_out, n, inv_n, eps, kperm);
    }
    return launch_status(name);
}

// ---------------------------------------------------------------------------
// elementwise
// ---------------------------------------------------------------------------
enum { OP_ADD = 0, OP_SILU_MUL = 1 };

__device__ __forceinline__ float silu_mul(float g, float u) {
    // silu(g) = g / (1 + exp(-g)), product in fp32 (elementwise.rs:178-183)
    return g / (expf(-g) + 1.0f) * u;
}

template <typename T, int OP>
__global__ void __launch_bounds__(256)
binary_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ out, int n, bool vector) {
    constexpr int VEC = Elem<T>::VEC;
    pdl_wait();
    pdl_launch_dependents();
    const int stride = gridDim.x * blockDim.x;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    const int nv = vector ? n / VEC : 0;
    for (int i = tid; i < nv; i += stride) {
        float x[VEC], y[VEC], o[VEC];
        Elem<T>::load(a + (size_t)i * VEC, x);
        Elem<T>::load(b + (size_t)i * VEC, y);
#pragma unroll
        for (int j = 0; j < VEC; ++j) o[j] = OP == OP_ADD ? x[j] + y[j] : silu_mul(x[j], y[j]);
        Elem<T>::store(out + (size_t)i * VEC, o);
    }
    for (int i = nv * VEC + tid; i < n; i += stride) {
        float x = Elem<T>::ld1(a + i), y = Elem<T>::ld1(b + i);
        Elem<T>::st1(out + i, OP == OP_ADD ? x + y : silu_mul(x, y));
    }
}

template <typename T, int OP>
static int binary_launch(const char *name, const T *a, const T *b, T *out, int n, cudaStream_t st) {
    B200K_REQUIRE(n >= 0, B200K_E_SHAPE, "%s: n = %d", name, n);
    if (n == 0) return 0;  // nothing to do; empty buffers may legitimately be NULL
    B200K_REQUIRE(a && b && out, B200K_E_NULL, "%s: NULL pointer", name);
    const bool vec = aligned16(a) && aligned16(b) && aligned16(out);
    const int work = ceil_div(n, Elem<T>::VEC);
    int blocks = ceil_div(work, 256);
    const int cap = sm_count() * 16;
    if (blocks > cap) blocks = cap;
    launch_kernel(binary_kernel<T, OP>, dim3(blocks), dim3(256), 0, st, a, b, out, n, vec);
    return launch_status(name);
}

// gate_up [B, 2*inter]: gate = row[0:inter], up = row[inter:2*inter]  (elementwise.rs:199-206)
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_interleaved_kernel(const T *__restrict__ gu, T *__restrict__ out, int inter, int total, bool vector, bool kperm) {
    constexpr int VEC = Elem<T>::VEC;
    pdl_wait();
    pdl_launch_dependents();
    const int stride = gridDim.x * blockDim.x;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (vector) {
        const int nv = total / VEC, rowv = inter / VEC;
        for (int i = tid; i < nv; i += stride) {
            const int b = i / rowv, c = (i - b * rowv) * VEC;
            const T *row = gu + (size_t)b * 2 * inter;
            float g[VEC], u[VEC], o[VEC];
            Elem<T>::load(row + c, g);
            Elem<T>::load(row + inter + c, u);
#pragma unroll
            for (int j = 0; j < VEC; ++j) o[j] = silu_mul(g[j], u[j]);
            if (kperm) Elem<T>::store_kperm(out + (size_t)i * VEC, o);
            else Elem<T>::store(out + (size_t)i * VEC, o);
        }
    } else {
        for (int i = tid; i < total; i += stride) {
            const int b = i / inter, c = i - b * inter;
            const T *row = gu + (size_t)b * 2 * inter;
            Elem<T>::st1(out + i, silu_mul(Elem<T>::ld1(row + c), Elem<T>::ld1(row + inter + c)));
        }
    }
}

template <typename T>
static int silu_interleaved_launch(const char *name, const T *gu, T *out, int inter, int total, cudaStream_t st, bool kperm = false) {
    B200K_REQUIRE(gu && out, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(inter > 0 && total >= 0 && total % inter == 0, B200K_E_SHAPE,
                  "%s: inter %d, total %d (total must be a multiple of inter)", name, inter, total);
    if (total == 0) return 0;
    const bool vec = inter % Elem<T>::VEC == 0 && aligned16(gu) && aligned16(out);
    int blocks = ceil_div(ceil_div(total, Elem<T>::VEC), 256);
    const int cap = sm_count() * 16;
    if (blocks > cap) blocks = cap;
    B200K_REQUIRE(!kperm || (vec && Elem<T>::VEC == 8), B200K_E_SHAPE, "%s: the permuted output needs fp16 rows of a multiple of 8, 16-byte aligned", name);
    launch_kernel(silu_mul_interleaved_kernel<T>, dim3(blocks), dim3(256), 0, st, gu, out, inter, total, vec, kperm);
    return launch_status(name);
}

// ---------------------------------------------------------------------------
// RoPE: pairs (i, i + D/2); lo' = x0*c - x1*s, hi' = x1*c + x0*s (positional.rs:45-46)
// One thread per pair; consecutive threads take consecutive pairs of a head row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
rope_kernel(const T *__restrict__ x, const float *__restrict__ cos_t, const float *__restrict__ sin_t,
            const int32_t *__restrict__ positions, T *__restrict__ out, int heads, int half, long total_pairs) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total_pairs; i += (long)gridDim.x * blockDim.x) {
        const long th = i / half;
        const int p = (int)(i - th * half);
        const int tok = (int)(th / heads);
        const long cs = positions ? (long)positions[tok] * half + p : p;
        const float c = cos_t[cs], s = sin_t[cs];
        const long lo = th * 2 * half + p, hi = lo + half;
        const float x0 = Elem<T>::ld1(x + lo), x1 = Elem<T>::ld1(x + hi);
        Elem<T>::st1(out + lo, x0 * c - x1 * s);
        Elem<T>::st1(out + hi, x1 * c + x0 * s);
    }
}

template <typename T>
static int rope_launch(const char *name, const T *x, const float *c, const float *s, const int32_t *pos, T *out,
                       int heads, int head_dim, int tokens, cudaStream_t st) {
    B200K_REQUIRE(x && c && s && out, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && heads > 0 && tokens >= 0, B200K_E_SHAPE,
                  "%s: heads %d, head_dim %d, tokens %d", name, heads, head_dim, tokens);
    const long pairs = (long)tokens * heads * (head_dim / 2);
    if (pairs == 0) return 0;
    long blocks = (pairs + 255) / 256;
    const long cap = (long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    rope_kernel<T><<<(int)blocks, 256, 0, st>>>(x, c, s, pos, out, heads, head_dim / 2, pairs);
    return launch_status(name);
}

// ---------------------------------------------------------------------------
// kv-cache append.  Destination row of (b, h):
//   seq-major shared cache [max_seq,H,D]  : (pos*H + h)*D            (cache.rs:38-46)
//   head-major batched     [B,H,max_len,D]: ((b*H + h)*max_len + pos)*D
// ---------------------------------------------------------------------------
template <typename T, bool HEAD_MAJOR>
__global__ void __launch_bounds__(256)
kv_append_kernel(const T *__restrict__ nk, const T *__restrict__ nv, T *__restrict__ kc, T *__restrict__ vc,
                 const int32_t *__restrict__ idx, int heads, int d, int max_len, long total, int *status) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long bh = i / d;
        const int c = (int)(i - bh * d);
        const int b = (int)(bh / heads), h = (int)(bh - (long)b * heads);
        const long pos = idx[b];
        if (HEAD_MAJOR && (unsigned long)pos >= (unsigned long)max_len) {
            // a row index outside the cache: nothing is stored for this sequence, the status word says so
            if (c == 0 && h == 0 && status) atomicOr(status, 4);
            continue;
        }
        const long dst = HEAD_MAJOR ? (((long)b * heads + h) * max_len + pos) * d + c : (pos * heads + h) * d + c;
        kc[dst] = nk[i];
        vc[dst] = nv[i];
    }
}

// rope(q), rope(k) + append of k, v from a fused QKV row; grid = (chunks of a row, batch rows),
// one thread per (head, pair) for q/k and per element pair for v.
__global__ void __launch_bounds__(256)
rope_kv_append_kernel(const __half *__restrict__ qkv, const float *__restrict__ cos_t,
                      const float *__restrict__ sin_t, const int32_t *__restrict__ positions,
                      __half *__restrict__ q_out, __half *__restrict__ kc, __half *__restrict__ vc,
                      int32_t *__restrict__ lens_out, int hq, int hkv, int d, int max_len, int *status) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.y;
    const int half = d / 2;
    int pos = positions[b];
    // A position outside the cache (a decode loop that ran past max_len, or a negative index): the K/V rows are not
    // stored, q is rotated with the nearest valid table row so that every read stays in range, the length handed to
    // attention stays within the cache, and bit 2 of the status word reports it.
    const bool in_range = (unsigned)pos < (unsigned)max_len;
    if (!in_range) {
        pos = pos < 0 ? 0 : max_len - 1;
        if (status && threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, 4);
    }
    if (lens_out && threadIdx.x == 0 && blockIdx.x == 0) lens_out[b] = pos + 1;   // rows attention covers after this append
    const __half *row = qkv + (size_t)b * (hq + 2 * hkv) * d;
    const float *cr = cos_t + (size_t)pos * half, *sr = sin_t + (size_t)pos * half;
    const int rot_pairs = (hq + hkv) * half;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rot_pairs + hkv * half; i += gridDim.x * blockDim.x) {
        if (i < rot_pairs) {
            const int h = i / half, p = i - h * half;
            const float c = cr[p], s = sr[p];
            const float x0 = __half2float(row[h * d + p]), x1 = __half2float(row[h * d + p + half]);
            const __half lo = __float2half_rn(x0 * c - x1 * s), hi = __float2half_rn(x1 * c + x0 * s);
            if (h < hq) {
                __half *o = q_out + ((size_t)b * hq + h) * d;
                o[p] = lo;
                o[p + half] = hi;
            } else if (in_range) {
                __half *o = kc + (((size_t)b * hkv + (h - hq)) * max_len + pos) * d;
                o[p] = lo;
                o[p + half] = hi;
            }
        } else if (in_range) {
            const int j = i - rot_pairs;            // pair index inside the v block
            const int h = j / half, p = (j - h * half) * 2;
            const __half2 v = *reinterpret_cast<const __half2 *>(row + (hq + hkv + h) * d + p);
            *reinterpret_cast<__half2 *>(vc + (((size_t)b * hkv + h) * max_len + pos) * d + p) = v;
        }
    }
}

int rope_kv_append_lens_launch(const __half *qkv, const float *cos_t, const float *sin_t, const int32_t *positions,
                               __half *q_out, __half *kc, __half *vc, int32_t *lens_out, int hq, int hkv, int d,
                               int max_len, int batch, cudaStream_t st) {
    B200K_REQUIRE(qkv && cos_t && sin_t && positions && q_out && kc && vc, B200K_E_NULL,
                  "rope_kv_append_hm_f16: NULL pointer");
    B200K_REQUIRE(hq > 0 && hkv > 0 && d > 0 && d % 2 == 0 && max_len > 0 && batch >= 0, B200K_E_SHAPE,
                  "rope_kv_append_hm_f16: Hq %d, Hkv %d, D %d, max_len %d, batch %d", hq, hkv, d, max_len, batch);
    if (batch == 0) return 0;
    const int items = (hq + 2 * hkv) * (d / 2);
    launch_kernel(rope_kv_append_kernel, dim3(ceil_div(items, 256), batch), dim3(256), 0, st, qkv, cos_t, sin_t, positions, q_out, kc, vc,
                  lens_out, hq, hkv, d, max_len, status_word());
    return launch_status("rope_kv_append_hm_f16");
}

}  // namespace b200k

using namespace b200k;

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
// fp16 variants whose output is written in the pre-permuted order (see Elem<__half>::store_kperm); used by the
// decode layer to feed its int4 GEMMs
namespace b200k {
int rms_norm_f16_kperm(const __half *x, const __half *w, __half *y, int n, float inv_n, float eps, int rows, cudaStream_t st) {
    return rms_norm_launch<__half, false>("rms_norm_f16", x, nullptr, w, y, nullptr, n, inv_n, eps, rows, st, true);
}
int fused_add_rms_norm_f16_kperm(const __half *x, const __half *res, const __half *w, __half *y, __half *res_out, int n,
                                 float inv_n, float eps, int rows, cudaStream_t st) {
    return rms_norm_launch<__half, true>("fused_add_rms_norm_f16", x, res, w, y, res_out, n, inv_n, eps, rows, st, true);
}
int silu_mul_interleaved_f16_kperm(const __half *gu, __half *out, int inter, int total, cudaStream_t st) {
    return silu_interleaved_launch<__half>("fused_silu_mul_interleaved_f16", gu, out, inter, total, st, true);
}
}  // namespace b200k

extern "C" int rms_norm_f16(const b200k_half *input, const b200k_half *weight, b200k_half *output, int row_size,
                            float inv_n, float eps, int num_rows, b200k_stream stream) {
    return rms_norm_launch<__half, false>("rms_norm_f16", (const __half *)input, nullptr, (const __half *)weight,
                                          (__half *)output, nullptr, row_size, inv_n, eps, num_rows, to_stream(stream));
}
extern "C" int rms_norm_f32(const float *input, const float *weight, float *output, int row_size, float inv_n,
                            float eps, int num_rows, b200k_stream stream) {
    return rms_norm_launch<float, false>("rms_norm_f32", input, nullptr, weight, output, nullptr, row_size, inv_n, eps,
                                         num_rows, to_stream(stream));
}
extern "C" int fused_add_rms_norm_f16(const b200k_half *input, const b200k_half *residual, const b200k_half *weight,
                                      b200k_half *output, b200k_half *residual_out, int hidden_size, float inv_n,
                                      float eps, int num_rows, b200k_stream stream) {
    return rms_norm_launch<__half, true>("fused_add_rms_norm_f16", (const __half *)input, (const __half *)residual,
                                         (const __half *)weight, (__half *)output, (__half *)residual_out, hidden_size,
                                         inv_n, eps, num_rows, to_stream(stream));
}
extern "C" int fused_add_rms_norm_f32(const float *input, const float *residual, const float *weight, float *output,
                                      float *residual_out, int hidden_size, float inv_n, float eps, int num_rows,
                                      b200k_stream stream) {
    return rms_norm_launch<float, true>("fused_add_rms_norm_f32", input, residual, weight, output, residual_out,
                                        hidden_size, inv_n, eps, num_rows, to_stream(stream));
}

extern "C" int residual_add_f16(const b200k_half *a, const b200k_half *b, b200k_half *out, int n, b200k_stream s) {
    return binary_launch<__half, OP_ADD>("residual_add_f16", (const __half *)a, (const __half *)b, (__half *)out, n,
                                         to_stream(s));
}
extern "C" int residual_add_f32(const float *a, const float *b, float *out, int n, b200k_stream s) {
    return binary_launch<float, OP_ADD>("residual_add_f32", a, b, out, n, to_stream(s));
}
extern "C" int residual_add_inplace_f16(b200k_half *a, const b200k_half *b, int n, b200k_stream s) {
    return binary_launch<__half, OP_ADD>("residual_add_inplace_f16", (const __half *)a, (const __half *)b, (__half *)a,
                                         n, to_stream(s));
}
extern "C" int residual_add_inplace_f32(float *a, const float *b, int n, b200k_stream s) {
    return binary_launch<float, OP_ADD>("residual_add_inplace_f32", a, b, a, n, to_stream(s));
}
extern "C" int fused_silu_mul_f16(const b200k_half *gate, const b200k_half *up, b200k_half *out, int n,
                                  b200k_stream s) {
    return binary_launch<__half, OP_SILU_MUL>("fused_silu_mul_f16", (const __half *)gate, (const __half *)up,
                                              (__half *)out, n, to_stream(s));
}
extern "C" int fused_silu_mul_f32(const float *gate, const float *up, float *out, int n, b200k_stream s) {
    return binary_launch<float, OP_SILU_MUL>("fused_silu_mul_f32", gate, up, out, n, to_stream(s));
}
extern "C" int fused_silu_mul_interleaved_f16(const b200k_half *gate_up, b200k_half *out, int inter, int total,
                                              b200k_stream s) {
    return silu_interleaved_launch<__half>("fused_silu_mul_interleaved_f16", (const __half *)gate_up, (__half *)out,
                                           inter, total, to_stream(s));
}
extern "C" int fused_silu_mul_interleaved_f32(const float *gate_up, float *out, int inter, int total, b200k_stream s) {
    return silu_interleaved_launch<float>("fused_silu_mul_interleaved_f32", gate_up, out, inter, total, to_stream(s));
}

extern "C" int rope_q_f32(const float *q, const float *cos_table, const float *sin_table, float *q_out, int head_dim,
                          int num_heads, b200k_stream s) {
    return rope_launch<float>("rope_q_f32", q, cos_table, sin_table, nullptr, q_out, num_heads, head_dim, 1,
                              to_stream(s));
}
extern "C" int rope_k_f32(const float *k, const float *cos_table, const float *sin_table, float *k_out, int head_dim,
                          int num_heads, b200k_stream s) {
    return rope_launch<float>("rope_k_f32", k, cos_table, sin_table, nullptr, k_out, num_heads, head_dim, 1,
                              to_stream(s));
}
extern "C" int rope_full_f32(const float *q, const float *cos_table, const float *sin_table, const int32_t *positions,
                             float *q_out, int num_heads, int head_dim, int num_tokens, b200k_stream s) {
    B200K_REQUIRE(positions, B200K_E_NULL, "rope_full_f32: positions is NULL");
    return rope_launch<float>("rope_full_f32", q, cos_table, sin_table, positions, q_out, num_heads, head_dim,
                              num_tokens, to_stream(s));
}
extern "C" int rope_full_f16(const b200k_half *q, const float *cos_table, const float *sin_table,
                             const int32_t *positions, b200k_half *q_out, int num_heads, int head_dim, int num_tokens,
                             b200k_stream s) {
    B200K_REQUIRE(positions, B200K_E_NULL, "rope_full_f16: positions is NULL");
    return rope_launch<__half>("rope_full_f16", (const __half *)q, cos_table, sin_table, positions, (__half *)q_out,
                               num_heads, head_dim, num_tokens, to_stream(s));
}

template <typename T, bool HM>
static int kv_append_launch(const char *name, const T *nk, const T *nv, T *kc, T *vc, const int32_t *idx, int heads,
                            int d, int max_len, int batch, cudaStream_t st) {
    B200K_REQUIRE(nk && nv && kc && vc && idx, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(heads > 0 && d > 0 && batch >= 0 && (!HM || max_len > 0), B200K_E_SHAPE,
                  "%s: heads %d, head_dim %d, batch %d", name, heads, d, batch);
    const long total = (long)batch * heads * d;
    if (total == 0) return 0;
    long blocks = (total + 255) / 256;
    const long cap = (long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    kv_append_kernel<T, HM><<<(int)blocks, 256, 0, st>>>(nk, nv, kc, vc, idx, heads, d, max_len, total, HM ? status_word() : nullptr);
    return launch_status(name);
}
extern "C" int kv_cache_append_f32(const float *new_keys, const float *new_values, float *k_cache, float *v_cache,
                                   const int32_t *cache_idx, int num_heads, int head_dim, int batch, b200k_stream s) {
    return kv_append_launch<float, false>("kv_cache_append_f32", new_keys, new_values, k_cache, v_cache, cache_idx,
                                          num_heads, head_dim, 0, batch, to_stream(s));
}
extern "C" int kv_cache_append_hm_f16(const b200k_half *new_keys, const b200k_half *new_values, b200k_half *k_cache,
                                      b200k_half *v_cache, const int32_t *cache_idx, int num_heads, int head_dim,
                                      int max_len, int batch, b200k_stream s) {
    return kv_append_launch<__half, true>("kv_cache_append_hm_f16", (const __half *)new_keys,
                                          (const __half *)new_values, (__half *)k_cache, (__half *)v_cache, cache_idx,
                                          num_heads, head_dim, max_len, batch, to_stream(s));
}
extern "C" int rope_kv_append_hm_f16(const b200k_half *qkv, const float *cos_table, const float *sin_table,
                                     const int32_t *positions, b200k_half *q_out, b200k_half *k_cache,
                                     b200k_half *v_cache, int num_q_heads, int num_kv_heads, int head_dim, int max_len,
                                     int batch, b200k_stream s) {
    return rope_kv_append_lens_launch((const __half *)qkv, cos_table, sin_table, positions, (__half *)q_out,
                                      (__half *)k_cache, (__half *)v_cache, nullptr, num_q_heads, num_kv_heads,
                                      head_dim, max_len, batch, to_stream(s));
}

// ---------------------------------------------------------------------------
// bf16 editions: the reference's `_typed` glue kernels are generic over T = f32 / f16 / bf16
// (crates/triton-dsl/tests/proc_macro_ferrum_typed.rs:6-19); same kernels, same fp32 arithmetic inside.
// ---------------------------------------------------------------------------
typedef __nv_bfloat16 bf16;
extern "C" int rms_norm_bf16(const b200k_bf16 *input, const b200k_bf16 *weight, b200k_bf16 *output, int row_size, float inv_n,
                             float eps, int num_rows, b200k_stream stream) {
    return rms_norm_launch<bf16, false>("rms_norm_bf16", (const bf16 *)input, nullptr, (const bf16 *)weight, (bf16 *)output, nullptr,
                                        row_size, inv_n, eps, num_rows, to_stream(stream));
}
extern "C" int fused_add_rms_norm_bf16(const b200k_bf16 *input, const b200k_bf16 *residual, const b200k_bf16 *weight,
                                       b200k_bf16 *output, b200k_bf16 *residual_out, int hidden_size, float inv_n, float eps,
                                       int num_rows, b200k_stream stream) {
    return rms_norm_launch<bf16, true>("fused_add_rms_norm_bf16", (const bf16 *)input, (const bf16 *)residual, (const bf16 *)weight,
                                       (bf16 *)output, (bf16 *)residual_out, hidden_size, inv_n, eps, num_rows, to_stream(stream));
}
extern "C" int residual_add_bf16(const b200k_bf16 *a, const b200k_bf16 *b, b200k_bf16 *out, int n, b200k_stream stream) {
    return binary_launch<bf16, OP_ADD>("residual_add_bf16", (const bf16 *)a, (const bf16 *)b, (bf16 *)out, n, to_stream(stream));
}
extern "C" int residual_add_inplace_bf16(b200k_bf16 *a, const b200k_bf16 *b, int n, b200k_stream stream) {
    return binary_launch<bf16, OP_ADD>("residual_add_inplace_bf16", (const bf16 *)a, (const bf16 *)b, (bf16 *)a, n, to_stream(stream));
}
extern "C" int fused_silu_mul_bf16(const b200k_bf16 *gate, const b200k_bf16 *up, b200k_bf16 *out, int n, b200k_stream stream) {
    return binary_launch<bf16, OP_SILU_MUL>("fused_silu_mul_bf16", (const bf16 *)gate, (const bf16 *)up, (bf16 *)out, n, to_stream(stream));
}
extern "C" int fused_silu_mul_interleaved_bf16(const b200k_bf16 *gate_up, b200k_bf16 *out, int inter, int total, b200k_stream stream) {
    return silu_interleaved_launch<bf16>("fused_silu_mul_interleaved_bf16", (const bf16 *)gate_up, (bf16 *)out, inter, total, to_stream(stream));
}
extern "C" int rope_full_bf16(const b200k_bf16 *q, const float *cos_table, const float *sin_table, const int32_t *positions,
                              b200k_bf16 *q_out, int num_heads, int head_dim, int num_tokens, b200k_stream stream) {
    B200K_REQUIRE(positions, B200K_E_NULL, "rope_full_bf16: positions is NULL");
    return rope_launch<bf16>("rope_full_bf16", (const bf16 *)q, cos_table, sin_table, positions, (bf16 *)q_out, num_heads, head_dim,
                             num_tokens, to_stream(stream));
}
extern "C" int kv_cache_append_hm_bf16(const b200k_bf16 *new_keys, const b200k_bf16 *new_values, b200k_bf16 *k_cache,
                                       b200k_bf16 *v_cache, const int32_t *cache_idx, int num_heads, int head_dim, int max_len,
                                       int batch, b200k_stream stream) {
    // a move of 16-bit elements: the fp16 kernel
    return kv_append_launch<__half, true>("kv_cache_append_hm_bf16", (const __half *)new_keys, (const __half *)new_values,
                                          (__half *)k_cache, (__half *)v_cache, cache_idx, num_heads, head_dim, max_len, batch,
                                          to_stream(stream));
}

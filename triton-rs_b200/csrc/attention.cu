// GQA decode attention over a KV cache.
//
// Two kernel families:
//  * attn_split_f16 (head_dim 128, fp16, GQA group size <= 8): split-KV flash-decode.
//    One CTA per (sequence, kv head, chunk of positions) serves ALL q heads of the
//    GQA group, so every K/V element is read from HBM once.  K/V tiles are staged into
//    shared memory by TMA tensor loads (4-D tensor map, 64 positions x 64 dims per box,
//    128-byte swizzle, mbarrier transaction counts) in a 3-deep ring of K+V tiles.
//    The products run on mma.sync m16n8k16 in transposed form (positions fill the 16
//    MMA rows, the group's q heads the 8 columns): one query token per sequence gives
//    at most 8 useful rows, far below the 64/128-row tcgen05 tile, and the kernel is
//    HBM-bound by a wide margin, so the warp-level MMA is the right-sized tool here.
//    Online softmax state is per warp; the four warps and then the chunks of a
//    (sequence, kv head) are merged by log-sum-exp, the latter by the last CTA to
//    arrive.  Every mbarrier wait is bounded and reports through a status word.
//  * attn_generic (any head_dim <= 256, fp16 or fp32): one CTA per (sequence, q head,
//    split); backs the f32 entry points and the explicit phase-1 / phase-2 API.
#include <stdlib.h>

#include <atomic>

#include <cuda_bf16.h>

#include "common.cuh"
#include "tma.cuh"

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
// split-KV fp16 family
// ---------------------------------------------------------------------------
constexpr int AT_D = 128;               // head_dim
#ifndef B200K_AT_WARPS
#define B200K_AT_WARPS 4
#endif
#ifndef B200K_AT_STAGES
#define B200K_AT_STAGES 3
#endif
constexpr int AT_THREADS = 32 * B200K_AT_WARPS;   // warp w owns rows [16w, 16w+16) of every tile
constexpr int AT_TILE = 16 * B200K_AT_WARPS;      // positions per stage
constexpr int AT_STAGES = B200K_AT_STAGES;        // each stage holds a K tile and a V tile
#ifdef B200K_AT_CTAS
constexpr int AT_CTAS_PER_SM = B200K_AT_CTAS;
#else
constexpr int AT_CTAS_PER_SM = (size_t)AT_STAGES * 4 * AT_TILE * 128 <= 100 * 1024 ? 2 : 1;
#endif
constexpr int AT_HALF_BYTES = AT_TILE * 128;   // one TMA box: AT_TILE rows x 64 dims (128 bytes), 128-byte swizzle
constexpr int AT_TILE_BYTES = 2 * AT_HALF_BYTES;
constexpr int AT_MAX_CH = 2048;         // largest chunk (positions)
constexpr int AT_NH = 8;                // head columns of one MMA (GQA group size <= 8)

struct AttnSplitArgs {
    const __half *q;        // [B, Hq, D]
    const __half *k, *v;
    __half *out;            // [B, Hq, D]
    const int32_t *lens;    // per sequence, or nullptr -> len_scalar
    int len_scalar;
    int hq, hkv, g;         // g = hq / hkv
    int chunk;              // positions per CTA, multiple of AT_TILE
    float scale_log2e;      // softmax scale * log2(e)
    int seq_major;          // tensor-map coordinate order: 0 = (d, pos, head, batch), 1 = (d, head, pos, batch)
    const int32_t *block_table;  // paged pools: batch coordinate = block_table[pos / block_size], pos -> slot
    int block_size, box_rows;    // rows per TMA box (64, or the block size of a paged pool when smaller)
    float *ws_acc;          // [B*Hkv*max_chunks, G, D]
    float *ws_ml;           // [B*Hkv*max_chunks, G, 2]  (max, sum)
    int *counters;          // [B*Hkv], zero between launches
    int *status;            // device status word (0 = ok; bit 0: a bounded wait gave up, bit 2: a length beyond max_len was clamped)
    int max_len;            // rows per (sequence, kv head) the cache holds: lengths are clamped to it
    int out_kperm;          // store every 8 output values of a head as (d0,d4,d1,d5,d2,d6,d3,d7), the order the int4 GEMM that
                            // consumes them wants (see gemm_tc.cu)
};

// index of element i of a row when every 8-chunk is stored as (0,4,1,5,2,6,3,7)
__device__ __forceinline__ long kperm_index(long i, int on) {
    const int e = (int)(i & 7);
    return on ? (i & ~7L) | (e < 4 ? 2 * e : 2 * (e - 4) + 1) : i;
}

struct AttnSmem {
    __align__(1024) unsigned char kv[AT_STAGES][2][2][AT_HALF_BYTES];   // [stage][K|V][dims 0-63 | 64-127][swizzled rows]
    float m[AT_THREADS / 32][AT_NH], l[AT_THREADS / 32][AT_NH];
    float wgt[AT_THREADS / 32][AT_NH], lsum[AT_NH], mfin[AT_NH];
    __align__(8) unsigned long long full[AT_STAGES];
    int abort_flag;
    int is_last;
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t movm_t(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The arithmetic runs transposed so that positions, not heads, fill the 16 rows of the
// MMA:  S^T[pos, head] = K[pos, :] . Q^T[:, head]   (A = K tile as stored, B = Q)
//       O^T[dim, head] += V^T[dim, pos] . P^T[pos, head]  (A = V tile via ldmatrix.trans,
//                                                          B = P^T via movmatrix)
// with up to 8 q heads of one GQA group in the 8 MMA columns.
__global__ void __launch_bounds__(AT_THREADS, AT_CTAS_PER_SM)
attn_split_f16_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                      AttnSplitArgs A) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    AttnSmem &S = *reinterpret_cast<AttnSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk_id = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int G = A.g;
    pdl_wait();                 // the lengths, q and the appended K/V rows come from the kernel before
    pdl_launch_dependents();
    int len = A.lens ? A.lens[b] : A.len_scalar;
    if (len > A.max_len) {
        // a length beyond the cache: attend to the rows that exist and say so (with more chunks than the grid has,
        // the arrival counter of this (sequence, kv head) would never reach its target)
        len = A.max_len;
        if (tid == 0 && chunk_id == 0) atomicOr(A.status, 4);
    }
    const int nchunks = (len + A.chunk - 1) / A.chunk;
    const long out_row0 = ((long)b * A.hq + (long)kvh * G) * AT_D;
    if (len <= 0) {
        // no keys: defined as a zero output row (the reference would divide 0 by 0)
        if (chunk_id == 0)
            for (int i = tid; i < G * AT_D; i += AT_THREADS) A.out[out_row0 + i] = __float2half_rn(0.f);
        return;
    }
    if (chunk_id >= nchunks) return;
    const int p0 = chunk_id * A.chunk;
    const int npos = min(A.chunk, len - p0);
    const int ntiles = (npos + AT_TILE - 1) / AT_TILE;

    if (tid == 0) {
        for (int s = 0; s < AT_STAGES; ++s) mbar_init(smem_u32(&S.full[s]), 1);
        S.abort_flag = 0;
        S.is_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // producer: one thread issues the four TMA boxes of tile t (K and V, two 64-dim halves each)
    // into stage t % STAGES.  A box always carries 64 rows: rows past the sequence end hold
    // whatever the cache holds there (or zeros past the tensor's extent); the consumer masks
    // their scores and clears their V rows.
    auto issue_tile = [&](int t) {
        const int st = t % AT_STAGES;
        const uint32_t bar = smem_u32(&S.full[st]);
        mbar_expect_tx(bar, 2 * AT_TILE_BYTES);
        for (int r0 = 0; r0 < AT_TILE; r0 += A.box_rows) {
            int pos = p0 + t * AT_TILE + r0, bc = b;
            if (A.block_table) {
                // a box past the sequence end may index past the table: clamp to the last valid block
                const int lb = min(pos, len - 1) / A.block_size;
                bc = A.block_table[lb];
                pos = pos % A.block_size;
            }
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const uint32_t kd = smem_u32(&S.kv[st][0][hf][r0 * 128]), vd = smem_u32(&S.kv[st][1][hf][r0 * 128]);
                if (A.seq_major) {
                    tma_load_4d(kd, &kmap, hf * 64, kvh, pos, bc, bar);
                    tma_load_4d(vd, &vmap, hf * 64, kvh, pos, bc, bar);
                } else {
                    tma_load_4d(kd, &kmap, hf * 64, pos, kvh, bc, bar);
                    tma_load_4d(vd, &vmap, hf * 64, pos, kvh, bc, bar);
                }
            }
        }
    };
    if (tid == 0) {
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
        for (int t = 0; t < min(AT_STAGES, ntiles); ++t) issue_tile(t);
    }

    // Q as the B operand: column n = head (lane / 4), k = dims 16*ks + 2*(lane%4) + {0,1} and +8
    uint32_t qf[8][2];
    {
        const int h = lane >> 2;
        const __half *qrow = A.q + out_row0 + (long)h * AT_D + 2 * (lane & 3);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qf[ks][0] = h < G ? *reinterpret_cast<const uint32_t *>(qrow + ks * 16) : 0u;
            qf[ks][1] = h < G ? *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + 8) : 0u;
        }
    }
    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) oacc[i][j] = 0.f;
    float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;   // heads 2*(lane%4) and +1

    // ldmatrix lane coordinates inside a tile, for this warp's 16 rows: row and 16-byte column
    const int k_row = warp * 16 + (lane & 15), k_c = lane >> 4;                          // K: A fragment as stored
    const int v_row = warp * 16 + ((lane >> 4) << 3) + (lane & 7), v_c = (lane >> 3) & 1; // V: A fragment transposed

    for (int t = 0; t < ntiles; ++t) {
        const int st = t % AT_STAGES;
        if (!S.abort_flag && !mbar_wait_bounded(smem_u32(&S.full[st]), (t / AT_STAGES) & 1)) {
            S.abort_flag = 1;
            atomicOr(A.status, 1);
        }
        const int rows_valid = npos - t * AT_TILE;     // < 64 only in the last tile of the sequence
        if (rows_valid < AT_TILE) {
            // P = 0 must multiply finite numbers: clear the V rows past the sequence end
            for (int i = tid; i < (AT_TILE - rows_valid) * 16; i += AT_THREADS) {
                const int r = rows_valid + (i >> 4), c = i & 15;
                *reinterpret_cast<uint4 *>(&S.kv[st][1][c >> 3][r * 128 + (c & 7) * 16]) = make_uint4(0, 0, 0, 0);
            }
            __syncthreads();
        }
        const int row0 = t * AT_TILE + warp * 16;      // first position of this warp's slab (within the chunk)
        if (row0 < npos) {
            const uint32_t kb = smem_u32(&S.kv[st][0][0][0]);
            const uint32_t vb = smem_u32(&S.kv[st][1][0][0]);
            float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a0, a1, a2, a3;
                ldsm_x4(kb + (ks >> 2) * AT_HALF_BYTES + swz128(k_row, (ks & 3) * 2 + k_c), a0, a1, a2, a3);
                mma_16816(s, a0, a1, a2, a3, qf[ks][0], qf[ks][1]);
            }
            // s[0],s[1]: position row0 + lane/4, heads 2*(lane%4), +1;  s[2],s[3]: position + 8
            const int pa = row0 + (lane >> 2);
            const bool va = pa < npos, vb8 = pa + 8 < npos;
            s[0] = va ? s[0] * A.scale_log2e : -1e30f;
            s[1] = va ? s[1] * A.scale_log2e : -1e30f;
            s[2] = vb8 ? s[2] * A.scale_log2e : -1e30f;
            s[3] = vb8 ? s[3] * A.scale_log2e : -1e30f;
            float t0 = fmaxf(s[0], s[2]), t1 = fmaxf(s[1], s[3]);
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, o));
                t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, o));
            }
            const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);
            const float al0 = exp2f(m0 - n0), al1 = exp2f(m1 - n1);
            m0 = n0;
            m1 = n1;
            const float p0v = exp2f(s[0] - n0), p1v = exp2f(s[1] - n1), p2v = exp2f(s[2] - n0), p3v = exp2f(s[3] - n1);
            l0 = l0 * al0 + p0v + p2v;
            l1 = l1 * al1 + p1v + p3v;
            if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    oacc[mt][0] *= al0; oacc[mt][1] *= al1; oacc[mt][2] *= al0; oacc[mt][3] *= al1;
                }
            }
            // P^T as the B operand: transpose the two 8x8 (position x head) blocks
            const uint32_t b0 = movm_t(f2_to_h2(p0v, p1v));
            const uint32_t b1 = movm_t(f2_to_h2(p2v, p3v));
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t a0, a1, a2, a3;
                ldsm_x4_t(vb + (mt >> 2) * AT_HALF_BYTES + swz128(v_row, (mt & 3) * 2 + v_c), a0, a1, a2, a3);
                mma_16816(oacc[mt], a0, a1, a2, a3, b0, b1);
            }
        }
        __syncthreads();  // every warp is done with stage st
        if (tid == 0 && t + AT_STAGES < ntiles) issue_tile(t + AT_STAGES);
    }

    // ---- merge the 4 warps: sums over the position lanes, then across warps ----
    // (the per-warp O^T partials reuse the K/V ring: every copy has landed and been consumed)
    float (*So)[AT_D][AT_NH] = reinterpret_cast<float (*)[AT_D][AT_NH]>(&S.kv[0][0][0][0]);
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    {
        const int h = 2 * (lane & 3), dr = lane >> 2;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            *reinterpret_cast<float2 *>(&So[warp][mt * 16 + dr][h]) = make_float2(oacc[mt][0], oacc[mt][1]);
            *reinterpret_cast<float2 *>(&So[warp][mt * 16 + dr + 8][h]) = make_float2(oacc[mt][2], oacc[mt][3]);
        }
        if (lane < 4) {
            S.m[warp][h] = m0; S.m[warp][h + 1] = m1;
            S.l[warp][h] = l0; S.l[warp][h + 1] = l1;
        }
    }
    __syncthreads();
    if (tid < AT_NH) {
        float M = S.m[0][tid];
        for (int w = 1; w < AT_THREADS / 32; ++w) M = fmaxf(M, S.m[w][tid]);
        float Ls = 0.f;
        for (int w = 0; w < AT_THREADS / 32; ++w) {
            const float wg = exp2f(S.m[w][tid] - M);
            S.wgt[w][tid] = wg;
            Ls += S.l[w][tid] * wg;
        }
        S.mfin[tid] = M;
        S.lsum[tid] = Ls;
    }
    __syncthreads();
    const long item = ((long)b * A.hkv + kvh) * gridDim.x + chunk_id;
    for (int i = tid; i < G * AT_D; i += AT_THREADS) {
        const int g = i / AT_D, d = i - g * AT_D;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < AT_THREADS / 32; ++w) o += So[w][d][g] * S.wgt[w][g];
        if (nchunks == 1)
            A.out[out_row0 + kperm_index(i, A.out_kperm)] = __float2half_rn(o / S.lsum[g]);
        else
            A.ws_acc[item * G * AT_D + i] = o;
    }
    if (nchunks == 1) return;
    if (tid < G) {
        A.ws_ml[(item * G + tid) * 2 + 0] = S.mfin[tid];
        A.ws_ml[(item * G + tid) * 2 + 1] = S.lsum[tid];
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
    // ---- last CTA of this (sequence, kv head): out = sum_c acc_c 2^(m_c - M) / sum_c l_c 2^(m_c - M) ----
    const long item0 = ((long)b * A.hkv + kvh) * gridDim.x;
    for (int i = tid; i < G * AT_D; i += AT_THREADS) {
        const int g = i / AT_D;
        float M = -1e30f;
        for (int c = 0; c < nchunks; ++c) M = fmaxf(M, __ldcg(&A.ws_ml[((item0 + c) * G + g) * 2]));
        float Lt = 0.f, o = 0.f;
        for (int c = 0; c < nchunks; ++c) {
            const float w = exp2f(__ldcg(&A.ws_ml[((item0 + c) * G + g) * 2]) - M);
            Lt += __ldcg(&A.ws_ml[((item0 + c) * G + g) * 2 + 1]) * w;
            o += __ldcg(&A.ws_acc[(item0 + c) * G * AT_D + i]) * w;
        }
        A.out[out_row0 + kperm_index(i, A.out_kperm)] = __float2half_rn(o / Lt);
    }
    if (tid == 0) A.counters[b * A.hkv + kvh] = 0;  // ready for the next launch
}

// Scratch layout (fixed offsets, so that the counters of one call shape can never be
// overwritten by the partials of another):
//   [0, 256)        status word
//   [256, 64 KiB)   arrival counters, one per (sequence, kv head); zero between launches
//   [64 KiB, 128 KiB) reserved for the GEMM family's counters
//   [128 KiB, ...)  (max, sum) pairs, then the un-normalised accumulators
constexpr size_t WS_COUNTERS_OFF = 256;
constexpr size_t WS_DATA_OFF = 128 * 1024;
constexpr int ATTN_MAX_COUNTERS = (64 * 1024 - 256) / 4;
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
    w.status = (int *)p;
    w.counters = (int *)(p + WS_COUNTERS_OFF);
    size_t off = WS_DATA_OFF;
    const size_t items = (size_t)batch * hkv * max_chunks;
    w.ml = (float *)(p + off);
    off += ((items * g * 2 * sizeof(float)) + 255) / 256 * 256;
    w.acc = (float *)(p + off);
    off += items * g * AT_D * sizeof(float);
    w.bytes = off;
    return w;
}

static int pick_chunk(int batch, int hkv, int max_len) {
    // The KV range of a sequence is cut into n equal chunks of whole tiles, one CTA each.  Measured on B200 at 4097
    // positions with 64 to 512 (sequence, kv head) rows: chunks of about 1100 positions (17 tiles) are the fastest at
    // every row count (up to 25 % ahead of both finer and coarser cuts): long enough to amortise a CTA's ring ramp
    // and its partial result, short enough that the last CTAs of the grid do not leave the machine idle for long.
    // Grids that cannot give every SM a CTA at that size are cut finer, down to 256 positions per chunk.
    {   // tuning override: positions per chunk (multiple of 64)
        const int v = env_int("B200K_ATTN_CHUNK", 0);
        if (v >= AT_TILE && v <= AT_MAX_CH && v % AT_TILE == 0) return v;
    }
    const long rows = (long)batch * hkv;
    int n = ceil_div(max_len, 1152);
    int chunk = ceil_div(ceil_div(max_len, n), AT_TILE) * AT_TILE;
    while (rows * n < sm_count() && n < 64) {
        const int finer = ceil_div(ceil_div(max_len, n + 1), AT_TILE) * AT_TILE;
        if (finer < 256) break;
        ++n;
        chunk = finer;
    }
    return min(chunk, AT_MAX_CH);
}

enum KvMode { KV_HEAD_MAJOR = 0, KV_SEQ_MAJOR = 1, KV_PAGED = 2 };
struct AttnCall {
    const __half *q, *k, *v;
    __half *out;
    const int32_t *lens;
    int len_scalar;
    int batch, hq, hkv, d;
    int max_len;        // longest sequence the grid must cover
    int mode;           // KvMode
    long pos_extent;    // extent of the position axis the TMA may touch (rows past it read as zero)
    long row_pitch;     // head-major: capacity (rows per head); seq-major: seq_len (rows per sequence)
    const int32_t *block_table;
    int block_size;
    float scale;
    void *ws;
    size_t ws_bytes;
    bool own_ws;
    cudaStream_t stream;
    bool out_kperm = false;
};

static int attn_split_launch(const char *name, AttnCall c) {
    const int g = c.hq / c.hkv;
    const int chunk = pick_chunk(c.batch, c.hkv, c.max_len);
    const int max_chunks = ceil_div(c.max_len, chunk);
    if (!c.ws && c.own_ws) {
        int rc = default_workspace(&c.ws, &c.ws_bytes);
        if (rc) return rc;
    }
    B200K_REQUIRE(c.ws, B200K_E_WORKSPACE, "%s: workspace is NULL", name);
    B200K_REQUIRE(c.batch * c.hkv <= ATTN_MAX_COUNTERS, B200K_E_SHAPE, "%s: batch * num_kv_heads = %d exceeds %d", name,
                  c.batch * c.hkv, ATTN_MAX_COUNTERS);
    AttnWs w = attn_ws_layout(c.ws, c.batch, c.hkv, g, max_chunks);
    B200K_REQUIRE(w.bytes <= c.ws_bytes, B200K_E_WORKSPACE, "%s: workspace %zu bytes, need %zu", name, c.ws_bytes, w.bytes);
    AttnSplitArgs A;
    A.q = c.q; A.k = c.k; A.v = c.v; A.out = c.out; A.lens = c.lens; A.len_scalar = c.len_scalar;
    A.out_kperm = c.out_kperm ? 1 : 0;
    A.hq = c.hq; A.hkv = c.hkv; A.g = g; A.chunk = chunk;
    A.scale_log2e = c.scale * 1.4426950408889634f;
    A.seq_major = c.mode != KV_HEAD_MAJOR;
    A.block_table = c.mode == KV_PAGED ? c.block_table : nullptr;
    A.block_size = c.block_size;
    A.box_rows = c.mode == KV_PAGED && c.block_size < AT_TILE ? c.block_size : AT_TILE;
    A.ws_acc = w.acc; A.ws_ml = w.ml; A.counters = w.counters; A.status = w.status; A.max_len = c.max_len;

    // tensor maps: innermost dimension = head_dim, then by ascending stride
    const uint64_t row = AT_D * 2;
    uint64_t dims[4], strides[3];
    uint32_t box[4];
    dims[0] = AT_D;
    box[0] = 64;
    if (c.mode == KV_HEAD_MAJOR) {          // [B, Hkv, pitch, D]
        dims[1] = (uint64_t)c.pos_extent; dims[2] = c.hkv; dims[3] = c.batch;
        strides[0] = row; strides[1] = (uint64_t)c.row_pitch * row; strides[2] = (uint64_t)c.hkv * c.row_pitch * row;
        box[1] = AT_TILE; box[2] = 1; box[3] = 1;
    } else if (c.mode == KV_SEQ_MAJOR) {    // [B, pitch, Hkv, D]
        dims[1] = c.hkv; dims[2] = (uint64_t)c.pos_extent; dims[3] = c.batch;
        strides[0] = row; strides[1] = (uint64_t)c.hkv * row; strides[2] = (uint64_t)c.row_pitch * c.hkv * row;
        box[1] = 1; box[2] = AT_TILE; box[3] = 1;
    } else {                                // [blocks, block_size, Hkv, D]
        dims[1] = c.hkv; dims[2] = c.block_size; dims[3] = 1u << 24;
        strides[0] = row; strides[1] = (uint64_t)c.hkv * row; strides[2] = (uint64_t)c.block_size * c.hkv * row;
        box[1] = 1; box[2] = A.box_rows; box[3] = 1;
    }
    CUtensorMap kmap, vmap;
    int rc = make_tensor_map(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, c.k, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tensor_map(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, c.v, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;

    const size_t smem = sizeof(AttnSmem) + 1024;
    {
        static OncePerDevice once;
        cudaError_t e = once.run([&] { return cudaFuncSetAttribute(attn_split_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
        if (e != cudaSuccess) return fail((int)e, "attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid(max_chunks, c.hkv, c.batch);
    launch_kernel(attn_split_f16_kernel, grid, dim3(AT_THREADS), smem, c.stream, kmap, vmap, A);
    return launch_status("decode attention (split-KV)");
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
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T *p, float v);
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
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

static bool split_ok(int hq, int hkv, int d, const void *q, const void *k, const void *v, const void *out) {
    const int g = hq / hkv;
    if (d != AT_D || g > AT_NH) return false;
    return aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out);
}

}  // namespace b200k

using namespace b200k;

// ---- fp16 single-sequence entry points ---------------------------------------
static int decode_f16_common(const char *name, const b200k_half *q, const b200k_half *k, const b200k_half *v,
                             b200k_half *out, int hq, int hkv, int d, int len, float scale, const KvLayout &L,
                             int mode, long row_pitch, b200k_stream stream) {
    int rc = attn_common_checks(name, q, k, v, out, hq, hkv, d, len);
    if (rc) return rc;
    bool fast = split_ok(hq, hkv, d, q, k, v, out);
    if (mode == KV_PAGED) {
        const int bs = L.block_size;   // whole TMA boxes: a power of two from 8 to 64, or a multiple of 64
        fast = fast && ((bs >= 8 && bs < 64 && (bs & (bs - 1)) == 0) || bs % 64 == 0);
    }
    if (fast) {
        AttnCall c = {};
        c.q = (const __half *)q; c.k = (const __half *)k; c.v = (const __half *)v; c.out = (__half *)out;
        c.lens = nullptr; c.len_scalar = len; c.batch = 1; c.hq = hq; c.hkv = hkv; c.d = d;
        c.max_len = len; c.mode = mode; c.pos_extent = len; c.row_pitch = row_pitch;
        c.block_table = L.block_table; c.block_size = L.block_size;
        c.scale = scale; c.ws = nullptr; c.own_ws = true;
        c.stream = to_stream(stream);
        return attn_split_launch(name, c);
    }
    return attn_generic_launch<__half>(name, q, k, v, out, 1, hq, hkv, d, len, scale, L, to_stream(stream));
}

extern "C" int decode_attention_f16(const b200k_half *q, const b200k_half *k_cache, const b200k_half *v_cache,
                                    b200k_half *output, int num_q_heads, int num_kv_heads, int head_dim,
                                    int valid_kv_len, float scale, b200k_stream stream) {
    KvLayout L = {0, head_dim, (long)num_kv_heads * head_dim, nullptr, 0, 0};
    return decode_f16_common("decode_attention_f16", q, k_cache, v_cache, output, num_q_heads, num_kv_heads, head_dim,
                             valid_kv_len, scale, L, KV_SEQ_MAJOR, valid_kv_len, stream);
}
extern "C" int decode_attention_hm_f16(const b200k_half *q, const b200k_half *k_cache, const b200k_half *v_cache,
                                       b200k_half *output, int num_q_heads, int num_kv_heads, int head_dim,
                                       int capacity, int valid_kv_len, float scale, b200k_stream stream) {
    B200K_REQUIRE(capacity >= valid_kv_len, B200K_E_SHAPE, "decode_attention_hm_f16: capacity %d < valid_kv_len %d",
                  capacity, valid_kv_len);
    KvLayout L = {0, (long)capacity * head_dim, head_dim, nullptr, 0, 0};
    return decode_f16_common("decode_attention_hm_f16", q, k_cache, v_cache, output, num_q_heads, num_kv_heads,
                             head_dim, valid_kv_len, scale, L, KV_HEAD_MAJOR, capacity, stream);
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
                             num_kv_heads, head_dim, valid_kv_len, scale, L, KV_PAGED, block_size, stream);
}

// ---- bf16 editions of the three `_typed` decode kernels (attention.rs:51-164, 182-273, 399-490 are generic over T):
// fp32 arithmetic on bf16 tensors, one CTA per (q head, split) on CUDA cores ---------------------------------------
extern "C" int decode_attention_bf16(const b200k_bf16 *q, const b200k_bf16 *k_cache, const b200k_bf16 *v_cache,
                                     b200k_bf16 *output, int num_q_heads, int num_kv_heads, int head_dim,
                                     int valid_kv_len, float scale, b200k_stream stream) {
    const char *name = "decode_attention_bf16";
    int rc = attn_common_checks(name, q, k_cache, v_cache, output, num_q_heads, num_kv_heads, head_dim, valid_kv_len);
    if (rc) return rc;
    KvLayout L = {0, head_dim, (long)num_kv_heads * head_dim, nullptr, 0, 0};
    return attn_generic_launch<__nv_bfloat16>(name, q, k_cache, v_cache, output, 1, num_q_heads, num_kv_heads, head_dim,
                                              valid_kv_len, scale, L, to_stream(stream));
}
extern "C" int decode_attention_hm_bf16(const b200k_bf16 *q, const b200k_bf16 *k_cache, const b200k_bf16 *v_cache,
                                        b200k_bf16 *output, int num_q_heads, int num_kv_heads, int head_dim, int capacity,
                                        int valid_kv_len, float scale, b200k_stream stream) {
    const char *name = "decode_attention_hm_bf16";
    int rc = attn_common_checks(name, q, k_cache, v_cache, output, num_q_heads, num_kv_heads, head_dim, valid_kv_len);
    if (rc) return rc;
    B200K_REQUIRE(capacity >= valid_kv_len, B200K_E_SHAPE, "%s: capacity %d < valid_kv_len %d", name, capacity, valid_kv_len);
    KvLayout L = {0, (long)capacity * head_dim, head_dim, nullptr, 0, 0};
    return attn_generic_launch<__nv_bfloat16>(name, q, k_cache, v_cache, output, 1, num_q_heads, num_kv_heads, head_dim,
                                              valid_kv_len, scale, L, to_stream(stream));
}
extern "C" int paged_decode_attention_bf16(const b200k_bf16 *q, const b200k_bf16 *k_block_pool, const b200k_bf16 *v_block_pool,
                                           const int32_t *block_table, b200k_bf16 *output, int num_q_heads, int num_kv_heads,
                                           int head_dim, int valid_kv_len, int block_size, float scale, b200k_stream stream) {
    const char *name = "paged_decode_attention_bf16";
    B200K_REQUIRE(block_table, B200K_E_NULL, "%s: block_table is NULL", name);
    B200K_REQUIRE(block_size > 0, B200K_E_SHAPE, "%s: block_size %d", name, block_size);
    int rc = attn_common_checks(name, q, k_block_pool, v_block_pool, output, num_q_heads, num_kv_heads, head_dim, valid_kv_len);
    if (rc) return rc;
    KvLayout L = {0, head_dim, (long)num_kv_heads * head_dim, block_table, block_size, (long)block_size * num_kv_heads * head_dim};
    return attn_generic_launch<__nv_bfloat16>(name, q, k_block_pool, v_block_pool, output, 1, num_q_heads, num_kv_heads, head_dim,
                                              valid_kv_len, scale, L, to_stream(stream));
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
    B200K_REQUIRE(split_ok(num_q_heads, num_kv_heads, head_dim, q, k_cache, v_cache, output), B200K_E_SHAPE,
                  "%s: needs head_dim 128, GQA group size <= 8 and 16-byte aligned tensors", name);
    AttnCall c = {};
    c.q = (const __half *)q; c.k = (const __half *)k_cache; c.v = (const __half *)v_cache; c.out = (__half *)output;
    c.lens = context_lens; c.len_scalar = 0; c.batch = batch_size; c.hq = num_q_heads; c.hkv = num_kv_heads;
    c.d = head_dim; c.max_len = max_len; c.mode = KV_HEAD_MAJOR; c.pos_extent = max_len; c.row_pitch = max_len;
    c.scale = scale;
    c.ws = workspace; c.ws_bytes = workspace_bytes; c.own_ws = workspace == nullptr;
    c.stream = to_stream(stream);
    return attn_split_launch(name, c);
}
// The same call with the output written in the pre-permuted order the int4 GEMM wants (used by the decode layer)
namespace b200k {
int batched_decode_attention_hm_f16_kperm(const __half *q, const __half *k_cache, const __half *v_cache,
                                          const int32_t *context_lens, __half *output, int batch_size, int num_q_heads,
                                          int num_kv_heads, int head_dim, int max_len, float scale, cudaStream_t st) {
    const char *name = "batched_decode_attention_hm_f16";
    B200K_REQUIRE(q && k_cache && v_cache && context_lens && output, B200K_E_NULL, "%s: NULL pointer", name);
    if (batch_size == 0) return 0;
    B200K_REQUIRE(split_ok(num_q_heads, num_kv_heads, head_dim, q, k_cache, v_cache, output), B200K_E_SHAPE,
                  "%s: needs head_dim 128, GQA group size <= 8 and 16-byte aligned tensors", name);
    AttnCall c = {};
    c.q = q; c.k = k_cache; c.v = v_cache; c.out = output;
    c.lens = context_lens; c.len_scalar = 0; c.batch = batch_size; c.hq = num_q_heads; c.hkv = num_kv_heads;
    c.d = head_dim; c.max_len = max_len; c.mode = KV_HEAD_MAJOR; c.pos_extent = max_len; c.row_pitch = max_len;
    c.scale = scale;
    c.ws = nullptr; c.ws_bytes = 0; c.own_ws = true;
    c.stream = st;
    c.out_kperm = true;
    return attn_split_launch(name, c);
}
}  // namespace b200k

extern "C" int batched_decode_attention_hm_f16(const b200k_half *q, const b200k_half *k_cache,
                                               const b200k_half *v_cache, const int32_t *context_lens,
                                               b200k_half *output, int batch_size, int num_q_heads, int num_kv_heads,
                                               int head_dim, int max_len, float scale, b200k_stream stream) {
    return batched_decode_attention_hm_f16_ws(q, k_cache, v_cache, context_lens, output, batch_size, num_q_heads,
                                              num_kv_heads, head_dim, max_len, scale, nullptr, 0, stream);
}
// ---- the same kernel for callers that cannot allocate ---------------------------------
// Scratch for the split-KV partials lives in this file-scope device array instead of a
// cudaMalloc'd workspace.  Every GPU that loads the library holds it until the process exits.
// In host code the array's name is only a stand-in; the device address is looked up once per
// device with cudaGetSymbolAddress and handed to the kernel like any other workspace.
static __device__ __align__(256) unsigned char g_attn_static_scratch[B200K_NOALLOC_SCRATCH_BYTES];

// Device address of the array on device `dev` (which must be current), looked up on first use and cached; the
// cache is an atomic pointer per device because first calls may come from several host threads (they all
// store the same value).  No allocation happens here.
static int noalloc_scratch(const char *name, int dev, void **out) {
    static std::atomic<void *> cache[16];
    void *p = cache[dev].load(std::memory_order_acquire);
    if (!p) {
        cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail((int)(e != cudaSuccess ? e : cudaErrorInvalidSymbol), "%s: cudaGetSymbolAddress: %s", name,
                        cudaGetErrorString(e));
        }
        cache[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return 0;
}

extern "C" int batched_decode_attention_hm_f16_noalloc(const b200k_half *q, const b200k_half *k_cache,
                                                       const b200k_half *v_cache, const int32_t *context_lens,
                                                       b200k_half *output, int batch_size, int num_q_heads,
                                                       int num_kv_heads, int head_dim, int max_len, float scale,
                                                       b200k_stream stream) {
    const char *name = "batched_decode_attention_hm_f16_noalloc";
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 16) {
        cudaGetLastError();
        return fail(B200K_E_DEVICE, "%s: no usable current device", name);
    }
    void *scratch = nullptr;
    int rc = noalloc_scratch(name, dev, &scratch);
    if (rc) return rc;
    const size_t need = b200k_attention_workspace_bytes(batch_size, num_q_heads, num_kv_heads, head_dim, max_len);
    B200K_REQUIRE(need <= (size_t)B200K_NOALLOC_SCRATCH_BYTES, B200K_E_WORKSPACE,
                  "%s: this call needs %zu bytes of scratch, the built-in array holds %zu (batch %d, kv heads %d, "
                  "max_len %d): use batched_decode_attention_hm_f16_ws with a caller-owned workspace",
                  name, need, (size_t)B200K_NOALLOC_SCRATCH_BYTES, batch_size, num_kv_heads, max_len);
    return batched_decode_attention_hm_f16_ws(q, k_cache, v_cache, context_lens, output, batch_size, num_q_heads,
                                              num_kv_heads, head_dim, max_len, scale, scratch,
                                              (size_t)B200K_NOALLOC_SCRATCH_BYTES, stream);
}

extern "C" int b200k_noalloc_status(int *host_status_out, b200k_stream stream) {
    const char *name = "b200k_noalloc_status";
    B200K_REQUIRE(host_status_out, B200K_E_NULL, "%s: NULL pointer", name);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 16) {
        cudaGetLastError();
        return fail(B200K_E_DEVICE, "%s: no usable current device", name);
    }
    void *scratch = nullptr;
    int rc = noalloc_scratch(name, dev, &scratch);
    if (rc) return rc;
    return b200k_workspace_status(scratch, host_status_out, stream);
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

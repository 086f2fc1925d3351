// Causal prefill attention (flash_attn_full, fp16, head_dim 128) on the 5th-generation tensor cores.
//
// One CTA per (sequence, q head, tile of 128 query rows).  Both contractions of a KV tile of 128 positions are
// tcgen05.mma instructions with their accumulators in tensor memory:
//     S = Q K^T     A = Q tile (shared memory, K-major), B = K tile (shared memory, K-major)      128 x 128 x 128
//     O'= P V       A = P (fp16, written to tensor memory by the softmax warps), B = V tile (shared memory, MN-major)
// Warp roles:  warps 0..3  softmax + output: thread = one query row = one tensor-memory lane; running max, sum and the
//                          128 output values of its row stay in registers (fp32)
//              warp 4      TMA producer: Q once, K and V tiles into two-deep rings (4-D tensor maps, 128-byte swizzle)
//              warp 5      MMA issuer (one thread)
// Per KV tile j the issuer queues S(j+1) ahead of P(j) V(j), so the tensor pipe computes the next scores while the
// softmax warps turn S(j) into P(j), and P(j) V(j) runs while they take the row maxima of S(j+1):
//     softmax(j):  wait S(j) -> row max, alpha = 2^(m_old - m_new) -> wait P(j-1)V(j-1): O = (O + O') * alpha
//                  -> P(j) = 2^(S(j) - m_new), l = l * alpha + sum P(j) -> tensor memory -> signal
// Causal structure: query row i sees kv positions 0 .. min(pos_offset + i, kv_len - 1); KV tiles entirely above the
// diagonal of the query tile are never loaded, tiles entirely below it skip the mask.
// Every mbarrier wait is bounded; a wait that gives up sets the status word and the CTA drains.
#include "tcgen05.cuh"
#include "tma.cuh"

namespace b200k {

constexpr int PT_D = 128, PT_BQ = 128, PT_BKV = 128;
constexpr int PT_THREADS = 192;
constexpr int PT_TILE_BYTES = PT_BQ * PT_D * 2;           // 32 KiB: two halves of [128 rows][64 dims] (128-byte rows, swizzled)
constexpr int PT_HALF_BYTES = PT_TILE_BYTES / 2;
constexpr int PT_STAGES = 2;
// tensor-memory columns
constexpr uint32_t PT_COL_S = 0;        // S(j) at 128 * (j % 2)
constexpr uint32_t PT_COL_O = 256;      // P V of the current tile (fp32)
constexpr uint32_t PT_COL_P = 384;      // P as fp16 pairs: 64 columns
constexpr uint32_t PT_COLS = 512;

struct PtArgs {
    __half *out;
    int hq, hkv, q_len, kv_len, pos_offset;
    float scale_log2e;
    int *status;
};

enum {
    PB_Q = 0,
    PB_KFULL = 1,                    // [2] K tile landed
    PB_KFREE = 3,                    // [2] K tile consumed (S MMAs retired)
    PB_VFULL = 5,                    // [2]
    PB_VFREE = 7,                    // [2] V tile consumed (P V MMAs retired)
    PB_SFULL = 9,                    // [2] S(j) complete in tensor memory
    PB_SFREE = 11,                   // [2] S(j) read by the softmax warps for the last time (4 arrivals)
    PB_PFULL = 13,                   // P(j) written (4 arrivals)
    PB_ODONE = 14,                   // P(j) V(j) retired
    PB_COUNT = 15
};

__global__ void __launch_bounds__(PT_THREADS, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                  const __grid_constant__ CUtensorMap vmap, PtArgs A) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *q_tile = smem;                                   // 32 KiB
    unsigned char *k_tile = q_tile + PT_TILE_BYTES;                 // [2][32 KiB]
    unsigned char *v_tile = k_tile + PT_STAGES * PT_TILE_BYTES;     // [2][32 KiB]
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(v_tile + PT_STAGES * PT_TILE_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + PB_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = gridDim.x - 1 - blockIdx.x;        // long tiles first
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / (A.hq / A.hkv);
    const int q0 = qt * PT_BQ;
    // KV tiles this query tile needs: positions 0 .. min(pos_offset + q0 + 127, kv_len - 1)
    const int last_pos = min(A.pos_offset + min(q0 + PT_BQ, A.q_len) - 1, A.kv_len - 1);
    const int ntiles = last_pos / PT_BKV + 1;

    if (tid == 0) {
        mbar_init(smem_u32(&bars[PB_Q]), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bars[PB_KFULL + s]), 1);
            mbar_init(smem_u32(&bars[PB_KFREE + s]), 1);
            mbar_init(smem_u32(&bars[PB_VFULL + s]), 1);
            mbar_init(smem_u32(&bars[PB_VFREE + s]), 1);
            mbar_init(smem_u32(&bars[PB_SFULL + s]), 1);
            mbar_init(smem_u32(&bars[PB_SFREE + s]), 4);
        }
        mbar_init(smem_u32(&bars[PB_PFULL]), 4);
        mbar_init(smem_u32(&bars[PB_ODONE]), 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), PT_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    auto wait = [&](int bar_idx, uint32_t parity) {
        const uint32_t bar = smem_u32(&bars[bar_idx]);
        if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;                     // some wait already gave up: drain without waiting again
        if (!mbar_wait_bounded(bar, parity)) {
            *abort_flag = 1;
            atomicOr(A.status, 2);
        }
    };

    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&qmap);
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&vmap);
            const uint32_t qb = smem_u32(&bars[PB_Q]);
            mbar_expect_tx(qb, PT_TILE_BYTES);
            tma_load_4d(smem_u32(q_tile), &qmap, 0, q0, h, b, qb);
            tma_load_4d(smem_u32(q_tile + PT_HALF_BYTES), &qmap, 64, q0, h, b, qb);
            for (int j = 0; j < ntiles; ++j) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)(j >> 1) & 1u;
                if (j >= PT_STAGES) wait(PB_KFREE + s, ph ^ 1u);
                const uint32_t kb = smem_u32(&bars[PB_KFULL + s]);
                mbar_expect_tx(kb, PT_TILE_BYTES);
                tma_load_4d(smem_u32(k_tile + s * PT_TILE_BYTES), &kmap, 0, j * PT_BKV, kvh, b, kb);
                tma_load_4d(smem_u32(k_tile + s * PT_TILE_BYTES + PT_HALF_BYTES), &kmap, 64, j * PT_BKV, kvh, b, kb);
                if (j >= PT_STAGES) wait(PB_VFREE + s, ph ^ 1u);
                const uint32_t vb = smem_u32(&bars[PB_VFULL + s]);
                mbar_expect_tx(vb, PT_TILE_BYTES);
                tma_load_4d(smem_u32(v_tile + s * PT_TILE_BYTES), &vmap, 0, j * PT_BKV, kvh, b, vb);
                tma_load_4d(smem_u32(v_tile + s * PT_TILE_BYTES + PT_HALF_BYTES), &vmap, 64, j * PT_BKV, kvh, b, vb);
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc(PT_BQ, PT_BKV, 0);          // A, B K-major
            const uint32_t idesc_o = umma_idesc_b_mn(PT_BQ, PT_D);          // A from tensor memory, B (V) MN-major
            const uint64_t dq = umma_desc(smem_u32(q_tile), 16, 1024);
            auto issue_s = [&](int j) {
                const int s = j & 1;
                wait(PB_KFULL + s, (uint32_t)(j >> 1) & 1u);
                if (j >= 2) wait(PB_SFREE + s, ((uint32_t)(j >> 1) & 1u) ^ 1u);      // S(j - 2) has been read
                tc_fence_after();
                const uint64_t dk = umma_desc(smem_u32(k_tile + s * PT_TILE_BYTES), 16, 1024);
#pragma unroll
                for (int kk = 0; kk < PT_D / 16; ++kk) {
                    // 16 dims per MMA: 32 bytes inside the 128-byte swizzle row; dims 64.. live in the second half tile
                    const uint64_t off = (uint64_t)(((kk >> 2) * PT_HALF_BYTES + (kk & 3) * 32) >> 4);
                    tc_mma_f16(tmem + PT_COL_S + s * 128, dq + off, dk + off, idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit(smem_u32(&bars[PB_SFULL + s]));
                tc_commit(smem_u32(&bars[PB_KFREE + s]));
            };
            wait(PB_Q, 0);
            issue_s(0);
            for (int j = 0; j < ntiles; ++j) {
                if (j + 1 < ntiles) issue_s(j + 1);
                const int s = j & 1;
                wait(PB_VFULL + s, (uint32_t)(j >> 1) & 1u);
                wait(PB_PFULL, (uint32_t)j & 1u);
                tc_fence_after();
                const uint64_t dv = umma_desc(smem_u32(v_tile + s * PT_TILE_BYTES), PT_HALF_BYTES, 1024);   // MN-major: dim halves 16 KiB apart
#pragma unroll
                for (int kk = 0; kk < PT_BKV / 16; ++kk)      // 16 kv positions per MMA: 8 columns of P, 16 rows (2 KiB) of V
                    tc_mma_f16_ts(tmem + PT_COL_O, tmem + PT_COL_P + kk * 8, dv + (uint64_t)((kk * 2048) >> 4), idesc_o, kk > 0 ? 1u : 0u);
                tc_commit(smem_u32(&bars[PB_ODONE]));
                tc_commit(smem_u32(&bars[PB_VFREE + s]));
            }
        }
    } else {
        // ---------------- softmax + output: thread = query row ----------------
        const int row = warp * 32 + lane;                 // tensor-memory lane
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        const int qi = q0 + row;
        const int limit = min(A.pos_offset + qi, A.kv_len - 1);      // last kv position this row sees
        float o[PT_D];
#pragma unroll
        for (int i = 0; i < PT_D; ++i) o[i] = 0.f;
        float m = -1e30f, l = 0.f;
        for (int j = 0; j < ntiles; ++j) {
            const int s = j & 1, k0 = j * PT_BKV;
            const bool masked = k0 + PT_BKV - 1 > A.pos_offset + q0 || k0 + PT_BKV > A.kv_len;     // some row of the tile needs the mask
            wait(PB_SFULL + s, (uint32_t)(j >> 1) & 1u);
            tc_fence_after();
            // pass 1: row maximum
            float mx = -1e30f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(lane_base + PT_COL_S + s * 128 + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float v = __uint_as_float(r[i]);
                    if (masked && k0 + c * 32 + i > limit) v = -1e30f;
                    mx = fmaxf(mx, v);
                }
            }
            const float m_new = fmaxf(m, mx * A.scale_log2e);     // scores are compared in the scaled, base-2 domain
            const float alpha = exp2f(m - m_new);
            // the product of the tile before: O = (O + P V) * alpha
            if (j > 0) {
                wait(PB_ODONE, (uint32_t)(j - 1) & 1u);
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld32(lane_base + PT_COL_O + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(r[i])) * alpha;
                }
            }
            // pass 2: P = 2^(s * scale * log2e - m_new), written to tensor memory as fp16 pairs
            float psum = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(lane_base + PT_COL_S + s * 128 + c * 32, r);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = exp2f(__uint_as_float(r[i]) * A.scale_log2e - m_new);
                    float p1 = exp2f(__uint_as_float(r[i + 1]) * A.scale_log2e - m_new);
                    if (masked) {
                        if (k0 + c * 32 + i > limit) p0 = 0.f;
                        if (k0 + c * 32 + i + 1 > limit) p1 = 0.f;
                    }
                    // the sum runs over the fp16-rounded probabilities that the second product sees
                    const __half2 hp = __floats2half2_rn(p0, p1);
                    const float2 back = __half22float2(hp);
                    psum += back.x + back.y;
                    pk[i >> 1] = *reinterpret_cast<const uint32_t *>(&hp);
                }
                // 16 columns of P per 32 scores
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                    ::"r"(lane_base + PT_COL_P + c * 16), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]),
                      "r"(pk[6]), "r"(pk[7]), "r"(pk[8]), "r"(pk[9]), "r"(pk[10]), "r"(pk[11]), "r"(pk[12]), "r"(pk[13]),
                      "r"(pk[14]), "r"(pk[15])
                    : "memory");
            }
            tmem_st_wait();
            tc_fence_before();
            l = l * alpha + psum;
            m = m_new;
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&bars[PB_PFULL]));          // P(j) is in tensor memory
                mbar_arrive(smem_u32(&bars[PB_SFREE + s]));      // S(j) will not be read again
            }
        }
        // the last tile's product
        wait(PB_ODONE, (uint32_t)(ntiles - 1) & 1u);
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const bool live = qi < A.q_len;
        __half *dst = A.out + (((long)b * A.hq + h) * A.q_len + qi) * PT_D;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(lane_base + PT_COL_O + c * 32, r);
            tmem_ld_wait();
            if (live) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 u;
                    u.x = f2_to_h2((o[c * 32 + i] + __uint_as_float(r[i])) * inv, (o[c * 32 + i + 1] + __uint_as_float(r[i + 1])) * inv);
                    u.y = f2_to_h2((o[c * 32 + i + 2] + __uint_as_float(r[i + 2])) * inv, (o[c * 32 + i + 3] + __uint_as_float(r[i + 3])) * inv);
                    u.z = f2_to_h2((o[c * 32 + i + 4] + __uint_as_float(r[i + 4])) * inv, (o[c * 32 + i + 5] + __uint_as_float(r[i + 5])) * inv);
                    u.w = f2_to_h2((o[c * 32 + i + 6] + __uint_as_float(r[i + 6])) * inv, (o[c * 32 + i + 7] + __uint_as_float(r[i + 7])) * inv);
                    *reinterpret_cast<uint4 *>(dst + c * 32 + i) = u;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, PT_COLS);
}

// Returns TC-style "not covered" (-1000) when the shape is outside this kernel (the caller then runs the general one).
int prefill_tc_launch(const __half *q, const __half *k, const __half *v, __half *out, int batch, int hq, int hkv, int q_len,
                      int kv_len, int d, int pos_offset, float scale, cudaStream_t st) {
    constexpr int NOT_COVERED = -1000;
    if (d != PT_D || pos_offset < 0 || kv_len < 1 || q_len < 1 || hq % hkv) return NOT_COVERED;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return NOT_COVERED;
    if (hq > 65535 || batch > 65535) return NOT_COVERED;
    int *status = status_word();
    if (!status) return NOT_COVERED;
    const uint64_t row = PT_D * 2;
    CUtensorMap qmap, kmap, vmap;
    const uint32_t box[4] = {64, PT_BQ, 1, 1};
    {
        const uint64_t dims[4] = {PT_D, (uint64_t)q_len, (uint64_t)hq, (uint64_t)batch};
        const uint64_t str[3] = {row, (uint64_t)q_len * row, (uint64_t)hq * q_len * row};
        if (make_tensor_map(&qmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return NOT_COVERED;
    }
    {
        const uint64_t dims[4] = {PT_D, (uint64_t)kv_len, (uint64_t)hkv, (uint64_t)batch};
        const uint64_t str[3] = {row, (uint64_t)kv_len * row, (uint64_t)hkv * kv_len * row};
        if (make_tensor_map(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, k, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return NOT_COVERED;
        if (make_tensor_map(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, v, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return NOT_COVERED;
    }
    PtArgs A;
    A.out = out; A.hq = hq; A.hkv = hkv; A.q_len = q_len; A.kv_len = kv_len; A.pos_offset = pos_offset;
    A.scale_log2e = scale * 1.4426950408889634f;
    A.status = status;
    const size_t smem = (size_t)(1 + 2 * PT_STAGES) * PT_TILE_BYTES + PB_COUNT * 8 + 16 + 1024;
    {
        static OncePerDevice once;
        cudaError_t e = once.run([&] { return cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
        if (e != cudaSuccess) return fail((int)e, "flash_attn_full_f16: shared memory %zu: %s", smem, cudaGetErrorString(e));
    }
    const dim3 grid(ceil_div(q_len, PT_BQ), hq, batch);
    prefill_tc_kernel<<<grid, PT_THREADS, smem, st>>>(qmap, kmap, vmap, A);
    return launch_status("flash_attn_full_f16");
}

}  // namespace b200k

// Causal prefill attention (flash_attn_full, fp16 or bf16, head_dim 128) on the 5th-generation tensor cores.
//
// One CTA per (sequence, q head, PAIR of 128-row query tiles a, b).  Both contractions of a KV tile of 128 positions
// are tcgen05.mma instructions with their accumulators in tensor memory:
//     S = Q K^T     A = Q tile (shared memory, K-major), B = K tile (shared memory, K-major)      128 x 128 x 128
//     O += P V      A = P (fp16, written to tensor memory by the softmax warps), B = V tile (shared memory, MN-major)
// Tensor memory (512 columns): S_a [0,128)  S_b [128,256)  O_a [256,384)  O_b [384,512).  P_x overwrites the first 64
// columns of S_x: a thread owns one query row = one lane, holds its whole S row in registers before it writes P, and the
// tensor pipe runs one CTA's MMAs in issue order, so S_x(j+1) is issued behind P_x(j) V(j) and cannot overtake it.
// Warp roles:  warps 0..3 / 4..7  softmax of tile a / b (thread = query row = tensor-memory lane)
//              warp 8             TMA producer: both Q tiles once, K and V tiles into two-deep rings shared by a and b
//                                 (4-D tensor maps, 128-byte swizzle)
//              warp 9             MMA issuer (one thread)
//              warps 10, 11       idle (they complete the warpgroup whose registers setmaxnreg gives away)
// Issue order per KV tile j:  P_a(j)V(j), S_a(j+1), P_b(j)V(j), S_b(j+1): while one tile's softmax warps work, the tensor
// pipe serves the other tile.
// Softmax per row, base-2 domain: the output accumulates in tensor memory across KV tiles without being read back.  The
// running maximum m is only raised when the tile's maximum exceeds it by more than 8 (a factor 256, far inside fp16 and
// fp32 range); then the warp rescales its 32 rows of O in tensor memory (load, multiply, store) and l.  Otherwise P is
// computed against the older m, which the final division by l cancels exactly.
// Causal structure: query row i sees kv positions 0 .. min(pos_offset + i, kv_len - 1); KV tiles entirely above the
// diagonal of a query tile are never multiplied for it (and never loaded if neither tile needs them), tiles entirely
// below it skip the mask.
// Every mbarrier wait is bounded; a wait that gives up sets the status word and the CTA drains.
#include <cuda_bf16.h>

#include "tcgen05.cuh"
#include "tma.cuh"

namespace b200k {

constexpr int PT_D = 128, PT_BQ = 128, PT_BKV = 128;
constexpr int PT_SOFTMAX_WARPS = 8;
constexpr int PT_THREADS = (PT_SOFTMAX_WARPS + 4) * 32;     // third warpgroup: TMA warp, MMA warp, two idle warps
// Registers: 384 threads get 168 each at launch; the third warpgroup hands most of its share to the softmax warps
// (2 x 128 x 232 + 128 x 40 = 384 x 168), whose rows of 128 scores live in registers.
constexpr int PT_REGS_SOFTMAX = 232, PT_REGS_AUX = 40;
constexpr int PT_TILE_BYTES = PT_BQ * PT_D * 2;           // 32 KiB: two halves of [128 rows][64 dims] (128-byte rows, swizzled)
constexpr int PT_HALF_BYTES = PT_TILE_BYTES / 2;
constexpr int PT_STAGES = 2;
constexpr uint32_t PT_COL_S = 0;        // S_x at 128 x; P_x on its first 64 columns
constexpr uint32_t PT_COL_O = 256;      // O_x at 256 + 128 x
constexpr uint32_t PT_COLS = 512;
constexpr float PT_RESCALE_THRESHOLD = 8.f;

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
    PB_SFULL = 9,                    // [2: tile a, b] S_x(j) complete in tensor memory (and every MMA issued before it)
    PB_PFULL = 11,                   // [2: tile a, b] P_x(j) written (4 arrivals)
    PB_OFINAL = 13,                  // [2: tile a, b] last P_x V retired
    PB_COUNT = 15
};

// two fp32 -> one word of two 16-bit elements (fp16 or bf16), round to nearest even
template <bool BF> __device__ __forceinline__ uint32_t pack2(float a, float b) {
    if (BF) {
        const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&r);
    }
    return f2_to_h2(a, b);
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool BF>
__global__ void __launch_bounds__(PT_THREADS, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                  const __grid_constant__ CUtensorMap vmap, PtArgs A) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *q_tile = smem;                                   // [2][32 KiB]: tiles a, b
    unsigned char *k_tile = q_tile + 2 * PT_TILE_BYTES;             // [2][32 KiB]
    unsigned char *v_tile = k_tile + PT_STAGES * PT_TILE_BYTES;     // [2][32 KiB]
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(v_tile + PT_STAGES * PT_TILE_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + PB_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // CTAs are dispatched in block-index order, x fastest: x runs over (sequence, head), y over the query pairs from the
    // last (longest KV range) to the first, so the long CTAs of every head start before any short one
    const int qp = gridDim.y - 1 - blockIdx.y;
    const int h = blockIdx.x % A.hq, b = blockIdx.x / A.hq, kvh = h / (A.hq / A.hkv);
    const int q0 = qp * 2 * PT_BQ;
    // KV tiles that query tile x (rows q0 + 128 x ..) needs: positions 0 .. min(pos_offset + its last row, kv_len - 1);
    // none when the tile lies beyond q_len
    auto tiles_of = [&](int x) {
        const int r0 = q0 + x * PT_BQ;
        if (r0 >= A.q_len) return 0;
        const int last_pos = min(A.pos_offset + min(r0 + PT_BQ, A.q_len) - 1, A.kv_len - 1);
        return last_pos / PT_BKV + 1;
    };
    const int nt_a = tiles_of(0), nt_b = tiles_of(1);
    const int ntiles = max(nt_a, nt_b);

    if (tid == 0) {
        mbar_init(smem_u32(&bars[PB_Q]), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bars[PB_KFULL + s]), 1);
            mbar_init(smem_u32(&bars[PB_KFREE + s]), 1);
            mbar_init(smem_u32(&bars[PB_VFULL + s]), 1);
            mbar_init(smem_u32(&bars[PB_VFREE + s]), 1);
            mbar_init(smem_u32(&bars[PB_SFULL + s]), 1);
            mbar_init(smem_u32(&bars[PB_PFULL + s]), 4);
            mbar_init(smem_u32(&bars[PB_OFINAL + s]), 1);
        }
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

    if (warp >= PT_SOFTMAX_WARPS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PT_REGS_AUX));
        if (warp == PT_SOFTMAX_WARPS) {
            // ---------------- TMA producer ----------------
            if (lane == 0) {
                tma_prefetch_desc(&qmap);
                tma_prefetch_desc(&kmap);
                tma_prefetch_desc(&vmap);
                const uint32_t qb = smem_u32(&bars[PB_Q]);
                mbar_expect_tx(qb, 2 * PT_TILE_BYTES);         // rows beyond q_len arrive as zeros and still count
                for (int x = 0; x < 2; ++x) {
                    tma_load_4d(smem_u32(q_tile + x * PT_TILE_BYTES), &qmap, 0, q0 + x * PT_BQ, h, b, qb);
                    tma_load_4d(smem_u32(q_tile + x * PT_TILE_BYTES + PT_HALF_BYTES), &qmap, 64, q0 + x * PT_BQ, h, b, qb);
                }
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
        } else if (warp == PT_SOFTMAX_WARPS + 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                const uint32_t fmt = BF ? (1u << 7) | (1u << 10) : 0u;           // A, B element format: f16 or bf16
                const uint32_t idesc_s = umma_idesc(PT_BQ, PT_BKV, 0) | fmt;     // A, B K-major
                const uint32_t idesc_o = umma_idesc_b_mn(PT_BQ, PT_D) | fmt;     // A from tensor memory, B (V) MN-major
                // S_x(j) = Q_x K(j)^T; the caller has seen K(j) land
                auto issue_s = [&](int x, int j) {
                    const uint64_t dq = umma_desc(smem_u32(q_tile + x * PT_TILE_BYTES), 16, 1024);
                    const uint64_t dk = umma_desc(smem_u32(k_tile + (j & 1) * PT_TILE_BYTES), 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < PT_D / 16; ++kk) {
                        // 16 dims per MMA: 32 bytes inside the 128-byte swizzle row; dims 64.. live in the second half tile
                        const uint64_t off = (uint64_t)(((kk >> 2) * PT_HALF_BYTES + (kk & 3) * 32) >> 4);
                        tc_mma_f16(tmem + PT_COL_S + x * 128, dq + off, dk + off, idesc_s, kk > 0 ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&bars[PB_SFULL + x]));
                };
                // O_x (+)= P_x(j) V(j); the caller has seen V(j) land
                auto issue_pv = [&](int x, int j) {
                    wait(PB_PFULL + x, (uint32_t)j & 1u);
                    tc_fence_after();
                    const uint64_t dv = umma_desc(smem_u32(v_tile + (j & 1) * PT_TILE_BYTES), PT_HALF_BYTES, 1024);   // MN-major: dim halves 16 KiB apart
#pragma unroll
                    for (int kk = 0; kk < PT_BKV / 16; ++kk)      // 16 kv positions per MMA: 8 columns of P, 16 rows (2 KiB) of V
                        tc_mma_f16_ts(tmem + PT_COL_O + x * 128, tmem + PT_COL_S + x * 128 + kk * 8, dv + (uint64_t)((kk * 2048) >> 4), idesc_o,
                                      (j > 0 || kk > 0) ? 1u : 0u);
                };
                wait(PB_Q, 0);
                wait(PB_KFULL, 0);
                tc_fence_after();
                if (nt_a > 0) issue_s(0, 0);
                if (nt_b > 0) issue_s(1, 0);
                tc_commit(smem_u32(&bars[PB_KFREE]));
                for (int j = 0; j < ntiles; ++j) {
                    const int s = j & 1, s1 = (j + 1) & 1;
                    const bool more = j + 1 < ntiles;
                    wait(PB_VFULL + s, (uint32_t)(j >> 1) & 1u);
                    if (more) wait(PB_KFULL + s1, (uint32_t)((j + 1) >> 1) & 1u);
                    tc_fence_after();
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const int nt_x = x ? nt_b : nt_a;
                        if (j < nt_x) {
                            issue_pv(x, j);
                            if (j + 1 < nt_x) issue_s(x, j + 1);
                            else tc_commit(smem_u32(&bars[PB_OFINAL + x]));
                        }
                    }
                    tc_commit(smem_u32(&bars[PB_VFREE + s]));
                    if (more) tc_commit(smem_u32(&bars[PB_KFREE + s1]));
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PT_REGS_SOFTMAX));
        // ---------------- softmax + output: thread = query row ----------------
        const int x = warp >> 2;                          // query tile of the pair
        const int nt_x = x ? nt_b : nt_a;
        const int row = (warp & 3) * 32 + lane;           // tensor-memory lane
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_base + PT_COL_S + x * 128, o_addr = lane_base + PT_COL_O + x * 128;
        const int r0 = q0 + x * PT_BQ, qi = r0 + row;
        const int limit = min(A.pos_offset + qi, A.kv_len - 1);      // last kv position this row sees
        float m = 0.f, l = 0.f;
        for (int j = 0; j < nt_x; ++j) {
            const int k0 = j * PT_BKV;
            const bool masked = k0 + PT_BKV - 1 > A.pos_offset + r0 || k0 + PT_BKV > A.kv_len;     // some row of the tile needs the mask
            wait(PB_SFULL + x, (uint32_t)j & 1u);
            tc_fence_after();
            float sc[PT_BKV];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sc[c * 32]));
            tmem_ld_wait();
            if (masked) {
#pragma unroll
                for (int i = 0; i < PT_BKV; ++i)
                    if (k0 + i > limit) sc[i] = -INFINITY;
            }
            float mx0 = sc[0], mx1 = sc[1], mx2 = sc[2], mx3 = sc[3];
#pragma unroll
            for (int i = 4; i < PT_BKV; i += 4) {
                mx0 = fmaxf(mx0, sc[i]);
                mx1 = fmaxf(mx1, sc[i + 1]);
                mx2 = fmaxf(mx2, sc[i + 2]);
                mx3 = fmaxf(mx3, sc[i + 3]);
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * A.scale_log2e;     // scaled, base-2 domain
            if (j == 0) {
                m = mx;                                    // tile 0 holds position 0, which every row sees: finite
            } else {
                const bool raise = mx - m > PT_RESCALE_THRESHOLD;
                if (__any_sync(0xffffffffu, raise)) {
                    // S_x(j) was issued behind P_x(j-1) V(j-1) and has completed, so O_x is at rest
                    const float alpha = raise ? ex2_approx(m - mx) : 1.f;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t r[32];
                        tmem_ld32(o_addr + c * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st32(o_addr + c * 32, r);
                    }
                    l *= alpha;
                    if (raise) m = mx;
                }
            }
            // P = 2^(s * scale * log2e - m), written over the row's own S columns as fp16 pairs
            float ps0 = 0.f, ps1 = 0.f, ps2 = 0.f, ps3 = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float p0 = ex2_approx(fmaf(sc[c * 32 + i], A.scale_log2e, -m));
                    const float p1 = ex2_approx(fmaf(sc[c * 32 + i + 1], A.scale_log2e, -m));
                    const float p2 = ex2_approx(fmaf(sc[c * 32 + i + 2], A.scale_log2e, -m));
                    const float p3 = ex2_approx(fmaf(sc[c * 32 + i + 3], A.scale_log2e, -m));
                    ps0 += p0;
                    ps1 += p1;
                    ps2 += p2;
                    ps3 += p3;
                    pk[i >> 1] = pack2<BF>(p0, p1);
                    pk[(i >> 1) + 1] = pack2<BF>(p2, p3);
                }
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                    ::"r"(s_addr + c * 16), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]),
                      "r"(pk[6]), "r"(pk[7]), "r"(pk[8]), "r"(pk[9]), "r"(pk[10]), "r"(pk[11]), "r"(pk[12]), "r"(pk[13]),
                      "r"(pk[14]), "r"(pk[15])
                    : "memory");
            }
            tmem_st_wait();
            tc_fence_before();
            l += (ps0 + ps1) + (ps2 + ps3);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[PB_PFULL + x]));          // P_x(j) (and a rescaled O_x) is in tensor memory
        }
        if (nt_x > 0) {
            wait(PB_OFINAL + x, 0);
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const bool live = qi < A.q_len;
            __half *dst = A.out + (((long)b * A.hq + h) * A.q_len + qi) * PT_D;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(o_addr + c * 32, r);
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 u;
                        u.x = pack2<BF>(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                        u.y = pack2<BF>(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        u.z = pack2<BF>(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                        u.w = pack2<BF>(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                        *reinterpret_cast<uint4 *>(dst + c * 32 + i) = u;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, PT_COLS);
}

// Returns TC-style "not covered" (-1000) when the shape is outside this kernel (the caller then runs the general one).
// bf16: the four tensors hold bfloat16 (passed as 16-bit words).
int prefill_tc_launch(const __half *q, const __half *k, const __half *v, __half *out, int batch, int hq, int hkv, int q_len,
                      int kv_len, int d, int pos_offset, float scale, bool bf16, cudaStream_t st) {
    constexpr int NOT_COVERED = -1000;
    if (d != PT_D || pos_offset < 0 || kv_len < 1 || q_len < 1 || hq % hkv || !(scale > 0.f)) return NOT_COVERED;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return NOT_COVERED;
    if (ceil_div(q_len, 2 * PT_BQ) > 65535 || (long)hq * batch > 0x7fffffffL) return NOT_COVERED;
    int *status = status_word();
    if (!status) return NOT_COVERED;
    const uint64_t row = PT_D * 2;
    CUtensorMap qmap, kmap, vmap;
    const CUtensorMapDataType dtype = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const uint32_t box[4] = {64, PT_BQ, 1, 1};
    {
        const uint64_t dims[4] = {PT_D, (uint64_t)q_len, (uint64_t)hq, (uint64_t)batch};
        const uint64_t str[3] = {row, (uint64_t)q_len * row, (uint64_t)hq * q_len * row};
        if (make_tensor_map(&qmap, dtype, 4, q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return NOT_COVERED;
    }
    {
        const uint64_t dims[4] = {PT_D, (uint64_t)kv_len, (uint64_t)hkv, (uint64_t)batch};
        const uint64_t str[3] = {row, (uint64_t)kv_len * row, (uint64_t)hkv * kv_len * row};
        if (make_tensor_map(&kmap, dtype, 4, k, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return NOT_COVERED;
        if (make_tensor_map(&vmap, dtype, 4, v, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return NOT_COVERED;
    }
    PtArgs A;
    A.out = out; A.hq = hq; A.hkv = hkv; A.q_len = q_len; A.kv_len = kv_len; A.pos_offset = pos_offset;
    A.scale_log2e = scale * 1.4426950408889634f;
    A.status = status;
    const size_t smem = (size_t)(2 + 2 * PT_STAGES) * PT_TILE_BYTES + PB_COUNT * 8 + 16 + 1024;
    auto kern = bf16 ? prefill_tc_kernel<true> : prefill_tc_kernel<false>;
    {
        static OncePerDevice once[2];
        cudaError_t e = once[bf16].run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
        if (e != cudaSuccess) return fail((int)e, "flash_attn_full: shared memory %zu: %s", smem, cudaGetErrorString(e));
    }
    const dim3 grid(hq * batch, ceil_div(q_len, 2 * PT_BQ), 1);
    kern<<<grid, PT_THREADS, smem, st>>>(qmap, kmap, vmap, A);
    return launch_status(bf16 ? "flash_attn_full_bf16" : "flash_attn_full_f16");
}

}  // namespace b200k

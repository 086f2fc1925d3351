// Tensor-core W4A16 GEMM for sm_100a: tcgen05.mma with the accumulator in TMEM.
//
// The product is computed transposed, C^T[n, m] = sum_k W^T[n, k] * A^T[k, m], so that
// the 128 rows of the MMA are 128 weight columns and the MMA's N extent is the token
// tile (16..256): a decode batch of 16-64 tokens then wastes nothing of the 128-row
// instruction, and the dequantised weight tile is the A operand.
//
// Per CTA: one 128-column slab of the weight, one token tile, one K split.  Roles:
//   warp 0      TMA producer of the packed int4 words of a pipeline step (64 or 128 k), with the step's
//               scale row and packed zero-points (ring of up to 16 steps: this is all the HBM traffic)
//   warp 3      TMA producer of the activation tiles (128-byte swizzle; from L2)
//   warps 4..   NG = 2 or 4 groups of 4 dequant warps, taking the steps round-robin: nibbles -> fp16 (or
//               bf16) in registers (magic-number trick, exact (q - zero), one multiply by the scale =
//               the reference's rounding).  GPTQ: a thread owns one weight column = one TMEM lane and
//               writes its 64 k of a sub-block with tcgen05.st into a ring of operand tiles in TENSOR
//               MEMORY (the MMA reads A from there).  AWQ: a word holds 8 adjacent columns of one k, so
//               the tile goes to shared memory in the UMMA MN-major 128-byte-swizzled layout.
//   warps 1, 2  MMA issuers: one thread issues 4 x tcgen05.mma (K = 16 each) per 64 k and commits to the
//               step's "operand consumed" barrier; at token tiles <= 64 two issuers with an accumulator
//               each take the steps alternately
//   warps 4..   epilogue: tcgen05.ld of the 128 x TT fp32 accumulator(s), fp16 store (optionally silu(gate) * up
//               of paired columns); with a K split the CTAs of a cluster exchange partial tiles through
//               distributed shared memory and each reduces a share of the rows in a fixed order
// Grouped mode (fused MoE): a row segment per expert with its own weight matrix, token tiles from a work list.
// Every wait on an mbarrier is bounded; a wait that gives up sets a status word and the
// kernel drains and frees its TMEM as usual.
#include <cooperative_groups.h>
#include <stdlib.h>

#include "gemm.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace cg = cooperative_groups;

namespace b200k {

constexpr int TC_BN = 128;        // weight columns per CTA = MMA M
constexpr int TC_BK = 64;         // K per stage = one 128-byte swizzle row of fp16
constexpr int TC_GROUP_WARPS = 4;  // dequant / epilogue warps come in groups of 4 (128 threads = 128 operand rows);
                                   // NG groups take K blocks round-robin: 2 groups (two CTAs per SM) for small token
                                   // tiles, 4 groups for large ones, where the tensor pipe would otherwise wait for operands
constexpr int TC_DQ_WARP0 = 4;    // warps 0..3: weight producer, MMA issuer, second MMA issuer (small token tiles), activation producer
constexpr int tc_threads(int ng) { return 32 * (TC_DQ_WARP0 + TC_GROUP_WARPS * ng); }
constexpr int TC_A_BYTES = TC_BN * TC_BK * 2;   // 16 KiB dequantised tile
constexpr int TC_W_BYTES = TC_BN * TC_BK / 2;   // 4 KiB packed weight words of one K block
constexpr int TC_SC_BYTES = TC_BN * 2;          // the block's scale row (one group) for the 128 columns
constexpr int TC_ZP_BYTES = TC_BN / 2;          // and its 16 packed zero-point words
// ring slot: a multiple of 128 bytes (TMA destinations are 128-byte aligned)
constexpr int TC_RAW_BYTES = TC_W_BYTES + TC_SC_BYTES + 128;

struct TcArgs {
    const __half *scales;
    const int32_t *qzeros;
    __half *c;
    int m, n, k, group;
    int s_sk, s_qzk, s_cm;
    int zero_offset;
    int tt;            // token tile = MMA N (16, 32, 64, 128, 256)
    int dq_log2;       // log2 of SD: ring of dequantised operand tiles (on-chip producer and consumer: shallow)
    int act_log2;      // log2 of SA: ring of activation tiles (TMA from L2: deep enough to cover its latency)
    int raw_log2;      // log2 of R: ring of packed-weight tiles; deepest, because 4 KiB per K block is all
                       //    the HBM traffic there is and enough of it must be in flight
    int ksplit;        // cluster size along K
    int kb_per_split;  // K blocks per split
    int *status;
    const int *seg_offsets;   // grouped mode: row segments of A / C, one weight matrix per segment (blockIdx.z)
    const int2 *tile_list;    // grouped mode: (segment, first row) per work item, or nullptr (blockIdx.z = segment, blockIdx.y = tile)
    const int *tile_count;
    int silu_inter;           // fused silu_mul epilogue: number of output columns (the weight holds twice as many), else 0
    int c_kperm;              // fused silu_mul epilogue: store every 8 consecutive output columns as (0,4,1,5,2,6,3,7)
    int w_rows_per_seg;       // rows of the packed weight tensor per segment (K/8 for GPTQ, K for AWQ)
    int g_rows_per_seg;       // rows of the scale / zero tensors per segment (K / group)
};

// The depths of the three rings are powers of two, so the slot of block i and the parity of the phase it
// belongs to are bit fields of i: nothing but i is carried from block to block (ring cursors kept in
// registers and advanced block by block cost a tenth of the dequant warps' instruction stream).
__device__ __forceinline__ int ring_slot(int i, int lg) { return i & ((1 << lg) - 1); }
__device__ __forceinline__ uint32_t ring_phase(int i, int lg) { return (uint32_t)(i >> lg) & 1u; }

// TS: the dequantised operand tile goes to tensor memory (tcgen05.st) instead of shared memory and the
// MMA reads it from there.  GPTQ only: a thread that owns weight column n holds, word by word, 8
// consecutive k of that column, which is exactly one TMEM lane (operand row) and 4 columns of it.
// It saves the 16 KiB shared-memory write and the 16 KiB read the tensor pipe would make per K block.
// NMMA = 2: two issuing warps, each with its own accumulator, take the K blocks alternately (block i goes
// to issuer i % 2, which is also dequant group i % 2 when there are two groups); the epilogue adds the two
// accumulators.  At token tiles of 16..64 one thread cannot issue 4 MMAs, wait and commit fast enough to
// keep up with the operand stream; at 128 and above the MMAs themselves take longer than their issue.
// KPERM: the activations arrive with every 8 consecutive k stored as (k0,k4,k1,k5,k2,k6,k3,k7), the order in which the
// nibble trick yields a word's values; the 4 byte-permutes per word that would restore k order then disappear (they
// run on the half-rate integer pipe, the busiest unit of this kernel).  A contraction may visit k in any order as
// long as both operands agree.
// SILU: the CTA's 128 operand rows are 64 gate columns [64 bx, 64 bx + 64) and the 64 up columns I + the same; the epilogue
// stores silu(gate) * up, 64 columns of an [M, I] output (the product the reference computes with a separate kernel,
// fused_silu_mul_interleaved, on the GEMM's fp16 output; here it is taken from the fp32 accumulators).
// BF: activations, scales and output are bfloat16 (the MMA's operand format follows).
// Wide steps (KK = 2; operand in tensor memory, token tiles up to 64): a pipeline step covers 128 k -- one
// TMA box of 16 packed rows, the step's scale row and zero words once, two swizzled activation boxes, two operand
// sub-tiles of 32 TMEM columns, eight MMAs and one commit.  Every role's hand-over (a barrier in, a barrier out, the
// issue of its copies or MMAs) is then paid once per 128 k; at token tiles <= 64 those hand-overs, not the arithmetic
// or the tensor pipe, are most of a 64-k block's time.
template <int FMT, int NG, bool TS, int NMMA, bool KPERM, bool SILU = false, bool BF = false, int KK = 1>
__global__ void __launch_bounds__(tc_threads(NG), NG == 2 ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap amap,
               const __grid_constant__ CUtensorMap smap, const __grid_constant__ CUtensorMap zmap, TcArgs P) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int LSD = P.dq_log2, LSA = P.act_log2, LR = P.raw_log2, TT = P.tt;
    const int SD = 1 << LSD, SA = 1 << LSA, R = 1 << LR;
    static_assert(KK == 1 || (KK == 2 && TS), "wide steps: operand in tensor memory");
    const int b_bytes = TT * TC_BK * 2 * KK;                    // KK swizzled boxes of [TT][128 B], one behind the other
    const int w_bytes = TC_W_BYTES * KK, raw_bytes = w_bytes + TC_SC_BYTES + 128;
    unsigned char *a_tile = smem;                               // [SD][16 KiB] (absent when the operand tile lives in TMEM)
    unsigned char *b_tile = a_tile + (TS ? 0 : (size_t)SD * TC_A_BYTES);   // [SA][KK][TT * 128]
    unsigned char *raw = b_tile + (size_t)SA * b_bytes;         // [R][4 or 8 KiB + scales + zero words]
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(raw + (size_t)R * raw_bytes);
    // barrier map
    const int B_ACTF = 0;               // [SA] activation tile landed (TMA)
    const int B_ACTE = SA;              // [SA] activation tile consumed (released by the dequant group that sees its MMAs retired)
    const int B_DQF = 2 * SA;           // [SD] operand tile written (one arrival per dequant warp)
    const int B_DQE = 2 * SA + SD;      // [SD] operand tile consumed (tcgen05.commit)
    const int B_RAWF = 2 * SA + 2 * SD;       // [R] packed words landed (TMA)
    const int B_RAWE = 2 * SA + 2 * SD + R;   // [R] packed words read (one arrival per dequant warp)
    const int B_ACC = 2 * SA + 2 * SD + 2 * R;  // accumulator complete
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + B_ACC + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = SILU ? blockIdx.x * (TC_BN / 2) : blockIdx.x * TC_BN;     // SILU: first gate column; up columns at silu_inter + n0
    int m0 = blockIdx.y * TT, m_end = P.m, w_row0 = 0, g_row0 = 0;
    if (P.seg_offsets) {
        pdl_wait();   // the segment offsets (and the work list) are written by the kernel before
        // grouped mode: this CTA works on one token tile of one segment with that segment's weights; no K split
        int e;
        if (P.tile_list) {
            const int item = blockIdx.y;
            if (item >= *P.tile_count) return;      // uniform across the CTA, before any barrier or TMEM allocation
            const int2 w = P.tile_list[item];
            e = w.x;
            m0 = w.y;
        } else {
            e = blockIdx.z;
            m0 += P.seg_offsets[e];
        }
        m_end = P.seg_offsets[e + 1];
        if (m0 >= m_end) return;
        w_row0 = e * P.w_rows_per_seg;
        g_row0 = e * P.g_rows_per_seg;
    }
    const int kb_total = P.k / (TC_BK * KK);        // pipeline steps ("K blocks" below) over the whole K
    // K split: blockIdx.z, except in grouped mode without a work list, where blockIdx.z is the segment
    const int kb_begin = P.seg_offsets && !P.tile_list ? 0 : blockIdx.z * P.kb_per_split;
    const int kb_end = min(kb_total, kb_begin + P.kb_per_split);
    const int nkb = max(0, kb_end - kb_begin);
    // TMEM columns: NMMA fp32 accumulators [128 lanes][TT]; with TS, SD operand tiles of 32 columns behind them
    const uint32_t a_col0 = NMMA * TT < 32 ? 32 : NMMA * TT;
    uint32_t tmem_cols = 32;
    while (tmem_cols < (TS ? a_col0 + 32u * KK * SD : (uint32_t)(NMMA * TT))) tmem_cols <<= 1;

    // one barrier per thread (up to ~60 of them: initialised one after the other by a single thread they cost a microsecond)
    if (tid <= B_ACC) {
        const int count = (tid >= B_DQF && tid < B_DQE) || (tid >= B_RAWE && tid < B_ACC) ? TC_GROUP_WARPS : tid == B_ACC ? NMMA : 1;
        mbar_init(smem_u32(&bars[tid]), count);
    }
    if (tid == 0) *abort_flag = 0;
    if (tid <= B_ACC) mbar_init_fence();
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot;
    // Barriers, tensor memory and descriptors are set up.  The packed weights, scales and zero-points do not depend on
    // the kernel before this one, so their stream and the dequantisation start at once; only the activation producer
    // waits for the predecessor, and every global write of this kernel comes after the MMAs that consume its tiles
    // (the epilogue waits once more, formally, before it stores).
    pdl_launch_dependents();

    auto wait = [&](int bar_idx, uint32_t parity) {
        const uint32_t bar = smem_u32(&bars[bar_idx]);
        if (mbar_try_wait(bar, parity)) return;      // the common case costs one instruction
        if (*abort_flag) return;                     // some wait already gave up: drain without waiting again
        if (!mbar_wait_bounded(bar, parity)) {
            *abort_flag = 1;
            atomicExch(P.status, 2);
        }
    };

    // For a barrier already tested once (result `ok`): nothing to do when that test succeeded.
    auto wait_after_test = [&](bool ok, int bar_idx, uint32_t parity) {
        if (!ok) wait(bar_idx, parity);
    };

    if (warp == 0) {
        // ---------------- TMA producer, packed weights: R blocks ahead ----------------
        if (lane == 0) {
            const int group_shift = 31 - __clz(P.group);   // group sizes on this path are powers of two
            tma_prefetch_desc(&wmap);
            tma_prefetch_desc(&smap);
            if (P.qzeros) tma_prefetch_desc(&zmap);
            for (int i = 0; i < nkb; ++i) {
                const int r = ring_slot(i, LR), kb = kb_begin + i;
                if (i >= R) wait(B_RAWE + r, ring_phase(i, LR) ^ 1u);
                const uint32_t bar = smem_u32(&bars[B_RAWF + r]);
                const uint32_t dst = smem_u32(raw + (size_t)r * raw_bytes);
                mbar_expect_tx(bar, w_bytes + TC_SC_BYTES + (P.qzeros ? TC_ZP_BYTES : 0));
                const int grp = (kb * TC_BK * KK) >> group_shift;
                if (SILU) {
                    // the tensors are described as [rows][2][I]: one box of 64 columns x {gate, up} per tensor lands as
                    // [8 rows][gate 64 | up 64] words, 64 + 64 scales, 8 + 8 zero-point words -- the layout of an
                    // ordinary 128-column tile, at half the copies two boxes per tensor would take
                    tma_load_3d(dst, &wmap, n0, 0, w_row0 + kb * (TC_BK / 8) * KK, bar);
                    tma_load_3d(dst + w_bytes, &smap, n0, 0, g_row0 + grp, bar);
                    if (P.qzeros) tma_load_3d(dst + w_bytes + TC_SC_BYTES, &zmap, n0 / 8, 0, g_row0 + grp, bar);
                } else {
                    if (FMT == FMT_GPTQ)
                        tma_load_2d(dst, &wmap, n0, w_row0 + kb * (TC_BK / 8) * KK, bar);      // the map's box holds 8 KK rows
                    else
                        tma_load_2d(dst, &wmap, n0 / 8, w_row0 + kb * TC_BK, bar);
                    // the block's quantisation group rides along: scale row and packed zero-points
                    tma_load_2d(dst + w_bytes, &smap, n0, g_row0 + grp, bar);
                    if (P.qzeros) tma_load_2d(dst + w_bytes + TC_SC_BYTES, &zmap, n0 / 8, g_row0 + grp, bar);
                }
            }
        }
    } else if (warp == 3) {
        // ---------------- TMA producer, activation tiles: SA blocks ahead ----------------
        if (lane == 0) {
            tma_prefetch_desc(&amap);
            pdl_wait();   // the activations come from the kernel before
            for (int i = 0; i < nkb; ++i) {
                const int s = ring_slot(i, LSA);
                if (i >= SA) wait(B_ACTE + s, ring_phase(i, LSA) ^ 1u);
                const uint32_t bar = smem_u32(&bars[B_ACTF + s]);
                mbar_expect_tx(bar, b_bytes);
                for (int h = 0; h < KK; ++h)
                    tma_load_2d(smem_u32(b_tile + (size_t)s * b_bytes + (size_t)h * TT * 128), &amap, ((kb_begin + i) * KK + h) * TC_BK, m0, bar);
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ---------------- MMA issuers ----------------
        // One thread per issuing warp; its per-block work is the critical path at small token tiles, so it
        // waits on one barrier (an operand tile is published only after its activation tile has landed) and
        // commits to one barrier per block.
        const int mw = warp - 1;
        if (lane == 0 && mw < NMMA) {
            // MMA N = the rows this tile really holds, rounded up to 16: a segment of 130 rows in a 256-row tile, or the
            // last tile of an ordinary GEMM, costs the tensor pipe what it uses (accumulator columns beyond stay unwritten
            // and are never stored)
            const int tt_mma = min(TT, ((min(m_end, m0 + TT) - m0 + 15) >> 4) << 4);
            const uint32_t idesc = umma_idesc(TC_BN, tt_mma, FMT == FMT_AWQ ? 1 : 0) | (BF ? (1u << 7) | (1u << 10) : 0u);   // A, B format: f16 or bf16
            const uint64_t da0 = FMT == FMT_GPTQ ? umma_desc(smem_u32(a_tile), 16, 1024)       // K-major: 8-row groups 1 KiB apart
                                                 : umma_desc(smem_u32(a_tile), 8192, 1024);    // MN-major: 64-column halves 8 KiB apart, 8-k groups 1 KiB apart
            const uint64_t db0 = umma_desc(smem_u32(b_tile), 16, 1024);
            const uint32_t a_step = (FMT == FMT_GPTQ ? 32 : 2048) >> 4;     // descriptor address units of 16 bytes
            const uint32_t acc = tmem_acc + mw * TT;
            for (int i = mw; i < nkb; i += NMMA) {
                const int sd = ring_slot(i, LSD), sa = ring_slot(i, LSA);
                wait(B_DQF + sd, ring_phase(i, LSD));
                tc_fence_after();
                const uint64_t da = da0 + (uint64_t)((sd * TC_A_BYTES) >> 4);
                const uint64_t db = db0 + (uint64_t)((sa * b_bytes) >> 4);
                for (int h = 0; h < KK; ++h) {
#pragma unroll
                    for (int j = 0; j < TC_BK / 16; ++j) {
                        const uint32_t accumulate = (i >= NMMA || h > 0 || j > 0) ? 1u : 0u;
                        if (TS)
                            tc_mma_f16_ts(acc, tmem_acc + a_col0 + (sd * KK + h) * 32 + j * 8,
                                          db + (uint64_t)((h * TT * 128) >> 4) + (uint64_t)(j * 2), idesc, accumulate);
                        else
                            tc_mma_f16(acc, da + (uint64_t)(j * a_step), db + (uint64_t)(j * 2), idesc, accumulate);
                    }
                }
                tc_commit(smem_u32(&bars[B_DQE + sd]));   // operand tile (and, through it, the activation tile) reusable once these retire
            }
            tc_commit(smem_u32(&bars[B_ACC]));            // this issuer's accumulator complete (immediately, if it had no block)
        }
    } else {
        // ---------------- dequant warps: NG groups of 128 threads, group g takes K blocks g, g+NG, ... ----------------
        // (the waits, fences and arrivals of one block then overlap the arithmetic of the other group's block)
        const int tg = tid - 32 * TC_DQ_WARP0;
        // t = operand row; the hardware warp's TMEM lane quadrant is warp % 4, and a group is 4 consecutive warps
        const int grp_id = tg >> 7, t = ((warp & 3) << 5) | lane, warp_in_group = (tg & 127) >> 5;
        for (int i = grp_id; i < nkb; i += NG) {
            const int s = ring_slot(i, LSD), r = ring_slot(i, LR);
            // The three barriers of this block are tested back to back: a test costs well over a hundred cycles even
            // when the phase is long complete, and the tests are independent, so their latencies overlap.
            // (test_wait: a test that does not park the thread when the phase is still open)
            const bool ok_raw = mbar_test_wait(smem_u32(&bars[B_RAWF + r]), ring_phase(i, LR));
            const bool ok_dqe = i < SD || mbar_test_wait(smem_u32(&bars[B_DQE + s]), ring_phase(i, LSD) ^ 1u);
            const bool ok_act = mbar_test_wait(smem_u32(&bars[B_ACTF + ring_slot(i, LSA)]), ring_phase(i, LSA));
            wait_after_test(ok_raw, B_RAWF + r, ring_phase(i, LR));                               // packed words, scales, zero-points landed
            const unsigned char *slot = raw + (size_t)r * raw_bytes;
            const uint32_t *rw = reinterpret_cast<const uint32_t *>(slot);
            uint32_t w[8 * KK];
            if (FMT == FMT_GPTQ) {
                // thread t = weight column t (operand row t): its 8 words per 64 k are the 8 16-byte chunks of the row
                const uint32_t s2 = (uint32_t)reinterpret_cast<const uint16_t *>(slot + w_bytes)[t] * 0x10001u;   // the column's scale in both halves
                int z = 8;
                if (P.qzeros) {
                    z = (int)((reinterpret_cast<const uint32_t *>(slot + w_bytes + TC_SC_BYTES)[t >> 3] >> (4 * (t & 7))) & 15u) +
                        P.zero_offset;
                }
                uint32_t zm[4];
                zero_magic4<BF>(z, zm);
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j] = rw[j * TC_BN + t];     // (fused silu: rows 0..63 gate columns, 64..127 up columns)
                if (KK == 2) {
#pragma unroll
                    for (int j = 8; j < 8 * KK; ++j) w[j] = rw[j * TC_BN + t];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars[B_RAWE + r]));  // this warp is done with the packed tile
                if (i >= SD) {
                    wait_after_test(ok_dqe, B_DQE + s, ring_phase(i, LSD) ^ 1u);   // block i - SD retired: its operand tile is free, and so is its activation tile
                    if (TS) tc_fence_after();         // the tensor-memory store below is ordered after the MMAs that read the tile
                    if (warp_in_group == 0 && lane == 0) mbar_arrive(smem_u32(&bars[B_ACTE + ring_slot(i - SD, LSA)]));
                }
                unsigned char *arow = a_tile + (size_t)s * TC_A_BYTES + t * 128;
#pragma unroll
                for (int h = 0; h < KK; ++h) {
                    uint32_t v[32];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint32_t x[4];
                        nib4<BF>(w[h * 8 + j], x);
                        const uint32_t v04 = sub_mul<BF>(x[0], zm[0], s2), v15 = sub_mul<BF>(x[1], zm[1], s2);
                        const uint32_t v26 = sub_mul<BF>(x[2], zm[2], s2), v37 = sub_mul<BF>(x[3], zm[3], s2);
                        uint4 o;
                        if (KPERM) {
                            o = make_uint4(v04, v15, v26, v37);    // (k0 k4) (k1 k5) (k2 k6) (k3 k7): the activations' order
                        } else {
                            o.x = __byte_perm(v04, v15, 0x5410);   // k0 k1
                            o.y = __byte_perm(v26, v37, 0x5410);   // k2 k3
                            o.z = __byte_perm(v04, v15, 0x7632);   // k4 k5
                            o.w = __byte_perm(v26, v37, 0x7632);   // k6 k7
                        }
                        if (TS) {
                            v[4 * j] = o.x; v[4 * j + 1] = o.y; v[4 * j + 2] = o.z; v[4 * j + 3] = o.w;
                        } else {
                            *reinterpret_cast<uint4 *>(arow + ((j ^ (t & 7)) << 4)) = o;
                        }
                    }
                    // lane t of tensor memory = operand row t; columns = this sub-block's 64 k, two per column
                    if (TS) tmem_st32(tmem_acc + ((uint32_t)(t & 96) << 16) + a_col0 + (s * KK + h) * 32, v);
                }
                if (TS) {
                    tmem_st_wait();
                    tc_fence_before();
                }
            } else {
                // thread t: word column n8 = t % 16 (8 weight columns), k rows t / 16 + 8 j
                const int n8 = t & 15, kr = t >> 4;
                const uint4 su = reinterpret_cast<const uint4 *>(slot + TC_W_BYTES)[n8];
                const uint32_t zw = reinterpret_cast<const uint32_t *>(slot + TC_W_BYTES + TC_SC_BYTES)[n8];
                uint32_t zq[4];
                nib4<BF>(zw, zq);      // the zero word has the weights' nibble order: its pairs in biased form are the subtrahends
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j] = rw[(kr + 8 * j) * 16 + n8];
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars[B_RAWE + r]));
                if (i >= SD) {
                    wait_after_test(ok_dqe, B_DQE + s, ring_phase(i, LSD) ^ 1u);   // block i - SD retired: its operand tile is free, and so is its activation tile
                    if (warp_in_group == 0 && lane == 0) mbar_arrive(smem_u32(&bars[B_ACTE + ring_slot(i - SD, LSA)]));
                }
                unsigned char *ahalf = a_tile + (size_t)s * TC_A_BYTES + (n8 >> 3) * 8192;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int kk = kr + 8 * j;
                    uint32_t x[4];
                    nib4<BF>(w[j], x);
                    uint4 o;
                    o.x = sub_mul<BF>(x[0], zq[0], su.x);   // columns 0,1 (nibbles 0,4)
                    o.y = sub_mul<BF>(x[1], zq[1], su.y);   // columns 2,3 (nibbles 1,5)
                    o.z = sub_mul<BF>(x[2], zq[2], su.z);   // columns 4,5 (nibbles 2,6)
                    o.w = sub_mul<BF>(x[3], zq[3], su.w);   // columns 6,7 (nibbles 3,7)
                    *reinterpret_cast<uint4 *>(ahalf + kk * 128 + (((n8 & 7) ^ (kk & 7)) << 4)) = o;
                }
            }
            if (!TS) fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                wait_after_test(ok_act, B_ACTF + ring_slot(i, LSA), ring_phase(i, LSA));     // the MMA issuer waits on B_DQF alone
                mbar_arrive(smem_u32(&bars[B_DQF + s]));
            }
        }
        // ---------------- epilogue: TMEM -> registers -> C (or the split-K exchange) ----------------
        if (nkb > 0) {
            wait(B_ACC, 0);
            tc_fence_after();
        }
        pdl_wait();   // nothing of this kernel is stored before the predecessor has completed
        const int q = warp & 3;                       // TMEM lane quadrant this warp may read
        const int chunk0 = (warp - TC_DQ_WARP0) >> 2; // the NG warps of a quadrant take 16-column chunks round-robin
        const int row = q * 32 + lane;                // accumulator row = weight column n0 + row
        const int n = n0 + row;
        float *red = reinterpret_cast<float *>(smem);     // [TT][128] fp32, reuses the rings (all copies landed, all MMAs retired)
        if (SILU) {
            // rows 0..63 hold gate columns, rows 64..127 the matching up columns: the up half goes through shared memory
            // to the warps that hold the gate half, which store silu(gate) * up
            for (int base = 0; base < TT; base += 16 * NG) {      // every warp makes the same number of rounds (named barrier inside)
                const int c0 = base + chunk0 * 16;
                const bool active = c0 < TT;
                uint32_t rr[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) rr[j] = 0u;
                if (active && nkb > 0) {
                    tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + c0, rr);
                    if (NMMA == 2 && nkb > 1) {
                        uint32_t r2[16];
                        tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + TT + c0, r2);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) rr[j] = __float_as_uint(__uint_as_float(rr[j]) + __uint_as_float(r2[j]));
                    }
                    tmem_ld_wait();
                }
                if (active && q >= 2) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) red[(c0 + j) * (TC_BN / 2) + row - TC_BN / 2] = __uint_as_float(rr[j]);
                }
                asm volatile("bar.sync 1, %0;" ::"r"(NG * 128) : "memory");      // the dequant / epilogue warps only
                if (active && q < 2 && n < P.silu_inter) {
                    // the consumer of a pre-permuted activation tensor reads column k of an 8-block at slot 2 (k & 3) + (k >> 2)
                    const int n_st = P.c_kperm ? (n & ~7) | ((n & 3) << 1) | ((n >> 2) & 1) : n;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c0 + j;
                        const float gt = __uint_as_float(rr[j]), up = red[(c0 + j) * (TC_BN / 2) + row];
                        if (m < m_end) store_elem<BF>(P.c + (long)m * P.s_cm + n_st, gt / (1.f + expf(-gt)) * up);
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"r"(NG * 128) : "memory");      // before the next round overwrites the staging rows
            }
        } else
        for (int c0 = chunk0 * 16; c0 < TT; c0 += 16 * NG) {
            uint32_t rr[16];
            if (nkb > 0) {
                tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + c0, rr);
                if (NMMA == 2 && nkb > 1) {
                    uint32_t r2[16];
                    tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + TT + c0, r2);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) rr[j] = __float_as_uint(__uint_as_float(rr[j]) + __uint_as_float(r2[j]));
                }
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) rr[j] = 0u;
            }
            if (P.ksplit == 1) {
                if (n < P.n) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c0 + j;
                        if (m < m_end) store_elem<BF>(P.c + (long)m * P.s_cm + n, __uint_as_float(rr[j]));
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) red[(c0 + j) * TC_BN + row] = __uint_as_float(rr[j]);
            }
        }
    }

    if (P.ksplit > 1) {
        // every CTA of the cluster holds a partial [TT][128] tile; CTA r reduces rows r, r+ksplit, ...
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (warp >= TC_DQ_WARP0) {
            const int t = tid - 32 * TC_DQ_WARP0, row = t & (TC_BN - 1), sub = t >> 7;
            const int n = n0 + row;
            float *red = reinterpret_cast<float *>(smem);
            const int rank = (int)cluster.block_rank();
            for (int mm = rank + sub * P.ksplit; mm < TT; mm += NG * P.ksplit) {
                const int m = m0 + mm;
                if (m >= m_end) break;
                float acc = 0.f;
                for (int r = 0; r < P.ksplit; ++r) acc += cluster.map_shared_rank(red, r)[mm * TC_BN + row];
                if (n < P.n) store_elem<BF>(P.c + (long)m * P.s_cm + n, acc);
            }
        }
        cluster.sync();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_acc, tmem_cols);
}

int gemm_tc_token_tile(int m, int segments);
static int pick_tt(int m) {
    if (const int v = env_int("B200K_TC_TT", 0)) return v;      // tuning override
    if (m <= 16) return 16;
    if (m <= 32) return 32;
    if (m <= 64) return 64;
    if (m <= 128) return 128;
    return 256;
}

// Grouped mode: segments are unequal (router counts scatter around the mean), and every token tile of a segment
// dequantises the segment's weights again, whatever its width.  The tile therefore leaves head-room above the mean -- a
// quarter of it, or three standard deviations of a count that scatters like a Poisson variable, whichever is more -- so that a
// segment above the mean still fits one tile.  Up to 192 rows the tile is a multiple of 16 and two CTAs share an SM
// (tensor memory: 256 columns each); above, one CTA per SM with 256-row tiles.
int gemm_tc_token_tile(int m, int segments) {
    if (const int v = env_int("B200K_TC_GTT", 0)) return v;      // tuning override
    const int mean = ceil_div(m, segments < 1 ? 1 : segments);
    const int spread = (int)(3.f * sqrtf((float)mean)) + 1;
    const int want = mean + (mean / 4 > spread ? mean / 4 : spread);
    if (want <= 64) return pick_tt(want);
    return want <= 192 ? (want + 15) / 16 * 16 : 256;
}

int gemm_tc_launch(const GemmArgs &g) {
    const bool silu = g.silu_inter > 0;
    if (silu && (g.format != FMT_GPTQ || g.n != 2 * g.silu_inter || g.silu_inter % 64)) return TC_NOT_COVERED;
    if (g.k % TC_BK || g.group % TC_BK || (g.group & (g.group - 1)) || g.n % 8) return TC_NOT_COVERED;
    if (g.format == FMT_AWQ && !g.qzeros) return TC_NOT_COVERED;
    if (g.qzeros && (g.s_qzk % 4 || !aligned16(g.qzeros))) return TC_NOT_COVERED;   // zero-point rows travel by TMA: 16-byte pitch
    const bool grouped = g.seg_offsets != nullptr;
    // grouped: the token tile follows the average segment (plus head-room); the grid covers the worst case (every row
    // in one segment) and CTAs past their segment's end return at once
    const int m_plan = grouped && g.expected_m > 0 ? g.expected_m : g.m;      // rows the launch is planned for
    int tt = grouped ? gemm_tc_token_tile(m_plan, g.num_segments) : pick_tt(g.m);
    const int kb_total = g.k / TC_BK;
    // Above 64 tokens an ordinary GEMM has two forms: a 256-token tile on one CTA of four dequant groups per SM, or a
    // 128-token tile on two CTAs of two groups per SM (the same four groups, grid units half as large).  Form and K split
    // are chosen together by a cost model fitted to measurements: a CTA costs ~4 us of set-up and drain plus its K blocks
    // (0.48 us each at 256 tokens, where the activation tiles' way from L2 sets the pace; 0.62 us when two 128-token CTAs
    // share an SM, 0.45 us when one has it alone), CTAs beyond the resident ones wait for a whole wave, and a K split costs
    // ~5 us plus the exchange of the partial tiles.
    bool pair128 = grouped && tt > 64 && tt <= 192 && env_int("B200K_TC_GPAIR", 1) != 0;     // (ordinary GEMMs: decided below)
    int planned_split = 0;
    if (!grouped && !silu && g.m > 64 && !env_int("B200K_TC_TT", 0)) {
        const int sms = sm_count(), cols = ceil_div(g.n, TC_BN);
        const bool pair_ok = env_int("B200K_TC_PAIR128", 1) != 0;
        const bool wide = g.format == FMT_GPTQ && g.k % (2 * TC_BK) == 0 && g.group % (2 * TC_BK) == 0 && env_char("B200K_TC_OPERAND") != 's';
        float best = 1e30f;
        for (int form = 0; form < 2; ++form) {      // 0: paired 128-token tiles, 1: 256-token tiles (128 with four groups up to 128 tokens)
            if (form == 0 && !pair_ok) continue;
            if (form == 1 && pair_ok && g.m <= 128) continue;
            const int t = form == 0 || g.m <= 128 ? 128 : 256;
            const int toks = ceil_div(g.m, t), slots = form == 0 ? 2 * sms : sms;
            for (int ks = 1; ks <= 8; ks *= 2) {
                if (ks > 1 && (kb_total <= 8 || kb_total / ks < 4)) break;
                if (ks > 1 && cols * toks * (ks / 2) >= slots) break;     // a grid that fills the machine is not split further
                const int ctas = cols * toks * ks, waves = ceil_div(ctas, slots);
                // (the paired form with 128-k steps, GPTQ layouts: 0.49 us per 64 k measured where 64-k steps take 0.62)
                const float per_block = form == 0 ? (ctas > sms ? 0.62f : 0.45f) * (wide ? 0.78f : 1.f) : (t == 256 ? 0.48f : 0.22f);
                const float us = waves * (4.f + ceil_div(kb_total, ks) * per_block) + (ks > 1 ? 5.f + t / 64.f : 0.f);
                if (us < best) {
                    best = us;
                    tt = t;
                    pair128 = form == 0;
                    planned_split = ks;
                }
            }
        }
    }
    const int col_tiles = silu ? g.silu_inter / 64 : ceil_div(g.n, TC_BN), tok_tiles = ceil_div(g.m, tt);
    const int tiles = col_tiles * tok_tiles;
    // Shared memory: two CTAs per SM while the token tile is small (or in the paired form), one otherwise.
    const int ctas_per_sm = tt <= 64 || pair128 ? 2 : 1;
    const int budget = (ctas_per_sm == 2 ? 111 : 222) * 1024;
    const int ng = ctas_per_sm == 2 ? 2 : 4;         // dequant groups
    // operand tile in tensor memory (GPTQ) or in shared memory (AWQ; B200K_TC_OPERAND=smem forces it)
    bool ts = g.format == FMT_GPTQ;
    if (env_char("B200K_TC_OPERAND") == 's') ts = false;
    // pipeline steps of 128 k (two 64-k sub-blocks) at token tiles up to 64 of an ordinary GEMM with the operand in tensor memory
    const int kk = ts && !(g.bf16 && (silu || grouped)) && (tt <= 64 || (pair128 && tt <= 128 && env_int("B200K_TC_KK128", 1))) && g.k % (2 * TC_BK) == 0 && g.group % (2 * TC_BK) == 0 &&
                           env_int("B200K_TC_KK", 2) == 2 ? 2 : 1;
    const int act_bytes = tt * TC_BK * 2 * kk;
    const int raw_bytes = TC_W_BYTES * kk + TC_SC_BYTES + 128;
    const int a_bytes = ts ? 0 : TC_A_BYTES;
    // Ring depths, powers of two (slot and phase of a block are then bit fields of its index).  The operand ring
    // is shallow (producer and consumer are on chip) and at least as deep as there are dequant groups; an
    // activation slot is handed back when the operand tile SD blocks later is recycled, so the activation ring
    // is at least as deep as the operand ring (the last SD blocks never hand theirs back) and an activation
    // tile is requested SA - SD blocks ahead; the ring of packed words takes what is left, 16 at most.
    const int nmma = tt <= 64 ? 2 : 1;           // issuing warps (each with its own accumulator)
    const bool g2m1 = ng == 2 && nmma == 1;      // the paired 128-token form
    auto pow2_floor = [](int v) { int p = 1; while (p * 2 <= v) p *= 2; return p; };
    auto log2i = [](int v) { int l = 0; while ((1 << l) < v) ++l; return l; };
    int dq_stages, act_stages;
    if (ts) {   // operand tiles cost 32 TMEM columns each: 256 columns per CTA with two CTAs per SM, 512 with one
        dq_stages = (pair128 && tt > 128) || kk == 2 ? 2 : 4;      // two CTAs per SM: accumulators + 32 kk x depth <= 256 columns
        act_stages = kk == 2 ? (tt > 64 ? 2 : 4) : tt <= 128 && !pair128 ? 8 : 4;
    } else {
        dq_stages = tt <= 64 || pair128 ? 2 : 4;
        act_stages = tt <= 32 ? 8 : pair128 && tt > 128 ? 2 : 4;
    }
    if (const int v = env_int("B200K_TC_DQ_STAGES", 0)) dq_stages = pow2_floor(v < 1 ? 1 : v);     // tuning overrides
    if (const int v = env_int("B200K_TC_ACT_STAGES", 0)) act_stages = pow2_floor(v < 1 ? 1 : v);
    if (dq_stages < ng) dq_stages = ng;
    if (ts && (nmma * tt < 32 ? 32 : nmma * tt) + 32 * kk * dq_stages > (ctas_per_sm == 2 ? 256 : 512)) return TC_NOT_COVERED;
    if (act_stages < dq_stages) act_stages = dq_stages;
    int raw_stages = (budget - dq_stages * a_bytes - act_stages * act_bytes - 1024) / raw_bytes;
    if (raw_stages < 2) return TC_NOT_COVERED;
    raw_stages = pow2_floor(raw_stages > 16 / kk ? 16 / kk : raw_stages);
    {
        const int v = env_int("B200K_TC_RAW_STAGES", 0);
        if (v >= 2 && v <= raw_stages) raw_stages = pow2_floor(v);
    }
    // K split (cluster of 1, 2, 4 or 8 CTAs along K).  A CTA costs ~6 us of fill, drain and exchange
    // whatever its length, so: the fewest CTAs that still occupy most SMs; one more doubling only when
    // the machine is at most once covered and every CTA keeps a long K range.
    // The exchange tile ([tt][128] fp32) reuses the three rings, idle by then.
    const size_t ring_bytes = (size_t)dq_stages * a_bytes + (size_t)act_stages * act_bytes + (size_t)raw_stages * raw_bytes;
    const bool listed = grouped && g.tile_list;
    const bool can_split = (!grouped || listed) && !silu && ring_bytes >= (size_t)tt * TC_BN * 4;
    if (silu && ring_bytes < (size_t)tt * TC_BN * 2) return TC_NOT_COVERED;      // the epilogue stages the up half in the rings' space
    int ksplit = 1;
    // (a cluster launch with its two cluster barriers and the exchange costs ~5 us, a K block ~0.33 us per CTA: measured at 64
    // tokens, 8 blocks in one CTA take 5.7 us, split over a pair of CTAs 9.8 us.  Up to 8 blocks there is nothing to split.)
    if (planned_split) {
        ksplit = can_split ? planned_split : 1;
    } else if (grouped) {
        // a work list of few tiles with a long K (the second expert GEMM with one or two experts per GPU): split while the
        // expected tiles leave resident slots empty and every CTA keeps at least 8 K blocks
        const int expected = col_tiles * (ceil_div(m_plan, tt) > g.num_segments ? ceil_div(m_plan, tt) : g.num_segments);
        const int slots = sm_count() * ctas_per_sm;
        while (can_split && ksplit < 8 && expected * ksplit * 2 <= slots && kb_total / (ksplit * 2) >= 8) ksplit *= 2;
    } else if (can_split && kb_total > 8) {
        const int sms = sm_count();
        while (ksplit < 8 && tiles * ksplit < (sms * 7) / 8 && kb_total / (ksplit * 2) >= 4) ksplit *= 2;
        if (ksplit < 8 && ksplit > 1 && tiles * ksplit <= sms && kb_total / (ksplit * 2) >= 24) ksplit *= 2;
    }
    {   // tuning override
        const int v = env_int("B200K_TC_KSPLIT", 0);
        if (v >= 1 && v <= 8 && (v == 1 || can_split)) ksplit = v;
    }
    if (g.plan_out) {
        int *o = g.plan_out;
        o[0] = tt; o[1] = ng; o[2] = dq_stages; o[3] = act_stages; o[4] = raw_stages; o[5] = ksplit;
        o[6] = ceil_div(kb_total / kk, ksplit); o[7] = tok_tiles * col_tiles; o[8] = nmma; o[9] = ts ? 1 : 0;
        return 0;
    }
    const size_t smem = (size_t)dq_stages * a_bytes + (size_t)act_stages * act_bytes +
                        (size_t)raw_stages * raw_bytes + (2 * act_stages + 2 * dq_stages + 2 * raw_stages + 1) * 8 +
                        16 + 1024;

    // tensor maps: packed weight words (no swizzle) and activations (128-byte swizzle)
    CUtensorMap wmap, amap, smap, zmap;
    int rc;
    const uint64_t nseg = grouped ? (uint64_t)g.num_segments : 1;
    if (silu) {
        // [rows][2][I] views of the packed words, scales and zero-points: a box takes 64 gate columns and the 64 up columns
        // I further on in one copy
        const uint64_t inter = (uint64_t)g.silu_inter;
        const uint64_t dims[3] = {inter, 2, (uint64_t)(g.k / 8) * nseg}, str[2] = {inter * 4, (uint64_t)g.s_qwk * 4};
        const uint32_t box[3] = {TC_BN / 2, 2, (uint32_t)(TC_BK / 8 * kk)};
        rc = make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, g.qweight, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else if (g.format == FMT_GPTQ) {
        const uint64_t dims[2] = {(uint64_t)g.n, (uint64_t)(g.k / 8) * nseg}, str[1] = {(uint64_t)g.s_qwk * 4};
        const uint32_t box[2] = {TC_BN, (uint32_t)(TC_BK / 8 * kk)};
        rc = make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, g.qweight, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else {
        const uint64_t dims[2] = {(uint64_t)(g.n / 8), (uint64_t)g.k * nseg}, str[1] = {(uint64_t)g.s_qwk * 4};
        const uint32_t box[2] = {TC_BN / 8, TC_BK};
        rc = make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, g.qweight, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (rc) return TC_NOT_COVERED;
    {
        const uint64_t dims[2] = {(uint64_t)g.k, (uint64_t)g.m}, str[1] = {(uint64_t)g.s_am * 2};
        const uint32_t box[2] = {TC_BK, (uint32_t)tt};
        rc = make_tensor_map(&amap, g.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc) return TC_NOT_COVERED;   // layout the TMA cannot describe: the strided family takes it
    const CUtensorMapDataType elem = g.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (silu) {
        const uint64_t inter = (uint64_t)g.silu_inter;
        const uint64_t dims[3] = {inter, 2, (uint64_t)(g.k / g.group) * nseg}, str[2] = {inter * 2, (uint64_t)g.s_sk * 2};
        const uint32_t box[3] = {TC_BN / 2, 2, 1};
        rc = make_tensor_map(&smap, elem, 3, g.scales, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else {
        const uint64_t dims[2] = {(uint64_t)g.n, (uint64_t)(g.k / g.group) * nseg}, str[1] = {(uint64_t)g.s_sk * 2};
        const uint32_t box[2] = {TC_BN, 1};
        rc = make_tensor_map(&smap, elem, 2, g.scales, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (rc) return TC_NOT_COVERED;
    zmap = smap;
    if (g.qzeros && silu) {
        const uint64_t inter8 = (uint64_t)g.silu_inter / 8;
        const uint64_t dims[3] = {inter8, 2, (uint64_t)(g.k / g.group) * nseg}, str[2] = {inter8 * 4, (uint64_t)g.s_qzk * 4};
        const uint32_t box[3] = {TC_BN / 16, 2, 1};
        rc = make_tensor_map(&zmap, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, g.qzeros, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return TC_NOT_COVERED;
    } else if (g.qzeros) {
        const uint64_t dims[2] = {(uint64_t)(g.n / 8), (uint64_t)(g.k / g.group) * nseg}, str[1] = {(uint64_t)g.s_qzk * 4};
        const uint32_t box[2] = {TC_BN / 8, 1};
        rc = make_tensor_map(&zmap, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, g.qzeros, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return TC_NOT_COVERED;
    }

    TcArgs P;
    P.scales = g.scales; P.qzeros = g.qzeros; P.c = g.c;
    P.m = g.m; P.n = g.n; P.k = g.k; P.group = g.group;
    P.s_sk = g.s_sk; P.s_qzk = g.s_qzk; P.s_cm = g.s_cm;
    P.zero_offset = g.zero_offset;
    P.tt = tt; P.dq_log2 = log2i(dq_stages); P.act_log2 = log2i(act_stages); P.raw_log2 = log2i(raw_stages); P.ksplit = ksplit;
    P.kb_per_split = ceil_div(kb_total / kk, ksplit);      // in pipeline steps
    P.seg_offsets = g.seg_offsets;
    P.tile_list = grouped ? g.tile_list : nullptr;
    P.tile_count = g.tile_count;
    P.silu_inter = g.silu_inter;
    P.c_kperm = g.c_kperm ? 1 : 0;
    P.w_rows_per_seg = g.format == FMT_GPTQ ? g.k / 8 : g.k;
    P.g_rows_per_seg = g.k / g.group;
    P.status = (int *)g.ws;   // status word at the start of the scratch buffer
    if (!P.status) return fail(B200K_E_WORKSPACE, "w4a16 gemm (tensor core): workspace is NULL");

    if (g.a_kperm && !ts) return TC_NOT_COVERED;   // pre-permuted activations: only the tensor-memory operand variants take them
    if (silu && !ts) return TC_NOT_COVERED;
    if (g.bf16 && (silu || g.a_kperm || (g.format == FMT_GPTQ && !ts))) return TC_NOT_COVERED;
    auto kern = kk == 2 && silu ? (g2m1 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 1, false, true, false, 2>
                                        : g.a_kperm ? gemm_tc_kernel<FMT_GPTQ, 2, true, 2, true, true, false, 2> : gemm_tc_kernel<FMT_GPTQ, 2, true, 2, false, true, false, 2>)
                : kk == 2 && g2m1 ? (g.bf16 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 1, false, false, true, 2>
                                          : g.a_kperm ? gemm_tc_kernel<FMT_GPTQ, 2, true, 1, true, false, false, 2> : gemm_tc_kernel<FMT_GPTQ, 2, true, 1, false, false, false, 2>)
                : kk == 2 ? (g.bf16 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 2, false, false, true, 2>
                                  : g.a_kperm ? gemm_tc_kernel<FMT_GPTQ, 2, true, 2, true, false, false, 2> : gemm_tc_kernel<FMT_GPTQ, 2, true, 2, false, false, false, 2>)
                : g.bf16 && g2m1 ? (g.format == FMT_AWQ ? gemm_tc_kernel<FMT_AWQ, 2, false, 1, false, false, true> : gemm_tc_kernel<FMT_GPTQ, 2, true, 1, false, false, true>)
                : g.bf16 ? (g.format == FMT_AWQ ? (ng == 2 ? gemm_tc_kernel<FMT_AWQ, 2, false, 2, false, false, true> : gemm_tc_kernel<FMT_AWQ, 4, false, 1, false, false, true>)
                                              : (ng == 2 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 2, false, false, true> : gemm_tc_kernel<FMT_GPTQ, 4, true, 1, false, false, true>))
                : silu && g2m1 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 1, false, true>
                : silu ? (g.a_kperm ? (ng == 2 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 2, true, true> : gemm_tc_kernel<FMT_GPTQ, 4, true, 1, true, true>)
                                  : (ng == 2 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 2, false, true> : gemm_tc_kernel<FMT_GPTQ, 4, true, 1, false, true>))
                : g2m1 ? (g.format == FMT_AWQ ? gemm_tc_kernel<FMT_AWQ, 2, false, 1, false>
                          : ts ? (g.a_kperm ? gemm_tc_kernel<FMT_GPTQ, 2, true, 1, true> : gemm_tc_kernel<FMT_GPTQ, 2, true, 1, false>)
                               : gemm_tc_kernel<FMT_GPTQ, 2, false, 1, false>)
                : g.format == FMT_AWQ ? (ng == 2 ? gemm_tc_kernel<FMT_AWQ, 2, false, 2, false> : gemm_tc_kernel<FMT_AWQ, 4, false, 1, false>)
                : ts ? (g.a_kperm ? (ng == 2 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 2, true> : gemm_tc_kernel<FMT_GPTQ, 4, true, 1, true>)
                                  : (ng == 2 ? gemm_tc_kernel<FMT_GPTQ, 2, true, 2, false> : gemm_tc_kernel<FMT_GPTQ, 4, true, 1, false>))
                     : (ng == 2 ? gemm_tc_kernel<FMT_GPTQ, 2, false, 2, false> : gemm_tc_kernel<FMT_GPTQ, 4, false, 1, false>);
    {
        static OncePerDevice once[8][5];
        const int variant = g.bf16 ? (g.format == FMT_AWQ ? 7 : 6) : silu ? (g.a_kperm ? 5 : 4) : g.format == FMT_AWQ ? 1 : (ts ? (g.a_kperm ? 3 : 2) : 0);
        cudaError_t e = once[variant][kk == 2 ? (g2m1 ? 4 : 3) : g2m1 ? 2 : ng == 4].run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); });
        if (e != cudaSuccess) return fail((int)e, "w4a16 gemm (tensor core): shared memory: %s", cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    // grouped with a work list: one grid slice per listed (segment, token tile); without: the worst case per segment
    cfg.gridDim = dim3(col_tiles, listed ? g.max_tiles : tok_tiles, grouped && !listed ? g.num_segments : ksplit);
    cfg.blockDim = dim3(tc_threads(ng), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = grouped && !listed ? 1 : ksplit;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, wmap, amap, smap, zmap, P);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail((int)e, "w4a16 gemm (tensor core) launch: %s", cudaGetErrorString(e));
    }
    return 0;
}

}  // namespace b200k

// W4A16 GEMV (M = 1, group 128) on the integer dot-product instruction.
//
// The fp16 GEMV spends about three instructions per weight (nibble -> fp16, subtract the zero-point, half2 FMA,
// widening), and at 45 weights per clock per SM that the HBM stream of a B200 delivers, instruction issue is the
// limit, not memory.  Here the nibbles are never converted:
//     sum_k a_k (q_k - z) s  =  s * sa * ( sum_k A_k q_k  -  z * sum_k A_k ),     a_k ~ sa * A_k,
// with the 128 activations of a quantisation group turned once into 15-bit integers A_k = 128 ah_k + al_k
// (sa = max|a| / 16383 per group: the quantisation step is 3e-5 of the group's largest activation, an order of
// magnitude below fp16's own spacing at that magnitude), and the sums over k taken by dp4a on bytes: one LOP3
// extracts four nibbles of a packed word as four bytes, and two dp4a (ah, al) accumulate them in int32.  The odd
// nibbles are used in place, as bytes 16 q, and their sums shifted down at the end of the group (exact).
// The products are exact integers, so the only roundings are the activation quantisation and the final fp32
// scaling: closer to the exact result than products with fp16-rounded weights, inside the same tolerance.
// A group in which one activation dwarfs the rest (max |a| > 64 mean |a|: the "massive activation" channels of LLMs) would
// leave the other values too few levels; such a group is multiplied in fp32 instead, nibble by nibble (three times the
// instructions, for the few groups it concerns).
//
// Work split as in the fp16 GEMV: a cluster of KSPLIT CTAs shares one block of columns and splits K by
// quantisation group over its warps; the cluster reduces through distributed shared memory in a fixed order.
//   GPTQ [K/8, N]: a word = 8 k of one column; a thread owns 4 adjacent columns (one 16-byte load per packed row);
//                  activation bytes are laid out per packed row as (k0,k2,k4,k6) and (k1,k3,k5,k7).
//   AWQ  [K, N/8]: a word = 8 columns of one k; a thread owns one word column; four rows are transposed as 4 x 4
//                  byte matrices (PRMT) so that a word holds four k of one column.
#include <cooperative_groups.h>

#include "gemm.cuh"

namespace cg = cooperative_groups;

namespace b200k {

constexpr int GI_THREADS = 256;
constexpr int GI_WARPS = GI_THREADS / 32;
constexpr int GI_GROUP = 128;

__device__ __forceinline__ int dp4a_us(uint32_t w_unsigned_bytes, uint32_t a_signed_bytes, int acc) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(w_unsigned_bytes), "r"(a_signed_bytes), "r"(acc));
    return d;
}
__device__ __forceinline__ uint32_t ldg_nc_word(const void *p) {
    uint32_t r;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}

// The 128 activations of one group -> 15-bit integers; lane i holds stored positions 4i .. 4i+3.  Returns the
// lane's four high bytes and four low bytes (byte j = stored position 4i + j), the group's scale and sum(A).
// `outlier`: one activation holds more than half of the group's total magnitude (max |a| > 64 mean |a|).  The 15-bit grid
// is then too coarse for the other 127 values (its step is max |a| / 16383), and the caller multiplies that group in fp32.
__device__ __forceinline__ void quantise_group(const __half *a_group, int lane, uint32_t &qh, uint32_t &ql, float &sa, int &asum,
                                               bool &outlier) {
    const uint2 u = *reinterpret_cast<const uint2 *>(a_group + lane * 4);
    const float2 f01 = h2_to_f2(u.x), f23 = h2_to_f2(u.y);
    float amax = fmaxf(fmaxf(fabsf(f01.x), fabsf(f01.y)), fmaxf(fabsf(f23.x), fabsf(f23.y)));
    float aabs = (fabsf(f01.x) + fabsf(f01.y)) + (fabsf(f23.x) + fabsf(f23.y));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        aabs += __shfl_xor_sync(0xffffffffu, aabs, o);
    }
    outlier = 2.f * amax > aabs;
    sa = amax * (1.f / 16383.f);
    const float inv = amax > 0.f ? 16383.f / amax : 0.f;
    const int i0 = __float2int_rn(f01.x * inv), i1 = __float2int_rn(f01.y * inv);
    const int i2 = __float2int_rn(f23.x * inv), i3 = __float2int_rn(f23.y * inv);
    asum = __reduce_add_sync(0xffffffffu, i0 + i1 + i2 + i3);
    qh = (uint32_t)((i0 >> 7) & 255) | ((uint32_t)((i1 >> 7) & 255) << 8) | ((uint32_t)((i2 >> 7) & 255) << 16) |
         ((uint32_t)((i3 >> 7) & 255) << 24);
    ql = (uint32_t)(i0 & 127) | ((uint32_t)(i1 & 127) << 8) | ((uint32_t)(i2 & 127) << 16) | ((uint32_t)(i3 & 127) << 24);
}

// Fixed-order reduction of per-thread totals: over the k-warps of the CTA, then over the CTAs of the cluster
// (distributed shared memory); rank 0 stores fp16.  NV = values per thread (4 or 8), laid out as float4s.
template <int NV>
__device__ __forceinline__ void reduce_and_store(float (&tot)[NV], float4 *red4, int part, int parts, int slot, int slots_per_part,
                                                 int ksplit, bool live, __half *dst) {
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int Q = NV / 4;
    if (part > 0) {
#pragma unroll
        for (int q = 0; q < Q; ++q)
            red4[(((part - 1) * slots_per_part + slot) * Q) + q] = make_float4(tot[4 * q], tot[4 * q + 1], tot[4 * q + 2], tot[4 * q + 3]);
    }
    __syncthreads();
    if (part == 0) {
        for (int j = 0; j < parts - 1; ++j) {
#pragma unroll
            for (int q = 0; q < Q; ++q) {
                const float4 o = red4[((j * slots_per_part + slot) * Q) + q];
                tot[4 * q] += o.x; tot[4 * q + 1] += o.y; tot[4 * q + 2] += o.z; tot[4 * q + 3] += o.w;
            }
        }
    }
    __syncthreads();
    if (part == 0) {
#pragma unroll
        for (int q = 0; q < Q; ++q) red4[slot * Q + q] = make_float4(tot[4 * q], tot[4 * q + 1], tot[4 * q + 2], tot[4 * q + 3]);
    }
    cluster.sync();
    if (cluster.block_rank() == 0 && part == 0 && live) {
        float s[NV];
#pragma unroll
        for (int c = 0; c < NV; ++c) s[c] = 0.f;
        for (int r = 0; r < ksplit; ++r) {
            const float4 *peer = cluster.map_shared_rank(red4, r);
#pragma unroll
            for (int q = 0; q < Q; ++q) {
                const float4 o = peer[slot * Q + q];
                s[4 * q] += o.x; s[4 * q + 1] += o.y; s[4 * q + 2] += o.z; s[4 * q + 3] += o.w;
            }
        }
        uint32_t o[NV / 2];
#pragma unroll
        for (int c = 0; c < NV / 2; ++c) o[c] = f2_to_h2(s[2 * c], s[2 * c + 1]);
        if (NV == 4) *reinterpret_cast<uint2 *>(dst) = make_uint2(o[0], o[1]);
        else *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[NV / 2 - 2], o[NV / 2 - 1]);
    }
    cluster.sync();  // peers keep their shared memory alive until rank 0 has read it
}

// CW = column-warps per CTA (each covers 128 columns); the other 8 / CW warps split K.
template <int CW>
__global__ void __launch_bounds__(GI_THREADS)
gemv_gptq_i8_kernel(GemmArgs g, int ksplit) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint4 *act = reinterpret_cast<uint4 *>(smem_raw);                              // [GI_WARPS][16 packed rows]: (Eh, Oh, El, Ol)
    float4 *red4 = reinterpret_cast<float4 *>(smem_raw + GI_WARPS * 16 * sizeof(uint4));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cw = warp % CW, kw = warp / CW;
    constexpr int KW = GI_WARPS / CW;
    const int col = blockIdx.x * (128 * CW) + cw * 128 + lane * 4;
    const int kslot = blockIdx.y * KW + kw, kslots = ksplit * KW;
    const int groups = g.k / GI_GROUP;
    const bool live = col < g.n;
    uint4 *my_act = act + warp * 16;

    uint4 wreg[16];
    uint2 su = make_uint2(0, 0);
    uint32_t zw = 0;
    auto request = [&](int grp) {
        if (g.qzeros) zw = ldg_nc_word(g.qzeros + (long)grp * g.s_qzk + col / 8);
        su = *reinterpret_cast<const uint2 *>(g.scales + (long)grp * g.s_sk + col);
        const int32_t *wp = g.qweight + (long)grp * 16 * g.s_qwk + col;
#pragma unroll
        for (int r = 0; r < 16; ++r) wreg[r] = ldg_nc_v4(wp + (long)r * g.s_qwk);
    };
    if (live && kslot < groups) request(kslot);

    pdl_wait();                 // the activation vector comes from the kernel before; the weights do not
    pdl_launch_dependents();

    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    for (int grp = kslot; grp < groups; grp += kslots) {
        if (live && grp != kslot) request(grp);
        // activations of the group -> bytes, per packed row r (lanes 2r, 2r+1): even k and odd k of the row
        uint32_t qh, ql;
        float sa;
        int asum;
        bool outlier;
        quantise_group(g.a + (long)grp * GI_GROUP, lane, qh, ql, sa, asum, outlier);
        if (outlier) {
            // fp32 for this group: sum_k a_k (q_k - z), every lane reading the same activation (one broadcast load each)
            if (!live) continue;
            const float2 s01 = h2_to_f2(su.x), s23 = h2_to_f2(su.y);
            const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
            const uint32_t zsh = zw >> (4 * (col % 8));
            float zf[4], accx[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 4; ++c) zf[c] = (float)(g.qzeros ? (int)((zsh >> (4 * c)) & 15u) + g.zero_offset : 8);
            const __half *ag = g.a + (long)grp * GI_GROUP;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const uint32_t w[4] = {wreg[r].x, wreg[r].y, wreg[r].z, wreg[r].w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int pos = g.a_kperm ? ((j & 3) * 2 + (j >> 2)) : j;      // where k = 8r + j sits in its 8-block
                    const float av = __half2float(ag[8 * r + pos]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) accx[c] = fmaf(av, (float)((w[c] >> (4 * j)) & 15u) - zf[c], accx[c]);
                }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) tot[c] += accx[c] * sc[c];
            continue;
        }
        {
            const uint32_t ph = __shfl_xor_sync(0xffffffffu, qh, 1), pl = __shfl_xor_sync(0xffffffffu, ql, 1);
            const bool odd = lane & 1;
            const uint32_t h0 = odd ? ph : qh, h1 = odd ? qh : ph;      // stored positions 0..3 and 4..7 of the row
            const uint32_t l0 = odd ? pl : ql, l1 = odd ? ql : pl;
            // plain order: positions are k0..k7; pre-permuted order: (k0,k4,k1,k5 | k2,k6,k3,k7)
            const uint32_t sel_e = g.a_kperm ? 0x5140u : 0x6420u, sel_o = g.a_kperm ? 0x7362u : 0x7531u;
            const uint2 mine = odd ? make_uint2(__byte_perm(l0, l1, sel_e), __byte_perm(l0, l1, sel_o))
                                   : make_uint2(__byte_perm(h0, h1, sel_e), __byte_perm(h0, h1, sel_o));
            __syncwarp();       // the previous group's reads of this warp's rows are done
            reinterpret_cast<uint2 *>(my_act + (lane >> 1))[odd ? 1 : 0] = mine;
            __syncwarp();
        }
        if (!live) continue;
        int ae[4][2], ao[4][2];     // per column: sums over even / odd k (odd: 16 x) against (ah, al)
#pragma unroll
        for (int c = 0; c < 4; ++c) ae[c][0] = ae[c][1] = ao[c][0] = ao[c][1] = 0;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const uint4 av = my_act[r];
            const uint32_t w[4] = {wreg[r].x, wreg[r].y, wreg[r].z, wreg[r].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t e = w[c] & 0x0F0F0F0Fu, o = w[c] & 0xF0F0F0F0u;
                ae[c][0] = dp4a_us(e, av.x, ae[c][0]);
                ae[c][1] = dp4a_us(e, av.z, ae[c][1]);
                ao[c][0] = dp4a_us(o, av.y, ao[c][0]);
                ao[c][1] = dp4a_us(o, av.w, ao[c][1]);
            }
        }
        const float2 s01 = h2_to_f2(su.x), s23 = h2_to_f2(su.y);
        const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
        const uint32_t zsh = zw >> (4 * (col % 8));
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int z = g.qzeros ? (int)((zsh >> (4 * c)) & 15u) + g.zero_offset : 8;
            const int dot = 128 * (ae[c][0] + (ao[c][0] >> 4)) + ae[c][1] + (ao[c][1] >> 4);
            tot[c] += (float)(dot - z * asum) * (sc[c] * sa);
        }
    }
    reduce_and_store<4>(tot, red4, kw, KW, cw * 32 + lane, 32 * CW, ksplit, live, g.c + col);
}

// UR consecutive activations (one per lane group) -> 15-bit integers with their own scale: lane i returns the bytes of
// positions 4i .. 4i+3 of the unit (lanes >= UR / 4 return zeros).  UR = 128: a whole quantisation group, 4 values per
// lane; UR = 32: one value per lane, packed by fours.
template <int UR>
__device__ __forceinline__ void quantise_unit(const __half *a_unit, int lane, uint32_t &qh, uint32_t &ql, float &sa, int &asum,
                                              bool &outlier) {
    if (UR == 128) {
        quantise_group(a_unit, lane, qh, ql, sa, asum, outlier);
        return;
    }
    const float f = __half2float(a_unit[lane]);
    float amax = fabsf(f), aabs = fabsf(f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        aabs += __shfl_xor_sync(0xffffffffu, aabs, o);
    }
    outlier = 2.f * amax > aabs;      // one value holds more than half of the unit's magnitude
    sa = amax * (1.f / 16383.f);
    const float inv = amax > 0.f ? 16383.f / amax : 0.f;
    const int i0 = __float2int_rn(f * inv);
    asum = __reduce_add_sync(0xffffffffu, i0);
    // lane l holds position l: gather positions 4i .. 4i+3 into lane i
    uint32_t h = 0, l = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int v = __shfl_sync(0xffffffffu, i0, (lane * 4 + j) & 31);
        h |= (uint32_t)((v >> 7) & 255) << (8 * j);
        l |= (uint32_t)(v & 127) << (8 * j);
    }
    qh = lane < 8 ? h : 0u;
    ql = lane < 8 ? l : 0u;
}

// fp32 product of `rows` rows of one word column (8 weight columns) with their activations: acc[c] = sum_k a_k (q_kc - z_c).
// Out of line on purpose: it is the rare path, and inlined it costs the fast path its registers.
__device__ __noinline__ void awq_rows_fp32(const __half *a, const int32_t *wp, long stride, int rows, uint32_t zw, float *acc) {
    float x[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) x[c] = 0.f;
#pragma unroll 2
    for (int j = 0; j < rows; ++j) {
        const float av = __half2float(a[j]);            // every lane reads the same activation: one broadcast load
        const uint32_t wj = ldg_nc_word(wp + (long)j * stride);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int sh = 4 * awq_slot(c);
            x[c] = fmaf(av, (float)((wj >> sh) & 15u) - (float)((zw >> sh) & 15u), x[c]);
        }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = x[c];
}

// A warp covers 256 columns (one word per lane and row) and walks units of UR rows: a whole quantisation group, or a
// quarter of one when the matrix is too narrow to fill the machine with whole groups per warp.  Every unit quantises its
// own activations (its own scale: the identity above holds for any subset of k).  Rows are requested in half-batches of
// 16 held in NB register buffers that rotate: while one is multiplied, NB - 1 are in flight (narrow matrices have few
// warps, so each must keep more bytes in flight).
// CW = columns per warp.  256: a lane owns one word column (8 weight columns) over all rows of the warp's units.  128: a
// half-warp owns 16 word columns and half the rows of every unit (the halves are added by a shuffle at the end), which
// doubles the column blocks of a narrow matrix: at N = 4096 the widest cluster gives 128 CTAs of 256 columns, fewer than SMs.
template <int UR, int NB, int CW>
__global__ void __launch_bounds__(GI_THREADS, 2)      // 128 registers: narrow matrices need two CTAs per SM to run in one wave
gemv_awq_i8_kernel(GemmArgs g, int ksplit) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint2 *act = reinterpret_cast<uint2 *>(smem_raw);                              // [GI_WARPS][32]: (ah, al) of 4 consecutive k
    float4 *red4 = reinterpret_cast<float4 *>(smem_raw + GI_WARPS * 16 * sizeof(uint4));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool HALF = CW == 128;
    const int hp = HALF ? lane >> 4 : 0;              // which half of a unit's rows this lane reads
    const int wl = HALF ? lane & 15 : lane;           // word column within the warp's block
    constexpr int RL = HALF ? UR / 2 : UR;            // rows of a unit per lane
    const int col = blockIdx.x * CW + wl * 8;         // 8 columns per thread
    const int uslot = blockIdx.y * GI_WARPS + warp, uslots = ksplit * GI_WARPS;
    const int units = g.k / UR;
    const bool live = col < g.n;
    uint2 *my_act = act + warp * 32;
    constexpr int HB = 16;                            // rows per half-batch
    constexpr int HPU = RL / HB;                      // half-batches per unit (and lane)
    constexpr int UPG = GI_GROUP / UR;                // units per quantisation group

    uint32_t w[NB][HB];
    uint4 su = make_uint4(0, 0, 0, 0);
    uint32_t zw = 0;
    auto request_meta = [&](int unit) {
        if (unit < units) {
            zw = ldg_nc_word(g.qzeros + (long)(unit / UPG) * g.s_qzk + col / 8);
            su = *reinterpret_cast<const uint4 *>(g.scales + (long)(unit / UPG) * g.s_sk + col);
        }
    };
    // half-batch number t of this warp's sequence (unit uslot + (t / HPU) uslots, part t % HPU) -> buffer b
    auto request_rows = [&](uint32_t (&buf)[HB], int first_unit, int t) {
        const int unit = first_unit + (t / HPU) * uslots;
        if (unit < units) {
            const int32_t *wp = g.qweight + (long)(unit * UR + hp * RL + (t % HPU) * HB) * g.s_qwk + col / 8;
#pragma unroll
            for (int j = 0; j < HB; ++j) buf[j] = ldg_nc_word(wp + (long)j * g.s_qwk);
        }
    };
    if (live) {
        request_meta(uslot);
#pragma unroll
        for (int b = 0; b < NB; ++b) request_rows(w[b], uslot, b);
    }

    pdl_wait();
    pdl_launch_dependents();

    float tot[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) tot[c] = 0.f;
    // HPU and NB are powers of two, so the buffer of half-batch t is t % NB with t counted from this warp's first unit; a
    // pass of the loop below covers max(HPU, NB) half-batches, i.e. one or more whole units, and ends on buffer 0 again
    constexpr int UPP = NB > HPU ? NB / HPU : 1;      // units per pass
    for (int u0 = uslot; u0 < units; u0 += UPP * uslots) {
#pragma unroll
        for (int uu = 0; uu < UPP; ++uu) {
            const int u = u0 + uu * uslots;
            if (u >= units) break;
            uint32_t qh, ql;
            float sa;
            int asum;
            bool outlier;
            quantise_unit<UR>(g.a + (long)u * UR, lane, qh, ql, sa, asum, outlier);
            __syncwarp();
            my_act[lane] = make_uint2(qh, ql);          // bytes already in k order: lane i = k 4i .. 4i+3
            __syncwarp();
            if (!live) continue;
            const uint4 su_now = su;
            const uint32_t zw_now = zw;
            request_meta(u + uslots);
            // byte b of the even-nibble words = nibble 2b = column (0,4,1,5)[b]; of the odd-nibble words = nibble 2b+1 =
            // column (2,6,3,7)[b] (the AWQ order [0,4,1,5,2,6,3,7] maps column -> nibble)
            if (outlier) {
                // fp32 for this unit; its rows are read again (from L2: rare), the register buffers only turn
                float accx[8];
                awq_rows_fp32(g.a + (long)u * UR + hp * RL, g.qweight + ((long)u * UR + hp * RL) * g.s_qwk + col / 8, g.s_qwk, RL, zw_now, accx);
                const float2 sA = h2_to_f2(su_now.x), sB = h2_to_f2(su_now.y), sC = h2_to_f2(su_now.z), sD = h2_to_f2(su_now.w);
                const float sc[8] = {sA.x, sA.y, sB.x, sB.y, sC.x, sC.y, sD.x, sD.y};
#pragma unroll
                for (int c = 0; c < 8; ++c) tot[c] += accx[c] * sc[c];
#pragma unroll
                for (int hb = 0; hb < HPU; ++hb) request_rows(w[(uu * HPU + hb) % NB], u0, uu * HPU + hb + NB);
                continue;
            }
            int ae[4][2], ao[4][2];
#pragma unroll
            for (int c = 0; c < 4; ++c) ae[c][0] = ae[c][1] = ao[c][0] = ao[c][1] = 0;
#pragma unroll
            for (int hb = 0; hb < HPU; ++hb) {
                const int t = uu * HPU + hb;            // half-batch number within the pass
                uint32_t (&buf)[HB] = w[t % NB];
#pragma unroll
                for (int j = 0; j < HB; j += 4) {
                    const uint2 av = my_act[(hp * RL + hb * HB + j) >> 2];
                    uint32_t e[4], o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        e[i] = buf[j + i] & 0x0F0F0F0Fu;
                        o[i] = buf[j + i] & 0xF0F0F0F0u;
                    }
                    // 4 x 4 byte transposes: word i (row k+i, four columns) -> word c (column c, rows k .. k+3)
                    const uint32_t e01l = __byte_perm(e[0], e[1], 0x5140), e23l = __byte_perm(e[2], e[3], 0x5140);
                    const uint32_t e01h = __byte_perm(e[0], e[1], 0x7362), e23h = __byte_perm(e[2], e[3], 0x7362);
                    const uint32_t o01l = __byte_perm(o[0], o[1], 0x5140), o23l = __byte_perm(o[2], o[3], 0x5140);
                    const uint32_t o01h = __byte_perm(o[0], o[1], 0x7362), o23h = __byte_perm(o[2], o[3], 0x7362);
                    const uint32_t ce[4] = {__byte_perm(e01l, e23l, 0x5410), __byte_perm(e01l, e23l, 0x7632),
                                            __byte_perm(e01h, e23h, 0x5410), __byte_perm(e01h, e23h, 0x7632)};
                    const uint32_t co[4] = {__byte_perm(o01l, o23l, 0x5410), __byte_perm(o01l, o23l, 0x7632),
                                            __byte_perm(o01h, o23h, 0x5410), __byte_perm(o01h, o23h, 0x7632)};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        ae[c][0] = dp4a_us(ce[c], av.x, ae[c][0]);
                        ae[c][1] = dp4a_us(ce[c], av.y, ae[c][1]);
                        ao[c][0] = dp4a_us(co[c], av.x, ao[c][0]);
                        ao[c][1] = dp4a_us(co[c], av.y, ao[c][1]);
                    }
                }
                request_rows(buf, u0, t + NB);          // the half-batch that uses this buffer next
            }
            const float2 sA = h2_to_f2(su_now.x), sB = h2_to_f2(su_now.y), sC = h2_to_f2(su_now.z), sD = h2_to_f2(su_now.w);
            const float sc[8] = {sA.x, sA.y, sB.x, sB.y, sC.x, sC.y, sD.x, sD.y};
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int ce_col = (b & 1) * 4 + (b >> 1);          // (0,4,1,5)[b]
                const int co_col = ce_col + 2;                      // (2,6,3,7)[b]
                const int ze = (int)((zw_now >> (8 * b)) & 15u), zo = (int)((zw_now >> (8 * b + 4)) & 15u);
                const int de = 128 * ae[b][0] + ae[b][1];
                const int dn = 128 * (ao[b][0] >> 4) + (ao[b][1] >> 4);
                // (two halves of the rows in two half-warps: the zero-point term of the whole unit goes with the first)
                const int asum_h = hp == 0 ? asum : 0;
                tot[ce_col] += (float)(de - ze * asum_h) * (sc[ce_col] * sa);
                tot[co_col] += (float)(dn - zo * asum_h) * (sc[co_col] * sa);
            }
        }
    }
    if (HALF) {
#pragma unroll
        for (int c = 0; c < 8; ++c) tot[c] += __shfl_xor_sync(0xffffffffu, tot[c], 16);
    }
    reduce_and_store<8>(tot, red4, warp, GI_WARPS, wl, HALF ? 16 : 32, ksplit, live && hp == 0, g.c + col);
}

static inline int imin(int a, int b) { return a < b ? a : b; }
static inline int imax(int a, int b) { return a > b ? a : b; }

int gemv_i8_launch(const GemmArgs &g) {
    if (g.m != 1 || g.group != GI_GROUP || g.bf16 || g.k % GI_GROUP) return TC_NOT_COVERED;
    const int groups = g.k / GI_GROUP;
    // GPTQ: 256 columns per CTA (2 column-warps x 4 k-warps), or 128 (1 x 8) when 256-column blocks with the largest
    // cluster would leave SMs without a CTA.  AWQ: 256 columns per CTA, all 8 warps split K, by whole groups, or by
    // quarter groups when K is short and whole groups per warp with the largest cluster would leave most SMs without a CTA.
    const bool narrow = ceil_div(g.n, 256) * 8 < 2 * sm_count();
    const int cw = g.format != FMT_GPTQ ? 1 : narrow ? 1 : 2;
    int awq_cols = narrow ? 128 : 256;       // AWQ: columns per warp (= per CTA)
    {   // tuning override
        const int v = env_int("B200K_GEMV_AWQ_COLS", 0);
        if (v == 128 || v == 256) awq_cols = v;
    }
    const int colblocks = g.format == FMT_GPTQ ? ceil_div(g.n, 128 * cw) : ceil_div(g.n, awq_cols);
    const int kwarps = GI_WARPS / cw;
    int unit_rows = GI_GROUP;
    // (measured with 128-column blocks: whole groups win -- 4096 x 4096 4.6 against 6.1 us, 4096 x 6144 5.6 against 10.6 us)
    if (g.format == FMT_AWQ && awq_cols == 256 && groups < 64 && colblocks * imin(8, imax(1, groups / (2 * kwarps))) < sm_count()) unit_rows = 32;
    {   // tuning override
        const int v = env_int("B200K_GEMV_UNIT", 0);
        if (g.format == FMT_AWQ && (v == 32 || v == 128)) unit_rows = v;
    }
    const int units = g.k / unit_rows;
    // enough CTAs for ~2 per SM, cluster size a power of two <= 8, no warp without a unit
    int ksplit = 1;
    while (ksplit < 8 && colblocks * ksplit < 2 * sm_count() && ksplit * 2 * kwarps <= units) {
        // 256-column blocks: never past two CTAs per SM (4096 x 28672: AWQ 224 CTAs 16.7 us, 448 CTAs 18.2 us; GPTQ 12.6 and 14.4 us)
        if ((g.format == FMT_AWQ ? awq_cols == 256 : cw == 2) && colblocks * ksplit * 2 > 2 * sm_count()) break;
        ksplit *= 2;
    }
    {   // tuning override
        const int v = env_int("B200K_GEMV_KSPLIT", 0);
        if ((v == 1 || v == 2 || v == 4 || v == 8) && v * kwarps <= units) ksplit = v;
    }
    const size_t smem = GI_WARPS * 16 * sizeof(uint4) + (size_t)GI_WARPS * 256 * sizeof(float);
    void (*kern)(GemmArgs, int);
    if (g.format == FMT_GPTQ) kern = cw == 2 ? gemv_gptq_i8_kernel<2> : gemv_gptq_i8_kernel<1>;
    else {
        // four half-batches per warp in flight (measured: ahead of two at every shape of the Llama-3-8B projections)
        int nb = 4;
        const int v = env_int("B200K_GEMV_DEPTH", 0);      // tuning override
        if (v == 2 || v == 4) nb = v;
        if (awq_cols == 128)
            kern = unit_rows == 32 ? (nb == 4 ? gemv_awq_i8_kernel<32, 4, 128> : gemv_awq_i8_kernel<32, 2, 128>)
                                   : (nb == 4 ? gemv_awq_i8_kernel<128, 4, 128> : gemv_awq_i8_kernel<128, 2, 128>);
        else
            kern = unit_rows == 32 ? (nb == 4 ? gemv_awq_i8_kernel<32, 4, 256> : gemv_awq_i8_kernel<32, 2, 256>)
                                   : (nb == 4 ? gemv_awq_i8_kernel<128, 4, 256> : gemv_awq_i8_kernel<128, 2, 256>);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(colblocks, ksplit, 1);
    cfg.blockDim = dim3(GI_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ksplit;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, g, ksplit);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail((int)e, "gemv launch: %s", cudaGetErrorString(e));
    }
    return 0;
}

}  // namespace b200k

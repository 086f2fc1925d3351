// Shared description of one W4A16 GEMM call, handed from the C-ABI entry points to
// the kernel families (strided CUDA-core, split-K GEMV, tcgen05 tensor-core).
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace b200k {

enum WeightFormat { FMT_GPTQ = 0, FMT_AWQ = 1 };

struct GemmArgs {
    const __half *a;
    const int32_t *qweight;
    const __half *scales;
    const int32_t *qzeros;  // nullptr: symmetric zero-point 8 (GPTQ only)
    __half *c;
    int m, n, k, group;
    int s_am, s_ak, s_qwk, s_qwn, s_sk, s_sn, s_qzk, s_qzn, s_cm, s_cn;
    int format;       // WeightFormat
    int zero_offset;  // added to the stored zero nibble (GPTQ GEMM: 1, AWQ: 0)
    // grouped mode (fused MoE): `a` and `c` hold num_segments row segments back to back, segment e =
    // rows [seg_offsets[e], seg_offsets[e+1]) (device array), multiplied by weight matrix e of a stack
    // [num_segments, K/8 (or K), ...] laid out contiguously; m = total rows.  nullptr: ordinary GEMM.
    const int *seg_offsets;
    int num_segments;
    // fused silu_mul epilogue (tensor-core path, GPTQ): the weight holds 2 * silu_inter columns, gate columns first, up
    // columns second (the half-split layout of fused_silu_mul_interleaved, elementwise.rs:199-206); c has silu_inter
    // columns and receives silu(gate) * up.  n is then 2 * silu_inter.  0: plain GEMM.
    int silu_inter;
    // grouped mode only: compact list of (segment, first row) work items, one per token tile that holds rows, and their
    // number (device memory, written by the kernel that builds the segments); max_tiles bounds the grid.  nullptr: one
    // grid slice per segment and token tile of the worst case.
    const int2 *tile_list;
    const int *tile_count;
    int max_tiles;
    int expected_m;   // grouped: rows expected over all segments when m is only a capacity (expert-parallel MoE), else 0
    bool bf16;        // a, scales and c are bfloat16 instead of fp16 (tensor-core and strided families)
    bool c_kperm;     // fused silu_mul epilogue only: write the output in the pre-permuted order (it feeds a GEMM that reads it so)
    bool a_kperm;     // activations pre-permuted per 8 consecutive k to (k0,k4,k1,k5,k2,k6,k3,k7) (tensor-core GPTQ path, GEMV)
    int *plan_out;    // host pointer: when set, the tensor-core family writes its launch plan there and launches nothing
    void *ws;         // scratch (may be nullptr when the chosen path needs none)
    size_t ws_bytes;
    cudaStream_t stream;
};

// True when every inner stride is 1 and the row strides / pointers allow 16-byte access.
bool gemm_layout_is_canonical(const GemmArgs &g);

// Kernel families.  Each returns 0 on launch, a B200K_E_* / CUDA code on failure.
int gemm_strided_launch(const GemmArgs &g);
int gemv_launch(const GemmArgs &g);
// Integer dot-product GEMV (gemv_i8.cu): M = 1, fp16, group 128; TC_NOT_COVERED otherwise.
int gemv_i8_launch(const GemmArgs &g);
// C [M, inter] = silu(A Wgate) * (A Wup) for a GPTQ weight [K, 2 * inter] whose first `inter` columns are the gate
// projection (tensor-core family, silu in the GEMM's epilogue).  TC_NOT_COVERED when the shape is outside it.
int gptq_gemm_silu_mul_launch(const __half *a, const int32_t *qweight, const __half *scales, const int32_t *qzeros, __half *c,
                              int m, int inter, int k, int group, bool a_kperm, bool c_kperm, cudaStream_t stream);
// Tensor-core path (tcgen05 + TMEM).  Returns TC_NOT_COVERED when the shape is outside what it
// covers (the caller then takes another family); the value is distinct from every B200K_E_* code
// and from every cudaError_t.
constexpr int TC_NOT_COVERED = -1000;
int gemm_tc_launch(const GemmArgs &g);
// Token tile (MMA N extent) the tensor-core path uses for m rows in `segments` row segments (1: ordinary GEMM).
int gemm_tc_token_tile(int m, int segments);

// ---- nibble -> fp16 helpers (device) -----------------------------------------
// For a 32-bit word w holding nibbles n0..n7 (n_i at bits 4i..4i+3):
//   lo(w)      = (w & 0x000F000F) | 0x64006400  -> half2 (1024+n0, 1024+n4)
//   hi(w)      = (w & 0x00F000F0) | 0x54005400  -> half2 (  64+n1,   64+n5)
//   lo(w >> 8), hi(w >> 8)                      -> (n2, n6), (n3, n7)
// Subtracting (1024+z) resp. (64+z) in fp16 is exact for z in 0..16, so the result
// is the integer (n - z) with no rounding; one fp16 multiply by the scale then
// rounds once, the same value as the reference's f32 product rounded to fp16
// (w4a16_gptq_gemm_typed.rs:256-260): an integer of at most 5 bits times an 11-bit
// significand is exact in fp32.
__device__ __forceinline__ uint32_t nib_lo(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x64006400, 0xEA;" : "=r"(r) : "r"(w));
    return r;
}
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x00F000F0, 0x54005400, 0xEA;" : "=r"(r) : "r"(w));
    return r;
}
__device__ __forceinline__ __half2 u2h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t h22u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// Magic zero constants for a zero-point z (0..16): (1024+z) and (64+z) in both halves,
// built with integer arithmetic on the fp16 bit patterns (ulp is 1 at 1024 and 1/16 at 64).
__device__ __forceinline__ void zero_magic(int z, __half2 &zlo, __half2 &zhi) {
    zlo = u2h2((uint32_t)(0x6400 + z) * 0x10001u);
    zhi = u2h2((uint32_t)(0x5400 + (z << 4)) * 0x10001u);
}

// ---- the same for bf16 (7 mantissa bits): only a nibble at bits 0..3 of a half can be turned into a number by
// OR-ing an exponent, (w & 0x000F000F) | 0x43004300 -> (128 + n0, 128 + n4); the other three pairs come from
// w >> 4, w >> 8, w >> 12.  Subtracting (128 + z) is exact and one bf16 multiply by the scale rounds once, like the
// reference's f32 product rounded to bf16 (a 5-bit integer times an 8-bit significand is exact in fp32).
__device__ __forceinline__ uint32_t nib_bf(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(r) : "r"(w));
    return r;
}
// The four value pairs of a word, (n0,n4) (n1,n5) (n2,n6) (n3,n7), as biased numbers of the element type
template <bool BF> __device__ __forceinline__ void nib4(uint32_t w, uint32_t (&x)[4]) {
    if (BF) {
        x[0] = nib_bf(w); x[1] = nib_bf(w >> 4); x[2] = nib_bf(w >> 8); x[3] = nib_bf(w >> 12);
    } else {
        const uint32_t w8 = w >> 8;
        x[0] = nib_lo(w); x[1] = nib_hi(w); x[2] = nib_lo(w8); x[3] = nib_hi(w8);
    }
}
// The biases of those four pairs plus a zero-point z, in both halves
template <bool BF> __device__ __forceinline__ void zero_magic4(int z, uint32_t (&m)[4]) {
    if (BF) {
        m[0] = m[1] = m[2] = m[3] = (uint32_t)(0x4300 + z) * 0x10001u;
    } else {
        __half2 zl, zh;
        zero_magic(z, zl, zh);
        m[0] = m[2] = h22u(zl);
        m[1] = m[3] = h22u(zh);
    }
}
// (x - z) * s on a pair, in the element type: exact difference, one rounding
template <bool BF> __device__ __forceinline__ uint32_t sub_mul(uint32_t x, uint32_t z, uint32_t s) {
    if (BF) {
        const __nv_bfloat162 r = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162 *>(&x), *reinterpret_cast<__nv_bfloat162 *>(&z)),
                                         *reinterpret_cast<__nv_bfloat162 *>(&s));
        return *reinterpret_cast<const uint32_t *>(&r);
    }
    return h22u(__hmul2(__hsub2(u2h2(x), u2h2(z)), u2h2(s)));
}
template <bool BF> __device__ __forceinline__ void store_elem(__half *p, float v) {
    if (BF) *reinterpret_cast<__nv_bfloat16 *>(p) = __float2bfloat16_rn(v);
    else *p = __float2half_rn(v);
}

// position of column j (0..7) inside an AWQ word (awq_gemm_int4_typed.rs:137-151)
__host__ __device__ __forceinline__ int awq_slot(int j) { return (j >> 1) + ((j & 1) << 2); }

}  // namespace b200k

// Fused MoE (top-k routing, token permute, grouped int4 expert GEMMs with silu_mul in the first one's
// epilogue, weighted un-permute): six launches -- route, permute (+ the GEMMs' work list), gather, w13 GEMM,
// w2 GEMM, combine.  The reference has no such kernel; the pieces follow its conventions: GPTQ
// weight layout of w4a16_gptq_gemm_typed, and the half-split gate|up layout of
// fused_silu_mul_interleaved (gate = first half of a row, up = second half).
//
// Bit-exact contract (the tests compare indices with ==): experts are ranked by router logit,
// highest first, ties to the lowest expert index (softmax is monotonic, so this is the top-k
// of the softmax without depending on how exp rounds); pair p = token*k + j; the segmented
// list orders pairs by expert, then by pair index.
#include "comm.cuh"
#include "gemm.cuh"

namespace b200k {

constexpr int MOE_MAX_E = 64;
constexpr int MOE_MAX_K = 8;

// one thread per token
__global__ void __launch_bounds__(256)
moe_route_kernel(const float *__restrict__ logits, int32_t *__restrict__ ids, float *__restrict__ wts, int tokens,
                 int experts, int top_k) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    const float *x = logits + (long)t * experts;
    float m = x[0];
    for (int e = 1; e < experts; ++e) m = fmaxf(m, x[e]);
    int sel[MOE_MAX_K];
    float p[MOE_MAX_K], psum = 0.f;
    for (int j = 0; j < top_k; ++j) {
        int best = -1;
        float bv = 0.f;
        for (int e = 0; e < experts; ++e) {
            bool taken = false;
            for (int i = 0; i < j; ++i) taken |= (sel[i] == e);
            if (taken) continue;
            const float v = x[e];
            if (best < 0 || v > bv) {   // strict: the lowest index wins a tie
                best = e;
                bv = v;
            }
        }
        sel[j] = best;
        p[j] = expf(bv - m);            // softmax numerator; the denominator cancels in the renormalisation
        psum += p[j];
    }
    for (int j = 0; j < top_k; ++j) {
        ids[(long)t * top_k + j] = sel[j];
        wts[(long)t * top_k + j] = p[j] / psum;
    }
}

// Bucket of an expert id: experts [first, first + local) map to buckets 0..local-1, every other expert to the
// extra bucket `local` (expert-parallel ranks keep only their own experts' pairs; the rest sort to the end).
__device__ __forceinline__ int moe_bucket(int e, int first, int local) {
    const int b = e - first;
    return (b >= 0 && b < local) ? b : local;
}

// Single CTA: counts, offsets, stable segmented order and its inverse, over `experts` buckets
// (experts = local, or local + 1 when some ids fall outside [first, first + local)).
// With `tiles`: also the work list of the grouped GEMMs -- one (expert, first row) item per token tile of `tt` rows that
// holds rows of a local expert -- and its length, so that their grids need no slices for tiles that do not exist.
__global__ void __launch_bounds__(1024)
moe_permute_kernel(const int32_t *__restrict__ ids, int pairs, int experts, int first, int local,
                   int32_t *__restrict__ counts, int32_t *__restrict__ offsets, int32_t *__restrict__ sorted_pairs,
                   int32_t *__restrict__ inv, int tt, int2 *__restrict__ tiles, int32_t *__restrict__ ntiles) {
    __shared__ int s_count[MOE_MAX_E];
    __shared__ int s_off[MOE_MAX_E + 1];
    __shared__ int s_run[MOE_MAX_E];          // pairs of each expert placed so far
    __shared__ int s_warp[32][MOE_MAX_E];     // per-warp counts of the current chunk
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    if (tid < experts) s_count[tid] = 0;
    __syncthreads();
    for (int p = tid; p < pairs; p += blockDim.x) atomicAdd(&s_count[moe_bucket(ids[p], first, local)], 1);   // integer counts: order-independent
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int e = 0; e < experts; ++e) {
            s_off[e] = acc;
            acc += s_count[e];
        }
        s_off[experts] = acc;
        if (tiles) {
            int cnt = 0;
            for (int e = 0; e < local; ++e)
                for (int m = s_off[e]; m < s_off[e + 1]; m += tt) tiles[cnt++] = make_int2(e, m);
            *ntiles = cnt;
        }
    }
    if (tid < experts) s_run[tid] = 0;
    __syncthreads();
    if (tid <= experts) offsets[tid] = s_off[tid];
    if (tid < experts) counts[tid] = s_count[tid];
    // chunks of blockDim pairs in pair order; inside a chunk the rank of a pair among those of its expert is
    // (pairs of that expert in lower warps) + (in lower lanes of its warp)
    for (int base = 0; base < pairs; base += blockDim.x) {
        const int p = base + tid;
        const int e = p < pairs ? moe_bucket(ids[p], first, local) : -1;
        int my_rank = 0;
        for (int x = 0; x < experts; ++x) {
            const unsigned mask = __ballot_sync(0xffffffffu, e == x);
            if (lane == 0) s_warp[warp][x] = __popc(mask);
            if (e == x) my_rank = __popc(mask & ((1u << lane) - 1u));
        }
        __syncthreads();
        if (e >= 0) {
            int before = 0;
            for (int w = 0; w < warp; ++w) before += s_warp[w][e];
            const int pos = s_off[e] + s_run[e] + before + my_rank;
            sorted_pairs[pos] = p;
            inv[p] = pos;
        }
        __syncthreads();
        if (tid < experts) {
            int tot = 0;
            for (int w = 0; w < nwarps; ++w) tot += s_warp[w][tid];
            s_run[tid] += tot;
        }
        __syncthreads();
    }
}

// x_perm[i, :] = x[sorted_pairs[i] / k, :]   (16 bytes per thread)
// (rows at and beyond *nrows belong to experts of other ranks and are not gathered)
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __half *__restrict__ x, const int32_t *__restrict__ sorted_pairs, __half *__restrict__ xp,
                  const int32_t *__restrict__ nrows, int hidden, int top_k) {
    const int hv = hidden / 8;
    const int pairs = *nrows;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < (long)pairs * hv; i += (long)gridDim.x * blockDim.x) {
        const int row = (int)(i / hv), c = (int)(i - (long)row * hv);
        const int tok = sorted_pairs[row] / top_k;
        reinterpret_cast<uint4 *>(xp)[(long)row * hv + c] = reinterpret_cast<const uint4 *>(x)[(long)tok * hv + c];
    }
}

// out[t, :] = sum_j w[t, j] * y_perm[inv[t*k + j], :]   (fp32 sum in slot order, fp16 out)
// (pairs whose row is at or beyond *nrows went to experts of other ranks: they add nothing here)
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __half *__restrict__ yp, const int32_t *__restrict__ inv, const float *__restrict__ wts,
                   const int32_t *__restrict__ nrows, __half *__restrict__ out, int tokens, int hidden, int top_k) {
    const int hv = hidden / 8;
    const int rows = *nrows;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < (long)tokens * hv; i += (long)gridDim.x * blockDim.x) {
        const int t = (int)(i / hv), c = (int)(i - (long)t * hv);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < top_k; ++j) {
            const float w = wts[(long)t * top_k + j];
            const int r = inv[(long)t * top_k + j];
            if (r >= rows) continue;
            const uint4 v = reinterpret_cast<const uint4 *>(yp)[(long)r * hv + c];
            const float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y), cc = h2_to_f2(v.z), d = h2_to_f2(v.w);
            acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
            acc[4] += w * cc.x; acc[5] += w * cc.y; acc[6] += w * d.x; acc[7] += w * d.y;
        }
        uint4 o;
        o.x = f2_to_h2(acc[0], acc[1]); o.y = f2_to_h2(acc[2], acc[3]);
        o.z = f2_to_h2(acc[4], acc[5]); o.w = f2_to_h2(acc[6], acc[7]);
        reinterpret_cast<uint4 *>(out)[(long)t * hv + c] = o;
    }
}


// ---------------------------------------------------------------------------------------------------------------
// Expert parallelism by token exchange (dispatch / combine over NVLink peer memory).  Rank r of a group of N holds the
// tokens [r T, (r + 1) T) and the experts [r E/N, (r + 1) E/N).  A call runs three phases on every rank:
//   1. dispatch: route the local tokens; write the hidden row of every (token, choice) pair straight into the receive
//      region of the rank that owns the chosen expert (plain peer stores), and the pair's expert id -- or -1 -- into the
//      id table of every rank; the last CTA to finish publishes "rank r has delivered" on every peer.
//   2. experts: wait (bounded) for every rank's delivery; permute the received pairs by local expert, gather, the two
//      grouped expert GEMMs, and scatter the result rows back to their (source rank, pair) position in this rank's result
//      region; the last CTA publishes "rank r's results are up".
//   3. combine: wait (bounded) for every rank's results; for each local token, load the rows of its k choices from the
//      result regions of the owners (plain peer loads) and add them with the routing weights.
// A pair has a fixed position (source rank, token, choice) in the owner's regions, so no counts or offsets travel.
// Per rank a call moves T k rows out and T k rows in, against (N - 1) T N rows read by the all-reduce form.
// Regions in a rank's exchange buffer: slot 0 = received rows [N T k][H] fp16 followed by the id table [N T k] int32;
// slot 1 = result rows [N T k][H] fp16.  The round counter lives in the buffer and is advanced by phase 3.
// A region is rewritten only after every reader has passed a later barrier: phase 1 of the next call runs behind phase
// 3 of this one, which has seen every rank's phase 2 complete; phase 2 of the next call runs behind its own wait, which
// has seen every rank's next phase 1 and therefore the end of its phase 3.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned *comm_words(unsigned char *buf) { return reinterpret_cast<unsigned *>(buf); }

// All stores of the calling grid to peer memory are complete when the last CTA gets here: it then raises this rank's
// flag (word `flag0 + rank`) on every peer to the current round.
__device__ __forceinline__ void a2a_publish(unsigned char *const *peers, int rank, int world, int flag0, int counter) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned *mine = comm_words(peers[rank]);
        if (atomicAdd(mine + counter, 1u) == gridDim.x * gridDim.y - 1) {
            mine[counter] = 0;
            const unsigned round = *reinterpret_cast<volatile unsigned *>(mine + COMM_W_A2A_ROUND) + 1;
            __threadfence_system();
            for (int r = 0; r < world; ++r) st_release_sys(comm_words(peers[r]) + flag0 + rank, round);
        }
    }
}

// One CTA: waits until every rank's flag (words flag0 .. flag0 + world - 1 of this rank's buffer) has reached the
// current round; gives up after `wait_cycles` and sets the status word.
__global__ void __launch_bounds__(32)
a2a_wait_kernel(unsigned char *const *__restrict__ peers, int rank, int world, int flag0, long long wait_cycles) {
    unsigned *mine = comm_words(peers[rank]);
    const unsigned round = *reinterpret_cast<volatile unsigned *>(mine + COMM_W_A2A_ROUND) + 1;
    if ((int)threadIdx.x < world) {
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(mine + flag0 + threadIdx.x) - round) < 0) {
            if (clock64() - t0 > wait_cycles) {
                atomicExch(mine + COMM_W_STATUS, 1u);
                break;
            }
        }
    }
}

// phase 1: x [T][H], ids [T k] (global expert ids of the local tokens)
__global__ void __launch_bounds__(256)
a2a_dispatch_kernel(unsigned char *const *__restrict__ peers, int rank, int world, const __half *__restrict__ x,
                    const int32_t *__restrict__ ids, int pairs_local, int top_k, int hidden, int experts_per_rank, size_t rows_off,
                    size_t ids_off) {
    const int hv = hidden / 8;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < (long)pairs_local * hv; i += (long)gridDim.x * blockDim.x) {
        const int p = (int)(i / hv), c = (int)(i - (long)p * hv);
        const int e = ids[p], owner = e / experts_per_rank;
        const long slot = (long)rank * pairs_local + p;
        reinterpret_cast<uint4 *>(peers[owner] + rows_off)[slot * hv + c] = reinterpret_cast<const uint4 *>(x)[(long)(p / top_k) * hv + c];
        if (c == 0)
            for (int r = 0; r < world; ++r) reinterpret_cast<int32_t *>(peers[r] + ids_off)[slot] = r == owner ? e : -1;
    }
    a2a_publish(peers, rank, world, COMM_W_A2A_SENT, COMM_W_A2A_COUNT);
}

// phase 2, last step: result[sorted_pairs[row]] = y[row] for the rows of local experts
__global__ void __launch_bounds__(256)
a2a_scatter_kernel(unsigned char *const *__restrict__ peers, int rank, int world, const __half *__restrict__ yp,
                   const int32_t *__restrict__ sorted_pairs, const int32_t *__restrict__ nrows, int hidden, size_t res_off) {
    const int hv = hidden / 8;
    const int rows = *nrows;
    uint4 *res = reinterpret_cast<uint4 *>(peers[rank] + res_off);
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < (long)rows * hv; i += (long)gridDim.x * blockDim.x) {
        const int row = (int)(i / hv), c = (int)(i - (long)row * hv);
        res[(long)sorted_pairs[row] * hv + c] = reinterpret_cast<const uint4 *>(yp)[(long)row * hv + c];
    }
    a2a_publish(peers, rank, world, COMM_W_A2A_DONE, COMM_W_A2A_COUNT + 1);
}

// phase 3: out[t] = sum_j w[t, j] * result_of_owner(ids[t, j])[rank, t, j]   (fp32 sum in choice order, fp16 out)
__global__ void __launch_bounds__(256)
a2a_combine_kernel(unsigned char *const *__restrict__ peers, int rank, const int32_t *__restrict__ ids, const float *__restrict__ wts,
                   __half *__restrict__ out, int tokens, int top_k, int hidden, int experts_per_rank, size_t res_off) {
    const int hv = hidden / 8;
    const long pairs_local = (long)tokens * top_k;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < (long)tokens * hv; i += (long)gridDim.x * blockDim.x) {
        const int t = (int)(i / hv), c = (int)(i - (long)t * hv);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < top_k; ++j) {
            const long p = (long)t * top_k + j;
            const float w = wts[p];
            const int owner = ids[p] / experts_per_rank;
            const uint4 v = reinterpret_cast<const uint4 *>(peers[owner] + res_off)[((long)rank * pairs_local + p) * hv + c];
            const float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y), cc = h2_to_f2(v.z), d = h2_to_f2(v.w);
            acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
            acc[4] += w * cc.x; acc[5] += w * cc.y; acc[6] += w * d.x; acc[7] += w * d.y;
        }
        uint4 o;
        o.x = f2_to_h2(acc[0], acc[1]); o.y = f2_to_h2(acc[2], acc[3]);
        o.z = f2_to_h2(acc[4], acc[5]); o.w = f2_to_h2(acc[6], acc[7]);
        reinterpret_cast<uint4 *>(out)[(long)t * hv + c] = o;
    }
    // the last CTA closes the round
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned *mine = comm_words(peers[rank]);
        __threadfence();
        if (atomicAdd(mine + COMM_W_A2A_COUNT + 2, 1u) == gridDim.x - 1) {
            mine[COMM_W_A2A_COUNT + 2] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned *>(mine + COMM_W_A2A_ROUND) += 1;
        }
    }
}

struct MoeWs {
    int32_t *ids, *counts, *offsets, *sorted_pairs, *inv, *ntiles;
    int2 *tiles;
    float *wts;
    __half *xp, *act, *yp;
    size_t bytes;
};
static MoeWs moe_ws_layout(void *base, int tokens, int hidden, int experts, int top_k, int inter) {
    MoeWs w;
    unsigned char *p = (unsigned char *)base;
    size_t off = 128 * 1024;   // status word and the counter regions of the other kernels stay untouched
    auto take = [&](size_t bytes) {
        unsigned char *r = p + off;
        off += (bytes + 255) / 256 * 256;
        return r;
    };
    const size_t pairs = (size_t)tokens * top_k;
    w.ids = (int32_t *)take(pairs * 4);
    w.wts = (float *)take(pairs * 4);
    w.counts = (int32_t *)take((size_t)experts * 4);
    w.offsets = (int32_t *)take((size_t)(experts + 1) * 4);
    w.sorted_pairs = (int32_t *)take(pairs * 4);
    w.inv = (int32_t *)take(pairs * 4);
    w.ntiles = (int32_t *)take(4);
    w.tiles = (int2 *)take((pairs / 16 + (size_t)experts + 1) * sizeof(int2));     // at most pairs / (smallest tile) + experts items
    w.xp = (__half *)take(pairs * hidden * 2);
    w.act = (__half *)take(pairs * (size_t)inter * 2);
    w.yp = (__half *)take(pairs * hidden * 2);
    w.bytes = off;
    return w;
}

static int grid_for(long work) {
    long blocks = (work + 255) / 256;
    const long cap = (long)sm_count() * 16;
    return (int)(blocks > cap ? cap : blocks);
}

}  // namespace b200k

using namespace b200k;

extern "C" int moe_route_topk_f32(const float *router_logits, int32_t *topk_ids, float *topk_weights, int num_tokens,
                                  int num_experts, int top_k, b200k_stream stream) {
    B200K_REQUIRE(num_tokens >= 0 && num_experts >= 1 && num_experts <= MOE_MAX_E && top_k >= 1 &&
                      top_k <= MOE_MAX_K && top_k <= num_experts,
                  B200K_E_SHAPE, "moe_route_topk_f32: tokens %d, experts %d (<= %d), top_k %d (<= %d)", num_tokens,
                  num_experts, MOE_MAX_E, top_k, MOE_MAX_K);
    if (num_tokens == 0) return 0;
    B200K_REQUIRE(router_logits && topk_ids && topk_weights, B200K_E_NULL, "moe_route_topk_f32: NULL pointer");
    moe_route_kernel<<<ceil_div(num_tokens, 256), 256, 0, to_stream(stream)>>>(router_logits, topk_ids, topk_weights,
                                                                              num_tokens, num_experts, top_k);
    return launch_status("moe_route_topk_f32");
}

extern "C" int moe_permute(const int32_t *topk_ids, int32_t *counts, int32_t *offsets, int32_t *sorted_pairs,
                           int32_t *inverse, int num_pairs, int num_experts, b200k_stream stream) {
    B200K_REQUIRE(num_pairs >= 0 && num_experts >= 1 && num_experts <= MOE_MAX_E, B200K_E_SHAPE,
                  "moe_permute: pairs %d, experts %d (<= %d)", num_pairs, num_experts, MOE_MAX_E);
    B200K_REQUIRE(topk_ids && counts && offsets && sorted_pairs && inverse, B200K_E_NULL, "moe_permute: NULL pointer");
    moe_permute_kernel<<<1, 1024, 0, to_stream(stream)>>>(topk_ids, num_pairs, num_experts, 0, num_experts, counts,
                                                         offsets, sorted_pairs, inverse, 0, nullptr, nullptr);
    return launch_status("moe_permute");
}

extern "C" size_t fused_moe_workspace_bytes(int num_tokens, int hidden, int num_experts, int top_k, int intermediate) {
    if (num_tokens <= 0 || hidden <= 0 || num_experts <= 0 || top_k <= 0 || intermediate <= 0) return 0;
    return moe_ws_layout(nullptr, num_tokens, hidden, num_experts, top_k, intermediate).bytes;
}

// Shared body: experts [expert_first, expert_first + num_local) are the ones whose weights this call holds
// (w13 / w2 stacks of num_local matrices); `out` receives their share of every token's weighted sum.
static int moe_run(const char *name, const b200k_half *x, const float *router_logits, const int32_t *w13_qweight,
                   const b200k_half *w13_scales, const int32_t *w13_qzeros, const int32_t *w2_qweight,
                   const b200k_half *w2_scales, const int32_t *w2_qzeros, b200k_half *out, int num_tokens, int hidden,
                   int num_experts, int expert_first, int num_local, int top_k, int intermediate, int group_size,
                   void *workspace, size_t workspace_bytes, b200k_stream stream) {
    B200K_REQUIRE(x && router_logits && w13_qweight && w13_scales && w2_qweight && w2_scales && out, B200K_E_NULL,
                  "%s: NULL pointer", name);
    B200K_REQUIRE(num_tokens >= 0 && num_experts >= 1 && num_experts <= MOE_MAX_E && top_k >= 1 &&
                      top_k <= MOE_MAX_K && top_k <= num_experts && hidden > 0 && hidden % 64 == 0 &&
                      intermediate > 0 && intermediate % 64 == 0 && group_size >= 64 &&
                      (group_size & (group_size - 1)) == 0 && hidden % group_size == 0 &&
                      intermediate % group_size == 0,
                  B200K_E_SHAPE, "%s: unsupported extents (tokens %d, hidden %d, experts %d, top_k %d, inter %d, group %d)",
                  name, num_tokens, hidden, num_experts, top_k, intermediate, group_size);
    B200K_REQUIRE(expert_first >= 0 && num_local >= 1 && expert_first + num_local <= num_experts, B200K_E_SHAPE,
                  "%s: local experts [%d, %d) outside 0..%d", name, expert_first, expert_first + num_local, num_experts);
    if (num_tokens == 0) return 0;
    if (!workspace) {
        int rc = default_workspace(&workspace, &workspace_bytes);
        if (rc) return rc;
    }
    MoeWs w = moe_ws_layout(workspace, num_tokens, hidden, num_experts, top_k, intermediate);
    B200K_REQUIRE(w.bytes <= workspace_bytes, B200K_E_WORKSPACE, "%s: workspace %zu bytes, need %zu", name,
                  workspace_bytes, w.bytes);
    cudaStream_t st = to_stream(stream);
    const int pairs = num_tokens * top_k;
    const int buckets = num_local == num_experts ? num_local : num_local + 1;
    const int32_t *nrows = w.offsets + num_local;    // rows of the segmented list that belong to local experts
    int rc;
    if ((rc = moe_route_topk_f32(router_logits, w.ids, w.wts, num_tokens, num_experts, top_k, stream))) return rc;
    // the token tile both expert GEMMs will use follows the rows EXPECTED on the local experts; the grids cover the worst case
    const int expected = (int)((long)pairs * num_local / num_experts) > 0 ? (int)((long)pairs * num_local / num_experts) : 1;
    const int tt = gemm_tc_token_tile(expected, num_local);
    const int max_tiles = ceil_div(pairs, tt) + num_local;
    moe_permute_kernel<<<1, 1024, 0, st>>>(w.ids, pairs, buckets, expert_first, num_local, w.counts, w.offsets,
                                           w.sorted_pairs, w.inv, tt, w.tiles, w.ntiles);
    if ((rc = launch_status(name))) return rc;
    moe_gather_kernel<<<grid_for((long)pairs * hidden / 8), 256, 0, st>>>((const __half *)x, w.sorted_pairs, w.xp, nrows,
                                                                          hidden, top_k);
    if ((rc = launch_status(name))) return rc;

    GemmArgs g = {};
    g.format = FMT_GPTQ; g.group = group_size; g.stream = st; g.ws = workspace; g.ws_bytes = workspace_bytes;
    g.seg_offsets = w.offsets; g.num_segments = num_local;
    g.tile_list = w.tiles; g.tile_count = w.ntiles; g.max_tiles = max_tiles; g.expected_m = expected;
    g.s_ak = g.s_qwn = g.s_sn = g.s_qzn = g.s_cn = 1;
    // up-projection with the silu_mul fused into its epilogue: [pairs, H] x W13_e [H, gate I | up I] -> silu(gate) * up [pairs, I]
    g.a = w.xp; g.qweight = w13_qweight; g.scales = (const __half *)w13_scales; g.qzeros = w13_qzeros; g.c = w.act;
    g.m = pairs; g.n = 2 * intermediate; g.k = hidden; g.silu_inter = intermediate;
    g.s_am = hidden; g.s_qwk = g.n; g.s_sk = g.n; g.s_qzk = g.n / 8; g.s_cm = intermediate;
    g.zero_offset = w13_qzeros ? 1 : 0;
    rc = gemm_tc_launch(g);
    if (rc) return rc == TC_NOT_COVERED ? fail(B200K_E_SHAPE, "%s: expert GEMM shape not covered by the tensor-core path", name) : rc;
    g.silu_inter = 0;
    // down-projection: [pairs, I] x W2_e [I, H] -> [pairs, H]
    g.a = w.act; g.qweight = w2_qweight; g.scales = (const __half *)w2_scales; g.qzeros = w2_qzeros; g.c = w.yp;
    g.n = hidden; g.k = intermediate;
    g.s_am = intermediate; g.s_qwk = g.n; g.s_sk = g.n; g.s_qzk = g.n / 8; g.s_cm = g.n;
    g.zero_offset = w2_qzeros ? 1 : 0;
    rc = gemm_tc_launch(g);
    if (rc) return rc == TC_NOT_COVERED ? fail(B200K_E_SHAPE, "%s: expert GEMM shape not covered by the tensor-core path", name) : rc;
    moe_combine_kernel<<<grid_for((long)num_tokens * hidden / 8), 256, 0, st>>>(w.yp, w.inv, w.wts, nrows, (__half *)out,
                                                                                num_tokens, hidden, top_k);
    return launch_status(name);
}

extern "C" int fused_moe_gptq_f16(const b200k_half *x, const float *router_logits, const int32_t *w13_qweight,
                                  const b200k_half *w13_scales, const int32_t *w13_qzeros, const int32_t *w2_qweight,
                                  const b200k_half *w2_scales, const int32_t *w2_qzeros, b200k_half *out,
                                  int num_tokens, int hidden, int num_experts, int top_k, int intermediate,
                                  int group_size, void *workspace, size_t workspace_bytes, b200k_stream stream) {
    return moe_run("fused_moe_gptq_f16", x, router_logits, w13_qweight, w13_scales, w13_qzeros, w2_qweight, w2_scales,
                   w2_qzeros, out, num_tokens, hidden, num_experts, 0, num_experts, top_k, intermediate, group_size,
                   workspace, workspace_bytes, stream);
}

extern "C" int fused_moe_gptq_ep_f16(const b200k_half *x, const float *router_logits, const int32_t *w13_qweight,
                                     const b200k_half *w13_scales, const int32_t *w13_qzeros, const int32_t *w2_qweight,
                                     const b200k_half *w2_scales, const int32_t *w2_qzeros, b200k_half *partial_out,
                                     int num_tokens, int hidden, int num_experts, int expert_first,
                                     int num_local_experts, int top_k, int intermediate, int group_size, void *workspace,
                                     size_t workspace_bytes, b200k_stream stream) {
    return moe_run("fused_moe_gptq_ep_f16", x, router_logits, w13_qweight, w13_scales, w13_qzeros, w2_qweight, w2_scales,
                   w2_qzeros, partial_out, num_tokens, hidden, num_experts, expert_first, num_local_experts, top_k,
                   intermediate, group_size, workspace, workspace_bytes, stream);
}

// Bytes of one slot that fused_moe_gptq_a2a_f16 needs for `tokens_local` tokens per rank in a group of `world`.
extern "C" size_t fused_moe_a2a_slot_bytes(int tokens_local, int hidden, int top_k, int world) {
    const size_t slots = (size_t)world * tokens_local * top_k;
    return (slots * hidden * 2 + 255) / 256 * 256 + slots * 4;
}

extern "C" int fused_moe_gptq_a2a_f16(struct b200k_comm *comm, const b200k_half *x_local, const float *router_logits_local,
                                      const int32_t *w13_qweight, const b200k_half *w13_scales, const int32_t *w13_qzeros,
                                      const int32_t *w2_qweight, const b200k_half *w2_scales, const int32_t *w2_qzeros,
                                      b200k_half *out_local, int tokens_local, int hidden, int num_experts, int top_k,
                                      int intermediate, int group_size, int phases, void *workspace, size_t workspace_bytes,
                                      b200k_stream stream) {
    const char *name = "fused_moe_gptq_a2a_f16";
    B200K_REQUIRE(comm && x_local && router_logits_local && w13_qweight && w13_scales && w2_qweight && w2_scales && out_local,
                  B200K_E_NULL, "%s: NULL pointer", name);
    const CommView cv = comm_view(comm);
    B200K_REQUIRE(cv.mapped, B200K_E_STATE, "%s: a peer buffer is not mapped (b200k_comm_open_peers)", name);
    B200K_REQUIRE(tokens_local >= 1 && num_experts >= 1 && num_experts <= MOE_MAX_E && num_experts % cv.world == 0 && top_k >= 1 &&
                      top_k <= MOE_MAX_K && top_k <= num_experts && hidden > 0 && hidden % 64 == 0 && intermediate > 0 &&
                      intermediate % 64 == 0 && group_size >= 64 && (group_size & (group_size - 1)) == 0 &&
                      hidden % group_size == 0 && intermediate % group_size == 0,
                  B200K_E_SHAPE, "%s: unsupported extents (tokens per rank %d >= 1, hidden %d, experts %d over %d ranks, top_k %d, inter %d, group %d)",
                  name, tokens_local, hidden, num_experts, cv.world, top_k, intermediate, group_size);
    B200K_REQUIRE(phases >= 1 && phases <= 7, B200K_E_SHAPE, "%s: phases %d (bit 0 dispatch, bit 1 experts, bit 2 combine)", name, phases);
    const int world = cv.world, rank = cv.rank, per = num_experts / world;
    const int pairs_local = tokens_local * top_k, slots = world * pairs_local;
    const size_t need = fused_moe_a2a_slot_bytes(tokens_local, hidden, top_k, world);
    B200K_REQUIRE(need <= cv.slot_bytes, B200K_E_WORKSPACE, "%s: the exchange buffer's slots hold %zu bytes, need %zu (fused_moe_a2a_slot_bytes)",
                  name, cv.slot_bytes, need);
    if (!workspace) {
        int rc = default_workspace(&workspace, &workspace_bytes);
        if (rc) return rc;
    }
    // scratch sized for the worst case: every pair of the group lands on this rank
    MoeWs w = moe_ws_layout(workspace, world * tokens_local, hidden, num_experts, top_k, intermediate);
    B200K_REQUIRE(w.bytes <= workspace_bytes, B200K_E_WORKSPACE, "%s: workspace %zu bytes, need %zu", name, workspace_bytes, w.bytes);
    cudaStream_t st = to_stream(stream);
    const size_t rows_off = COMM_FLAGS_BYTES, ids_off = rows_off + ((size_t)slots * hidden * 2 + 255) / 256 * 256;
    const size_t res_off = COMM_FLAGS_BYTES + cv.slot_bytes;
    int rc;
    if (phases & 1) {
        // w.ids / w.wts keep the local tokens' routing until phase 3
        if ((rc = moe_route_topk_f32(router_logits_local, w.ids, w.wts, tokens_local, num_experts, top_k, stream))) return rc;
        a2a_dispatch_kernel<<<grid_for((long)pairs_local * hidden / 8), 256, 0, st>>>(cv.d_peers, rank, world, (const __half *)x_local, w.ids,
                                                                                     pairs_local, top_k, hidden, per, rows_off, ids_off);
        if ((rc = launch_status(name))) return rc;
    }
    if (phases & 2) {
        a2a_wait_kernel<<<1, 32, 0, st>>>(cv.d_peers, rank, world, COMM_W_A2A_SENT, cv.wait_cycles);
        if ((rc = launch_status(name))) return rc;
        const int32_t *recv_ids = reinterpret_cast<const int32_t *>(cv.local + ids_off);
        const __half *recv_rows = reinterpret_cast<const __half *>(cv.local + rows_off);
        const int32_t *nrows = w.offsets + per;
        const int expected = (int)((long)slots * per / num_experts) > 0 ? (int)((long)slots * per / num_experts) : 1;
        const int tt = gemm_tc_token_tile(expected, per);      // planned for the expected rows, grids for the worst case
        const int max_tiles = ceil_div(slots, tt) + per;
        moe_permute_kernel<<<1, 1024, 0, st>>>(recv_ids, slots, per + 1, rank * per, per, w.counts, w.offsets, w.sorted_pairs, w.inv, tt,
                                               w.tiles, w.ntiles);
        if ((rc = launch_status(name))) return rc;
        moe_gather_kernel<<<grid_for((long)slots * hidden / 8), 256, 0, st>>>(recv_rows, w.sorted_pairs, w.xp, nrows, hidden, 1);
        if ((rc = launch_status(name))) return rc;
        GemmArgs g = {};
        g.format = FMT_GPTQ; g.group = group_size; g.stream = st; g.ws = workspace; g.ws_bytes = workspace_bytes;
        g.seg_offsets = w.offsets; g.num_segments = per;
        g.tile_list = w.tiles; g.tile_count = w.ntiles; g.max_tiles = max_tiles; g.expected_m = expected;
        g.s_ak = g.s_qwn = g.s_sn = g.s_qzn = g.s_cn = 1;
        g.a = w.xp; g.qweight = w13_qweight; g.scales = (const __half *)w13_scales; g.qzeros = w13_qzeros; g.c = w.act;
        g.m = slots; g.n = 2 * intermediate; g.k = hidden; g.silu_inter = intermediate;
        g.s_am = hidden; g.s_qwk = g.n; g.s_sk = g.n; g.s_qzk = g.n / 8; g.s_cm = intermediate;
        g.zero_offset = w13_qzeros ? 1 : 0;
        rc = gemm_tc_launch(g);
        if (rc) return rc == TC_NOT_COVERED ? fail(B200K_E_SHAPE, "%s: expert GEMM shape not covered by the tensor-core path", name) : rc;
        g.silu_inter = 0;
        g.a = w.act; g.qweight = w2_qweight; g.scales = (const __half *)w2_scales; g.qzeros = w2_qzeros; g.c = w.yp;
        g.n = hidden; g.k = intermediate;
        g.s_am = intermediate; g.s_qwk = g.n; g.s_sk = g.n; g.s_qzk = g.n / 8; g.s_cm = g.n;
        g.zero_offset = w2_qzeros ? 1 : 0;
        rc = gemm_tc_launch(g);
        if (rc) return rc == TC_NOT_COVERED ? fail(B200K_E_SHAPE, "%s: expert GEMM shape not covered by the tensor-core path", name) : rc;
        a2a_scatter_kernel<<<grid_for((long)slots * hidden / 8), 256, 0, st>>>(cv.d_peers, rank, world, w.yp, w.sorted_pairs, nrows, hidden, res_off);
        if ((rc = launch_status(name))) return rc;
    }
    if (phases & 4) {
        a2a_wait_kernel<<<1, 32, 0, st>>>(cv.d_peers, rank, world, COMM_W_A2A_DONE, cv.wait_cycles);
        if ((rc = launch_status(name))) return rc;
        a2a_combine_kernel<<<grid_for((long)tokens_local * hidden / 8), 256, 0, st>>>(cv.d_peers, rank, w.ids, w.wts, (__half *)out_local,
                                                                                     tokens_local, top_k, hidden, per, res_off);
        if ((rc = launch_status(name))) return rc;
    }
    return 0;
}

// One Llama-shape W4A16 decode layer as a fixed call sequence over the library's own
// entry points, optionally captured in a CUDA graph.  Host-side C++ only; every
// arithmetic step is one of the kernels declared in b200_kernels.h.
#include <stdlib.h>

#include <array>
#include <map>
#include <vector>

#include "gemm.cuh"

namespace b200k {
int rope_kv_append_lens_launch(const __half *qkv, const float *cos_t, const float *sin_t, const int32_t *positions,
                               __half *q_out, __half *kc, __half *vc, int32_t *lens_out, int hq, int hkv, int d,
                               int max_len, int batch, cudaStream_t st);
// peer-to-peer all-reduce (comm.cu): the partial sums sit in slot `slot` of every rank's exchange buffer
int comm_allreduce_f16(struct ::b200k_comm *comm, int slot, __half *out, size_t count, cudaStream_t st);
int comm_allreduce_add_f16(struct ::b200k_comm *comm, int slot, const __half *addend, __half *out, size_t count, cudaStream_t st);
int comm_allreduce_add_rmsnorm_f16(struct ::b200k_comm *comm, int slot, const __half *residual, const __half *w, __half *y,
                                   __half *res_out, int n, float inv_n, float eps, int rows, bool kperm, cudaStream_t st);
__half *comm_slot(struct ::b200k_comm *comm, int slot);
size_t comm_slot_capacity(struct ::b200k_comm *comm);
// producers that write their fp16 output with every 8 values stored as (0,4,1,5,2,6,3,7): the order the GPTQ
// tensor-core GEMM consumes without its byte-permutes (w4a16_gptq_gemm_kperm_f16)
int rms_norm_f16_kperm(const __half *x, const __half *w, __half *y, int n, float inv_n, float eps, int rows, cudaStream_t st);
int fused_add_rms_norm_f16_kperm(const __half *x, const __half *res, const __half *w, __half *y, __half *res_out, int n,
                                 float inv_n, float eps, int rows, cudaStream_t st);
int silu_mul_interleaved_f16_kperm(const __half *gu, __half *out, int inter, int total, cudaStream_t st);
int batched_decode_attention_hm_f16_kperm(const __half *q, const __half *k_cache, const __half *v_cache,
                                          const int32_t *context_lens, __half *output, int batch_size, int num_q_heads,
                                          int num_kv_heads, int head_dim, int max_len, float scale, cudaStream_t st);
}  // namespace b200k

struct b200k_layer {
    b200k_layer_config cfg;
    const int32_t *qw[4];
    const b200k_half *sc[4];
    const int32_t *qz[4];
    const b200k_half *ln1, *ln2;
    const float *cos_t, *sin_t;
    b200k_half *kc, *vc;
    struct b200k_comm *comm;
    // activations (device), sized for max_batch
    b200k_half *x_in, *n1, *qkv, *qrot, *att, *o, *h1, *n2, *gu, *act, *dn, *y_out;
    int32_t *pos, *lens;
    // (batch, input, positions, output, host buffers?) -> captured chain.  The caller's pointers are part of the
    // captured nodes, so a decode loop that reuses its buffers replays one graph with no staging copies.
    std::map<std::array<uintptr_t, 5>, cudaGraphExec_t> graphs;
    cudaStream_t cap_stream;                 // capture happens here: the caller's stream may be the legacy default stream
    int launches;
    bool fused_silu;   // gate_up GEMM with silu(gate) * up in its epilogue (GPTQ weights, tensor-core shapes)
    bool kperm;   // GEMM inputs travel in the pre-permuted order (GPTQ weights, shapes the tensor-core path covers)
};

using namespace b200k;

static int gemm(b200k_layer *L, int which, const b200k_half *a, b200k_half *c, int m, int n, int k,
                b200k_stream st) {
    const int g = L->cfg.group_size;
    if (L->kperm) return w4a16_gptq_gemm_kperm_f16(a, L->qw[which], L->sc[which], L->qz[which], c, m, n, k, g, st);
    if (L->cfg.weight_format == 1)
        return awq_gemm_int4_f16(a, L->qw[which], L->sc[which], L->qz[which], c, m, n, k, g, k, 1, n / 8, 1, n, 1, n / 8,
                                 1, n, 1, st);
    if (!L->qz[which])
        return w4a16_gptq_gemm_sym_f16(a, L->qw[which], L->sc[which], c, m, n, k, g, k, 1, n, 1, n, 1, n, 1, st);
    return w4a16_gptq_gemm_f16(a, L->qw[which], L->sc[which], L->qz[which], c, m, n, k, g, k, 1, n, 1, n, 1, n / 8, 1, n,
                               1, st);
}

// stage 0: hidden -> partial o_proj output
static int stage0(b200k_layer *L, const b200k_half *hidden, const int32_t *positions, b200k_half *o_out, int b,
                  b200k_stream st) {
    const b200k_layer_config &c = L->cfg;
    const int H = c.hidden, hq = c.num_q_heads, hkv = c.num_kv_heads, d = c.head_dim;
    int rc;
    if (L->kperm) rc = rms_norm_f16_kperm((const __half *)hidden, (const __half *)L->ln1, (__half *)L->n1, H, 1.0f / H, c.rms_eps, b, to_stream(st));
    else rc = rms_norm_f16(hidden, L->ln1, L->n1, H, 1.0f / H, c.rms_eps, b, st);
    if (rc) return rc;
    if ((rc = gemm(L, 0, L->n1, L->qkv, b, (hq + 2 * hkv) * d, H, st))) return rc;
    if ((rc = rope_kv_append_lens_launch((const __half *)L->qkv, L->cos_t, L->sin_t, positions, (__half *)L->qrot,
                                         (__half *)L->kc, (__half *)L->vc, L->lens, hq, hkv, d, c.max_len, b,
                                         to_stream(st))))
        return rc;
    if (L->kperm)
        rc = batched_decode_attention_hm_f16_kperm((const __half *)L->qrot, (const __half *)L->kc, (const __half *)L->vc, L->lens,
                                                   (__half *)L->att, b, hq, hkv, d, c.max_len, 1.0f / sqrtf((float)d), to_stream(st));
    else
        rc = batched_decode_attention_hm_f16(L->qrot, L->kc, L->vc, L->lens, L->att, b, hq, hkv, d, c.max_len,
                                             1.0f / sqrtf((float)d), st);
    if (rc) return rc;
    return gemm(L, 1, L->att, o_out, b, H, hq * d, st);
}
// the MLP from the normed activations n2 up to the partial down output
static int mlp(b200k_layer *L, b200k_half *dn_out, int b, b200k_stream st) {
    const b200k_layer_config &c = L->cfg;
    const int H = c.hidden, I = c.intermediate;
    int rc;
    // gate_up GEMM with silu(gate) * up in its epilogue: no [b, 2I] intermediate, one launch fewer.  A single token
    // stays on the two-kernel path, whose GEMM is the M = 1 GEMV.
    rc = L->fused_silu && b > 1 ? gptq_gemm_silu_mul_launch((const __half *)L->n2, L->qw[2], (const __half *)L->sc[2], L->qz[2],
                                                            (__half *)L->act, b, I, H, c.group_size, L->kperm, L->kperm, to_stream(st))
                                : TC_NOT_COVERED;
    if (rc == TC_NOT_COVERED) {
        if ((rc = gemm(L, 2, L->n2, L->gu, b, 2 * I, H, st))) return rc;
        if (L->kperm) rc = silu_mul_interleaved_f16_kperm((const __half *)L->gu, (__half *)L->act, I, b * I, to_stream(st));
        else rc = fused_silu_mul_interleaved_f16(L->gu, L->act, I, b * I, st);
    }
    if (rc) return rc;
    return gemm(L, 3, L->act, dn_out, b, H, I, st);
}
// stage 1: reduced o + hidden -> h1, then the MLP up to the partial down output
static int stage1(b200k_layer *L, const b200k_half *hidden, const b200k_half *o_red, b200k_half *dn_out, int b,
                  b200k_stream st) {
    const b200k_layer_config &c = L->cfg;
    const int H = c.hidden, I = c.intermediate;
    int rc;
    if (L->kperm)
        rc = fused_add_rms_norm_f16_kperm((const __half *)o_red, (const __half *)hidden, (const __half *)L->ln2, (__half *)L->n2,
                                          (__half *)L->h1, H, 1.0f / H, c.rms_eps, b, to_stream(st));
    else
        rc = fused_add_rms_norm_f16(o_red, hidden, L->ln2, L->n2, L->h1, H, 1.0f / H, c.rms_eps, b, st);
    if (rc) return rc;
    return mlp(L, dn_out, b, st);
}
static int stage2(b200k_layer *L, const b200k_half *dn_red, b200k_half *out, int b, b200k_stream st) {
    return residual_add_f16(L->h1, dn_red, out, b * L->cfg.hidden, st);
}

static int chain(b200k_layer *L, const b200k_half *hidden, const int32_t *positions, b200k_half *out, int b,
                 b200k_stream st) {
    int rc;
    const size_t count = (size_t)b * L->cfg.hidden;
    if (!L->comm) {
        if ((rc = stage0(L, hidden, positions, L->o, b, st))) return rc;
        if ((rc = stage1(L, hidden, L->o, L->dn, b, st))) return rc;
        return stage2(L, L->dn, out, b, st);
    }
    // tensor parallel: the row-parallel GEMMs write their partial sums into the exchange buffer the peers can read;
    // each all-reduce is fused with the step that consumes it (residual add + rms_norm after o_proj, the closing
    // residual add after down), so the reduced tensor never makes a round trip through memory: 10 launches
    const b200k_layer_config &c = L->cfg;
    if ((rc = stage0(L, hidden, positions, (b200k_half *)comm_slot(L->comm, 0), b, st))) return rc;
    if ((rc = comm_allreduce_add_rmsnorm_f16(L->comm, 0, (const __half *)hidden, (const __half *)L->ln2, (__half *)L->n2,
                                             (__half *)L->h1, c.hidden, 1.0f / c.hidden, c.rms_eps, b, L->kperm, to_stream(st))))
        return rc;
    if ((rc = mlp(L, (b200k_half *)comm_slot(L->comm, 1), b, st))) return rc;
    (void)count;
    return comm_allreduce_add_f16(L->comm, 1, (const __half *)L->h1, (__half *)out, (size_t)b * c.hidden, to_stream(st));
}

static int check_ready(const b200k_layer *L, int batch, const char *name) {
    B200K_REQUIRE(L, B200K_E_NULL, "%s: layer is NULL", name);
    for (int i = 0; i < 4; ++i)
        B200K_REQUIRE(L->qw[i] && L->sc[i], B200K_E_STATE, "%s: weight %d not set", name, i);
    B200K_REQUIRE(L->ln1 && L->ln2 && L->cos_t && L->sin_t, B200K_E_STATE, "%s: norms / RoPE tables not set", name);
    B200K_REQUIRE(L->kc && L->vc, B200K_E_STATE, "%s: KV cache not set", name);
    B200K_REQUIRE(batch >= 0 && batch <= L->cfg.max_batch, B200K_E_SHAPE, "%s: batch %d outside 0..%d", name, batch,
                  L->cfg.max_batch);
    return 0;
}

extern "C" int b200k_layer_create(const b200k_layer_config *config, b200k_layer **out_layer) {
    B200K_REQUIRE(config && out_layer, B200K_E_NULL, "b200k_layer_create: NULL pointer");
    const b200k_layer_config &c = *config;
    B200K_REQUIRE(c.head_dim == 128, B200K_E_SHAPE, "b200k_layer_create: head_dim %d (128 supported)", c.head_dim);
    B200K_REQUIRE(c.hidden > 0 && c.hidden % 8 == 0 && c.num_q_heads > 0 && c.num_kv_heads > 0 &&
                      c.num_q_heads % c.num_kv_heads == 0 && c.num_q_heads / c.num_kv_heads <= 8 &&
                      c.intermediate > 0 && c.intermediate % 8 == 0 && c.group_size > 0 && c.max_batch > 0 &&
                      c.max_len > 0 && (c.weight_format == 0 || c.weight_format == 1),
                  B200K_E_SHAPE, "b200k_layer_create: unsupported extents");
    B200K_REQUIRE(c.hidden % c.group_size == 0 && (c.num_q_heads * c.head_dim) % c.group_size == 0 &&
                      c.intermediate % c.group_size == 0,
                  B200K_E_SHAPE, "b200k_layer_create: every K extent must be a multiple of group_size %d", c.group_size);
    b200k_layer *L = new b200k_layer();
    L->cfg = c;
    const size_t B = c.max_batch, H = c.hidden, NQ = (size_t)(c.num_q_heads + 2 * c.num_kv_heads) * c.head_dim;
    const size_t QD = (size_t)c.num_q_heads * c.head_dim, I = c.intermediate;
    struct { b200k_half **p; size_t n; } bufs[] = {
        {&L->x_in, B * H}, {&L->n1, B * H}, {&L->qkv, B * NQ}, {&L->qrot, B * QD}, {&L->att, B * QD}, {&L->o, B * H},
        {&L->h1, B * H}, {&L->n2, B * H}, {&L->gu, B * 2 * I}, {&L->act, B * I}, {&L->dn, B * H}, {&L->y_out, B * H}};
    size_t total = 0;
    for (auto &b : bufs) total += (b.n * 2 + 255) / 256 * 256;
    total += 2 * ((B * 4 + 255) / 256 * 256);
    unsigned char *base = nullptr;
    cudaError_t e = cudaMalloc(&base, total);
    if (e != cudaSuccess) {
        cudaGetLastError();
        delete L;
        return fail((int)e, "b200k_layer_create: cudaMalloc of %zu bytes: %s", total, cudaGetErrorString(e));
    }
    size_t off = 0;
    for (auto &b : bufs) {
        *b.p = (b200k_half *)(base + off);
        off += (b.n * 2 + 255) / 256 * 256;
    }
    L->pos = (int32_t *)(base + off);
    off += (B * 4 + 255) / 256 * 256;
    L->lens = (int32_t *)(base + off);
    // rms_norm, gemm, rope+append, attention, gemm, add+norm, gemm (+ silu in its epilogue, or a silu kernel), gemm, add
    // The fused form is off unless B200K_LAYER_FUSED_SILU=1: at 64 tokens its GEMM (two 64-column boxes per tensor, the up
    // half exchanged through shared memory in the epilogue) costs 10 us more than the plain one, the launch it saves 3 us.
    L->fused_silu = c.weight_format == 0 && env_char("B200K_LAYER_FUSED_SILU") == '1' && c.group_size >= 64 &&
                    (c.group_size & (c.group_size - 1)) == 0 && c.hidden % 64 == 0 && c.intermediate % 64 == 0;
    L->launches = L->fused_silu ? 9 : 10;
    {
        // Pre-permuted GEMM inputs: GPTQ weights and extents the tensor-core GEMM family covers for all four projections
        // (K a multiple of 64, group a power of two >= 64, N a multiple of 32).  B200K_LAYER_KPERM=0 turns it off.
        const int g = c.group_size, qd = c.num_q_heads * c.head_dim, nq = (c.num_q_heads + 2 * c.num_kv_heads) * c.head_dim;
        L->kperm = c.weight_format == 0 && env_char("B200K_LAYER_KPERM") != '0' && g >= 64 && (g & (g - 1)) == 0 && c.hidden % 64 == 0 &&
                   qd % 64 == 0 && c.intermediate % 64 == 0 && c.hidden % 32 == 0 && nq % 32 == 0 && (2 * c.intermediate) % 32 == 0;
    }
    *out_layer = L;
    return 0;
}

extern "C" void b200k_layer_destroy(b200k_layer *L) {
    if (!L) return;
    for (auto &kv : L->graphs)
        if (kv.second) cudaGraphExecDestroy(kv.second);
    if (L->cap_stream) cudaStreamDestroy(L->cap_stream);
    cudaFree(L->x_in);  // base of the single allocation
    delete L;
}

static void drop_graphs(b200k_layer *L) {
    for (auto &kv : L->graphs)
        if (kv.second) cudaGraphExecDestroy(kv.second);
    L->graphs.clear();
}

extern "C" int b200k_layer_set_weight(b200k_layer *L, int which, const int32_t *qweight, const b200k_half *scales,
                                      const int32_t *qzeros) {
    B200K_REQUIRE(L && qweight && scales, B200K_E_NULL, "b200k_layer_set_weight: NULL pointer");
    B200K_REQUIRE(which >= 0 && which < 4, B200K_E_SHAPE, "b200k_layer_set_weight: which = %d", which);
    B200K_REQUIRE(L->cfg.weight_format == 0 || qzeros, B200K_E_NULL, "b200k_layer_set_weight: AWQ needs qzeros");
    L->qw[which] = qweight; L->sc[which] = scales; L->qz[which] = qzeros;
    drop_graphs(L);
    return 0;
}
extern "C" int b200k_layer_set_norms_rope(b200k_layer *L, const b200k_half *ln1, const b200k_half *ln2,
                                          const float *cos_table, const float *sin_table) {
    B200K_REQUIRE(L && ln1 && ln2 && cos_table && sin_table, B200K_E_NULL, "b200k_layer_set_norms_rope: NULL pointer");
    L->ln1 = ln1; L->ln2 = ln2; L->cos_t = cos_table; L->sin_t = sin_table;
    drop_graphs(L);
    return 0;
}
extern "C" int b200k_layer_set_kv_cache(b200k_layer *L, b200k_half *k_cache, b200k_half *v_cache) {
    B200K_REQUIRE(L && k_cache && v_cache, B200K_E_NULL, "b200k_layer_set_kv_cache: NULL pointer");
    L->kc = k_cache; L->vc = v_cache;
    drop_graphs(L);
    return 0;
}
extern "C" int b200k_layer_set_comm(b200k_layer *L, struct b200k_comm *comm) {
    B200K_REQUIRE(L, B200K_E_NULL, "b200k_layer_set_comm: layer is NULL");
    B200K_REQUIRE(!comm || comm_slot_capacity(comm) >= (size_t)L->cfg.max_batch * L->cfg.hidden * 2, B200K_E_SHAPE,
                  "b200k_layer_set_comm: exchange slots of %zu bytes are smaller than max_batch x hidden fp16 (%zu bytes)",
                  comm_slot_capacity(comm), (size_t)L->cfg.max_batch * L->cfg.hidden * 2);
    L->comm = comm;
    drop_graphs(L);
    return 0;
}
extern "C" int b200k_layer_launches_per_forward(const b200k_layer *L) {
    return L ? L->launches : 0;      // tensor parallel: the two all-reduces replace the add + norm and the closing add
}

// The whole call as it would be issued eagerly: for host buffers the copies in and out around the chain.
static int issue(b200k_layer *L, const b200k_half *hidden_in, const int32_t *positions, b200k_half *hidden_out, int batch,
                 bool host, b200k_stream stream) {
    if (!host) return chain(L, hidden_in, positions, hidden_out, batch, stream);
    cudaStream_t st = to_stream(stream);
    const size_t hb = (size_t)batch * L->cfg.hidden * 2;
    cudaError_t e = cudaMemcpyAsync(L->x_in, hidden_in, hb, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(L->pos, positions, (size_t)batch * 4, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail((int)e, "layer: copy in: %s", cudaGetErrorString(e));
    int rc = chain(L, L->x_in, L->pos, L->y_out, batch, stream);
    if (rc) return rc;
    e = cudaMemcpyAsync(hidden_out, L->y_out, hb, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return fail((int)e, "layer: copy out: %s", cudaGetErrorString(e));
    return 0;
}

constexpr size_t MAX_GRAPHS = 64;   // distinct (batch, buffers) combinations kept; beyond that calls run eagerly

// Runs one call, through a captured graph when enabled.  The first call with a given batch and set of
// buffers runs eagerly (first-use set-up such as the default workspace and function attributes must not
// happen inside a capture) and captures the same sequence for the calls that follow.
static int run(b200k_layer *L, const b200k_half *hidden_in, const int32_t *positions, b200k_half *hidden_out, int batch,
               bool host, b200k_stream stream) {
    if (!L->cfg.use_graph) return issue(L, hidden_in, positions, hidden_out, batch, host, stream);
    const std::array<uintptr_t, 5> key = {(uintptr_t)batch, (uintptr_t)hidden_in, (uintptr_t)positions, (uintptr_t)hidden_out,
                                          (uintptr_t)host};
    auto it = L->graphs.find(key);
    if (it != L->graphs.end()) {
        if (!it->second) return issue(L, hidden_in, positions, hidden_out, batch, host, stream);   // capture was not possible
        cudaError_t e = cudaGraphLaunch(it->second, to_stream(stream));
        if (e != cudaSuccess) return fail((int)e, "layer: graph launch: %s", cudaGetErrorString(e));
        return 0;
    }
    int rc = issue(L, hidden_in, positions, hidden_out, batch, host, stream);
    if (rc || L->graphs.size() >= MAX_GRAPHS) return rc;
    cudaGraph_t graph = nullptr;
    cudaError_t e;
    if (!L->cap_stream) {
        e = cudaStreamCreateWithFlags(&L->cap_stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) return fail((int)e, "layer: stream create: %s", cudaGetErrorString(e));
    }
    e = cudaStreamBeginCapture(L->cap_stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) return fail((int)e, "layer: begin capture: %s", cudaGetErrorString(e));
    rc = issue(L, hidden_in, positions, hidden_out, batch, host, (b200k_stream)L->cap_stream);
    e = cudaStreamEndCapture(L->cap_stream, &graph);
    if (rc || e != cudaSuccess) {
        // e.g. copies from pageable host memory cannot be captured: this set of buffers stays eager
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        L->graphs[key] = nullptr;
        return 0;   // the eager pass above already produced this call's result
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return fail((int)e, "layer: graph instantiate: %s", cudaGetErrorString(e));
    L->graphs[key] = exec;
    return 0;   // the eager pass above already produced this call's result
}

extern "C" int b200k_layer_forward(b200k_layer *L, const b200k_half *hidden_in, const int32_t *positions,
                                   b200k_half *hidden_out, int batch, b200k_stream stream) {
    int rc = check_ready(L, batch, "b200k_layer_forward");
    if (rc) return rc;
    B200K_REQUIRE(hidden_in && positions && hidden_out, B200K_E_NULL, "b200k_layer_forward: NULL pointer");
    if (batch == 0) return 0;
    return run(L, hidden_in, positions, hidden_out, batch, false, stream);
}

extern "C" int b200k_layer_forward_host(b200k_layer *L, const b200k_half *host_hidden_in,
                                        const int32_t *host_positions, b200k_half *host_hidden_out, int batch,
                                        b200k_stream stream) {
    int rc = check_ready(L, batch, "b200k_layer_forward_host");
    if (rc) return rc;
    B200K_REQUIRE(host_hidden_in && host_positions && host_hidden_out, B200K_E_NULL,
                  "b200k_layer_forward_host: NULL pointer");
    if (batch == 0) return 0;
    return run(L, host_hidden_in, host_positions, host_hidden_out, batch, true, stream);
}

extern "C" int b200k_layer_forward_stage(b200k_layer *L, int stage, const b200k_half *hidden_in,
                                         const int32_t *positions, const b200k_half *reduced_in,
                                         b200k_half *partial_out, b200k_half *hidden_out, int batch,
                                         b200k_stream stream) {
    int rc = check_ready(L, batch, "b200k_layer_forward_stage");
    if (rc) return rc;
    if (batch == 0) return 0;
    switch (stage) {
        case 0:
            B200K_REQUIRE(hidden_in && positions && partial_out, B200K_E_NULL, "b200k_layer_forward_stage 0: NULL pointer");
            return stage0(L, hidden_in, positions, partial_out, batch, stream);
        case 1:
            B200K_REQUIRE(hidden_in && reduced_in && partial_out, B200K_E_NULL, "b200k_layer_forward_stage 1: NULL pointer");
            return stage1(L, hidden_in, reduced_in, partial_out, batch, stream);
        case 2:
            B200K_REQUIRE(reduced_in && hidden_out, B200K_E_NULL, "b200k_layer_forward_stage 2: NULL pointer");
            return stage2(L, reduced_in, hidden_out, batch, stream);
    }
    return fail(B200K_E_SHAPE, "b200k_layer_forward_stage: stage %d", stage);
}

extern "C" int b200k_device_status(int *host_status_out, b200k_stream stream) {
    B200K_REQUIRE(host_status_out, B200K_E_NULL, "b200k_device_status: NULL pointer");
    void *ws = nullptr;
    size_t bytes = 0;
    int rc = default_workspace(&ws, &bytes);
    if (rc) return rc;
    cudaError_t e = cudaMemcpyAsync(host_status_out, ws, sizeof(int), cudaMemcpyDeviceToHost, to_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(to_stream(stream));
    if (e != cudaSuccess) return fail((int)e, "b200k_device_status: %s", cudaGetErrorString(e));
    return 0;
}

extern "C" int b200k_device_clear_status(b200k_stream stream) {
    void *ws = nullptr;
    size_t bytes = 0;
    int rc = default_workspace(&ws, &bytes);
    if (rc) return rc;
    return b200k_workspace_clear_status(ws, stream);
}

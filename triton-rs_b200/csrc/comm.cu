// One-shot all-reduce over NVLink peer memory for the two row-parallel GEMMs of a
// tensor-parallel decode layer (messages of a few hundred KiB, latency-bound).
//
// Every rank owns one device buffer: [flags | slot 0 | slot 1].  The buffers are exchanged as CUDA IPC
// handles by the host code (one process per GPU) and mapped by every peer.  A row-parallel GEMM writes
// its partial sums straight into a slot of its own buffer; the all-reduce kernel then
//   1. publishes "my slot is complete" by storing a sequence number into its flag on every peer
//      (system-scope release store),
//   2. waits -- bounded, ~1 s, reporting through a status word -- until every peer's flag carries the
//      same sequence number,
//   3. sums the slot of all ranks in rank order with plain peer loads (nothing is reduced inside the switch),
//      fp32 accumulate, and writes the fp16 result to a local buffer.  Every rank computes the same
//      bits.
// The sequence number lives in device memory and is advanced by the kernel, so a CUDA graph that
// contains the call can be replayed.  Slots alternate between the two all-reduces of a layer; a slot is
// rewritten only after a later all-reduce has passed its barrier, i.e. after every peer finished
// reading it.  The consumers of a layer's exchanges are fused into the same kernel (residual add; residual add +
// rms_norm), and large tensors take a two-shot form (allreduce_twoshot_kernel).
#include "comm.cuh"

struct b200k_comm {
    int rank, world;
    size_t slot_bytes;
    unsigned char *local;          // this rank's buffer (cudaMalloc)
    unsigned char *peer[8];        // mapped buffers, peer[rank] == local
    bool opened[8];
    unsigned char **d_peers;       // device copy of peer[]
    long long wait_cycles;         // SM clock cycles a kernel waits for its peers before it gives up
};

namespace b200k {

// (layout of the flags page: comm.cuh)
constexpr int COMM_MAX_WORLD = 8;
constexpr long long COMM_DEFAULT_WAIT_CYCLES = 2000000000LL;   // about a second of SM clock

__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t h22(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// Entry protocol shared by the all-reduce kernels: publish "my slot holds round `seq`" to every peer (CTA 0), wait --
// bounded -- until every peer has published the same round.  Returns false when a peer never arrived (status word set).
__device__ __forceinline__ bool exchange_enter(unsigned char *const *peers, int rank, int world, long long wait_cycles,
                                               unsigned &seq, int *s_fail) {
    unsigned *my_flags = reinterpret_cast<unsigned *>(peers[rank]);
    unsigned *seq_p = my_flags + 16, *status_p = my_flags + 18;
    seq = *reinterpret_cast<volatile unsigned *>(seq_p) + 1;   // advanced by the last CTA of the round before
    if (threadIdx.x == 0) *s_fail = 0;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x < world) {
        // the GEMM that filled my slot ran earlier on this stream: its stores are ordered before this thread by the kernel
        // boundary, and the release store orders them before the flag (a system fence in front of it cost 2-3 us more)
        st_release_sys(reinterpret_cast<unsigned *>(peers[threadIdx.x]) + rank, seq);
    }
    if (threadIdx.x < world) {
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(my_flags + threadIdx.x) - seq) < 0) {
            if (clock64() - t0 > wait_cycles) {   // a peer never arrived: report, do not spin for ever
                *s_fail = 1;
                atomicExch(status_p, 1u);
                break;
            }
        }
    }
    __syncthreads();
    return *s_fail == 0;
}
// Exit protocol: the last CTA of the grid to get here advances the round counter (kept in device memory, so a CUDA
// graph that contains the call can be replayed).
__device__ __forceinline__ void exchange_leave(unsigned char *const *peers, int rank, unsigned seq) {
    unsigned *my_flags = reinterpret_cast<unsigned *>(peers[rank]);
    unsigned *seq_p = my_flags + 16, *done_p = my_flags + 17;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done_p, 1u) == gridDim.x - 1) {
            *done_p = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned *>(seq_p) = seq;
        }
    }
}

// Sum over the ranks, in rank order, of 8 fp16 values at byte offset `off` of every rank's buffer: fp32 accumulate.
// Every rank's chunk is requested before any is used: the loads cross NVLink (microseconds each), and issued one behind
// the other's use they would serialise -- eight round trips per chunk at eight ranks instead of one.
__device__ __forceinline__ void peer_sum8(unsigned char *const *peers, int world, size_t off, float (&acc)[8]) {
    uint4 v[COMM_MAX_WORLD];
#pragma unroll
    for (int r = 0; r < COMM_MAX_WORLD; ++r)
        if (r < world) v[r] = *reinterpret_cast<const uint4 *>(peers[r] + off);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int r = 0; r < COMM_MAX_WORLD; ++r) {
        if (r < world) {
            const float2 a = h2_to_f2(v[r].x), b = h2_to_f2(v[r].y), c = h2_to_f2(v[r].z), d = h2_to_f2(v[r].w);
            acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
            acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
        }
    }
}

// out = all-reduce(slot)                         (addend == nullptr)
// out = addend + fp16(all-reduce(slot))          (the closing residual add of a layer, fused: the sum is rounded to
//                                                 fp16 first, as a separate all-reduce would have stored it)
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(unsigned char *const *__restrict__ peers, int rank, int world, int slot, size_t slot_bytes,
                         const __half *__restrict__ addend, __half *__restrict__ out, size_t count, long long wait_cycles) {
    pdl_wait();                 // the partial sums in my slot come from the kernel before
    pdl_launch_dependents();
    __shared__ int s_fail;
    unsigned seq;
    if (exchange_enter(peers, rank, world, wait_cycles, seq, &s_fail)) {
        const size_t nvec = count / 8;                          // 16-byte chunks
        const size_t off = COMM_FLAGS_BYTES + (size_t)slot * slot_bytes;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
            float acc[8];
            peer_sum8(peers, world, off + i * 16, acc);
            uint4 o;
            o.x = f2_to_h2(acc[0], acc[1]); o.y = f2_to_h2(acc[2], acc[3]);
            o.z = f2_to_h2(acc[4], acc[5]); o.w = f2_to_h2(acc[6], acc[7]);
            if (addend) {
                const uint4 h = reinterpret_cast<const uint4 *>(addend)[i];
                o.x = h22(__hadd2(u2h(h.x), u2h(o.x))); o.y = h22(__hadd2(u2h(h.y), u2h(o.y)));
                o.z = h22(__hadd2(u2h(h.z), u2h(o.z))); o.w = h22(__hadd2(u2h(h.w), u2h(o.w)));
            }
            reinterpret_cast<uint4 *>(out)[i] = o;
        }
    }
    exchange_leave(peers, rank, seq);
}

// Two-shot form for large tensors.  Rank r sums the r-th share of the vectors over all ranks (the same rank-order fp32
// sum, one rounding) and stores the fp16 result into the OTHER slot of every rank; after a second round of flags every
// rank copies that slot out.  One-shot makes every rank read (world - 1) x count over NVLink; here a rank reads
// (world - 1) / world x count and writes as much.  The other slot is free for the duration: between the entry barrier of
// this call (every rank has left the call before it) and the next call on it (slots are used alternately) nobody reads it.
// The CTAs of a grid wait on one another through the peers (the last CTA through its share publishes this rank's flag),
// so the whole grid must be resident: at most 128 CTAs.
__global__ void __launch_bounds__(512)
allreduce_twoshot_kernel(unsigned char *const *__restrict__ peers, int rank, int world, int slot, size_t slot_bytes,
                         const __half *__restrict__ addend, __half *__restrict__ out, size_t count, long long wait_cycles) {
    pdl_wait();                 // the partial sums in my slot come from the kernel before
    pdl_launch_dependents();
    __shared__ int s_fail;
    unsigned seq;
    unsigned *my_flags = reinterpret_cast<unsigned *>(peers[rank]);
    const bool entered = exchange_enter(peers, rank, world, wait_cycles, seq, &s_fail);
    const size_t nvec = count / 8;                          // 16-byte chunks
    const size_t off_in = COMM_FLAGS_BYTES + (size_t)slot * slot_bytes, off_res = COMM_FLAGS_BYTES + (size_t)(slot ^ 1) * slot_bytes;
    if (entered) {
        const size_t share = (nvec + world - 1) / world;
        const size_t lo = (size_t)rank * share < nvec ? (size_t)rank * share : nvec, hi = lo + share < nvec ? lo + share : nvec;
        for (size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (size_t)gridDim.x * blockDim.x) {
            float acc[8];
            peer_sum8(peers, world, off_in + i * 16, acc);
            uint4 o;
            o.x = f2_to_h2(acc[0], acc[1]); o.y = f2_to_h2(acc[2], acc[3]);
            o.z = f2_to_h2(acc[4], acc[5]); o.w = f2_to_h2(acc[6], acc[7]);
#pragma unroll
            for (int r = 0; r < COMM_MAX_WORLD; ++r)
                if (r < world) *reinterpret_cast<uint4 *>(peers[r] + off_res + i * 16) = o;
        }
    }
    // second round: this rank's share is in every rank's result slot once all CTAs of the grid are through
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(my_flags + COMM_W_AR2_COUNT, 1u) == gridDim.x - 1) {
            my_flags[COMM_W_AR2_COUNT] = 0;
            __threadfence_system();
            for (int r = 0; r < world; ++r) st_release_sys(reinterpret_cast<unsigned *>(peers[r]) + COMM_W_AR2 + rank, seq);
        }
    }
    if (entered && threadIdx.x < world) {
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(my_flags + COMM_W_AR2 + threadIdx.x) - seq) < 0) {
            if (clock64() - t0 > wait_cycles) {   // a peer never delivered: report, do not spin for ever
                s_fail = 1;
                atomicExch(my_flags + COMM_W_STATUS, 1u);
                break;
            }
        }
    }
    __syncthreads();
    if (entered && !s_fail) {
        const uint4 *res = reinterpret_cast<const uint4 *>(peers[rank] + off_res);
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
            uint4 o = res[i];
            if (addend) {
                const uint4 h = reinterpret_cast<const uint4 *>(addend)[i];
                o.x = h22(__hadd2(u2h(h.x), u2h(o.x))); o.y = h22(__hadd2(u2h(h.y), u2h(o.y)));
                o.z = h22(__hadd2(u2h(h.z), u2h(o.z))); o.w = h22(__hadd2(u2h(h.w), u2h(o.w)));
            }
            reinterpret_cast<uint4 *>(out)[i] = o;
        }
    }
    exchange_leave(peers, rank, seq);
}

// all-reduce(slot) + residual add + rms_norm in one pass, one CTA per row of n values (the step after o_proj of a
// tensor-parallel layer): r = residual + fp16(sum over ranks); residual_out = fp16(r); y = r * rsqrt(mean(r^2) + eps) * w
// from the unrounded fp32 r, the arithmetic of fused_add_rms_norm_f16.  KPERM stores every 8 outputs of y as
// (0,4,1,5,2,6,3,7), the order the int4 GEMM that follows consumes.
template <bool KPERM>
__global__ void __launch_bounds__(1024)
allreduce_add_rmsnorm_kernel(unsigned char *const *__restrict__ peers, int rank, int world, int slot, size_t slot_bytes,
                             const __half *__restrict__ residual, const __half *__restrict__ w, __half *__restrict__ y,
                             __half *__restrict__ res_out, int n, float inv_n, float eps, long long wait_cycles) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ int s_fail;
    __shared__ float red[32];
    unsigned seq;
    if (exchange_enter(peers, rank, world, wait_cycles, seq, &s_fail)) {
        constexpr int ITERS = 4;
        const int nv = n / 8;
        const size_t row = (size_t)blockIdx.x * n;
        const size_t off = COMM_FLAGS_BYTES + (size_t)slot * slot_bytes + row * 2;
        float v[ITERS][8];
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int i = threadIdx.x + it * blockDim.x;
            if (i < nv) {
                float acc[8];
                peer_sum8(peers, world, off + (size_t)i * 16, acc);
                const uint4 h = *reinterpret_cast<const uint4 *>(residual + row + (size_t)i * 8);
                const float2 a = h2_to_f2(h.x), b = h2_to_f2(h.y), c = h2_to_f2(h.z), d = h2_to_f2(h.w);
                const float x[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[it][j] = x[j] + __half2float(__float2half_rn(acc[j]));   // the reduced value is an fp16 tensor
                    ss += v[it][j] * v[it][j];
                }
                uint4 o;
                o.x = f2_to_h2(v[it][0], v[it][1]); o.y = f2_to_h2(v[it][2], v[it][3]);
                o.z = f2_to_h2(v[it][4], v[it][5]); o.w = f2_to_h2(v[it][6], v[it][7]);
                *reinterpret_cast<uint4 *>(res_out + row + (size_t)i * 8) = o;
            }
        }
        const float inv = rsqrtf(block_sum(ss, red) * inv_n + eps);
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int i = threadIdx.x + it * blockDim.x;
            if (i < nv) {
                const uint4 wv = *reinterpret_cast<const uint4 *>(w + (size_t)i * 8);
                const float2 a = h2_to_f2(wv.x), b = h2_to_f2(wv.y), c = h2_to_f2(wv.z), d = h2_to_f2(wv.w);
                const float ww[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[it][j] * inv * ww[j];
                uint4 u;
                if (KPERM) {
                    u.x = f2_to_h2(o[0], o[4]); u.y = f2_to_h2(o[1], o[5]); u.z = f2_to_h2(o[2], o[6]); u.w = f2_to_h2(o[3], o[7]);
                } else {
                    u.x = f2_to_h2(o[0], o[1]); u.y = f2_to_h2(o[2], o[3]); u.z = f2_to_h2(o[4], o[5]); u.w = f2_to_h2(o[6], o[7]);
                }
                *reinterpret_cast<uint4 *>(y + row + (size_t)i * 8) = u;
            }
        }
    }
    exchange_leave(peers, rank, seq);
}

int comm_allreduce_add_f16(struct ::b200k_comm *c, int slot, const __half *addend, __half *out, size_t count, cudaStream_t st);
int comm_allreduce_f16(struct ::b200k_comm *c, int slot, __half *out, size_t count, cudaStream_t st) {
    return comm_allreduce_add_f16(c, slot, nullptr, out, count, st);
}

int comm_allreduce_add_rmsnorm_f16(struct ::b200k_comm *c, int slot, const __half *residual, const __half *w, __half *y,
                                   __half *res_out, int n, float inv_n, float eps, int rows, bool kperm, cudaStream_t st) {
    B200K_REQUIRE(c && residual && w && y && res_out, B200K_E_NULL, "all-reduce + add + rms_norm: NULL pointer");
    B200K_REQUIRE(slot == 0 || slot == 1, B200K_E_SHAPE, "all-reduce + add + rms_norm: slot %d", slot);
    B200K_REQUIRE(n > 0 && n % 8 == 0 && n / 8 <= 4096 && rows >= 0 && (size_t)rows * n * 2 <= c->slot_bytes, B200K_E_SHAPE,
                  "all-reduce + add + rms_norm: %d rows of %d (a multiple of 8, at most 32768) do not fit a slot of %zu bytes",
                  rows, n, c->slot_bytes);
    B200K_REQUIRE(aligned16(residual) && aligned16(w) && aligned16(y) && aligned16(res_out), B200K_E_ALIGN,
                  "all-reduce + add + rms_norm: pointers must be 16-byte aligned");
    for (int r = 0; r < c->world; ++r)
        B200K_REQUIRE(c->peer[r], B200K_E_STATE, "all-reduce: peer %d is not mapped (b200k_comm_open_peers)", r);
    if (rows == 0) return 0;
    const int nv = n / 8;
    const int threads = nv <= 128 ? 128 : (nv <= 256 ? 256 : (nv <= 512 ? 512 : 1024));
    if (kperm)
        launch_kernel(allreduce_add_rmsnorm_kernel<true>, dim3(rows), dim3(threads), 0, st, c->d_peers, c->rank, c->world, slot,
                      c->slot_bytes, residual, w, y, res_out, n, inv_n, eps, c->wait_cycles);
    else
        launch_kernel(allreduce_add_rmsnorm_kernel<false>, dim3(rows), dim3(threads), 0, st, c->d_peers, c->rank, c->world, slot,
                      c->slot_bytes, residual, w, y, res_out, n, inv_n, eps, c->wait_cycles);
    return launch_status("all-reduce + add + rms_norm (peer to peer)");
}

int comm_allreduce_add_f16(struct ::b200k_comm *c, int slot, const __half *addend, __half *out, size_t count, cudaStream_t st) {
    B200K_REQUIRE(c && out, B200K_E_NULL, "all-reduce: NULL pointer");
    B200K_REQUIRE(slot == 0 || slot == 1, B200K_E_SHAPE, "all-reduce: slot %d", slot);
    B200K_REQUIRE(count % 8 == 0 && count * 2 <= c->slot_bytes, B200K_E_SHAPE,
                  "all-reduce: %zu elements do not fit a slot of %zu bytes (or are not a multiple of 8)", count, c->slot_bytes);
    for (int r = 0; r < c->world; ++r)
        B200K_REQUIRE(c->peer[r], B200K_E_STATE, "all-reduce: peer %d is not mapped (b200k_comm_open_peers)", r);
    if (count == 0) return 0;
    int blocks = (int)((count / 8 + 511) / 512);
    if (blocks > 128) blocks = 128;
    // Two-shot when what it saves on the wire outweighs its second round (remote stores fenced, flags, copy-out: measured
    // 14 us at four ranks and 512 KB, where the one-shot form takes 14.6 us in all): one-shot moves (world - 1) x bytes into
    // every rank, two-shot 2 (world - 1) / world x bytes, at ~700 GB/s
    const double saved_bytes = (double)count * 2 * (c->world - 1) * (1.0 - 2.0 / c->world);
    bool two_shot = c->world >= 3 && saved_bytes > 10e6;
    if (const int v = env_char("B200K_COMM_TWOSHOT")) two_shot = v == '1';      // tuning / test override
    if (two_shot)
        launch_kernel(allreduce_twoshot_kernel, dim3(blocks), dim3(512), 0, st, c->d_peers, c->rank, c->world, slot, c->slot_bytes, addend, out, count, c->wait_cycles);
    else
        launch_kernel(allreduce_oneshot_kernel, dim3(blocks), dim3(512), 0, st, c->d_peers, c->rank, c->world, slot, c->slot_bytes, addend, out, count, c->wait_cycles);
    return launch_status("all-reduce (peer to peer)");
}

__half *comm_slot(struct ::b200k_comm *c, int slot) {
    return reinterpret_cast<__half *>(c->local + COMM_FLAGS_BYTES + (size_t)slot * c->slot_bytes);
}

size_t comm_slot_capacity(struct ::b200k_comm *c) { return c ? c->slot_bytes : 0; }

CommView comm_view(struct ::b200k_comm *c) {
    CommView v = {};
    if (!c) return v;
    v.d_peers = c->d_peers; v.local = c->local; v.rank = c->rank; v.world = c->world;
    v.slot_bytes = c->slot_bytes; v.wait_cycles = c->wait_cycles;
    v.mapped = true;
    for (int r = 0; r < c->world; ++r) v.mapped = v.mapped && c->peer[r] != nullptr;
    return v;
}

}  // namespace b200k

using namespace b200k;

static int upload_peers(struct b200k_comm *comm, const char *name);

extern "C" int b200k_comm_create(int rank, int world, size_t slot_bytes, struct b200k_comm **out_comm) {
    B200K_REQUIRE(out_comm, B200K_E_NULL, "b200k_comm_create: NULL pointer");
    B200K_REQUIRE(world >= 1 && world <= COMM_MAX_WORLD && rank >= 0 && rank < world && slot_bytes > 0, B200K_E_SHAPE,
                  "b200k_comm_create: rank %d, world %d (<= %d), slot_bytes %zu", rank, world, COMM_MAX_WORLD, slot_bytes);
    b200k_comm *c = new b200k_comm();
    c->rank = rank; c->world = world;
    c->wait_cycles = COMM_DEFAULT_WAIT_CYCLES;
    c->slot_bytes = (slot_bytes + 255) / 256 * 256;
    const size_t total = COMM_FLAGS_BYTES + 2 * c->slot_bytes;
    cudaError_t e = cudaMalloc(&c->local, total);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, total);
    if (e == cudaSuccess) e = cudaMalloc(&c->d_peers, sizeof(unsigned char *) * COMM_MAX_WORLD);
    if (e != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return fail((int)e, "b200k_comm_create: %s", cudaGetErrorString(e));
    }
    c->peer[rank] = c->local;
    *out_comm = c;
    return 0;
}

extern "C" int b200k_comm_ipc_handle(struct b200k_comm *comm, void *host_handle_64_bytes) {
    B200K_REQUIRE(comm && host_handle_64_bytes, B200K_E_NULL, "b200k_comm_ipc_handle: NULL pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaError_t e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(host_handle_64_bytes), comm->local);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail((int)e, "b200k_comm_ipc_handle: %s", cudaGetErrorString(e));
    }
    return 0;
}

extern "C" int b200k_comm_open_peers(struct b200k_comm *comm, const void *host_all_handles) {
    B200K_REQUIRE(comm && host_all_handles, B200K_E_NULL, "b200k_comm_open_peers: NULL pointer");
    const cudaIpcMemHandle_t *h = reinterpret_cast<const cudaIpcMemHandle_t *>(host_all_handles);
    for (int r = 0; r < comm->world; ++r) {
        if (r == comm->rank || comm->peer[r]) continue;
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h[r], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail((int)e, "b200k_comm_open_peers: rank %d cannot map the buffer of rank %d: %s", comm->rank, r,
                        cudaGetErrorString(e));
        }
        comm->peer[r] = (unsigned char *)p;
        comm->opened[r] = true;
    }
    return upload_peers(comm, "b200k_comm_open_peers");
}

static int upload_peers(struct b200k_comm *comm, const char *name) {
    cudaError_t e = cudaMemcpy(comm->d_peers, comm->peer, sizeof(unsigned char *) * COMM_MAX_WORLD, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail((int)e, "%s: %s", name, cudaGetErrorString(e));
    return 0;
}

extern "C" int b200k_comm_buffer(struct b200k_comm *comm, void **host_out_ptr) {
    B200K_REQUIRE(comm && host_out_ptr, B200K_E_NULL, "b200k_comm_buffer: NULL pointer");
    *host_out_ptr = comm->local;
    return 0;
}

extern "C" int b200k_comm_set_peer_pointer(struct b200k_comm *comm, int peer_rank, void *peer_buffer) {
    B200K_REQUIRE(comm && peer_buffer, B200K_E_NULL, "b200k_comm_set_peer_pointer: NULL pointer");
    B200K_REQUIRE(peer_rank >= 0 && peer_rank < comm->world && peer_rank != comm->rank, B200K_E_SHAPE,
                  "b200k_comm_set_peer_pointer: peer rank %d (world %d, own rank %d)", peer_rank, comm->world, comm->rank);
    if (comm->opened[peer_rank]) {
        cudaIpcCloseMemHandle(comm->peer[peer_rank]);
        comm->opened[peer_rank] = false;
    }
    comm->peer[peer_rank] = (unsigned char *)peer_buffer;
    return upload_peers(comm, "b200k_comm_set_peer_pointer");
}

extern "C" int b200k_comm_set_timeout_cycles(struct b200k_comm *comm, int64_t cycles) {
    B200K_REQUIRE(comm, B200K_E_NULL, "b200k_comm_set_timeout_cycles: NULL pointer");
    comm->wait_cycles = cycles > 0 ? (long long)cycles : COMM_DEFAULT_WAIT_CYCLES;
    return 0;
}

extern "C" int b200k_comm_clear_status(struct b200k_comm *comm, b200k_stream stream) {
    B200K_REQUIRE(comm, B200K_E_NULL, "b200k_comm_clear_status: NULL pointer");
    cudaError_t e = cudaMemsetAsync(comm->local + 72, 0, sizeof(int), to_stream(stream));
    if (e != cudaSuccess) return fail((int)e, "b200k_comm_clear_status: %s", cudaGetErrorString(e));
    return 0;
}

extern "C" int b200k_comm_allreduce_f16(struct b200k_comm *comm, int slot, const b200k_half *input, b200k_half *output,
                                        size_t count, b200k_stream stream) {
    B200K_REQUIRE(comm && output, B200K_E_NULL, "b200k_comm_allreduce_f16: NULL pointer");
    B200K_REQUIRE(slot == 0 || slot == 1, B200K_E_SHAPE, "b200k_comm_allreduce_f16: slot %d", slot);
    B200K_REQUIRE(count * 2 <= comm->slot_bytes, B200K_E_SHAPE, "b200k_comm_allreduce_f16: %zu elements exceed the slot", count);
    if (input) {   // stage a caller buffer into the slot; NULL = the data is already there (b200k_comm_slot)
        cudaError_t e = cudaMemcpyAsync(comm_slot(comm, slot), input, count * 2, cudaMemcpyDeviceToDevice, to_stream(stream));
        if (e != cudaSuccess) return fail((int)e, "b200k_comm_allreduce_f16: %s", cudaGetErrorString(e));
    }
    return comm_allreduce_f16(comm, slot, (__half *)output, count, to_stream(stream));
}

static int stage_input(struct b200k_comm *comm, int slot, const b200k_half *input, size_t count, b200k_stream stream, const char *name) {
    B200K_REQUIRE(comm, B200K_E_NULL, "%s: NULL pointer", name);
    B200K_REQUIRE(slot == 0 || slot == 1, B200K_E_SHAPE, "%s: slot %d", name, slot);
    B200K_REQUIRE(count * 2 <= comm->slot_bytes, B200K_E_SHAPE, "%s: %zu elements exceed the slot", name, count);
    if (input) {
        cudaError_t e = cudaMemcpyAsync(comm_slot(comm, slot), input, count * 2, cudaMemcpyDeviceToDevice, to_stream(stream));
        if (e != cudaSuccess) return fail((int)e, "%s: %s", name, cudaGetErrorString(e));
    }
    return 0;
}

extern "C" int b200k_comm_allreduce_add_f16(struct b200k_comm *comm, int slot, const b200k_half *input, const b200k_half *addend,
                                            b200k_half *output, size_t count, b200k_stream stream) {
    B200K_REQUIRE(addend && output, B200K_E_NULL, "b200k_comm_allreduce_add_f16: NULL pointer");
    int rc = stage_input(comm, slot, input, count, stream, "b200k_comm_allreduce_add_f16");
    if (rc) return rc;
    return comm_allreduce_add_f16(comm, slot, (const __half *)addend, (__half *)output, count, to_stream(stream));
}

extern "C" int b200k_comm_allreduce_add_rms_norm_f16(struct b200k_comm *comm, int slot, const b200k_half *input,
                                                     const b200k_half *residual, const b200k_half *weight, b200k_half *output,
                                                     b200k_half *residual_out, int hidden_size, float inv_n, float eps,
                                                     int num_rows, b200k_stream stream) {
    B200K_REQUIRE(hidden_size > 0 && num_rows >= 0, B200K_E_SHAPE, "b200k_comm_allreduce_add_rms_norm_f16: %d rows of %d", num_rows, hidden_size);
    int rc = stage_input(comm, slot, input, (size_t)num_rows * hidden_size, stream, "b200k_comm_allreduce_add_rms_norm_f16");
    if (rc) return rc;
    return comm_allreduce_add_rmsnorm_f16(comm, slot, (const __half *)residual, (const __half *)weight, (__half *)output,
                                          (__half *)residual_out, hidden_size, inv_n, eps, num_rows, false, to_stream(stream));
}

extern "C" int b200k_comm_slot(struct b200k_comm *comm, int slot, b200k_half **out_ptr) {
    B200K_REQUIRE(comm && out_ptr, B200K_E_NULL, "b200k_comm_slot: NULL pointer");
    B200K_REQUIRE(slot == 0 || slot == 1, B200K_E_SHAPE, "b200k_comm_slot: slot %d", slot);
    *out_ptr = (b200k_half *)comm_slot(comm, slot);
    return 0;
}

extern "C" int b200k_comm_status(struct b200k_comm *comm, int *host_status_out, b200k_stream stream) {
    B200K_REQUIRE(comm && host_status_out, B200K_E_NULL, "b200k_comm_status: NULL pointer");
    cudaError_t e = cudaMemcpyAsync(host_status_out, comm->local + 72, sizeof(int), cudaMemcpyDeviceToHost, to_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(to_stream(stream));
    if (e != cudaSuccess) return fail((int)e, "b200k_comm_status: %s", cudaGetErrorString(e));
    return 0;
}

extern "C" void b200k_comm_destroy(struct b200k_comm *comm) {
    if (!comm) return;
    for (int r = 0; r < comm->world; ++r)
        if (comm->opened[r]) cudaIpcCloseMemHandle(comm->peer[r]);
    cudaFree(comm->d_peers);
    cudaFree(comm->local);
    delete comm;
}

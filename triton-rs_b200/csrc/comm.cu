// One-shot all-reduce over NVLink peer memory for the two row-parallel GEMMs of a
// tensor-parallel decode layer (messages of a few hundred KiB, latency-bound).
//
// Every rank owns one device buffer: [flags | slot 0 | slot 1].  The buffers are exchanged as CUDA IPC
// handles by the host code (one process per GPU) and mapped by every peer.  A row-parallel GEMM writes
// its partial sums straight into a slot of its own buffer; the all-reduce kernel then
//   1. publishes "my slot is complete" by storing a sequence number into its flag on every peer
//      (system-scope release after a system fence),
//   2. waits -- bounded, ~1 s, reporting through a status word -- until every peer's flag carries the
//      same sequence number,
//   3. sums the slot of all ranks in rank order with plain peer loads (nothing is reduced inside the switch),
//      fp32 accumulate, and writes the fp16 result to a local buffer.  Every rank computes the same
//      bits.
// The sequence number lives in device memory and is advanced by the kernel, so a CUDA graph that
// contains the call can be replayed.  Slots alternate between the two all-reduces of a layer; a slot is
// rewritten only after a later all-reduce has passed its barrier, i.e. after every peer finished
// reading it.
#include "common.cuh"

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

constexpr size_t COMM_FLAGS_BYTES = 4096;   // [0,32): flags (one per peer, written by that peer); [64]: sequence; [68]: done counter; [72]: status
constexpr int COMM_MAX_WORLD = 8;
constexpr long long COMM_DEFAULT_WAIT_CYCLES = 2000000000LL;   // about a second of SM clock

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(unsigned char *const *__restrict__ peers, int rank, int world, int slot, size_t slot_bytes,
                         __half *__restrict__ out, size_t count, long long wait_cycles) {
    pdl_wait();                 // the partial sums in my slot come from the kernel before
    pdl_launch_dependents();
    unsigned char *mine = peers[rank];
    unsigned *my_flags = reinterpret_cast<unsigned *>(mine);
    unsigned *seq_p = my_flags + 16, *done_p = my_flags + 17, *status_p = my_flags + 18;
    __shared__ int s_fail;
    const unsigned seq = *reinterpret_cast<volatile unsigned *>(seq_p) + 1;   // advanced by the last CTA to finish
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x < world) {
        __threadfence_system();   // the GEMM that filled my slot ran earlier on this stream
        st_release_sys(reinterpret_cast<unsigned *>(peers[threadIdx.x]) + rank, seq);
    }
    if (threadIdx.x < world) {
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(my_flags + threadIdx.x) - seq) < 0) {
            if (clock64() - t0 > wait_cycles) {   // a peer never arrived: report, do not spin for ever
                s_fail = 1;
                atomicExch(status_p, 1u);
                break;
            }
        }
    }
    __syncthreads();
    if (!s_fail) {
        const size_t nvec = count / 8;                          // 16-byte chunks
        const size_t off = COMM_FLAGS_BYTES + (size_t)slot * slot_bytes;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < world; ++r) {
                const uint4 v = reinterpret_cast<const uint4 *>(peers[r] + off)[i];
                const float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y), c = h2_to_f2(v.z), d = h2_to_f2(v.w);
                acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
                acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
            }
            uint4 o;
            o.x = f2_to_h2(acc[0], acc[1]); o.y = f2_to_h2(acc[2], acc[3]);
            o.z = f2_to_h2(acc[4], acc[5]); o.w = f2_to_h2(acc[6], acc[7]);
            reinterpret_cast<uint4 *>(out)[i] = o;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done_p, 1u) == gridDim.x - 1) {   // last CTA of this call
            *done_p = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned *>(seq_p) = seq;
        }
    }
}

int comm_allreduce_f16(struct ::b200k_comm *c, int slot, __half *out, size_t count, cudaStream_t st) {
    B200K_REQUIRE(c && out, B200K_E_NULL, "all-reduce: NULL pointer");
    B200K_REQUIRE(slot == 0 || slot == 1, B200K_E_SHAPE, "all-reduce: slot %d", slot);
    B200K_REQUIRE(count % 8 == 0 && count * 2 <= c->slot_bytes, B200K_E_SHAPE,
                  "all-reduce: %zu elements do not fit a slot of %zu bytes (or are not a multiple of 8)", count, c->slot_bytes);
    for (int r = 0; r < c->world; ++r)
        B200K_REQUIRE(c->peer[r], B200K_E_STATE, "all-reduce: peer %d is not mapped (b200k_comm_open_peers)", r);
    if (count == 0) return 0;
    int blocks = (int)((count / 8 + 511) / 512);
    if (blocks > 32) blocks = 32;
    launch_kernel(allreduce_oneshot_kernel, dim3(blocks), dim3(512), 0, st, c->d_peers, c->rank, c->world, slot, c->slot_bytes, out, count, c->wait_cycles);
    return launch_status("all-reduce (peer to peer)");
}

__half *comm_slot(struct ::b200k_comm *c, int slot) {
    return reinterpret_cast<__half *>(c->local + COMM_FLAGS_BYTES + (size_t)slot * c->slot_bytes);
}

size_t comm_slot_capacity(struct ::b200k_comm *c) { return c ? c->slot_bytes : 0; }

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

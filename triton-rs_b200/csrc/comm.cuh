// What other translation units may know about a tensor-parallel exchange buffer (comm.cu owns it).
#pragma once
#include "common.cuh"

struct b200k_comm;

namespace b200k {

constexpr size_t COMM_FLAGS_BYTES = 4096;
// Words of the flags page, [0, 4096) of every rank's buffer (unsigned, index = byte offset / 4):
//   [0, 8)   all-reduce flags, one per peer, written by that peer      [16] all-reduce round   [17] its done counter
//   [18]     status word (any bounded wait that gave up)
//   [20, 28) two-shot all-reduce: "rank r has delivered its share" flags   [28] its done counter
//   [32, 40) token exchange: "rank r has delivered its tokens" flags   [40, 48) "rank r has published its results" flags
//   [48]     token-exchange round   [49], [50], [51] done counters of its three phases
constexpr int COMM_W_AR2 = 20, COMM_W_AR2_COUNT = 28;
constexpr int COMM_W_STATUS = 18, COMM_W_A2A_SENT = 32, COMM_W_A2A_DONE = 40, COMM_W_A2A_ROUND = 48, COMM_W_A2A_COUNT = 49;

struct CommView {
    unsigned char *const *d_peers;   // device array of the ranks' buffers (this rank's own included)
    unsigned char *local;
    int rank, world;
    size_t slot_bytes;
    long long wait_cycles;
    bool mapped;                     // every peer's buffer is mapped
};
CommView comm_view(struct ::b200k_comm *c);

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

}  // namespace b200k

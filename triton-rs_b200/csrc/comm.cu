// Peer-to-peer all-reduce over NVLink for the two row-parallel GEMMs of a tensor-parallel
// layer.  Placeholder: reports that no communicator is available.
#include "common.cuh"
namespace b200k {
int comm_allreduce_f16(struct ::b200k_comm *, __half *, size_t, cudaStream_t) {
    return fail(B200K_E_STATE, "peer-to-peer all-reduce is not built yet");
}
}  // namespace b200k

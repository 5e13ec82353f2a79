// Placeholder until the tcgen05 grouped-GEMM path lands: reports "not supported" so every
// shape takes the weight-streaming path.
#include "common.cuh"

namespace smoe {
struct PrefillArgs;
bool prefill_supported(int, uint32_t, uint32_t) { return false; }
size_t prefill_scratch_bytes(uint32_t, uint32_t) { return 0; }
int launch_prefill(const PrefillArgs&, cudaStream_t, cudaEvent_t) { return -1; }
}  // namespace smoe

// placeholder, replaced below
#include "device_plan.hpp"
namespace cutespmm {
bool brick_supports(uint32_t, uint64_t, uint64_t, const void *, const void *) { return false; }
cudaError_t launch_brick(const BrickArgs &, int, cudaStream_t) { return cudaErrorNotSupported; }
}

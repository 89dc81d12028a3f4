// Prefill SGMV tiles for tall segments (placeholder until the tcgen05 kernel lands).
#include "lora_common.cuh"

namespace b200lora {

bool sgmv_tiles_supported(const ApplyParams&) { return false; }

cudaError_t launch_sgmv_tiles(const ApplyParams&, int, int, cudaStream_t) { return cudaSuccess; }

}  // namespace b200lora

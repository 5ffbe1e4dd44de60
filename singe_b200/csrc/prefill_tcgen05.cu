// placeholder until the tcgen05 prefill kernel lands
#include "common.cuh"
namespace singe {
bool prefill_fast_path(size_t, size_t, size_t, const void *, const void *, const void *, const void *) { return false; }
int prefill_tcgen05_bf16(cudaStream_t, void *, float *, const void *, const void *, const void *, const int32_t *,
                         const int32_t *, const int32_t *, size_t, size_t, size_t, size_t, size_t, size_t, int, float) {
    return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
}
}  // namespace singe

// Process-wide runtime state of the library: the sticky device error word kernels report internal
// failures to (a bounded wait that ran out), and the debug entry point that reads and clears it.
#include "common.cuh"

namespace singe {

__device__ uint32_t g_device_error = 0;

uint32_t *device_error_word() {
    constexpr int kMaxDevices = 64;
    static uint32_t *words[kMaxDevices] = {nullptr};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        return nullptr;
    }
    if (words[device] == nullptr) {
        void *address = nullptr;
        if (cudaGetSymbolAddress(&address, g_device_error) != cudaSuccess) {
            return nullptr;
        }
        words[device] = static_cast<uint32_t *>(address);
    }
    return words[device];
}

}  // namespace singe

extern "C" {

// Reads and clears the sticky device error word of the current device (synchronises the device).
// 0 = no kernel-side failure since the last call.
int singe_debug_take_device_error(uint32_t *value) {
    SINGE_CUDA_TRY(cudaDeviceSynchronize());
    uint32_t *word = singe::device_error_word();
    if (word == nullptr) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    uint32_t host = 0;
    SINGE_CUDA_TRY(cudaMemcpy(&host, word, sizeof(host), cudaMemcpyDeviceToHost));
    SINGE_CUDA_TRY(cudaMemset(word, 0, sizeof(host)));
    if (value != nullptr) *value = host;
    return SINGE_OK;
}

}  // extern "C"

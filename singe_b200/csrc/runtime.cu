// Process-wide runtime state of the library: the sticky device error word kernels report internal
// failures to (a bounded wait that ran out), and the entry point that reads and clears it.
#include "common.cuh"

namespace singe {

__device__ uint32_t g_device_error = 0;

uint32_t *device_error_word() {
    static uint32_t *words[kMaxDevices] = {nullptr};
    const int device = device_slot();
    if (device < 0) return nullptr;
    if (words[device] == nullptr) {
        void *address = nullptr;
        if (cudaGetSymbolAddress(&address, g_device_error) != cudaSuccess) {
            return nullptr;
        }
        words[device] = static_cast<uint32_t *>(address);
    }
    return words[device];
}

namespace {
thread_local WarmRange g_pending_warm = {nullptr, 0};
}

WarmRange take_pending_warm() {
    const WarmRange taken = g_pending_warm;
    g_pending_warm = {nullptr, 0};
    return taken;
}

}  // namespace singe

extern "C" {

// Attaches [pointer, pointer + bytes) to the next kernel this host thread enqueues through the library: that kernel
// pulls the range into L2 beside its own work.  See WarmRange in common.cuh.
int singe_warm_l2_with_next_launch(const void *pointer, size_t bytes) {
    if (pointer == nullptr && bytes != 0) return SINGE_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(pointer) & 15u) != 0) return SINGE_ERR_INVALID_ARGUMENT;
    singe::g_pending_warm = {pointer, static_cast<unsigned long long>(bytes)};
    return SINGE_OK;
}

// Reads and clears the sticky device error word of the current device (synchronises the device).
// 0 = no kernel-side failure since the last call.
int singe_take_device_error(uint32_t *value) {
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

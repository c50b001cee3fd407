// Library-wide entry points: version, error text, device check, status word.
#include <atomic>

#include "host_common.h"

namespace i8f {

static thread_local char t_error[512] = {0};
static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
char* error_buffer() { return t_error; }

// One status word per device; kernels receive its address as an argument.
__device__ int g_status_word;

static constexpr int kMaxDevices = 64;
static int* s_status_addr[kMaxDevices] = {nullptr};

int* device_status_word() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (s_status_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        s_status_addr[dev] = static_cast<int*>(p);
    }
    return s_status_addr[dev];
}

}  // namespace i8f

extern "C" {

int i8f_version(void) { return I8F_VERSION; }

uint64_t i8f_launch_count(void) { return i8f::g_launches.load(std::memory_order_relaxed); }

const char* i8f_last_error(void) { return i8f::error_buffer(); }

int i8f_device_check(void) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return i8f::fail(I8F_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    int major = 0, minor = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (major != 10 || minor != 0)
        return i8f::fail(I8F_ERR_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev, major, minor);
    return I8F_OK;
}

int i8f_device_status(int* status_out, int reset) {
    I8F_REQUIRE(status_out != nullptr, I8F_ERR_INVALID_ARG, "status_out is NULL");
    int* w = i8f::device_status_word();
    I8F_REQUIRE(w != nullptr, I8F_ERR_CUDA, "status word unavailable on this device");
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return i8f::fail(I8F_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    e = cudaMemcpy(status_out, w, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return i8f::fail(I8F_ERR_CUDA, "cudaMemcpy: %s", cudaGetErrorString(e));
    if (reset) {
        e = cudaMemset(w, 0, sizeof(int));
        if (e != cudaSuccess) return i8f::fail(I8F_ERR_CUDA, "cudaMemset: %s", cudaGetErrorString(e));
    }
    return I8F_OK;
}

}  // extern "C"

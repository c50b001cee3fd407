// i8f_linear_forward_static: the whole quantised-linear forward for callers
// that are not able to hand over (or allocate) a workspace.
//
// Who needs this: code that runs where device allocation is off limits -- a
// host application that has given the whole device to its own memory pool, a
// real-time loop that must not touch the allocator, a plugin sandbox whose
// only CUDA rights are "launch on this stream".  i8f_linear_forward needs a
// caller-owned workspace for the int8 activations and their scales; here that
// workspace is a fixed array that is part of the library image, so the call
// allocates nothing: no cudaMalloc / cudaFree, no pool, no library routine
// that allocates behind the scenes.
//
// Consequences the caller has to know (also stated in include/i8f.h):
//   * Every GPU that uses this entry point holds the array
//     (I8F_STATIC_WORKSPACE_BYTES) until the process exits.  The driver backs
//     it with device memory when this module is first touched on a device --
//     with lazy module loading that is the first call here, which can
//     therefore fail with I8F_ERR_CUDA on a GPU with nothing left; make it
//     before the rest of the device is handed to a pool.
//   * Problems whose workspace does not fit are refused with
//     I8F_ERR_WORKSPACE; nothing is launched.
//   * All calls on a device share the one array.  Calls that can overlap on
//     the GPU (different streams, no ordering between them) race on it; keep
//     such calls on one stream or order them with events.
//   * The array keeps whatever the previous call left in it.  Nothing in it
//     has to start at zero: each call first overwrites every int8 row and
//     every scale it later reads.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress).  Make that first call outside any stream
//     capture.
#include "host_common.h"

namespace i8f {
namespace {

// In host code this name is only a handle for the runtime's symbol table, not
// a device address: it must never be passed to a kernel as is.
static __device__ __align__(256) unsigned char g_static_workspace[I8F_STATIC_WORKSPACE_BYTES];

constexpr int kMaxDevices = 64;
// Written without a lock: two host threads that race on a device's first call both look the address up and store
// the same value, so the unsynchronised write is idempotent.
unsigned char* s_workspace_addr[kMaxDevices] = {nullptr};

// Device address of the array on the CURRENT device (looked up once per device).
int static_workspace(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    I8F_REQUIRE(dev >= 0 && dev < kMaxDevices, I8F_ERR_UNSUPPORTED, "device index %d out of range", dev);
    if (s_workspace_addr[dev] == nullptr) {
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_workspace);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(I8F_ERR_CUDA, "cudaGetSymbolAddress(static workspace): %s", cudaGetErrorString(e));
        s_workspace_addr[dev] = ptr;
    }
    *out = s_workspace_addr[dev];
    return I8F_OK;
}

}  // namespace
}  // namespace i8f

using namespace i8f;

extern "C" int i8f_linear_forward_static(const void* x, int x_dtype, int64_t ldx, int hadamard128, const int8_t* w,
                                         int64_t ldw, const float* w_scale, int w_scale_mode, const void* bias,
                                         int bias_dtype, void* out, int out_dtype, int64_t ldo, int64_t M, int64_t N,
                                         int64_t K, int epilogue_order, void* stream) {
    I8F_REQUIRE(M > 0 && N > 0 && K > 0, I8F_ERR_INVALID_ARG, "empty problem");
    I8F_REQUIRE(K % 16 == 0, I8F_ERR_ALIGNMENT, "K=%lld must be a multiple of 16", (long long)K);
    // refuse before anything is enqueued; M * K is checked in a way that cannot overflow
    I8F_REQUIRE(M <= static_cast<int64_t>(I8F_STATIC_WORKSPACE_BYTES) / K, I8F_ERR_WORKSPACE,
                "M*K = %lld x %lld does not fit the built-in %zu-byte workspace; use i8f_linear_forward with your own",
                (long long)M, (long long)K, static_cast<size_t>(I8F_STATIC_WORKSPACE_BYTES));
    const size_t need = i8f_linear_workspace_bytes(M, K);
    I8F_REQUIRE(need <= static_cast<size_t>(I8F_STATIC_WORKSPACE_BYTES), I8F_ERR_WORKSPACE,
                "this problem needs %zu bytes of workspace, the built-in one has %zu; use i8f_linear_forward with your own",
                need, static_cast<size_t>(I8F_STATIC_WORKSPACE_BYTES));
    unsigned char* ws = nullptr;
    int rc = static_workspace(&ws);
    if (rc != I8F_OK) return rc;
    // same split of the workspace as i8f_linear_forward: int8 rows first, then the scales
    int8_t* q = reinterpret_cast<int8_t*>(ws);
    float* xs = reinterpret_cast<float*>(ws + ((static_cast<size_t>(M) * static_cast<size_t>(K) + 255) & ~size_t(255)));
    rc = i8f_quant_rowwise(x, x_dtype, M, K, ldx, q, K, xs, hadamard128, nullptr, stream);
    if (rc != I8F_OK) return rc;
    return i8f_linear_w8a8(q, K, xs, w, ldw, w_scale, w_scale_mode, bias, bias_dtype, out, out_dtype, ldo, M, N, K,
                           epilogue_order, stream);
}

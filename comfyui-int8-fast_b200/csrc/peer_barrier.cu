// Meeting point of the ranks of a column-parallel linear (one process per GPU), as a kernel on the caller's stream.
//
// Every rank owns an array of `n_ranks` 32-bit flags that its peers can write (symmetric memory or any other
// peer mapping).  To meet at `epoch`, rank r stores `epoch` into slot r of EVERY rank's array (plain system-scope
// stores over NVLink, preceded by a system fence so that everything this stream wrote before -- including the
// epilogue stores of a GEMM into peer buffers -- is visible first), then waits until all slots of its OWN array
// have reached `epoch`.  Only local memory is polled; nothing is loaded from a peer.  Epochs grow monotonically
// (compared modulo 2^32), so the flags never have to be cleared between meetings.
//
// The wait is bounded: when a peer does not arrive within `limit_cycles` SM clocks the kernel records
// kStPeerWait in the device status word and returns, so a rank that failed on the host leaves the others with
// an error to read instead of a GPU that spins until the process is killed.
#include "host_common.h"

namespace i8f {
namespace {

constexpr int kMaxRanks = 8;
enum : int { kStPeerWait = 105 };

struct PeerFlags {
    uint32_t* p[kMaxRanks];
};

__global__ void peer_barrier_kernel(const PeerFlags flags, int n_ranks, int rank, uint32_t epoch, long long limit_cycles,
                                    int* status) {
    const int peer = threadIdx.x;
    if (peer >= n_ranks) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[peer] + rank), "r"(epoch) : "memory");
    const uint32_t* mine = flags.p[rank] + peer;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if (static_cast<int32_t>(seen - epoch) >= 0) break;
        if ((it & 15u) == 0u && clock64() - t0 > limit_cycles) {
            atomicCAS(status, 0, kStPeerWait);
            break;
        }
        __nanosleep(64);
    }
    __threadfence_system();
}

}  // namespace
}  // namespace i8f

using namespace i8f;

extern "C" int i8f_peer_barrier(void* const* flag_arrays, int n_ranks, int rank, uint32_t epoch, int64_t limit_cycles,
                                void* stream) {
    I8F_REQUIRE(flag_arrays != nullptr && n_ranks >= 1 && n_ranks <= kMaxRanks, I8F_ERR_INVALID_ARG,
                "n_ranks must be 1..%d", kMaxRanks);
    I8F_REQUIRE(rank >= 0 && rank < n_ranks, I8F_ERR_INVALID_ARG, "rank %d out of range", rank);
    I8F_REQUIRE(limit_cycles > 0 && limit_cycles <= 20000000000LL, I8F_ERR_INVALID_ARG, "limit_cycles out of range");
    PeerFlags f{};
    for (int i = 0; i < n_ranks; ++i) {
        I8F_REQUIRE(flag_arrays[i] != nullptr && (reinterpret_cast<uintptr_t>(flag_arrays[i]) & 3u) == 0, I8F_ERR_ALIGNMENT,
                    "flag array %d is NULL or not 4-byte aligned", i);
        f.p[i] = static_cast<uint32_t*>(flag_arrays[i]);
    }
    int* status = device_status_word();
    I8F_REQUIRE(status != nullptr, I8F_ERR_CUDA, "device status word unavailable");
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, n_ranks, rank, epoch, limit_cycles, status);
    return check_launch("peer_barrier_kernel");
}

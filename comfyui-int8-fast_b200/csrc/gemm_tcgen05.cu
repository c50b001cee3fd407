// C[M,N] = A[M,K] * B[N,K]^T on the sm_100a tensor cores (tcgen05.mma), with
// both operands K-major in global memory, staged by TMA into a shared-memory
// ring, accumulated in tensor memory and drained by a fused epilogue.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0 (one lane)  TMA producer: fills ring stages, signals `full`
//   warp 1 (one lane)  MMA issuer:   4 x tcgen05.mma per stage (32 bytes of K
//                                    each), tcgen05.commit frees the stage
//                                    (`empty`) and publishes a finished tile
//                                    (`acc_full`)
//   warps 2..5         epilogue:     tcgen05.ld the 128 x BN accumulator (one
//                                    row per thread), dequantise / cast, store,
//                                    then hand the TMEM buffer back (`acc_empty`)
// The accumulator is double buffered in tensor memory (2 x BN columns) so the
// epilogue of tile i overlaps the MMAs of tile i+1.  The fused dynamic-LoRA
// configuration (a third, fp32 accumulator for t @ lora_b^T next to the int32
// ones) keeps 256-wide tiles with ONE int32 buffer instead and has eight
// epilogue warps (two per 32-lane quarter, 320 threads) to keep the un-hidden
// epilogue short.  16-bit outputs are computed as packed pairs and leave
// through shared memory and TMA stores.
//
// PAIR variant (cta_group::2): two CTAs of a cluster work on one 256 x BN
// tile.  Each loads its own 128 rows of A and its own BN/2 rows of B (half the
// shared-memory fill bandwidth per SM for the same MMA work), the even CTA
// issues the 256-row MMAs for both, each keeps and drains its own 128
// accumulator rows.  Stage-full barriers live in the leader and count both
// CTAs' TMA bytes; stage-empty / accumulator-full signals are committed to
// both CTAs; accumulator-empty arrivals of both CTAs go to the leader.
//
// Every mbarrier wait is bounded: a wait that runs out writes a code to the
// device status word, raises a CTA-wide abort flag and all roles fall through
// to the common teardown (which still frees the tensor memory).
//
// No TMA load in this file uses cluster multicast.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"
#include "ptx_sm100.cuh"

namespace i8f {
namespace {

constexpr int kBM = 128;            // rows of A per CTA == TMEM lanes
constexpr int kStageRowBytes = 128; // one 128-byte swizzle span of K per stage

enum Kind : int { kKindI8 = 0, kKindBF16 = 1, kKindF16 = 2 };
enum EpiMode : int { kEpiI32 = 0, kEpiDequant = 1, kEpiCast = 2, kEpiAccum = 3 };

// status codes written by bounded waits
enum : int { kStEmptyWait = 101, kStFullWait = 102, kStAccEmptyWait = 103, kStAccFullWait = 104 };

struct GemmParams {
    int M, N;
    int num_k_blocks;
    int tiles_m, tiles_n;
    void* out;
    long long ldo;
    int out_dtype;
    const float* a_scale;
    const float* w_scale;
    int w_scale_mode;
    const void* bias;
    int bias_dtype;
    int epi_mode;
    int epi_order;
    int add_existing;  // dequant mode: out = round(round(result) + out) (a LoRA term already stored in out)
    const void* gate;  // with add_existing: out = round(out + gate[n] * round(result)), gate [N] in the output type
    int vec_ok;  // out pointer / pitch allow 16-byte row-segment stores
    int tma_out; // 16-bit output leaves through shared memory and TMA stores (needs vec_ok)
    int lora_k_blocks;  // fused dynamic LoRA: 64-element slabs of the rank (0 = none)
    int lora_bf16;      // its operand type (else fp16)
    int wide_out;       // scatter mode: 64-column (128-byte) store boxes
    int n_out;   // number of destinations (tensor maps) every output chunk is stored to
    int out_col0; // column of the destination matrices at which this launch's block starts
    int k_split;  // 1, or 2: the two CTAs of a cluster each take half of K for the same tile (single-CTA kernels)
    int* status;
};

constexpr int kMaxOutputs = 8;

// Tensor maps of the output: one for an ordinary launch; one per destination (this GPU's and its peers' copies of
// the full activation matrix) when the result block is scattered to several GPUs from the epilogue.
struct alignas(64) OutMaps {
    CUtensorMap m[kMaxOutputs];
};

// LORA: a second, fp32 accumulator per buffer holds t @ lora_b^T (kind::f16 MMAs issued after the int8 K loop of
// the same tile), so the dynamic-LoRA term is added in the epilogue without ever touching global memory.
struct alignas(64) LoraMaps {
    CUtensorMap t;   // t [M, r], box 64 x 128 rows
    CUtensorMap b;   // lora_b [N, r], box 64 x (rows of B per CTA)
};

template <int BN, bool PAIR, bool LORA = false>
struct Cfg {
    static constexpr int kBRows = PAIR ? BN / 2 : BN;  // rows of B this CTA stages
    static constexpr int kABytes = kBM * kStageRowBytes;
    static constexpr int kBBytes = kBRows * kStageRowBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    // Epilogue warps: four (one per 32-lane quarter of tensor memory) or, where the epilogue cannot hide under the
    // next tile's MMAs (single accumulator buffer, below), eight: two per quarter, each taking half of the columns.
    static constexpr int kEpiWarps = (LORA && 3 * BN > 512) ? 8 : 4;
    static constexpr int kThreads = 64 + 32 * kEpiWarps;
    static constexpr int kRingBudget = (kEpiWarps == 8 ? 160 : 192) * 1024;   // eight warps need more staging space
    static constexpr int kStages = kRingBudget / kStageBytes > 8 ? 8 : kRingBudget / kStageBytes;
    // TMEM: two int32/fp32 accumulator buffers at columns 0 and BN, so the epilogue of a tile overlaps the MMAs of the
    // next; with LORA one more fp32 accumulator behind them.  The LoRA accumulator needs no double buffering: it is
    // written at the very end of a tile's MMA sequence, long after the epilogue of the previous tile has drained it.
    // Three buffers of 256 columns do not fit the 512 columns: that configuration keeps ONE int32 buffer (the
    // epilogue then runs between two tiles' MMAs instead of under them) and the full-rate 256-wide tile.
    static constexpr int kAccBufs = (LORA && 3 * BN > 512) ? 1 : 2;
    static constexpr int kLoraCol = kAccBufs * BN;
    static constexpr int kColsUsed = (kAccBufs + (LORA ? 1 : 0)) * BN;
    static constexpr int kTmemCols = kColsUsed <= 128 ? 128 : (kColsUsed <= 256 ? 256 : 512);   // power of two >= 32
    static_assert(kColsUsed <= 512, "tensor memory has 512 columns");
    static constexpr int kBarrierBytes = 1024;
    static constexpr int kEpiBytes = kEpiWarps * 2 * BN * 4;  // per epilogue warp: BN column scales + BN biases (fp32)
    static constexpr int kOutStageBytes = kEpiWarps * 2 * 2048;  // per epilogue warp: two 32-row x 64-byte output chunks
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + kEpiBytes + kOutStageBytes + 1024;  // + slack
    static constexpr int kTileM = PAIR ? 2 * kBM : kBM;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& m_blk, int& n_blk) {
    // groups of 8 row-blocks, row-block fastest inside a group
    const int group_sz = 8 * tiles_n;
    const int group = t / group_sz;
    const int first_m = group * 8;
    const int gm = min(tiles_m - first_m, 8);
    const int r = t - group * group_sz;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
}

template <int DT>
__device__ __forceinline__ float round_out(float x) {
    if constexpr (DT == I8F_BF16) return __bfloat162float(__float2bfloat16_rn(x));
    else return __half2float(__float2half_rn(x));
}
template <int DT>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if constexpr (DT == I8F_BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    } else {
        const __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
}
template <int DT>
__device__ __forceinline__ float unpack_lo(uint32_t w) {
    if constexpr (DT == I8F_BF16) return __uint_as_float(w << 16);
    else return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xFFFFu)));
}
template <int DT>
__device__ __forceinline__ float unpack_hi(uint32_t w) {
    if constexpr (DT == I8F_BF16) return __uint_as_float(w & 0xFFFF0000u);
    else return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}

__device__ __forceinline__ float load_as_f32(const void* p, int dt, long long i) {
    if (dt == I8F_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    if (dt == I8F_F16) return __half2float(static_cast<const __half*>(p)[i]);
    return static_cast<const float*>(p)[i];
}

// a + b on two packed 16-bit values, one rounding per lane.  Bit-identical to what the reference's tensor add does
// (widen to fp32, add, round to the 16-bit type): the fp32 sum of two bf16 / fp16 values is either exact or so
// lopsided that neither rounding can land on a tie.
template <int DT>
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
    if constexpr (DT == I8F_BF16) {
        const __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    } else {
        const __half2 r = __hadd2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
}

// Store 32 consecutive 16-bit outputs of one row, given as 16 packed pairs.
__device__ __forceinline__ void store_row32(const GemmParams& p, long long row, int col, const uint32_t (&yp)[16]) {
    using T16 = unsigned short;
    T16* dst = static_cast<T16*>(p.out) + row * p.ldo + col;
    if (p.vec_ok && col + 32 <= p.N) {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int g = 0; g < 4; ++g) d4[g] = make_uint4(yp[4 * g], yp[4 * g + 1], yp[4 * g + 2], yp[4 * g + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < p.N) dst[j] = static_cast<T16>((j & 1) ? (yp[j >> 1] >> 16) : (yp[j >> 1] & 0xFFFFu));
    }
}

template <int OUT>
__device__ __forceinline__ void load_row32(const GemmParams& p, long long row, int col, float (&y)[32]) {
    using T16 = unsigned short;
    const T16* src = static_cast<const T16*>(p.out) + row * p.ldo + col;
    if (p.vec_ok && col + 32 <= p.N) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint4 o = s4[g];
            const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                y[8 * g + 2 * i] = unpack_lo<OUT>(w[i]);
                y[8 * g + 2 * i + 1] = unpack_hi<OUT>(w[i]);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) y[j] = (col + j < p.N) ? unpack_lo<OUT>(src[j]) : 0.f;
    }
}

// Existing output values of one 32-column row segment, fetched ahead of use (4 x 16 bytes per thread).
struct OldChunk {
    uint4 raw[4];
    bool valid;   // raw[] holds the segment (full in-range segment, vector path)
};

__device__ __forceinline__ void prefetch_old(const GemmParams& p, long long row, bool row_ok, int col, OldChunk& o) {
    o.valid = row_ok && p.vec_ok && col + 32 <= p.N;
    if (o.valid) {
        const uint4* s4 = reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(p.out) + row * p.ldo + col);
#pragma unroll
        for (int g = 0; g < 4; ++g) o.raw[g] = s4[g];
    }
}

template <int OUT>
__device__ __forceinline__ void old_values(const GemmParams& p, long long row, int col, const OldChunk& o, uint32_t (&yp)[16]) {
    if (o.valid) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            yp[4 * g] = o.raw[g].x;
            yp[4 * g + 1] = o.raw[g].y;
            yp[4 * g + 2] = o.raw[g].z;
            yp[4 * g + 3] = o.raw[g].w;
        }
    } else {
        float y[32];
        load_row32<OUT>(p, row, col, y);
#pragma unroll
        for (int i = 0; i < 16; ++i) yp[i] = pack2<OUT>(y[2 * i], y[2 * i + 1]);   // exact: the values are 16-bit already
    }
}

// One 32-column chunk of one accumulator row.  `cs` points at this chunk's 32 column scales (fp32) in shared
// memory; `cb` at its biases: 32 fp32 values for the single-rounding order, 16 packed pairs already rounded to
// OUT for the reference order.  Every lane reads the same address, a broadcast.  In the reference order every
// intermediate is a 16-bit tensor, so after the scaling the chunk lives as 16 packed pairs and each further
// term (bias, LoRA, previous output) is one packed add per pair.  The result goes either straight to global
// memory or, when `stage` is non-zero, into this warp's shared-memory staging chunk (row = lane, 64 bytes per
// row, 16-byte pieces XOR-swizzled with (row >> 1) & 3 as the TMA 64-byte swizzle expects).
template <int OUT, bool LORA>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, long long row, bool row_ok, int col,
                                               const uint32_t (&v)[32], const uint32_t (&lv)[LORA ? 32 : 1], float row_scale,
                                               float ws_scalar, const float* cs, const float* cb, const OldChunk& old,
                                               uint32_t stage, int lane, int wide_half = -1, const uint32_t* cg = nullptr) {
    uint32_t yp[16];
    if (p.epi_mode == kEpiDequant) {
        const bool per_ch = p.w_scale_mode == I8F_WSCALE_CHANNEL;
        const bool single = p.epi_order == I8F_EPI_SINGLE;
        float y[32];
        if (!per_ch) {
            // reference order: (ws * xs) first, then times the accumulator
            const float total = __fmul_rn(ws_scalar, row_scale);
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = __fmul_rn(__int2float_rn(static_cast<int>(v[j])), total);
        } else if (!single) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                y[j] = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[j])), row_scale), cs[j]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                y[j] = __fmul_rn(__int2float_rn(static_cast<int>(v[j])), __fmul_rn(row_scale, cs[j]));
        }
        if (single && p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = __fadd_rn(y[j], cb[j]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) yp[i] = pack2<OUT>(y[2 * i], y[2 * i + 1]);
        if (!single && p.bias != nullptr) {
            const uint32_t* cbp = reinterpret_cast<const uint32_t*>(cb);
#pragma unroll
            for (int i = 0; i < 16; ++i) yp[i] = add2<OUT>(yp[i], cbp[i]);
        }
        if constexpr (LORA) {
            // y + lora_y.to(y.dtype): both terms are in the output type, as in the reference
#pragma unroll
            for (int i = 0; i < 16; ++i)
                yp[i] = add2<OUT>(yp[i], pack2<OUT>(__uint_as_float(lv[2 * i]), __uint_as_float(lv[2 * i + 1])));
        }
        if (p.add_existing && row_ok) {
            uint32_t prev[16];
            old_values<OUT>(p, row, col, old, prev);
            if (cg != nullptr) {
                // gated residual: prev + gate * y in fp32 (the product of two 16-bit values is exact, so the sum is
                // rounded once), then to the output type -- what torch.addcmul(prev, gate, y) computes
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t g = cg[i];
                    yp[i] = pack2<OUT>(__fmaf_rn(unpack_lo<OUT>(g), unpack_lo<OUT>(yp[i]), unpack_lo<OUT>(prev[i])),
                                       __fmaf_rn(unpack_hi<OUT>(g), unpack_hi<OUT>(yp[i]), unpack_hi<OUT>(prev[i])));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) yp[i] = add2<OUT>(yp[i], prev[i]);
            }
        }
    } else if (p.epi_mode == kEpiCast) {
#pragma unroll
        for (int i = 0; i < 16; ++i) yp[i] = pack2<OUT>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
    } else {  // kEpiAccum: out = round(out + round(acc))
        if (row_ok) old_values<OUT>(p, row, col, old, yp);
        else {
#pragma unroll
            for (int i = 0; i < 16; ++i) yp[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i)
            yp[i] = add2<OUT>(yp[i], pack2<OUT>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])));
    }
    if (stage != 0) {
        // narrow: 64-byte rows, 64-byte swizzle; wide (wide_half 0/1): this chunk is one half of a 128-byte row,
        // 128-byte swizzle (16-byte piece index XOR row & 7)
        const bool wide = wide_half >= 0;
        const uint32_t row_addr = stage + static_cast<uint32_t>(lane) * (wide ? 128u : 64u);
        const uint32_t x = wide ? (static_cast<uint32_t>(lane) & 7u) : (static_cast<uint32_t>(lane >> 1) & 3u);
        const uint32_t g0 = wide ? static_cast<uint32_t>(wide_half) * 4u : 0u;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t a = row_addr + (((g0 + static_cast<uint32_t>(g)) ^ x) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(yp[4 * g]), "r"(yp[4 * g + 1]),
                         "r"(yp[4 * g + 2]), "r"(yp[4 * g + 3])
                         : "memory");
        }
    } else if (row_ok) {
        store_row32(p, row, col, yp);
    }
}

__device__ __forceinline__ void store_i32_row32(const GemmParams& p, long long row, int col, const uint32_t (&v)[32]) {
    int* dst = static_cast<int*>(p.out) + row * p.ldo + col;
    if (p.vec_ok && col + 32 <= p.N) {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int g = 0; g < 8; ++g) d4[g] = make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < p.N) dst[j] = static_cast<int>(v[j]);
    }
}

template <int KIND, int BN, bool PAIR, bool LORA>
__global__ void __launch_bounds__((Cfg<BN, PAIR, LORA>::kThreads), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ OutMaps outs, const __grid_constant__ LoraMaps lora, const GemmParams p) {
    using C = Cfg<BN, PAIR, LORA>;
    static_assert(!LORA || (KIND == kKindI8 && PAIR), "the fused LoRA accumulator exists for the paired int8 kernel");
    constexpr int kElemsPerStage = (KIND == kKindI8) ? kStageRowBytes : kStageRowBytes / 2;
    constexpr uint32_t kIdesc = (KIND == kKindI8)     ? make_idesc(kDFmtS32, kFmtS8, C::kTileM, BN)
                                : (KIND == kKindBF16) ? make_idesc(kDFmtF32, kFmtBF16, C::kTileM, BN)
                                                      : make_idesc(kDFmtF32, kFmtF16, C::kTileM, BN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    constexpr int kBarOff = C::kStages * C::kStageBytes;
    // barrier block: full[kStages], empty[kStages], acc_full[2], acc_empty[2], tmem slot, abort flag
    const uint32_t full0 = smem_base + kBarOff;
    const uint32_t empty0 = full0 + 8 * C::kStages;
    const uint32_t accfull0 = full0 + 16 * C::kStages;
    const uint32_t accempty0 = accfull0 + 16;
    const uint32_t tmem_slot = accempty0 + 16;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + kBarOff + 16 * C::kStages + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + kBarOff + 16 * C::kStages + 36);
    float* epi_smem = reinterpret_cast<float*>(gen_base + kBarOff + C::kBarrierBytes);
    const uint32_t out_stage0 = smem_base + kBarOff + C::kBarrierBytes + C::kEpiBytes;  // 1024-byte aligned

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;   // position in the CTA pair
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accfull0 + 8 * b, 1);
            mbar_init(accempty0 + 8 * b, (PAIR ? 2 : 1) * C::kEpiWarps);  // one arrival per epilogue warp (of both CTAs)
        }
        *abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (p.tma_out)
            for (int d = 0; d < p.n_out; ++d) tma_prefetch_desc(&outs.m[d]);
    }
    if (warp == 1) {
        if constexpr (PAIR) tmem_alloc_pair<C::kTmemCols>(tmem_slot);
        else tmem_alloc<C::kTmemCols>(tmem_slot);
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) {  // the peer must see initialised barriers before it signals them
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;
    // Programmatic dependent launch: everything above (barriers, tensor memory, descriptor prefetch) may run while the
    // kernel before this one in the stream is still finishing; nothing below may start before its results are visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int num_tiles = p.tiles_m * p.tiles_n;
    // K split (single-CTA kernels, sub-wave problems): a cluster of two CTAs owns ONE tile, each CTA runs half of the K
    // slabs into its own tensor memory, the second CTA hands its partial tile to the first through distributed shared
    // memory and the first one runs the epilogue.  The tensor core takes one row of A per cycle whatever the tile's
    // width, so a narrow problem gets faster only by putting more SMs on its rows x K.
    const bool ksplit = !PAIR && p.k_split == 2;
    const uint32_t krank = ksplit ? cluster_ctarank() : 0u;
    const int tile_step = (PAIR || ksplit) ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const int tile_first = (PAIR || ksplit) ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int kb_begin = ksplit ? static_cast<int>(krank) * (p.num_k_blocks >> 1) : 0;
    const int kb_end = (ksplit && krank == 0) ? (p.num_k_blocks >> 1) : p.num_k_blocks;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = tile_first; ok && t < num_tiles; t += tile_step) {
                int m_blk, n_blk;
                tile_coords(t, p.tiles_m, p.tiles_n, m_blk, n_blk);
                const int row_a = m_blk * C::kTileM + static_cast<int>(rank) * kBM;
                const int row_b = n_blk * BN + static_cast<int>(rank) * C::kBRows;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1u, abort_flag, p.status, kStEmptyWait)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + stage * C::kStageBytes;
                    const uint32_t b_dst = a_dst + C::kABytes;
                    if constexpr (PAIR) {
                        // both CTAs' bytes are counted on the leader's barrier; the leader alone arms it
                        const uint32_t bar = mapa_cluster(full0 + 8 * stage, 0);
                        if (leader) mbar_arrive_expect_tx(full0 + 8 * stage, 2 * C::kStageBytes);
                        tma_load_2d_pair(a_dst, &tmA, bar, kb * kElemsPerStage, row_a);
                        tma_load_2d_pair(b_dst, &tmB, bar, kb * kElemsPerStage, row_b);
                    } else {
                        mbar_arrive_expect_tx(full0 + 8 * stage, C::kStageBytes);
                        tma_load_2d(a_dst, &tmA, full0 + 8 * stage, kb * kElemsPerStage, row_a);
                        tma_load_2d(b_dst, &tmB, full0 + 8 * stage, kb * kElemsPerStage, row_b);
                    }
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if constexpr (LORA) {
                    // the low-rank operands ride the same ring: t rows where A rows go, lora_b rows where W rows go
                    for (int lb = 0; ok && lb < p.lora_k_blocks; ++lb) {
                        if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1u, abort_flag, p.status, kStEmptyWait)) {
                            ok = false;
                            break;
                        }
                        const uint32_t a_dst = smem_base + stage * C::kStageBytes;
                        const uint32_t bar = mapa_cluster(full0 + 8 * stage, 0);
                        if (leader) mbar_arrive_expect_tx(full0 + 8 * stage, 2 * C::kStageBytes);
                        tma_load_2d_pair(a_dst, &lora.t, bar, lb * 64, row_a);
                        tma_load_2d_pair(a_dst + C::kABytes, &lora.b, bar, lb * 64, row_b);
                        if (++stage == C::kStages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
            }
        }
        if (ksplit) {   // every thread of both CTAs takes part in the two barriers of the hand-over (see the epilogue)
            cluster_arrive();
            cluster_wait();
            cluster_arrive();
            cluster_wait();
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            // `ready`: the full barrier of the slab about to be consumed was already seen complete.  Each iteration
            // asks for the NEXT slab's barrier before it issues its own MMAs, so the round trip of that query passes
            // under the MMA issue instead of in front of it (the issue loop, not the tensor core, bounds narrow tiles).
            bool ready = false;
            for (int t = tile_first; ok && t < num_tiles; t += tile_step) {
                if (!mbar_wait_bounded(accempty0 + 8 * buf, acc_phase ^ 1u, abort_flag, p.status, kStAccEmptyWait)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
                for (int kb = 0; kb < kb_end - kb_begin; ++kb) {
                    if (!ready && !mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, p.status, kStFullWait)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    {
                        const int next_stage = stage + 1 == C::kStages ? 0 : stage + 1;
                        const uint32_t next_phase = stage + 1 == C::kStages ? phase ^ 1u : phase;
                        ready = mbar_try_wait(full0 + 8 * next_stage, next_phase);
                    }
                    const uint32_t a_src = smem_base + stage * C::kStageBytes;
                    const uint64_t adesc = make_smem_desc_sw128(a_src);
                    const uint64_t bdesc = make_smem_desc_sw128(a_src + C::kABytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // +32 bytes of K per instruction: 2 in the (address >> 4) field
                        const uint32_t accumulate = (kb | k) != 0 ? 1u : 0u;
                        if constexpr (PAIR) {
                            if constexpr (KIND == kKindI8) mma_i8_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, accumulate);
                            else mma_f16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, accumulate);
                        } else {
                            if constexpr (KIND == kKindI8) mma_i8(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, accumulate);
                            else mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, accumulate);
                        }
                    }
                    // stage reusable (in both CTAs) once these MMAs have read it
                    if constexpr (PAIR) mma_commit_pair(empty0 + 8 * stage);
                    else mma_commit(empty0 + 8 * stage);
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if constexpr (LORA) {
                    const uint32_t idesc_lora = p.lora_bf16 ? make_idesc(kDFmtF32, kFmtBF16, C::kTileM, BN)
                                                            : make_idesc(kDFmtF32, kFmtF16, C::kTileM, BN);
                    // the (single) LoRA accumulator was last read by the epilogue of the previous tile, which owns the
                    // other int32 buffer: its hand-back covers both.  Re-waiting a completed phase returns at once.
                    if (C::kAccBufs == 2 && t != tile_first) {
                        const uint32_t prev_phase = (buf == 1) ? acc_phase : (acc_phase ^ 1u);
                        if (!mbar_wait_bounded(accempty0 + 8 * (buf ^ 1), prev_phase, abort_flag, p.status, kStAccEmptyWait)) break;
                        tc_fence_after_sync();
                    }
                    for (int lb = 0; lb < p.lora_k_blocks; ++lb) {
                        if (!ready && !mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, p.status, kStFullWait)) {
                            ok = false;
                            break;
                        }
                        ready = false;
                        tc_fence_after_sync();
                        const uint32_t a_src = smem_base + stage * C::kStageBytes;
                        const uint64_t adesc = make_smem_desc_sw128(a_src);
                        const uint64_t bdesc = make_smem_desc_sw128(a_src + C::kABytes);
#pragma unroll
                        for (int k = 0; k < 4; ++k)   // 16 elements = 32 bytes of the rank per instruction
                            mma_f16_pair(tmem_base + C::kLoraCol, adesc + 2 * k, bdesc + 2 * k, idesc_lora, (lb | k) != 0 ? 1u : 0u);
                        mma_commit_pair(empty0 + 8 * stage);
                        if (++stage == C::kStages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                    if (!ok) break;
                }
                if constexpr (PAIR) mma_commit_pair(accfull0 + 8 * buf);  // accumulator complete
                else mma_commit(accfull0 + 8 * buf);
                if constexpr (C::kAccBufs == 2) buf ^= 1;
                if (buf == 0) acc_phase ^= 1u;
            }
        }
        if (ksplit) {
            cluster_arrive();
            cluster_wait();
            cluster_arrive();
            cluster_wait();
        }
    } else {
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
        float* col_scale = epi_smem + (warp - 2) * 2 * BN;
        float* col_bias = col_scale + BN;
        int buf = 0;
        uint32_t acc_phase = 0;
        const bool dequant = p.epi_mode == kEpiDequant;
        const bool per_ch = dequant && p.w_scale_mode == I8F_WSCALE_CHANNEL;
        const bool has_bias = dequant && p.bias != nullptr;
        const bool has_gate = dequant && p.add_existing && p.gate != nullptr;
        const int bias_step = p.epi_order == I8F_EPI_PYTORCH ? 16 : 32;   // packed pairs or fp32 per 32-column chunk
        const float ws_scalar = (dequant && !per_ch) ? __ldg(p.w_scale) : 0.f;
        const uint32_t accempty_leader = PAIR ? mapa_cluster(accempty0, 0) : accempty0;
        const bool need_old = (dequant && p.add_existing) || p.epi_mode == kEpiAccum;
        const bool tma_out = p.tma_out != 0;
        const bool wide_out = p.wide_out != 0;   // implies tma_out; N is a multiple of 64
        const uint32_t out_stage = out_stage0 + static_cast<uint32_t>(warp - 2) * 4096u;
        uint32_t out_chunk = 0;
        for (int t = tile_first; t < num_tiles; t += tile_step) {
            int m_blk, n_blk;
            tile_coords(t, p.tiles_m, p.tiles_n, m_blk, n_blk);
            // stage this tile's column scales and biases (fp32) for broadcast reads
            if (per_ch || has_bias || has_gate) {
                __syncwarp();
                for (int j = lane; j < BN; j += 32) {
                    const int col = n_blk * BN + j;
                    const bool in = col < p.N;
                    if (per_ch) col_scale[j] = in ? __ldg(p.w_scale + col) : 0.f;
                    if (has_bias && p.epi_order != I8F_EPI_PYTORCH) col_bias[j] = in ? load_as_f32(p.bias, p.bias_dtype, col) : 0.f;
                }
                if (has_gate) {
                    // packed pairs in the upper half of the bias area (the reference order keeps its biases as packed
                    // pairs in the lower half; the gated form exists for that order only)
                    uint32_t* packed = reinterpret_cast<uint32_t*>(col_bias) + BN / 2;
                    for (int j = lane; j < BN / 2; j += 32) {
                        const int col = n_blk * BN + 2 * j;
                        const float g0 = col < p.N ? load_as_f32(p.gate, p.out_dtype, col) : 0.f;
                        const float g1 = col + 1 < p.N ? load_as_f32(p.gate, p.out_dtype, col + 1) : 0.f;
                        packed[j] = p.out_dtype == I8F_BF16 ? pack2<I8F_BF16>(g0, g1) : pack2<I8F_F16>(g0, g1);
                    }
                }
                if (has_bias && p.epi_order == I8F_EPI_PYTORCH) {
                    // the reference casts the bias to the output type and adds 16-bit tensors: keep it as packed pairs
                    uint32_t* packed = reinterpret_cast<uint32_t*>(col_bias);
                    for (int j = lane; j < BN / 2; j += 32) {
                        const int col = n_blk * BN + 2 * j;
                        const float b0 = col < p.N ? load_as_f32(p.bias, p.bias_dtype, col) : 0.f;
                        const float b1 = col + 1 < p.N ? load_as_f32(p.bias, p.bias_dtype, col + 1) : 0.f;
                        packed[j] = p.out_dtype == I8F_BF16 ? pack2<I8F_BF16>(b0, b1) : pack2<I8F_F16>(b0, b1);
                    }
                }
                __syncwarp();
            }
            const long long row = static_cast<long long>(m_blk) * C::kTileM + static_cast<int>(rank) * kBM + quarter * 32 + lane;
            const long long warp_row0 = row - lane;
            const bool row_ok = row < p.M;
            const float row_scale = (dequant && row_ok) ? __ldg(p.a_scale + row) : 0.f;
            // this warp's share of the tile's 32-column chunks (all of them with four epilogue warps), cut at N
            constexpr int kChunksPerWarp = (BN / 32) / (C::kEpiWarps / 4);
            const int c_first = ((warp - 2) >> 2) * kChunksPerWarp;
            const int chunks_in_n = static_cast<int>((p.N - static_cast<long long>(n_blk) * BN + 31) / 32);
            const int c_end = min(c_first + kChunksPerWarp, chunks_in_n);
            OldChunk old_next;
            old_next.valid = false;
            if (need_old && c_first < c_end)   // in flight while the MMAs finish
                prefetch_old(p, row, row_ok, n_blk * BN + c_first * 32, old_next);
            const bool acc_ok = mbar_wait_bounded(accfull0 + 8 * buf, acc_phase, abort_flag, p.status, kStAccFullWait);
            if (!acc_ok && !ksplit) break;
            tc_fence_after_sync();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * BN);
            if constexpr (!PAIR) {
                if (ksplit) {
                    // Both CTAs' MMAs are complete once both have passed this barrier: the first CTA's operand ring is
                    // then free and serves as the landing zone, [chunk][word of the row's 32][row of the tile]: a warp's
                    // remote store and the first CTA's later load both cover 128 contiguous bytes.
                    cluster_arrive();
                    cluster_wait();
                    if (krank == 1 && acc_ok) {
                        const int row_in_tile = quarter * 32 + lane;
                        for (int c = c_first; c < c_end; ++c) {
                            uint32_t v[32];
                            tmem_ld_32x32(t_addr + c * 32, v);
                            tmem_ld_wait();
                            // word j of row r at [chunk][j][r]: a warp's store covers 128 contiguous bytes
                            const uint32_t dst0 = mapa_cluster(smem_base + static_cast<uint32_t>(c * kBM * 128 + row_in_tile * 4), 0);
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(dst0 + static_cast<uint32_t>(j * kBM * 4)), "r"(v[j])
                                             : "memory");
                        }
                    }
                    cluster_arrive();      // release: the partial tile is written ...
                    cluster_wait();        // ... acquire: and visible to the first CTA
                    if (krank == 1 || !acc_ok) break;
                }
            }
            const uint32_t t_lora = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(C::kLoraCol);
            bool released = false;
#pragma unroll 1
            for (int c = c_first; c < c_end; ++c) {
                const int col = n_blk * BN + c * 32;
                uint32_t v[32];
                tmem_ld_32x32(t_addr + c * 32, v);
                uint32_t lv[LORA ? 32 : 1];
                if constexpr (LORA) tmem_ld_32x32(t_lora + c * 32, lv);
                const OldChunk old_cur = old_next;
                if (need_old && c + 1 < c_end) prefetch_old(p, row, row_ok, col + 32, old_next);
                uint32_t stage = 0;
                const int wide_half = wide_out ? (c & 1) : -1;
                if (wide_out) {
                    // scatter mode: one 4 KB buffer per warp holds 32 rows x 128 bytes (two chunks); the stores of the
                    // previous pair of chunks must have read it before it is rewritten
                    stage = out_stage;
                    if (wide_half == 0) {
                        if (lane == 0) tma_store_wait_read<0>();
                        __syncwarp();
                    }
                } else if (tma_out) {
                    stage = out_stage + static_cast<uint32_t>(out_chunk & 1) * 2048u;
                    // the store that last read this staging chunk (two chunks ago) must be done with it
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                }
                tmem_ld_wait();
                if constexpr (!PAIR) {
                    if (ksplit) {   // + the second CTA's half of K: exact for int32, one more fp32 add for the 16-bit kinds
                        const int row_in_tile = quarter * 32 + lane;
                        const uint32_t* col0 = reinterpret_cast<const uint32_t*>(gen_base + c * kBM * 128) + row_in_tile;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t part = col0[j * kBM];
                            if constexpr (KIND == kKindI8) v[j] += part;
                            else v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), __uint_as_float(part)));
                        }
                    }
                }
                if (C::kAccBufs == 1 && c == c_end - 1) {
                    // single accumulator buffer (the next tile's MMAs wait for this): the last values of this warp's
                    // share are in registers, hand the accumulator back before the arithmetic and the store of this
                    // chunk.  With two buffers the hand-back stays after the loop, which measured 1 % faster.
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (PAIR) mbar_arrive_cluster(accempty_leader + 8 * buf);
                        else mbar_arrive(accempty0 + 8 * buf);
                    }
                    released = true;
                }
                if (p.epi_mode == kEpiI32) {
                    if (row_ok) store_i32_row32(p, row, col, v);
                } else if (p.out_dtype == I8F_BF16) {
                    epilogue_chunk<I8F_BF16, LORA>(p, row, row_ok, col, v, lv, row_scale, ws_scalar, col_scale + c * 32,
                                                   col_bias + c * bias_step, old_cur, stage, lane, wide_half,
                                                   has_gate ? reinterpret_cast<const uint32_t*>(col_bias) + BN / 2 + c * 16 : nullptr);
                } else {
                    epilogue_chunk<I8F_F16, LORA>(p, row, row_ok, col, v, lv, row_scale, ws_scalar, col_scale + c * 32,
                                                  col_bias + c * bias_step, old_cur, stage, lane, wide_half,
                                                  has_gate ? reinterpret_cast<const uint32_t*>(col_bias) + BN / 2 + c * 16 : nullptr);
                }
                if (wide_out) {
                    if (wide_half == 1) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            for (int d = 0; d < p.n_out; ++d)   // 128-byte row segments: full-size NVLink writes
                                tma_store_2d(&outs.m[d], stage, p.out_col0 + col - 32, static_cast<int>(warp_row0));
                            tma_store_commit();
                        }
                    }
                } else if (tma_out) {
                    fence_proxy_async_smem();               // generic-proxy writes -> visible to the TMA engine
                    __syncwarp();
                    if (lane == 0) {
                        // rows past M (and, for a single destination, columns past N) are clipped by the TMA unit
                        for (int d = 0; d < p.n_out; ++d)
                            tma_store_2d(&outs.m[d], stage, p.out_col0 + col, static_cast<int>(warp_row0));
                        tma_store_commit();
                    }
                    ++out_chunk;
                }
            }
            if (!released) {   // a warp whose share lies past N read nothing
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (PAIR) mbar_arrive_cluster(accempty_leader + 8 * buf);
                    else mbar_arrive(accempty0 + 8 * buf);
                }
            }
            if constexpr (C::kAccBufs == 2) buf ^= 1;
            if (buf == 0) acc_phase ^= 1u;
        }
        if (tma_out && lane == 0) tma_store_wait_all<0>();   // shared memory must outlive the last store's reads
    }

    // common teardown (also reached after an aborted wait)
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // give copies that are still in flight time to land before the CTA exits
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if constexpr (PAIR) {  // neither CTA may leave while the other can still touch its memory
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        if constexpr (PAIR) tmem_dealloc_pair<C::kTmemCols>(tmem_base);
        else tmem_dealloc<C::kTmemCols>(tmem_base);
    }
}

// Self-test of the bounded wait: one CTA waits on a barrier that nothing ever signals.  The wait must give up
// after `limit_cycles`, record kStSelfTest in the status word and let the kernel end normally.
enum : int { kStSelfTest = 199 };
__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    // thread 0 hits the limit; the others see the abort flag it raises and give up as well
    mbar_wait_bounded(smem_u32(&bar), 0u, &abort_flag, status, kStSelfTest, threadIdx.x == 0 ? limit_cycles : 4 * limit_cycles);
    __syncthreads();
}

// ------------------------------------------------------------------ host
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
    static EncodeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeFn>(f);
    }();
    return fn;
}

// Encoded tensor maps depend only on the address and the geometry, and a model calls the same layers with the same
// buffers step after step (weights, a reused workspace, allocator-recycled outputs): a small per-thread cache saves
// the driver call, about a microsecond per map, three maps per launch.
struct MapKey {
    const void* base;
    int64_t rows, cols, ld;
    int tag;        // operand: kind * 1024 + box rows; output: -1 narrow box, -2 wide box
    int device;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && tag == o.tag && device == o.device;
    }
};
struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool valid;
};
constexpr int kMapCacheSlots = 64;
MapSlot* map_cache_slot(const MapKey& k) {
    static thread_local MapSlot slots[kMapCacheSlots] = {};
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) >> 4;
    h = (h ^ (h >> 17)) * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(k.rows) * 31 + static_cast<uint64_t>(k.cols) * 131 +
        static_cast<uint64_t>(k.ld) * 7 + static_cast<uint64_t>(k.tag + 8);
    return &slots[(h >> 20) % kMapCacheSlots];
}

int current_device();

// K-major [rows, k_elems] matrix, box = one 128-byte span of K x box_rows, 128-byte swizzle.
int make_operand_map(CUtensorMap* tm, int kind, const void* base, int64_t rows, int64_t k_elems, int64_t ld_elems,
                     int box_rows) {
    const MapKey key{base, rows, k_elems, ld_elems, kind * 1024 + box_rows, current_device()};
    MapSlot* slot = map_cache_slot(key);
    if (slot->valid && slot->key == key) {
        *tm = slot->map;
        return I8F_OK;
    }
    EncodeFn enc = get_encode_fn();
    I8F_REQUIRE(enc != nullptr, I8F_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const int esz = kind == kKindI8 ? 1 : 2;
    const CUtensorMapDataType dt = kind == kKindI8     ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : kind == kKindBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k_elems), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems) * esz};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kStageRowBytes / esz), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    I8F_REQUIRE(r == CUDA_SUCCESS, I8F_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    slot->key = key;
    slot->map = *tm;
    slot->valid = true;
    return I8F_OK;
}

// Output [rows, cols] of 16-bit elements, box = 32 columns x 32 rows (one epilogue warp's chunk), 64-byte swizzle.
int make_out_map(CUtensorMap* tm, const void* base, int64_t rows, int64_t cols, int64_t ld_elems, bool wide = false) {
    const MapKey key{base, rows, cols, ld_elems, wide ? -2 : -1, current_device()};
    MapSlot* slot = map_cache_slot(key);
    if (slot->valid && slot->key == key) {
        *tm = slot->map;
        return I8F_OK;
    }
    EncodeFn enc = get_encode_fn();
    I8F_REQUIRE(enc != nullptr, I8F_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems) * 2};
    const cuuint32_t box[2] = {wide ? 64u : 32u, 32};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, wide ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                           CU_TENSOR_MAP_L2_PROMOTION_NONE,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    I8F_REQUIRE(r == CUDA_SUCCESS, I8F_ERR_CUDA, "cuTensorMapEncodeTiled(out) failed with CUresult %d", static_cast<int>(r));
    slot->key = key;
    slot->map = *tm;
    slot->valid = true;
    return I8F_OK;
}

int current_device() {
    int dev = 0;
    cudaGetDevice(&dev);
    return (dev < 0 || dev >= 64) ? 0 : dev;
}

int sm_count() {
    static int cached[64] = {0};
    const int dev = current_device();
    if (cached[dev] == 0) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev] > 0 ? cached[dev] : 148;
}

struct Scatter {
    void* const* dests;   // base pointers of the destination matrices ([M, n_total], pitch ld elements)
    int n_dests;
    int64_t n_total;
    int64_t ld;
    int64_t col_offset;
};

struct LoraOperands {
    const void* t;        // [M, r], pitch ldt
    int64_t ldt;
    const void* b;        // [N, r], pitch ldb
    int64_t ldb;
    int64_t r;
    int kind;             // kKindBF16 or kKindF16
};

template <int KIND, int BN, bool PAIR, bool LORA = false>
int launch_gemm(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t M, int64_t N, int64_t K, GemmParams p,
                cudaStream_t st, const Scatter* scatter = nullptr, const LoraOperands* lo = nullptr, int k_split = 1) {
    using C = Cfg<BN, PAIR, LORA>;
    CUtensorMap tmA, tmB;
    LoraMaps lmaps{};
    if (LORA) {
        int rc_l = make_operand_map(&lmaps.t, lo->kind, lo->t, M, lo->r, lo->ldt, kBM);
        if (rc_l != I8F_OK) return rc_l;
        rc_l = make_operand_map(&lmaps.b, lo->kind, lo->b, N, lo->r, lo->ldb, C::kBRows);
        if (rc_l != I8F_OK) return rc_l;
        p.lora_k_blocks = static_cast<int>((lo->r + 63) / 64);
        p.lora_bf16 = lo->kind == kKindBF16 ? 1 : 0;
    }
    int rc = make_operand_map(&tmA, KIND, a, M, K, lda, kBM);
    if (rc != I8F_OK) return rc;
    rc = make_operand_map(&tmB, KIND, b, N, K, ldb, C::kBRows);
    if (rc != I8F_OK) return rc;
    static const int no_tma_store = [] {
        const char* e = getenv("I8F_GEMM_DIRECT_STORE");
        return (e != nullptr && e[0] == '1') ? 1 : 0;
    }();
    OutMaps outs{};
    if (scatter != nullptr) {
        // one map per destination over the whole [M, n_total] matrix; the block lands at column out_col0
        p.tma_out = 1;
        p.wide_out = (N % 64 == 0) ? 1 : 0;
        p.n_out = scatter->n_dests;
        p.out_col0 = static_cast<int>(scatter->col_offset);
        for (int d = 0; d < scatter->n_dests; ++d) {
            rc = make_out_map(&outs.m[d], scatter->dests[d], M, scatter->n_total, scatter->ld, p.wide_out != 0);
            if (rc != I8F_OK) return rc;
        }
    } else {
        p.tma_out = (p.epi_mode != kEpiI32 && p.vec_ok && !no_tma_store) ? 1 : 0;
        p.n_out = p.tma_out;
        p.out_col0 = 0;
        if (p.tma_out) {
            rc = make_out_map(&outs.m[0], p.out, M, N, p.ldo);
            if (rc != I8F_OK) return rc;
        }
    }
    const int esz = KIND == kKindI8 ? 1 : 2;
    const int k_per_stage = kStageRowBytes / esz;
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.num_k_blocks = static_cast<int>((K + k_per_stage - 1) / k_per_stage);
    p.k_split = (!PAIR && k_split == 2) ? 2 : 1;
    p.tiles_m = static_cast<int>((M + C::kTileM - 1) / C::kTileM);
    p.tiles_n = static_cast<int>((N + BN - 1) / BN);
    p.status = device_status_word();
    I8F_REQUIRE(p.status != nullptr, I8F_ERR_CUDA, "device status word unavailable");
    auto kern = gemm_tcgen05_kernel<KIND, BN, PAIR, LORA>;
    static bool attr_done[64] = {false};
    static int max_clusters[64] = {0};
    const int dev = current_device();
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "cudaFuncSetAttribute(smem=%d): %s", C::kSmemBytes, cudaGetErrorString(e));
        if (PAIR) {
            cudaLaunchConfig_t probe{};
            probe.gridDim = dim3(static_cast<unsigned>(sm_count() & ~1), 1, 1);
            probe.blockDim = dim3(C::kThreads, 1, 1);
            probe.dynamicSmemBytes = C::kSmemBytes;
            cudaLaunchAttribute at{};
            at.id = cudaLaunchAttributeClusterDimension;
            at.val.clusterDim.x = 2;
            at.val.clusterDim.y = 1;
            at.val.clusterDim.z = 1;
            probe.attrs = &at;
            probe.numAttrs = 1;
            int n = 0;
            e = cudaOccupancyMaxActiveClusters(&n, kern, &probe);
            if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "cudaOccupancyMaxActiveClusters: %s", cudaGetErrorString(e));
            max_clusters[dev] = n;
        }
        attr_done[dev] = true;
    }
    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(C::kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    static const int use_pdl = [] {
        const char* e = getenv("I8F_PDL");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    cudaLaunchAttribute at[3]{};
    int n_at = 0;
    if (PAIR) {
        I8F_REQUIRE(max_clusters[dev] > 0, I8F_ERR_CUDA, "no CTA pair fits on this device");
        const long long clusters = tiles < max_clusters[dev] ? tiles : max_clusters[dev];
        cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters), 1, 1);
        at[n_at].id = cudaLaunchAttributeClusterDimension;
        at[n_at].val.clusterDim.x = 2;
        at[n_at].val.clusterDim.y = 1;
        at[n_at].val.clusterDim.z = 1;
        ++n_at;
    } else if (p.k_split == 2) {
        // one tile per cluster of two CTAs (the caller checked that they fit one wave and that K has two halves)
        I8F_REQUIRE(2 * tiles <= sm_count() && p.num_k_blocks >= 2, I8F_ERR_INVALID_ARG, "K split needs 2 * tiles <= SMs");
        cfg.gridDim = dim3(static_cast<unsigned>(2 * tiles), 1, 1);
        at[n_at].id = cudaLaunchAttributeClusterDimension;
        at[n_at].val.clusterDim.x = 2;
        at[n_at].val.clusterDim.y = 1;
        at[n_at].val.clusterDim.z = 1;
        ++n_at;
    } else {
        cfg.gridDim = dim3(static_cast<unsigned>(tiles < sm_count() ? tiles : sm_count()), 1, 1);
    }
    if (use_pdl) {
        // let this kernel's set-up overlap the tail of the kernel before it (the activation quantiser)
        at[n_at].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n_at].val.programmaticStreamSerializationAllowed = 1;
        ++n_at;
    }
    cfg.attrs = n_at ? at : nullptr;
    cfg.numAttrs = n_at;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, outs, lmaps, p);
    if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "gemm_tcgen05_kernel launch: %s", cudaGetErrorString(e));
    return check_launch("gemm_tcgen05_kernel");
}

// Tile shape by problem shape: CTA pairs on 256 x 256 tiles when both extents
// are large, single CTAs with 128 x {256,128,64} tiles otherwise (LoRA ranks,
// short batches).
// Tile configuration of one GEMM: 1 pair 256 x 256, 2 single 128 x 256, 3 single 128 x 128, 4 single 128 x 64,
// 5 single 128 x 32; k_split 1 or 2 (two CTAs of a cluster share a tile's K range).
struct GemmPlan {
    int choice;
    int k_split;
};

// I8F_GEMM_TILE = pair256 | s256 | s128 | s64 | s32 forces one tile configuration (experiments);
// I8F_GEMM_SINGLE_CTA=1 is the older spelling of "never pair"; I8F_KSPLIT=0 switches the K split off.
int forced_tile() {
    static const int forced = [] {
        const char* e = getenv("I8F_GEMM_TILE");
        if (e != nullptr) {
            if (e[0] == 'p') return 1;
            if (e[0] == 's' && e[1] == '2') return 2;
            if (e[0] == 's' && e[1] == '1') return 3;
            if (e[0] == 's' && e[1] == '6') return 4;
            if (e[0] == 's' && e[1] == '3') return 6;
        }
        const char* f = getenv("I8F_GEMM_SINGLE_CTA");
        return (f != nullptr && f[0] == '1') ? 5 : 0;
    }();
    return forced;
}
bool ksplit_enabled() {
    static const int on = [] {
        const char* e = getenv("I8F_KSPLIT");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    return on != 0;
}

// Pure function of the shape, the SM count and the switches.  elem_bytes: 1 for int8 operands, 2 for the 16-bit kinds.
GemmPlan plan_gemm(int64_t M, int64_t N, int64_t K, int elem_bytes, int64_t sms, bool scatter, int forced, bool ksplit_on) {
    GemmPlan plan{0, 1};
    if ((forced >= 1 && forced <= 4) || forced == 6) {
        plan.choice = forced == 6 ? 5 : forced;
        return plan;
    }
    // Problems that do not fill the GPU with 256-wide tiles are bound by how many SMs work on them (one tile's K loop
    // costs the same whatever its width): take the configuration with the most CTAs that still fit one wave, and among
    // equals the one with the least padded work.  Everything larger runs the paired 256 x 256 tiles.  (Measured on
    // M = 17 .. 2048, N = 4096 / 12288, K = 4096.)
    const int64_t m128 = (M + 127) / 128, m256 = (M + 255) / 256;
    const int64_t ctas[6] = {0, 2 * m256 * ((N + 255) / 256), m128 * ((N + 255) / 256), m128 * ((N + 127) / 128),
                             m128 * ((N + 63) / 64), m128 * ((N + 31) / 32)};
    const int64_t work[6] = {0, m256 * 256 * ((N + 255) / 256) * 256, m128 * 128 * ((N + 255) / 256) * 256,
                             m128 * 128 * ((N + 127) / 128) * 128, m128 * 128 * ((N + 63) / 64) * 64,
                             m128 * 128 * ((N + 31) / 32) * 32};
    int choice = 0;
    for (int c = 1; c <= 5; ++c) {
        if (c == 1 && forced == 5) continue;
        if (c == 5 && scatter) continue;   // the scatter epilogue stores 64-column pieces
        if (ctas[c] > sms) continue;
        if (choice == 0 || ctas[c] > ctas[choice] || (ctas[c] == ctas[choice] && work[c] < work[choice])) choice = c;
    }
    if (choice == 0) choice = N > 128 ? ((M > 128 && forced != 5) ? 1 : 2) : (N > 64 ? 3 : 4);
    plan.choice = choice;
    // K split: when a single-CTA configuration leaves at least half of the SMs without a tile, two CTAs may share
    // each tile's K range.  Estimated cycles of one CTA, fitted to measurements on M = 17 .. 512, K = 3072 .. 12288:
    // K slabs x max(560 issue-and-tensor cycles, operand bytes at 72 B/clk), 1100 per 32-column chunk of the epilogue,
    // 3700 + 950 per chunk for the hand-over.  The split is taken when its best candidate is at least 7 % cheaper than
    // the best unsplit one.
    if (ksplit_on && !scatter && forced == 0) {
        const int64_t nkb = (K * elem_bytes + kStageRowBytes - 1) / kStageRowBytes;
        const int bn_of[6] = {0, 256, 256, 128, 64, 32};
        auto est = [&](int c, int split) -> int64_t {
            const int64_t chunks = bn_of[c] / 32;
            const int64_t slab_bytes = (c == 1 ? 16384 + 128 * 128 : 16384 + bn_of[c] * 128);
            const int64_t slab = slab_bytes / 72 > 560 ? slab_bytes / 72 : 560;
            return (nkb / split) * slab + chunks * 1100 + (split == 2 ? 3700 + chunks * 950 : 0);
        };
        int64_t best[3] = {0, -1, -1};
        int best_c = 0;
        for (int c = 1; c <= 5; ++c) {
            if (ctas[c] > sms) continue;
            for (int split = 1; split <= 2; ++split) {
                if (split == 2 && (c == 1 || 2 * ctas[c] > sms || nkb < 8)) continue;
                const int64_t e = est(c, split);
                if (best[split] < 0 || e < best[split]) {
                    best[split] = e;
                    if (split == 2) best_c = c;
                }
            }
        }
        if (best_c != 0 && best[2] >= 0 && best[1] >= 0 && best[2] * 100 < best[1] * 93) {
            plan.choice = best_c;
            plan.k_split = 2;
        }
    }
    return plan;
}

template <int KIND>
int launch_gemm_auto(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t M, int64_t N, int64_t K,
                     const GemmParams& p, cudaStream_t st, const Scatter* scatter = nullptr) {
    const GemmPlan plan = plan_gemm(M, N, K, KIND == kKindI8 ? 1 : 2, sm_count(), scatter != nullptr, forced_tile(), ksplit_enabled());
    const int k_split = plan.k_split;
    switch (plan.choice) {
        case 1: return launch_gemm<KIND, 256, true>(a, lda, b, ldb, M, N, K, p, st, scatter);
        case 2: return launch_gemm<KIND, 256, false>(a, lda, b, ldb, M, N, K, p, st, scatter, nullptr, k_split);
        case 3: return launch_gemm<KIND, 128, false>(a, lda, b, ldb, M, N, K, p, st, scatter, nullptr, k_split);
        case 5: return launch_gemm<KIND, 32, false>(a, lda, b, ldb, M, N, K, p, st, scatter, nullptr, k_split);
        default: return launch_gemm<KIND, 64, false>(a, lda, b, ldb, M, N, K, p, st, scatter, nullptr, k_split);
    }
}

int check_operands(const void* a, int64_t lda, const void* b, int64_t ldb, int esz, int64_t M, int64_t N, int64_t K) {
    I8F_REQUIRE(M > 0 && N > 0 && K > 0, I8F_ERR_INVALID_ARG, "empty problem M=%lld N=%lld K=%lld", (long long)M,
                (long long)N, (long long)K);
    I8F_REQUIRE(M < (1LL << 31) - 256 && N < (1LL << 31) - 256 && K < (1LL << 31) - 256, I8F_ERR_UNSUPPORTED,
                "dimension too large");
    I8F_REQUIRE(a != nullptr && b != nullptr, I8F_ERR_INVALID_ARG, "NULL operand");
    I8F_REQUIRE(lda >= K && ldb >= K, I8F_ERR_INVALID_ARG, "operand pitch smaller than K");
    I8F_REQUIRE(aligned16(a) && aligned16(b), I8F_ERR_ALIGNMENT, "operands must be 16-byte aligned (TMA)");
    I8F_REQUIRE((lda * esz) % 16 == 0 && (ldb * esz) % 16 == 0, I8F_ERR_ALIGNMENT,
                "operand row pitch must be a multiple of 16 bytes (TMA): lda=%lld ldb=%lld elem=%d", (long long)lda,
                (long long)ldb, esz);
    return I8F_OK;
}

}  // namespace
}  // namespace i8f

using namespace i8f;

extern "C" {

int i8f_gemm_plan(int64_t M, int64_t N, int64_t K, int elem_bytes, int sm_count_or_0, int* tile_rows, int* tile_cols,
                  int* ctas_per_tile, int* k_split) {
    I8F_REQUIRE(M > 0 && N > 0 && K > 0 && (elem_bytes == 1 || elem_bytes == 2), I8F_ERR_INVALID_ARG, "bad shape or element size");
    I8F_REQUIRE(tile_rows != nullptr && tile_cols != nullptr && ctas_per_tile != nullptr && k_split != nullptr, I8F_ERR_INVALID_ARG,
                "NULL output pointer");
    const GemmPlan plan = plan_gemm(M, N, K, elem_bytes, sm_count_or_0 > 0 ? sm_count_or_0 : sm_count(), false, 0, true);
    const int rows_of[6] = {0, 256, 128, 128, 128, 128}, cols_of[6] = {0, 256, 256, 128, 64, 32};
    *tile_rows = rows_of[plan.choice];
    *tile_cols = cols_of[plan.choice];
    *k_split = plan.k_split;
    *ctas_per_tile = (plan.choice == 1 ? 2 : 1) * plan.k_split;
    return I8F_OK;
}

int i8f_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
    I8F_REQUIRE(limit_cycles > 0 && limit_cycles <= 4000000000LL, I8F_ERR_INVALID_ARG, "limit_cycles out of range");
    int* status = device_status_word();
    I8F_REQUIRE(status != nullptr, I8F_ERR_CUDA, "device status word unavailable");
    bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_cycles);
    return check_launch("bounded_wait_selftest_kernel");
}

int i8f_gemm_i8_i32(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw, int32_t* acc, int64_t ldacc, int64_t M,
                    int64_t N, int64_t K, void* stream) {
    int rc = check_operands(a, lda, w, ldw, 1, M, N, K);
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(acc != nullptr && ldacc >= N, I8F_ERR_INVALID_ARG, "bad accumulator output");
    GemmParams p{};
    p.out = acc;
    p.ldo = ldacc;
    p.epi_mode = kEpiI32;
    p.vec_ok = aligned16(acc) && (ldacc % 4 == 0);
    return launch_gemm_auto<kKindI8>(a, lda, w, ldw, M, N, K, p, static_cast<cudaStream_t>(stream));
}

static int linear_w8a8_impl(const int8_t* a, int64_t lda, const float* a_scale, const int8_t* w, int64_t ldw,
                            const float* w_scale, int w_scale_mode, const void* bias, int bias_dtype, void* out,
                            int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K, int epilogue_order,
                            int add_existing, void* stream, const Scatter* scatter = nullptr, const void* gate = nullptr) {
    int rc = check_operands(a, lda, w, ldw, 1, M, N, K);
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(a_scale != nullptr && w_scale != nullptr, I8F_ERR_INVALID_ARG, "NULL scale pointer");
    I8F_REQUIRE(w_scale_mode == I8F_WSCALE_TENSOR || w_scale_mode == I8F_WSCALE_CHANNEL, I8F_ERR_INVALID_ARG,
                "unknown w_scale_mode %d", w_scale_mode);
    I8F_REQUIRE(out != nullptr && ldo >= N, I8F_ERR_INVALID_ARG, "bad output");
    I8F_REQUIRE(out_dtype == I8F_BF16 || out_dtype == I8F_F16, I8F_ERR_UNSUPPORTED, "out_dtype must be bf16 or f16");
    I8F_REQUIRE(bias == nullptr || dtype_size(bias_dtype) != 0, I8F_ERR_INVALID_ARG, "unknown bias dtype %d", bias_dtype);
    I8F_REQUIRE(epilogue_order == I8F_EPI_PYTORCH || epilogue_order == I8F_EPI_SINGLE, I8F_ERR_INVALID_ARG,
                "unknown epilogue_order %d", epilogue_order);
    GemmParams p{};
    p.out = out;
    p.ldo = ldo;
    p.out_dtype = out_dtype;
    p.a_scale = a_scale;
    p.w_scale = w_scale;
    p.w_scale_mode = w_scale_mode;
    p.bias = bias;
    p.bias_dtype = bias_dtype;
    p.epi_mode = kEpiDequant;
    p.epi_order = epilogue_order;
    p.add_existing = add_existing;
    p.gate = gate;
    p.vec_ok = aligned16(out) && (ldo % 8 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    return launch_gemm_auto<kKindI8>(a, lda, w, ldw, M, N, K, p, st, scatter);
}

int i8f_linear_w8a8(const int8_t* a, int64_t lda, const float* a_scale, const int8_t* w, int64_t ldw,
                    const float* w_scale, int w_scale_mode, const void* bias, int bias_dtype, void* out, int out_dtype,
                    int64_t ldo, int64_t M, int64_t N, int64_t K, int epilogue_order, void* stream) {
    return linear_w8a8_impl(a, lda, a_scale, w, ldw, w_scale, w_scale_mode, bias, bias_dtype, out, out_dtype, ldo, M, N, K,
                            epilogue_order, 0, stream);
}

int i8f_linear_w8a8_add(const int8_t* a, int64_t lda, const float* a_scale, const int8_t* w, int64_t ldw,
                        const float* w_scale, int w_scale_mode, const void* bias, int bias_dtype, void* out,
                        int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K, int epilogue_order, void* stream) {
    return linear_w8a8_impl(a, lda, a_scale, w, ldw, w_scale, w_scale_mode, bias, bias_dtype, out, out_dtype, ldo, M, N, K,
                            epilogue_order, 1, stream);
}

int i8f_linear_w8a8_gated_add(const int8_t* a, int64_t lda, const float* a_scale, const int8_t* w, int64_t ldw,
                              const float* w_scale, int w_scale_mode, const void* bias, int bias_dtype, const void* gate,
                              void* out, int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream) {
    I8F_REQUIRE(gate != nullptr, I8F_ERR_INVALID_ARG, "gate is NULL");
    return linear_w8a8_impl(a, lda, a_scale, w, ldw, w_scale, w_scale_mode, bias, bias_dtype, out, out_dtype, ldo, M, N, K,
                            I8F_EPI_PYTORCH, 1, stream, nullptr, gate);
}

int i8f_linear_w8a8_lora(const int8_t* a, int64_t lda, const float* a_scale, const int8_t* w, int64_t ldw,
                         const float* w_scale, int w_scale_mode, const void* bias, int bias_dtype, const void* t, int64_t ldt,
                         const void* lora_b, int64_t ldb, int64_t r, void* out, int out_dtype, int64_t ldo, int64_t M,
                         int64_t N, int64_t K, int epilogue_order, void* stream) {
    I8F_REQUIRE(out_dtype == I8F_BF16 || out_dtype == I8F_F16, I8F_ERR_UNSUPPORTED, "out_dtype must be bf16 or f16");
    if (r <= 0)
        return i8f_linear_w8a8(a, lda, a_scale, w, ldw, w_scale, w_scale_mode, bias, bias_dtype, out, out_dtype, ldo, M, N, K,
                               epilogue_order, stream);
    I8F_REQUIRE(t != nullptr && lora_b != nullptr && ldt >= r && ldb >= r, I8F_ERR_INVALID_ARG, "bad low-rank operands");
    static const int no_fuse = [] {
        const char* e = getenv("I8F_LORA_UNFUSED");
        return (e != nullptr && e[0] == '1') ? 1 : 0;
    }();
    const bool fused = M > 128 && N > 128 && !no_fuse;
    if (!fused) {
        // small shapes: the low-rank term is stored first, the int8 GEMM adds onto it in its epilogue
        int rc0 = i8f_lora_up(t, ldt, lora_b, ldb, out, ldo, out_dtype, M, N, r, stream);
        if (rc0 != I8F_OK) return rc0;
        return i8f_linear_w8a8_add(a, lda, a_scale, w, ldw, w_scale, w_scale_mode, bias, bias_dtype, out, out_dtype, ldo, M, N,
                                   K, epilogue_order, stream);
    }
    int rc = check_operands(a, lda, w, ldw, 1, M, N, K);
    if (rc != I8F_OK) return rc;
    rc = check_operands(t, ldt, lora_b, ldb, 2, M, N, r);
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(a_scale != nullptr && w_scale != nullptr, I8F_ERR_INVALID_ARG, "NULL scale pointer");
    I8F_REQUIRE(w_scale_mode == I8F_WSCALE_TENSOR || w_scale_mode == I8F_WSCALE_CHANNEL, I8F_ERR_INVALID_ARG,
                "unknown w_scale_mode %d", w_scale_mode);
    I8F_REQUIRE(out != nullptr && ldo >= N, I8F_ERR_INVALID_ARG, "bad output");
    I8F_REQUIRE(bias == nullptr || dtype_size(bias_dtype) != 0, I8F_ERR_INVALID_ARG, "unknown bias dtype %d", bias_dtype);
    I8F_REQUIRE(epilogue_order == I8F_EPI_PYTORCH || epilogue_order == I8F_EPI_SINGLE, I8F_ERR_INVALID_ARG,
                "unknown epilogue_order %d", epilogue_order);
    GemmParams p{};
    p.out = out;
    p.ldo = ldo;
    p.out_dtype = out_dtype;
    p.a_scale = a_scale;
    p.w_scale = w_scale;
    p.w_scale_mode = w_scale_mode;
    p.bias = bias;
    p.bias_dtype = bias_dtype;
    p.epi_mode = kEpiDequant;
    p.epi_order = epilogue_order;
    p.vec_ok = aligned16(out) && (ldo % 8 == 0);
    const LoraOperands lo{t, ldt, lora_b, ldb, r, out_dtype == I8F_BF16 ? kKindBF16 : kKindF16};
    // tile width of the fused kernel: 256 (one int32 accumulator buffer, full-rate tile; default), 160 (double-buffered
    // accumulators, narrower tile) or 128; I8F_LORA_BN selects the others for comparison
    static const int bn = [] {
        const char* e = getenv("I8F_LORA_BN");
        const int v = e != nullptr ? atoi(e) : 256;
        return (v == 128 || v == 160) ? v : 256;
    }();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (bn == 160) return launch_gemm<kKindI8, 160, true, true>(a, lda, w, ldw, M, N, K, p, st, nullptr, &lo);
    if (bn == 128) return launch_gemm<kKindI8, 128, true, true>(a, lda, w, ldw, M, N, K, p, st, nullptr, &lo);
    return launch_gemm<kKindI8, 256, true, true>(a, lda, w, ldw, M, N, K, p, st, nullptr, &lo);
}

int i8f_linear_w8a8_scatter(const int8_t* a, int64_t lda, const float* a_scale, const int8_t* w, int64_t ldw,
                            const float* w_scale, int w_scale_mode, const void* bias, int bias_dtype, void* const* dests,
                            int n_dests, int64_t ld_dest, int64_t n_total, int64_t col_offset, int out_dtype, int64_t M,
                            int64_t N, int64_t K, int epilogue_order, void* stream) {
    I8F_REQUIRE(dests != nullptr && n_dests >= 1 && n_dests <= kMaxOutputs, I8F_ERR_INVALID_ARG,
                "n_dests must be 1..%d", kMaxOutputs);
    I8F_REQUIRE(N % 32 == 0, I8F_ERR_UNSUPPORTED,
                "the block width N=%lld must be a multiple of 32 (a partial chunk would spill into the neighbour's columns)",
                (long long)N);
    I8F_REQUIRE(col_offset >= 0 && col_offset % 8 == 0 && col_offset + N <= n_total && ld_dest >= n_total && ld_dest % 8 == 0,
                I8F_ERR_INVALID_ARG, "bad destination geometry: col_offset=%lld N=%lld n_total=%lld ld=%lld",
                (long long)col_offset, (long long)N, (long long)n_total, (long long)ld_dest);
    for (int d = 0; d < n_dests; ++d)
        I8F_REQUIRE(dests[d] != nullptr && aligned16(dests[d]), I8F_ERR_ALIGNMENT, "destination %d is NULL or not 16-byte aligned", d);
    const Scatter sc{dests, n_dests, n_total, ld_dest, col_offset};
    // `out` / `ldo` of the ordinary path are only used for validation here: point them at the first destination
    return linear_w8a8_impl(a, lda, a_scale, w, ldw, w_scale, w_scale_mode, bias, bias_dtype, dests[0], out_dtype, ld_dest, M,
                            N, K, epilogue_order, 0, stream, &sc);
}

size_t i8f_linear_workspace_bytes(int64_t M, int64_t K) {
    if (M <= 0 || K <= 0) return 0;
    const size_t q = (static_cast<size_t>(M) * static_cast<size_t>(K) + 255) & ~static_cast<size_t>(255);
    const size_t s = (static_cast<size_t>(M) * sizeof(float) + 255) & ~static_cast<size_t>(255);
    return q + s;
}

int i8f_linear_forward(const void* x, int x_dtype, int64_t ldx, int hadamard128, const int8_t* w, int64_t ldw,
                       const float* w_scale, int w_scale_mode, const void* bias, int bias_dtype, void* out,
                       int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K, int epilogue_order, void* workspace,
                       size_t workspace_bytes, void* stream) {
    I8F_REQUIRE(M > 0 && N > 0 && K > 0, I8F_ERR_INVALID_ARG, "empty problem");
    I8F_REQUIRE(K % 16 == 0, I8F_ERR_ALIGNMENT, "K=%lld must be a multiple of 16", (long long)K);
    const size_t need = i8f_linear_workspace_bytes(M, K);
    I8F_REQUIRE(workspace != nullptr && workspace_bytes >= need, I8F_ERR_WORKSPACE,
                "workspace too small: have %zu bytes, need %zu", workspace_bytes, need);
    I8F_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, I8F_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
    int8_t* q = static_cast<int8_t*>(workspace);
    float* xs = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ((static_cast<size_t>(M) * K + 255) & ~size_t(255)));
    int rc = i8f_quant_rowwise(x, x_dtype, M, K, ldx, q, K, xs, hadamard128, nullptr, stream);
    if (rc != I8F_OK) return rc;
    return i8f_linear_w8a8(q, K, xs, w, ldw, w_scale, w_scale_mode, bias, bias_dtype, out, out_dtype, ldo, M, N, K,
                           epilogue_order, stream);
}

int i8f_lora_down(const void* x, int64_t ldx, const void* lora_a, int64_t lda, void* t, int64_t ldt, int dtype, int64_t M,
                  int64_t K, int64_t r, void* stream) {
    I8F_REQUIRE(dtype == I8F_BF16 || dtype == I8F_F16, I8F_ERR_UNSUPPORTED, "dtype must be bf16 or f16");
    int rc = check_operands(x, ldx, lora_a, lda, 2, M, r, K);
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(t != nullptr && ldt >= r, I8F_ERR_INVALID_ARG, "bad output");
    GemmParams p{};
    p.out = t;
    p.ldo = ldt;
    p.out_dtype = dtype;
    p.epi_mode = kEpiCast;
    p.vec_ok = aligned16(t) && (ldt % 8 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == I8F_BF16) return launch_gemm_auto<kKindBF16>(x, ldx, lora_a, lda, M, r, K, p, st);
    return launch_gemm_auto<kKindF16>(x, ldx, lora_a, lda, M, r, K, p, st);
}

int i8f_lora_up(const void* t, int64_t ldt, const void* lora_b, int64_t ldb, void* y, int64_t ldy, int dtype, int64_t M,
                int64_t N, int64_t r, void* stream) {
    I8F_REQUIRE(dtype == I8F_BF16 || dtype == I8F_F16, I8F_ERR_UNSUPPORTED, "dtype must be bf16 or f16");
    int rc = check_operands(t, ldt, lora_b, ldb, 2, M, N, r);
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(y != nullptr && ldy >= N, I8F_ERR_INVALID_ARG, "bad output");
    GemmParams p{};
    p.out = y;
    p.ldo = ldy;
    p.out_dtype = dtype;
    p.epi_mode = kEpiCast;
    p.vec_ok = aligned16(y) && (ldy % 8 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == I8F_BF16) return launch_gemm_auto<kKindBF16>(t, ldt, lora_b, ldb, M, N, r, p, st);
    return launch_gemm_auto<kKindF16>(t, ldt, lora_b, ldb, M, N, r, p, st);
}

int i8f_lora_up_add(const void* t, int64_t ldt, const void* lora_b, int64_t ldb, void* y, int64_t ldy, int dtype,
                    int64_t M, int64_t N, int64_t r, void* stream) {
    I8F_REQUIRE(dtype == I8F_BF16 || dtype == I8F_F16, I8F_ERR_UNSUPPORTED, "dtype must be bf16 or f16");
    int rc = check_operands(t, ldt, lora_b, ldb, 2, M, N, r);
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(y != nullptr && ldy >= N, I8F_ERR_INVALID_ARG, "bad output");
    GemmParams p{};
    p.out = y;
    p.ldo = ldy;
    p.out_dtype = dtype;
    p.epi_mode = kEpiAccum;
    p.vec_ok = aligned16(y) && (ldy % 8 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == I8F_BF16) return launch_gemm_auto<kKindBF16>(t, ldt, lora_b, ldb, M, N, r, p, st);
    return launch_gemm_auto<kKindF16>(t, ldt, lora_b, ldb, M, N, r, p, st);
}

}  // extern "C"

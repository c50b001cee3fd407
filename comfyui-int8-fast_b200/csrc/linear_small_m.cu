// Linear layer for M <= 16 tokens on int8 weights: y = x . dt(w * scale)^T + dt(bias).
//
// The node pack's Linear does not quantise the activations of tiny batches (modulation and embedding sized
// calls): it dequantises the whole weight matrix to the activation dtype and calls a float matmul
// (int8_quant.py:756-760), i.e. reads N*K int8, writes and re-reads N*K 16-bit values every call.  This
// kernel computes the same expression in one pass over the int8 weights: HBM-bound on N*K bytes.
//
// Work split: a CTA of 8 warps owns 16 consecutive output features; the warps split K in interleaved
// 64-element chunks and their partial sums meet in shared memory in a fixed order (deterministic).
// Inside a warp the product runs on mma.sync.m16n8k16 (sixteen weight rows as the A operand, up to eight
// tokens of x as B), which leaves the issue slots to the dequantisation: byte -> fp32 by a byte permute into the
// mantissa of 2^23 and one exact subtraction, one fp32 multiply by the scale (the reference's
// `w.float() * scale`), one packed conversion to the 16-bit dtype (its `.to(x.dtype)`).
// A lane loads 16 consecutive weights of one row with one 128-bit load; the k index inside the MMA is a
// permutation of the real one (lane t of a quad supplies real k = 16 t + 4 j + {0,1,2,3} to MMA j), applied to
// x and w alike, so the sum is unchanged.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"

namespace i8f {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxSmallM = 16;

template <int DT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (DT == I8F_BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    } else {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
}

template <int DT>
__device__ __forceinline__ float round_dt(float v) {
    if constexpr (DT == I8F_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    else return __half2float(__float2half_rn(v));
}

template <int DT>
__device__ __forceinline__ void store_dt(void* out, int64_t idx, float v) {
    if constexpr (DT == I8F_BF16) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
    else static_cast<__half*>(out)[idx] = __float2half_rn(v);
}

__device__ __forceinline__ float load_bias(const void* bias, int bias_dt, int64_t n) {
    if (bias_dt == I8F_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
    if (bias_dt == I8F_F16) return __half2float(static_cast<const __half*>(bias)[n]);
    return static_cast<const float*>(bias)[n];
}

// Four int8 in a word -> two packed 16-bit pairs of dt(fp32(w) * s).
template <int DT>
__device__ __forceinline__ void dequant4(uint32_t word, float s, uint32_t& lo, uint32_t& hi) {
    constexpr uint32_t kTwo23 = 0x4B000000u;      // 2^23: its low mantissa byte receives w + 128
    constexpr float kOffset = 8388736.0f;         // 2^23 + 128
    const uint32_t u = word ^ 0x80808080u;
    const float f0 = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(u, kTwo23, 0x7440)), kOffset), s);
    const float f1 = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(u, kTwo23, 0x7441)), kOffset), s);
    const float f2 = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(u, kTwo23, 0x7442)), kOffset), s);
    const float f3 = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(u, kTwo23, 0x7443)), kOffset), s);
    lo = pack2<DT>(f0, f1);
    hi = pack2<DT>(f2, f3);
}

template <int DT>
__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    if constexpr (DT == I8F_BF16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// 16 activations of up to two tokens per lane for one 64-element K chunk.
struct XFrag {
    uint4 a[2], b[2];
};

template <bool HI_ROWS>
__device__ __forceinline__ void load_x(XFrag& f, const uint16_t* xap, const uint16_t* xbp, int off) {
    f.a[0] = __ldg(reinterpret_cast<const uint4*>(xap + off));
    f.a[1] = __ldg(reinterpret_cast<const uint4*>(xap + off) + 1);
    if constexpr (HI_ROWS) {
        f.b[0] = __ldg(reinterpret_cast<const uint4*>(xbp + off));
        f.b[1] = __ldg(reinterpret_cast<const uint4*>(xbp + off) + 1);
    }
}

// The weights are the A operand (16 features x 16 k, built in registers by the dequantisation, so the four
// registers of a fragment need no shuffling), the activations the B operand (16 k x 8 tokens, whose register
// pairs are consecutive words of the 128-bit loads).
template <int DT, bool HI_ROWS>
__device__ __forceinline__ void consume_chunk(const uint4& wlo, const uint4& whi, const XFrag& x, float sc_lo, float sc_hi,
                                              float (&acc)[HI_ROWS ? 2 : 1][4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t a0, a1, a2, a3;
        dequant4<DT>(word_of(wlo, j), sc_lo, a0, a2);
        dequant4<DT>(word_of(whi, j), sc_hi, a1, a3);
        // x words 2j and 2j+1 of the lane's 8 (two elements each) = real k 4j..4j+3
        mma_16x8x16<DT>(acc[0], a0, a1, a2, a3, word_of(x.a[j >> 1], (2 * j) & 3), word_of(x.a[j >> 1], (2 * j + 1) & 3));
        if constexpr (HI_ROWS)
            mma_16x8x16<DT>(acc[1], a0, a1, a2, a3, word_of(x.b[j >> 1], (2 * j) & 3), word_of(x.b[j >> 1], (2 * j + 1) & 3));
    }
}


// DT: dtype of x and out.  HI_ROWS: M > 8 (a second MMA per fragment covers tokens 8..15).
//
// A CTA owns 16 consecutive output features; lane (g, t) of every warp reads features g and g+8.  Features and
// tokens are independent in the accumulator, so lanes whose feature or token is past the end read a valid
// stand-in (the last feature / token 0) instead of carrying predicates; those results are never stored.
// kDepth: weight chunks in flight per lane (a register ring); the activations (L1/L2 hits) are fetched per chunk.
template <int DT, bool HI_ROWS, int kDepth>
__global__ void __launch_bounds__(kThreads, HI_ROWS ? 3 : 4)
small_m_kernel(const void* __restrict__ x, int64_t ldx, const int8_t* __restrict__ w, int64_t ldw,
               const float* __restrict__ w_scale, int per_row, const void* __restrict__ bias, int bias_dt,
               void* __restrict__ out, int64_t ldo, int M, int64_t N, int64_t K) {
    constexpr int kHalves = HI_ROWS ? 2 : 1;
    __shared__ float4 s_part[2][kWarps][kHalves][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n_blocks = (N + 15) / 16;
    const int64_t full_chunks = K / 64;
    const int my_chunks = warp < full_chunks ? static_cast<int>((full_chunks - warp + kWarps - 1) / kWarps) : 0;
    const bool has_tail = (K % 64) != 0 && warp == static_cast<int>(full_chunks % kWarps);
    const uint16_t* xp = static_cast<const uint16_t*>(x);
    const uint16_t* xa0 = xp + static_cast<int64_t>(g < M ? g : 0) * ldx + t * 16;
    const uint16_t* xb0 = xp + static_cast<int64_t>(g + 8 < M ? g + 8 : 0) * ldx + t * 16;
    constexpr int kStride = kWarps * 64;   // bytes of weights (elements of x) between a warp's chunks

    // Per-lane pointers of a feature block: features g and g+8, this lane's 16-byte column, this warp's first chunk.
    const int8_t *row_lo, *row_hi;
    float sc_lo, sc_hi;
    uint4 ring_lo[kDepth], ring_hi[kDepth];
    auto open_block = [&](int64_t nb, float& s_lo, float& s_hi) {
        int64_t n_lo = nb * 16 + g, n_hi = n_lo + 8;
        n_lo = n_lo < N ? n_lo : N - 1;
        n_hi = n_hi < N ? n_hi : N - 1;
        row_lo = w + n_lo * ldw + t * 16;
        row_hi = w + n_hi * ldw + t * 16;
#pragma unroll
        for (int s = 0; s < kDepth; ++s) {
            if (s < my_chunks) {
                ring_lo[s] = __ldg(reinterpret_cast<const uint4*>(row_lo + warp * 64 + s * kStride));
                ring_hi[s] = __ldg(reinterpret_cast<const uint4*>(row_hi + warp * 64 + s * kStride));
            }
        }
        s_lo = per_row ? __ldg(w_scale + n_lo) : __ldg(w_scale);
        s_hi = per_row ? __ldg(w_scale + n_hi) : s_lo;
    };

    int64_t nb = blockIdx.x;          // the grid never exceeds the number of blocks
    open_block(nb, sc_lo, sc_hi);
    for (int iter = 0;; ++iter) {
        float acc[kHalves][4];
#pragma unroll
        for (int h = 0; h < kHalves; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.0f;
        const int8_t* wlo = row_lo + warp * 64;
        const int8_t* whi = row_hi + warp * 64;
        const uint16_t* xap = xa0 + warp * 64;
        const uint16_t* xbp = xb0 + warp * 64;

        for (int base = 0; base < my_chunks; base += kDepth) {
#pragma unroll
            for (int s = 0; s < kDepth; ++s) {
                const int i = base + s;
                if (i < my_chunks) {   // warp-uniform
                    XFrag xf;
                    load_x<HI_ROWS>(xf, xap, xbp, s * kStride);
                    consume_chunk<DT, HI_ROWS>(ring_lo[s], ring_hi[s], xf, sc_lo, sc_hi, acc);
                    if (i + kDepth < my_chunks) {
                        ring_lo[s] = __ldg(reinterpret_cast<const uint4*>(wlo + (s + kDepth) * kStride));
                        ring_hi[s] = __ldg(reinterpret_cast<const uint4*>(whi + (s + kDepth) * kStride));
                    }
                }
            }
            wlo += kDepth * kStride;
            whi += kDepth * kStride;
            xap += kDepth * kStride;
            xbp += kDepth * kStride;
        }
        if (has_tail) {   // warp-uniform.  K is a multiple of 16, so a lane's 16 elements are all inside or all outside
            const int k0 = static_cast<int>(full_chunks * 64);
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            uint4 tlo = z, thi = z;
            XFrag xf;
            xf.a[0] = xf.a[1] = xf.b[0] = xf.b[1] = z;
            if (k0 + t * 16 < K) {
                tlo = __ldg(reinterpret_cast<const uint4*>(row_lo + k0));
                thi = __ldg(reinterpret_cast<const uint4*>(row_hi + k0));
                load_x<HI_ROWS>(xf, xa0, xb0, k0);
            }
            // every lane of the warp executes the MMAs (mma.sync is a warp-wide operation); lanes past K feed zeros
            consume_chunk<DT, HI_ROWS>(tlo, thi, xf, sc_lo, sc_hi, acc);
        }

        // the next block's first weights are in flight while this block's partial sums meet
        const int64_t nb_next = nb + gridDim.x;
        float next_lo = 0.0f, next_hi = 0.0f;
        if (nb_next < n_blocks) open_block(nb_next, next_lo, next_hi);

        // s_part is double-buffered, so one barrier per block is enough: a buffer is rewritten two blocks later, and
        // every warp has passed the barrier in between only after the reader of the older block was done with it
        const int buf = iter & 1;
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
            s_part[buf][warp][h][lane] = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
        __syncthreads();
        const int first = (iter * kHalves) % kWarps;     // the summing duty rotates over the warps
        if (warp >= first && warp < first + kHalves) {
            const int h = warp - first;
            float4 s = s_part[buf][0][h][lane];
#pragma unroll
            for (int r = 1; r < kWarps; ++r) {
                const float4 p = s_part[buf][r][h][lane];
                s.x = __fadd_rn(s.x, p.x); s.y = __fadd_rn(s.y, p.y); s.z = __fadd_rn(s.z, p.z); s.w = __fadd_rn(s.w, p.w);
            }
            // accumulator fragment: (feature g, tokens 2t, 2t+1) and (feature g+8, same tokens)
            const float v[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int m = h * 8 + 2 * t + (e & 1);
                const int64_t n = nb * 16 + g + (e >> 1) * 8;
                if (m < M && n < N) {
                    const float b = bias != nullptr ? round_dt<DT>(load_bias(bias, bias_dt, n)) : 0.0f;
                    store_dt<DT>(out, static_cast<int64_t>(m) * ldo + n, __fadd_rn(v[e], b));
                }
            }
        }
        if (nb_next >= n_blocks) break;
        nb = nb_next;
        sc_lo = next_lo;
        sc_hi = next_hi;
    }
}

template <int DT>
int dispatch_small(const void* x, int64_t ldx, const int8_t* w, int64_t ldw, const float* w_scale, int per_row,
                   const void* bias, int bias_dt, void* out, int64_t ldo, int M, int64_t N, int64_t K,
                   cudaStream_t stream) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t blocks = (N + 15) / 16;
    const bool hi = M > 8;
    auto kernel = hi ? small_m_kernel<DT, true, 2> : small_m_kernel<DT, false, 2>;
    // persistent: as many CTAs as are resident at once, each walking feature blocks with a grid stride
    static int s_resident[2][2] = {};
    int& per_sm = s_resident[DT == I8F_BF16 ? 0 : 1][hi ? 1 : 0];
    if (per_sm == 0) {
        int occ = 0;
        const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, kThreads, 0);
        if (e != cudaSuccess || occ < 1) return fail(I8F_ERR_CUDA, "small_m_kernel does not fit an SM");
        per_sm = occ;
    }
    const int64_t resident = static_cast<int64_t>(per_sm) * sms;
    const int grid = static_cast<int>(blocks < resident ? blocks : resident);
    kernel<<<grid, kThreads, 0, stream>>>(x, ldx, w, ldw, w_scale, per_row, bias, bias_dt, out, ldo, M, N, K);
    return check_launch("small_m_kernel");
}

}  // namespace
}  // namespace i8f

extern "C" int i8f_linear_w8a16_small(const void* x, int x_dtype, int64_t ldx, const int8_t* w, int64_t ldw,
                                      const float* w_scale, int w_scale_mode, const void* bias, int bias_dtype,
                                      void* out, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream_) {
    using namespace i8f;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    I8F_REQUIRE(x != nullptr && w != nullptr && w_scale != nullptr && out != nullptr, I8F_ERR_INVALID_ARG,
                "x, w, w_scale and out must not be NULL");
    I8F_REQUIRE(x_dtype == I8F_BF16 || x_dtype == I8F_F16, I8F_ERR_UNSUPPORTED, "x_dtype must be bf16 or fp16");
    I8F_REQUIRE(w_scale_mode == I8F_WSCALE_TENSOR || w_scale_mode == I8F_WSCALE_CHANNEL, I8F_ERR_INVALID_ARG,
                "w_scale_mode must be I8F_WSCALE_TENSOR or I8F_WSCALE_CHANNEL");
    I8F_REQUIRE(bias == nullptr || dtype_size(bias_dtype) != 0, I8F_ERR_INVALID_ARG, "unknown bias_dtype %d", bias_dtype);
    I8F_REQUIRE(M >= 0 && M <= kMaxSmallM, I8F_ERR_UNSUPPORTED, "M = %lld: this entry point takes at most %d rows",
                static_cast<long long>(M), kMaxSmallM);
    I8F_REQUIRE(N >= 0 && K >= 0, I8F_ERR_INVALID_ARG, "negative size");
    I8F_REQUIRE(ldx >= K && ldw >= K && ldo >= N, I8F_ERR_INVALID_ARG, "a pitch is smaller than its row");
    I8F_REQUIRE(K % 16 == 0 && ldw % 16 == 0 && ldx % 8 == 0 && aligned16(x) && aligned16(w), I8F_ERR_ALIGNMENT,
                "K and ldw must be multiples of 16, ldx of 8, x and w 16-byte aligned");
    if (M == 0 || N == 0) return I8F_OK;
    const int per_row = w_scale_mode == I8F_WSCALE_CHANNEL;
    if (x_dtype == I8F_BF16)
        return dispatch_small<I8F_BF16>(x, ldx, w, ldw, w_scale, per_row, bias, bias_dtype, out, ldo, static_cast<int>(M), N,
                                        K, stream);
    return dispatch_small<I8F_F16>(x, ldx, w, ldw, w_scale, per_row, bias, bias_dtype, out, ldo, static_cast<int>(M), N, K,
                                   stream);
}

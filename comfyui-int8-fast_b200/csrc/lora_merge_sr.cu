// Stochastic-rounding merge of a low-rank update into int8 weights.
//
// A CTA owns one 128-column block of K (so the optional Hadamard rotation of
// the delta is CTA-local) and walks down a band of rows, 32 rows at a time.
// The [r x 128] slice of `down` is staged once in shared memory as fp32; each
// thread accumulates a 2 x 8 patch of the delta in registers with the rank
// index ascending (acc = acc + up*down, separate multiply and add, which fixes
// the fp32 rounding), then scales, rotates, divides by the weight scale,
// rounds stochastically and adds into the int8 weights.  The only HBM
// traffic is the weights (read + write), the factors and, if supplied, the
// uniforms.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"

namespace i8f {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerIter = 32;
constexpr float kNormF32 = 0.088388346135616302f;

__device__ __forceinline__ float load_f(const void* p, int dt, long long i) {
    if (dt == I8F_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    if (dt == I8F_F16) return __half2float(static_cast<const __half*>(p)[i]);
    return static_cast<const float*>(p)[i];
}

// Philox4x32-10, counter (c0, c1, 0, 0).  The ten round keys (key + i * Weyl constants) depend on the seed only;
// the host computes them once and they reach the kernel as launch parameters (constant bank operands).
struct PhiloxKeys {
    uint32_t k0[10], k1[10];
};

inline PhiloxKeys make_philox_keys(unsigned long long seed) {
    PhiloxKeys k;
    uint32_t a = static_cast<uint32_t>(seed), b = static_cast<uint32_t>(seed >> 32);
    for (int i = 0; i < 10; ++i) {
        k.k0[i] = a;
        k.k1[i] = b;
        a += 0x9E3779B9u;
        b += 0xBB67AE85u;
    }
    return k;
}

__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, const PhiloxKeys& key) {
    uint32_t x0 = c0, x1 = c1, x2 = 0u, x3 = 0u;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const unsigned long long p0 = static_cast<unsigned long long>(0xD2511F53u) * x0;   // one wide multiply each
        const unsigned long long p1 = static_cast<unsigned long long>(0xCD9E8D57u) * x2;
        const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ x1 ^ key.k0[i];
        const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ x3 ^ key.k1[i];
        x0 = n0; x1 = static_cast<uint32_t>(p1); x2 = n2; x3 = static_cast<uint32_t>(p0);
    }
    return make_uint4(x0, x1, x2, x3);
}
// Uniform in [0, 1) from 16 random bits: exactly representable, below 1.  One Philox block (four 32-bit words) thus
// serves EIGHT weights; the generator is the largest single cost of the merge, and 2^-16 is far below the resolution
// at which a rounding probability matters for weights that move by whole int8 steps.
__device__ __forceinline__ float u01_16(uint32_t h) { return static_cast<float>(h) * 1.52587890625e-5f; }
__device__ __forceinline__ void uniforms8(const uint4& r, float (&u)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        u[2 * i] = u01_16(w[i] & 0xFFFFu);
        u[2 * i + 1] = u01_16(w[i] >> 16);
    }
}

// floor(x/ws) + [u < frac], clamped to int8 range.  The IEEE division, floorf and the float->int conversion are
// kept on purpose: a reciprocal-and-correct division and a magic-number floor were measured 1 - 3 % SLOWER here,
// because they move work from the conversion pipe onto the ALU/FMA pipes this kernel already saturates.
__device__ __forceinline__ int sr_round(float delta, float ws, float u) {
    const float xs = __fdiv_rn(delta, ws);
    const float fl = floorf(xs);
    const float fr = __fsub_rn(xs, fl);
    const float r = (u < fr) ? __fadd_rn(fl, 1.0f) : fl;
    return static_cast<int>(fminf(fmaxf(r, -128.0f), 127.0f));
}

__device__ __forceinline__ void wht128_lanes16(float (&v)[8], int lane) {
#pragma unroll
    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if ((i & h) == 0) {
                const float a = v[i], b = v[i + h];
                v[i] = __fadd_rn(a, b);
                v[i + h] = __fsub_rn(a, b);
            }
#pragma unroll
    for (int d = 1; d < 16; d <<= 1) {
        const bool upper = (lane & d) != 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float p = __shfl_xor_sync(0xFFFFFFFFu, v[i], d);
            v[i] = upper ? __fsub_rn(p, v[i]) : __fadd_rn(v[i], p);
        }
    }
}

// 16-byte chunk swizzle of a 128-float row so that the 16 threads of a row
// group, each reading 8 consecutive floats as two float4, hit distinct banks.
__device__ __forceinline__ int swz(int col) {
    const int chunk = col >> 2;
    return ((chunk ^ ((chunk >> 3) & 1)) << 2) | (col & 3);
}

// Byte `i` of a word, sign-extended: one byte permute whose upper three selectors replicate the sign of the byte
// (selector nibble 8 | i; the __byte_perm intrinsic keeps only three bits per selector, so the PTX form is used).
__device__ __forceinline__ int sext_byte(uint32_t word, int i) {
    int v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(word), "r"(0u), "r"(0x8880u + 0x1111u * static_cast<uint32_t>(i)));
    return v;
}

// Four ints -> four int8 in a word (byte 0 = a), each saturated to [-128, 127].
__device__ __forceinline__ uint32_t pack4_sat(int a, int b, int c, int d) {
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(b), "r"(a), "r"(hi));
    return w;
}

// The two 8-byte weight words and the row scales a thread will need in the tail, fetched at the top of a tile so
// that the HBM latency passes under the rank-r product.
struct TilePrefetch {
    uint2 old[2];
    float ws[2];
    bool vec[2];   // old[i] holds the eight weights (row in range, full 8-byte aligned octet)
};
__device__ __forceinline__ void prefetch_tile(TilePrefetch& pf, const int8_t* __restrict__ w, long long ldw,
                                              const float* __restrict__ w_scale, int ws_mode, int n_first, int row_end, int kc,
                                              int K, int w_vec_ok) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int n = n_first + i;
        const bool in = n < row_end && kc < K;
        pf.vec[i] = in && w_vec_ok && kc + 8 <= K;
        pf.old[i] = pf.vec[i] ? *reinterpret_cast<const uint2*>(w + static_cast<long long>(n) * ldw + kc) : make_uint2(0u, 0u);
        pf.ws[i] = in ? (ws_mode == I8F_WSCALE_CHANNEL ? __ldg(w_scale + n) : __ldg(w_scale)) : 1.f;
    }
}

// Shared tail of both merge kernels.  acc[i][c] is the un-scaled delta of row n_first + i, columns
// kc..kc+7 (the thread's 2 x 8 patch; 16 adjacent lanes hold one 128-column block of a row).
template <bool HAD>
__device__ __forceinline__ void merge_tail(float (&acc)[2][8], int8_t* __restrict__ w, long long ldw, const TilePrefetch& pf,
                                           int n_first, int row_end, int kc, int K, int lane, float lora_scale,
                                           const float* __restrict__ uniforms, const PhiloxKeys& keys) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[i][c] = __fmul_rn(acc[i][c], lora_scale);
        if constexpr (HAD) {
            wht128_lanes16(acc[i], lane);
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[i][c] = __fmul_rn(acc[i][c], kNormF32);
        }
        const int n = n_first + i;
        if (n >= row_end || kc >= K) continue;
        const float ws = pf.ws[i];
        float u[8];
        if (uniforms != nullptr) {
#pragma unroll
            for (int c = 0; c < 8; ++c) u[c] = (kc + c < K) ? __ldg(uniforms + static_cast<long long>(n) * K + kc + c) : 1.f;
        } else {
            uniforms8(philox4x32_10(static_cast<uint32_t>(n), static_cast<uint32_t>(kc >> 3), keys), u);
        }
        int8_t* wp = w + static_cast<long long>(n) * ldw + kc;
        if (pf.vec[i]) {
            const uint32_t ow[2] = {pf.old[i].x, pf.old[i].y};
            uint32_t nw[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int v[4];
#pragma unroll
                for (int b = 0; b < 4; ++b)   // sign-extended byte b of the old word + the rounded delta
                    v[b] = sext_byte(ow[h], b) + sr_round(acc[i][4 * h + b], ws, u[4 * h + b]);
                nw[h] = pack4_sat(v[0], v[1], v[2], v[3]);    // the second clamp of the reference, as a saturating pack
            }
            *reinterpret_cast<uint2*>(wp) = make_uint2(nw[0], nw[1]);
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                if (kc + c < K) {
                    const int s = max(-128, min(127, static_cast<int>(wp[c]) + sr_round(acc[i][c], ws, u[c])));
                    wp[c] = static_cast<int8_t>(s);
                }
            }
        }
    }
}

template <bool HAD>
__global__ void __launch_bounds__(kThreads)
lora_merge_kernel(int8_t* __restrict__ w, long long ldw, const float* __restrict__ w_scale, int ws_mode,
                  const void* __restrict__ up, long long ldup, const void* __restrict__ down, long long lddown, int fdt,
                  int N, int K, int r, float lora_scale, const float* __restrict__ uniforms,
                  const __grid_constant__ PhiloxKeys keys, int rows_per_cta, int w_vec_ok) {
    extern __shared__ float smem[];
    float* s_down = smem;            // [r][128] swizzled
    float* s_up = smem + r * 128;    // [32][r + 1] (padded: the two row pairs of a warp land in different banks)
    const int rs = r + 1;
    const int k0 = blockIdx.x * 128;
    for (int idx = threadIdx.x; idx < r * 128; idx += kThreads) {
        const int j = idx >> 7, c = idx & 127;
        s_down[j * 128 + swz(c)] = (k0 + c < K) ? load_f(down, fdt, static_cast<long long>(j) * lddown + k0 + c) : 0.f;
    }
    const int row_begin = blockIdx.y * rows_per_cta;
    const int row_end = min(N, row_begin + rows_per_cta);
    const int tr = threadIdx.x >> 4;   // row pair index 0..15
    const int tc = threadIdx.x & 15;   // column octet
    const int lane = threadIdx.x & 31;
    const int kc = k0 + tc * 8;

    for (int n0 = row_begin; n0 < row_end; n0 += kRowsPerIter) {
        TilePrefetch pf;
        prefetch_tile(pf, w, ldw, w_scale, ws_mode, n0 + 2 * tr, row_end, kc, K, w_vec_ok);
        __syncthreads();
        for (int rr = threadIdx.x >> 5; rr < kRowsPerIter; rr += kThreads / 32)   // a warp per row: no index division
            for (int j = threadIdx.x & 31; j < r; j += 32)
                s_up[rr * rs + j] = (n0 + rr < row_end) ? load_f(up, fdt, static_cast<long long>(n0 + rr) * ldup + j) : 0.f;
        __syncthreads();
        float acc[2][8];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[i][c] = 0.f;
        const float* u0p = s_up + (2 * tr) * rs;
        const float* u1p = u0p + rs;
        const int c0 = swz(tc * 8), c1 = swz(tc * 8 + 4);
        for (int j = 0; j < r; ++j) {
            const float4 da = *reinterpret_cast<const float4*>(s_down + j * 128 + c0);
            const float4 db = *reinterpret_cast<const float4*>(s_down + j * 128 + c1);
            const float d[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
            const float ua = u0p[j], ub = u1p[j];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                acc[0][c] = __fadd_rn(acc[0][c], __fmul_rn(ua, d[c]));
                acc[1][c] = __fadd_rn(acc[1][c], __fmul_rn(ub, d[c]));
            }
        }
        merge_tail<HAD>(acc, w, ldw, pf, n0 + 2 * tr, row_end, kc, K, lane, lora_scale, uniforms, keys);
    }
}

// Tensor-core form for 16-bit factors.  The rank-r product of a 32 x 128 tile runs on mma.sync
// (m16n8k16, fp32 accumulate) from shared memory: `down` is staged once per CTA transposed as
// [128 columns][r] so that consecutive rank indices are adjacent (B fragments), `up` rows as [32][r]
// (A fragments); rows are padded by 8 elements, which makes the 32-bit fragment loads conflict free.
// The accumulators go through shared memory into the 2 x 8 per-thread patches of the common tail.
// Tensor-core accumulation is not the sequential fp32 sum of the exact kernel, so a delta can differ in
// its last place; after stochastic rounding that shows up as a +-1 difference in about one weight per
// million.  This is what makes the merge bandwidth- instead of FMA-bound.
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2], bool is_bf16) {
    if (is_bf16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

constexpr int kAccStride = 132;  // floats per row of the accumulator tile in shared memory

template <bool HAD>
__global__ void __launch_bounds__(kThreads)
lora_merge_tc_kernel(int8_t* __restrict__ w, long long ldw, const float* __restrict__ w_scale, int ws_mode,
                     const unsigned short* __restrict__ up, long long ldup, const unsigned short* __restrict__ down,
                     long long lddown, int is_bf16, int N, int K, int r, int r16, float lora_scale,
                     const float* __restrict__ uniforms, const __grid_constant__ PhiloxKeys keys, int rows_per_cta,
                     int w_vec_ok, int up_vec_ok) {
    extern __shared__ float smem[];
    const int rp = r16 + 8;                                        // padded rank (16-bit elements per row)
    float* s_acc = smem;                                            // [32][kAccStride] fp32
    unsigned short* s_downT = reinterpret_cast<unsigned short*>(smem + kRowsPerIter * kAccStride);  // [128][rp]
    unsigned short* s_up = s_downT + 128 * rp;                      // [32][rp]
    const int k0 = blockIdx.x * 128;
    for (int idx = threadIdx.x; idx < r16 * 128; idx += kThreads) {
        const int j = idx >> 7, c = idx & 127;                      // coalesced along the columns of `down`
        s_downT[c * rp + j] = (j < r && k0 + c < K) ? down[static_cast<long long>(j) * lddown + k0 + c] : 0;
    }
    const int row_begin = blockIdx.y * rows_per_cta;
    const int row_end = min(N, row_begin + rows_per_cta);
    const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int wm = (warp & 1) * 16;                                 // this warp's 16 rows ...
    const int wn = (warp >> 1) * 32;                                // ... and 32 columns of the tile
    const int kc = k0 + tc * 8;

    for (int n0 = row_begin; n0 < row_end; n0 += kRowsPerIter) {
        TilePrefetch pf;
        prefetch_tile(pf, w, ldw, w_scale, ws_mode, n0 + 2 * tr, row_end, kc, K, w_vec_ok);
        __syncthreads();                                            // previous tile fully consumed (s_up, s_acc)
        // rows of `up` into shared memory: a warp takes rows warp, warp + 8, ...; a lane one 8-element (16-byte) piece of
        // a row, so there is no index division in the loop.  Pieces past the rank, rows past the band: zeros.
        for (int rr = warp; rr < kRowsPerIter; rr += kThreads / 32) {
            const bool row_in = n0 + rr < row_end;
            const unsigned short* src = up + static_cast<long long>(n0 + rr) * ldup;
            for (int j = lane * 8; j < r16; j += 256) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (row_in) {
                    if (up_vec_ok && j + 8 <= r) {
                        v = __ldg(reinterpret_cast<const uint4*>(src + j));
                    } else {
                        unsigned short e[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) e[q] = (j + q < r) ? src[j + q] : static_cast<unsigned short>(0);
                        v = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
                    }
                }
                *reinterpret_cast<uint4*>(s_up + rr * rp + j) = v;   // rp is a multiple of 8: 16-byte aligned
            }
        }
        __syncthreads();
        float d[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) d[nt][e] = 0.f;
        // fragments by ldmatrix: one x4 for the 16 x 16 piece of `up`, one x4 per pair of 8-column groups of `down`
        // (rows of both tiles are rp * 2 bytes apart, an odd multiple of 16 bytes: conflict free)
        const uint32_t a_addr = smem_addr(s_up + (wm + (lane & 15)) * rp + ((lane >> 4) << 3));
        const uint32_t b_addr = smem_addr(s_downT + (wn + (lane & 7) + ((lane >> 4) << 3)) * rp + (((lane >> 3) & 1) << 3));
        for (int kk = 0; kk < r16; kk += 16) {
            uint32_t a[4];
            ldmatrix_x4(a, a_addr + kk * 2);
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b[4];   // {k 0-7, k 8-15} of columns 16 np .. 16 np + 7, then of 16 np + 8 .. 16 np + 15
                ldmatrix_x4(b, b_addr + (np * 16 * rp + kk) * 2);
                const uint32_t b_lo[2] = {b[0], b[1]}, b_hi[2] = {b[2], b[3]};
                mma_16816(d[2 * np], a, b_lo, is_bf16 != 0);
                mma_16816(d[2 * np + 1], a, b_hi, is_bf16 != 0);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float* o = s_acc + (wm + g) * kAccStride + wn + nt * 8 + 2 * t4;
            *reinterpret_cast<float2*>(o) = make_float2(d[nt][0], d[nt][1]);
            *reinterpret_cast<float2*>(o + 8 * kAccStride) = make_float2(d[nt][2], d[nt][3]);
        }
        __syncthreads();
        float acc[2][8];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float4 lo = *reinterpret_cast<const float4*>(s_acc + (2 * tr + i) * kAccStride + tc * 8);
            const float4 hi = *reinterpret_cast<const float4*>(s_acc + (2 * tr + i) * kAccStride + tc * 8 + 4);
            acc[i][0] = lo.x; acc[i][1] = lo.y; acc[i][2] = lo.z; acc[i][3] = lo.w;
            acc[i][4] = hi.x; acc[i][5] = hi.y; acc[i][6] = hi.z; acc[i][7] = hi.w;
        }
        merge_tail<HAD>(acc, w, ldw, pf, n0 + 2 * tr, row_end, kc, K, lane, lora_scale, uniforms, keys);
    }
}

// Element-wise stochastic rounding of an fp32 delta; one thread per group of
// eight columns (one Philox block).
__global__ void __launch_bounds__(kThreads)
stochastic_round_kernel(const float* __restrict__ delta, long long ldd, const float* __restrict__ w_scale, int ws_mode,
                        int8_t* __restrict__ d8, long long ldq, int N, int K, const float* __restrict__ uniforms,
                        const __grid_constant__ PhiloxKeys keys) {
    const int groups = (K + 7) >> 3;
    const long long total = static_cast<long long>(N) * groups;
    for (long long g = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; g < total;
         g += static_cast<long long>(gridDim.x) * kThreads) {
        const int n = static_cast<int>(g / groups);
        const int kg = static_cast<int>(g - static_cast<long long>(n) * groups);
        const float ws = ws_mode == I8F_WSCALE_CHANNEL ? __ldg(w_scale + n) : __ldg(w_scale);
        float u[8];
        if (uniforms != nullptr) {
#pragma unroll
            for (int c = 0; c < 8; ++c) u[c] = (8 * kg + c < K) ? __ldg(uniforms + static_cast<long long>(n) * K + 8 * kg + c) : 1.f;
        } else {
            uniforms8(philox4x32_10(static_cast<uint32_t>(n), static_cast<uint32_t>(kg), keys), u);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int k = 8 * kg + c;
            if (k < K) d8[static_cast<long long>(n) * ldq + k] = static_cast<int8_t>(sr_round(__ldg(delta + static_cast<long long>(n) * ldd + k), ws, u[c]));
        }
    }
}

// Shared memory of one CTA: the whole [r x 128] slice of `down` plus 32 rows of `up` (and, in the tensor-core
// form, the fp32 accumulator tile).  This is what bounds the rank one launch can take.
constexpr size_t kMergeSmemLimit = 200 * 1024;
inline size_t merge_smem_bytes(bool tensor_path, int64_t r) {
    const size_t r16 = static_cast<size_t>((r + 15) / 16 * 16);
    return tensor_path ? static_cast<size_t>(kRowsPerIter) * kAccStride * sizeof(float) + static_cast<size_t>(128 + kRowsPerIter) * (r16 + 8) * 2
                       : (static_cast<size_t>(r) * 128 + static_cast<size_t>(kRowsPerIter) * (r + 1)) * sizeof(float);
}

}  // namespace
}  // namespace i8f

using namespace i8f;

extern "C" {

int64_t i8f_lora_merge_max_rank(int factor_dtype, int with_uniforms) {
    const bool tensor_path = factor_dtype != I8F_F32 && !with_uniforms;
    int64_t r = 0;
    while (merge_smem_bytes(tensor_path, r + 1) <= kMergeSmemLimit) ++r;
    return r;
}

int i8f_lora_merge_sr(int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode, const void* up, int64_t ldup,
                      const void* down, int64_t lddown, int factor_dtype, int64_t N, int64_t K, int64_t r,
                      float lora_scale, int hadamard128, const float* uniforms, uint64_t seed, void* stream) {
    I8F_REQUIRE(N >= 0 && K >= 0 && r >= 0, I8F_ERR_INVALID_ARG, "negative shape");
    if (N == 0 || K == 0) return I8F_OK;
    I8F_REQUIRE(w != nullptr && w_scale != nullptr, I8F_ERR_INVALID_ARG, "NULL weight or scale");
    I8F_REQUIRE(r == 0 || (up != nullptr && down != nullptr), I8F_ERR_INVALID_ARG, "NULL factor");
    I8F_REQUIRE(dtype_size(factor_dtype) != 0, I8F_ERR_INVALID_ARG, "unknown factor dtype %d", factor_dtype);
    I8F_REQUIRE(w_scale_mode == I8F_WSCALE_TENSOR || w_scale_mode == I8F_WSCALE_CHANNEL, I8F_ERR_INVALID_ARG,
                "unknown w_scale_mode %d", w_scale_mode);
    I8F_REQUIRE(ldw >= K && ldup >= r && lddown >= K, I8F_ERR_INVALID_ARG, "pitch smaller than the row length");
    I8F_REQUIRE(!hadamard128 || K % 128 == 0, I8F_ERR_UNSUPPORTED, "Hadamard rotation needs K %% 128 == 0");
    I8F_REQUIRE(N < (1LL << 31) && K < (1LL << 31), I8F_ERR_UNSUPPORTED, "dimension too large");
    // 16-bit factors with the in-kernel counter RNG take the tensor-core kernel; fp32 factors, and any call that
    // supplies its own uniforms (the bit-exact parity mode), take the sequential fp32 kernel
    const bool tensor_path = factor_dtype != I8F_F32 && uniforms == nullptr && r > 0 && ldup % 2 == 0 && lddown % 2 == 0;
    const int r16 = static_cast<int>((r + 15) / 16 * 16);
    const size_t smem = merge_smem_bytes(tensor_path, r);
    I8F_REQUIRE(smem <= kMergeSmemLimit, I8F_ERR_UNSUPPORTED,
                "rank %lld too large for one pass (limit %lld for this factor type; see i8f_lora_merge_max_rank)", (long long)r,
                (long long)i8f_lora_merge_max_rank(factor_dtype, uniforms != nullptr ? 1 : 0));
    const int col_blocks = static_cast<int>((K + 127) / 128);
    // enough row bands to fill the GPU a few times over, each band a multiple of 32 rows
    int bands = (148 * 4 + col_blocks - 1) / col_blocks;
    const int max_bands = static_cast<int>((N + kRowsPerIter - 1) / kRowsPerIter);
    if (bands > max_bands) bands = max_bands;
    if (bands < 1) bands = 1;
    if (bands > 65535) bands = 65535;
    int rows_per_cta = static_cast<int>((N + bands - 1) / bands);
    rows_per_cta = (rows_per_cta + kRowsPerIter - 1) / kRowsPerIter * kRowsPerIter;
    bands = static_cast<int>((N + rows_per_cta - 1) / rows_per_cta);
    const int w_vec_ok = ((reinterpret_cast<uintptr_t>(w) & 7u) == 0 && ldw % 8 == 0) ? 1 : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(col_blocks, bands);
    if (tensor_path) {
        auto launch_tc = [&](auto kern) -> int {
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
                if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            }
            kern<<<grid, kThreads, smem, st>>>(w, ldw, w_scale, w_scale_mode, static_cast<const unsigned short*>(up), ldup,
                                               static_cast<const unsigned short*>(down), lddown,
                                               factor_dtype == I8F_BF16 ? 1 : 0, static_cast<int>(N), static_cast<int>(K),
                                               static_cast<int>(r), r16, lora_scale, uniforms, make_philox_keys(seed), rows_per_cta, w_vec_ok,
                                               ((reinterpret_cast<uintptr_t>(up) & 15u) == 0 && ldup % 8 == 0) ? 1 : 0);
            return check_launch("lora_merge_tc_kernel");
        };
        return hadamard128 ? launch_tc(lora_merge_tc_kernel<true>) : launch_tc(lora_merge_tc_kernel<false>);
    }
    auto launch = [&](auto kern) -> int {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        }
        kern<<<grid, kThreads, smem, st>>>(w, ldw, w_scale, w_scale_mode, up, ldup, down, lddown, factor_dtype,
                                           static_cast<int>(N), static_cast<int>(K), static_cast<int>(r), lora_scale,
                                           uniforms, make_philox_keys(seed), rows_per_cta, w_vec_ok);
        return check_launch("lora_merge_kernel");
    };
    return hadamard128 ? launch(lora_merge_kernel<true>) : launch(lora_merge_kernel<false>);
}

int i8f_stochastic_round(const float* delta, int64_t ldd, const float* w_scale, int w_scale_mode, int8_t* d8,
                         int64_t ldq, int64_t N, int64_t K, const float* uniforms, uint64_t seed, void* stream) {
    I8F_REQUIRE(N >= 0 && K >= 0, I8F_ERR_INVALID_ARG, "negative shape");
    if (N == 0 || K == 0) return I8F_OK;
    I8F_REQUIRE(delta != nullptr && d8 != nullptr && w_scale != nullptr, I8F_ERR_INVALID_ARG, "NULL pointer");
    I8F_REQUIRE(ldd >= K && ldq >= K, I8F_ERR_INVALID_ARG, "pitch smaller than K");
    I8F_REQUIRE(w_scale_mode == I8F_WSCALE_TENSOR || w_scale_mode == I8F_WSCALE_CHANNEL, I8F_ERR_INVALID_ARG,
                "unknown w_scale_mode %d", w_scale_mode);
    I8F_REQUIRE(N < (1LL << 31) && K < (1LL << 31), I8F_ERR_UNSUPPORTED, "dimension too large");
    const long long total = N * ((K + 7) / 8);
    long long blocks = (total + kThreads - 1) / kThreads;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    stochastic_round_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        delta, ldd, w_scale, w_scale_mode, d8, ldq, static_cast<int>(N), static_cast<int>(K), uniforms, make_philox_keys(seed));
    return check_launch("stochastic_round_kernel");
}

}  // extern "C"

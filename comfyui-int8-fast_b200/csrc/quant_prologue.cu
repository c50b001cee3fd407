// Activation quantiser with the element-wise step that precedes a quantised linear in a diffusion transformer
// folded in, so that the activation makes one pass through HBM instead of three or four:
//
//   i8f_quant_rowwise_ln_modulate   y = LayerNorm(x) * (1 + scale) + shift        -> per-token int8
//   i8f_quant_rowwise_gelu          y = [ x_plain | GELU_tanh(x_gelu) ]           -> per-token int8
//   i8f_rmsnorm_heads               per-head RMS norm of the q and k columns of a fused qkv buffer, in place
//
// All three define their arithmetic completely (every fp32 operation and the order of every sum), so that a CPU
// restatement reproduces their results bit for bit; nothing here relies on approximate hardware functions.
//
// Layout of the two quantisers: a row belongs to 128 threads (two rows per CTA); thread t holds the 8-element
// vectors t, t + 128, t + 256, ... of its row, packed as loaded.  Row sums are taken in a fixed order:
//   vector:  ((((((e0 + e1) + e2) + e3) + e4) + e5) + e6) + e7
//   thread:  its vectors' sums, in slot order, sequentially
//   warp:    butterfly over lane distances 1, 2, 4, 8, 16 (a balanced binary tree over the 32 lanes)
//   row:     the four warps' sums, sequentially
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "f32x2.cuh"
#include "host_common.h"

namespace i8f {
namespace {

constexpr int kThreads = 256;
constexpr int kThreadsPerRow = 128;
constexpr float kScaleFloor = 1e-30f;

template <int DT>
__device__ __forceinline__ void unpack8(const uint4& r, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (DT == I8F_BF16) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
}
// The same widening, but opaque to the optimiser: a kernel that walks its packed row several times would otherwise
// keep all the widened values alive between the passes (twice the registers, half the occupancy).
template <int DT>
__device__ __forceinline__ void unpack8_again(const uint4& r, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (DT == I8F_BF16) {
            uint32_t lo, hi;
            asm volatile("shl.b32 %0, %2, 16;\n\tand.b32 %1, %2, 0xFFFF0000;" : "=r"(lo), "=r"(hi) : "r"(w[i]));
            v[2 * i] = __uint_as_float(lo);
            v[2 * i + 1] = __uint_as_float(hi);
        } else {
            uint32_t x;
            asm volatile("mov.b32 %0, %1;" : "=r"(x) : "r"(w[i]));
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&x));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
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
__device__ __forceinline__ float load_scalar(const void* p, int64_t i) {
    if constexpr (DT == I8F_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    else return __half2float(static_cast<const __half*>(p)[i]);
}
template <int DT>
__device__ __forceinline__ float round_to_dt(float x) {
    if constexpr (DT == I8F_BF16) return __bfloat162float(__float2bfloat16_rn(x));
    else return __half2float(__float2half_rn(x));
}

// rint(x * inv) for the eight values of a vector: the product is rounded first (scalar __fmul_rn, which the assembler
// never contracts with the add that follows; a two-wide multiply was seen contracted), then the magic add runs
// two-wide.  |x * inv| <= 127.00002, see quant_rowwise.cu.
__device__ __forceinline__ uint2 quant8_pairs(const float (&f)[8], float inv) {
    constexpr float kMagic = 12582912.0f;
    const f32x2 magic2 = pair_of(kMagic, kMagic);
    uint32_t u[8];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        halves_bits(add2(pair_of(__fmul_rn(f[2 * j], inv), __fmul_rn(f[2 * j + 1], inv)), magic2), u[2 * j], u[2 * j + 1]);
    uint2 o;
    o.x = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
    o.y = __byte_perm(__byte_perm(u[4], u[5], 0x0040), __byte_perm(u[6], u[7], 0x0040), 0x5410);
    return o;
}

// seq_sum8 of two vectors at once, one in each lane of the two-wide registers (same order of additions per vector).
__device__ __forceinline__ void seq_sum8_two(const float (&a)[8], const float (&b)[8], float& sa, float& sb) {
    f32x2 s = add2(pair_of(a[0], b[0]), pair_of(a[1], b[1]));
#pragma unroll
    for (int j = 2; j < 8; ++j) s = add2(s, pair_of(a[j], b[j]));
    halves(s, sa, sb);
}

// Sum over the 128 threads of a row of one value per thread, in the fixed order of the header.  `s_part` has one
// float per warp of the CTA; two barriers per call.
// Barrier among the 128 threads (four warps) of one row only: the rows of a CTA run independently of each other, so
// that one row's loads are in flight while another row computes.
__device__ __forceinline__ void row_barrier(int row_in_cta) {
    asm volatile("bar.sync %0, 128;" ::"r"(row_in_cta + 1) : "memory");
}
__device__ __forceinline__ float row_sum(float v, float* s_part, int row_in_cta) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
    const int warp = threadIdx.x >> 5;
    row_barrier(row_in_cta);               // previous use of this row's slots of s_part is over
    if ((threadIdx.x & 31) == 0) s_part[warp] = v;
    row_barrier(row_in_cta);
    const float* w = s_part + row_in_cta * 4;
    return __fadd_rn(__fadd_rn(__fadd_rn(w[0], w[1]), w[2]), w[3]);
}
__device__ __forceinline__ float row_max(float v, float* s_part, int row_in_cta) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
    const int warp = threadIdx.x >> 5;
    row_barrier(row_in_cta);
    if ((threadIdx.x & 31) == 0) s_part[warp] = v;
    row_barrier(row_in_cta);
    const float* w = s_part + row_in_cta * 4;
    return fmaxf(fmaxf(w[0], w[1]), fmaxf(w[2], w[3]));
}

__device__ __forceinline__ float seq_sum8(const float (&f)[8]) {
    float s = __fadd_rn(f[0], f[1]);
#pragma unroll
    for (int j = 2; j < 8; ++j) s = __fadd_rn(s, f[j]);
    return s;
}

// Absmax of the packed row held by this thread (16-bit SIMD max on the sign-cleared patterns).
template <int DT, int VPT>
__device__ __forceinline__ float packed_absmax(const uint4 (&raw)[VPT]) {
    uint32_t m2 = 0u;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        m2 = __vmaxu2(m2, raw[i].x & 0x7FFF7FFFu);
        m2 = __vmaxu2(m2, raw[i].y & 0x7FFF7FFFu);
        m2 = __vmaxu2(m2, raw[i].z & 0x7FFF7FFFu);
        m2 = __vmaxu2(m2, raw[i].w & 0x7FFF7FFFu);
    }
    const uint32_t m16 = max(m2 & 0xFFFFu, m2 >> 16);
    if constexpr (DT == I8F_BF16) return __uint_as_float(m16 << 16);
    else return __half2float(__ushort_as_half(static_cast<unsigned short>(m16)));
}

template <int DT, int VPT>
__device__ __forceinline__ void quantise_and_store(const uint4 (&raw)[VPT], float amax, bool row_ok, int64_t row, int t, int nvec,
                                                   int8_t* __restrict__ q, int64_t ldq, float* __restrict__ scale) {
    const float sc = fmaxf(__fdiv_rn(amax, 127.0f), kScaleFloor);
    const float inv = __fdiv_rn(1.0f, sc);
    if (row_ok && t == 0) scale[row] = sc;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vec = i * kThreadsPerRow + t;
        if (row_ok && vec < nvec) {
            float f[8];
            unpack8<DT>(raw[i], f);
            *reinterpret_cast<uint2*>(q + row * ldq + static_cast<int64_t>(vec) * 8) = quant8_pairs(f, inv);
        }
    }
}

// ------------------------------------------------------------------ LayerNorm * (1 + scale) + shift -> int8
//   mean = rowsum(x) / K                     var = rowsum((x - mean)^2) / K         rstd = 1 / sqrt(var + eps)
//   ln   = rnd((x - mean) * rstd)            y = rnd(ln * rnd(1 + scale[k]) + shift[k])      (rnd: to the 16-bit type)
// The last line is ONE rounding of the exact value ln * gain + shift to the 16-bit type (a fused multiply-add in that
// type).  Then q = rint(y * (1 / s)), s = max(absmax(y) / 127, 1e-30), as in the plain quantiser.
// This kernel (128 threads per row, sums in the order of the file header) serves rows longer than 4096 elements.
template <int DT, int VPT>
__global__ void __launch_bounds__(kThreads)
ln_modulate_quant_kernel(const void* __restrict__ x, int64_t M, int64_t K, int64_t ldx, const void* __restrict__ shift,
                         const void* __restrict__ mscale, float eps, int8_t* __restrict__ q, int64_t ldq,
                         float* __restrict__ scale, void* __restrict__ y_out, int64_t ldy) {
    __shared__ float s_part[kThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int t = threadIdx.x & (kThreadsPerRow - 1);
    const int row_in_cta = threadIdx.x >> 7;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 2 + row_in_cta;
    const bool row_ok = row < M;
    const int nvec = static_cast<int>(K >> 3);
    uint4 raw[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vec = i * kThreadsPerRow + t;
        raw[i] = (row_ok && vec < nvec)
                     ? __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(x) + row * ldx + static_cast<int64_t>(vec) * 8))
                     : make_uint4(0u, 0u, 0u, 0u);
    }
    const float kf = static_cast<float>(K);
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        float f[8];
        unpack8<DT>(raw[i], f);
        const float s = seq_sum8(f);
        part = (i == 0) ? s : __fadd_rn(part, s);
    }
    const float mean = __fdiv_rn(row_sum(part, s_part, row_in_cta), kf);
    part = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vec = i * kThreadsPerRow + t;
        float f[8];
        unpack8<DT>(raw[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float d = (vec < nvec) ? __fsub_rn(f[j], mean) : 0.f;
            f[j] = __fmul_rn(d, d);
        }
        const float s = seq_sum8(f);
        part = (i == 0) ? s : __fadd_rn(part, s);
    }
    const float var = __fdiv_rn(row_sum(part, s_part, row_in_cta), kf);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vec = i * kThreadsPerRow + t;
        if (vec < nvec) {
            float f[8], sh[8], ms[8];
            unpack8<DT>(raw[i], f);
            unpack8<DT>(__ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(shift) + static_cast<int64_t>(vec) * 8)), sh);
            unpack8<DT>(__ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(mscale) + static_cast<int64_t>(vec) * 8)), ms);
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // rnd(ln * rnd(1 + scale) + shift): one fused multiply-add in the 16-bit type (exact value, one rounding)
                const uint32_t ln2 = pack2<DT>(__fmul_rn(__fsub_rn(f[2 * j], mean), rstd), __fmul_rn(__fsub_rn(f[2 * j + 1], mean), rstd));
                const uint32_t gain2 = pack2<DT>(__fadd_rn(1.0f, ms[2 * j]), __fadd_rn(1.0f, ms[2 * j + 1]));
                const uint32_t sh2 = pack2<DT>(sh[2 * j], sh[2 * j + 1]);
                if constexpr (DT == I8F_BF16) {
                    const __nv_bfloat162 y = __hfma2(*reinterpret_cast<const __nv_bfloat162*>(&ln2), *reinterpret_cast<const __nv_bfloat162*>(&gain2),
                                                     *reinterpret_cast<const __nv_bfloat162*>(&sh2));
                    w[j] = *reinterpret_cast<const uint32_t*>(&y);
                } else {
                    const __half2 y = __hfma2(*reinterpret_cast<const __half2*>(&ln2), *reinterpret_cast<const __half2*>(&gain2),
                                              *reinterpret_cast<const __half2*>(&sh2));
                    w[j] = *reinterpret_cast<const uint32_t*>(&y);
                }
            }
            raw[i] = make_uint4(w[0], w[1], w[2], w[3]);
            if (y_out != nullptr && row_ok)
                *reinterpret_cast<uint4*>(static_cast<unsigned short*>(y_out) + row * ldy + static_cast<int64_t>(vec) * 8) = raw[i];
        }
    }
    const float amax = row_max(packed_absmax<DT, VPT>(raw), s_part, row_in_cta);
    quantise_and_store<DT, VPT>(raw, amax, row_ok, row, t, nvec, q, ldq, scale);
}

// Rows of at most 4096 elements (the hidden size of the transformer, where this kernel runs) belong to ONE WARP: lane l
// holds the vectors l, l + 32, ..., packed as loaded, so the three row reductions are shuffle butterflies with no
// shared memory and no barrier, and the eight rows of a CTA proceed independently.  Order of a row sum here: the 8
// elements of a vector left to right; a lane's vector sums in slot order; the 32 lanes as a balanced binary tree.
// The modulation is one fused multiply-add per pair in the 16-bit type: rnd(ln * rnd(1 + scale) + shift) with a single
// rounding of the exact value.
template <int DT>
__global__ void __launch_bounds__(kThreads, 2)
ln_modulate_quant_warp_kernel(const void* __restrict__ x, int64_t M, int64_t K, int64_t ldx, const void* __restrict__ shift,
                              const void* __restrict__ mscale, float eps, int8_t* __restrict__ q, int64_t ldq,
                              float* __restrict__ scale, void* __restrict__ y_out, int64_t ldy) {
    constexpr int VPL = 16;     // vectors per lane: 32 lanes x 16 x 8 = 4096 elements
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    if (row >= M) return;                      // whole warps leave together; nothing below synchronises across warps
    const int nvec = static_cast<int>(K >> 3);
    const float kf = static_cast<float>(K);
    uint4 raw[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vec = i * 32 + lane;
        raw[i] = vec < nvec ? __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(x) + row * ldx + static_cast<int64_t>(vec) * 8))
                            : make_uint4(0u, 0u, 0u, 0u);
    }
    auto warp_sum = [](float v) {
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
        return v;
    };
    // the two sum passes take the lane's vectors two at a time, one vector in each lane of the two-wide registers
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; i += 2) {
        float fa[8], fb[8], sa, sb;
        unpack8_again<DT>(raw[i], fa);
        unpack8_again<DT>(raw[i + 1], fb);
        seq_sum8_two(fa, fb, sa, sb);
        part = (i == 0) ? sa : __fadd_rn(part, sa);
        part = __fadd_rn(part, sb);
    }
    const float mean = __fdiv_rn(warp_sum(part), kf);
    const f32x2 mean2 = pair_of(mean, mean);
    part = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; i += 2) {
        const bool oka = i * 32 + lane < nvec, okb = (i + 1) * 32 + lane < nvec;
        float fa[8], fb[8];
        unpack8_again<DT>(raw[i], fa);
        unpack8_again<DT>(raw[i + 1], fb);
        f32x2 sq[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float da, db;
            halves(sub2(pair_of(fa[j], fb[j]), mean2), da, db);
            sq[j] = pair_of(__fmul_rn(da, da), __fmul_rn(db, db));   // scalar: never contracted with the sums below
        }
        f32x2 s2 = add2(sq[0], sq[1]);
#pragma unroll
        for (int j = 2; j < 8; ++j) s2 = add2(s2, sq[j]);
        float sa, sb;
        halves(s2, sa, sb);
        sa = oka ? sa : 0.f;      // vectors beyond the row contribute zeros
        sb = okb ? sb : 0.f;
        part = (i == 0) ? sa : __fadd_rn(part, sa);
        part = __fadd_rn(part, sb);
    }
    const float var = __fdiv_rn(warp_sum(part), kf);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    const f32x2 rstd2 = pair_of(rstd, rstd);
    uint32_t m2 = 0u;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vec = i * 32 + lane;
        if (vec < nvec) {
            float f[8];
            unpack8_again<DT>(raw[i], f);
            const uint4 sh = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(shift) + static_cast<int64_t>(vec) * 8));
            const uint4 ms = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(mscale) + static_cast<int64_t>(vec) * 8));
            const uint32_t shw[4] = {sh.x, sh.y, sh.z, sh.w}, msw[4] = {ms.x, ms.y, ms.z, ms.w};
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float lnlo, lnhi;
                halves(mul2(sub2(pair_of(f[2 * j], f[2 * j + 1]), mean2), rstd2), lnlo, lnhi);
                const uint32_t ln2 = pack2<DT>(lnlo, lnhi);
                if constexpr (DT == I8F_BF16) {
                    const __nv_bfloat162 one = __floats2bfloat162_rn(1.0f, 1.0f);
                    const __nv_bfloat162 gain = __hadd2(one, *reinterpret_cast<const __nv_bfloat162*>(&msw[j]));
                    const __nv_bfloat162 y = __hfma2(*reinterpret_cast<const __nv_bfloat162*>(&ln2), gain, *reinterpret_cast<const __nv_bfloat162*>(&shw[j]));
                    w[j] = *reinterpret_cast<const uint32_t*>(&y);
                } else {
                    const __half2 one = __floats2half2_rn(1.0f, 1.0f);
                    const __half2 gain = __hadd2(one, *reinterpret_cast<const __half2*>(&msw[j]));
                    const __half2 y = __hfma2(*reinterpret_cast<const __half2*>(&ln2), gain, *reinterpret_cast<const __half2*>(&shw[j]));
                    w[j] = *reinterpret_cast<const uint32_t*>(&y);
                }
                m2 = __vmaxu2(m2, w[j] & 0x7FFF7FFFu);
            }
            raw[i] = make_uint4(w[0], w[1], w[2], w[3]);
            if (y_out != nullptr)
                *reinterpret_cast<uint4*>(static_cast<unsigned short*>(y_out) + row * ldy + static_cast<int64_t>(vec) * 8) = raw[i];
        } else {
            raw[i] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    const uint32_t m16 = max(m2 & 0xFFFFu, m2 >> 16);
    float amax;
    if constexpr (DT == I8F_BF16) amax = __uint_as_float(m16 << 16);
    else amax = __half2float(__ushort_as_half(static_cast<unsigned short>(m16)));
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
    const float sc = fmaxf(__fdiv_rn(amax, 127.0f), kScaleFloor);
    const float inv = __fdiv_rn(1.0f, sc);
    if (lane == 0) scale[row] = sc;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vec = i * 32 + lane;
        if (vec < nvec) {
            float f[8];
            unpack8_again<DT>(raw[i], f);
            *reinterpret_cast<uint2*>(q + row * ldq + static_cast<int64_t>(vec) * 8) = quant8_pairs(f, inv);
        }
    }
}

// ------------------------------------------------------------------ [ plain | GELU(tanh) ] -> int8
// GELU in its tanh form, written as x * sigmoid(2u), u = x * (c0 + c1 * x^2), with the exponential spelled out in
// correctly rounded fp32 operations only (no fused multiply-add, no approximate unit):
//   t = clamp(u * (-2 log2 e), -125, 125)    n = rint(t)    f = t - n  (exact)
//   p = ((((a5 f + a4) f + a3) f + a2) f + a1) f + 1        (2^f on [-1/2, 1/2], every step a rounded mul then add)
//   e = p * 2^n  (exponent arithmetic)       g = x * (1 / (1 + e))
constexpr float kGeluC0 = 0.7978845608028654f;          // sqrt(2 / pi)
constexpr float kGeluC1 = 0.035677408136300125f;        // sqrt(2 / pi) * 0.044715
constexpr float kNeg2Log2e = -2.8853900817779268f;      // -2 / ln 2
constexpr float kExp2A1 = 0.6931471805599453f, kExp2A2 = 0.2402265069591007f, kExp2A3 = 0.05550410866482158f,
                kExp2A4 = 0.009618129107628477f, kExp2A5 = 0.0013333558146428443f;

__device__ __forceinline__ float gelu_tanh_exact(float x) {
    const float x2 = __fmul_rn(x, x);
    const float u = __fmul_rn(x, __fadd_rn(__fmul_rn(x2, kGeluC1), kGeluC0));
    const float t = fminf(fmaxf(__fmul_rn(u, kNeg2Log2e), -125.0f), 125.0f);
    const float r = __fadd_rn(t, 12582912.0f);
    const float nf = __fsub_rn(r, 12582912.0f);
    const float f = __fsub_rn(t, nf);
    float p = __fadd_rn(__fmul_rn(kExp2A5, f), kExp2A4);
    p = __fadd_rn(__fmul_rn(p, f), kExp2A3);
    p = __fadd_rn(__fmul_rn(p, f), kExp2A2);
    p = __fadd_rn(__fmul_rn(p, f), kExp2A1);
    p = __fadd_rn(__fmul_rn(p, f), 1.0f);
    const int n = static_cast<int>(__float_as_uint(r)) - 0x4B400000;      // low mantissa bits of r hold rint(t)
    const float e = __uint_as_float(__float_as_uint(p) + (static_cast<uint32_t>(n) << 23));
    return __fmul_rn(x, __fdiv_rn(1.0f, __fadd_rn(1.0f, e)));
}

template <int DT, int VPT>
__global__ void __launch_bounds__(kThreads)
gelu_quant_kernel(const void* __restrict__ x0, int64_t K0, int64_t ld0, const void* __restrict__ x1, int64_t K1, int64_t ld1,
                  int64_t M, int8_t* __restrict__ q, int64_t ldq, float* __restrict__ scale, void* __restrict__ y_out,
                  int64_t ldy) {
    __shared__ float s_part[kThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int t = threadIdx.x & (kThreadsPerRow - 1);
    const int row_in_cta = threadIdx.x >> 7;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 2 + row_in_cta;
    const bool row_ok = row < M;
    const int nvec0 = static_cast<int>(K0 >> 3);
    const int nvec = nvec0 + static_cast<int>(K1 >> 3);
    uint4 raw[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vec = i * kThreadsPerRow + t;
        raw[i] = make_uint4(0u, 0u, 0u, 0u);
        if (row_ok && vec < nvec0)
            raw[i] = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(x0) + row * ld0 + static_cast<int64_t>(vec) * 8));
        else if (row_ok && vec < nvec)
            raw[i] = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(x1) + row * ld1 + static_cast<int64_t>(vec - nvec0) * 8));
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vec = i * kThreadsPerRow + t;
        if (vec >= nvec0 && vec < nvec) {
            float f[8];
            unpack8<DT>(raw[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = gelu_tanh_exact(f[j]);
            raw[i] = make_uint4(pack2<DT>(f[0], f[1]), pack2<DT>(f[2], f[3]), pack2<DT>(f[4], f[5]), pack2<DT>(f[6], f[7]));
        }
        if (y_out != nullptr && row_ok && vec < nvec)
            *reinterpret_cast<uint4*>(static_cast<unsigned short*>(y_out) + row * ldy + static_cast<int64_t>(vec) * 8) = raw[i];
    }
    const float amax = row_max(packed_absmax<DT, VPT>(raw), s_part, row_in_cta);
    quantise_and_store<DT, VPT>(raw, amax, row_ok, row, t, nvec, q, ldq, scale);
}

// The same quantiser for large inputs: a 16-bit activation has only 65536 possible values, so rnd(GELU(x)) is read from
// a table (built once per device by gelu_table_kernel with the very arithmetic above, so the bits are the same) that
// every CTA of a persistent grid keeps in shared memory.  One table look-up per element instead of some forty fp32
// instructions, which left the direct kernel at a quarter of the memory rate.
constexpr int kTableThreads = 384;     // three rows at a time; 170 registers per thread leave room for the prefetched row
__device__ unsigned short g_gelu_table[2][65536];      // [0] bf16, [1] fp16

template <int DT>
__global__ void gelu_table_kernel(unsigned short* __restrict__ table) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 65536u) return;
    float x;
    if constexpr (DT == I8F_BF16) x = __uint_as_float(i << 16);
    else x = __half2float(__ushort_as_half(static_cast<unsigned short>(i)));
    table[i] = static_cast<unsigned short>(pack2<DT>(gelu_tanh_exact(x), 0.f) & 0xFFFFu);
}

template <int DT, int VPT>
__global__ void __launch_bounds__(kTableThreads)
gelu_quant_table_kernel(const void* __restrict__ x0, int64_t K0, int64_t ld0, const void* __restrict__ x1, int64_t K1,
                        int64_t ld1, int64_t M, int8_t* __restrict__ q, int64_t ldq, float* __restrict__ scale,
                        void* __restrict__ y_out, int64_t ldy, const unsigned short* __restrict__ table) {
    constexpr int kRows = kTableThreads / kThreadsPerRow;      // rows a CTA works on at a time
    extern __shared__ __align__(16) unsigned short s_table[];
    __shared__ float s_part[kTableThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int t = threadIdx.x & (kThreadsPerRow - 1);
    const int row_in_cta = threadIdx.x >> 7;
    const int nvec0 = static_cast<int>(K0 >> 3);
    const int nvec = nvec0 + static_cast<int>(K1 >> 3);
    auto load_row = [&](int64_t row, uint4 (&dst)[VPT]) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vec = i * kThreadsPerRow + t;
            dst[i] = make_uint4(0u, 0u, 0u, 0u);
            if (row < M && vec < nvec0)
                dst[i] = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(x0) + row * ld0 + static_cast<int64_t>(vec) * 8));
            else if (row < M && vec < nvec)
                dst[i] = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(x1) + row * ld1 + static_cast<int64_t>(vec - nvec0) * 8));
        }
    };
    uint4 raw[VPT], next[VPT];
    load_row(static_cast<int64_t>(blockIdx.x) * kRows + row_in_cta, raw);      // in flight while the table is copied
    for (int i = threadIdx.x; i < 65536 / 8; i += kTableThreads)
        reinterpret_cast<uint4*>(s_table)[i] = __ldg(reinterpret_cast<const uint4*>(table) + i);
    __syncthreads();
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kRows;
    for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRows; row0 < M; row0 += stride) {
        const int64_t row = row0 + row_in_cta;
        const bool row_ok = row < M;
        load_row(row + stride, next);          // the next row's loads fly under this row's look-ups and stores
        auto look2 = [&](uint32_t w) -> uint32_t {
            return static_cast<uint32_t>(s_table[w & 0xFFFFu]) | (static_cast<uint32_t>(s_table[w >> 16]) << 16);
        };
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vec = i * kThreadsPerRow + t;
            if (row_ok && vec >= nvec0 && vec < nvec)
                raw[i] = make_uint4(look2(raw[i].x), look2(raw[i].y), look2(raw[i].z), look2(raw[i].w));
            if (y_out != nullptr && row_ok && vec < nvec)
                *reinterpret_cast<uint4*>(static_cast<unsigned short*>(y_out) + row * ldy + static_cast<int64_t>(vec) * 8) = raw[i];
        }
        const float amax = row_max(packed_absmax<DT, VPT>(raw), s_part, row_in_cta);
        quantise_and_store<DT, VPT>(raw, amax, row_ok, row, t, nvec, q, ldq, scale);
#pragma unroll
        for (int i = 0; i < VPT; ++i) raw[i] = next[i];
    }
}

// Device address of the table for `dt` on the current device.  The first call on a device builds it with a kernel on
// that call's stream and records an event behind it; until the event has completed, calls on other streams are made
// to wait for it (stream-side, the host never blocks).  While `st` is being captured into a graph and the table is
// not known to be complete, the build is captured with the launch instead (and not remembered: it has not run yet).
int gelu_table(int dt, cudaStream_t st, const unsigned short** out) {
    struct State {
        unsigned short* table;
        cudaEvent_t built_event;
        int phase;        // 0 nothing, 1 build enqueued (event recorded), 2 known complete
    };
    static State states[64][2] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(I8F_ERR_CUDA, "cudaGetDevice failed");
    const int which = dt == I8F_BF16 ? 0 : 1;
    State& s = states[dev][which];
    if (s.table == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_gelu_table);
        if (e != cudaSuccess || p == nullptr) return fail(I8F_ERR_CUDA, "cudaGetSymbolAddress(GELU table): %s", cudaGetErrorString(e));
        s.table = static_cast<unsigned short*>(p) + which * 65536;
    }
    *out = s.table;
    if (s.phase == 2) return I8F_OK;
    if (s.phase == 1 && cudaEventQuery(s.built_event) == cudaSuccess) {
        s.phase = 2;
        return I8F_OK;
    }
    auto build = [&]() -> int {
        if (which == 0) gelu_table_kernel<I8F_BF16><<<256, 256, 0, st>>>(s.table);
        else gelu_table_kernel<I8F_F16><<<256, 256, 0, st>>>(s.table);
        return check_launch("gelu_table_kernel");
    };
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(st, &cap);
    if (cap != cudaStreamCaptureStatusNone) return build();       // part of the graph; rebuilding the same values is harmless
    if (s.phase == 1) {
        const cudaError_t e = cudaStreamWaitEvent(st, s.built_event, 0);
        if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "cudaStreamWaitEvent(GELU table): %s", cudaGetErrorString(e));
        return I8F_OK;
    }
    int rc = build();
    if (rc != I8F_OK) return rc;
    cudaError_t e = cudaEventCreateWithFlags(&s.built_event, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(s.built_event, st);
    if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "recording the GELU table event: %s", cudaGetErrorString(e));
    s.phase = 1;
    return I8F_OK;
}

// ------------------------------------------------------------------ per-head RMS norm, in place
// Rows of `head_dim` = 128 elements (one attention head of one token): y = rnd(x * (1 / sqrt(sum(x^2) / 128 + eps))).
// Sixteen lanes hold a head (8 elements each): squares summed sequentially per lane, then a butterfly over lane
// distances 1, 2, 4, 8.  The matrix is [rows, cols] with cols a multiple of 128; each 128-column block of a row is
// one head.
template <int DT>
__global__ void __launch_bounds__(256)
rmsnorm_heads_kernel(void* __restrict__ x, int64_t rows, int64_t cols, int64_t ldx, float eps) {
    const int heads_per_row = static_cast<int>(cols >> 7);
    const int64_t total = rows * heads_per_row;
    const int lane16 = threadIdx.x & 15;
    for (int64_t h = static_cast<int64_t>(blockIdx.x) * 16 + (threadIdx.x >> 4); h < total;
         h += static_cast<int64_t>(gridDim.x) * 16) {
        const int64_t r = h / heads_per_row;
        const int hc = static_cast<int>(h - r * heads_per_row);
        unsigned short* p = static_cast<unsigned short*>(x) + r * ldx + static_cast<int64_t>(hc) * 128 + lane16 * 8;
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        float f[8], sq[8];
        unpack8<DT>(raw, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) sq[j] = __fmul_rn(f[j], f[j]);
        float s = seq_sum8(sq);
#pragma unroll
        for (int d = 1; d < 16; d <<= 1) s = __fadd_rn(s, __shfl_xor_sync(0xFFFFFFFFu, s, d));
        const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(s, 0.0078125f), eps)));
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(f[j], rstd);
        *reinterpret_cast<uint4*>(p) = make_uint4(pack2<DT>(f[0], f[1]), pack2<DT>(f[2], f[3]), pack2<DT>(f[4], f[5]), pack2<DT>(f[6], f[7]));
    }
}

int check_rows(const void* x, int dt, int64_t M, int64_t K, int64_t ld, const char* what) {
    I8F_REQUIRE(dt == I8F_BF16 || dt == I8F_F16, I8F_ERR_UNSUPPORTED, "%s: dtype must be bf16 or f16", what);
    I8F_REQUIRE(x != nullptr && ld >= K, I8F_ERR_INVALID_ARG, "%s: NULL input or row pitch smaller than the row", what);
    I8F_REQUIRE(K % 8 == 0, I8F_ERR_UNSUPPORTED, "%s: row length %lld must be a multiple of 8", what, (long long)K);
    I8F_REQUIRE(aligned16(x) && (ld * 2) % 16 == 0, I8F_ERR_ALIGNMENT, "%s: input must be 16-byte aligned with a 16-byte multiple row pitch", what);
    I8F_REQUIRE(M >= 0 && M < (1LL << 31), I8F_ERR_INVALID_ARG, "%s: bad row count", what);
    return I8F_OK;
}

int check_out(const int8_t* q, int64_t ldq, const float* scale, int64_t K, const void* y_out, int64_t ldy) {
    I8F_REQUIRE(q != nullptr && scale != nullptr && ldq >= K, I8F_ERR_INVALID_ARG, "NULL output or int8 pitch smaller than the row");
    I8F_REQUIRE((reinterpret_cast<uintptr_t>(q) & 7u) == 0 && ldq % 8 == 0, I8F_ERR_ALIGNMENT,
                "int8 output must be 8-byte aligned with an 8-byte multiple row pitch");
    I8F_REQUIRE(y_out == nullptr || (aligned16(y_out) && ldy >= K && (ldy * 2) % 16 == 0), I8F_ERR_ALIGNMENT,
                "y_out must be 16-byte aligned with a 16-byte multiple row pitch of at least the row length");
    return I8F_OK;
}

}  // namespace
}  // namespace i8f

using namespace i8f;

#define I8F_DISPATCH_VPT(KERNEL, DT, nvec, ...)                                                       \
    do {                                                                                              \
        const int vpt_ = static_cast<int>(((nvec) + kThreadsPerRow - 1) / kThreadsPerRow);            \
        if (vpt_ <= 4) KERNEL<DT, 4><<<grid, kThreads, 0, st>>>(__VA_ARGS__);                         \
        else if (vpt_ <= 8) KERNEL<DT, 8><<<grid, kThreads, 0, st>>>(__VA_ARGS__);                    \
        else if (vpt_ <= 12) KERNEL<DT, 12><<<grid, kThreads, 0, st>>>(__VA_ARGS__);                  \
        else KERNEL<DT, 16><<<grid, kThreads, 0, st>>>(__VA_ARGS__);                                  \
    } while (0)

extern "C" {

int i8f_quant_rowwise_ln_modulate(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* shift,
                                  const void* scale, float eps, int8_t* q, int64_t ldq, float* row_scale, void* y_out,
                                  int64_t ldy, void* stream) {
    int rc = check_rows(x, x_dtype, M, K, ldx, "i8f_quant_rowwise_ln_modulate");
    if (rc != I8F_OK) return rc;
    if (M == 0) return I8F_OK;
    I8F_REQUIRE(K > 0 && K <= 16384, I8F_ERR_UNSUPPORTED, "row length %lld exceeds the 16384-element limit", (long long)K);
    I8F_REQUIRE(shift != nullptr && scale != nullptr && aligned16(shift) && aligned16(scale), I8F_ERR_ALIGNMENT,
                "shift and scale must be 16-byte aligned vectors of K elements");
    I8F_REQUIRE(eps >= 0.f, I8F_ERR_INVALID_ARG, "eps must not be negative");
    rc = check_out(q, ldq, row_scale, K, y_out, ldy);
    if (rc != I8F_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t nvec = K / 8;
    if (nvec <= 512) {
        // rows of at most 4096 elements: one warp per row
        const unsigned grid_w = static_cast<unsigned>((M + kThreads / 32 - 1) / (kThreads / 32));
        if (x_dtype == I8F_BF16)
            ln_modulate_quant_warp_kernel<I8F_BF16><<<grid_w, kThreads, 0, st>>>(x, M, K, ldx, shift, scale, eps, q, ldq, row_scale, y_out, ldy);
        else
            ln_modulate_quant_warp_kernel<I8F_F16><<<grid_w, kThreads, 0, st>>>(x, M, K, ldx, shift, scale, eps, q, ldq, row_scale, y_out, ldy);
        return check_launch("ln_modulate_quant_warp_kernel");
    }
    const unsigned grid = static_cast<unsigned>((M + 1) / 2);
    if (x_dtype == I8F_BF16)
        I8F_DISPATCH_VPT(ln_modulate_quant_kernel, I8F_BF16, nvec, x, M, K, ldx, shift, scale, eps, q, ldq, row_scale, y_out, ldy);
    else
        I8F_DISPATCH_VPT(ln_modulate_quant_kernel, I8F_F16, nvec, x, M, K, ldx, shift, scale, eps, q, ldq, row_scale, y_out, ldy);
    return check_launch("ln_modulate_quant_kernel");
}

int i8f_quant_rowwise_gelu(const void* x_plain, int64_t K0, int64_t ld0, const void* x_gelu, int64_t K1, int64_t ld1,
                           int x_dtype, int64_t M, int8_t* q, int64_t ldq, float* row_scale, void* y_out, int64_t ldy,
                           void* stream) {
    I8F_REQUIRE(K0 >= 0 && K1 >= 0 && K0 + K1 > 0, I8F_ERR_INVALID_ARG, "empty row");
    I8F_REQUIRE(K0 + K1 <= 16384, I8F_ERR_UNSUPPORTED, "row length %lld exceeds the 16384-element limit", (long long)(K0 + K1));
    int rc = I8F_OK;
    if (K0 > 0) rc = check_rows(x_plain, x_dtype, M, K0, ld0, "i8f_quant_rowwise_gelu (plain part)");
    if (rc != I8F_OK) return rc;
    if (K1 > 0) rc = check_rows(x_gelu, x_dtype, M, K1, ld1, "i8f_quant_rowwise_gelu (GELU part)");
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(x_dtype == I8F_BF16 || x_dtype == I8F_F16, I8F_ERR_UNSUPPORTED, "dtype must be bf16 or f16");
    if (M == 0) return I8F_OK;
    rc = check_out(q, ldq, row_scale, K0 + K1, y_out, ldy);
    if (rc != I8F_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t nvec = (K0 + K1) / 8;
    static const int table_mode = [] {      // I8F_GELU_TABLE = 0 never, 1 always, unset: by size
        const char* e = getenv("I8F_GELU_TABLE");
        return e == nullptr ? -1 : (e[0] == '0' ? 0 : 1);
    }();
    const bool use_table = table_mode == 1 || (table_mode == -1 && M * K1 >= (1 << 21));
    if (use_table) {
        // large inputs: persistent CTAs with the 128 KB look-up table in shared memory (same bits as the direct kernel)
        const unsigned short* table = nullptr;
        rc = gelu_table(x_dtype, st, &table);
        if (rc != I8F_OK) return rc;
        int sms = 148;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int64_t want = (M + 2) / 3;
        const unsigned grid = static_cast<unsigned>(want < sms ? want : sms);
        constexpr int kTableBytes = 65536 * 2;
#define I8F_TABLE_GO(DT, V)                                                                                              \
    do {                                                                                                                 \
        auto kern = gelu_quant_table_kernel<DT, V>;                                                                      \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kTableBytes);            \
        if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));              \
        kern<<<grid, kTableThreads, kTableBytes, st>>>(x_plain, K0, ld0, x_gelu, K1, ld1, M, q, ldq, row_scale, y_out,   \
                                                      ldy, table);                                                       \
    } while (0)
        const int vpt = static_cast<int>((nvec + kThreadsPerRow - 1) / kThreadsPerRow);
        if (x_dtype == I8F_BF16) {
            if (vpt <= 4) I8F_TABLE_GO(I8F_BF16, 4);
            else if (vpt <= 8) I8F_TABLE_GO(I8F_BF16, 8);
            else if (vpt <= 12) I8F_TABLE_GO(I8F_BF16, 12);
            else I8F_TABLE_GO(I8F_BF16, 16);
        } else {
            if (vpt <= 4) I8F_TABLE_GO(I8F_F16, 4);
            else if (vpt <= 8) I8F_TABLE_GO(I8F_F16, 8);
            else if (vpt <= 12) I8F_TABLE_GO(I8F_F16, 12);
            else I8F_TABLE_GO(I8F_F16, 16);
        }
#undef I8F_TABLE_GO
        return check_launch("gelu_quant_table_kernel");
    }
    const unsigned grid = static_cast<unsigned>((M + 1) / 2);
    if (x_dtype == I8F_BF16)
        I8F_DISPATCH_VPT(gelu_quant_kernel, I8F_BF16, nvec, x_plain, K0, ld0, x_gelu, K1, ld1, M, q, ldq, row_scale, y_out, ldy);
    else
        I8F_DISPATCH_VPT(gelu_quant_kernel, I8F_F16, nvec, x_plain, K0, ld0, x_gelu, K1, ld1, M, q, ldq, row_scale, y_out, ldy);
    return check_launch("gelu_quant_kernel");
}

int i8f_rmsnorm_heads(void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ldx, float eps, void* stream) {
    int rc = check_rows(x, x_dtype, rows, cols, ldx, "i8f_rmsnorm_heads");
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(cols % 128 == 0, I8F_ERR_UNSUPPORTED, "cols=%lld must be a multiple of the head size 128", (long long)cols);
    I8F_REQUIRE(eps >= 0.f, I8F_ERR_INVALID_ARG, "eps must not be negative");
    if (rows == 0 || cols == 0) return I8F_OK;
    const int64_t heads = rows * (cols / 128);
    int64_t blocks = (heads + 15) / 16;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_dtype == I8F_BF16) rmsnorm_heads_kernel<I8F_BF16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(x, rows, cols, ldx, eps);
    else rmsnorm_heads_kernel<I8F_F16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(x, rows, cols, ldx, eps);
    return check_launch("rmsnorm_heads_kernel");
}

}  // extern "C"

// Absmax int8 quantisation of matrix rows, optionally fused with the
// 128-block Walsh-Hadamard rotation.  HBM-bound: every element is read once
// with 128-bit loads, kept in registers across the absmax reduction, and
// written once as int8.
//
// Thread layout: a row is owned by TPR threads (power of two, 16..256); thread
// t holds the 8-element vectors t, t+TPR, t+2*TPR, ...  A 128-element
// Hadamard block is therefore spread over 16 consecutive lanes of one warp:
// butterfly strides 1,2,4 stay inside a thread, strides 8..64 are lane
// exchanges (shuffle-xor 1,2,4,8).  The stage order and the a+b / a-b
// assignment follow the natural-order in-place butterfly, which fixes the
// fp32 rounding of every partial sum.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "f32x2.cuh"
#include "host_common.h"

namespace i8f {
namespace {

constexpr int kThreads = 256;
constexpr float kNormHalf = 0.08837890625f;      // bf16(1/sqrt(128)) == fp16(1/sqrt(128))
constexpr float kNormF32 = 0.088388346135616302f;  // fp32(1)/fp32(sqrt(128))
constexpr float kScaleFloor = 1e-30f;

enum Mode : int { kRowwise = 0, kAbsmaxOnly = 1, kGlobalScale = 2 };

template <int DT>
__device__ __forceinline__ void load8(const void* base, int64_t elem_off, float (&v)[8]) {
    if constexpr (DT == I8F_BF16) {
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + elem_off));
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    } else if constexpr (DT == I8F_F16) {
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(base) + elem_off));
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            const float2 f = __half22float2(h);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    } else {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
        const float4 a = __ldg(p), b = __ldg(p + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// Two floats rounded (nearest even) to the 16-bit type DT, packed in a word (a in the low half).
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

// Eight 16-bit values held as loaded (four words) -> eight floats.
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

// Round an fp32 value to the storage type and return it as fp32.
template <int DT>
__device__ __forceinline__ float round_to_dt(float x) {
    if constexpr (DT == I8F_BF16) return __bfloat162float(__float2bfloat16_rn(x));
    else if constexpr (DT == I8F_F16) return __half2float(__float2half_rn(x));
    else return x;
}

template <int DT>
__device__ __forceinline__ void store8(void* base, int64_t elem_off, const float (&v)[8]) {
    if constexpr (DT == I8F_BF16) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + elem_off) = make_uint4(w[0], w[1], w[2], w[3]);
    } else if constexpr (DT == I8F_F16) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(static_cast<__half*>(base) + elem_off) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
        float4* p = reinterpret_cast<float4*>(static_cast<float*>(base) + elem_off);
        p[0] = make_float4(v[0], v[1], v[2], v[3]);
        p[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// 128-point Walsh-Hadamard butterfly over 16 lanes x 8 registers.
__device__ __forceinline__ void wht128(float (&v)[8], int lane) {
#pragma unroll
    for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((i & h) == 0) {
                const float a = v[i], b = v[i + h];
                v[i] = __fadd_rn(a, b);
                v[i + h] = __fsub_rn(a, b);
            }
        }
    }
    // lane exchange stages: the lane with the stride bit clear takes a+b, its partner a-b.  Written as
    // p + s*v with s = +-1 (one fused multiply-add; s*v is exact, so the rounding is that of the add).
#pragma unroll
    for (int d = 1; d < 16; d <<= 1) {
        const float s = (lane & d) != 0 ? -1.0f : 1.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float p = __shfl_xor_sync(0xFFFFFFFFu, v[i], d);
            v[i] = __fmaf_rn(s, v[i], p);
        }
    }
}

// The same 128-point butterfly for a block held by FOUR lanes x four vectors x 8 registers (element index =
// ((c * 4 + l) * 8 + r) for vector c, lane l of the quad, register r): strides 1, 2, 4 inside a vector, strides 8, 16
// across the quad (two shuffle stages instead of four), strides 32, 64 across the thread's vectors.  Same stage
// order and the same a+b / a-b assignment as wht128, hence the same bits.
__device__ __forceinline__ void wht128_quad(float (&v)[4][8], int lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if ((i & h) == 0) {
                    const float a = v[c][i], b = v[c][i + h];
                    v[c][i] = __fadd_rn(a, b);
                    v[c][i + h] = __fsub_rn(a, b);
                }
            }
        }
    }
#pragma unroll
    for (int d = 1; d < 4; d <<= 1) {
        const float s = (lane & d) != 0 ? -1.0f : 1.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float p = __shfl_xor_sync(0xFFFFFFFFu, v[c][i], d);
                v[c][i] = __fmaf_rn(s, v[c][i], p);
            }
        }
    }
#pragma unroll
    for (int h = 1; h < 4; h <<= 1) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if ((c & h) == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float a = v[c][i], b = v[c + h][i];
                    v[c][i] = __fadd_rn(a, b);
                    v[c + h][i] = __fsub_rn(a, b);
                }
            }
        }
    }
}

// One word of two 16-bit values -> the two fp32 values.
template <int DT>
__device__ __forceinline__ void widen2(uint32_t w, float& a, float& b) {
    if constexpr (DT == I8F_BF16) {
        a = __uint_as_float(w << 16);
        b = __uint_as_float(w & 0xFFFF0000u);
    } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        a = f.x;
        b = f.y;
    }
}

// wht128_quad on PAIRED registers: p[c][j] holds elements (2j, 2j+1) of vector c as one two-wide fp32 register, and
// every butterfly stage except stride 1 (whose partners share a pair) is one two-wide add or subtract per pair.
// The stride-1 stage is done while the 16-bit words are widened.  Same operations on the same operands in the same
// order as wht128_quad, hence the same bits, in about 60 % of the instructions.
template <int DT>
__device__ __forceinline__ void wht128_quad_pairs(const uint4 (&raw)[4], f32x2 (&p)[4][4], int lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float a, b;
            widen2<DT>(w[j], a, b);
            p[c][j] = pair_of(__fadd_rn(a, b), __fsub_rn(a, b));   // stride 1
        }
        const f32x2 t0 = add2(p[c][0], p[c][1]), t1 = sub2(p[c][0], p[c][1]);   // stride 2
        const f32x2 t2 = add2(p[c][2], p[c][3]), t3 = sub2(p[c][2], p[c][3]);
        p[c][0] = add2(t0, t2);                                                 // stride 4
        p[c][2] = sub2(t0, t2);
        p[c][1] = add2(t1, t3);
        p[c][3] = sub2(t1, t3);
    }
#pragma unroll
    for (int d = 1; d < 4; d <<= 1) {   // strides 8, 16: across the quad of lanes
        const float s = (lane & d) != 0 ? -1.0f : 1.0f;
        const f32x2 s2 = pair_of(s, s);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float lo, hi;
                halves(p[c][j], lo, hi);
                const f32x2 partner = pair_of(__shfl_xor_sync(0xFFFFFFFFu, lo, d), __shfl_xor_sync(0xFFFFFFFFu, hi, d));
                p[c][j] = fma2(s2, p[c][j], partner);
            }
        }
    }
#pragma unroll
    for (int h = 1; h < 4; h <<= 1) {   // strides 32, 64: across the thread's vectors
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if ((c & h) == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const f32x2 a = p[c][j], b = p[c + h][j];
                    p[c][j] = add2(a, b);
                    p[c + h][j] = sub2(a, b);
                }
            }
        }
    }
}

// Eight 16-bit values as loaded -> eight int8: rint(x * inv) per value through the magic add of quant4, the add
// two-wide.  The multiply stays a scalar __fmul_rn: the product must be rounded BEFORE the add (x * inv often rounds
// to an exact tie such as 63.5 when x is half the row maximum), and the assembler was seen to contract a two-wide
// multiply followed by a two-wide add into one fused operation, whereas a scalar mul.rn is never contracted.
template <int DT>
__device__ __forceinline__ uint2 quant8_packed(const uint4& r, float inv) {
    constexpr float kMagic = 12582912.0f;
    const f32x2 magic2 = pair_of(kMagic, kMagic);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    uint32_t u[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float a, b;
        widen2<DT>(w[j], a, b);
        halves_bits(add2(pair_of(__fmul_rn(a, inv), __fmul_rn(b, inv)), magic2), u[2 * j], u[2 * j + 1]);
    }
    uint2 o;
    o.x = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
    o.y = __byte_perm(__byte_perm(u[4], u[5], 0x0040), __byte_perm(u[6], u[7], 0x0040), 0x5410);
    return o;
}

// Four values -> four int8 packed in a word.  y = x*inv is rounded to the nearest-even integer by
// adding 1.5*2^23 (the sum's low mantissa bits then hold the two's-complement integer), which is
// rint(y) for |y| < 2^22; here |y| <= 127.00002 by construction of the scale, so no clamp is needed.
__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d, float inv) {
    constexpr float kMagic = 12582912.0f;
    const uint32_t ua = __float_as_uint(__fadd_rn(__fmul_rn(a, inv), kMagic));
    const uint32_t ub = __float_as_uint(__fadd_rn(__fmul_rn(b, inv), kMagic));
    const uint32_t uc = __float_as_uint(__fadd_rn(__fmul_rn(c, inv), kMagic));
    const uint32_t ud = __float_as_uint(__fadd_rn(__fmul_rn(d, inv), kMagic));
    return __byte_perm(__byte_perm(ua, ub, 0x0040), __byte_perm(uc, ud, 0x0040), 0x5410);
}

// DT: storage type of x.  VPT: 8-element vectors per thread.  HAD: rotate.
// ROT_F32: rotate in fp32 with the fp32 norm and no rounding (weight rule);
// otherwise the rotated value is rounded to DT (activation rule).
template <int DT, int VPT, bool HAD, bool ROT_F32, int MODE>
__global__ void __launch_bounds__(kThreads)
quant_rows_kernel(const void* __restrict__ x, int64_t M, int64_t K, int64_t ldx, int8_t* __restrict__ q, int64_t ldq,
                  float* __restrict__ scale, void* __restrict__ xrot, float* __restrict__ gmax, int tpr_log2) {
    __shared__ float s_part[kThreads / 32];
    // a GEMM launched behind this kernel with programmatic serialization may begin its set-up once every CTA of
    // this grid has started; it still waits for this grid to complete before it reads anything
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int tpr = 1 << tpr_log2;
    const int rows_per_cta = static_cast<int>(blockDim.x) >> tpr_log2;
    const int t = threadIdx.x & (tpr - 1);
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_cta + (threadIdx.x >> tpr_log2);
    const bool row_ok = row < M;
    const int nvec = static_cast<int>(K >> 3);

    // Which 8-element vector of the row sits in slot i of this thread.  Plain layout: vectors t, t + tpr, ... (a warp
    // load covers 512 contiguous bytes).  With the rotation and at least four vectors per thread, a 128-element
    // block belongs to a QUAD of lanes instead of sixteen: slot i = 4 s + c holds chunk 4 c + (t & 3) of block
    // s * tpr / 4 + t / 4, so a warp load covers eight 64-byte pieces and the butterfly needs half the shuffles.
    constexpr bool kQuad = HAD && (VPT % 4 == 0);
    auto vec_of = [&](int i) -> int {
        if constexpr (kQuad) return (((i >> 2) * (tpr >> 2) + (t >> 2)) << 4) + ((i & 3) << 2) + (t & 3);
        else return i * tpr + t;
    };
    // Without the rotation a 16-bit row stays in registers AS LOADED (four words per vector instead of eight floats)
    // until it is quantised: half the registers, so long rows (8 or 16 vectors per thread) keep 4 / 2 CTAs per SM
    // instead of 2 / 1.  The row maximum is taken on the packed values: non-negative bf16 / fp16 order like their
    // bit patterns, so it is a 16-bit unsigned SIMD max after clearing the sign bits.
    // The same holds with the activation rule of the rotation, whose result is rounded to the 16-bit type anyway:
    // the row is loaded packed, one block at a time is widened, rotated, rounded and packed again.
    constexpr bool kPacked = DT != I8F_F32 && !(HAD && ROT_F32);
    float v[kPacked ? 1 : VPT][8];
    uint4 raw[kPacked ? VPT : 1];
    if constexpr (kPacked) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vec = vec_of(i);
            raw[i] = (row_ok && vec < nvec)
                         ? __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(x) + row * ldx +
                                                                static_cast<int64_t>(vec) * 8))
                         : make_uint4(0u, 0u, 0u, 0u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vec = vec_of(i);
            if (row_ok && vec < nvec) {
                load8<DT>(x, row * ldx + static_cast<int64_t>(vec) * 8, v[i]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
            }
        }
    }

    if constexpr (HAD && kPacked) {
        constexpr float norm = kNormHalf;
        auto repack = [&](const float (&w)[8], uint4& dst) {   // (w * norm) rounded to DT, as packed pairs
            dst.x = pack2<DT>(__fmul_rn(w[0], norm), __fmul_rn(w[1], norm));
            dst.y = pack2<DT>(__fmul_rn(w[2], norm), __fmul_rn(w[3], norm));
            dst.z = pack2<DT>(__fmul_rn(w[4], norm), __fmul_rn(w[5], norm));
            dst.w = pack2<DT>(__fmul_rn(w[6], norm), __fmul_rn(w[7], norm));
        };
        if constexpr (kQuad) {
#pragma unroll
            for (int sgrp = 0; sgrp < VPT / 4; ++sgrp) {
                f32x2 p[4][4];
                wht128_quad_pairs<DT>(*reinterpret_cast<const uint4(*)[4]>(&raw[4 * sgrp]), p, lane);
                const f32x2 norm2 = pair_of(norm, norm);
#pragma unroll
                for (int c = 0; c < 4; ++c) {   // (w * norm) rounded to DT, as packed pairs
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float lo, hi;
                        halves(mul2(p[c][j], norm2), lo, hi);
                        o[j] = pack2<DT>(lo, hi);
                    }
                    raw[4 * sgrp + c] = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                float w[8];
                unpack8<DT>(raw[i], w);
                wht128(w, lane);
                repack(w, raw[i]);
            }
        }
        if constexpr (MODE == kRowwise) {
            if (xrot != nullptr && row_ok) {
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int vec = vec_of(i);
                    if (vec < nvec)
                        *reinterpret_cast<uint4*>(static_cast<unsigned short*>(xrot) + row * ldx + static_cast<int64_t>(vec) * 8) = raw[i];
                }
            }
        }
    } else if constexpr (HAD) {
        constexpr float norm = kNormF32;   // fp32 rule: rotate in fp32, fp32 norm, no rounding (DT == fp32 or weights)
        if constexpr (kQuad) {
#pragma unroll
            for (int sgrp = 0; sgrp < VPT / 4; ++sgrp) wht128_quad(*reinterpret_cast<float(*)[4][8]>(&v[4 * sgrp]), lane);
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if constexpr (!kQuad) wht128(v[i], lane);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float r = __fmul_rn(v[i][j], norm);
                v[i][j] = ROT_F32 ? r : round_to_dt<DT>(r);
            }
            if constexpr (MODE == kRowwise) {
                const int vec = vec_of(i);
                if (xrot != nullptr && row_ok && vec < nvec) store8<DT>(xrot, row * ldx + static_cast<int64_t>(vec) * 8, v[i]);
            }
        }
    }

    float amax = 0.f;
    if constexpr (MODE != kGlobalScale) {
        if constexpr (kPacked) {
            uint32_t m2 = 0u;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                m2 = __vmaxu2(m2, raw[i].x & 0x7FFF7FFFu);
                m2 = __vmaxu2(m2, raw[i].y & 0x7FFF7FFFu);
                m2 = __vmaxu2(m2, raw[i].z & 0x7FFF7FFFu);
                m2 = __vmaxu2(m2, raw[i].w & 0x7FFF7FFFu);
            }
            const uint32_t m16 = max(m2 & 0xFFFFu, m2 >> 16);
            if constexpr (DT == I8F_BF16) amax = __uint_as_float(m16 << 16);
            else amax = __half2float(__ushort_as_half(static_cast<unsigned short>(m16)));
        } else {
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int j = 0; j < 8; j += 2) amax = fmaxf(fmaxf(amax, fabsf(v[i][j])), fabsf(v[i][j + 1]));
        }
        // reduce over the lanes of this row that share a warp
        // (the whole warp when only the tensor-wide maximum is wanted)
        const int span = (MODE == kAbsmaxOnly || tpr > 32) ? 32 : tpr;
        for (int d = 1; d < span; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
        if (tpr > 32 || MODE == kAbsmaxOnly) {
            if (lane == 0) s_part[threadIdx.x >> 5] = amax;
            __syncthreads();
            if constexpr (MODE == kAbsmaxOnly) {
                if (threadIdx.x == 0) {
                    float m = 0.f;
                    for (int w = 0; w < static_cast<int>(blockDim.x) / 32; ++w) m = fmaxf(m, s_part[w]);
                    // non-negative floats order like their bit patterns
                    atomicMax(reinterpret_cast<int*>(gmax), __float_as_int(m));
                }
                return;
            } else {
                const int warps_per_row = tpr >> 5;
                const int first = (threadIdx.x >> tpr_log2) * warps_per_row;
                float m = 0.f;
                for (int w = 0; w < warps_per_row; ++w) m = fmaxf(m, s_part[first + w]);
                amax = m;
            }
        }
    } else {
        amax = *gmax;
    }

    const float sc = fmaxf(__fdiv_rn(amax, 127.0f), kScaleFloor);
    const float inv = __fdiv_rn(1.0f, sc);
    if constexpr (MODE == kRowwise) {
        if (row_ok && t == 0) scale[row] = sc;
    } else {
        if (blockIdx.x == 0 && threadIdx.x == 0) scale[0] = sc;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vec = vec_of(i);
        if (row_ok && vec < nvec) {
            uint2 o;
            if constexpr (kPacked) {
                o = quant8_packed<DT>(raw[i], inv);
            } else {
                o.x = quant4(v[i][0], v[i][1], v[i][2], v[i][3], inv);
                o.y = quant4(v[i][4], v[i][5], v[i][6], v[i][7], inv);
            }
            *reinterpret_cast<uint2*>(q + row * ldq + static_cast<int64_t>(vec) * 8) = o;
        }
    }
}

struct Plan {
    int tpr_log2;
    int vpt;
};

// Pick threads-per-row and vectors-per-thread: prefer 4 vectors (64 bytes of
// bf16) in flight per thread, grow the row group up to the whole CTA, then
// grow the per-thread count up to 16.
inline bool make_plan(int64_t K, Plan* p) {
    const int64_t nvec = K / 8;
    int tpr_log2 = 4;
    while (tpr_log2 < 8 && (nvec + (int64_t(1) << tpr_log2) - 1) / (int64_t(1) << tpr_log2) > 4) ++tpr_log2;
    const int64_t need = (nvec + (int64_t(1) << tpr_log2) - 1) >> tpr_log2;
    int vpt = 1;
    while (vpt < need) vpt <<= 1;
    if (vpt > 16) return false;
    p->tpr_log2 = tpr_log2;
    p->vpt = vpt;
    return true;
}

template <int DT, bool HAD, bool ROT_F32, int MODE>
int launch_vpt(const Plan& p, const void* x, int64_t M, int64_t K, int64_t ldx, int8_t* q, int64_t ldq, float* scale,
               void* xrot, float* gmax, cudaStream_t st) {
    // CTA size: 128 threads where a row needs no more (finer-grained CTAs: 14.6 -> 14.3 us with rotation and
    // 10.3 -> 10.0 us without at 4096 x 4096), else 256; I8F_K1_THREADS=256 forces the larger one
    static const int want_threads = [] {
        const char* e = getenv("I8F_K1_THREADS");
        return (e != nullptr && atoi(e) == 256) ? 256 : 128;
    }();
    const int threads = (want_threads == 128 && p.tpr_log2 <= 7) ? 128 : kThreads;
    const int rows_per_cta = threads >> p.tpr_log2;
    const unsigned grid = static_cast<unsigned>((M + rows_per_cta - 1) / rows_per_cta);
#define I8F_LAUNCH(V)                                                                                              \
    quant_rows_kernel<DT, V, HAD, ROT_F32, MODE><<<grid, threads, 0, st>>>(x, M, K, ldx, q, ldq, scale, xrot, gmax, \
                                                                            p.tpr_log2)
    switch (p.vpt) {
        case 1: I8F_LAUNCH(1); break;
        case 2: I8F_LAUNCH(2); break;
        case 4: I8F_LAUNCH(4); break;
        case 8: I8F_LAUNCH(8); break;
        default: I8F_LAUNCH(16); break;
    }
#undef I8F_LAUNCH
    return check_launch("quant_rows_kernel");
}

template <bool ROT_F32, int MODE>
int launch_any(int dt, bool had, const Plan& p, const void* x, int64_t M, int64_t K, int64_t ldx, int8_t* q, int64_t ldq,
               float* scale, void* xrot, float* gmax, cudaStream_t st) {
#define I8F_GO(DT)                                                                                           \
    (had ? launch_vpt<DT, true, ROT_F32, MODE>(p, x, M, K, ldx, q, ldq, scale, xrot, gmax, st)                \
         : launch_vpt<DT, false, ROT_F32, MODE>(p, x, M, K, ldx, q, ldq, scale, xrot, gmax, st))
    switch (dt) {
        case I8F_BF16: return I8F_GO(I8F_BF16);
        case I8F_F16: return I8F_GO(I8F_F16);
        default: return I8F_GO(I8F_F32);
    }
#undef I8F_GO
}

int check_common(const void* x, int dt, int64_t M, int64_t K, int64_t ldx, const int8_t* q, int64_t ldq, int had,
                 Plan* plan) {
    I8F_REQUIRE(dtype_size(dt) != 0, I8F_ERR_INVALID_ARG, "unknown dtype code %d", dt);
    I8F_REQUIRE(M >= 0 && K >= 0, I8F_ERR_INVALID_ARG, "negative shape M=%lld K=%lld", (long long)M, (long long)K);
    if (M == 0 || K == 0) return I8F_OK;
    I8F_REQUIRE(x != nullptr && q != nullptr, I8F_ERR_INVALID_ARG, "NULL input or output pointer");
    I8F_REQUIRE(ldx >= K && ldq >= K, I8F_ERR_INVALID_ARG, "row pitch smaller than K");
    I8F_REQUIRE(K % 8 == 0, I8F_ERR_UNSUPPORTED, "K=%lld must be a multiple of 8", (long long)K);
    I8F_REQUIRE(!had || K % 128 == 0, I8F_ERR_UNSUPPORTED, "Hadamard rotation needs K %% 128 == 0 (K=%lld)", (long long)K);
    I8F_REQUIRE(aligned16(x) && (ldx * dtype_size(dt)) % 16 == 0, I8F_ERR_ALIGNMENT,
                "input must be 16-byte aligned with a 16-byte multiple row pitch");
    I8F_REQUIRE((reinterpret_cast<uintptr_t>(q) & 7u) == 0 && ldq % 8 == 0, I8F_ERR_ALIGNMENT,
                "int8 output must be 8-byte aligned with an 8-byte multiple row pitch");
    I8F_REQUIRE(make_plan(K, plan), I8F_ERR_UNSUPPORTED, "K=%lld exceeds the 32768-element row limit", (long long)K);
    return I8F_OK;
}

}  // namespace
}  // namespace i8f

using namespace i8f;

extern "C" {

int i8f_quant_rowwise(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* q, int64_t ldq,
                      float* scale, int hadamard128, void* x_rot_out, void* stream) {
    Plan plan{};
    int rc = check_common(x, x_dtype, M, K, ldx, q, ldq, hadamard128, &plan);
    if (rc != I8F_OK) return rc;
    if (M == 0) return I8F_OK;
    I8F_REQUIRE(scale != nullptr, I8F_ERR_INVALID_ARG, "scale is NULL");
    if (K == 0) {
        // empty rows: absmax 0 -> floor scale (matches the clamp on an empty reduction of zeros)
        return fail(I8F_ERR_UNSUPPORTED, "K == 0 is not supported");
    }
    I8F_REQUIRE(x_rot_out == nullptr || aligned16(x_rot_out), I8F_ERR_ALIGNMENT, "x_rot_out must be 16-byte aligned");
    return launch_any<false, kRowwise>(x_dtype, hadamard128 != 0, plan, x, M, K, ldx, q, ldq, scale,
                                       hadamard128 ? x_rot_out : nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

int i8f_quant_weight_rows(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int8_t* q, int64_t ldq,
                          float* scale, int hadamard128, void* stream) {
    Plan plan{};
    int rc = check_common(w, w_dtype, N, K, ldw, q, ldq, hadamard128, &plan);
    if (rc != I8F_OK) return rc;
    if (N == 0) return I8F_OK;
    I8F_REQUIRE(scale != nullptr && K > 0, I8F_ERR_INVALID_ARG, "scale is NULL or K == 0");
    return launch_any<true, kRowwise>(w_dtype, hadamard128 != 0, plan, w, N, K, ldw, q, ldq, scale, nullptr, nullptr,
                                      static_cast<cudaStream_t>(stream));
}

int i8f_quant_tensorwise(const void* x, int x_dtype, int64_t N, int64_t K, int64_t ldx, int8_t* q, int64_t ldq,
                         float* scale_out, int hadamard128, void* scratch, void* stream) {
    Plan plan{};
    int rc = check_common(x, x_dtype, N, K, ldx, q, ldq, hadamard128, &plan);
    if (rc != I8F_OK) return rc;
    I8F_REQUIRE(N > 0 && K > 0, I8F_ERR_INVALID_ARG, "empty tensor");
    I8F_REQUIRE(scale_out != nullptr && scratch != nullptr, I8F_ERR_INVALID_ARG, "scale_out or scratch is NULL");
    I8F_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 3u) == 0, I8F_ERR_ALIGNMENT, "scratch must be 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* gmax = static_cast<float*>(scratch);
    cudaError_t e = cudaMemsetAsync(gmax, 0, sizeof(float), st);
    if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    rc = launch_any<true, kAbsmaxOnly>(x_dtype, hadamard128 != 0, plan, x, N, K, ldx, q, ldq, scale_out, nullptr, gmax, st);
    if (rc != I8F_OK) return rc;
    return launch_any<true, kGlobalScale>(x_dtype, hadamard128 != 0, plan, x, N, K, ldx, q, ldq, scale_out, nullptr, gmax, st);
}

}  // extern "C"

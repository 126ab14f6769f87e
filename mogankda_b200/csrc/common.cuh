// Shared device helpers for the KDA / GDN kernels (sm_100a).
//
// Numerics policy: every contraction runs on the tensor cores with the error-compensated three-product split
// (a = hi + lo, a*b ~ lo_a*hi_b + hi_a*lo_b + hi_a*hi_b) and fp32 accumulation: bf16 halves on tcgen05 in the chunk
// kernels (umma.cuh), TF32 halves on mma.sync in the small prefix-combine kernel (PREC = 3 below; PREC = 1 is the plain
// single product).  Inputs may be fp32, bf16 or fp16 in global memory; they are widened to fp32 when staged.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mkda.h"

namespace mkda {

constexpr int CH = 64;    // chunk length
constexpr int DK = 128;   // key dim
constexpr int DV = 128;   // value dim
constexpr float RCP_LN2 = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------------------
// typed global access: 4 consecutive elements starting at element index `idx` (idx % 4 == 0)
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float4 ld4(const void* base, int dtype, size_t idx) {
    if (dtype == MKDA_F32) return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
    uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + idx);
    float4 r;
    if (dtype == MKDA_BF16) {
        r.x = __uint_as_float(raw.x << 16);
        r.y = __uint_as_float(raw.x & 0xffff0000u);
        r.z = __uint_as_float(raw.y << 16);
        r.w = __uint_as_float(raw.y & 0xffff0000u);
    } else {
        __half2 a = *reinterpret_cast<__half2*>(&raw.x), b = *reinterpret_cast<__half2*>(&raw.y);
        float2 fa = __half22float2(a), fb = __half22float2(b);
        r = make_float4(fa.x, fa.y, fb.x, fb.y);
    }
    return r;
}

// 8 consecutive elements starting at element index `idx` (idx % 8 == 0): one 16-byte load for the 16-bit types
__device__ __forceinline__ void ld8(const void* base, int dtype, size_t idx, float (&v)[8]) {
    if (dtype == MKDA_F32) {
        const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
        const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        return;
    }
    const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + idx);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (dtype == MKDA_BF16) {
            v[2 * e] = __uint_as_float(w[e] << 16);
            v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            v[2 * e] = f.x; v[2 * e + 1] = f.y;
        }
    }
}

// The same eight elements as raw bytes (one 16-byte piece, two for fp32), widened later by unpack8.  A conversion next to the
// load makes the thread wait for the data there and then; a load whose bytes are only parked in registers stays in flight
// until its first real use, which may be a whole phase (or the top of the next item) later.
struct Raw8 { uint4 a, b; };
template <int DT>
__device__ __forceinline__ void ldraw8(const void* base, size_t idx, Raw8& r) {
    if (DT == MKDA_F32) {
        r.a = *reinterpret_cast<const uint4*>(static_cast<const float*>(base) + idx);
        r.b = *reinterpret_cast<const uint4*>(static_cast<const float*>(base) + idx + 4);
    } else {
        r.a = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + idx);
    }
}
template <int DT>
__device__ __forceinline__ void unpack8(const Raw8& r, float (&v)[8]) {
    if (DT == MKDA_F32) {
        v[0] = __uint_as_float(r.a.x); v[1] = __uint_as_float(r.a.y); v[2] = __uint_as_float(r.a.z); v[3] = __uint_as_float(r.a.w);
        v[4] = __uint_as_float(r.b.x); v[5] = __uint_as_float(r.b.y); v[6] = __uint_as_float(r.b.z); v[7] = __uint_as_float(r.b.w);
        return;
    }
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (DT == MKDA_BF16) {
            v[2 * e] = __uint_as_float(w[e] << 16);
            v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            v[2 * e] = f.x; v[2 * e + 1] = f.y;
        }
    }
}
// one element, raw (zero-extended for the 16-bit types) and widened later
template <int DT>
__device__ __forceinline__ uint32_t ldraw1(const void* base, size_t idx) {
    if (DT == MKDA_F32) return static_cast<const uint32_t*>(base)[idx];
    return static_cast<const uint16_t*>(base)[idx];
}
template <int DT>
__device__ __forceinline__ float unpack1(uint32_t w) {
    if (DT == MKDA_F32) return __uint_as_float(w);
    if (DT == MKDA_BF16) return __uint_as_float(w << 16);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(w)));
}

__device__ __forceinline__ float ld1(const void* base, int dtype, size_t idx) {
    if (dtype == MKDA_F32) return static_cast<const float*>(base)[idx];
    if (dtype == MKDA_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    return __half2float(static_cast<const __half*>(base)[idx]);
}

__device__ __forceinline__ void st1(void* base, int dtype, size_t idx, float v) {
    if (dtype == MKDA_F32) static_cast<float*>(base)[idx] = v;
    else if (dtype == MKDA_BF16) static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
    else static_cast<__half*>(base)[idx] = __float2half_rn(v);
}

__device__ __forceinline__ void st2(void* base, int dtype, size_t idx, float a, float b) {   // idx % 2 == 0
    if (dtype == MKDA_F32) {
        *reinterpret_cast<float2*>(static_cast<float*>(base) + idx) = make_float2(a, b);
    } else if (dtype == MKDA_BF16) {
        *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(base) + idx) = __floats2bfloat162_rn(a, b);
    } else {
        *reinterpret_cast<__half2*>(static_cast<__half*>(base) + idx) = __floats2half2_rn(a, b);
    }
}

__device__ __forceinline__ void st4(void* base, int dtype, size_t idx, float4 v) {          // idx % 4 == 0
    if (dtype == MKDA_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = v;
    } else if (dtype == MKDA_BF16) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(base) + idx) = raw;
    } else {
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 raw = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(base) + idx) = raw;
    }
}

// ---------------------------------------------------------------------------------------------------------
// tensor-core primitive: m16n8k8 TF32, fp32 accumulate.
// Fragment ownership (g = lane >> 2, t = lane & 3):
//   A (16x8):  a0 (g, t)  a1 (g+8, t)  a2 (g, t+4)  a3 (g+8, t+4)
//   B (8x8):   b0 (k = t, n = g)       b1 (k = t+4, n = g)
//   C (16x8):  c0 (g, 2t) c1 (g, 2t+1) c2 (g+8, 2t) c3 (g+8, 2t+1)
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void mma_tf32_raw(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int PREC>
struct FragA {
    uint32_t hi[4];
    uint32_t lo[PREC == 3 ? 4 : 1];
    __device__ __forceinline__ void set(int i, float x) {
        hi[i] = to_tf32(x);
        if (PREC == 3) lo[i] = to_tf32(x - __uint_as_float(hi[i]));
    }
};
template <int PREC>
struct FragB {
    uint32_t hi[2];
    uint32_t lo[PREC == 3 ? 2 : 1];
    __device__ __forceinline__ void set(int i, float x) {
        hi[i] = to_tf32(x);
        if (PREC == 3) lo[i] = to_tf32(x - __uint_as_float(hi[i]));
    }
};

template <int PREC>
__device__ __forceinline__ void mma_frag(float (&d)[4], const FragA<PREC>& a, const FragB<PREC>& b) {
    if (PREC == 3) {
        uint32_t alo[4] = {a.lo[0], a.lo[PREC == 3 ? 1 : 0], a.lo[PREC == 3 ? 2 : 0], a.lo[PREC == 3 ? 3 : 0]};
        uint32_t blo[2] = {b.lo[0], b.lo[PREC == 3 ? 1 : 0]};
        mma_tf32_raw(d, alo, b.hi);
        mma_tf32_raw(d, a.hi, blo);
    }
    mma_tf32_raw(d, a.hi, b.hi);
}

// acc[NT][4] += A(16 x Kd) * B(Kd x 8*NT) for one warp.
//   A(m, k) = A[m * ARS + k * ACS]   (pointer already offset to the warp's first row)
//   B(k, n) = B[k * BKS + n * BNS]   (pointer already offset to the warp's first column)
// Kd must be a multiple of 8.
template <int NT, int PREC, int ARS, int ACS, int BKS, int BNS>
__device__ __forceinline__ void warp_mma(float (&acc)[NT][4], const float* __restrict__ A,
                                         const float* __restrict__ B, int Kd) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const float* ap = A + g * ARS + t * ACS;
    const float* bp = B + t * BKS + g * BNS;
#pragma unroll 2
    for (int k0 = 0; k0 < Kd; k0 += 8) {
        FragA<PREC> fa;
        fa.set(0, ap[k0 * ACS]);
        fa.set(1, ap[8 * ARS + k0 * ACS]);
        fa.set(2, ap[(k0 + 4) * ACS]);
        fa.set(3, ap[8 * ARS + (k0 + 4) * ACS]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            FragB<PREC> fb;
            fb.set(0, bp[k0 * BKS + nt * 8 * BNS]);
            fb.set(1, bp[(k0 + 4) * BKS + nt * 8 * BNS]);
            mma_frag<PREC>(acc[nt], fa, fb);
        }
    }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
}

// 2^x in one MUFU instruction (max relative error ~2^-22); used where 2^x scales tensor-core operands
__device__ __forceinline__ float ex2f_(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Stable scalar math on the MUFU unit (ex2 / lg2 / rcp approximations, relative error ~1e-7 each, absolute error of
// softplus < 1e-7): the gate and epilogue kernels evaluate several of these per element and were ALU-bound with the
// precise library versions.
__device__ __forceinline__ float expf_(float x) { return ex2f_(x * RCP_LN2); }
__device__ __forceinline__ float sigmoidf_(float z) { return __fdividef(1.f, 1.f + expf_(-z)); }
__device__ __forceinline__ float softplusf_(float s) { return fmaxf(s, 0.f) + __log2f(1.f + expf_(-fabsf(s))) * LN2; }

// Chunk geometry shared by all chunk-parallel kernels: flattened first token and number of valid rows.
struct ChunkGeom {
    int start, len;
};
__device__ __forceinline__ ChunkGeom chunk_geom(const int* chunk_start, const int* chunk_len, int c) {
    ChunkGeom gmt;
    gmt.start = chunk_start[c];
    gmt.len = chunk_len[c];
    return gmt;
}

}  // namespace mkda

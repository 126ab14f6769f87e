// Serial chunk recurrences (forward state pass, reverse state-gradient pass), the chunk-parallel output kernel and
// the per-segment prefix combine used by context parallelism.
//
// Work decomposition of the serial kernels: one CTA (8 warps) per (64-column block of the state, v-head, segment).
// The [128 x 64] fp32 state block lives in the MMA accumulators of the 8 warps (warp w owns K rows 16w..16w+15)
// across the whole segment; a shared-memory copy is refreshed once per chunk because the next chunk consumes the
// state as a B operand.
#include "common.cuh"
#include "host.h"

#ifndef MKDA_PREC_STATE
#define MKDA_PREC_STATE 1
#endif
#ifndef MKDA_PREC_DH
#define MKDA_PREC_DH 1
#endif
#ifndef MKDA_PREC_OUT
#define MKDA_PREC_OUT 1
#endif
#ifndef MKDA_PREC_COMBINE
#define MKDA_PREC_COMBINE 3
#endif

namespace mkda {

constexpr int LDA = 132;   // [64][128] tile read as A(m = row, k = col)          (row stride = 4 mod 32)
constexpr int LDT = 136;   // [64][128] tile read as A(m = col, k = row) or B(k = row, n = col)   (8 mod 32)
constexpr int LDS = 72;    // [128][64] / [64][64] tile read as B(k = row, n = col)
constexpr int LDM = 68;    // [64][64] tile read as A(m = row, k = col)

__device__ __forceinline__ size_t state_index(bool v_first, int kk, int vv) {
    return v_first ? (size_t)vv * DK + kk : (size_t)kk * DV + vv;
}

// ---------------------------------------------------------------------------------------------------------
// forward state pass
// ---------------------------------------------------------------------------------------------------------
constexpr int RECUR_SMEM = (DK * LDS + CH * LDA + CH * LDT + CH * LDS + DK) * 4;

template <int PREC>
__global__ void __launch_bounds__(256, 1) recur_fwd_kernel(const MkdaRecurFwd p) {
    extern __shared__ __align__(16) float smem[];
    float* sS = smem;                  // [128][LDS]  state block, B(k = K index, n = column)
    float* sW = sS + DK * LDS;         // [64][LDA]   nw rows, A(m = token, k = K index)
    float* sKb = sW + CH * LDA;        // [64][LDT]   kbar rows, A(m = K index, k = token)
    float* sVd = sKb + CH * LDT;       // [64][LDS]   Vd block, B(k = token, n = column)
    float* sGl = sVd + CH * LDS;       // [128]       2^(g at last valid row)

    const int cb = blockIdx.x, h = blockIdx.y, seg = blockIdx.z, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const bool trans = cb >= 2;                    // transition-matrix columns
    const int col0 = (cb & 1) * 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp & 3, wn = warp >> 2;
    const bool vf = p.state_v_first != 0;

    // state accumulators: rows kr0 = 16 warp + g, kr0 + 8; columns col0 + nt*8 + 2t (+1)
    float S[8][4];
    const int kr0 = warp * 16 + g, kr1 = kr0 + 8;
    {
        const int h0row = p.seg_h0 ? p.seg_h0[seg] : seg;
        const float* h0 = (!trans && p.h0 && h0row >= 0) ? p.h0 + ((size_t)h0row * HV + h) * DK * DV : nullptr;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = (e & 2) ? kr1 : kr0, cc = col0 + nt * 8 + 2 * t + (e & 1);
                float v = 0.f;
                if (trans) v = (kk == cc) ? 1.f : 0.f;
                else if (h0) v = h0[state_index(vf, kk, cc)];
                S[nt][e] = v;
            }
        }
    }

    const int c_beg = p.L.seg_chunk_off[seg], c_end = p.L.seg_chunk_off[seg + 1];
    for (int c = c_beg; c < c_end; ++c) {
        const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
        // publish the entering state: shared copy for the MMA, optional global copy for the backward
        float* hc = (p.h && !trans) ? p.h + ((size_t)c * HV + h) * DK * DV : nullptr;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int cc = nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(sS + kr0 * LDS + cc) = make_float2(S[nt][0], S[nt][1]);
            *reinterpret_cast<float2*>(sS + kr1 * LDS + cc) = make_float2(S[nt][2], S[nt][3]);
            if (hc) {
                *reinterpret_cast<float2*>(hc + (size_t)kr0 * DV + col0 + cc) = make_float2(S[nt][0], S[nt][1]);
                *reinterpret_cast<float2*>(hc + (size_t)kr1 * DV + col0 + cc) = make_float2(S[nt][2], S[nt][3]);
            }
        }
        // stage nw and kbar = k 2^(g_last - g); rows >= len are zero
        const float* glast = p.g_c + ((size_t)(start + len - 1) * HV + h) * 128;
        for (int i = tid; i < CH * 32; i += 256) {
            const int r = i >> 5, c4 = (i & 31) * 4;
            float4 w = make_float4(0.f, 0.f, 0.f, 0.f), kb = w;
            if (r < len) {
                const size_t th = (size_t)(start + r) * HV + h;
                w = *reinterpret_cast<const float4*>(p.nw + th * 128 + c4);
                const size_t tk = (size_t)(start + r) * HK + hk;
                kb = ld4(p.k, p.k_dtype, tk * 128 + c4);
                const float rs = p.k_rstd ? p.k_rstd[tk] : 1.f;
                const float4 gr = *reinterpret_cast<const float4*>(p.g_c + th * 128 + c4);
                const float4 gL = *reinterpret_cast<const float4*>(glast + c4);
                kb.x *= rs * exp2f(gL.x - gr.x); kb.y *= rs * exp2f(gL.y - gr.y);
                kb.z *= rs * exp2f(gL.z - gr.z); kb.w *= rs * exp2f(gL.w - gr.w);
            }
            *reinterpret_cast<float4*>(sW + r * LDA + c4) = w;
            *reinterpret_cast<float4*>(sKb + r * LDT + c4) = kb;
        }
        if (tid < DK) sGl[tid] = exp2f(glast[tid]);
        // Vd block = u + nw S  (warp (wm, wn): rows 16 wm.., columns 32 wn..)
        float acc[4][4];
        {
            const int r0 = wm * 16 + g, r1 = r0 + 8;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int cc = col0 + wn * 32 + nt * 8 + 2 * t;
                float2 a = make_float2(0.f, 0.f), b = a;
                if (!trans) {
                    if (r0 < len) a = *reinterpret_cast<const float2*>(p.u + ((size_t)(start + r0) * HV + h) * 128 + cc);
                    if (r1 < len) b = *reinterpret_cast<const float2*>(p.u + ((size_t)(start + r1) * HV + h) * 128 + cc);
                }
                acc[nt][0] = a.x; acc[nt][1] = a.y; acc[nt][2] = b.x; acc[nt][3] = b.y;
            }
        }
        __syncthreads();
        warp_mma<4, PREC, LDA, 1, LDS, 1>(acc, sW + wm * 16 * LDA, sS + wn * 32, DK);
        {
            const int r0 = wm * 16 + g, r1 = r0 + 8;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int cl = wn * 32 + nt * 8 + 2 * t;
                *reinterpret_cast<float2*>(sVd + r0 * LDS + cl) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2*>(sVd + r1 * LDS + cl) = make_float2(acc[nt][2], acc[nt][3]);
                if (p.Vd && !trans) {
                    if (r0 < len) *reinterpret_cast<float2*>(p.Vd + ((size_t)(start + r0) * HV + h) * 128 + col0 + cl) = make_float2(acc[nt][0], acc[nt][1]);
                    if (r1 < len) *reinterpret_cast<float2*>(p.Vd + ((size_t)(start + r1) * HV + h) * 128 + col0 + cl) = make_float2(acc[nt][2], acc[nt][3]);
                }
            }
        }
        __syncthreads();
        // S <- diag(gl) S + kbar^T Vd
        {
            const float g0 = sGl[kr0], g1 = sGl[kr1];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) { S[nt][0] *= g0; S[nt][1] *= g0; S[nt][2] *= g1; S[nt][3] *= g1; }
        }
        warp_mma<8, PREC, 1, LDT, LDS, 1>(S, sKb + warp * 16, sVd, CH);
        __syncthreads();
    }
    // state leaving the segment
    float* out = nullptr;
    if (trans) { if (p.mt) out = p.mt + ((size_t)seg * HV + h) * DK * DK; }
    else if (p.ht) out = p.ht + ((size_t)seg * HV + h) * DK * DV;
    if (out) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = (e & 2) ? kr1 : kr0, cc = col0 + nt * 8 + 2 * t + (e & 1);
                out[trans ? (size_t)kk * DK + cc : state_index(vf, kk, cc)] = S[nt][e];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// chunk-parallel output (+ gated RMSNorm epilogue): one CTA per (chunk, v-head), warp (wm, wn) owns rows 16 wm..
// and columns 64 wn..
// ---------------------------------------------------------------------------------------------------------
constexpr int OUT_SMEM = (DK * LDT + CH * LDA + CH * LDM + CH * LDT + 2 * CH) * 4;

template <int PREC>
__global__ void __launch_bounds__(256, 1) out_fwd_kernel(const MkdaOutFwd p) {
    extern __shared__ __align__(16) float smem[];
    float* sH = smem;                  // [128][LDT]  B(k = K index, n = v)
    float* sQ = sH + DK * LDT;         // [64][LDA]   scale q 2^g, A(m = token, k = K index)
    float* sA = sQ + CH * LDA;         // [64][LDM]   Aqk, A(m = i, k = j)
    float* sVd = sA + CH * LDM;        // [64][LDT]   B(k = token, n = v)
    float* sRed = sVd + CH * LDT;      // [2][64]

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp & 3, wn = warp >> 2;

    const float* hc = p.h + ((size_t)c * HV + h) * DK * DV;
    for (int i = tid; i < DK * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        *reinterpret_cast<float4*>(sH + r * LDT + c4) = *reinterpret_cast<const float4*>(hc + (size_t)r * DV + c4);
    }
    for (int i = tid; i < CH * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f), vd = q;
        if (r < len) {
            const size_t th = (size_t)(start + r) * HV + h, tk = (size_t)(start + r) * HK + hk;
            q = ld4(p.q, p.q_dtype, tk * 128 + c4);
            const float m = p.scale * (p.q_rstd ? p.q_rstd[tk] : 1.f);
            const float4 gr = *reinterpret_cast<const float4*>(p.g_c + th * 128 + c4);
            q.x *= m * exp2f(gr.x); q.y *= m * exp2f(gr.y); q.z *= m * exp2f(gr.z); q.w *= m * exp2f(gr.w);
            vd = *reinterpret_cast<const float4*>(p.Vd + th * 128 + c4);
        }
        *reinterpret_cast<float4*>(sQ + r * LDA + c4) = q;
        *reinterpret_cast<float4*>(sVd + r * LDT + c4) = vd;
    }
    stage_rows64<LDM, 256>(sA, p.Aqk, start, len, HV, h);
    __syncthreads();

    float acc[8][4];
    zero_acc<8>(acc);
    warp_mma<8, PREC, LDA, 1, LDT, 1>(acc, sQ + wm * 16 * LDA, sH + wn * 64, DK);
    warp_mma<8, PREC, LDM, 1, LDT, 1>(acc, sA + wm * 16 * LDM, sVd + wn * 64, 16 * (wm + 1));   // Aqk is lower triangular

    const int r0 = wm * 16 + g, r1 = r0 + 8;
    float rs0 = 1.f, rs1 = 1.f;
    if (p.has_norm) {
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            s0 += acc[nt][0] * acc[nt][0] + acc[nt][1] * acc[nt][1];
            s1 += acc[nt][2] * acc[nt][2] + acc[nt][3] * acc[nt][3];
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        if (t == 0) { sRed[wn * CH + r0] = s0; sRed[wn * CH + r1] = s1; }
        __syncthreads();
        rs0 = 1.f / sqrtf((sRed[r0] + sRed[CH + r0]) * (1.f / 128.f) + p.eps);
        rs1 = 1.f / sqrtf((sRed[r1] + sRed[CH + r1]) * (1.f / 128.f) + p.eps);
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        const int col = wn * 64 + nt * 8 + 2 * t;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? r1 : r0;
            if (r >= len) continue;
            const size_t off = ((size_t)(start + r) * HV + h) * 128 + col;
            float a = acc[nt][2 * half], b = acc[nt][2 * half + 1];
            if (p.o_raw) *reinterpret_cast<float2*>(p.o_raw + off) = make_float2(a, b);
            if (p.has_norm) {
                const float rs = half ? rs1 : rs0;
                float w0 = 1.f, w1 = 1.f;
                if (p.norm_w) { w0 = ld1(p.norm_w, p.norm_w_dtype, col); w1 = ld1(p.norm_w, p.norm_w_dtype, col + 1); }
                const float z0 = ld1(p.gate, p.gate_dtype, off), z1 = ld1(p.gate, p.gate_dtype, off + 1);
                const float s0 = sigmoidf_(z0), s1 = sigmoidf_(z1);
                a *= rs * w0 * (p.act == MKDA_ACT_SILU ? z0 * s0 : s0);
                b *= rs * w1 * (p.act == MKDA_ACT_SILU ? z1 * s1 : s1);
            }
            st2(p.out, p.out_dtype, off, a, b);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// reverse state-gradient chain: one CTA per (64-column block, v-head, segment).  With dS' the gradient of the state
// leaving the chunk:   dVd = Aqk^T dO + kbar dS';   dS = diag(gl) dS' + (scale q 2^g)^T dO + nw^T dVd.
// ---------------------------------------------------------------------------------------------------------
constexpr int BWD_DH_SMEM = (DK * LDS + CH * LDS + CH * LDS + CH * LDA + 2 * CH * LDT + CH * LDS + DK) * 4;

template <int PREC>
__global__ void __launch_bounds__(256, 1) bwd_dh_kernel(const MkdaBwdDh p) {
    extern __shared__ __align__(16) float smem[];
    float* sD = smem;                  // [128][LDS]  dS' block, B(k = K index, n = column)
    float* sAq = sD + DK * LDS;        // [64][LDS]   Aqk, A(m = j, k = i) read transposed
    float* sDo = sAq + CH * LDS;       // [64][LDS]   dO block, B(k = token, n = column)
    float* sKb = sDo + CH * LDS;       // [64][LDA]   kbar, A(m = token, k = K index)
    float* sQt = sKb + CH * LDA;       // [64][LDT]   scale q 2^g, A(m = K index, k = token)
    float* sW = sQt + CH * LDT;        // [64][LDT]   nw, A(m = K index, k = token)
    float* sDv = sW + CH * LDT;        // [64][LDS]   dVd block, B(k = token, n = column)
    float* sGl = sDv + CH * LDS;       // [128]

    const int cb = blockIdx.x, h = blockIdx.y, seg = blockIdx.z, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int col0 = cb * 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp & 3, wn = warp >> 2;
    const bool vf = p.state_v_first != 0;
    const int kr0 = warp * 16 + g, kr1 = kr0 + 8;

    float D[8][4];
    {
        const int row = p.seg_dht ? p.seg_dht[seg] : seg;
        const float* src = (p.dht && row >= 0) ? p.dht + ((size_t)row * HV + h) * DK * DV : nullptr;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = (e & 2) ? kr1 : kr0, cc = col0 + nt * 8 + 2 * t + (e & 1);
                D[nt][e] = src ? src[state_index(vf, kk, cc)] : 0.f;
            }
    }
    const int c_beg = p.L.seg_chunk_off[seg], c_end = p.L.seg_chunk_off[seg + 1];
    for (int c = c_end - 1; c >= c_beg; --c) {
        const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
        float* dhc = p.dh + ((size_t)c * HV + h) * DK * DV;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int cc = nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(sD + kr0 * LDS + cc) = make_float2(D[nt][0], D[nt][1]);
            *reinterpret_cast<float2*>(sD + kr1 * LDS + cc) = make_float2(D[nt][2], D[nt][3]);
            *reinterpret_cast<float2*>(dhc + (size_t)kr0 * DV + col0 + cc) = make_float2(D[nt][0], D[nt][1]);
            *reinterpret_cast<float2*>(dhc + (size_t)kr1 * DV + col0 + cc) = make_float2(D[nt][2], D[nt][3]);
        }
        const float* glast = p.g_c + ((size_t)(start + len - 1) * HV + h) * 128;
        for (int i = tid; i < CH * 32; i += 256) {
            const int r = i >> 5, c4 = (i & 31) * 4;
            float4 w = make_float4(0.f, 0.f, 0.f, 0.f), kb = w, qt = w;
            if (r < len) {
                const size_t th = (size_t)(start + r) * HV + h, tk = (size_t)(start + r) * HK + hk;
                w = *reinterpret_cast<const float4*>(p.nw + th * 128 + c4);
                kb = ld4(p.k, p.qk_dtype, tk * 128 + c4);
                qt = ld4(p.q, p.qk_dtype, tk * 128 + c4);
                const float rk = p.k_rstd ? p.k_rstd[tk] : 1.f;
                const float rq = p.scale * (p.q_rstd ? p.q_rstd[tk] : 1.f);
                const float4 gr = *reinterpret_cast<const float4*>(p.g_c + th * 128 + c4);
                const float4 gL = *reinterpret_cast<const float4*>(glast + c4);
                kb.x *= rk * exp2f(gL.x - gr.x); kb.y *= rk * exp2f(gL.y - gr.y);
                kb.z *= rk * exp2f(gL.z - gr.z); kb.w *= rk * exp2f(gL.w - gr.w);
                qt.x *= rq * exp2f(gr.x); qt.y *= rq * exp2f(gr.y); qt.z *= rq * exp2f(gr.z); qt.w *= rq * exp2f(gr.w);
            }
            *reinterpret_cast<float4*>(sW + r * LDT + c4) = w;
            *reinterpret_cast<float4*>(sKb + r * LDA + c4) = kb;
            *reinterpret_cast<float4*>(sQt + r * LDT + c4) = qt;
        }
        for (int i = tid; i < CH * 16; i += 256) {
            const int r = i >> 4, c4 = (i & 15) * 4;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), d = a;
            if (r < len) {
                const size_t th = (size_t)(start + r) * HV + h;
                a = *reinterpret_cast<const float4*>(p.Aqk + th * 64 + c4);
                d = ld4(p.d_o, p.do_dtype, th * 128 + col0 + c4);
            }
            *reinterpret_cast<float4*>(sAq + r * LDS + c4) = a;
            *reinterpret_cast<float4*>(sDo + r * LDS + c4) = d;
        }
        if (tid < DK) sGl[tid] = exp2f(glast[tid]);
        __syncthreads();
        // dVd block (rows j = 16 wm.., columns 32 wn..) = Aqk^T dO + kbar dS'
        float acc[4][4];
        zero_acc<4>(acc);
        // Aqk^T: A(m = j, k = i) = sAq[i][j]; rows i < 16 wm contribute nothing (Aqk is lower triangular)
        warp_mma<4, PREC, 1, LDS, LDS, 1>(acc, sAq + wm * 16 * LDS + wm * 16, sDo + wm * 16 * LDS + wn * 32, CH - 16 * wm);
        warp_mma<4, PREC, LDA, 1, LDS, 1>(acc, sKb + wm * 16 * LDA, sD + wn * 32, DK);
        {
            const int r0 = wm * 16 + g, r1 = r0 + 8;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int cl = wn * 32 + nt * 8 + 2 * t;
                *reinterpret_cast<float2*>(sDv + r0 * LDS + cl) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2*>(sDv + r1 * LDS + cl) = make_float2(acc[nt][2], acc[nt][3]);
                if (r0 < len) *reinterpret_cast<float2*>(p.dVd + ((size_t)(start + r0) * HV + h) * 128 + col0 + cl) = make_float2(acc[nt][0], acc[nt][1]);
                if (r1 < len) *reinterpret_cast<float2*>(p.dVd + ((size_t)(start + r1) * HV + h) * 128 + col0 + cl) = make_float2(acc[nt][2], acc[nt][3]);
            }
        }
        __syncthreads();
        {
            const float g0 = sGl[kr0], g1 = sGl[kr1];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) { D[nt][0] *= g0; D[nt][1] *= g0; D[nt][2] *= g1; D[nt][3] *= g1; }
        }
        warp_mma<8, PREC, 1, LDT, LDS, 1>(D, sQt + warp * 16, sDo, CH);
        warp_mma<8, PREC, 1, LDT, LDS, 1>(D, sW + warp * 16, sDv, CH);
        __syncthreads();
    }
    if (p.dh0) {
        float* out = p.dh0 + ((size_t)seg * HV + h) * DK * DV;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = (e & 2) ? kr1 : kr0, cc = col0 + nt * 8 + 2 * t + (e & 1);
                out[state_index(vf, kk, cc)] = D[nt][e];
            }
    }
}

// ---------------------------------------------------------------------------------------------------------
// prefix combine over the segments of a group: one CTA per (64-column block, v-head, group).
//   forward:  X <- M_s X + H_s          backward: X <- M_s^T X + D_s
// X enters segment s before the update (stored to s_in[s]).  Error-compensated TF32 keeps the carried state at
// fp32 accuracy however many segments are chained.
// ---------------------------------------------------------------------------------------------------------
constexpr int COMBINE_SMEM = (DK * LDS + DK * LDA) * 4;

template <int PREC>
__global__ void __launch_bounds__(256, 1) combine_kernel(const MkdaCombine p) {
    extern __shared__ __align__(16) float smem[];
    float* sX = smem;                  // [128][LDS]  B(k, n)
    float* sM = sX + DK * LDS;         // [128][LDA]  A(m, k) = M[m][k]  (forward) or M[k][m] (reverse)
    const int cb = blockIdx.x, h = blockIdx.y, grp = blockIdx.z, HV = p.HV;
    const int col0 = cb * 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int kr0 = warp * 16 + g, kr1 = kr0 + 8;
    float X[8][4];
    {
        const float* src = p.carry ? p.carry + ((size_t)grp * HV + h) * DK * DV : nullptr;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = (e & 2) ? kr1 : kr0, cc = col0 + nt * 8 + 2 * t + (e & 1);
                X[nt][e] = src ? src[(size_t)kk * DV + cc] : 0.f;
            }
    }
    const int s_beg = p.grp_seg_off[grp], s_end = p.grp_seg_off[grp + 1];
    for (int i = 0; i < s_end - s_beg; ++i) {
        const int s = p.reverse ? s_end - 1 - i : s_beg + i;
        const size_t base = ((size_t)s * HV + h) * DK * DV;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int cc = nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(sX + kr0 * LDS + cc) = make_float2(X[nt][0], X[nt][1]);
            *reinterpret_cast<float2*>(sX + kr1 * LDS + cc) = make_float2(X[nt][2], X[nt][3]);
            if (p.s_in) {
                *reinterpret_cast<float2*>(p.s_in + base + (size_t)kr0 * DV + col0 + cc) = make_float2(X[nt][0], X[nt][1]);
                *reinterpret_cast<float2*>(p.s_in + base + (size_t)kr1 * DV + col0 + cc) = make_float2(X[nt][2], X[nt][3]);
            }
        }
        for (int j = tid; j < DK * 32; j += 256) {
            const int r = j >> 5, c4 = (j & 31) * 4;
            *reinterpret_cast<float4*>(sM + r * LDA + c4) = *reinterpret_cast<const float4*>(p.ms + base + (size_t)r * DK + c4);
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int cc = col0 + nt * 8 + 2 * t;
            float2 a = make_float2(0.f, 0.f), b = a;
            if (p.hs) {
                a = *reinterpret_cast<const float2*>(p.hs + base + (size_t)kr0 * DV + cc);
                b = *reinterpret_cast<const float2*>(p.hs + base + (size_t)kr1 * DV + cc);
            }
            X[nt][0] = a.x; X[nt][1] = a.y; X[nt][2] = b.x; X[nt][3] = b.y;
        }
        __syncthreads();
        if (p.reverse) warp_mma<8, PREC, 1, LDA, LDS, 1>(X, sM + warp * 16, sX, DK);
        else warp_mma<8, PREC, LDA, 1, LDS, 1>(X, sM + warp * 16 * LDA, sX, DK);
        __syncthreads();
    }
    if (p.s_out) {
        float* out = p.s_out + ((size_t)grp * HV + h) * DK * DV;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int cc = col0 + nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(out + (size_t)kr0 * DV + cc) = make_float2(X[nt][0], X[nt][1]);
            *reinterpret_cast<float2*>(out + (size_t)kr1 * DV + cc) = make_float2(X[nt][2], X[nt][3]);
        }
    }
}

}  // namespace mkda

using namespace mkda;

extern "C" int mkda_recur_fwd(const MkdaRecurFwd* p, void* stream) {
    if (!p || !p->nw || !p->u || !p->k || !p->g_c) return set_error(MKDA_ERR_ARG, "recur_fwd: null argument");
    if (p->want_transition && !p->mt) return set_error(MKDA_ERR_ARG, "recur_fwd: want_transition needs mt");
    if (p->L.NS == 0) return MKDA_OK;
    if (!legacy_kernels()) return launch_recur_fwd_tc(p, (cudaStream_t)stream);
    auto kern = recur_fwd_kernel<MKDA_PREC_STATE>;
    if (int e = ensure_smem((const void*)kern, RECUR_SMEM, "recur_fwd")) return e;
    kern<<<dim3(p->want_transition ? 4 : 2, p->L.HV, p->L.NS), 256, RECUR_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("recur_fwd");
}

extern "C" int mkda_out_fwd(const MkdaOutFwd* p, void* stream) {
    if (!p || !p->q || !p->g_c || !p->Aqk || !p->Vd || !p->h || !p->out) return set_error(MKDA_ERR_ARG, "out_fwd: null argument");
    if (p->has_norm && !p->gate) return set_error(MKDA_ERR_ARG, "out_fwd: the gated norm needs a gate tensor");
    if (p->L.NC == 0) return MKDA_OK;
    if (!legacy_kernels()) return launch_out_fwd_tc(p, (cudaStream_t)stream);
    auto kern = out_fwd_kernel<MKDA_PREC_OUT>;
    if (int e = ensure_smem((const void*)kern, OUT_SMEM, "out_fwd")) return e;
    kern<<<dim3(p->L.NC, p->L.HV), 256, OUT_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("out_fwd");
}

extern "C" int mkda_bwd_dh(const MkdaBwdDh* p, void* stream) {
    if (!p || !p->d_o || !p->q || !p->k || !p->g_c || !p->Aqk || !p->nw || !p->dh || !p->dVd)
        return set_error(MKDA_ERR_ARG, "bwd_dh: null argument");
    if (p->L.NS == 0) return MKDA_OK;
    if (!legacy_kernels()) return launch_bwd_dh_tc(p, (cudaStream_t)stream);
    auto kern = bwd_dh_kernel<MKDA_PREC_DH>;
    if (int e = ensure_smem((const void*)kern, BWD_DH_SMEM, "bwd_dh")) return e;
    kern<<<dim3(2, p->L.HV, p->L.NS), 256, BWD_DH_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("bwd_dh");
}

extern "C" int mkda_state_combine(const MkdaCombine* p, void* stream) {
    if (!p || !p->grp_seg_off || !p->ms || (!p->s_in && !p->s_out)) return set_error(MKDA_ERR_ARG, "state_combine: null argument");
    if (p->NG == 0) return MKDA_OK;
    auto kern = combine_kernel<MKDA_PREC_COMBINE>;
    if (int e = ensure_smem((const void*)kern, COMBINE_SMEM, "state_combine")) return e;
    kern<<<dim3(2, p->HV, p->NG), 256, COMBINE_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("state_combine");
}

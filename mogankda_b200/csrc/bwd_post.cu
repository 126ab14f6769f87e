// Chunk-parallel backward kernels that consume the per-chunk states: gradients through the WY solve (bwd_wy) and
// through the state contractions (bwd_sgrad).  One CTA (8 warps) per (chunk, v-head); warp (wm, wn) owns the 16 rows
// 16 wm.. of every 64-row output tile and half of its columns.
#include "common.cuh"
#include "host.h"

#ifndef MKDA_PREC_WY
#define MKDA_PREC_WY 1
#endif
#ifndef MKDA_PREC_SGRAD
#define MKDA_PREC_SGRAD 1
#endif

namespace mkda {

constexpr int LDA = 132;
constexpr int LDT = 136;
constexpr int LDM = 68;

// ---------------------------------------------------------------------------------------------------------
// bwd_wy.  With S the state entering the chunk, k~ = k 2^g, Ab = A diag(beta):
//   X = V - k~ S        Vd = Ab X        dAqk = lower(dO Vd^T)
//   dW = A^T dVd        dX = diag(beta) dW (= dV)       dbeta_w = rowsum(dW * X)
//   dA = (dVd X^T) diag(beta)          dL = -strictlower(A^T dA A^T)
// ---------------------------------------------------------------------------------------------------------
constexpr int WY_SMEM = (DK * LDT + 2 * CH * LDA + 4 * CH * LDM + 3 * CH) * 4;

template <int PREC>
__global__ void __launch_bounds__(256, 1) bwd_wy_kernel(const MkdaBwdWy p) {
    extern __shared__ __align__(16) float smem[];
    float* R0 = smem;                   // S [128][LDT]; later Vd [64][LDA] | dO [64][LDA]
    float* R1 = R0 + DK * LDT;          // k~ [64][LDA]; later dVd
    float* R2 = R1 + CH * LDA;          // V -> X [64][LDA]
    float* sA = R2 + CH * LDA;          // A [64][LDM]
    float* sAb = sA + CH * LDM;         // A diag(beta)
    float* sT = sAb + CH * LDM;         // dA, [64][LDM]
    float* sY = sT + CH * LDM;          // dA A^T
    float* sBeta = sY + CH * LDM;       // [64]
    float* sRed = sBeta + CH;           // [2][64]
    float* sVd = R0;
    float* sDo = R0 + CH * LDA;

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp & 3, wn = warp >> 2;
    const int r0 = wm * 16 + g, r1 = r0 + 8;

    // ---- stage S, k~, V, A, A diag(beta) ----------------------------------------------------------------
    if (tid < CH) sBeta[tid] = tid < len ? p.beta[(size_t)(start + tid) * HV + h] : 0.f;
    const float* hc = p.h + ((size_t)c * HV + h) * DK * DV;
    for (int i = tid; i < DK * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        *reinterpret_cast<float4*>(R0 + r * LDT + c4) = *reinterpret_cast<const float4*>(hc + (size_t)r * DV + c4);
    }
    for (int i = tid; i < CH * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        float4 kt = make_float4(0.f, 0.f, 0.f, 0.f), v = kt;
        if (r < len) {
            const size_t th = (size_t)(start + r) * HV + h, tk = (size_t)(start + r) * HK + hk;
            kt = ld4(p.k, p.kv_dtype, tk * 128 + c4);
            const float rk = p.k_rstd ? p.k_rstd[tk] : 1.f;
            const float4 gr = *reinterpret_cast<const float4*>(p.g_c + th * 128 + c4);
            kt.x *= rk * exp2f(gr.x); kt.y *= rk * exp2f(gr.y); kt.z *= rk * exp2f(gr.z); kt.w *= rk * exp2f(gr.w);
            v = ld4(p.v, p.kv_dtype, th * 128 + c4);
        }
        *reinterpret_cast<float4*>(R1 + r * LDA + c4) = kt;
        *reinterpret_cast<float4*>(R2 + r * LDA + c4) = v;
    }
    __syncthreads();   // sBeta visible
    for (int i = tid; i < CH * 16; i += 256) {
        const int r = i >> 4, c4 = (i & 15) * 4;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < len) a = *reinterpret_cast<const float4*>(p.A + ((size_t)(start + r) * HV + h) * 64 + c4);
        *reinterpret_cast<float4*>(sA + r * LDM + c4) = a;
        a.x *= sBeta[c4]; a.y *= sBeta[c4 + 1]; a.z *= sBeta[c4 + 2]; a.w *= sBeta[c4 + 3];
        *reinterpret_cast<float4*>(sAb + r * LDM + c4) = a;
    }
    __syncthreads();

    float acc[8][4];
    // ---- X = V - k~ S ------------------------------------------------------------------------------------
    zero_acc<8>(acc);
    warp_mma<8, PREC, LDA, 1, LDT, 1>(acc, R1 + wm * 16 * LDA, R0 + wn * 64, DK);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        const int col = wn * 64 + nt * 8 + 2 * t;
        float2* x0 = reinterpret_cast<float2*>(R2 + r0 * LDA + col);
        float2* x1 = reinterpret_cast<float2*>(R2 + r1 * LDA + col);
        *x0 = make_float2(x0->x - acc[nt][0], x0->y - acc[nt][1]);
        *x1 = make_float2(x1->x - acc[nt][2], x1->y - acc[nt][3]);
    }
    __syncthreads();   // X complete; S and k~ dead
    // ---- Vd = Ab X; stage dO and dVd ------------------------------------------------------------------------
    zero_acc<8>(acc);
    warp_mma<8, PREC, LDM, 1, LDA, 1>(acc, sAb + wm * 16 * LDM, R2 + wn * 64, 16 * (wm + 1));
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        const int col = wn * 64 + nt * 8 + 2 * t;
        *reinterpret_cast<float2*>(sVd + r0 * LDA + col) = make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(sVd + r1 * LDA + col) = make_float2(acc[nt][2], acc[nt][3]);
        if (r0 < len) *reinterpret_cast<float2*>(p.Vd + ((size_t)(start + r0) * HV + h) * 128 + col) = make_float2(acc[nt][0], acc[nt][1]);
        if (r1 < len) *reinterpret_cast<float2*>(p.Vd + ((size_t)(start + r1) * HV + h) * 128 + col) = make_float2(acc[nt][2], acc[nt][3]);
    }
    for (int i = tid; i < CH * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        float4 d = make_float4(0.f, 0.f, 0.f, 0.f), dv = d;
        if (r < len) {
            const size_t th = (size_t)(start + r) * HV + h;
            d = ld4(p.d_o, p.do_dtype, th * 128 + c4);
            dv = *reinterpret_cast<const float4*>(p.dVd + th * 128 + c4);
        }
        *reinterpret_cast<float4*>(sDo + r * LDA + c4) = d;
        *reinterpret_cast<float4*>(R1 + r * LDA + c4) = dv;
    }
    __syncthreads();
    // ---- dAqk = lower(dO Vd^T): rows i = 16 wm.., columns j = 32 wn.. ----------------------------------------
    {
        float a4[4][4];
        zero_acc<4>(a4);
        warp_mma<4, PREC, LDA, 1, 1, LDA>(a4, sDo + wm * 16 * LDA, sVd + wn * 32 * LDA, DV);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int j = wn * 32 + nt * 8 + 2 * t;
            if (r0 < len) *reinterpret_cast<float2*>(p.dAqk + ((size_t)(start + r0) * HV + h) * 64 + j) =
                make_float2(j <= r0 ? a4[nt][0] : 0.f, j + 1 <= r0 ? a4[nt][1] : 0.f);
            if (r1 < len) *reinterpret_cast<float2*>(p.dAqk + ((size_t)(start + r1) * HV + h) * 64 + j) =
                make_float2(j <= r1 ? a4[nt][2] : 0.f, j + 1 <= r1 ? a4[nt][3] : 0.f);
        }
    }
    // ---- dW = A^T dVd (rows j = 16 wm.., only i >= 16 wm contribute); dX, dbeta_w -------------------------------
    zero_acc<8>(acc);
    warp_mma<8, PREC, 1, LDM, LDA, 1>(acc, sA + wm * 16 * LDM + wm * 16, R1 + wm * 16 * LDA + wn * 64, CH - 16 * wm);
    {
        const float b0 = sBeta[r0], b1 = sBeta[r1];
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int col = wn * 64 + nt * 8 + 2 * t;
            const float2 x0 = *reinterpret_cast<const float2*>(R2 + r0 * LDA + col);
            const float2 x1 = *reinterpret_cast<const float2*>(R2 + r1 * LDA + col);
            s0 += acc[nt][0] * x0.x + acc[nt][1] * x0.y;
            s1 += acc[nt][2] * x1.x + acc[nt][3] * x1.y;
            if (r0 < len) *reinterpret_cast<float2*>(p.dX + ((size_t)(start + r0) * HV + h) * 128 + col) = make_float2(b0 * acc[nt][0], b0 * acc[nt][1]);
            if (r1 < len) *reinterpret_cast<float2*>(p.dX + ((size_t)(start + r1) * HV + h) * 128 + col) = make_float2(b1 * acc[nt][2], b1 * acc[nt][3]);
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        if (t == 0) { sRed[wn * CH + r0] = s0; sRed[wn * CH + r1] = s1; }
    }
    // ---- dA = (dVd X^T) diag(beta): rows i = 16 wm.., columns j = 32 wn.. --------------------------------------
    {
        float a4[4][4];
        zero_acc<4>(a4);
        warp_mma<4, PREC, LDA, 1, 1, LDA>(a4, R1 + wm * 16 * LDA, R2 + wn * 32 * LDA, DV);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int j = wn * 32 + nt * 8 + 2 * t;
            const float bj0 = sBeta[j], bj1 = sBeta[j + 1];
            *reinterpret_cast<float2*>(sT + r0 * LDM + j) = make_float2(a4[nt][0] * bj0, a4[nt][1] * bj1);
            *reinterpret_cast<float2*>(sT + r1 * LDM + j) = make_float2(a4[nt][2] * bj0, a4[nt][3] * bj1);
        }
    }
    __syncthreads();
    if (tid < len) p.dbeta_w[(size_t)(start + tid) * HV + h] = sRed[tid] + sRed[CH + tid];
    // ---- Y = dA A^T: Y[a][j] = sum_b dA[a][b] A[j][b], b <= j ------------------------------------------------------
    {
        float a4[4][4];
        zero_acc<4>(a4);
        warp_mma<4, PREC, LDM, 1, 1, LDM>(a4, sT + wm * 16 * LDM, sA + wn * 32 * LDM, 32 * (wn + 1));
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int j = wn * 32 + nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(sY + r0 * LDM + j) = make_float2(a4[nt][0], a4[nt][1]);
            *reinterpret_cast<float2*>(sY + r1 * LDM + j) = make_float2(a4[nt][2], a4[nt][3]);
        }
    }
    __syncthreads();
    // ---- dL = -strictlower(A^T Y): Z[i][j] = sum_{a >= i} A[a][i] Y[a][j] ----------------------------------------
    {
        float a4[4][4];
        zero_acc<4>(a4);
        warp_mma<4, PREC, 1, LDM, LDM, 1>(a4, sA + wm * 16 * LDM + wm * 16, sY + wm * 16 * LDM + wn * 32, CH - 16 * wm);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int j = wn * 32 + nt * 8 + 2 * t;
            if (r0 < len) *reinterpret_cast<float2*>(p.dL + ((size_t)(start + r0) * HV + h) * 64 + j) =
                make_float2(j < r0 ? -a4[nt][0] : 0.f, j + 1 < r0 ? -a4[nt][1] : 0.f);
            if (r1 < len) *reinterpret_cast<float2*>(p.dL + ((size_t)(start + r1) * HV + h) * 64 + j) =
                make_float2(j < r1 ? -a4[nt][2] : 0.f, j + 1 < r1 ? -a4[nt][3] : 0.f);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// bwd_sgrad.  With S / dS' the state entering / state-gradient leaving the chunk, up = 2^g, rest = 2^(g_L - g):
//   dq~ = scale dO S^T     dk~ = -dX S^T     dkbar = Vd dS'^T     dgl = rowsum_v(S * dS')
//   dq_p = dq~ up          dk_p = dk~ up + dkbar rest
//   dg_p = q~ dq~ + k~ dk~ - kbar dkbar;   last valid row += colsum(kbar dkbar) + gl dgl
// ---------------------------------------------------------------------------------------------------------
constexpr int SG_SMEM = (DK * LDA + 2 * CH * LDA + DK + 4 * DK) * 4;

template <int PREC>
__global__ void __launch_bounds__(256, 1) bwd_sgrad_kernel(const MkdaBwdSgrad p) {
    extern __shared__ __align__(16) float smem[];
    float* R0 = smem;                   // S then dS' as [K index][v], B(k = v, n = K index)
    float* R1 = R0 + DK * LDA;          // dO then Vd, A(m = token, k = v)
    float* R2 = R1 + CH * LDA;          // dX
    float* sDgl = R2 + CH * LDA;        // [128]
    float* sCol = sDgl + DK;            // [4][128]

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp & 3, wn = warp >> 2;
    const int r0 = wm * 16 + g, r1 = r0 + 8;
    const size_t sbase = ((size_t)c * HV + h) * DK * DV;

    for (int i = tid; i < DK * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        *reinterpret_cast<float4*>(R0 + r * LDA + c4) = *reinterpret_cast<const float4*>(p.h + sbase + (size_t)r * DV + c4);
    }
    stage_rows128<LDA, 256>(R1, p.d_o, p.do_dtype, start, len, HV, h, nullptr);
    stage_rows128<LDA, 256>(R2, p.dX, MKDA_F32, start, len, HV, h, nullptr);
    __syncthreads();

    float aQ[8][4], aK[8][4], aB[8][4];
    zero_acc<8>(aQ);
    zero_acc<8>(aK);
    zero_acc<8>(aB);
    warp_mma<8, PREC, LDA, 1, 1, LDA>(aQ, R1 + wm * 16 * LDA, R0 + wn * 64 * LDA, DV);
    warp_mma<8, PREC, LDA, 1, 1, LDA>(aK, R2 + wm * 16 * LDA, R0 + wn * 64 * LDA, DV);
    __syncthreads();
    // replace S by dS' in place while reducing S * dS' over v (one warp covers one K row per step)
    for (int i = tid; i < DK * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        const float4 d = *reinterpret_cast<const float4*>(p.dh + sbase + (size_t)r * DV + c4);
        float4* sp = reinterpret_cast<float4*>(R0 + r * LDA + c4);
        const float4 s = *sp;
        *sp = d;
        float pr = (s.x * d.x + s.y * d.y) + (s.z * d.z + s.w * d.w);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pr += __shfl_xor_sync(0xffffffffu, pr, o);
        if (lane == 0) sDgl[r] = pr;
    }
    stage_rows128<LDA, 256>(R1, p.Vd, MKDA_F32, start, len, HV, h, nullptr);
    __syncthreads();
    warp_mma<8, PREC, LDA, 1, 1, LDA>(aB, R1 + wm * 16 * LDA, R0 + wn * 64 * LDA, DV);

    // ---- row-local epilogue ------------------------------------------------------------------------------------
    const float* glast = p.g_c + ((size_t)(start + len - 1) * HV + h) * 128;
    // pass 0: column sums of kbar * dkbar; pass 1: outputs
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int col = wn * 64 + nt * 8 + 2 * t;
            const float2 gL = *reinterpret_cast<const float2*>(glast + col);
            float cs0 = 0.f, cs1 = 0.f;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = half ? r1 : r0;
                if (r >= len) continue;
                const size_t th = (size_t)(start + r) * HV + h, tk = (size_t)(start + r) * HK + hk;
                const float2 gr = *reinterpret_cast<const float2*>(p.g_c + th * 128 + col);
                const float rk = p.k_rstd ? p.k_rstd[tk] : 1.f;
                const float k0 = ld1(p.k, p.qk_dtype, tk * 128 + col) * rk, k1 = ld1(p.k, p.qk_dtype, tk * 128 + col + 1) * rk;
                const float re0 = exp2f(gL.x - gr.x), re1 = exp2f(gL.y - gr.y);
                const float dkb0 = aB[nt][2 * half], dkb1 = aB[nt][2 * half + 1];
                const float kbd0 = k0 * re0 * dkb0, kbd1 = k1 * re1 * dkb1;
                if (pass == 0) { cs0 += kbd0; cs1 += kbd1; continue; }
                const float rq = p.q_rstd ? p.q_rstd[tk] : 1.f;
                const float q0 = ld1(p.q, p.qk_dtype, tk * 128 + col) * rq, q1 = ld1(p.q, p.qk_dtype, tk * 128 + col + 1) * rq;
                const float up0 = exp2f(gr.x), up1 = exp2f(gr.y);
                const float dqt0 = p.scale * aQ[nt][2 * half], dqt1 = p.scale * aQ[nt][2 * half + 1];
                const float dkt0 = -aK[nt][2 * half], dkt1 = -aK[nt][2 * half + 1];
                float dg0 = q0 * up0 * dqt0 + k0 * up0 * dkt0 - kbd0;
                float dg1 = q1 * up1 * dqt1 + k1 * up1 * dkt1 - kbd1;
                if (r == len - 1) {
                    dg0 += ((sCol[col] + sCol[DK + col]) + (sCol[2 * DK + col] + sCol[3 * DK + col])) + exp2f(gL.x) * sDgl[col];
                    dg1 += ((sCol[col + 1] + sCol[DK + col + 1]) + (sCol[2 * DK + col + 1] + sCol[3 * DK + col + 1])) + exp2f(gL.y) * sDgl[col + 1];
                }
                *reinterpret_cast<float2*>(p.dq_p + th * 128 + col) = make_float2(dqt0 * up0, dqt1 * up1);
                *reinterpret_cast<float2*>(p.dk_p + th * 128 + col) = make_float2(dkt0 * up0 + dkb0 * re0, dkt1 * up1 + dkb1 * re1);
                *reinterpret_cast<float2*>(p.dg_p + th * 128 + col) = make_float2(dg0, dg1);
            }
            if (pass == 0) {
                // add the 8 row groups of this warp (fixed tree), then publish per row block
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    cs0 += __shfl_xor_sync(0xffffffffu, cs0, o);
                    cs1 += __shfl_xor_sync(0xffffffffu, cs1, o);
                }
                if (g == 0) { sCol[wm * DK + col] = cs0; sCol[wm * DK + col + 1] = cs1; }
            }
        }
        if (pass == 0) __syncthreads();
    }
}

}  // namespace mkda

using namespace mkda;

extern "C" int mkda_bwd_wy(const MkdaBwdWy* p, void* stream) {
    if (!p || !p->k || !p->v || !p->g_c || !p->beta || !p->A || !p->h || !p->d_o || !p->dVd || !p->Vd || !p->dX ||
        !p->dbeta_w || !p->dAqk || !p->dL)
        return set_error(MKDA_ERR_ARG, "bwd_wy: null argument");
    if (p->L.NC == 0) return MKDA_OK;
    if (!legacy_kernels()) return launch_bwd_wy_tc(p, (cudaStream_t)stream);
    auto kern = bwd_wy_kernel<MKDA_PREC_WY>;
    if (int e = ensure_smem((const void*)kern, WY_SMEM, "bwd_wy")) return e;
    kern<<<dim3(p->L.NC, p->L.HV), 256, WY_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("bwd_wy");
}

extern "C" int mkda_bwd_sgrad(const MkdaBwdSgrad* p, void* stream) {
    if (!p || !p->q || !p->k || !p->g_c || !p->d_o || !p->dX || !p->Vd || !p->h || !p->dh || !p->dq_p || !p->dk_p || !p->dg_p)
        return set_error(MKDA_ERR_ARG, "bwd_sgrad: null argument");
    if (p->L.NC == 0) return MKDA_OK;
    if (!legacy_kernels()) return launch_bwd_sgrad_tc(p, (cudaStream_t)stream);
    auto kern = bwd_sgrad_kernel<MKDA_PREC_SGRAD>;
    if (int e = ensure_smem((const void*)kern, SG_SMEM, "bwd_sgrad")) return e;
    kern<<<dim3(p->L.NC, p->L.HV), 256, SG_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("bwd_sgrad");
}

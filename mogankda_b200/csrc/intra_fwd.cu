// Chunk-parallel WY preparation, one CTA (8 warps) per (chunk, v-head).
//
//   Gamma_ij = sum_c k_ic k_jc 2^(g_ic - g_jc)  (i > j)        Aqk_ij = scale sum_c q_ic k_jc 2^(g_ic - g_jc)  (i >= j)
//   A  = (I + strictlower(diag(beta) Gamma))^-1
//   nw = -A diag(beta) (k 2^g)                                  u = A diag(beta) v
//
// Range / prefix-invariance: the per-channel decay cannot be factored out of the K contraction, so each 16-row
// block I uses its first row a = 16 I as anchor: row operand k_i 2^(g_i - g_a) (<= 1), column operand
// k_j 2^(g_a - g_j) (<= 1 for j < a, <= 2^(15*5/ln2) inside the diagonal block).  An output element (i, j)
// therefore depends on rows i, j and a <= i only, never on later rows.
// Rows past the end of the sequence are staged as zeros (their g as the last valid row's), so they produce
// identity rows in A and are never stored.
#include "common.cuh"
#include "host.h"

#ifndef MKDA_PREC_INTRA
#define MKDA_PREC_INTRA 1
#endif

namespace mkda {

constexpr int KLD = 132;   // leading dimension of [64][128] tiles read row-wise by the MMA fragments
constexpr int MLD = 68;    // leading dimension of [64][64] tiles
constexpr int INTRA_SMEM = (3 * CH * KLD + 2 * CH * MLD + CH) * 4;

template <int PREC>
__global__ void __launch_bounds__(256, 1) intra_fwd_kernel(const MkdaIntraFwd p) {
    extern __shared__ __align__(16) float smem[];
    float* sK = smem;
    float* sQ = sK + CH * KLD;
    float* sG = sQ + CH * KLD;
    float* sM = sG + CH * KLD;
    float* sP = sM + CH * MLD;
    float* sBeta = sP + CH * MLD;
    float* sInv = sQ;                       // reused once Gamma / Aqk are done

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    // ---- phase 0: stage q, k (L2-normalised on the fly), g_c, beta --------------------------------------------
    stage_rows128<KLD, 256>(sK, p.k, p.qkv_dtype, start, len, HK, hk, p.k_rstd);
    stage_rows128<KLD, 256>(sQ, p.q, p.qkv_dtype, start, len, HK, hk, p.q_rstd);
    for (int i = tid; i < CH * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        const int rr = r < len ? r : len - 1;
        *reinterpret_cast<float4*>(sG + r * KLD + c4) =
            *reinterpret_cast<const float4*>(p.g_c + ((size_t)(start + rr) * HV + h) * 128 + c4);
    }
    for (int i = tid; i < CH * CH; i += 256) {
        const int r = i >> 6, j = i & 63;
        sM[r * MLD + j] = (r == j) ? 1.f : 0.f;
        sP[r * MLD + j] = 0.f;
    }
    if (tid < CH) sBeta[tid] = tid < len ? p.beta[(size_t)(start + tid) * HV + h] : 0.f;
    __syncthreads();

    // ---- phase 1: Gamma and Q K^T for row block I; the two warps of a block split its column tiles ------------
    {
        const int I = warp >> 1, half = warp & 1, a = 16 * I;
        float accG[4][4], accP[4][4];
        zero_acc<4>(accG);
        zero_acc<4>(accP);
        if (a < len) {
            const int r0 = a + g, r1 = r0 + 8;
            for (int k0 = 0; k0 < DK; k0 += 8) {
                const int c0 = k0 + t, c1 = c0 + 4;
                const float ga0 = sG[a * KLD + c0], ga1 = sG[a * KLD + c1];
                const float e00 = exp2f(sG[r0 * KLD + c0] - ga0), e10 = exp2f(sG[r1 * KLD + c0] - ga0);
                const float e01 = exp2f(sG[r0 * KLD + c1] - ga1), e11 = exp2f(sG[r1 * KLD + c1] - ga1);
                FragA<PREC> fk, fq;
                fk.set(0, sK[r0 * KLD + c0] * e00); fk.set(1, sK[r1 * KLD + c0] * e10);
                fk.set(2, sK[r0 * KLD + c1] * e01); fk.set(3, sK[r1 * KLD + c1] * e11);
                fq.set(0, sQ[r0 * KLD + c0] * e00); fq.set(1, sQ[r1 * KLD + c0] * e10);
                fq.set(2, sQ[r0 * KLD + c1] * e01); fq.set(3, sQ[r1 * KLD + c1] * e11);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (i <= I) {
                        const int j = (half * (I + 1) + i) * 8 + g;
                        FragB<PREC> fb;
                        fb.set(0, sK[j * KLD + c0] * exp2f(ga0 - sG[j * KLD + c0]));
                        fb.set(1, sK[j * KLD + c1] * exp2f(ga1 - sG[j * KLD + c1]));
                        mma_frag<PREC>(accG[i], fk, fb);
                        mma_frag<PREC>(accP[i], fq, fb);
                    }
                }
            }
            const float b0 = sBeta[r0], b1 = sBeta[r1];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i <= I) {
                    const int j0 = (half * (I + 1) + i) * 8 + 2 * t;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int r = (e & 2) ? r1 : r0, j = j0 + (e & 1);
                        const float bt = (e & 2) ? b1 : b0;
                        if (j < r) sM[r * MLD + j] = bt * accG[i][e];
                        if (j <= r) sP[r * MLD + j] = p.scale * accP[i][e];
                    }
                }
            }
        }
    }
    __syncthreads();

    // ---- phase 2: warps 0-1 invert the unit lower triangle by forward substitution (column per lane, fp32, fixed
    //      order); warps 2-7 meanwhile turn sK into diag(beta) k 2^g and load diag(beta) v into sG ---------------
    if (warp < 2) {
        const int col = tid;
        float x[CH];
#pragma unroll
        for (int r = 0; r < CH; ++r) {
            float s = (r == col) ? 1.f : 0.f;
#pragma unroll
            for (int q = 0; q < r; ++q) s = fmaf(-sM[r * MLD + q], x[q], s);
            x[r] = s;
        }
#pragma unroll
        for (int r = 0; r < CH; ++r) sInv[r * MLD + col] = x[r];
    } else {
        const int u = tid - 64;
        for (int i = u; i < CH * 32; i += 192) {
            const int r = i >> 5, c4 = (i & 31) * 4;
            float4 kv = *reinterpret_cast<float4*>(sK + r * KLD + c4);
            const float4 gv = *reinterpret_cast<const float4*>(sG + r * KLD + c4);
            const float b = sBeta[r];
            kv.x *= b * exp2f(gv.x); kv.y *= b * exp2f(gv.y); kv.z *= b * exp2f(gv.z); kv.w *= b * exp2f(gv.w);
            *reinterpret_cast<float4*>(sK + r * KLD + c4) = kv;
        }
        asm volatile("bar.sync 1, 192;" ::: "memory");
        for (int i = u; i < CH * 32; i += 192) {
            const int r = i >> 5, c4 = (i & 31) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < len) {
                v = ld4(p.v, p.qkv_dtype, ((size_t)(start + r) * HV + h) * 128 + c4);
                const float b = sBeta[r];
                v.x *= b; v.y *= b; v.z *= b; v.w *= b;
            }
            *reinterpret_cast<float4*>(sG + r * KLD + c4) = v;
        }
    }
    __syncthreads();

    // ---- phase 3: nw = -A (beta k~), u = A (beta v); A is lower triangular so row block wm needs 16 (wm + 1) terms --
    {
        const int wm = warp & 3, wn = warp >> 2;
        const int r0 = wm * 16 + g, r1 = r0 + 8;
        float acc[8][4];
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
            zero_acc<8>(acc);
            warp_mma<8, PREC, MLD, 1, KLD, 1>(acc, sInv + wm * 16 * MLD, (pass ? sG : sK) + wn * 64, 16 * (wm + 1));
            float* out = pass ? p.u : p.nw;
            const float sgn = pass ? 1.f : -1.f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const int col = wn * 64 + nt * 8 + 2 * t;
                if (r0 < len)
                    *reinterpret_cast<float2*>(out + ((size_t)(start + r0) * HV + h) * 128 + col) = make_float2(sgn * acc[nt][0], sgn * acc[nt][1]);
                if (r1 < len)
                    *reinterpret_cast<float2*>(out + ((size_t)(start + r1) * HV + h) * 128 + col) = make_float2(sgn * acc[nt][2], sgn * acc[nt][3]);
            }
        }
    }
    // A and Aqk rows, coalesced
    for (int i = tid; i < CH * 16; i += 256) {
        const int r = i >> 4, c4 = (i & 15) * 4;
        if (r < len) {
            const size_t o = ((size_t)(start + r) * HV + h) * 64 + c4;
            *reinterpret_cast<float4*>(p.A + o) = *reinterpret_cast<const float4*>(sInv + r * MLD + c4);
            *reinterpret_cast<float4*>(p.Aqk + o) = *reinterpret_cast<const float4*>(sP + r * MLD + c4);
        }
    }
}

}  // namespace mkda

using namespace mkda;

extern "C" int mkda_intra_fwd(const MkdaIntraFwd* p, void* stream) {
    if (!p || !p->q || !p->k || !p->v || !p->g_c || !p->beta || !p->A || !p->Aqk || !p->nw || !p->u)
        return set_error(MKDA_ERR_ARG, "intra_fwd: null argument");
    if (p->L.HK <= 0 || p->L.HV % p->L.HK) return set_error(MKDA_ERR_ARG, "intra_fwd: HV must be a multiple of HK");
    if (p->L.NC == 0) return MKDA_OK;
    if (!legacy_kernels()) return launch_intra_fwd_tc(p, (cudaStream_t)stream);
    auto kern = intra_fwd_kernel<MKDA_PREC_INTRA>;
    if (int e = ensure_smem((const void*)kern, INTRA_SMEM, "intra_fwd")) return e;
    kern<<<dim3(p->L.NC, p->L.HV), 256, INTRA_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("intra_fwd");
}

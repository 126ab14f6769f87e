// Chunk-parallel gradients through the decayed K K^T / Q K^T blocks, one CTA (8 warps) per (chunk, v-head).
//
// With E_ij = 2^(g_i - g_j) per channel (i > j), Wq = scale strictlower(dAqk), dLs = strictlower(dL):
//   dq_row_i = sum_j Wq_ij k_j E_ij                     T_i = sum_j dLs_ij k_j E_ij
//   dk_col_j = sum_i (Wq_ij q_i + beta_i dLs_ij k_i) E_ij
//   dq = dq_p + dq_row + scale dAqk_ii k       dk = dk_p + beta T + dk_col + scale dAqk_ii q
//   dg' = dg_p + q dq_row + k beta T - k dk_col           dbeta_g = sum_c k T
// E_ij is factored through the first row a of i's 16-row block, E_ij = 2^(g_i - g_a) 2^(g_a - g_j): both factors are
// <= 1 off the diagonal block and bounded by 2^(15*5/ln2) inside it, and nothing depends on rows later than i.
// Warp w owns channels 16w..16w+15 for every row block; row blocks are walked from the last to the first so that a
// block's rows are complete (all column contributions received) when it is finalised.
#include "common.cuh"
#include "host.h"

#ifndef MKDA_PREC_INTRA_BWD
#define MKDA_PREC_INTRA_BWD 1
#endif

namespace mkda {

constexpr int KLD = 132;
constexpr int MLD = 68;
constexpr int INTRA_BWD_SMEM = (3 * CH * KLD + 3 * CH * MLD + 2 * CH + 8 * CH) * 4;

template <int PREC>
__global__ void __launch_bounds__(256, 1) bwd_intra_kernel(const MkdaBwdIntra p) {
    extern __shared__ __align__(16) float smem[];
    float* sK = smem;
    float* sQ = sK + CH * KLD;
    float* sG = sQ + CH * KLD;
    float* sWq = sG + CH * KLD;         // scale * strictlower(dAqk)
    float* sDl = sWq + CH * MLD;        // strictlower(dL)
    float* sBd = sDl + CH * MLD;        // diag(beta) strictlower(dL)
    float* sBeta = sBd + CH * MLD;
    float* sDiag = sBeta + CH;          // scale * dAqk_ii
    float* sRed = sDiag + CH;           // [8][64]

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int cs = warp * 16;

    stage_rows128<KLD, 256>(sK, p.k, p.qk_dtype, start, len, HK, hk, p.k_rstd);
    stage_rows128<KLD, 256>(sQ, p.q, p.qk_dtype, start, len, HK, hk, p.q_rstd);
    for (int i = tid; i < CH * 32; i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        const int rr = r < len ? r : len - 1;
        *reinterpret_cast<float4*>(sG + r * KLD + c4) =
            *reinterpret_cast<const float4*>(p.g_c + ((size_t)(start + rr) * HV + h) * 128 + c4);
    }
    for (int i = tid; i < CH * CH; i += 256) {
        const int r = i >> 6, j = i & 63;
        float wq = 0.f, dl = 0.f, bt = 0.f;
        if (r < len) {
            const size_t th = (size_t)(start + r) * HV + h;
            bt = p.beta[th];
            const float aq = p.scale * p.dAqk[th * 64 + j];
            if (j < r) { wq = aq; dl = p.dL[th * 64 + j]; }
            if (j == r) sDiag[r] = aq;
        } else if (j == r) {
            sDiag[r] = 0.f;
        }
        sWq[r * MLD + j] = wq;
        sDl[r * MLD + j] = dl;
        sBd[r * MLD + j] = bt * dl;
        if (j == 0) sBeta[r] = bt;
    }
    for (int i = tid; i < 8 * CH; i += 256) sRed[i] = 0.f;
    __syncthreads();

    float dkc[4][2][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) zero_acc<2>(dkc[a]);

#pragma unroll
    for (int II = 0; II < 4; ++II) {
        const int I = 3 - II, a = 16 * I;
        if (a >= len) continue;                                   // block-uniform
        const int r0 = a + g, r1 = r0 + 8;
        // ---- row terms: [Wq_I; dLs_I] (32 x 16(I+1)) times the column operand k_j 2^(g_a - g_j) -------------------
        float rq[2][4], rt[2][4];
        zero_acc<2>(rq);
        zero_acc<2>(rt);
        for (int j0 = 0; j0 < 16 * (I + 1); j0 += 8) {
            FragA<PREC> fq, ft;
            fq.set(0, sWq[r0 * MLD + j0 + t]); fq.set(1, sWq[r1 * MLD + j0 + t]);
            fq.set(2, sWq[r0 * MLD + j0 + t + 4]); fq.set(3, sWq[r1 * MLD + j0 + t + 4]);
            ft.set(0, sDl[r0 * MLD + j0 + t]); ft.set(1, sDl[r1 * MLD + j0 + t]);
            ft.set(2, sDl[r0 * MLD + j0 + t + 4]); ft.set(3, sDl[r1 * MLD + j0 + t + 4]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int cc = cs + nt * 8 + g;
                const float ga = sG[a * KLD + cc];
                FragB<PREC> fb;
                fb.set(0, sK[(j0 + t) * KLD + cc] * exp2f(ga - sG[(j0 + t) * KLD + cc]));
                fb.set(1, sK[(j0 + t + 4) * KLD + cc] * exp2f(ga - sG[(j0 + t + 4) * KLD + cc]));
                mma_frag<PREC>(rq[nt], fq, fb);
                mma_frag<PREC>(rt[nt], ft, fb);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = (e & 2) ? r1 : r0, cc = cs + nt * 8 + 2 * t + (e & 1);
                const float sc = exp2f(sG[r * KLD + cc] - sG[a * KLD + cc]);
                rq[nt][e] *= sc;
                rt[nt][e] *= sc;
            }
        // ---- column terms: Wq_I^T (q_i 2^(g_i - g_a)) + (beta dLs)_I^T (k_i 2^(g_i - g_a)), then 2^(g_a - g_j) -------
        FragB<PREC> bq[2][2], bk[2][2];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int cc = cs + nt * 8 + g, i0 = a + ks * 8 + t, i1 = i0 + 4;
                const float ga = sG[a * KLD + cc];
                const float e0 = exp2f(sG[i0 * KLD + cc] - ga), e1 = exp2f(sG[i1 * KLD + cc] - ga);
                bq[ks][nt].set(0, sQ[i0 * KLD + cc] * e0); bq[ks][nt].set(1, sQ[i1 * KLD + cc] * e1);
                bk[ks][nt].set(0, sK[i0 * KLD + cc] * e0); bk[ks][nt].set(1, sK[i1 * KLD + cc] * e1);
            }
#pragma unroll
        for (int jt = 0; jt < 4; ++jt) {
            if (jt > I) continue;
            float cc4[2][4];
            zero_acc<2>(cc4);
            const int j0 = jt * 16 + g, j1 = j0 + 8;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                const int i0 = a + ks * 8 + t, i1 = i0 + 4;
                FragA<PREC> fw, fd;
                fw.set(0, sWq[i0 * MLD + j0]); fw.set(1, sWq[i0 * MLD + j1]);
                fw.set(2, sWq[i1 * MLD + j0]); fw.set(3, sWq[i1 * MLD + j1]);
                fd.set(0, sBd[i0 * MLD + j0]); fd.set(1, sBd[i0 * MLD + j1]);
                fd.set(2, sBd[i1 * MLD + j0]); fd.set(3, sBd[i1 * MLD + j1]);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    mma_frag<PREC>(cc4[nt], fw, bq[ks][nt]);
                    mma_frag<PREC>(cc4[nt], fd, bk[ks][nt]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = (e & 2) ? j1 : j0, cc = cs + nt * 8 + 2 * t + (e & 1);
                    dkc[jt][nt][e] += cc4[nt][e] * exp2f(sG[a * KLD + cc] - sG[j * KLD + cc]);
                }
        }
        // ---- finalise the rows of block I ---------------------------------------------------------------------------
        float bs0 = 0.f, bs1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int cc = cs + nt * 8 + 2 * t;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = half ? r1 : r0;
                const float bt = sBeta[r], dgn = sDiag[r];
                const float k0 = sK[r * KLD + cc], k1 = sK[r * KLD + cc + 1];
                const float q0 = sQ[r * KLD + cc], q1 = sQ[r * KLD + cc + 1];
                const float dq0 = rq[nt][2 * half], dq1 = rq[nt][2 * half + 1];
                const float T0 = rt[nt][2 * half], T1 = rt[nt][2 * half + 1];
                const float dc0 = dkc[I][nt][2 * half], dc1 = dkc[I][nt][2 * half + 1];
                if (half) bs1 += k0 * T0 + k1 * T1; else bs0 += k0 * T0 + k1 * T1;
                if (r >= len) continue;
                const size_t off = ((size_t)(start + r) * HV + h) * 128 + cc;
                const float2 pq = *reinterpret_cast<const float2*>(p.dq_p + off);
                const float2 pk = *reinterpret_cast<const float2*>(p.dk_p + off);
                const float2 pg = *reinterpret_cast<const float2*>(p.dg_p + off);
                *reinterpret_cast<float2*>(p.dq_v + off) = make_float2(pq.x + dq0 + dgn * k0, pq.y + dq1 + dgn * k1);
                *reinterpret_cast<float2*>(p.dk_v + off) = make_float2(pk.x + bt * T0 + dc0 + dgn * q0, pk.y + bt * T1 + dc1 + dgn * q1);
                *reinterpret_cast<float2*>(p.dgp + off) = make_float2(pg.x + q0 * dq0 + k0 * bt * T0 - k0 * dc0,
                                                                      pg.y + q1 * dq1 + k1 * bt * T1 - k1 * dc1);
            }
        }
        bs0 += __shfl_xor_sync(0xffffffffu, bs0, 1); bs0 += __shfl_xor_sync(0xffffffffu, bs0, 2);
        bs1 += __shfl_xor_sync(0xffffffffu, bs1, 1); bs1 += __shfl_xor_sync(0xffffffffu, bs1, 2);
        if (t == 0) { sRed[warp * CH + r0] = bs0; sRed[warp * CH + r1] = bs1; }
    }
    __syncthreads();
    if (tid < len) {
        const size_t th = (size_t)(start + tid) * HV + h;
        float s = sRed[tid];
        for (int w = 1; w < 8; ++w) s += sRed[w * CH + tid];
        float db = p.dbeta_w[th] + s;
        if (p.beta_sigmoid) {
            const float sg = sigmoidf_(ld1(p.beta_raw, p.beta_dtype, th));
            db *= p.beta_scale * sg * (1.f - sg);
        }
        st1(p.dbeta, p.dbeta_dtype, th, db);
    }
}

}  // namespace mkda

using namespace mkda;

extern "C" int mkda_bwd_intra(const MkdaBwdIntra* p, void* stream) {
    if (!p || !p->q || !p->k || !p->g_c || !p->beta || !p->dAqk || !p->dL || !p->dq_p || !p->dk_p || !p->dg_p ||
        !p->dbeta_w || !p->dq_v || !p->dk_v || !p->dgp || !p->dbeta)
        return set_error(MKDA_ERR_ARG, "bwd_intra: null argument");
    if (p->beta_sigmoid && !p->beta_raw) return set_error(MKDA_ERR_ARG, "bwd_intra: sigmoid beta needs the raw input");
    if (p->L.NC == 0) return MKDA_OK;
    if (!legacy_kernels()) return launch_bwd_intra_tc(p, (cudaStream_t)stream);
    auto kern = bwd_intra_kernel<MKDA_PREC_INTRA_BWD>;
    if (int e = ensure_smem((const void*)kern, INTRA_BWD_SMEM, "bwd_intra")) return e;
    kern<<<dim3(p->L.NC, p->L.HV), 256, INTRA_BWD_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("bwd_intra");
}

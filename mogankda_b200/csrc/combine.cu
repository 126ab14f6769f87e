// Prefix combine of per-segment (state, transition) pairs: the step that joins the segments of one long sequence, and
// the ranks of a context-parallel group, into the states entering each segment.
#include "common.cuh"
#include "host.h"

namespace mkda {

constexpr int LDA = 132;   // [128][128] tile read as A(m = row, k = col) or A(m = col, k = row)
constexpr int CW = 32;     // state columns per CTA
constexpr int LDS = CW + 8;   // [128][CW] tile read as B(k = row, n = col)

// ---------------------------------------------------------------------------------------------------------
// prefix combine over the segments of a group: one CTA per (32-column block, v-head, group).
//   forward:  X <- M_s X + H_s          backward: X <- M_s^T X + D_s
// X enters segment s before the update (stored to s_in[s]).  Error-compensated TF32 keeps the carried state at
// fp32 accuracy however many segments are chained.  The chain is serial, so the next segment's transition matrix is
// copied into the second buffer (cp.async) and its H / D block into registers while the current product runs.
// ---------------------------------------------------------------------------------------------------------
constexpr int COMBINE_SMEM = (DK * LDS + 2 * DK * LDA) * 4;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}

__global__ void __launch_bounds__(256, 1) combine_kernel(const MkdaCombine p) {
    extern __shared__ __align__(16) float smem[];
    float* sX = smem;                                  // [128][LDS]  B(k, n)
    float* sMb[2] = {sX + DK * LDS, sX + DK * LDS + DK * LDA};   // [128][LDA]  A(m, k) = M[m][k] (forward) or M[k][m] (reverse)
    const int cb = blockIdx.x, h = blockIdx.y, grp = blockIdx.z, HV = p.HV;
    const int col0 = cb * CW;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int kr0 = warp * 16 + g, kr1 = kr0 + 8;
    constexpr int NT = CW / 8;
    float X[NT][4], Hn[NT][4];
    {
        const float* src = p.carry ? p.carry + ((size_t)grp * HV + h) * DK * DV : nullptr;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = (e & 2) ? kr1 : kr0, cc = col0 + nt * 8 + 2 * t + (e & 1);
                X[nt][e] = src ? src[(size_t)kk * DV + cc] : 0.f;
            }
    }
    const int s_beg = p.grp_seg_off[grp], s_end = p.grp_seg_off[grp + 1], n = s_end - s_beg;
    auto seg = [&](int i) { return p.reverse ? s_end - 1 - i : s_beg + i; };
    auto fetch_m = [&](int i, float* dst) {            // 64 KB, 16 x 16 bytes per thread
        const float* src = p.ms + ((size_t)seg(i) * HV + h) * DK * DK;
        for (int j = tid; j < DK * 32; j += 256) {
            const int r = j >> 5, c4 = (j & 31) * 4;
            cp_async16(dst + r * LDA + c4, src + (size_t)r * DK + c4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto fetch_h = [&](int i) {
        const size_t base = ((size_t)seg(i) * HV + h) * DK * DV;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int cc = col0 + nt * 8 + 2 * t;
            float2 a = make_float2(0.f, 0.f), b = a;
            if (p.hs) {
                a = *reinterpret_cast<const float2*>(p.hs + base + (size_t)kr0 * DV + cc);
                b = *reinterpret_cast<const float2*>(p.hs + base + (size_t)kr1 * DV + cc);
            }
            Hn[nt][0] = a.x; Hn[nt][1] = a.y; Hn[nt][2] = b.x; Hn[nt][3] = b.y;
        }
    };
    if (n > 0) { fetch_m(0, sMb[0]); fetch_h(0); }
    for (int i = 0; i < n; ++i) {
        const int cur = i & 1;
        const size_t base = ((size_t)seg(i) * HV + h) * DK * DV;
        if (i + 1 < n) fetch_m(i + 1, sMb[cur ^ 1]);   // its last reader, the product of step i - 1, is behind a barrier
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int cc = nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(sX + kr0 * LDS + cc) = make_float2(X[nt][0], X[nt][1]);
            *reinterpret_cast<float2*>(sX + kr1 * LDS + cc) = make_float2(X[nt][2], X[nt][3]);
            if (p.s_in) {
                *reinterpret_cast<float2*>(p.s_in + base + (size_t)kr0 * DV + col0 + cc) = make_float2(X[nt][0], X[nt][1]);
                *reinterpret_cast<float2*>(p.s_in + base + (size_t)kr1 * DV + col0 + cc) = make_float2(X[nt][2], X[nt][3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) X[nt][e] = Hn[nt][e];
        if (i + 1 < n) {
            fetch_h(i + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");     // this step's matrix has landed, the next may be in flight
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (p.reverse) warp_mma<NT, 3, 1, LDA, LDS, 1>(X, sMb[cur] + warp * 16, sX, DK);
        else warp_mma<NT, 3, LDA, 1, LDS, 1>(X, sMb[cur] + warp * 16 * LDA, sX, DK);
        __syncthreads();
    }
    if (p.s_out) {
        float* out = p.s_out + ((size_t)grp * HV + h) * DK * DV;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int cc = col0 + nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(out + (size_t)kr0 * DV + cc) = make_float2(X[nt][0], X[nt][1]);
            *reinterpret_cast<float2*>(out + (size_t)kr1 * DV + cc) = make_float2(X[nt][2], X[nt][3]);
        }
    }
}

}  // namespace mkda

using namespace mkda;

extern "C" int mkda_state_combine(const MkdaCombine* p, void* stream) {
    if (!p || !p->grp_seg_off || !p->ms || (!p->s_in && !p->s_out)) return set_error(MKDA_ERR_ARG, "state_combine: null argument");
    if (p->NG == 0) return MKDA_OK;
    if (int e = ensure_smem((const void*)combine_kernel, COMBINE_SMEM, "state_combine")) return e;
    combine_kernel<<<dim3(DV / CW, p->HV, p->NG), 256, COMBINE_SMEM, (cudaStream_t)stream>>>(*p);
    return check_launch("state_combine");
}

// Intra-chunk kernels on the Blackwell tensor cores: WY preparation (forward) and the gradients through the decayed
// K K^T / Q K^T blocks (backward).  One CTA (16 warps) per (chunk, v-head).
//
// The per-channel decay 2^(g_i - g_j) does not factor out of the contraction over channels, so each 16-row block I is
// anchored at its first row a = 16 I (see intra_fwd.cu for the range / prefix-invariance argument):
//   row operand     Kr[i] = k_i 2^(g_i - g_a(i)),  Qr[i] = q_i 2^(g_i - g_a(i))      one tile for all 64 rows
//   column operand  Kc_I[j] = k_j 2^(g_aI - g_j),  j < 16 (I + 1)                    one tile per row block
// With M = 128 mandatory, the column operand goes on M:  D_I[j][r] = Kc_I[j] . [Kr_I; Qr_I][r]  (N = 32, K = 128);
// lanes j >= 16 (I + 1) read whatever follows the tile and are ignored (a D row depends on its own A row only).
#include "common.cuh"
#include "host.h"
#include "umma.cuh"

namespace mkda {

using umma::store_split8;

__device__ __forceinline__ void ldg8(const void* base, int dtype, size_t idx, float (&v)[8]) {
    const float4 a = ld4(base, dtype, idx), b = ld4(base, dtype, idx + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void lds8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void publish() {
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
}

struct IntraShared {
    uint64_t bar;
    uint32_t tmem;
    float beta[CH];
    float T[3][16][17];
};

constexpr int MLD = 68;
// byte offsets of the column-operand tiles (hi; lo follows hi) inside the operand region
__host__ __device__ constexpr int kc_off(int I) { return I == 0 ? 0 : I == 1 ? 8192 : I == 2 ? 24576 : 49152; }
__host__ __device__ constexpr int kc_bytes(int I) { return 16 * (I + 1) * 128 * 2; }          // one of hi / lo
constexpr int KQ_OFF = 81920;                              // [128][128] hi 32 KB, lo 32 KB
constexpr int OPND_BYTES = KQ_OFF + 65536;                 // 144 KB
constexpr int INTRA_TC_SMEM = OPND_BYTES + 3 * CH * MLD * 4 + 1024;

// Blocked inverse of the unit lower-triangular 64 x 64 matrix sM into sInv (fp32, fixed summation order):
// the four 16 x 16 diagonal blocks by forward substitution, then block row I = 1..3 from the rows above it.
__device__ __forceinline__ void invert_unit_lower(const float* __restrict__ sM, float* __restrict__ sInv, IntraShared& sh) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (warp < 4 && lane < 16) {
        const int o = 16 * warp;
        float x[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            float s = (r == lane) ? 1.f : 0.f;
#pragma unroll
            for (int c = 0; c < r; ++c) s = fmaf(-sM[(o + r) * MLD + o + c], x[c], s);
            x[r] = s;
        }
#pragma unroll
        for (int r = 0; r < 16; ++r) sInv[(o + r) * MLD + o + lane] = x[r];
    }
    __syncthreads();
    for (int I = 1; I < 4; ++I) {
        const int J = tid >> 8, r = (tid >> 4) & 15, c = tid & 15;
        const bool on = J < I;            // tid < 512 -> J in {0, 1}; block row 3 needs J = 2 as well, done by a second pass
        for (int pass = 0; pass < 2; ++pass) {
            const int JJ = J + 2 * pass;
            if (JJ < I && (pass == 0 ? on : true)) {
                float s = 0.f;
                for (int kb = JJ; kb < I; ++kb)
#pragma unroll
                    for (int e = 0; e < 16; ++e) s = fmaf(sM[(16 * I + r) * MLD + 16 * kb + e], sInv[(16 * kb + e) * MLD + 16 * JJ + c], s);
                sh.T[JJ][r][c] = s;
            }
        }
        __syncthreads();
        for (int pass = 0; pass < 2; ++pass) {
            const int JJ = J + 2 * pass;
            if (JJ < I) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < 16; ++e) s = fmaf(sInv[(16 * I + r) * MLD + 16 * I + e], sh.T[JJ][e][c], s);
                sInv[(16 * I + r) * MLD + 16 * JJ + c] = -s;
            }
        }
        __syncthreads();
    }
}

template <int DT>
__global__ void __launch_bounds__(512, 1) intra_fwd_tc_kernel(const MkdaIntraFwd p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ IntraShared sh;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKQ = base + KQ_OFF;
    float* sM = reinterpret_cast<float*>(base + OPND_BYTES);
    float* sInv = sM + CH * MLD;
    float* sP = sInv + CH * MLD;
    float* sG = sInv;                                  // [64][128] fp32 cumsum tile while the operands are built
    uint8_t* sBk = base;                               // phase 3: beta k~ [j][K index], hi 16 KB + lo 16 KB
    uint8_t* sBv = base + 32768;                       // beta v [j][v]
    uint8_t* sTA = base + 65536;                       // A [i][j], hi 8 KB + lo 8 KB

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, cg = warp >> 2, row = q * 32 + lane;

    MKDA_TRACE_AT(3, 0);
    if (warp == 0) umma::tmem_alloc(&sh.tmem, 256);
    if (tid == 0) { umma::mbar_init(&sh.bar, 1); umma::fence_barrier_init(); }
    if (tid < CH) sh.beta[tid] = tid < len ? p.beta[(size_t)(start + tid) * HV + h] : 0.f;

    // ---- phase 0: fetch k, q, g (2 (row, chunk) pairs per thread); park g in shared memory for the anchor look-ups ----
    float vk[2][8], vq[2][8], vg[2][8], rk[2], rq[2];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
        const size_t tk = (size_t)(start + rr) * HK + hk;
        ldg8(p.k, DT, tk * 128 + k8 * 8, vk[n]);
        ldg8(p.q, DT, tk * 128 + k8 * 8, vq[n]);
        ldg8(p.g_c, MKDA_F32, ((size_t)(start + rr) * HV + h) * 128 + k8 * 8, vg[n]);
        rk[n] = r < len ? (p.k_rstd ? p.k_rstd[tk] : 1.f) : 0.f;
        rq[n] = r < len ? (p.q_rstd ? p.q_rstd[tk] : 1.f) : 0.f;
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
        *reinterpret_cast<float4*>(sG + r * 128 + k8 * 8) = make_float4(vg[n][0], vg[n][1], vg[n][2], vg[n][3]);
        *reinterpret_cast<float4*>(sG + r * 128 + k8 * 8 + 4) = make_float4(vg[n][4], vg[n][5], vg[n][6], vg[n][7]);
#pragma unroll
        for (int e = 0; e < 8; ++e) { vk[n][e] *= rk[n]; vq[n][e] *= rq[n]; }
    }
    MKDA_TRACE_AT(3, 1);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = sh.tmem;
    MKDA_TRACE_AT(3, 2);
    // ---- operands ---------------------------------------------------------------------------------------------------
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15, I0 = r >> 4;
        float ga[8], t8[8];
        lds8(sG + (16 * I0) * 128 + k8 * 8, ga);
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = vk[n][e] * ex2f_(vg[n][e] - ga[e]);
        store_split8(sKQ, sKQ + 32768, 128, 32 * I0 + (r & 15), k8, t8);
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = vq[n][e] * ex2f_(vg[n][e] - ga[e]);
        store_split8(sKQ, sKQ + 32768, 128, 32 * I0 + 16 + (r & 15), k8, t8);
#pragma unroll
        for (int I = 0; I < 4; ++I) {
            if (I < I0) continue;
            if (I > I0) lds8(sG + (16 * I) * 128 + k8 * 8, ga);
#pragma unroll
            for (int e = 0; e < 8; ++e) t8[e] = vk[n][e] * ex2f_(ga[e] - vg[n][e]);
            store_split8(base + kc_off(I), base + kc_off(I) + kc_bytes(I), 16 * (I + 1), r, k8, t8);
        }
    }
    MKDA_TRACE_AT(3, 3);
    publish();
    if (tid == 0) {
#pragma unroll
        for (int I = 0; I < 4; ++I)
            umma::gemm(tmem + 32 * I, umma::opnd_k(base + kc_off(I), base + kc_off(I) + kc_bytes(I), 16 * (I + 1)),
                       umma::opnd_k(sKQ, sKQ + 32768, 128, 32 * I), 128, 32, 128, 0u);
        umma::commit(&sh.bar);
    }
    // v for phase 3 is fetched while the products run
    float vv[2][8];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
        ldg8(p.v, DT, ((size_t)(start + rr) * HV + h) * 128 + k8 * 8, vv[n]);
    }
    MKDA_TRACE_AT(3, 4);
    umma::mbar_wait(&sh.bar, 0);
    umma::fence_after_sync();
    MKDA_TRACE_AT(3, 5);
    // phase-3 operands over the dead phase-1 tiles: beta k 2^g and beta v (rows past the end are zero)
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
        const float b = sh.beta[r];          // 0 for rows past the end
        float t8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = b * vk[n][e] * ex2f_(vg[n][e]);
        store_split8(sBk, sBk + 16384, 64, r, k8, t8);
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = b * vv[n][e];
        store_split8(sBv, sBv + 16384, 64, r, k8, t8);
    }
    __syncthreads();                          // every thread is done with the cumsum tile (sP / sInv alias it)
    for (int i = tid; i < CH * MLD; i += 512) sInv[i] = 0.f;
    if (q < 2) {                              // lane = column j, cg = row block I: Gamma / Q K^T entries (16 I + r, j)
        float v[32];
        umma::tmem_ld32(umma::tmem_addr(tmem, warp, 32 * cg), v);
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int i = 16 * cg + r;
            sM[i * MLD + row] = row < i ? sh.beta[i] * v[r] : (row == i ? 1.f : 0.f);
            sP[i * MLD + row] = row <= i ? p.scale * v[16 + r] : 0.f;
        }
    }
    __syncthreads();
    MKDA_TRACE_AT(3, 6);
    invert_unit_lower(sM, sInv, sh);
    MKDA_TRACE_AT(3, 7);
    {   // A as the B operand of phase 3, plus the global copies of A and Aqk (full rows, coalesced)
        const int r = tid >> 3, k8 = tid & 7;
        float a8[8];
        lds8(sInv + r * MLD + k8 * 8, a8);
        store_split8(sTA, sTA + 8192, 64, r, k8, a8);
        if (r < len) {
            const size_t o = ((size_t)(start + r) * HV + h) * 64 + k8 * 8;
            *reinterpret_cast<float4*>(p.A + o) = make_float4(a8[0], a8[1], a8[2], a8[3]);
            *reinterpret_cast<float4*>(p.A + o + 4) = make_float4(a8[4], a8[5], a8[6], a8[7]);
            *reinterpret_cast<float4*>(p.Aqk + o) = *reinterpret_cast<const float4*>(sP + r * MLD + k8 * 8);
            *reinterpret_cast<float4*>(p.Aqk + o + 4) = *reinterpret_cast<const float4*>(sP + r * MLD + k8 * 8 + 4);
        }
    }
    publish();
    if (tid == 0) {
        const umma::Opnd bA = umma::opnd_k(sTA, sTA + 8192, 64);
        umma::gemm(tmem + 128, umma::opnd_mn(sBk, sBk + 16384, 64), bA, 128, 64, 64, 0u);
        umma::gemm(tmem + 192, umma::opnd_mn(sBv, sBv + 16384, 64), bA, 128, 64, 64, 0u);
        umma::commit(&sh.bar);
    }
    MKDA_TRACE_AT(3, 8);
    umma::mbar_wait(&sh.bar, 1);
    umma::fence_after_sync();
    MKDA_TRACE_AT(3, 9);
    {
        float a[16], b[16];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 128 + 16 * cg), a);
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 192 + 16 * cg), b);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int i = 16 * cg + j;
            if (i < len) {
                const size_t o = ((size_t)(start + i) * HV + h) * 128 + row;
                p.nw[o] = -a[j];
                p.u[o] = b[j];
            }
        }
    }
    MKDA_TRACE_AT(3, 10);
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------------------
// bwd_intra on the tensor cores (math in intra_bwd.cu).  Channels go on M.  Per row block I (anchor a = 16 I):
//   row terms   R_I^T[c][r]  = sum_j Kc_I[j][c] W[16 I + r][j]       W = Wq (-> dq_row) or dLs (-> T); N = 16 each
//   col terms   C_I^T[c][j]  = sum_{i in I} Qr[i][c] Wq[i][j] + Kr[i][c] (beta dLs)[i][j]              N = 64
// then per thread (channel c, row block cg): dq_row = R 2^(g_i - g_a), T likewise, dk_col[j] = sum_{I >= cg} C_I 2^(g_aI - g_j).
// All A operands are MN-major views of the untransposed Kc / [Kr; Qr] tiles.
// ---------------------------------------------------------------------------------------------------------
constexpr int INTRA_BWD_TC_SMEM = OPND_BYTES + 3 * 16384 + 1024;

template <int DT>
__global__ void __launch_bounds__(512, 1) bwd_intra_tc_kernel(const MkdaBwdIntra p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ IntraShared sh;
    __shared__ float sDiag[CH];
    __shared__ float sRed[4][CH];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKQ = base + KQ_OFF;
    uint8_t* sWq = base + OPND_BYTES;                  // scale strictlower(dAqk) [i][j], hi 8 KB + lo 8 KB
    uint8_t* sDl = sWq + 16384;                        // strictlower(dL)
    uint8_t* sBd = sDl + 16384;                        // diag(beta) strictlower(dL)
    float* sG = reinterpret_cast<float*>(sWq);         // [64][128] fp32 cumsum tile while the Kc / KQ operands are built

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, cg = warp >> 2, row = q * 32 + lane;

    MKDA_TRACE_AT(4, 0);
    if (warp == 0) umma::tmem_alloc(&sh.tmem, 512);
    if (tid == 0) { umma::mbar_init(&sh.bar, 1); umma::fence_barrier_init(); }
    if (tid < CH) sh.beta[tid] = tid < len ? p.beta[(size_t)(start + tid) * HV + h] : 0.f;

    float vk[2][8], vq[2][8], vg[2][8], rk[2], rq[2], wa[8], wl[8];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
        const size_t tk = (size_t)(start + rr) * HK + hk;
        ldg8(p.k, DT, tk * 128 + k8 * 8, vk[n]);
        ldg8(p.q, DT, tk * 128 + k8 * 8, vq[n]);
        ldg8(p.g_c, MKDA_F32, ((size_t)(start + rr) * HV + h) * 128 + k8 * 8, vg[n]);
        rk[n] = r < len ? (p.k_rstd ? p.k_rstd[tk] : 1.f) : 0.f;
        rq[n] = r < len ? (p.q_rstd ? p.q_rstd[tk] : 1.f) : 0.f;
    }
    {
        const int i = tid >> 3, k8 = tid & 7, ii = i < len ? i : len - 1;
        const size_t o = ((size_t)(start + ii) * HV + h) * 64 + k8 * 8;
        ldg8(p.dAqk, MKDA_F32, o, wa);
        ldg8(p.dL, MKDA_F32, o, wl);
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
        *reinterpret_cast<float4*>(sG + r * 128 + k8 * 8) = make_float4(vg[n][0], vg[n][1], vg[n][2], vg[n][3]);
        *reinterpret_cast<float4*>(sG + r * 128 + k8 * 8 + 4) = make_float4(vg[n][4], vg[n][5], vg[n][6], vg[n][7]);
#pragma unroll
        for (int e = 0; e < 8; ++e) { vk[n][e] *= rk[n]; vq[n][e] *= rq[n]; }
    }
    MKDA_TRACE_AT(4, 1);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = sh.tmem;
    MKDA_TRACE_AT(4, 2);
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15, I0 = r >> 4;
        float ga[8], t8[8];
        lds8(sG + (16 * I0) * 128 + k8 * 8, ga);
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = vk[n][e] * ex2f_(vg[n][e] - ga[e]);
        store_split8(sKQ, sKQ + 32768, 128, 32 * I0 + (r & 15), k8, t8);
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = vq[n][e] * ex2f_(vg[n][e] - ga[e]);
        store_split8(sKQ, sKQ + 32768, 128, 32 * I0 + 16 + (r & 15), k8, t8);
#pragma unroll
        for (int I = 0; I < 4; ++I) {
            if (I < I0) continue;
            if (I > I0) lds8(sG + (16 * I) * 128 + k8 * 8, ga);
#pragma unroll
            for (int e = 0; e < 8; ++e) t8[e] = vk[n][e] * ex2f_(ga[e] - vg[n][e]);
            store_split8(base + kc_off(I), base + kc_off(I) + kc_bytes(I), 16 * (I + 1), r, k8, t8);
        }
    }
    MKDA_TRACE_AT(4, 3);
    __syncthreads();                                   // the cumsum tile is dead: its space becomes the W tiles
    {
        const int i = tid >> 3, k8 = tid & 7;
        const float bt = sh.beta[i];
        float w8[8], d8[8], b8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int j = k8 * 8 + e;
            const bool lo = j < i && i < len;
            w8[e] = lo ? p.scale * wa[e] : 0.f;
            d8[e] = lo ? wl[e] : 0.f;
            b8[e] = bt * d8[e];
            if (j == i) sDiag[i] = i < len ? p.scale * wa[e] : 0.f;
        }
        store_split8(sWq, sWq + 8192, 64, i, k8, w8);
        store_split8(sDl, sDl + 8192, 64, i, k8, d8);
        store_split8(sBd, sBd + 8192, 64, i, k8, b8);
    }
    MKDA_TRACE_AT(4, 4);
    publish();
    if (tid == 0) {
#pragma unroll
        for (int I = 0; I < 4; ++I) {
            const umma::Opnd aKc = umma::opnd_mn(base + kc_off(I), base + kc_off(I) + kc_bytes(I), 16 * (I + 1));
            umma::gemm(tmem + 32 * I, aKc, umma::opnd_k(sWq, sWq + 8192, 64, 16 * I), 128, 16, 16 * (I + 1), 0u);
            umma::gemm(tmem + 32 * I + 16, aKc, umma::opnd_k(sDl, sDl + 8192, 64, 16 * I), 128, 16, 16 * (I + 1), 0u);
            umma::gemm(tmem + 128 + 64 * I, umma::opnd_mn(sKQ, sKQ + 32768, 128, 32 * I + 16), umma::opnd_mn(sWq, sWq + 8192, 64, 16 * I),
                       128, 64, 16, 0u);
            umma::gemm(tmem + 128 + 64 * I, umma::opnd_mn(sKQ, sKQ + 32768, 128, 32 * I), umma::opnd_mn(sBd, sBd + 8192, 64, 16 * I),
                       128, 64, 16, 1u);
        }
        umma::commit(&sh.bar);
    }
    // epilogue inputs for (channel `row`, rows 16 cg .. 16 cg + 15) are fetched while the products run
    float kq[16], qq[16], gg[16], pq[16], pk[16], pg[16], ga[4];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int i = 16 * cg + r, ii = i < len ? i : len - 1;
        const size_t tk = (size_t)(start + ii) * HK + hk, off = ((size_t)(start + ii) * HV + h) * 128 + row;
        kq[r] = ld1(p.k, DT, tk * 128 + row) * (p.k_rstd ? p.k_rstd[tk] : 1.f);
        qq[r] = ld1(p.q, DT, tk * 128 + row) * (p.q_rstd ? p.q_rstd[tk] : 1.f);
        gg[r] = p.g_c[off];
        pq[r] = p.dq_p[off]; pk[r] = p.dk_p[off]; pg[r] = p.dg_p[off];
    }
#pragma unroll
    for (int I = 0; I < 4; ++I) {
        const int a = 16 * I < len ? 16 * I : len - 1;
        ga[I] = p.g_c[((size_t)(start + a) * HV + h) * 128 + row];
    }
    MKDA_TRACE_AT(4, 5);
    umma::mbar_wait(&sh.bar, 0);
    umma::fence_after_sync();
    MKDA_TRACE_AT(4, 6);
    float v[32], dkc[16];
    umma::tmem_ld32(umma::tmem_addr(tmem, warp, 32 * cg), v);
#pragma unroll
    for (int r = 0; r < 16; ++r) dkc[r] = 0.f;
#pragma unroll
    for (int I = 0; I < 4; ++I) {
        if (I < cg) continue;                          // warp-uniform
        float c16[16];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 128 + 64 * I + 16 * cg), c16);
#pragma unroll
        for (int r = 0; r < 16; ++r) dkc[r] += c16[r] * ex2f_(ga[I] - gg[r]);
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int i = 16 * cg + r;
        const float e = ex2f_(gg[r] - ga[cg]);
        const float dqr = v[r] * e, T = v[16 + r] * e, bt = sh.beta[i], dgn = sDiag[i];
        float bs = kq[r] * T;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) bs += __shfl_xor_sync(0xffffffffu, bs, o);
        if (lane == 0) sRed[q][i] = bs;
        if (i < len) {
            const size_t off = ((size_t)(start + i) * HV + h) * 128 + row;
            p.dq_v[off] = pq[r] + dqr + dgn * kq[r];
            p.dk_v[off] = pk[r] + bt * T + dkc[r] + dgn * qq[r];
            p.dgp[off] = pg[r] + qq[r] * dqr + kq[r] * bt * T - kq[r] * dkc[r];
        }
    }
    MKDA_TRACE_AT(4, 7);
    __syncthreads();
    if (tid < len) {
        const size_t th = (size_t)(start + tid) * HV + h;
        float db = p.dbeta_w[th] + ((sRed[0][tid] + sRed[1][tid]) + (sRed[2][tid] + sRed[3][tid]));
        if (p.beta_sigmoid) {
            const float sg = sigmoidf_(ld1(p.beta_raw, p.beta_dtype, th));
            db *= p.beta_scale * sg * (1.f - sg);
        }
        st1(p.dbeta, p.dbeta_dtype, th, db);
    }
    MKDA_TRACE_AT(4, 8);
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 512);
}

template <int DT>
static int launch_bwd_intra_tc_t(const MkdaBwdIntra* p, cudaStream_t stream) {
    auto kern = bwd_intra_tc_kernel<DT>;
    if (int e = ensure_smem((const void*)kern, INTRA_BWD_TC_SMEM, "bwd_intra")) return e;
    kern<<<dim3(p->L.NC, p->L.HV), 512, INTRA_BWD_TC_SMEM, stream>>>(*p);
    return check_launch("bwd_intra");
}
int launch_bwd_intra_tc(const MkdaBwdIntra* p, cudaStream_t stream) {
    switch (p->qk_dtype) {
        case MKDA_F32: return launch_bwd_intra_tc_t<MKDA_F32>(p, stream);
        case MKDA_BF16: return launch_bwd_intra_tc_t<MKDA_BF16>(p, stream);
        case MKDA_F16: return launch_bwd_intra_tc_t<MKDA_F16>(p, stream);
    }
    return set_error(MKDA_ERR_ARG, "bwd_intra: unsupported dtype");
}

#ifdef MKDA_TRACE
extern "C" int mkda_trace_read_intra(long long* out) { return cudaMemcpyFromSymbol(out, umma::g_trace, sizeof(long long) * 8 * 24) == cudaSuccess ? 0 : -1; }
#endif
int tc_intra_status(unsigned int* out) {
    return cudaMemcpyFromSymbol(out, umma::g_timeout_flag, sizeof(unsigned int)) == cudaSuccess ? 0 : -1;
}

template <int DT>
static int launch_intra_fwd_tc_t(const MkdaIntraFwd* p, cudaStream_t stream) {
    auto kern = intra_fwd_tc_kernel<DT>;
    if (int e = ensure_smem((const void*)kern, INTRA_TC_SMEM, "intra_fwd")) return e;
    kern<<<dim3(p->L.NC, p->L.HV), 512, INTRA_TC_SMEM, stream>>>(*p);
    return check_launch("intra_fwd");
}
int launch_intra_fwd_tc(const MkdaIntraFwd* p, cudaStream_t stream) {
    switch (p->qkv_dtype) {
        case MKDA_F32: return launch_intra_fwd_tc_t<MKDA_F32>(p, stream);
        case MKDA_BF16: return launch_intra_fwd_tc_t<MKDA_BF16>(p, stream);
        case MKDA_F16: return launch_intra_fwd_tc_t<MKDA_F16>(p, stream);
    }
    return set_error(MKDA_ERR_ARG, "intra_fwd: unsupported dtype");
}

}  // namespace mkda

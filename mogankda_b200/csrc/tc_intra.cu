// Intra-chunk kernels on the Blackwell tensor cores: WY preparation (forward) and the gradients through the decayed
// K K^T / Q K^T blocks (backward).  One CTA (16 warps) per (chunk, v-head).
//
// Forward:
//   Gamma_ij = sum_c k_ic k_jc 2^(g_ic - g_jc)  (i > j)        Aqk_ij = scale sum_c q_ic k_jc 2^(g_ic - g_jc)  (i >= j)
//   A  = (I + strictlower(diag(beta) Gamma))^-1
//   nw = -A diag(beta) (k 2^g)                                  u = A diag(beta) v
//
// Range / prefix invariance: the per-channel decay 2^(g_i - g_j) does not factor out of the contraction over channels,
// so each 16-row block I uses its first row a = 16 I as anchor: row operand k_i 2^(g_i - g_a) (<= 1), column operand
// k_j 2^(g_a - g_j) (<= 1 for j < a, <= 2^(15*5/ln2) inside the diagonal block).  An output element (i, j) therefore
// depends on rows i, j and a <= i only, never on later rows.  Rows past the end of the sequence are staged as zeros
// (their g as the last valid row's), so they produce identity rows in A and are never stored.
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
    ld8(base, dtype, idx, v);
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
    uint64_t bar, ldin;
    uint32_t tmem;
    float beta[CH];
    __align__(16) float T[32][36];
};
constexpr int TLD = 36;

constexpr int MLD = 68;
// byte offsets of the column-operand tiles (hi; lo follows hi) inside the operand region
__host__ __device__ constexpr int kc_off(int I) { return I == 0 ? 0 : I == 1 ? 8192 : I == 2 ? 24576 : 49152; }
__host__ __device__ constexpr int kc_bytes(int I) { return 16 * (I + 1) * 128 * 2; }          // one of hi / lo
// forward kernel: the same four column tiles stacked by rows into one 160-row tile (hi 40 KB, then lo)
__host__ __device__ constexpr int kc_row(int I) { return I == 0 ? 0 : I == 1 ? 16 : I == 2 ? 48 : 96; }
constexpr int KC_ALL_ROWS = 160;
constexpr int KC_ALL_BYTES = KC_ALL_ROWS * 128 * 2;        // one of hi / lo
constexpr int KQ_OFF = 81920;                              // [128][128] hi 32 KB, lo 32 KB
constexpr int OPND_BYTES = KQ_OFF + 65536;                 // 144 KB
// The 16-bit k, q and the g rows of the NEXT item arrive by tiled copy (one 64 x 128 box per tensor) while the current item's
// inverse and second products run: k and g rows in the upper 48 KB of the [Kr; Qr] tile, dead once the first products are
// done, q rows behind sP.  They are read back into registers before the next item's operands are staged over them.  (Loads
// into registers at that point are accepted only as fast as their data returns and occupied every thread for a fifth of
// the item; one small bulk copy per row is slower still.)
struct IntraMaps { CUtensorMap k, q, g; };
constexpr int RAW_K = 98304;                               // [64][128] 16-bit, 16 KB
constexpr int RAW_G = RAW_K + 16384;                       // [64][128] fp32, 32 KB
constexpr int RAW_Q = OPND_BYTES + 53248;                  // [64][128] 16-bit, 16 KB
constexpr int INTRA_TC_SMEM = RAW_Q + 16384 + 1024;        // operands + (two 32 KB hand-over tiles, later sM / sInv / sP) + q rows
static_assert(RAW_G + 32768 <= OPND_BYTES, "k / g rows must fit in the dead part of the operand region");
static_assert(3 * CH * MLD * 4 <= 53248, "sM / sInv / sP must end below the q rows");

// out[2][4] = A[2 rows][KD] * B[KD][4 columns] with fp32 FMAs in ascending k (the order every entry of the inverse has always
// been summed in); A rows are `lda` floats apart, B rows `ldb`; all pointers 16-byte aligned.  A 2 x 4 register tile needs
// 6 shared loads per 32 FMAs: the merges below are bound by shared-memory load issue, not by arithmetic.
template <int KD>
__device__ __forceinline__ void mm_tile_2x4(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb, float (&out)[2][4]) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) out[i][j] = 0.f;
#pragma unroll
    for (int k4 = 0; k4 < KD; k4 += 4) {
        const float4 a0 = *reinterpret_cast<const float4*>(A + k4), a1 = *reinterpret_cast<const float4*>(A + lda + k4);
        const float am[2][4] = {{a0.x, a0.y, a0.z, a0.w}, {a1.x, a1.y, a1.z, a1.w}};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float4 b4 = *reinterpret_cast<const float4*>(B + (k4 + k) * ldb);
            const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) out[i][j] = fmaf(am[i][k], bv[j], out[i][j]);
        }
    }
}

// Inverse of the unit lower-triangular 64 x 64 matrix sM into sInv (fp32, fixed summation order) by recursive halving:
// the four 16 x 16 diagonal blocks by forward substitution, then the off-diagonal block of each 32 x 32 half and finally
// the 32 x 32 block below the diagonal, each as  X = -B^-1 (C A^-1)  with A^-1 / B^-1 the inverses above / beside it.
// Every entry depends on the rows up to its own only, and the order of the sums is fixed by the indices.
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
    {   // 16 x 16 blocks (1, 0) and (3, 2): 32 threads per block, thread = (row pair, column quad)
        const int hb = tid >> 5, rp = (tid >> 2) & 7, cq = tid & 3;
        const int ro = 32 * hb + 16, co = 32 * hb;            // block origin; A^-1 at (co, co), B^-1 at (ro, ro)
        float o[2][4];
        if (tid < 64) {
            mm_tile_2x4<16>(sM + (ro + 2 * rp) * MLD + co, MLD, sInv + co * MLD + co + 4 * cq, MLD, o);
#pragma unroll
            for (int i = 0; i < 2; ++i)
                *reinterpret_cast<float4*>(&sh.T[16 * hb + 2 * rp + i][4 * cq]) = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
        }
        __syncthreads();
        if (tid < 64) {
            mm_tile_2x4<16>(sInv + (ro + 2 * rp) * MLD + ro, MLD, &sh.T[16 * hb][4 * cq], TLD, o);
#pragma unroll
            for (int i = 0; i < 2; ++i)
                *reinterpret_cast<float4*>(sInv + (ro + 2 * rp + i) * MLD + co + 4 * cq) = make_float4(-o[i][0], -o[i][1], -o[i][2], -o[i][3]);
        }
    }
    __syncthreads();
    {   // 32 x 32 block (rows 32.., columns 0..31): 128 threads, thread = (row pair, column quad)
        const int rp = tid >> 3, cq = tid & 7;
        float o[2][4];
        if (tid < 128) {
            mm_tile_2x4<32>(sM + (32 + 2 * rp) * MLD, MLD, sInv + 4 * cq, MLD, o);
#pragma unroll
            for (int i = 0; i < 2; ++i)
                *reinterpret_cast<float4*>(&sh.T[2 * rp + i][4 * cq]) = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
        }
        __syncthreads();
        if (tid < 128) {
            mm_tile_2x4<32>(sInv + (32 + 2 * rp) * MLD + 32, MLD, &sh.T[0][4 * cq], TLD, o);
#pragma unroll
            for (int i = 0; i < 2; ++i)
                *reinterpret_cast<float4*>(sInv + (32 + 2 * rp + i) * MLD + 4 * cq) = make_float4(-o[i][0], -o[i][1], -o[i][2], -o[i][3]);
        }
    }
    __syncthreads();
}

// SCALAR: the gate is one decay per token (the same cumsum in all 128 channels).  It then commutes with the contraction
// over channels, Gamma_ij = (k_i . k_j) 2^(g_i - g_j), so the products are plain K K^T / Q K^T (one product over a stacked
// [K; Q] tile) and the decay is applied to the accumulators, element by element and for i >= j only: nothing is anchored,
// no exponent is ever positive, and any g <= 0 is in range (the per-channel path needs g >= -5 per token).
template <int DT, bool SCALAR, bool TMA>
__global__ void __launch_bounds__(512, 1) intra_fwd_tc_kernel(const MkdaIntraFwd p, const __grid_constant__ IntraMaps maps) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ IntraShared sh;
    __shared__ __align__(16) float sGa[5][DK];         // cumsum rows of the four block anchors, [4] = last valid row
    __shared__ float sGs[CH];                          // SCALAR: the cumsum of every row (rows past the end: the last valid one)
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKQ = base + KQ_OFF;
    float* sM = reinterpret_cast<float*>(base + OPND_BYTES);
    float* sInv = sM + CH * MLD;
    float* sP = sInv + CH * MLD;
    uint8_t* sBk = base;                               // phase 3: beta k~ [j][K index], hi 16 KB + lo 16 KB
    uint8_t* sBv = base + 32768;                       // beta v [j][v]
    uint8_t* sTA = base + 65536;                       // A [i][j], hi 8 KB + lo 8 KB
    uint8_t* sTQ = base + 81920;                       // Aqk [i][j], hi 8 KB + lo 8 KB (only copied out)
    uint8_t* sKB = base + OPND_BYTES;                  // kbar [tok][K index] hi + lo (32 KB), only copied out; under sM ...
    uint8_t* sQS = sKB + 32768;                        // scale q 2^g [tok][K index] hi + lo (32 KB), likewise

    const int HV = p.L.HV, HK = p.L.HK, total = p.L.NC * HV, stride = gridDim.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, cg = warp >> 2, row = q * 32 + lane;

    // Persistent: one CTA per SM walks the (chunk, v-head) items gridDim.x apart, heads fastest.  The k, q, g rows (and beta,
    // the L2 statistics) of the NEXT item are requested into registers as soon as the current item has no more use for
    // its own, half way through the item, so that they travel while the inverse and the second products run.
    // k and q stay raw (unconverted) in registers until the item starts, so that nothing waits for them here.
    constexpr bool BULK = TMA && DT != MKDA_F32;       // fp32 rows would not fit: they travel through registers
    float vk[2][8], vq[2][8], vg[2][8], rk[2], rq[2], beta_r = 0.f;
    Raw8 wk[2], wq[2];
    uint32_t nin = 0;                                  // phase counter of the input-row barrier
    // the chunk table entries are read one item ahead of load_inputs: every address of an item depends on them
    int cur_start = 0, cur_len = 1, next_start = 0, next_len = 1;
    auto table_ahead = [&](int it) {
        if (it < total) { next_start = p.L.chunk_start[it / HV]; next_len = p.L.chunk_len[it / HV]; }
    };
    auto load_inputs = [&](int it) {
        const int c = it / HV, h = it - c * HV, hk = h / (HV / HK);
        const int start = next_start, len = next_len;
        cur_start = start; cur_len = len;
        if (tid < CH) beta_r = tid < len ? p.beta[(size_t)(start + tid) * HV + h] : 0.f;
        if (BULK && tid == 64) {                       // rows past the chunk's end belong to the next sequence (or read as zeros) and are never used
            umma::mbar_expect_tx(&sh.ldin, 16384u + 16384u + 32768u);
            umma::tma_load_rows(base + RAW_K, &maps.k, hk * 128, start, &sh.ldin);
            umma::tma_load_rows(base + RAW_Q, &maps.q, hk * 128, start, &sh.ldin);
            umma::tma_load_rows(base + RAW_G, &maps.g, h * 128, start, &sh.ldin);
        }
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
            const size_t tk = (size_t)(start + rr) * HK + hk;
            if (!BULK) {
                ldraw8<DT>(p.k, tk * 128 + k8 * 8, wk[n]);
                ldraw8<DT>(p.q, tk * 128 + k8 * 8, wq[n]);
                ldg8(p.g_c, MKDA_F32, ((size_t)(start + rr) * HV + h) * 128 + k8 * 8, vg[n]);
            }
            rk[n] = r < len ? (p.k_rstd ? p.k_rstd[tk] : 1.f) : 0.f;
            rq[n] = r < len ? (p.q_rstd ? p.q_rstd[tk] : 1.f) : 0.f;
        }
    };
    if (warp == 0) umma::tmem_alloc(&sh.tmem, 256);
    if (tid == 0) { umma::mbar_init(&sh.bar, 1); umma::mbar_init(&sh.ldin, 1); umma::fence_barrier_init(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = sh.tmem;
    table_ahead(blockIdx.x);
    if ((int)blockIdx.x < total) load_inputs(blockIdx.x);

    for (int item = blockIdx.x; item < total; item += stride) {
    const int c = item / HV, h = item - c * HV;
    const int start = cur_start, len = cur_len;
    table_ahead(item + stride);
    // ---- phase 0: this item's k, q, g rows into registers; park the anchor rows of g in shared memory ----
    if (tid < CH) sh.beta[tid] = beta_r;
    if (BULK) {
        umma::mbar_wait(&sh.ldin, nin & 1); ++nin;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
            wk[n].a = *reinterpret_cast<const uint4*>(base + RAW_K + rr * 256 + k8 * 16);
            wq[n].a = *reinterpret_cast<const uint4*>(base + RAW_Q + rr * 256 + k8 * 16);
            lds8(reinterpret_cast<const float*>(base + RAW_G + rr * 512 + k8 * 32), vg[n]);
        }
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
        if ((r & 15) == 0) {
            *reinterpret_cast<float4*>(&sGa[r >> 4][k8 * 8]) = make_float4(vg[n][0], vg[n][1], vg[n][2], vg[n][3]);
            *reinterpret_cast<float4*>(&sGa[r >> 4][k8 * 8 + 4]) = make_float4(vg[n][4], vg[n][5], vg[n][6], vg[n][7]);
        }
        if (r == len - 1) {
            *reinterpret_cast<float4*>(&sGa[4][k8 * 8]) = make_float4(vg[n][0], vg[n][1], vg[n][2], vg[n][3]);
            *reinterpret_cast<float4*>(&sGa[4][k8 * 8 + 4]) = make_float4(vg[n][4], vg[n][5], vg[n][6], vg[n][7]);
        }
        if (SCALAR && k8 == 0) sGs[r] = vg[n][0];
        unpack8<DT>(wk[n], vk[n]);
        unpack8<DT>(wq[n], vq[n]);
#pragma unroll
        for (int e = 0; e < 8; ++e) { vk[n][e] *= rk[n]; vq[n][e] *= rq[n]; }
    }
    if (tid == 0) umma::bulk_store_wait_read();        // the previous item's tiles have left shared memory
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- operands ---------------------------------------------------------------------------------------------------
    if (SCALAR) {          // one stacked tile: rows 0..63 = k, rows 64..127 = q (L2 statistics applied, zero past the end)
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
            store_split8(sKQ, sKQ + 32768, 128, r, k8, vk[n]);
            store_split8(sKQ, sKQ + 32768, 128, 64 + r, k8, vq[n]);
        }
    } else {
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int i = tid + n * 512, r = i >> 4, k8 = i & 15, I0 = r >> 4;
            float ga[8], t8[8];
            lds8(&sGa[I0][k8 * 8], ga);
#pragma unroll
            for (int e = 0; e < 8; ++e) t8[e] = vk[n][e] * ex2f_(vg[n][e] - ga[e]);
            store_split8(sKQ, sKQ + 32768, 128, 32 * I0 + (r & 15), k8, t8);
#pragma unroll
            for (int e = 0; e < 8; ++e) t8[e] = vq[n][e] * ex2f_(vg[n][e] - ga[e]);
            store_split8(sKQ, sKQ + 32768, 128, 32 * I0 + 16 + (r & 15), k8, t8);
#pragma unroll
            for (int I = 0; I < 4; ++I) {
                if (I < I0) continue;
                if (I > I0) lds8(&sGa[I][k8 * 8], ga);
#pragma unroll
                for (int e = 0; e < 8; ++e) t8[e] = vk[n][e] * ex2f_(ga[e] - vg[n][e]);
                store_split8(base, base + KC_ALL_BYTES, KC_ALL_ROWS, kc_row(I) + r, k8, t8);      // the four column tiles stacked by rows
            }
        }
    }
    publish();
    if (umma::mma_issuer()) {
        if (SCALAR) {      // D[m][j]: lanes 0..63 = K K^T rows, lanes 64..127 = Q K^T rows; columns j = K rows of the same tile
            umma::gemm(tmem, umma::opnd_k(sKQ, sKQ + 32768, 128), umma::opnd_k(sKQ, sKQ + 32768, 128), 128, 64, 128, 0u);
        } else {
            // ONE product over the stacked column tiles: D[32 I + t][kc_row(I') + j].  Only the blocks I' = I are meaningful (the
            // anchors of the two operands match there) and read back; the others are finite and ignored.  An MMA costs
            // (4 KB of A + 32 N bytes of B) / 128 B per cycle, so N = 160 once is far cheaper than N = 32 four times.
            umma::gemm(tmem, umma::opnd_k(sKQ, sKQ + 32768, 128), umma::opnd_k(base, base + KC_ALL_BYTES, KC_ALL_ROWS), 128, KC_ALL_ROWS, 128, 0u);
        }
        umma::commit(&sh.bar);
    }
    // v for phase 3 is fetched while the products run
    Raw8 wv[2];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
        ldraw8<DT>(p.v, ((size_t)(start + rr) * HV + h) * 128 + k8 * 8, wv[n]);
    }
    // ... and so are the hand-over tiles, built and sent off in the shadow of the products
    // The state kernels' scaled operands, as ready-made tiles: kbar = k 2^(gL - g) (gL = last valid row) and scale q 2^g,
    // plus gl = 2^gL.  Rows past the end are zero (their k / q were zeroed above).
    {
        float gLv[8];
        lds8(&sGa[4][(tid & 15) * 8], gLv);
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
            float t8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) t8[e] = vk[n][e] * ex2f_(gLv[e] - vg[n][e]);
            store_split8(sKB, sKB + 16384, 64, r, k8, t8);
#pragma unroll
            for (int e = 0; e < 8; ++e) t8[e] = p.scale * vq[n][e] * ex2f_(vg[n][e]);
            store_split8(sQS, sQS + 16384, 64, r, k8, t8);
        }
        if (tid < 16) {
            float* dst = p.gl + ((size_t)c * HV + h) * 128 + tid * 8;
            *reinterpret_cast<float4*>(dst) = make_float4(ex2f_(gLv[0]), ex2f_(gLv[1]), ex2f_(gLv[2]), ex2f_(gLv[3]));
            *reinterpret_cast<float4*>(dst + 4) = make_float4(ex2f_(gLv[4]), ex2f_(gLv[5]), ex2f_(gLv[6]), ex2f_(gLv[7]));
        }
    }
    umma::fence_async_smem();
    __syncthreads();
    if (tid == 0) {
        const size_t it = (size_t)c * HV + h;
        umma::bulk_store(reinterpret_cast<uint8_t*>(p.kbar) + it * umma::CHUNK_TILE_BYTES, sKB, umma::CHUNK_TILE_BYTES);
        umma::bulk_store(reinterpret_cast<uint8_t*>(p.qs) + it * umma::CHUNK_TILE_BYTES, sQS, umma::CHUNK_TILE_BYTES);
    }
    umma::mbar_wait(&sh.bar, 0);
    umma::fence_after_sync();
    // phase-3 operands over the dead phase-1 tiles: beta k 2^g and beta v (rows past the end are zero)
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
        const float b = sh.beta[r];          // 0 for rows past the end
        float t8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = b * vk[n][e] * ex2f_(vg[n][e]);
        store_split8(sBk, sBk + 16384, 64, r, k8, t8);
        unpack8<DT>(wv[n], t8);
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] *= b;
        store_split8(sBv, sBv + 16384, 64, r, k8, t8);
    }
    if (tid == 0) umma::bulk_store_wait_read();    // the two tiles under sM / sInv / sP (and the q rows) have left shared memory
    __syncthreads();
    if (item + stride < total) load_inputs(item + stride);     // k, q, g, beta of the next item start travelling
    for (int i = tid; i < CH * MLD / 4; i += 512) reinterpret_cast<float4*>(sInv)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (SCALAR) {                             // lane = row (K rows, then Q rows), cg = 16 columns j: decay applied here, for i >= j only
        float v[16];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 16 * cg), v);
        const int i = row & 63;
        const float gi = sGs[i], bi = sh.beta[i];
        float* dst = (q < 2 ? sM : sP) + i * MLD + 16 * cg;
#pragma unroll
        for (int j4 = 0; j4 < 16; j4 += 4) {
            float o4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = 16 * cg + j4 + e;
                const float E = ex2f_(fminf(gi - sGs[j], 0.f));
                if (q < 2) o4[e] = j < i ? bi * v[j4 + e] * E : (j == i ? 1.f : 0.f);
                else o4[e] = j <= i ? p.scale * v[j4 + e] * E : 0.f;
            }
            *reinterpret_cast<float4*>(dst + j4) = make_float4(o4[0], o4[1], o4[2], o4[3]);
        }
    } else {                                  // warp quadrant = row block I (lanes: 16 rows of Gamma, then 16 rows of Q K^T), cg = 16 columns j
        const int I = q, i = 16 * I + (lane & 15);
        const bool isq = lane >= 16;
        float v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = 0.f;
        if (cg <= I) umma::tmem_ld16(umma::tmem_addr(tmem, warp, kc_row(I) + 16 * cg), v);      // warp-uniform condition
        const float bi = sh.beta[i];
        float* dst = (isq ? sP : sM) + i * MLD + 16 * cg;
#pragma unroll
        for (int j4 = 0; j4 < 16; j4 += 4) {
            float o4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = 16 * cg + j4 + e;
                if (isq) o4[e] = j <= i ? p.scale * v[j4 + e] : 0.f;
                else o4[e] = j < i ? bi * v[j4 + e] : (j == i ? 1.f : 0.f);
            }
            *reinterpret_cast<float4*>(dst + j4) = make_float4(o4[0], o4[1], o4[2], o4[3]);
        }
    }
    __syncthreads();
    invert_unit_lower(sM, sInv, sh);
    {   // A as the B operand of phase 3; A and Aqk also leave as ready-made [row][column] operand tiles (rows past the end:
        // identity rows of A, zero rows of Aqk)
        const int r = tid >> 3, k8 = tid & 7;
        float a8[8], q8[8];
        lds8(sInv + r * MLD + k8 * 8, a8);
        lds8(sP + r * MLD + k8 * 8, q8);
        store_split8(sTA, sTA + 8192, 64, r, k8, a8);
        store_split8(sTQ, sTQ + 8192, 64, r, k8, q8);
    }
    publish();
    if (tid == 0) {
        const size_t it = (size_t)c * HV + h;
        umma::bulk_store(reinterpret_cast<uint8_t*>(p.A) + it * umma::QUARTER_TILE_BYTES, sTA, umma::QUARTER_TILE_BYTES);
        umma::bulk_store(reinterpret_cast<uint8_t*>(p.Aqk) + it * umma::QUARTER_TILE_BYTES, sTQ, umma::QUARTER_TILE_BYTES);
    }
    if (umma::mma_issuer()) {
        const umma::Opnd bA = umma::opnd_k(sTA, sTA + 8192, 64);
        umma::gemm(tmem + 128, umma::opnd_mn(sBk, sBk + 16384, 64), bA, 128, 64, 64, 0u);
        umma::gemm(tmem + 192, umma::opnd_mn(sBv, sBv + 16384, 64), bA, 128, 64, 64, 0u);
        umma::commit(&sh.bar);
    }
    umma::mbar_wait(&sh.bar, 1);
    umma::fence_after_sync();
    {   // nw^T [K index][tok] leaves as a ready-made chunk tile (the serial kernels fetch it with one bulk copy; token
        // columns past the end are exact zeros: beta is 0 there)
        float a[16], n0[8], n1[8];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 128 + 16 * cg), a);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (j < 8) n0[j] = -a[j]; else n1[j - 8] = -a[j];
        }
        store_split8(base, base + 16384, 128, row, 2 * cg, n0);          // every operand tile is dead by now
        store_split8(base, base + 16384, 128, row, 2 * cg + 1, n1);
    }
    umma::fence_async_smem();
    __syncthreads();
    if (tid == 0) umma::bulk_store(reinterpret_cast<uint8_t*>(p.nw) + ((size_t)c * HV + h) * umma::CHUNK_TILE_BYTES, base, umma::CHUNK_TILE_BYTES);
    {   // u^T [v][tok] leaves the same way (token columns past the end are exact zeros: A has identity rows there and
        // beta v zero rows), built next to the nw tile while that one is being copied
        float b[16], u0[8], u1[8];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 192 + 16 * cg), b);
#pragma unroll
        for (int j = 0; j < 8; ++j) { u0[j] = b[j]; u1[j] = b[8 + j]; }
        store_split8(base + 32768, base + 32768 + 16384, 128, row, 2 * cg, u0);
        store_split8(base + 32768, base + 32768 + 16384, 128, row, 2 * cg + 1, u1);
    }
    umma::fence_async_smem();
    __syncthreads();
    if (tid == 0) umma::bulk_store(reinterpret_cast<uint8_t*>(p.u) + ((size_t)c * HV + h) * umma::CHUNK_TILE_BYTES, base + 32768, umma::CHUNK_TILE_BYTES);
    }   // items
    if (tid == 0) umma::bulk_store_wait_read();
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------------------
// bwd_chunk: every gradient that is local to a (chunk, v-head) once the state gradients are known, in one CTA.
//
// WY part.  With S the state entering the chunk, k~ = k 2^g, Ab = A diag(beta):
//   X = V - k~ S        Vd = Ab X (saved by the forward pass)        dAqk = lower(dO Vd^T)
//   dW = A^T dVd        dX = diag(beta) dW (= dV)       dbeta_w = rowsum(dW * X)
//   dA = (dVd X^T) diag(beta)          dL = -strictlower(A^T dA A^T)
// State part.  With dS' the state gradient leaving the chunk, up = 2^g, rest = 2^(g_L - g):
//   dq~ = scale dO S^T     dk~ = -dX S^T     dkbar = Vd dS'^T     dgl = rowsum_v(S * dS')
//   dq_p = dq~ up          dk_p = dk~ up + dkbar rest
//   dg_p = q~ dq~ + k~ dk~ - kbar dkbar;   last valid row += colsum(kbar dkbar) + gl dgl
// Intra-chunk part.  With E_ij = 2^(g_i - g_j) per channel (i > j), Wq = scale strictlower(dAqk), dLs = strictlower(dL):
//   dq_row_i = sum_j Wq_ij k_j E_ij                     T_i = sum_j dLs_ij k_j E_ij
//   dk_col_j = sum_i (Wq_ij q_i + beta_i dLs_ij k_i) E_ij
//   dq = dq_p + dq_row + scale dAqk_ii k       dk = dk_p + beta T + dk_col + scale dAqk_ii q
//   dg' = dg_p + q dq_row + k beta T - k dk_col           dbeta = dbeta_w + sum_c k T
// E_ij is factored through the anchor a of i's 16-row block exactly as in the forward kernel.  Channels go on M.  Per row
// block I (anchor a = 16 I):
//   row terms   R_I^T[c][r]  = sum_j Kc_I[j][c] W[16 I + r][j]       W = Wq (-> dq_row) or dLs (-> T); N = 16 each
//   col terms   C_I^T[c][j]  = sum_{i in I} Qr[i][c] Wq[i][j] + Kr[i][c] (beta dLs)[i][j]      N = 16 (I + 1)
// then per thread (channel c, row block cg): dq_row = R 2^(g_i - g_a), T likewise, dk_col[j] = sum_{I >= cg} C_I 2^(g_aI - g_j).
//
// Every tile operand arrives by bulk copy: S and dS' (state tiles), Vd^T (the forward pass's chunk tile), A (quarter tile),
// dO (row tile) and dVd^T (chunk tile) as written by the reverse state chain.  Only k, q, g and v pass through registers.
// Products (M = 128 throughout; a 64-row operand on M leaves lanes 64..127 of its accumulator undefined and unread), in
// issue order:
//   P7  Db^T[c x tok]  = dS' Vd^T        P6a Dq^T[c x tok] = S dO^T        P3a D1[i x j] = dO Vd^T      (dgl meanwhile)
//   P1  X^T[v x tok]   = V^T - S^T k~^T  P2  dW^T[v x j] = dVd^T A         (k~ and dVd^T take the place of dS')
//   P3b D2[64 + i][j]  = dVd X^T (operand shifted so that the result lands in lanes 64..127: both halves of the CTA read
//                        their accumulators at the same time)              P6b Dk^T[c x tok] = S dX^T
//   P4  Y[a x j]       = (D2 diag(beta)) A^T             P5  Z[i x j] = A^T Y         dL = -strictlower(Z)
//   then the row / column products of the intra-chunk part, whose operands are rebuilt over the dead tiles while P4 and
//   P5 run.
// dX, dAqk, dL and dbeta_w never leave the SM.  The three outputs per token and channel leave as fp32 [64 tokens][128]
// tiles per (chunk, v-head), written from registers (128 consecutive bytes per warp and token).
//
// Shared memory (U = 32 KB): S [0, 2U) | dS' [2U, 4U) -> k~ -> X^T [2U, 3U), dVd^T [3U, 4U) | dO -> dX^T [4U, 5U) |
// A -> beta dLs [5U, 5U + 16K) | Vd^T -> dv rows -> (D2 beta | Y) -> [Wq; dLs] [5U + 16K, 6U + 16K); the intra-chunk operands (column
// tiles, [Kr; Qr]) go to [0, 4.5U).
// TMEM columns: X -> Y 0, dW -> Z 64, D1 128, Dq 192, D2 256, Dk 320, Db 384; later R_I 32 I, C_I {304, 448, 256, 128}.
// ---------------------------------------------------------------------------------------------------------
constexpr int BU = 32768;
constexpr int BC_T = 2 * BU, BC_D = 3 * BU, BC_O = 4 * BU, BC_A = 5 * BU, BC_V = 5 * BU + 16384;
constexpr int BWD_CHUNK_SMEM = 6 * BU + 16384 + 1024;
static_assert(KQ_OFF + 65536 <= BC_A, "the intra-chunk operands must end below the weight tiles");
// A 64-row (or 64-column) operand issued with M = 128 makes the tensor core read the 8 or 16 KB that follow its tile: A
// lies in front of the last region, not at the end, so that every such read stays inside the allocation.
__host__ __device__ constexpr int ccol_off(int I) { return I == 0 ? 304 : I == 1 ? 448 : I == 2 ? 256 : 128; }

struct BwdShared {
    uint64_t barA, barB, barC, barD, ld0, ld1, ld2;
    uint32_t tmem;
    float beta[CH];
};

// the intra-chunk operands of rows `n` (this thread's n-th (row, 8-channel) pair): [Kr; Qr] and the column tiles; with a
// scalar gate just the stacked [K; Q] tile (rows 0..63 = k, 64..127 = q), the decay goes into the weights instead
// fire-and-forget fp32 addition in global memory
__device__ __forceinline__ void red_add(float* addr, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" :: "l"(addr), "f"(v) : "memory");
}

template <bool SCALAR>
__device__ __forceinline__ void stage_intra_operands(uint8_t* base, const float (*sGa)[DK], int tid, int n, const float (&vk)[8],
                                                     const float (&vq)[8], const float (&vg)[8]) {
    uint8_t* sKQ = base + KQ_OFF;
    const int i = tid + n * 512, r = i >> 4, k8 = i & 15, I0 = r >> 4;
    if (SCALAR) {
        store_split8(sKQ, sKQ + 32768, 128, r, k8, vk);
        store_split8(sKQ, sKQ + 32768, 128, 64 + r, k8, vq);
        return;
    }
    float ga[8], t8[8];
    lds8(&sGa[I0][k8 * 8], ga);
#pragma unroll
    for (int e = 0; e < 8; ++e) t8[e] = vk[e] * ex2f_(vg[e] - ga[e]);
    store_split8(sKQ, sKQ + 32768, 128, 32 * I0 + (r & 15), k8, t8);
#pragma unroll
    for (int e = 0; e < 8; ++e) t8[e] = vq[e] * ex2f_(vg[e] - ga[e]);
    store_split8(sKQ, sKQ + 32768, 128, 32 * I0 + 16 + (r & 15), k8, t8);
#pragma unroll
    for (int I = 0; I < 4; ++I) {
        if (I < I0) continue;
        if (I > I0) lds8(&sGa[I][k8 * 8], ga);
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = vk[e] * ex2f_(ga[e] - vg[e]);
        store_split8(base + kc_off(I), base + kc_off(I) + kc_bytes(I), 16 * (I + 1), r, k8, t8);
    }
}

// CTAs are persistent: one per SM walks the items gridDim.x apart.  The epilogue of an item touches no tile in shared
// memory (it reads accumulators and global memory and writes global memory), so all five tiles of the next item travel
// while it runs.  (Output tiles staged in shared memory and sent by bulk copy kept the S and dO regions busy until the very
// end of the item, and the next item then began by waiting for 96 KB.)  One elected lane of warp 0 issues every
// tensor-core product and the tile loads.  (A 17th, issue-only warp was tried: five warps on one SM sub-partition cap the
// kernel at 96 registers per thread and the spills cost far more than the overlap returns.)
constexpr int BWD_CHUNK_THREADS = 512;

// SCALAR (one decay per token): the intra-chunk part contracts the plain k / q rows with weights that already carry
// E_ij = 2^(g_i - g_j) (i > j, never a positive exponent):  [dq_row | T]^T = K^T [Wq E; dLs E]^T (N = 128),
// dk_col^T = Q^T (Wq E) + K^T (beta dLs E); no anchors, and any g <= 0 is in range.  TMEM: [dq_row | T] 0, dk_col 128.
template <int DT, bool SCALAR>
__global__ void __launch_bounds__(BWD_CHUNK_THREADS, 1) bwd_chunk_tc_kernel(const MkdaBwdChunk p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ BwdShared sh;
    __shared__ float sDiag[CH], sDbw[CH];
    __shared__ float sRed[4][CH];
    __shared__ float sRedW[2][CH];
    __shared__ float sDgl[DK];
    __shared__ float sCol[4][DK];
    __shared__ float sRk[CH], sRq[CH];                 // L2-norm scales of the chunk's rows (0 past the end)
    __shared__ __align__(16) float sPart[16][DK];
    __shared__ __align__(16) float sGa[4][DK];         // cumsum rows of the four block anchors
    __shared__ float sGs[CH];                          // SCALAR: the cumsum of every row (rows past the end: the last valid one)
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sS = base;                                // S^T [v][K index] state tile (hi, lo)
    uint8_t* sT = base + BC_T;                         // dS'^T state tile; later:
    uint8_t* sK = sT;                                  //   k~ [tok][K index] -> X^T [v][tok]
    uint8_t* sD = base + BC_D;                         //   dVd^T [v][tok]
    uint8_t* sO = base + BC_O;                         // dO [tok][v] -> dX^T [v][tok]
    uint8_t* sV = base + BC_V;                         // Vd^T [v][tok] -> dv rows -> D2 diag(beta) [a][b] | Y [a][j] -> [Wq; dLs]
    uint8_t* sA = base + BC_A;                         // A [i][j] -> diag(beta) strictlower(dL) [i][j]
    uint8_t* sDA = sV;
    uint8_t* sY = sV + 16384;
    uint8_t* sKQ = base + KQ_OFF;
    uint8_t* sWD = sV;                                 // rows 32 I + r = scale strictlower(dAqk)[16 I + r], rows 32 I + 16 + r = strictlower(dL)[16 I + r]
    uint8_t* sBd = sA;

    const int HV = p.L.HV, HK = p.L.HK;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, cg = warp >> 2, row = q * 32 + lane;
    const int stride = gridDim.x;

    auto fetch_early = [&](size_t it) {                // dS', Vd^T, A: their regions are free once the intra-chunk products are done
        umma::mbar_expect_tx(&sh.ld0, umma::STATE_TILE_BYTES + umma::CHUNK_TILE_BYTES + umma::QUARTER_TILE_BYTES);
        umma::bulk_load(sT, reinterpret_cast<const uint8_t*>(p.dh) + it * umma::STATE_TILE_BYTES, umma::STATE_TILE_BYTES, &sh.ld0);
        umma::bulk_load(sV, reinterpret_cast<const uint8_t*>(p.Vd) + it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ld0);
        umma::bulk_load(sA, reinterpret_cast<const uint8_t*>(p.A) + it * umma::QUARTER_TILE_BYTES, umma::QUARTER_TILE_BYTES, &sh.ld0);
    };
    auto fetch_late = [&](size_t it) {                 // S, dO
        umma::mbar_expect_tx(&sh.ld2, umma::STATE_TILE_BYTES + umma::CHUNK_TILE_BYTES);
        umma::bulk_load(sS, reinterpret_cast<const uint8_t*>(p.h) + it * umma::STATE_TILE_BYTES, umma::STATE_TILE_BYTES, &sh.ld2);
        umma::bulk_load(sO, reinterpret_cast<const uint8_t*>(p.dO_t) + it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ld2);
    };

    if (warp == 0) umma::tmem_alloc(&sh.tmem, 512);
    if (tid == 0) {
        umma::mbar_init(&sh.barA, 1); umma::mbar_init(&sh.barB, 1); umma::mbar_init(&sh.barC, 1); umma::mbar_init(&sh.barD, 1);
        umma::mbar_init(&sh.ld0, 1); umma::mbar_init(&sh.ld1, 1); umma::mbar_init(&sh.ld2, 1);
        umma::fence_barrier_init();
    }
    publish();
    const uint32_t tmem = sh.tmem;
    if (tid == 0 && (int)blockIdx.x < p.L.NC * HK) {       // the first item of this CTA: group blockIdx.x, its first v-head
        const size_t it0 = (size_t)(blockIdx.x / HK) * HV + (size_t)(blockIdx.x % HK) * (HV / HK);
        fetch_early(it0);
        fetch_late(it0);
    }
    // phase counters of the barriers (every thread walks the same sequence of phases)
    uint32_t nA = 0, nB = 0, nC = 0, nD = 0, n0 = 0, n1 = 0, n2 = 0;
    // A CTA walks (chunk, q/k head) groups gridDim.x apart (heads fastest: CTAs that run together read neighbouring
    // memory) and, inside a group, the G = HV / HK v-heads that share the q/k head one after the other.  Their dq and dk
    // contributions are summed where they are written: the first v-head of a group stores its fp32 tile, the others add to it
    // (red.global.add.f32 by the same thread to the same address, in the fixed order of the v-heads: deterministic, and
    // the same association as a separate sum would use).  The tile lives in L2 between the two passes.
    const int G = HV / HK, ngroups = p.L.NC * HK;
    // the chunk table entries are read one item ahead: every address of an item depends on them
    int next_start = 0, next_len = 1;
    if ((int)blockIdx.x < ngroups) { next_start = p.L.chunk_start[blockIdx.x / HK]; next_len = p.L.chunk_len[blockIdx.x / HK]; }

    for (int grp = blockIdx.x, j = 0; grp < ngroups; ) {
        const int c = grp / HK, hk = grp - c * HK, h = hk * G + j;
        const int item = c * HV + h;
        const int start = next_start, len = next_len;
        // the item after this one: the next v-head of the group, else the first v-head of this CTA's next group
        const bool last_of_group = j + 1 == G;
        const bool more = !last_of_group || grp + stride < ngroups;
        if (last_of_group && more) { next_start = p.L.chunk_start[(grp + stride) / HK]; next_len = p.L.chunk_len[(grp + stride) / HK]; }

        // ---- state products whose operands are all copies | register loads, dgl ------------------------
        if (umma::mma_issuer()) {
            umma::mbar_wait(&sh.ld0, n0 & 1);
            umma::fence_after_sync();
            umma::gemm(tmem + 384, umma::opnd_mn(sT, sT + BU, 128), umma::opnd_mn(sV, sV + 16384, 128), 128, 64, 128, 0u);   // P7
            umma::commit(&sh.barC);
            umma::mbar_wait(&sh.ld2, n2 & 1);
            umma::gemm(tmem + 192, umma::opnd_mn(sS, sS + BU, 128), umma::opnd_k(sO, sO + 16384, 64), 128, 64, 128, 0u);     // P6a
            umma::gemm(tmem + 128, umma::opnd_k(sO, sO + 16384, 64), umma::opnd_mn(sV, sV + 16384, 128), 128, 64, 128, 0u);  // P3a
            umma::commit(&sh.barD);
        }
        float vk[2][8], vg[2][8], vq[2][8], vv[16];
        Raw8 wk[2], wq[2];                                 // k, q and v stay raw until their first use: no thread waits for them where they are requested
        uint32_t wv[16];
        {
            // k, g and this thread's column of v are requested now and used once the first products are under way
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
                ldraw8<DT>(p.k, ((size_t)(start + rr) * HK + hk) * 128 + k8 * 8, wk[n]);
                ldg8(p.g_c, MKDA_F32, ((size_t)(start + rr) * HV + h) * 128 + k8 * 8, vg[n]);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int t = cg * 16 + j, tt = t < len ? t : len - 1;
                wv[j] = ldraw1<DT>(p.v, ((size_t)(start + tt) * HV + h) * 128 + row);
            }
            // beta and the L2 statistics of the rows: requested now, parked in shared memory after the dgl sums (a value
            // stored at once would be waited for here)
            float small0 = 0.f, small1 = 0.f;
            if (tid < CH) small0 = tid < len ? p.beta[(size_t)(start + tid) * HV + h] : 0.f;
            if (tid >= CH && tid < 2 * CH) {
                const int r = tid - CH;
                const size_t tk = (size_t)(start + (r < len ? r : len - 1)) * HK + hk;
                small0 = r < len ? (p.k_rstd ? p.k_rstd[tk] : 1.f) : 0.f;
                small1 = r < len ? (p.q_rstd ? p.q_rstd[tk] : 1.f) : 0.f;
            }
            // dgl[c] = sum_v S[c][v] dS'[c][v] from the two tiles: chunk (v row, 8 channels) per thread, four rows each
            umma::mbar_wait(&sh.ld0, n0 & 1);
            umma::mbar_wait(&sh.ld2, n2 & 1);
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const int i = tid + n * 512;
                const uint32_t off = umma::tile_chunk_offset(128, i >> 4, i & 15);
                const uint4 a4 = *reinterpret_cast<const uint4*>(sS + off), b4 = *reinterpret_cast<const uint4*>(sS + BU + off);
                const uint4 c4 = *reinterpret_cast<const uint4*>(sT + off), d4 = *reinterpret_cast<const uint4*>(sT + BU + off);
                const uint32_t ah[4] = {a4.x, a4.y, a4.z, a4.w}, al[4] = {b4.x, b4.y, b4.z, b4.w};
                const uint32_t dh[4] = {c4.x, c4.y, c4.z, c4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float s0 = __uint_as_float(ah[e] << 16) + __uint_as_float(al[e] << 16);
                    const float s1 = __uint_as_float(ah[e] & 0xffff0000u) + __uint_as_float(al[e] & 0xffff0000u);
                    const float d0 = __uint_as_float(dh[e] << 16) + __uint_as_float(dl[e] << 16);
                    const float d1 = __uint_as_float(dh[e] & 0xffff0000u) + __uint_as_float(dl[e] & 0xffff0000u);
                    acc[2 * e] = fmaf(s0, d0, acc[2 * e]);
                    acc[2 * e + 1] = fmaf(s1, d1, acc[2 * e + 1]);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 16);
            if (lane < 16) {
                *reinterpret_cast<float4*>(&sPart[warp][lane * 8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(&sPart[warp][lane * 8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) vv[j] = cg * 16 + j < len ? unpack1<DT>(wv[j]) : 0.f;
            if (tid < CH) sh.beta[tid] = small0;
            if (tid >= CH && tid < 2 * CH) { sRk[tid - CH] = small0; sRq[tid - CH] = small1; }
        }
        ++n0; ++n2;
        umma::mbar_wait(&sh.barC, nC & 1); ++nC;           // dS' Vd^T done
        umma::fence_after_sync();
        __syncthreads();                                   // ... and every thread has read its part of dS': the tile is dead
        if (tid == 0) {                                        // its second half receives dVd^T, its first half k~
            umma::mbar_expect_tx(&sh.ld1, umma::CHUNK_TILE_BYTES);
            umma::bulk_load(sD, reinterpret_cast<const uint8_t*>(p.dVd_t) + (size_t)item * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ld1);
        }
        {
            if (tid < DK) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < 16; ++w) t += sPart[w][tid];
                sDgl[tid] = t;
            }
            // scale k by its L2 statistics (rows past the end become zero); park the anchor rows of g; k~ = k 2^g
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
                const float rk = sRk[r];
                float t8[8];
                unpack8<DT>(wk[n], vk[n]);
#pragma unroll
                for (int e = 0; e < 8; ++e) { vk[n][e] *= rk; t8[e] = vk[n][e] * ex2f_(vg[n][e]); }
                store_split8(sK, sK + 16384, 64, r, k8, t8);
                if ((r & 15) == 0) {
                    *reinterpret_cast<float4*>(&sGa[r >> 4][k8 * 8]) = make_float4(vg[n][0], vg[n][1], vg[n][2], vg[n][3]);
                    *reinterpret_cast<float4*>(&sGa[r >> 4][k8 * 8 + 4]) = make_float4(vg[n][4], vg[n][5], vg[n][6], vg[n][7]);
                }
                if (SCALAR && k8 == 0) sGs[r] = vg[n][0];
            }
        }
        publish();
        if (umma::mma_issuer()) {
            umma::gemm(tmem + 0, umma::opnd_k(sS, sS + BU, 128), umma::opnd_k(sK, sK + 16384, 64), 128, 64, 128, 0u);        // P1
            umma::commit(&sh.barA);
            umma::mbar_wait(&sh.ld1, n1 & 1);
            umma::gemm(tmem + 64, umma::opnd_k(sD, sD + 16384, 128), umma::opnd_mn(sA, sA + 8192, 64), 128, 64, 64, 0u);     // P2
            umma::commit(&sh.barB);
        }
        ++n1;
        {
            // q for the intra-chunk operands is requested while the products run
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
                ldraw8<DT>(p.q, ((size_t)(start + rr) * HK + hk) * 128 + k8 * 8, wq[n]);
            }
            umma::mbar_wait(&sh.barA, nA & 1);
            umma::fence_after_sync();
            float d[16], x0[8], x1[8];
            umma::tmem_ld16(umma::tmem_addr(tmem, warp, cg * 16), d);
#pragma unroll
            for (int j = 0; j < 8; ++j) { x0[j] = vv[j] - d[j]; x1[j] = vv[8 + j] - d[8 + j]; }
            store_split8(sK, sK + 16384, 128, row, 2 * cg, x0);            // k~ is dead: the region now holds X^T
            store_split8(sK, sK + 16384, 128, row, 2 * cg + 1, x1);
            umma::mbar_wait(&sh.barB, nB & 1);
            umma::mbar_wait(&sh.barD, nD & 1);                             // P6a and P3a done long ago: the dO and Vd^T tiles are dead
            umma::fence_after_sync();
            float dw[16];
            umma::tmem_ld16(umma::tmem_addr(tmem, warp, 64 + cg * 16), dw);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                dw[j] *= sh.beta[cg * 16 + j];                             // dX = diag(beta) dW; beta is 0 past the end
                // dv rows are staged [tok][v] in the dtype of v over the dead Vd^T tile and leave with 16-byte stores below
                if (DT == MKDA_F32) reinterpret_cast<float*>(sV)[(cg * 16 + j) * 128 + row] = dw[j];
                else if (DT == MKDA_BF16) reinterpret_cast<__nv_bfloat16*>(sV)[(cg * 16 + j) * 128 + row] = __float2bfloat16_rn(dw[j]);
                else reinterpret_cast<__half*>(sV)[(cg * 16 + j) * 128 + row] = __float2half_rn(dw[j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) { x0[j] = dw[j]; x1[j] = dw[8 + j]; }
            store_split8(sO, sO + 16384, 128, row, 2 * cg, x0);
            store_split8(sO, sO + 16384, 128, row, 2 * cg + 1, x1);
        }
        ++nA; ++nB; ++nD;
        publish();
        if (umma::mma_issuer()) {
            umma::Opnd aD = umma::opnd_mn(sD, sD + 16384, 128);            // (m = token, k = v) of the dVd^T tile, moved one 64-group up:
            aD.hi -= 16384; aD.lo -= 16384;                                // rows 0..63 of the operand read the 16 KB in front of each half
            umma::gemm(tmem + 256, aD, umma::opnd_mn(sK, sK + 16384, 128), 128, 64, 128, 0u);                                // P3b
            umma::commit(&sh.barA);
            umma::gemm(tmem + 320, umma::opnd_mn(sS, sS + BU, 128), umma::opnd_mn(sO, sO + 16384, 128), 128, 64, 128, 0u);   // P6b
            umma::commit(&sh.barB);
        }
        {
            // dv: 64 rows of 128 values
            constexpr int ROWB = DT == MKDA_F32 ? 512 : 256;               // bytes per row
            constexpr int PER = ROWB / 16;                                 // 16-byte pieces per row
#pragma unroll
            for (int n = 0; n < 64 * PER / 512; ++n) {
                const int i = tid + n * 512, r = i / PER, pc = i % PER;
                if (r < len) {
                    const uint4 val = *reinterpret_cast<const uint4*>(sV + r * ROWB + pc * 16);
                    *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.dv) + ((size_t)(start + r) * HV + h) * ROWB + pc * 16) = val;
                }
            }
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const float rq = sRq[(tid + n * 512) >> 4];
                unpack8<DT>(wq[n], vq[n]);
#pragma unroll
                for (int e = 0; e < 8; ++e) vq[n][e] *= rq;
            }
        }
        __syncthreads();                                   // the dv rows have left shared memory
        umma::mbar_wait(&sh.barA, nA & 1); ++nA;
        umma::mbar_wait(&sh.barB, nB & 1); ++nB;           // every state-phase tile except A is dead now
        umma::fence_after_sync();
        if (q >= 2) {                           // rows i = row - 64 of D2 = dVd X^T: dbeta_w partials and D2 diag(beta)
            const int i = row - 64;
            float d[16], a0[8], a1[8];
            umma::tmem_ld16(umma::tmem_addr(tmem, warp, 256 + cg * 16), d);
            umma::load_tile8(sA, sA + 8192, 64, i, 2 * cg, a0);
            umma::load_tile8(sA, sA + 8192, 64, i, 2 * cg + 1, a1);
            float pr[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                pr[j] = d[j] * (j < 8 ? a0[j] : a1[j - 8]);
                const float da = d[j] * sh.beta[cg * 16 + j];
                if (j < 8) a0[j] = da; else a1[j - 8] = da;
            }
            // sums over the 32 lanes for the 16 columns at once: every exchange halves the number of columns a lane carries
            // (16 shuffles instead of 80); the lane whose bits 4..1 spell the column ends up with its sum
#pragma unroll
            for (int w = 8, bit = 16; w >= 1; w >>= 1, bit >>= 1) {
#pragma unroll
                for (int j = 0; j < w; ++j) {
                    const float recv = __shfl_xor_sync(0xffffffffu, (lane & bit) ? pr[j] : pr[j + w], bit);
                    pr[j] = ((lane & bit) ? pr[j + w] : pr[j]) + recv;
                }
            }
            pr[0] += __shfl_xor_sync(0xffffffffu, pr[0], 1);
            if ((lane & 1) == 0) sRedW[q - 2][cg * 16 + ((lane >> 1) & 15)] = pr[0];
            store_split8(sDA, sDA + 8192, 64, i, 2 * cg, a0);
            store_split8(sDA, sDA + 8192, 64, i, 2 * cg + 1, a1);
        }
        publish();
        if (umma::mma_issuer()) {
            umma::gemm(tmem + 0, umma::opnd_k(sDA, sDA + 8192, 64), umma::opnd_k(sA, sA + 8192, 64), 128, 64, 64, 0u);        // P4
            umma::commit(&sh.barA);
        }
        {
            if (tid < CH) sDbw[tid] = sRedW[0][tid] + sRedW[1][tid];
            stage_intra_operands<SCALAR>(base, sGa, tid, 0, vk[0], vq[0], vg[0]);     // over the dead S / X^T / dVd^T / dX^T tiles, while P4 runs
            umma::mbar_wait(&sh.barA, nA & 1);
            umma::fence_after_sync();
            if (q < 2) {
                float y[16], a0[8], a1[8];
                umma::tmem_ld16(umma::tmem_addr(tmem, warp, cg * 16), y);
#pragma unroll
                for (int j = 0; j < 8; ++j) { a0[j] = y[j]; a1[j] = y[8 + j]; }
                store_split8(sY, sY + 8192, 64, row, 2 * cg, a0);
                store_split8(sY, sY + 8192, 64, row, 2 * cg + 1, a1);
            }
        }
        ++nA;
        publish();
        if (umma::mma_issuer()) {
            umma::gemm(tmem + 64, umma::opnd_mn(sA, sA + 8192, 64), umma::opnd_mn(sY, sY + 8192, 64), 128, 64, 64, 0u);       // P5
            umma::commit(&sh.barA);
        }
        {
            stage_intra_operands<SCALAR>(base, sGa, tid, 1, vk[1], vq[1], vg[1]);     // the other half, while P5 runs
            umma::mbar_wait(&sh.barA, nA & 1);                 // Z done: A, D2 diag(beta) and Y are dead
            umma::fence_after_sync();
            if (q < 2) {                                       // rows i = row of D1 = dO Vd^T and Z: the weights of the intra-chunk part
                const int i = row;
                const float bt = sh.beta[i];
                float d[16], z[16];
                umma::tmem_ld16(umma::tmem_addr(tmem, warp, 128 + cg * 16), d);
                umma::tmem_ld16(umma::tmem_addr(tmem, warp, 64 + cg * 16), z);
                const float gi = SCALAR ? sGs[i] : 0.f;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    float w8[8], d8[8], b8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int j = cg * 16 + hf * 8 + e;
                        const bool lo = j < i && i < len;
                        const float E = SCALAR ? ex2f_(fminf(gi - sGs[j], 0.f)) : 1.f;
                        w8[e] = lo ? p.scale * d[hf * 8 + e] * E : 0.f;
                        d8[e] = lo ? -z[hf * 8 + e] * E : 0.f;
                        b8[e] = bt * d8[e];
                        if (j == i) sDiag[i] = i < len ? p.scale * d[hf * 8 + e] : 0.f;
                    }
                    if (SCALAR) {      // [Wq E; dLs E] stacked by rows
                        store_split8(sWD, sWD + 16384, 128, i, 2 * cg + hf, w8);
                        store_split8(sWD, sWD + 16384, 128, 64 + i, 2 * cg + hf, d8);
                    } else {
                        store_split8(sWD, sWD + 16384, 128, 32 * (i >> 4) + (i & 15), 2 * cg + hf, w8);
                        store_split8(sWD, sWD + 16384, 128, 32 * (i >> 4) + 16 + (i & 15), 2 * cg + hf, d8);
                    }
                    store_split8(sBd, sBd + 8192, 64, i, 2 * cg + hf, b8);
                }
            }
        }
        ++nA;
        publish();
        if (umma::mma_issuer()) {
            if (SCALAR) {
                umma::gemm(tmem + 0, umma::opnd_mn(sKQ, sKQ + 32768, 128, 0), umma::opnd_k(sWD, sWD + 16384, 128), 128, 128, 64, 0u);
                umma::gemm(tmem + 128, umma::opnd_mn(sKQ, sKQ + 32768, 128, 64), umma::opnd_mn(sWD, sWD + 16384, 128, 0), 128, 64, 64, 0u);
                umma::gemm(tmem + 128, umma::opnd_mn(sKQ, sKQ + 32768, 128, 0), umma::opnd_mn(sBd, sBd + 8192, 64, 0), 128, 64, 64, 1u);
            } else {
#pragma unroll
                for (int I = 0; I < 4; ++I) {
                    const int nj = 16 * (I + 1);
                    const umma::Opnd aKc = umma::opnd_mn(base + kc_off(I), base + kc_off(I) + kc_bytes(I), nj);
                    // both row terms (dq_row | T) of the block in one N = 32 product
                    umma::gemm(tmem + 32 * I, aKc, umma::opnd_k(sWD, sWD + 16384, 128, 32 * I), 128, 32, nj, 0u);
                    umma::gemm(tmem + ccol_off(I), umma::opnd_mn(sKQ, sKQ + 32768, 128, 32 * I + 16), umma::opnd_mn(sWD, sWD + 16384, 128, 32 * I),
                               128, nj, 16, 0u);
                    umma::gemm(tmem + ccol_off(I), umma::opnd_mn(sKQ, sKQ + 32768, 128, 32 * I), umma::opnd_mn(sBd, sBd + 8192, 64, 16 * I),
                               128, nj, 16, 1u);
                }
            }
            umma::commit(&sh.barA);
            if (more) {                                        // every operand tile is dead once these products are done (the epilogue
                umma::mbar_wait(&sh.barA, nA & 1);             // reads accumulators and writes global memory): all five tiles of the
                size_t next_item = (size_t)item + 1;           // next item travel under it
                if (last_of_group) {
                    const int ng = grp + stride, nc = ng / HK;
                    next_item = (size_t)nc * HV + (size_t)(ng - nc * HK) * G;
                }
                fetch_early(next_item);
                fetch_late(next_item);
            }
        }
        {
            // epilogue inputs for (channel `row`, rows 16 cg .. 16 cg + 15) are fetched while the products run
            float kq[16], qq[16], gg[16], ga[4];
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const int i = 16 * cg + r, ii = i < len ? i : len - 1;
                const size_t tk = (size_t)(start + ii) * HK + hk;
                kq[r] = ld1(p.k, DT, tk * 128 + row) * (i < len ? sRk[i] : sRk[len - 1]);
                qq[r] = ld1(p.q, DT, tk * 128 + row) * (i < len ? sRq[i] : sRq[len - 1]);
                gg[r] = p.g_c[((size_t)(start + ii) * HV + h) * 128 + row];
            }
#pragma unroll
            for (int I = 0; I < 4; ++I) ga[I] = sGa[I][row];   // anchor rows (the last valid row stands in for anchors past the end)
            const float gL = p.g_c[((size_t)(start + len - 1) * HV + h) * 128 + row];
            umma::mbar_wait(&sh.barA, nA & 1);
            umma::fence_after_sync();
            {   // column sum of the inter-chunk k gradient for the last row's gate term
                float ab[16];
                umma::tmem_ld16(umma::tmem_addr(tmem, warp, 384 + 16 * cg), ab);
                float cs = 0.f;
#pragma unroll
                for (int r = 0; r < 16; ++r)
                    if (16 * cg + r < len) cs += kq[r] * ex2f_(gL - gg[r]) * ab[r];
                sCol[cg][row] = cs;
            }
            __syncthreads();
            const float extra = ((sCol[0][row] + sCol[1][row]) + (sCol[2][row] + sCol[3][row])) + ex2f_(gL) * sDgl[row];
            // the three outputs per (token, channel) go straight to their fp32 [64 tokens][128] tiles: a warp writes 128
            // consecutive bytes per token, and shared memory stays free for the next item's tiles
            const size_t ob = (size_t)item * (size_t)(CH * DK) + row;
            const size_t obk = ((size_t)c * HK + hk) * (size_t)(CH * DK) + row;      // dq / dk: one tile per q/k head
            float* __restrict__ oq = p.dq_v + obk;
            float* __restrict__ ok = p.dk_v + obk;
            float* __restrict__ og = p.dgp + ob;
            const bool first_of_group = j == 0;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int c0 = 16 * cg + 8 * hf;
                float aq[8], ak[8], ab[8], vr[8], vt[8], dkc[8];
                umma::tmem_ld8(umma::tmem_addr(tmem, warp, 192 + c0), aq);
                umma::tmem_ld8(umma::tmem_addr(tmem, warp, 320 + c0), ak);
                umma::tmem_ld8(umma::tmem_addr(tmem, warp, 384 + c0), ab);
                if (SCALAR) {
                    umma::tmem_ld8(umma::tmem_addr(tmem, warp, c0), vr);
                    umma::tmem_ld8(umma::tmem_addr(tmem, warp, 64 + c0), vt);
                    umma::tmem_ld8(umma::tmem_addr(tmem, warp, 128 + c0), dkc);
                } else {
                    umma::tmem_ld8(umma::tmem_addr(tmem, warp, 32 * cg + 8 * hf), vr);
                    umma::tmem_ld8(umma::tmem_addr(tmem, warp, 32 * cg + 16 + 8 * hf), vt);
#pragma unroll
                    for (int r = 0; r < 8; ++r) dkc[r] = 0.f;
#pragma unroll
                    for (int I = 0; I < 4; ++I) {
                        if (I < cg) continue;                  // warp-uniform
                        float c8[8];
                        umma::tmem_ld8(umma::tmem_addr(tmem, warp, ccol_off(I) + c0), c8);
#pragma unroll
                        for (int r = 0; r < 8; ++r) dkc[r] += c8[r] * ex2f_(ga[I] - gg[8 * hf + r]);
                    }
                }
                float bsv[8];
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const int i = c0 + r, rr = 8 * hf + r;
                    const float g = gg[rr], kv = kq[rr], qv = qq[rr];
                    const float up = ex2f_(g), re = ex2f_(gL - g), e = SCALAR ? 1.f : ex2f_(g - ga[cg]);
                    const float dqt = p.scale * aq[r], dkt = -ak[r], dkb = ab[r];
                    const float dqr = vr[r] * e, T = vt[r] * e, bt = sh.beta[i], dgn = sDiag[i];
                    bsv[r] = kv * T;
                    float dg = qv * up * dqt + kv * up * dkt - kv * re * dkb;
                    if (i == len - 1) dg += extra;
                    const bool ok_row = i < len;
                    const float dq_e = ok_row ? dqt * up + dqr + dgn * kv : 0.f;
                    const float dk_e = ok_row ? (dkt * up + dkb * re) + bt * T + dkc[r] + dgn * qv : 0.f;
                    if (first_of_group) { oq[i * DK] = dq_e; ok[i * DK] = dk_e; }
                    else { red_add(oq + i * DK, dq_e); red_add(ok + i * DK, dk_e); }
                    og[i * DK] = ok_row ? dg + qv * dqr + kv * bt * T - kv * dkc[r] : 0.f;
                }
                // sum over the 32 channels of this warp for the 8 rows at once: every exchange halves the number of rows a lane
                // carries (9 shuffles instead of 40); the lane whose bits 4..2 spell the row ends up with its sum
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float recv = __shfl_xor_sync(0xffffffffu, (lane & 16) ? bsv[r] : bsv[r + 4], 16);
                    bsv[r] = ((lane & 16) ? bsv[r + 4] : bsv[r]) + recv;
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const float recv = __shfl_xor_sync(0xffffffffu, (lane & 8) ? bsv[r] : bsv[r + 2], 8);
                    bsv[r] = ((lane & 8) ? bsv[r + 2] : bsv[r]) + recv;
                }
                {
                    const float recv = __shfl_xor_sync(0xffffffffu, (lane & 4) ? bsv[0] : bsv[1], 4);
                    bsv[0] = ((lane & 4) ? bsv[1] : bsv[0]) + recv;
                }
                bsv[0] += __shfl_xor_sync(0xffffffffu, bsv[0], 2);
                bsv[0] += __shfl_xor_sync(0xffffffffu, bsv[0], 1);
                if ((lane & 3) == 0) sRed[q][c0 + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1)] = bsv[0];
            }
        }
        ++nA;
        umma::fence_before_sync();
        __syncthreads();                                       // sRed complete; every accumulator has been read
        umma::fence_after_sync();
        if (tid < len) {
            const size_t th = (size_t)(start + tid) * HV + h;
            float db = sDbw[tid] + ((sRed[0][tid] + sRed[1][tid]) + (sRed[2][tid] + sRed[3][tid]));
            if (p.beta_sigmoid) {
                const float sg = sigmoidf_(ld1(p.beta_raw, p.beta_dtype, th));
                db *= p.beta_scale * sg * (1.f - sg);
            }
            st1(p.dbeta, p.dbeta_dtype, th, db);
        }
        __syncthreads();
        if (last_of_group) { j = 0; grp += stride; } else ++j;
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 512);
}

template <int DT, bool SCALAR>
static int launch_bwd_chunk_tc_t(const MkdaBwdChunk* p, cudaStream_t stream) {
    auto kern = bwd_chunk_tc_kernel<DT, SCALAR>;
    if (int e = ensure_smem((const void*)kern, BWD_CHUNK_SMEM, "bwd_chunk")) return e;
    const int groups = p->L.NC * p->L.HK;              // a CTA takes whole (chunk, q/k head) groups
    kern<<<groups < sm_count() ? groups : sm_count(), BWD_CHUNK_THREADS, BWD_CHUNK_SMEM, stream>>>(*p);
    return check_launch("bwd_chunk");
}
int launch_bwd_chunk_tc(const MkdaBwdChunk* p, cudaStream_t stream) {
    switch (p->qkv_dtype * 2 + (p->scalar_gate ? 1 : 0)) {
        case MKDA_F32 * 2: return launch_bwd_chunk_tc_t<MKDA_F32, false>(p, stream);
        case MKDA_BF16 * 2: return launch_bwd_chunk_tc_t<MKDA_BF16, false>(p, stream);
        case MKDA_F16 * 2: return launch_bwd_chunk_tc_t<MKDA_F16, false>(p, stream);
        case MKDA_F32 * 2 + 1: return launch_bwd_chunk_tc_t<MKDA_F32, true>(p, stream);
        case MKDA_BF16 * 2 + 1: return launch_bwd_chunk_tc_t<MKDA_BF16, true>(p, stream);
        case MKDA_F16 * 2 + 1: return launch_bwd_chunk_tc_t<MKDA_F16, true>(p, stream);
    }
    return set_error(MKDA_ERR_ARG, "bwd_chunk: unsupported dtype");
}

int tc_intra_status(unsigned int* out) {
    return cudaMemcpyFromSymbol(out, umma::g_timeout_flag, sizeof(unsigned int)) == cudaSuccess ? 0 : -1;
}
int tc_intra_status_clear() {
    const unsigned int z = 0;
    return cudaMemcpyToSymbol(umma::g_timeout_flag, &z, sizeof(z)) == cudaSuccess ? 0 : -1;
}

template <int DT, bool SCALAR, bool TMA>
static int launch_intra_fwd_tc_tt(const MkdaIntraFwd* p, const IntraMaps& maps, cudaStream_t stream) {
    auto kern = intra_fwd_tc_kernel<DT, SCALAR, TMA>;
    if (int e = ensure_smem((const void*)kern, INTRA_TC_SMEM, "intra_fwd")) return e;
    const int items = p->L.NC * p->L.HV;
    kern<<<items < sm_count() ? items : sm_count(), 512, INTRA_TC_SMEM, stream>>>(*p, maps);
    return check_launch("intra_fwd");
}
template <int DT, bool SCALAR>
static int launch_intra_fwd_tc_t(const MkdaIntraFwd* p, cudaStream_t stream) {
    IntraMaps maps;
    memset(&maps, 0, sizeof(maps));
    // 16-bit rows travel by tiled copy when the tensors can be described (16-byte aligned); otherwise through registers
    if (DT != MKDA_F32 && make_rows_map(&maps.k, p->k, 2, (unsigned long long)p->L.TT, (unsigned long long)p->L.HK * 128, "intra_fwd") == MKDA_OK &&
        make_rows_map(&maps.q, p->q, 2, (unsigned long long)p->L.TT, (unsigned long long)p->L.HK * 128, "intra_fwd") == MKDA_OK &&
        make_rows_map(&maps.g, p->g_c, 4, (unsigned long long)p->L.TT, (unsigned long long)p->L.HV * 128, "intra_fwd") == MKDA_OK)
        return launch_intra_fwd_tc_tt<DT, SCALAR, true>(p, maps, stream);
    return launch_intra_fwd_tc_tt<DT, SCALAR, false>(p, maps, stream);
}
int launch_intra_fwd_tc(const MkdaIntraFwd* p, cudaStream_t stream) {
    switch (p->qkv_dtype * 2 + (p->scalar_gate ? 1 : 0)) {
        case MKDA_F32 * 2: return launch_intra_fwd_tc_t<MKDA_F32, false>(p, stream);
        case MKDA_BF16 * 2: return launch_intra_fwd_tc_t<MKDA_BF16, false>(p, stream);
        case MKDA_F16 * 2: return launch_intra_fwd_tc_t<MKDA_F16, false>(p, stream);
        case MKDA_F32 * 2 + 1: return launch_intra_fwd_tc_t<MKDA_F32, true>(p, stream);
        case MKDA_BF16 * 2 + 1: return launch_intra_fwd_tc_t<MKDA_BF16, true>(p, stream);
        case MKDA_F16 * 2 + 1: return launch_intra_fwd_tc_t<MKDA_F16, true>(p, stream);
    }
    return set_error(MKDA_ERR_ARG, "intra_fwd: unsupported dtype");
}

}  // namespace mkda

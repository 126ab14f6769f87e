// Chunk-parallel kernels on the Blackwell tensor cores (tcgen05.mma, TMEM accumulators): one CTA (16 warps) per
// (chunk, v-head).  Every product puts a 128-wide dimension (K or V index, or two stacked 64-row operands) on the MMA M
// axis and the chunk rows on N, so all accumulators are [128 lanes x 64 / 128 columns] fp32 tiles in tensor memory.
// Operands either arrive as ready-made tiles by bulk copy (states, Vd, nw, A, Aqk, the scaled q / k) or are produced by
// the CUDA cores (gate scaling, L2 statistics, bf16 hi/lo split) straight into the swizzled tile layout; see umma.cuh.
#include "common.cuh"
#include "host.h"
#include "umma.cuh"

#include <type_traits>

namespace mkda {

using umma::smem_u32;
using umma::store_split8;
using umma::tile_bytes;

__device__ __forceinline__ void load8(const void* base, int dtype, size_t idx, float (&v)[8]) {   // idx % 8 == 0
    ld8(base, dtype, idx, v);
}
__device__ __forceinline__ void zero8(float (&v)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
}

// Batched staging: a thread first issues the global loads of all CNT of its chunks (independent, so they are all in
// flight together), then splits and stores them.  Chunk n of thread t is linear index t + n * NTHR; ALONG_K maps the
// index to (row = i / (KT/8), chunk = i % (KT/8)), otherwise to (chunk = i / R, row = i % R).
template <int CNT, int NTHR, bool ALONG_K, class F>
__device__ __forceinline__ void load_chunks(float (&v)[CNT][8], int R, int KT, F f) {
    const int nk8 = KT >> 3;
#pragma unroll
    for (int n = 0; n < CNT; ++n) {
        const int i = threadIdx.x + n * NTHR;
        const int r = ALONG_K ? i / nk8 : i % R, k8 = ALONG_K ? i % nk8 : i / R;
        f(r, k8, v[n]);
    }
}
template <int CNT, int NTHR, bool ALONG_K>
__device__ __forceinline__ void store_chunks(uint8_t* hi, uint8_t* lo, const float (&v)[CNT][8], int R, int KT) {
    const int nk8 = KT >> 3;
#pragma unroll
    for (int n = 0; n < CNT; ++n) {
        const int i = threadIdx.x + n * NTHR;
        const int r = ALONG_K ? i / nk8 : i % R, k8 = ALONG_K ? i % nk8 : i / R;
        store_split8(hi, lo, R, r, k8, v[n]);
    }
}

struct TcShared {
    uint64_t bar;
    uint32_t tmem;
};

// common prologue / epilogue of a tensor-core CTA
__device__ __forceinline__ uint8_t* tc_begin(uint8_t* smem_raw, TcShared* sh, uint32_t tmem_cols) {
    if ((threadIdx.x >> 5) == 0) umma::tmem_alloc(&sh->tmem, tmem_cols);
    if (threadIdx.x == 0) { umma::mbar_init(&sh->bar, 1); umma::fence_barrier_init(); }
    return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
}
// all operand tiles written: publish them to the tensor core and read the TMEM base
__device__ __forceinline__ uint32_t tc_operands_ready(TcShared* sh) {
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    return sh->tmem;
}
__device__ __forceinline__ void tc_end(TcShared* sh, uint32_t tmem, uint32_t tmem_cols) {
    umma::fence_before_sync();
    __syncthreads();
    if ((threadIdx.x >> 5) == 0) umma::tmem_dealloc(tmem, tmem_cols);
}

// ---------------------------------------------------------------------------------------------------------
// output:  O^T[v x tok] = H^T qs^T + Vd^T Aqk^T (qs = scale q 2^g), then the row-wise epilogue (gated RMSNorm) from a shared
// [tok][v] staging tile so that all global stores are full 512-byte rows.
// Persistent: one CTA per SM walks the (chunk, v-head) items gridDim.x apart.  All four operands of an item arrive as
// ready-made tiles by bulk copy, so as soon as an item's products are done its tile buffers are handed to the copies of
// the next item, which then travel while the epilogue of the current item runs (its staging tile has its own space).
constexpr int OLD = 132;   // leading dimension of the fp32 [tok][v] staging tile
constexpr int OUT_TC_OPND = 2 * tile_bytes(128, 128) + 2 * tile_bytes(64, 128) + 2 * tile_bytes(128, 64) + 2 * tile_bytes(64, 64);
constexpr int OUT_TC_SMEM = OUT_TC_OPND + CH * OLD * 4 + 1024;

template <int GDT>
__global__ void __launch_bounds__(512, 1) out_fwd_tc_kernel(const MkdaOutFwd p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ TcShared sh;
    __shared__ uint64_t ldbar;
    uint8_t* base = tc_begin(smem_raw, &sh, 64);
    uint8_t* a1h = base;                                    // S^T [v][K index]
    uint8_t* a1l = a1h + tile_bytes(128, 128);
    uint8_t* b1h = a1l + tile_bytes(128, 128);              // scale q 2^g [tok][K index]
    uint8_t* b1l = b1h + tile_bytes(64, 128);
    uint8_t* a2h = b1l + tile_bytes(64, 128);               // Vd^T [v][tok]
    uint8_t* a2l = a2h + tile_bytes(128, 64);
    uint8_t* b2h = a2l + tile_bytes(128, 64);               // Aqk [i][j]
    uint8_t* b2l = b2h + tile_bytes(64, 64);
    float* sO = reinterpret_cast<float*>(base + OUT_TC_OPND);   // [64][OLD] fp32 staging of the output rows

    const int HV = p.L.HV;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int total = p.L.NC * HV, stride = gridDim.x;

    auto request = [&](int it) {                        // thread 0: the four tiles of item `it`, counted on one barrier
        umma::mbar_expect_tx(&ldbar, umma::STATE_TILE_BYTES + 2 * umma::CHUNK_TILE_BYTES + umma::QUARTER_TILE_BYTES);
        umma::bulk_load(b2h, reinterpret_cast<const uint8_t*>(p.Aqk) + (size_t)it * umma::QUARTER_TILE_BYTES, umma::QUARTER_TILE_BYTES, &ldbar);
        umma::bulk_load(a2h, reinterpret_cast<const uint8_t*>(p.Vd) + (size_t)it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &ldbar);
        umma::bulk_load(b1h, reinterpret_cast<const uint8_t*>(p.qs) + (size_t)it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &ldbar);
        umma::bulk_load(a1h, reinterpret_cast<const uint8_t*>(p.h) + (size_t)it * umma::STATE_TILE_BYTES, umma::STATE_TILE_BYTES, &ldbar);
    };
    if (tid == 0) {
        umma::mbar_init(&ldbar, 1);
        umma::fence_barrier_init();
        if ((int)blockIdx.x < total) request(blockIdx.x);
    }
    float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
    if (p.has_norm && p.norm_w) w = ld4(p.norm_w, p.norm_w_dtype, 4 * lane);
    const uint32_t tmem = tc_operands_ready(&sh);

    int k = 0;
    for (int item = blockIdx.x; item < total; item += stride, ++k) {
        const int c = item / HV, h = item - c * HV;
        const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
        if (umma::mma_issuer()) {
            umma::mbar_wait(&ldbar, k & 1);                // this item's tiles have landed
            umma::gemm(tmem, umma::opnd_k(a2h, a2l, 128), umma::opnd_k(b2h, b2l, 64), 128, 64, 64, 0u);
            umma::gemm(tmem, umma::opnd_k(a1h, a1l, 128), umma::opnd_k(b1h, b1l, 64), 128, 64, 128, 1u);
            umma::commit(&sh.bar);
        }
        // the row pass (warp w owns rows w, w + 16, ...) fetches its gate values while the products run
        float4 zg[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = warp + 16 * i, rr = r < len ? r : len - 1;
            zg[i] = p.has_norm ? ld4(p.gate, GDT, ((size_t)(start + rr) * HV + h) * 128 + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        umma::mbar_wait(&sh.bar, k & 1);
        umma::fence_after_sync();
        if (tid == 0 && item + stride < total) request(item + stride);   // the tile buffers are free: next item's copies start now
        {   // TMEM [v lanes][tok cols] -> shared [tok][v]
            float v[16];
            const int t0 = (warp >> 2) * 16, vi = (warp & 3) * 32 + lane;
            umma::tmem_ld16(umma::tmem_addr(tmem, warp, t0), v);
#pragma unroll
            for (int j = 0; j < 16; ++j) sO[(t0 + j) * OLD + vi] = v[j];
        }
        umma::fence_before_sync();
        __syncthreads();                                   // staging tile complete; the accumulator may be overwritten
        umma::fence_after_sync();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = warp + 16 * i;
            if (r >= len) continue;                                   // warp-uniform
            float4 o = *reinterpret_cast<const float4*>(sO + r * OLD + 4 * lane);
            const size_t off = ((size_t)(start + r) * HV + h) * 128 + 4 * lane;
            if (p.o_raw) *reinterpret_cast<float4*>(p.o_raw + off) = o;
            if (p.has_norm) {
                float ss = (o.x * o.x + o.y * o.y) + (o.z * o.z + o.w * o.w);
#pragma unroll
                for (int sft = 16; sft > 0; sft >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sft);
                const float rs = 1.f / sqrtf(ss * (1.f / 128.f) + p.eps);
                const float zz[4] = {zg[i].x, zg[i].y, zg[i].z, zg[i].w};
                float a[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float sg = sigmoidf_(zz[e]);
                    a[e] = p.act == MKDA_ACT_SILU ? zz[e] * sg : sg;
                }
                o = make_float4(o.x * rs * w.x * a[0], o.y * rs * w.y * a[1], o.z * rs * w.z * a[2], o.w * rs * w.w * a[3]);
            }
            st4(p.out, p.out_dtype, off, o);
        }
        __syncthreads();                                   // the staging tile is free for the next item
    }
    tc_end(&sh, tmem, 64);
}

int tc_chunk_status(unsigned int* out) {
    return cudaMemcpyFromSymbol(out, umma::g_timeout_flag, sizeof(unsigned int)) == cudaSuccess ? 0 : -1;
}

template <int GDT>
static int launch_out_fwd_tc_t(const MkdaOutFwd* p, cudaStream_t stream) {
    auto kern = out_fwd_tc_kernel<GDT>;
    if (int e = ensure_smem((const void*)kern, OUT_TC_SMEM, "out_fwd")) return e;
    const int items = p->L.NC * p->L.HV;
    kern<<<items < sm_count() ? items : sm_count(), 512, OUT_TC_SMEM, stream>>>(*p);
    return check_launch("out_fwd");
}
// dispatch on runtime dtypes to kernels specialised at compile time (keeps every load loop free of branches)
#define MKDA_DISPATCH2(FN, A, B, ...)                                                                        \
    switch ((A) * 3 + (B)) {                                                                                 \
        case 0: return FN<0, 0>(__VA_ARGS__); case 1: return FN<0, 1>(__VA_ARGS__); case 2: return FN<0, 2>(__VA_ARGS__); \
        case 3: return FN<1, 0>(__VA_ARGS__); case 4: return FN<1, 1>(__VA_ARGS__); case 5: return FN<1, 2>(__VA_ARGS__); \
        case 6: return FN<2, 0>(__VA_ARGS__); case 7: return FN<2, 1>(__VA_ARGS__); case 8: return FN<2, 2>(__VA_ARGS__); \
        default: return set_error(MKDA_ERR_ARG, "unsupported dtype");                                        \
    }
int launch_out_fwd_tc(const MkdaOutFwd* p, cudaStream_t stream) {
    switch (p->has_norm ? p->gate_dtype : 0) {
        case MKDA_F32: return launch_out_fwd_tc_t<MKDA_F32>(p, stream);
        case MKDA_BF16: return launch_out_fwd_tc_t<MKDA_BF16>(p, stream);
        case MKDA_F16: return launch_out_fwd_tc_t<MKDA_F16>(p, stream);
    }
    return set_error(MKDA_ERR_ARG, "out_fwd: unsupported dtype");
}

// reconstruct 8 fp32 values from the hi / lo tiles at (row r, chunk k8)
__device__ __forceinline__ void load_tile8(const uint8_t* hi, const uint8_t* lo, int R, int r, int k8, float (&v)[8]) {
    const uint32_t off = umma::tile_chunk_offset(R, r, k8);
    const uint4 a = *reinterpret_cast<const uint4*>(hi + off), b = *reinterpret_cast<const uint4*>(lo + off);
    const uint32_t hw[4] = {a.x, a.y, a.z, a.w}, lw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        v[2 * e] = __uint_as_float(hw[e] << 16) + __uint_as_float(lw[e] << 16);
        v[2 * e + 1] = __uint_as_float(hw[e] & 0xffff0000u) + __uint_as_float(lw[e] & 0xffff0000u);
    }
}

// ---------------------------------------------------------------------------------------------------------
// bwd_wy.  With S the state entering the chunk, k~ = k 2^g, Ab = A diag(beta):
//   X = V - k~ S        Vd = Ab X (saved by the forward pass)        dAqk = lower(dO Vd^T)
//   dW = A^T dVd        dX = diag(beta) dW (= dV)       dbeta_w = rowsum(dW * X)
//   dA = (dVd X^T) diag(beta)          dL = -strictlower(A^T dA A^T)
// Five dependent products, each with a 128-wide axis on M (TMEM columns in brackets):
//   G1 [0]    X^T[v x tok]  = V^T - S^T k~^T                       (A = the saved state tile as it is)
//             Vd^T[v x i]   = X^T (A diag(beta))^T is not recomputed: the forward pass's Vd^T tile is fetched instead
//   G4 [256]  dW^T[v x j]   = dVd^T A                              (both operands MN-major views of natural tiles)
//   G3 [128]  [dO; dVd] [Vd; X]^T  -> rows 0..63 / cols 0..63 = dO Vd^T, rows 64..127 / cols 64..127 = dVd X^T
//   G5 [320]  Y[a x j]      = (dVd X^T diag(beta)) A^T
//   G6 [384]  Z[i x j]      = A^T Y          dL = -strictlower(Z)
// dbeta_w[j] = sum_v dW[j][v] X[j][v] is evaluated as sum_i A[i][j] (dVd X^T)[i][j], which needs no extra product.
// Shared-memory tiles are recycled as soon as the product reading them has completed.
// ---------------------------------------------------------------------------------------------------------
constexpr int WY_TC_SMEM = 192 * 1024 + 1024;

template <int KVDT, int DODT>
__global__ void __launch_bounds__(512, 1) bwd_wy_tc_kernel(const MkdaBwdWy p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ TcShared sh;
    __shared__ float sBeta[CH];
    __shared__ float sRed[2][CH];
    uint8_t* base = tc_begin(smem_raw, &sh, 512);
    uint8_t* sSh = base;                      // S [kidx][v]; later [dO; dVd] [tok][v]
    uint8_t* sSl = sSh + 32768;
    uint8_t* sKh = sSl + 32768;               // k~ [tok][kidx]; later dA diag(beta) [a][b]
    uint8_t* sKl = sKh + 16384;
    uint8_t* sVh = sKl + 16384;               // Vd^T [v][i] | X^T [v][j] (hi), then the same pair (lo)
    uint8_t* sXh = sVh + 16384;
    uint8_t* sVl = sXh + 16384;
    uint8_t* sXl = sVl + 16384;
    uint8_t* sAh = sXl + 16384;               // A [i][j]
    uint8_t* sAl = sAh + 8192;
    uint8_t* sBh = sAl + 8192;                // Y [a][j]
    uint8_t* sBl = sBh + 8192;

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, cg = warp >> 2, row = q * 32 + lane;      // TMEM lane owned by this thread, 16-column group
    uint32_t phase = 0;

    if (tid < CH) sBeta[tid] = tid < len ? p.beta[(size_t)(start + tid) * HV + h] : 0.f;
    __shared__ uint64_t ldbar;
    if (tid == 0) {   // S^T [v][K index], A [i][j] and the forward pass's Vd^T [v][i] arrive as ready-made operand tiles
        const size_t it = (size_t)c * HV + h;
        const uint8_t* vd = reinterpret_cast<const uint8_t*>(p.Vd) + it * umma::CHUNK_TILE_BYTES;
        umma::mbar_init(&ldbar, 1);
        umma::fence_barrier_init();
        umma::mbar_expect_tx(&ldbar, umma::STATE_TILE_BYTES + umma::QUARTER_TILE_BYTES + umma::CHUNK_TILE_BYTES);
        umma::bulk_load(sSh, reinterpret_cast<const uint8_t*>(p.h) + it * umma::STATE_TILE_BYTES, umma::STATE_TILE_BYTES, &ldbar);
        umma::bulk_load(sAh, reinterpret_cast<const uint8_t*>(p.A) + it * umma::QUARTER_TILE_BYTES, umma::QUARTER_TILE_BYTES, &ldbar);
        umma::bulk_load(sVh, vd, umma::CHUNK_TILE_BYTES / 2, &ldbar);                          // hi half, left column block
        umma::bulk_load(sVl, vd + umma::CHUNK_TILE_BYTES / 2, umma::CHUNK_TILE_BYTES / 2, &ldbar);   // lo half
    }
    // everything the first three stages need from global memory is requested up front: k, g, A, then [dO; dVd] rows and
    // this thread's V column, which stay in registers until G1 has released the state tile
    float vT[4][8], vv[16];
    {
        float vK[2][8], vG[2][8];
        load_chunks<2, 512, true>(vK, 64, 128, [&](int r, int k8, float (&v)[8]) {
            const int rr = r < len ? r : len - 1;
            load8(p.k, KVDT, ((size_t)(start + rr) * HK + hk) * 128 + k8 * 8, v);
        });
        load_chunks<2, 512, true>(vG, 64, 128, [&](int r, int k8, float (&v)[8]) {
            const int rr = r < len ? r : len - 1;
            load8(p.g_c, MKDA_F32, ((size_t)(start + rr) * HV + h) * 128 + k8 * 8, v);
        });
        load_chunks<4, 512, true>(vT, 128, 128, [&](int r, int k8, float (&v)[8]) {
            const int t = r & 63, tt = t < len ? t : len - 1;
            const size_t off = ((size_t)(start + tt) * HV + h) * 128 + k8 * 8;
            if (r < 64) load8(p.d_o, DODT, off, v); else load8(p.dVd, MKDA_F32, off, v);
        });
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = cg * 16 + j, tt = t < len ? t : len - 1;
            vv[j] = ld1(p.v, KVDT, ((size_t)(start + tt) * HV + h) * 128 + row);
        }
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int i = tid + n * 512, r = i >> 4;
            const int rr = r < len ? r : len - 1;
            const float rk = r < len ? (p.k_rstd ? p.k_rstd[(size_t)(start + rr) * HK + hk] : 1.f) : 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) vK[n][e] *= rk * ex2f_(vG[n][e]);
        }
        store_chunks<2, 512, true>(sKh, sKl, vK, 64, 128);
    }
    const uint32_t tmem = tc_operands_ready(&sh);
    if (umma::mma_issuer()) {
        umma::mbar_wait(&ldbar, 0);                        // the state tile has landed
        umma::gemm(tmem + 0, umma::opnd_k(sSh, sSl, 128), umma::opnd_k(sKh, sKl, 64), 128, 64, 128, 0u);
        umma::commit(&sh.bar);
    }
    {
#pragma unroll
        for (int n = 0; n < 4; ++n)
            if ((((tid + n * 512) >> 4) & 63) >= len) zero8(vT[n]);
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (cg * 16 + j >= len) vv[j] = 0.f;
        umma::mbar_wait(&sh.bar, phase); phase ^= 1;
        umma::mbar_wait(&ldbar, 0);                            // long complete: makes the A tile visible to every reader below
        umma::fence_after_sync();
        float d[16], x0[8], x1[8];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, cg * 16), d);
#pragma unroll
        for (int j = 0; j < 8; ++j) { x0[j] = vv[j] - d[j]; x1[j] = vv[8 + j] - d[8 + j]; }
        store_split8(sXh, sXl, 128, row, 2 * cg, x0);
        store_split8(sXh, sXl, 128, row, 2 * cg + 1, x1);
        store_chunks<4, 512, true>(sSh, sSl, vT, 128, 128);      // S is dead: the region now holds [dO; dVd]
    }
    tc_operands_ready(&sh);
    if (umma::mma_issuer()) {   // Vd^T is the forward pass's tile (the barrier it came on was awaited before G1): G4 and G3 go together
        umma::gemm(tmem + 256, umma::opnd_mn(sSh, sSl, 128, 64), umma::opnd_mn(sAh, sAl, 64), 128, 64, 64, 0u);
        umma::gemm(tmem + 128, umma::opnd_k(sSh, sSl, 128), umma::opnd_mn(sVh, sVl, 128), 128, 128, 128, 0u);
        umma::commit(&sh.bar);
    }
    umma::mbar_wait(&sh.bar, phase); phase ^= 1;
    umma::fence_after_sync();
    {
        float dw[16];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 256 + cg * 16), dw);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = cg * 16 + j;
            if (t < len) p.dX[((size_t)(start + t) * HV + h) * 128 + row] = sBeta[t] * dw[j];
        }
    }
    if (q < 2) {                                   // rows i = row: dAqk = lower(dO Vd^T)
        float d[16];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 128 + cg * 16), d);
        if (row < len) {
            float* dst = p.dAqk + ((size_t)(start + row) * HV + h) * 64 + cg * 16;
#pragma unroll
            for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(cg * 16 + j <= row ? d[j] : 0.f, cg * 16 + j + 1 <= row ? d[j + 1] : 0.f,
                                                                  cg * 16 + j + 2 <= row ? d[j + 2] : 0.f, cg * 16 + j + 3 <= row ? d[j + 3] : 0.f);
        }
    } else {                                       // rows i = row - 64: dVd X^T -> dbeta_w partials and dA diag(beta)
        const int i = row - 64;
        float d[16], a0[8], a1[8];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 128 + 64 + cg * 16), d);
        load_tile8(sAh, sAl, 64, i, 2 * cg, a0);
        load_tile8(sAh, sAl, 64, i, 2 * cg + 1, a1);
        float pr[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            pr[j] = d[j] * (j < 8 ? a0[j] : a1[j - 8]);
            const float da = d[j] * sBeta[cg * 16 + j];
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
        if ((lane & 1) == 0) sRed[q - 2][cg * 16 + ((lane >> 1) & 15)] = pr[0];
        store_split8(sKh, sKl, 128, i, 2 * cg, a0);
        store_split8(sKh, sKl, 128, i, 2 * cg + 1, a1);
    }
    tc_operands_ready(&sh);
    if (tid < len) p.dbeta_w[(size_t)(start + tid) * HV + h] = sRed[0][tid] + sRed[1][tid];
    if (umma::mma_issuer()) {
        umma::gemm(tmem + 320, umma::opnd_k(sKh, sKl, 128), umma::opnd_k(sAh, sAl, 64), 128, 64, 64, 0u);
        umma::commit(&sh.bar);
    }
    umma::mbar_wait(&sh.bar, phase); phase ^= 1;
    umma::fence_after_sync();
    if (q < 2) {
        float y[16], a0[8], a1[8];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 320 + cg * 16), y);
#pragma unroll
        for (int j = 0; j < 8; ++j) { a0[j] = y[j]; a1[j] = y[8 + j]; }
        store_split8(sBh, sBl, 64, row, 2 * cg, a0);
        store_split8(sBh, sBl, 64, row, 2 * cg + 1, a1);
    }
    tc_operands_ready(&sh);
    if (umma::mma_issuer()) {
        umma::gemm(tmem + 384, umma::opnd_mn(sAh, sAl, 64), umma::opnd_mn(sBh, sBl, 64), 128, 64, 64, 0u);
        umma::commit(&sh.bar);
    }
    umma::mbar_wait(&sh.bar, phase); phase ^= 1;
    umma::fence_after_sync();
    if (q < 2) {
        float z[16];
        umma::tmem_ld16(umma::tmem_addr(tmem, warp, 384 + cg * 16), z);      // warp-collective: never under a per-lane condition
        if (row < len) {
        float* dst = p.dL + ((size_t)(start + row) * HV + h) * 64 + cg * 16;
#pragma unroll
        for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(cg * 16 + j < row ? -z[j] : 0.f, cg * 16 + j + 1 < row ? -z[j + 1] : 0.f,
                                                              cg * 16 + j + 2 < row ? -z[j + 2] : 0.f, cg * 16 + j + 3 < row ? -z[j + 3] : 0.f);
        }
    }
    tc_end(&sh, tmem, 512);
}

template <int KVDT, int DODT>
static int launch_bwd_wy_tc_t(const MkdaBwdWy* p, cudaStream_t stream) {
    auto kern = bwd_wy_tc_kernel<KVDT, DODT>;
    if (int e = ensure_smem((const void*)kern, WY_TC_SMEM, "bwd_wy")) return e;
    kern<<<dim3(p->L.NC, p->L.HV), 512, WY_TC_SMEM, stream>>>(*p);
    return check_launch("bwd_wy");
}
int launch_bwd_wy_tc(const MkdaBwdWy* p, cudaStream_t stream) {
    MKDA_DISPATCH2(launch_bwd_wy_tc_t, p->kv_dtype, p->do_dtype, p, stream)
}

}  // namespace mkda

// Chunk-parallel kernels on the Blackwell tensor cores (tcgen05.mma, TMEM accumulators): one CTA (8 warps) per
// (chunk, v-head).  Every product puts a 128-wide state dimension (K or V index) on the MMA M axis and the 64 chunk rows
// on N, so all accumulators are [128 lanes x 64 columns] fp32 tiles in tensor memory.  Operands are produced by the CUDA
// cores (gate scaling, L2 statistics, bf16 hi/lo split) straight into the swizzled K-major tile layout; see umma.cuh.
#include "common.cuh"
#include "host.h"
#include "umma.cuh"

namespace mkda {

using umma::smem_u32;
using umma::store_split8;
using umma::tile_bytes;

// Stage R x KT values with lanes walking along K (source contiguous along K): f(r, k8, v[8]) fills 8 consecutive k.
template <int NTHR, class F>
__device__ __forceinline__ void stage_along_k(uint8_t* hi, uint8_t* lo, int R, int KT, F f) {
    const int nk8 = KT >> 3, total = R * nk8;
    for (int i = threadIdx.x; i < total; i += 2 * NTHR) {
        const int i2 = i + NTHR;
        const int r = i / nk8, k8 = i - r * nk8, r2 = i2 / nk8, k82 = i2 - r2 * nk8;
        float v[8], w[8];
        f(r, k8, v);
        if (i2 < total) f(r2, k82, w);
        store_split8(hi, lo, R, r, k8, v);
        if (i2 < total) store_split8(hi, lo, R, r2, k82, w);
    }
}
// Stage with lanes walking along the rows (source contiguous along the row index: a transposed read).
template <int NTHR, class F>
__device__ __forceinline__ void stage_along_rows(uint8_t* hi, uint8_t* lo, int R, int KT, F f) {
    const int nk8 = KT >> 3, total = R * nk8;
    for (int i = threadIdx.x; i < total; i += 2 * NTHR) {
        const int i2 = i + NTHR;
        const int k8 = i / R, r = i - k8 * R, k82 = i2 / R, r2 = i2 - k82 * R;
        float v[8], w[8];
        f(r, k8, v);
        if (i2 < total) f(r2, k82, w);
        store_split8(hi, lo, R, r, k8, v);
        if (i2 < total) store_split8(hi, lo, R, r2, k82, w);
    }
}

__device__ __forceinline__ void load8(const void* base, int dtype, size_t idx, float (&v)[8]) {   // idx % 8 == 0
    const float4 a = ld4(base, dtype, idx), b = ld4(base, dtype, idx + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void zero8(float (&v)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
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
// output:  O^T[v x tok] = H^T (scale q 2^g)^T + Vd^T Aqk^T, then the row-wise epilogue (gated RMSNorm) from a shared
// [tok][v] staging tile so that all global stores are full 512-byte rows.
// ---------------------------------------------------------------------------------------------------------
constexpr int OUT_TC_SMEM = 2 * tile_bytes(128, 128) + 2 * tile_bytes(64, 128) + 2 * tile_bytes(128, 64) + 2 * tile_bytes(64, 64) + 1024;
constexpr int OLD = 132;   // leading dimension of the fp32 [tok][v] staging tile

__global__ void __launch_bounds__(512, 1) out_fwd_tc_kernel(const MkdaOutFwd p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ TcShared sh;
    uint8_t* base = tc_begin(smem_raw, &sh, 64);
    uint8_t* a1h = base;
    uint8_t* a1l = a1h + tile_bytes(128, 128);
    uint8_t* b1h = a1l + tile_bytes(128, 128);
    uint8_t* b1l = b1h + tile_bytes(64, 128);
    uint8_t* a2h = b1l + tile_bytes(64, 128);
    uint8_t* a2l = a2h + tile_bytes(128, 64);
    uint8_t* b2h = a2l + tile_bytes(128, 64);
    uint8_t* b2l = b2h + tile_bytes(64, 64);
    float* sO = reinterpret_cast<float*>(base);            // reused after the MMAs: [64][OLD]

    const int c = blockIdx.x, h = blockIdx.y, HV = p.L.HV, HK = p.L.HK;
    const int hk = h / (HV / HK);
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const float* hc = p.h + ((size_t)c * HV + h) * DK * DV;
    // A1(v, kidx) = H[kidx][v]
    stage_along_rows<512>(a1h, a1l, 128, 128, [&](int r, int k8, float (&v)[8]) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = hc[(size_t)(k8 * 8 + e) * DV + r];
    });
    // B1(tok, kidx) = scale q rstd 2^g
    stage_along_k<512>(b1h, b1l, 64, 128, [&](int r, int k8, float (&v)[8]) {
        if (r >= len) { zero8(v); return; }
        const size_t th = (size_t)(start + r) * HV + h, tk = (size_t)(start + r) * HK + hk;
        load8(p.q, p.q_dtype, tk * 128 + k8 * 8, v);
        float g[8];
        load8(p.g_c, MKDA_F32, th * 128 + k8 * 8, g);
        const float m = p.scale * (p.q_rstd ? p.q_rstd[tk] : 1.f);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] *= m * exp2f(g[e]);
    });
    // A2(v, j) = Vd[j][v]
    stage_along_rows<512>(a2h, a2l, 128, 64, [&](int r, int k8, float (&v)[8]) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int j = k8 * 8 + e;
            v[e] = j < len ? p.Vd[((size_t)(start + j) * HV + h) * 128 + r] : 0.f;
        }
    });
    // B2(i, j) = Aqk[i][j]
    stage_along_k<512>(b2h, b2l, 64, 64, [&](int r, int k8, float (&v)[8]) {
        if (r >= len) { zero8(v); return; }
        load8(p.Aqk, MKDA_F32, ((size_t)(start + r) * HV + h) * 64 + k8 * 8, v);
    });
    const uint32_t tmem = tc_operands_ready(&sh);
    if (tid == 0) {
        const uint32_t idesc = umma::idesc_bf16(128, 64);
        umma::gemm_split(tmem, smem_u32(a1h), smem_u32(a1l), 128, smem_u32(b1h), smem_u32(b1l), 64, 128, idesc, 0u);
        umma::gemm_split(tmem, smem_u32(a2h), smem_u32(a2l), 128, smem_u32(b2h), smem_u32(b2l), 64, 64, idesc, 1u);
        umma::commit(&sh.bar);
    }
    umma::mbar_wait(&sh.bar, 0);
    umma::fence_after_sync();
    if (warp < 8) {   // TMEM [v lanes][tok cols] -> shared [tok][v]
        float v[32];
        const int t0 = (warp >> 2) * 32, vi = (warp & 3) * 32 + lane;
        umma::tmem_ld32(umma::tmem_addr(tmem, warp, t0), v);
#pragma unroll
        for (int j = 0; j < 32; ++j) sO[(t0 + j) * OLD + vi] = v[j];
    }
    __syncthreads();
    float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
    if (p.has_norm && p.norm_w) w = ld4(p.norm_w, p.norm_w_dtype, 4 * lane);
    for (int r = warp; r < len; r += 16) {
        float4 o = *reinterpret_cast<const float4*>(sO + r * OLD + 4 * lane);
        const size_t off = ((size_t)(start + r) * HV + h) * 128 + 4 * lane;
        if (p.o_raw) *reinterpret_cast<float4*>(p.o_raw + off) = o;
        if (p.has_norm) {
            float ss = (o.x * o.x + o.y * o.y) + (o.z * o.z + o.w * o.w);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
            const float rs = 1.f / sqrtf(ss * (1.f / 128.f) + p.eps);
            const float4 z = ld4(p.gate, p.gate_dtype, off);
            const float zz[4] = {z.x, z.y, z.z, z.w};
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
    tc_end(&sh, tmem, 64);
}

int tc_chunk_status(unsigned int* out) {
    return cudaMemcpyFromSymbol(out, umma::g_timeout_flag, sizeof(unsigned int)) == cudaSuccess ? 0 : -1;
}

int launch_out_fwd_tc(const MkdaOutFwd* p, cudaStream_t stream) {
    if (int e = ensure_smem((const void*)out_fwd_tc_kernel, OUT_TC_SMEM, "out_fwd")) return e;
    out_fwd_tc_kernel<<<dim3(p->L.NC, p->L.HV), 512, OUT_TC_SMEM, stream>>>(*p);
    return check_launch("out_fwd");
}

}  // namespace mkda

// Chunk-parallel output kernel on the Blackwell tensor cores (tcgen05.mma, TMEM accumulators): work items are
// (chunk, v-head) pairs.  Every product puts a 128-wide dimension (K or V index, or two stacked 64-row operands) on the MMA M
// axis and the chunk rows on N, so all accumulators are [128 lanes x 64 / 128 columns] fp32 tiles in tensor memory.
// Operands either arrive as ready-made tiles by bulk copy (states, Vd, nw, A, Aqk, the scaled q / k) or are produced by
// the CUDA cores (gate scaling, L2 statistics, bf16 hi/lo split) straight into the swizzled tile layout; see umma.cuh.
#include "common.cuh"
#include "host.h"
#include "umma.cuh"

namespace mkda {

using umma::smem_u32;
using umma::store_split8;
using umma::tile_bytes;

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
int tc_chunk_status_clear() {
    const unsigned int z = 0;
    return cudaMemcpyToSymbol(umma::g_timeout_flag, &z, sizeof(z)) == cudaSuccess ? 0 : -1;
}

template <int GDT>
static int launch_out_fwd_tc_t(const MkdaOutFwd* p, cudaStream_t stream) {
    auto kern = out_fwd_tc_kernel<GDT>;
    if (int e = ensure_smem((const void*)kern, OUT_TC_SMEM, "out_fwd")) return e;
    const int items = p->L.NC * p->L.HV;
    kern<<<items < sm_count() ? items : sm_count(), 512, OUT_TC_SMEM, stream>>>(*p);
    return check_launch("out_fwd");
}
int launch_out_fwd_tc(const MkdaOutFwd* p, cudaStream_t stream) {
    switch (p->has_norm ? p->gate_dtype : 0) {
        case MKDA_F32: return launch_out_fwd_tc_t<MKDA_F32>(p, stream);
        case MKDA_BF16: return launch_out_fwd_tc_t<MKDA_BF16>(p, stream);
        case MKDA_F16: return launch_out_fwd_tc_t<MKDA_F16>(p, stream);
    }
    return set_error(MKDA_ERR_ARG, "out_fwd: unsupported dtype");
}

}  // namespace mkda

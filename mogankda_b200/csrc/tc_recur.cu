// Serial state recurrences on the Blackwell tensor cores.
//
// One CTA (16 warps) per (v-head, segment) carries the whole 128 x 128 state, TRANSPOSED, in tensor memory:
// St[v lanes][K-index columns] fp32.  With that orientation every operand that has to be regenerated from the
// accumulators (the state itself, Vd^T) is written by its owning thread as plain 16-byte row chunks of a K-major tile,
// and every operand that comes from global memory is a ready-made tile written by the intra-chunk kernel (nw^T, kbar,
// scale q 2^g, Aqk), fetched by bulk copy and read through a K-major or MN-major view; only u and dO pass through registers.
// Per chunk:   Vd^T[v x tok] = u^T + St nw^T          St <- St diag(gl) + Vd^T kbar
// The forward kernel double-buffers its tiles: the next chunk's copies are in flight while the current products run.
#include "common.cuh"
#include "host.h"
#include "umma.cuh"

namespace mkda {

using umma::store_split8;

struct RecurShared {
    uint64_t bar;
    uint64_t ldw[2];       // arrival of the nw chunk tiles (bulk copies)
    uint64_t ldu;          // arrival of the u chunk tile
    uint32_t tmem;
    float gl[2][DK];
};

__device__ __forceinline__ void publish_operands() {
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
}

constexpr int RECUR_TC_SMEM = 64 * 1024 + 5 * 32 * 1024 + 1024;

__global__ void __launch_bounds__(512, 1) recur_fwd_tc_kernel(const MkdaRecurFwd p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ RecurShared sh;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sAh = base;                         // St as A(m = v, k = K index) [128][128]
    uint8_t* sAl = sAh + 32768;
    uint8_t* sW[2] = {sAl + 32768, sAl + 32768 + 65536};            // nw^T chunk tile [K index][tok] (hi, lo 16 KB each); later Vd^T [v][tok]
    uint8_t* sK[2] = {sW[0] + 32768, sW[1] + 32768};                 // kbar row tile [tok][K index], fetched by bulk copy
    uint8_t* sU = sAl + 32768 + 2 * 65536;                           // u^T chunk tile [v][tok] of the current chunk

    const bool trans = blockIdx.x == 1;
    const int h = blockIdx.y, seg = blockIdx.z, HV = p.L.HV;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, cg = warp >> 2, row = q * 32 + lane;
    const bool vf = p.state_v_first != 0;

    if (warp == 0) umma::tmem_alloc(&sh.tmem, 256);
    if (tid == 0) { umma::mbar_init(&sh.bar, 1); umma::mbar_init(&sh.ldw[0], 1); umma::mbar_init(&sh.ldw[1], 1); umma::mbar_init(&sh.ldu, 1); umma::fence_barrier_init(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = sh.tmem;
    uint32_t phase = 0;

    // Warm-up truncation (a pass from zero only): where the decay accumulated from chunk warm_start to the segment's end
    // hides everything before it, the pass starts there; the transition is then zero and its CTA visits no chunk.
    int c_beg = p.L.seg_chunk_off[seg];
    const int c_end = p.L.seg_chunk_off[seg + 1];
    bool cut = false;
    if (p.warm_start) {
        const int w = p.warm_start[seg * HV + h];
        if (w > c_beg) { cut = true; c_beg = trans ? c_end : w; }
    }
    {   // initial state: columns [32 cg, 32 cg + 32) of row `row`
        float s[32];
        const int h0row = p.seg_h0 ? p.seg_h0[seg] : seg;
        const float* h0 = (!trans && !cut && p.h0 && h0row >= 0) ? p.h0 + ((size_t)h0row * HV + h) * DK * DV : nullptr;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int kk = cg * 32 + j;
            float v = 0.f;
            if (trans) v = (kk == row && !cut) ? 1.f : 0.f;
            else if (h0) v = vf ? h0[(size_t)row * DK + kk] : h0[(size_t)kk * DV + row];
            s[j] = v;
        }
        umma::tmem_st32(umma::tmem_addr(tmem, warp, cg * 32), s);
        umma::tmem_wait_st();
    }

    // nw^T and kbar arrive as the ready-made tiles written by the intra-chunk kernel: two bulk copies per chunk on one
    // barrier (thread 0).  The 128 decay factors of the chunk are read by the first four warps into a register and parked
    // in shared memory at the end of the step: a load stored at once would make those warps (and, at the next barrier,
    // everybody) wait for it in every step of the chain.
    float gl_next = 0.f;
    auto fetch = [&](int c, int buf) {
        const size_t it = (size_t)c * HV + h;
        if (tid == 0) {
            umma::mbar_expect_tx(&sh.ldw[buf], 2 * umma::CHUNK_TILE_BYTES);
            umma::bulk_load(sW[buf], reinterpret_cast<const uint8_t*>(p.nw) + it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ldw[buf]);
            umma::bulk_load(sK[buf], reinterpret_cast<const uint8_t*>(p.kbar) + it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ldw[buf]);
        }
        if (tid < DK) gl_next = p.gl[it * 128 + tid];
    };

    // u^T of a chunk arrives as the chunk tile written by the intra-chunk kernel (one buffer: requested as soon as the
    // previous chunk has consumed its own)
    auto fetch_u = [&](int c) {
        if (tid == 0 && !trans) {
            umma::mbar_expect_tx(&sh.ldu, umma::CHUNK_TILE_BYTES);
            umma::bulk_load(sU, reinterpret_cast<const uint8_t*>(p.u) + ((size_t)c * HV + h) * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ldu);
        }
    };
    if (c_beg < c_end) {
        fetch(c_beg, 0);
        fetch_u(c_beg);
        if (tid < DK) sh.gl[0][tid] = gl_next;
    }
    for (int c = c_beg; c < c_end; ++c) {
        const int buf = (c - c_beg) & 1;
        const bool more = c + 1 < c_end;
        if (tid == 0) umma::bulk_store_wait_read();         // the previous chunk's saved tiles have left shared memory
        if (more) fetch(c + 1, buf ^ 1);                    // ... so the other buffers (last read by chunk c - 1) take the next tiles
        __syncthreads();                                   // sh.gl[buf] is complete; the saved state tile has left
        {   // state entering the chunk: operand tile (optionally saved as it is by the issuing thread below), decay
            float s[32];
            umma::tmem_ld32(umma::tmem_addr(tmem, warp, cg * 32), s);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v8[e] = s[i * 8 + e];
                store_split8(sAh, sAl, 128, row, cg * 4 + i, v8);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) s[j] *= sh.gl[buf][cg * 32 + j];
            umma::tmem_st32(umma::tmem_addr(tmem, warp, cg * 32), s);
            umma::tmem_wait_st();
        }
        publish_operands();
        if (umma::mma_issuer()) {
            umma::mbar_wait(&sh.ldw[buf], ((c - c_beg) >> 1) & 1);            // this chunk's nw and kbar tiles have landed
            umma::gemm(tmem + 128, umma::opnd_k(sAh, sAl, 128), umma::opnd_mn(sW[buf], sW[buf] + 16384, 128), 128, 64, 128, 0u);
            umma::commit(&sh.bar);
        }
        umma::mbar_wait(&sh.bar, phase); phase ^= 1;
        umma::fence_after_sync();
        // The operand tile doubles as the saved state of this chunk: one asynchronous 64 KB copy, issued and later awaited
        // by thread 0, started once the product that reads the tile is done; nothing writes the tile again before the top
        // of the next iteration.
        if (tid == 0 && p.h && !trans)
            umma::bulk_store(reinterpret_cast<uint8_t*>(p.h) + ((size_t)c * HV + h) * umma::STATE_TILE_BYTES, sAh, umma::STATE_TILE_BYTES);
        {   // Vd^T = u^T + St nw^T as the operand tile A(m = v, k = tok)
            float d[16], a0[8], a1[8];
            umma::tmem_ld16(umma::tmem_addr(tmem, warp, 128 + cg * 16), d);
            if (!trans) {
                umma::mbar_wait(&sh.ldu, (c - c_beg) & 1);
                umma::load_tile8(sU, sU + 16384, 128, row, 2 * cg, a0);
                umma::load_tile8(sU, sU + 16384, 128, row, 2 * cg + 1, a1);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) a0[j] = a1[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j < 8) a0[j] += d[j]; else a1[j - 8] += d[j];
            }
            store_split8(sW[buf], sW[buf] + 16384, 128, row, 2 * cg, a0);       // the nw tile is dead: it becomes Vd^T
            store_split8(sW[buf], sW[buf] + 16384, 128, row, 2 * cg + 1, a1);
        }
        publish_operands();
        if (more) fetch_u(c + 1);                           // every thread has read its part of the u tile
        // the Vd^T operand tile is also what the output kernel consumes: saved as it is (columns past the end are zero)
        if (tid == 0 && p.Vd && !trans)
            umma::bulk_store(reinterpret_cast<uint8_t*>(p.Vd) + ((size_t)c * HV + h) * umma::CHUNK_TILE_BYTES, sW[buf], umma::CHUNK_TILE_BYTES);
        if (umma::mma_issuer()) {
            umma::gemm(tmem, umma::opnd_k(sW[buf], sW[buf] + 16384, 128), umma::opnd_mn(sK[buf], sK[buf] + 16384, 64), 128, 128, 64, 1u);
            umma::commit(&sh.bar);
        }
        umma::mbar_wait(&sh.bar, phase); phase ^= 1;
        umma::fence_after_sync();
        if (more && tid < DK) sh.gl[buf ^ 1][tid] = gl_next;   // requested a whole step ago; read after the barrier at the top
    }
    if (tid == 0) umma::bulk_store_wait_read();
    {   // state leaving the segment
        float s[32];
        umma::tmem_ld32(umma::tmem_addr(tmem, warp, cg * 32), s);
        float* out = nullptr;
        if (trans) { if (p.mt) out = p.mt + ((size_t)seg * HV + h) * DK * DK; }
        else if (p.ht) out = p.ht + ((size_t)seg * HV + h) * DK * DV;
        if (out) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int kk = cg * 32 + j;
                // transition: M[K out][K in] with this thread holding row `row` = K in; state: [K][V] or [V][K]
                if (trans || !vf) out[(size_t)kk * DV + row] = s[j];
                else out[(size_t)row * DK + kk] = s[j];
            }
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

int tc_recur_status(unsigned int* out) {
    return cudaMemcpyFromSymbol(out, umma::g_timeout_flag, sizeof(unsigned int)) == cudaSuccess ? 0 : -1;
}
int tc_recur_status_clear() {
    const unsigned int z = 0;
    return cudaMemcpyToSymbol(umma::g_timeout_flag, &z, sizeof(z)) == cudaSuccess ? 0 : -1;
}

int launch_recur_fwd_tc(const MkdaRecurFwd* p, cudaStream_t stream) {
    auto kern = recur_fwd_tc_kernel;
    if (int e = ensure_smem((const void*)kern, RECUR_TC_SMEM, "recur_fwd")) return e;
    kern<<<dim3(p->want_transition ? 2 : 1, p->L.HV, p->L.NS), 512, RECUR_TC_SMEM, stream>>>(*p);
    return check_launch("recur_fwd");
}

}  // namespace mkda

namespace mkda {

// ---------------------------------------------------------------------------------------------------------
// Reverse state-gradient chain on the tensor cores.  dSt[v lanes][K-index columns] (transposed, fp32, TMEM) is the
// gradient of the state leaving the current chunk; per chunk, walking backwards:
//   dVd^T[v x j] = dO^T Aqk + dSt kbar^T                 (saved as a chunk tile, with dO as a row tile, for mkda_bwd_chunk)
//   dSt <- dSt diag(gl) + dO^T (scale q 2^g) + dVd^T nw
// dO, Aqk, kbar, q~ and nw are staged untransposed; the views (K-major / MN-major) supply the transposes.
// ---------------------------------------------------------------------------------------------------------
constexpr int DH_TC_SMEM = 64 * 1024 + 32 * 1024 + 16 * 1024 + 3 * 32 * 1024 + 1024;

// DODT = dtype of the dO rows staged through registers, or DO_TILE: dO arrives as the row tile written by the chunked
// gated-RMSNorm backward and is fetched by bulk copy like the other operands.
constexpr int DO_TILE = 3;
template <int DODT>
__global__ void __launch_bounds__(512, 1) bwd_dh_tc_kernel(const MkdaBwdDh p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ RecurShared sh;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sAh = base;                         // dSt as A(m = v, k = K index)
    uint8_t* sAl = sAh + 32768;
    uint8_t* sDo = sAl + 32768;                  // dO [i][v]          hi 16 KB, lo 16 KB
    uint8_t* sAq = sDo + 32768;                  // Aqk [i][j] quarter tile (hi 8 KB, lo 8 KB), fetched by bulk copy
    uint8_t* sKb = sAq + 16384;                  // kbar row tile [j][K index] (bulk copy); later dVd^T [v][j]
    uint8_t* sQs = sKb + 32768;                  // scale q 2^g row tile [i][K index] (bulk copy)
    uint8_t* sNw = sQs + 32768;                  // nw^T chunk tile [K index][j], fetched by bulk copy

    const int h = blockIdx.y, seg = blockIdx.z, HV = p.L.HV;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, cg = warp >> 2, row = q * 32 + lane;
    const bool vf = p.state_v_first != 0;

    if (warp == 0) umma::tmem_alloc(&sh.tmem, 256);
    if (tid == 0) { umma::mbar_init(&sh.bar, 1); umma::mbar_init(&sh.ldw[0], 1); umma::mbar_init(&sh.ldw[1], 1); umma::fence_barrier_init(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = sh.tmem;
    uint32_t phase = 0;

    // Warm-up truncation (a pass from zero only): the reverse chain starts below chunk warm_end where the decay accumulated
    // over the segment's first chunks hides every later contribution from the segment's entrance.
    const int c_beg = p.L.seg_chunk_off[seg];
    int c_end = p.L.seg_chunk_off[seg + 1];
    bool cut = false;
    if (p.warm_end) {
        const int w = p.warm_end[seg * HV + h];
        if (w < c_end) { cut = true; c_end = w; }
    }
    {
        float s[32];
        const int drow = p.seg_dht ? p.seg_dht[seg] : seg;
        const float* src = (p.dht && drow >= 0 && !cut) ? p.dht + ((size_t)drow * HV + h) * DK * DV : nullptr;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int kk = cg * 32 + j;
            s[j] = src ? (vf ? src[(size_t)row * DK + kk] : src[(size_t)kk * DV + row]) : 0.f;
        }
        umma::tmem_st32(umma::tmem_addr(tmem, warp, cg * 32), s);
        umma::tmem_wait_st();
    }
    // decay factors: the next chunk's are read into a register one iteration ahead and parked in shared memory at the end
    // of the step (a load stored at once would be waited for in every step of the chain)
    float gl_next = 0.f;
    if (c_beg < c_end && tid < DK) sh.gl[0][tid] = p.gl[((size_t)(c_end - 1) * HV + h) * 128 + tid];
    for (int c = c_end - 1; c >= c_beg; --c) {
        const int start = DODT != DO_TILE ? p.L.chunk_start[c] : 0, len = DODT != DO_TILE ? p.L.chunk_len[c] : CH;
        const int par = (c_end - 1 - c) & 1;
        {   // Five of the six operands arrive as ready-made tiles (their last readers, the previous chunk's products, are
            // done): Aqk and kbar for the first product on one barrier, scale q 2^g and nw^T for the second on the other.
            // Only dO goes through registers.
            const size_t it = (size_t)c * HV + h;
            if (tid == 0) {
                umma::bulk_store_wait_read();              // the previous chunk's saved tiles (dS', dO, dVd^T) have left shared memory
                umma::mbar_expect_tx(&sh.ldw[1], umma::QUARTER_TILE_BYTES + umma::CHUNK_TILE_BYTES + (DODT == DO_TILE ? umma::CHUNK_TILE_BYTES : 0u));
                if (DODT == DO_TILE)
                    umma::bulk_load(sDo, reinterpret_cast<const uint8_t*>(p.dO_in_t) + it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ldw[1]);
                umma::bulk_load(sAq, reinterpret_cast<const uint8_t*>(p.Aqk) + it * umma::QUARTER_TILE_BYTES, umma::QUARTER_TILE_BYTES, &sh.ldw[1]);
                umma::bulk_load(sKb, reinterpret_cast<const uint8_t*>(p.kbar) + it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ldw[1]);
                umma::mbar_expect_tx(&sh.ldw[0], 2 * umma::CHUNK_TILE_BYTES);
                umma::bulk_load(sQs, reinterpret_cast<const uint8_t*>(p.qs) + it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ldw[0]);
                umma::bulk_load(sNw, reinterpret_cast<const uint8_t*>(p.nw) + it * umma::CHUNK_TILE_BYTES, umma::CHUNK_TILE_BYTES, &sh.ldw[0]);
            }
            if (c > c_beg && tid < DK) gl_next = p.gl[(it - HV) * 128 + tid];
        }
        float vo[2][8];
        if (DODT != DO_TILE) {
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int i = tid + n * 512, r = i >> 4, k8 = i & 15, rr = r < len ? r : len - 1;
                ld8(p.d_o, DODT == DO_TILE ? MKDA_F32 : DODT, ((size_t)(start + rr) * HV + h) * 128 + k8 * 8, vo[n]);
            }
        }
        __syncthreads();                                   // sh.gl is complete; no copy reads the dO or dS' tile any more
        if (DODT != DO_TILE) {
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int i = tid + n * 512, r = i >> 4, k8 = i & 15;
                if (r >= len) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) vo[n][e] = 0.f;
                }
                store_split8(sDo, sDo + 16384, 64, r, k8, vo[n]);
            }
        }
        {   // gradient leaving the chunk: operand tile (saved as it is by the issuing thread below), decay
            float s[32];
            umma::tmem_ld32(umma::tmem_addr(tmem, warp, cg * 32), s);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v8[e] = s[i * 8 + e];
                store_split8(sAh, sAl, 128, row, cg * 4 + i, v8);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) s[j] *= sh.gl[par][cg * 32 + j];
            umma::tmem_st32(umma::tmem_addr(tmem, warp, cg * 32), s);
            umma::tmem_wait_st();
        }
        publish_operands();
        // the operand tile is also this chunk's saved gradient: one asynchronous 64 KB copy, awaited by the same thread
        // before the tile is rebuilt in the next iteration (measured: starting it here is faster than after the products);
        // the staged dO tile leaves the same way for the chunk-parallel kernel that follows
        if (tid == 0) {
            const size_t it = (size_t)c * HV + h;
            if (p.dh) umma::bulk_store(reinterpret_cast<uint8_t*>(p.dh) + it * umma::STATE_TILE_BYTES, sAh, umma::STATE_TILE_BYTES);
            if (DODT != DO_TILE && p.dO_t) umma::bulk_store(reinterpret_cast<uint8_t*>(p.dO_t) + it * umma::CHUNK_TILE_BYTES, sDo, umma::CHUNK_TILE_BYTES);
        }
        if (umma::mma_issuer()) {
            umma::mbar_wait(&sh.ldw[1], ((c_end - 1 - c) & 1));               // this chunk's Aqk and kbar tiles have landed
            umma::gemm(tmem + 128, umma::opnd_mn(sDo, sDo + 16384, 64), umma::opnd_mn(sAq, sAq + 8192, 64), 128, 64, 64, 0u);
            umma::gemm(tmem + 128, umma::opnd_k(sAh, sAl, 128), umma::opnd_k(sKb, sKb + 16384, 64), 128, 64, 128, 1u);
            umma::commit(&sh.bar);
        }
        umma::mbar_wait(&sh.bar, phase); phase ^= 1;
        umma::fence_after_sync();
        {
            float d[16], a0[8], a1[8];
            umma::tmem_ld16(umma::tmem_addr(tmem, warp, 128 + cg * 16), d);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j < 8) a0[j] = d[j]; else a1[j - 8] = d[j];
            }
            store_split8(sKb, sKb + 16384, 128, row, 2 * cg, a0);              // the kbar tile is dead: it becomes dVd^T
            store_split8(sKb, sKb + 16384, 128, row, 2 * cg + 1, a1);
        }
        publish_operands();
        // dVd^T leaves as the chunk tile just built (token columns past the end are exact zeros: Aqk has no such column
        // and kbar no such row)
        if (tid == 0 && p.dVd_t)
            umma::bulk_store(reinterpret_cast<uint8_t*>(p.dVd_t) + ((size_t)c * HV + h) * umma::CHUNK_TILE_BYTES, sKb, umma::CHUNK_TILE_BYTES);
        if (umma::mma_issuer()) {
            umma::mbar_wait(&sh.ldw[0], ((c_end - 1 - c) & 1));               // this chunk's q and nw tiles have landed
            umma::gemm(tmem, umma::opnd_mn(sDo, sDo + 16384, 64), umma::opnd_mn(sQs, sQs + 16384, 64), 128, 128, 64, 1u);
            umma::gemm(tmem, umma::opnd_k(sKb, sKb + 16384, 128), umma::opnd_k(sNw, sNw + 16384, 128), 128, 128, 64, 1u);
            umma::commit(&sh.bar);
        }
        umma::mbar_wait(&sh.bar, phase); phase ^= 1;
        umma::fence_after_sync();
        if (c > c_beg && tid < DK) sh.gl[par ^ 1][tid] = gl_next;   // requested a whole step ago; read after the barrier at the top
    }
    if (tid == 0) umma::bulk_store_wait_read();
    if (p.dh0) {
        float s[32];
        umma::tmem_ld32(umma::tmem_addr(tmem, warp, cg * 32), s);
        float* out = p.dh0 + ((size_t)seg * HV + h) * DK * DV;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int kk = cg * 32 + j;
            if (vf) out[(size_t)row * DK + kk] = s[j]; else out[(size_t)kk * DV + row] = s[j];
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

template <int DODT>
static int launch_bwd_dh_tc_t(const MkdaBwdDh* p, cudaStream_t stream) {
    auto kern = bwd_dh_tc_kernel<DODT>;
    if (int e = ensure_smem((const void*)kern, DH_TC_SMEM, "bwd_dh")) return e;
    kern<<<dim3(1, p->L.HV, p->L.NS), 512, DH_TC_SMEM, stream>>>(*p);
    return check_launch("bwd_dh");
}
int launch_bwd_dh_tc(const MkdaBwdDh* p, cudaStream_t stream) {
    if (p->dO_in_t) return launch_bwd_dh_tc_t<DO_TILE>(p, stream);
    switch (p->do_dtype) {
        case MKDA_F32: return launch_bwd_dh_tc_t<MKDA_F32>(p, stream);
        case MKDA_BF16: return launch_bwd_dh_tc_t<MKDA_BF16>(p, stream);
        case MKDA_F16: return launch_bwd_dh_tc_t<MKDA_F16>(p, stream);
    }
    return set_error(MKDA_ERR_ARG, "bwd_dh: unsupported dtype");
}

}  // namespace mkda

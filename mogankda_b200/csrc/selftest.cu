// Self-test of the tcgen05 plumbing: D[128 x N] = A[128 x K] * B[N x K]^T with fp32 inputs staged as bf16 hi/lo tiles.
// Exists so that descriptor encodings, the swizzled tile addressing and the TMEM read-back can be checked in
// isolation from the KDA kernels (tests/test_kernels_gpu.py).
#include "common.cuh"
#include "host.h"
#include "umma.cuh"

namespace mkda {

__global__ void __launch_bounds__(128, 1) selftest_umma_kernel(const MkdaSelfTest p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int N = p.N, K = p.K;
    uint8_t* a_hi = base;
    uint8_t* a_lo = a_hi + umma::tile_bytes(128, K);
    uint8_t* b_hi = a_lo + umma::tile_bytes(128, K);
    uint8_t* b_lo = b_hi + umma::tile_bytes(N, K);
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) umma::tmem_alloc(&tmem_slot, 128);
    if (tid == 0) { umma::mbar_init(&bar, 1); umma::fence_barrier_init(); }
    // stage: chunk index i -> (row, 8-column chunk); lanes walk along K for A and along rows for B (both addressings)
    const int a_mn = p.mode & 2, b_mn = p.mode & 1;
    if (!a_mn) {
        for (int i = tid; i < 128 * (K / 8); i += 128) {
            const int r = i / (K / 8), k8 = i % (K / 8);
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = p.A[(size_t)r * K + k8 * 8 + e];
            umma::store_split8(a_hi, a_lo, 128, r, k8, v);
        }
    } else {            // physical tile P[k][m] (K rows, 128 columns)
        for (int i = tid; i < K * 16; i += 128) {
            const int k = i / 16, m8 = i % 16;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = p.A[(size_t)(m8 * 8 + e) * K + k];
            umma::store_split8(a_hi, a_lo, K, k, m8, v);
        }
    }
    if (!b_mn) {
        for (int i = tid; i < N * (K / 8); i += 128) {
            const int r = i % N, k8 = i / N;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = p.B[(size_t)r * K + k8 * 8 + e];
            umma::store_split8(b_hi, b_lo, N, r, k8, v);
        }
    } else {            // physical tile P[k][n] (K rows, N columns)
        for (int i = tid; i < K * (N / 8); i += 128) {
            const int k = i / (N / 8), n8 = i % (N / 8);
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = p.B[(size_t)(n8 * 8 + e) * K + k];
            umma::store_split8(b_hi, b_lo, K, k, n8, v);
        }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = tmem_slot;
    if (tid == 0) {
        const umma::Opnd oa = a_mn ? umma::opnd_mn(a_hi, a_lo, K) : umma::opnd_k(a_hi, a_lo, 128);
        const umma::Opnd ob = b_mn ? umma::opnd_mn(b_hi, b_lo, K) : umma::opnd_k(b_hi, b_lo, N);
        umma::gemm(tmem, oa, ob, 128, N, K, 0u);
        umma::commit(&bar);
    }
    umma::mbar_wait(&bar, 0);
    umma::fence_after_sync();
    for (int c0 = 0; c0 < N; c0 += 32) {
        float v[32];
        umma::tmem_ld32(umma::tmem_addr(tmem, warp, c0), v);
#pragma unroll
        for (int j = 0; j < 32; ++j) p.D[(size_t)tid * N + c0 + j] = v[j];
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 128);
}

// A wait that nothing will ever satisfy: every thread waits on a barrier without arrivals for at most `limit_cycles`,
// reports the expiry in the caller's own status word and leaves in good order (tensor memory released).
__global__ void __launch_bounds__(128, 1) selftest_wait_kernel(const MkdaSelfTestWait p) {
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) umma::tmem_alloc(&tmem_slot, 32);
    if (tid == 0) { umma::mbar_init(&bar, 1); umma::fence_barrier_init(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const bool ok = umma::mbar_wait_limited(&bar, 0, p.limit_cycles, p.status);
    if (ok && tid == 0) p.status[1] = 1u;          // must never happen
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem_slot, 32);
}

int selftest_status(unsigned int* out) {
    return cudaMemcpyFromSymbol(out, umma::g_timeout_flag, sizeof(unsigned int)) == cudaSuccess ? 0 : -1;
}
int selftest_status_clear() {
    const unsigned int z = 0;
    return cudaMemcpyToSymbol(umma::g_timeout_flag, &z, sizeof(z)) == cudaSuccess ? 0 : -1;
}

}  // namespace mkda

using namespace mkda;

extern "C" int mkda_selftest_umma(const MkdaSelfTest* p, void* stream) {
    if (!p || !p->A || !p->B || !p->D) return set_error(MKDA_ERR_ARG, "selftest_umma: null argument");
    if ((p->N != 64 && p->N != 128) || (p->K != 64 && p->K != 128)) return set_error(MKDA_ERR_ARG, "selftest_umma: N, K must be 64 or 128");
    const int smem = 2 * umma::tile_bytes(128, p->K) + 2 * umma::tile_bytes(p->N, p->K) + 1024;
    if (int e = ensure_smem((const void*)selftest_umma_kernel, smem, "selftest_umma")) return e;
    selftest_umma_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(*p);
    return check_launch("selftest_umma");
}

extern "C" int mkda_selftest_wait(const MkdaSelfTestWait* p, void* stream) {
    if (!p || !p->status) return set_error(MKDA_ERR_ARG, "selftest_wait: null argument");
    if (p->limit_cycles < 1 || p->limit_cycles > (1 << 24)) return set_error(MKDA_ERR_ARG, "selftest_wait: limit_cycles must be in [1, 2^24]");
    selftest_wait_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(*p);
    return check_launch("selftest_wait");
}

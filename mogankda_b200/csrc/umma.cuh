// Blackwell tensor-core plumbing used by the *_tc kernels: tcgen05.mma with shared-memory operands in the K-major
// 128-byte-swizzle canonical layout, fp32 accumulators in tensor memory (TMEM), completion through an mbarrier.
//
// Operand precision: every fp32 operand value a is split into two bf16 tiles, hi = bf16(a) and lo = bf16(a - hi), and a
// product is issued as three kind::f16 MMAs (lo*hi + hi*lo + hi*hi) accumulating in fp32.  That carries ~16 mantissa
// bits per operand (relative error ~2^-16 per product) for 1.5x the tensor time of one TF32 MMA, in the same
// shared-memory footprint as an fp32 tile.
//
// Every wait is bounded in time: on expiry the waiter records a timeout in a global status word and goes on
// (results are then garbage but the kernel terminates and frees its TMEM).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace mkda {
namespace umma {

static __device__ unsigned int g_timeout_flag;      // one per translation unit, read back by mkda_device_status()

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- operand tiles -------------------------------------------------------------------------------------------
// A tile holds R rows (multiple of 8) by KT bf16 columns (multiple of 64), K-major.  It is stored as KT/64 column
// blocks of R x 64 (each row 128 bytes, 8-row groups 1024 bytes apart, 16-byte chunks XOR-swizzled with the row
// index).  The tile base must be 1024-byte aligned.
__device__ __forceinline__ uint32_t tile_chunk_offset(int R, int r, int k8) {   // k8 = index of the 8-element chunk
    const int blk = k8 >> 3, c = k8 & 7;
    return (uint32_t)(blk * R * 128 + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}
__host__ __device__ constexpr int tile_bytes(int R, int KT) { return R * KT * 2; }

// split 8 fp32 values into bf16 hi / lo chunks and store them at (row r, chunk k8) of the two tiles
// two fp32 -> packed bf16x2 (lower half = a), one instruction
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
}
__device__ __forceinline__ void store_split8(uint8_t* hi, uint8_t* lo, int R, int r, int k8, const float (&v)[8]) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        h[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
        const float ra = v[2 * i] - __uint_as_float(h[i] << 16);
        const float rb = v[2 * i + 1] - __uint_as_float(h[i] & 0xffff0000u);
        l[i] = pack_bf16x2(ra, rb);
    }
    const uint32_t off = tile_chunk_offset(R, r, k8);
    *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
}

// reconstruct 8 fp32 values from the hi / lo tiles at (row r, chunk k8)
__device__ __forceinline__ void load_tile8(const uint8_t* hi, const uint8_t* lo, int R, int r, int k8, float (&v)[8]) {
    const uint32_t off = tile_chunk_offset(R, r, k8);
    const uint4 a = *reinterpret_cast<const uint4*>(hi + off), b = *reinterpret_cast<const uint4*>(lo + off);
    const uint32_t hw[4] = {a.x, a.y, a.z, a.w}, lw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        v[2 * e] = __uint_as_float(hw[e] << 16) + __uint_as_float(lw[e] << 16);
        v[2 * e + 1] = __uint_as_float(hw[e] & 0xffff0000u) + __uint_as_float(lw[e] & 0xffff0000u);
    }
}

// ---- descriptors ---------------------------------------------------------------------------------------------
// shared-memory matrix descriptor: K-major, SWIZZLE_128B, 8-row groups 1024 B apart (SBO = 64 x 16 B), version 1
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo16 = 1u) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo16 & 0x3FFFu) << 16) | ((uint64_t)64 << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M x N tile
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn = 0, int b_mn = 0) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// An operand as the MMA sees it.  The same physical tile (rows x 64-column blocks, see tile_chunk_offset) can be read
//   K-major : operand(mn = tile row, k = tile column);  `blk` = bytes between 64-column blocks (= rows * 128)
//   MN-major: operand(mn = tile column, k = tile row);  `blk` = bytes between 64-column blocks, which the hardware
//             takes as the distance between 64-element groups of the MN axis (leading byte offset)
// `hi` / `lo` are shared-memory byte addresses of the first row / column the operand uses; lo = 0 means the values
// are exact in bf16 (no second tile).
struct Opnd {
    uint32_t hi, lo, blk;
    int mn;
};
__device__ __forceinline__ Opnd opnd_k(const void* hi, const void* lo, int rows, int first_row = 0) {
    Opnd o;
    o.hi = smem_u32(hi) + first_row * 128;
    o.lo = lo ? smem_u32(lo) + first_row * 128 : 0u;
    o.blk = rows * 128;
    o.mn = 0;
    return o;
}
// MN-major view starting at tile row `first_row` (k origin, multiple of 8) and tile column `first_col` (multiple of 64)
__device__ __forceinline__ Opnd opnd_mn(const void* hi, const void* lo, int rows, int first_row = 0, int first_col = 0) {
    Opnd o;
    const uint32_t off = (first_col >> 6) * rows * 128 + first_row * 128;
    o.hi = smem_u32(hi) + off;
    o.lo = lo ? smem_u32(lo) + off : 0u;
    o.blk = rows * 128;
    o.mn = 1;
    return o;
}
__device__ __forceinline__ uint64_t opnd_desc(const Opnd& o, uint32_t base, int ks) {
    if (o.mn) return make_desc(base + ks * 2048, o.blk >> 4);
    return make_desc(base + (ks >> 2) * o.blk + (ks & 3) * 32);
}

// D[M x N] (+)= A[M x 16] * B[N x 16]^T, one elected thread
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// D[M x N] (+)= A B^T over KT (multiple of 16) with the hi/lo split; products whose lo tile is absent are skipped.
// The four base descriptors are built once; a k-step only adds its byte offset (>> 4) to the start-address field, so
// the issuing thread spends a handful of instructions per MMA (KT is a literal at every call site: the loop unrolls).
__device__ __forceinline__ uint64_t opnd_base_desc(const Opnd& o, uint32_t addr) {
    return o.mn ? make_desc(addr, o.blk >> 4) : make_desc(addr);
}
__device__ __forceinline__ uint32_t opnd_step16(const Opnd& o, int ks) {       // offset of k-step ks in 16-byte units
    return o.mn ? (uint32_t)(ks * 128) : (uint32_t)(((ks >> 2) * o.blk + (ks & 3) * 32) >> 4);
}
__device__ __forceinline__ void gemm(uint32_t tmem_d, const Opnd& a, const Opnd& b, int M, int N, int KT, uint32_t accumulate) {
    const uint32_t idesc = idesc_bf16(M, N, a.mn, b.mn);
    const uint64_t ah = opnd_base_desc(a, a.hi), al = opnd_base_desc(a, a.lo);
    const uint64_t bh = opnd_base_desc(b, b.hi), bl = opnd_base_desc(b, b.lo);
#pragma unroll
    for (int ks = 0; ks < KT / 16; ++ks) {
        const uint32_t ao = opnd_step16(a, ks), bo = opnd_step16(b, ks);
        if (a.lo) { mma_bf16(tmem_d, al + ao, bh + bo, idesc, accumulate); accumulate = 1u; }
        if (b.lo) { mma_bf16(tmem_d, ah + ao, bl + bo, idesc, accumulate); accumulate = 1u; }
        mma_bf16(tmem_d, ah + ao, bh + bo, idesc, accumulate);
        accumulate = 1u;
    }
}

// ---- synchronisation -----------------------------------------------------------------------------------------
// True in exactly one thread of warp 0 (call with warp 0 converged).  The warp index comes from a shuffle and the lane
// from elect.sync, so the compiler sees a warp-uniform branch around the MMA issue and can keep the descriptors and
// addresses in uniform registers, where tcgen05.mma takes them, instead of moving them over per instruction.
__device__ __forceinline__ bool mma_issuer() {
    const int w = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    if (w != 0) return false;
    __syncwarp();
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// make generic-proxy shared-memory writes visible to the tensor core (async proxy)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrive on `bar` once every tcgen05 operation issued so far by this thread has completed
__device__ __forceinline__ void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
// Waits for the phase of `bar` with the given parity, for at most `limit` SM clock cycles.  On expiry 1 is written to
// `*flag` and false is returned: the caller goes on (with garbage) to its exit, so a launch never hangs.  try_wait parks
// the thread for at most the hinted microsecond per attempt, so waiting warps do not compete for issue slots with the
// thread issuing MMAs.
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, long long limit, unsigned int* flag) {
    const uint32_t addr = smem_u32(bar);
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(addr), "r"(parity), "r"(1000u) : "memory");
        if (ok) return true;
        if (clock64() - t0 > limit) break;
    }
    atomicExch(flag, 1u);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    // Bounded by wall time (SM clock): ~70 ms for the first wait that fails on a device, ~35 us afterwards, so a broken
    // launch drains quickly instead of serialising one long timeout per CTA.  The flag stays set until
    // mkda_device_status_clear().
    const long long limit = *(volatile unsigned int*)&g_timeout_flag ? (1ll << 16) : (1ll << 27);
    return mbar_wait_limited(bar, parity, limit, &g_timeout_flag);
}

// ---- bulk copies of whole operand tiles ---------------------------------------------------------------------------
// Per-chunk states travel between kernels as ready-made operand tiles ("state tile": hi tile then lo tile of the
// transposed state, rows = v, K-major over the K index, 2 x 32 KB), so a consumer fills its shared-memory operand with one
// asynchronous copy and no register staging, and the producer writes it straight from the tile it built for its own MMA.
constexpr uint32_t STATE_TILE_BYTES = 65536;
// "chunk tile": a [128][64 tokens] operand (hi 16 KB, lo 16 KB), e.g. Vd^T [v][tok], handed over the same way
constexpr uint32_t CHUNK_TILE_BYTES = 32768;
// "quarter tile": a [64][64] operand (hi 8 KB, lo 8 KB): the intra-chunk matrices A and Aqk [row][column]
constexpr uint32_t QUARTER_TILE_BYTES = 16384;
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// global -> shared, completion counted in bytes on `bar`; addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Tiled copy of one 64 x 128 box of a row tensor (host.h: make_rows_map) starting at element column x (x times the element
// size a multiple of 16 bytes) and row y; lands as a dense [64][128] block at the 128-byte aligned `smem_dst`, completion
// counted in bytes (the whole box, rows past the tensor's end included) on `bar`.
__device__ __forceinline__ void tma_load_rows(void* smem_dst, const void* tmap, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// shared -> global; the source must stay untouched until bulk_store_wait_read() returns in the issuing thread
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// Hint: bring `bytes` (multiple of 16) from the 16-byte aligned global address into L2; nothing waits for it.
__device__ __forceinline__ void l2_prefetch(const void* gsrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(gsrc), "r"(bytes) : "memory");
}

// One thread: initialise `bar` and start the asynchronous fetch of state tile `idx` of the array `tiles` into `smem_dst`
// (1024-byte aligned).  Waiters use mbar_wait(bar, 0) after a CTA-wide barrier that follows this call.
__device__ __forceinline__ void fetch_state_tile(uint64_t* bar, void* smem_dst, const void* tiles, size_t idx) {
    mbar_init(bar, 1);
    fence_barrier_init();
    mbar_expect_tx(bar, STATE_TILE_BYTES);
    bulk_load(smem_dst, static_cast<const uint8_t*>(tiles) + idx * STATE_TILE_BYTES, STATE_TILE_BYTES, bar);
}

// ---- tensor memory -------------------------------------------------------------------------------------------
// one full warp allocates `ncols` (power of two >= 32) columns and publishes the base address through `slot`
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 columns: thread t of the warp receives columns [col, col+32) of TMEM lane (quadrant base + t)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        :: "r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
           "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
           "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
           "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
           "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
           "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
           "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
           "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
// TMEM address of (lane quadrant of this warp, column)
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int warp, int col) {
    return base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)col;
}

}  // namespace umma
}  // namespace mkda

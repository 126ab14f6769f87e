// HBM-bound elementwise / scan kernels around the chunk contractions:
//   gate activation + chunk-local cumsum (forward), gate backward with the reverse cumsum folded in,
//   L2-norm statistics, GVA group sum + L2-norm backward, gated RMSNorm backward, deterministic partial reductions.
// All of them move each tensor once with 128-bit accesses; one warp covers one 128-wide row.
#include "common.cuh"
#include <stdio.h>

#include "host.h"

namespace mkda {

__device__ __forceinline__ float4 splat4(float a) { return make_float4(a, a, a, a); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 scale4(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
__device__ __forceinline__ float hsum4(float4 a) { return (a.x + a.y) + (a.z + a.w); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// natural-log decay for one element; s = x + dt_bias, E = exp(A_log), lb = lower bound (< 0)
__device__ __forceinline__ float gate_value(int mode, float s, float E, float lb) {
    if (mode == MKDA_GATE_GDN) return fmaxf(-E * softplusf_(s), lb);
    if (mode == MKDA_GATE_KIMI) return lb * sigmoidf_(E * s);
    if (mode == MKDA_GATE_EDA) return lb + (-lb) * expf_(-(E / fabsf(lb)) * softplusf_(s));
    return s;
}
// d gate / d s  and  d gate / d A_log
__device__ __forceinline__ void gate_grad(int mode, float s, float E, float lb, float& ds, float& dA) {
    if (mode == MKDA_GATE_GDN) {
        const float sp = softplusf_(s);
        const float keep = (-E * sp >= lb) ? 1.f : 0.f;    // clamp passes no gradient
        ds = keep * (-E) * sigmoidf_(s);
        dA = keep * (-E) * sp;
    } else if (mode == MKDA_GATE_KIMI) {
        const float u = E * s, sg = sigmoidf_(u), d = lb * sg * (1.f - sg);
        ds = d * E;
        dA = d * u;
    } else if (mode == MKDA_GATE_EDA) {
        const float sp = softplusf_(s), c = E / fabsf(lb), w = expf_(-c * sp), d = lb * w * c;
        ds = d * sigmoidf_(s);
        dA = d * sp;
    } else {
        ds = 1.f;
        dA = 0.f;
    }
}

// ---------------------------------------------------------------------------------------------------------
// forward: grid NC x HV, heads fastest so that CTAs running together read one contiguous token range; 128 threads.  Warp w owns rows 16w..16w+15 of the chunk, lane l channels 4l..4l+3.
// The chunk-local inclusive sum is (sum of the earlier warps' totals, in warp order) + (running sum inside the
// warp): the association depends only on the row index, never on later rows.
// ---------------------------------------------------------------------------------------------------------
template <int XDT>
__global__ void __launch_bounds__(128, 5) gate_cumsum_fwd_kernel(const MkdaGateFwd p) {
    const int HV = p.L.HV, c = blockIdx.x / HV, h = blockIdx.x - c * HV;
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ float4 tot[4][32];
    const float E = p.A_log ? expf(p.A_log[h]) : 1.f;
    float4 bias = splat4(0.f);
    if (p.dt_bias) bias = p.scalar_gate ? splat4(p.dt_bias[h]) : *reinterpret_cast<const float4*>(p.dt_bias + h * 128 + 4 * lane);
    float4 vals[16];
    // all 16 rows of this warp are requested before the first one is used (rows past the end re-read the last one)
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int row = warp * 16 + r, rr = row < len ? row : len - 1;
        const size_t th = (size_t)(start + rr) * HV + h;
        vals[r] = p.scalar_gate ? splat4(ld1(p.x, XDT, th)) : ld4(p.x, XDT, th * 128 + 4 * lane);
    }
    float4 run = splat4(0.f);
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int row = warp * 16 + r;
        float4 gv = splat4(0.f);
        if (row < len) {
            const float4 xv = add4(vals[r], bias);
            gv.x = gate_value(p.mode, xv.x, E, p.lower_bound);
            gv.y = gate_value(p.mode, xv.y, E, p.lower_bound);
            gv.z = gate_value(p.mode, xv.z, E, p.lower_bound);
            gv.w = gate_value(p.mode, xv.w, E, p.lower_bound);
        }
        run = add4(run, gv);
        vals[r] = run;
    }
    tot[warp][lane] = run;
    __syncthreads();
    float4 pre = splat4(0.f);
    for (int w = 0; w < warp; ++w) pre = add4(pre, tot[w][lane]);
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int row = warp * 16 + r;
        if (row < len) {
            const size_t th = (size_t)(start + row) * HV + h;
            *reinterpret_cast<float4*>(p.g_c + th * 128 + 4 * lane) = scale4(add4(pre, vals[r]), RCP_LN2);
        }
    }
    if (p.beta_raw && threadIdx.x < len) {
        const size_t th = (size_t)(start + threadIdx.x) * HV + h;
        const float b = ld1(p.beta_raw, p.beta_dtype, th);
        p.beta_out[th] = p.beta_sigmoid ? p.beta_scale * sigmoidf_(b) : b;
    }
}

// ---------------------------------------------------------------------------------------------------------
// backward: same tiling; suffix sums instead of prefix sums.
// ---------------------------------------------------------------------------------------------------------
// CTA (h, g), heads fastest, walks chunks g, g + gridDim.y, ... and keeps the parameter-gradient partials in registers, so the second
// stage only has gridDim.y rows to add (fixed assignment and order: deterministic).
// 16 warps of four rows each: 64 registers per thread, so two CTAs (half of the SM's thread slots) are resident and their
// loads, special-function work and stores overlap (four warps of sixteen rows needed 128 registers: a quarter of the slots).
constexpr int GB_WARPS = 16, GB_ROWS = CH / GB_WARPS;
template <int XDT>
__global__ void __launch_bounds__(32 * GB_WARPS, 2) gate_bwd_kernel(const MkdaGateBwd p) {
    const int h = blockIdx.x, HV = p.L.HV;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ float4 tot[GB_WARPS][32];
    __shared__ float4 red[2][GB_WARPS][32];
    const float E = p.A_log ? expf(p.A_log[h]) : 1.f;
    float4 bias = splat4(0.f);
    if (p.dt_bias) bias = p.scalar_gate ? splat4(p.dt_bias[h]) : *reinterpret_cast<const float4*>(p.dt_bias + h * 128 + 4 * lane);
    float4 pa = splat4(0.f), pb = splat4(0.f);
    for (int c = blockIdx.y; c < p.L.NC; c += gridDim.y) {
        const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
        float4 vals[GB_ROWS], xs[GB_ROWS];
#pragma unroll
        for (int r = 0; r < GB_ROWS; ++r) {
            const int row = warp * GB_ROWS + r, rr = row < len ? row : len - 1;
            vals[r] = *reinterpret_cast<const float4*>(p.dgp + (((size_t)c * HV + h) * CH + rr) * 128 + 4 * lane);
            const size_t th = (size_t)(start + rr) * HV + h;
            xs[r] = p.scalar_gate ? splat4(ld1(p.x, XDT, th)) : ld4(p.x, XDT, th * 128 + 4 * lane);
        }
        float4 run = splat4(0.f);
#pragma unroll
        for (int r = GB_ROWS - 1; r >= 0; --r) {
            if (warp * GB_ROWS + r < len) run = add4(run, vals[r]);
            vals[r] = run;
        }
        __syncthreads();                                   // previous chunk's readers of tot are done
        tot[warp][lane] = run;
        __syncthreads();
        float4 post = splat4(0.f);
        for (int w = GB_WARPS - 1; w > warp; --w) post = add4(post, tot[w][lane]);
#pragma unroll
        for (int r = 0; r < GB_ROWS; ++r) {
            const int row = warp * GB_ROWS + r;
            if (row >= len) continue;                       // warp-uniform
            const size_t th = (size_t)(start + row) * HV + h;
            const float4 dg = add4(vals[r], post);
            if (p.scalar_gate) {
                const float dgs = warp_sum(hsum4(dg));
                float ds, dA;
                gate_grad(p.mode, xs[r].x + bias.x, E, p.lower_bound, ds, dA);
                const float dxs = dgs * ds;
                if (lane == 0) st1(p.dx, p.dx_dtype, th, dxs);
                pb.x += dxs;
                pa.x += dgs * dA;
            } else {
                const float4 xv = add4(xs[r], bias);
                float4 ds, dA;
                gate_grad(p.mode, xv.x, E, p.lower_bound, ds.x, dA.x);
                gate_grad(p.mode, xv.y, E, p.lower_bound, ds.y, dA.y);
                gate_grad(p.mode, xv.z, E, p.lower_bound, ds.z, dA.z);
                gate_grad(p.mode, xv.w, E, p.lower_bound, ds.w, dA.w);
                const float4 dxv = mul4(dg, ds);
                st4(p.dx, p.dx_dtype, th * 128 + 4 * lane, dxv);
                pb = add4(pb, dxv);
                pa = add4(pa, mul4(dg, dA));
            }
        }
    }
    if (!p.part_bias && !p.part_alog) return;
    red[0][warp][lane] = pb;
    red[1][warp][lane] = pa;
    __syncthreads();
    if (warp == 0) {
        float4 sb = red[0][0][lane], sa = red[1][0][lane];
        for (int w = 1; w < GB_WARPS; ++w) { sb = add4(sb, red[0][w][lane]); sa = add4(sa, red[1][w][lane]); }
        const size_t ch = (size_t)blockIdx.y * HV + h;
        if (p.scalar_gate) {
            if (lane == 0) {
                if (p.part_bias) p.part_bias[ch] = sb.x;
                if (p.part_alog) p.part_alog[ch] = sa.x;
            }
        } else {
            if (p.part_bias) *reinterpret_cast<float4*>(p.part_bias + ch * 128 + 4 * lane) = sb;
            if (p.part_alog) *reinterpret_cast<float4*>(p.part_alog + ch * 128 + 4 * lane) = sa;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// deterministic second-stage reductions
// ---------------------------------------------------------------------------------------------------------
// group == 1: block (32, 8); thread (x, y) sums rows y, y+8, ... of column j (four running sums, so that four loads are
// in flight), then the 8 partials are added in order.
__global__ void __launch_bounds__(256) reduce_cols_kernel(const float* __restrict__ in, int rows, int cols, float* __restrict__ out) {
    __shared__ float part[8][33];
    const int j = blockIdx.x * 32 + threadIdx.x;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (j < cols) {
        int r = threadIdx.y;
        for (; r + 24 < rows; r += 32) {
            s0 += in[(size_t)r * cols + j];
            s1 += in[(size_t)(r + 8) * cols + j];
            s2 += in[(size_t)(r + 16) * cols + j];
            s3 += in[(size_t)(r + 24) * cols + j];
        }
        for (; r < rows; r += 8) s0 += in[(size_t)r * cols + j];
    }
    part[threadIdx.y][threadIdx.x] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (threadIdx.y == 0 && j < cols) {
        float t = part[0][threadIdx.x];
        for (int y = 1; y < 8; ++y) t += part[y][threadIdx.x];
        out[j] = t;
    }
}
// group > 1: one block of 128 threads per output; warp w walks rows w, w+4, ... and its lanes the group's elements, again
// with four running sums; lanes, then warps, are combined in a fixed order.
__global__ void __launch_bounds__(128) reduce_groups_kernel(const float* __restrict__ in, int rows, int cols, int group, float* __restrict__ out) {
    __shared__ float part[4];
    const int j = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = lane; i < group; i += 32) {
        const float* col = in + (size_t)j * group + i;
        int r = warp;
        for (; r + 12 < rows; r += 16) {
            s0 += col[(size_t)r * cols];
            s1 += col[(size_t)(r + 4) * cols];
            s2 += col[(size_t)(r + 8) * cols];
            s3 += col[(size_t)(r + 12) * cols];
        }
        for (; r < rows; r += 4) s0 += col[(size_t)r * cols];
    }
    const float s = warp_sum((s0 + s1) + (s2 + s3));
    if (lane == 0) part[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) out[j] = (part[0] + part[1]) + (part[2] + part[3]);
}

// ---------------------------------------------------------------------------------------------------------
// L2-norm statistics: 16 lanes per row of 128, eight rows per warp.
// ---------------------------------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(128) l2norm_rstd_kernel(const MkdaL2Norm p) {
    const int lane = threadIdx.x & 31, sub = lane & 15;
    const int row0 = (blockIdx.x * 4 + (threadIdx.x >> 5)) * 8 + (lane >> 4);
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + 2 * i, rr = row < p.rows ? row : p.rows - 1;
        a[i] = ld4(p.x, DT, (size_t)rr * 128 + 8 * sub);
        b[i] = ld4(p.x, DT, (size_t)rr * 128 + 8 * sub + 4);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float ss = hsum4(mul4(a[i], a[i])) + hsum4(mul4(b[i], b[i]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const int row = row0 + 2 * i;
        if (sub == 0 && row < p.rows) p.rstd[row] = 1.f / sqrtf(ss + p.eps);
    }
}

// L2-norm backward of the q / k gradients.  Block (chunk, q/k head, which of q / k); warp w takes rows w, w + 4, ... of the
// chunk.  The gradients arrive as the fp32 [64][128] tiles of the chunk backward, already summed over the v-heads of the
// q/k head (the chunk backward adds them up where it writes them).
__global__ void __launch_bounds__(128) qk_grad_finish_kernel(const MkdaQkGrad p) {
    const int HK = p.L.HK;
    const int c = blockIdx.x / HK, hk = blockIdx.x - c * HK, which = blockIdx.y;
    const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* d_v = (which ? p.dk_v : p.dq_v) + ((size_t)c * HK + hk) * CH * 128 + 4 * lane;
    const void* x = which ? p.k : p.q;
    const float* rstd = which ? p.k_rstd : p.q_rstd;
    void* dx = which ? p.dk : p.dq;
    for (int r0 = warp; r0 < len; r0 += 16) {
        float4 s[4], xr[4];
        float rs[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {                      // four rows in flight per warp
            const int r = r0 + 4 * u, rr = r < len ? r : len - 1;
            const size_t rowi = (size_t)(start + rr) * HK + hk;
            s[u] = *reinterpret_cast<const float4*>(d_v + (size_t)rr * 128);
            if (rstd) {
                rs[u] = rstd[rowi];
                xr[u] = ld4(x, p.x_dtype, rowi * 128 + 4 * lane);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int r = r0 + 4 * u;
            if (r >= len) break;                           // warp-uniform
            const size_t rowi = (size_t)(start + r) * HK + hk;
            float4 t = s[u];
            if (rstd) {
                const float4 y = scale4(xr[u], rs[u]);
                const float dot = warp_sum(hsum4(mul4(t, y)));
                t = make_float4((t.x - dot * y.x) * rs[u], (t.y - dot * y.y) * rs[u], (t.z - dot * y.z) * rs[u], (t.w - dot * y.w) * rs[u]);
            }
            st4(dx, p.x_dtype, rowi * 128 + 4 * lane, t);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// gated RMSNorm backward: block of 4 warps covers 64 rows (warp w rows w, w+4, ...); per-block weight partials.
//   n = o rs, rs = rsqrt(mean o^2 + eps);  y = n w a(z);  dn = dy w a;  do = rs (dn - n mean(dn n));
//   dz = dy n w a'(z);  dw = sum dy n a
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) epilogue_bwd_kernel(const MkdaEpilogueBwd p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ float4 red[4][32];
    float4 w = splat4(1.f);
    if (p.norm_w) w = ld4(p.norm_w, p.norm_w_dtype, 4 * lane);
    float4 dw = splat4(0.f);
    const int ngroups = (p.rows + 63) / 64;
    for (int grp = blockIdx.x; grp < ngroups; grp += gridDim.x)
    for (int i = 0; i < 16; ++i) {
        const int row = grp * 64 + i * 4 + warp;
        if (row >= p.rows) break;
        const size_t off = (size_t)row * 128 + 4 * lane;
        const float4 o = *reinterpret_cast<const float4*>(p.o_raw + off);
        const float4 dy = ld4(p.dy, p.dy_dtype, off);
        const float4 z = ld4(p.gate, p.gate_dtype, off);
        const float rs = 1.f / sqrtf(warp_sum(hsum4(mul4(o, o))) * (1.f / 128.f) + p.eps);
        float a[4], da[4];
        const float zz[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float sg = sigmoidf_(zz[e]);
            if (p.act == MKDA_ACT_SILU) { a[e] = zz[e] * sg; da[e] = sg * (1.f + zz[e] * (1.f - sg)); }
            else { a[e] = sg; da[e] = sg * (1.f - sg); }
        }
        const float4 n = scale4(o, rs);
        const float4 av = make_float4(a[0], a[1], a[2], a[3]), dav = make_float4(da[0], da[1], da[2], da[3]);
        const float4 dn = mul4(mul4(dy, w), av);
        const float m = warp_sum(hsum4(mul4(dn, n))) * (1.f / 128.f);
        const float4 dov = make_float4(rs * (dn.x - n.x * m), rs * (dn.y - n.y * m), rs * (dn.z - n.z * m), rs * (dn.w - n.w * m));
        *reinterpret_cast<float4*>(p.d_o + off) = dov;
        st4(p.dgate, p.dgate_dtype, off, mul4(mul4(mul4(dy, n), w), dav));
        dw = add4(dw, mul4(mul4(dy, n), av));
    }
    if (!p.part_w) return;
    red[warp][lane] = dw;
    __syncthreads();
    if (warp == 0) {
        float4 s = red[0][lane];
        for (int k = 1; k < 4; ++k) s = add4(s, red[k][lane]);
        *reinterpret_cast<float4*>(p.part_w + (size_t)blockIdx.x * 128 + 4 * lane) = s;
    }
}

// ---------------------------------------------------------------------------------------------------------
// gated RMSNorm backward, chunk-structured: the same arithmetic as epilogue_bwd_kernel, but dO leaves as the bf16 hi / lo
// row tile [64 tokens][128] per (chunk, v-head) that the tensor-core kernels of the backward pass fetch by bulk copy
// (rows past the end of the chunk are zero), instead of as fp32 rows that each of them would have to convert again.
// CTA b walks the items b, b + gridDim.x, ...; half a warp covers one row of 128 (8 values per lane = one 16-byte piece
// of the tile), a warp two rows at a time.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// DYMODE: how dy is addressed: 0 = dense rows (16-byte loads), 1 = one value per row (column stride 0), 2 = any strides
template <int DYMODE>
__global__ void __launch_bounds__(128) epilogue_bwd_tiles_kernel(const MkdaEpilogueBwdTiles p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & 15, hw = lane >> 4;
    __shared__ float red[8][128];
    const int HV = p.L.HV, total = p.L.NC * HV;
    float w8[8], dw8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { w8[e] = 1.f; dw8[e] = 0.f; }
    if (p.norm_w) ld8(p.norm_w, p.norm_w_dtype, 8 * sub, w8);
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
        const int c = item / HV, h = item - c * HV;
        const int start = p.L.chunk_start[c], len = p.L.chunk_len[c];
        uint8_t* tile = reinterpret_cast<uint8_t*>(p.dO_t) + (size_t)item * 32768;
#pragma unroll 2
        for (int it = 0; it < 8; ++it) {
            const int r = it * 8 + warp * 2 + hw;
            const uint32_t toff = ((sub >> 3) * 64 * 128) + (r >> 3) * 1024 + (r & 7) * 128 + (((sub & 7) ^ (r & 7)) << 4);
            // rows past the end re-read the last valid row (so that the shuffles below run unconditionally) and are zeroed
            const bool valid = r < len;
            const size_t off = ((size_t)(start + (valid ? r : len - 1)) * HV + h) * 128 + 8 * sub;
            float o[8], dy[8], z[8], dov[8];
            ld8(p.o_raw, MKDA_F32, off, o);
            {
                const size_t drow = ((size_t)(start + (valid ? r : len - 1)) * HV + h) * (size_t)p.dy_row_stride;
                if (DYMODE == 0) {
                    ld8(p.dy, p.dy_dtype, drow + 8 * sub, dy);
                } else if (DYMODE == 1) {
                    const float d = ld1(p.dy, p.dy_dtype, drow);
#pragma unroll
                    for (int e = 0; e < 8; ++e) dy[e] = d;
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) dy[e] = ld1(p.dy, p.dy_dtype, drow + (size_t)(8 * sub + e) * p.dy_col_stride);
                }
            }
            ld8(p.gate, p.gate_dtype, off, z);
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(o[e], o[e], ss);
            const float rs = 1.f / sqrtf(half_warp_sum(ss) * (1.f / 128.f) + p.eps);
            float n[8], dn[8], dz[8], m = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float sg = sigmoidf_(z[e]);
                float a, da;
                if (p.act == MKDA_ACT_SILU) { a = z[e] * sg; da = sg * (1.f + z[e] * (1.f - sg)); }
                else { a = sg; da = sg * (1.f - sg); }
                n[e] = o[e] * rs;
                dn[e] = dy[e] * w8[e] * a;
                m = fmaf(dn[e], n[e], m);
                dz[e] = dy[e] * n[e] * w8[e] * da;
                if (valid) dw8[e] = fmaf(dy[e] * n[e], a, dw8[e]);
            }
            m = half_warp_sum(m) * (1.f / 128.f);
#pragma unroll
            for (int e = 0; e < 8; ++e) dov[e] = valid ? rs * (dn[e] - n[e] * m) : 0.f;
            if (valid) {
                st4(p.dgate, p.dgate_dtype, off, make_float4(dz[0], dz[1], dz[2], dz[3]));
                st4(p.dgate, p.dgate_dtype, off + 4, make_float4(dz[4], dz[5], dz[6], dz[7]));
            }
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 hb = __floats2bfloat162_rn(dov[2 * e], dov[2 * e + 1]);
                hi[e] = *reinterpret_cast<uint32_t*>(&hb);
                const float ra = dov[2 * e] - __uint_as_float(hi[e] << 16);
                const float rb = dov[2 * e + 1] - __uint_as_float(hi[e] & 0xffff0000u);
                __nv_bfloat162 lb = __floats2bfloat162_rn(ra, rb);
                lo[e] = *reinterpret_cast<uint32_t*>(&lb);
            }
            *reinterpret_cast<uint4*>(tile + toff) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(tile + 16384 + toff) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
    }
    if (!p.part_w) return;
    // per-CTA partial of d weight: the eight (warp, half) partials of every column, added in a fixed order
#pragma unroll
    for (int e = 0; e < 8; ++e) red[warp * 2 + hw][8 * sub + e] = dw8[e];
    __syncthreads();
    float t = red[0][threadIdx.x];
#pragma unroll
    for (int k = 1; k < 8; ++k) t += red[k][threadIdx.x];
    p.part_w[(size_t)blockIdx.x * 128 + threadIdx.x] = t;
}

// Warm-up truncation table: one CTA per (segment, v-head), one thread per key channel (see MkdaWarmup).
// gl = 2^gL may have underflowed to zero: log2 gives -inf, i.e. fully decayed.
__global__ void __launch_bounds__(128) warmup_chunks_kernel(const MkdaWarmup p) {
    const int seg = blockIdx.x, h = blockIdx.y, ch = threadIdx.x, HV = p.L.HV;
    const int c_beg = p.L.seg_chunk_off[seg], c_end = p.L.seg_chunk_off[seg + 1];
    int ws = c_beg, we = c_end;
    float acc = 0.f;
    for (int c = c_end - 1; c > c_beg; --c) {              // forward pass: decay from chunk c to the segment's end
        acc += log2f(p.gl[((size_t)c * HV + h) * 128 + ch]);
        if (__syncthreads_and(acc < p.threshold_log2)) { ws = c; break; }
    }
    acc = 0.f;
    for (int c = c_beg; c < c_end - 1; ++c) {              // reverse pass: decay from the segment's start through chunk c
        acc += log2f(p.gl[((size_t)c * HV + h) * 128 + ch]);
        if (__syncthreads_and(acc < p.threshold_log2)) { we = c + 1; break; }
    }
    if (ch == 0) {
        p.warm_start[seg * HV + h] = ws;
        p.warm_end[seg * HV + h] = we;
    }
}

}  // namespace mkda

using namespace mkda;

// number of weight-gradient partial rows (= CTAs) of the gated RMSNorm backward
static int epilogue_part_rows(int rows) {
    const int groups = (rows + 63) / 64;
    return groups < MKDA_EPILOGUE_MAX_PART_ROWS ? groups : MKDA_EPILOGUE_MAX_PART_ROWS;
}

extern "C" int mkda_warmup_chunks(const MkdaWarmup* p, void* stream) {
    if (!p || !p->gl || !p->warm_start || !p->warm_end || !p->L.seg_chunk_off) return set_error(MKDA_ERR_ARG, "warmup_chunks: null argument");
    if (!(p->threshold_log2 < 0.f)) return set_error(MKDA_ERR_ARG, "warmup_chunks: the threshold must be negative");
    if (p->L.NS == 0 || p->L.HV == 0) return MKDA_OK;
    warmup_chunks_kernel<<<dim3(p->L.NS, p->L.HV), 128, 0, (cudaStream_t)stream>>>(*p);
    return check_launch("warmup_chunks");
}

extern "C" int mkda_gate_cumsum_fwd(const MkdaGateFwd* p, void* stream) {
    if (!p || !p->x || !p->g_c || p->L.NC < 0) return set_error(MKDA_ERR_ARG, "gate_cumsum_fwd: null argument");
    if (any_misaligned(p->g_c) || (!p->scalar_gate && any_misaligned(p->x, p->dt_bias))) return set_error(MKDA_ERR_ARG, "gate_cumsum_fwd: tensors must be 16-byte aligned");
    if (p->mode != MKDA_GATE_PRECOMPUTED && !(p->lower_bound < 0.f)) return set_error(MKDA_ERR_ARG, "gate_cumsum_fwd: lower_bound must be < 0");
    if (p->beta_raw && !p->beta_out) return set_error(MKDA_ERR_ARG, "gate_cumsum_fwd: beta_out missing");
    if (p->L.NC == 0) return MKDA_OK;
    const int grid = p->L.NC * p->L.HV;
    switch (p->x_dtype) {
        case MKDA_F32: gate_cumsum_fwd_kernel<MKDA_F32><<<grid, 128, 0, (cudaStream_t)stream>>>(*p); break;
        case MKDA_BF16: gate_cumsum_fwd_kernel<MKDA_BF16><<<grid, 128, 0, (cudaStream_t)stream>>>(*p); break;
        case MKDA_F16: gate_cumsum_fwd_kernel<MKDA_F16><<<grid, 128, 0, (cudaStream_t)stream>>>(*p); break;
        default: return set_error(MKDA_ERR_ARG, "gate_cumsum_fwd: unsupported dtype");
    }
    return check_launch("gate_cumsum_fwd");
}

extern "C" int mkda_gate_bwd(const MkdaGateBwd* p, void* stream) {
    if (!p || !p->x || !p->dgp || !p->dx) return set_error(MKDA_ERR_ARG, "gate_bwd: null argument");
    if (any_misaligned(p->dgp) || (!p->scalar_gate && any_misaligned(p->x, p->dx, p->dt_bias))) return set_error(MKDA_ERR_ARG, "gate_bwd: tensors must be 16-byte aligned");
    if (p->L.NC == 0) return MKDA_OK;
    if (p->part_rows < 1) return set_error(MKDA_ERR_ARG, "gate_bwd: part_rows must be >= 1");
    const dim3 grid(p->L.HV, p->part_rows < p->L.NC ? p->part_rows : p->L.NC);
    if ((p->part_bias || p->part_alog) && (int)grid.y != p->part_rows)
        return set_error(MKDA_ERR_ARG, "gate_bwd: part_rows must not exceed the number of chunks when partials are requested");
    switch (p->x_dtype) {
        case MKDA_F32: gate_bwd_kernel<MKDA_F32><<<grid, 32 * GB_WARPS, 0, (cudaStream_t)stream>>>(*p); break;
        case MKDA_BF16: gate_bwd_kernel<MKDA_BF16><<<grid, 32 * GB_WARPS, 0, (cudaStream_t)stream>>>(*p); break;
        case MKDA_F16: gate_bwd_kernel<MKDA_F16><<<grid, 32 * GB_WARPS, 0, (cudaStream_t)stream>>>(*p); break;
        default: return set_error(MKDA_ERR_ARG, "gate_bwd: unsupported dtype");
    }
    return check_launch("gate_bwd");
}

extern "C" int mkda_reduce_partials(const MkdaReduce* p, void* stream) {
    if (!p || !p->in || !p->out || p->group < 1 || p->cols % p->group) return set_error(MKDA_ERR_ARG, "reduce_partials: bad argument");
    if (p->cols == 0) return MKDA_OK;
    if (p->group == 1)
        reduce_cols_kernel<<<(p->cols + 31) / 32, dim3(32, 8), 0, (cudaStream_t)stream>>>(p->in, p->rows, p->cols, p->out);
    else
        reduce_groups_kernel<<<p->cols / p->group, 128, 0, (cudaStream_t)stream>>>(p->in, p->rows, p->cols, p->group, p->out);
    return check_launch("reduce_partials");
}

extern "C" int mkda_l2norm_rstd(const MkdaL2Norm* p, void* stream) {
    if (!p || !p->x || !p->rstd) return set_error(MKDA_ERR_ARG, "l2norm_rstd: null argument");
    if (any_misaligned(p->x)) return set_error(MKDA_ERR_ARG, "l2norm_rstd: x must be 16-byte aligned");
    if (p->rows == 0) return MKDA_OK;
    const int grid = (p->rows + 31) / 32;
    switch (p->dtype) {
        case MKDA_F32: l2norm_rstd_kernel<MKDA_F32><<<grid, 128, 0, (cudaStream_t)stream>>>(*p); break;
        case MKDA_BF16: l2norm_rstd_kernel<MKDA_BF16><<<grid, 128, 0, (cudaStream_t)stream>>>(*p); break;
        case MKDA_F16: l2norm_rstd_kernel<MKDA_F16><<<grid, 128, 0, (cudaStream_t)stream>>>(*p); break;
        default: return set_error(MKDA_ERR_ARG, "l2norm_rstd: unsupported dtype");
    }
    return check_launch("l2norm_rstd");
}

extern "C" int mkda_qk_grad_finish(const MkdaQkGrad* p, void* stream) {
    if (!p || !p->dq_v || !p->dk_v || !p->dq || !p->dk || !p->q || !p->k || p->L.HK <= 0 || p->L.HV % p->L.HK)
        return set_error(MKDA_ERR_ARG, "qk_grad_finish: bad argument");
    if (any_misaligned(p->dq_v, p->dk_v, p->dq, p->dk, p->q, p->k)) return set_error(MKDA_ERR_ARG, "qk_grad_finish: tensors must be 16-byte aligned");
    if (p->L.NC == 0) return MKDA_OK;
    const dim3 grid(p->L.NC * p->L.HK, 2);
    qk_grad_finish_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(*p);
    return check_launch("qk_grad_finish");
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant of the gated RMSNorm backward: the per-block weight-gradient partials live in a static device
// array instead of a caller-provided buffer, and the second-stage reduction is launched here as well.
// `g_noalloc_scratch` names the array for DEVICE code; on the host the same identifier is only a handle, so the host
// asks the runtime for the array's device address (once per device) and passes that pointer to the kernels.
// ---------------------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_noalloc_scratch[(MKDA_NOALLOC_MAX_ROWS / 64) * 128];
static_assert(MKDA_NOALLOC_MAX_ROWS / 64 >= MKDA_EPILOGUE_MAX_PART_ROWS, "the built-in scratch must hold every partial row");
static float* g_noalloc_ptr[64] = {nullptr};          // device address of the scratch, per device ordinal

static int noalloc_scratch(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return set_error(MKDA_ERR_LAUNCH, "epilogue_bwd_noalloc: cannot identify the current device");
    if (!g_noalloc_ptr[dev]) {
        float* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) {
            (void)cudaGetLastError();
            return set_error(MKDA_ERR_LAUNCH, "epilogue_bwd_noalloc: cudaGetSymbolAddress failed for the built-in scratch");
        }
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return MKDA_OK;
}

extern "C" int mkda_epilogue_bwd_noalloc(const MkdaEpilogueBwdNoAlloc* p, void* stream) {
    if (!p || !p->dy || !p->o_raw || !p->gate || !p->d_o || !p->dgate || !p->dweight)
        return set_error(MKDA_ERR_ARG, "epilogue_bwd_noalloc: null argument");
    if (p->rows < 0 || p->rows > MKDA_NOALLOC_MAX_ROWS)
    {
        static char msg[192];
        snprintf(msg, sizeof(msg), "epilogue_bwd_noalloc: rows exceeds the built-in scratch (MKDA_NOALLOC_MAX_ROWS = %d); "
                                   "use mkda_epilogue_bwd with a caller-provided part_w", MKDA_NOALLOC_MAX_ROWS);
        return set_error(MKDA_ERR_ARG, msg);
    }
    float* scratch = nullptr;
    if (int e = noalloc_scratch(&scratch)) return e;
    const int nblk = epilogue_part_rows(p->rows);
    if (nblk == 0) {
        if (cudaMemsetAsync(p->dweight, 0, 128 * sizeof(float), (cudaStream_t)stream) != cudaSuccess)
            return set_error(MKDA_ERR_LAUNCH, "epilogue_bwd_noalloc: memset failed");
        return MKDA_OK;
    }
    MkdaEpilogueBwd q;
    q.rows = p->rows; q.dy = p->dy; q.dy_dtype = p->dy_dtype; q.o_raw = p->o_raw; q.norm_w = p->norm_w;
    q.norm_w_dtype = p->norm_w_dtype; q.gate = p->gate; q.gate_dtype = p->gate_dtype; q.act = p->act; q.eps = p->eps;
    q.d_o = p->d_o; q.dgate = p->dgate; q.dgate_dtype = p->dgate_dtype;
    q.part_w = scratch;                 // every block overwrites its whole row: nothing has to be cleared first
    epilogue_bwd_kernel<<<nblk, 128, 0, (cudaStream_t)stream>>>(q);
    if (int e = check_launch("epilogue_bwd_noalloc")) return e;
    reduce_cols_kernel<<<4, dim3(32, 8), 0, (cudaStream_t)stream>>>(scratch, nblk, 128, p->dweight);
    return check_launch("epilogue_bwd_noalloc (reduce)");
}

extern "C" int mkda_epilogue_bwd_tiles(const MkdaEpilogueBwdTiles* p, void* stream) {
    if (!p || !p->dy || !p->o_raw || !p->gate || !p->dO_t || !p->dgate) return set_error(MKDA_ERR_ARG, "epilogue_bwd_tiles: null argument");
    if (any_misaligned(p->o_raw, p->gate, p->norm_w, p->dO_t, p->dgate) || (p->dy_col_stride == 1 && any_misaligned(p->dy)))
        return set_error(MKDA_ERR_ARG, "epilogue_bwd_tiles: tensors must be 16-byte aligned");
    if (p->dy_row_stride < 0 || p->dy_col_stride < 0 || (p->dy_col_stride == 1 && p->dy_row_stride % 8))
        return set_error(MKDA_ERR_ARG, "epilogue_bwd_tiles: dy strides must be >= 0 (row stride a multiple of 8 when the rows are dense)");
    const int items = p->L.NC * p->L.HV;
    if (items == 0) return MKDA_OK;
    const int grid = items < MKDA_EPILOGUE_MAX_PART_ROWS ? items : MKDA_EPILOGUE_MAX_PART_ROWS;
    if (p->part_w && p->part_rows != grid) return set_error(MKDA_ERR_ARG, "epilogue_bwd_tiles: part_rows must be min(NC * HV, MKDA_EPILOGUE_MAX_PART_ROWS)");
    if (p->dy_col_stride == 1) epilogue_bwd_tiles_kernel<0><<<grid, 128, 0, (cudaStream_t)stream>>>(*p);
    else if (p->dy_col_stride == 0) epilogue_bwd_tiles_kernel<1><<<grid, 128, 0, (cudaStream_t)stream>>>(*p);
    else epilogue_bwd_tiles_kernel<2><<<grid, 128, 0, (cudaStream_t)stream>>>(*p);
    return check_launch("epilogue_bwd_tiles");
}

extern "C" int mkda_epilogue_bwd(const MkdaEpilogueBwd* p, void* stream) {
    if (!p || !p->dy || !p->o_raw || !p->gate || !p->d_o || !p->dgate) return set_error(MKDA_ERR_ARG, "epilogue_bwd: null argument");
    if (p->rows == 0) return MKDA_OK;
    epilogue_bwd_kernel<<<epilogue_part_rows(p->rows), 128, 0, (cudaStream_t)stream>>>(*p);
    return check_launch("epilogue_bwd");
}

/* C ABI of libmkda: hand-written sm_100a kernels for chunked Kimi Delta Attention (per-channel gate) and the
 * gated delta rule (scalar gate), forward and backward.
 *
 * Conventions
 *  - Every entry point takes a pointer to a plain parameter struct and a CUDA stream (passed as void*), launches
 *    on that stream and returns 0 on success or a negative MKDA_ERR_* code; mkda_last_error() gives the text.
 *    Nothing is allocated or freed by the library: every buffer (inputs, outputs, workspaces) belongs to the caller.
 *    Inputs are never written.  No exception crosses this boundary.
 *  - Tokens are addressed in the flattened [TT = B*T] space.  Per-token tensors are row-major
 *    [TT, heads, 128] (or [TT, heads, 64] for the chunk-local matrices, [TT, heads] for scalars).
 *  - A "chunk" is up to 64 consecutive tokens of ONE sequence; chunk ids are sequence-major.  chunk_start[c] is the
 *    flattened index of its first token and chunk_len[c] (1..64) its number of valid rows.  This is the layout the
 *    reference builds in mogan_kda/utils/index.py:93-116 (prepare_chunk_indices / prepare_chunk_offsets).
 *  - A "segment" is a run of consecutive chunks of one sequence processed by one serial recurrence
 *    (seg_chunk_off[s] .. seg_chunk_off[s+1]); without context parallelism a segment is a whole sequence.
 *  - Key dim = value dim = 128, chunk = 64 (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:18,46).
 *  - States are fp32 [.., HV, 128(K), 128(V)]; with state_v_first the caller-visible ones are [.., HV, V, K]
 *    (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:38-40).  Per-chunk states h / dh are always [K, V].
 */
#ifndef MKDA_H_
#define MKDA_H_

#ifdef __cplusplus
extern "C" {
#endif

enum { MKDA_F32 = 0, MKDA_BF16 = 1, MKDA_F16 = 2 };
enum { MKDA_GATE_PRECOMPUTED = 0, MKDA_GATE_EDA = 1, MKDA_GATE_KIMI = 2, MKDA_GATE_GDN = 3 };
enum { MKDA_ACT_SILU = 0, MKDA_ACT_SIGMOID = 1 };
enum { MKDA_OK = 0, MKDA_ERR_ARG = -1, MKDA_ERR_LAUNCH = -2 };

/* Chunk / segment tables shared by all kernels (device pointers, int32). */
typedef struct {
    int TT;                    /* flattened tokens */
    int NC;                    /* chunks */
    int NS;                    /* segments */
    int HK;                    /* q/k heads */
    int HV;                    /* v heads (HV % HK == 0) */
    const int* chunk_start;    /* [NC] */
    const int* chunk_len;      /* [NC] */
    const int* seg_chunk_off;  /* [NS+1] */
} MkdaLayout;

/* Fused gate activation + chunk-local cumsum (log2 domain) + optional beta activation.
 * Replaces kda_gate_cumsum_fwd (mogan_kda/ops/kimi_delta_rule/gate.py:378-406), _beta
 * (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:184-189) and, for a scalar gate, chunk_local_cumsum
 * (mogan_kda/ops/utils/cumsum.py:296-373) with the result broadcast over the 128 channels. */
typedef struct {
    MkdaLayout L;
    const void* x; int x_dtype; int scalar_gate;   /* [TT,HV,128] or [TT,HV] */
    const float* A_log;                            /* [HV] or NULL (=0) */
    const float* dt_bias;                          /* [HV*128] ([HV] if scalar_gate) or NULL */
    int mode; float lower_bound;
    const void* beta_raw; int beta_dtype;          /* [TT,HV] or NULL (skip beta) */
    int beta_sigmoid; float beta_scale;
    float* beta_out;                               /* [TT,HV] fp32 */
    float* g_c;                                    /* [TT,HV,128] fp32 */
} MkdaGateFwd;
int mkda_gate_cumsum_fwd(const MkdaGateFwd* p, void* stream);

/* Gate backward with the chunk-local reverse cumsum folded in; per-chunk partials for the parameter gradients.
 * Replaces kda_gate_bwd (mogan_kda/ops/kimi_delta_rule/gate.py:409-459, dg_is_prime=True) and K5
 * (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:120-124). */
typedef struct {
    MkdaLayout L;
    const void* x; int x_dtype; int scalar_gate;
    const float* A_log; const float* dt_bias;
    int mode; float lower_bound;
    const float* dgp;          /* [NC,HV] fp32 [64][128] tiles: gradient w.r.t. the log2 cumsum as written by mkda_bwd_chunk */
    void* dx; int dx_dtype;    /* [TT,HV,128] or [TT,HV] */
    int part_rows;             /* number of partial rows R (1 <= R <= NC): chunk c accumulates into row c % R */
    float* part_bias;          /* [R,HV,128] ([R,HV] scalar) partial sums of d/d(x+bias), or NULL */
    float* part_alog;          /* same shape, partial sums of d/dA_log, or NULL */
} MkdaGateBwd;
int mkda_gate_bwd(const MkdaGateBwd* p, void* stream);

/* out[j] = sum_r sum_{i<group} in[r*cols + j*group + i], fixed summation tree (deterministic).  Second stage of
 * every parameter-gradient reduction (mogan_kda/ops/kimi_delta_rule/gate.py:452-458, epilogue.py:204). */
typedef struct {
    const float* in; int rows; int cols; int group;
    float* out;                /* [cols/group] */
} MkdaReduce;
int mkda_reduce_partials(const MkdaReduce* p, void* stream);

/* rstd[r] = rsqrt(sum_c x[r,c]^2 + eps) for rows of 128.  Replaces l2norm_fwd (mogan_kda/utils/math.py:22-35);
 * the normalised rows themselves are never materialised (consumers multiply by rstd in fp32). */
typedef struct {
    const void* x; int dtype; int rows; float eps;
    float* rstd;
} MkdaL2Norm;
int mkda_l2norm_rstd(const MkdaL2Norm* p, void* stream);

/* Chunk-parallel WY preparation.  Per (chunk, v-head): decayed K K^T and Q K^T with per-16-row anchoring, the
 * unit-lower-triangular inverse, and the two products the recurrence consumes.
 * Replaces kkt_solve_kda (mogan_kda/ops/kimi_delta_rule/chunk/hopper/kkt_solve_kda.py:546-623) and bwd_w_kda
 * (.../hopper/bwd_prep.py:317-347); with scalar_gate the gate-free K K^T with the decay applied afterwards, as kkt_solve +
 * the G scaling of fused_gdr_fwd do (mogan_kda/ops/gated_delta_rule/chunk/blackwell/kkt_solve.py:105-121,
 * blackwell/fused_fwd.py:425-445). */
typedef struct {
    MkdaLayout L;
    const void* q; const void* k; const void* v; int qkv_dtype;
    const float* q_rstd; const float* k_rstd;      /* [TT,HK] or NULL */
    const float* g_c; const float* beta;           /* [TT,HV,128], [TT,HV] */
    int scalar_gate;           /* 1: g_c holds the same value in all 128 channels of a (token, head) (one decay per token, as
                                * mkda_gate_cumsum_fwd writes it for a [TT,HV] gate): the scalar-gate path is taken, which
                                * accepts any decay <= 0; 0: per-channel path, contract: decay >= -5 per token */
    float scale;
    float* A;      /* [NC,HV] quarter tiles: (I + strictlower(diag(beta) Gamma))^-1 */
    float* Aqk;    /* [NC,HV] quarter tiles: scale * lower(Q K^T with decay) */
    float* nw;     /* [NC,HV] chunk tiles: nw^T [K index][token], nw = -A (beta k 2^g) */
    float* u;      /* [NC,HV] chunk tiles: u^T [v][token], u = A (beta v) */
    float* kbar;   /* [NC,HV] row tiles: k 2^(gL - g) with gL the cumsum at the chunk's last token */
    float* qs;     /* [NC,HV] row tiles: scale q 2^g */
    float* gl;     /* [NC,HV,128] 2^gL, the decay of the state over the whole chunk */
} MkdaIntraFwd;
int mkda_intra_fwd(const MkdaIntraFwd* p, void* stream);

/* State tile: how the per-chunk states `h` (state entering a chunk) and `dh` (gradient of the state leaving it) travel
 * between the kernels.  One tile per (chunk, v-head), MKDA_STATE_TILE_BYTES each, is the tensor-core operand itself: the
 * transposed state [v][K index] split into bf16 hi (first 32 KB) and lo = bf16(x - hi) (second 32 KB); each half is two
 * column blocks (K index 0-63, 64-127) of 128 rows x 128 bytes, 8-row groups 1024 bytes apart, with the eight 16-byte
 * chunks of a row XOR-swizzled by (row & 7).  Producers write it with one asynchronous copy from shared memory and
 * consumers fetch it the same way; hi + lo carries 16 mantissa bits, which is what the products consume anyway.
 * The buffers are typed float* only for size ([NC,HV,128,128] floats = NC*HV tiles). */
#define MKDA_STATE_TILE_BYTES 65536
/* Chunk tile: the same idea for a [128][64 tokens] operand, MKDA_CHUNK_TILE_BYTES per (chunk, v-head): bf16 hi (16 KB)
 * then lo (16 KB), 128 rows x 128 bytes each, same swizzle.  Used for Vd^T [v][token] between mkda_recur_fwd and mkda_out_fwd
 * (token columns past the end of the chunk are zero), for nw^T [K index][token] and u^T [v][token]
 * between mkda_intra_fwd and the serial kernels, and for dVd^T [v][token] between mkda_bwd_dh and mkda_bwd_chunk.
 * Row tile: the same 32 KB for a [64 tokens][128] operand (rows = tokens; hi 16 KB then lo 16 KB, each two column blocks of
 * 64 rows x 128 bytes): the scaled operands kbar and qs, token rows past the end of the chunk are zero. */
#define MKDA_CHUNK_TILE_BYTES 32768
/* Quarter tile: a [64][64] operand, MKDA_QUARTER_TILE_BYTES per (chunk, v-head): bf16 hi (8 KB) then lo (8 KB), 64 rows x
 * 128 bytes, same swizzle.  Used for the intra-chunk matrices A and Aqk, [row i][column j]; rows past the end of the chunk
 * are identity rows in A and zero rows in Aqk. */
#define MKDA_QUARTER_TILE_BYTES 16384

/* Serial state recurrence per (segment, v-head):  Vd = u + nw S;  S <- diag(gl) S + kbar^T Vd.
 * With want_transition a second CTA per (segment, v-head) carries the segment's K x K transition matrix (same
 * recurrence with u = 0 started from the identity).  Replaces the state part of fused_fwd_kda
 * (mogan_kda/ops/kimi_delta_rule/chunk/hopper/fused_fwd.py:523-616) and, for context parallelism, the role of
 * fused_gdr_h (mogan_kda/ops/gated_delta_rule/chunk/blackwell/prepare_h.py:336-403). */
typedef struct {
    MkdaLayout L;
    const float* nw;           /* [NC,HV] chunk tiles as written by mkda_intra_fwd */
    const float* u;            /* [NC,HV] chunk tiles as written by mkda_intra_fwd */
    const float* kbar;         /* [NC,HV] row tiles as written by mkda_intra_fwd */
    const float* gl;           /* [NC,HV,128] as written by mkda_intra_fwd */
    const float* h0;           /* [*,HV,128,128] or NULL */
    const int* seg_h0;         /* [NS] row of h0 for each segment, -1 = start from zero; NULL = identity map */
    int state_v_first;         /* layout of h0 / ht */
    float* h;                  /* [NC,HV] state tiles: state entering each chunk, or NULL */
    float* Vd;                 /* [NC,HV] chunk tiles: Vd^T, or NULL */
    float* ht;                 /* [NS,HV,128,128] state leaving each segment, or NULL */
    int want_transition;
    float* mt;                 /* [NS,HV,128,128] transition (row = output K index), needs want_transition */
    const int* warm_start;     /* [NS,HV] from mkda_warmup_chunks, or NULL.  A pass from zero (the segment pre-pass) may start
                                * at this chunk instead of the segment's first one; where it does, the transition is written
                                * as zero without being computed. */
} MkdaRecurFwd;
int mkda_recur_fwd(const MkdaRecurFwd* p, void* stream);

/* Chunk-parallel output  o = qs h + Aqk Vd  (qs = scale q 2^g) with the optional gated RMSNorm epilogue fused.
 * Replaces the output part of fused_fwd_kda and rmsnorm_gated_fwd
 * (mogan_kda/ops/kimi_delta_rule/epilogue.py:183-190). */
typedef struct {
    MkdaLayout L;
    const float* qs;           /* [NC,HV] row tiles (scale q 2^g) as written by mkda_intra_fwd */
    const float* Aqk;          /* [NC,HV] quarter tiles as written by mkda_intra_fwd */
    const float* Vd;           /* [NC,HV] chunk tiles as written by mkda_recur_fwd */
    const float* h;            /* [NC,HV] state tiles */
    int has_norm; const void* norm_w; int norm_w_dtype;   /* [128] or NULL (=1) */
    const void* gate; int gate_dtype;                     /* [TT,HV,128] */
    int act; float eps;
    float* o_raw;              /* [TT,HV,128] fp32 pre-norm output kept for the backward, or NULL */
    void* out; int out_dtype;  /* [TT,HV,128] */
} MkdaOutFwd;
int mkda_out_fwd(const MkdaOutFwd* p, void* stream);

/* Gated RMSNorm backward.  Replaces rmsnorm_gated_bwd (mogan_kda/ops/kimi_delta_rule/epilogue.py:193-205). */
/* CTA b of the gated RMSNorm backward walks the 64-row groups b, b + R, ... and writes one partial row. */
#define MKDA_EPILOGUE_MAX_PART_ROWS 1184
typedef struct {
    int rows;                  /* TT*HV */
    const void* dy; int dy_dtype;
    const float* o_raw;
    const void* norm_w; int norm_w_dtype;
    const void* gate; int gate_dtype;
    int act; float eps;
    float* d_o;                /* [rows,128] fp32 */
    void* dgate; int dgate_dtype;
    float* part_w;             /* [min(ceil(rows/64), MKDA_EPILOGUE_MAX_PART_ROWS),128] partial sums of d weight, or NULL */
} MkdaEpilogueBwd;
int mkda_epilogue_bwd(const MkdaEpilogueBwd* p, void* stream);

/* Gated RMSNorm backward for the chunked backward pass: the same arithmetic as mkda_epilogue_bwd, addressed through the
 * chunk tables; dO leaves as the row tile per (chunk, v-head) that mkda_bwd_dh and mkda_bwd_chunk fetch by bulk copy (rows
 * past the end of a chunk are zero) instead of as fp32 rows.  CTA b walks the (chunk, head) items b, b + part_rows, ... and
 * writes one partial row of d weight.  Replaces rmsnorm_gated_bwd (mogan_kda/ops/kimi_delta_rule/epilogue.py:193-205). */
typedef struct {
    MkdaLayout L;
    const void* dy; int dy_dtype;                  /* element (row, c) of [TT*HV, 128] at dy[row * dy_row_stride + c * dy_col_stride] */
    int dy_row_stride; int dy_col_stride;          /* in elements: (128, 1) for a contiguous gradient; a gradient that autograd
                                                    * hands over as a broadcast view (strides 0) is read as it is, not copied */
    const float* o_raw;                            /* [TT,HV,128] */
    const void* norm_w; int norm_w_dtype;
    const void* gate; int gate_dtype;
    int act; float eps;
    float* dO_t;               /* [NC,HV] row tiles */
    void* dgate; int dgate_dtype;                  /* [TT,HV,128]; tokens outside every chunk are not written */
    int part_rows;             /* min(NC * HV, MKDA_EPILOGUE_MAX_PART_ROWS) */
    float* part_w;             /* [part_rows,128] partial sums of d weight, or NULL */
} MkdaEpilogueBwdTiles;
int mkda_epilogue_bwd_tiles(const MkdaEpilogueBwdTiles* p, void* stream);

/* Gated RMSNorm backward for callers that cannot allocate.  It has no counterpart in the reference (whose wrapper
 * creates the per-block weight-gradient partials with torch.empty on every call).
 *
 * Who needs it: a host that fixed its device-memory plan before the step starts -- a runtime whose caching allocator is
 * frozen after warm-up, an engine that carved one arena at start-up, a thread that must not take the allocator lock.
 * Such a caller can still provide the inputs and the outputs, but it cannot produce the [R, 128] fp32
 * scratch that mkda_epilogue_bwd wants in `part_w`, nor the second launch's workspace.  This entry point keeps that
 * scratch inside the library, in one file-scope device array of MKDA_NOALLOC_MAX_ROWS / 64 * 128 floats (2 MiB) that
 * every GPU which loads the library holds until the process exits, and it also runs the second-stage reduction, so
 * `dweight` [128] comes back finished.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *  - rows > MKDA_NOALLOC_MAX_ROWS is rejected with MKDA_ERR_ARG ("... exceeds the built-in scratch ...").
 *  - The first call on each device looks up the device address of the scratch array (cudaGetSymbolAddress, with that
 *    device current) and caches it; make that first call before any stream capture is opened.
 *  - All calls share the one array and it keeps whatever the last call left.  Nothing in it has to start at zero:
 *    every row the reduction reads was written by the same call.  Two calls that overlap on the GPU (different
 *    streams, or different host threads) race on it: serialise them.
 *  - d_o, dgate, dweight are bit-identical to mkda_epilogue_bwd + mkda_reduce_partials on the same inputs. */
#define MKDA_NOALLOC_MAX_ROWS 262144
typedef struct {
    int rows;                  /* TT*HV, at most MKDA_NOALLOC_MAX_ROWS */
    const void* dy; int dy_dtype;
    const float* o_raw;
    const void* norm_w; int norm_w_dtype;
    const void* gate; int gate_dtype;
    int act; float eps;
    float* d_o;                /* [rows,128] fp32 */
    void* dgate; int dgate_dtype;
    float* dweight;            /* [128] fp32, finished sum */
} MkdaEpilogueBwdNoAlloc;
int mkda_epilogue_bwd_noalloc(const MkdaEpilogueBwdNoAlloc* p, void* stream);

/* Reverse state chain per (segment, v-head, 64-column block).
 * Replaces bwd_dh_kda (mogan_kda/ops/kimi_delta_rule/chunk/hopper/bwd_dh.py:390-448). */
typedef struct {
    MkdaLayout L;
    const void* d_o; int do_dtype;                 /* [TT,HV,128], or NULL when dO_in_t is given */
    const float* dO_in_t;      /* [NC,HV] row tiles of dO as written by mkda_epilogue_bwd_tiles, or NULL (then d_o is staged
                                * through registers and, if dO_t is given, written there in tile form) */
    const float* kbar;         /* [NC,HV] row tiles as written by mkda_intra_fwd */
    const float* qs;           /* [NC,HV] row tiles as written by mkda_intra_fwd */
    const float* gl;           /* [NC,HV,128] as written by mkda_intra_fwd */
    const float* Aqk;          /* [NC,HV] quarter tiles as written by mkda_intra_fwd */
    const float* nw;           /* [NC,HV] chunk tiles as written by mkda_intra_fwd */
    const float* dht;          /* [*,HV,128,128] or NULL */
    const int* seg_dht;        /* [NS] row of dht per segment, -1 = zero; NULL = identity map */
    int state_v_first;         /* layout of dht / dh0 */
    float* dh;                 /* [NC,HV] state tiles: gradient of the state leaving each chunk, or NULL (not stored) */
    float* dVd_t;              /* [NC,HV] chunk tiles: dVd^T [v][token] (token columns past the end are zero), or NULL */
    float* dO_t;               /* [NC,HV] row tiles: dO [token][v] as staged for the products (zero rows past the end), or NULL */
    float* dh0;                /* [NS,HV,128,128] gradient of the state entering each segment, or NULL */
    const int* warm_end;       /* [NS,HV] from mkda_warmup_chunks, or NULL: a reverse pass from zero (the segment pre-pass)
                                * may start below this chunk index instead of at the segment's last chunk */
} MkdaBwdDh;
int mkda_bwd_dh(const MkdaBwdDh* p, void* stream);

/* Every gradient that is local to a (chunk, v-head) once the state gradients are known, in one kernel:
 *  - through Vd = A diag(beta)(V - k~ S): dv, the WY part of dbeta, dAqk and dL (K3a of bwd_post_kda,
 *    mogan_kda/ops/kimi_delta_rule/chunk/hopper/bwd_post.py:72-400);
 *  - through the states: the row-local parts of dq, dk and of the gate gradient (K3b, .../bwd_post.py:412-766);
 *  - through the decayed K K^T / Q K^T blocks (bwd_intra_kda, .../hopper/bwd_intra.py:529-600);
 *  - the beta activation derivative (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:256-258).
 * dX, dAqk, dL, the WY part of dbeta and the row-local partials, which the reference passes between those kernels through
 * HBM, stay in shared / tensor memory.  Every tile operand (h, dh, Vd, A, dO, dVd) arrives by bulk copy. */
typedef struct {
    MkdaLayout L;
    const void* q; const void* k; const void* v; int qkv_dtype; const float* q_rstd; const float* k_rstd;
    const float* g_c; const float* beta;
    int scalar_gate;           /* as in MkdaIntraFwd */
    const float* A;            /* [NC,HV] quarter tiles as written by mkda_intra_fwd */
    const float* h; const float* dh;               /* state tiles, see MKDA_STATE_TILE_BYTES */
    const float* Vd;           /* [NC,HV] chunk tiles as written by mkda_recur_fwd in the forward pass */
    const float* dO_t;         /* [NC,HV] row tiles as written by mkda_bwd_dh or mkda_epilogue_bwd_tiles */
    const float* dVd_t;        /* [NC,HV] chunk tiles as written by mkda_bwd_dh */
    float scale;
    const void* beta_raw; int beta_dtype; int beta_sigmoid; float beta_scale;
    float* dq_v; float* dk_v;  /* [NC,HK] fp32 [64 tokens][128] tiles per (chunk, q/k head): the contributions of the HV / HK
                                * v-heads of the head are added up in the tile (first one stored, the others added in
                                * order, by the one CTA that owns the head's group); rows past the end are zero */
    float* dgp;                /* [NC,HV] tiles of the same form per (chunk, v-head): gradient w.r.t. the log2 cumsum */
    void* dbeta; int dbeta_dtype;
    void* dv;                  /* [TT,HV,128] in qkv_dtype */
} MkdaBwdChunk;
int mkda_bwd_chunk(const MkdaBwdChunk* p, void* stream);

/* Sum over the v-heads sharing a q/k head, then L2-norm backward; writes dq and dk in the input dtype (one launch for
 * both).  Replaces group_reduce_vector (mogan_kda/ops/utils/group_reduce.py:60-79) and l2norm_bwd
 * (mogan_kda/utils/math.py:38-72). */
typedef struct {
    MkdaLayout L;
    const float* dq_v; const float* dk_v;          /* [NC,HK] fp32 [64][128] tiles as written by mkda_bwd_chunk (summed over
                                                    * the v-heads of each q/k head) */
    const void* q; const void* k; int x_dtype;     /* raw q, k [TT,HK,128] */
    const float* q_rstd; const float* k_rstd;      /* [TT,HK], or NULL (no L2 norm) */
    void* dq; void* dk;                            /* [TT,HK,128] in x_dtype; tokens outside every chunk are not written */
} MkdaQkGrad;
int mkda_qk_grad_finish(const MkdaQkGrad* p, void* stream);

/* Prefix combine of per-segment (state, transition) pairs along each sequence:
 *   forward : S_in[s+1] = M_s S_in[s] + H_s        (reverse = 0, segments of a group in increasing order)
 *   backward: G_out[s-1] = M_s^T G_out[s] + D_s    (reverse = 1, decreasing order)
 * Groups are runs of segments (grp_seg_off) that belong to one sequence; `carry` is the value entering the first
 * (last, when reversed) segment of each group or NULL for zero.  Replaces correct_initial_states /
 * correct_terminal_states (mogan_kda/ops/gated_delta_rule/chunk/blackwell/cp_fwd.py:552-681). */
typedef struct {
    int NG; int HV;
    const int* grp_seg_off;    /* [NG+1] */
    const float* hs;           /* [NS,HV,128,128] per-segment local result ([K,V]); NULL = zero (composes transitions) */
    const float* ms;           /* [NS,HV,128,128] per-segment transition */
    const float* carry;        /* [NG,HV,128,128] ([K,V]) or NULL */
    int reverse;
    float* s_in;               /* [NS,HV,128,128] value entering each segment ([K,V]), or NULL */
    float* s_out;              /* [NG,HV,128,128] value leaving the last (first) segment of each group, or NULL */
} MkdaCombine;
int mkda_state_combine(const MkdaCombine* p, void* stream);

/* Warm-up truncation of the segment pre-passes.  The state entering a chunk reaches the end of its segment multiplied, per
 * key channel, by the decay of all chunks from there on.  Where the slowest channel's accumulated decay is already below
 * the threshold, what came before cannot be seen at the segment's end and a pass from zero need not visit it:
 *   warm_start[seg][h] = the last chunk c of the segment with  max_channel sum_{c' >= c} log2 gl[c'] < threshold_log2
 *                        (the segment's first chunk if there is none: nothing is skipped),
 *   warm_end[seg][h]   = one past the first chunk c with  max_channel sum_{c' <= c} log2 gl[c'] < threshold_log2
 *                        (one past the segment's last chunk if there is none), for the reverse chain.
 * An approximation with relative error 2^threshold_log2 in the segment-level states (the per-chunk main passes stay exact
 * given their entering state).  Follows get_warmup_chunks
 * (mogan_kda/ops/gated_delta_rule/chunk/blackwell/cp_fwd.py:81-115, threshold -10 in natural-log units there), extended to
 * the per-channel gate through the maximum over channels. */
typedef struct {
    MkdaLayout L;
    const float* gl;           /* [NC,HV,128] as written by mkda_intra_fwd */
    float threshold_log2;
    int* warm_start;           /* [NS,HV] */
    int* warm_end;             /* [NS,HV] */
} MkdaWarmup;
int mkda_warmup_chunks(const MkdaWarmup* p, void* stream);

/* Self-test of the tensor-core path: D[128,N] = A[128,K] B[N,K]^T (fp32 in, bf16 hi/lo split, fp32 out); N, K in
 * {64, 128}.  No counterpart in the reference; used by the tests to validate the tcgen05 plumbing in isolation. */
typedef struct {
    const float* A; const float* B; float* D; int N; int K;
    int mode;      /* bit 0: stage B MN-major, bit 1: stage A MN-major (exercises both operand views) */
} MkdaSelfTest;
int mkda_selftest_umma(const MkdaSelfTest* p, void* stream);

/* Self-test of the bounded waits: a kernel whose only wait can never complete (a barrier nothing arrives on).  After at
 * most `limit_cycles` SM clock cycles (1 .. 2^24, i.e. under 10 ms) every thread gives up, status[0] is set to 1, the
 * kernel releases its tensor memory and returns; the device stays usable and the process-wide flag behind
 * mkda_device_status() is not touched.  status[1] must stay 0.  No counterpart in the reference. */
typedef struct {
    int limit_cycles;
    unsigned int* status;      /* [2] device words, zeroed by the caller */
} MkdaSelfTestWait;
int mkda_selftest_wait(const MkdaSelfTestWait* p, void* stream);

/* Every wait inside a tensor-core kernel is bounded (about 70 ms); a wait that expires sets a device-side flag and the
 * kernel runs on to its exit with undefined results.  mkda_device_status() synchronises the current device and returns
 * 0 if no wait has expired since the flag was last cleared, else 1: poll it wherever the host synchronises anyway (end
 * of a step, checkpoint).  While the flag is set later waits give up after ~35 us, so that a broken launch drains fast;
 * mkda_device_status_clear() (synchronises) resets it and restores the long limit. */
int mkda_device_status(void);
int mkda_device_status_clear(void);

const char* mkda_last_error(void);
int mkda_abi_version(void);
/* sizeof() of every parameter struct, in declaration order, so bindings can verify their mirror of this header. */
int mkda_struct_sizes(int* out, int n);

#ifdef __cplusplus
}
#endif
#endif /* MKDA_H_ */

/*
 * jla_b200.h - C ABI of the B200 (sm_100a) kernels for the chunkwise gated delta rule family
 * (simple GLA / Mamba-2 SSD core, DeltaNet, Gated DeltaNet, KDA), forward and backward.
 *
 * The reference (jla-org/jax-linear-attention) is pure Python: its kernels are Pallas programs that JAX
 * lowers to XLA custom calls, so it has no foreign-function layer of its own. These entry points are what an
 * XLA typed-FFI handler (one per entry point) or a ctypes host binds instead of:
 *
 *   src/jla/ops/mosaic_gpu/scalar_gate.py:309-348   _forward      (kkt_fwd + fused_fwd_wy / fused_fwd)
 *   src/jla/ops/mosaic_gpu/scalar_gate.py:357-452   _backward     (state_fwd, state_bwd, chunk_grads / dqkwg)
 *   src/jla/ops/mosaic_gpu/vector_gate_ops.py:98-164 KDA forward / backward kernel chains
 *   src/jla/ops/reference.py:105-205                _recurrence   (fp32 token scan, cu_seqlens semantics)
 *
 * Rules of the ABI:
 *   - plain C types only; all pointers are DEVICE pointers owned by the caller (except the args struct itself,
 *     which is host memory and is read before the call returns);
 *   - every call only enqueues work on `stream` and returns; nothing here allocates, frees or synchronises;
 *   - scratch and residual memory is provided by the caller, sized by the *_bytes() queries (XLA custom calls
 *     must not allocate: declare them as extra result buffers);
 *   - return value 0 = enqueued, negative = rejected (jla_status); jla_last_error() gives the reason text.
 *
 * Tensor layouts (row-major, innermost last), following src/jla/ops/reference.py:8-35:
 *   q, k    [B, T, Hk, K]   dtype            v, o, do, dv [B, T, H, V]   dtype      (H % Hk == 0)
 *   g       [B, T, H] f32 (scalar gates) or [B, T, H, K] f32 (KDA), natural-log decay, <= 0
 *   beta    [B, T, H] f32
 *   h0/final/dht/dh0 [R, H, K, V] f32 with R = B, or R = num_seqs when cu_seqlens is given (then B must be 1)
 *   segment_ids [B, T] int32 (state restarts where the id changes along T)
 *   cu_seqlens  [num_seqs + 1] int32, cu[0] == 0, cu[num_seqs] == T
 *   dq, dk  [B, T, Hk, K]   dtype (summed over each group's heads in fp32, rounded once)
 *   dg      like g, f32;   dbeta [B, T, H] f32
 */
#ifndef JLA_B200_H_
#define JLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* jla_stream_t; /* a cudaStream_t */

enum jla_kind {              /* src/jla/ops/__init__.py:47-60 (KINDS) */
  JLA_KIND_SIMPLE_GLA = 0,   /* S = exp(g) S + k^T v                      (Mamba-2 SSD core)          */
  JLA_KIND_DELTANET = 1,     /* S = S + beta k^T (v - k S)                                            */
  JLA_KIND_GATED_DELTANET = 2, /* S' = exp(g) S; S = S' + beta k^T (v - k S')                         */
  JLA_KIND_KDA = 3           /* S' = diag(exp(g)) S; S = S' + beta k^T (v - k S')   (g per key channel) */
};
/* Gated DeltaNet-2 (src/jla/ops/reference.py:313-343, S = S' + k^T (w v - (b k) S') with an erase gate b per key
 * channel and a write gate w per value channel) is KDA with beta = 1, the values w * v and a separate read key
 * b * k: see jla_problem.k_read. */

enum jla_dtype { JLA_DTYPE_BF16 = 0, JLA_DTYPE_F16 = 1, JLA_DTYPE_F32 = 2 };

enum jla_path {
  JLA_PATH_AUTO = 0,      /* f32 tensors: RECURRENT; bf16/f16: CHUNKED where it applies (KDA: K = V = 128).
                           * A call with k_read has chunked kernels for KDA only: the other kinds run RECURRENT
                           * with it, whatever is asked for here. */
  JLA_PATH_RECURRENT = 1, /* fp32 token scan in the order of reference.py:140-157 (any K, V <= 256)            */
  JLA_PATH_CHUNKED = 2    /* chunk-64 tensor-core kernels (bf16/f16, K and V in {64, 128})                      */
};

enum jla_flags {
  JLA_FLAG_QK_L2NORM = 1,     /* normalise q and k over the head dim in fp32, eps 1e-6 (reference.py:65-69)   */
  JLA_FLAG_SAVE_RESIDUALS = 2, /* forward: fill `residuals` for a later jla_linear_attention_bwd             */
  /* The two flags below serve callers that run several passes over the same tokens (documents cut into pieces
   * joined by affine maps: src/jla/ops/mosaic_gpu/scalar_gate.py:129-148). Chunked path only; ignored elsewhere. */
  JLA_FLAG_PREP_DONE = 4,      /* forward: the buffer passed as residuals (or scratch) already holds the chunk table,
                                * gates, T0/Ag and normalised q/k of an earlier forward with the same k, g, beta,
                                * segment_ids / cu_seqlens and (with the L2 norm) q: skip recomputing them          */
  JLA_FLAG_STATE_GRADS_ONLY = 8, /* backward: run the reverse state pass only: dh0 and dv are written, dq, dk, dg and
                                 * dbeta are left untouched                                                         */
  JLA_FLAG_STATE_ONLY = 16      /* forward: only final_state (and residuals) are wanted; o may be left unwritten
                                 * (the tcgen05 forward then skips the score and output products)                  */
};

enum jla_status {
  JLA_OK = 0,
  JLA_ERR_BAD_ARGUMENT = -1,  /* null pointer, inconsistent sizes, unknown enum                                 */
  JLA_ERR_UNSUPPORTED = -2,   /* valid call that no kernel here covers (reason in jla_last_error)              */
  JLA_ERR_WORKSPACE = -3,     /* scratch or residual buffer smaller than the *_bytes() query                    */
  JLA_ERR_CUDA = -4           /* a CUDA runtime call failed at enqueue time                                    */
};

typedef struct jla_problem {
  int32_t kind;       /* enum jla_kind */
  int32_t dtype;      /* enum jla_dtype of q, k, v, o and their gradients */
  int32_t path;       /* enum jla_path */
  int32_t flags;      /* enum jla_flags, or-ed */
  int32_t B, T, H, Hk, K, V;
  int32_t num_seqs;   /* sequences in cu_seqlens, 0 without */
  float scale;        /* applied to q (reference.py:130-132); the caller resolves None to K^-0.5 */
  const void* q;
  const void* k;
  const void* v;
  const float* g;            /* NULL for DELTANET */
  const float* beta;         /* NULL for SIMPLE_GLA */
  const float* h0;           /* optional initial state */
  const int32_t* segment_ids; /* optional */
  const int32_t* cu_seqlens;  /* optional; excludes segment_ids */
  const void* k_read;         /* optional, delta-rule kinds: [B, T, H, K] dtype, one row per VALUE head. When given, the
                               * recall reads the state with it (S = S' + beta k^T (v - k_read S')), k still writes.
                               * It is used as passed (JLA_FLAG_QK_L2NORM normalises q and k only). */
} jla_problem;

typedef struct jla_fwd_io {
  void* o;              /* [B, T, H, V] dtype */
  float* final_state;   /* optional [R, H, K, V] */
  void* residuals;      /* jla_residual_bytes() bytes when JLA_FLAG_SAVE_RESIDUALS, else may be NULL */
  size_t residual_bytes;
  void* scratch;        /* jla_fwd_scratch_bytes() bytes */
  size_t scratch_bytes;
} jla_fwd_io;

typedef struct jla_bwd_io {
  const void* d_o;          /* [B, T, H, V] dtype: cotangent of o */
  const float* d_final;     /* optional [R, H, K, V]: cotangent of the final state */
  void* dq;                 /* [B, T, Hk, K] dtype */
  void* dk;                 /* [B, T, Hk, K] dtype */
  void* dv;                 /* [B, T, H, V] dtype */
  float* dg;                /* like g; NULL for DELTANET */
  float* dbeta;             /* [B, T, H]; NULL for SIMPLE_GLA */
  float* dh0;               /* optional [R, H, K, V] */
  const void* residuals;    /* what the forward wrote (same problem, JLA_FLAG_SAVE_RESIDUALS) */
  size_t residual_bytes;
  void* scratch;            /* jla_bwd_scratch_bytes() bytes */
  size_t scratch_bytes;
  void* dk_read;            /* [B, T, H, K] dtype: gradient of k_read (required when the problem has one) */
} jla_bwd_io;

/* Library/ABI version: major * 1000 + minor. */
int jla_abi_version(void);

/* Text of the last rejected call on this host thread ("" if none). */
const char* jla_last_error(void);

/* NULL if the library has a kernel for `p`, else the reason as text. Of the pointers in `p` only k_read is looked
 * at, and only whether it is NULL (a call with a read key takes another path).
 * Mirrors unsupported_reason() of src/jla/ops/mosaic_gpu/scalar_gate.py:476-515 and
 * src/jla/ops/mosaic_gpu/vector_gate_ops.py:262-304. */
const char* jla_unsupported_reason(const jla_problem* p);

/* Buffer sizes in bytes for problem `p` (0 is a valid answer; of the pointers in `p` only k_read is looked at, and
 * only whether it is NULL). */
size_t jla_residual_bytes(const jla_problem* p);
size_t jla_fwd_scratch_bytes(const jla_problem* p);
size_t jla_bwd_scratch_bytes(const jla_problem* p);

/* Forward: o and (optionally) the final state; replaces scalar_gate._forward / the KDA forward chain. */
int jla_linear_attention_fwd(const jla_problem* p, const jla_fwd_io* io, jla_stream_t stream);

/* Backward for cotangents (d_o, d_final); replaces scalar_gate._backward / the KDA backward chain. */
int jla_linear_attention_bwd(const jla_problem* p, const jla_bwd_io* io, jla_stream_t stream);

/* Forward for hosts that have no scratch buffer to pass and are not allowed to allocate one (a custom call inside
 * another runtime's executor that reserved no workspace, a server whose memory pool is frozen after start-up).
 * This entry point has no counterpart in the reference. Same computation and results as jla_linear_attention_fwd
 * without JLA_FLAG_SAVE_RESIDUALS; the scratch is a fixed array of jla_noalloc_scratch_limit() bytes (32 MiB) of
 * device memory that belongs to the library and is held on every GPU that loads it until the process exits.
 * It calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - A call whose jla_fwd_scratch_bytes() exceeds the limit is rejected with JLA_ERR_WORKSPACE.
 *   - The first call on a device looks up the array's device address (one cudaGetSymbolAddress, with that device
 *     current); make that first call before any stream capture begins.
 *   - All calls on a device share the array: calls that may overlap on the GPU (different streams) race on it.
 *     Keep them on one stream or order them with events. Nothing needs clearing between calls.
 *   - JLA_FLAG_SAVE_RESIDUALS and JLA_FLAG_PREP_DONE are rejected (JLA_ERR_BAD_ARGUMENT): the array belongs to the
 *     library, so no caller can know that an earlier call's tables are still in it. */
size_t jla_noalloc_scratch_limit(void);
int jla_linear_attention_fwd_noalloc(const jla_problem* p, void* o, float* final_state, jla_stream_t stream);

/* Element-wise glue of Gated DeltaNet-2 around the KDA kernels (src/jla/ops/reference.py:152-154: the erase gate b
 * multiplies the key where it reads the state, the write gate w the value; the XLA fusions next to the kernel call in
 * src/jla/ops/mosaic_gpu/vector_gate_ops.py). All tensors share `dtype` and are flat: n_k elements for k, b, k_read
 * and their gradients, n_v for v, w, v_gated and theirs (multiples of 8).
 *   inputs_fwd:  k_read = k * b, v_gated = v * w              (the call then passes k_read as jla_problem.k_read,
 *                                                              v_gated as v and beta = 1 with JLA_KIND_KDA)
 *   inputs_bwd:  dk = dk_read * b, db = dk_read * k, dv = dv_gated * w, dw = dv_gated * v
 *                (dk is the read side's share; the caller adds the dk the backward call returned) */
int jla_gdn2_inputs_fwd(int dtype, int64_t n_k, int64_t n_v, const void* k, const void* b, const void* v, const void* w,
                        void* k_read, void* v_gated, jla_stream_t stream);
int jla_gdn2_inputs_bwd(int dtype, int64_t n_k, int64_t n_v, const void* k, const void* b, const void* v, const void* w,
                        const void* dk_read, const void* dv_gated, void* dk, void* db, void* dv, void* dw,
                        jla_stream_t stream);

/* Element-wise glue of the Mamba-2 SSD layer around the simple_gla kernels, fused so every [tokens, H, P] tensor is
 * read and written once; replaces the XLA fusions around the kernel call in mamba2_ssd (src/jla/layers/ssm.py:207-229)
 * and their transposes (ssm.py:76-84). 16-bit x, v, o, y and gradients; dt, A, D, g and their gradients f32;
 * tokens = B * T; P a multiple of 8. dA and dD ([H]) are zeroed by the call before it accumulates into them.
 *   inputs_fwd:  v = round(x * dt), g = dt * A
 *   inputs_bwd:  dx = round(dv * dt), ddt = sum_p dv * x + dg * A, dA = sum_tokens dg * dt
 *   output_fwd:  y = round(o + D * x)
 *   output_bwd:  dx = round(D * dy), dD = sum_{tokens, p} dy * x      (do = dy needs no kernel)
 *   layer_bwd:   inputs_bwd and output_bwd in one pass for a layer with a D term: dx = round(dv * dt + D * dy),
 *                ddt, dA, dD as above; x, dv and dy are read once and no partial dx tensors are summed afterwards */
int jla_ssd_inputs_fwd(int dtype, int64_t tokens, int H, int P, const void* x, const float* dt, const float* a, void* v,
                       float* g, jla_stream_t stream);
int jla_ssd_inputs_bwd(int dtype, int64_t tokens, int H, int P, const void* x, const float* dt, const float* a,
                       const void* dv, const float* dg, void* dx, float* ddt, float* da, jla_stream_t stream);
int jla_ssd_output_fwd(int dtype, int64_t tokens, int H, int P, const void* o, const void* x, const float* d, void* y,
                       jla_stream_t stream);
int jla_ssd_output_bwd(int dtype, int64_t tokens, int H, int P, const void* dy, const void* x, const float* d, void* dx,
                       float* dd, jla_stream_t stream);
int jla_ssd_layer_bwd(int dtype, int64_t tokens, int H, int P, const void* x, const float* dt, const float* a,
                      const float* d, const void* dv, const float* dg, const void* dy, void* dx, float* ddt, float* da,
                      float* dd, jla_stream_t stream);

/* Gate activations in front of the kernels, forward and backward in one pass each; replaces the XLA fusions of
 * _mamba_gate and _write_strength in the Gated DeltaNet and KDA mixers (src/jla/layers/linear_attention.py:84-86,
 * 159-162, 295-297, 324-328):
 *   g = -exp(A_log[h]) * softplus(a + dt_bias)      a [tokens, H, C] dtype (C = 1, or K for KDA), dt_bias [H, C] f32,
 *                                                   A_log [H] f32, g [tokens, H, C] f32
 *   beta = m * sigmoid(b), m = allow_neg_eigval ? 2 : 1     b [tokens, H] dtype (may be NULL), beta [tokens, H] f32
 * Backward: da, db in dtype; dA_log [H] and ddt_bias [H, C] f32 are zeroed by the call and then accumulated.
 * H * C / 8 (H * C itself when it is no multiple of 8) must divide 32 or be a multiple of it. */
int jla_gate_prologue_fwd(int dtype, int64_t tokens, int H, int C, const void* a, const float* a_log,
                          const float* dt_bias, const void* b, int allow_neg_eigval, float* g, float* beta,
                          jla_stream_t stream);
int jla_gate_prologue_bwd(int dtype, int64_t tokens, int H, int C, const void* a, const float* a_log,
                          const float* dt_bias, const void* b, int allow_neg_eigval, const float* dg, const float* dbeta,
                          void* da, void* db, float* da_log, float* ddt_bias, jla_stream_t stream);

/* Short causal depthwise convolution (+ SiLU) (+ per-head L2 norm), the q / k prologue of the delta-rule mixers,
 * forward and backward in one pass each; replaces ShortConv.__call__ (src/jla/layers/conv.py:97-142) followed by the
 * op's use_qk_l2norm, i.e. the fused kernels of src/jla/ops/mosaic_gpu/short_conv_l2norm.py.
 *   x, y, dy, dx [B, T, C] dtype; weight, dweight [C, K] f32 (1 <= K <= 4); bias, dbias [C] f32 or NULL;
 *   segment_ids [B, T] int32 or NULL (taps into an earlier document contribute zero); state, dstate [B, K - 1, C]
 *   dtype or NULL (the inputs before t = 0; they count as the first token's document); head_dim > 0 normalises each
 *   head_dim consecutive channels to unit L2 norm (eps 1e-6) in float32 before the single rounding; 0 = no norm.
 * dweight and dbias are zeroed by the call, then accumulated. The state after the call (the last K - 1 inputs) is
 * input data and is assembled by the host. */
int jla_short_conv_fwd(int dtype, int B, int T, int C, int K, int head_dim, int activation, const void* x,
                       const float* weight, const float* bias, const int32_t* segment_ids, const void* state, void* y,
                       jla_stream_t stream);
int jla_short_conv_bwd(int dtype, int B, int T, int C, int K, int head_dim, int activation, const void* x,
                       const float* weight, const float* bias, const int32_t* segment_ids, const void* state,
                       const void* dy, void* dx, float* dweight, float* dbias, void* dstate, jla_stream_t stream);

/* Gated RMS norm behind the kernels (the mixers' output norm; with norm_before_gate = 0 the Mamba-2 norm), forward
 * and backward in one pass each; replaces GatedRMSNorm.__call__ (src/jla/layers/norm.py:60-112) and its transpose.
 *   gate = silu(z), or sigmoid(z) with sigmoid_gate;  u = x (norm_before_gate) or x * gate;
 *   y = u * rsqrt(mean over each group of `group` channels of u^2 + eps) * weight (* gate with norm_before_gate)
 * x, z, y, dy, dx, dz [rows, dim] dtype; weight, dweight [dim] f32 (dweight is zeroed by the call, then accumulated).
 * `group` divides dim and is 8 times a power of two, at most 8192. */
int jla_gated_rmsnorm_fwd(int dtype, int64_t rows, int dim, int group, const void* x, const void* z, const float* weight,
                          float eps, int sigmoid_gate, int norm_before_gate, void* y, jla_stream_t stream);
int jla_gated_rmsnorm_bwd(int dtype, int64_t rows, int dim, int group, const void* x, const void* z, const float* weight,
                          float eps, int sigmoid_gate, int norm_before_gate, const void* dy, void* dx, void* dz,
                          float* dweight, jla_stream_t stream);

/* Diagnostics: where the chunked path keeps its intermediates, so that tests can compare them stage by stage
 * with the CPU model (the reference checks its kernels per stage too:
 * tests/test_mosaic_gpu_gated_delta_rule.py:104-146). Byte offsets into the residual buffer written by a forward
 * with JLA_FLAG_SAVE_RESIDUALS (meta .. vn) and into the backward scratch (dh .. dk_acc). Chunk slot c of head h:
 *   gates [c][h][128] f32 (G[64], beta[64])    runs [c][64] u8    t0, ag [c][h][64][64] dtype (ag = t0 * D * beta_j)
 *   h [c][h][K][V] dtype (state entering the chunk)    vn [c][h][64][V] dtype
 *   dh [c][h][K][V] dtype (gradient of the state leaving the chunk)    dvn [c][h][64][V] dtype
 * With K = V = 128 (the tcgen05 kernels; JLA_B200_LEGACY=1 in the environment turns them off) h, vn, dh and dvn are
 * stored transposed ([V][K], [V][64]), and three more buffers exist: w [c][h][V][64] dtype (W^T = (V - cin Gamma K S)^T),
 * dp [c][h] 64x64 dtype tiles in the 128-byte-swizzled shared-memory layout, dga [c][h][64] f32 (dG partial sums). */
typedef struct jla_chunked_layout {
  int32_t num_chunk_slots;
  size_t meta, row_chunks, gates, runs, t0, ag, qn, kn, h, vn, w, residual_bytes;
  size_t dh, dvn, dq_acc, dk_acc, dp, dga, bwd_scratch_bytes;
} jla_chunked_layout;
int jla_chunked_get_layout(const jla_problem* p, jla_chunked_layout* out);

/* Diagnostics: per-kernel device time. While enabled, every kernel launch of the library is bracketed by CUDA
 * events on its stream (no synchronisation at launch). jla_profile_read() waits for the recorded events and returns
 * the summed duration and launch count of one kernel since the last jla_profile_reset(); kernel ids run from 0 until
 * jla_profile_kernel_name() returns NULL. (The reference times its kernels with CUPTI: benchmarks/harness.py:55-80.) */
int jla_profile_enable(int on);
int jla_profile_reset(void);
const char* jla_profile_kernel_name(int kernel_id);
int jla_profile_read(int kernel_id, double* total_ms, int* launches);

/* Diagnostics: one-CTA check of the tcgen05 primitive layer. Computes C[m][n] (f32) = A * B with bf16 operands
 * staged in 128-byte-swizzled shared memory: a = A[m][kd] (K-major view) or A^T[kd][m] (MN-major view, a_mn_major),
 * b = B^T[n][kd] or B[kd][n] (b_mn_major). *status is set to 1 if the MMA completion never arrived (bounded wait).
 * Shapes: (64,128,128), (64,64,64), (64,64,128), (128,128,64). No counterpart in the reference. */
int jla_selftest_umma(int m, int n, int kd, int a_mn_major, int b_mn_major, const void* a, const void* b, float* c,
                      int* status, jla_stream_t stream);

/* Scan over the pieces of a sequence cut into independently processed pieces that are joined by affine maps
 * S_out[p] = M[p] S_in[p] + E[p]; replaces gdr_piece_scan / gdr_piece_scan_bwd
 * (src/jla/ops/mosaic_gpu/scalar_gate_scan.py:49-140), the fp32 scan between the passes of the reference's intra-GPU
 * sequence split (src/jla/ops/mosaic_gpu/scalar_gate.py:199-271). All tensors fp32, device memory:
 *   maps [P, H, K, K]; cont [P] int32 (piece p continues the document of piece p - 1: its entering state is the
 *   state leaving p - 1, otherwise zero and its map is never read); boundary [H, K, V] or NULL (= zero);
 *   forward  (backward = 0): states [P, H, K, V] holds E on entry and S_out on return for pieces p_lo .. p_hi - 1
 *            (piece 0 continues `boundary`); ds_out is ignored;
 *   backward (backward = 1): states holds dS_in (the entering-state gradients for a zero final-state cotangent) and
 *            gets M^T dS_out added; ds_out [P, H, K, V] (zero-filled by the caller) receives every piece's
 *            final-state cotangent; pieces p_hi - 1 down to p_lo; piece P - 1 takes `boundary` as its cotangent.
 * K in {64, 128}, V a multiple of 32. The range arguments let a caller scan the pieces that do not depend on a
 * neighbouring rank's state before that state has arrived. */
int jla_piece_scan(int backward, int P, int H, int K, int V, const float* maps, const int32_t* cont, const float* boundary,
                   float* states, float* ds_out, int p_lo, int p_hi, jla_stream_t stream);

/* Failure status of the tensor-core kernels. Every wait inside them (on a TMA copy, an MMA completion or another
 * warp role) is bounded: a wait that runs out makes the kernel return normally with a non-zero code in a status
 * word that lives on the GPU (one word per GPU that loads the library), and the results of that launch are
 * undefined. jla_device_status() waits for `stream`, copies the word of the CURRENT device to *out and clears it:
 * 0 = every launch since the last query completed its waits; 1 = a chunk-gradient kernel, 2 = a forward state
 * pass, 3 = a reverse state pass gave up; 9 = jla_selftest_bounded_wait. It blocks the host (diagnostic call; the
 * compute entry points never do). No counterpart in the reference, whose Pallas kernels wait without a bound. */
int jla_device_status(int* out, jla_stream_t stream);

/* Diagnostics: launches one small CTA whose bounded wait on a barrier nobody arrives on gives up after
 * `spin_limit` polls (1 .. 2^20), records status 9 and exits normally -- the path a lost arrival takes in the real
 * kernels, exercised without a fault or a hang. No counterpart in the reference. */
int jla_selftest_bounded_wait(uint32_t spin_limit, jla_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* JLA_B200_H_ */

// Orchestration of the chunked path: support predicate, buffer sizes, and the kernel sequences of the forward
// (tables -> gates -> [L2 norm] -> T0 -> fused forward) and the backward (reverse state pass -> chunk gradients
// -> key-gradient epilogue).
#include <stdlib.h>

#include "chunked.cuh"

namespace jla {

const char* chunked_unsupported(const jla_problem& p) {
  if (p.dtype == JLA_DTYPE_F32) return "the chunked tensor-core kernels take bf16 or f16 tensors (f32 runs the recurrent path)";
  if ((p.K != 64 && p.K != 128) || (p.V != 64 && p.V != 128)) return "head dims K, V must be in (64, 128)";
  if (p.kind == JLA_KIND_KDA && !use_tc_kernels(p)) {
    return "the chunked KDA forward takes bf16 or f16 tensors with K = V = 128 (other calls run the recurrent path)";
  }
  return nullptr;
}

bool use_tc_kernels(const jla_problem& p) {
  static const bool legacy = [] {
    const char* e = getenv("JLA_B200_LEGACY");
    return e && e[0] == '1';
  }();
  return !legacy && p.K == 128 && p.V == 128 && p.dtype != JLA_DTYPE_F32;
}

bool kda_scan_backward() {
  static const bool scan = [] {
    const char* e = getenv("JLA_B200_KDA_SCAN_BWD");
    return e && e[0] == '1';
  }();
  return scan;
}

size_t chunked_residual_bytes(const jla_problem& p) { return make_plan(p).residual_bytes; }

size_t chunked_fwd_scratch_bytes(const jla_problem& p) {
  const Plan pl = make_plan(p);
  return pl.save ? 0 : pl.fwd_scratch_bytes;
}

size_t chunked_bwd_scratch_bytes(const jla_problem& p) { return make_plan(p).bwd_scratch_bytes; }

static ChunkedCtx make_ctx(const jla_problem& p, char* res) {
  ChunkedCtx c;
  c.p = p;
  c.plan = make_plan(p);
  c.res = res;
  c.q_eff = c.plan.l2norm ? static_cast<const void*>(res + c.plan.qn) : p.q;
  c.k_eff = c.plan.l2norm ? static_cast<const void*>(res + c.plan.kn) : p.k;
  return c;
}

// A call without tokens launches no chunk kernel: the state passes through unchanged.
static int copy_state(float* dst, const float* src, const jla_problem& p, cudaStream_t stream) {
  if (!dst) return JLA_OK;
  const size_t rows = p.num_seqs > 0 ? p.num_seqs : p.B;
  const size_t bytes = rows * p.H * p.K * p.V * sizeof(float);
  if (bytes == 0) return JLA_OK;
  if (src) JLA_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream));
  else JLA_CUDA_OK(cudaMemsetAsync(dst, 0, bytes, stream));
  return JLA_OK;
}

int chunked_fwd(const jla_problem& p, const jla_fwd_io& io, cudaStream_t stream) {
  if ((long)p.B * p.T == 0) return copy_state(io.final_state, p.h0, p, stream);
  const Plan pl = make_plan(p);
  char* res;
  if (pl.save) {
    if (!io.residuals || io.residual_bytes < pl.residual_bytes) {
      set_error("residual buffer too small: %zu < %zu bytes", io.residuals ? io.residual_bytes : (size_t)0,
                pl.residual_bytes);
      return JLA_ERR_WORKSPACE;
    }
    res = static_cast<char*>(io.residuals);
  } else {
    if (!io.scratch || io.scratch_bytes < pl.fwd_scratch_bytes) {
      set_error("forward scratch too small: %zu < %zu bytes", io.scratch ? io.scratch_bytes : (size_t)0,
                pl.fwd_scratch_bytes);
      return JLA_ERR_WORKSPACE;
    }
    res = static_cast<char*>(io.scratch);
  }
  const ChunkedCtx c = make_ctx(p, res);
  if (!(p.flags & JLA_FLAG_PREP_DONE)) {
    const int rc = launch_prep(c, stream);
    if (rc != JLA_OK) return rc;
  }
  return use_tc_kernels(p) ? launch_sg_fwd_tc(c, io, stream) : launch_sg_fwd(c, io, stream);
}

int chunked_bwd(const jla_problem& p, const jla_bwd_io& io, cudaStream_t stream) {
  if ((long)p.B * p.T == 0) return copy_state(io.dh0, io.d_final, p, stream);
  jla_problem ps = p;
  ps.flags |= JLA_FLAG_SAVE_RESIDUALS;
  const Plan pl = make_plan(ps);
  if (!io.residuals || io.residual_bytes < pl.residual_bytes) {
    set_error("residual buffer too small: %zu < %zu bytes", io.residuals ? io.residual_bytes : (size_t)0,
              pl.residual_bytes);
    return JLA_ERR_WORKSPACE;
  }
  if (pl.bwd_scratch_bytes && (!io.scratch || io.scratch_bytes < pl.bwd_scratch_bytes)) {
    set_error("backward scratch too small: %zu < %zu bytes", io.scratch ? io.scratch_bytes : (size_t)0,
              pl.bwd_scratch_bytes);
    return JLA_ERR_WORKSPACE;
  }
  const ChunkedCtx c = make_ctx(ps, static_cast<char*>(const_cast<void*>(io.residuals)));
  return launch_sg_bwd(c, io, static_cast<char*>(io.scratch), stream);
}

}  // namespace jla

extern "C" int jla_chunked_get_layout(const jla_problem* p, jla_chunked_layout* out) {
  if (!p || !out) return JLA_ERR_BAD_ARGUMENT;
  jla_problem ps = *p;
  ps.flags |= JLA_FLAG_SAVE_RESIDUALS;
  const jla::Plan pl = jla::make_plan(ps);
  out->num_chunk_slots = pl.nc;
  out->meta = pl.meta; out->row_chunks = pl.row_chunks; out->gates = pl.gates; out->runs = pl.runs;
  out->t0 = pl.t0; out->ag = pl.ag; out->qn = pl.qn; out->kn = pl.kn; out->h = pl.h; out->vn = pl.vn; out->w = pl.w;
  out->residual_bytes = pl.residual_bytes;
  out->dh = pl.dh; out->dvn = pl.dvn; out->dq_acc = pl.dq_acc; out->dk_acc = pl.dk_acc; out->dp = pl.dp; out->dga = pl.dga;
  out->bwd_scratch_bytes = pl.bwd_scratch_bytes;
  return JLA_OK;
}

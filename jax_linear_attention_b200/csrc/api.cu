// extern "C" surface of libjla_b200.so (declared in include/jla_b200.h): argument validation, path
// selection, workspace sizing. No kernel lives here.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace jla {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

const char* recurrent_unsupported(const jla_problem& p);
const char* chunked_unsupported(const jla_problem& p);
bool kda_scan_backward();
size_t chunked_residual_bytes(const jla_problem& p);
size_t chunked_fwd_scratch_bytes(const jla_problem& p);
size_t chunked_bwd_scratch_bytes(const jla_problem& p);
int chunked_fwd(const jla_problem& p, const jla_fwd_io& io, cudaStream_t stream);
int chunked_bwd(const jla_problem& p, const jla_bwd_io& io, cudaStream_t stream);

namespace {

// With JLA_B200_KDA_SCAN_BWD=1 the KDA backward is the token scan (it recomputes what it needs from the inputs, so the
// chunked KDA forward then keeps no residuals).
int resolve_path(const jla_problem& p, bool bwd = false) {
  if (bwd && p.kind == JLA_KIND_KDA && kda_scan_backward()) return JLA_PATH_RECURRENT;
  if (p.k_read && p.kind != JLA_KIND_KDA) return JLA_PATH_RECURRENT;  // only the KDA chunk kernels take a read key
  if (p.path == JLA_PATH_AUTO) {
    // f32 tensors run the exact token scan; so does whatever the chunked kernels do not cover (chunked_unsupported()).
    if (p.dtype == JLA_DTYPE_F32 || chunked_unsupported(p) != nullptr) {
      return recurrent_unsupported(p) == nullptr || p.dtype == JLA_DTYPE_F32 ? JLA_PATH_RECURRENT : JLA_PATH_CHUNKED;
    }
    return JLA_PATH_CHUNKED;
  }
  return p.path;
}

// Shape-level validation shared by every entry point (pointers are not looked at).
const char* shape_problem(const jla_problem& p) {
  static thread_local char buf[256];
  if (p.kind < JLA_KIND_SIMPLE_GLA || p.kind > JLA_KIND_KDA) return "unknown kind";
  if (p.dtype < JLA_DTYPE_BF16 || p.dtype > JLA_DTYPE_F32) return "unknown dtype";
  if (p.path < JLA_PATH_AUTO || p.path > JLA_PATH_CHUNKED) return "unknown path";
  if (p.B < 0 || p.T < 0 || p.H <= 0 || p.Hk <= 0 || p.K <= 0 || p.V <= 0) return "negative or zero dimension";
  if (p.H % p.Hk) {
    snprintf(buf, sizeof(buf), "value heads %d must be a multiple of key heads %d", p.H, p.Hk);
    return buf;
  }
  if (p.num_seqs < 0) return "num_seqs must be >= 0";
  if (p.num_seqs > 0 && p.B != 1) return "cu_seqlens packs sequences along T and requires batch size 1";
  if ((p.flags & JLA_FLAG_QK_L2NORM) && p.kind == JLA_KIND_SIMPLE_GLA) return "use_qk_l2norm is a delta-rule option";
  if ((long)p.B * p.T * p.H * (p.K > p.V ? p.K : p.V) >= (1L << 46)) return "tensor too large";
  return nullptr;
}

const char* unsupported(const jla_problem& p) {
  if (const char* why = shape_problem(p)) return why;
  return resolve_path(p) == JLA_PATH_RECURRENT ? recurrent_unsupported(p) : chunked_unsupported(p);
}

int check_common(const jla_problem* p) {
  if (!p) {
    set_error("null problem");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (const char* why = shape_problem(*p)) {
    set_error("%s", why);
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (const char* why = unsupported(*p)) {
    set_error("%s", why);
    return JLA_ERR_UNSUPPORTED;
  }
  const bool has_tokens = (long)p->B * p->T > 0;
  if (has_tokens && (!p->q || !p->k || !p->v)) {
    set_error("q, k, v must not be null");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (has_tokens && p->kind != JLA_KIND_DELTANET && !p->g) {
    set_error("this kind takes a gate g");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (has_tokens && p->kind != JLA_KIND_SIMPLE_GLA && !p->beta) {
    set_error("this kind takes beta");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (p->k_read && p->kind == JLA_KIND_SIMPLE_GLA) {
    set_error("k_read is an option of the delta-rule kinds");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (p->cu_seqlens && p->segment_ids) {
    set_error("pass cu_seqlens or segment_ids, not both");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if ((p->cu_seqlens != nullptr) != (p->num_seqs > 0)) {
    set_error("cu_seqlens and num_seqs must be given together");
    return JLA_ERR_BAD_ARGUMENT;
  }
  return JLA_OK;
}

}  // namespace
}  // namespace jla

using namespace jla;

extern "C" {

int jla_abi_version(void) { return 1001; }

const char* jla_last_error(void) { return g_error; }

const char* jla_unsupported_reason(const jla_problem* p) { return p ? unsupported(*p) : "null problem"; }

size_t jla_residual_bytes(const jla_problem* p) {
  if (!p || unsupported(*p) || (p->kind == JLA_KIND_KDA && kda_scan_backward())) return 0;
  return resolve_path(*p) == JLA_PATH_RECURRENT ? 0 : chunked_residual_bytes(*p);
}

size_t jla_fwd_scratch_bytes(const jla_problem* p) {
  if (!p || unsupported(*p)) return 0;
  return resolve_path(*p) == JLA_PATH_RECURRENT ? 0 : chunked_fwd_scratch_bytes(*p);
}

size_t jla_bwd_scratch_bytes(const jla_problem* p) {
  if (!p || unsupported(*p)) return 0;
  return resolve_path(*p, true) == JLA_PATH_RECURRENT ? recurrent_bwd_scratch_bytes(*p) : chunked_bwd_scratch_bytes(*p);
}

int jla_linear_attention_fwd(const jla_problem* p, const jla_fwd_io* io, jla_stream_t stream) {
  g_error[0] = 0;
  if (int rc = check_common(p)) return rc;
  if (!io || ((long)p->B * p->T > 0 && !io->o)) {
    set_error("null output");
    return JLA_ERR_BAD_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return resolve_path(*p) == JLA_PATH_RECURRENT ? recurrent_fwd(*p, *io, s) : chunked_fwd(*p, *io, s);
}

int jla_linear_attention_bwd(const jla_problem* p, const jla_bwd_io* io, jla_stream_t stream) {
  g_error[0] = 0;
  if (int rc = check_common(p)) return rc;
  const bool has_tokens = (long)p->B * p->T > 0;
  if (!io || (has_tokens && (!io->d_o || !io->dq || !io->dk || !io->dv))) {
    set_error("null gradient buffer");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (has_tokens && p->k_read && !io->dk_read) {
    set_error("null gradient buffer for k_read");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (has_tokens && ((p->kind != JLA_KIND_DELTANET && !io->dg) || (p->kind != JLA_KIND_SIMPLE_GLA && !io->dbeta))) {
    set_error("null gate gradient buffer");
    return JLA_ERR_BAD_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return resolve_path(*p, true) == JLA_PATH_RECURRENT ? recurrent_bwd(*p, *io, s) : chunked_bwd(*p, *io, s);
}

}  // extern "C"

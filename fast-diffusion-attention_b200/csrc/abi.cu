// extern "C" surface of libfda_sm100 (declared in include/fda.h): argument validation with the reference's
// error vocabulary (csrc/fda/flash_api.cpp:92-139, :322-458, :461-643 there), workspace sizing, and the calls
// into the launchers. Nothing here allocates device memory or synchronises, except fda_device_status().
#include "geometry.h"
#include "host_util.h"

namespace fda {

size_t bwd_workspace_bytes(const FdaProblem& p);  // bwd_sm100.cu
size_t fwd_workspace_bytes(const FdaProblem& p);  // fwd_sm100.cu

namespace {

int check_problem(const FdaProblem& p, bool backward) {
  if (p.dtype != FDA_BF16 && p.dtype != FDA_FP16 && p.dtype != FDA_E4M3) return FDA_ERR_DTYPE;
  if (backward && p.dtype == FDA_E4M3) return FDA_ERR_DTYPE;
  if (p.block_size < 1) return FDA_ERR_BLOCK_SIZE;
  if (p.batch < 0 || p.heads < 1 || p.heads_k < 1 || p.seqlen < 0 || p.total < 0) return FDA_ERR_SHAPE;
  if (p.cu_seqlens == nullptr) {
    if (p.seqlen % 2 != 0) return FDA_ERR_ODD_LENGTH;
    if (static_cast<int64_t>(p.batch) * p.seqlen != p.total) return FDA_ERR_SHAPE;
  }
  if (p.head_dim < 8 || p.head_dim > 256) return FDA_ERR_HEAD_DIM;
  if (p.head_dim % (p.dtype == FDA_E4M3 ? 16 : 8) != 0) return FDA_ERR_HEAD_DIM;
  if (p.heads % p.heads_k != 0) return FDA_ERR_HEADS;
  return FDA_OK;
}

}  // namespace
}  // namespace fda

extern "C" {

size_t fda_fwd_workspace_bytes(const FdaProblem* p) {
  if (!p) return 0;
  return fda::fwd_workspace_bytes(*p);
}

size_t fda_bwd_workspace_bytes(const FdaProblem* p) {
  if (!p) return 0;
  return fda::bwd_workspace_bytes(*p);
}

int fda_fwd(const FdaFwdArgs* a, void* stream) {
  if (!a) return FDA_ERR_NULL;
  int rc = fda::check_problem(a->p, false);
  if (rc) return rc;
  if (a->p.total == 0 || a->p.batch == 0) return FDA_OK;
  if (!a->q.ptr || !a->k.ptr || !a->v.ptr || !a->out.ptr || !a->lse) return FDA_ERR_NULL;
  return fda::launch_fwd(*a, static_cast<cudaStream_t>(stream));
}

int fda_bwd_stages(const FdaBwdArgs* a, unsigned stage_mask, void* stream) {
  if (!a) return FDA_ERR_NULL;
  int rc = fda::check_problem(a->p, true);
  if (rc) return rc;
  if (a->p.total == 0 || a->p.batch == 0) return FDA_OK;
  if (!a->q.ptr || !a->k.ptr || !a->v.ptr || !a->out.ptr || !a->dout.ptr || !a->dq.ptr || !a->dk.ptr ||
      !a->dv.ptr || !a->lse) {
    return FDA_ERR_NULL;
  }
  if (!a->workspace || a->workspace_bytes < fda::bwd_workspace_bytes(a->p)) return FDA_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 255) != 0) return FDA_ERR_WORKSPACE;
  return fda::launch_bwd(*a, static_cast<cudaStream_t>(stream), stage_mask);
}

int fda_bwd(const FdaBwdArgs* a, void* stream) { return fda_bwd_stages(a, 7u, stream); }

// Same checks as fda_bwd except for the workspace, which this variant does not take from the caller.
int fda_bwd_noalloc(const FdaBwdArgs* a, void* stream) {
  if (!a) return FDA_ERR_NULL;
  int rc = fda::check_problem(a->p, true);
  if (rc) return rc;
  if (a->p.total == 0 || a->p.batch == 0) return FDA_OK;
  if (!a->q.ptr || !a->k.ptr || !a->v.ptr || !a->out.ptr || !a->dout.ptr || !a->dq.ptr || !a->dk.ptr ||
      !a->dv.ptr || !a->lse) {
    return FDA_ERR_NULL;
  }
  return fda::launch_bwd_noalloc(*a, static_cast<cudaStream_t>(stream));
}

const char* fda_strerror(int status) {
  switch (status) {
    case FDA_OK: return "success";
    case FDA_ERR_NULL: return "a required pointer is NULL";
    case FDA_ERR_DTYPE:
      return "fast-diffusion-attention only supports fp16, bf16 and fp8_e4m3 inputs (backward: fp16 and bf16 only)";
    case FDA_ERR_ODD_LENGTH: return "The sequence length must be even: [noisy half | clean half]";
    case FDA_ERR_BLOCK_SIZE: return "block_size must be a positive integer";
    case FDA_ERR_HEAD_DIM:
      return "head_size must be a multiple of 8 (16 for fp8) and at most 256";
    case FDA_ERR_HEADS: return "Number of heads in key/value must divide number of heads in query";
    case FDA_ERR_STRIDE:
      return "Input tensor must have contiguous last dimension and 16-byte aligned row/head/batch strides";
    case FDA_ERR_DETERMINISTIC: return "deterministic backward is not supported for this head dimension";
    case FDA_ERR_WORKSPACE: return "workspace is missing, misaligned or too small";
    case FDA_ERR_CUDA: return "a CUDA call failed (see fda_last_cuda_error)";
    case FDA_ERR_ARCH: return "fast-diffusion-attention for B200 only supports sm_100 devices";
    case FDA_ERR_UNSUPPORTED: return "this feature combination is not built";
    case FDA_ERR_SHAPE: return "inconsistent tensor sizes";
    case FDA_ERR_DEVICE_WAIT: return "a bounded device-side wait expired";
    case FDA_ERR_SCRATCH_LIMIT:
      return "problem too large for the built-in scratch of fda_bwd_noalloc (FDA_NOALLOC_SCRATCH_BYTES); use fda_bwd "
             "with a caller-provided workspace";
    default: return "unknown status";
  }
}

const char* fda_last_cuda_error(void) { return fda::cuda_error_buf(); }

int fda_device_status(int32_t* out4) {
  if (!out4) return FDA_ERR_NULL;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fda::note_cuda_error(e, "cudaDeviceSynchronize");
  int32_t tmp[4];
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
  int (*readers[4])(int32_t*) = {fda::read_status_fwd, fda::read_status_bwd, fda::read_status_bwd_fused,
                                   fda::read_status_selftest};
  for (auto reader : readers) {
    int rc = reader(tmp);
    if (rc) return rc;
    if (tmp[0] != 0 && out4[0] == 0) {
      for (int i = 0; i < 4; ++i) out4[i] = tmp[i];
    }
  }
  return out4[0] == 0 ? FDA_OK : FDA_ERR_DEVICE_WAIT;
}

const char* fda_version(void) { return "0.1.0"; }

int fda_geom_key_plan(int qh, int qa, int qb, int n, int bs, int bn, int32_t* out_half, int32_t* out_tile, int cap) {
  const fda::KeyPlan plan = fda::make_key_plan(qh, qa, qb, n, bs, bn);
  const int steps = plan.steps();
  for (int s = 0; s < steps && s < cap; ++s) {
    int kh, kt;
    plan.step(s, kh, kt);
    out_half[s] = kh;
    out_tile[s] = kt;
  }
  return steps;
}

int fda_geom_query_plan(int kh, int k0, int k1, int n, int bs, int bm, int32_t* out_half, int32_t* out_tile, int cap) {
  const fda::QueryPlan plan = fda::make_query_plan(kh, k0, k1, n, bs, bm);
  const int steps = plan.steps();
  for (int s = 0; s < steps && s < cap; ++s) {
    int qh, qt;
    plan.step(s, kh, qh, qt);
    out_half[s] = qh;
    out_tile[s] = qt;
  }
  return steps;
}

int fda_geom_classify(int qh, int kh, int qa, int qb, int k0, int bn, int n, int bs, int bm, int need_full_rows) {
  (void)bm;
  if (need_full_rows == 0) {
    // query-tile-stationary form used by the forward and dQ kernels
    return fda::key_span(qh, kh, qa, qb, n, bs).classify(k0, bn);
  }
  // key-tile-stationary form used by the dK/dV kernel: a key tile that runs past n is never "full"
  const int k1 = fda::imin(k0 + bn, n);
  int c = fda::query_span(qh, kh, k0, k1, n, bs).classify(qa, qb - qa);
  if (c == fda::kTileFull && k1 - k0 < bn) c = fda::kTileMasked;
  return c;
}

int fda_geom_item_order(int idx, int per_group, int n_groups, int short8, int ctas, int32_t* out_group, int32_t* out_rank) {
  if (per_group < 1 || n_groups < 1 || ctas < 1 || short8 < 0 || short8 > 8 || idx < 0 ||
      static_cast<long long>(idx) >= static_cast<long long>(per_group) * n_groups || !out_group || !out_rank) {
    return -1;
  }
  const int n_long = fda::order_n_long(per_group, short8, static_cast<long long>(per_group) * n_groups, ctas);
  int group = 0, rank = 0;
  fda::two_phase_order(idx, per_group, n_long, n_groups, group, rank);
  *out_group = group;
  *out_rank = rank;
  return 0;
}

int fda_selftest_wait(long long limit_cycles, void* stream) {
  return fda::launch_selftest_wait(limit_cycles, static_cast<cudaStream_t>(stream));
}

int fda_selftest_umma(int mode, const void* a, const void* b, float* c, int n, int k, void* stream) {
  return fda::launch_selftest_umma(mode, a, b, c, n, k, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

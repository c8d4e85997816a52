/* C ABI of libfda_sm100: block-diffusion attention for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a host framework binds: plain pointers, sizes and element strides, no framework types.
 * It stands where the reference project registers its torch operators `fda::fwd` and `fda::bwd`
 * (csrc/fda/flash_api.cpp:645-682 there) and where its Python layer calls them
 * (fast_diffusion_attention/interface.py:57 and :110).
 *
 * Conventions
 *  - Every sample is [noisy half (n rows) | clean half (n rows)], 2n rows. Batched tensors are
 *    (batch, 2n, heads, head_dim); packed ("varlen") tensors are (total, heads, head_dim) with
 *    cu_seqlens (batch + 1 int32 on the device) and batch strides ignored.
 *  - Strides are in ELEMENTS. The last dimension is contiguous. Base pointers and row/head/batch strides of every
 *    tensor (inputs and outputs) must be multiples of 16 bytes: the kernels move tiles with TMA and rows with
 *    16-byte vector accesses. Anything else is refused with FDA_ERR_STRIDE.
 *  - All pointers are device pointers on the current CUDA device. The library allocates nothing: outputs and
 *    the workspace are the caller's. Work is enqueued on `stream` (a cudaStream_t); no host synchronisation.
 *  - Return value 0 = success, otherwise an FdaStatus; fda_strerror() gives the message. Messages of argument
 *    errors carry the same key words as the reference's checks (flash_api.cpp:96-137, :504-505).
 */
#ifndef FDA_H_
#define FDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum FdaStatus {
  FDA_OK = 0,
  FDA_ERR_NULL = 1,            /* a required pointer is NULL */
  FDA_ERR_DTYPE = 2,           /* unsupported dtype for this pass */
  FDA_ERR_ODD_LENGTH = 3,      /* "The sequence length must be even" */
  FDA_ERR_BLOCK_SIZE = 4,      /* "block_size must be a positive integer" */
  FDA_ERR_HEAD_DIM = 5,        /* head_dim > 256 or not a multiple of 8 (16 for fp8) */
  FDA_ERR_HEADS = 6,           /* heads % heads_k != 0 */
  FDA_ERR_STRIDE = 7,          /* a stride is not a multiple of 16 bytes / last dim not contiguous */
  FDA_ERR_DETERMINISTIC = 8,   /* kept for ABI stability: deterministic backward unsupported for this shape */
  FDA_ERR_WORKSPACE = 9,       /* workspace missing or too small */
  FDA_ERR_CUDA = 10,           /* a CUDA runtime / driver call failed; see fda_last_cuda_error() */
  FDA_ERR_ARCH = 11,           /* the current device is not sm_100 */
  FDA_ERR_UNSUPPORTED = 12,    /* feature combination not built */
  FDA_ERR_SHAPE = 13,          /* inconsistent sizes */
  FDA_ERR_DEVICE_WAIT = 14,    /* a bounded device-side wait expired (reported by fda_device_status) */
  FDA_ERR_SCRATCH_LIMIT = 15   /* fda_bwd_noalloc: the problem needs more scratch than the built-in array holds */
} FdaStatus;

typedef enum FdaDtype { FDA_BF16 = 0, FDA_FP16 = 1, FDA_E4M3 = 2 } FdaDtype;

/* One (rows, heads, head_dim) tensor view. */
typedef struct FdaTensor {
  void* ptr;
  int64_t batch_stride; /* ignored when cu_seqlens != NULL */
  int64_t row_stride;
  int64_t head_stride;
} FdaTensor;

/* Problem description shared by forward and backward.
 * Mirrors the fields of the reference's Qkv_params / Flash_fwd_params that are not sm90-specific
 * (csrc/fda/flash.h:15-137). */
typedef struct FdaProblem {
  int32_t dtype;          /* FdaDtype of q, k, v */
  int32_t batch;          /* number of samples */
  int32_t seqlen;         /* 2n (batched) or the maximum sample length (varlen) */
  int32_t total;          /* total rows: batch * seqlen (batched) or cu_seqlens[batch] (varlen) */
  int32_t heads;          /* query heads */
  int32_t heads_k;        /* key/value heads, divides heads */
  int32_t head_dim;
  int32_t block_size;     /* diffusion block size, >= 1 */
  float softmax_scale;
  float softcap;          /* 0 = off */
  int32_t sm_margin;      /* SMs to leave free */
  int32_t deterministic;  /* backward only: bitwise reproducible accumulation order */
  const int32_t* cu_seqlens; /* device, batch + 1 entries, or NULL */
} FdaProblem;

/* Forward arguments; replaces mha_fwd (csrc/fda/flash_api.cpp:322-458).
 * out: same dtype as q (bf16 for e4m3 inputs). lse: float32, (batch, heads, 2n) or (heads, total) for varlen,
 * natural-log units. Descales: (batch, heads_k) float32 with the given strides, or NULL. */
typedef struct FdaFwdArgs {
  FdaProblem p;
  FdaTensor q, k, v, out;
  float* lse;
  const float* q_descale; const float* k_descale; const float* v_descale;
  int64_t descale_batch_stride[3];
  int64_t descale_head_stride[3];
  void* workspace;          /* fda_fwd_workspace_bytes() bytes, 256-byte aligned */
  size_t workspace_bytes;
} FdaFwdArgs;

/* Backward arguments; replaces mha_bwd (csrc/fda/flash_api.cpp:461-643).
 * dq/dk/dv are written (not accumulated). lse is the forward's output. */
typedef struct FdaBwdArgs {
  FdaProblem p;
  FdaTensor q, k, v, out, dout, dq, dk, dv;
  const float* lse;
  void* workspace;          /* fda_bwd_workspace_bytes() bytes, 256-byte aligned */
  size_t workspace_bytes;
} FdaBwdArgs;

/* Workspace sizes (bytes) for a problem; never fails for valid sizes. Stand in for the allocations the
 * reference makes inside mha_fwd / mha_bwd (flash_api.cpp:396-407, :565-572, :614-625). */
size_t fda_fwd_workspace_bytes(const FdaProblem* p);
size_t fda_bwd_workspace_bytes(const FdaProblem* p);

/* Enqueue the forward / backward pass on `stream`. */
int fda_fwd(const FdaFwdArgs* args, void* stream);
int fda_bwd(const FdaBwdArgs* args, void* stream);

/* Same as fda_bwd but runs only the stages selected by `stage_mask`, in order, on `stream`. Later stages read
 * what earlier ones left in the workspace. For profiling and per-kernel timing; the reference has the same
 * stages as separate launches (csrc/fda/flash_bwd_launch_template.h:47-239).
 * The backward has two forms. The single-pass form (deterministic == 0 and head_dim <= 128) computes dK, dV and
 * the partial dQ of every (key tile, query tile) pair in one kernel and adds the partials into an fp32
 * accumulator in the workspace; the order of those adds varies from run to run. The split form (everything
 * else, or FDA_BWD_FORCE_SPLIT) runs a dK/dV kernel and a dQ kernel with no cross-block reduction; its result
 * is bitwise reproducible. */
#define FDA_BWD_STAGE_PREPROCESS 1u /* delta = rowsum(dO * O) and LSE * log2(e) into the workspace */
#define FDA_BWD_STAGE_MAIN 2u       /* single-pass kernel (with its accumulator zero-fill), or the dK/dV kernel */
#define FDA_BWD_STAGE_DQ 4u         /* accumulator -> dQ conversion, or the dQ kernel */
#define FDA_BWD_FORCE_SPLIT 8u      /* use the split form even where the single-pass form applies */
int fda_bwd_stages(const FdaBwdArgs* args, unsigned stage_mask, void* stream);

/* Backward pass for callers that cannot hand the library a workspace. Some hosts of this library own no device
 * allocator at the point of the call: a serving process whose device memory was carved up at start-up and that
 * forbids allocator calls on its request path, a host language binding that reaches CUDA only through this ABI,
 * or a training loop that runs under a memory plan fixed ahead of time. For them fda_bwd is unusable because it
 * needs fda_bwd_workspace_bytes() of caller-provided scratch. This entry point takes the same arguments but
 * ignores args->workspace / args->workspace_bytes. It always runs the split form of the backward (see
 * fda_bwd_stages), whose scratch is small: the per-row statistics and the two work counters, kept in a fixed
 * array of FDA_NOALLOC_SCRATCH_BYTES that is part of the library image on every GPU that loads it (it is held
 * until the process exits). The caller still provides every input and output tensor; the result is bitwise the
 * one fda_bwd gives with deterministic = 1.
 *  - The scratch need is what fda_bwd_workspace_bytes() returns for the same problem with deterministic = 1.
 *    Problems that need more than the array holds are rejected with FDA_ERR_SCRATCH_LIMIT; nothing is launched.
 *  - It never calls cudaMalloc / cudaFree or any allocating routine. The first call on a device looks up the
 *    device address of the array (cudaGetSymbolAddress) with that device current; make that first call outside
 *    of any stream capture.
 *  - All calls share the one array: two calls whose kernels may overlap on the GPU (different streams, no
 *    ordering between them) race on it. Calls on one stream are safe; each call rewrites what it reads and
 *    re-zeroes the counters itself, so stale contents of an earlier call do not matter.
 * It has no counterpart in the reference, whose operator allocates its workspaces with torch inside the call. */
#define FDA_NOALLOC_SCRATCH_BYTES (16u << 20)
int fda_bwd_noalloc(const FdaBwdArgs* args, void* stream);

/* Message for a status code. */
const char* fda_strerror(int status);
/* Last CUDA error string seen by this thread inside the library ("" if none). */
const char* fda_last_cuda_error(void);

/* Reads and clears the device status words (synchronises the device). out4 = {code, block, thread, detail};
 * code 0 means no bounded wait has expired since the last call. Returns FDA_OK or FDA_ERR_DEVICE_WAIT. */
int fda_device_status(int32_t* out4);

/* Library version "major.minor.patch". */
const char* fda_version(void);

/* ---- host-only geometry probes (no GPU needed); used by the unit tests of the tile enumeration ---------- */
/* Key tiles visited by query rows [qa, qb) of half qh: fills (key_half, key_tile) pairs, returns the count. */
int fda_geom_key_plan(int qh, int qa, int qb, int n, int bs, int bn, int32_t* out_half, int32_t* out_tile, int cap);
/* Query tiles visited by keys [k0, k1) of half kh. */
int fda_geom_query_plan(int kh, int k0, int k1, int n, int bs, int bm, int32_t* out_half, int32_t* out_tile, int cap);
/* 0 skip, 1 fully visible, 2 needs the element mask. need_full_rows = 0 classifies with the query tile fixed
 * (forward, dQ kernel); 1 with the key tile [k0, min(k0 + bn, n)) fixed (dK/dV kernel). Both must agree with the
 * mask; bm is unused. */
int fda_geom_classify(int qh, int kh, int qa, int qb, int k0, int bn, int n, int bs, int bm, int need_full_rows);

/* Position idx of the order in which a persistent kernel takes its items: writes the group (sample x head) and the
 * rank inside the group (0 = longest item). per_group items per group, n_groups groups, `short8` eighths of a group
 * counted as short, ctas persistent blocks; returns 0, or -1 for arguments out of range. No counterpart in the
 * reference (its schedulers are tile_scheduler.hpp:51-482 there). */
int fda_geom_item_order(int idx, int per_group, int n_groups, int short8, int ctas, int32_t* out_group, int32_t* out_rank);

/* ---- tensor-core self test (GPU): C[128 x n] = A[128 x k] * B with the operand layouts the kernels use ---- */
/* mode 0: A, B both K-major from shared memory; mode 1: A from tensor memory, B MN-major from shared memory;
 * mode 2: A and B both MN-major from shared memory (the dQ^T product of the single-pass backward).
 * a, b, c are device pointers: a (128, k) bf16 row-major, for mode 2 its transpose (k, 128) row-major; b (n, k)
 * bf16 row-major for mode 0, (k, n) row-major for modes 1 and 2; c (128, n) float32. k and n are multiples of 64,
 * at most 128 (k) / 256 (n). */
int fda_selftest_umma(int mode, const void* a, const void* b, float* c, int n, int k, void* stream);

/* ---- bounded-wait self test (GPU) ------------------------------------------------------------------------- */
/* Launches one block whose wait on a barrier nobody arrives at gives up after `limit_cycles` SM clocks (1e3 .. 1e8),
 * then leaves through the kernels' ordinary exit path (tensor memory freed, kernel returns). Afterwards
 * fda_device_status() reports FDA_ERR_DEVICE_WAIT with code 110 once, and the device is as usable as before.
 * Every device-side wait of the library is bounded in this way (the kernels' own limit is about two seconds); when
 * fda_device_status() reports an expired wait the outputs of the calls since the last check are undefined.
 * No counterpart in the reference, whose deterministic backward spins without a bound
 * (csrc/fda/mainloop_bwd_sm90_tma_gmma_ws.hpp:641-644). */
int fda_selftest_wait(long long limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FDA_H_ */

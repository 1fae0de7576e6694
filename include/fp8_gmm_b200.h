/*
 * fp8_gmm_b200 -- C ABI of the B200 (sm_100a) FP8 grouped-GEMM library.
 *
 * This header is the drop-in boundary: every entry point replaces one function of the reference's
 * pybind11 module `fp8_gmm_backend` (reference csrc/ops.cu:9-16) or one library call the reference
 * reaches through Transformer Engine.  Signatures use plain pointers and sizes only: no torch, no
 * pybind, no C++ types.  All device pointers are borrowed for the duration of the enqueued work;
 * the caller keeps the memory alive and orders other streams against `stream` itself.
 *
 * Conventions
 *   - every function returns 0 on success and a non-zero fp8gmm_status otherwise; it never throws,
 *     aborts or synchronises the device (except fp8gmm_device_status, which says so);
 *     fp8gmm_last_error() gives a thread-local message for the last non-zero return;
 *   - `stream` is a cudaStream_t passed as void*; NULL means the legacy default stream;
 *   - fp8 buffers are raw bytes in the OCP formats E4M3 (finite-only, max 448) and E5M2 (max 57344);
 *   - "scale" pointers are device fp32; a NULL scale pointer means 1.0; amax pointers may be NULL;
 *   - per-group fp32 metadata is addressed as base[g * stride] (stride in elements), which is how the
 *     reference indexes Transformer Engine's meta vectors (reference fp8_gmm/utils.py:98-103).
 */
#ifndef FP8_GMM_B200_H_
#define FP8_GMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FP8GMM_OK = 0,
  FP8GMM_INVALID_ARGUMENT = 1, /* shape / alignment / NULL-pointer contract violated; nothing was launched */
  FP8GMM_CUDA_ERROR = 2,       /* a CUDA runtime or driver call failed; see fp8gmm_last_error() */
  FP8GMM_UNSUPPORTED = 3,      /* device is not sm_100, or a size exceeds a documented limit */
  FP8GMM_DEVICE_TIMEOUT = 4    /* reported by fp8gmm_device_status(): a bounded wait in a kernel ran out */
} fp8gmm_status;

typedef enum { FP8GMM_E4M3 = 0, FP8GMM_E5M2 = 1 } fp8gmm_format;

typedef enum { FP8GMM_ACT_NONE = 0, FP8GMM_ACT_GELU = 1, FP8GMM_ACT_SWIGLU = 2, FP8GMM_ACT_DSWIGLU = 3 } fp8gmm_activation;

/* Library version (major * 1000 + minor). */
int fp8gmm_version(void);

/* Thread-local, NUL-terminated description of the last failure on this thread ("" if none). */
const char* fp8gmm_last_error(void);

/*
 * Synchronises `stream`, then reads and clears the device-side status word of the current device.
 * Returns FP8GMM_OK, FP8GMM_DEVICE_TIMEOUT (a kernel gave up on a bounded wait and returned without
 * finishing; outputs of that launch are undefined) or FP8GMM_CUDA_ERROR.  Meant for tests and
 * debugging; the hot path does not call it.
 */
int fp8gmm_device_status(void* stream);

/*
 * Enqueues on `stream` a copy of the device-side status word into `host_word` (page-locked host memory owned by
 * the caller) without synchronising and without clearing the word.  A training loop calls it at the end of a step
 * and looks at `*host_word` when it starts the next one: non-zero means a bounded wait ran out in some earlier
 * launch, whose outputs are then undefined.
 */
int fp8gmm_device_status_async(int* host_word, void* stream);

/*
 * Limits of the bounded waits, in nanoseconds, process-wide, for launches made from now on; 0 keeps the current
 * value.  `gemm_wait_ns`: how long a role of the grouped-GEMM kernel waits on an mbarrier (default 1 s).
 * `peer_wait_ns`: how long fp8gmm_peer_wait spins on its sequence numbers (default 2 s) -- raise it where a rank
 * may legitimately be seconds late (a checkpoint write, a stalled data loader).
 */
int fp8gmm_set_wait_limits(int64_t gemm_wait_ns, int64_t peer_wait_ns);

/*
 * Number of kernels this library has launched in this process so far (all devices, all threads).
 * Benchmarks difference it around a timed region to state how much of the work ran in these kernels.
 */
uint64_t fp8gmm_launch_count(void);

/* ------------------------------------------------------------------------------------------------
 * Multi-tensor elementwise kernels (HBM-bound).
 *
 * One descriptor per tensor; any number of tensors per call (the reference caps a call at 64:
 * csrc/multi_pointwise.cu:13, csrc/multi_pad_fusion.cu:14).  Descriptors live in host memory and are
 * consumed before the function returns.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* in;      /* (rows x cols) row-major: bf16 for the cast ops, fp8 for fp8gmm_multi_pad_transpose */
  const void* in2;     /* dgelu: pre-activation bf16 (rows x cols); dswiglu: pre-activation bf16 (rows x 2*cols); else NULL */
  void* out;           /* fp8 (rows x cols) [dswiglu: (rows x 2*cols)], or NULL to skip */
  void* out_t;         /* fp8 (cols x padded_rows) [dswiglu: (2*cols x padded_rows)], rows >= `rows` are padding; or NULL */
  const float* scale;  /* device fp32, NULL = 1.0 */
  float* amax;         /* device fp32, max-merged: *amax = max(*amax, max|x|) over the unscaled values; or NULL */
  int64_t rows;
  int64_t cols;
  int64_t padded_rows; /* >= rows; ignored when out_t is NULL */
} fp8gmm_tensor_desc;

/*
 * bf16 -> fp8 `OType(scale * fp32(x))` (round-to-nearest-even, saturating) + amax, flat over
 * rows*cols elements; `in2`, `out_t`, `padded_rows` are ignored.  `out` may be NULL (amax only).
 * Replaces MultiQuantize (reference csrc/multi_pointwise.h:9-11, csrc/multi_pointwise.cu:155-214).
 */
int fp8gmm_multi_quantize(const fp8gmm_tensor_desc* descs, int count, int out_format, void* stream);

/*
 * fp8 -> fp8 transpose into (cols x padded_rows) with zero bytes in the padding.
 * Replaces MultiPadTranspose (reference csrc/multi_pad_fusion.h:9-11, csrc/multi_pad_fusion.cu:442-503).
 */
int fp8gmm_multi_pad_transpose(const fp8gmm_tensor_desc* descs, int count, void* stream);

/*
 * bf16 -> fp8 cast written twice (same shape to `out`, padded transpose to `out_t`) + amax.
 * Padding bytes are `OType(scale * 0)` exactly as in the reference.
 * Replaces MultiPadCastTranspose (reference csrc/multi_pad_fusion.h:13-19, csrc/multi_pad_fusion.cu:505-585).
 */
int fp8gmm_multi_pad_cast_transpose(const fp8gmm_tensor_desc* descs, int count, int out_format, void* stream);

/*
 * As above with x = in * dgelu_tanh(in2) fused in front of the cast (amax over x).
 * Replaces MultiPadCastTransposeDgelu (reference csrc/multi_pad_fusion.h:21-23, csrc/multi_pad_fusion.cu:587-670).
 */
int fp8gmm_multi_pad_cast_transpose_dgelu(const fp8gmm_tensor_desc* descs, int count, int out_format, void* stream);

/*
 * SwiGLU backward fused in front of the cast: in = d(act) (rows x cols), in2 = pre-activation
 * h = [gate | up] (rows x 2*cols); writes d(h) = [d gate | d up] as fp8 (rows x 2*cols) and its padded
 * transpose (2*cols x padded_rows); one amax over d(h).  No counterpart in the reference (it has
 * GELU only, reference fp8_gmm/grouped_mlp.py:254-287); modelled on the dgelu entry point.
 */
int fp8gmm_multi_pad_cast_transpose_dswiglu(const fp8gmm_tensor_desc* descs, int count, int out_format, void* stream);

typedef struct {
  void* data;          /* bf16, updated in place */
  const float* scale1; /* device fp32, NULL = 1.0 */
  const float* scale2; /* device fp32, NULL = 1.0 */
  int64_t numel;
} fp8gmm_scale_mul_desc;

/*
 * In place x = bf16(fp32(x) * scale1 * scale2).
 * Replaces MultiScaleMul (reference csrc/multi_pointwise.h:13-15, csrc/multi_pointwise.cu:216-259).
 */
int fp8gmm_multi_scale_mul(const fp8gmm_scale_mul_desc* descs, int count, void* stream);

/*
 * Grouped convenience form of fp8gmm_multi_pad_cast_transpose for the layout the modules use
 * (reference fp8_gmm/grouped_linear.py:32-52,133-149): `in` is one (sum rows x cols) bf16 matrix whose
 * row blocks are the groups; group g is cast into out[row_offsets[g]..] and, when out_t != NULL,
 * transposed into the block of out_t that starts at byte t_offsets[g] * cols and holds
 * (cols x (t_offsets[g+1] - t_offsets[g])) bytes.  row_offsets / t_offsets are host arrays of
 * num_groups + 1 prefix sums.  in2 / activation select the fused backward variants (0 none, 1 dgelu,
 * 2 dswiglu); scale and amax are addressed as base[g * stride].
 */
typedef struct {
  const void* in;
  const void* in2;
  void* out;
  void* out_t;
  const int64_t* row_offsets;
  const int64_t* t_offsets;
  int num_groups;
  int64_t cols;
  const float* scale;
  int64_t scale_stride;
  float* amax;
  int64_t amax_stride;
  int out_format;
  int activation;
  int in_is_fp8; /* 1: `in` is already fp8 and the call is a pure padded transpose (scale/amax/out ignored) */
} fp8gmm_grouped_cast_args;

int fp8gmm_grouped_pad_cast_transpose(const fp8gmm_grouped_cast_args* args, void* stream);

/*
 * Cast with a block permutation, for rows that arrive in another order than the grouped GEMM wants them
 * (expert parallelism: an all-to-all delivers rows source-major, the GEMM consumes them expert-major).
 * Block b is `rows[b]` consecutive rows: read from in[src_start[b] ...] (bf16, `cols` wide), cast with
 * scale[group[b] * scale_stride] into out[dst_start[b] ...] (fp8), its amax merged into
 * amax[group[b] * amax_stride].  The four block arrays are HOST int64[num_blocks].  No transposed copy is
 * written (fp8gmm_grouped_pad_cast_transpose on `out` with in_is_fp8 = 1 produces it).  No counterpart in the
 * reference, which is single-GPU (its routing is megablocks gather/scatter, reference fp8_gmm/example.py:52-59).
 */
typedef struct {
  const void* in;
  void* out;
  const int64_t* src_start;
  const int64_t* dst_start;
  const int64_t* rows;
  const int64_t* group;
  int64_t num_blocks;
  int64_t cols;
  const float* scale;
  int64_t scale_stride;
  float* amax;
  int64_t amax_stride;
  int out_format;
} fp8gmm_blocked_cast_args;

int fp8gmm_blocked_cast(const fp8gmm_blocked_cast_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Grouped GEMM (tensor-core bound): tcgen05 / TMEM kernel with TMA-fed FP8 tiles.
 * ---------------------------------------------------------------------------------------------- */

/* Row-map entries that name a destination rank (fp8gmm_gemm_args.c_peers): the rank sits in the bits from this one up,
 * the destination row in the bits below (so a destination buffer holds fewer than 2^26 rows, a group at most 32 ranks). */
#define FP8GMM_ROW_MAP_PEER_SHIFT 26

/*
 * Forward / dgrad:  C_g = act( (A_g B_g^T) * a_scale_inv[g] * b_scale_inv[g] )  for every group g.
 *   a        fp8 (sum m x K) row-major, groups are consecutive row blocks of m_sizes[g] rows
 *   b        fp8 (G x N x K) row-major ("column-major B", both operands K-major)
 *   c        bf16 (sum m x N): the (de-scaled) product, or the pre-activation when activation != NONE
 *   m_sizes  HOST int64[num_groups] (the reference requires a CPU tensor, csrc/fp8_gmm.cu:165-167);
 *            zero-sized groups are allowed
 *   activation != NONE additionally writes act_out = e4m3( act(.) * act_scale[g] ) and merges
 *            max|act(.)| into act_amax[g]: GELU: act_out is (sum m x N); SWIGLU: b holds [gate rows |
 *            up rows] (N = 2F) and act_out is (sum m x N/2).
 *            DSWIGLU (backward; no counterpart in the reference, which has GELU only and runs the
 *            activation backward as a separate cast kernel, fp8_gmm/grouped_mlp.py:254-287): the product is
 *            d(act) (sum m x N), rounded to bf16 as the plain epilogue would store it; with aux_in = the forward
 *            pre-activation [gate | up] it becomes d[gate | up], written as act_out = fp8(. * act_scale[g])
 *            (sum m x 2N, format act_out_format) with max|.| merged into act_amax[g].  c is not written and may be NULL.
 * N and K must be multiples of 16 (the reference assumes the same: fp8_gmm/grouped_linear.py:69).
 * Replaces Fp8GroupedGemm + MultiScaleMul (reference csrc/fp8_gmm.h:7-11, csrc/fp8_gmm.cu:163-205,
 * fp8_gmm/backend.py:78-82) and the per-group te_gemm loop with its GELU-aux epilogue (reference
 * fp8_gmm/backend.py:26-54,84-96).
 */
typedef struct {
  const void* a;
  const void* b;
  void* c;
  const int64_t* m_sizes;
  int num_groups;
  int64_t n;
  int64_t k;
  int a_format;
  int b_format;
  const float* a_scale_inv;
  int64_t a_scale_inv_stride;
  const float* b_scale_inv;
  int64_t b_scale_inv_stride;
  int activation;
  void* act_out;
  const float* act_scale;
  int64_t act_scale_stride;
  float* act_amax;
  int64_t act_amax_stride;
  const int32_t* c_row_map; /* optional, activation == NONE only: device int32[sum m]; row r of the product is stored
                               at row c_row_map[r] of c (lets the epilogue write straight into a buffer laid out for
                               the combine all-to-all); NULL = identity */
  int b_layout;             /* 0: b is (G x N x K), contraction contiguous (forward).  1: b is (G x K x N) row-major,
                               i.e. C_g = A_g B_g without a transpose: what dgrad needs with the forward weights
                               (G x out x in) as they are -- the tensor cores read B MN-major, so the per-expert
                               weight transposes of the reference (fp8_gmm/grouped_linear.py:70-73) are not needed.
                               activation must be NONE or DSWIGLU. */
  const void* aux_in;       /* activation == DSWIGLU only: bf16 (sum m x 2N), the forward pre-activation [gate | up] */
  int act_out_format;       /* activation == DSWIGLU only: fp8 format of act_out (the forward epilogues write E4M3) */
  const void* const* c_peers; /* optional, needs c_row_map: device array of base addresses, one bf16 (rows x n) result
                               buffer per rank of an expert-parallel group (peer-mapped memory of the other GPUs of
                               the node, this GPU's own buffer at its own index).  A c_row_map entry is then
                               (rank << FP8GMM_ROW_MAP_PEER_SHIFT) | row: the epilogue stores the row straight into
                               that rank's buffer with plain stores, so the combine exchange needs no copy; `c` is
                               not used and may be NULL.  The caller orders the launch after the owners of the
                               buffers have released them and signals them after it (fp8gmm_peer_wait /
                               fp8gmm_peer_signal). */
} fp8gmm_gemm_args;

int fp8gmm_grouped_gemm(const fp8gmm_gemm_args* args, void* stream);

/*
 * Weight gradient, one launch for all groups:
 *   C_g (N x K) = (A_t,g  B_t,g^T) * a_scale_inv[g] * b_scale_inv[g]
 * on the padded-transposed operands the cast kernels produce:
 *   a_t  fp8, group g is an (N x L_g) row-major block at byte offset t_offsets[g] * N
 *   b_t  fp8, group g is a  (K x L_g) row-major block at byte offset t_offsets[g] * K
 *   L_g = t_offsets[g+1] - t_offsets[g] must be a multiple of 16; L_g = 0 gives C_g = 0
 *   c    bf16 (G x N x K)
 *   t_offsets  HOST int64[num_groups + 1]
 * `workspace` is device memory of at least fp8gmm_wgrad_workspace_bytes(num_groups) bytes, 128-byte
 * aligned, owned by the caller and reusable as soon as work enqueued on `stream` after this call runs;
 * the call fills it with per-group TMA descriptors by an asynchronous copy on `stream`.
 * Replaces the per-group cublas_fp8_gemm wgrad loop (reference fp8_gmm/grouped_linear.py:165-182,
 * fp8_gmm/grouped_mlp.py:226-242,304-322).
 */
typedef struct {
  const void* a_t;
  const void* b_t;
  void* c;
  const int64_t* t_offsets;
  int num_groups;
  int64_t n;
  int64_t k;
  int a_format;
  int b_format;
  const float* a_scale_inv;
  int64_t a_scale_inv_stride;
  const float* b_scale_inv;
  int64_t b_scale_inv_stride;
  void* workspace;
  size_t workspace_bytes;
} fp8gmm_wgrad_args;

size_t fp8gmm_wgrad_workspace_bytes(int num_groups);
int fp8gmm_grouped_wgrad(const fp8gmm_wgrad_args* args, void* stream);

/*
 * Process-wide switches of the grouped-GEMM launches, for tests and experiments; no counterpart in the reference.
 * ctas: 0 = choose per call (default), 1 = single-CTA 128 x 256 tiles, 2 = CTA-pair 256 x 256 tiles.
 * tail_split (default 1): with pair tiles, group tails of at most 128 rows go to a second launch on 128-row tiles.
 * tma_epilogue (default 1): full 32-row slabs of a tile leave through shared memory and TMA stores.
 * All variants compute every output element with the same arithmetic, so results are bit-identical.
 */
int fp8gmm_set_gemm_variant(int ctas, int tail_split, int tma_epilogue);

/*
 * fp8gmm_grouped_wgrad for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Same arguments and results as fp8gmm_grouped_wgrad, except that `workspace` and
 * `workspace_bytes` are ignored: the per-group TMA descriptors go into a fixed 32 KiB array inside the
 * library image (held by every GPU that loads the library, until the process exits) instead of into
 * caller memory.  It is meant for hosts that own all device memory themselves -- a framework whose pool
 * has already reserved the GPU, so a fresh cudaMalloc would fail or stall the device, or a runtime that
 * forbids plug-ins to allocate after start-up.  Limits and rules:
 *   - at most 128 groups per call; more returns FP8GMM_UNSUPPORTED with a message;
 *   - the call performs no cudaMalloc / cudaFree and calls no allocating library routine;
 *   - the first call on each device resolves the array's device address (with that device current): make
 *     that first call before any stream capture begins.  The call itself copies its descriptors from a
 *     buffer on the host stack, so it returns FP8GMM_UNSUPPORTED on a stream that is being captured (so do
 *     fp8gmm_grouped_wgrad and fp8gmm_grouped_wgrad_rowmajor, whose host staging is as short-lived);
 *   - all calls on one device share the array; each call rewrites every slot it reads, but calls whose GPU
 *     work may overlap (different streams without ordering) race on it -- keep them on one stream;
 *   - host threads are serialised inside the call, so concurrent callers cannot interleave each other's
 *     descriptor copies and launches.
 */
int fp8gmm_grouped_wgrad_static(const fp8gmm_wgrad_args* args, void* stream);

/*
 * Limits the number of SMs the (persistent) grouped-GEMM kernels occupy from now on; 0 restores "all SMs".
 * Process-wide.  Used when a collective runs concurrently on another stream (expert parallelism): a grid that
 * fills every SM would otherwise wait as a whole for the SMs the collective's kernel holds.  No counterpart in
 * the reference.
 */
int fp8gmm_set_gemm_sm_limit(int sms);

/*
 * Weight gradients without the padded-transposed operands: a_t / b_t of fp8gmm_wgrad_args are here the ROW-MAJOR fp8
 * activations, a_t = dY (sum m x n) and b_t = X (sum m x k), and t_offsets the plain row prefix sums of the groups
 * (any sizes, zero allowed; no rounding to 16).  C_g (n x k) = (dY_g * sa[g])^T (X_g * sb[g]); the tensor cores read
 * both operands MN-major, rows past a group's end are zero-filled by TMA.  Same result as fp8gmm_grouped_wgrad on
 * the padded transposes of the same rows (reference fp8_gmm/grouped_linear.py:165-182), without the transposes the
 * reference builds solely for this GEMM (fp8_gmm/grouped_linear.py:32-52,133-149).  Workspace as for
 * fp8gmm_grouped_wgrad.
 */
int fp8gmm_grouped_wgrad_rowmajor(const fp8gmm_wgrad_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Delayed-scaling recipe update (the Transformer Engine hook the reference relies on through
 * prepare_forward, reference fp8_gmm/grouped_linear.py:206): for each of `n` metas
 *   amax = max over history rows (algo 0) or history row 0 (algo 1);
 *   scale = fp8_max / amax / 2^margin where amax is positive and finite, else unchanged;
 *   scale_inv = 1 / scale; history rolled by one row with row 0 zeroed.
 * amax_history is (history_len x n) fp32 row-major, updated in place.
 * ---------------------------------------------------------------------------------------------- */
int fp8gmm_delayed_scaling_update(float* amax_history, float* scale, float* scale_inv, int history_len, int n,
                                  float fp8_max, float margin, int algo, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Router-side row permutation of an MoE block: the steps either side of the grouped GEMMs that the reference's
 * example takes from megablocks (reference fp8_gmm/example.py:26-32 sort / histogram / inclusive_cumsum,
 * :52,:87,:118 gather, :59,:92,:121 scatter).  All pointers are device memory; rows are bf16.
 * ---------------------------------------------------------------------------------------------- */

/* Router (reference fp8_gmm/example.py:14-23: softmax in fp32 over the expert logits, torch.topk, optional
 * renormalisation): logits (tokens x num_experts) fp32 or bf16 -> weights (tokens x top_k) fp32, the top_k largest
 * probabilities in descending order (equal values: lower expert id first), divided by their sum when `renormalize`;
 * experts (tokens x top_k) int32 their ids; probs (tokens x num_experts) fp32 the full softmax, or NULL.
 * num_experts <= 1024. */
int fp8gmm_moe_topk(const void* logits, int logits_are_bf16, int64_t tokens, int num_experts, int top_k, int renormalize,
                    float* probs, float* weights, int32_t* experts, void* stream);

/* Stable counting sort of n = tokens * top_k expert ids (int32, values in [0, num_experts)):
 *   indices[i]  flat (token, slot) position held by sorted row i        bin_ids[i]  expert of sorted row i
 *   inverse[p]  sorted row of flat position p                           tokens_per_expert[e], bins[e] = inclusive cumsum
 * Equal ids keep their order, so the result is deterministic.  An id outside [0, num_experts) is reported through the
 * device status word (see fp8gmm_device_status); its row is left out of the permutation (indices / inverse hold -1
 * there) and the gather / scatter / rowdot kernels skip such entries instead of dereferencing them. */
int fp8gmm_moe_sort(const int32_t* expert_ids, int64_t n, int num_experts, int32_t* indices, int32_t* bin_ids,
                    int32_t* inverse, int64_t* bins, int64_t* tokens_per_expert, void* stream);

/* out[i, :] = x[indices[i] / top_k, :] for i < rows, multiplied by weights[indices[i]] when weights != NULL. */
int fp8gmm_moe_gather(const void* x, const int32_t* indices, const float* weights, int top_k, int64_t rows, int64_t cols,
                      void* out, void* stream);

/* out[t, :] = sum_k weights[t*top_k + k] * x[inverse[t*top_k + k], :] (weights NULL = 1), fp32 accumulation with k
 * ascending, one rounding to bf16. */
int fp8gmm_moe_scatter(const void* x, const int32_t* inverse, const float* weights, int top_k, int64_t tokens, int64_t cols,
                       void* out, void* stream);

/* d_weights[p] = dot(grad[p / top_k, :], x[inverse[p], :]) for p < n: the gradient of the scatter w.r.t. its weights. */
int fp8gmm_moe_rowdot(const void* grad, const void* x, const int32_t* inverse, int top_k, int64_t n, int64_t cols,
                      float* d_weights, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Peer-memory transport for the expert-parallel row exchange (dispatch / combine between the GPUs of one
 * NVSwitch node).  No counterpart in the reference, which is single-GPU apart from one all-reduce
 * (reference fp8_gmm/grouped_mlp.py:300-303) and permutes rows on one device (fp8_gmm/example.py:52-59).
 * Rows move as device-to-device copies executed by the copy engines (no SM is taken from a GEMM running
 * at the same time); completion is announced through per-(receiver, sender) 32-bit sequence numbers.
 * ---------------------------------------------------------------------------------------------- */
#define FP8GMM_PEER_HANDLE_BYTES 64

/* cudaMalloc of `bytes` on the current device plus its CUDA IPC handle (FP8GMM_PEER_HANDLE_BYTES bytes written
 * to `handle`), to be sent to the other ranks.  The first 4 KiB are zeroed (sequence-number pages start at 0). */
int fp8gmm_peer_alloc(size_t bytes, void** ptr, void* handle);
int fp8gmm_peer_free(void* ptr);
/* Maps a buffer another process of this node exported with fp8gmm_peer_alloc; `*ptr` is valid in this process
 * until fp8gmm_peer_close.  Peer access between the two devices is enabled on first use. */
int fp8gmm_peer_open(const void* handle, void** ptr);
int fp8gmm_peer_close(void* ptr);

typedef struct {
  void* dst;       /* local or peer-mapped device address */
  const void* src; /* local or peer-mapped device address */
  size_t bytes;    /* 0 = skipped */
} fp8gmm_copy_block;

/* Enqueues one device-to-device copy per block on `stream`, in order. */
int fp8gmm_peer_copy_blocks(const fp8gmm_copy_block* blocks, int count, void* stream);

/* Block permutation of rows in local memory: for every block b, `rows[b]` consecutive rows of `row_bytes` bytes (a
 * multiple of 16) are copied from row src_start[b] of `src` to row dst_start[b] of `dst`.  The three arrays are HOST
 * int64[num_blocks]; blocks must not overlap at the destination.  Used by the expert-parallel forward to bring rows
 * that arrived source-major (one large copy per sending rank) into the expert-major order the grouped GEMM reads.
 * No counterpart in the reference. */
int fp8gmm_block_permute_rows(const void* src, void* dst, const int64_t* src_start, const int64_t* dst_start,
                              const int64_t* rows, int64_t num_blocks, int64_t row_bytes, void* stream);

/* One-warp kernel on `stream`: stores `value` to each of the `count` (<= 64) addresses in `flags` (host array of
 * device addresses, normally one word in every peer's memory; NULL entries are skipped) with system-scope
 * ordering after everything the stream did before. */
int fp8gmm_peer_signal(uint32_t* const* flags, int count, uint32_t value, void* stream);

/* One-warp kernel on `stream`: returns once all of flags[0..count) (device array in local memory, count <= 64) have
 * reached `value` (compared modulo 2^32).  The wait is bounded (two seconds unless fp8gmm_set_wait_limits changed
 * it); when it runs out the kernel sets a bit in the device status word (see fp8gmm_device_status) and returns. */
int fp8gmm_peer_wait(const uint32_t* flags, int count, uint32_t value, void* stream);

/*
 * Sum of a bf16 buffer over the ranks of a tensor-parallel group in two steps over peer memory (plain peer loads,
 * issued by a few CTAs that run beside the GEMMs).  Replaces the NCCL all-reduce of the MLP's input gradient
 * (reference fp8_gmm/grouped_mlp.py:300-303,323-324) so that it proceeds chunk by chunk behind the fc1 data-gradient
 * GEMM.  `bufs` is a HOST array of `world` device addresses: the same staging buffer on every rank as mapped into
 * this process (fp8gmm_peer_alloc / fp8gmm_peer_open), bufs[rank] being the local one.  The element range
 * [elem_offset, elem_offset + numel) (multiples of 8) is cut into `world` equal slices of 16-byte vectors.
 *   reduce_scatter: slice `rank` of bufs[rank] = sum over r (ascending, fp32, one rounding) of slice `rank` of bufs[r];
 *   all_gather:     out[range] (local memory laid out like the staging buffer) = slice s taken from bufs[s], all s.
 * The caller orders the steps across ranks (fp8gmm_peer_signal / fp8gmm_peer_wait): every rank's partial sums must
 * be complete before any reduce_scatter of the range starts, every reduce_scatter before any all_gather.
 * max_ctas: upper bound on the CTAs used (0 = 64).
 */
int fp8gmm_peer_reduce_scatter_bf16(void* const* bufs, int world, int rank, int64_t elem_offset, int64_t numel, int max_ctas,
                                    void* stream);
int fp8gmm_peer_all_gather_bf16(void* const* bufs, int world, int rank, int64_t elem_offset, int64_t numel, void* out, int max_ctas,
                                void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FP8_GMM_B200_H_ */

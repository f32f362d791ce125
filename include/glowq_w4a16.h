/*
 * glowq_w4a16.h - C ABI of the B200 (sm_100a) corrected W4A16 linear
 *
 *     y_i = dequant(Q_i) . x  +  alpha * L_i . (R_g . x)  (+ bias_i)
 *
 * Q_i: int4 codes, 8 per int32 (nibble j of word w = input column 8w+j), asymmetric, one fp16
 * scale and one 4-bit zero-point per (output row, group of `group_size` input columns); zero-points
 * are packed 8 per int32 the same way.  This is GlowQ's CudaW4A16Linear buffer layout
 * (src/cuda_w4a16/linear.py:42-46, 75-88, 104-106) and is consumed unchanged.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name ends in _host;
 *   - fp16 data are passed as `const void*` (IEEE binary16 bits);
 *   - the caller owns all memory, including outputs, the r cache and the workspace; nothing here
 *     allocates per call (the reference allocates its output and a full fp16 weight temporary per call:
 *     csrc/gemv_w4a16.cu:187, csrc/gemm_w4a16.cu:106);
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and no call synchronises
 *     except the *_host variant and glowq_w4a16_read_status;
 *   - every function returns GLOWQ_OK or a GLOWQ_ERR_* code and never throws or aborts; the
 *     reference reports the same conditions through TORCH_CHECK (csrc/gemv_w4a16.cu:152-185);
 *   - there is no CPU fallback: on a device that is not compute capability 10.x every compute entry
 *     point returns GLOWQ_ERR_UNSUPPORTED_DEVICE.
 */
#ifndef GLOWQ_W4A16_H_
#define GLOWQ_W4A16_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GLOWQ_W4A16_ABI_VERSION 2

enum {
  GLOWQ_OK = 0,
  GLOWQ_ERR_BAD_ARGUMENT = 1,       /* null pointer, non-positive size, rank/mode mismatch          */
  GLOWQ_ERR_BAD_GROUP_SIZE = 2,     /* group_size <= 0 or not a multiple of 8                        */
  GLOWQ_ERR_BAD_STRIDE = 3,         /* packed columns / scales / zero words too few for IC           */
  GLOWQ_ERR_WORKSPACE_TOO_SMALL = 4,
  GLOWQ_ERR_UNSUPPORTED_DEVICE = 5, /* not an sm_100-class GPU                                       */
  GLOWQ_ERR_CUDA = 6,               /* a CUDA runtime call failed; see glowq_w4a16_last_cuda_error   */
  GLOWQ_ERR_DEVICE_TIMEOUT = 7,     /* a bounded device-side wait ran out (read from the status word) */
  GLOWQ_ERR_UNSUPPORTED_SHAPE = 8,
  GLOWQ_ERR_TOO_LARGE = 9
};

enum { GLOWQ_OUT_F16 = 0, GLOWQ_OUT_F32 = 1 };

/* What a launch does about the shared right-factor product r = R_g . x  (the device-side analogue of
 * MiniGroupCache: src/step3_eval_dataset.py:417-444 and the role logic at :481-504). */
enum {
  GLOWQ_R_NONE = 0,    /* plain W4A16 (no wrapper, alpha == 0, or a GlowQ-S group that is switched off) */
  GLOWQ_R_COMPUTE = 1, /* roles q / gate / solo: compute r in this launch and leave it in r_buf           */
  GLOWQ_R_LOAD = 2     /* roles k / v / up on a cache hit: r_buf already holds r for this x               */
};

enum { GLOWQ_KERNEL_AUTO = 0, GLOWQ_KERNEL_GEMV = 1, GLOWQ_KERNEL_GEMM = 2 };

#define GLOWQ_MAX_MEMBERS 4

/* One quantised linear of a group (q_proj, k_proj, ... ). */
typedef struct glowq_w4a16_member {
  const int32_t* qweight; /* [OC, weight_stride_i32]                                          */
  const void* scales;     /* fp16 [OC, scale_stride]                                          */
  const int32_t* qzeros;  /* [OC, zero_stride_i32]                                            */
  const void* bias;       /* fp16 [OC] or NULL                                                */
  const void* L;          /* fp16 [OC, L_stride] left factor (A_q) or NULL = no correction    */
  void* out;              /* [M, out_stride] fp16 or fp32                                     */
  int32_t OC;
  int32_t weight_stride_i32;
  int32_t zero_stride_i32;
  int32_t scale_stride;
  int32_t L_stride;
  int32_t out_stride;
  float alpha;            /* alpha_svd of this member (step3_eval_dataset.py:511)             */
  int32_t reserved;       /* must be 0                                                          */
} glowq_w4a16_member_t;

/* A group of 1..4 linears that consume the same x and share one right factor R_g. */
typedef struct glowq_w4a16_group {
  const void* x;          /* fp16 [M, x_stride]                                               */
  const void* R;          /* fp16 [rank, R_stride] (B_q); used when r_mode == GLOWQ_R_COMPUTE */
  void* r_buf;            /* fp16 [M, rank]: r = R.x, written (COMPUTE) or read (LOAD)        */
  void* workspace;        /* >= glowq_w4a16_workspace_bytes(); zero it once after allocation  */
  size_t workspace_bytes;
  void* stream;           /* cudaStream_t                                                     */
  int32_t M;
  int32_t IC;
  int32_t x_stride;
  int32_t R_stride;
  int32_t rank;           /* 0 with GLOWQ_R_NONE                                              */
  int32_t group_size;
  int32_t r_mode;
  int32_t out_dtype;      /* GLOWQ_OUT_F16 / GLOWQ_OUT_F32 (W4A16_KERNEL_OUT_DTYPE)           */
  int32_t kernel;         /* GLOWQ_KERNEL_AUTO: streaming kernel for M <= 8, tensor-core GEMM above          */
  int32_t n_members;
  int32_t split_k;        /* 0 = choose; >0 forces the number of K slices of the GEMV         */
  int32_t reserved;       /* must be 0 (GLOWQ_ERR_BAD_ARGUMENT otherwise)                       */
  /* Optional hint: the group call that will follow this one on the same stream (NULL = unknown).  Only its
   * pointers and sizes are read, at call time: the streaming kernel asks L2 for the head of that call's packed
   * weights and its right factor while its own launch drains, so that HBM does not idle between launches.
   * Nothing is computed for `next`, and a wrong hint costs bandwidth, not correctness.  The reference has
   * no counterpart (its launches are independent: csrc/gemv_w4a16.cu:194-211). */
  const struct glowq_w4a16_group* next;
  /* Optional, tensor-parallel row-split linears (o_proj, down_proj shards): the launch performs the all-reduce of its
   * result itself.  As its tiles finish it stores this rank's partial sums into slot [push_site][rank] of EVERY rank's
   * `ll_buf`, each element as one 8-byte word {value, epoch} (no fences, no flags), and its last CTAs poll - bounded,
   * status 4 in the workspace on expiry - the words of all ranks' slots in the local `ll_buf`, add them in rank order
   * (fp32) and write the fp16 sums to `out`: when the launch is complete, `out` holds the same bits on every rank.
   * Every rank issues the same call; a site may be reused once the call on the other site has been issued.
   * Requirements: one member, fp16 output, out_stride == OC, M * OC <= peers->max_n and a multiple of 8, M <= 8
   * (the weight-streaming kernel); GLOWQ_ERR_UNSUPPORTED_SHAPE otherwise.  NULL = no push.  See glowq_w4a16_peers_t
   * below for the buffers. */
  const struct glowq_w4a16_peers* push;
  int32_t push_site;
  int32_t reserved2;      /* must be 0 */
  /* Optional input transform fused into the activation staging (the residual add and RMSNorm that sit in front of
   * q/k/v and gate/up in Llama / Qwen decoder blocks; the reference runs them as separate PyTorch modules of the model):
   *     h  = fp16(x + residual)                                  (residual NULL: h = x)
   *     xn = norm_weight * fp16(h * rsqrt(mean_k(h^2) + norm_eps))   (statistics in fp32, per token)
   * and the linears (and r = R . xn) consume xn.  hidden_out, if not NULL, receives h ([M, x_stride] fp16: the new
   * residual stream).  norm_weight NULL = no transform.  Requirements: weight-streaming kernel (M <= 8), IC a multiple
   * of 8, x / residual / norm_weight / hidden_out 16-byte aligned rows; GLOWQ_ERR_UNSUPPORTED_SHAPE otherwise. */
  const void* norm_weight; /* fp16 [IC]                                                        */
  const void* residual;    /* fp16 [M, x_stride] or NULL                                       */
  void* hidden_out;        /* fp16 [M, x_stride] or NULL                                       */
  float norm_eps;
  int32_t reserved3;       /* must be 0 */
  glowq_w4a16_member_t members[GLOWQ_MAX_MEMBERS];
} glowq_w4a16_group_t;

/* ABI version of the loaded library (compare with GLOWQ_W4A16_ABI_VERSION). */
int glowq_w4a16_version(void);

/* Static text for a status code. */
const char* glowq_w4a16_strerror(int status);

/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
int glowq_w4a16_last_cuda_error(void);

/* Dequantise a whole weight: out_w[OC, IC] fp16 = half_rn((code - zero) * scale).
 * Replaces dequant_w4a16_asym_i32_kernel (csrc/gemm_w4a16.cu:19-50); bit-exact with it and with
 * CudaW4A16Linear._dequant_chunk (src/cuda_w4a16/linear.py:248-253). */
int glowq_w4a16_dequant(const int32_t* qweight, const void* scales, const int32_t* qzeros, void* out_w,
                        int OC, int IC, int group_size, int weight_stride_i32, int zero_stride_i32,
                        int scale_stride, void* stream);

/* Plain W4A16 product out[M, OC] (fp16) = x[M, IC] . dequant(Q)^T with the weight-streaming kernel.
 * Replaces w4a16_gemv_forward_cuda / gemv_w4a16_asym (csrc/gemv_w4a16.cu:146-214, csrc/pybind.cpp:19-34).
 * The caller allocates `out`; `workspace` as for a group call. */
int glowq_w4a16_gemv_forward(const void* x, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                             void* out, int M, int IC, int OC, int group_size, int weight_stride_i32,
                             int zero_stride_i32, int scale_stride, void* workspace, size_t workspace_bytes,
                             void* stream);

/* Same product with the tensor-core kernel.  Replaces w4a16_gemm_forward_cuda
 * (csrc/gemm_w4a16.cu:76-135); `split_k_iters` is accepted and ignored as there (:83). */
int glowq_w4a16_gemm_forward(const void* x, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                             void* out, int M, int IC, int OC, int group_size, int split_k_iters,
                             int weight_stride_i32, int zero_stride_i32, int scale_stride, void* workspace,
                             size_t workspace_bytes, void* stream);

/* The corrected linear for a whole group in one launch.  Replaces, per member, the sequence
 * CudaW4A16Linear.forward (src/cuda_w4a16/linear.py:155-187) -> F.linear(x, B_q) or cache hit ->
 * F.linear(r, A_q) -> z.add_(.., alpha) of AddSVDCorrection.forward (src/step3_eval_dataset.py:470-511). */
int glowq_w4a16_group_forward(const glowq_w4a16_group_t* group);

/* `n` group calls issued back to back on their streams, in array order (one C call for a whole token step:
 * the reference pays one Python dispatch per module, src/cuda_w4a16/linear.py:155-187).  Stops at and
 * returns the first failing status.  A call whose `next` is NULL is given its array successor as the hint. */
int glowq_w4a16_group_forward_many(const glowq_w4a16_group_t* groups, int n);

/* Same call with HOST activations: copies x_host[M, IC] (fp16, dense) to group->x, runs the group,
 * copies each member's output to out_host[i] (dense [M, OC_i] in out_dtype) and synchronises the stream.
 * Weights, factors, r_buf and workspace stay device-resident, as the reference keeps them after .to(device)
 * (src/step3_eval_dataset.py:1047-1050). */
int glowq_w4a16_group_forward_host(const glowq_w4a16_group_t* group, const void* x_host, void* const* out_host);

/* Plain W4A16 product like glowq_w4a16_gemv_forward, for callers that cannot hand over a scratch buffer.
 * This entry point has no counterpart in the reference.
 *
 * Some hosts may not allocate device memory on our behalf and cannot size or own a workspace either: a plug-in
 * that only ever receives input and output pointers from its host, a serving loop whose memory plan was frozen
 * before the first request, code that must not touch the CUDA allocator between steps.  For them the scratch
 * (tile counters and split-K partial sums) lives in one array that is part of the library image itself,
 * GLOWQ_W4A16_STATIC_SCRATCH_BYTES large; every GPU that loads the library carries it until the process exits.
 * Calls whose launch plan needs more scratch than that return GLOWQ_ERR_TOO_LARGE and launch nothing.
 *
 * The first call on each device looks up the array's device address (with that device current); make that
 * first call outside any stream capture.  All calls on a device share the one array: the kernels leave their
 * counters at zero when they finish and this entry point re-zeroes the counter area on `stream` before every
 * launch, but two calls that overlap on the GPU (different streams, no ordering between them) race on it.
 * No cudaMalloc / cudaFree or other allocating routine is called. */
#define GLOWQ_W4A16_STATIC_SCRATCH_BYTES (4u << 20)
int glowq_w4a16_gemv_forward_static(const void* x, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                                    void* out, int M, int IC, int OC, int group_size, int weight_stride_i32,
                                    int zero_stride_i32, int scale_stride, void* stream);

/* Tensor-parallel decode: sum a small fp16 vector (the [M, hidden] output of a row-split o_proj / down_proj) over
 * the ranks of one NVLink domain with plain peer stores - no NCCL call, so a token step can be replayed from one
 * CUDA graph.  The reference has no multi-GPU path; this implements the all-reduce point of the tensor-parallel
 * layout (row-split linears) that the benchmark configurations prescribe.
 *
 * Every rank owns a staging buffer of sites * world * max_n fp16 and sites * world uint32 epoch flags, both zeroed
 * once and mapped into every other rank (e.g. torch symmetric memory); `buf[r]` / `flag[r]` are rank r's, as seen
 * from this process.  `epoch` (sites uint32, zeroed once) and `status` (one uint32) are local device memory.  All
 * ranks must make the same sequence of calls per `site`; a site must not be reused before every rank has finished
 * its previous call on it (two sites used alternately are enough).  `inout`: n fp16 values, n % 8 == 0, 16-byte
 * aligned, replaced by the sum.  A rank that waits too long for a peer records status 4 and returns. */
#define GLOWQ_MAX_RANKS 8
typedef struct glowq_w4a16_peers {
  void* buf[GLOWQ_MAX_RANKS];
  void* flag[GLOWQ_MAX_RANKS];
  void* epoch;
  void* status;
  int32_t world, rank, sites, max_n;
  /* Only for launches that push their result themselves (glowq_w4a16_group_t.push): every rank's second staging
   * buffer of sites * world * max_n 8-byte words, zeroed once and mapped into every rank like `buf`.  A pushed
   * element travels as ONE 8-byte store {fp16 value, epoch of the call}: whoever sums polls each word until
   * it carries the current epoch, so neither fences nor flags are involved.  NULL entries: push is refused. */
  void* ll_buf[GLOWQ_MAX_RANKS];
} glowq_w4a16_peers_t;
int glowq_w4a16_allreduce_f16(const glowq_w4a16_peers_t* peers, void* inout, int n, int site, void* stream);

/* The summing half of a pushed all-reduce as a call of its own: poll - bounded, status 4 on expiry - every element of
 * every rank's slot of `site` in the local `ll_buf` until it carries the epoch of this rank's latest push on that
 * site, add the `world` values in rank order (fp32) and write the n fp16 sums to `out`.  A pushing launch does this
 * itself; the call is for callers that want the sum in a second buffer, and yields the same bits. */
int glowq_w4a16_allreduce_finish_f16(const glowq_w4a16_peers_t* peers, void* out, int n, int site, void* stream);

/* Bytes of workspace a group call with these sizes needs (sync words + split-K partial sums). */
size_t glowq_w4a16_workspace_bytes(int M, int IC, int OC_total, int rank, int n_members);

/* Copy the device status word of a workspace to the host (synchronises `stream`) and clear it.
 * Returns GLOWQ_OK or GLOWQ_ERR_DEVICE_TIMEOUT.  workspace == NULL reads the status word of the built-in
 * scratch that glowq_w4a16_gemv_forward_static uses on the current device (that entry point never clears it). */
int glowq_w4a16_read_status(void* workspace, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GLOWQ_W4A16_H_ */

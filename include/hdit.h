/*
 * hdit.h -- C ABI of libhdit_b200.so: hand-written sm_100a kernels for the
 * denoising-stage parallel hot path of Hetu-DiT (USP attention, PipeFusion
 * patch movement, stale-KV scatter, parameter-slice migration).
 *
 * Conventions for every entry point:
 *   - plain pointers and sizes only; all buffers are caller-owned device memory
 *     unless a comment says "host";
 *   - the CUDA stream is passed explicitly as an opaque pointer (cudaStream_t);
 *     calls are asynchronous with respect to the host;
 *   - the return value is an hdit_status; 0 means the work was enqueued.
 *     hdit_last_error() gives a host-side message for the calling thread;
 *   - no entry point allocates device memory. Kernels report a bounded wait
 *     that ran out into a small file-scope device array of the library; read
 *     it with hdit_device_status() (a blocking copy, so synchronise first).
 *   - kernels never trap or spin for ever: every device-side wait has an
 *     iteration limit, after which the kernel records where it gave up and
 *     returns.
 *
 * Each declaration cites the reference (PKU-DAIR/Hetu-DiT, paths relative to
 * its repository root) interface it stands in for.
 */
#ifndef HDIT_H_
#define HDIT_H_

#include <stddef.h>
#include <stdint.h>

#if defined(HDIT_BUILDING) && defined(__GNUC__)
#define HDIT_API __attribute__((visibility("default")))
#else
#define HDIT_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum hdit_status {
  HDIT_OK = 0,
  HDIT_ERR_BAD_ARG = 1,        /* null pointer, negative size, unknown enum   */
  HDIT_ERR_SHAPE = 2,          /* unsupported head_dim / alignment / too many segments */
  HDIT_ERR_CUDA = 3,           /* a CUDA runtime / driver call failed          */
  HDIT_ERR_NOT_INITIALISED = 4,
  HDIT_ERR_PEER_TIMEOUT = 5,   /* a bounded device-side wait ran out           */
  HDIT_ERR_TOO_LARGE = 6       /* exceeds a documented fixed capacity          */
} hdit_status;

typedef enum hdit_dtype { HDIT_BF16 = 0, HDIT_FP16 = 1, HDIT_FP32 = 2 } hdit_dtype;

#define HDIT_MAX_Q_SEG 2
#define HDIT_MAX_KV_SEG 10

/* Library version as major*10000 + minor*100 + patch. */
HDIT_API int hdit_version(void);

/* Host message describing the last non-zero status returned on this thread. */
HDIT_API const char* hdit_last_error(void);

/*
 * Device-side status block: out[0] = code (0 = clean, otherwise an
 * hdit_status), out[1] = blockIdx.x, out[2] = role / wait identifier,
 * out[3] = loop iteration. Synchronise the stream first. `clear` != 0 resets it.
 */
HDIT_API int hdit_device_status(int device, int32_t out[4], int clear);

/* One sequence segment of a (B, S, H, D) tensor whose last dim is contiguous.
 * Strides are in elements. `len` is this segment's S. */
typedef struct hdit_seg {
  const void* ptr;
  int64_t len;
  int64_t stride_b;
  int64_t stride_s;
  int64_t stride_h;
} hdit_seg;

/* How the attention epilogue treats its result. */
typedef enum hdit_attn_mode {
  HDIT_ATTN_FINAL = 0,        /* write softmax(QK^T)V in `dtype` to out (+ lse)                  */
  HDIT_ATTN_PARTIAL_FIRST = 1,/* write fp32 partial result to acc_out, its log-sum-exp to acc_lse */
  HDIT_ATTN_PARTIAL_MERGE = 2,/* log-sum-exp merge with (acc_out, acc_lse), write both back       */
  HDIT_ATTN_MERGE_FINAL = 3   /* merge as above, then write `dtype` to out (+ lse)                */
} hdit_attn_mode;

/*
 * Joint (text + image/video) flash-attention forward on tcgen05/TMEM tiles fed
 * by TMA; non-causal, no dropout, fp32 accumulation, online softmax.
 *
 * Q is the concatenation of n_q_seg segments along S, K/V of n_kv_seg segments
 * (e.g. [image; text] for the "rear" joint strategy, [text; image] for "front",
 * or the KV blocks a ring step contributes); no concatenated copy is ever
 * materialised. Output rows follow the Q concatenation order.
 *
 * Replaces, in the reference:
 *   flash_attn `_flash_attn_forward` as called by ring_flash_attn_forward
 *     (hetu_dit/core/parallel/ring/ring_flash_attn.py:76-87),
 *   the torch.cat of joint K/V around it (:60-71),
 *   `update_out_and_lse` (:88) via the PARTIAL_* / MERGE_* modes,
 *   `flash_attn_func` / F.scaled_dot_product_attention in the attention
 *     processors (hetu_dit/model_executor/diffusion_executor/layers/
 *     attention_processor.py:592,602,752,772,962,969,1139,1149,1516,1524).
 *
 * Requirements: head_dim in {64, 128}; dtype bf16 or fp16; every pointer
 * 16-byte aligned and every stride a multiple of 8 elements; strides of `out`
 * as for a (B, Sq, H, D) tensor; lse is (B, H, Sq) fp32 contiguous (may be
 * NULL in FINAL mode); acc_out is (B, Sq, H, D) fp32 contiguous and acc_lse
 * (B, H, Sq) fp32 contiguous (PARTIAL and MERGE modes only).
 */
typedef struct hdit_attn_args {
  int32_t dtype;      /* hdit_dtype: HDIT_BF16 or HDIT_FP16 */
  int32_t mode;       /* hdit_attn_mode */
  int32_t batch;
  int32_t heads;
  int32_t head_dim;
  int32_t n_q_seg;
  int32_t n_kv_seg;
  float softmax_scale; /* <= 0 selects head_dim^-0.5 */
  hdit_seg q[HDIT_MAX_Q_SEG];
  hdit_seg k[HDIT_MAX_KV_SEG];
  hdit_seg v[HDIT_MAX_KV_SEG];
  void* out;
  int64_t out_stride_b, out_stride_s, out_stride_h;
  float* lse;
  float* acc_out;
  float* acc_lse;
  void* stream;
  /* Optional scatter of the 16-bit result rows over n_out_dst buffers that share out_stride_* (`out` is then
   * unused): row r of Q segment s goes to destination r / q_rows_per_dst[s], at row q_dst_row0[s] +
   * r % q_rows_per_dst[s]; q_rows_per_dst[s] == 0 sends the segment's rows to every destination, at row
   * q_dst_row0[s] + r. With the Ulysses peers' output buffers as destinations (mapped peer memory, plain
   * stores) this is the sequence<-head all-to-all that follows attention, SeqAllToAll4D.apply(ulysses_pg,
   * context, scatter_idx=1, gather_idx=2) at hetu_dit/core/parallel/hybrid/attn_layer.py:134-136, 269-271,
   * 390-392, done by the attention epilogue instead of a separate pass over the context. n_out_dst = 0: off. */
  int32_t n_out_dst;
  /* 0: the library decides, 1: never, 2: always -- run one Q tile per CTA with its two halves on the even and
   * odd KV blocks, merged in shared memory (for grids with fewer Q tile pairs than SMs). */
  int32_t kv_interleave;
  void* out_dst[8];
  int64_t q_rows_per_dst[HDIT_MAX_Q_SEG];
  int64_t q_dst_row0[HDIT_MAX_Q_SEG];
  /* Optional: before its first load every CTA waits (bounded by wait_spins polls, default about 2 s; on expiry
   * HDIT_ERR_PEER_TIMEOUT, where = 9, iteration = silent peer) until each non-NULL wait_slots[p] -- a flag in this
   * rank's memory that peer p bumps, see hdit_norm_rope_args.signal_slots -- has reached *wait_epoch. This is the
   * waiting half of the barrier between the Ulysses head exchange and attention, folded into the consumer.
   * n_wait = 0: off. */
  int32_t n_wait;
  int32_t reserved1;
  const int32_t* wait_slots[8];
  const int32_t* wait_epoch;
  int64_t wait_spins;
} hdit_attn_args;

HDIT_API int hdit_attn_fwd(const hdit_attn_args* args);

/*
 * One strided box to move: n_outer x rows x row_bytes, with independent source and
 * destination pitches (all in bytes). src and dst may live on different GPUs of one
 * NVSwitch domain when the pointer is a mapped peer address.
 */
typedef struct hdit_copy_piece {
  const void* src;
  void* dst;
  int64_t n_outer, src_outer_pitch, dst_outer_pitch;
  int64_t rows, src_pitch, dst_pitch;
  int64_t row_bytes;
} hdit_copy_piece;

/*
 * Moves `n` pieces (host array) with one vectorised, coalesced copy kernel per 40
 * pieces; the piece table travels in kernel parameter space.
 *
 * Replaces, in the reference, the data plane of parameter-slice migration: the
 * NIXL/UCX WRITE built from per-piece descriptors in
 * hetu_dit/core/distributed/nixl_manager.py:186-252 (destination side) and
 * hetu_dit/worker/worker.py:2336-2406 (source side), where a row-split piece is one
 * contiguous span and a column-split piece is one descriptor per weight row (here:
 * one piece with rows = out_features); and the pinned-buffer slice copies of the CPU
 * back-fill, hetu_dit/model_executor/cache/base_cache.py:907-996. It also carries
 * the PipeFusion patch hand-off that the reference does with NCCL isend/irecv,
 * hetu_dit/core/distributed/group_coordinator.py:982-1002.
 */
HDIT_API int hdit_copy_pieces(const hdit_copy_piece* pieces, int64_t n, void* stream);

/*
 * Stale-KV scatter: writes the fresh K and V rows of one PipeFusion patch into the
 * per-layer stale buffer, whose layout is the reference's [K || V] concatenation on
 * the last dim: (batch, cache_tokens, 2 * row_bytes). new_k / new_v hold n_tokens rows
 * of row_bytes each, new_token_pitch / new_batch_pitch bytes apart.
 *
 * Replaces torch.cat([k, v], -1) + kv_cache[:, start:end] = new_kv + torch.chunk in
 * CacheManager.update_and_get_kv_cache / _update_kv_in_dim
 * (hetu_dit/core/resource_manager/cache_manager.py:88-90,113,134-148,186-205,208-231).
 */
HDIT_API int hdit_kv_scatter(void* kv_cache, const void* new_k, const void* new_v, int64_t batch,
                             int64_t cache_tokens, int64_t token_start, int64_t n_tokens, int64_t row_bytes,
                             int64_t new_token_pitch, int64_t new_batch_pitch, void* stream);

/* One tensor handled by hdit_qk_norm_rope: (B, S, H, D) in, the same logical tensor out. */
typedef struct hdit_norm_rope_tensor {
  const void* x;
  int64_t x_stride_b, x_stride_s, x_stride_h;   /* elements; D contiguous */
  const void* norm_weight;                      /* (D) in `dtype`, or NULL for a weightless norm */
  const void* norm_bias;                        /* (D) in `dtype` or NULL; used by the LayerNorm mode only */
  int32_t do_norm;                              /* 0 = no norm, 1 = RMSNorm, 2 = LayerNorm over head_dim */
  int32_t do_rope;                              /* 0 = skip rotary embedding */
  void* dst[8];                                 /* n_dst destinations; dst[j] receives heads [j*H/n_dst, (j+1)*H/n_dst) */
  int64_t dst_stride_b, dst_stride_s, dst_stride_h;
  int64_t dst_seq_offset;                       /* token s lands at row s + dst_seq_offset of the destination */
} hdit_norm_rope_tensor;

/*
 * Fused per-head RMSNorm (or, for the CogVideoX-style QK norm, LayerNorm over head_dim: fp32 arithmetic, one
 * rounding) + rotary embedding for up to three tensors of one layer (Q, K
 * and, copy only, V), written in place, to a plain destination, or head-sliced into
 * n_dst buffers at a sequence offset. With the buffers of the Ulysses peers as
 * destinations this is the head->sequence all-to-all done as peer stores from the
 * QKV-projection epilogue.
 *
 * Replaces, in the reference:
 *   attn.norm_q / norm_k / norm_added_q / norm_added_k calls
 *     (hetu_dit/model_executor/diffusion_executor/layers/attention_processor.py:
 *      552-555, 859-862, 881-888, 1069-1072, 1404-1407, 1452-1455),
 *   apply_rotary_emb, use_real=True, use_real_unbind_dim=-1 (:68-120; call sites
 *     :903-905, :1075-1082, :1410-1434),
 *   SeqAllToAll4D.apply(ulysses_pg, x, scatter_idx=2, gather_idx=1)
 *     (hetu_dit/core/parallel/hybrid/attn_layer.py:102-110, 234-242, 355-363).
 *
 * cos / sin are (rope_rows, D) fp32 tables; token s >= rope_seq_start uses table row
 * (s - rope_seq_start + rope_row0); earlier tokens (e.g. the text prefix of CogVideoX /
 * HunyuanVideo) are not rotated. eps is the RMSNorm epsilon.
 */
typedef struct hdit_norm_rope_args {
  int32_t dtype;
  int32_t batch, seq, heads, head_dim;
  int32_t n_tensors;
  int32_t n_dst;
  float eps;
  const float* cos;
  const float* sin;
  int64_t rope_rows;
  int64_t rope_seq_start;
  int64_t rope_row0;
  hdit_norm_rope_tensor t[3];
  void* stream;
  /* Optional second row range in the same launch: tokens [range2_start, seq) take these norm weights / biases,
   * rotate (or not) per tensor, and use table row (s - range2_start + range2_rope_row0); tokens below it follow
   * the fields above. range2_start <= 0 or >= seq: none. (Text and image rows of a joint sequence differ in
   * their norm weights and rotary rows; one launch covers both.) */
  int64_t range2_start;
  const void* range2_norm_weight[3];
  const void* range2_norm_bias[3];
  int32_t range2_do_rope[3];
  int32_t reserved0;
  int64_t range2_rope_row0;
  /* Optional: when every CTA has stored its rows, the last one publishes the next epoch of `epoch_counter` (a
   * device int32 of this rank, advanced by the kernel) with release / system scope to signal_slots[p] for every
   * p != signal_me -- the signalling half of hdit_peer_barrier folded into the kernel that performs the Ulysses
   * head exchange. `ticket` is a zero-initialised device word the launches of one stream share. n_signal = 0: off. */
  int32_t n_signal;
  int32_t signal_me;
  int32_t* signal_slots[8];
  int32_t* epoch_counter;
  int32_t* ticket;
} hdit_norm_rope_args;

HDIT_API int hdit_qk_norm_rope(const hdit_norm_rope_args* args);

/* ------------------------------------------------------------------------------------------
 * Peer memory within one NVSwitch domain (one process per GPU).
 *
 * The reference keeps a pool of NCCL communicators for every rank subset
 * (hetu_dit/core/distributed/parallel_state.py:1126-1510) and moves activations with NCCL
 * all-to-all / isend / irecv and weights with NIXL. Here every rank owns one symmetric heap
 * that all peers map once; "switching a plan" is choosing which peers' base pointers a kernel
 * receives. The functions below are set-up (they may allocate and synchronise) except the
 * flag kernels.
 * ------------------------------------------------------------------------------------------ */

/* cudaMalloc + zero a heap of `bytes` on the current device (set-up time only). */
HDIT_API int hdit_heap_alloc(int64_t bytes, void** out);
HDIT_API int hdit_heap_free(void* ptr);

/* CUDA IPC handle (64 bytes) of a heap, to be sent to the peers over any host channel. */
HDIT_API int hdit_ipc_export(void* ptr, unsigned char handle[64]);
/* Maps a peer's heap into this process; the returned pointer is valid in kernels of the
 * current device. */
HDIT_API int hdit_ipc_open(const unsigned char handle[64], void** out);
HDIT_API int hdit_ipc_close(void* ptr);

/*
 * Barrier among n <= 8 ranks on `stream`: rank `me` stores `epoch` (release, system scope) to
 * peer_slots[p] in every peer's heap, then polls my_slots[p] in its own heap until it holds at
 * least `epoch`. Everything enqueued on the stream before the call (peer stores included) is
 * visible to the peers' work enqueued after their matching call. Epochs must grow by one per
 * barrier on every rank. With `epoch_counter` (a device int32 of this rank, e.g. in its heap) the
 * kernel takes the epoch from that counter and advances it itself, which keeps a captured CUDA
 * graph containing the barrier replayable; `epoch` is then ignored. After `max_spins` polls without an answer the kernel records
 * HDIT_ERR_PEER_TIMEOUT (where = 100, iteration = silent peer) and returns.
 *
 * Stands in for the synchronisation implied by the reference's NCCL collectives
 * (SeqAllToAll4D, hybrid/attn_layer.py:102-110,134-136; RingComm.wait, ring_flash_attn.py:91).
 */
HDIT_API int hdit_peer_barrier(int32_t* const* peer_slots, const int32_t* const* my_slots, int n, int me,
                               int32_t epoch, int32_t* epoch_counter, int64_t max_spins, void* stream);

/*
 * One-way flag: hdit_peer_signal publishes `value` to a flag in a peer's heap after all earlier
 * work of `stream`; hdit_peer_wait holds `stream` until a flag in the own heap reaches `value`
 * (bounded as above; where = 101, iteration = tag). Together with hdit_copy_pieces into the
 * peer's receive slot they replace PipelineGroupCoordinator.pipeline_isend / pipeline_recv /
 * get_pipeline_recv_data (hetu_dit/core/distributed/group_coordinator.py:931-1002) without the
 * shape handshake of :848-929 (shapes follow from the patch bookkeeping). With `seq_counter` (a device int32 of
 * the calling rank: one per link and direction) the kernel takes the sequence number from that counter and
 * advances it itself, which keeps a captured CUDA graph containing the call replayable; `value` is then ignored.
 */
HDIT_API int hdit_peer_signal(int32_t* flag, int32_t value, int32_t* seq_counter, void* stream);
HDIT_API int hdit_peer_wait(const int32_t* flag, int32_t value, int32_t* seq_counter, int64_t max_spins, int32_t tag,
                            void* stream);

/*
 * hdit_attn_fwd (mode HDIT_ATTN_FINAL) with the KV range split over n_split CTAs per query tile
 * pair, for calls whose grid would leave SMs idle. Replaces the same call sites as hdit_attn_fwd:
 * after the Ulysses all-to-all (hetu_dit/core/parallel/hybrid/attn_layer.py:150-166) a rank holds
 * heads / U heads of the whole sequence, so at U = 8 a 24-head model launches only 3 heads' worth of
 * query tiles -- fewer CTAs than a B200 has SMs.
 *
 * Launch 1 runs the attention kernel on a (tile pairs * heads * batch, splits) grid; split s attends
 * KV blocks [s * ceil(n_blocks / n_split), ...) of the concatenated segment list (blocks of 128 rows,
 * never crossing a segment boundary) and writes a normalised fp32 partial result. Launch 2 merges
 * the partials by log-sum-exp and writes `out` (+ `lse`). The result equals hdit_attn_fwd's up to fp32
 * summation order.
 *
 * split_out: n_split * batch * Sq * heads * head_dim floats, 16-byte aligned; split_lse: n_split *
 * batch * heads * Sq floats. Both are scratch: contents before and after the call mean nothing.
 * n_split in [1, 16]; 1 (or fewer than 2 KV blocks) is hdit_attn_fwd itself.
 */
HDIT_API int hdit_attn_fwd_splitkv(const hdit_attn_args* args, int32_t n_split, float* split_out,
                                   float* split_lse);

/*
 * hdit_attn_fwd in two launches without any caller-provided or freshly allocated scratch.
 * (No counterpart in the reference: it exists for hosts that cannot allocate device memory
 * around the call -- e.g. a serving process whose HBM is entirely owned by its own pool, or a
 * denoising loop that must not incur the device-wide synchronisation of cudaMalloc/cudaFree.)
 *
 * KV segments [0, first_pass_kv_segs) are attended first, the rest second; the second launch merges
 * by log-sum-exp and writes `out` (+ `lse`), so the result equals hdit_attn_fwd(mode = FINAL) over
 * all segments. This is the ring-attention pattern: the local KV block first, the blocks pulled from
 * peers afterwards. args->mode must be HDIT_ATTN_FINAL; acc_out / acc_lse are ignored.
 *
 * The fp32 partial result between the launches lives in a file-scope device array of the library
 * (32 MiB + 512 KiB, held by every GPU that loads the library until exit). Limits:
 * batch * Sq * heads * head_dim <= 8 Mi elements and batch * heads * Sq <= 128 Ki; larger problems
 * get HDIT_ERR_TOO_LARGE. The function calls no cudaMalloc / cudaFree or allocating library routine.
 * The first call on a device looks the array's device address up (cudaGetSymbolAddress); make that
 * first call outside any stream capture. All calls on a device share the one array: two calls that
 * overlap on the GPU (different streams) race; calls on one stream are safe. Nothing in the array has
 * to start at zero -- the first launch overwrites every row the second one reads.
 */
HDIT_API int hdit_attn_fwd_split_static(const hdit_attn_args* args, int32_t first_pass_kv_segs);

/*
 * adaLN-Zero glue around the attention and MLP sub-layers of a DiT block, one pass each.
 *   hdit_ln_modulate  : out[r, :] = LayerNorm(x[r, :]) * (1 + scale[b, :]) + shift[b, :]
 *   hdit_gate_residual: out[r, :] = x[r, :] + gate[b, :] * y[r, :]
 * with b = r / rows_per_batch, LayerNorm without affine parameters (biased variance, `eps`), fp32
 * arithmetic, 16-bit storage. Strides in elements; `dim` a multiple of 8, at most 8192.
 *
 * The reference inherits these steps from the diffusers block definitions it wraps (norm1 / norm1_context
 * modulation and the gated residuals around hetuDiTAttentionWrapper.forward,
 * hetu_dit/model_executor/diffusion_executor/layers/attention_processor.py:207-449, and
 * hetuDiTFeedForwardWrapper.forward, layers/feedforward.py:73-78), where they run as chains of eager
 * elementwise kernels.
 */
HDIT_API int hdit_ln_modulate(int32_t dtype, const void* x, const void* shift, const void* scale, void* out,
                              int64_t rows, int64_t dim, int64_t rows_per_batch, int64_t x_row_stride,
                              int64_t out_row_stride, int64_t mod_batch_stride, float eps, void* stream);
HDIT_API int hdit_gate_residual(int32_t dtype, const void* x, const void* gate, const void* y, void* out,
                                int64_t rows, int64_t dim, int64_t rows_per_batch, int64_t x_row_stride,
                                int64_t y_row_stride, int64_t out_row_stride, int64_t gate_batch_stride, void* stream);

/*
 * out[r, :] = GELU(x[r, :]) with the tanh approximation (fp32 arithmetic, tanh on the special-function
 * unit), rows strided on both sides so the result can land in a column block of a wider buffer.
 * Stands in for the activation inside the MLPs the reference takes from diffusers (call sites
 * hetu_dit/model_executor/diffusion_executor/layers/feedforward.py:73-78).
 */
HDIT_API int hdit_gelu_tanh(int32_t dtype, const void* x, void* out, int64_t rows, int64_t dim, int64_t x_row_stride,
                            int64_t out_row_stride, void* stream);

/*
 * Classifier-free guidance and the flow-matching Euler step of one latent patch, fused:
 *   pred = uncond + guidance_scale * (cond - uncond)        (16-bit arithmetic, one rounding per operation)
 *   out  = sample + ((sample - (sample - round16(pred * sigma))) / sigma) * (sigmas[step_index + 1] - sigma),
 *          sigma = sigmas[step_index]: the operation order of the reference's scheduler wrapper, fp32 with one
 *          rounding per operation after the 16-bit product, the result rounded to the 16-bit type once
 * cond == NULL skips the guidance (uncond is the prediction). `sigmas` is a device array, so the call does not
 * depend on host state and can be replayed from a CUDA graph with the step index baked in. out_peer (optional) gets
 * the same result: with the next pipeline stage's inbox slot as out_peer this is also the wrap-around send of the
 * new latent patch. All pointers 16-byte aligned, n_elems a multiple of 8.
 *
 * Replaces, in the reference, the eager chain of pipeline_stable_diffusion_3.py:1703-1713 (chunk, sub, mul, add)
 * and schedulers/scheduling_flow_match_euler_discrete.py:22-129 (upcast, mul, add, downcast) that runs per patch on
 * the last pipeline stage (:1585-1611), plus the isend of the result (:1625-1631).
 */
HDIT_API int hdit_cfg_euler_step(int32_t dtype, const void* uncond, const void* cond, const void* sample, void* out,
                                 void* out_peer, int64_t n_elems, float guidance_scale, const float* sigmas,
                                 int32_t step_index, void* stream);

/*
 * Linear layer with a fused tail:  out[r, :] = tail(a[r, :] . w^T + bias)  for a (m, k) and w (n, k), both with k
 * contiguous (the layout torch.nn.Linear stores), 16-bit storage, fp32 accumulation on the tensor cores
 * (tcgen05.mma, accumulators in tensor memory), the bias added in fp32 and the sum rounded to the storage type
 * once -- the value an unfused linear layer writes -- before the tail:
 *   HDIT_GEMM_BIAS               : nothing more
 *   HDIT_GEMM_BIAS_GELU_TANH     : GELU, tanh approximation (as hdit_gelu_tanh)
 *   HDIT_GEMM_BIAS_GATE_RESIDUAL : residual[r, :] + gate[r / rows_per_batch, :] * value (as hdit_gate_residual)
 *                                  (rows_per_batch >= 32 unless there is a single batch entry)
 * Row strides (lda, ldw, ldo, ldr, gate_batch_stride) in elements, multiples of 8; pointers 16-byte aligned; n and k
 * multiples of 8; m, n, k ragged against the tile sizes are handled. `out` may alias `residual`. bias may be NULL.
 * tile_m x tile_n: output tile of one CTA, 128 x 256, 128 x 128 or 256 x 256; cta_pair = 2 makes two CTAs of a
 * cluster (an SM pair) share 256 x 256 tiles with tcgen05.mma.cta_group::2, each loading half of the W tile. Zeros
 * let the library choose by the number of waves. max_ctas: 0 = one persistent CTA per SM.
 *
 * In the reference these are the torch.nn.Linear layers of the blocks it wraps followed by eager elementwise
 * kernels: the MLP of hetuDiTFeedForwardWrapper.forward (layers/feedforward.py:73-78: linear, GELU, linear) and the
 * output projections and gated residual additions around hetuDiTAttentionWrapper.forward
 * (layers/attention_processor.py:207-449).
 */
enum { HDIT_GEMM_BIAS = 0, HDIT_GEMM_BIAS_GELU_TANH = 1, HDIT_GEMM_BIAS_GATE_RESIDUAL = 2 };

typedef struct hdit_gemm_args {
  int32_t dtype;     /* HDIT_BF16 / HDIT_FP16 */
  int32_t epilogue;  /* HDIT_GEMM_* */
  int64_t m, n, k;
  const void* a;
  int64_t lda;
  const void* w;
  int64_t ldw;
  const void* bias; /* n elements or NULL */
  void* out;
  int64_t ldo;
  const void* residual; /* (m, n), HDIT_GEMM_BIAS_GATE_RESIDUAL only */
  int64_t ldr;
  const void* gate; /* (m / rows_per_batch, n) */
  int64_t gate_batch_stride;
  int64_t rows_per_batch;
  int32_t tile_n;
  int32_t max_ctas;
  void* stream;
  int32_t tile_m;
  int32_t cta_pair; /* 0 = choose, 1 = never, 2 = always: two CTAs of a cluster share 256 x 256 tiles */
} hdit_gemm_args;

HDIT_API int hdit_linear_fused(const hdit_gemm_args* args);

#ifdef __cplusplus
}
#endif
#endif /* HDIT_H_ */

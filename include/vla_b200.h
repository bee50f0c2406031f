/* C ABI of libvla_b200.so: the Pi0 / Pi05 single-observation forward of realtime-vla on one B200.
 *
 * The reference has no native interface: its boundary is the Python object Pi0Inference / Pi05Inference
 * (pi0_infer.py:1238-1361, pi05_infer.py:530-826).  These entry points are what a Python (ctypes), C or
 * C++ caller binds to get the same object life cycle without Triton or PyTorch: create -> load the
 * converted-checkpoint tensors by key -> finalize (builds tables, captures one CUDA graph) -> forward.
 *
 * Conventions: every function returns 0 on success and a non-zero vla_error otherwise; nothing throws or
 * aborts; vla_last_error() gives the message of the last failure on that handle (or of the last failed
 * vla_create / op call when given NULL).  One handle = one GPU = one stream at a time (not re-entrant,
 * like the reference object with its static buffers).  The caller owns every pointer it passes in; the
 * library owns weights, activations and I/O buffers.
 */
#ifndef VLA_B200_H
#define VLA_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct vla_model* vla_handle;

enum vla_error {
  VLA_OK = 0,
  VLA_ERR_CUDA = 1,        /* a CUDA runtime/driver call failed */
  VLA_ERR_KEY = 2,         /* unknown checkpoint key (the reference raises KeyError, pi0_infer.py:1337-1338) */
  VLA_ERR_SHAPE = 3,       /* shape mismatch (the reference raises RuntimeError from Tensor.copy_) */
  VLA_ERR_STATE = 4,       /* call out of order (e.g. forward before finalize) */
  VLA_ERR_LIMIT = 5,       /* size beyond what the kernels support (keys per query > 1024 tokens etc.) */
  VLA_ERR_DEVICE = 6       /* device-side status word was raised (bounded wait ran out) */
};

enum vla_model_kind { VLA_PI0 = 0, VLA_PI05 = 1 };
enum vla_dtype { VLA_BF16 = 0, VLA_F32 = 1 };

/* Mirrors the constructor arguments: Pi0Inference(checkpoint, num_views, chunk_size) (pi0_infer.py:1239),
 * Pi05Inference(checkpoint, num_views, chunk_size, ..., max_prompt_len) (pi05_infer.py:531-561).
 * prompt_len is the allocated prompt window: len(checkpoint['language_embeds']) for Pi0 and for Pi05 with
 * discrete_state_input=False, max_prompt_len otherwise.  Layer/step counts default to the model's
 * (27 / 18 / 10) when 0; smaller values exist for tests. */
typedef struct vla_config {
  int model;          /* vla_model_kind */
  int num_views;      /* 1..3 camera views of 224x224x3 */
  int chunk_size;     /* action chunk length */
  int prompt_len;     /* allocated prompt tokens */
  int batch;          /* independent observations per forward (1 = the reference's behaviour) */
  int device;         /* CUDA device ordinal */
  int n_vit_layers;   /* 0 -> 27 */
  int n_layers;       /* 0 -> 18 */
  int n_steps;        /* 0 -> 10 */
  int flags;          /* bit 0: disable programmatic dependent launch; bit 1: run without a CUDA graph;
                         bit 2: SigLIP attention on the legacy mma.sync kernel instead of tcgen05;
                         bit 3: prefix / suffix attention of batched forwards on the legacy mma.sync kernel;
                         bit 4: action expert as per-operator launches instead of the persistent kernel (which serves
                                single-observation handles with at most 52 suffix tokens);
                         bit 6: let the tiling model run GEMMs as tcgen05 CTA pairs (two CTAs share an activation tile,
                                each loading half; off by default: measured no faster than single CTAs) */
} vla_config;

/* Replaces Pi0Inference.__init__ / Pi05Inference.__init__ up to buffer allocation (pi0_infer.py:1245-1317). */
int vla_create(const vla_config* cfg, vla_handle* out);

/* Replaces `self.weights[k].copy_(v)` (pi0_infer.py:1337-1338, pi05_infer.py:666-668): `data` is a
 * contiguous host or device tensor of the checkpoint's shape ([in, out] weights, layers stacked on dim 0),
 * bf16 or fp32.  The library repacks it into its own layout.  Any subset of keys may be loaded; keys never
 * loaded stay zero.  'language_embeds' sets the prompt (rows <= prompt_len).  'embedding_weight' ((vocab, 2048),
 * optional) is the token table used by vla_set_prompt_ids. */
int vla_load_weight(vla_handle h, const char* key, const void* data, const int64_t* shape, int ndim, int dtype);

/* Replaces the tail of the constructors: RoPE tables (pi0_infer.py:1319-1335), Pi05 out-projection scaling
 * and time/style precompute (pi05_infer.py:669-722) and record_infer_graph (pi0_infer.py:1347-1354). */
int vla_finalize(vla_handle h);

/* Pi05 per-call prompt (pi05_infer.py:819-822): copies `len` rows of bf16 [len,2048] prompt embeddings
 * (host or device) into the prompt window, sets the valid prefix length and the suffix RoPE start
 * (num_views*256 + len - 1).  For Pi0 it only replaces the prompt rows (len must equal prompt_len).
 * The updates are enqueued on `stream` (a cudaStream_t), like the reference's fill_/copy_ on the current stream:
 * pass the stream the forwards run on and they are ordered between the previous forward and the next. */
int vla_set_prompt(vla_handle h, const void* embeds_bf16, int len, void* stream);

/* Pi05 per-call prompt from token ids (pi05_infer.py:769-785: embedding(ids) * sqrt(2048) in bf16, then the
 * copy into encoder_x, pi05_infer.py:819-822).  Needs the token table loaded with vla_load_weight under the key
 * 'embedding_weight' ((vocab, 2048), the reference's optional checkpoint entry, pi05_infer.py:726-743) BEFORE
 * vla_finalize: the gather then runs inside the captured graph and this call only copies `len` int32 ids (host or
 * device memory) and three scalars.  Ids outside the table are clamped and raise the device status word.
 * The tokenizer stays with the caller.  For Pi0 len must equal prompt_len.  Enqueued on `stream` like vla_set_prompt;
 * host ids may be reused as soon as the call returns. */
int vla_set_prompt_ids(vla_handle h, const int32_t* ids, int len, void* stream);

/* Device address and size of a named library-owned buffer, so that a host framework can wrap it without a
 * copy: "observation_images_normalized" bf16 (batch,nv,224,224,3), "observation_state_normalized" bf16
 * (batch,32) (Pi0), "diffusion_noise" bf16 (batch,chunk,32) (input noise, overwritten by the actions:
 * the reference returns this same buffer, pi0_infer.py:1361), plus intermediate buffers used by the tests
 * ("vision_x", "encoder_x", "encoder_K", "encoder_V", "decoder_x"). */
int vla_buffer(vla_handle h, const char* name, void** dev_ptr, size_t* bytes);

/* Replaces infer_graph.replay() (pi0_infer.py:1360): runs the forward on `stream` (a cudaStream_t, NULL =
 * default stream) over the library-owned I/O buffers.  Asynchronous; the caller synchronises, and a caller that
 * wants to know about device-side trouble reads vla_status_word after synchronising (the reference has no such
 * check; vla_forward_host does it for its callers). */
int vla_forward(vla_handle h, void* stream);

/* Runs a subset of the forward: stage_mask is a combination of 1 = vision towers + projector into the prefix
 * residual stream ("encoder_x", fp32 [batch*P, 2048], view v in rows 256v..256v+255), 2 = prompt rows + prefix
 * prefill (fills the K/V cache), 4 = action expert.  Used by the multi-GPU latency mode, where each view's
 * tower runs on its own GPU and the projected tiles are gathered into the prefill GPU's "encoder_x" between
 * stage 1 and stage 2.  No counterpart in the reference (single GPU, one graph: pi0_infer.py:1232-1236). */
int vla_forward_stages(vla_handle h, int stage_mask, void* stream);

/* ---- multi-view latency mode with the exchange inside the graphs ------------------------------------------
 * None of these has a counterpart in the reference, which runs on one GPU (pi0_infer.py:598-646 processes the views
 * as one batch).  One process per GPU.  A "tower" is a single-view handle that runs stage 1 (vision) for one camera
 * view; the "trunk" is the full handle that runs stages 2 and 4.  After the calls below, the last kernel of a tower's
 * vision stage copies its (256, 2048) fp32 tile with plain peer stores over NVLink into a staging slot of the trunk's
 * mailbox and raises a flag there; the first kernel of the trunk's prefix stage waits for the flags of all views,
 * copies the slots into rows 256 v.. of "encoder_x" and acknowledges to every tower.  Forwards are counted on both
 * sides, two staging slots alternate, and a tower does not overwrite a slot before the trunk has acknowledged the
 * forward that used it, so towers may run ahead of the trunk by one forward and no more.  Every wait gives up after
 * one second and raises the status word.  Every forward must run the vision stage of every tower and the prefix
 * stage of the trunk exactly once (vla_forward_stages(tower, 1), vla_forward_stages(trunk, 2 | 4)).
 *
 * Set-up, after vla_finalize and before the first vla_forward_stages:
 *   trunk process:  vla_link_trunk_create -> 64-byte CUDA IPC handle (for other processes) and the local pointer
 *                   (for a tower in the same process, which cannot open its own process's handle)
 *   tower process:  vla_link_tower_create -> the same pair for the tower's mailbox
 *   exchange the handles (the Python wrapper uses torch.distributed.all_gather_object), vla_link_open them, then
 *   vla_link_tower_connect(tower, trunk mailbox, view, n_views) and, per view, vla_link_trunk_connect(trunk, view,
 *   that tower's mailbox).  Pointers returned by vla_link_open are closed by vla_destroy of the handle given. */
int vla_link_trunk_create(vla_handle trunk, int n_views, unsigned char* ipc_handle_out, void** local_ptr_out);
int vla_link_tower_create(vla_handle tower, unsigned char* ipc_handle_out, void** local_ptr_out);
int vla_link_open(vla_handle h, const unsigned char* ipc_handle, void** ptr_out);
int vla_link_tower_connect(vla_handle tower, void* trunk_mailbox, int view, int n_views);
int vla_link_trunk_connect(vla_handle trunk, int view, void* tower_mailbox);

/* Replaces Pi0Inference.forward / Pi05Inference.forward for a caller holding HOST memory
 * (pi0_infer.py:1356-1361): copies bf16 images/state/noise in, runs, copies the bf16 (batch,chunk,32)
 * actions out and synchronises.  `state` is ignored for Pi05 (may be NULL).  Returns VLA_ERR_DEVICE (and clears the
 * word) when the device status word was raised during the call: the actions are then not to be trusted. */
int vla_forward_host(vla_handle h, const void* images, const void* state, const void* noise, void* actions_out);

/* ---- the steps either side of the forward in a robot loop -----------------------------------------------
 * The reference does these on the host with PIL and numpy in its evaluation script (test.py:82-151, 180-204);
 * here they run on the device and give bit-identical results. */

/* Camera frame -> model input (test.py:99-116, 157-162): `frame` is uint8 (height, width, 3) RGB in host or device
 * memory.  Resized keeping the aspect ratio with Pillow's BILINEAR resample (Image.resize), pasted centred on a
 * black 224 x 224 canvas, scaled to x / 255 * 2 - 1 and stored as bf16 into view `view` of observation `obs` of
 * "observation_images_normalized".  A 224 x 224 frame is only scaled.  Asynchronous on `stream`. */
int vla_preprocess_image(vla_handle h, int obs, int view, const uint8_t* frame, int height, int width, void* stream);

/* Robot state -> model input (test.py:118-131), float64: mode 0 (Pi0) (state - a) / (b + 1e-6) with a = mean,
 * b = std; mode 1 (Pi05) (state - a) / (b - a + 1e-6) * 2 - 1 with a = q01, b = q99.  n <= 32 host values each.
 * For Pi0 the result is rounded to float32 then bf16 and zero-padded into "observation_state_normalized" of
 * observation `obs`; when normalized_out is not NULL the n float64 values are also returned (Pi05 digitises them
 * into prompt tokens on the host, test.py:136-137) and the call synchronises `stream`. */
int vla_preprocess_state(vla_handle h, int obs, const double* state, const double* a, const double* b, int n, int mode,
                         double* normalized_out, void* stream);

/* Action chunk -> robot command (test.py:139-151, 196-200), float64: the bf16 actions of observation `obs` are
 * un-normalised (mode 0: x * (b + 1e-6) + a with a = mean, b = std; mode 1: (x + 1) / 2 * (b - a + 1e-6) + a with
 * a = q01, b = q99; statistics beyond n_stats count as zero), cut to action_dim columns, and the raw state is added
 * (delta -> absolute) except to the last dimension of every 7-wide arm.  `out` (chunk, action_dim) float64, host
 * or device; the call synchronises `stream`. */
int vla_postprocess_actions(vla_handle h, int obs, const double* a, const double* b, int n_stats, int mode,
                            const double* state_raw, int n_state, int action_dim, double* out, void* stream);

/* Device status word: OR of bounded-wait timeouts (bit 0) / shape violations such as a clamped token id (bit 1) seen by
 * any kernel since the last clear (0 = clean).  Synchronises the device. */
int vla_status_word(vla_handle h, int* out);
int vla_clear_status(vla_handle h);

/* Number of kernel launches in one forward, and device bytes held. */
int vla_stats(vla_handle h, int* n_kernels, size_t* device_bytes);

/* Kernel launches of one forward per stage: vision, prefix, decoder (their sum is vla_stats' n_kernels). */
int vla_stage_kernels(vla_handle h, int* n3);

/* Per-stage device time of one forward (ms, CUDA events, outside the graph): vision, prefix, decoder. */
int vla_time_stages(vla_handle h, float* ms3);

/* Timeline of the persistent action-expert kernel (diagnostic, no counterpart in the reference): runs the expert
 * stage once and returns, for every grid barrier of the kernel in order, the time CTA 0 arrived at it and the time
 * it was released (out[2 i], out[2 i + 1], nanoseconds of the GPU's global timer).  The phases per Euler step are:
 * action in-projection, (Pi0) action MLP, then per layer QKV, attention, attention merge, attention-out, GeGLU,
 * down, and finally the out-projection with the Euler update.  *n_written = entries stored (<= max_entries). */
int vla_expert_timeline(vla_handle h, unsigned long long* out, int max_entries, int* n_written);

int vla_destroy(vla_handle h);
const char* vla_last_error(vla_handle h);

/* ---- single operators (used by the kernel-level parity tests and micro-benchmarks) ------------------
 * All pointers are device pointers; `stream` is a cudaStream_t.  Each call repacks/allocates what it needs
 * and frees it before returning (synchronous). */

/* Y = epilogue(X[tokens,K] @ W[K,N]) through the tcgen05 kernel.
 * epi: 0 = bf16 out (+bias, act: 0 none, 1 gelu-tanh, 2 silu, 3 GeGLU with W2), 1 = fp32 residual
 * (outf = res + bias + gate*acc, in place when res == outf), 2 = QKV+RoPE (N must be 2560; q, kcache, vcache out, vt = optional transposed value cache [256, vt_ld]).
 * split = cluster size along K (0 = library heuristic), bn = token tile (0 = heuristic), pair = two 128-feature
 * tiles of W per CTA sharing the activation tile (0 = heuristic, 1 = force, -1 = never; ignored with W2), or
 * 2 = tcgen05 CTA pairs: two CTAs on neighbouring feature tiles share the activation tile, each loading half of it
 * (token tiles of 128 or 256, split <= 4; with W2 only unsplit 256-token tiles),
 * tok_tile = tokens per CTA (0 = heuristic: the token tiles are evened out; else a multiple of 32, <= bn). */
typedef struct vla_gemm_desc {
  const void* x; int tokens; int K;
  const void* w; const void* w2; int N;
  const float* bias; int epi; int act;
  void* out_bf16; int ld_out;
  float* out_f32; const float* res; const float* gate; int res_mod;
  void* q; void* kcache; void* vcache; void* vt; int vt_ld; int pos_off; int rows_per_obs; int kv_obs_stride; int kv_row_off;
  int split; int bn; int iters; float* ms_per_iter;
  int pair;
  int tok_tile;
} vla_gemm_desc;
int vla_op_gemm(const vla_gemm_desc* d, void* stream);

/* O = softmax(mask(Q K^T * scale)) V, bf16.  head_dim 72 or 256.  See attention.cuh for the mask rule. */
typedef struct vla_attn_desc {
  const void* q; const void* k; const void* v; void* o;
  int ldq, ldk, ldv, ldo;
  int groups_outer, groups_inner;
  long long q_go, q_gi, k_go, k_gi, v_go, v_gi, o_go, o_gi;
  int n_q, n_keys, head_dim;
  int prefix_alloc, valid_prefix, restrict_rows;
  float scale; int ksplit; int iters; float* ms_per_iter;
} vla_attn_desc;
int vla_op_attention(const vla_attn_desc* d, void* stream);

/* Same attention on the tcgen05 tensor cores for head dim 256 and one group: q bf16 [n_q,256], k bf16
 * [k_rows,256] (the first n_keys rows are used), vt bf16 [256, vt_ld] = transposed values (vt_ld % 8 == 0),
 * o bf16 [n_q,256].  Mask rule as for vla_op_attention. */
typedef struct vla_attn_tc_desc {
  const void* q; const void* k; const void* vt; void* o;
  int n_q, n_keys, k_rows, vt_ld;
  int prefix_alloc, valid_prefix, restrict_rows;
  float scale; int ksplit; int iters; float* ms_per_iter;
} vla_attn_tc_desc;
int vla_op_attention_tc(const vla_attn_tc_desc* d, void* stream);

/* SigLIP attention on the tcgen05 tensor cores (AttnMultiKey of the reference, pi0_infer.py:588-596): qkv bf16
 * [views * 256, 3456] = [Q | K | V] with 16 heads of 72 each, o bf16 [views * 256, 1152]; per view and head
 * softmax(Q K^T * scale) V over the view's 256 tokens, no mask. */
int vla_op_vit_attention_tc(const void* qkv, void* o, int views, float scale, int iters, float* ms_per_iter, void* stream);

/* Y = X[tokens,K] @ W + bias as bf16, for callers that must not allocate device memory: code running inside
 * a real-time control loop with a fixed memory budget, or on a thread that may not take the allocator's
 * locks.  It has no counterpart in the reference (whose kernels get every buffer from PyTorch's allocator).
 * Same tcgen05 split-K kernel as vla_op_gemm, but it calls no cudaMalloc/cudaFree or any other allocating
 * routine: the caller provides the input, the weight ALREADY in the kernel's layout (bf16 [n_pad, k_pad],
 * i.e. transposed to K-major and zero padded to multiples of 128 x 64) and the output, and the split-K
 * partial tiles go to a 4 MiB scratch array that is part of the library image on every GPU.
 *   - Shapes whose partial tiles exceed 4 MiB (split * token tiles * feature tiles * 128 * tile rows * 4 B;
 *     e.g. more than 128 CTAs of a 64-token tile) are rejected with VLA_ERR_LIMIT.
 *   - The first call on each device looks up the scratch address and sets kernel attributes; make that call
 *     before any stream capture.  Later calls only enqueue the kernel on `stream` (asynchronous).
 *   - split = 0 lets the library choose and then halves its choice until the partial tiles fit the 4 MiB (an unsplit
 *     launch needs none); only an explicit split that does not fit is refused.
 *   - A bounded wait inside the kernel that runs out cannot be reported by this asynchronous call: it sets a status
 *     word that also lives in the library image; vla_op_gemm_noalloc_status (synchronising, allocation-free) returns
 *     and clears it.  Non-zero means the output of an earlier call on this device is not to be trusted.
 *   - All calls share the one scratch array: calls that can overlap on the GPU (different streams) race on it.
 *     Calls on one stream are safe.  Nothing needs clearing between calls: every scratch element a call reads
 *     was written earlier by the same call.  split: 0 = heuristic, else 1, 2, 4 or 8. */
typedef struct vla_gemm_noalloc_desc {
  const void* x; int tokens; int K;
  const void* w_nk; int N; int n_pad; int k_pad;
  const float* bias;
  void* out_bf16;
  int split;
} vla_gemm_noalloc_desc;
int vla_op_gemm_noalloc(const vla_gemm_noalloc_desc* d, void* stream);
int vla_op_gemm_noalloc_status(int* out);

/* y bf16 [rows,D] = norm(x fp32 [rows,D]); mode 0 LayerNorm (w,b), 1 RMS, 2 adaRMS (w = style[3*D]); D 1024|1152|2048. */
int vla_op_norm(const float* x, void* y, int rows, int D, int mode, const float* w, const float* b, void* stream);

#ifdef __cplusplus
}
#endif
#endif

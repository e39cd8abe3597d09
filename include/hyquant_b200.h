/*
 * hyquant_b200 — C ABI of the B200 (sm_100a) hybrid-precision attention path.
 *
 * The reference (jerrysfls/HyQuant) exposes this path only as Python
 * functions (src/ops, src/patch) that launch Triton kernels; it has no C
 * interface of its own.  Each entry point below names the reference function
 * (file:line inside the reference project) whose device work it replaces.  The
 * Python package `hyquant_b200` binds these with ctypes and keeps the
 * reference's Python signatures on top.
 *
 * Conventions
 *  - every pointer is a borrowed DEVICE pointer unless the name says `host`;
 *  - `stream` is a cudaStream_t (pass 0 for the legacy default stream); all
 *    work is stream-ordered and no entry point synchronises the device;
 *  - no entry point allocates or frees device memory: scratch is passed in as
 *    `workspace` (size from the matching *_workspace_bytes call);
 *  - return value: HQ_OK (0) or a negative HQ_ERR_* code; hq_last_error()
 *    returns a thread-local message for the last failure on this thread;
 *  - dtype codes: HQ_BF16 / HQ_F16 / HQ_F32.
 */
#ifndef HYQUANT_B200_H_
#define HYQUANT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HQ_OK                 0
#define HQ_ERR_INVALID       -1   /* bad argument (null pointer, negative size, ...) */
#define HQ_ERR_UNSUPPORTED   -2   /* shape / dtype / bit-width outside what is built */
#define HQ_ERR_ALIGNMENT     -3   /* a pointer or stride breaks a 16-byte rule        */
#define HQ_ERR_WORKSPACE     -4   /* workspace missing or too small                   */
#define HQ_ERR_CUDA          -5   /* a CUDA runtime call failed (see hq_last_error)   */
#define HQ_ERR_TIMEOUT       -6   /* a bounded device-side wait expired               */

#define HQ_BF16 0
#define HQ_F16  1
#define HQ_F32  2

#define HQ_GROUP_SIZE 128         /* staging flush threshold, decode_d_stage.py:19 */

/* Library identification and error text. */
const char* hq_version(void);
const char* hq_last_error(void);

/* --------------------------------------------------------------------------
 * Per-token symmetric INT4 quantise + nibble pack, appended in place.
 * Replaces quantize_per_token(x, 4) + _pack_int4 (src/ops/decode_d_stage.py:50-77,
 * 104-111) as used by DStageLayerCache._flush_staging_buffer and freeze
 * (src/ops/d_stage_kv_cache.py:209-217, 168-169), and removes the torch.cat
 * growth of the prefix (:213-216): rows are written at token `dst_token_offset`
 * of pre-allocated capacity buffers.
 *
 *   x        [BH, n, 128] in_dtype, row stride x_stride_n, head stride x_stride_bh (elements; rows 16-byte aligned,
 *            strides multiples of 8 elements)
 *   packed   int8  [BH, cap, 16 * nbits] (64 bytes per token at 4 bits), head stride packed_stride_bh (bytes; rows
 *            aligned to 2 * nbits bytes)
 *   scale    fp16  [BH, cap],     head stride scale_stride_bh (elements)
 *   scale_mode 0: scale = half(max(|x|,1e-5) / 7)            (IEEE divide; CPU-eager PyTorch)
 *              1: scale = half(max(|x|,1e-5) * (1.0f/7.0f))  (CUDA-eager PyTorch)
 * Codes at 4 bits: q = clamp(rint(x / float(scale)), -8, 7); byte = (q[2i] & 15) | (q[2i+1] << 4).
 * hq_quant_pack takes the bit width (8, 4 or 2: q_max = 127, 7, 1 in place of 7; 8 bits one byte per channel,
 * 2 bits four channels per byte, lowest bits first), reference quantize_per_token / _pack_int2
 * (src/ops/decode_d_stage.py:50-77, 129-135).
 */
int hq_quant_pack(const void* x, int in_dtype, int64_t x_stride_bh, int64_t x_stride_n,
                  int BH, int n, int nbits, void* packed, int64_t packed_stride_bh,
                  void* scale, int64_t scale_stride_bh,
                  int64_t dst_token_offset, int scale_mode, void* stream);
/* nbits = 4 */
int hq_quant_pack_int4(const void* x, int in_dtype, int64_t x_stride_bh, int64_t x_stride_n,
                       int BH, int n,
                       void* packed, int64_t packed_stride_bh,
                       void* scale, int64_t scale_stride_bh,
                       int64_t dst_token_offset, int scale_mode, void* stream);

/* One decode token per head into slot `slot` (0..127) of the staging buffers — the device work of
 * DStageLayerCache.append_staging (src/ops/d_stage_kv_cache.py:195-207) for a single new token.
 *   k_new/v_new bf16 [BH, 128] with row strides in elements; staging_k/v bf16 [BH, 128, 128]. */
int hq_staging_append(const void* k_new, const void* v_new, int64_t k_stride, int64_t v_stride,
                      void* staging_k, void* staging_v, int BH, int slot, void* stream);

/* --------------------------------------------------------------------------
 * Split-K decode attention over the four-segment cache, one launch.
 * Replaces fused_d_stage_decode / fused_d_stage_decode_splitk and the kernels
 * _fused_d_stage_decode_kernel, _splitk_partial_kernel, _splitk_reduce_kernel
 * (src/ops/decode_d_stage.py:916-1005, 823-913, 270-469, 481-743, 746-782),
 * i.e. the device work of DStageLayerCache.decode_attention
 * (src/ops/d_stage_kv_cache.py:219-303), without the torch.cat of the BF16
 * segments (:848-849).
 *
 * Strides are in ELEMENTS of the tensor's dtype except where noted.  The
 * innermost (channel) dimension must be contiguous; packed rows must be 64
 * bytes apart and BF16 rows 128 elements apart; every base pointer and head
 * stride must keep rows 16-byte aligned (HQ_ERR_ALIGNMENT otherwise).
 */
/* hq_decode_args.flags.  HQ_DECODE_OVERLAP_PREVIOUS launches the kernel with programmatic
 * stream serialisation: its blocks may become resident while the kernel launched just before
 * it on the same stream is still finishing, and they fetch their first cache units in that
 * time.  q, the staging buffers, the newest 128 tokens of the INT4 prefix (codes and scales),
 * the output and the workspace are touched only after the previous kernel has completed, so
 * the previous kernel may write any of those (a staging append, a staging flush, the producer
 * of q, the previous decode call).  The caller promises that it writes nothing else of this
 * call's cache: not the older prefix, nor the vertical-line and window segments. */
#define HQ_DECODE_OVERLAP_PREVIOUS 1

typedef struct hq_decode_args {
  int32_t struct_bytes;        /* sizeof(hq_decode_args), checked */
  int32_t BH_KV;               /* batch * kv heads */
  int32_t kv_repeat;           /* query heads per kv head (1..16) */
  int32_t head_dim;            /* 128 */
  int32_t n_quant;             /* quantised prefix tokens */
  int32_t n_topk;              /* frozen BF16 vertical-line tokens */
  int32_t n_staging;           /* live tokens in the staging buffer (0..128) */
  int32_t n_window;            /* BF16 window tokens */
  int32_t out_dtype;           /* HQ_BF16 / HQ_F16 / HQ_F32 */
  int32_t num_splits;          /* 0 = choose automatically */
  float   sm_scale;            /* softmax scale, e.g. head_dim^-0.5 */
  int32_t flags;               /* 0, or HQ_DECODE_OVERLAP_PREVIOUS */
  int32_t k_bits;              /* bit width of the quantised K prefix: 8, 4 or 2 (0 = 4) */
  int32_t v_bits;              /* the same for V; every pair is one instantiation of the same kernel */
  const void* q;               /* bf16 [BH_KV*kv_repeat, 128] */
  int64_t q_stride;            /* elements between query rows */
  const void* k_packed;        /* int8 [BH_KV, n_quant, 16 * k_bits] (4 bits: 64 bytes per token) */
  const void* v_packed;        /* Any placement works.  When k_bits == v_bits and the two are planes of one
                                * tensor [BH_KV, 2, cap, row] (v_packed = k_packed + cap * row bytes, both head
                                * strides = 2 * cap * row), a unit's K and V rows are fetched with one tensor-map
                                * request instead of two copies; results are the same bit for bit. */
  int64_t kp_stride_bh;        /* BYTES between heads */
  int64_t vp_stride_bh;
  const void* k_scale;         /* fp16 [BH_KV, n_quant] */
  const void* v_scale;
  int64_t ks_stride_bh;
  int64_t vs_stride_bh;
  const void* k_topk;          /* bf16 [BH_KV, n_topk, 128] */
  const void* v_topk;
  int64_t kt_stride_bh;
  int64_t vt_stride_bh;
  const void* k_staging;       /* bf16 [BH_KV, n_staging, 128] */
  const void* v_staging;
  int64_t kg_stride_bh;
  int64_t vg_stride_bh;
  const void* k_window;        /* bf16 [BH_KV, n_window, 128] */
  const void* v_window;
  int64_t kw_stride_bh;
  int64_t vw_stride_bh;
  void*   out;                 /* out_dtype [BH_KV*kv_repeat, 128]; may be NULL in partial mode */
  int64_t out_stride;
  /* Partial mode (sequence-sharded decode): when partial_acc != NULL the
   * un-normalised base-2 softmax state of this shard is written instead of
   * `out`: partial_m/partial_l fp32 [BH_Q], partial_acc fp32 [BH_Q, 128]. */
  float*  partial_m;
  float*  partial_l;
  float*  partial_acc;
  void*   workspace;           /* hq_decode_workspace_bytes(); zero-filled once by the caller */
  int64_t workspace_bytes;
  /* Optional: the step's new token, bf16 [BH_KV, 128] with row strides in elements.  The call
   * attends to it in addition to the n_staging tokens already in the staging buffers and copies it into
   * staging slot n_staging, so the caller need not append it first (a fused form of the reference's
   * append_staging + decode_attention, src/ops/d_stage_kv_cache.py:195-303).  The caller then counts it. */
  const void* k_new; const void* v_new; int64_t kn_stride; int64_t vn_stride;
  /* Optional: sequence-sharded decode in one launch.  With peer_world > 1 the call covers this rank's shard of the
   * sequence, stores its un-normalised softmax state into the peers' exchange buffers (peer_bufs[j]: rank j's buffer
   * of hq_peer_exchange_bytes(peer_world, BH_KV * kv_repeat) bytes as addressable from this process), waits - with
   * the time limit - for theirs and writes the merged, normalised result to `out`, like hq_peer_exchange_merge
   * below but without a second launch.  peer_seq = 1, 2, 3, ..., the same on every rank for the same call, shared
   * with hq_peer_exchange_merge calls on the same buffers.  partial_* must be NULL. */
  void* const* peer_bufs; int32_t peer_world; int32_t peer_rank; uint32_t peer_seq; int32_t peer_reserved;
  int64_t peer_timeout_ns;     /* 0 = 2 s */
  /* Optional: a device record {int32 n_quant, int32 n_staging} that overrides the two fields above when the kernel
   * runs, so that a launch captured in a CUDA graph stays valid while the cache grows (the reference keeps both on
   * the host and grows its tensors with torch.cat, src/ops/d_stage_kv_cache.py:195-217).  n_quant / n_staging above
   * are then only used to choose the split count.  The record must be complete before the kernel launched just
   * before this one starts (e.g. written by the copy that brings the step's inputs), because an overlapped launch
   * (HQ_DECODE_OVERLAP_PREVIOUS) reads it at once; the staging pointers must be set. */
  const int32_t* lengths;
  /* Optional: rotary position embedding applied inside the call (rotate_half form, bf16 arithmetic of Hugging Face's
   * apply_rotary_pos_emb, which the reference's patched forwards run as separate eager kernels before the cache,
   * src/patch/patch_llama.py:58-65): q and k_new arrive UNROTATED, the kernel rotates the query rows while it loads them
   * and the new K row both where it attends to it and where it stores it into the staging buffer (V is not rotated).
   * rope_cos / rope_sin: bf16 [batch, 128], rope_stride elements between batch rows; rope_heads_per_batch = kv heads
   * per batch entry (head index / rope_heads_per_batch selects the row). */
  const void* rope_cos; const void* rope_sin; int64_t rope_stride; int32_t rope_heads_per_batch; int32_t rope_reserved;
} hq_decode_args;

int hq_decode_workspace_bytes(int BH_KV, int kv_repeat, int64_t* bytes);
int hq_decode_splitk(const hq_decode_args* args, void* stream);

/* The same decode call for callers that cannot supply device scratch: hosts that forbid
 * cudaMalloc inside their callbacks, or processes whose GPU memory belongs to another
 * allocator.  It has no counterpart in the reference.  The split-K partials and tickets
 * live in a 4 MiB array that is part of the library image (each GPU that loads the library
 * holds it until exit); `workspace` / `workspace_bytes` in `args` are ignored.  Shapes that
 * need more than 4 MiB of scratch (see hq_decode_workspace_bytes) fail with HQ_ERR_WORKSPACE.
 * The first call on a device resolves the array's device address: make it before any stream
 * capture.  All calls share the array, so calls that can overlap on the GPU race — issue them
 * in one stream.  Allocates nothing.  The ticket words are cleared in-stream before every call; the
 * status word (bit 0: a bounded device wait ran out, that call's output is invalid) is left to accumulate
 * until hq_decode_static_status, a synchronising call, reads and clears it. */
int hq_decode_splitk_static(const hq_decode_args* args, void* stream);
int hq_decode_static_status(int* status);

/* --------------------------------------------------------------------------
 * Log-sum-exp merge of G shards' partials (the algebra of _splitk_reduce_kernel,
 * src/ops/decode_d_stage.py:764-781, applied across GPUs after an all-gather).
 *   m, l  fp32 [G, rows];  acc fp32 [G, rows, 128];  out out_dtype [rows, 128]
 */
int hq_lse_merge(const float* m, const float* l, const float* acc, int G, int rows,
                 void* out, int out_dtype, int64_t out_stride, void* stream);
/* The same with a stride (in floats) between consecutive shards of each array, for partials that arrive as one
 * message per shard (m | l | acc back to back, all-gathered into [G][rows * 130]). */
int hq_lse_merge_strided(const float* m, const float* l, const float* acc, int64_t m_stride, int64_t l_stride,
                         int64_t acc_stride, int G, int rows, void* out, int out_dtype, int64_t out_stride, void* stream);
/* The merged state left un-normalised: out_m, out_l fp32 [rows], out_acc fp32 [rows, 128] (a further merge can follow). */
int hq_lse_merge_partial(const float* m, const float* l, const float* acc, int64_t m_stride, int64_t l_stride,
                         int64_t acc_stride, int G, int rows, float* out_m, float* out_l, float* out_acc, void* stream);

/* ---- sequence-sharded decode: exchange + merge over peer memory, one launch per call ----------------------
 * No counterpart in the reference (its decode call, src/ops/d_stage_kv_cache.py:219-303, runs on one GPU).
 * Each rank holds a shard of the sequence, runs hq_decode_splitk in partial mode with partial_m / partial_l /
 * partial_acc pointing into its own exchange buffer (hq_peer_slot), then launches hq_peer_exchange_merge: the
 * kernel stores the rank's (m, l, acc) elements into every peer's buffer through peer pointers (plain 8-byte stores
 * over NVLink, no multicast; each carries the value and the call's sequence number), polls its own buffer for the
 * peers' elements with a time limit and writes the merged, normalised result.  A wait that runs out sets bit 1 of the buffer's first
 * word (the status) and the call completes with whatever arrived.
 *   bufs[j]: rank j's exchange buffer as addressable from this process (bufs[rank] is the local one);
 *   seq: 1, 2, 3, ... - the same value on every rank for the same call; rows = batch * query heads.
 * hq_peer_buffer_create / open / close / destroy allocate an exchange buffer with cudaMalloc (zero-filled) and
 * share it between the processes of one node through a 64-byte CUDA IPC handle. */
typedef struct hq_peer_exchange_args {
  int32_t struct_bytes;
  int32_t world, rank, rows;
  uint32_t seq;
  int32_t out_dtype;
  int64_t out_stride;          /* elements between output rows */
  void*   out;                 /* out_dtype [rows, 128] */
  int64_t timeout_ns;          /* limit of the wait for the peers; 0 = 2 s */
  void*   bufs[16];
} hq_peer_exchange_args;
int hq_peer_exchange_bytes(int world, int rows, int64_t* bytes);
int hq_peer_slot(void* buf, int world, int rows, uint32_t seq, float** m, float** l, float** acc);
/* Where rank src_rank's elements of call seq arrive in `buf`: rows * 130 words of {fp32 value, uint32 seq}, in the
 * order m [rows] | l [rows] | acc [rows][128] (for tests and tools; the kernel addresses it itself). */
int hq_peer_recv_slot(void* buf, int world, int rows, uint32_t seq, int src_rank, void** words);
int hq_peer_exchange_merge(const hq_peer_exchange_args* a, void* stream);
int hq_peer_status(const void* buf, int* status);     /* synchronising read of the local buffer's status word */
int hq_peer_buffer_create(int64_t bytes, void** ptr, void* handle64);
int hq_peer_buffer_open(const void* handle64, void** ptr);
int hq_peer_buffer_close(void* ptr);
int hq_peer_buffer_destroy(void* ptr);


/* --------------------------------------------------------------------------
 * Vertical-line scores: mean of the last `tail_len` queries, dotted with every
 * candidate key.  Replaces the mean/matmul/einsum of compute_vertical_indices
 * (src/patch/_common.py:161-185).
 *   q       io_dtype [B, H_Q, n_q, 128] (strides in elements)
 *   k       io_dtype [B, H_KV, *, 128]; candidates are rows [0, n_cand)
 *   pooled  fp32 [B, H_Q, 128]  (out: the pooled query; also the kernel's scratch)
 *   scores  fp32 [B, H_Q, n_cand]
 * kv_repeat = H_Q / H_KV.  round_mean != 0 rounds the pooled query to io_dtype
 * first (what the reference's in-dtype mean does); round_scores != 0 rounds the
 * scores to io_dtype as the reference's in-dtype matmul does.
 */
int hq_vertical_scores(const void* q, int io_dtype, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                       int B, int H_Q, int n_q, int tail_len,
                       const void* k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                       int H_KV, int n_cand, int round_mean, int round_scores,
                       float* pooled, float* scores, void* stream);

/* The same for the selection inside DStageLayerCache.freeze (src/ops/d_stage_kv_cache.py:131-136): the saved
 * queries q [B, H_KV * group, n_q, 128] are first averaged over the `group` query heads of each kv-head (per token,
 * rounded to io_dtype like the reference's in-dtype mean), then pooled and scored per KV head:
 * pooled fp32 [B, H_KV, 128], scores fp32 [B, H_KV, n_cand]. */
int hq_vertical_scores_grouped(const void* q, int io_dtype, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                               int B, int H_KV, int group, int n_q, int tail_len,
                               const void* k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                               int n_cand, int round_mean, int round_scores,
                               float* pooled, float* scores, void* stream);

/* Top-k of each row of `scores` ([rows, n] fp32, row stride `scores_stride`),
 * descending, ties towards the lower index.  Replaces torch.topk(..., sorted=True)
 * in compute_vertical_indices (src/patch/_common.py:187-190).  idx_desc int64
 * [rows, k]; idx_asc int32 [rows, k] (the same set in ascending position, may be
 * NULL).  1 <= k <= min(n, 16384).  Uses no global scratch. */
int hq_topk(const float* scores, int64_t scores_stride, int rows, int n, int k,
            int64_t* idx_desc, int32_t* idx_asc, void* stream);

/* --------------------------------------------------------------------------
 * Prefill -> decode cache reorganisation.  Replaces the gather / scatter / sort
 * / gather / quantise chain of DStageLayerCache.freeze
 * (src/ops/d_stage_kv_cache.py:119-169).
 *   keys/values io_dtype(bf16) [BH, N, 128] (head stride kv_stride_bh, row stride 128)
 *   prefix_len  = N - W; window rows [prefix_len, N) are copied to k/v_window
 *   vidx_desc   int64 [BH, T] rows to keep in BF16, in output order
 *   vidx_asc    int32 [BH, T] the same rows in ascending position
 *   k/v_topk    bf16 [BH, T, 128]
 *   packed/scale as in hq_quant_pack_int4, written from token 0; n_quant = prefix_len - T
 */
int hq_cache_reorganize(const void* keys, const void* values, int64_t kv_stride_bh,
                        int BH, int N, int window, int T,
                        const int64_t* vidx_desc, const int32_t* vidx_asc,
                        void* k_topk, void* v_topk,
                        void* k_window, void* v_window,
                        void* k_packed, void* v_packed, int64_t packed_stride_bh,
                        void* k_scale, void* v_scale, int64_t scale_stride_bh,
                        int scale_mode, void* stream);
/* The same with a bit width per tensor (8, 4 or 2) and a head stride per packed tensor. */
int hq_cache_reorganize_bits(const void* keys, const void* values, int64_t kv_stride_bh,
                             int BH, int N, int window, int T,
                             const int64_t* vidx_desc, const int32_t* vidx_asc,
                             void* k_topk, void* v_topk, void* k_window, void* v_window,
                             void* k_packed, void* v_packed, int64_t kp_stride_bh, int64_t vp_stride_bh,
                             void* k_scale, void* v_scale, int64_t scale_stride_bh,
                             int k_bits, int v_bits, int scale_mode, void* stream);

/* --------------------------------------------------------------------------
 * Hybrid prefill, step 1: operand preparation.  Replaces per_block_int8 and the
 * K-smoothing / query pre-scaling of sage_vertical_attention_v2
 * (src/ops/vendor/sageattention/triton/quant_per_block.py:21-101,
 *  src/ops/sage_unified.py:565-576).
 *   q [B,H_Q,N,128] bf16, k [B,H_KV,N,128] bf16 (strides in elements)
 *   q_i8 int8 [B,H_Q,N,128], q_bf bf16 (contiguous copy of q), q_scale fp32 [B,H_Q,Npad] (one per row; Npad = N rounded up to 64)
 *   k_i8 int8 [B,H_KV,N,128], k_bf bf16 (k - mean), k_scale fp32 [B,H_KV,Npad], k_mean bf16 [B,H_KV,128]
 * smooth_k == 0 leaves K unshifted.
 */
int hq_prefill_quant_workspace_bytes(int B, int H_KV, int64_t* bytes);
int hq_prefill_quant(const void* q, int64_t q_sb, int64_t q_sh, int64_t q_sn,
                     const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn,
                     int B, int H_Q, int H_KV, int N, float sm_scale, int smooth_k,
                     void* q_i8, void* q_bf, float* q_scale,
                     void* k_i8, void* k_bf, float* k_scale, void* k_mean,
                     void* workspace, int64_t workspace_bytes, void* stream);

/* The same preparation with the reference's scale granularity: one scale per block of 128 query rows and per
 * block of 64 key rows (per_block_int8 with BLKQ = 128, BLKK = 64, quant_per_block.py:49-101).  The scale arrays
 * keep the per-row layout above (a block's scale repeated for each of its rows), so hq_prefill_hybrid runs
 * unchanged on either. */
int hq_prefill_quant_blocks(const void* q, int64_t q_sb, int64_t q_sh, int64_t q_sn,
                            const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn,
                            int B, int H_Q, int H_KV, int N, float sm_scale, int smooth_k,
                            void* q_i8, void* q_bf, float* q_scale,
                            void* k_i8, void* k_bf, float* k_scale, void* k_mean,
                            void* workspace, int64_t workspace_bytes, void* stream);

/* One tensor through the reference's block quantiser, quant_per_block_int8_kernel
 * (src/ops/vendor/sageattention/triton/quant_per_block.py:21-47), bit for bit (the two fp32 divisions are the
 * approximate div.full.f32 the Triton kernel compiles to):
 *   x bf16 [B,H,L,128] (strides in elements), mean bf16 [B*H,128] or NULL (x - mean rounded to bf16 first, as
 *   per_block_int8 forms k - km in the input dtype, :53-54), mul: the factor applied before quantising
 *   (sm_scale * log2(e) for queries, 1 for keys);
 *   x_i8 int8 [B,H,L,128] (strides in elements, multiples of 8); scale fp32 [B,H,ceil(L/blk)]. */
int hq_per_block_int8(const void* x, int64_t x_sb, int64_t x_sh, int64_t x_sn, int B, int H, int L, int blk,
                      float mul, const void* mean, void* x_i8, int64_t o_sb, int64_t o_sh, int64_t o_sn,
                      float* scale, void* stream);

/* Step 2: vertical-line bookkeeping.  Replaces reorder_kv_for_vertical
 * (src/ops/sage_unified.py:499-547) without expanding K/V to query heads:
 *   vidx_asc int32 [B,H_Q,T] ascending distinct positions
 *   vert_k bf16 [B,H_Q,Tpad,128] gathered rows of k_bf (Tpad = T rounded up to 64, tail rows zero),
 *   vert_vt bf16 [B,H_Q,128,Tpad] the gathered rows of v, transposed;
 *   k_bias fp32 [B,H_Q,Npad]: the additive term of the INT8 score conversion for every key of every
 *   query head, -12582912 * k_scale[key], or -inf where the key is a vertical line of the head (the
 *   kernel serves those from vert_k);
 *   nv_valid int32 [B,H_Q,ceil(N/128)] = number of vertical lines below the window start of a query block.
 * Call it for every prefill: with T == 0 it fills k_bias only and the vertical pointers may be null.
 */
int hq_prefill_vertical_prepare(const int32_t* vidx_asc, int B, int H_Q, int H_KV, int N, int window, int T,
                                const void* k_bf, const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
                                const float* k_scale, void* vert_k, void* vert_vt, float* k_bias, int32_t* nv_valid,
                                void* stream);

/* V transposed for the K-major operands of the tensor-memory kernel (the job of the reference's
 * TransposePadPermuteKernel, vendor/sageattention/csrc/fused/fused.cu:264-315, without the fragment
 * permutation): v bf16 [B,H_KV,N,128] -> v_t bf16 [B,H_KV,128,Npad], columns >= N zero. */
int hq_prefill_transpose_v(const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn, int B, int H_KV, int N,
                           void* v_t, void* stream);

/* Step 3: the attention kernel (tcgen05.mma kind::i8 / kind::f16 with tensor-memory accumulators,
 * TMA tensor-map tile loads).  Replaces _attn_fwd_vertical_v2 / _attn_fwd_unified
 * (src/ops/sage_unified.py:398-496, 112-231): causal, GQA-native, INT8 QK^T for the
 * non-vertical prefix, BF16 QK^T for vertical lines and for the window; one online softmax.
 * window == N gives plain BF16 causal attention (full_attention_fp16_triton,
 * src/ops/v_sageattention.py:14-51); T == 0 gives sage_unified_attention.
 */
typedef struct hq_prefill_args {
  int32_t struct_bytes;
  int32_t B, H_Q, H_KV, N, head_dim;
  int32_t window;              /* W; keys within W-1 of a query block's start (64-aligned) are BF16 */
  int32_t T;                   /* vertical lines per query head (0 = none) */
  int32_t out_dtype;
  float   sm_scale;            /* same value as given to hq_prefill_quant */
  const void* q_i8; const void* q_bf; const float* q_scale;     /* from hq_prefill_quant */
  const void* k_i8; const void* k_bf; const float* k_scale;
  const float* k_bias;         /* fp32 [B,H_Q,Npad] from hq_prefill_vertical_prepare (always) */
  const void* v_t;             /* bf16 [B,H_KV,128,Npad] from hq_prefill_transpose_v */
  const void* vert_k;          /* from hq_prefill_vertical_prepare (T > 0) */
  const void* vert_vt;
  const int32_t* nv_valid;
  void* out; int64_t o_sb, o_sh, o_sn;         /* [B,H_Q,N,128], strides in elements (multiples of 8) */
  int32_t* status;             /* device word, zeroed by the caller; bit 1 = a bounded wait expired */
  /* FP8 P V (pv_fp8 != 0): P~ = 2^(s - m + 8.807) rounded to e4m3 against the exact running maximum,
   * V^T as e4m3 with one scale per channel (hq_prefill_quant_v_fp8), the product on tcgen05 kind::f8f6f4, the row sum
   * in fp32 before the cast - the arithmetic of the reference's sage_fp8_attention
   * (src/ops/sage_fp8_attention.py:15-45 -> vendor/sageattention/core_sm90.py:116-165,
   *  csrc/qattn/attn_utils.cuh:30,354-458, csrc/qattn/qk_int_sv_f8_cuda_sm90.cu:259-364,490-515). v_t is not used then. */
  const void* v_t8;            /* e4m3 [B,H_KV,128,Npad] */
  const float* v_scale8;       /* fp32 [B,H_KV,128] */
  int32_t pv_fp8; int32_t reserved0;
  const void* vert_vt8;        /* T > 0: e4m3 [B,H_Q,128,Tpad] from hq_prefill_vertical_gather_v_fp8 (vert_vt is not used then) */
} hq_prefill_args;
int hq_prefill_hybrid(const hq_prefill_args* args, void* stream);

/* V for the FP8 P V product: the reference's per_channel_fp8 with smooth_v off
 * (vendor/sageattention/quant.py:134-166; MeanScaleKernel, csrc/fused/fused.cu:318-429):
 *   v bf16 [B,H_KV,N,128] -> v_t8 e4m3 [B,H_KV,128,Npad] (transposed, columns >= N zero), v_scale fp32 [B,H_KV,128] =
 *   max_n |v| / 448.  amax_scratch: B * H_KV * 128 * 4 bytes of device scratch (cleared here, in stream). */
int hq_prefill_quant_v_fp8(const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn, int B, int H_KV, int N,
                           void* v_t8, float* v_scale, void* amax_scratch, void* stream);
/* The vertical-line rows of V for FP8 P V: gathered per query head (vidx_asc as for hq_prefill_vertical_prepare),
 * quantised with the kv head's channel scales (v_scale from hq_prefill_quant_v_fp8), transposed:
 * vert_vt8 e4m3 [B,H_Q,128,Tpad], columns >= T zero. */
int hq_prefill_vertical_gather_v_fp8(const int32_t* vidx_asc, int B, int H_Q, int H_KV, int N, int T, const void* v,
                                     int64_t v_sb, int64_t v_sh, int64_t v_sn, const float* v_scale, void* vert_vt8,
                                     void* stream);

/* --------------------------------------------------------------------------
 * Tensor-pipe peak probe (no counterpart in the reference): runs tcgen05.mma products of `kind` (0 = kind::i8,
 * 1 = kind::f8f6f4 on e4m3, 2 = kind::f16 on bf16) back to back on every SM, operands resident in shared memory,
 * accumulators in tensor memory.  One launch does sms * steps products of 128 x 256 x K (K = 128 for the 8-bit kinds,
 * 64 for bf16); the caller times it.  The benchmark uses the result as the measured denominator of the prefill
 * kernel's tensor-pipe fraction.  status: device word, zeroed by the caller; bit 2 = a bounded wait expired. */
int hq_tc_peak(int kind, int steps, int* status, int* sms_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* HYQUANT_B200_H_ */

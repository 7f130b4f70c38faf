/* dtb200_attn.h — C ABI of the B200 joint (text + image/video token) attention forward.
 *
 * Every entry point is a plain `extern "C"` function taking raw device pointers and sizes, so it can
 * be bound from a torch custom op (ctypes / cpp extension), from a `jax.ffi` custom call handler or
 * from any other host language.  No entry point allocates or frees device memory except where stated,
 * none synchronises the stream, and all work is enqueued on the `stream` argument.
 *
 * Tensors are bf16 laid out [B, H, S, D] with arbitrary element strides for B, H and S and a
 * contiguous last dimension (D == 128).  Byte strides must be multiples of 16 and base pointers
 * 16-byte aligned (TMA tensor-map rules).
 *
 * Each declaration cites the function of the reference project (shungcp/diffusers-tpu) that it
 * replaces, by path within that project.
 */
#ifndef DTB200_ATTN_H_
#define DTB200_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Host-side status codes returned by every entry point (0 = success). */
enum dtb_status {
  DTB_OK = 0,
  DTB_ERR_NULL = 1,      /* a required pointer is NULL                                   */
  DTB_ERR_DTYPE = 2,     /* unsupported element type                                     */
  DTB_ERR_SHAPE = 3,     /* unsupported shape (head_dim != 128, H % Hkv != 0, sizes <= 0) */
  DTB_ERR_ALIGN = 4,     /* pointer or stride breaks the 16-byte rule                    */
  DTB_ERR_ARCH = 5,      /* the current device is not sm_100                             */
  DTB_ERR_WORKSPACE = 6, /* workspace missing or too small                               */
  DTB_ERR_LAUNCH = 7,    /* CUDA reported an error when encoding maps or launching       */
  DTB_ERR_TIMEOUT = 8,   /* a bounded device wait ran out (reported via the status word) */
  DTB_ERR_UNSUPPORTED = 9
};

/* Flags for dtb_attn_params.flags */
#define DTB_FLAG_ZERO_PADDED_ROWS 0x1u /* write exact zeros to query rows >= kv_len[b]            */
#define DTB_FLAG_BOUNDED_LOGITS 0x2u   /* per-head constant softmax offset from `mk` (fixed-m)    */
#define DTB_FLAG_QK_FP8 0x8u           /* q and k are E4M3 bytes (strides in bytes); dtb_attn_fwd and dtb_attn_fwd_residual */

/* One attention call.  All pointers are device pointers unless noted. */
typedef struct dtb_attn_params {
  const void* q; /* bf16 [B, Hq,  Sq,  D] */
  const void* k; /* bf16 [B, Hkv, Skv, D] */
  const void* v; /* bf16 [B, Hkv, Skv, D] */
  void* o;       /* bf16 [B, Hq,  Sq,  D] (ignored by the residual entry point) */
  int32_t B, Hq, Hkv, Sq, Skv, D;
  /* element strides of the batch, head and sequence axes (last axis is contiguous) */
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  int64_t v_stride_b, v_stride_h, v_stride_s;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  const int32_t* kv_len; /* [B] valid key count per batch element (keys >= kv_len are masked); NULL = all */
  const float* mk;       /* [2, Hq] bounded-logit operand: row 0 = integral bound m, row 1 = eligibility; NULL = online softmax */
  float scale;           /* softmax scale; <= 0 means 1/sqrt(D) */
  uint32_t flags;        /* DTB_FLAG_* */
  int32_t num_splits;    /* 0 = automatic: one CTA per query block, the last wave of the launch cut into equal runs of key
                            tiles when its query blocks would leave SMs idle (uses workspace when given); 1 = no splitting;
                            n > 1 = every query block's keys split n ways (needs workspace) */
  int32_t* status;       /* optional [4] int32 device status words written when a bounded wait runs out; must be zeroed by the caller */
} dtb_attn_params;

/* Running state of a residual (ring) accumulation, in the reference's units: `m` and `lse` are in
 * log2 units of the scaled logits.  o_acc f32 [B, Hq, Sq, D] contiguous; m, l f32 [B, Hq, Sq]. */
typedef struct dtb_attn_residual {
  float* o_acc;
  float* m;
  float* l;
  int32_t kv_offset; /* global index of this shard's first key (kv_len is compared against global indices) */
  int32_t q_offset;  /* global index of the first query row of this call (used to zero padded rows) */
  int32_t init;      /* non-zero: start from the empty state instead of reading o_acc / m / l */
} dtb_attn_residual;

/* Destination of a head-parallel call whose output is sequence-sharded over `n_peers` GPUs: query row s of
 * local head h is written to out_ptrs[s / shard_rows], a contiguous bf16 [B, total_heads, shard_rows, D]
 * buffer (possibly another GPU's memory, mapped into this process), at head head_offset + h. */
typedef struct dtb_attn_scatter {
  void* out_ptrs[8];
  int32_t n_peers;
  int32_t shard_rows;
  int32_t head_offset;
  int32_t total_heads;
  void* workspace;        /* optional scratch of dtb_attn_workspace_bytes(p) bytes (device, 16-byte aligned): lets an */
  size_t workspace_bytes; /* automatic call (p->num_splits == 0) balance its last wave; NULL / 0 = plain launch      */
} dtb_attn_scatter;

/* Sequence shards -> head shards for up to three tensors at once (q, k, v): this rank's bf16
 * [B, H, S_local, D] tensors (element strides given) are written straight into every rank's contiguous
 * [B, H / n_peers, n_peers * S_local, D] buffers dst[tensor][peer], rows [rank * S_local, (rank+1) * S_local). */
typedef struct dtb_scatter_heads_params {
  const void* src[3];
  int64_t stride_b[3], stride_h[3], stride_s[3];
  void* dst[3][8];
  int32_t n_tensors, n_peers, rank;
  int32_t B, H, S_local, D;
} dtb_scatter_heads_params;

/* The step in front of the attention call in every DiT block: per-head RMSNorm of q and k, rotary embedding,
 * zeroing of padded rows and the [B, S, H, D] -> [B, H, S, D] layout change, one read and one write per tensor.
 * Strides are element strides of the (batch, sequence, head) axes of the inputs; outputs are contiguous [B, H, S, D]. */
typedef struct dtb_prepass_params {
  const void* q_in; const void* k_in; const void* v_in;   /* bf16 [B, S, H, D]; v_in may be NULL (then v_out too) */
  int64_t q_strides[3], k_strides[3], v_strides[3];
  void* q_out; void* k_out; void* v_out;                   /* bf16 [B, H, S, D] contiguous */
  const float* q_weight; const float* k_weight;            /* RMSNorm scales [D], NULL = ones */
  const float* cos; const float* sin;                      /* [S, rotary] f32 (rotary % 16 == 0), both NULL = none */
  const int32_t* kv_len;                                   /* [B] or NULL: rows >= kv_len[b] are written as zeros */
  float* norms;                                            /* scratch [2 * H] f32, required with mk_out */
  float* mk_out;                                           /* [2, H] bounded-logit operand of the outputs, or NULL */
  float eps, scale, gate;                                  /* scale <= 0: 1/sqrt(D); gate <= 0: 213 */
  int32_t B, S, H, D, rotary;
} dtb_prepass_params;

/* Block-sparsity table at the kernel's own granularity (256 query rows x 128 keys): query block qb of a head in
 * class c visits key tiles kv_table[(c * q_blocks + qb) * width + i] for i < kv_count[c * q_blocks + qb], in ascending
 * order.  All arrays are int32 on the device; head_class ([Hq]) may be NULL when n_classes == 1. */
typedef struct dtb_block_table {
  const int32_t* kv_table;
  const int32_t* kv_count;
  const int32_t* head_class;
  int32_t n_classes, q_blocks, width;
} dtb_block_table;

/* Library version and a human-readable string for a status code. */
int dtb_version(void);
const char* dtb_status_string(int status);
/* Text naming the CUDA error behind the calling thread's most recent DTB_ERR_LAUNCH ("" if none). */
const char* dtb_last_error_detail(void);

/* 1 when the call described by `p` is supported on the current device, else 0 and *why (if not NULL)
 * receives the status that dtb_attn_fwd would return. */
int dtb_attn_supported(const dtb_attn_params* p, int* why);

/* Scratch bytes dtb_attn_fwd can use for `p` (0 when no form of key splitting applies).  In automatic mode a
 * missing or smaller workspace is not an error: the call runs unsplit. */
size_t dtb_attn_workspace_bytes(const dtb_attn_params* p);

/* How dtb_attn_fwd would launch the call described by `p` in automatic mode on a GPU with `sms` SMs (0: the current
 * device's count, or a B200's 148 where there is no device): the first whole_units (batch, head, 256-row query block)
 * units - numbered query block fastest, then head, then batch - are swept whole, one CTA each; when n_pieces > 0 the
 * remaining tail_units units are swept in n_pieces pieces, piece i being key tiles [tile_begin[i], tile_end[i]) of unit
 * unit[i], listed longest first; a piece with slot[i] >= 0 leaves its state in that scratch slot for the merge, and
 * the slots of one unit are consecutive in key order.  n_pieces == 0 means the plain launch.  The plan depends only
 * on the static shape; it plays the role of the reference's per-shape tile resolution, which logs one line per
 * resolved shape (diffusers_tpu/kernels/mesh_attention.py:199-216, diffusers_tpu/kernels/block_sizes.py:442-577). */
#define DTB_MAX_PIECES 304
typedef struct dtb_launch_plan {
  int32_t units, key_tiles, whole_units, tail_units, n_pieces, n_slots;
  int32_t unit[DTB_MAX_PIECES];
  uint16_t tile_begin[DTB_MAX_PIECES];
  uint16_t tile_end[DTB_MAX_PIECES];
  int16_t slot[DTB_MAX_PIECES];
} dtb_launch_plan;

int dtb_attn_launch_plan(const dtb_attn_params* p, int32_t sms, dtb_launch_plan* out);

/* Normalised joint attention forward: o = softmax(scale * q k^T + key_mask) v.
 * Replaces diffusers_tpu/kernels/splash.py:566-650 `attention(...)` (and the per-sample loop around it
 * in diffusers_tpu/models/moss_image/jax_dit.py:199-203: kv_len is per batch element here). */
int dtb_attn_fwd(const dtb_attn_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* dtb_attn_fwd for a head shard [B, H/P, S, D] whose output goes back to sequence shards: the epilogue stores each
 * output row directly into the buffer of the rank that owns it (peer stores over NVLink), which fuses the
 * heads -> sequence all-to-all of diffusers_tpu/backends/qwen21_core_tt.py:116-121 (and the output sharding
 * constraint of diffusers_tpu/kernels/mesh_attention.py:118-120, 145) into the kernel.  p->o is ignored.
 * The caller synchronises the ranks before the buffers are read. */
int dtb_attn_fwd_scatter(const dtb_attn_params* p, const dtb_attn_scatter* sc, void* stream);

/* The sequence -> heads exchange of q, k and v as one kernel of peer stores; replaces the first all-to-all of
 * diffusers_tpu/backends/qwen21_core_tt.py:108-115 (`_a2a` to heads).  The caller synchronises the ranks before
 * the destination buffers are read. */
int dtb_scatter_heads(const dtb_scatter_heads_params* sp, void* stream);

/* Block-sparse forward: the same arithmetic, but each query block only visits the key tiles its table row lists, so
 * skipped tiles cost neither loads nor MMAs; a full table gives the dense result bit for bit.  kv_len still applies.
 * Replaces diffusers_tpu/kernels/sparse_splash.py:568-649 `attention(..., kv_table= | kv_table_dyn=)`. */
int dtb_attn_fwd_sparse(const dtb_attn_params* p, const dtb_block_table* tb, void* stream);

/* Residual forward over one KV shard: folds this shard into the running (o_acc, m, l) state.
 * Replaces diffusers_tpu/kernels/splash.py:665-742 `residual_attention(...)` together with the
 * LSE-space merge its docstring prescribes (splash.py:657-662, 688-691). */
int dtb_attn_fwd_residual(const dtb_attn_params* p, const dtb_attn_residual* r, void* stream);

/* Normalises a finished running state: o = o_acc / l, cast to bf16 (rows with l == 0 give zeros).
 * Replaces the epilogue of diffusers_tpu/kernels/splash.py:367-375 applied after a ring. */
int dtb_attn_finalize(const dtb_attn_params* p, const dtb_attn_residual* r, void* stream);

/* Bounded-logit operand: mk[0,h] = ceil(max_row|q*scale*log2e| * max_row|k|), mk[1,h] = (bound <= gate).
 * `norms` is a scratch of Hq + Hkv floats (device).  Replaces
 * diffusers_tpu/kernels/fixed_m_bound.py:57-118 `max_row_norm_per_head` + `fixed_m_operands`. */
int dtb_fixed_m_operands(const dtb_attn_params* p, float gate, float* norms, float* mk_out, void* stream);

/* Bytes of scratch built into the library image for dtb_attn_fwd_static_scratch (32 MiB per device). */
#define DTB_STATIC_SCRATCH_BYTES (32u << 20)

/* Same result as dtb_attn_fwd, for callers that have nowhere to get scratch memory from: a handler
 * running inside another runtime's execution callback (an XLA FFI custom call, a graph node, a plugin
 * of a serving engine) or a foreign-language binding that only ever sees the input and output buffers
 * it was given.  Such callers must not call cudaMalloc themselves and cannot pass a workspace, so the
 * split-KV partials are kept in a fixed DTB_STATIC_SCRATCH_BYTES array that is part of the library and
 * stays resident on every device that loads it.  The call allocates nothing.  Calls whose partials
 * would not fit return DTB_ERR_WORKSPACE (dtb_last_error_detail() gives both sizes); p->num_splits
 * is honoured as in dtb_attn_fwd.  The first call on each device looks up the array's device address;
 * make that first call outside any stream capture.  The address is kept per device ordinal for the life of
 * the process and is not looked up again after a cudaDeviceReset: do not reset a device this entry point has
 * been used on.  All calls on a device share the array: calls that may overlap on the GPU race and must be
 * ordered by the caller.
 * This entry point has no counterpart in the reference project. */
int dtb_attn_fwd_static_scratch(const dtb_attn_params* p, void* stream);

/* Fused q/k RMSNorm + rotary embedding + pad zeroing + layout change, optionally producing the bounded-logit
 * operand of its outputs for free.  Replaces the per-block sequence diffusers_tpu/models/minimax_h3/jax_dit.py:362-388
 * (norm_q / norm_k :191-195, apply_rope :251-262, pad zeroing :372-381, swapaxes :388), its torch twin
 * diffusers_tpu/backends/ours_splash_tt.py:189-213, and the operand pass diffusers_tpu/kernels/fixed_m_bound.py:57-118. */
int dtb_qk_prepass(const dtb_prepass_params* pp, void* stream);

/* Row chunks the key-smoothing pass sums separately (fixes the size of its scratch). */
#define DTB_SMOOTH_K_CHUNKS 64

/* k-smoothing of a bf16 [B, H, S, 128] key tensor: out = k - mean over the valid rows of k (f32 sum, mean rounded
 * to bf16 before the subtraction), rows >= kv_len[b] written as zeros.  `out` may be `k` itself (in place).
 * `scratch` holds dtb_smooth_k_scratch_bytes(B, H) bytes of device memory; `k_norm_max` (optional, [H] f32) receives
 * the largest output row norm per head, the key half of the bounded-logit operand. */
typedef struct dtb_smooth_k_params {
  const void* k;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  void* out;
  int64_t out_stride_b, out_stride_h, out_stride_s;
  const int32_t* kv_len; /* [B] or NULL */
  void* scratch;
  size_t scratch_bytes;
  float* k_norm_max;     /* [H] or NULL */
  int32_t B, H, S, D;
} dtb_smooth_k_params;

size_t dtb_smooth_k_scratch_bytes(int32_t B, int32_t H);

/* The caller-side preconditioning the bounded-logit softmax presumes: zero-mean key columns make every query row's
 * mean logit zero, hence its largest logit non-negative.  Replaces `k - mean(k, axis=2)` of
 * diffusers_tpu/kernels/mesh_attention.py:234-237 and diffusers_tpu/backends/ours_splash_tt.py:136-137, and the
 * padded form of diffusers_tpu/models/minimax_h3/jax_server.py:276-281. */
int dtb_smooth_k(const dtb_smooth_k_params* sp, void* stream);

/* mk[0,h] = ceil(q_norms[h] * k_norms[h / (Hq/Hkv)]), mk[1,h] = (that product <= gate), from per-head row-norm
 * maxima already on the device (gate <= 0: 213).  Replaces diffusers_tpu/kernels/fixed_m_bound.py:98-118
 * `fixed_m_operands` for norms collected by dtb_qk_prepass and dtb_smooth_k. */
int dtb_fixed_m_from_norms(const float* q_norms, const float* k_norms, int32_t Hq, int32_t Hkv, float gate,
                           float* mk_out, void* stream);

/* Output projection behind head-sharded attention output: y[b, s, :] (+)= sum over the local heads h of
 * o[b, h, s, :] . w[h * 128 : (h + 1) * 128, :], bf16 operands, f32 accumulation.  o is the attention output in its
 * [B, H_local, S, 128] layout (element strides given), w the H_local * 128 rows of the projection weight that belong
 * to these heads ([K, N] row-major, row stride w_stride_k), N a multiple of 8.
 *   n_dest == 0: y is written as bf16 [B, S, N] (out, element strides out_stride_b / out_stride_s).
 *   n_dest  > 0: the reduce-scatter half of the all-reduce over head shards, fused into the kernel.  Row g = b * S + s
 *                of the flattened result belongs to destination g / rows_per_dest (a buffer that may live on another
 *                GPU), local row g % rows_per_dest.
 *                partials != 0: this rank's bf16 partial rows are stored into slot src_rank of the destination's
 *                  staging buffer, bf16 [n_src, rows_per_dest, N]; the owner sums the slots with dtb_sum_partials.
 *                partials == 0: the f32 partial sums are added (vector reductions, order not fixed) into the
 *                  destination's f32 [rows_per_dest, N] buffer, which must hold zeros (or what to add to) before.
 *                The caller synchronises the ranks around the call. */
typedef struct dtb_out_proj_params {
  const void* o;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  const void* w;
  int64_t w_stride_k;
  void* out;
  int64_t out_stride_b, out_stride_s;
  void* red_dst[8];
  int32_t n_dest, rows_per_dest;
  int32_t partials, src_rank;
  int32_t B, H_local, S, D, N;
  int32_t* status;       /* optional [4] int32 device status words, as in dtb_attn_params */
} dtb_out_proj_params;

/* Replaces the `to_out` linear that follows keep-heads attention and the all-reduce XLA inserts behind it
 * (diffusers_tpu/models/minimax_h3/jax_image_pipeline.py:574-593). */
int dtb_out_proj(const dtb_out_proj_params* pp, void* stream);

/* out[rows, N] (bf16) = sum over n_src slots of staged[n_src, rows, N] (bf16, f32 accumulation in slot order): the
 * owner's half of the fused reduce-scatter above.  No counterpart in the reference (XLA's all-reduce does it). */
int dtb_sum_partials(const void* staged, int32_t n_src, int64_t rows, int32_t N, void* out, void* stream);

/* Saturating E4M3 cast of a bf16 [B, H, S, 128] tensor, x * mult clamped to +-448, written contiguously; feeds the
 * DTB_FLAG_QK_FP8 variant of dtb_attn_fwd.  Replaces diffusers_tpu/kernels/fp8_cast.py:28-39 `quantize_saturating` as
 * applied to q and k in diffusers_tpu/kernels/splash.py:420-424. */
int dtb_quantize_e4m3(const void* x, int64_t stride_b, int64_t stride_h, int64_t stride_s, int32_t B, int32_t H, int32_t S,
                      int32_t D, float mult, void* out, void* stream);

/* Hardware self-tests of the descriptor encodings the kernels rely on (one 128x128x128 tile each).
 * They write f32 [128,128] results for the host to compare; no reference counterpart. */
int dtb_selftest_tmem_roundtrip(const float* in, float* out, int32_t* status, void* stream);
int dtb_selftest_qk(const void* q, const void* k, float* s_out, int32_t* status, void* stream);
int dtb_selftest_pv(const void* p, const void* v, float* o_out, int32_t* status, void* stream);
/* Bounded-wait probe: one warp waits on a barrier that is never signalled; after budget_ns (<= 2 s) the wait gives up,
 * writes {1 (timeout), site, CTA, parity} to `status` (4 x int32, zeroed by the caller) and 2 to *returned. */
int dtb_selftest_wait_timeout(unsigned long long budget_ns, int site, int32_t* status, int32_t* returned, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DTB200_ATTN_H_ */

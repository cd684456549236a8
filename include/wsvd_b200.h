/*
 * wsvd_b200 — C ABI of the B200 (sm_100a) latent flash-decoding library.
 *
 * Every entry point takes plain pointers and sizes.  The library never allocates or
 * frees device memory and never synchronises the device: all work is enqueued on the
 * stream the caller passes (a cudaStream_t cast to void*; NULL = the legacy default
 * stream).  All functions return a WsvdStatus (0 = success) and never throw or abort.
 *
 * Tensor conventions follow the reference (WSVD, efficiency/kernel/):
 *   q            [B, Hq, D]          f16, innermost stride 1
 *   latent_k/v   [T, Hkv, Rk|Rv]     int8 (with f16 scales [T, Hkv]) or f16
 *   wk           [Rk, Hkv*D]         f16, or int8 with a per-column f16 scale [Hkv*D]
 *   req_to_token [n_req, max_len]    int32 page table: logical position -> token slot
 *   b_req_idx, b_seq_len [B]         int32
 * Strides are in ELEMENTS of the tensor's own dtype.  The innermost dimension of every
 * tensor must be contiguous.  A head-major cache [B, H, S, R] is expressed with
 * stride_t = R, stride_h = S*R and a page table req_to_token[b][s] = b*H*S + s.
 */
#ifndef WSVD_B200_H_
#define WSVD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WSVD_ABI_VERSION 1

typedef enum WsvdStatus {
  WSVD_OK = 0,
  WSVD_ERR_NULL_POINTER = 1,     /* a required pointer is NULL */
  WSVD_ERR_BAD_SHAPE = 2,        /* head_dim/rank/head counts outside the supported set */
  WSVD_ERR_BAD_DTYPE = 3,        /* unknown dtype code, or scales missing for int8 */
  WSVD_ERR_BAD_STRIDE = 4,       /* stride/alignment precondition violated */
  WSVD_ERR_WORKSPACE_TOO_SMALL = 5,
  WSVD_ERR_CUDA = 6,             /* a CUDA runtime call failed; see wsvd_last_cuda_error() */
  WSVD_ERR_UNSUPPORTED = 7,      /* valid request that this build has no kernel for */
  WSVD_ERR_TOO_LARGE = 8         /* size beyond a documented fixed limit */
} WsvdStatus;

typedef enum WsvdDtype { WSVD_I8 = 0, WSVD_F16 = 1, WSVD_F32 = 2 /* quant-append input only */ } WsvdDtype;
typedef enum WsvdRopeLayout { WSVD_ROPE_HALF = 0, WSVD_ROPE_INTERLEAVED = 1 } WsvdRopeLayout;

/* Which stage-1 kernel to run.  AUTO picks the tcgen05 kernel when the shape allows. */
typedef enum WsvdKernel {
  WSVD_KERNEL_AUTO = 0,     /* tcgen05 kernel if the problem fits it, else warp-MMA, else generic */
  WSVD_KERNEL_GENERIC = 1,  /* CUDA-core kernel, any shape */
  WSVD_KERNEL_TC = 2,       /* tcgen05 + TMA kernel or WSVD_ERR_UNSUPPORTED */
  WSVD_KERNEL_MMA = 3       /* warp-MMA kernel (f16 or int8 latents, head_dim 16..128, even ranks) or WSVD_ERR_UNSUPPORTED */
} WsvdKernel;

/*
 * Arguments of the latent decode-attention op.  Mirrors the tensors that
 * token_decode_attention_flash_int8_latent_per_head_decoding_rope and its f16 sibling
 * pass to their kernels (efficiency/kernel/flash_decoding.py:3-55, :57-95;
 * flash_int8_latent_per_head_decoding_rope_stage1.py:33-56,250-280).
 */
typedef struct WsvdLatentDecodeParams {
  const void* q;            int64_t q_stride_b, q_stride_h;
  const void* latent_k;     int64_t k_stride_t, k_stride_h;
  const void* k_scale;      int64_t ks_stride_t, ks_stride_h;   /* NULL for f16 latents */
  const void* latent_v;     int64_t v_stride_t, v_stride_h;
  const void* v_scale;      int64_t vs_stride_t, vs_stride_h;   /* NULL for f16 latents */
  const void* wk;           int64_t wk_stride_r;                /* [Rk, Hkv*D], column stride 1 */
  const void* wk_scale;                                         /* f16 [Hkv*D], NULL when wk is f16 */
  const void* wv;           int64_t wv_stride_r;                /* optional f16 [Rv, Hkv*D]: out = O_lat . wv */
  const int32_t* req_to_token; int64_t rtt_stride;              /* row stride; column stride 1 */
  const int32_t* b_req_idx;
  const int32_t* b_seq_len;
  const int32_t* pos_offset;  /* optional [B]: RoPE position of token s is pos_offset[b] + s */
  void* out;                int64_t out_stride_b, out_stride_h; /* f16 [B,Hq,Rv], or [B,Hq,D] when wv != NULL */
  int32_t batch, n_q_heads, n_kv_heads, head_dim, rank_k, rank_v;
  int32_t max_len;          /* >= every b_seq_len[b]; sizes the grid and the workspace */
  int32_t latent_dtype;     /* WsvdDtype of latent_k/latent_v */
  int32_t wk_dtype;         /* WsvdDtype of wk */
  int32_t rope_layout;      /* WsvdRopeLayout; the reference kernels use HALF */
  int32_t split_len;        /* tokens per split-KV partial; 0 = library default */
  int32_t kernel;           /* WsvdKernel */
  float theta;              /* RoPE base, 10000 in the reference (stage1.py:269) */
  float sm_scale;           /* 0 = 1/sqrt(head_dim) (stage1.py:244) */
  const void* rope_table;   /* optional: table made by wsvd_rope_table_init for the same theta/head_dim */
  int32_t rope_table_rows;  /* positions it covers (>= max_len rounded up to 128) */
  int64_t n_token_slots;    /* T, the extent of latent_k/v along the token-slot axis; 0 = unknown (the
                               tensor-core kernel then gathers rows with cp.async instead of TMA) */
} WsvdLatentDecodeParams;

/* Version of this header the library was built from. */
int wsvd_abi_version(void);

/* Static text for a status code. */
const char* wsvd_status_string(int status);

/* cudaError_t (as int) of the last failed CUDA call made by this library on the
 * calling thread, 0 if none. */
int wsvd_last_cuda_error(void);

/*
 * cos/sin position table used by the tensor-core kernel (the reference recomputes
 * cos/sin per tile with fast-math intrinsics, stage1.py:8-14,157-159).  It depends only on
 * theta, head_dim and the number of positions, so a caller can build it once and pass it in
 * WsvdLatentDecodeParams.rope_table; without it wsvd_latent_decode rebuilds it in the
 * workspace on every call.  `positions` is rounded up to a multiple of 128 by both calls.
 */
size_t wsvd_rope_table_bytes(int32_t positions, int32_t head_dim);
int wsvd_rope_table_init(void* table, size_t table_bytes, int32_t positions, int32_t head_dim, float theta,
                         void* stream);

/*
 * Device-side status of the kernels: 0, or the highest code recorded since the last reset:
 * 1-3 a bounded wait of the tensor-core kernel timed out (1 copy issuer, 2 MMA issuer,
 * 3 epilogue), 4 its shared-memory base was misaligned, 5 wsvd_latent_quant_append_i8 met
 * a position outside [0, max_len) and skipped that row, 6 the group barrier of
 * wsvd_latent_decode_gather gave up waiting for a peer.  SYNCHRONISES the device; meant
 * for tests and diagnostics, and for a serving loop to poll at a point where it synchronises
 * anyway.  wsvd_kernel_status_reset clears it.  A tensor-core work item whose wait timed out
 * writes NaN instead of its result, so the affected output rows are NaN, not plausible numbers.
 */
int wsvd_kernel_status(uint32_t* status);
int wsvd_kernel_status_reset(void);

/*
 * Fixed-length split plan: tokens per split and number of split slots per (b, h).  Replaces the
 * BLOCK_SEQ constant that the reference hard-codes on the host (flash_decoding.py:18,31-36)
 * while its kernel autotunes it.  It is what runs when p->split_len > 0 and on the generic
 * kernel.  With p->split_len == 0 and a problem the tensor-core kernel accepts (head_dim 128,
 * int8 latents, ranks multiples of 16 up to 64, 16-byte aligned rows), wsvd_latent_decode does
 * not use fixed-length splits at all: one kernel, one persistent CTA per SM, cuts the batch's
 * tiles of 128 positions into equal shares from the sequence lengths on the device (ragged
 * batches load every SM alike), and the CTA that completes a head's last partial merges the
 * partials, applies U_v and writes the output row, so that no merge kernel runs; the plan
 * returned here is then only what wsvd_latent_decode_stage1 would run.
 */
int wsvd_latent_decode_plan(const WsvdLatentDecodeParams* p, int32_t* split_len, int32_t* n_splits);

/* Bytes of scratch the op needs: the partial results and their log-sum-exp in f32 (the mid_o /
 * mid_o_logexpsum tensors of flash_decoding.py:31-36), the tile prefix sums and arrival counters
 * of the balanced mode, and the cos/sin position table when p->rope_table is NULL.  Device
 * independent.  Nothing in it has to be initialised by the caller. */
size_t wsvd_latent_decode_workspace_bytes(const WsvdLatentDecodeParams* p);

/*
 * The whole op: split-KV stage 1 then the merge, on `stream`.
 * Replaces token_decode_attention_flash_int8_latent_per_head_decoding_rope
 * (flash_decoding.py:3-55) and token_decode_attention_flash_latent_per_head_decoding_rope
 * (flash_decoding.py:57-95), selected by p->latent_dtype.
 */
int wsvd_latent_decode(const WsvdLatentDecodeParams* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The arithmetic of the balanced work distribution, exposed for tests and for hosts that want to
 * know where a CTA's share starts: `total` tiles in the order (sequence, head group, tile) are cut
 * into n_shares = min(CTAs, total) shares; share c is [wsvd_share_begin(c), wsvd_share_begin(c+1)),
 * and wsvd_share_owner inverts that for 0 <= tile < total.  Pure host functions, no CUDA call.
 */
int64_t wsvd_share_begin(int32_t c, int64_t total, int32_t n_shares);
int32_t wsvd_share_owner(int64_t tile, int64_t total, int32_t n_shares);

/*
 * wsvd_latent_decode without the merge: stage 1 with the work distribution the whole op uses,
 * the partials left in `workspace` in the library's own layout.  For timing the dominant kernel
 * alone; p->out is not written and may be NULL.
 */
int wsvd_latent_decode_partials(const WsvdLatentDecodeParams* p, void* workspace, size_t workspace_bytes,
                                void* stream);

/*
 * Stage 1 alone, writing normalised partials mid_o [B,Hq,n_splits,Rv] f32 (contiguous)
 * and lse [B,Hq,n_splits] f32 for splits of p->split_len tokens (must be > 0 here).
 * Replaces flash_int8_latent_per_head_decode_rope_stage1
 * (flash_int8_latent_per_head_decoding_rope_stage1.py:221-281) and
 * flash_latent_per_head_decode_rope_stage1 (flash_latent_per_head_decoding_rope_stage1.py:169-213).
 * p->out and p->wv are ignored.
 */
int wsvd_latent_decode_stage1(const WsvdLatentDecodeParams* p, float* mid_o, float* lse, int32_t n_splits, void* stream);

/*
 * Stage 2 alone: merge the first ceil(len_b/split_len) partials of every (b, h) by
 * their log-sum-exp weights; a sequence of length 0 yields zeros.
 * Replaces flash_decode_stage2 (flash_latent_per_head_decoding_stage2.py:52-69 and
 * flash_decoding_stage2.py:48-64).  `width` is Rv (or D for the dense op).
 * When wv != NULL (f16 [width, n_kv_heads*head_dim], row stride wv_stride_r) the merged
 * row is multiplied by the head's slice of wv and `out` is [B,Hq,head_dim].
 */
int wsvd_decode_stage2(const float* mid_o, const float* lse, const int32_t* b_seq_len,
                       void* out, int64_t out_stride_b, int64_t out_stride_h,
                       int32_t batch, int32_t n_q_heads, int32_t n_splits, int32_t width, int32_t split_len,
                       const void* wv, int64_t wv_stride_r, int32_t n_kv_heads, int32_t head_dim,
                       void* stream);

/*
 * Dense f16 flash-decoding baseline on full K/V caches [T, Hkv, D] (K stored rotated, no
 * RoPE in the kernel), same page-table interface and split-KV structure.
 * Replaces token_decode_attention_flash_decoding (flash_decoding.py:98-131;
 * flash_decoding_stage1.py:75-105, flash_decoding_stage2.py:48-64).  out: f16 [B,Hq,D].
 */
typedef struct WsvdDenseDecodeParams {
  const void* q;            int64_t q_stride_b, q_stride_h;
  const void* k;            int64_t k_stride_t, k_stride_h;     /* f16 [T, Hkv, D] */
  const void* v;            int64_t v_stride_t, v_stride_h;
  const int32_t* req_to_token; int64_t rtt_stride;
  const int32_t* b_req_idx;
  const int32_t* b_seq_len;
  void* out;                int64_t out_stride_b, out_stride_h;
  int32_t batch, n_q_heads, n_kv_heads, head_dim;
  int32_t max_len;
  int32_t split_len;        /* 0 = library default */
  float sm_scale;           /* 0 = 1/sqrt(head_dim) */
} WsvdDenseDecodeParams;
size_t wsvd_dense_decode_workspace_bytes(const WsvdDenseDecodeParams* p);
int wsvd_dense_decode_f16(const WsvdDenseDecodeParams* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Decode-step producer of the latent cache: quantise the new token's K and V latents
 * x_k [B, Hkv, Rk], x_v [B, Hkv, Rv] (f16 or f32, innermost stride 1) per (sequence, head)
 * to int8 with an f16 scale, and store them at token slot
 * req_to_token[b_req_idx[b]][b_seq_len[b]], i.e. b_seq_len holds the lengths BEFORE the
 * append and the caller increments it afterwards.  Quantiser: scale = max|x| / 127 (1 for
 * an all-zero row) stored as f16, q = clamp(round_half_even(x / f16(scale)), -128, 127)
 * (fake_quant/quant_utils.py:30-33,175-184).  The reference has no such kernel: its layer
 * wrapper computes the new latents and drops them (efficiency/layer_utils.py:319-321) and
 * its test script fills the caches with torch ops (efficiency/test_timing_layer.py:267-275).
 * A sequence whose position is outside [0, max_len) is skipped and status 5 is recorded
 * (wsvd_kernel_status).  rank_k, rank_v <= 128.
 */
typedef struct WsvdQuantAppendParams {
  const void* x_k;          int64_t xk_stride_b, xk_stride_h;
  const void* x_v;          int64_t xv_stride_b, xv_stride_h;
  void* latent_k;           int64_t k_stride_t, k_stride_h;     /* int8 [T, Hkv, Rk] */
  void* k_scale;            int64_t ks_stride_t, ks_stride_h;   /* f16  [T, Hkv] */
  void* latent_v;           int64_t v_stride_t, v_stride_h;
  void* v_scale;            int64_t vs_stride_t, vs_stride_h;
  const int32_t* req_to_token; int64_t rtt_stride;
  const int32_t* b_req_idx;
  const int32_t* b_seq_len;
  int32_t batch, n_kv_heads, rank_k, rank_v;
  int32_t max_len;          /* columns of req_to_token */
  int32_t x_dtype;          /* WSVD_F16 or WSVD_F32 */
} WsvdQuantAppendParams;
int wsvd_latent_quant_append_i8(const WsvdQuantAppendParams* p, void* stream);

/*
 * Element-wise pieces of the decode step around the attention op, one kernel each (in the
 * reference's accuracy pipeline they are chains of small torch ops: LlamaRMSNorm,
 * apply_rotary_pos_emb and the MLP's act_fn * up, fake_quant/svd_utils.py:1628-1674).  f16 in
 * and out, fp32 arithmetic; strides in elements, so that the inputs may be column slices of one
 * wider GEMM output (q | k | v, or up | gate).
 *  - wsvd_rms_norm_f16: y[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps), no weight vector;
 *    contiguous rows.
 *  - wsvd_add_rms_norm_f16: x_out = x + delta (rounded to f16), y = RMSNorm(x_out): the residual
 *    update and the next block's normalisation in one pass; x_out may alias x.
 *  - wsvd_rope_half_f16: in place on q [batch, heads, head_dim] with q_stride_b elements between
 *    sequences (heads contiguous inside a sequence): the pairs (i, i + head_dim/2) are rotated by
 *    pos[b] * inv_freq[i] (inv_freq: head_dim/2 floats on the device).
 *  - wsvd_silu_mul_f16: out[r,c] = up[r,c] * silu(gate[r,c]), silu rounded to f16 before the
 *    product; up and gate [rows, cols] with leading dimensions up_ld, gate_ld; out contiguous.
 */
int wsvd_rms_norm_f16(const void* x, void* y, int32_t rows, int32_t cols, float eps, void* stream);
int wsvd_add_rms_norm_f16(const void* x, const void* delta, void* x_out, void* y, int32_t rows, int32_t cols, float eps,
                          void* stream);
int wsvd_rope_half_f16(void* q, int64_t q_stride_b, const int32_t* pos, const float* inv_freq, int32_t batch,
                       int32_t heads, int32_t head_dim, void* stream);
int wsvd_silu_mul_f16(const void* up, int64_t up_ld, const void* gate, int64_t gate_ld, void* out, int32_t rows,
                      int32_t cols, void* stream);

/*
 * Head-sharded multi-GPU decode with the all-gather fused into the op's own kernels.
 *
 * The op shards by attention head with no exchange between heads
 * (flash_int8_latent_per_head_decoding_rope_stage1.py:60, program_id(1) = head); the one
 * exchange of the path is the all-gather of the [B, H/g, D] outputs.  The reference is
 * single-GPU and has no counterpart.  Here the kernel that finishes an output row (the decode
 * kernel itself when it balances the work over persistent CTAs, else the merge kernel) stores
 * it straight into the gathered [B, H_total, D] f16 buffer of EVERY rank (plain 16-byte peer
 * stores, no multicast), and its last block runs the group barrier: a system-scope fence, one
 * flag store per peer and a bounded wait for the peers' flags.  When the call's kernels have
 * finished on every rank, every rank's buffer holds all heads.
 *
 *  - out[i], flags[i]: rank i's gathered buffer and flag array (WSVD_MAX_PEERS uint32,
 *    zero before the first call) as mapped in THIS process; entry `rank` is local memory.
 *    counter: one local uint32, zero before the first call.
 *  - epoch: the same value on all ranks for a given step, never 0, +1 per step.  When
 *    epoch_counter is set the kernel takes *epoch_counter + 1 instead and stores it back, so
 *    that nothing in the argument block changes from step to step and the call can sit in a
 *    captured CUDA graph; `epoch` is then ignored.
 *  - Every rank must make the call with the same batch, which must not be 0 (a rank that launched
 *    nothing would leave its peers waiting: WSVD_ERR_BAD_SHAPE); p->out is ignored; p->n_q_heads is
 *    the LOCAL head count and head_offset the first global head of the shard.
 *  - Reuse: a rank may overwrite a peer's buffer for step e+1 while that peer still reads
 *    step e.  Alternate between two buffers by epoch parity and consume a buffer on the
 *    stream that makes the next call: a peer passes the barrier of step e+1 only after this
 *    rank has enqueued step e+1 behind its readers of step e.
 *  - A wait that runs out (timeout_ms, 0 = 2000) records status 6 and the kernel returns;
 *    the context stays usable.
 */
#define WSVD_MAX_PEERS 8
typedef struct WsvdPeerSet {
  void* out[WSVD_MAX_PEERS];
  uint32_t* flags[WSVD_MAX_PEERS];
  uint32_t* counter;
  int32_t n_peers, rank;
  int32_t head_offset;
  uint32_t epoch;
  int64_t out_stride_b, out_stride_h;  /* of the gathered buffers, in f16 elements */
  int32_t timeout_ms;
  uint32_t* epoch_counter;  /* optional: local uint32, zero before the first call, equal on all ranks */
} WsvdPeerSet;
int wsvd_latent_decode_gather(const WsvdLatentDecodeParams* p, const WsvdPeerSet* peers, void* workspace,
                              size_t workspace_bytes, void* stream);

/*
 * Device memory that the other ranks of a node can map (CUDA IPC), for the buffers of
 * WsvdPeerSet.  wsvd_peer_alloc returns zeroed memory from cudaMalloc (these calls are the
 * only ones in the library that allocate, and they synchronise); wsvd_peer_export writes
 * the 64-byte handle to send to the peers; wsvd_peer_import maps a peer's handle and
 * enables peer access; wsvd_peer_release unmaps it.
 */
#define WSVD_PEER_HANDLE_BYTES 64
int wsvd_peer_alloc(size_t bytes, void** ptr);
int wsvd_peer_free(void* ptr);
int wsvd_peer_export(void* ptr, unsigned char handle[WSVD_PEER_HANDLE_BYTES]);
int wsvd_peer_import(const unsigned char handle[WSVD_PEER_HANDLE_BYTES], void** ptr);
int wsvd_peer_release(void* ptr);

/*
 * The whole op for callers that cannot supply a workspace.  No counterpart in the
 * reference (its wrapper always allocates mid_o with torch).
 *
 * Meant for hosts that must not, or cannot, allocate device memory around the call: an
 * inference server whose KV-cache pool already owns all free HBM, a plugin invoked where a
 * cudaMalloc would stall the device or upset the host's allocator bookkeeping, a bare C
 * caller with no allocator.  The split-KV scratch (and the position table, when
 * p->rope_table is NULL) is a fixed array of WSVD_STATIC_SCRATCH_BYTES inside the library;
 * each GPU that loads the library keeps that much memory until the process exits.
 *
 *  - Same arguments, result and status codes as wsvd_latent_decode, minus the workspace.
 *  - Returns WSVD_ERR_TOO_LARGE when wsvd_latent_decode_workspace_bytes(p) exceeds
 *    WSVD_STATIC_SCRATCH_BYTES (pass a prebuilt rope_table to leave more room for
 *    partials, or use wsvd_latent_decode).
 *  - The first call on each device looks up the array's device address (one
 *    cudaGetSymbolAddress, with the calling thread's current device); make that first call
 *    before starting any stream capture.  No call allocates or frees memory.
 *  - All calls on a device share the one array, which still holds the previous call's
 *    partials; nothing in it needs clearing.  Two calls whose kernels can overlap on the
 *    GPU (different streams, or concurrent host threads) race on it: serialise them.
 */
#define WSVD_STATIC_SCRATCH_BYTES (8u << 20)
int wsvd_latent_decode_static(const WsvdLatentDecodeParams* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* WSVD_B200_H_ */

// extern "C" entry points: validation, split plan, launches.  No allocation, no
// synchronisation; everything is enqueued on the caller's stream.
#include <math.h>
#include <string.h>

#include "common.cuh"

namespace {

thread_local int g_last_cuda_error = 0;

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return WSVD_ERR_CUDA;
}

bool is_pow2_dim(int d) { return d == 16 || d == 32 || d == 64 || d == 128; }

// Preconditions of the reference wrappers (stage1.py:231-243) plus the ones its kernels
// assume silently (contiguous innermost dims, positive sizes).
int validate(const WsvdLatentDecodeParams* p, bool need_out) {
  if (!p) return WSVD_ERR_NULL_POINTER;
  if (!p->q || !p->latent_k || !p->latent_v || !p->wk || !p->req_to_token || !p->b_req_idx || !p->b_seq_len)
    return WSVD_ERR_NULL_POINTER;
  if (need_out && !p->out) return WSVD_ERR_NULL_POINTER;
  if (p->latent_dtype != WSVD_I8 && p->latent_dtype != WSVD_F16) return WSVD_ERR_BAD_DTYPE;
  if (p->wk_dtype != WSVD_I8 && p->wk_dtype != WSVD_F16) return WSVD_ERR_BAD_DTYPE;
  if (p->latent_dtype == WSVD_I8 && (!p->k_scale || !p->v_scale)) return WSVD_ERR_BAD_DTYPE;
  if (p->wk_dtype == WSVD_I8 && !p->wk_scale) return WSVD_ERR_BAD_DTYPE;
  if (p->rope_layout != WSVD_ROPE_HALF && p->rope_layout != WSVD_ROPE_INTERLEAVED) return WSVD_ERR_BAD_DTYPE;
  if (p->batch < 0 || p->max_len < 0) return WSVD_ERR_BAD_SHAPE;
  if (!is_pow2_dim(p->head_dim)) return WSVD_ERR_BAD_SHAPE;
  if (p->n_q_heads <= 0 || p->n_kv_heads <= 0 || p->n_q_heads % p->n_kv_heads != 0) return WSVD_ERR_BAD_SHAPE;
  if (p->rank_k <= 0 || p->rank_k > 128 || p->rank_v <= 0 || p->rank_v > 128) return WSVD_ERR_BAD_SHAPE;
  if (p->batch > 65535 || p->n_q_heads > 65535) return WSVD_ERR_TOO_LARGE;
  if (p->split_len < 0) return WSVD_ERR_BAD_SHAPE;
  if (p->kernel < WSVD_KERNEL_AUTO || p->kernel > WSVD_KERNEL_MMA) return WSVD_ERR_BAD_DTYPE;
  if (!(p->theta > 0.f)) return WSVD_ERR_BAD_SHAPE;
  return WSVD_OK;
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

// The tcgen05 kernel covers the decode shapes of the 7B/13B models with an int8 cache; the
// warp-MMA kernel takes f16 latents, other head dimensions and any even rank; the rest runs on the
// generic kernel.
bool tc_eligible(const WsvdLatentDecodeParams* p) {
  if (p->kernel == WSVD_KERNEL_GENERIC || p->kernel == WSVD_KERNEL_MMA) return false;
  if (p->head_dim != 128) return false;
  if (p->rank_k % 16 != 0 || p->rank_k > 64 || p->rank_v % 16 != 0 || p->rank_v > 64) return false;
  if (p->latent_dtype != WSVD_I8) return false;
  // with position offsets the table must reach max(pos_offset) + max_len, which only the caller knows
  if (p->pos_offset != nullptr && p->rope_table == nullptr) return false;
  if (p->split_len % 128 != 0) return false;
  if (!aligned16(p->latent_k) || !aligned16(p->latent_v)) return false;
  if (!aligned16(p->q) || p->q_stride_b % 8 || p->q_stride_h % 8) return false;  // 16-byte loads of q
  if (p->k_stride_t % 16 || p->k_stride_h % 16 || p->v_stride_t % 16 || p->v_stride_h % 16) return false;
  if (p->rope_table && (!aligned16(p->rope_table) || p->rope_table_rows < ((p->max_len + 127) / 128) * 128))
    return false;
  return true;
}

// the caller's position table serves the warp-MMA kernel too ([2][rows][64] f16 is its layout for head_dim 128)
bool mma_caller_table(const WsvdLatentDecodeParams* p) {
  return p->rope_table && p->head_dim == 128 && aligned16(p->rope_table) &&
         p->rope_table_rows >= ((p->max_len + 127) / 128) * 128;
}

bool mma_eligible(const WsvdLatentDecodeParams* p) {
  if (p->kernel == WSVD_KERNEL_GENERIC || p->kernel == WSVD_KERNEL_TC) return false;
  if (p->head_dim < 16) return false;
  // pairs of latents are loaded at once
  if (p->rank_k % 2 || p->rank_v % 2) return false;
  if (p->k_stride_t % 2 || p->k_stride_h % 2 || p->v_stride_t % 2 || p->v_stride_h % 2) return false;
  // token strides are multiplied as 32-bit values
  if (p->k_stride_t < 0 || p->k_stride_t > INT32_MAX || p->v_stride_t < 0 || p->v_stride_t > INT32_MAX) return false;
  const uintptr_t pair = p->latent_dtype == WSVD_I8 ? 1 : 3;
  if ((reinterpret_cast<uintptr_t>(p->latent_k) & pair) || (reinterpret_cast<uintptr_t>(p->latent_v) & pair)) return false;
  // with position offsets the table must reach max(pos_offset) + max_len, which only the caller knows
  if (p->pos_offset != nullptr && !mma_caller_table(p)) return false;
  return true;
}

int table_rows_for(int max_len) {
  int rows = ((max_len + 127) / 128) * 128;
  return rows < 128 ? 128 : rows;
}

void plan(const WsvdLatentDecodeParams* p, int* split_len, int* n_splits) {
  int sl = p->split_len;
  if (sl <= 0 && tc_eligible(p)) {
    // one CTA per (split, group of 4 heads, sequence): aim at ~6 CTAs per SM
    const long items = (long)p->batch * ((p->n_q_heads + 3) / 4);
    const long target = 148L * 6;
    long want = items > 0 ? (target + items - 1) / items : 1;
    if (want < 1) want = 1;
    long len = (p->max_len + want - 1) / want;
    len = ((len + 127) / 128) * 128;
    if (len < 128) len = 128;
    if (len > 8192) len = 8192;
    sl = (int)len;
  } else if (sl <= 0 && mma_eligible(p)) {
    // one CTA per (split, group of 4 heads, sequence), three resident per SM: a few waves of them
    const long items = (long)p->batch * ((p->n_q_heads + 3) / 4);
    const long target = 148L * 8;
    long want = items > 0 ? (target + items - 1) / items : 1;
    if (want < 1) want = 1;
    long len = (p->max_len + want - 1) / want;
    len = ((len + 127) / 128) * 128;
    if (len < 256) len = 256;
    if (len > 4096) len = 4096;
    sl = (int)len;
  } else if (sl <= 0) {
    // enough (b, h, split) items to fill 148 SMs a few times over, but never splits
    // shorter than 256 tokens (the reference's BLOCK_SEQ, flash_decoding.py:18)
    const long items = (long)p->batch * p->n_q_heads;
    const long target = 148L * 8;
    long want = items > 0 ? (target + items - 1) / items : 1;
    if (want < 1) want = 1;
    long len = (p->max_len + want - 1) / want;
    len = ((len + 127) / 128) * 128;
    if (len < 256) len = 256;
    if (len > 4096) len = 4096;
    sl = (int)len;
  }
  *split_len = sl;
  int ns = (p->max_len + sl - 1) / sl;
  *n_splits = ns < 1 ? 1 : ns;
}

void fill_args(const WsvdLatentDecodeParams* p, float* mid_o, float* lse, int split_len, int n_splits,
               wsvd::KArgs* a) {
  a->p = *p;
  const int h2 = p->head_dim / 2;
  for (int i = 0; i < wsvd::kMaxHalfDim; ++i)
    a->inv_freq[i] = i < h2 ? (float)(1.0 / pow((double)p->theta, (2.0 * i) / (double)p->head_dim)) : 0.f;
  a->mid_o = mid_o;
  a->lse = lse;
  a->split_len = split_len;
  a->n_splits = n_splits;
  a->sm_scale = p->sm_scale != 0.f ? p->sm_scale : (float)(1.0 / sqrt((double)p->head_dim));
}

// `scratch_table`: where to build the position table when the caller gave none (may be null);
// `work`: how the tensor-core kernel distributes its work (ignored by the generic kernel, which
// always runs fixed-length splits).
int run_stage1(const wsvd::KArgs& a, void* scratch_table, const wsvd::Stage1Work& work, cudaStream_t stream) {
  if (a.p.batch == 0) return WSVD_OK;
  const bool tc = tc_eligible(&a.p) && a.split_len % 128 == 0 && (a.p.rope_table || scratch_table);
  if (!tc) {
    if (a.p.kernel == WSVD_KERNEL_TC) return WSVD_ERR_UNSUPPORTED;
    if (mma_eligible(&a.p) && (mma_caller_table(&a.p) || scratch_table)) {
      const void* table = a.p.rope_table;
      int rows = a.p.rope_table_rows;
      if (!mma_caller_table(&a.p)) {
        rows = table_rows_for(a.p.max_len);
        cudaError_t e = wsvd::launch_mma_table(scratch_table, rows, a, stream);
        if (e != cudaSuccess) return cuda_fail(e);
        table = scratch_table;
      }
      cudaError_t e = wsvd::launch_stage1_mma(a, table, rows, stream);
      return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
    }
    if (a.p.kernel == WSVD_KERNEL_MMA) return WSVD_ERR_UNSUPPORTED;
    cudaError_t e = wsvd::launch_stage1_generic(a, stream);
    return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
  }
  const void* table = a.p.rope_table;
  int rows = a.p.rope_table_rows;
  if (!table) {
    rows = table_rows_for(a.p.max_len);
    cudaError_t e = wsvd::launch_rope_table(scratch_table, rows, a, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    table = scratch_table;
  }
  cudaError_t e = wsvd::launch_stage1_tc(a, table, rows, work, stream);
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

// Without a split length from the caller, a problem the tensor-core kernel can run is cut into
// equal shares of tiles, one per SM, instead of fixed-length splits.
bool balanced_mode(const WsvdLatentDecodeParams* p) { return p->split_len == 0 && tc_eligible(p); }

size_t align256(size_t b) { return (b + 255) & ~(size_t)255; }

// Workspace: partials (mid_o, then lse), [balanced mode: tile prefix sums per sequence, arrival
// counters per (sequence, head),] [the position table when the caller passed none].  Sizes do not
// depend on the device.
struct Layout {
  size_t slots;         // partial results: one per (sequence, head, split) or per (item, head of the group)
  size_t prefix_off;    // balanced mode only
  size_t arrivals_off;  // balanced mode only
  size_t table_off;
  size_t table_bytes;   // 0: the caller's table is used, or the kernel needs none
  size_t total;
};
Layout workspace_layout(const WsvdLatentDecodeParams* p, int n_splits) {
  Layout l = {};
  const bool bal = balanced_mode(p);
  const size_t n_hg = ((size_t)p->n_q_heads + wsvd::kBalancedGroup - 1) / wsvd::kBalancedGroup;
  l.slots = bal ? ((size_t)p->batch * n_hg + wsvd::kMaxBalancedCtas) * wsvd::kBalancedGroup
                : (size_t)p->batch * p->n_q_heads * n_splits;
  size_t off = align256(l.slots * ((size_t)p->rank_v + 1) * sizeof(float));
  if (bal) {
    l.prefix_off = off;
    off += align256(((size_t)p->batch + 2) * sizeof(int32_t));
    l.arrivals_off = off;
    off += align256((size_t)p->batch * p->n_q_heads * sizeof(uint32_t));
  }
  l.table_off = off;
  if (tc_eligible(p)) {
    if (!p->rope_table) l.table_bytes = wsvd::rope_table_bytes(table_rows_for(p->max_len));
  } else if (mma_eligible(p) && !mma_caller_table(p)) {
    l.table_bytes = wsvd::mma_table_bytes(table_rows_for(p->max_len), p->head_dim);
  }
  l.total = off + l.table_bytes;
  return l;
}

// persistent CTAs of the balanced mode: one per SM, never more than there can be tiles
int balanced_ctas(const WsvdLatentDecodeParams* p, int* n_ctas) {
  static int sm_count[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  int sms = dev >= 0 && dev < 64 ? sm_count[dev] : 0;
  if (sms == 0) {
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev >= 0 && dev < 64) sm_count[dev] = sms;
  }
  const long n_hg = (p->n_q_heads + wsvd::kBalancedGroup - 1) / wsvd::kBalancedGroup;
  const long most = (long)p->batch * n_hg * ((p->max_len + 127) / 128);
  long n = sms < wsvd::kMaxBalancedCtas ? sms : wsvd::kMaxBalancedCtas;
  if (n > most) n = most;
  *n_ctas = n < 1 ? 1 : (int)n;
  return WSVD_OK;
}

}  // namespace

namespace wsvd {
int record_cuda_error(cudaError_t e) { return cuda_fail(e); }
int validate_decode_params(const WsvdLatentDecodeParams* p) { return validate(p, true); }
}  // namespace wsvd

extern "C" {

int wsvd_abi_version(void) { return WSVD_ABI_VERSION; }

const char* wsvd_status_string(int status) {
  switch (status) {
    case WSVD_OK: return "ok";
    case WSVD_ERR_NULL_POINTER: return "a required pointer is NULL";
    case WSVD_ERR_BAD_SHAPE: return "unsupported head_dim / rank / head count / length";
    case WSVD_ERR_BAD_DTYPE: return "unknown dtype or layout code, or int8 data without its scales";
    case WSVD_ERR_BAD_STRIDE: return "stride or alignment precondition violated";
    case WSVD_ERR_WORKSPACE_TOO_SMALL: return "workspace smaller than wsvd_latent_decode_workspace_bytes()";
    case WSVD_ERR_CUDA: return "a CUDA runtime call failed (see wsvd_last_cuda_error)";
    case WSVD_ERR_UNSUPPORTED: return "no kernel in this build for the requested combination";
    case WSVD_ERR_TOO_LARGE: return "size beyond a fixed limit of this entry point";
    default: return "unknown status";
  }
}

int wsvd_last_cuda_error(void) { return g_last_cuda_error; }

int wsvd_latent_decode_plan(const WsvdLatentDecodeParams* p, int32_t* split_len, int32_t* n_splits) {
  if (!split_len || !n_splits) return WSVD_ERR_NULL_POINTER;
  if (!p) return WSVD_ERR_NULL_POINTER;
  if (p->max_len < 0 || p->split_len < 0 || p->batch < 0 || p->n_q_heads <= 0) return WSVD_ERR_BAD_SHAPE;
  int sl, ns;
  plan(p, &sl, &ns);
  *split_len = sl;
  *n_splits = ns;
  return WSVD_OK;
}

size_t wsvd_latent_decode_workspace_bytes(const WsvdLatentDecodeParams* p) {
  if (!p || p->max_len < 0 || p->split_len < 0 || p->batch < 0 || p->n_q_heads <= 0 || p->rank_v <= 0) return 0;
  int sl, ns;
  plan(p, &sl, &ns);
  return workspace_layout(p, ns).total;
}

size_t wsvd_rope_table_bytes(int32_t positions, int32_t head_dim) {
  if (positions < 0 || head_dim != 128) return 0;
  return wsvd::rope_table_bytes(table_rows_for(positions));
}

int wsvd_rope_table_init(void* table, size_t table_bytes, int32_t positions, int32_t head_dim, float theta,
                         void* stream) {
  if (!table) return WSVD_ERR_NULL_POINTER;
  if (head_dim != 128) return WSVD_ERR_UNSUPPORTED;
  if (positions < 0 || !(theta > 0.f)) return WSVD_ERR_BAD_SHAPE;
  if (!aligned16(table)) return WSVD_ERR_BAD_STRIDE;
  const int rows = table_rows_for(positions);
  if (table_bytes < wsvd::rope_table_bytes(rows)) return WSVD_ERR_WORKSPACE_TOO_SMALL;
  WsvdLatentDecodeParams p = {};
  p.head_dim = head_dim;
  p.theta = theta;
  wsvd::KArgs a;
  fill_args(&p, nullptr, nullptr, 128, 1, &a);
  cudaError_t e = wsvd::launch_rope_table(table, rows, a, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

int wsvd_kernel_status(uint32_t* status) {
  if (!status) return WSVD_ERR_NULL_POINTER;
  unsigned int v = 0, w = 0, x = 0;
  cudaError_t e = wsvd::read_tc_status(&v);
  if (e == cudaSuccess) e = wsvd::read_append_status(&w);
  if (e == cudaSuccess) e = wsvd::read_peer_status(&x);
  *status = v > w ? v : w;
  if (x > *status) *status = x;
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

int wsvd_kernel_status_reset(void) {
  cudaError_t e = wsvd::reset_tc_status();
  if (e == cudaSuccess) e = wsvd::reset_append_status();
  if (e == cudaSuccess) e = wsvd::reset_peer_status();
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

int wsvd_latent_quant_append_i8(const WsvdQuantAppendParams* p, void* stream) {
  if (!p) return WSVD_ERR_NULL_POINTER;
  if (p->batch < 0 || p->n_kv_heads <= 0 || p->max_len < 0) return WSVD_ERR_BAD_SHAPE;
  if (p->rank_k <= 0 || p->rank_k > 128 || p->rank_v <= 0 || p->rank_v > 128) return WSVD_ERR_BAD_SHAPE;
  if (p->x_dtype != WSVD_F16 && p->x_dtype != WSVD_F32) return WSVD_ERR_BAD_DTYPE;
  if (p->batch == 0) return WSVD_OK;
  if (!p->x_k || !p->x_v || !p->latent_k || !p->latent_v || !p->k_scale || !p->v_scale || !p->req_to_token ||
      !p->b_req_idx || !p->b_seq_len)
    return WSVD_ERR_NULL_POINTER;
  if ((int64_t)p->batch * p->n_kv_heads > (int64_t)1 << 28) return WSVD_ERR_TOO_LARGE;
  cudaError_t e = wsvd::launch_quant_append(*p, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

static int decode_impl(const WsvdLatentDecodeParams* p, const WsvdPeerSet* peers, void* workspace,
                       size_t workspace_bytes, void* stream, bool merge = true) {
  int st = validate(p, peers == nullptr && merge);
  if (st != WSVD_OK) return st;
  if (p->batch == 0) return WSVD_OK;
  const size_t need = wsvd_latent_decode_workspace_bytes(p);
  if (!workspace) return WSVD_ERR_NULL_POINTER;
  if (workspace_bytes < need) return WSVD_ERR_WORKSPACE_TOO_SMALL;
  if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return WSVD_ERR_BAD_STRIDE;
  int sl, ns;
  plan(p, &sl, &ns);
  const Layout l = workspace_layout(p, ns);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  float* mid_o = reinterpret_cast<float*>(ws);
  float* lse = mid_o + l.slots * p->rank_v;
  wsvd::KArgs a;
  fill_args(p, mid_o, lse, sl, ns, &a);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  void* scratch_table = l.table_bytes ? ws + l.table_off : nullptr;
  wsvd::PartialIndex where = {nullptr, 0, ns, sl};
  wsvd::Stage1Work work = {0, nullptr, nullptr, nullptr};
  wsvd::PeerArgs pa;
  if (balanced_mode(p)) {
    st = balanced_ctas(p, &work.n_ctas);
    if (st != WSVD_OK) return st;
    where.n_ctas = work.n_ctas;
    if (merge) {
      // one kernel: the CTA that completes a head's last partial merges and writes the output row
      // (into every rank's gathered buffer when there are peers, followed by the group's barrier)
      work.arrivals = reinterpret_cast<unsigned int*>(ws + l.arrivals_off);
      if (peers) {
        // 16-byte peer stores need aligned rows; anything else goes through the merge kernel
        bool vec = peers->out_stride_b % 8 == 0 && peers->out_stride_h % 8 == 0;
        for (int i = 0; i < peers->n_peers; ++i) vec = vec && aligned16(peers->out[i]);
        if (vec) {
          pa = wsvd::make_peer_args(*peers);
          work.peers = &pa;
        } else {
          work.arrivals = nullptr;
        }
      }
      if (work.arrivals) return run_stage1(a, scratch_table, work, s);
    }
    work.prefix = reinterpret_cast<int32_t*>(ws + l.prefix_off);
    where.prefix = work.prefix;
  }
  st = run_stage1(a, scratch_table, work, s);
  if (st != WSVD_OK || !merge) return st;
  cudaError_t e =
      peers ? wsvd::launch_stage2_peers(mid_o, lse, p->b_seq_len, *peers, p->batch, p->n_q_heads, where, p->rank_v,
                                        p->wv, p->wv_stride_r, p->n_kv_heads, p->head_dim, s)
            : wsvd::launch_stage2(mid_o, lse, p->b_seq_len, p->out, p->out_stride_b, p->out_stride_h, p->batch,
                                  p->n_q_heads, where, p->rank_v, p->wv, p->wv_stride_r, p->n_kv_heads,
                                  p->head_dim, s);
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

int wsvd_latent_decode(const WsvdLatentDecodeParams* p, void* workspace, size_t workspace_bytes, void* stream) {
  return decode_impl(p, nullptr, workspace, workspace_bytes, stream);
}

int64_t wsvd_share_begin(int32_t c, int64_t total, int32_t n_shares) {
  return n_shares > 0 ? wsvd::share_begin(c, total, n_shares) : 0;
}
int32_t wsvd_share_owner(int64_t tile, int64_t total, int32_t n_shares) {
  return total > 0 ? wsvd::share_owner(tile, total, n_shares) : 0;
}

int wsvd_latent_decode_partials(const WsvdLatentDecodeParams* p, void* workspace, size_t workspace_bytes,
                                void* stream) {
  return decode_impl(p, nullptr, workspace, workspace_bytes, stream, false);
}

int wsvd_latent_decode_gather(const WsvdLatentDecodeParams* p, const WsvdPeerSet* peers, void* workspace,
                              size_t workspace_bytes, void* stream) {
  if (!peers) return WSVD_ERR_NULL_POINTER;
  if (peers->n_peers < 1 || peers->n_peers > WSVD_MAX_PEERS || peers->rank < 0 || peers->rank >= peers->n_peers)
    return WSVD_ERR_BAD_SHAPE;
  if ((peers->epoch == 0 && !peers->epoch_counter) || peers->head_offset < 0 || peers->timeout_ms < 0)
    return WSVD_ERR_BAD_SHAPE;
  if (!peers->counter) return WSVD_ERR_NULL_POINTER;
  for (int i = 0; i < peers->n_peers; ++i)
    if (!peers->out[i] || !peers->flags[i]) return WSVD_ERR_NULL_POINTER;
  // a rank without sequences would launch nothing and leave its peers waiting at the group barrier
  if (p && p->batch == 0) return WSVD_ERR_BAD_SHAPE;
  return decode_impl(p, peers, workspace, workspace_bytes, stream);
}

// ---- device memory that other processes of the node can map (CUDA IPC)
int wsvd_peer_alloc(size_t bytes, void** ptr) {
  if (!ptr || bytes == 0) return WSVD_ERR_NULL_POINTER;
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}
int wsvd_peer_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}
int wsvd_peer_export(void* ptr, unsigned char handle[WSVD_PEER_HANDLE_BYTES]) {
  if (!ptr || !handle) return WSVD_ERR_NULL_POINTER;
  static_assert(sizeof(cudaIpcMemHandle_t) == WSVD_PEER_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return cuda_fail(e);
  memcpy(handle, &h, sizeof(h));
  return WSVD_OK;
}
int wsvd_peer_import(const unsigned char handle[WSVD_PEER_HANDLE_BYTES], void** ptr) {
  if (!ptr || !handle) return WSVD_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}
int wsvd_peer_release(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

int wsvd_latent_decode_stage1(const WsvdLatentDecodeParams* p, float* mid_o, float* lse, int32_t n_splits,
                              void* stream) {
  int st = validate(p, false);
  if (st != WSVD_OK) return st;
  if (!mid_o || !lse) return WSVD_ERR_NULL_POINTER;
  if (p->split_len <= 0) return WSVD_ERR_BAD_SHAPE;
  if ((long)n_splits * p->split_len < p->max_len) return WSVD_ERR_WORKSPACE_TOO_SMALL;
  wsvd::KArgs a;
  fill_args(p, mid_o, lse, p->split_len, n_splits, &a);
  return run_stage1(a, nullptr, wsvd::Stage1Work{0, nullptr, nullptr, nullptr}, reinterpret_cast<cudaStream_t>(stream));
}

static void dense_plan(const WsvdDenseDecodeParams* p, int* sl, int* ns) {
  int len = p->split_len;
  if (len <= 0) {
    const long items = (long)p->batch * p->n_q_heads;
    long want = items > 0 ? (148L * 16 + items - 1) / items : 1;
    if (want < 1) want = 1;
    long l = (p->max_len + want - 1) / want;
    l = ((l + 63) / 64) * 64;
    if (l < 256) l = 256;
    len = (int)l;
  }
  *sl = len;
  int n = (p->max_len + len - 1) / len;
  *ns = n < 1 ? 1 : n;
}

size_t wsvd_dense_decode_workspace_bytes(const WsvdDenseDecodeParams* p) {
  if (!p || p->batch < 0 || p->n_q_heads <= 0 || p->head_dim <= 0 || p->max_len < 0 || p->split_len < 0) return 0;
  int sl, ns;
  dense_plan(p, &sl, &ns);
  return (size_t)p->batch * p->n_q_heads * ns * ((size_t)p->head_dim + 1) * sizeof(float);
}

int wsvd_dense_decode_f16(const WsvdDenseDecodeParams* p, void* workspace, size_t workspace_bytes, void* stream) {
  if (!p) return WSVD_ERR_NULL_POINTER;
  if (!p->q || !p->k || !p->v || !p->req_to_token || !p->b_req_idx || !p->b_seq_len || !p->out)
    return WSVD_ERR_NULL_POINTER;
  if (!is_pow2_dim(p->head_dim)) return WSVD_ERR_BAD_SHAPE;
  if (p->batch < 0 || p->max_len < 0 || p->split_len < 0) return WSVD_ERR_BAD_SHAPE;
  if (p->n_q_heads <= 0 || p->n_kv_heads <= 0 || p->n_q_heads % p->n_kv_heads != 0) return WSVD_ERR_BAD_SHAPE;
  if (p->batch > 65535 || p->n_q_heads > 65535) return WSVD_ERR_TOO_LARGE;
  // 16-byte row loads
  if (p->head_dim >= 64 && (!aligned16(p->k) || !aligned16(p->v) || p->k_stride_t % 8 || p->k_stride_h % 8 ||
                            p->v_stride_t % 8 || p->v_stride_h % 8))
    return WSVD_ERR_BAD_STRIDE;
  if (p->batch == 0) return WSVD_OK;
  if (!workspace) return WSVD_ERR_NULL_POINTER;
  if (workspace_bytes < wsvd_dense_decode_workspace_bytes(p)) return WSVD_ERR_WORKSPACE_TOO_SMALL;
  if (!aligned16(workspace)) return WSVD_ERR_BAD_STRIDE;
  int sl, ns;
  dense_plan(p, &sl, &ns);
  wsvd::DenseArgs a;
  a.q = reinterpret_cast<const __half*>(p->q); a.q_stride_b = p->q_stride_b; a.q_stride_h = p->q_stride_h;
  a.k = reinterpret_cast<const __half*>(p->k); a.k_stride_t = p->k_stride_t; a.k_stride_h = p->k_stride_h;
  a.v = reinterpret_cast<const __half*>(p->v); a.v_stride_t = p->v_stride_t; a.v_stride_h = p->v_stride_h;
  a.req_to_token = p->req_to_token; a.rtt_stride = p->rtt_stride;
  a.b_req_idx = p->b_req_idx; a.b_seq_len = p->b_seq_len;
  a.mid_o = reinterpret_cast<float*>(workspace);
  a.lse = a.mid_o + (size_t)p->batch * p->n_q_heads * ns * p->head_dim;
  a.batch = p->batch; a.n_q_heads = p->n_q_heads; a.n_kv_heads = p->n_kv_heads; a.head_dim = p->head_dim;
  a.split_len = sl; a.n_splits = ns;
  a.sm_scale = p->sm_scale != 0.f ? p->sm_scale : (float)(1.0 / sqrt((double)p->head_dim));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = wsvd::launch_dense_stage1(a, s);
  if (e != cudaSuccess) return cuda_fail(e);
  e = wsvd::launch_stage2(a.mid_o, a.lse, p->b_seq_len, p->out, p->out_stride_b, p->out_stride_h, p->batch,
                          p->n_q_heads, wsvd::PartialIndex{nullptr, 0, ns, sl}, p->head_dim, nullptr, 0, 1,
                          p->head_dim, s);
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

int wsvd_decode_stage2(const float* mid_o, const float* lse, const int32_t* b_seq_len, void* out,
                       int64_t out_stride_b, int64_t out_stride_h, int32_t batch, int32_t n_q_heads,
                       int32_t n_splits, int32_t width, int32_t split_len, const void* wv, int64_t wv_stride_r,
                       int32_t n_kv_heads, int32_t head_dim, void* stream) {
  if (!mid_o || !lse || !b_seq_len || !out) return WSVD_ERR_NULL_POINTER;
  if (batch < 0 || n_q_heads <= 0 || n_splits <= 0 || split_len <= 0) return WSVD_ERR_BAD_SHAPE;
  if (width <= 0 || width > 128) return WSVD_ERR_BAD_SHAPE;
  if (batch > 65535) return WSVD_ERR_TOO_LARGE;
  if (wv && (n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 || head_dim <= 0 || head_dim > 1024))
    return WSVD_ERR_BAD_SHAPE;
  if (batch == 0) return WSVD_OK;
  cudaError_t e = wsvd::launch_stage2(mid_o, lse, b_seq_len, out, out_stride_b, out_stride_h, batch, n_q_heads,
                                      wsvd::PartialIndex{nullptr, 0, n_splits, split_len}, width, wv, wv_stride_r,
                                      wv ? n_kv_heads : 1, head_dim, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? WSVD_OK : cuda_fail(e);
}

}  // extern "C"

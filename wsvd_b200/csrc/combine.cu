// Split-KV stage 2: merge the per-split normalised partials of one (sequence, head) by
// their log-sum-exp weights, optionally multiply the merged latent-space row by the
// head's slice of U_v, and write f16.
//
//   O = sum_i e^{lse_i - m} mid_i / sum_i e^{lse_i - m},  i < ceil(len/split_len)
// (efficiency/kernel/flash_latent_per_head_decoding_stage2.py:25,35-47).  A sequence of
// length 0 gives zeros; the reference divides by zero there.
#include "common.cuh"

//
// With a peer set the kernel is also the head all-gather of a head-sharded group of GPUs: every
// row is stored into the gathered [B, H_total, D] buffer of EVERY rank (plain stores through
// peer mappings, NVLink), and the last block of the grid then runs the group's barrier:
// a system-scope fence, one flag store per peer ("rank r has delivered epoch e"), and a
// bounded wait until every peer's flag for this rank shows the epoch.  There is no separate
// collective call and no second pass over the data.
namespace wsvd {
namespace {

constexpr int kThreads = 128;
constexpr int kMaxOutRow = 1024;  // widest output row (head_dim) the entry points accept
__device__ unsigned int g_peer_status = 0;

template <bool kPeers>
__global__ void __launch_bounds__(kThreads)
stage2_kernel(const float* __restrict__ mid_o, const float* __restrict__ lse, const int32_t* __restrict__ b_seq_len,
              __half* __restrict__ out, int64_t out_stride_b, int64_t out_stride_h, int n_q_heads,
              const PartialIndex where, int width, const __half* __restrict__ wv, int64_t wv_stride_r, int n_kv_heads,
              int head_dim, const __grid_constant__ PeerArgs pa) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int n = b_seq_len[b];
  // partial i of this (sequence, head) sits in slot slot0 + i * step
  int ns = 0;
  int64_t slot0 = 0, step = 1;
  if (n > 0 && where.prefix == nullptr) {
    ns = min(where.n_splits, (n + where.split_len - 1) / where.split_len);
    slot0 = ((int64_t)b * n_q_heads + h) * where.n_splits;
  } else if (n > 0) {
    const int n_hg = (n_q_heads + kBalancedGroup - 1) / kBalancedGroup, hg = h / kBalancedGroup;
    const int before = where.prefix[b], tiles_b = where.prefix[b + 1] - before;
    const int64_t total = (int64_t)where.prefix[gridDim.y] * n_hg;
    const int shares = where.prefix[gridDim.y + 1];
    const int64_t first = (int64_t)before * n_hg + (int64_t)hg * tiles_b;
    const int c0 = share_owner(first, total, shares), c1 = share_owner(first + tiles_b - 1, total, shares);
    ns = c1 - c0 + 1;
    slot0 = ((int64_t)b * n_hg + hg + c0) * kBalancedGroup + h % kBalancedGroup;
    step = kBalancedGroup;
  }
  __shared__ float row[128];

  // every thread computes the (tiny) max and weight sum itself: ns <= a few hundred
  float m = -INFINITY;
  for (int i = 0; i < ns; ++i) m = fmaxf(m, lse[slot0 + i * step]);
  float wsum = 0.f;
  for (int i = 0; i < ns; ++i) wsum += __expf(lse[slot0 + i * step] - m);

  const int r = threadIdx.x;
  float o = 0.f;
  if (r < width && ns > 0) {
    for (int i = 0; i < ns; ++i) o = fmaf(__expf(lse[slot0 + i * step] - m), mid_o[(slot0 + i * step) * width + r], o);
    o /= wsum;
  }
  const int64_t doff = kPeers ? (int64_t)b * pa.out_stride_b + (int64_t)(h + pa.head_offset) * pa.out_stride_h
                              : (int64_t)b * out_stride_b + (int64_t)h * out_stride_h;
  // With peers the finished row is staged in shared memory and leaves as 16-byte stores, one per
  // thread per peer (a 128-dim row is 16 such stores per peer), instead of one 2-byte store per
  // element per peer: NVLink carries far fewer, fuller packets.
  __shared__ __align__(16) __half orow[kPeers ? kMaxOutRow : 8];
  auto store = [&](int d, float y) {
    const __half v = __float2half_rn(y);
    if constexpr (kPeers) {
      orow[d] = v;
    } else {
      out[doff + d] = v;
    }
  };
  if (wv == nullptr) {
    if (r < width) store(r, o);
  } else {
    if (r < width) row[r] = o;
    __syncthreads();
    const int hk = h / (n_q_heads / n_kv_heads);
    for (int d = threadIdx.x; d < head_dim; d += kThreads) {
      // four partial sums and a deep unroll: the loads of U_v (L2) are independent of one
      // another, so many are in flight at once instead of one per dependent step
      float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
      const __half* w = wv + (int64_t)hk * head_dim + d;
      int k = 0;
#pragma unroll 4
      for (; k + 4 <= width; k += 4) {
        y0 = fmaf(row[k], __half2float(__ldg(w + (int64_t)k * wv_stride_r)), y0);
        y1 = fmaf(row[k + 1], __half2float(__ldg(w + (int64_t)(k + 1) * wv_stride_r)), y1);
        y2 = fmaf(row[k + 2], __half2float(__ldg(w + (int64_t)(k + 2) * wv_stride_r)), y2);
        y3 = fmaf(row[k + 3], __half2float(__ldg(w + (int64_t)(k + 3) * wv_stride_r)), y3);
      }
      for (; k < width; ++k) y0 = fmaf(row[k], __half2float(__ldg(w + (int64_t)k * wv_stride_r)), y0);
      store(d, (y0 + y1) + (y2 + y3));
    }
  }
  if constexpr (kPeers) {
    const int n_out = wv == nullptr ? width : head_dim;
    __syncthreads();
    bool vec = (n_out & 7) == 0 && (doff & 7) == 0;
#pragma unroll
    for (int i = 0; i < WSVD_MAX_PEERS; ++i)
      if (i < pa.n_peers) vec = vec && (reinterpret_cast<uintptr_t>(pa.out[i]) & 15) == 0;
    if (vec) {
      const int chunks = n_out >> 3;
      for (int idx = threadIdx.x; idx < chunks * pa.n_peers; idx += kThreads) {
        const int peer = idx / chunks, c = idx - peer * chunks;
        *reinterpret_cast<uint4*>(pa.out[peer] + doff + 8 * c) = reinterpret_cast<const uint4*>(orow)[c];
      }
    } else {
      for (int d = threadIdx.x; d < n_out; d += kThreads)
        for (int i = 0; i < pa.n_peers; ++i) pa.out[i][doff + d] = orow[d];
    }
    // ---- group barrier, run by whichever block finishes last
    __shared__ bool last;
    __threadfence_system();  // this thread's peer stores are ordered before what follows
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int done = atomicAdd(pa.counter, 1u) + 1u;
      last = done == gridDim.x * gridDim.y;
    }
    __syncthreads();
    if (!last) return;
    if (threadIdx.x == 0) *pa.counter = 0u;  // ready for the next launch
    peer_group_barrier(pa, &g_peer_status);
  }
}

}  // namespace

cudaError_t launch_stage2(const float* mid_o, const float* lse, const int32_t* b_seq_len, void* out,
                          int64_t out_stride_b, int64_t out_stride_h, int batch, int n_q_heads,
                          const PartialIndex& where, int width, const void* wv, int64_t wv_stride_r, int n_kv_heads,
                          int head_dim, cudaStream_t stream) {
  dim3 grid(n_q_heads, batch);
  stage2_kernel<false><<<grid, kThreads, 0, stream>>>(mid_o, lse, b_seq_len, reinterpret_cast<__half*>(out),
                                                      out_stride_b, out_stride_h, n_q_heads, where, width,
                                                      reinterpret_cast<const __half*>(wv), wv_stride_r,
                                                      n_kv_heads, head_dim, PeerArgs{});
  return cudaGetLastError();
}

cudaError_t launch_stage2_peers(const float* mid_o, const float* lse, const int32_t* b_seq_len,
                                const WsvdPeerSet& peers, int batch, int n_q_heads, const PartialIndex& where,
                                int width, const void* wv, int64_t wv_stride_r, int n_kv_heads, int head_dim,
                                cudaStream_t stream) {
  const PeerArgs pa = make_peer_args(peers);
  dim3 grid(n_q_heads, batch);
  stage2_kernel<true><<<grid, kThreads, 0, stream>>>(mid_o, lse, b_seq_len, nullptr, 0, 0, n_q_heads, where, width,
                                                     reinterpret_cast<const __half*>(wv), wv_stride_r, n_kv_heads,
                                                     head_dim, pa);
  return cudaGetLastError();
}

cudaError_t read_peer_status(unsigned int* out) { return cudaMemcpyFromSymbol(out, g_peer_status, sizeof(unsigned int)); }
cudaError_t reset_peer_status() {
  const unsigned int zero = 0;
  return cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(unsigned int));
}

}  // namespace wsvd

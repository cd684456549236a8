// Shared device-side definitions for the latent flash-decoding kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "wsvd_b200.h"

namespace wsvd {

constexpr int kMaxHalfDim = 64;  // head_dim <= 128

// Kernel argument block, passed by value (__grid_constant__).
struct KArgs {
  WsvdLatentDecodeParams p;
  float inv_freq[kMaxHalfDim];  // theta^(-2i/D), rounded once from double on the host
  float* mid_o;                 // [B, Hq, n_splits, Rv] normalised partials
  float* lse;                   // [B, Hq, n_splits]     max + log(sum)
  int32_t split_len;
  int32_t n_splits;
  float sm_scale;
};

// Kernel argument block of the dense baseline.
struct DenseArgs {
  const __half* q;  int64_t q_stride_b, q_stride_h;
  const __half* k;  int64_t k_stride_t, k_stride_h;
  const __half* v;  int64_t v_stride_t, v_stride_h;
  const int32_t* req_to_token; int64_t rtt_stride;
  const int32_t* b_req_idx;
  const int32_t* b_seq_len;
  float* mid_o;
  float* lse;
  int32_t batch, n_q_heads, n_kv_heads, head_dim, split_len, n_splits;
  float sm_scale;
};

__device__ __forceinline__ float to_float(int8_t v) { return static_cast<float>(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Balanced work distribution of the tensor-core kernel: `total` tiles in a fixed order are cut into
// n_ctas shares; share c is [share_begin(c), share_begin(c + 1)), and share_owner inverts that.
__host__ __device__ __forceinline__ int64_t share_begin(int c, int64_t total, int n_ctas) {
  return (int64_t)c * total / n_ctas;
}
// the c with share_begin(c) <= tile < share_begin(c + 1), for 0 <= tile < total
__host__ __device__ __forceinline__ int share_owner(int64_t tile, int64_t total, int n_ctas) {
  return (int)(((tile + 1) * n_ctas - 1) / total);
}
constexpr int kBalancedGroup = 4;  // query heads per work item of the tensor-core kernel
constexpr int kMaxBalancedCtas = 256;

// Where the merge finds the partials.  Split mode (prefix null): [B, Hq, n_splits] slots, the first
// ceil(len / split_len) of a row used.  Balanced mode: slot (b * n_hg + hg + c) * 4 + h % 4 for every
// CTA c whose share holds tiles of (sequence b, head group hg); prefix[b] = tiles in sequences before
// b, prefix[batch + 1] = number of shares (both written by stage 1).
struct PartialIndex {
  const int32_t* prefix;  // [batch + 2], or null
  int32_t n_ctas;         // CTAs of the stage-1 grid (>= the number of shares)
  int32_t n_splits;
  int32_t split_len;
};

// Shared by the entry points that live outside capi.cu: the argument checks of
// wsvd_latent_decode, and the per-thread record behind wsvd_last_cuda_error()
// (returns WSVD_ERR_CUDA).
int validate_decode_params(const WsvdLatentDecodeParams* p);
int record_cuda_error(cudaError_t e);

// Launchers implemented in the kernel translation units.
cudaError_t launch_stage1_generic(const KArgs& a, cudaStream_t stream);
// A head-sharded group of GPUs: where every rank's gathered [B, H_total, D] buffer and flag array are
// mapped, and the state of the group barrier (see combine.cu).
struct PeerArgs {
  __half* out[WSVD_MAX_PEERS];
  uint32_t* flags[WSVD_MAX_PEERS];
  uint32_t* counter;
  uint32_t* epoch_counter;
  int64_t out_stride_b, out_stride_h;
  int32_t n_peers, rank, head_offset;
  uint32_t epoch;
  uint64_t timeout_ns;
};
constexpr unsigned int kPeerWaitTimedOut = 6;

inline PeerArgs make_peer_args(const WsvdPeerSet& peers) {
  PeerArgs pa{};
  for (int i = 0; i < peers.n_peers; ++i) {
    pa.out[i] = reinterpret_cast<__half*>(peers.out[i]);
    pa.flags[i] = peers.flags[i];
  }
  pa.counter = peers.counter;
  pa.epoch_counter = peers.epoch_counter;
  pa.out_stride_b = peers.out_stride_b;
  pa.out_stride_h = peers.out_stride_h;
  pa.n_peers = peers.n_peers;
  pa.rank = peers.rank;
  pa.head_offset = peers.head_offset;
  pa.epoch = peers.epoch;
  pa.timeout_ns = peers.timeout_ms > 0 ? (uint64_t)peers.timeout_ms * 1000000ull : 2000000000ull;
  return pa;
}

#ifdef __CUDACC__
// The group's barrier, run by every thread of the block that finishes last (the caller has made
// sure that every block's peer stores are fenced and counted): bump the step's epoch, tell every
// peer "rank r has delivered epoch e" and wait, with a time limit, until every peer's word for this
// rank shows the epoch.  On a time-out kPeerWaitTimedOut is recorded in *status.
__device__ __forceinline__ void peer_group_barrier(const PeerArgs& pa, unsigned int* status) {
  // the step's epoch: the caller's, or one more than the device-side count of past steps
  uint32_t epoch = pa.epoch;
  if (pa.epoch_counter != nullptr) {
    epoch = *reinterpret_cast<volatile uint32_t*>(pa.epoch_counter) + 1u;
    __syncthreads();  // every thread of this (last) block has read the old count
    if (threadIdx.x == 0) *pa.epoch_counter = epoch;
  }
  __threadfence_system();
  const int i = threadIdx.x;
  if (i < pa.n_peers) {
    // "rank pa.rank has delivered epoch e" into peer i's flag array ...
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pa.flags[i] + pa.rank), "r"(epoch) : "memory");
    // ... and wait for peer i's word in ours; epochs only grow (wrap-safe comparison)
    const uint32_t* mine = pa.flags[pa.rank] + i;
    uint64_t t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      uint64_t now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now - t0 > pa.timeout_ns) {
        atomicMax(status, kPeerWaitTimedOut);
        break;
      }
    }
  }
}
#endif

// How the tensor-core kernel distributes its work.  n_ctas == 0: one CTA per (split, head group,
// sequence), partials in the split layout.  n_ctas > 0: that many persistent CTAs with equal shares
// of the tile list, partials in the balanced layout; then either `prefix` ([batch + 2] int32, written
// by the kernel for the merge kernel) or `arrivals` ([batch * n_q_heads] uint32, zeroed by the
// launcher: the kernel merges, applies U_v and writes the output rows itself) is given.  With
// `arrivals` and `peers`, the rows go into every rank's gathered buffer instead of p.out and the CTA
// that finishes last runs the group's barrier: the head all-gather is part of the kernel.
struct Stage1Work {
  int n_ctas;
  int32_t* prefix;
  unsigned int* arrivals;
  const PeerArgs* peers;
};
cudaError_t launch_stage1_tc(const KArgs& a, const void* table, int table_rows, const Stage1Work& work,
                             cudaStream_t stream);
cudaError_t launch_rope_table(void* table, int rows, const KArgs& a, cudaStream_t stream);
// warp-MMA kernel: its table is [2][rows][head_dim / 2] f16 (the same bytes as the table above for head_dim 128)
cudaError_t launch_stage1_mma(const KArgs& a, const void* table, int rows, cudaStream_t stream);
cudaError_t launch_mma_table(void* table, int rows, const KArgs& a, cudaStream_t stream);
size_t mma_table_bytes(int rows, int head_dim);
size_t rope_table_bytes(int rows);
cudaError_t read_tc_status(unsigned int* out);
cudaError_t reset_tc_status();
cudaError_t launch_dense_stage1(const DenseArgs& a, cudaStream_t stream);
cudaError_t launch_stage2_peers(const float* mid_o, const float* lse, const int32_t* b_seq_len,
                                const WsvdPeerSet& peers, int batch, int n_q_heads, const PartialIndex& where,
                                int width, const void* wv, int64_t wv_stride_r, int n_kv_heads, int head_dim,
                                cudaStream_t stream);
cudaError_t read_peer_status(unsigned int* out);
cudaError_t reset_peer_status();
cudaError_t launch_quant_append(const WsvdQuantAppendParams& p, cudaStream_t stream);
cudaError_t read_append_status(unsigned int* out);
cudaError_t reset_append_status();
cudaError_t launch_stage2(const float* mid_o, const float* lse, const int32_t* b_seq_len, void* out,
                          int64_t out_stride_b, int64_t out_stride_h, int batch, int n_q_heads,
                          const PartialIndex& where, int width, const void* wv, int64_t wv_stride_r, int n_kv_heads,
                          int head_dim, cudaStream_t stream);

}  // namespace wsvd

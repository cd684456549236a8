// Dense f16 flash-decoding baseline: softmax(q.K^T / sqrt(D)).V on full K/V caches
// [T, Hkv, D] read through the page table, no RoPE (K is stored rotated).  Same split-KV
// skeleton and partial format as the latent kernels; it exists to measure the
// rank-reduction speed-up against a dense kernel of equal shape on the same GPU
// (efficiency/kernel/flash_decoding_stage1.py:6-105; the reference runs it with one warp
// per CTA and 16-token tiles).
//
// A warp handles four tokens per step: lane = (token slot, eighth of the head dim), each
// lane loads D/8 f16 of the K and V rows with 16-byte loads, the score is reduced over the
// eight lanes of a token, and every lane keeps the output accumulator of its dims.
#include "common.cuh"

namespace wsvd {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;

template <int D>
__global__ void __launch_bounds__(kThreads) dense_stage1_kernel(const __grid_constant__ DenseArgs a) {
  constexpr int E = D / 8;  // elements per lane
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n = a.b_seq_len[b];
  const int lo = split * a.split_len;
  const int hi = min(n, lo + a.split_len);
  if (hi <= lo) return;
  const int hk = h / (a.n_q_heads / a.n_kv_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ts = lane >> 3, part = lane & 7;

  float qf[E];
  {
    const __half* qp = a.q + (int64_t)b * a.q_stride_b + (int64_t)h * a.q_stride_h + part * E;
#pragma unroll
    for (int e = 0; e < E; ++e) qf[e] = __half2float(qp[e]) * a.sm_scale;
  }
  const int32_t* page = a.req_to_token + (int64_t)a.b_req_idx[b] * a.rtt_stride;
  const __half* kb = a.k + (int64_t)hk * a.k_stride_h + part * E;
  const __half* vb = a.v + (int64_t)hk * a.v_stride_h + part * E;

  float m = -INFINITY, l = 0.f, acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;

  for (int s0 = lo + warp * 4; s0 < hi; s0 += kWarps * 4) {
    const int s = s0 + ts;
    const bool valid = s < hi;
    const int64_t t = valid ? page[s] : 0;
    __align__(16) __half kr[E], vr[E];
    if (valid) {
      const __half* kp = kb + t * a.k_stride_t;
      const __half* vp = vb + t * a.v_stride_t;
      if constexpr (E >= 8) {
#pragma unroll
        for (int e = 0; e < E; e += 8) {
          *reinterpret_cast<uint4*>(kr + e) = *reinterpret_cast<const uint4*>(kp + e);
          *reinterpret_cast<uint4*>(vr + e) = *reinterpret_cast<const uint4*>(vp + e);
        }
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          kr[e] = kp[e];
          vr[e] = vp[e];
        }
      }
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) kr[e] = vr[e] = __float2half(0.f);
    }
    float part_dot = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) part_dot = fmaf(qf[e], __half2float(kr[e]), part_dot);
    part_dot += __shfl_xor_sync(0xffffffffu, part_dot, 1);
    part_dot += __shfl_xor_sync(0xffffffffu, part_dot, 2);
    part_dot += __shfl_xor_sync(0xffffffffu, part_dot, 4);
    const float z = valid ? part_dot : -INFINITY;
    const float m_new = fmaxf(m, z);
    const float sc = m_new == -INFINITY ? 0.f : __expf(m - m_new);
    const float pr = valid ? __expf(z - m_new) : 0.f;
    l = l * sc + pr;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = fmaf(pr, __half2float(vr[e]), acc[e] * sc);
    m = m_new;
  }

  // merge the four token slots of the warp, then the warps
  __shared__ float red[kWarps][2 + D];
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    const float mo = __shfl_xor_sync(0xffffffffu, m, o);
    const float lo_ = __shfl_xor_sync(0xffffffffu, l, o);
    const float mm = fmaxf(m, mo);
    const float w0 = m == -INFINITY ? 0.f : __expf(m - mm), w1 = mo == -INFINITY ? 0.f : __expf(mo - mm);
    l = l * w0 + lo_ * w1;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = acc[e] * w0 + __shfl_xor_sync(0xffffffffu, acc[e], o) * w1;
    m = mm;
  }
  if (ts == 0) {
    if (part == 0) {
      red[warp][0] = m;
      red[warp][1] = l;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) red[warp][2 + part * E + e] = acc[e];
  }
  __syncthreads();
  if (warp == 0) {
    float mm = -INFINITY;
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, red[w][0]);
    float wgt[kWarps], ll = 0.f;
    for (int w = 0; w < kWarps; ++w) {
      wgt[w] = red[w][0] == -INFINITY ? 0.f : __expf(red[w][0] - mm);
      ll += wgt[w] * red[w][1];
    }
    const int64_t slot = ((int64_t)b * a.n_q_heads + h) * a.n_splits + split;
    for (int d = lane; d < D; d += 32) {
      float o = 0.f;
      for (int w = 0; w < kWarps; ++w) o += wgt[w] * red[w][2 + d];
      a.mid_o[slot * D + d] = o / ll;
    }
    if (lane == 0) a.lse[slot] = mm + logf(ll);
  }
}

}  // namespace

cudaError_t launch_dense_stage1(const DenseArgs& a, cudaStream_t stream) {
  dim3 grid(a.n_splits, a.n_q_heads, a.batch);
  switch (a.head_dim) {
    case 16: dense_stage1_kernel<16><<<grid, kThreads, 0, stream>>>(a); break;
    case 32: dense_stage1_kernel<32><<<grid, kThreads, 0, stream>>>(a); break;
    case 64: dense_stage1_kernel<64><<<grid, kThreads, 0, stream>>>(a); break;
    case 128: dense_stage1_kernel<128><<<grid, kThreads, 0, stream>>>(a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace wsvd

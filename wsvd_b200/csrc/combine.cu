// Split-KV stage 2: merge the per-split normalised partials of one (sequence, head) by
// their log-sum-exp weights, optionally multiply the merged latent-space row by the
// head's slice of U_v, and write f16.
//
//   O = sum_i e^{lse_i - m} mid_i / sum_i e^{lse_i - m},  i < ceil(len/split_len)
// (efficiency/kernel/flash_latent_per_head_decoding_stage2.py:25,35-47).  A sequence of
// length 0 gives zeros; the reference divides by zero there.
#include "common.cuh"

namespace wsvd {
namespace {

constexpr int kThreads = 128;

__global__ void __launch_bounds__(kThreads)
stage2_kernel(const float* __restrict__ mid_o, const float* __restrict__ lse, const int32_t* __restrict__ b_seq_len,
              __half* __restrict__ out, int64_t out_stride_b, int64_t out_stride_h, int n_q_heads, int n_splits,
              int width, int split_len, const __half* __restrict__ wv, int64_t wv_stride_r, int n_kv_heads,
              int head_dim) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int n = b_seq_len[b];
  const int ns = n <= 0 ? 0 : min(n_splits, (n + split_len - 1) / split_len);
  const int64_t slot0 = ((int64_t)b * n_q_heads + h) * n_splits;
  __shared__ float row[128];

  // every thread computes the (tiny) max and weight sum itself: ns <= a few hundred
  float m = -INFINITY;
  for (int i = 0; i < ns; ++i) m = fmaxf(m, lse[slot0 + i]);
  float wsum = 0.f;
  for (int i = 0; i < ns; ++i) wsum += __expf(lse[slot0 + i] - m);

  const int r = threadIdx.x;
  float o = 0.f;
  if (r < width && ns > 0) {
    for (int i = 0; i < ns; ++i) o = fmaf(__expf(lse[slot0 + i] - m), mid_o[(slot0 + i) * width + r], o);
    o /= wsum;
  }
  __half* dst = out + (int64_t)b * out_stride_b + (int64_t)h * out_stride_h;
  if (wv == nullptr) {
    if (r < width) dst[r] = __float2half_rn(o);
    return;
  }
  if (r < width) row[r] = o;
  __syncthreads();
  const int hk = h / (n_q_heads / n_kv_heads);
  for (int d = threadIdx.x; d < head_dim; d += kThreads) {
    float y = 0.f;
    const __half* w = wv + (int64_t)hk * head_dim + d;
    for (int k = 0; k < width; ++k) y = fmaf(row[k], __half2float(w[(int64_t)k * wv_stride_r]), y);
    dst[d] = __float2half_rn(y);
  }
}

}  // namespace

cudaError_t launch_stage2(const float* mid_o, const float* lse, const int32_t* b_seq_len, void* out,
                          int64_t out_stride_b, int64_t out_stride_h, int batch, int n_q_heads, int n_splits,
                          int width, int split_len, const void* wv, int64_t wv_stride_r, int n_kv_heads,
                          int head_dim, cudaStream_t stream) {
  dim3 grid(n_q_heads, batch);
  stage2_kernel<<<grid, kThreads, 0, stream>>>(mid_o, lse, b_seq_len, reinterpret_cast<__half*>(out), out_stride_b,
                                               out_stride_h, n_q_heads, n_splits, width, split_len,
                                               reinterpret_cast<const __half*>(wv), wv_stride_r, n_kv_heads,
                                               head_dim);
  return cudaGetLastError();
}

}  // namespace wsvd

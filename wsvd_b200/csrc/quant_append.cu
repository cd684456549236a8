// wsvd_latent_quant_append_i8: quantise the new token's K and V latents per (sequence, head)
// to int8 with an f16 scale and write them into the latent cache at the token slot the page
// table gives for position b_seq_len[b].
//
// The reference computes the new token's latents in its layer wrapper and drops them
// (efficiency/layer_utils.py:319-321); its caches are filled by the test script with
// torch ops (efficiency/test_timing_layer.py:267-275).  The quantiser restated here is the
// accuracy pipeline's symmetric per-token one (fake_quant/quant_utils.py:30-33 for the
// rounding and clamp, :175-184 for scale = amax/maxq with 1 for an all-zero row), with the
// rounding done against the f16 value of the scale that the cache stores.
//
// One warp per (sequence, kv head, K|V): at most 128 values, a max-reduction, one divide
// per value.  The kernel is launch-latency sized; nothing here is tuned beyond coalescing.
#include "common.cuh"

namespace wsvd {
namespace {

constexpr unsigned int kAppendOutOfRange = 5;
__device__ unsigned int g_append_status = 0;

__device__ __forceinline__ float load_as_float(const void* base, int64_t idx, int dtype) {
  return dtype == WSVD_F32 ? reinterpret_cast<const float*>(base)[idx]
                           : __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

__global__ void __launch_bounds__(128) quant_append_kernel(const __grid_constant__ WsvdQuantAppendParams p) {
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int total = p.batch * p.n_kv_heads * 2;
  if (warp >= total) return;
  const int is_v = warp & 1, hk = (warp >> 1) % p.n_kv_heads, b = (warp >> 1) / p.n_kv_heads;
  const int pos = p.b_seq_len[b];
  if (pos < 0 || pos >= p.max_len) {  // no slot for this position: skip the row and say so
    if (lane == 0) atomicMax(&g_append_status, kAppendOutOfRange);
    return;
  }
  const int64_t slot = p.req_to_token[(int64_t)p.b_req_idx[b] * p.rtt_stride + pos];
  const int R = is_v ? p.rank_v : p.rank_k;
  const void* x = is_v ? p.x_v : p.x_k;
  const int64_t xoff = is_v ? (int64_t)b * p.xv_stride_b + (int64_t)hk * p.xv_stride_h
                            : (int64_t)b * p.xk_stride_b + (int64_t)hk * p.xk_stride_h;
  float v[4];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = lane + 32 * i;
    v[i] = r < R ? load_as_float(x, xoff + r, p.x_dtype) : 0.f;
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  // The stored scale is f16: amax/127 below the smallest positive f16 would round to 0 (and the
  // divide below to inf/NaN), above the largest finite f16 to inf.  Clamp to the f16 range.
  const float scale = amax == 0.f ? 1.f : fminf(fmaxf(amax / 127.f, 5.9604644775390625e-8f), 65504.f);
  const __half scale_h = __float2half_rn(scale);
  const float sf = __half2float(scale_h);
  int8_t* dst = reinterpret_cast<int8_t*>(is_v ? p.latent_v : p.latent_k) +
                (is_v ? slot * p.v_stride_t + (int64_t)hk * p.v_stride_h : slot * p.k_stride_t + (int64_t)hk * p.k_stride_h);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = lane + 32 * i;
    if (r < R) dst[r] = (int8_t)fminf(fmaxf(rintf(v[i] / sf), -128.f), 127.f);
  }
  if (lane == 0) {
    __half* sdst = reinterpret_cast<__half*>(is_v ? p.v_scale : p.k_scale) +
                   (is_v ? slot * p.vs_stride_t + (int64_t)hk * p.vs_stride_h
                         : slot * p.ks_stride_t + (int64_t)hk * p.ks_stride_h);
    *sdst = scale_h;
  }
}

}  // namespace

cudaError_t read_append_status(unsigned int* out) {
  return cudaMemcpyFromSymbol(out, g_append_status, sizeof(unsigned int));
}
cudaError_t reset_append_status() {
  const unsigned int zero = 0;
  return cudaMemcpyToSymbol(g_append_status, &zero, sizeof(unsigned int));
}

cudaError_t launch_quant_append(const WsvdQuantAppendParams& p, cudaStream_t stream) {
  const int warps = p.batch * p.n_kv_heads * 2;
  if (warps == 0) return cudaSuccess;
  quant_append_kernel<<<(warps + 3) / 4, 128, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace wsvd

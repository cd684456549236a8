// Element-wise kernels of the decode step around the attention op: RMSNorm, rotary embedding of
// the new query, SiLU(gate) * up.  In the accuracy pipeline these are chains of small torch ops
// (fake_quant/svd_utils.py:1628-1674: LlamaRMSNorm, apply_rotary_pos_emb, the MLP's act_fn); a
// decode step of batch 64 spends a third of its time launching them, so each chain is one kernel
// here.  f16 in and out, fp32 arithmetic, rounding at the same places as the torch chains.
#include "common.cuh"

namespace wsvd {
namespace {

// y[r, :] = f16( x[r, :] * rsqrt(mean(x[r, :]^2) + eps) ), one block per row
__global__ void __launch_bounds__(256) rms_norm_kernel(const __half* __restrict__ x, __half* __restrict__ y, int cols,
                                                       float eps) {
  const __half* xr = x + (int64_t)blockIdx.x * cols;
  __half* yr = y + (int64_t)blockIdx.x * cols;
  float ss = 0.f;
  for (int i = threadIdx.x; i < cols; i += 256) {
    const float v = __half2float(xr[i]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += part[w];
  const float scale = rsqrtf(tot / (float)cols + eps);
  for (int i = threadIdx.x; i < cols; i += 256) yr[i] = __float2half_rn(__half2float(xr[i]) * scale);
}

// x_out[r, :] = f16(x[r, :] + delta[r, :]) (the residual add), y[r, :] = RMSNorm of the rounded sum:
// the residual update and the next block's normalisation in one pass over the row
__global__ void __launch_bounds__(256) add_rms_norm_kernel(const __half* __restrict__ x, const __half* __restrict__ delta,
                                                           __half* __restrict__ x_out, __half* __restrict__ y, int cols,
                                                           float eps) {
  const int64_t off = (int64_t)blockIdx.x * cols;
  float ss = 0.f;
  for (int i = threadIdx.x; i < cols; i += 256) {
    const __half sum = __float2half_rn(__half2float(x[off + i]) + __half2float(delta[off + i]));
    x_out[off + i] = sum;
    const float v = __half2float(sum);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += part[w];
  const float scale = rsqrtf(tot / (float)cols + eps);
  // each thread re-reads the elements it wrote itself
  for (int i = threadIdx.x; i < cols; i += 256) y[off + i] = __float2half_rn(__half2float(x_out[off + i]) * scale);
}

// half-split rotary embedding in place: q[b, h, i], q[b, h, i + D/2] rotated by pos[b] * inv_freq[i]
__global__ void rope_half_kernel(__half* __restrict__ q, int64_t q_stride_b, const int32_t* __restrict__ pos,
                                 const float* __restrict__ inv_freq, int heads, int half_dim, int64_t total) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int i = (int)(idx % half_dim);
  const int64_t bh = idx / half_dim;
  const int b = (int)(bh / heads);
  float sn, cs;
  sincosf((float)pos[b] * inv_freq[i], &sn, &cs);
  __half* row = q + (int64_t)b * q_stride_b + (bh - (int64_t)b * heads) * (2 * half_dim);
  const float lo = __half2float(row[i]), hi = __half2float(row[i + half_dim]);
  row[i] = __float2half_rn(lo * cs - hi * sn);
  row[i + half_dim] = __float2half_rn(hi * cs + lo * sn);
}

// out = up * f16(silu(gate)), the product rounded to f16 (the two roundings of the torch chain)
__global__ void silu_mul_kernel(const __half* __restrict__ up, int64_t up_ld, const __half* __restrict__ gate,
                                int64_t gate_ld, __half* __restrict__ out, int cols, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t r = i / cols, c = i - r * cols;
  const float g = __half2float(gate[r * gate_ld + c]);
  const __half s = __float2half_rn(g / (1.f + expf(-g)));
  out[i] = __float2half_rn(__half2float(up[r * up_ld + c]) * __half2float(s));
}

}  // namespace
}  // namespace wsvd

extern "C" {

int wsvd_rms_norm_f16(const void* x, void* y, int32_t rows, int32_t cols, float eps, void* stream) {
  if (!x || !y) return WSVD_ERR_NULL_POINTER;
  if (rows < 0 || cols <= 0) return WSVD_ERR_BAD_SHAPE;
  if (rows == 0) return WSVD_OK;
  wsvd::rms_norm_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __half*>(x), reinterpret_cast<__half*>(y), cols, eps);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? WSVD_OK : wsvd::record_cuda_error(e);
}

int wsvd_add_rms_norm_f16(const void* x, const void* delta, void* x_out, void* y, int32_t rows, int32_t cols, float eps,
                          void* stream) {
  if (!x || !delta || !x_out || !y) return WSVD_ERR_NULL_POINTER;
  if (rows < 0 || cols <= 0) return WSVD_ERR_BAD_SHAPE;
  if (rows == 0) return WSVD_OK;
  wsvd::add_rms_norm_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __half*>(x), reinterpret_cast<const __half*>(delta), reinterpret_cast<__half*>(x_out),
      reinterpret_cast<__half*>(y), cols, eps);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? WSVD_OK : wsvd::record_cuda_error(e);
}

int wsvd_rope_half_f16(void* q, int64_t q_stride_b, const int32_t* pos, const float* inv_freq, int32_t batch,
                       int32_t heads, int32_t head_dim, void* stream) {
  if (!q || !pos || !inv_freq) return WSVD_ERR_NULL_POINTER;
  if (batch < 0 || heads <= 0 || head_dim <= 0 || head_dim % 2) return WSVD_ERR_BAD_SHAPE;
  if (q_stride_b < (int64_t)heads * head_dim) return WSVD_ERR_BAD_STRIDE;
  const int64_t total = (int64_t)batch * heads * (head_dim / 2);
  if (total == 0) return WSVD_OK;
  wsvd::rope_half_kernel<<<(unsigned)((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__half*>(q), q_stride_b, pos, inv_freq, heads, head_dim / 2, total);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? WSVD_OK : wsvd::record_cuda_error(e);
}

int wsvd_silu_mul_f16(const void* up, int64_t up_ld, const void* gate, int64_t gate_ld, void* out, int32_t rows,
                      int32_t cols, void* stream) {
  if (!up || !gate || !out) return WSVD_ERR_NULL_POINTER;
  if (rows < 0 || cols <= 0) return WSVD_ERR_BAD_SHAPE;
  if (up_ld < cols || gate_ld < cols) return WSVD_ERR_BAD_STRIDE;
  const int64_t n = (int64_t)rows * cols;
  if (n == 0) return WSVD_OK;
  wsvd::silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __half*>(up), up_ld, reinterpret_cast<const __half*>(gate), gate_ld,
      reinterpret_cast<__half*>(out), cols, n);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? WSVD_OK : wsvd::record_cuda_error(e);
}

}  // extern "C"

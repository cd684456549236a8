// Generic split-KV stage 1 of the latent decode attention: any head_dim in
// {16,32,64,128}, any rank <= 128, int8 or f16 latents, paged or contiguous cache, GQA,
// both RoPE pairings.  One CTA per (split, head, sequence); one warp per token.
//
// Math per token s of sequence b, head h (KV head hk), following the reference kernel
// (efficiency/kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:117-216) with
// fp32 kept through the scaling (the reference rounds to f16 before it, :152-153):
//   K[d]   = sk[t_s,hk] * sum_r Lk[t_s,hk,r] * U[hk,d,r]
//   K'     = RoPE(K, position s)            (pairs (i, i+D/2), or (2i, 2i+1))
//   z      = sm_scale * q . K'
//   online softmax over the split; acc[r] += p * sv[t_s,hk] * Lv[t_s,hk,r]
// Output: normalised partial acc/sum and lse = max + log(sum) (:211-216).
//
// This is the catch-all path and an independent witness for the tensor-core kernel;
// it reconstructs K on the CUDA cores and is not tuned.
#include "common.cuh"

namespace wsvd {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxPairs = 2;  // (D/2)/32 for D = 128
constexpr int kMaxRankRegs = 4;  // 128/32

template <typename LT>
__global__ void __launch_bounds__(kThreads) stage1_generic_kernel(const __grid_constant__ KArgs a) {
  const WsvdLatentDecodeParams& p = a.p;
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n = p.b_seq_len[b];
  const int lo = split * a.split_len;
  const int hi = min(n, lo + a.split_len);
  if (hi <= lo) return;  // empty split: nothing is written (stage1.py:211)

  const int D = p.head_dim, h2 = D >> 1, Rk = p.rank_k, Rv = p.rank_v;
  const int hk = h / (p.n_q_heads / p.n_kv_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool interleaved = p.rope_layout == WSVD_ROPE_INTERLEAVED;

  extern __shared__ float smem[];
  float* Ut = smem;                                    // [Rk][D]  U^T with wk_scale applied
  float* red = smem + Rk * D;                          // [kWarps][2 + Rv]

  // U^T from wk [Rk, Hkv*D] (+ per-column scale), stage1.py:94-108
  for (int idx = threadIdx.x; idx < Rk * D; idx += kThreads) {
    const int r = idx / D, d = idx - r * D;
    const int64_t off = (int64_t)r * p.wk_stride_r + (int64_t)hk * D + d;
    float w;
    if (p.wk_dtype == WSVD_I8) {
      w = (float)reinterpret_cast<const int8_t*>(p.wk)[off] *
          __half2float(reinterpret_cast<const __half*>(p.wk_scale)[hk * D + d]);
    } else {
      w = __half2float(reinterpret_cast<const __half*>(p.wk)[off]);
    }
    Ut[idx] = w;
  }

  // this lane's RoPE pairs and q values
  int d0[kMaxPairs], d1[kMaxPairs];
  float q0[kMaxPairs], q1[kMaxPairs], fr[kMaxPairs];
  const __half* qp = reinterpret_cast<const __half*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)h * p.q_stride_h;
#pragma unroll
  for (int k = 0; k < kMaxPairs; ++k) {
    const int i = lane + 32 * k;
    const bool on = i < h2;
    d0[k] = on ? (interleaved ? 2 * i : i) : 0;
    d1[k] = on ? (interleaved ? 2 * i + 1 : i + h2) : 0;
    q0[k] = on ? __half2float(qp[d0[k]]) : 0.f;
    q1[k] = on ? __half2float(qp[d1[k]]) : 0.f;
    fr[k] = on ? a.inv_freq[i] : 0.f;
  }
  __syncthreads();

  const int32_t* page = p.req_to_token + (int64_t)p.b_req_idx[b] * p.rtt_stride;
  const float pos0 = p.pos_offset ? (float)p.pos_offset[b] : 0.f;
  const LT* lk_base = reinterpret_cast<const LT*>(p.latent_k) + (int64_t)hk * p.k_stride_h;
  const LT* lv_base = reinterpret_cast<const LT*>(p.latent_v) + (int64_t)hk * p.v_stride_h;
  const __half* ks_base = reinterpret_cast<const __half*>(p.k_scale);
  const __half* vs_base = reinterpret_cast<const __half*>(p.v_scale);

  float m = -INFINITY, l = 0.f;
  float acc[kMaxRankRegs];
#pragma unroll
  for (int k = 0; k < kMaxRankRegs; ++k) acc[k] = 0.f;

  for (int s = lo + warp; s < hi; s += kWarps) {
    const int64_t t = page[s];  // 64-bit: T*Hkv*R can exceed 2^31 (stage1.py:123)
    const LT* lk = lk_base + t * p.k_stride_t;
    const LT* lv = lv_base + t * p.v_stride_t;
    float lkr[kMaxRankRegs], lvr[kMaxRankRegs];
#pragma unroll
    for (int k = 0; k < kMaxRankRegs; ++k) {
      const int r = lane + 32 * k;
      lkr[k] = r < Rk ? to_float(lk[r]) : 0.f;
      lvr[k] = r < Rv ? to_float(lv[r]) : 0.f;
    }
    float sk = 1.f, sv = 1.f;
    if (ks_base) {
      sk = __half2float(ks_base[t * p.ks_stride_t + (int64_t)hk * p.ks_stride_h]);
      sv = __half2float(vs_base[t * p.vs_stride_t + (int64_t)hk * p.vs_stride_h]);
    }

    float k0[kMaxPairs] = {0.f, 0.f}, k1[kMaxPairs] = {0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < kMaxRankRegs; ++kk) {
      if (kk * 32 < Rk) {
        const int rn = min(32, Rk - kk * 32);
        for (int rr = 0; rr < rn; ++rr) {
          const float x = __shfl_sync(0xffffffffu, lkr[kk], rr);
          const float* u = Ut + (kk * 32 + rr) * D;
#pragma unroll
          for (int k = 0; k < kMaxPairs; ++k) {
            k0[k] = fmaf(x, u[d0[k]], k0[k]);
            k1[k] = fmaf(x, u[d1[k]], k1[k]);
          }
        }
      }
    }
    const float pos = pos0 + (float)s;
    float part = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxPairs; ++k) {
      float sn, cs;
      sincosf(pos * fr[k], &sn, &cs);
      const float a0 = k0[k] * sk, a1 = k1[k] * sk;
      const float r0 = a0 * cs - a1 * sn;
      const float r1 = a1 * cs + a0 * sn;
      part = fmaf(q0[k], r0, part);
      part = fmaf(q1[k], r1, part);
    }
    const float z = warp_sum(part) * a.sm_scale;
    const float m_new = fmaxf(m, z);
    const float sc = __expf(m - m_new);  // m = -inf on the first token -> 0
    const float pr = __expf(z - m_new);
    l = l * sc + pr;
    const float pv = pr * sv;
#pragma unroll
    for (int k = 0; k < kMaxRankRegs; ++k) acc[k] = fmaf(pv, lvr[k], acc[k] * sc);
    m = m_new;
  }

  // merge the warps' running states
  float* my = red + warp * (2 + Rv);
  if (lane == 0) { my[0] = m; my[1] = l; }
#pragma unroll
  for (int k = 0; k < kMaxRankRegs; ++k) {
    const int r = lane + 32 * k;
    if (r < Rv) my[2 + r] = acc[k];
  }
  __syncthreads();
  if (warp == 0) {
    float mm = -INFINITY;
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, red[w * (2 + Rv)]);
    float ll = 0.f;
    float wgt[kWarps];
    for (int w = 0; w < kWarps; ++w) {
      const float mw = red[w * (2 + Rv)];
      wgt[w] = mw == -INFINITY ? 0.f : __expf(mw - mm);
      ll += wgt[w] * red[w * (2 + Rv) + 1];
    }
    const int64_t slot = ((int64_t)b * p.n_q_heads + h) * a.n_splits + split;
    for (int r = lane; r < Rv; r += 32) {
      float o = 0.f;
      for (int w = 0; w < kWarps; ++w) o += wgt[w] * red[w * (2 + Rv) + 2 + r];
      a.mid_o[slot * Rv + r] = o / ll;
    }
    if (lane == 0) a.lse[slot] = mm + logf(ll);
  }
}

}  // namespace

cudaError_t launch_stage1_generic(const KArgs& a, cudaStream_t stream) {
  const WsvdLatentDecodeParams& p = a.p;
  const size_t smem = sizeof(float) * ((size_t)p.rank_k * p.head_dim + kWarps * (2 + p.rank_v));
  dim3 grid(a.n_splits, p.n_q_heads, p.batch);
  auto kern = p.latent_dtype == WSVD_I8 ? stage1_generic_kernel<int8_t> : stage1_generic_kernel<__half>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<grid, kThreads, smem, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace wsvd

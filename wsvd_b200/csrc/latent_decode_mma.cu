// Split-KV stage 1 of the latent decode attention for the shapes the tcgen05 kernel does not take:
// f16 or int8 latents, head_dim 16..128, any even rank up to 128, fixed-length splits.  Same
// algebra as the tcgen05 kernel, on warp-level tensor-core instructions (mma.sync m16n8k16) and
// plain or cp.async loads; its only waits are block barriers:
//
//   z_s = sk_s * sum_r Lk[s, r] * W[s, r],   W = [cos(s f_i) | sin(s f_i)] x [P; Q]
//   P[i, r] = c (q[d0] U[d0, r] + q[d1] U[d1, r]),  Q[i, r] = c (q[d1] U[d0, r] - q[d0] U[d1, r])
//
// with (d0, d1) the rotation pair of frequency i, U = wk of the head, c = sm_scale * log2(e).
// This is q . RoPE_s(sk_s * Lk[s] U^T) of the reference kernels
// (efficiency/kernel/flash_latent_per_head_decoding_rope_stage1.py:84-165 for f16 latents,
// efficiency/kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:117-216 for int8), with the
// rotation moved onto the query side: the position-dependent factor is a [tokens x head_dim] table
// tile, and K is never rebuilt.  Per token and head that is D*Rk multiply-adds on the tensor
// cores and Rk + Rv on the CUDA cores, against D*Rk on the CUDA cores in the generic kernel.
//
// One CTA per (split, group of four query heads, sequence), eight warps: warp w serves head
// w & 3 and the 16-token tiles of parity w >> 2.  [P; Q] of the four heads sits in shared memory as
// the B operand ([rank][frequency], rows padded by 16 bytes: conflict-free ldmatrix).  The four
// warps of a parity share each table tile: their 128 threads copy its 16 rows into shared memory
// with 16-byte asynchronous copies, one tile ahead (two buffers, one named barrier per tile), and
// read it as the A operand with ldmatrix.  W stays in the accumulators, where the thread that
// holds W[s, r] multiplies it with Lk[s, r]; the ranks are assigned to accumulator columns so
// that a thread's share of a K row is one contiguous run, fetched with 16-byte loads.  A tile's K
// and V rows are requested a tile ahead, as soon as the registers that receive them are free.
#include "common.cuh"

namespace wsvd {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kHeads = 4;      // query heads per CTA
constexpr int kRowPad = 8;     // halfs of padding per B row
constexpr int kMaxRank = 128;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// [2][rows][h2] f16: plane 0 cos(pos * f_i), plane 1 sin(pos * f_i)
__global__ void mma_table_kernel(__half* table, int rows, int h2, KArgs a) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int pos = idx / h2, i = idx - pos * h2;
  if (pos >= rows) return;
  float sn, cs;
  sincosf((float)pos * a.inv_freq[i], &sn, &cs);
  table[(size_t)pos * h2 + i] = __float2half_rn(cs);
  table[((size_t)rows + pos) * h2 + i] = __float2half_rn(sn);
}

// 16-byte asynchronous copy global -> shared
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
// barrier among the four warps of one tile parity
__device__ __forceinline__ void group_sync(int parity) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(1 + parity), "r"(kHeads * 32) : "memory");
}

// the thread's e-th pair of consecutive latents out of the 32-bit words it loaded
__device__ __forceinline__ float2 pair_at(const uint32_t* words, int e, __half) {
  return __half22float2(*reinterpret_cast<const __half2*>(&words[e]));
}
__device__ __forceinline__ float2 pair_at(const uint32_t* words, int e, int8_t) {
  const uint32_t w = words[e >> 1] >> ((e & 1) * 16);
  return make_float2((float)(int8_t)(w & 0xff), (float)(int8_t)((w >> 8) & 0xff));
}

// NT: 8-wide rank tiles held in the accumulators (8: rank_k <= 64, 16: rank_k <= 128).
// Column n = 8j + 2t + e of W (t = lane & 3) stands for rank 2NT*t + 2j + e: the 2NT ranks a thread
// meets in its accumulators are consecutive in memory, so it fetches them with 16-byte loads.
// KD: head_dim when known at compile time (128), else 0.
template <typename LT, int NT, int KD>
__global__ void __launch_bounds__(kThreads, NT == 8 ? 2 : 1)
stage1_mma_kernel(const __grid_constant__ KArgs a, const __half* __restrict__ table, int table_rows) {
  constexpr int kMine = 2 * NT;                              // consecutive ranks of K per thread and row
  constexpr int kWords = kMine * (int)sizeof(LT) / 4;        // 32-bit words that hold them
  const WsvdLatentDecodeParams& p = a.p;
  const int split = blockIdx.x, hg = blockIdx.y, b = blockIdx.z;
  const int n = p.b_seq_len[b];
  const int lo = split * a.split_len;
  const int hi = min(n, lo + a.split_len);
  if (hi <= lo) return;  // empty split: nothing is written, the merge does not look here

  const int D = KD ? KD : p.head_dim, h2 = D >> 1, Rk = p.rank_k, Rv = p.rank_v;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int hw = warp & 3, parity = warp >> 2;
  const int h = hg * kHeads + hw;
  const bool live = h < p.n_q_heads;
  const int gqa = p.n_q_heads / p.n_kv_heads;
  const int hk = (live ? h : p.n_q_heads - 1) / gqa;
  const bool interleaved = p.rope_layout == WSVD_ROPE_INTERLEAVED;

  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int ldb = D + kRowPad;                                    // halfs per row of B and of a table tile
  __half* Bs = reinterpret_cast<__half*>(smem_raw);               // [kHeads][NT * 8][ldb]
  __half* Ts = Bs + (size_t)kHeads * NT * 8 * ldb;                // [2 parities][2 buffers][16][ldb]
  float* red = reinterpret_cast<float*>(Ts + (size_t)4 * 16 * ldb);  // [kWarps][2 + kMaxRank]

  // ---- [P; Q] of the four heads: column k < h2 of row n is P[k, rank(n)], column h2 + k is Q[k, rank(n)].
  //      A thread keeps one frequency of one head (its two q values are loaded once) and walks the
  //      ranks; neighbouring threads read neighbouring dimensions of U.
  {
    const float qscale = a.sm_scale * 1.4426950408889634f;
    const int sh = 31 - __clz(h2);                       // h2 is a power of two
    const int i = threadIdx.x & (h2 - 1);
    const int hh = (threadIdx.x >> sh) & (kHeads - 1);
    const int r_first = threadIdx.x >> (sh + 2), r_step = kThreads >> (sh + 2);
    const int head = hg * kHeads + hh;
    const bool on_head = head < p.n_q_heads;
    const int hkk = (on_head ? head : 0) / gqa;
    const int d0 = interleaved ? 2 * i : i, d1 = interleaved ? 2 * i + 1 : i + h2;
    float q0 = 0.f, q1 = 0.f, s0 = 1.f, s1 = 1.f;
    if (on_head) {
      const __half* qp = reinterpret_cast<const __half*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)head * p.q_stride_h;
      q0 = __half2float(qp[d0]) * qscale;
      q1 = __half2float(qp[d1]) * qscale;
      if (p.wk_dtype == WSVD_I8) {
        const __half* ws = reinterpret_cast<const __half*>(p.wk_scale) + (int64_t)hkk * D;
        s0 = __half2float(ws[d0]);
        s1 = __half2float(ws[d1]);
      }
    }
    __half* rows = Bs + (size_t)hh * NT * 8 * ldb;
    const bool wk_i8 = p.wk_dtype == WSVD_I8;
    const int64_t col = (int64_t)hkk * D;
    auto rank_of = [](int nrow) { return kMine * ((nrow & 7) >> 1) + 2 * (nrow >> 3) + (nrow & 1); };
    // Eight rows at a time: their loads of U are unconditional (row and rank clamped to valid ones),
    // so all sixteen are in flight together instead of one L2 round trip per row.
    constexpr int kBatch = 8;
    for (int base = r_first; base < NT * 8; base += r_step * kBatch) {
      float u0[kBatch], u1[kBatch];
      if (wk_i8) {
        const int8_t* w = reinterpret_cast<const int8_t*>(p.wk) + col;
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
          const int64_t off = (int64_t)min(rank_of(min(base + k * r_step, NT * 8 - 1)), Rk - 1) * p.wk_stride_r;
          u0[k] = (float)w[off + d0] * s0;
          u1[k] = (float)w[off + d1] * s1;
        }
      } else {
        const __half* w = reinterpret_cast<const __half*>(p.wk) + col;
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
          const int64_t off = (int64_t)min(rank_of(min(base + k * r_step, NT * 8 - 1)), Rk - 1) * p.wk_stride_r;
          u0[k] = __half2float(w[off + d0]);
          u1[k] = __half2float(w[off + d1]);
        }
      }
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        const int nrow = base + k * r_step;
        if (nrow < NT * 8) {
          const bool on = on_head && rank_of(nrow) < Rk;
          rows[nrow * ldb + i] = __float2half_rn(on ? q0 * u0[k] + q1 * u1[k] : 0.f);
          rows[nrow * ldb + h2 + i] = __float2half_rn(on ? q1 * u0[k] - q0 * u1[k] : 0.f);
        }
      }
    }
  }

  const int32_t* page = p.req_to_token + (int64_t)p.b_req_idx[b] * p.rtt_stride;
  const int pos0 = p.pos_offset ? p.pos_offset[b] : 0;
  const LT* lk_base = reinterpret_cast<const LT*>(p.latent_k) + (int64_t)hk * p.k_stride_h;
  const LT* lv_base = reinterpret_cast<const LT*>(p.latent_v) + (int64_t)hk * p.v_stride_h;
  const __half* ks_base = reinterpret_cast<const __half*>(p.k_scale);
  const __half* vs_base = reinterpret_cast<const __half*>(p.v_scale);
  const int k_st = (int)p.k_stride_t, v_st = (int)p.v_stride_t;  // below 2^31 (checked by the host); offsets are 64-bit
  const bool wide_v = Rv > 64;
  // this thread's ranks of K: [kMine * t, kMine * (t + 1)); whole 16-byte loads when they all exist and
  // every row starts on a 16-byte boundary, pair loads otherwise
  const int rk_first = kMine * t;
  const bool k_all = rk_first + kMine <= Rk && (reinterpret_cast<uintptr_t>(p.latent_k) & 15) == 0 &&
                     (p.k_stride_t * (int64_t)sizeof(LT)) % 16 == 0 && (p.k_stride_h * (int64_t)sizeof(LT)) % 16 == 0;

  // shared-memory addresses for ldmatrix.x4.
  // B: lanes 0-7 rank tile j / columns k0.., 8-15 tile j / k0+8.., 16-23 tile j+1 / k0.., 24-31 tile j+1 / k0+8..
  const uint32_t b_lane = (uint32_t)__cvta_generic_to_shared(Bs + (size_t)hw * NT * 8 * ldb) +
                          (uint32_t)((((lane >> 4) * 8 + (lane & 7)) * ldb + ((lane >> 3) & 1) * 8) * sizeof(__half));
  // A (a table tile): lanes 0-7 rows 0-7 / k0.., 8-15 rows 8-15 / k0.., 16-23 rows 0-7 / k0+8.., 24-31 rows 8-15 / k0+8..
  const uint32_t t_group = (uint32_t)__cvta_generic_to_shared(Ts + (size_t)parity * 2 * 16 * ldb);
  const uint32_t t_lane = (uint32_t)(((((lane >> 3) & 1) * 8 + (lane & 7)) * ldb + (lane >> 4) * 8) * sizeof(__half));
  const uint32_t t_buf_bytes = (uint32_t)(16 * ldb * sizeof(__half));

  // the group's 128 threads copy a tile's 16 table rows (cos half, sin half) in 16-byte pieces:
  // 16 * D/8 pieces, at most two per thread, the same (row, column) in every tile
  const int gtid = threadIdx.x & 127;
  int pc_row[2];
  uint32_t pc_dst[2];
  int64_t pc_src[2];  // offset within a table row's plane, in halfs; the row is added per tile
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int c = gtid + 128 * u;
    const int sh = 31 - __clz(D / 8);
    const int row = c >> sh, pc = c & (D / 8 - 1);
    const bool is_sin = pc >= D / 16;
    pc_row[u] = row < 16 ? row : -1;
    pc_dst[u] = (uint32_t)((row * ldb + pc * 8) * sizeof(__half));
    pc_src[u] = (is_sin ? (int64_t)table_rows * h2 : 0) + (is_sin ? pc - D / 16 : pc) * 8;
  }
  auto request_table_tile = [&](int s_base, int buf) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (pc_row[u] >= 0) {
        const int pos = min(pos0 + min(s_base + pc_row[u], hi - 1), table_rows - 1);
        cp_async_16(t_group + buf * t_buf_bytes + pc_dst[u], table + pc_src[u] + (int64_t)pos * h2);
      }
    }
  };

  float m_run = -INFINITY, l_run = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};  // ranks 2*lane, 2*lane+1, 64 + 2*lane, 64 + 2*lane + 1
  const int rv0 = 2 * lane, rv1 = 64 + 2 * lane;

  request_table_tile(lo + parity * 16, 0);
  __syncthreads();  // [P; Q] complete

  // A tile's K rows (with their scales) and V rows live in registers from the moment the tile before
  // it has consumed its own: K is requested right after the previous tile's scores, V right after its
  // P.V, so their latency runs under the rest of that tile and the MMAs of this one.
  uint32_t kw0[kWords], kw1[kWords];
  uint32_t vw[16], vx[16];  // the tile's 16 V rows: this lane's pair of ranks (and the pair 64 further)
  float sk0 = 1.f, sk1 = 1.f, sv0 = 1.f, sv1 = 1.f;
  auto load_k = [&](int ta, int tb) {
    const LT* lk0 = lk_base + (int64_t)ta * k_st + rk_first;
    const LT* lk1 = lk_base + (int64_t)tb * k_st + rk_first;
    if (k_all) {
#pragma unroll
      for (int v = 0; v < kWords / 4; ++v) {
        *reinterpret_cast<uint4*>(&kw0[4 * v]) = __ldg(reinterpret_cast<const uint4*>(lk0) + v);
        *reinterpret_cast<uint4*>(&kw1[4 * v]) = __ldg(reinterpret_cast<const uint4*>(lk1) + v);
      }
    } else if (sizeof(LT) == 2) {
#pragma unroll
      for (int e = 0; e < kWords; ++e) {
        const bool on = rk_first + 2 * e < Rk;  // rank_k is even: a pair never straddles the end
        kw0[e] = on ? *reinterpret_cast<const uint32_t*>(lk0 + 2 * e) : 0u;
        kw1[e] = on ? *reinterpret_cast<const uint32_t*>(lk1 + 2 * e) : 0u;
      }
    } else {
#pragma unroll
      for (int e = 0; e < kWords; ++e) {
        const bool on_a = rk_first + 4 * e < Rk, on_b = rk_first + 4 * e + 2 < Rk;
        const uint32_t a0 = on_a ? *reinterpret_cast<const uint16_t*>(lk0 + 4 * e) : 0u;
        const uint32_t b0 = on_b ? *reinterpret_cast<const uint16_t*>(lk0 + 4 * e + 2) : 0u;
        const uint32_t a1 = on_a ? *reinterpret_cast<const uint16_t*>(lk1 + 4 * e) : 0u;
        const uint32_t b1 = on_b ? *reinterpret_cast<const uint16_t*>(lk1 + 4 * e + 2) : 0u;
        kw0[e] = a0 | (b0 << 16);
        kw1[e] = a1 | (b1 << 16);
      }
    }
    if (ks_base) {
      sk0 = __half2float(ks_base[(int64_t)ta * p.ks_stride_t + (int64_t)hk * p.ks_stride_h]);
      sk1 = __half2float(ks_base[(int64_t)tb * p.ks_stride_t + (int64_t)hk * p.ks_stride_h]);
    }
  };
  auto load_v = [&](int ta, int tb) {
    if (vs_base) {
      sv0 = __half2float(vs_base[(int64_t)ta * p.vs_stride_t + (int64_t)hk * p.vs_stride_h]);
      sv1 = __half2float(vs_base[(int64_t)tb * p.vs_stride_t + (int64_t)hk * p.vs_stride_h]);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int tt = __shfl_sync(0xffffffffu, i < 8 ? ta : tb, (i & 7) * 4);
      const LT* lv = lv_base + (int64_t)tt * v_st;
      vx[i] = 0u;
      if (sizeof(LT) == 2) {
        vw[i] = rv0 < Rv ? *reinterpret_cast<const uint32_t*>(lv + rv0) : 0u;
        if (wide_v) vx[i] = rv1 < Rv ? *reinterpret_cast<const uint32_t*>(lv + rv1) : 0u;
      } else {
        vw[i] = rv0 < Rv ? *reinterpret_cast<const uint16_t*>(lv + rv0) : 0u;
        if (wide_v) vx[i] = rv1 < Rv ? *reinterpret_cast<const uint16_t*>(lv + rv1) : 0u;
      }
    }
  };

  // token slots of this thread's two rows, fetched two tiles ahead (rows past the end take the last
  // valid token): the slots of the next tile are in registers when this tile asks for its K and V
  int t0_next = 0, t1_next = 0, t0_after = 0, t1_after = 0;
  if (live && lo + parity * 16 < hi) {
    t0_next = page[min(lo + parity * 16 + g, hi - 1)];
    t1_next = page[min(lo + parity * 16 + g + 8, hi - 1)];
    t0_after = page[min(lo + parity * 16 + g + 32, hi - 1)];
    t1_after = page[min(lo + parity * 16 + g + 40, hi - 1)];
    load_k(t0_next, t1_next);
    load_v(t0_next, t1_next);
  }

  int it = 0;
  for (int s_base = lo + parity * 16; s_base < hi; s_base += 32, ++it) {
    // this thread's two rows of the tile; rows past the end count as -inf
    const int s0 = s_base + g, s1 = s0 + 8;
    const bool ok0 = s0 < hi, ok1 = s1 < hi;
    const bool more = s_base + 32 < hi;  // this warp has another tile after this one
    t0_next = t0_after;                  // now the next tile's slots
    t1_next = t1_after;
    if (live && more) {
      t0_after = page[min(s0 + 64, hi - 1)];
      t1_after = page[min(s1 + 64, hi - 1)];
    }

    // the tile's table rows have landed (own copies, then everybody's); every warp of the group is
    // also past the previous tile, so its buffer can take the next one
    cp_async_wait_all();
    group_sync(parity);
    if (more) request_table_tile(s_base + 32, (it + 1) & 1);
    if (!live) continue;

    // W tile: 16 tokens x NT*8 ranks
    float w[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) w[j][0] = w[j][1] = w[j][2] = w[j][3] = 0.f;
    const uint32_t t_addr = t_group + (it & 1) * t_buf_bytes + t_lane;
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16) {
      uint32_t af[4];
      ldmatrix_x4(af, t_addr + (uint32_t)(k0 * sizeof(__half)));
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t bf[4];
        ldmatrix_x4(bf, b_lane + (uint32_t)((j * 8 * ldb + k0) * sizeof(__half)));
        mma_16816(w[j], af, bf[0], bf[1]);
        mma_16816(w[j + 1], af, bf[2], bf[3]);
      }
    }

    // scores (log2 domain): W[s, 2NT*t + 2j + e] sits in w[j][e] (row g) and w[j][2 + e] (row g + 8)
    float z0 = 0.f, z1 = 0.f;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const float2 x0 = pair_at(kw0, j, LT()), x1 = pair_at(kw1, j, LT());
      z0 = fmaf(x0.x, w[j][0], z0);
      z0 = fmaf(x0.y, w[j][1], z0);
      z1 = fmaf(x1.x, w[j][2], z1);
      z1 = fmaf(x1.y, w[j][3], z1);
    }
    z0 += __shfl_xor_sync(0xffffffffu, z0, 1);
    z0 += __shfl_xor_sync(0xffffffffu, z0, 2);
    z1 += __shfl_xor_sync(0xffffffffu, z1, 1);
    z1 += __shfl_xor_sync(0xffffffffu, z1, 2);
    z0 = ok0 ? z0 * sk0 : -INFINITY;
    z1 = ok1 ? z1 * sk1 : -INFINITY;
    if (more) load_k(t0_next, t1_next);  // this tile's K is consumed

    // online softmax over the tile (row s_base is always valid, so the maximum is finite)
    float tmax = fmaxf(z0, z1);
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
    const float m_new = fmaxf(m_run, tmax);
    const float sc = exp2f(m_run - m_new);  // 0 on the first tile
    const float e0 = exp2f(z0 - m_new), e1 = exp2f(z1 - m_new);
    float es = e0 + e1;
    es += __shfl_xor_sync(0xffffffffu, es, 4);
    es += __shfl_xor_sync(0xffffffffu, es, 8);
    es += __shfl_xor_sync(0xffffffffu, es, 16);
    l_run = fmaf(l_run, sc, es);
    m_run = m_new;
    const float pw0 = e0 * sv0, pw1 = e1 * sv1;

    // acc[r] = acc[r] * sc + sum_s p_s sv_s Lv[s, r]
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] *= sc;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float pw = __shfl_sync(0xffffffffu, i < 8 ? pw0 : pw1, (i & 7) * 4);
      const float2 va = pair_at(&vw[i], 0, LT());
      acc[0] = fmaf(pw, va.x, acc[0]);
      acc[1] = fmaf(pw, va.y, acc[1]);
      if (wide_v) {
        const float2 vb = pair_at(&vx[i], 0, LT());
        acc[2] = fmaf(pw, vb.x, acc[2]);
        acc[3] = fmaf(pw, vb.y, acc[3]);
      }
    }
    if (more) load_v(t0_next, t1_next);  // this tile's V is consumed
  }

  cp_async_wait_all();  // a group without tiles still has its first request in flight

  // ---- merge the two warps of a head, normalise, write the partial
  float* my = red + warp * (2 + kMaxRank);
  if (lane == 0) {
    my[0] = m_run;
    my[1] = l_run;
  }
  if (rv0 < Rv) {
    my[2 + rv0] = acc[0];
    my[3 + rv0] = acc[1];
  }
  if (rv1 < Rv) {
    my[2 + rv1] = acc[2];
    my[3 + rv1] = acc[3];
  }
  __syncthreads();
  if (parity == 0 && live) {
    const float* other = red + (warp + 4) * (2 + kMaxRank);
    const float ma = my[0], mb = other[0];
    const float mm = fmaxf(ma, mb);  // warps 0..3 always had the split's first tile: finite
    const float wa = exp2f(ma - mm), wb = mb == -INFINITY ? 0.f : exp2f(mb - mm);
    const float ll = wa * my[1] + wb * other[1];
    const int64_t slot = ((int64_t)b * p.n_q_heads + h) * a.n_splits + split;
    for (int r = lane; r < Rv; r += 32) a.mid_o[slot * Rv + r] = (wa * my[2 + r] + wb * other[2 + r]) / ll;
    if (lane == 0) a.lse[slot] = (mm + log2f(ll)) * kLn2;
  }
}

size_t smem_bytes(int head_dim, int nt) {
  return ((size_t)kHeads * nt * 8 + 4 * 16) * (head_dim + kRowPad) * sizeof(__half) +
         (size_t)kWarps * (2 + kMaxRank) * sizeof(float);
}

template <typename LT, int NT>
cudaError_t launch(const KArgs& a, const __half* table, int rows, cudaStream_t stream) {
  const WsvdLatentDecodeParams& p = a.p;
  const size_t smem = smem_bytes(p.head_dim, NT);
  auto kern = p.head_dim == 128 ? stage1_mma_kernel<LT, NT, 128> : stage1_mma_kernel<LT, NT, 0>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(a.n_splits, (p.n_q_heads + kHeads - 1) / kHeads, p.batch);
  kern<<<grid, kThreads, smem, stream>>>(a, table, rows);
  return cudaGetLastError();
}

}  // namespace

size_t mma_table_bytes(int rows, int head_dim) { return (size_t)rows * head_dim * sizeof(__half); }

cudaError_t launch_mma_table(void* table, int rows, const KArgs& a, cudaStream_t stream) {
  const int h2 = a.p.head_dim / 2;
  const long total = (long)rows * h2;
  if (total == 0) return cudaSuccess;
  mma_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(reinterpret_cast<__half*>(table), rows, h2, a);
  return cudaGetLastError();
}

cudaError_t launch_stage1_mma(const KArgs& a, const void* table, int rows, cudaStream_t stream) {
  const __half* tb = reinterpret_cast<const __half*>(table);
  const bool i8 = a.p.latent_dtype == WSVD_I8;
  if (a.p.rank_k <= 64) return i8 ? launch<int8_t, 8>(a, tb, rows, stream) : launch<__half, 8>(a, tb, rows, stream);
  return i8 ? launch<int8_t, 16>(a, tb, rows, stream) : launch<__half, 16>(a, tb, rows, stream);
}

}  // namespace wsvd

// Split-KV stage 1 of the latent decode attention on the Blackwell tensor cores
// (tcgen05.mma with the accumulator in tensor memory), for head_dim 128, rank_k 64,
// rank_v in {16,32,48,64}, int8 latents.
//
// Formulation.  For one head, query q and position s the score is
//   z_s = c * sk_s * sum_r Lk[s,r] * W[s,r],
//   W[s,r] = sum_i cos(s f_i) P[r,i] + sin(s f_i) Q[r,i],
//   P[r,i] = q_i U[i,r] + q_{i+64} U[i+64,r],   Q[r,i] = q_{i+64} U[i,r] - q_i U[i+64,r]
// which is the reference's reconstruct -> RoPE -> q.K' chain
// (efficiency/kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:149-169) with
// the sums reordered: the rotation is moved from K onto the query side.  W is one GEMM
//   [128 positions x 128 (cos|sin)] x [128 x 64*G ranks]
// per tile of 128 positions and group of G <= 4 heads: the A operand is a tile of a
// position table of cos/sin values (f16, shared by every head and sequence, read from
// L2), the B operand [P;Q] is built once per CTA and stays in shared memory.  The int8
// latents never pass through the tensor core: each epilogue thread owns one token,
// reads its row of W from tensor memory and dots it with the token's int8 K row (from
// shared memory) in fp32.  P.V runs on the CUDA cores in fp32 from the int8 V rows.
// Nothing is rounded to f16 except the two GEMM operands.
//
// CTA = one (split, group of 4 heads, sequence); 20 warps:
//   warps 0-15   epilogue, 4 per head: warp w owns tensor-memory lanes 32*(w%4)..+31.  A warp
//                copies its 32 K rows and its V rows from the ring slot to registers as soon as
//                they have landed and hands the slot back before any arithmetic.
//   warp 16      one thread issues the table tile loads (cp.async.bulk) and the MMAs
//   warps 17-19  request the K and V rows: every head has a ring of three 8 KB slots of half a
//                tile (64 tokens), producer warp p owns slot p of every head; two TMA tensor
//                copies per slot when the half-tile's token slots are consecutive (lane g
//                serves head g on its own), else a gather of rows with 16-byte cp.async
//                through the page table.
// More than 16 warps cap the kernel at 96 registers per thread; the four non-epilogue warps
// fill exactly one warp slot per scheduler.
// Every wait on an mbarrier is bounded; on a time-out the kernel records a status code
// and every role falls through to the common exit, which frees the tensor memory.
#include <cuda.h>
#include <string.h>

#include "common.cuh"

namespace wsvd {
namespace tc {

constexpr int kG = 4;          // heads per CTA
constexpr int kTile = 128;     // positions per MMA tile (= tensor-memory lanes)
constexpr int kRk = 64;
constexpr int kEpiWarps = 4 * kG;
constexpr int kMmaWarp = kEpiWarps;
constexpr int kProducers = 3;   // copy-issuing warps; with the MMA warp they fill one warp slot per scheduler
constexpr int kThreads = (kEpiWarps + 1 + kProducers) * 32;
// Latent ring: every head owns kSlots slots, each holding half a tile (64 tokens): K rows
// at a 64-byte pitch followed by V rows at a rank_v pitch.  A slot is only ever reused by
// the same head, whose warps consume their slots in order; with slots shared between heads
// a warp could get two phases ahead of a slot's mbarrier, which a parity wait cannot see.
constexpr int kHalf = kTile / 2;
constexpr int kSlots = 3;
constexpr int kStages = kG * kSlots;
static_assert(kProducers == kSlots, "producer warp p owns ring slot p of every head");
constexpr uint32_t kKBytes = kHalf * 64;            // K rows of one half-tile
constexpr uint32_t kUnitBytes = 2 * kKBytes;        // + V rows
constexpr uint32_t kAHalfBytes = kTile * 128;       // 128 rows x 64 f16
constexpr uint32_t kABufBytes = 2 * kAHalfBytes;    // cos half + sin half
constexpr uint32_t kBHalfBytes = kG * kRk * 128;    // 256 rows x 64 f16
constexpr uint32_t kTmemCols = 512;                 // 2 buffers x (kG*kRk) fp32 columns

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffB = 0;
constexpr uint32_t kOffA = kOffB + 2 * kBHalfBytes;
constexpr uint32_t kOffRing = kOffA + 2 * kABufBytes;
constexpr uint32_t kOffMerge = kOffB;  // end-of-CTA merge scratch reuses the B operand (all MMAs are done by then)
constexpr uint32_t kMergeFloats = kG * 4 * (2 + 64);
constexpr uint32_t kOffQ = kOffRing + kStages * kUnitBytes;
constexpr uint32_t kOffBar = kOffQ + kG * 128 * 4;
constexpr int kNumBars = 2 * kStages + 2 + 2 + 2 + 2 + 1;
constexpr uint32_t kOffTmemSlot = kOffBar + kNumBars * 8;
constexpr uint32_t kOffIssued = kOffTmemSlot + 16;   // per ring slot: number of units requested so far
constexpr uint32_t kSmemBytes = kOffIssued + kStages * 4;  // the dynamic shared-memory base is 1024-byte aligned

enum Status : unsigned int { kOk = 0, kTimeoutProducer = 1, kTimeoutMma = 2, kTimeoutEpilogue = 3, kBadSmemAlignment = 4 };

__device__ unsigned int g_status = 0;

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// try_wait with a suspend-time hint: the waiting thread is parked by the hardware until
// the phase completes or the hint (ns) expires, instead of spinning on issue slots that
// the producer and MMA warps need.
constexpr uint32_t kWaitHintNs = 20000;
__device__ __forceinline__ uint32_t mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kWaitHintNs)
      : "memory");
  return ok;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after about two seconds and reports false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    if (global_ns() - t0 > 2000000000ull) return false;
  }
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// warp-wide maximum in one instruction (sm_100a)
__device__ __forceinline__ float warp_max_redux(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// packed fp32 pairs (sm_100)
__device__ __forceinline__ uint64_t pk(float x, float y) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
  return r;
}
__device__ __forceinline__ void upk(uint64_t v, float& x, float& y) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
// Four int8 packed in `w` (already XORed with 0x80808080) -> two fp32 pairs holding the
// exact signed values: byte -> low mantissa of 2^23, then subtract 2^23 + 128.
__device__ __forceinline__ void cvt4(uint32_t w, uint64_t& lo, uint64_t& hi) {
  const uint32_t magic = 0x4B000000u;
  const uint64_t bias = pk(-8388736.f, -8388736.f);
  lo = add2(pk(__uint_as_float(__byte_perm(w, magic, 0x7650)), __uint_as_float(__byte_perm(w, magic, 0x7651))), bias);
  hi = add2(pk(__uint_as_float(__byte_perm(w, magic, 0x7652)), __uint_as_float(__byte_perm(w, magic, 0x7653))), bias);
}

// UMMA shared-memory descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                       // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}
// UMMA instruction descriptor: f16 x f16 -> f32, both operands K-major, M x N.
__device__ __forceinline__ uint32_t instr_desc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct TcArgs {
  KArgs k;
  const uint8_t* table;   // [2][rows][128 B] cos | sin halves, f16, 16-byte chunks XOR-swizzled by row%8
  int32_t table_rows;
  // TMA descriptors of the K and V latent tensors as 3-D byte tensors (rank, and the
  // token-slot and head axes ordered by stride).  K rows land with the 64-byte swizzle,
  // which is the XOR pattern the score loop reads with; V rows land dense.
  int32_t use_tma;        // 0: rows are gathered with cp.async
  int32_t slot_axis;      // 1 or 2: which tensor-map coordinate is the token slot
  alignas(64) CUtensorMap tmap_k;
  alignas(64) CUtensorMap tmap_v;
};

// ------------------------------------------------------------------ position table
__global__ void rope_table_kernel(uint8_t* table, int rows, KArgs a) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int pos = idx >> 6, i = idx & 63;
  if (pos >= rows) return;
  float sn, cs;
  sincosf((float)pos * a.inv_freq[i], &sn, &cs);
  const size_t off = (size_t)pos * 128 + ((((i >> 3) ^ (pos & 7)) << 4) + ((i & 7) << 1));
  *reinterpret_cast<__half*>(table + off) = __float2half_rn(cs);
  *reinterpret_cast<__half*>(table + (size_t)rows * 128 + off) = __float2half_rn(sn);
}

// ------------------------------------------------------------------ stage 1
__global__ void __launch_bounds__(kThreads, 1) stage1_tc_kernel(const __grid_constant__ TcArgs ta) {
  const KArgs& a = ta.k;
  const WsvdLatentDecodeParams& p = a.p;
  const int split = blockIdx.x, hg = blockIdx.y, b = blockIdx.z;
  const int n = p.b_seq_len[b];
  const int lo = split * a.split_len;
  const int hi = min(n, lo + a.split_len);
  if (hi <= lo) return;  // empty split writes nothing
  const int h0 = hg * kG;
  const int G = min(kG, p.n_q_heads - h0);
  const int ntiles = (hi - lo + kTile - 1) / kTile;
  const int gqa = p.n_q_heads / p.n_kv_heads;
  const int Rv = p.rank_v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t sbase = smem_u32(smem_raw);
  uint8_t* sm = smem_raw;
  if ((sbase & 1023u) != 0) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicMax(&g_status, (unsigned)kBadSmemAlignment);
    return;
  }
  const uint32_t sB = sbase + kOffB, sA = sbase + kOffA, sRing = sbase + kOffRing;
  float* merge = reinterpret_cast<float*>(sm + kOffMerge);
  float* qs = reinterpret_cast<float*>(sm + kOffQ);
  const uint32_t bars = sbase + kOffBar;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_empty = [&](int s) { return bars + 8u * (kStages + s); };
  auto bar_a_full = [&](int i) { return bars + 8u * (2 * kStages + i); };
  auto bar_a_empty = [&](int i) { return bars + 8u * (2 * kStages + 2 + i); };
  auto bar_w_full = [&](int i) { return bars + 8u * (2 * kStages + 4 + i); };
  auto bar_w_empty = [&](int i) { return bars + 8u * (2 * kStages + 6 + i); };
  const uint32_t bar_pq = bars + 8u * (2 * kStages + 8);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + kOffTmemSlot);

  const int32_t* page = p.req_to_token + (int64_t)p.b_req_idx[b] * p.rtt_stride;

  // 16-byte vector loads of wk need f16 data with 16-byte aligned rows
  const bool wk_vec = p.wk_dtype == WSVD_F16 && (p.wk_stride_r & 7) == 0 &&
                      (reinterpret_cast<uintptr_t>(p.wk) & 15) == 0;
  uint4 wpre[8];
  // requested during set-up so that their latency is hidden behind it: the epilogue
  // lanes' first two page entries and first scales, the producers' first page entries
  int slot0 = -1, slot_n = -1, pe0 = -1, pe1 = -1, pfirst = 0;
  unsigned short sk_raw = 0, sv_raw = 0;

  // ---- set-up: barriers + tensor memory (MMA warp), scaled q to shared memory (epilogue warps)
  if (warp == kMmaWarp) {
    // one lane per barrier: lanes 0..11 the ring's full/empty pairs, lanes 12..15 the pairs of
    // the table and W buffers, lane 16 the [P;Q] barrier
    if (lane < kStages) {
      mbar_init(bar_full(lane), 32);   // one arrive per lane of the warp that issues the copy
      mbar_init(bar_empty(lane), 2);   // the two epilogue warps that own the half-tile's tokens
      reinterpret_cast<volatile int*>(sm + kOffIssued)[lane] = 0;
    } else if (lane < kStages + 2) {
      mbar_init(bar_a_full(lane - kStages), 1);
      mbar_init(bar_a_empty(lane - kStages), 1);
    } else if (lane < kStages + 4) {
      mbar_init(bar_w_full(lane - kStages - 2), 1);
      mbar_init(bar_w_empty(lane - kStages - 2), 4 * G);
    } else if (lane == kStages + 4) {
      mbar_init(bar_pq, 4 * G);
    }
    fence_barrier_init();
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  } else if (warp > kMmaWarp) {
    if (ta.use_tma && lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&ta.tmap_k)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&ta.tmap_v)) : "memory");
    }
    // page entries of this producer's first unit (same indexing as fetch_entries below)
    const int n = warp - kMmaWarp - 1;
    if (n < 2 * ntiles) {
      const int s0t = lo + (n >> 1) * kTile, sa = s0t + (n & 1) * kHalf + 2 * lane;
      if (sa < hi) pe0 = page[sa];
      if (sa + 1 < hi) pe1 = page[sa + 1];
      pfirst = page[s0t];
    }
  } else if (warp < 4 * G) {
    {
      const int s_first = lo + (warp & 3) * 32 + lane;
      if (s_first < hi) slot0 = page[s_first];
      if (s_first + kTile < hi) slot_n = page[s_first + kTile];
    }
    // the head's slice of wk for the [P;Q] build: requested now, used after the barrier
    if (wk_vec) {
      const int hk_pre = (h0 + (warp >> 2)) / gqa;
      const bool il = p.rope_layout == WSVD_ROPE_INTERLEAVED;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int task = (threadIdx.x & 127) + 128 * i, r = task >> 3, ic = task & 7;
        const __half* w = reinterpret_cast<const __half*>(p.wk) + (int64_t)r * p.wk_stride_r + (int64_t)hk_pre * 128;
        wpre[2 * i] = *reinterpret_cast<const uint4*>(w + (il ? ic * 16 : ic * 8));
        wpre[2 * i + 1] = *reinterpret_cast<const uint4*>(w + (il ? ic * 16 + 8 : 64 + ic * 8));
      }
    }
    // q * sm_scale * log2(e): scores come out in the log2 domain
    const float qscale = a.sm_scale * 1.4426950408889634f;
    for (int idx = threadIdx.x; idx < G * 128; idx += 128 * G) {
      const int g = idx >> 7, d = idx & 127;
      const __half* qp = reinterpret_cast<const __half*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)(h0 + g) * p.q_stride_h;
      qs[idx] = __half2float(qp[d]) * qscale;
    }
    if (slot0 >= 0) {
      const int hk_pre = (h0 + (warp >> 2)) / gqa;
      sk_raw = reinterpret_cast<const unsigned short*>(p.k_scale)[(int64_t)hk_pre * p.ks_stride_h + (int64_t)slot0 * p.ks_stride_t];
      sv_raw = reinterpret_cast<const unsigned short*>(p.v_scale)[(int64_t)hk_pre * p.vs_stride_h + (int64_t)slot0 * p.vs_stride_t];
    }
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == kMmaWarp) {
    // ================================================================= table loads + MMA issue
    if (lane == 0) {
      const uint32_t idesc = instr_desc_f16(kTile, kRk * G);
      auto issue_table = [&](int t) {
        const int buf = t & 1;
        const size_t row = (size_t)(lo + t * kTile);
        mbar_expect_tx(bar_a_full(buf), kABufBytes);
        bulk_g2s(sA + buf * kABufBytes, ta.table + row * 128, kAHalfBytes, bar_a_full(buf));
        bulk_g2s(sA + buf * kABufBytes + kAHalfBytes, ta.table + ((size_t)ta.table_rows + row) * 128, kAHalfBytes,
                 bar_a_full(buf));
      };
      issue_table(0);
      if (ntiles > 1) issue_table(1);
      // descriptors: only the start-address field changes between k-steps and buffers
      const uint64_t adesc0 = smem_desc_sw128(sA), bdesc0 = smem_desc_sw128(sB);
      bool ok = mbar_wait(bar_pq, 0);
      for (int t = 0; t < ntiles && ok; ++t) {
        const int buf = t & 1;
        // The table tile of t+1 goes into the buffer MMA(t-1) read; that MMA was issued a
        // whole iteration ago, so this wait is short and the load overlaps MMA(t).
        if (t >= 1 && t + 1 < ntiles) {
          ok = mbar_wait(bar_a_empty((t + 1) & 1), ((t - 1) >> 1) & 1);
          if (!ok) break;
          issue_table(t + 1);
        }
        ok = mbar_wait(bar_a_full(buf), (t >> 1) & 1);
        if (ok && t >= 2) ok = mbar_wait(bar_w_empty(buf), ((t >> 1) - 1) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem + buf * (kG * kRk);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t koff = (kk & 3) * 32;
          const uint64_t ad = adesc0 + ((buf * kABufBytes + (kk >> 2) * kAHalfBytes + koff) >> 4);
          const uint64_t bd = bdesc0 + (((kk >> 2) * kBHalfBytes + koff) >> 4);
          umma_f16(d_tmem, ad, bd, idesc, kk > 0);
        }
        umma_commit(bar_w_full(buf));
        umma_commit(bar_a_empty(buf));
      }
      if (!ok) atomicMax(&g_status, (unsigned)kTimeoutMma);
    }
    __syncwarp();
  } else if (warp > kMmaWarp) {
    // ================================================================= latent copies
    // Every head's half-tiles (units n = 2*tile + half) cycle through its kSlots ring slots.
    // Producer warp pw owns ring slot pw of every head, i.e. the units n = pw (mod kSlots).
    // Unit n of a head is requested as soon as the pair of epilogue warps that consumed unit
    // n - kSlots has handed the slot back.  On the TMA path lane g serves head g on its own:
    // it waits for that head's slot and issues the two copies, so the heads do not queue
    // behind one another.
    const int pw = warp - kMmaWarp - 1;
    const uint32_t unit_tx = kKBytes + kHalf * Rv;
    const int n_units = 2 * ntiles;
    // page entries of the unit's 64 rows (two per lane) and of its tile's first row
    auto fetch_entries = [&](int n, int& e0, int& e1, int& first) {
      const int s0t = lo + (n >> 1) * kTile, sa = s0t + (n & 1) * kHalf + 2 * lane;
      e0 = -1;
      e1 = -1;
      if (sa < hi) e0 = page[sa];
      if (sa + 1 < hi) e1 = page[sa + 1];
      first = page[s0t];
    };
    // Publishing "unit `use` of this slot has been requested": a consumer waits for this
    // before it waits on the slot's mbarrier.  The request is made only after the slot's
    // previous unit was consumed, so from then on the parity wait cannot be a phase ahead
    // or behind.
    auto publish = [&](int stage, int use) {
      asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(sbase + kOffIssued + 4u * stage), "r"(use + 1) : "memory");
    };
    int e0 = pe0, e1 = pe1, first = pfirst;  // unit pw's entries were requested during set-up
    bool ok = true;
    int use = 0;
    for (int n = pw; n < n_units && ok; n += kSlots, ++use) {
      int f0 = -1, f1 = -1, ffirst = 0;
      if (n + kSlots < n_units) fetch_entries(n + kSlots, f0, f1, ffirst);  // the next unit's, one unit ahead
      const int sl0 = first + (n & 1) * kHalf;  // slot of the unit's first row if the tile is affine
      const bool affine = (e0 < 0 || e0 == sl0 + 2 * lane) && (e1 < 0 || e1 == sl0 + 2 * lane + 1);
      if (ta.use_tma && __all_sync(0xffffffffu, affine)) {
        // two TMA copies of 64 consecutive token slots per head
        if (lane < G) {
          const int stage = lane * kSlots + pw, hk = (h0 + lane) / gqa;
          if (use > 0) ok = mbar_wait(bar_empty(stage), (use - 1) & 1);
          if (ok) {
            const int c1 = ta.slot_axis == 1 ? sl0 : hk, c2 = ta.slot_axis == 1 ? hk : sl0;
            mbar_expect_tx(bar_full(stage), unit_tx);
            tma_load_3d(sRing + stage * kUnitBytes, &ta.tmap_k, 0, c1, c2, bar_full(stage));
            tma_load_3d(sRing + stage * kUnitBytes + kKBytes, &ta.tmap_v, 0, c1, c2, bar_full(stage));
            mbar_arrive_n(bar_full(stage), 31);  // the arrivals the gather path makes lane by lane
            publish(stage, use);
          }
        }
        ok = __all_sync(0xffffffffu, ok);
      } else {
        // Gather through the page table, head after head: lane (r0 = lane/4, c = lane%4)
        // copies 16-byte chunk c of rows r0 + 8k.  K chunks are XOR-swizzled with (row/2)%4
        // exactly as the TMA 64-byte swizzle places them; (row/2)%4 does not depend on k.
        const int c = lane & 3, r0 = lane >> 2;
        const uint32_t doff_k = r0 * 64 + ((c ^ ((r0 >> 1) & 3)) << 4);
        const uint32_t doff_v = kKBytes + r0 * Rv + c * 16;
        const bool v_on = c < (Rv >> 4);
        const int s0 = lo + (n >> 1) * kTile + (n & 1) * kHalf + r0;
        for (int g = 0; g < G; ++g) {
          const int stage = g * kSlots + pw, hk = (h0 + g) / gqa;
          if (use > 0) ok = mbar_wait(bar_empty(stage), (use - 1) & 1);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const uint8_t* kbase = reinterpret_cast<const uint8_t*>(p.latent_k) + (int64_t)hk * p.k_stride_h;
          const uint8_t* vbase_g = reinterpret_cast<const uint8_t*>(p.latent_v) + (int64_t)hk * p.v_stride_h;
          const uint32_t dst = sRing + stage * kUnitBytes;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const bool valid = s0 + 8 * k < hi;  // rows past the end are zero-filled
            const int64_t sl = valid ? page[s0 + 8 * k] : 0;
            cp_async16(dst + doff_k + k * 512, kbase + c * 16 + sl * p.k_stride_t, valid ? 16u : 0u);
            if (v_on) cp_async16(dst + doff_v + k * 8 * Rv, vbase_g + c * 16 + sl * p.v_stride_t, valid ? 16u : 0u);
          }
          cp_async_arrive_noinc(bar_full(stage));
          __syncwarp();
          if (lane == 0) publish(stage, use);
        }
      }
      e0 = f0;
      e1 = f1;
      first = ffirst;
    }
    if (!ok) atomicMax(&g_status, (unsigned)kTimeoutProducer);
  } else if (warp < 4 * G) {
    // ================================================================= epilogue
    const int g = warp >> 2, q4 = warp & 3;
    const int h = h0 + g, hk = h / gqa;
    const int row = q4 * 32 + lane;
    const bool interleaved = p.rope_layout == WSVD_ROPE_INTERLEAVED;

    auto wait_issued = [&](int stage, int uses) -> bool {
      const uint32_t addr = sbase + kOffIssued + 4u * stage;
      const uint64_t t0 = global_ns();
      for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
        if ((int)v >= uses) return true;
        if (global_ns() - t0 > 2000000000ull) return false;
      }
    };
    // ---- B operand: P (cos coefficients) and Q (sin coefficients) of this head, f16,
    //      rows n = g*64 + r, 64 frequencies per row, 128-byte swizzle
    {
      const float* qg = qs + g * 128;
      const int tid = threadIdx.x & 127;
      const int64_t col = (int64_t)hk * 128;
      if (wk_vec && !interleaved) {
        // Common case (f16 wk, half-split pairing): packed f16 arithmetic.  The operands are
        // rounded to f16 for the MMA anyway; forming them with one extra f16 rounding of a
        // product keeps the error of the scores within a few 1e-5.  This thread's chunk of 8
        // frequencies is the same for its four ranks, so q is converted once.
        const int ic = tid & 7;
        __half2 qa[4], qb[4], nqa[4];
        {
          const float4 a0 = *reinterpret_cast<const float4*>(qg + ic * 8);
          const float4 a1 = *reinterpret_cast<const float4*>(qg + ic * 8 + 4);
          const float4 b0 = *reinterpret_cast<const float4*>(qg + 64 + ic * 8);
          const float4 b1 = *reinterpret_cast<const float4*>(qg + 64 + ic * 8 + 4);
          qa[0] = __floats2half2_rn(a0.x, a0.y);
          qa[1] = __floats2half2_rn(a0.z, a0.w);
          qa[2] = __floats2half2_rn(a1.x, a1.y);
          qa[3] = __floats2half2_rn(a1.z, a1.w);
          qb[0] = __floats2half2_rn(b0.x, b0.y);
          qb[1] = __floats2half2_rn(b0.z, b0.w);
          qb[2] = __floats2half2_rn(b1.x, b1.y);
          qb[3] = __floats2half2_rn(b1.z, b1.w);
#pragma unroll
          for (int e = 0; e < 4; ++e) nqa[e] = __hneg2(qa[e]);
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int r = (tid + 128 * it) >> 3;
          const __half2* ua = reinterpret_cast<const __half2*>(&wpre[2 * it]);      // U[d = ic*8 .. +7]
          const __half2* ub = reinterpret_cast<const __half2*>(&wpre[2 * it + 1]);  // U[64 + ic*8 .. +7]
          __align__(16) __half2 pv[4];
          __align__(16) __half2 qv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            pv[e] = __hfma2(qa[e], ua[e], __hmul2(qb[e], ub[e]));   // P = q_i U_i + q_{i+64} U_{i+64}
            qv[e] = __hfma2(nqa[e], ub[e], __hmul2(qb[e], ua[e]));  // Q = q_{i+64} U_i - q_i U_{i+64}
          }
          const int nrow = g * 64 + r;
          const uint32_t off = nrow * 128 + ((ic ^ (nrow & 7)) << 4);
          *reinterpret_cast<uint4*>(sm + kOffB + off) = *reinterpret_cast<const uint4*>(pv);
          *reinterpret_cast<uint4*>(sm + kOffB + kBHalfBytes + off) = *reinterpret_cast<const uint4*>(qv);
        }
      } else
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int task = tid + 128 * it;
        const int r = task >> 3, ic = task & 7;  // rank, chunk of 8 frequencies
        float u0[8], u1[8];
        if (wk_vec) {
          // half layout: dims ic*8.. and 64+ic*8..; interleaved: 16 consecutive dims
          const uint4 a0 = wpre[2 * it], a1 = wpre[2 * it + 1];
          const __half* h0p = reinterpret_cast<const __half*>(&a0);
          const __half* h1p = reinterpret_cast<const __half*>(&a1);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            if (interleaved) {
              const __half* src = e < 4 ? h0p : h1p;
              u0[e] = __half2float(src[(2 * e) & 7]);
              u1[e] = __half2float(src[(2 * e + 1) & 7]);
            } else {
              u0[e] = __half2float(h0p[e]);
              u1[e] = __half2float(h1p[e]);
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int i = ic * 8 + e;
            const int d0 = interleaved ? 2 * i : i, d1 = interleaved ? 2 * i + 1 : i + 64;
            if (p.wk_dtype == WSVD_I8) {
              const int8_t* w = reinterpret_cast<const int8_t*>(p.wk) + (int64_t)r * p.wk_stride_r + col;
              const __half* ws = reinterpret_cast<const __half*>(p.wk_scale) + col;
              u0[e] = (float)w[d0] * __half2float(ws[d0]);
              u1[e] = (float)w[d1] * __half2float(ws[d1]);
            } else {
              const __half* w = reinterpret_cast<const __half*>(p.wk) + (int64_t)r * p.wk_stride_r + col;
              u0[e] = __half2float(w[d0]);
              u1[e] = __half2float(w[d1]);
            }
          }
        }
        __align__(16) __half pv[8];
        __align__(16) __half qv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int i = ic * 8 + e;
          const int d0 = interleaved ? 2 * i : i, d1 = interleaved ? 2 * i + 1 : i + 64;
          pv[e] = __float2half_rn(qg[d0] * u0[e] + qg[d1] * u1[e]);
          qv[e] = __float2half_rn(qg[d1] * u0[e] - qg[d0] * u1[e]);
        }
        const int nrow = g * 64 + r;
        const uint32_t off = nrow * 128 + ((ic ^ (nrow & 7)) << 4);
        *reinterpret_cast<uint4*>(sm + kOffB + off) = *reinterpret_cast<const uint4*>(pv);
        *reinterpret_cast<uint4*>(sm + kOffB + kBHalfBytes + off) = *reinterpret_cast<const uint4*>(qv);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pq);
    }

    const __half* ksc = reinterpret_cast<const __half*>(p.k_scale) + (int64_t)hk * p.ks_stride_h;
    const __half* vsc = reinterpret_cast<const __half*>(p.v_scale) + (int64_t)hk * p.vs_stride_h;
    // Scales are read straight from global memory by the lane that owns the token, two
    // tiles deep: the page entry of tile t+2 and the scales of tile t+1 are requested at
    // the top of iteration t, so no load is waited on in the iteration that issues it.
    auto load_slot = [&](int s, int& sl) {
      sl = -1;
      if (s < hi) sl = page[s];  // predicated load: nothing consumes the value here
    };
    auto load_scales = [&](int sl, unsigned short& sk, unsigned short& sv) {
      sk = 0;
      sv = 0;
      if (sl >= 0) {
        sk = reinterpret_cast<const unsigned short*>(ksc)[(int64_t)sl * p.ks_stride_t];
        sv = reinterpret_cast<const unsigned short*>(vsc)[(int64_t)sl * p.vs_stride_t];
      }
    };

    float m_w = -INFINITY, l_lane = 0.f;
    uint64_t acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0ull;
    const int rg = lane & 3, tg = lane >> 2;
    const bool pv_on = rg < (Rv >> 4);
    unsigned short sk_n = 0, sv_n = 0;
    uint4 v_cur[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v_cur[k] = make_uint4(0u, 0u, 0u, 0u);
    bool ok = true;

    for (int t = 0; t < ntiles; ++t) {
      const int s = lo + t * kTile + row;
      const bool valid = s < hi;
      // this warp's 32 tokens lie in half-tile q4/2 of the tile: the head's nth half-tile
      const int nth = 2 * t + (q4 >> 1);
      const int stage = g * kSlots + nth % kSlots, buf = t & 1;
      load_scales(slot_n, sk_n, sv_n);
      load_slot(s + 2 * kTile, slot_n);
      ok = wait_issued(stage, nth / kSlots + 1) && mbar_wait(bar_full(stage), (nth / kSlots) & 1);
      if (!ok) break;

      // ---- the warp's 32 K rows (lane = token) and V rows (lane (rg, tg): chunk rg of rows
      //      tg + 8k) go to registers at once, so that the ring slot is handed back and
      //      refilled before any arithmetic: the register file is the second buffer stage
      uint4 kreg[4];
      {
        const uint32_t krow = sRing + stage * kUnitBytes + (row & (kHalf - 1)) * 64;
        const uint32_t sw = (row >> 1) & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(kreg[c].x), "=r"(kreg[c].y), "=r"(kreg[c].z), "=r"(kreg[c].w)
                       : "r"(krow + ((c ^ sw) << 4)));
      }
      if (pv_on) {
        const uint32_t vsm = sRing + stage * kUnitBytes + kKBytes + ((q4 & 1) * 32 + tg) * Rv + rg * 16;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(v_cur[k].x), "=r"(v_cur[k].y), "=r"(v_cur[k].z), "=r"(v_cur[k].w)
                       : "r"(vsm + k * 8 * Rv));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty(stage));

      ok = mbar_wait(bar_w_full(buf), (t >> 1) & 1);
      if (!ok) break;
      tc_fence_after();

      // ---- score: dot of this token's int8 K row with its row of W, in two halves of 32
      //      ranks, four independent accumulators
      const uint32_t taddr = tmem + ((uint32_t)(q4 * 32) << 16) + buf * (kG * kRk) + g * kRk;
      uint64_t dot[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t w[2][16];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) tmem_ld16(taddr + (2 * hf + cc) * 16, w[cc]);
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const uint4 kq = kreg[2 * hf + cc];
          const uint32_t kws[4] = {kq.x ^ 0x80808080u, kq.y ^ 0x80808080u, kq.z ^ 0x80808080u, kq.w ^ 0x80808080u};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint64_t x01, x23;
            cvt4(kws[j], x01, x23);
            dot[2 * cc] = fma2(x01, pk(__uint_as_float(w[cc][4 * j]), __uint_as_float(w[cc][4 * j + 1])), dot[2 * cc]);
            dot[2 * cc + 1] =
                fma2(x23, pk(__uint_as_float(w[cc][4 * j + 2]), __uint_as_float(w[cc][4 * j + 3])), dot[2 * cc + 1]);
          }
        }
      }
      const uint64_t dot2 = add2(add2(dot[0], dot[1]), add2(dot[2], dot[3]));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_w_empty(buf));  // this warp has read its rows of W
      float d0, d1;
      upk(dot2, d0, d1);
      const float sk = __half2float(__ushort_as_half(sk_raw)), sv = __half2float(__ushort_as_half(sv_raw));
      const float z = valid ? (d0 + d1) * sk : -INFINITY;

      // ---- online softmax, per warp
      const float tmax = warp_max_redux(z);
      if (tmax > m_w) {
        const float sc = fast_exp2(m_w - tmax);  // m_w = -inf -> 0
        const uint64_t sc2 = pk(sc, sc);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fma2(acc[e], sc2, 0ull);
        l_lane *= sc;
        m_w = tmax;
      }
      const float pr = valid ? fast_exp2(z - m_w) : 0.f;
      l_lane += pr;
      const float pvs = pr * sv;

      // ---- P.V on the CUDA cores: this lane owns 16 ranks (chunk rg) of tokens tg + 8k
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float pj = __shfl_sync(0xffffffffu, pvs, tg + 8 * k);
        const uint32_t vws[4] = {v_cur[k].x ^ 0x80808080u, v_cur[k].y ^ 0x80808080u, v_cur[k].z ^ 0x80808080u,
                                 v_cur[k].w ^ 0x80808080u};
        const uint64_t pj2 = pk(pj, pj);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          uint64_t x01, x23;
          cvt4(vws[jj], x01, x23);
          acc[2 * jj] = fma2(x01, pj2, acc[2 * jj]);
          acc[2 * jj + 1] = fma2(x23, pj2, acc[2 * jj + 1]);
        }
      }
      sk_raw = sk_n;
      sv_raw = sv_n;
    }
    if (!ok) atomicMax(&g_status, (unsigned)kTimeoutEpilogue);

    // ---- merge: lanes sharing a rank chunk, then the four warps of the head
    float accf[16];
#pragma unroll
    for (int e = 0; e < 8; ++e) upk(acc[e], accf[2 * e], accf[2 * e + 1]);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      accf[e] += __shfl_xor_sync(0xffffffffu, accf[e], 4);
      accf[e] += __shfl_xor_sync(0xffffffffu, accf[e], 8);
      accf[e] += __shfl_xor_sync(0xffffffffu, accf[e], 16);
    }
    const float l_w = warp_sum(l_lane);
    float* mine = merge + (g * 4 + q4) * (2 + 64);
    if (lane == 0) {
      mine[0] = m_w;
      mine[1] = l_w;
    }
    if (tg == 0 && pv_on) {
#pragma unroll
      for (int e = 0; e < 16; ++e) mine[2 + rg * 16 + e] = accf[e];
    }
    named_barrier(1 + g, 128);
    if (q4 == 0) {
      const float* mg = merge + g * 4 * (2 + 64);
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mg[w * 66]);
      float wgt[4], ll = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        wgt[w] = mg[w * 66] == -INFINITY ? 0.f : fast_exp2(mg[w * 66] - mm);
        ll += wgt[w] * mg[w * 66 + 1];
      }
      const int64_t slot = ((int64_t)b * p.n_q_heads + h) * a.n_splits + split;
      for (int r = lane; r < Rv; r += 32) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) o += wgt[w] * mg[w * 66 + 2 + r];
        a.mid_o[slot * Rv + r] = o / ll;
      }
      // natural-log lse, as the merge kernel expects (stage1.py:216)
      if (lane == 0) a.lse[slot] = mm * 0.6931471805599453f + logf(ll);
    }
  }

  // ---- common exit
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace tc

namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// One latent tensor [T, Hkv, R] int8 with byte strides (st, sh) as a 3-D tensor map whose
// outer axes are ordered by stride; box = 64 token slots x 1 head x R bytes.
bool encode_one(CUtensorMap* map, const void* base, int64_t st, int64_t sh, int64_t T, int Hkv, int R,
                CUtensorMapSwizzle swz, int* slot_axis) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || T <= 0 || T > 0xffffffffll) return false;
  const bool slot_first = st <= sh;  // head-major storage: the slot axis has the smaller stride
  cuuint64_t dims[3] = {(cuuint64_t)R, (cuuint64_t)(slot_first ? T : Hkv), (cuuint64_t)(slot_first ? Hkv : T)};
  cuuint64_t strides[2] = {(cuuint64_t)(slot_first ? st : sh), (cuuint64_t)(slot_first ? sh : st)};
  cuuint32_t box[3] = {(cuuint32_t)R, (cuuint32_t)(slot_first ? kHalf : 1), (cuuint32_t)(slot_first ? 1 : kHalf)};
  cuuint32_t estr[3] = {1, 1, 1};
  *slot_axis = slot_first ? 1 : 2;
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

void encode_latent_maps(const WsvdLatentDecodeParams& p, TcArgs* ta) {
  ta->use_tma = 0;
  ta->slot_axis = 1;
  memset(&ta->tmap_k, 0, sizeof(CUtensorMap));
  memset(&ta->tmap_v, 0, sizeof(CUtensorMap));
  if (p.n_token_slots <= 0) return;
  int ax_k = 1;
  if (!encode_one(&ta->tmap_k, p.latent_k, p.k_stride_t, p.k_stride_h, p.n_token_slots, p.n_kv_heads, kRk,
                  CU_TENSOR_MAP_SWIZZLE_64B, &ax_k))
    return;
  int ax_v = 1;
  if (!encode_one(&ta->tmap_v, p.latent_v, p.v_stride_t, p.v_stride_h, p.n_token_slots, p.n_kv_heads, p.rank_v,
                  CU_TENSOR_MAP_SWIZZLE_NONE, &ax_v) || ax_v != ax_k)
    return;
  ta->slot_axis = ax_k;
  ta->use_tma = 1;
}

}  // namespace tc

size_t rope_table_bytes(int rows) { return (size_t)rows * 256; }

cudaError_t launch_rope_table(void* table, int rows, const KArgs& a, cudaStream_t stream) {
  const int total = rows * 64;
  tc::rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(reinterpret_cast<uint8_t*>(table), rows, a);
  return cudaGetLastError();
}

cudaError_t launch_stage1_tc(const KArgs& a, const void* table, int table_rows, cudaStream_t stream) {
  static_assert(tc::kSmemBytes <= 232448, "shared memory budget");
  cudaError_t e = cudaFuncSetAttribute(tc::stage1_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)tc::kSmemBytes);
  if (e != cudaSuccess) return e;
  tc::TcArgs ta;
  ta.k = a;
  ta.table = reinterpret_cast<const uint8_t*>(table);
  ta.table_rows = table_rows;
  tc::encode_latent_maps(a.p, &ta);
  dim3 grid(a.n_splits, (a.p.n_q_heads + tc::kG - 1) / tc::kG, a.p.batch);
  tc::stage1_tc_kernel<<<grid, tc::kThreads, tc::kSmemBytes, stream>>>(ta);
  return cudaGetLastError();
}

cudaError_t read_tc_status(unsigned int* out) {
  return cudaMemcpyFromSymbol(out, tc::g_status, sizeof(unsigned int));
}

cudaError_t reset_tc_status() {
  const unsigned int zero = 0;
  return cudaMemcpyToSymbol(tc::g_status, &zero, sizeof(unsigned int));
}

}  // namespace wsvd

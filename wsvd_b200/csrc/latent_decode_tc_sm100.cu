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
// reads its row of W from tensor memory and dots it with the token's int8 row in fp32.
// P.V runs on the CUDA cores in fp32 from the int8 rows.  Nothing is rounded to f16
// except the two GEMM operands.
//
// CTA = one (split, group of 4 heads, sequence); 19 warps:
//   warps 0-15  epilogue, 4 per head: warp w owns tensor-memory lanes 32*(w%4)..+31
//   warps 16-17 producers: gather 64-byte latent rows with 16-byte cp.async through the
//               page table into a 5-stage shared-memory ring (16 KB per head-tile)
//   warp 18     one thread issues the table tile loads (cp.async.bulk) and the MMAs
// Every wait on an mbarrier is bounded; on a time-out the kernel records a status code
// and every role falls through to the common exit, which frees the tensor memory.
#include "common.cuh"

namespace wsvd {
namespace tc {

constexpr int kG = 4;          // heads per CTA
constexpr int kTile = 128;     // positions per MMA tile (= tensor-memory lanes)
constexpr int kRk = 64;
constexpr int kEpiWarps = 4 * kG;
#ifndef WSVD_TC_PRODUCER_WARPS
#define WSVD_TC_PRODUCER_WARPS 2
#endif
constexpr int kProducerWarps = WSVD_TC_PRODUCER_WARPS;  // even: K rows, odd: V rows; split further by row range
constexpr int kRowSplit = kProducerWarps / 2;            // producers per tensor
constexpr int kKPerLane = 16 / kRowSplit;                 // rows per lane per head-tile
constexpr int kProducerWarp0 = kEpiWarps;
constexpr int kMmaWarp = kEpiWarps + kProducerWarps;
constexpr int kThreads = (kEpiWarps + kProducerWarps + 1) * 32;
constexpr int kStages = 5;
#ifndef WSVD_TC_PREFETCH_TILES
#define WSVD_TC_PREFETCH_TILES 3
#endif
constexpr int kPrefetchTiles = WSVD_TC_PREFETCH_TILES;   // latent rows are requested into L2 this many tiles ahead
constexpr uint32_t kKBytes = kTile * 64;            // one head-tile of K rows
constexpr uint32_t kUnitBytes = 2 * kKBytes;        // K rows + V rows (padded to 64 B)
constexpr uint32_t kAHalfBytes = kTile * 128;       // 128 rows x 64 f16
constexpr uint32_t kABufBytes = 2 * kAHalfBytes;    // cos half + sin half
constexpr uint32_t kBHalfBytes = kG * kRk * 128;    // 256 rows x 64 f16
constexpr uint32_t kTmemCols = 512;                 // 2 buffers x (kG*kRk) fp32 columns

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffB = 0;
constexpr uint32_t kOffA = kOffB + 2 * kBHalfBytes;
constexpr uint32_t kOffRing = kOffA + 2 * kABufBytes;
constexpr uint32_t kOffMerge = kOffRing + kStages * kUnitBytes;
constexpr uint32_t kMergeFloats = kG * 4 * (2 + 64);
constexpr uint32_t kOffQ = kOffMerge + kMergeFloats * 4;
constexpr uint32_t kOffBar = kOffQ + kG * 128 * 4;
constexpr int kNumBars = 2 * kStages + 2 + 2 + 2 + 2 + 1;
constexpr uint32_t kOffTmemSlot = kOffBar + kNumBars * 8;
constexpr uint32_t kSmemBytes = kOffTmemSlot + 16 + 1024;  // + slack for the manual alignment

enum Status : unsigned int { kOk = 0, kTimeoutProducer = 1, kTimeoutMma = 2, kTimeoutEpilogue = 3 };

__device__ unsigned int g_status = 0;

// Optional cycle-stamp trace of one CTA (compile with -DWSVD_TC_TRACE): role x tile x event.
#ifdef WSVD_TC_TRACE
__device__ long long g_trace[8][64][8];
#define WSVD_TRACE(role, t, ev)                                                         \
  do {                                                                                  \
    if (trace_cta && lane == 0 && (t) < 64) g_trace[role][t][ev] = clock64();          \
  } while (0)
#else
#define WSVD_TRACE(role, t, ev)
#endif

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// try_wait with a suspend-time hint: the waiting thread is parked by the hardware until
// the phase completes or the hint (ns) expires, instead of spinning on issue slots that
// the producer and MMA warps need.
#ifndef WSVD_TC_WAIT_HINT_NS
#define WSVD_TC_WAIT_HINT_NS 20000
#endif
__device__ __forceinline__ uint32_t mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"((uint32_t)WSVD_TC_WAIT_HINT_NS)
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
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
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
#ifdef WSVD_TC_TRACE
  const bool trace_cta = blockIdx.x == 1 && blockIdx.y == 1 && blockIdx.z == 1;
  if (warp == 0) WSVD_TRACE(7, 0, 0);
#endif

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - raw);
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

  // ---- set-up: barriers + tensor memory (warp 17), scaled q to shared memory (epilogue warps)
  if (warp == kMmaWarp) {
    if (lane == 0) {
      for (int s = 0; s < kStages; ++s) {
        mbar_init(bar_full(s), 32 * kProducerWarps);   // one asynchronous arrive per producer lane
        mbar_init(bar_empty(s), 4);   // one arrive per epilogue warp of the owning head
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(bar_a_full(i), 1);
        mbar_init(bar_a_empty(i), 1);
        mbar_init(bar_w_full(i), 1);
        mbar_init(bar_w_empty(i), 4 * G);
      }
      mbar_init(bar_pq, 4 * G);
      fence_barrier_init();
    }
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  } else if (warp < 4 * G) {
    // q * sm_scale * log2(e): scores come out in the log2 domain
    const float qscale = a.sm_scale * 1.4426950408889634f;
    for (int idx = threadIdx.x; idx < G * 128; idx += 128 * G) {
      const int g = idx >> 7, d = idx & 127;
      const __half* qp = reinterpret_cast<const __half*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)(h0 + g) * p.q_stride_h;
      qs[idx] = __half2float(qp[d]) * qscale;
    }
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (warp == 0) WSVD_TRACE(7, 0, 1);

  if (warp >= kProducerWarp0 && warp < kProducerWarp0 + kProducerWarps) {
    // ================================================================= producers
    // Producer 0 copies the K rows and producer 1 the V rows of every head-tile, so both
    // walk the ring in the same order (a waiter can then never be two phases ahead of an
    // mbarrier, which a parity wait could not tell from "done").
    // Lane (r0 = lane/4, c = lane%4) copies 16-byte chunk c of rows r0 + 8k, k < 16.  The
    // destination chunk is XOR-swizzled with (row/2)%4 so that both "lane = row" 16-byte
    // reads (scores) and "quarter-warp = two rows" reads (P.V) are bank-conflict free;
    // (row/2)%4 does not depend on k, so the destination offsets are immediates.
    const int pw = warp - kProducerWarp0;
    const int is_v = pw & 1, kbase = (pw >> 1) * kKPerLane;
    const int c = lane & 3, r0 = (lane >> 2) + 8 * kbase;
    const bool chunk_on = !is_v || c < (Rv >> 4);
    const uint8_t* base = reinterpret_cast<const uint8_t*>(is_v ? p.latent_v : p.latent_k) + c * 16;
    const int64_t hstride = is_v ? p.v_stride_h : p.k_stride_h;
    const int tstride = (int)(is_v ? p.v_stride_t : p.k_stride_t);
    const uint32_t doff = (is_v ? kKBytes : 0u) + r0 * 64 + ((c ^ ((r0 >> 1) & 3)) << 4);
    int32_t slot_cur[kKPerLane], slot_nxt[kKPerLane];
#pragma unroll
    for (int k = 0; k < kKPerLane; ++k) {
      const int s = lo + r0 + 8 * k;
      slot_nxt[k] = -1;
      if (s < hi) slot_nxt[k] = page[s];
    }
    bool ok = true;
    int u = 0;
    for (int t = 0; t < ntiles && ok; ++t) {
      if (pw == 0) WSVD_TRACE(0, t, 0);
#pragma unroll
      for (int k = 0; k < kKPerLane; ++k) slot_cur[k] = slot_nxt[k];
      if (t + 1 < ntiles) {
#pragma unroll
        for (int k = 0; k < kKPerLane; ++k) {
          const int s = lo + (t + 1) * kTile + r0 + 8 * k;
          slot_nxt[k] = -1;
          if (s < hi) slot_nxt[k] = page[s];
        }
      }
      const bool full_tile = lo + (t + 1) * kTile <= hi;
      for (int g = 0; g < G; ++g, ++u) {
        const int stage = u % kStages;
        if (pw == 0) WSVD_TRACE(6, u, 0);
        if (u >= kStages && !mbar_wait(bar_empty(stage), ((u / kStages) - 1) & 1)) {
          atomicMax(&g_status, (unsigned)kTimeoutProducer);
          ok = false;
          break;
        }
        if (pw == 0) WSVD_TRACE(6, u, 1);
        const uint8_t* src = base + (int64_t)((h0 + g) / gqa) * hstride;
        const uint32_t dst = sRing + stage * kUnitBytes + doff;
        if (chunk_on) {
          if (full_tile) {
#pragma unroll
            for (int k = 0; k < kKPerLane; ++k) cp_async16(dst + k * 512, src + (int64_t)slot_cur[k] * tstride, 16u);
          } else {
#pragma unroll
            for (int k = 0; k < kKPerLane; ++k) {
              const bool valid = slot_cur[k] >= 0;  // rows past the end are zero-filled
              cp_async16(dst + k * 512, src + (int64_t)(valid ? slot_cur[k] : 0) * tstride, valid ? 16u : 0u);
            }
          }
        }
        if (pw == 0) WSVD_TRACE(6, u, 3);
        cp_async_arrive_noinc(bar_full(stage));
        if (pw == 0) WSVD_TRACE(6, u, 2);
      }
      // Ask for the rows of tile t + kPrefetchTiles to be brought into L2 (one bulk
      // prefetch per head when the 128 rows are contiguous in memory) so that the ring
      // only has to cover the L2 -> shared-memory latency, not the DRAM latency.
      if (kPrefetchTiles > 0 && pw < 2 && lane == 0 && t + kPrefetchTiles < ntiles) {
        const int s0 = lo + (t + kPrefetchTiles) * kTile;
        const int rows = min(kTile, hi - s0);
        const int rowbytes = is_v ? Rv : kRk;
        if (tstride == rowbytes && page[s0 + rows - 1] - page[s0] == rows - 1) {
          const int64_t sl0 = page[s0];
          for (int g = 0; g < G; ++g)
            prefetch_l2_bulk(base - c * 16 + (int64_t)((h0 + g) / gqa) * hstride + sl0 * tstride, rows * rowbytes);
        }
      }
      if (pw == 0) WSVD_TRACE(0, t, 1);
    }
    cp_async_wait_all();
  } else if (warp == kMmaWarp) {
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
      bool ok = mbar_wait(bar_pq, 0);
      for (int t = 0; t < ntiles && ok; ++t) {
        const int buf = t & 1;
        WSVD_TRACE(1, t, 0);
        ok = mbar_wait(bar_a_full(buf), (t >> 1) & 1);
        WSVD_TRACE(1, t, 1);
        if (ok && t >= 2) ok = mbar_wait(bar_w_empty(buf), ((t >> 1) - 1) & 1);
        WSVD_TRACE(1, t, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem + buf * (kG * kRk);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t koff = (kk & 3) * 32;
          const uint64_t ad = smem_desc_sw128(sA + buf * kABufBytes + (kk >> 2) * kAHalfBytes + koff);
          const uint64_t bd = smem_desc_sw128(sB + (kk >> 2) * kBHalfBytes + koff);
          umma_f16(d_tmem, ad, bd, idesc, kk > 0);
        }
        umma_commit(bar_w_full(buf));
        umma_commit(bar_a_empty(buf));
        WSVD_TRACE(1, t, 3);
        if (t + 1 < ntiles && t + 1 >= 2) {
          ok = mbar_wait(bar_a_empty((t + 1) & 1), (((t + 1) >> 1) - 1) & 1);
          if (ok) issue_table(t + 1);
        }
        WSVD_TRACE(1, t, 4);
      }
      if (!ok) atomicMax(&g_status, (unsigned)kTimeoutMma);
    }
    __syncwarp();
  } else if (warp < 4 * G) {
    // ================================================================= epilogue
    const int g = warp >> 2, q4 = warp & 3;
    const int h = h0 + g, hk = h / gqa;
    const int row = q4 * 32 + lane;
    const bool interleaved = p.rope_layout == WSVD_ROPE_INTERLEAVED;

    // ---- B operand: P (cos coefficients) and Q (sin coefficients) of this head, f16,
    //      rows n = g*64 + r, 64 frequencies per row, 128-byte swizzle
    {
      const float* qg = qs + g * 128;
      const int tid = threadIdx.x & 127;
      const int64_t col = (int64_t)hk * 128;
      const bool vec = p.wk_dtype == WSVD_F16 && (p.wk_stride_r & 7) == 0 &&
                       (reinterpret_cast<uintptr_t>(p.wk) & 15) == 0;
      for (int task = tid; task < 64 * 8; task += 128) {
        const int r = task >> 3, ic = task & 7;  // rank, chunk of 8 frequencies
        float u0[8], u1[8];
        if (vec) {
          // half layout: dims ic*8.. and 64+ic*8..; interleaved: 16 consecutive dims
          const __half* w = reinterpret_cast<const __half*>(p.wk) + (int64_t)r * p.wk_stride_r + col;
          const uint4 a0 = *reinterpret_cast<const uint4*>(w + (interleaved ? ic * 16 : ic * 8));
          const uint4 a1 = *reinterpret_cast<const uint4*>(w + (interleaved ? ic * 16 + 8 : 64 + ic * 8));
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
    if (warp == 0) WSVD_TRACE(7, 0, 2);

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
    unsigned short sk_raw, sv_raw, sk_n = 0, sv_n = 0;
    int slot_n;
    load_slot(lo + row, slot_n);
    load_scales(slot_n, sk_raw, sv_raw);
    load_slot(lo + kTile + row, slot_n);
    const int rg = lane & 3, tg = lane >> 2;
    const bool pv_on = rg < (Rv >> 4);
    bool ok = true;

    for (int t = 0; t < ntiles; ++t) {
      const int s = lo + t * kTile + row;
      const bool valid = s < hi;
      const int u = t * G + g, stage = u % kStages, buf = t & 1;
      if (q4 == 0) WSVD_TRACE(2 + g, t, 0);
      load_scales(slot_n, sk_n, sv_n);
      load_slot(s + 2 * kTile, slot_n);
      if (q4 == 0) WSVD_TRACE(2 + g, t, 1);
      ok = mbar_wait(bar_full(stage), (u / kStages) & 1);
      if (q4 == 0) WSVD_TRACE(2 + g, t, 2);
      ok = ok && mbar_wait(bar_w_full(buf), (t >> 1) & 1);
      if (q4 == 0) WSVD_TRACE(2 + g, t, 3);
      if (!ok) break;
      tc_fence_after();

      // ---- score: dot of this token's int8 K row with its row of W, in two halves of 32
      //      ranks, four independent accumulators
      const uint32_t krow = sRing + stage * kUnitBytes + row * 64;
      const uint32_t sw = (row >> 1) & 3;
      const uint32_t taddr = tmem + ((uint32_t)(q4 * 32) << 16) + buf * (kG * kRk) + g * kRk;
      uint64_t dot[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t w[2][16];
        uint4 kw[2];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = 2 * hf + cc;
          tmem_ld16(taddr + c * 16, w[cc]);
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(kw[cc].x), "=r"(kw[cc].y), "=r"(kw[cc].z), "=r"(kw[cc].w)
                       : "r"(krow + ((c ^ sw) << 4)));
        }
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const uint32_t kws[4] = {kw[cc].x ^ 0x80808080u, kw[cc].y ^ 0x80808080u, kw[cc].z ^ 0x80808080u,
                                   kw[cc].w ^ 0x80808080u};
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
      if (lane == 0) mbar_arrive(bar_w_empty(buf));
      if (q4 == 0) WSVD_TRACE(2 + g, t, 4);
      float d0, d1;
      upk(dot2, d0, d1);
      const float sk = __half2float(__ushort_as_half(sk_raw)), sv = __half2float(__ushort_as_half(sv_raw));
      const float z = valid ? (d0 + d1) * sk : -INFINITY;

      // ---- online softmax, per warp
      const float tmax = warp_max(z);
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
      if (q4 == 0) WSVD_TRACE(2 + g, t, 5);

      // ---- P.V on the CUDA cores: this lane owns 16 ranks (chunk rg) of tokens tg + 8k
      const uint32_t vbase = sRing + stage * kUnitBytes + kKBytes + (q4 * 32) * 64;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int j = tg + 8 * k;
        const float pj = __shfl_sync(0xffffffffu, pvs, j);
        if (pv_on) {
          const int vr = q4 * 32 + j;
          uint4 vw;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(vw.x), "=r"(vw.y), "=r"(vw.z), "=r"(vw.w)
                       : "r"(vbase + j * 64 + ((rg ^ ((vr >> 1) & 3)) << 4)));
          const uint32_t vws[4] = {vw.x ^ 0x80808080u, vw.y ^ 0x80808080u, vw.z ^ 0x80808080u, vw.w ^ 0x80808080u};
          const uint64_t pj2 = pk(pj, pj);
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            uint64_t x01, x23;
            cvt4(vws[jj], x01, x23);
            acc[2 * jj] = fma2(x01, pj2, acc[2 * jj]);
            acc[2 * jj + 1] = fma2(x23, pj2, acc[2 * jj + 1]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty(stage));
      if (q4 == 0) WSVD_TRACE(2 + g, t, 6);
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
  dim3 grid(a.n_splits, (a.p.n_q_heads + tc::kG - 1) / tc::kG, a.p.batch);
  tc::stage1_tc_kernel<<<grid, tc::kThreads, tc::kSmemBytes, stream>>>(ta);
  return cudaGetLastError();
}

cudaError_t read_tc_status(unsigned int* out) {
  return cudaMemcpyFromSymbol(out, tc::g_status, sizeof(unsigned int));
}

#ifdef WSVD_TC_TRACE
extern "C" int wsvd_debug_read_trace(long long* dst) {
  return (int)cudaMemcpyFromSymbol(dst, tc::g_trace, sizeof(long long) * 8 * 64 * 8);
}
#endif

cudaError_t reset_tc_status() {
  const unsigned int zero = 0;
  return cudaMemcpyToSymbol(tc::g_status, &zero, sizeof(unsigned int));
}

}  // namespace wsvd

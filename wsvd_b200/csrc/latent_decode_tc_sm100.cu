// Split-KV stage 1 of the latent decode attention on the Blackwell tensor cores
// (tcgen05.mma with accumulators in tensor memory), for head_dim 128, int8 latents,
// rank_k and rank_v in {16,32,48,64}.
//
// Scores.  For one head, query q and position s
//   z_s = c * sk_s * sum_r Lk[s,r] * W[s,r],
//   W[s,r] = sum_i cos(s f_i) P[r,i] + sin(s f_i) Q[r,i],
//   P[r,i] = q_i U[i,r] + q_{i+64} U[i+64,r],   Q[r,i] = q_{i+64} U[i,r] - q_i U[i+64,r]
// which is the reference's reconstruct -> RoPE -> q.K' chain
// (efficiency/kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:149-169) with
// the sums reordered: the rotation is moved from K onto the query side.  W is one f16 GEMM
//   [128 positions x 128 (cos|sin)] x [128 x 64*(heads of a pair)]
// per tile of 128 positions and pair of heads: the A operand is a tile of a position table
// of cos/sin values (f16, shared by every head and sequence, read from L2 by TMA), the B
// operand [P;Q] is built once per CTA and stays in shared memory, the accumulator is fp32
// in tensor memory (three 128-column buffers).  Each epilogue thread owns one token: it
// reads its row of W from tensor memory and dots it in fp32 with the token's int8 K row,
// which it fetched itself from global memory into registers one tile ahead.
//
// Values.  O[r] = sum_s p_s sv_s Lv[s,r] is a true contraction over the tokens and runs on
// the tensor cores as an int8 MMA (kind::i8): the A operand is the V half-tile exactly as
// TMA wrote it (64 tokens x 64 bytes, 64-byte swizzle = the MN-major canonical layout), the
// B operand is the tile's weights a_s = 2^(y_s - max y), y_s = z_s + log2 sv_s, written by
// their owner threads as three unsigned 8-bit digit planes of round(a_s * (2^24 - 256));
// the int32 accumulator (64 ranks x 8 columns per head) is read back once per tile and
// folded into a running fp32 sum under a running reference max(y).  The weights lose nothing
// that fp32 would keep: 24 bits relative to the largest weight of the tile.  The softmax
// denominator is accumulated by the owner threads in fp32.
//
// CTA = one (split, group of 4 heads, sequence); 20 warps:
//   warps 0-15   epilogue, 4 per head: warp w owns tensor-memory lanes 32*(w%4)..+31, i.e.
//                tokens 32*(w%4).. of every tile of head w/4; lane 0 of the head's first warp
//                issues the head's value MMAs
//   warp 16      one thread issues the table-tile loads and the score MMAs
//   warps 17-19  request the V rows: every head has a ring of kVSlots half-tiles; one TMA
//                tensor copy per half-tile when its token slots are consecutive (lane g serves
//                head g), else a gather of rows with 16-byte cp.async through the page table
// Every wait inside the tile loop is an mbarrier wait with a time limit; on a time-out the
// kernel records a status code and every role falls through to the common exit, which frees
// the tensor memory.
#include <cuda.h>
#include <string.h>

#include "common.cuh"

namespace wsvd {
namespace tc {

constexpr int kG = 4;          // heads per CTA
constexpr int kTile = 128;     // positions per MMA tile (= tensor-memory lanes)
constexpr int kHalf = kTile / 2;
constexpr int kRkMax = 64;
constexpr int kEpiWarps = 4 * kG;
constexpr int kMmaWarp = kEpiWarps;
constexpr int kProducers = 3;  // with the MMA warp they fill one warp slot per scheduler
constexpr int kThreads = (kEpiWarps + 1 + kProducers) * 32;
constexpr int kVSlots = 5;     // half-tiles of V in flight or in use, per head
constexpr int kWBufs = 3;      // W accumulators of 128 columns (one pair of heads each)

constexpr uint32_t kVSlotBytes = kHalf * 64;        // 64 tokens x 64 bytes (rank_v < 64: zero-filled)
constexpr uint32_t kAHalfBytes = kTile * 128;       // 128 rows x 64 f16
constexpr uint32_t kABufBytes = 2 * kAHalfBytes;    // cos half + sin half
constexpr uint32_t kBHalfBytes = kG * kRkMax * 128; // 256 rows x 64 f16
constexpr uint32_t kPlaneBytes = 256;               // per warp: 2 chunks of 16 tokens x 8 rows x 16 bytes
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemD = kWBufs * 128;           // first column of the value accumulators (8 per head)
constexpr float kPlaneScale = 16776960.f;           // 2^24 - 256: a weight of 1 is 0xFFFF00

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffB = 0;
constexpr uint32_t kOffA = kOffB + 2 * kBHalfBytes;
constexpr uint32_t kOffV = kOffA + 2 * kABufBytes;
constexpr uint32_t kOffPlanes = kOffV + kG * kVSlots * kVSlotBytes;
constexpr uint32_t kOffQ = kOffPlanes + kEpiWarps * kPlaneBytes;
constexpr uint32_t kOffXch = kOffQ + kG * 128 * 4;            // [head][tile parity][warp] (max z, max y)
constexpr uint32_t kOffSum = kOffXch + kG * 2 * 4 * 8;        // [head][warp] partial denominators
constexpr uint32_t kOffBar = kOffSum + kG * 4 * 4;
// barriers: V full/empty per (head, slot), table full/empty x2, W full/empty x3, D full per head,
// max-exchange x2 per head, planes-ready per head, [P;Q] ready
constexpr int kBarVFull = 0;
constexpr int kBarVEmpty = kBarVFull + kG * kVSlots;
constexpr int kBarAFull = kBarVEmpty + kG * kVSlots;
constexpr int kBarAEmpty = kBarAFull + 2;
constexpr int kBarWFull = kBarAEmpty + 2;
constexpr int kBarWEmpty = kBarWFull + kWBufs;
constexpr int kBarDFull = kBarWEmpty + kWBufs;
constexpr int kBarXch = kBarDFull + kG;
constexpr int kBarPlanes = kBarXch + 2 * kG;
constexpr int kBarPq = kBarPlanes + kG;
constexpr int kNumBars = kBarPq + 1;
constexpr uint32_t kOffTmemSlot = kOffBar + kNumBars * 8;
constexpr uint32_t kSmemBytes = kOffTmemSlot + 16;  // the dynamic shared-memory base is 1024-byte aligned
static_assert(kOffA % 1024 == 0 && kOffV % 1024 == 0 && kOffPlanes % 256 == 0 && kOffBar % 8 == 0, "alignment");

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
// the phase completes or the hint (ns) expires, instead of spinning on issue slots.
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
// The same for a whole warp: every lane waits, and the warp agrees on the outcome so that no
// lane leaves a loop that the others stay in.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
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
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
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
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
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

// UMMA shared-memory descriptors (sm_100 descriptor version 1).
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}
// MN-major operand, 64-byte swizzle: 64 bytes along M per K index, 8 K indices per 512 bytes.
__device__ __forceinline__ uint64_t smem_desc_mn_sw64(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                       // leading byte offset (one 64-byte atom along M: unused)
  d |= (uint64_t)(512 >> 4) << 32;              // stride byte offset between groups of 8 K indices
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;                       // SWIZZLE_64B
  return d;
}
// K-major operand without swizzle, 8 rows: 16-byte K chunks 128 bytes apart, rows 16 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k_plain(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)(128 >> 4) << 16;              // leading byte offset: between the K chunks
  d |= (uint64_t)(256 >> 4) << 32;              // stride byte offset between 8-row groups (one group: unused)
  d |= (uint64_t)1 << 46;
  return d;
}
// Instruction descriptors.  f16 x f16 -> f32, both operands K-major.
__device__ __forceinline__ uint32_t instr_desc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// s8 (A, MN-major) x u8 (B, K-major) -> s32.
__device__ __forceinline__ uint32_t instr_desc_i8(int m, int n) {
  return (2u << 4) | (1u << 7) | (0u << 10) | (1u << 15) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct TcArgs {
  KArgs k;
  int32_t table_rows;
  int32_t use_tma;        // 0: V rows are gathered with cp.async
  int32_t slot_axis;      // 1 or 2: which coordinate of tmap_v is the token slot
  alignas(64) CUtensorMap tmap_v;      // V latents as a 3-D byte tensor, box 64 bytes x 64 slots, 64-byte swizzle
  alignas(64) CUtensorMap tmap_table;  // [2][rows][64] f16, box 64 x 128 x 1, 128-byte swizzle
};

// ------------------------------------------------------------------ position table
// [2][rows][64] f16: plane 0 cos(pos * f_i), plane 1 sin(pos * f_i).
__global__ void rope_table_kernel(__half* table, int rows, KArgs a) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int pos = idx >> 6, i = idx & 63;
  if (pos >= rows) return;
  float sn, cs;
  sincosf((float)pos * a.inv_freq[i], &sn, &cs);
  table[(size_t)pos * 64 + i] = __float2half_rn(cs);
  table[((size_t)rows + pos) * 64 + i] = __float2half_rn(sn);
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
  const int npairs = (G + 1) >> 1;
  const int ntiles = (hi - lo + kTile - 1) / kTile;
  const int n_units = (hi - lo + kHalf - 1) / kHalf;  // half-tiles that hold at least one token
  const int gqa = p.n_q_heads / p.n_kv_heads;
  const int Rk = p.rank_k, Rv = p.rank_v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos0 = (p.pos_offset != nullptr ? p.pos_offset[b] : 0) + lo;  // RoPE position of token lo

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t sbase = smem_u32(smem_raw);
  uint8_t* sm = smem_raw;
  if ((sbase & 1023u) != 0) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicMax(&g_status, (unsigned)kBadSmemAlignment);
    return;
  }
  const uint32_t sB = sbase + kOffB, sA = sbase + kOffA, sV = sbase + kOffV, sPl = sbase + kOffPlanes;
  float* qs = reinterpret_cast<float*>(sm + kOffQ);
  const uint32_t bars = sbase + kOffBar;
  auto bar = [&](int i) { return bars + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + kOffTmemSlot);

  const int32_t* page = p.req_to_token + (int64_t)p.b_req_idx[b] * p.rtt_stride;

  // 16-byte vector loads of wk need f16 data with 16-byte aligned rows
  const bool wk_vec = p.wk_dtype == WSVD_F16 && (p.wk_stride_r & 7) == 0 &&
                      (reinterpret_cast<uintptr_t>(p.wk) & 15) == 0;
  uint4 wpre[8];
  // requested during set-up so that their latency is hidden behind it
  int slot_n = -1, pe0 = -1, pe1 = -1, pfirst = 0;
  unsigned short sk_raw = 0, sv_raw = 0;
  uint4 kreg[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) kreg[c] = make_uint4(0u, 0u, 0u, 0u);

  // ---- set-up: barriers + tensor memory (MMA warp), scaled q to shared memory (epilogue warps)
  if (warp == kMmaWarp) {
    for (int i = lane; i < kNumBars; i += 32) {
      uint32_t count = 1;                                    // one TMA or commit arrival
      if (i < kBarVEmpty) count = 32;                        // V full: one arrive per copying lane
      else if (i >= kBarWEmpty && i < kBarDFull) count = 8;  // W empty: 8 warp arrivals (see w_empty_arrivals)
      else if (i >= kBarXch && i < kBarPq) count = 4;        // the head's four warps
      else if (i == kBarPq) count = 4 * G;
      mbar_init(bar(i), count);
    }
    if (lane == 0)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&ta.tmap_table)) : "memory");
    fence_barrier_init();
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  } else if (warp > kMmaWarp) {
    if (ta.use_tma && lane == 0)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&ta.tmap_v)) : "memory");
    // page entries of this producer's first unit (same indexing as fetch_entries below)
    const int nu = warp - kMmaWarp - 1;
    if (nu < n_units) {
      const int s0 = lo + (nu >> 1) * kTile + (nu & 1) * kHalf, sa = s0 + 2 * lane;
      if (sa < hi) pe0 = page[sa];
      if (sa + 1 < hi) pe1 = page[sa + 1];
      pfirst = page[s0];
    }
  } else if (warp < 4 * G) {
    const int hk_pre = (h0 + (warp >> 2)) / gqa;
    {
      // this lane's first token: page entry, K row, scales; and the page entry of its next token
      const int s_first = lo + (warp & 3) * 32 + lane;
      int slot0 = -1;
      if (s_first < hi) slot0 = page[s_first];
      if (s_first + kTile < hi) slot_n = page[s_first + kTile];
      if (slot0 >= 0) {
        const uint8_t* krow = reinterpret_cast<const uint8_t*>(p.latent_k) + (int64_t)hk_pre * p.k_stride_h +
                              (int64_t)slot0 * p.k_stride_t;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (c * 16 < Rk) kreg[c] = __ldg(reinterpret_cast<const uint4*>(krow) + c);
        sk_raw = reinterpret_cast<const unsigned short*>(p.k_scale)[(int64_t)hk_pre * p.ks_stride_h + (int64_t)slot0 * p.ks_stride_t];
        sv_raw = reinterpret_cast<const unsigned short*>(p.v_scale)[(int64_t)hk_pre * p.vs_stride_h + (int64_t)slot0 * p.vs_stride_t];
      }
    }
    // the head's slice of wk for the [P;Q] build: requested now, used after the barrier
    if (wk_vec) {
      const bool il = p.rope_layout == WSVD_ROPE_INTERLEAVED;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int task = (threadIdx.x & 127) + 128 * i, r = task >> 3, ic = task & 7;
        wpre[2 * i] = make_uint4(0u, 0u, 0u, 0u);
        wpre[2 * i + 1] = make_uint4(0u, 0u, 0u, 0u);
        if (r < Rk) {
          const __half* w = reinterpret_cast<const __half*>(p.wk) + (int64_t)r * p.wk_stride_r + (int64_t)hk_pre * 128;
          wpre[2 * i] = *reinterpret_cast<const uint4*>(w + (il ? ic * 16 : ic * 8));
          wpre[2 * i + 1] = *reinterpret_cast<const uint4*>(w + (il ? ic * 16 + 8 : 64 + ic * 8));
        }
      }
    }
    // q * sm_scale * log2(e): scores come out in the log2 domain
    const float qscale = a.sm_scale * 1.4426950408889634f;
    for (int idx = threadIdx.x; idx < G * 128; idx += 128 * G) {
      const int g = idx >> 7, d = idx & 127;
      const __half* qp = reinterpret_cast<const __half*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)(h0 + g) * p.q_stride_h;
      qs[idx] = __half2float(qp[d]) * qscale;
    }
    // this warp's digit planes: rows 3..7 of both chunks stay zero for the whole kernel
    reinterpret_cast<uint2*>(sm + kOffPlanes + warp * kPlaneBytes)[lane] = make_uint2(0u, 0u);
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == kMmaWarp) {
    // ================================================================= table loads + score MMAs
    if (lane == 0) {
      auto issue_table = [&](int t) {
        const int buf = t & 1;
        const int row = pos0 + t * kTile;
        mbar_expect_tx(bar(kBarAFull + buf), kABufBytes);
        tma_load_3d(sA + buf * kABufBytes, &ta.tmap_table, 0, row, 0, bar(kBarAFull + buf));
        tma_load_3d(sA + buf * kABufBytes + kAHalfBytes, &ta.tmap_table, 0, row, 1, bar(kBarAFull + buf));
      };
      issue_table(0);
      if (ntiles > 1) issue_table(1);
      // descriptors: only the start-address field changes between k-steps, buffers and pairs
      const uint64_t adesc0 = smem_desc_sw128(sA), bdesc0 = smem_desc_sw128(sB);
      bool ok = mbar_wait(bar(kBarPq), 0);
      int u = 0;  // running count of (tile, pair) units: unit u uses W buffer u % kWBufs
      for (int t = 0; t < ntiles && ok; ++t) {
        const int buf = t & 1;
        // The table tile of t+1 goes into the buffer MMA(t-1) read; that MMA was issued a
        // whole iteration ago, so this wait is short and the load overlaps MMA(t).
        if (t >= 1 && t + 1 < ntiles) {
          ok = mbar_wait(bar(kBarAEmpty + ((t + 1) & 1)), ((t - 1) >> 1) & 1);
          if (!ok) break;
          issue_table(t + 1);
        }
        ok = mbar_wait(bar(kBarAFull + buf), (t >> 1) & 1);
        for (int pr = 0; pr < npairs && ok; ++pr, ++u) {
          const int wb = u % kWBufs;
          if (u >= kWBufs) ok = mbar_wait(bar(kBarWEmpty + wb), ((u / kWBufs) - 1) & 1);
          if (!ok) break;
          tc_fence_after();
          const int heads = min(2, G - 2 * pr);
          const uint32_t idesc = instr_desc_f16(kTile, kRkMax * heads);
          const uint32_t d_tmem = tmem + wb * 128;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t koff = (kk & 3) * 32;
            const uint64_t ad = adesc0 + ((buf * kABufBytes + (kk >> 2) * kAHalfBytes + koff) >> 4);
            const uint64_t bd = bdesc0 + (((kk >> 2) * kBHalfBytes + pr * (2 * kRkMax * 128) + koff) >> 4);
            umma_f16(d_tmem, ad, bd, idesc, kk > 0);
          }
          umma_commit(bar(kBarWFull + wb));
        }
        if (ok) umma_commit(bar(kBarAEmpty + buf));
      }
      if (!ok) atomicMax(&g_status, (unsigned)kTimeoutMma);
    }
    __syncwarp();
  } else if (warp > kMmaWarp) {
    // ================================================================= V copies
    // Every head's half-tiles (units n = 2*tile + half) cycle through its kVSlots ring slots; unit n
    // is requested as soon as the value MMAs that read unit n - kVSlots have completed (their commit
    // arrives on the slot's "empty" barrier).  Producer warp pw takes the units n = pw (mod 3).  On
    // the TMA path lane g serves head g on its own, so the heads do not queue behind one another.
    const int pw = warp - kMmaWarp - 1;
    // page entries of the unit's 64 rows (two per lane) and of its first row
    auto fetch_entries = [&](int nu, int& e0, int& e1, int& first) {
      const int s0 = lo + (nu >> 1) * kTile + (nu & 1) * kHalf, sa = s0 + 2 * lane;
      e0 = -1;
      e1 = -1;
      if (sa < hi) e0 = page[sa];
      if (sa + 1 < hi) e1 = page[sa + 1];
      first = page[s0];
    };
    int e0 = pe0, e1 = pe1, first = pfirst;  // unit pw's entries were requested during set-up
    bool ok = true;
    for (int nu = pw; nu < n_units && ok; nu += kProducers) {
      int f0 = -1, f1 = -1, ffirst = 0;
      if (nu + kProducers < n_units) fetch_entries(nu + kProducers, f0, f1, ffirst);  // one unit ahead
      const int vslot = nu % kVSlots, use = nu / kVSlots;
      const bool affine = (e0 < 0 || e0 == first + 2 * lane) && (e1 < 0 || e1 == first + 2 * lane + 1);
      if (ta.use_tma && __all_sync(0xffffffffu, affine)) {
        if (lane < G) {
          const int stage = lane * kVSlots + vslot, hk = (h0 + lane) / gqa;
          if (use > 0) ok = mbar_wait(bar(kBarVEmpty + stage), (use - 1) & 1);
          if (ok) {
            const int c1 = ta.slot_axis == 1 ? first : hk, c2 = ta.slot_axis == 1 ? hk : first;
            mbar_expect_tx(bar(kBarVFull + stage), kVSlotBytes);
            tma_load_3d(sV + stage * kVSlotBytes, &ta.tmap_v, 0, c1, c2, bar(kBarVFull + stage));
            mbar_arrive_n(bar(kBarVFull + stage), 31);  // the arrivals the gather path makes lane by lane
          }
        }
        ok = __all_sync(0xffffffffu, ok);
      } else {
        // Gather through the page table, head after head: lane (r0 = lane/4, c = lane%4) copies
        // 16-byte chunk c of rows r0 + 8k, placed as the 64-byte swizzle places it: chunk index
        // XOR (row/2)%4, which does not depend on k.  Rows past the end and chunks past rank_v
        // are zero-filled.
        const int c = lane & 3, r0 = lane >> 2;
        const uint32_t doff = r0 * 64 + ((c ^ ((r0 >> 1) & 3)) << 4);
        const bool c_on = c * 16 < Rv;
        const int s0 = lo + (nu >> 1) * kTile + (nu & 1) * kHalf + r0;
        for (int g = 0; g < G; ++g) {
          const int stage = g * kVSlots + vslot, hk = (h0 + g) / gqa;
          if (use > 0) ok = mbar_wait(bar(kBarVEmpty + stage), (use - 1) & 1);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const uint8_t* vbase = reinterpret_cast<const uint8_t*>(p.latent_v) + (int64_t)hk * p.v_stride_h;
          const uint32_t dst = sV + stage * kVSlotBytes;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const bool valid = c_on && s0 + 8 * k < hi;
            const int64_t sl = valid ? page[s0 + 8 * k] : 0;
            cp_async16(dst + doff + k * 512, vbase + (valid ? c * 16 + sl * p.v_stride_t : 0), valid ? 16u : 0u);
          }
          cp_async_arrive_noinc(bar(kBarVFull + stage));
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
    const int pr = g >> 1;
    const int row = q4 * 32 + lane;
    const bool interleaved = p.rope_layout == WSVD_ROPE_INTERLEAVED;

    // ---- B operand: P (cos coefficients) and Q (sin coefficients) of this head, f16,
    //      rows n = g*64 + r, 64 frequencies per row, 128-byte swizzle; rows r >= rank_k are zero
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
        if (r >= Rk) {
#pragma unroll
          for (int e = 0; e < 8; ++e) u0[e] = u1[e] = 0.f;
        } else if (wk_vec) {
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
      fence_proxy_async();  // also covers the zeroed digit planes
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPq));
    }

    const uint8_t* kbase = reinterpret_cast<const uint8_t*>(p.latent_k) + (int64_t)hk * p.k_stride_h;
    const __half* ksc = reinterpret_cast<const __half*>(p.k_scale) + (int64_t)hk * p.ks_stride_h;
    const __half* vsc = reinterpret_cast<const __half*>(p.v_scale) + (int64_t)hk * p.vs_stride_h;
    float2* xch = reinterpret_cast<float2*>(sm + kOffXch) + g * 8;  // [tile parity][warp]
    const uint32_t my_planes = sPl + warp * kPlaneBytes + (lane >> 4) * 128 + (lane & 15);
    // A W buffer serves the two pairs in turn and its "empty" barrier always counts 8 warp
    // arrivals: the four warps of a pair that holds a single head arrive twice each.
    const uint32_t w_empty_arrivals = (G - 2 * pr) >= 2 ? 1u : 2u;

    // running state: m_run / l_lane for the softmax denominator (reference: max z so far),
    // big_m / acc for the value sum (reference: max y so far); lanes 0..15 of warp q4 hold rank 16*q4 + lane
    float m_run = -INFINITY, l_lane = 0.f, big_m = -INFINITY, acc = 0.f, my_prev = -INFINITY;
    bool ok = true;
    const uint32_t d_addr = tmem + ((uint32_t)(q4 * 32) << 16) + kTmemD + 8 * g;
    auto fold_values = [&](float my_tile) {
      // D[rank][0..2]: the three digit-plane sums of the tile whose max y was my_tile
      uint32_t d[4];
      tmem_ld4(d_addr, d);
      tmem_wait_ld();
      if (my_tile > -INFINITY) {
        const float v = fmaf((float)(int32_t)d[2], 65536.f, fmaf((float)(int32_t)d[1], 256.f, (float)(int32_t)d[0])) *
                        (1.f / kPlaneScale);
        const float m_new = fmaxf(big_m, my_tile);
        acc = acc * fast_exp2(big_m - m_new) + v * fast_exp2(my_tile - m_new);  // big_m = -inf -> factor 0
        big_m = m_new;
      }
    };

    for (int t = 0; t < ntiles; ++t) {
      const int s = lo + t * kTile + row;
      const bool valid = s < hi;
      const int u = t * npairs + pr, wb = u % kWBufs;
      ok = warp_wait(bar(kBarWFull + wb), (u / kWBufs) & 1);
      if (!ok) break;
      tc_fence_after();

      // ---- score: dot of this token's int8 K row with its row of W, 16 ranks at a time
      const uint32_t taddr = tmem + ((uint32_t)(q4 * 32) << 16) + wb * 128 + (g & 1) * kRkMax;
      uint64_t dot[2] = {0ull, 0ull};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[16];
        tmem_ld16(taddr + c * 16, w);
        tmem_wait_ld();
        const uint4 kq = kreg[c];
        const uint32_t kws[4] = {kq.x ^ 0x80808080u, kq.y ^ 0x80808080u, kq.z ^ 0x80808080u, kq.w ^ 0x80808080u};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint64_t x01, x23;
          cvt4(kws[j], x01, x23);
          dot[0] = fma2(x01, pk(__uint_as_float(w[4 * j]), __uint_as_float(w[4 * j + 1])), dot[0]);
          dot[1] = fma2(x23, pk(__uint_as_float(w[4 * j + 2]), __uint_as_float(w[4 * j + 3])), dot[1]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_n(bar(kBarWEmpty + wb), w_empty_arrivals);  // this warp has read its rows of W
      float d0, d1;
      upk(add2(dot[0], dot[1]), d0, d1);
      const float sk = __half2float(__ushort_as_half(sk_raw)), sv = __half2float(__ushort_as_half(sv_raw));
      const float z = valid ? (d0 + d1) * sk : -INFINITY;
      const float y = (valid && sv > 0.f) ? z + fast_log2(sv) : -INFINITY;

      // ---- the K row is consumed: fetch the next tile's row, scales and the page entry after that
      {
        const int sn = s + kTile;
#pragma unroll
        for (int c = 0; c < 4; ++c) kreg[c] = make_uint4(0u, 0u, 0u, 0u);
        sk_raw = 0;
        sv_raw = 0;
        if (sn < hi) {
          const uint4* krow = reinterpret_cast<const uint4*>(kbase + (int64_t)slot_n * p.k_stride_t);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (c * 16 < Rk) kreg[c] = __ldg(krow + c);
          sk_raw = reinterpret_cast<const unsigned short*>(ksc)[(int64_t)slot_n * p.ks_stride_t];
          sv_raw = reinterpret_cast<const unsigned short*>(vsc)[(int64_t)slot_n * p.vs_stride_t];
        }
        slot_n = -1;
        if (sn + kTile < hi) slot_n = page[sn + kTile];
      }

      // ---- tile maxima of z and y over the head's 128 tokens: per warp, then through shared memory
      const float mz_w = warp_max_redux(z), my_w = warp_max_redux(y);
      if (lane == 0) {
        xch[(t & 1) * 4 + q4] = make_float2(mz_w, my_w);
        mbar_arrive(bar(kBarXch + 2 * g + (t & 1)));
      }
      ok = warp_wait(bar(kBarXch + 2 * g + (t & 1)), (t >> 1) & 1);
      if (!ok) break;
      float mz = -INFINITY, my = -INFINITY;
#pragma unroll
      for (int w4 = 0; w4 < 4; ++w4) {
        const float2 e = xch[(t & 1) * 4 + w4];
        mz = fmaxf(mz, e.x);
        my = fmaxf(my, e.y);
      }

      // ---- the previous tile's value sums are in tensor memory by now: fold them in.  This also
      //      orders every reader of D (and, through the MMA's completion, of the digit planes) before
      //      the planes of this tile are written and before its MMAs are issued.
      if (t > 0) {
        ok = warp_wait(bar(kBarDFull + g), (t - 1) & 1);
        if (!ok) break;
        tc_fence_after();
        fold_values(my_prev);
      }
      my_prev = my;

      // ---- softmax denominator (fp32, by the owner threads)
      {
        const float m_new = fmaxf(m_run, mz);  // finite: the tile holds at least one token
        l_lane = l_lane * fast_exp2(m_run - m_new) + (valid ? fast_exp2(z - m_new) : 0.f);
        m_run = m_new;
      }
      // ---- this token's weight for the value MMA as three 8-bit digits
      {
        const float w = y > -INFINITY ? fast_exp2(y - my) : 0.f;  // <= 1
        const uint32_t nq = __float2uint_rn(w * kPlaneScale);
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(my_planes), "r"(nq) : "memory");
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(my_planes + 16), "r"(nq >> 8) : "memory");
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(my_planes + 32), "r"(nq >> 16) : "memory");
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(kBarPlanes + g));
        if (q4 == 0) {
          // ---- the head's value MMAs for this tile: one per warp of 32 tokens
          ok = mbar_wait(bar(kBarPlanes + g), t & 1);
          const int n0 = 2 * t, n1 = 2 * t + 1;
          const int st0 = g * kVSlots + n0 % kVSlots, st1 = g * kVSlots + n1 % kVSlots;
          if (ok) ok = mbar_wait(bar(kBarVFull + st0), (n0 / kVSlots) & 1);
          if (ok && n1 < n_units) ok = mbar_wait(bar(kBarVFull + st1), (n1 / kVSlots) & 1);
          if (ok) {
            tc_fence_after();
            const uint32_t idesc = instr_desc_i8(64, 8);
            const uint32_t d_tmem = tmem + kTmemD + 8 * g;
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4) {
              if (w4 >= 2 && n1 >= n_units) break;
              const uint32_t va = sV + (w4 < 2 ? st0 : st1) * kVSlotBytes + (w4 & 1) * 2048;
              umma_i8(d_tmem, smem_desc_mn_sw64(va), smem_desc_k_plain(sPl + (4 * g + w4) * kPlaneBytes), idesc,
                      w4 > 0);
            }
            umma_commit(bar(kBarDFull + g));
            umma_commit(bar(kBarVEmpty + st0));
            if (n1 < n_units) umma_commit(bar(kBarVEmpty + st1));
          }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
    }
    // ---- the last tile's value sums
    if (ok) {
      ok = warp_wait(bar(kBarDFull + g), (ntiles - 1) & 1);
      if (ok) {
        tc_fence_after();
        fold_values(my_prev);
      }
    }
    if (!ok) atomicMax(&g_status, (unsigned)kTimeoutEpilogue);

    // ---- the head's denominator: sum over its four warps (all use the same reference m_run)
    const float l_w = warp_sum(l_lane);
    float* sums = reinterpret_cast<float*>(sm + kOffSum) + g * 4;
    if (lane == 0) sums[q4] = l_w;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(128) : "memory");
    const float l_tot = (sums[0] + sums[1]) + (sums[2] + sums[3]);
    const int64_t slot = ((int64_t)b * p.n_q_heads + h) * a.n_splits + split;
    const int r = 16 * q4 + lane;
    if (lane < 16 && r < Rv) {
      // sum_s 2^z sv Lv / sum_s 2^z  =  acc * 2^(big_m - m_run) / l
      const float o = big_m > -INFINITY ? acc * fast_exp2(big_m - m_run) / l_tot : 0.f;
      a.mid_o[slot * Rv + r] = o;
    }
    // natural-log lse, as the merge kernel expects (stage1.py:216)
    if (q4 == 0 && lane == 0) a.lse[slot] = m_run * 0.6931471805599453f + logf(l_tot);
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

// The V latents [T, Hkv, Rv] int8 with byte strides (st, sh) as a 3-D tensor map whose outer axes
// are ordered by stride; box = 64 bytes x 64 token slots x 1 head.  The box is wider than the
// tensor when rank_v < 64: the missing bytes arrive as zeros.
bool encode_v(CUtensorMap* map, const void* base, int64_t st, int64_t sh, int64_t T, int Hkv, int R, int* slot_axis) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || T <= 0 || T > 0xffffffffll) return false;
  const bool slot_first = st <= sh;  // head-major storage: the slot axis has the smaller stride
  cuuint64_t dims[3] = {(cuuint64_t)R, (cuuint64_t)(slot_first ? T : Hkv), (cuuint64_t)(slot_first ? Hkv : T)};
  cuuint64_t strides[2] = {(cuuint64_t)(slot_first ? st : sh), (cuuint64_t)(slot_first ? sh : st)};
  cuuint32_t box[3] = {64, (cuuint32_t)(slot_first ? kHalf : 1), (cuuint32_t)(slot_first ? 1 : kHalf)};
  cuuint32_t estr[3] = {1, 1, 1};
  *slot_axis = slot_first ? 1 : 2;
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The position table [2][rows][64] f16; box = one 128-position tile of one plane, 128-byte swizzle
// (the K-major operand layout of the score MMA).  Rows past the table read as zeros.
bool encode_table(CUtensorMap* map, const void* table, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || rows <= 0) return false;
  cuuint64_t dims[3] = {64, (cuuint64_t)rows, 2};
  cuuint64_t strides[2] = {128, (cuuint64_t)rows * 128};
  cuuint32_t box[3] = {64, (cuuint32_t)kTile, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(table), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace tc

size_t rope_table_bytes(int rows) { return (size_t)rows * 256; }

cudaError_t launch_rope_table(void* table, int rows, const KArgs& a, cudaStream_t stream) {
  const int total = rows * 64;
  tc::rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(reinterpret_cast<__half*>(table), rows, a);
  return cudaGetLastError();
}

cudaError_t launch_stage1_tc(const KArgs& a, const void* table, int table_rows, cudaStream_t stream) {
  static_assert(tc::kSmemBytes <= 232448, "shared memory budget");
  cudaError_t e = cudaFuncSetAttribute(tc::stage1_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)tc::kSmemBytes);
  if (e != cudaSuccess) return e;
  tc::TcArgs ta;
  ta.k = a;
  ta.table_rows = table_rows;
  ta.use_tma = 0;
  ta.slot_axis = 1;
  memset(&ta.tmap_v, 0, sizeof(CUtensorMap));
  if (!tc::encode_table(&ta.tmap_table, table, table_rows)) return cudaErrorInvalidValue;
  if (a.p.n_token_slots > 0) {
    int ax = 1;
    if (tc::encode_v(&ta.tmap_v, a.p.latent_v, a.p.v_stride_t, a.p.v_stride_h, a.p.n_token_slots, a.p.n_kv_heads,
                     a.p.rank_v, &ax)) {
      ta.slot_axis = ax;
      ta.use_tma = 1;
    }
  }
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

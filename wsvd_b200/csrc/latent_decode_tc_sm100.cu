// The latent decode attention on the Blackwell tensor cores (tcgen05.mma with accumulators in
// tensor memory), for head_dim 128, int8 latents, rank_k and rank_v in {16,32,48,64}: split-KV
// stage 1 and, in the balanced mode, also the merge, the U_v projection and the head all-gather.
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
// operand [P;Q] is built once per work item and stays in shared memory, the accumulator is fp32
// in tensor memory (three 128-column buffers).  Each epilogue thread owns one token: it
// reads its row of W from tensor memory and dots it in fp32 with the token's int8 K row,
// which it copied from the K ring into registers at the top of the tile (so that the ring
// slot is refilled a whole tile before its next use).
//
// Values.  O[r] = sum_s p_s sv_s Lv[s,r] is a true contraction over the tokens and runs on
// the tensor cores as an int8 MMA (kind::i8): the A operand is a quarter of the V tile exactly as
// TMA wrote it (32 tokens x 64 bytes, 64-byte swizzle = the MN-major canonical layout), the
// B operand is the tile's weights a_s = 2^(y_s - max y), y_s = z_s + log2 sv_s, written by
// their owner threads as three unsigned 8-bit digit planes of round(a_s * (2^24 - 256));
// the int32 accumulator (64 ranks x 8 columns per head) is read back once per tile and
// folded into a running fp32 sum under a running reference max(y).  The weights lose nothing
// that fp32 would keep: 24 bits relative to the largest weight of the warp's 32 tokens.  The softmax
// denominator is accumulated by the owner threads in fp32.
//
// Work.  A work item is a run of consecutive tiles of one (sequence, group of 4 heads); it ends
// in one partial result (normalised latent-space row + log-sum-exp per head) for the merge kernel.
//  - Balanced mode: all tiles of the batch, ordered by (sequence, head group, tile), are cut
//    into equal shares, one per persistent CTA (one CTA per SM).  A share covers a few items: the
//    tail of one (sequence, head group), whole ones, the head of another.  No SM idles in a
//    partial last wave whatever the sequence lengths, the [P;Q] build is paid once per item, and
//    tensor memory is allocated once.  Every CTA computes its share itself from the sequence
//    lengths (a block-wide prefix sum at the start of the kernel).  The partial of item (sequence
//    b, head group hg) of CTA c goes to slot (b * n_hg + hg + c), which is unique because along
//    the tile order every new item advances the (sequence, head group) index or the CTA index.
//    With arrival counters (one per (sequence, head), zeroed before the launch) the kernel is the
//    whole op: the CTA that completes a head's last partial merges the partials, multiplies by
//    the head's slice of U_v and writes the output row; an item that one CTA covers alone skips
//    the partials altogether.  With a peer set on top, the row goes to every rank's gathered
//    buffer (16-byte peer stores) and the CTA that exits last runs the group's barrier.  Without
//    counters the partials and the prefix sums are left for the merge kernel.
//  - Split mode (no plan): CTA blockIdx.x handles split blockIdx.x % n_splits of a fixed-length
//    split plan, partials in the [B, Hq, n_splits] layout of the reference's stage 1.
// 20 warps:
//   warps 0-15   epilogue, 4 per head: warp w owns tensor-memory lanes 32*(w%4)..+31, i.e.
//                tokens 32*(w%4).. of every tile of head w/4
//   warp 16      one thread issues the score MMAs
//   warp 17      requests the table tiles and the K and V rows
//   warps 18-19  one pair of heads each (lane 0 and lane 1 one head each): issue the value MMAs
// The 16 epilogue warps and the 4 control warps are two register groups: after the launch the
// control warpgroup gives registers back and the epilogue warpgroups take them (setmaxnreg).
// Latent rows travel in units of one tile (128 tokens) of ALL the group's heads: one TMA tensor
// copy of 32 KB (64 bytes x 128 token slots x 4 heads) when the tile's token slots are consecutive
// and the cache is head-major, else one copy per head, else a gather of rows with 16-byte
// cp.async through the page table.  In the busy SM a control thread needs 20-40 cycles per
// instruction, so waiting for a slot and issuing one copy costs 600-800 cycles whatever the size
// of the copy: with five copies per tile (half-tile units) the requesting warp, not HBM, set the
// pace of the whole kernel.  Hence few and large copies: 3 per tile and CTA (table, K, V).
// Every wait inside the tile loop is an mbarrier wait with a time limit; on a time-out the
// kernel records a status code and every role falls through to the common exit, which frees
// the tensor memory.
#include <cuda.h>
#include <string.h>

#include "common.cuh"

namespace wsvd {
namespace tc {

constexpr int kG = 4;          // heads per CTA
static_assert(kG == kBalancedGroup, "the merge kernel indexes balanced partials by groups of kG heads");
constexpr int kTile = 128;     // positions per MMA tile (= tensor-memory lanes)
constexpr int kRkMax = 64;
constexpr int kEpiWarps = 4 * kG;
constexpr int kMmaWarp = kEpiWarps;
constexpr int kProducers = 3;  // with the MMA warp they fill one warp slot per scheduler
constexpr int kThreads = (kEpiWarps + 1 + kProducers) * 32;
// Registers per thread after the two groups have re-balanced them.  The pool is the CTA's own: what
// the control warpgroup hands back, (96 - 64) * 128, is exactly what the epilogue warpgroups take,
// (104 - 96) * 512.  (A request the pool cannot satisfy would block for ever.)
constexpr int kLaunchRegs = 96;  // what 640 threads per CTA leave the compiler
constexpr int kEpiRegs = 104;
constexpr int kCtlRegs = 64;
static_assert((kLaunchRegs - kCtlRegs) * 4 * 32 >= (kEpiRegs - kLaunchRegs) * kEpiWarps * 32, "register pool");
static_assert(kProducers == 3, "the control warps must form one warpgroup (4 warps) for setmaxnreg");
constexpr int kKSlots = 1;     // tiles of K: a tile's rows are copied to registers at the top of the tile
constexpr int kVSlots = 2;     // tiles of V: the tile whose value MMAs are pending, and the next tile in flight
constexpr int kWBufs = 3;      // W accumulators of 128 columns (one pair of heads each)

constexpr uint32_t kHeadBytes = kTile * 64;         // one head's part of a unit: 128 tokens x 64 bytes (rank < 64: zero-filled)
constexpr uint32_t kUnitBytes = kG * kHeadBytes;    // a ring slot: one tile of K or V for up to 4 KV heads
constexpr uint32_t kAHalfBytes = kTile * 128;       // 128 rows x 64 f16
constexpr uint32_t kABufBytes = 2 * kAHalfBytes;    // cos half + sin half
constexpr uint32_t kBHalfBytes = kG * kRkMax * 128; // 256 rows x 64 f16
constexpr uint32_t kPlaneBytes = 256;               // per pair of warps: 2 chunks of 16 tokens x 8 rows x 16 bytes
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemD = kWBufs * 128;           // first column of the value accumulators: 8 per (head, warp)
constexpr float kPlaneScale = 16776960.f;           // 2^24 - 256: a weight of 1 is 0xFFFF00

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffB = 0;
constexpr uint32_t kOffA = kOffB + 2 * kBHalfBytes;
constexpr uint32_t kOffV = kOffA + 2 * kABufBytes;
constexpr uint32_t kOffK = kOffV + kVSlots * kUnitBytes;
constexpr uint32_t kOffPlanes = kOffK + kKSlots * kUnitBytes;
constexpr uint32_t kOffRef = kOffPlanes + (kEpiWarps / 2) * kPlaneBytes;  // [head][tile parity][warp] reference max y of the planes
constexpr uint32_t kOffSum = kOffRef + kG * 2 * 4 * 4;        // [head][warp] (max z, denominator) at the end
constexpr uint32_t kOffBar = kOffSum + kG * 4 * 8;
// barriers: V and K full/empty per ring slot, table full/empty x2, W full/empty x3, per head: D
// full, planes ready; [P;Q] ready
constexpr int kBarVFull = 0;
constexpr int kBarKFull = kBarVFull + kVSlots;
constexpr int kBarVEmpty = kBarKFull + kKSlots;
constexpr int kBarKEmpty = kBarVEmpty + kVSlots;
constexpr int kBarAFull = kBarKEmpty + kKSlots;
constexpr int kBarAEmpty = kBarAFull + 2;
constexpr int kBarWFull = kBarAEmpty + 2;
constexpr int kBarWEmpty = kBarWFull + kWBufs;
constexpr int kBarDFull = kBarWEmpty + kWBufs;
constexpr int kBarPlanes = kBarDFull + kG;
constexpr int kBarPq = kBarPlanes + kG;
constexpr int kNumBars = kBarPq + 1;
constexpr uint32_t kOffTmemSlot = kOffBar + 2 * kNumBars * 8;  // two sets of barriers, used by alternate items
constexpr uint32_t kSmemBytes = kOffTmemSlot + 16;  // the dynamic shared-memory base is 1024-byte aligned
static_assert(kOffA % 1024 == 0 && kOffV % 1024 == 0 && kOffPlanes % 256 == 0 && kOffBar % 8 == 0, "alignment");

enum Status : unsigned int { kOk = 0, kTimeoutProducer = 1, kTimeoutMma = 2, kTimeoutEpilogue = 3, kBadSmemAlignment = 4 };

__device__ unsigned int g_status = 0;

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_inval(uint32_t bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
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
constexpr uint32_t kSpinSleepNs = 32;
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
    for (int i = 0; i < 256; ++i) {
      if (mbar_try(bar, parity)) return true;
      __nanosleep(kSpinSleepNs);  // leave the issue slots to the warps this one is waiting for
    }
    if (global_ns() - t0 > 2000000000ull) return false;
  }
}
// The same for a whole warp: every lane waits, and the warp agrees on the outcome so that no
// lane leaves a loop that the others stay in.  (The epilogue's tile loop calls mbar_wait without
// the vote: its lanes run in lockstep, wait on the same barrier and read the same timer, so they
// reach the same verdict, and the three votes per tile were 1 % of the kernel's time.)
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

// Four int8 packed in `w` (already XORed with 0x80808080) -> two fp32 pairs holding the exact
// signed values: byte -> low mantissa of 2^23, then subtract 2^23 + 128.  Packed fp32 arithmetic
// (sm_100 float2 intrinsics): the compiler keeps the pairs in aligned register pairs.
__device__ __forceinline__ void cvt4(uint32_t w, float2& lo, float2& hi) {
  const uint32_t magic = 0x4B000000u;
  const float2 bias = make_float2(-8388736.f, -8388736.f);
  lo = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(w, magic, 0x7650)), __uint_as_float(__byte_perm(w, magic, 0x7651))), bias);
  hi = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(w, magic, 0x7652)), __uint_as_float(__byte_perm(w, magic, 0x7653))), bias);
}

// Byte offset, inside one head's part of a ring slot, of 16-byte chunk c of token tok (0..127):
// rows of 64 bytes with the 64-byte swizzle (chunk index XOR (tok/2)%4).
__device__ __forceinline__ uint32_t latent_off(int tok, int c) {
  return (uint32_t)(tok * 64 + ((c ^ ((tok >> 1) & 3)) << 4));
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
  int32_t use_tma;        // 0: latent rows are gathered with cp.async
  int32_t slot_axis;      // 1 or 2: which coordinate of tmap_k / tmap_v is the token slot
  int32_t box_heads;      // KV heads one tensor copy fetches: up to 4 (head-major caches), else 1
  int32_t balanced;        // 0: split mode
  int32_t* prefix_out;     // balanced mode: [batch + 2] tile prefix sums and share count for the merge kernel, or null
  unsigned int* arrivals;  // balanced mode: [batch * n_q_heads] zeroed arrival counters = merge inside this kernel, or null
  int32_t has_peers;       // with arrivals: output rows go to every rank's gathered buffer, group barrier at the end
  PeerArgs peers;
  alignas(64) CUtensorMap tmap_k;      // latents as 3-D byte tensors: box 64 bytes x 64 slots x box_heads,
  alignas(64) CUtensorMap tmap_v;      // 64-byte swizzle
  alignas(64) CUtensorMap tmap_table;  // [2][rows][64] f16, box 64 x 128 x 2 (cos and sin tile), 128-byte swizzle
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

// The walk over this CTA's work items, for the epilogue warps (kEpi) or for the four control warps.
// Two instantiations, because the two groups run with different register budgets (see the kernel):
// everything a group executes after its setmaxnreg has to be code of its own.
template <bool kEpi>
__device__ __forceinline__ void run_share(const TcArgs& ta, uint8_t* sm) {
  const KArgs& a = ta.k;
  const WsvdLatentDecodeParams& p = a.p;
  const int gqa = p.n_q_heads / p.n_kv_heads;
  const int Rk = p.rank_k, Rv = p.rank_v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_hg = (p.n_q_heads + kG - 1) / kG;

  const uint32_t sbase = smem_u32(sm);
  const uint32_t sB = sbase + kOffB, sA = sbase + kOffA, sV = sbase + kOffV, sK = sbase + kOffK;
  const uint32_t sPl = sbase + kOffPlanes;
  uint32_t bars = sbase + kOffBar;
  auto bar = [&](int i) { return bars + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + kOffTmemSlot);
  // 16-byte vector loads of wk need f16 data with 16-byte aligned rows
  const bool wk_vec = p.wk_dtype == WSVD_F16 && (p.wk_stride_r & 7) == 0 &&
                      (reinterpret_cast<uintptr_t>(p.wk) & 15) == 0;

  uint32_t tmem = 0;
  // ---- this CTA's work: every thread walks the same items (uniform loads, no broadcast needed)
  const bool balanced = ta.balanced != 0;
  const bool fused = balanced && ta.arrivals != nullptr;
  int b = 0, hg = 0, t_first = 0, tiles_left = 0, split = 0;
  int before_b = 0;     // balanced mode: tiles in the sequences before b
  int64_t total = 0;    // balanced mode: entries of the tile list
  int shares = 0;       // balanced mode: CTAs that have a share
  if (balanced) {
    // Tiles per sequence -> block-wide sums -> this CTA's share [begin, end) of the tile list and the
    // (sequence, head group, tile) it starts at.  Scratch: the reference/sum area, unused until the
    // first tile.
    int* plan_sm = reinterpret_cast<int*>(sm + kOffRef);  // [0, 20): per-warp sums; [24], [25]: start sequence, tiles before it
    constexpr int kWarps = kThreads / 32;
    auto tiles_of = [&](int i) {
      const int n = i < p.batch ? p.b_seq_len[i] : 0;
      return n > 0 ? (n + kTile - 1) / kTile : 0;
    };
    int mine = 0;
    for (int i = threadIdx.x; i < p.batch; i += kThreads) mine += tiles_of(i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) plan_sm[warp] = mine;
    __syncthreads();
    int all_tiles = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) all_tiles += plan_sm[w];
    __syncthreads();
    total = (int64_t)all_tiles * n_hg;
    shares = (int)min((int64_t)gridDim.x, total);
    const bool has_share = (int)blockIdx.x < shares;
    const int64_t begin = has_share ? share_begin(blockIdx.x, total, shares) : 0;
    if (has_share) tiles_left = (int)(share_begin(blockIdx.x + 1, total, shares) - begin);
    if (has_share || (blockIdx.x == 0 && ta.prefix_out != nullptr)) {
      int carry = 0;
      for (int base = 0; base < p.batch; base += kThreads) {
        const int i = base + threadIdx.x;
        const int v = tiles_of(i);
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += up;
        }
        if (lane == 31) plan_sm[warp] = incl;
        __syncthreads();
        int lower = 0, chunk = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const int x = plan_sm[w];
          if (w < warp) lower += x;
          chunk += x;
        }
        const int excl = carry + lower + incl - v;
        if (has_share && v > 0 && (int64_t)excl * n_hg <= begin && begin < (int64_t)(excl + v) * n_hg) {
          plan_sm[24] = i;
          plan_sm[25] = excl;
        }
        if (blockIdx.x == 0 && ta.prefix_out != nullptr && i < p.batch) ta.prefix_out[i] = excl;
        carry += chunk;
        __syncthreads();
      }
      if (blockIdx.x == 0 && ta.prefix_out != nullptr && threadIdx.x == 0) {
        ta.prefix_out[p.batch] = all_tiles;
        ta.prefix_out[p.batch + 1] = shares;
      }
      if (has_share) {
        b = plan_sm[24];
        before_b = plan_sm[25];
        const int tiles_b = tiles_of(b);
        const int64_t rem = begin - (int64_t)before_b * n_hg;
        hg = (int)(rem / tiles_b);
        t_first = (int)(rem % tiles_b);
      }
      __syncthreads();  // the scratch area is handed back
    }
    // sequences without tokens belong to no share: their output rows are zeros
    if (fused) {
      const int n_out = p.wv != nullptr ? p.head_dim : Rv;
      for (int bb = blockIdx.x; bb < p.batch; bb += gridDim.x) {
        if (p.b_seq_len[bb] > 0) continue;
        if (ta.has_peers) {
          for (int i = threadIdx.x; i < p.n_q_heads * n_out * ta.peers.n_peers; i += kThreads) {
            const int peer = i / (p.n_q_heads * n_out), j = i % (p.n_q_heads * n_out);
            ta.peers.out[peer][(int64_t)bb * ta.peers.out_stride_b +
                               (int64_t)(j / n_out + ta.peers.head_offset) * ta.peers.out_stride_h + j % n_out] =
                __float2half_rn(0.f);
          }
        } else {
          __half* orow = reinterpret_cast<__half*>(p.out) + (int64_t)bb * p.out_stride_b;
          for (int i = threadIdx.x; i < p.n_q_heads * n_out; i += kThreads)
            orow[(int64_t)(i / n_out) * p.out_stride_h + i % n_out] = __float2half_rn(0.f);
        }
      }
    }
  } else {
    split = blockIdx.x % a.n_splits, hg = (blockIdx.x / a.n_splits) % n_hg, b = blockIdx.x / (a.n_splits * n_hg);
    tiles_left = 1;
  }
  // The barriers of an item are re-made for the next one.  Two sets are used in turn, so that a set
  // is invalidated and re-initialised a whole item after its last use.
  for (int round = 0; tiles_left > 0 && b < p.batch; ++round) {
  const int req = p.b_req_idx[b];  // requested together with the length: one round trip, not two
  const int n = p.b_seq_len[b];
  int lo, hi;
  int tiles_b = 0, n_parts = 1, c_first = 0;  // balanced mode: the CTAs that share this (sequence, head group)
  if (balanced) {
    tiles_b = (n + kTile - 1) / kTile;
    const int seg = min(tiles_left, tiles_b - t_first);
    lo = t_first * kTile;
    hi = min(n, (t_first + seg) * kTile);
    tiles_left -= seg;
    const int64_t first = (int64_t)before_b * n_hg + (int64_t)hg * tiles_b;
    c_first = share_owner(first, total, shares);
    n_parts = share_owner(first + tiles_b - 1, total, shares) - c_first + 1;
  } else {
    lo = split * a.split_len;
    hi = min(n, lo + a.split_len);
    tiles_left = 0;
  }
  if (hi <= lo) break;  // an empty split writes nothing (a balanced share never holds an empty item)
  bars = sbase + kOffBar + (round & 1) * (kNumBars * 8);
  const int h0 = hg * kG;
  const int G = min(kG, p.n_q_heads - h0);
  const int npairs = (G + 1) >> 1;
  const int ntiles = (hi - lo + kTile - 1) / kTile;
  const int pos0 = (p.pos_offset != nullptr ? p.pos_offset[b] : 0) + lo;  // RoPE position of token lo

  const int32_t* page = p.req_to_token + (int64_t)req * p.rtt_stride;

  uint4 wpre[8], qpre[2];
  // requested during set-up so that their latency is hidden behind it
  int slot_n = -1;
  unsigned short sk_raw = 0, sv_raw = 0;
  int slot0 = -1;  // epilogue: token slot of this lane's first token
  int ent[4];      // requesting warp: page entries of the tile it requests next (see check_run)

  // ---- set-up of the item: barriers (MMA warp), first loads (the others).  Nothing here waits for
  //      a load: what was requested is used after the barrier, so that the barrier is reached after
  //      one round trip (the sequence length) and not after the three of the page-table look-ups.
  if constexpr (!kEpi) {
  if (warp == kMmaWarp) {
    for (int i = lane; i < kNumBars; i += 32) {
      if (round >= 2) mbar_inval(bar(i));
      uint32_t count = 1;                                    // one TMA or commit arrival
      if (i < kBarVEmpty) count = 32;                        // V/K full: one arrive per lane of the copying warp
      else if (i < kBarKEmpty) count = G;                    // V empty: one commit per head, after the head's value MMAs on the slot
      else if (i < kBarAFull) count = 4 * G;                 // K empty: every warp that copies rows out of the slot
      else if (i >= kBarWEmpty && i < kBarDFull) count = 8;  // W empty: 8 warp arrivals (see w_empty_arrivals)
      else if (i >= kBarPlanes && i < kBarPq) count = 4;     // planes ready: the head's four warps
      else if (i == kBarPq) count = 4 * G;
      mbar_init(bar(i), count);
    }
    fence_barrier_init();
  } else if (warp == kMmaWarp + 1) {
    // page entries of tile 0, for the run check that precedes the first copies
    const int s0 = lo + 4 * lane;
#pragma unroll
    for (int j = 0; j < 4; ++j) ent[j] = s0 + j < hi ? page[s0 + j] : -1;
  }
  } else {
  if (warp < 4 * G) {
    const int hk_pre = (h0 + (warp >> 2)) / gqa;
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
    // the 16 query values this thread's chunk of 8 frequencies needs (two 16-byte loads)
    {
      const bool il = p.rope_layout == WSVD_ROPE_INTERLEAVED;
      const int ic = threadIdx.x & 7;
      const __half* qp = reinterpret_cast<const __half*>(p.q) + (int64_t)b * p.q_stride_b +
                         (int64_t)(h0 + (warp >> 2)) * p.q_stride_h;
      qpre[0] = *reinterpret_cast<const uint4*>(qp + (il ? ic * 16 : ic * 8));
      qpre[1] = *reinterpret_cast<const uint4*>(qp + (il ? ic * 16 + 8 : 64 + ic * 8));
    }
    {
      // this lane's first token and its next one: page entries (the first token's scales are
      // requested once its entry is here, after the [P;Q] build)
      const int s_first = lo + (warp & 3) * 32 + lane;
      if (s_first < hi) slot0 = page[s_first];
      if (s_first + kTile < hi) slot_n = page[s_first + kTile];
    }
  }
  }
  __syncthreads();
  tc_fence_after();
  tmem = *tmem_slot;

  if constexpr (!kEpi) {
  if (warp == kMmaWarp) {
    // ================================================================= score MMAs
    if (lane == 0) {
      // descriptors: only the start-address field changes between k-steps, buffers and pairs
      const uint64_t adesc0 = smem_desc_sw128(sA), bdesc0 = smem_desc_sw128(sB);
      bool ok = mbar_wait(bar(kBarPq), 0);
      int u = 0;  // running count of (tile, pair) units: unit u uses W buffer u % kWBufs
      for (int t = 0; t < ntiles && ok; ++t) {
        const int buf = t & 1;
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
      // nothing may still be on its way to a barrier when the next item re-makes them: the releases
      // of the last two table buffers are the only arrivals nobody else waits for
      for (int t = max(0, ntiles - 2); t < ntiles && ok; ++t) ok = mbar_wait(bar(kBarAEmpty + (t & 1)), (t >> 1) & 1);
      if (!ok) atomicMax(&g_status, (unsigned)kTimeoutMma);
    }
    __syncwarp();
  } else {
    // ================================================================= copies, value MMAs
    // Latent rows travel in units of one tile (128 tokens) of all the group's KV heads; tile n uses
    // ring slot n % kKSlots (K) or n % kVSlots (V); KV head hk0 + j sits at j * kHeadBytes inside
    // the slot.  Warp 17 requests the table tiles and the K and V tiles: a K slot is free again once
    // every warp has copied its rows to registers, at the top of the tile; a V slot once every
    // head's value MMAs on it are complete.  Warps 18 and 19 each serve one pair of heads (lane 0
    // and lane 1 one head each): they wait for the digit planes of the head's four warps and issue
    // the head's value MMAs (one per warp of 32 tokens, each into its own 8 columns of tensor
    // memory); two commits then tell the epilogue warps (D full) and the requesting warp (V empty)
    // when the MMAs have completed.
    const int pw = warp - kMmaWarp - 1;
    const bool is_loader = pw == 0;
    const int hk0 = h0 / gqa, nkv = (h0 + G - 1) / gqa - hk0 + 1;  // the group's KV heads
    bool ok = true;
    // A tensor copy needs the tile's token slots to be one run of consecutive slots (true for a cache
    // laid out sequence by sequence, and for every tile inside a page of a paged cache).  The
    // requesting warp checks that tile by tile: lane l holds the page entries of tokens 4l..4l+3 of
    // the tile it will request next (fetched one tile ahead), and the warp votes.  `run_first`: the
    // slot of the tile's first token.
    int run_tile = -1, run_first = 0;
    bool run_ok = false;
    auto fetch_entries = [&](int nu) {
      const int s0 = lo + nu * kTile + 4 * lane;
#pragma unroll
      for (int j = 0; j < 4; ++j) ent[j] = (nu < ntiles && s0 + j < hi) ? page[s0 + j] : -1;
    };
    auto check_run = [&](int nu) {  // tiles are asked for in order, each at most twice in a row
      if (nu == run_tile) return;
      run_first = __shfl_sync(0xffffffffu, ent[0], 0);
      bool good = true;
#pragma unroll
      for (int j = 0; j < 4; ++j) good = good && (ent[j] < 0 || ent[j] == run_first + 4 * lane + j);
      run_ok = __all_sync(0xffffffffu, good) && ta.use_tma != 0;
      run_tile = nu;
      fetch_entries(nu + 1);
    };
    // Request tile `nu` of K (is_k) or V once its ring slot is free.
    auto load_unit = [&](int nu, bool is_k) {
      check_run(nu);
      const int nslots = is_k ? kKSlots : kVSlots;
      const int bar_full = is_k ? kBarKFull : kBarVFull, bar_empty = is_k ? kBarKEmpty : kBarVEmpty;
      const int slot = nu % nslots, use = nu / nslots;
      if (use > 0) ok = warp_wait(bar(bar_empty + slot), (use - 1) & 1);
      if (!ok) return;
      const uint32_t dst = (is_k ? sK : sV) + slot * kUnitBytes, full = bar(bar_full + slot);
      if (run_ok) {
        // one copy for all heads, or one per KV head (lane j: head hk0 + j)
        const int copies = ta.box_heads > 1 ? 1 : nkv;
        if (lane < copies) {
          const int hk = hk0 + lane, first = run_first;
          const int c1 = ta.slot_axis == 1 ? first : hk, c2 = ta.slot_axis == 1 ? hk : first;
          mbar_expect_tx(full, ta.box_heads * kHeadBytes);
          tma_load_3d(dst + lane * kHeadBytes, is_k ? &ta.tmap_k : &ta.tmap_v, 0, c1, c2, full);
        }
        if (lane == 0) mbar_arrive_n(full, 32 - copies);  // the arrivals the gather path makes lane by lane
      } else {
        // Gather through the page table, head after head: lane (r0 = lane/4, c = lane%4) copies
        // 16-byte chunk c of rows r0 + 8k to where the tensor copy would have placed it.  Rows past
        // the end and chunks past the rank are zero-filled.
        const int R = is_k ? Rk : Rv;
        const int64_t stride_t = is_k ? p.k_stride_t : p.v_stride_t, stride_h = is_k ? p.k_stride_h : p.v_stride_h;
        const uint8_t* latent = reinterpret_cast<const uint8_t*>(is_k ? p.latent_k : p.latent_v);
        const int c = lane & 3, r0 = lane >> 2;
        const bool c_on = c * 16 < R;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          const int s0 = lo + nu * kTile + half * 64 + r0;
          int64_t sl[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) sl[k] = (c_on && s0 + 8 * k < hi) ? page[s0 + 8 * k] : -1;
          for (int j = 0; j < nkv; ++j) {
            const uint8_t* base = latent + (int64_t)(hk0 + j) * stride_h;
#pragma unroll
            for (int k = 0; k < 8; ++k)
              cp_async16(dst + j * kHeadBytes + latent_off(half * 64 + r0 + 8 * k, c),
                         base + (sl[k] >= 0 ? c * 16 + sl[k] * stride_t : 0), sl[k] >= 0 ? 16u : 0u);
          }
        }
        cp_async_arrive_noinc(full);
      }
    };
    if (is_loader) {
      auto issue_table = [&](int t) {
        if (lane == 0) {
          const int buf = t & 1;
          mbar_expect_tx(bar(kBarAFull + buf), kABufBytes);
          tma_load_3d(sA + buf * kABufBytes, &ta.tmap_table, 0, pos0 + t * kTile, 0, bar(kBarAFull + buf));
        }
      };
      // start: K of tile 0, table tiles 0 and 1, V of tiles 0 and 1 (tile 0's page entries were
      // requested before the barrier)
      load_unit(0, true);
      issue_table(0);
      load_unit(0, false);
      if (ntiles > 1) {
        load_unit(1, false);
        issue_table(1);
      }
      for (int t = 0; t < ntiles && ok; ++t) {
        // In the order in which their slots come free during tile t: the table tile of t+2 (the
        // score MMAs of tile t have read its buffer), K of tile t+1 (tile t's rows were copied to
        // registers at the top of the tile), V of tile t+1 (tile t-1's value MMAs completed shortly
        // after the end of tile t-1).
        if (t + 2 < ntiles) {
          ok = warp_wait(bar(kBarAEmpty + (t & 1)), (t >> 1) & 1);
          if (!ok) break;
          issue_table(t + 2);
        }
        if (t + 1 < ntiles) load_unit(t + 1, true);
        if (t >= 1 && t + 1 < ntiles && ok) load_unit(t + 1, false);
      }
    } else if (2 * (pw - 1) < G) {
      // Value MMAs of one pair of heads: lane 0 and lane 1 one head each.
      const int g = 2 * (pw - 1) + lane;
      const bool agent = lane < 2 && g < G;
      const int sub = agent ? (h0 + g) / gqa - hk0 : 0;
      const uint32_t idesc = instr_desc_i8(64, 8);
      const uint64_t vdesc0 = smem_desc_mn_sw64(sV + sub * kHeadBytes);
      const uint64_t pdesc0 = smem_desc_k_plain(sPl + 2 * g * kPlaneBytes);
      const uint32_t d_tmem = tmem + kTmemD + 32 * g;
      for (int t = 0; t < ntiles && ok; ++t) {
        if (agent) {
          const int vslot = t % kVSlots;
          // the V rows arrive long before the planes are ready: wait for them first, off the
          // critical path from "planes ready" to "D full"
          ok = mbar_wait(bar(kBarVFull + vslot), (t / kVSlots) & 1);
          if (ok) ok = mbar_wait(bar(kBarPlanes + g), t & 1);
          if (ok) {
            tc_fence_after();
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4) {
              const uint32_t voff = vslot * kUnitBytes + w4 * 2048;  // the 32 tokens of warp w4: 32 rows of 64 bytes
              umma_i8(d_tmem + 8 * w4, vdesc0 + (voff >> 4), pdesc0 + (((w4 >> 1) * kPlaneBytes) >> 4), idesc, 0);
            }
            // completion of the MMAs tells the epilogue warps (D full) and hands the V slot back
            umma_commit(bar(kBarDFull + g));
            umma_commit(bar(kBarVEmpty + vslot));
          }
        }
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    if (!ok) atomicMax(&g_status, (unsigned)kTimeoutProducer);
  }
  } else {
  if (warp < 4 * G) {
    // ================================================================= epilogue
    const int g = warp >> 2, q4 = warp & 3;
    const int h = h0 + g, hk = h / gqa;
    const int pr = g >> 1;
    const int row = q4 * 32 + lane;
    const bool interleaved = p.rope_layout == WSVD_ROPE_INTERLEAVED;

    // ---- B operand: P (cos coefficients) and Q (sin coefficients) of this head, f16,
    //      rows n = g*64 + r, 64 frequencies per row, 128-byte swizzle; rows r >= rank_k are zero
    {
      const int tid = threadIdx.x & 127;
      // q * sm_scale * log2(e) (scores come out in the log2 domain): qlo[e] pairs with dimension
      // d0 and qhi[e] with its rotation partner d1 of frequency ic*8 + e
      float qlo[8], qhi[8];
      {
        const float qscale = a.sm_scale * 1.4426950408889634f;
        const __half* q0 = reinterpret_cast<const __half*>(&qpre[0]);
        const __half* q1 = reinterpret_cast<const __half*>(&qpre[1]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          if (interleaved) {
            const __half* src = e < 4 ? q0 : q1;
            qlo[e] = __half2float(src[(2 * e) & 7]) * qscale;
            qhi[e] = __half2float(src[(2 * e + 1) & 7]) * qscale;
          } else {
            qlo[e] = __half2float(q0[e]) * qscale;
            qhi[e] = __half2float(q1[e]) * qscale;
          }
        }
      }
      const int64_t col = (int64_t)hk * 128;
      if (wk_vec && !interleaved) {
        // Common case (f16 wk, half-split pairing): packed f16 arithmetic.  The operands are
        // rounded to f16 for the MMA anyway; forming them with one extra f16 rounding of a
        // product keeps the error of the scores within a few 1e-5.  This thread's chunk of 8
        // frequencies is the same for its four ranks, so q is converted once.
        const int ic = tid & 7;
        __half2 qa[4], qb[4], nqa[4];
        {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            qa[e] = __floats2half2_rn(qlo[2 * e], qlo[2 * e + 1]);
            qb[e] = __floats2half2_rn(qhi[2 * e], qhi[2 * e + 1]);
          }
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
          pv[e] = __float2half_rn(qlo[e] * u0[e] + qhi[e] * u1[e]);
          qv[e] = __float2half_rn(qhi[e] * u0[e] - qlo[e] * u1[e]);
        }
        const int nrow = g * 64 + r;
        const uint32_t off = nrow * 128 + ((ic ^ (nrow & 7)) << 4);
        *reinterpret_cast<uint4*>(sm + kOffB + off) = *reinterpret_cast<const uint4*>(pv);
        *reinterpret_cast<uint4*>(sm + kOffB + kBHalfBytes + off) = *reinterpret_cast<const uint4*>(qv);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPq));
    }
    if (slot0 >= 0) {
      sk_raw = reinterpret_cast<const unsigned short*>(p.k_scale)[(int64_t)hk * p.ks_stride_h + (int64_t)slot0 * p.ks_stride_t];
      sv_raw = reinterpret_cast<const unsigned short*>(p.v_scale)[(int64_t)hk * p.vs_stride_h + (int64_t)slot0 * p.vs_stride_t];
    }

    const __half* ksc = reinterpret_cast<const __half*>(p.k_scale) + (int64_t)hk * p.ks_stride_h;
    const __half* vsc = reinterpret_cast<const __half*>(p.v_scale) + (int64_t)hk * p.vs_stride_h;
    float* refs = reinterpret_cast<float*>(sm + kOffRef) + g * 8;  // [tile parity][warp]: max y the warp's planes refer to
    // Digit planes: the two warps of half a tile share one 8-row block (the MMA's B operand has 8
    // rows): rows 0..2 hold the even warp's digits, rows 3..5 the odd warp's.  Each warp's MMA reads
    // the whole block, so its columns 3..5 (or 0..2) are the other warp's weights times this warp's
    // V rows: garbage that nobody reads.  Rows 6 and 7 are never written.
    const uint32_t my_planes = sPl + (2 * g + (q4 >> 1)) * kPlaneBytes + (lane >> 4) * 128 + (q4 & 1) * 48 + (lane & 15);
    const int sub = hk - h0 / gqa;  // this head's KV head inside a unit
    // A W buffer serves the two pairs in turn and its "empty" barrier always counts 8 warp
    // arrivals: the four warps of a pair that holds a single head arrive twice each.
    const uint32_t w_empty_arrivals = (G - 2 * pr) >= 2 ? 1u : 2u;

    // Running state.  Softmax denominator: l_lane under this warp's own running max m_run of z.
    // Value sum: lanes 0..15 hold rank 16*q4 + lane of the whole head (all four warps' tokens): acc
    // under the running reference big_m (max y of every (tile, warp) folded in so far).
    float m_run = -INFINITY, l_lane = 0.f, big_m = -INFINITY, acc = 0.f;
    bool ok = true;
    const uint32_t d_addr = tmem + ((uint32_t)(q4 * 32) << 16) + kTmemD + 32 * g;
    // Fold in the value sums of tile tp: D[rank][8*w + 0..2] are the three digit-plane sums over the
    // 32 tokens of warp w, whose weights were taken relative to refs[tp & 1][w].
    auto fold_values = [&](int tp) {
      uint32_t d[4][4];
#pragma unroll
      for (int w4 = 0; w4 < 4; ++w4) tmem_ld4(d_addr + 8 * w4 + 3 * (w4 & 1), d[w4]);
      const float4 rf = *reinterpret_cast<const float4*>(refs + (tp & 1) * 4);
      const float ref[4] = {rf.x, rf.y, rf.z, rf.w};
      tmem_wait_ld();
      float m_new = big_m;
#pragma unroll
      for (int w4 = 0; w4 < 4; ++w4) m_new = fmaxf(m_new, ref[w4]);
      if (m_new > -INFINITY) {
        acc *= fast_exp2(big_m - m_new);  // big_m = -inf -> factor 0
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) {
          if (ref[w4] > -INFINITY) {  // (a warp without tokens in this tile has no MMA and reference -inf)
            // the two low digit sums are combined as integers (|d| <= 32 * 255 * 128 < 2^21)
            const float v = fmaf((float)(int32_t)d[w4][2], 65536.f,
                                 (float)((int32_t)d[w4][1] * 256 + (int32_t)d[w4][0]));
            acc = fmaf(v, fast_exp2(ref[w4] - m_new) * (1.f / kPlaneScale), acc);
          }
        }
        big_m = m_new;
      }
    };

    unsigned short sk_n = 0, sv_n = 0;
    for (int t = 0; t < ntiles; ++t) {
      const int s = lo + t * kTile + row;
      const bool valid = s < hi;
      const int u = t * npairs + pr, wb = u % kWBufs;
      // ---- the next tile's scales and the page entry of the tile after it: requested a whole
      //      tile before they are used
      sk_n = 0;
      sv_n = 0;
      if (slot_n >= 0) {
        sk_n = reinterpret_cast<const unsigned short*>(ksc)[(int64_t)slot_n * p.ks_stride_t];
        sv_n = reinterpret_cast<const unsigned short*>(vsc)[(int64_t)slot_n * p.vs_stride_t];
      }
      slot_n = -1;
      if (s + 2 * kTile < hi) slot_n = page[s + 2 * kTile];
      // ---- this warp's 32 K rows (lane = token) go from the ring slot to registers at once and
      //      the slot is handed back: its refill has the whole tile to arrive
      uint4 kreg[4];
      {
        const int kslot = t % kKSlots;
        ok = mbar_wait(bar(kBarKFull + kslot), (t / kKSlots) & 1);
        if (!ok) break;
        const uint32_t krows = sK + kslot * kUnitBytes + sub * kHeadBytes;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(kreg[c].x), "=r"(kreg[c].y), "=r"(kreg[c].z), "=r"(kreg[c].w)
                       : "r"(krows + latent_off(row, c)));
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarKEmpty + kslot));
      }
      ok = mbar_wait(bar(kBarWFull + wb), (u / kWBufs) & 1);
      if (!ok) break;
      tc_fence_after();

      // ---- score: dot of this token's int8 K row with its row of W, 16 ranks at a time
      const uint32_t taddr = tmem + ((uint32_t)(q4 * 32) << 16) + wb * 128 + (g & 1) * kRkMax;
      float2 dot0 = make_float2(0.f, 0.f), dot1 = make_float2(0.f, 0.f);
      // two 16-column loads in flight alternately: the next chunk of W travels while this one is used
      uint32_t wa[16], wb16[16];
      auto mac16 = [&](const uint32_t (&w)[16], const uint4 kq) {
        const uint32_t kws[4] = {kq.x ^ 0x80808080u, kq.y ^ 0x80808080u, kq.z ^ 0x80808080u, kq.w ^ 0x80808080u};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 x01, x23;
          cvt4(kws[j], x01, x23);
          dot0 = __ffma2_rn(x01, make_float2(__uint_as_float(w[4 * j]), __uint_as_float(w[4 * j + 1])), dot0);
          dot1 = __ffma2_rn(x23, make_float2(__uint_as_float(w[4 * j + 2]), __uint_as_float(w[4 * j + 3])), dot1);
        }
      };
      tmem_ld16(taddr, wa);
      tmem_wait_ld();
      tmem_ld16(taddr + 16, wb16);
      mac16(wa, kreg[0]);
      tmem_wait_ld();
      tmem_ld16(taddr + 32, wa);
      mac16(wb16, kreg[1]);
      tmem_wait_ld();
      tmem_ld16(taddr + 48, wb16);
      mac16(wa, kreg[2]);
      tmem_wait_ld();
      mac16(wb16, kreg[3]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_n(bar(kBarWEmpty + wb), w_empty_arrivals);  // this warp has read its rows of W
      const float2 dsum = __fadd2_rn(dot0, dot1);
      const float sk = __half2float(__ushort_as_half(sk_raw)), sv = __half2float(__ushort_as_half(sv_raw));
      const float z = valid ? (dsum.x + dsum.y) * sk : -INFINITY;
      const float y = valid ? z + fast_log2(sv) : -INFINITY;  // log2(0) = -inf: a zero scale drops the token's value
      sk_raw = sk_n;
      sv_raw = sv_n;

      // ---- softmax denominator under this warp's own running max (fp32, by the owner threads)
      const float mz_w = warp_max_redux(z), my_w = warp_max_redux(y);
      if (mz_w > -INFINITY) {
        const float m_new = fmaxf(m_run, mz_w);
        l_lane = fmaf(l_lane, fast_exp2(m_run - m_new), fast_exp2(z - m_new));  // 2^-inf = 0: m_run = -inf, masked tokens
        m_run = m_new;
      }

      // ---- the previous tile's value sums are in tensor memory by now: fold them in.  This also
      //      orders this warp's reads of D and of the references (and, through the MMAs' completion,
      //      the MMAs' reads of its digit planes) before the planes of this tile are written.
      if (t > 0) {
        ok = mbar_wait(bar(kBarDFull + g), (t - 1) & 1);
        if (!ok) break;
        tc_fence_after();
        fold_values(t - 1);
      }

      // ---- this token's weight for the value MMA, relative to the warp's largest, as three 8-bit digits
      {
        const float w = y > -INFINITY ? fast_exp2(y - my_w) : 0.f;  // <= 1
        const uint32_t nq = __float2uint_rn(w * kPlaneScale);
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(my_planes), "r"(nq) : "memory");
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(my_planes + 16), "r"(nq >> 8) : "memory");
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(my_planes + 32), "r"(nq >> 16) : "memory");
      }
      fence_proxy_async();
      tc_fence_before();
      if (lane == 0) refs[(t & 1) * 4 + q4] = my_w;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPlanes + g));
    }
    // ---- the last tile's value sums
    if (ok) {
      ok = warp_wait(bar(kBarDFull + g), (ntiles - 1) & 1);
      if (ok) {
        tc_fence_after();
        fold_values(ntiles - 1);
      }
    }
    if (!ok) atomicMax(&g_status, (unsigned)kTimeoutEpilogue);

    // ---- the head's denominator: the four warps' (max z, sum) pairs under a common maximum
    const float l_w = warp_sum(l_lane);
    float2* sums = reinterpret_cast<float2*>(sm + kOffSum) + g * 4;
    if (lane == 0) sums[q4] = make_float2(m_run, l_w);
    asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(128) : "memory");
    float m_all = -INFINITY;
#pragma unroll
    for (int w4 = 0; w4 < 4; ++w4) m_all = fmaxf(m_all, sums[w4].x);
    float l_tot = 0.f;
#pragma unroll
    for (int w4 = 0; w4 < 4; ++w4)
      if (sums[w4].x > -INFINITY) l_tot = fmaf(sums[w4].y, fast_exp2(sums[w4].x - m_all), l_tot);
    const int64_t slot = balanced ? ((int64_t)b * n_hg + hg + blockIdx.x) * kG + g
                                  : ((int64_t)b * p.n_q_heads + h) * a.n_splits + split;
    const int r = 16 * q4 + lane;
    // sum_s 2^z sv Lv / sum_s 2^z  =  acc * 2^(big_m - m_all) / l
    // (after a wait that timed out the item's result is poisoned: NaN here propagates through the
    // merge into the output row, so a time-out cannot pass for a valid result)
    const float o = !ok ? __int_as_float(0x7fc00000) : big_m > -INFINITY ? acc * fast_exp2(big_m - m_all) / l_tot : 0.f;
    const bool alone = fused && n_parts == 1;  // this CTA covered the whole (sequence, head): no partials
    if (!alone) {
      if (lane < 16 && r < Rv) a.mid_o[slot * Rv + r] = o;
      // natural-log lse, as the merge kernel expects (stage1.py:216)
      if (q4 == 0 && lane == 0) a.lse[slot] = m_all * 0.6931471805599453f + logf(l_tot);
    }
    if (fused) {
      // The head's merged latent-space row goes to shared memory (the head's digit-plane area: its
      // value MMAs are complete), then the head's 128 threads apply U_v and write the output row.
      float* o_row = reinterpret_cast<float*>(sm + kOffPlanes + 2 * g * kPlaneBytes);
      int* verdict = reinterpret_cast<int*>(sm + kOffSum) + g * 8;  // the head's (max, sum) pairs were read above
      bool finish = alone;
      if (alone) {
        if (lane < 16 && r < Rv) o_row[r] = o;
      } else {
        // the CTA that adds the head's last partial merges them all
        __threadfence();
        asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(128) : "memory");
        if (q4 == 0 && lane == 0) {
          const unsigned int seen = atomicAdd(ta.arrivals + (int64_t)b * p.n_q_heads + h, 1u);
          __threadfence();
          verdict[0] = seen + 1u == (unsigned int)n_parts;
        }
        asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(128) : "memory");
        finish = verdict[0] != 0;
        if (finish) {
          const int64_t slot0 = ((int64_t)b * n_hg + hg + c_first) * kG + g;
          const int rr = q4 * 32 + lane;  // one rank per thread of the head
          // the first four partials (a head is rarely shared by more CTAs) are requested at once
          float ls[4], mo[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            ls[i] = i < n_parts ? __ldcg(a.lse + slot0 + (int64_t)i * kG) : -INFINITY;
            mo[i] = i < n_parts && rr < Rv ? __ldcg(a.mid_o + (slot0 + (int64_t)i * kG) * Rv + rr) : 0.f;
          }
          float m = fmaxf(fmaxf(ls[0], ls[1]), fmaxf(ls[2], ls[3]));
          for (int i = 4; i < n_parts; ++i) m = fmaxf(m, __ldcg(a.lse + slot0 + (int64_t)i * kG));
          float wsum = 0.f, osum = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float w = ls[i] > -INFINITY ? __expf(ls[i] - m) : 0.f;
            wsum += w;
            osum = fmaf(w, mo[i], osum);
          }
          for (int i = 4; i < n_parts; ++i) {
            const float w = __expf(__ldcg(a.lse + slot0 + (int64_t)i * kG) - m);
            wsum += w;
            if (rr < Rv) osum = fmaf(w, __ldcg(a.mid_o + (slot0 + (int64_t)i * kG) * Rv + rr), osum);
          }
          if (rr < Rv) o_row[rr] = osum / wsum;
        }
      }
      if (finish) {
        asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(128) : "memory");
        // with peers the finished row is staged (second half of the head's plane area) and leaves as
        // 16-byte stores, one per thread per peer
        __half* stage = reinterpret_cast<__half*>(sm + kOffPlanes + 2 * g * kPlaneBytes + kPlaneBytes);
        __half* out = ta.has_peers ? stage
                                   : reinterpret_cast<__half*>(p.out) + (int64_t)b * p.out_stride_b + (int64_t)h * p.out_stride_h;
        const int d = q4 * 32 + lane;
        if (p.wv == nullptr) {
          if (d < Rv) out[d] = __float2half_rn(o_row[d]);
        } else {
          // out[d] = sum_r O_lat[r] U_v[r, hk*128 + d]: consecutive d in consecutive lanes, four sums and
          // 32 loads of U_v (L2) in flight
          const __half* w = reinterpret_cast<const __half*>(p.wv) + (int64_t)hk * p.head_dim + d;
          float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll 8
          for (int k = 0; k < Rv; k += 4) {
            y0 = fmaf(o_row[k], __half2float(__ldg(w + (int64_t)k * p.wv_stride_r)), y0);
            y1 = fmaf(o_row[k + 1], __half2float(__ldg(w + (int64_t)(k + 1) * p.wv_stride_r)), y1);
            y2 = fmaf(o_row[k + 2], __half2float(__ldg(w + (int64_t)(k + 2) * p.wv_stride_r)), y2);
            y3 = fmaf(o_row[k + 3], __half2float(__ldg(w + (int64_t)(k + 3) * p.wv_stride_r)), y3);
          }
          out[d] = __float2half_rn((y0 + y1) + (y2 + y3));
        }
        if (ta.has_peers) {
          asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(128) : "memory");
          const int chunks = (p.wv == nullptr ? Rv : p.head_dim) >> 3;
          const int64_t doff = (int64_t)b * ta.peers.out_stride_b + (int64_t)(h + ta.peers.head_offset) * ta.peers.out_stride_h;
          for (int idx = d; idx < chunks * ta.peers.n_peers; idx += 128) {
            const int peer = idx / chunks, c = idx - peer * chunks;
            *reinterpret_cast<uint4*>(ta.peers.out[peer] + doff + 8 * c) = reinterpret_cast<const uint4*>(stage)[c];
          }
        }
      }
    }
  }
  }

  // ---- end of the item: every role is done with the barriers, the rings and the tensor memory
  tc_fence_before();
  __syncthreads();
  // the next item of the share: the next head group, or the next sequence that has tokens
  t_first = 0;
  if (++hg == n_hg) {
    hg = 0;
    before_b += tiles_b;
    do ++b; while (b < p.batch && p.b_seq_len[b] <= 0);
  }
  }  // items
}

// ------------------------------------------------------------------ stage 1
__global__ void __launch_bounds__(kThreads, 1) stage1_tc_kernel(const __grid_constant__ TcArgs ta) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t sbase = smem_u32(smem_raw);
  uint8_t* sm = smem_raw;
  if ((sbase & 1023u) != 0) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicMax(&g_status, (unsigned)kBadSmemAlignment);
    return;
  }
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + kOffTmemSlot);

  // ---- once per CTA: tensor memory, descriptor prefetch
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  } else if (warp > kMmaWarp && lane == 0) {
    if (warp == kMmaWarp + 1)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&ta.tmap_table)) : "memory");
    if (ta.use_tma)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(warp == kMmaWarp + 1 ? &ta.tmap_k : &ta.tmap_v))
                   : "memory");
  }

  // ---- register budgets.  The launch gives every thread 96 registers (640 threads); the tile loop of
  //      the epilogue needs more and the control warps far fewer, so the control warpgroup hands
  //      registers back to the pool and the four epilogue warpgroups take them.
  if (warp < kEpiWarps) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpiRegs));
    run_share<true>(ta, sm);
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kCtlRegs));
    run_share<false>(ta, sm);
  }

  // ---- common exit
  tc_fence_before();
  if (ta.has_peers) __threadfence_system();  // this thread's peer stores are ordered before the count below
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(*tmem_slot, kTmemCols);
  }
  if (ta.has_peers) {
    // the group's barrier, run by whichever CTA finishes last
    volatile int* last = reinterpret_cast<volatile int*>(sm + kOffSum);
    if (threadIdx.x == 0) {
      const unsigned int done = atomicAdd(ta.peers.counter, 1u) + 1u;
      *last = done == gridDim.x;
      if (done == gridDim.x) *ta.peers.counter = 0u;  // ready for the next launch
    }
    __syncthreads();
    if (*last) peer_group_barrier(ta.peers, &g_status);
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

// One latent tensor [T, Hkv, R] int8 with byte strides (st, sh) as a 3-D tensor map whose outer
// axes are ordered by stride; box = 64 bytes x 128 token slots x `heads` KV heads (head-major caches,
// where a head's 128 rows then sit together in shared memory) or x 1 head.  The box is wider than the
// tensor when the rank is below 64, and may reach past the last head: the missing bytes arrive as zeros.
bool encode_latent(CUtensorMap* map, const void* base, int64_t st, int64_t sh, int64_t T, int Hkv, int R, int heads,
                   int* slot_axis) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || T <= 0 || T > 0xffffffffll) return false;
  const bool slot_first = st <= sh;  // head-major storage: the slot axis has the smaller stride
  if (!slot_first) heads = 1;
  cuuint64_t dims[3] = {(cuuint64_t)R, (cuuint64_t)(slot_first ? T : Hkv), (cuuint64_t)(slot_first ? Hkv : T)};
  cuuint64_t strides[2] = {(cuuint64_t)(slot_first ? st : sh), (cuuint64_t)(slot_first ? sh : st)};
  cuuint32_t box[3] = {64, (cuuint32_t)(slot_first ? kTile : 1), (cuuint32_t)(slot_first ? heads : kTile)};
  cuuint32_t estr[3] = {1, 1, 1};
  *slot_axis = slot_first ? 1 : 2;
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The position table [2][rows][64] f16; box = one 128-position tile of both planes (cos tile, then
// sin tile), 128-byte swizzle (the K-major operand layout of the score MMA).  Rows past the table
// read as zeros.
bool encode_table(CUtensorMap* map, const void* table, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || rows <= 0) return false;
  cuuint64_t dims[3] = {64, (cuuint64_t)rows, 2};
  cuuint64_t strides[2] = {128, (cuuint64_t)rows * 128};
  cuuint32_t box[3] = {64, (cuuint32_t)kTile, 2};
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

cudaError_t launch_stage1_tc(const KArgs& a, const void* table, int table_rows, const Stage1Work& work,
                             cudaStream_t stream) {
  static_assert(tc::kSmemBytes <= 232448, "shared memory budget");
  cudaError_t e = cudaFuncSetAttribute(tc::stage1_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)tc::kSmemBytes);
  if (e != cudaSuccess) return e;
  tc::TcArgs ta;
  ta.k = a;
  ta.table_rows = table_rows;
  ta.use_tma = 0;
  ta.slot_axis = 1;
  ta.box_heads = 1;
  memset(&ta.tmap_k, 0, sizeof(CUtensorMap));
  memset(&ta.tmap_v, 0, sizeof(CUtensorMap));
  if (!tc::encode_table(&ta.tmap_table, table, table_rows)) return cudaErrorInvalidValue;
  if (a.p.n_token_slots > 0) {
    // KV heads one group of 4 query heads can touch (its first head is a multiple of 4)
    const int gqa = a.p.n_q_heads / a.p.n_kv_heads;
    const int heads = gqa == 1 ? 4 : gqa == 2 ? 2 : gqa % 4 == 0 ? 1 : 2;
    int ax_k = 1, ax_v = 1;
    if (tc::encode_latent(&ta.tmap_k, a.p.latent_k, a.p.k_stride_t, a.p.k_stride_h, a.p.n_token_slots,
                          a.p.n_kv_heads, a.p.rank_k, heads, &ax_k) &&
        tc::encode_latent(&ta.tmap_v, a.p.latent_v, a.p.v_stride_t, a.p.v_stride_h, a.p.n_token_slots,
                          a.p.n_kv_heads, a.p.rank_v, heads, &ax_v) &&
        ax_k == ax_v) {
      ta.slot_axis = ax_k;
      ta.use_tma = 1;
      ta.box_heads = ax_k == 1 ? heads : 1;
    }
  }
  ta.balanced = work.n_ctas > 0;
  ta.prefix_out = work.prefix;
  ta.arrivals = work.arrivals;
  ta.has_peers = work.arrivals != nullptr && work.peers != nullptr;
  if (ta.has_peers) ta.peers = *work.peers;
  else memset(&ta.peers, 0, sizeof(ta.peers));
  const int grid = work.n_ctas > 0 ? work.n_ctas : a.n_splits * ((a.p.n_q_heads + tc::kG - 1) / tc::kG) * a.p.batch;
  if (work.n_ctas > 0 && work.arrivals != nullptr) {
    e = cudaMemsetAsync(work.arrivals, 0, sizeof(unsigned int) * (size_t)a.p.batch * a.p.n_q_heads, stream);
    if (e != cudaSuccess) return e;
  }
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

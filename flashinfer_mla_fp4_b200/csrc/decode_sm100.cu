// FP4 MLA decode for sm_100a: persistent, warp-specialised, tcgen05 + TMEM + TMA.
//
// One CTA per SM walks a contiguous range of 128-token KV tiles (common.cuh: work partition).
// For a tile of request b and a group of 64 query heads the CTA computes, with tokens on the
// MMA M axis ("swapped" orientation, so 64 heads do not waste half of a 128-row MMA):
//
//   S_lat^T [128 tok, 64 head] = K_lat (E2M1, 128x512)  . Q_lat^T(E4M3)  16 x tcgen05.mma K=32
//   S_rope^T[128 tok, 64 head] = K_rope(E4M3, 128x64)   . Q_rope^T        2 x tcgen05.mma
//   x = (scale_t * S_lat + S_rope) * softmax_scale*log2(e)              per token row, registers
//   P' = exp2(x - m_head) * scale_t, split into E4M3 hi + E4M3 lo       (two terms ~ 8 mantissa bits)
//   O^T[512 dim, 64 head] += V^T (E2M1, MN-major view of the same K_lat tile) . (P'_hi + P'_lo)
//
// The packed E2M1 latent goes from global memory to shared memory by TMA with the 4-bit tensor-map
// type that writes every 16 codes as 8 bytes of data + 8 bytes of padding: the form in which
// tcgen05.mma.kind::f8f6f4 reads 4-bit operands.  A 128-dim block of a tile is then [128 tokens][128 B]
// with the 128-byte swizzle, and the very same bytes serve as the K-major A operand of QK^T and as the
// MN-major A operand of PV: there is no conversion pass and no copy of the tile in any other format.
// (Earlier versions expanded the codes to E4M3 with eight warps; those warps competed with the softmax
// warps for issue slots and with the MMAs for shared-memory bandwidth, and were the busiest role.)
// RoPE bytes, per-token scales and Q arrive by TMA as well; pages four tiles ahead are prefetched into L2.
// The latent blocks live in a ring of ten 16 KiB blocks (two and a half tiles): a block's copy is issued as soon as the
// PV of the block ten positions earlier has completed, so the loads of a tile do not wait for the whole of the tile two
// back.  To make room for the ten blocks there is one P buffer (the softmax warps keep a tile's P' in registers until the
// PV of the previous tile has completed) and one RoPE buffer (released right after the two RoPE MMAs of a tile).
//
// Warp roles (384 threads): 0 QK^T issue, 1 TMA issue (lane i owns page i of the tile), 2 and 3 PV issue,
// two 128-dim blocks each (issue warps run warp-uniform code, one elected lane per instruction),
// 4-11 softmax / O rescale / epilogue (TMEM lane = token or dim; two warps share a lane quarter and
// split the 64 heads).
//
// Requests that are split across CTAs are merged at the end of the same kernel (tail_merge): the
// CTAs publish their partials through a flag in each slot and each takes a share of the output dims.  The two-kernel mode leaves the merge to the combine kernel instead.
//
// The per-role loops are kept small on purpose: the instruction streams share one
// instruction cache, and an MMA-issue or softmax loop that misses it starves the tensor pipe.
//
// Every wait is bounded: when a wait expires the CTA records MLA_FP4_ERR_DEVICE_TIMEOUT in the
// status words, stops issuing work, drains and exits normally.
#include <atomic>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "launch.h"
#include "ptx_sm100.cuh"

namespace mla {

namespace {

// Warp roles.  One issue warp per warp scheduler (warp id mod 4), each next to two softmax warps.
constexpr int kWarpQK = 0, kWarpTMA = 1, kWarpPV = 2, kWarpPV2 = 3;
constexpr int kWarpSoftmax0 = 4;       // 8 warps; warp & 3 is the TMEM lane quarter the warp may access
constexpr int kThreads = 384;          // 12 warps, three per scheduler
constexpr int kSoftmaxThreads = 256;   // 8 warps: warp w works on TMEM lanes 32*(w%4).. and heads 32*(w/4)..
constexpr int kSStages = 2;                // S accumulators in TMEM and per-token scale buffers
constexpr int kRing = 10;                  // latent blocks in flight: two and a half tiles
constexpr int kBlocks = 4;                 // 128-dim blocks of the latent
constexpr int kBlockBytes = kTile * 128;   // 16 KiB: [128 tokens][128 B], 128B swizzle
constexpr int kMaxSeg = 16;                // segments staged per round
constexpr float kPShift = 4.0f;            // P' = 2^(y - M + 4): keeps the E4M3 lo term out of the subnormals
constexpr float kLazyThreshold = 4.75f;    // the reference is refreshed only when beaten by 2^4.75: P' <= 2^8.75 = 430.5, just inside
                                           // E4M3 (448).  A refresh costs a CTA a tile and a half, and the CTAs that had one set the
                                           // kernel's end; at 2^4 the north-star data had eight of them, at 2^4.75 none.

// shared memory map (bytes from a 1024-aligned base)
constexpr uint32_t kOffKV = 0;                                            // [10][16384]
constexpr uint32_t kOffRope = kOffKV + kRing * kBlockBytes;               // [128][64]  64B swizzle
constexpr uint32_t kOffQLat = kOffRope + kTile * 64;                      // [4][64][128]  128B swizzle
constexpr uint32_t kOffQRope = kOffQLat + kBlocks * kGroupHeads * 128;    // [64][64]      64B swizzle
constexpr uint32_t kOffP = kOffQRope + kGroupHeads * 64;                  // [hi,lo][128][64] 64B swizzle (MN-major)
constexpr uint32_t kOffScale = kOffP + 2 * kTile * 64;                    // [2][128] f32
constexpr uint32_t kOffM = kOffScale + kSStages * kTile * 4;              // [64] f32 NEGATED reference -(M - shift)
constexpr uint32_t kOffF = kOffM + kGroupHeads * 4;                       // [64] f32 rescale factor
constexpr uint32_t kOffDelta = kOffF + kGroupHeads * 4;                   // [64] f32 how far the reference moved at its last refresh
constexpr uint32_t kOffWmax = kOffDelta + kGroupHeads * 4;                // [4][64] f32 per-warp column max / sum
constexpr uint32_t kOffLinv = kOffWmax + 4 * kGroupHeads * 4;             // [64] f32 output_scale / l
constexpr uint32_t kOffLse = kOffLinv + kGroupHeads * 4;                  // [64] f32
constexpr uint32_t kOffScMax = kOffLse + kGroupHeads * 4;                 // [8] f32 per-warp largest token scale
constexpr uint32_t kOffBars = kOffScMax + 8 * 4;                          // mbarriers (8 B each)
// barrier indices
__device__ __forceinline__ constexpr int bar_kv_full(int slot) { return slot; }            // a ring block has landed
__device__ __forceinline__ constexpr int bar_kv_empty(int slot) { return kRing + slot; }   // PV has finished with it
__device__ __forceinline__ constexpr int bar_sc_full(int s) { return 2 * kRing + s; }      // per-token scales of a tile
__device__ __forceinline__ constexpr int bar_s_full(int s) { return 2 * kRing + 2 + s; }
__device__ __forceinline__ constexpr int bar_s_empty(int s) { return 2 * kRing + 4 + s; }
constexpr int kBarRopeFull = 2 * kRing + 6, kBarRopeEmpty = 2 * kRing + 7, kBarPFull = 2 * kRing + 8, kBarPEmpty = 2 * kRing + 9,
              kBarQFull = 2 * kRing + 10, kBarQEmpty = 2 * kRing + 11, kBarOFree = 2 * kRing + 12, kBarDrain = 2 * kRing + 13,
              kBarTail = 2 * kRing + 14;
constexpr int kNumBars = 2 * kRing + 15;
constexpr uint32_t kOffTail = kOffBars + kNumBars * 8;                    // merge plan: [148] slot ids, then [64] f32 1/sum of weights
constexpr uint32_t kOffTailInv = (kOffTail + kMaxCombineSlots * 4 + 15u) & ~15u;
static_assert(kOffTailInv % 16 == 0, "read with 16-byte shared loads");
constexpr uint32_t kOffSegs = kOffTailInv + kGroupHeads * 4;              // Segment[kMaxSeg]
constexpr uint32_t kOffMisc = kOffSegs + kMaxSeg * 24;                    // tmem base, abort flag, walker
constexpr uint32_t kSmemBytes = kOffMisc + 256;
constexpr uint32_t kSmemAlloc = kSmemBytes + 1024;                        // slack for manual 1024-alignment
static_assert(sizeof(Segment) == 24, "segment staging layout");
static_assert(kSmemAlloc <= 232448, "shared memory budget exceeded");
static_assert(kOffBars % 8 == 0 && kOffSegs % 8 == 0 && kOffMisc % 8 == 0, "alignment");

// TMEM columns
constexpr uint32_t kColSLat = 0;     // + 64 * stage
constexpr uint32_t kColSRope = 128;  // + 64 * stage
constexpr uint32_t kColO = 256;      // + 64 * block

constexpr uint32_t kFmtE2M1 = 5u << 7;  // A operand format field of kind::f8f6f4 (E4M3 = 0)
constexpr uint32_t kIdescQKRope = ptx::idesc_e4m3(128, kGroupHeads, false, false);       // E4M3 x E4M3
constexpr uint32_t kIdescQK = ptx::idesc_e4m3(128, kGroupHeads, false, false) | kFmtE2M1;  // E2M1 (K tile) x E4M3 (Q)
constexpr uint32_t kIdescPV = ptx::idesc_e4m3(128, kGroupHeads, true, true) | kFmtE2M1;    // E2M1 (V^T, MN-major) x E4M3 (P)

// A split request this CTA wrote a partial for (at most two: its first and its last segment).
struct MergeReq {
  int b, g, tiles;
  int counter;    // the first CTA of the request's span
  int slot;       // the slot this CTA wrote (even: the segment was the CTA's first)
  flat_t start;   // flat tile index of the request's first tile
};
struct Misc {
  uint32_t tmem_base;
  volatile int abort;
  int nseg;   // segments staged for the current round
  int more;   // another round follows
  Walker walker;
  int n_merge;
  MergeReq merge[2];
  // the merge plan (plan_merge)
  int n_slots, n_part, rank, merge_k;
  int unit0, unit1;  // this CTA's share of every slot of the merged request: units [unit0, unit1) of 32 bytes
  int32_t gen;       // generation of this decode step, fetched once per CTA
};
static_assert(sizeof(Misc) <= 256, "misc area");

struct Ctx {
  uint32_t smem;      // shared-space address of the aligned base
  uint8_t* smem_ptr;  // generic pointer to the same
  Misc* misc;
  int32_t* status;
  uint32_t polls;     // poll budget of a bounded wait
  int32_t gen;        // generation of this decode step (flags of its partial slots carry it)
#ifdef MLA_FP4_TRACE
  int trace_cta;  // the CTA whose timeline is recorded (status word 7; the last CTA when negative)
#endif
};

// running position of a role across rounds
struct RoleState {
  uint32_t it;   // tiles processed so far by this CTA (selects stage and barrier phase)
  uint32_t seg;  // segments processed so far
  uint32_t part; // partial segments processed so far (softmax role)
  uint32_t slot, lap;  // ring block of the role's next latent block, and how many times the ring has been filled before it
  uint32_t n_rope, n_sc;  // TMA role: RoPE and scale buffers armed so far
  __device__ __forceinline__ void advance(uint32_t n) {
    slot += n;
    if (slot >= uint32_t(kRing)) { slot -= kRing; ++lap; }
  }
};

__device__ __forceinline__ uint32_t bar_addr(const Ctx& c, int idx) { return c.smem + kOffBars + 8u * idx; }
__device__ __forceinline__ const Segment* segs(const Ctx& c) { return reinterpret_cast<const Segment*>(c.smem_ptr + kOffSegs); }

// A bounded wait expired: flag the CTA (every role then stops issuing and drains) and leave a record.
__device__ __noinline__ void flag_timeout(const Ctx& c, int idx, uint32_t parity) {
  c.misc->abort = 1;
  if (c.status) {
    if (atomicCAS(c.status, 0, MLA_FP4_ERR_DEVICE_TIMEOUT) == 0) {
      c.status[1] = idx;
      c.status[2] = blockIdx.x;
      c.status[3] = threadIdx.x;
      c.status[4] = int(parity);
    }
  }
}
// Bounded wait.  Returns false (and flags the CTA) when the wait expires or the CTA is aborting.
__device__ __noinline__ bool wait_slow(const Ctx& c, int idx, uint32_t parity) {
  const uint32_t bar = bar_addr(c, idx);
#pragma unroll 1
  for (uint32_t i = 0; i < c.polls; ++i) {
    if (c.misc->abort) return false;
    if (ptx::mbar_try_wait(bar, parity)) return true;  // suspends in hardware for a while: not a hot spin
    if (i > 4096) __nanosleep(128);
  }
  flag_timeout(c, idx, parity);
  return false;
}
__device__ __forceinline__ bool wait(const Ctx& c, int idx, uint32_t parity) {
  if (ptx::mbar_try_wait(bar_addr(c, idx), parity)) return true;
  return wait_slow(c, idx, parity);
}
// One lane polls for the warp; the warp barrier orders the other lanes after its acquire.
__device__ __forceinline__ bool wait_warp(const Ctx& c, int idx, uint32_t parity) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = wait(c, idx, parity) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// Bounded wait that ignores the abort flag: lets in-flight asynchronous work land before exit.
__device__ __noinline__ void drain_wait(const Ctx& c, int idx, uint32_t parity) {
  const uint32_t bar = bar_addr(c, idx);
  const uint32_t limit = c.polls < (1u << 20) ? c.polls : (1u << 20);
#pragma unroll 1
  for (uint32_t i = 0; i < limit; ++i) {
    if (ptx::mbar_try_wait(bar, parity)) return;
    __nanosleep(64);
  }
}

__device__ __forceinline__ int ld_acquire(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed(const int32_t* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int32_t* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Optional timeline trace (debug builds only, -DMLA_FP4_TRACE): clock64 stamps of the last CTA for the
// first 16 tiles, written after the 8 status words (the status buffer must then be larger).
#ifdef MLA_FP4_TRACE
#define MLA_TRACE(role, tile, ev)                                                                      \
  do {                                                                                                 \
    if (int(blockIdx.x) == c.trace_cta && (tile) < 16u && c.status)                                                   \
      reinterpret_cast<long long*>(c.status + 8)[((role) * 16 + (tile)) * 8 + (ev)] = clock64();       \
  } while (0)
#else
#define MLA_TRACE(role, tile, ev)
#endif

// ------------------------------------------------------------------------------------------
// role: TMA issue (warp 1): Q per segment; per tile the packed latent (four blocks), RoPE bytes and scales
// ------------------------------------------------------------------------------------------
// The whole warp runs this role: lane i owns page i of the current tile (at most 16 pages of 8 tokens),
// keeps its page id in a register and issues that page's copies; lane 0 does the waits and arms the barriers.
//
// Order of a tile's copies: latent blocks 0 and 1, RoPE, scales, latent blocks 2 and 3.  That is the order in which
// their buffers come free in the steady state (blocks 0, 1 <- PV of the tile three back; RoPE <- the RoPE MMAs of
// the previous tile; scales <- the softmax of the tile two back; blocks 2, 3 <- PV of the tile two back), so a wait
// never holds up a copy whose buffer is already free.
__device__ __forceinline__ void tma_role(const DecodeParams& p, const Ctx& c, const CUtensorMap* map_q_lat,
                                         const CUtensorMap* map_q_rope, const CUtensorMap* map_rope,
                                         const CUtensorMap* map_lat, RoleState& st) {
  const int nseg = c.misc->nseg;
  const Segment* sg = segs(c);
  const int lane = threadIdx.x & 31;
  const int ppt = kTile / p.page_size;  // pages per tile
  const uint32_t page_rope_bytes = uint32_t(p.page_size) * 64u;
  const uint32_t page_scale_bytes = uint32_t(p.page_size) * 4u;
  const uint32_t page_block_bytes = uint32_t(p.page_size) * 128u;  // one 128-dim block of a page as it lies in shared memory
#pragma unroll 1
  for (int si = 0; si < nseg; ++si, ++st.seg) {
    const Segment g = sg[si];
    if (st.seg >= 1) wait_warp(c, kBarQEmpty, (st.seg - 1) & 1);
    if (lane == 0 && !c.misc->abort) {
      int qpos, head0;
      group_coords(g.g, p.num_heads, qpos, head0);
      const uint32_t bar = bar_addr(c, kBarQFull);
      ptx::mbar_arrive_expect_tx(bar, kGroupHeads * kQDim);
#pragma unroll 1
      for (int j = 0; j < kBlocks; ++j)
        ptx::tma_load_4d(c.smem + kOffQLat + j * kGroupHeads * 128, map_q_lat, bar, 128 * j, head0, qpos, g.b);
      ptx::tma_load_4d(c.smem + kOffQRope, map_q_rope, bar, kLatent, head0, qpos, g.b);
    }
    const int pages_total = (g.seq_len + p.page_size - 1) / p.page_size;
    const int32_t* bt_req = p.block_tables + size_t(g.b) * p.block_table_stride;
    // This lane's page id for a tile (never read beyond the request's pages); an id outside the pool is never turned into
    // an address: the tile's barrier then never completes and the bounded wait reports it.
    auto page_of = [&](int tile) {
      const int lp = tile * ppt + lane;
      const int id = (tile < g.tile_end && lane < ppt && lp < pages_total) ? __ldg(bt_req + lp) : -1;
      return int64_t(id) < p.num_pages ? id : -1;
    };
    // Rows are prefetched into L2 kAhead tiles ahead of their copy: HBM latency is paid there, and the copy, issued
    // when a ring block comes free, finds the rows in L2.  The 32 lanes share the lines of each page (a page is one
    // contiguous range).
    constexpr int kAhead = 4;
    auto prefetch_tile = [&](int pg_mine) {
      const uint32_t page_bytes = uint32_t(p.page_size) * kRowBytes;
#pragma unroll 1
      for (int i = 0; i < ppt; ++i) {
        const int pgi = __shfl_sync(0xffffffffu, pg_mine, i);
        if (pgi < 0) break;
        const uint8_t* base = reinterpret_cast<const uint8_t*>(p.kv_cache) + size_t(pgi) * page_bytes;
#pragma unroll 1
        for (uint32_t off = uint32_t(lane) * 128u; off < page_bytes; off += 32u * 128u)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off) : "memory");
      }
    };
    int pg = page_of(g.tile_begin), pg1 = page_of(g.tile_begin + 1), pg2 = page_of(g.tile_begin + 2), pg3 = page_of(g.tile_begin + 3);
#pragma unroll 1
    for (int t = g.tile_begin; t < g.tile_end; ++t, ++st.it) {
      const uint32_t s = st.it & 1, k = st.it >> 1;
      if (lane == 0) MLA_TRACE(1, st.it, 0);
      const int np = min(ppt, pages_total - t * ppt);
      const bool mine = pg >= 0;
      const int pg4 = page_of(t + kAhead);  // in flight while this tile is issued
      // Every CTA of the grid asks for its first tiles at the same moment, and what is asked for first arrives first:
      // nothing is prefetched while the ring fills (the copies of the first two and a half tiles go out at once anyway);
      // from the second tile on, the tile kAhead ahead is prefetched, one per tile.
      if (t != g.tile_begin) prefetch_tile(pg4);
      // The packed E2M1 latent: the tensor map's 4-bit type makes the copy write every 16 values as
      // 8 bytes of data + 8 bytes of padding, the form the MMA reads 4-bit operands in, so a block is
      // [128 tokens][128 B] with the same 128-byte swizzle as an 8-bit tile and needs no conversion pass.
      auto issue_block = [&](int j) {
        if (st.lap >= 1) wait_warp(c, bar_kv_empty(st.slot), (st.lap - 1) & 1);  // PV of the block ten positions back has completed
        if (!c.misc->abort) {
          if (lane == 0) MLA_TRACE(1, st.it, 1 + j);
          const uint32_t bar = bar_addr(c, bar_kv_full(st.slot));
          if (lane == 0) ptx::mbar_arrive_expect_tx(bar, uint32_t(np) * (page_block_bytes / 2));  // the transaction count is in packed bytes
          __syncwarp();
          if (mine)
            ptx::tma_load_3d(c.smem + kOffKV + st.slot * kBlockBytes + uint32_t(lane) * page_block_bytes, map_lat, bar, 128 * j, 0, pg);
        }
        st.advance(1);
      };
      issue_block(0);
      issue_block(1);
      // RoPE bytes: the one buffer is free once the two RoPE MMAs of the previous tile have completed
      if (st.it >= 1) wait_warp(c, kBarRopeEmpty, (st.it - 1) & 1);
      if (lane == 0) MLA_TRACE(1, st.it, 5);
      if (!c.misc->abort) {
        const uint32_t bar = bar_addr(c, kBarRopeFull);
        if (lane == 0) ptx::mbar_arrive_expect_tx(bar, uint32_t(np) * page_rope_bytes);
        __syncwarp();
        if (mine) ptx::tma_load_3d(c.smem + kOffRope + uint32_t(lane) * page_rope_bytes, map_rope, bar, kLatent / 2, 0, pg);
        ++st.n_rope;
      }
      // per-token scales: this stage was last read by the softmax of tile it-2
      if (lane == 0) MLA_TRACE(1, st.it, 6);
      if (k >= 1) wait_warp(c, bar_s_empty(s), (k - 1) & 1);
      if (lane == 0) MLA_TRACE(1, st.it, 7);
      if (!c.misc->abort) {
        const uint32_t bar = bar_addr(c, bar_sc_full(s));
        if (lane == 0) ptx::mbar_arrive_expect_tx(bar, uint32_t(np) * page_scale_bytes);
        __syncwarp();
        if (mine)
          ptx::bulk_load(c.smem + kOffScale + s * kTile * 4 + uint32_t(lane) * page_scale_bytes,
                         p.kv_cache_sf + size_t(pg) * p.page_size, page_scale_bytes, bar);
        ++st.n_sc;
      }
      issue_block(2);
      issue_block(3);
      if (c.misc->abort) break;
      pg = pg1;
      pg1 = pg2;
      pg2 = pg3;
      pg3 = pg4;
    }
  }
  if (c.misc->abort && lane == 0) {  // let copies that were issued but never consumed land before exit
    // Whatever has been armed either completes (its copies were issued) or never will (a page id was refused): a
    // bounded look at every barrier that can still be in its current phase is enough.
    for (int slot = 0; slot < kRing; ++slot) {
      const uint32_t pos = st.slot, lap = st.lap;  // next position to be filled: positions before it were armed
      const bool used = lap > 0 || uint32_t(slot) < pos;
      if (used) drain_wait(c, bar_kv_full(slot), ((uint32_t(slot) < pos ? lap : lap - 1)) & 1);
    }
    const uint32_t n_rope = st.n_rope, n_sc = st.n_sc;
    if (n_rope >= 1) drain_wait(c, kBarRopeFull, (n_rope - 1) & 1);
    if (n_sc >= 1) drain_wait(c, bar_sc_full((n_sc - 1) & 1), ((n_sc - 1) >> 1) & 1);
    if (n_sc >= 2) drain_wait(c, bar_sc_full(n_sc & 1), ((n_sc - 2) >> 1) & 1);
    if (st.seg >= 1) drain_wait(c, kBarQFull, (st.seg - 1) & 1);
  }
  __syncwarp();
}

// ------------------------------------------------------------------------------------------
// role: MMA issue (warps 0 and 2).  The whole warp runs this code with uniform control flow; only the
// tcgen05 instructions sit under elect_one(), so their operands stay in uniform registers.
// ------------------------------------------------------------------------------------------
// A shared-memory descriptor as two words.  Only the 14-bit address field (bytes >> 4) in the low word
// changes from one instruction to the next and it cannot carry out (shared memory is smaller than
// 2^18 bytes), so stepping a descriptor is ONE 32-bit add; with 64-bit descriptors the compiler has to
// propagate a carry it cannot rule out.  The issue warps share their schedulers with two busy
// compute warps each, so every instruction they do not execute shortens the tensor pipe's waits.
struct Desc {
  uint32_t lo, hi;
  __device__ __forceinline__ uint64_t at(uint32_t off16) const { return (uint64_t(hi) << 32) | uint64_t(lo + off16); }
};
__device__ __forceinline__ Desc make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  const uint64_t d = ptx::smem_desc(addr, lbo, sbo, layout);
  return Desc{uint32_t(d), uint32_t(d >> 32)};
}
// Descriptors of every operand, built once.
struct MmaDescs {
  Desc kv_k;    // K tile block, K-major, 128B swizzle          (+ ring block * 1024 + kstep*2)
  Desc kv_mn;   // same bytes as V^T, MN-major                  (+ ring block * 1024 + kstep*256)
  Desc q_lat;   // Q latent block, K-major, 128B swizzle        (+ block*512 + kstep*2)
  Desc rope;    // K rope, K-major, 64B swizzle                 (+ kstep*2)
  Desc q_rope;  // Q rope                                       (+ kstep*2)
  Desc p;       // P^T hi, MN-major, 64B swizzle                (+ lo*512 + kstep*128)
};

// QK^T of one 128-dim block of tile `it` held in ring block `slot` (4 MMAs); after the last block the commit that
// hands S to the softmax warps.  The caller has seen the operands' barriers complete.
__device__ __forceinline__ void issue_qk_block(const Ctx& c, const MmaDescs& d, uint32_t it, uint32_t j, uint32_t slot, uint32_t tmem) {
  const uint32_t s = it & 1;
  const uint32_t d_lat = tmem + kColSLat + 64u * s;
  const uint32_t a_off = slot * (kBlockBytes >> 4);
  const uint32_t b_off = j * ((kGroupHeads * 128) >> 4);
  ptx::tc_fence_after();
  if (ptx::elect_one()) {
#pragma unroll
    for (uint32_t ks = 0; ks < 4; ++ks)
      ptx::umma_f8(d_lat, d.kv_k.at(a_off + 2 * ks), d.q_lat.at(b_off + 2 * ks), kIdescQK, (j | ks) ? 1u : 0u);
    if (j == kBlocks - 1) ptx::umma_commit(bar_addr(c, bar_s_full(s)));
  }
  __syncwarp();
}
// The RoPE part of QK^T of tile `it` (2 MMAs), first in the tile: its commit frees the one RoPE buffer for the next tile.
__device__ __forceinline__ void issue_qk_rope(const Ctx& c, const MmaDescs& d, uint32_t it, uint32_t tmem) {
  const uint32_t d_rope = tmem + kColSRope + 64u * (it & 1);
  ptx::tc_fence_after();
  if (ptx::elect_one()) {
#pragma unroll
    for (uint32_t ks = 0; ks < 2; ++ks) ptx::umma_f8(d_rope, d.rope.at(2 * ks), d.q_rope.at(2 * ks), kIdescQKRope, ks);
    ptx::umma_commit(bar_addr(c, kBarRopeEmpty));
  }
  __syncwarp();
}

// PV of one 128-dim block of a tile held in ring block `slot`: 4 token steps x (hi, lo); the commit frees the ring block.
__device__ __forceinline__ void issue_pv_block(const Ctx& c, const MmaDescs& d, uint32_t j, uint32_t slot, uint32_t tmem, bool first_of_segment) {
  const uint32_t p_hi = 0, p_lo = (kTile * 64) >> 4;
  const uint32_t acc0 = first_of_segment ? 0u : 1u;
  // A = V^T block: MN-major, 128-byte swizzle; 32 tokens per step = 4 groups of 8 rows (4096 B)
  const uint32_t a_off = slot * (kBlockBytes >> 4);
  const uint32_t dd = tmem + kColO + 64u * j;
  if (ptx::elect_one()) {
#pragma unroll
    for (uint32_t ks = 0; ks < 4; ++ks) {
      // B = P^T: MN-major (64 heads contiguous), 64-byte swizzle; 32 tokens per step = 2048 B.
      // The hi and the lo term share A: it is fetched once and kept in the collector for the second.
      ptx::umma_f8_a_fill(dd, d.kv_mn.at(a_off + 256 * ks), d.p.at(p_hi + 128 * ks), kIdescPV, ks ? 1u : acc0);
      ptx::umma_f8_a_lastuse(dd, d.kv_mn.at(a_off + 256 * ks), d.p.at(p_lo + 128 * ks), kIdescPV, 1u);
    }
    ptx::umma_commit(bar_addr(c, bar_kv_empty(slot)));
  }
  __syncwarp();
}

// QK^T and PV are issued by two different warps.  Each runs straight-line code with blocking waits, so
// neither's issue latency (a few hundred cycles per block of MMAs, on one warp with no parallelism
// to hide it) delays the other; the tensor pipe serialises the two streams in hardware, and every
// data hazard between them is already covered by a barrier.
__device__ __forceinline__ MmaDescs make_descs(const Ctx& c) {
  MmaDescs d;
  d.kv_k = make_desc(c.smem + kOffKV, 16, 1024, 2);
  d.kv_mn = make_desc(c.smem + kOffKV, kBlockBytes, 1024, 2);
  d.q_lat = make_desc(c.smem + kOffQLat, 16, 1024, 2);
  d.rope = make_desc(c.smem + kOffRope, 16, 512, 4);
  d.q_rope = make_desc(c.smem + kOffQRope, 16, 512, 4);
  d.p = make_desc(c.smem + kOffP, 512, 512, 4);
  return d;
}

// role: QK^T issue (warp 0)
__device__ __forceinline__ void qk_role(const Ctx& c, uint32_t tmem, RoleState& st) {
  const MmaDescs d = make_descs(c);
  const int nseg = c.misc->nseg;
  const Segment* sg = segs(c);
#pragma unroll 1
  for (int si = 0; si < nseg; ++si, ++st.seg) {
    const uint32_t n = uint32_t(sg[si].tile_end - sg[si].tile_begin);
    bool ok = wait_warp(c, kBarQFull, st.seg & 1);
#pragma unroll 1
    for (uint32_t t = 0; t < n && ok; ++t) {
      const uint32_t it = st.it + t, s = it & 1, k = it >> 1;
      // S of this stage has been read by the softmax of tile it-2; the RoPE bytes of this tile have landed
      if (k >= 1) ok = wait_warp(c, bar_s_empty(s), (k - 1) & 1);
      ok = ok && wait_warp(c, kBarRopeFull, it & 1);
      MLA_TRACE(2, it, 0);
      if (ok) issue_qk_rope(c, d, it, tmem);
#pragma unroll
      for (uint32_t j = 0; j < kBlocks; ++j) {
        ok = ok && wait_warp(c, bar_kv_full(st.slot), st.lap & 1);
        MLA_TRACE(2, it, j == 0 ? 7 : (j == 1 ? 1 : (j == 2 ? 6 : 3)));  // block j has landed
        if (ok) issue_qk_block(c, d, it, j, st.slot, tmem);
        st.advance(1);
      }
      MLA_TRACE(2, it, 2);
    }
    // every QK^T of this segment has been issued: Q may be overwritten once they complete
    if (ptx::elect_one()) ptx::umma_commit(bar_addr(c, kBarQEmpty));
    __syncwarp();
    st.it += n;
  }
}

// role: PV issue (warps 2 and 3: two of the four 128-dim blocks each, so that the 32 MMAs of a tile are
// issued through two warp schedulers; an issue warp shares its scheduler with two compute warps)
__device__ __forceinline__ void pv_role(const Ctx& c, uint32_t tmem, RoleState& st, uint32_t part) {
  const MmaDescs d = make_descs(c);
  const int nseg = c.misc->nseg;
  const Segment* sg = segs(c);
#pragma unroll 1
  for (int si = 0; si < nseg; ++si, ++st.seg) {
    const uint32_t n = uint32_t(sg[si].tile_end - sg[si].tile_begin);
    // O^T of the previous segment has been read out
    bool ok = st.seg == 0 || wait_warp(c, kBarOFree, (st.seg - 1) & 1);
#pragma unroll 1
    for (uint32_t t = 0; t < n && ok; ++t) {
      const uint32_t it = st.it + t;
      ok = wait_warp(c, kBarPFull, it & 1);
      if (!ok) break;
      if (part == 0) MLA_TRACE(2, it, 4);
      ptx::tc_fence_after();
      if (part == 1) st.advance(2);  // this warp's blocks are the tile's third and fourth
      issue_pv_block(c, d, 2 * part, st.slot, tmem, t == 0);
      st.advance(1);
      issue_pv_block(c, d, 2 * part + 1, st.slot, tmem, t == 0);
      st.advance(1);
      if (part == 0) st.advance(2);
      // both warps' commits together tell the softmax warps that P may be overwritten
      if (ptx::elect_one()) ptx::umma_commit(bar_addr(c, kBarPEmpty));
      __syncwarp();
      if (part == 1) MLA_TRACE(2, it, 5);
    }
    st.it += n;
  }
}

// ------------------------------------------------------------------------------------------
// role: softmax / rescale / epilogue (warps 4..11, thread = TMEM lane)
// ------------------------------------------------------------------------------------------
// ---- packed FP32 pairs (sm_100 f32x2 arithmetic)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ void lds_pairs(uint32_t addr, uint64_t& p0, uint64_t& p1) {
  asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(p0), "=l"(p1) : "r"(addr) : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 lds_u32x4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 lds_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// two-term E4M3 split of a pair: hi = e4m3(v), lo = e4m3(v - hi); returns hi (16 bits), lo via reference.
// Five two-wide instructions; the softmax pass is bound by instruction issue (two warps per scheduler), and a
// split on the FMA pipe (Veltkamp) measured slower because it needs one more.
__device__ __forceinline__ uint32_t split_e4m3x2(uint64_t v2, uint32_t& lo) {
  float a, b;
  unpack2(v2, a, b);
  __half2 h = __floats2half2_rn(a, b);
  const __nv_fp8x2_storage_t hi = __nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&h), __NV_SATFINITE, __NV_E4M3);
  __half2_raw back = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
  __half2 r = __hsub2(h, *reinterpret_cast<__half2*>(&back));
  lo = __nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&r), __NV_SATFINITE, __NV_E4M3);
  return hi;
}

// Sum over the 32 lanes of 32 per-lane values held as 16 pairs; lane L ends with the total of value L.
constexpr int kHalfHeads = kGroupHeads / 2;  // heads per softmax warp
__device__ __forceinline__ float warp_transpose_sum32(uint64_t (&l2)[kHalfHeads / 2], int lane) {
  float v[kHalfHeads];
#pragma unroll
  for (int i = 0; i < kHalfHeads / 2; ++i) unpack2(l2[i], v[2 * i], v[2 * i + 1]);
#pragma unroll
  for (int o = 16, n = kHalfHeads; o > 0; o >>= 1, n >>= 1) {
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float keep = up ? v[i + n / 2] : v[i];
      const float send = up ? v[i] : v[i + n / 2];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
  }
  return v[0];
}

struct SoftmaxTile {
  uint32_t t_lat, t_rope;  // TMEM addresses of this thread's lane, S columns of the stage
  uint32_t negm;           // shared address of the negated references (-m) of this warp's 32 heads
  uint32_t p_hi, p_lo;     // shared addresses of this thread's P' rows
  uint32_t psw;            // swizzle term of the row
  uint32_t half;           // which 32 heads this warp owns
  uint64_t sc2, cs2;       // (scale_t, scale_t), (c, c)
  uint64_t cap2, rcap2;    // soft-cap variant: (cap, cap), (1/cap, 1/cap)
  bool valid;
};
// A thread's P' of one tile: 32 heads x (hi, lo) as bytes, kept in registers until the P buffer is free.
struct PRegs {
  uint32_t hi[8], lo[8];
};

// One pass over the 32 heads this thread owns of its token: e = exp2(x*c - m) and P' = e*scale_t split into two
// E4M3 terms (left in registers: the one P buffer may still be in use by the PV of the previous tile).
//
// First pass (kSecond = false), speculative, with the reference as it stands: the row sums take e, and the largest
// exponent argument seen is returned for the lazy-reference check.  An argument above kArgCap is clamped before it
// is exponentiated: a score may beat the reference by hundreds of binades (heavy-tailed token scales), 2^arg would be
// infinite and the sums lost.  Such a tile always has its reference refreshed and its P' recomputed.
//
// Second pass (kSecond = true), after a refresh that moved the reference of head h by delta_h: the caller has scaled the
// sums by f = 2^-delta, which turns every e of the first pass into its new value, (l + e_old) * f = l * f + e_new,
// except where the first pass clamped: there 2^(kArgCap - delta) went in instead of e_new, and this pass adds the difference.
//
// The pass is bound by instruction issue (two softmax warps per scheduler), so it is written for the fewest
// instructions per pair of heads; a version that collected the arguments of a chunk first measured 25 % slower.
constexpr float kArgCap = 64.f;
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float tanh_approx(float x) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// kSoftCap: the raw score x = q.k passes through cap * tanh(x / cap) first (compiled only into the soft-cap kernel).
template <bool kSecond, bool kSoftCap>
__device__ __forceinline__ float softmax_pass(const SoftmaxTile& t, uint64_t (&l2)[kHalfHeads / 2], PRegs& pr) {
  float mx = -INFINITY;
#pragma unroll
  for (int cidx = 0; cidx < 2; ++cidx) {
    uint32_t a[16], b[16];
    ptx::tmem_ld16(t.t_lat + 16 * cidx, a);
    ptx::tmem_ld16(t.t_rope + 16 * cidx, b);
    ptx::tmem_wait_ld();
    uint32_t hi16[8], lo16[8];
    if (!t.valid) {  // token beyond seq_len: weight exactly zero, whatever its row holds (its RoPE bytes may decode to NaN)
#pragma unroll
      for (int q = 0; q < 8; ++q) hi16[q] = lo16[q] = 0u;
    } else {
#pragma unroll
    for (int q = 0; q < 4; ++q) {  // 4 heads per shared load of the references
      uint64_t nm0, nm1, dl0 = 0, dl1 = 0;
      lds_pairs(t.negm + 64 * cidx + 16 * q, nm0, nm1);
      if (kSecond) lds_pairs(t.negm + (kOffDelta - kOffM) + 64 * cidx + 16 * q, dl0, dl1);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = 4 * q + 2 * h;
        uint64_t x2 = fma2(pack2u(a[i], a[i + 1]), t.sc2, pack2u(b[i], b[i + 1]));
        if (kSoftCap) {
          float x0, x1;
          unpack2(mul2(x2, t.rcap2), x0, x1);
          x2 = mul2(pack2(tanh_approx(x0), tanh_approx(x1)), t.cap2);
        }
        const uint64_t arg2 = fma2(x2, t.cs2, h ? nm1 : nm0);
        float a0, a1;
        unpack2(arg2, a0, a1);
        uint64_t e2;
        if (!kSecond) {
          mx = max3(mx, a0, a1);
          e2 = pack2(ptx::ex2(fminf(a0, kArgCap)), ptx::ex2(fminf(a1, kArgCap)));
          l2[8 * cidx + 2 * q + h] = add2(l2[8 * cidx + 2 * q + h], e2);
        } else {
          const float e0 = ptx::ex2(a0), e1 = ptx::ex2(a1);
          e2 = pack2(e0, e1);
          float d0, d1;
          unpack2(h ? dl1 : dl0, d0, d1);
          const float c0 = (a0 + d0 > kArgCap) ? e0 - ptx::ex2(kArgCap - d0) : 0.f;
          const float c1 = (a1 + d1 > kArgCap) ? e1 - ptx::ex2(kArgCap - d1) : 0.f;
          l2[8 * cidx + 2 * q + h] = add2(l2[8 * cidx + 2 * q + h], pack2(c0, c1));
        }
        hi16[2 * q + h] = split_e4m3x2(mul2(e2, t.sc2), lo16[2 * q + h]);
      }
    }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      pr.hi[4 * cidx + q] = hi16[2 * q] | (hi16[2 * q + 1] << 16);
      pr.lo[4 * cidx + q] = lo16[2 * q] | (lo16[2 * q + 1] << 16);
    }
  }
  return mx;
}
// Write a thread's P' row (32 of the 64 heads, hi and lo) to the swizzled P buffer.
__device__ __forceinline__ void store_p(const SoftmaxTile& t, const PRegs& pr) {
#pragma unroll
  for (int cidx = 0; cidx < 2; ++cidx) {
    const uint32_t off = (((2 * t.half + uint32_t(cidx)) ^ t.psw) << 4);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(t.p_hi + off), "r"(pr.hi[4 * cidx]), "r"(pr.hi[4 * cidx + 1]),
                 "r"(pr.hi[4 * cidx + 2]), "r"(pr.hi[4 * cidx + 3]) : "memory");
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(t.p_lo + off), "r"(pr.lo[4 * cidx]), "r"(pr.lo[4 * cidx + 1]),
                 "r"(pr.lo[4 * cidx + 2]), "r"(pr.lo[4 * cidx + 3]) : "memory");
  }
}

// Refresh the per-head reference: column max of y = x*c + log2(scale_t) over the tile's tokens,
// m = max(m_old, colmax - shift); f = 2^(m_old - m) (0 when there was no reference yet).
template <bool kSoftCap>
__device__ __noinline__ void refresh_reference(const Ctx& c, uint32_t t_lat, uint32_t t_rope, float sc, bool valid,
                                               float cscale, float lg, bool have_m, int tid, float cap) {
  const float rcap = kSoftCap ? 1.f / cap : 0.f;
  const int warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3, half = warp >> 2;  // t_lat / t_rope already point at this warp's 32 columns
  const uint32_t wred = c.smem + kOffWmax;
#pragma unroll 1
  for (int cidx = 0; cidx < 2; ++cidx) {
    uint32_t a[16], b[16];
    ptx::tmem_ld16(t_lat + 16 * cidx, a);
    ptx::tmem_ld16(t_rope + 16 * cidx, b);
    ptx::tmem_wait_ld();
    float mine = -INFINITY;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float x = fmaf(__uint_as_float(a[i]), sc, __uint_as_float(b[i]));
      if (kSoftCap) x = cap * tanh_approx(x * rcap);
      const float y = fmaf(x, cscale, lg);
      const float r = ptx::redux_max_f32(valid ? y : -INFINITY);
      if ((lane & 15) == i) mine = r;
    }
    if (lane < 16) sts_f32(wred + 4 * (quarter * kGroupHeads + 32 * half + 16 * cidx + lane), mine);
  }
  ptx::bar_sync(1, kSoftmaxThreads);
  if (tid < kGroupHeads) {
    float mnew = fmaxf(fmaxf(lds_f32(wred + 4 * tid), lds_f32(wred + 4 * (kGroupHeads + tid))),
                       fmaxf(lds_f32(wred + 4 * (2 * kGroupHeads + tid)), lds_f32(wred + 4 * (3 * kGroupHeads + tid)))) - kPShift;
    const float mold = have_m ? -lds_f32(c.smem + kOffM + 4 * tid) : -INFINITY;
    mnew = fmaxf(mnew, mold);
    sts_f32(c.smem + kOffF + 4 * tid, have_m ? ptx::ex2(mold - mnew) : 0.f);
    sts_f32(c.smem + kOffDelta + 4 * tid, have_m ? mnew - mold : 0.f);
    sts_f32(c.smem + kOffM + 4 * tid, -mnew);
  }
  ptx::bar_sync(1, kSoftmaxThreads);
}

// O^T *= f per head column, in TMEM (all four 128-dim blocks of this thread's lane)
__device__ __noinline__ void rescale_output(const Ctx& c, uint32_t tmem_lane, uint32_t half) {
#pragma unroll 1
  for (int jc = 0; jc < kBlocks * 2; ++jc) {
    uint32_t o[16];
    const uint32_t col = 64u * (jc >> 1) + 32u * half + 16u * (jc & 1);
    const uint32_t ta = tmem_lane + kColO + col;
    ptx::tmem_ld16(ta, o);
    ptx::tmem_wait_ld();
    const uint32_t f = c.smem + kOffF + 4 * (col & 63);
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * lds_f32(f + 4 * i));
    ptx::tmem_st16(ta, o);
  }
  ptx::tmem_wait_st();
}

// Normalise O^T and write it: to the output tensor (slot < 0) or to a split-KV partial slot.
// Runs once per segment, so its instructions are fetched cold: rolled loops over (block, 16 heads), a small body.
// Normalise O^T and write it to the output tensor (a segment that covers its request).  Runs once per segment, so
// its instructions are fetched cold, and a workload of many short requests runs it between every few tiles: rolled
// loops over (block, 16 heads), a small body (unrolled four times it slowed the variable-length workload by 10 %).
// One instantiation per output type and for a full group of 64 heads (no per-head predicates: half the instructions):
// a call fetches the instructions of its own form only.
template <int kOutDtype, bool kAllHeads>
__device__ __noinline__ void write_final(const DecodeParams& p, const Ctx& c, uint32_t tmem_lane, int row, int half,
                                         int tid, int b, int g) {
  int qpos, head0;
  group_coords(g, p.num_heads, qpos, head0);
  const int heads_here = min(kGroupHeads, p.num_heads - head0);
  const size_t row0 = (size_t(b) * p.q_len + qpos) * p.num_heads + head0;
  constexpr uint32_t esz = kOutDtype == MLA_FP4_OUT_F32 ? 4u : (kOutDtype == MLA_FP4_OUT_BF16 ? 2u : 1u);
#pragma unroll 1
  for (int jb = 0; jb < kBlocks; ++jb) {  // a block of 128 dims: this thread's 32 heads as two TMEM loads in flight together
    uint32_t o[2][16];
    ptx::tmem_ld16(tmem_lane + kColO + 64u * uint32_t(jb) + uint32_t(32 * half), o[0]);
    ptx::tmem_ld16(tmem_lane + kColO + 64u * uint32_t(jb) + uint32_t(32 * half + 16), o[1]);
    const int dim = 128 * jb + row;
    ptx::tmem_wait_ld();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int h0 = 32 * half + 16 * hh;
      char* dst = static_cast<char*>(p.out) + ((row0 + h0) * kLatent + dim) * esz;
#pragma unroll
      for (int q = 0; q < 4; ++q) {  // output_scale / l of four heads per shared load
        const float4 f = lds_f32x4(c.smem + kOffLinv + 4 * (h0 + 4 * q));
        const float fs[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = 4 * q + e;
          if (kAllHeads || h0 + i < heads_here) {
            const float v = __uint_as_float(o[hh][i]) * fs[e];
            char* d = dst + size_t(i) * kLatent * esz;
            if (kOutDtype == MLA_FP4_OUT_BF16) *reinterpret_cast<__nv_bfloat16*>(d) = __float2bfloat16_rn(v);
            else if (kOutDtype == MLA_FP4_OUT_F32) *reinterpret_cast<float*>(d) = v;
            else *reinterpret_cast<uint8_t*>(d) = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
          }
        }
      }
    }
  }
  if (p.lse && tid < heads_here) p.lse[row0 + tid] = lds_f32(c.smem + kOffLse + 4 * tid);
}

// Normalise O^T and write it to a split-KV partial slot, as fp16 divided by the slot scale.  A block of 128 dims per
// round: this thread's 32 heads as two TMEM loads.  The loads of the next block are in flight while this one is
// scaled, converted and stored (a round is bound by the latencies of load -> convert -> store, not by their amounts:
// 64 registers of buffer buy the overlap).
__device__ __noinline__ void write_partial(const DecodeParams& p, const Ctx& c, uint32_t tmem_lane, int row, int half,
                                           int tid, int slot, float slot_scale_v) {
  __half* so = reinterpret_cast<__half*>(slot_o(p.workspace, slot));
  const float post = 1.f / slot_scale_v;  // a partial is stored divided by its slot scale
  // Two blocks per round of a rolled loop (this runs once per partial: unrolled four times its instructions took
  // longer to fetch than the overlap saved).
  uint32_t o[2][2][16];
  ptx::tmem_ld16(tmem_lane + kColO + uint32_t(32 * half), o[0][0]);
  ptx::tmem_ld16(tmem_lane + kColO + uint32_t(32 * half + 16), o[0][1]);
  auto convert_store = [&](const uint32_t (&ob)[2][16], int jb) {
    const int dim = 128 * jb + row;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int h0 = 32 * half + 16 * hh;
      uint32_t pk[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {  // output_scale / l of four heads per shared load
        const float4 f = lds_f32x4(c.smem + kOffLinv + 4 * (h0 + 4 * q));
        __half2 a = __floats2half2_rn(__uint_as_float(ob[hh][4 * q]) * (f.x * post), __uint_as_float(ob[hh][4 * q + 1]) * (f.y * post));
        __half2 b2 = __floats2half2_rn(__uint_as_float(ob[hh][4 * q + 2]) * (f.z * post), __uint_as_float(ob[hh][4 * q + 3]) * (f.w * post));
        pk[2 * q] = *reinterpret_cast<uint32_t*>(&a);
        pk[2 * q + 1] = *reinterpret_cast<uint32_t*>(&b2);
      }
      // the warp's 32 dims x 8 heads are 512 contiguous bytes of the slot
      *reinterpret_cast<uint4*>(so + slot_o_index(dim, h0)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      *reinterpret_cast<uint4*>(so + slot_o_index(dim, h0 + 8)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    }
  };
#pragma unroll 1
  for (int jp = 0; jp < kBlocks / 2; ++jp) {
    if (tid == 0) MLA_TRACE(10, uint32_t(2 * jp), 0);
    ptx::tmem_wait_ld();
    ptx::tmem_ld16(tmem_lane + kColO + 64u * uint32_t(2 * jp + 1) + uint32_t(32 * half), o[1][0]);
    ptx::tmem_ld16(tmem_lane + kColO + 64u * uint32_t(2 * jp + 1) + uint32_t(32 * half + 16), o[1][1]);
    convert_store(o[0], 2 * jp);
    ptx::tmem_wait_ld();
    if (jp + 1 < kBlocks / 2) {
      ptx::tmem_ld16(tmem_lane + kColO + 64u * uint32_t(2 * jp + 2) + uint32_t(32 * half), o[0][0]);
      ptx::tmem_ld16(tmem_lane + kColO + 64u * uint32_t(2 * jp + 2) + uint32_t(32 * half + 16), o[0][1]);
    }
    convert_store(o[1], 2 * jp + 1);
  }
  if (tid == 0) MLA_TRACE(10, 4u, 0);
  if (tid < kGroupHeads) {
    slot_lse(p.workspace, slot)[tid] = lds_f32(c.smem + kOffLse + 4 * tid);
    if (tid == 0) slot_scale(p.workspace, slot)[0] = slot_scale_v;
  }
}

template <bool kSoftCap>
__device__ __forceinline__ void softmax_role(const DecodeParams& p, const Ctx& c, uint32_t tmem, int tid, RoleState& st) {
  const int nseg = c.misc->nseg;
  const Segment* sg = segs(c);
  const int warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3;           // TMEM lane quarter this warp may access
  const int half = warp >> 2;             // heads [32*half, 32*half + 32)
  const int row = quarter * 32 + lane;    // token of the tile (S) / dim of the block (O) of this thread
  const uint32_t tmem_lane = tmem + ((uint32_t(quarter) * 32u) << 16);
  const float cscale = p.softmax_scale * kLog2e;
  SoftmaxTile t;
  t.negm = c.smem + kOffM + 4 * kHalfHeads * half;
  t.cs2 = pack2(cscale, cscale);
  const float cap = kSoftCap ? p.soft_cap : 0.f;
  t.cap2 = pack2(cap, cap);
  t.rcap2 = pack2(kSoftCap ? 1.f / cap : 0.f, kSoftCap ? 1.f / cap : 0.f);
  t.psw = (uint32_t(row) >> 1) & 3u;
  t.half = uint32_t(half);
  int pending0 = 0, pending1 = 0, n_pending = 0;  // slots of the partials written in this call, published together at its end

#pragma unroll 1
  for (int si = 0; si < nseg; ++si, ++st.seg) {
    const Segment g = sg[si];
    uint64_t l2[kHalfHeads / 2];
#pragma unroll
    for (int h = 0; h < kHalfHeads / 2; ++h) l2[h] = 0ull;
    float sc_max = 0.f;  // largest |token scale| this thread has seen in the segment
#pragma unroll 1
    for (int tt = g.tile_begin; tt < g.tile_end; ++tt, ++st.it) {
      const uint32_t it = st.it;
      const uint32_t s = it & 1, k = it >> 1;
      const bool first = tt == g.tile_begin;
      if (tid == 0) MLA_TRACE(0, it, 0);
      // per-token scale
      wait(c, bar_sc_full(s), k & 1);
      t.valid = (tt * kTile + row) < g.seq_len;
      float sc = lds_f32(c.smem + kOffScale + 4 * (s * kTile + row));
      sc = t.valid ? sc : 0.f;
      sc_max = fmaxf(sc_max, fabsf(sc));
      const float lg = t.valid ? __log2f(fmaxf(fabsf(sc), 8.67361738e-19f)) : 0.f;  // floor 2^-60
      t.sc2 = pack2(sc, sc);
      t.t_lat = tmem_lane + kColSLat + 64u * s + uint32_t(kHalfHeads * half);
      t.t_rope = tmem_lane + kColSRope + 64u * s + uint32_t(kHalfHeads * half);
      t.p_hi = c.smem + kOffP + uint32_t(row) * 64u;
      t.p_lo = t.p_hi + kTile * 64;

      wait(c, bar_s_full(s), k & 1);
      if (tid == 0) MLA_TRACE(0, it, 1);
      ptx::tc_fence_after();

      // first tile of a segment: set the reference before anything is exponentiated
      if (first) refresh_reference<kSoftCap>(c, t.t_lat, t.t_rope, sc, t.valid, cscale, lg, false, tid, cap);
      if (tid == 0) MLA_TRACE(0, it, 2);

      // Speculative pass with the current reference.  It stands unless some score beat the
      // reference by more than the lazy threshold (P' would leave the E4M3 range).
      PRegs pr;
      const float mx = softmax_pass<false, kSoftCap>(t, l2, pr);
      const bool need = t.valid && (mx + lg > kPShift + kLazyThreshold);
      const bool refresh = ptx::bar_or(1, kSoftmaxThreads, need);
      if (refresh) {
        // Refresh the reference.  (l + e_old) * f equals l * f + e_new, so the row sums only need
        // the factor; O^T is rescaled in TMEM; P' is recomputed with the new reference.
        refresh_reference<kSoftCap>(c, t.t_lat, t.t_rope, sc, t.valid, cscale, lg, true, tid, cap);
#pragma unroll
        for (int q = 0; q < kHalfHeads / 4; ++q) {
          uint64_t f0, f1;
          lds_pairs(c.smem + kOffF + 4 * kHalfHeads * half + 16 * q, f0, f1);
          l2[2 * q] = mul2(l2[2 * q], f0);
          l2[2 * q + 1] = mul2(l2[2 * q + 1], f1);
        }
        (void)softmax_pass<true, kSoftCap>(t, l2, pr);
      }
      if (tid == 0) MLA_TRACE(0, it, 3);
      ptx::tc_fence_before();  // orders the S reads before the arrive
      ptx::mbar_arrive(bar_addr(c, bar_s_empty(s)));
      // The one P buffer (and, for a rescale, O^T) is free once the PV of the previous tile has completed; until then
      // this tile's P' stays in registers.
      if (it >= 1) wait(c, kBarPEmpty, (it - 1) & 1);
      if (refresh && !first) {  // O^T holds earlier tiles of the segment: rescale it
        ptx::tc_fence_after();
        rescale_output(c, tmem_lane, uint32_t(half));
        ptx::tc_fence_before();
      }
      store_p(t, pr);
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(bar_addr(c, kBarPFull));
      if (tid == 0) MLA_TRACE(0, it, 5);
    }

    // ---- segment epilogue
    {
      const uint32_t lit = st.it - 1;  // last tile of the segment
      const float r = warp_transpose_sum32(l2, lane);  // lane L: this warp's tokens, head 32*half + L
      const uint32_t wred = c.smem + kOffWmax;
      sts_f32(wred + 4 * (quarter * kGroupHeads + kHalfHeads * half + lane), r);
      const float sc_warp = ptx::redux_max_f32(sc_max);
      if (lane == 0) sts_f32(c.smem + kOffScMax + 4 * warp, sc_warp);
      ptx::bar_sync(1, kSoftmaxThreads);
      if (tid < kGroupHeads) {
        const float L = (lds_f32(wred + 4 * tid) + lds_f32(wred + 4 * (kGroupHeads + tid))) +
                        (lds_f32(wred + 4 * (2 * kGroupHeads + tid)) + lds_f32(wred + 4 * (3 * kGroupHeads + tid)));
        float m = -lds_f32(c.smem + kOffM + 4 * tid);
        float Ls = L, fo = 1.f;
        if (p.sink && g.tile_begin == 0) {  // the sink: a virtual token with a zero value row, counted with the first tile of a request
          int qpos, head0;
          group_coords(g.g, p.num_heads, qpos, head0);
          if (head0 + tid < p.num_heads) {
            const float sk = __ldg(p.sink + head0 + tid) * kLog2e;
            const float mm = fmaxf(m, sk);
            fo = ptx::ex2(m - mm);  // the reference may lie far below the sink: fold it into the output factor, not into L
            Ls = L * fo + ptx::ex2(sk - mm);
            m = mm;
          }
        }
        sts_f32(c.smem + kOffLinv + 4 * tid, p.output_scale * fo / Ls);
        sts_f32(c.smem + kOffLse + 4 * tid, __log2f(Ls) + m);
      }
      ptx::bar_sync(1, kSoftmaxThreads);
      // wait for the PV of the last tile
      wait(c, kBarPEmpty, lit & 1);
      ptx::tc_fence_after();
      float sc_all = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kSoftmaxThreads / 32; ++w8) sc_all = fmaxf(sc_all, lds_f32(c.smem + kOffScMax + 4 * w8));
      const float slot_scale_v = slot_scale_for(6.f * sc_all * fabsf(p.output_scale));
      if (tid == 0) MLA_TRACE(0, lit, 7);
      if (!c.misc->abort) {
        if (g.slot >= 0) write_partial(p, c, tmem_lane, row, half, tid, g.slot, slot_scale_v);
        else if ((p.num_heads & (kGroupHeads - 1)) == 0) {  // every group is full
          if (p.out_dtype == MLA_FP4_OUT_BF16) write_final<MLA_FP4_OUT_BF16, true>(p, c, tmem_lane, row, half, tid, g.b, g.g);
          else if (p.out_dtype == MLA_FP4_OUT_F32) write_final<MLA_FP4_OUT_F32, true>(p, c, tmem_lane, row, half, tid, g.b, g.g);
          else write_final<MLA_FP4_OUT_E4M3, true>(p, c, tmem_lane, row, half, tid, g.b, g.g);
        } else {
          if (p.out_dtype == MLA_FP4_OUT_BF16) write_final<MLA_FP4_OUT_BF16, false>(p, c, tmem_lane, row, half, tid, g.b, g.g);
          else if (p.out_dtype == MLA_FP4_OUT_F32) write_final<MLA_FP4_OUT_F32, false>(p, c, tmem_lane, row, half, tid, g.b, g.g);
          else write_final<MLA_FP4_OUT_E4M3, false>(p, c, tmem_lane, row, half, tid, g.b, g.g);
        }
      }
      if (tid == 0) MLA_TRACE(0, lit, 4);
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar_addr(c, kBarOFree));
      if (g.slot >= 0) {  // a partial: published (below) once this CTA has written all its partials of the round
        if (p.fused_merge && n_pending < 2) {
          if (n_pending == 0) pending0 = g.slot;
          else pending1 = g.slot;
          ++n_pending;
        }
        ++st.part;
      }
      if (tid == 0) MLA_TRACE(0, lit, 6);
    }
  }
  // Publish the partials: the tail merge of their requests' CTAs waits for these flags.  One fence for
  // all of them, after the last segment: a fence in the middle would hold up the next segment's first tile,
  // and nobody can use a partial before this CTA, itself a writer of the later request, is done anyway.
  if (n_pending > 0) {
#ifdef MLA_FP4_FENCE_ALL
    __threadfence();
#endif
    // One release for the whole CTA: the barrier orders every thread's stores before thread 0's release, and a release is
    // cumulative (a fence by each of the 256 threads before the barrier measured no better).
    ptx::bar_sync(1, kSoftmaxThreads);
    if (tid == 0) {
      st_release(slot_flag(p.workspace, pending0), c.gen);
      if (n_pending > 1) st_release(slot_flag(p.workspace, pending1), c.gen);
      MLA_TRACE(3, 2u, 0);
#ifdef MLA_FP4_TRACE
      if (c.status) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        (reinterpret_cast<unsigned long long*>(c.status + 8) + 12 * 16 * 8 + 4 * blockIdx.x)[3] = t;
      }
#endif
    }
  }
}

// Stage up to kMaxSeg segments of this CTA's walk into shared memory (one thread).
__device__ __noinline__ void stage_segments(const Ctx& c) {
  Walker w = c.misc->walker;
  Segment* out = reinterpret_cast<Segment*>(c.smem_ptr + kOffSegs);
  int n = 0;
  Segment s;
  bool more = false;
  while (n < kMaxSeg) {
    if (!w.next(s)) break;
    out[n++] = s;
    if (s.slot >= 0 && c.misc->n_merge < 2) {
      MergeReq& m = c.misc->merge[c.misc->n_merge++];
      m.b = s.b;
      m.g = s.g;
      m.tiles = vtiles_of(s.seq_len);       // of the flat space: phantom tiles included
      m.start = w.f - flat_t(w.t);          // w.f and w.t are the flat and the in-request position just past this segment
      m.counter = cta_of_tile(w.Tt, int(gridDim.x), m.start);
      m.slot = s.slot;
    }
  }
  if (n == kMaxSeg) {  // is there anything left?
    Walker probe = w;
    more = probe.next(s);
  }
  c.misc->walker = w;
  c.misc->nseg = n;
  c.misc->more = more ? 1 : 0;
}

// ------------------------------------------------------------------------------------------
// tail: merge of the split-KV partials inside the decode kernel
// ------------------------------------------------------------------------------------------
// Every CTA that wrote a partial of a split request stamps the slot's flag (the last words of the slot)
// with the generation of this step.  In the tail, the CTAs whose partial of a request was their
// first segment merge it, each a share of the 512 output dims: thread i watches the flag of the
// request's i-th slot and, the moment it is up, starts bulk copies of that slot's LSEs and of this
// CTA's share of its rows into shared memory (the main loop's buffers are idle by now).  The slots
// therefore stream in as their writers finish; what is left after the last writer is one copy and one
// pass over shared memory:  out = sum_i w_i * O_i  with  w_i = 2^(lse_i - max) / sum * slot scale,
// accumulated in slot order whatever the order of arrival (bit-reproducible).  A CTA has published
// everything it will ever publish before it waits for anybody else, so the waits cannot form a cycle;
// the launch is cooperative, so every CTA of the grid is resident; the waits are bounded like all others.
constexpr uint32_t kTailLseBytes = uint32_t(kSlotTailBytes);            // a slot's tail: 64 LSEs, the slot scale, the flag, padding
constexpr uint32_t kTailStage = kOffKV;                                 // staging: [slots][this CTA's bytes of a slot], then the tails
constexpr uint32_t kTailStageBytes = kOffScale - kOffKV;                // the KV ring, the RoPE stages, Q and P
static_assert(kTailStageBytes >= 2 * kSlotOBytes + 4 * kTailLseBytes, "two whole slots fit (a request cut once)");
static_assert(kTailStageBytes >= kSlotOBytes + kSlotOBytes / 8 + kWsTailsBytes, "a request cut 148 times fits");

// two consecutive output elements (an even index) in the output's element type
__device__ __noinline__ void store_out_pair(void* out, int out_dtype, size_t idx, float a, float b) {
  if (out_dtype == MLA_FP4_OUT_BF16) {
    __nv_bfloat162 b2 = __floats2bfloat162_rn(a, b);
    *reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(out) + idx) = *reinterpret_cast<uint32_t*>(&b2);
  } else if (out_dtype == MLA_FP4_OUT_F32) {
    *reinterpret_cast<float2*>(static_cast<float*>(out) + idx) = make_float2(a, b);
  } else {
    *reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(out) + idx) = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  }
}

// The tail runs once per CTA, so its instructions are fetched cold: it is written for few
// instructions (rolled loops, no 64-bit division, approximate exp2/log2), not for peak throughput.
__device__ __noinline__ void zero_empty_requests(const DecodeParams& p, int tid) {
  const int total = p.groups * p.batch;
  const uint32_t esz = uint32_t(out_elem_bytes(p.out_dtype));
#pragma unroll 1
  for (int v = blockIdx.x; v < total; v += gridDim.x) {
    const int g = v / p.batch, b = v - g * p.batch;
    if (capped_len(p.seq_lens, b, p.seq_cap) > 0) continue;
    int qpos, head0;
    group_coords(g, p.num_heads, qpos, head0);
    const int heads_here = min(kGroupHeads, p.num_heads - head0);
    const size_t row0 = (size_t(b) * p.q_len + qpos) * p.num_heads + head0;
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(p.out) + row0 * kLatent * esz);
    const uint32_t n16 = uint32_t(heads_here) * kLatent * esz / 16u;
#pragma unroll 1
    for (uint32_t i = tid; i < n16; i += kThreads) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    // no token at all: with a sink the softmax is over the sink alone (zero value row), whose logit is the LSE
    if (p.lse && tid < heads_here) p.lse[row0 + tid] = p.sink ? __ldg(p.sink + head0 + tid) * kLog2e : -INFINITY;
  }
}

// The merge plan of this CTA, made by one warp while the main loop is still waiting for its first tile: the slots
// of the request this CTA merges (in CTA order), how many CTAs merge it and this CTA's place among them.
// A CTA merges only the request of its first segment (even slot): every CTA then takes part in at most one
// merge, and the first writer of a request, which reaches it last, in none.  Writers of the request: CTA m.counter,
// then every following CTA whose range starts before the request ends and holds a real tile of it.  The first
// writer uses slot 2i+1 unless its range starts with the request; the others start inside the request, use slot 2i
// and take part in the merge.
__device__ __noinline__ void plan_merge(const Ctx& c, int lane) {
  Misc* misc = c.misc;
  const int n = gridDim.x;
  int k = -1;
  for (int i = 0; i < misc->n_merge; ++i)
    if (!(misc->merge[i].slot & 1)) k = i;
  if (k < 0) {
    if (lane == 0) misc->n_slots = 0;
    return;
  }
  const MergeReq m = misc->merge[k];
  const flat_t Tt = misc->walker.Tt;
  const flat_t end = m.start + m.tiles;
  int cnt = 0, part = 0, rank = 0;
#pragma unroll 1
  for (int base = m.counter & ~31; base < n; base += 32) {
    const int i = base + lane;
    bool writer = false, merger = false;
    if (i < n && i >= m.counter) {
      const flat_t lo = cta_lo(Tt, n, i), nlo = cta_lo(Tt, n, i + 1);
      writer = lo < end && nlo > lo && nlo > m.start + kPhantom;  // holds at least one real tile of the request
      merger = writer && lo >= m.start;
    }
    const uint32_t bw = __ballot_sync(0xffffffffu, writer), bm = __ballot_sync(0xffffffffu, merger);
    const uint32_t below = (1u << lane) - 1u;
    if (writer) {
      const int pos = cnt + __popc(bw & below);
      if (pos < kMaxCombineSlots) sts_f32(c.smem + kOffTail + 4u * uint32_t(pos), __int_as_float(slot_of(i, merger)));
    }
    const int mine = (i == int(blockIdx.x) && merger) ? part + __popc(bm & below) : 0;
    rank += __reduce_add_sync(0xffffffffu, mine);
    cnt += __popc(bw);
    part += __popc(bm);
    if (bw == 0 && cnt > 0) break;  // past the request
  }
  if (lane == 0) {
    const int ns = min(cnt, kMaxCombineSlots);
    misc->n_slots = ns;
    misc->n_part = part;
    misc->rank = rank;
    misc->merge_k = k;
    // what the tail would otherwise compute on its critical path: the share, and the barrier its copies complete on
    misc->unit0 = part > 0 ? (2048 * rank) / part : 0;
    misc->unit1 = part > 0 ? (2048 * (rank + 1)) / part : 0;
    if (ns > 0) {
      ptx::mbar_init(bar_addr(c, kBarTail), uint32_t(ns));  // one arrival per slot
      ptx::fence_barrier_init();
    }
  }
}

// The tail runs once per CTA: small loop bodies, shared memory read with ld.shared in batches (a chain of
// dependent load-then-add iterations is what made an earlier version slow, not the amount of work).
// Geometry of this CTA's part in the merge (from the plan).
struct TailGeo {
  int ns, U0, U1;
  uint32_t share_bytes, rows, tails, list;
  bool fits;
};
__device__ __forceinline__ TailGeo tail_geo(const Ctx& c) {
  const Misc* misc = c.misc;
  TailGeo g;
  g.ns = misc->n_slots;
  // This CTA's share of every slot: units [2048*rank/np, 2048*(rank+1)/np) of 32 bytes (a pair of dims of one head
  // group, in the slot's own order), so a share is one contiguous range of the slot: one bulk copy.
  g.U0 = misc->unit0;
  g.U1 = misc->unit1;
  g.share_bytes = uint32_t(g.U1 - g.U0) * 32u;
  g.list = c.smem + kOffTail;
  g.rows = c.smem + kTailStage;
  g.tails = g.rows + uint32_t(g.ns) * g.share_bytes;  // the tails of the listed slots, in list order
  g.fits = uint32_t(g.ns) * (g.share_bytes + kTailLseBytes) <= kTailStageBytes;
  return g;
}

// Fetching the partials: run by the four warps that issue copies and MMAs (QK, TMA, PV, PV2), which have nothing left
// to do once the last tile's MMAs have drained, while the eight softmax warps still normalise, write and publish this
// CTA's own partial: the staging area (the KV ring, RoPE, Q and P buffers) is free from that moment, and whatever the
// other CTAs have published by then is on its way before this CTA's own partial is out.  Slot i (and i + 128) belongs to
// lane i / 4 of helper warp i % 4: wait for its flag, then fetch this CTA's share of it and its tail (LSEs, scale).  A
// bulk copy costs about fifty clocks to issue whatever its size and the lanes of a warp issue theirs one after the other,
// so the slots are dealt round the warps.  The lanes of a warp poll in step (a ballot ends the loop).
__device__ __noinline__ void tail_fetch(const DecodeParams& p, const Ctx& c, int hw, int lane) {
  Misc* misc = c.misc;
  void* ws = p.workspace;
  const TailGeo g = tail_geo(c);
  if (g.ns == 0) return;
  if (hw == 0 && lane == 0) {
    if (!g.fits) flag_timeout(c, 200, uint32_t(g.ns));  // cannot happen: mergers >= writers - 1
    MLA_TRACE(3, 1u, 1);
  }
  const uint32_t bar = bar_addr(c, kBarTail);
#pragma unroll 1
  for (int i = lane * 4 + hw; i < kMaxCombineSlots + 128; i += 128) {  // the loop bound is uniform; a lane without a slot idles
    const bool mine = i < g.ns;
    if (!__any_sync(0xffffffffu, mine) || misc->abort) break;
    const int slot = mine ? int(lds_u32(g.list + 4u * uint32_t(i))) : 0;
    const int32_t* flag = slot_flag(ws, slot);
    bool done = !mine;
#pragma unroll 1
    for (uint32_t it = 0; it < c.polls; ++it) {
      const bool now = !done && ld_acquire(flag) == c.gen;  // acquire: the slot's bytes, written before the flag, are read after it
      if (now) {
        done = true;
#ifdef MLA_FP4_TRACE
        if (int(blockIdx.x) == c.trace_cta && c.status && i < 96) {
          unsigned long long t;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
          long long* tr = reinterpret_cast<long long*>(c.status + 8) + ((4 + (i >> 4)) * 16 + (i & 15)) * 8;
          tr[0] = (long long)t;
          tr[1] = slot;
        }
#endif
        if (g.fits) {
          // The copy reads the slot from L2, where its writer's release put it before the flag: no proxy fence is
          // needed for that, and a full fence.proxy.async here cost microseconds.
          ptx::mbar_arrive_expect_tx(bar, g.share_bytes + kTailLseBytes);
          ptx::bulk_load(g.rows + uint32_t(i) * g.share_bytes, reinterpret_cast<const char*>(slot_o(ws, slot)) + size_t(g.U0) * 32, g.share_bytes, bar);
          ptx::bulk_load(g.tails + uint32_t(i) * kTailLseBytes, slot_lse(ws, slot), kTailLseBytes, bar);  // its LSEs and scale
        } else {
          ptx::mbar_arrive(bar);
        }
      }
      if (__all_sync(0xffffffffu, done) || misc->abort) break;
      __nanosleep(64);
    }
    if (!done) {  // the budget ran out (or the CTA is giving up): the barrier still gets this slot's arrival
      if (!misc->abort) flag_timeout(c, 100, uint32_t(slot));
      ptx::mbar_arrive(bar);
    }
  }
  if (hw == 0 && lane == 0) MLA_TRACE(3, 1u, 2);
}

__device__ __noinline__ void tail_merge(const DecodeParams& p, const Ctx& c, int tid) {
  Misc* misc = c.misc;
  const TailGeo geo = tail_geo(c);
  const int ns = geo.ns;
  if (ns == 0) return;
  const int rank = misc->rank;
  const MergeReq m = misc->merge[misc->merge_k];
  int qpos, head0;
  group_coords(m.g, p.num_heads, qpos, head0);
  const int heads_here = min(kGroupHeads, p.num_heads - head0);
  const size_t row0 = (size_t(m.b) * p.q_len + qpos) * p.num_heads + head0;
  const int U0 = geo.U0, U1 = geo.U1;
  const uint32_t share_bytes = geo.share_bytes, rows = geo.rows, tails = geo.tails;
  const bool landed = wait(c, kBarTail, 0);
  if (tid == 0) MLA_TRACE(3, 1u, 3);
  if (landed && !misc->abort) {
    // The tail runs once: what it costs is mostly the fetching of its instructions (8 KB of straight-line code added
    // here cost the north-star step 3 us, 0.4 us per KB), so the loops below are rolled and small rather than
    // unrolled for throughput.
    // weights: four lanes per head split the slots; butterflies give all four the results.  w_i = 2^(lse_i - max) *
    // slot scale, left in place of the LSE; the division by their sum is one multiply per output at the end.
    if (tid < 4 * kGroupHeads) {
      const int h = tid >> 2, j = tid & 3;
      const uint32_t col = tails + 4u * uint32_t(h);
      float mx = -INFINITY;
#pragma unroll 1
      for (int i = j; i < ns; i += 4) mx = fmaxf(mx, lds_f32(col + uint32_t(i) * kTailLseBytes));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      float dsum = 0.f;
#pragma unroll 1
      for (int i = j; i < ns; i += 4) {
        const uint32_t at = uint32_t(i) * kTailLseBytes;
        const float l = lds_f32(col + at);
        const float e = (l == -INFINITY) ? 0.f : ptx::ex2(l - mx);
        sts_f32(col + at, e * lds_f32(tails + at + 4u * kGroupHeads));
        dsum += e;
      }
      dsum += __shfl_xor_sync(0xffffffffu, dsum, 1);
      dsum += __shfl_xor_sync(0xffffffffu, dsum, 2);
      if (j == 0) {
        sts_f32(c.smem + kOffTailInv + 4u * uint32_t(h), dsum > 0.f ? __frcp_rn(dsum) : 0.f);
        if (rank == 0 && p.lse && h < heads_here) p.lse[row0 + h] = (dsum > 0.f) ? (__log2f(dsum) + mx) : -INFINITY;
      }
    }
    __syncthreads();
    if (tid == 0) MLA_TRACE(3, 1u, 4);
    // An item is (unit of this CTA's share, pair of heads of the unit's group): 4 bytes per dim and slot; the sums
    // run in slot order (bit-reproducible whatever the order of arrival), four slots' loads in flight together.
    const int items = (U1 - U0) * 4;
#pragma unroll 1
    for (int item = tid; item < items; item += kThreads) {
      const int u = U0 + (item >> 2), hq = item & 3;
      const int head = 8 * (u >> 8) + 2 * hq, dim = 2 * (u & 255);
      uint32_t src = rows + uint32_t(item >> 2) * 32u + 4u * uint32_t(hq);
      uint32_t wcol = tails + 4u * uint32_t(head);
      float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;  // [dim][head]
      int i = 0;
#pragma unroll 1
      for (; i + 4 <= ns; i += 4) {
        uint32_t u0[4], u1[4];
        float2 wv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          u0[q] = lds_u32(src);
          u1[q] = lds_u32(src + 16u);
          wv[q] = lds_f32x2(wcol);
          src += share_bytes;
          wcol += kTailLseBytes;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u0[q])), f1 = __half22float2(*reinterpret_cast<const __half2*>(&u1[q]));
          a00 += wv[q].x * f0.x;
          a01 += wv[q].y * f0.y;
          a10 += wv[q].x * f1.x;
          a11 += wv[q].y * f1.y;
        }
      }
#pragma unroll 1
      for (; i < ns; ++i) {
        const uint32_t u0 = lds_u32(src), u1 = lds_u32(src + 16u);
        const float2 wv = lds_f32x2(wcol);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u0)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&u1));
        a00 += wv.x * f0.x;
        a01 += wv.y * f0.y;
        a10 += wv.x * f1.x;
        a11 += wv.y * f1.y;
        src += share_bytes;
        wcol += kTailLseBytes;
      }
      const float2 inv = lds_f32x2(c.smem + kOffTailInv + 4u * uint32_t(head));
      const size_t idx = (row0 + head) * kLatent + dim;
      if (head < heads_here) store_out_pair(p.out, p.out_dtype, idx, a00 * inv.x, a10 * inv.x);
      if (head + 1 < heads_here) store_out_pair(p.out, p.out_dtype, idx + kLatent, a01 * inv.y, a11 * inv.y);
    }
    if (tid == 0) MLA_TRACE(3, 1u, 5);
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------
template <bool kSoftCap>
__global__ void __launch_bounds__(kThreads, 1)
mla_fp4_decode_sm100_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_q_lat,
                            const __grid_constant__ CUtensorMap map_q_rope, const __grid_constant__ CUtensorMap map_rope,
                            const __grid_constant__ CUtensorMap map_lat) {
  extern __shared__ uint8_t smem_raw[];
#ifdef MLA_FP4_TRACE
  const long long t_entry = clock64();
#endif
  Ctx c;
  {
    uint32_t raw = ptx::smem_u32(smem_raw);
    uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
    c.smem = raw + pad;
    c.smem_ptr = smem_raw + pad;
  }
  c.misc = reinterpret_cast<Misc*>(c.smem_ptr + kOffMisc);
  c.status = p.status;
  c.polls = p.wait_polls;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;

  // What needs nothing an earlier kernel wrote comes first: with a programmatic dependent launch this part runs
  // while the kernel before this one on the stream is still draining.
  if (warp == 0) {
    ptx::tmem_alloc(c.smem + kOffMisc + offsetof(Misc, tmem_base), 512);
    ptx::tmem_relinquish();
  } else if (warp == kWarpTMA && (tid & 31) == 0) {
    for (int slot = 0; slot < kRing; ++slot) {
      ptx::mbar_init(bar_addr(c, bar_kv_full(slot)), 1);
      ptx::mbar_init(bar_addr(c, bar_kv_empty(slot)), 1);
    }
    for (int s = 0; s < kSStages; ++s) {
      ptx::mbar_init(bar_addr(c, bar_sc_full(s)), 1);
      ptx::mbar_init(bar_addr(c, bar_s_full(s)), 1);
      ptx::mbar_init(bar_addr(c, bar_s_empty(s)), kSoftmaxThreads);
    }
    ptx::mbar_init(bar_addr(c, kBarRopeFull), 1);
    ptx::mbar_init(bar_addr(c, kBarRopeEmpty), 1);
    ptx::mbar_init(bar_addr(c, kBarPFull), kSoftmaxThreads);
    ptx::mbar_init(bar_addr(c, kBarPEmpty), 2);  // the two PV issue warps
    ptx::mbar_init(bar_addr(c, kBarQFull), 1);
    ptx::mbar_init(bar_addr(c, kBarQEmpty), 1);
    ptx::mbar_init(bar_addr(c, kBarOFree), kSoftmaxThreads);
    ptx::mbar_init(bar_addr(c, kBarDrain), 3);
    ptx::fence_barrier_init();
  } else if (warp == kWarpPV && (tid & 31) == 0) {
    ptx::prefetch_tensormap(&map_q_lat);
    ptx::prefetch_tensormap(&map_q_rope);
    ptx::prefetch_tensormap(&map_rope);
    ptx::prefetch_tensormap(&map_lat);
  }
  // From here on the kernel reads what earlier kernels wrote (sequence lengths, q, the cache, the workspace).
  if (p.pdl_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
  // The generation of this step: one more than that of the last completed step.  No CTA of this step
  // can have advanced it yet (that takes every CTA of the grid to have finished).
  // One thread of a warp that has nothing else to do here fetches it: an acquire load holds back the loads behind it,
  // and the warp that walks the partition (sequence lengths, a cold DRAM round trip) should not queue behind that.
#ifdef MLA_FP4_TRACE
  long long t_pro[4] = {0, 0, 0, 0};
  t_pro[0] = clock64();
#endif
  if (warp == kWarpPV && (tid & 31) == 0) c.misc->gen = p.fused_merge ? ld_acquire(ws_generation(p.workspace)) + 1 : 0;
  if (warp == 0) {
    Walker w = make_walker(p.seq_lens, p.batch, p.seq_cap, p.groups, blockIdx.x, gridDim.x);
#ifdef MLA_FP4_TRACE
    t_pro[1] = clock64();
#endif
    if (tid == 0) {
      c.misc->walker = w;
      c.misc->abort = 0;
      c.misc->n_merge = 0;
      if (w.Tt < 0) {  // the flat tile space does not fit 32 bits: nothing is decoded, the status says why
        c.misc->nseg = 0;
        c.misc->more = 0;
        if (p.status) atomicCAS(p.status, 0, MLA_FP4_ERR_UNSUPPORTED);
      } else {
        stage_segments(c);
      }
    }
#ifdef MLA_FP4_TRACE
    t_pro[2] = clock64();
#endif
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  c.gen = c.misc->gen;
#ifdef MLA_FP4_TRACE
  c.trace_cta = (p.status && p.status[7] >= 0 && p.status[7] < int(gridDim.x) && p.status[7] != 0) ? p.status[7] : int(gridDim.x) - 1;
  if (tid == 0 && int(blockIdx.x) == c.trace_cta && c.status) {
    long long* tr = reinterpret_cast<long long*>(c.status + 8) + (11 * 16 + 0) * 8;
    tr[1] = t_pro[0]; tr[2] = t_pro[1]; tr[3] = t_pro[2]; tr[4] = clock64();
  }
#endif
  const uint32_t tmem = c.misc->tmem_base;
  if (tid == 0) MLA_TRACE(3, 0u, 0);
#ifdef MLA_FP4_TRACE
  if (tid == 0 && int(blockIdx.x) == c.trace_cta && c.status) reinterpret_cast<long long*>(c.status + 8)[(11 * 16 + 0) * 8 + 0] = t_entry;
  auto gtimer = [] { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
  unsigned long long* cta_times = p.status ? reinterpret_cast<unsigned long long*>(p.status + 8) + 12 * 16 * 8 + 4 * blockIdx.x : nullptr;
  if (tid == 0 && cta_times) cta_times[0] = gtimer();
#endif
  // Let a dependent kernel (the split-KV combine) start its launch and prologue early; it still waits
  // for this whole grid before it reads the partial slots.
  if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // the PV issue warps have nothing to do until the first P is there: one of them makes the merge plan meanwhile
  if (warp == kWarpPV2 && p.fused_merge) plan_merge(c, tid & 31);

  RoleState st;
  st.it = 0;
  st.seg = 0;
  st.part = 0;
  st.slot = 0;
  st.lap = 0;
  st.n_rope = 0;
  st.n_sc = 0;
  // Rounds: almost always exactly one; more only when a CTA's range spans more than kMaxSeg requests.
  for (;;) {
    if (warp >= kWarpSoftmax0) {
      softmax_role<kSoftCap>(p, c, tmem, tid - 32 * kWarpSoftmax0, st);
    } else if (warp == kWarpQK) {
      qk_role(c, tmem, st);
    } else if (warp == kWarpPV || warp == kWarpPV2) {
      pv_role(c, tmem, st, uint32_t(warp - kWarpPV));
    } else if (warp == kWarpTMA) {
      tma_role(p, c, &map_q_lat, &map_q_rope, &map_rope, &map_lat, st);
    }
    const int more = c.misc->more;
    if (!more && warp < kWarpSoftmax0) {
      // Last round: drain (everything issued has completed before TMEM is released and before shared memory is reused:
      // a commit covers the MMAs of the thread that executes it), then these four warps, idle from here on, fetch the
      // partials of the request this CTA merges while the softmax warps finish with its own.
      if (warp != kWarpTMA && ptx::elect_one()) ptx::umma_commit(bar_addr(c, kBarDrain));
      __syncwarp();
      if ((tid & 31) == 0) drain_wait(c, kBarDrain, 0);
      __syncwarp();
      if (p.fused_merge) tail_fetch(p, c, warp, tid & 31);
    }
    __syncthreads();  // every role is done with the staged segments
    if (!more) break;
    if (tid == 0) stage_segments(c);
    __syncthreads();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (tid == 0) MLA_TRACE(3, 0u, 1);
#ifdef MLA_FP4_TRACE
  if (tid == 0 && cta_times) cta_times[1] = gtimer();
#endif
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
  if (p.fused_merge) {
    tail_merge(p, c, tid);
    zero_empty_requests(p, tid);
    if (tid == 0) MLA_TRACE(3, 0u, 5);
#ifdef MLA_FP4_TRACE
    if (tid == 0 && cta_times) cta_times[2] = gtimer();
#endif
    // The last CTA to finish advances the generation: the next step's flags differ from all of this one's.
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(ws_finished(p.workspace), 1) == int(gridDim.x) - 1) {
        *ws_finished(p.workspace) = 0;
        st_release(ws_generation(p.workspace), c.gen);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(ptr);
    return static_cast<EncodeTiledFn>(nullptr);
  }();
  return fn;
}

bool encode_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                const uint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t gd[5], gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { gd[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_bytes[i];
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The four tensor maps of a launch depend only on the query's address and strides, the cache's address and the
// shapes.  A serving loop calls with the same ones step after step, and encoding four maps cost more host time than
// the rest of the call: the last set is kept per thread and reused when its key matches.
struct MapKey {
  const void* q;
  const void* kv;
  int64_t sb, sq, sh, num_pages;
  int32_t batch, q_len, num_heads, page_size;
  bool operator==(const MapKey& o) const {
    return q == o.q && kv == o.kv && sb == o.sb && sq == o.sq && sh == o.sh && num_pages == o.num_pages && batch == o.batch &&
           q_len == o.q_len && num_heads == o.num_heads && page_size == o.page_size;
  }
};
struct MapSet {
  MapKey key;
  bool valid = false;
  CUtensorMap q_lat, q_rope, rope, lat;
};

}  // namespace

cudaError_t launch_decode_sm100(const DecodeParams& p, int num_ctas, cudaStream_t stream, const char** err) {
  *err = nullptr;
  static thread_local MapSet cache;
  const MapKey key{p.q, p.kv_cache, p.q_stride_batch, p.q_stride_qpos, p.q_stride_head, p.num_pages, p.batch, p.q_len, p.num_heads, p.page_size};
  if (!(cache.valid && cache.key == key)) {
    cache.valid = false;
    CUtensorMap& map_q_lat = cache.q_lat;
    CUtensorMap& map_q_rope = cache.q_rope;
    CUtensorMap& map_rope = cache.rope;
    CUtensorMap& map_lat = cache.lat;
    {
      // q viewed as [576, H, q_len, B] bytes
      uint64_t sq = p.q_len > 1 ? uint64_t(p.q_stride_qpos) : uint64_t(p.q_stride_head) * uint64_t(p.num_heads);
      uint64_t sb = p.batch > 1 ? uint64_t(p.q_stride_batch) : sq * uint64_t(p.q_len);
      uint64_t dims[4] = {uint64_t(kQDim), uint64_t(p.num_heads), uint64_t(p.q_len), uint64_t(p.batch)};
      uint64_t strides[3] = {uint64_t(p.q_stride_head), sq, sb};
      uint32_t box_lat[4] = {128, uint32_t(kGroupHeads), 1, 1};
      uint32_t box_rope[4] = {64, uint32_t(kGroupHeads), 1, 1};
      if (!encode_map(&map_q_lat, p.q, 4, dims, strides, box_lat, CU_TENSOR_MAP_SWIZZLE_128B) ||
          !encode_map(&map_q_rope, p.q, 4, dims, strides, box_rope, CU_TENSOR_MAP_SWIZZLE_64B)) {
        *err = "cuTensorMapEncodeTiled failed for q (check alignment and strides)";
        return cudaErrorInvalidValue;
      }
    }
    {
      uint64_t dims[3] = {uint64_t(kRowBytes), uint64_t(p.page_size), uint64_t(p.num_pages)};
      uint64_t strides[2] = {uint64_t(kRowBytes), uint64_t(kRowBytes) * uint64_t(p.page_size)};
      uint32_t box[3] = {64, uint32_t(p.page_size), 1};
      if (!encode_map(&map_rope, p.kv_cache, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B)) {
        *err = "cuTensorMapEncodeTiled failed for kv_cache (check alignment)";
        return cudaErrorInvalidValue;
      }
    }
    {
      // the cache as 4-bit elements: 640 per row (the 512 latent codes, then the RoPE bytes seen as nibbles and
      // never fetched through this map), page_size rows per page; a box is one 128-dim block of one page
      EncodeTiledFn fn = get_encode_fn();
      cuuint64_t gd[3] = {cuuint64_t(2 * kRowBytes), cuuint64_t(p.page_size), cuuint64_t(p.num_pages)};
      cuuint64_t gs[2] = {cuuint64_t(kRowBytes), cuuint64_t(kRowBytes) * cuuint64_t(p.page_size)};
      cuuint32_t bx[3] = {128, cuuint32_t(p.page_size), 1};
      cuuint32_t es[3] = {1, 1, 1};
      if (!fn || fn(&map_lat, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, const_cast<void*>(p.kv_cache), gd, gs, bx, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
        *err = "cuTensorMapEncodeTiled failed for the packed latent (kv_cache must be 32-byte aligned)";
        return cudaErrorInvalidValue;
      }
    }
    cache.key = key;
    cache.valid = true;
  }
  const CUtensorMap& map_q_lat = cache.q_lat;
  const CUtensorMap& map_q_rope = cache.q_rope;
  const CUtensorMap& map_rope = cache.rope;
  const CUtensorMap& map_lat = cache.lat;
  {
    static std::atomic<bool> attr_done[64];  // zero-initialised; setting the attribute twice is harmless
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !attr_done[dev].load(std::memory_order_acquire)) {
      e = cudaFuncSetAttribute(mla_fp4_decode_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemAlloc));
      if (e != cudaSuccess) return e;
      e = cudaFuncSetAttribute(mla_fp4_decode_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemAlloc));
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_done[dev].store(true, std::memory_order_release);
    }
  }
  // the attention variant with a score transform is a kernel of its own: the standard one carries none of its instructions
  auto* kernel = p.soft_cap > 0.f ? mla_fp4_decode_sm100_kernel<true> : mla_fp4_decode_sm100_kernel<false>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemAlloc;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (p.fused_merge) {
    attr[n_attr].id = cudaLaunchAttributeCooperative;  // the CTAs wait for one another in the tail merge
    attr[n_attr].val.cooperative = 1;
    ++n_attr;
  }
  // Programmatic dependent launch of this kernel itself: its CTAs are placed and run their prologue while the kernel
  // before it on the stream drains, then wait for that kernel's completion.  Whether the driver takes the attribute
  // together with the cooperative one is found out once per process, on a launch outside stream capture (a launch that
  // fails inside a capture would invalidate it); until then, and if it does not, the kernel is launched without it.
  static std::atomic<int> chain_state{0};  // 0 unknown, 1 accepted, 2 refused
  DecodeParams pp = p;
  pp.pdl_wait = 0;
#ifndef MLA_FP4_NO_PDL_CHAIN
  if (p.pdl) {
    int state = chain_state.load(std::memory_order_acquire);
    if (state == 0) {
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) state = 2;  // not now
    }
    if (state != 2) {
      attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = n_attr + 1;
      pp.pdl_wait = 1;
      cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, pp, map_q_lat, map_q_rope, map_rope, map_lat);
      if (e == cudaSuccess) {
        chain_state.store(1, std::memory_order_release);
        return e;
      }
      if (state == 1) return e;
      (void)cudaGetLastError();  // refused: remember, and launch without the attribute
      chain_state.store(2, std::memory_order_release);
      pp.pdl_wait = 0;
    }
  }
#endif
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, kernel, pp, map_q_lat, map_q_rope, map_rope, map_lat);
}

}  // namespace mla

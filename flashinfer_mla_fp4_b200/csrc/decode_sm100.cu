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
// RoPE bytes, per-token scales and Q arrive by TMA as well; pages two tiles ahead are prefetched into L2.
//
// Warp roles (384 threads): 0 QK^T issue, 1 TMA issue (lane i owns page i of the tile), 2 and 3 PV issue,
// two 128-dim blocks each (issue warps run warp-uniform code, one elected lane per instruction),
// 4-11 softmax / O rescale / epilogue (TMEM lane = token or dim; two warps share a lane quarter and
// split the 64 heads).
//
// Requests that are split across CTAs are merged at the end of the same kernel (tail_merge): the
// CTAs publish their partials through counters in the workspace header and each takes a share of
// the output dims.  The two-kernel mode leaves the merge to the combine kernel instead.
//
// The per-role loops are kept small on purpose: the instruction streams share one
// instruction cache, and an MMA-issue or softmax loop that misses it starves the tensor pipe.
//
// Every wait is bounded: when a wait expires the CTA records MLA_FP4_ERR_DEVICE_TIMEOUT in the
// status words, stops issuing work, drains and exits normally.
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
constexpr int kStages = 2;
constexpr int kBlocks = 4;                 // 128-dim blocks of the latent
constexpr int kBlockBytes = kTile * 128;   // 16 KiB: [128 tokens][128 B], 128B swizzle
constexpr int kMaxSeg = 48;                // segments staged per round
constexpr float kPShift = 4.0f;            // P' = 2^(y - M + 4): keeps the E4M3 lo term out of the subnormals
constexpr float kLazyThreshold = 4.0f;     // the reference is refreshed only when beaten by 2^4 (P' <= 2^8 < 448)

// shared memory map (bytes from a 1024-aligned base)
constexpr uint32_t kOffKV = 0;                                            // [2][4][16384]
constexpr uint32_t kOffRope = kOffKV + kStages * kBlocks * kBlockBytes;   // [2][128][64]  64B swizzle
constexpr uint32_t kOffQLat = kOffRope + kStages * kTile * 64;            // [4][64][128]  128B swizzle
constexpr uint32_t kOffQRope = kOffQLat + kBlocks * kGroupHeads * 128;    // [64][64]      64B swizzle
constexpr uint32_t kOffP = kOffQRope + kGroupHeads * 64;                  // [2][hi,lo][128][64] 64B swizzle (MN-major)
constexpr uint32_t kOffScale = kOffP + kStages * 2 * kTile * 64;          // [2][128] f32
constexpr uint32_t kOffM = kOffScale + kStages * kTile * 4;               // [64] f32 NEGATED reference -(M - shift)
constexpr uint32_t kOffF = kOffM + kGroupHeads * 4;                       // [64] f32 rescale factor
constexpr uint32_t kOffWmax = kOffF + kGroupHeads * 4;                    // [4][64] f32 per-warp column max / sum
constexpr uint32_t kOffLinv = kOffWmax + 4 * kGroupHeads * 4;             // [64] f32 output_scale / l
constexpr uint32_t kOffLse = kOffLinv + kGroupHeads * 4;                  // [64] f32
constexpr uint32_t kOffScMax = kOffLse + kGroupHeads * 4;                 // [8] f32 per-warp largest token scale
constexpr uint32_t kOffBars = kOffScMax + 8 * 4;                          // mbarriers (8 B each)
constexpr int kNumBars = 2 * 4 /*kv_full*/ + 2 * 4 /*kv_empty*/ + 2 /*aux_full*/ + 2 /*s_full*/ + 2 /*s_empty*/ +
                         2 /*p_full*/ + 1 /*q_full*/ + 1 /*q_empty*/ + 1 /*o_free*/ + 1 /*drain*/;
constexpr uint32_t kOffSegs = kOffBars + kNumBars * 8;                    // Segment[kMaxSeg]
constexpr uint32_t kOffMisc = kOffSegs + kMaxSeg * 24;                    // tmem base, abort flag, walker
constexpr uint32_t kSmemBytes = kOffMisc + 256;
constexpr uint32_t kSmemAlloc = kSmemBytes + 1024;                        // slack for manual 1024-alignment
static_assert(sizeof(Segment) == 24, "segment staging layout");
static_assert(kSmemAlloc <= 232448, "shared memory budget exceeded");
static_assert(kOffBars % 8 == 0 && kOffSegs % 8 == 0 && kOffMisc % 8 == 0, "alignment");

// barrier indices
__device__ __forceinline__ constexpr int bar_kv_full(int s, int j) { return s * 4 + j; }
__device__ __forceinline__ constexpr int bar_kv_empty(int s, int j) { return 8 + s * 4 + j; }
__device__ __forceinline__ constexpr int bar_aux_full(int s) { return 16 + s; }
__device__ __forceinline__ constexpr int bar_s_full(int s) { return 18 + s; }
__device__ __forceinline__ constexpr int bar_s_empty(int s) { return 20 + s; }
__device__ __forceinline__ constexpr int bar_p_full(int s) { return 22 + s; }
constexpr int kBarQFull = 24, kBarQEmpty = 25, kBarOFree = 26, kBarDrain = 27;

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
  int counter;    // index of the request's counters in the workspace header: the first CTA of its span
  int slot;       // the slot this CTA wrote (even: the segment was the CTA's first)
  int64_t start;  // flat tile index of the request's first tile
};
struct Misc {
  uint32_t tmem_base;
  volatile int abort;
  int nseg;   // segments staged for the current round
  int more;   // another round follows
  Walker walker;
  int n_merge;
  MergeReq merge[2];
  // scratch of the tail merge
  int64_t total_tiles;
  int n_slots, n_part, rank;
};
static_assert(sizeof(Misc) <= 256, "misc area");

struct Ctx {
  uint32_t smem;      // shared-space address of the aligned base
  uint8_t* smem_ptr;  // generic pointer to the same
  Misc* misc;
  int32_t* status;
#ifdef MLA_FP4_TRACE
  int trace_cta;  // the CTA whose timeline is recorded (status word 7; the last CTA when negative)
#endif
};

// running position of a role across rounds
struct RoleState {
  uint32_t it;   // tiles processed so far by this CTA (selects stage and barrier phase)
  uint32_t seg;  // segments processed so far
  uint32_t part; // partial segments processed so far (softmax role)
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
  for (uint32_t i = 0; i < (1u << 22); ++i) {
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
#pragma unroll 1
  for (uint32_t i = 0; i < (1u << 20); ++i) {
    if (ptx::mbar_try_wait(bar, parity)) return;
    __nanosleep(64);
  }
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
    // This lane's page id for the current tile and the two after it, loaded a tile ahead of their use
    // (never beyond the request's pages).
    auto page_of = [&](int tile) {
      const int lp = tile * ppt + lane;
      return (tile < g.tile_end && lane < ppt && lp < pages_total) ? __ldg(bt_req + lp) : -1;
    };
    int pg = page_of(g.tile_begin), pg1 = page_of(g.tile_begin + 1), pg2 = page_of(g.tile_begin + 2);
#pragma unroll 1
    for (int t = g.tile_begin; t < g.tile_end; ++t, ++st.it) {
      const uint32_t s = st.it & 1, k = st.it >> 1;
      if (lane == 0) MLA_TRACE(1, st.it, 0);
      const int np = min(ppt, pages_total - t * ppt);
      const bool mine = pg >= 0;
      const int pg3 = page_of(t + 3);  // in flight while this tile is issued
      // Two tiles ahead there is no free shared-memory stage yet, but L2 can take the rows already: the
      // copy issued later (when PV frees the stage) then finds them there instead of waiting for HBM.
      // The 32 lanes share the lines of each page of that tile (a page is one contiguous range).
      {
        const uint32_t page_bytes = uint32_t(p.page_size) * kRowBytes;
#pragma unroll 1
        for (int i = 0; i < ppt; ++i) {
          const int pgi = __shfl_sync(0xffffffffu, pg2, i);
          if (pgi < 0) break;
          const uint8_t* base = reinterpret_cast<const uint8_t*>(p.kv_cache) + size_t(pgi) * page_bytes;
#pragma unroll 1
          for (uint32_t off = uint32_t(lane) * 128u; off < page_bytes; off += 32u * 128u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off) : "memory");
        }
      }
      // The RoPE tile of this stage was last read by QK of tile it-2 and the scales by the softmax
      // of tile it-2; both are over once the softmax threads have released S of that tile.
      if (k >= 1) wait_warp(c, bar_s_empty(s), (k - 1) & 1);
      if (!c.misc->abort) {
        const uint32_t bar = bar_addr(c, bar_aux_full(s));
        if (lane == 0) ptx::mbar_arrive_expect_tx(bar, uint32_t(np) * (page_rope_bytes + page_scale_bytes));
        __syncwarp();
        if (mine) {
          ptx::tma_load_3d(c.smem + kOffRope + s * kTile * 64 + uint32_t(lane) * page_rope_bytes, map_rope, bar, kLatent / 2, 0, pg);
          ptx::bulk_load(c.smem + kOffScale + s * kTile * 4 + uint32_t(lane) * page_scale_bytes,
                         p.kv_cache_sf + size_t(pg) * p.page_size, page_scale_bytes, bar);
        }
      }
      // The packed E2M1 latent: the tensor map's 4-bit type makes the copy write every 16 values as
      // 8 bytes of data + 8 bytes of padding, the form the MMA reads 4-bit operands in, so a block is
      // [128 tokens][128 B] with the same 128-byte swizzle as an 8-bit tile and needs no conversion pass.
      // Block j of this stage is free once PV of tile it-2 has finished with it.
#pragma unroll 1
      for (int j = 0; j < kBlocks; ++j) {
        if (k >= 1) wait_warp(c, bar_kv_empty(s, j), (k - 1) & 1);
        if (c.misc->abort) break;
        if (lane == 0) MLA_TRACE(1, st.it, 1 + j);
        const uint32_t bar = bar_addr(c, bar_kv_full(s, j));
        if (lane == 0) ptx::mbar_arrive_expect_tx(bar, uint32_t(np) * (page_block_bytes / 2));  // the transaction count is in packed bytes
        __syncwarp();
        if (mine)
          ptx::tma_load_3d(c.smem + kOffKV + (s * kBlocks + j) * kBlockBytes + uint32_t(lane) * page_block_bytes, map_lat, bar,
                           128 * j, 0, pg);
      }
      pg = pg1;
      pg1 = pg2;
      pg2 = pg3;
    }
  }
  if (c.misc->abort && lane == 0) {  // let copies that were issued but never consumed land before exit
    for (uint32_t s = 0; s < kStages; ++s) {
      const uint32_t used = (st.it + 1 - s) >> 1;  // tiles issued on stage s
      if (used >= 1) {
        drain_wait(c, bar_aux_full(s), (used - 1) & 1);
        for (int j = 0; j < kBlocks; ++j) drain_wait(c, bar_kv_full(s, j), (used - 1) & 1);
      }
    }
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
  Desc kv_k;    // K tile block, K-major, 128B swizzle          (+ (stage*4+block)*1024 + kstep*2)
  Desc kv_mn;   // same bytes as V^T, MN-major                  (+ (stage*4+block)*1024 + kstep*256)
  Desc q_lat;   // Q latent block, K-major, 128B swizzle        (+ block*512 + kstep*2)
  Desc rope;    // K rope, K-major, 64B swizzle                 (+ stage*512 + kstep*2)
  Desc q_rope;  // Q rope                                       (+ kstep*2)
  Desc p;       // P^T hi, MN-major, 64B swizzle                (+ stage*1024 + lo*512 + kstep*128)
};

// QK^T of one 128-dim block of tile `it` (4 MMAs); with the first block also the RoPE part, after the
// last block the commit that hands S to the softmax warps.  The caller has seen the operands' barriers complete.
__device__ __forceinline__ void issue_qk_block(const Ctx& c, const MmaDescs& d, uint32_t it, uint32_t j, uint32_t tmem) {
  const uint32_t s = it & 1;
  const uint32_t d_lat = tmem + kColSLat + 64u * s;
  const uint32_t a_off = (s * kBlocks + j) * (kBlockBytes >> 4);
  const uint32_t b_off = j * ((kGroupHeads * 128) >> 4);
  ptx::tc_fence_after();
  if (ptx::elect_one()) {
    if (j == 0) {  // the RoPE part first: its operands arrive by TMA long before the last latent block
      const uint32_t d_rope = tmem + kColSRope + 64u * s;
      const uint32_t r_off = s * ((kTile * 64) >> 4);
#pragma unroll
      for (uint32_t ks = 0; ks < 2; ++ks) ptx::umma_f8(d_rope, d.rope.at(r_off + 2 * ks), d.q_rope.at(2 * ks), kIdescQKRope, ks);
    }
#pragma unroll
    for (uint32_t ks = 0; ks < 4; ++ks)
      ptx::umma_f8(d_lat, d.kv_k.at(a_off + 2 * ks), d.q_lat.at(b_off + 2 * ks), kIdescQK, (j | ks) ? 1u : 0u);
    if (j == kBlocks - 1) ptx::umma_commit(bar_addr(c, bar_s_full(s)));
  }
  __syncwarp();
}

// PV of tile `it`, blocks [j_begin, j_end): per block 4 token steps x (hi, lo); every block commits the barrier that frees it.
__device__ __forceinline__ void issue_pv(const Ctx& c, const MmaDescs& d, uint32_t it, uint32_t tmem, bool first_of_segment,
                                         uint32_t j_begin, uint32_t j_end) {
  const uint32_t s = it & 1;
  ptx::tc_fence_after();
  const uint32_t p_hi = s * ((2 * kTile * 64) >> 4);
  const uint32_t p_lo = p_hi + ((kTile * 64) >> 4);
  const uint32_t acc0 = first_of_segment ? 0u : 1u;
#pragma unroll
  for (uint32_t j = j_begin; j < j_end; ++j) {
    // A = V^T block: MN-major, 128-byte swizzle; 32 tokens per step = 4 groups of 8 rows (4096 B)
    const uint32_t a_off = (s * kBlocks + j) * (kBlockBytes >> 4);
    const uint32_t dd = tmem + kColO + 64u * j;
    if (ptx::elect_one()) {
#pragma unroll
      for (uint32_t ks = 0; ks < 4; ++ks) {
        // B = P^T: MN-major (64 heads contiguous), 64-byte swizzle; 32 tokens per step = 2048 B.
        // The hi and the lo term share A: it is fetched once and kept in the collector for the second.
        ptx::umma_f8_a_fill(dd, d.kv_mn.at(a_off + 256 * ks), d.p.at(p_hi + 128 * ks), kIdescPV, ks ? 1u : acc0);
        ptx::umma_f8_a_lastuse(dd, d.kv_mn.at(a_off + 256 * ks), d.p.at(p_lo + 128 * ks), kIdescPV, 1u);
      }
      ptx::umma_commit(bar_addr(c, bar_kv_empty(s, j)));
    }
    __syncwarp();
  }
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
      // S of this stage has been read by the softmax of tile it-2; RoPE bytes of this tile have landed
      if (k >= 1) ok = wait_warp(c, bar_s_empty(s), (k - 1) & 1);
      ok = ok && wait_warp(c, bar_aux_full(s), k & 1);
      MLA_TRACE(2, it, 0);
#pragma unroll
      for (uint32_t j = 0; j < kBlocks; ++j) {
        ok = ok && wait_warp(c, bar_kv_full(s, j), k & 1);
        MLA_TRACE(2, it, j == 0 ? 7 : (j == 1 ? 1 : (j == 2 ? 6 : 3)));  // block j has landed
        if (ok) issue_qk_block(c, d, it, j, tmem);
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
      const uint32_t it = st.it + t, s = it & 1, k = it >> 1;
      ok = wait_warp(c, bar_p_full(s), k & 1);
      if (!ok) break;
      if (part == 0) MLA_TRACE(2, it, 4);
      if (part == 0) issue_pv(c, d, it, tmem, t == 0, 0, kBlocks / 2);
      else issue_pv(c, d, it, tmem, t == 0, kBlocks / 2, kBlocks);
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
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// two-term E4M3 split of a pair: hi = e4m3(v), lo = e4m3(v - hi); returns hi (16 bits), lo via reference
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
  bool valid;
};

// One pass over the 32 heads this thread owns of its token: e = exp2(x*c - m), l += acc * e, and
// P' = e*scale_t split into two E4M3 terms and written to the swizzled P rows.  Returns the
// largest exponent argument seen (for the lazy-reference check).
__device__ __forceinline__ float softmax_pass(const SoftmaxTile& t, uint64_t (&l2)[kHalfHeads / 2], uint64_t acc2) {
  float mx = -INFINITY;
#pragma unroll
  for (int cidx = 0; cidx < 2; ++cidx) {
    uint32_t a[16], b[16];
    ptx::tmem_ld16(t.t_lat + 16 * cidx, a);
    ptx::tmem_ld16(t.t_rope + 16 * cidx, b);
    ptx::tmem_wait_ld();
    const uint32_t off = (((2 * t.half + uint32_t(cidx)) ^ t.psw) << 4);
    if (t.valid) {
      uint32_t hi16[8], lo16[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {  // 4 heads per shared load of the references
        uint64_t nm0, nm1;
        lds_pairs(t.negm + 64 * cidx + 16 * q, nm0, nm1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int i = 4 * q + 2 * h;
          const uint64_t x2 = fma2(pack2u(a[i], a[i + 1]), t.sc2, pack2u(b[i], b[i + 1]));
          const uint64_t arg2 = fma2(x2, t.cs2, h ? nm1 : nm0);
          float a0, a1;
          unpack2(arg2, a0, a1);
          mx = fmaxf(mx, fmaxf(a0, a1));
          const uint64_t e2 = pack2(ptx::ex2(a0), ptx::ex2(a1));
          l2[8 * cidx + 2 * q + h] = fma2(e2, acc2, l2[8 * cidx + 2 * q + h]);
          hi16[2 * q + h] = split_e4m3x2(mul2(e2, t.sc2), lo16[2 * q + h]);
        }
      }
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(t.p_hi + off), "r"(hi16[0] | (hi16[1] << 16)),
                   "r"(hi16[2] | (hi16[3] << 16)), "r"(hi16[4] | (hi16[5] << 16)), "r"(hi16[6] | (hi16[7] << 16)) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(t.p_lo + off), "r"(lo16[0] | (lo16[1] << 16)),
                   "r"(lo16[2] | (lo16[3] << 16)), "r"(lo16[4] | (lo16[5] << 16)), "r"(lo16[6] | (lo16[7] << 16)) : "memory");
    } else {  // token beyond seq_len: weight exactly zero, whatever its row holds
      asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(t.p_hi + off), "r"(0u) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(t.p_lo + off), "r"(0u) : "memory");
    }
  }
  return mx;
}

// Refresh the per-head reference: column max of y = x*c + log2(scale_t) over the tile's tokens,
// m = max(m_old, colmax - shift); f = 2^(m_old - m) (0 when there was no reference yet).
__device__ __noinline__ void refresh_reference(const Ctx& c, uint32_t t_lat, uint32_t t_rope, float sc, bool valid,
                                               float cscale, float lg, bool have_m, int tid) {
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
      const float y = fmaf(fmaf(__uint_as_float(a[i]), sc, __uint_as_float(b[i])), cscale, lg);
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
__device__ __noinline__ void write_output(const DecodeParams& p, const Ctx& c, uint32_t tmem_lane, int row, int half,
                                          int tid, int b, int g, int slot, float slot_scale_v) {
  int qpos, head0;
  group_coords(g, p.num_heads, qpos, head0);
  const int heads_here = min(kGroupHeads, p.num_heads - head0);
  const size_t row0 = (size_t(b) * p.q_len + qpos) * p.num_heads + head0;
  const bool direct = slot < 0;
  __half* so = reinterpret_cast<__half*>(slot_o(p.workspace, direct ? 0 : slot));
  // output_scale / l of this thread's 32 heads (times 1 / slot scale for a partial), read once
  const float post = direct ? 1.f : 1.f / slot_scale_v;
  float li[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) li[i] = lds_f32(c.smem + kOffLinv + 4 * (32 * half + i)) * post;
#pragma unroll 1
  for (int jb = 0; jb < kBlocks; ++jb) {
    uint32_t o[2][16];  // both 16-head halves of the block in flight before one wait
    ptx::tmem_ld16(tmem_lane + kColO + 64u * uint32_t(jb) + uint32_t(32 * half), o[0]);
    ptx::tmem_ld16(tmem_lane + kColO + 64u * uint32_t(jb) + uint32_t(32 * half + 16), o[1]);
    ptx::tmem_wait_ld();
    const int dim = 128 * jb + row;
    const int h0 = 32 * half;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i >> 4][i & 15]) * li[i];
    if (!direct) {
      uint32_t pk[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        __half2 h2 = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
        pk[q] = *reinterpret_cast<uint32_t*>(&h2);
      }
      uint4* dst = reinterpret_cast<uint4*>(so + size_t(dim) * kGroupHeads + h0);
#pragma unroll
      for (int q = 0; q < 4; ++q) dst[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
    } else if (p.out_dtype == MLA_FP4_OUT_BF16) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (row0 + h0) * kLatent + dim;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (h0 + i < heads_here) dst[size_t(i) * kLatent] = __float2bfloat16_rn(v[i]);
    } else if (p.out_dtype == MLA_FP4_OUT_F32) {
      float* dst = reinterpret_cast<float*>(p.out) + (row0 + h0) * kLatent + dim;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (h0 + i < heads_here) dst[size_t(i) * kLatent] = v[i];
    } else {
      uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + (row0 + h0) * kLatent + dim;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (h0 + i < heads_here) dst[size_t(i) * kLatent] = __nv_cvt_float_to_fp8(v[i], __NV_SATFINITE, __NV_E4M3);
    }
  }
  const float lse = lds_f32(c.smem + kOffLse + 4 * (tid & 63));
  if (direct) {
    if (p.lse && tid < heads_here) p.lse[row0 + tid] = lse;
  } else if (tid < kGroupHeads) {
    slot_lse(p.workspace, slot)[tid] = lse;
    if (tid == 0) slot_scale(p.workspace, slot)[0] = slot_scale_v;
  }
}

__device__ __forceinline__ void softmax_role(const DecodeParams& p, const Ctx& c, uint32_t tmem, int tid, RoleState& st) {
  const int nseg = c.misc->nseg;
  const Segment* sg = segs(c);
  const int warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3;           // TMEM lane quarter this warp may access
  const int half = warp >> 2;             // heads [32*half, 32*half + 32)
  const int row = quarter * 32 + lane;    // token of the tile (S) / dim of the block (O) of this thread
  const uint32_t tmem_lane = tmem + ((uint32_t(quarter) * 32u) << 16);
  const float cscale = p.softmax_scale * kLog2e;
  const uint64_t one2 = pack2(1.f, 1.f);
  SoftmaxTile t;
  t.negm = c.smem + kOffM + 4 * kHalfHeads * half;
  t.cs2 = pack2(cscale, cscale);
  t.psw = (uint32_t(row) >> 1) & 3u;
  t.half = uint32_t(half);
  int pending0 = 0, pending1 = 0, n_pending = 0;  // counters of the partials written in this call, published together at its end

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
      wait(c, bar_aux_full(s), k & 1);
      t.valid = (tt * kTile + row) < g.seq_len;
      float sc = lds_f32(c.smem + kOffScale + 4 * (s * kTile + row));
      sc = t.valid ? sc : 0.f;
      sc_max = fmaxf(sc_max, fabsf(sc));
      const float lg = t.valid ? __log2f(fmaxf(fabsf(sc), 8.67361738e-19f)) : 0.f;  // floor 2^-60
      t.sc2 = pack2(sc, sc);
      t.t_lat = tmem_lane + kColSLat + 64u * s + uint32_t(kHalfHeads * half);
      t.t_rope = tmem_lane + kColSRope + 64u * s + uint32_t(kHalfHeads * half);
      t.p_hi = c.smem + kOffP + s * 2 * kTile * 64 + uint32_t(row) * 64u;
      t.p_lo = t.p_hi + kTile * 64;

      // the P buffer of this stage is free once PV of tile it-2 has completed
      if (k >= 1) {  // both PV issue warps' last blocks
        wait(c, bar_kv_empty(s, 1), (k - 1) & 1);
        wait(c, bar_kv_empty(s, 3), (k - 1) & 1);
      }
      wait(c, bar_s_full(s), k & 1);
      if (tid == 0) MLA_TRACE(0, it, 1);
      ptx::tc_fence_after();

      // first tile of a segment: set the reference before anything is exponentiated
      if (first) refresh_reference(c, t.t_lat, t.t_rope, sc, t.valid, cscale, lg, false, tid);
      if (tid == 0) MLA_TRACE(0, it, 2);

      // Speculative pass with the current reference.  It stands unless some score beat the
      // reference by more than the lazy threshold (P' would leave the E4M3 range).
      const float mx = softmax_pass(t, l2, one2);
      const bool need = t.valid && (mx + lg > kPShift + kLazyThreshold);
      if (ptx::bar_or(1, kSoftmaxThreads, need)) {
        // Refresh the reference.  (l + e_old) * f equals l * f + e_new, so the row sums only need
        // the factor; O^T is rescaled in TMEM; P' is recomputed with the new reference.
        refresh_reference(c, t.t_lat, t.t_rope, sc, t.valid, cscale, lg, true, tid);
#pragma unroll
        for (int q = 0; q < kHalfHeads / 4; ++q) {
          uint64_t f0, f1;
          lds_pairs(c.smem + kOffF + 4 * kHalfHeads * half + 16 * q, f0, f1);
          l2[2 * q] = mul2(l2[2 * q], f0);
          l2[2 * q + 1] = mul2(l2[2 * q + 1], f1);
        }
        if (!first) {  // O^T holds earlier tiles: rescale once their PV has completed
          const uint32_t pit = it - 1;
          wait(c, bar_kv_empty(pit & 1, 1), (pit >> 1) & 1);
          wait(c, bar_kv_empty(pit & 1, 3), (pit >> 1) & 1);
          ptx::tc_fence_after();
          rescale_output(c, tmem_lane, uint32_t(half));
        }
        (void)softmax_pass(t, l2, 0ull);
      }
      if (tid == 0) MLA_TRACE(0, it, 3);
      ptx::tc_fence_before();  // orders the S reads and any O rescale before the arrives
      ptx::mbar_arrive(bar_addr(c, bar_s_empty(s)));
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(bar_addr(c, bar_p_full(s)));
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
        sts_f32(c.smem + kOffLinv + 4 * tid, p.output_scale / L);
        sts_f32(c.smem + kOffLse + 4 * tid, __log2f(L) - lds_f32(c.smem + kOffM + 4 * tid));
      }
      ptx::bar_sync(1, kSoftmaxThreads);
      // wait for the PV of the last tile
      wait(c, bar_kv_empty(lit & 1, 1), (lit >> 1) & 1);
      wait(c, bar_kv_empty(lit & 1, 3), (lit >> 1) & 1);
      ptx::tc_fence_after();
      float sc_all = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kSoftmaxThreads / 32; ++w8) sc_all = fmaxf(sc_all, lds_f32(c.smem + kOffScMax + 4 * w8));
      const float slot_scale_v = slot_scale_for(6.f * sc_all * fabsf(p.output_scale));
      if (!c.misc->abort) write_output(p, c, tmem_lane, row, half, tid, g.b, g.g, g.slot, slot_scale_v);
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar_addr(c, kBarOFree));
      if (g.slot >= 0) {  // a partial: published (below) once this CTA has written all its partials of the round
        if (p.fused_merge && n_pending < 2) {
          const int counter = c.misc->merge[st.part].counter;
          if (n_pending == 0) pending0 = counter;
          else pending1 = counter;
          ++n_pending;
        }
        ++st.part;
      }
      if (tid == 0) MLA_TRACE(0, lit, 6);
    }
  }
  // Publish the partials: the tail merge of their requests' CTAs waits for these counts.  One fence for
  // all of them, after the last segment: a fence in the middle would hold up the next segment's first tile,
  // and nobody can use a partial before this CTA, itself a writer of the later request, is done anyway.
  if (n_pending > 0) {
    __threadfence();
    ptx::bar_sync(1, kSoftmaxThreads);
    if (tid == 0) {
      atomicAdd(ws_arrived(p.workspace) + pending0, 1);
      if (n_pending > 1) atomicAdd(ws_arrived(p.workspace) + pending1, 1);
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
      m.start = w.f - int64_t(w.t);         // w.f and w.t are the flat and the in-request position just past this segment
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
// Every CTA that wrote a partial of a split request publishes it (a counter in the workspace
// header) right after writing it.  In the tail, the CTAs whose partial of a request was their
// first segment wait until all partials of that request are there and then merge, each, a share
// of the 512 output dims: out = sum_i w_i * O_i with w_i = 2^(lse_i - max) / sum * slot scale, the
// same arithmetic as the combine kernel.  A CTA has published everything it will ever publish
// before it waits for anybody else, so the waits cannot form a cycle; the launch is cooperative,
// so every CTA of the grid is resident; the waits are bounded like all others.  The last CTA to
// finish a request's merge zeroes its counters again.
constexpr int kTailLseStride = kGroupHeads + 4;                        // padded: the slot lanes of a unit hit different banks
constexpr uint32_t kTailLse = kOffKV;                                  // [148][68] f32: LSEs, then weights
constexpr uint32_t kTailList = kTailLse + kMaxCombineSlots * kTailLseStride * 4;  // [148] slot ids
constexpr uint32_t kTailScale = kTailList + kMaxCombineSlots * 4;      // [148] f32 slot scales
static_assert(kTailScale + kMaxCombineSlots * 4 <= kOffKV + kStages * kBlocks * kBlockBytes, "tail scratch fits the idle KV ring");

// Loads that happen only under a predicate and leave the destination untouched otherwise (the caller
// never reads a destination whose load was off): no zero fill, no branch.
__device__ __forceinline__ void ldcg_v4_if(uint4& d, const void* ptr, bool on) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t@p ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}"
               : "=r"(d.x), "=r"(d.y), "=r"(d.z), "=r"(d.w)
               : "l"(ptr), "r"(uint32_t(on))
               : "memory");
}
__device__ __forceinline__ void ldcg_f32_if(float& d, const float* ptr, bool on) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %2, 0;\n\t@p ld.global.cg.f32 %0, [%1];\n\t}" : "=f"(d) : "l"(ptr), "r"(uint32_t(on)) : "memory");
}

__device__ __forceinline__ int ld_acquire(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The tail runs once per CTA, so its instructions are fetched cold: it is written for few
// instructions (rolled loops, no 64-bit division, approximate exp2/log2), not for peak throughput.
__device__ __noinline__ void zero_empty_requests(const DecodeParams& p, int tid) {
  const int total = p.groups * p.batch;
  const uint32_t esz = uint32_t(out_elem_bytes(p.out_dtype));
#pragma unroll 1
  for (int v = blockIdx.x; v < total; v += gridDim.x) {
    const int g = v / p.batch, b = v - g * p.batch;
    if (p.seq_lens[b] > 0) continue;
    int qpos, head0;
    group_coords(g, p.num_heads, qpos, head0);
    const int heads_here = min(kGroupHeads, p.num_heads - head0);
    const size_t row0 = (size_t(b) * p.q_len + qpos) * p.num_heads + head0;
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(p.out) + row0 * kLatent * esz);
    const uint32_t n16 = uint32_t(heads_here) * kLatent * esz / 16u;
#pragma unroll 1
    for (uint32_t i = tid; i < n16; i += kThreads) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    if (p.lse && tid < heads_here) p.lse[row0 + tid] = -INFINITY;
  }
}

__device__ __noinline__ void tail_merge(const DecodeParams& p, const Ctx& c, int tid) {
  Misc* misc = c.misc;
  float* lse_s = reinterpret_cast<float*>(c.smem_ptr + kTailLse);
  int* list_s = reinterpret_cast<int*>(c.smem_ptr + kTailList);
  float* scale_s = reinterpret_cast<float*>(c.smem_ptr + kTailScale);
  void* ws = p.workspace;
  const int n = gridDim.x;
  const int n_merge = misc->n_merge;

#pragma unroll 1
  for (int k = 0; k < n_merge; ++k) {
    const MergeReq m = misc->merge[k];
    // A CTA merges only the request of its first segment (even slot): every CTA then takes part in
    // at most one merge, and the first writer of a request, which reaches it last, in none.
    if (m.slot & 1) continue;
    int32_t* arrived = ws_arrived(ws) + m.counter;
    int32_t* done = ws_done(ws) + m.counter;
    // Writers of the request: CTA m.counter, then every following CTA whose range starts before the
    // request ends and is not empty.  The first writer uses slot 2i+1 unless its range starts with the
    // request; the others start inside the request, use slot 2i and take part in the merge.  Thread i
    // looks at CTA i (one thread walking the CTAs cost 6000 clocks of dependent 64-bit arithmetic);
    // ballots and per-warp counts give every writer its place in the list, in CTA order.
    static_assert(kMaxCombineSlots <= kThreads, "one thread per CTA of the grid");
    {
      const int64_t Tt = misc->walker.Tt;
      const int64_t end = m.start + m.tiles;
      bool writer = false, merger = false;
      if (tid < n && tid >= m.counter) {
        int64_t lo, nlo;
        if (Tt * n < (int64_t(1) << 32)) {  // the usual case: 32-bit division
          lo = int64_t(uint32_t(Tt) * uint32_t(tid) / uint32_t(n));
          nlo = int64_t(uint32_t(Tt) * uint32_t(tid + 1) / uint32_t(n));
        } else {
          lo = cta_lo(Tt, n, tid);
          nlo = cta_lo(Tt, n, tid + 1);
        }
        writer = lo < end && nlo > lo && nlo > m.start + kPhantom;  // holds at least one real tile of the request
        merger = writer && lo >= m.start;
      }
      const uint32_t bw = __ballot_sync(0xffffffffu, writer), bm = __ballot_sync(0xffffffffu, merger);
      int* wcount = reinterpret_cast<int*>(scale_s);  // [12][2]; the slot scales are written two barriers later
      const int warp = tid >> 5;
      if ((tid & 31) == 0) {
        wcount[2 * warp] = __popc(bw);
        wcount[2 * warp + 1] = __popc(bm);
      }
      __syncthreads();
      int before_w = 0, before_m = 0, cnt = 0, part = 0;
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) {
        const int cw = wcount[2 * w], cm = wcount[2 * w + 1];
        if (w < warp) { before_w += cw; before_m += cm; }
        cnt += cw;
        part += cm;
      }
      const uint32_t below = (1u << (tid & 31)) - 1u;
      if (writer) {
        const int pos = before_w + __popc(bw & below);
        if (pos < kMaxCombineSlots) list_s[pos] = slot_of(tid, merger);
      }
      if (tid == int(blockIdx.x)) misc->rank = merger ? before_m + __popc(bm & below) : 0;
      if (tid == 0) {
        const int ns = min(cnt, kMaxCombineSlots);
        MLA_TRACE(3, 1u, 1);
        misc->n_slots = ns;
        misc->n_part = part;
        bool ok = false;  // bounded wait for the other writers
#pragma unroll 1
        for (uint32_t i = 0; i < (1u << 22); ++i) {
          if (ld_acquire(arrived) >= ns) { ok = true; break; }
          if (misc->abort) break;
          __nanosleep(32);
        }
        if (!ok && !misc->abort) flag_timeout(c, 100 + k, uint32_t(ns));
      }
    }
    __syncthreads();
    const int ns = misc->n_slots, np = misc->n_part, rank = misc->rank;
    if (tid == 0) MLA_TRACE(3, 1u, 2);
    if (!misc->abort) {
      int qpos, head0;
      group_coords(m.g, p.num_heads, qpos, head0);
      const int heads_here = min(kGroupHeads, p.num_heads - head0);
      const size_t row0 = (size_t(m.b) * p.q_len + qpos) * p.num_heads + head0;
      // This CTA's dims: pairs [256*rank/np, 256*(rank+1)/np).  A unit is (pair of dims, 8 heads, slot
      // lane); the SL lanes of a unit are consecutive lanes of a warp, split the slots (eight per batch,
      // all their loads in flight together) and add their sums with a fixed shuffle tree
      // (bit-reproducible).  Lane 0 of the unit writes 8 x 2 outputs.
      // (integer quotients through float: the operands are small and never within 1/300 of a boundary)
      const float rnp = 1.0f / float(np);
      const int u0 = int((float(256 * rank) + 0.5f) * rnp), u1 = int((float(256 * (rank + 1)) + 0.5f) * rnp);
      const int d0 = 2 * u0, pairs = u1 - u0;
      const int og = (heads_here + 7) >> 3;  // 8-head groups that hold heads of this launch
      const float rog = 1.0f / float(og);
      const int items = pairs * og;
      constexpr int kBatch = 8;  // slots whose rows a unit lane has in flight together
      int SL = 1, lg = 0;
      while (SL < 32 && kBatch * SL < ns && items * SL * 2 <= kThreads) { SL *= 2; ++lg; }  // one round of threads if possible
      const int units = items << lg;
      const char* slot0 = reinterpret_cast<const char*>(slot_o(ws, 0));
      auto load_batch = [&](const char* src, bool live_unit, int i0, uint4 (&a)[kBatch][2]) {
#pragma unroll
        for (int qq = 0; qq < kBatch; ++qq) {
          const bool ld = live_unit && i0 + qq * SL < ns;  // no load for a slot that does not exist (its list entry is stale)
          const char* sp = src + size_t(list_s[i0 + qq * SL]) * kSlotBytes;
          ldcg_v4_if(a[qq][0], sp, ld);
          ldcg_v4_if(a[qq][1], sp + kGroupHeads * 2, ld);
        }
      };
      // LSEs and slot scales: four lanes per head split the slots; a lane has eight slots' loads in flight
      // together (one round of latency for up to 32 slots).  They go out first: the weights are computed
      // while the partial rows, requested right behind them, are still on their way.
      const bool wlane = tid < 4 * kGroupHeads;
      const int wh = tid >> 2, wj = tid & 3;
      float v[8], sc[8];
      auto load_lse = [&](int i0) {
#pragma unroll
        for (int qq = 0; qq < 8; ++qq) {
          const int i = i0 + 4 * qq;
          const float* src = slot_lse(ws, list_s[i]);
          ldcg_f32_if(v[qq], src + wh, i < ns);
          ldcg_f32_if(sc[qq], src + kGroupHeads, i < ns);  // element 64 is the slot scale
        }
      };
      if (wlane) load_lse(wj);
      // The first batch of partial rows does not depend on the weights: its loads go out in the same round.
      uint4 a[kBatch][2];
      const int base0 = tid & ~31;
      if (base0 < units) {
        const int unit = tid;
        const int item = min(unit, units - 1) >> lg, sl = unit & (SL - 1);
        const int pr = int((float(item) + 0.5f) * rog), o = item - pr * og;
        load_batch(slot0 + (size_t(d0 + 2 * pr) * kGroupHeads + 8 * o) * 2, unit < units, sl, a);
      }
      // A weight lane keeps the running maximum and leaves the values in shared memory for its own second
      // pass; butterflies give all four lanes of a head the results.
      if (tid == 0) MLA_TRACE(3, 1u, 3);
      if (wlane) {
        const int h = wh, j = wj;
        float* col = lse_s + h;
        float mx = -INFINITY;
#pragma unroll 1
        for (int i0 = j; i0 < ns; i0 += 32) {
          if (i0 != j) load_lse(i0);
#pragma unroll
          for (int qq = 0; qq < 8; ++qq) {
            const int i = i0 + 4 * qq;
            if (i < ns) {
              col[i * kTailLseStride] = v[qq];
              scale_s[i] = sc[qq];  // every head's lane writes the same value; a lane reads back only what it wrote
              mx = fmaxf(mx, v[qq]);
            }
          }
        }
#pragma unroll
        for (int off = 2; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        float dsum = 0.f;
#pragma unroll 4
        for (int i = j; i < ns; i += 4) {
          const float l = col[i * kTailLseStride];
          const float e = (l == -INFINITY) ? 0.f : ptx::ex2(l - mx);
          col[i * kTailLseStride] = e;
          dsum += e;
        }
#pragma unroll
        for (int off = 2; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);
        const float inv = dsum > 0.f ? __frcp_rn(dsum) : 0.f;
#pragma unroll 4
        for (int i = j; i < ns; i += 4) col[i * kTailLseStride] *= inv * scale_s[i];  // weights, times the slot's fp16 scale
        if (j == 0 && rank == 0 && p.lse && h < heads_here) p.lse[row0 + h] = (dsum > 0.f) ? (__log2f(dsum) + mx) : -INFINITY;
      }
      __syncthreads();
      if (tid == 0) MLA_TRACE(3, 1u, 4);
#pragma unroll 1
      for (int base = (tid & ~31); base < units; base += kThreads) {
        const int unit = base + (tid & 31);
        const bool live_unit = unit < units;
        const int item = min(unit, units - 1) >> lg, sl = unit & (SL - 1);
        const int pr = int((float(item) + 0.5f) * rog), o = item - pr * og;
        const char* src = slot0 + (size_t(d0 + 2 * pr) * kGroupHeads + 8 * o) * 2;
        const float* wrow = lse_s + 8 * o;
        float acc[2][8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[0][e] = acc[1][e] = 0.f;
#pragma unroll 1
        for (int i0 = sl; i0 < ns; i0 += kBatch * SL) {  // eight slots x two dims: sixteen independent 16-byte loads in flight
          if (!(base == base0 && i0 == sl)) load_batch(src, live_unit, i0, a);  // the first batch is already here
#pragma unroll
          for (int qq = 0; qq < kBatch; ++qq) {
            const int i = i0 + qq * SL;
            if (i >= ns) break;  // the remaining slots of the batch do not exist
            const float* w = wrow + i * kTailLseStride;
            const float4 w0 = *reinterpret_cast<const float4*>(w), w1 = *reinterpret_cast<const float4*>(w + 4);
            const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int dd = 0; dd < 2; ++dd) {
              const uint32_t u[4] = {a[qq][dd].x, a[qq][dd].y, a[qq][dd].z, a[qq][dd].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[e]));
                acc[dd][2 * e] += wv[2 * e] * f.x;
                acc[dd][2 * e + 1] += wv[2 * e + 1] * f.y;
              }
            }
          }
        }
#pragma unroll 1
        for (int off = SL >> 1; off > 0; off >>= 1) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            acc[0][e] += __shfl_down_sync(0xffffffffu, acc[0][e], off);
            acc[1][e] += __shfl_down_sync(0xffffffffu, acc[1][e], off);
          }
        }
        if (live_unit && sl == 0) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int h = 8 * o + e;
            if (h < heads_here) {
              const size_t idx = (row0 + h) * kLatent + d0 + 2 * pr;
              if (p.out_dtype == MLA_FP4_OUT_BF16) {
                __nv_bfloat162 b2 = __floats2bfloat162_rn(acc[0][e], acc[1][e]);
                *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(p.out) + idx) = *reinterpret_cast<uint32_t*>(&b2);
              } else if (p.out_dtype == MLA_FP4_OUT_F32) {
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + idx) = make_float2(acc[0][e], acc[1][e]);
              } else {
                *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(p.out) + idx) =
                    __nv_cvt_float2_to_fp8x2(make_float2(acc[0][e], acc[1][e]), __NV_SATFINITE, __NV_E4M3);
              }
            }
          }
        }
      }
      if (tid == 0) MLA_TRACE(3, 1u, 5);
    }
    __syncthreads();
    if (tid == 0) {  // the last CTA through leaves the counters of this request at zero
      const int old = atomicAdd(done, 1);
      if (old == np - 1) {
        *done = 0;
        *arrived = 0;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1)
mla_fp4_decode_sm100_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_q_lat,
                            const __grid_constant__ CUtensorMap map_q_rope, const __grid_constant__ CUtensorMap map_rope,
                            const __grid_constant__ CUtensorMap map_lat) {
  extern __shared__ uint8_t smem_raw[];
  Ctx c;
  {
    uint32_t raw = ptx::smem_u32(smem_raw);
    uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
    c.smem = raw + pad;
    c.smem_ptr = smem_raw + pad;
  }
  c.misc = reinterpret_cast<Misc*>(c.smem_ptr + kOffMisc);
  c.status = p.status;
#ifdef MLA_FP4_TRACE
  c.trace_cta = (p.status && p.status[7] >= 0 && p.status[7] < int(gridDim.x) && p.status[7] != 0) ? p.status[7] : int(gridDim.x) - 1;
#endif
  const int tid = threadIdx.x;
  const int warp = tid >> 5;

  if (warp == 0) {
    Walker w = make_walker(p.seq_lens, p.batch, p.groups, blockIdx.x, gridDim.x);
    if (tid == 0) {
      c.misc->walker = w;
      c.misc->abort = 0;
      c.misc->n_merge = 0;
      stage_segments(c);
    }
    __syncwarp();
    ptx::tmem_alloc(c.smem + kOffMisc + offsetof(Misc, tmem_base), 512);
    ptx::tmem_relinquish();
  } else if (warp == kWarpTMA && (tid & 31) == 0) {
    for (int s = 0; s < kStages; ++s) {
      for (int j = 0; j < kBlocks; ++j) {
        ptx::mbar_init(bar_addr(c, bar_kv_full(s, j)), 1);
        ptx::mbar_init(bar_addr(c, bar_kv_empty(s, j)), 1);
      }
      ptx::mbar_init(bar_addr(c, bar_aux_full(s)), 1);
      ptx::mbar_init(bar_addr(c, bar_s_full(s)), 1);
      ptx::mbar_init(bar_addr(c, bar_s_empty(s)), kSoftmaxThreads);
      ptx::mbar_init(bar_addr(c, bar_p_full(s)), kSoftmaxThreads);
    }
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
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = c.misc->tmem_base;
  if (tid == 0) MLA_TRACE(3, 0u, 0);
#ifdef MLA_FP4_TRACE
  auto gtimer = [] { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
  unsigned long long* cta_times = p.status ? reinterpret_cast<unsigned long long*>(p.status + 8) + 12 * 16 * 8 + 3 * blockIdx.x : nullptr;
  if (tid == 0 && cta_times) cta_times[0] = gtimer();
#endif
  // Let a dependent kernel (the split-KV combine) start its launch and prologue early; it still waits
  // for this whole grid before it reads the partial slots.
  if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  RoleState st;
  st.it = 0;
  st.seg = 0;
  st.part = 0;
  // Rounds: almost always exactly one; more only when a CTA's range spans more than kMaxSeg requests.
  for (;;) {
    if (warp >= kWarpSoftmax0) {
      softmax_role(p, c, tmem, tid - 32 * kWarpSoftmax0, st);
    } else if (warp == kWarpQK) {
      qk_role(c, tmem, st);
    } else if (warp == kWarpPV || warp == kWarpPV2) {
      pv_role(c, tmem, st, uint32_t(warp - kWarpPV));
    } else if (warp == kWarpTMA) {
      tma_role(p, c, &map_q_lat, &map_q_rope, &map_rope, &map_lat, st);
    }
    const int more = c.misc->more;
    __syncthreads();  // every role is done with the staged segments
    if (!more) break;
    if (tid == 0) stage_segments(c);
    __syncthreads();
  }

  // drain: everything issued has completed before TMEM is released
  if (warp == kWarpQK || warp == kWarpPV || warp == kWarpPV2) {  // a commit covers the MMAs of the thread that executes it
    if (ptx::elect_one()) {
      ptx::umma_commit(bar_addr(c, kBarDrain));
      drain_wait(c, kBarDrain, 0);
    }
    __syncwarp();
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

}  // namespace

cudaError_t launch_decode_sm100(const DecodeParams& p, int num_ctas, cudaStream_t stream, const char** err) {
  *err = nullptr;
  CUtensorMap map_q_lat, map_q_rope, map_rope;
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
  CUtensorMap map_lat;
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
  {
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
      e = cudaFuncSetAttribute(mla_fp4_decode_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemAlloc));
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemAlloc;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // the CTAs wait for one another in the tail merge
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.fused_merge ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, mla_fp4_decode_sm100_kernel, p, map_q_lat, map_q_rope, map_rope, map_lat);
}

}  // namespace mla

// FP4 MLA decode for sm_100a: persistent, warp-specialised, tcgen05 + TMEM + TMA.
//
// One CTA per SM walks a contiguous range of 128-token KV tiles (common.cuh: work partition).
// For a tile of request b and a group of 64 query heads the CTA computes, with tokens on the
// MMA M axis ("swapped" orientation, so 64 heads do not waste half of a 128-row MMA):
//
//   S_lat^T [128 tok, 64 head] = K_lat (E4M3, 128x512)  . Q_lat^T      16 x tcgen05.mma K=32
//   S_rope^T[128 tok, 64 head] = K_rope(E4M3, 128x64)   . Q_rope^T      2 x tcgen05.mma
//   x = (scale_t * S_lat + S_rope) * softmax_scale*log2(e)              per token row, registers
//   P' = exp2(x - m_head) * scale_t, split into E4M3 hi + E4M3 lo       (two terms ~ 8 mantissa bits)
//   O^T[512 dim, 64 head] += V^T (E4M3, MN-major view of the same K_lat tile) . (P'_hi + P'_lo)
//
// The packed E2M1 latent is read from global memory straight into the registers of eight
// dequant warps (one tile ahead), expanded to E4M3 with a byte-permute table and written once
// into 128-byte-swizzled shared memory, where the very same bytes serve as the K-major A operand
// of QK^T and as the MN-major A operand of PV.  RoPE bytes, per-token scales and Q arrive by TMA.
//
// Warp roles (512 threads): 0-3 softmax / O rescale / epilogue (TMEM lane = token or dim),
// 4-11 latent load + dequant, 12 MMA issue, 13 TMA issue, 14-15 idle.
//
// Every wait is bounded: when a wait expires the CTA records MLA_FP4_ERR_DEVICE_TIMEOUT in the
// status words, stops issuing work, drains and exits normally.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <mutex>

#include "common.cuh"
#include "dequant.cuh"
#include "launch.h"
#include "ptx_sm100.cuh"

namespace mla {

namespace {

constexpr int kThreads = 512;
constexpr int kSoftmaxThreads = 128;
constexpr int kDequantThreads = 256;
constexpr int kDequantWarps = kDequantThreads / 32;
constexpr int kStages = 2;
constexpr int kBlocks = 4;                 // 128-dim blocks of the latent
constexpr int kBlockBytes = kTile * 128;   // 16 KiB: [128 tokens][128 B], 128B swizzle
constexpr float kPShift = 6.0f;            // P' = 2^(y - M + 6): keeps the E4M3 lo term out of the subnormals
constexpr float kLazyThreshold = 2.0f;     // running max is refreshed only when exceeded by 2^2

// shared memory map (bytes from a 1024-aligned base)
constexpr uint32_t kOffKV = 0;                                            // [2][4][16384]
constexpr uint32_t kOffRope = kOffKV + kStages * kBlocks * kBlockBytes;   // [2][128][64]  64B swizzle
constexpr uint32_t kOffQLat = kOffRope + kStages * kTile * 64;            // [4][64][128]  128B swizzle
constexpr uint32_t kOffQRope = kOffQLat + kBlocks * kGroupHeads * 128;    // [64][64]      64B swizzle
constexpr uint32_t kOffP = kOffQRope + kGroupHeads * 64;                  // [2][hi,lo][128][64] 64B swizzle (MN-major)
constexpr uint32_t kOffScale = kOffP + kStages * 2 * kTile * 64;          // [2][128] f32
constexpr uint32_t kOffM = kOffScale + kStages * kTile * 4;               // [64] f32 running reference (M - shift)
constexpr uint32_t kOffF = kOffM + kGroupHeads * 4;                       // [64] f32 rescale factor
constexpr uint32_t kOffWmax = kOffF + kGroupHeads * 4;                    // [4][64] f32 per-warp column max / sum
constexpr uint32_t kOffLinv = kOffWmax + 4 * kGroupHeads * 4;             // [64] f32 output_scale / l
constexpr uint32_t kOffLse = kOffLinv + kGroupHeads * 4;                  // [64] f32
constexpr uint32_t kOffBars = kOffLse + kGroupHeads * 4;                  // mbarriers (8 B each)
constexpr int kNumBars = 2 * 4 /*kv_full*/ + 2 * 4 /*kv_empty*/ + 2 /*aux_full*/ + 2 /*s_full*/ + 2 /*s_empty*/ +
                         2 /*p_full*/ + 1 /*q_full*/ + 1 /*q_empty*/ + 1 /*o_free*/ + 1 /*drain*/;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;                    // tmem base, abort flag, walker
constexpr uint32_t kSmemBytes = kOffMisc + 256;
constexpr uint32_t kSmemAlloc = kSmemBytes + 1024;                        // slack for manual 1024-alignment
static_assert(kSmemAlloc <= 232448, "shared memory budget exceeded");
static_assert(kOffBars % 8 == 0 && kOffMisc % 8 == 0, "barrier alignment");

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

constexpr uint32_t kIdescQK = ptx::idesc_e4m3(128, kGroupHeads, false, false);
constexpr uint32_t kIdescPV = ptx::idesc_e4m3(128, kGroupHeads, true, true);

struct Misc {
  uint32_t tmem_base;
  volatile int abort;
  Walker walker;
};

struct Ctx {
  uint32_t smem;      // shared-space address of the aligned base
  uint8_t* smem_ptr;  // generic pointer to the same
  Misc* misc;
  int32_t* status;
};

__device__ __forceinline__ uint32_t bar_addr(const Ctx& c, int idx) { return c.smem + kOffBars + 8u * idx; }

// Bounded wait.  Returns false (and flags the CTA) when the wait expires or the CTA is aborting.
__device__ __forceinline__ bool wait_slow(const Ctx& c, int idx, uint32_t parity) {
  const uint32_t bar = bar_addr(c, idx);
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if (c.misc->abort) return false;
    if (i > 64) __nanosleep(64);
  }
  c.misc->abort = 1;
  if (c.status) {
    if (atomicCAS(c.status, 0, MLA_FP4_ERR_DEVICE_TIMEOUT) == 0) {
      c.status[1] = idx;
      c.status[2] = blockIdx.x;
      c.status[3] = threadIdx.x;
      c.status[4] = int(parity);
    }
  }
  return false;
}
__device__ __forceinline__ bool wait(const Ctx& c, int idx, uint32_t parity) {
  if (c.misc->abort) return false;
  if (ptx::mbar_try_wait(bar_addr(c, idx), parity)) return true;
  return wait_slow(c, idx, parity);
}

// Bounded wait that ignores the abort flag: used only to let in-flight asynchronous work land
// before the CTA exits.
__device__ __forceinline__ void drain_wait(const Ctx& c, int idx, uint32_t parity) {
  const uint32_t bar = bar_addr(c, idx);
  for (uint32_t i = 0; i < (1u << 20); ++i) {
    if (ptx::mbar_try_wait(bar, parity)) return;
    __nanosleep(64);
  }
}

// Tile cursor: the CTA's tiles in order, with the segment each belongs to.
struct Cursor {
  Walker w;
  Segment s;
  int t;
  bool valid;
  int seg_index;  // running count of segments entered
  __device__ __forceinline__ void init(const Walker& wk) { w = wk; valid = false; t = 0; seg_index = -1; s.tile_end = 0; }
  // advance to the next tile; returns false at the end of the CTA's range
  __device__ __forceinline__ bool advance() {
    if (valid && t + 1 < s.tile_end) { ++t; return true; }
    valid = w.next(s);
    if (valid) { t = s.tile_begin; ++seg_index; }
    return valid;
  }
  __device__ __forceinline__ bool first_of_segment() const { return t == s.tile_begin; }
  __device__ __forceinline__ bool last_of_segment() const { return t + 1 == s.tile_end; }
};

// ------------------------------------------------------------------------------------------
// role: latent load + dequant (warps 4..11)
// ------------------------------------------------------------------------------------------
struct RowSrc {
  const uint8_t* p0;  // row pointer of token (tile*128 + r0), nullptr when the token is beyond seq_len
  const uint8_t* p1;  // same for r0 + 64
};

__device__ __forceinline__ RowSrc row_sources(const DecodeParams& p, const Cursor& c, int r0) {
  RowSrc rs;
  const uint8_t* cache = reinterpret_cast<const uint8_t*>(p.kv_cache);
  const int tok0 = c.t * kTile + r0, tok1 = tok0 + 64;
  rs.p0 = nullptr; rs.p1 = nullptr;
  if (tok0 < c.s.seq_len) {
    int pg = __ldg(p.block_tables + size_t(c.s.b) * p.block_table_stride + tok0 / p.page_size);
    rs.p0 = cache + (size_t(pg) * p.page_size + tok0 % p.page_size) * kRowBytes;
  }
  if (tok1 < c.s.seq_len) {
    int pg = __ldg(p.block_tables + size_t(c.s.b) * p.block_table_stride + tok1 / p.page_size);
    rs.p1 = cache + (size_t(pg) * p.page_size + tok1 % p.page_size) * kRowBytes;
  }
  return rs;
}

__device__ __forceinline__ uint4 ldg_nc(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// 16 packed bytes (32 codes) -> two 16-byte E4M3 chunks stored at dst and dst2 (already swizzled)
__device__ __forceinline__ void dequant_store(const uint4& v, uint32_t dst_a, uint32_t dst_b) {
  uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
  e2m1x8_to_e4m3x8(v.x, a0, a1);
  e2m1x8_to_e4m3x8(v.y, a2, a3);
  e2m1x8_to_e4m3x8(v.z, b0, b1);
  e2m1x8_to_e4m3x8(v.w, b2, b3);
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst_a), "r"(a0), "r"(a1), "r"(a2), "r"(a3) : "memory");
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst_b), "r"(b0), "r"(b1), "r"(b2), "r"(b3) : "memory");
}

__device__ __forceinline__ void dequant_role(const DecodeParams& p, const Ctx& c, int dtid) {
  const int r0 = dtid >> 2;    // 0..63, second row is r0 + 64
  const int ch = dtid & 3;     // 16-byte packed chunk inside the 64-byte slice of a block
  const int lane = dtid & 31;
  Cursor cur;
  cur.init(c.misc->walker);
  if (!cur.advance()) return;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 regs[kBlocks][2];
  RowSrc src = row_sources(p, cur, r0);
#pragma unroll
  for (int j = 0; j < kBlocks; ++j) {
    regs[j][0] = src.p0 ? ldg_nc(src.p0 + 64 * j + 16 * ch) : zero;
    regs[j][1] = src.p1 ? ldg_nc(src.p1 + 64 * j + 16 * ch) : zero;
  }
  // swizzled destinations inside a block: row*128 + ((2*ch + e) ^ (row & 7)) * 16
  const uint32_t sw0 = uint32_t(r0 & 7);  // (r0 + 64) & 7 is the same
  const uint32_t off_a = uint32_t(r0) * 128u + ((uint32_t(2 * ch) ^ sw0) << 4);
  const uint32_t off_b = uint32_t(r0) * 128u + ((uint32_t(2 * ch + 1) ^ sw0) << 4);

  uint32_t it = 0;
  bool more = true;
  while (more) {
    const int s = it & 1;
    const uint32_t k = it >> 1;
    Cursor nxt = cur;
    more = nxt.advance();
    RowSrc nsrc;
    nsrc.p0 = nullptr; nsrc.p1 = nullptr;
    if (more) nsrc = row_sources(p, nxt, r0);
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      if (k >= 1) wait(c, bar_kv_empty(s, j), (k - 1) & 1);
      const uint32_t base = c.smem + kOffKV + uint32_t(s * kBlocks + j) * kBlockBytes;
      dequant_store(regs[j][0], base + off_a, base + off_b);
      dequant_store(regs[j][1], base + off_a + 64u * 128u, base + off_b + 64u * 128u);
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_addr(c, bar_kv_full(s, j)));
      if (more) {
        regs[j][0] = nsrc.p0 ? ldg_nc(nsrc.p0 + 64 * j + 16 * ch) : zero;
        regs[j][1] = nsrc.p1 ? ldg_nc(nsrc.p1 + 64 * j + 16 * ch) : zero;
      }
    }
    cur = nxt;
    ++it;
  }
}

// ------------------------------------------------------------------------------------------
// role: TMA issue (warp 13, one lane): Q per segment; RoPE bytes + scales per tile
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_role(const DecodeParams& p, const Ctx& c, const CUtensorMap* map_q_lat,
                                         const CUtensorMap* map_q_rope, const CUtensorMap* map_rope) {
  Cursor cur;
  cur.init(c.misc->walker);
  uint32_t it = 0;
  const int ppt = kTile / p.page_size;  // pages per tile
  const uint32_t page_rope_bytes = uint32_t(p.page_size) * 64u;
  const uint32_t page_scale_bytes = uint32_t(p.page_size) * 4u;
  while (cur.advance()) {
    if (cur.first_of_segment()) {
      const uint32_t seg = uint32_t(cur.seg_index);
      if (seg >= 1) wait(c, kBarQEmpty, (seg - 1) & 1);
      if (!c.misc->abort) {
        int qpos, head0;
        group_coords(cur.s.g, p.num_heads, qpos, head0);
        const uint32_t bar = bar_addr(c, kBarQFull);
        ptx::mbar_arrive_expect_tx(bar, kGroupHeads * kQDim);
#pragma unroll
        for (int j = 0; j < kBlocks; ++j)
          ptx::tma_load_4d(c.smem + kOffQLat + j * kGroupHeads * 128, map_q_lat, bar, 128 * j, head0, qpos, cur.s.b);
        ptx::tma_load_4d(c.smem + kOffQRope, map_q_rope, bar, kLatent, head0, qpos, cur.s.b);
      }
    }
    const int s = it & 1;
    const uint32_t k = it >> 1;
    if (k >= 1) wait(c, bar_kv_empty(s, 3), (k - 1) & 1);
    if (!c.misc->abort) {
      const int tok0 = cur.t * kTile;
      const int pages_total = (cur.s.seq_len + p.page_size - 1) / p.page_size;
      const int lp0 = tok0 / p.page_size;
      const int np = min(ppt, pages_total - lp0);
      const uint32_t bar = bar_addr(c, bar_aux_full(s));
      ptx::mbar_arrive_expect_tx(bar, uint32_t(np) * (page_rope_bytes + page_scale_bytes));
      const int32_t* bt = p.block_tables + size_t(cur.s.b) * p.block_table_stride + lp0;
      for (int i = 0; i < np; ++i) {
        const int pg = __ldg(bt + i);
        ptx::tma_load_3d(c.smem + kOffRope + uint32_t(s) * kTile * 64 + uint32_t(i) * page_rope_bytes, map_rope, bar,
                         kLatent / 2, 0, pg);
        ptx::bulk_load(c.smem + kOffScale + uint32_t(s) * kTile * 4 + uint32_t(i) * page_scale_bytes,
                       p.kv_cache_sf + size_t(pg) * p.page_size, page_scale_bytes, bar);
      }
    }
    ++it;
  }
  if (c.misc->abort) {  // let copies that were issued but never consumed land before exit
    for (int s = 0; s < kStages; ++s) {
      const uint32_t used = (it + 1 - s) >> 1;  // tiles issued on stage s
      if (used >= 1) drain_wait(c, bar_aux_full(s), (used - 1) & 1);
    }
    if (cur.seg_index >= 0) drain_wait(c, kBarQFull, uint32_t(cur.seg_index) & 1);
  }
}

// ------------------------------------------------------------------------------------------
// role: MMA issue (warp 12, one lane)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void issue_qk(const Ctx& c, uint32_t it, uint32_t tmem) {
  const int s = it & 1;
  const uint32_t k = it >> 1;
  if (k >= 1) wait(c, bar_s_empty(s), (k - 1) & 1);
  wait(c, bar_aux_full(s), k & 1);
  const uint32_t d_lat = tmem + kColSLat + 64u * s;
  const uint32_t d_rope = tmem + kColSRope + 64u * s;
#pragma unroll
  for (int j = 0; j < kBlocks; ++j) {
    wait(c, bar_kv_full(s, j), k & 1);
    if (c.misc->abort) continue;
    ptx::tc_fence_after();
    const uint32_t a_base = c.smem + kOffKV + uint32_t(s * kBlocks + j) * kBlockBytes;
    const uint32_t b_base = c.smem + kOffQLat + uint32_t(j) * kGroupHeads * 128;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint64_t ad = ptx::smem_desc(a_base + 32 * ks, 16, 1024, 2);
      const uint64_t bd = ptx::smem_desc(b_base + 32 * ks, 16, 1024, 2);
      ptx::umma_f8(d_lat, ad, bd, kIdescQK, (j | ks) ? 1u : 0u);
    }
  }
  if (!c.misc->abort) {
    const uint32_t a_base = c.smem + kOffRope + uint32_t(s) * kTile * 64;
    const uint32_t b_base = c.smem + kOffQRope;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const uint64_t ad = ptx::smem_desc(a_base + 32 * ks, 16, 512, 4);
      const uint64_t bd = ptx::smem_desc(b_base + 32 * ks, 16, 512, 4);
      ptx::umma_f8(d_rope, ad, bd, kIdescQK, ks ? 1u : 0u);
    }
    ptx::umma_commit(bar_addr(c, bar_s_full(s)));
  }
}

__device__ __forceinline__ void issue_pv(const Ctx& c, uint32_t it, uint32_t tmem, bool first_of_segment, uint32_t seg) {
  const int s = it & 1;
  const uint32_t k = it >> 1;
  wait(c, bar_p_full(s), k & 1);
  if (first_of_segment && seg >= 1) wait(c, kBarOFree, (seg - 1) & 1);
  if (c.misc->abort) return;
  ptx::tc_fence_after();
  const uint32_t p_hi = c.smem + kOffP + uint32_t(s) * 2 * kTile * 64;
  const uint32_t p_lo = p_hi + kTile * 64;
#pragma unroll
  for (int j = 0; j < kBlocks; ++j) {
    const uint32_t a_base = c.smem + kOffKV + uint32_t(s * kBlocks + j) * kBlockBytes;
    const uint32_t d = tmem + kColO + 64u * j;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      // A = V^T: MN-major, 128-byte swizzle; 32 tokens per step = 4 groups of 8 rows of 128 B
      const uint64_t ad = ptx::smem_desc(a_base + 4096 * ks, kBlockBytes, 1024, 2);
      // B = P^T: MN-major (64 heads contiguous), 64-byte swizzle; 32 tokens per step = 2048 B
      const uint64_t bh = ptx::smem_desc(p_hi + 2048 * ks, 512, 512, 4);
      const uint64_t bl = ptx::smem_desc(p_lo + 2048 * ks, 512, 512, 4);
      ptx::umma_f8(d, ad, bh, kIdescPV, (first_of_segment && ks == 0) ? 0u : 1u);
      ptx::umma_f8(d, ad, bl, kIdescPV, 1u);
    }
    ptx::umma_commit(bar_addr(c, bar_kv_empty(s, j)));
  }
}

__device__ __forceinline__ void mma_role(const Ctx& c, uint32_t tmem) {
  Cursor cur;
  cur.init(c.misc->walker);
  uint32_t it = 0;
  bool have = cur.advance();
  while (have) {
    // one segment
    const uint32_t seg = uint32_t(cur.seg_index);
    const int n = cur.s.tile_end - cur.s.tile_begin;
    wait(c, kBarQFull, seg & 1);
    issue_qk(c, it, tmem);
    for (int i = 0; i < n; ++i) {
      if (i + 1 < n) issue_qk(c, it + i + 1, tmem);
      else if (!c.misc->abort) ptx::umma_commit(bar_addr(c, kBarQEmpty));  // every QK of this segment has been issued
      issue_pv(c, it + i, tmem, i == 0, seg);
    }
    it += n;
    // skip the cursor to the next segment
    for (int i = 0; i < n; ++i) have = cur.advance();
  }
  // drain: everything issued has completed before TMEM is released
  ptx::umma_commit(bar_addr(c, kBarDrain));
  drain_wait(c, kBarDrain, 0);
}

// ------------------------------------------------------------------------------------------
// role: softmax / rescale / epilogue (warps 0..3, thread = TMEM lane)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float* smem_f(const Ctx& c, uint32_t off) { return reinterpret_cast<float*>(c.smem_ptr + off); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float cc, float d, uint32_t& lo_out) {
  // two-term split of four values: hi = e4m3(v), lo = e4m3(v - hi)
  __half2 h01 = __floats2half2_rn(a, b), h23 = __floats2half2_rn(cc, d);
  __nv_fp8x2_storage_t hi01 = __nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&h01), __NV_SATFINITE, __NV_E4M3);
  __nv_fp8x2_storage_t hi23 = __nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&h23), __NV_SATFINITE, __NV_E4M3);
  __half2_raw b01 = __nv_cvt_fp8x2_to_halfraw2(hi01, __NV_E4M3);
  __half2_raw b23 = __nv_cvt_fp8x2_to_halfraw2(hi23, __NV_E4M3);
  __half2 r01 = __hsub2(h01, *reinterpret_cast<__half2*>(&b01));
  __half2 r23 = __hsub2(h23, *reinterpret_cast<__half2*>(&b23));
  __nv_fp8x2_storage_t lo01 = __nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&r01), __NV_SATFINITE, __NV_E4M3);
  __nv_fp8x2_storage_t lo23 = __nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&r23), __NV_SATFINITE, __NV_E4M3);
  lo_out = uint32_t(lo01) | (uint32_t(lo23) << 16);
  return uint32_t(hi01) | (uint32_t(hi23) << 16);
}

__device__ __forceinline__ void store_out_elem(void* out, int out_dtype, size_t idx, float v) {
  if (out_dtype == MLA_FP4_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(out)[idx] = v;
}

__device__ __forceinline__ void softmax_role(const DecodeParams& p, const Ctx& c, uint32_t tmem, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  const uint32_t lane_base = (uint32_t(warp) * 32u) << 16;
  const float cscale = p.softmax_scale * kLog2e;
  float* m_s = smem_f(c, kOffM);
  float* f_s = smem_f(c, kOffF);
  float* wred = smem_f(c, kOffWmax);
  float* linv_s = smem_f(c, kOffLinv);
  float* lse_s = smem_f(c, kOffLse);

  Cursor cur;
  cur.init(c.misc->walker);
  uint32_t it = 0;
  float l[kGroupHeads];
  bool have_m = false;

  while (cur.advance()) {
    const int s = it & 1;
    const uint32_t k = it >> 1;
    if (cur.first_of_segment()) {
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) l[h] = 0.f;
      have_m = false;
    }
    // per-token scale
    wait(c, bar_aux_full(s), k & 1);
    const bool valid = (cur.t * kTile + tid) < cur.s.seq_len;
    float sc = smem_f(c, kOffScale)[s * kTile + tid];
    sc = valid ? sc : 0.f;
    const float lg = valid ? log2f(fmaxf(fabsf(sc), 8.67361738e-19f)) : 0.f;  // floor 2^-60

    wait(c, bar_s_full(s), k & 1);
    ptx::tc_fence_after();
    const uint32_t t_lat = tmem + lane_base + kColSLat + 64u * s;
    const uint32_t t_rope = tmem + lane_base + kColSRope + 64u * s;

    // ---- pass 1: does any score exceed the running reference by more than the lazy threshold?
    bool need = !have_m;
    if (have_m) {
      float mx = -INFINITY;
#pragma unroll
      for (int cidx = 0; cidx < 4; ++cidx) {
        uint32_t a[16], b[16];
        ptx::tmem_ld16(t_lat + 16 * cidx, a);
        ptx::tmem_ld16(t_rope + 16 * cidx, b);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x = fmaf(__uint_as_float(a[i]), sc, __uint_as_float(b[i])) * cscale;
          mx = fmaxf(mx, x - m_s[16 * cidx + i]);
        }
      }
      need = valid && (mx > (kPShift + kLazyThreshold) - lg);
    }
    const bool update = ptx::bar_or(1, kSoftmaxThreads, need);

    if (update) {
      // ---- column max of y = x + log2(scale_t) over the 128 tokens of the tile
      float mine0 = -INFINITY, mine1 = -INFINITY;
#pragma unroll
      for (int cidx = 0; cidx < 4; ++cidx) {
        uint32_t a[16], b[16];
        ptx::tmem_ld16(t_lat + 16 * cidx, a);
        ptx::tmem_ld16(t_rope + 16 * cidx, b);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x = fmaf(__uint_as_float(a[i]), sc, __uint_as_float(b[i])) * cscale;
          float y = valid ? x + lg : -INFINITY;
          float r = ptx::redux_max_f32(y);
          const int h = 16 * cidx + i;
          if (lane == (h & 31)) { if (h < 32) mine0 = r; else mine1 = r; }
        }
      }
      wred[warp * kGroupHeads + lane] = mine0;
      wred[warp * kGroupHeads + 32 + lane] = mine1;
      ptx::bar_sync(1, kSoftmaxThreads);
      if (tid < kGroupHeads) {
        float mnew = fmaxf(fmaxf(wred[tid], wred[kGroupHeads + tid]),
                           fmaxf(wred[2 * kGroupHeads + tid], wred[3 * kGroupHeads + tid])) - kPShift;
        float mold = have_m ? m_s[tid] : -INFINITY;
        mnew = fmaxf(mnew, mold);
        f_s[tid] = have_m ? ptx::ex2(mold - mnew) : 0.f;
        m_s[tid] = mnew;
      }
      ptx::bar_sync(1, kSoftmaxThreads);
      if (have_m) {
#pragma unroll
        for (int h = 0; h < kGroupHeads; ++h) l[h] *= f_s[h];
        // O^T is rescaled in place once the previous tile's PV has completed
        const uint32_t pit = it - 1;
        wait(c, bar_kv_empty(pit & 1, 3), (pit >> 1) & 1);
        ptx::tc_fence_after();
#pragma unroll 1
        for (int j = 0; j < kBlocks; ++j) {
#pragma unroll
          for (int cidx = 0; cidx < 4; ++cidx) {
            uint32_t o[16];
            const uint32_t ta = tmem + lane_base + kColO + 64u * j + 16u * cidx;
            ptx::tmem_ld16(ta, o);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f_s[16 * cidx + i]);
            ptx::tmem_st16(ta, o);
          }
        }
        ptx::tmem_wait_st();
      }
      have_m = true;
    }

    // ---- the P buffer of this stage is free once PV of tile it-2 has completed
    if (k >= 1) wait(c, bar_kv_empty(s, 3), (k - 1) & 1);

    // ---- pass 2: probabilities, row sums, two-term E4M3 P' into shared memory
    const uint32_t p_hi = c.smem + kOffP + uint32_t(s) * 2 * kTile * 64 + uint32_t(tid) * 64u;
    const uint32_t p_lo = p_hi + kTile * 64;
    const uint32_t psw = (uint32_t(tid) >> 1) & 3u;
#pragma unroll
    for (int cidx = 0; cidx < 4; ++cidx) {
      uint32_t a[16], b[16];
      ptx::tmem_ld16(t_lat + 16 * cidx, a);
      ptx::tmem_ld16(t_rope + 16 * cidx, b);
      ptx::tmem_wait_ld();
      if (cidx == 3) {  // every S column of this stage has been read
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_addr(c, bar_s_empty(s)));
      }
      float pv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float x = fmaf(__uint_as_float(a[i]), sc, __uint_as_float(b[i])) * cscale;
        float e = valid ? ptx::ex2(x - m_s[16 * cidx + i]) : 0.f;
        l[16 * cidx + i] += e;
        pv[i] = e * sc;
      }
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) hi[q4] = pack_e4m3x4(pv[4 * q4], pv[4 * q4 + 1], pv[4 * q4 + 2], pv[4 * q4 + 3], lo[q4]);
      const uint32_t off = ((uint32_t(cidx) ^ psw) << 4);
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(p_hi + off), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(p_lo + off), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before();  // orders the O rescale (tcgen05.st) before the arrive as well
    ptx::mbar_arrive(bar_addr(c, bar_p_full(s)));

    // ---- segment epilogue
    if (cur.last_of_segment()) {
      // total row sums: reduce the per-token partial sums over the 128 token threads
      float mine0 = 0.f, mine1 = 0.f;
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) {
        float v = l[h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == (h & 31)) { if (h < 32) mine0 = v; else mine1 = v; }
      }
      ptx::bar_sync(1, kSoftmaxThreads);  // wred is free (column-max readers are done)
      wred[warp * kGroupHeads + lane] = mine0;
      wred[warp * kGroupHeads + 32 + lane] = mine1;
      ptx::bar_sync(1, kSoftmaxThreads);
      if (tid < kGroupHeads) {
        float L = (wred[tid] + wred[kGroupHeads + tid]) + (wred[2 * kGroupHeads + tid] + wred[3 * kGroupHeads + tid]);
        linv_s[tid] = p.output_scale / L;
        lse_s[tid] = log2f(L) + m_s[tid];
      }
      ptx::bar_sync(1, kSoftmaxThreads);

      int qpos, head0;
      group_coords(cur.s.g, p.num_heads, qpos, head0);
      const int heads_here = min(kGroupHeads, p.num_heads - head0);
      const size_t row0 = (size_t(cur.s.b) * p.q_len + qpos) * p.num_heads + head0;
      // wait for the PV of this (last) tile
      wait(c, bar_kv_empty(s, 3), k & 1);
      ptx::tc_fence_after();
      const bool ok = !c.misc->abort;
      if (cur.s.slot < 0) {
#pragma unroll 1
        for (int j = 0; j < kBlocks; ++j) {
#pragma unroll
          for (int cidx = 0; cidx < 4; ++cidx) {
            uint32_t o[16];
            ptx::tmem_ld16(tmem + lane_base + kColO + 64u * j + 16u * cidx, o);
            ptx::tmem_wait_ld();
            if (ok) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int h = 16 * cidx + i;
                if (h < heads_here)
                  store_out_elem(p.out, p.out_dtype, (row0 + h) * kLatent + 128 * j + tid, __uint_as_float(o[i]) * linv_s[h]);
              }
            }
          }
        }
        if (ok && p.lse && tid < heads_here) p.lse[row0 + tid] = lse_s[tid];
      } else {
        float* so = reinterpret_cast<float*>(p.workspace) + size_t(cur.s.slot) * kSlotFloats;
#pragma unroll 1
        for (int j = 0; j < kBlocks; ++j) {
          float4* dst = reinterpret_cast<float4*>(so + size_t(128 * j + tid) * kGroupHeads);
#pragma unroll
          for (int cidx = 0; cidx < 4; ++cidx) {
            uint32_t o[16];
            ptx::tmem_ld16(tmem + lane_base + kColO + 64u * j + 16u * cidx, o);
            ptx::tmem_wait_ld();
            if (ok) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                float4 v;
                v.x = __uint_as_float(o[4 * q4 + 0]) * linv_s[16 * cidx + 4 * q4 + 0];
                v.y = __uint_as_float(o[4 * q4 + 1]) * linv_s[16 * cidx + 4 * q4 + 1];
                v.z = __uint_as_float(o[4 * q4 + 2]) * linv_s[16 * cidx + 4 * q4 + 2];
                v.w = __uint_as_float(o[4 * q4 + 3]) * linv_s[16 * cidx + 4 * q4 + 3];
                dst[4 * cidx + q4] = v;
              }
            }
          }
        }
        if (ok && tid < kGroupHeads) so[kSlotOFloats + tid] = lse_s[tid];
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar_addr(c, kBarOFree));
    }
    ++it;
  }
}

// ------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1)
mla_fp4_decode_sm100_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_q_lat,
                            const __grid_constant__ CUtensorMap map_q_rope, const __grid_constant__ CUtensorMap map_rope) {
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
  const int tid = threadIdx.x;
  const int warp = tid >> 5;

  if (warp == 0) {
    Walker w = make_walker(p.seq_lens, p.batch, p.groups, blockIdx.x, gridDim.x);
    if (tid == 0) {
      c.misc->walker = w;
      c.misc->abort = 0;
    }
    __syncwarp();
    ptx::tmem_alloc(c.smem + kOffMisc + offsetof(Misc, tmem_base), 512);
    ptx::tmem_relinquish();
  } else if (warp == 1 && (tid & 31) == 0) {
    for (int s = 0; s < kStages; ++s) {
      for (int j = 0; j < kBlocks; ++j) {
        ptx::mbar_init(bar_addr(c, bar_kv_full(s, j)), kDequantWarps);
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
    ptx::mbar_init(bar_addr(c, kBarDrain), 1);
    ptx::fence_barrier_init();
  } else if (warp == 13 && (tid & 31) == 0) {
    ptx::prefetch_tensormap(&map_q_lat);
    ptx::prefetch_tensormap(&map_q_rope);
    ptx::prefetch_tensormap(&map_rope);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = c.misc->tmem_base;

  if (warp < 4) {
    ptx::setmaxnreg_inc<216>();
    softmax_role(p, c, tmem, tid);
  } else if (warp < 12) {
    ptx::setmaxnreg_dec<96>();
    dequant_role(p, c, tid - 128);
  } else {
    ptx::setmaxnreg_dec<88>();
    if (warp == 12) {
      if ((tid & 31) == 0) mma_role(c, tmem);
      __syncwarp();
    } else if (warp == 13) {
      if ((tid & 31) == 0) tma_role(p, c, &map_q_lat, &map_q_rope, &map_rope);
      __syncwarp();
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
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
  mla_fp4_decode_sm100_kernel<<<num_ctas, kThreads, kSmemAlloc, stream>>>(p, map_q_lat, map_q_rope, map_rope);
  return cudaGetLastError();
}

}  // namespace mla

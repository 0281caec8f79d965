// Shared definitions of the FP4 MLA decode engine: constants, the work partition
// (used identically by the host planner, the decode kernels and the combine kernel)
// and small device helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mla_fp4_b200.h"

#define MLA_HD __host__ __device__ __forceinline__

namespace mla {

constexpr int kLatent = MLA_FP4_LATENT_DIM;        // 512
constexpr int kRope = MLA_FP4_ROPE_DIM;            // 64
constexpr int kQDim = kLatent + kRope;             // 576
constexpr int kRowBytes = MLA_FP4_ROW_BYTES;       // 320
constexpr int kTile = MLA_FP4_TILE_TOKENS;         // 128 KV tokens per tile
constexpr int kGroupHeads = MLA_FP4_GROUP_HEADS;   // 64 query heads per CTA
constexpr float kLog2e = 1.4426950408889634f;

// Split-KV partials in the workspace.  Layout:  header | tails [296] | partial O [slots]
//   * partial O of slot s: normalised O as fp16 [8 head groups][512 dims][8 heads] divided by a per-slot
//     scale (the decode kernel's lanes own one dim each: with this order a warp stores 32 dims x 8 heads =
//     512 contiguous bytes at a time; with heads innermost over all 64 it would store 16 bytes every 128).
//   * tail of slot s (272 bytes): the base-2 LSE of the 64 heads as f32, that scale (f32), the slot's flag
//     (int32, see below), 8 bytes of padding.  The tails of all slots lie side by side, so the tails of the
//     consecutive slots of one split request are one contiguous range (one bulk copy for a merging CTA).
// The scale is 6 * max|token scale| * |output_scale| / 32768 rounded up to a power of two: an
// upper bound of |O| mapped below the fp16 maximum, so the 11-bit partials can neither overflow nor
// lose the small values (fp16 spans 29 binades below that bound).  Half the bytes of f32 partials.
constexpr size_t kSlotOBytes = size_t(kLatent) * kGroupHeads * 2;
constexpr size_t kSlotTailBytes = kGroupHeads * sizeof(float) + 16;
constexpr size_t kSlotBytes = kSlotOBytes + kSlotTailBytes;  // per slot, tail and partial O together
constexpr float kSlotHalfRange = 32768.f;
// A request can be split over at most this many CTAs (= the largest decode grid accepted).
constexpr int kMaxCombineSlots = 148;
constexpr int kMaxSlots = 2 * kMaxCombineSlots;
// The workspace starts with a header.  Header words (int32):
//   [0]  generation of the last decode step that completed on this workspace
//   [1]  CTAs of the running step that have finished (zero whenever no step is running)
// Every slot's tail holds a flag: the generation of the step that last published the slot.  A step uses
// generation g = header[0] + 1.  A writer stamps the flag of a slot with g once the slot's bytes are
// visible; a merger waits until the flags of a request's slots equal g.  Flags of earlier steps never
// match, so nothing has to be reset between steps, and a step that gave up on a wait leaves the workspace
// consistent (its last CTA still advances the generation).  Each flag has a cache line of its own.
constexpr size_t kWsHeaderBytes = MLA_FP4_WORKSPACE_HEADER_BYTES;
constexpr size_t kWsTailsBytes = size_t(kMaxSlots) * kSlotTailBytes;
constexpr size_t kWsFixedBytes = kWsHeaderBytes + kWsTailsBytes;  // what mla_fp4_workspace_init zeroes
MLA_HD int32_t* ws_generation(void* ws) { return static_cast<int32_t*>(ws); }
MLA_HD int32_t* ws_finished(void* ws) { return static_cast<int32_t*>(ws) + 1; }
MLA_HD uint16_t* slot_o(void* ws, int slot) { return reinterpret_cast<uint16_t*>(static_cast<char*>(ws) + kWsFixedBytes + size_t(slot) * kSlotOBytes); }
MLA_HD const uint16_t* slot_o(const void* ws, int slot) { return reinterpret_cast<const uint16_t*>(static_cast<const char*>(ws) + kWsFixedBytes + size_t(slot) * kSlotOBytes); }
MLA_HD float* slot_lse(void* ws, int slot) { return reinterpret_cast<float*>(static_cast<char*>(ws) + kWsHeaderBytes + size_t(slot) * kSlotTailBytes); }
MLA_HD const float* slot_lse(const void* ws, int slot) { return reinterpret_cast<const float*>(static_cast<const char*>(ws) + kWsHeaderBytes + size_t(slot) * kSlotTailBytes); }
MLA_HD float* slot_scale(void* ws, int slot) { return slot_lse(ws, slot) + kGroupHeads; }
MLA_HD const float* slot_scale(const void* ws, int slot) { return slot_lse(ws, slot) + kGroupHeads; }
MLA_HD int32_t* slot_flag(void* ws, int slot) { return reinterpret_cast<int32_t*>(slot_scale(ws, slot) + 1); }
// element (dim, head) of a slot's partial O
MLA_HD size_t slot_o_index(int dim, int head) { return (size_t(head >> 3) * kLatent + size_t(dim)) * 8 + size_t(head & 7); }
// bytes a grid of num_ctas CTAs needs: the fixed part and two partial-O slots per CTA
__host__ __device__ constexpr size_t workspace_bytes_for(int num_ctas) { return kWsFixedBytes + size_t(2) * size_t(num_ctas) * kSlotOBytes; }
// power-of-two scale that maps `bound` (an upper bound of |O|) to at most kSlotHalfRange
MLA_HD float slot_scale_for(float bound) { return exp2f(ceilf(log2f(fmaxf(bound, 1e-30f) / kSlotHalfRange))); }

MLA_HD int out_elem_bytes(int out_dtype) { return out_dtype == MLA_FP4_OUT_F32 ? 4 : (out_dtype == MLA_FP4_OUT_BF16 ? 2 : 1); }

// ----------------------------------------------------------------------------------------------
// Work partition.
//
// A "virtual request" v = g * batch + b is request b seen by head group g (a group is 64 query
// heads of one query position).  Request b has tiles_b = ceil(seq_len_b / 128) tiles.  All tiles
// of all virtual requests, in v order, form a flat space of Tt = groups * sum_b tiles_b tiles.
// CTA i of n owns the contiguous flat range [Tt*i/n, Tt*(i+1)/n).  A CTA therefore walks a list
// of segments (v, tile_begin, tile_end); only its first and its last segment can cover a request
// partially.  A partial segment writes a split-KV partial into workspace slot 2*i (first
// segment of the CTA) or 2*i+1 (any later one); a segment that covers its request completely
// writes the final output itself.  The slots of every split request are merged at the end of the
// decode kernel by the CTAs that wrote them (or, in the two-kernel mode, by the combine kernel).
// ----------------------------------------------------------------------------------------------

MLA_HD int tiles_of(int seq_len) { return seq_len > 0 ? (seq_len - 1) / kTile + 1 : 0; }  // no overflow near INT_MAX

// A sequence length as the kernels use it: never more than `cap` tokens (the tokens a block-table row can
// address), so a garbage seq_lens entry cannot walk a kernel past the row.
MLA_HD int capped_len(const int32_t* seq_lens, int b, int cap) {
  const int n = seq_lens[b];
  return n < cap ? n : cap;
}

// The flat space that is cut into CTA ranges counts kPhantom extra tiles in front of every non-empty
// request: moving on to another request costs a CTA about as much as two tiles (the epilogue of the
// old one, a fresh query, a cold pipeline), so a CTA whose range holds the start of a request gets
// that many tiles less.  A piece of a range that holds nothing but phantom tiles is no segment.
constexpr int kPhantom = MLA_FP4_PHANTOM_TILES;  // measured: 2 and 3 are equally good, 1 and 4 worse
MLA_HD int vtiles_of(int seq_len) { return seq_len > 0 ? tiles_of(seq_len) + kPhantom : 0; }

// Short requests are not split.  When no request has more than kWholeTiles tiles and there are no more (request, head
// group) pairs than CTAs, pair v is decoded whole by CTA v: walking four tiles costs less than writing a partial,
// publishing it and merging (about three to four tile times), which is all a split would buy.  Every user of the
// partition (the decode kernels, the combine kernel, the host planner) takes the same decision from the same inputs.
constexpr int kWholeTiles = 4;
MLA_HD bool whole_requests(int max_real_tiles, int64_t pairs, int n) { return max_real_tiles <= kWholeTiles && pairs <= int64_t(n); }

MLA_HD int num_groups(int q_len, int num_heads) {
  return q_len * ((num_heads + kGroupHeads - 1) / kGroupHeads);
}

// Positions in the flat tile space are 32-bit: a 64-bit division is a subroutine of a hundred instructions and these
// run in the prologue of every CTA, where every instruction is fetched cold.  Valid while (Tt + 1) * (n + 1) < 2^32
// (hundreds of millions of tokens); partition_fits says so and the kernels refuse a launch beyond it.
typedef int32_t flat_t;
MLA_HD bool partition_fits(int64_t Tt, int n) { return (Tt + 1) * int64_t(n + 1) < (int64_t(1) << 32); }

MLA_HD flat_t cta_lo(flat_t Tt, int n, int i) { return flat_t((uint32_t(Tt) * uint32_t(i)) / uint32_t(n)); }

// CTA that owns flat tile f: the largest i with cta_lo(i) <= f.
MLA_HD int cta_of_tile(flat_t Tt, int n, flat_t f) {
  return int((uint32_t(f + 1) * uint32_t(n) + uint32_t(Tt) - 1u) / uint32_t(Tt)) - 1;
}

// Does CTA i write a partial of the split request whose flat range (phantom tiles first) is
// [start, start + vtiles)?  Its range must hold at least one of the request's real tiles.
MLA_HD bool cta_writes(flat_t Tt, int n, int i, flat_t start, int vtiles) {
  const flat_t lo = cta_lo(Tt, n, i), hi = cta_lo(Tt, n, i + 1);
  const flat_t a = lo > start + kPhantom ? lo : start + kPhantom, b = hi < start + vtiles ? hi : start + vtiles;
  return a < b;
}

MLA_HD int slot_of(int cta, bool first_segment_of_cta) { return 2 * cta + (first_segment_of_cta ? 0 : 1); }

// Where request (virtual) v with flat start `start` and `tiles` tiles lands: the CTAs that touch it.
struct Span {
  int cta_first, cta_last;  // inclusive
  bool split;               // more than one CTA
};
MLA_HD Span span_of(flat_t Tt, int n, flat_t start, int tiles) {
  Span s;
  s.cta_first = cta_of_tile(Tt, n, start);
  s.cta_last = cta_of_tile(Tt, n, start + tiles - 1);
  s.split = s.cta_last != s.cta_first;
  return s;
}
// Slot written by CTA i for a split request whose flat start is `start`.
MLA_HD int slot_in_span(flat_t Tt, int n, int i, flat_t start) {
  return slot_of(i, cta_lo(Tt, n, i) >= start);
}

// One segment of a CTA's walk.
struct Segment {
  int b, g;                 // request, head group
  int tile_begin, tile_end; // tiles of the request, [begin, end)
  int seq_len;
  int slot;                 // -1: covers the whole request (writes the final output)
};

// Sequential walker over the segments of one CTA.  `start_*` describe the position of the CTA's
// first flat tile and are found once per CTA (find_start on the device, a plain loop on the host).
struct Walker {
  const int32_t* seq_lens;
  int cap;         // most tokens a request may have (see capped_len)
  int batch, groups;
  flat_t f, hi;    // current flat tile, end of the CTA's range
  int b, g, t;     // current request, group, tile inside the request
  bool first;      // next segment is the first of this CTA
  int cta;
  flat_t Tt;       // size of the flat tile space (device walkers only)

  MLA_HD bool next(Segment& s) {
    while (f < hi) {
      if (g >= groups) return false;
      int sl = capped_len(seq_lens, b, cap);
      int tb = vtiles_of(sl);  // t, end, room and f count phantom tiles; the segment holds real ones
      if (t >= tb) {
        t = 0;
        if (++b == batch) { b = 0; ++g; }
        continue;
      }
      flat_t room = hi - f;
      int end = (tb - t) <= room ? tb : t + int(room);
      const bool whole = t <= kPhantom && end == tb;  // all real tiles of the request
      const int real_begin = (t > kPhantom ? t : kPhantom) - kPhantom, real_end = end - kPhantom;
      f += end - t;
      t = end;
      if (real_end <= real_begin) continue;  // nothing but phantom tiles
      s.b = b; s.g = g; s.tile_begin = real_begin; s.tile_end = real_end; s.seq_len = sl;
      s.slot = whole ? -1 : slot_of(cta, first);
      first = false;
      return true;
    }
    return false;
  }
};

// Decoded head group: which query position and which first head it covers.
MLA_HD void group_coords(int g, int num_heads, int& qpos, int& head0) {
  int per = (num_heads + kGroupHeads - 1) / kGroupHeads;
  qpos = g / per;
  head0 = (g % per) * kGroupHeads;
}

#ifdef __CUDACC__
// Warp-cooperative: total tile count of the batch. All 32 lanes must call; all get the result.
__device__ __forceinline__ int64_t warp_total_tiles(const int32_t* seq_lens, int batch, int cap, int* max_real_tiles = nullptr) {
  int lane = threadIdx.x & 31;
  int64_t acc = 0;
  int mx = 0;
  for (int i = lane; i < batch; i += 32) {
    const int v = vtiles_of(capped_len(seq_lens, i, cap));
    acc += v;
    mx = max(mx, v);
  }
  for (int o = 16; o > 0; o >>= 1) {
    acc += __shfl_xor_sync(0xffffffffu, acc, o);
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (max_real_tiles) *max_real_tiles = mx > 0 ? mx - kPhantom : 0;  // of any request
  return acc;
}

// Warp-cooperative: locate flat tile r (0 <= r < T, within one group) -> request b and tile t.
__device__ __forceinline__ void warp_locate(const int32_t* seq_lens, int batch, int cap, flat_t r, int& b_out, int& t_out) {
  int lane = threadIdx.x & 31;
  flat_t run = 0;
  b_out = batch; t_out = 0;
  for (int base = 0; base < batch; base += 32) {
    int i = base + lane;
    flat_t v = i < batch ? vtiles_of(capped_len(seq_lens, i, cap)) : 0;
    flat_t inc = v;
    for (int o = 1; o < 32; o <<= 1) {
      flat_t u = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += u;
    }
    flat_t tot = __shfl_sync(0xffffffffu, inc, 31);
    if (r < run + tot) {
      unsigned m = __ballot_sync(0xffffffffu, run + inc > r);
      int l = __ffs(m) - 1;
      flat_t exc = __shfl_sync(0xffffffffu, inc - v, l);
      b_out = base + l;
      t_out = int(r - (run + exc));
      return;
    }
    run += tot;
  }
}

// Initialise a walker for CTA `cta` of `n`. Warp-cooperative (all 32 lanes call, all get it).
__device__ __forceinline__ Walker make_walker(const int32_t* seq_lens, int batch, int cap, int groups, int cta, int n) {
  Walker w;
  w.seq_lens = seq_lens; w.cap = cap; w.batch = batch; w.groups = groups; w.cta = cta; w.first = true;
  int max_tiles;
  const int64_t T64 = warp_total_tiles(seq_lens, batch, cap, &max_tiles);
  w.f = 0; w.hi = 0; w.b = 0; w.g = groups; w.t = 0; w.Tt = 0;
  if (!partition_fits(T64 * groups, n)) {  // never with real caches; the caller reports it
    w.Tt = -1;
    return w;
  }
  const flat_t T = flat_t(T64), Tt = T * groups;
  w.Tt = Tt;
  if (whole_requests(max_tiles, int64_t(batch) * groups, n)) {  // CTA v: pair v, whole
    if (cta < batch * groups) {
      w.g = cta / batch;
      w.b = cta - w.g * batch;
      w.hi = vtiles_of(capped_len(seq_lens, w.b, cap));
    }
    return w;
  }
  w.f = cta_lo(Tt, n, cta);
  w.hi = cta_lo(Tt, n, cta + 1);
  if (T > 0 && w.f < w.hi) {
    w.g = int(uint32_t(w.f) / uint32_t(T));
    warp_locate(seq_lens, batch, cap, w.f - flat_t(w.g) * T, w.b, w.t);
  }
  return w;
}
#endif  // __CUDACC__

}  // namespace mla

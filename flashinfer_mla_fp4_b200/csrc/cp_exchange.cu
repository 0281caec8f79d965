// Decode context parallel: exchange of the per-rank partials over NVLink and their merge, in ONE kernel.
//
// Every rank has decoded its shard of the KV cache into a packed partial  [rows][512] f32 | [rows] f32 (base-2 LSE).
// The kernel on rank r, one CTA per row (round robin when there are more rows than CTAs):
//   A. pushes the row into slot r of every peer's gather buffer with ordinary 16-byte stores to peer memory (posted
//      writes over NVLink; nothing is read from a peer, no multicast of any kind).  A row travels as 512 fp16 values
//      divided by a power-of-two row scale (the row's largest magnitude mapped just below 32768, so the 11-bit values
//      neither overflow nor lose the small ones) plus its LSE and that scale.  Every 16-byte store is
//      { 4 bytes data, step, 4 bytes data, step }: the data carries its own arrival tag (each 8-byte half of an aligned
//      vector store lands whole), so there is NO flag and NO fence.  The first version of this kernel pushed bare data,
//      then fence.sys + a flag: a system-scope fence has to wait for the acknowledgement of every NVLink write in flight
//      and cost 5-7 us each (10-15 us per step, measured with globaltimer stamps), more than the transfer itself,
//   B. waits - bounded, like every wait of this library - for the same row from every peer in its OWN memory, polling
//      each 16-byte word until both tags carry the step number,
//   C. merges:  out[row] = sum_s w_s * partial_s[row],  w_s = 2^(lse_s - max) / sum  (ranks with an empty shard
//      have lse = -inf and weight 0), the arithmetic of the split-KV reduction with ranks in place of splits; the
//      rank's own row is rounded the way its peers see it, so that all ranks produce bit-identical outputs.
// Two forms, chosen by the number of ranks (or by the caller):
//   all-gather (above; 2 or 3 ranks): every rank receives every row of every peer: (world-1) x 1 MiB per rank in each
//      direction for 512 rows, one NVLink hop;
//   reduce-scatter (4 ranks and more): row i belongs to rank i % world.  Ranks push a row only to its owner; the owner
//      merges it, stores it and pushes the FINAL row, in the output type, with its LSE into the result area of every
//      peer, whose CTA of that row copies it out.  2 x (world-1)/world x 1 MiB per rank and direction whatever the
//      number of ranks, two hops.  At 8 ranks the all-gather form took 80 us per north-star step against 56 us for the
//      decode kernel alone, the NVLink volume being the limit.
// CTAs never wait for other CTAs of their grid, only for data written by other GPUs, so an ordinary launch is enough
// (all CTAs must be resident at once: a CTA that waits holds its place), and no CTA touches a word another CTA of its
// grid writes.  The step number lives in device memory, one word per CTA which that CTA advances when it is done, so a
// CUDA graph that holds the launch can be replayed (all ranks make the same sequence of calls, so CTA i of every rank
// counts alike; after a wait that ran out they no longer do: make a new exchange block).  Buffers alternate between two
// parities: a peer can be at most one step ahead (its next step needs this rank's rows of the current one), so it never
// overwrites what is being merged, and what lies in a buffer from two steps ago carries an older tag.  The launch may be
// a programmatic dependent launch: the kernel then starts while the decode kernel before it drains and waits for that
// kernel's completion before it reads.
//
// Exchange block of a rank (one allocation, zeroed, mapped by every peer through CUDA IPC):
//   int32 step[1024] (per CTA) | gather[2][world] of [max_rows] rows of 129 tagged 16-byte words
//   (128 x four fp16 values, then LSE and row scale as f32) | result[2] of [max_rows] rows of 257 tagged words
//   (up to 2 x 128 words of output values, then the LSE)
#include "common.cuh"
#include "launch.h"

#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace mla {

namespace {

constexpr int kCpThreads = 128;  // one thread per four output dims of a row

// a tagged 16-byte word: { lo, tag, hi, tag }
__device__ __forceinline__ void st_tagged(void* p, uint32_t lo, uint32_t hi, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(lo), "r"(tag), "r"(hi), "r"(tag) : "memory");
}
__device__ __forceinline__ bool ld_tagged(const void* p, uint32_t tag, uint32_t& lo, uint32_t& hi) {
  uint32_t t0, t1;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(lo), "=r"(t0), "=r"(hi), "=r"(t1) : "l"(p) : "memory");
  return t0 == tag && t1 == tag;
}
// bounded poll of one tagged word; false when it never arrived
__device__ __forceinline__ bool wait_tagged(const void* p, uint32_t tag, uint32_t polls, uint32_t& lo, uint32_t& hi) {
  for (uint32_t i = 0; i < polls; ++i) {
    if (ld_tagged(p, tag, lo, hi)) return true;
    if (i > 64) __nanosleep(100);
  }
  return false;
}
// the row as its peers see it: fp16 of value / scale, scale the power of two that maps the row's maximum below 32768
__device__ __forceinline__ float row_scale(const float4& v, float* s_max, int tid) {
  float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __syncthreads();
  if ((tid & 31) == 0) s_max[tid >> 5] = m;
  __syncthreads();
  return slot_scale_for(fmaxf(fmaxf(s_max[0], s_max[1]), fmaxf(s_max[2], s_max[3])));
}
__device__ __forceinline__ uint2 pack_row(const float4& v, float scale) {
  const float inv = 1.f / scale;  // a power of two: the division and the multiplication back are exact
  __half2 h0 = __floats2half2_rn(v.x * inv, v.y * inv), h1 = __floats2half2_rn(v.z * inv, v.w * inv);
  return make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
}
__device__ __forceinline__ float4 unpack_row(uint32_t lo, uint32_t hi) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo)), b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  return make_float4(a.x, a.y, b.x, b.y);
}
#ifdef MLA_FP4_CP_TRACE
#define CP_STAMP(i) do { if (tid == 0 && (blockIdx.x <= 1 || blockIdx.x == gridDim.x - 1)) { asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ts[i])); } } while (0)
#else
#define CP_STAMP(i)
#endif

__device__ __forceinline__ void report_timeout(const CpExchangeParams& p, int where, uint32_t step) {
  if (p.status && atomicCAS(p.status, 0, MLA_FP4_ERR_DEVICE_TIMEOUT) == 0) {
    p.status[1] = where;  // 300 + rank: that peer's row (its LSE word) never arrived; 310: values of a row; 320: a final row
    p.status[2] = blockIdx.x;
    p.status[3] = int(step);
  }
}

// four output values of a thread as they lie in `out`: 16 bytes (f32), 8 (bf16) or 4 (E4M3)
__device__ __forceinline__ uint4 pack_out(const float4& v, int out_dtype) {
  if (out_dtype == MLA_FP4_OUT_F32) return make_uint4(__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w));
  if (out_dtype == MLA_FP4_OUT_BF16) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    return make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b), 0u, 0u);
  }
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x, v.y), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z, v.w), __NV_SATFINITE, __NV_E4M3);
  return make_uint4(lo | (hi << 16), 0u, 0u, 0u);
}
__device__ __forceinline__ void store_packed(void* out, int out_dtype, size_t idx, const uint4& w) {
  if (out_dtype == MLA_FP4_OUT_F32) *reinterpret_cast<uint4*>(static_cast<float*>(out) + idx) = w;
  else if (out_dtype == MLA_FP4_OUT_BF16) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + idx) = make_uint2(w.x, w.y);
  else *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(out) + idx) = w.x;
}

__global__ void __launch_bounds__(kCpThreads) cp_exchange_merge_kernel(const CpExchangeParams p) {
#ifdef MLA_FP4_CP_TRACE
  unsigned long long ts[8] = {};
#endif
  __shared__ float s_w[MLA_FP4_CP_MAX_RANKS];
  __shared__ float s_max[kCpThreads / 32];
  __shared__ float s_lse;
  const int tid = threadIdx.x;
  void* const my = p.block[p.rank];
  CP_STAMP(0);
  if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");  // the decode kernel before this one has completed
  CP_STAMP(1);
  // the step of this launch: one more than the last one this CTA completed
  const uint32_t step = uint32_t(*cp_step_word(my, blockIdx.x)) + 1u;
  const int parity = int(step & 1u);
  const uint32_t polls = p.wait_polls;
  const bool scatter = p.algo == MLA_FP4_CP_REDUCE_SCATTER;

  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const int owner = int(row % p.world);  // reduce-scatter: the rank that merges this row
    const bool merges = !scatter || owner == p.rank;
    // A. push the row, as the peers will see it, into this rank's slot of the gather buffer of every peer / of the owner
    const float4 own = __ldcg(reinterpret_cast<const float4*>(p.part + row * kLatent) + tid);
    const float own_lse = __ldcg(p.part + p.rows * kLatent + row);
    const float own_scale = row_scale(own, s_max, tid);
    const uint2 pk = pack_row(own, own_scale);
    for (int s = 0; s < p.world; ++s) {
      if (s == p.rank || (scatter && s != owner)) continue;
      char* g = cp_gather(p.block[s], parity, p.world, p.rank, p.max_rows) + row * kCpRowBytes;
      st_tagged(g + tid * 16, pk.x, pk.y, step);
      if (tid == 0) st_tagged(g + kCpThreads * 16, __float_as_uint(own_lse), __float_as_uint(own_scale), step);
    }
    CP_STAMP(2);
    bool ok = true;
    if (merges) {
      // B. the LSEs and row scales of all ranks -> merge weights (warp 0, lane s for rank s)
      if (tid < 32) {
        float l = -INFINITY, sc = 1.f;
        if (tid < p.world) {
          if (tid == p.rank) {
            l = own_lse;
            sc = own_scale;
          } else {
            uint32_t lo = 0, hi = 0;
            ok = wait_tagged(cp_gather(my, parity, p.world, tid, p.max_rows) + row * kCpRowBytes + kCpThreads * 16, step, polls, lo, hi);
            if (ok) {
              l = __uint_as_float(lo);
              sc = __uint_as_float(hi);
            } else {
              report_timeout(p, 300 + tid, step);
            }
          }
        }
        float m = l;
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float e = (l == -INFINITY) ? 0.f : exp2f(l - m);
        float den = e;
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        if (tid < p.world) s_w[tid] = den > 0.f ? e / den * sc : 0.f;  // the weight, times the scale of the fp16 row
        if (tid == 0) s_lse = den > 0.f ? log2f(den) + m : -INFINITY;
      }
      ok = __syncthreads_and(ok);
      CP_STAMP(3);
      // C. merge, ranks in order
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ok) {
        for (int s = 0; s < p.world; ++s) {
          uint32_t lo = pk.x, hi = pk.y;
          if (s != p.rank)  // also for a rank of weight 0: its words must have arrived before its buffer is written again
            ok = wait_tagged(cp_gather(my, parity, p.world, s, p.max_rows) + row * kCpRowBytes + tid * 16, step, polls, lo, hi) && ok;
          const float w = s_w[s];
          if (w != 0.f) {
            const float4 v = unpack_row(lo, hi);
            acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
          }
        }
        if (!ok) report_timeout(p, 310, step);
      }
      if (ok) {
        const uint4 w = pack_out(acc, p.out_dtype);
        if (scatter) {  // D. the final row goes to every peer
          const float lse = s_lse;
          for (int s = 0; s < p.world; ++s) {
            if (s == p.rank) continue;
            char* r = cp_result(p.block[s], parity, p.world, p.max_rows) + row * kCpResultRowBytes;
            st_tagged(r + tid * 16, w.x, w.y, step);
            if (p.out_dtype == MLA_FP4_OUT_F32) st_tagged(r + (kCpThreads + tid) * 16, w.z, w.w, step);
            if (tid == 0) st_tagged(r + 2 * kCpThreads * 16, __float_as_uint(lse), 0u, step);
          }
        }
        store_packed(p.out, p.out_dtype, size_t(row) * kLatent + 4 * tid, w);
        if (tid == 0 && p.lse) p.lse[row] = s_lse;
      }
    } else {
      // E. a row of another rank: its final form arrives in the result area
      const char* r = cp_result(my, parity, p.world, p.max_rows) + row * kCpResultRowBytes;
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      ok = wait_tagged(r + tid * 16, step, polls, w.x, w.y);
      if (ok && p.out_dtype == MLA_FP4_OUT_F32) ok = wait_tagged(r + (kCpThreads + tid) * 16, step, polls, w.z, w.w);
      if (ok) store_packed(p.out, p.out_dtype, size_t(row) * kLatent + 4 * tid, w);
      if (ok && tid == 0) {  // the LSE word is consumed in any case: the buffer must be clear of this step before it is reused
        uint32_t lo = 0, hi = 0;
        ok = wait_tagged(r + 2 * kCpThreads * 16, step, polls, lo, hi);
        if (ok && p.lse) p.lse[row] = __uint_as_float(lo);
      }
      if (!ok) report_timeout(p, 320, step);
    }
    CP_STAMP(4);
  }
  // done (or given up): this CTA's step word advances
  __syncthreads();
  if (tid == 0) *cp_step_word(my, blockIdx.x) = int(step);
#ifdef MLA_FP4_CP_TRACE
  CP_STAMP(5);
  if (tid == 0 && (blockIdx.x <= 1 || blockIdx.x == gridDim.x - 1) && (step & 15) <= 1)
    printf("cptrace rank %d cta %d step %u t0 %llu wait %llu push %llu lse %llu merge %llu fin %llu\n", p.rank, blockIdx.x, step,
           ts[0] % 100000000ull, ts[1] - ts[0], ts[2] - ts[1], ts[3] - ts[2], ts[4] - ts[3], ts[5] - ts[4]);
#endif
}

}  // namespace

cudaError_t launch_cp_exchange_merge(const CpExchangeParams& p, int num_ctas, cudaStream_t stream) {
  if (p.rows == 0) return cudaSuccess;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(num_ctas));
  cfg.blockDim = dim3(kCpThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, cp_exchange_merge_kernel, p);
}

}  // namespace mla

// Split-KV combine: merges the partial slots of every request that the decode kernel split
// across CTAs, and zero-fills requests with seq_len == 0.
//
// grid = (512 / 16 dim chunks, groups * batch), block = 256.  A CTA owns 16 output dims of the
// 64 heads of one (request, head group).  It re-derives which CTAs touched the request from the
// same partition arithmetic the decode kernel used, reads their slots ([head group][dim][8 heads] fp16 + 64
// base-2 LSEs) and accumulates  sum_i exp2(lse_i - max) / den * O_i ; its 8 warps split the slots.
#include "common.cuh"
#include "launch.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace mla {

namespace {
constexpr int kCombDims = 16;
constexpr int kCombThreads = 256;
}

__global__ void __launch_bounds__(kCombThreads) combine_kernel(CombineParams p) {
  __shared__ float lse_s[kMaxCombineSlots][kGroupHeads];  // LSE of every slot of the request, then its weight
  __shared__ float tile[kGroupHeads][kCombDims + 1];
  __shared__ int slot_list[kMaxCombineSlots];
  __shared__ int n_slots;
  __shared__ flat_t s_T;
  __shared__ flat_t s_start;
  __shared__ int s_whole;

  const int v = blockIdx.y;
  const int dchunk = blockIdx.x;
  const int g = v / p.batch, b = v % p.batch;
  const int tid = threadIdx.x;
  if (tid < 32) {  // seq_lens is an input of the step, not a product of the decode kernel
    int mxt;
    const int64_t T64 = warp_total_tiles(p.seq_lens, p.batch, p.seq_cap, &mxt);
    const flat_t T = partition_fits(T64 * p.groups, p.num_ctas) ? flat_t(T64) : -1;  // -1: the decode kernel refused the step
    flat_t run = 0;
    for (int i = tid; i < b; i += 32) run += vtiles_of(capped_len(p.seq_lens, i, p.seq_cap));
    for (int o = 16; o > 0; o >>= 1) run += __shfl_xor_sync(0xffffffffu, run, o);
    if (tid == 0) { s_T = T; s_start = run; s_whole = whole_requests(mxt, int64_t(p.batch) * p.groups, p.num_ctas) ? 1 : 0; }
  }
  __syncthreads();
  const flat_t T = s_T;
  if (T < 0) return;
  const flat_t Tt = T * p.groups;
  const int tiles = vtiles_of(capped_len(p.seq_lens, b, p.seq_cap));  // of the flat space: phantom tiles included
  int qpos, head0;
  group_coords(g, p.num_heads, qpos, head0);
  const int heads_here = min(kGroupHeads, p.num_heads - head0);
  const size_t row0 = (size_t(b) * p.q_len + qpos) * p.num_heads + head0;
  const int h_out = tid >> 2;             // output phase: head
  const int d_out = (tid & 3) * 4;        // output phase: 4 consecutive dims of the chunk
  const size_t out_idx = (row0 + h_out) * kLatent + size_t(dchunk) * kCombDims + d_out;

  if (tiles == 0) {  // empty request: zeros and lse = -inf (the sink's logit when there is a sink)
    if (h_out < heads_here) {
      if (p.out_dtype == MLA_FP4_OUT_BF16) {
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + out_idx) = make_uint2(0u, 0u);
      } else if (p.out_dtype == MLA_FP4_OUT_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + out_idx) = make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(p.out) + out_idx) = 0u;
      }
    }
    if (dchunk == 0 && p.lse && tid < heads_here) p.lse[row0 + tid] = p.sink ? __ldg(p.sink + head0 + tid) * kLog2e : -INFINITY;
    return;
  }
  const flat_t start = flat_t(g) * T + s_start;
  const Span sp = span_of(Tt, p.num_ctas, start + kPhantom, tiles - kPhantom);  // CTAs that hold its real tiles
  if (!sp.split || s_whole) return;  // the decode kernel wrote the final output itself

  // slots of this request, computed once (the partition arithmetic is 64-bit division heavy)
  if (tid < 32) {
    int n = 0;
    for (int base = sp.cta_first; base <= sp.cta_last; base += 32) {
      const int i = base + tid;
      const bool live = i <= sp.cta_last && cta_writes(Tt, p.num_ctas, i, start, tiles);
      const unsigned m = __ballot_sync(0xffffffffu, live);
      if (live) {
        const int pos = n + __popc(m & ((1u << tid) - 1u));
        if (pos < kMaxCombineSlots) slot_list[pos] = slot_in_span(Tt, p.num_ctas, i, start);
      }
      n += __popc(m);
    }
    if (tid == 0) n_slots = min(n, kMaxCombineSlots);
  }
  for (int i = tid; i < kGroupHeads * (kCombDims + 1); i += kCombThreads) (&tile[0][0])[i] = 0.f;
#if __CUDA_ARCH__ >= 900
  if (p.pdl) cudaGridDependencySynchronize();  // from here on the decode kernel's slots are read
#endif
  __syncthreads();
  const int ns = n_slots;
  const void* ws = p.workspace;
  // all LSEs of the request in one round of independent loads
  for (int idx = tid; idx < ns * kGroupHeads; idx += kCombThreads) {
    const int i = idx >> 6, h = idx & 63;
    lse_s[i][h] = slot_lse(ws, slot_list[i])[h];
  }
  __syncthreads();
  if (tid < kGroupHeads) {
    float m = -INFINITY;
    for (int i = 0; i < ns; ++i) m = fmaxf(m, lse_s[i][tid]);
    float dsum = 0.f;
    for (int i = 0; i < ns; ++i) {
      const float l = lse_s[i][tid];
      dsum += (l == -INFINITY) ? 0.f : exp2f(l - m);
    }
    const float inv = dsum > 0.f ? 1.f / dsum : 0.f;
    for (int i = 0; i < ns; ++i) {  // the LSEs become the weights (times the slot's fp16 scale)
      const float l = lse_s[i][tid];
      lse_s[i][tid] = (l == -INFINITY) ? 0.f : exp2f(l - m) * inv * slot_scale(ws, slot_list[i])[0];
    }
    if (dchunk == 0 && p.lse && tid < heads_here) p.lse[row0 + tid] = (dsum > 0.f) ? (log2f(dsum) + m) : -INFINITY;
  }
  __syncthreads();

  // accumulate: the 8 warps split the slots; a lane owns 8 heads (h8) x 4 dims (dq, dq+4, dq+8, dq+12),
  // i.e. 4 independent 16-byte loads (8 fp16 each) per slot
  const int warp = tid >> 5, lane = tid & 31;
  const int h8 = lane & 7, dq = lane >> 3;
  float acc[kCombDims / 4][8];
#pragma unroll
  for (int q = 0; q < kCombDims / 4; ++q)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[q][e] = 0.f;
#pragma unroll 4
  for (int i = warp; i < ns; i += kCombThreads / 32) {
    const uint16_t* so = slot_o(ws, slot_list[i]);
    const float4 w0 = *reinterpret_cast<const float4*>(&lse_s[i][8 * h8]);
    const float4 w1 = *reinterpret_cast<const float4*>(&lse_s[i][8 * h8 + 4]);
    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    const uint16_t* row = so + slot_o_index(dchunk * kCombDims + dq, 8 * h8);  // 8 heads of one dim: 16 contiguous bytes
#pragma unroll
    for (int q = 0; q < kCombDims / 4; ++q) {
      const uint4 a = *reinterpret_cast<const uint4*>(row + size_t(4 * q) * 8);
      const uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[e]));
        acc[q][2 * e] += w[2 * e] * f.x;
        acc[q][2 * e + 1] += w[2 * e + 1] * f.y;
      }
    }
  }
  // fixed-order reduction over the warps (bit-reproducible from run to run)
  for (int wsel = 0; wsel < kCombThreads / 32; ++wsel) {
    if (warp == wsel) {
#pragma unroll
      for (int q = 0; q < kCombDims / 4; ++q)
#pragma unroll
        for (int e = 0; e < 8; ++e) tile[8 * h8 + e][4 * q + dq] += acc[q][e];
    }
    __syncthreads();
  }
  if (h_out < heads_here) {
    const float* t = &tile[h_out][d_out];
    if (p.out_dtype == MLA_FP4_OUT_BF16) {
      __nv_bfloat162 v0 = __floats2bfloat162_rn(t[0], t[1]), v1 = __floats2bfloat162_rn(t[2], t[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&v0); pk.y = *reinterpret_cast<uint32_t*>(&v1);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + out_idx) = pk;
    } else if (p.out_dtype == MLA_FP4_OUT_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + out_idx) = make_float4(t[0], t[1], t[2], t[3]);
    } else {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(t[0], t[1]), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(t[2], t[3]), __NV_SATFINITE, __NV_E4M3);
      *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(p.out) + out_idx) = lo | (hi << 16);
    }
  }
}

cudaError_t launch_combine(const CombineParams& p, cudaStream_t stream) {
  if (p.batch * p.groups == 0) return cudaSuccess;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kLatent / kCombDims, p.batch * p.groups);
  cfg.blockDim = dim3(kCombThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, combine_kernel, p);
}

}  // namespace mla

// Split-KV combine: merges the partial slots of every request that the decode kernel split
// across CTAs, and zero-fills requests with seq_len == 0.
//
// grid = (512 / 32 dim chunks, groups * batch), block = 256.  A CTA owns 32 output dims of the
// 64 heads of one (request, head group).  It re-derives which CTAs touched the request from the
// same partition arithmetic the decode kernel used, reads their slots ([dim][head] f32 + 64
// base-2 LSEs) and accumulates  sum_i exp2(lse_i - max) / den * O_i .
#include "common.cuh"
#include "launch.h"

#include <cuda_bf16.h>

namespace mla {

namespace {
constexpr int kCombDims = 32;
constexpr int kCombThreads = 256;
}

__global__ void __launch_bounds__(kCombThreads) combine_kernel(CombineParams p) {
  __shared__ float lse_max[kGroupHeads];
  __shared__ float inv_den[kGroupHeads];
  __shared__ float tile[kGroupHeads][kCombDims + 1];
  __shared__ int64_t s_T;
  __shared__ int64_t s_start;

  const int v = blockIdx.y;
  const int dchunk = blockIdx.x;
  const int g = v / p.batch, b = v % p.batch;
  const int tid = threadIdx.x;
  if (tid < 32) {  // seq_lens is an input of the step, not a product of the decode kernel
    int64_t T = warp_total_tiles(p.seq_lens, p.batch);
    int64_t run = 0;
    for (int i = tid; i < b; i += 32) run += tiles_of(p.seq_lens[i]);
    for (int o = 16; o > 0; o >>= 1) run += __shfl_xor_sync(0xffffffffu, run, o);
    if (tid == 0) { s_T = T; s_start = run; }
  }
  __syncthreads();
  const int64_t T = s_T;
  const int64_t Tt = T * p.groups;
  const int tiles = tiles_of(p.seq_lens[b]);
  int qpos, head0;
  group_coords(g, p.num_heads, qpos, head0);
  const int heads_here = min(kGroupHeads, p.num_heads - head0);
  const size_t row0 = (size_t(b) * p.q_len + qpos) * p.num_heads + head0;
  const int h_out = tid >> 2;             // output phase: head
  const int d_out = (tid & 3) * 8;        // output phase: 8 consecutive dims of the chunk
  const size_t out_idx = (row0 + h_out) * kLatent + size_t(dchunk) * kCombDims + d_out;

  if (tiles == 0) {  // empty request: zeros and lse = -inf
    if (h_out < heads_here) {
      if (p.out_dtype == MLA_FP4_OUT_BF16) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + out_idx) = make_uint4(0u, 0u, 0u, 0u);
      } else {
        float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + out_idx);
        o[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        o[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    if (dchunk == 0 && p.lse && tid < heads_here) p.lse[row0 + tid] = -INFINITY;
    return;
  }
  const int64_t start = int64_t(g) * T + s_start;
  const Span sp = span_of(Tt, p.num_ctas, start, tiles);
  if (!sp.split) return;  // the decode kernel wrote the final output itself

#if __CUDA_ARCH__ >= 900
  if (p.pdl) cudaGridDependencySynchronize();  // from here on the decode kernel's slots are read
#endif
  const float* ws = reinterpret_cast<const float*>(p.workspace);
  if (tid < kGroupHeads) {
    float m = -INFINITY;
    for (int i = sp.cta_first; i <= sp.cta_last; ++i) {
      if (cta_is_empty(Tt, p.num_ctas, i)) continue;
      m = fmaxf(m, ws[size_t(slot_in_span(Tt, p.num_ctas, i, start)) * kSlotFloats + kSlotOFloats + tid]);
    }
    float dsum = 0.f;
    for (int i = sp.cta_first; i <= sp.cta_last; ++i) {
      if (cta_is_empty(Tt, p.num_ctas, i)) continue;
      float l = ws[size_t(slot_in_span(Tt, p.num_ctas, i, start)) * kSlotFloats + kSlotOFloats + tid];
      dsum += (l == -INFINITY) ? 0.f : exp2f(l - m);
    }
    lse_max[tid] = m;
    inv_den[tid] = dsum > 0.f ? 1.f / dsum : 0.f;
    if (dchunk == 0 && p.lse && tid < heads_here) p.lse[row0 + tid] = (dsum > 0.f) ? (log2f(dsum) + m) : -INFINITY;
  }
  __syncthreads();

  // accumulate: thread = 4 heads (h4) x 2 dims (dsub, dsub + 16) of the chunk
  const int h4 = tid & 15, dsub = tid >> 4;
  const float4 mx = *reinterpret_cast<const float4*>(&lse_max[4 * h4]);
  const float4 iv = *reinterpret_cast<const float4*>(&inv_den[4 * h4]);
  float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
  for (int i = sp.cta_first; i <= sp.cta_last; ++i) {
    if (cta_is_empty(Tt, p.num_ctas, i)) continue;
    const float* so = ws + size_t(slot_in_span(Tt, p.num_ctas, i, start)) * kSlotFloats;
    const float4 l = *reinterpret_cast<const float4*>(so + kSlotOFloats + 4 * h4);
    float4 w;
    w.x = (l.x == -INFINITY) ? 0.f : exp2f(l.x - mx.x) * iv.x;
    w.y = (l.y == -INFINITY) ? 0.f : exp2f(l.y - mx.y) * iv.y;
    w.z = (l.z == -INFINITY) ? 0.f : exp2f(l.z - mx.z) * iv.z;
    w.w = (l.w == -INFINITY) ? 0.f : exp2f(l.w - mx.w) * iv.w;
    const float4 a = *reinterpret_cast<const float4*>(so + size_t(dchunk * kCombDims + dsub) * kGroupHeads + 4 * h4);
    const float4 c = *reinterpret_cast<const float4*>(so + size_t(dchunk * kCombDims + dsub + 16) * kGroupHeads + 4 * h4);
    acc0.x += w.x * a.x; acc0.y += w.y * a.y; acc0.z += w.z * a.z; acc0.w += w.w * a.w;
    acc1.x += w.x * c.x; acc1.y += w.y * c.y; acc1.z += w.z * c.z; acc1.w += w.w * c.w;
  }
  tile[4 * h4 + 0][dsub] = acc0.x; tile[4 * h4 + 1][dsub] = acc0.y;
  tile[4 * h4 + 2][dsub] = acc0.z; tile[4 * h4 + 3][dsub] = acc0.w;
  tile[4 * h4 + 0][dsub + 16] = acc1.x; tile[4 * h4 + 1][dsub + 16] = acc1.y;
  tile[4 * h4 + 2][dsub + 16] = acc1.z; tile[4 * h4 + 3][dsub + 16] = acc1.w;
  __syncthreads();
  if (h_out < heads_here) {
    const float* t = &tile[h_out][d_out];
    if (p.out_dtype == MLA_FP4_OUT_BF16) {
      __nv_bfloat162 v0 = __floats2bfloat162_rn(t[0], t[1]), v1 = __floats2bfloat162_rn(t[2], t[3]);
      __nv_bfloat162 v2 = __floats2bfloat162_rn(t[4], t[5]), v3 = __floats2bfloat162_rn(t[6], t[7]);
      uint4 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&v0); pk.y = *reinterpret_cast<uint32_t*>(&v1);
      pk.z = *reinterpret_cast<uint32_t*>(&v2); pk.w = *reinterpret_cast<uint32_t*>(&v3);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + out_idx) = pk;
    } else {
      float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + out_idx);
      o[0] = make_float4(t[0], t[1], t[2], t[3]);
      o[1] = make_float4(t[4], t[5], t[6], t[7]);
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

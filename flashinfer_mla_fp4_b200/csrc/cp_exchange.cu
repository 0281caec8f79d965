// Decode context parallel: exchange of the per-rank partials over NVLink and their merge, in ONE kernel.
//
// Every rank has decoded its shard of the KV cache into a packed partial  [rows][512] f32 | [rows] f32 (base-2 LSE).
// The kernel on rank r, one CTA per row (round robin when there are more rows than CTAs),
//   A. pushes that partial into slot r of every peer's gather buffer with ordinary stores to peer memory
//      (posted writes over NVLink; nothing is read from a peer, no multicast of any kind): a row travels as 512 fp16
//      values divided by a power-of-two row scale (the row's largest magnitude mapped just below 32768, so the 11-bit
//      values neither overflow nor lose the small ones) followed by its LSE and that scale: half the bytes of f32,
//   B. once all its CTAs have pushed (a counter, nobody waits on it), stamps flag[r] in every peer's exchange
//      block with the step number (st.release.sys after a system-wide fence),
//   C. waits - bounded, like every wait of this library - until the flags of all peers in its OWN block carry the
//      step number: from then on all partials of the step lie in its own memory,
//   D. merges:  out[row] = sum_s w_s * partial_s[row],  w_s = 2^(lse_s - max) / sum  (ranks with an empty shard
//      have lse = -inf and weight 0), the arithmetic of the split-KV reduction with ranks in place of splits; the
//      rank's own partial is taken in f32 from where the decode kernel wrote it.
// The CTAs of one grid never wait for one another, only for flags written by other GPUs, so an ordinary launch
// is enough (all CTAs must be resident at once: a CTA that waits holds its place).  The step number lives in device
// memory (the last CTA to finish advances it), so a CUDA graph that holds the launch can be replayed.  Buffers
// alternate between two parities: a peer can be at most one step ahead (its next step needs this rank's flag of the
// current one), so it never overwrites what is being merged.  The launch may be a programmatic dependent launch: the
// kernel then starts while the decode kernel before it drains and waits for that kernel's completion before it reads.
//
// Exchange block of a rank (one allocation, mapped by every peer through CUDA IPC):
//   int32 flags[8] | int32 pushed | int32 finished | int32 step | pad to 256 B | gather[2][world] of
//   { fp16 [max_rows][512] | f32 [max_rows][2] (LSE, row scale) }
#include "common.cuh"
#include "launch.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace mla {

namespace {

constexpr int kCpThreads = 128;  // one thread per four output dims of a row

__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void store_out4(void* out, int out_dtype, size_t idx, float4 v) {
  if (out_dtype == MLA_FP4_OUT_BF16) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&a);
    pk.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + idx) = pk;
  } else if (out_dtype == MLA_FP4_OUT_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(out) + idx) = v;
  } else {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x, v.y), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z, v.w), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(out) + idx) = lo | (hi << 16);
  }
}

__global__ void __launch_bounds__(kCpThreads) cp_exchange_merge_kernel(const CpExchangeParams p) {
  __shared__ int s_ok;
  __shared__ float s_w[MLA_FP4_CP_MAX_RANKS];
  __shared__ float s_max[kCpThreads / 32];
  const int tid = threadIdx.x;
  int32_t* my = reinterpret_cast<int32_t*>(p.block[p.rank]);
  int32_t* pushed = my + kCpPushedWord;
  int32_t* finished = my + kCpFinishedWord;
  if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");  // the decode kernel before this one has completed
  // the step of this launch: one more than the last completed one (no CTA advances it before all have read it)
  const int step = ld_acquire_sys(my + kCpStepWord) + 1;
  const int parity = step & 1;

  // A. push this rank's partial, row by row, into its slot of every peer's gather buffer
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(p.part + row * kLatent) + tid);
    float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();
    if ((tid & 31) == 0) s_max[tid >> 5] = m;
    __syncthreads();
    m = fmaxf(fmaxf(s_max[0], s_max[1]), fmaxf(s_max[2], s_max[3]));
    const float scale = slot_scale_for(m);  // power of two: the division and the multiplication back are exact
    const float inv = 1.f / scale;
    __half2 h0 = __floats2half2_rn(v.x * inv, v.y * inv), h1 = __floats2half2_rn(v.z * inv, v.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&h0);
    pk.y = *reinterpret_cast<uint32_t*>(&h1);
    const float lse = __ldcg(p.part + p.rows * kLatent + row);
    for (int s = 0; s < p.world; ++s) {
      if (s == p.rank) continue;
      char* g = cp_gather(p.block[s], parity, p.world, p.rank, p.max_rows);
      reinterpret_cast<uint2*>(g + row * (kLatent * 2))[tid] = pk;
      if (tid == 0) *reinterpret_cast<float2*>(g + p.max_rows * (kLatent * 2) + row * 8) = make_float2(lse, scale);
    }
  }
  // B. the last CTA through tells every peer that the whole partial is there
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    if (atomicAdd(pushed, 1) == int(gridDim.x) - 1) {
      *pushed = 0;
      __threadfence_system();
      for (int s = 0; s < p.world; ++s)
        if (s != p.rank) st_release_sys(reinterpret_cast<int32_t*>(p.block[s]) + p.rank, step);
    }
  }
  // C. wait for the partials of all peers (their flags in this rank's own block)
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < p.world && tid != p.rank) {
    bool ok = false;
    int seen = 0;
    for (uint32_t i = 0; i < p.wait_polls; ++i) {
      seen = ld_acquire_sys(my + tid);
      if (seen - step >= 0) { ok = true; break; }  // a peer is never more than one step ahead; its flag only grows
      __nanosleep(200);
    }
    if (!ok) {
      s_ok = 0;
      if (p.status && atomicCAS(p.status, 0, MLA_FP4_ERR_DEVICE_TIMEOUT) == 0) {
        p.status[1] = 300 + tid;  // which peer never arrived
        p.status[2] = blockIdx.x;
        p.status[3] = step;       // the step this rank is in
        p.status[4] = seen;       // the last step that peer has flagged here
      }
    }
  }
  __syncthreads();
  // D. merge the rows of this CTA
  if (s_ok) {
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
      __syncthreads();
      if (tid < 32) {
        float l = -INFINITY, sc = 1.f;
        if (tid < p.world) {
          if (tid == p.rank) {
            l = __ldcg(p.part + p.rows * kLatent + row);
          } else {
            const float2 t = __ldcg(reinterpret_cast<const float2*>(cp_gather(my, parity, p.world, tid, p.max_rows) + p.max_rows * (kLatent * 2) + row * 8));
            l = t.x;
            sc = t.y;
          }
        }
        float m = l;
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float e = (l == -INFINITY) ? 0.f : exp2f(l - m);
        float den = e;
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        if (tid < p.world) s_w[tid] = den > 0.f ? e / den * sc : 0.f;  // the weight, times the row scale of a peer's fp16 row
        if (tid == 0 && p.lse) p.lse[row] = den > 0.f ? log2f(den) + m : -INFINITY;
      }
      __syncthreads();
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < p.world; ++s) {  // in rank order, own partial rounded like the peers' copies of it: all ranks get bit-identical outputs
        const float w = s_w[s];
        if (w == 0.f) continue;
        float4 v;
        if (s == p.rank) {
          v = __ldcg(reinterpret_cast<const float4*>(p.part + row * kLatent) + tid);
          // what the peers see of this row: fp16 of value / row scale.  Recomputed here so that every rank adds the same numbers.
          float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          __syncthreads();
          if ((tid & 31) == 0) s_max[tid >> 5] = m;
          __syncthreads();
          m = fmaxf(fmaxf(s_max[0], s_max[1]), fmaxf(s_max[2], s_max[3]));
          const float scale = slot_scale_for(m), inv = 1.f / scale;
          const float2 a = __half22float2(__floats2half2_rn(v.x * inv, v.y * inv)), b = __half22float2(__floats2half2_rn(v.z * inv, v.w * inv));
          v = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
        } else {
          const uint2 pk = __ldcg(reinterpret_cast<const uint2*>(cp_gather(my, parity, p.world, s, p.max_rows) + row * (kLatent * 2)) + tid);
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&pk.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&pk.y));
          v = make_float4(a.x, a.y, b.x, b.y);
        }
        acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
      }
      store_out4(p.out, p.out_dtype, size_t(row) * kLatent + 4 * tid, acc);
    }
  }
  // the last CTA to finish advances the step
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(finished, 1) == int(gridDim.x) - 1) {
      *finished = 0;
      st_release_sys(my + kCpStepWord, step);
    }
  }
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

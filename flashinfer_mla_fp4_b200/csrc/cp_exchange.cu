// Decode context parallel: exchange of the per-rank partials over NVLink and their merge, in ONE kernel.
//
// Every rank has decoded its shard of the KV cache into a packed partial  [rows][512] f32 | [rows] f32 (base-2 LSE).
// The kernel on rank r
//   A. pushes that partial into slot r of every peer's gather buffer with ordinary stores to peer memory
//      (posted writes over NVLink; nothing is read from a peer, no multicast of any kind),
//   B. once all its CTAs have pushed (a counter, nobody waits on it), stamps flag[r] in every peer's exchange
//      block with the step number (st.release.sys after a system-wide fence),
//   C. waits - bounded, like every wait of this library - until the flags of all peers in its OWN block carry the
//      step number: from then on all partials of the step lie in its own memory,
//   D. merges:  out[row] = sum_s w_s * partial_s[row],  w_s = 2^(lse_s - max) / sum  (ranks with an empty shard
//      have lse = -inf and weight 0), the arithmetic of the split-KV reduction with ranks in place of splits.
// The CTAs of one grid never wait for one another, only for flags written by other GPUs, so an ordinary launch
// is enough.  The step number lives in device memory (the last CTA to finish advances it), so a CUDA graph that
// holds the launch can be replayed.  Buffers alternate between two parities: a peer can be at most one step
// ahead (its next step needs this rank's flag of the current one), so it never overwrites what is being merged.
//
// Exchange block of a rank (one allocation, mapped by every peer through CUDA IPC):
//   int32 flags[8] | int32 pushed | int32 finished | int32 step | pad to 256 B | f32 gather[2][world][n]
#include "common.cuh"
#include "launch.h"

#include <cuda_bf16.h>
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
  const int tid = threadIdx.x;
  int32_t* my = reinterpret_cast<int32_t*>(p.block[p.rank]);
  int32_t* pushed = my + kCpPushedWord;
  int32_t* finished = my + kCpFinishedWord;
  // the step of this launch: one more than the last completed one (no CTA advances it before all have read it)
  const int step = ld_acquire_sys(my + kCpStepWord) + 1;
  const int parity = step & 1;
  const int64_t n4 = p.n / 4;

  // A. push this rank's partial into its slot of every peer's gather buffer
  {
    const float4* src = reinterpret_cast<const float4*>(p.part);
    for (int64_t i = int64_t(blockIdx.x) * kCpThreads + tid; i < n4; i += int64_t(gridDim.x) * kCpThreads) {
      const float4 v = __ldcg(src + i);
      for (int s = 0; s < p.world; ++s) {
        if (s == p.rank) continue;
        float4* dst = reinterpret_cast<float4*>(cp_gather(p.block[s], parity, p.world, p.rank, p.n));
        dst[i] = v;
      }
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
    for (uint32_t i = 0; i < p.wait_polls; ++i) {
      if (ld_acquire_sys(my + tid) == step) { ok = true; break; }
      __nanosleep(200);
    }
    if (!ok) {
      s_ok = 0;
      if (p.status && atomicCAS(p.status, 0, MLA_FP4_ERR_DEVICE_TIMEOUT) == 0) {
        p.status[1] = 300 + tid;  // which peer never arrived
        p.status[2] = blockIdx.x;
        p.status[3] = step;
      }
    }
  }
  __syncthreads();
  // D. merge the rows of this CTA
  if (s_ok) {
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
      __syncthreads();
      if (tid < 32) {
        const float l = tid < p.world ? __ldcg((tid == p.rank ? p.part : cp_gather(my, parity, p.world, tid, p.n)) + p.rows * kLatent + row)
                                      : -INFINITY;
        float m = l;
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float e = (l == -INFINITY) ? 0.f : exp2f(l - m);
        float den = e;
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        if (tid < p.world) s_w[tid] = den > 0.f ? e / den : 0.f;
        if (tid == 0 && p.lse) p.lse[row] = den > 0.f ? log2f(den) + m : -INFINITY;
      }
      __syncthreads();
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < p.world; ++s) {  // in rank order on every rank: all ranks get bit-identical outputs
        const float w = s_w[s];
        if (w == 0.f) continue;
        const float* base = s == p.rank ? p.part : cp_gather(my, parity, p.world, s, p.n);
        const float4 v = __ldcg(reinterpret_cast<const float4*>(base + row * kLatent) + tid);
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
  cp_exchange_merge_kernel<<<dim3(unsigned(num_ctas)), kCpThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace mla

// CUDA-core kernels of the FP4 MLA decode engine:
//   * merge_partials_kernel- context-parallel merge of per-rank partial outputs + LSE
//   * fp32_check_kernel    - plain-FP32 decode over the same work partition; a slow, exact-
//                            arithmetic cross-check of the tcgen05 kernel used by tests
//   * dequant_kernel       - E2M1 -> E4M3 byte dequantisation (the routine fp32_check_kernel uses), for the
//                            bit-exact table test; the tcgen05 kernel hands the packed codes to the MMA unchanged
#include "common.cuh"
#include "dequant.cuh"
#include "launch.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace mla {

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

__device__ __forceinline__ void store_out(void* out, int out_dtype, size_t idx, float v) {
  if (out_dtype == MLA_FP4_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else if (out_dtype == MLA_FP4_OUT_F32) reinterpret_cast<float*>(out)[idx] = v;
  else reinterpret_cast<uint8_t*>(out)[idx] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// ------------------------------------------------------------------------------------------
// Context-parallel merge: out[row] = sum_r w_r * partial[r][row], w_r = exp2(lse_r - lse_max)/den.
// grid = rows, block = 128 (4 dims per thread).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) merge_partials_kernel(const float* __restrict__ po, const float* __restrict__ pl,
                                                             int parts, int64_t rows, int64_t stride_o, int64_t stride_l,
                                                             void* out, int out_dtype, float* lse) {
  const int64_t row = blockIdx.x;
  float m = -INFINITY;
  for (int r = 0; r < parts; ++r) m = fmaxf(m, pl[size_t(r) * stride_l + row]);
  float den = 0.f;
  for (int r = 0; r < parts; ++r) {
    float l = pl[size_t(r) * stride_l + row];
    den += (l == -INFINITY) ? 0.f : exp2f(l - m);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < parts; ++r) {
    float l = pl[size_t(r) * stride_l + row];
    if (l == -INFINITY || den <= 0.f) continue;
    float w = exp2f(l - m) / den;
    float4 v = reinterpret_cast<const float4*>(po + size_t(r) * stride_o + size_t(row) * kLatent)[threadIdx.x];
    acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
  }
  size_t o = size_t(row) * kLatent + 4 * threadIdx.x;
  store_out(out, out_dtype, o + 0, acc.x); store_out(out, out_dtype, o + 1, acc.y);
  store_out(out, out_dtype, o + 2, acc.z); store_out(out, out_dtype, o + 3, acc.w);
  if (lse && threadIdx.x == 0) lse[row] = den > 0.f ? log2f(den) + m : -INFINITY;
}

// ------------------------------------------------------------------------------------------
// Plain-FP32 decode (cross-check).  One CTA per grid slot walks the same segments as the tcgen05
// kernel; 256 threads; 16 tokens per step; Q (64 heads) kept decoded in shared memory.
// ------------------------------------------------------------------------------------------
constexpr int kChkTok = 16;
constexpr int kChkStride = kQDim + 1;  // padded row stride (floats)

__global__ void __launch_bounds__(256) fp32_check_kernel(DecodeParams p) {
  extern __shared__ float smem[];
  float* q_s = smem;                                  // [64][577]
  float* k_s = q_s + kGroupHeads * kChkStride;        // [16][577] latent*scale | rope
  float* p_s = k_s + kChkTok * kChkStride;            // [64][16]
  float* f_s = p_s + kGroupHeads * kChkTok;           // [64] rescale factor
  float* l_s = f_s + kGroupHeads;                     // [64] running sum
  float* m_s = l_s + kGroupHeads;                     // [64] running max (log2 domain)
  __shared__ Walker s_walker;

  const int tid = threadIdx.x;
  if (tid < 32) {
    Walker w = make_walker(p.seq_lens, p.batch, p.seq_cap, p.groups, blockIdx.x, gridDim.x);
    if (tid == 0) s_walker = w;
  }
  __syncthreads();
  Walker w = s_walker;
  const float c = p.softmax_scale * kLog2e;
  const uint8_t* cache = reinterpret_cast<const uint8_t*>(p.kv_cache);
  const uint8_t* q = reinterpret_cast<const uint8_t*>(p.q);

  Segment s;
  while (w.next(s)) {
    int qpos, head0;
    group_coords(s.g, p.num_heads, qpos, head0);
    const int heads_here = min(kGroupHeads, p.num_heads - head0);
    __syncthreads();
    for (int i = tid; i < kGroupHeads * kQDim; i += blockDim.x) {
      int h = i / kQDim, k = i % kQDim;
      float v = 0.f;
      if (h < heads_here)
        v = e4m3_to_float(q[size_t(s.b) * p.q_stride_batch + size_t(qpos) * p.q_stride_qpos +
                            size_t(head0 + h) * p.q_stride_head + k]);
      q_s[h * kChkStride + k] = v;
    }
    if (tid < kGroupHeads) { l_s[tid] = 0.f; m_s[tid] = -INFINITY; }
    float o0[kGroupHeads], o1[kGroupHeads];
#pragma unroll
    for (int h = 0; h < kGroupHeads; ++h) { o0[h] = 0.f; o1[h] = 0.f; }

    const int tok_begin = s.tile_begin * kTile;
    const int tok_end = min(s.seq_len, s.tile_end * kTile);
    for (int t0 = tok_begin; t0 < tok_end; t0 += kChkTok) {
      const int nt = min(kChkTok, tok_end - t0);
      __syncthreads();
      // dequantise nt tokens: latent * scale and rope
      for (int i = tid; i < kChkTok * (kRowBytes / 4); i += blockDim.x) {
        int t = i / (kRowBytes / 4), wv = i % (kRowBytes / 4);
        float* dst = k_s + t * kChkStride;
        if (t < nt) {
          int tok = t0 + t;
          int page = p.block_tables[size_t(s.b) * p.block_table_stride + tok / p.page_size];
          if (page < 0 || page >= p.num_pages) {  // a page id outside the pool: report it, read page 0 instead
            if (p.status) atomicCAS(p.status, 0, MLA_FP4_ERR_DEVICE_TIMEOUT);
            page = 0;
          }
          size_t rowi = size_t(page) * p.page_size + tok % p.page_size;
          uint32_t word = *reinterpret_cast<const uint32_t*>(cache + rowi * kRowBytes + 4 * wv);
          if (wv < kLatent / 8) {
            float sc = p.kv_cache_sf[rowi];
            uint32_t lo, hi;
            e2m1x8_to_e4m3x8(word, lo, hi);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              dst[8 * wv + j] = e4m3_to_float((lo >> (8 * j)) & 0xff) * sc;
              dst[8 * wv + 4 + j] = e4m3_to_float((hi >> (8 * j)) & 0xff) * sc;
            }
          } else {
            int k0 = kLatent + 4 * (wv - kLatent / 8);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[k0 + j] = e4m3_to_float((word >> (8 * j)) & 0xff);
          }
        } else {
          if (wv < kLatent / 8) {
            for (int j = 0; j < 8; ++j) dst[8 * wv + j] = 0.f;
          } else {
            int k0 = kLatent + 4 * (wv - kLatent / 8);
            for (int j = 0; j < 4; ++j) dst[k0 + j] = 0.f;
          }
        }
      }
      __syncthreads();
      // scores: thread -> head tid/4, tokens tid%4 + 4j
      {
        int h = tid >> 2;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const float* qr = q_s + h * kChkStride;
        for (int k = 0; k < kQDim; ++k) {
          float qv = qr[k];
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] += qv * k_s[((tid & 3) + 4 * j) * kChkStride + k];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int t = (tid & 3) + 4 * j;
          const float raw = p.soft_cap > 0.f ? p.soft_cap * tanhf(acc[j] / p.soft_cap) : acc[j];
          p_s[h * kChkTok + t] = (t < nt) ? raw * c : -INFINITY;
        }
      }
      __syncthreads();
      if (tid < kGroupHeads) {
        float m_old = m_s[tid], m = m_old;
        for (int t = 0; t < kChkTok; ++t) m = fmaxf(m, p_s[tid * kChkTok + t]);
        float f = (m_old == -INFINITY) ? 0.f : exp2f(m_old - m);
        float sum = 0.f;
        for (int t = 0; t < kChkTok; ++t) {
          float x = p_s[tid * kChkTok + t];
          float pv = (x == -INFINITY) ? 0.f : exp2f(x - m);
          p_s[tid * kChkTok + t] = pv;
          sum += pv;
        }
        m_s[tid] = m; f_s[tid] = f; l_s[tid] = l_s[tid] * f + sum;
      }
      __syncthreads();
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) {
        float f = f_s[h];
        float a0 = o0[h] * f, a1 = o1[h] * f;
#pragma unroll
        for (int t = 0; t < kChkTok; ++t) {
          float pv = p_s[h * kChkTok + t];
          a0 += pv * k_s[t * kChkStride + tid];
          a1 += pv * k_s[t * kChkStride + tid + 256];
        }
        o0[h] = a0; o1[h] = a1;
      }
    }
    __syncthreads();
    if (p.sink && s.tile_begin == 0) {  // the sink: a virtual token with a zero value row, counted with the first tile of the request
      if (tid < kGroupHeads) {
        float f = 1.f;
        if (tid < heads_here) {
          const float sk = p.sink[head0 + tid] * kLog2e;
          const float m = fmaxf(m_s[tid], sk);
          f = (m_s[tid] == -INFINITY) ? 0.f : exp2f(m_s[tid] - m);
          l_s[tid] = l_s[tid] * f + exp2f(sk - m);
          m_s[tid] = m;
        }
        f_s[tid] = f;
      }
      __syncthreads();
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) { o0[h] *= f_s[h]; o1[h] *= f_s[h]; }
      __syncthreads();
    }
    // epilogue
    const size_t row0 = (size_t(s.b) * p.q_len + qpos) * p.num_heads + head0;
    if (s.slot < 0) {
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) {
        if (h < heads_here) {
          float inv = p.output_scale / l_s[h];
          store_out(p.out, p.out_dtype, (row0 + h) * kLatent + tid, o0[h] * inv);
          store_out(p.out, p.out_dtype, (row0 + h) * kLatent + tid + 256, o1[h] * inv);
        }
      }
      if (p.lse && tid < heads_here) p.lse[row0 + tid] = log2f(l_s[tid]) + m_s[tid];
    } else {
      // slot scale from the largest |O| of the segment (any bound of |O| is a valid slot scale)
      float amax = 0.f;
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) {
        float inv = p.output_scale / l_s[h];
        amax = fmaxf(amax, fmaxf(fabsf(o0[h] * inv), fabsf(o1[h] * inv)));
      }
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      __syncthreads();
      if ((tid & 31) == 0) f_s[tid >> 5] = amax;
      __syncthreads();
      amax = 0.f;
      for (int w8 = 0; w8 < 8; ++w8) amax = fmaxf(amax, f_s[w8]);
      const float sscale = slot_scale_for(amax);
      __half* so = reinterpret_cast<__half*>(slot_o(p.workspace, s.slot));
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) {
        float inv = p.output_scale / l_s[h] / sscale;
        so[slot_o_index(tid, h)] = __float2half_rn(o0[h] * inv);
        so[slot_o_index(tid + 256, h)] = __float2half_rn(o1[h] * inv);
      }
      if (tid == 0) slot_scale(p.workspace, s.slot)[0] = sscale;
      if (tid < kGroupHeads) slot_lse(p.workspace, s.slot)[tid] = log2f(l_s[tid]) + m_s[tid];
    }
  }
}

__global__ void dequant_kernel(const uint32_t* __restrict__ in, uint2* __restrict__ out, int64_t n_words) {
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i < n_words) {
    uint32_t lo, hi;
    e2m1x8_to_e4m3x8(in[i], lo, hi);
    out[i] = make_uint2(lo, hi);
  }
}

// ------------------------------------------------------------------------------------------ launchers

cudaError_t launch_merge_partials(const float* po, const float* pl, int parts, int64_t rows, int64_t stride_o,
                                  int64_t stride_l, void* out, int out_dtype, float* lse, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  merge_partials_kernel<<<dim3((unsigned)rows), 128, 0, stream>>>(po, pl, parts, rows, stride_o, stride_l, out, out_dtype, lse);
  return cudaGetLastError();
}

cudaError_t launch_fp32_check(const DecodeParams& p, int num_ctas, cudaStream_t stream) {
  size_t smem = sizeof(float) * (size_t(kGroupHeads) * kChkStride + size_t(kChkTok) * kChkStride +
                                 size_t(kGroupHeads) * kChkTok + 3 * kGroupHeads);
  cudaError_t e = cudaFuncSetAttribute(fp32_check_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (e != cudaSuccess) return e;
  fp32_check_kernel<<<num_ctas, 256, smem, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_dequant(const void* in, void* out, int64_t n_bytes, cudaStream_t stream) {
  int64_t n_words = n_bytes / 4;
  if (n_words == 0) return cudaSuccess;
  dequant_kernel<<<unsigned((n_words + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(in),
                                                                       reinterpret_cast<uint2*>(out), n_words);
  return cudaGetLastError();
}

}  // namespace mla

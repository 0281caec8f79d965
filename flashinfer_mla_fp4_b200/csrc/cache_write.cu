// KV-cache writer: the producer of the cache format the decode kernel reads.
//
// Per token: amax over the 512 latent values -> scale = amax / 6 (1 for an all-zero token, or a
// caller-provided scale) -> x / scale rounded to the nearest E2M1 magnitude {0,.5,1,1.5,2,3,4,6}
// with a tie going to the smaller one -> 256 packed bytes (low nibble = even element, bit 3 = sign);
// the 64 RoPE values are cast to E4M3 (as torch casts: beyond 464 the byte is NaN); row and scale are scattered to the token's slot
// (page * page_size + offset) of the paged cache.  Same arithmetic, in the same order and with IEEE
// division, as the reference's fixture builder (tests/test_cute_dsl_mla_fp4.py:56-93), so the bytes
// are identical to it; the reference leaves cache writes to the caller (README.md:81-83).
//
// One warp per token, 16 consecutive latent values per lane: 2 x 16-byte loads (16-bit inputs), one
// 8-byte store of packed codes per lane (256 contiguous bytes per warp), 2 RoPE values per lane.
// HBM-bound: 576 input elements read and 324 bytes written per token, nothing is read twice.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "launch.h"

namespace mla {

namespace {

constexpr int kWriterWarps = 8;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// 16 consecutive elements of a row (rows are 16-byte aligned: checked by the launcher): the raw
// 16-byte loads of the next token are issued before the current one is converted.
template <typename T> struct Raw16 {
  static constexpr int kPer = 16 / sizeof(T);  // elements per 16-byte load
  uint4 r[16 / kPer];
  T rope0, rope1;
  int64_t slot;
};
template <typename T> __device__ __forceinline__ void convert16(const Raw16<T>& raw, float (&v)[16]) {
  constexpr int kPer = Raw16<T>::kPer;
#pragma unroll
  for (int q = 0; q < 16 / kPer; ++q) {
    const T* e = reinterpret_cast<const T*>(&raw.r[q]);
#pragma unroll
    for (int i = 0; i < kPer; ++i) v[q * kPer + i] = to_f32<T>(e[i]);
  }
}

// E2M1 code of x / scale: magnitude = number of thresholds strictly below |n| (a tie stays on the
// smaller magnitude), bit 3 = n < 0.
__device__ __noinline__ uint32_t e2m1_code(float x, float scale) {
  const float n = __fdiv_rn(x, scale);
  const float a = fabsf(n);
  uint32_t m = 0;
  m += a > 0.25f;
  m += a > 0.75f;
  m += a > 1.25f;
  m += a > 1.75f;
  m += a > 2.5f;
  m += a > 3.5f;
  m += a > 5.0f;
  return m | (n < 0.f ? 8u : 0u);
}

// float -> E4M3 byte as the reference's writer (a torch cast) does it: round to nearest even; up to
// 464 (the midpoint above the largest finite value) rounds to 448, anything larger and NaN become NaN.
__device__ __forceinline__ uint32_t rope_e4m3(float x) {
  if (!(fabsf(x) <= 464.f)) return 0x7fu | ((__float_as_uint(x) >> 24) & 0x80u);
  return __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// The same codes without the division, for all but a few values in a million.  q = x * (1/scale)
// is within 3 units in the last place of the correctly rounded quotient n, and every rounding
// threshold is a float whose low 21 mantissa bits are zero.  So unless bits(q) lies within 8 of a
// multiple of 2^21, q and n fall between the same two thresholds and are not on one: round-to-
// nearest-even and "a tie goes to the smaller magnitude" agree there, and the hardware conversion
// cvt.rn.satfinite.e2m1x2.f32 of q gives the code (it saturates at 6 and keeps the sign of values
// that round to magnitude zero, as the rule above does).  The fused add of +0 turns a product of
// -0.0 into +0.0: a zero carries no sign bit.  The other values (including q = 0 from an underflow,
// and infinity) are redone with the exact division afterwards.
__device__ __forceinline__ bool needs_exact(float q, float x) {
  return (((__float_as_uint(q) + 8u) & 0x1ffff0u) == 0u) && (__float_as_uint(x) << 1) != 0u;
}
// eight values -> eight packed codes (value 0 in the low nibble)
__device__ __forceinline__ uint32_t e2m1x8(const float (&q)[8]) {
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(out)
      : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
  return out;
}

template <typename T>
__global__ void __launch_bounds__(kWriterWarps * 32)
cache_write_kernel(const T* __restrict__ latent, int64_t latent_stride, const T* __restrict__ rope, int64_t rope_stride,
                   const float* __restrict__ scale_in, const int64_t* __restrict__ slot_mapping, int64_t num_tokens,
                   uint8_t* __restrict__ cache, float* __restrict__ cache_sf, int64_t num_slots) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = int64_t(gridDim.x) * kWriterWarps;
  auto fetch = [&](int64_t t, Raw16<T>& raw) {
    raw.slot = slot_mapping ? __ldg(slot_mapping + t) : t;
    const uint4* p = reinterpret_cast<const uint4*>(latent + t * latent_stride + 16 * lane);
#pragma unroll
    for (int q = 0; q < 16 / Raw16<T>::kPer; ++q) raw.r[q] = __ldg(p + q);
    const T* rp = rope + t * rope_stride + 2 * lane;
    raw.rope0 = rp[0];
    raw.rope1 = rp[1];
  };
  int64_t t = int64_t(blockIdx.x) * kWriterWarps + (threadIdx.x >> 5);
  Raw16<T> cur;
  if (t < num_tokens) fetch(t, cur);
  for (; t < num_tokens; t += warps) {
    Raw16<T> nxt;
    if (t + warps < num_tokens) fetch(t + warps, nxt);  // in flight while this token is quantised
    const Raw16<T> raw = cur;
    cur = nxt;
    const int64_t slot = raw.slot;
    if (slot < 0 || slot >= num_slots) continue;  // padding token (negative) or out of the pool: nothing is written
    float v[16];
    convert16<T>(raw, v);
    float scale;
    if (scale_in) {
      scale = scale_in[t];
    } else {
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      scale = __fdiv_rn(amax, 6.0f);
      if (!(scale > 0.f)) scale = 1.0f;
    }
    const float inv_scale = __frcp_rn(scale);
    uint32_t w[2];
    uint32_t redo = 0u;  // positions whose code must come from the exact division (a few per million)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float q[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        q[i] = fmaf(v[8 * h + i], inv_scale, 0.0f);
        redo |= needs_exact(q[i], v[8 * h + i]) ? (1u << (8 * h + i)) : 0u;
      }
      w[h] = e2m1x8(q);
    }
    while (redo) {
      const int i = __ffs(redo) - 1;
      redo &= redo - 1u;
      const uint32_t code = e2m1_code(to_f32<T>(latent[t * latent_stride + 16 * lane + i]), scale);
      const uint32_t sh = 4u * (uint32_t(i) & 7u);
      uint32_t& word = (i >> 3) ? w[1] : w[0];
      word = (word & ~(0xfu << sh)) | (code << sh);
    }
    uint8_t* row = cache + slot * kRowBytes;
    *reinterpret_cast<uint2*>(row + 8 * lane) = make_uint2(w[0], w[1]);
    // RoPE: two values per lane
    const uint32_t r0 = rope_e4m3(to_f32<T>(raw.rope0)), r1 = rope_e4m3(to_f32<T>(raw.rope1));
    *reinterpret_cast<uint16_t*>(row + kLatent / 2 + 2 * lane) = uint16_t(r0 | (r1 << 8));
    if (lane == 0) cache_sf[slot] = scale;
  }
}

template <typename T>
cudaError_t launch_t(const void* latent, int64_t ls, const void* rope, int64_t rs, const float* scale_in,
                     const int64_t* slots, int64_t n, void* cache, float* sf, int64_t num_slots, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  // a whole number of waves: 8 CTAs of 8 warps per SM, fewer when the token count is small
  const int64_t want = (n + kWriterWarps - 1) / kWriterWarps;
  const int grid = int(want < int64_t(sms) * 8 ? want : int64_t(sms) * 8);
  cache_write_kernel<T><<<grid, kWriterWarps * 32, 0, stream>>>(
      static_cast<const T*>(latent), ls, static_cast<const T*>(rope), rs, scale_in, slots, n,
      static_cast<uint8_t*>(cache), sf, num_slots);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_cache_write(const void* latent, int64_t latent_stride, const void* rope, int64_t rope_stride, int in_dtype,
                               const float* scale_in, const int64_t* slot_mapping, int64_t num_tokens, void* cache,
                               float* cache_sf, int64_t num_slots, cudaStream_t stream) {
  if (num_tokens == 0) return cudaSuccess;
  switch (in_dtype) {
    case MLA_FP4_IN_BF16:
      return launch_t<__nv_bfloat16>(latent, latent_stride, rope, rope_stride, scale_in, slot_mapping, num_tokens, cache, cache_sf, num_slots, stream);
    case MLA_FP4_IN_F16:
      return launch_t<__half>(latent, latent_stride, rope, rope_stride, scale_in, slot_mapping, num_tokens, cache, cache_sf, num_slots, stream);
    default:
      return launch_t<float>(latent, latent_stride, rope, rope_stride, scale_in, slot_mapping, num_tokens, cache, cache_sf, num_slots, stream);
  }
}

}  // namespace mla

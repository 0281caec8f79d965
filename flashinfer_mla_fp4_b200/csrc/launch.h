// Kernel parameter blocks and launcher prototypes shared by the translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mla {

struct DecodeParams {
  const void* q;
  int64_t q_stride_batch, q_stride_qpos, q_stride_head;
  const void* kv_cache;
  const float* kv_cache_sf;
  const int32_t* block_tables;
  int64_t block_table_stride;
  const int32_t* seq_lens;
  void* out;
  float* lse;
  void* workspace;
  int32_t* status;
  int32_t batch, q_len, num_heads, page_size, groups;
  int64_t num_pages;
  float softmax_scale, output_scale;
  int32_t out_dtype;
  int32_t pdl;          // let a dependent kernel start early (griddepcontrol.launch_dependents)
  int32_t pdl_wait;     // set by the launcher: this kernel itself is a dependent launch and waits for the one before it
  int32_t fused_merge;  // the decode kernel merges the split-KV partials itself (cooperative launch)
  int32_t seq_cap;      // most tokens a request may have: block-table width * page_size (INT_MAX when not given)
  uint32_t wait_polls;  // poll budget of every bounded wait
  float soft_cap;       // > 0: raw scores pass through cap * tanh(s / cap)
  const float* sink;    // per-head sink logits or null
};

struct CombineParams {
  const int32_t* seq_lens;
  const void* workspace;
  void* out;
  float* lse;
  int32_t batch, q_len, num_heads, groups, num_ctas, out_dtype, pdl;
  int32_t seq_cap;  // as in DecodeParams
  const float* sink;  // as in DecodeParams: gives the LSE of a request without tokens
};

// Exchange block of the context-parallel exchange (cp_exchange.cu): a step word per CTA, then the gather area: two
// parities x `world` sources x max_rows rows of 129 tagged 16-byte words (8 bytes of data and two 4-byte tags each),
// then the result area of the reduce-scatter form: two parities x max_rows rows of 257 tagged words.
constexpr int kCpMaxCtas = 1024;  // all CTAs of an exchange launch are resident at once
constexpr size_t kCpHeaderBytes = size_t(kCpMaxCtas) * 4;
constexpr size_t kCpRowBytes = 129 * 16;
constexpr size_t kCpResultRowBytes = 257 * 16;
__host__ __device__ inline int32_t* cp_step_word(void* block, int cta) { return static_cast<int32_t*>(block) + cta; }
__host__ __device__ inline size_t cp_partial_bytes(int64_t max_rows) { return size_t(max_rows) * kCpRowBytes; }
__host__ __device__ inline char* cp_gather(void* block, int parity, int world, int src, int64_t max_rows) {
  return static_cast<char*>(block) + kCpHeaderBytes + (size_t(parity) * world + src) * cp_partial_bytes(max_rows);
}
__host__ __device__ inline char* cp_result(void* block, int parity, int world, int64_t max_rows) {
  return static_cast<char*>(block) + kCpHeaderBytes + size_t(2) * world * cp_partial_bytes(max_rows) +
         size_t(parity) * size_t(max_rows) * kCpResultRowBytes;
}
__host__ __device__ inline size_t cp_block_bytes(int world, int64_t max_rows) {
  return kCpHeaderBytes + size_t(2) * world * cp_partial_bytes(max_rows) + size_t(2) * size_t(max_rows) * kCpResultRowBytes;
}
struct CpExchangeParams {
  void* block[8];     // exchange block of every rank as mapped into this process (own block at [rank])
  const float* part;  // this rank's packed partial: [rows][512] f32, then [rows] f32 LSEs
  int64_t rows, max_rows;
  void* out;
  float* lse;
  int32_t* status;
  int32_t world, rank, out_dtype, pdl, algo;
  uint32_t wait_polls;
};
cudaError_t launch_cp_exchange_merge(const CpExchangeParams& p, int num_ctas, cudaStream_t stream);

cudaError_t launch_combine(const CombineParams& p, cudaStream_t stream);
cudaError_t launch_merge_partials(const float* po, const float* pl, int parts, int64_t rows, int64_t stride_o,
                                  int64_t stride_l, void* out, int out_dtype, float* lse, cudaStream_t stream);
cudaError_t launch_fp32_check(const DecodeParams& p, int num_ctas, cudaStream_t stream);
cudaError_t launch_cache_write(const void* latent, int64_t latent_stride, const void* rope, int64_t rope_stride, int in_dtype,
                               const float* scale_in, const int64_t* slot_mapping, int64_t num_tokens, void* cache,
                               float* cache_sf, int64_t num_slots, cudaStream_t stream);
cudaError_t launch_dequant(const void* in, void* out, int64_t n_bytes, cudaStream_t stream);
// tcgen05 decode kernel (decode_sm100.cu). Returns cudaErrorNotSupported-like codes through `err`.
cudaError_t launch_decode_sm100(const DecodeParams& p, int num_ctas, cudaStream_t stream, const char** err);

}  // namespace mla

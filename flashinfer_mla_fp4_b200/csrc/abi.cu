// extern "C" boundary of libmla_fp4_b200.so: argument validation, host planner, launches.
#include <atomic>
#include <climits>
#include <cstdio>
#include <cstring>
#include <string>

#include "common.cuh"
#include "launch.h"

namespace {

thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

int sm_count(int* out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  int n = 0;
  e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
  *out = n;
  return MLA_FP4_OK;
}

bool page_size_ok(int ps) { return ps >= 8 && ps <= 128 && (128 % ps) == 0; }

// Zero the header (generation, finished count) and the tails of all slots (their flags): one asynchronous memset.
int clear_workspace(void* ws, size_t bytes, cudaStream_t stream) {
  if (bytes < mla::kWsFixedBytes) return fail(MLA_FP4_ERR_WORKSPACE_TOO_SMALL, "workspace is smaller than its header and slot tails");
  cudaError_t e = cudaMemsetAsync(ws, 0, mla::kWsFixedBytes, stream);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
  return MLA_FP4_OK;
}

}  // namespace

extern "C" {

int mla_fp4_abi_version(void) { return MLA_FP4_ABI_VERSION; }

const char* mla_fp4_last_error(void) { return g_last_error.c_str(); }

int mla_fp4_workspace_bytes(int32_t batch, int32_t q_len, int32_t num_heads, int32_t num_ctas, size_t* bytes_out) {
  if (!bytes_out) return fail(MLA_FP4_ERR_BAD_ARG, "bytes_out is null");
  if (batch < 0 || q_len <= 0 || num_heads <= 0) return fail(MLA_FP4_ERR_BAD_ARG, "batch/q_len/num_heads out of range");
  if (num_ctas <= 0) {
    int rc = sm_count(&num_ctas);
    if (rc) return rc;
  }
  // the header and the slot tails, then two partial-O slots per CTA (its first and its last segment), whatever the batch is
  *bytes_out = mla::workspace_bytes_for(num_ctas);
  return MLA_FP4_OK;
}

int mla_fp4_plan_partition(const int32_t* seq_lens_host, int32_t batch, int32_t q_len, int32_t num_heads,
                           int32_t num_ctas, int32_t max_segments, int32_t* seg_cta, int32_t* seg_request,
                           int32_t* seg_group, int32_t* seg_tile_begin, int32_t* seg_tile_end, int32_t* seg_slot,
                           int32_t* num_segments) {
  if (!num_segments || (batch > 0 && !seq_lens_host)) return fail(MLA_FP4_ERR_BAD_ARG, "null pointer");
  if (batch < 0 || q_len <= 0 || num_heads <= 0 || num_ctas <= 0)
    return fail(MLA_FP4_ERR_BAD_ARG, "batch/q_len/num_heads/num_ctas out of range");
  const int groups = mla::num_groups(q_len, num_heads);
  int64_t T = 0;
  for (int b = 0; b < batch; ++b) T += mla::vtiles_of(seq_lens_host[b]);
  if (!mla::partition_fits(T * groups, num_ctas)) return fail(MLA_FP4_ERR_UNSUPPORTED, "the work partition is computed in 32 bits: too many tiles x CTAs");
  const mla::flat_t Tt = mla::flat_t(T * groups);
  int max_tiles = 0;
  for (int b = 0; b < batch; ++b) max_tiles = std::max(max_tiles, mla::tiles_of(seq_lens_host[b]));
  const bool whole = mla::whole_requests(max_tiles, int64_t(batch) * groups, num_ctas);
  int count = 0;
  for (int i = 0; i < num_ctas; ++i) {
    mla::Walker w;
    w.seq_lens = seq_lens_host; w.cap = INT_MAX; w.batch = batch; w.groups = groups; w.cta = i; w.first = true;
    w.f = mla::cta_lo(Tt, num_ctas, i);
    w.hi = mla::cta_lo(Tt, num_ctas, i + 1);
    w.b = 0; w.g = groups; w.t = 0;
    if (whole) {  // short requests: (request, head group) pair i, whole, on CTA i
      w.f = 0; w.hi = 0;
      if (i < batch * groups) {
        w.g = i / batch;
        w.b = i - w.g * batch;
        w.hi = mla::vtiles_of(seq_lens_host[w.b]);
      }
    } else if (T > 0 && w.f < w.hi) {
      w.g = int(w.f / T);
      int64_t r = w.f % T, run = 0;  // (host: plain 64-bit arithmetic, same values)
      for (int b = 0; b < batch; ++b) {
        int tb = mla::vtiles_of(seq_lens_host[b]);
        if (r < run + tb) { w.b = b; w.t = int(r - run); break; }
        run += tb;
      }
    }
    mla::Segment s;
    while (w.next(s)) {
      if (count < max_segments) {
        if (seg_cta) seg_cta[count] = i;
        if (seg_request) seg_request[count] = s.b;
        if (seg_group) seg_group[count] = s.g;
        if (seg_tile_begin) seg_tile_begin[count] = s.tile_begin;
        if (seg_tile_end) seg_tile_end[count] = s.tile_end;
        if (seg_slot) seg_slot[count] = s.slot;
      }
      ++count;
    }
  }
  *num_segments = count;
  return MLA_FP4_OK;
}

int mla_fp4_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace) return fail(MLA_FP4_ERR_BAD_ARG, "workspace is null");
  return clear_workspace(workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int mla_fp4_decode(const MlaFp4DecodeArgs* a) {
  if (!a) return fail(MLA_FP4_ERR_BAD_ARG, "args is null");
  if (a->batch < 0 || a->q_len <= 0 || a->num_heads <= 0) return fail(MLA_FP4_ERR_BAD_ARG, "batch/q_len/num_heads out of range");
  if (a->batch == 0) return MLA_FP4_OK;
  if (!a->q || !a->kv_cache || !a->kv_cache_sf || !a->block_tables || !a->seq_lens || !a->out)
    return fail(MLA_FP4_ERR_BAD_ARG, "a required device pointer is null");
  if (!page_size_ok(a->page_size))
    return fail(MLA_FP4_ERR_UNSUPPORTED, "page_size must be one of 8, 16, 32, 64, 128");
  if (a->num_heads > 128) return fail(MLA_FP4_ERR_UNSUPPORTED, "num_heads must be <= 128");
  if (a->out_dtype != MLA_FP4_OUT_BF16 && a->out_dtype != MLA_FP4_OUT_F32 && a->out_dtype != MLA_FP4_OUT_E4M3)
    return fail(MLA_FP4_ERR_UNSUPPORTED, "out_dtype must be MLA_FP4_OUT_BF16, MLA_FP4_OUT_F32 or MLA_FP4_OUT_E4M3");
  if (reinterpret_cast<uintptr_t>(a->kv_cache) % 32) return fail(MLA_FP4_ERR_BAD_ARG, "kv_cache must be 32-byte aligned");
  if (reinterpret_cast<uintptr_t>(a->kv_cache_sf) % 16) return fail(MLA_FP4_ERR_BAD_ARG, "kv_cache_sf must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(a->q) % 16 || a->q_stride_head % 16 || a->q_stride_qpos % 16 || a->q_stride_batch % 16)
    return fail(MLA_FP4_ERR_BAD_ARG, "q must be 16-byte aligned with strides that are multiples of 16");
  if (reinterpret_cast<uintptr_t>(a->out) % 16) return fail(MLA_FP4_ERR_BAD_ARG, "out must be 16-byte aligned");
  if (a->num_pages <= 0) return fail(MLA_FP4_ERR_BAD_ARG, "num_pages must be positive");

  int num_ctas = a->num_ctas;
  if (num_ctas <= 0) {
    int rc = sm_count(&num_ctas);
    if (rc) return rc;
  }
  if (num_ctas > mla::kMaxCombineSlots) return fail(MLA_FP4_ERR_UNSUPPORTED, "num_ctas must be <= 148");
  size_t need = mla::workspace_bytes_for(num_ctas);
  if (!a->workspace || a->workspace_bytes < need) {
    char buf[160];
    snprintf(buf, sizeof buf, "workspace has %zu bytes, but %zu are required", a->workspace ? a->workspace_bytes : size_t(0), need);
    return fail(MLA_FP4_ERR_WORKSPACE_TOO_SMALL, buf);
  }
  if (reinterpret_cast<uintptr_t>(a->workspace) % 16) return fail(MLA_FP4_ERR_BAD_ARG, "workspace must be 16-byte aligned");

  mla::DecodeParams p;
  p.q = a->q; p.q_stride_batch = a->q_stride_batch; p.q_stride_qpos = a->q_stride_qpos; p.q_stride_head = a->q_stride_head;
  p.kv_cache = a->kv_cache; p.kv_cache_sf = a->kv_cache_sf;
  p.block_tables = a->block_tables; p.block_table_stride = a->block_table_stride;
  p.seq_lens = a->seq_lens; p.out = a->out; p.lse = a->lse; p.workspace = a->workspace; p.status = a->status;
  p.batch = a->batch; p.q_len = a->q_len; p.num_heads = a->num_heads; p.page_size = a->page_size;
  p.groups = mla::num_groups(a->q_len, a->num_heads);
  p.num_pages = a->num_pages;
  p.softmax_scale = a->softmax_scale; p.output_scale = a->output_scale;
  p.out_dtype = a->out_dtype; p.pdl = a->enable_pdl ? 1 : 0;
  if (a->max_pages_per_request < 0 || a->wait_polls < 0) return fail(MLA_FP4_ERR_BAD_ARG, "max_pages_per_request/wait_polls must not be negative");
  p.seq_cap = INT_MAX;
  if (a->max_pages_per_request > 0) {
    const int64_t cap = int64_t(a->max_pages_per_request) * a->page_size;
    p.seq_cap = cap < INT_MAX ? int32_t(cap) : INT_MAX;
  }
  p.wait_polls = a->wait_polls > 0 ? uint32_t(a->wait_polls) : (1u << 22);
  if (!(a->logits_soft_cap >= 0.f)) return fail(MLA_FP4_ERR_BAD_ARG, "logits_soft_cap must be >= 0 (0 = off)");
  p.soft_cap = a->logits_soft_cap;
  p.sink = a->sink;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);

  cudaError_t e = cudaSuccess;
  const bool fused = a->kernel == MLA_FP4_KERNEL_TCGEN05;
  p.fused_merge = fused ? 1 : 0;
  const bool do_decode = fused || a->phase_mask == 0 || (a->phase_mask & 1);
  const bool do_combine = !fused && (a->phase_mask == 0 || (a->phase_mask & 2));
  if (!do_decode) {
  } else if (a->kernel == MLA_FP4_KERNEL_FP32_CHECK) {
    p.pdl = 0;
    e = mla::launch_fp32_check(p, num_ctas, stream);
  } else if (a->kernel == MLA_FP4_KERNEL_TCGEN05 || a->kernel == MLA_FP4_KERNEL_TCGEN05_2PASS) {
    const char* why = nullptr;
    e = mla::launch_decode_sm100(p, num_ctas, stream, &why);
    if (e != cudaSuccess && why) return fail(MLA_FP4_ERR_UNSUPPORTED, why);
  } else {
    return fail(MLA_FP4_ERR_BAD_ARG, "unknown kernel id");
  }
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("decode launch: ") + cudaGetErrorString(e));

  if (!do_combine) return MLA_FP4_OK;
  mla::CombineParams c;
  c.seq_lens = a->seq_lens; c.workspace = a->workspace; c.out = a->out; c.lse = a->lse;
  c.batch = a->batch; c.q_len = a->q_len; c.num_heads = a->num_heads; c.groups = p.groups;
  c.num_ctas = num_ctas; c.out_dtype = a->out_dtype; c.pdl = (p.pdl && do_decode) ? 1 : 0;
  c.seq_cap = p.seq_cap;
  c.sink = p.sink;
  e = mla::launch_combine(c, stream);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("combine launch: ") + cudaGetErrorString(e));
  return MLA_FP4_OK;
}

}  // extern "C"

// Scratch of the allocation-free entry point: the counter header (zero-initialised static storage)
// and the split-KV partial slots of the largest accepted grid.  On the host this name is only a handle; the device address is looked up per device.
static __device__ __align__(256) unsigned char g_static_scratch[MLA_FP4_STATIC_SCRATCH_BYTES];
static_assert(MLA_FP4_STATIC_SCRATCH_BYTES == mla::workspace_bytes_for(MLA_FP4_STATIC_MAX_CTAS), "static scratch size");

namespace {
// Set-up of the built-in scratch, once per device, with that device current: the device address of the
// array (the array's name is only a handle on the host).  Two threads racing here both look it up
// and store the same value.
int static_scratch_address(int dev, void** out) {
  static std::atomic<void*> scratch_addr[64];
  void* ptr = scratch_addr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(MLA_FP4_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
    scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return MLA_FP4_OK;
}
}  // namespace

extern "C" {

int mla_fp4_static_reset(void* stream) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(MLA_FP4_ERR_UNSUPPORTED, "device ordinal out of range for the static scratch table");
  void* scratch = nullptr;
  int rc = static_scratch_address(dev, &scratch);
  if (rc) return rc;
  return clear_workspace(scratch, size_t(MLA_FP4_STATIC_SCRATCH_BYTES), reinterpret_cast<cudaStream_t>(stream));
}

int mla_fp4_decode_static(const MlaFp4DecodeArgs* a) {
  if (!a) return fail(MLA_FP4_ERR_BAD_ARG, "args is null");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(MLA_FP4_ERR_UNSUPPORTED, "device ordinal out of range for the static scratch table");
  int num_ctas = a->num_ctas;
  if (num_ctas <= 0) {
    int rc = sm_count(&num_ctas);
    if (rc) return rc;
  }
  if (num_ctas > MLA_FP4_STATIC_MAX_CTAS) {
    char buf[160];
    snprintf(buf, sizeof buf, "mla_fp4_decode_static supports at most %d CTAs (built-in scratch of %d bytes), got %d",
             MLA_FP4_STATIC_MAX_CTAS, int(MLA_FP4_STATIC_SCRATCH_BYTES), num_ctas);
    return fail(MLA_FP4_ERR_UNSUPPORTED, buf);
  }
  void* scratch = nullptr;
  int rc = static_scratch_address(dev, &scratch);
  if (rc) return rc;
  MlaFp4DecodeArgs b = *a;
  b.workspace = scratch;
  b.workspace_bytes = size_t(MLA_FP4_STATIC_SCRATCH_BYTES);
  b.num_ctas = num_ctas;
  return mla_fp4_decode(&b);
}

int mla_fp4_merge_partials(const float* partial_out, const float* partial_lse, int32_t parts, int64_t rows,
                           int64_t part_stride_out, int64_t part_stride_lse, void* out, int32_t out_dtype, float* lse,
                           void* stream) {
  if (parts <= 0 || rows < 0) return fail(MLA_FP4_ERR_BAD_ARG, "parts/rows out of range");
  if (rows == 0) return MLA_FP4_OK;
  if (!partial_out || !partial_lse || !out) return fail(MLA_FP4_ERR_BAD_ARG, "null pointer");
  if (out_dtype != MLA_FP4_OUT_BF16 && out_dtype != MLA_FP4_OUT_F32 && out_dtype != MLA_FP4_OUT_E4M3)
    return fail(MLA_FP4_ERR_UNSUPPORTED, "bad out_dtype");
  if (reinterpret_cast<uintptr_t>(partial_out) % 16) return fail(MLA_FP4_ERR_BAD_ARG, "partial_out must be 16-byte aligned");
  if (part_stride_out == 0) part_stride_out = rows * mla::kLatent;
  if (part_stride_lse == 0) part_stride_lse = rows;
  if (part_stride_out % 4) return fail(MLA_FP4_ERR_BAD_ARG, "part_stride_out must be a multiple of 4 floats");
  cudaError_t e = mla::launch_merge_partials(partial_out, partial_lse, parts, rows, part_stride_out, part_stride_lse, out,
                                             out_dtype, lse,
                                             reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("merge launch: ") + cudaGetErrorString(e));
  return MLA_FP4_OK;
}

int mla_fp4_cp_exchange_bytes(int32_t world, int64_t max_rows, size_t* bytes_out) {
  if (!bytes_out || world < 1 || world > MLA_FP4_CP_MAX_RANKS || max_rows < 0) return fail(MLA_FP4_ERR_BAD_ARG, "world/max_rows out of range");
  *bytes_out = mla::cp_block_bytes(world, max_rows);
  return MLA_FP4_OK;
}

int mla_fp4_cp_alloc(size_t bytes, void** block_out, unsigned char* handle_out) {
  if (!block_out || !handle_out || bytes < mla::kCpHeaderBytes) return fail(MLA_FP4_ERR_BAD_ARG, "null pointer or too few bytes");
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, bytes);
  if (e == cudaSuccess) e = cudaMemset(ptr, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) {
    if (ptr) cudaFree(ptr);
    return fail(MLA_FP4_ERR_CUDA, std::string("exchange block allocation: ") + cudaGetErrorString(e));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == MLA_FP4_CP_HANDLE_BYTES, "IPC handle size");
  memcpy(handle_out, &h, sizeof h);
  *block_out = ptr;
  return MLA_FP4_OK;
}

int mla_fp4_cp_open(const unsigned char* handle, void** block_out) {
  if (!handle || !block_out) return fail(MLA_FP4_ERR_BAD_ARG, "null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  void* ptr = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
  *block_out = ptr;
  return MLA_FP4_OK;
}

int mla_fp4_cp_close(void* peer_block) {
  if (!peer_block) return MLA_FP4_OK;
  cudaError_t e = cudaIpcCloseMemHandle(peer_block);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cudaIpcCloseMemHandle: ") + cudaGetErrorString(e));
  return MLA_FP4_OK;
}

int mla_fp4_cp_free(void* own_block) {
  if (!own_block) return MLA_FP4_OK;
  cudaError_t e = cudaFree(own_block);
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cudaFree: ") + cudaGetErrorString(e));
  return MLA_FP4_OK;
}

int mla_fp4_cp_exchange_merge(void* const* blocks, int32_t world, int32_t rank, const float* partial, int64_t rows, int64_t max_rows,
                              void* out, int32_t out_dtype, float* lse, int32_t* status, int32_t wait_polls, int32_t enable_pdl,
                              int32_t algo, void* stream) {
  if (!blocks || world < 1 || world > MLA_FP4_CP_MAX_RANKS || rank < 0 || rank >= world) return fail(MLA_FP4_ERR_BAD_ARG, "blocks/world/rank out of range");
  if (rows < 0 || wait_polls < 0 || rows > max_rows) return fail(MLA_FP4_ERR_BAD_ARG, "rows/max_rows/wait_polls out of range");
  if (rows == 0) return MLA_FP4_OK;
  if (!partial || !out) return fail(MLA_FP4_ERR_BAD_ARG, "null pointer");
  if (out_dtype != MLA_FP4_OUT_BF16 && out_dtype != MLA_FP4_OUT_F32 && out_dtype != MLA_FP4_OUT_E4M3)
    return fail(MLA_FP4_ERR_UNSUPPORTED, "bad out_dtype");
  if (reinterpret_cast<uintptr_t>(partial) % 16 || reinterpret_cast<uintptr_t>(out) % 16) return fail(MLA_FP4_ERR_BAD_ARG, "partial and out must be 16-byte aligned");
  mla::CpExchangeParams p;
  for (int s = 0; s < 8; ++s) p.block[s] = s < world ? blocks[s] : nullptr;
  for (int s = 0; s < world; ++s)
    if (!p.block[s] || reinterpret_cast<uintptr_t>(p.block[s]) % 16) return fail(MLA_FP4_ERR_BAD_ARG, "an exchange block is null or misaligned");
  p.part = partial; p.rows = rows; p.max_rows = max_rows;
  p.out = out; p.lse = lse; p.status = status; p.world = world; p.rank = rank; p.out_dtype = out_dtype;
  p.pdl = enable_pdl ? 1 : 0;
  if (algo != MLA_FP4_CP_AUTO && algo != MLA_FP4_CP_ALL_GATHER && algo != MLA_FP4_CP_REDUCE_SCATTER)
    return fail(MLA_FP4_ERR_BAD_ARG, "algo must be MLA_FP4_CP_AUTO, _ALL_GATHER or _REDUCE_SCATTER");
  p.algo = algo != MLA_FP4_CP_AUTO ? algo : (world >= 4 ? MLA_FP4_CP_REDUCE_SCATTER : MLA_FP4_CP_ALL_GATHER);
  p.wait_polls = wait_polls > 0 ? uint32_t(wait_polls) : (1u << 22);
  // every CTA of the grid must be resident at once (CTAs that wait for peers hold their place): one per row, capped at what
  // half the SMs of the smallest supported part hold (128 threads and a few bytes of shared memory each)
  const int ctas = int(rows < mla::kCpMaxCtas ? rows : mla::kCpMaxCtas);
  cudaError_t e = mla::launch_cp_exchange_merge(p, ctas, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("exchange launch: ") + cudaGetErrorString(e));
  return MLA_FP4_OK;
}

int mla_fp4_cache_write(const void* latent, int64_t latent_stride, const void* rope, int64_t rope_stride,
                        int32_t in_dtype, const float* token_scale, const int64_t* slot_mapping,
                        int64_t num_tokens, void* kv_cache, float* kv_cache_sf, int64_t num_slots, void* stream) {
  if (num_tokens < 0 || num_slots < 0) return fail(MLA_FP4_ERR_BAD_ARG, "num_tokens/num_slots out of range");
  if (num_tokens == 0) return MLA_FP4_OK;
  if (!latent || !rope || !kv_cache || !kv_cache_sf) return fail(MLA_FP4_ERR_BAD_ARG, "null pointer");
  if (in_dtype != MLA_FP4_IN_BF16 && in_dtype != MLA_FP4_IN_F16 && in_dtype != MLA_FP4_IN_F32)
    return fail(MLA_FP4_ERR_UNSUPPORTED, "in_dtype must be MLA_FP4_IN_BF16, MLA_FP4_IN_F16 or MLA_FP4_IN_F32");
  const int64_t esz = in_dtype == MLA_FP4_IN_F32 ? 4 : 2;
  if (latent_stride < mla::kLatent || rope_stride < mla::kRope) return fail(MLA_FP4_ERR_BAD_ARG, "row strides smaller than the rows");
  if (reinterpret_cast<uintptr_t>(latent) % 16 || (latent_stride * esz) % 16)
    return fail(MLA_FP4_ERR_BAD_ARG, "latent rows must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(rope) % (2 * esz) || rope_stride % 2) return fail(MLA_FP4_ERR_BAD_ARG, "rope rows must be aligned to two elements");
  if (reinterpret_cast<uintptr_t>(kv_cache) % 32) return fail(MLA_FP4_ERR_BAD_ARG, "kv_cache must be 32-byte aligned");
  cudaError_t e = mla::launch_cache_write(latent, latent_stride, rope, rope_stride, in_dtype, token_scale, slot_mapping, num_tokens,
                                          kv_cache, kv_cache_sf, num_slots, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("cache write launch: ") + cudaGetErrorString(e));
  return MLA_FP4_OK;
}

int mla_fp4_dequant_e2m1_to_e4m3(const void* packed, void* out, int64_t n_bytes, void* stream) {
  if (n_bytes < 0 || (n_bytes % 4)) return fail(MLA_FP4_ERR_BAD_ARG, "n_bytes must be a non-negative multiple of 4");
  if (n_bytes == 0) return MLA_FP4_OK;
  if (!packed || !out) return fail(MLA_FP4_ERR_BAD_ARG, "null pointer");
  if (reinterpret_cast<uintptr_t>(packed) % 4 || reinterpret_cast<uintptr_t>(out) % 8)
    return fail(MLA_FP4_ERR_BAD_ARG, "packed must be 4-byte and out 8-byte aligned");
  cudaError_t e = mla::launch_dequant(packed, out, n_bytes, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(MLA_FP4_ERR_CUDA, std::string("dequant launch: ") + cudaGetErrorString(e));
  return MLA_FP4_OK;
}

}  // extern "C"

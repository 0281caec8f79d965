/*
 * C ABI of the B200 FP4 MLA decode engine (libmla_fp4_b200.so).
 *
 * Every entry point is extern "C", takes plain pointers and sizes, returns an
 * int status (0 = OK), never throws, never takes ownership of a buffer, and
 * -- unless its comment says otherwise -- neither allocates device memory nor
 * synchronises the stream.  All device buffers are caller-owned.
 *
 * The reference project has no native code; its kernel is a CuTe-DSL callable
 * produced by JIT compilation.  Each declaration below names the reference
 * interface it stands in for (path inside the reference project : line).
 */
#ifndef MLA_FP4_B200_H_
#define MLA_FP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLA_FP4_ABI_VERSION 5

/* status codes */
#define MLA_FP4_OK 0
#define MLA_FP4_ERR_BAD_ARG 1            /* null pointer, bad shape/stride/alignment          */
#define MLA_FP4_ERR_UNSUPPORTED 2        /* page size / head count / dtype outside the build  */
#define MLA_FP4_ERR_WORKSPACE_TOO_SMALL 3
#define MLA_FP4_ERR_CUDA 4               /* a CUDA runtime/driver call failed                  */
#define MLA_FP4_ERR_DEVICE_TIMEOUT 5     /* a bounded device-side wait expired (status word)   */
#define MLA_FP4_ERR_NOT_BUILT 6          /* library built without the sm_100a kernels          */

/* fixed problem constants (reference wrappers/batch_mla_fp4.py:206-221) */
#define MLA_FP4_LATENT_DIM 512
#define MLA_FP4_ROPE_DIM 64
#define MLA_FP4_ROW_BYTES 320
#define MLA_FP4_TILE_TOKENS 128          /* KV tokens per work tile                            */
#define MLA_FP4_GROUP_HEADS 64           /* query heads handled by one CTA                     */
#ifndef MLA_FP4_PHANTOM_TILES
#define MLA_FP4_PHANTOM_TILES 2          /* tiles the work partition charges for a request's start */
#endif

/* kernel selection for mla_fp4_decode */
#define MLA_FP4_KERNEL_TCGEN05 0         /* the product path: TMA + tcgen05/TMEM, one kernel that
                                            also merges the split-KV partials                  */
#define MLA_FP4_KERNEL_FP32_CHECK 1      /* plain-FP32 CUDA-core kernel, a test cross-check    */
#define MLA_FP4_KERNEL_TCGEN05_2PASS 2   /* the tcgen05 kernel followed by a separate combine
                                            kernel (the reference's two-kernel structure)      */

/* The workspace starts with a header of this many bytes (the generation of the last decode step
   that completed on it and a count of the CTAs that have finished the running one), followed by
   296 slot tails of 272 bytes (64 LSEs, the slot scale, and a flag: the generation that last
   published the slot) and then the partial slots of 65536 bytes.  Header and tails must be zero
   before the first decode step on that workspace (mla_fp4_workspace_init); completed steps keep
   them consistent by themselves.  After a step that reported MLA_FP4_ERR_DEVICE_TIMEOUT call
   mla_fp4_workspace_init again. */
#define MLA_FP4_WORKSPACE_HEADER_BYTES 2048

/* input element types of mla_fp4_cache_write */
#define MLA_FP4_IN_BF16 0
#define MLA_FP4_IN_F16 1
#define MLA_FP4_IN_F32 2

/* output element types (reference: out dtype bf16 default, wrappers/batch_mla_fp4.py:228) */
#define MLA_FP4_OUT_BF16 0
#define MLA_FP4_OUT_F32 1
#define MLA_FP4_OUT_E4M3 2           /* round to nearest even, saturating at +-448 (reference: out in {bf16, e4m3}) */

typedef struct MlaFp4DecodeArgs {
  /* query, E4M3 bytes, logical shape [batch, q_len, num_heads, 576], unit last stride;
     strides in bytes(=elements).  Replaces q_latent/q_rope of the compiled callable
     (wrappers/batch_mla_fp4.py:381-383, :441-443). */
  const void* q;
  int64_t q_stride_batch, q_stride_qpos, q_stride_head;
  /* cache rows, uint8 [num_pages, page_size, 320] contiguous, 32-byte aligned
     (wrappers/batch_mla_fp4.py:384-388). */
  const void* kv_cache;
  /* per-token FP32 scale [num_pages, page_size, 1] contiguous (wrappers/batch_mla_fp4.py:388). */
  const float* kv_cache_sf;
  /* physical page ids, int32 [batch, block_table_stride] row-major (wrappers/batch_mla_fp4.py:446). */
  const int32_t* block_tables;
  int64_t block_table_stride;
  /* int32 [batch] attended tokens per request (wrappers/batch_mla_fp4.py:438-440, :451). */
  const int32_t* seq_lens;
  /* output [batch, q_len, num_heads, 512] contiguous, element type out_dtype (wrappers/...:422-432). */
  void* out;
  /* optional base-2 log-sum-exp [batch, q_len, num_heads] f32; may be NULL.  The reference
     computes it (wrappers/batch_mla_fp4.py:433-437) but does not return it. */
  float* lse;
  /* caller-owned scratch for split-KV partials (the reference slices the wrapper's
     int8 workspace buffer, wrappers/batch_mla_fp4.py:413-420); 16-byte aligned, prepared once
     with mla_fp4_workspace_init. */
  void* workspace;
  size_t workspace_bytes;
  /* int32[8] device status words, zeroed by the caller before first use; word 0 becomes
     non-zero when a bounded device-side wait expired.  May be NULL. */
  int32_t* status;
  int32_t batch, q_len, num_heads, page_size;
  int64_t num_pages;
  float softmax_scale, output_scale;
  int32_t out_dtype;   /* MLA_FP4_OUT_*    */
  int32_t kernel;      /* MLA_FP4_KERNEL_* */
  int32_t num_ctas;    /* CTAs of the persistent decode grid; 0 = one per SM of the current device */
  int32_t enable_pdl;  /* programmatic dependent launch: lets the next kernel on the stream start its
                          prologue while the decode kernel drains (0/1) */
  int32_t phase_mask;  /* two-kernel modes only: 0 = decode + combine; 1 = decode kernel only;
                          2 = combine kernel only (profiling) */
  void* stream;        /* cudaStream_t */
  /* Width of a block-table row in pages (block_tables.shape[1]).  The kernels never read a row
     beyond it: a seq_lens entry larger than max_pages_per_request * page_size is treated as
     that many tokens.  0 = not given (rows are trusted to cover seq_lens). */
  int32_t max_pages_per_request;
  /* Poll budget of every bounded device-side wait (0 = the default, 2^22).  When a wait runs
     out the kernel records MLA_FP4_ERR_DEVICE_TIMEOUT in the status words and returns. */
  int32_t wait_polls;
  /* Attention variants, compiled into the kernels (the reference passes an AttentionVariant object whose hooks are
     traced into its kernel, wrappers/batch_mla_fp4.py:237-253; the two hooks in use there are restated as data):
     logits_soft_cap > 0: every raw score s = q.k becomes cap * tanh(s / cap) before softmax_scale is applied (the
       score_mod hook of a soft-capping variant); 0 = off.
     sink: f32 [num_heads] on the device or NULL: one virtual token per head with logit sink[h] (natural-log units,
       compared with the scaled scores) and a zero value row: it only adds exp(sink[h]) to the softmax denominator
       (the update_statistics hook of the sink variant, applied with the first tile of a request). */
  float logits_soft_cap;
  const float* sink;
} MlaFp4DecodeArgs;

/* ABI version of the loaded library (== MLA_FP4_ABI_VERSION of the header it was built from). */
int mla_fp4_abi_version(void);

/* Message of the last non-zero status returned on the calling thread. */
const char* mla_fp4_last_error(void);

/* Scratch bytes mla_fp4_decode needs for (batch, q_len, num_heads) on a grid of num_ctas CTAs
   (0 = SM count of the current device).  Stands in for
   flashinfer cute_dsl/attention/scheduler/mla_persistent.py:285-291 (mla_get_workspace_size),
   reached from wrappers/batch_mla_fp4.py:390-396.  Host only. */
int mla_fp4_workspace_bytes(int32_t batch, int32_t q_len, int32_t num_heads, int32_t num_ctas,
                            size_t* bytes_out);

/* Host copy of the work partition the decode kernel derives on the device: request b, head
   group g and tile range of every segment of every CTA.  seq_lens is a HOST array.  Arrays
   hold up to max_segments entries; *num_segments receives the count (the required count when
   it exceeds max_segments).  Stands in for the reference's split heuristic + static tile
   scheduler (flashinfer cute_dsl/attention/scheduler/mla_persistent.py:137-282).  Host only. */
int mla_fp4_plan_partition(const int32_t* seq_lens_host, int32_t batch, int32_t q_len,
                           int32_t num_heads, int32_t num_ctas, int32_t max_segments,
                           int32_t* seg_cta, int32_t* seg_request, int32_t* seg_group,
                           int32_t* seg_tile_begin, int32_t* seg_tile_end, int32_t* seg_slot,
                           int32_t* num_segments);

/* Zero the header of a workspace (an asynchronous memset on `stream`).  Call once after
   allocating the workspace, and again after a step that reported MLA_FP4_ERR_DEVICE_TIMEOUT.
   The reference's workspace needs no preparation (wrappers/batch_mla_fp4.py:413-420). */
int mla_fp4_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* One decode step on args->stream: one persistent kernel that computes the attention and merges
   the split-KV partials (its CTAs wait for one another at the end, so it is launched
   cooperatively: the grid must fit the device).  Stands in for the compiled callable invoked at
   wrappers/batch_mla_fp4.py:441-457 (mla_decode_fp4.py:60-305: split_kv_kernel +
   reduction_kernel). */
int mla_fp4_decode(const MlaFp4DecodeArgs* args);

/* Merge `parts` normalised partial outputs with base-2 LSEs (decode context parallel):
   partial_out f32 [parts, rows, 512], partial_lse f32 [parts, rows] ->
   out [rows, 512] (out_dtype) and optional lse [rows].  part_stride_out / part_stride_lse are
   the distances, in floats, between consecutive parts (0 = dense: rows*512 and rows), so that
   partials gathered as one packed buffer per rank can be merged in place.  Same arithmetic as the split-KV
   reduction (flashinfer cute_dsl/attention/mla_decode.py:614-710); the reference has no
   multi-GPU path of its own. */
int mla_fp4_merge_partials(const float* partial_out, const float* partial_lse, int32_t parts,
                           int64_t rows, int64_t part_stride_out, int64_t part_stride_lse, void* out,
                           int32_t out_dtype, float* lse, void* stream);

/* Decode context parallel without a library collective (no counterpart in the reference, which has no
   multi-GPU path).  Every rank owns an "exchange block" of device memory that all peers map through CUDA
   IPC; mla_fp4_cp_exchange_merge is ONE kernel per rank and step that pushes the rank's partial rows into the
   peers' blocks with plain stores over NVLink (every 16-byte word carries the step number as its arrival tag:
   no flags, no fences), waits (bounded) for the peers' rows in its own block and merges.  Nothing is read from
   a peer's memory.  One process per GPU, all GPUs in one NVLink domain, at most
   MLA_FP4_CP_MAX_RANKS ranks; every rank must make the same sequence of calls.
     mla_fp4_cp_exchange_bytes: size of a block for partials of up to max_rows rows (rows = batch*q_len*heads).
     mla_fp4_cp_alloc:  allocates (cudaMalloc) and zeroes this rank's block and returns its IPC handle
                        (MLA_FP4_CP_HANDLE_BYTES bytes) for the caller to send to the peers.  Allocates and
                        synchronises; call it once, at set-up.
     mla_fp4_cp_open / _close: map / unmap a peer's block from its handle.   mla_fp4_cp_free: free the own block.
     mla_fp4_cp_exchange_merge: blocks[world] are the blocks as mapped here (own block at [rank]); partial is this
                        rank's packed partial, f32 [rows][512] followed by f32 [rows] LSEs (base 2), 16-byte
                        aligned, as mla_fp4_decode writes them with out_dtype F32 and lse pointing behind the rows;
                        max_rows is the value the blocks were sized with (the same on every rank); enable_pdl launches
                        the kernel as a programmatic dependent launch (it starts while the kernel before it on the
                        stream drains and waits for that kernel's end before it reads anything);
                        out [rows][512] (out_dtype), optional lse [rows]; status as in MlaFp4DecodeArgs (word 0 set
                        to MLA_FP4_ERR_DEVICE_TIMEOUT when a peer's rows do not arrive within wait_polls polls,
                        0 = default); asynchronous on `stream`, CUDA-graph capturable (the step counters live in
                        the block).  After a reported time-out the ranks' step counters disagree: free the
                        blocks and set up new ones. */
#define MLA_FP4_CP_MAX_RANKS 8
#define MLA_FP4_CP_HANDLE_BYTES 64
/* form of the exchange: every rank receives every peer's rows and merges them all (one NVLink hop, (world-1) partials
   per rank), or every row is merged by one owner rank which sends the final row to the others (two hops, under two
   partials per rank whatever the number of ranks).  AUTO: all-gather below four ranks.  All ranks pass the same value. */
#define MLA_FP4_CP_AUTO 0
#define MLA_FP4_CP_ALL_GATHER 1
#define MLA_FP4_CP_REDUCE_SCATTER 2
int mla_fp4_cp_exchange_bytes(int32_t world, int64_t max_rows, size_t* bytes_out);
int mla_fp4_cp_alloc(size_t bytes, void** block_out, unsigned char* handle_out);
int mla_fp4_cp_open(const unsigned char* handle, void** block_out);
int mla_fp4_cp_close(void* peer_block);
int mla_fp4_cp_free(void* own_block);
int mla_fp4_cp_exchange_merge(void* const* blocks, int32_t world, int32_t rank, const float* partial, int64_t rows,
                              int64_t max_rows, void* out, int32_t out_dtype, float* lse, int32_t* status,
                              int32_t wait_polls, int32_t enable_pdl, int32_t algo, void* stream);

/* Bit-exact E2M1 nibble -> E4M3 byte dequantisation of `n_bytes` packed bytes on the device
   (out holds 2*n_bytes E4M3 bytes, low nibble first).  Pins the table of
   tests/test_cute_dsl_mla_fp4.py:80-84.  (The decode kernel itself hands the packed codes to the
   tensor core unchanged; this is the routine of the FP32 cross-check kernel.) */
int mla_fp4_dequant_e2m1_to_e4m3(const void* packed, void* out, int64_t n_bytes, void* stream);

/* Write `num_tokens` tokens into the paged cache (the producer of the format mla_fp4_decode reads):
   per token amax -> scale = amax / 6 (1 for an all-zero token), x / scale rounded to the nearest E2M1
   magnitude with a tie going to the smaller one, packed low nibble = even element with the sign in
   bit 3, the 64 RoPE values cast to E4M3 (round to nearest even; |x| > 464 becomes NaN, as a torch
   cast does), row and FP32 scale
   stored at slot_mapping[t] = page * page_size + offset of kv_cache [num_slots, 320] / kv_cache_sf
   [num_slots].  latent [num_tokens, 512] and rope [num_tokens, 64] have element type in_dtype
   (MLA_FP4_IN_*), unit inner stride, row strides in elements (latent rows 16-byte aligned).
   token_scale (f32 [num_tokens]) replaces the amax scale when not NULL; slot_mapping NULL means
   slot t; a slot that is negative or >= num_slots is skipped (padding tokens).  Byte-identical to the
   reference's fixture builder (tests/test_cute_dsl_mla_fp4.py:56-93); the reference itself leaves
   cache writes to the caller (README.md:81-83). */
int mla_fp4_cache_write(const void* latent, int64_t latent_stride, const void* rope, int64_t rope_stride,
                        int32_t in_dtype, const float* token_scale, const int64_t* slot_mapping,
                        int64_t num_tokens, void* kv_cache, float* kv_cache_sf, int64_t num_slots,
                        void* stream);

/* Largest decode grid the allocation-free variant below accepts, and the bytes of device memory
   its built-in scratch occupies on every GPU that loads the library (until the process exits). */
#define MLA_FP4_STATIC_MAX_CTAS 148
#define MLA_FP4_STATIC_SCRATCH_BYTES (MLA_FP4_WORKSPACE_HEADER_BYTES + 2 * MLA_FP4_STATIC_MAX_CTAS * 65808)

/* No counterpart in the reference.  Same decode step as mla_fp4_decode, for callers that may not
   allocate device memory and have no workspace buffer to lend: plugins running inside an engine
   whose memory pool owns the whole device, code running under a framework that forbids cudaMalloc
   on its worker threads, or a step that has to run when the caching allocator is exhausted.
   args->workspace and args->workspace_bytes are ignored; the split-KV partials go to a scratch
   array built into the library (MLA_FP4_STATIC_SCRATCH_BYTES of device memory per GPU, reserved
   when the library is loaded on that GPU).  q, cache, block tables, seq_lens, out, lse and the
   status words are still the caller's.  Nothing is allocated or freed, here or in the kernels.
   - Limit: the decode grid (args->num_ctas, or the SM count when 0) must not exceed
     MLA_FP4_STATIC_MAX_CTAS; a larger grid is rejected with MLA_FP4_ERR_UNSUPPORTED.
   - The first call on a device looks the scratch address up once (with that device current) and
     keeps it; make that first call before any stream capture begins.
   - All calls on a device share the one scratch array.  It keeps the previous call's partials, which
     is harmless: a step only reads slots whose flag carries its own generation.  Its header starts
     at zero (static storage) and every step whose kernel returns leaves it consistent, a step that
     reported MLA_FP4_ERR_DEVICE_TIMEOUT included.  Should a kernel ever be torn down half-way (a
     sticky CUDA error in the process), mla_fp4_static_reset puts the header back to zero.
     Two calls whose kernels overlap on the GPU (different streams) would overwrite each other's
     partials: run them in order on one stream, or use mla_fp4_decode with separate workspaces. */
int mla_fp4_decode_static(const MlaFp4DecodeArgs* args);

/* No counterpart in the reference.  Zero the header of the built-in scratch of mla_fp4_decode_static
   on the current device (an asynchronous memset on `stream`; allocates nothing).  The caller cannot
   reach that array with mla_fp4_workspace_init, since its address never leaves the library.  Needed
   only after a decode kernel did not run to its end; harmless at any other time between steps. */
int mla_fp4_static_reset(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MLA_FP4_B200_H_ */

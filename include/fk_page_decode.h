/*
 * fk_page_decode.h -- C ABI of the paged-KV decode attention for B200 (sm_100a).
 *
 * One query token per request attends over that request's key/value pages, grouped-query
 * attention with the rotary embedding applied inside the kernel. It replaces, entry point for
 * entry point, the reference's
 *     csrc/ops/clustered_page_decode/clustered_page_decode.h:16-25   clustered_page_decode_forward
 * whose launcher and two kernels are csrc/kernels/clustered_page_decode/clustered_page_decode.cu
 * (:111-328 one warp per query head, :330-669 one cluster per request / kv head / head tile,
 * :1085-1160 validation and dispatch). Tensor meanings are the reference's:
 *
 *   query        [batch, num_q_heads, head_dim]                      bf16
 *   key_pages    [pages, num_kv_heads, page_size, head_dim]          bf16 | e4m3 | int8
 *   value_pages  same shape and type as key_pages
 *   key_scales   [pages, num_kv_heads, head_dim / 64]                fp32, NULL for bf16 pages
 *   value_scales [pages, num_kv_heads, page_size, head_dim / 64]     fp32, NULL for bf16 pages
 *   run_*        [num_runs] int32: a run is `page_count` physically consecutive pages starting at
 *                `base_page`; its first page is logical page `logical_start` of the request (what
 *                the rotary position of a key is counted from); the run's LAST page holds
 *                `last_page_len` tokens, every other page `page_size`
 *   request_run_offsets [batch + 1] int32: request b owns runs [offsets[b], offsets[b + 1])
 *   seq_lens     [batch] int32: the query of request b sits at position seq_lens[b] - 1
 *   output       [batch, num_q_heads, head_dim]                      bf16
 *
 * A request with seq_lens <= 0 or without runs gets zeros. head_dim is 64 or 128, page_size 16 or
 * 32, num_q_heads a multiple of num_kv_heads. With keys_are_rotated != 0 the keys in the pages
 * already carry their rotary embedding and only the query is rotated; such calls run on the tensor
 * cores (mma.sync with the query and the probabilities as exact 16-bit head + remainder pairs, 8-bit
 * pages converted to f16 rows on the fly), all others on fp32 FMAs. Both forms accumulate in fp32
 * and keep every scale in fp32; results agree with an fp64 evaluation of the same bytes to
 * 2e-3 + 8e-3 |y| (the bound of the parity tests) and are bit-reproducible run to run.
 *
 * All pointers are device pointers. Calls are asynchronous on `stream`. Plain C: no C++ or
 * framework types cross this boundary.
 */
#ifndef FK_PAGE_DECODE_H_
#define FK_PAGE_DECODE_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FK_PAGE_DECODE_API __attribute__((visibility("default")))
#else
#define FK_PAGE_DECODE_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define FK_PAGE_DECODE_OK 0
#define FK_PAGE_DECODE_ERR_INVALID_ARGUMENT (-1) /* std::invalid_argument / ValueError */
#define FK_PAGE_DECODE_ERR_CUDA (-2)             /* a CUDA call failed: std::runtime_error */

/* KvFormat of the reference (clustered_page_decode.h:8-12). */
#define FK_PAGE_DECODE_KV_BF16 0
#define FK_PAGE_DECODE_KV_FP8_E4M3 1
#define FK_PAGE_DECODE_KV_INT8 2

/* The kernel is launched with programmatic stream serialisation: it may be scheduled while the
 * kernel before it in the stream is still draining, and waits for that kernel's completion before
 * it touches global memory. With this flag the caller states that the preceding kernel does not
 * write the request descriptors (the run arrays, request_run_offsets, seq_lens) -- the usual case,
 * they come from the host -- and the kernel reads and sorts them before it waits. Queries, pages,
 * scales and outputs are never touched early. */
#define FK_PAGE_DECODE_FLAG_EARLY_DESCRIPTORS 1

typedef struct fk_page_decode_args {
  const void* query;
  const void* key_pages;
  const void* value_pages;
  const float* key_scales;
  const float* value_scales;
  const int32_t* run_base_pages;
  const int32_t* run_page_counts;
  const int32_t* run_logical_starts;
  const int32_t* run_last_page_lens;
  const int32_t* request_run_offsets;
  const int32_t* seq_lens;
  void* output;
  /* Scratch of at least fk_page_decode_workspace_bytes(...) bytes, zero before the first call
   * (fk_page_decode_workspace_init); every call leaves the part that must be zero, zero again.
   * One workspace serves calls that are ordered on one stream; overlapping calls need their own.
   * May be NULL when `splits` is 1. */
  void* workspace;
  size_t workspace_bytes;
  int32_t batch;
  int32_t num_runs;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_dim;
  int32_t page_size;
  /* Query heads of one kv head that one thread block carries together (1, 2, 4 or 8; 0 = the
   * smallest of those that covers the group, capped at 8). The reference's `group_tile`. An upper
   * bound: with few tasks the launcher may carry 4 where 8 were asked for (more warps per block);
   * results agree to fp32 rounding. */
  int32_t group_tile;
  int32_t kv_format;
  int32_t keys_are_rotated;
  /* How many thread blocks share the pages of one (request, kv head, head tile): 0 = as many as
   * fill the device, 1 = one block and no scratch, n = exactly n (at most 64). The blocks'
   * partial results are merged in block order: for 2 or 4 blocks inside a thread-block cluster
   * through shared memory (no scratch), otherwise through the workspace by the block that
   * finishes last. */
  int32_t splits;
  /* Upper bound of the pages of one request if the caller knows it (it bounds `splits` so that
   * short requests are not cut into empty pieces), 0 = unknown. */
  int32_t max_pages_hint;
  float softmax_scale;
  float rope_theta;
  void* stream;
  /* FK_PAGE_DECODE_FLAG_* bits, 0 = none. */
  int32_t flags;
} fk_page_decode_args;

FK_PAGE_DECODE_API const char* fk_page_decode_last_error(void);

/* Scratch for any call with these head counts on the current device, whatever `splits`. */
FK_PAGE_DECODE_API size_t fk_page_decode_workspace_bytes(int batch, int num_q_heads, int num_kv_heads,
                                                         int head_dim);
FK_PAGE_DECODE_API int fk_page_decode_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Replaces clustered_page_decode_forward (clustered_page_decode.h:16-25). */
FK_PAGE_DECODE_API int fk_page_decode_forward(const fk_page_decode_args* args);

/* Reads and clears the device status word of the current device: 0 = fine, 1 = a bounded wait for
 * a page copy gave up (the outputs of that call are not valid; re-initialise the workspace). */
FK_PAGE_DECODE_API int fk_page_decode_device_status(int* status);

/* One line that says how a call with these arguments would be launched
 * ("blocks=... splits=... warps=... stages=... shared=..."), for benchmarks and tests. */
FK_PAGE_DECODE_API int fk_page_decode_describe_plan(const fk_page_decode_args* args, char* text, size_t capacity);

/* Launch overrides for tuning runs: warps per block (0 = default) and ring depth per warp
 * (0 = default). Process-wide. */
FK_PAGE_DECODE_API int fk_page_decode_set_launch_config(int warps_per_block, int stages);

#ifdef __cplusplus
}
#endif

#endif /* FK_PAGE_DECODE_H_ */

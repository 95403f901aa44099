/*
 * fk_w4a16.h -- C ABI of the sm_100a W4A16 decode-GEMV library (libfk_w4a16.so).
 *
 * This is the boundary a host program binds to: plain pointers and sizes, no C++ or torch types,
 * no exceptions. Every pointer is a DEVICE address unless the comment says otherwise; `stream` is
 * a cudaStream_t passed as void* (NULL = the default stream). All work is enqueued on `stream`
 * and nothing synchronises the host. Functions return FK_W4A16_OK or a negative error code;
 * fk_w4a16_last_error() gives the message for the calling thread.
 *
 * Each entry point names the function of the reference (SamMausberg/fast-kernels) that it
 * replaces, as file:line in that project.
 *
 * Data layout ("ARC packets", csrc/kernels/decode_quant_linear/arc_w4a16.cu:87-122): the weight
 * matrix W[n, k] is cut into tiles of 128 output columns and groups of `group_size` input
 * features. Packet (tile t, group g) starts at byte (t * k/group_size + g) * stride and holds
 *   uint32 words[group_size/8][128]  word (r, c): nibble i (bits 4i..4i+3) = q[128t + c, g*G + 8r + i]
 *   16-bit alpha[128]                scale of column 128t + c in group g
 *   16-bit beta[128]                 offset, beta = -(alpha * zero_point) rounded in the 16-bit type
 * with stride = 64 * group_size + 512 bytes, and W[n, k] = alpha * q + beta.
 */
#ifndef FK_W4A16_H_
#define FK_W4A16_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FK_W4A16_API __attribute__((visibility("default")))
#else
#define FK_W4A16_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define FK_W4A16_OK 0
#define FK_W4A16_ERR_INVALID_ARGUMENT (-1) /* maps to std::invalid_argument / ValueError */
#define FK_W4A16_ERR_CUDA (-2)             /* a CUDA or cuBLAS call failed: std::runtime_error */
#define FK_W4A16_ERR_DEVICE_STATUS (-3)    /* a bounded device-side wait gave up */

/* 16-bit element type of activations, scales, offsets and outputs. */
#define FK_W4A16_DTYPE_F16 0
#define FK_W4A16_DTYPE_BF16 1

/* Message for the last error on the calling thread ("" if none). Host pointer, valid until the
 * thread's next failing call. */
FK_W4A16_API const char* fk_w4a16_last_error(void);

/* Library version string and the CUDA architecture it was compiled for ("100a"). Host pointers. */
FK_W4A16_API const char* fk_w4a16_version(void);
FK_W4A16_API const char* fk_w4a16_cuda_arch(void);

/* Packet stride in bytes for a group size (32, 64 or 128), or a negative error code.
 * Reference: expected_packet_stride_bytes, arc_w4a16.cu:23-26. */
FK_W4A16_API int fk_w4a16_packet_stride_bytes(int group_size);

/* q_u8[n, k/2] (low nibble = even k), alpha/beta[n, k/group_size] -> packets.
 * Reference: pack_arc_w4a16_packets, arc_w4a16.cu:649-669 (kernel :87-122). */
FK_W4A16_API int fk_w4a16_pack_packets(const void* q, const void* alpha, const void* beta, void* packets, int n,
                          int k, int group_size, int packet_stride_bytes, void* stream);

/* sums[batch, k/group_size] (fp32) = per-group sums of the activations.
 * Reference: compute_arc_w4a16_group_sums, arc_w4a16.cu:671-685 (kernel :124-158). */
FK_W4A16_API int fk_w4a16_group_sums(const void* activations, float* sums, int batch, int k, int group_size,
                        int dtype, void* stream);

/* Scratch the fused GEMV needs for a problem, in bytes (a multiple of 256; never 0). The caller
 * allocates it on the device, zero-fills it ONCE (fk_w4a16_workspace_init or cudaMemset) and may
 * then reuse it for any number of calls whose requirement is not larger. Calls that run
 * concurrently on the GPU need separate workspaces. */
FK_W4A16_API size_t fk_w4a16_workspace_bytes(int batch, int n, int k, int group_size);
FK_W4A16_API int fk_w4a16_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* The hot path: out[batch, n] = activations[batch, k] . W^T in ONE launch -- activation group
 * sums, int4 unpack, scale/offset, fp32 accumulation, split-K finish and the 16-bit rounding of
 * the output all happen inside it. batch <= 4 streams on CUDA cores; larger batches are
 * processed 4 rows at a time.
 * Reference: arc_w4a16_forward, arc_w4a16.cu:687-707, together with the group-sum prepass
 * (:671-685) and the split-K pair (:709-751) that its Python caller chains around it
 * (src/fast_kernels/ops/decode_quant_linear.py:383-439). */
FK_W4A16_API int fk_w4a16_gemv(const void* activations, const void* packets, void* output, void* workspace,
                  size_t workspace_bytes, int batch, int n, int k, int group_size,
                  int packet_stride_bytes, int dtype, void* stream);

/* fk_w4a16_gemv for callers whose activations and results live in HOST memory (no counterpart in
 * the reference, whose ops take device pointers only): enqueues, on `stream`, the copy of
 * activations[batch, k] from `host_activations` to `device_activations`, the GEMV into
 * `device_output`, and the copy of output[batch, n] back to `host_output`. The two device buffers
 * are caller-owned staging (batch*k and batch*n 16-bit elements) and hold the same data afterwards.
 * Nothing synchronises: read `host_output` after synchronising `stream`.
 * With pinned host memory that the device can address (cudaHostAlloc / cudaHostRegister; what
 * torch's pin_memory() gives) no copy engine is involved: a small kernel pulls the activations over
 * PCIe and the GEMV kernel itself stores each finished tile to `host_output` (set
 * FK_W4A16_HOST_ZERO_COPY=0 to force plain copies). Pageable memory takes cudaMemcpyAsync. */
FK_W4A16_API int fk_w4a16_gemv_host(const void* host_activations, const void* packets, void* host_output,
                       void* device_activations, void* device_output, void* workspace,
                       size_t workspace_bytes, int batch, int n, int k, int group_size,
                       int packet_stride_bytes, int dtype, void* stream);

/* The same GEMV with every option spelled out; fk_w4a16_gemv(...) is this call with the options
 * at their defaults. The options exist for layers that are sharded over the GPUs of one node
 * (no counterpart in the reference, which is single-GPU):
 *   - output_f32: write unrounded fp32 sums instead of 16-bit outputs (a K-shard's partial result);
 *   - output_ld / output_col0: place the n local columns inside a wider row-major matrix
 *     (an N-shard's slice of the full output);
 *   - peer_outputs: up to 7 more buffers -- other GPUs' memory mapped into this process -- that
 *     receive the same tiles by plain stores over NVLink while the kernel runs, so the exchange
 *     overlaps the computation tile by tile;
 *   - local_signal / peer_signals / wait_value: 32-bit counters in device memory, one per GPU of
 *     the group. Every CTA of the kernel, once its own stores are done everywhere, adds 1 (system
 *     scope, released after those stores) to each counter, and the kernel does not complete before
 *     local_signal has reached wait_value x (CTAs of its grid) -- bounded: after two seconds
 *     ("peer_wait_ms" of fk_w4a16_set_tuning) it gives up and sets the device status word. With
 *     wait_value = calls_so_far * (GPUs in the group), kernels queued after this call on the same
 *     stream see every GPU's contribution. Every GPU of the group must run the same problem shape
 *     on the same kind of device (the counters count CTAs). wait_value is fixed per call, so a call
 *     recorded into a CUDA graph cannot be replayed with these counters: the ll_* exchange below
 *     keeps its call count on the device for that. Leave local_signal NULL for single-GPU use.
 *   - reduce_input / reduce_output / reduce_slots: a K-split layer's sum over GPUs, fused behind the
 *     exchange: see the fields.
 *   - ll_epoch and the ll_* fields: the same exchange with the flag inside every stored word
 *     instead of counters: see the fields.
 *   - residual, epilogue, norm_weight / norm_eps: see the fields.
 * Zero-initialise the struct; unset fields then mean "default". */
#define FK_W4A16_MAX_PEERS 7
#define FK_W4A16_EPILOGUE_NONE 0
#define FK_W4A16_EPILOGUE_SILU_MUL 1
typedef struct fk_w4a16_gemv_args {
  const void* activations;
  const void* packets;
  void* output;
  void* workspace;
  size_t workspace_bytes;
  int batch, n, k, group_size, packet_stride_bytes, dtype;
  int output_f32;
  long long output_ld;   /* elements between rows of `output`; 0 means n */
  long long output_col0; /* column of `output` that receives local column 0 */
  int num_peers;
  void* peer_outputs[FK_W4A16_MAX_PEERS];
  unsigned int* peer_signals[FK_W4A16_MAX_PEERS];
  unsigned int* local_signal;
  unsigned int wait_value;
  void* stream;
  /* Fused residual add (a decoder's o_proj / down_proj): a 16-bit matrix laid out like `output`
   * (same output_ld and output_col0), or NULL. Every output becomes round16(y + residual) -- or
   * y + residual in fp32 with output_f32 -- with one rounding. May be the output buffer itself. */
  const void* residual;
  /* Fused epilogue. FK_W4A16_EPILOGUE_SILU_MUL treats the layer as a stacked [gate; up] projection
   * (a decoder's fused MLP input layer: rows 0 .. n/2-1 of W are the gate, the rest the up part):
   * the output has n/2 columns, out[m, j] = silu(y[m, j]) * y[m, j + n/2], computed in fp32 from
   * the unrounded sums and rounded once. n must be a multiple of 256; output_ld defaults to n/2;
   * batch * n/2 may not exceed 98304 (the two halves of a column meet in the workspace header). */
  int epilogue;
  /* Fused RMSNorm in front of the GEMV (a decoder's input_layernorm -> qkv, post_attention
   * layernorm -> gate/up), or NULL: `activations` holds the un-normalised rows x, and the GEMV
   * multiplies round16(norm_weight[k] * round16(x[k] * rsqrt(mean_k(x[k]^2) + norm_eps))) -- the
   * two roundings of the usual module. norm_weight: [k] of the 16-bit type. batch <= 4. */
  const void* norm_weight;
  float norm_eps;
  /* Fused reduction behind the exchange, or reduce_slots = 0. A K-split layer writes its unrounded
   * fp32 partial [batch, n] into slot `rank` of a [reduce_slots][batch][n] fp32 buffer on every GPU
   * (output / peer_outputs with output_f32). With these fields set, the kernel itself -- once the
   * counters show that every GPU has delivered -- adds the reduce_slots partials found in
   * reduce_input (this GPU's buffer, slot 0) in slot order and writes round16 of the sum to
   * reduce_output [batch, n]: no second launch. Needs local_signal. */
  const float* reduce_input;
  void* reduce_output;
  int reduce_slots;
  /* Flag-in-data exchange, or ll_epoch = 0: the lowest-latency way to share a sharded layer's
   * result. With ll_epoch != 0, `output` and `peer_outputs` are arrays of 8-byte words laid out
   * like an fp32 output (output_ld / output_col0 count words), and every result is written as
   * {fp32 value, ll_epoch}: an 8-byte store is atomic, so a word whose flag shows this call's epoch
   * carries this call's value -- no fence, no counter, no round trip over NVLink. ll_input is this
   * GPU's receive area, [ll_slots][batch][ll_slot_cols] words, one slot per GPU of the group (its
   * own included: point `output` at it); the kernel's first CTAs wait (bounded, "peer_wait_ms") for
   * each word and write ll_output (16-bit): [batch][ll_slots * ll_slot_cols], the slots' columns
   * side by side (ll_reduce = 0, an N-split), or [batch][ll_slot_cols], the slots added in order
   * and rounded once (ll_reduce = 1, a K-split). The epoch comes from the caller (ll_epoch: a
   * different value, never 0, for every call that writes the same receive area; alternate between
   * two areas so that a GPU that runs ahead cannot overwrite words its peers have not read yet) or
   * lives on the device: with ll_epoch_counter -- two consecutive 32-bit words in this GPU's
   * memory, zero before the first call -- a call's epoch is the counter plus one, the kernel adds
   * one when the call is complete, and the receive areas of odd epochs (`output`, every
   * peer_output and ll_input alike) lie ll_parity_words words behind those of even ones. Nothing
   * about the exchange is then baked into the launch, so a call recorded into a CUDA graph can be
   * replayed. Every GPU of the group must make the same calls in the same order. Excludes
   * local_signal, reduce_slots and the SiLU-and-multiply epilogue. */
  unsigned int ll_epoch;
  unsigned int* ll_epoch_counter;
  long long ll_parity_words;
  const void* ll_input;
  void* ll_output;
  int ll_slots;
  int ll_slot_cols;
  int ll_reduce;
} fk_w4a16_gemv_args;
FK_W4A16_API int fk_w4a16_gemv_ex(const fk_w4a16_gemv_args* args);

/* A chain of GEMVs in ONE persistent launch (no counterpart in the reference, whose Python caller
 * launches two or three kernels per GEMV). Step i + 1 may read what step i wrote -- a decoder's
 * o_proj -> gate/up -> down_proj -> next qkv with the fused residual / SiLU-and-multiply / RMSNorm
 * options in between -- and the results are those of the same steps issued one after another as
 * fk_w4a16_gemv_ex calls on the stream. What the chain saves is what lies between two launches
 * (grid completion, CTA launch, first copies: several microseconds per call at decode sizes): the
 * grid stays resident, steps are separated by a grid-wide barrier inside the kernel, and every warp
 * starts copying its share of the next step's weights as soon as it has consumed its share of the
 * current one. All steps share batch (at most 4), group size, packet stride and element type.
 * Workspace: fk_w4a16_chain_workspace_bytes(batch, group_size) bytes, zero-filled once
 * (fk_w4a16_workspace_init), reusable, one per chain running at a time. The kernel needs
 * every SM of the device for itself while it runs (one CTA per SM, all resident: they wait for one
 * another); its waits are bounded ("peer_wait_ms") and report through the device status word. */
#define FK_W4A16_MAX_CHAIN_STEPS 8
typedef struct fk_w4a16_chain_step {
  const void* activations; /* [batch, k] */
  const void* packets;     /* the layer's ARC packets */
  void* output;            /* [batch, n], or [batch, n/2] with the SiLU-and-multiply epilogue */
  int n, k;
  const void* residual;    /* as in fk_w4a16_gemv_args, or NULL */
  int epilogue;            /* FK_W4A16_EPILOGUE_* */
  const void* norm_weight; /* as in fk_w4a16_gemv_args, or NULL */
  float norm_eps;
} fk_w4a16_chain_step;
FK_W4A16_API size_t fk_w4a16_chain_workspace_bytes(int batch, int group_size);
FK_W4A16_API int fk_w4a16_gemv_chain(const fk_w4a16_chain_step* steps, int count, void* workspace,
                        size_t workspace_bytes, int batch, int group_size, int packet_stride_bytes,
                        int dtype, void* stream);

/* fk_w4a16_gemv for callers that cannot hand over scratch memory. This entry point has no
 * counterpart in the reference. It is meant for hosts where device allocation is off the table
 * once start-up is over: a serving process that has already handed all free device memory to its
 * own pools (so a later cudaMalloc fails or has to be carved out of someone else's budget), and
 * decode loops that cannot afford the device-wide stall an allocation implies. The scratch is a
 * fixed array of FK_W4A16_STATIC_SCRATCH_BYTES inside the library's device image; every GPU that
 * loads the library holds that much until the process exits, whether or not this function is used.
 *
 * Same arguments and results as fk_w4a16_gemv minus the workspace. Batches of 1 to 4 always run on
 * the CUDA-core kernels here, whose scratch (at most 862 KB on a 148-SM device) fits the array for
 * every layer shape -- so for batch 3 and 4 on large layers the result can differ in the last bit
 * from fk_w4a16_gemv, which moves those to the tensor-core kernel. Batches above 4 need more than
 * the array holds (the tensor-core plan's slots and staged activations) and are refused with
 * FK_W4A16_ERR_INVALID_ARGUMENT and a message that states both sizes. The function calls no
 * allocator of any kind. The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current); make that first call outside stream capture
 * (a lookup that fails is retried by the next call).
 * All calls on a device share the one array: the part a call depends on being zero is cleared on
 * `stream` before each launch, but two calls that overlap on the GPU (different streams, no
 * ordering between them) would race on it -- serialise them or use fk_w4a16_gemv with separate
 * workspaces. */
#define FK_W4A16_STATIC_SCRATCH_BYTES (1024 * 1024)
FK_W4A16_API int fk_w4a16_gemv_static(const void* activations, const void* packets, void* output, int batch,
                         int n, int k, int group_size, int packet_stride_bytes, int dtype,
                         void* stream);

/* Caller-visible split-K: partials[split_k_slices, batch, n] (fp32), slice s covering groups
 * [s * ceil(NG/S), ...). Reference: arc_w4a16_forward_split_k, arc_w4a16.cu:709-737. */
FK_W4A16_API int fk_w4a16_gemv_split_k(const void* activations, const void* packets, float* partials, int batch,
                          int n, int k, int group_size, int packet_stride_bytes,
                          int split_k_slices, int dtype, void* stream);

/* output[batch, n] = round16(sum over slices, in slice order).
 * Reference: reduce_arc_w4a16_split_k_partials, arc_w4a16.cu:739-751. */
FK_W4A16_API int fk_w4a16_reduce_partials(const float* partials, void* output, int batch, int n,
                             int split_k_slices, int dtype, void* stream);

/* weight[n, k] (16-bit) = alpha * q + beta, bit-exact with the reference.
 * Reference: dequant_w4a16_to_fp16, arc_w4a16.cu:753-770. */
FK_W4A16_API int fk_w4a16_dequant_rowmajor(const void* q, const void* alpha, const void* beta, void* weight,
                              int n, int k, int group_size, int dtype, void* stream);

/* The same from packets. Reference: dequant_arc_w4a16_packets_to_fp16, arc_w4a16.cu:772-789. */
FK_W4A16_API int fk_w4a16_dequant_packets(const void* packets, void* weight, int n, int k, int group_size,
                             int packet_stride_bytes, int dtype, void* stream);

/* Vendor baseline subject: output[batch, n] = activations[batch, k] . weight[n, k]^T through
 * cuBLASLt with fp32 compute. `lt_workspace` may be NULL when lt_workspace_bytes is 0.
 * Reference: cublaslt_fp16_with_weight, arc_w4a16.cu:791-803 (run_cublaslt_matmul :577-645). */
FK_W4A16_API int fk_w4a16_cublaslt_matmul(const void* activations, const void* weight, void* output,
                             void* lt_workspace, size_t lt_workspace_bytes, int batch, int n,
                             int k, int dtype, void* stream);

/* Reads (and clears) the device status word of the current device into *status (host pointer):
 * 0 = no device-side wait ever timed out. Synchronises the device. After a non-zero status the
 * outputs of the calls since the last check are undefined and their workspaces may hold
 * half-finished split-K state: zero them again (fk_w4a16_workspace_init) before reuse. */
FK_W4A16_API int fk_w4a16_device_status(int* status);

/* Launch-shape knobs of the fused GEMV, for tuning and tests: warps per CTA (1..16, 0 = auto),
 * ring stages per warp (1..8, 0 = auto) and CTAs in the grid (0 = one per SM). Process-wide. */
FK_W4A16_API int fk_w4a16_set_launch_config(int warps_per_cta, int stages, int ctas);

/* Writes a one-line description of the launch fk_w4a16_gemv would make for a problem on the current
 * device -- kernel name with its template arguments, grid, cluster size, warps, ring stages,
 * shared memory -- into text[capacity] (host pointer). For benchmarks and profiles that attribute
 * time to kernels; no counterpart in the reference. */
FK_W4A16_API int fk_w4a16_describe_plan(int batch, int n, int k, int group_size, int dtype, char* text,
                           size_t capacity);

/* Launch-plan thresholds, process-wide, for tuning and tests (no counterpart in the reference).
 * Each knob starts from an environment variable that is read once, at the library's first
 * planning call: "mma_min_batch" (FK_W4A16_MMA_MIN_BATCH: smallest batch that takes the mma.sync
 * kernel, 0 = built-in rule), "cluster_min" / "cluster_size" (FK_W4A16_CLUSTER_MIN / _SIZE),
 * "wmma" (FK_W4A16_WMMA: batches 1-2 on the warp-level mma.sync form of the stream kernel),
 * "cluster" (FK_W4A16_CLUSTER: 0 keeps every layer off the cluster kernel),
 * "umma_min_batch" (FK_W4A16_UMMA_MIN_BATCH: smallest batch that takes the pipelined tcgen05
 * kernel, 0 = never, -1 = built-in default), "peer_wait_ms" (FK_W4A16_PEER_WAIT_MS: how long a
 * multi-GPU call waits for the other GPUs before it gives up, default 2000). Results never depend
 * on them beyond the order of fp32 additions. */
FK_W4A16_API int fk_w4a16_set_tuning(const char* name, int value);

/* Kernel variant of the fused GEMV, process-wide, for measurements and tests (no counterpart in
 * the reference). AUTO picks per problem between the CUDA-core stream kernel, its cluster form and
 * the mma.sync kernel; TCGEN05 forces the warp-specialised tcgen05 / tensor-memory kernel for every
 * batch size -- same results, slower on decode shapes (its header says why); CLASSIC never uses
 * it. The environment variable FK_W4A16_TC5=1 selects TCGEN05 when this function was never
 * called. */
#define FK_W4A16_VARIANT_AUTO 0
#define FK_W4A16_VARIANT_TCGEN05 1
#define FK_W4A16_VARIANT_CLASSIC 2
FK_W4A16_API int fk_w4a16_set_variant(int variant);

#ifdef __cplusplus
}
#endif

#endif /* FK_W4A16_H_ */

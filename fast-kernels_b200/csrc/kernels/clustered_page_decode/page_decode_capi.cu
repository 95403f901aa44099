// extern "C" entry points of include/fk_page_decode.h: validation, launch plan, launch.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>

#include "fk_page_decode.h"
#include "page_decode_launch.h"

namespace fk_page_decode {

__device__ int g_page_decode_status = 0;

namespace {

thread_local std::string t_last_error;

int fail(int code, const std::string& message) {
  t_last_error = message;
  return code;
}

int fail_cuda(const char* what, cudaError_t err) {
  return fail(FK_PAGE_DECODE_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(err));
}

constexpr int kMaxDevices = 64;
constexpr size_t kTicketBytes = 64 * 1024;      // fixed header: one counter per task
constexpr int kMaxTicketTasks = kTicketBytes / 4;
constexpr int kWorkspaceBlocks = 1024;          // partial results the documented size has room for
constexpr int kMaxClusterMerge = 4;              // blocks of one task that merge inside a cluster
constexpr int kSharedBudget = 220 * 1024;       // of the 227 KB a block may use

struct DeviceInfo {
  bool known = false;
  int sm_count = 0;
  int* status = nullptr;
};

// Filled on first use per device; a failed query is retried by the next call.
int device_info(DeviceInfo* out) {
  static std::mutex mutex;
  static DeviceInfo table[kMaxDevices];
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    return fail_cuda("cudaGetDevice", err);
  }
  if (device < 0 || device >= kMaxDevices) {
    return fail(FK_PAGE_DECODE_ERR_CUDA, "device ordinal out of range");
  }
  std::lock_guard<std::mutex> lock(mutex);
  DeviceInfo& slot = table[device];
  if (!slot.known) {
    int sms = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (err != cudaSuccess) {
      return fail_cuda("cudaDeviceGetAttribute", err);
    }
    void* status = nullptr;
    err = cudaGetSymbolAddress(&status, g_page_decode_status);
    if (err != cudaSuccess) {
      return fail_cuda("cudaGetSymbolAddress", err);
    }
    slot.sm_count = sms;
    slot.status = static_cast<int*>(status);
    slot.known = true;
  }
  *out = slot;
  return FK_PAGE_DECODE_OK;
}

// FK_PAGE_DECODE_CLUSTER_MERGE=0 sends every split call through global scratch (for comparisons).
bool cluster_merge_enabled() {
  static const bool enabled = [] {
    const char* text = std::getenv("FK_PAGE_DECODE_CLUSTER_MERGE");
    return text == nullptr || text[0] != '0';
  }();
  return enabled;
}

// FK_PAGE_DECODE_TENSOR_CORES=0 keeps every call on the fp32 path (for comparisons).
bool tensor_cores_enabled() {
  static const bool enabled = [] {
    const char* text = std::getenv("FK_PAGE_DECODE_TENSOR_CORES");
    return text == nullptr || text[0] != '0';
  }();
  return enabled;
}

// Shared memory of a block such that two of them fit one SM (228 KB, 1 KB of it taken per block).
constexpr int kSharedPerResidentPair = 113 * 1024;

std::atomic<int> g_warps_override{0};
std::atomic<int> g_stages_override{0};

struct Plan {
  bool cluster_merge = false;
  Variant variant;
  int head_tiles = 0;
  int tasks = 0;
  int splits = 1;
  int warps = 0;
  int stages = 0;
  int shared_bytes = 0;
  size_t workspace_need = 0;
};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int smallest_tile_for(int heads) { return heads <= 1 ? 1 : heads <= 2 ? 2 : heads <= 4 ? 4 : 8; }

size_t partial_floats(int group_tile, int head_dim) { return static_cast<size_t>(group_tile) * (head_dim + 4); }

// Mirrors the checks of the reference's launcher (clustered_page_decode.cu:1095-1131), then plans.
int make_plan(const fk_page_decode_args& a, Plan* plan, bool check_workspace = true) {
  if (a.batch <= 0 || a.num_q_heads <= 0 || a.num_kv_heads <= 0) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "page decode received empty inputs");
  }
  if (a.num_runs < 0) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "num_runs must be non-negative");
  }
  if (a.head_dim != 64 && a.head_dim != 128) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "page decode only supports head_dim 64 or 128");
  }
  if (a.page_size != 16 && a.page_size != 32) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "page decode only supports page_size 16 or 32");
  }
  if (a.num_q_heads % a.num_kv_heads != 0) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "num_q_heads must be divisible by num_kv_heads");
  }
  if (a.group_tile != 0 && a.group_tile != 1 && a.group_tile != 2 && a.group_tile != 4 && a.group_tile != 8) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "group_tile must be one of {1, 2, 4, 8} (or 0)");
  }
  if (a.kv_format != FK_PAGE_DECODE_KV_BF16 && a.kv_format != FK_PAGE_DECODE_KV_FP8_E4M3 &&
      a.kv_format != FK_PAGE_DECODE_KV_INT8) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "unsupported kv_format");
  }
  if (a.splits < 0 || a.splits > kMaxSplits) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "splits must be in [0, 64]");
  }
  if ((a.flags & ~FK_PAGE_DECODE_FLAG_EARLY_DESCRIPTORS) != 0) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "unknown bits in flags");
  }
  if (a.max_pages_hint < 0) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "max_pages_hint must be non-negative");
  }
  if (a.query == nullptr || a.key_pages == nullptr || a.value_pages == nullptr || a.output == nullptr ||
      a.request_run_offsets == nullptr || a.seq_lens == nullptr) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "query, pages, output, request_run_offsets and seq_lens must not be NULL");
  }
  if (a.num_runs > 0 && (a.run_base_pages == nullptr || a.run_page_counts == nullptr ||
                         a.run_logical_starts == nullptr || a.run_last_page_lens == nullptr)) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "the run arrays must not be NULL when num_runs > 0");
  }
  if (a.kv_format != FK_PAGE_DECODE_KV_BF16 && (a.key_scales == nullptr || a.value_scales == nullptr)) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "quantised pages need key_scales and value_scales");
  }
  // bulk copies start at page boundaries: 16-byte aligned as soon as the bases are
  if (!aligned16(a.query) || !aligned16(a.key_pages) || !aligned16(a.value_pages) || !aligned16(a.output) ||
      (a.kv_format != FK_PAGE_DECODE_KV_BF16 && !aligned16(a.value_scales))) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "query, pages, value_scales and output must be 16-byte aligned");
  }
  if (!std::isfinite(a.softmax_scale) || !(a.rope_theta > 0.0f) || !std::isfinite(a.rope_theta)) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "softmax_scale must be finite and rope_theta positive");
  }

  DeviceInfo info;
  if (const int code = device_info(&info); code != FK_PAGE_DECODE_OK) {
    return code;
  }
  const int group = a.num_q_heads / a.num_kv_heads;
  const int wanted = a.group_tile == 0 ? 8 : a.group_tile;
  Plan out;
  int tile = smallest_tile_for(std::min(wanted, group));
  if (tile == 8 && static_cast<long long>(a.batch) * a.num_kv_heads * ((group + 7) / 8) * 2 <= info.sm_count) {
    // Few tasks: the call is bound by latency, not by traffic, and a tile of 4 heads runs 12 warps
    // per block where a tile of 8 has registers for 8 (measured on 2 requests x 4 kv heads x 4096
    // tokens, 8 heads per kv head: 15.5 us against 16.7). The tile is a tiling choice only: results
    // agree to fp32 rounding.
    tile = 4;
  }
  out.variant = Variant{a.head_dim, a.kv_format, a.keys_are_rotated != 0, tile};
  if (tensor_cores_enabled() && a.keys_are_rotated != 0) {
    // keys that carry their rotation are exact tensor-core operands (8-bit elements convert to
    // bf16 exactly): logits and weighted values as mma.sync, always with the full tile of 8 heads
    // (the MMA has the rows anyway)
    out.variant.tensor_cores = true;
    out.variant.group_tile = 8;
  }
  const int gt = out.variant.group_tile;
  out.head_tiles = (group + gt - 1) / gt;
  const long long tasks = static_cast<long long>(a.batch) * a.num_kv_heads * out.head_tiles;
  if (tasks > (1LL << 30)) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "too many (request, kv head, head tile) tasks");
  }
  out.tasks = static_cast<int>(tasks);

  // ring: as many warps as fit with `stages` buffers each
  out.stages = g_stages_override.load() > 0 ? g_stages_override.load() : 2;
  // The tensor-core variant: 12 warps keep HBM busy when most SMs have a task of their own (long
  // work per block); with few tasks the call is bound by latency and 8 warps (less to set up and
  // to merge) are quicker (4 x 8 x 256 tokens: 7.0 against 7.6 us; 2 x 4 x 4096: 12.6 against 14.8).
  const int warp_limit = out.variant.tensor_cores ? kMaxWarpsNarrow : max_warps_for(gt);
  int chosen_warps = out.variant.tensor_cores ? (out.tasks * 2 > info.sm_count ? kMaxWarpsNarrow : 8) : warp_limit;
  const long long waves_whole = (tasks + info.sm_count - 1) / info.sm_count;
  const long long waves_halved = (tasks + 2 * info.sm_count - 1) / (2 * info.sm_count);
  if (out.variant.tensor_cores && out.tasks > info.sm_count && 10 * waves_halved <= 6 * waves_whole &&
      variant_shared_bytes(out.variant, 6, out.stages) <= kSharedPerResidentPair) {
    // With more tasks than SMs, blocks of 12 warps run in waves and the last one leaves SMs idle;
    // blocks of 6 warps fit two to an SM, take twice as long each and start twice as many at
    // once, and one block's prologue and merge overlap the other's streaming. They win unless
    // they add more than a fifth to the wave count (bf16, requests x 8 kv heads x tokens, us with
    // 6 / 12 warps: 24 x 4096 73 / 89, 32 x 4096 87 / 93, 40 x 4096 155 / 136, 64 x 2048 92 / 111,
    // 75 x 2048 131 / 134, 100 x 1024 83 / 106; int8 pages alike).
    chosen_warps = 6;
  }
  int warps = g_warps_override.load() > 0 ? std::min(g_warps_override.load(), warp_limit) : chosen_warps;
  while (warps > 1 && variant_shared_bytes(out.variant, warps, out.stages) > kSharedBudget) {
    --warps;
  }
  out.warps = warps;
  out.shared_bytes = variant_shared_bytes(out.variant, warps, out.stages);
  if (out.shared_bytes < 0 || out.shared_bytes > 227 * 1024) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "launch configuration does not fit shared memory");
  }

  int splits = a.splits;
  if (splits == 0) {
    // Units (16 tokens) of the longest request, if the caller said; a block wants at least two
    // rounds of its warps' worth so that the ring has something to overlap.
    const long long units = static_cast<long long>(a.max_pages_hint) * (a.page_size / kUnitTokens);
    const int most = a.max_pages_hint > 0 ? static_cast<int>(std::max(1LL, units / (2LL * warps))) : kMaxSplits;
    // one block per SM: as many splits as fill the device. With more tasks than SMs every SM is
    // busy anyway and cutting further only adds merges (measured: 32 requests x 8 kv heads of 4096
    // tokens, 155 us uncut, 173 us cut in 4).
    splits = out.tasks <= info.sm_count ? info.sm_count / out.tasks : 1;
    splits = std::max(1, std::min({splits, most, kMaxSplits}));
    // 2 or 4 blocks per task can be one thread-block cluster and merge through shared memory (no
    // scratch, no ticket; 4 requests x 8 kv heads x 2048 tokens: 16.1 us against 16.9); worth it
    // when that power of two is not much below the count that fills the device. Clusters of 8
    // blocks of this size do not pack: 16 of them ran in two waves (26.7 us against 15.5 with 9
    // blocks per task through the workspace).
    int pow2 = 1;
    while (pow2 * 2 <= std::min(splits, kMaxClusterMerge)) {
      pow2 *= 2;
    }
    if (cluster_merge_enabled() && pow2 >= 2 && pow2 * 4 >= splits * 3) {
      splits = pow2;
    }
    // 8-bit pages on the tensor cores are bound by their instruction stream, so SMs without a task
    // are what costs: with more than half but at most two thirds of the SMs taken, three 6-warp
    // blocks per task (two resident per SM, merge through the workspace) bring every SM in. 10
    // and 12 requests x 8 kv heads x 4096 tokens, int8: 39.6 and 40.4 us against 48.2 and 49.1
    // (bf16 pages, bound by HBM: 40.4 and 44.1 against 40.6 and 42.3, left as they are).
    const int resident_splits = 2 * info.sm_count / std::max(1, out.tasks);
    if (out.variant.tensor_cores && a.kv_format != FK_PAGE_DECODE_KV_BF16 && g_warps_override.load() <= 0 &&
        splits == 1 && out.tasks <= info.sm_count && resident_splits >= 3 && a.max_pages_hint > 0 &&
        units / resident_splits >= 8LL * 6 && out.tasks <= kMaxTicketTasks && a.workspace != nullptr &&
        variant_shared_bytes(out.variant, 6, out.stages) <= kSharedPerResidentPair) {
      splits = resident_splits;
      out.warps = 6;
      out.shared_bytes = variant_shared_bytes(out.variant, 6, out.stages);
    }
  }
  out.cluster_merge = cluster_merge_enabled() && (splits == 2 || splits == 4);
  if (out.tasks > kMaxTicketTasks) {
    if (a.splits > 1) {
      return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "splits > 1 supports at most 16384 tasks");
    }
    splits = 1;
  }
  out.splits = splits;
  if (out.variant.tensor_cores && g_warps_override.load() <= 0 && out.warps == 8 && a.max_pages_hint > 0) {
    // Few tasks but long ones: 8 warps are the quicker choice only while a warp sees a handful of
    // units (prologue and merge weigh more than the streaming). From 8 units per warp of a
    // 12-warp block on, 12 warps win on 8-bit pages, whose conversion keeps the schedulers busy
    // (4 requests x 8 kv heads x 16384 tokens, int8: 53.4 us against 61.0; bf16 pages, bound by
    // HBM at that size, do not care: 53.6 against 54.4).
    const long long units = static_cast<long long>(a.max_pages_hint) * (a.page_size / kUnitTokens);
    if (units / splits >= 8LL * kMaxWarpsNarrow &&
        variant_shared_bytes(out.variant, kMaxWarpsNarrow, out.stages) <= kSharedBudget) {
      out.warps = kMaxWarpsNarrow;
      out.shared_bytes = variant_shared_bytes(out.variant, out.warps, out.stages);
    }
  }
  out.workspace_need =
      (splits == 1 || out.cluster_merge) ? 0 : kTicketBytes + static_cast<size_t>(out.tasks) * splits * partial_floats(gt, a.head_dim) * 4;
  if (out.workspace_need > 0 && check_workspace) {
    if (a.workspace == nullptr || a.workspace_bytes < out.workspace_need) {
      char text[160];
      std::snprintf(text, sizeof text, "workspace too small: %zu bytes needed for %d tasks x %d splits, %zu given",
                    out.workspace_need, out.tasks, splits, a.workspace == nullptr ? size_t{0} : a.workspace_bytes);
      return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, text);
    }
    if (!aligned16(a.workspace)) {
      return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "workspace must be 16-byte aligned");
    }
  }
  *plan = out;
  return FK_PAGE_DECODE_OK;
}

}  // namespace

#define FK_PD_DISPATCH(CALL)                                                        \
  if (v.head_dim == 64 && v.kv_format == kKvBf16) return CALL(d64_bf16);            \
  if (v.head_dim == 64 && v.kv_format == kKvFp8) return CALL(d64_fp8);              \
  if (v.head_dim == 64 && v.kv_format == kKvInt8) return CALL(d64_int8);            \
  if (v.head_dim == 128 && v.kv_format == kKvBf16) return CALL(d128_bf16);          \
  if (v.head_dim == 128 && v.kv_format == kKvFp8) return CALL(d128_fp8);            \
  if (v.head_dim == 128 && v.kv_format == kKvInt8) return CALL(d128_int8);

int variant_shared_bytes(const Variant& v, int warps, int stages) {
  if (v.tensor_cores) {
#define FK_PD_SHARED_MMA(NAME) shared_bytes_mma_##NAME(warps, stages)
    FK_PD_DISPATCH(FK_PD_SHARED_MMA)
#undef FK_PD_SHARED_MMA
    return -1;
  }
#define FK_PD_SHARED(NAME) shared_bytes_##NAME(v.keys_are_rotated, v.group_tile, warps, stages)
  FK_PD_DISPATCH(FK_PD_SHARED)
#undef FK_PD_SHARED
  return -1;
}

cudaError_t launch_variant(const Variant& v, const DecodeParams& params, int blocks, int warps, int stages,
                           cudaStream_t stream) {
  if (v.tensor_cores) {
#define FK_PD_LAUNCH_MMA(NAME) launch_mma_##NAME(params, blocks, warps, stages, stream)
    FK_PD_DISPATCH(FK_PD_LAUNCH_MMA)
#undef FK_PD_LAUNCH_MMA
    return cudaErrorInvalidValue;
  }
#define FK_PD_LAUNCH(NAME) launch_##NAME(v.keys_are_rotated, v.group_tile, params, blocks, warps, stages, stream)
  FK_PD_DISPATCH(FK_PD_LAUNCH)
#undef FK_PD_LAUNCH
  return cudaErrorInvalidValue;
}
#undef FK_PD_DISPATCH

}  // namespace fk_page_decode

using namespace fk_page_decode;

extern "C" {

FK_PAGE_DECODE_API const char* fk_page_decode_last_error(void) { return t_last_error.c_str(); }

FK_PAGE_DECODE_API size_t fk_page_decode_workspace_bytes(int batch, int num_q_heads, int num_kv_heads, int head_dim) {
  if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || (head_dim != 64 && head_dim != 128)) {
    fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "workspace_bytes: batch and head counts must be positive, head_dim 64 or 128");
    return 0;
  }
  // the fixed ticket header plus kWorkspaceBlocks partial results of the widest head tile: more
  // than any automatic plan uses (at most one block per SM shares a task with others)
  return kTicketBytes + static_cast<size_t>(kWorkspaceBlocks) * partial_floats(8, head_dim) * 4;
}

FK_PAGE_DECODE_API int fk_page_decode_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (workspace == nullptr || workspace_bytes < kTicketBytes) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "workspace_init: workspace is NULL or smaller than its header");
  }
  const cudaError_t err = cudaMemsetAsync(workspace, 0, kTicketBytes, static_cast<cudaStream_t>(stream));
  return err == cudaSuccess ? FK_PAGE_DECODE_OK : fail_cuda("cudaMemsetAsync", err);
}

FK_PAGE_DECODE_API int fk_page_decode_forward(const fk_page_decode_args* args) {
  if (args == nullptr) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "args must not be NULL");
  }
  const fk_page_decode_args& a = *args;
  Plan plan;
  if (const int code = make_plan(a, &plan); code != FK_PAGE_DECODE_OK) {
    return code;
  }
  DeviceInfo info;
  if (const int code = device_info(&info); code != FK_PAGE_DECODE_OK) {
    return code;
  }
  DecodeParams params{};
  params.query = static_cast<const uint16_t*>(a.query);
  params.key_pages = static_cast<const uint8_t*>(a.key_pages);
  params.value_pages = static_cast<const uint8_t*>(a.value_pages);
  params.key_scales = a.key_scales;
  params.value_scales = a.value_scales;
  params.run_base_pages = a.run_base_pages;
  params.run_page_counts = a.run_page_counts;
  params.run_logical_starts = a.run_logical_starts;
  params.run_last_page_lens = a.run_last_page_lens;
  params.request_run_offsets = a.request_run_offsets;
  params.seq_lens = a.seq_lens;
  params.output = static_cast<uint16_t*>(a.output);
  params.tickets = static_cast<unsigned*>(a.workspace);
  params.partials = a.workspace == nullptr
                        ? nullptr
                        : reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) + kTicketBytes);
  params.status = info.status;
  params.num_q_heads = a.num_q_heads;
  params.num_kv_heads = a.num_kv_heads;
  params.group_size = a.num_q_heads / a.num_kv_heads;
  params.head_tiles = plan.head_tiles;
  params.page_size = a.page_size;
  params.splits = plan.splits;
  params.stages = plan.stages;
  params.cluster_merge = plan.cluster_merge ? 1 : 0;
  params.early_descriptors = (a.flags & FK_PAGE_DECODE_FLAG_EARLY_DESCRIPTORS) != 0 ? 1 : 0;
  params.scale_log2e = static_cast<float>(static_cast<double>(a.softmax_scale) * 1.4426950408889634);
  for (int i = 0; i < a.head_dim / 2; ++i) {
    params.inv_freq[i] = static_cast<float>(
        std::pow(static_cast<double>(a.rope_theta), -2.0 * static_cast<double>(i) / static_cast<double>(a.head_dim)));
  }
  const long long blocks = static_cast<long long>(plan.tasks) * plan.splits;
  if (blocks > 0x7fffffffLL) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "grid too large");
  }
  const cudaError_t err = launch_variant(plan.variant, params, static_cast<int>(blocks), plan.warps, plan.stages,
                                         static_cast<cudaStream_t>(a.stream));
  return err == cudaSuccess ? FK_PAGE_DECODE_OK : fail_cuda("page decode launch", err);
}

FK_PAGE_DECODE_API int fk_page_decode_device_status(int* status) {
  if (status == nullptr) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "status must not be NULL");
  }
  DeviceInfo info;
  if (const int code = device_info(&info); code != FK_PAGE_DECODE_OK) {
    return code;
  }
  int value = 0;
  cudaError_t err = cudaMemcpy(&value, info.status, sizeof value, cudaMemcpyDeviceToHost);
  if (err == cudaSuccess && value != 0) {
    err = cudaMemset(info.status, 0, sizeof value);
  }
  if (err != cudaSuccess) {
    return fail_cuda("device status", err);
  }
  *status = value;
  return FK_PAGE_DECODE_OK;
}

FK_PAGE_DECODE_API int fk_page_decode_describe_plan(const fk_page_decode_args* args, char* text, size_t capacity) {
  if (args == nullptr || text == nullptr || capacity == 0) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "describe_plan: args and text must not be NULL");
  }
  Plan plan;
  if (const int code = make_plan(*args, &plan, false); code != FK_PAGE_DECODE_OK) {
    return code;
  }
  std::snprintf(text, capacity, "kernel=%s blocks=%lld tasks=%d splits=%d merge=%s group_tile=%d warps=%d stages=%d shared=%d",
                plan.variant.tensor_cores ? "page_decode_mma" : "page_decode",
                static_cast<long long>(plan.tasks) * plan.splits, plan.tasks, plan.splits,
                plan.splits == 1 ? "none" : plan.cluster_merge ? "cluster" : "global", plan.variant.group_tile,
                plan.warps, plan.stages, plan.shared_bytes);
  return FK_PAGE_DECODE_OK;
}

FK_PAGE_DECODE_API int fk_page_decode_set_launch_config(int warps_per_block, int stages) {
  if (warps_per_block < 0 || warps_per_block > kMaxWarpsNarrow || stages < 0 || stages > 8) {
    return fail(FK_PAGE_DECODE_ERR_INVALID_ARGUMENT, "warps_per_block must be in [0, 12], stages in [0, 8]");
  }
  g_warps_override.store(warps_per_block);
  g_stages_override.store(stages);
  return FK_PAGE_DECODE_OK;
}

}  // extern "C"

// Host side of libfk_w4a16.so: argument checks, launch planning and the extern "C" entry points
// declared in include/fk_w4a16.h. Nothing here allocates device memory or synchronises, except
// fk_w4a16_device_status() which is documented to.
#include "fk_w4a16.h"

#include <cublasLt.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <sstream>
#include <string>
#include <type_traits>

#include "w4a16_common.cuh"
#include "w4a16_gemv_stream.cuh"
#include "w4a16_gemm_mma.cuh"
#include "w4a16_gemv_cluster.cuh"
#include "w4a16_gemv_chain.cuh"
#include "w4a16_gemv_wmma.cuh"
#include "w4a16_launch.h"
#include "w4a16_umma_plan.cuh"
#include "w4a16_prep.cuh"

#ifndef FK_W4A16_VERSION
#define FK_W4A16_VERSION "0.1.0"
#endif

namespace fk_w4a16 {
namespace {

__device__ int g_device_status = 0;

// Scratch of fk_w4a16_gemv_static. In host code this name is only a handle for
// cudaGetSymbolAddress; kernels are given the address that call returns.
static __device__ __align__(256) unsigned char g_static_scratch[FK_W4A16_STATIC_SCRATCH_BYTES];

thread_local std::string t_last_error;

int fail(int code, const std::string& message) {
  t_last_error = message;
  return code;
}

#define FK_TRY_CUDA(expr)                                                                 \
  do {                                                                                    \
    const cudaError_t status__ = (expr);                                                  \
    if (status__ != cudaSuccess) {                                                        \
      return fail(FK_W4A16_ERR_CUDA,                                                      \
                  std::string(#expr) + " failed: " + cudaGetErrorString(status__));       \
    }                                                                                     \
  } while (false)

#define FK_TRY_CUBLAS(expr)                                                               \
  do {                                                                                    \
    const cublasStatus_t status__ = (expr);                                               \
    if (status__ != CUBLAS_STATUS_SUCCESS) {                                              \
      return fail(FK_W4A16_ERR_CUDA,                                                      \
                  std::string(#expr) + " failed: " + cublasLtGetStatusString(status__));  \
    }                                                                                     \
  } while (false)

#define FK_TRY(expr)                  \
  do {                                \
    const int rc__ = (expr);          \
    if (rc__ != FK_W4A16_OK) {        \
      return rc__;                    \
    }                                 \
  } while (false)

// ---- argument checks (same rules and wording as the reference, arc_w4a16.cu:28-57) -----------
bool group_supported(int group_size) {
  return group_size == 32 || group_size == 64 || group_size == 128;
}

int check_group_and_k(int batch, int k, int group_size) {
  if (batch <= 0 || k <= 0) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "batch and k must be positive");
  }
  if (!group_supported(group_size)) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "group_size must be 32, 64 or 128");
  }
  if (k % group_size != 0) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "k must be divisible by group_size");
  }
  return FK_W4A16_OK;
}

int check_dimensions(int batch, int n, int k, int group_size) {
  FK_TRY(check_group_and_k(batch, k, group_size));
  if (n <= 0) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "n must be positive");
  }
  if (n % kTileCols != 0) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "n must be a multiple of 128");
  }
  if (static_cast<long long>(n / kTileCols) * (k / group_size) > (1LL << 30)) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "n * k is too large: more than 2^30 packets");
  }
  return FK_W4A16_OK;
}

int check_stride(int group_size, int packet_stride_bytes) {
  const int expected = packet_stride(group_size);
  if (packet_stride_bytes != expected) {
    std::ostringstream oss;
    oss << "packet_stride_bytes=" << packet_stride_bytes << " does not match expected " << expected;
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, oss.str());
  }
  return FK_W4A16_OK;
}

int check_dtype(int dtype) {
  if (dtype != FK_W4A16_DTYPE_F16 && dtype != FK_W4A16_DTYPE_BF16) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "dtype must be FK_W4A16_DTYPE_F16 or _BF16");
  }
  return FK_W4A16_OK;
}

int check_pointer(const void* ptr, const char* name, size_t alignment) {
  if (ptr == nullptr) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, std::string(name) + " must not be null");
  }
  if ((reinterpret_cast<uintptr_t>(ptr) % alignment) != 0) {
    std::ostringstream oss;
    oss << name << " must be aligned to " << alignment << " bytes";
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, oss.str());
  }
  return FK_W4A16_OK;
}

// ---- per-device facts, read once ---------------------------------------------------------
constexpr int kMaxDevices = 64;
struct DeviceInfo {
  int sm_count = 0;
  int max_smem_optin = 0;
  int* status_word = nullptr;
};

int device_info(DeviceInfo** out) {
  static DeviceInfo infos[kMaxDevices];
  static std::atomic<bool> ready[kMaxDevices];
  static std::mutex lock;
  int device = 0;
  FK_TRY_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) {
    return fail(FK_W4A16_ERR_CUDA, "device index out of range");
  }
  if (!ready[device].load(std::memory_order_acquire)) {
    // A lookup that fails (a first call made while a stream is being captured, say) leaves the
    // entry unset, so a later call made under better conditions can still succeed.
    std::lock_guard<std::mutex> guard(lock);
    if (!ready[device].load(std::memory_order_relaxed)) {
      DeviceInfo info;
      cudaError_t err = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device);
      if (err == cudaSuccess) {
        err = cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                     device);
      }
      if (err == cudaSuccess) {
        void* addr = nullptr;
        err = cudaGetSymbolAddress(&addr, g_device_status);
        info.status_word = static_cast<int*>(addr);
      }
      if (err != cudaSuccess || info.status_word == nullptr) {
        return fail(FK_W4A16_ERR_CUDA,
                    std::string("device query failed: ") + cudaGetErrorString(err));
      }
      infos[device] = info;
      ready[device].store(true, std::memory_order_release);
    }
  }
  *out = &infos[device];
  return FK_W4A16_OK;
}

// ---- launch planning for the fused GEMV --------------------------------------------------
// A caller-owned workspace starts with a fixed header that must be zero before the first call
// and that every call leaves zero again: the ticket area, then the pair-exchange area (see
// finish_cta). Per-plan scratch follows the header.
constexpr size_t kTicketBytes = 256 * 1024;
constexpr int kTicketCapacity = static_cast<int>(kTicketBytes / sizeof(int));
constexpr size_t kExchangeBytes = 768 * 1024;
constexpr size_t kHeaderBytes = kTicketBytes + kExchangeBytes;
constexpr int kMaxWarps = 16;
constexpr int kMaxStages = 8;
constexpr int kUmmaDefaultMinBatch = 0;  // 0: the pipelined tcgen05 kernel is opt-in

struct LaunchConfig {
  int warps = 0;
  int stages = 0;
  int ctas = 0;
};
LaunchConfig g_config;
std::once_flag g_config_env_once;

int env_int(const char* name) {
  const char* value = std::getenv(name);
  return value == nullptr ? 0 : std::atoi(value);
}

const LaunchConfig& launch_config() {
  std::call_once(g_config_env_once, [] {
    if (g_config.warps == 0) g_config.warps = env_int("FK_W4A16_WARPS");
    if (g_config.stages == 0) g_config.stages = env_int("FK_W4A16_STAGES");
    if (g_config.ctas == 0) g_config.ctas = env_int("FK_W4A16_CTAS");
  });
  return g_config;
}

// Tuning knobs of the launch plan. Each starts from its environment variable, read ONCE (a
// getenv per knob on every call costs more host time than the launch itself), and can be
// changed at run time with fk_w4a16_set_tuning().
struct Tuning {
  int mma_min_batch = 0;   // FK_W4A16_MMA_MIN_BATCH: smallest batch for the mma.sync kernel (0 = rule)
  int cluster_min = 0;     // FK_W4A16_CLUSTER_MIN: smallest cluster size tried (0 = 2)
  int cluster_size = 0;    // FK_W4A16_CLUSTER_SIZE: forced cluster size (0 = rule)
  int wmma = 0;            // FK_W4A16_WMMA: batches 1-2 on the warp-level mma.sync form
  int umma_min_batch = -1; // FK_W4A16_UMMA_MIN_BATCH: smallest batch for the pipelined tcgen05 kernel
                           // (-1 = built-in default, 0 = never)
  int peer_wait_ms = 2000; // FK_W4A16_PEER_WAIT_MS: how long a multi-GPU call waits for the other GPUs
  int cluster = 1;         // FK_W4A16_CLUSTER: 0 keeps layers with few tiles off the cluster kernel
};
Tuning g_tuning;
std::once_flag g_tuning_once;
Tuning& tuning() {
  std::call_once(g_tuning_once, [] {
    g_tuning.mma_min_batch = env_int("FK_W4A16_MMA_MIN_BATCH");
    g_tuning.cluster_min = env_int("FK_W4A16_CLUSTER_MIN");
    g_tuning.cluster_size = env_int("FK_W4A16_CLUSTER_SIZE");
    g_tuning.wmma = env_int("FK_W4A16_WMMA");
    const char* text = std::getenv("FK_W4A16_UMMA_MIN_BATCH");
    g_tuning.umma_min_batch = text == nullptr ? -1 : std::atoi(text);
    if (env_int("FK_W4A16_PEER_WAIT_MS") > 0) {
      g_tuning.peer_wait_ms = env_int("FK_W4A16_PEER_WAIT_MS");
    }
    const char* cluster = std::getenv("FK_W4A16_CLUSTER");
    g_tuning.cluster = cluster == nullptr || std::atoi(cluster) != 0 ? 1 : 0;
  });
  return g_tuning;
}

int m_tile_for_batch(int batch) { return batch <= 1 ? 1 : (batch <= 2 ? 2 : 4); }

struct Plan {
  int m_tile = 1;
  int row_tiles = 1;
  int warps = 1;
  int stages = 0;  // 0 means the configuration does not fit in shared memory
  int grid_x = 1;
  int active_warps = 1;
  uint32_t total_packets = 0;
  size_t smem_bytes = 0;
  size_t scratch_bytes = 0;
  int cluster_size = 1;       // > 1: the cluster kernel, one cluster of this many CTAs per tile
  bool tensor_cores = false;  // batch > 4: the MMA kernel, rows in tiles of 8 or 16
  bool wmma = false;          // batch <= 2: the stream kernel with its inner product on mma.sync
  bool umma = false;          // the pipelined tcgen05 kernel: one run per CTA, rows in {1,2,4,8,16}
  size_t staged_bytes = 0;    // its pre-staged activations, behind the scratch slots
};

// Shared memory of the tensor-core kernel: barriers | one slot per warp | rings.
size_t mma_smem_bytes(int warps, int stages, int group, int mt) {
  const size_t stage = (3 * ((group / 32) * 512 + 32)) + ((group / 32) * 512) + kScaleBytes +
                       (static_cast<size_t>(mt) * mma_act_pitch(group));
  return (((static_cast<size_t>(warps) * stages * 8) + 127) & ~size_t{127}) +
         (static_cast<size_t>(warps) * mt * kTileCols * 4) + (static_cast<size_t>(warps) * stages * stage);
}

// `sm_count` and `max_smem` describe the device; the plan is a pure function of its arguments
// so that fk_w4a16_workspace_bytes() and fk_w4a16_gemv() always agree.
bool cluster_mode_enabled() { return tuning().cluster != 0; }

Plan make_plan(int batch, int n, int k, int group_size, int sm_count, int max_smem,
               const LaunchConfig& cfg, bool allow_cluster = false, bool cuda_cores_only = false) {
  Plan plan;
  const long long total_packets = static_cast<long long>(n / kTileCols) * (k / group_size);
  plan.total_packets = static_cast<uint32_t>(total_packets);
  // Batches 3 and 4 also go to the tensor-core kernel when the layer is large enough to hide its
  // activation prepass (measured on B200: 23 us against 35 on 28672 x 4096, 18.5 against 22 on
  // 4096 x 14336, but 13 against 7.7 on 4096 x 4096).
  // ... and batches of 2 as well on layers too wide for the cluster kernel (28672 x 8192: 32.2
  // against 37.3 us; 28672 x 4096: 20.5 against 22.6), where the CUDA-core kernel pays its FMAs
  // twice; the cluster kernel keeps batch 2 (4096 x 14336: 13.5 against 16.6 us).
  const bool cluster_shape = static_cast<long long>(n / kTileCols) * 2 <= sm_count;
  const int mma_min_batch = tuning().mma_min_batch > 0 ? tuning().mma_min_batch
                            : total_packets >= 3072    ? (cluster_shape ? 3 : 2)
                                                       : 5;
  if (batch >= mma_min_batch && !(cuda_cores_only && batch <= 4)) {
    plan.tensor_cores = true;
    plan.m_tile = batch <= 8 ? 8 : 16;
    plan.row_tiles = (batch + plan.m_tile - 1) / plan.m_tile;
    // The unit of work is a PAIR of warps per packet; `warps` counts pairs from here on.
    int warps = cfg.warps > 0 ? cfg.warps : (plan.m_tile == 8 ? 8 : 6);
    warps = warps > 8 ? 8 : warps;
    const int ctas = (cfg.ctas > 0 ? cfg.ctas : sm_count) > 256 ? 256 : (cfg.ctas > 0 ? cfg.ctas : sm_count);
    long long workers = static_cast<long long>(ctas) * warps;
    workers = workers > total_packets ? total_packets : workers;
    warps = static_cast<int>((workers + ctas - 1) / ctas);
    plan.warps = warps;
    plan.grid_x = static_cast<int>((workers + warps - 1) / warps);
    plan.active_warps = static_cast<int>(workers);
    const long long longest_run = (total_packets + workers - 1) / workers;
    int wanted = cfg.stages > 0 ? cfg.stages : 3;
    wanted = wanted > longest_run ? static_cast<int>(longest_run) : wanted;
    plan.stages = 0;
    for (int candidate = wanted; candidate >= 1; --candidate) {
      if (mma_smem_bytes(warps, candidate, group_size, plan.m_tile) <= static_cast<size_t>(max_smem)) {
        plan.stages = candidate;
        break;
      }
    }
    plan.smem_bytes = mma_smem_bytes(warps, plan.stages < 1 ? 1 : plan.stages, group_size, plan.m_tile);
    plan.scratch_bytes = static_cast<size_t>(plan.row_tiles) * plan.grid_x * 2 *
                         (plan.m_tile * kTileCols) * sizeof(float);
    plan.staged_bytes = static_cast<size_t>(plan.row_tiles) * (k / group_size) * plan.m_tile *
                        mma_act_pitch(group_size);
    return plan;
  }
  plan.m_tile = m_tile_for_batch(batch);
  plan.row_tiles = (batch + plan.m_tile - 1) / plan.m_tile;
  const int stage_bytes = packet_stride(group_size);

  // Two or more CTAs per tile: every tile is shared by several CTAs anyway, so give each tile a
  // cluster of CTAs that finishes it through distributed shared memory. The cluster size is the
  // largest power of two that fits (#SM / tiles, at most 8): clusters of 3 do not pack into the
  // GPCs one CTA per SM and run in two waves (6144 x 4096: 9.4 us with 3, 5.7 with 2, 6.8 on the
  // stream kernel), and the idle SMs of a power-of-two grid cost less than the global-memory
  // finish even on large layers (8192 x 8192: 10.3 against 12.6 us; 8192 x 28672: 25.7 / 26.2).
  const int tiles = n / kTileCols;
  const int groups = k / group_size;
  const int min_cluster = tuning().cluster_min > 0 ? tuning().cluster_min : 2;
  if (allow_cluster && cluster_mode_enabled() && cfg.ctas == 0 && tiles * min_cluster <= sm_count) {
    int cluster = sm_count / tiles;
    cluster = cluster >= 8 ? 8 : (cluster >= 4 ? 4 : 2);
    if (tuning().cluster_size > 0) {
      cluster = tuning().cluster_size;
    }
    cluster = cluster > groups ? groups : cluster;
    if (cluster >= 2) {
      int want_warps = (groups + cluster - 1) / cluster;
      const int warp_cap = cfg.warps > 0 ? cfg.warps : kMaxWarps;
      want_warps = want_warps > warp_cap ? warp_cap : want_warps;
      for (int warps = want_warps; warps >= 1; --warps) {
        const int longest_run = (groups + (cluster * warps) - 1) / (cluster * warps);
        int stages = cfg.stages > 0 ? cfg.stages : 3;
        stages = stages > longest_run ? longest_run : stages;
        const int floor_stages = longest_run < 2 ? 1 : 2;
        for (; stages >= floor_stages; --stages) {
          if (cluster_smem_plan(warps, stages, group_size, plan.m_tile).total <=
              static_cast<uint32_t>(max_smem)) {
            break;
          }
        }
        if (stages >= floor_stages) {
          plan.cluster_size = cluster;
          plan.warps = warps;
          plan.stages = stages;
          plan.grid_x = tiles * cluster;
          plan.active_warps = plan.grid_x * warps;
          plan.smem_bytes = cluster_smem_plan(warps, stages, group_size, plan.m_tile).total;
          // Ask for more than half an SM's shared memory, so that no SM ever holds two CTAs of
          // this kernel. The grid leaves SMs idle, and the block scheduler otherwise stacks two
          // or three CTAs on some SMs while launches overlap, where they compete for issue slots
          // (measured: the stacked CTAs finish 1.3-2.5 us late on a 4096 x 4096 layer).
          {
            const size_t floor_bytes = (static_cast<size_t>(max_smem) / 2) + 1024;
            if (floor_bytes > plan.smem_bytes) {
              plan.smem_bytes = floor_bytes;
            }
          }
          plan.scratch_bytes = 0;
          return plan;
        }
      }
    }
  }

  // Batches of 1 and 2 may take the warp-level MMA form of the stream kernel (opt-in while it is
  // being measured): same plan, slightly larger ring stages.
  plan.wmma = plan.m_tile <= 2 && tuning().wmma != 0;
  const int ring_stage_bytes = plan.wmma ? wmma_stage_bytes(group_size) : stage_bytes;
  auto smem_plan = [&](int w, int s) {
    return plan.wmma ? wmma_smem_plan(w, s, group_size, plan.m_tile)
                     : stream_smem_plan(w, s, group_size, plan.m_tile);
  };

  // Default: as many warps as fit with a two-deep ring each (more warps hide more latency than
  // deeper rings do), at most 16.
  int warps = cfg.warps;
  if (warps <= 0) {
    const int per_warp = (2 * ring_stage_bytes) + (2 * plan.m_tile * kTileCols * 4) +
                         (plan.m_tile * group_size * 2) + 16;
    warps = (max_smem - 256) / per_warp;
    warps = warps > kMaxWarps ? kMaxWarps : (warps < 1 ? 1 : warps);
  }
  warps = warps > kMaxWarps ? kMaxWarps : warps;
  const int ctas = (cfg.ctas > 0 ? cfg.ctas : sm_count) > 256 ? 256 : (cfg.ctas > 0 ? cfg.ctas : sm_count);
  long long workers = static_cast<long long>(ctas) * warps;
  if (workers > total_packets) {
    workers = total_packets;
  }
  // Spread the workers over all CTAs rather than filling the first ones.
  warps = static_cast<int>((workers + ctas - 1) / ctas);
  plan.warps = warps;
  plan.grid_x = static_cast<int>((workers + warps - 1) / warps);
  plan.active_warps = static_cast<int>(workers);

  // A ring deeper than the longest run is wasted shared memory -- and a small footprint is what
  // lets the next launch's CTAs move in early under programmatic dependent launch.
  const long long longest_run = (total_packets + workers - 1) / workers;
  int wanted = cfg.stages > 0 ? cfg.stages : 4;
  wanted = wanted > kMaxStages ? kMaxStages : wanted;
  if (wanted > longest_run) {
    wanted = static_cast<int>(longest_run);
  }
  int stages = 0;
  for (int candidate = wanted; candidate >= (longest_run < 2 ? 1 : 2); --candidate) {
    if (smem_plan(warps, candidate).total <= static_cast<uint32_t>(max_smem)) {
      stages = candidate;
      break;
    }
  }
  plan.stages = stages;
  plan.smem_bytes = smem_plan(warps, stages < 1 ? 1 : stages).total;
  plan.scratch_bytes = static_cast<size_t>(plan.row_tiles) * plan.grid_x * 2 *
                       (plan.m_tile * kTileCols) * sizeof(float);
  return plan;
}

std::atomic<int> g_variant{-1};  // -1: not set, take FK_W4A16_TC5 from the environment
// 1: every batch size takes the tcgen05 kernel; 0: none does; -1: the default rule.
int umma_forced() {
  const int variant = g_variant.load(std::memory_order_relaxed);
  if (variant >= 0) {
    return variant == FK_W4A16_VARIANT_TCGEN05 ? 1 : (variant == FK_W4A16_VARIANT_AUTO ? -1 : 0);
  }
  static const int from_env = std::getenv("FK_W4A16_TC5") == nullptr ? -1 : (env_int("FK_W4A16_TC5") != 0 ? 1 : 0);
  return from_env;
}

// Which problems take the pipelined tcgen05 kernel by default (FK_W4A16_UMMA_MIN_BATCH overrides
// the batch threshold; 0 there means "never").
bool umma_wanted(int batch, int n, int k, int group_size) {
  const int forced = umma_forced();
  if (forced >= 0) {
    return forced == 1;
  }
  (void)n; (void)k; (void)group_size;
  const int min_batch = tuning().umma_min_batch < 0 ? kUmmaDefaultMinBatch : tuning().umma_min_batch;
  return min_batch > 0 && batch >= min_batch;
}

// Plan of the pipelined tcgen05 kernel: one run of the packet stream per CTA.
Plan make_umma_plan(int batch, int n, int k, int group_size, int sm_count, int max_smem,
                    const LaunchConfig& cfg) {
  Plan plan;
  plan.umma = true;
  const long long total_packets = static_cast<long long>(n / kTileCols) * (k / group_size);
  plan.total_packets = static_cast<uint32_t>(total_packets);
  plan.m_tile = umma_rows_for_batch(batch);
  plan.row_tiles = (batch + plan.m_tile - 1) / plan.m_tile;
  int ctas = cfg.ctas > 0 ? cfg.ctas : sm_count;
  ctas = ctas > 256 ? 256 : ctas;
  const long long workers = ctas < total_packets ? ctas : total_packets;
  plan.warps = 1;
  plan.grid_x = static_cast<int>(workers);
  plan.active_warps = static_cast<int>(workers);
  const long long longest_run = (total_packets + workers - 1) / workers;
  int wanted = cfg.stages > 0 ? cfg.stages : kUmmaMaxStages;
  wanted = wanted > kUmmaMaxStages ? kUmmaMaxStages : wanted;
  wanted = wanted > longest_run ? static_cast<int>(longest_run) : wanted;
  plan.stages = 0;
  for (int candidate = wanted; candidate >= 1; --candidate) {
    if (umma_smem_plan(candidate, group_size, plan.m_tile).total <= static_cast<uint32_t>(max_smem)) {
      plan.stages = candidate;
      break;
    }
  }
  plan.smem_bytes = umma_smem_plan(plan.stages < 1 ? 1 : plan.stages, group_size, plan.m_tile).total;
  // one CTA per SM: each allocates all of the SM's tensor memory
  const size_t floor_bytes = (static_cast<size_t>(max_smem) / 2) + 1024;
  plan.smem_bytes = plan.smem_bytes < floor_bytes ? floor_bytes : plan.smem_bytes;
  plan.scratch_bytes = static_cast<size_t>(plan.row_tiles) * plan.grid_x * 2 *
                       (plan.m_tile * kTileCols) * sizeof(float);
  return plan;
}

size_t workspace_bytes_for(const Plan& plan, size_t header_bytes = kHeaderBytes) {
  return header_bytes + ((plan.scratch_bytes + 255) & ~size_t{255}) +
         ((plan.staged_bytes + 255) & ~size_t{255});
}

// Opts a kernel in to the device's full dynamic shared memory, once per function and device
// (minus whatever the kernel declares statically). `flags` must be distinct per instantiation.
template <class Kernel>
int ensure_smem_optin(Kernel kernel, std::once_flag (&flags)[kMaxDevices], size_t bytes,
                      int max_smem) {
  int device = 0;
  FK_TRY_CUDA(cudaGetDevice(&device));
  cudaError_t err = cudaSuccess;
  std::call_once(flags[device], [&] {
    cudaFuncAttributes attrs{};
    err = cudaFuncGetAttributes(&attrs, kernel);
    if (err == cudaSuccess) {
      err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 max_smem - static_cast<int>(attrs.sharedSizeBytes));
    }
  });
  if (err != cudaSuccess) {
    return fail(FK_W4A16_ERR_CUDA,
                std::string("cudaFuncSetAttribute failed: ") + cudaGetErrorString(err));
  }
  if (bytes > static_cast<size_t>(max_smem)) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "launch needs more shared memory than the device has");
  }
  return FK_W4A16_OK;
}

// Launches with programmatic stream serialisation: the kernel may begin (and prefetch weights)
// while its predecessor in the stream drains; it orders itself with griddepcontrol.wait before it
// reads activations or writes anything. FK_W4A16_PDL=0 turns the attribute off.
bool pdl_enabled() {
  static const bool enabled = [] {
    const char* value = std::getenv("FK_W4A16_PDL");
    return value == nullptr || std::atoi(value) != 0;
  }();
  return enabled;
}

template <class Params>
cudaError_t launch_kernel(void (*kernel)(Params), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, const Params& params, int cluster_size = 1) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2]{};
  unsigned count = 0;
  if (pdl_enabled()) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  if (cluster_size > 1) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = static_cast<unsigned>(cluster_size);
    attributes[count].val.clusterDim.y = 1;
    attributes[count].val.clusterDim.z = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  return cudaLaunchKernelEx(&config, kernel, params);
}

template <class E>
using UnpackModeFor = std::conditional_t<std::is_same<E, BF16>::value, UnpackBF16, UnpackF16>;

template <int G, int M_TILE, class E>
int launch_stream(const GemvParams& params, const Plan& plan, int max_smem, cudaStream_t stream) {
  auto kernel = w4a16_gemv_stream_kernel<G, M_TILE, UnpackModeFor<E>>;
  static std::once_flag optin_flags[kMaxDevices];
  FK_TRY(ensure_smem_optin(kernel, optin_flags, plan.smem_bytes, max_smem));
  const dim3 grid(static_cast<unsigned>(plan.grid_x), static_cast<unsigned>(plan.row_tiles), 1);
  FK_TRY_CUDA(launch_kernel(kernel, grid, dim3(plan.warps * 32), plan.smem_bytes, stream, params));
  return FK_W4A16_OK;
}

template <int G, int M_TILE, class E>
int launch_cluster(const GemvParams& params, const Plan& plan, int max_smem, cudaStream_t stream) {
  auto kernel = w4a16_gemv_cluster_kernel<G, M_TILE, UnpackModeFor<E>>;
  static std::once_flag optin_flags[kMaxDevices];
  FK_TRY(ensure_smem_optin(kernel, optin_flags, plan.smem_bytes, max_smem));
  const dim3 grid(static_cast<unsigned>(plan.grid_x), static_cast<unsigned>(plan.row_tiles), 1);
  FK_TRY_CUDA(launch_kernel(kernel, grid, dim3(plan.warps * 32), plan.smem_bytes, stream, params,
                            plan.cluster_size));
  return FK_W4A16_OK;
}

template <int G, int M_TILE, class E>
int launch_chain(const ChainParams& params, int grid, int warps, size_t smem_bytes, int max_smem,
                 cudaStream_t stream) {
  auto kernel = w4a16_gemv_chain_kernel<G, M_TILE, UnpackModeFor<E>>;
  static std::once_flag optin_flags[kMaxDevices];
  FK_TRY(ensure_smem_optin(kernel, optin_flags, smem_bytes, max_smem));
  FK_TRY_CUDA(launch_kernel(kernel, dim3(static_cast<unsigned>(grid)), dim3(warps * 32), smem_bytes, stream,
                            params));
  return FK_W4A16_OK;
}

template <int G, int M_TILE, class E>
int launch_wmma(const GemvParams& params, const Plan& plan, int max_smem, cudaStream_t stream) {
  if constexpr (M_TILE <= 2) {
    auto kernel = w4a16_gemv_wmma_kernel<G, M_TILE, UnpackModeFor<E>>;
    static std::once_flag optin_flags[kMaxDevices];
    FK_TRY(ensure_smem_optin(kernel, optin_flags, plan.smem_bytes, max_smem));
    const dim3 grid(static_cast<unsigned>(plan.grid_x), static_cast<unsigned>(plan.row_tiles), 1);
    FK_TRY_CUDA(launch_kernel(kernel, grid, dim3(plan.warps * 32), plan.smem_bytes, stream, params));
    return FK_W4A16_OK;
  } else {
    (void)params; (void)plan; (void)max_smem; (void)stream;
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "the warp-level MMA kernel takes batches of 1 and 2");
  }
}

template <int G, int MT, class E>
int launch_mma(const GemvParams& params, const Plan& plan, uint8_t* staged, int max_smem,
               cudaStream_t stream) {
  using Mode = UnpackModeFor<E>;
  auto kernel = w4a16_gemm_mma_kernel<G, MT, Mode>;
  static std::once_flag optin_flags[kMaxDevices];
  FK_TRY(ensure_smem_optin(kernel, optin_flags, plan.smem_bytes, max_smem));
  // Prepass, then the GEMM, both with programmatic serialisation (each waits inside the kernel).
  StageMmaParams stage{};
  stage.act = static_cast<const uint16_t*>(params.act);
  stage.staged = staged;
  stage.batch = params.m;
  stage.k = params.k;
  stage.num_groups = params.num_groups;
  stage.mt = MT;
  stage.total_items = static_cast<long long>(plan.row_tiles) * params.num_groups * MT;
  FK_TRY_CUDA(launch_kernel(stage_activations_mma_kernel<G, Mode>,
                            dim3(static_cast<unsigned>((stage.total_items + 3) / 4)), dim3(128), 0,
                            stream, stage));
  MmaParams mma_params{};
  mma_params.base = params;
  mma_params.staged = staged;
  const dim3 grid(static_cast<unsigned>(plan.grid_x), static_cast<unsigned>(plan.row_tiles), 1);
  FK_TRY_CUDA(launch_kernel(kernel, grid, dim3(plan.warps * 64), plan.smem_bytes, stream, mma_params));
  return FK_W4A16_OK;
}

template <class E, class Fn>
int for_group_mt(int group_size, int mt, Fn&& fn) {
  switch (group_size) {
    case 32: return mt == 8 ? fn(std::integral_constant<int, 32>{}, std::integral_constant<int, 8>{}, E{})
                            : fn(std::integral_constant<int, 32>{}, std::integral_constant<int, 16>{}, E{});
    case 64: return mt == 8 ? fn(std::integral_constant<int, 64>{}, std::integral_constant<int, 8>{}, E{})
                            : fn(std::integral_constant<int, 64>{}, std::integral_constant<int, 16>{}, E{});
    default: return mt == 8 ? fn(std::integral_constant<int, 128>{}, std::integral_constant<int, 8>{}, E{})
                            : fn(std::integral_constant<int, 128>{}, std::integral_constant<int, 16>{}, E{});
  }
}

template <int G, int M_TILE, class E>
int launch_split_k(const SplitKParams& params, int row_tiles, int max_smem, cudaStream_t stream) {
  auto kernel = w4a16_split_k_kernel<G, M_TILE, UnpackModeFor<E>>;
  constexpr int kWarps = 4;
  const int stage_bytes = packet_stride(G);
  const size_t smem = (((kWarps * params.base.stages * 8) + 127) & ~127) +
                      (static_cast<size_t>(kWarps) * params.base.stages * stage_bytes);
  static std::once_flag optin_flags[kMaxDevices];
  FK_TRY(ensure_smem_optin(kernel, optin_flags, smem, max_smem));
  const dim3 grid(static_cast<unsigned>(params.base.num_tiles), static_cast<unsigned>(row_tiles),
                  static_cast<unsigned>(params.slices));
  FK_TRY_CUDA(launch_kernel(kernel, grid, dim3(kWarps * 32), smem, stream, params));
  return FK_W4A16_OK;
}

// Compile-time fan-out over (group size, rows per pass, element type).
template <int G, class E, class Fn>
int for_m_tile(int m_tile, Fn&& fn) {
  switch (m_tile) {
    case 1: return fn(std::integral_constant<int, G>{}, std::integral_constant<int, 1>{}, E{});
    case 2: return fn(std::integral_constant<int, G>{}, std::integral_constant<int, 2>{}, E{});
    default: return fn(std::integral_constant<int, G>{}, std::integral_constant<int, 4>{}, E{});
  }
}
template <class E, class Fn>
int for_group(int group_size, int m_tile, Fn&& fn) {
  switch (group_size) {
    case 32: return for_m_tile<32, E>(m_tile, fn);
    case 64: return for_m_tile<64, E>(m_tile, fn);
    default: return for_m_tile<128, E>(m_tile, fn);
  }
}
template <class Fn>
int dispatch(int group_size, int m_tile, int dtype, Fn&& fn) {
  return dtype == FK_W4A16_DTYPE_BF16 ? for_group<BF16>(group_size, m_tile, fn)
                                      : for_group<F16>(group_size, m_tile, fn);
}

int grid_for(long long items, int threads, int sm_count) {
  const long long blocks = (items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count) * 32;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

cublasLtHandle_t g_lt_handle = nullptr;
std::once_flag g_lt_once;

}  // namespace
}  // namespace fk_w4a16

using namespace fk_w4a16;

extern "C" {

const char* fk_w4a16_last_error(void) { return t_last_error.c_str(); }
const char* fk_w4a16_version(void) { return FK_W4A16_VERSION; }
const char* fk_w4a16_cuda_arch(void) { return "100a"; }

int fk_w4a16_packet_stride_bytes(int group_size) {
  if (!group_supported(group_size)) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "group_size must be 32, 64 or 128");
  }
  return packet_stride(group_size);
}

int fk_w4a16_set_launch_config(int warps_per_cta, int stages, int ctas) {
  // ctas * warps stays below 4096: the kernels' run arithmetic divides by it with a 40-bit reciprocal
  if (warps_per_cta < 0 || warps_per_cta > kMaxWarps || stages < 0 || stages > kMaxStages ||
      ctas < 0 || ctas > 256) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "launch config out of range");
  }
  (void)launch_config();  // settle the environment defaults first so they cannot override this
  g_config.warps = warps_per_cta;
  g_config.stages = stages;
  g_config.ctas = ctas;
  return FK_W4A16_OK;
}

int fk_w4a16_set_tuning(const char* name, int value) {
  if (name == nullptr) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "name must not be null");
  }
  Tuning& t = tuning();
  const std::string key(name);
  if (key == "mma_min_batch") {
    t.mma_min_batch = value;
  } else if (key == "cluster_min") {
    t.cluster_min = value;
  } else if (key == "cluster_size") {
    t.cluster_size = value;
  } else if (key == "wmma") {
    t.wmma = value;
  } else if (key == "umma_min_batch") {
    t.umma_min_batch = value;
  } else if (key == "cluster") {
    t.cluster = value != 0 ? 1 : 0;
  } else if (key == "peer_wait_ms") {
    if (value <= 0 || value > 10000) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "peer_wait_ms must be between 1 and 10000");
    }
    t.peer_wait_ms = value;
  } else {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "unknown tuning knob: " + key);
  }
  return FK_W4A16_OK;
}

int fk_w4a16_set_variant(int variant) {
  if (variant != FK_W4A16_VARIANT_AUTO && variant != FK_W4A16_VARIANT_TCGEN05 &&
      variant != FK_W4A16_VARIANT_CLASSIC) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "unknown kernel variant");
  }
  g_variant.store(variant, std::memory_order_relaxed);
  return FK_W4A16_OK;
}

int fk_w4a16_pack_packets(const void* q, const void* alpha, const void* beta, void* packets, int n,
                          int k, int group_size, int packet_stride_bytes, void* stream) {
  FK_TRY(check_dimensions(1, n, k, group_size));
  FK_TRY(check_stride(group_size, packet_stride_bytes));
  FK_TRY(check_pointer(q, "q", 16));
  FK_TRY(check_pointer(alpha, "alpha", 2));
  FK_TRY(check_pointer(beta, "beta", 2));
  FK_TRY(check_pointer(packets, "packets", 16));
  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));
  const int num_groups = k / group_size;
  const long long total = static_cast<long long>(n / kTileCols) * num_groups;
  const long long cap = static_cast<long long>(info->sm_count) * 16;
  const int grid = static_cast<int>(total < cap ? total : cap);
  auto* s = static_cast<cudaStream_t>(stream);
  auto* qp = static_cast<const uint8_t*>(q);
  auto* ap = static_cast<const uint16_t*>(alpha);
  auto* bp = static_cast<const uint16_t*>(beta);
  auto* pp = static_cast<uint8_t*>(packets);
  switch (group_size) {
    case 32: pack_packets_kernel<32><<<grid, 128, 0, s>>>(qp, ap, bp, pp, k, num_groups, total); break;
    case 64: pack_packets_kernel<64><<<grid, 128, 0, s>>>(qp, ap, bp, pp, k, num_groups, total); break;
    default: pack_packets_kernel<128><<<grid, 128, 0, s>>>(qp, ap, bp, pp, k, num_groups, total); break;
  }
  FK_TRY_CUDA(cudaGetLastError());
  return FK_W4A16_OK;
}

int fk_w4a16_group_sums(const void* activations, float* sums, int batch, int k, int group_size,
                        int dtype, void* stream) {
  FK_TRY(check_group_and_k(batch, k, group_size));
  FK_TRY(check_dtype(dtype));
  FK_TRY(check_pointer(activations, "activations", 4));
  FK_TRY(check_pointer(sums, "sums", 4));
  const int num_groups = k / group_size;
  const long long total = static_cast<long long>(batch) * num_groups;
  const int grid = static_cast<int>((total + 3) / 4);
  auto* s = static_cast<cudaStream_t>(stream);
  auto* act = static_cast<const uint16_t*>(activations);
  const int rc = dispatch(group_size, 1, dtype, [&](auto g, auto, auto e) {
    using E = decltype(e);
    group_sums_kernel<decltype(g)::value, E><<<grid, 128, 0, s>>>(act, sums, k, num_groups, total);
    return FK_W4A16_OK;
  });
  FK_TRY(rc);
  FK_TRY_CUDA(cudaGetLastError());
  return FK_W4A16_OK;
}

size_t fk_w4a16_workspace_bytes(int batch, int n, int k, int group_size) {
  if (check_dimensions(batch, n, k, group_size) != FK_W4A16_OK) {
    return 0;
  }
  DeviceInfo* info = nullptr;
  if (device_info(&info) != FK_W4A16_OK) {
    return 0;
  }
  const Plan plan =
      make_plan(batch, n, k, group_size, info->sm_count, info->max_smem_optin, launch_config());
  const Plan umma_plan =
      make_umma_plan(batch, n, k, group_size, info->sm_count, info->max_smem_optin, launch_config());
  size_t need = workspace_bytes_for(plan);
  need = need > workspace_bytes_for(umma_plan) ? need : workspace_bytes_for(umma_plan);
  return need;
}

int fk_w4a16_describe_plan(int batch, int n, int k, int group_size, int dtype, char* text,
                           size_t capacity) {
  FK_TRY(check_dimensions(batch, n, k, group_size));
  FK_TRY(check_dtype(dtype));
  if (text == nullptr || capacity == 0) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "text must point to a buffer");
  }
  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));
  const bool use_umma = umma_wanted(batch, n, k, group_size);
  const Plan plan =
      use_umma ? make_umma_plan(batch, n, k, group_size, info->sm_count, info->max_smem_optin, launch_config())
               : make_plan(batch, n, k, group_size, info->sm_count, info->max_smem_optin, launch_config(),
                      /*allow_cluster=*/true, /*cuda_cores_only=*/false);
  const char* kernel = plan.umma            ? "w4a16_gemm_umma_kernel"
                       : plan.tensor_cores  ? "w4a16_gemm_mma_kernel"
                       : plan.wmma          ? "w4a16_gemv_wmma_kernel"
                       : plan.cluster_size > 1 ? "w4a16_gemv_cluster_kernel"
                                               : "w4a16_gemv_stream_kernel";
  std::ostringstream oss;
  oss << kernel << "<" << group_size << ", " << plan.m_tile << ", "
      << (dtype == FK_W4A16_DTYPE_BF16 ? "UnpackBF16" : "UnpackF16") << "> grid=" << plan.grid_x << "x"
      << plan.row_tiles << " cluster=" << plan.cluster_size << " warps=" << plan.warps
      << " stages=" << plan.stages << " smem=" << plan.smem_bytes;
  const std::string line = oss.str();
  if (line.size() + 1 > capacity) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "text buffer is too small");
  }
  std::memcpy(text, line.c_str(), line.size() + 1);
  return FK_W4A16_OK;
}

int fk_w4a16_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  FK_TRY(check_pointer(workspace, "workspace", 256));
  if (workspace_bytes < kHeaderBytes) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "workspace is smaller than its fixed header");
  }
  FK_TRY_CUDA(cudaMemsetAsync(workspace, 0, kHeaderBytes, static_cast<cudaStream_t>(stream)));
  return FK_W4A16_OK;
}

namespace {
// `with_exchange_area`: the workspace has the full header (ticket + pair-exchange areas); without
// it -- the library's own static scratch -- the header is the ticket area alone.
// `small_batch_on_cuda_cores`: batches of at most 4 never take the tensor-core plan (whose slots
// and staged activations need more scratch than the static array holds).
int gemv_impl(const fk_w4a16_gemv_args* args, bool with_exchange_area, bool small_batch_on_cuda_cores);
}  // namespace

int fk_w4a16_gemv_ex(const fk_w4a16_gemv_args* args) { return gemv_impl(args, true, false); }

namespace {
int gemv_impl(const fk_w4a16_gemv_args* args, bool with_exchange_area, bool small_batch_on_cuda_cores) {
  if (args == nullptr) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "args must not be null");
  }
  const size_t header_bytes = with_exchange_area ? kHeaderBytes : kTicketBytes;
  const int batch = args->batch;
  const int n = args->n;
  const int k = args->k;
  const int group_size = args->group_size;
  FK_TRY(check_dimensions(batch, n, k, group_size));
  FK_TRY(check_stride(group_size, args->packet_stride_bytes));
  FK_TRY(check_dtype(args->dtype));
  FK_TRY(check_pointer(args->activations, "activations", 16));
  FK_TRY(check_pointer(args->packets, "packets", 16));
  FK_TRY(check_pointer(args->output, "output", args->output_f32 != 0 ? 16 : 8));
  FK_TRY(check_pointer(args->workspace, "workspace", 256));
  if (args->epilogue != FK_W4A16_EPILOGUE_NONE && args->epilogue != FK_W4A16_EPILOGUE_SILU_MUL) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "unknown epilogue");
  }
  const bool gated = args->epilogue == FK_W4A16_EPILOGUE_SILU_MUL;
  if (gated && (n % (2 * kTileCols)) != 0) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                "the SiLU-and-multiply epilogue needs n to be a multiple of 256 ([gate; up] halves of whole tiles)");
  }
  const int n_out = gated ? n / 2 : n;  // columns the caller receives
  const long long out_ld = args->output_ld == 0 ? n_out : args->output_ld;
  if (out_ld < n_out || args->output_col0 < 0 || args->output_col0 + n_out > out_ld ||
      (out_ld % 4) != 0 || (args->output_col0 % 4) != 0) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                "output_ld / output_col0 must place the output columns inside a row, in multiples of 4");
  }
  if (args->num_peers < 0 || args->num_peers > FK_W4A16_MAX_PEERS) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "num_peers must be between 0 and 7");
  }
  for (int peer = 0; peer < args->num_peers; ++peer) {
    FK_TRY(check_pointer(args->peer_outputs[peer], "peer_outputs[i]", args->output_f32 != 0 ? 16 : 8));
    if (args->local_signal != nullptr) {
      FK_TRY(check_pointer(args->peer_signals[peer], "peer_signals[i]", 4));
    }
  }
  if (args->local_signal != nullptr) {
    FK_TRY(check_pointer(args->local_signal, "local_signal", 4));
  }
  if (args->residual != nullptr) {
    FK_TRY(check_pointer(args->residual, "residual", 8));
  }
  if (args->ll_epoch_counter != nullptr) {
    FK_TRY(check_pointer(args->ll_epoch_counter, "ll_epoch_counter", 8));
    if (args->ll_epoch != 0 || args->ll_parity_words < 0 || (args->ll_parity_words % 2) != 0) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                  "with ll_epoch_counter, ll_epoch must be 0 and ll_parity_words a non-negative even number");
    }
  }
  if (args->ll_epoch != 0 || args->ll_epoch_counter != nullptr) {
    if (args->local_signal != nullptr || args->reduce_slots != 0 || gated) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                  "the flag-in-data exchange (ll_epoch) excludes the counter exchange, reduce_slots and the "
                  "SiLU-and-multiply epilogue");
    }
    if (args->ll_slots < 1 || args->ll_slots > FK_W4A16_MAX_PEERS + 1 || args->ll_slot_cols < 1 ||
        (args->ll_slot_cols % 4) != 0) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                  "ll_slots must be between 1 and 8 and ll_slot_cols a positive multiple of 4");
    }
    FK_TRY(check_pointer(args->ll_input, "ll_input", 16));
    FK_TRY(check_pointer(args->ll_output, "ll_output", 2));
    FK_TRY(check_pointer(args->output, "output", 16));
    for (int peer = 0; peer < args->num_peers; ++peer) {
      FK_TRY(check_pointer(args->peer_outputs[peer], "peer_outputs[i]", 16));
    }
  }
  if (args->reduce_slots != 0) {
    if (args->reduce_slots < 0 || args->reduce_slots > FK_W4A16_MAX_PEERS + 1 || args->local_signal == nullptr) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                  "reduce_slots must be between 1 and 8 and needs the exchange counters (local_signal)");
    }
    FK_TRY(check_pointer(args->reduce_input, "reduce_input", 16));
    FK_TRY(check_pointer(args->reduce_output, "reduce_output", 8));
  }

  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));
  // The workspace requirement is that of the packet-stream plan whichever kernel runs, so that
  // fk_w4a16_workspace_bytes() is a safe answer for every option combination.
  const Plan stream_plan = make_plan(batch, n, k, group_size, info->sm_count, info->max_smem_optin,
                                     launch_config(), false, small_batch_on_cuda_cores);
  const bool normalise = args->norm_weight != nullptr;
  if (normalise) {
    FK_TRY(check_pointer(args->norm_weight, "norm_weight", 16));
    if (batch > 4 || !(args->norm_eps >= 0.0f)) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                  "the fused RMSNorm needs batch <= 4 and a non-negative norm_eps");
    }
  }
  // The fused RMSNorm lives in the CUDA-core kernels (stream and cluster).
  const bool use_umma = !normalise && !small_batch_on_cuda_cores && umma_wanted(batch, n, k, group_size);
  const Plan plan =
      use_umma
          ? make_umma_plan(batch, n, k, group_size, info->sm_count, info->max_smem_optin, launch_config())
          : make_plan(batch, n, k, group_size, info->sm_count, info->max_smem_optin, launch_config(),
                      /*allow_cluster=*/true,
                      /*cuda_cores_only=*/normalise || small_batch_on_cuda_cores);
  if (plan.stages < 1) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "launch config does not fit in shared memory");
  }
  if (args->workspace_bytes < workspace_bytes_for(stream_plan, header_bytes) ||
      args->workspace_bytes < workspace_bytes_for(plan, header_bytes)) {
    std::ostringstream oss;
    oss << "workspace_bytes=" << args->workspace_bytes << " is smaller than the required "
        << workspace_bytes_for(stream_plan, header_bytes);
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, oss.str());
  }
  const int num_tiles = n / kTileCols;
  if (static_cast<long long>(plan.row_tiles) * num_tiles > kTicketCapacity - 2) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "n * batch exceeds the ticket area of a workspace");
  }

  GemvParams params{};
#ifdef FK_W4A16_TRACE
  static std::atomic<int> trace_launches{0};
  params.trace_id = trace_launches.fetch_add(1) % kTraceLaunches;
#endif
  params.act = args->activations;
  params.packets = static_cast<const uint8_t*>(args->packets);
  params.out = args->output;
  params.tickets = static_cast<int*>(args->workspace);
  params.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(args->workspace) + header_bytes);
  // Pair exchange: one area of m_tile x 128 64-bit words per boundary between neighbouring CTAs.
  params.exchange = nullptr;
  params.gated = nullptr;
  size_t exchange_bytes = static_cast<size_t>(plan.row_tiles) * static_cast<size_t>(plan.grid_x) *
                          plan.m_tile * kTileCols * sizeof(unsigned long long);
  const size_t gated_bytes =
      gated ? static_cast<size_t>(batch) * (n / 2) * sizeof(unsigned long long) : 0;
  const bool wants_exchange =
      with_exchange_area && !plan.tensor_cores && plan.cluster_size == 1 && plan.m_tile <= 4;
  // (the pipelined tcgen05 kernel finishes split tiles like the packet-stream kernel does)
  if (!wants_exchange || exchange_bytes + gated_bytes > kExchangeBytes) {
    exchange_bytes = 0;  // split tiles take the ticket finish; the area is the epilogue's alone
  }
  if (gated) {
    if (!with_exchange_area || gated_bytes > kExchangeBytes) {
      std::ostringstream oss;
      oss << "the SiLU-and-multiply epilogue needs " << gated_bytes
          << " bytes of the workspace header's exchange area, which holds " << kExchangeBytes
          << " (batch * n / 2 <= " << kExchangeBytes / sizeof(unsigned long long) << ")";
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT, oss.str());
    }
    params.gated = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(args->workspace) +
                                                         kTicketBytes + exchange_bytes);
  }
  if (exchange_bytes > 0) {
    params.exchange = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(args->workspace) +
                                                            kTicketBytes);
  }
  params.status = info->status_word;
  params.out_ld = out_ld;
  params.out_col0 = args->output_col0;
  params.out_f32 = args->output_f32 != 0 ? 1 : 0;
  params.num_peers = args->num_peers;
  for (int peer = 0; peer < args->num_peers; ++peer) {
    params.peer_out[peer] = args->peer_outputs[peer];
    params.peer_signal[peer] = args->peer_signals[peer];
  }
  params.residual = args->residual;
  params.norm_weight = args->norm_weight;
  params.norm_eps = args->norm_eps;
  params.local_signal = args->local_signal;
  params.wait_value = args->wait_value;
  params.peer_wait_ns = static_cast<unsigned long long>(tuning().peer_wait_ms) * 1000000ull;
  params.reduce_input = args->reduce_input;
  params.reduce_output = args->reduce_output;
  params.reduce_slots = args->reduce_slots;
  params.ll_epoch = args->ll_epoch;
  params.ll_epoch_counter = args->ll_epoch_counter;
  params.ll_ticket = args->ll_epoch_counter != nullptr ? args->ll_epoch_counter + 1 : nullptr;
  params.ll_parity_words = args->ll_parity_words;
  params.ll_input = static_cast<const unsigned long long*>(args->ll_input);
  params.ll_output = args->ll_output;
  params.ll_slots = args->ll_slots;
  params.ll_slot_cols = args->ll_slot_cols;
  params.ll_reduce = args->ll_reduce != 0 ? 1 : 0;
  params.m = batch;
  params.n = n;
  params.k = k;
  params.num_groups = k / group_size;
  params.num_tiles = num_tiles;
  params.active_warps = plan.active_warps;
  params.stages = plan.stages;
  params.total_packets = plan.total_packets;
  params.run_base = plan.total_packets / static_cast<uint32_t>(plan.active_warps);
  params.run_rem = plan.total_packets % static_cast<uint32_t>(plan.active_warps);
  params.run_magic = ((uint64_t{1} << 40) / static_cast<uint64_t>(plan.active_warps)) + 1;
  params.run_inv = static_cast<float>(static_cast<double>(plan.active_warps) /
                                      static_cast<double>(plan.total_packets));
  auto* s = static_cast<cudaStream_t>(args->stream);
  const int max_smem = info->max_smem_optin;
  if (plan.umma) {
    if (plan.smem_bytes > static_cast<size_t>(max_smem)) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "launch needs more shared memory than the device has");
    }
    UmmaLaunch launch{};
    launch.group_size = group_size;
    launch.rows = plan.m_tile;
    launch.bf16 = args->dtype == FK_W4A16_DTYPE_BF16;
    launch.grid_x = plan.grid_x;
    launch.row_tiles = plan.row_tiles;
    launch.smem_bytes = plan.smem_bytes;
    launch.max_smem = max_smem;
    launch.programmatic = pdl_enabled();
    launch.stream = s;
    FK_TRY_CUDA(launch_umma_kernel(params, launch));
    return FK_W4A16_OK;
  }
  if (plan.tensor_cores) {
    uint8_t* staged = static_cast<uint8_t*>(args->workspace) + header_bytes +
                      ((plan.scratch_bytes + 255) & ~size_t{255});
    auto run = [&](auto g, auto mt, auto e) {
      return launch_mma<decltype(g)::value, decltype(mt)::value, decltype(e)>(params, plan, staged,
                                                                               max_smem, s);
    };
    return args->dtype == FK_W4A16_DTYPE_BF16 ? for_group_mt<BF16>(group_size, plan.m_tile, run)
                                              : for_group_mt<F16>(group_size, plan.m_tile, run);
  }
  if (plan.wmma) {
    return dispatch(group_size, plan.m_tile, args->dtype, [&](auto g, auto mt, auto e) {
      return launch_wmma<decltype(g)::value, decltype(mt)::value, decltype(e)>(params, plan, max_smem, s);
    });
  }
  if (plan.cluster_size > 1) {
    return dispatch(group_size, plan.m_tile, args->dtype, [&](auto g, auto mt, auto e) {
      return launch_cluster<decltype(g)::value, decltype(mt)::value, decltype(e)>(params, plan,
                                                                                    max_smem, s);
    });
  }
  return dispatch(group_size, plan.m_tile, args->dtype, [&](auto g, auto mt, auto e) {
    return launch_stream<decltype(g)::value, decltype(mt)::value, decltype(e)>(params, plan,
                                                                                 max_smem, s);
  });
}
}  // namespace

int fk_w4a16_gemv(const void* activations, const void* packets, void* output, void* workspace,
                  size_t workspace_bytes, int batch, int n, int k, int group_size,
                  int packet_stride_bytes, int dtype, void* stream) {
  fk_w4a16_gemv_args args{};
  args.activations = activations;
  args.packets = packets;
  args.output = output;
  args.workspace = workspace;
  args.workspace_bytes = workspace_bytes;
  args.batch = batch;
  args.n = n;
  args.k = k;
  args.group_size = group_size;
  args.packet_stride_bytes = packet_stride_bytes;
  args.dtype = dtype;
  args.stream = stream;
  return fk_w4a16_gemv_ex(&args);
}

namespace {

// Device-side address of `ptr` if it is mapped (pinned) host memory, else nullptr. The driver
// query costs about a microsecond, as much as a launch, so answers are remembered per calling
// thread in a small direct-mapped table keyed by the host address (a registration is stable for
// as long as the memory stays pinned; a caller that unpins a buffer and pins other memory at the
// same address with a different mapping must not expect the zero-copy path to notice).
void* mapped_host_address(const void* ptr) {
  struct Entry {
    const void* host = nullptr;
    void* device = nullptr;
  };
  constexpr int kEntries = 64;
  thread_local Entry table[kEntries];
  Entry& entry = table[(reinterpret_cast<uintptr_t>(ptr) >> 6) % kEntries];
  if (entry.host == ptr && ptr != nullptr) {
    return entry.device;
  }
  cudaPointerAttributes attrs{};
  if (cudaPointerGetAttributes(&attrs, ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  void* device = attrs.type == cudaMemoryTypeHost ? attrs.devicePointer : nullptr;
  if (device != nullptr) {
    entry.host = ptr;
    entry.device = device;
  }
  return device;
}

bool host_zero_copy_enabled() {
  static const bool enabled = [] {
    const char* value = std::getenv("FK_W4A16_HOST_ZERO_COPY");
    return value == nullptr || std::atoi(value) != 0;
  }();
  return enabled;
}

}  // namespace

int fk_w4a16_gemv_host(const void* host_activations, const void* packets, void* host_output,
                       void* device_activations, void* device_output, void* workspace,
                       size_t workspace_bytes, int batch, int n, int k, int group_size,
                       int packet_stride_bytes, int dtype, void* stream) {
  FK_TRY(check_dimensions(batch, n, k, group_size));
  FK_TRY(check_pointer(host_activations, "host_activations", 2));
  FK_TRY(check_pointer(host_output, "host_output", 2));
  FK_TRY(check_pointer(device_activations, "device_activations", 16));
  FK_TRY(check_pointer(device_output, "device_output", 8));
  auto* s = static_cast<cudaStream_t>(stream);
  const size_t act_bytes = static_cast<size_t>(batch) * k * 2;
  const size_t out_bytes = static_cast<size_t>(batch) * n * 2;

  // Pinned, mapped host buffers: no copy engine at all. A small kernel pulls the activations over
  // PCIe into the staging buffer, and the GEMV stores every finished tile to the host buffer as
  // well as to the device one, so a call costs two launches instead of three stream operations on
  // two engines with a semaphore between each.
  void* act_mapped = nullptr;
  void* out_mapped = nullptr;
  if (host_zero_copy_enabled() && (reinterpret_cast<uintptr_t>(host_activations) % 16) == 0 &&
      (reinterpret_cast<uintptr_t>(host_output) % 8) == 0) {
    act_mapped = mapped_host_address(host_activations);
    out_mapped = act_mapped != nullptr ? mapped_host_address(host_output) : nullptr;
  }
  if (act_mapped != nullptr && out_mapped != nullptr) {
    StageHostParams stage{};
    stage.src = static_cast<const uint4*>(act_mapped);
    stage.dst = static_cast<uint4*>(device_activations);
    stage.count = static_cast<int>(act_bytes / 16);
    const unsigned blocks = static_cast<unsigned>((stage.count + 255) / 256);
    FK_TRY_CUDA(launch_kernel(stage_host_activations_kernel, dim3(blocks), dim3(256), 0, s, stage));
    fk_w4a16_gemv_args args{};
    args.activations = device_activations;
    args.packets = packets;
    args.output = device_output;
    args.workspace = workspace;
    args.workspace_bytes = workspace_bytes;
    args.batch = batch;
    args.n = n;
    args.k = k;
    args.group_size = group_size;
    args.packet_stride_bytes = packet_stride_bytes;
    args.dtype = dtype;
    args.num_peers = 1;
    args.peer_outputs[0] = out_mapped;
    args.stream = stream;
    return fk_w4a16_gemv_ex(&args);
  }

  FK_TRY_CUDA(cudaMemcpyAsync(device_activations, host_activations, act_bytes,
                              cudaMemcpyHostToDevice, s));
  FK_TRY(fk_w4a16_gemv(device_activations, packets, device_output, workspace, workspace_bytes, batch,
                       n, k, group_size, packet_stride_bytes, dtype, stream));
  FK_TRY_CUDA(cudaMemcpyAsync(host_output, device_output, out_bytes, cudaMemcpyDeviceToHost, s));
  return FK_W4A16_OK;
}

int fk_w4a16_gemv_static(const void* activations, const void* packets, void* output, int batch,
                         int n, int k, int group_size, int packet_stride_bytes, int dtype,
                         void* stream) {
  FK_TRY(check_dimensions(batch, n, k, group_size));
  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));

  // Once per device, with that device current: the device address of the static array. A failed
  // lookup is not remembered, so a first call that came at a bad moment (during stream capture)
  // does not poison the device for the rest of the process.
  static void* scratch_address[kMaxDevices] = {};
  static std::mutex scratch_lock;
  int device = 0;
  FK_TRY_CUDA(cudaGetDevice(&device));
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(scratch_lock);
    if (scratch_address[device] == nullptr) {
      void* address = nullptr;
      const cudaError_t lookup = cudaGetSymbolAddress(&address, g_static_scratch);
      if (lookup != cudaSuccess || address == nullptr) {
        return fail(FK_W4A16_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch) failed: ") +
                                           cudaGetErrorString(lookup));
      }
      scratch_address[device] = address;
    }
    scratch = scratch_address[device];
  }

  // Batches of at most 4 stay on the CUDA-core kernels here (their scratch always fits); the plan
  // below is the one gemv_impl makes with the same flag.
  const Plan plan = make_plan(batch, n, k, group_size, info->sm_count, info->max_smem_optin,
                              launch_config(), /*allow_cluster=*/false, /*cuda_cores_only=*/true);
  const size_t need = workspace_bytes_for(plan, kTicketBytes);
  if (need > static_cast<size_t>(FK_W4A16_STATIC_SCRATCH_BYTES)) {
    std::ostringstream oss;
    oss << "this problem needs " << need << " bytes of scratch but the static array holds "
        << FK_W4A16_STATIC_SCRATCH_BYTES << "; use fk_w4a16_gemv with a caller-owned workspace";
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, oss.str());
  }
  // The tickets this call will use must start at zero whatever an earlier call left behind.
  const size_t ticket_bytes =
      static_cast<size_t>(plan.row_tiles) * static_cast<size_t>(n / kTileCols) * sizeof(int);
  if (ticket_bytes > kTicketBytes) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "n * batch exceeds the ticket area of a workspace");
  }
  FK_TRY_CUDA(cudaMemsetAsync(scratch, 0, ticket_bytes, static_cast<cudaStream_t>(stream)));
  fk_w4a16_gemv_args args{};
  args.activations = activations;
  args.packets = packets;
  args.output = output;
  args.workspace = scratch;
  args.workspace_bytes = FK_W4A16_STATIC_SCRATCH_BYTES;
  args.batch = batch;
  args.n = n;
  args.k = k;
  args.group_size = group_size;
  args.packet_stride_bytes = packet_stride_bytes;
  args.dtype = dtype;
  args.stream = stream;
  return gemv_impl(&args, /*with_exchange_area=*/false, /*small_batch_on_cuda_cores=*/true);
}

namespace {
// Warps per CTA and ring depth of the chain kernel for (group size, rows per pass): as many warps
// as fit with a two-deep ring each, then the deepest ring (at most 4) that still fits.
void chain_geometry(int group_size, int m_tile, int max_smem, int* warps_out, int* stages_out) {
  const int per_warp = (2 * packet_stride(group_size)) + (2 * m_tile * kTileCols * 4) +
                       (m_tile * group_size * 2) + 16;
  int warps = (max_smem - 256) / per_warp;
  warps = warps > kMaxWarps ? kMaxWarps : (warps < 1 ? 1 : warps);
  int stages = 2;
  for (int candidate = 4; candidate >= 2; --candidate) {
    if (stream_smem_plan(warps, candidate, group_size, m_tile).total <= static_cast<uint32_t>(max_smem)) {
      stages = candidate;
      break;
    }
  }
  *warps_out = warps;
  *stages_out = stages;
}
}  // namespace

size_t fk_w4a16_chain_workspace_bytes(int batch, int group_size) {
  if (batch <= 0 || batch > 4 || !group_supported(group_size)) {
    return 0;
  }
  DeviceInfo* info = nullptr;
  if (device_info(&info) != FK_W4A16_OK) {
    return 0;
  }
  const size_t scratch = static_cast<size_t>(info->sm_count) * 2 * (m_tile_for_batch(batch) * kTileCols) * sizeof(float);
  return kHeaderBytes + ((scratch + 255) & ~size_t{255});
}

int fk_w4a16_gemv_chain(const fk_w4a16_chain_step* steps, int count, void* workspace,
                        size_t workspace_bytes, int batch, int group_size, int packet_stride_bytes,
                        int dtype, void* stream) {
  if (steps == nullptr || count < 1 || count > FK_W4A16_MAX_CHAIN_STEPS) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "a chain has between 1 and 8 steps");
  }
  if (batch > 4) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "a chain takes batches of at most 4");
  }
  FK_TRY(check_dtype(dtype));
  FK_TRY(check_pointer(workspace, "workspace", 256));
  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));
  for (int i = 0; i < count; ++i) {
    FK_TRY(check_dimensions(batch, steps[i].n, steps[i].k, group_size));
  }
  FK_TRY(check_stride(group_size, packet_stride_bytes));
  const size_t need = fk_w4a16_chain_workspace_bytes(batch, group_size);
  if (workspace_bytes < need) {
    std::ostringstream oss;
    oss << "workspace_bytes=" << workspace_bytes << " is smaller than the required " << need;
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, oss.str());
  }
  const int m_tile = m_tile_for_batch(batch);
  int warps = 0;
  int stages = 0;
  chain_geometry(group_size, m_tile, info->max_smem_optin, &warps, &stages);
  const int grid = info->sm_count;
  const size_t smem_bytes = stream_smem_plan(warps, stages, group_size, m_tile).total;

  ChainParams chain{};
  chain.count = count;
  chain.barrier = reinterpret_cast<unsigned int*>(static_cast<int*>(workspace) + (kTicketCapacity - 2));
  chain.exit_count = reinterpret_cast<unsigned int*>(static_cast<int*>(workspace) + (kTicketCapacity - 1));
  chain.barrier_wait_ns = static_cast<unsigned long long>(tuning().peer_wait_ms) * 1000000ull;
  const size_t exchange_bytes =
      static_cast<size_t>(grid) * m_tile * kTileCols * sizeof(unsigned long long);
  for (int i = 0; i < count; ++i) {
    const fk_w4a16_chain_step& step = steps[i];
    FK_TRY(check_pointer(step.activations, "activations", 16));
    FK_TRY(check_pointer(step.packets, "packets", 16));
    FK_TRY(check_pointer(step.output, "output", 8));
    if (step.epilogue != FK_W4A16_EPILOGUE_NONE && step.epilogue != FK_W4A16_EPILOGUE_SILU_MUL) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "unknown epilogue");
    }
    const bool gated = step.epilogue == FK_W4A16_EPILOGUE_SILU_MUL;
    if (gated && (step.n % (2 * kTileCols)) != 0) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                  "the SiLU-and-multiply epilogue needs n to be a multiple of 256 ([gate; up] halves of whole tiles)");
    }
    const size_t gated_bytes = gated ? static_cast<size_t>(batch) * (step.n / 2) * sizeof(unsigned long long) : 0;
    if (exchange_bytes + gated_bytes > kExchangeBytes) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                  "the SiLU-and-multiply epilogue of this step does not fit the workspace header's exchange area");
    }
    if (step.residual != nullptr) {
      FK_TRY(check_pointer(step.residual, "residual", 8));
    }
    if (step.norm_weight != nullptr) {
      FK_TRY(check_pointer(step.norm_weight, "norm_weight", 16));
      if (!(step.norm_eps >= 0.0f)) {
        return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "the fused RMSNorm needs a non-negative norm_eps");
      }
    }
    const int num_tiles = step.n / kTileCols;
    if (num_tiles > kTicketCapacity - 2) {
      return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "n exceeds the ticket area of a workspace");
    }
    const long long total_packets = static_cast<long long>(num_tiles) * (step.k / group_size);
    long long workers = static_cast<long long>(grid) * warps;
    workers = workers > total_packets ? total_packets : workers;

    GemvParams& params = chain.step[i];
    params.act = step.activations;
    params.packets = static_cast<const uint8_t*>(step.packets);
    params.out = step.output;
    params.tickets = static_cast<int*>(workspace);
    params.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kHeaderBytes);
    params.exchange = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(workspace) + kTicketBytes);
    params.gated = gated ? reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(workspace) + kTicketBytes +
                                                                 exchange_bytes)
                         : nullptr;
    params.status = info->status_word;
    params.out_ld = gated ? step.n / 2 : step.n;
    params.out_col0 = 0;
    params.out_f32 = 0;
    params.num_peers = 0;
    params.residual = step.residual;
    params.norm_weight = step.norm_weight;
    params.norm_eps = step.norm_eps;
    params.local_signal = nullptr;
    params.m = batch;
    params.n = step.n;
    params.k = step.k;
    params.num_groups = step.k / group_size;
    params.num_tiles = num_tiles;
    params.active_warps = static_cast<int>(workers);
    params.stages = stages;
    params.total_packets = static_cast<uint32_t>(total_packets);
    params.run_base = params.total_packets / static_cast<uint32_t>(workers);
    params.run_rem = params.total_packets % static_cast<uint32_t>(workers);
    params.run_magic = ((uint64_t{1} << 40) / static_cast<uint64_t>(workers)) + 1;
    params.run_inv = static_cast<float>(static_cast<double>(workers) / static_cast<double>(total_packets));
  }
  auto* s = static_cast<cudaStream_t>(stream);
  return dispatch(group_size, m_tile, dtype, [&](auto g, auto mt, auto e) {
    return launch_chain<decltype(g)::value, decltype(mt)::value, decltype(e)>(chain, grid, warps, smem_bytes,
                                                                               info->max_smem_optin, s);
  });
}

int fk_w4a16_gemv_split_k(const void* activations, const void* packets, float* partials, int batch,
                          int n, int k, int group_size, int packet_stride_bytes,
                          int split_k_slices, int dtype, void* stream) {
  FK_TRY(check_dimensions(batch, n, k, group_size));
  FK_TRY(check_stride(group_size, packet_stride_bytes));
  FK_TRY(check_dtype(dtype));
  if (split_k_slices <= 1) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "split_k_slices must be greater than 1");
  }
  const int num_groups = k / group_size;
  if (split_k_slices > num_groups) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                "split_k_slices must not exceed the number of groups");
  }
  FK_TRY(check_pointer(activations, "activations", 16));
  FK_TRY(check_pointer(packets, "packets", 16));
  FK_TRY(check_pointer(partials, "partials", 4));
  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));

  const int m_tile = m_tile_for_batch(batch);
  SplitKParams params{};
  params.base.act = activations;
  params.base.packets = static_cast<const uint8_t*>(packets);
  params.base.status = info->status_word;
  params.base.m = batch;
  params.base.n = n;
  params.base.k = k;
  params.base.num_groups = num_groups;
  params.base.num_tiles = n / kTileCols;
  params.base.stages = 2;
  params.base.total_packets = static_cast<uint32_t>(params.base.num_tiles) * num_groups;
  params.partials = partials;
  params.slices = split_k_slices;
  params.groups_per_slice = (num_groups + split_k_slices - 1) / split_k_slices;
  const int row_tiles = (batch + m_tile - 1) / m_tile;
  auto* s = static_cast<cudaStream_t>(stream);
  const int max_smem = info->max_smem_optin;
  return dispatch(group_size, m_tile, dtype, [&](auto g, auto mt, auto e) {
    return launch_split_k<decltype(g)::value, decltype(mt)::value, decltype(e)>(params, row_tiles,
                                                                                  max_smem, s);
  });
}

int fk_w4a16_reduce_partials(const float* partials, void* output, int batch, int n,
                             int split_k_slices, int dtype, void* stream) {
  if (batch <= 0 || n <= 0 || split_k_slices <= 1) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT,
                "batch, n, and split_k_slices must be positive with split_k_slices > 1");
  }
  FK_TRY(check_dtype(dtype));
  FK_TRY(check_pointer(partials, "partials", 4));
  FK_TRY(check_pointer(output, "output", 2));
  const long long total = static_cast<long long>(batch) * n;
  const int grid = static_cast<int>((total + 255) / 256);
  auto* s = static_cast<cudaStream_t>(stream);
  auto* out = static_cast<uint16_t*>(output);
  if (dtype == FK_W4A16_DTYPE_BF16) {
    reduce_partials_kernel<BF16><<<grid, 256, 0, s>>>(partials, out, total, split_k_slices);
  } else {
    reduce_partials_kernel<F16><<<grid, 256, 0, s>>>(partials, out, total, split_k_slices);
  }
  FK_TRY_CUDA(cudaGetLastError());
  return FK_W4A16_OK;
}

int fk_w4a16_dequant_rowmajor(const void* q, const void* alpha, const void* beta, void* weight,
                              int n, int k, int group_size, int dtype, void* stream) {
  FK_TRY(check_dimensions(1, n, k, group_size));
  FK_TRY(check_dtype(dtype));
  FK_TRY(check_pointer(q, "q", 4));
  FK_TRY(check_pointer(alpha, "alpha", 2));
  FK_TRY(check_pointer(beta, "beta", 2));
  FK_TRY(check_pointer(weight, "weight", 16));
  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));
  const long long total_words = static_cast<long long>(n) * (k / 8);
  const int grid = grid_for(total_words, 256, info->sm_count);
  auto* s = static_cast<cudaStream_t>(stream);
  const int rc = dispatch(group_size, 1, dtype, [&](auto g, auto, auto e) {
    dequant_rowmajor_kernel<decltype(g)::value, decltype(e)><<<grid, 256, 0, s>>>(
        static_cast<const uint8_t*>(q), static_cast<const uint16_t*>(alpha),
        static_cast<const uint16_t*>(beta), static_cast<uint16_t*>(weight), total_words, k,
        k / group_size);
    return FK_W4A16_OK;
  });
  FK_TRY(rc);
  FK_TRY_CUDA(cudaGetLastError());
  return FK_W4A16_OK;
}

int fk_w4a16_dequant_packets(const void* packets, void* weight, int n, int k, int group_size,
                             int packet_stride_bytes, int dtype, void* stream) {
  FK_TRY(check_dimensions(1, n, k, group_size));
  FK_TRY(check_stride(group_size, packet_stride_bytes));
  FK_TRY(check_dtype(dtype));
  FK_TRY(check_pointer(packets, "packets", 4));
  FK_TRY(check_pointer(weight, "weight", 16));
  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));
  const long long total_words = static_cast<long long>(n) * (k / 8);
  const int grid = grid_for(total_words, 256, info->sm_count);
  auto* s = static_cast<cudaStream_t>(stream);
  const int rc = dispatch(group_size, 1, dtype, [&](auto g, auto, auto e) {
    dequant_packets_kernel<decltype(g)::value, decltype(e)><<<grid, 256, 0, s>>>(
        static_cast<const uint8_t*>(packets), static_cast<uint16_t*>(weight), total_words, k,
        k / group_size);
    return FK_W4A16_OK;
  });
  FK_TRY(rc);
  FK_TRY_CUDA(cudaGetLastError());
  return FK_W4A16_OK;
}

int fk_w4a16_cublaslt_matmul(const void* activations, const void* weight, void* output,
                             void* lt_workspace, size_t lt_workspace_bytes, int batch, int n,
                             int k, int dtype, void* stream) {
  if (batch <= 0 || n <= 0 || k <= 0) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "batch, n, and k must be positive");
  }
  FK_TRY(check_dtype(dtype));
  FK_TRY(check_pointer(activations, "activations", 2));
  FK_TRY(check_pointer(weight, "weight", 2));
  FK_TRY(check_pointer(output, "output", 2));

  cublasStatus_t create_status = CUBLAS_STATUS_SUCCESS;
  std::call_once(g_lt_once, [&] { create_status = cublasLtCreate(&g_lt_handle); });
  if (create_status != CUBLAS_STATUS_SUCCESS || g_lt_handle == nullptr) {
    return fail(FK_W4A16_ERR_CUDA, "cublasLtCreate failed");
  }

  // Row-major C[batch, n] = A[batch, k] . B[n, k]^T is, in cuBLAS's column-major terms,
  // C^T[n, batch] = op_T(B as [k, n], ld k) . (A as [k, batch], ld k).
  const cudaDataType_t type = dtype == FK_W4A16_DTYPE_BF16 ? CUDA_R_16BF : CUDA_R_16F;
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t w_layout = nullptr;
  cublasLtMatrixLayout_t a_layout = nullptr;
  cublasLtMatrixLayout_t c_layout = nullptr;
  cublasLtMatmulPreference_t pref = nullptr;
  int rc = FK_W4A16_OK;
  auto cleanup = [&] {
    if (pref != nullptr) cublasLtMatmulPreferenceDestroy(pref);
    if (c_layout != nullptr) cublasLtMatrixLayoutDestroy(c_layout);
    if (a_layout != nullptr) cublasLtMatrixLayoutDestroy(a_layout);
    if (w_layout != nullptr) cublasLtMatrixLayoutDestroy(w_layout);
    if (op != nullptr) cublasLtMatmulDescDestroy(op);
  };
  auto body = [&]() -> int {
    const cublasOperation_t transpose = CUBLAS_OP_T;
    FK_TRY_CUBLAS(cublasLtMatmulDescCreate(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F));
    FK_TRY_CUBLAS(cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSA, &transpose,
                                                 sizeof(transpose)));
    FK_TRY_CUBLAS(cublasLtMatrixLayoutCreate(&w_layout, type, k, n, k));
    FK_TRY_CUBLAS(cublasLtMatrixLayoutCreate(&a_layout, type, k, batch, k));
    FK_TRY_CUBLAS(cublasLtMatrixLayoutCreate(&c_layout, type, n, batch, n));
    FK_TRY_CUBLAS(cublasLtMatmulPreferenceCreate(&pref));
    size_t ws_bytes = lt_workspace == nullptr ? 0 : lt_workspace_bytes;
    void* ws = lt_workspace;
    cublasLtMatmulHeuristicResult_t heuristic{};
    int found = 0;
    for (int attempt = 0; attempt < 2 && found == 0; ++attempt) {
      FK_TRY_CUBLAS(cublasLtMatmulPreferenceSetAttribute(
          pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws_bytes, sizeof(ws_bytes)));
      FK_TRY_CUBLAS(cublasLtMatmulAlgoGetHeuristic(g_lt_handle, op, w_layout, a_layout, c_layout,
                                                   c_layout, pref, 1, &heuristic, &found));
      if (found == 0) {  // retry without workspace, as the reference does
        ws_bytes = 0;
        ws = nullptr;
      }
    }
    if (found == 0) {
      return fail(FK_W4A16_ERR_CUDA, "cublasLtMatmulAlgoGetHeuristic returned no usable algorithm");
    }
    const float one = 1.0f;
    const float zero = 0.0f;
    FK_TRY_CUBLAS(cublasLtMatmul(g_lt_handle, op, &one, weight, w_layout, activations, a_layout,
                                 &zero, output, c_layout, output, c_layout, &heuristic.algo, ws,
                                 ws_bytes, static_cast<cudaStream_t>(stream)));
    return FK_W4A16_OK;
  };
  rc = body();
  cleanup();
  return rc;
}

#ifdef FK_W4A16_TRACE
// Tuning builds only: copies the timeline marks (16 launches x 148 x 16 x 8 timestamps) to a host buffer.
__attribute__((visibility("default"))) int fk_w4a16_trace_read(unsigned long long* host) {
  FK_TRY_CUDA(cudaDeviceSynchronize());
  FK_TRY_CUDA(cudaMemcpyFromSymbol(host, g_trace, sizeof(unsigned long long) * kTraceLaunches * 148 * 16 * kTraceSlots));
  return FK_W4A16_OK;
}
#endif

int fk_w4a16_device_status(int* status) {
  if (status == nullptr) {
    return fail(FK_W4A16_ERR_INVALID_ARGUMENT, "status must not be null");
  }
  DeviceInfo* info = nullptr;
  FK_TRY(device_info(&info));
  FK_TRY_CUDA(cudaDeviceSynchronize());
  FK_TRY_CUDA(cudaMemcpy(status, info->status_word, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) {
    FK_TRY_CUDA(cudaMemset(info->status_word, 0, sizeof(int)));
  }
  return FK_W4A16_OK;
}

}  // extern "C"

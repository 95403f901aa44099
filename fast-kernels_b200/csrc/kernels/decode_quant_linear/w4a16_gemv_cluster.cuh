// The decode GEMV for layers with fewer tiles than SMs (o_proj, qkv, down_proj of an 8B model).
//
// With so few tiles every tile has to be shared by several CTAs, and in the packet-stream kernel
// (w4a16_gemv_stream.cuh) that sharing is settled through global memory: partial sums, a fence, a
// ticket, a second round of loads -- three dependent L2 round trips, 2-3 us at the end of a 5-10 us
// kernel. Here one thread-block CLUSTER owns a whole tile instead: its C CTAs x W warps split the
// tile's K/G packets into contiguous runs (same warp routine, same rings and bulk copies), each
// CTA adds its warps' sums in shared memory and PUSHES the result into rank 0's shared memory
// (st.async through distributed shared memory, counted by an mbarrier there), after which it is
// free to leave; rank 0 waits for the C - 1 deliveries, adds the per-CTA sums in rank order and
// stores the outputs. No scratch, no atomics, one split cluster barrier (arrive at kernel start,
// wait before the push: it only guards the mbarrier's initialisation); summation order is fixed,
// so results are bit-reproducible.
// C = floor(#SM / tiles) (2..8), so 128-144 of the 148 SMs stream -- the few idle SMs cost less
// than the global finish did.
#pragma once

#include "w4a16_gemv_stream.cuh"

namespace fk_w4a16 {

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_cta_count() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_index() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_barrier_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
// 16 bytes from registers into another CTA's shared memory; the mbarrier there (also a cluster
// address) counts the bytes when they have landed.
__device__ __forceinline__ void st_async_f4(uint32_t remote_addr, float4 v, uint32_t remote_bar) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1,%2,%3,%4}, [%5];" ::"r"(
          remote_addr),
      "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)), "r"(__float_as_uint(v.z)),
      "r"(__float_as_uint(v.w)), "r"(remote_bar)
      : "memory");
}
// Shared memory: ring barriers + the delivery barrier | per-warp slots [W][M_TILE][128] | CTA sum
// [M_TILE][128] | delivered sums [8][M_TILE][128] (used in rank 0) | per-warp activation buffers |
// rings.
constexpr int kMaxClusterCtas = 8;
struct ClusterSmem {
  uint32_t recv_bar, slots, cta_sum, recv, acts, rings, total;
};
__host__ __device__ inline ClusterSmem cluster_smem_plan(int warps, int stages, int group, int m_tile) {
  ClusterSmem plan;
  plan.recv_bar = static_cast<uint32_t>(warps) * stages * 8;
  plan.slots = (plan.recv_bar + 8u + 127u) & ~127u;
  plan.cta_sum = plan.slots + (static_cast<uint32_t>(warps) * m_tile * kTileCols * 4);
  plan.recv = plan.cta_sum + (static_cast<uint32_t>(m_tile) * kTileCols * 4);
  plan.acts = plan.recv + (static_cast<uint32_t>(kMaxClusterCtas) * m_tile * kTileCols * 4);
  plan.rings = plan.acts + (static_cast<uint32_t>(warps) * m_tile * group * 2);
  plan.total = plan.rings + (static_cast<uint32_t>(warps) * stages * packet_stride(group));
  return plan;
}

// Grid: (tiles * C, row tiles), cluster dimension (C, 1, 1); cluster i owns tile i.
template <int G, int M_TILE, class Mode>
__global__ void __launch_bounds__(512, 1)
    w4a16_gemv_cluster_kernel(const __grid_constant__ GemvParams p) {
  using E = typename Mode::Elem;
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kStageBytes = packet_stride(G);
  constexpr int kSlotFloats = M_TILE * kTileCols;

  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int warps_per_cta = static_cast<int>(blockDim.x) >> 5;
  const uint32_t rank = cluster_cta_rank();
  const uint32_t cluster_ctas = cluster_cta_count();
  const uint32_t tile = cluster_index();
  const int row_tile = static_cast<int>(blockIdx.y);
  const int row0 = row_tile * M_TILE;
  const int m_act = (p.m - row0) < M_TILE ? (p.m - row0) : M_TILE;
  const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);
  const int stages = p.stages;

  const ClusterSmem plan = cluster_smem_plan(warps_per_cta, stages, G, M_TILE);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_addr = smem_base + (warp * stages * 8);
  const uint32_t act_addr = smem_base + plan.acts + (warp * M_TILE * G * 2);
  const uint32_t ring_addr = smem_base + plan.rings + (warp * stages * kStageBytes);
  float* slots = reinterpret_cast<float*>(smem + plan.slots);
  float* cta_sum = reinterpret_cast<float*>(smem + plan.cta_sum);

  // This warp's share of the tile's groups: worker s of S = C * W takes
  // groups [floor(s NG / S), floor((s + 1) NG / S)): lengths differ by at most one, evenly spread.
  const uint32_t workers = cluster_ctas * static_cast<uint32_t>(warps_per_cta);
  const uint32_t s = (rank * warps_per_cta) + warp;
  const uint32_t g_begin = (s * num_groups) / workers;
  const uint32_t g_end = ((s + 1) * num_groups) / workers;

  trace_mark(0);
  const uint32_t recv_bar = smem_base + plan.recv_bar;
  if (rank == 0 && threadIdx.x == 0) {
    mbar_init(recv_bar, 1);
    mbar_init_fence();
  }
  cluster_barrier_arrive();  // the matching wait sits in front of the push, after the runs
  float y[M_TILE][4];
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      y[m][c] = 0.0f;
    }
  }
  if (g_end > g_begin) {
    if (lane == 0) {
      for (int st = 0; st < stages; ++st) {
        mbar_init(bar_addr + (st * 8), 1);
      }
      mbar_init_fence();
    }
    __syncwarp();
    auto keep = [](uint32_t, uint32_t, uint32_t) {};
    const uint32_t first_pkt = tile * num_groups;
    auto after_wait = [&](float (&inv_rms)[M_TILE]) {
      if (p.norm_weight != nullptr) {
        cta_inverse_rms<M_TILE, E>(p, row0, m_act, inv_rms);
      }
    };
    (void)consume_packet_run<G, M_TILE, Mode>(p, ring_addr, bar_addr, act_addr, row0, m_act,
                                              first_pkt + g_begin, first_pkt + g_end, lane, y, keep,
                                              after_wait);
  } else {
    pdl_launch_dependents();
    pdl_wait_for_prerequisites();
    if (p.norm_weight != nullptr) {  // the CTA-wide step of the fused RMSNorm needs every warp
      float unused[M_TILE];
      cta_inverse_rms<M_TILE, E>(p, row0, m_act, unused);
    }
  }

  trace_mark(3);
  // warp sums -> CTA sum (warp order)
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
    reinterpret_cast<float4*>(slots + (warp * kSlotFloats) + (m * kTileCols))[lane] =
        make_float4(y[m][0], y[m][1], y[m][2], y[m][3]);
  }
  __syncthreads();
  cluster_barrier_wait();  // rank 0's delivery barrier is initialised
  trace_mark(4);
  const uint32_t cta_bytes = static_cast<uint32_t>(kSlotFloats) * 4u;
  for (int idx = static_cast<int>(threadIdx.x); idx < kSlotFloats / 4; idx += static_cast<int>(blockDim.x)) {
    float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int w = 0; w < warps_per_cta; ++w) {
      const float4 part = reinterpret_cast<const float4*>(slots + (w * kSlotFloats))[idx];
      total.x += part.x;
      total.y += part.y;
      total.z += part.z;
      total.w += part.w;
    }
    if (rank == 0) {
      reinterpret_cast<float4*>(cta_sum)[idx] = total;
    } else {
      // push into rank 0: delivered[rank][idx]
      st_async_f4(cluster_map(smem_base + plan.recv + (rank * cta_bytes) + (idx * 16), 0), total,
                  cluster_map(recv_bar, 0));
    }
  }
  if (rank == 0) {
    // CTA sums -> outputs, in rank order, once every other CTA of the cluster has delivered
    if (threadIdx.x == 0) {
      mbar_expect_tx(recv_bar, (cluster_ctas - 1) * cta_bytes);
    }
    __syncthreads();  // own sums written; the arrival above is in place
    if (!mbar_wait_bounded(recv_bar, 0)) {
      if (threadIdx.x == 0) {
        atomicExch(p.status, static_cast<int>(kStatusCopyWaitTimeout));
      }
    } else {
      const float* delivered = reinterpret_cast<const float*>(smem + plan.recv);
      for (int idx = static_cast<int>(threadIdx.x); idx < kSlotFloats / 4; idx += static_cast<int>(blockDim.x)) {
        float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t r = 0; r < cluster_ctas; ++r) {
          const float4 part = r == 0 ? reinterpret_cast<const float4*>(cta_sum)[idx]
                                     : reinterpret_cast<const float4*>(delivered + (r * kSlotFloats))[idx];
          total[0] += part.x;
          total[1] += part.y;
          total[2] += part.z;
          total[3] += part.w;
        }
        const int m = idx / (kTileCols / 4);
        if (m < m_act) {
          store_tile_row<E>(p, row0 + m, tile, idx % (kTileCols / 4), total);
        }
      }
    }
  }
  trace_mark(5);
  exchange_complete<E>(p);  // multi-GPU calls: signal every GPU, wait for all of them
}

}  // namespace fk_w4a16

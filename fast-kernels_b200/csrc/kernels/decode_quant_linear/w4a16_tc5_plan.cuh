// Launch geometry of the tcgen05 kernel (w4a16_gemm_tc5.cuh), shared by host planning and device.
#pragma once

#include "w4a16_common.cuh"

namespace fk_w4a16 {

constexpr int kTc5TmemColumns = 256;       // allocation per CTA: two CTAs fit on an SM
constexpr int kTc5MaxGroups = 3;           // warpgroups per CTA (2 when a pass covers 8 or 16 rows)
constexpr int kTc5GroupTmemColumns = 80;   // 64 (A, G = 128) + 16 (D)
constexpr int kTc5N = 16;                  // MMA N: batch rows, padded

constexpr int kTc5StepBytes = 512;  // one K = 16 step of B: 16 rows x 32 bytes

// Shared-memory plan, used by host and device alike.
struct Tc5Smem {
  uint32_t tmem_slot;  // the TMEM base address lands here
  uint32_t fail_flags; // one word per warpgroup
  uint32_t barriers;   // per warpgroup: `stages` copy barriers + 1 MMA barrier (8 bytes each)
  uint32_t scalars;    // per warpgroup: [2][2][rows] floats (S_g, B_g of the packet in flight / next)
  uint32_t slots;      // per warpgroup: [2][rows][128] floats (partial sums of its first / last tile)
  uint32_t b_tiles;    // per warpgroup: G/16 steps x 512 bytes
  uint32_t rings;      // per warpgroup: stages x packet
  uint32_t total;
};
__host__ __device__ inline Tc5Smem tc5_smem_plan(int groups, int stages, int group_size, int rows) {
  Tc5Smem plan;
  plan.tmem_slot = 0;
  plan.fail_flags = 16;
  plan.barriers = 64;
  plan.scalars = plan.barriers + (static_cast<uint32_t>(groups) * (stages + 1) * 8);
  plan.scalars = (plan.scalars + 15u) & ~15u;
  plan.slots = plan.scalars + (static_cast<uint32_t>(groups) * 4 * rows * 4);
  plan.slots = (plan.slots + 127u) & ~127u;
  plan.b_tiles = plan.slots + (static_cast<uint32_t>(groups) * 2 * rows * kTileCols * 4);
  plan.rings = plan.b_tiles + (static_cast<uint32_t>(groups) * (group_size / 16) * kTc5StepBytes);
  plan.total = plan.rings + (static_cast<uint32_t>(groups) * stages * packet_stride(group_size));
  return plan;
}

__host__ __device__ constexpr int tc5_groups_for_rows(int rows) { return rows >= 8 ? 2 : kTc5MaxGroups; }

}  // namespace fk_w4a16

// Launch geometry of the pipelined tcgen05 kernel (w4a16_gemm_umma.cuh), shared by host planning
// and device code.
#pragma once

#include "w4a16_common.cuh"

namespace fk_w4a16 {

constexpr int kUmmaN = 16;              // MMA N: batch rows of a pass, padded
constexpr int kUmmaDepth = 4;           // depth P of the A / B / D / scalar rings
constexpr int kUmmaStepBytes = 512;     // one K = 16 step of B: 16 rows x 32 bytes
constexpr int kUmmaTmemColumns = 512;   // P x 64 columns of A (G = 128) + P x 16 of D, rounded up
constexpr int kUmmaDColumn0 = kUmmaDepth * 64;
constexpr int kUmmaUnpackGroups = 2;    // warpgroups that unpack, packets alternate between them

// Warp roles. Warpgroups that touch tensor memory start at a multiple of 4: warp w reaches TMEM
// lanes 32 (w % 4) .. 32 (w % 4) + 31.
constexpr int kUmmaProducerWarp = 0;
constexpr int kUmmaIssuerWarp = 1;
constexpr int kUmmaFirstUnpackWarp = 4;
constexpr int kUmmaFirstStagerWarp = kUmmaFirstUnpackWarp + (4 * kUmmaUnpackGroups);
constexpr int kUmmaStagerGroups = 2;     // warpgroups that stage activations, packets alternate
constexpr int kUmmaFirstEpilogueWarp = kUmmaFirstStagerWarp + (4 * kUmmaStagerGroups);
constexpr int kUmmaThreads = (kUmmaFirstEpilogueWarp + 4) * 32;
constexpr int kUmmaMaxStages = 24;

struct UmmaSmem {
  uint32_t tmem_slot;  // the TMEM base address lands here
  uint32_t fail_flag;
  uint32_t barriers;   // full[stages], empty[stages], ready[P], done[P], d_free[P], 8 bytes each
  uint32_t scalars;    // [2P][2][rows] floats: S_g and B_g of a packet
  uint32_t scales;     // [2P][128] 32-bit: alpha | beta << 16 of a packet
  uint32_t slots;      // [2][rows][128] floats: partial sums of the CTA's first / last tile
  uint32_t b_tiles;    // [P][G/16 steps][512 bytes]
  uint32_t rings;      // [stages][packet]
  uint32_t total;
};
__host__ __device__ inline UmmaSmem umma_smem_plan(int stages, int group_size, int rows) {
  UmmaSmem plan;
  plan.tmem_slot = 0;
  plan.fail_flag = 8;
  plan.barriers = 16;
  plan.scalars = plan.barriers + (static_cast<uint32_t>((2 * stages) + (3 * kUmmaDepth)) * 8);
  plan.scalars = (plan.scalars + 15u) & ~15u;
  plan.scales = plan.scalars + (static_cast<uint32_t>(2 * kUmmaDepth) * 2 * rows * 4);
  plan.slots = plan.scales + (static_cast<uint32_t>(2 * kUmmaDepth) * kTileCols * 4);
  plan.slots = (plan.slots + 127u) & ~127u;
  plan.b_tiles = plan.slots + (2u * rows * kTileCols * 4);
  plan.rings = plan.b_tiles + (static_cast<uint32_t>(kUmmaDepth) * (group_size / 16) * kUmmaStepBytes);
  plan.total = plan.rings + (static_cast<uint32_t>(stages) * packet_stride(group_size));
  return plan;
}

__host__ __device__ constexpr int umma_rows_for_batch(int batch) {
  return batch <= 1 ? 1 : (batch <= 2 ? 2 : (batch <= 4 ? 4 : (batch <= 8 ? 8 : 16)));
}

}  // namespace fk_w4a16

// The stream kernel (w4a16_gemv_stream.cuh) with its inner product on the legacy tensor path, for
// batches of 1 and 2: same warp-per-run structure, same in-warp activation staging, same finish,
// but the 512 mixed-precision FMAs of a packet become 64 mma.sync.m16n8k16 -- the streaming phase
// of the CUDA-core kernel is bound by instruction issue (1150 warp instructions per packet), and
// an MMA mixed into a stream of ALU work costs 3-5 issue slots where the eight FMAs it replaces
// cost eight (microbenchmark: 8 mma.sync + 64 independent LOP3 per iteration).
//
// Outcome (B200, measured): same results as the CUDA-core kernel, and slower -- 28672 x 4096 at
// batch 1: 17.3 us against 15.3 on the same box; 6144 x 4096: 7.5 against 6.8 -- so it is opt-in
// (FK_W4A16_WMMA=1) and the FMA kernel stays the default for batches 1 and 2.
//
// Operand mapping (that of w4a16_gemm_mma.cuh, one warp covering both column halves): A = weights
// (16 output columns x 16 k), B = activations (16 k x 8 "batch" columns, of which only the first
// M_TILE are real: every other column repeats a real one and is ignored), D = 16 x 8 fp32. Lane
// (g = lane / 4, t = lane % 4) takes whole 32-bit words: word-row t * (G/32) + b of columns
// 64 s + 4 g + j (MMA row g) and 64 s + 32 + 4 g + j (MMA row g + 8) for tile (s, j), and spends
// each word on two k-steps -- pairs (0,4)(2,6), then (1,5)(3,7) -- against the staged activations
// of the same word-row, which the warp's own staging step has left in shared memory in exactly
// that pair order. The packet's word-rows are copied as four chunks with a 32-byte skew so that
// the 128-bit fragment loads are bank-conflict free. B_g and S_g come from the staging step's
// warp sums, as in the stream kernel.
#pragma once

#include "w4a16_gemm_mma.cuh"

namespace fk_w4a16 {

template <int G>
struct WmmaGeom {
  static constexpr int kChunkRows = G / 32;
  static constexpr int kChunkBytes = kChunkRows * kTileCols * 4;
  static constexpr int kChunkPitch = kChunkBytes + 32;
  static constexpr int kScaleOffset = (3 * kChunkPitch) + kChunkBytes;
  static constexpr int kStageBytes = kScaleOffset + kScaleBytes;
};
__host__ __device__ constexpr int wmma_stage_bytes(int group) {
  return (3 * (((group / 32) * kTileCols * 4) + 32)) + ((group / 32) * kTileCols * 4) + kScaleBytes;
}

// Shared-memory plan: that of the stream kernel with the skewed stage size.
__host__ __device__ inline StreamSmem wmma_smem_plan(int warps, int stages, int group, int m_tile) {
  StreamSmem plan;
  plan.barriers = 0;
  plan.slots = ((static_cast<uint32_t>(warps) * stages * 8) + 127u) & ~127u;
  plan.acts = plan.slots + (static_cast<uint32_t>(warps) * 2 * m_tile * kTileCols * 4);
  plan.rings = plan.acts + (static_cast<uint32_t>(warps) * m_tile * group * 2);
  plan.total = plan.rings + (static_cast<uint32_t>(warps) * stages * wmma_stage_bytes(group));
  return plan;
}

template <int G, int M_TILE, class Mode>
__global__ void __launch_bounds__(512, 1)
    w4a16_gemv_wmma_kernel(const __grid_constant__ GemvParams p) {
  static_assert(M_TILE == 1 || M_TILE == 2, "rows per pass");
  using E = typename Mode::Elem;
  using Geom = WmmaGeom<G>;
  constexpr int kStride = packet_stride(G);
  constexpr int kActBytes = G * 2;
  constexpr int kActLanes = G / 4;
  constexpr int kSlotFloats = M_TILE * kTileCols;
  extern __shared__ __align__(128) uint8_t smem[];

  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int warps_per_cta = static_cast<int>(blockDim.x) >> 5;
  const uint32_t v = (blockIdx.x * warps_per_cta) + warp;
  const uint32_t workers = static_cast<uint32_t>(p.active_warps);
  const bool active = v < workers;
  const int row_tile = static_cast<int>(blockIdx.y);
  const int row0 = row_tile * M_TILE;
  const int m_act = (p.m - row0) < M_TILE ? (p.m - row0) : M_TILE;
  const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);
  const int stages = p.stages;

  const StreamSmem plan = wmma_smem_plan(warps_per_cta, stages, G, M_TILE);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_addr = smem_base + plan.barriers + (warp * stages * 8);
  const uint32_t act_addr = smem_base + plan.acts + (warp * M_TILE * kActBytes);
  const uint32_t ring_addr = smem_base + plan.rings + (warp * stages * Geom::kStageBytes);
  float* slots = reinterpret_cast<float*>(smem + plan.slots);  // [warp][2][kSlotFloats]

  const uint32_t p_begin = active ? run_begin(v, p) : 0;
  const uint32_t p_end = active ? run_begin(v + 1, p) : 0;
  const uint32_t count = p_end - p_begin;
  const uint32_t first_tile = p_begin / num_groups;

  if (active) {
    if (lane == 0) {
      for (int s = 0; s < stages; ++s) {
        mbar_init(bar_addr + (s * 8), 1);
      }
      mbar_init_fence();
    }
    __syncwarp();

    const uint64_t weight_policy = l2_evict_first_policy();
    const auto* act_bytes = static_cast<const uint8_t*>(p.act);
    uint32_t issue_idx = 0;
    int issue_slot = 0;
    auto issue_next = [&]() {
      const uint32_t bar = bar_addr + (issue_slot * 8);
      const uint32_t dst = ring_addr + (issue_slot * Geom::kStageBytes);
      const uint8_t* src = p.packets + (static_cast<size_t>(p_begin + issue_idx) * kStride);
      mbar_expect_tx(bar, static_cast<uint32_t>(kStride));
#pragma unroll
      for (int c = 0; c < 3; ++c) {
        bulk_copy_g2s(dst + (c * Geom::kChunkPitch), src + (c * Geom::kChunkBytes), Geom::kChunkBytes,
                      bar, weight_policy);
      }
      bulk_copy_g2s(dst + (3 * Geom::kChunkPitch), src + (3 * Geom::kChunkBytes),
                    Geom::kChunkBytes + kScaleBytes, bar, weight_policy);
      ++issue_idx;
      issue_slot = (issue_slot + 1 == stages) ? 0 : issue_slot + 1;
    };
    if (lane == 0) {
      const uint32_t prefill = count < static_cast<uint32_t>(stages) ? count : stages;
      for (uint32_t j = 0; j < prefill; ++j) {
        issue_next();
      }
    }
    // The weight copies do not depend on the kernel before this one; everything below does.
    pdl_launch_dependents();
    pdl_wait_for_prerequisites();
    float inv_rms[M_TILE];
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      inv_rms[m] = 1.0f;
    }
    const bool normalise = p.norm_weight != nullptr;
    if (normalise) {
      cta_inverse_rms<M_TILE, E>(p, row0, m_act, inv_rms);
    }

    uint32_t tile = first_tile;
    uint32_t act_group = p_begin - (tile * num_groups);
    uint2 next_weight = make_uint2(0u, 0u);
    uint2 next_raw[M_TILE];
    auto load_activations = [&]() {
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        next_raw[m] = make_uint2(0u, 0u);
        if (m < m_act && lane < kActLanes) {
          const size_t elem = (static_cast<size_t>(row0 + m) * p.k) + (act_group * G);
          next_raw[m] = __ldg(reinterpret_cast<const uint2*>(act_bytes + (elem * 2)) + lane);
        }
      }
      if (normalise && lane < kActLanes) {
        next_weight = __ldg(reinterpret_cast<const uint2*>(static_cast<const unsigned short*>(p.norm_weight) +
                                                           (static_cast<size_t>(act_group) * G)) + lane);
      }
      act_group = (act_group + 1 == num_groups) ? 0 : act_group + 1;
    };
    load_activations();

    // y[tile (s, j)][c]: column 64 s + 4 (g + 8 (c >> 1)) + j, batch row 2 t + (c & 1): only the
    // lanes with t == 0 hold real rows (0 and 1).
    float y[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        y[i][c] = 0.0f;
      }
    }
    auto on_tile_done = [&](uint32_t tile_index, uint32_t first_pkt, uint32_t end_pkt) {
      if (t != 0) {
        return;
      }
      const bool full = (end_pkt - first_pkt) == num_groups;
      float* slot = slots + (((warp * 2) + (tile_index == first_tile ? 0 : 1)) * kSlotFloats);
#pragma unroll
      for (int s = 0; s < 2; ++s) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int block = (16 * s) + g + (8 * half);  // 4-column block of the tile
#pragma unroll
          for (int m = 0; m < M_TILE; ++m) {
            const float four[4] = {y[(4 * s) + 0][(2 * half) + m], y[(4 * s) + 1][(2 * half) + m],
                                   y[(4 * s) + 2][(2 * half) + m], y[(4 * s) + 3][(2 * half) + m]};
            if (!full) {
              reinterpret_cast<float4*>(slot + (m * kTileCols))[block] =
                  make_float4(four[0], four[1], four[2], four[3]);
            } else if (m < m_act) {
              store_tile_row<E>(p, row0 + m, tile_index, block, four);
            }
          }
        }
      }
    };

    uint32_t pkt = p_begin;
    uint32_t tile_end = (tile + 1) * num_groups;
    uint32_t tile_first = p_begin;
    int slot_index = 0;
    uint32_t parity = 0;
    bool ok = true;
    const int b_row = g < M_TILE ? g : M_TILE - 1;  // the batch row this lane's B column repeats

    for (uint32_t j = 0; j < count; ++j, ++pkt) {
      if (pkt == tile_end) {
        on_tile_done(tile, tile_first, pkt);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            y[i][c] = 0.0f;
          }
        }
        ++tile;
        tile_first = pkt;
        tile_end += num_groups;
      }
      const uint32_t stage = ring_addr + (slot_index * Geom::kStageBytes);
      if (!mbar_wait_bounded(bar_addr + (slot_index * 8), parity)) {
        ok = false;
        break;
      }

      float group_sum[M_TILE];
      float bias[M_TILE];
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        group_sum[m] = 0.0f;
        bias[m] = 0.0f;
        if (m < m_act) {
          const uint2 raw = normalise ? normalise4<E>(next_raw[m], next_weight, inv_rms[m]) : next_raw[m];
          stage_activations<G, Mode>(raw, act_addr + (m * kActBytes), lane, group_sum[m], bias[m]);
        }
      }
      if (j + 1 < count) {
        load_activations();
      }
      __syncwarp();

      float acc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          acc[i][c] = 0.0f;
        }
      }
      const uint32_t w_base = stage + (t * Geom::kChunkPitch) + (g * 16);
      const uint32_t a_base = act_addr + (b_row * kActBytes) + (t * Geom::kChunkRows * 16);
#pragma unroll 2
      for (int b = 0; b < Geom::kChunkRows; ++b) {
        const uint4 bq = lds128(a_base + (b * 16));
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint4 w_lo = lds128(w_base + (b * kTileCols * 4) + (s * 256));
          const uint4 w_hi = lds128(w_base + (b * kTileCols * 4) + (s * 256) + 128);
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const NibblePairs lo = Mode::unpack(word_of(w_lo, jj));
            const NibblePairs hi = Mode::unpack(word_of(w_hi, jj));
            mma_word_pair<Mode>(acc[(4 * s) + jj], lo, hi, bq);
          }
        }
      }

      // group epilogue: y += alpha * (acc - B) + beta * S for this lane's 16 columns x 2 rows
#pragma unroll
      for (int s = 0; s < 2; ++s) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int col0 = (64 * s) + (4 * (g + (8 * half)));
          const uint2 a_raw = lds64(stage + Geom::kScaleOffset + (col0 * 2));
          const uint2 b_raw = lds64(stage + Geom::kScaleOffset + (kTileCols * 2) + (col0 * 2));
          const unsigned short a_bits[4] = {
              static_cast<unsigned short>(a_raw.x & 0xffffu), static_cast<unsigned short>(a_raw.x >> 16),
              static_cast<unsigned short>(a_raw.y & 0xffffu), static_cast<unsigned short>(a_raw.y >> 16)};
          const unsigned short b_bits[4] = {
              static_cast<unsigned short>(b_raw.x & 0xffffu), static_cast<unsigned short>(b_raw.x >> 16),
              static_cast<unsigned short>(b_raw.y & 0xffffu), static_cast<unsigned short>(b_raw.y >> 16)};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const float alpha = E::to_float(a_bits[jj]);
            const float beta = E::to_float(b_bits[jj]);
#pragma unroll
            for (int m = 0; m < M_TILE; ++m) {
              float& out = y[(4 * s) + jj][(2 * half) + m];
              out = fmaf(alpha, acc[(4 * s) + jj][(2 * half) + m] - bias[m], out);
              out = fmaf(beta, group_sum[m], out);
            }
          }
        }
      }

      __syncwarp();
      if (lane == 0 && issue_idx < count) {
        proxy_fence_async();
        issue_next();
      }
      if (++slot_index == stages) {
        slot_index = 0;
        parity ^= 1u;
      }
    }

    if (ok) {
      on_tile_done(tile, tile_first, pkt);
    } else {
      // A copy never landed: record it and give the copies in flight a bounded chance to finish.
      issue_idx = __shfl_sync(0xffffffffu, issue_idx, 0);
      if (lane == 0) {
        atomicExch(p.status, static_cast<int>(kStatusCopyWaitTimeout));
      }
      for (uint32_t j = pkt - p_begin; j < issue_idx; ++j) {
        (void)mbar_wait_bounded(bar_addr + (slot_index * 8), parity);
        if (++slot_index == stages) {
          slot_index = 0;
          parity ^= 1u;
        }
      }
    }
  } else {
    pdl_launch_dependents();
    pdl_wait_for_prerequisites();
    if (p.norm_weight != nullptr) {
      float unused[M_TILE];
      cta_inverse_rms<M_TILE, E>(p, row0, m_act, unused);
    }
  }
  __syncthreads();
  finish_cta<M_TILE, E>(p, slots, 2 * kSlotFloats, slots + kSlotFloats, 2 * kSlotFloats, warp, lane,
                        warps_per_cta, row_tile, row0, m_act);
}

}  // namespace fk_w4a16

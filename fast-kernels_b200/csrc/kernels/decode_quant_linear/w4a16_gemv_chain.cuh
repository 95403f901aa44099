// A CHAIN of decode GEMVs in one persistent launch: step i + 1 may read what step i wrote (a
// decoder's o_proj -> gate/up -> down_proj -> next layer's qkv, with the fused residual, SiLU-and-
// multiply and RMSNorm callers in between), exactly as if the steps were separate calls of the
// packet-stream kernel on one stream -- but without the per-call launch: between two calls of the
// stream kernel ~1.5 us pass from the last exit of one to the first copy issued by the next (grid
// completion, CTA launch, cold instruction cache), and another ~2.4 us until every warp has its
// first packet, because all rings are filled at once. Here the grid stays resident:
//   * a warp that has consumed the last packet of its run in step i at once issues the first
//     `stages` copies of its run in step i + 1 -- weights do not depend on step i -- so the rings
//     are full again by the time step i is finished everywhere;
//   * steps are separated by a grid-wide barrier in software (one release-add per CTA to a counter
//     in the workspace, bounded polling by one thread per CTA) instead of a kernel boundary;
//   * activations, residuals and norm weights are read with L2-coherent loads (ld.global.cg): what
//     step i wrote must not be served from a stale L1 line.
// Work split, rings, per-packet math, split-K finish and summation order of every step are those of
// the packet-stream kernel for the same problem (same plan arithmetic), so a chain gives the bits
// that the same steps give as separate stream-kernel calls with one CTA per SM. All steps share
// batch (<= 4), group size and element type; each has its own n, k, buffers and fused options.
// Every CTA of the grid must be resident for the barrier (grid = #SM, one CTA per SM by shared
// memory); all waits are bounded and report through the status word.
#pragma once

#include "w4a16_gemv_stream.cuh"

namespace fk_w4a16 {

constexpr int kMaxChainSteps = 8;

struct ChainParams {
  GemvParams step[kMaxChainSteps];
  int count;
  unsigned int* barrier;      // grid barrier counter, zero between calls
  unsigned int* exit_count;   // zero between calls: the last CTA to leave resets the barrier
  unsigned long long barrier_wait_ns;
};

__device__ __forceinline__ uint2 ldcg_u2(const void* ptr) {
  uint2 v;
  asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr) : "memory");
  return v;
}

// Warps of a CTA that take part in a step: ceil(V / grid), as the stream kernel's launch plan has it.
__device__ __forceinline__ int chain_step_warps(const GemvParams& p) {
  return (p.active_warps + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
}

template <int G, int M_TILE, class Mode>
__global__ void __launch_bounds__(512, 1)
    w4a16_gemv_chain_kernel(const __grid_constant__ ChainParams cp) {
  using E = typename Mode::Elem;
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kStride = packet_stride(G);
  constexpr int kStageBytes = kStride;
  constexpr int kSlotFloats = M_TILE * kTileCols;
  constexpr int kActLanes = G / 4;
  __shared__ int barrier_ok;
  __shared__ int cta_failed;  // a copy of some warp never arrived: the whole CTA stops at the next barrier

  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int warps_per_cta = static_cast<int>(blockDim.x) >> 5;
  const uint32_t cta = blockIdx.x;
  const int stages = cp.step[0].stages;

  const StreamSmem plan = stream_smem_plan(warps_per_cta, stages, G, M_TILE);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_addr = smem_base + plan.barriers + (warp * stages * 8);
  const uint32_t act_addr = smem_base + plan.acts + (warp * M_TILE * G * 2);
  const uint32_t ring_addr = smem_base + plan.rings + (warp * stages * kStageBytes);
  float* slots = reinterpret_cast<float*>(smem + plan.slots);  // [warp][2][kSlotFloats]

  if (lane == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_addr + (s * 8), 1);
    }
    mbar_init_fence();
  }
  if (threadIdx.x == 0) {
    cta_failed = 0;
  }
  __syncwarp();
  const uint64_t weight_policy = l2_evict_first_policy();

  // The warp's ring, continuous over all steps: copies are issued into `issue_slot`, packets are
  // consumed from `slot` under `parity`.
  int issue_slot = 0;
  int slot = 0;
  uint32_t parity = 0;
  auto issue_packet = [&](const GemvParams& p, uint32_t packet) {
    const uint32_t bar = bar_addr + (issue_slot * 8);
    mbar_expect_tx(bar, static_cast<uint32_t>(kStride));
    bulk_copy_g2s(ring_addr + (issue_slot * kStageBytes), p.packets + (static_cast<size_t>(packet) * kStride),
                  kStride, bar, weight_policy);
    issue_slot = (issue_slot + 1 == stages) ? 0 : issue_slot + 1;
  };
  // This warp's run in a step: [begin, end), empty if the warp does not take part.
  auto run_of = [&](const GemvParams& p, uint32_t& begin, uint32_t& end) {
    const int step_warps = chain_step_warps(p);
    const uint32_t v = (cta * static_cast<uint32_t>(step_warps)) + static_cast<uint32_t>(warp);
    const bool active = warp < step_warps && v < static_cast<uint32_t>(p.active_warps);
    begin = active ? run_begin(v, p) : 0u;
    end = active ? run_begin(v + 1, p) : 0u;
  };
  auto prefill = [&](const GemvParams& p, uint32_t begin, uint32_t end) -> uint32_t {
    const uint32_t count = end - begin;
    const uint32_t ahead = count < static_cast<uint32_t>(stages) ? count : static_cast<uint32_t>(stages);
    if (lane == 0) {
      for (uint32_t j = 0; j < ahead; ++j) {
        issue_packet(p, begin + j);
      }
    }
    return ahead;
  };

  uint32_t p_begin = 0;
  uint32_t p_end = 0;
  run_of(cp.step[0], p_begin, p_end);
  uint32_t issued = prefill(cp.step[0], p_begin, p_end);  // packets of this run already issued

  // Programmatic dependent launch: the copies above do not depend on the kernel before this one.
  pdl_launch_dependents();
  pdl_wait_for_prerequisites();
  __syncthreads();

  bool ok = true;
  for (int step = 0; step < cp.count; ++step) {
    const GemvParams& p = cp.step[step];
    const int row_tile = 0;
    const int row0 = 0;
    const int m_act = p.m < M_TILE ? p.m : M_TILE;
    const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);
    const int step_warps = chain_step_warps(p);
    const uint32_t count = p_end - p_begin;
    const uint32_t first_tile = count > 0 ? p_begin / num_groups : 0u;

    float inv_rms[M_TILE];
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      inv_rms[m] = 1.0f;
    }
    if (p.norm_weight != nullptr) {  // the CTA-wide step of the fused RMSNorm needs every warp
      cta_inverse_rms<M_TILE, E>(p, row0, m_act, inv_rms);
    }
    const bool normalise = p.norm_weight != nullptr;

    // the next step's run, known now so that its first copies can follow this run's last packet
    uint32_t next_begin = 0;
    uint32_t next_end = 0;
    if (step + 1 < cp.count) {
      run_of(cp.step[step + 1], next_begin, next_end);
    }
    uint32_t next_issued = 0;

    if (count > 0 && ok) {
      float y[M_TILE][4];
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          y[m][c] = 0.0f;
        }
      }
      auto on_tile_done = [&](uint32_t tile, uint32_t first_pkt, uint32_t end_pkt) {
        if ((end_pkt - first_pkt) == num_groups) {
#pragma unroll
          for (int m = 0; m < M_TILE; ++m) {
            if (m < m_act) {
              store_tile_row<E>(p, row0 + m, tile, lane, y[m]);
            }
          }
          return;
        }
        float* slot_ptr = slots + (((warp * 2) + (tile == first_tile ? 0 : 1)) * kSlotFloats);
#pragma unroll
        for (int m = 0; m < M_TILE; ++m) {
          reinterpret_cast<float4*>(slot_ptr + (m * kTileCols))[lane] =
              make_float4(y[m][0], y[m][1], y[m][2], y[m][3]);
        }
      };

      const auto* act_bytes = static_cast<const uint8_t*>(p.act);
      uint32_t tile = first_tile;
      uint32_t act_group = p_begin - (tile * num_groups);
      uint2 next_weight = make_uint2(0u, 0u);
      auto load_activations = [&](uint2 (&dst)[M_TILE]) {
#pragma unroll
        for (int m = 0; m < M_TILE; ++m) {
          dst[m] = make_uint2(0u, 0u);
          if (m < m_act && lane < kActLanes) {
            const size_t elem = (static_cast<size_t>(row0 + m) * p.k) + (act_group * G);
            dst[m] = ldcg_u2(reinterpret_cast<const uint2*>(act_bytes + (elem * 2)) + lane);
          }
        }
        if (normalise && lane < kActLanes) {
          next_weight = ldcg_u2(reinterpret_cast<const uint2*>(static_cast<const unsigned short*>(p.norm_weight) +
                                                              (static_cast<size_t>(act_group) * G)) + lane);
        }
        act_group = (act_group + 1 == num_groups) ? 0 : act_group + 1;
      };
      uint2 next_raw[M_TILE];
      load_activations(next_raw);

      uint32_t pkt = p_begin;
      uint32_t tile_end = (tile + 1) * num_groups;
      uint32_t tile_first = p_begin;
      for (uint32_t j = 0; j < count; ++j, ++pkt) {
        if (pkt == tile_end) {
          on_tile_done(tile, tile_first, pkt);
#pragma unroll
          for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              y[m][c] = 0.0f;
            }
          }
          ++tile;
          tile_first = pkt;
          tile_end += num_groups;
        }
        const uint32_t stage = ring_addr + (slot * kStageBytes);
        if (!mbar_wait_bounded(bar_addr + (slot * 8), parity)) {
          ok = false;
          cta_failed = 1;
          break;
        }
        uint2 raw[M_TILE];
#pragma unroll
        for (int m = 0; m < M_TILE; ++m) {
          raw[m] = normalise ? normalise4<E>(next_raw[m], next_weight, inv_rms[m]) : next_raw[m];
        }
        if (j + 1 < count) {
          load_activations(next_raw);
        }
        multiply_packet<G, M_TILE, Mode>(stage, act_addr, raw, m_act, lane, y);

        // The whole warp is done reading this buffer: refill it -- with this run's next packet,
        // or, once the run is fully issued, with the first packets of the next step's run.
        __syncwarp();
        if (lane == 0) {
          if (issued < count) {
            proxy_fence_async();
            issue_packet(p, p_begin + issued);
          } else if (next_issued < (next_end - next_begin) && next_issued < static_cast<uint32_t>(stages)) {
            proxy_fence_async();
            issue_packet(cp.step[step + 1], next_begin + next_issued);
          }
        }
        // every lane keeps the counters (cheap, and the next step's loop needs them)
        if (issued < count) {
          ++issued;
        } else if (next_issued < (next_end - next_begin) && next_issued < static_cast<uint32_t>(stages)) {
          ++next_issued;
        }
        if (++slot == stages) {
          slot = 0;
          parity ^= 1u;
        }
      }
      if (ok) {
        on_tile_done(tile, tile_first, pkt);
      }
    }
    // A warp without a run in this step (or with a run shorter than the ring) still owes the next
    // step its first copies: every packet of this run is consumed, so the buffers are free.
    if (ok && step + 1 < cp.count && lane == 0) {
      const uint32_t next_count = next_end - next_begin;
      const uint32_t want = next_count < static_cast<uint32_t>(stages) ? next_count : static_cast<uint32_t>(stages);
      if (next_issued < want) {
        proxy_fence_async();
      }
      while (next_issued < want) {
        issue_packet(cp.step[step + 1], next_begin + next_issued);
        ++next_issued;
      }
    }
    if (step + 1 < cp.count) {
      const uint32_t next_count = next_end - next_begin;
      next_issued = next_count < static_cast<uint32_t>(stages) ? next_count : static_cast<uint32_t>(stages);
    }

    __syncthreads();
    if (cta_failed != 0) {  // the same for every thread of the CTA
      ok = false;
      break;
    }
    // warps (and CTAs) without a run in this step have nothing to finish
    if (warp < step_warps && (cta * static_cast<uint32_t>(step_warps)) < static_cast<uint32_t>(p.active_warps)) {
      finish_cta<M_TILE, E>(p, slots, 2 * kSlotFloats, slots + kSlotFloats, 2 * kSlotFloats, warp, lane,
                            step_warps, row_tile, row0, m_act);
    }

    if (step + 1 < cp.count) {
      // ---- grid barrier: every CTA's outputs of this step are visible before any CTA reads them
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(cp.barrier, 1u);
        const unsigned int target = gridDim.x * static_cast<unsigned int>(step + 1);
        const unsigned long long start = global_timer_ns();
        bool arrived = false;
        for (;;) {
          const unsigned int seen = *reinterpret_cast<volatile unsigned int*>(cp.barrier);
          if (seen >= target) {
            arrived = true;
            break;
          }
          if (global_timer_ns() - start > cp.barrier_wait_ns) {
            break;
          }
        }
        __threadfence();
        barrier_ok = arrived ? 1 : 0;
      }
      __syncthreads();
      if (barrier_ok == 0) {
        ok = false;
        break;
      }
      p_begin = next_begin;
      p_end = next_end;
      issued = next_issued;
    }
  }

  if (!ok) {
    // A copy or the grid barrier never completed (every thread of the CTA arrives here together).
    // Record it; give the copies still in flight a bounded chance to land before this CTA's shared
    // memory is handed on.
    if (lane == 0) {
      atomicExch(cp.step[0].status, static_cast<int>(kStatusCopyWaitTimeout));
      for (int s = 0; s < stages; ++s) {
        (void)mbar_wait_bounded(bar_addr + (s * 8), parity);
      }
    }
  }
  // The last CTA to leave puts the barrier counter back to zero for the next call.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int left = atomicAdd(cp.exit_count, 1u);
    if (left == gridDim.x - 1) {
      *cp.barrier = 0u;
      *cp.exit_count = 0u;
      __threadfence();
    }
  }
}

}  // namespace fk_w4a16

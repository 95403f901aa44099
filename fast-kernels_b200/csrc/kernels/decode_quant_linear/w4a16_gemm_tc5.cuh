// Fifth-generation tensor-core variant (tcgen05 + tensor memory) of the packet-stream kernel, for
// 1 <= M <= 16 rows per pass.
//
// Why: on CUDA cores one packet costs ~1140 warp instructions, 512 of them FMAs, and at decode
// batch sizes the stream kernel is bound by instruction issue, not by HBM. Here the multiply-adds
// leave the SM's issue slots altogether: the unpacked weights go from registers straight into
// tensor memory (TMEM) and one elected thread issues tcgen05.mma for the whole 128-column tile.
//
// Outcome (B200, measured): bit-for-bit the same bar as the other kernels (within the 16-bit
// output rounding of the fp64 oracle for every group size, type and batch), but NOT faster, so it
// is opt-in (fk_w4a16_set_variant / FK_W4A16_TC5=1) and the CUDA-core kernels stay the default.
// A tcgen05.mma kind::f16 instruction occupies the tensor core for ~141 clocks whatever its shape
// (M = 64 or 128, N = 16 ... 256, A from TMEM or from shared memory -- timed by issuing 4096 of
// them back to back from one thread). A packet needs G/16 of them, so an SM consumes at most
// 128 x 16 weights per 141 clocks = 14.5 weights/clk, i.e. ~2 TB/s of 4-bit weights over 148 SMs:
// a third of what HBM delivers. The tensor core is built for N = 256; at decode batch sizes the
// instruction floor, not the math, sets the rate. (Layer set: 14.8 us per call against 8.7.)
//
// Operand mapping. One warpgroup (4 warps, 128 threads) owns a packet; thread i owns output column
// i of the tile = TMEM lane i = row i of the MMA's A operand (M = 128). Per packet of group size G:
//   A  [128 x G]   "constant + q" 16-bit floats exactly as the LOP3 unpack produces them (never
//                  converted, never scaled), written with tcgen05.st: 32-bit TMEM column c of a
//                  K = 16 step holds k-slots (2c, 2c + 1) = one unpacked pair (nibbles i, i + 4);
//   B  [16 x G]    the activations of the group, k-permuted to match and in the pair formats of
//                  the unpack mode, in shared memory (K-major, no swizzle: core matrices of 8 rows
//                  x 16 bytes). Rows >= batch stay zero (the MMA's N is 16);
//   D  [128 x 16]  fp32 in TMEM, overwritten by the first MMA of every packet.
// Which real k an MMA k-slot means is free as long as A and B agree, so a K = 16 step is made of
// the pairs of one type from four consecutive word-rows: for bf16, G/32 steps of bf16 x bf16
// (pairs (0,4) and (2,6): 128 + q against the raw activation) and G/32 steps of fp16 x fp16 (pairs
// (1,5) and (3,7): 1024 + 16 q against fp16(a / 16)); for fp16, all steps are of the second kind.
// After the packet's MMAs, y += alpha * (D - B_g) + beta * S_g per column, with the constant term
// B_g and the activation sum S_g of the group computed in fp32 on CUDA cores while staging B.
//
// Flow per warpgroup and packet j: wait for the packet's bulk copy; every thread unpacks its
// column (G/8 conflict-free 32-bit loads, 5 ALU instructions per word); one warp (in rotation)
// stages the group's activations; wait for MMA j-1, read its D and fold it into y; store A and B;
// barrier; one thread issues the MMAs and a commit, then refills the ring slot.
// Tile bookkeeping, split-K finish, output placement and peer stores are those of the stream
// kernel (a warpgroup plays the part of a warp there).
#pragma once

#include "w4a16_gemv_stream.cuh"
#include "w4a16_tc5_plan.cuh"

namespace fk_w4a16 {

// ---- tcgen05 wrappers ----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&d)[N]) {
  static_assert(N == 1 || N == 2 || N == 4 || N == 8 || N == 16, "rows per pass");
  uint32_t r[16];
  if constexpr (N == 1) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r[0]) : "r"(taddr));
  } else if constexpr (N == 2) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1])
                 : "r"(taddr));
  } else if constexpr (N == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr));
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                   "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
  } else {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
  }
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    d[i] = __uint_as_float(r[i]);
  }
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]; `accumulate` = 0 overwrites D.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// The mbarrier receives one arrival when every MMA this thread has issued so far is complete.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void group_barrier(int group) {
  asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Instruction descriptor of tcgen05.mma kind::f16: fp32 accumulate (bits 4-5 = 1), A and B formats
// (bits 7-9 and 10-12: 0 = fp16, 1 = bf16), both operands K-major (bits 15, 16 = 0), N / 8 in bits
// 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc(bool bf16) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
         (static_cast<uint32_t>(kTc5N / 8) << 17) | (static_cast<uint32_t>(128 / 16) << 24);
}
// Shared-memory descriptor of one K = 16 step of B: K-major, no swizzle. Address, leading-dimension
// offset (between the two 16-byte K chunks: 128 B) and stride-dimension offset (between groups of
// 8 rows: 256 B) in 16-byte units at bits 0-13, 16-29, 32-45; descriptor version 1 at bit 46.
__device__ __forceinline__ uint64_t umma_b_desc(uint32_t smem_address) {
  return static_cast<uint64_t>((smem_address & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 16) |
         (static_cast<uint64_t>(256 >> 4) << 32) | (uint64_t{1} << 46);
}

template <int G, int ROWS, class Mode>
__global__ void __launch_bounds__(tc5_groups_for_rows(ROWS) * 128, 1)
    w4a16_gemm_tc5_kernel(const __grid_constant__ GemvParams p) {
  using E = typename Mode::Elem;
  constexpr int kStride = packet_stride(G);
  constexpr int kQBytes = packet_q_bytes(G);
  constexpr int kWordRows = G / 8;
  constexpr int kStepsPerKind = G / 32;       // K = 16 steps of each pair kind
  constexpr int kACols = G / 2;               // TMEM columns of A
  constexpr int kSlotFloats = ROWS * kTileCols;
  constexpr uint32_t kIdescFirst = umma_idesc(Mode::kEvenNibblesBf16);
  constexpr uint32_t kIdescSecond = umma_idesc(false);
  extern __shared__ __align__(128) uint8_t smem[];

  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int wg = warp >> 2;          // warpgroup within the CTA
  const int quarter = warp & 3;      // this warp reaches TMEM lanes 32 * quarter .. + 31
  const int col = (quarter * 32) + lane;
  const bool leader = (static_cast<int>(threadIdx.x) & 127) == 0;
  const int groups_per_cta = static_cast<int>(blockDim.x) >> 7;
  const uint32_t v = (blockIdx.x * groups_per_cta) + wg;
  const uint32_t workers = static_cast<uint32_t>(p.active_warps);  // here: warpgroups
  const bool active = v < workers;
  const int row_tile = static_cast<int>(blockIdx.y);
  const int row0 = row_tile * ROWS;
  const int m_act = (p.m - row0) < ROWS ? (p.m - row0) : ROWS;
  const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);
  const int stages = p.stages;

  const Tc5Smem plan = tc5_smem_plan(groups_per_cta, stages, G, ROWS);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_addr = smem_base + plan.barriers + (wg * (stages + 1) * 8);
  const uint32_t mma_bar = bar_addr + (stages * 8);
  const uint32_t b_addr = smem_base + plan.b_tiles + (wg * (G / 16) * kTc5StepBytes);
  const uint32_t ring_addr = smem_base + plan.rings + (wg * stages * kStride);
  float* scalars = reinterpret_cast<float*>(smem + plan.scalars) + (wg * 4 * ROWS);
  float* head_slots = reinterpret_cast<float*>(smem + plan.slots);
  volatile uint32_t* fail_flag = reinterpret_cast<volatile uint32_t*>(smem + plan.fail_flags) + wg;

  const uint32_t p_begin = active ? run_begin(v, p) : 0;
  const uint32_t p_end = active ? run_begin(v + 1, p) : 0;
  const uint32_t count = p_end - p_begin;
  const uint32_t first_tile = p_begin / num_groups;

  // ---- prologue: barriers, B tile zeroed, first copies in flight, TMEM ------------------------
  if (leader) {
    *fail_flag = 0u;
    if (active) {
      for (int s = 0; s < stages; ++s) {
        mbar_init(bar_addr + (s * 8), 1);
      }
      mbar_init(mma_bar, 1);
      mbar_init_fence();
    }
  }
  for (int i = static_cast<int>(threadIdx.x) & 127; i < (G / 16) * kTc5StepBytes / 16; i += 128) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(b_addr + (i * 16)), "r"(0u) : "memory");
  }
  proxy_fence_async();  // the tensor core reads B through the async proxy
  const uint64_t weight_policy = l2_evict_first_policy();
  uint32_t issue_idx = 0;
  int issue_slot = 0;
  auto issue_next = [&]() {
    const uint32_t bar = bar_addr + (issue_slot * 8);
    mbar_expect_tx(bar, static_cast<uint32_t>(kStride));
    bulk_copy_g2s(ring_addr + (issue_slot * kStride),
                  p.packets + (static_cast<size_t>(p_begin + issue_idx) * kStride), kStride, bar,
                  weight_policy);
    ++issue_idx;
    issue_slot = (issue_slot + 1 == stages) ? 0 : issue_slot + 1;
  };
  if (leader && active) {
    const uint32_t prefill = count < static_cast<uint32_t>(stages) ? count : stages;
    for (uint32_t j = 0; j < prefill; ++j) {
      issue_next();
    }
  }
  if (warp == 0) {
    tmem_alloc(smem_base + plan.tmem_slot, kTc5TmemColumns);
    tmem_relinquish();
  }
  // The copies above and the allocation do not depend on earlier kernels in the stream;
  // activations, outputs and scratch do.
  pdl_launch_dependents();
  pdl_wait_for_prerequisites();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem + plan.tmem_slot);
  // this thread's lane of the warpgroup's A and D columns
  const uint32_t a_tmem = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                          static_cast<uint32_t>(wg * kTc5GroupTmemColumns);
  const uint32_t d_tmem = a_tmem + 64;
  // lane 0 of the same columns, as the MMA addresses them
  const uint32_t a_mma = tmem_base + static_cast<uint32_t>(wg * kTc5GroupTmemColumns);
  const uint32_t d_mma = a_mma + 64;

  float y[ROWS];
#pragma unroll
  for (int m = 0; m < ROWS; ++m) {
    y[m] = 0.0f;
  }

  if (active) {
    const auto* act_bytes = static_cast<const uint8_t*>(p.act);
    const uint32_t first_group = p_begin - (first_tile * num_groups);

    auto on_tile_done = [&](uint32_t tile, uint32_t first_pkt, uint32_t end_pkt) {
      if ((end_pkt - first_pkt) == num_groups) {
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
          if (m < m_act) {
            store_tile_element<E>(p, row0 + m, tile, col, y[m]);
          }
        }
        return;
      }
      float* slot = head_slots + (((wg * 2) + (tile == first_tile ? 0 : 1)) * kSlotFloats);
#pragma unroll
      for (int m = 0; m < ROWS; ++m) {
        slot[(m * kTileCols) + col] = y[m];
      }
    };

    // Activation staging is one warp's job per packet, in rotation: warp `quarter` stages packets
    // j with j % 4 == quarter, and fetches their raw activations (from L2) a turn ahead.
    uint2 next_raw[ROWS];
    auto load_raw = [&](uint32_t j) {
      uint32_t group = first_group + j;
      group -= (group / num_groups) * num_groups;
#pragma unroll
      for (int m = 0; m < ROWS; ++m) {
        next_raw[m] = make_uint2(0u, 0u);
        if (m < m_act && lane < G / 4) {
          const size_t elem = (static_cast<size_t>(row0 + m) * p.k) + (static_cast<size_t>(group) * G);
          next_raw[m] = __ldg(reinterpret_cast<const uint2*>(act_bytes + (elem * 2)) + lane);
        }
      }
    };
    if (static_cast<uint32_t>(quarter) < count) {
      load_raw(static_cast<uint32_t>(quarter));
    }

    uint32_t pkt = p_begin;
    uint32_t tile = first_tile;
    uint32_t tile_end = (tile + 1) * num_groups;
    uint32_t tile_first = p_begin;
    int slot = 0;
    uint32_t parity = 0;
    uint32_t mma_parity = 0;
    float alpha_prev = 0.0f;
    float beta_prev = 0.0f;
    bool ok = true;

    // D of the packet before `j` -> y; then a finished tile -> outputs or slot
    auto fold_previous = [&](uint32_t j) {
      if (!mbar_wait_bounded(mma_bar, mma_parity)) {
        *fail_flag = 1u;
      }
      mma_parity ^= 1u;
      tc_fence_after_sync();
      float d[ROWS];
      tmem_ld<ROWS>(d_tmem, d);
      const float* sc = scalars + (((j - 1) & 1u) * 2 * ROWS);
#pragma unroll
      for (int m = 0; m < ROWS; ++m) {
        y[m] = fmaf(alpha_prev, d[m] - sc[ROWS + m], y[m]);
        y[m] = fmaf(beta_prev, sc[m], y[m]);
      }
      if (pkt == tile_end) {  // the packet before this one closed its tile
        on_tile_done(tile, tile_first, pkt);
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
          y[m] = 0.0f;
        }
        ++tile;
        tile_first = pkt;
        tile_end += num_groups;
      }
    };

    for (uint32_t j = 0; j < count; ++j, ++pkt) {
      const uint32_t stage = ring_addr + (slot * kStride);
      if (!mbar_wait_bounded(bar_addr + (slot * 8), parity)) {
        *fail_flag = 1u;
      }

      // this column's words -> A registers: column 8 s + 2 w + e of kind `first` / `second`
      uint32_t a_regs[kACols];
#pragma unroll
      for (int r = 0; r < kWordRows; ++r) {
        const NibblePairs u = Mode::unpack(lds32(stage + (r * kTileCols * 4) + (col * 4)));
        const int base = (8 * (r / 4)) + (2 * (r % 4));
        a_regs[base] = u.p04;
        a_regs[base + 1] = u.p26;
        a_regs[(8 * kStepsPerKind) + base] = u.p15;
        a_regs[(8 * kStepsPerKind) + base + 1] = u.p37;
      }
      unsigned short alpha_bits;
      unsigned short beta_bits;
      asm volatile("ld.shared.u16 %0, [%1];" : "=h"(alpha_bits) : "r"(stage + kQBytes + (col * 2)));
      asm volatile("ld.shared.u16 %0, [%1];"
                   : "=h"(beta_bits)
                   : "r"(stage + kQBytes + (kTileCols * 2) + (col * 2)));

      // the staging warp's share: pairs and sums of every row, kept in registers for now
      const bool stager = (j & 3u) == static_cast<uint32_t>(quarter);
      uint2 staged[ROWS];
      float s_sum[ROWS];
      float b_sum[ROWS];
      if (stager) {
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
          float s = 0.0f;
          float b = 0.0f;
          staged[m] = stage_pairs<G, Mode>(next_raw[m], lane, s, b);
          s_sum[m] = warp_sum(s);
          b_sum[m] = warp_sum(b);
        }
        if (j + 4 < count) {
          load_raw(j + 4);
        }
      }

      if (j > 0) {
        fold_previous(j);
      }

      // A -> TMEM, B and the group's scalars -> shared memory
#pragma unroll
      for (int c = 0; c < kACols; c += 16) {
        tmem_st16(a_tmem + c, a_regs + c);
      }
      if (stager) {
        if (lane < G / 4) {
          const int r = lane >> 1;
          const int e = lane & 1;
          const int c = (2 * (r % 4)) + e;  // 32-bit column inside the step
#pragma unroll
          for (int m = 0; m < ROWS; ++m) {
            if (m < m_act) {
              const uint32_t at = b_addr + ((r / 4) * kTc5StepBytes) + ((m / 8) * 256) +
                                  ((c / 4) * 128) + ((m % 8) * 16) + ((c % 4) * 4);
              sts32(at, staged[m].x);
              sts32(at + (kStepsPerKind * kTc5StepBytes), staged[m].y);
            }
          }
        }
        if (lane == 0) {
          float* sc = scalars + ((j & 1u) * 2 * ROWS);
#pragma unroll
          for (int m = 0; m < ROWS; ++m) {
            sc[m] = s_sum[m];
            sc[ROWS + m] = b_sum[m];
          }
        }
        proxy_fence_async();  // generic-proxy writes of B, read by the tensor core
      }
      tmem_wait_st();
      tc_fence_before_sync();
      group_barrier(wg);

      if (*fail_flag != 0u) {
        ok = false;
        break;
      }
      if (leader) {
        tc_fence_after_sync();
#pragma unroll
        for (int s = 0; s < 2 * kStepsPerKind; ++s) {
          umma_f16_ts(d_mma, a_mma + (8 * s), umma_b_desc(b_addr + (s * kTc5StepBytes)),
                      s < kStepsPerKind ? kIdescFirst : kIdescSecond, s == 0 ? 0u : 1u);
        }
        umma_commit(mma_bar);
        // every thread of the group has read this ring slot: hand it back to the copy engine
        if (issue_idx < count) {
          proxy_fence_async();
          issue_next();
        }
      }
      alpha_prev = E::to_float(alpha_bits);
      beta_prev = E::to_float(beta_bits);
      if (++slot == stages) {
        slot = 0;
        parity ^= 1u;
      }
    }

    if (ok) {
      fold_previous(count);
      group_barrier(wg);
      if (*fail_flag != 0u) {
        ok = false;
      }
    }
    if (ok) {
      if (pkt != tile_first) {
        on_tile_done(tile, tile_first, pkt);
      }
    } else {
      // A copy or an MMA never completed. Record it; give copies still in flight a bounded chance
      // to land before the shared memory is released.
      if (leader) {
        atomicExch(p.status, static_cast<int>(kStatusCopyWaitTimeout));
        for (int s = 0; s < stages; ++s) {
          (void)mbar_wait_bounded(bar_addr + (s * 8), parity);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTc5TmemColumns);
  }
  // The leading warp of each warpgroup carries the finish (run index = warpgroup).
  finish_cta<ROWS, E>(p, head_slots, 2 * kSlotFloats, head_slots + kSlotFloats, 2 * kSlotFloats,
                      quarter == 0 ? wg : (1 << 20), lane, groups_per_cta, row_tile, row0, m_act);
}

}  // namespace fk_w4a16

// Batched decode on the fifth-generation tensor cores: tcgen05.mma with both the unpacked weights
// (operand A) and the accumulators (D) in tensor memory, as a warp-specialised pipeline.
//
// Why this shape. A tcgen05.mma kind::f16 of M = 128 occupies the tensor core for ~45 clocks for
// every N up to 64 (measured on B200 by issuing 4096 of them from one thread: 44.8 clk at N = 16,
// 32 and 64; 64 clk at N = 128; 128 clk at N = 256), and a packet of group size G needs G/16 of
// them: 358 clocks per 8704-byte packet and SM, i.e. ~7 TB/s of packed weights over 148 SMs --
// above what HBM delivers, and the same for 1 row as for 16. The CUDA-core kernels pay 512 FMAs
// per packet and ROW, the mma.sync kernel is bound by instruction issue; here the multiply-adds
// leave the issue slots altogether and what remains per packet is the unpack (5 integer
// instructions per 8 weights), the staging of the group's activations and a short epilogue.
//
// Roles of a CTA (one CTA per SM, persistent over a contiguous run of the packet stream):
//   producer   1 thread   bulk-copies packets into a ring of `stages` shared-memory buffers;
//   unpackers  U x 128    packet j goes to warpgroup j % U: thread c reads the G/8 words of output
//                         column c (conflict-free 32-bit loads), turns them into "constant + q"
//                         16-bit pairs with LOP3 and stores them to tensor memory (tcgen05.st):
//                         TMEM lane c = row c of A; also hands the column's scale and offset on;
//   stagers    2 x 128    packet j goes to group j % 2: the group's activations -> operand B in shared memory (K-major core
//                         matrices, rows >= batch stay zero), in the pair formats and the
//                         k-permutation of the unpack, plus S_g = sum a and the constant term B_g;
//   issuers    2 threads  alternate packets: G/16 tcgen05.mma per packet (A from TMEM, B by
//                         descriptor, D in TMEM), then tcgen05.commit onto the packet's mbarrier;
//   epilogue   128        thread c reads row c of D (tcgen05.ld) and folds the packet into its
//                         running sums: y[m] += alpha_c * (D[m] - B_g[m]) + beta_c * S_g[m]; at a
//                         tile's end it stores the outputs or leaves a partial sum for the finish.
// A, B, D and the per-packet scalars are P-deep rings indexed by packet number, so the unpack of
// packet j + 1 ... j + P - 1, the MMAs of packet j and the epilogue of packet j - 1 overlap.
// Synchronisation is by mbarriers only (every wait bounded): full / empty per ring buffer,
// operands_ready[p] (unpackers + stagers -> issuer), mma_done[p] (commit -> epilogue, and "A, B
// are free again" for unpackers and stagers), d_free[p] (epilogue -> issuer).
//
// Operand mapping: a K = 16 step takes the
// pairs of one kind from four consecutive word-rows -- for bf16, G/32 steps of bf16 x bf16 (pairs
// (0,4), (2,6): 128 + q against the raw activation) and G/32 steps of fp16 x fp16 (pairs (1,5),
// (3,7): 1024 + 16 q against fp16(a / 16)); for fp16 all steps are of the second kind. No weight
// is converted or scaled before the MMA.
// Tile bookkeeping, split-K finish between CTAs, output placement, residual / SiLU epilogues and
// peer stores are those of the packet-stream kernel (a CTA plays the part of a warp there).
#pragma once

#include "w4a16_gemv_stream.cuh"
#include "w4a16_umma_plan.cuh"

namespace fk_w4a16 {

// ---- tcgen05 wrappers ----------------------------------------------------------------------
namespace umma {

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
__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// Row `lane` of a 128 x 16 fp32 accumulator.
__device__ __forceinline__ void ld16(uint32_t taddr, float (&d)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  wait_ld();
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    d[i] = __uint_as_float(r[i]);
  }
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]; `accumulate` = 0 overwrites D.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier receives one arrival when every MMA this thread has issued so far is complete.
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

// Instruction descriptor of tcgen05.mma kind::f16: fp32 accumulate (bits 4-5 = 1), A and B formats
// (bits 7-9 and 10-12: 0 = fp16, 1 = bf16), both operands K-major (bits 15, 16 = 0), N / 8 in bits
// 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t idesc(bool bf16) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
         (static_cast<uint32_t>(kUmmaN / 8) << 17) | (static_cast<uint32_t>(128 / 16) << 24);
}
// Shared-memory descriptor of one K = 16 step of B: K-major, no swizzle. Address, leading-dimension
// offset (between the two 16-byte K chunks: 128 B) and stride-dimension offset (between groups of
// 8 rows: 256 B) in 16-byte units at bits 0-13, 16-29, 32-45; descriptor version 1 at bit 46.
__device__ __forceinline__ uint64_t b_desc(uint32_t smem_address) {
  return static_cast<uint64_t>((smem_address & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 16) |
         (static_cast<uint64_t>(256 >> 4) << 32) | (uint64_t{1} << 46);
}

}  // namespace umma

// Optional per-packet timeline for tuning builds (-DFK_W4A16_UMMA_TRACE): CTA 0 records the SM clock
// at eight milestones of its first 96 packets. Compiled out of the shipped library.
#ifdef FK_W4A16_UMMA_TRACE
constexpr int kUmmaTracePackets = 96;
__device__ long long g_umma_trace[kUmmaTracePackets * 8];
__device__ __forceinline__ void umma_trace(uint32_t j, int what, bool elected) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && elected && j < kUmmaTracePackets) {
#ifdef FK_W4A16_UMMA_TRACE_STAGER
    if (what < 8) return;
    what -= 8;
#else
    if (what >= 8) return;
#endif
    g_umma_trace[(j * 8) + what] = clock64();
  }
}
#else
__device__ __forceinline__ void umma_trace(uint32_t, int, bool) {}
#endif

// Phase parity of the `use`-th completion (0, 1, 2, ...) of an mbarrier.
__device__ __forceinline__ uint32_t use_parity(uint32_t use) { return use & 1u; }

template <int G, int ROWS, class Mode>
__global__ void __launch_bounds__(kUmmaThreads, 1)
    w4a16_gemm_umma_kernel(const __grid_constant__ GemvParams p) {
  using E = typename Mode::Elem;
  static_assert(ROWS == 1 || ROWS == 2 || ROWS == 4 || ROWS == 8 || ROWS == 16, "rows per pass");
  constexpr int kStride = packet_stride(G);
  constexpr int kQBytes = packet_q_bytes(G);
  constexpr int kWordRows = G / 8;
  constexpr int kStepsPerKind = G / 32;            // K = 16 steps of each pair kind
  constexpr int kSteps = 2 * kStepsPerKind;
  constexpr int kACols = G / 2;                    // TMEM columns of one A buffer
  constexpr int kChunkRows = kWordRows < 8 ? kWordRows : 8;  // word-rows unpacked per tcgen05.st pair
  constexpr int kChunks = kWordRows / kChunkRows;
  constexpr int kKChunks = G / 16;                 // 16-k chunks per batch row (one per stager thread)
  constexpr int kSlotFloats = ROWS * kTileCols;
  constexpr int P = kUmmaDepth;
  constexpr uint32_t kIdescFirst = umma::idesc(Mode::kEvenNibblesBf16);
  constexpr uint32_t kIdescSecond = umma::idesc(false);
  extern __shared__ __align__(128) uint8_t smem[];

  const int tid = static_cast<int>(threadIdx.x);
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const uint32_t cta = blockIdx.x;
  const uint32_t workers = static_cast<uint32_t>(p.active_warps);  // here: CTAs
  const bool active = cta < workers;
  const int row_tile = static_cast<int>(blockIdx.y);
  const int row0 = row_tile * ROWS;
  const int m_act = (p.m - row0) < ROWS ? (p.m - row0) : ROWS;
  const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);
  const int stages = p.stages;

  const UmmaSmem plan = umma_smem_plan(stages, G, ROWS);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t full_bar = smem_base + plan.barriers;                 // [stages]
  const uint32_t empty_bar = full_bar + (stages * 8);                  // [stages]
  const uint32_t ready_bar = empty_bar + (stages * 8);                 // [P] operands ready
  const uint32_t done_bar = ready_bar + (P * 8);                       // [P] MMAs complete
  const uint32_t dfree_bar = done_bar + (P * 8);                       // [P] D read out
  const uint32_t b_addr = smem_base + plan.b_tiles;                    // [P][G/16 steps][512]
  const uint32_t ring_addr = smem_base + plan.rings;
  // Written for packet j + 2P only after the MMAs of packet j + P are complete, which the issuer
  // starts only after the epilogue has read packet j's entries: rings of 2P need no barrier.
  volatile float* scalars = reinterpret_cast<volatile float*>(smem + plan.scalars);  // [2P][2][ROWS]
  volatile uint32_t* scales = reinterpret_cast<volatile uint32_t*>(smem + plan.scales);  // [2P][128]
  float* slots = reinterpret_cast<float*>(smem + plan.slots);          // [2][ROWS][128]
  volatile uint32_t* fail_flag = reinterpret_cast<volatile uint32_t*>(smem + plan.fail_flag);

  const uint32_t p_begin = active ? run_begin(cta, p) : 0;
  const uint32_t p_end = active ? run_begin(cta + 1, p) : 0;
  const uint32_t count = p_end - p_begin;
  const uint32_t first_tile = p_begin / num_groups;
  const uint32_t first_group = p_begin - (first_tile * num_groups);

  // ---- prologue ------------------------------------------------------------------------------
  if (tid == 0) {
    *fail_flag = 0u;
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar + (s * 8), 1);
      mbar_init(empty_bar + (s * 8), kUmmaUnpackGroups > 1 ? 4 : 4);  // the 4 warps of the unpacking group
    }
    // stager warps that hold at least one batch row (the others have nothing to do and leave)
    const int stager_warps = ((m_act * kKChunks) + 31) / 32;
    for (int i = 0; i < P; ++i) {
      mbar_init(ready_bar + (i * 8), 4 + stager_warps);  // unpacker warps + working stager warps
      mbar_init(done_bar + (i * 8), 1);   // tcgen05.commit
      mbar_init(dfree_bar + (i * 8), 4);  // 4 epilogue warps
    }
    mbar_init_fence();
  }
  // B buffers start (and, in rows >= batch, stay) zero
  for (int i = tid; i < (P * kSteps * kUmmaStepBytes) / 16; i += kUmmaThreads) {
    umma::sts128(b_addr + (i * 16), 0u, 0u, 0u, 0u);
  }
  proxy_fence_async();  // the tensor core reads B through the async proxy
  if (warp == kUmmaIssuerWarp) {
    umma::tmem_alloc(smem_base + plan.tmem_slot, kUmmaTmemColumns);
    umma::tmem_relinquish();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem + plan.tmem_slot);

  const uint64_t weight_policy = l2_evict_first_policy();
  auto issue_copy = [&](uint32_t j) {
    const uint32_t s = j % static_cast<uint32_t>(stages);
    mbar_expect_tx(full_bar + (s * 8), static_cast<uint32_t>(kStride));
    bulk_copy_g2s(ring_addr + (s * kStride), p.packets + (static_cast<size_t>(p_begin + j) * kStride),
                  kStride, full_bar + (s * 8), weight_policy);
  };
  // The first ring-full of weight copies does not depend on earlier work in the stream.
  uint32_t issued = 0;
  if (warp == kUmmaProducerWarp && lane == 0 && active) {
    const uint32_t prefill = count < static_cast<uint32_t>(stages) ? count : stages;
    for (; issued < prefill; ++issued) {
      issue_copy(issued);
    }
  }
  pdl_launch_dependents();
  pdl_wait_for_prerequisites();

  auto failed = [&]() -> bool { return *fail_flag != 0u; };
  auto give_up = [&]() {
    *fail_flag = 1u;
    atomicExch(p.status, static_cast<int>(kStatusCopyWaitTimeout));
  };

  if (active && warp == kUmmaProducerWarp) {
    // ---- producer --------------------------------------------------------------------------
    if (lane == 0) {
      for (uint32_t j = issued; j < count && !failed(); ++j) {
        const uint32_t s = j % static_cast<uint32_t>(stages);
        const uint32_t use = j / static_cast<uint32_t>(stages);  // >= 1 here
        if (!mbar_wait_parked(empty_bar + (s * 8), use_parity(use - 1))) {
          give_up();
          break;
        }
        proxy_fence_async();
        issue_copy(j);
        issued = j + 1;
      }
    }
  } else if (active && (warp == kUmmaIssuerWarp || warp == kUmmaIssuerWarp + 1)) {
    // ---- MMA issuers ------------------------------------------------------------------------
    // Two threads (of two warps) take alternate packets. Issuing a packet's MMAs holds a thread
    // until the tensor core has taken them in, and the waits for the next packet's operands cost
    // it a few hundred clocks more even when they are long satisfied; with two issuers one waits
    // while the other feeds the tensor core. Every instruction between two MMAs is time the
    // tensor core may idle, so the descriptors are derived from the first one by constants.
    if (lane == 0) {
      const uint32_t first = static_cast<uint32_t>(warp - kUmmaIssuerWarp);
      const uint64_t b_desc0 = umma::b_desc(b_addr);
      constexpr uint64_t kDescStep = kUmmaStepBytes >> 4;
      for (uint32_t j = first; j < count; j += 2) {
        const uint32_t slot = j % P;
        const uint32_t use = j / P;
#ifdef FK_W4A16_UMMA_TRACE_ISSUER
        umma_trace(j, 6, true);
#endif
        if (!mbar_wait_parked(ready_bar + (slot * 8), use_parity(use))) {
          give_up();
          break;
        }
#ifdef FK_W4A16_UMMA_TRACE_ISSUER
        umma_trace(j, 7, true);
#endif
        if (use > 0 && !mbar_wait_parked(dfree_bar + (slot * 8), use_parity(use - 1))) {
          give_up();
          break;
        }
        umma::fence_after_sync();
        umma_trace(j, 2, true);
        const uint32_t a_tmem = tmem_base + (slot * kACols);
        const uint32_t d_tmem = tmem_base + kUmmaDColumn0 + (slot * kUmmaN);
        const uint64_t b_desc = b_desc0 + (static_cast<uint64_t>(slot * kSteps) * kDescStep);
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
          umma::mma_f16_ts(d_tmem, a_tmem + (8 * s), b_desc + (s * kDescStep),
                           s < kStepsPerKind ? kIdescFirst : kIdescSecond, s == 0 ? 0u : 1u);
        }
        umma::commit(done_bar + (slot * 8));
#ifdef FK_W4A16_UMMA_TRACE_ISSUER
        umma_trace(j, 3, true);
#endif
      }
    }
  } else if (active && warp >= kUmmaFirstUnpackWarp && warp < kUmmaFirstUnpackWarp + (4 * kUmmaUnpackGroups)) {
    // ---- unpackers ---------------------------------------------------------------------------
    const int wg = (warp - kUmmaFirstUnpackWarp) >> 2;
    const int quarter = warp & 3;  // this warp reaches TMEM lanes 32 * quarter .. + 31
    const int col = (quarter * 32) + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    for (uint32_t j = static_cast<uint32_t>(wg); j < count; j += kUmmaUnpackGroups) {
      if (failed()) {
        break;
      }
      const uint32_t slot = j % P;
      const uint32_t use = j / P;
      const uint32_t s = j % static_cast<uint32_t>(stages);
      const uint32_t stage = ring_addr + (s * kStride);
      bool ok = mbar_wait_parked(full_bar + (s * 8), use_parity(j / static_cast<uint32_t>(stages)));
      // the A buffer is free once the MMAs of the packet that used it last are complete
      if (ok && use > 0) {
        ok = mbar_wait_parked(done_bar + (slot * 8), use_parity(use - 1));
      }
      if (!ok) {
        give_up();
        break;
      }
      umma::fence_after_sync();
      umma_trace(j, 0, warp == kUmmaFirstUnpackWarp + (4 * wg) && lane == 0);
      const uint32_t a_tmem = lane_base + (slot * kACols);
#pragma unroll
      for (int chunk = 0; chunk < kChunks; ++chunk) {
        uint32_t first[2 * kChunkRows];
        uint32_t second[2 * kChunkRows];
#pragma unroll
        for (int i = 0; i < kChunkRows; ++i) {
          const int r = (chunk * kChunkRows) + i;
          const NibblePairs u = Mode::unpack(umma::lds32(stage + (r * kTileCols * 4) + (col * 4)));
          first[2 * i] = u.p04;
          first[(2 * i) + 1] = u.p26;
          second[2 * i] = u.p15;
          second[(2 * i) + 1] = u.p37;
        }
        // column 8 (r / 4) + 2 (r % 4) + e of the kind's half == 2 r + e: chunks are contiguous
        if constexpr (kChunkRows == 8) {
          umma::st16(a_tmem + (chunk * 16), first);
          umma::st16(a_tmem + (8 * kStepsPerKind) + (chunk * 16), second);
        } else {
          umma::st8(a_tmem + (chunk * 8), first);
          umma::st8(a_tmem + (8 * kStepsPerKind) + (chunk * 8), second);
        }
      }
      unsigned short alpha_bits;
      unsigned short beta_bits;
      asm volatile("ld.shared.u16 %0, [%1];" : "=h"(alpha_bits) : "r"(stage + kQBytes + (col * 2)));
      asm volatile("ld.shared.u16 %0, [%1];"
                   : "=h"(beta_bits)
                   : "r"(stage + kQBytes + (kTileCols * 2) + (col * 2)));
      scales[((j % (2 * P)) * kTileCols) + col] =
          static_cast<uint32_t>(alpha_bits) | (static_cast<uint32_t>(beta_bits) << 16);
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        umma::mbar_arrive(empty_bar + (s * 8));   // every lane of this warp has read the buffer
        umma::mbar_arrive(ready_bar + (slot * 8));
      }
      umma_trace(j, 1, warp == kUmmaFirstUnpackWarp + (4 * wg) && lane == 0);
    }
  } else if (active && warp >= kUmmaFirstStagerWarp &&
             warp < kUmmaFirstStagerWarp + (4 * kUmmaStagerGroups) &&
             ((warp - kUmmaFirstStagerWarp) & 3) * 32 < m_act * kKChunks) {
    // ---- stagers -----------------------------------------------------------------------------
    // Packet j goes to stager group j % 2. Within a group, thread t: batch row t / (G/16),
    // k-chunk t % (G/16) = word-rows 2 ch, 2 ch + 1 of the packet's quantisation group.
    const int stager_group = (warp - kUmmaFirstStagerWarp) >> 2;
    const int t = (tid - (kUmmaFirstStagerWarp * 32)) & 127;
    const int m = t / kKChunks;
    const int ch = t % kKChunks;
    const bool has_row = m < m_act;
    const auto* act_row = static_cast<const uint8_t*>(p.act) +
                          (static_cast<size_t>(row0 + (has_row ? m : 0)) * p.k * 2) + (ch * 32);
    // The raw activations come from L2 (several hundred clocks away) and a packet lasts about as
    // long, so they are fetched kAhead packets ahead into a small register queue.
    constexpr int kAhead = 2;
    uint4 queue_lo[kAhead];
    uint4 queue_hi[kAhead];
    uint32_t group = (first_group + static_cast<uint32_t>(stager_group)) % num_groups;
    auto load_raw = [&](uint4& lo, uint4& hi) {
      lo = make_uint4(0u, 0u, 0u, 0u);
      hi = make_uint4(0u, 0u, 0u, 0u);
      if (has_row) {
        const auto* src = reinterpret_cast<const uint4*>(act_row + (static_cast<size_t>(group) * G * 2));
        lo = __ldg(src);
        hi = __ldg(src + 1);
      }
      group += kUmmaStagerGroups;
      group = group >= num_groups ? (group - num_groups) % num_groups : group;
    };
    // this group's packets: j = stager_group + 2 i
    const uint32_t my_count = count > static_cast<uint32_t>(stager_group)
                                  ? (count - stager_group + kUmmaStagerGroups - 1) / kUmmaStagerGroups
                                  : 0u;
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      queue_lo[i] = make_uint4(0u, 0u, 0u, 0u);
      queue_hi[i] = make_uint4(0u, 0u, 0u, 0u);
      if (static_cast<uint32_t>(i) < my_count) {
        load_raw(queue_lo[i], queue_hi[i]);
      }
    }
    // Queue entry i serves packets i, i + kAhead, ...: the loop is unrolled kAhead times so that
    // every entry is a fixed set of registers (shifting entries would make each iteration wait
    // for the load the previous one issued).
    for (uint32_t i0 = 0; i0 < my_count && !failed(); i0 += kAhead) {
#pragma unroll
      for (int qi = 0; qi < kAhead; ++qi) {
      const uint32_t mine = i0 + static_cast<uint32_t>(qi);
      if (mine >= my_count || failed()) {
        break;
      }
      const uint32_t j = (mine * kUmmaStagerGroups) + static_cast<uint32_t>(stager_group);
      umma_trace(j, 8, t == 0);
      const uint32_t slot = j % P;
      const uint32_t use = j / P;
      const uint4 lo = queue_lo[qi];
      const uint4 hi = queue_hi[qi];
      if (mine + kAhead < my_count) {
        load_raw(queue_lo[qi], queue_hi[qi]);
      }
      umma_trace(j, 9, t == 0);
      // pairs of this thread's two word-rows, in the formats the unpack mode multiplies with
      float s_sum = 0.0f;
      float b_sum = 0.0f;
      uint32_t first[4];
      uint32_t second[4];
      auto stage_row = [&](const uint4& v, int i) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float f[8];
        uint32_t h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          f[e] = E::to_float(static_cast<unsigned short>((w[e >> 1] >> ((e & 1) * 16)) & 0xffffu));
          h[e] = Mode::stage(f[e], (e & 1) != 0, b_sum);
        }
        s_sum += ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
        first[2 * i] = h[0] | (h[4] << 16);         // (a0, a4)
        first[(2 * i) + 1] = h[2] | (h[6] << 16);   // (a2, a6)
        second[2 * i] = h[1] | (h[5] << 16);        // (a1, a5)
        second[(2 * i) + 1] = h[3] | (h[7] << 16);  // (a3, a7)
      };
      if (has_row) {
        stage_row(lo, 0);
        stage_row(hi, 1);
      }
      // sum over the row's G/16 threads (neighbouring lanes)
#pragma unroll
      for (int off = kKChunks / 2; off > 0; off >>= 1) {
        s_sum += __shfl_xor_sync(0xffffffffu, s_sum, off);
        b_sum += __shfl_xor_sync(0xffffffffu, b_sum, off);
      }
      umma_trace(j, 10, t == 0);
      // the B buffer is free once the MMAs of the packet that used it last are complete
      if (use > 0 && !mbar_wait_parked(done_bar + (slot * 8), use_parity(use - 1))) {
        give_up();
        break;
      }
#ifndef FK_W4A16_UMMA_TRACE_ISSUER
      umma_trace(j, 6, t == 0);
#endif
      umma_trace(j, 11, t == 0);
      if (has_row) {
        // word-rows 2 ch and 2 ch + 1 sit in step ch / 2, 16-byte K chunk ch % 2, columns {0,1} {2,3}
        const uint32_t at = b_addr + (slot * kSteps * kUmmaStepBytes) + ((ch >> 1) * kUmmaStepBytes) +
                            ((m >> 3) * 256) + ((ch & 1) * 128) + ((m & 7) * 16);
        umma::sts128(at, first[0], first[1], first[2], first[3]);
        umma::sts128(at + (kStepsPerKind * kUmmaStepBytes), second[0], second[1], second[2], second[3]);
        if (ch == 0) {
          scalars[((j % (2 * P)) * 2 * ROWS) + m] = s_sum;
          scalars[((j % (2 * P)) * 2 * ROWS) + ROWS + m] = b_sum;
        }
        umma_trace(j, 12, t == 0);
        proxy_fence_async();  // generic-proxy writes of B, read by the tensor core
      }
      umma_trace(j, 13, t == 0);
      __syncwarp();
      if (lane == 0) {
        umma::mbar_arrive(ready_bar + (slot * 8));
      }
      umma_trace(j, 14, t == 0);
#ifndef FK_W4A16_UMMA_TRACE_ISSUER
      umma_trace(j, 7, t == 0);
#endif
      }
    }
  } else if (active && warp >= kUmmaFirstEpilogueWarp && warp < kUmmaFirstEpilogueWarp + 4) {
    // ---- epilogue ----------------------------------------------------------------------------
    const int quarter = warp & 3;
    const int col = (quarter * 32) + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float y[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
      y[m] = 0.0f;
    }
    uint32_t pkt = p_begin;
    uint32_t tile = first_tile;
    uint32_t tile_end = (tile + 1) * num_groups;
    uint32_t tile_first = p_begin;
    auto on_tile_done = [&](uint32_t first_pkt, uint32_t end_pkt) {
      if ((end_pkt - first_pkt) == num_groups) {
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
          if (m < m_act) {
            store_tile_element<E>(p, row0 + m, tile, col, y[m]);
          }
        }
        return;
      }
      float* slot = slots + ((tile == first_tile ? 0 : 1) * kSlotFloats);
#pragma unroll
      for (int m = 0; m < ROWS; ++m) {
        slot[(m * kTileCols) + col] = y[m];
      }
    };
    bool ok = true;
    for (uint32_t j = 0; j < count; ++j, ++pkt) {
      if (failed()) {
        ok = false;
        break;
      }
      const uint32_t slot = j % P;
      const uint32_t use = j / P;
      if (!mbar_wait_parked(done_bar + (slot * 8), use_parity(use))) {
        give_up();
        ok = false;
        break;
      }
      umma::fence_after_sync();
      umma_trace(j, 4, warp == kUmmaFirstEpilogueWarp && lane == 0);
      float d[16];
      umma::ld16(lane_base + kUmmaDColumn0 + (slot * kUmmaN), d);
      const uint32_t ab = scales[((j % (2 * P)) * kTileCols) + col];
      // D is in registers: the slot may be reused
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        umma::mbar_arrive(dfree_bar + (slot * 8));
      }
      const float alpha = E::to_float(static_cast<unsigned short>(ab & 0xffffu));
      const float beta = E::to_float(static_cast<unsigned short>(ab >> 16));
      // y[m] += alpha * (D[m] - B_g[m]) + beta * S_g[m]; the per-row scalars come in vectors of 4
      // (their ring is 2P deep, so they outlive the slot)
      const uint32_t sc_addr = smem_base + plan.scalars + ((j % (2 * P)) * 2 * ROWS * 4);
      if constexpr (ROWS >= 4) {
#pragma unroll
        for (int m4 = 0; m4 < ROWS; m4 += 4) {
          const uint4 s4 = lds128(sc_addr + (m4 * 4));
          const uint4 b4 = lds128(sc_addr + ((ROWS + m4) * 4));
          const float sg[4] = {__uint_as_float(s4.x), __uint_as_float(s4.y), __uint_as_float(s4.z), __uint_as_float(s4.w)};
          const float bg[4] = {__uint_as_float(b4.x), __uint_as_float(b4.y), __uint_as_float(b4.z), __uint_as_float(b4.w)};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            y[m4 + i] = fmaf(alpha, d[m4 + i] - bg[i], y[m4 + i]);
            y[m4 + i] = fmaf(beta, sg[i], y[m4 + i]);
          }
        }
      } else {
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
          y[m] = fmaf(alpha, d[m] - scalars[((j % (2 * P)) * 2 * ROWS) + ROWS + m], y[m]);
          y[m] = fmaf(beta, scalars[((j % (2 * P)) * 2 * ROWS) + m], y[m]);
        }
      }
      umma_trace(j, 5, warp == kUmmaFirstEpilogueWarp && lane == 0);
      if (pkt + 1 == tile_end) {
        on_tile_done(tile_first, pkt + 1);
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
          y[m] = 0.0f;
        }
        ++tile;
        tile_first = pkt + 1;
        tile_end += num_groups;
      }
    }
    if (ok && pkt != tile_first) {
      on_tile_done(tile_first, pkt);
    }
  }

  // ---- wind-down -------------------------------------------------------------------------------
  umma::fence_before_sync();
  __syncthreads();
  if (*fail_flag != 0u && warp == kUmmaProducerWarp && lane == 0) {
    // A wait gave up. Give the copies still in flight a bounded chance to land before this CTA's
    // shared memory is handed to another one.
    for (uint32_t j = 0; j < issued; ++j) {
      const uint32_t s = j % static_cast<uint32_t>(stages);
      if (j + static_cast<uint32_t>(stages) >= issued) {  // the last copy into each buffer
        (void)mbar_wait_bounded(full_bar + (s * 8), use_parity(j / static_cast<uint32_t>(stages)));
      }
    }
  }
  if (warp == kUmmaIssuerWarp) {
    umma::fence_after_sync();
    umma::tmem_dealloc(tmem_base, kUmmaTmemColumns);
  }
  // The first epilogue warp carries the CTA's finish (run index = CTA).
  finish_cta<ROWS, E>(p, slots, 2 * kSlotFloats, slots + kSlotFloats, 2 * kSlotFloats,
                      warp == kUmmaFirstEpilogueWarp ? 0 : (1 << 20), lane, 1, row_tile, row0, m_act);
}

}  // namespace fk_w4a16

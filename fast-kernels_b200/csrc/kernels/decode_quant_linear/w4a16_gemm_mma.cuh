// Batched decode, 5 <= M <= 16 rows per pass: the same packet stream, ring, split-K finish and
// launch plan as the M <= 4 GEMV (w4a16_gemv_stream.cuh), with the inner product on the tensor
// cores -- at this batch size the contraction is dense enough that CUDA-core FMAs (8 per word per
// batch row) would be the bottleneck, while one mma.sync.m16n8k16 covers 16 weights x 8 batch rows.
//
// Operand mapping. The MMA computes out^T: A = weights (16 output columns x 16 k), B =
// activations (16 k x 8 batch rows), D = 16 columns x 8 rows, fp32. Lane (g = lane / 4,
// t = lane % 4) holds, per the m16n8k16 fragment layout, A rows g and g+8 at k-slots
// {2t, 2t+1, 2t+8, 2t+9} and B column g at the same k-slots. Which real k a slot means is free as
// long as A and B agree, so lane t takes one whole 32-bit weight word per column (8 real k) and
// spends it on TWO k-steps: the unpack's pairs (nibbles i, i+4) are already MMA register pairs,
//     k-step 0:  {a0,a2} = pairs (0,4) (2,6) of the word,   k-step 1:  {a0,a2} = pairs (1,5) (3,7)
// and B's registers are the matching pairs of the staged activations (one 128-bit load serves both
// steps). No weight is ever converted: the A registers are the "constant + q" 16-bit floats the
// LOP3 unpack produces; the constant is removed per group exactly as in the GEMV, except that B_g
// and S_g come out of the MMA too, from one extra "column" whose weights are all-constant.
//   * bf16: k-step 0 is a bf16 MMA (128 + q against the raw bf16 activation), k-step 1 an fp16 MMA
//     (1024 + 16 q against fp16(a / 16)); fp16: both steps are fp16 MMAs in the 1024 + 16 q form.
// Column mapping. A warp's 128 columns form 8 MMA tiles: tile (s, j), s in {0,1}, j in 0..3, holds
// columns 64 s + 4 rho + j for MMA row rho, so that one 128-bit load (4 adjacent columns of one
// word-row) feeds row rho of four tiles.
//
// Shared-memory layout of a stage (bank-conflict free for those loads): the packet's G/8 word-rows
// are copied as 4 chunks of G/32 rows, chunk c (lane t = c reads it) at c * (chunk bytes + 32);
// scales ride behind the last chunk; the M activations of the group, pre-staged by a small prepass
// kernel into [group][row][pitch] with pitch = 20/12/4 x 16 B for G = 128/64/32, follow.
#pragma once

#include "w4a16_gemv_stream.cuh"

namespace fk_w4a16 {

template <int G, int MT>
struct MmaGeom {
  static constexpr int kChunkRows = G / 32;                 // word-rows per chunk
  static constexpr int kChunkBytes = kChunkRows * kTileCols * 4;
  static constexpr int kChunkPitch = kChunkBytes + 32;
  static constexpr int kScaleOffset = (3 * kChunkPitch) + kChunkBytes;
  static constexpr int kActOffset = kScaleOffset + kScaleBytes;
  static constexpr int kActRowUnits = G / 8;                // 16-byte units per batch row
  static constexpr int kActPitch = (kActRowUnits + ((12 - (kActRowUnits % 8)) % 8)) * 16;
  static constexpr int kActBytes = MT * kActPitch;
  static constexpr int kStageBytes = kActOffset + kActBytes;
  static constexpr int kSlotFloats = MT * kTileCols;
};

__host__ __device__ constexpr int mma_act_pitch(int group) {
  return ((group / 8) + ((12 - ((group / 8) % 8)) % 8)) * 16;
}

// Prepass: act[batch, k] -> staged[row_tile][group][MT][pitch] in the pair formats of the unpack
// mode, 16-byte unit (4 b + t) of a row holding word-row t * (G/32) + b. Rows beyond `batch` are
// zero. One warp per (row tile, group, row). Launched with programmatic stream serialisation: it
// lets the GEMM behind it start its weight copies at once, and itself waits for the work ahead of
// it (which may produce the activations, or still read the staging area) before it touches either.
struct StageMmaParams {
  const uint16_t* act;
  uint8_t* staged;
  int batch;
  int k;
  int num_groups;
  int mt;
  long long total_items;
};
template <int G, class Mode>
__global__ void __launch_bounds__(128) stage_activations_mma_kernel(
    const __grid_constant__ StageMmaParams sp) {
  constexpr int kChunkRows = G / 32;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const long long item = (static_cast<long long>(blockIdx.x) * 4) + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait_for_prerequisites();
  if (item >= sp.total_items) {
    return;
  }
  const int m = static_cast<int>(item % sp.mt);
  const long long rest = item / sp.mt;
  const int group = static_cast<int>(rest % sp.num_groups);
  const long long row_tile = rest / sp.num_groups;
  const long long row = (row_tile * sp.mt) + m;
  uint2 raw = make_uint2(0u, 0u);
  if (row < sp.batch && lane < G / 4) {
    raw = __ldg(reinterpret_cast<const uint2*>(sp.act + (row * sp.k) + (static_cast<long long>(group) * G)) + lane);
  }
  float s = 0.0f;
  float b = 0.0f;
  const uint2 pairs = stage_pairs<G, Mode>(raw, lane, s, b);
  if (lane < G / 4) {
    const int word_row = lane >> 1;
    const int unit = (4 * (word_row % kChunkRows)) + (word_row / kChunkRows);
    uint8_t* dst = sp.staged + (item * mma_act_pitch(G)) + (unit * 16) + ((lane & 1) * 8);
    *reinterpret_cast<uint2*>(dst) = pairs;
  }
}

struct MmaParams {
  GemvParams base;
  const uint8_t* staged;  // [row_tiles][num_groups][MT][pitch]
};

__device__ __forceinline__ uint32_t word_of(const uint4& v, int j) {
  return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}

// One k-block's worth of MMAs for one accumulator tile: the even-nibble step and the odd-nibble
// step. `lo` / `hi` are the unpacked words of MMA rows g and g + 8, `b` the staged activations.
template <class Mode>
__device__ __forceinline__ void mma_word_pair(float (&d)[4], const NibblePairs& lo,
                                              const NibblePairs& hi, const uint4& b) {
  if (Mode::kEvenNibblesBf16) {
    mma_16816_bf16(d, lo.p04, hi.p04, lo.p26, hi.p26, b.x, b.z);
  } else {
    mma_16816_f16(d, lo.p04, hi.p04, lo.p26, hi.p26, b.x, b.z);
  }
  mma_16816_f16(d, lo.p15, hi.p15, lo.p37, hi.p37, b.y, b.w);
}

// Two warps share every packet: warp `side` (0 / 1) of a pair owns columns 64 side .. 64 side + 63
// (MMA tiles 4 side .. 4 side + 3). That halves the accumulator registers per thread, so that 16
// warps fit on an SM -- with fewer, the schedulers run dry between MMAs. The pair owns one ring;
// side 0's lane 0 issues the copies, and a 64-thread named barrier per packet hands a consumed
// buffer back.
__device__ __forceinline__ void pair_barrier(int pair) {
  asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
}

template <int G, int MT, class Mode>
__global__ void __launch_bounds__(512, 1)
    w4a16_gemm_mma_kernel(const __grid_constant__ MmaParams mp) {
  using E = typename Mode::Elem;
  using Geom = MmaGeom<G, MT>;
  constexpr int H = MT / 8;  // batch halves of 8 rows
  constexpr int kStride = packet_stride(G);
  extern __shared__ __align__(128) uint8_t smem[];

  const GemvParams& p = mp.base;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int pair = warp >> 1;
  const int side = warp & 1;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int pairs_per_cta = static_cast<int>(blockDim.x) >> 6;
  const uint32_t v = (blockIdx.x * pairs_per_cta) + pair;
  const uint32_t workers = static_cast<uint32_t>(p.active_warps);  // here: number of pairs
  const bool active = v < workers;
  const int row_tile = static_cast<int>(blockIdx.y);
  const int row0 = row_tile * MT;
  const int m_act = (p.m - row0) < MT ? (p.m - row0) : MT;
  const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);
  const int stages = p.stages;

  // shared memory: barriers | one slot per pair [MT][128] | rings
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_addr = smem_base + (pair * stages * 8);
  const uint32_t slots_off = ((static_cast<uint32_t>(pairs_per_cta) * stages * 8) + 127u) & ~127u;
  const uint32_t rings_off = slots_off + (static_cast<uint32_t>(pairs_per_cta) * Geom::kSlotFloats * 4);
  float* head_slots = reinterpret_cast<float*>(smem + slots_off);
  const uint32_t ring_stride = static_cast<uint32_t>(stages) * Geom::kStageBytes;
  const uint32_t ring_addr = smem_base + rings_off + (pair * ring_stride);
  float* tail_slots = reinterpret_cast<float*>(smem + rings_off);

  const uint32_t p_begin = active ? run_begin(v, p) : 0;
  const uint32_t p_end = active ? run_begin(v + 1, p) : 0;
  const uint32_t count = p_end - p_begin;
  const uint32_t first_tile = p_begin / num_groups;
  const uint8_t* staged = mp.staged + (static_cast<size_t>(row_tile) * num_groups * Geom::kActBytes);
  const bool issuer = side == 0 && lane == 0;

  if (active) {
    if (issuer) {
      for (int s = 0; s < stages; ++s) {
        mbar_init(bar_addr + (s * 8), 1);
      }
      mbar_init_fence();
    }
    const uint64_t weight_policy = l2_evict_first_policy();
    const uint64_t act_policy = l2_evict_last_policy();

    uint32_t issue_idx = 0;
    uint32_t issue_group = p_begin - (first_tile * num_groups);
    int issue_slot = 0;
    auto issue_weights = [&](uint32_t idx, int slot) {
      const uint32_t bar = bar_addr + (slot * 8);
      const uint32_t dst = ring_addr + (slot * Geom::kStageBytes);
      const uint8_t* src = p.packets + (static_cast<size_t>(p_begin + idx) * kStride);
      mbar_expect_tx(bar, static_cast<uint32_t>(kStride + Geom::kActBytes));
#pragma unroll
      for (int c = 0; c < 3; ++c) {
        bulk_copy_g2s(dst + (c * Geom::kChunkPitch), src + (c * Geom::kChunkBytes), Geom::kChunkBytes,
                      bar, weight_policy);
      }
      bulk_copy_g2s(dst + (3 * Geom::kChunkPitch), src + (3 * Geom::kChunkBytes),
                    Geom::kChunkBytes + kScaleBytes, bar, weight_policy);
    };
    auto issue_acts = [&](uint32_t group, int slot) {
      bulk_copy_g2s(ring_addr + (slot * Geom::kStageBytes) + Geom::kActOffset,
                    staged + (static_cast<size_t>(group) * Geom::kActBytes), Geom::kActBytes,
                    bar_addr + (slot * 8), act_policy);
    };
    const uint32_t prefill = count < static_cast<uint32_t>(stages) ? count : stages;
    if (issuer) {
      for (uint32_t j = 0; j < prefill; ++j) {
        issue_weights(j, static_cast<int>(j));
      }
    }
    // Weights do not depend on earlier kernels in the stream; the staged activations do.
    pdl_launch_dependents();
    pdl_wait_for_prerequisites();
    if (issuer) {
      for (uint32_t j = 0; j < prefill; ++j) {
        issue_acts(issue_group, static_cast<int>(j));
        issue_group = (issue_group + 1 == num_groups) ? 0 : issue_group + 1;
      }
      issue_idx = prefill;
      issue_slot = (prefill == static_cast<uint32_t>(stages)) ? 0 : static_cast<int>(prefill);
    }
    pair_barrier(pair);  // the partner may not wait on barriers that are not initialised yet

    float y[4][H][4];
#pragma unroll
    for (int tile = 0; tile < 4; ++tile) {
#pragma unroll
      for (int h = 0; h < H; ++h) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          y[tile][h][c] = 0.0f;
        }
      }
    }

    // y element (tile j, h, c): column 64 side + 4 (g + 8 (c >> 1)) + j, row 8 h + 2 t + (c & 1)
    auto on_tile_done = [&](uint32_t tile_index, uint32_t first_pkt, uint32_t end_pkt) {
      const bool full = (end_pkt - first_pkt) == num_groups;
      float* slot = (tile_index == first_tile) ? head_slots + (pair * Geom::kSlotFloats)
                                               : tail_slots + (pair * (ring_stride / 4));
#pragma unroll
      for (int tile = 0; tile < 4; ++tile) {
#pragma unroll
        for (int h = 0; h < H; ++h) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int col = (64 * side) + (4 * (g + (8 * (c >> 1)))) + tile;
            const int row = (8 * h) + (2 * t) + (c & 1);
            if (!full) {
              slot[(row * kTileCols) + col] = y[tile][h][c];
            } else if (row < m_act) {
              store_tile_element<E>(p, row0 + row, tile_index, col, y[tile][h][c]);
            }
          }
        }
      }
    };

    uint32_t pkt = p_begin;
    uint32_t tile_index = first_tile;
    uint32_t tile_end = (tile_index + 1) * num_groups;
    uint32_t tile_first = p_begin;
    int slot = 0;
    uint32_t parity = 0;
    bool ok = true;
    const uint32_t const_even = g == 0 ? Mode::kEvenConstB : (g == 1 ? Mode::kEvenConstS : 0u);
    const uint32_t const_odd = g == 0 ? Mode::kOddConstB : (g == 1 ? Mode::kOddConstS : 0u);

    for (uint32_t j = 0; j < count; ++j, ++pkt) {
      if (pkt == tile_end) {
        on_tile_done(tile_index, tile_first, pkt);
#pragma unroll
        for (int tile = 0; tile < 4; ++tile) {
#pragma unroll
          for (int h = 0; h < H; ++h) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              y[tile][h][c] = 0.0f;
            }
          }
        }
        ++tile_index;
        tile_first = pkt;
        tile_end += num_groups;
      }
      const uint32_t stage = ring_addr + (slot * Geom::kStageBytes);
      if (!mbar_wait_bounded(bar_addr + (slot * 8), parity)) {
        ok = false;  // the partner times out on the same barrier, so both leave the loop here
        break;
      }

      float acc[4][H][4];
      float vacc[H][4];
#pragma unroll
      for (int h = 0; h < H; ++h) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          vacc[h][c] = 0.0f;
#pragma unroll
          for (int tile = 0; tile < 4; ++tile) {
            acc[tile][h][c] = 0.0f;
          }
        }
      }

      const uint32_t w_base = stage + (t * Geom::kChunkPitch) + (g * 16) + (side * 256);
      const uint32_t a_base = stage + Geom::kActOffset + (g * Geom::kActPitch) + (t * 16);
#pragma unroll 2
      for (int b = 0; b < Geom::kChunkRows; ++b) {
        uint4 bq[H];
#pragma unroll
        for (int h = 0; h < H; ++h) {
          bq[h] = lds128(a_base + (h * 8 * Geom::kActPitch) + (b * 64));
        }
        const uint4 w_lo = lds128(w_base + (b * kTileCols * 4));
        const uint4 w_hi = lds128(w_base + (b * kTileCols * 4) + 128);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const NibblePairs lo = Mode::unpack(word_of(w_lo, jj));
          const NibblePairs hi = Mode::unpack(word_of(w_hi, jj));
#pragma unroll
          for (int h = 0; h < H; ++h) {
            mma_word_pair<Mode>(acc[jj][h], lo, hi, bq[h]);
          }
        }
        // the all-constant column: row 0 of this MMA tile yields B, row 1 yields S
#pragma unroll
        for (int h = 0; h < H; ++h) {
          if (Mode::kEvenNibblesBf16) {
            mma_16816_bf16(vacc[h], const_even, 0u, const_even, 0u, bq[h].x, bq[h].z);
          } else {
            mma_16816_f16(vacc[h], const_even, 0u, const_even, 0u, bq[h].x, bq[h].z);
          }
          mma_16816_f16(vacc[h], const_odd, 0u, const_odd, 0u, bq[h].y, bq[h].w);
        }
      }

      // group epilogue: y += alpha * (acc - B) + beta * S
      {
        float bias[H][2];
        float sum[H][2];
#pragma unroll
        for (int h = 0; h < H; ++h) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            bias[h][e] = __shfl_sync(0xffffffffu, vacc[h][e], t);     // lane (g = 0, t)
            sum[h][e] = __shfl_sync(0xffffffffu, vacc[h][e], 4 + t);  // lane (g = 1, t)
          }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int col0 = (64 * side) + (4 * (g + (8 * half)));
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
            for (int h = 0; h < H; ++h) {
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int c = (2 * half) + e;
                float& out = y[jj][h][c];
                out = fmaf(alpha, acc[jj][h][c] - bias[h][e], out);
                out = fmaf(beta, sum[h][e], out);
              }
            }
          }
        }
      }

      // Both warps are done with this buffer: hand it back to the copy engine.
      pair_barrier(pair);
      if (issuer && issue_idx < count) {
        proxy_fence_async();
        issue_weights(issue_idx, issue_slot);
        issue_acts(issue_group, issue_slot);
        ++issue_idx;
        issue_group = (issue_group + 1 == num_groups) ? 0 : issue_group + 1;
        issue_slot = (issue_slot + 1 == stages) ? 0 : issue_slot + 1;
      }
      if (++slot == stages) {
        slot = 0;
        parity ^= 1u;
      }
    }

    if (ok) {
      on_tile_done(tile_index, tile_first, pkt);
    } else {
      // A copy never landed: record it and give the copies still in flight a bounded chance to
      // finish. Packets [pkt - p_begin, min(count, that + stages)) were issued.
      if (issuer) {
        atomicExch(p.status, static_cast<int>(kStatusCopyWaitTimeout));
      }
      uint32_t issued_end = (pkt - p_begin) + static_cast<uint32_t>(stages);
      issued_end = issued_end < count ? issued_end : count;
      for (uint32_t j = pkt - p_begin; j < issued_end; ++j) {
        (void)mbar_wait_bounded(bar_addr + (slot * 8), parity);
        if (++slot == stages) {
          slot = 0;
          parity ^= 1u;
        }
      }
    }
  } else {
    pdl_launch_dependents();
    pdl_wait_for_prerequisites();
  }
  __syncthreads();
  // Side-0 warps carry the finish (warp index = pair); side-1 warps only take part in its
  // CTA-wide steps.
  finish_cta<MT, E>(p, head_slots, Geom::kSlotFloats, tail_slots, ring_stride / 4,
                    side == 0 ? pair : (1 << 20), lane, pairs_per_cta, row_tile, row0, m_act);
}

}  // namespace fk_w4a16

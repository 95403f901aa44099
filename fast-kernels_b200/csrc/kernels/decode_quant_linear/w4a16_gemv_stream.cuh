// The decode GEMV: out[m, n] = sum_k act[m, k] * (alpha[n, g] * q[n, k] + beta[n, g]), M <= 4.
//
// Replaces the reference's three-launch path (group-sum prepass, arc_w4a16_kernel or
// arc_w4a16_split_k_kernel, partial reduction: csrc/kernels/decode_quant_linear/arc_w4a16.cu
// :124-158, :222-402) with ONE persistent launch whose unit of work is a whole packet.
//
// Work split. The T*NG packets of a layer are one contiguous byte stream (tile-major,
// group-minor). The stream is cut into V nearly equal contiguous runs, one per warp, V = warps
// resident on the GPU (or fewer for small layers). A warp is an independent worker: it owns a
// private ring of `stages` shared-memory buffers, lane 0 refills a buffer with one bulk
// asynchronous copy per packet (plus one small copy per batch row for that group's activations)
// as soon as the warp has consumed it, and all 32 lanes wait on the buffer's mbarrier. There is
// no CTA-wide barrier anywhere, so warps never stall on each other.
//
// Inside a packet each lane owns 4 adjacent output columns: one 128-bit shared-memory load per
// word-row brings 4 columns x 8 nibbles, five integer instructions per word turn the nibbles
// into fp16 values 1024 + q (or 1024 + 16 q), and eight mixed-precision FMAs per word multiply
// them with the fp16 activations into fp32 accumulators. The +1024 bias, the per-group scale and
// the per-group offset are settled once per group in fp32:
//     y += alpha * (acc - B_g) + beta * S_g,  S_g = sum_k a_k,  B_g = 1024 * sum_k a'_k
// where a' are the staged activations (odd nibbles pre-divided by 16). Products are exact in
// fp32, so the only roundings are the fp32 additions.
//
// Split tiles. A run may start or end inside a tile. Such a warp writes its 128 partial sums to
// a scratch slot that only it owns and takes a ticket for the tile; the warp that draws the last
// ticket adds the slots in run order (a fixed order, so results are reproducible bit for bit)
// and stores the output. Tiles that one warp covers alone never touch scratch.
#pragma once

#include "w4a16_common.cuh"

namespace fk_w4a16 {

struct GemvParams {
  const void* act;         // [m, k] 16-bit, row-major
  const uint8_t* packets;  // [num_tiles * num_groups, stride]
  void* out;               // [m, n] 16-bit, row-major
  float* scratch;          // [row_tiles][active_warps][2][M_TILE * 128] fp32
  int* tickets;            // [row_tiles][num_tiles], zero between calls
  int* status;             // device status word
  int m, n, k;
  int num_groups;          // k / G
  int num_tiles;           // n / 128
  int active_warps;        // V
  int stages;              // ring depth per warp
  long long total_packets; // num_tiles * num_groups
};

// First packet of worker v's run.
__device__ __forceinline__ long long run_begin(long long v, long long total, int workers) {
  return (v * total) / workers;
}
// Worker whose run holds packet p: the largest v with run_begin(v) <= p.
__device__ __forceinline__ int run_owner(long long p, long long total, int workers) {
  return static_cast<int>((((p + 1) * workers) - 1) / total);
}

// Rewrites one group's raw activations (G 16-bit values, row `m` of the stage) in place into the
// order the unpack produces -- per word-row the four half2 (a0,a4) (a1/16,a5/16) (a2,a6)
// (a3/16,a7/16) -- converting to fp16, and returns S = sum a and B = 1024 * sum a'.
template <int G, class E>
__device__ __forceinline__ void stage_activations(uint32_t act_addr, int lane, float& s_out,
                                                  float& b_out) {
  constexpr int kActiveLanes = G / 4;
  float s = 0.0f;
  float b = 0.0f;
  uint32_t p01 = 0;
  uint32_t p23 = 0;
  if (lane < kActiveLanes) {
    const uint2 raw = lds64(act_addr + lane * 8);
    const float f0 = E::to_float(static_cast<unsigned short>(raw.x & 0xffffu));
    const float f1 = E::to_float(static_cast<unsigned short>(raw.x >> 16));
    const float f2 = E::to_float(static_cast<unsigned short>(raw.y & 0xffffu));
    const float f3 = E::to_float(static_cast<unsigned short>(raw.y >> 16));
    s = (f0 + f1) + (f2 + f3);
    const __half h0 = __float2half_rn(f0);
    const __half h1 = __float2half_rn(f1 * 0.0625f);
    const __half h2 = __float2half_rn(f2);
    const __half h3 = __float2half_rn(f3 * 0.0625f);
    b = (__half2float(h0) + __half2float(h1)) + (__half2float(h2) + __half2float(h3));
    p01 = static_cast<uint32_t>(__half_as_ushort(h0)) |
          (static_cast<uint32_t>(__half_as_ushort(h1)) << 16);
    p23 = static_cast<uint32_t>(__half_as_ushort(h2)) |
          (static_cast<uint32_t>(__half_as_ushort(h3)) << 16);
  }
  // Even lanes hold nibbles 0-3 of a word-row, odd lanes nibbles 4-7. Swap one register with
  // the neighbour so each lane can write two finished (low nibble, high nibble) pairs.
  const bool odd = (lane & 1) != 0;
  const uint32_t recv = __shfl_xor_sync(0xffffffffu, odd ? p01 : p23, 1);
  if (lane < kActiveLanes) {
    uint2 staged;
    if (!odd) {
      staged.x = __byte_perm(p01, recv, 0x5410);  // (a0, a4)
      staged.y = __byte_perm(p01, recv, 0x7632);  // (a1', a5')
    } else {
      staged.x = __byte_perm(recv, p23, 0x5410);  // (a2, a6)
      staged.y = __byte_perm(recv, p23, 0x7632);  // (a3', a7')
    }
    sts64(act_addr + lane * 8, staged);
  }
  s_out = warp_sum(s);
  b_out = kNibbleBias * warp_sum(b);
}

template <class E>
__device__ __forceinline__ void store_tile_row(void* out, long long elem_offset, int lane,
                                               const float (&y)[4]) {
  uint2 packed;
  packed.x = static_cast<uint32_t>(E::from_float(y[0])) |
             (static_cast<uint32_t>(E::from_float(y[1])) << 16);
  packed.y = static_cast<uint32_t>(E::from_float(y[2])) |
             (static_cast<uint32_t>(E::from_float(y[3])) << 16);
  auto* dst = reinterpret_cast<uint2*>(static_cast<unsigned short*>(out) + elem_offset) + lane;
  *dst = packed;
}

// One warp's pass over packets [p_begin, p_end) of one tile-major packet stream, accumulating
// `y` per tile and handing every finished tile run to `on_tile_done(tile, first_pkt, last_pkt)`.
template <int G, int M_TILE, class E, class TileDone>
__device__ __forceinline__ bool consume_packet_run(const GemvParams& p, uint32_t ring_addr,
                                                   uint32_t bar_addr, int row0, int m_act,
                                                   long long p_begin, long long p_end, int lane,
                                                   float (&y)[M_TILE][4], TileDone&& on_tile_done) {
  constexpr int kStride = packet_stride(G);
  constexpr int kQBytes = packet_q_bytes(G);
  constexpr int kActBytes = G * 2;
  constexpr int kStageBytes = kStride + (M_TILE * kActBytes);
  constexpr int kWordRows = G / 8;

  const int stages = p.stages;
  const long long count = p_end - p_begin;
  const uint64_t weight_policy = l2_evict_first_policy();
  const uint64_t act_policy = l2_evict_last_policy();
  const auto* act_bytes = static_cast<const uint8_t*>(p.act);

  auto issue = [&](long long j) {
    const int slot = static_cast<int>(j % stages);
    const long long pkt = p_begin + j;
    const int group = static_cast<int>(pkt % p.num_groups);
    const uint32_t bar = bar_addr + (slot * 8);
    const uint32_t dst = ring_addr + (slot * kStageBytes);
    mbar_expect_tx(bar, static_cast<uint32_t>(kStride + (m_act * kActBytes)));
    bulk_copy_g2s(dst, p.packets + (pkt * kStride), kStride, bar, weight_policy);
    for (int m = 0; m < m_act; ++m) {
      const long long elem = (static_cast<long long>(row0 + m) * p.k) +
                             (static_cast<long long>(group) * G);
      bulk_copy_g2s(dst + kStride + (m * kActBytes), act_bytes + (elem * 2), kActBytes, bar,
                    act_policy);
    }
  };

  if (lane == 0) {
    const long long prefill = count < stages ? count : stages;
    for (long long j = 0; j < prefill; ++j) {
      issue(j);
    }
  }

  long long pkt = p_begin;
  int tile = static_cast<int>(p_begin / p.num_groups);
  long long tile_end = static_cast<long long>(tile + 1) * p.num_groups;
  long long tile_first = p_begin;
  int slot = 0;
  uint32_t parity = 0;
  bool ok = true;

  for (long long j = 0; j < count; ++j, ++pkt) {
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
      tile_end += p.num_groups;
    }

    const uint32_t bar = bar_addr + (slot * 8);
    const uint32_t stage = ring_addr + (slot * kStageBytes);
    if (!mbar_wait_bounded(bar, parity)) {
      ok = false;
      break;
    }

    float group_sum[M_TILE];
    float acc[M_TILE][4][2];
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      float bias = 0.0f;
      group_sum[m] = 0.0f;
      if (m < m_act) {
        stage_activations<G, E>(stage + kStride + (m * kActBytes), lane, group_sum[m], bias);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc[m][c][0] = -bias;
        acc[m][c][1] = 0.0f;
      }
    }
    __syncwarp();

#pragma unroll 4
    for (int r = 0; r < kWordRows; ++r) {
      const uint4 wq = lds128(stage + (r * (kTileCols * 4)) + (lane * 16));
      BiasedNibbles u[4];
      u[0] = unpack_word(wq.x);
      u[1] = unpack_word(wq.y);
      u[2] = unpack_word(wq.z);
      u[3] = unpack_word(wq.w);
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        const uint4 a = lds128(stage + kStride + (m * kActBytes) + (r * 16));
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          fma2_f32_f16(acc[m][c][0], acc[m][c][1], u[c].p04, a.x);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          fma2_f32_f16(acc[m][c][0], acc[m][c][1], u[c].p15, a.y);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          fma2_f32_f16(acc[m][c][0], acc[m][c][1], u[c].p26, a.z);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          fma2_f32_f16(acc[m][c][0], acc[m][c][1], u[c].p37, a.w);
        }
      }
    }

    {
      const uint2 a_raw = lds64(stage + kQBytes + (lane * 8));
      const uint2 b_raw = lds64(stage + kQBytes + (kTileCols * 2) + (lane * 8));
      float alpha[4];
      float beta[4];
      alpha[0] = E::to_float(static_cast<unsigned short>(a_raw.x & 0xffffu));
      alpha[1] = E::to_float(static_cast<unsigned short>(a_raw.x >> 16));
      alpha[2] = E::to_float(static_cast<unsigned short>(a_raw.y & 0xffffu));
      alpha[3] = E::to_float(static_cast<unsigned short>(a_raw.y >> 16));
      beta[0] = E::to_float(static_cast<unsigned short>(b_raw.x & 0xffffu));
      beta[1] = E::to_float(static_cast<unsigned short>(b_raw.x >> 16));
      beta[2] = E::to_float(static_cast<unsigned short>(b_raw.y & 0xffffu));
      beta[3] = E::to_float(static_cast<unsigned short>(b_raw.y >> 16));
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float dot = acc[m][c][0] + acc[m][c][1];
          y[m][c] = fmaf(alpha[c], dot, y[m][c]);
          y[m][c] = fmaf(beta[c], group_sum[m], y[m][c]);
        }
      }
    }

    // The whole warp is done reading this buffer: hand it back to the copy engine.
    __syncwarp();
    if (lane == 0 && (j + stages) < count) {
      proxy_fence_async();
      issue(j + stages);
    }
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }

  if (ok) {
    on_tile_done(tile, tile_first, pkt);
    return true;
  }

  // A copy never landed. Record it, then give the copies still in flight a bounded chance to
  // finish before this warp's shared memory can be handed to another CTA.
  if (lane == 0) {
    atomicExch(p.status, static_cast<int>(kStatusCopyWaitTimeout));
  }
  const long long issued_end = (pkt - p_begin) + stages < count ? (pkt - p_begin) + stages : count;
  for (long long j = pkt - p_begin; j < issued_end; ++j) {
    const uint32_t bar = bar_addr + (slot * 8);
    (void)mbar_wait_bounded(bar, parity);
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
  return false;
}

template <int G, int M_TILE, class E>
__global__ void __launch_bounds__(512, 1) w4a16_gemv_stream_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kStageBytes = packet_stride(G) + (M_TILE * G * 2);

  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int warps_per_cta = static_cast<int>(blockDim.x) >> 5;
  const int v = (static_cast<int>(blockIdx.x) * warps_per_cta) + warp;
  if (v >= p.active_warps) {
    return;  // whole warps leave; nothing below uses a CTA-wide barrier
  }
  const int row_tile = static_cast<int>(blockIdx.y);
  const int row0 = row_tile * M_TILE;
  const int m_act = (p.m - row0) < M_TILE ? (p.m - row0) : M_TILE;

  // Shared memory: all warps' barriers first (8 bytes each), then the rings.
  const int stages = p.stages;
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_addr = smem_base + (warp * stages * 8);
  const uint32_t ring_base = smem_base + (((warps_per_cta * stages * 8) + 127) & ~127);
  const uint32_t ring_addr = ring_base + (warp * stages * kStageBytes);
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_addr + (s * 8), 1);
    }
    mbar_init_fence();
  }
  __syncwarp();

  const long long total = p.total_packets;
  const int workers = p.active_warps;
  const long long p_begin = run_begin(v, total, workers);
  const long long p_end = run_begin(v + 1, total, workers);
  const int first_tile = static_cast<int>(p_begin / p.num_groups);

  float* scratch = p.scratch + (static_cast<size_t>(row_tile) * workers * 2 * (M_TILE * kTileCols));
  int* tickets = p.tickets + (static_cast<size_t>(row_tile) * p.num_tiles);

  float y[M_TILE][4];
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      y[m][c] = 0.0f;
    }
  }

  auto on_tile_done = [&](int tile, long long first_pkt, long long end_pkt) {
    const long long out_col = static_cast<long long>(tile) * kTileCols;
    if ((end_pkt - first_pkt) == p.num_groups) {
      // This warp saw every group of the tile: the sums are final.
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        if (m < m_act) {
          store_tile_row<E>(p.out, (static_cast<long long>(row0 + m) * p.n) + out_col, lane, y[m]);
        }
      }
      return;
    }

    // Partial tile: publish, take a ticket, and let the last arrival finish the tile.
    float* my_slot = scratch + ((static_cast<size_t>(v) * 2 + (tile == first_tile ? 0 : 1)) *
                                (M_TILE * kTileCols));
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      reinterpret_cast<float4*>(my_slot + (m * kTileCols))[lane] =
          make_float4(y[m][0], y[m][1], y[m][2], y[m][3]);
    }
    __threadfence();
    __syncwarp();

    const long long tile_first_pkt = static_cast<long long>(tile) * p.num_groups;
    const int v_first = run_owner(tile_first_pkt, total, workers);
    const int v_last = run_owner(tile_first_pkt + p.num_groups - 1, total, workers);
    int ticket = 0;
    if (lane == 0) {
      ticket = atomicAdd(&tickets[tile], 1);
    }
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != (v_last - v_first)) {
      return;
    }
    __threadfence();

    float total_y[M_TILE][4];
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        total_y[m][c] = 0.0f;
      }
    }
    for (int u = v_first; u <= v_last; ++u) {
      const int u_first_tile = static_cast<int>(run_begin(u, total, workers) / p.num_groups);
      const float* slot = scratch + ((static_cast<size_t>(u) * 2 + (tile == u_first_tile ? 0 : 1)) *
                                     (M_TILE * kTileCols));
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        const float4 part = __ldcg(reinterpret_cast<const float4*>(slot + (m * kTileCols)) + lane);
        total_y[m][0] += part.x;
        total_y[m][1] += part.y;
        total_y[m][2] += part.z;
        total_y[m][3] += part.w;
      }
    }
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      if (m < m_act) {
        store_tile_row<E>(p.out, (static_cast<long long>(row0 + m) * p.n) + out_col, lane,
                          total_y[m]);
      }
    }
    if (lane == 0) {
      tickets[tile] = 0;  // ready for the next call on this workspace
    }
  };

  (void)consume_packet_run<G, M_TILE, E>(p, ring_addr, bar_addr, row0, m_act, p_begin, p_end, lane,
                                         y, on_tile_done);
}

// ---------------------------------------------------------------------------------------------
// Caller-visible split-K (the reference's arc_w4a16_forward_split_k + reduce, arc_w4a16.cu
// :341-402): slice s covers groups [s*gps, min((s+1)*gps, NG)), gps = ceil(NG / S), and writes
// fp32 partials[s, m, n]. One CTA per (tile, slice); its warps take the slice's packets
// round-robin and add their sums through shared memory in warp order.
// ---------------------------------------------------------------------------------------------
struct SplitKParams {
  GemvParams base;
  float* partials;  // [slices, m, n]
  int slices;
  int groups_per_slice;
};

template <int G, int M_TILE, class E>
__global__ void __launch_bounds__(128, 1) w4a16_split_k_kernel(const __grid_constant__ SplitKParams sp) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kStageBytes = packet_stride(G) + (M_TILE * G * 2);
  constexpr int kWarps = 4;
  __shared__ float reduce_buf[kWarps][M_TILE][kTileCols];

  const GemvParams& p = sp.base;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int tile = static_cast<int>(blockIdx.x);
  const int slice = static_cast<int>(blockIdx.z);
  const int row0 = static_cast<int>(blockIdx.y) * M_TILE;
  const int m_act = (p.m - row0) < M_TILE ? (p.m - row0) : M_TILE;

  const int g_begin = slice * sp.groups_per_slice;
  int g_end = g_begin + sp.groups_per_slice;
  g_end = g_end < p.num_groups ? g_end : p.num_groups;
  const int slice_groups = g_end > g_begin ? g_end - g_begin : 0;
  // Warp w takes a contiguous share of the slice.
  const int w_begin = g_begin + ((slice_groups * warp) / kWarps);
  const int w_end = g_begin + ((slice_groups * (warp + 1)) / kWarps);

  const int stages = p.stages;
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_addr = smem_base + (warp * stages * 8);
  const uint32_t ring_addr =
      smem_base + (((kWarps * stages * 8) + 127) & ~127) + (warp * stages * kStageBytes);
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_addr + (s * 8), 1);
    }
    mbar_init_fence();
  }
  __syncwarp();

  float y[M_TILE][4];
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      y[m][c] = 0.0f;
    }
  }
  if (w_end > w_begin) {
    const long long base_pkt = static_cast<long long>(tile) * p.num_groups;
    auto keep = [](int, long long, long long) {};
    (void)consume_packet_run<G, M_TILE, E>(p, ring_addr, bar_addr, row0, m_act, base_pkt + w_begin,
                                           base_pkt + w_end, lane, y, keep);
  }
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
    reinterpret_cast<float4*>(&reduce_buf[warp][m][0])[lane] =
        make_float4(y[m][0], y[m][1], y[m][2], y[m][3]);
  }
  __syncthreads();
  for (int idx = static_cast<int>(threadIdx.x); idx < m_act * kTileCols; idx += kWarps * 32) {
    const int m = idx / kTileCols;
    const int c = idx % kTileCols;
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      sum += reduce_buf[w][m][c];
    }
    const size_t off = ((static_cast<size_t>(slice) * p.m + (row0 + m)) * p.n) +
                       (static_cast<size_t>(tile) * kTileCols) + c;
    sp.partials[off] = sum;
  }
}

}  // namespace fk_w4a16

// The decode GEMV: out[m, n] = sum_k act[m, k] * (alpha[n, g] * q[n, k] + beta[n, g]), M <= 4.
//
// Replaces the reference's three-launch path (group-sum prepass, arc_w4a16_kernel or
// arc_w4a16_split_k_kernel, partial reduction: csrc/kernels/decode_quant_linear/arc_w4a16.cu
// :124-158, :222-402) with ONE persistent launch whose unit of work is a whole packet.
//
// Work split. The T*NG packets of a layer are one contiguous byte stream (tile-major,
// group-minor). The stream is cut into V contiguous runs whose lengths differ by at most one
// packet, one run per warp, V = warps resident on the GPU (or fewer for small layers); warps of a
// CTA hold neighbouring runs. A warp is an independent worker: it owns a private ring of `stages`
// shared-memory buffers, lane 0 refills a buffer with one bulk asynchronous copy per packet (plus
// one small copy per batch row for that group's activations) as soon as the warp has consumed it,
// and all 32 lanes wait on the buffer's mbarrier. No warp waits for another until its run is done.
//
// Inside a packet each lane owns 4 adjacent output columns: one 128-bit shared-memory load per
// word-row brings 4 columns x 8 nibbles, a handful of integer instructions per word turn the
// nibbles into 16-bit floats "constant + q", and eight mixed-precision FMAs per word multiply them
// with the staged activations into fp32 accumulators (see w4a16_common.cuh). The constant, the
// per-group scale and the per-group offset are settled once per group in fp32:
//     y += alpha * (acc - B_g) + beta * S_g,    S_g = sum_k a_k,   B_g = sum_k constant_k * a'_k
//
// Finishing a tile (split-K, two levels, fixed summation order => bit-reproducible results):
//   1. a warp whose run covers all groups of a tile stores that tile's outputs itself;
//   2. otherwise the warp leaves its partial sums in a shared-memory slot; after one CTA-wide
//      barrier at the end of the runs, the CTA adds the slots of each tile in warp order and
//      stores tiles that lie wholly inside the CTA's packet range;
//   3. a tile shared with a neighbouring CTA is written to a global scratch slot that only this
//      CTA owns, followed by a ticket; the CTA that draws the tile's last ticket adds the slots in
//      CTA order and stores the outputs, then resets the ticket for the next call.
#pragma once

#include "w4a16_common.cuh"

namespace fk_w4a16 {

// Optional timeline instrumentation for tuning builds (-DFK_W4A16_TRACE): lane 0 of every warp
// records the global timer at a few milestones. Compiled out of the shipped library.
#ifdef FK_W4A16_TRACE
constexpr int kTraceSlots = 8;
constexpr int kTraceLaunches = 16;  // launches are told apart by a host-side counter modulo this
__device__ unsigned long long g_trace[kTraceLaunches * 148 * 16 * kTraceSlots];  // one TU's
__device__ __forceinline__ void trace_mark_at(int launch, int slot) {
  if ((threadIdx.x & 31) == 0 && blockIdx.x < 148 && (threadIdx.x >> 5) < 16) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    const size_t base =
        ((((static_cast<size_t>(launch) * 148) + blockIdx.x) * 16) + (threadIdx.x >> 5)) * kTraceSlots;
    g_trace[base + slot] = t;
    if (slot == 0) {
      unsigned int smid;
      asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
      g_trace[base + 6] = smid;
    }
  }
}
#define trace_mark(slot) trace_mark_at(p.trace_id, (slot))
#else
#define trace_mark(slot) ((void)0)
#endif

constexpr int kMaxPeers = 7;
constexpr uint32_t kExchangePresent = 0x50415254u;  // upper half of a filled pair-exchange word

struct GemvParams {
#ifdef FK_W4A16_TRACE
  int trace_id;
#endif
  const void* act;         // [m, k] 16-bit, row-major
  const uint8_t* packets;  // [num_tiles * num_groups, stride]
  void* out;               // [m, n] 16-bit, row-major
  float* scratch;          // [row_tiles][ctas][2][M_TILE * 128] fp32
  int* tickets;            // [row_tiles][num_tiles], zero between calls
  // Pair exchange, or null: [row_tiles][ctas][M_TILE * 128] 64-bit words, zero between calls; area
  // c serves the tile that straddles the boundary between CTA c and CTA c + 1.
  unsigned long long* exchange;
  int* status;             // device status word
  // Output placement. Element (row, col) of the result goes to out[row * out_ld + out_col0 + col]
  // and to the same offset in each of peer_out[0 .. num_peers) -- buffers of other GPUs mapped
  // into this process (plain stores over NVLink). out_f32 selects unrounded fp32 outputs.
  long long out_ld;
  long long out_col0;
  int out_f32;
  int num_peers;
  void* peer_out[kMaxPeers];
  // Optional fused residual add: a 16-bit matrix laid out like the output (same out_ld and
  // out_col0); every output becomes round(y + residual), one rounding. May alias `out`.
  const void* residual;
  // Optional fused SiLU-and-multiply over a stacked [gate; up] layer, or null: the output has n/2
  // columns, out[j] = silu(y[j]) * y[j + n/2]. The two halves of a column are finished by
  // different warps at different times; they meet in `gated` ([m][n/2] 64-bit words, zero between
  // calls) exactly like the two halves of a split tile meet in `exchange`.
  unsigned long long* gated;
  // Optional fused RMSNorm in front of the GEMV, or null: the activations the GEMV multiplies are
  // round16(norm_weight[k] * round16(x[k] * rsqrt(mean_k(x^2) + norm_eps))) per row.
  const void* norm_weight;  // [k] 16-bit
  float norm_eps;
  // Exchange completion. When local_signal is set, every CTA, once its own stores are done, adds 1
  // (system scope, released after those stores) to local_signal and to every peer_signal; the
  // kernel does not complete before local_signal has reached wait_value x (CTAs of the grid),
  // i.e. before every CTA of every GPU of the group has delivered. Every GPU of the group must
  // therefore run the same launch shape (same problem on the same kind of device).
  unsigned int* peer_signal[kMaxPeers];
  unsigned int* local_signal;
  unsigned int wait_value;
  unsigned long long peer_wait_ns;  // the wait gives up after this long and sets the status word
  // Optional fused reduction behind the exchange (a K-split layer's sum over GPUs), or
  // reduce_slots == 0: once everything has arrived, out16[m][n] = round16(sum over s <
  // reduce_slots of reduce_input[s][m][n]), slots added in index order, each CTA a slice.
  const float* reduce_input;        // [reduce_slots][m][n] fp32 in THIS GPU's memory
  void* reduce_output;              // [m][n] 16-bit
  int reduce_slots;
  // Flag-in-data exchange, or ll_epoch == 0. Outputs are then written -- to `out` and to every
  // peer_out -- as 8-byte words {fp32 value, ll_epoch}: an 8-byte store is atomic, so a word whose
  // flag shows this call's epoch carries this call's value, and the exchange needs no fence, no
  // counter and no round trip. ll_input is this GPU's receive area [ll_slots][m][ll_slot_cols]
  // words (one slot per GPU of the group, its own included); once a word has arrived, the first
  // few CTAs turn it into the final 16-bit output: ll_reduce == 0 concatenates the slots' columns
  // (an N-split), ll_reduce == 1 adds the slots in order (a K-split).
  // The epoch is either given (ll_epoch) or kept on the device (ll_epoch_counter: the epoch of a
  // call is *counter + 1, and the last receiving CTA adds 1 when the call is complete), which is
  // what lets a captured call be replayed: nothing about the exchange is baked into the launch.
  // With the counter, the receive area alternates between two copies ll_parity_words apart
  // (epoch & 1), here and in every peer_out, so that a GPU that runs one call ahead cannot
  // overwrite words that a peer has not read yet.
  unsigned int ll_epoch;
  unsigned int* ll_epoch_counter;   // device word, zero before the first call; or null
  unsigned int* ll_ticket;          // device word, zero between calls (counts finished receivers)
  long long ll_parity_words;
  const unsigned long long* ll_input;
  void* ll_output;                  // [m][ll_slots * ll_slot_cols] or [m][ll_slot_cols] 16-bit
  int ll_slots;
  int ll_slot_cols;
  int ll_reduce;
  int m, n, k;
  int num_groups;          // k / G
  int num_tiles;           // n / 128
  int active_warps;        // V: number of runs
  int stages;              // ring depth per warp
  uint32_t total_packets;  // num_tiles * num_groups
  // Runs: run v holds packets [floor(v T / V), floor((v + 1) T / V)) with T = total_packets --
  // lengths differ by at most one and the longer runs are spread evenly over the CTAs.
  uint32_t run_base;       // T / V
  uint32_t run_rem;        // T % V
  uint64_t run_magic;      // floor(2^40 / V) + 1: exact division of x < 2^24 by V (V <= 4096)
  float run_inv;           // V / T, for the inverse map
};

// floor(x / V) for x < 2^24 (see run_magic).
__device__ __forceinline__ uint32_t div_by_workers(uint32_t x, const GemvParams& p) {
  return static_cast<uint32_t>((static_cast<uint64_t>(x) * p.run_magic) >> 40);
}
__device__ __forceinline__ uint32_t run_begin(uint32_t v, const GemvParams& p) {
  return (v * p.run_base) + div_by_workers(v * p.run_rem, p);
}
// Run that holds packet `pkt`: an estimate from the reciprocal, corrected by at most a step or two.
__device__ __forceinline__ uint32_t run_owner(uint32_t pkt, const GemvParams& p) {
  const uint32_t last = static_cast<uint32_t>(p.active_warps) - 1;
  uint32_t v = static_cast<uint32_t>(static_cast<float>(pkt) * p.run_inv);
  v = v > last ? last : v;
  while (v < last && run_begin(v + 1, p) <= pkt) {
    ++v;
  }
  while (v > 0 && run_begin(v, p) > pkt) {
    --v;
  }
  return v;
}

// Turns this lane's 4 consecutive raw activations of a group (`raw`; lanes >= G/4 hold nothing)
// into the 8 bytes it contributes to the staged layout: per word-row the four pairs (a0,a4)
// (a1,a5) (a2,a6) (a3,a7) in the formats the unpack mode multiplies with. Even lanes end up with
// pairs 0 and 1 of word-row lane/2, odd lanes with pairs 2 and 3. Also accumulates this lane's
// share of S = sum a and of the constant term B.
template <int G, class Mode>
__device__ __forceinline__ uint2 stage_pairs(uint2 raw, int lane, float& s, float& b) {
  using E = typename Mode::Elem;
  constexpr int kActiveLanes = G / 4;
  uint32_t p01 = 0;
  uint32_t p23 = 0;
  if (lane < kActiveLanes) {
    const float f0 = E::to_float(static_cast<unsigned short>(raw.x & 0xffffu));
    const float f1 = E::to_float(static_cast<unsigned short>(raw.x >> 16));
    const float f2 = E::to_float(static_cast<unsigned short>(raw.y & 0xffffu));
    const float f3 = E::to_float(static_cast<unsigned short>(raw.y >> 16));
    s += (f0 + f1) + (f2 + f3);
    // This lane holds nibbles 4*(lane&1) + {0,1,2,3} of a word-row: positions 1 and 3 are odd.
    const uint32_t h0 = Mode::stage(f0, false, b);
    const uint32_t h1 = Mode::stage(f1, true, b);
    const uint32_t h2 = Mode::stage(f2, false, b);
    const uint32_t h3 = Mode::stage(f3, true, b);
    p01 = h0 | (h1 << 16);
    p23 = h2 | (h3 << 16);
  }
  // Even lanes hold nibbles 0-3 of a word-row, odd lanes nibbles 4-7. Swap one register with
  // the neighbour so each lane can write two finished (nibble i, nibble i+4) pairs.
  const bool odd_lane = (lane & 1) != 0;
  const uint32_t recv = __shfl_xor_sync(0xffffffffu, odd_lane ? p01 : p23, 1);
  uint2 staged;
  if (!odd_lane) {
    staged.x = __byte_perm(p01, recv, 0x5410);  // (a0, a4)
    staged.y = __byte_perm(p01, recv, 0x7632);  // (a1, a5)
  } else {
    staged.x = __byte_perm(recv, p23, 0x5410);  // (a2, a6)
    staged.y = __byte_perm(recv, p23, 0x7632);  // (a3, a7)
  }
  return staged;
}

// Stages one group's activations into the warp's shared-memory buffer and returns S and B.
template <int G, class Mode>
__device__ __forceinline__ void stage_activations(uint2 raw, uint32_t act_addr, int lane,
                                                  float& s_out, float& b_out) {
  float s = 0.0f;
  float b = 0.0f;
  const uint2 staged = stage_pairs<G, Mode>(raw, lane, s, b);
  if (lane < G / 4) {
    sts64(act_addr + lane * 8, staged);
  }
  s_out = warp_sum(s);
  b_out = warp_sum(b);
}

// Epoch of this call in the flag-in-data exchange; 0 when that exchange is off.
__device__ __forceinline__ unsigned int ll_epoch_now(const GemvParams& p) {
  if (p.ll_epoch_counter != nullptr) {
    return __ldcg(p.ll_epoch_counter) + 1u;
  }
  return p.ll_epoch;
}

// A flag-in-data word: value in the low half, the call's epoch in the high half.
__device__ __forceinline__ unsigned long long ll_word(float value, unsigned int epoch) {
  return (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(value);
}

template <class E>
__device__ __forceinline__ void store_tile_row_to(void* out, int out_f32, long long elem_offset,
                                                  int lane, const float (&y)[4], unsigned int ll_epoch = 0) {
  if (ll_epoch != 0) {
    // four 8-byte words as two 16-byte stores; each word is valid on its own
    auto* dst = reinterpret_cast<ulonglong2*>(static_cast<unsigned long long*>(out) + elem_offset) + (lane * 2);
    dst[0] = make_ulonglong2(ll_word(y[0], ll_epoch), ll_word(y[1], ll_epoch));
    dst[1] = make_ulonglong2(ll_word(y[2], ll_epoch), ll_word(y[3], ll_epoch));
    return;
  }
  if (out_f32 != 0) {
    auto* dst = reinterpret_cast<float4*>(static_cast<float*>(out) + elem_offset) + lane;
    *dst = make_float4(y[0], y[1], y[2], y[3]);
    return;
  }
  uint2 packed;
  packed.x = static_cast<uint32_t>(E::from_float(y[0])) |
             (static_cast<uint32_t>(E::from_float(y[1])) << 16);
  packed.y = static_cast<uint32_t>(E::from_float(y[2])) |
             (static_cast<uint32_t>(E::from_float(y[3])) << 16);
  auto* dst = reinterpret_cast<uint2*>(static_cast<unsigned short*>(out) + elem_offset) + lane;
  *dst = packed;
}

constexpr uint32_t kGatedGate = 0x47415445u;  // upper half of a `gated` word holding a gate value
constexpr uint32_t kGatedUp = 0x55505550u;    // ... holding an up value

__device__ __forceinline__ float silu_times(float gate, float up) {
  return (gate / (1.0f + __expf(-gate))) * up;
}

// SiLU-and-multiply meeting point for one element: swaps (value, kind) into the column's word;
// returns true, with the finished product in `value` and the output column in `out_col`, when the
// other half was already there (the word is cleared for the next call).
__device__ __forceinline__ bool gated_meet(const GemvParams& p, int row, uint32_t tile, int col,
                                           float& value, long long& out_col) {
  const uint32_t half_tiles = static_cast<uint32_t>(p.num_tiles) >> 1;
  const bool is_gate = tile < half_tiles;
  out_col = (static_cast<long long>(is_gate ? tile : tile - half_tiles) * kTileCols) + col;
  unsigned long long* word = p.gated + ((static_cast<long long>(row) * (p.n >> 1)) + out_col);
  const unsigned long long mine =
      (static_cast<unsigned long long>(is_gate ? kGatedGate : kGatedUp) << 32) | __float_as_uint(value);
  const unsigned long long seen = atomicExch(word, mine);
  if (static_cast<uint32_t>(seen >> 32) != (is_gate ? kGatedUp : kGatedGate)) {
    return false;
  }
  const float other = __uint_as_float(static_cast<uint32_t>(seen));
  value = is_gate ? silu_times(value, other) : silu_times(other, value);
  *word = 0ull;
  return true;
}

template <class E>
__device__ __forceinline__ void store_element_at(const GemvParams& p, long long offset, float value) {
  if (p.residual != nullptr) {
    value += E::to_float(__ldcg(static_cast<const unsigned short*>(p.residual) + offset));
  }
  const unsigned int epoch = ll_epoch_now(p);
  const long long ll_offset = offset + ((epoch & 1u) != 0 ? p.ll_parity_words : 0);
  for (int dest = -1; dest < p.num_peers; ++dest) {
    void* out = dest < 0 ? p.out : p.peer_out[dest];
    if (epoch != 0) {
      static_cast<unsigned long long*>(out)[ll_offset] = ll_word(value, epoch);
    } else if (p.out_f32 != 0) {
      static_cast<float*>(out)[offset] = value;
    } else {
      static_cast<unsigned short*>(out)[offset] = E::from_float(value);
    }
  }
}

// Stores one element of a finished tile locally and on every peer. Deliberately not inlined: it
// is called from many places in every kernel instantiation and sits outside the streaming loop.
template <class E>
__device__ __noinline__ void store_tile_element(const GemvParams& p, int row, uint32_t tile,
                                                   int col, float value) {
  if (p.gated != nullptr) {
    long long out_col;
    if (gated_meet(p, row, tile, col, value, out_col)) {
      store_element_at<E>(p, (static_cast<long long>(row) * p.out_ld) + p.out_col0 + out_col, value);
    }
    return;
  }
  store_element_at<E>(p, (static_cast<long long>(row) * p.out_ld) + p.out_col0 +
                             (static_cast<long long>(tile) * kTileCols) + col, value);
}

// Stores one row of a finished tile (this lane's 4 columns) locally and on every peer.
template <class E>
__device__ __forceinline__ void store_tile_row(const GemvParams& p, int row, uint32_t tile, int lane,
                                               const float (&y)[4]) {
  if (p.gated != nullptr) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      store_tile_element<E>(p, row, tile, (lane * 4) + c, y[c]);
    }
    return;
  }
  const long long offset = (static_cast<long long>(row) * p.out_ld) + p.out_col0 +
                           (static_cast<long long>(tile) * kTileCols);
  float v[4] = {y[0], y[1], y[2], y[3]};
  if (p.residual != nullptr) {
    // L2-coherent load: in a chain of steps inside one launch the residual may be what another SM
    // wrote a step ago
    const uint2 r = __ldcg(reinterpret_cast<const uint2*>(static_cast<const unsigned short*>(p.residual) + offset) + lane);
    v[0] += E::to_float(static_cast<unsigned short>(r.x & 0xffffu));
    v[1] += E::to_float(static_cast<unsigned short>(r.x >> 16));
    v[2] += E::to_float(static_cast<unsigned short>(r.y & 0xffffu));
    v[3] += E::to_float(static_cast<unsigned short>(r.y >> 16));
  }
  const unsigned int epoch = ll_epoch_now(p);
  const long long placed = offset + ((epoch & 1u) != 0 ? p.ll_parity_words : 0);
  store_tile_row_to<E>(p.out, p.out_f32, placed, lane, v, epoch);
  for (int peer = 0; peer < p.num_peers; ++peer) {
    store_tile_row_to<E>(p.peer_out[peer], p.out_f32, placed, lane, v, epoch);
  }
}

// Fused RMSNorm, part one: 1 / rms of each of the CTA's rows, computed by the whole CTA (every
// thread must call this once; it contains a CTA barrier). Sum of squares in a fixed order: per
// thread over a strided share of the row, then the warp tree, then the warps in order.
template <int M_TILE, class E>
__device__ __forceinline__ void cta_inverse_rms(const GemvParams& p, int row0, int m_act,
                                                float (&inv_rms)[M_TILE]) {
  __shared__ float partial[16][M_TILE];
  __shared__ float result[M_TILE];
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int warps = static_cast<int>(blockDim.x) >> 5;
  const int units = p.k >> 3;  // 16-byte units per row
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
    float acc = 0.0f;
    if (m < m_act) {
      const uint4* row = reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(p.act) +
                                                        (static_cast<size_t>(row0 + m) * p.k));
      for (int i = static_cast<int>(threadIdx.x); i < units; i += static_cast<int>(blockDim.x)) {
        const uint4 v = __ldcg(row + i);  // L2-coherent: see the chain kernel
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = E::to_float(static_cast<unsigned short>(w[j] & 0xffffu));
          const float hi = E::to_float(static_cast<unsigned short>(w[j] >> 16));
          acc = fmaf(lo, lo, acc);
          acc = fmaf(hi, hi, acc);
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      partial[warp][m] = acc;
    }
  }
  __syncthreads();
  if (threadIdx.x < M_TILE) {
    float total = 0.0f;
    for (int w = 0; w < warps; ++w) {
      total += partial[w][threadIdx.x];
    }
    result[threadIdx.x] = rsqrtf((total / static_cast<float>(p.k)) + p.norm_eps);
  }
  __syncthreads();
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
    inv_rms[m] = result[m];
  }
}

// Fused RMSNorm, part two: this lane's four raw activations -> the four normalised ones.
template <class E>
__device__ __forceinline__ uint2 normalise4(uint2 raw, uint2 weight, float inv_rms) {
  auto one = [&](uint32_t x, uint32_t w) -> uint32_t {
    const float scaled = E::to_float(static_cast<unsigned short>(x)) * inv_rms;
    const float rounded = E::to_float(E::from_float(scaled));
    return E::from_float(rounded * E::to_float(static_cast<unsigned short>(w)));
  };
  uint2 out;
  out.x = one(raw.x & 0xffffu, weight.x & 0xffffu) | (one(raw.x >> 16, weight.x >> 16) << 16);
  out.y = one(raw.y & 0xffffu, weight.y & 0xffffu) | (one(raw.y >> 16, weight.y >> 16) << 16);
  return out;
}

// One packet's worth of work for a warp: stages the group's activations (`raw`: this lane's four
// consecutive 16-bit activations per batch row) into the warp's shared-memory buffer `act_addr`,
// multiplies the packet at shared-memory address `stage` with them and folds scale, offset and the
// unpack constant into the running sums: y += alpha * (acc - B_g) + beta * S_g.
template <int G, int M_TILE, class Mode>
__device__ __forceinline__ void multiply_packet(uint32_t stage, uint32_t act_addr,
                                                const uint2 (&raw)[M_TILE], int m_act, int lane,
                                                float (&y)[M_TILE][4]) {
  using E = typename Mode::Elem;
  constexpr int kQBytes = packet_q_bytes(G);
  constexpr int kActBytes = G * 2;
  constexpr int kWordRows = G / 8;
  float group_sum[M_TILE];
  float acc[M_TILE][4][2];
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
    float bias = 0.0f;
    group_sum[m] = 0.0f;
    if (m < m_act) {
      stage_activations<G, Mode>(raw[m], act_addr + (m * kActBytes), lane, group_sum[m], bias);
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
    NibblePairs u[4];
    u[0] = Mode::unpack(wq.x);
    u[1] = Mode::unpack(wq.y);
    u[2] = Mode::unpack(wq.z);
    u[3] = Mode::unpack(wq.w);
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      const uint4 a = lds128(act_addr + (m * kActBytes) + (r * 16));
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        Mode::mac(acc[m][c][0], acc[m][c][1], u[c], a);
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
}

// One warp's pass over packets [p_begin, p_end) of the tile-major packet stream, accumulating
// `y` per tile and handing every finished tile run to on_tile_done(tile, first_pkt, end_pkt).
// Returns false if a copy never arrived (the status word is set).
// `after_wait(inv_rms)` runs once, right after the kernel has waited for the work ahead of it in
// the stream: the place for CTA-wide preparation that reads the activations (fused RMSNorm).
struct NoPreparation {
  template <int M_TILE>
  __device__ __forceinline__ void operator()(float (&)[M_TILE]) const {}
};
template <int G, int M_TILE, class Mode, class TileDone, class AfterWait = NoPreparation>
__device__ __forceinline__ bool consume_packet_run(const GemvParams& p, uint32_t ring_addr,
                                                   uint32_t bar_addr, uint32_t act_addr, int row0,
                                                   int m_act,
                                                   uint32_t p_begin, uint32_t p_end, int lane,
                                                   float (&y)[M_TILE][4], TileDone&& on_tile_done,
                                                   AfterWait&& after_wait = AfterWait{}) {
  using E = typename Mode::Elem;
  constexpr int kStride = packet_stride(G);
  constexpr int kQBytes = packet_q_bytes(G);
  constexpr int kActBytes = G * 2;
  constexpr int kStageBytes = kStride;
  constexpr int kWordRows = G / 8;
  constexpr int kActLanes = G / 4;

  const int stages = p.stages;
  const uint32_t count = p_end - p_begin;
  const uint64_t weight_policy = l2_evict_first_policy();
  const auto* act_bytes = static_cast<const uint8_t*>(p.act);
  const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);

  uint32_t tile = p_begin / num_groups;
  const uint32_t first_group = p_begin - (tile * num_groups);

  // Issue side: lane 0 alone issues copies; the counters are cheap enough to keep in every lane.
  uint32_t issue_idx = 0;
  int issue_slot = 0;
  auto issue_next = [&]() {
    const uint32_t bar = bar_addr + (issue_slot * 8);
    mbar_expect_tx(bar, static_cast<uint32_t>(kStride));
    bulk_copy_g2s(ring_addr + (issue_slot * kStageBytes),
                  p.packets + (static_cast<size_t>(p_begin + issue_idx) * kStride), kStride, bar,
                  weight_policy);
    ++issue_idx;
    issue_slot = (issue_slot + 1 == stages) ? 0 : issue_slot + 1;
  };

  if (lane == 0) {
    const uint32_t prefill = count < static_cast<uint32_t>(stages) ? count : stages;
    for (uint32_t j = 0; j < prefill; ++j) {
      issue_next();
    }
  }
  trace_mark(1);

  // Programmatic dependent launch: the weight copies above do not depend on the kernel before
  // this one in the stream, so they are already in flight; let the kernel after this one start
  // its own prologue, then wait for the one before us before touching activations, outputs or
  // scratch (all of which it may have written).
  pdl_launch_dependents();
  pdl_wait_for_prerequisites();
  float inv_rms[M_TILE];
#pragma unroll
  for (int m = 0; m < M_TILE; ++m) {
    inv_rms[m] = 1.0f;
  }
  after_wait(inv_rms);
  const bool normalise = p.norm_weight != nullptr;

  // Activations: plain global loads (they stay in L2), one packet ahead, straight to registers.
  uint32_t act_group = first_group;
  uint2 next_weight = make_uint2(0u, 0u);  // the group's RMSNorm weights, when fused
  auto load_activations = [&](uint2 (&dst)[M_TILE]) {
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      dst[m] = make_uint2(0u, 0u);
      if (m < m_act && lane < kActLanes) {
        const size_t elem = (static_cast<size_t>(row0 + m) * p.k) + (act_group * G);
        dst[m] = __ldg(reinterpret_cast<const uint2*>(act_bytes + (elem * 2)) + lane);
      }
    }
    if (normalise && lane < kActLanes) {
      next_weight = __ldg(reinterpret_cast<const uint2*>(static_cast<const unsigned short*>(p.norm_weight) +
                                                         (static_cast<size_t>(act_group) * G)) + lane);
    }
    act_group = (act_group + 1 == num_groups) ? 0 : act_group + 1;
  };
  uint2 next_raw[M_TILE];
  load_activations(next_raw);

  uint32_t pkt = p_begin;
  uint32_t tile_end = (tile + 1) * num_groups;
  uint32_t tile_first = p_begin;
  int slot = 0;
  uint32_t parity = 0;
  bool ok = true;

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

    const uint32_t bar = bar_addr + (slot * 8);
    const uint32_t stage = ring_addr + (slot * kStageBytes);
    if (!mbar_wait_bounded(bar, parity)) {
      ok = false;
      break;
    }
    if (j == 0) {
      trace_mark(2);
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

    // The whole warp is done reading this buffer: hand it back to the copy engine.
    __syncwarp();
    if (lane == 0 && issue_idx < count) {
      proxy_fence_async();
      issue_next();
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
  issue_idx = __shfl_sync(0xffffffffu, issue_idx, 0);
  if (lane == 0) {
    atomicExch(p.status, static_cast<int>(kStatusCopyWaitTimeout));
  }
  for (uint32_t j = pkt - p_begin; j < issue_idx; ++j) {
    (void)mbar_wait_bounded(bar_addr + (slot * 8), parity);
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
  return false;
}

// ---------------------------------------------------------------------------------------------
// Exchange completion of a multi-GPU call (no-op when local_signal is null). Every thread of the
// CTA calls it once, after the CTA's last output store.
//
// Signalling is per CTA, not per GPU: after a CTA barrier, thread 0 executes ONE system-scope
// fence -- cumulative over the barrier, so it covers every thread's peer stores; a fence in every
// thread costs tens of microseconds, system-scope fences of one SM do not overlap -- and then
// adds 1 to the counter of every GPU with fire-and-forget reductions. No exit ticket, no "last
// CTA": the slowest CTA's stores are the only thing the other GPUs ever wait for.
// Who waits: without the fused reduction one thread of the grid (CTA 0) holds the kernel open
// until the local counter shows every CTA of every GPU; with it, the first few CTAs wait and then
// share the sum of the partials. Waits are bounded (peer_wait_ns) and report through the status
// word; the waiting CTAs never hold back the signalling ones, so no CTA needs another to be
// resident.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void red_add_system(unsigned int* counter) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
}
__device__ __forceinline__ unsigned int load_counter_system(const unsigned int* counter) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_system() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

constexpr unsigned int kReduceCtas = 8;

__device__ __forceinline__ unsigned long long load_word_system(const unsigned long long* word) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(word) : "memory");
  return v;
}

// The receiving side of the flag-in-data exchange: every CTA of the grid, once its own work is
// done, takes a share of this GPU's final outputs, waits for the words they are made of to show
// the call's epoch and writes them in the 16-bit type. A thread has one or two outputs; the loads
// of all the words of an output (one per slot for a K-split) are issued together and only the
// missing ones are polled again (bounded by peer_wait_ns). Polling with a few threads instead --
// each walking many words one L2 round trip after the other -- cost microseconds.
template <class E>
__device__ __forceinline__ void ll_receive(const GemvParams& p) {
  const unsigned int ctas_total = gridDim.x * gridDim.y;
  const unsigned int cta_index = (blockIdx.y * gridDim.x) + blockIdx.x;
  const unsigned int epoch = ll_epoch_now(p);  // read before any waiting: it moves when the call is complete
  const unsigned long long* input = p.ll_input + ((epoch & 1u) != 0 ? p.ll_parity_words : 0);
  const long long slot_words = static_cast<long long>(p.m) * p.ll_slot_cols;
  const long long out_cols = p.ll_reduce != 0 ? p.ll_slot_cols : static_cast<long long>(p.ll_slots) * p.ll_slot_cols;
  const long long total = static_cast<long long>(p.m) * out_cols;
  const unsigned long long start = global_timer_ns();
  bool gave_up = false;
  auto* out = static_cast<unsigned short*>(p.ll_output);
  for (long long e = (static_cast<long long>(cta_index) * blockDim.x) + threadIdx.x; e < total;
       e += static_cast<long long>(ctas_total) * blockDim.x) {
    const long long row = e / out_cols;
    const long long col = e - (row * out_cols);
    const unsigned long long* word[kMaxPeers + 1];
    unsigned long long seen[kMaxPeers + 1];
    int words = 1;
    if (p.ll_reduce != 0) {
      words = p.ll_slots;
#pragma unroll
      for (int s = 0; s < kMaxPeers + 1; ++s) {
        word[s] = input + (s * slot_words) + (row * p.ll_slot_cols) + col;
      }
    } else {
      const long long s = col / p.ll_slot_cols;
      word[0] = input + (s * slot_words) + (row * p.ll_slot_cols) + (col - (s * p.ll_slot_cols));
    }
#pragma unroll
    for (int s = 0; s < kMaxPeers + 1; ++s) {
      if (s < words) {
        seen[s] = load_word_system(word[s]);
      }
    }
    float value = 0.0f;
#pragma unroll
    for (int s = 0; s < kMaxPeers + 1; ++s) {  // slots in order: the sum is reproducible
      if (s < words) {
        while (static_cast<unsigned int>(seen[s] >> 32) != epoch && !gave_up) {
          if (global_timer_ns() - start > p.peer_wait_ns) {
            gave_up = true;
            break;
          }
          seen[s] = load_word_system(word[s]);
        }
        value += __uint_as_float(static_cast<unsigned int>(seen[s]));
      }
    }
    out[e] = E::from_float(value);
  }
  if (gave_up) {
    atomicExch(p.status, static_cast<int>(kStatusPeerWaitTimeout));
  }
  if (p.ll_epoch_counter != nullptr) {
    // The last CTA to finish closes the call: every word has been read and every CTA has read the
    // epoch, so the counter may move on.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.ll_ticket, 1u) == ctas_total - 1) {
        *p.ll_ticket = 0u;
        *p.ll_epoch_counter = epoch;
        __threadfence();
      }
    }
  }
}

template <class E>
__device__ __forceinline__ void exchange_complete(const GemvParams& p) {
  if (p.ll_epoch != 0 || p.ll_epoch_counter != nullptr) {
    ll_receive<E>(p);
    return;
  }
  if (p.local_signal == nullptr) {
    return;
  }
  __shared__ int arrived_flag;
  __syncthreads();
  const unsigned int ctas_total = gridDim.x * gridDim.y;
  const unsigned int target = p.wait_value * ctas_total;
  const bool reduce = p.reduce_slots > 0;
  // The fused reduction is small (batch x n outputs): a handful of CTAs wait and share it, the
  // others leave at once, so that the next kernel in the stream can move in behind them.
  const unsigned int cta_index = (blockIdx.y * gridDim.x) + blockIdx.x;
  const unsigned int reducers = ctas_total < kReduceCtas ? ctas_total : kReduceCtas;
  const bool waiter = reduce ? cta_index < reducers : cta_index == 0;
  if (threadIdx.x == 0) {
    fence_acq_rel_system();  // release: this CTA's stores, local and remote, before the signals
    for (int peer = 0; peer < p.num_peers; ++peer) {
      red_add_system(p.peer_signal[peer]);
    }
    red_add_system(p.local_signal);
    if (waiter) {
      bool arrived = false;
      const unsigned long long start = global_timer_ns();
      for (;;) {
        const unsigned int seen = load_counter_system(p.local_signal);
        if (static_cast<int>(seen - target) >= 0) {
          arrived = true;
          break;
        }
        if (global_timer_ns() - start > p.peer_wait_ns) {
          break;
        }
        __nanosleep(40);
      }
      if (!arrived) {
        atomicExch(p.status, static_cast<int>(kStatusPeerWaitTimeout));
      }
      fence_acq_rel_system();  // acquire: the other GPUs' stores behind their signals
      arrived_flag = arrived ? 1 : 0;
    }
  }
  if (!reduce || !waiter) {
    return;
  }
  __syncthreads();
  if (arrived_flag == 0) {
    return;
  }
  // this CTA's slice of the [m][n] outputs, in units of 4 elements
  const long long units = (static_cast<long long>(p.m) * p.n) >> 2;
  const long long cta = cta_index;
  const long long per_cta = (units + reducers - 1) / reducers;
  const long long begin = cta * per_cta;
  long long end = begin + per_cta;
  end = end < units ? end : units;
  const long long slot_units = units;
  for (long long u = begin + threadIdx.x; u < end; u += blockDim.x) {
    float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < p.reduce_slots; ++s) {
      const float4 part = __ldcg(reinterpret_cast<const float4*>(p.reduce_input) + (s * slot_units) + u);
      total.x += part.x;
      total.y += part.y;
      total.z += part.z;
      total.w += part.w;
    }
    uint2 packed;
    packed.x = static_cast<uint32_t>(E::from_float(total.x)) | (static_cast<uint32_t>(E::from_float(total.y)) << 16);
    packed.y = static_cast<uint32_t>(E::from_float(total.z)) | (static_cast<uint32_t>(E::from_float(total.w)) << 16);
    reinterpret_cast<uint2*>(p.reduce_output)[u] = packed;
  }
}

// ---------------------------------------------------------------------------------------------
// The finish shared by the GEMV kernels, run by every warp of a CTA after the CTA-wide barrier that
// ends the runs: adds the per-warp partial-sum slots of each tile in warp order, stores tiles
// that lie wholly inside the CTA's packet range, hands tiles shared with neighbouring CTAs to the
// global slot + ticket protocol, and (multi-GPU calls) signals and awaits exchange completion.
// ---------------------------------------------------------------------------------------------
// Warp u's slot for its first tile is head_slots + u * head_stride, the one for its last tile
// tail_slots + u * tail_stride (strides in floats); each holds [ROWS][128] floats.
template <int ROWS, class E>
__device__ __forceinline__ void finish_cta(const GemvParams& p, const float* head_slots,
                                           uint32_t head_stride, const float* tail_slots,
                                           uint32_t tail_stride, int warp, int lane,
                                           int warps_per_cta, int row_tile, int row0, int m_act) {
  constexpr int M_TILE = ROWS;
  constexpr int kSlotFloats = ROWS * kTileCols;
  const uint32_t cta = blockIdx.x;
  const uint32_t workers = static_cast<uint32_t>(p.active_warps);
  const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);

  // ---- CTA-level finish ---------------------------------------------------------------------
  const uint32_t cta_first_run = cta * warps_per_cta;
  uint32_t cta_end_run = cta_first_run + warps_per_cta;
  cta_end_run = cta_end_run < workers ? cta_end_run : workers;
  const uint32_t cta_begin = run_begin(cta_first_run, p);
  const uint32_t cta_end = run_begin(cta_end_run, p);
  const uint32_t cta_first_tile = cta_begin / num_groups;
  const uint32_t cta_last_tile = (cta_end - 1) / num_groups;
  float* scratch = p.scratch + (static_cast<size_t>(row_tile) * gridDim.x * 2 * kSlotFloats);
  int* tickets = p.tickets + (static_cast<size_t>(row_tile) * p.num_tiles);

  for (uint32_t tile = cta_first_tile + warp; tile <= cta_last_tile; tile += warps_per_cta) {
    const uint32_t tile_lo = tile * num_groups;
    const uint32_t tile_hi = tile_lo + num_groups;
    const uint32_t lo = tile_lo > cta_begin ? tile_lo : cta_begin;
    const uint32_t hi = tile_hi < cta_end ? tile_hi : cta_end;
    const uint32_t run_a = run_owner(lo, p);
    const uint32_t run_b = run_owner(hi - 1, p);
    if (run_a == run_b && run_begin(run_a, p) <= tile_lo && run_begin(run_a + 1, p) >= tile_hi) {
      continue;  // one warp saw the whole tile and stored it
    }

    float sum[M_TILE][4];
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        sum[m][c] = 0.0f;
      }
    }
    for (uint32_t u = run_a; u <= run_b; ++u) {
      // the tile is run u's first tile exactly when the run starts inside it
      const uint32_t local = u - cta_first_run;
      const float* slot = run_begin(u, p) >= tile_lo ? head_slots + (local * head_stride)
                                                     : tail_slots + (local * tail_stride);
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        const float4 part = reinterpret_cast<const float4*>(slot + (m * kTileCols))[lane];
        sum[m][0] += part.x;
        sum[m][1] += part.y;
        sum[m][2] += part.z;
        sum[m][3] += part.w;
      }
    }

    if (cta_begin <= tile_lo && cta_end >= tile_hi) {
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        if (m < m_act) {
          store_tile_row<E>(p, row0 + m, tile, lane, sum[m]);
        }
      }
      continue;
    }

    const uint32_t cta_a = run_owner(tile_lo, p) / warps_per_cta;
    const uint32_t cta_b = run_owner(tile_hi - 1, p) / warps_per_cta;

    // The tile continues in ONE neighbouring CTA (the usual case when a CTA's share is at least
    // a tile): each element is swapped, together with a "present" mark, into the boundary's word
    // with one atomic. Whoever finds the neighbour's value there adds the two -- the sum of two
    // floats does not depend on their order -- stores the output and clears the word; whoever
    // finds it empty is done. One round trip to L2, no fence, no ticket, no second pass.
    if (ROWS <= 4 && p.exchange != nullptr && cta_b == cta_a + 1) {
      unsigned long long* area =
          p.exchange + ((((static_cast<size_t>(row_tile) * gridDim.x) + cta_a) * kSlotFloats) + (lane * 4));
      unsigned long long seen[M_TILE][4];
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const unsigned long long mine =
              (static_cast<unsigned long long>(kExchangePresent) << 32) | __float_as_uint(sum[m][c]);
          seen[m][c] = atomicExch(area + (m * kTileCols) + c, mine);
        }
      }
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        bool present[4];
        bool all = true;
        bool any = false;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          present[c] = static_cast<uint32_t>(seen[m][c] >> 32) == kExchangePresent;
          all = all && present[c];
          any = any || present[c];
          sum[m][c] += __uint_as_float(static_cast<uint32_t>(seen[m][c]));
        }
        if (!any) {
          continue;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (present[c]) {
            area[(m * kTileCols) + c] = 0ull;
          }
        }
        if (m >= m_act) {
          continue;
        }
        if (all) {
          store_tile_row<E>(p, row0 + m, tile, lane, sum[m]);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (present[c]) {
              store_tile_element<E>(p, row0 + m, tile, (lane * 4) + c, sum[m][c]);
            }
          }
        }
      }
      continue;
    }

    // The tile is shared by three or more CTAs: publish, take a ticket, last one finishes.
    float* mine = scratch + (((static_cast<size_t>(cta) * 2) + (cta_begin >= tile_lo ? 0 : 1)) *
                             kSlotFloats);
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      __stcg(reinterpret_cast<float4*>(mine + (m * kTileCols)) + lane,
             make_float4(sum[m][0], sum[m][1], sum[m][2], sum[m][3]));
    }
    __threadfence();
    __syncwarp();
    int ticket = 0;
    if (lane == 0) {
      ticket = atomicAdd(&tickets[tile], 1);
    }
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != static_cast<int>(cta_b - cta_a)) {
      continue;
    }
    __threadfence();

#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        sum[m][c] = 0.0f;
      }
    }
    // independent loads in flight per step (fewer for tall slots, to stay in registers); the order
    // of addition is fixed either way
    constexpr int kBatch = M_TILE <= 4 ? 4 : 1;
    for (uint32_t base = cta_a; base <= cta_b; base += kBatch) {
      float4 part[kBatch][M_TILE];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const uint32_t cc = base + i;
        if (cc <= cta_b) {
          const int which = run_begin(cc * warps_per_cta, p) >= tile_lo ? 0 : 1;
          const float* theirs =
              scratch + (((static_cast<size_t>(cc) * 2) + which) * kSlotFloats);
#pragma unroll
          for (int m = 0; m < M_TILE; ++m) {
            part[i][m] = __ldcg(reinterpret_cast<const float4*>(theirs + (m * kTileCols)) + lane);
          }
        } else {
#pragma unroll
          for (int m = 0; m < M_TILE; ++m) {
            part[i][m] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
#pragma unroll
        for (int m = 0; m < M_TILE; ++m) {
          sum[m][0] += part[i][m].x;
          sum[m][1] += part[i][m].y;
          sum[m][2] += part[i][m].z;
          sum[m][3] += part[i][m].w;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M_TILE; ++m) {
      if (m < m_act) {
        store_tile_row<E>(p, row0 + m, tile, lane, sum[m]);
      }
    }
    if (lane == 0) {
      tickets[tile] = 0;  // ready for the next call on this workspace
    }
  }

  // ---- exchange completion (multi-GPU calls only) ------------------------------------------
  exchange_complete<E>(p);
}

// Shared-memory plan of the stream kernel, used by host and device alike.
struct StreamSmem {
  uint32_t barriers;  // offset of warp 0's barriers (8 bytes per stage)
  uint32_t slots;     // offset of the per-warp partial-sum slots (2 x M_TILE x 128 floats each)
  uint32_t acts;      // offset of the per-warp staged activations (M_TILE x G 16-bit values each)
  uint32_t rings;     // offset of warp 0's ring (stages x packet)
  uint32_t total;
};
__host__ __device__ inline StreamSmem stream_smem_plan(int warps, int stages, int group,
                                                       int m_tile) {
  StreamSmem plan;
  plan.barriers = 0;
  plan.slots = ((static_cast<uint32_t>(warps) * stages * 8) + 127u) & ~127u;
  plan.acts = plan.slots + (static_cast<uint32_t>(warps) * 2 * m_tile * kTileCols * 4);
  plan.rings = plan.acts + (static_cast<uint32_t>(warps) * m_tile * group * 2);
  plan.total = plan.rings + (static_cast<uint32_t>(warps) * stages * packet_stride(group));
  return plan;
}

template <int G, int M_TILE, class Mode>
__global__ void __launch_bounds__(512, 1)
    w4a16_gemv_stream_kernel(const __grid_constant__ GemvParams p) {
  using E = typename Mode::Elem;
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kStageBytes = packet_stride(G);
  constexpr int kSlotFloats = M_TILE * kTileCols;

  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int warps_per_cta = static_cast<int>(blockDim.x) >> 5;
  const uint32_t cta = blockIdx.x;
  const uint32_t v = (cta * warps_per_cta) + warp;
  const uint32_t workers = static_cast<uint32_t>(p.active_warps);
  const bool active = v < workers;
  const int row_tile = static_cast<int>(blockIdx.y);
  const int row0 = row_tile * M_TILE;
  const int m_act = (p.m - row0) < M_TILE ? (p.m - row0) : M_TILE;
  const uint32_t num_groups = static_cast<uint32_t>(p.num_groups);

  const int stages = p.stages;
  const StreamSmem plan = stream_smem_plan(warps_per_cta, stages, G, M_TILE);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_addr = smem_base + plan.barriers + (warp * stages * 8);
  const uint32_t act_addr = smem_base + plan.acts + (warp * M_TILE * G * 2);
  const uint32_t ring_addr = smem_base + plan.rings + (warp * stages * kStageBytes);
  float* slots = reinterpret_cast<float*>(smem + plan.slots);  // [warp][2][kSlotFloats]

  const uint32_t p_begin = active ? run_begin(v, p) : 0;
  const uint32_t p_end = active ? run_begin(v + 1, p) : 0;
  const uint32_t first_tile = p_begin / num_groups;

  trace_mark(0);
  if (active) {
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
      float* slot = slots + (((warp * 2) + (tile == first_tile ? 0 : 1)) * kSlotFloats);
#pragma unroll
      for (int m = 0; m < M_TILE; ++m) {
        reinterpret_cast<float4*>(slot + (m * kTileCols))[lane] =
            make_float4(y[m][0], y[m][1], y[m][2], y[m][3]);
      }
    };
    auto after_wait = [&](float (&inv_rms)[M_TILE]) {
      if (p.norm_weight != nullptr) {
        cta_inverse_rms<M_TILE, E>(p, row0, m_act, inv_rms);
      }
    };
    (void)consume_packet_run<G, M_TILE, Mode>(p, ring_addr, bar_addr, act_addr, row0, m_act,
                                              p_begin, p_end, lane, y, on_tile_done, after_wait);
  } else {
    pdl_launch_dependents();
    pdl_wait_for_prerequisites();
    if (p.norm_weight != nullptr) {  // the CTA-wide step of the fused RMSNorm needs every warp
      float unused[M_TILE];
      cta_inverse_rms<M_TILE, E>(p, row0, m_act, unused);
    }
  }
  trace_mark(3);
  __syncthreads();
  trace_mark(4);

  finish_cta<M_TILE, E>(p, slots, 2 * kSlotFloats, slots + kSlotFloats, 2 * kSlotFloats, warp, lane,
                        warps_per_cta, row_tile, row0, m_act);
  trace_mark(5);
}

// ---------------------------------------------------------------------------------------------
// Caller-visible split-K (the reference's arc_w4a16_forward_split_k + reduce, arc_w4a16.cu
// :341-402): slice s covers groups [s*gps, min((s+1)*gps, NG)), gps = ceil(NG / S), and writes
// fp32 partials[s, m, n]. One CTA per (tile, slice); its warps take contiguous shares of the
// slice's packets and add their sums through shared memory in warp order.
// ---------------------------------------------------------------------------------------------
struct SplitKParams {
  GemvParams base;
  float* partials;  // [slices, m, n]
  int slices;
  int groups_per_slice;
};

template <int G, int M_TILE, class Mode>
__global__ void __launch_bounds__(128, 1)
    w4a16_split_k_kernel(const __grid_constant__ SplitKParams sp) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kStageBytes = packet_stride(G);
  constexpr int kWarps = 4;
  __shared__ float reduce_buf[kWarps][M_TILE][kTileCols];
  __shared__ __align__(16) unsigned short act_buf[kWarps][M_TILE][G];

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
    const uint32_t base_pkt = static_cast<uint32_t>(tile) * p.num_groups;
    auto keep = [](uint32_t, uint32_t, uint32_t) {};
    (void)consume_packet_run<G, M_TILE, Mode>(p, ring_addr, bar_addr,
                                              smem_addr(&act_buf[warp][0][0]), row0, m_act,
                                              base_pkt + w_begin, base_pkt + w_end, lane, y, keep);
  } else {
    pdl_launch_dependents();
    pdl_wait_for_prerequisites();
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

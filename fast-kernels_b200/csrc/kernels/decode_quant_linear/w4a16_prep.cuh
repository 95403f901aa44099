// Weight preparation and the small helper kernels around the GEMV: packet packing, the two
// dequantisers (bit-exact with the reference), the group-sum prepass and the split-K reduction.
#pragma once

#include "w4a16_common.cuh"

namespace fk_w4a16 {

// ---------------------------------------------------------------------------------------------
// pack: row-major nibbles q[n, k/2] + alpha/beta[n, k/G]  ->  ARC packets.
// Same bytes as the reference's pack_arc_packets_kernel (arc_w4a16.cu:87-122). One CTA of 128
// threads builds one packet; thread c reads column c's G/2 bytes with 128-bit loads and writes
// word r to packet_words[r * 128 + c], so every store instruction of a warp is one contiguous
// 128-byte line.
// ---------------------------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(128) pack_packets_kernel(const uint8_t* __restrict__ q,
                                                           const uint16_t* __restrict__ alpha,
                                                           const uint16_t* __restrict__ beta,
                                                           uint8_t* __restrict__ packets, int k,
                                                           int num_groups, long long total_packets) {
  constexpr int kWordRows = G / 8;
  constexpr int kVecs = kWordRows / 4;  // 128-bit loads per column
  const int c = static_cast<int>(threadIdx.x);
  for (long long pkt = blockIdx.x; pkt < total_packets; pkt += gridDim.x) {
    const long long tile = pkt / num_groups;
    const int group = static_cast<int>(pkt % num_groups);
    const long long row = (tile * kTileCols) + c;
    const uint8_t* src = q + (row * (k / 2)) + (static_cast<long long>(group) * (G / 2));
    uint8_t* packet = packets + (pkt * packet_stride(G));
    auto* words = reinterpret_cast<uint32_t*>(packet);
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(src) + v);
      words[(((v * 4) + 0) * kTileCols) + c] = w.x;
      words[(((v * 4) + 1) * kTileCols) + c] = w.y;
      words[(((v * 4) + 2) * kTileCols) + c] = w.z;
      words[(((v * 4) + 3) * kTileCols) + c] = w.w;
    }
    auto* scales = reinterpret_cast<uint16_t*>(packet + packet_q_bytes(G));
    scales[c] = alpha[(row * num_groups) + group];
    scales[kTileCols + c] = beta[(row * num_groups) + group];
  }
}

// ---------------------------------------------------------------------------------------------
// dequant: W[n, k] = round16( float(alpha) * q + float(beta) ), the reference's
// dequant_w4a16_kernel / dequant_arc_packets_kernel (arc_w4a16.cu:160-220). alpha * q is exact
// in fp32 (at most 11 x 4 significant bits), so a fused multiply-add and a multiply followed by
// an add round identically; results match the reference bit for bit. One thread expands one
// 32-bit word (8 weights) and stores 16 bytes.
// ---------------------------------------------------------------------------------------------
template <class E>
__device__ __forceinline__ uint4 dequant_word(uint32_t w, float a, float b) {
  unsigned short h[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float qv = static_cast<float>((w >> (4 * i)) & 0xfu);
    h[i] = E::from_float(fmaf(a, qv, b));
  }
  uint4 out;
  out.x = h[0] | (static_cast<uint32_t>(h[1]) << 16);
  out.y = h[2] | (static_cast<uint32_t>(h[3]) << 16);
  out.z = h[4] | (static_cast<uint32_t>(h[5]) << 16);
  out.w = h[6] | (static_cast<uint32_t>(h[7]) << 16);
  return out;
}

template <int G, class E>
__global__ void __launch_bounds__(256) dequant_rowmajor_kernel(const uint8_t* __restrict__ q,
                                                               const uint16_t* __restrict__ alpha,
                                                               const uint16_t* __restrict__ beta,
                                                               uint16_t* __restrict__ out,
                                                               long long total_words, int k,
                                                               int num_groups) {
  const int words_per_row = k / 8;
  for (long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x) + threadIdx.x;
       idx < total_words; idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / words_per_row;
    const int word = static_cast<int>(idx % words_per_row);
    const int group = (word * 8) / G;
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(q) + idx);
    const float a = E::to_float(alpha[(row * num_groups) + group]);
    const float b = E::to_float(beta[(row * num_groups) + group]);
    reinterpret_cast<uint4*>(out)[idx] = dequant_word<E>(w, a, b);
  }
}

template <int G, class E>
__global__ void __launch_bounds__(256) dequant_packets_kernel(const uint8_t* __restrict__ packets,
                                                              uint16_t* __restrict__ out,
                                                              long long total_words, int k,
                                                              int num_groups) {
  constexpr int kWordRows = G / 8;
  // Index space: (packet, word-row r, column c) with c fastest, so packet reads are coalesced;
  // each thread writes 16 contiguous bytes of row c.
  for (long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x) + threadIdx.x;
       idx < total_words; idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % kTileCols);
    const long long rest = idx / kTileCols;
    const int r = static_cast<int>(rest % kWordRows);
    const long long pkt = rest / kWordRows;
    const long long tile = pkt / num_groups;
    const int group = static_cast<int>(pkt % num_groups);
    const uint8_t* packet = packets + (pkt * packet_stride(G));
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(packet) + (r * kTileCols) + c);
    const auto* scales = reinterpret_cast<const uint16_t*>(packet + packet_q_bytes(G));
    const float a = E::to_float(scales[c]);
    const float b = E::to_float(scales[kTileCols + c]);
    const long long row = (tile * kTileCols) + c;
    const long long out_elem = (row * k) + (static_cast<long long>(group) * G) + (r * 8);
    *reinterpret_cast<uint4*>(out + out_elem) = dequant_word<E>(w, a, b);
  }
}

// ---------------------------------------------------------------------------------------------
// group sums: S[m, g] = sum_{k in g} act[m, k] in fp32 (compute_arc_group_sums_kernel,
// arc_w4a16.cu:124-158). The additions are done in the same pairing order as the reference's
// 128-thread shared-memory tree -- element pairs first, then halving strides -- so fp16 results
// are bit-identical to it. One warp per (m, g).
// ---------------------------------------------------------------------------------------------
template <int G, class E>
__global__ void __launch_bounds__(128) group_sums_kernel(const uint16_t* __restrict__ act,
                                                         float* __restrict__ sums, int k,
                                                         int num_groups, long long total) {
  constexpr int kPairs = G / 2;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const long long item = (static_cast<long long>(blockIdx.x) * 4) + (threadIdx.x >> 5);
  if (item >= total) {
    return;
  }
  const long long row = item / num_groups;
  const int group = static_cast<int>(item % num_groups);
  const auto* pairs =
      reinterpret_cast<const uint32_t*>(act + (row * k) + (static_cast<long long>(group) * G));
  auto pair_sum = [&](int idx) {
    const uint32_t raw = pairs[idx];
    return E::to_float(static_cast<unsigned short>(raw & 0xffffu)) +
           E::to_float(static_cast<unsigned short>(raw >> 16));
  };
  float v = 0.0f;
  if (kPairs == 64) {
    v = pair_sum(lane) + pair_sum(lane + 32);
  } else if (lane < kPairs) {
    v = pair_sum(lane);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float other = __shfl_down_sync(0xffffffffu, v, off);
    if (off < kPairs) {
      v += other;
    }
  }
  if (lane == 0) {
    sums[item] = v;
  }
}

// out[m, n] = round16( sum_s partials[s, m, n] ), slices added in index order
// (reduce_arc_w4a16_split_k_partials_kernel, arc_w4a16.cu:388-402).
template <class E>
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partials,
                                                              uint16_t* __restrict__ out,
                                                              long long total, int slices) {
  const long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x) + threadIdx.x;
  if (idx >= total) {
    return;
  }
  float sum = 0.0f;
  for (int s = 0; s < slices; ++s) {
    sum += partials[(static_cast<long long>(s) * total) + idx];
  }
  out[idx] = E::from_float(sum);
}

// Host-resident activations: copies `count` 16-byte units from mapped (pinned) host memory into
// device memory. The loads cross PCIe before the kernel waits for the work ahead of it in the
// stream -- which may still be reading `dst` -- so their latency hides behind that work's tail.
struct StageHostParams {
  const uint4* src;  // device-side address of mapped host memory
  uint4* dst;
  int count;
};
__global__ void __launch_bounds__(256) stage_host_activations_kernel(
    const __grid_constant__ StageHostParams sp) {
  const int i = static_cast<int>((blockIdx.x * blockDim.x) + threadIdx.x);
  pdl_launch_dependents();
  uint4 value = make_uint4(0u, 0u, 0u, 0u);
  if (i < sp.count) {
    value = __ldcv(sp.src + i);  // never from a cache: the host rewrites this memory between calls
  }
  pdl_wait_for_prerequisites();
  if (i < sp.count) {
    sp.dst[i] = value;
  }
}

}  // namespace fk_w4a16

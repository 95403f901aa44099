// Paged-KV decode attention for sm_100a: one query token per request, grouped-query heads, rotary
// embedding applied in the kernel, pages of bf16 / e4m3 / int8 keys and values.
//
// What it computes is what the reference's two kernels compute
// (csrc/kernels/clustered_page_decode/clustered_page_decode.cu:111-328 and :330-669): for request b,
// query head h of kv head j, over the tokens of the request's runs of pages,
//     logit_t = scale * < R(pos_q) q , R(pos_t) k_t >,   out = sum_t softmax(logit)_t * v_t
// with pos_q = seq_len - 1, pos_t = logical_page * page_size + token, R the Llama pair rotation
// (:96-108), quantised elements multiplied by their scale (:74-94: keys one scale per page, kv
// head and 64-dim block; values one per token and 64-dim block).
//
// How it is laid out here:
//  * The unit of work is 16 tokens of one page (a page of 32 tokens is two units). A thread block
//    serves one (request, kv head, tile of GT query heads, split s of S): the flattened list of
//    the request's units is dealt round-robin over the S blocks, a block's units round-robin over
//    its warps. The S partial results (running maximum, denominator, weighted
//    value sum) meet in global scratch; the block that takes the last ticket adds them in split
//    order and writes the output, so results do not depend on timing.
//  * Every warp streams its own units: a unit's keys and values for one kv head are two contiguous
//    blocks of 16 x head_dim elements (plus the values' scales), fetched by bulk asynchronous
//    copies into a ring of `stages` buffers per warp, completion on an mbarrier. No block-wide
//    barrier while units stream.
//  * Lane l owns head dimensions [l*EPL, (l+1)*EPL) (EPL = head_dim / 32) of every key, value,
//    query and accumulator. The rotated, scaled query of the tile's heads sits in registers. Only
//    the token part of a key's rotation is applied to the key (a table e^{i t theta}, t < 16,
//    built once per block); the unit's part goes to the query:
//    <R(a) q, R(P + t) k> = <R(a - P) q, R(t) k>. Key scales and the softmax scale ride on the
//    query as well, value scales on the probabilities.
//  * Partial dot products of TB tokens x GT heads (32 values per lane) are summed across lanes by
//    a butterfly that halves the values a lane keeps at every step: one shuffle per value instead
//    of five, and lane l ends up with the logit of (token l / GT, head l % GT).
//  * Every wait on a copy is bounded: on a time-out the block sets the status word, gives up on
//    its pages and still takes part in the barriers and the ticket.
#pragma once

#include <cuda_fp8.h>

#include "../decode_quant_linear/w4a16_common.cuh"
#include "page_decode_mma.cuh"

namespace fk_page_decode {

using fk_w4a16::lds128;
using fk_w4a16::lds64;
using fk_w4a16::mbar_expect_tx;
using fk_w4a16::mbar_init;
using fk_w4a16::mbar_init_fence;
using fk_w4a16::mbar_wait_bounded;
using fk_w4a16::proxy_fence_async;
using fk_w4a16::smem_addr;

constexpr int kKvBf16 = 0;
constexpr int kKvFp8 = 1;
constexpr int kKvInt8 = 2;
constexpr int kUnitTokens = 16;       // tokens per unit of work; pages hold one or two units
constexpr int kEntryCapacity = 512;   // units of one block that are listed in shared memory at a time
constexpr int kMaxWarpsWide = 8;      // head tiles of 8: ~208 registers per thread
constexpr int kMaxWarpsNarrow = 12;   // head tiles of 1, 2, 4: up to ~160 registers per thread
constexpr int kMaxPairs = 64;
constexpr int kMaxSplits = 64;
constexpr int kStatusCopyWaitTimeout = 1;

__host__ __device__ constexpr int max_warps_for(int group_tile) {
  return group_tile >= 8 ? kMaxWarpsWide : kMaxWarpsNarrow;
}

struct DecodeParams {
  const uint16_t* query;
  const uint8_t* key_pages;
  const uint8_t* value_pages;
  const float* key_scales;
  const float* value_scales;
  const int32_t* run_base_pages;
  const int32_t* run_page_counts;
  const int32_t* run_logical_starts;
  const int32_t* run_last_page_lens;
  const int32_t* request_run_offsets;
  const int32_t* seq_lens;
  uint16_t* output;
  float* partials;    // [task * splits + s][GT][head_dim + 4]: weighted values, maximum, denominator, pad
  unsigned* tickets;  // [task], zero between calls
  int* status;
  int num_q_heads;
  int num_kv_heads;
  int group_size;
  int head_tiles;
  int page_size;      // 16 or 32
  int splits;
  int stages;
  int early_descriptors;  // the run arrays and seq_lens are not written by the preceding kernel
  int cluster_merge;      // the S blocks of a task are one thread-block cluster: merge through shared memory
  float scale_log2e;  // softmax scale times log2(e): the kernel works with exp2
  float inv_freq[kMaxPairs];  // theta^(-2 i / head_dim), rounded once from double
};

__host__ __device__ constexpr int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Shared-memory layout, the same arithmetic on host (size) and device (offsets).
template <int D, int KV, bool ROT, int GT, bool MMA = false>
struct Layout {
  static constexpr int kElemBytes = KV == kKvBf16 ? 2 : 1;
  static constexpr bool kQuant = KV != kKvBf16;
  static constexpr int kDimBlocks = D / 64;
  static constexpr int kDbq = kQuant ? kDimBlocks : 1;  // copies of a probability (one per value scale)
  static constexpr int kUnitBytes = kUnitTokens * D * kElemBytes;
  static constexpr int kVScaleBytes = kQuant ? kUnitTokens * kDimBlocks * 4 : 0;
  // The tensor-core variant keeps pairs of rows with a skew between them (see page_decode_mma.cuh).
  static constexpr bool kPairStage = MMA && !kQuant;  // bf16 pages land in the tensor-core layout directly
  static constexpr int kUnitSmem = kPairStage ? MmaWarp<D, false>::kUnitSmem : kUnitBytes;
  // 8-bit pages on tensor cores: the unit is converted to bf16 rows (keys, values) per warp
  static constexpr int kConvertedBytes = (MMA && kQuant) ? 2 * MmaWarp<D, false>::kUnitSmem : 0;
  static constexpr int kStageBytes = 2 * kUnitSmem;  // keys, then values, of one unit
  static constexpr int kRopeBytes = ROT ? 0 : kUnitTokens * D * 4;  // per token and pair: cos, sin
  // The key block of a stage and the rotation table are addressed as base ^ (row offset), which
  // needs them aligned to their own size (16 rows). Both sit at the end of the layout behind one
  // run-time alignment of the shared-memory address; kAlign bytes of slack pay for it.
  static constexpr int kAlign = ROT ? kUnitBytes : (kRopeBytes > kUnitBytes ? kRopeBytes : kUnitBytes);
  static constexpr int kEpl = D / 32;

  int bars, entries, kscales, inv_freq, vscales, probs, alphas, converted, tail, total;

  __host__ __device__ Layout(int warps, int stages) {
    int at = 0;
    bars = at;
    at += round_up(warps * stages * 8, 128);
    entries = at;
    at += kEntryCapacity * 8;
    kscales = at;
    at += kQuant ? kEntryCapacity * kDimBlocks * 4 : 0;
    inv_freq = at;
    at += kMaxPairs * 4;
    vscales = at;
    at += round_up(warps * stages * kVScaleBytes, 128);
    probs = at;
    // each probability twice: a ready-made pair (p, p); the tensor-core form only needs D floats of scratch
    at += warps * (MMA ? D * 4 : kUnitTokens * kDbq * GT * 8);
    alphas = at;
    at += round_up(warps * GT * 4, 128);
    converted = at;
    at += warps * kConvertedBytes;
    tail = at;  // aligned at run time: rotation table, then the ring
    const int ring_bytes = warps * stages * kStageBytes;
    // after the stream the ring's memory holds per-warp results [warps][GT][D + 2], then (merging
    // block of a task) the splits' maxima and weights [GT][kMaxSplits] twice, then the block's own
    // result [GT][D + 4] for the merge inside a cluster
    const int merge_bytes = round_up(warps * GT * (D + 2), 4) * 4 + 2 * GT * kMaxSplits * 4 + GT * (D + 4) * 4;
    at += kAlign + kRopeBytes + (ring_bytes > merge_bytes ? ring_bytes : merge_bytes);
    total = at;
  }
};

__device__ __forceinline__ void bulk_copy_plain(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// Thread-block cluster: barrier, address of a peer block's shared memory, loads from it.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 ld_cluster_f2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

// Packed fp32 pairs: sm_100 multiplies and accumulates two fp32 lanes with one instruction
// (fma.rn.f32x2 / mul.rn.f32x2 on 64-bit registers), each lane an ordinary IEEE fma. The inner
// products below keep accumulators, queries, keys and values as such pairs.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// EPL elements of one row of a page, starting at this lane's first dimension, as floats
// (unscaled: the scale rides on the query or the probability).
template <int KV, int EPL>
__device__ __forceinline__ void load_elements(uint32_t addr, float (&x)[EPL]) {
  if constexpr (KV == kKvBf16) {
    uint32_t w[EPL / 2];
    if constexpr (EPL == 4) {
      const uint2 v = lds64(addr);
      w[0] = v.x;
      w[1] = v.y;
    } else {
      w[0] = lds32(addr);
    }
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
    const uint32_t w = EPL == 4 ? lds32(addr) : lds16(addr);
    if constexpr (KV == kKvInt8) {
      // byte + 128 dropped into the mantissa of 2^23: exact, no integer-to-float conversion
      const uint32_t u = w ^ 0x80808080u;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        x[i] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540u + i)) - 8388736.0f;
      }
    } else {
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) {
        const __half2_raw h2 =
            __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((w >> (16 * i)) & 0xffffu), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
      }
    }
  }
}

// Four 8-bit elements of a page (one word) as two f16 pairs, exactly. SHIFTED (e4m3 only): by bit
// operations alone, which yields the values times 2^-8 -- sign | magnitude bits << 7 reads, as f16,
// as the same mantissa under an exponent 8 lower, subnormals included.
// The conversion instruction (two bytes per cvt) and the bit operations (seven per four bytes) run
// on different pipes, but bit operations for both keys and values are the quickest (32 requests x
// 8 kv heads x 4096 tokens: 93.9 us; keys only 95.4, values only 96.8; before the rest of the
// per-unit work was trimmed the mix with keys by cvt had been ahead, 107.8 against 109.0).
constexpr bool kFp8ShiftKeys = true;
constexpr bool kFp8ShiftValues = true;
template <int KV, bool SHIFTED = false>
__device__ __forceinline__ void bytes_to_half2(uint32_t w, uint32_t& first, uint32_t& second) {
  if constexpr (KV == kKvFp8 && SHIFTED) {
    const uint32_t upper = ((w >> 1) & 0x3f3f3f3fu) | (w & 0x80808080u);  // per byte: sign, magnitude >> 1
    const uint32_t lower = (w << 7) & 0x80808080u;                        // per byte: lowest magnitude bit, on top
    first = __byte_perm(upper, lower, 0x1504u);
    second = __byte_perm(upper, lower, 0x3726u);
  } else if constexpr (KV == kKvInt8) {
    // byte + 128 dropped into the mantissa of 1024 (0x64xx = 1024 + x + 128), then minus 1152
    const uint32_t u = w ^ 0x80808080u;
    const __half2 offset = __half2half2(__ushort_as_half(0x6480));
    const uint32_t lo = __byte_perm(u, 0x64646464u, 0x4140u), hi = __byte_perm(u, 0x64646464u, 0x4342u);
    const __half2 a = __hsub2(*reinterpret_cast<const __half2*>(&lo), offset);
    const __half2 b = __hsub2(*reinterpret_cast<const __half2*>(&hi), offset);
    first = *reinterpret_cast<const uint32_t*>(&a);
    second = *reinterpret_cast<const uint32_t*>(&b);
  } else {
    const __half2_raw a = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xffffu), __NV_E4M3);
    const __half2_raw b = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
    first = static_cast<uint32_t>(a.x) | (static_cast<uint32_t>(a.y) << 16);
    second = static_cast<uint32_t>(b.x) | (static_cast<uint32_t>(b.y) << 16);
  }
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Sum over lanes of NV values per lane; lane l is left with the total of value (l % NV) in v[0].
// Value index = token * GT + head. A step with lane offset o settles index bit o: a lane keeps the
// half whose bit equals its own lane bit and hands the other half to its partner. For the token
// bits (o >= GT) the caller has ALREADY permuted the tokens per lane -- local token tl stands for
// token tl ^ ((lane / GT) % TB) -- so the half to keep is always the lower one and no selects are
// needed; the head bits (o < GT) cannot be permuted that way (the queries sit in registers).
// The permutation makes the row address of a token a per-lane value instead of an immediate (a
// few integer instructions per token), which pays from head tiles of 4 on: FLIP says whether the
// caller did it.
template <int NV, int GT, bool FLIP>
__device__ __forceinline__ void butterfly_sum(float (&v)[NV], int lane) {
#pragma unroll
  for (int o = NV / 2; o >= 1; o >>= 1) {
    if (FLIP && o >= GT) {
#pragma unroll
      for (int i = 0; i < o; ++i) {
        v[i] += __shfl_xor_sync(0xffffffffu, v[i + o], o);
      }
    } else {
      const bool upper = (lane & o) != 0;
#pragma unroll
      for (int i = 0; i < o; ++i) {
        const float keep = upper ? v[i + o] : v[i];
        const float give = upper ? v[i] : v[i + o];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, give, o);
      }
    }
  }
#pragma unroll
  for (int o = NV; o < 32; o <<= 1) {
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
  }
}

template <int D, int KV, bool ROT, int GT, bool MMA = false>
__global__ void __launch_bounds__((MMA ? kMaxWarpsNarrow : max_warps_for(GT)) * 32, 1)
    page_decode_kernel(const __grid_constant__ DecodeParams p) {
  static_assert(!MMA || (ROT && GT == 8), "the tensor-core variant: rotated keys, tiles of 8");
  using L = Layout<D, KV, ROT, GT, MMA>;
  constexpr bool PAIRS = L::kPairStage;  // the stage itself holds skewed row pairs (bf16 pages on tensor cores)
  constexpr int EPL = L::kEpl;
  constexpr int EB = L::kElemBytes;
  constexpr bool QUANT = L::kQuant;
  constexpr int DB = L::kDimBlocks;
  constexpr int DBQ = L::kDbq;
  constexpr int U = kUnitTokens;
  constexpr int TB = (32 / GT) < U ? (32 / GT) : U;  // tokens per butterfly round
  constexpr int NV = TB * GT;                       // values per lane per round
  constexpr int NR = U / TB;                        // rounds per unit
  constexpr int CAP = kEntryCapacity;
  constexpr int ROW = D + 4;  // floats per head of a partial result in global scratch (16-byte rows)
  static_assert(NV <= 32 && (NV & (NV - 1)) == 0);

  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int scan_totals[kMaxWarpsNarrow];
  __shared__ int last_flag;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int warps = blockDim.x >> 5;
  const int threads = blockDim.x;
  const int stages = p.stages;
  const L layout(warps, stages);
  const int PS = p.page_size;
  const int UPP = PS / U;  // units per page: 1 or 2
  const int upp_shift = UPP - 1;  // log2(UPP)

  const int S = p.splits;
  const int task = blockIdx.x / S;
  const int split = blockIdx.x - task * S;
  const int tasks_per_request = p.num_kv_heads * p.head_tiles;
  const int request = task / tasks_per_request;
  const int within = task - request * tasks_per_request;
  const int kv_head = within / p.head_tiles;
  const int tile = within - kv_head * p.head_tiles;
  const int tile_base = tile * GT;
  const int tile_heads = min(GT, p.group_size - tile_base);
  const int first_q_head = kv_head * p.group_size + tile_base;
  const size_t out_base = (static_cast<size_t>(request) * p.num_q_heads + first_q_head) * D;

  const uint32_t bars = smem_addr(smem + layout.bars);
  int2* entries = reinterpret_cast<int2*>(smem + layout.entries);
  float* kscales = reinterpret_cast<float*>(smem + layout.kscales);
  float* inv_freq_s = reinterpret_cast<float*>(smem + layout.inv_freq);
  float2* probs = reinterpret_cast<float2*>(smem + layout.probs) + warp * (MMA ? D / 2 : U * DBQ * GT);
  float* alphas = reinterpret_cast<float*>(smem + layout.alphas) + warp * GT;
  const float* vscales = reinterpret_cast<const float*>(smem + layout.vscales) + warp * stages * (L::kVScaleBytes / 4);
  const uint32_t vscales_addr = smem_addr(smem + layout.vscales) + warp * stages * L::kVScaleBytes;
  // rotation table and ring behind one run-time alignment (see Layout)
  const uint32_t tail_addr = (smem_addr(smem + layout.tail) + (L::kAlign - 1)) & ~static_cast<uint32_t>(L::kAlign - 1);
  unsigned char* tail_ptr = smem + layout.tail + (tail_addr - smem_addr(smem + layout.tail));
  float* rope = reinterpret_cast<float*>(tail_ptr);
  const uint32_t rope_addr = tail_addr;
  unsigned char* ring_ptr = tail_ptr + L::kRopeBytes;
  const uint32_t ring = tail_addr + L::kRopeBytes + warp * stages * L::kStageBytes;
  const uint32_t my_bars = bars + warp * stages * 8;

  for (int i = tid; i < warps * stages; i += threads) {
    mbar_init(bars + i * 8, 1);
  }
  for (int i = tid; i < D / 2; i += threads) {  // a block may have fewer threads than pairs
    inv_freq_s[i] = p.inv_freq[i];
  }
  mbar_init_fence();
  // Programmatic dependent launch (no-ops without the launch attribute): the next kernel of the
  // stream may be scheduled from here on. What follows up to the wait touches no global memory:
  // the table e^{i t theta} of the keys' token rotation.
  fk_w4a16::pdl_launch_dependents();
  __syncthreads();
  if constexpr (!ROT) {
    // rope[(t * D/2 + pair) * 2 + {0, 1}] = cos, sin of t * theta_pair; lane l owns pairs
    // l * EPL/2 ..., i.e. floats [t * D + l * EPL, + EPL)
    for (int idx = tid; idx < U * (D / 2); idx += threads) {
      const int t = idx / (D / 2);
      const int pair = idx - t * (D / 2);
      float sn, cs;
      sincosf(static_cast<float>(t) * inv_freq_s[pair], &sn, &cs);
      *reinterpret_cast<float2*>(&rope[idx * 2]) = make_float2(cs, sn);
    }
  }
  // Nothing of global memory is read before the previous kernel of the stream has completed --
  // except, if the caller says that kernel does not write them, the request descriptors.
  if (!p.early_descriptors) {
    fk_w4a16::pdl_wait_for_prerequisites();
  }

  const int query_position = p.seq_lens[request] - 1;
  const int run_begin = p.request_run_offsets[request];
  const int run_end = p.request_run_offsets[request + 1];
  if (query_position < 0 || run_begin >= run_end) {
    if (p.early_descriptors) {
      fk_w4a16::pdl_wait_for_prerequisites();
    }
    if (split == 0) {
      for (int idx = tid; idx < tile_heads * D; idx += threads) {
        p.output[out_base + idx] = 0;
      }
    }
    return;  // every block of the task takes this branch: nobody waits for a ticket
  }

  float q_in[GT][EPL];  // this lane's part of the tile's queries, loaded once the descriptors are read
  f32x2 acc[GT][EPL / 2];  // weighted values, pairs of neighbouring dimensions
#pragma unroll
  for (int h = 0; h < GT; ++h) {
#pragma unroll
    for (int e = 0; e < EPL / 2; ++e) {
      acc[h][e] = pack2(0.0f, 0.0f);
    }
  }
  // Softmax state of head (lane % GT): the running maximum is the same on all lanes of a head,
  // the denominator is this lane's share (summed over lanes at the end).
  float m_run = -INFINITY;
  float l_run = 0.0f;
  const int my_head = lane % GT;
  const int my_token = (lane % NV) / GT;  // within a butterfly round
  constexpr bool FLIP = GT >= 4;
  const int token_flip = FLIP ? (lane / GT) % TB : 0;  // local token tl of a round stands for token tl ^ token_flip
  const bool holds_value = lane < NV;
  const int lane_db = (DB == 2) ? (lane >> 4) : 0;

  uint32_t iteration = 0;  // units this warp has consumed: stage = iteration % stages
  bool failed = false;

  // entries[i] = (physical unit = page * UPP + sub, (logical unit << 5) | tokens in the unit)
  auto issue = [&](int entry_index, int stage) {
    const int physical_unit = entries[entry_index].x;
    const int page = physical_unit >> upp_shift;
    const int sub = physical_unit & (UPP - 1);
    // this kv head's unit among all units of the pool (a page of one kv head is UPP units in a row)
    const size_t pool_unit = ((static_cast<size_t>(page) * p.num_kv_heads + kv_head) << upp_shift) + sub;
    const size_t offset = pool_unit * L::kUnitBytes;
    const uint32_t dst = ring + stage * L::kStageBytes;
    const uint32_t bar = my_bars + stage * 8;
    if constexpr (PAIRS) {
      // called by the whole warp: lane 0 announces the bytes, then lanes 0-7 fetch one pair of key
      // rows each and lanes 8-15 one pair of value rows each into the skewed pairs of the stage
      if (lane == 0) {
        mbar_expect_tx(bar, 2 * L::kUnitBytes);
      }
      __syncwarp();
      if (lane < 16) {
        const int pair = lane & 7;
        const uint8_t* base = lane < 8 ? p.key_pages : p.value_pages;
        bulk_copy_plain(dst + (lane < 8 ? 0 : L::kUnitSmem) + pair * MmaWarp<D, false>::kPairBytes,
                        base + offset + pair * (2 * D * EB), 2 * D * EB, bar);
      }
    } else {
      mbar_expect_tx(bar, 2 * L::kUnitBytes + L::kVScaleBytes);
      bulk_copy_plain(dst, p.key_pages + offset, L::kUnitBytes, bar);
      bulk_copy_plain(dst + L::kUnitBytes, p.value_pages + offset, L::kUnitBytes, bar);
      if constexpr (QUANT) {
        bulk_copy_plain(vscales_addr + stage * L::kVScaleBytes, p.value_scales + pool_unit * (U * DB),
                        L::kVScaleBytes, bar);
      }
    }
  };
  using Tensor = MmaWarp<D, L::kQuant>;  // 8-bit pages: f16 operands
  constexpr bool kShiftKeys = KV == kKvFp8 && kFp8ShiftKeys;
  constexpr bool kShiftValues = KV == kKvFp8 && kFp8ShiftValues;
  Tensor tensor;  // state of the tensor-core variant (unused otherwise)

  float inv_freq_lane[EPL / 2];
  // Rotation of the query for the current unit, e^{i (a - P) theta} (for keys that come rotated:
  // e^{i a theta}, fixed). A warp's units normally follow one another at a fixed distance, so the
  // next rotation is the current one times a fixed e^{-i 16 step theta}; sincosf is called afresh
  // whenever the distance differs and every kResync units, which keeps rounding from piling up.
  constexpr int kResync = 32;
  float rot_cos[EPL / 2], rot_sin[EPL / 2], step_cos[EPL / 2], step_sin[EPL / 2];
  int rot_unit = 0, rot_age = kResync;
  const int unit_step = S * warps;
  // per-lane parts of the key and table addresses (see the logits loop)
  const uint32_t flip_row = static_cast<uint32_t>(token_flip);

  int total_units = 0;
  for (int round = 0;; ++round) {
    const int local_base = round * CAP;
    // ---- list this block's units: flattened unit q of the request belongs to split q % S ----
    int carry = 0;
    for (int r0 = run_begin; r0 < run_end; r0 += threads) {
      const int r = r0 + tid;
      const bool valid = r < run_end;
      const int pages = valid ? max(p.run_page_counts[r], 0) : 0;
      const int base = valid ? p.run_base_pages[r] : 0;
      const int logical_start = valid ? p.run_logical_starts[r] : 0;
      const int last_len = valid ? min(max(p.run_last_page_lens[r], 0), PS) : 0;
      const int count = pages * UPP;
      int inclusive = count;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, inclusive, o);
        if (lane >= o) {
          inclusive += up;
        }
      }
      if (lane == 31) {
        scan_totals[warp] = inclusive;
      }
      __syncthreads();
      int before = 0, chunk_total = 0;
      for (int w = 0; w < warps; ++w) {
        const int v = scan_totals[w];
        before += w < warp ? v : 0;
        chunk_total += v;
      }
      const int first = carry + before + inclusive - count;
      if (count > 0) {
        int q = first + ((split - first % S) + S) % S;
        for (; q < first + count; q += S) {
          const int i = (q - split) / S - local_base;
          if (i >= CAP) {
            break;
          }
          if (i >= 0) {
            const int off = q - first;           // unit within the run
            const int page_off = off >> upp_shift;
            const int sub = off & (UPP - 1);
            const int page_tokens = page_off == pages - 1 ? last_len : PS;
            const int tokens = min(max(page_tokens - sub * U, 0), U);
            entries[i] = make_int2((base + page_off) * UPP + sub, (((logical_start + page_off) * UPP + sub) << 5) | tokens);
          }
        }
      }
      carry += chunk_total;
      __syncthreads();
    }
    total_units = carry;
    const int mine = total_units > split ? (total_units - split + S - 1) / S : 0;
    const int in_round = max(0, min(CAP, mine - local_base));

    // ---- first copies of the round, then the per-block tables while they fly ----
    if (round == 0 && p.early_descriptors) {
      fk_w4a16::pdl_wait_for_prerequisites();
    }
    if ((PAIRS || lane == 0) && !failed) {
      for (int k = 0; k < stages; ++k) {
        const int entry_index = warp + k * warps;
        if (entry_index < in_round) {
          issue(entry_index, (iteration + k) % stages);
        }
      }
    }
    if (round == 0 && MMA) {
      const int head = lane >> 2;
      tensor.prepare(head < tile_heads ? p.query + out_base + static_cast<size_t>(head) * D : nullptr, lane,
                     query_position, inv_freq_s, p.scale_log2e, reinterpret_cast<float*>(probs),
                     kShiftKeys ? 256.0f : 1.0f, kShiftValues ? 256.0f : 1.0f);
    }
    if (round == 0 && !MMA) {
#pragma unroll
      for (int h = 0; h < GT; ++h) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          q_in[h][e] = 0.0f;
        }
        if (h < tile_heads) {
          const uint16_t* src = p.query + out_base + static_cast<size_t>(h) * D + lane * EPL;
#pragma unroll
          for (int e = 0; e < EPL; e += 2) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(src + e);
            q_in[h][e] = __uint_as_float(w << 16);
            q_in[h][e + 1] = __uint_as_float(w & 0xffff0000u);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) {
        inv_freq_lane[i] = inv_freq_s[lane * (EPL / 2) + i];
        if constexpr (ROT) {
          sincosf(static_cast<float>(query_position) * inv_freq_lane[i], &rot_sin[i], &rot_cos[i]);
        } else {
          sincosf(static_cast<float>(-U * unit_step) * inv_freq_lane[i], &step_sin[i], &step_cos[i]);
        }
      }
    }
    if constexpr (QUANT) {
      for (int idx = tid; idx < in_round * DB; idx += threads) {
        const int i = idx / DB;
        const int b = idx - i * DB;
        const size_t page_head = static_cast<size_t>(entries[i].x >> upp_shift) * p.num_kv_heads + kv_head;
        kscales[idx] = p.key_scales[page_head * DB + b];
      }
    }
    __syncthreads();

    // ---- this warp's units ----
    for (int i = warp; i < in_round && !failed; i += warps, ++iteration) {
      const int stage = iteration % stages;
      if (!mbar_wait_bounded(my_bars + stage * 8, (iteration / stages) & 1)) {
        failed = true;
        if (lane == 0) {
          atomicExch(p.status, kStatusCopyWaitTimeout);
        }
        break;
      }
      const int2 entry = entries[i];
      const int logical_unit = entry.y >> 5;
      const int tokens = entry.y & 31;
      const uint32_t k_stage = ring + stage * L::kStageBytes;
      const uint32_t v_stage = k_stage + L::kUnitSmem;
      if constexpr (MMA && QUANT) {
        // 8-bit unit -> f16 rows in the tensor-core layout (exact: int8 and e4m3 values are f16
        // values); scales stay out of it. A lane takes 8 elements of a row: one 8-byte load, one
        // 16-byte store, both free of bank conflicts.
        const uint32_t k_rows = smem_addr(smem + layout.converted) + warp * L::kConvertedBytes;
        const uint32_t v_rows = k_rows + Tensor::kUnitSmem;
        constexpr int kLanesPerRow = D / 8;
        constexpr int kRowsPerStep = 32 / kLanesPerRow;
        const uint32_t to = Tensor::row_address(0, lane / kLanesPerRow) + (lane % kLanesPerRow) * 16;
#pragma unroll
        for (int step = 0; step < U / kRowsPerStep; ++step) {
          const uint2 kb = lds64(k_stage + step * 256 + lane * 8);
          const uint2 vb = lds64(v_stage + step * 256 + lane * 8);
          uint32_t kh[4], vh[4];
          bytes_to_half2<KV, kShiftKeys>(kb.x, kh[0], kh[1]);
          bytes_to_half2<KV, kShiftKeys>(kb.y, kh[2], kh[3]);
          bytes_to_half2<KV, kShiftValues>(vb.x, vh[0], vh[1]);
          bytes_to_half2<KV, kShiftValues>(vb.y, vh[2], vh[3]);
          const uint32_t at = to + step * (kRowsPerStep / 2) * Tensor::kPairBytes;
          sts128(k_rows + at, make_uint4(kh[0], kh[1], kh[2], kh[3]));
          sts128(v_rows + at, make_uint4(vh[0], vh[1], vh[2], vh[3]));
        }
        if (tokens < U) {
          // value rows past the unit's end may hold anything; a zero weight times a NaN is a NaN
          __syncwarp();
          for (int idx = lane; idx < (U - tokens) * (D / 8); idx += 32) {
            const int row = tokens + idx / (D / 8);
            sts128(Tensor::row_address(v_rows, row) + (idx % (D / 8)) * 16, make_uint4(0u, 0u, 0u, 0u));
          }
        }
        float value_scales[DB][4];
        if (tokens == U) {
          Tensor::template lane_value_scales<DB, true>(vscales + stage * (L::kVScaleBytes / 4), tokens, lane,
                                                       value_scales);
        } else {
          Tensor::template lane_value_scales<DB, false>(vscales + stage * (L::kVScaleBytes / 4), tokens, lane,
                                                        value_scales);
        }
        __syncwarp();
        // the stage is read out: its next unit can fly while this one is worked on
        if (lane == 0 && i + stages * warps < in_round) {
          proxy_fence_async();
          issue(i + stages * warps, stage);
        }
        if (tokens == U) {
          tensor.template unit<DB, true>(k_rows, v_rows, tokens, lane, &kscales[i * DB], value_scales);
        } else {
          tensor.template unit<DB, false>(k_rows, v_rows, tokens, lane, &kscales[i * DB], value_scales);
        }
      } else if constexpr (MMA) {
        if (tokens < U) {
          // value rows past the unit's end may hold anything; a zero weight times a NaN is a NaN
          for (int idx = lane; idx < (U - tokens) * (D / 8); idx += 32) {
            const int row = tokens + idx / (D / 8);
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(Tensor::row_address(v_stage, row) +
                                                                      (idx % (D / 8)) * 16),
                         "r"(0u)
                         : "memory");
          }
          __syncwarp();
        }
        const float no_scales[1][4] = {{1.0f, 1.0f, 1.0f, 1.0f}};
        if (tokens == U) {
          tensor.template unit<0, true>(k_stage, v_stage, tokens, lane, nullptr, no_scales);
        } else {
          tensor.template unit<0, false>(k_stage, v_stage, tokens, lane, nullptr, no_scales);
        }
      } else {

      // query of this unit: rotation by (a - P), key scale, softmax scale
      if constexpr (!ROT) {
        const bool follows = rot_age < kResync && logical_unit == rot_unit + unit_step;
#pragma unroll
        for (int pi = 0; pi < EPL / 2; ++pi) {
          if (follows) {
            const float c = rot_cos[pi], sn = rot_sin[pi];
            rot_cos[pi] = c * step_cos[pi] - sn * step_sin[pi];
            rot_sin[pi] = sn * step_cos[pi] + c * step_sin[pi];
          } else {
            const int delta = query_position - logical_unit * U;
            sincosf(static_cast<float>(delta) * inv_freq_lane[pi], &rot_sin[pi], &rot_cos[pi]);
          }
        }
        rot_age = follows ? rot_age + 1 : 0;
        rot_unit = logical_unit;
      }
      f32x2 q_rot[GT][EPL / 2];
#pragma unroll
      for (int pi = 0; pi < EPL / 2; ++pi) {
        float factor = p.scale_log2e;
        if constexpr (QUANT) {
          factor *= kscales[i * DB + lane_db];
        }
        const float cs = rot_cos[pi] * factor;
        const float sn = rot_sin[pi] * factor;
#pragma unroll
        for (int h = 0; h < GT; ++h) {
          q_rot[h][pi] = pack2(q_in[h][2 * pi] * cs - q_in[h][2 * pi + 1] * sn,
                               q_in[h][2 * pi] * sn + q_in[h][2 * pi + 1] * cs);
        }
      }
      // Row t of the unit's keys sits at k_stage + t * row bytes, and k_stage is aligned to the 16
      // rows, so "+" is "^" and the per-lane token permutation (t = tl ^ flip) becomes one XOR of
      // a per-lane base with a compile-time constant. The same for the rotation table.
      const uint32_t k_lane = (k_stage + lane * (EPL * EB)) ^ (flip_row * (D * EB));
      const uint32_t rope_lane = (rope_addr + lane * (EPL * 4)) ^ (flip_row * (D * 4));

      // ---- logits: TB tokens x GT heads per butterfly round ----
      float logit[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        logit[r] = -INFINITY;
        if (r * TB < tokens) {
          float vals[NV];
#pragma unroll
          for (int tl = 0; tl < TB; ++tl) {
            float kk[EPL];
            load_elements<KV, EPL>(k_lane ^ static_cast<uint32_t>((r * TB + tl) * (D * EB)), kk);
            if constexpr (!ROT) {
              float cs_sn[EPL];
              const uint32_t table = rope_lane ^ static_cast<uint32_t>((r * TB + tl) * (D * 4));
              if constexpr (EPL == 4) {
                const uint4 c4 = lds128(table);
                cs_sn[0] = __uint_as_float(c4.x), cs_sn[1] = __uint_as_float(c4.y);
                cs_sn[2] = __uint_as_float(c4.z), cs_sn[3] = __uint_as_float(c4.w);
              } else {
                const uint2 c2 = lds64(table);
                cs_sn[0] = __uint_as_float(c2.x), cs_sn[1] = __uint_as_float(c2.y);
              }
#pragma unroll
              for (int pi = 0; pi < EPL / 2; ++pi) {
                const float ke = kk[2 * pi], ko = kk[2 * pi + 1];
                kk[2 * pi] = ke * cs_sn[2 * pi] - ko * cs_sn[2 * pi + 1];
                kk[2 * pi + 1] = ke * cs_sn[2 * pi + 1] + ko * cs_sn[2 * pi];
              }
            }
            f32x2 kk2[EPL / 2];
#pragma unroll
            for (int pi = 0; pi < EPL / 2; ++pi) {
              kk2[pi] = pack2(kk[2 * pi], kk[2 * pi + 1]);
            }
#pragma unroll
            for (int h = 0; h < GT; ++h) {
              f32x2 sum = mul2(q_rot[h][0], kk2[0]);
#pragma unroll
              for (int pi = 1; pi < EPL / 2; ++pi) {
                sum = fma2(q_rot[h][pi], kk2[pi], sum);
              }
              float lo, hi;
              unpack2(sum, lo, hi);
              vals[tl * GT + h] = lo + hi;
            }
          }
          butterfly_sum<NV, GT, FLIP>(vals, lane);
          const int t = r * TB + my_token;
          logit[r] = t < tokens ? vals[0] : -INFINITY;
        }
      }

      // ---- online softmax for head (lane % GT) ----
      float unit_max = logit[0];
#pragma unroll
      for (int r = 1; r < NR; ++r) {
        unit_max = fmaxf(unit_max, logit[r]);
      }
#pragma unroll
      for (int o = GT; o < 32; o <<= 1) {
        unit_max = fmaxf(unit_max, __shfl_xor_sync(0xffffffffu, unit_max, o));
      }
      const float m_new = fmaxf(m_run, unit_max);
      const float m_ref = m_new == -INFINITY ? 0.0f : m_new;
      const float alpha = exp2f(m_run - m_ref);
      float p_sum = 0.0f;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const float prob = exp2f(logit[r] - m_ref);
        p_sum += prob;
        if (holds_value && r * TB < tokens) {
          const int t = r * TB + my_token;
          if constexpr (QUANT) {
            const float* vs = vscales + stage * (L::kVScaleBytes / 4) + t * DB;
#pragma unroll
            for (int b = 0; b < DB; ++b) {
              probs[(t * DBQ + b) * GT + my_head] = make_float2(prob * vs[b], prob * vs[b]);
            }
          } else {
            probs[t * GT + my_head] = make_float2(prob, prob);
          }
        }
      }
      l_run = l_run * alpha + (holds_value ? p_sum : 0.0f);
      m_run = m_new;
      if (lane < GT) {
        alphas[lane] = alpha;
      }
      __syncwarp();

      // ---- weighted values ----
#pragma unroll
      for (int h = 0; h < GT; ++h) {
        const float a = alphas[h];
        const f32x2 a2 = pack2(a, a);
#pragma unroll
        for (int e = 0; e < EPL / 2; ++e) {
          acc[h][e] = mul2(acc[h][e], a2);
        }
      }
      const uint32_t prob_row = smem_addr(probs) + lane_db * (QUANT ? GT * 8 : 0);
#pragma unroll 4
      for (int t = 0; t < tokens; ++t) {
        float vv[EPL];
        load_elements<KV, EPL>(v_stage + t * (D * EB) + lane * (EPL * EB), vv);
        f32x2 vv2[EPL / 2];
#pragma unroll
        for (int e = 0; e < EPL / 2; ++e) {
          vv2[e] = pack2(vv[2 * e], vv[2 * e + 1]);
        }
        f32x2 pr[GT];  // (p, p) of every head, as stored
        if constexpr (GT >= 2) {
#pragma unroll
          for (int h = 0; h < GT; h += 2) {
            const uint4 two = lds128(prob_row + (t * (DBQ * GT) + h) * 8);
            pr[h] = static_cast<f32x2>(two.x) | (static_cast<f32x2>(two.y) << 32);
            pr[h + 1] = static_cast<f32x2>(two.z) | (static_cast<f32x2>(two.w) << 32);
          }
        } else {
          const uint2 one = lds64(prob_row + t * (DBQ * GT) * 8);
          pr[0] = static_cast<f32x2>(one.x) | (static_cast<f32x2>(one.y) << 32);
        }
#pragma unroll
        for (int h = 0; h < GT; ++h) {
#pragma unroll
          for (int e = 0; e < EPL / 2; ++e) {
            acc[h][e] = fma2(pr[h], vv2[e], acc[h][e]);
          }
        }
      }

      }  // !MMA

      // ---- hand the buffer back ----
      __syncwarp();
      const int refill = i + stages * warps;
      if constexpr (PAIRS) {
        if (refill < in_round) {
          proxy_fence_async();  // every lane has read the stage through the generic proxy
          __syncwarp();
          issue(refill, stage);
        }
      } else if (!(MMA && QUANT) && lane == 0 && refill < in_round) {
        proxy_fence_async();
        issue(refill, stage);
      }
    }
    if (failed) {
      // Copies that are still in flight write into this block's shared memory: give each a bounded
      // chance to land before the memory is reused below.
      for (int k = 1; k < stages; ++k) {
        (void)mbar_wait_bounded(my_bars + ((iteration + k) % stages) * 8, ((iteration + k) / stages) & 1);
      }
    }
    if (local_base + CAP >= mine) {
      break;
    }
    __syncthreads();  // the list is rewritten for the next round
  }

  // ---- this warp's result -> shared memory, block result, then the splits ----
  if constexpr (MMA) {
    tensor.finish();
    tensor.l_run += __shfl_xor_sync(0xffffffffu, tensor.l_run, 1);
    tensor.l_run += __shfl_xor_sync(0xffffffffu, tensor.l_run, 2);
  } else {
#pragma unroll
    for (int o = GT; o < 32; o <<= 1) {
      l_run += __shfl_xor_sync(0xffffffffu, l_run, o);
    }
  }
  __syncthreads();  // every warp is done with its ring: the merge area overlays it
  float* merge = reinterpret_cast<float*>(ring_ptr);
  float* merge_m = merge;                     // [warps][GT]
  float* merge_l = merge + warps * GT;        // [warps][GT]
  float* merge_acc = merge + 2 * warps * GT;  // [warps][GT][D]
  float* split_m = merge + round_up(warps * GT * (D + 2), 4);  // [GT][kMaxSplits] maxima, then weights
  float* split_l = split_m + GT * kMaxSplits;     // [GT][kMaxSplits] denominators
  float* block_result = split_l + GT * kMaxSplits;  // [GT][ROW]: this block's result, read by the cluster's rank 0
  if constexpr (MMA) {
    const int head = lane >> 2, c = lane & 3;  // rows past the tile carry zero queries: written, never read
    if (c == 0) {
      merge_m[warp * GT + head] = tensor.m_run;
      merge_l[warp * GT + head] = tensor.l_run;
    }
#pragma unroll
    for (int t = 0; t < D / 8; ++t) {  // head part (c0, c1) + remainder part (c2, c3) of the probabilities
      *reinterpret_cast<float2*>(&merge_acc[(warp * GT + head) * D + t * 8 + 2 * c]) =
          make_float2(tensor.o[t][0] + tensor.o[t][2], tensor.o[t][1] + tensor.o[t][3]);
    }
  } else {
    if (lane < GT) {
      merge_m[warp * GT + lane] = m_run;
      merge_l[warp * GT + lane] = l_run;
    }
#pragma unroll
    for (int h = 0; h < GT; ++h) {
#pragma unroll
      for (int e = 0; e < EPL / 2; ++e) {
        float lo, hi;
        unpack2(acc[h][e], lo, hi);
        *reinterpret_cast<float2*>(&merge_acc[(warp * GT + h) * D + lane * EPL + 2 * e]) = make_float2(lo, hi);
      }
    }
  }
  __syncthreads();

  float* my_partial = p.partials + (static_cast<size_t>(task) * S + split) * (GT * ROW);
  for (int idx = tid; idx < tile_heads * D; idx += threads) {
    const int h = idx / D;
    const int d = idx - h * D;
    float m_all = -INFINITY;
    for (int w = 0; w < warps; ++w) {
      m_all = fmaxf(m_all, merge_m[w * GT + h]);
    }
    const float m_ref = m_all == -INFINITY ? 0.0f : m_all;
    float l_all = 0.0f, a_all = 0.0f;
    for (int w = 0; w < warps; ++w) {
      const float weight = exp2f(merge_m[w * GT + h] - m_ref);
      l_all += weight * merge_l[w * GT + h];
      a_all += weight * merge_acc[(w * GT + h) * D + d];
    }
    if (S == 1) {
      const float y = l_all == 0.0f ? 0.0f : a_all / l_all;
      p.output[out_base + idx] = __bfloat16_as_ushort(__float2bfloat16_rn(y));
    } else {
      float* dst = p.cluster_merge ? block_result : my_partial;
      dst[h * ROW + d] = a_all;
      if (d == 0) {
        dst[h * ROW + D] = m_all;
        dst[h * ROW + D + 1] = l_all;
      }
    }
  }
  if (S == 1) {
    return;
  }
  if (p.cluster_merge) {
    // The S blocks of the task are one cluster (rank = split). Everybody's result sits in its own
    // shared memory; rank 0 reads them in rank order -- same arithmetic as the path through
    // global memory below, no scratch, no ticket -- and nobody leaves before it is done.
    cluster_sync_all();
    if (cluster_rank() == 0) {
      const uint32_t result_addr = smem_addr(block_result);
      for (int idx = tid; idx < tile_heads * S; idx += threads) {
        const int h = idx / S;
        const int s = idx - h * S;
        const float2 ml = ld_cluster_f2(cluster_map(result_addr + (h * ROW + D) * 4, s));
        split_m[h * kMaxSplits + s] = ml.x;
        split_l[h * kMaxSplits + s] = ml.y;
      }
      __syncthreads();
      if (tid < tile_heads) {
        float m_all = -INFINITY;
        for (int s = 0; s < S; ++s) {
          m_all = fmaxf(m_all, split_m[tid * kMaxSplits + s]);
        }
        const float m_ref = m_all == -INFINITY ? 0.0f : m_all;
        float l_all = 0.0f;
        for (int s = 0; s < S; ++s) {
          const float weight = exp2f(split_m[tid * kMaxSplits + s] - m_ref);
          l_all += weight * split_l[tid * kMaxSplits + s];
          split_m[tid * kMaxSplits + s] = weight;
        }
        split_l[tid * kMaxSplits] = l_all == 0.0f ? 0.0f : 1.0f / l_all;
      }
      __syncthreads();
      for (int idx = tid; idx < tile_heads * (D / 4); idx += threads) {
        const int h = idx / (D / 4);
        const int d = (idx - h * (D / 4)) * 4;
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
        for (int s = 0; s < S; ++s) {
          const float4 v = ld_cluster_f4(cluster_map(result_addr + (h * ROW + d) * 4, s));
          const float weight = split_m[h * kMaxSplits + s];
          sum.x = fmaf(weight, v.x, sum.x);
          sum.y = fmaf(weight, v.y, sum.y);
          sum.z = fmaf(weight, v.z, sum.z);
          sum.w = fmaf(weight, v.w, sum.w);
        }
        const float inv = split_l[h * kMaxSplits];
        const __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x * inv, sum.y * inv);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(sum.z * inv, sum.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.output + out_base + static_cast<size_t>(h) * D + d) = packed;
      }
    }
    cluster_sync_all();
    return;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    last_flag = atomicAdd(&p.tickets[task], 1u) == static_cast<unsigned>(S - 1);
  }
  __syncthreads();
  if (!last_flag) {
    return;
  }
  // The last block of the task adds the S partial results in split order. First the maxima and
  // denominators (one load each, all in flight together), then the weights, then the values as
  // 16-byte loads with the splits unrolled so that many are in flight.
  __threadfence();
  const float* task_partials = p.partials + static_cast<size_t>(task) * S * (GT * ROW);
  for (int idx = tid; idx < tile_heads * S; idx += threads) {
    const int h = idx / S;
    const int s = idx - h * S;
    const float* src = task_partials + static_cast<size_t>(s) * (GT * ROW) + h * ROW + D;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(src));
    split_m[h * kMaxSplits + s] = ml.x;
    split_l[h * kMaxSplits + s] = ml.y;
  }
  __syncthreads();
  if (tid < tile_heads) {
    float m_all = -INFINITY;
    for (int s = 0; s < S; ++s) {
      m_all = fmaxf(m_all, split_m[tid * kMaxSplits + s]);
    }
    const float m_ref = m_all == -INFINITY ? 0.0f : m_all;
    float l_all = 0.0f;
    for (int s = 0; s < S; ++s) {
      const float weight = exp2f(split_m[tid * kMaxSplits + s] - m_ref);
      l_all += weight * split_l[tid * kMaxSplits + s];
      split_m[tid * kMaxSplits + s] = weight;
    }
    split_l[tid * kMaxSplits] = l_all == 0.0f ? 0.0f : 1.0f / l_all;
  }
  __syncthreads();
  for (int idx = tid; idx < tile_heads * (D / 4); idx += threads) {
    const int h = idx / (D / 4);
    const int d = (idx - h * (D / 4)) * 4;
    const float* src = task_partials + h * ROW + d;
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
    for (int s = 0; s < S; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(s) * (GT * ROW)));
      const float weight = split_m[h * kMaxSplits + s];
      sum.x = fmaf(weight, v.x, sum.x);
      sum.y = fmaf(weight, v.y, sum.y);
      sum.z = fmaf(weight, v.z, sum.z);
      sum.w = fmaf(weight, v.w, sum.w);
    }
    const float inv = split_l[h * kMaxSplits];
    const __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x * inv, sum.y * inv);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(sum.z * inv, sum.w * inv);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo);
    packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p.output + out_base + static_cast<size_t>(h) * D + d) = packed;
  }
  if (tid == 0) {
    p.tickets[task] = 0;
  }
}

}  // namespace fk_page_decode

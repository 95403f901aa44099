// Shared device-side building blocks for the sm_100a W4A16 kernels.
//
// Weight format (fixed by the reference, csrc/kernels/decode_quant_linear/arc_w4a16.cu:87-122):
// an "ARC packet" covers one tile of 128 output columns and one quantisation group of G input
// features. Its bytes are
//     [G/8 rows][128 columns] uint32   word-major; word (r, c) holds q[c, 8r .. 8r+7],
//                                       nibble i (bits 4i..4i+3) = input feature 8r + i
//     [128] 16-bit scale  (alpha)
//     [128] 16-bit offset (beta = -(alpha * zero_point), rounded once in the 16-bit type)
// and packet (tile t, group g) lives at byte offset (t * K/G + g) * stride, stride = 64*G + 512.
// A packet is therefore one contiguous, 16-byte aligned block, which is what lets the GEMV
// stream it with one bulk asynchronous copy.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace fk_w4a16 {

constexpr int kTileCols = 128;          // output columns per packet
constexpr int kScaleBytes = 2 * kTileCols * 2;  // alpha + beta block at the packet's end

__host__ __device__ constexpr int packet_q_bytes(int group) { return kTileCols * group / 2; }
__host__ __device__ constexpr int packet_stride(int group) {
  return packet_q_bytes(group) + kScaleBytes;
}

// Element-type tags. The 16-bit type is used for activations, scales, offsets and outputs alike.
struct F16 {
  using T = __half;
  static __device__ __forceinline__ float to_float(unsigned short bits) {
    return __half2float(__ushort_as_half(bits));
  }
  static __device__ __forceinline__ unsigned short from_float(float x) {
    return __half_as_ushort(__float2half_rn(x));
  }
};
struct BF16 {
  using T = __nv_bfloat16;
  static __device__ __forceinline__ float to_float(unsigned short bits) {
    return __uint_as_float(static_cast<uint32_t>(bits) << 16);
  }
  static __device__ __forceinline__ unsigned short from_float(float x) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
  }
};

// Device-side status word. Non-zero means a bounded wait gave up; the host reads it through
// fk_w4a16_device_status().
enum DeviceStatus : int {
  kStatusOk = 0,
  kStatusCopyWaitTimeout = 1,
  kStatusPeerWaitTimeout = 2,
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers: shared-memory addresses, mbarriers and 1-D bulk copies (the untiled TMA form).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the asynchronous (TMA) proxy.
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Orders this thread's earlier generic-proxy shared-memory accesses before later
// asynchronous-proxy writes (a bulk copy that refills a buffer the warp has just read).
__device__ __forceinline__ void proxy_fence_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ uint64_t l2_evict_last_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

// Global -> this CTA's shared memory, `bytes` a multiple of 16, both addresses 16-byte aligned.
// Completion is signalled on `bar` as transferred bytes. No cluster multicast is ever used.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait: returns false when the limit is hit instead of spinning forever.
constexpr uint32_t kCopyWaitLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kCopyWaitLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) {
      return true;
    }
  }
  return false;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint2 v) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(v.x), "r"(v.y) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Nibble unpack. One LOP3 per pair: (w & mask) | 0x6400 puts a nibble into the low mantissa bits
// of an fp16 whose exponent makes the mantissa LSB worth 1, i.e. the half value 1024 + q (nibble
// in bits 0-3) or 1024 + 16 q (nibble in bits 4-7). The four results pair nibbles (0,4), (1,5),
// (2,6), (3,7) as (low half, high half).
// ---------------------------------------------------------------------------------------------
template <uint32_t kMask>
__device__ __forceinline__ uint32_t nibble_pair_to_biased_half2(uint32_t w) {
  uint32_t r;
  // LUT 0xEA = (a & b) | c
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "n"(kMask), "n"(0x64006400u));
  return r;
}

struct BiasedNibbles {
  uint32_t p04, p15, p26, p37;  // half2 bit patterns; p15 and p37 carry 16*q
};
__device__ __forceinline__ BiasedNibbles unpack_word(uint32_t w) {
  BiasedNibbles u;
  u.p04 = nibble_pair_to_biased_half2<0x000f000fu>(w);
  u.p15 = nibble_pair_to_biased_half2<0x00f000f0u>(w);
  const uint32_t w8 = w >> 8;
  u.p26 = nibble_pair_to_biased_half2<0x000f000fu>(w8);
  u.p37 = nibble_pair_to_biased_half2<0x00f000f0u>(w8);
  return u;
}
constexpr float kNibbleBias = 1024.0f;  // every unpacked half carries +1024 (times its activation)

// acc_lo += q.lo * a.lo ; acc_hi += q.hi * a.hi with fp16 operands, exact fp32 products and
// fp32 accumulation (the sm_100 mixed-precision FMA: no conversion instructions).
__device__ __forceinline__ void fma2_f32_f16(float& acc_lo, float& acc_hi, uint32_t q2,
                                             uint32_t a2) {
  asm("{\n"
      ".reg .b16 ql, qh, al, ah;\n"
      "mov.b32 {ql, qh}, %2;\n"
      "mov.b32 {al, ah}, %3;\n"
      "fma.rn.f32.f16 %0, ql, al, %0;\n"
      "fma.rn.f32.f16 %1, qh, ah, %1;\n"
      "}\n"
      : "+f"(acc_lo), "+f"(acc_hi)
      : "r"(q2), "r"(a2));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    v += __shfl_xor_sync(0xffffffffu, v, off);
  }
  return v;
}

}  // namespace fk_w4a16

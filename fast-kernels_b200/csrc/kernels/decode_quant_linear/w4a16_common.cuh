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
}

// Programmatic dependent launch (griddepcontrol). Both are no-ops when the kernel was launched
// without the programmatic-serialisation attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_for_prerequisites() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
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
// Completion is signalled on `bar` as transferred bytes. Every copy has exactly one destination CTA.
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

constexpr uint32_t kPeerWaitLimit = 8u << 20;  // polls of >= 200 ns each while waiting for peers

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

// The same test with a suspend-time hint: the hardware may park the thread for up to `hint_ns`
// and wakes it when the phase completes, so a waiting warp does not take issue slots from the
// warps it is waiting for. For kernels whose warps wait on one another (warp-specialised
// pipelines); a warp that waits only for its own copies loses nothing by polling.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}
// Bounded: gives up after kParkedWaitRounds parks of up to kParkedWaitNs each (about a second).
constexpr uint32_t kParkedWaitNs = 20000;
constexpr uint32_t kParkedWaitRounds = 1u << 16;
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity) {
  for (uint32_t round = 0; round < kParkedWaitRounds; ++round) {
    if (mbar_try_wait_parked(bar, parity, kParkedWaitNs)) {
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
// Nibble unpack and multiply-accumulate.
//
// One LOP3, (w & mask) | magic, drops a nibble into the low mantissa bits of a 16-bit float whose
// exponent makes the result an exact small integer plus a constant:
//     fp16  magic 0x6400, nibble in bits 4-7  ->  1024 + 16 q     ("high" placement)
//     fp16  magic 0x6400, nibble in bits 0-3  ->  1024 + q        ("low" placement)
//     bf16  magic 0x4300, nibble in bits 0-3  ->   128 + q        (bf16 has 7 mantissa bits)
// Each 32-bit result is a pair (low half, high half) = nibbles (i, i+4) of the word. The constant
// rides along as constant * activation and is removed once per group in fp32, so its size sets the
// rounding error of the fp32 accumulation: relative to q it is 64 for the high placement (the
// activation is pre-divided by 16), 128 for bf16-low and 1024 for fp16-low. The two unpack modes
// below therefore avoid fp16-low:
//     UnpackF16   all four pairs in high placement            (3 shifts + 4 LOP3 per word)
//     UnpackBF16  pairs (0,4),(2,6) bf16-low, (1,5),(3,7) fp16-high   (1 shift + 4 LOP3 per word)
// Products of two 16-bit floats are exact in fp32 and the sm_100 mixed-precision FMA
// (fma.rn.f32.f16 / .bf16) adds them to an fp32 accumulator without conversion instructions.
// ---------------------------------------------------------------------------------------------
template <uint32_t kMask, uint32_t kMagic>
__device__ __forceinline__ uint32_t mask_or(uint32_t w) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "n"(kMask), "n"(kMagic));  // (a&b)|c
  return r;
}

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
__device__ __forceinline__ void fma2_f32_bf16(float& acc_lo, float& acc_hi, uint32_t q2,
                                              uint32_t a2) {
  asm("{\n"
      ".reg .b16 ql, qh, al, ah;\n"
      "mov.b32 {ql, qh}, %2;\n"
      "mov.b32 {al, ah}, %3;\n"
      "fma.rn.f32.bf16 %0, ql, al, %0;\n"
      "fma.rn.f32.bf16 %1, qh, ah, %1;\n"
      "}\n"
      : "+f"(acc_lo), "+f"(acc_hi)
      : "r"(q2), "r"(a2));
}

struct NibblePairs {
  uint32_t p04, p15, p26, p37;
};

// What the staging step must put in shared memory for one word-row of one batch row: four 32-bit
// pairs (a0,a4) (a1,a5) (a2,a6) (a3,a7) in the formats the mode multiplies with, and the constant
// term B such that sum_i pair_i * staged_i = sum_k q_k a_k + B.
struct UnpackF16 {
  using Elem = F16;
  // Tensor-core variant: both k-steps of a word multiply fp16 pairs. A constant-valued weight
  // row (all kConstB / all kConstS) makes the MMA itself deliver B and S for every batch row.
  static constexpr bool kEvenNibblesBf16 = false;
  static constexpr uint32_t kEvenConstB = 0x64006400u;  // 1024 : sum 1024 * a' = B
  static constexpr uint32_t kEvenConstS = 0x4C004C00u;  // 16   : sum 16 * (a / 16) = S
  static constexpr uint32_t kOddConstB = 0x64006400u;
  static constexpr uint32_t kOddConstS = 0x4C004C00u;
  static __device__ __forceinline__ NibblePairs unpack(uint32_t w) {
    NibblePairs u;
    u.p04 = mask_or<0x00f000f0u, 0x64006400u>(w << 4);
    u.p15 = mask_or<0x00f000f0u, 0x64006400u>(w);
    u.p26 = mask_or<0x00f000f0u, 0x64006400u>(w >> 4);
    u.p37 = mask_or<0x00f000f0u, 0x64006400u>(w >> 8);
    return u;
  }
  static __device__ __forceinline__ void mac(float& lo, float& hi, const NibblePairs& u,
                                             const uint4& a) {
    fma2_f32_f16(lo, hi, u.p04, a.x);
    fma2_f32_f16(lo, hi, u.p15, a.y);
    fma2_f32_f16(lo, hi, u.p26, a.z);
    fma2_f32_f16(lo, hi, u.p37, a.w);
  }
  // Staged value and bias contribution of activation `f` sitting at an even / odd nibble.
  static __device__ __forceinline__ unsigned short stage(float f, bool /*odd*/, float& bias) {
    const __half h = __float2half_rn(f * 0.0625f);
    bias += 1024.0f * __half2float(h);
    return __half_as_ushort(h);
  }
};

struct UnpackBF16 {
  using Elem = BF16;
  static constexpr bool kEvenNibblesBf16 = true;
  static constexpr uint32_t kEvenConstB = 0x43004300u;  // bf16 128 : sum 128 * a
  static constexpr uint32_t kEvenConstS = 0x3F803F80u;  // bf16 1   : sum a
  static constexpr uint32_t kOddConstB = 0x64006400u;   // fp16 1024
  static constexpr uint32_t kOddConstS = 0x4C004C00u;   // fp16 16
  static __device__ __forceinline__ NibblePairs unpack(uint32_t w) {
    NibblePairs u;
    const uint32_t w8 = w >> 8;
    u.p04 = mask_or<0x000f000fu, 0x43004300u>(w);
    u.p15 = mask_or<0x00f000f0u, 0x64006400u>(w);
    u.p26 = mask_or<0x000f000fu, 0x43004300u>(w8);
    u.p37 = mask_or<0x00f000f0u, 0x64006400u>(w8);
    return u;
  }
  static __device__ __forceinline__ void mac(float& lo, float& hi, const NibblePairs& u,
                                             const uint4& a) {
    fma2_f32_bf16(lo, hi, u.p04, a.x);
    fma2_f32_f16(lo, hi, u.p15, a.y);
    fma2_f32_bf16(lo, hi, u.p26, a.z);
    fma2_f32_f16(lo, hi, u.p37, a.w);
  }
  static __device__ __forceinline__ unsigned short stage(float f, bool odd, float& bias) {
    if (odd) {
      const __half h = __float2half_rn(f * 0.0625f);
      bias += 1024.0f * __half2float(h);
      return __half_as_ushort(h);
    }
    bias += 128.0f * f;  // f is a bf16 value: kept as is, exactly
    return static_cast<unsigned short>(__float_as_uint(f) >> 16);
  }
};

// D += A * B for one m16n8k16 tile, fp32 accumulate; A row-major 16x16, B 16x8 (k-major pairs).
__device__ __forceinline__ void mma_16816_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_16816_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    v += __shfl_xor_sync(0xffffffffu, v, off);
  }
  return v;
}

}  // namespace fk_w4a16

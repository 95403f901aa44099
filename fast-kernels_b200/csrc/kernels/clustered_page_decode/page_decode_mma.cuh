// Tensor-core form of the per-unit arithmetic of the paged-KV decode attention, for pages whose keys
// were rotated ahead of time (what serving engines store): logits and weighted values of a 16-token
// unit as mma.sync.m16n8k16 (16-bit operands, fp32 accumulate) instead of fp32 FMAs per lane.
//
// Nothing is rounded that the fp32 path does not round. bf16 pages: the tensor cores take bf16,
// keys and values ARE bf16, and the two fp32 operands -- the rotated, scaled query and the
// probabilities -- are split into a bf16 head and a bf16 remainder (x = hi + lo to 2^-17). The
// split costs no extra instruction: a tile has at most 8 heads and the MMA has 16 rows, so row g
// carries the head part and row g + 8 the remainder of head g, and both land in the SAME lane's
// accumulator registers (c0, c1 = row g; c2, c3 = row g + 8), which are added.
//
// 8-bit pages (HALF = true): e4m3 and int8 elements are f16 values exactly and become f16 cheaply
// (one cvt per two e4m3 bytes; a byte permute into 0x64xx = 1024 + x and one packed subtraction
// per two int8 bytes), so the unit is converted to f16 rows in shared memory and the MMAs take
// f16. f16 has the mantissa (head + remainder = 22 bits) but not the range, so the fp32 operands
// are brought to [-2, 2) by exact powers of two first: the query row by the exponent of its largest
// element (undone on the logits together with the key scale), and the probabilities -- which carry
// the per-token value scales -- by a RUNNING exponent of the largest value scale seen so far, kept
// like the running maximum of the softmax: when it grows, the accumulated values are rescaled by
// the power of two in the same multiplication that applies the softmax correction.
//
// Fragment geometry (lane l: g = l / 4, c = l % 4):
//   logits   A = query [16 rows x 16 dims], B = keys  [16 dims x 8 tokens]   -> C [rows x 8 tokens]
//   values   A = probs [16 rows x 16 tokens], B = values [16 tokens x 8 dims] -> C [rows x 8 dims]
//   C of the logits (two 8-token tiles) is, register for register, A of the values: lane l holds
//   tokens {2c, 2c+1} of tile 0 and of tile 1, which are k-slots {2c, 2c+1, 2c+8, 2c+9}.
// Keys and values of a unit sit in shared memory as 8 PAIRS of token rows (tokens 2j and 2j + 1 back
// to back, as in the page: one 2-row bulk copy each), pairs 16 bytes apart from a multiple of 128.
// The 8-token tiles are the EVEN and the ODD tokens -- which token an MMA column stands for is
// free, the values' k-slots follow the same order -- so the 8 rows of every ldmatrix phase come from
// the 8 different pairs and hit 8 different bank groups. (Rows copied one by one with a skew each
// are conflict-free too but take 32 copies per unit, which bounds the kernel at ~4.4 TB/s; two
// 4 KB copies without skew leave 8-way conflicts, 2.8 TB/s.)
//
// Keys stored UNROTATED stay on the fp32 path: rotating them here in fp32 and splitting the result
// into two bf16 operands (a second set of key MMAs) was built and measured at 225 us against 132
// on 32 requests x 8 kv heads x 4096 tokens -- the rotation and split of every key element costs
// more than the FMAs it replaces, and the extra rows leave room for 7 warps only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace fk_page_decode {

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <bool HALF>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (HALF) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// x = hi + lo with hi = the 16-bit rounding of x, lo = that of x - hi; returns the packed pairs
// (first, second). HALF: f16 (the caller keeps |x| < 2), else bf16.
template <bool HALF>
__device__ __forceinline__ void split_pair(float first, float second, uint32_t& hi, uint32_t& lo) {
  if constexpr (HALF) {
    const __half2 h = __floats2half2_rn(first, second);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const float2 back = __half22float2(h);
    const __half2 l = __floats2half2_rn(first - back.x, second - back.y);
    lo = *reinterpret_cast<const uint32_t*>(&l);
  } else {
    const __nv_bfloat162 h = __floats2bfloat162_rn(first, second);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const __nv_bfloat162 l =
        __floats2bfloat162_rn(first - __uint_as_float(hi << 16), second - __uint_as_float(hi & 0xffff0000u));
    lo = *reinterpret_cast<const uint32_t*>(&l);
  }
}

// 2^x for x <= 0 in one instruction (2 ulp; results below the normal range become 0).
__device__ __forceinline__ float exp2_quick(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Exponent fields (bits of a float, mantissa cleared) the power-of-two scalings stay within, so
// that 2^e and 2^-e are both normal numbers.
constexpr int kMinExponentBits = 7 << 23;    // 2^-120
constexpr int kMaxExponentBits = 237 << 23;  // 2^110 (times the fixed 2^8 of shifted e4m3 operands: still finite)
__device__ __forceinline__ int exponent_bits(float magnitude) {
  return min(max(__float_as_int(magnitude) & 0x7f800000, kMinExponentBits), kMaxExponentBits);
}
__device__ __forceinline__ float inverse_power(int bits) { return __int_as_float(0x7f000000 - bits); }  // 2^-e

template <int D, bool HALF>
struct MmaWarp {
  static constexpr int kRowBytes = 2 * D;                 // one token
  static constexpr int kPairBytes = 2 * kRowBytes + 16;   // tokens 2j, 2j + 1 and the skew
  static constexpr int kUnitSmem = 8 * kPairBytes;        // 16 tokens of keys (or values)
  static constexpr int kSteps = D / 16;         // k-steps of the logits
  static constexpr int kTiles = D / 8;          // 8-dim tiles of the values

  uint32_t q[kSteps][4];  // A fragments of the query: rows g = head part, rows g + 8 = remainder
  float o[kTiles][4];     // weighted values, C fragments (c0, c1: head part; c2, c3: remainder part)
  float m_run;            // running maximum of head g (the same on its four lanes)
  float l_run;            // this lane's share of head g's denominator
  float q_power;          // HALF: the power of two the query row of head g was divided by
  int o_exponent;         // HALF: exponent bits of the power of two `o` is divided by (running)
  float o_power;          // HALF: a fixed power of two `o` is divided by on top of that

  // `query_row` -> bf16 query of head g (nullptr for a row past the tile); rotated by
  // position * theta, scaled by `scale`. `scratch`: D floats of this warp's shared memory, used to
  // hand the D/2 (cos, sin) pairs -- two sincosf per lane -- to the lanes that need them.
  // HALF: the key rows hold the keys divided by `key_power`, the value rows the values divided by
  // `value_power` (powers of two).
  __device__ __forceinline__ void prepare(const uint16_t* query_row, int lane, int position, const float* inv_freq,
                                          float scale, float* scratch, float key_power = 1.0f,
                                          float value_power = 1.0f) {
    o_power = value_power;
    const int c = lane & 3;
#pragma unroll
    for (int t = 0; t < kTiles; ++t) {
      o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f;
    }
    m_run = -INFINITY;
    l_run = 0.0f;
    for (int pair = lane; pair < D / 2; pair += 32) {
      float sn, cs;
      sincosf(static_cast<float>(position) * inv_freq[pair], &sn, &cs);
      *reinterpret_cast<float2*>(scratch + 2 * pair) = make_float2(cs * scale, sn * scale);
    }
    __syncwarp();
    float rotated[kSteps][2][2];
    float largest = 0.0f;
#pragma unroll
    for (int kk = 0; kk < kSteps; ++kk) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int dim = kk * 16 + half * 8 + 2 * c;  // an even dimension: (dim, dim + 1) is one rotary pair
        float even = 0.0f, odd = 0.0f;
        if (query_row != nullptr) {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(query_row + dim);
          const float qe = __uint_as_float(w << 16), qo = __uint_as_float(w & 0xffff0000u);
          const float2 cs_sn = *reinterpret_cast<const float2*>(scratch + dim);
          even = qe * cs_sn.x - qo * cs_sn.y;
          odd = qe * cs_sn.y + qo * cs_sn.x;
        }
        rotated[kk][half][0] = even;
        rotated[kk][half][1] = odd;
        largest = fmaxf(largest, fmaxf(fabsf(even), fabsf(odd)));
      }
    }
    float shrink = 1.0f;
    q_power = 1.0f;
    o_exponent = kMinExponentBits;
    if constexpr (HALF) {
      largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, 1));  // the four lanes of head g
      largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, 2));
      const int bits = exponent_bits(largest);
      q_power = __int_as_float(bits) * key_power;
      shrink = inverse_power(bits);
    }
#pragma unroll
    for (int kk = 0; kk < kSteps; ++kk) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        split_pair<HALF>(rotated[kk][half][0] * shrink, rotated[kk][half][1] * shrink, q[kk][2 * half],
                         q[kk][2 * half + 1]);
      }
    }
    __syncwarp();
  }

  // Shared-memory address of token `row` of a unit that starts at `base`.
  static __device__ __forceinline__ uint32_t row_address(uint32_t base, int row) {
    return base + (row >> 1) * kPairBytes + (row & 1) * kRowBytes;
  }

  // One unit: `k_rows` / `v_rows` shared-memory addresses of the 8 row pairs, `tokens` <= 16 of the
  // rows real. Rows past `tokens` of the VALUES must hold finite numbers (the caller zeroes them):
  // a zero probability times a NaN would still poison the sum.
  // BLOCKS > 1 (8-bit pages, unscaled elements in the rows): the logits of every 64-dim block are
  // accumulated apart and multiplied by `key_scale[block]` (fp32), and the probabilities that meet
  // the values of block b carry the value scales `scales` (lane_value_scales). BLOCKS = 0: no scales.
  // This lane's value scales of a unit, in the order unit() takes them: [block][j], j = the lane's
  // four tokens {2c, 2c + 1} of the even tile and of the odd tile; 0 for a token past the end.
  template <int NB, bool FULL>
  static __device__ __forceinline__ void lane_value_scales(const float* value_scales, int tokens, int lane,
                                                           float (&scales)[NB][4]) {
    // the lane's tokens are 4c .. 4c + 3 (j = 0, 2, 1, 3): NB * 4 neighbouring floats, 16-byte aligned
    const int c = lane & 3;
    float raw[4][NB];  // [token - 4c][block]
    const float4* src = reinterpret_cast<const float4*>(value_scales + 4 * c * NB);
#pragma unroll
    for (int v = 0; v < NB; ++v) {
      const float4 x = src[v];
      const float four[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        raw[(v * 4 + e) / NB][(v * 4 + e) % NB] = four[e];
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int offset = 2 * (j & 1) + (j >> 1);  // token - 4c
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        // (a token past the end has probability 0; its scale may be anything, finite or not)
        scales[b][j] = (FULL || 4 * c + offset < tokens) ? raw[offset][b] : 0.0f;
      }
    }
  }

  // FULL: the caller knows that all 16 tokens are real (no masks).
  template <int BLOCKS, bool FULL>
  __device__ __forceinline__ void unit(uint32_t k_rows, uint32_t v_rows, int tokens, int lane, const float* key_scale,
                                       const float (&scales)[BLOCKS > 0 ? BLOCKS : 1][4]) {
    constexpr int NB = BLOCKS > 0 ? BLOCKS : 1;
    const int c = lane & 3;
    // ---- logits: 16 (head | remainder) rows x 16 tokens; tile 0 = even tokens, tile 1 = odd ----
    float s[NB][2][4];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        s[b][nt][0] = s[b][nt][1] = s[b][nt][2] = s[b][nt][3] = 0.0f;
      }
    }
    // lane i addresses row (i % 8) of matrix (i / 8), i.e. token 2 (i % 8) + tile: matrices 0, 1 =
    // dims +0, +8 of step kk; 2, 3 = of step kk + 1
    const uint32_t k_lane = k_rows + (lane & 7) * kPairBytes + (lane >> 3) * 16;
#pragma unroll
    for (int kk = 0; kk < kSteps; kk += 2) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        uint32_t b[4];
        ldmatrix_x4(k_lane + nt * kRowBytes + kk * 32, b);
        mma_16816<HALF>(s[kk / (kSteps / NB)][nt], q[kk], b[0], b[1]);
        mma_16816<HALF>(s[kk / (kSteps / NB)][nt], q[kk + 1], b[2], b[3]);
      }
    }
    // head part + remainder part (times the block's key scale); tokens past the unit's end do not count
    float logit[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int token = 2 * (2 * c + j) + nt;  // column 2c + j of the even (nt = 0) or odd (nt = 1) tile
        float value = 0.0f;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const float part = s[b][nt][j] + s[b][nt][j + 2];
          value = BLOCKS > 0 ? fmaf(part, key_scale[b], value) : part;
        }
        if constexpr (HALF) {
          value *= q_power;
        }
        logit[nt * 2 + j] = (FULL || token < tokens) ? value : -INFINITY;
      }
    }
    float unit_max = fmaxf(fmaxf(logit[0], logit[1]), fmaxf(logit[2], logit[3]));
    unit_max = fmaxf(unit_max, __shfl_xor_sync(0xffffffffu, unit_max, 1));
    unit_max = fmaxf(unit_max, __shfl_xor_sync(0xffffffffu, unit_max, 2));
    const float m_new = fmaxf(m_run, unit_max);
    const float m_ref = m_new == -INFINITY ? 0.0f : m_new;
    const float alpha = exp2_quick(m_run - m_ref);
    float prob[4];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      prob[j] = exp2_quick(logit[j] - m_ref);
      sum += prob[j];
    }
    l_run = l_run * alpha + sum;
    m_run = m_new;
    // ---- probabilities as the A operand: k-slots 2c, 2c+1 (even tile) and 2c+8, 2c+9 (odd tile) ----
    uint32_t pa[NB][4];
    float largest = 0.0f;
    if constexpr (HALF) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          largest = fmaxf(largest, fabsf(scales[b][j]));
        }
      }
    }
    float shrink = 1.0f;   // what the weights are multiplied by before they are split
    float carry = alpha;   // what the accumulated values are multiplied by
    if constexpr (HALF) {
      largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, 1));  // all 16 tokens
      largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, 2));
      const int exponent = max(o_exponent, exponent_bits(largest));
      // 2^(old - new): exactly 0 once the old sum is more than 2^126 below the new scale
      carry = alpha * __int_as_float(max(0x3f800000 + (o_exponent - exponent), 0));
      o_exponent = exponent;
      shrink = inverse_power(exponent);
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float weight[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        weight[j] = BLOCKS > 0 ? prob[j] * (HALF ? scales[b][j] * shrink : scales[b][j]) : prob[j];
      }
      split_pair<HALF>(weight[0], weight[1], pa[b][0], pa[b][1]);
      split_pair<HALF>(weight[2], weight[3], pa[b][2], pa[b][3]);
    }
    // ---- weighted values: 16 rows x head_dim ----
    // k-slots 0-7 are the even tokens, 8-15 the odd ones (the order of the logits' tiles). Lane i
    // addresses token 2 (i % 8) + ((i / 8) % 2) of dim tile (i / 16): matrices 0, 1 = even, odd
    // tokens of tile t; 2, 3 = of tile t + 1
    const uint32_t v_lane = v_rows + (lane & 7) * kPairBytes + ((lane >> 3) & 1) * kRowBytes + (lane >> 4) * 16;
    // once the running maximum (and exponent) has settled, most units leave the sum as it is
    if (__any_sync(0xffffffffu, carry != 1.0f)) {
#pragma unroll
      for (int t = 0; t < kTiles; ++t) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[t][j] *= carry;
        }
      }
    }
#pragma unroll
    for (int t = 0; t < kTiles; t += 2) {
      uint32_t b[4];
      ldmatrix_x4_trans(v_lane + t * 16, b);
      mma_16816<HALF>(o[t], pa[t / (kTiles / NB)], b[0], b[1]);
      mma_16816<HALF>(o[t + 1], pa[t / (kTiles / NB)], b[2], b[3]);
    }
  }

  // After the last unit: `o` back in plain units.
  __device__ __forceinline__ void finish() {
    if constexpr (HALF) {
      const float power = __int_as_float(o_exponent) * o_power;
#pragma unroll
      for (int t = 0; t < kTiles; ++t) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[t][j] *= power;
        }
      }
    }
  }
};

}  // namespace fk_page_decode

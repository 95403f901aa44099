// Tensor-core form of the per-unit arithmetic of the paged-KV decode attention, for pages that hold
// bf16 keys rotated ahead of time (what serving engines store): logits and weighted values of a
// 16-token unit as mma.sync.m16n8k16 (bf16 in, fp32 accumulate) instead of fp32 FMAs per lane.
//
// Nothing is rounded that the fp32 path does not round: the tensor cores take bf16, keys and values
// ARE bf16, and the two fp32 operands -- the rotated, scaled query and the probabilities -- are
// split into a bf16 head and a bf16 remainder (x = hi + lo to 2^-17). The split costs no extra
// instruction: a tile has at most 8 heads and the MMA has 16 rows, so row g carries the head part
// and row g + 8 the remainder of head g, and both land in the SAME lane's accumulator registers
// (c0, c1 = row g; c2, c3 = row g + 8), which are added.
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
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// x = hi + lo with hi = bf16(x), lo = bf16(x - hi); returns the packed pairs (first, second).
__device__ __forceinline__ void split_pair(float first, float second, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(first, second);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  const __nv_bfloat162 l = __floats2bfloat162_rn(first - __uint_as_float(hi << 16), second - __uint_as_float(hi & 0xffff0000u));
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

template <int D>
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

  // `query_row` -> bf16 query of head g (nullptr for a row past the tile); rotated by
  // position * theta, scaled by `scale`. `scratch`: D floats of this warp's shared memory, used to
  // hand the D/2 (cos, sin) pairs -- two sincosf per lane -- to the lanes that need them.
  __device__ __forceinline__ void prepare(const uint16_t* query_row, int lane, int position, const float* inv_freq,
                                          float scale, float* scratch) {
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
        split_pair(even, odd, q[kk][2 * half], q[kk][2 * half + 1]);
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
  __device__ __forceinline__ void unit(uint32_t k_rows, uint32_t v_rows, int tokens, int lane) {
    const int c = lane & 3;
    // ---- logits: 16 (head | remainder) rows x 16 tokens; tile 0 = even tokens, tile 1 = odd ----
    float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
    // lane i addresses row (i % 8) of matrix (i / 8), i.e. token 2 (i % 8) + tile: matrices 0, 1 =
    // dims +0, +8 of step kk; 2, 3 = of step kk + 1
    const uint32_t k_lane = k_rows + (lane & 7) * kPairBytes + (lane >> 3) * 16;
#pragma unroll
    for (int kk = 0; kk < kSteps; kk += 2) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        uint32_t b[4];
        ldmatrix_x4(k_lane + nt * kRowBytes + kk * 32, b);
        mma_bf16_16816(s[nt], q[kk], b[0], b[1]);
        mma_bf16_16816(s[nt], q[kk + 1], b[2], b[3]);
      }
    }
    // head part + remainder part; tokens past the unit's end do not count
    float logit[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int token = 2 * (2 * c + j) + nt;  // column 2c + j of the even (nt = 0) or odd (nt = 1) tile
        logit[nt * 2 + j] = token < tokens ? s[nt][j] + s[nt][j + 2] : -INFINITY;
      }
    }
    float unit_max = fmaxf(fmaxf(logit[0], logit[1]), fmaxf(logit[2], logit[3]));
    unit_max = fmaxf(unit_max, __shfl_xor_sync(0xffffffffu, unit_max, 1));
    unit_max = fmaxf(unit_max, __shfl_xor_sync(0xffffffffu, unit_max, 2));
    const float m_new = fmaxf(m_run, unit_max);
    const float m_ref = m_new == -INFINITY ? 0.0f : m_new;
    const float alpha = exp2f(m_run - m_ref);
    float prob[4];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      prob[j] = exp2f(logit[j] - m_ref);
      sum += prob[j];
    }
    l_run = l_run * alpha + sum;
    m_run = m_new;
    // ---- probabilities as the A operand: k-slots 2c, 2c+1 (even tile) and 2c+8, 2c+9 (odd tile) ----
    uint32_t pa[4];
    split_pair(prob[0], prob[1], pa[0], pa[1]);
    split_pair(prob[2], prob[3], pa[2], pa[3]);
    // ---- weighted values: 16 rows x head_dim ----
    // k-slots 0-7 are the even tokens, 8-15 the odd ones (the order of the logits' tiles). Lane i
    // addresses token 2 (i % 8) + ((i / 8) % 2) of dim tile (i / 16): matrices 0, 1 = even, odd
    // tokens of tile t; 2, 3 = of tile t + 1
    const uint32_t v_lane = v_rows + (lane & 7) * kPairBytes + ((lane >> 3) & 1) * kRowBytes + (lane >> 4) * 16;
#pragma unroll
    for (int t = 0; t < kTiles; t += 2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[t][j] *= alpha;
        o[t + 1][j] *= alpha;
      }
      uint32_t b[4];
      ldmatrix_x4_trans(v_lane + t * 16, b);
      mma_bf16_16816(o[t], pa, b[0], b[1]);
      mma_bf16_16816(o[t + 1], pa, b[2], b[3]);
    }
  }
};

}  // namespace fk_page_decode

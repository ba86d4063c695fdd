// Per-token routing (softmax / top-k / renormalisation) as a warp-level device function, shared by the
// router kernels of router.cu.
#pragma once
#include "common.cuh"

namespace b200 {

// Selection key: order-preserving 16-bit image of a bf16 value (high half of the 32-bit key) and the
// inverted expert index (low half), so that a warp-wide max picks (value desc, expert asc).
__device__ __forceinline__ uint32_t order_key(uint32_t bf16_bits) {
  if (bf16_bits == 0x8000u) bf16_bits = 0u;  // -0 and +0 compare equal
  return (bf16_bits & 0x8000u) ? (~bf16_bits & 0xffffu) : (bf16_bits | 0x8000u);
}
__device__ __forceinline__ uint32_t key_to_bits(uint32_t key16) {
  return (key16 & 0x8000u) ? (key16 & 0x7fffu) : (~key16 & 0xffffu);
}

constexpr int kMaxPerLane = 8;   // experts per lane -> E <= 256
constexpr int kMaxTopK = 32;

// One warp routes token t.  L2: read the logits with ld.global.cg (they were written by other
// CTAs of the same launch).
template <bool L2>
__device__ __forceinline__ void route_topk_token(const __nv_bfloat16* logits, int t, int lane, int E, int k, int mode,
                                                 int renorm, uint32_t* __restrict__ idx,
                                                 __nv_bfloat16* __restrict__ scores,
                                                 __nv_bfloat16* __restrict__ probs /*nullable [T,E]*/) {
  const unsigned short* row = reinterpret_cast<const unsigned short*>(logits) + (size_t)t * E;

  uint32_t bits[kMaxPerLane];
  float lf[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    int e = lane + 32 * i;
    bits[i] = (e < E) ? (L2 ? __ldcg(row + e) : row[e]) : 0xff80u;  // -inf padding
    lf[i] = bf16_bits_to_f32(bits[i]);
  }

  if (mode == 0) {
    float m = lf[0];
#pragma unroll
    for (int i = 1; i < kMaxPerLane; ++i) m = fmaxf(m, lf[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    double ex[kMaxPerLane];
    double s = 0.0;
    const int nper = (E + 31) >> 5;  // experts per lane that exist (warp-uniform bound of the loops below)
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      ex[i] = 0.0;
      if (i < nper) {
        const int e = lane + 32 * i;
        if (e < E) ex[i] = exp((double)lf[i] - (double)m);
        s += ex[i];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      bits[i] = 0xff80u;
      if (i < nper && e < E) {
        bits[i] = f64_to_bf16_bits(ex[i] / s);
        if (probs) probs[(size_t)t * E + e] = __ushort_as_bfloat16((unsigned short)bits[i]);
      }
    }
  }

  uint32_t keys[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    int e = lane + 32 * i;
    keys[i] = (e < E) ? ((order_key(bits[i]) << 16) | (0xffffu - (uint32_t)e)) : 0u;
  }

  uint32_t my_sel = 0;  // lane j keeps the j-th winner
  for (int j = 0; j < k; ++j) {
    uint32_t best = keys[0];
#pragma unroll
    for (int i = 1; i < kMaxPerLane; ++i) best = max(best, keys[i]);
    best = __reduce_max_sync(0xffffffffu, best);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (keys[i] == best) keys[i] = 0u;
    if (lane == j) my_sel = best;
  }

  const bool active = lane < k;
  const uint32_t e_sel = 0xffffu - (my_sel & 0xffffu);
  const uint32_t v_bits = key_to_bits(my_sel >> 16);
  const float v = active ? bf16_bits_to_f32(v_bits) : 0.f;
  uint32_t out_bits = v_bits;
  if (mode == 0) {
    if (renorm) {
      double s = active ? (double)v : 0.0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      out_bits = f64_to_bf16_bits((double)v / s);
    }
  } else {
    float m = __shfl_sync(0xffffffffu, v, 0);  // winner 0 holds the largest logit
    double ex = active ? exp((double)v - (double)m) : 0.0;
    double s = ex;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    out_bits = f64_to_bf16_bits(ex / s);
  }
  if (active) {
    idx[(size_t)t * k + lane] = e_sel;
    scores[(size_t)t * k + lane] = __ushort_as_bfloat16((unsigned short)out_bits);
  }
}


}  // namespace b200

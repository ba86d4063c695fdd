// Building blocks of the memory-bound grouped quantized product (few rows per expert), shared by
// the kernels of qmm_decode.cu.
//
// Contract: gather_qmm(x, w, scales, biases, rhs_indices, transpose=true) of the reference
// (mlx-rs/src/ops/quantization.rs:160-230) on rows grouped by expert, i.e. for every row
//   out[n] = sum_g ( scale[n,g] * sum_{k in g} q[n,k] x[k]  +  bias[n,g] * sum_{k in g} x[k] )
// which is the affine dequantisation w_hat = scale*q + bias applied exactly, in float32.
//
// How a warp computes it.  Packed codes are loaded straight from HBM into registers (64-bit loads
// for 4-bit codes, 128-bit for 8-bit) and become fp16 operands of mma.sync m16n8k16 with ONE logic
// instruction per pair of codes: OR-ing a 4-bit code into the mantissa of fp16 1024.0 gives 1024+q
// when the nibble sits at bits 0..3 and 1024+16q when it sits at bits 4..7 (taken in place, no
// shift); an 8-bit code placed under the byte 0x64 gives 1024+q.  The other operand, the activation
// row, is prepared once per row (prepare_rows_small_kernel): fp16, the row scaled by a power of
// two, every aligned group of eight elements stored in the order [0,4,1,5,2,6,3,7] in which the
// nibble pairs come out of a word, and the elements that meet an in-place nibble (1,3,5,7)
// divided by 16.  One quantisation group (64 k) is four MMAs whose accumulator starts at
//   -C = -(1024 * sum of the stored activations of the group)
// so that it ends at sum_k q_k x_k, and the group is folded as
//   total += scale * acc + bias * S,   S = sum of the group's true activations.
// Per 16 x 64 weight tile a lane issues 2 weight loads, 20 logic/shift, 4 MMA and 8 FMA instructions.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace qs {

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3) {
  // (not volatile: the groups of a block are independent chains of four dependent MMAs, and the compiler may interleave
  // them only if it is free to reorder these statements)
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

constexpr uint32_t kMagic = 0x64006400u;  // fp16 (1024.0, 1024.0)

// (a & mask) | magic as ONE logic instruction (the compiler otherwise emits an AND and an OR when both
// constants are immediates)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t magic) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(magic));
  return d;
}

template <int BITS>
struct WVec;
template <>
struct WVec<4> {
  using T = uint2;  // 16 codes of one row
  static __device__ __forceinline__ T load(const uint32_t* p) { return ldg_nc_v2(p); }
  static __device__ __forceinline__ T zero() { return make_uint2(0, 0); }
};
template <>
struct WVec<8> {
  using T = uint4;  // 16 codes of one row
  static __device__ __forceinline__ T load(const uint32_t* p) { return ldg_nc_v4(p); }
  static __device__ __forceinline__ T zero() { return make_uint4(0, 0, 0, 0); }
};

// A-operand registers of MMA i (0..3) of a group for the two weight rows (g, g+8) a lane holds.
template <int BITS>
__device__ __forceinline__ void a_frag(const typename WVec<BITS>::T& ra, const typename WVec<BITS>::T& rb, int i,
                                       uint32_t (&a)[4]) {
  if constexpr (BITS == 4) {
    // word -> pairs (q0,q4) (16q1,16q5) | after >> 8: (q2,q6) (16q3,16q7)
    const uint32_t wa = ((i < 2) ? ra.x : ra.y) >> ((i & 1) * 8);
    const uint32_t wb = ((i < 2) ? rb.x : rb.y) >> ((i & 1) * 8);
    a[0] = and_or(wa, 0x000f000fu, kMagic);
    a[1] = and_or(wb, 0x000f000fu, kMagic);
    a[2] = and_or(wa, 0x00f000f0u, kMagic);
    a[3] = and_or(wb, 0x00f000f0u, kMagic);
  } else {
    const uint32_t wa = (i == 0) ? ra.x : (i == 1) ? ra.y : (i == 2) ? ra.z : ra.w;
    const uint32_t wb = (i == 0) ? rb.x : (i == 1) ? rb.y : (i == 2) ? rb.z : rb.w;
    a[0] = __byte_perm(wa, 0x64646464u, 0x4140);  // (1024+q0, 1024+q1)
    a[1] = __byte_perm(wb, 0x64646464u, 0x4140);
    a[2] = __byte_perm(wa, 0x64646464u, 0x4342);  // (1024+q2, 1024+q3)
    a[3] = __byte_perm(wb, 0x64646464u, 0x4342);
  }
}

// bf16 number u (0..3) of a packed uint2 as float32
__device__ __forceinline__ float bf16_of(const uint2& v, int u) {
  const uint32_t w = (u & 2) ? v.y : v.x;
  return __uint_as_float((u & 1) ? (w & 0xffff0000u) : (w << 16));
}

// Shared-memory image of `rows` prepared activation rows of length K (G = K / 64 groups):
//   xs  [rows][XS bytes], XS = 2K + 16 (the pad keeps the rows of a quad pair on distinct banks)
//   c4  [G][ceil(rows/2)] float4 (-C(2p), -C(2p+1), -C(2p), -C(2p+1)) per group and row pair: the C operand
//       of a group's first MMA, ready to load
//   ss  [G][rows] float: S per group and row
//   rs  [rows] power-of-two row scale
struct Staged {
  unsigned char* xs;
  float4* c4;
  float* ss;
  float* rs;
  int XS;
};
__host__ __device__ inline size_t staged_bytes(int K, int rows) {
  const size_t G = (size_t)(K / 64), pairs = (size_t)((rows + 1) / 2);
  return (size_t)rows * (2 * K + 16) + 16 * G * pairs + sizeof(float) * G * rows + sizeof(float) * rows;
}
__device__ __forceinline__ Staged staged_at(unsigned char* smem, int K, int rows) {
  Staged s;
  const size_t G = (size_t)(K / 64), pairs = (size_t)((rows + 1) / 2);
  s.XS = 2 * K + 16;
  s.xs = smem;
  s.c4 = reinterpret_cast<float4*>(smem + (size_t)rows * s.XS);
  s.ss = reinterpret_cast<float*>(s.c4 + G * pairs);
  s.rs = s.ss + G * rows;
  return s;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// After the copies have landed (cp_async_wait_all + barrier by the caller): per (row, group) the sums S and -C of
// the first n_valid of the `rows` staged rows (the others are never read back: an MMA column only depends on its
// own activation row, and results of unused rows are not stored).
// BITS == 4: stored elements at positions 2,3,6,7 of every eight are true elements / 16.
template <int BITS>
__device__ __forceinline__ void stage_sums(const Staged& s, int rows, int n_valid, int K, int tid, int nthreads) {
  const int G = K / 64, pairs = (rows + 1) / 2;
  for (int i = tid; i < n_valid * G; i += nthreads) {
    const int r = i / G, g = i % G;
    const uint4* p = reinterpret_cast<const uint4*>(s.xs + (size_t)r * s.XS + g * 128);
    float plain = 0.f, div = 0.f;  // sums of the stored values at plain / divided positions
#pragma unroll
    for (int cc = 0; cc < 8; ++cc) {
      const uint4 v = p[(cc + g) & 7];  // rotate the chunk order so that a warp's lanes hit distinct banks
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
      const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
      const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
      plain += (a.x + a.y) + (c.x + c.y);
      div += (b.x + b.y) + (d.x + d.y);
    }
    float S, nC;
    if constexpr (BITS == 4) {
      S = plain + 16.0f * div;
      nC = -1024.0f * (plain + div);
    } else {
      S = plain + div;
      nC = -1024.0f * S;
    }
    s.ss[(size_t)g * rows + r] = S;
    float* c = reinterpret_cast<float*>(s.c4 + (size_t)g * pairs + (r >> 1));
    c[r & 1] = nC;
    c[(r & 1) + 2] = nC;
  }
}

// One group of one 8-row tile: four MMAs starting from -C, then the affine fold.
template <int BITS>
__device__ __forceinline__ void group_step(const typename WVec<BITS>::T& wa, const typename WVec<BITS>::T& wb, const uint4& x0,
                                           const uint4& x1, const float4& c4, const float2& s2, float fsa, float fba, float fsb,
                                           float fbb, float (&tot)[4]) {
  float acc[4];
  uint32_t a[4];
  a_frag<BITS>(wa, wb, 0, a);
  mma_f16_16816(acc, a[0], a[1], a[2], a[3], x0.x, x0.y, c4.x, c4.y, c4.z, c4.w);
  a_frag<BITS>(wa, wb, 1, a);
  mma_f16_16816(acc, a[0], a[1], a[2], a[3], x0.z, x0.w, acc[0], acc[1], acc[2], acc[3]);
  a_frag<BITS>(wa, wb, 2, a);
  mma_f16_16816(acc, a[0], a[1], a[2], a[3], x1.x, x1.y, acc[0], acc[1], acc[2], acc[3]);
  a_frag<BITS>(wa, wb, 3, a);
  mma_f16_16816(acc, a[0], a[1], a[2], a[3], x1.z, x1.w, acc[0], acc[1], acc[2], acc[3]);
  tot[0] = fmaf(fsa, acc[0], fmaf(fba, s2.x, tot[0]));
  tot[1] = fmaf(fsa, acc[1], fmaf(fba, s2.y, tot[1]));
  tot[2] = fmaf(fsb, acc[2], fmaf(fbb, s2.x, tot[2]));
  tot[3] = fmaf(fsb, acc[3], fmaf(fbb, s2.y, tot[3]));
}

// One warp: NT tiles of 8 activation rows against 16 weight rows of one expert matrix over the quantisation
// groups of the blocks blk0, blk0 + step, ... (a block = GB groups: 4 for 4-bit, 2 for 8-bit codes, 64 bytes per
// lane either way); adds into tot[nt][4] (c-fragment layout: [0],[1] = weight row A against rows 2t, 2t+1 of
// the tile; [2],[3] = weight row B).  Two blocks are always in flight (two register buffers, each refilled as
// soon as its products are issued), and start() issues the loads of the first two so that the caller can
// overlap them with staging the activation rows.
//   fetch.block(g0) then fetch(u, nt, x0, x1, c4, s2): the lane's 16 prepared activations of group g0+u of tile
//       row gq (its B fragments), the C operand (-C of rows 2t, 2t+1, twice) and S of rows 2t, 2t+1
//   wa_lane / wb_lane : packed words of the lane's weight rows A (tile row gq) and B (gq+8), already advanced to the
//       lane's share of a group (t * words-per-lane); rows beyond N point at any valid row (results unused)
//   s_a, b_a, s_b, b_b : the rows' bf16 scales and biases (G per row)
// G % GB != 0 (K not a multiple of 256 / 128) takes a guarded path, one group at a time.
template <int BITS>
struct WeightStream {
  static constexpr int GB = (BITS == 4) ? 4 : 2;   // groups per block
  static constexpr int WPG = (BITS == 4) ? 8 : 16;  // packed words per group per row
  using WV = WVec<BITS>;
  struct Buf {
    typename WV::T wa[GB], wb[GB];
    uint2 sa, ba, sb, bb;  // GB bf16 scales / biases per row (8-bit: .x only)
  };
  const uint32_t *pa, *pb;
  const unsigned short *s_a, *b_a, *s_b, *b_b;
  int G, nblk, blk, step;
  bool full;
  Buf A, B;

  __device__ __forceinline__ void load(Buf& b, int bk) const {
    const uint32_t* qa = pa + bk * (GB * WPG);
    const uint32_t* qb = pb + bk * (GB * WPG);
#pragma unroll
    for (int u = 0; u < GB; ++u) {
      b.wa[u] = WV::load(qa + u * WPG);
      b.wb[u] = WV::load(qb + u * WPG);
    }
    if constexpr (GB == 4) {
      b.sa = ldg_nc_v2(s_a + bk * 4);
      b.ba = ldg_nc_v2(b_a + bk * 4);
      b.sb = ldg_nc_v2(s_b + bk * 4);
      b.bb = ldg_nc_v2(b_b + bk * 4);
    } else {
      b.sa = make_uint2(__ldg(reinterpret_cast<const unsigned int*>(s_a + bk * 2)), 0);
      b.ba = make_uint2(__ldg(reinterpret_cast<const unsigned int*>(b_a + bk * 2)), 0);
      b.sb = make_uint2(__ldg(reinterpret_cast<const unsigned int*>(s_b + bk * 2)), 0);
      b.bb = make_uint2(__ldg(reinterpret_cast<const unsigned int*>(b_b + bk * 2)), 0);
    }
  }
  // Sets the stream up and issues the loads of its first block.
  __device__ __forceinline__ void start(const uint32_t* wa_lane, const uint32_t* wb_lane, const unsigned short* sa_,
                                        const unsigned short* ba_, const unsigned short* sb_, const unsigned short* bb_,
                                        int G_, int blk0, int blk_step) {
    pa = wa_lane;
    pb = wb_lane;
    s_a = sa_;
    b_a = ba_;
    s_b = sb_;
    b_b = bb_;
    G = G_;
    nblk = (G_ + GB - 1) / GB;
    blk = blk0;
    step = blk_step;
    full = (G_ % GB) == 0;
    if (full && blk < nblk) load(A, blk);
    if (full && blk + step < nblk) load(B, blk + step);
  }
  template <int NT, class Fetch>
  __device__ __forceinline__ void products(const Buf& b, int bk, Fetch& fetch, float (&tot)[NT][4]) const {
    fetch.block(bk * GB);
#pragma unroll
    for (int u = 0; u < GB; ++u) {
      const float fsa = bf16_of(b.sa, u), fba = bf16_of(b.ba, u), fsb = bf16_of(b.sb, u), fbb = bf16_of(b.bb, u);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        uint4 x0, x1;
        float4 c4;
        float2 s2;
        fetch(u, nt, x0, x1, c4, s2);
        group_step<BITS>(b.wa[u], b.wb[u], x0, x1, c4, s2, fsa, fba, fsb, fbb, tot[nt]);
      }
    }
  }
  // The products of all blocks of the stream (after the activation rows are staged).
  template <int NT, class Fetch>
  __device__ __forceinline__ void run(Fetch fetch, float (&tot)[NT][4]) {
    if (full) {  // two blocks are always in flight: the buffer just consumed is refilled two blocks ahead
      for (int bk = blk; bk < nblk; bk += 2 * step) {
        products<NT>(A, bk, fetch, tot);
        if (bk + 2 * step < nblk) load(A, bk + 2 * step);
        if (bk + step < nblk) {
          products<NT>(B, bk + step, fetch, tot);
          if (bk + 3 * step < nblk) load(B, bk + 3 * step);
        }
      }
    } else {  // ragged last block: one group at a time
      for (int bk = blk; bk < nblk; bk += step) {
        fetch.block(bk * GB);
        for (int u = 0; u < GB; ++u) {
          const int g = bk * GB + u;
          if (g >= G) break;
          const typename WV::T wa = WV::load(pa + g * WPG), wb = WV::load(pb + g * WPG);
          const float fsa = bf16_bits_to_f32(__ldg(s_a + g)), fba = bf16_bits_to_f32(__ldg(b_a + g));
          const float fsb = bf16_bits_to_f32(__ldg(s_b + g)), fbb = bf16_bits_to_f32(__ldg(b_b + g));
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            uint4 x0, x1;
            float4 c4;
            float2 s2;
            fetch(u, nt, x0, x1, c4, s2);
            group_step<BITS>(wa, wb, x0, x1, c4, s2, fsa, fba, fsb, fbb, tot[nt]);
          }
        }
      }
    }
  }
};

// The fetch of a CTA whose ROWS staged rows are the tile rows themselves (row r of the tile = staged row r).
template <int ROWS>
struct StagedFetch {
  const unsigned char* xl;  // xs + gq * XS + t * 32
  const float4* cl;         // c4 + t
  const float* sl;          // ss + 2 * t
  int XS;
  const unsigned char* xb;
  const float4* cb;
  const float* sb;
  __device__ __forceinline__ StagedFetch(const Staged& s, int gq, int t)
      : xl(s.xs + (size_t)gq * s.XS + t * 32), cl(s.c4 + t), sl(s.ss + 2 * t), XS(s.XS), xb(nullptr), cb(nullptr), sb(nullptr) {}
  __device__ __forceinline__ void block(int g0) {
    xb = xl + g0 * 128;
    cb = cl + g0 * (ROWS / 2);
    sb = sl + g0 * ROWS;
  }
  __device__ __forceinline__ void operator()(int u, int nt, uint4& x0, uint4& x1, float4& c4, float2& s2) const {
    const uint4* xp = reinterpret_cast<const uint4*>(xb + (size_t)nt * 8 * XS + u * 128);
    x0 = xp[0];
    x1 = xp[1];
    c4 = cb[u * (ROWS / 2) + nt * 4];
    s2 = *reinterpret_cast<const float2*>(sb + u * ROWS + nt * 8);
  }
};

// The fetch of a warp whose tile is ONE staged row (row j of `rows` staged rows) in all eight columns: column 0 of the
// result (lanes t == 0, elements [0] and [2]) is that row's product, the other columns repeat it.
struct SingleRowFetch {
  const unsigned char* xl;  // xs + j * XS + t * 32
  const float* cj;          // the row's -C inside c4[g][pair]
  const float* sj;          // ss + j
  int rows, pairs;
  const unsigned char* xb;
  const float* cb;
  const float* sb;
  __device__ __forceinline__ SingleRowFetch(const Staged& s, int rows_, int j, int t)
      : xl(s.xs + (size_t)j * s.XS + t * 32),
        cj(reinterpret_cast<const float*>(s.c4 + (j >> 1)) + (j & 1)),
        sj(s.ss + j),
        rows(rows_),
        pairs((rows_ + 1) / 2),
        xb(nullptr),
        cb(nullptr),
        sb(nullptr) {}
  __device__ __forceinline__ void block(int g0) {
    xb = xl + g0 * 128;
    cb = cj + (size_t)g0 * pairs * 4;
    sb = sj + (size_t)g0 * rows;
  }
  __device__ __forceinline__ void operator()(int u, int, uint4& x0, uint4& x1, float4& c4, float2& s2) const {
    const uint4* xp = reinterpret_cast<const uint4*>(xb + u * 128);
    x0 = xp[0];
    x1 = xp[1];
    const float c = cb[(size_t)u * pairs * 4], sv = sb[(size_t)u * rows];
    c4 = make_float4(c, c, c, c);
    s2 = make_float2(sv, sv);
  }
};

// Position of element n of a row in the prepared layout, and the factor it is stored with.
template <int BITS>
__device__ __forceinline__ int prepared_pos(int n) {
  if constexpr (BITS == 4) {
    const int j = n & 7;
    return (n & ~7) | ((j & 3) * 2 + (j >> 2));
  } else {
    return n;
  }
}
template <int BITS>
__device__ __forceinline__ float prepared_factor(int n) {
  if constexpr (BITS == 4)
    return (n & 1) ? 0.0625f : 1.0f;
  else
    return 1.0f;
}
// float32 -> fp16 bits, round to nearest, finite overflow saturates
__device__ __forceinline__ unsigned short f16_sat_bits(float f) {
  unsigned short h;
  asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
  return h;
}

// Prepares one activation row (one warp): xs[:] = fp16( x[:] * 2^-e ) where 2^e (written to *row_scale) brings the
// row's largest magnitude into [2^14, 2^15); BITS == 4: aligned groups of eight elements are stored as
// [0,4,1,5,2,6,3,7] with elements 1,3,5,7 divided by 16.  The scaling is exact for bf16 and fp16 input
// unless an element is more than 2^24 below the row maximum.  x: bf16 (IN_F16: fp16), 8 elements per uint4.
template <int BITS, bool IN_F16>
__device__ __forceinline__ void prepare_row_warp(const uint4* __restrict__ xr, int vec_per_row, uint4* __restrict__ out,
                                                 float* __restrict__ row_scale, int lane) {
  auto widen = [](uint32_t u, float& lo, float& hi) {
    if constexpr (IN_F16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u));
      lo = f.x;
      hi = f.y;
    } else {
      lo = __uint_as_float(u << 16);
      hi = __uint_as_float(u & 0xffff0000u);
    }
  };
  float mx = 0.f;
  for (int c = lane; c < vec_per_row; c += 32) {
    const uint4 v = __ldg(xr + c);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float lo, hi;
      widen(u[q], lo, hi);
      mx = fmaxf(mx, fmaxf(fabsf(lo), fabsf(hi)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  int ex = (mx > 0.f && mx < 3.0e38f) ? (ilogbf(mx) - 14) : 0;
  ex = max(-100, min(100, ex));
  const float f = ldexpf(1.0f, -ex);
  if (lane == 0) *row_scale = ldexpf(1.0f, ex);
  for (int c = lane; c < vec_per_row; c += 32) {
    const uint4 v = __ldg(xr + c);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    float e[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) widen(u[q], e[2 * q], e[2 * q + 1]);
    auto pack = [&](float a, float b) {
      __half2 h2 = __floats2half2_rn(a * f, b * f);
      return *reinterpret_cast<uint32_t*>(&h2);
    };
    uint4 o;
    if constexpr (BITS == 4) {
      const float f16th = 0.0625f;
      o.x = pack(e[0], e[4]);
      o.y = pack(e[1] * f16th, e[5] * f16th);
      o.z = pack(e[2], e[6]);
      o.w = pack(e[3] * f16th, e[7] * f16th);
    } else {
      o.x = pack(e[0], e[1]);
      o.y = pack(e[2], e[3]);
      o.z = pack(e[4], e[5]);
      o.w = pack(e[6], e[7]);
    }
    out[c] = o;
  }
}

}  // namespace qs
}  // namespace b200

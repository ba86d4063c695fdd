// Grouped quantized expert GEMM for the memory-bound regime (few rows per expert).
//
// Replaces gather_qmm(x, w, scales, biases, rhs_indices, transpose=true, sorted_indices=true)
// (mlx-rs/src/ops/quantization.rs:160-230) for rows already grouped by expert, with the two
// epilogues of the routed block fused in:
//   NMAT = 2: gate and up projections in one pass, h = silu(x.Wg^T) * (x.Wu^T)
//             (nn::silu, mlx-rs/src/nn/activation.rs:876-880, and multiply);
//   NMAT = 1: down projection, each output row optionally multiplied by its routing weight
//             (multiply before sum_axis, mlx-rs/src/ops/reduction.rs:260-275) and written to
//             its un-sorted position (take with the inverse order).
//
// Every packed weight byte is read from HBM exactly once per pass, with 64-bit (4-bit codes)
// or 128-bit (8-bit codes) coalesced loads straight into registers, and never touches shared
// memory.  The codes are turned into exact small bf16 integers in registers (q+128 for 4-bit
// by OR-ing the nibble into the mantissa of 128.0; q via a float32 magic number for 8-bit) and
// fed to mma.sync m16n8k16 as the A operand: 16 output features x 16 k, against B = 8 rows of
// x from shared memory.  One quantisation group (64 k) is exactly four MMAs of a quad's data,
// so the group's integer dot product lands in a fresh float32 accumulator and is folded as
//   total += scale * acc + (bias - 128*scale) * sum_k(x)          (4-bit)
// which is the affine dequantisation applied exactly, in float32, with no rounding of the
// dequantised weight.  The k order inside an MMA is permuted identically on both operands.
//
// CTA = 8 warps = RT row tiles (16 output features each) x KS slices of the K groups;
// partial sums of the KS slices meet in shared memory in a fixed order.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 4-bit: nibbles j and j+4 of a word -> bf16x2 (128+q_j, 128+q_{j+4})
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, int j) { return ((w >> (4 * j)) & 0x000f000fu) | 0x43004300u; }
// 8-bit: bytes j and j+1 of a word -> bf16x2 (q_j, q_{j+1})
__device__ __forceinline__ uint32_t byte_pair(uint32_t w, int j) {
  float f0 = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7440 + j)) - 8388608.0f;
  float f1 = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7440 + j + 1)) - 8388608.0f;
  __nv_bfloat162 p = __floats2bfloat162_rn(f0, f1);
  return *reinterpret_cast<uint32_t*>(&p);
}

template <int BITS>
struct WVec;
template <>
struct WVec<4> {
  using T = uint2;  // 16 codes
  static __device__ __forceinline__ T load(const uint32_t* p) { return ldg_nc_v2(p); }
  static __device__ __forceinline__ T zero() { return make_uint2(0, 0); }
};
template <>
struct WVec<8> {
  using T = uint4;  // 16 codes
  static __device__ __forceinline__ T load(const uint32_t* p) { return ldg_nc_v4(p); }
  static __device__ __forceinline__ T zero() { return make_uint4(0, 0, 0, 0); }
};

// A-operand registers of MMA i (0..3) of a group for the two rows (g, g+8) a thread holds
template <int BITS>
__device__ __forceinline__ void a_frag(const typename WVec<BITS>::T& ra, const typename WVec<BITS>::T& rb, int i,
                                       uint32_t (&a)[4]) {
  if constexpr (BITS == 4) {
    uint32_t wa = (i < 2) ? ra.x : ra.y, wb = (i < 2) ? rb.x : rb.y;
    int j = (i & 1) * 2;
    a[0] = nib_pair(wa, j);
    a[1] = nib_pair(wb, j);
    a[2] = nib_pair(wa, j + 1);
    a[3] = nib_pair(wb, j + 1);
  } else {
    uint32_t wa = (i == 0) ? ra.x : (i == 1) ? ra.y : (i == 2) ? ra.z : ra.w;
    uint32_t wb = (i == 0) ? rb.x : (i == 1) ? rb.y : (i == 2) ? rb.z : rb.w;
    a[0] = byte_pair(wa, 0);
    a[1] = byte_pair(wb, 0);
    a[2] = byte_pair(wa, 2);
    a[3] = byte_pair(wb, 2);
  }
}

template <int BITS, int NMAT, int RT, int NT>
__global__ void __launch_bounds__(256) grouped_qmm_small_kernel(GroupedArgs p) {
  constexpr int KS = 8 / RT;
  constexpr int UG = 4;           // groups in flight per warp
  constexpr int ROWS = 8 * NT;    // x rows per pass
  constexpr int WPG = (BITS == 4) ? 8 : 16;    // packed words per group per row
  constexpr int WPT = (BITS == 4) ? 2 : 4;     // packed words per thread per group per row
  constexpr float kOff = (BITS == 4) ? 128.0f : 0.0f;
  using WV = WVec<BITS>;

  pdl_prologue();
  const int ea = blockIdx.y;
  if (ea >= (int)*p.n_active) return;
  const int e = p.active[ea];
  const uint32_t seg0 = p.offsets[e];
  const int m = (int)(p.offsets[e + 1] - seg0);
  if (m <= 0) return;

  const int K = p.K, N = p.N, G = K / 64;
  const int XS = 2 * K + 16;  // bytes per staged x row (+16 keeps the two rows of a quad-pair on distinct banks)
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* xs = smem;
  float* xsum = reinterpret_cast<float*>(smem + (size_t)ROWS * XS);  // [G][ROWS]
  float* red = reinterpret_cast<float*>(smem);                          // aliases xs after the K loop

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, t = lane & 3;
  const int rt = warp % RT, ks = warp / RT;
  const int n0 = blockIdx.x * (16 * RT) + rt * 16;
  const int wrow = K * BITS / 32;  // packed words per weight row

  const uint32_t* wbase[NMAT];
  const unsigned short* sbase[NMAT];
  const unsigned short* bbase[NMAT];
#pragma unroll
  for (int mt = 0; mt < NMAT; ++mt) {
    wbase[mt] = p.w[mt] + ((size_t)e * N + n0) * wrow;
    sbase[mt] = reinterpret_cast<const unsigned short*>(p.scales[mt]) + ((size_t)e * N + n0) * G;
    bbase[mt] = reinterpret_cast<const unsigned short*>(p.biases[mt]) + ((size_t)e * N + n0) * G;
  }
  const bool row_ok_a = (n0 + gq) < N, row_ok_b = (n0 + gq + 8) < N;

  for (int p0 = 0; p0 < m; p0 += ROWS) {
    // ---- stage up to ROWS rows of x: k-permuted bf16 + per-group sums --------------------
    {
      const int pieces = K / 16;  // 16-element pieces per row; 4 pieces = one group
      for (int i = tid; i < ROWS * pieces; i += 256) {
        const int r = i / pieces, c = i % pieces;
        const int pr = p0 + r;
        uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
        if (pr < m) {
          uint32_t sp = seg0 + pr;
          uint32_t src;
          if (p.src_mode == kSrcIdent)
            src = sp;
          else if (p.src_mode == kSrcPermDiv)
            src = p.perm[sp] / (uint32_t)p.src_div;
          else
            src = p.src_map[p.perm[sp]];
          const uint4* g = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(p.x) + ((size_t)src * K + c * 16) * 2);
          v0 = __ldg(g);
          v1 = __ldg(g + 1);
        }
        float s = 0.f;
        {
          const uint32_t u[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int q = 0; q < 8; ++q) s += __uint_as_float(u[q] << 16) + __uint_as_float(u[q] & 0xffff0000u);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if ((c & 3) == 0) xsum[(c >> 2) * ROWS + r] = s;
        if constexpr (BITS == 4) {  // element order [0,4,1,5,2,6,3,7] inside each 8
          uint4 o0, o1;
          o0.x = __byte_perm(v0.x, v0.z, 0x5410);
          o0.y = __byte_perm(v0.x, v0.z, 0x7632);
          o0.z = __byte_perm(v0.y, v0.w, 0x5410);
          o0.w = __byte_perm(v0.y, v0.w, 0x7632);
          o1.x = __byte_perm(v1.x, v1.z, 0x5410);
          o1.y = __byte_perm(v1.x, v1.z, 0x7632);
          o1.z = __byte_perm(v1.y, v1.w, 0x5410);
          o1.w = __byte_perm(v1.y, v1.w, 0x7632);
          v0 = o0;
          v1 = o1;
        }
        uint4* d = reinterpret_cast<uint4*>(xs + (size_t)r * XS + c * 32);
        d[0] = v0;
        d[1] = v1;
      }
    }
    __syncthreads();

    float tot[NMAT][NT][4];
#pragma unroll
    for (int mt = 0; mt < NMAT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) tot[mt][nt][q] = 0.f;

    for (int g0 = ks; g0 < G; g0 += KS * UG) {
      typename WV::T wa[UG][NMAT], wb[UG][NMAT];
      unsigned short sa[UG][NMAT], sb[UG][NMAT], ba[UG][NMAT], bb[UG][NMAT];
#pragma unroll
      for (int u = 0; u < UG; ++u) {
        const int g = g0 + u * KS;
#pragma unroll
        for (int mt = 0; mt < NMAT; ++mt) {
          const bool ok = g < G;
          const uint32_t* pa = wbase[mt] + (size_t)gq * wrow + g * WPG + t * WPT;
          wa[u][mt] = (ok && row_ok_a) ? WV::load(pa) : WV::zero();
          wb[u][mt] = (ok && row_ok_b) ? WV::load(pa + (size_t)8 * wrow) : WV::zero();
          sa[u][mt] = (ok && row_ok_a) ? __ldg(sbase[mt] + (size_t)gq * G + g) : (unsigned short)0;
          ba[u][mt] = (ok && row_ok_a) ? __ldg(bbase[mt] + (size_t)gq * G + g) : (unsigned short)0;
          sb[u][mt] = (ok && row_ok_b) ? __ldg(sbase[mt] + (size_t)(gq + 8) * G + g) : (unsigned short)0;
          bb[u][mt] = (ok && row_ok_b) ? __ldg(bbase[mt] + (size_t)(gq + 8) * G + g) : (unsigned short)0;
        }
      }
#pragma unroll
      for (int u = 0; u < UG; ++u) {
        const int g = g0 + u * KS;
        if (g < G) {
          float acc[NMAT][NT][4];
#pragma unroll
          for (int mt = 0; mt < NMAT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int q = 0; q < 4; ++q) acc[mt][nt][q] = 0.f;
          uint4 xv[NT][2];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + gq) * XS + (g * 4 + t) * 32);
            xv[nt][0] = xp[0];
            xv[nt][1] = xp[1];
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int mt = 0; mt < NMAT; ++mt) {
              uint32_t a[4];
              a_frag<BITS>(wa[u][mt], wb[u][mt], i, a);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const uint4& v = xv[nt][i >> 1];
                uint32_t b0 = (i & 1) ? v.z : v.x, b1 = (i & 1) ? v.w : v.y;
                mma_bf16_16816(acc[mt][nt], a[0], a[1], a[2], a[3], b0, b1);
              }
            }
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const float2 xsm = *reinterpret_cast<const float2*>(&xsum[g * ROWS + nt * 8 + 2 * t]);
#pragma unroll
            for (int mt = 0; mt < NMAT; ++mt) {
              const float s_a = bf16_bits_to_f32(sa[u][mt]), s_b = bf16_bits_to_f32(sb[u][mt]);
              const float b_a = bf16_bits_to_f32(ba[u][mt]) - kOff * s_a, b_b = bf16_bits_to_f32(bb[u][mt]) - kOff * s_b;
              tot[mt][nt][0] += s_a * acc[mt][nt][0] + b_a * xsm.x;
              tot[mt][nt][1] += s_a * acc[mt][nt][1] + b_a * xsm.y;
              tot[mt][nt][2] += s_b * acc[mt][nt][2] + b_b * xsm.x;
              tot[mt][nt][3] += s_b * acc[mt][nt][3] + b_b * xsm.y;
            }
          }
        }
      }
    }
    __syncthreads();  // everyone is done with xs / xsum: red may overwrite them

    // ---- partial sums -> shared, [warp][mat][nt][row16][tok8] ------------------------------
#pragma unroll
    for (int mt = 0; mt < NMAT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float* r = red + ((size_t)(warp * NMAT + mt) * NT + nt) * 128;
        r[gq * 8 + 2 * t] = tot[mt][nt][0];
        r[gq * 8 + 2 * t + 1] = tot[mt][nt][1];
        r[(gq + 8) * 8 + 2 * t] = tot[mt][nt][2];
        r[(gq + 8) * 8 + 2 * t + 1] = tot[mt][nt][3];
      }
    __syncthreads();

    // ---- epilogue: fixed-order sum over the K slices, activation / routing weight, store ----
    for (int o = tid; o < 16 * RT * ROWS; o += 256) {
      const int rl = o % (16 * RT), tok = o / (16 * RT);
      const int pr = p0 + tok, n = blockIdx.x * (16 * RT) + rl;
      if (pr >= m || n >= N) continue;
      const int ert = rl >> 4, r16 = rl & 15, nt = tok >> 3, t8 = tok & 7;
      float v[NMAT];
#pragma unroll
      for (int mt = 0; mt < NMAT; ++mt) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < KS; ++q) s += red[((size_t)((q * RT + ert) * NMAT + mt) * NT + nt) * 128 + r16 * 8 + t8];
        v[mt] = s;
      }
      const uint32_t sp = seg0 + pr;
      const uint32_t dst = p.dst_perm ? p.perm[sp] : sp;
      float outv;
      if constexpr (NMAT == 2) {
        outv = v[0] / (1.0f + __expf(-v[0])) * v[1];
      } else {
        outv = v[0];
        if (p.row_scale) outv *= bf16_bits_to_f32(reinterpret_cast<const unsigned short*>(p.row_scale)[dst]);
      }
      if (p.out_row_addr)
        reinterpret_cast<__nv_bfloat16*>(p.out_row_addr[sp])[n] = __float2bfloat16_rn(outv);
      else if (p.out_f32)
        reinterpret_cast<float*>(p.out)[(size_t)dst * N + n] = outv;
      else
        reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)dst * N + n] = __float2bfloat16_rn(outv);
    }
    __syncthreads();
  }
}

template <int BITS, int NMAT, int RT, int NT>
static int launch_cfg(const GroupedArgs& a, int max_active, cudaStream_t st) {
  const int K = a.K;
  size_t smem = (size_t)8 * NT * (2 * K + 16) + sizeof(float) * (K / 64) * 8 * NT;
  size_t red = sizeof(float) * 8 * NMAT * NT * 128;
  if (red > smem) smem = red;
  auto kern = grouped_qmm_small_kernel<BITS, NMAT, RT, NT>;
  static DynSmemCache attr;
  B200_CUDA(ensure_dyn_smem(kern, smem, attr));
  dim3 grid(cdiv(a.N, 16 * RT), max_active);
  B200_CUDA(launch_pdl(kern, grid, dim3(256), smem, st, a));
  return 0;
}

template <int BITS, int NMAT>
static int launch_bits_nmat(const GroupedArgs& a, int max_active, int64_t rows, cudaStream_t st) {
  // largest row tile that still yields at least two CTAs per SM; more x rows per pass once
  // the experts are expected to hold more than eight rows each
  const int64_t per = rows / (max_active > 0 ? max_active : 1);
  const bool wide = per > 8;
  int rt = 1;
  for (int cand : {8, 4, 2}) {
    if ((int64_t)cdiv(a.N, 16 * cand) * max_active >= 296) {
      rt = cand;
      break;
    }
  }
  // shared memory for the wide variant: 32 rows of x must fit
  const bool wide_fits = ((size_t)32 * (2 * a.K + 16) + sizeof(float) * (a.K / 64) * 32) <= 200 * 1024;
#define B200_DISPATCH_RT(RTV)                                                          \
  case RTV:                                                                            \
    return (wide && wide_fits) ? launch_cfg<BITS, NMAT, RTV, 4>(a, max_active, st)     \
                               : launch_cfg<BITS, NMAT, RTV, 1>(a, max_active, st);
  switch (rt) {
    B200_DISPATCH_RT(1)
    B200_DISPATCH_RT(2)
    B200_DISPATCH_RT(4)
    B200_DISPATCH_RT(8)
  }
#undef B200_DISPATCH_RT
  return 0;
}

int launch_grouped_qmm_small(const GroupedArgs& a, int nmat, int bits, int max_active, int64_t rows, cudaStream_t st) {
  if (rows == 0 || max_active == 0) return 0;
  B200_REQUIRE(a.K % 64 == 0, "K must be a multiple of the group size 64");
  B200_REQUIRE((size_t)8 * (2 * a.K + 16) + sizeof(float) * (a.K / 64) * 8 <= 220 * 1024, "K too large for the staged x rows");
  if (bits == 4) return nmat == 2 ? launch_bits_nmat<4, 2>(a, max_active, rows, st) : launch_bits_nmat<4, 1>(a, max_active, rows, st);
  if (bits == 8) return nmat == 2 ? launch_bits_nmat<8, 2>(a, max_active, rows, st) : launch_bits_nmat<8, 1>(a, max_active, rows, st);
  B200_FAIL("bits must be 4 or 8");
}

}  // namespace b200

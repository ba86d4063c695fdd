// Router kernels: gate Linear (exact, correctly rounded bf16 logits), softmax / top-k /
// renormalisation per token, plus the stand-alone softmax, argpartition and take_along_axis
// ops of the reference surface.
//
// Reference call sites replaced: nn::Linear forward (mlx-rs/src/nn/linear.rs:83-95),
// softmax_axis (mlx-rs/src/ops/arithmetic.rs:1312-1327), argpartition_axis
// (mlx-rs/src/ops/sort.rs:186-226), take_along_axis (mlx-rs/src/ops/indexing/mod.rs:424-453),
// sum_axis + divide for the renormalisation.
//
// Routing must be bit-exact, so every value a routing decision depends on is defined as the
// correctly rounded bf16 of an exactly specified quantity: the logit is the exact dot product
// of the bf16 operands (accumulated in float64: products of two bf16 numbers are exact in
// float64 and the sum carries ~2^-53 relative error, far below half a bf16 ulp), the
// probability is the exact softmax of those bf16 logits.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "permute_small.cuh"
#include "router_common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------
// logits[t,e] = RN_bf16( sum_h x[t,h] * w[e,h] )   in float64.
// CTA tile: (RT*TGX) tokens x (4*EGX) experts, 256 threads.  A thread owns an RT x 4 output
// tile (tokens tgx + TGX*j, experts egx + EGX*i) and a K-slice: the 256 threads are split
// into KS = 256/(TGX*EGX) slices of every staged K-chunk.  Operands are converted to float64
// once while staging them k-major in shared memory, so the inner loop is LDS.64 + DFMA.
// ---------------------------------------------------------------------------------------
template <int RT, int TGX, int EGX>
__global__ void __launch_bounds__(256) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            const float* __restrict__ logit_bias,
                                                            __nv_bfloat16* __restrict__ logits, int T, int H, int E) {
  constexpr int TT = RT * TGX, TE = 4 * EGX, NTILE = TGX * EGX, KS = 256 / NTILE;
  constexpr int KC = (TT + TE > 64) ? 32 : 64;  // keeps static shared memory under 48 KB
  static_assert(256 % NTILE == 0 && KC % KS == 0, "tile shape");
  constexpr int KPT = KC / KS;  // k-steps per thread per chunk
  // rows padded by one double so that the transposing stores below spread over all banks
  __shared__ double xs[KC][TT + 1];
  __shared__ double ws[KC][TE + 1];

  const int tid = threadIdx.x;
  const int tile = tid % NTILE, ks = tid / NTILE;
  const int tgx = tile % TGX, egx = tile / TGX;
  const int t0 = blockIdx.y * TT, e0 = blockIdx.x * TE;

  double acc[RT][4];
#pragma unroll
  for (int j = 0; j < RT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.0;

  const unsigned short* xb = reinterpret_cast<const unsigned short*>(x);
  const unsigned short* wb = reinterpret_cast<const unsigned short*>(w);

  for (int k0 = 0; k0 < H; k0 += KC) {
    // stage: rows along tid / KC, k along tid % KC (coalesced 128 B per row segment)
    for (int i = tid; i < TT * KC; i += 256) {
      int r = i / KC, k = i % KC;
      int t = t0 + r;
      uint32_t b = (t < T && k0 + k < H) ? xb[(size_t)t * H + k0 + k] : 0u;
      xs[k][r] = bf16_bits_to_f64(b);
    }
    for (int i = tid; i < TE * KC; i += 256) {
      int r = i / KC, k = i % KC;
      int e = e0 + r;
      uint32_t b = (e < E && k0 + k < H) ? wb[(size_t)e * H + k0 + k] : 0u;
      ws[k][r] = bf16_bits_to_f64(b);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KPT; ++kk) {
      const int k = ks * KPT + kk;
      double xv[RT], wv[4];
#pragma unroll
      for (int j = 0; j < RT; ++j) xv[j] = xs[k][tgx + TGX * j];
#pragma unroll
      for (int i = 0; i < 4; ++i) wv[i] = ws[k][egx + EGX * i];
#pragma unroll
      for (int j = 0; j < RT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = fma(xv[j], wv[i], acc[j][i]);
    }
    __syncthreads();
  }

  // cross-slice reduction in a fixed order (slice 0 + slice 1 + ...)
  if constexpr (KS > 1) {
    __shared__ double red[256 * RT * 4];
#pragma unroll
    for (int j = 0; j < RT; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[(j * 4 + i) * 256 + tid] = acc[j][i];
    __syncthreads();
    if (ks == 0) {
#pragma unroll
      for (int j = 0; j < RT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          double s = acc[j][i];
          for (int q = 1; q < KS; ++q) s += red[(j * 4 + i) * 256 + q * NTILE + tile];
          acc[j][i] = s;
        }
    }
  }
  if (ks == 0) {
#pragma unroll
    for (int j = 0; j < RT; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int t = t0 + tgx + TGX * j, e = e0 + egx + EGX * i;
        if (t < T && e < E) {
          uint32_t bits = f64_to_bf16_bits(acc[j][i]);
          if (logit_bias) bits = f32_to_bf16_bits(bf16_bits_to_f32(bits) + logit_bias[e]);
          logits[(size_t)t * E + e] = __ushort_as_bfloat16((unsigned short)bits);
        }
      }
  }
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// Warp-per-expert variant for token counts that cannot fill the GPU with tiles.
// CTA = 8 warps = 8 experts against kWarpTokens tokens; the token rows and the eight weight rows are
// staged in shared memory as raw bf16 with asynchronous copies.  The weight rows are constants of the
// chain of kernels, so their copies are issued BEFORE the programmatic-dependent-launch wait and land
// while the previous kernel is still finishing.  The loops are deliberately not unrolled: this code
// runs once per launch, and fully unrolled float64 arithmetic costs more in instruction fetch than it
// saves in issue slots (measured: 23 us against 5 us for the same sums).
// ---------------------------------------------------------------------------------------
constexpr int kWarpTokens = 2;  // tokens per pass over the staged weight row
constexpr int kWarpTokensMax = 8;  // most tokens a CTA stages (it then makes four passes)

// copies of the CTA's eight weight rows (experts e0 .. e0+7, clamped) into ws4 [8][nvec]
__device__ __forceinline__ void stage_router_weights(uint4* ws4, const __nv_bfloat16* __restrict__ w, int e0, int E, int H,
                                                     int tid) {
  const int nvec = H / 8;
  for (int i = tid; i < 8 * nvec; i += 256) {
    const int e = min(e0 + i / nvec, E - 1);
    cp_async16(ws4 + i, reinterpret_cast<const uint4*>(w + (size_t)e * H) + i % nvec);
  }
}
// copies of the token rows t0 .. t0+n-1 (those that exist) into xs4 [n][nvec]
__device__ __forceinline__ void stage_router_tokens(uint4* xs4, const __nv_bfloat16* __restrict__ x, int t0, int n, int T,
                                                    int H, int tid) {
  const int nvec = H / 8;
  for (int i = tid; i < n * nvec; i += 256) {
    const int r = i / nvec;
    if (t0 + r < T) cp_async16(xs4 + i, reinterpret_cast<const uint4*>(x + (size_t)(t0 + r) * H) + i % nvec);
  }
}
// logits[t0 + j, e] for two staged tokens (j = 0, 1): exact float64 dot product of the warp's staged weight row with each
// token row, correctly rounded to bf16 (+ the optional float32 logit bias, rounded again).
__device__ __forceinline__ void warp_expert_logits(const uint4* xs4, const uint4* wrow, int nvec, int lane, int t0, int T,
                                                   int e, int E, const float* __restrict__ logit_bias,
                                                   __nv_bfloat16* __restrict__ logits) {
  const bool two = t0 + 1 < T;
  const uint4* xrow0 = xs4;
  const uint4* xrow1 = xs4 + (two ? nvec : 0);
  double a0 = 0.0, a1 = 0.0, b0 = 0.0, b1 = 0.0;
#pragma unroll 1
  for (int c = lane; c < nvec; c += 32) {
    const uint4 wv = wrow[c], xv = xrow0[c], yv = xrow1[c];
    const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w}, xu[4] = {xv.x, xv.y, xv.z, xv.w}, yu[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const double wl = bf16_bits_to_f64(wu[q] & 0xffffu), wh = bf16_bits_to_f64(wu[q] >> 16);
      a0 = fma(bf16_bits_to_f64(xu[q] & 0xffffu), wl, a0);
      a1 = fma(bf16_bits_to_f64(xu[q] >> 16), wh, a1);
      b0 = fma(bf16_bits_to_f64(yu[q] & 0xffffu), wl, b0);
      b1 = fma(bf16_bits_to_f64(yu[q] >> 16), wh, b1);
    }
  }
  double sum0 = a0 + a1, sum1 = b0 + b1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, o);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, o);
  }
  if (e < E && lane < 2 && (lane == 0 || two)) {
    uint32_t bits = f64_to_bf16_bits(lane == 0 ? sum0 : sum1);
    if (logit_bias) bits = f32_to_bf16_bits(bf16_bits_to_f32(bits) + logit_bias[e]);
    logits[(size_t)(t0 + lane) * E + e] = __ushort_as_bfloat16((unsigned short)bits);
  }
}

// The stand-alone kernel (9 to 255 tokens) converts its TPC token rows to float64 ONCE per CTA, into shared memory
// (chunk q of the 8-element vector c of token j at ((j * 4 + q) * nvec + c) * 16 bytes, so that the lanes of a warp
// read consecutive 16-byte chunks), instead of once per expert warp: with the conversions of the token side gone
// from the inner loop, an iteration is 8 weight conversions, 4 * TPC shared loads and 8 * TPC float64 FMAs.
template <int TPC>
__global__ void __launch_bounds__(256) router_logits_warp_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 const float* __restrict__ logit_bias,
                                                                 __nv_bfloat16* __restrict__ logits, int T, int H, int E) {
  extern __shared__ __align__(16) unsigned char rsm[];  // [8 weight rows, raw bf16][TPC token rows, float64]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.y * TPC, nvec = H / 8;
  uint4* ws4 = reinterpret_cast<uint4*>(rsm);
  double2* xd = reinterpret_cast<double2*>(ws4 + (size_t)8 * nvec);
  pdl_trigger();
  stage_router_weights(ws4, w, blockIdx.x * 8, E, H, tid);  // constants: on their way before the wait
  pdl_wait();
  for (int i = tid; i < TPC * nvec; i += 256) {
    const int j = i / nvec, c = i % nvec;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t0 + j < T) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(t0 + j) * H) + c);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q)
      xd[(size_t)(j * 4 + q) * nvec + c] = make_double2(bf16_bits_to_f64(u[q] & 0xffffu), bf16_bits_to_f64(u[q] >> 16));
  }
  cp_async_wait_all();
  __syncthreads();
  const int e = blockIdx.x * 8 + warp;
  const uint4* wrow = ws4 + (size_t)warp * nvec;
  double acc[TPC][2];
#pragma unroll
  for (int j = 0; j < TPC; ++j) acc[j][0] = acc[j][1] = 0.0;
#pragma unroll 1
  for (int c = lane; c < nvec; c += 32) {
    const uint4 wv = wrow[c];
    const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
    double wl[4], wh[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      wl[q] = bf16_bits_to_f64(wu[q] & 0xffffu);
      wh[q] = bf16_bits_to_f64(wu[q] >> 16);
    }
#pragma unroll
    for (int j = 0; j < TPC; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const double2 xv = xd[(size_t)(j * 4 + q) * nvec + c];
        acc[j][0] = fma(xv.x, wl[q], acc[j][0]);
        acc[j][1] = fma(xv.y, wh[q], acc[j][1]);
      }
  }
#pragma unroll
  for (int j = 0; j < TPC; ++j) {
    double sum = acc[j][0] + acc[j][1];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0 && e < E && t0 + j < T) {
      uint32_t bits = f64_to_bf16_bits(sum);
      if (logit_bias) bits = f32_to_bf16_bits(bf16_bits_to_f32(bits) + logit_bias[e]);
      logits[(size_t)(t0 + j) * E + e] = __ushort_as_bfloat16((unsigned short)bits);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Mid and large token counts: float64 tensor-core variant.  CTA = 8 warps over MT*8 tokens x NE*64
// experts; a warp owns all the tokens x NE*8 experts as 8x8 accumulator tiles of mma.sync m8n8k4 (f64).  The
// operands are converted to float64 once per 32-wide K chunk while they are staged in shared
// memory (row-major, rows padded by 32 bytes so that fragment loads spread over all banks);
// two buffers, and the next chunk's global loads are issued before the current chunk's products.
// The tile shape is chosen per launch so that the waves over 148 SMs are full
// (T = 8192: 56 tokens x 128 experts -> 147 CTAs; T = 2048: 32 x 64 -> 128 CTAs).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void dmma_884(double (&c)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c[0]), "+d"(c[1])
               : "d"(a), "d"(b));
}

// Router weight -> float64, once per call (E*H elements): the tiles then stage weight rows with plain
// 16-byte asynchronous copies instead of converting the same rows again in every token tile.
__global__ void router_weight_f64_kernel(const __nv_bfloat16* __restrict__ w, double* __restrict__ w64, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) w64[i] = bf16_bits_to_f64((uint32_t)__bfloat16_as_ushort(w[i]));
}

// W64: the weight arrives as float64 (w64) and is copied, only the token rows are converted.
template <int MT, int NE, int KC, bool W64>
__global__ void __launch_bounds__(256) router_logits_dmma_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 const double* __restrict__ w64,
                                                                 const float* __restrict__ logit_bias,
                                                                 __nv_bfloat16* __restrict__ logits, int T, int H, int E) {
  constexpr int LD = KC + 4, TE = 64 * NE, TT = MT * 8;  // a warp owns NE 8-expert tiles; KC = k per staged chunk
  constexpr int ROWS = W64 ? TT : TT + TE;             // rows that pass through registers (converted)
  constexpr int NLD = (ROWS * (KC / 8) + 255) / 256;  // 128-bit loads per thread and chunk
  extern __shared__ __align__(16) unsigned char dsm[];
  double* buf0 = reinterpret_cast<double*>(dsm);       // two buffers of [TT + TE][LD]
  constexpr int BUF = (TT + TE) * LD;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.x * TT, e0 = blockIdx.y * TE;
  const int r = lane >> 2, kq = lane & 3;

  // small tiles give a warp one or two accumulator tiles: consecutive k steps then alternate between KI
  // independent partial sums so that the tensor-pipe latency of one step does not serialise the next
  constexpr int KI = (MT * NE <= 2) ? 4 : (MT * NE <= 4) ? 2 : 1;
  double acc[KI][MT][NE][2];
#pragma unroll
  for (int q = 0; q < KI; ++q)
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NE; ++j) acc[q][i][j][0] = acc[q][i][j][1] = 0.0;

  uint4 pre[NLD];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int u = 0; u < NLD; ++u) {
      const int i = tid + u * 256;
      const int row = i / (KC / 8), c = i % (KC / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (i < ROWS * (KC / 8) && k0 + c * 8 < H) {
        if (row < TT) {
          if (t0 + row < T) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(t0 + row) * H + k0) + c);
        } else if (e0 + row - TT < E) {
          v = __ldg(reinterpret_cast<const uint4*>(w + (size_t)(e0 + row - TT) * H + k0) + c);
        }
      }
      pre[u] = v;
    }
  };
  auto stash = [&](double* buf) {  // convert the prefetched chunk and store it
#pragma unroll
    for (int u = 0; u < NLD; ++u) {
      const int i = tid + u * 256;
      if (i >= ROWS * (KC / 8)) break;
      const int row = i / (KC / 8), c = i % (KC / 8);
      double* d = buf + row * LD + c * 8;
      const uint32_t q4[4] = {pre[u].x, pre[u].y, pre[u].z, pre[u].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        d[2 * q] = bf16_bits_to_f64(q4[q] & 0xffffu);
        d[2 * q + 1] = bf16_bits_to_f64(q4[q] >> 16);
      }
    }
  };

  auto copy_w = [&](int k0, double* buf) {  // float64 weight rows: 16-byte asynchronous copies (2 elements each)
    if constexpr (W64) {
      for (int i = tid; i < TE * (KC / 2); i += 256) {
        const int row = i / (KC / 2), c = i % (KC / 2);
        double* d = buf + (TT + row) * LD + c * 2;
        if (e0 + row < E && k0 + c * 2 < H)
          cp_async16(d, w64 + (size_t)(e0 + row) * H + k0 + c * 2);
        else
          d[0] = d[1] = 0.0;
      }
    }
  };

  fetch(0);
  copy_w(0, buf0);
  stash(buf0);
  cp_async_wait_all();
  __syncthreads();
  int cur = 0;
  for (int k0 = 0; k0 < H; k0 += KC) {
    const bool more = k0 + KC < H;
    if (more) {
      fetch(k0 + KC);                               // global loads in flight under the products below
      copy_w(k0 + KC, buf0 + (cur ^ 1) * BUF);      // the other buffer was last read before the previous barrier
    }
    const double* xs = buf0 + cur * BUF;
    const double* ws = xs + TT * LD;
#pragma unroll
    for (int kk = 0; kk < KC; kk += 4) {
      double a[MT], b[NE];
#pragma unroll
      for (int i = 0; i < MT; ++i) a[i] = xs[(i * 8 + r) * LD + kk + kq];
#pragma unroll
      for (int j = 0; j < NE; ++j) b[j] = ws[(warp * (8 * NE) + j * 8 + r) * LD + kk + kq];
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NE; ++j) dmma_884(acc[(kk / 4) % KI][i][j], a[i], b[j]);
    }
    if (more) stash(buf0 + (cur ^ 1) * BUF);
    cp_async_wait_all();
    __syncthreads();
    cur ^= 1;
  }
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NE; ++j)
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int t = t0 + i * 8 + r, e = e0 + warp * (8 * NE) + j * 8 + kq * 2 + q;
        if (t < T && e < E) {
          double sum = acc[0][i][j][q];
#pragma unroll
          for (int u = 1; u < KI; ++u) sum += acc[u][i][j][q];
          uint32_t bits = f64_to_bf16_bits(sum);
          if (logit_bias) bits = f32_to_bf16_bits(bf16_bits_to_f32(bits) + logit_bias[e]);
          logits[(size_t)t * E + e] = __ushort_as_bfloat16((unsigned short)bits);
        }
      }
}

template <int MT, int NE>
static int launch_router_dmma(const __nv_bfloat16* xp, const __nv_bfloat16* wp, const double* w64, const float* logit_bias,
                              __nv_bfloat16* lp, int T, int H, int E, cudaStream_t st) {
  // small tiles are bound by the barrier + load round trip per chunk, not by the products: longer chunks
  constexpr int KC = (MT * NE <= 2) ? 128 : (MT * NE <= 4) ? 64 : 32;
  constexpr size_t smem = sizeof(double) * 2 * (MT * 8 + 64 * NE) * (KC + 4);
  dim3 grid(cdiv(T, MT * 8), cdiv(E, 64 * NE));
  if (w64 && H % 2 == 0) {
    auto kern = router_logits_dmma_kernel<MT, NE, KC, true>;
    static DynSmemCache attr;
    B200_CUDA(ensure_dyn_smem(kern, smem, attr));
    const int64_t n = (int64_t)E * H;
    router_weight_f64_kernel<<<cdiv(n, 256), 256, 0, st>>>(wp, const_cast<double*>(w64), n);
    kern<<<grid, 256, smem, st>>>(xp, wp, w64, logit_bias, lp, T, H, E);
  } else {
    auto kern = router_logits_dmma_kernel<MT, NE, KC, false>;
    static DynSmemCache attr;
    B200_CUDA(ensure_dyn_smem(kern, smem, attr));
    kern<<<grid, 256, smem, st>>>(xp, wp, nullptr, logit_bias, lp, T, H, E);
  }
  return 0;
}

// Tile shape (MT*8 tokens x NE*64 experts per CTA) with the least estimated time on 148 SMs:
// waves x (products of a tile + the staging/conversion work of its rows, weighted).
static void dmma_tile_shape(int T, int E, int& mt_best, int& ne_best) {
  double best = 1e300;
  mt_best = 8;
  ne_best = 2;
  for (int ne = 2; ne >= 1; --ne)
    for (int mt = 8; mt >= 1; --mt) {
      const long tiles = (long)cdiv(T, mt * 8) * cdiv(E, 64 * ne);
      const long waves = (tiles + 147) / 148;
      const double cost = (double)waves * ((double)(mt * 8) * (64 * ne) + 8.0 * (mt * 8 + 64 * ne));
      if (cost < best - 1e-9) {
        best = cost;
        mt_best = mt;
        ne_best = ne;
      }
    }
}

template <int TPC>
static int launch_router_warp_tpc(const __nv_bfloat16* xp, const __nv_bfloat16* wp, const float* logit_bias,
                                  __nv_bfloat16* lp, int T, int H, int E, cudaStream_t st) {
  const size_t smem = (size_t)8 * H * 2 + (size_t)TPC * H * 8;
  static DynSmemCache attr;
  B200_CUDA(ensure_dyn_smem(router_logits_warp_kernel<TPC>, smem, attr));
  dim3 grid(cdiv(E, 8), cdiv(T, TPC));
  B200_CUDA(launch_pdl(router_logits_warp_kernel<TPC>, grid, dim3(256), smem, st, xp, wp, logit_bias, lp, T, H, E));
  return 0;
}
// tokens per CTA: two while that keeps the re-staging of the weight rows small, more beyond (as far as the float64
// rows fit in shared memory)
static int router_warp_tpc(int T, int H) {
  int tpc = T <= 32 ? 2 : (T <= 128 ? 4 : kWarpTokensMax);
  while (tpc > 2 && (size_t)8 * H * 2 + (size_t)tpc * H * 8 > 200 * 1024) tpc >>= 1;
  return tpc;
}
static int launch_router_warp(const __nv_bfloat16* xp, const __nv_bfloat16* wp, const float* logit_bias,
                              __nv_bfloat16* lp, int T, int H, int E, cudaStream_t st) {
  switch (router_warp_tpc(T, H)) {
    case 2: return launch_router_warp_tpc<2>(xp, wp, logit_bias, lp, T, H, E, st);
    case 4: return launch_router_warp_tpc<4>(xp, wp, logit_bias, lp, T, H, E, st);
    default: return launch_router_warp_tpc<8>(xp, wp, logit_bias, lp, T, H, E, st);
  }
}

int launch_router_logits(const void* x, const void* w, const float* logit_bias, void* logits, int T, int H, int E,
                         double* w64, cudaStream_t st) {
  auto xp = static_cast<const __nv_bfloat16*>(x);
  auto wp = static_cast<const __nv_bfloat16*>(w);
  auto lp = static_cast<__nv_bfloat16*>(logits);
#ifdef B200_DEV
  static const int force = [] {
    const char* v = getenv("B200_ROUTER_KERNEL");  // "warp" / "tile" / "dmma": development override
    return !v ? 0 : (v[0] == 'w' ? 1 : (v[0] == 't' ? 2 : 3));
  }();
#else
  constexpr int force = 0;
#endif
  const bool warp_ok = (H % 8 == 0) && ((size_t)8 * H * 2 + (size_t)2 * H * 8 <= 200 * 1024);
  const bool dmma_ok = (H % 8 == 0);
  if (dmma_ok && (force == 3 || (!force && T >= 256))) {
    int mt, ne;
    dmma_tile_shape(T, E, mt, ne);
#define B200_DMMA_CASE(MTV)                                                                  \
  case MTV:                                                                                  \
    return ne == 2 ? launch_router_dmma<MTV, 2>(xp, wp, w64, logit_bias, lp, T, H, E, st)         \
                   : launch_router_dmma<MTV, 1>(xp, wp, w64, logit_bias, lp, T, H, E, st);
    switch (mt) {
      B200_DMMA_CASE(1)
      B200_DMMA_CASE(2)
      B200_DMMA_CASE(3)
      B200_DMMA_CASE(4)
      B200_DMMA_CASE(5)
      B200_DMMA_CASE(6)
      B200_DMMA_CASE(7)
      default:
        return ne == 2 ? launch_router_dmma<8, 2>(xp, wp, w64, logit_bias, lp, T, H, E, st)
                       : launch_router_dmma<8, 1>(xp, wp, w64, logit_bias, lp, T, H, E, st);
    }
#undef B200_DMMA_CASE
  }
  const bool use_warp = force ? (force == 1 && warp_ok) : warp_ok;
  if (use_warp) return launch_router_warp(xp, wp, logit_bias, lp, T, H, E, st);
  if (T <= 256) {
    dim3 grid(cdiv(E, 16), cdiv(T, 8));
    router_logits_kernel<4, 2, 4><<<grid, 256, 0, st>>>(xp, wp, logit_bias, lp, T, H, E);
  } else {
    dim3 grid(cdiv(E, 64), cdiv(T, 64));
    router_logits_kernel<4, 16, 16><<<grid, 256, 0, st>>>(xp, wp, logit_bias, lp, T, H, E);
  }
  return 0;
}

// ---------------------------------------------------------------------------------------
// Per-token routing: one warp per token, each lane keeps E/32 (<= 8) experts.
// mode 0: p = RN_bf16(softmax_f64(logits)); top-k by (p desc, expert asc); score = p or
//         RN_bf16(p / sum of selected p).   mode 1: top-k by (logit desc, expert asc);
//         score = RN_bf16(softmax_f64 over the k selected logits).
// Selection key: order-preserving 16-bit image of the bf16 value in the high half, inverted
// expert index in the low half; k rounds of warp-wide max.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) route_topk_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int k,
                                                         int mode, int renorm, uint32_t* __restrict__ idx,
                                                         __nv_bfloat16* __restrict__ scores,
                                                         __nv_bfloat16* __restrict__ probs /*nullable [T,E]*/) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  route_topk_token<false>(logits, t, lane, E, k, mode, renorm, idx, scores, probs);
}

// ---------------------------------------------------------------------------------------
// Routing and the token -> expert sort in one launch, for T*k <= 1024 assignments: a warp per token
// for the top-k, then every CTA publishes its indices (fence) and takes a ticket; the CTA that draws
// the last one runs the single-chunk permutation.  Nobody waits; the ticket word is reset by the
// last CTA for the next launch.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) route_topk_sort_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int k,
                                                              int mode, int renorm, uint32_t* idx, __nv_bfloat16* scores,
                                                              uint32_t* __restrict__ perm, uint32_t* __restrict__ inv,
                                                              uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                                                              uint32_t* __restrict__ active, uint32_t* __restrict__ n_active,
                                                              unsigned int* ticket, int* __restrict__ err) {
  extern __shared__ int topk_sort_sh[];  // the permutation's tables
  __shared__ unsigned int s_ticket;
  pdl_prologue();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = blockIdx.x * 8 + warp;
  if (t < T) route_topk_token<false>(logits, t, lane, E, k, mode, renorm, idx, scores, nullptr);
  __threadfence();
  __syncthreads();
  if (tid == 0) s_ticket = atomicAdd(ticket, 1u);
  __syncthreads();
  if (s_ticket != gridDim.x - 1) return;
  __threadfence();
  if (tid == 0) *ticket = 0u;
  permute_small_block<256>(idx, T * k, E, perm, inv, counts, offsets, active, n_active, err, topk_sort_sh);
}

bool route_topk_sort_ok(int T, int E, int k) { return (int64_t)T * k <= kChunk && E <= kMaxPerLane * 32; }

int launch_route_topk_sort(const void* logits, int T, int E, int k, int mode, int renorm, uint32_t* idx, void* scores,
                           uint32_t* perm, uint32_t* inv, uint32_t* counts, uint32_t* offsets, uint32_t* active,
                           uint32_t* n_active, unsigned int* ticket, int* err, cudaStream_t st) {
  if (T == 0) return 0;
  const size_t smem = sizeof(int) * 33 * E;
  static DynSmemCache attr;
  B200_CUDA(ensure_dyn_smem(route_topk_sort_kernel, smem, attr));
  B200_CUDA(launch_pdl(route_topk_sort_kernel, dim3(cdiv(T, 8)), dim3(256), smem, st, static_cast<const __nv_bfloat16*>(logits), T,
                       E, k, mode, renorm, idx, static_cast<__nv_bfloat16*>(scores), perm, inv, counts, offsets, active, n_active,
                       ticket, err));
  return 0;
}

// ---------------------------------------------------------------------------------------
// Small batches (T*k <= 1024): logits, routing and the token -> expert sort in ONE launch.
// Every CTA computes its logits like router_logits_warp_kernel, publishes them (fence) and takes a
// ticket; the CTA that draws the last ticket knows that all logits are in memory and finishes the
// job alone: a warp per token for the top-k, then the single-chunk permutation.  Nobody waits:
// the other CTAs simply exit.  The ticket word is reset by the last CTA for the next launch.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) router_fused_small_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const float* __restrict__ logit_bias,
    __nv_bfloat16* logits, int T, int H, int E, int k, int mode, int renorm, uint32_t* idx, __nv_bfloat16* scores,
    uint32_t* __restrict__ perm, uint32_t* __restrict__ inv, uint32_t* __restrict__ counts,
    uint32_t* __restrict__ offsets, uint32_t* __restrict__ active, uint32_t* __restrict__ n_active,
    unsigned int* ticket, int* __restrict__ err, uint32_t* __restrict__ desc, int desc_entries) {
  extern __shared__ __align__(16) unsigned char rsm[];  // token and weight rows (bf16), later the permutation's tables
  __shared__ unsigned int s_ticket;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.y * kWarpTokens, nvec = H / 8;
  {
    uint4* xs4 = reinterpret_cast<uint4*>(rsm);
    uint4* ws4 = xs4 + (size_t)kWarpTokens * nvec;
    pdl_trigger();
    stage_router_weights(ws4, w, blockIdx.x * 8, E, H, tid);  // constants: on their way before the wait
    pdl_wait();
    stage_router_tokens(xs4, x, t0, kWarpTokens, T, H, tid);
    cp_async_wait_all();
    __syncthreads();
    warp_expert_logits(xs4, ws4 + (size_t)warp * nvec, nvec, lane, t0, T, blockIdx.x * 8 + warp, E, logit_bias, logits);
  }
  // publish, then take a ticket
  __threadfence();
  __syncthreads();
  if (tid == 0) s_ticket = atomicAdd(ticket, 1u);
  __syncthreads();
  if (s_ticket != gridDim.x * gridDim.y - 1) return;
  __threadfence();
  if (tid == 0) *ticket = 0u;
  for (int t = warp; t < T; t += 8) route_topk_token<true>(logits, t, lane, E, k, mode, renorm, idx, scores, nullptr);
  __syncthreads();  // idx written by this block is read back below
  permute_small_block<256>(idx, T * k, E, perm, inv, counts, offsets, active, n_active, err,
                           reinterpret_cast<int*>(rsm));
  if (desc) {
    // per active expert one record {expert, first sorted position, rows, 0, token of the first eight rows, ...}: the
    // grouped products' CTAs then start with one load instead of the chain n_active -> active -> offsets -> perm
    __syncthreads();  // perm, offsets and active of this block are in memory
    const int na = (int)*n_active;
    for (int i = tid; i < desc_entries * kExpertDescWords; i += 256) {
      const int ea = i / kExpertDescWords, wd = i % kExpertDescWords;
      uint32_t v = 0;
      if (ea < na) {
        const uint32_t e = active[ea], seg0 = offsets[e], m = offsets[e + 1] - seg0;
        if (wd == 0) v = e;
        if (wd == 1) v = seg0;
        if (wd == 2) v = m;
        if (wd >= 4 && wd < 12 && (uint32_t)(wd - 4) < m) v = perm[seg0 + (uint32_t)(wd - 4)] / (uint32_t)k;
        if (wd >= 12 && wd < 20) v = 0x3f800000u;  // (row scales are computed by the CTAs that prepare the rows)
      }
      desc[i] = v;
    }
  }
}

bool router_fused_small_ok(int T, int H, int E, int k) {
  return T <= 8 && (int64_t)T * k <= kChunk && H % 8 == 0 && (size_t)(kWarpTokens + 8) * H * 2 <= 200 * 1024 &&
         E <= kMaxPerLane * 32;
}

int launch_router_fused_small(const void* x, const void* w, const float* logit_bias, void* logits, int T, int H, int E,
                              int k, int mode, int renorm, uint32_t* idx, void* scores, uint32_t* perm, uint32_t* inv,
                              uint32_t* counts, uint32_t* offsets, uint32_t* active, uint32_t* n_active,
                              unsigned int* ticket, int* err, uint32_t* desc, int desc_entries, cudaStream_t st) {
  auto xp = static_cast<const __nv_bfloat16*>(x);
  auto wp = static_cast<const __nv_bfloat16*>(w);
  auto lp = static_cast<__nv_bfloat16*>(logits);
  auto sp = static_cast<__nv_bfloat16*>(scores);
  size_t smem = (size_t)(kWarpTokens + 8) * H * 2;
  const size_t need = sizeof(int) * 33 * E;
  if (smem < need) smem = need;
  static DynSmemCache attr;
  B200_CUDA(ensure_dyn_smem(router_fused_small_kernel, smem, attr));
  dim3 grid(cdiv(E, 8), cdiv(T, kWarpTokens));
  B200_CUDA(launch_pdl(router_fused_small_kernel, grid, dim3(256), smem, st, xp, wp, logit_bias, lp, T, H, E, k, mode, renorm, idx,
                       sp, perm, inv, counts, offsets, active, n_active, ticket, err, desc, desc_entries));
  return 0;
}

int launch_route_topk(const void* logits, int T, int E, int k, int mode, int renorm, uint32_t* idx, void* scores,
                      void* probs, cudaStream_t st) {
  if (T == 0) return 0;
  B200_CUDA(launch_pdl(route_topk_kernel, dim3(cdiv(T, 4)), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(logits), T, E, k,
                       mode, renorm, idx, static_cast<__nv_bfloat16*>(scores), static_cast<__nv_bfloat16*>(probs)));
  return 0;
}

// ---------------------------------------------------------------------------------------
// argpartition_axis(a, kth, axis=-1) over bf16 rows: the first kth+1 output columns are the
// kth+1 smallest elements in (value ascending, index ascending) order, the remaining columns
// are the other indices in ascending index order (the reference leaves the order inside a
// partition undefined).  One warp per row, cols <= 256.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) argpartition_kernel(const __nv_bfloat16* __restrict__ a, int rows, int cols,
                                                           int kth, uint32_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const unsigned short* row = reinterpret_cast<const unsigned short*>(a) + (size_t)r * cols;
  uint32_t keys[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    int e = lane + 32 * i;
    // smallest value first, smallest index first -> maximise (inverted value, inverted index)
    keys[i] = (e < cols) ? (((0xffffu - order_key(row[e])) << 16) | (0xffffu - (uint32_t)e)) : 0u;
  }
  for (int j = 0; j <= kth; ++j) {
    uint32_t best = keys[0];
#pragma unroll
    for (int i = 1; i < kMaxPerLane; ++i) best = max(best, keys[i]);
    best = __reduce_max_sync(0xffffffffu, best);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (keys[i] == best) keys[i] = 0u;
    if (lane == 0) out[(size_t)r * cols + j] = 0xffffu - (best & 0xffffu);
  }
  // remaining indices in ascending order: warp-wide compaction
  int base = kth + 1;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    int e = lane + 32 * i;
    bool left = (e < cols) && keys[i] != 0u;
    uint32_t m = __ballot_sync(0xffffffffu, left);
    if (left) out[(size_t)r * cols + base + __popc(m & ((1u << lane) - 1u))] = (uint32_t)e;
    base += __popc(m);
  }
}

// topk_axis(a, k, -1) over bf16 rows (mlx-rs/src/ops/indexing/mod.rs:674-700): the k largest values of a row, written
// in ascending order.  One warp per row, cols <= 256: k rounds of a warp-wide max over (value, inverted index) keys.
__global__ void __launch_bounds__(128) topk_values_kernel(const __nv_bfloat16* __restrict__ a, int rows, int cols, int k,
                                                          __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const unsigned short* row = reinterpret_cast<const unsigned short*>(a) + (size_t)r * cols;
  uint32_t keys[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    keys[i] = (e < cols) ? ((order_key(row[e]) << 16) | (0xffffu - (uint32_t)e)) : 0u;
  }
  for (int j = 0; j < k; ++j) {
    uint32_t best = keys[0];
#pragma unroll
    for (int i = 1; i < kMaxPerLane; ++i) best = max(best, keys[i]);
    best = __reduce_max_sync(0xffffffffu, best);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (keys[i] == best) keys[i] = 0u;
    if (lane == 0) out[(size_t)r * k + (k - 1 - j)] = __ushort_as_bfloat16((unsigned short)key_to_bits(best >> 16));
  }
}

int launch_topk_values(const void* a, int rows, int cols, int k, void* out, cudaStream_t st) {
  if (rows == 0) return 0;
  topk_values_kernel<<<cdiv(rows, 4), 128, 0, st>>>(static_cast<const __nv_bfloat16*>(a), rows, cols, k,
                                                    static_cast<__nv_bfloat16*>(out));
  return 0;
}

int launch_argpartition(const void* a, int rows, int cols, int kth, uint32_t* out, cudaStream_t st) {
  if (rows == 0) return 0;
  argpartition_kernel<<<cdiv(rows, 4), 128, 0, st>>>(static_cast<const __nv_bfloat16*>(a), rows, cols, kth, out);
  return 0;
}

// softmax_axis(-1, precise) over bf16 rows (cols <= 256): exact softmax, correctly rounded.
__global__ void __launch_bounds__(128) softmax_kernel(const __nv_bfloat16* __restrict__ a, int rows, int cols,
                                                      __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const unsigned short* row = reinterpret_cast<const unsigned short*>(a) + (size_t)r * cols;
  float lf[kMaxPerLane];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    int e = lane + 32 * i;
    lf[i] = (e < cols) ? bf16_bits_to_f32(row[e]) : -INFINITY;
    m = fmaxf(m, lf[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  double ex[kMaxPerLane], s = 0.0;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    ex[i] = (lane + 32 * i < cols) ? exp((double)lf[i] - (double)m) : 0.0;
    s += ex[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    int e = lane + 32 * i;
    if (e < cols) out[(size_t)r * cols + e] = __ushort_as_bfloat16((unsigned short)f64_to_bf16_bits(ex[i] / s));
  }
}

int launch_softmax(const void* a, int rows, int cols, void* out, cudaStream_t st) {
  if (rows == 0) return 0;
  softmax_kernel<<<cdiv(rows, 4), 128, 0, st>>>(static_cast<const __nv_bfloat16*>(a), rows, cols,
                                                static_cast<__nv_bfloat16*>(out));
  return 0;
}

// take_along_axis(a, idx, axis=-1) for 2-byte elements.  Out-of-range indices set *err = 1.
__global__ void take_along_kernel(const unsigned short* __restrict__ a, int rows, int cols,
                                  const uint32_t* __restrict__ idx, int icol, unsigned short* __restrict__ out,
                                  int* __restrict__ err) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * icol) return;
  size_t r = i / icol;
  uint32_t j = idx[i];
  if (j >= (uint32_t)cols) {
    *err = 1;
    out[i] = 0;
    return;
  }
  out[i] = a[r * cols + j];
}

int launch_take_along(const void* a, int rows, int cols, const uint32_t* idx, int icol, void* out, int* err,
                      cudaStream_t st) {
  size_t n = (size_t)rows * icol;
  if (n == 0) return 0;
  take_along_kernel<<<cdiv(n, 256), 256, 0, st>>>(static_cast<const unsigned short*>(a), rows, cols, idx, icol,
                                                  static_cast<unsigned short*>(out), err);
  return 0;
}

}  // namespace b200

// Memory-bound helpers of the quantized path: affine quantize / dequantize, the k-way
// combine, residual-add + RMSNorm, and small index utilities.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

// ---------------------------------------------------------------------------------------
// quantize (mlx-rs/src/ops/quantization.rs:48-83, mode "affine"): one thread per group.
// The group extreme with the larger magnitude is made exactly representable, the scale takes
// its sign from which extreme that is, the bias is that extreme (or 0 when it rounds to code
// 0); codes use the unrounded float32 scale and bias; element i of a word sits in bits
// [bits*i, bits*i+bits).  Every operation is a single IEEE float32 operation so that the
// result is reproducible bit for bit on any conforming implementation.
// ---------------------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(128) quantize_kernel(const void* __restrict__ w, int64_t n_groups, int gs, int bits,
                                                       uint32_t* __restrict__ wq, void* __restrict__ scales,
                                                       void* __restrict__ biases) {
  int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gi >= n_groups) return;
  const float n_bins = (float)((1 << bits) - 1);
  const int epw = 32 / bits;
  auto ld = [&](int i) -> float {
    if constexpr (BF16)
      return bf16_bits_to_f32(static_cast<const unsigned short*>(w)[gi * gs + i]);
    else
      return static_cast<const float*>(w)[gi * gs + i];
  };
  float wmin = ld(0), wmax = wmin;
  for (int i = 1; i < gs; ++i) {
    float v = ld(i);
    wmin = fminf(wmin, v);
    wmax = fmaxf(wmax, v);
  }
  float scale = fmaxf(__fdiv_rn(__fsub_rn(wmax, wmin), n_bins), 1e-7f);
  const bool side = fabsf(wmin) > fabsf(wmax);
  scale = side ? scale : -scale;
  const float edge = side ? wmin : wmax;
  const float q0 = roundf(__fdiv_rn(edge, scale));
  const bool at_zero = (q0 == 0.0f);
  scale = at_zero ? scale : __fdiv_rn(edge, q0);
  const float bias = at_zero ? 0.0f : edge;
  if constexpr (BF16) {
    static_cast<__nv_bfloat16*>(scales)[gi] = __float2bfloat16_rn(scale);
    static_cast<__nv_bfloat16*>(biases)[gi] = __float2bfloat16_rn(bias);
  } else {
    static_cast<float*>(scales)[gi] = scale;
    static_cast<float*>(biases)[gi] = bias;
  }
  for (int i = 0; i < gs; i += epw) {
    uint32_t word = 0;
    for (int j = 0; j < epw; ++j) {
      float q = roundf(__fdiv_rn(__fsub_rn(ld(i + j), bias), scale));
      q = fminf(fmaxf(q, 0.0f), n_bins);
      word |= (uint32_t)q << (bits * j);
    }
    wq[(gi * gs + i) / epw] = word;
  }
}

int launch_quantize(const void* w, int is_bf16, int64_t rows, int64_t K, int gs, int bits, uint32_t* wq, void* scales,
                    void* biases, cudaStream_t st) {
  int64_t ng = rows * (K / gs);
  if (ng == 0) return 0;
  if (is_bf16)
    quantize_kernel<true><<<cdiv(ng, 128), 128, 0, st>>>(w, ng, gs, bits, wq, scales, biases);
  else
    quantize_kernel<false><<<cdiv(ng, 128), 128, 0, st>>>(w, ng, gs, bits, wq, scales, biases);
  return 0;
}

// dequantize (mlx-rs/src/ops/quantization.rs:129-158): w_hat = scale*q + bias, one float32
// multiply then one float32 add, stored in the dtype of the scales.  One thread per word.
template <bool BF16>
__global__ void dequantize_kernel(const uint32_t* __restrict__ wq, const void* __restrict__ scales,
                                  const void* __restrict__ biases, int64_t n_words, int gs, int bits,
                                  void* __restrict__ out) {
  int64_t wi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (wi >= n_words) return;
  const int epw = 32 / bits;
  const uint32_t mask = (1u << bits) - 1u;
  const uint32_t word = wq[wi];
  const int64_t gi = wi * epw / gs;
  float s, b;
  if constexpr (BF16) {
    s = bf16_bits_to_f32(static_cast<const unsigned short*>(scales)[gi]);
    b = bf16_bits_to_f32(static_cast<const unsigned short*>(biases)[gi]);
  } else {
    s = static_cast<const float*>(scales)[gi];
    b = static_cast<const float*>(biases)[gi];
  }
  for (int j = 0; j < epw; ++j) {
    float v = __fadd_rn(__fmul_rn(s, (float)((word >> (bits * j)) & mask)), b);
    if constexpr (BF16)
      static_cast<__nv_bfloat16*>(out)[wi * epw + j] = __float2bfloat16_rn(v);
    else
      static_cast<float*>(out)[wi * epw + j] = v;
  }
}

int launch_dequantize(const uint32_t* wq, const void* scales, const void* biases, int is_bf16, int64_t rows, int64_t K,
                      int gs, int bits, void* out, cudaStream_t st) {
  int64_t nw = rows * (K * bits / 32);
  if (nw == 0) return 0;
  if (is_bf16)
    dequantize_kernel<true><<<cdiv(nw, 256), 256, 0, st>>>(wq, scales, biases, nw, gs, bits, out);
  else
    dequantize_kernel<false><<<cdiv(nw, 256), 256, 0, st>>>(wq, scales, biases, nw, gs, bits, out);
  return 0;
}

// combine: out[t, c] = bf16( sum_j yk[t, j, c] ), j ascending, float32 throughout (sum_axis(-2),
// mlx-rs/src/ops/reduction.rs:260-275; the routing weights were applied by the producer, whose
// float32 results are summed here without an intermediate rounding).
__global__ void combine_kernel(const float4* __restrict__ yk, int64_t T, int k, int64_t H4, uint2* __restrict__ out,
                               float4* __restrict__ out_f32) {
  pdl_prologue();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * H4) return;
  const int64_t t = i / H4, c = i % H4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < k; ++j) {
    const float4 v = __ldg(&yk[(t * k + j) * H4 + c]);
    acc.x += v.x;
    acc.y += v.y;
    acc.z += v.z;
    acc.w += v.w;
  }
  uint2 o;
  o.x = f32_to_bf16_bits(acc.x) | (f32_to_bf16_bits(acc.y) << 16);
  o.y = f32_to_bf16_bits(acc.z) | (f32_to_bf16_bits(acc.w) << 16);
  out[i] = o;
  if (out_f32) out_f32[i] = acc;  // the sum before its rounding to bf16
}

// Same sum over 16-bit inputs: bf16 rows, or the fp16 rows the tensor-core down projection stores
// (half the traffic of float32 rows; fp16's 11 significant bits keep the k-way sum an order of
// magnitude inside the output tolerance, bf16's 8 would not).
template <bool F16>
__global__ void combine_16_kernel(const uint2* __restrict__ yk, int64_t T, int k, int64_t H4, uint2* __restrict__ out,
                                  float4* __restrict__ out_f32) {
  pdl_prologue();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * H4) return;
  const int64_t t = i / H4, c = i % H4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < k; ++j) {
    const uint2 v = __ldg(&yk[(t * k + j) * H4 + c]);
    if constexpr (F16) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
      acc.x += a.x;
      acc.y += a.y;
      acc.z += b.x;
      acc.w += b.y;
    } else {
      acc.x += __uint_as_float(v.x << 16);
      acc.y += __uint_as_float(v.x & 0xffff0000u);
      acc.z += __uint_as_float(v.y << 16);
      acc.w += __uint_as_float(v.y & 0xffff0000u);
    }
  }
  uint2 o;
  o.x = f32_to_bf16_bits(acc.x) | (f32_to_bf16_bits(acc.y) << 16);
  o.y = f32_to_bf16_bits(acc.z) | (f32_to_bf16_bits(acc.w) << 16);
  out[i] = o;
  if (out_f32) out_f32[i] = acc;
}

int launch_combine(const void* yk, int yk_fmt, int64_t T, int k, int64_t H, void* out, void* out_f32, cudaStream_t st) {
  if (T == 0) return 0;
  B200_REQUIRE(H % 4 == 0, "hidden size must be a multiple of 4");
  const int64_t n4 = T * (H / 4);
  if (yk_fmt == kOutF16)
    B200_CUDA(launch_pdl(combine_16_kernel<true>, dim3(cdiv(n4, 256)), dim3(256), 0, st, static_cast<const uint2*>(yk), T, k,
                         H / 4, static_cast<uint2*>(out), static_cast<float4*>(out_f32)));
  else if (yk_fmt == kOutBf16)
    B200_CUDA(launch_pdl(combine_16_kernel<false>, dim3(cdiv(n4, 256)), dim3(256), 0, st, static_cast<const uint2*>(yk), T, k,
                         H / 4, static_cast<uint2*>(out), static_cast<float4*>(out_f32)));
  else
    B200_CUDA(launch_pdl(combine_kernel, dim3(cdiv(n4, 256)), dim3(256), 0, st, static_cast<const float4*>(yk), T, k, H / 4,
                         static_cast<uint2*>(out), static_cast<float4*>(out_f32)));
  return 0;
}

// take_axis(x, indices / div, axis=0) for rows of 2-byte elements (mlx-rs/src/ops/indexing/mod.rs:374-401
// composed with floor_divide, mlx-rs/src/ops/arithmetic.rs:401): out[p, :] = x[indices[p] / div, :].
__global__ void take_rows_kernel(const uint4* __restrict__ x, const uint32_t* __restrict__ indices, uint32_t div,
                                 int64_t n_rows, int64_t x_rows, int vec_per_row, uint4* __restrict__ out,
                                 int* __restrict__ err) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * vec_per_row) return;
  const int64_t r = i / vec_per_row;
  const int c = (int)(i % vec_per_row);
  const uint32_t src = indices[r] / div;
  if (src >= x_rows) {
    *err = 1;
    out[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  out[i] = __ldg(x + (size_t)src * vec_per_row + c);
}

int launch_take_rows(const void* x, const uint32_t* indices, uint32_t div, int64_t n_rows, int64_t x_rows, int64_t cols,
                     void* out, int* err, cudaStream_t st) {
  if (n_rows == 0) return 0;
  int64_t n = n_rows * (cols / 8);
  take_rows_kernel<<<cdiv(n, 256), 256, 0, st>>>(static_cast<const uint4*>(x), indices, div, n_rows, x_rows,
                                                 (int)(cols / 8), static_cast<uint4*>(out), err);
  return 0;
}

// Weighted un-sort + combine for expert outputs that arrive as bf16 rows in sorted order
// (expert-parallel return path): out[t, :] = bf16( sum_j score[t, j] * y[inv[t*k + j], :] ),
// float32 accumulation, j ascending (take with the inverse order, multiply, sum_axis(-2)).
__global__ void gather_combine_kernel(const uint2* __restrict__ y, const uint32_t* __restrict__ inv,
                                      const unsigned short* __restrict__ scores, int64_t T, int k, int64_t H4,
                                      uint2* __restrict__ out, float4* __restrict__ out_f32) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * H4) return;
  const int64_t t = i / H4, c = i % H4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < k; ++j) {
    const float s = bf16_bits_to_f32(scores[t * k + j]);
    const uint2 v = __ldg(&y[(size_t)inv[t * k + j] * H4 + c]);
    acc.x += s * __uint_as_float(v.x << 16);
    acc.y += s * __uint_as_float(v.x & 0xffff0000u);
    acc.z += s * __uint_as_float(v.y << 16);
    acc.w += s * __uint_as_float(v.y & 0xffff0000u);
  }
  uint2 o;
  o.x = f32_to_bf16_bits(acc.x) | (f32_to_bf16_bits(acc.y) << 16);
  o.y = f32_to_bf16_bits(acc.z) | (f32_to_bf16_bits(acc.w) << 16);
  out[i] = o;
  if (out_f32) out_f32[i] = acc;
}

int launch_gather_combine(const void* y, const uint32_t* inv, const void* scores, int64_t T, int k, int64_t H, void* out,
                          void* out_f32, cudaStream_t st) {
  if (T == 0) return 0;
  int64_t n = T * (H / 4);
  gather_combine_kernel<<<cdiv(n, 256), 256, 0, st>>>(static_cast<const uint2*>(y), inv,
                                                      static_cast<const unsigned short*>(scores), T, k, H / 4,
                                                      static_cast<uint2*>(out), static_cast<float4*>(out_f32));
  return 0;
}

// Residual add + RMSNorm (fast::rms_norm, mlx-rs/src/fast.rs:178-205; residual wiring as in
// mlx-lm/src/models/qwen3.rs:310-325).  s = bf16(x + residual) is written to sum_out (when
// given) and the norm is taken over that rounded sum: out = w * s * rsqrt(mean(s^2) + eps).
__global__ void __launch_bounds__(256) rms_norm_kernel(const __nv_bfloat16* __restrict__ x,
                                                       const __nv_bfloat16* __restrict__ residual,
                                                       const __nv_bfloat16* __restrict__ weight, float eps, int64_t cols,
                                                       __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ sum_out) {
  pdl_prologue();
  const int64_t r = blockIdx.x;
  __shared__ float part[8];
  block_rms_norm_row(x + r * cols, residual ? residual + r * cols : nullptr, weight, eps, cols, out + r * cols,
                     (residual && sum_out) ? sum_out + r * cols : nullptr, part);
}

int launch_rms_norm(const void* x, const void* residual, const void* weight, float eps, int64_t rows, int64_t cols,
                    void* out, void* sum_out, cudaStream_t st) {
  if (rows == 0) return 0;
  B200_CUDA(launch_pdl(rms_norm_kernel, dim3((unsigned)rows), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x),
                       static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(weight), eps, cols,
                       static_cast<__nv_bfloat16*>(out), static_cast<__nv_bfloat16*>(sum_out)));
  return 0;
}

__global__ void add_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, int64_t n, __nv_bfloat16* out) {
  pdl_prologue();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(__bfloat162float(a[i]) + __bfloat162float(b[i]));
}
int launch_add(const void* a, const void* b, int64_t n, void* out, cudaStream_t st) {
  if (n == 0) return 0;
  B200_CUDA(launch_pdl(add_kernel, dim3(cdiv(n, 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(a),
                       static_cast<const __nv_bfloat16*>(b), n, static_cast<__nv_bfloat16*>(out)));
  return 0;
}

// General form of quantized_matmul / gather_qmm (mlx-rs/src/ops/quantization.rs:88-122, 160-230) on CUDA cores:
// any activation dtype (float32, bfloat16, float16; scales, biases and the result share it), group sizes 32 / 64 /
// 128, bits 2 / 4 / 8, both orientations of w, optional index arrays.
//   transpose != 0: w [E, N, K*bits/32] quantised along K, out[i] = x[lhs[i]] . w_hat[rhs[i]]^T
//   transpose == 0: w [E, K, N*bits/32] quantised along N, out[i] = x[lhs[i]] . w_hat[rhs[i]]
// float32 arithmetic throughout (the dequantised weight is one multiply and one add, the dot product a chain of
// fused multiply-adds in k order), so float32 callers get float32-accurate results; it is the reference
// tests' configuration (float32 arrays, `:319-342`, `:346-423`) and the fallback for shapes the fast kernels do
// not take.  One thread per output element.
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) gather_qmm_generic_kernel(const T* __restrict__ x, const uint32_t* __restrict__ wq,
                                                                 const T* __restrict__ scales, const T* __restrict__ biases,
                                                                 const uint32_t* __restrict__ lhs, const uint32_t* __restrict__ rhs,
                                                                 int64_t Bx, int64_t M, int64_t K, int64_t E, int64_t N,
                                                                 int64_t n_idx, int transpose, int gs, int bits,
                                                                 T* __restrict__ out, int* __restrict__ err) {
  const int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n_idx * M * N) return;
  const int64_t n = o % N, m = (o / N) % M, i = o / (N * M);
  uint32_t bx = lhs ? lhs[i] : (uint32_t)i, e = rhs ? rhs[i] : 0u;
  if ((int64_t)bx >= Bx || (int64_t)e >= E) {  // reported through the status word; the access is redirected, never out of bounds
    *err = (int64_t)e >= E ? 2 : 1;
    bx = 0;
    e = 0;
  }
  const int epw = 32 / bits;
  const uint32_t mask = (1u << bits) - 1u;
  const T* xr = x + ((int64_t)bx * M + m) * K;
  float acc = 0.f;
  if (transpose) {
    const int64_t Wp = K / epw, G = K / gs;
    const uint32_t* wr = wq + ((int64_t)e * N + n) * Wp;
    const T* sr = scales + ((int64_t)e * N + n) * G;
    const T* br = biases + ((int64_t)e * N + n) * G;
    for (int64_t g = 0; g < G; ++g) {
      const float s = to_f32(sr[g]), b = to_f32(br[g]);
      for (int kk = 0; kk < gs; kk += epw) {
        const uint32_t word = wr[(g * gs + kk) / epw];
        for (int j = 0; j < epw; ++j) {
          const float wv = __fadd_rn(__fmul_rn(s, (float)((word >> (bits * j)) & mask)), b);
          acc = fmaf(to_f32(xr[g * gs + kk + j]), wv, acc);
        }
      }
    }
  } else {
    const int64_t Wp = N / epw, G = N / gs;
    const uint32_t* we = wq + (int64_t)e * K * Wp;
    const T* se = scales + (int64_t)e * K * G;
    const T* be = biases + (int64_t)e * K * G;
    for (int64_t k = 0; k < K; ++k) {
      const uint32_t q = (we[k * Wp + n / epw] >> (bits * (n % epw))) & mask;
      const float wv = __fadd_rn(__fmul_rn(to_f32(se[k * G + n / gs]), (float)q), to_f32(be[k * G + n / gs]));
      acc = fmaf(to_f32(xr[k]), wv, acc);
    }
  }
  out[o] = from_f32<T>(acc);
}

int launch_gather_qmm_generic(const void* x, const uint32_t* wq, const void* scales, const void* biases, const uint32_t* lhs,
                              const uint32_t* rhs, int dtype, int64_t Bx, int64_t M, int64_t K, int64_t E, int64_t N,
                              int64_t n_idx, int transpose, int gs, int bits, void* out, int* err, cudaStream_t st) {
  const int64_t total = n_idx * M * N;
  if (total == 0) return 0;
  const dim3 grid(cdiv(total, 256)), block(256);
  if (dtype == 0)
    gather_qmm_generic_kernel<float><<<grid, block, 0, st>>>(
        static_cast<const float*>(x), wq, static_cast<const float*>(scales), static_cast<const float*>(biases), lhs, rhs, Bx, M, K,
        E, N, n_idx, transpose, gs, bits, static_cast<float*>(out), err);
  else if (dtype == 1)
    gather_qmm_generic_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), wq, static_cast<const __nv_bfloat16*>(scales),
        static_cast<const __nv_bfloat16*>(biases), lhs, rhs, Bx, M, K, E, N, n_idx, transpose, gs, bits,
        static_cast<__nv_bfloat16*>(out), err);
  else
    gather_qmm_generic_kernel<__half><<<grid, block, 0, st>>>(
        static_cast<const __half*>(x), wq, static_cast<const __half*>(scales), static_cast<const __half*>(biases), lhs, rhs, Bx, M,
        K, E, N, n_idx, transpose, gs, bits, static_cast<__half*>(out), err);
  return 0;
}

// One segment holding every row (dense quantized Linear as the E = 1 case of the grouped kernel).
__global__ void dense_segments_kernel(uint32_t* counts, uint32_t* offsets, uint32_t* active, uint32_t* n_active, uint32_t rows) {
  counts[0] = rows;
  offsets[0] = 0;
  offsets[1] = rows;
  active[0] = 0;
  *n_active = rows ? 1u : 0u;
}
int launch_dense_segments(uint32_t* counts, uint32_t* offsets, uint32_t* active, uint32_t* n_active, uint32_t rows,
                          cudaStream_t st) {
  dense_segments_kernel<<<1, 1, 0, st>>>(counts, offsets, active, n_active, rows);
  return 0;
}

// gather_mm(a, b, lhs_indices, rhs_indices) (mlx-rs/src/ops/arithmetic.rs:1568-1632), un-quantised:
// out[i] = a[lhs[i]] @ b[rhs[i]] with a bf16 [Ba, M, K], b bf16 [Bb, K, N] (row-major, not transposed),
// float32 accumulation, bf16 output.  The routed block never takes this path (its experts are
// quantised); it completes the op surface for callers that keep some SwitchLinear layers in bf16.
// One CTA = one batch entry x 128 output columns x up to 8 rows of a (staged in shared memory);
// a thread owns one output column, so every load of b is a coalesced row segment read once.
constexpr int kGmmRows = 8, kGmmKc = 512;
__global__ void __launch_bounds__(128) gather_mm_kernel(const __nv_bfloat16* __restrict__ a,
                                                        const __nv_bfloat16* __restrict__ b,
                                                        const uint32_t* __restrict__ lhs, const uint32_t* __restrict__ rhs,
                                                        int64_t Ba, int64_t Bb, int M, int K, int N,
                                                        __nv_bfloat16* __restrict__ out, int* __restrict__ err) {
  __shared__ float as[kGmmRows][kGmmKc];
  const int64_t i = blockIdx.y;
  const uint32_t la = lhs ? lhs[i] : (uint32_t)i, rb = rhs ? rhs[i] : (uint32_t)i;
  if (la >= Ba || rb >= Bb) {
    if (threadIdx.x == 0) *err = 1;
    return;
  }
  const int n = blockIdx.x * 128 + threadIdx.x;
  const __nv_bfloat16* arow = a + (size_t)la * M * K;
  const __nv_bfloat16* bmat = b + (size_t)rb * K * N;
  for (int m0 = 0; m0 < M; m0 += kGmmRows) {
    const int mr = min(kGmmRows, M - m0);
    float acc[kGmmRows];
#pragma unroll
    for (int r = 0; r < kGmmRows; ++r) acc[r] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kGmmKc) {
      const int kc = min(kGmmKc, K - k0);
      __syncthreads();
      for (int t = threadIdx.x; t < mr * kc; t += 128) {
        const int r = t / kc, kk = t % kc;
        as[r][kk] = __bfloat162float(arow[(size_t)(m0 + r) * K + k0 + kk]);
      }
      __syncthreads();
      if (n < N) {
        for (int kk = 0; kk < kc; ++kk) {
          const float bv = __bfloat162float(bmat[(size_t)(k0 + kk) * N + n]);
#pragma unroll
          for (int r = 0; r < kGmmRows; ++r)
            if (r < mr) acc[r] = fmaf(as[r][kk], bv, acc[r]);
        }
      }
    }
    if (n < N)
      for (int r = 0; r < mr; ++r) out[((size_t)i * M + m0 + r) * N + n] = __float2bfloat16_rn(acc[r]);
  }
}

int launch_gather_mm(const void* a, const void* b, const uint32_t* lhs, const uint32_t* rhs, int64_t Ba, int64_t Bb,
                     int64_t M, int64_t K, int64_t N, int64_t n_idx, void* out, int* err, cudaStream_t st) {
  if (n_idx == 0 || M == 0 || N == 0) return 0;
  B200_REQUIRE(n_idx < 65536, "at most 65535 index entries per call");
  dim3 grid(cdiv(N, 128), (unsigned)n_idx);
  gather_mm_kernel<<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), lhs, rhs,
                                         Ba, Bb, (int)M, (int)K, (int)N, static_cast<__nv_bfloat16*>(out), err);
  return 0;
}

// gather_qmm with M rows per batch entry: assignment i*M + m uses expert rhs[i] and source
// row lhs[i]*M + m (lhs == null: i*M + m).  A batch index >= Bx sets *err = 1 and reads batch entry 0
// instead (the access is skipped, never out of bounds); expert indices are checked by the sort.
__global__ void expand_indices_kernel(const uint32_t* __restrict__ lhs, const uint32_t* __restrict__ rhs, int64_t n_idx,
                                      int M, int64_t Bx, uint32_t* __restrict__ flat_expert,
                                      uint32_t* __restrict__ flat_src, int* __restrict__ err) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_idx * M) return;
  int64_t b = i / M, m = i % M;
  flat_expert[i] = rhs ? rhs[b] : (uint32_t)b;
  uint32_t src = lhs ? lhs[b] : (uint32_t)b;
  if ((int64_t)src >= Bx) {
    *err = 1;
    src = 0;
  }
  flat_src[i] = src * (uint32_t)M + (uint32_t)m;
}
// out[p, :] = x[src_map[perm[p]], :] for rows of 2-byte elements (16-byte vectors): the rows of a gathered product
// in the order of its sort.  Only the first *n_valid sorted positions exist (assignments whose matrix index was out
// of range are left out of the sort and perm holds nothing for the tail).
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const uint32_t* __restrict__ perm,
                                   const uint32_t* __restrict__ src_map, int64_t n_rows,
                                   const uint32_t* __restrict__ n_valid, int vec_per_row, uint4* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * vec_per_row) return;
  const int64_t r = i / vec_per_row;
  if (r >= (int64_t)*n_valid) return;
  const uint32_t a = perm[r];
  if ((int64_t)a >= n_rows) return;
  out[i] = __ldg(x + (size_t)src_map[a] * vec_per_row + (i % vec_per_row));
}
int launch_gather_rows(const void* x, const uint32_t* perm, const uint32_t* src_map, int64_t n_rows, const uint32_t* n_valid,
                       int64_t cols, void* out, cudaStream_t st) {
  if (n_rows == 0) return 0;
  const int64_t n = n_rows * (cols / 8);
  gather_rows_kernel<<<cdiv(n, 256), 256, 0, st>>>(static_cast<const uint4*>(x), perm, src_map, n_rows, n_valid, (int)(cols / 8),
                                                   static_cast<uint4*>(out));
  return 0;
}

int launch_expand_indices(const uint32_t* lhs, const uint32_t* rhs, int64_t n_idx, int M, int64_t Bx, uint32_t* flat_expert,
                          uint32_t* flat_src, int* err, cudaStream_t st) {
  if (n_idx * M == 0) return 0;
  expand_indices_kernel<<<cdiv(n_idx * M, 256), 256, 0, st>>>(lhs, rhs, n_idx, M, Bx, flat_expert, flat_src, err);
  return 0;
}

}  // namespace b200

// CPU oracle for the quantized mixture-of-experts path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, on the CPU, what the reference's op wrappers ask the (out-of-tree)
// MLX library to compute.  Nothing that ships may call it: only the test-suite, the smoke
// check and the CPU-baseline legs of the benchmark load this library, and only as the
// checker.
//
// PARITY UNPINNED: the reference (oxiglade/mlx-rs) is a Rust binding whose arithmetic lives
// in the un-vendored mlx-c / MLX submodule (.gitmodules:1-3, directory empty, version not
// recoverable).  Its tests hold no golden vectors for this path, only relations between ops
// (mlx-rs/src/ops/quantization.rs:297-423, mlx-rs/src/ops/arithmetic.rs:3140-3238); those
// relations are replayed by the test-suite against this file.  The affine quantiser follows
// MLX's published algorithm as documented for mlx.core.quantize; packing order, tie-breaks
// and rounding points are fixed here by a canonical rule stated next to each function.
//
// Every function names the reference call site whose semantics it follows
// (paths relative to the reference project root).
//
// All tensors are plain row-major host arrays.  bf16 tensors are carried as float32 holding
// bf16-representable values unless a signature says uint16_t.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---- bf16 helpers ---------------------------------------------------------------------
inline float bf16_bits_to_f32(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// round-to-nearest-even float32 -> bf16 bits
inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return static_cast<uint16_t>(u >> 16);
}
inline float round_bf16(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }

// round-to-nearest-even float64 -> bf16 in ONE rounding (no float32 detour): the double is
// first squeezed to float32 with round-to-odd (truncate, then OR a sticky bit), which keeps
// enough information for the final 8-bit rounding to be correct.
inline uint16_t f64_to_bf16_bits(double d) {
  float f = static_cast<float>(d);  // RN; fix up to round-to-odd below
  if (std::isnan(d)) return 0x7fc0;
  if (std::isinf(f)) return f32_to_bf16_bits(f);
  double back = static_cast<double>(f);
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if (back != d) {
    // make |f| the truncation of |d| ...
    if (std::fabs(back) > std::fabs(d)) u -= 1;  // step one ulp toward zero (same sign bits)
    u |= 1u;                                     // ... and set the sticky bit
  }
  std::memcpy(&f, &u, 4);
  return f32_to_bf16_bits(f);
}
inline float round_bf16_from_f64(double d) { return bf16_bits_to_f32(f64_to_bf16_bits(d)); }

inline int elems_per_word(int bits) { return 32 / bits; }

// order-preserving key for (value descending, index ascending) selection
struct ValIdx {
  float v;
  uint32_t i;
};

}  // namespace

// dense row-major helper: out[M,N] = a[M,K] . b[N,K]^T with float32 accumulation.
// Every dot product is summed the same way whatever the blocking: eight interleaved partial sums
// over k (lane j takes k = j mod 8), combined pairwise at the end, then the tail of K.  A block
// of MB rows of a against NB rows of b shares the loads (register blocking); results are
// bit-identical to one dot product at a time.
template <int MB, int NB>
static inline void dot_block(const float* a, const float* b, int64_t K, int64_t lda, int64_t ldb, float* out, int64_t ldo) {
  float acc[MB][NB][8];
  for (int i = 0; i < MB; ++i)
    for (int j = 0; j < NB; ++j)
      for (int l = 0; l < 8; ++l) acc[i][j][l] = 0.f;
  int64_t k = 0;
  for (; k + 8 <= K; k += 8)
    for (int i = 0; i < MB; ++i)
      for (int j = 0; j < NB; ++j)
        for (int l = 0; l < 8; ++l) acc[i][j][l] += a[i * lda + k + l] * b[j * ldb + k + l];
  for (int i = 0; i < MB; ++i)
    for (int j = 0; j < NB; ++j) {
      const float* c = acc[i][j];
      float s = ((c[0] + c[1]) + (c[2] + c[3])) + ((c[4] + c[5]) + (c[6] + c[7]));
      for (int64_t kk = k; kk < K; ++kk) s += a[i * lda + kk] * b[j * ldb + kk];
      out[i * ldo + j] = s;
    }
}

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// The launcher of multi-process runs exports OMP_NUM_THREADS=1; a caller that owns the host (the
// timed CPU baseline) can ask for all cores again.  n <= 0: one thread per available processor.
int orc_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n > 0 ? n : omp_get_num_procs());
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

void orc_f32_to_bf16(const float* in, int64_t n, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16_bits(in[i]);
}
void orc_bf16_to_f32(const uint16_t* in, int64_t n, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_bits_to_f32(in[i]);
}
void orc_f64_to_bf16(const double* in, int64_t n, uint16_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = f64_to_bf16_bits(in[i]);
}

// quantize  — mlx-rs/src/ops/quantization.rs:48-83 (mlx_quantize, mode "affine").
// Groups of `gs` consecutive elements of the last axis share one scale and one bias; the
// `32/bits` codes of a word sit little-endian, element i in bits [bits*i, bits*i+bits).
// Scale/bias derivation follows MLX's affine quantiser: the group extreme with the larger
// magnitude is made exactly representable (the scale takes its sign from which extreme that
// is) and the bias is that extreme, or zero when it rounds to code 0.
// `round_params_bf16` != 0 rounds scale and bias to bf16 on output (weights given as bf16);
// the codes are always computed from the unrounded float32 scale and bias.
int orc_quantize(const float* w, int64_t rows, int64_t K, int gs, int bits, int round_params_bf16,
                 uint32_t* wq, float* scales, float* biases) {
  if (!(bits == 2 || bits == 4 || bits == 8) || gs <= 0 || K % gs != 0 || gs % elems_per_word(bits))
    return 1;
  const int epw = elems_per_word(bits);
  const float n_bins = static_cast<float>((1 << bits) - 1);
  const int64_t G = K / gs, Wp = K / epw;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t g = 0; g < G; ++g) {
      const float* p = w + r * K + g * gs;
      float wmin = p[0], wmax = p[0];
      for (int i = 1; i < gs; ++i) {
        wmin = std::fmin(wmin, p[i]);
        wmax = std::fmax(wmax, p[i]);
      }
      float scale = std::fmax((wmax - wmin) / n_bins, 1e-7f);
      bool side = std::fabs(wmin) > std::fabs(wmax);
      scale = side ? scale : -scale;
      float edge = side ? wmin : wmax;
      float q0 = std::round(edge / scale);
      bool at_zero = (q0 == 0.0f);
      scale = at_zero ? scale : edge / q0;
      float bias = at_zero ? 0.0f : edge;
      scales[r * G + g] = round_params_bf16 ? round_bf16(scale) : scale;
      biases[r * G + g] = round_params_bf16 ? round_bf16(bias) : bias;
      for (int i = 0; i < gs; i += epw) {
        uint32_t word = 0;
        for (int j = 0; j < epw; ++j) {
          float q = std::round((p[i + j] - bias) / scale);
          q = std::fmin(std::fmax(q, 0.0f), n_bins);
          word |= static_cast<uint32_t>(q) << (bits * j);
        }
        wq[r * Wp + (g * gs + i) / epw] = word;
      }
    }
  }
  return 0;
}

// dequantize — mlx-rs/src/ops/quantization.rs:129-158: w_hat = scale*q + bias, float32.
int orc_dequantize(const uint32_t* wq, const float* scales, const float* biases, int64_t rows,
                   int64_t K, int gs, int bits, float* out) {
  if (!(bits == 2 || bits == 4 || bits == 8) || gs <= 0 || K % gs != 0) return 1;
  const int epw = elems_per_word(bits);
  const uint32_t mask = (1u << bits) - 1u;
  const int64_t G = K / gs, Wp = K / epw;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t g = 0; g < G; ++g) {
      const float s = scales[r * G + g], b = biases[r * G + g];
      const uint32_t* pw = wq + r * Wp + g * (gs / epw);
      float* po = out + r * K + g * gs;
      for (int w = 0; w < gs / epw; ++w) {
        const uint32_t word = pw[w];
        for (int j = 0; j < epw; ++j) po[w * epw + j] = s * static_cast<float>((word >> (bits * j)) & mask) + b;
      }
    }
  return 0;
}

static void matmul_nt(const float* a, const float* b, int64_t M, int64_t N, int64_t K, float* out) {
  const int64_t mb = (M + 3) / 4, nb = (N + 1) / 2;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t bm = 0; bm < mb; ++bm)
    for (int64_t bn = 0; bn < nb; ++bn) {
      const int64_t m = bm * 4, n = bn * 2;
      const int mr = static_cast<int>(std::min<int64_t>(4, M - m)), nr = static_cast<int>(std::min<int64_t>(2, N - n));
      const float* pa = a + m * K;
      const float* pb = b + n * K;
      float* po = out + m * N + n;
      switch (mr * 2 + (nr - 1)) {
        case 2: dot_block<1, 1>(pa, pb, K, K, K, po, N); break;
        case 3: dot_block<1, 2>(pa, pb, K, K, K, po, N); break;
        case 4: dot_block<2, 1>(pa, pb, K, K, K, po, N); break;
        case 5: dot_block<2, 2>(pa, pb, K, K, K, po, N); break;
        case 6: dot_block<3, 1>(pa, pb, K, K, K, po, N); break;
        case 7: dot_block<3, 2>(pa, pb, K, K, K, po, N); break;
        case 8: dot_block<4, 1>(pa, pb, K, K, K, po, N); break;
        default: dot_block<4, 2>(pa, pb, K, K, K, po, N); break;
      }
    }
}

// quantized_matmul — mlx-rs/src/ops/quantization.rs:88-122.
// transpose != 0: w is [N, K/epw], result x . w_hat^T.   transpose == 0: w is [K, N/epw]
// (quantised along N), result x . w_hat.  float32 accumulation, float32 result.
int orc_quantized_matmul(const float* x, int64_t M, int64_t K, const uint32_t* wq, const float* scales,
                         const float* biases, int64_t N, int transpose, int gs, int bits, float* out) {
  if (transpose) {
    std::vector<float> wh(static_cast<size_t>(N) * K);
    if (orc_dequantize(wq, scales, biases, N, K, gs, bits, wh.data())) return 1;
    matmul_nt(x, wh.data(), M, N, K, out);
  } else {
    std::vector<float> wh(static_cast<size_t>(K) * N), wt(static_cast<size_t>(N) * K);
    if (orc_dequantize(wq, scales, biases, K, N, gs, bits, wh.data())) return 1;
    for (int64_t k = 0; k < K; ++k)
      for (int64_t n = 0; n < N; ++n) wt[n * K + k] = wh[k * N + n];
    matmul_nt(x, wt.data(), M, N, K, out);
  }
  return 0;
}

// gather_mm — mlx-rs/src/ops/arithmetic.rs:1568-1632: out[i] = a[lhs[i]] . b[rhs[i]],
// a [Ba,M,K], b [Bb,K,N], batch dims flattened before indexing (tests :3147-3211).
int orc_gather_mm(const float* a, int64_t Ba, int64_t M, int64_t K, const float* b, int64_t Bb, int64_t N,
                  const uint32_t* lhs, const uint32_t* rhs, int64_t n_idx, float* out) {
  for (int64_t i = 0; i < n_idx; ++i) {
    uint32_t ia = lhs ? lhs[i] : static_cast<uint32_t>(i);
    uint32_t ib = rhs ? rhs[i] : static_cast<uint32_t>(i);
    if (ia >= Ba || ib >= Bb) return 2;
    const float* pa = a + static_cast<int64_t>(ia) * M * K;
    const float* pb = b + static_cast<int64_t>(ib) * K * N;
    for (int64_t m = 0; m < M; ++m)
      for (int64_t n = 0; n < N; ++n) {
        float s = 0.f;
        for (int64_t k = 0; k < K; ++k) s += pa[m * K + k] * pb[k * N + n];
        out[(i * M + m) * N + n] = s;
      }
  }
  return 0;
}

// gather_qmm — mlx-rs/src/ops/quantization.rs:160-230 (transpose = true form):
// out[i] = x[lhs[i]] . dequantize(w[rhs[i]])^T, x [Bx,M,K], w [E,N,K/epw], out [n_idx,M,N].
// A null lhs means lhs[i] = i (x has one batch entry per index).
int orc_gather_qmm(const float* x, int64_t Bx, int64_t M, int64_t K, const uint32_t* wq, const float* scales,
                   const float* biases, int64_t E, int64_t N, const uint32_t* lhs, const uint32_t* rhs,
                   int64_t n_idx, int gs, int bits, float* out) {
  const int epw = elems_per_word(bits);
  const int64_t G = K / gs, Wp = K / epw;
  // visit indices grouped by expert so that each expert is dequantised once
  std::vector<int64_t> order(n_idx);
  std::iota(order.begin(), order.end(), 0);
  for (int64_t i = 0; i < n_idx; ++i)
    if (rhs[i] >= E || (lhs ? lhs[i] : i) >= Bx) return 2;
  std::stable_sort(order.begin(), order.end(), [&](int64_t p, int64_t q) { return rhs[p] < rhs[q]; });
  std::vector<float> wh(static_cast<size_t>(N) * K);
  int64_t cur = -1;
  for (int64_t s = 0; s < n_idx;) {
    int64_t e = rhs[order[s]];
    int64_t t = s;
    while (t < n_idx && rhs[order[t]] == e) ++t;
    if (e != cur) {
      if (orc_dequantize(wq + e * N * Wp, scales + e * N * G, biases + e * N * G, N, K, gs, bits, wh.data()))
        return 1;
      cur = e;
    }
    for (int64_t u = s; u < t; ++u) {
      int64_t i = order[u];
      int64_t ia = lhs ? lhs[i] : i;
      matmul_nt(x + ia * M * K, wh.data(), M, N, K, out + i * M * N);
    }
    s = t;
  }
  return 0;
}

// softmax_axis(-1, precise) — mlx-rs/src/ops/arithmetic.rs:1312-1327.  Canonical rule: the
// exact softmax of the given values, correctly rounded; realised in float64.  float64 out.
void orc_softmax_f64(const float* in, int64_t rows, int64_t cols, double* out) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* p = in + r * cols;
    double m = p[0];
    for (int64_t c = 1; c < cols; ++c) m = std::max<double>(m, p[c]);
    double s = 0;
    for (int64_t c = 0; c < cols; ++c) {
      out[r * cols + c] = std::exp(static_cast<double>(p[c]) - m);
      s += out[r * cols + c];
    }
    for (int64_t c = 0; c < cols; ++c) out[r * cols + c] /= s;
  }
}

// argsort_axis(-1) — mlx-rs/src/ops/sort.rs:57-83.  Canonical rule: STABLE ascending order
// (equal keys keep their input order).  Unsigned-integer keys.
void orc_argsort_u32(const uint32_t* keys, int64_t rows, int64_t cols, uint32_t* out) {
  for (int64_t r = 0; r < rows; ++r) {
    uint32_t* o = out + r * cols;
    std::iota(o, o + cols, 0u);
    const uint32_t* k = keys + r * cols;
    std::stable_sort(o, o + cols, [&](uint32_t a, uint32_t b) { return k[a] < k[b]; });
  }
}

// argpartition_axis(a, kth, -1) — mlx-rs/src/ops/sort.rs:186-226.  The reference leaves the
// order inside the partitions undefined; the canonical rule used here is the stable ascending
// argsort, which is one valid answer.  Float keys.
void orc_argpartition_f32(const float* a, int64_t rows, int64_t cols, int kth, uint32_t* out) {
  (void)kth;
  for (int64_t r = 0; r < rows; ++r) {
    uint32_t* o = out + r * cols;
    std::iota(o, o + cols, 0u);
    const float* k = a + r * cols;
    std::stable_sort(o, o + cols, [&](uint32_t x, uint32_t y) { return k[x] < k[y]; });
  }
}

// take_along_axis(-1) — mlx-rs/src/ops/indexing/mod.rs:424-453.
int orc_take_along_last(const float* a, int64_t rows, int64_t cols, const uint32_t* idx, int64_t icol, float* out) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < icol; ++c) {
      uint32_t j = idx[r * icol + c];
      if (j >= cols) return 2;
      out[r * icol + c] = a[r * cols + j];
    }
  return 0;
}

// fast::rms_norm — mlx-rs/src/fast.rs:178-205: w * x * rsqrt(mean(x^2) + eps), float32 math.
void orc_rms_norm(const float* x, const float* w, int64_t rows, int64_t cols, float eps, float* out) {
  for (int64_t r = 0; r < rows; ++r) {
    double ss = 0;
    for (int64_t c = 0; c < cols; ++c) ss += static_cast<double>(x[r * cols + c]) * x[r * cols + c];
    float inv = 1.0f / std::sqrt(static_cast<float>(ss / cols) + eps);
    for (int64_t c = 0; c < cols; ++c) out[r * cols + c] = (w ? w[c] : 1.0f) * (x[r * cols + c] * inv);
  }
}

// ---- the routed block ------------------------------------------------------------------
// Router: gate Linear (mlx-rs/src/nn/linear.rs:83-95, x . W^T) -> softmax -> top-k ->
// take_along_axis -> optional renormalisation (sum_axis + divide).
// Canonical rules: logits[t,e] = exact dot product of the bf16 operands, correctly rounded to
// bf16 (float64 accumulation).  mode 0 ("softmax then top-k"): p = exact softmax of the bf16
// logits, correctly rounded to bf16; top-k by (p descending, expert ascending); score = p, or
// p / sum(selected p) correctly rounded to bf16 when `renorm`.  mode 1 ("top-k then softmax"):
// top-k by (logit descending, expert ascending); score = softmax over the k selected logits,
// correctly rounded to bf16.  `logit_bias` (float32 [E], may be null) is added to the bf16
// logits in float32 and the sum is rounded to bf16 before routing (skewed-routing workload).
int orc_router(const float* x, const float* wr, int64_t T, int64_t H, int64_t E, int k, int mode, int renorm,
               const float* logit_bias, float* logits_out /*[T,E] or null*/, uint32_t* idx /*[T,k]*/,
               float* scores /*[T,k]*/) {
  if (k <= 0 || k > E) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    std::vector<float> lg(E);
    std::vector<float> pv(E);
    for (int64_t e = 0; e < E; ++e) {
      double acc = 0;
      const float* px = x + t * H;
      const float* pw = wr + e * H;
      for (int64_t h = 0; h < H; ++h) acc += static_cast<double>(px[h]) * static_cast<double>(pw[h]);
      float l = round_bf16_from_f64(acc);
      if (logit_bias) l = round_bf16(l + logit_bias[e]);
      lg[e] = l;
      if (logits_out) logits_out[t * E + e] = l;
    }
    if (mode == 0) {
      double m = lg[0];
      for (int64_t e = 1; e < E; ++e) m = std::max<double>(m, lg[e]);
      std::vector<double> ex(E);
      double s = 0;
      for (int64_t e = 0; e < E; ++e) {
        ex[e] = std::exp(static_cast<double>(lg[e]) - m);
        s += ex[e];
      }
      for (int64_t e = 0; e < E; ++e) pv[e] = round_bf16_from_f64(ex[e] / s);
    } else {
      pv = lg;
    }
    std::vector<uint32_t> o(E);
    std::iota(o.begin(), o.end(), 0u);
    std::stable_sort(o.begin(), o.end(), [&](uint32_t a, uint32_t b) { return pv[a] > pv[b]; });
    if (mode == 0) {
      double s = 0;
      for (int j = 0; j < k; ++j) s += pv[o[j]];
      for (int j = 0; j < k; ++j) {
        idx[t * k + j] = o[j];
        scores[t * k + j] = renorm ? round_bf16_from_f64(static_cast<double>(pv[o[j]]) / s) : pv[o[j]];
      }
    } else {
      double m = pv[o[0]], s = 0;
      std::vector<double> ex(k);
      for (int j = 0; j < k; ++j) {
        ex[j] = std::exp(static_cast<double>(pv[o[j]]) - m);
        s += ex[j];
      }
      for (int j = 0; j < k; ++j) {
        idx[t * k + j] = o[j];
        scores[t * k + j] = round_bf16_from_f64(ex[j] / s);
      }
    }
  }
  return 0;
}

// Token -> expert permutation: order = stable argsort of the token-major flat index list
// (mlx-rs/src/ops/sort.rs:57-83), inv = its inverse, counts = histogram, offsets = exclusive
// prefix sum.  Integer work; the CUDA path must reproduce every array bit for bit.
int orc_permute(const uint32_t* idx, int64_t n, int64_t E, uint32_t* perm, uint32_t* inv, uint32_t* counts,
                uint32_t* offsets /*[E+1]*/) {
  std::fill(counts, counts + E, 0u);
  for (int64_t i = 0; i < n; ++i) {
    if (idx[i] >= E) return 2;
    counts[idx[i]]++;
  }
  offsets[0] = 0;
  for (int64_t e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
  std::vector<uint32_t> cur(offsets, offsets + E);
  for (int64_t i = 0; i < n; ++i) {
    uint32_t p = cur[idx[i]]++;
    perm[p] = static_cast<uint32_t>(i);
    inv[i] = p;
  }
  return 0;
}

// SwitchGLU over sorted assignments + weighted combine.
//   x       [T,H]   bf16-valued float32
//   idx     [T,k]   expert of each assignment;   scores [T,k] (null: no combine, y_k written)
//   gate/up [E,I,H/epw] + scales/biases [E,I,H/gs];  down [E,H,I/epw] + [E,H,I/gs]
//   out     [T,H]   (combined)   or   y_k [T,k,H] when scores == null
// Rounding points: h = bf16(silu(g) * u) always; the final output is rounded to bf16 when
// `round_out` != 0 and left as the float32 accumulation otherwise (the tolerance of the parity
// tests is tighter than one bf16 ulp of a large output, so they compare with the unrounded
// value).  `round_every_op` != 0 additionally rounds g, u, silu(g), y, s*y and the running
// sum, which is the literal op-by-op dataflow of a bf16 graph
// (mlx-rs/src/nn/activation.rs:876-880, mlx-rs/src/ops/reduction.rs:260-275).
int orc_switch_glu(const float* x, int64_t T, int64_t H, int64_t E, int64_t I, int k, const uint32_t* idx,
                   const float* scores, const uint32_t* gq, const float* gs_, const float* gb,
                   const uint32_t* uq, const float* us, const float* ub, const uint32_t* dq, const float* ds,
                   const float* db, int gs, int bits, int round_every_op, int round_out, float* out) {
  const int epw = elems_per_word(bits);
  const int64_t n = T * k;
  std::vector<uint32_t> perm(n), inv(n), counts(E), offsets(E + 1);
  if (orc_permute(idx, n, E, perm.data(), inv.data(), counts.data(), offsets.data())) return 2;
  std::vector<float> yk(static_cast<size_t>(n) * H);
  const int64_t HW = H / epw, HG = H / gs, IW = I / epw, IG = I / gs;
  std::vector<float> wg(static_cast<size_t>(I) * H), wu(static_cast<size_t>(I) * H), wd(static_cast<size_t>(H) * I);
  for (int64_t e = 0; e < E; ++e) {
    int64_t m = counts[e];
    if (!m) continue;
    orc_dequantize(gq + e * I * HW, gs_ + e * I * HG, gb + e * I * HG, I, H, gs, bits, wg.data());
    orc_dequantize(uq + e * I * HW, us + e * I * HG, ub + e * I * HG, I, H, gs, bits, wu.data());
    orc_dequantize(dq + e * H * IW, ds + e * H * IG, db + e * H * IG, H, I, gs, bits, wd.data());
    std::vector<float> xs(static_cast<size_t>(m) * H), g(static_cast<size_t>(m) * I), u(static_cast<size_t>(m) * I),
        y(static_cast<size_t>(m) * H);
    for (int64_t r = 0; r < m; ++r)
      std::memcpy(&xs[r * H], x + static_cast<int64_t>(perm[offsets[e] + r] / k) * H, sizeof(float) * H);
    matmul_nt(xs.data(), wg.data(), m, I, H, g.data());
    matmul_nt(xs.data(), wu.data(), m, I, H, u.data());
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m * I; ++i) {
      float gv = g[i], uv = u[i];
      if (round_every_op) {
        gv = round_bf16(gv);
        uv = round_bf16(uv);
        float sg = round_bf16(1.0f / (1.0f + std::exp(-gv)));
        g[i] = round_bf16(round_bf16(gv * sg) * uv);
      } else {
        g[i] = round_bf16(gv / (1.0f + std::exp(-gv)) * uv);
      }
    }
    matmul_nt(g.data(), wd.data(), m, H, I, y.data());
    for (int64_t r = 0; r < m; ++r) {
      float* dst = &yk[static_cast<int64_t>(perm[offsets[e] + r]) * H];
      for (int64_t c = 0; c < H; ++c) dst[c] = round_every_op ? round_bf16(y[r * H + c]) : y[r * H + c];
    }
  }
  if (!scores) {
    for (int64_t i = 0; i < n * H; ++i) out[i] = round_out ? round_bf16(yk[i]) : yk[i];
    return 0;
  }
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t)
    for (int64_t c = 0; c < H; ++c) {
      float acc = 0.f;
      for (int j = 0; j < k; ++j) {
        float v = scores[t * k + j] * yk[(t * k + j) * H + c];
        if (round_every_op) {
          v = round_bf16(v);
          acc = round_bf16(acc + v);
        } else {
          acc += v;
        }
      }
      out[t * H + c] = round_out ? round_bf16(acc) : acc;
    }
  return 0;
}

}  // extern "C"

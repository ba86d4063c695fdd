// Grouped quantized expert GEMM for the memory-bound regime (few rows per expert).
//
// Replaces gather_qmm(x, w, scales, biases, rhs_indices, transpose=true, sorted_indices=true)
// (mlx-rs/src/ops/quantization.rs:160-230) for rows already grouped by expert, with the two
// epilogues of the routed block fused in:
//   NMAT = 2: gate and up projections in one launch, h = silu(x.Wg^T) * (x.Wu^T)
//             (nn::silu, mlx-rs/src/nn/activation.rs:876-880, and multiply);
//   NMAT = 1: down projection, each output row optionally multiplied by its routing weight
//             (multiply before sum_axis, mlx-rs/src/ops/reduction.rs:260-275) and written to
//             its un-sorted position (take with the inverse order).
//
// Every packed weight byte is read from HBM exactly once per pass, with 64-bit (4-bit codes) or
// 128-bit (8-bit codes) loads straight into registers, and never touches shared memory; the
// arithmetic is described in qmm_small.cuh.  Activations arrive PREPARED (fp16, row-scaled, unpack
// order; prepare_rows_small_kernel below, or the gate/up epilogue for the down projection) and are
// staged per CTA with 16-byte asynchronous copies.
//
// CTA = 8 warps = NMAT matrices x RT row tiles (16 output features each) x KS slices of the K
// groups (in blocks of four groups); partial sums of the KS slices meet in shared memory in a
// fixed order.  A warp handles ONE matrix, which keeps it near 64 registers (four CTAs per SM).
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "qmm_small.cuh"

namespace b200 {

using namespace qs;

template <int BITS, int NMAT, int RT, int NT>
__global__ void __launch_bounds__(256, NT == 1 ? 2 : 1) grouped_qmm_small_kernel(GroupedArgs p) {
  constexpr int KS = 8 / (NMAT * RT);
  constexpr int ROWS = 8 * NT;  // activation rows per pass
  static_assert(NMAT * RT * KS == 8, "eight warps");

  pdl_prologue();
  const int ea = blockIdx.y;
  if (ea >= (int)*p.n_active) return;
  const int e = p.active[ea];
  const uint32_t seg0 = p.offsets[e];
  const int m = (int)(p.offsets[e + 1] - seg0);
  if (m <= 0) return;

  const int K = p.K, N = p.N, G = K / 64;
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_src[ROWS];
  const Staged s = staged_at(smem, K, ROWS);
  float* red = reinterpret_cast<float*>(smem);  // aliases the staged rows after the K loop

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, t = lane & 3;
  const int mt = warp % NMAT, rt = (warp / NMAT) % RT, ks = warp / (NMAT * RT);
  const int n0 = blockIdx.x * (16 * RT) + rt * 16;
  const int wrow = K * BITS / 32;  // packed words per weight row

  // weight rows of this lane (rows beyond N are clamped: their results are never stored)
  constexpr int WPT = (BITS == 4) ? 2 : 4;  // packed words per lane per group per row
  const size_t row_a = (size_t)e * N + min(n0 + gq, N - 1), row_b = (size_t)e * N + min(n0 + gq + 8, N - 1);
  const uint32_t* w_a = p.w[mt] + row_a * wrow + t * WPT;
  const uint32_t* w_b = p.w[mt] + row_b * wrow + t * WPT;
  const unsigned short* sc_base = reinterpret_cast<const unsigned short*>(p.scales[mt]);
  const unsigned short* bi_base = reinterpret_cast<const unsigned short*>(p.biases[mt]);
  const __half* x16 = static_cast<const __half*>(p.x);

  const size_t soff_a = row_a * G, soff_b = row_b * G;
  // The CTA's weight rows start their way from DRAM to L2 now, all of them: the register stream below holds only two
  // blocks per lane in flight (64 KB per SM), too little to cover DRAM latency at full bandwidth; with the rows already
  // on their way its loads find them in L2.  Lanes t = 0 / 1 ask for the packed rows a / b, t = 2 / 3 for their scales
  // and biases.
  if (ks == 0 && !p.no_l2_prefetch) {
    if (t < 2) {
      l2_prefetch_bulk(p.w[mt] + (t == 0 ? row_a : row_b) * wrow, (uint32_t)wrow * 4u);
    } else {
      const size_t so = (t == 2 ? soff_a : soff_b);
      const char* ps = reinterpret_cast<const char*>(sc_base + so);
      const char* pb = reinterpret_cast<const char*>(bi_base + so);
      for (int o = 0; o < G * 2 + 127; o += 128) {
        l2_prefetch_line(ps + min(o, G * 2 - 1));
        l2_prefetch_line(pb + min(o, G * 2 - 1));
      }
    }
  }
  for (int p0 = 0; p0 < m; p0 += ROWS) {
    const int nrows = min(ROWS, m - p0);
    // the first block of weights is on its way while the activation rows are staged
    WeightStream<BITS> ws;
    ws.start(w_a, w_b, sc_base + soff_a, bi_base + soff_a, sc_base + soff_b, bi_base + soff_b, G, ks, KS);
    // ---- stage the nrows prepared rows of this pass -------------------------------------------
    if (tid < nrows) {
      const uint32_t sp = seg0 + p0 + tid;
      int src;
      if (p.src_mode == kSrcIdent)
        src = (int)sp;
      else if (p.src_mode == kSrcPermDiv)
        src = (int)(p.perm[sp] / (uint32_t)p.src_div);
      else if (p.src_mode == kSrcMapDirect)
        src = (int)p.src_map[sp];
      else
        src = (int)p.src_map[p.perm[sp]];
      s_src[tid] = src;
      s.rs[tid] = p.x_rowscale ? p.x_rowscale[src] : 1.0f;
    }
    __syncthreads();
    {
      const int nvec = K / 8;
      for (int i = tid; i < nrows * nvec; i += 256) {
        const int r = i / nvec, c = i % nvec;
        cp_async16(s.xs + (size_t)r * s.XS + c * 16, reinterpret_cast<const unsigned char*>(x16 + (size_t)s_src[r] * K) + c * 16);
      }
      cp_async_wait_all();
    }
    __syncthreads();
    stage_sums<BITS>(s, ROWS, nrows, K, tid, 256);
    __syncthreads();

    float tot[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int q = 0; q < 4; ++q) tot[nt][q] = 0.f;

    ws.template run<NT>(StagedFetch<ROWS>(s, gq, t), tot);

    // row scales leave shared memory before the partial sums overwrite it
    float rsv[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      rsv[nt][0] = s.rs[nt * 8 + 2 * t];
      rsv[nt][1] = s.rs[nt * 8 + 2 * t + 1];
    }
    __syncthreads();  // everyone is done with the staged rows: red may overwrite them

    // ---- partial sums -> shared, [warp][nt][row16][tok8], already multiplied by the row scale ----
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float* r = red + ((size_t)warp * NT + nt) * 128;
      r[gq * 8 + 2 * t] = tot[nt][0] * rsv[nt][0];
      r[gq * 8 + 2 * t + 1] = tot[nt][1] * rsv[nt][1];
      r[(gq + 8) * 8 + 2 * t] = tot[nt][2] * rsv[nt][0];
      r[(gq + 8) * 8 + 2 * t + 1] = tot[nt][3] * rsv[nt][1];
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
      for (int q = 0; q < NMAT; ++q) {
        float sum = 0.f;
#pragma unroll
        for (int z = 0; z < KS; ++z)
          sum += red[((size_t)((z * RT + ert) * NMAT + q) * NT + nt) * 128 + r16 * 8 + t8];
        v[q] = sum;
      }
      const uint32_t sp = seg0 + pr;
      const uint32_t dst = p.dst_perm ? p.perm[sp] : sp;
      float outv;
      if constexpr (NMAT == 2) {
        outv = v[0] / (1.0f + __expf(-v[0])) * v[1];
        if (p.out_f16) {  // h for the down projection of this same path: bf16-rounded value, prepared layout
          const float hb = __uint_as_float(f32_to_bf16_bits(outv) << 16) * prepared_factor<BITS>(n);
          reinterpret_cast<unsigned short*>(p.out)[(size_t)dst * N + prepared_pos<BITS>(n)] = f16_sat_bits(hb);
          continue;
        }
      } else {
        outv = v[0];
        if (p.row_scale) outv *= bf16_bits_to_f32(reinterpret_cast<const unsigned short*>(p.row_scale)[dst]);
      }
      if (p.out_row_addr) {
        const unsigned long long da = p.out_row_addr[sp];  // 0: the table's builder found no room for this row
        if (da) reinterpret_cast<__nv_bfloat16*>(da)[n] = __float2bfloat16_rn(outv);
      } else if (p.out_f32)
        reinterpret_cast<float*>(p.out)[(size_t)dst * N + n] = outv;
      else
        reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)dst * N + n] = __float2bfloat16_rn(outv);
    }
    __syncthreads();
  }
}

// ---- activation preparation ---------------------------------------------------------------------
// One warp per row: xs[r, :] = fp16( x[r, :] * 2^-e_r ) where 2^e_r (written to row_scale[r]) brings the
// row's largest magnitude into [2^14, 2^15); BITS == 4: aligned groups of eight elements are stored as
// [0,4,1,5,2,6,3,7] with elements 1,3,5,7 divided by 16 (see qmm_small.cuh).  The scaling is exact for bf16
// and fp16 input unless an element is more than 2^24 below the row maximum.
template <int BITS, bool IN_F16>
__global__ void __launch_bounds__(256) prepare_rows_small_kernel(const uint4* __restrict__ x, int64_t n_rows,
                                                                 const uint32_t* __restrict__ n_rows_dev, int vec_per_row,
                                                                 uint4* __restrict__ xs, float* __restrict__ row_scale) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= n_rows || (n_rows_dev && r >= (int64_t)*n_rows_dev)) return;
  prepare_row_warp<BITS, IN_F16>(x + (size_t)r * vec_per_row, vec_per_row, xs + (size_t)r * vec_per_row, row_scale + r, lane);
}

int launch_prepare_rows_small(const void* x, int in_f16, int64_t n_rows, const uint32_t* n_rows_dev, int K, int bits,
                              void* xs, float* row_scale, cudaStream_t st) {
  if (n_rows == 0) return 0;
  B200_REQUIRE(K % 8 == 0, "K must be a multiple of 8");
  const dim3 grid(cdiv(n_rows, 8)), block(256);
  const uint4* xp = static_cast<const uint4*>(x);
  uint4* op = static_cast<uint4*>(xs);
  if (bits == 4 && !in_f16)
    B200_CUDA(launch_pdl(prepare_rows_small_kernel<4, false>, grid, block, 0, st, xp, n_rows, n_rows_dev, K / 8, op, row_scale));
  else if (bits == 4)
    B200_CUDA(launch_pdl(prepare_rows_small_kernel<4, true>, grid, block, 0, st, xp, n_rows, n_rows_dev, K / 8, op, row_scale));
  else if (!in_f16)
    B200_CUDA(launch_pdl(prepare_rows_small_kernel<8, false>, grid, block, 0, st, xp, n_rows, n_rows_dev, K / 8, op, row_scale));
  else
    B200_CUDA(launch_pdl(prepare_rows_small_kernel<8, true>, grid, block, 0, st, xp, n_rows, n_rows_dev, K / 8, op, row_scale));
  return 0;
}

// ---- launch ----------------------------------------------------------------------------------------
template <int BITS, int NMAT, int RT, int NT>
static int launch_cfg(const GroupedArgs& a, int max_active, cudaStream_t st) {
  size_t smem = staged_bytes(a.K, 8 * NT);
  const size_t red = sizeof(float) * 8 * NT * 128;
  if (red > smem) smem = red;
  auto kern = grouped_qmm_small_kernel<BITS, NMAT, RT, NT>;
  static DynSmemCache attr;
  B200_CUDA(ensure_dyn_smem(kern, smem, attr));
  dim3 grid(cdiv(a.N, 16 * RT), max_active);
#ifdef B200_DEV
  GroupedArgs dev_args = a;
  if (getenv("B200_SMALL_NO_PREFETCH")) dev_args.no_l2_prefetch = 1;
  B200_CUDA(launch_pdl(kern, grid, dim3(256), smem, st, dev_args));
  return 0;
#endif
  B200_CUDA(launch_pdl(kern, grid, dim3(256), smem, st, a));
  return 0;
}

// Rows per expert above which a pass stages 32 rows instead of 8 (one CTA per SM then, but the weights are read once
// for four times the rows); below, an expert with more than eight rows takes several 8-row passes whose weight
// re-reads hit L2.
constexpr int64_t kWideAbove = 16;

template <int BITS, int NMAT>
static int launch_bits_nmat(const GroupedArgs& a, int max_active, int64_t rows, cudaStream_t st) {
  // more activation rows per pass once the experts are expected to hold more than eight rows each
  const int64_t per = rows / (max_active > 0 ? max_active : 1);
  int64_t wide_above = kWideAbove;
#ifdef B200_DEV
  if (const char* v = getenv("B200_SMALL_WIDE_ABOVE")) wide_above = atoi(v);
#endif
  const bool wide = per > wide_above && staged_bytes(a.K, 32) <= 200 * 1024;
  // row tiles per CTA: the largest that still gives three CTAs per SM, among those whose K slices
  // (8 / (NMAT * RT) of them, in blocks of four (4-bit) or two (8-bit) groups) all have work
  const int gb = BITS == 4 ? 4 : 2;  // groups per block of the weight stream
  const int nblk = (a.K / 64 + gb - 1) / gb;
  int rt = 8 / NMAT;
  for (int cand = 8 / NMAT; cand >= 1; cand >>= 1) {
    if (8 / (NMAT * cand) > nblk) break;
    rt = cand;
    if ((int64_t)cdiv(a.N, 16 * cand) * max_active >= 444) break;
  }
#define B200_DISPATCH_RT(RTV)                                                                        \
  case RTV:                                                                                          \
    if constexpr (RTV * NMAT <= 8)                                                                   \
      return wide ? launch_cfg<BITS, NMAT, RTV, 4>(a, max_active, st) : launch_cfg<BITS, NMAT, RTV, 1>(a, max_active, st); \
    break;
  switch (rt) {
    B200_DISPATCH_RT(1)
    B200_DISPATCH_RT(2)
    B200_DISPATCH_RT(4)
    B200_DISPATCH_RT(8)
  }
#undef B200_DISPATCH_RT
  B200_FAIL("no launch configuration");
}

bool small_shape_ok(int K) { return K % 64 == 0 && staged_bytes(K, 8) <= 200 * 1024; }

int launch_grouped_qmm_small(const GroupedArgs& a, int nmat, int bits, int max_active, int64_t rows, cudaStream_t st) {
  if (rows == 0 || max_active == 0) return 0;
  B200_REQUIRE(a.K % 64 == 0, "K must be a multiple of the group size 64");
  B200_REQUIRE(small_shape_ok(a.K), "K too large for the staged activation rows");
  if (bits == 4) return nmat == 2 ? launch_bits_nmat<4, 2>(a, max_active, rows, st) : launch_bits_nmat<4, 1>(a, max_active, rows, st);
  if (bits == 8) return nmat == 2 ? launch_bits_nmat<8, 2>(a, max_active, rows, st) : launch_bits_nmat<8, 1>(a, max_active, rows, st);
  B200_FAIL("bits must be 4 or 8");
}

}  // namespace b200

// Grouped quantized expert product for the memory-bound regime (a few rows per expert) on
// tensor memory: the unpack of a 4-bit code costs one logic instruction per TWO weights and
// nothing else, because the codes go to the tensor core as they are.
//
// Same contract as grouped_qmm_small_kernel (gather_qmm with sorted rows,
// mlx-rs/src/ops/quantization.rs:160-230, SiLU-gate / routing-weight epilogues fused).
//
//   work item = 16 sorted rows of one expert ("row tile")  x  128 output features
//               (NMAT = 2: the 128 gate features and the same 128 up features)
//   A operand = the weights: 128 rows x 64 k (one quantisation group) per stage, fp16, written by
//               the dequant warps as 1024+q (or 1024+16q for the nibbles that sit at bits 4..7 of
//               a byte: OR-ing a code into the mantissa of 1024.0 needs no shift there)
//   B operand = the 16 activation rows, fp16, brought by TMA from a buffer that
//               prepare_rows_mb_kernel wrote: each row scaled by a power of two, k-permuted the
//               way the codes unpack, and pre-divided by 16 at the 1024+16q positions
//   D         = one 128 x 16 float32 accumulator PER GROUP in tensor memory (a ring of 32), so that
//               the affine fold stays exact:  out[r, j] = sum_g s[r,g] * (D_g[r,j] - C_g[j]) + b[r,g] * X_g[j]
//               with C_g[j] = 1024 * (sum of the stored activations of group g) and X_g[j] the
//               group's plain activation sum, both tabulated by prepare_rows_mb_kernel
//
// Warp roles (15 warps): 0-3 fold + epilogue (a thread owns one weight row = one TMEM lane),
// 4-11 unpack (TMA-staged packed words -> A stages), 12 TMA producer for the packed weights,
// 13 TMA / bulk-copy producer for activations, tables, scales and biases, 14 MMA issuer (owns the
// TMEM allocation).  All hand-overs are mbarriers with bounded waits (tc_common.cuh); no load
// uses cluster multicast; no CTA waits on another.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace b200 {

namespace {

using namespace tc;

constexpr int MB_M = 128;          // weight rows per item (TMEM lanes)
constexpr int MB_N = 16;           // activation rows per item (accumulator columns per group)
constexpr int MB_A_STAGES = 2;     // unpacked A stages (16 KB each)
constexpr int MB_A_BYTES = MB_M * 64 * 2;
constexpr int MB_W_BOX = MB_M * 64;  // one TMA box of packed words: 128 rows x 64 bytes
constexpr int MB_SLOTS = 512 / MB_N;  // group accumulators in tensor memory
constexpr int MB_FOLD = 128, MB_DEQ = 256;
constexpr int MB_WARP_TMA_W = (MB_FOLD + MB_DEQ) / 32, MB_WARP_AUX = MB_WARP_TMA_W + 1, MB_WARP_MMA = MB_WARP_TMA_W + 2;
constexpr int MB_THREADS = MB_FOLD + MB_DEQ + 96;
constexpr int MB_MAX_K = 2048;     // activations of a row tile stay resident: 16 rows x K x 2 bytes
constexpr int MB_BAR_WORDS = 160;  // 64-bit slots reserved for barriers and flags

template <int NMAT>
struct MbCfg {
  static constexpr int W_STAGES = (NMAT == 2) ? 5 : 8;
  static constexpr int W_STAGE_BYTES = NMAT * MB_W_BOX;
};

struct MbArgs {
  const void* scales[2];
  const void* biases[2];
  const float2* tab;            // [rows + 16][G]: (X_g, C_g) of every prepared row
  const float* a_row_scale;     // by sorted position: the power of two each row was divided by
  const uint32_t* tile_expert;  // per row tile: expert
  const uint32_t* tile_row0;    // first sorted position
  const uint32_t* tile_rows;    // valid rows (<= 16)
  const uint32_t* n_row_tiles;  // device scalar
  const uint32_t* perm;
  int dst_perm;
  const void* row_scale;        // bf16 by out row, or null
  void* out;
  int out_f32;
  int K, N;
  int* err;
  int debug;                    // development: 32 = CTA 0 writes per-role wait cycles to err[16..]
};

// 8 codes of one 4-bit word -> 16 bytes of fp16: (1024+q0, 1024+q4), (1024+16 q1, 1024+16 q5),
// (1024+q2, 1024+q6), (1024+16 q3, 1024+16 q7): one shift and four logic operations.
__device__ __forceinline__ uint4 raw_word4(uint32_t w) {
  const uint32_t v = w >> 8;
  uint4 o;
  o.x = (w & 0x000f000fu) | 0x64006400u;
  o.y = (w & 0x00f000f0u) | 0x64006400u;
  o.z = (v & 0x000f000fu) | 0x64006400u;
  o.w = (v & 0x00f000f0u) | 0x64006400u;
  return o;
}
// 8 codes of two 8-bit words -> 16 bytes of fp16 1024+q in natural order
__device__ __forceinline__ uint4 raw_word8(uint32_t w0, uint32_t w1) {
  uint4 o;
  o.x = __byte_perm(w0, 0x64646464u, 0x4140);
  o.y = __byte_perm(w0, 0x64646464u, 0x4342);
  o.z = __byte_perm(w1, 0x64646464u, 0x4140);
  o.w = __byte_perm(w1, 0x64646464u, 0x4342);
  return o;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
template <int NJ>
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[16]) {
  if constexpr (NJ == 4) {
    uint32_t t[4];
    tmem_ld4(taddr, t);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = t[i];
  } else if constexpr (NJ == 8) {
    uint32_t t[8];
    tmem_ld8(taddr, t);
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = t[i];
  } else {
    tmem_ld16(taddr, r);
  }
}

constexpr uint32_t kMbIdesc = umma_idesc_f16(MB_M, MB_N);

// Shared-memory map (offsets from the 1024-byte aligned base).
template <int NMAT>
struct MbSmem {
  static constexpr int a_off = 0;
  static constexpr int w_off = a_off + MB_A_STAGES * MB_A_BYTES;
  static constexpr int x_off = w_off + MbCfg<NMAT>::W_STAGES * MbCfg<NMAT>::W_STAGE_BYTES;   // [G][16 rows][128 B]
  static constexpr int x_bytes = MB_N * MB_MAX_K * 2;
  static constexpr int tab_off = x_off + x_bytes;                                            // [16][G] float2
  static constexpr int tab_bytes = MB_N * (MB_MAX_K / 64) * 8;
  static constexpr int sb_off = tab_off + tab_bytes;                                         // [NMAT][2][128][G] bf16
  static constexpr int sb_bytes = NMAT * 2 * MB_M * (MB_MAX_K / 64) * 2;
  static constexpr int bar_off = sb_off + sb_bytes;
  static constexpr int total = bar_off + MB_BAR_WORDS * 8 + 1024;
};

// Fold of one item for a row tile with at most NJ valid rows.
template <int BITS, int NMAT, int NJ>
__device__ __forceinline__ bool mb_fold_item(const MbArgs& p, int G, uint32_t tmem_lane, const unsigned char* sb_st,
                                             const float2* tab_st, uint32_t tfull0, uint32_t tempty0, uint32_t& sc,
                                             volatile int* abort_flag, int row, int lane, float (&tot)[NMAT][16]) {
#pragma unroll
  for (int mt = 0; mt < NMAT; ++mt)
#pragma unroll
    for (int j = 0; j < 16; ++j) tot[mt][j] = 0.f;
  uint2 sv[NMAT], bv[NMAT];
  for (int g = 0; g < G; ++g) {
    if ((g & 3) == 0) {
#pragma unroll
      for (int mt = 0; mt < NMAT; ++mt) {
        sv[mt] = *reinterpret_cast<const uint2*>(sb_st + ((size_t)((mt * 2 + 0) * MB_M + row) * G + g) * 2);
        bv[mt] = *reinterpret_cast<const uint2*>(sb_st + ((size_t)((mt * 2 + 1) * MB_M + row) * G + g) * 2);
      }
    }
    float2 xc[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) xc[j] = tab_st[j * G + g];
#pragma unroll
    for (int mt = 0; mt < NMAT; ++mt) {
      const uint32_t sw = (g & 2) ? sv[mt].y : sv[mt].x, bw = (g & 2) ? bv[mt].y : bv[mt].x;
      const float s = (g & 1) ? __uint_as_float(sw & 0xffff0000u) : __uint_as_float(sw << 16);
      const float b = (g & 1) ? __uint_as_float(bw & 0xffff0000u) : __uint_as_float(bw << 16);
      const uint32_t slot = sc % MB_SLOTS, ph = (sc / MB_SLOTS) & 1u;
      ++sc;
      if (!mbar_wait(tfull0 + 8u * slot, ph, abort_flag)) return false;
      tc_fence_after();
      uint32_t d[16];
      tmem_ld_n<NJ>(tmem_lane + slot * MB_N, d);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(tempty0 + 8u * slot, lane);
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        // s * (D - C) + b * X, with the correction taken first (it does not depend on the accumulator)
        const float corr = fmaf(b, xc[j].x, -s * xc[j].y);
        tot[mt][j] += fmaf(s, __uint_as_float(d[j]), corr);
      }
    }
  }
  return true;
}

template <int BITS, int NMAT>
__global__ void __launch_bounds__(MB_THREADS, 1)
grouped_qmm_mb_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w0,
                      const __grid_constant__ CUtensorMap tmap_w1, MbArgs p) {
  using S = MbSmem<NMAT>;
  constexpr int W_STAGES = MbCfg<NMAT>::W_STAGES, W_STAGE_BYTES = MbCfg<NMAT>::W_STAGE_BYTES;
  constexpr int KPS = (BITS == 4) ? 2 : 1;  // groups covered by one W stage (64 packed bytes per row)
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* a_st = smem + S::a_off;
  unsigned char* w_st = smem + S::w_off;
  unsigned char* x_st = smem + S::x_off;
  const float2* tab_st = reinterpret_cast<const float2*>(smem + S::tab_off);
  unsigned char* sb_st = smem + S::sb_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::bar_off);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 100);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 101);
  const uint32_t bar0 = smem_u32(bars);
  auto wfull = [&](int s) { return bar0 + 8u * s; };
  auto wempty = [&](int s) { return bar0 + 8u * (8 + s); };
  auto afull = [&](int s) { return bar0 + 8u * (16 + s); };
  auto aempty = [&](int s) { return bar0 + 8u * (18 + s); };
  const uint32_t xfull = bar0 + 8u * 20, xempty = bar0 + 8u * 21, sbfull = bar0 + 8u * 22, sbempty = bar0 + 8u * 23;
  const uint32_t tfull0 = bar0 + 8u * 32, tempty0 = bar0 + 8u * 64;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.K / 64;
  const int n_col = p.N / MB_M;

  if (tid == 0) {
    for (int s = 0; s < W_STAGES; ++s) {
      mbar_init(wfull(s), 1);
      mbar_init(wempty(s), MB_DEQ / 32);
    }
    for (int s = 0; s < MB_A_STAGES; ++s) {
      mbar_init(afull(s), MB_DEQ / 32);
      mbar_init(aempty(s), 1);
    }
    mbar_init(xfull, 1);
    mbar_init(xempty, 1 + MB_FOLD / 32);
    mbar_init(sbfull, 1);
    mbar_init(sbempty, MB_FOLD / 32);
    for (int s = 0; s < MB_SLOTS; ++s) {
      mbar_init(tfull0 + 8u * s, 1);
      mbar_init(tempty0 + 8u * s, MB_FOLD / 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MB_WARP_MMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // this CTA's contiguous range of items (consecutive items share a row tile, hence the activations)
  const int total = (int)(*p.n_row_tiles) * n_col;
  const int t_begin = (int)(((long long)blockIdx.x * total) / (int)gridDim.x);
  const int t_end = (int)(((long long)(blockIdx.x + 1) * total) / (int)gridDim.x);

  if (warp < MB_FOLD / 32) {
    // ------------------------------- fold + epilogue ------------------------------------
    const int row = tid;
    const uint32_t tmem_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
    uint32_t sc = 0;
    int xph = 0, sbph = 0, prev_rt = -1;
    RoleTimer tm((p.debug & 32) && blockIdx.x == 0 && tid == 0);
    const long long t_start = clock64();
    for (int t = t_begin; t < t_end; ++t) {
      const int rt = t / n_col, ct = t % n_col;
      tm.start();
      if (rt != prev_rt) {
        if (prev_rt >= 0) mbar_arrive_warp(xempty, lane);  // done with the previous row tile's table
        if (!mbar_wait(xfull, xph, abort_flag)) break;
        xph ^= 1;
        prev_rt = rt;
      }
      if (!mbar_wait(sbfull, sbph, abort_flag)) break;
      sbph ^= 1;
      tm.stop(0);
      tm.start();
      const uint32_t row0 = p.tile_row0[rt];
      const int rows = (int)p.tile_rows[rt];
      float tot[NMAT][16];
      bool ok;
      if (rows <= 4)
        ok = mb_fold_item<BITS, NMAT, 4>(p, G, tmem_lane, sb_st, tab_st, tfull0, tempty0, sc, abort_flag, row, lane, tot);
      else if (rows <= 8)
        ok = mb_fold_item<BITS, NMAT, 8>(p, G, tmem_lane, sb_st, tab_st, tfull0, tempty0, sc, abort_flag, row, lane, tot);
      else
        ok = mb_fold_item<BITS, NMAT, 16>(p, G, tmem_lane, sb_st, tab_st, tfull0, tempty0, sc, abort_flag, row, lane, tot);
      if (!ok) break;
      tm.stop(1);
      tm.start();
      mbar_arrive_warp(sbempty, lane);  // scales and biases of this item are consumed
      const int n = ct * MB_M + row;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (j < rows) {
          const uint32_t sp = row0 + j;
          const uint32_t dst = p.dst_perm ? p.perm[sp] : sp;
          const float ar = p.a_row_scale[sp];
          float outv;
          if constexpr (NMAT == 2) {
            const float gv = tot[0][j] * ar, uv = tot[1][j] * ar;
            outv = gv / (1.0f + __expf(-gv)) * uv;
          } else {
            outv = tot[0][j] * ar;
            if (p.row_scale) outv *= bf16_bits_to_f32(static_cast<const unsigned short*>(p.row_scale)[dst]);
          }
          if (p.out_f32)
            static_cast<float*>(p.out)[(size_t)dst * p.N + n] = outv;
          else
            static_cast<__nv_bfloat16*>(p.out)[(size_t)dst * p.N + n] = __float2bfloat16_rn(outv);
        }
      }
      tm.stop(2);
    }
    if (prev_rt >= 0) mbar_arrive_warp(xempty, lane);
    tm.acc[3] = clock64() - t_start;
    tm.flush(p.err + 16);
  } else if (warp < (MB_FOLD + MB_DEQ) / 32) {
    // ------------------------------- unpack: packed words -> A stages ---------------------
    const int td = tid - MB_FOLD;
    const int row = td >> 1, half = td & 1;
    const uint32_t a_row_off = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
    const uint32_t sw = (uint32_t)(row & 7), wsw = (uint32_t)((row >> 1) & 3);
    int ws = 0, wph = 0, as = 0, aph = 0;
    bool dead = false;
    RoleTimer tm((p.debug & 32) && blockIdx.x == 0 && tid == MB_FOLD);
    const long long t_start = clock64();
    for (int t = t_begin; t < t_end && !dead; ++t) {
      for (int kb = 0; kb < G && !dead; ++kb) {
        const int kin = kb % KPS;
        tm.start();
        if (kin == 0 && !mbar_wait(wfull(ws), wph, abort_flag)) {
          dead = true;
          break;
        }
        tm.stop(0);
#pragma unroll
        for (int mt = 0; mt < NMAT; ++mt) {
          const unsigned char* wsrc = w_st + (size_t)ws * W_STAGE_BYTES + mt * MB_W_BOX + row * 64;
          uint4 r0, r1 = make_uint4(0, 0, 0, 0);
          if constexpr (BITS == 4) {
            r0 = *reinterpret_cast<const uint4*>(wsrc + (((uint32_t)(kin * 2 + half) ^ wsw) << 4));
          } else {
            r0 = *reinterpret_cast<const uint4*>(wsrc + (((uint32_t)(half * 2) ^ wsw) << 4));
            r1 = *reinterpret_cast<const uint4*>(wsrc + (((uint32_t)(half * 2 + 1) ^ wsw) << 4));
          }
          tm.start();
          if (!mbar_wait(aempty(as), aph ^ 1, abort_flag)) {
            dead = true;
            break;
          }
          tm.stop(1);
          tm.start();
          unsigned char* dst = a_st + (size_t)as * MB_A_BYTES + a_row_off;
          uint4 o[4];
          if constexpr (BITS == 4) {
            o[0] = raw_word4(r0.x);
            o[1] = raw_word4(r0.y);
            o[2] = raw_word4(r0.z);
            o[3] = raw_word4(r0.w);
          } else {
            o[0] = raw_word8(r0.x, r0.y);
            o[1] = raw_word8(r0.z, r0.w);
            o[2] = raw_word8(r1.x, r1.y);
            o[3] = raw_word8(r1.z, r1.w);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(dst + (((uint32_t)(half * 4 + i) ^ sw) << 4)) = o[i];
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_arrive_warp(afull(as), lane);
          tm.stop(2);
          if (++as == MB_A_STAGES) {
            as = 0;
            aph ^= 1;
          }
        }
        if (!dead && (kin == KPS - 1 || kb == G - 1)) {
          mbar_arrive_warp(wempty(ws), lane);
          if (++ws == W_STAGES) {
            ws = 0;
            wph ^= 1;
          }
        }
      }
    }
    tm.acc[3] = clock64() - t_start;
    tm.flush(p.err + 20);
  } else if (warp == MB_WARP_TMA_W) {
    // ------------------------------- TMA producer: packed weights ---------------------------
    if (lane == 0) {
      int ws = 0, wph = 0;
      bool dead = false;
      const int n_wst = (G + KPS - 1) / KPS;
      for (int t = t_begin; t < t_end && !dead; ++t) {
        const int rt = t / n_col, ct = t % n_col;
        const int row_base = (int)p.tile_expert[rt] * p.N + ct * MB_M;
        for (int wk = 0; wk < n_wst; ++wk) {
          if (!mbar_wait(wempty(ws), wph ^ 1, abort_flag)) {
            dead = true;
            break;
          }
          mbar_arrive_expect_tx(wfull(ws), W_STAGE_BYTES);
          const uint32_t dst = smem_u32(w_st + (size_t)ws * W_STAGE_BYTES);
          tma_load_2d(dst, &tmap_w0, wfull(ws), wk * 16, row_base);
          if constexpr (NMAT == 2) tma_load_2d(dst + MB_W_BOX, &tmap_w1, wfull(ws), wk * 16, row_base);
          if (++ws == W_STAGES) {
            ws = 0;
            wph ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == MB_WARP_AUX) {
    // ------------------------------- producer: activations, tables, scales, biases ----------
    if (lane == 0) {
      int xph = 0, sbph = 0, prev_rt = -1;
      const uint32_t sb_each = (uint32_t)MB_M * G * 2;
      for (int t = t_begin; t < t_end; ++t) {
        const int rt = t / n_col, ct = t % n_col;
        if (rt != prev_rt) {
          if (!mbar_wait(xempty, xph ^ 1, abort_flag)) break;
          xph ^= 1;
          const int row0 = (int)p.tile_row0[rt];
          mbar_arrive_expect_tx(xfull, (uint32_t)G * (MB_N * 128) + (uint32_t)MB_N * G * 8);
          for (int g = 0; g < G; ++g) tma_load_2d(smem_u32(x_st + (size_t)g * (MB_N * 128)), &tmap_x, xfull, g * 64, row0);
          bulk_g2s(smem_u32(tab_st), p.tab + (size_t)row0 * G, (uint32_t)MB_N * G * 8, xfull);
          prev_rt = rt;
        }
        if (!mbar_wait(sbempty, sbph ^ 1, abort_flag)) break;
        sbph ^= 1;
        const size_t wr = ((size_t)p.tile_expert[rt] * p.N + (size_t)ct * MB_M) * G;
        mbar_arrive_expect_tx(sbfull, NMAT * 2 * sb_each);
#pragma unroll
        for (int mt = 0; mt < NMAT; ++mt) {
          bulk_g2s(smem_u32(sb_st + (size_t)(mt * 2 + 0) * sb_each), static_cast<const unsigned short*>(p.scales[mt]) + wr,
                   sb_each, sbfull);
          bulk_g2s(smem_u32(sb_st + (size_t)(mt * 2 + 1) * sb_each), static_cast<const unsigned short*>(p.biases[mt]) + wr,
                   sb_each, sbfull);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- MMA issuer ----------------------------------------------
    if (lane == 0) {
      int as = 0, aph = 0, xph = 0, prev_rt = -1;
      uint32_t sc = 0;
      bool dead = false;
      RoleTimer tm((p.debug & 32) && blockIdx.x == 0);
      const long long t_start = clock64();
      for (int t = t_begin; t < t_end && !dead; ++t) {
        const int rt = t / n_col;
        if (rt != prev_rt) {
          if (prev_rt >= 0) umma_commit(xempty);  // every product that read the previous activations has completed
          if (!mbar_wait(xfull, xph, abort_flag)) break;
          xph ^= 1;
          prev_rt = rt;
        }
        for (int kb = 0; kb < G && !dead; ++kb) {
          const uint32_t x_addr = smem_u32(x_st + (size_t)kb * (MB_N * 128));
#pragma unroll
          for (int mt = 0; mt < NMAT; ++mt) {
            const uint32_t slot = sc % MB_SLOTS, ph = (sc / MB_SLOTS) & 1u;
            ++sc;
            tm.start();
            if (!mbar_wait(afull(as), aph, abort_flag)) {
              dead = true;
              break;
            }
            tm.stop(0);
            tm.start();
            if (!mbar_wait(tempty0 + 8u * slot, ph ^ 1u, abort_flag)) {
              dead = true;
              break;
            }
            tm.stop(1);
            tc_fence_after();
            const uint32_t a_addr = smem_u32(a_st + (size_t)as * MB_A_BYTES);
            const uint32_t d_addr = tmem_base + slot * MB_N;
            if (!(p.debug & 2)) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_f16(d_addr, umma_desc(a_addr + k * 32), umma_desc(x_addr + k * 32), kMbIdesc, k ? 1u : 0u);
            }
            umma_commit(aempty(as));
            umma_commit(tfull0 + 8u * slot);
            if (++as == MB_A_STAGES) {
              as = 0;
              aph ^= 1;
            }
          }
        }
      }
      if (prev_rt >= 0 && !dead) umma_commit(xempty);
      tm.acc[3] = clock64() - t_start;
      tm.flush(p.err + 28);
    }
    __syncwarp();
  }

  // ------------------------------- teardown ------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicExch(p.err, 3);
    __nanosleep(200000);  // let copies and MMAs that are still in flight land before the CTA goes away
  }
  if (warp == MB_WARP_MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
}

// Activation preparation, one warp per row:
//   xs[p, :]  = fp16( x[src(p), :] * 2^-e_p ), 2^e_p (written to row_scale[p]) bringing the row's largest
//               magnitude into [2^14, 2^15); for 4-bit weights every aligned group of eight is stored in
//               the order [0,4,1,5,2,6,3,7] and the elements paired with the in-place nibbles (original
//               positions 1,3,5,7) are divided by 16 (exact: a power of two)
//   tab[p, g] = ( X = sum of the group's effective activations (stored value, x16 where it was divided),
//                 C = 1024 * sum of the group's stored values ), computed from the ROUNDED fp16 values,
//               i.e. from exactly what the tensor core multiplies
__global__ void __launch_bounds__(256) prepare_rows_mb_kernel(const uint4* __restrict__ x, const uint32_t* __restrict__ perm,
                                                              int src_div, int64_t n_rows, int vec_per_row, int four_bit,
                                                              uint4* __restrict__ xs, float* __restrict__ row_scale,
                                                              float2* __restrict__ tab) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const uint32_t src = perm ? perm[r] / (uint32_t)src_div : (uint32_t)r;
  const uint4* xr = x + (size_t)src * vec_per_row;
  uint32_t mxbits = 0;
  for (int c = lane; c < vec_per_row; c += 32) {
    const uint4 v = __ldg(xr + c);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) mxbits = max(mxbits, max(u[q] & 0x7fffu, (u[q] >> 16) & 0x7fffu));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mxbits = max(mxbits, __shfl_xor_sync(0xffffffffu, mxbits, o));
  const float mx = bf16_bits_to_f32(mxbits);
  int ex = (mx > 0.f && mx < 3.0e38f) ? (ilogbf(mx) - 14) : 0;
  ex = max(-100, min(100, ex));
  const float f = ldexpf(1.0f, -ex);
  if (lane == 0) row_scale[r] = ldexpf(1.0f, ex);
  const int G = vec_per_row / 8;
  for (int c0 = 0; c0 < vec_per_row; c0 += 32) {   // vec_per_row is a multiple of 32 (K % 256 == 0)
    const int c = c0 + lane;
    const uint4 v = __ldg(xr + c);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    float e8[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      e8[2 * q] = __uint_as_float(u[q] << 16) * f;
      e8[2 * q + 1] = __uint_as_float(u[q] & 0xffff0000u) * f;
    }
    float sx = 0.f, sc = 0.f;
    uint32_t hh[4];
    if (four_bit) {
      // stored order [0,4,1,5,2,6,3,7]; original positions 1,5,3,7 pair with the in-place nibbles
      const int order[8] = {0, 4, 1, 5, 2, 6, 3, 7};
      __half hv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool div = (i & 2) != 0;  // stored positions 2,3,6,7
        hv[i] = __float2half_rn(div ? e8[order[i]] * 0.0625f : e8[order[i]]);
        const float st = __half2float(hv[i]);
        sc += st;
        sx += div ? st * 16.f : st;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) hh[q] = (uint32_t)__half_as_ushort(hv[2 * q]) | ((uint32_t)__half_as_ushort(hv[2 * q + 1]) << 16);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const __half a = __float2half_rn(e8[2 * q]), b = __float2half_rn(e8[2 * q + 1]);
        sc += __half2float(a) + __half2float(b);
        hh[q] = (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
      }
      sx = sc;
    }
    xs[(size_t)r * vec_per_row + c] = make_uint4(hh[0], hh[1], hh[2], hh[3]);
    // a group = 8 consecutive vectors = 8 consecutive lanes
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      sx += __shfl_xor_sync(0xffffffffu, sx, o);
      sc += __shfl_xor_sync(0xffffffffu, sc, o);
    }
    if ((lane & 7) == 0) tab[(size_t)r * G + (c >> 3)] = make_float2(sx, 1024.f * sc);
  }
}

}  // namespace

bool mb_shape_ok(int K, int N) { return K % 256 == 0 && K <= MB_MAX_K && N % MB_M == 0; }

int launch_prepare_rows_mb(const void* x, const uint32_t* perm, int src_div, int64_t n_rows, int K, int bits, void* xs,
                           float* row_scale, void* tab, cudaStream_t st) {
  if (n_rows == 0) return 0;
  prepare_rows_mb_kernel<<<cdiv(n_rows, 8), 256, 0, st>>>(static_cast<const uint4*>(x), perm, src_div, n_rows, K / 8,
                                                         bits == 4, static_cast<uint4*>(xs), row_scale,
                                                         static_cast<float2*>(tab));
  return 0;
}

// xs: prepared rows [rows + 16, K] fp16 (the 16 rows of padding are read, never used); tab likewise.
int launch_grouped_qmm_mb(const void* xs, const float* a_row_scale, const void* tab, int64_t rows, const GroupedArgs& g,
                          int nmat, int bits, const uint32_t* tile_expert, const uint32_t* tile_row0,
                          const uint32_t* tile_rows, const uint32_t* n_row_tiles, int E, int* err, cudaStream_t st) {
  if (rows == 0) return 0;
  B200_REQUIRE(mb_shape_ok(g.K, g.N), "shape not supported by the tensor-memory small-batch path");
  EncodeTiledFn enc = encode_fn();
  B200_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap tmap_x;
  {
    cuuint64_t dims[2] = {(cuuint64_t)g.K, (cuuint64_t)(rows + MB_N)};
    cuuint64_t strides[1] = {(cuuint64_t)g.K * 2};
    cuuint32_t box[2] = {64, MB_N};
    CUresult cr = enc(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(xs), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for the prepared rows");
  }
  CUtensorMap tmap_w[2];
  for (int i = 0; i < nmat; ++i) {
    cuuint64_t wd[2] = {(cuuint64_t)g.K * bits / 32, (cuuint64_t)E * g.N};
    cuuint64_t ws_[1] = {(cuuint64_t)g.K * bits / 8};
    cuuint32_t wb[2] = {16, MB_M};
    CUresult cr = enc(&tmap_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(g.w[i]), wd, ws_, wb, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for the packed weights (16-byte alignment required)");
  }
  if (nmat == 1) tmap_w[1] = tmap_w[0];

  MbArgs p{};
  for (int i = 0; i < 2; ++i) {
    p.scales[i] = g.scales[i];
    p.biases[i] = g.biases[i];
  }
  p.tab = static_cast<const float2*>(tab);
  p.a_row_scale = a_row_scale;
  p.tile_expert = tile_expert;
  p.tile_row0 = tile_row0;
  p.tile_rows = tile_rows;
  p.n_row_tiles = n_row_tiles;
  p.perm = g.perm;
  p.dst_perm = g.dst_perm;
  p.row_scale = g.row_scale;
  p.out = g.out;
  p.out_f32 = g.out_f32;
  p.K = g.K;
  p.N = g.N;
  p.err = err;
  {
    static const int dbg = [] { const char* v = getenv("B200_TC_DEBUG"); return v ? atoi(v) : 0; }();
    p.debug = dbg;
  }

  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  }
  const int64_t max_items = (int64_t)(rows / MB_N + E + 1) * (g.N / MB_M);
  const int grid = (int)(max_items < n_sm ? max_items : n_sm);

#define B200_MB_LAUNCH(BITSV, NMATV)                                                                            \
  do {                                                                                                          \
    auto kern = grouped_qmm_mb_kernel<BITSV, NMATV>;                                                            \
    static bool attr = false;                                                                                   \
    if (!attr) {                                                                                                \
      B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MbSmem<NMATV>::total)); \
      attr = true;                                                                                              \
    }                                                                                                           \
    kern<<<grid, MB_THREADS, MbSmem<NMATV>::total, st>>>(tmap_x, tmap_w[0], tmap_w[1], p);                      \
  } while (0)
  if (bits == 4 && nmat == 2)
    B200_MB_LAUNCH(4, 2);
  else if (bits == 4 && nmat == 1)
    B200_MB_LAUNCH(4, 1);
  else if (bits == 8 && nmat == 2)
    B200_MB_LAUNCH(8, 2);
  else if (bits == 8 && nmat == 1)
    B200_MB_LAUNCH(8, 1);
  else
    B200_FAIL("bits must be 4 or 8");
#undef B200_MB_LAUNCH
  return 0;
}

}  // namespace b200

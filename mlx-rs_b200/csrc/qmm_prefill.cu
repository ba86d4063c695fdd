// Grouped quantized expert GEMM for the dense (prefill) regime: tcgen05 tensor cores with
// TMEM accumulators, A tiles staged by TMA, B tiles dequantised into shared memory.
//
// Same contract as the memory-bound kernel (gather_qmm with sorted rows,
// mlx-rs/src/ops/quantization.rs:160-230, with the SiLU-gate and routing-weight epilogues
// fused), chosen when experts own many rows.  Per CTA (persistent over a tile list):
//
//   tile    = 256 rows of one expert's segment (two 128-row accumulators)  x  256 accumulator columns
//             (NMAT = 2: 128 gate features + the same 128 up features; NMAT = 1: 256 features);
//             both accumulators consume every dequantised B stage, which halves the
//             dequantisation work per product
//   K loop  = blocks of 64 (= one quantisation group), 2 x 4 UMMA instructions m128 n256 k16 each
//   A       = activations [rows, K] fp16, two TMA tile loads (128 x 64, 128-byte swizzle) per block
//   W       = the packed weights of the tile's 256 accumulator columns, 128 bytes per row (four
//             4-bit or two 8-bit K blocks) per TMA stage: per-lane loads of 32 bytes from 256
//             different rows cost the L1 a cycle per row, bulk tensor copies do not
//   B       = one thread per accumulator column reads its row's 32 (4-bit) or 64 (8-bit) packed
//             bytes from the W stage plus its scale and bias, forms w_hat = fp16(scale*q + bias) with one
//             fused multiply-add per pair, and writes the row's 128 bytes in the same swizzled
//             K-major layout TMA produces.  fp16 (11 significant bits) rather than bf16 (8) keeps
//             the dequantisation error an order of magnitude below the output tolerance; its
//             narrow exponent range is handled by scaling every weight row by a power of two
//             (exact) chosen from the row's largest |bias| + qmax*|scale|, undone per accumulator
//             column in the epilogue.  kind::f16 wants both operands in one format, so A is
//             converted to fp16 too, each row scaled by its own power of two (undone per
//             accumulator row in the epilogue).
//   D       = float32 in tensor memory: the two accumulators fill all 512 columns, so the
//             epilogue of a tile and the main loop of the next one do not overlap (the short K
//             of the down projection pays for that)
//
// Warp roles (19 warps): 0-7 epilogue (0-3 drain the first accumulator, 4-7 the second; one TMEM lane
// quarter each, through shared memory to row-contiguous stores), 8-15 dequantisation,
// 16 TMA producer for A, 17 MMA issuer (also owns the TMEM allocation), 18 TMA producer for W.  Stages hand over through
// mbarriers; every wait is bounded by a 2 s timer after which the CTA sets a status word, drops
// out of its loops, releases its tensor memory and returns.
//
// 4-bit codes are unpacked pairwise (elements j and j+4 of a word land in one bf16x2), so a
// row's k order inside each group of eight is [0,4,1,5,2,6,3,7]; the A operand is written in
// that same order by its producer (the row gather for gate/up, the gate/up epilogue for down),
// which leaves every dot product unchanged.  No load in this file uses cluster multicast.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace b200 {

namespace {

using namespace tc;

constexpr int BM = 128, BMT = 256, BK = 64, NCOL = 256;  // BMT: rows per tile = two 128-row accumulators sharing B
// STAGES = dequantised-B stages.  (Measured alternatives in the same shared memory: two activation + four
// packed-weight stages 3-7 % slower at every batch size; two activation + three dequantised-B stages no
// different.  With few rows per expert a K block costs ~1.7 k cycles whatever the number of MMAs: the
// hand-over latency between the unpack warps and the MMA issuer, not the stage count, sets that floor.)
constexpr int STAGES = 2, W_STAGES = 2;
// BITS == 16 is the un-quantised product (gather_mm): the "packed" stage then holds a raw bf16 tile of b
// (64 k x 256 n, 32 KB) that the unpack warps transpose into the K-major operand layout; two activation
// stages instead of three pay for its size.
__host__ __device__ constexpr int a_stages(int bits) { return bits == 16 ? 2 : 3; }
constexpr int A_BYTES = BM * BK * 2;                     // 16 KB per 128-row sub-tile
constexpr int A_STAGE_BYTES = 2 * A_BYTES;               // both sub-tiles of a K block
constexpr int B_BYTES = NCOL * BK * 2;                   // 32 KB
__host__ __device__ constexpr int w_bytes(int bits) { return bits == 16 ? NCOL * BK * 2 : NCOL * 64; }  // 16 KB: 64 packed bytes of each of the 256 weight rows
constexpr int N_EPI = 256, N_DEQ = 256;
constexpr int WARP_TMA_A = (N_EPI + N_DEQ) / 32, WARP_MMA = WARP_TMA_A + 1, WARP_TMA_W = WARP_TMA_A + 2;
constexpr int N_THREADS = N_EPI + N_DEQ + 96;            // + TMA(A) warp + MMA warp + TMA(W) warp
constexpr int CS_BUFS = 4;                // column-scale buffers (tiles in flight between dequantisation and epilogue)
__host__ __device__ constexpr int ring_bytes(int bits) {
  return a_stages(bits) * A_STAGE_BYTES + STAGES * B_BYTES + W_STAGES * w_bytes(bits);
}
constexpr int STG_LD = 20;                // floats per staged row (16 + 4): 16-byte aligned, quarter-warps hit distinct banks
__host__ __device__ constexpr int smem_bytes(int bits) {
  return 1024 + ring_bytes(bits) + 512 + CS_BUFS * NCOL * 4 + (N_EPI / 32) * 32 * STG_LD * 4;
}

// kind::f16, A = B = fp16, D = f32, both operands K-major, M = 128, N = 256
constexpr uint32_t kIdesc = umma_idesc_f16(BM, NCOL);
// the same with A = B = bf16 (format 1 in both operand fields): the un-quantised product
constexpr uint32_t kIdescBf16 = kIdesc | (1u << 7) | (1u << 10);
template <int BITS>
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  umma_f16(d_tmem, adesc, bdesc, BITS == 16 ? kIdescBf16 : kIdesc, accumulate);
}

// two float32 -> packed fp16 pair (lo in the low half), round to nearest, finite overflow saturates
__device__ __forceinline__ uint32_t f16x2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float round_to_bf16(float f) { return __uint_as_float(f32_to_bf16_bits(f) << 16); }
__device__ __forceinline__ uint32_t bf16x2(float lo, float hi) { return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16); }

struct PrefillArgs {
  const uint32_t* w[2];
  const void* scales[2];
  const void* biases[2];
  const uint32_t* tile_expert;  // per row tile: expert
  const uint32_t* tile_row0;    // first sorted position of the tile
  const uint32_t* tile_rows;    // valid rows (<= 128)
  const uint32_t* n_row_tiles;  // device scalar
  const uint32_t* perm;         // sorted position -> flat assignment index
  int dst_perm;                 // out row = perm[p] instead of p
  const float* a_row_scale;     // by sorted position: the power of two each A row was divided by (null: rows are unscaled)
  const void* row_scale;        // bf16 by out row, or null
  void* out;
  const unsigned long long* out_row_addr;  // optional, by sorted position: where the row's bf16 output goes
  int out_fmt;                  // kOutBf16 / kOutF32 / kOutF16 (fp16 with saturation instead of infinities)
  int K, N;                     // reduction length, output features per matrix
  int* err;
  int debug;                    // development builds (-DB200_DEV) only: 1 = skip the dequantisation work, 2 = skip the MMAs,
                                // 32 = per-role self-timing; always 0 otherwise
  int alt;                      // 1: row tiles hold <= 128 rows and alternate between the two accumulators
};

// dequantise 8 codes of one 4-bit word -> 16 bytes of fp16 (k order [0,4,1,5,2,6,3,7]).
// OR-ing a nibble into the mantissa of 1024.0 gives 1024+q (low nibbles) or 1024+16q (nibbles
// taken in place at bits 4..7); both are brought back to q exactly before the affine step.
// (mask and magic number are register operands of ONE lop3; written as C the AND and the OR become two
// instructions with an immediate each)
__device__ __forceinline__ uint32_t and_or_b32(uint32_t a, uint32_t mask, uint32_t magic) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(magic));
  return d;
}
__device__ __forceinline__ uint4 deq_word4(uint32_t w, __half2 s2, __half2 b2) {
  const __half2 k1024 = __floats2half2_rn(1024.f, 1024.f);
  const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f), km64 = __floats2half2_rn(-64.f, -64.f);
  uint4 o;
  uint32_t* ou = &o.x;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t v = w >> (8 * h);
    uint32_t lo = and_or_b32(v, 0x000f000fu, 0x64006400u);  // (1024 + q_j,     1024 + q_{j+4}),     j = 2h
    uint32_t hi = and_or_b32(v, 0x00f000f0u, 0x64006400u);  // (1024 + 16 q_j', 1024 + 16 q_{j'+4}), j' = 2h+1
    __half2 q0 = __hsub2(*reinterpret_cast<__half2*>(&lo), k1024);
    __half2 q1 = __hfma2(*reinterpret_cast<__half2*>(&hi), k16th, km64);
    __half2 v0 = __hfma2(q0, s2, b2), v1 = __hfma2(q1, s2, b2);
    ou[2 * h] = *reinterpret_cast<uint32_t*>(&v0);
    ou[2 * h + 1] = *reinterpret_cast<uint32_t*>(&v1);
  }
  return o;
}
// dequantise 8 codes of two 8-bit words -> 16 bytes of fp16 (natural k order)
__device__ __forceinline__ uint4 deq_word8(uint32_t w0, uint32_t w1, __half2 s2, __half2 b2) {
  const __half2 k1024 = __floats2half2_rn(1024.f, 1024.f);
  uint4 o;
  uint32_t* ou = &o.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t w = j < 2 ? w0 : w1;
    int b = (j & 1) * 2;
    uint32_t m = __byte_perm(w, 0x64646464u, 0x4040 | ((b + 1) << 8) | b);  // (1024 + q_b, 1024 + q_{b+1})
    __half2 v = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&m), k1024), s2, b2);
    ou[j] = *reinterpret_cast<uint32_t*>(&v);
  }
  return o;
}

template <int BITS, int NMAT>
__global__ void __launch_bounds__(N_THREADS, 1)
grouped_qmm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w0,
                      const __grid_constant__ CUtensorMap tmap_w1, PrefillArgs p) {
  constexpr int FEAT = (NMAT == 2) ? 128 : 256;  // output features per tile
  constexpr int WPB = BK * BITS / 32;            // packed words per row per K block (8 or 16)
  constexpr int KPS = BITS == 16 ? 1 : 16 / WPB; // K blocks covered by one W stage (2 or 1)
  constexpr int CPK = BITS == 16 ? 1 : WPB / 4;  // 16-byte chunks of a row per K block (2 or 4)
  constexpr int A_STAGES = a_stages(BITS), W_BYTES = w_bytes(BITS), RING_BYTES = ring_bytes(BITS);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* a_st = smem;
  unsigned char* b_st = smem + A_STAGES * A_STAGE_BYTES;
  unsigned char* w_st = b_st + STAGES * B_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + RING_BYTES);
  // bars: b_full[4] 0.., b_empty[4] 4.., tmem_full 8/10, tmem_empty 9/11, w_full[8] 40.., w_empty[8] 48..,
  //       a_full[8] 16.., a_empty[8] 24.., then tmem base + abort flag
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 33);
  float* colscale = reinterpret_cast<float*>(smem + RING_BYTES + 512);  // [CS_BUFS][NCOL]
  float* stage_buf = colscale + CS_BUFS * NCOL;                          // N_EPI/32 warps x [32][STG_LD]
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (4 + s); };
  // accumulator barriers: [0] is the pair's (or accumulator 0's), [1] accumulator 1's in alternating mode
  auto tfull_bar = [&](int a) { return bar0 + 8u * (a ? 10 : 8); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (a ? 11 : 9); };
  const bool alt = p.alt != 0;
  auto wfull_bar = [&](int s) { return bar0 + 8u * (40 + s); };
  auto wempty_bar = [&](int s) { return bar0 + 8u * (48 + s); };
  auto afull_bar = [&](int s) { return bar0 + 8u * (16 + s); };
  auto aempty_bar = [&](int s) { return bar0 + 8u * (24 + s); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KB = p.K / BK;
  const int n_col_tiles = (p.N + FEAT - 1) / FEAT;  // the un-quantised product may end in a partial column tile
  const int G = p.K / 64;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), N_DEQ / 32);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < A_STAGES; ++s) {
      mbar_init(afull_bar(s), 1);
      mbar_init(aempty_bar(s), 1);
    }
    mbar_init(tfull_bar(0), 1);
    mbar_init(tempty_bar(0), alt ? N_EPI / 64 : N_EPI / 32);
    mbar_init(tfull_bar(1), 1);
    mbar_init(tempty_bar(1), N_EPI / 64);
    for (int w = 0; w < W_STAGES; ++w) {
      mbar_init(wfull_bar(w), 1);
      mbar_init(wempty_bar(w), N_DEQ / 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WARP_MMA) {  // whole warp: allocate all 512 tensor-memory columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = (int)(*p.n_row_tiles) * n_col_tiles;

  if (warp < N_EPI / 32) {
    // ------------------------------- epilogue -------------------------------------------
    // Warps 0-3 drain accumulator 0 (rows 0..127 of the tile), warps 4-7 accumulator 1 (rows
    // 128..255); a thread owns one accumulator row (its TMEM lane).  Results pass through a
    // per-warp staging buffer (32 rows x 16 columns, float32) so that a global store instruction
    // covers whole row segments instead of 32 different lines.
    const int sub = warp >> 2, q4 = warp & 3;
    int tphase = 0, tcount = 0;
    RoleTimer tm((p.debug & 32) && blockIdx.x == 0 && tid == 0);
    RoleTimer tm2((p.debug & 32) && blockIdx.x == 0 && tid == 0 && NMAT == 1);
    float* stg = stage_buf + warp * (32 * STG_LD);
    const int tb = alt ? sub : 0;  // which accumulator barrier pair this warp uses
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tcount) {
      // alternating mode: tile i of this CTA lives in accumulator i & 1 and is drained by that
      // accumulator's four warps while the other accumulator is being filled
      if (alt && (tcount & 1) != sub) continue;
      const int rt = tile / n_col_tiles, ct = tile % n_col_tiles;
      const float* cs = colscale + (tcount % CS_BUFS) * NCOL;
      tm.start();
      const uint32_t row0 = p.tile_row0[rt];
      const int rows = (int)p.tile_rows[rt];
      const int r = (alt ? 0 : sub * 128) + q4 * 32 + lane;  // row of the tile
      const bool row_ok = r < rows;
      const uint32_t sp = row0 + r;
      const uint32_t dst = row_ok ? (p.dst_perm ? p.perm[sp] : sp) : 0xffffffffu;  // 0xffffffff: row not stored
      const float ar = (row_ok && p.a_row_scale) ? p.a_row_scale[sp] : 1.0f;
      const unsigned long long daddr = (row_ok && p.out_row_addr) ? p.out_row_addr[sp] : 0ull;
      if (!mbar_wait(tfull_bar(tb), tphase, abort_flag)) break;
      tphase ^= 1;
      tm.stop(0);
      tm.start();
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(sub * NCOL);
      bool released = false;  // (warp-uniform) the accumulator has been handed back before the last stores
      if (alt || sub * 128 < rows) {  // (warp-uniform) this accumulator holds rows of the tile
        if constexpr (NMAT == 2) {
          // A pass covers 32 h columns: the thread computes its row's values from two 16-column loads of each
          // matrix, converts them and stages 64 bytes (chunks XOR-swizzled as in the down projection's epilogue
          // below); a store instruction covers 8 rows x 64 contiguous bytes.
          uint32_t g[16], u[16];
          tmem_ld16(lane_addr, g);
          tmem_ld16(lane_addr + 128, u);
          unsigned char* stg8 = reinterpret_cast<unsigned char*>(stg);
          const uint32_t my_row = (uint32_t)lane * 64u, my_sw = (uint32_t)(lane >> 1) & 3u;
#pragma unroll 1
          for (int c = 0; c < 128; c += 32) {
            __syncwarp();  // the previous pass's readers are done with the staging buffer
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int cc0 = c + half * 16;
              tmem_ld_wait();
              if (cc0 + 16 >= 128) {  // the last columns are in registers: the accumulator can be refilled from here on
                tc_fence_before();
                mbar_arrive_warp(tempty_bar(tb), lane);
                released = true;
              }
              float h[16];
#pragma unroll
              for (int i = 0; i < 16; i += 4) {
                const float4 cg = *reinterpret_cast<const float4*>(cs + cc0 + i);
                const float4 cu = *reinterpret_cast<const float4*>(cs + 128 + cc0 + i);
                const float cgs[4] = {cg.x, cg.y, cg.z, cg.w}, cus[4] = {cu.x, cu.y, cu.z, cu.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float gv = __uint_as_float(g[i + q]) * (cgs[q] * ar), uv = __uint_as_float(u[i + q]) * (cus[q] * ar);
                  h[i + q] = __fdividef(gv, 1.0f + __expf(-gv)) * uv;
                }
              }
              if (cc0 + 16 < 128) {  // the next accumulator columns travel while these are converted and stored
                tmem_ld16(lane_addr + cc0 + 16, g);
                tmem_ld16(lane_addr + 128 + cc0 + 16, u);
              }
              // h = bf16(silu(g) * u) is the value the down projection consumes; kOutF16 stores that same
              // value as fp16 (exact for 2^-14 <= |h| <= 65504, saturating beyond), the A-operand format of
              // the tensor-core down projection, so no conversion pass is needed between the two products
              uint32_t o[8];
#pragma unroll
              for (int g8 = 0; g8 < 2; ++g8) {
                const float* e = h + g8 * 8;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  // 4-bit consumer (down projection) reads k in [0,4,1,5,2,6,3,7] order within a group of eight
                  const float lo = (BITS == 4) ? e[q] : e[2 * q], hi = (BITS == 4) ? e[q + 4] : e[2 * q + 1];
                  o[g8 * 4 + q] = (p.out_fmt == kOutF16) ? f16x2_sat(round_to_bf16(lo), round_to_bf16(hi)) : bf16x2(lo, hi);
                }
              }
              *reinterpret_cast<uint4*>(stg8 + my_row + ((((uint32_t)half * 2u) ^ my_sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<uint4*>(stg8 + my_row + ((((uint32_t)half * 2u + 1u) ^ my_sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
            }
            __syncwarp();
            const uint32_t ch = (uint32_t)lane & 3u;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int rr = it * 8 + (lane >> 2);
              const uint32_t d = __shfl_sync(0xffffffffu, dst, rr);
              const uint4 o4 = *reinterpret_cast<const uint4*>(stg8 + rr * 64 + ((ch ^ ((uint32_t)(rr >> 1) & 3u)) << 4));
              if (d != 0xffffffffu)
                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)d * p.N + ct * FEAT + c + (int)ch * 8) = o4;
            }
          }
        } else {
          const float sc = ar * ((row_ok && p.row_scale)
                                     ? bf16_bits_to_f32(static_cast<const unsigned short*>(p.row_scale)[dst])
                                     : 1.0f);
          uint32_t v[16];
          tmem_ld16(lane_addr, v);
          if (p.out_fmt == kOutF32) {
#pragma unroll 1
            for (int c = 0; c < 256; c += 16) {
              tmem_ld_wait();
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(stg + lane * STG_LD + i) =
                    make_float4(__uint_as_float(v[i]) * sc, __uint_as_float(v[i + 1]) * sc, __uint_as_float(v[i + 2]) * sc,
                                __uint_as_float(v[i + 3]) * sc);
              if (c + 16 < 256) tmem_ld16(lane_addr + c + 16, v);
              __syncwarp();
              // 4 lanes per row (4 columns = 16 bytes each): 64 bytes per row, 8 rows per instruction
              const int c4 = (lane & 3) * 4;
              const float4 cc = *reinterpret_cast<const float4*>(cs + c + c4);
#pragma unroll
              for (int it = 0; it < 4; ++it) {
                const int rr = it * 8 + (lane >> 2);
                const uint32_t d = __shfl_sync(0xffffffffu, dst, rr);
                float4 x4 = *reinterpret_cast<const float4*>(stg + rr * STG_LD + c4);
                x4.x *= cc.x;
                x4.y *= cc.y;
                x4.z *= cc.z;
                x4.w *= cc.w;
                if (d != 0xffffffffu && ct * FEAT + c + c4 < p.N)
                  *reinterpret_cast<float4*>(static_cast<float*>(p.out) + (size_t)d * p.N + ct * FEAT + c + c4) = x4;
              }
            }
          } else {
            // 2-byte outputs: a pass covers 32 columns.  The thread scales and converts its row's values and
            // stages them as 64 bytes (16-byte chunks XOR-swizzled by (row / 2) % 4: the row-wise writes and the
            // reads below, 4 lanes per row, both touch every bank once); a store instruction then covers 8 rows x
            // 64 contiguous bytes, half as many separate segments per byte as a 16-column pass would give.
            unsigned char* stg8 = reinterpret_cast<unsigned char*>(stg);
            const uint32_t my_row = (uint32_t)lane * 64u, my_sw = (uint32_t)(lane >> 1) & 3u;
#pragma unroll 1
            for (int c = 0; c < 256; c += 32) {
              tm2.start();
              __syncwarp();  // the previous pass's readers are done with the staging buffer
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                tmem_ld_wait();
                if (c + half * 16 + 16 >= 256) {  // last columns in registers: release the accumulator now
                  tc_fence_before();
                  mbar_arrive_warp(tempty_bar(tb), lane);
                  released = true;
                }
                uint32_t o[8];
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                  const float4 cc = *reinterpret_cast<const float4*>(cs + c + half * 16 + i);
                  const float x0 = (__uint_as_float(v[i]) * sc) * cc.x, x1 = (__uint_as_float(v[i + 1]) * sc) * cc.y;
                  const float x2 = (__uint_as_float(v[i + 2]) * sc) * cc.z, x3 = (__uint_as_float(v[i + 3]) * sc) * cc.w;
                  if (p.out_fmt == kOutF16) {
                    o[i / 2] = f16x2_sat(x0, x1);
                    o[i / 2 + 1] = f16x2_sat(x2, x3);
                  } else {
                    o[i / 2] = bf16x2(x0, x1);
                    o[i / 2 + 1] = bf16x2(x2, x3);
                  }
                }
                if (c + half * 16 + 16 < 256) tmem_ld16(lane_addr + c + half * 16 + 16, v);
                *reinterpret_cast<uint4*>(stg8 + my_row + ((((uint32_t)half * 2u) ^ my_sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                *reinterpret_cast<uint4*>(stg8 + my_row + ((((uint32_t)half * 2u + 1u) ^ my_sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
              }
              __syncwarp();
              tm2.stop(1);
              tm2.start();
              const uint32_t ch = (uint32_t)lane & 3u;
              const int col = ct * FEAT + c + (int)ch * 8;
#pragma unroll
              for (int it = 0; it < 4; ++it) {
                const int rr = it * 8 + (lane >> 2);
                const uint32_t d = __shfl_sync(0xffffffffu, dst, rr);
                unsigned long long da = 0ull;
                if (p.out_row_addr) da = __shfl_sync(0xffffffffu, daddr, rr);
                const uint4 o4 = *reinterpret_cast<const uint4*>(stg8 + rr * 64 + ((ch ^ ((uint32_t)(rr >> 1) & 3u)) << 4));
                if (d != 0xffffffffu && col < p.N && !(p.out_row_addr && da == 0ull)) {
                  __nv_bfloat16* orow = p.out_row_addr ? reinterpret_cast<__nv_bfloat16*>(da)
                                                       : static_cast<__nv_bfloat16*>(p.out) + (size_t)d * p.N;
                  *reinterpret_cast<uint4*>(orow + col) = o4;
                }
              }
              tm2.stop(2);
            }
          }
        }
      }
      if (!released) {
        tc_fence_before();
        mbar_arrive_warp(tempty_bar(tb), lane);
      }
      tm.stop(1);
    }
    tm.flush(p.err + 16 + (NMAT == 1 ? 24 : 0));
    tm2.flush(p.err + 60);
  } else if (warp < (N_EPI + N_DEQ) / 32) {
    // ------------------------------- B dequantisation --------------------------------------
    const int col = tid - N_EPI;  // accumulator column = B tile row, 0..255
    const int mt = (NMAT == 2) ? (col >> 7) : 0;
    const int fcol = (NMAT == 2) ? (col & 127) : col;
    const uint32_t sw = (uint32_t)(col & 7);
    const uint32_t row_off = (uint32_t)(col >> 3) * 1024u + (uint32_t)(col & 7) * 128u;
    // W stage: two boxes of 128 rows x 64 bytes, 64-byte swizzle (16-byte chunk index ^ (row/2 % 4))
    const int bx = col >> 7, rr = col & 127;
    const uint32_t w_row_off = (uint32_t)bx * 8192u + (uint32_t)rr * 64u;
    const uint32_t wsw = (uint32_t)((rr >> 1) & 3);
    if constexpr (BITS == 16) {
      // un-quantised product: this thread transposes its column of the raw [64 k][256 n] bf16 stage into the K-major
      // operand row (natural k order, no scaling)
      int s = 0, phase = 0, tcount = 0, ws = 0, wphase = 0;
      bool dead = false;
      for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x, ++tcount) {
        colscale[(tcount % CS_BUFS) * NCOL + col] = 1.0f;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(wfull_bar(ws), wphase, abort_flag) || !mbar_wait(empty_bar(s), phase ^ 1, abort_flag)) {
            dead = true;
            break;
          }
          const unsigned short* src = reinterpret_cast<const unsigned short*>(w_st + (size_t)ws * W_BYTES) + col;
          unsigned char* dst = b_st + (size_t)s * B_BYTES + row_off;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t lo = src[(c * 8 + 2 * q) * NCOL], hi = src[(c * 8 + 2 * q + 1) * NCOL];
              v[q] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4*>(dst + (((uint32_t)c ^ sw) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_arrive_warp(full_bar(s), lane);
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
          mbar_arrive_warp(wempty_bar(ws), lane);
          if (++ws == W_STAGES) {
            ws = 0;
            wphase ^= 1;
          }
        }
      }
    } else {
    int s = 0, phase = 0, tcount = 0, ws = 0, wphase = 0;
    constexpr float kQmax = (BITS == 4) ? 15.f : 255.f;
    RoleTimer tm((p.debug & 32) && blockIdx.x == 0 && tid == N_EPI);
    const long long t_begin = B200_DEV_CLOCK();
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tcount) {
      const int rt = tile / n_col_tiles, ct = tile % n_col_tiles;
      const int e = (int)p.tile_expert[rt];
      const size_t wr = (size_t)e * p.N + (size_t)ct * FEAT + fcol;
      const unsigned short* sp = static_cast<const unsigned short*>(p.scales[mt]) + wr * G;
      const unsigned short* bp = static_cast<const unsigned short*>(p.biases[mt]) + wr * G;
      // power-of-two normalisation of this weight row for fp16: largest |w_hat| lands in [2^13, 2^14)
      // (all loads of the row's scales and biases are issued before the first use: one round trip)
      float mx = 0.f;
      const bool sb_vec = (G & 3) == 0;
      uint2 s_first = make_uint2(0, 0), b_first = s_first;
      if (sb_vec) {
        for (int g0 = 0; g0 < G; g0 += 32) {
          uint2 sv[8], bv[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const bool ok = g0 + 4 * q < G;
            sv[q] = ok ? __ldg(reinterpret_cast<const uint2*>(sp + g0) + q) : make_uint2(0, 0);
            bv[q] = ok ? __ldg(reinterpret_cast<const uint2*>(bp + g0) + q) : make_uint2(0, 0);
          }
          if (g0 == 0) {
            s_first = sv[0];
            b_first = bv[0];
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t su[2] = {sv[q].x, sv[q].y}, bu[2] = {bv[q].x, bv[q].y};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              mx = fmaxf(mx, fabsf(__uint_as_float(bu[j] << 16)) + kQmax * fabsf(__uint_as_float(su[j] << 16)));
              mx = fmaxf(mx, fabsf(__uint_as_float(bu[j] & 0xffff0000u)) + kQmax * fabsf(__uint_as_float(su[j] & 0xffff0000u)));
            }
          }
        }
      } else {
#pragma unroll 4
        for (int g = 0; g < G; ++g)
          mx = fmaxf(mx, fabsf(bf16_bits_to_f32(__ldg(bp + g))) + kQmax * fabsf(bf16_bits_to_f32(__ldg(sp + g))));
      }
      // pull the first lines of the next tile's scales and biases into L2 meanwhile
      {
        const int ntile = tile + gridDim.x;
        if (ntile < total_tiles) {
          const int nrt = ntile / n_col_tiles, nct = ntile % n_col_tiles;
          const size_t nwr = (size_t)p.tile_expert[nrt] * p.N + (size_t)nct * FEAT + fcol;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const unsigned short*>(p.scales[mt]) + nwr * G));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const unsigned short*>(p.biases[mt]) + nwr * G));
        }
      }
      // exponent of mx straight from its bits (mx is a finite non-negative float here)
      int ex = 0;
      if (mx > 0.f && mx < 3.0e38f) ex = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 127 - 13;
      ex = max(-100, min(100, ex));
      const float down_f = __uint_as_float((uint32_t)(127 - ex) << 23);
      colscale[(tcount % CS_BUFS) * NCOL + col] = __uint_as_float((uint32_t)(127 + ex) << 23);
      // scale / bias: four K blocks' worth per 8-byte load, fetched one chunk ahead
      uint2 s_cur = make_uint2(0, 0), b_cur = s_cur, s_nxt = s_first, b_nxt = b_first;
      bool dead = false;
      for (int kb = 0; kb < KB; ++kb) {
        const int kin = kb % KPS;
        tm.start();
        if (kin == 0 && !mbar_wait(wfull_bar(ws), wphase, abort_flag)) {
          dead = true;
          break;
        }
        unsigned short cs, cb;
        if (sb_vec) {
          if ((kb & 3) == 0) {
            s_cur = s_nxt;
            b_cur = b_nxt;
            if (kb + 4 < G) {
              s_nxt = __ldg(reinterpret_cast<const uint2*>(sp + kb + 4));
              b_nxt = __ldg(reinterpret_cast<const uint2*>(bp + kb + 4));
            }
          }
          const uint32_t sw2 = (kb & 2) ? s_cur.y : s_cur.x, bw2 = (kb & 2) ? b_cur.y : b_cur.x;
          cs = (unsigned short)((kb & 1) ? (sw2 >> 16) : (sw2 & 0xffffu));
          cb = (unsigned short)((kb & 1) ? (bw2 >> 16) : (bw2 & 0xffffu));
        } else {
          cs = __ldg(sp + kb);
          cb = __ldg(bp + kb);
        }
        if (!mbar_wait(empty_bar(s), phase ^ 1, abort_flag)) {
          dead = true;
          break;
        }
        tm.stop(0);
        tm.start();
#ifdef B200_DEV
        if (p.debug & 1) {
          mbar_arrive_warp(full_bar(s), lane);
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
          if (kin == KPS - 1 || kb == KB - 1) {
            mbar_arrive_warp(wempty_bar(ws), lane);
            if (++ws == W_STAGES) {
              ws = 0;
              wphase ^= 1;
            }
          }
          continue;
        }
#endif
        const __half2 s2 = __float2half2_rn(bf16_bits_to_f32(cs) * down_f);
        const __half2 b2 = __float2half2_rn(bf16_bits_to_f32(cb) * down_f);
        const unsigned char* wsrc = w_st + (size_t)ws * W_BYTES + w_row_off;
        uint4 cur[CPK];
#pragma unroll
        for (int q = 0; q < CPK; ++q)
          cur[q] = *reinterpret_cast<const uint4*>(wsrc + (((uint32_t)(kin * CPK + q) ^ wsw) << 4));
        unsigned char* dst = b_st + (size_t)s * B_BYTES + row_off;
        const uint32_t* cw = &cur[0].x;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 o;
          if constexpr (BITS == 4)
            o = deq_word4(cw[c], s2, b2);
          else
            o = deq_word8(cw[2 * c], cw[2 * c + 1], s2, b2);
          *reinterpret_cast<uint4*>(dst + (((uint32_t)c ^ sw) << 4)) = o;
        }
        tm.stop(1);
        tm.start();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive_warp(full_bar(s), lane);
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
        if (kin == KPS - 1 || kb == KB - 1) {  // this warp is done with the W stage
          mbar_arrive_warp(wempty_bar(ws), lane);
          if (++ws == W_STAGES) {
            ws = 0;
            wphase ^= 1;
          }
        }
        tm.stop(2);
      }
      if (dead) break;
    }
    tm.total(t_begin);
    tm.flush(p.err + 20 + (NMAT == 1 ? 24 : 0));
    }
  } else if (warp == WARP_TMA_A) {
    // ------------------------------- TMA producer (A) ---------------------------------------
    if (lane == 0) {
      int s = 0, phase = 0;
      bool dead = false;
      RoleTimer tm((p.debug & 32) && blockIdx.x == 0);
      const long long t_begin = B200_DEV_CLOCK();
      for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
        const int rt = tile / n_col_tiles;
        const int row0 = (int)p.tile_row0[rt];
        const int n_sub = (!alt && (int)p.tile_rows[rt] > BM) ? 2 : 1;
        for (int kb = 0; kb < KB; ++kb) {
          tm.start();
          if (!mbar_wait(aempty_bar(s), phase ^ 1, abort_flag)) {
            dead = true;
            break;
          }
          tm.stop(0);
          mbar_arrive_expect_tx(afull_bar(s), n_sub * A_BYTES);
          const uint32_t dst = smem_u32(a_st + (size_t)s * A_STAGE_BYTES);
          tma_load_2d(dst, &tmap_a, afull_bar(s), kb * BK, row0);
          if (n_sub == 2) tma_load_2d(dst + A_BYTES, &tmap_a, afull_bar(s), kb * BK, row0 + BM);
          if (++s == A_STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
      }
      tm.total(t_begin);
      tm.flush(p.err + 24 + (NMAT == 1 ? 24 : 0));
    }
    __syncwarp();
  } else if (warp == WARP_MMA) {
    // ------------------------------- MMA issuer ----------------------------------------------
    if (lane == 0) {
      int s = 0, phase = 0, sa = 0, aphase = 0, tcount = 0;
      int tph[2] = {0, 0};
      bool dead = false;
      RoleTimer tm((p.debug & 32) && blockIdx.x == 0);
      const long long t_begin = B200_DEV_CLOCK();
      for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x, ++tcount) {
        const int rt = tile / n_col_tiles;
        const int n_sub = (!alt && (int)p.tile_rows[rt] > BM) ? 2 : 1;
        const int acc = alt ? (tcount & 1) : 0;
        const uint32_t d_addr = tmem_base + (uint32_t)(acc * NCOL);
        tm.start();
        if (!mbar_wait(tempty_bar(acc), tph[acc] ^ 1, abort_flag)) break;
        tph[acc] ^= 1;
        tm.stop(2);
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb) {
          tm.start();
          if (!mbar_wait(afull_bar(sa), aphase, abort_flag)) {
            dead = true;
            break;
          }
          tm.stop(0);
          tm.start();
          if (!mbar_wait(full_bar(s), phase, abort_flag)) {
            dead = true;
            break;
          }
          tm.stop(1);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(a_st + (size_t)sa * A_STAGE_BYTES), b_addr = smem_u32(b_st + (size_t)s * B_BYTES);
#ifdef B200_DEV
          if (!(p.debug & 2))
#endif
          {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t bd = umma_desc(b_addr + k * 32);
              umma_bf16<BITS>(d_addr, umma_desc(a_addr + k * 32), bd, (kb | k) ? 1u : 0u);
              if (n_sub == 2) umma_bf16<BITS>(tmem_base + NCOL, umma_desc(a_addr + A_BYTES + k * 32), bd, (kb | k) ? 1u : 0u);
            }
          }
          umma_commit(aempty_bar(sa));  // both stages are free once these MMAs have read them
          umma_commit(empty_bar(s));
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
          if (++sa == A_STAGES) {
            sa = 0;
            aphase ^= 1;
          }
        }
        if (dead) break;
        umma_commit(tfull_bar(acc));  // accumulators complete
      }
      tm.total(t_begin);
      tm.flush(p.err + 28 + (NMAT == 1 ? 24 : 0));
    }
    __syncwarp();
  } else {
    // ------------------------------- TMA producer (packed weights) ---------------------------
    if (lane == 0) {
      int ws = 0, wphase = 0;
      bool dead = false;
      const int n_wst = (KB + KPS - 1) / KPS;
      RoleTimer tm((p.debug & 32) && blockIdx.x == 0);
      const long long t_begin = B200_DEV_CLOCK();
      for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
        const int rt = tile / n_col_tiles, ct = tile % n_col_tiles;
        const int row_base = (int)p.tile_expert[rt] * p.N + ct * FEAT;
        for (int wk = 0; wk < n_wst; ++wk) {
          tm.start();
          if (!mbar_wait(wempty_bar(ws), wphase ^ 1, abort_flag)) {
            dead = true;
            break;
          }
          tm.stop(0);
          mbar_arrive_expect_tx(wfull_bar(ws), W_BYTES);
          const uint32_t dst = smem_u32(w_st + (size_t)ws * W_BYTES);
          if constexpr (BITS == 16) {  // raw bf16 tile of b[e]: 64 k rows x 256 n (columns beyond N read as zero)
            tma_load_2d(dst, &tmap_w0, wfull_bar(ws), ct * FEAT, (int)p.tile_expert[rt] * p.K + wk * BK);
          } else if constexpr (NMAT == 2) {
            tma_load_2d(dst, &tmap_w0, wfull_bar(ws), wk * 16, row_base);
            tma_load_2d(dst + 8192, &tmap_w1, wfull_bar(ws), wk * 16, row_base);
          } else {
            tma_load_2d(dst, &tmap_w0, wfull_bar(ws), wk * 16, row_base);
            tma_load_2d(dst + 8192, &tmap_w0, wfull_bar(ws), wk * 16, row_base + 128);
          }
          if (++ws == W_STAGES) {
            ws = 0;
            wphase ^= 1;
          }
        }
      }
      tm.total(t_begin);
      tm.flush(p.err + 32 + (NMAT == 1 ? 24 : 0));
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
  if (warp == WARP_MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
}

// ---- helpers: row-tile map and the permuted row gather ----------------------------------------
__global__ void __launch_bounds__(256) build_row_tiles_kernel(const uint32_t* __restrict__ counts,
                                                              const uint32_t* __restrict__ offsets, int E,
                                                              uint32_t* __restrict__ tile_expert,
                                                              uint32_t* __restrict__ tile_row0,
                                                              uint32_t* __restrict__ tile_rows,
                                                              uint32_t* __restrict__ n_row_tiles, uint32_t bmt) {
  __shared__ uint32_t pre[257];
  const int e = threadIdx.x;
  const uint32_t c = (e < E) ? counts[e] : 0u;
  const uint32_t nt = (c + bmt - 1) / bmt;
  pre[e + 1] = nt;
  if (e == 0) pre[0] = 0;
  __syncthreads();
  if (e == 0) {
    for (int i = 1; i <= 256; ++i) pre[i] += pre[i - 1];
    *n_row_tiles = pre[256];
  }
  __syncthreads();
  if (e < E) {
    const uint32_t base = pre[e], o = offsets[e];
    for (uint32_t i = 0; i < nt; ++i) {
      tile_expert[base + i] = (uint32_t)e;
      tile_row0[base + i] = o + i * bmt;
      tile_rows[base + i] = min(bmt, c - i * bmt);
    }
  }
}

// A-operand preparation, one warp per row: xs[p, :] = fp16( x[src(p), :] * 2^-e_p ) where 2^e_p
// (written to row_scale[p]) brings the row's largest magnitude into [2^14, 2^15); optionally each
// aligned group of eight elements is stored as [0,4,1,5,2,6,3,7] (the order 4-bit codes unpack in).
// The scaling is exact (bf16 has fewer significant bits than fp16) unless an element is more
// than 2^28 below the row maximum.
__global__ void __launch_bounds__(256) prepare_rows_kernel(const uint4* __restrict__ x, const uint32_t* __restrict__ perm,
                                                           const uint32_t* __restrict__ src_map, int src_div, int64_t n_rows,
                                                           const uint32_t* __restrict__ n_rows_dev, int vec_per_row,
                                                           int permute8, uint4* __restrict__ xs,
                                                           float* __restrict__ row_scale) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  // n_rows is the host's bound; the number of rows that exist may live on the device (expert-parallel exchange)
  if (r >= n_rows || (n_rows_dev && r >= (int64_t)*n_rows_dev)) return;
  // source row of sorted position r: r itself, src_map[r], perm[r] / src_div, or src_map[perm[r]]
  uint32_t a = (uint32_t)r;
  if (perm) {
    a = perm[r];
    if ((int64_t)a >= n_rows) return;  // not an assignment of this call (never written by the sort): no row to read
  }
  const uint32_t src = !perm ? (src_map ? src_map[r] : (uint32_t)r) : (src_map ? src_map[a] : a / (uint32_t)src_div);
  const uint4* xr = x + (size_t)src * vec_per_row;
  uint32_t mxbits = 0;  // max over |x| as bf16 bit patterns (monotonic for non-negative floats)
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
  for (int c = lane; c < vec_per_row; c += 32) {
    const uint4 v = __ldg(xr + c);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    uint32_t hh[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __half2 h2 = __floats2half2_rn(__uint_as_float(u[q] << 16) * f, __uint_as_float(u[q] & 0xffff0000u) * f);
      hh[q] = *reinterpret_cast<uint32_t*>(&h2);
    }
    uint4 o = make_uint4(hh[0], hh[1], hh[2], hh[3]);
    if (permute8) {
      o.x = __byte_perm(hh[0], hh[2], 0x5410);
      o.y = __byte_perm(hh[0], hh[2], 0x7632);
      o.z = __byte_perm(hh[1], hh[3], 0x5410);
      o.w = __byte_perm(hh[1], hh[3], 0x7632);
    }
    xs[(size_t)r * vec_per_row + c] = o;
  }
}

}  // namespace

size_t prefill_tile_words(int64_t rows, int E) { return (size_t)(rows / BM + E + 1); }  // enough for 128-row tiles

bool prefill_shape_ok(int K, int N, int nmat) { return K % 64 == 0 && N % (nmat == 2 ? 128 : 256) == 0; }

int launch_build_row_tiles(const uint32_t* counts, const uint32_t* offsets, int E, uint32_t* tile_expert,
                           uint32_t* tile_row0, uint32_t* tile_rows, uint32_t* n_row_tiles, int rows_per_tile,
                           cudaStream_t st) {
  build_row_tiles_kernel<<<1, 256, 0, st>>>(counts, offsets, E, tile_expert, tile_row0, tile_rows, n_row_tiles,
                                            (uint32_t)rows_per_tile);
  return 0;
}

int launch_prepare_rows(const void* x, const uint32_t* perm, const uint32_t* src_map, int src_div, int64_t n_rows,
                        const uint32_t* n_rows_dev, int K, int permute8, void* xs, float* row_scale, cudaStream_t st) {
  if (n_rows == 0) return 0;
  prepare_rows_kernel<<<cdiv(n_rows, 8), 256, 0, st>>>(static_cast<const uint4*>(x), perm, src_map, src_div, n_rows, n_rows_dev,
                                                       K / 8, permute8, static_cast<uint4*>(xs), row_scale);
  return 0;
}

// a: activations [rows, K] fp16 (rows scaled by 1/a_row_scale) in the k order the weights are unpacked in.
int launch_grouped_qmm_tc(const void* a, const float* a_row_scale, int64_t rows, const GroupedArgs& g, int nmat, int bits, const uint32_t* tile_expert,
                          const uint32_t* tile_row0, const uint32_t* tile_rows, const uint32_t* n_row_tiles, int E,
                          bool alternate, int* err, cudaStream_t st) {
  if (rows == 0) return 0;
  B200_REQUIRE(!alternate || nmat == 1, "alternating accumulators are for single-matrix products");
  B200_REQUIRE(prefill_shape_ok(g.K, g.N, nmat), "shape not supported by the tensor-core path");
  EncodeTiledFn enc = encode_fn();
  B200_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap tmap;
  cuuint64_t dims[2] = {(cuuint64_t)g.K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)g.K * 2};
  cuuint32_t box[2] = {BK, BM};
  cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(a), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (the activation buffer must be 16-byte aligned)");
  // packed weights as [E*N rows, K*bits/32 words] uint32; one box = 128 rows x 64 bytes
  CUtensorMap tmap_w[2];
  for (int i = 0; i < nmat; ++i) {
    cuuint64_t wd[2] = {(cuuint64_t)g.K * bits / 32, (cuuint64_t)E * g.N};
    cuuint64_t ws_[1] = {(cuuint64_t)g.K * bits / 8};
    cuuint32_t wb[2] = {16, 128};
    cr = enc(&tmap_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(g.w[i]), wd, ws_, wb, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for the packed weights (16-byte alignment required)");
  }
  if (nmat == 1) tmap_w[1] = tmap_w[0];

  PrefillArgs p{};
  for (int i = 0; i < 2; ++i) {
    p.w[i] = g.w[i];
    p.scales[i] = g.scales[i];
    p.biases[i] = g.biases[i];
  }
  p.tile_expert = tile_expert;
  p.tile_row0 = tile_row0;
  p.tile_rows = tile_rows;
  p.n_row_tiles = n_row_tiles;
  p.perm = g.perm;
  p.dst_perm = g.dst_perm;
  p.a_row_scale = a_row_scale;
  p.row_scale = g.row_scale;
  p.out = g.out;
  p.out_row_addr = g.out_row_addr;
  p.out_fmt = g.out_f32 ? kOutF32 : (g.out_f16 ? kOutF16 : kOutBf16);
  p.K = g.K;
  p.N = g.N;
  p.err = err;
  p.alt = alternate ? 1 : 0;
#ifdef B200_DEV
  {
    static const int dbg = [] { const char* v = getenv("B200_TC_DEBUG"); return v ? atoi(v) : 0; }();
    p.debug = dbg;
  }
#endif
  const int n_sm = current_sm_count();
  const int feat = nmat == 2 ? 128 : 256;
  const int64_t max_tiles = (int64_t)prefill_tile_words(rows, E) * (g.N / feat);
  const int grid = (int)(max_tiles < n_sm ? max_tiles : n_sm);

#define B200_TC_LAUNCH(BITSV, NMATV)                                                                          \
  do {                                                                                                        \
    auto kern = grouped_qmm_tc_kernel<BITSV, NMATV>;                                                          \
    static DynSmemCache attr;                                                                                 \
    B200_CUDA(ensure_dyn_smem(kern, smem_bytes(BITSV), attr));                                                \
    kern<<<grid, N_THREADS, smem_bytes(BITSV), st>>>(tmap, tmap_w[0], tmap_w[1], p);                              \
  } while (0)
  if (bits == 4 && nmat == 2)
    B200_TC_LAUNCH(4, 2);
  else if (bits == 4 && nmat == 1)
    B200_TC_LAUNCH(4, 1);
  else if (bits == 8 && nmat == 2)
    B200_TC_LAUNCH(8, 2);
  else if (bits == 8 && nmat == 1)
    B200_TC_LAUNCH(8, 1);
  else
    B200_FAIL("bits must be 4 or 8");
#undef B200_TC_LAUNCH
  return 0;
}

// Un-quantised grouped product on the same kernel (gather_mm, mlx-rs/src/ops/arithmetic.rs:1568-1632): rows of
// a_sorted [rows, K] bf16 grouped by matrix, b [Bb, K, N] bf16 row-major, out[perm[p], :] = a_sorted[p, :] . b[matrix of p].
// K % 64 == 0 and N % 8 == 0.
int launch_gather_mm_tc(const void* a_sorted, int64_t rows, const void* b, int Bb, int K, int N, const uint32_t* perm, void* out,
                        const uint32_t* tile_expert, const uint32_t* tile_row0, const uint32_t* tile_rows,
                        const uint32_t* n_row_tiles, int* err, cudaStream_t st) {
  if (rows == 0) return 0;
  B200_REQUIRE(K % 64 == 0 && N % 8 == 0, "shape not supported by the tensor-core path");
  EncodeTiledFn enc = encode_fn();
  B200_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap tmap_a, tmap_b;
  cuuint32_t estr[2] = {1, 1};
  {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {BK, BM};
    CUresult cr = enc(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a_sorted), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (the activation buffer must be 16-byte aligned)");
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)Bb * K};
    cuuint64_t strides[1] = {(cuuint64_t)N * 2};
    cuuint32_t box[2] = {NCOL, BK};
    CUresult cr = enc(&tmap_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(b), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for b (16-byte alignment required)");
  }
  PrefillArgs p{};
  p.tile_expert = tile_expert;
  p.tile_row0 = tile_row0;
  p.tile_rows = tile_rows;
  p.n_row_tiles = n_row_tiles;
  p.perm = perm;
  p.dst_perm = perm ? 1 : 0;
  p.out = out;
  p.out_fmt = kOutBf16;
  p.K = K;
  p.N = N;
  p.err = err;
  p.alt = 0;  // 256-row tiles: both accumulators share every transposed stage of b
  const int n_sm = current_sm_count();
  const int64_t max_tiles = (int64_t)prefill_tile_words(rows, Bb) * ((N + NCOL - 1) / NCOL);
  const int grid = (int)(max_tiles < n_sm ? max_tiles : n_sm);
  auto kern = grouped_qmm_tc_kernel<16, 1>;
  static DynSmemCache attr;
  B200_CUDA(ensure_dyn_smem(kern, smem_bytes(16), attr));
  kern<<<grid, N_THREADS, smem_bytes(16), st>>>(tmap_a, tmap_b, tmap_b, p);
  return 0;
}

}  // namespace b200

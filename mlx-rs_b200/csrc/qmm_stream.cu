// Grouped quantized expert GEMM for the memory-bound (decode) regime, second generation:
// persistent CTAs, packed weights streamed by TMA through a deep shared-memory ring, integer
// codes fed to mma.sync as exact fp16 values, affine scale/bias folded per group in float32.
//
// Same contract as qmm_decode.cu (gather_qmm with sorted rows,
// mlx-rs/src/ops/quantization.rs:160-230, SiLU-gate or routing-weight epilogue fused), for 4-bit
// or 8-bit codes, group 64, K a multiple of 256, N a multiple of the feature block.  Measured on
// B200 it matches the first-generation kernel (64.6 vs 69.3 us for gate+up at 16 tokens, 114 vs
// 106 us at 64 tokens of the 128-expert shape) without beating it: both end up bound by the
// instructions spent per packed weight, not by memory.  It is therefore selectable
// (B200_QMM_STREAM) but not the default.  What it does differently from the first kernel:
//
//  * weights no longer travel through per-thread global loads.  One producer thread issues TMA
//    tile loads (128 packed bytes x 128 weight rows = 16 KB per stage, 128-byte swizzle) into a
//    ring of RING stages, running ahead across work items; the eight compute warps only ever
//    wait on shared-memory barriers, so HBM latency is covered by ~100 KB in flight per SM.
//  * 4-bit codes are turned into fp16 with ONE logic op per pair: OR-ing a nibble into the
//    mantissa of 1024.0 gives 1024+q for nibbles at bits 0..3 and 1024+16q for nibbles taken in
//    place at bits 4..7.  The factor 16 is undone on the other operand (odd k positions of the
//    staged activations hold x/16) and the 1024 offsets are cancelled by starting every group's
//    accumulator at -(1024*sum_even(x) + 64*sum_odd(x)), a per-(token, group) constant computed
//    while the activations are staged.  Per group the float32 accumulator then holds
//    sum_k q_k x_k, folded as  total += scale*acc + bias*sum_k(x_k).
//  * a warp's m16 tile pairs 8 gate rows with the 8 up rows of the same features, so
//    silu(gate)*up happens in registers.
//
// Activations are staged per (expert, pass of up to 8*NT rows) as fp16, every row scaled by a
// power of two that brings its largest magnitude into [2^10, 2^11) (exact; undone in the
// epilogue), in the k order the unpacking produces.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

namespace {

constexpr int WROWS = 128;                 // weight rows per stage (NMAT = 2: 64 gate + 64 up)
constexpr int STAGE_BYTES = WROWS * 128;   // 16 KB
constexpr int N_COMPUTE = 256;             // 8 compute warps
constexpr int N_THREADS_S = N_COMPUTE + 32;  // + producer warp
constexpr uint64_t kWaitNs = 2000000000ull;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t gtimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait (2 s): false when the abort flag is up or the limit has passed.
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 31u) == 31u) {
      if (*abort_flag) return false;
      uint64_t now = gtimer();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
// 1-D bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16)
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
// D = A*B + C with separate C (read) and D (written) registers
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1, float c0, float c1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void mma_f16_16816_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct StreamArgs {
  const void* x;             // bf16 source rows [*, K]
  const void* scales[2];     // bf16 [E, N, K/64]
  const void* biases[2];
  const uint32_t* offsets;   // [E+1]
  const uint32_t* active;    // experts that own rows
  const uint32_t* n_active;  // device scalar
  const uint32_t* perm;
  const uint32_t* src_map;
  int src_mode, src_div, dst_perm;
  const void* row_scale;     // bf16 by out row, or null
  void* out;
  int out_f32;
  int K, N;
  int* err;
  int debug;                 // development: bit 5 = CTA 0 writes per-role cycle counts to err[16..]
};


constexpr int MAX_RING = 10;

struct STimer {
  long long acc[4] = {0, 0, 0, 0};
  long long t0 = 0;
  bool on;
  __device__ explicit STimer(bool e) : on(e) {}
  __device__ __forceinline__ void start() {
    if (on) t0 = clock64();
  }
  __device__ __forceinline__ void stop(int i) {
    if (on) acc[i] += clock64() - t0;
  }
  __device__ void flush(int* dst) {
    if (on)
      for (int i = 0; i < 4; ++i) dst[i] = (int)(acc[i] >> 10);
  }
};

template <int BITS, int NMAT, int NT>
__global__ void __launch_bounds__(N_THREADS_S, 1)
grouped_qmm_stream_kernel(const __grid_constant__ CUtensorMap tmap_w0, const __grid_constant__ CUtensorMap tmap_w1,
                          StreamArgs p, int ring) {
  constexpr int FB = (NMAT == 2) ? 64 : 128;  // output features per work item
  constexpr int GPS = (BITS == 4) ? 4 : 2;    // quantisation groups per stage (128 packed bytes per row)
  constexpr int ROWS = 8 * NT;                // activation rows per pass
  const int K = p.K, N = p.N, G = K / 64;
  const int XS = 2 * K + 16;                  // bytes per staged row (+16: the two rows of a lane pair use distinct banks)
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* w_ring = smem;
  unsigned char* xs = smem + (size_t)ring * STAGE_BYTES;
  float* negc = reinterpret_cast<float*>(xs + (size_t)ROWS * XS);  // [G][ROWS]
  float* xsum = negc + G * ROWS;                                     // [G][ROWS]
  float* rowsc = xsum + G * ROWS;                                    // [ROWS]
  uint64_t* bars = reinterpret_cast<uint64_t*>(rowsc + ROWS + 2);    // full[MAX_RING], empty[MAX_RING] (8-byte aligned: ROWS even)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * MAX_RING + 5);
  const uint32_t xbar = s_u32(bars + 2 * MAX_RING);  // compute-warp rendezvous around the activation staging
  // scale/bias slots: per work item the four (NMAT = 2) or two contiguous blocks [rows][G] of bf16
  // scales and biases of the item's weight rows, fetched by bulk copies one item ahead
  const uint32_t sbfull0 = s_u32(bars + 2 * MAX_RING + 1), sbempty0 = s_u32(bars + 2 * MAX_RING + 3);
  const int SB_BLOCK = (WROWS / NMAT) * G * 2;       // bytes of one block
  const int SB_SLOT = 2 * NMAT * SB_BLOCK;           // scales + biases of every matrix
  unsigned char* sb_base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(bars + 2 * MAX_RING + 8) + 15) & ~uintptr_t(15));
  const uint32_t bar0 = s_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (MAX_RING + s); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < ring; ++s) {
      bar_init(full_bar(s), 1);
      bar_init(empty_bar(s), N_COMPUTE / 32);
    }
    bar_init(xbar, N_COMPUTE / 32);
    for (int i = 0; i < 2; ++i) {
      bar_init(sbfull0 + 8u * i, 1);
      bar_init(sbempty0 + 8u * i, N_COMPUTE / 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int nfb = N / FB;
  const int n_items = (int)(*p.n_active) * nfb;
  const int i0 = (int)((long long)blockIdx.x * n_items / gridDim.x);
  const int i1 = (int)((long long)(blockIdx.x + 1) * n_items / gridDim.x);
  const int n_st = G / GPS;  // stages per pass

  if (warp == N_COMPUTE / 32) {
    // ------------------------------- producer: TMA weight stream ----------------------------
    if (lane == 0) {
      int s = 0, ph = 0, sl = 0, slph = 0;
      bool dead = false;
      STimer tm((p.debug & 32) && blockIdx.x == 0);
      const long long tb = clock64();
      // units are visited run by run (a run = this CTA's consecutive items of one expert), pass by
      // pass inside a run, item by item inside a pass: the activation rows staged for a pass
      // then serve every item of the run
      for (int it0 = i0; it0 < i1 && !dead;) {
        tm.start();
        const int ea = it0 / nfb;
        const int run_end = min(i1, (ea + 1) * nfb);
        const int e = (int)p.active[ea];
        const int m = (int)(p.offsets[e + 1] - p.offsets[e]);
        tm.stop(2);
        for (int p0 = 0; p0 < m && !dead; p0 += ROWS) {
          for (int item = it0; item < run_end && !dead; ++item) {
            const int row_base = e * N + (item % nfb) * FB;
            {  // scales and biases of this item's rows -> slot sl
              tm.start();
              if (!bar_wait(sbempty0 + 8u * sl, slph ^ 1, abort_flag)) {
                dead = true;
                break;
              }
              tm.stop(1);
              bar_expect_tx(sbfull0 + 8u * sl, (uint32_t)SB_SLOT);
              const uint32_t dst = s_u32(sb_base + (size_t)sl * SB_SLOT);
#pragma unroll
              for (int mt = 0; mt < NMAT; ++mt) {
                const size_t off = (size_t)row_base * G * 2;
                bulk_copy(dst + (2 * mt) * SB_BLOCK, static_cast<const unsigned char*>(p.scales[mt]) + off, SB_BLOCK, sbfull0 + 8u * sl);
                bulk_copy(dst + (2 * mt + 1) * SB_BLOCK, static_cast<const unsigned char*>(p.biases[mt]) + off, SB_BLOCK, sbfull0 + 8u * sl);
              }
              if (++sl == 2) {
                sl = 0;
                slph ^= 1;
              }
            }
            for (int st = 0; st < n_st; ++st) {
              tm.start();
              if (!bar_wait(empty_bar(s), ph ^ 1, abort_flag)) {
                dead = true;
                break;
              }
              tm.stop(0);
              bar_expect_tx(full_bar(s), STAGE_BYTES);
              const uint32_t dst = s_u32(w_ring + (size_t)s * STAGE_BYTES);
              if constexpr (NMAT == 2) {
                tma_2d(dst, &tmap_w0, full_bar(s), st * 32, row_base);
                tma_2d(dst + STAGE_BYTES / 2, &tmap_w1, full_bar(s), st * 32, row_base);
              } else {
                tma_2d(dst, &tmap_w0, full_bar(s), st * 32, row_base);
              }
              if (++s == ring) {
                s = 0;
                ph ^= 1;
              }
            }
          }
        }
        it0 = run_end;
      }
      tm.acc[3] = clock64() - tb;
      tm.flush(p.err + 16);
    }
    __syncwarp();
  } else {
    // ------------------------------- compute warps ------------------------------------------
    const int gq = lane >> 2, t = lane & 3;
    // smem rows of this thread's two weight rows, and their output features
    const int rA = (NMAT == 2) ? (8 * warp + gq) : (16 * warp + gq);
    const int rB = (NMAT == 2) ? (64 + 8 * warp + gq) : (16 * warp + gq + 8);
    const int fA = (NMAT == 2) ? (8 * warp + gq) : rA, fB = (NMAT == 2) ? fA : rB;  // feature inside the item
    const uint32_t offA = (uint32_t)rA * 128u, offB = (uint32_t)rB * 128u;
    const uint32_t swA = (uint32_t)(rA & 7), swB = (uint32_t)(rB & 7);
    int s = 0, ph = 0;
    int staged_e = -1, staged_p0 = -1, xph = 0, sl = 0, slph = 0;
    STimer tm((p.debug & 32) && blockIdx.x == 0 && tid == 0);
    const long long tb = clock64();
    bool dead = false;
    // rendezvous of the eight compute warps on an mbarrier, with the same bounded wait as every
    // other wait of the kernel (a plain bar.sync could not give up)
    auto rendezvous = [&]() -> bool {
      __syncwarp();
      if (lane == 0) bar_arrive(xbar);
      const bool ok = bar_wait(xbar, xph, abort_flag);
      xph ^= 1;
      return ok;
    };
    for (int it0 = i0; it0 < i1 && !dead;) {
     const int ea = it0 / nfb;
     const int run_end = min(i1, (ea + 1) * nfb);
     const int e = (int)p.active[ea];
     const uint32_t seg0 = p.offsets[e];
     const int m = (int)(p.offsets[e + 1] - seg0);
     for (int p0 = 0; p0 < m && !dead; p0 += ROWS) {
      for (int item = it0; item < run_end && !dead; ++item) {
      const int fb = item % nfb;
      // this item's scales / biases: blocks [scales0, biases0, (scales1, biases1)] of [rows][G] bf16 in slot sl
      tm.start();
      if (!bar_wait(sbfull0 + 8u * sl, slph, abort_flag)) {
        dead = true;
        break;
      }
      tm.stop(2);
      const unsigned char* slot = sb_base + (size_t)sl * SB_SLOT;
      const unsigned short* sA = reinterpret_cast<const unsigned short*>(slot) + (size_t)fA * G;
      const unsigned short* bA = reinterpret_cast<const unsigned short*>(slot + SB_BLOCK) + (size_t)fA * G;
      const unsigned short* sB = reinterpret_cast<const unsigned short*>(slot + (NMAT == 2 ? 2 : 0) * SB_BLOCK) + (size_t)fB * G;
      const unsigned short* bB = reinterpret_cast<const unsigned short*>(slot + (NMAT == 2 ? 3 : 1) * SB_BLOCK) + (size_t)fB * G;
      {
        tm.start();
        if (e != staged_e || p0 != staged_p0) {
          // ---- stage the activation rows of this (expert, pass): fp16, row-normalised, permuted ----
          if (!rendezvous()) {  // every compute warp is done with the old rows
            dead = true;
            break;
          }
          for (int r = warp; r < ROWS; r += N_COMPUTE / 32) {
            const int pr = p0 + r;
            const bool ok = pr < m;
            const uint4* src = nullptr;
            if (ok) {
              const uint32_t sp = seg0 + pr;
              uint32_t sr;
              if (p.src_mode == kSrcIdent)
                sr = sp;
              else if (p.src_mode == kSrcPermDiv)
                sr = p.perm[sp] / (uint32_t)p.src_div;
              else
                sr = p.src_map[p.perm[sp]];
              src = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(p.x) + (size_t)sr * K * 2);
            }
            uint32_t mxb = 0;
            for (int c = lane; c < K / 8 && ok; c += 32) {
              const uint4 v = __ldg(src + c);
              const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) mxb = max(mxb, max(u[q] & 0x7fffu, (u[q] >> 16) & 0x7fffu));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mxb = max(mxb, __shfl_xor_sync(0xffffffffu, mxb, o));
            const float mx = bf16_bits_to_f32(mxb);
            int ex = 0;
            if (mx > 0.f && mx < 3.0e38f) ex = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 127 - 10;
            ex = max(-100, min(100, ex));
            const float f = __uint_as_float((uint32_t)(127 - ex) << 23);
            if (lane == 0) rowsc[r] = __uint_as_float((uint32_t)(127 + ex) << 23);
            for (int c = lane; c < K / 8; c += 32) {  // K/8 is a multiple of 32: all lanes iterate together
              uint4 v = make_uint4(0, 0, 0, 0);
              if (ok) v = __ldg(src + c);
              const uint32_t u[4] = {v.x, v.y, v.z, v.w};
              float e8[8];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                e8[2 * q] = __uint_as_float(u[q] << 16) * f;
                e8[2 * q + 1] = __uint_as_float(u[q] & 0xffff0000u) * f;
              }
              __half h8[8];
              float se = 0.f, so = 0.f;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                if (BITS == 4 && (q & 1)) {
                  h8[q] = __float2half_rn(e8[q] * 0.0625f);
                  so += __half2float(h8[q]) * 16.0f;
                } else {
                  h8[q] = __float2half_rn(e8[q]);
                  se += __half2float(h8[q]);
                }
              }
              uint4 o;
              if constexpr (BITS == 4) {  // element order [0,4,1,5,2,6,3,7]
                o.x = (uint32_t)__half_as_ushort(h8[0]) | ((uint32_t)__half_as_ushort(h8[4]) << 16);
                o.y = (uint32_t)__half_as_ushort(h8[1]) | ((uint32_t)__half_as_ushort(h8[5]) << 16);
                o.z = (uint32_t)__half_as_ushort(h8[2]) | ((uint32_t)__half_as_ushort(h8[6]) << 16);
                o.w = (uint32_t)__half_as_ushort(h8[3]) | ((uint32_t)__half_as_ushort(h8[7]) << 16);
              } else {
                o.x = (uint32_t)__half_as_ushort(h8[0]) | ((uint32_t)__half_as_ushort(h8[1]) << 16);
                o.y = (uint32_t)__half_as_ushort(h8[2]) | ((uint32_t)__half_as_ushort(h8[3]) << 16);
                o.z = (uint32_t)__half_as_ushort(h8[4]) | ((uint32_t)__half_as_ushort(h8[5]) << 16);
                o.w = (uint32_t)__half_as_ushort(h8[6]) | ((uint32_t)__half_as_ushort(h8[7]) << 16);
              }
              *reinterpret_cast<uint4*>(xs + (size_t)r * XS + (size_t)c * 16) = o;
              // a group is 8 consecutive chunks = 8 consecutive lanes
#pragma unroll
              for (int o2 = 1; o2 < 8; o2 <<= 1) {
                se += __shfl_xor_sync(0xffffffffu, se, o2);
                so += __shfl_xor_sync(0xffffffffu, so, o2);
              }
              if ((lane & 7) == 0) {
                const int g = c >> 3;
                negc[g * ROWS + r] = (BITS == 4) ? -(1024.0f * se + 64.0f * so) : -1024.0f * (se + so);
                xsum[g * ROWS + r] = se + so;
              }
            }
          }
          if (!rendezvous()) {
            dead = true;
            break;
          }
          staged_e = e;
          staged_p0 = p0;
        }
        tm.stop(1);
        // ---- K loop over the streamed weight stages ---------------------------------------
        float tot[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int q = 0; q < 4; ++q) tot[nt][q] = 0.f;
        const bool sb_vec = (BITS == 4) ? ((G & 3) == 0) : ((G & 1) == 0);
        for (int st = 0; st < n_st; ++st) {
          // scale / bias of this stage's groups for the thread's two rows (bf16, GPS per row)
          uint32_t sAw[2], bAw[2], sBw[2], bBw[2];
          const int g0 = st * GPS;
          if (sb_vec) {
            if constexpr (BITS == 4) {
              const uint2 a = *reinterpret_cast<const uint2*>(sA + g0), b = *reinterpret_cast<const uint2*>(bA + g0);
              const uint2 c = *reinterpret_cast<const uint2*>(sB + g0), d = *reinterpret_cast<const uint2*>(bB + g0);
              sAw[0] = a.x; sAw[1] = a.y; bAw[0] = b.x; bAw[1] = b.y;
              sBw[0] = c.x; sBw[1] = c.y; bBw[0] = d.x; bBw[1] = d.y;
            } else {
              sAw[0] = *reinterpret_cast<const uint32_t*>(sA + g0); bAw[0] = *reinterpret_cast<const uint32_t*>(bA + g0);
              sBw[0] = *reinterpret_cast<const uint32_t*>(sB + g0); bBw[0] = *reinterpret_cast<const uint32_t*>(bB + g0);
              sAw[1] = bAw[1] = sBw[1] = bBw[1] = 0;
            }
          } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              sAw[h] = bAw[h] = sBw[h] = bBw[h] = 0;
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const int gi = 2 * h + j;
                if (gi < GPS) {
                  sAw[h] |= (uint32_t)sA[g0 + gi] << (16 * j);
                  bAw[h] |= (uint32_t)bA[g0 + gi] << (16 * j);
                  sBw[h] |= (uint32_t)sB[g0 + gi] << (16 * j);
                  bBw[h] |= (uint32_t)bB[g0 + gi] << (16 * j);
                }
              }
            }
          }
          tm.start();
          if (!bar_wait(full_bar(s), ph, abort_flag)) {
            dead = true;
            break;
          }
          tm.stop(0);
          const unsigned char* wst = w_ring + (size_t)s * STAGE_BYTES;
          // All operands of the stage's GPS groups are fetched first and the MMAs are issued
          // group-interleaved (MMA i of every group before MMA i+1 of any), so that GPS*NT
          // independent accumulator chains hide the tensor-pipe latency.
          uint32_t wA[GPS][4], wB[GPS][4];
#pragma unroll
          for (int gi = 0; gi < GPS; ++gi) {
            if constexpr (BITS == 4) {
              const uint32_t ch = (uint32_t)(2 * gi + (t >> 1));
              const uint2 a = *reinterpret_cast<const uint2*>(wst + offA + ((ch ^ swA) << 4) + (t & 1) * 8);
              const uint2 b = *reinterpret_cast<const uint2*>(wst + offB + ((ch ^ swB) << 4) + (t & 1) * 8);
              wA[gi][0] = a.x; wA[gi][1] = a.y; wB[gi][0] = b.x; wB[gi][1] = b.y;
              wA[gi][2] = wA[gi][3] = wB[gi][2] = wB[gi][3] = 0;
            } else {
              const uint32_t ch = (uint32_t)(4 * gi + t);
              const uint4 a = *reinterpret_cast<const uint4*>(wst + offA + ((ch ^ swA) << 4));
              const uint4 b = *reinterpret_cast<const uint4*>(wst + offB + ((ch ^ swB) << 4));
              wA[gi][0] = a.x; wA[gi][1] = a.y; wA[gi][2] = a.z; wA[gi][3] = a.w;
              wB[gi][0] = b.x; wB[gi][1] = b.y; wB[gi][2] = b.z; wB[gi][3] = b.w;
            }
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            if (nt > 0 && nt * 8 >= m - p0) break;  // (warp-uniform) this n-tile holds no row of the pass
            uint4 x0[GPS], x1[GPS];
            float acc[GPS][4];
#pragma unroll
            for (int gi = 0; gi < GPS; ++gi) {
              const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + gq) * XS + (size_t)((g0 + gi) * 4 + t) * 32);
              x0[gi] = xp[0];
              x1[gi] = xp[1];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
              for (int gi = 0; gi < GPS; ++gi) {
                const uint4& xv = (i < 2) ? x0[gi] : x1[gi];
                const uint32_t b0 = (i & 1) ? xv.z : xv.x, b1 = (i & 1) ? xv.w : xv.y;
                uint32_t a0, a1, a2, a3;
                if constexpr (BITS == 4) {
                  constexpr uint32_t LO = 0x000f000fu, HI = 0x00f000f0u, MG = 0x64006400u;
                  const uint32_t a = wA[gi][i >> 1] >> (8 * (i & 1)), b = wB[gi][i >> 1] >> (8 * (i & 1));
                  a0 = (a & LO) | MG; a1 = (b & LO) | MG; a2 = (a & HI) | MG; a3 = (b & HI) | MG;
                } else {
                  constexpr uint32_t MG8 = 0x64646464u;
                  a0 = __byte_perm(wA[gi][i], MG8, 0x4140); a1 = __byte_perm(wB[gi][i], MG8, 0x4140);
                  a2 = __byte_perm(wA[gi][i], MG8, 0x4342); a3 = __byte_perm(wB[gi][i], MG8, 0x4342);
                }
                if (i == 0) {
                  const float2 nc = *reinterpret_cast<const float2*>(&negc[(g0 + gi) * ROWS + nt * 8 + 2 * t]);
                  mma_f16_16816(acc[gi], a0, a1, a2, a3, b0, b1, nc.x, nc.y);
                } else {
                  mma_f16_16816_acc(acc[gi], a0, a1, a2, a3, b0, b1);
                }
              }
            }
#pragma unroll
            for (int gi = 0; gi < GPS; ++gi) {
              const float2 xsm = *reinterpret_cast<const float2*>(&xsum[(g0 + gi) * ROWS + nt * 8 + 2 * t]);
              const float s_a = __uint_as_float((gi & 1) ? (sAw[gi >> 1] & 0xffff0000u) : (sAw[gi >> 1] << 16));
              const float b_a = __uint_as_float((gi & 1) ? (bAw[gi >> 1] & 0xffff0000u) : (bAw[gi >> 1] << 16));
              const float s_b = __uint_as_float((gi & 1) ? (sBw[gi >> 1] & 0xffff0000u) : (sBw[gi >> 1] << 16));
              const float b_b = __uint_as_float((gi & 1) ? (bBw[gi >> 1] & 0xffff0000u) : (bBw[gi >> 1] << 16));
              tot[nt][0] = fmaf(s_a, acc[gi][0], fmaf(b_a, xsm.x, tot[nt][0]));
              tot[nt][1] = fmaf(s_a, acc[gi][1], fmaf(b_a, xsm.y, tot[nt][1]));
              tot[nt][2] = fmaf(s_b, acc[gi][2], fmaf(b_b, xsm.x, tot[nt][2]));
              tot[nt][3] = fmaf(s_b, acc[gi][3], fmaf(b_b, xsm.y, tot[nt][3]));
            }
          }
          __syncwarp();
          if (lane == 0) bar_arrive(empty_bar(s));
          if (++s == ring) {
            s = 0;
            ph ^= 1;
          }
        }
        if (dead) break;
        // ---- epilogue: undo the row normalisation, activation / routing weight, store ------
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int tok = nt * 8 + 2 * t + j, pr = p0 + tok;
            if (pr >= m) continue;
            const float rs = rowsc[tok];
            const uint32_t sp = seg0 + pr;
            const uint32_t dst = p.dst_perm ? p.perm[sp] : sp;
            const float vA = tot[nt][j] * rs, vB = tot[nt][2 + j] * rs;
            if constexpr (NMAT == 2) {
              const float h = __fdividef(vA, 1.0f + __expf(-vA)) * vB;
              static_cast<__nv_bfloat16*>(p.out)[(size_t)dst * N + fb * FB + fA] = __float2bfloat16_rn(h);
            } else {
              float sc = 1.0f;
              if (p.row_scale) sc = bf16_bits_to_f32(static_cast<const unsigned short*>(p.row_scale)[dst]);
              if (p.out_f32) {
                static_cast<float*>(p.out)[(size_t)dst * N + fb * FB + fA] = vA * sc;
                static_cast<float*>(p.out)[(size_t)dst * N + fb * FB + fB] = vB * sc;
              } else {
                static_cast<__nv_bfloat16*>(p.out)[(size_t)dst * N + fb * FB + fA] = __float2bfloat16_rn(vA * sc);
                static_cast<__nv_bfloat16*>(p.out)[(size_t)dst * N + fb * FB + fB] = __float2bfloat16_rn(vB * sc);
              }
            }
          }
      }
      if (dead) break;
      __syncwarp();
      if (lane == 0) bar_arrive(sbempty0 + 8u * sl);  // this warp is done with the item's scales
      if (++sl == 2) {
        sl = 0;
        slph ^= 1;
      }
      }
     }
     it0 = run_end;
    }
    tm.acc[3] = clock64() - tb;
    tm.flush(p.err + 20);
    if ((p.debug & 32) && tid == 0) {
      atomicMax(p.err + 24, (int)((clock64() - tb) >> 10));
      atomicAdd(p.err + 25, (int)((clock64() - tb) >> 10));
      atomicAdd(p.err + 26, i1 - i0);
    }
  }
  __syncthreads();
  if (*abort_flag && tid == 0) atomicExch(p.err, 3);
}


typedef CUresult (*EncodeTiledFnS)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFnS encode_fn_s() {
  static EncodeTiledFnS fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFnS>(f);
  }();
  return fn;
}

static size_t stream_fixed_smem(int K, int rows) {
  const int G = K / 64;
  const size_t sb = (size_t)2 * 4 * 64 * G * 2;  // two slots of scales + biases for 128 weight rows
  return (size_t)rows * (2 * K + 16) + sizeof(float) * (2 * G * rows + rows + 2) + 8 * (2 * MAX_RING + 8) + 16 + sb + 1024;
}

}  // namespace

bool stream_shape_ok(int K, int N, int nmat, int bits) {
  if (!(bits == 4 || bits == 8) || K % 256 != 0 || N % (nmat == 2 ? 64 : 128) != 0) return false;
  return stream_fixed_smem(K, 8) + 4 * STAGE_BYTES <= 227 * 1024;
}

// g: the same description the first-generation kernel takes; n_experts: number of stacked matrices.
int launch_grouped_qmm_stream(const GroupedArgs& g, int nmat, int bits, int n_experts, int max_active, int64_t rows,
                              int* err, cudaStream_t st) {
  if (rows == 0 || max_active == 0) return 0;
  B200_REQUIRE(stream_shape_ok(g.K, g.N, nmat, bits), "shape not supported by the streaming kernel");
  EncodeTiledFnS enc = encode_fn_s();
  B200_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap tmap_w[2];
  cuuint32_t estr[2] = {1, 1};
  for (int i = 0; i < nmat; ++i) {
    cuuint64_t wd[2] = {(cuuint64_t)g.K * bits / 32, (cuuint64_t)n_experts * g.N};
    cuuint64_t ws_[1] = {(cuuint64_t)g.K * bits / 8};
    cuuint32_t wb[2] = {32, (cuuint32_t)(nmat == 2 ? 64 : 128)};
    CUresult cr = enc(&tmap_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(g.w[i]), wd, ws_, wb, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for the packed weights (16-byte alignment required)");
  }
  if (nmat == 1) tmap_w[1] = tmap_w[0];

  StreamArgs p{};
  p.x = g.x;
  for (int i = 0; i < 2; ++i) {
    p.scales[i] = g.scales[i];
    p.biases[i] = g.biases[i];
  }
  p.offsets = g.offsets;
  p.active = g.active;
  p.n_active = g.n_active;
  p.perm = g.perm;
  p.src_map = g.src_map;
  p.src_mode = g.src_mode;
  p.src_div = g.src_div;
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
  // 16 rows per pass as soon as some expert must own more than one row
  const int nt = (rows > max_active && stream_fixed_smem(g.K, 16) + 4 * STAGE_BYTES <= 227 * 1024) ? 2 : 1;
  const size_t fixed = stream_fixed_smem(g.K, 8 * nt);
  int ring = (int)((227 * 1024 - fixed) / STAGE_BYTES);
  if (ring > MAX_RING) ring = MAX_RING;
  const size_t smem = fixed + (size_t)ring * STAGE_BYTES;
  const int64_t items = (int64_t)max_active * (g.N / (nmat == 2 ? 64 : 128));
  const int grid = (int)(items < n_sm ? items : n_sm);

#define B200_STREAM_LAUNCH(BITSV, NMATV, NTV)                                                                \
  do {                                                                                                       \
    auto kern = grouped_qmm_stream_kernel<BITSV, NMATV, NTV>;                                                \
    static size_t attr = 0;                                                                                  \
    if (smem > attr) {                                                                                       \
      B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));         \
      attr = smem;                                                                                           \
    }                                                                                                        \
    kern<<<grid, N_THREADS_S, smem, st>>>(tmap_w[0], tmap_w[1], p, ring);                                    \
  } while (0)
#define B200_STREAM_NT(BITSV, NMATV)   \
  do {                                 \
    if (nt == 2)                       \
      B200_STREAM_LAUNCH(BITSV, NMATV, 2); \
    else                               \
      B200_STREAM_LAUNCH(BITSV, NMATV, 1); \
  } while (0)
  if (bits == 4 && nmat == 2)
    B200_STREAM_NT(4, 2);
  else if (bits == 4)
    B200_STREAM_NT(4, 1);
  else if (nmat == 2)
    B200_STREAM_NT(8, 2);
  else
    B200_STREAM_NT(8, 1);
#undef B200_STREAM_NT
#undef B200_STREAM_LAUNCH
  return 0;
}

}  // namespace b200

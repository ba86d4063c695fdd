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

constexpr int kDownCombineMaxK = 32;  // top-k slots the fused down projection and sum keeps in shared memory

template <int BITS, int NMAT, int RT, int NT>
__global__ void __launch_bounds__(256, NT == 1 ? 2 : 1) grouped_qmm_small_kernel(GroupedArgs p) {
  constexpr int KS = 8 / (NMAT * RT);
  constexpr int ROWS = 8 * NT;  // activation rows per pass
  static_assert(NMAT * RT * KS == 8, "eight warps");

  if (p.late_trigger) {  // the next kernel starts once this one's predecessors are complete, not before
    pdl_wait();
    pdl_trigger();
  } else {
    pdl_prologue();
  }
  const int ea = blockIdx.y;
  int e, m;
  uint32_t seg0;
  if (p.desc) {  // one load instead of the chain n_active -> active -> offsets
    const uint4 d = __ldg(reinterpret_cast<const uint4*>(p.desc + (size_t)ea * kExpertDescWords));
    e = (int)d.x;
    seg0 = d.y;
    m = (int)d.z;
  } else {
    if (ea >= (int)*p.n_active) return;
    e = p.active[ea];
    seg0 = p.offsets[e];
    m = (int)(p.offsets[e + 1] - seg0);
  }
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
      else if (p.desc && p0 == 0 && tid < 8)  // (a record holds the first eight source rows)
        src = (int)__ldg(p.desc + (size_t)ea * kExpertDescWords + 4 + tid);
      else if (p.src_mode == kSrcPermDiv)
        src = (int)(p.perm[sp] / (uint32_t)p.src_div);
      else if (p.src_mode == kSrcMapDirect)
        src = (int)p.src_map[sp];
      else
        src = (int)p.src_map[p.perm[sp]];
      s_src[tid] = src;
      if (!p.x_bf16) s.rs[tid] = p.x_rowscale ? p.x_rowscale[src] : 1.0f;
    }
    __syncthreads();
    if (p.x_bf16) {  // plain bf16 rows: warp r prepares row r straight into the staged image
      for (int r = warp; r < nrows; r += 8)
        prepare_row_warp<BITS, false>(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.x) + (size_t)s_src[r] * K),
                                      K / 8, reinterpret_cast<uint4*>(s.xs + (size_t)r * s.XS), s.rs + r, lane);
    } else {
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

// ---- per-expert records --------------------------------------------------------------------------------------
// What a CTA of the grouped product needs to know about its expert, gathered into one 64-byte record so that the
// CTA's prologue is one load instead of a chain of four dependent ones (n_active -> active -> offsets -> perm).
__global__ void __launch_bounds__(256) expert_desc_kernel(const uint32_t* __restrict__ active, const uint32_t* __restrict__ n_active,
                                                          const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ perm,
                                                          const uint32_t* __restrict__ src_map, int src_mode, int src_div,
                                                          const float* __restrict__ row_scale, int max_active,
                                                          uint32_t* __restrict__ desc) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int ea = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (ea >= max_active) return;
  uint32_t v = 0;
  if (ea < (int)*n_active) {
    const uint32_t e = active[ea], seg0 = offsets[e], m = offsets[e + 1] - seg0;
    if (lane == 0) v = e;
    if (lane == 1) v = seg0;
    if (lane == 2) v = m;
    if (lane >= 4 && lane < 20 && (uint32_t)((lane - 4) & 7) < m) {
      const uint32_t sp = seg0 + (uint32_t)((lane - 4) & 7);
      if (src_mode == kSrcIdent)
        v = sp;
      else if (src_mode == kSrcPermDiv)
        v = perm[sp] / (uint32_t)src_div;
      else if (src_mode == kSrcMapDirect)
        v = src_map[sp];
      else
        v = src_map[perm[sp]];
      if (lane >= 12) v = __float_as_uint(row_scale ? row_scale[v] : 1.0f);
    }
  }
  desc[(size_t)ea * kExpertDescWords + lane] = v;
}

int launch_expert_descs(const uint32_t* active, const uint32_t* n_active, const uint32_t* offsets, const uint32_t* perm,
                        const uint32_t* src_map, int src_mode, int src_div, const float* row_scale, int max_active,
                        uint32_t* desc, cudaStream_t st) {
  if (max_active == 0) return 0;
  B200_CUDA(launch_pdl(expert_desc_kernel, dim3(cdiv(max_active, 8)), dim3(256), 0, st, active, n_active, offsets, perm, src_map,
                       src_mode, src_div, row_scale, max_active, desc));
  return 0;
}

// ---- the same product with the CTA's whole weight slice requested up front --------------------------------------
// The register stream above keeps two blocks per lane in flight, and a CTA's prologue (segment look-up, row
// staging, sums: 4-5 us measured) runs with only those two on their way, so the memory system idles for a third of
// a CTA's life.  Here every warp asks for ALL blocks of its 16 rows x K slice at once, with 16-byte asynchronous
// copies into shared memory (one commit group per block), before anything else; the prologue then runs under the
// transfer and the K loop waits block by block (cp.async.wait_group) and reads the codes back with 64/128-bit
// shared loads.  A row of a block is 128 bytes (four 4-bit groups or two 8-bit groups); its 16-byte chunk c is
// stored at chunk c ^ ((row * (BITS == 4 ? 2 : 4)) & 7), which spreads the half-warp (4-bit, 8-byte reads) or
// quarter-warp (8-bit, 16-byte reads) of a read over all banks.  The blocks' scales and biases (8 or 4 bytes per
// row and block) travel the same way.  One pass of at most eight rows per expert (NT = 1); used when two CTAs fit
// on an SM.
constexpr int kStagedBlockBytes = 16 * 128 + 256;  // one block of a warp: 16 rows x 128 bytes of codes + scales/biases

__device__ __forceinline__ void cp_async_small(void* smem_dst, const void* gmem_src, int bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  if (bytes == 8)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gmem_src) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most n of this thread's most recent commit groups are pending (n <= 7)
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
  }
}

template <int BITS, int NMAT, int RT>
__global__ void __launch_bounds__(256, 2) grouped_qmm_staged_kernel(GroupedArgs p) {
  constexpr int KS = 8 / (NMAT * RT);
  constexpr int ROWS = 8;
  constexpr int GB = (BITS == 4) ? 4 : 2;   // groups per block
  constexpr int SW = (BITS == 4) ? 2 : 4;   // swizzle step per row
  static_assert(NMAT * RT * KS == 8, "eight warps");

  pdl_prologue();
  const int ea = blockIdx.y;
  int e, m;
  uint32_t seg0;
  if (p.desc) {  // one load instead of the chain n_active -> active -> offsets
    const uint4 d = __ldg(reinterpret_cast<const uint4*>(p.desc + (size_t)ea * kExpertDescWords));
    e = (int)d.x;
    seg0 = d.y;
    m = (int)d.z;
    if (m == 0) return;
  } else {
    if (ea >= (int)*p.n_active) return;
    e = p.active[ea];
    seg0 = 0;
    m = -1;  // looked up below, after the weight copies are on their way
  }
  const int K = p.K, N = p.N, G = K / 64;
  const int bpw = (G / GB) / KS;  // blocks per warp (the launcher guarantees the divisions are exact, bpw <= 8)
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_src[ROWS];
  const Staged s = staged_at(smem, K, ROWS);
  unsigned char* after = smem + ((staged_bytes(K, ROWS) + 15) & ~size_t(15));
  float* red = reinterpret_cast<float*>(after);  // [8 warps][128]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* wsm = after + sizeof(float) * 8 * 128 + (size_t)warp * bpw * kStagedBlockBytes;
  const int gq = lane >> 2, t = lane & 3;
  const int mt = warp % NMAT, rt = (warp / NMAT) % RT, ks = warp / (NMAT * RT);
  const int n0 = blockIdx.x * (16 * RT) + rt * 16;
  const int wrow_bytes = K * BITS / 8;

  // With a record, the first pass's rows are known at once: warp r asks for row r FIRST (commit group 0), then come
  // the weights, so that the rows can be waited for alone and the K loop waits block by block.  Without a record the
  // rows follow the weights and one wait covers everything.
  const bool rows_first = p.desc && p.src_mode != kSrcIdent ? true : (p.src_mode == kSrcIdent && m >= 0);
  const int nvec = K / 8;
  if (rows_first && !p.x_bf16) {
    const int nrows0 = min(ROWS, m);
    if (warp < nrows0) {
      const int src = p.src_mode == kSrcIdent ? (int)(seg0 + warp) : (int)__ldg(p.desc + (size_t)ea * kExpertDescWords + 4 + warp);
      const unsigned char* srow = static_cast<const unsigned char*>(p.x) + (size_t)src * K * 2;
      unsigned char* drow = s.xs + (size_t)warp * s.XS;
      for (int cc = lane; cc < nvec; cc += 32) cp_async16(drow + cc * 16, srow + cc * 16);
    }
    if (tid < nrows0) {
      float rsv = 1.0f;
      if (p.src_mode != kSrcIdent)
        rsv = __uint_as_float(__ldg(p.desc + (size_t)ea * kExpertDescWords + 12 + tid));
      else if (p.x_rowscale)
        rsv = p.x_rowscale[seg0 + tid];
      s.rs[tid] = rsv;
    }
    cp_async_commit();
  }
  // ---- all weight blocks of this warp, on their way ---------------------------------------------
  {
    const unsigned char* wb = reinterpret_cast<const unsigned char*>(p.w[mt]);
    const int c = lane & 7;
    const unsigned char* rowp[4];  // the four rows this lane copies chunk c of
    uint32_t dsto[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = (lane >> 3) + 4 * q;
      rowp[q] = wb + ((size_t)e * N + min(n0 + r, N - 1)) * wrow_bytes + c * 16;
      dsto[q] = (uint32_t)(r * 128 + ((c ^ ((r * SW) & 7)) << 4));
    }
    const int sb_row = lane & 15;
    const unsigned char* sb_src = reinterpret_cast<const unsigned char*>((lane >> 4) ? p.biases[mt] : p.scales[mt]) +
                                  ((size_t)e * N + min(n0 + sb_row, N - 1)) * G * 2;
    const uint32_t sb_dst = 2048 + (lane >> 4) * 128 + sb_row * 8;
    for (int j = 0; j < bpw; ++j) {
      const int bk = ks + j * KS;
      unsigned char* blk = wsm + (size_t)j * kStagedBlockBytes;
#pragma unroll
      for (int q = 0; q < 4; ++q) cp_async16(blk + dsto[q], rowp[q] + (size_t)bk * 128);
      cp_async_small(blk + sb_dst, sb_src + (size_t)bk * GB * 2, GB * 2);
      cp_async_commit();
    }
  }

  if (m < 0) {
    seg0 = p.offsets[e];
    m = (int)(p.offsets[e + 1] - seg0);
  }
  const int swa = (gq * SW) & 7;  // rows gq and gq + 8 share the swizzle
  // passes of eight rows; after the first one the weights are resident in shared memory
  for (int p0 = 0; p0 < m; p0 += ROWS) {
  const int nrows = min(ROWS, m - p0);
  bool block_waits = p.x_bf16 != 0;  // the K loop waits for its blocks one by one
  if (rows_first && !p.x_bf16 && p0 == 0) {
    cp_async_wait_pending(bpw);  // the rows (group 0); the weights' groups may still be on their way
    block_waits = true;
  } else {
    // ---- stage the prepared rows: asynchronous copies in a group BEHIND the weights' (groups complete in order, so
    //      the wait below also covers the weights - which have had the whole prologue to arrive) ----
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
      if (!p.x_bf16) s.rs[tid] = p.x_rowscale ? p.x_rowscale[src] : 1.0f;
    }
    __syncthreads();
    if (p.x_bf16) {
      for (int r = warp; r < nrows; r += 8)
        prepare_row_warp<BITS, false>(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.x) + (size_t)s_src[r] * K),
                                      K / 8, reinterpret_cast<uint4*>(s.xs + (size_t)r * s.XS), s.rs + r, lane);
    } else {
      const unsigned char* x16 = static_cast<const unsigned char*>(p.x);
      for (int r = warp; r < nrows; r += 8) {  // warp r copies row r
        const unsigned char* srow = x16 + (size_t)s_src[r] * K * 2;
        unsigned char* drow = s.xs + (size_t)r * s.XS;
        for (int cc = lane; cc < nvec; cc += 32) cp_async16(drow + cc * 16, srow + cc * 16);
      }
      cp_async_commit();
      cp_async_wait_pending(0);
    }
  }
  __syncthreads();
  stage_sums<BITS>(s, ROWS, nrows, K, tid, 256);
  __syncthreads();

  // ---- K loop: block by block as the copies land ----------------------------------------------
  float tot[1][4] = {{0.f, 0.f, 0.f, 0.f}};
  StagedFetch<ROWS> fetch(s, gq, t);
  for (int j = 0; j < bpw; ++j) {
    if (block_waits) {  // (otherwise the wait for the rows has covered the weights)
      cp_async_wait_pending(bpw - 1 - j);
      __syncwarp();  // every lane's copies of block j have landed
    }
    const int bk = ks + j * KS;
    const unsigned char* blk = wsm + (size_t)j * kStagedBlockBytes;
    fetch.block(bk * GB);
    // the block's scales and biases of rows gq and gq + 8: one 8-byte load each (GB bf16 numbers per row)
    const uint2 sc_a = *reinterpret_cast<const uint2*>(blk + 2048 + gq * 8), sc_b = *reinterpret_cast<const uint2*>(blk + 2048 + (gq + 8) * 8);
    const uint2 bi_a = *reinterpret_cast<const uint2*>(blk + 2176 + gq * 8), bi_b = *reinterpret_cast<const uint2*>(blk + 2176 + (gq + 8) * 8);
#pragma unroll
    for (int u = 0; u < GB; ++u) {
      typename WVec<BITS>::T wa, wb;
      if constexpr (BITS == 4) {
        const int off = (((u * 2 + (t >> 1)) ^ swa) << 4) + (t & 1) * 8;
        wa = *reinterpret_cast<const uint2*>(blk + gq * 128 + off);
        wb = *reinterpret_cast<const uint2*>(blk + (gq + 8) * 128 + off);
      } else {
        const int off = ((u * 4 + t) ^ swa) << 4;
        wa = *reinterpret_cast<const uint4*>(blk + gq * 128 + off);
        wb = *reinterpret_cast<const uint4*>(blk + (gq + 8) * 128 + off);
      }
      const float fsa = bf16_of(sc_a, u), fba = bf16_of(bi_a, u), fsb = bf16_of(sc_b, u), fbb = bf16_of(bi_b, u);
      uint4 x0, x1;
      float4 c4;
      float2 s2;
      fetch(u, 0, x0, x1, c4, s2);
      group_step<BITS>(wa, wb, x0, x1, c4, s2, fsa, fba, fsb, fbb, tot[0]);
    }
  }

  // ---- partial sums -> shared, [warp][row16][tok8], already multiplied by the row scale ----
  {
    const float rs0 = s.rs[2 * t], rs1 = s.rs[2 * t + 1];
    float* r = red + (size_t)warp * 128;
    r[gq * 8 + 2 * t] = tot[0][0] * rs0;
    r[gq * 8 + 2 * t + 1] = tot[0][1] * rs1;
    r[(gq + 8) * 8 + 2 * t] = tot[0][2] * rs0;
    r[(gq + 8) * 8 + 2 * t + 1] = tot[0][3] * rs1;
  }
  __syncthreads();
  // ---- epilogue: fixed-order sum over the K slices, activation / routing weight, store ----
  for (int o = tid; o < 16 * RT * ROWS; o += 256) {
    const int rl = o % (16 * RT), tok = o / (16 * RT);
    const int n = blockIdx.x * (16 * RT) + rl;
    if (tok >= nrows || n >= N) continue;
    const int ert = rl >> 4, r16 = rl & 15;
    float v[NMAT];
#pragma unroll
    for (int q = 0; q < NMAT; ++q) {
      float sum = 0.f;
#pragma unroll
      for (int z = 0; z < KS; ++z) sum += red[(size_t)((z * RT + ert) * NMAT + q) * 128 + r16 * 8 + tok];
      v[q] = sum;
    }
    const uint32_t sp = seg0 + p0 + tok;
    const uint32_t dst = p.dst_perm ? p.perm[sp] : sp;
    float outv;
    if constexpr (NMAT == 2) {
      outv = v[0] / (1.0f + __expf(-v[0])) * v[1];
      if (p.out_f16) {
        const float hb = __uint_as_float(f32_to_bf16_bits(outv) << 16) * prepared_factor<BITS>(n);
        reinterpret_cast<unsigned short*>(p.out)[(size_t)dst * N + prepared_pos<BITS>(n)] = f16_sat_bits(hb);
        continue;
      }
    } else {
      outv = v[0];
      if (p.row_scale) outv *= bf16_bits_to_f32(reinterpret_cast<const unsigned short*>(p.row_scale)[dst]);
    }
    if (p.out_row_addr) {
      const unsigned long long da = p.out_row_addr[sp];
      if (da) reinterpret_cast<__nv_bfloat16*>(da)[n] = __float2bfloat16_rn(outv);
    } else if (p.out_f32)
      reinterpret_cast<float*>(p.out)[(size_t)dst * N + n] = outv;
    else
      reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)dst * N + n] = __float2bfloat16_rn(outv);
  }
  __syncthreads();
  }
  cp_async_wait_pending(0);  // (an expert without rows: nothing may stay in flight when the CTA ends)
}

template <int NMAT>
static size_t staged_smem_bytes(int K, int bits, int rt) {
  const int gb = bits == 4 ? 4 : 2, ks = 8 / (NMAT * rt);
  const size_t bpw = (size_t)(K / 64 / gb) / ks;
  return ((staged_bytes(K, 8) + 15) & ~size_t(15)) + sizeof(float) * 8 * 128 + 8 * bpw * kStagedBlockBytes;
}
constexpr size_t kStagedMaxSmem = 112 * 1024;  // two CTAs per SM

template <int NMAT>
static bool staged_feasible(int K, int bits) {
  const int gbs = bits == 4 ? 4 : 2;
  if ((K / 64) % gbs) return false;
  const int nb = K / 64 / gbs;
  for (int cand = 8 / NMAT; cand >= 1; cand >>= 1) {
    const int ks = 8 / (NMAT * cand);
    if (nb % ks == 0 && nb / ks <= 8 && staged_smem_bytes<NMAT>(K, bits, cand) <= kStagedMaxSmem) return true;
  }
  return false;
}

template <int BITS, int NMAT, int RT>
static int launch_staged(const GroupedArgs& a, int max_active, cudaStream_t st) {
  const size_t smem = staged_smem_bytes<NMAT>(a.K, BITS, RT);
  auto kern = grouped_qmm_staged_kernel<BITS, NMAT, RT>;
  static DynSmemCache attr;
  B200_CUDA(ensure_dyn_smem(kern, smem, attr));
  dim3 grid(cdiv(a.N, 16 * RT), max_active);
  B200_CUDA(launch_pdl(kern, grid, dim3(256), smem, st, a));
  return 0;
}

// ---- down projection + weighted k-way sum for a handful of tokens ----------------------------------
// out[t, n0..n0+16) = bf16( sum_j score[t, j] * (h[row(t, j), :] . W_down[e(t, j)][n, :]) ), j ascending: the down
// projection with the routing weight (multiply before sum_axis, mlx-rs/src/ops/reduction.rs:260-275), the take with
// the inverse order and the k-way sum in ONE launch - no per-assignment buffer, no combine kernel.  One CTA per
// (token, 16 output features); warp j streams the 16 weight rows of the expert in slot j (then j + 8, ...) over the
// whole K, against the token's staged row of that slot.
template <int BITS>
__global__ void __launch_bounds__(256, 2) down_combine_small_kernel(DownCombineArgs p) {
  // With early_routing the routing outputs (written two kernels back) are complete when this CTA starts: they and the
  // first weight blocks - constants - are fetched BEFORE the dependency wait, under the gate/up kernel's tail; only
  // h, which that kernel writes, waits.
  pdl_trigger();
  if (!p.early_routing) pdl_wait();
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ uint32_t s_e[kDownCombineMaxK], s_row[kDownCombineMaxK];
  __shared__ float s_sc[kDownCombineMaxK];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, t = lane & 3;
  constexpr int WPT = (BITS == 4) ? 2 : 4;
  const int K = p.K, N = p.N, k = p.k, G = K / 64;
  const int tiles = (N + 15) / 16;
  const int tok = blockIdx.x / tiles, n0 = (blockIdx.x % tiles) * 16;
  const int wrow = K * BITS / 32;
  const Staged s = staged_at(smem, K, k);
  float* red = reinterpret_cast<float*>(smem + ((staged_bytes(K, k) + 15) & ~size_t(15)));  // [k][16]
  if (tid < k) {
    s_e[tid] = p.idx[(size_t)tok * k + tid];
    s_row[tid] = p.inv[(size_t)tok * k + tid];
    s_sc[tid] = bf16_bits_to_f32(reinterpret_cast<const unsigned short*>(p.scores)[(size_t)tok * k + tid]);
    s.rs[tid] = 1.0f;
  }
  __syncthreads();
  const unsigned short* scb = reinterpret_cast<const unsigned short*>(p.scales);
  const unsigned short* bib = reinterpret_cast<const unsigned short*>(p.biases);
  WeightStream<BITS> ws;
  auto start_slot = [&](int j) {
    const size_t e = s_e[j];
    const size_t row_a = e * N + min(n0 + gq, N - 1), row_b = e * N + min(n0 + gq + 8, N - 1);
    ws.start(p.w + row_a * wrow + t * WPT, p.w + row_b * wrow + t * WPT, scb + row_a * G, bib + row_a * G, scb + row_b * G,
             bib + row_b * G, G, 0, 1);
  };
  if (warp < k) start_slot(warp);  // the first blocks of weights are on their way while the rows are staged
  if (p.early_routing) pdl_wait();
  {
    const int nvec = K / 8;
    const unsigned char* hb = static_cast<const unsigned char*>(p.h);
    for (int i = tid; i < k * nvec; i += 256) {
      const int r = i / nvec, c = i % nvec;
      cp_async16(s.xs + (size_t)r * s.XS + c * 16, hb + ((size_t)s_row[r] * K) * 2 + c * 16);
    }
    cp_async_wait_all();
  }
  __syncthreads();
  stage_sums<BITS>(s, k, k, K, tid, 256);
  __syncthreads();
  for (int j = warp; j < k; j += 8) {
    if (j != warp) start_slot(j);
    float tot[1][4] = {{0.f, 0.f, 0.f, 0.f}};
    ws.template run<1>(SingleRowFetch(s, k, j, t), tot);
    if (t == 0) {  // column 0 of the tile is the token's row: lanes t == 0 hold weight rows gq and gq + 8
      red[j * 16 + gq] = tot[0][0] * s_sc[j];
      red[j * 16 + gq + 8] = tot[0][2] * s_sc[j];
    }
  }
  __syncthreads();
  if (tid < 16 && n0 + tid < N) {
    float acc = 0.f;
    for (int j = 0; j < k; ++j) acc += red[j * 16 + tid];
    const size_t o = (size_t)tok * N + n0 + tid;
    if (p.out_f32) p.out_f32[o] = acc;
    static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(acc);
  }
}

static size_t down_combine_smem(int K, int k) { return ((staged_bytes(K, k) + 15) & ~size_t(15)) + sizeof(float) * 16 * k; }

bool down_combine_small_ok(int64_t T, int k, int K) {
  return T >= 1 && T <= 8 && k >= 1 && k <= kDownCombineMaxK && K % 64 == 0 && down_combine_smem(K, k) <= 100 * 1024;
}

int launch_down_combine_small(const DownCombineArgs& a, int bits, cudaStream_t st) {
  B200_REQUIRE(down_combine_small_ok(a.T, a.k, a.K), "shape not supported by the fused down projection and sum");
  B200_REQUIRE(bits == 4 || bits == 8, "bits must be 4 or 8");
  const size_t smem = down_combine_smem(a.K, a.k);
  const dim3 grid((unsigned)(a.T * cdiv(a.N, 16)));
  if (bits == 4) {
    static DynSmemCache attr;
    B200_CUDA(ensure_dyn_smem(down_combine_small_kernel<4>, smem, attr));
    B200_CUDA(launch_pdl(down_combine_small_kernel<4>, grid, dim3(256), smem, st, a));
  } else {
    static DynSmemCache attr;
    B200_CUDA(ensure_dyn_smem(down_combine_small_kernel<8>, smem, attr));
    B200_CUDA(launch_pdl(down_combine_small_kernel<8>, grid, dim3(256), smem, st, a));
  }
  return 0;
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
  B200_CUDA(launch_pdl(kern, grid, dim3(256), smem, st, a));
  return 0;
}

// Rows per expert above which a pass stages 32 rows instead of 8 (one CTA per SM then, but the weights are read once
// for four times the rows); below, an expert with more than eight rows takes several 8-row passes whose weight
// re-reads hit L2 - or, in the variant that keeps its weight slice in shared memory, cost no weight traffic at all,
// which moves the limit up (20 rows per expert: 0.344 ms per block against 0.419 with 32-row passes).
constexpr int64_t kWideAbove = 16, kWideAboveStaged = 32;

template <int BITS, int NMAT>
static int launch_bits_nmat(const GroupedArgs& a, int max_active, int64_t rows, cudaStream_t st) {
  // more activation rows per pass once the experts are expected to hold more than eight rows each
  const int64_t per = rows / (max_active > 0 ? max_active : 1);
  int64_t wide_above = staged_feasible<NMAT>(a.K, BITS) ? kWideAboveStaged : kWideAbove;
#ifdef B200_DEV
  if (const char* v = getenv("B200_SMALL_WIDE_ABOVE")) wide_above = atoi(v);
#endif
  const bool wide = per > wide_above && staged_bytes(a.K, 32) <= 200 * 1024;
  // row tiles per CTA: the largest that still gives three CTAs per SM, among those whose K slices
  // (8 / (NMAT * RT) of them, in blocks of four (4-bit) or two (8-bit) groups) all have work.  When even the
  // smallest tiles give fewer CTAs than that, a grid between one and one and a half waves (two CTAs per SM are
  // resident) would run a nearly empty second wave of latency-bound CTAs: the next larger tile, which fits one
  // wave, is taken instead.
  const int gb = BITS == 4 ? 4 : 2;  // groups per block of the weight stream
  const int nblk = (a.K / 64 + gb - 1) / gb;
  const int64_t one_wave = 2 * (int64_t)current_sm_count();
  bool avoid_second_wave = true;
#ifdef B200_DEV
  if (getenv("B200_SMALL_TWO_WAVES")) avoid_second_wave = false;
#endif
  int rt = 8 / NMAT;
  for (int cand = 8 / NMAT; cand >= 1; cand >>= 1) {
    if (8 / (NMAT * cand) > nblk) break;
    const int64_t ctas = (int64_t)cdiv(a.N, 16 * cand) * max_active;
    if (avoid_second_wave && cand < 8 / NMAT && ctas > one_wave && ctas < one_wave * 3 / 2 &&
        (int64_t)cdiv(a.N, 32 * cand) * max_active >= one_wave / 2)
      break;  // keep the previous (larger) tile
    rt = cand;
    if (ctas >= one_wave * 3 / 2) break;
  }
  // few rows per expert: the variant that requests its whole weight slice up front, with the tile chosen above or
  // the next smaller one whose K slices divide the blocks evenly and whose shared memory lets two CTAs share an SM
  // (a handful of tokens, where every CTA prepares its own rows, measured faster on the register stream: 0.0370
  // against 0.0415 ms per block at one token)
  bool try_staged = !wide && !a.x_bf16;
  int rt_first = rt;
#ifdef B200_DEV
  if (getenv("B200_SMALL_NO_STAGED")) try_staged = false;
  if (const char* v = getenv("B200_STAGED_RT")) rt_first = atoi(v) < rt ? atoi(v) : rt;
#endif
  if (try_staged && (a.K / 64) % gb == 0) {
    const int nb = a.K / 64 / gb;
    int pick = 0;
    for (int cand = rt_first; cand >= 1 && !pick; cand >>= 1) {
      const int ks = 8 / (NMAT * cand);
      if (nb % ks == 0 && nb / ks <= 8 && staged_smem_bytes<NMAT>(a.K, BITS, cand) <= kStagedMaxSmem) pick = cand;
    }
#define B200_STAGED_RT(RTV)                                                \
  case RTV:                                                                \
    if constexpr (RTV * NMAT <= 8) return launch_staged<BITS, NMAT, RTV>(a, max_active, st); \
    break;
    switch (pick) {
      B200_STAGED_RT(1)
      B200_STAGED_RT(2)
      B200_STAGED_RT(4)
      B200_STAGED_RT(8)
    }
#undef B200_STAGED_RT
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

bool small_staged_ok(int K, int bits, int nmat) {
  if (K % 64 || (bits != 4 && bits != 8)) return false;
  return nmat == 2 ? staged_feasible<2>(K, bits) : staged_feasible<1>(K, bits);
}

int launch_grouped_qmm_small(const GroupedArgs& a, int nmat, int bits, int max_active, int64_t rows, cudaStream_t st) {
  if (rows == 0 || max_active == 0) return 0;
  B200_REQUIRE(a.K % 64 == 0, "K must be a multiple of the group size 64");
  B200_REQUIRE(small_shape_ok(a.K), "K too large for the staged activation rows");
  if (bits == 4) return nmat == 2 ? launch_bits_nmat<4, 2>(a, max_active, rows, st) : launch_bits_nmat<4, 1>(a, max_active, rows, st);
  if (bits == 8) return nmat == 2 ? launch_bits_nmat<8, 2>(a, max_active, rows, st) : launch_bits_nmat<8, 1>(a, max_active, rows, st);
  B200_FAIL("bits must be 4 or 8");
}

}  // namespace b200

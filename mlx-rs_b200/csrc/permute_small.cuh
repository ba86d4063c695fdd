// Single-chunk (n <= 1024) token -> expert permutation as a block-level device function, shared by
// the stand-alone permutation kernel and the fused small-batch router kernel.
#pragma once
#include <stdint.h>

namespace b200 {

constexpr int kChunk = 1024;

// warp_cnt[w*E + e] := number of assignments of expert e in warp w (shared memory, zeroed by caller)
__device__ __forceinline__ int warp_rank_and_count(uint32_t e, bool valid, int lane, int warp, int E, int* warp_cnt) {
  uint32_t key = valid ? e : 0xffffffffu;
  uint32_t m = __match_any_sync(0xffffffffu, key);
  int rank = __popc(m & ((1u << lane) - 1u));
  if (valid && rank == 0) warp_cnt[warp * E + e] = __popc(m);
  return rank;
}

// All NT threads of the block call this (NT = 1024 / R, R assignments per thread).  `sh` holds
// (32 + 1) * E ints.  Assignment i lives in "virtual warp" i / 32, so the result is identical for
// every NT.  idx may have been written earlier by this block (the caller synchronises).
template <int NT>
__device__ __forceinline__ void permute_small_block(const uint32_t* idx, int n, int E, uint32_t* __restrict__ perm,
                                                    uint32_t* __restrict__ inv, uint32_t* __restrict__ counts,
                                                    uint32_t* __restrict__ offsets, uint32_t* __restrict__ active,
                                                    uint32_t* __restrict__ n_active, int* __restrict__ err, int* sh) {
  constexpr int R = kChunk / NT;
  int* base = sh + 32 * E;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += NT) sh[i] = 0;
  __syncthreads();
  uint32_t e[R];
  bool valid[R];
  int rank[R];
#pragma unroll
  for (int q = 0; q < R; ++q) {
    const int i = q * NT + threadIdx.x;
    valid[q] = i < n;
    e[q] = valid[q] ? __ldcg(idx + i) : 0u;  // possibly written by other CTAs of the same launch: read at L2
    if (valid[q] && e[q] >= (uint32_t)E) {
      *err = 2;
      valid[q] = false;
    }
    rank[q] = warp_rank_and_count(e[q], valid[q], lane, q * (NT / 32) + warp, E, sh);
  }
  __syncthreads();
  for (int ee = threadIdx.x; ee < E; ee += NT) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      int v = sh[w * E + ee];
      sh[w * E + ee] = run;
      run += v;
    }
    base[ee] = run;  // total of expert ee
    counts[ee] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t run = 0, na = 0;
    for (int ee = 0; ee < E; ++ee) {
      uint32_t c = base[ee];
      offsets[ee] = run;
      base[ee] = run;
      if (c) active[na++] = ee;
      run += c;
    }
    offsets[E] = run;
    *n_active = na;
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < R; ++q)
    if (valid[q]) {
      const int i = q * NT + threadIdx.x;
      uint32_t p = base[e[q]] + sh[(q * (NT / 32) + warp) * E + e[q]] + rank[q];
      perm[p] = (uint32_t)i;
      inv[i] = p;
    }
}

}  // namespace b200

// Token -> expert permutation: histogram, exclusive prefix sum and stable scatter.
//
// Replaces the reference composition argsort_axis (mlx-rs/src/ops/sort.rs:57-83) of the
// token-major flat index list, its inverse, floor_divide (mlx-rs/src/ops/arithmetic.rs:401)
// and take_axis (mlx-rs/src/ops/indexing/mod.rs:374-401).  Integer work: every output equals
// what a stable argsort produces, bit for bit, independent of launch geometry:
//   perm[p]   = flat index (token*k + slot) at sorted position p
//   inv[i]    = sorted position of flat index i
//   counts[e] = assignments of expert e,  offsets = exclusive prefix sum ([E+1])
//   active    = ascending list of experts with counts > 0, *n_active its length
//
// The flat list is cut into chunks of 1024 assignments (one per thread).  Inside a chunk the
// stable rank of an assignment is (#same-expert assignments in earlier warps) + (#same-expert
// lanes below it in its warp, from __match_any_sync).  Across chunks a per-expert running sum
// over chunk histograms gives each chunk its base.
#include "common.cuh"
#include "kernels.h"

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

// Phase 1 (multi-chunk path): chunk histograms.  chunk_cnt [nchunks, E]
__global__ void __launch_bounds__(kChunk) permute_hist_kernel(const uint32_t* __restrict__ idx, int n, int E,
                                                              uint32_t* __restrict__ chunk_cnt, int* __restrict__ err) {
  extern __shared__ int sh[];
  for (int i = threadIdx.x; i < E; i += kChunk) sh[i] = 0;
  __syncthreads();
  int i = blockIdx.x * kChunk + threadIdx.x;
  if (i < n) {
    uint32_t e = idx[i];
    if (e < (uint32_t)E)
      atomicAdd(&sh[e], 1);
    else
      *err = 2;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kChunk) chunk_cnt[(size_t)blockIdx.x * E + e] = sh[e];
}

// Phase 2: per-expert running sum over chunks, expert prefix sum, active list.  One CTA.
// On exit chunk_cnt[c,e] holds the absolute base position of expert e's assignments of chunk c.
__global__ void __launch_bounds__(1024) permute_scan_kernel(uint32_t* __restrict__ chunk_cnt, int nchunks, int E,
                                                            uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                                                            uint32_t* __restrict__ active, uint32_t* __restrict__ n_active) {
  extern __shared__ int sh[];  // [E] totals -> exclusive offsets
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    uint32_t run = 0;
    for (int c = 0; c < nchunks; ++c) {
      uint32_t v = chunk_cnt[(size_t)c * E + e];
      chunk_cnt[(size_t)c * E + e] = run;
      run += v;
    }
    sh[e] = run;
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // E is at most a few hundred: a serial scan costs well under a microsecond
    uint32_t run = 0, na = 0;
    for (int e = 0; e < E; ++e) {
      uint32_t c = sh[e];
      offsets[e] = run;
      sh[e] = run;
      if (c) active[na++] = e;
      run += c;
    }
    offsets[E] = run;
    *n_active = na;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int c = 0; c < nchunks; ++c) chunk_cnt[(size_t)c * E + e] += sh[e];
}

// Phase 3: stable scatter of one chunk.
__global__ void __launch_bounds__(kChunk) permute_scatter_kernel(const uint32_t* __restrict__ idx, int n, int E,
                                                                 const uint32_t* __restrict__ chunk_base,
                                                                 uint32_t* __restrict__ perm, uint32_t* __restrict__ inv) {
  extern __shared__ int sh[];  // warp_cnt [32, E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += kChunk) sh[i] = 0;
  __syncthreads();
  int i = blockIdx.x * kChunk + threadIdx.x;
  bool valid = i < n;
  uint32_t e = valid ? idx[i] : 0u;
  valid = valid && e < (uint32_t)E;
  int rank = warp_rank_and_count(e, valid, lane, warp, E, sh);
  __syncthreads();
  for (int ee = threadIdx.x; ee < E; ee += kChunk) {  // exclusive prefix over warps
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      int v = sh[w * E + ee];
      sh[w * E + ee] = run;
      run += v;
    }
  }
  __syncthreads();
  if (valid) {
    uint32_t p = chunk_base[(size_t)blockIdx.x * E + e] + sh[warp * E + e] + rank;
    perm[p] = (uint32_t)i;
    inv[i] = p;
  }
}

// Single-chunk path (n <= 1024): everything in one CTA, one launch.
__global__ void __launch_bounds__(kChunk) permute_small_kernel(const uint32_t* __restrict__ idx, int n, int E,
                                                               uint32_t* __restrict__ perm, uint32_t* __restrict__ inv,
                                                               uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                                                               uint32_t* __restrict__ active, uint32_t* __restrict__ n_active,
                                                               int* __restrict__ err) {
  extern __shared__ int sh[];  // warp_cnt [32, E] then base [E]
  int* base = sh + 32 * E;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += kChunk) sh[i] = 0;
  __syncthreads();
  int i = threadIdx.x;
  bool valid = i < n;
  uint32_t e = valid ? idx[i] : 0u;
  if (valid && e >= (uint32_t)E) {
    *err = 2;
    valid = false;
  }
  int rank = warp_rank_and_count(e, valid, lane, warp, E, sh);
  __syncthreads();
  for (int ee = threadIdx.x; ee < E; ee += kChunk) {
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
  if (valid) {
    uint32_t p = base[e] + sh[warp * E + e] + rank;
    perm[p] = (uint32_t)i;
    inv[i] = p;
  }
}

int launch_permute(const uint32_t* idx, int64_t n, int E, uint32_t* perm, uint32_t* inv, uint32_t* counts,
                   uint32_t* offsets, uint32_t* active, uint32_t* n_active, uint32_t* chunk_scratch, int* err,
                   cudaStream_t st) {
  const size_t sh_scatter = sizeof(int) * 32 * E;
  if (n <= kChunk) {
    permute_small_kernel<<<1, kChunk, sh_scatter + sizeof(int) * E, st>>>(idx, (int)n, E, perm, inv, counts, offsets,
                                                                        active, n_active, err);
    return 0;
  }
  const int nchunks = cdiv(n, kChunk);
  permute_hist_kernel<<<nchunks, kChunk, sizeof(int) * E, st>>>(idx, (int)n, E, chunk_scratch, err);
  permute_scan_kernel<<<1, 1024, sizeof(int) * E, st>>>(chunk_scratch, nchunks, E, counts, offsets, active, n_active);
  permute_scatter_kernel<<<nchunks, kChunk, sh_scatter, st>>>(idx, (int)n, E, chunk_scratch, perm, inv);
  return 0;
}

size_t permute_scratch_words(int64_t n, int E) { return (size_t)cdiv(n, kChunk) * E; }

}  // namespace b200

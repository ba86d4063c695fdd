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
#include "permute_small.cuh"

namespace b200 {

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

// Phase 2: per-expert running sum over chunks, expert prefix sum, active list.  One CTA of 1024
// threads = floor(1024 / E) groups x E experts; a group owns a contiguous range of chunks, so the
// running sums are short chains (a single chain over 64 chunks cost 22 us of load latency).
// On exit chunk_cnt[c,e] holds the absolute base position of expert e's assignments of chunk c.
__global__ void __launch_bounds__(1024) permute_scan_kernel(uint32_t* __restrict__ chunk_cnt, int nchunks, int E,
                                                            uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                                                            uint32_t* __restrict__ active, uint32_t* __restrict__ n_active) {
  extern __shared__ int sh[];  // [ngrp][E] partial sums, then [E] exclusive offsets
  const int ngrp = max(1, (int)blockDim.x / E);
  int* off = sh + ngrp * E;
  const int grp = threadIdx.x / E, e = threadIdx.x % E;
  const bool live = grp < ngrp;
  const int cpg = (nchunks + ngrp - 1) / ngrp;
  const int c0 = min(nchunks, grp * cpg), c1 = min(nchunks, c0 + cpg);
  if (live) {
    uint32_t sum = 0;
    for (int c = c0; c < c1; ++c) sum += chunk_cnt[(size_t)c * E + e];
    sh[grp * E + e] = (int)sum;
  }
  __syncthreads();
  uint32_t before = 0;  // assignments of expert e in the chunks of earlier groups
  if (live) {
    uint32_t total = 0;
    for (int g = 0; g < ngrp; ++g) {
      if (g == grp) before = total;
      total += (uint32_t)sh[g * E + e];
    }
    if (grp == 0) {
      off[e] = (int)total;
      counts[e] = total;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // E is at most a few hundred: a serial scan costs well under a microsecond
    uint32_t run = 0, na = 0;
    for (int ee = 0; ee < E; ++ee) {
      uint32_t c = (uint32_t)off[ee];
      offsets[ee] = run;
      off[ee] = (int)run;
      if (c) active[na++] = ee;
      run += c;
    }
    offsets[E] = run;
    *n_active = na;
  }
  __syncthreads();
  if (live) {
    uint32_t run = (uint32_t)off[e] + before;
    for (int c = c0; c < c1; ++c) {
      const uint32_t v = chunk_cnt[(size_t)c * E + e];
      chunk_cnt[(size_t)c * E + e] = run;
      run += v;
    }
  }
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
  pdl_prologue();
  permute_small_block<kChunk>(idx, n, E, perm, inv, counts, offsets, active, n_active, err, sh);
}

int launch_permute(const uint32_t* idx, int64_t n, int E, uint32_t* perm, uint32_t* inv, uint32_t* counts,
                   uint32_t* offsets, uint32_t* active, uint32_t* n_active, uint32_t* chunk_scratch, int* err,
                   cudaStream_t st) {
  const size_t sh_scatter = sizeof(int) * 32 * E;
  if (n <= kChunk) {
    B200_CUDA(launch_pdl(permute_small_kernel, dim3(1), dim3(kChunk), sh_scatter + sizeof(int) * E, st, idx, (int)n, E, perm, inv,
                         counts, offsets, active, n_active, err));
    return 0;
  }
  const int nchunks = cdiv(n, kChunk);
  permute_hist_kernel<<<nchunks, kChunk, sizeof(int) * E, st>>>(idx, (int)n, E, chunk_scratch, err);
  permute_scan_kernel<<<1, 1024, sizeof(int) * (1024 / E + 1) * E, st>>>(chunk_scratch, nchunks, E, counts, offsets, active,
                                                                          n_active);
  permute_scatter_kernel<<<nchunks, kChunk, sh_scatter, st>>>(idx, (int)n, E, chunk_scratch, perm, inv);
  return 0;
}

size_t permute_scratch_words(int64_t n, int E) { return (size_t)cdiv(n, kChunk) * E; }


// ---------------------------------------------------------------------------------------
// Allocation-free variant of the token -> expert sort.
//
// b200_moe_permute needs scratch in global memory (the chunk table, the list of active
// experts) and takes it from the context's arena, which is grown with cudaMalloc.  Some
// callers cannot live with that: a serving process that hands all of the device's memory to
// its own pool at start-up (so a later cudaMalloc by a library fails or fragments the pool),
// or a latency-critical token loop that must never hit the implicit device-wide
// synchronisation of cudaMalloc / cudaFree.  For them the same kernels run here on a scratch
// area that is part of the library image: a file-scope __device__ array of fixed size.  Every
// GPU that loads the library carries these 258 KB until the process exits.
//
// In host code the array's name is only a host-side handle, not a device address, so the
// address is looked up once per device with cudaGetSymbolAddress (with that device current)
// and cached; kernels receive that pointer.
// ---------------------------------------------------------------------------------------
constexpr int kStaticTableWords = 1 << 16;  // chunk table capacity: ceil(n/1024) * n_experts <= 65536
constexpr int kStaticTailWords = 512;       // active list (<= 257), n_active, status word
static __device__ __align__(256) uint32_t g_permute_static_scratch[kStaticTableWords + kStaticTailWords];

static uint32_t* g_static_scratch_addr[kMaxDevices] = {};

}  // namespace b200

extern "C" int b200_moe_permute_static(const uint32_t* indices, int64_t n, int n_experts, uint32_t* perm,
                                       uint32_t* inv_perm, uint32_t* counts, uint32_t* offsets, void* stream) {
  using namespace b200;
  B200_REQUIRE(n_experts > 0 && n_experts <= 256, "n_experts must be in 1..256");
  B200_REQUIRE(n >= 0 && n < (int64_t(1) << 31), "bad assignment count");
  B200_REQUIRE(counts && offsets, "counts and offsets are required");
  B200_REQUIRE(n == 0 || (indices && perm && inv_perm), "null tensor");
  B200_REQUIRE(permute_scratch_words(n, n_experts) <= (size_t)kStaticTableWords,
               "problem exceeds the static scratch: ceil(n/1024) * n_experts must not exceed 65536 "
               "(use b200_moe_permute, which allocates, for larger inputs)");
  int dev = -1;
  B200_CUDA(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal out of range");
  if (!g_static_scratch_addr[dev]) {  // set-up on the first call on this device
    uint32_t* ptr = nullptr;
    B200_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_permute_static_scratch));
    B200_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned a null address");
    g_static_scratch_addr[dev] = ptr;
  }
  uint32_t* base = g_static_scratch_addr[dev];
  uint32_t* active = base + kStaticTableWords;
  uint32_t* n_active = active + 260;
  int* status = reinterpret_cast<int*>(active + 264);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  Nothing in it has to start at zero: the chunk
  // table, the active list and n_active are fully rewritten by the kernels before they are read, and
  // the status word is write-only (the kernels set it when they skip an out-of-range expert index;
  // nothing reads it back - this entry point has no context to report through).
  launch_permute(indices, n, n_experts, perm, inv_perm, counts, offsets, active, n_active, base, status, st);
  cudaError_t le = cudaGetLastError();
  if (le != cudaSuccess) B200_FAIL(std::string("kernel launch failed: ") + cudaGetErrorString(le));
  return 0;
}

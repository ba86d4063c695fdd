// Expert-parallel exchange over peer memory (one process per GPU, all GPUs of one NVSwitch node).
//
// The reference has no distributed layer; these kernels exist because the routed block shards
// naturally by expert.  Rank r owns the contiguous experts [r*Eg, (r+1)*Eg).  Every rank holds two
// exchange buffers that its peers map (CUDA IPC): `rows` (tokens arriving for its experts) and
// `y` (its experts' outputs).  Both use the same row numbering on the owning rank:
//
//     [local expert 0: rows from rank 0 | rank 1 | ... ][local expert 1: ...] ...
//
// so arriving rows are already grouped by expert and the grouped products run on them in place.
//   dispatch : the gather into expert order and the send are one kernel - each sorted row is read
//              from this rank's tokens and stored straight into the owner's `rows` buffer
//              (plain 16-byte peer stores over NVLink).
//   combine  : the return and the weighted k-way sum are one kernel - each token reads its k
//              expert outputs straight out of the owners' `y` buffers (peer loads) and
//              accumulates in float32.
// Neither kernel waits on another GPU.  Ordering between ranks comes from stream-ordered
// collectives issued by the host layer between the phases (a kernel's peer stores are complete
// when it ends; a collective that every rank joins after that kernel cannot finish anywhere
// before all of those kernels have ended).
#include "common.cuh"
#include "kernels.h"

namespace b200 {

// ---- segment tables from per-expert counts ------------------------------------------------
__global__ void segments_from_counts_kernel(const uint32_t* __restrict__ counts, int E, uint32_t* __restrict__ offsets,
                                            uint32_t* __restrict__ active, uint32_t* __restrict__ n_active) {
  if (threadIdx.x != 0) return;
  uint32_t run = 0, na = 0;
  for (int e = 0; e < E; ++e) {
    offsets[e] = run;
    const uint32_t c = counts[e];
    if (c) active[na++] = e;
    run += c;
  }
  offsets[E] = run;
  *n_active = na;
}

int launch_segments_from_counts(const uint32_t* counts, int E, uint32_t* offsets, uint32_t* active, uint32_t* n_active,
                                cudaStream_t st) {
  segments_from_counts_kernel<<<1, 32, 0, st>>>(counts, E, offsets, active, n_active);
  return 0;
}

// ---- where this rank's rows land on their owners ---------------------------------------------
// all_counts[s*E + e] = rows that rank s routes to expert e.  For this rank (`rank`):
//   dst_row0[e]     = row, in the buffers of the rank that owns e, of this rank's first row of e
//   local_counts[l] = rows arriving here for local expert l (summed over sources)
// *err is set when a rank would receive more than `capacity` rows.
__global__ void ep_layout_kernel(const uint32_t* __restrict__ all_counts, int G, int E, int rank, uint32_t capacity,
                                 uint32_t* __restrict__ dst_row0, uint32_t* __restrict__ local_counts,
                                 int* __restrict__ err) {
  const int Eg = E / G;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / Eg, first = d * Eg;
    uint32_t row = 0;
    for (int f = first; f < e; ++f)
      for (int s = 0; s < G; ++s) row += all_counts[s * E + f];
    for (int s = 0; s < rank; ++s) row += all_counts[s * E + e];
    dst_row0[e] = row;
    if (row + all_counts[rank * E + e] > capacity) *err = 5;
    if (d == rank) {
      uint32_t c = 0;
      for (int s = 0; s < G; ++s) c += all_counts[s * E + e];
      local_counts[e - first] = c;
    }
  }
}

int launch_ep_layout(const uint32_t* all_counts, int G, int E, int rank, uint32_t capacity, uint32_t* dst_row0,
                     uint32_t* local_counts, int* err, cudaStream_t st) {
  ep_layout_kernel<<<1, 256, 0, st>>>(all_counts, G, E, rank, capacity, dst_row0, local_counts, err);
  return 0;
}

// ---- dispatch: gather into expert order + store to the owning rank ----------------------------
// Sorted position j holds assignment a = perm[j] (token a / k, expert idx[a]).
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const uint4* __restrict__ x, const uint32_t* __restrict__ idx,
                                                          const uint32_t* __restrict__ perm,
                                                          const uint32_t* __restrict__ offsets,
                                                          const uint32_t* __restrict__ dst_row0, int64_t n, uint32_t k,
                                                          int vec_per_row, int E, int Eg, int rank, EpPeers peers,
                                                          uint32_t capacity, int* __restrict__ err) {
  // Sorted rows are grouped by destination rank (contiguous experts).  Walking them front to back
  // would make every source write to destination 0 first, then 1, ...: all GPUs on one ingress
  // link at a time (measured at 8 GPUs: 0.44 ms + 0.23 ms of waiting for the slowest rank).  Each
  // source therefore starts with the destination after itself and wraps around, the classic
  // all-to-all schedule; its own rows come last.
  __shared__ uint32_t s_cum[kEpMaxRanks + 1], s_base[kEpMaxRanks];
  const int G = E / Eg;
  if (threadIdx.x == 0) {
    uint32_t run = 0;
    for (int i = 0; i < G; ++i) {
      const int d = (rank + 1 + i) % G;
      const uint32_t b = offsets[d * Eg], e_ = offsets[(d + 1) * Eg];
      s_base[i] = b;
      s_cum[i] = run;
      run += e_ - b;
    }
    s_cum[G] = run;
  }
  __syncthreads();
  // one warp per row; a lane keeps eight 16-byte pieces in flight before it stores them
  const int lane = threadIdx.x & 31, wpc = blockDim.x >> 5;
  for (int64_t v = (int64_t)blockIdx.x * wpc + (threadIdx.x >> 5); v < n; v += (int64_t)gridDim.x * wpc) {
    int i = 0;
    while (i + 1 < G && (uint32_t)v >= s_cum[i + 1]) ++i;
    const int64_t j = (int64_t)s_base[i] + (v - (int64_t)s_cum[i]);
    if (j >= n) {   // counts that do not add up to n: a routing table that does not belong to these rows
      if (lane == 0) *err = 6;
      continue;
    }
    const uint32_t a = perm[j];
    if (a >= n) {
      if (lane == 0) *err = 6;
      continue;
    }
    const uint32_t e = idx[a];
    if (e >= (uint32_t)E) {
      if (lane == 0) *err = 6;
      continue;
    }
    const uint32_t row = dst_row0[e] + (uint32_t)j - offsets[e];
    if (row >= capacity) {
      if (lane == 0) *err = 5;
      continue;
    }
    const uint4* src = x + (size_t)(a / k) * vec_per_row;
    uint4* dst = static_cast<uint4*>(peers.p[e / Eg]) + (size_t)row * vec_per_row;
    for (int c0 = 0; c0 < vec_per_row; c0 += 256) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < vec_per_row) v[u] = __ldg(src + c);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < vec_per_row) dst[c] = v[u];
      }
    }
  }
}

int launch_ep_dispatch(const void* x, const uint32_t* idx, const uint32_t* perm, const uint32_t* offsets,
                       const uint32_t* dst_row0, int64_t n, int k, int64_t H, int E, int G, int rank, const EpPeers& peers,
                       uint32_t capacity, int* err, cudaStream_t st) {
  if (n == 0) return 0;
  // 128 threads x 32 registers: small enough to share an SM with a resident 608-thread tensor-core CTA
  // (7168 registers are left beside it), so that a dispatch on a side stream overlaps the products
  const int grid = (int)(n < 148 * 16 ? n : 148 * 16);
  ep_dispatch_kernel<<<grid, 128, 0, st>>>(static_cast<const uint4*>(x), idx, perm, offsets, dst_row0, n, (uint32_t)k,
                                           (int)(H / 8), E, E / G, rank, peers, capacity, err);
  return 0;
}

// ---- return path fused into the down projection ------------------------------------------------
// For every row this rank received (numbered by local expert, source rank, source order) the address
// of its output row in the SOURCE rank's return buffer, which is laid out in the source's own sorted
// order: row (offsets_s[e] + j) for the j-th row rank s routed to expert e.  The grouped product's
// epilogue stores each finished row straight to that address (peer stores), so the transfer back
// overlaps the products tile by tile and the source's combine reads local memory only.
// One CTA per (local expert, source rank) segment.
__global__ void __launch_bounds__(256) ep_return_table_kernel(const uint32_t* __restrict__ all_counts, int G, int E,
                                                              int rank, EpPeers peers_y, int64_t row_bytes,
                                                              unsigned long long* __restrict__ row_addr) {
  const int Eg = E / G;
  const int el = blockIdx.x / G, s = blockIdx.x % G;
  const int e = rank * Eg + el;
  __shared__ uint32_t s_start, s_src0;
  if (threadIdx.x == 0) {
    uint32_t start = 0;
    for (int f = rank * Eg; f < e; ++f)
      for (int q = 0; q < G; ++q) start += all_counts[q * E + f];
    for (int q = 0; q < s; ++q) start += all_counts[q * E + e];
    uint32_t src0 = 0;
    for (int f = 0; f < e; ++f) src0 += all_counts[s * E + f];
    s_start = start;
    s_src0 = src0;
  }
  __syncthreads();
  const uint32_t len = all_counts[s * E + e];
  const unsigned long long base = reinterpret_cast<unsigned long long>(peers_y.p[s]);
  for (uint32_t j = threadIdx.x; j < len; j += blockDim.x)
    row_addr[s_start + j] = base + (unsigned long long)(s_src0 + j) * (unsigned long long)row_bytes;
}

int launch_ep_return_table(const uint32_t* all_counts, int G, int E, int rank, const EpPeers& peers_y, int64_t H,
                           unsigned long long* row_addr, cudaStream_t st) {
  ep_return_table_kernel<<<(E / G) * G, 256, 0, st>>>(all_counts, G, E, rank, peers_y, H * 2, row_addr);
  return 0;
}

// ---- combine: read the k expert outputs from their owners + weighted sum ------------------------
// out[t, :] = bf16( sum_j score[t, j] * y_owner(idx[t,j])[row(t, j), :] ), float32 accumulation, j ascending.
__device__ __forceinline__ uint4 ld_cg_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

constexpr int kEpMaxTopK = 32;

__global__ void __launch_bounds__(256) ep_combine_kernel(EpPeers peers, const uint32_t* __restrict__ idx,
                                                         const uint32_t* __restrict__ inv,
                                                         const uint32_t* __restrict__ offsets,
                                                         const uint32_t* __restrict__ dst_row0,
                                                         const unsigned short* __restrict__ scores, int64_t T, int k,
                                                         int vec_per_row, int E, int Eg, uint32_t capacity,
                                                         uint4* __restrict__ out, int* __restrict__ err) {
  __shared__ const uint4* s_row[kEpMaxTopK];
  __shared__ float s_w[kEpMaxTopK];
  for (int64_t t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < k) {
      const int64_t a = t * k + threadIdx.x;
      const uint32_t e = idx[a];
      const uint4* ptr = nullptr;
      if (e < (uint32_t)E) {
        const uint32_t row = dst_row0[e] + inv[a] - offsets[e];
        if (row < capacity) ptr = static_cast<const uint4*>(peers.p[e / Eg]) + (size_t)row * vec_per_row;
      }
      if (!ptr) *err = 6;
      s_row[threadIdx.x] = ptr;
      s_w[threadIdx.x] = bf16_bits_to_f32(scores[a]);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      int j = 0;
      for (; j + 4 <= k; j += 4) {  // four peer loads in flight per thread
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = s_row[j + u] ? ld_cg_v4(s_row[j + u] + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float s = s_w[j + u];
          const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            acc[2 * q] += s * __uint_as_float(w[q] << 16);
            acc[2 * q + 1] += s * __uint_as_float(w[q] & 0xffff0000u);
          }
        }
      }
      for (; j < k; ++j) {
        const uint4 v = s_row[j] ? ld_cg_v4(s_row[j] + c) : make_uint4(0, 0, 0, 0);
        const float s = s_w[j];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[2 * q] += s * __uint_as_float(w[q] << 16);
          acc[2 * q + 1] += s * __uint_as_float(w[q] & 0xffff0000u);
        }
      }
      uint4 o;
      o.x = f32_to_bf16_bits(acc[0]) | (f32_to_bf16_bits(acc[1]) << 16);
      o.y = f32_to_bf16_bits(acc[2]) | (f32_to_bf16_bits(acc[3]) << 16);
      o.z = f32_to_bf16_bits(acc[4]) | (f32_to_bf16_bits(acc[5]) << 16);
      o.w = f32_to_bf16_bits(acc[6]) | (f32_to_bf16_bits(acc[7]) << 16);
      out[(size_t)t * vec_per_row + c] = o;
    }
  }
}

int launch_ep_combine(const EpPeers& peers, const uint32_t* idx, const uint32_t* inv, const uint32_t* offsets,
                      const uint32_t* dst_row0, const void* scores, int64_t T, int k, int64_t H, int E, int G,
                      uint32_t capacity, void* out, int* err, cudaStream_t st) {
  if (T == 0) return 0;
  B200_REQUIRE(k <= kEpMaxTopK, "top_k above 32");
  const int grid = (int)(T < 148 * 16 ? T : 148 * 16);
  ep_combine_kernel<<<grid, 128, 0, st>>>(peers, idx, inv, offsets, dst_row0, static_cast<const unsigned short*>(scores), T,
                                          k, (int)(H / 8), E, E / G, capacity, static_cast<uint4*>(out), err);
  return 0;
}

}  // namespace b200

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
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

// two float32 -> packed fp16 pair (lo in the low half), round to nearest, finite overflow saturates
__device__ __forceinline__ uint32_t f16x2_sat_bits(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// ---- segment tables from per-expert counts ------------------------------------------------
// counts_out is counts cut off where the running sum would pass n_rows (the rows the caller's buffers hold): the
// grouped products walk counts_out / offsets, so counts that promise more rows than exist cannot make them read or
// write past the buffers; *err = 6 reports the cut.
__global__ void segments_from_counts_kernel(const uint32_t* __restrict__ counts, int E, int64_t n_rows,
                                            uint32_t* __restrict__ counts_out, uint32_t* __restrict__ offsets,
                                            uint32_t* __restrict__ active, uint32_t* __restrict__ n_active,
                                            int* __restrict__ err) {
  if (threadIdx.x != 0) return;
  uint32_t run = 0, na = 0;
  for (int e = 0; e < E; ++e) {
    offsets[e] = run;
    uint32_t c = counts[e];
    if ((int64_t)run + c > n_rows) {
      c = (uint32_t)(n_rows - run);
      *err = 6;
    }
    counts_out[e] = c;
    if (c) active[na++] = e;
    run += c;
  }
  offsets[E] = run;
  *n_active = na;
}

int launch_segments_from_counts(const uint32_t* counts, int E, int64_t n_rows, uint32_t* counts_out, uint32_t* offsets,
                                uint32_t* active, uint32_t* n_active, int* err, cudaStream_t st) {
  segments_from_counts_kernel<<<1, 32, 0, st>>>(counts, E, n_rows, counts_out, offsets, active, n_active, err);
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
    if (dst_row0[e] == 0xffffffffu) continue;  // the owner would overflow: it takes no rows this step (status 5 is set)
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
                                                              int rank, EpPeers peers_y, int64_t row_bytes, int64_t n_rows,
                                                              int64_t capacity_rows,
                                                              unsigned long long* __restrict__ row_addr,
                                                              int* __restrict__ err) {
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
  for (uint32_t j = threadIdx.x; j < len; j += blockDim.x) {
    const int64_t slot = (int64_t)s_start + j, dst = (int64_t)s_src0 + j;
    if (slot >= n_rows) {  // the table itself ends here
      *err = 5;
      continue;
    }
    if (dst >= capacity_rows) {  // the source's return buffer ends before this row: address 0 = "drop the row"
      *err = 5;
      row_addr[slot] = 0ull;
      continue;
    }
    row_addr[slot] = base + (unsigned long long)dst * (unsigned long long)row_bytes;
  }
}

int launch_ep_return_table(const uint32_t* all_counts, int G, int E, int rank, const EpPeers& peers_y, int64_t H, int64_t n_rows,
                           int64_t capacity_rows, unsigned long long* row_addr, int* err, cudaStream_t st) {
  ep_return_table_kernel<<<(E / G) * G, 256, 0, st>>>(all_counts, G, E, rank, peers_y, H * 2, n_rows, capacity_rows, row_addr, err);
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
      const bool dropped = e < (uint32_t)E && dst_row0[e] == 0xffffffffu;  // owner overflowed (status 5): contributes zero
      if (e < (uint32_t)E && !dropped) {
        const uint32_t row = dst_row0[e] + inv[a] - offsets[e];
        if (row < capacity) ptr = static_cast<const uint4*>(peers.p[e / Eg]) + (size_t)row * vec_per_row;
      }
      if (!ptr && !dropped) *err = 6;
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


// ---- device-side synchronisation between the ranks (one process per GPU) -------------------------------
// The one-call expert-parallel block (b200_moe_block_forward_ep) needs no host round trip and no collective
// library: every rank owns a small control block that its peers map, and three tiny kernels per step order the
// phases through it with release stores and bounded acquire spins.  Layout of a control block (32-bit words):
//     counts_in   [G][E]   rows rank s routes to expert e (written by rank s: the all-gather of the counts)
//     flag_counts [G]      step number up to which rank s has published its counts here
//     flag_rows   [G]      step number up to which rank s has finished storing its rows into this rank's buffer
//     flag_done   [G]      step number up to which rank s has finished its experts' outputs (written by rank s
//                          into EVERY rank's block: "my y buffer may be read")
//     epoch                this rank's own step counter (local)
// A flag only ever grows, waits compare with >=, so a fast peer that is already one step ahead does no harm.
// Single buffering is safe: a rank stores into a peer's buffers for step i+1 only after its own combine of step
// i, which waited for every peer's flag_done of step i, i.e. until the peer had finished reading what step i
// put there (its rows, the count table) - see the order of the calls in b200_moe_block_forward_ep.
// Every wait gives up after 2 s, raises the context's status word (3) and lets the step run to its end on
// whatever is there; nothing is ever waited for without a bound.  These kernels must not be used with two ranks
// on one GPU (nothing guarantees that both run at the same time).
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool ep_wait_ge(const uint32_t* p, uint32_t target) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
    __nanosleep(100);
    if ((it & 63u) == 63u) {
      uint64_t now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0)
        t0 = now;
      else if (now - t0 > 2000000000ull)
        return false;
    }
  }
}

__host__ __device__ inline size_t ep_ctl_words(int G, int E) { return (size_t)G * (E + G) + 3 * (size_t)G + 8; }
size_t ep_ctl_bytes(int G, int E) { return sizeof(uint32_t) * ep_ctl_words(G, E); }
// control block: counts_in [G][E + G] (per source: its E per-expert counts, then its token rows per destination),
// flag_counts [G], flag_rows [G], flag_done [G], epoch
__device__ __forceinline__ uint32_t* ctl_of(const EpExchange& x, int r) { return static_cast<uint32_t*>(x.peer[kEpCtl][r]); }

// ---- which tokens go to which rank ---------------------------------------------------------------------------
// One CTA per destination rank d: flag[t] = some expert of token t lives on d; slot[d][t] = number of flagged tokens
// before t (token order is kept), ntok[d] = their number.
__global__ void __launch_bounds__(1024) ep_token_slots_kernel(const uint32_t* __restrict__ idx, int T, int k, int Eg,
                                                              uint32_t* __restrict__ slot, uint32_t* __restrict__ ntok) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_run;
  const int d = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_run = 0;
  __syncthreads();
  for (int base = 0; base < T; base += 1024) {
    const int t = base + threadIdx.x;
    bool flag = false;
    if (t < T)
      for (int j = 0; j < k; ++j) flag |= (int)(idx[(size_t)t * k + j] / (uint32_t)Eg) == d;
    const uint32_t m = __ballot_sync(0xffffffffu, flag);
    if (lane == 0) s_warp[warp] = __popc(m);
    __syncthreads();
    uint32_t before = s_run;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    if (t < T) slot[(size_t)d * T + t] = flag ? before + __popc(m & ((1u << lane) - 1u)) : 0xffffffffu;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t tot = 0;
      for (int w = 0; w < 32; ++w) tot += s_warp[w];
      s_run += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) ntok[d] = s_run;
}

int launch_ep_token_slots(const uint32_t* idx, int64_t T, const EpExchange& x, uint32_t* slot, cudaStream_t st) {
  ep_token_slots_kernel<<<x.G, 1024, 0, st>>>(idx, (int)T, x.k, x.E / x.G, slot, x.ntok);
  return 0;
}

// Step begin: bump the local step counter, publish this rank's per-expert counts and per-destination token counts
// in every rank's block, wait for everybody's, then compute the layout of the exchange:
//   dst_row0[e]   row, in the owner's assignment order, of this rank's first assignment of expert e
//   tokbase[d]    row, in rank d's token buffer, of this rank's first token row
//   local_counts  assignments arriving here per local expert, *n_recv their total, *n_tok_recv the token rows
// A rank that would overflow either buffer takes nothing this step (status 5): every source marks it as dropped
// (0xffffffff) and it sees zero arrivals itself, so nothing is stored or multiplied out of bounds.
__global__ void __launch_bounds__(256) ep_counts_exchange_kernel(EpExchange x, const uint32_t* __restrict__ counts,
                                                                 int* __restrict__ err) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_fail;
  __shared__ uint32_t s_rows[kEpMaxRanks], s_toks[kEpMaxRanks];
  const int G = x.G, E = x.E, rank = x.rank, W = E + G;
  uint32_t* mine = ctl_of(x, rank);
  uint32_t* epoch_word = mine + (size_t)G * W + 3 * G;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_word + 1u;
    *epoch_word = s_epoch;
    s_fail = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  for (int i = threadIdx.x; i < G * W; i += blockDim.x) {
    const int d = i / W, w = i % W;
    ctl_of(x, d)[(size_t)rank * W + w] = w < E ? counts[w] : x.ntok[w - E];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < G) {
    st_release_sys(ctl_of(x, threadIdx.x) + (size_t)G * W + rank, epoch);
    if (!ep_wait_ge(mine + (size_t)G * W + threadIdx.x, epoch)) s_fail = 1;
  }
  __syncthreads();
  if (s_fail && threadIdx.x == 0) atomicExch(err, 3);
  const volatile uint32_t* all = mine;  // [G][W], written by the peers: read around the L1
  const int Eg = E / G;
  if (threadIdx.x < G) {  // what arrives on rank threadIdx.x
    const int d = threadIdx.x;
    uint32_t rows = 0, toks = 0;
    for (int s = 0; s < G; ++s) {
      for (int e = d * Eg; e < (d + 1) * Eg; ++e) rows += all[s * W + e];
      toks += all[s * W + E + d];
    }
    const bool over = rows > x.cap_rows || toks > x.cap_tok;
    if (over) *err = 5;
    s_rows[d] = over ? 0xffffffffu : rows;
    s_toks[d] = toks;
    uint32_t tb = 0;
    for (int s = 0; s < rank; ++s) tb += all[s * W + E + d];
    x.tokbase[d] = over ? 0xffffffffu : tb;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / Eg, first = d * Eg;
    const bool over = s_rows[d] == 0xffffffffu;
    uint32_t row = 0;
    for (int f = first; f < e; ++f)
      for (int s = 0; s < G; ++s) row += all[s * W + f];
    for (int s = 0; s < rank; ++s) row += all[s * W + e];
    x.dst_row0[e] = over ? 0xffffffffu : row;
    if (d == rank) {
      uint32_t c = 0;
      for (int s = 0; s < G; ++s) c += all[s * W + e];
      x.local_counts[e - first] = over ? 0u : c;
    }
  }
  if (threadIdx.x == 0) {
    const bool over = s_rows[rank] == 0xffffffffu;
    *x.n_recv = over ? 0u : s_rows[rank];
    *x.n_tok_recv = over ? 0u : s_toks[rank];
  }
}

// which: 1 = "my rows are stored in your buffers" (flag_rows), 2 = "my partial sums are complete" (flag_done).
// Signals every peer, then waits until every peer has signalled this rank.  The kernels whose stores are being
// announced ran earlier on the same stream.
__global__ void __launch_bounds__(32) ep_signal_wait_kernel(EpExchange x, int which, int* __restrict__ err) {
  const int G = x.G, W = x.E + x.G;
  uint32_t* mine = ctl_of(x, x.rank);
  const uint32_t epoch = mine[(size_t)G * W + 3 * G];
  const size_t off = (size_t)G * W + (size_t)which * G;
  __threadfence_system();
  if ((int)threadIdx.x < G) {
    st_release_sys(ctl_of(x, threadIdx.x) + off + x.rank, epoch);
    if (!ep_wait_ge(mine + off + threadIdx.x, epoch)) atomicExch(err, 3);
  }
}

__global__ void add_u32_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, int n, uint32_t* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + b[i];
}
int launch_add_u32(const uint32_t* a, const uint32_t* b, int n, uint32_t* out, cudaStream_t st) {
  if (n > 0) add_u32_kernel<<<cdiv(n, 256), 256, 0, st>>>(a, b, n, out);
  return 0;
}

int launch_ep_counts_exchange(const EpExchange& x, const uint32_t* counts, int* err, cudaStream_t st) {
  ep_counts_exchange_kernel<<<1, 256, 0, st>>>(x, counts, err);
  return 0;
}
int launch_ep_signal_wait(const EpExchange& x, int which, int* err, cudaStream_t st) {
  ep_signal_wait_kernel<<<1, 32, 0, st>>>(x, which, err);
  return 0;
}

// ---- de-duplicated dispatch ------------------------------------------------------------------------------------
// A token travels ONCE to every rank that owns at least one of its experts (not once per assignment): one warp per
// (destination, token) pair stores the token row into the destination's token buffer and, per assignment of the
// token on that rank, the bookkeeping the owner needs - rowmap[assignment row] = token row (the gather index of
// its grouped products), and per token row the k assignment rows and routing weights (the list its partial sum
// walks; 0xffffffff = slot j of the token belongs to another rank).  Destinations are visited in all-to-all order
// (the rank after this one first), so that the ranks do not all store into the same GPU at the same time.
__global__ void __launch_bounds__(128) ep_dispatch_dedup_kernel(const uint4* __restrict__ xrows, const uint32_t* __restrict__ idx,
                                                                const uint32_t* __restrict__ inv,
                                                                const uint32_t* __restrict__ offsets,
                                                                const unsigned short* __restrict__ scores,
                                                                const uint32_t* __restrict__ slot, int T, EpExchange x,
                                                                int* __restrict__ err) {
  const int G = x.G, Eg = x.E / x.G, k = x.k, vec_per_row = (int)(x.H / 8);
  const int lane = threadIdx.x & 31, wpc = blockDim.x >> 5;
  const int64_t pairs = (int64_t)G * T;
  for (int64_t p = (int64_t)blockIdx.x * wpc + (threadIdx.x >> 5); p < pairs; p += (int64_t)gridDim.x * wpc) {
    const int d = (x.rank + 1 + (int)(p / T)) % G, t = (int)(p % T);
    const uint32_t sl = slot[(size_t)d * T + t];
    const uint32_t tb = x.tokbase[d];
    if (sl == 0xffffffffu || tb == 0xffffffffu) continue;  // no expert of the token there / the rank takes no rows this step
    const uint32_t trow = tb + sl;
    if (trow >= x.cap_tok) {
      if (lane == 0) *err = 6;
      continue;
    }
    const uint4* src = xrows + (size_t)t * vec_per_row;
    uint4* dst = static_cast<uint4*>(x.peer[kEpTok][d]) + (size_t)trow * vec_per_row;
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
    if (lane < k) {
      const size_t a = (size_t)t * k + lane;
      const uint32_t e = idx[a];
      uint32_t orow = 0xffffffffu;
      if (e < (uint32_t)x.E && (int)(e / (uint32_t)Eg) == d && x.dst_row0[e] != 0xffffffffu) {
        orow = x.dst_row0[e] + inv[a] - offsets[e];
        if (orow >= x.cap_rows) {
          *err = 6;
          orow = 0xffffffffu;
        } else {
          static_cast<uint32_t*>(x.peer[kEpRowMap][d])[orow] = trow;
        }
      }
      static_cast<uint32_t*>(x.peer[kEpSlotRows][d])[(size_t)trow * k + lane] = orow;
      static_cast<unsigned short*>(x.peer[kEpSlotScores][d])[(size_t)trow * k + lane] = scores[a];
    }
  }
}

int launch_ep_dispatch_dedup(const void* xrows, const uint32_t* idx, const uint32_t* inv, const uint32_t* offsets,
                             const void* scores, const uint32_t* slot, int64_t T, const EpExchange& x, int* err, cudaStream_t st) {
  if (T == 0) return 0;
  const int64_t pairs = (int64_t)x.G * T;
  const int grid = (int)(pairs / 4 + 1 < 148 * 16 ? pairs / 4 + 1 : 148 * 16);
  ep_dispatch_dedup_kernel<<<grid, 128, 0, st>>>(static_cast<const uint4*>(xrows), idx, inv, offsets,
                                                 static_cast<const unsigned short*>(scores), slot, (int)T, x, err);
  return 0;
}

// ---- owner: partial weighted sums per arrived token ------------------------------------------------------------
// part[token row, :] = fp16( sum_j score_j * y[assignment row j, :] ) over the token's assignments on this rank, float32
// accumulation, slot order j ascending.  y holds this rank's expert outputs by assignment row (local memory; fp16
// from the tensor-core kernel, bf16 from the register kernel).  fp16's 11 significant bits keep the partial sums'
// rounding well inside the output tolerance (bf16's 8 would use most of it up).
template <bool Y_F16>
__global__ void __launch_bounds__(128) ep_partial_combine_kernel(const uint4* __restrict__ y, EpExchange x, int* __restrict__ err) {
  __shared__ const uint4* s_row[kEpMaxTopK];
  __shared__ float s_w[kEpMaxTopK];
  const int k = x.k, vec_per_row = (int)(x.H / 8);
  const uint32_t n_tok = *x.n_tok_recv;
  const uint32_t* slot_rows = static_cast<const uint32_t*>(x.peer[kEpSlotRows][x.rank]);
  const unsigned short* slot_scores = static_cast<const unsigned short*>(x.peer[kEpSlotScores][x.rank]);
  uint4* part = static_cast<uint4*>(x.peer[kEpPart][x.rank]);
  for (uint32_t r = blockIdx.x; r < n_tok; r += gridDim.x) {
    __syncthreads();
    if ((int)threadIdx.x < k) {
      const uint32_t orow = __ldcg(slot_rows + (size_t)r * k + threadIdx.x);  // written by a peer: around the L1
      const uint4* ptr = nullptr;
      if (orow != 0xffffffffu) {
        if (orow < x.cap_rows)
          ptr = y + (size_t)orow * vec_per_row;
        else
          *err = 6;
      }
      s_row[threadIdx.x] = ptr;
      s_w[threadIdx.x] = bf16_bits_to_f32(__ldcg(slot_scores + (size_t)r * k + threadIdx.x));
    }
    __syncthreads();
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        if (!s_row[j]) continue;
        const uint4 v = __ldg(s_row[j] + c);
        const float w = s_w[j];
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if constexpr (Y_F16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[q]));
            acc[2 * q] += w * f.x;
            acc[2 * q + 1] += w * f.y;
          } else {
            acc[2 * q] += w * __uint_as_float(u[q] << 16);
            acc[2 * q + 1] += w * __uint_as_float(u[q] & 0xffff0000u);
          }
        }
      }
      uint4 o;
      o.x = f16x2_sat_bits(acc[0], acc[1]);
      o.y = f16x2_sat_bits(acc[2], acc[3]);
      o.z = f16x2_sat_bits(acc[4], acc[5]);
      o.w = f16x2_sat_bits(acc[6], acc[7]);
      part[(size_t)r * vec_per_row + c] = o;
    }
  }
}

int launch_ep_partial_combine(const void* y, bool y_f16, const EpExchange& x, int* err, cudaStream_t st) {
  B200_REQUIRE(x.k <= kEpMaxTopK, "top_k above 32");
  const int grid = (int)(x.cap_tok < 148u * 16u ? x.cap_tok : 148u * 16u);
  if (y_f16)
    ep_partial_combine_kernel<true><<<grid, 128, 0, st>>>(static_cast<const uint4*>(y), x, err);
  else
    ep_partial_combine_kernel<false><<<grid, 128, 0, st>>>(static_cast<const uint4*>(y), x, err);
  return 0;
}

// ---- source: sum of the partial sums, read from their owners ---------------------------------------------------
// out[t, :] = bf16( sum_d part_d[token row of t on d, :] ), destinations ascending, float32 accumulation (fp16 rows).
__global__ void __launch_bounds__(128) ep_final_combine_kernel(const uint32_t* __restrict__ slot, int T, EpExchange x,
                                                               uint4* __restrict__ out) {
  __shared__ const uint4* s_row[kEpMaxRanks];
  const int G = x.G, vec_per_row = (int)(x.H / 8);
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if ((int)threadIdx.x < G) {
      const int d = threadIdx.x;
      const uint32_t sl = slot[(size_t)d * T + t], tb = x.tokbase[d];
      const uint4* ptr = nullptr;
      if (sl != 0xffffffffu && tb != 0xffffffffu && tb + sl < x.cap_tok)
        ptr = static_cast<const uint4*>(x.peer[kEpPart][d]) + (size_t)(tb + sl) * vec_per_row;
      s_row[d] = ptr;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int d0 = 0; d0 < G; d0 += 4) {  // up to four peer loads in flight per thread
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = (d0 + u < G && s_row[d0 + u]) ? ld_cg_v4(s_row[d0 + u] + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
            acc[2 * q] += f.x;
            acc[2 * q + 1] += f.y;
          }
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

int launch_ep_final_combine(const uint32_t* slot, int64_t T, const EpExchange& x, void* out, cudaStream_t st) {
  if (T == 0) return 0;
  const int grid = (int)(T < 148 * 16 ? T : 148 * 16);
  ep_final_combine_kernel<<<grid, 128, 0, st>>>(slot, (int)T, x, static_cast<uint4*>(out));
  return 0;
}

}  // namespace b200

// Internal launch interface between the C-ABI layer (api.cu) and the kernel files.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

enum { kSrcIdent = 0, kSrcPermDiv = 1, kSrcMap = 2, kSrcMapDirect = 3 };
enum { kOutBf16 = 0, kOutF32 = 1, kOutF16 = 2, kOutNone = 3 };  // element format of a grouped product's output / of the combine's input (none: the product finished the block)

// One grouped product over rows that are sorted by expert.
constexpr int kExpertDescWords = 32;  // uint32 words of a per-expert record (launch_expert_descs)

struct GroupedArgs {
  const void* x;              // source rows [*, K]: bf16 for the tensor-core path's own preparation; PREPARED fp16 rows
                              // (launch_prepare_rows_small, or an out_f16 gate/up epilogue) for the register kernel
  const float* x_rowscale;    // register kernel: power of two each prepared source row was divided by (null: 1)
  const uint32_t* w[2];       // packed weights [E, N, K*bits/32]   ([1] = second matrix when NMAT == 2)
  const void* scales[2];      // bf16 [E, N, K/64]
  const void* biases[2];      // bf16 [E, N, K/64]
  const uint32_t* offsets;    // [E+1] first sorted position of each expert
  const uint32_t* active;     // experts that own at least one row
  const uint32_t* n_active;   // device scalar
  const uint32_t* perm;       // sorted position -> flat assignment index (may be null for identity modes)
  const uint32_t* src_map;    // flat assignment index -> source row (kSrcMap)
  int src_mode;               // kSrcIdent: row p; kSrcPermDiv: perm[p] / src_div; kSrcMap: src_map[perm[p]];
                              // kSrcMapDirect: src_map[p]
  int src_div;
  int dst_perm;               // 0: out row = sorted position, 1: out row = perm[p]
  const void* row_scale;      // bf16, indexed by out row; may be null
  void* out;                  // [rows, N], bf16 or float32
  const unsigned long long* out_row_addr;  // optional, by sorted position: address of the row's bf16 output
                                           // (overrides out/dst_perm; rows may live on peer GPUs)
  int out_f32;                // 1: float32 output (no rounding before the k-way combine)
  int out_f16;                // 1: fp16 output with saturation, out_f32 wins when both are set.  Two-matrix products write h
                              // in the A-operand layout of the same path's down projection (register kernel: prepared rows)
  int K, N;
  int n_experts;              // number of stacked weight matrices
  const uint32_t* desc;       // register kernel, optional: per active expert one 64-byte record (launch_expert_descs) that
                              // replaces the look-ups of n_active, active, offsets and the first eight source rows
  int late_trigger;           // register kernel: 1 = let the next kernel launch only after this one's own dependency wait,
                              // so that the next kernel may read the outputs of this one's predecessors before ITS wait
  int x_bf16;                 // register kernel: 1 = x holds plain bf16 rows and every CTA prepares the rows it stages
                              // itself (a handful of rows per expert: cheaper than a preparation launch)
};

// Down projection and weighted k-way sum of a handful of tokens in one launch (register kernel family).
struct DownCombineArgs {
  const void* h;              // prepared fp16 rows [T*k, K] in sorted order (a gate/up epilogue with out_f16)
  const uint32_t* idx;        // [T, k] expert of every assignment
  const uint32_t* inv;        // [T*k] sorted position of every assignment
  const void* scores;         // bf16 [T, k] routing weights
  const uint32_t* w;          // packed down weights [E, N, K*bits/32]
  const void* scales;         // bf16 [E, N, K/64]
  const void* biases;
  void* out;                  // bf16 [T, N]
  float* out_f32;             // optional [T, N]: the sum before its rounding
  int T, k, K, N;
  int early_routing;          // 1: idx, inv and scores are complete when this kernel's CTAs start (its predecessor was
                              // launched with late_trigger), so they and the first weight blocks are fetched before the wait
};
// desc [max_active][32] uint32: {expert, first sorted position, rows, 0, source row of the first eight sorted
// positions (by the given gather mode), the row scale of those eight source rows (float bits; 1.0 without
// row_scale), 0...}; entries past the number of active experts have rows = 0.
int launch_expert_descs(const uint32_t* active, const uint32_t* n_active, const uint32_t* offsets, const uint32_t* perm,
                        const uint32_t* src_map, int src_mode, int src_div, const float* row_scale, int max_active,
                        uint32_t* desc, cudaStream_t st);
// whether the register kernel's variant that keeps a CTA's weight slice in shared memory applies to a product over K
bool small_staged_ok(int K, int bits, int nmat);
bool down_combine_small_ok(int64_t T, int k, int K);
int launch_down_combine_small(const DownCombineArgs& a, int bits, cudaStream_t st);

// router.cu
// w64: optional scratch of E*H doubles (the float64 image of the router weight, rewritten by the call)
int launch_router_logits(const void* x, const void* w, const float* logit_bias, void* logits, int T, int H, int E,
                         double* w64, cudaStream_t st);
int launch_route_topk(const void* logits, int T, int E, int k, int mode, int renorm, uint32_t* idx, void* scores,
                      void* probs, cudaStream_t st);
// logits + top-k + token -> expert sort in one launch (T*k <= 1024); `ticket` is a zero-initialised device word
bool router_fused_small_ok(int T, int H, int E, int k);
int launch_router_fused_small(const void* x, const void* w, const float* logit_bias, void* logits, int T, int H, int E,
                              int k, int mode, int renorm, uint32_t* idx, void* scores, uint32_t* perm, uint32_t* inv,
                              uint32_t* counts, uint32_t* offsets, uint32_t* active, uint32_t* n_active,
                              unsigned int* ticket, int* err, uint32_t* desc, int desc_entries, cudaStream_t st);
// top-k + token -> expert sort in one launch (T*k <= 1024); `ticket` is a zero-initialised device word
bool route_topk_sort_ok(int T, int E, int k);
int launch_route_topk_sort(const void* logits, int T, int E, int k, int mode, int renorm, uint32_t* idx, void* scores,
                           uint32_t* perm, uint32_t* inv, uint32_t* counts, uint32_t* offsets, uint32_t* active,
                           uint32_t* n_active, unsigned int* ticket, int* err, cudaStream_t st);
int launch_argpartition(const void* a, int rows, int cols, int kth, uint32_t* out, cudaStream_t st);
int launch_topk_values(const void* a, int rows, int cols, int k, void* out, cudaStream_t st);
int launch_softmax(const void* a, int rows, int cols, void* out, cudaStream_t st);
int launch_take_along(const void* a, int rows, int cols, const uint32_t* idx, int icol, void* out, int* err,
                      cudaStream_t st);

// permute.cu
int launch_permute(const uint32_t* idx, int64_t n, int E, uint32_t* perm, uint32_t* inv, uint32_t* counts,
                   uint32_t* offsets, uint32_t* active, uint32_t* n_active, uint32_t* chunk_scratch, int* err,
                   cudaStream_t st);
size_t permute_scratch_words(int64_t n, int E);

// qmm_decode.cu (register kernel of the memory-bound regime)
bool small_shape_ok(int K);
// x [n_rows, K] bf16 (in_f16: fp16) -> prepared fp16 rows xs [n_rows, K] + row_scale [n_rows]
int launch_prepare_rows_small(const void* x, int in_f16, int64_t n_rows, const uint32_t* n_rows_dev, int K, int bits,
                              void* xs, float* row_scale, cudaStream_t st);
int launch_grouped_qmm_small(const GroupedArgs& a, int nmat, int bits, int max_active, int64_t rows, cudaStream_t st);

// qmm_prefill.cu (tcgen05 path)
size_t prefill_tile_words(int64_t rows, int E);
bool prefill_shape_ok(int K, int N, int nmat);
int launch_build_row_tiles(const uint32_t* counts, const uint32_t* offsets, int E, uint32_t* tile_expert,
                           uint32_t* tile_row0, uint32_t* tile_rows, uint32_t* n_row_tiles, int rows_per_tile,
                           cudaStream_t st);
// n_rows_dev (nullable): device word with the number of rows that exist (<= n_rows, the host's bound)
int launch_prepare_rows(const void* x, const uint32_t* perm, const uint32_t* src_map, int src_div, int64_t n_rows,
                        const uint32_t* n_rows_dev, int K, int permute8, void* xs, float* row_scale, cudaStream_t st);
int launch_grouped_qmm_tc(const void* a, const float* a_row_scale, int64_t rows, const GroupedArgs& g, int nmat, int bits, const uint32_t* tile_expert,
                          const uint32_t* tile_row0, const uint32_t* tile_rows, const uint32_t* n_row_tiles, int E,
                          bool alternate, int* err, cudaStream_t st);

// misc.cu
int launch_quantize(const void* w, int is_bf16, int64_t rows, int64_t K, int gs, int bits, uint32_t* wq, void* scales,
                    void* biases, cudaStream_t st);
int launch_dequantize(const uint32_t* wq, const void* scales, const void* biases, int is_bf16, int64_t rows, int64_t K,
                      int gs, int bits, void* out, cudaStream_t st);
int launch_combine(const void* yk, int yk_fmt, int64_t T, int k, int64_t H, void* out, void* out_f32, cudaStream_t st);
int launch_take_rows(const void* x, const uint32_t* indices, uint32_t div, int64_t n_rows, int64_t x_rows, int64_t cols,
                     void* out, int* err, cudaStream_t st);
int launch_gather_combine(const void* y, const uint32_t* inv, const void* scores, int64_t T, int k, int64_t H, void* out,
                          void* out_f32, cudaStream_t st);
int launch_rms_norm(const void* x, const void* residual, const void* weight, float eps, int64_t rows, int64_t cols,
                    void* out, void* sum_out, cudaStream_t st);
int launch_add(const void* a, const void* b, int64_t n, void* out, cudaStream_t st);
// dtype: 0 float32, 1 bfloat16, 2 float16 (activations, scales, biases and result alike)
int launch_gather_qmm_generic(const void* x, const uint32_t* wq, const void* scales, const void* biases, const uint32_t* lhs,
                              const uint32_t* rhs, int dtype, int64_t Bx, int64_t M, int64_t K, int64_t E, int64_t N,
                              int64_t n_idx, int transpose, int gs, int bits, void* out, int* err, cudaStream_t st);
int launch_gather_mm(const void* a, const void* b, const uint32_t* lhs, const uint32_t* rhs, int64_t Ba, int64_t Bb,
                     int64_t M, int64_t K, int64_t N, int64_t n_idx, void* out, int* err, cudaStream_t st);
int launch_gather_rows(const void* x, const uint32_t* perm, const uint32_t* src_map, int64_t n_rows, const uint32_t* n_valid,
                       int64_t cols, void* out, cudaStream_t st);
int launch_gather_mm_tc(const void* a_sorted, int64_t rows, const void* b, int Bb, int K, int N, const uint32_t* perm, void* out,
                        const uint32_t* tile_expert, const uint32_t* tile_row0, const uint32_t* tile_rows,
                        const uint32_t* n_row_tiles, int* err, cudaStream_t st);
int launch_dense_segments(uint32_t* counts, uint32_t* offsets, uint32_t* active, uint32_t* n_active, uint32_t rows,
                          cudaStream_t st);
int launch_expand_indices(const uint32_t* lhs, const uint32_t* rhs, int64_t n_idx, int M, int64_t Bx, uint32_t* flat_expert,
                          uint32_t* flat_src, int* err, cudaStream_t st);


// ep.cu (expert-parallel exchange over peer memory)
constexpr int kEpMaxRanks = 16;
struct EpPeers {
  void* p[kEpMaxRanks];       // the same exchange buffer on every rank, indexed by rank (own entry = local pointer)
};
int launch_segments_from_counts(const uint32_t* counts, int E, int64_t n_rows, uint32_t* counts_out, uint32_t* offsets,
                                uint32_t* active, uint32_t* n_active, int* err, cudaStream_t st);
int launch_ep_layout(const uint32_t* all_counts, int G, int E, int rank, uint32_t capacity, uint32_t* dst_row0,
                     uint32_t* local_counts, int* err, cudaStream_t st);
int launch_ep_dispatch(const void* x, const uint32_t* idx, const uint32_t* perm, const uint32_t* offsets,
                       const uint32_t* dst_row0, int64_t n, int k, int64_t H, int E, int G, int rank, const EpPeers& peers,
                       uint32_t capacity, int* err, cudaStream_t st);
int launch_ep_return_table(const uint32_t* all_counts, int G, int E, int rank, const EpPeers& peers_y, int64_t H, int64_t n_rows,
                           int64_t capacity_rows, unsigned long long* row_addr, int* err, cudaStream_t st);
int launch_ep_combine(const EpPeers& peers, const uint32_t* idx, const uint32_t* inv, const uint32_t* offsets,
                      const uint32_t* dst_row0, const void* scores, int64_t T, int k, int64_t H, int E, int G,
                      uint32_t capacity, void* out, int* err, cudaStream_t st);

// One-call expert-parallel block: device-side phase ordering through control blocks mapped between the ranks, and
// the de-duplicated exchange (one row per token and destination rank).  kEpBufs peer-mapped buffers per rank:
enum { kEpTok = 0, kEpPart = 1, kEpRowMap = 2, kEpSlotRows = 3, kEpSlotScores = 4, kEpCtl = 5, kEpBufs = 6 };
struct EpExchange {
  void* peer[kEpBufs][kEpMaxRanks];  // every rank's buffers (own entry = local pointer)
  int G, E, rank, k;
  int64_t H;
  uint32_t cap_rows;   // assignments a rank can receive per step
  uint32_t cap_tok;    // token rows a rank can receive per step
  // device words of this rank: dst_row0 [E], local_counts [E/G], n_recv, tokbase [G], n_tok_recv, ntok [G]
  uint32_t *dst_row0, *local_counts, *n_recv, *tokbase, *n_tok_recv, *ntok;
};
size_t ep_ctl_bytes(int G, int E);
// slot [G][T]: position of token t among this rank's tokens that have an expert on rank d (0xffffffff: none)
int launch_ep_token_slots(const uint32_t* idx, int64_t T, const EpExchange& x, uint32_t* slot, cudaStream_t st);
int launch_ep_counts_exchange(const EpExchange& x, const uint32_t* counts, int* err, cudaStream_t st);
int launch_ep_signal_wait(const EpExchange& x, int which, int* err, cudaStream_t st);
int launch_ep_dispatch_dedup(const void* xrows, const uint32_t* idx, const uint32_t* inv, const uint32_t* offsets,
                             const void* scores, const uint32_t* slot, int64_t T, const EpExchange& x, int* err, cudaStream_t st);
int launch_ep_partial_combine(const void* y, bool y_f16, const EpExchange& x, int* err, cudaStream_t st);
int launch_ep_final_combine(const uint32_t* slot, int64_t T, const EpExchange& x, void* out, cudaStream_t st);
int launch_add_u32(const uint32_t* a, const uint32_t* b, int n, uint32_t* out, cudaStream_t st);

}  // namespace b200

/*
 * b200_moe.h - C ABI of the B200-native quantized mixture-of-experts path.
 *
 * A drop-in for the part of oxiglade/mlx-rs that an MLX-affine-quantized MoE block runs
 * through: one function per op wrapper of the reference (same names, argument order and
 * defaults), plus fused entry points for the routed block.  It sits beside mlx-sys: where the
 * reference binds `int mlx_<op>(mlx_array* res, ..., mlx_stream s)` (status int, result
 * handle first; mlx-rs/src/utils/guard.rs:20-49), this library exports
 * `int b200_<op>(b200_ctx*, <device pointers and sizes>, void* cuda_stream)`.
 *
 * Conventions
 *  - return 0 on success, non-zero on failure; the message is available from
 *    b200_last_error() (thread-local) and is also passed to the handler registered with
 *    b200_set_error_handler(), whose signature equals the one mlx_set_error_handler() takes
 *    (mlx-rs/src/error.rs:232-251).  Bad arguments never abort and never launch anything.
 *  - every pointer is a DEVICE pointer unless stated otherwise; inputs are const, outputs are
 *    caller-allocated.  bf16 tensors are `void*`.  Indices are uint32 like the reference's.
 *  - calls are eager and stream-ordered: work is enqueued on `stream` (a cudaStream_t passed
 *    as void*) and the call returns; "eval" is cudaStreamSynchronize.
 *  - a b200_ctx owns scratch memory (it grows on demand; b200_ctx_reserve pre-sizes it) and is
 *    used by one thread at a time on one device, like the reference's per-thread streams.
 *  - quantized layout = MLX affine: `32/bits` codes per uint32, element i in bits
 *    [bits*i, bits*i+bits), one bf16 scale and bias per `group_size` elements of the last axis,
 *    w_hat = scale*q + bias.  Matmul kernels require group_size 64 and bits 4 or 8.
 */
#ifndef B200_MOE_H_
#define B200_MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_DEFAULT_GROUP_SIZE 64 /* mlx-rs/src/ops/quantization.rs:12 */
#define B200_DEFAULT_BITS 4        /* mlx-rs/src/ops/quantization.rs:13 */

typedef struct b200_ctx b200_ctx;

enum { B200_F32 = 0, B200_BF16 = 1, B200_F16 = 2 };
enum { B200_ROUTER_SOFTMAX_TOPK = 0, B200_ROUTER_TOPK_SOFTMAX = 1 };

/* Stacked quantized projection of all experts: weight [E, out, in*bits/32] uint32,
 * scales/biases [E, out, in/group_size] bf16 (field names as in QuantizedLinear,
 * mlx-rs/src/nn/quantized.rs:307-328). */
typedef struct {
  const uint32_t* weight;
  const void* scales;
  const void* biases;
} b200_qlinear;

typedef struct {
  int32_t hidden;         /* H */
  int32_t inter;          /* I, moe_intermediate_size */
  int32_t n_experts;      /* E (<= 256) */
  int32_t top_k;          /* k (<= 32) */
  int32_t bits;           /* 4 or 8 */
  int32_t group_size;     /* 64 */
  int32_t router_mode;    /* B200_ROUTER_* */
  int32_t norm_topk_prob; /* renormalise the selected probabilities (mode 0) */
} b200_moe_config;

typedef struct {
  const void* router_weight;      /* bf16 [E, H]  (Linear layout [out,in], mlx-rs/src/nn/linear.rs:39) */
  const float* router_logit_bias; /* optional float32 [E] added to the logits; NULL for none */
  b200_qlinear gate_proj;         /* [E, I, H] */
  b200_qlinear up_proj;           /* [E, I, H] */
  b200_qlinear down_proj;         /* [E, H, I] */
} b200_moe_params;

/* Optional routing outputs of the block; any pointer may be NULL. */
typedef struct {
  uint32_t* indices;  /* [T, k]   selected experts, (value desc, expert asc) order */
  void* scores;       /* [T, k]   bf16 routing weights */
  uint32_t* perm;     /* [T*k]    stable argsort of the flat index list */
  uint32_t* inv_perm; /* [T*k]    inverse of perm */
  uint32_t* counts;   /* [E]      assignments per expert */
  uint32_t* offsets;  /* [E+1]    exclusive prefix sum of counts */
  void* logits;       /* [T, E]   bf16 router logits */
  float* out_f32;     /* [T, H]   the block output before its final rounding to bf16 (out == bf16(out_f32)) */
} b200_moe_aux;

/* ---- library / context ----------------------------------------------------------------- */

/* Message of the last failing call on this thread (valid until the next failing call). */
const char* b200_last_error(void);
/* Same contract as mlx_set_error_handler (mlx-rs/src/error.rs:232-251). */
void b200_set_error_handler(void (*handler)(const char* msg, void* data), void* data, void (*dtor)(void*));
/* Creates a context on CUDA device `device` (cudaSetDevice is called).
 *
 * A context owns ONE scratch arena, and every call that takes a context starts handing it out from the
 * beginning again.  Hence: one thread at a time, and one stream at a time - two calls on the same context
 * whose kernels can overlap on the GPU (different streams without an event between them) race on the arena
 * (tile tables, intermediate rows, the status words).  Use one context per concurrently used stream.
 * Calls that take no scratch and may go to any stream: b200_moe_combine, b200_take_rows, b200_add,
 * b200_rms_norm, b200_add_rms_norm, b200_softmax_axis, b200_argpartition_axis, b200_take_along_axis, b200_take_axis,
 * b200_topk_axis, b200_quantize, b200_ep_layout, b200_ep_dispatch, b200_ep_combine, b200_ep_return_table and the b200_ep_buffer_* calls.
 *
 * The arena grows on demand (free + cudaMalloc after cudaDeviceSynchronize).  Growth invalidates the addresses
 * that CUDA graphs captured earlier hold and is refused (status 1, nothing launched) while the call's stream is
 * being captured: size the arena with b200_ctx_reserve before capturing or replaying graphs. */
int b200_ctx_create(b200_ctx** out, int device);
int b200_ctx_destroy(b200_ctx* ctx);
/* Pre-sizes the scratch memory for blocks of up to `max_tokens` tokens so that later calls
 * do not allocate (allocation synchronises the device). */
int b200_ctx_reserve(b200_ctx* ctx, const b200_moe_config* cfg, int64_t max_tokens);
/* Scratch bytes one b200_moe_block_forward over max_tokens tokens needs (what b200_ctx_reserve allocates). */
int b200_workspace_bytes(const b200_moe_config* cfg, int64_t max_tokens, size_t* bytes);
/* Synchronises `stream` and reports device-side findings (an expert or gather index out of
 * range) of the calls issued since the last check; they surface here because argument values
 * living on the device cannot be validated before launch. */
int b200_ctx_check(b200_ctx* ctx, void* stream);
/* Number of kernels launched through this context so far. */
int64_t b200_ctx_launch_count(const b200_ctx* ctx);
/* Which grouped-product kernel the routed block uses.  AUTO: the register-load mma.sync kernel
 * while experts own few rows, the tcgen05 tensor-core kernel beyond that (when inter % 128 == 0
 * and hidden % 256 == 0).  A pinned kernel falls back when the shape does not allow it. */
enum { B200_QMM_AUTO = 0, B200_QMM_SMALL = 1, B200_QMM_TENSOR_CORE = 2 };
int b200_ctx_set_qmm_path(b200_ctx* ctx, int path);
/* Diagnostic: synchronises the device and copies the first n (<= 64) 32-bit words of the
 * context's status buffer to HOST memory.  Word 0 is the status b200_ctx_check reports; words
 * 16.. hold the tensor-core kernel's self-timing (kilo-cycles per role and wait) when the
 * environment variable B200_TC_DEBUG has bit 5 set. */
int b200_ctx_debug_words(b200_ctx* ctx, int32_t* host_out, int n);
/* Per-stage CUDA-event times of the last b200_moe_block_forward (profiling on): router logits, top-k,
 * sort (+ tile lists), activation preparation for gate/up, gate/up product, activation preparation
 * for down, down product, combine. */
#define B200_N_STAGES 8
int b200_ctx_set_profiling(b200_ctx* ctx, int enable);
int b200_ctx_stage_ms(b200_ctx* ctx, float* ms, int n);

/* ---- op surface of the reference -------------------------------------------------------- */

/* quantize(w, group_size, bits) -> (w_q, scales, biases); mlx-rs/src/ops/quantization.rs:48-83.
 * w [rows, K] of `dtype` (B200_F32 or B200_BF16); scales/biases come back in the same dtype.
 * group_size in {32, 64, 128}, bits in {2, 4, 8}. */
int b200_quantize(b200_ctx* ctx, const void* w, int dtype, int64_t rows, int64_t K, int group_size, int bits,
                  uint32_t* w_q, void* scales, void* biases, void* stream);

/* dequantize(w, scales, biases, group_size, bits); mlx-rs/src/ops/quantization.rs:129-158.
 * Output [rows, K] in the dtype of the scales. */
int b200_dequantize(b200_ctx* ctx, const uint32_t* w_q, const void* scales, const void* biases, int dtype, int64_t rows,
                    int64_t K, int group_size, int bits, void* out, void* stream);

/* quantized_matmul(x, w, scales, biases, transpose, group_size, bits);
 * mlx-rs/src/ops/quantization.rs:88-122.  x [M, K]; transpose != 0: w [N, K*bits/32] and out = x . w_hat^T (the
 * form every layer uses, mlx-rs/src/nn/quantized.rs:363-381); transpose == 0: w [K, N*bits/32] and out = x . w_hat.
 * out [M, N].  `dtype` (B200_F32 / B200_BF16 / B200_F16) is the type of x, scales, biases and out alike (MLX keeps
 * the scales in the type of the weights they came from).  bfloat16 with transpose != 0, group_size 64 and 4 or 8
 * bits runs on the tensor cores; every other combination (float32 - the reference's own tests, `:319-342` -
 * float16, transpose == 0, group sizes 32 / 128, 2 bits) takes an exact float32 CUDA-core kernel. */
int b200_quantized_matmul(b200_ctx* ctx, const void* x, const uint32_t* w, const void* scales, const void* biases,
                          int transpose, int group_size, int bits, int dtype, int64_t M, int64_t K, int64_t N, void* out,
                          void* stream);

/* gather_mm(a, b, lhs_indices, rhs_indices); mlx-rs/src/ops/arithmetic.rs:1568-1632 (un-quantised).
 * out[i] = a[lhs[i]] @ b[rhs[i]] with a bf16 [Ba, M, K], b bf16 [Bb, K, N], out bf16 [n_idx, M, N], float32
 * accumulation.  Either index array may be NULL (identity).  n_idx < 65536 per call. */
int b200_gather_mm(b200_ctx* ctx, const void* a, const void* b, const uint32_t* lhs_indices, const uint32_t* rhs_indices,
                   int64_t Ba, int64_t Bb, int64_t M, int64_t K, int64_t N, int64_t n_idx, void* out, void* stream);

/* gather_qmm(x, w, scales, biases, lhs_indices, rhs_indices, transpose, group_size, bits,
 * sorted_indices); mlx-rs/src/ops/quantization.rs:160-230.
 * out[i] = x[lhs[i]] . dequantize(w[rhs[i]])^T (transpose != 0; w [E, N, K*bits/32]) or x[lhs[i]] . dequantize(w[rhs[i]])
 * (transpose == 0; w [E, K, N*bits/32]) with x [Bx, M, K], out [n_idx, M, N].  lhs_indices may be NULL (lhs[i] = i).
 * `dtype` and the fast / exact split as for b200_quantized_matmul (the fast form also needs E <= 256): few rows
 * per matrix run the register kernel, many the tcgen05 kernel.  `sorted_indices` is accepted for signature parity;
 * rows are always grouped internally.  Index values out of range are reported by b200_ctx_check. */
int b200_gather_qmm(b200_ctx* ctx, const void* x, const uint32_t* w, const void* scales, const void* biases,
                    const uint32_t* lhs_indices, const uint32_t* rhs_indices, int transpose, int group_size, int bits,
                    int sorted_indices, int dtype, int64_t Bx, int64_t M, int64_t K, int64_t E, int64_t N, int64_t n_idx,
                    void* out, void* stream);

/* softmax_axis(a, -1, precise); mlx-rs/src/ops/arithmetic.rs:1312-1327.  bf16 [rows, cols],
 * cols <= 256.  Always the precise form: exact softmax, correctly rounded to bf16. */
int b200_softmax_axis(b200_ctx* ctx, const void* a, int64_t rows, int64_t cols, int precise, void* out, void* stream);

/* argpartition_axis(a, kth, -1); mlx-rs/src/ops/sort.rs:186-226.  bf16 [rows, cols], cols <= 256.
 * Columns 0..kth hold the kth+1 smallest elements in (value asc, index asc) order, the rest
 * hold the remaining indices in ascending order. */
int b200_argpartition_axis(b200_ctx* ctx, const void* a, int64_t rows, int64_t cols, int kth, uint32_t* out, void* stream);

/* take_along_axis(a, indices, -1); mlx-rs/src/ops/indexing/mod.rs:424-453.  2-byte elements:
 * a [rows, cols], indices [rows, icols] -> out [rows, icols]. */
int b200_take_along_axis(b200_ctx* ctx, const void* a, int64_t rows, int64_t cols, const uint32_t* indices, int64_t icols,
                         void* out, void* stream);

/* take_axis(x, indices / div, 0) for rows of bf16: out[p, :] = x[indices[p] / div, :]
 * (take_axis, mlx-rs/src/ops/indexing/mod.rs:374-401, composed with floor_divide,
 * mlx-rs/src/ops/arithmetic.rs:401 - the "x[order // k]" step of the token sort).
 * x [x_rows, cols], indices [n_rows], cols a multiple of 8. */
int b200_take_rows(b200_ctx* ctx, const void* x, const uint32_t* indices, uint32_t div, int64_t n_rows, int64_t x_rows,
                   int64_t cols, void* out, void* stream);
/* take_axis(x, indices, 0); mlx-rs/src/ops/indexing/mod.rs:374-401, 641-660: b200_take_rows without the division. */
int b200_take_axis(b200_ctx* ctx, const void* x, const uint32_t* indices, int64_t n_rows, int64_t x_rows, int64_t cols,
                   void* out, void* stream);

/* argsort_axis(a, -1) for rows of small unsigned keys (expert indices); mlx-rs/src/ops/sort.rs:57-83.
 * keys uint32 [rows, cols], every key < key_bound <= 256 -> out uint32 [rows, cols], the STABLE ascending order of
 * each row (the order the token -> expert sort uses).  Keys >= key_bound are reported by b200_ctx_check. */
int b200_argsort_axis(b200_ctx* ctx, const uint32_t* keys, int64_t rows, int64_t cols, int key_bound, uint32_t* out,
                      void* stream);

/* topk_axis(a, k, -1); mlx-rs/src/ops/indexing/mod.rs:674-700.  bf16 [rows, cols], cols <= 256 -> out bf16 [rows, k]:
 * the k largest values of each row, ascending (MLX leaves their order unspecified). */
int b200_topk_axis(b200_ctx* ctx, const void* a, int64_t rows, int64_t cols, int k, void* out, void* stream);

/* fast::rms_norm(x, weight, eps); mlx-rs/src/fast.rs:178-205.  bf16 [rows, cols]; weight
 * bf16 [cols] or NULL for ones. */
int b200_rms_norm(b200_ctx* ctx, const void* x, const void* weight, float eps, int64_t rows, int64_t cols, void* out,
                  void* stream);
/* Residual add fused with the norm (the wiring of mlx-lm/src/models/qwen3.rs:310-325):
 * sum_out = bf16(x + residual), out = rms_norm(sum_out, weight, eps). */
int b200_add_rms_norm(b200_ctx* ctx, const void* x, const void* residual, const void* weight, float eps, int64_t rows,
                      int64_t cols, void* sum_out, void* out, void* stream);
/* out = bf16(a + b), n elements. */
int b200_add(b200_ctx* ctx, const void* a, const void* b, int64_t n, void* out, void* stream);

/* ---- fused entry points of the routed block ---------------------------------------------- */

/* Router: gate Linear (mlx-rs/src/nn/linear.rs:83-95) + softmax_axis + argpartition_axis +
 * take_along_axis + sum_axis/divide in the order the router mode prescribes.
 * x bf16 [T, H] -> indices [T, k], scores bf16 [T, k]; logits (bf16 [T, E]) may be NULL. */
int b200_router_topk(b200_ctx* ctx, const b200_moe_config* cfg, const void* x, const void* router_weight,
                     const float* logit_bias, int64_t T, uint32_t* indices, void* scores, void* logits, void* stream);

/* Token -> expert sort: argsort_axis (mlx-rs/src/ops/sort.rs:57-83) of the flat index list,
 * its inverse, histogram and prefix sum.  indices [n]; perm, inv_perm [n]; counts [E];
 * offsets [E+1].  Bit-exact with a stable argsort. */
int b200_moe_permute(b200_ctx* ctx, const uint32_t* indices, int64_t n, int n_experts, uint32_t* perm, uint32_t* inv_perm,
                     uint32_t* counts, uint32_t* offsets, void* stream);

/* Allocation-free variant of b200_moe_permute.  It has no counterpart in the reference (whose
 * arrays are always allocated by MLX); it exists for callers of THIS library that must not
 * trigger a device allocation: a server that gave all device memory to its own pool at start-up,
 * or a token loop that cannot afford the device-wide synchronisation cudaMalloc/cudaFree imply.
 * Same arguments and results as b200_moe_permute, but no context: the scratch memory is a fixed
 * 258 KB __device__ array inside the library (held by every GPU that loads it, until exit).
 * Limit: ceil(n/1024) * n_experts <= 65536 (e.g. n <= 524288 at 128 experts); larger problems
 * are rejected with an error.  The call performs no cudaMalloc/cudaFree and uses no allocating
 * library routine.  Its first call on a device resolves the array's device address
 * (cudaGetSymbolAddress) and should therefore happen before any stream capture begins.  All
 * calls share the one array and it keeps the previous call's contents (nothing in it has to start
 * at zero: every word is rewritten by the call before it is read): calls whose kernels overlap on
 * the GPU - two streams, two threads - race on it, so serialise them.  Expert indices >= n_experts
 * are skipped, not reported: counts then sums to less than n and the skipped positions of perm /
 * inv_perm keep what the caller's buffers held (compare offsets[n_experts] with n to detect it). */
int b200_moe_permute_static(const uint32_t* indices, int64_t n, int n_experts, uint32_t* perm, uint32_t* inv_perm,
                            uint32_t* counts, uint32_t* offsets, void* stream);

/* Weighted un-sort and combine of expert outputs held in sorted order (the return path of the
 * expert-parallel exchange): out[t, :] = bf16( sum_j scores[t, j] * y_sorted[inv_perm[t*k + j], :] )
 * in float32, j ascending (take with the inverse order + multiply + sum_axis(-2),
 * mlx-rs/src/ops/reduction.rs:260-275).  y_sorted bf16 [T*k, hidden]; out_f32 (optional) receives
 * the sum before rounding. */
int b200_moe_combine(b200_ctx* ctx, const void* y_sorted, const uint32_t* inv_perm, const void* scores, int64_t T,
                     int top_k, int64_t hidden, void* out, float* out_f32, void* stream);

/* SwitchGLU forward: (x bf16 [T, H], indices [T, k]) -> out bf16 [T, k, H],
 * out[t, j] = down_e( silu(gate_e(x_t)) * up_e(x_t) ), e = indices[t, j]. */
int b200_switch_glu_forward(b200_ctx* ctx, const b200_moe_config* cfg, const b200_moe_params* params, const void* x,
                            const uint32_t* indices, int64_t T, void* out, void* stream);

/* SwitchGLU over rows that are already grouped by expert: rows bf16 [n, H] with counts[e] consecutive
 * rows for expert e (device array, sum == n); out bf16 [n, H] in the same order.  The sorted-input
 * case of gather_qmm (mlx-rs/src/ops/quantization.rs:160-230 with sorted_indices = true; module template
 * mlx-lm/src/models/qwen3.rs:204-255) without the sort; used on the rows a rank receives in the
 * expert-parallel exchange. */
int b200_switch_glu_sorted(b200_ctx* ctx, const b200_moe_config* cfg, const b200_moe_params* params, const void* rows,
                           const uint32_t* counts, int64_t n, void* out, void* stream);

/* ---- expert parallelism over peer memory --------------------------------------------------------
 * None of the b200_ep_* entry points has a counterpart in the reference, which has no distributed
 * layer.  One process per GPU; rank r owns experts [r*E/G, (r+1)*E/G).  Every rank allocates two
 * exchange buffers of capacity_rows x hidden bf16 (arriving rows, expert outputs) with
 * b200_ep_buffer_alloc, passes the 64-byte handles to its peers by any host channel, and maps
 * theirs with b200_ep_buffer_open.  Row numbering on the owning rank: by local expert, then by
 * source rank, then in the source's sorted order.  No kernel here waits on another GPU: the
 * caller orders the phases with stream-ordered collectives that every rank joins
 * (all-gather of the counts -> layout -> dispatch -> barrier -> b200_switch_glu_sorted ->
 * barrier -> combine; the next step's all-gather keeps buffers from being overwritten early). */
#define B200_EP_HANDLE_BYTES 64
int b200_ep_buffer_alloc(b200_ctx* ctx, size_t bytes, void** ptr, unsigned char* handle);
int b200_ep_buffer_open(b200_ctx* ctx, const unsigned char* handle, void** ptr);
int b200_ep_buffer_close(b200_ctx* ctx, void* ptr);
int b200_ep_buffer_free(b200_ctx* ctx, void* ptr);
/* Return path fused into the down projection.  b200_ep_return_table fills row_addr[i], for every
 * row i this rank received, with the address of that row's output in the SOURCE rank's return buffer
 * (peer_y[s], bf16 [T_s * top_k, hidden] in the source's own sorted order); b200_switch_glu_sorted_scatter
 * is b200_switch_glu_sorted whose epilogue stores each finished row to row_addr[i] (peer stores), so
 * the transfer back overlaps the products tile by tile and the source finishes with a local
 * b200_moe_combine after one barrier.  n_rows = entries of row_addr (rows this rank received), capacity_rows = rows
 * of every source's return buffer: an entry past either bound is not written (the table) or written as address 0,
 * which the epilogue skips (the buffer), and b200_ctx_check reports it.  The grouped products likewise follow
 * `counts` only up to `n` rows in total and report counts that promise more. */
int b200_ep_return_table(b200_ctx* ctx, const uint32_t* all_counts, int n_ranks, int n_experts, int rank,
                         void* const* peer_y, int64_t hidden, int64_t n_rows, int64_t capacity_rows,
                         unsigned long long* row_addr, void* stream);
int b200_switch_glu_sorted_scatter(b200_ctx* ctx, const b200_moe_config* cfg, const b200_moe_params* params,
                                   const void* rows, const uint32_t* counts, int64_t n,
                                   const unsigned long long* out_row_addr, void* stream);
/* all_counts [n_ranks, n_experts] (rows rank s routes to expert e, on the device) ->
 * dst_row0 [n_experts]: row on the owner of e where this rank's rows of e start;
 * local_counts [n_experts / n_ranks]: rows arriving here per local expert. */
int b200_ep_layout(b200_ctx* ctx, const uint32_t* all_counts, int n_ranks, int n_experts, int rank, uint32_t capacity_rows,
                   uint32_t* dst_row0, uint32_t* local_counts, void* stream);
/* Gather into expert order fused with the send: sorted position j (assignment perm[j], token
 * perm[j] / top_k, expert indices[perm[j]]) is stored into the owner's rows buffer
 * peer_rows[owner] (host array of n_ranks device pointers, own entry local).  Rows are sent destination by
 * destination starting after `rank` and wrapping around, so that the ranks do not all write to the same
 * GPU at the same time. */
int b200_ep_dispatch(b200_ctx* ctx, const void* x, const uint32_t* indices, const uint32_t* perm, const uint32_t* offsets,
                     const uint32_t* dst_row0, int64_t n, int top_k, int64_t hidden, int n_experts, int n_ranks, int rank,
                     void* const* peer_rows, uint32_t capacity_rows, void* stream);
/* Return fused with the weighted combine: out[t, :] = bf16( sum_j scores[t, j] * y_owner[row(t, j), :] ),
 * float32 accumulation, j ascending, read from the owners' output buffers peer_y. */
int b200_ep_combine(b200_ctx* ctx, void* const* peer_y, const uint32_t* indices, const uint32_t* inv_perm,
                    const uint32_t* offsets, const uint32_t* dst_row0, const void* scores, int64_t T, int top_k,
                    int64_t hidden, int n_experts, int n_ranks, uint32_t capacity_rows, void* out, void* stream);

/* ---- expert-parallel block in one call ------------------------------------------------------------
 * b200_moe_block_forward_ep is b200_moe_block_forward for a rank of an expert-parallel group: the slot a
 * transformer block's MLP fills (mlx-lm/src/models/qwen3.rs:310-325), with the experts sharded over the GPUs of
 * one node.  The whole step - route, sort, exchange of the counts, dispatch, this rank's experts, combine - is
 * enqueued on `stream` by ONE call, with no host synchronisation and no collective library: the ranks order
 * their phases through small control blocks in each other's memory (release stores, acquire spins with a 2 s
 * bound; expiry and buffer overflow are reported by b200_ctx_check).  Requirements: one process (or thread) per
 * GPU, every rank makes the call for every step (a rank without tokens passes T = 0), params->router_weight is
 * the full [E, H] router while gate/up/down hold THIS rank's experts [E / n_ranks, ...] (rank r owns the
 * contiguous experts [r*E/n_ranks, (r+1)*E/n_ranks)).
 *
 * The exchange is de-duplicated: a token travels once to every rank that owns at least one of its experts (not
 * once per assignment), the owner gathers its assignments' rows from those token rows, sums the token's expert
 * outputs with their routing weights locally, and one partial sum per (token, rank) travels back.
 *
 * Set-up (collective, host side): every rank calls b200_ep_comm_create, which allocates its exchange buffers
 * (token rows and partial sums: capacity_tokens x hidden bf16 each; bookkeeping; a control block) and returns
 * B200_EP_COMM_HANDLES 64-byte handles; the ranks exchange the handles by any host channel and each calls
 * b200_ep_comm_connect with all of them, rank-major ([n_ranks][B200_EP_COMM_HANDLES][64] bytes); a host barrier
 * after connect and before destroy keeps a fast rank from touching memory that is not mapped yet / any more.
 * capacity_rows bounds the ASSIGNMENTS (token, expert) a rank can receive in one step, capacity_tokens the token
 * rows (at most the tokens of all ranks together); a rank that would receive more takes nothing that step (its
 * experts' contributions are dropped, status 5). */
#define B200_EP_COMM_HANDLES 6
typedef struct b200_ep_comm b200_ep_comm;
int b200_ep_comm_create(b200_ctx* ctx, int n_ranks, int rank, int n_experts, int top_k, int64_t hidden,
                        uint32_t capacity_rows, uint32_t capacity_tokens, b200_ep_comm** out,
                        unsigned char* handles /* [B200_EP_COMM_HANDLES][B200_EP_HANDLE_BYTES] */);
int b200_ep_comm_connect(b200_ctx* ctx, b200_ep_comm* comm, const unsigned char* all_handles);
int b200_ep_comm_destroy(b200_ctx* ctx, b200_ep_comm* comm);
/* Half-steps per step, 1 (default) or 2; EVERY rank of the group must set the same value before the next step.
 * With 2 a step runs as two complete exchanges over consecutive halves of each rank's tokens, on separate buffers and
 * control words (a communicator always holds both sets): the exchange kernels go to a stream the communicator owns
 * and are joined back into the caller's stream before the call's work ends there, so that the dispatch of the second
 * half and the return of the first run under the other half's expert products.  Measured at 8192 tokens per rank on 2
 * and 4 GPUs it is slower than one step (the second set of small launches costs more than the overlap returns), so
 * it is left to the caller; aux->perm / inv_perm / offsets (which describe one sort of the whole step) cannot be
 * asked for then. */
int b200_ep_comm_set_chunks(b200_ctx* ctx, b200_ep_comm* comm, int chunks);
/* aux->out_f32 is not produced here (the returned expert outputs are bf16); the other aux fields are. */
int b200_moe_block_forward_ep(b200_ctx* ctx, b200_ep_comm* comm, const b200_moe_config* cfg, const b200_moe_params* params,
                              const void* x, int64_t T, void* out, const b200_moe_aux* aux, void* stream);

/* MoE block forward: x bf16 [T, H] -> out bf16 [T, H]; aux may be NULL. */
int b200_moe_block_forward(b200_ctx* ctx, const b200_moe_config* cfg, const b200_moe_params* params, const void* x,
                           int64_t T, void* out, const b200_moe_aux* aux, void* stream);
/* The block with the pre-norm of a transformer layer's MLP half in front of it (mlx-lm/src/models/qwen3.rs:310-325,
 * fast::rms_norm mlx-rs/src/fast.rs:178-205):  s = bf16(x + residual)  (residual NULL: s = x),
 * out = block(rms_norm(s, norm_weight, eps)).  sum_out (optional, only with a residual) receives s, the new residual
 * stream.  Same results, bit for bit, as b200_add_rms_norm followed by b200_moe_block_forward, in one call. */
int b200_moe_block_forward_prenorm(b200_ctx* ctx, const b200_moe_config* cfg, const b200_moe_params* params, const void* x,
                                   const void* residual, const void* norm_weight, float eps, int64_t T, void* sum_out,
                                   void* out, const b200_moe_aux* aux, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_MOE_H_ */

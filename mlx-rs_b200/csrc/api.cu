// C ABI of the library (see include/b200_moe.h): argument validation, scratch management and
// the composition of kernels behind every entry point.  No kernel lives here.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200_moe.h"
#include "common.cuh"
#include "kernels.h"

namespace b200 {

#ifdef B200_DEV
bool pdl_enabled() {
  static const bool on = getenv("B200_NO_PDL") == nullptr;
  return on;
}
#endif

// ---- error slot: thread-local message + optional process-wide handler ----------------------
static thread_local std::string g_last_error;
static std::mutex g_handler_mu;
static void (*g_handler)(const char*, void*) = nullptr;
static void* g_handler_data = nullptr;
static void (*g_handler_dtor)(void*) = nullptr;

void set_error(const std::string& msg) {
  g_last_error = msg;
  std::lock_guard<std::mutex> lk(g_handler_mu);
  if (g_handler) g_handler(g_last_error.c_str(), g_handler_data);
}

}  // namespace b200

using namespace b200;

// ---- context ----------------------------------------------------------------------------------
struct b200_ctx {
  int device = 0;
  unsigned char* ws = nullptr;  // scratch arena
  size_t ws_bytes = 0;
  size_t ws_used = 0;           // bump pointer of the call in progress
  int* err = nullptr;           // device status word
  int64_t launches = 0;
  int qmm_path = B200_QMM_AUTO;
  bool profiling = false;       // record an event after every stage of the block forward
  cudaEvent_t ev[B200_N_STAGES + 1] = {};
  bool ev_valid = false;

  void begin() { ws_used = 0; }
  void mark(int i, cudaStream_t st) {
    if (profiling) cudaEventRecord(ev[i], st);
  }
  // Bump-allocates from the arena; returns null when it does not fit (caller grows first).
  void* take(size_t bytes) {
    size_t off = (ws_used + 255) & ~size_t(255);
    if (off + bytes > ws_bytes) return nullptr;
    ws_used = off + bytes;
    return ws + off;
  }
};

// Growing frees and reallocates the arena after a device-wide synchronisation.  Neither is legal while `stream` is
// being captured into a graph (and graphs captured earlier hold addresses inside the old arena), so a capture in
// progress makes the call fail instead: reserve the arena (b200_ctx_reserve) before capturing.
static int ctx_grow(b200_ctx* c, size_t bytes, void* stream = nullptr) {
  if (bytes <= c->ws_bytes) return 0;
  if (stream) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    B200_CUDA(cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &cap));
    B200_REQUIRE(cap == cudaStreamCaptureStatusNone,
                 "the scratch arena would have to grow during stream capture: call b200_ctx_reserve before capturing");
  }
  B200_CUDA(cudaDeviceSynchronize());
  if (c->ws) B200_CUDA(cudaFree(c->ws));
  c->ws = nullptr;
  c->ws_bytes = 0;
  size_t want = bytes + bytes / 8 + (1 << 20);
  B200_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->ws), want));
  c->ws_bytes = want;
  return 0;
}

static inline size_t al(size_t b) { return (b + 255) & ~size_t(255); }

// scratch needed by one block forward over T tokens
static size_t block_scratch_bytes(const b200_moe_config& cfg, int64_t T) {
  const int64_t n = T * cfg.top_k, E = cfg.n_experts;
  size_t b = 0;
  b += al(sizeof(uint16_t) * T * E);                 // logits
  b += al(sizeof(double) * E * cfg.hidden);          // float64 image of the router weight
  b += al(sizeof(uint32_t) * n) * 3;                 // idx, perm, inv
  b += al(sizeof(uint16_t) * n);                     // scores
  b += al(sizeof(uint32_t) * (E + 1)) * 4 + al(16);  // counts (twice: the caller's and the bounded copy), offsets, active, n_active
  b += al(sizeof(uint32_t) * permute_scratch_words(n, (int)E));
  b += al(sizeof(uint16_t) * n * cfg.inter);         // h (bf16, or fp16 on the tensor-core path)
  b += al(sizeof(float) * n * cfg.hidden);           // per-assignment outputs (float32, or fp16 on the tensor-core path)
  b += al(sizeof(uint16_t) * n * cfg.hidden);        // rows gathered into expert order, fp16 (tensor-core path)
  b += al(sizeof(float) * n);                        // their row scales
  b += (al(sizeof(uint32_t) * prefill_tile_words(n, (int)E)) * 3 + al(16)) * 2;
  b += al(sizeof(uint32_t) * kExpertDescWords * (size_t)(E < n ? E : n));  // per-expert records of the register kernels
  b += al(sizeof(uint16_t) * T * cfg.hidden);        // normalised rows of the pre-norm entry point
  return b + 4096;
}

static int check_cfg(const b200_moe_config* cfg) {
  B200_REQUIRE(cfg != nullptr, "config is null");
  B200_REQUIRE(cfg->bits == 4 || cfg->bits == 8, "bits must be 4 or 8");
  B200_REQUIRE(cfg->group_size == 64, "group_size must be 64");
  B200_REQUIRE(cfg->hidden > 0 && cfg->hidden % 64 == 0, "hidden must be a positive multiple of 64");
  B200_REQUIRE(cfg->inter > 0 && cfg->inter % 64 == 0, "inter must be a positive multiple of 64");
  B200_REQUIRE(cfg->n_experts > 0 && cfg->n_experts <= 256, "n_experts must be in 1..256");
  B200_REQUIRE(cfg->top_k > 0 && cfg->top_k <= 32 && cfg->top_k <= cfg->n_experts, "top_k must be in 1..min(32, n_experts)");
  B200_REQUIRE(cfg->router_mode == B200_ROUTER_SOFTMAX_TOPK || cfg->router_mode == B200_ROUTER_TOPK_SOFTMAX,
               "unknown router_mode");
  return 0;
}

#define CTX_ENTER(ctx)                             \
  B200_REQUIRE((ctx) != nullptr, "context is null"); \
  B200_CUDA(cudaSetDevice((ctx)->device));          \
  (ctx)->begin()

#define LAUNCHED(ctx, n)                                                        \
  do {                                                                          \
    (ctx)->launches += (n);                                                     \
    cudaError_t _le = cudaGetLastError();                                       \
    if (_le != cudaSuccess) B200_FAIL(std::string("kernel launch failed: ") + cudaGetErrorString(_le)); \
  } while (0)

static inline int permute_launches(int64_t n) { return n <= 1024 ? 1 : 3; }
// rows per expert (average over the experts that can be active) from which the tensor-core kernel is used
constexpr int64_t kTensorCoreRowsPerExpert = 14;
// the same when both products of the block can use the register kernel's shared-memory-resident variant, whose
// further passes over an expert's rows cost no weight traffic
constexpr int64_t kTensorCoreRowsPerExpertStaged = 19;
constexpr int kTicketWord = 8;  // word of the status block that the fused small-batch router uses as its ticket counter
// Status block of a context: word 0 = device-side status, word 8 = ticket of the fused router, words 16..63 =
// self-timing of development builds.
constexpr size_t kStatusBytes = 1024;

extern "C" {

const char* b200_last_error(void) { return g_last_error.c_str(); }

void b200_set_error_handler(void (*handler)(const char*, void*), void* data, void (*dtor)(void*)) {
  std::lock_guard<std::mutex> lk(g_handler_mu);
  if (g_handler_dtor && g_handler_data) g_handler_dtor(g_handler_data);
  g_handler = handler;
  g_handler_data = data;
  g_handler_dtor = dtor;
}

int b200_ctx_create(b200_ctx** out, int device) {
  B200_REQUIRE(out != nullptr, "out is null");
  int n = 0;
  B200_CUDA(cudaGetDeviceCount(&n));
  B200_REQUIRE(device >= 0 && device < n, "no such CUDA device");
  B200_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  B200_CUDA(cudaGetDeviceProperties(&prop, device));
  B200_REQUIRE(prop.major == 10, "this library contains sm_100a code only; a Blackwell B200 is required");
  b200_ctx* c = new b200_ctx();
  c->device = device;
  if (cudaMalloc(reinterpret_cast<void**>(&c->err), kStatusBytes) != cudaSuccess ||
      cudaMemset(c->err, 0, kStatusBytes) != cudaSuccess) {
    delete c;
    B200_FAIL("cannot allocate the status word");
  }
  *out = c;
  return 0;
}

int b200_ctx_destroy(b200_ctx* c) {
  if (!c) return 0;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  if (c->ws) cudaFree(c->ws);
  if (c->err) cudaFree(c->err);
  for (auto& e : c->ev)
    if (e) cudaEventDestroy(e);
  delete c;
  return 0;
}

int b200_ctx_reserve(b200_ctx* c, const b200_moe_config* cfg, int64_t max_tokens) {
  CTX_ENTER(c);
  if (check_cfg(cfg)) return 1;
  B200_REQUIRE(max_tokens >= 0, "max_tokens is negative");
  return ctx_grow(c, block_scratch_bytes(*cfg, max_tokens));
}

int b200_workspace_bytes(const b200_moe_config* cfg, int64_t max_tokens, size_t* bytes) {
  if (check_cfg(cfg)) return 1;
  B200_REQUIRE(bytes != nullptr && max_tokens >= 0, "bad arguments");
  *bytes = block_scratch_bytes(*cfg, max_tokens);
  return 0;
}

int b200_ctx_check(b200_ctx* c, void* stream) {
  CTX_ENTER(c);
  B200_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int h = 0;
  B200_CUDA(cudaMemcpy(&h, c->err, sizeof(int), cudaMemcpyDeviceToHost));
  if (h != 0) {
    B200_CUDA(cudaMemset(c->err, 0, sizeof(int)));
    // a kernel that gave up waiting may have left its ticket half-way
    if (h == 3) B200_CUDA(cudaMemset(c->err + kTicketWord, 0, kStatusBytes - sizeof(int) * kTicketWord));
    B200_FAIL(h == 2   ? "an expert index was out of range"
              : h == 3 ? "a kernel gave up waiting on its own pipeline (2 s limit)"
              : h == 5 ? "a rank would receive more rows than its exchange buffers hold"
              : h == 6 ? "per-expert counts or an expert-parallel routing table did not agree with the row count"
                       : "a gather index was out of range");
  }
  return 0;
}

int64_t b200_ctx_launch_count(const b200_ctx* c) { return c ? c->launches : 0; }

int b200_ctx_debug_words(b200_ctx* c, int32_t* host_out, int n) {
  CTX_ENTER(c);
  B200_REQUIRE(host_out != nullptr && n > 0 && n <= 64, "n must be in 1..64");
  B200_CUDA(cudaDeviceSynchronize());
  B200_CUDA(cudaMemcpy(host_out, c->err, sizeof(int32_t) * n, cudaMemcpyDeviceToHost));
  return 0;
}

int b200_ctx_set_qmm_path(b200_ctx* c, int path) {
  CTX_ENTER(c);
  B200_REQUIRE(path == B200_QMM_AUTO || path == B200_QMM_SMALL || path == B200_QMM_TENSOR_CORE, "unknown path");
  c->qmm_path = path;
  return 0;
}

int b200_ctx_set_profiling(b200_ctx* c, int enable) {
  CTX_ENTER(c);
  if (enable && !c->ev[0])
    for (auto& e : c->ev) B200_CUDA(cudaEventCreate(&e));
  c->profiling = enable != 0;
  c->ev_valid = false;
  return 0;
}

int b200_ctx_stage_ms(b200_ctx* c, float* ms, int n) {
  CTX_ENTER(c);
  B200_REQUIRE(ms != nullptr && n >= B200_N_STAGES, "ms must hold B200_N_STAGES floats");
  B200_REQUIRE(c->profiling && c->ev_valid, "no profiled b200_moe_block_forward call to report");
  B200_CUDA(cudaEventSynchronize(c->ev[B200_N_STAGES]));
  for (int i = 0; i < B200_N_STAGES; ++i) B200_CUDA(cudaEventElapsedTime(&ms[i], c->ev[i], c->ev[i + 1]));
  return 0;
}

// ---- plain ops ----------------------------------------------------------------------------------

static int check_quant_args(int gs, int bits, int64_t K) {
  B200_REQUIRE(bits == 2 || bits == 4 || bits == 8, "bits must be 2, 4 or 8");
  B200_REQUIRE(gs == 32 || gs == 64 || gs == 128, "group_size must be 32, 64 or 128");
  B200_REQUIRE(K > 0 && K % gs == 0, "the last axis must be a multiple of group_size");
  return 0;
}

int b200_quantize(b200_ctx* c, const void* w, int dtype, int64_t rows, int64_t K, int gs, int bits, uint32_t* wq,
                  void* scales, void* biases, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(dtype == B200_F32 || dtype == B200_BF16, "dtype must be float32 or bfloat16");
  if (check_quant_args(gs, bits, K)) return 1;
  B200_REQUIRE(rows >= 0, "rows is negative");
  B200_REQUIRE(rows == 0 || (w && wq && scales && biases), "null tensor");
  if (launch_quantize(w, dtype == B200_BF16, rows, K, gs, bits, wq, scales, biases, static_cast<cudaStream_t>(stream)))
    return 1;
  LAUNCHED(c, rows ? 1 : 0);
  return 0;
}

int b200_dequantize(b200_ctx* c, const uint32_t* wq, const void* scales, const void* biases, int dtype, int64_t rows,
                    int64_t K, int gs, int bits, void* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(dtype == B200_F32 || dtype == B200_BF16, "dtype must be float32 or bfloat16");
  if (check_quant_args(gs, bits, K)) return 1;
  B200_REQUIRE(rows >= 0, "rows is negative");
  B200_REQUIRE(rows == 0 || (wq && scales && biases && out), "null tensor");
  if (launch_dequantize(wq, scales, biases, dtype == B200_BF16, rows, K, gs, bits, out, static_cast<cudaStream_t>(stream)))
    return 1;
  LAUNCHED(c, rows ? 1 : 0);
  return 0;
}

// Shared by quantized_matmul and gather_qmm (bf16, transpose = true, group 64, 4 or 8 bits): one grouped product
// of n sorted rows over bf16 source rows x [src_rows, K].  Few rows per weight matrix: the register kernel on
// prepared rows; many: the tcgen05 kernel on gathered fp16 rows (same rule as the routed block).
static bool grouped_wants_tensor_cores(const b200_ctx* c, int K, int N, int64_t n, int max_active) {
  if (!prefill_shape_ok(K, N, 1)) return false;
  if (!small_shape_ok(K) || c->qmm_path == B200_QMM_TENSOR_CORE) return true;
  if (c->qmm_path == B200_QMM_SMALL) return false;
  return n / (max_active > 0 ? max_active : 1) >= kTensorCoreRowsPerExpert;
}
static size_t grouped_scratch_bytes(int64_t n, int64_t src_rows, int64_t K, int64_t E) {
  const int64_t r = n > src_rows ? n : src_rows;
  return al(sizeof(uint16_t) * r * K) + al(sizeof(float) * r) + (al(sizeof(uint32_t) * prefill_tile_words(n, (int)E)) * 3 + al(16));
}
static int run_grouped(b200_ctx* c, GroupedArgs& a, int bits, int max_active, int64_t n, const void* x, int64_t src_rows,
                       const uint32_t* counts, cudaStream_t st) {
  if (n == 0) return 0;
  const int E = a.n_experts;
  if (grouped_wants_tensor_cores(c, a.K, a.N, n, max_active)) {
    const size_t tw = prefill_tile_words(n, E);
    uint32_t* tile_expert = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    uint32_t* tile_row0 = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    uint32_t* tile_rows = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    uint32_t* n_row_tiles = static_cast<uint32_t*>(c->take(16));
    void* xs = c->take(sizeof(uint16_t) * n * a.K);
    float* rs = static_cast<float*>(c->take(sizeof(float) * n));
    B200_REQUIRE(tile_expert && tile_row0 && tile_rows && n_row_tiles && xs && rs, "scratch arena too small");
    launch_build_row_tiles(counts, a.offsets, E, tile_expert, tile_row0, tile_rows, n_row_tiles, 256, st);
    // rows that exist = offsets[E]: assignments with an out-of-range matrix index were left out of the sort
    launch_prepare_rows(x, a.perm, a.src_map, 1, n, a.offsets + E, a.K, bits == 4, xs, rs, st);
    if (launch_grouped_qmm_tc(xs, rs, n, a, 1, bits, tile_expert, tile_row0, tile_rows, n_row_tiles, E, false, c->err, st))
      return 1;
    LAUNCHED(c, 3);
    return 0;
  }
  B200_REQUIRE(small_shape_ok(a.K), "K too large");
  void* xs = c->take(sizeof(uint16_t) * src_rows * a.K);
  float* rs = static_cast<float*>(c->take(sizeof(float) * src_rows));
  B200_REQUIRE(xs && rs, "scratch arena too small");
  if (launch_prepare_rows_small(x, 0, src_rows, nullptr, a.K, bits, xs, rs, st)) return 1;
  a.x = xs;
  a.x_rowscale = rs;
  if (launch_grouped_qmm_small(a, 1, bits, max_active, n, st)) return 1;
  LAUNCHED(c, 2);
  return 0;
}

static int check_qmm_common(int gs, int bits, int dtype, int transpose, int64_t K, int64_t N) {
  B200_REQUIRE(dtype == B200_F32 || dtype == B200_BF16 || dtype == B200_F16, "dtype must be float32, bfloat16 or float16");
  B200_REQUIRE(bits == 2 || bits == 4 || bits == 8, "bits must be 2, 4 or 8");
  B200_REQUIRE(gs == 32 || gs == 64 || gs == 128, "group_size must be 32, 64 or 128");
  if (transpose)
    B200_REQUIRE(K % gs == 0, "K must be a multiple of group_size");
  else
    B200_REQUIRE(N % gs == 0, "N must be a multiple of group_size when transpose is false");
  return 0;
}
static bool fast_qmm_form(int gs, int bits, int dtype, int transpose) {
  return dtype == B200_BF16 && transpose && gs == 64 && (bits == 4 || bits == 8);
}

int b200_quantized_matmul(b200_ctx* c, const void* x, const uint32_t* w, const void* scales, const void* biases,
                          int transpose, int gs, int bits, int dtype, int64_t M, int64_t K, int64_t N, void* out,
                          void* stream) {
  CTX_ENTER(c);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_REQUIRE(M >= 0 && K > 0 && N > 0 && M < (int64_t(1) << 31), "bad shape");
  if (check_qmm_common(gs, bits, dtype, transpose, K, N)) return 1;
  B200_REQUIRE(biases != nullptr, "biases are required in affine mode");
  B200_REQUIRE(M == 0 || (x && w && scales && out), "null tensor");
  if (M == 0) return 0;
  if (!fast_qmm_form(gs, bits, dtype, transpose) || (!small_shape_ok((int)K) && !prefill_shape_ok((int)K, (int)N, 1))) {
    if (launch_gather_qmm_generic(x, w, scales, biases, nullptr, nullptr, dtype, 1, M, K, 1, N, 1, transpose, gs, bits, out, c->err,
                                  st))
      return 1;
    LAUNCHED(c, 1);
    return 0;
  }
  if (ctx_grow(c, 4096 + grouped_scratch_bytes(M, M, K, 1), stream)) return 1;
  uint32_t* seg = static_cast<uint32_t*>(c->take(64));
  launch_dense_segments(seg + 0, seg + 4, seg + 8, seg + 12, (uint32_t)M, st);
  LAUNCHED(c, 1);
  GroupedArgs a{};
  a.w[0] = w;
  a.scales[0] = scales;
  a.biases[0] = biases;
  a.offsets = seg + 4;
  a.active = seg + 8;
  a.n_active = seg + 12;
  a.src_mode = kSrcIdent;
  a.dst_perm = 0;
  a.out = out;
  a.K = (int)K;
  a.N = (int)N;
  a.n_experts = 1;
  return run_grouped(c, a, bits, 1, M, x, M, seg + 0, st);
}

int b200_gather_qmm(b200_ctx* c, const void* x, const uint32_t* w, const void* scales, const void* biases,
                    const uint32_t* lhs, const uint32_t* rhs, int transpose, int gs, int bits, int sorted_indices, int dtype,
                    int64_t Bx, int64_t M, int64_t K, int64_t E, int64_t N, int64_t n_idx, void* out, void* stream) {
  (void)sorted_indices;
  CTX_ENTER(c);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_REQUIRE(Bx > 0 && M > 0 && K > 0 && N > 0 && n_idx >= 0, "bad shape");
  if (check_qmm_common(gs, bits, dtype, transpose, K, N)) return 1;
  B200_REQUIRE(lhs != nullptr || n_idx <= Bx, "without lhs_indices x needs one batch entry per index");
  B200_REQUIRE(E > 0, "w needs at least one matrix");
  B200_REQUIRE(biases != nullptr, "biases are required in affine mode");
  B200_REQUIRE(rhs != nullptr, "rhs_indices is required");
  if (n_idx == 0) return 0;
  B200_REQUIRE(x && w && scales && out, "null tensor");
  const int64_t n = n_idx * M;
  B200_REQUIRE(n < (int64_t(1) << 31), "too many rows");
  if (!fast_qmm_form(gs, bits, dtype, transpose) || E > 256 ||
      (!small_shape_ok((int)K) && !prefill_shape_ok((int)K, (int)N, 1))) {
    if (launch_gather_qmm_generic(x, w, scales, biases, lhs, rhs, dtype, Bx, M, K, E, N, n_idx, transpose, gs, bits, out, c->err,
                                  st))
      return 1;
    LAUNCHED(c, 1);
    return 0;
  }
  size_t need = al(sizeof(uint32_t) * n) * 4 + al(sizeof(uint32_t) * (E + 1)) * 3 + al(16) +
                al(sizeof(uint32_t) * permute_scratch_words(n, (int)E)) + grouped_scratch_bytes(n, Bx * M, K, E) + 4096;
  if (ctx_grow(c, need, stream)) return 1;
  uint32_t* flat_e = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
  uint32_t* flat_s = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
  uint32_t* perm = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
  uint32_t* inv = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
  uint32_t* counts = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* offsets = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* active = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* n_active = static_cast<uint32_t*>(c->take(16));
  uint32_t* chunk = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * permute_scratch_words(n, (int)E)));
  launch_expand_indices(lhs, rhs, n_idx, (int)M, Bx, flat_e, flat_s, c->err, st);
  launch_permute(flat_e, n, (int)E, perm, inv, counts, offsets, active, n_active, chunk, c->err, st);
  LAUNCHED(c, 1 + permute_launches(n));
  GroupedArgs a{};
  a.w[0] = w;
  a.scales[0] = scales;
  a.biases[0] = biases;
  a.offsets = offsets;
  a.active = active;
  a.n_active = n_active;
  a.perm = perm;
  a.src_map = flat_s;
  a.src_mode = kSrcMap;
  a.dst_perm = 1;
  a.out = out;
  a.K = (int)K;
  a.N = (int)N;
  a.n_experts = (int)E;
  return run_grouped(c, a, bits, (int)(E < n ? E : n), n, x, Bx * M, counts, st);
}

int b200_gather_mm(b200_ctx* c, const void* a, const void* b, const uint32_t* lhs_indices, const uint32_t* rhs_indices,
                   int64_t Ba, int64_t Bb, int64_t M, int64_t K, int64_t N, int64_t n_idx, void* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(Ba > 0 && Bb > 0 && M >= 0 && K > 0 && N >= 0 && n_idx >= 0, "bad shape");
  B200_REQUIRE(M < (1 << 20) && K < (1 << 24) && N < (1 << 24), "dimension too large");
  B200_REQUIRE(lhs_indices || n_idx <= Ba, "without lhs_indices a needs one batch entry per index");
  B200_REQUIRE(rhs_indices || n_idx <= Bb, "without rhs_indices b needs one batch entry per index");
  if (n_idx == 0 || M == 0 || N == 0) return 0;
  B200_REQUIRE(a && b && out, "null tensor");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n = n_idx * M;
  // enough rows to fill 128-row tiles and a shape the tensor-core kernel takes: sort the rows by matrix, gather a
  // into that order and run the grouped tcgen05 kernel without its dequantisation stage
  if (K % 64 == 0 && N % 8 == 0 && Bb <= 256 && n >= 512 && n < (int64_t(1) << 31) && c->qmm_path != B200_QMM_SMALL) {
    const int E = (int)Bb;
    const size_t tw = prefill_tile_words(n, E);
    size_t need = al(sizeof(uint32_t) * n) * 4 + al(sizeof(uint32_t) * (E + 1)) * 3 + al(16) +
                  al(sizeof(uint32_t) * permute_scratch_words(n, E)) + al(sizeof(uint16_t) * n * K) +
                  (al(sizeof(uint32_t) * tw) * 3 + al(16)) + 4096;
    if (ctx_grow(c, need, stream)) return 1;
    uint32_t* flat_e = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
    uint32_t* flat_s = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
    uint32_t* perm = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
    uint32_t* inv = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
    uint32_t* counts = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
    uint32_t* offsets = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
    uint32_t* active = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
    uint32_t* n_active = static_cast<uint32_t*>(c->take(16));
    uint32_t* chunk = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * permute_scratch_words(n, E)));
    void* a_sorted = c->take(sizeof(uint16_t) * n * K);
    uint32_t* tile_expert = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    uint32_t* tile_row0 = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    uint32_t* tile_rows = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    uint32_t* n_row_tiles = static_cast<uint32_t*>(c->take(16));
    B200_REQUIRE(flat_e && flat_s && perm && inv && counts && offsets && active && n_active && chunk && a_sorted && tile_expert &&
                     tile_row0 && tile_rows && n_row_tiles,
                 "scratch arena too small");
    launch_expand_indices(lhs_indices, rhs_indices, n_idx, (int)M, Ba, flat_e, flat_s, c->err, st);
    launch_permute(flat_e, n, E, perm, inv, counts, offsets, active, n_active, chunk, c->err, st);
    launch_gather_rows(a, perm, flat_s, n, offsets + E, K, a_sorted, st);
    launch_build_row_tiles(counts, offsets, E, tile_expert, tile_row0, tile_rows, n_row_tiles, 256, st);
    if (launch_gather_mm_tc(a_sorted, n, b, E, (int)K, (int)N, perm, out, tile_expert, tile_row0, tile_rows, n_row_tiles, c->err, st))
      return 1;
    LAUNCHED(c, 4 + permute_launches(n));
    return 0;
  }
  if (launch_gather_mm(a, b, lhs_indices, rhs_indices, Ba, Bb, M, K, N, n_idx, out, c->err, st)) return 1;
  LAUNCHED(c, 1);
  return 0;
}

int b200_softmax_axis(b200_ctx* c, const void* a, int64_t rows, int64_t cols, int precise, void* out, void* stream) {
  (void)precise;
  CTX_ENTER(c);
  B200_REQUIRE(cols > 0 && cols <= 256, "cols must be in 1..256");
  B200_REQUIRE(rows >= 0 && (rows == 0 || (a && out)), "bad arguments");
  launch_softmax(a, (int)rows, (int)cols, out, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, rows ? 1 : 0);
  return 0;
}

int b200_argpartition_axis(b200_ctx* c, const void* a, int64_t rows, int64_t cols, int kth, uint32_t* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(cols > 0 && cols <= 256, "cols must be in 1..256");
  B200_REQUIRE(kth >= 0 && kth < cols, "kth is out of range for the axis");
  B200_REQUIRE(rows >= 0 && (rows == 0 || (a && out)), "bad arguments");
  launch_argpartition(a, (int)rows, (int)cols, kth, out, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, rows ? 1 : 0);
  return 0;
}

int b200_take_along_axis(b200_ctx* c, const void* a, int64_t rows, int64_t cols, const uint32_t* idx, int64_t icols,
                         void* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(rows >= 0 && cols > 0 && icols >= 0, "bad shape");
  B200_REQUIRE(rows * icols == 0 || (a && idx && out), "null tensor");
  launch_take_along(a, (int)rows, (int)cols, idx, (int)icols, out, c->err, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, rows * icols ? 1 : 0);
  return 0;
}

int b200_take_rows(b200_ctx* c, const void* x, const uint32_t* indices, uint32_t div, int64_t n_rows, int64_t x_rows,
                   int64_t cols, void* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(div >= 1, "div must be at least 1");
  B200_REQUIRE(n_rows >= 0 && x_rows >= 0 && cols > 0 && cols % 8 == 0, "cols must be a positive multiple of 8");
  B200_REQUIRE(n_rows == 0 || (x && indices && out), "null tensor");
  launch_take_rows(x, indices, div, n_rows, x_rows, cols, out, c->err, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, n_rows ? 1 : 0);
  return 0;
}

int b200_take_axis(b200_ctx* c, const void* x, const uint32_t* indices, int64_t n_rows, int64_t x_rows, int64_t cols,
                   void* out, void* stream) {
  return b200_take_rows(c, x, indices, 1, n_rows, x_rows, cols, out, stream);
}

int b200_argsort_axis(b200_ctx* c, const uint32_t* keys, int64_t rows, int64_t cols, int key_bound, uint32_t* out,
                      void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(key_bound > 0 && key_bound <= 256, "key_bound must be in 1..256");
  B200_REQUIRE(rows >= 0 && cols >= 0 && cols < (int64_t(1) << 31), "bad shape");
  if (rows * cols == 0) return 0;
  B200_REQUIRE(keys && out, "null tensor");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int E = key_bound;
  size_t need = al(sizeof(uint32_t) * cols) + al(sizeof(uint32_t) * (E + 1)) * 3 + al(16) +
                al(sizeof(uint32_t) * permute_scratch_words(cols, E)) + 4096;
  if (ctx_grow(c, need, stream)) return 1;
  uint32_t* inv = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * cols));
  uint32_t* counts = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* offsets = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* active = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* n_active = static_cast<uint32_t*>(c->take(16));
  uint32_t* chunk = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * permute_scratch_words(cols, E)));
  B200_REQUIRE(inv && counts && offsets && active && n_active && chunk, "scratch arena too small");
  for (int64_t r = 0; r < rows; ++r) {  // stream order keeps the rows from sharing the scratch at the same time
    launch_permute(keys + r * cols, cols, E, out + r * cols, inv, counts, offsets, active, n_active, chunk, c->err, st);
    LAUNCHED(c, permute_launches(cols));
  }
  return 0;
}

int b200_topk_axis(b200_ctx* c, const void* a, int64_t rows, int64_t cols, int k, void* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(cols > 0 && cols <= 256, "cols must be in 1..256");
  B200_REQUIRE(k > 0 && k <= cols, "k is out of range for the axis");
  B200_REQUIRE(rows >= 0 && (rows == 0 || (a && out)), "bad arguments");
  launch_topk_values(a, (int)rows, (int)cols, k, out, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, rows ? 1 : 0);
  return 0;
}

int b200_moe_combine(b200_ctx* c, const void* y_sorted, const uint32_t* inv_perm, const void* scores, int64_t T, int top_k,
                     int64_t hidden, void* out, float* out_f32, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(T >= 0 && top_k > 0 && hidden > 0 && hidden % 4 == 0, "bad shape");
  B200_REQUIRE(T == 0 || (y_sorted && inv_perm && scores && out), "null tensor");
  launch_gather_combine(y_sorted, inv_perm, scores, T, top_k, hidden, out, out_f32, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, T ? 1 : 0);
  return 0;
}

int b200_rms_norm(b200_ctx* c, const void* x, const void* weight, float eps, int64_t rows, int64_t cols, void* out,
                  void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(rows >= 0 && cols > 0 && (rows == 0 || (x && out)), "bad arguments");
  launch_rms_norm(x, nullptr, weight, eps, rows, cols, out, nullptr, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, rows ? 1 : 0);
  return 0;
}

int b200_add_rms_norm(b200_ctx* c, const void* x, const void* residual, const void* weight, float eps, int64_t rows,
                      int64_t cols, void* sum_out, void* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(rows >= 0 && cols > 0 && (rows == 0 || (x && residual && out)), "bad arguments");
  launch_rms_norm(x, residual, weight, eps, rows, cols, out, sum_out, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, rows ? 1 : 0);
  return 0;
}

int b200_add(b200_ctx* c, const void* a, const void* b, int64_t n, void* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(n >= 0 && (n == 0 || (a && b && out)), "bad arguments");
  launch_add(a, b, n, out, static_cast<cudaStream_t>(stream));
  LAUNCHED(c, n ? 1 : 0);
  return 0;
}

// ---- fused entry points ---------------------------------------------------------------------------

int b200_router_topk(b200_ctx* c, const b200_moe_config* cfg, const void* x, const void* wr, const float* logit_bias,
                     int64_t T, uint32_t* indices, void* scores, void* logits, void* stream) {
  CTX_ENTER(c);
  if (check_cfg(cfg)) return 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_REQUIRE(T >= 0 && T < (1 << 24), "bad token count");
  if (T == 0) return 0;
  B200_REQUIRE(x && wr && indices && scores, "null tensor");
  const size_t w64_bytes = sizeof(double) * (size_t)cfg->n_experts * cfg->hidden;
  if (ctx_grow(c, al(sizeof(uint16_t) * T * cfg->n_experts) + al(w64_bytes) + 4096, stream)) return 1;
  if (!logits) logits = c->take(sizeof(uint16_t) * T * cfg->n_experts);
  double* w64 = static_cast<double*>(c->take(w64_bytes));
  B200_REQUIRE(logits && w64, "scratch arena too small");
  launch_router_logits(x, wr, logit_bias, logits, (int)T, cfg->hidden, cfg->n_experts, w64, st);
  launch_route_topk(logits, (int)T, cfg->n_experts, cfg->top_k, cfg->router_mode, cfg->norm_topk_prob, indices, scores,
                    nullptr, st);
  LAUNCHED(c, 2);
  return 0;
}

int b200_moe_permute(b200_ctx* c, const uint32_t* indices, int64_t n, int E, uint32_t* perm, uint32_t* inv,
                     uint32_t* counts, uint32_t* offsets, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(E > 0 && E <= 256, "n_experts must be in 1..256");
  B200_REQUIRE(n >= 0 && n < (int64_t(1) << 31), "bad assignment count");
  B200_REQUIRE(counts && offsets, "counts and offsets are required");
  B200_REQUIRE(n == 0 || (indices && perm && inv), "null tensor");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  size_t need = al(sizeof(uint32_t) * (E + 1)) + al(16) + al(sizeof(uint32_t) * permute_scratch_words(n, E)) + 4096;
  if (ctx_grow(c, need, stream)) return 1;
  uint32_t* active = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* n_active = static_cast<uint32_t*>(c->take(16));
  uint32_t* chunk = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * permute_scratch_words(n, E)));
  launch_permute(indices, n, E, perm, inv, counts, offsets, active, n_active, chunk, c->err, st);
  LAUNCHED(c, permute_launches(n));
  return 0;
}

// Which grouped-product kernel a block of n assignments over at most `max_active` experts uses.
static bool use_tensor_core_path(const b200_ctx* c, const b200_moe_config& cfg, int64_t n, int max_active) {
  if (!prefill_shape_ok(cfg.hidden, cfg.inter, 2) || !prefill_shape_ok(cfg.inter, cfg.hidden, 1)) return false;
  // the memory-bound kernels stage eight activation rows of length K in shared memory; beyond
  // that (e.g. the 14336-wide down projection of a Mixtral-shaped layer) only the tensor-core
  // kernel, which streams activations by TMA, applies
  if (!small_shape_ok(cfg.hidden) || !small_shape_ok(cfg.inter)) return true;
  if (c->qmm_path == B200_QMM_SMALL) return false;
  if (c->qmm_path == B200_QMM_TENSOR_CORE) return true;
  // measured crossover (whole block, register kernel against tensor-core kernel).  Qwen3-235B-A22B layer (gate/up
  // too wide for the shared-memory-resident variant): 12 rows per expert 1.01 against 1.10 ms, 16 rows 1.14 against
  // 1.05.  Qwen3-30B-A3B layer (resident variant for both products): 16 rows 0.292 against 0.332 ms, 18 rows 0.316
  // against 0.333, 20 rows 0.344 against 0.333
  const bool resident = small_staged_ok(cfg.hidden, cfg.bits, 2) && small_staged_ok(cfg.inter, cfg.bits, 1);
  return n / (max_active > 0 ? max_active : 1) >= (resident ? kTensorCoreRowsPerExpertStaged : kTensorCoreRowsPerExpert);
}

// Rows of an expert-parallel exchange: the sorted rows are gathered from a buffer of token rows through `map`
// (sorted position -> token row); the numbers of sorted rows and of token rows live on the device.
// The block's output buffers, for batches small enough that the down projection finishes the block itself (routing
// weights and the k-way sum in its epilogue): experts_sorted then reports *yk_fmt = kOutNone and the caller skips
// the combine.
struct SmallTail {
  const uint32_t* idx;  // [T, k]
  const uint32_t* inv;  // [T*k]
  void* out;            // bf16 [T, H]
  float* out_f32;       // optional
  int64_t T;
  const uint32_t* desc; // per-expert records written by the routing kernel (tokens as source rows, no row scales)
};

struct ExchangeRows {
  const uint32_t* map;          // [n] sorted position -> row of x
  int64_t src_rows_bound;       // host bound on the rows of x
  const uint32_t* src_rows_dev; // device word: rows of x that exist
  const uint32_t* n_dev;        // device word: sorted rows that exist
};

// Gate/up and down products over rows that are grouped by expert (offsets/active/n_active describe
// the groups).  `perm` non-null: source row of sorted position p is perm[p] / src_div and the output
// row is perm[p] (un-sorted on the fly); `perm` null: rows are already in expert order and stay so.
static int experts_sorted(b200_ctx* c, const b200_moe_config& cfg, const b200_moe_params& p, const void* x,
                          const uint32_t* perm, int src_div, const uint32_t* counts, const uint32_t* offsets,
                          const uint32_t* active, const uint32_t* n_active, int64_t n, const void* scores, void* yk,
                          cudaStream_t st, int* yk_fmt, const unsigned long long* out_row_addr = nullptr,
                          const ExchangeRows* xr = nullptr, const SmallTail* tail = nullptr);

// Outputs of the token -> expert sort (scratch, or the caller's aux buffers where given).
struct SortBufs {
  uint32_t *perm, *inv, *counts, *offsets, *active, *n_active, *chunk;
};
static int take_sort_bufs(b200_ctx* c, int64_t n, int E, const b200_moe_aux* aux, SortBufs& sb) {
  sb.perm = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
  sb.inv = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
  sb.counts = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  sb.offsets = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  sb.active = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  sb.n_active = static_cast<uint32_t*>(c->take(16));
  sb.chunk = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * permute_scratch_words(n, E)));
  B200_REQUIRE(sb.perm && sb.inv && sb.counts && sb.offsets && sb.active && sb.n_active && sb.chunk,
               "scratch arena too small");
  if (aux) {
    if (aux->perm) sb.perm = aux->perm;
    if (aux->inv_perm) sb.inv = aux->inv_perm;
    if (aux->counts) sb.counts = aux->counts;
    if (aux->offsets) sb.offsets = aux->offsets;
  }
  return 0;
}

// Shared tail of switch_glu_forward and moe_block_forward: permute, gate/up, down.
// `scores` null: unweighted per-assignment outputs go to `yk` ([T*k, H]).
static int experts_forward(b200_ctx* c, const b200_moe_config& cfg, const b200_moe_params& p, const void* x,
                           const uint32_t* idx, const void* scores, int64_t T, void* yk, const b200_moe_aux* aux,
                           cudaStream_t st, int* yk_fmt = nullptr) {
  const int64_t n = T * cfg.top_k;
  const int E = cfg.n_experts;
  SortBufs sb;
  if (take_sort_bufs(c, n, E, aux, sb)) return 1;
  launch_permute(idx, n, E, sb.perm, sb.inv, sb.counts, sb.offsets, sb.active, sb.n_active, sb.chunk, c->err, st);
  LAUNCHED(c, permute_launches(n));
  return experts_sorted(c, cfg, p, x, sb.perm, cfg.top_k, sb.counts, sb.offsets, sb.active, sb.n_active, n, scores, yk, st,
                        yk_fmt);
}

static int experts_sorted(b200_ctx* c, const b200_moe_config& cfg, const b200_moe_params& p, const void* x,
                          const uint32_t* perm, int src_div, const uint32_t* counts, const uint32_t* offsets,
                          const uint32_t* active, const uint32_t* n_active, int64_t n, const void* scores, void* yk,
                          cudaStream_t st, int* yk_fmt, const unsigned long long* out_row_addr, const ExchangeRows* xr,
                          const SmallTail* tail) {
  // n is the host's bound on the number of rows; with `xr` the rows that exist are counted on the device
  // (everything below is driven by the device-side segment tables, only the row preparation needs the extra
  // words) and are gathered from x through xr->map
  const uint32_t* n_dev = xr ? xr->n_dev : offsets + cfg.n_experts;  // (sorted rows that exist: offsets[E])
  const int E = cfg.n_experts;
  void* h = c->take(sizeof(uint16_t) * n * cfg.inter);
  B200_REQUIRE(h, "scratch arena too small");
  const int max_active = (int)(E < n ? E : n);

  // Regime: the tensor-core path once experts own enough rows to fill 128-row tiles.
  const bool tc = use_tensor_core_path(c, cfg, n, max_active);
  // two row-tile lists: 256-row tiles for gate/up (both accumulators share each dequantised weight
  // stage), 128-row tiles for down (short K: the accumulators alternate so that the drain of one
  // tile runs under the products of the next)
  uint32_t *tile_expert = nullptr, *tile_row0 = nullptr, *tile_rows = nullptr, *n_row_tiles = nullptr;
  uint32_t *tile_expert1 = nullptr, *tile_row01 = nullptr, *tile_rows1 = nullptr, *n_row_tiles1 = nullptr;
  void* xs = nullptr;
  float* rs_x = nullptr;
  // down projection: 256-row tiles whose two accumulators share every dequantised weight stage, like gate/up, once
  // experts hold enough rows to use both accumulators.  (128-row tiles alternating between the accumulators, so that
  // one tile's drain runs under the next tile's products, measured slower at every K once the outputs became fp16:
  // 1.132 against 1.111 ms per step at K = 768, 3.86 against 3.58 ms at K = 1536, 14.6 against 12.5 ms at K = 14336.)
  // With fewer than 128 rows per expert a tile never reaches its second accumulator, and alternating is what hides
  // the drain: 88 against 116 us at 32 rows per expert.
  bool alt_down = n / (max_active > 0 ? max_active : 1) < 128;
#ifdef B200_DEV
  if (const char* v = getenv("B200_ALT_DOWN")) alt_down = atoi(v) != 0;
#endif
  if (tc) {
    const size_t tw = prefill_tile_words(n, E);
    tile_expert = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    tile_row0 = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    tile_rows = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    n_row_tiles = static_cast<uint32_t*>(c->take(16));
    tile_expert1 = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    tile_row01 = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    tile_rows1 = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * tw));
    n_row_tiles1 = static_cast<uint32_t*>(c->take(16));
    B200_REQUIRE(tile_expert1 && tile_row01 && tile_rows1 && n_row_tiles1, "scratch arena too small");
    xs = c->take(sizeof(uint16_t) * n * cfg.hidden);
    rs_x = static_cast<float*>(c->take(sizeof(float) * n));
    B200_REQUIRE(tile_expert && tile_row0 && tile_rows && n_row_tiles && xs && rs_x, "scratch arena too small");
    launch_build_row_tiles(counts, offsets, E, tile_expert, tile_row0, tile_rows, n_row_tiles, 256, st);
    if (alt_down) launch_build_row_tiles(counts, offsets, E, tile_expert1, tile_row01, tile_rows1, n_row_tiles1, 128, st);
    LAUNCHED(c, alt_down ? 2 : 1);
  }
  c->mark(3, st);

  uint32_t* expert_desc = nullptr;
  GroupedArgs gu{};
  gu.x = x;
  gu.w[0] = p.gate_proj.weight;
  gu.scales[0] = p.gate_proj.scales;
  gu.biases[0] = p.gate_proj.biases;
  gu.w[1] = p.up_proj.weight;
  gu.scales[1] = p.up_proj.scales;
  gu.biases[1] = p.up_proj.biases;
  gu.offsets = offsets;
  gu.active = active;
  gu.n_active = n_active;
  gu.perm = perm;
  gu.src_mode = perm ? kSrcPermDiv : kSrcIdent;
  gu.src_div = src_div;
  gu.dst_perm = 0;
  gu.out = h;
  gu.out_f16 = tc ? 1 : 0;  // the tensor-core down projection takes fp16 rows: its producer writes them directly
  gu.K = cfg.hidden;
  gu.N = cfg.inter;
  gu.n_experts = E;
  if (tc) {
    // rows gathered into expert order, converted to row-normalised fp16, in the k order the 4-bit unpack produces
    launch_prepare_rows(x, perm, xr ? xr->map : nullptr, perm ? src_div : 1, n, n_dev, cfg.hidden, cfg.bits == 4, xs, rs_x, st);
    c->mark(4, st);
    if (launch_grouped_qmm_tc(xs, rs_x, n, gu, 2, cfg.bits, tile_expert, tile_row0, tile_rows, n_row_tiles, E, false,
                              c->err, st))
      return 1;
    LAUNCHED(c, 2);
  } else {
    // register kernel: the source rows (the tokens when rows are gathered through perm, else the n rows
    // themselves) are prepared once - fp16, row-scaled, unpack order - and every CTA copies what it needs
    const int64_t src_rows = xr ? xr->src_rows_bound : (perm ? n / src_div : n);
    if (!xr && src_rows <= 8) {
      // a handful of rows: every CTA prepares the rows it stages itself, which costs less than a launch
      gu.x_bf16 = 1;
      if (tail && tail->desc && perm && src_div == cfg.top_k) gu.desc = tail->desc;
      gu.late_trigger = 1;  // lets the fused down projection fetch routing outputs and weights before its wait
      c->mark(4, st);
    } else {
      void* xp = c->take(sizeof(uint16_t) * src_rows * cfg.hidden);
      float* rp = static_cast<float*>(c->take(sizeof(float) * src_rows));
      B200_REQUIRE(xp && rp, "scratch arena too small");
      if (launch_prepare_rows_small(x, 0, src_rows, xr ? xr->src_rows_dev : nullptr, cfg.hidden, cfg.bits, xp, rp, st)) return 1;
      LAUNCHED(c, 1);
      c->mark(4, st);
      gu.x = xp;
      gu.x_rowscale = rp;
    }
    if (xr) {
      gu.src_mode = kSrcMapDirect;
      gu.src_map = xr->map;
    }
    gu.out_f16 = 1;  // h in the prepared layout, ready for the down projection
    if (!gu.x_bf16) {
      // one record per active expert: the products' CTAs then start with one load instead of four dependent ones
      expert_desc = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * kExpertDescWords * (size_t)max_active));
      B200_REQUIRE(expert_desc, "scratch arena too small");
      if (launch_expert_descs(active, n_active, offsets, gu.perm, gu.src_map, gu.src_mode, gu.src_div, gu.x_rowscale, max_active,
                              expert_desc, st))
        return 1;
      LAUNCHED(c, 1);
      gu.desc = expert_desc;
#ifdef B200_DEV
      if (getenv("B200_SMALL_NO_DESC")) gu.desc = expert_desc = nullptr;
#endif
    }
    if (launch_grouped_qmm_small(gu, 2, cfg.bits, max_active, n, st)) return 1;
    LAUNCHED(c, 1);
  }
  c->mark(5, st);

  if (!tc && tail && scores && !xr && !out_row_addr && down_combine_small_ok(tail->T, cfg.top_k, cfg.inter)) {
    // a handful of tokens: down projection, routing weights and the k-way sum in one launch
    DownCombineArgs dc{};
    dc.h = h;
    dc.idx = tail->idx;
    dc.inv = tail->inv;
    dc.scores = scores;
    dc.w = p.down_proj.weight;
    dc.scales = p.down_proj.scales;
    dc.biases = p.down_proj.biases;
    dc.out = tail->out;
    dc.out_f32 = tail->out_f32;
    dc.T = (int)tail->T;
    dc.k = cfg.top_k;
    dc.K = cfg.inter;
    dc.N = cfg.hidden;
    dc.early_routing = gu.late_trigger;
    c->mark(6, st);
    if (launch_down_combine_small(dc, cfg.bits, st)) return 1;
    LAUNCHED(c, 1);
    c->mark(7, st);
    if (yk_fmt) *yk_fmt = kOutNone;
    return 0;
  }

  GroupedArgs dn{};
  dn.x = h;
  dn.w[0] = p.down_proj.weight;
  dn.scales[0] = p.down_proj.scales;
  dn.biases[0] = p.down_proj.biases;
  dn.offsets = offsets;
  dn.active = active;
  dn.n_active = n_active;
  dn.perm = perm;
  dn.src_mode = kSrcIdent;
  dn.dst_perm = perm ? 1 : 0;
  dn.row_scale = scores;
  dn.out = yk;
  // weighted rows keep more than bf16's 8 significant bits until the combine (bf16 rows measured 0.017 of
  // the 2e-2 bar at T=512): float32 from the register kernel, fp16 (11 bits, half the traffic of the
  // store-bound epilogue and of the combine's reads) from the tensor-core kernel; SwitchGlu's own output is bf16
  dn.out_f32 = scores != nullptr && !tc;
  dn.out_f16 = tc && !out_row_addr && (scores != nullptr || xr != nullptr);  // exchanged rows: fp16 outputs feed the partial sums
  dn.out_row_addr = out_row_addr;   // rows go to per-row addresses (bf16): the expert-parallel return path
  if (yk_fmt) *yk_fmt = dn.out_f32 ? kOutF32 : (dn.out_f16 ? kOutF16 : kOutBf16);
  dn.K = cfg.inter;
  dn.N = cfg.hidden;
  dn.n_experts = E;
  if (tc) {
    // h is already fp16 in unpack order, unscaled (stage 6, the former conversion pass, is empty)
    c->mark(6, st);
    if (alt_down ? launch_grouped_qmm_tc(h, nullptr, n, dn, 1, cfg.bits, tile_expert1, tile_row01, tile_rows1, n_row_tiles1,
                                         E, true, c->err, st)
                 : launch_grouped_qmm_tc(h, nullptr, n, dn, 1, cfg.bits, tile_expert, tile_row0, tile_rows, n_row_tiles, E,
                                         false, c->err, st))
      return 1;
    LAUNCHED(c, 1);
  } else {
    c->mark(6, st);
    dn.desc = expert_desc;  // (its source rows are the sorted positions themselves)
    if (launch_grouped_qmm_small(dn, 1, cfg.bits, max_active, n, st)) return 1;
    LAUNCHED(c, 1);
  }
  c->mark(7, st);
  return 0;
}

static int check_params(const b200_moe_params* p, bool need_router) {
  B200_REQUIRE(p != nullptr, "params is null");
  B200_REQUIRE(!need_router || p->router_weight, "router_weight is null");
  B200_REQUIRE(p->gate_proj.weight && p->gate_proj.scales && p->gate_proj.biases, "gate_proj is incomplete");
  B200_REQUIRE(p->up_proj.weight && p->up_proj.scales && p->up_proj.biases, "up_proj is incomplete");
  B200_REQUIRE(p->down_proj.weight && p->down_proj.scales && p->down_proj.biases, "down_proj is incomplete");
  return 0;
}

int b200_switch_glu_forward(b200_ctx* c, const b200_moe_config* cfg, const b200_moe_params* params, const void* x,
                            const uint32_t* indices, int64_t T, void* out, void* stream) {
  CTX_ENTER(c);
  if (check_cfg(cfg) || check_params(params, false)) return 1;
  B200_REQUIRE(T >= 0 && T * cfg->top_k < (int64_t(1) << 31), "bad token count");
  if (T == 0) return 0;
  B200_REQUIRE(x && indices && out, "null tensor");
  if (ctx_grow(c, block_scratch_bytes(*cfg, T), stream)) return 1;
  return experts_forward(c, *cfg, *params, x, indices, nullptr, T, out, nullptr, static_cast<cudaStream_t>(stream));
}

// The pre-norm in front of a block (mlx-lm/src/models/qwen3.rs:310-325: h + mlp(post_attention_layernorm(h))):
// hs = x (+ residual), the block runs on rms_norm(hs, weight, eps).
struct BlockPreNorm {
  const void* residual;  // optional
  const void* weight;    // optional
  float eps;
  void* sum_out;         // optional: x + residual
};

static int block_forward_impl(b200_ctx* c, const b200_moe_config* cfg, const b200_moe_params* params, const void* x,
                              const BlockPreNorm* pre, int64_t T, void* out, const b200_moe_aux* aux, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ctx_grow(c, block_scratch_bytes(*cfg, T), stream)) return 1;
  const int64_t n = T * cfg->top_k;
  const bool fused_small = router_fused_small_ok((int)T, cfg->hidden, cfg->n_experts, cfg->top_k);
  if (pre) {
    // (Folding the norm into the small-batch routing kernel was measured on a 24-layer stack at one token: 38.0 us
    // per layer against 34.3-36.1 with the separate launch - the routing kernel stages its weight rows before its
    // dependency wait, i.e. UNDER the norm kernel, and that overlap is worth more than the launch.)
    void* normed = c->take(sizeof(uint16_t) * T * cfg->hidden);
    B200_REQUIRE(normed, "scratch arena too small");
    if (launch_rms_norm(x, pre->residual, pre->weight, pre->eps, T, cfg->hidden, normed, pre->sum_out, st)) return 1;
    LAUNCHED(c, 1);
    x = normed;
  }
  const void* x_experts = x;
  void* logits = c->take(sizeof(uint16_t) * T * cfg->n_experts);
  uint32_t* idx = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
  void* scores = c->take(sizeof(uint16_t) * n);
  void* yk = c->take(sizeof(float) * n * cfg->hidden);
  B200_REQUIRE(logits && idx && scores && yk, "scratch arena too small");
  if (aux) {
    if (aux->logits) logits = aux->logits;
    if (aux->indices) idx = aux->indices;
    if (aux->scores) scores = aux->scores;
  }
  c->mark(0, st);
  int yk_fmt = kOutF32;
  if (fused_small) {
    // small batch: logits, routing and the sort in one launch (stages 1 and 2 read as zero)
    SortBufs sb;
    if (take_sort_bufs(c, n, cfg->n_experts, aux, sb)) return 1;
    const int desc_entries = (int)(cfg->n_experts < n ? cfg->n_experts : n);
    uint32_t* desc = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * kExpertDescWords * (size_t)desc_entries));
    B200_REQUIRE(desc, "scratch arena too small");
    if (launch_router_fused_small(x, params->router_weight, params->router_logit_bias, logits, (int)T, cfg->hidden,
                                  cfg->n_experts, cfg->top_k, cfg->router_mode, cfg->norm_topk_prob, idx, scores, sb.perm,
                                  sb.inv, sb.counts, sb.offsets, sb.active, sb.n_active,
                                  reinterpret_cast<unsigned int*>(c->err + kTicketWord), c->err, desc, desc_entries, st))
      return 1;
    LAUNCHED(c, 1);
    c->mark(1, st);
    c->mark(2, st);
    const SmallTail tail{idx, sb.inv, out, aux ? aux->out_f32 : nullptr, T, desc};
    if (experts_sorted(c, *cfg, *params, x_experts, sb.perm, cfg->top_k, sb.counts, sb.offsets, sb.active, sb.n_active, n,
                       scores, yk, st, &yk_fmt, nullptr, nullptr, &tail))
      return 1;
  } else {
    double* w64 = static_cast<double*>(c->take(sizeof(double) * (size_t)cfg->n_experts * cfg->hidden));
    B200_REQUIRE(w64, "scratch arena too small");
    launch_router_logits(x, params->router_weight, params->router_logit_bias, logits, (int)T, cfg->hidden, cfg->n_experts,
                         w64, st);
    c->mark(1, st);
    if (route_topk_sort_ok((int)T, cfg->n_experts, cfg->top_k)) {
      // up to 1024 assignments: the routing kernel's last CTA also sorts them (stage 2 reads as zero)
      SortBufs sb;
      if (take_sort_bufs(c, n, cfg->n_experts, aux, sb)) return 1;
      if (launch_route_topk_sort(logits, (int)T, cfg->n_experts, cfg->top_k, cfg->router_mode, cfg->norm_topk_prob, idx, scores,
                                 sb.perm, sb.inv, sb.counts, sb.offsets, sb.active, sb.n_active,
                                 reinterpret_cast<unsigned int*>(c->err + kTicketWord), c->err, st))
        return 1;
      c->mark(2, st);
      LAUNCHED(c, 2);
      if (experts_sorted(c, *cfg, *params, x, sb.perm, cfg->top_k, sb.counts, sb.offsets, sb.active, sb.n_active, n, scores,
                         yk, st, &yk_fmt))
        return 1;
    } else {
      launch_route_topk(logits, (int)T, cfg->n_experts, cfg->top_k, cfg->router_mode, cfg->norm_topk_prob, idx, scores,
                        nullptr, st);
      c->mark(2, st);
      LAUNCHED(c, 2);
      if (experts_forward(c, *cfg, *params, x, idx, scores, T, yk, aux, st, &yk_fmt)) return 1;
    }
  }
  if (yk_fmt != kOutNone) {
    if (launch_combine(yk, yk_fmt, T, cfg->top_k, cfg->hidden, out, aux ? aux->out_f32 : nullptr, st)) return 1;
    LAUNCHED(c, 1);
  }
  c->mark(8, st);
  c->ev_valid = c->profiling;
  return 0;
}

int b200_moe_block_forward(b200_ctx* c, const b200_moe_config* cfg, const b200_moe_params* params, const void* x,
                           int64_t T, void* out, const b200_moe_aux* aux, void* stream) {
  CTX_ENTER(c);
  if (check_cfg(cfg) || check_params(params, true)) return 1;
  B200_REQUIRE(T >= 0 && T < (1 << 24) && T * cfg->top_k < (int64_t(1) << 31), "bad token count");
  if (T == 0) return 0;
  B200_REQUIRE(x && out, "null tensor");
  return block_forward_impl(c, cfg, params, x, nullptr, T, out, aux, stream);
}

int b200_moe_block_forward_prenorm(b200_ctx* c, const b200_moe_config* cfg, const b200_moe_params* params, const void* x,
                                   const void* residual, const void* norm_weight, float eps, int64_t T, void* sum_out,
                                   void* out, const b200_moe_aux* aux, void* stream) {
  CTX_ENTER(c);
  if (check_cfg(cfg) || check_params(params, true)) return 1;
  B200_REQUIRE(T >= 0 && T < (1 << 24) && T * cfg->top_k < (int64_t(1) << 31), "bad token count");
  B200_REQUIRE(eps >= 0.f, "eps is negative");
  if (T == 0) return 0;
  B200_REQUIRE(x && out, "null tensor");
  B200_REQUIRE(!sum_out || residual, "sum_out without a residual");
  const BlockPreNorm pre{residual, norm_weight, eps, sum_out};
  return block_forward_impl(c, cfg, params, x, &pre, T, out, aux, stream);
}

// ---- expert-parallel exchange over peer memory ----------------------------------------------------

int b200_switch_glu_sorted(b200_ctx* c, const b200_moe_config* cfg, const b200_moe_params* params, const void* rows,
                           const uint32_t* counts, int64_t n, void* out, void* stream) {
  CTX_ENTER(c);
  if (check_cfg(cfg) || check_params(params, false)) return 1;
  B200_REQUIRE(n >= 0 && n < (int64_t(1) << 31), "bad row count");
  if (n == 0) return 0;
  B200_REQUIRE(rows && counts && out, "null tensor");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  b200_moe_config one = *cfg;
  one.top_k = 1;  // n rows, one assignment each
  if (ctx_grow(c, block_scratch_bytes(one, n), stream)) return 1;
  const int E = cfg->n_experts;
  uint32_t* offsets = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* active = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* n_active = static_cast<uint32_t*>(c->take(16));
  uint32_t* cnt = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  B200_REQUIRE(offsets && active && n_active && cnt, "scratch arena too small");
  launch_segments_from_counts(counts, E, n, cnt, offsets, active, n_active, c->err, st);
  LAUNCHED(c, 1);
  return experts_sorted(c, one, *params, rows, nullptr, 1, cnt, offsets, active, n_active, n, nullptr, out, st, nullptr);
}

static int fill_peers(EpPeers& pe, void* const* peers, int G);

int b200_switch_glu_sorted_scatter(b200_ctx* c, const b200_moe_config* cfg, const b200_moe_params* params, const void* rows,
                                   const uint32_t* counts, int64_t n, const unsigned long long* out_row_addr, void* stream) {
  CTX_ENTER(c);
  if (check_cfg(cfg) || check_params(params, false)) return 1;
  B200_REQUIRE(n >= 0 && n < (int64_t(1) << 31), "bad row count");
  if (n == 0) return 0;
  B200_REQUIRE(rows && counts && out_row_addr, "null tensor");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  b200_moe_config one = *cfg;
  one.top_k = 1;
  if (ctx_grow(c, block_scratch_bytes(one, n), stream)) return 1;
  const int E = cfg->n_experts;
  uint32_t* offsets = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* active = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  uint32_t* n_active = static_cast<uint32_t*>(c->take(16));
  uint32_t* cnt = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (E + 1)));
  B200_REQUIRE(offsets && active && n_active && cnt, "scratch arena too small");
  launch_segments_from_counts(counts, E, n, cnt, offsets, active, n_active, c->err, st);
  LAUNCHED(c, 1);
  return experts_sorted(c, one, *params, rows, nullptr, 1, cnt, offsets, active, n_active, n, nullptr, nullptr, st,
                        nullptr, out_row_addr);
}

int b200_ep_return_table(b200_ctx* c, const uint32_t* all_counts, int n_ranks, int n_experts, int rank, void* const* peer_y,
                         int64_t hidden, int64_t n_rows, int64_t capacity_rows, unsigned long long* row_addr, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(all_counts && row_addr, "null tensor");
  B200_REQUIRE(n_ranks >= 1 && n_ranks <= kEpMaxRanks && rank >= 0 && rank < n_ranks, "bad rank");
  B200_REQUIRE(n_experts > 0 && n_experts % n_ranks == 0, "experts must divide evenly over the ranks");
  B200_REQUIRE(hidden > 0 && hidden % 8 == 0, "hidden must be a multiple of 8");
  EpPeers pe;
  if (fill_peers(pe, peer_y, n_ranks)) return 1;
  B200_REQUIRE(n_rows >= 0 && capacity_rows >= 0, "bad row bounds");
  launch_ep_return_table(all_counts, n_ranks, n_experts, rank, pe, hidden, n_rows, capacity_rows, row_addr, c->err,
                         static_cast<cudaStream_t>(stream));
  LAUNCHED(c, 1);
  return 0;
}

int b200_ep_buffer_alloc(b200_ctx* c, size_t bytes, void** ptr, unsigned char* handle) {
  CTX_ENTER(c);
  B200_REQUIRE(ptr && handle && bytes > 0, "bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == B200_EP_HANDLE_BYTES, "handle size");
  void* p = nullptr;
  B200_CUDA(cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    B200_FAIL(std::string("cudaIpcGetMemHandle -> ") + cudaGetErrorString(e));
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return 0;
}

int b200_ep_buffer_open(b200_ctx* c, const unsigned char* handle, void** ptr) {
  CTX_ENTER(c);
  B200_REQUIRE(ptr && handle, "bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  B200_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}

int b200_ep_buffer_close(b200_ctx* c, void* ptr) {
  CTX_ENTER(c);
  if (ptr) B200_CUDA(cudaIpcCloseMemHandle(ptr));
  return 0;
}

int b200_ep_buffer_free(b200_ctx* c, void* ptr) {
  CTX_ENTER(c);
  if (ptr) {
    B200_CUDA(cudaDeviceSynchronize());
    B200_CUDA(cudaFree(ptr));
  }
  return 0;
}

static int fill_peers(EpPeers& pe, void* const* peers, int G) {
  B200_REQUIRE(peers != nullptr && G >= 1 && G <= kEpMaxRanks, "between 1 and 16 ranks");
  for (int i = 0; i < kEpMaxRanks; ++i) pe.p[i] = i < G ? peers[i] : nullptr;
  for (int i = 0; i < G; ++i) B200_REQUIRE(pe.p[i] != nullptr, "a peer buffer pointer is null");
  return 0;
}

int b200_ep_layout(b200_ctx* c, const uint32_t* all_counts, int n_ranks, int n_experts, int rank, uint32_t capacity_rows,
                   uint32_t* dst_row0, uint32_t* local_counts, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(all_counts && dst_row0 && local_counts, "null tensor");
  B200_REQUIRE(n_ranks >= 1 && n_ranks <= kEpMaxRanks && rank >= 0 && rank < n_ranks, "bad rank");
  B200_REQUIRE(n_experts > 0 && n_experts % n_ranks == 0, "experts must divide evenly over the ranks");
  launch_ep_layout(all_counts, n_ranks, n_experts, rank, capacity_rows, dst_row0, local_counts, c->err,
                   static_cast<cudaStream_t>(stream));
  LAUNCHED(c, 1);
  return 0;
}

int b200_ep_dispatch(b200_ctx* c, const void* x, const uint32_t* indices, const uint32_t* perm, const uint32_t* offsets,
                     const uint32_t* dst_row0, int64_t n, int top_k, int64_t hidden, int n_experts, int n_ranks, int rank,
                     void* const* peer_rows, uint32_t capacity_rows, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(n >= 0 && n < (int64_t(1) << 31) && top_k > 0, "bad row count");
  B200_REQUIRE(hidden > 0 && hidden % 8 == 0, "hidden must be a multiple of 8");
  B200_REQUIRE(n_experts > 0 && n_ranks > 0 && n_experts % n_ranks == 0, "experts must divide evenly over the ranks");
  B200_REQUIRE(rank >= 0 && rank < n_ranks, "bad rank");
  EpPeers pe;
  if (fill_peers(pe, peer_rows, n_ranks)) return 1;
  if (n == 0) return 0;
  B200_REQUIRE(x && indices && perm && offsets && dst_row0, "null tensor");
  launch_ep_dispatch(x, indices, perm, offsets, dst_row0, n, top_k, hidden, n_experts, n_ranks, rank, pe, capacity_rows, c->err,
                     static_cast<cudaStream_t>(stream));
  LAUNCHED(c, 1);
  return 0;
}

int b200_ep_combine(b200_ctx* c, void* const* peer_y, const uint32_t* indices, const uint32_t* inv_perm,
                    const uint32_t* offsets, const uint32_t* dst_row0, const void* scores, int64_t T, int top_k,
                    int64_t hidden, int n_experts, int n_ranks, uint32_t capacity_rows, void* out, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(T >= 0 && top_k > 0 && T * top_k < (int64_t(1) << 31), "bad token count");
  B200_REQUIRE(hidden > 0 && hidden % 8 == 0, "hidden must be a multiple of 8");
  B200_REQUIRE(n_experts > 0 && n_ranks > 0 && n_experts % n_ranks == 0, "experts must divide evenly over the ranks");
  EpPeers pe;
  if (fill_peers(pe, peer_y, n_ranks)) return 1;
  if (T == 0) return 0;
  B200_REQUIRE(indices && inv_perm && offsets && dst_row0 && scores && out, "null tensor");
  if (launch_ep_combine(pe, indices, inv_perm, offsets, dst_row0, scores, T, top_k, hidden, n_experts, n_ranks,
                        capacity_rows, out, c->err, static_cast<cudaStream_t>(stream)))
    return 1;
  LAUNCHED(c, 1);
  return 0;
}

// ---- one-call expert-parallel block with device-side phase ordering ------------------------------------------
constexpr int kEpChunks = 2;  // exchange sets per communicator: a step may run as two half-steps that overlap
struct b200_ep_comm {
  EpExchange x{};               // shape; peer pointers and device words of exchange set 0
  EpExchange xc[kEpChunks];     // the exchange sets: every peer-mapped buffer holds kEpChunks equal parts
  size_t part_bytes[kEpBufs] = {};
  void* own[kEpBufs] = {};      // this rank's six peer-mapped buffers
  void* peer_base[kEpBufs][kEpMaxRanks] = {};
  bool opened[kEpBufs][kEpMaxRanks] = {};
  void* y = nullptr;            // this rank's expert outputs by assignment row (local only; the half-steps use it in turn)
  uint32_t* dev = nullptr;      // backing store of the device words
  bool connected = false;
  int chunks = 1;               // half-steps per step (b200_ep_comm_set_chunks)
  cudaStream_t side = nullptr;  // exchange kernels of one half-step run here under the other half-step's products
  cudaEvent_t ev_fork = nullptr, ev_a[kEpChunks] = {}, ev_b[kEpChunks] = {}, ev_join = nullptr;
};
static void ep_comm_views(b200_ep_comm* e) {
  for (int ch = 0; ch < kEpChunks; ++ch) {
    EpExchange& v = e->xc[ch];
    const EpExchange keep = v;
    v = e->x;
    v.dst_row0 = keep.dst_row0;
    v.local_counts = keep.local_counts;
    v.n_recv = keep.n_recv;
    v.tokbase = keep.tokbase;
    v.n_tok_recv = keep.n_tok_recv;
    v.ntok = keep.ntok;
    for (int i = 0; i < kEpBufs; ++i)
      for (int r = 0; r < e->x.G; ++r)
        v.peer[i][r] = e->peer_base[i][r] ? static_cast<unsigned char*>(e->peer_base[i][r]) + (size_t)ch * e->part_bytes[i] : nullptr;
  }
}

int b200_ep_comm_create(b200_ctx* c, int n_ranks, int rank, int n_experts, int top_k, int64_t hidden,
                        uint32_t capacity_rows, uint32_t capacity_tokens, b200_ep_comm** out, unsigned char* handles) {
  CTX_ENTER(c);
  B200_REQUIRE(out && handles, "null argument");
  B200_REQUIRE(n_ranks >= 1 && n_ranks <= kEpMaxRanks && rank >= 0 && rank < n_ranks, "bad rank");
  B200_REQUIRE(n_experts > 0 && n_experts <= 256 && n_experts % n_ranks == 0, "experts must divide evenly over the ranks");
  B200_REQUIRE(top_k > 0 && top_k <= 32, "top_k must be in 1..32");
  B200_REQUIRE(hidden > 0 && hidden % 8 == 0 && capacity_rows > 0 && capacity_tokens > 0, "bad buffer shape");
  b200_ep_comm* e = new b200_ep_comm();
  EpExchange& x = e->x;
  x.G = n_ranks;
  x.E = n_experts;
  x.rank = rank;
  x.k = top_k;
  x.H = hidden;
  x.cap_rows = capacity_rows;
  x.cap_tok = capacity_tokens;
  size_t bytes[kEpBufs];
  bytes[kEpTok] = (size_t)capacity_tokens * hidden * 2;
  bytes[kEpPart] = (size_t)capacity_tokens * hidden * 2;
  bytes[kEpRowMap] = sizeof(uint32_t) * (size_t)capacity_rows;
  bytes[kEpSlotRows] = sizeof(uint32_t) * (size_t)capacity_tokens * top_k;
  bytes[kEpSlotScores] = sizeof(uint16_t) * (size_t)capacity_tokens * top_k;
  bytes[kEpCtl] = ep_ctl_bytes(n_ranks, n_experts);
  const int Eg = n_experts / n_ranks;
  bool ok = true;
  for (int i = 0; i < kEpBufs && ok; ++i) {
    bytes[i] = al(bytes[i]);
    e->part_bytes[i] = bytes[i];
    ok = cudaMalloc(&e->own[i], kEpChunks * bytes[i]) == cudaSuccess;
    if (ok && i == kEpCtl) ok = cudaMemset(e->own[i], 0, kEpChunks * bytes[i]) == cudaSuccess;
    cudaIpcMemHandle_t h;
    if (ok) ok = cudaIpcGetMemHandle(&h, e->own[i]) == cudaSuccess;
    if (ok) memcpy(handles + (size_t)i * B200_EP_HANDLE_BYTES, &h, sizeof(h));
  }
  if (ok) ok = cudaMalloc(&e->y, (size_t)capacity_rows * hidden * 2) == cudaSuccess;
  const size_t words = (size_t)n_experts + Eg + 1 + n_ranks + 1 + n_ranks + 8;
  if (ok) ok = cudaMalloc(reinterpret_cast<void**>(&e->dev), sizeof(uint32_t) * words * kEpChunks) == cudaSuccess;
  if (ok) ok = cudaMemset(e->dev, 0, sizeof(uint32_t) * words * kEpChunks) == cudaSuccess;
  int prio_lo = 0, prio_hi = 0;
  if (ok) ok = cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi) == cudaSuccess;
  if (ok) ok = cudaStreamCreateWithPriority(&e->side, cudaStreamNonBlocking, prio_hi) == cudaSuccess;
  cudaEvent_t* evs[] = {&e->ev_fork, &e->ev_a[0], &e->ev_a[1], &e->ev_b[0], &e->ev_b[1], &e->ev_join};
  for (cudaEvent_t* ev : evs)
    if (ok) ok = cudaEventCreateWithFlags(ev, cudaEventDisableTiming) == cudaSuccess;
  if (ok) ok = cudaDeviceSynchronize() == cudaSuccess;
  if (!ok) {
    const std::string why = cudaGetErrorString(cudaGetLastError());
    for (void* p : e->own)
      if (p) cudaFree(p);
    if (e->y) cudaFree(e->y);
    if (e->dev) cudaFree(e->dev);
    if (e->side) cudaStreamDestroy(e->side);
    for (cudaEvent_t* ev : evs)
      if (*ev) cudaEventDestroy(*ev);
    delete e;
    B200_FAIL("cannot allocate the exchange buffers: " + why);
  }
  for (int ch = 0; ch < kEpChunks; ++ch) {
    EpExchange& v = e->xc[ch];
    v.dst_row0 = e->dev + (size_t)ch * words;
    v.local_counts = v.dst_row0 + n_experts;
    v.n_recv = v.local_counts + Eg;
    v.tokbase = v.n_recv + 1;
    v.n_tok_recv = v.tokbase + n_ranks;
    v.ntok = v.n_tok_recv + 1;
  }
  for (int i = 0; i < kEpBufs; ++i) e->peer_base[i][rank] = e->own[i];
  ep_comm_views(e);
  *out = e;
  return 0;
}

int b200_ep_comm_set_chunks(b200_ctx* c, b200_ep_comm* e, int chunks) {
  CTX_ENTER(c);
  B200_REQUIRE(e != nullptr, "null communicator");
  B200_REQUIRE(chunks >= 1 && chunks <= kEpChunks, "chunks must be 1 or 2");
  e->chunks = chunks;
  return 0;
}

int b200_ep_comm_connect(b200_ctx* c, b200_ep_comm* e, const unsigned char* all_handles) {
  CTX_ENTER(c);
  B200_REQUIRE(e && all_handles, "null argument");
  B200_REQUIRE(!e->connected, "already connected");
  for (int r = 0; r < e->x.G; ++r) {
    if (r == e->x.rank) continue;
    for (int i = 0; i < kEpBufs; ++i) {
      cudaIpcMemHandle_t h;
      memcpy(&h, all_handles + ((size_t)r * kEpBufs + i) * B200_EP_HANDLE_BYTES, sizeof(h));
      B200_CUDA(cudaIpcOpenMemHandle(&e->peer_base[i][r], h, cudaIpcMemLazyEnablePeerAccess));
      e->opened[i][r] = true;
    }
  }
  ep_comm_views(e);
  e->connected = true;
  return 0;
}

int b200_ep_comm_destroy(b200_ctx* c, b200_ep_comm* e) {
  if (!e) return 0;
  CTX_ENTER(c);
  cudaDeviceSynchronize();
  for (int i = 0; i < kEpBufs; ++i)
    for (int r = 0; r < e->x.G; ++r)
      if (e->opened[i][r]) cudaIpcCloseMemHandle(e->peer_base[i][r]);
  for (void* p : e->own)
    if (p) cudaFree(p);
  if (e->y) cudaFree(e->y);
  if (e->dev) cudaFree(e->dev);
  if (e->side) cudaStreamDestroy(e->side);
  for (cudaEvent_t ev : {e->ev_fork, e->ev_a[0], e->ev_a[1], e->ev_b[0], e->ev_b[1], e->ev_join})
    if (ev) cudaEventDestroy(ev);
  delete e;
  return 0;
}

int b200_moe_block_forward_ep(b200_ctx* c, b200_ep_comm* e, const b200_moe_config* cfg, const b200_moe_params* params,
                              const void* x, int64_t T, void* out, const b200_moe_aux* aux, void* stream) {
  CTX_ENTER(c);
  B200_REQUIRE(e != nullptr && (e->connected || e->x.G == 1), "the communicator is not connected");
  if (check_cfg(cfg) || check_params(params, true)) return 1;
  const int G = e->x.G, E = cfg->n_experts, Eg = E / G, k = cfg->top_k;
  B200_REQUIRE(E == e->x.E && cfg->hidden == e->x.H && k == e->x.k, "the communicator was created for another layer shape");
  B200_REQUIRE(T >= 0 && T < (1 << 24) && T * k < (int64_t(1) << 31), "bad token count");
  B200_REQUIRE(T == 0 || (x && out), "null tensor");
  const int nch = e->chunks;
  B200_REQUIRE(nch == 1 || !aux || (!aux->perm && !aux->inv_perm && !aux->offsets),
               "perm, inv_perm and offsets of the whole step do not exist when the step runs as two half-steps");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // every rank takes part in every step, also with no tokens of its own (its experts may still receive rows)
  const int64_t n = T * k, cap = e->x.cap_rows;
  b200_moe_config local = *cfg;  // the experts this rank owns, one assignment per arriving row
  local.n_experts = Eg;
  local.top_k = 1;
  const size_t route_bytes = al(sizeof(uint16_t) * T * E) + al(sizeof(double) * (size_t)E * cfg->hidden) +
                             al(sizeof(uint32_t) * n) * 3 + al(sizeof(uint16_t) * n) +
                             (al(sizeof(uint32_t) * (E + 1)) * 4 + al(16)) * (kEpChunks + 1) +
                             al(sizeof(uint32_t) * permute_scratch_words(n, E)) * kEpChunks + al(sizeof(uint32_t) * (size_t)G * T) * 2 +
                             al(sizeof(uint16_t) * (size_t)e->x.cap_tok * cfg->hidden) + al(sizeof(float) * e->x.cap_tok) + 8192;
  if (ctx_grow(c, route_bytes + block_scratch_bytes(local, cap), stream)) return 1;
  void* logits = c->take(sizeof(uint16_t) * T * E);
  uint32_t* idx = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * n));
  void* scores = c->take(sizeof(uint16_t) * n);
  double* w64 = static_cast<double*>(c->take(sizeof(double) * (size_t)E * cfg->hidden));
  B200_REQUIRE(logits && idx && scores && w64, "scratch arena too small");
  if (aux) {
    if (aux->logits) logits = aux->logits;
    if (aux->indices) idx = aux->indices;
    if (aux->scores) scores = aux->scores;
  }
  // 1. route this rank's tokens
  if (T > 0) {
    launch_router_logits(x, params->router_weight, params->router_logit_bias, logits, (int)T, cfg->hidden, E, w64, st);
    launch_route_topk(logits, (int)T, E, k, cfg->router_mode, cfg->norm_topk_prob, idx, scores, nullptr, st);
    LAUNCHED(c, 2);
  }
  // The step runs as nch half-steps over consecutive halves of the tokens, each a complete exchange on its own set of
  // buffers and control words.  With two, the exchange kernels (small enough to share an SM with the persistent
  // tensor-core CTAs) go to the communicator's side stream: the dispatch of the second half and the return of the
  // first run under the other half's expert products.
  struct Half {
    int64_t t0, Tc;
    SortBufs sb;
    uint32_t* slot;
  } half[kEpChunks];
  for (int ch = 0; ch < nch; ++ch) {
    Half& h = half[ch];
    h.t0 = ch == 0 ? 0 : half[0].Tc;
    h.Tc = nch == 1 ? T : (ch == 0 ? (T + 1) / 2 : T - (T + 1) / 2);
    const int64_t nc = h.Tc * k;
    if (take_sort_bufs(c, nc, E, nch == 1 ? aux : nullptr, h.sb)) return 1;
    h.slot = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (size_t)G * (h.Tc > 0 ? h.Tc : 1)));
    B200_REQUIRE(h.slot, "scratch arena too small");
    // sort of the half's assignments; which of its tokens goes to which rank
    launch_permute(idx + h.t0 * k, nc, E, h.sb.perm, h.sb.inv, h.sb.counts, h.sb.offsets, h.sb.active, h.sb.n_active, h.sb.chunk,
                   c->err, st);
    launch_ep_token_slots(idx + h.t0 * k, h.Tc, e->xc[ch], h.slot, st);
    LAUNCHED(c, permute_launches(nc) + 1);
  }
  if (nch == 2 && aux && aux->counts) {
    launch_add_u32(half[0].sb.counts, half[1].sb.counts, E, aux->counts, st);
    LAUNCHED(c, 1);
  }
  const unsigned char* xb = static_cast<const unsigned char*>(x);
  unsigned char* ob = static_cast<unsigned char*>(out);
  const size_t row_bytes = (size_t)cfg->hidden * 2;
  // 2.-3. all-gather of the counts through the control blocks, layout of the exchange; dispatch: every token once per
  //       destination rank, plus the owners' bookkeeping; "my rows have landed" to every peer, wait for all peers
  auto exchange_out = [&](int ch, cudaStream_t s_) {
    const Half& h = half[ch];
    launch_ep_counts_exchange(e->xc[ch], h.sb.counts, c->err, s_);
    launch_ep_dispatch_dedup(xb + h.t0 * row_bytes, idx + h.t0 * k, h.sb.inv, h.sb.offsets,
                             static_cast<const unsigned char*>(scores) + h.t0 * k * 2, h.slot, h.Tc, e->xc[ch], c->err, s_);
    launch_ep_signal_wait(e->xc[ch], 1, c->err, s_);
    LAUNCHED(c, 2 + (h.Tc ? 1 : 0));
  };
  // 4. this rank's experts on the assignments that arrived (their number lives on the device: the launches are sized
  //    for the buffers' capacity and follow the device-side segment tables), then the partial weighted sums
  const size_t scratch_mark = c->ws_used;
  auto experts = [&](int ch, cudaStream_t s_) -> int {
    c->ws_used = scratch_mark;  // the half-steps' products run one after the other on the same stream: same scratch
    const EpExchange& ex = e->xc[ch];
    uint32_t* offsets = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (Eg + 1)));
    uint32_t* active = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (Eg + 1)));
    uint32_t* n_active = static_cast<uint32_t*>(c->take(16));
    uint32_t* cnt = static_cast<uint32_t*>(c->take(sizeof(uint32_t) * (Eg + 1)));
    B200_REQUIRE(offsets && active && n_active && cnt, "scratch arena too small");
    launch_segments_from_counts(ex.local_counts, Eg, cap, cnt, offsets, active, n_active, c->err, s_);
    LAUNCHED(c, 1);
    ExchangeRows xr{static_cast<const uint32_t*>(ex.peer[kEpRowMap][ex.rank]), (int64_t)ex.cap_tok, ex.n_tok_recv, ex.n_recv};
    int y_fmt = kOutBf16;
    if (experts_sorted(c, local, *params, ex.peer[kEpTok][ex.rank], nullptr, 1, cnt, offsets, active, n_active, cap, nullptr, e->y,
                       s_, &y_fmt, nullptr, &xr))
      return 1;
    if (launch_ep_partial_combine(e->y, y_fmt == kOutF16, ex, c->err, s_)) return 1;
    LAUNCHED(c, 1);
    return 0;
  };
  // 5. "my partial sums are complete" to every peer, wait for all peers; combine: each token sums the partial sums of
  //    the ranks that own its experts
  auto exchange_back = [&](int ch, cudaStream_t s_) {
    const Half& h = half[ch];
    launch_ep_signal_wait(e->xc[ch], 2, c->err, s_);
    launch_ep_final_combine(h.slot, h.Tc, e->xc[ch], ob + h.t0 * row_bytes, s_);
    LAUNCHED(c, 1 + (h.Tc ? 1 : 0));
  };
  if (nch == 1) {
    exchange_out(0, st);
    if (experts(0, st)) return 1;
    exchange_back(0, st);
    return 0;
  }
  cudaStream_t side = e->side;
  B200_CUDA(cudaEventRecord(e->ev_fork, st));
  B200_CUDA(cudaStreamWaitEvent(side, e->ev_fork, 0));
  exchange_out(0, side);
  B200_CUDA(cudaEventRecord(e->ev_a[0], side));
  exchange_out(1, side);  // under the first half's products
  B200_CUDA(cudaEventRecord(e->ev_a[1], side));
  B200_CUDA(cudaStreamWaitEvent(st, e->ev_a[0], 0));
  if (experts(0, st)) return 1;
  B200_CUDA(cudaEventRecord(e->ev_b[0], st));
  B200_CUDA(cudaStreamWaitEvent(side, e->ev_b[0], 0));
  exchange_back(0, side);  // under the second half's products
  B200_CUDA(cudaStreamWaitEvent(st, e->ev_a[1], 0));
  if (experts(1, st)) return 1;
  B200_CUDA(cudaEventRecord(e->ev_b[1], st));
  B200_CUDA(cudaStreamWaitEvent(side, e->ev_b[1], 0));
  exchange_back(1, side);
  B200_CUDA(cudaEventRecord(e->ev_join, side));
  B200_CUDA(cudaStreamWaitEvent(st, e->ev_join, 0));
  return 0;
}

}  // extern "C"

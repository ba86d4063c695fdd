// Shared device/host helpers for the quantized mixture-of-experts kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace b200 {

// ---- error plumbing (status int + thread-local message, like the reference's
// mlx_set_error_handler convention: mlx-rs/src/error.rs:226-280) --------------------------
void set_error(const std::string& msg);
#define B200_FAIL(msg)                                   \
  do {                                                   \
    ::b200::set_error(std::string(__func__) + ": " + (msg)); \
    return 1;                                            \
  } while (0)
#define B200_REQUIRE(cond, msg) \
  do {                          \
    if (!(cond)) B200_FAIL(msg); \
  } while (0)
#define B200_CUDA(expr)                                                      \
  do {                                                                       \
    cudaError_t _e = (expr);                                                 \
    if (_e != cudaSuccess) B200_FAIL(std::string(#expr) + " -> " + cudaGetErrorString(_e)); \
  } while (0)

static inline int cdiv(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

// ---- bf16 bit helpers ------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f)));
}

// float64 -> bf16 with a single round-to-nearest-even: squeeze to float32 with round-to-odd
// (truncate, OR a sticky bit when inexact), then round that to bf16.
__device__ __forceinline__ uint32_t f64_to_bf16_bits(double d) {
  float f = __double2float_rz(d);
  uint32_t u = __float_as_uint(f);
  if (static_cast<double>(f) != d && (u & 0x7f800000u) != 0x7f800000u) u |= 1u;
  return f32_to_bf16_bits(__uint_as_float(u));
}

// exact bf16 -> float64 (normal numbers by integer re-biasing; zero/subnormal/inf/nan by cvt)
__device__ __forceinline__ double bf16_bits_to_f64(uint32_t b) {
  uint32_t ex = b & 0x7f80u;
  if (ex != 0u && ex != 0x7f80u) {
    uint32_t f = b << 16;
    uint32_t hi = (f & 0x80000000u) | (((f & 0x7fffffffu) >> 3) + (896u << 20));
    return __hiloint2double(static_cast<int>(hi), 0);
  }
  return static_cast<double>(bf16_bits_to_f32(b));
}

// ---- programmatic dependent launch ---------------------------------------------------------
// The kernels of the small-batch path are a chain of short launches.  Each of them begins with
// pdl_prologue(): it lets the NEXT kernel of the stream start launching at once (its blocks become
// resident and then sit in their own pdl_prologue) and waits until the PREVIOUS kernel has
// completed and its writes are visible.  Because every kernel of the chain waits before it touches
// memory, the order of all reads and writes is the stream order; only launch latency overlaps.
// launch_pdl() is the matching launch; a kernel launched with it MUST start with pdl_prologue().
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// The two halves of pdl_prologue() for kernels that fetch CONSTANT inputs (weights, which no kernel of the chain
// writes) between them: those fetches then run while the previous kernel is still finishing.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#ifdef B200_DEV
bool pdl_enabled();  // development build: false when the environment variable B200_NO_PDL is set
#else
inline bool pdl_enabled() { return true; }
#endif

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// One row of residual add + RMSNorm by a block of 256 threads (all of them call it): s = bf16(x + residual) where a
// residual is given (written to sum_out when asked for), out = bf16(w * s * rsqrt(mean(s^2) + eps)).  `part` is
// shared scratch of 8 floats.  The reduction order is fixed, so every caller gets the same bits.
__device__ __forceinline__ void block_rms_norm_row(const __nv_bfloat16* __restrict__ xr, const __nv_bfloat16* __restrict__ res,
                                                   const __nv_bfloat16* __restrict__ weight, float eps, int64_t cols,
                                                   __nv_bfloat16* out, __nv_bfloat16* sum_out, float* part) {
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += 256) {
    float v = __bfloat162float(xr[c]);
    if (res) {
      __nv_bfloat16 s = __float2bfloat16_rn(v + __bfloat162float(res[c]));
      if (sum_out) sum_out[c] = s;
      v = __bfloat162float(s);
    }
    ss += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __syncthreads();  // (part may still be read by a previous call)
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += part[i];
  const float inv = rsqrtf(tot / (float)cols + eps);
  for (int64_t c = threadIdx.x; c < cols; c += 256) {
    float v = __bfloat162float(xr[c]);
    if (res) v = __bfloat162float(__float2bfloat16_rn(v + __bfloat162float(res[c])));
    const float wv = weight ? __bfloat162float(weight[c]) : 1.0f;
    out[c] = __float2bfloat16_rn(wv * (v * inv));
  }
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the CURRENT device only, and one process
// may hold contexts on several devices: remember, per kernel instantiation and device, the largest size
// that has been set.  One cache object per kernel (a function-local static at the launch site).
constexpr int kMaxDevices = 64;
struct DynSmemCache {
  size_t bytes[kMaxDevices] = {};
};
template <typename Kern>
inline cudaError_t ensure_dyn_smem(Kern kern, size_t bytes, DynSmemCache& cache) {
  if (bytes <= 16 * 1024) return cudaSuccess;  // static + dynamic stay below the 48 KB every kernel may use (static <= 32 KB here)
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool cached = dev >= 0 && dev < kMaxDevices;
  if (cached && bytes <= cache.bytes[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && cached) cache.bytes[dev] = bytes;
  return e;
}
// Number of SMs of the current device (cached per device).
inline int current_sm_count() {
  static int n_sm[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 0 || dev >= kMaxDevices) {
    int n = 148;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }
  if (!n_sm[dev]) cudaDeviceGetAttribute(&n_sm[dev], cudaDevAttrMultiProcessorCount, dev);
  return n_sm[dev] > 0 ? n_sm[dev] : 148;
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

}  // namespace b200

// Shared declarations of the kernel library: dtype codes, status codes, the last-error
// string, and small device helpers.  Every entry point is `extern "C"`, takes raw device
// pointers and a stream, validates its arguments on the host before any launch and returns a
// status; nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "sonicboom_b200.h"      // the public types and every entry point's declaration

// Rows of a fused gate/up matrix alternate in blocks of this many: 8 gate rows, then the 8 up
// rows of the same outputs.  Every GEMM kernel's SwiGLU epilogue pairs column c with c + 8.
#define SB_SWIGLU_BLOCK 8

void sb_set_error(const char* fmt, ...);

#define SB_FAIL(code, ...)        \
  do {                            \
    sb_set_error(__VA_ARGS__);    \
    return (code);                \
  } while (0)

#define SB_CHECK_LAUNCH(name)                                                      \
  do {                                                                             \
    cudaError_t e__ = cudaGetLastError();                                          \
    if (e__ != cudaSuccess)                                                        \
      SB_FAIL(SB_ERR_CUDA, "%s: launch failed: %s", name, cudaGetErrorString(e__)); \
  } while (0)

template <typename T>
__device__ __forceinline__ float sb_to_f32(T v);
template <>
__device__ __forceinline__ float sb_to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float sb_to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T>
__device__ __forceinline__ T sb_from_f32(float v);
template <>
__device__ __forceinline__ float sb_from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 sb_from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// x / (1 + exp(-x)) with the accurate expf, as the reference's silu
// (core/src/nn/activation.cpp:41-50, core/src/nn/cuda_elementwise.cu:203-212).
__device__ __forceinline__ float sb_silu(float x) { return x / (1.0f + expf(-x)); }

// The rotation of one pair (a at index i, b at i + rot/2): lo = a cos - b sin, hi = a sin + b cos,
// every product and the sum rounded on its own (no fused multiply-add), so that every kernel
// that rotates gives the same bits whatever the compiler would contract.
__device__ __forceinline__ float sb_rot_lo(float a, float b, float c, float s) {
  return __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
}
__device__ __forceinline__ float sb_rot_hi(float a, float b, float c, float s) {
  return __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
}

__device__ __forceinline__ float sb_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float sb_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Programmatic dependent launch (optional, see sb_pdl_enabled): a kernel launched this way may
// start while its predecessor in the stream is still running.  A kernel calls sb_pdl_wait()
// before it first touches anything a predecessor wrote; what it does before the wait (barrier
// set-up, requesting weights) overlaps the predecessor's tail.  It calls sb_pdl_launch() where
// its successor may be scheduled: small kernels at their start, the products and the attention
// once their own operands have been requested, so that a successor does not take resources the
// kernel still wants.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void sb_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void sb_pdl_launch() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

// Asks for memory that a later kernel will stream (weights) to be brought into L2: a kernel
// calls this once its own loads have landed, where the rest of it (a merge) leaves the memory
// system idle and the next kernel's blocks cannot start yet.  (The tcgen05 products need no such
// hint from the kernel before them: launched early, they request their first tiles themselves.)  Block `bid` of `n_blocks` asks for its share; `ptr` is 16-byte
// aligned and `bytes` a multiple of 16.  A hint only: nothing waits for it.
constexpr uint32_t SB_WARM_CHUNK = 16384;
constexpr size_t SB_WARM_MAX = (size_t)32 << 20;
__device__ __forceinline__ void sb_warm_l2(const char* ptr, size_t bytes, size_t bid, size_t n_blocks) {
  for (size_t off = bid * SB_WARM_CHUNK; off < bytes; off += n_blocks * SB_WARM_CHUNK) {
    const uint32_t n = (uint32_t)(bytes - off < SB_WARM_CHUNK ? bytes - off : SB_WARM_CHUNK);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(ptr + off), "r"(n) : "memory");
  }
}
// The bytes of a hint as the kernels take them: nothing for an unaligned pointer, at most
// SB_WARM_MAX (what the idle stretch of a decode kernel can bring in), a multiple of 16.
static inline size_t sb_warm_bytes(const void* ptr, size_t bytes) {
  if (!ptr || ((uintptr_t)ptr & 15)) return 0;
  return (bytes < SB_WARM_MAX ? bytes : SB_WARM_MAX) & ~(size_t)15;
}


template <int CLS = SB_K_OTHER, typename... Exp, typename... Act>
inline cudaError_t sb_launch(void (*kernel)(Exp...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Act&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (sb_pdl_enabled() & CLS) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Exp>(args)...);
}

// Dispatch helpers: run `BODY` with `T` bound to the C++ type of a dtype code.
#define SB_DISPATCH_DTYPE(code, T, ...)                           \
  do {                                                            \
    if ((code) == SB_F32) {                                       \
      using T = float;                                            \
      __VA_ARGS__                                                 \
    } else {                                                      \
      using T = __nv_bfloat16;                                    \
      __VA_ARGS__                                                 \
    }                                                             \
  } while (0)

static inline bool sb_valid_dtype(int d) { return d == SB_F32 || d == SB_BF16; }

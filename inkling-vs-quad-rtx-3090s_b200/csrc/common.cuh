// Shared device helpers for the NVFP4 routed-expert kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "these kernels are written for sm_100a"
#endif

namespace ink {

// ---------------------------------------------------------------- error plumbing
void set_error(const char* fmt, ...);  // host side; message returned by ink_last_error()

enum Status : int {
  kOk = 0,
  kBadArgument = -1,
  kUnsupportedShape = -2,
  kLaunchFailed = -3,
  kMisaligned = -4,
};

// bits of the optional device status word the kernels OR into
enum DeviceFlag : int {
  kFlagExpertOutOfRange = 1,   // a route named an expert < 0 or > max_expert
  kFlagWaitTimedOut = 2,       // a bounded wait gave up
};

#define INK_REQUIRE(cond, code, ...)          \
  do {                                        \
    if (!(cond)) {                            \
      ink::set_error(__VA_ARGS__);            \
      return (code);                          \
    }                                         \
  } while (0)

#define INK_CHECK_LAUNCH(what)                                              \
  do {                                                                      \
    cudaError_t e_ = cudaGetLastError();                                    \
    if (e_ != cudaSuccess) {                                                \
      ink::set_error("%s: launch failed: %s", what, cudaGetErrorString(e_)); \
      return ink::kLaunchFailed;                                            \
    }                                                                       \
  } while (0)

// Every kernel of the library asks for the largest shared-memory carve-out, so that the
// SMs are not re-partitioned between L1 and shared memory from one launch to the next
// (the streaming kernels need almost all of it).
#define INK_PREFER_MAX_SMEM(kernel)                                                             \
  do {                                                                                          \
    static bool done_ = false;                                                                  \
    if (!done_) {                                                                               \
      cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,              \
                           (int)cudaSharedmemCarveoutMaxShared);                                \
      done_ = true;                                                                             \
    }                                                                                           \
  } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------- BF16 <-> FP32
__device__ __forceinline__ float bf16_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }
__device__ __forceinline__ float bf16lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

// round to nearest even: what a cast to BF16 does (one instruction; a NaN becomes the canonical BF16 NaN)
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
  uint16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float round_bf16(float v) { return bf16_to_f32(f32_to_bf16_bits(v)); }

// ------------------------------------------------------------------ packed converts
// four bytes of E2M1 codes (8 weights, low nibble first) -> four f16x2 registers
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n"
      " .reg .b8 b0, b1, b2, b3;\n"
      " mov.b32 {b0, b1, b2, b3}, %4;\n"
      " cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      " cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      " cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      " cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
// two E4M3 bytes -> f16x2 (exact: every E4M3 value is an FP16 value)
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t s) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(s));
  return r;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ float f16lo_to_f32(uint32_t h2) {
  float f;
  asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.f32.f16 %0, lo; }" : "=f"(f) : "r"(h2));
  return f;
}
__device__ __forceinline__ float f16hi_to_f32(uint32_t h2) {
  float f;
  asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.f32.f16 %0, hi; }" : "=f"(f) : "r"(h2));
  return f;
}
__device__ __forceinline__ uint32_t f32x2_to_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// ------------------------------------------------------------------------- loads
// streaming 128-bit load: weights are read once, keep them out of L1
__device__ __forceinline__ uint4 ldg_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.f + __expf(-gate)) * up; }

// power-of-two normalisation of a BF16 vector so that its largest magnitude lies in
// [1, 2): `amax_bits` is max(bits & 0x7fff). Returns the FP32 multiplier 2^-e; the
// inverse 2^e is returned through `inverse`.
__device__ __forceinline__ float pow2_normaliser(uint32_t amax_bits, float* inverse) {
  int field = (int)((amax_bits >> 7) & 0xffu);
  field = field < 1 ? 127 : (field > 253 ? 253 : (field < 16 ? 16 : field));   // the multiplier stays below 2^112: callers scale it further
  if (amax_bits == 0) field = 127;
  *inverse = __uint_as_float((uint32_t)field << 23);
  return __uint_as_float((uint32_t)(254 - field) << 23);
}

}  // namespace ink

// Per-warp arithmetic shared by the streaming kernels: NVFP4 and BF16 dot products on
// shared-memory tiles, multi-row warp reductions, activation staging.
#pragma once
#include "common.cuh"

namespace ink {

// How the E2M1 codes become FP16: with the conversion instruction (cvt.rn.f16x2.e2m1x2, two
// codes each) or with integer logic. The logic path uses that a code's three magnitude bits,
// placed on an FP16's two low exponent bits and top mantissa bit, ARE the code's value times
// 2^-14 (the code's subnormal 0.5 lands on an FP16 subnormal), so a shift and a mask per field
// decode two codes at once; the staged activations carry the 2^14 back (see stage_pack8) and are
// permuted so that the codes j and j+4 of a word share a register with their activations.
// Measured on B200 in the one-launch kernel (4096 x 2048, one GPU, per block of the stack):
//   0: every word with the conversion instruction                      48.9 us
//   1: every word with logic (15 operations a word against 4)          56.7 us
//   2: words 0, 1 of a 16-byte group converted, words 2, 3 with logic  53.3 us
// The conversions run on the XU pipe and keep it busy for 3/4 of the kernel's time, yet moving work
// from it to the integer pipe only costs: the consumer warps hold a ring slot for as long as they
// compute on it, and every instruction more keeps bytes out of flight. The switch stays for parts
// where the balance differs.
#ifndef INK_E2M1_ON_ALU
#define INK_E2M1_ON_ALU 0
#endif

// whether word `word` (0..3) of a 16-byte group of codes is decoded with integer logic
__host__ __device__ constexpr bool e2m1_word_on_alu(int word) {
  return INK_E2M1_ON_ALU == 1 || (INK_E2M1_ON_ALU == 2 && (word & 2) != 0);
}

// eight codes of a word -> four f16x2: h[j] = (code j, code j + 4), each times 2^-14
__device__ __forceinline__ void e2m1x8_alu(uint32_t w, uint32_t (&h)[4]) {
  h[0] = ((w << 9) & 0x0E000E00u) | ((w << 12) & 0x80008000u);
  h[1] = ((w << 5) & 0x0E000E00u) | ((w << 8) & 0x80008000u);
  h[2] = ((w << 1) & 0x0E000E00u) | ((w << 4) & 0x80008000u);
  h[3] = ((w >> 3) & 0x0E000E00u) | (w & 0x80008000u);
}
template <bool ALU>
__device__ __forceinline__ void e2m1x8_decode(uint32_t w, uint32_t (&h)[4]) {
  if constexpr (ALU) e2m1x8_alu(w, h);
  else e2m1x8_to_f16x2(w, h);
}

// eight consecutive BF16 activations times `scale` -> eight FP16 in the order dot32 wants them for
// word `word` (0..3) of their group of 32
__device__ __forceinline__ uint4 stage_pack8(const uint4& v, float scale, int word) {
  uint4 h;
  if (e2m1_word_on_alu(word)) {
    const float s = scale * 16384.f;   // the decoded weights are 2^-14 too small
    h.x = f32x2_to_f16x2(bf16lo(v.x) * s, bf16lo(v.z) * s);   // (x0, x4)
    h.y = f32x2_to_f16x2(bf16hi(v.x) * s, bf16hi(v.z) * s);   // (x1, x5)
    h.z = f32x2_to_f16x2(bf16lo(v.y) * s, bf16lo(v.w) * s);   // (x2, x6)
    h.w = f32x2_to_f16x2(bf16hi(v.y) * s, bf16hi(v.w) * s);   // (x3, x7)
  } else {
    h.x = f32x2_to_f16x2(bf16lo(v.x) * scale, bf16hi(v.x) * scale);
    h.y = f32x2_to_f16x2(bf16lo(v.y) * scale, bf16hi(v.y) * scale);
    h.z = f32x2_to_f16x2(bf16lo(v.z) * scale, bf16hi(v.z) * scale);
    h.w = f32x2_to_f16x2(bf16lo(v.w) * scale, bf16hi(v.w) * scale);
  }
  return h;
}

// 32 weights x 32 FP16 activations (staged by stage_pack8) with their two block scales -> FP32
__device__ __forceinline__ float dot32(const uint4& q, uint32_t scale_pair, const uint32_t* x) {
  uint32_t h[4];
  uint32_t a0 = 0u, a1 = 0u;
  e2m1x8_decode<e2m1_word_on_alu(0)>(q.x, h);
  a0 = hfma2(h[0], x[0], a0); a0 = hfma2(h[1], x[1], a0); a0 = hfma2(h[2], x[2], a0); a0 = hfma2(h[3], x[3], a0);
  e2m1x8_decode<e2m1_word_on_alu(1)>(q.y, h);
  a0 = hfma2(h[0], x[4], a0); a0 = hfma2(h[1], x[5], a0); a0 = hfma2(h[2], x[6], a0); a0 = hfma2(h[3], x[7], a0);
  e2m1x8_decode<e2m1_word_on_alu(2)>(q.z, h);
  a1 = hfma2(h[0], x[8], a1); a1 = hfma2(h[1], x[9], a1); a1 = hfma2(h[2], x[10], a1); a1 = hfma2(h[3], x[11], a1);
  e2m1x8_decode<e2m1_word_on_alu(3)>(q.w, h);
  a1 = hfma2(h[0], x[12], a1); a1 = hfma2(h[1], x[13], a1); a1 = hfma2(h[2], x[14], a1); a1 = hfma2(h[3], x[15], a1);
  // The two block sums are added in FP16 (b = (a0.lo + a0.hi, a1.lo + a1.hi)) and multiplied by their
  // E4M3 scales with FP32-accumulating mixed-precision FMAs.
  const uint32_t s = e4m3x2_to_f16x2((uint16_t)scale_pair);
  const uint32_t lows = __byte_perm(a0, a1, 0x5410), highs = __byte_perm(a0, a1, 0x7632);
  uint32_t b;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(b) : "r"(lows), "r"(highs));
  float acc = 0.f;
  asm("{\n .reg .b16 s0, s1, b0, b1;\n mov.b32 {s0, s1}, %1;\n mov.b32 {b0, b1}, %2;\n"
      " fma.rn.f32.f16 %0, s0, b0, %0;\n fma.rn.f32.f16 %0, s1, b1, %0;\n}\n"
      : "+f"(acc)
      : "r"(s), "r"(b));
  return acc;
}

// 8 BF16 weights x 8 BF16 activations, FP32 accumulate
__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
  acc = fmaf(bf16lo(w.x), bf16lo(x.x), acc); acc = fmaf(bf16hi(w.x), bf16hi(x.x), acc);
  acc = fmaf(bf16lo(w.y), bf16lo(x.y), acc); acc = fmaf(bf16hi(w.y), bf16hi(x.y), acc);
  acc = fmaf(bf16lo(w.z), bf16lo(x.z), acc); acc = fmaf(bf16hi(w.z), bf16hi(x.z), acc);
  acc = fmaf(bf16lo(w.w), bf16lo(x.w), acc); acc = fmaf(bf16hi(w.w), bf16hi(x.w), acc);
  return acc;
}

// Sums R per-lane values over the 32 lanes in R/2 + R/4 + ... + (5 - log2 R) shuffles.
// Every lane returns the total of row `reduced_row<R>(lane)`.
template <int R>
__device__ __forceinline__ float multi_reduce(float (&v)[R], int lane) {
  int o = 16;
#pragma unroll
  for (int n = R; n > 1; n >>= 1, o >>= 1) {
    const bool upper = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = upper ? v[i] : v[i + n / 2];
      const float keep = upper ? v[i + n / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
  }
#pragma unroll
  for (; o > 0; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
  return v[0];
}
template <int R>
__device__ __forceinline__ int reduced_row(int lane) {
  int row = 0, o = 16;
#pragma unroll
  for (int n = R; n > 1; n >>= 1, o >>= 1) row += (lane & o) ? n / 2 : 0;
  return row;
}
template <int R>
__device__ __forceinline__ bool reduced_owner(int lane) {  // one lane per row
  return (lane & ((32 / R) - 1)) == 0;
}

// One warp: K BF16 values written by other blocks (read through L2, never from a stale L1 line)
// -> FP16 scaled by a power of two into [1, 2); returns the inverse. One round trip: every lane
// loads its K / 256 groups of eight values at once and keeps them for the second pass.
template <int K>
__device__ __forceinline__ float warp_stage_f16(const uint16_t* src, uint16_t* dst, int lane) {
  constexpr int N = K / 256;
  static_assert(K % 256 == 0, "a warp stages whole rounds of 32 x 8 values");
  uint4 v[N];
  uint32_t amax = 0;
#pragma unroll
  for (int n = 0; n < N; ++n) {
    v[n] = __ldcg(reinterpret_cast<const uint4*>(src) + n * 32 + lane);
    const uint32_t w4[4] = {v[n].x, v[n].y, v[n].z, v[n].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) amax = max(amax, max(w4[k] & 0x7fffu, (w4[k] >> 16) & 0x7fffu));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float inverse;
  const float scale = pow2_normaliser(amax, &inverse);
#pragma unroll
  for (int n = 0; n < N; ++n) {
    const uint4 h = stage_pack8(v[n], scale, lane & 3);   // group n * 32 + lane of eight: word (lane & 3) of its 32
    reinterpret_cast<uint4*>(dst)[n * 32 + lane] = h;
  }
  return inverse;
}

}  // namespace ink

// Residual add + RMS norm between two MoE blocks: one block per token.
#include "../../include/inkling_b200.h"
#include "common.cuh"

namespace ink {

constexpr int kNormThreads = 256;
constexpr int kNormMaxPerThread = 8;  // 8-element groups per thread: hidden <= 256 * 8 * 8

__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(const float* __restrict__ partial,
                                                                    uint16_t* __restrict__ residual,
                                                                    const uint16_t* __restrict__ weight, float eps,
                                                                    uint16_t* __restrict__ normed, int hidden) {
  __shared__ float s_red[kNormThreads / 32];
  const int token = blockIdx.x, tid = threadIdx.x;
  const float* p = partial + (size_t)token * hidden;
  uint16_t* r = residual + (size_t)token * hidden;
  uint16_t* y = normed + (size_t)token * hidden;
  const int groups = hidden / 8;
  float h[kNormMaxPerThread][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxPerThread; ++i) {
    const int gidx = i * kNormThreads + tid;
    if (gidx < groups) {
      const float4 a = *reinterpret_cast<const float4*>(p + gidx * 8);
      const float4 b = *reinterpret_cast<const float4*>(p + gidx * 8 + 4);
      const uint4 q = *reinterpret_cast<const uint4*>(r + gidx * 8);
      const float add[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      const uint32_t res[4] = {q.x, q.y, q.z, q.w};
      uint32_t packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = round_bf16(bf16lo(res[j]) + round_bf16(add[2 * j]));
        const float hi = round_bf16(bf16hi(res[j]) + round_bf16(add[2 * j + 1]));
        h[i][2 * j] = lo;
        h[i][2 * j + 1] = hi;
        sum = fmaf(lo, lo, sum);
        sum = fmaf(hi, hi, sum);
        packed[j] = f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
      }
      *reinterpret_cast<uint4*>(r + gidx * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  }
  sum = warp_sum(sum);
  if ((tid & 31) == 0) s_red[tid >> 5] = sum;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) total += s_red[w];
  const float scale = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < kNormMaxPerThread; ++i) {
    const int gidx = i * kNormThreads + tid;
    if (gidx < groups) {
      const uint4 wq = *reinterpret_cast<const uint4*>(weight + gidx * 8);
      const uint32_t wv[4] = {wq.x, wq.y, wq.z, wq.w};
      uint32_t packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = round_bf16(h[i][2 * j] * scale) * bf16lo(wv[j]);
        const float hi = round_bf16(h[i][2 * j + 1] * scale) * bf16hi(wv[j]);
        packed[j] = f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
      }
      *reinterpret_cast<uint4*>(y + gidx * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  }
}

}  // namespace ink

using namespace ink;

extern "C" int ink_add_rmsnorm(const float* partial, void* residual, const void* weight, float eps, void* normed,
                               int tokens, int hidden, ink_stream_t stream) {
  INK_REQUIRE(partial && residual && weight && normed, kBadArgument, "add_rmsnorm: null pointer argument");
  INK_REQUIRE(tokens >= 0 && hidden > 0 && hidden % 8 == 0 && hidden <= kNormThreads * kNormMaxPerThread * 8,
              kUnsupportedShape, "add_rmsnorm: tokens=%d hidden=%d unsupported", tokens, hidden);
  INK_REQUIRE(aligned16(partial) && aligned16(residual) && aligned16(weight) && aligned16(normed), kMisaligned,
              "add_rmsnorm: buffers must be 16-byte aligned");
  if (tokens == 0) return kOk;
  INK_PREFER_MAX_SMEM(add_rmsnorm_kernel);
  add_rmsnorm_kernel<<<tokens, kNormThreads, 0, (cudaStream_t)stream>>>(
      partial, (uint16_t*)residual, (const uint16_t*)weight, eps, (uint16_t*)normed, hidden);
  INK_CHECK_LAUNCH("add_rmsnorm");
  return kOk;
}

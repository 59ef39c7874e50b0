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

// Short convolution of one new token per sequence with its cached FP32 history, the skip
// connection and the decoder residual: one thread per channel. XF32 = 1: x is the block's
// FP32 output, cast to BF16 first (what the expert runtime returns to the layer).
template <int TAPS, bool XF32>
__global__ void __launch_bounds__(256) short_conv_kernel(const void* __restrict__ x_raw, const float* __restrict__ taps,
                                                          float* __restrict__ history, const uint16_t* __restrict__ residual,
                                                          uint16_t* __restrict__ y, int hidden) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= hidden) return;
  const size_t at = (size_t)blockIdx.y * hidden + d;
  float current;
  if (XF32) current = round_bf16(reinterpret_cast<const float*>(x_raw)[at]);
  else current = bf16_to_f32(reinterpret_cast<const uint16_t*>(x_raw)[at]);
  float* h = history + at * TAPS;
  const float* w = taps + (size_t)d * TAPS;
  float past[TAPS], tap[TAPS];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) {
    past[j] = h[j];
    tap[j] = w[j];
  }
  // separate multiplies and adds in tap order, as the reference kernel computes them (no fused multiply-add)
  float total = 0.f;
#pragma unroll
  for (int j = 0; j + 1 < TAPS; ++j) {
    total = __fadd_rn(total, __fmul_rn(past[j + 1], tap[j]));
    h[j] = past[j + 1];
  }
  total = __fadd_rn(total, __fmul_rn(current, tap[TAPS - 1]));
  h[TAPS - 1] = current;
  float out = round_bf16(__fadd_rn(total, current));
  if (residual) out = round_bf16(__fadd_rn(out, bf16_to_f32(residual[at])));
  y[at] = (uint16_t)f32_to_bf16_bits(out);
}

}  // namespace ink

using namespace ink;

extern "C" int ink_short_conv(const void* x, int x_is_fp32, const float* taps, float* history, const void* residual,
                              void* y, int batch, int hidden, int kernel_size, ink_stream_t stream) {
  INK_REQUIRE(x && taps && history && y, kBadArgument, "short_conv: null pointer argument");
  INK_REQUIRE(batch >= 0 && hidden > 0, kBadArgument, "short_conv: batch=%d hidden=%d", batch, hidden);
  INK_REQUIRE(kernel_size >= 2 && kernel_size <= 4, kUnsupportedShape, "short_conv: kernel_size=%d (2..4 are built)",
              kernel_size);
  if (batch == 0) return kOk;
  const dim3 grid((unsigned)((hidden + 255) / 256), (unsigned)batch);
  cudaStream_t s = (cudaStream_t)stream;
  const uint16_t* r = (const uint16_t*)residual;
  uint16_t* out = (uint16_t*)y;
#define INK_SCONV_CASE(T)                                                                              \
  if (kernel_size == T) {                                                                              \
    if (x_is_fp32) short_conv_kernel<T, true><<<grid, 256, 0, s>>>(x, taps, history, r, out, hidden);  \
    else short_conv_kernel<T, false><<<grid, 256, 0, s>>>(x, taps, history, r, out, hidden);           \
  }
  INK_SCONV_CASE(2)
  INK_SCONV_CASE(3)
  INK_SCONV_CASE(4)
#undef INK_SCONV_CASE
  INK_CHECK_LAUNCH("short_conv");
  return kOk;
}

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

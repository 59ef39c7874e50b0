// Decode attention with the learned relative-position bias: one query token per sequence against the
// layer's K/V cache (a ring of `window` slots in a sliding layer, `slots` positions in a full one).
// One block per (head, sequence); the relative logits of the head, the scores and the softmax live in
// shared memory, K and V are read once per block (heads of one group share them through the L2).
#include "../../include/inkling_b200.h"
#include "common.cuh"

namespace ink {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;

struct AttnArgs {
  const uint16_t* q;        // [bs, h, c] after q_norm
  const uint16_t* r;        // [bs, h, d_rel] relative states
  const uint16_t* proj;     // [d_rel, extent]
  const uint16_t* k;        // [bs, hk, slots, c], the current token already stored
  const uint16_t* v;
  const int64_t* position;  // device scalar: tokens stored before this one
  const int64_t* pad_counts;   // [bs] or null
  uint16_t* out;            // [bs, h, c]
  int heads, kv_heads, c, d_rel, extent, slots, window, n_floor;
  float alpha, scale;
};

__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int w = 1; w < kAttnWarps; ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  return m;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < kAttnWarps; ++w) s += red[w];
  __syncthreads();
  return s;
}

// Shared memory: q [c] | logits [extent] | scores [slots] | partial sums [kAttnThreads * 2]
__global__ void __launch_bounds__(kAttnThreads) decode_attention_kernel(AttnArgs a) {
  extern __shared__ __align__(16) float smem[];
  __shared__ float s_red[kAttnWarps];
  float* s_q = smem;
  float* s_logits = s_q + a.c;
  float* s_scores = s_logits + a.extent;
  float* s_part = s_scores + a.slots;
  const int head = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kv_head = head / (a.heads / a.kv_heads);
  const long long position = *a.position;
  const long long pad = a.pad_counts ? a.pad_counts[b] : 0;
  // logarithmic scaling of full-attention layers: query and bias times tau, each rounded to BF16 (the reference
  // multiplies in FP32 and casts back, my_inkling/model.py:583-590)
  const bool scaled = a.window == 0 && a.n_floor > 0;
  float tau = 1.f;
  if (scaled) tau = 1.f + a.alpha * logf(fmaxf((float)(position + 1) / (float)a.n_floor, 1.f));
  const uint16_t* q = a.q + ((size_t)b * a.heads + head) * a.c;
  for (int i = tid; i < a.c; i += kAttnThreads) {
    const float x = bf16_to_f32(q[i]);
    s_q[i] = scaled ? round_bf16(x * tau) : x;
  }
  // relative logits of this head: r @ proj, a BF16 matmul (FP32 sum, rounded once)
  const uint16_t* r = a.r + ((size_t)b * a.heads + head) * a.d_rel;
  for (int e = tid; e < a.extent; e += kAttnThreads) {
    float sum = 0.f;
    for (int j = 0; j < a.d_rel; ++j) sum = fmaf(bf16_to_f32(r[j]), bf16_to_f32(a.proj[(size_t)j * a.extent + e]), sum);
    s_logits[e] = round_bf16(sum);
  }
  __syncthreads();
  // scores: one warp per cache slot
  const uint16_t* keys = a.k + ((size_t)b * a.kv_heads + kv_head) * a.slots * a.c;
  float local_max = -INFINITY;
  for (int slot = warp; slot < a.slots; slot += kAttnWarps) {
    long long distance = position - slot;
    if (a.window) distance = ((distance % a.window) + a.window) % a.window;
    const bool allowed = distance >= 0 && distance <= position - pad;
    float score = -INFINITY;
    if (allowed) {
      const uint32_t* row = reinterpret_cast<const uint32_t*>(keys + (size_t)slot * a.c);
      float dot = 0.f;
      for (int i = lane; i < a.c / 2; i += 32) {
        const uint32_t w = __ldg(row + i);
        dot = fmaf(s_q[2 * i], bf16lo(w), dot);
        dot = fmaf(s_q[2 * i + 1], bf16hi(w), dot);
      }
      dot = warp_sum(dot);
      float bias = distance < a.extent ? s_logits[distance] : 0.f;
      if (scaled) bias = round_bf16(bias * tau);
      score = dot * a.scale + bias;
    }
    if (lane == 0) s_scores[slot] = score;
    local_max = fmaxf(local_max, score);
  }
  __syncthreads();
  const float top = block_max(local_max, s_red);
  float local_sum = 0.f;
  for (int slot = tid; slot < a.slots; slot += kAttnThreads) {
    const float s = s_scores[slot];
    const float p = s == -INFINITY ? 0.f : __expf(s - top);
    s_scores[slot] = p;
    local_sum += p;
  }
  const float total = block_sum(local_sum, s_red);   // (its barriers also publish the weights)
  // weighted sum of the values: a thread owns a pair of channels and every `parts`-th slot
  const int pairs = a.c / 2, parts = kAttnThreads / pairs;
  const int pair = tid % pairs, part = tid / pairs;
  float acc0 = 0.f, acc1 = 0.f;
  if (part < parts) {
    const uint16_t* values = a.v + ((size_t)b * a.kv_heads + kv_head) * a.slots * a.c;
    for (int slot = part; slot < a.slots; slot += parts) {
      const float p = s_scores[slot];
      if (p != 0.f) {
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(values + (size_t)slot * a.c) + pair);
        acc0 = fmaf(p, bf16lo(w), acc0);
        acc1 = fmaf(p, bf16hi(w), acc1);
      }
    }
  }
  s_part[2 * tid] = acc0;
  s_part[2 * tid + 1] = acc1;
  __syncthreads();
  if (tid < pairs) {
    float o0 = 0.f, o1 = 0.f;
    for (int p = 0; p < parts; ++p) {
      o0 += s_part[2 * (p * pairs + tid)];
      o1 += s_part[2 * (p * pairs + tid) + 1];
    }
    const float inv = 1.f / total;
    uint32_t* out = reinterpret_cast<uint32_t*>(a.out + ((size_t)b * a.heads + head) * a.c);
    out[tid] = f32_to_bf16_bits(o0 * inv) | (f32_to_bf16_bits(o1 * inv) << 16);
  }
}

// the new token's key and value into slot `position` (modulo the window in a sliding layer) of both caches
__global__ void update_kv_kernel(const uint16_t* __restrict__ new_k, const uint16_t* __restrict__ new_v,
                                 uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache,
                                 const int64_t* __restrict__ position, int c, int slots, int window) {
  const long long p = *position;
  const long long slot = window ? p % window : p;
  if (slot < 0 || slot >= slots) return;   // a full cache: nothing is written (the host-side check reports it)
  const size_t row = blockIdx.x;           // (sequence, kv head)
  for (int i = threadIdx.x; i < c; i += blockDim.x) {
    k_cache[(row * slots + slot) * c + i] = new_k[row * c + i];
    v_cache[(row * slots + slot) * c + i] = new_v[row * c + i];
  }
}

}  // namespace ink

using namespace ink;

extern "C" int ink_decode_attention(const void* q, const void* r, const void* proj, const void* k_cache,
                                    const void* v_cache, const int64_t* position, const int64_t* pad_counts, void* out,
                                    int batch, int heads, int kv_heads, int head_dim, int d_rel, int rel_extent, int slots,
                                    int window, int n_floor, float alpha, float scale, ink_stream_t stream) {
  INK_REQUIRE(q && r && proj && k_cache && v_cache && position && out, kBadArgument, "decode_attention: null pointer argument");
  INK_REQUIRE(batch >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, kBadArgument,
              "decode_attention: batch=%d heads=%d kv_heads=%d", batch, heads, kv_heads);
  INK_REQUIRE(head_dim >= 2 && head_dim % 2 == 0 && head_dim <= 2 * kAttnThreads && kAttnThreads % (head_dim / 2) == 0,
              kUnsupportedShape, "decode_attention: head_dim=%d unsupported (even, a divisor of %d)", head_dim, 2 * kAttnThreads);
  INK_REQUIRE(d_rel > 0 && rel_extent > 0 && slots > 0 && window >= 0 && (window == 0 || window <= slots), kBadArgument,
              "decode_attention: d_rel=%d rel_extent=%d slots=%d window=%d", d_rel, rel_extent, slots, window);
  const size_t smem = sizeof(float) * ((size_t)head_dim + rel_extent + slots + 2 * kAttnThreads);
  INK_REQUIRE(smem <= 200 * 1024, kUnsupportedShape, "decode_attention: %d slots + %d relative positions do not fit shared memory",
              slots, rel_extent);
  INK_REQUIRE(aligned16(q) && aligned16(k_cache) && aligned16(v_cache) && aligned16(out) && (head_dim * 2) % 4 == 0, kMisaligned,
              "decode_attention: buffers must be 16-byte aligned");
  if (batch == 0) return kOk;
  AttnArgs a{(const uint16_t*)q, (const uint16_t*)r, (const uint16_t*)proj, (const uint16_t*)k_cache, (const uint16_t*)v_cache,
             position, pad_counts, (uint16_t*)out, heads, kv_heads, head_dim, d_rel, rel_extent, slots, window, n_floor, alpha, scale};
  cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "decode_attention: %s", cudaGetErrorString(e));
  decode_attention_kernel<<<dim3(heads, batch), kAttnThreads, smem, (cudaStream_t)stream>>>(a);
  INK_CHECK_LAUNCH("decode_attention");
  return kOk;
}

extern "C" int ink_update_kv(const void* new_k, const void* new_v, void* k_cache, void* v_cache, const int64_t* position,
                             int batch, int kv_heads, int head_dim, int slots, int window, ink_stream_t stream) {
  INK_REQUIRE(new_k && new_v && k_cache && v_cache && position, kBadArgument, "update_kv: null pointer argument");
  INK_REQUIRE(batch >= 0 && kv_heads > 0 && head_dim > 0 && slots > 0 && window >= 0 && (window == 0 || window <= slots),
              kBadArgument, "update_kv: batch=%d kv_heads=%d head_dim=%d slots=%d window=%d", batch, kv_heads, head_dim, slots, window);
  if (batch == 0) return kOk;
  update_kv_kernel<<<batch * kv_heads, 128, 0, (cudaStream_t)stream>>>((const uint16_t*)new_k, (const uint16_t*)new_v,
                                                                       (uint16_t*)k_cache, (uint16_t*)v_cache, position,
                                                                       head_dim, slots, window);
  INK_CHECK_LAUNCH("update_kv");
  return kOk;
}

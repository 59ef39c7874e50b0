// Decode attention with the learned relative-position bias: one query token per sequence against the
// layer's K/V cache (a ring of `window` slots in a sliding layer, `slots` positions in a full one).
// One block per (head, sequence); the relative logits of the head, the scores and the softmax live in
// shared memory, K and V are read once per block (heads of one group share them through the L2).
#include "../../include/inkling_b200.h"
#include "common.cuh"

namespace ink {

constexpr int kAttnThreads = 256;   // (128 and 512 threads, i.e. 32 and 128 slots per block, measured the same)
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnKeys = 8;                                // cache slots a warp scores side by side
constexpr int kAttnSlots = kAttnWarps * kAttnKeys;          // slots per block: 64
constexpr int kAttnPartial = 2;                             // floats in front of a partial result: running maximum, sum

struct AttnArgs {
  const uint16_t* q;        // [bs, h, c] after q_norm
  const uint16_t* r;        // [bs, h, d_rel] relative states
  const uint16_t* proj;     // [d_rel, extent]
  const uint16_t* k;        // [bs, hk, slots, c], the current token already stored
  const uint16_t* v;
  const int64_t* position;  // device scalar: tokens stored before this one
  const int64_t* pad_counts;   // [bs] or null
  const uint16_t* new_k;    // [bs, hk, c] the current token's key and value, or null when the caches hold them already
  const uint16_t* new_v;
  uint16_t* k_store;        // the caches again, writable: where the current token is stored when new_k is given
  uint16_t* v_store;
  float* partial;           // [bs, h, splits, 2 + c]: maximum, sum of exponentials, unnormalised weighted values
  unsigned* arrived;        // [bs, h] blocks of a (sequence, head) that have stored their partial; zero between launches
  uint16_t* out;            // [bs, h, c]
  int heads, kv_heads, c, d_rel, extent, slots, window, n_floor, splits;
  float alpha, scale;
};

// One block per (head, sequence, group of 64 cache slots). A decode step has few (head, sequence) pairs and every
// load is a trip to DRAM, so the work is cut along the cache (as in split-K / flash decoding) and every block asks
// for ALL it needs at once: its key rows, its value rows (which slots are allowed is known before any score),
// the query and the relative states. It leaves a partial softmax (maximum, sum, weighted values); the block that
// stores the last partial of a (sequence, head) joins them.
template <int C>
__global__ void __launch_bounds__(kAttnThreads) decode_attention_kernel(AttnArgs a) {
  constexpr int kWords = C / 2;                          // 32-bit words of a row = channel pairs
  constexpr int kPerLane = (kWords + 31) / 32;           // words of a key row per lane
  constexpr int kParts = kAttnThreads / kWords;          // threads per channel pair in the value pass
  constexpr int kValues = kAttnSlots / kParts;           // value rows per thread
  static_assert(kAttnThreads % kWords == 0 && kAttnSlots % kParts == 0, "head_dim does not tile the block");
  __shared__ float s_q[C];
  __shared__ float s_bias[kAttnSlots];
  __shared__ float s_scores[kAttnSlots];
  __shared__ float s_part[kAttnThreads * 2];
  const int head = blockIdx.x, b = blockIdx.y, split = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kv_head = head / (a.heads / a.kv_heads);
  const int slot_base = split * kAttnSlots;
  // positions fit 32 bits; the ring arithmetic is done once per block (position modulo the window), not per slot
  const int position = (int)*a.position;
  const int reach = position - (int)(a.pad_counts ? a.pad_counts[b] : 0);   // largest distance that is not padding
  const int ring_position = a.window ? position % a.window : 0;
  auto distance_of = [&](int slot) -> int {
    if (!a.window) return position - slot;
    const int d = ring_position - (slot < a.window ? slot : slot % a.window);
    return d < 0 ? d + a.window : d;
  };
  auto allowed_at = [&](int slot) -> bool {
    const int d = distance_of(slot);
    return slot < a.slots && d >= 0 && d <= reach;
  };
  // ---- everything from memory, in flight together
  const uint16_t* keys = a.k + ((size_t)b * a.kv_heads + kv_head) * a.slots * C;
  const uint16_t* values = a.v + ((size_t)b * a.kv_heads + kv_head) * a.slots * C;
  // The current token may not be in the caches yet (new_k / new_v given): every block takes its row from there, and
  // the block of the group's first head whose slots include it stores it for the steps to come.
  const int fresh_slot = a.new_k ? (a.window ? ring_position : position) : -1;
  const uint16_t* fresh_k = a.new_k ? a.new_k + ((size_t)b * a.kv_heads + kv_head) * C : nullptr;
  const uint16_t* fresh_v = a.new_k ? a.new_v + ((size_t)b * a.kv_heads + kv_head) * C : nullptr;
  if (a.new_k && head % (a.heads / a.kv_heads) == 0 && fresh_slot >= slot_base && fresh_slot < slot_base + kAttnSlots &&
      fresh_slot < a.slots && tid < kWords) {
    const size_t at = (((size_t)b * a.kv_heads + kv_head) * a.slots + fresh_slot) * C;
    reinterpret_cast<uint32_t*>(a.k_store + at)[tid] = __ldg(reinterpret_cast<const uint32_t*>(fresh_k) + tid);
    reinterpret_cast<uint32_t*>(a.v_store + at)[tid] = __ldg(reinterpret_cast<const uint32_t*>(fresh_v) + tid);
  }
  bool k_allowed[kAttnKeys];
  uint32_t kw[kAttnKeys][kPerLane];
#pragma unroll
  for (int j = 0; j < kAttnKeys; ++j) {
    const int slot = slot_base + warp * kAttnKeys + j;
    k_allowed[j] = allowed_at(slot);
    const uint32_t* row = reinterpret_cast<const uint32_t*>(slot == fresh_slot ? fresh_k : keys + (size_t)slot * C);
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) kw[j][i] = (k_allowed[j] && i * 32 + lane < kWords) ? __ldg(row + i * 32 + lane) : 0u;
  }
  const int pair = tid % kWords, part = tid / kWords;   // value pass: this thread's channel pair, its slots part, part + kParts, ...
  uint32_t vw[kValues];
#pragma unroll
  for (int n = 0; n < kValues; ++n) {
    const int slot = slot_base + part + n * kParts;
    // (a slot that is not allowed may hold anything: it is not read)
    vw[n] = allowed_at(slot) ? __ldg(reinterpret_cast<const uint32_t*>(slot == fresh_slot ? fresh_v : values + (size_t)slot * C) + pair) : 0u;
  }
  // logarithmic scaling of full-attention layers: query and bias times tau, each rounded to BF16 (the reference
  // multiplies in FP32 and casts back, my_inkling/model.py:583-590)
  const bool scaled = a.window == 0 && a.n_floor > 0;
  float tau = 1.f;
  if (scaled) tau = 1.f + a.alpha * logf(fmaxf((float)(position + 1) / (float)a.n_floor, 1.f));
  if (tid < C) {
    const float x = bf16_to_f32(a.q[((size_t)b * a.heads + head) * C + tid]);
    s_q[tid] = scaled ? round_bf16(x * tau) : x;
  }
  // relative bias of this block's slots: (r @ proj)[distance], a BF16 matmul (FP32 sum, rounded once)
  if (tid >= kAttnThreads - kAttnSlots) {
    const int i = tid - (kAttnThreads - kAttnSlots), slot = slot_base + i;
    const int d = distance_of(slot);
    float bias = 0.f;
    if (slot < a.slots && d >= 0 && d < a.extent) {
      const uint16_t* r = a.r + ((size_t)b * a.heads + head) * a.d_rel;
      float sum = 0.f;
#pragma unroll 8
      for (int j = 0; j < a.d_rel; ++j) sum = fmaf(bf16_to_f32(r[j]), bf16_to_f32(__ldg(a.proj + (size_t)j * a.extent + d)), sum);
      bias = round_bf16(sum);
      if (scaled) bias = round_bf16(bias * tau);
    }
    s_bias[i] = bias;
  }
  __syncthreads();
  // ---- scores: warp w holds the key rows of the slots w * 8 .. w * 8 + 7 of the block
  {
    float dot[kAttnKeys];
#pragma unroll
    for (int j = 0; j < kAttnKeys; ++j) {
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) {
        const int at = i * 32 + lane;
        if (at < kWords) {
          sum = fmaf(s_q[2 * at], bf16lo(kw[j][i]), sum);
          sum = fmaf(s_q[2 * at + 1], bf16hi(kw[j][i]), sum);
        }
      }
      dot[j] = sum;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int j = 0; j < kAttnKeys; ++j) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], o);
    }
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < kAttnKeys; ++j)
        s_scores[warp * kAttnKeys + j] = k_allowed[j] ? dot[j] * a.scale + s_bias[warp * kAttnKeys + j] : -INFINITY;
    }
  }
  __syncthreads();
  // the block's 64 scores: every warp finds the maximum for itself (two scores per lane, five shuffles), the
  // first two warps turn the scores into exponentials once for everybody
  static_assert(kAttnSlots % 32 == 0, "whole scores per lane");
  float top = s_scores[lane];
#pragma unroll
  for (int i = 1; i < kAttnSlots / 32; ++i) top = fmaxf(top, s_scores[lane + 32 * i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
  if (tid < kAttnSlots) {
    const float sc = s_scores[tid];
    s_bias[tid] = (sc == -INFINITY) ? 0.f : __expf(sc - top);   // (the biases are in the scores by now)
  }
  __syncthreads();
  float acc0 = 0.f, acc1 = 0.f, sum = 0.f;
#pragma unroll
  for (int n = 0; n < kValues; ++n) {
    const float p = s_bias[part + n * kParts];
    acc0 = fmaf(p, bf16lo(vw[n]), acc0);
    acc1 = fmaf(p, bf16hi(vw[n]), acc1);
    sum += p;
  }
  s_part[2 * tid] = acc0;
  s_part[2 * tid + 1] = acc1;
  __syncthreads();
  if (pair == 0) s_scores[part] = sum;   // (the scores are not needed any more) one partial sum of exponentials per part
  __syncthreads();
  if (tid < kWords) {
    float o0 = 0.f, o1 = 0.f, total = 0.f;
#pragma unroll
    for (int p = 0; p < kParts; ++p) {
      o0 += s_part[2 * (p * kWords + tid)];
      o1 += s_part[2 * (p * kWords + tid) + 1];
      total += s_scores[p];
    }
    if (a.splits == 1) {
      const float inv = 1.f / total;
      uint32_t* out = reinterpret_cast<uint32_t*>(a.out + ((size_t)b * a.heads + head) * C);
      out[tid] = f32_to_bf16_bits(o0 * inv) | (f32_to_bf16_bits(o1 * inv) << 16);
    } else {
      float* mine = a.partial + (((size_t)b * a.heads + head) * a.splits + split) * (kAttnPartial + C);
      if (tid == 0) {
        mine[0] = top;
        mine[1] = total;
      }
      mine[kAttnPartial + 2 * tid] = o0;
      mine[kAttnPartial + 2 * tid + 1] = o1;
      __threadfence();   // every writer pushes its own stores out before the block is counted
    }
  }
  if (a.splits == 1) return;
  // The block that stores the last partial of its (sequence, head) joins them all:
  //   out = sum_i acc_i e^(m_i - M) / sum_i l_i e^(m_i - M)
  __shared__ bool s_last;
  __syncthreads();
  if (tid == 0) {
    unsigned* arrived = a.arrived + (size_t)b * a.heads + head;
    s_last = atomicAdd(arrived, 1u) + 1u == (unsigned)a.splits;
    if (s_last) *arrived = 0u;   // left as found, for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int stride = kAttnPartial + C;
  const float* base = a.partial + ((size_t)b * a.heads + head) * a.splits * stride;
  float all_top = -INFINITY;
  for (int i = lane; i < a.splits; i += 32) all_top = fmaxf(all_top, __ldcg(base + (size_t)i * stride));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) all_top = fmaxf(all_top, __shfl_xor_sync(0xffffffffu, all_top, o));
  // thread = (channel pair, part): every part takes every kParts-th partial, then the parts are added up
  float o0 = 0.f, o1 = 0.f, total = 0.f;
  for (int i = part; i < a.splits; i += kParts) {
    const float* from = base + (size_t)i * stride;
    const float m = __ldcg(from);
    if (m == -INFINITY) continue;
    const float weight = __expf(m - all_top);
    total = fmaf(__ldcg(from + 1), weight, total);
    const float2 acc = __ldcg(reinterpret_cast<const float2*>(from + kAttnPartial) + pair);
    o0 = fmaf(acc.x, weight, o0);
    o1 = fmaf(acc.y, weight, o1);
  }
  s_part[2 * tid] = o0;
  s_part[2 * tid + 1] = o1;
  if (pair == 0) s_scores[part] = total;
  __syncthreads();
  if (tid < kWords) {
    float f0 = 0.f, f1 = 0.f, sum_all = 0.f;
#pragma unroll
    for (int p = 0; p < kParts; ++p) {
      f0 += s_part[2 * (p * kWords + tid)];
      f1 += s_part[2 * (p * kWords + tid) + 1];
      sum_all += s_scores[p];
    }
    const float inv = 1.f / sum_all;
    uint32_t* out = reinterpret_cast<uint32_t*>(a.out + ((size_t)b * a.heads + head) * C);
    out[tid] = f32_to_bf16_bits(f0 * inv) | (f32_to_bf16_bits(f1 * inv) << 16);
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

static size_t attention_counter_bytes(int batch, int heads) { return ((size_t)batch * heads * sizeof(unsigned) + 255) / 256 * 256; }

extern "C" size_t ink_decode_attention_workspace_bytes(int batch, int heads, int head_dim, int slots) {
  const size_t splits = ((size_t)slots + kAttnSlots - 1) / kAttnSlots;
  return splits <= 1 ? 0 : attention_counter_bytes(batch, heads) + sizeof(float) * (size_t)batch * heads * splits * (kAttnPartial + head_dim);
}

extern "C" int ink_decode_attention(const void* q, const void* r, const void* proj, void* k_cache,
                                    void* v_cache, const int64_t* position, const int64_t* pad_counts, void* out,
                                    int batch, int heads, int kv_heads, int head_dim, int d_rel, int rel_extent, int slots,
                                    int window, int n_floor, float alpha, float scale, const void* new_k,
                                    const void* new_v, void* workspace, size_t workspace_bytes, ink_stream_t stream) {
  INK_REQUIRE(q && r && proj && k_cache && v_cache && position && out, kBadArgument, "decode_attention: null pointer argument");
  INK_REQUIRE(batch >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, kBadArgument,
              "decode_attention: batch=%d heads=%d kv_heads=%d", batch, heads, kv_heads);
  INK_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, kUnsupportedShape,
              "decode_attention: head_dim=%d unsupported (built for 64, 128 and 256)", head_dim);
  INK_REQUIRE(d_rel > 0 && rel_extent > 0 && slots > 0 && window >= 0 && (window == 0 || window <= slots), kBadArgument,
              "decode_attention: d_rel=%d rel_extent=%d slots=%d window=%d", d_rel, rel_extent, slots, window);
  INK_REQUIRE((new_k == nullptr) == (new_v == nullptr), kBadArgument, "decode_attention: new_k and new_v come together");
  const int splits = (slots + kAttnSlots - 1) / kAttnSlots;
  INK_REQUIRE(splits <= 65535 && batch <= 65535, kUnsupportedShape, "decode_attention: %d slots or %d sequences exceed the grid", slots, batch);
  const size_t need = ink_decode_attention_workspace_bytes(batch, heads, head_dim, slots);
  INK_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), kBadArgument,
              "decode_attention: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  INK_REQUIRE(aligned16(q) && aligned16(k_cache) && aligned16(v_cache) && aligned16(out) && (need == 0 || aligned16(workspace)),
              kMisaligned, "decode_attention: buffers must be 16-byte aligned");
  if (batch == 0) return kOk;
  AttnArgs a{(const uint16_t*)q, (const uint16_t*)r, (const uint16_t*)proj, (const uint16_t*)k_cache, (const uint16_t*)v_cache,
             position, pad_counts, (const uint16_t*)new_k, (const uint16_t*)new_v, (uint16_t*)k_cache, (uint16_t*)v_cache,
             (float*)((char*)workspace + attention_counter_bytes(batch, heads)), (unsigned*)workspace, (uint16_t*)out, heads, kv_heads, head_dim, d_rel, rel_extent, slots, window,
             n_floor, splits, alpha, scale};
  const dim3 grid(heads, batch, splits);
  if (head_dim == 64) decode_attention_kernel<64><<<grid, kAttnThreads, 0, (cudaStream_t)stream>>>(a);
  else if (head_dim == 128) decode_attention_kernel<128><<<grid, kAttnThreads, 0, (cudaStream_t)stream>>>(a);
  else decode_attention_kernel<256><<<grid, kAttnThreads, 0, (cudaStream_t)stream>>>(a);
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

// Router (sigmoid scores, top-k, BF16 weight chain) and expert plan for the resident
// placement. One launch at decode: every block computes a few logits; the block that
// finishes last turns them into indices, weights and the plan tables.
#include <stdarg.h>
#include <stdio.h>

#include "../../include/inkling_b200.h"
#include "common.cuh"

namespace ink {

static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

constexpr int kTokenGroup = 8;           // tokens whose accumulators a warp holds at once
constexpr int kMaxScoresPerLane = 16;    // n_routed <= 512
constexpr int kFinishThreads = 256;
constexpr int kPlanSmallRoutes = 512;    // routes the single-block plan keeps in shared memory

struct RouterArgs {
  const uint16_t* x;
  const uint16_t* weight;
  const float* bias;
  const uint16_t* global_scale;
  float route_scale;
  int tokens, hidden, n_routed, n_shared, top_k;
  uint16_t* routed_logits;
  uint16_t* topk_weights;
  int64_t* topk_indices;
  uint16_t* shared_gammas;
  float* logits;           // workspace: [tokens, n_routed + n_shared] BF16-rounded logits as FP32
  float* scores;           // workspace: [tokens, n_routed] selection scores
  unsigned int* counter;   // workspace: blocks done
};

struct PlanArgs {
  const int64_t* indices;
  const int64_t* sources;
  int64_t* pointers;
  int32_t* experts;
  int32_t* counts;
  int32_t* rows;
  int start, local, stride, routes, capacity;
};

// ------------------------------------------------------------------ one token
// Executed by one warp. `score` is this warp's shared-memory scratch of n_routed floats:
// score[e] = bf16(sigmoid(logit_e)) + bias_e, computed by the blocks that produced the
// logits. Small loops on purpose: this code runs once, on one warp, straight out of a
// cold instruction cache.
__device__ void router_finish_token(const RouterArgs& a, int token, float* score, int* ids_out) {
  const int lane = threadIdx.x & 31;
  const int total = a.n_routed + a.n_shared;
  const float* logit = a.logits + (size_t)token * total;
  const float* scores = a.scores + (size_t)token * a.n_routed;
  for (int e = lane; e < a.n_routed; e += 32) {
    score[e] = __ldcg(scores + e);
    if (a.routed_logits) a.routed_logits[(size_t)token * a.n_routed + e] = (uint16_t)f32_to_bf16_bits(__ldcg(logit + e));
  }
  __syncwarp();
  // top-k by repeated arg-max; ties go to the lower expert id
  int my_choice = 0;  // lane r < top_k ends up holding the r-th choice
#pragma unroll 1
  for (int r = 0; r < a.top_k; ++r) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll 1
    for (int e = lane; e < a.n_routed; e += 32) {
      const float v = score[e];
      if (v > best) {  // ascending e within a lane: a later equal value never replaces
        best = v;
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) {
        best = ov;
        best_e = oe;
      }
    }
    if (best_e == 0x7fffffff) best_e = r;  // every score is -inf/NaN: fall back to a valid id
    if (lane == 0) score[best_e] = -INFINITY;
    if (lane == r) my_choice = best_e;
    __syncwarp();
  }
  // weights over the top_k selected logits followed by the shared logits
  const int n = a.top_k + a.n_shared;
  const bool live = lane < n;
  float l = 0.f;
  if (lane < a.top_k) l = __ldcg(logit + my_choice);
  else if (live) l = __ldcg(logit + a.n_routed + (lane - a.top_k));
  // logsigmoid = min(0, x) - log1p(exp(-|x|)), result rounded to BF16
  const float lp = live ? round_bf16(fminf(0.f, l) - log1pf(__expf(-fabsf(l)))) : -INFINITY;
  float m = lp;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (fabsf(m) == INFINITY) m = 0.f;
  // logsumexp as torch composes it: exp(bf16(lp - max)) rounded, FP32 sum rounded, log rounded, + max rounded
  const float ex = live ? round_bf16(__expf(round_bf16(lp - m))) : 0.f;
  float s = ex;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float lse = round_bf16(round_bf16(__logf(round_bf16(s))) + m);
  float w = round_bf16(__expf(round_bf16(lp - lse)));
  w = round_bf16(w * a.route_scale);
  w = round_bf16(w * bf16_to_f32(a.global_scale[0]));
  if (lane < a.top_k) {
    a.topk_indices[(size_t)token * a.top_k + lane] = my_choice;
    a.topk_weights[(size_t)token * a.top_k + lane] = (uint16_t)f32_to_bf16_bits(w);
    if (ids_out) ids_out[token * a.top_k + lane] = my_choice;
  } else if (live) {
    a.shared_gammas[(size_t)token * a.n_shared + (lane - a.top_k)] = (uint16_t)f32_to_bf16_bits(w);
  }
}

// ------------------------------------------------------------- single-block plan
// routes <= kPlanSmallRoutes. Whole block; `ids` is shared memory for the routes.
__device__ void plan_small(const PlanArgs& p, int* ids, int* warp_totals, bool ids_loaded) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  for (int r = tid; r < p.routes; r += blockDim.x) {
    const int64_t id = ids_loaded ? (int64_t)ids[r] : p.indices[r];
    ids[r] = (id >= p.start && id < (int64_t)p.start + p.local) ? (int)(id - p.start) : -1;
  }
  __syncthreads();
  int groups_before = 0;
  for (int base = 0; base < p.local; base += blockDim.x) {
    const int e = base + tid;
    int count = 0;
    if (e < p.local)
      for (int r = 0; r < p.routes; ++r) count += (ids[r] == e);
    const bool active = count > 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, active);
    if (lane == 0) warp_totals[warp] = __popc(ballot);
    __syncthreads();
    int before = groups_before;
    for (int w = 0; w < warp; ++w) before += warp_totals[w];
    int chunk_total = 0;
    for (int w = 0; w < warps; ++w) chunk_total += warp_totals[w];
    const int group = before + __popc(ballot & ((1u << lane) - 1u));
    if (e < p.local) {
      if (active) {
        p.experts[group] = p.start + e;
        p.counts[group] = count;
        int pos = 0;
        for (int r = 0; r < p.routes; ++r)
          if (ids[r] == e) p.rows[(size_t)group * p.capacity + pos++] = r;
      }
      for (int b = 0; b < p.stride; ++b)
        p.pointers[(size_t)(p.start + e) * p.stride + b] = active ? p.sources[(size_t)e * p.stride + b] : 0;
    }
    groups_before += chunk_total;
    __syncthreads();
  }
  for (int g = groups_before + tid; g < p.local; g += blockDim.x) {
    p.experts[g] = -1;
    p.counts[g] = 0;
  }
}

// ------------------------------------------------------------------- logits kernel
// kRowsPerBlock rows of the router weight per block, kWarpsPerRow warps per row, so a
// 4096-wide row is one round trip of four 16-byte loads per thread. TG tokens share
// one pass over the row.
constexpr int kRowsPerBlock = 2;
constexpr int kWarpsPerRow = kFinishThreads / 32 / kRowsPerBlock;

template <bool kFusePlan, int TG>
__global__ void __launch_bounds__(kFinishThreads) router_kernel(RouterArgs a, PlanArgs p) {
  __shared__ int s_ids[kPlanSmallRoutes];
  __shared__ int s_warp_totals[32];
  __shared__ float s_part[kRowsPerBlock][kWarpsPerRow][TG];
  __shared__ float s_score[kFinishThreads / 32][32 * kMaxScoresPerLane];
  __shared__ bool s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int total = a.n_routed + a.n_shared;
  const int local_row = warp / kWarpsPerRow, part = warp % kWarpsPerRow;
  const int row = blockIdx.x * kRowsPerBlock + local_row;
  const int chunks = a.hidden / 8;  // 16-byte chunks per row
  for (int t0 = 0; t0 < a.tokens; t0 += TG) {
    float acc[TG];
#pragma unroll
    for (int t = 0; t < TG; ++t) acc[t] = 0.f;
    if (row < total) {
      const uint4* w = reinterpret_cast<const uint4*>(a.weight + (size_t)row * a.hidden);
#pragma unroll 4
      for (int c = part * 32 + lane; c < chunks; c += 32 * kWarpsPerRow) {
        const uint4 q = __ldg(w + c);
#pragma unroll
        for (int t = 0; t < TG; ++t) {
          if (t0 + t < a.tokens) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.x + (size_t)(t0 + t) * a.hidden) + c);
            float s = acc[t];
            s = fmaf(bf16lo(q.x), bf16lo(v.x), s);
            s = fmaf(bf16hi(q.x), bf16hi(v.x), s);
            s = fmaf(bf16lo(q.y), bf16lo(v.y), s);
            s = fmaf(bf16hi(q.y), bf16hi(v.y), s);
            s = fmaf(bf16lo(q.z), bf16lo(v.z), s);
            s = fmaf(bf16hi(q.z), bf16hi(v.z), s);
            s = fmaf(bf16lo(q.w), bf16lo(v.w), s);
            s = fmaf(bf16hi(q.w), bf16hi(v.w), s);
            acc[t] = s;
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < TG; ++t) {
      const float s = warp_sum(acc[t]);
      if (lane == 0) s_part[local_row][part][t] = s;
    }
    __syncthreads();
    if (threadIdx.x < kRowsPerBlock * TG) {
      const int r = threadIdx.x / TG, t = threadIdx.x % TG;
      const int out_row = blockIdx.x * kRowsPerBlock + r;
      if (out_row < total && t0 + t < a.tokens) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsPerRow; ++w) s += s_part[r][w][t];
        const float l = round_bf16(s);
        a.logits[(size_t)(t0 + t) * total + out_row] = l;
        // BF16 sigmoid, then FP32 add of the FP32 bias: the value the top-k compares
        if (out_row < a.n_routed)
          a.scores[(size_t)(t0 + t) * a.n_routed + out_row] = round_bf16(1.f / (1.f + __expf(-l))) + a.bias[out_row];
      }
    }
    __syncthreads();
  }
  // the block that arrives last owns the tail of the computation
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(a.counter, 1u);
    s_last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int token = warp; token < a.tokens; token += warps)
    router_finish_token(a, token, s_score[warp], kFusePlan ? s_ids : nullptr);
  if (kFusePlan) {
    __syncthreads();
    plan_small(p, s_ids, s_warp_totals, true);
  }
  if (threadIdx.x == 0) *a.counter = 0u;  // leave the workspace ready for the next call
}

__global__ void __launch_bounds__(kFinishThreads) plan_small_kernel(PlanArgs p) {
  __shared__ int s_ids[kPlanSmallRoutes];
  __shared__ int s_warp_totals[32];
  plan_small(p, s_ids, s_warp_totals, false);
}

// ------------------------------------------------------------- plan, any size
// Pass 1 (one block): histogram of routes per expert, then compaction of the active
// experts and the pointer table. Pass 2 (one warp per expert): ordered list of routes.
__global__ void __launch_bounds__(1024) plan_count_kernel(PlanArgs p, int* histogram /* [local] zeroed by this kernel */) {
  __shared__ int s_warp_totals[32];
  __shared__ int s_base;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  for (int e = tid; e < p.local; e += blockDim.x) histogram[e] = 0;
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int r = tid; r < p.routes; r += blockDim.x) {
    const int64_t id = p.indices[r];
    if (id >= p.start && id < (int64_t)p.start + p.local) atomicAdd(&histogram[(int)(id - p.start)], 1);
  }
  __syncthreads();
  for (int base = 0; base < p.local; base += blockDim.x) {
    const int e = base + tid;
    const int count = e < p.local ? histogram[e] : 0;
    const bool active = count > 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, active);
    if (lane == 0) s_warp_totals[warp] = __popc(ballot);
    __syncthreads();
    int before = s_base, chunk_total = 0;
    for (int w = 0; w < warps; ++w) {
      if (w < warp) before += s_warp_totals[w];
      chunk_total += s_warp_totals[w];
    }
    const int group = before + __popc(ballot & ((1u << lane) - 1u));
    if (e < p.local) {
      if (active) {
        p.experts[group] = p.start + e;
        p.counts[group] = count;
      }
      for (int b = 0; b < p.stride; ++b)
        p.pointers[(size_t)(p.start + e) * p.stride + b] = active ? p.sources[(size_t)e * p.stride + b] : 0;
    }
    __syncthreads();
    if (tid == 0) s_base += chunk_total;
    __syncthreads();
  }
  for (int g = s_base + tid; g < p.local; g += blockDim.x) {
    p.experts[g] = -1;
    p.counts[g] = 0;
  }
}

__global__ void __launch_bounds__(256) plan_rows_kernel(PlanArgs p) {
  const int lane = threadIdx.x & 31;
  const int group = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (group >= p.local) return;
  const int expert = p.experts[group];
  if (expert < 0) return;
  int pos = 0;
  for (int base = 0; base < p.routes; base += 32) {
    const int r = base + lane;
    const bool match = r < p.routes && p.indices[r] == (int64_t)expert;
    const unsigned ballot = __ballot_sync(0xffffffffu, match);
    if (match) p.rows[(size_t)group * p.capacity + pos + __popc(ballot & ((1u << lane) - 1u))] = r;
    pos += __popc(ballot);
  }
}

static int check_router(const RouterArgs& a, size_t workspace_bytes) {
  INK_REQUIRE(a.tokens >= 0 && a.hidden > 0, kBadArgument, "router: tokens=%d hidden=%d", a.tokens, a.hidden);
  INK_REQUIRE(a.hidden % 8 == 0, kUnsupportedShape, "router: hidden=%d must be a multiple of 8", a.hidden);
  INK_REQUIRE(a.n_routed > 0 && a.n_routed <= 32 * kMaxScoresPerLane, kUnsupportedShape,
              "router: n_routed=%d must be between 1 and %d", a.n_routed, 32 * kMaxScoresPerLane);
  INK_REQUIRE(a.top_k >= 1 && a.top_k <= 32 && a.top_k <= a.n_routed && a.n_shared >= 0 && a.top_k + a.n_shared <= 32,
              kUnsupportedShape, "router: top_k=%d n_shared=%d unsupported", a.top_k, a.n_shared);
  INK_REQUIRE(a.x && a.weight && a.bias && a.global_scale && a.topk_weights && a.topk_indices &&
                  (a.n_shared == 0 || a.shared_gammas) && a.logits,
              kBadArgument, "router: null pointer argument");
  INK_REQUIRE(aligned16(a.x) && aligned16(a.weight), kMisaligned, "router: x and weight must be 16-byte aligned");
  INK_REQUIRE(workspace_bytes >= ink_router_workspace_bytes(a.tokens, a.n_routed + a.n_shared), kBadArgument,
              "router: workspace of %zu bytes is too small", workspace_bytes);
  return kOk;
}

static int check_plan(const PlanArgs& p) {
  INK_REQUIRE(p.indices && p.sources && p.pointers && p.experts && p.counts && p.rows, kBadArgument,
              "expert_plan: null pointer argument");
  INK_REQUIRE(p.local > 0 && p.start >= 0 && p.stride > 0 && p.routes >= 0 && p.capacity >= 1, kBadArgument,
              "expert_plan: start=%d local=%d stride=%d routes=%d capacity=%d", p.start, p.local, p.stride,
              p.routes, p.capacity);
  INK_REQUIRE(p.capacity >= p.routes || p.capacity >= 1, kBadArgument, "expert_plan: capacity too small");
  return kOk;
}

}  // namespace ink

using namespace ink;

extern "C" const char* ink_last_error(void) { return g_error; }
extern "C" int ink_abi_version(void) { return 1; }

extern "C" size_t ink_router_workspace_bytes(int tokens, int n_experts_total) {
  // 256 bytes of counters, then the FP32 logits and the FP32 selection scores
  return 256 + 2 * sizeof(float) * (size_t)(tokens > 0 ? tokens : 0) * (size_t)n_experts_total;
}

static RouterArgs make_router_args(const void* x, const void* weight, const float* bias, const void* global_scale,
                                   float route_scale, int tokens, int hidden, int n_routed, int n_shared,
                                   int top_k, void* routed_logits, void* topk_weights, int64_t* topk_indices,
                                   void* shared_gammas, void* workspace) {
  RouterArgs a;
  a.x = (const uint16_t*)x;
  a.weight = (const uint16_t*)weight;
  a.bias = bias;
  a.global_scale = (const uint16_t*)global_scale;
  a.route_scale = route_scale;
  a.tokens = tokens;
  a.hidden = hidden;
  a.n_routed = n_routed;
  a.n_shared = n_shared;
  a.top_k = top_k;
  a.routed_logits = (uint16_t*)routed_logits;
  a.topk_weights = (uint16_t*)topk_weights;
  a.topk_indices = topk_indices;
  a.shared_gammas = (uint16_t*)shared_gammas;
  a.counter = (unsigned int*)workspace;
  a.logits = workspace ? (float*)((char*)workspace + 256) : nullptr;
  a.scores = a.logits ? a.logits + (size_t)(tokens > 0 ? tokens : 0) * (size_t)(n_routed + n_shared) : nullptr;
  return a;
}

extern "C" int ink_router_forward(const void* x, const void* weight, const float* bias, const void* global_scale,
                                  float route_scale, int tokens, int hidden, int n_routed, int n_shared,
                                  int top_k, void* routed_logits, void* topk_weights, int64_t* topk_indices,
                                  void* shared_gammas, void* workspace, size_t workspace_bytes,
                                  ink_stream_t stream) {
  RouterArgs a = make_router_args(x, weight, bias, global_scale, route_scale, tokens, hidden, n_routed, n_shared,
                                  top_k, routed_logits, topk_weights, topk_indices, shared_gammas, workspace);
  if (int rc = check_router(a, workspace_bytes)) return rc;
  if (tokens == 0) return kOk;
  const int blocks = (n_routed + n_shared + kRowsPerBlock - 1) / kRowsPerBlock;
  INK_PREFER_MAX_SMEM((router_kernel<false, 1>));
  INK_PREFER_MAX_SMEM((router_kernel<false, kTokenGroup>));
  if (tokens == 1)
    router_kernel<false, 1><<<blocks, kFinishThreads, 0, (cudaStream_t)stream>>>(a, PlanArgs{});
  else
    router_kernel<false, kTokenGroup><<<blocks, kFinishThreads, 0, (cudaStream_t)stream>>>(a, PlanArgs{});
  INK_CHECK_LAUNCH("ink_router_forward");
  return kOk;
}

// ------------------------------------------------------------ router, no allocation
// Scratch for ink_router_forward_static: lives in the library image, so a process that
// loads the library holds these bytes on every GPU it uses, until it exits.
constexpr int kStaticRouterTokens = 8;
constexpr int kStaticRouterExperts = 32 * kMaxScoresPerLane + 32;   // routed + shared rows at most
constexpr size_t kStaticRouterBytes = 256 + 2 * sizeof(float) * kStaticRouterTokens * kStaticRouterExperts;
static __device__ __align__(256) unsigned char g_static_router_scratch[kStaticRouterBytes];

constexpr int kStaticMaxDevices = 64;
// Device address of the array, per device ordinal. Written without a lock: two host threads that
// make the first call on a device together both look the address up and store the same value.
// The address stays valid for the life of the process as long as the device is not reset.
static void* g_static_router_ptr[kStaticMaxDevices];

extern "C" int ink_router_forward_static(const void* x, const void* weight, const float* bias,
                                         const void* global_scale, float route_scale, int tokens, int hidden,
                                         int n_routed, int n_shared, int top_k, void* routed_logits,
                                         void* topk_weights, int64_t* topk_indices, void* shared_gammas,
                                         ink_stream_t stream) {
  INK_REQUIRE(tokens >= 0 && tokens <= kStaticRouterTokens, kUnsupportedShape,
              "router (static scratch): %d tokens, the built-in scratch holds at most %d", tokens,
              kStaticRouterTokens);
  INK_REQUIRE(n_routed > 0 && n_shared >= 0 && n_routed + n_shared <= kStaticRouterExperts, kUnsupportedShape,
              "router (static scratch): %d router rows, the built-in scratch holds at most %d",
              n_routed + n_shared, kStaticRouterExperts);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  INK_REQUIRE(e == cudaSuccess && device >= 0 && device < kStaticMaxDevices, kLaunchFailed,
              "router (static scratch): cannot identify the current device: %s", cudaGetErrorString(e));
  if (g_static_router_ptr[device] == nullptr) {
    // The array's name is only a handle on the host: ask the runtime for its address on
    // the device that is current now, once, and keep it.
    void* address = nullptr;
    e = cudaGetSymbolAddress(&address, g_static_router_scratch);
    INK_REQUIRE(e == cudaSuccess && address != nullptr, kLaunchFailed,
                "router (static scratch): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_static_router_ptr[device] = address;
  }
  void* scratch = g_static_router_ptr[device];
  // The block counter at the head of the scratch must be zero when the kernel starts; the
  // previous call normally leaves it so, but a call that was cut short would not.
  e = cudaMemsetAsync(scratch, 0, 256, (cudaStream_t)stream);
  INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "router (static scratch): memset failed: %s", cudaGetErrorString(e));
  return ink_router_forward(x, weight, bias, global_scale, route_scale, tokens, hidden, n_routed, n_shared, top_k,
                            routed_logits, topk_weights, topk_indices, shared_gammas, scratch, kStaticRouterBytes,
                            stream);
}

extern "C" int ink_router_plan_forward(const void* x, const void* weight, const float* bias,
                                       const void* global_scale, float route_scale, int tokens, int hidden,
                                       int n_routed, int n_shared, int top_k, void* routed_logits,
                                       void* topk_weights, int64_t* topk_indices, void* shared_gammas,
                                       void* workspace, size_t workspace_bytes, const int64_t* sources,
                                       int64_t* pointers, int32_t* experts, int32_t* counts, int32_t* rows,
                                       int start, int local, int stride, int capacity, ink_stream_t stream) {
  RouterArgs a = make_router_args(x, weight, bias, global_scale, route_scale, tokens, hidden, n_routed, n_shared,
                                  top_k, routed_logits, topk_weights, topk_indices, shared_gammas, workspace);
  if (int rc = check_router(a, workspace_bytes)) return rc;
  PlanArgs p{topk_indices, sources, pointers, experts, counts, rows, start, local, stride, tokens * top_k, capacity};
  if (int rc = check_plan(p)) return rc;
  INK_REQUIRE(p.routes <= kPlanSmallRoutes, kUnsupportedShape,
              "router_plan: %d routes exceed the fused limit of %d; call the router and the plan separately",
              p.routes, kPlanSmallRoutes);
  INK_REQUIRE(capacity >= p.routes || capacity >= tokens, kBadArgument, "router_plan: capacity=%d too small", capacity);
  if (tokens == 0) return kOk;
  const int blocks = (n_routed + n_shared + kRowsPerBlock - 1) / kRowsPerBlock;
  INK_PREFER_MAX_SMEM((router_kernel<true, 1>));
  INK_PREFER_MAX_SMEM((router_kernel<true, kTokenGroup>));
  if (tokens == 1)
    router_kernel<true, 1><<<blocks, kFinishThreads, 0, (cudaStream_t)stream>>>(a, p);
  else
    router_kernel<true, kTokenGroup><<<blocks, kFinishThreads, 0, (cudaStream_t)stream>>>(a, p);
  INK_CHECK_LAUNCH("ink_router_plan_forward");
  return kOk;
}

extern "C" int ink_expert_plan(const int64_t* indices, const int64_t* sources, int64_t* pointers,
                               int32_t* experts, int32_t* counts, int32_t* rows, int start, int local,
                               int stride, int routes, int capacity, ink_stream_t stream) {
  PlanArgs p{indices, sources, pointers, experts, counts, rows, start, local, stride, routes, capacity};
  if (int rc = check_plan(p)) return rc;
  if (routes <= kPlanSmallRoutes) {
    INK_PREFER_MAX_SMEM(plan_small_kernel);
    plan_small_kernel<<<1, kFinishThreads, 0, (cudaStream_t)stream>>>(p);
    INK_CHECK_LAUNCH("ink_expert_plan");
    return kOk;
  }
  // large plans borrow counts[] as the histogram: pass 1 rewrites it in compacted order
  // only after every histogram entry has been read into a register.
  INK_PREFER_MAX_SMEM(plan_count_kernel);
  INK_PREFER_MAX_SMEM(plan_rows_kernel);
  plan_count_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(p, p.counts);
  INK_CHECK_LAUNCH("ink_expert_plan(count)");
  const int warps = 8;
  plan_rows_kernel<<<(local + warps - 1) / warps, warps * 32, 0, (cudaStream_t)stream>>>(p);
  INK_CHECK_LAUNCH("ink_expert_plan(rows)");
  return kOk;
}

// One persistent cooperative kernel for a whole stack of MoE blocks at decode (one
// token): router, expert plan, routed NVFP4 and shared BF16 gate/up, down + combine and
// the residual add + RMS norm between blocks, all inside one launch.
//
// One block per SM. Warp 0 is the producer: it walks the block's tile list, layer after
// layer, and keeps a 20-slot shared-memory ring full with bulk asynchronous copies; it
// never waits for arithmetic, only for a free slot and -- before the first routed tile
// of a layer -- for that layer's routing. Warps 1..10 are consumers: consumer c takes
// tiles c, c+10, ... (the ring depth is a multiple of the consumer count, see the ring
// comment in stream_decode.cu). Warp 11 is the auxiliary warp: on the block that
// finishes the last router row it runs the top-k / weight chain / plan for the layer.
// Phases of a layer are ordered across blocks by three counters in global memory
// (shared gate/up done, routed gate/up done, down done); the weight stream itself never
// stops at them, because weight addresses do not depend on activations.
//
// Every wait (ring slot, routing flag, counter) is bounded; a wait that gives up sets
// kFlagWaitTimedOut in the status word, marks the launch as failed and every loop
// drains without further waiting.
#include <stdlib.h>

#include "../../include/inkling_b200.h"
#include "common.cuh"
#include "decode_args.cuh"
#include "pipe.cuh"
#include "stream_math.cuh"

namespace ink {

constexpr int kSC = 8;                                 // consumer warps
constexpr int kSStages = 2 * kSC;                      // ring slots
constexpr int kSSlot = 9216;                           // bytes per slot
constexpr int kSThreads = (kSC + 2) * 32;              // producer + consumers + auxiliary
constexpr int kSMaxTopK = 8;
constexpr int kSMaxShared = 2;
constexpr int kSMaxRows = 64;                          // output rows one block may own
constexpr int kSMaxExperts = 512;
constexpr int kSyncWordsPerLayer = 8;                  // counters of one layer
constexpr int kSMaxWorld = 8;                          // tensor-parallel ranks

constexpr int kTraceBlocks = 256;
constexpr int kTraceSlots = 16;
// phase stamps written by consumer warp 0 (and slot 12..14 by the producer) when tracing is on
enum TraceSlot {
  kTrLayerStart = 0, kTrRouterDone = 1, kTrShGuDone = 2, kTrRtGuDone = 3, kTrShGuAll = 4, kTrShDownDone = 5,
  kTrRtGuAll = 6, kTrActStaged = 7, kTrRtDownDone = 8, kTrDownAll = 9, kTrNormDone = 10,
  kTrProdRouteWait = 12, kTrProdRouteGot = 13, kTrProdLayerIssued = 14,
};
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define INK_TRACE(layer, slot)                                                                          \
  do {                                                                                                  \
    if (a.trace && blockIdx.x < kTraceBlocks)                                                           \
      a.trace[((size_t)(layer) * kTraceBlocks + blockIdx.x) * kTraceSlots + (slot)] = global_ns();      \
  } while (0)

enum SyncWord { kShGuDone = 0, kRtGuDone = 1, kRouterRows = 3, kRouteReady = 4 };

// What the layer's routing resolved to: written once per layer by the auxiliary warp
// of one block, read by every producer and consumer.
struct RouteEntry {
  const uint8_t* gu_codes;
  const uint8_t* gu_scales;
  const uint8_t* dn_codes;
  const uint8_t* dn_scales;
  float gu_scale2;
  float dn_scale2;
  float weight;      // router weight of the route
  int expert;
};
struct RouteTable {
  RouteEntry route[kSMaxTopK];
  float gamma[kSMaxShared];
  int pad[2];
};

struct StackLayer {
  const uint16_t* router_weight;   // [experts + n_shared, hidden] BF16
  const float* router_bias;        // [experts]
  const uint16_t* global_scale;    // [1] BF16
  const int64_t* sources;          // [experts, 6] addresses of the resident banks
  const uint16_t* shared_gate;     // [n_shared, f, hidden]
  const uint16_t* shared_up;
  const uint16_t* shared_down;     // [n_shared, hidden, f]
  const uint16_t* norm_weight;     // [hidden] weight of the norm that follows the block (glue mode)
  int64_t* topk_indices;           // [top_k] optional outputs of the router
  uint16_t* topk_weights;          // [top_k]
  uint16_t* gammas;                // [n_shared]
  float route_scale;
  int pad;
};

struct StackArgs {
  const StackLayer* layers;
  int n_layers;
  int experts, n_shared, top_k;
  int glue;                        // 1: h += bf16(moe(norm h)), norm between blocks; 0: one block, partial out only
  float eps;
  const uint16_t* x;               // [hidden] BF16 input (already normalised for the first block)
  uint16_t* residual;              // [2][hidden] BF16: slot 0 holds the incoming residual stream (glue mode)
  uint16_t* normed_out;            // [hidden] BF16 output of the last norm (glue mode)
  float* partial;                  // [hidden] FP32 output of the (last) block
  float* logits;                   // scratch [2][experts + n_shared]
  float* scores;                   // scratch [2][experts]
  uint16_t* activated;             // scratch [2][top_k][f]
  uint16_t* shared_activated;      // scratch [2][n_shared][f]
  RouteTable* routes;              // scratch [n_layers]
  unsigned* sync;                  // scratch [n_layers][kSyncWordsPerLayer]: counters that only grow (see epoch)
  unsigned* epoch;                 // scratch: launches completed so far on this rank; every target scales with it
  // tensor-parallel ranks (world == 1: the "peers" are this rank's own scratch)
  int rank, world;
  float* inbox;                    // this rank's [2][world][hidden] FP32: partial outputs as the ranks deliver them
  unsigned* xsync;                 // this rank's [n_layers] counters of delivered blocks
  float* peer_inbox[kSMaxWorld];   // the same two regions of every rank, as mapped into this process
  unsigned* peer_xsync[kSMaxWorld];
  int32_t* status;
  unsigned long long* trace;       // optional [n_layers][kTraceBlocks][kTraceSlots] nanosecond stamps
};

template <int D, int F>
struct StackShape {
  // router rows
  static constexpr int R_BYTES = D * 2;
  static constexpr int R_CPL = D / 256;                    // 16-byte chunks per lane per row
  // shared gate/up: a tile holds SG_PAIRS (gate, up) pairs over SG_COLS columns
  static constexpr int SG_SPLIT = D > 2048 ? D / 2048 : 1;
  static constexpr int SG_COLS = D / SG_SPLIT;
  static constexpr int SG_PAIRS = 2048 / SG_COLS;
  static constexpr int SG_PART = SG_PAIRS * SG_COLS * 2;   // bytes of the gate rows (= of the up rows): 4096
  static constexpr int SG_CPL = SG_COLS / 256;
  // routed gate/up
  static constexpr int QG_ROWS = 8192 / (D / 2);
  static constexpr int QG_PAIRS = QG_ROWS / 2;
  static constexpr int QG_CODES = 8192;
  static constexpr int QG_SCALES = QG_ROWS * (D / 16);
  static constexpr int QG_CPL = D / 1024;
  // down: groups of RT output rows
  static constexpr int CH = F / 32;
  static constexpr int LPR = CH < 32 ? CH : 32;
  static constexpr int QD_CPL = CH / LPR;
  static constexpr int RPP = 32 / LPR;
  static constexpr int RT = F >= 2048 ? 4 : 8192 / F;
  static constexpr int PASSES = RT / RPP;
  static constexpr int QD_CODES = RT * (F / 2);
  static constexpr int QD_SCALES = RT * (F / 16);
  static constexpr int SD_ROWS = 8192 / (F * 2) < RT ? 8192 / (F * 2) : RT;   // BF16 rows per tile
  static constexpr int SD_PER_GROUP = RT / SD_ROWS;
  static constexpr int SD_BYTES = SD_ROWS * F * 2;
  static constexpr int SD_CPL = F / 256;
  static_assert(R_BYTES <= kSSlot && 2 * SG_PART <= kSSlot && QG_CODES + QG_SCALES <= kSSlot, "tile exceeds slot");
  static_assert(QD_CODES + QD_SCALES <= kSSlot && SD_BYTES <= kSSlot, "tile exceeds slot");
  // staging that overlays: [x FP16 | x BF16] during gate/up, [routed act FP16 | shared act BF16] during down
  static constexpr int STAGING = (kSMaxTopK * F * 2 + kSMaxShared * F * 2) > D * 4
                                     ? (kSMaxTopK * F * 2 + kSMaxShared * F * 2) : D * 4;
  static constexpr int SMEM = kSStages * kSSlot + STAGING;
};

// The tile list of one block for one layer, identical for every layer.
struct TilePlan {
  int r0, n_r;            // router rows [r0, r0 + n_r)
  int u0, n_u;            // shared gate/up units (SG_PAIRS pairs each)
  int q0, n_q;            // routed gate/up tiles
  int g0, n_g;            // down row groups
  // section starts in the per-layer sequence
  int s_r, s_sg, s_qg, s_sd, s_qd, s_pad, per_layer;
  int n_sg, n_sd, n_qd;   // tiles in the sections (with padding where the section is padded)
};

template <int D, int F>
__device__ __forceinline__ TilePlan make_plan(const StackArgs& a) {
  using S = StackShape<D, F>;
  TilePlan p;
  const long long b = blockIdx.x, G = gridDim.x;
  const int rows = a.experts + a.n_shared;
  p.r0 = (int)(b * rows / G);
  p.n_r = (int)((b + 1) * rows / G) - p.r0;
  const int units = a.n_shared * (F / S::SG_PAIRS);
  p.u0 = (int)(b * units / G);
  p.n_u = (int)((b + 1) * units / G) - p.u0;
  const int qg = a.top_k * (2 * F / S::QG_ROWS);
  p.q0 = (int)(b * qg / G);
  p.n_q = (int)((b + 1) * qg / G) - p.q0;
  const int groups = D / S::RT;
  p.g0 = (int)(b * groups / G);
  p.n_g = (int)((b + 1) * groups / G) - p.g0;
  const int pad_r = (p.n_r + kSC - 1) / kSC * kSC;
  p.n_sg = (p.n_u + kSC - 1) / kSC * kSC * S::SG_SPLIT;
  p.n_sd = a.n_shared * p.n_g * S::SD_PER_GROUP;
  p.n_qd = a.top_k * p.n_g;
  p.s_r = 0;
  p.s_sg = pad_r;
  p.s_qg = p.s_sg + p.n_sg;
  p.s_sd = p.s_qg + p.n_q;
  p.s_qd = p.s_sd + p.n_sd;
  p.s_pad = p.s_qd + p.n_qd;
  p.per_layer = (p.s_pad + kSC - 1) / kSC * kSC;
  return p;
}

struct StackShared {
  uint64_t full[kSStages];
  uint64_t empty[kSStages];
  RouteTable routes[2];                 // by layer parity; filled by the producer warp
  float contrib[kSMaxTopK + kSMaxShared][kSMaxRows];
  float score[kSMaxExperts];            // auxiliary warp scratch
  float red[kSC][4];                    // consumer reductions
  float inverse[kSMaxTopK];             // inverse normalisers of the staged routed activations
  float x_inverse;                      // inverse normaliser of the staged x
  int done[2][3];                       // tiles finished per layer parity: shared g/u, routed g/u, down
  unsigned epoch1;                      // launches completed before this one, plus one: scales every target
  volatile int routed_layers;           // layers whose routing table is in `routes` (set by the auxiliary warp)
  volatile int failed;
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for a global counter to reach `target`. One lane polls.
__device__ __forceinline__ bool wait_global(const unsigned* p, unsigned target, StackShared* sh) {
  if (sh->failed) return false;
  if (ld_acquire_u32(p) >= target) return true;
  const long long t0 = clock64();
  while (ld_acquire_u32(p) < target) {
    if (sh->failed) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      sh->failed = 1;
      return false;
    }
    __nanosleep(32);
  }
  return true;
}

// The same for a counter that other GPUs add to.
__device__ __forceinline__ bool wait_system(const unsigned* p, unsigned target, StackShared* sh) {
  if (sh->failed) return false;
  if (ld_acquire_sys_u32(p) >= target) return true;
  const long long t0 = clock64();
  while (ld_acquire_u32(p) < target || ld_acquire_sys_u32(p) < target) {   // cheap poll first, system-scope acquire to finish
    if (sh->failed) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      sh->failed = 1;
      return false;
    }
    __nanosleep(32);
  }
  return true;
}

// Bounded wait until this block's auxiliary warp has resolved the routing of `layer`.
__device__ __forceinline__ bool wait_routing(int layer, StackShared* sh) {
  if (sh->failed) return false;
  if (sh->routed_layers > layer) {
    __threadfence_block();
    return true;
  }
  const long long t0 = clock64();
  while (sh->routed_layers <= layer) {
    if (sh->failed) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      sh->failed = 1;
      return false;
    }
  }
  __threadfence_block();
  return true;
}

__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kSC * 32) : "memory");
}

// -------------------------------------------------------------------- router tail
// One warp. logits/scores of the layer are complete in global memory.
__device__ void stack_router_tail(const StackArgs& a, const StackLayer& ly, int layer, StackShared* sh) {
  const int lane = threadIdx.x & 31;
  const int par = layer & 1;
  const float* logit = a.logits + (size_t)par * (a.experts + a.n_shared);
  const float* scores = a.scores + (size_t)par * a.experts;
  float* score = sh->score;
  for (int e = lane; e < a.experts; e += 32) score[e] = __ldcg(scores + e);
  __syncwarp();
  int my_choice = 0;
#pragma unroll 1
  for (int r = 0; r < a.top_k; ++r) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll 1
    for (int e = lane; e < a.experts; e += 32) {
      const float v = score[e];
      if (v > best) {
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
    if (best_e == 0x7fffffff) best_e = r;
    if (lane == 0) score[best_e] = -INFINITY;
    if (lane == r) my_choice = best_e;
    __syncwarp();
  }
  const int n = a.top_k + a.n_shared;
  const bool live = lane < n;
  float l = 0.f;
  if (lane < a.top_k) l = __ldcg(logit + my_choice);
  else if (live) l = __ldcg(logit + a.experts + (lane - a.top_k));
  const float lp = live ? round_bf16(fminf(0.f, l) - log1pf(__expf(-fabsf(l)))) : -INFINITY;
  float m = lp;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (fabsf(m) == INFINITY) m = 0.f;
  const float ex = live ? round_bf16(__expf(round_bf16(lp - m))) : 0.f;
  float s = ex;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float lse = round_bf16(round_bf16(__logf(round_bf16(s))) + m);
  float w = round_bf16(__expf(round_bf16(lp - lse)));
  w = round_bf16(w * ly.route_scale);
  w = round_bf16(w * bf16_to_f32(ly.global_scale[0]));
  RouteTable* table = &sh->routes[layer & 1];
  const bool publish = blockIdx.x == 0;   // one block also writes the optional router outputs
  if (lane < a.top_k) {
    const int64_t* entry = ly.sources + (size_t)my_choice * kBank;
    RouteEntry r;
    r.gu_codes = reinterpret_cast<const uint8_t*>(entry[0]);
    r.gu_scales = reinterpret_cast<const uint8_t*>(entry[1]);
    r.gu_scale2 = r.gu_codes ? *reinterpret_cast<const float*>(entry[2]) : 0.f;
    r.dn_codes = reinterpret_cast<const uint8_t*>(entry[3]);
    r.dn_scales = reinterpret_cast<const uint8_t*>(entry[4]);
    r.dn_scale2 = r.dn_codes ? *reinterpret_cast<const float*>(entry[5]) : 0.f;
    r.weight = w;
    r.expert = my_choice;
    table->route[lane] = r;
    if (publish && ly.topk_indices) ly.topk_indices[lane] = my_choice;
    if (publish && ly.topk_weights) ly.topk_weights[lane] = (uint16_t)f32_to_bf16_bits(w);
  } else if (live) {
    table->gamma[lane - a.top_k] = w;
    if (publish && ly.gammas) ly.gammas[lane - a.top_k] = (uint16_t)f32_to_bf16_bits(w);
  }
  __syncwarp();
  if (lane == 0) {
    __threadfence_block();
    sh->routed_layers = layer + 1;   // the producer and the consumers of this block may read the table
  }
}

// ---------------------------------------------------------------- x staging (consumers)
// All consumer threads: `value` holds this thread's elements i = ct + n * (kSC*32) of the
// new activation vector (already BF16-rounded, as FP32). Writes BF16 and normalised FP16.
template <int D>
__device__ __forceinline__ void stage_x(uint16_t* s_x16, uint16_t* s_xbf, const float (&value)[(D + kSC * 32 - 1) / (kSC * 32)],
                                        float amax_bound, StackShared* sh, int ct) {
  // power-of-two normaliser from an upper bound of the largest magnitude
  float inverse;
  const uint32_t bits = f32_to_bf16_bits(amax_bound) & 0x7fffu;
  const float scale = pow2_normaliser(bits + 0x80u > 0x7f7fu ? 0x7f7fu : bits + 0x80u, &inverse);  // one binade of margin
  constexpr int PER = (D + kSC * 32 - 1) / (kSC * 32);
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = ct + n * (kSC * 32);
    if (i < D) {
      s_xbf[i] = (uint16_t)f32_to_bf16_bits(value[n]);
      const uint32_t h2 = f32x2_to_f16x2(value[n] * scale, 0.f);
      s_x16[i] = (uint16_t)(h2 & 0xffffu);
    }
  }
  if (ct == 0) sh->x_inverse = inverse;
}

template <int D, int F>
__global__ void __launch_bounds__(kSThreads, 1) moe_stack_kernel(StackArgs a) {
  using S = StackShape<D, F>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ StackShared sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char* slots = smem;
  unsigned char* staging = smem + kSStages * kSSlot;
  uint16_t* s_x16 = reinterpret_cast<uint16_t*>(staging);            // [D] FP16 normalised (gate/up phases)
  uint16_t* s_xbf = s_x16 + D;                                        // [D] BF16
  uint16_t* s_act = reinterpret_cast<uint16_t*>(staging);            // [top_k][F] FP16 normalised (down phases)
  uint16_t* s_sact = s_act + (size_t)kSMaxTopK * F;                   // [n_shared][F] BF16 (act * gamma)
  const TilePlan plan = make_plan<D, F>(a);
  const int total_rows = a.experts + a.n_shared;
  const int n_jobs = a.top_k + a.n_shared;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSStages; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    sh.routed_layers = 0;
    sh.failed = 0;
    sh.epoch1 = *a.epoch + 1u;
    for (int i = 0; i < 6; ++i) (&sh.done[0][0])[i] = 0;
    mbar_init_fence();
  }
  for (int i = threadIdx.x; i < (kSMaxTopK + kSMaxShared) * kSMaxRows; i += blockDim.x) (&sh.contrib[0][0])[i] = 0.f;
  __syncthreads();

  if (warp == 0) {
    // =========================================================== producer (one lane)
    // The tile list is walked with running counters: a division per tile on a single
    // thread would cost more than issuing the copy.
    if (lane == 0) {
      long long issued = 0;   // tiles issued so far (all layers)
      bool alive = true;
      // claims the next ring slot; false once a wait has given up
      auto next_slot = [&](unsigned char*& dst, uint64_t*& bar) -> bool {
        const int slot = (int)(issued % kSStages);
        if (sh.failed) return false;
        if (issued >= kSStages && !mbar_wait(&sh.empty[slot], (uint32_t)((issued / kSStages) - 1) & 1)) {
          sh.failed = 1;
          return false;
        }
        dst = slots + (size_t)slot * kSSlot;
        bar = &sh.full[slot];
        ++issued;
        return true;
      };
      unsigned char* dst = nullptr;
      uint64_t* bar = nullptr;
      constexpr int kQgPerJob = 2 * F / S::QG_ROWS;
      for (int layer = 0; layer < a.n_layers && alive; ++layer) {
        const StackLayer ly = a.layers[layer];
        const unsigned* sync = a.sync + (size_t)layer * kSyncWordsPerLayer;
        // ---- router rows, padded to a multiple of the consumer count
        for (int t = 0; t < plan.s_sg && alive; ++t) {
          if (!(alive = next_slot(dst, bar))) break;
          if (t < plan.n_r) {
            mbar_expect_tx(bar, S::R_BYTES);
            bulk_g2s(dst, ly.router_weight + (size_t)(plan.r0 + t) * D, S::R_BYTES, bar);
          } else {
            mbar_expect_tx(bar, 0);
          }
        }
        // ---- shared gate/up: blocks of kSC units, each unit SG_SPLIT column slabs
        for (int unit0 = 0; unit0 < plan.n_u && alive; unit0 += kSC) {
          for (int h = 0; h < S::SG_SPLIT && alive; ++h) {
            for (int s = 0; s < kSC; ++s) {
              if (!(alive = next_slot(dst, bar))) break;
              const int unit = unit0 + s;
              if (unit < plan.n_u) {
                const size_t row = (size_t)(plan.u0 + unit) * S::SG_PAIRS;   // over [n_shared * F]
                const size_t off = row * D + (size_t)h * S::SG_COLS;
                mbar_expect_tx(bar, 2 * S::SG_PART);
                bulk_g2s(dst, ly.shared_gate + off, S::SG_PART, bar);
                bulk_g2s(dst + S::SG_PART, ly.shared_up + off, S::SG_PART, bar);
              } else {
                mbar_expect_tx(bar, 0);
              }
            }
          }
        }
        if (!alive) break;
        // ---- routing of this layer: wait, then bring the table into shared memory
        INK_TRACE(layer, kTrProdRouteWait);
        if (!wait_routing(layer, &sh)) break;
        INK_TRACE(layer, kTrProdRouteGot);
        const RouteTable& table = sh.routes[layer & 1];
        // ---- routed gate/up
        {
          int choice = plan.q0 / kQgPerJob, row0 = (plan.q0 % kQgPerJob) * S::QG_ROWS;
          for (int t = 0; t < plan.n_q; ++t) {
            if (!(alive = next_slot(dst, bar))) break;
            const RouteEntry& r = table.route[choice];
            if (r.gu_codes) {
              mbar_expect_tx(bar, S::QG_CODES + S::QG_SCALES);
              bulk_g2s(dst, r.gu_codes + (size_t)row0 * (D / 2), S::QG_CODES, bar);
              bulk_g2s(dst + S::QG_CODES, r.gu_scales + (size_t)row0 * (D / 16), S::QG_SCALES, bar);
            } else {
              mbar_expect_tx(bar, 0);
            }
            row0 += S::QG_ROWS;
            if (row0 == 2 * F) {
              row0 = 0;
              ++choice;
            }
          }
        }
        // ---- shared down: expert-major, then row group, then the tiles of a group
        for (int e = 0; e < a.n_shared && alive; ++e) {
          const uint16_t* w = ly.shared_down + ((size_t)e * D + (size_t)plan.g0 * S::RT) * F;
          for (int t = 0; t < plan.n_g * S::SD_PER_GROUP; ++t) {
            if (!(alive = next_slot(dst, bar))) break;
            mbar_expect_tx(bar, S::SD_BYTES);
            bulk_g2s(dst, w + (size_t)t * S::SD_ROWS * F, S::SD_BYTES, bar);
          }
        }
        // ---- routed down: choice-major, then row group
        for (int choice = 0; choice < a.top_k && alive; ++choice) {
          const RouteEntry& r = table.route[choice];
          for (int g = 0; g < plan.n_g; ++g) {
            if (!(alive = next_slot(dst, bar))) break;
            if (r.dn_codes) {
              const size_t row0 = (size_t)(plan.g0 + g) * S::RT;
              mbar_expect_tx(bar, S::QD_CODES + S::QD_SCALES);
              bulk_g2s(dst, r.dn_codes + row0 * (F / 2), S::QD_CODES, bar);
              bulk_g2s(dst + S::QD_CODES, r.dn_scales + row0 * (F / 16), S::QD_SCALES, bar);
            } else {
              mbar_expect_tx(bar, 0);
            }
          }
        }
        // ---- padding up to a multiple of the consumer count
        for (int t = plan.s_pad; t < plan.per_layer && alive; ++t) {
          if (!(alive = next_slot(dst, bar))) break;
          mbar_expect_tx(bar, 0);
        }
        INK_TRACE(layer, kTrProdLayerIssued);
      }
    }
  } else if (warp == kSC + 1) {
    // =========================================================== auxiliary warp
    for (int layer = 0; layer < a.n_layers; ++layer) {
      const unsigned* sync = a.sync + (size_t)layer * kSyncWordsPerLayer;
      // every block resolves the routing for itself (same inputs, same arithmetic, same result): the
      // code stays warm in this SM's instruction cache and nothing has to be published between blocks
      bool ok = true;
      if (lane == 0) ok = wait_global(sync + kRouterRows, sh.epoch1 * (unsigned)(a.experts + a.n_shared), &sh);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      stack_router_tail(a, a.layers[layer], layer, &sh);
      if (sh.failed) break;
    }
  } else {
    // =========================================================== consumers
    const int cw = warp - 1, ct = threadIdx.x - 32;
    constexpr int PER = (D + kSC * 32 - 1) / (kSC * 32);
    long long base = 0;   // index of this layer's first tile in the block's whole sequence

    // first tile index >= start that belongs to this consumer (tile t belongs to consumer t % kSC)
    auto first_of = [&](int start) -> int { return start + (cw - start % kSC + kSC) % kSC; };
    auto take = [&](int t, const unsigned char*& src, int& slot) -> bool {
      const long long i = base + t;
      slot = (int)(i % kSStages);
      bool ok = !sh.failed;
      if (ok) ok = mbar_wait(&sh.full[slot], (uint32_t)(i / kSStages) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        sh.failed = 1;
        return false;
      }
      src = slots + (size_t)slot * kSSlot;
      return true;
    };
    auto release = [&](int slot) {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.empty[slot]);
    };
    // one more tile of `section` (0 shared g/u, 1 routed g/u, 2 down) of this block is done;
    // returns true in the warp that finished the section's last tile
    // `fence`: this was the warp's last tile of the section, so everything the warp wrote to
    // global memory for the section is pushed out before the count moves (a fence per tile
    // costs more than the tile).
    auto section_done = [&](int layer, int section, int n_tiles, bool fence) -> bool {
      int done = 0;
      __syncwarp();
      if (lane == 0) {
        if (fence) __threadfence();
        done = atomicAdd(&sh.done[layer & 1][section], 1) + 1;
      }
      done = __shfl_sync(0xffffffffu, done, 0);
      return done == n_tiles;
    };

    // ---- first activation vector
    {
      float value[PER];
      float amax = 0.f;
#pragma unroll
      for (int n = 0; n < PER; ++n) {
        const int i = ct + n * (kSC * 32);
        value[n] = i < D ? bf16_to_f32(a.x[i]) : 0.f;
        amax = fmaxf(amax, fabsf(value[n]));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (lane == 0) sh.red[cw][0] = amax;
      consumer_sync();
      amax = 0.f;
      for (int w = 0; w < kSC; ++w) amax = fmaxf(amax, sh.red[w][0]);
      stage_x<D>(s_x16, s_xbf, value, amax, &sh, ct);
      consumer_sync();
    }

    for (int layer = 0; layer < a.n_layers; ++layer, base += plan.per_layer) {
      const float* router_bias = a.layers[layer].router_bias;
      const uint16_t* norm_weight = a.layers[layer].norm_weight;
      unsigned* sync = a.sync + (size_t)layer * kSyncWordsPerLayer;
      const int par = layer & 1;
      const unsigned epoch1 = sh.epoch1;
      // slot of the ranks' deliveries: alternates with every block of every launch
      const int xpar = (int)(((epoch1 - 1u) * (unsigned)a.n_layers + (unsigned)layer) & 1u);
      float* inbox = a.inbox + (size_t)xpar * a.world * D;
      const unsigned down_target = epoch1 * gridDim.x * (unsigned)a.world;
      const float x_inverse = sh.x_inverse;
      const bool tracer = (ct == 0);
      if (tracer) INK_TRACE(layer, kTrLayerStart);
      // blocks that own no tile of a section still have to be counted
      if (ct == 0) {
        if (plan.n_sg == 0) red_release_add(sync + kShGuDone, 1u);
        if (plan.n_q == 0) red_release_add(sync + kRtGuDone, 1u);
        if (plan.n_sd + plan.n_qd == 0) {
          if (a.world > 1)
            for (int r = 0; r < a.world; ++r) red_release_sys_add(a.peer_xsync[r] + layer, 1u);
          else
            red_release_add(a.xsync + layer, 1u);
        }
      }
      // ------------------------------------------------ router rows
      for (int t = first_of(plan.s_r); t < plan.s_sg; t += kSC) {
        const unsigned char* src;
        int slot;
        if (!take(t, src, slot)) break;
        if (t < plan.n_r) {
          float acc = 0.f;
#pragma unroll 2
          for (int c = 0; c < S::R_CPL; ++c) {
            const int chunk = c * 32 + lane;
            acc = dot8(*reinterpret_cast<const uint4*>(src + chunk * 16), reinterpret_cast<const uint4*>(s_xbf)[chunk], acc);
          }
          acc = warp_sum(acc);
          release(slot);
          const int row = plan.r0 + t;
          if (lane == 0) {
            const float l = round_bf16(acc);
            a.logits[(size_t)par * total_rows + row] = l;
            if (row < a.experts)
              a.scores[(size_t)par * a.experts + row] = round_bf16(1.f / (1.f + __expf(-l))) + router_bias[row];
            __threadfence();
            const unsigned done = atomicAdd(sync + kRouterRows, 1u) + 1u;
            (void)done;
          }
        } else {
          release(slot);
        }
      }
      if (tracer) INK_TRACE(layer, kTrRouterDone);
      // ------------------------------------------------ shared gate/up
      {
        float g[S::SG_PAIRS], u[S::SG_PAIRS];
        for (int t = first_of(plan.s_sg); t < plan.s_qg; t += kSC) {
          const unsigned char* src;
          int slot;
          if (!take(t, src, slot)) break;
          const int i = t - plan.s_sg;
          const int h = (i / kSC) % S::SG_SPLIT, blk = i / (kSC * S::SG_SPLIT);
          const int unit = blk * kSC + cw;
          if (unit < plan.n_u) {
            if (h == 0) {
#pragma unroll
              for (int p = 0; p < S::SG_PAIRS; ++p) g[p] = u[p] = 0.f;
            }
            const uint4* xs = reinterpret_cast<const uint4*>(s_xbf + h * S::SG_COLS);
            // short loop bodies on purpose: straight-line code as long as a tile does not fit the
            // instruction cache close to the schedulers, and fetching it becomes the bottleneck
#pragma unroll
            for (int p = 0; p < S::SG_PAIRS; ++p) {
#pragma unroll 2
              for (int c = 0; c < S::SG_CPL; ++c) {
                const int chunk = c * 32 + lane;
                const uint4 xv = xs[chunk];
                g[p] = dot8(*reinterpret_cast<const uint4*>(src + (size_t)p * S::SG_COLS * 2 + chunk * 16), xv, g[p]);
                u[p] = dot8(*reinterpret_cast<const uint4*>(src + S::SG_PART + (size_t)p * S::SG_COLS * 2 + chunk * 16), xv, u[p]);
              }
            }
            release(slot);
            if (h == S::SG_SPLIT - 1) {
              float gate = multi_reduce<S::SG_PAIRS>(g, lane);
              float up = multi_reduce<S::SG_PAIRS>(u, lane);
              if (reduced_owner<S::SG_PAIRS>(lane)) {
                gate = round_bf16(gate);
                up = round_bf16(up);
                const float act = round_bf16(gate / (1.f + expf(-gate)));
                const int pair = (plan.u0 + unit) * S::SG_PAIRS + reduced_row<S::SG_PAIRS>(lane);  // over [n_shared * F]
                a.shared_activated[(size_t)par * a.n_shared * F + pair] = (uint16_t)f32_to_bf16_bits(act * up);
              }
            }
          } else {
            release(slot);
          }
          if (section_done(layer, 0, plan.n_sg, t + kSC >= plan.s_qg) && lane == 0) red_release_add(sync + kShGuDone, 1u);
        }
      }
      if (tracer) INK_TRACE(layer, kTrShGuDone);
      // ------------------------------------------------ routed gate/up
      {
        uint32_t xr[S::QG_CPL][16];
#pragma unroll
        for (int j = 0; j < S::QG_CPL; ++j) {
          const uint4* p4 = reinterpret_cast<const uint4*>(s_x16 + (j * 32 + lane) * 32);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint4 t4 = p4[v];
            xr[j][4 * v + 0] = t4.x; xr[j][4 * v + 1] = t4.y; xr[j][4 * v + 2] = t4.z; xr[j][4 * v + 3] = t4.w;
          }
        }
        const int per_job = 2 * F / S::QG_ROWS;
        for (int t = first_of(plan.s_qg); t < plan.s_sd; t += kSC) {
          const unsigned char* src;
          int slot;
          if (!take(t, src, slot)) break;
          const int q = plan.q0 + (t - plan.s_qg);
          const int choice = q / per_job, row0 = (q % per_job) * S::QG_ROWS;
          const RouteEntry r = sh.routes[par].route[choice];
          if (r.gu_codes) {
            const float scale = r.gu_scale2 * x_inverse;
            uint16_t* y = a.activated + ((size_t)par * a.top_k + choice) * F + row0 / 2;
            float gate = 0.f;
#pragma unroll 1
            for (int row = 0; row < S::QG_ROWS; ++row) {   // even rows are gate, odd rows up
              const unsigned char* codes = src + (size_t)row * (D / 2) + lane * 16;
              const unsigned char* scales = src + S::QG_CODES + (size_t)row * (D / 16) + lane * 2;
              float acc = 0.f;
#pragma unroll
              for (int j = 0; j < S::QG_CPL; ++j)
                acc += dot32(*reinterpret_cast<const uint4*>(codes + j * 512), *reinterpret_cast<const uint16_t*>(scales + j * 64), xr[j]);
              acc = warp_sum(acc) * scale;
              if ((row & 1) == 0) gate = acc;
              else if (lane == 0) y[row >> 1] = (uint16_t)f32_to_bf16_bits(silu_mul(gate, acc));
            }
            release(slot);
          } else {
            release(slot);
          }
          if (section_done(layer, 1, plan.n_q, t + kSC >= plan.s_sd) && lane == 0) red_release_add(sync + kRtGuDone, 1u);
        }
      }
      if (tracer) INK_TRACE(layer, kTrRtGuDone);
      // every consumer of this block is past its gate/up tiles: x staging may be overwritten
      consumer_sync();
      // ------------------------------------------------ shared down
      if (lane == 0) {
        wait_global(sync + kShGuDone, epoch1 * gridDim.x, &sh);
        wait_routing(layer, &sh);
      }
      __syncwarp();
      if (tracer) INK_TRACE(layer, kTrShGuAll);
      if (!sh.failed) {
        for (int e = cw; e < a.n_shared; e += kSC) {
          const uint16_t* src = a.shared_activated + ((size_t)par * a.n_shared + e) * F;
          const float gamma = sh.routes[par].gamma[e];
          uint32_t* dst = reinterpret_cast<uint32_t*>(s_sact + (size_t)e * F);
          for (int i = lane; i < F / 2; i += 32) {
            const uint32_t v = __ldcg(reinterpret_cast<const uint32_t*>(src) + i);
            dst[i] = f32_to_bf16_bits(bf16lo(v) * gamma) | (f32_to_bf16_bits(bf16hi(v) * gamma) << 16);
          }
        }
      }
      consumer_sync();
      for (int t = first_of(plan.s_sd); t < plan.s_qd; t += kSC) {
        const unsigned char* src;
        int slot;
        if (!take(t, src, slot)) break;
        const int i = t - plan.s_sd;
        const int per_e = plan.n_g * S::SD_PER_GROUP;
        const int e = i / per_e, rem = i % per_e;
        const int local0 = (rem / S::SD_PER_GROUP) * S::RT + (rem % S::SD_PER_GROUP) * S::SD_ROWS;
        const uint4* xs = reinterpret_cast<const uint4*>(s_sact + (size_t)e * F);
#pragma unroll 1
        for (int row = 0; row < S::SD_ROWS; ++row) {
          float acc = 0.f;
#pragma unroll 2
          for (int c = 0; c < S::SD_CPL; ++c) {
            const int chunk = c * 32 + lane;
            acc = dot8(*reinterpret_cast<const uint4*>(src + (size_t)row * F * 2 + chunk * 16), xs[chunk], acc);
          }
          acc = warp_sum(acc);
          if (lane == 0) sh.contrib[a.top_k + e][local0 + row] = round_bf16(acc);
        }
        release(slot);
        // down tiles are counted together (shared + routed)
        section_done(layer, 2, plan.n_sd + plan.n_qd, false);
      }
      if (tracer) INK_TRACE(layer, kTrShDownDone);
      // ------------------------------------------------ routed down
      if (lane == 0) wait_global(sync + kRtGuDone, epoch1 * gridDim.x, &sh);
      __syncwarp();
      if (tracer) INK_TRACE(layer, kTrRtGuAll);
      if (!sh.failed) {
        for (int job = cw; job < a.top_k; job += kSC) {
          const float inverse = warp_stage_f16(a.activated + ((size_t)par * a.top_k + job) * F, s_act + (size_t)job * F, F, lane);
          if (lane == 0) sh.inverse[job] = inverse;
        }
      }
      consumer_sync();
      if (tracer) INK_TRACE(layer, kTrActStaged);
      {
        const int sl = lane % S::LPR, rp = lane / S::LPR;
        uint32_t xr[S::QD_CPL][16];
        int loaded = -1;
        bool last_of_block = false;
        for (int t = first_of(plan.s_qd); t < plan.s_pad; t += kSC) {
          const unsigned char* src;
          int slot;
          if (!take(t, src, slot)) break;
          const int i = t - plan.s_qd;
          const int choice = i / plan.n_g, local0 = (i % plan.n_g) * S::RT;
          const RouteEntry r = sh.routes[par].route[choice];
          if (r.dn_codes) {
            if (loaded != choice) {
              loaded = choice;
#pragma unroll
              for (int j = 0; j < S::QD_CPL; ++j) {
                const uint4* p4 = reinterpret_cast<const uint4*>(s_act + (size_t)choice * F + (j * S::LPR + sl) * 32);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  const uint4 t4 = p4[v];
                  xr[j][4 * v + 0] = t4.x; xr[j][4 * v + 1] = t4.y; xr[j][4 * v + 2] = t4.z; xr[j][4 * v + 3] = t4.w;
                }
              }
            }
            const float scale = r.dn_scale2 * sh.inverse[choice];
#pragma unroll 1
            for (int p = 0; p < S::PASSES; ++p) {
              const int row = p * S::RPP + rp;
              float acc = 0.f;
#pragma unroll
              for (int j = 0; j < S::QD_CPL; ++j) {
                const int chunk = j * S::LPR + sl;
                acc += dot32(*reinterpret_cast<const uint4*>(src + (size_t)row * (F / 2) + chunk * 16),
                             *reinterpret_cast<const uint16_t*>(src + S::QD_CODES + (size_t)row * (F / 16) + chunk * 2), xr[j]);
              }
#pragma unroll
              for (int o = S::LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
              if (sl == 0) {
                const float down = round_bf16(acc * scale);
                sh.contrib[choice][local0 + row] = round_bf16(down * r.weight);
              }
            }
            release(slot);
          } else {
            release(slot);
          }
          if (section_done(layer, 2, plan.n_sd + plan.n_qd, false)) last_of_block = true;
        }
        // padding tiles at the end of the layer
        for (int t = first_of(plan.s_pad); t < plan.per_layer; t += kSC) {
          const unsigned char* src;
          int slot;
          if (!take(t, src, slot)) break;
          release(slot);
        }
        // The warp that finished the block's last down tile sums the contributions in a
        // fixed order (routes in choice order, then the shared experts) and publishes them.
        // (Routed-down tiles start only after every shared-down tile of the block is done, so
        // the last tile is always a routed one.)
        if (last_of_block && !sh.failed) {
          __syncwarp();
          // deliver this block's rows to every rank (itself included), then count the block there
          for (int row = lane; row < plan.n_g * S::RT; row += 32) {
            float total = 0.f;
            for (int j = 0; j < n_jobs; ++j) total += sh.contrib[j][row];
            const size_t at = ((size_t)xpar * a.world + a.rank) * D + (size_t)plan.g0 * S::RT + row;
            for (int r = 0; r < a.world; ++r) a.peer_inbox[r][at] = total;
          }
          __syncwarp();
          if (lane == 0) {
            if (a.world > 1) {
              __threadfence_system();
              for (int r = 0; r < a.world; ++r) red_release_sys_add(a.peer_xsync[r] + layer, 1u);
            } else {
              __threadfence();
              red_release_add(a.xsync + layer, 1u);
            }
          }
        }
      }
      if (tracer) INK_TRACE(layer, kTrRtDownDone);
      // every block of every rank has delivered this layer's rows
      if (lane == 0) {
        if (a.world > 1) wait_system(a.xsync + layer, down_target, &sh);
        else wait_global(a.xsync + layer, down_target, &sh);
      }
      __syncwarp();
      if (tracer) INK_TRACE(layer, kTrDownAll);
      if (!a.glue) {
        // one block only: each block writes the sum over the ranks of its own rows
        if (!sh.failed)
          for (int row = ct; row < plan.n_g * S::RT; row += kSC * 32) {
            const size_t i = (size_t)plan.g0 * S::RT + row;
            float total = 0.f;
            for (int r = 0; r < a.world; ++r) total += __ldcg(inbox + (size_t)r * D + i);
            a.partial[i] = total;
          }
        break;
      }
      // ------------------------------------------------ residual add + RMS norm (every block, redundantly)
      float value[PER];
      {
        const uint16_t* res_in = a.residual + (size_t)par * D;
        uint16_t* res_out = a.residual + (size_t)(par ^ 1) * D;
        float sumsq = 0.f, amax_h = 0.f, amax_w = 0.f;
        // all loads first (they are independent), arithmetic after: one L2 round trip, not PER
        const bool live = !sh.failed;
        const int world = a.world;
        uint16_t res[PER], nw[PER];
        float part[PER];
#pragma unroll
        for (int n = 0; n < PER; ++n) {
          const int i = ct + n * (kSC * 32);
          const bool ok = live && i < D;
          res[n] = ok ? __ldcg(res_in + i) : (uint16_t)0;
          // every rank's delivery, summed in rank order (same bits on every rank); predicated loads of a
          // fixed trip count so that they all issue before the first add
          float got[kSMaxWorld];
#pragma unroll
          for (int r = 0; r < kSMaxWorld; ++r) got[r] = (ok && r < world) ? __ldcg(inbox + (size_t)r * D + i) : 0.f;
          float sum = 0.f;
#pragma unroll
          for (int r = 0; r < kSMaxWorld; ++r) sum += got[r];
          part[n] = sum;
          nw[n] = ok ? norm_weight[i] : (uint16_t)0;
        }
#pragma unroll
        for (int n = 0; n < PER; ++n) {
          const int i = ct + n * (kSC * 32);
          const float h = round_bf16(bf16_to_f32(res[n]) + round_bf16(part[n]));
          value[n] = h;
          sumsq = fmaf(h, h, sumsq);
          amax_h = fmaxf(amax_h, fabsf(h));
          amax_w = fmaxf(amax_w, fabsf(bf16_to_f32(nw[n])));
          if (blockIdx.x == 0 && live && i < D) {
            res_out[i] = (uint16_t)f32_to_bf16_bits(h);
            if (layer + 1 == a.n_layers) a.partial[i] = part[n];
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
          amax_h = fmaxf(amax_h, __shfl_xor_sync(0xffffffffu, amax_h, o));
          amax_w = fmaxf(amax_w, __shfl_xor_sync(0xffffffffu, amax_w, o));
        }
        if (lane == 0) {
          sh.red[cw][0] = sumsq;
          sh.red[cw][1] = amax_h;
          sh.red[cw][2] = amax_w;
        }
        consumer_sync();   // also: every consumer is past its down tiles, staging may be overwritten
        sumsq = 0.f;
        amax_h = 0.f;
        amax_w = 0.f;
        for (int w = 0; w < kSC; ++w) {
          sumsq += sh.red[w][0];
          amax_h = fmaxf(amax_h, sh.red[w][1]);
          amax_w = fmaxf(amax_w, sh.red[w][2]);
        }
        const float scale = rsqrtf(sumsq / (float)D + a.eps);
#pragma unroll
        for (int n = 0; n < PER; ++n) {
          const int i = ct + n * (kSC * 32);
          if (i < D) value[n] = round_bf16(round_bf16(value[n] * scale) * bf16_to_f32(nw[n]));
        }
        if (layer + 1 == a.n_layers) {
          if (blockIdx.x == 0) {
#pragma unroll
            for (int n = 0; n < PER; ++n) {
              const int i = ct + n * (kSC * 32);
              if (i < D) a.normed_out[i] = (uint16_t)f32_to_bf16_bits(value[n]);
            }
          }
        } else {
          stage_x<D>(s_x16, s_xbf, value, amax_h * scale * amax_w, &sh, ct);
          // contributions of inactive routes must read as zero in the next layer too
          for (int i = ct; i < (kSMaxTopK + kSMaxShared) * kSMaxRows; i += kSC * 32) (&sh.contrib[0][0])[i] = 0.f;
          if (ct < 3) sh.done[par ^ 1][ct] = 0;
        }
        consumer_sync();
        if (tracer) INK_TRACE(layer, kTrNormDone);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && sh.failed && a.status) atomicOr(a.status, kFlagWaitTimedOut);
  // Every block read the epoch before it could pass any counter, and block 0 gets here only after
  // the last counter of the launch, so this store cannot be seen by a block of the same launch.
  if (threadIdx.x == 0 && blockIdx.x == 0) *a.epoch = sh.epoch1;
}

// ------------------------------------------------------------------- host side
template <int D, int F>
static int launch_stack(const StackArgs& a, cudaStream_t stream) {
  using S = StackShape<D, F>;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_stack_kernel<D, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "moe_stack: %d bytes of shared memory refused: %s", S::SMEM,
                cudaGetErrorString(e));
    INK_PREFER_MAX_SMEM((moe_stack_kernel<D, F>));
    int device = 0, coop = 0, per_sm = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
    INK_REQUIRE(coop, kLaunchFailed, "moe_stack: the device cannot launch cooperative kernels");
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_stack_kernel<D, F>, kSThreads, S::SMEM);
    INK_REQUIRE(e == cudaSuccess && per_sm >= 1, kLaunchFailed, "moe_stack: the kernel does not fit on an SM");
    configured = true;
  }
  const int groups = D / S::RT;
  const int rows_per_block = ((groups + sms - 1) / sms) * S::RT;
  INK_REQUIRE(rows_per_block <= kSMaxRows, kUnsupportedShape, "moe_stack: %d output rows per block", rows_per_block);
  StackArgs args = a;
  void* params[] = {&args};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)moe_stack_kernel<D, F>, dim3(sms), dim3(kSThreads), params,
                                  (size_t)S::SMEM, stream);
  INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "moe_stack: launch failed: %s", cudaGetErrorString(e));
  return kOk;
}

}  // namespace ink

using namespace ink;

extern "C" size_t ink_moe_stack_layer_bytes(void) { return sizeof(StackLayer); }

static size_t pad256(size_t n) { return (n + 255) / 256 * 256; }

// The region other ranks write into: delivered-block counters, then the delivered rows.
extern "C" size_t ink_moe_stack_symmetric_bytes(int n_layers, int hidden, int world) {
  return pad256(sizeof(unsigned) * (size_t)n_layers) + pad256(sizeof(float) * 2 * (size_t)world * hidden);
}

extern "C" size_t ink_moe_stack_scratch_bytes(int n_layers, int hidden, int intermediate, int experts, int n_shared,
                                              int top_k) {
  size_t bytes = 0;
  bytes += pad256(sizeof(unsigned) * kSyncWordsPerLayer * (size_t)n_layers);   // sync
  bytes += pad256(sizeof(unsigned));                                            // epoch
  bytes += pad256(sizeof(RouteTable) * (size_t)n_layers);                       // routes
  bytes += pad256(sizeof(float) * 2 * (size_t)(experts + n_shared));            // logits
  bytes += pad256(sizeof(float) * 2 * (size_t)experts);                         // scores
  bytes += pad256(2 * 2 * (size_t)top_k * intermediate);                        // activated
  bytes += pad256(2 * 2 * (size_t)n_shared * intermediate);                     // shared activated
  bytes += pad256(2 * 2 * (size_t)hidden);                                      // residual double buffer
  bytes += ink_moe_stack_symmetric_bytes(n_layers, hidden, 1);                  // deliveries when there is one rank
  bytes += pad256(sizeof(unsigned long long) * (size_t)n_layers * kTraceBlocks * kTraceSlots);   // phase stamps (tracing)
  return bytes;
}

extern "C" size_t ink_moe_stack_trace_offset(int n_layers, int hidden, int intermediate, int experts,
                                             int n_shared, int top_k) {
  return ink_moe_stack_scratch_bytes(n_layers, hidden, intermediate, experts, n_shared, top_k) -
         pad256(sizeof(unsigned long long) * (size_t)n_layers * kTraceBlocks * kTraceSlots);
}

static int stack_decode(const void* layers, int n_layers, const void* x, void* residual_io, void* normed_out,
                        float* partial_out, int glue, float eps, int hidden, int intermediate, int experts,
                        int n_shared, int top_k, void* scratch, size_t scratch_bytes, int rank, int world,
                        const uint64_t* peer_regions, int32_t* status, ink_stream_t stream) {
  INK_REQUIRE(layers && x && partial_out && scratch, kBadArgument, "moe_stack: null pointer argument");
  INK_REQUIRE(n_layers >= 1 && (glue == 0 || glue == 1), kBadArgument, "moe_stack: n_layers=%d glue=%d", n_layers, glue);
  INK_REQUIRE(glue || n_layers == 1, kBadArgument, "moe_stack: without the glue only one block can run");
  INK_REQUIRE(!glue || (residual_io && normed_out), kBadArgument, "moe_stack: glue mode needs residual and normed buffers");
  INK_REQUIRE(top_k >= 1 && top_k <= kSMaxTopK && n_shared >= 0 && n_shared <= kSMaxShared && experts >= top_k &&
                  experts <= kSMaxExperts && top_k + n_shared <= 32,
              kUnsupportedShape, "moe_stack: experts=%d top_k=%d n_shared=%d unsupported", experts, top_k, n_shared);
  INK_REQUIRE(world >= 1 && world <= kSMaxWorld && rank >= 0 && rank < world && (world == 1 || peer_regions), kBadArgument,
              "moe_stack: rank=%d world=%d", rank, world);
  INK_REQUIRE(scratch_bytes >= ink_moe_stack_scratch_bytes(n_layers, hidden, intermediate, experts, n_shared, top_k),
              kBadArgument, "moe_stack: scratch of %zu bytes is too small", scratch_bytes);
  INK_REQUIRE(aligned16(x) && aligned16(scratch) && aligned16(partial_out), kMisaligned, "moe_stack: misaligned buffer");
  StackArgs a;
  a.layers = (const StackLayer*)layers;
  a.n_layers = n_layers;
  a.experts = experts;
  a.n_shared = n_shared;
  a.top_k = top_k;
  a.glue = glue;
  a.eps = eps;
  a.x = (const uint16_t*)x;
  a.normed_out = (uint16_t*)normed_out;
  a.partial = partial_out;
  a.status = status;
  a.rank = rank;
  a.world = world;
  char* p = (char*)scratch;
  auto take = [&](size_t n) { char* q = p; p += pad256(n); return q; };
  a.sync = (unsigned*)take(sizeof(unsigned) * kSyncWordsPerLayer * (size_t)n_layers);
  a.epoch = (unsigned*)take(sizeof(unsigned));
  a.routes = (RouteTable*)take(sizeof(RouteTable) * (size_t)n_layers);
  a.logits = (float*)take(sizeof(float) * 2 * (size_t)(experts + n_shared));
  a.scores = (float*)take(sizeof(float) * 2 * (size_t)experts);
  a.activated = (uint16_t*)take(2 * 2 * (size_t)top_k * intermediate);
  a.shared_activated = (uint16_t*)take(2 * 2 * (size_t)n_shared * intermediate);
  a.residual = (uint16_t*)take(2 * 2 * (size_t)hidden);
  char* own_region = take(ink_moe_stack_symmetric_bytes(n_layers, hidden, 1));
  for (int r = 0; r < kSMaxWorld; ++r) {
    a.peer_inbox[r] = nullptr;
    a.peer_xsync[r] = nullptr;
  }
  const size_t counters = pad256(sizeof(unsigned) * (size_t)n_layers);
  for (int r = 0; r < world; ++r) {
    char* region = world == 1 ? own_region : (char*)(uintptr_t)peer_regions[r];
    INK_REQUIRE(region != nullptr && aligned16(region), kBadArgument, "moe_stack: bad region for rank %d", r);
    a.peer_xsync[r] = (unsigned*)region;
    a.peer_inbox[r] = (float*)(region + counters);
  }
  a.xsync = a.peer_xsync[rank];
  a.inbox = a.peer_inbox[rank];
  // INKLING_STACK_TRACE=1: blocks stamp their phase boundaries (global nanosecond timer) into the
  // tail of the scratch, where ink_moe_stack_trace_offset() says
  const char* tracing = getenv("INKLING_STACK_TRACE");
  a.trace = (tracing && tracing[0] == '1') ? (unsigned long long*)p : nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  if (glue) {
    // the residual stream enters through slot 0 of the double buffer and leaves through residual_io
    cudaError_t e = cudaMemcpyAsync(a.residual, residual_io, 2 * (size_t)hidden, cudaMemcpyDeviceToDevice, s);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "moe_stack: copy failed: %s", cudaGetErrorString(e));
  }
  int rc = kUnsupportedShape;
  bool built = false;
#define INK_STACK_CASE(DD, FF)                   \
  if (hidden == DD && intermediate == FF) {      \
    built = true;                                \
    rc = launch_stack<DD, FF>(a, s);             \
  }
  INK_STACK_CASE(4096, 2048)
  INK_STACK_CASE(4096, 1024)
  INK_STACK_CASE(4096, 512)
  INK_STACK_CASE(4096, 256)
  INK_STACK_CASE(2048, 256)
  INK_STACK_CASE(1024, 512)
#undef INK_STACK_CASE
  if (!built) set_error("moe_stack: hidden=%d intermediate=%d is not a built shape", hidden, intermediate);
  if (rc != kOk) return rc;
  if (glue) {
    cudaError_t e = cudaMemcpyAsync(residual_io, a.residual + (size_t)(n_layers & 1) * hidden, 2 * (size_t)hidden,
                                    cudaMemcpyDeviceToDevice, s);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "moe_stack: copy failed: %s", cudaGetErrorString(e));
  }
  return kOk;
}

extern "C" int ink_moe_stack_decode(const void* layers, int n_layers, const void* x, void* residual_io,
                                    void* normed_out, float* partial_out, int glue, float eps, int hidden,
                                    int intermediate, int experts, int n_shared, int top_k, void* scratch,
                                    size_t scratch_bytes, int32_t* status, ink_stream_t stream) {
  return stack_decode(layers, n_layers, x, residual_io, normed_out, partial_out, glue, eps, hidden, intermediate,
                      experts, n_shared, top_k, scratch, scratch_bytes, 0, 1, nullptr, status, stream);
}

extern "C" int ink_moe_stack_decode_tp(const void* layers, int n_layers, const void* x, void* residual_io,
                                       void* normed_out, float* partial_out, int glue, float eps, int hidden,
                                       int intermediate, int experts, int n_shared, int top_k, void* scratch,
                                       size_t scratch_bytes, int rank, int world, const uint64_t* peer_regions,
                                       int32_t* status, ink_stream_t stream) {
  return stack_decode(layers, n_layers, x, residual_io, normed_out, partial_out, glue, eps, hidden, intermediate,
                      experts, n_shared, top_k, scratch, scratch_bytes, rank, world, peer_regions, status, stream);
}

// One persistent cooperative kernel for a whole stack of MoE blocks at decode (one
// token): router, expert plan, routed NVFP4 and shared BF16 gate/up, down + combine and
// the residual add + RMS norm between blocks, all inside one launch; with several
// tensor-parallel ranks also the all-reduce of every block (stores into the peers' inboxes).
//
// One block per SM. Warp 0 is the producer: it walks the block's tile list, layer after
// layer, and keeps a 16-slot shared-memory ring full with bulk asynchronous copies; it
// never waits for arithmetic, only for a free slot and -- before the first routed tile
// of a layer -- for that layer's routing. Warps 1..8 are consumers: consumer c takes
// tiles c, c+8, ... (the ring depth is a multiple of the consumer count, see the ring
// comment in stream_decode.cu). Warp 9 is the auxiliary warp: in every block it resolves
// the layer's routing (top-k, weight chain, bank addresses) from the scores all blocks
// wrote. The gate/up phases of a layer are ordered across blocks by counters in global memory
// (shared gate/up done, routed gate/up done); the weight stream itself never stops at them,
// because weight addresses do not depend on activations. Counters only grow: every target is a
// multiple of the number of launches so far, nothing is cleared, comparisons are modulo 2^32.
// What one block hands to all others in small pieces -- router scores, output rows -- travels
// as 8-byte words {FP32 value, tag of this launch and layer}: the reader polls the word it is
// about to use, so there is no fence, no counter and no last-arrival serialisation on that
// path, within a GPU and across GPUs alike (an aligned 8-byte store is one transaction).
//
// Template parameter TC selects how the routed experts are computed: on the CUDA cores
// (codes converted in registers, packed FP16 FMAs) or on the tensor cores (tc_path.cuh:
// eight more warps, the auxiliary warp issues the MMAs).
//
// Every wait (ring slot, routing flag, counter) is bounded; a wait that gives up sets
// kFlagWaitTimedOut in the status word, marks the launch as failed and every loop
// drains without further waiting.
#include <stdlib.h>
#include <string.h>

#include "../../include/inkling_b200.h"
#include "common.cuh"
#include "decode_args.cuh"
#include "pipe.cuh"
#include "stream_math.cuh"
#include "tc_path.cuh"

namespace ink {

constexpr int kSC = 8;                                 // consumer warps
constexpr int kSStages = 2 * kSC;                      // ring slots
constexpr unsigned kProducerLanes = (1u << kSStages) - 1u;   // the lanes of the producer warp that own a slot
constexpr int kSSlot = 9216;                           // bytes per slot
constexpr int kSThreads = (kSC + 2) * 32;              // producer + consumers + auxiliary
constexpr int kSThreadsTc = (kSC + 2 + 8) * 32;        // tensor-core variant: + 4 warps that write weight scales, 4 that read accumulators
constexpr int kSMaxTopK = 8;
constexpr int kSMaxShared = 2;
constexpr int kSMaxRows = 64;                          // output rows one block may own
constexpr int kSMaxExperts = 512;
constexpr int kSyncWordsPerLayer = 8;                  // counters of one layer
constexpr int kSMaxWorld = 8;                          // tensor-parallel ranks
constexpr int kTileCountersPerLayer = kSMaxTopK * 32 + 32;   // routed gate/up tiles (at most 8 x 32), then down row tiles

constexpr int kTraceBlocks = 256;
constexpr int kTraceSlots = 32;
// phase stamps written by consumer warp 0 (and slot 12..14 by the producer) when tracing is on
enum TraceSlot {
  kTrLayerStart = 0, kTrRouterDone = 1, kTrShGuDone = 2, kTrRtGuDone = 3, kTrShGuAll = 4, kTrShDownDone = 5,
  kTrRtGuAll = 6, kTrActStaged = 7, kTrRtDownDone = 8, kTrDownAll = 9, kTrNormDone = 10,
  kTrProdRouteWait = 12, kTrProdRouteGot = 13, kTrProdLayerIssued = 14,
  kTrXDigits = 11, kTrXVisible = 15,                                         // tensor-core variant, consumers
  kTrMmaGuStart = 16, kTrMmaGuEnd = 17, kTrMmaDownStart = 18, kTrMmaDownEnd = 19,   // the issuing thread
  kTrScalesGuEnd = 20, kTrScalesDownEnd = 21,                                // first warp that writes weight scales
  kTrRowsSent = 22, kTrNormReduced = 23,                                     // the warp that hands the block's rows over; consumers
  // not stamps but SM clock cycles that consumer warp 0 spent waiting for tiles in each section of the layer
  // (CUDA-core variant), and that producer lane 0 spent with a tile to issue but no free slot
  kTrWaitRouter = 24, kTrWaitShGu = 25, kTrWaitRtGu = 26, kTrWaitShDown = 27, kTrWaitRtDown = 28, kTrProdSlotWait = 29,
  kTrBusyShGu = 30, kTrBusyRtGu = 31,   // cycles consumer warp 0 held tiles of the shared / routed gate/up section
};
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define INK_TRACE_VALUE(layer, slot, value)                                                             \
  do {                                                                                                  \
    if (a.trace && blockIdx.x < kTraceBlocks)                                                           \
      a.trace[((size_t)(layer) * kTraceBlocks + blockIdx.x) * kTraceSlots + (slot)] = (value);          \
  } while (0)
#define INK_TRACE(layer, slot)                                                                          \
  do {                                                                                                  \
    if (a.trace && blockIdx.x < kTraceBlocks)                                                           \
      a.trace[((size_t)(layer) * kTraceBlocks + blockIdx.x) * kTraceSlots + (slot)] = global_ns();      \
  } while (0)

enum SyncWord { kShGuDone = 0, kRtGuDone = 1 };

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
  const void* tmaps;               // four TMA descriptors of the layer's banks (gate/up codes, gate/up scales, down codes,
                                   // down scales), or null: the routed experts then run on the CUDA cores
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
  unsigned long long* scores;      // scratch [2][experts + n_shared] router words {selection score, BF16 logit, 16-bit tag}
  uint16_t* activated;             // scratch [2][top_k][f]
  uint16_t* shared_activated;      // scratch [2][n_shared][f]
  RouteTable* routes;              // scratch [n_layers]
  float* gu_part;                  // scratch [top_k * 2f/128 tiles][hidden/256][128]: partial gate/up rows of a tile split between blocks
  float* dn_part;                  // scratch [top_k * hidden/128 tiles][f/256][128]: the same for the down projection
  float* sd_out;                   // scratch [2][n_shared][hidden]: shared experts' down rows (tensor-core variant)
  unsigned* act_amax;              // scratch [2][kSMaxTopK]: largest |activation| bits of each route (tensor-core variant)
  unsigned* tilesync;              // scratch [n_layers][tile counters]: blocks that have stored their part of a tile (epoch-based)
  unsigned* sync;                  // scratch [n_layers][kSyncWordsPerLayer]: counters that only grow (see epoch)
  unsigned* epoch;                 // scratch: launches completed so far on this rank; every target scales with it
  // tensor-parallel ranks
  int rank, world;
  unsigned long long* inbox;       // this rank's [2][world][hidden] tagged words: partial output rows as the ranks deliver them
  unsigned long long* peer_inbox[kSMaxWorld];   // the same region of every rank, as mapped into this process
  unsigned long long* summed;      // scratch [2][hidden] tagged words: the rows summed over the ranks, for every block of this rank
  long long wait_limit;            // SM clocks a wait may take before the launch gives up
  unsigned poll_pause_ns;          // pause between two polls of a hand-over word
                                   // when a lane issues its last tile of a layer: they arrive while the blocks hand their rows over
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
  static constexpr int QD_CODES = RT * (F / 2);             // one row group: 4096 bytes of codes ...
  static constexpr int QD_SCALES = RT * (F / 16);           // ... and 512 of scales
  // a routed down tile of the CUDA-core path holds up to QD_PAIR consecutive row groups (codes of all of them, then
  // their scales): one producer lane issues about two tiles per microsecond, so tiles have to be this large
  static constexpr int QD_PAIR = 2;
  static constexpr int SD_ROWS = 8192 / (F * 2) < RT ? 8192 / (F * 2) : RT;   // BF16 rows per tile
  static constexpr int SD_PER_GROUP = RT / SD_ROWS;
  static constexpr int SD_BYTES = SD_ROWS * F * 2;
  static constexpr int SD_CPL = F / 256;
  static_assert(R_BYTES <= kSSlot && 2 * SG_PART <= kSSlot && QG_CODES + QG_SCALES <= kSSlot, "tile exceeds slot");
  static_assert(QD_PAIR * (QD_CODES + QD_SCALES) <= kSSlot && SD_BYTES <= kSSlot, "tile exceeds slot");
  // staging that overlays: [x FP16 | x BF16] during gate/up, [routed act FP16 | shared act BF16] during down
  // tensor-core path: [x digit rows D*4 | x BF16] during gate/up
  static constexpr int GU_TILES = 2 * F / kTcRows;          // 128-row tiles per expert
  static constexpr int GU_CHUNKS = D / kTcChunkK;           // units per tile
  static constexpr int DN_TILES = D / kTcRows;              // 128-row tiles of the down projection per expert
  static constexpr int DN_CHUNKS = F / kTcChunkK;
  static constexpr int STAGING_A = kSMaxTopK * F * 2 + kSMaxShared * F * 2;
  // tensor-core variant: the shared experts' activations are staged while the digit rows of x are still
  // being read, so they sit behind both digit-row areas
  static constexpr int TC_SACT = D * 6 > F * 16 ? D * 6 : F * 16;
  static constexpr int STAGING_B = TC_SACT + kSMaxShared * F * 2;
  static constexpr int STAGING = STAGING_A > STAGING_B ? STAGING_A : STAGING_B;
  static constexpr int SMEM = kSStages * kSSlot + STAGING + 1024;   // the ring starts on a 1024-byte boundary
  static_assert(2 * kSSlot == kTcUnitBytes, "a tensor-core unit takes exactly two ring slots");
  static_assert(D % kTcChunkK == 0 && (2 * F) % kTcRows == 0 && D / 64 * 4 <= 512 - kTcColSfb, "shape does not tile");
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
  int qu0, n_qu;          // tensor-core path: routed gate/up units [qu0, qu0 + n_qu) of top_k * GU_TILES * GU_CHUNKS
  int du0, n_du;          // and routed down units of top_k * DN_TILES * DN_CHUNKS
  int n_sd_real;          // shared down tiles without the padding tile that keeps the units on even slots
  int n_gt;               // routed down tiles per route on the CUDA-core path (QD_PAIR row groups each, the last maybe fewer)
};

template <int D, int F>
__device__ __forceinline__ TilePlan make_plan(const StackArgs& a, bool tc) {
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
  const long long gu_units = (long long)a.top_k * S::GU_TILES * S::GU_CHUNKS;
  p.qu0 = (int)(b * gu_units / G);
  p.n_qu = (int)((b + 1) * gu_units / G) - p.qu0;
  if (tc) p.n_q = 2 * p.n_qu;   // a unit takes two consecutive ring slots
  const int groups = D / S::RT;
  p.g0 = (int)(b * groups / G);
  p.n_g = (int)((b + 1) * groups / G) - p.g0;
  // The router section is padded to whole rounds of the consumers only where the tensor-core units need their
  // even slots: empty tiles at the head of a layer take ring slots that could hold the next layer's first
  // weights while the rows are handed over.
  const int pad_r = tc ? (p.n_r + kSC - 1) / kSC * kSC : p.n_r;
  p.n_sg = (p.n_u + kSC - 1) / kSC * kSC * S::SG_SPLIT;
  p.n_sd = p.n_sd_real = a.n_shared * p.n_g * S::SD_PER_GROUP;
  p.n_gt = (p.n_g + S::QD_PAIR - 1) / S::QD_PAIR;
  p.n_qd = a.top_k * p.n_gt;
  const long long dn_units = (long long)a.top_k * S::DN_TILES * S::DN_CHUNKS;
  p.du0 = (int)(b * dn_units / G);
  p.n_du = (int)((b + 1) * dn_units / G) - p.du0;
  if (tc) {
    p.n_sd += p.n_sd & 1;
    p.n_qd = 2 * p.n_du;
  }
  p.s_r = 0;
  p.s_sg = pad_r;
  p.s_qg = p.s_sg + p.n_sg;
  p.s_sd = p.s_qg + p.n_q;
  p.s_qd = p.s_sd + p.n_sd;
  p.s_pad = p.s_qd + p.n_qd;
  p.per_layer = (p.s_pad + kSC - 1) / kSC * kSC;
  return p;
}

// What the routing of a layer needs besides the scores, brought into shared memory by the auxiliary warp
// while the previous layer is still streaming: under a saturated memory system a dependent global load
// takes microseconds, and the routing has four of them in a row on the layer's critical path.
struct RouteConsts {
  const uint8_t* bank[kSMaxExperts][4];   // gate/up codes, gate/up scales, down codes, down scales (null: not on this rank)
  float gu_scale2[kSMaxExperts];
  float dn_scale2[kSMaxExperts];
  float bias[kSMaxExperts];
  float global_scale, route_scale;
};

struct StackShared {
  uint64_t full[kSStages];
  uint64_t empty[kSStages];
  RouteTable routes[2];                 // by layer parity; filled by the producer warp
  float contrib[kSMaxTopK + kSMaxShared][kSMaxRows];
  float logit[kSMaxExperts + kSMaxShared];   // auxiliary warp scratch: the layer's BF16-rounded logits (routed rows, then shared rows)
  float red[kSC][4];                    // consumer reductions
  float inverse[kSMaxTopK];             // inverse normalisers of the staged routed activations
  float x_inverse;                      // inverse normaliser of the staged x
  int done[2][3];                       // tiles finished per layer parity: shared g/u, routed g/u, down
  unsigned epoch1;                      // launches completed before this one, plus one: scales every target
  long long limit;                      // SM clocks a wait may take
  unsigned pause;                       // nanoseconds between two polls of a word that other blocks write
  volatile int rows_seen;               // layers whose summed output rows consumer warp 0 has seen arrive
  volatile int routed_layers;           // layers whose routing table is in `routes` (set by the auxiliary warp)
  volatile int seen[2];                 // layers whose grid-wide counters (shared gate/up, routed gate/up) the auxiliary
                                        // warp has seen complete: one poller per block instead of one per warp
  volatile int sact_flag[kSMaxShared];  // layers whose shared-expert activations are staged, per shared expert
  volatile int act_flag[kSMaxTopK];     // layers whose routed activations are staged, per route
  volatile int failed;
  volatile int consts_layers;           // layers whose routing constants have been loaded into `consts` (set by the auxiliary warp)
  RouteConsts consts;
  // tensor-core path
  uint64_t sf_full[kTcSfSlots], sf_empty[kTcSfSlots];   // weight scales of a unit are in tensor memory / may be overwritten
  uint64_t d_full[2], d_empty[2];                        // accumulator of a tile segment is complete / has been read
  uint32_t tmem_base;
  volatile int x_ready;                 // layers whose activation digits and scales are staged
  volatile int act_ready;               // layers whose routed activations are staged as digit rows
  volatile int sg_done;                 // layers whose router rows and shared gate/up tiles this block has finished
  volatile long long issued;            // ring tiles the producer has issued (published after every tensor-core unit)
  int finisher;                         // this block stored the last part of the tile at hand
  float act_inverse[kSMaxTopK];         // inverse normalisers of the routed activations' digit rows
  uint8_t seg_parts[2][8], seg_index[2][8];   // how this block's first tile segments (gate/up, down) are split: computed once
  uint8_t dn_parts[kSMaxTopK][32];      // blocks that share a down tile (route, row tile)
  unsigned dn_target[32];               // arrivals that complete a row tile: routed parts of every route + shared-expert blocks
  uint8_t sfbx[kTcDigits][256];         // E4M3 block scales of the digit rows of x
  uint8_t sfba[4 * kSMaxTopK][128];     // and of the digit rows of the routed activations
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
// (Counters and targets wrap at 2^32 after some tens of millions of launches: the comparison is on the
// signed difference, which stays right as long as a counter is less than 2^31 away from its target.)
__device__ __forceinline__ bool reached(unsigned counter, unsigned target) { return (int)(counter - target) >= 0; }
__device__ __forceinline__ bool wait_global(const unsigned* p, unsigned target, StackShared* sh) {
  if (sh->failed) return false;
  if (reached(ld_acquire_u32(p), target)) return true;
  const long long t0 = clock64();
  while (!reached(ld_acquire_u32(p), target)) {
    if (sh->failed) return false;
    if (clock64() - t0 > sh->limit) {
      sh->failed = 1;
      return false;
    }
    __nanosleep(sh->pause);   // a counter is polled by every block: polling it harder only delays the increments
  }
  return true;
}

// ---- tagged words: {FP32 value (low half), tag (high half)} in one aligned 8-byte word
__device__ __forceinline__ unsigned long long tagged(float v, unsigned tag) {
  return (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
}
__device__ __forceinline__ void st_tagged(unsigned long long* p, float v, unsigned tag) {
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(tagged(v, tag)) : "memory");
}
__device__ __forceinline__ void st_tagged_sys(unsigned long long* p, float v, unsigned tag) {   // into a peer's memory
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(tagged(v, tag)) : "memory");
}
// two neighbouring words in one 16-byte store (p 16-byte aligned): each word carries its own tag, so it does not
// matter whether the two halves become visible together
__device__ __forceinline__ void st_tagged2_sys(unsigned long long* p, float v0, float v1, unsigned tag) {
  asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(tagged(v0, tag)), "l"(tagged(v1, tag)) : "memory");
}
__device__ __forceinline__ unsigned long long ld_tagged(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_tagged_sys(const unsigned long long* p) {   // written by a peer
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ld_tagged2(const unsigned long long* p, unsigned long long (&v)[2]) {   // 16-byte aligned pair
  asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(v[0]), "=l"(v[1]) : "l"(p) : "memory");
}
__device__ __forceinline__ bool has_tag(unsigned long long word, unsigned tag) { return (unsigned)(word >> 32) == tag; }
__device__ __forceinline__ float value_of(unsigned long long word) { return __uint_as_float((unsigned)word); }
// The tag of a layer of a launch. Never zero before the epoch wraps, so a zero-filled buffer matches nothing.
__device__ __forceinline__ unsigned layer_tag(unsigned epoch1, int n_layers, int layer) {
  return epoch1 * (unsigned)n_layers + (unsigned)layer;
}
// A router row's word: {FP32 selection score, BF16 logit, 16-bit tag} -- score and logit arrive together, so the
// routing needs one poll and no second round trip. The 16-bit tag is never zero and repeats only after 65 535
// layers, long after the word has been overwritten (the two sets of words alternate from layer to layer).
__device__ __forceinline__ unsigned router_tag(unsigned tag) { return tag % 65535u + 1u; }
__device__ __forceinline__ unsigned long long router_word(float score, float logit_bf16, unsigned tag16) {
  return (unsigned long long)__float_as_uint(score) | ((unsigned long long)(__float_as_uint(logit_bf16) >> 16) << 32) |
         ((unsigned long long)tag16 << 48);
}
// Bounded wait for one tagged word; the value, or 0 once the launch has failed.
__device__ __forceinline__ float wait_tagged(const unsigned long long* p, unsigned tag, StackShared* sh) {
  unsigned long long w = ld_tagged(p);
  if (has_tag(w, tag)) return value_of(w);
  const long long t0 = clock64();
  while (!sh->failed) {
    w = ld_tagged(p);
    if (has_tag(w, tag)) return value_of(w);
    if (clock64() - t0 > sh->limit) sh->failed = 1;
    __nanosleep(32);
  }
  return 0.f;
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
    if (clock64() - t0 > sh->limit) {
      sh->failed = 1;
      return false;
    }
  }
  __threadfence_block();
  return true;
}

// Bounded wait of a warp until a staging flag of this block has reached `layer + 1` (one lane polls).
__device__ __forceinline__ void wait_flag(volatile int* flag, int layer, StackShared* sh, int lane) {
  if (lane == 0 && *flag <= layer) {
    const long long t0 = clock64();
    while (*flag <= layer && !sh->failed) {
      if (clock64() - t0 > sh->limit) sh->failed = 1;
      __nanosleep(40);   // the warp next to this one on the scheduler is computing
    }
  }
  __syncwarp();
  __threadfence_block();
}

__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kSC * 32) : "memory");
}

// One warp: the routing constants of `layer` from global into shared memory (all loads of a pass in flight together).
__device__ void load_route_consts(const StackArgs& a, int layer, StackShared* sh) {
  const int lane = threadIdx.x & 31;
  const StackLayer* ly = a.layers + layer;
  const int64_t* sources = ly->sources;
  const float* bias = ly->router_bias;
  RouteConsts& c = sh->consts;
  if (lane == 0) {
    c.global_scale = bf16_to_f32(ly->global_scale[0]);
    c.route_scale = ly->route_scale;
  }
#pragma unroll 1
  for (int e0 = 0; e0 < a.experts; e0 += 128) {
    longlong2 row[4][3];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = e0 + i * 32 + lane;
#pragma unroll
      for (int k = 0; k < 3; ++k)
        row[i][k] = e < a.experts ? __ldg(reinterpret_cast<const longlong2*>(sources + (size_t)e * kBank) + k) : make_longlong2(0, 0);
    }
    float s2[4][2], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = e0 + i * 32 + lane;
      // entries: 0 codes, 1 scales, 2 scale2 | 3 codes, 4 scales, 5 scale2
      s2[i][0] = row[i][0].x ? __ldg(reinterpret_cast<const float*>(row[i][1].x)) : 0.f;
      s2[i][1] = row[i][1].y ? __ldg(reinterpret_cast<const float*>(row[i][2].y)) : 0.f;
      b[i] = e < a.experts ? __ldg(bias + e) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = e0 + i * 32 + lane;
      if (e < a.experts) {
        c.bank[e][0] = reinterpret_cast<const uint8_t*>(row[i][0].x);
        c.bank[e][1] = reinterpret_cast<const uint8_t*>(row[i][0].y);
        c.bank[e][2] = reinterpret_cast<const uint8_t*>(row[i][1].y);
        c.bank[e][3] = reinterpret_cast<const uint8_t*>(row[i][2].x);
        c.gu_scale2[e] = s2[i][0];
        c.dn_scale2[e] = s2[i][1];
        c.bias[e] = b[i];
      }
    }
  }
  __syncwarp();
  if (lane == 0) {
    __threadfence_block();
    sh->consts_layers = layer + 1;
  }
}

// -------------------------------------------------------------------- router tail
// One warp: the layer's router words as the blocks publish them. Lane l ends up with the selection scores
// of the experts l, l + 32, ... in registers (`sc`, -inf beyond the routed experts) and every row's logit in
// shared memory. One round of loads at a time, only the words still missing, with a pause between rounds:
// every block polls the same few lines, and on B200 polling them harder (two rounds in flight, no pause) made
// the words arrive later, not sooner -- the loads queue up in front of the stores. False: the launch failed.
template <int K>
__device__ __forceinline__ bool poll_router_words(const StackArgs& a, const unsigned long long* words, unsigned tag16, int rows,
                                                  float (&sc)[K], StackShared* sh) {
  const int lane = threadIdx.x & 31;
  float* logit = sh->logit;
  const unsigned long long found = (unsigned long long)tag16 << 48;   // stands for a row this lane does not have
#pragma unroll
  for (int i = 0; i < K; ++i) sc[i] = -INFINITY;
  unsigned long long w[K];
  unsigned missing = 0;
#pragma unroll
  for (int i = 0; i < K; ++i)
    if (i * 32 + lane < rows) missing |= 1u << i;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll
    for (int i = 0; i < K; ++i) w[i] = (missing >> i) & 1u ? ld_tagged(words + i * 32 + lane) : found;
#pragma unroll
    for (int i = 0; i < K; ++i) {
      const int e = i * 32 + lane;
      if (((missing >> i) & 1u) && (unsigned)(w[i] >> 48) == tag16) {
        if (e < a.experts) sc[i] = __uint_as_float((unsigned)w[i]);
        logit[e] = __uint_as_float((unsigned)(w[i] >> 32) << 16);
        missing &= ~(1u << i);
      }
    }
    if (__all_sync(0xffffffffu, missing == 0)) break;
    if (sh->failed) return false;
    if (clock64() - t0 > sh->limit) sh->failed = 1;
    __nanosleep(sh->pause);
  }
  return !sh->failed;
}

// The top_k largest scores over the lanes' registers (ties: the lower expert id); lane r returns choice r.
template <int K>
__device__ __forceinline__ int select_top_k(float (&sc)[K], int top_k) {
  // Every round: the lane's own best, then the warp's with two hardware reductions (largest score as an
  // order-preserving integer, then the lowest expert id among the lanes that hold it) instead of five rounds of
  // paired shuffles: this chain sits on the critical path of every layer once the experts are sliced thin.
  const int lane = threadIdx.x & 31;
  int my_choice = 0;
#pragma unroll 1
  for (int r = 0; r < top_k; ++r) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < K; ++i) {
      if (sc[i] > best) {
        best = sc[i];
        best_e = i * 32 + lane;
      }
    }
    const unsigned bits = __float_as_uint(best);
    const unsigned key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);   // a > b  <=>  key(a) > key(b)
    const unsigned top = __reduce_max_sync(0xffffffffu, key);
    int winner = (int)__reduce_min_sync(0xffffffffu, key == top ? (unsigned)best_e : 0x7fffffffu);
    if (winner == 0x7fffffff) winner = r;
#pragma unroll
    for (int i = 0; i < K; ++i)
      if (i * 32 + lane == winner) sc[i] = -INFINITY;
    if (lane == r) my_choice = winner;
  }
  return my_choice;
}

// One warp. Waits for the layer's scores as the blocks publish them (router words), then
// resolves the routing. Returns false if the launch failed while waiting.
__device__ bool stack_router_tail(const StackArgs& a, const StackLayer& ly, int layer, StackShared* sh) {
  const int lane = threadIdx.x & 31;
  const int par = layer & 1;
  const unsigned tag16 = router_tag(layer_tag(sh->epoch1, a.n_layers, layer));
  const int rows = a.experts + a.n_shared;
  const unsigned long long* words = a.scores + (size_t)par * rows;
  const float* logit = sh->logit;
  int my_choice;
  constexpr int kFew = 9, kMany = (kSMaxExperts + kSMaxShared + 31) / 32;   // router rows per lane: up to 288, up to 514
  if (rows <= kFew * 32) {
    float sc[kFew];
    if (!poll_router_words<kFew>(a, words, tag16, rows, sc, sh)) return false;
    if (lane == 0) INK_TRACE(layer, kTrXDigits);   // (CUDA-core variant: all scores of the layer have arrived)
    my_choice = select_top_k<kFew>(sc, a.top_k);
  } else {
    float sc[kMany];
    if (!poll_router_words<kMany>(a, words, tag16, rows, sc, sh)) return false;
    if (lane == 0) INK_TRACE(layer, kTrXDigits);
    my_choice = select_top_k<kMany>(sc, a.top_k);
  }
  __syncwarp();
  const int n = a.top_k + a.n_shared;
  const bool live = lane < n;
  float l = 0.f;
  if (lane < a.top_k) l = logit[my_choice];
  else if (live) l = logit[a.experts + (lane - a.top_k)];
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
  const RouteConsts& c = sh->consts;    // loaded for this layer before the scores could be complete (see the caller)
  w = round_bf16(w * c.route_scale);
  w = round_bf16(w * c.global_scale);
  RouteTable* table = &sh->routes[layer & 1];
  if (lane < a.top_k) {
    RouteEntry r;
    r.gu_codes = c.bank[my_choice][0];
    r.gu_scales = c.bank[my_choice][1];
    r.gu_scale2 = c.gu_scale2[my_choice];
    r.dn_codes = c.bank[my_choice][2];
    r.dn_scales = c.bank[my_choice][3];
    r.dn_scale2 = c.dn_scale2[my_choice];
    r.weight = w;
    r.expert = my_choice;
    table->route[lane] = r;
  } else if (live) {
    table->gamma[lane - a.top_k] = w;
  }
  __syncwarp();
  if (lane == 0) {
    __threadfence_block();
    sh->routed_layers = layer + 1;   // the producer and the consumers of this block may read the table
    INK_TRACE(layer, kTrXVisible);   // (CUDA-core variant: the routing is resolved)
  }
  if (blockIdx.x == 0) {   // one block also writes the optional router outputs (off the critical path)
    if (lane < a.top_k) {
      if (ly.topk_indices) ly.topk_indices[lane] = my_choice;
      if (ly.topk_weights) ly.topk_weights[lane] = (uint16_t)f32_to_bf16_bits(w);
    } else if (live && ly.gammas) {
      ly.gammas[lane - a.top_k] = (uint16_t)f32_to_bf16_bits(w);
    }
  }
  return true;
}

// ---------------------------------------------------------------- x staging (consumers)
// The activation vector between blocks lives in the consumer threads as groups of eight
// consecutive elements (packed BF16, 16 bytes): thread ct holds the groups g * VT + ct,
// g < VG, of the D / 8 groups; threads ct >= VT hold nothing (hidden sizes below 2048).
template <int D>
struct VecShape {
  static constexpr int VG = D >= 2048 ? D / 2048 : 1;
  static constexpr int VT = D / 8 / VG;
  static_assert(VT % 32 == 0 && VT <= kSC * 32, "whole warps hold the vector");
};

// CUDA-core variant: BF16 copy and a copy normalised by a power of two into FP16.
template <int D>
__device__ __forceinline__ void stage_x(uint16_t* s_x16, uint16_t* s_xbf, const uint4 (&xb)[VecShape<D>::VG], float amax_bound,
                                        StackShared* sh, int ct) {
  using V = VecShape<D>;
  // power-of-two normaliser from an upper bound of the largest magnitude
  float inverse;
  const uint32_t bits = f32_to_bf16_bits(amax_bound) & 0x7fffu;
  const float scale = pow2_normaliser(bits + 0x80u > 0x7f7fu ? 0x7f7fu : bits + 0x80u, &inverse);  // one binade of margin
  if (ct < V::VT) {
#pragma unroll
    for (int g = 0; g < V::VG; ++g) {
      const int group = g * V::VT + ct;
      reinterpret_cast<uint4*>(s_xbf)[group] = xb[g];
      const uint4 h = stage_pack8(xb[g], scale, ct & 3);   // group g * VT + ct of eight values, VT a multiple of 32
      reinterpret_cast<uint4*>(s_x16)[group] = h;
    }
  }
  if (ct == 0) sh->x_inverse = inverse;
}

// Bounded wait on a barrier of the tensor-core path that also gives up as soon as the launch has failed.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, StackShared* sh) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (sh->failed) return false;
    if (clock64() - t0 > sh->limit) {
      sh->failed = 1;
      return false;
    }
  }
  return true;
}
// A parity wait on a ring slot is only meaningful once the slot's previous use is over. The consumer
// warps get that from the order in which they take tiles; a warp that waits for a tile from far away
// (the tensor-core warps may be a whole lap ahead of the consumers) first waits until the producer
// has issued that very tile, which it does only after the slot's previous tile was consumed.
__device__ __forceinline__ bool tc_wait_issued(long long tile, StackShared* sh) {
  if (sh->issued > tile) {
    __threadfence_block();
    return true;
  }
  const long long t0 = clock64();
  while (sh->issued <= tile) {
    if (sh->failed) return false;
    if (clock64() - t0 > sh->limit) {
      sh->failed = 1;
      return false;
    }
  }
  __threadfence_block();
  return true;
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }
__device__ __forceinline__ void tc_group_sync() { asm volatile("bar.sync 3, 256;" ::: "memory"); }

// Items [first, last] of `total` dealt to `blocks` blocks as [total*b/blocks, total*(b+1)/blocks):
// how many blocks hold some of them, and the position of block `me` among those.
__device__ __forceinline__ int tc_split(long long first, long long last, long long total, int blocks, int me, int* my_index) {
  const int fb = tc_owner(first, total, blocks), lb = tc_owner(last, total, blocks);
  int parts = 0, index = 0;
  for (int b = fb; b <= lb; ++b) {
    if (total * b / blocks < total * (b + 1) / blocks) {   // blocks with an empty range hold nothing
      if (b == me) index = parts;
      ++parts;
    }
  }
  *my_index = index;
  return parts;
}

// Tensor-core variant: the same vector as BF16 (router, shared experts) and as four E2M1 digit rows
// in the swizzled N-operand layout, block scales to `sh->sfbx`. Whole warps of holders call it.
template <int D>
__device__ __forceinline__ void stage_x_tc(unsigned char* s_xdig, uint16_t* s_xbf, const uint4 (&xb)[VecShape<D>::VG], float amax_bound,
                                           StackShared* sh, int ct) {
  using V = VecShape<D>;
  float inverse;
  const uint32_t bits = f32_to_bf16_bits(amax_bound) & 0x7fffu;
  const float scale = 512.f * pow2_normaliser(bits + 0x80u > 0x7f7fu ? 0x7f7fu : bits + 0x80u, &inverse);  // below 1024
  if (ct < V::VT) {
#pragma unroll 1
    for (int g = 0; g < V::VG; ++g) {
      const int group = g * V::VT + ct;
      reinterpret_cast<uint4*>(s_xbf)[group] = xb[g];
      tc_stage8(xb[g], scale, s_xdig, 8, 0, group * 8, &sh->sfbx[0][0], 256);
    }
  }
  if (ct == 0) sh->x_inverse = inverse * (1.f / 512.f);
}

// ---- hand-over of the layer's output rows (the all-reduce of a block, for any number of ranks)
// The thread that holds this rank's total of output row `row` stores it, tagged, where the rows are
// summed: one rank -> straight into `summed`; several ranks -> into slot `rank` of every rank's inbox
// (plain 8-byte stores into peer memory).
template <int D>
__device__ __forceinline__ void send_row(const StackArgs& a, int xpar, unsigned tag, int row, float total) {
  if (a.world == 1) {
    st_tagged(a.summed + (size_t)xpar * D + row, total, tag);
  } else {
    const size_t at = ((size_t)xpar * a.world + a.rank) * D + row;
    for (int r = 0; r < a.world; ++r) st_tagged_sys(a.peer_inbox[r] + at, total, tag);
  }
}
// Several ranks: the same thread then waits for that row from every rank (all loads of a round in
// flight together, bounded), adds them in rank order -- every rank computes the same bits -- and
// publishes the sum for the blocks of this rank.
template <int D>
__device__ __forceinline__ void gather_row(const StackArgs& a, StackShared* sh, int xpar, unsigned tag, int row) {
  const unsigned long long* from = a.inbox + (size_t)xpar * a.world * D + row;
  unsigned long long w[kSMaxWorld];
  bool all = true;
#pragma unroll
  for (int r = 0; r < kSMaxWorld; ++r) {
    w[r] = r < a.world ? ld_tagged_sys(from + (size_t)r * D) : ((unsigned long long)tag << 32);
    all = all && has_tag(w[r], tag);
  }
  const long long t0 = clock64();
  while (!all && !sh->failed) {
    __nanosleep(64);
    all = true;
#pragma unroll
    for (int r = 0; r < kSMaxWorld; ++r) {
      if (r < a.world && !has_tag(w[r], tag)) w[r] = ld_tagged_sys(from + (size_t)r * D);
      all = all && has_tag(w[r], tag);
    }
    if (clock64() - t0 > sh->limit) sh->failed = 1;
  }
  float sum = 0.f;
#pragma unroll
  for (int r = 0; r < kSMaxWorld; ++r)
    if (r < a.world) sum += value_of(w[r]);
  if (!sh->failed) st_tagged(a.summed + (size_t)xpar * D + row, sum, tag);
}

// Tensor-core variant: every part of row tile `tile` (the routed projections' parts and the shared
// experts' rows) is in global memory. Sums them in a fixed order -- the parts of a route in block
// order, the routes in choice order, then the shared experts -- and stores the rows into every
// rank's inbox. Rows first, first + stride, ... of the tile.
template <int D, int F>
__device__ __forceinline__ void finish_row_tile(const StackArgs& a, StackShared* sh, int layer, int par, int xpar, int tile, int first,
                                                int stride) {
  using S = StackShape<D, F>;
  const unsigned tag = layer_tag(sh->epoch1, a.n_layers, layer);
  // the routes' activation maxima first (the same for every row), then per row all loads before any arithmetic:
  // this runs in one block per row tile at the very end of a layer, so its round trips to L2 are what it costs
  unsigned amax[kSMaxTopK];
#pragma unroll
  for (int j = 0; j < kSMaxTopK; ++j) amax[j] = j < a.top_k ? __ldcg(a.act_amax + par * kSMaxTopK + j) : 0u;
  for (int row = first; row < kTcRows; row += stride) {
    const size_t at_row = (size_t)tile * kTcRows + row;
    float part[kSMaxTopK][2], shared[kSMaxShared];
#pragma unroll
    for (int j = 0; j < kSMaxTopK; ++j) {
      const float* from = a.dn_part + (size_t)(j * S::DN_TILES + tile) * S::DN_CHUNKS * kTcRows + row;
      const int parts = j < a.top_k ? sh->dn_parts[j][tile] : 0;
      part[j][0] = parts > 0 ? __ldcg(from) : 0.f;
      part[j][1] = parts > 1 ? __ldcg(from + kTcRows) : 0.f;
    }
#pragma unroll
    for (int e = 0; e < kSMaxShared; ++e)
      shared[e] = e < a.n_shared ? __ldcg(a.sd_out + ((size_t)par * a.n_shared + e) * D + at_row) : 0.f;
    float total = 0.f;
#pragma unroll
    for (int j = 0; j < kSMaxTopK; ++j) {
      if (j < a.top_k) {
        const RouteEntry& r = sh->routes[par].route[j];
        const int parts = sh->dn_parts[j][tile];
        float acc = part[j][0] + part[j][1];   // block order; a tile cut in more than two parts is rare (narrow slices)
        const float* from = a.dn_part + (size_t)(j * S::DN_TILES + tile) * S::DN_CHUNKS * kTcRows + row;
        for (int p = 2; p < parts; ++p) acc += __ldcg(from + (size_t)p * kTcRows);
        if (r.dn_codes) {
          float inverse;
          pow2_normaliser(amax[j], &inverse);
          const float down = round_bf16(acc * (r.dn_scale2 * (inverse * (1.f / 512.f))));
          total += round_bf16(down * r.weight);
        }
      }
    }
#pragma unroll
    for (int e = 0; e < kSMaxShared; ++e) total += shared[e];
    send_row<D>(a, xpar, tag, (int)at_row, total);
  }
  if (a.world > 1)
    for (int row = first; row < kTcRows; row += stride) gather_row<D>(a, sh, xpar, tag, tile * kTcRows + row);
}
template <int D, int F, bool TC>
__global__ void __launch_bounds__(TC ? kSThreadsTc : kSThreads, 1) moe_stack_kernel(StackArgs a) {
  using S = StackShape<D, F>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ StackShared sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // TC: the layers carry TMA descriptors and the routed experts run on the tensor cores
  constexpr bool tc = TC;
  unsigned char* slots = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);   // swizzled tiles need 1024-byte alignment
  unsigned char* staging = slots + kSStages * kSSlot;
  uint16_t* s_x16 = reinterpret_cast<uint16_t*>(staging);            // [D] FP16 normalised (gate/up phases, CUDA-core path)
  unsigned char* s_xdig = staging;                                    // [D/256][8 rows][128 B] digit rows of x (tensor-core path)
  uint16_t* s_xbf = reinterpret_cast<uint16_t*>(staging + (tc ? D * 4 : D * 2));   // [D] BF16
  uint16_t* s_act = reinterpret_cast<uint16_t*>(staging);            // [top_k][F] FP16 normalised (down phases)
  unsigned char* s_adig = staging;                                    // [F/256][32 rows][128 B] digit rows of the routed activations
  uint16_t* s_sact = tc ? reinterpret_cast<uint16_t*>(staging + S::TC_SACT)
                        : s_act + (size_t)kSMaxTopK * F;              // [n_shared][F] BF16 (act * gamma)
  const TilePlan plan = make_plan<D, F>(a, tc);
  const int total_rows = a.experts + a.n_shared;
  const int n_jobs = a.top_k + a.n_shared;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSStages; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    for (int s = 0; s < kTcSfSlots; ++s) {
      mbar_init(&sh.sf_full[s], 4);
      mbar_init(&sh.sf_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh.d_full[s], 1);
      mbar_init(&sh.d_empty[s], 4);
    }
    sh.x_ready = 0;
    sh.act_ready = 0;
    sh.sg_done = 0;
    sh.issued = 0;
    sh.routed_layers = 0;
    sh.consts_layers = 0;
    for (int i = 0; i < 2; ++i) sh.seen[i] = 0;
    for (int i = 0; i < kSMaxShared; ++i) sh.sact_flag[i] = 0;
    for (int i = 0; i < kSMaxTopK; ++i) sh.act_flag[i] = 0;
    sh.failed = 0;
    sh.epoch1 = *a.epoch + 1u;
    sh.limit = a.wait_limit;
    sh.pause = a.poll_pause_ns;
    sh.rows_seen = 0;
    for (int i = 0; i < 6; ++i) (&sh.done[0][0])[i] = 0;
    mbar_init_fence();
  }
  for (int i = threadIdx.x; i < (kSMaxTopK + kSMaxShared) * kSMaxRows; i += blockDim.x) (&sh.contrib[0][0])[i] = 0.f;
  if (tc) {
    if (warp == kSC + 1) tc_alloc(&sh.tmem_base, 512);
    // how every down tile is split between blocks (the same for every layer)
    const long long dn_units = (long long)a.top_k * S::DN_TILES * S::DN_CHUNKS;
    for (int i = threadIdx.x; i < a.top_k * S::DN_TILES; i += blockDim.x) {
      int unused;
      sh.dn_parts[i / S::DN_TILES][i % S::DN_TILES] =
          (uint8_t)tc_split((long long)i * S::DN_CHUNKS, (long long)i * S::DN_CHUNKS + S::DN_CHUNKS - 1, dn_units, gridDim.x, 0, &unused);
    }
    if (blockIdx.x == 0 && threadIdx.x < 2 * kSMaxTopK) a.act_amax[threadIdx.x] = 0u;   // seen by all before the first routing exists
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tc && threadIdx.x < S::DN_TILES) {
    const int tile = threadIdx.x;
    unsigned target = 0;
    for (int j = 0; j < a.top_k; ++j) target += sh.dn_parts[j][tile];
    if (a.n_shared > 0) {
      int unused;
      const int groups = D / S::RT;
      target += (unsigned)tc_split(tile * kTcRows / S::RT, (tile * kTcRows + kTcRows - 1) / S::RT, groups, gridDim.x, 0, &unused);
    }
    sh.dn_target[tile] = target;
  }
  __syncthreads();
  const uint32_t tmem = tc ? sh.tmem_base : 0u;

  if (warp == 0 && !tc) {
    // =========================================================== producer (one lane per ring slot)
    // A single thread issues about two tiles per microsecond (a wait on the slot's barrier, the
    // transaction count, two bulk copies: each a long-latency instruction), which caps one block at
    // ~18 KB/us, a third of its share of the HBM bandwidth. So lane s of this warp owns ring slot s
    // and issues the tiles s, s + 16, ... of the block's whole sequence. The lanes run ONE loop
    // together: each tests its own slot (and its layer's routing) without blocking, and those that can
    // go work out their tile's place in the layer and issue it side by side. Lanes that each sat in a
    // blocking wait of their own would take turns, one lane's instructions at a time, and the warp
    // would again issue little more than a single thread.
    if (lane < kSStages) {
      constexpr int kQgPerJob = 2 * F / S::QG_ROWS;
      const long long n_total = (long long)a.n_layers * plan.per_layer;
      unsigned char* dst = slots + (size_t)lane * kSSlot;
      uint64_t* bar = &sh.full[lane];
      // the weight pointers of two layers (this one and the one the prefetches have reached), by layer parity
      struct LayerPointers { const uint16_t *router_weight, *shared_gate, *shared_up, *shared_down; int layer; } even, odd;
      even.layer = odd.layer = -1;
      auto pointers_of = [&](int layer) -> const LayerPointers& {
        LayerPointers& h = (layer & 1) ? odd : even;
        if (h.layer != layer) {
          const StackLayer* ly = a.layers + layer;
          h.router_weight = ly->router_weight;
          h.shared_gate = ly->shared_gate;
          h.shared_up = ly->shared_up;
          h.shared_down = ly->shared_down;
          h.layer = layer;
        }
        return h;
      };
      // One or two contiguous pieces of global memory that make up tile t of a layer; `second_at` is where the
      // second piece goes in the slot. A routed tile can only be described once its layer's routing is known.
      struct Tile { const void *first, *second; uint32_t first_bytes, second_bytes, second_at; };
      auto describe = [&](int layer, int t, Tile& d) -> bool {
        d.first = d.second = nullptr;
        d.first_bytes = d.second_bytes = d.second_at = 0;
        if (t < plan.s_sg) {
          // ---- router rows, padded to a multiple of the consumer count
          if (t < plan.n_r) {
            d.first = pointers_of(layer).router_weight + (size_t)(plan.r0 + t) * D;
            d.first_bytes = S::R_BYTES;
          }
        } else if (t < plan.s_qg) {
          // ---- shared gate/up: blocks of kSC units, each unit SG_SPLIT column slabs
          const int k = t - plan.s_sg;
          const int h = (k / kSC) % S::SG_SPLIT, unit = k / (kSC * S::SG_SPLIT) * kSC + k % kSC;
          if (unit < plan.n_u) {
            const size_t off = (size_t)(plan.u0 + unit) * S::SG_PAIRS * D + (size_t)h * S::SG_COLS;
            const LayerPointers& lp = pointers_of(layer);
            d.first = lp.shared_gate + off;
            d.second = lp.shared_up + off;
            d.first_bytes = d.second_bytes = d.second_at = S::SG_PART;
          }
        } else if (t < plan.s_sd) {
          // ---- routed gate/up
          if (sh.routed_layers <= layer) return false;
          __threadfence_block();
          const int q = plan.q0 + (t - plan.s_qg);
          const int choice = q / kQgPerJob, row0 = (q % kQgPerJob) * S::QG_ROWS;
          const RouteEntry& r = sh.routes[layer & 1].route[choice];
          if (r.gu_codes) {
            d.first = r.gu_codes + (size_t)row0 * (D / 2);
            d.second = r.gu_scales + (size_t)row0 * (D / 16);
            d.first_bytes = d.second_at = S::QG_CODES;
            d.second_bytes = S::QG_SCALES;
          }
        } else if (t < plan.s_qd) {
          // ---- shared down: expert-major, then row group, then the tiles of a group
          const int k = t - plan.s_sd, per_e = plan.n_g * S::SD_PER_GROUP;
          const int e = k / per_e, rem = k % per_e;
          d.first = pointers_of(layer).shared_down + ((size_t)e * D + (size_t)plan.g0 * S::RT) * F + (size_t)rem * S::SD_ROWS * F;
          d.first_bytes = S::SD_BYTES;
        } else if (t < plan.s_pad) {
          // ---- routed down: choice-major, then pairs of row groups
          if (sh.routed_layers <= layer) return false;
          __threadfence_block();
          const int k = t - plan.s_qd;
          const int choice = k / plan.n_gt, first = (k % plan.n_gt) * S::QD_PAIR;
          const uint32_t groups = (uint32_t)min(S::QD_PAIR, plan.n_g - first);
          const RouteEntry& r = sh.routes[layer & 1].route[choice];
          if (r.dn_codes) {
            const size_t row0 = (size_t)(plan.g0 + first) * S::RT;
            d.first = r.dn_codes + row0 * (F / 2);
            d.second = r.dn_scales + row0 * (F / 16);
            d.first_bytes = groups * S::QD_CODES;
            d.second_bytes = groups * S::QD_SCALES;
            d.second_at = S::QD_PAIR * S::QD_CODES;
          }
        }   // else: padding up to a multiple of the consumer count
        return true;
      };
      int layer = 0, t = lane;   // the tile to copy
      long long i = lane;        // its index in the block's whole sequence
      int asked = -1;            // (trace) the last layer whose routing this lane asked for
      long long stalled_since = clock64();
      long long slot_wait = 0, looked_at = clock64();   // (tracing, lane 0)
      while (true) {
        const bool more = i < n_total;
        if (!__any_sync(kProducerLanes, more)) break;
        if (__any_sync(kProducerLanes, sh.failed != 0)) break;
        bool ready = more;
        if (ready && ((t >= plan.s_qg && t < plan.s_sd) || (t >= plan.s_qd && t < plan.s_pad))) {
          if (t == plan.s_qg && asked != layer) {
            INK_TRACE(layer, kTrProdRouteWait);
            asked = layer;
          }
          ready = sh.routed_layers > layer;   // a routed tile: its layer's routing table must be there
        }
        if (ready && i >= kSStages) ready = mbar_test_wait(&sh.empty[lane], (uint32_t)((i / kSStages) - 1) & 1);
        if (ready) {
          __threadfence_block();
          if (t == plan.s_qg) INK_TRACE(layer, kTrProdRouteGot);
          Tile d;
          describe(layer, t, d);
          mbar_expect_tx(bar, d.first_bytes + d.second_bytes);
          if (d.first_bytes) bulk_g2s(dst, d.first, d.first_bytes, bar);
          if (d.second_bytes) bulk_g2s(dst + d.second_at, d.second, d.second_bytes, bar);
          if (t == plan.s_pad - 1) INK_TRACE(layer, kTrProdLayerIssued);
          if (lane == 0 && t + kSStages >= plan.per_layer) {
            INK_TRACE_VALUE(layer, kTrProdSlotWait, (unsigned long long)slot_wait);
            slot_wait = 0;
          }
          i += kSStages;
          t += kSStages;
          while (t >= plan.per_layer) {
            t -= plan.per_layer;
            ++layer;
          }
          stalled_since = clock64();
        } else if (more && clock64() - stalled_since > sh.limit) {
          sh.failed = 1;   // nothing for this lane within the limit: every wait of the launch gives up
        }
        if (a.trace && lane == 0 && more) {   // cycles with a tile to issue, its routing known, but the slot still in use
          const long long now = clock64();
          const bool routing_known = !((t >= plan.s_qg && t < plan.s_sd) || (t >= plan.s_qd && t < plan.s_pad)) || sh.routed_layers > layer;
          if (!ready && routing_known) slot_wait += now - looked_at;
          looked_at = now;
        }
        if (!__any_sync(kProducerLanes, ready)) __nanosleep(32);   // nothing to issue anywhere: leave the scheduler to the consumers
      }
    }
  } else if (warp == 0) {
    // =========================================================== producer (one lane, tensor-core variant)
    // The tile list is walked in order with running counters; the tensor-core warps rely on that order
    // (see tc_wait_issued).
    if (lane == 0) {
      long long issued = 0;   // tiles issued so far (all layers)
      bool alive = true;
      // claims the next ring slot; false once a wait has given up
      auto next_slot = [&](unsigned char*& dst, uint64_t*& bar) -> bool {
        const int slot = (int)(issued % kSStages);
        if (sh.failed) return false;
        if (issued >= kSStages && !mbar_wait(&sh.empty[slot], (uint32_t)((issued / kSStages) - 1) & 1, sh.limit)) {
          sh.failed = 1;
          return false;
        }
        dst = slots + (size_t)slot * kSSlot;
        bar = &sh.full[slot];
        ++issued;
        return true;
      };
      // tensor-core variant: tell the waiters how far the issue has come (see tc_wait_issued)
      auto publish = [&]() {
        if (tc) sh.issued = issued;
      };
      unsigned char* dst = nullptr;
      uint64_t* bar = nullptr;
      constexpr int kQgPerJob = 2 * F / S::QG_ROWS;
      for (int layer = 0; layer < a.n_layers && alive; ++layer) {
        const StackLayer ly = a.layers[layer];
        if (tc) {   // the layer's four TMA descriptors live in global memory: bring them to the copy engine early
          for (int m = 0; m < 4; ++m)
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<const unsigned char*>(ly.tmaps) + m * 128) : "memory");
        }
        // ---- router rows, padded to a multiple of the consumer count
        for (int t = 0; t < plan.s_sg && alive; ++t) {
          if (!(alive = next_slot(dst, bar))) break;
          if (t < plan.n_r) {
            mbar_expect_tx(bar, S::R_BYTES);
            bulk_g2s(dst, ly.router_weight + (size_t)(plan.r0 + t) * D, S::R_BYTES, bar);
          } else {
            mbar_expect_tx(bar, 0);
          }
          publish();
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
              publish();
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
        if (tc) {
          // units of 128 rows x 256 columns (codes and scales, two ring slots) for the tensor cores
          const unsigned char* maps = reinterpret_cast<const unsigned char*>(ly.tmaps);
          int chunk = plan.qu0 % S::GU_CHUNKS, tile = (plan.qu0 / S::GU_CHUNKS) % S::GU_TILES;
          int choice = plan.qu0 / (S::GU_CHUNKS * S::GU_TILES);
          for (int i = 0; i < plan.n_qu; ++i) {
            unsigned char* second = nullptr;
            uint64_t* bar2 = nullptr;
            if (!(alive = next_slot(dst, bar)) || !(alive = next_slot(second, bar2))) break;
            const RouteEntry& r = table.route[choice];
            const int expert = r.gu_codes ? r.expert : 0;   // an inactive route streams expert 0 and is zeroed at the end
            mbar_expect_tx(bar, kTcUnitBytes);
            tc_tma_3d(dst, maps, chunk * 128, tile * kTcRows, expert, bar);
            tc_tma_3d(dst + kTcCodeBytes, maps + 128, chunk * 16, tile * kTcRows, expert, bar);
            mbar_expect_tx(bar2, 0);
            publish();
            if (++chunk == S::GU_CHUNKS) {
              chunk = 0;
              if (++tile == S::GU_TILES) {
                tile = 0;
                ++choice;
              }
            }
          }
        } else {
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
            publish();
          }
        }
        if (tc && alive && (plan.n_sd_real & 1)) {   // keeps the units that follow on even slots
          if (!(alive = next_slot(dst, bar))) break;
          mbar_expect_tx(bar, 0);
          publish();
        }
        // ---- routed down: units of 128 rows x 256 columns for the tensor cores
        if (tc && alive) {
          const unsigned char* maps = reinterpret_cast<const unsigned char*>(ly.tmaps);
          int chunk = plan.du0 % S::DN_CHUNKS, tile = (plan.du0 / S::DN_CHUNKS) % S::DN_TILES;
          int choice = plan.du0 / (S::DN_CHUNKS * S::DN_TILES);
          for (int i = 0; i < plan.n_du; ++i) {
            unsigned char* second = nullptr;
            uint64_t* bar2 = nullptr;
            if (!(alive = next_slot(dst, bar)) || !(alive = next_slot(second, bar2))) break;
            const RouteEntry& r = table.route[choice];
            const int expert = r.dn_codes ? r.expert : 0;
            mbar_expect_tx(bar, kTcUnitBytes);
            tc_tma_3d(dst, maps + 256, chunk * 128, tile * kTcRows, expert, bar);
            tc_tma_3d(dst + kTcCodeBytes, maps + 384, chunk * 16, tile * kTcRows, expert, bar);
            mbar_expect_tx(bar2, 0);
            publish();
            if (++chunk == S::DN_CHUNKS) {
              chunk = 0;
              if (++tile == S::DN_TILES) {
                tile = 0;
                ++choice;
              }
            }
          }
        }
        // ---- routed down: choice-major, then row group
        for (int choice = 0; choice < a.top_k && alive && !tc; ++choice) {
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
          publish();
        }
        INK_TRACE(layer, kTrProdLayerIssued);
      }
    }
  } else if (warp == kSC + 1) {
    // =========================================================== auxiliary warp
    long long tc_base = 0, qseq = 0, dseq = 0;   // ring index of the layer's first tile; units and tile segments so far
    load_route_consts(a, 0, &sh);
    for (int layer = 0; layer < a.n_layers; ++layer) {
      const unsigned* sync = a.sync + (size_t)layer * kSyncWordsPerLayer;
      // every block resolves the routing for itself (same inputs, same arithmetic, same result): the
      // code stays warm in this SM's instruction cache and nothing has to be published between blocks
      if (!stack_router_tail(a, a.layers[layer], layer, &sh)) break;
      // the constants of this layer are in the route table now; fetch the next layer's while this one streams.
      // (The consumers read this layer's biases only before they publish its scores, i.e. before this point.)
      if (layer + 1 < a.n_layers) load_route_consts(a, layer + 1, &sh);
      if (!tc && lane == 0) {
        // One lane polls the layer's grid-wide counters for the whole block and raises a flag in shared memory
        // for each: eight polling warps per block crowd the counter's L2 line and hold up its increments.
        const unsigned epoch1 = sh.epoch1;
        wait_global(sync + kShGuDone, epoch1 * gridDim.x, &sh);
        __threadfence_block();
        sh.seen[0] = layer + 1;
        wait_global(sync + kRtGuDone, epoch1 * gridDim.x, &sh);
        __threadfence_block();
        sh.seen[1] = layer + 1;
      }
      if (tc && lane == 0 && !sh.failed) {
        // ---- the routed projections on the tensor cores: one thread issues. A unit is 128 weight rows x
        // 256 columns in two ring slots; four MMAs of 64 columns each accumulate it into the tile's accumulator.
        auto issue = [&](volatile int* ready, int first_tile, int u0, int n_units, int chunks, const unsigned char* operand,
                         int operand_chunk_bytes, uint32_t idesc) {
          const long long t0 = clock64();
          while (*ready <= layer && !sh.failed)
            if (clock64() - t0 > sh.limit) sh.failed = 1;
          __threadfence_block();
          tc_fence_after();
          if (ready == &sh.act_ready) INK_TRACE(layer, kTrMmaDownStart);
          int chunk = u0 % chunks;
          for (int i = 0; i < n_units && !sh.failed; ++i) {
            const long long t = tc_base + first_tile + 2 * i;
            const int slot = (int)(t % kSStages), sfs = (int)(qseq % kTcSfSlots), dbuf = (int)(dseq & 1);
            const bool seg_first = (i == 0 || chunk == 0), seg_last = (i + 1 == n_units || chunk == chunks - 1);
            if (seg_first && !tc_wait(&sh.d_empty[dbuf], (uint32_t)((dseq >> 1) & 1) ^ 1u, &sh)) break;
            if (!tc_wait_issued(t, &sh) || !tc_wait(&sh.full[slot], (uint32_t)(t / kSStages) & 1u, &sh)) break;
            if (!tc_wait(&sh.sf_full[sfs], (uint32_t)(qseq / kTcSfSlots) & 1u, &sh)) break;
            tc_fence_after();
            const uint64_t ad = tc_desc_sw128(smem_u32(slots + (size_t)slot * kSSlot));
            const uint64_t bd = tc_desc_sw128(smem_u32(operand + (size_t)chunk * operand_chunk_bytes));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc_mma(tmem + kTcColD + dbuf * 32, ad + 2 * k, bd + 2 * k, idesc, (seg_first && k == 0) ? 0u : 1u,
                     tmem + kTcColSfa + sfs * 16 + k * 4, tmem + kTcColSfb + (chunk * 4 + k) * 4);
            tc_commit(&sh.empty[slot]);
            tc_commit(&sh.empty[slot + 1]);
            tc_commit(&sh.sf_empty[sfs]);
            if (seg_last) {
              tc_commit(&sh.d_full[dbuf]);
              ++dseq;
            }
            ++qseq;
            if (++chunk == chunks) chunk = 0;
          }
        };
        INK_TRACE(layer, kTrMmaGuStart);
        issue(&sh.x_ready, plan.s_qg, plan.qu0, plan.n_qu, S::GU_CHUNKS, s_xdig, 8 * 128, tc_idesc(8));
        INK_TRACE(layer, kTrMmaGuEnd);
        issue(&sh.act_ready, plan.s_qd, plan.du0, plan.n_du, S::DN_CHUNKS, s_adig, 32 * 128, tc_idesc(32));
        INK_TRACE(layer, kTrMmaDownEnd);
      }
      tc_base += plan.per_layer;
      // the warp leaves the loop together: lane 0 may have been issuing for a long time
      __syncwarp();
      const int failed = sh.failed;
      if (__shfl_sync(0xffffffffu, failed, 0)) break;
    }
  } else if (warp <= kSC) {
    // =========================================================== consumers
    const int cw = warp - 1, ct = threadIdx.x - 32;
    constexpr int VG = VecShape<D>::VG, VT = VecShape<D>::VT;   // groups of eight elements per thread, threads that hold some
    const bool holder = ct < VT;

    long long waited = 0;   // (tracing) cycles this warp waited for tiles since the last section stamp
    long long busy = 0, tile_from = 0;   // (tracing) cycles between a tile's arrival and its release
    long long base = 0;   // index of this layer's first tile in the block's whole sequence
    // first tile index >= start that belongs to this consumer (tile t belongs to consumer t % kSC; a layer is a
    // whole number of rounds, so a ring slot always comes back to the same warp)
    auto first_of = [&](int start) -> int { return start + (cw - start % kSC + kSC) % kSC; };
    auto take = [&](int t, const unsigned char*& src, int& slot) -> bool {
      const long long i = base + t;
      slot = (int)(i % kSStages);
      bool ok = !sh.failed;
      if (tc) {   // the slot's previous tile may have been a tensor-core unit: one lane checks the issue count
        if (ok && lane == 0) ok = tc_wait_issued(i, &sh);
        ok = __all_sync(0xffffffffu, ok);
      }
      const long long wait_from = a.trace ? clock64() : 0;
      if (ok) ok = mbar_wait(&sh.full[slot], (uint32_t)(i / kSStages) & 1, sh.limit);
      if (a.trace) {
        tile_from = clock64();
        waited += tile_from - wait_from;
      }
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
      if (a.trace) busy += clock64() - tile_from;
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
    // The same per WARP: called once by each warp that has tiles in `section`, after its last one; `warps` is
    // how many such warps the block has. (A shared-memory atomic with its answer and a shuffle cost ~500 cycles
    // next to a tile's 1200..2000, and the consumers are what the kernel waits for: so not once per tile.)
    auto warp_done = [&](int layer, int section, int warps, bool fence) -> bool {
      int done = 0;
      __syncwarp();
      if (lane == 0) {
        if (fence) __threadfence();
        else __threadfence_block();
        done = atomicAdd(&sh.done[layer & 1][section], 1) + 1;
        __threadfence_block();
      }
      done = __shfl_sync(0xffffffffu, done, 0);
      return done == warps;
    };

    const int sub = warp & 3;   // the tensor-memory subpartition this warp can reach
    // stages the next activation vector for the gate/up phases; `ready` = layers staged once this returns
    auto stage = [&](const uint4 (&xb)[VG], float amax_bound, int ready) {
      if (!tc) {
        stage_x<D>(s_x16, s_xbf, xb, amax_bound, &sh, ct);
        return;
      }
      stage_x_tc<D>(s_xdig, s_xbf, xb, amax_bound, &sh, ct);
      if (ct == 0 && ready >= 2) INK_TRACE(ready - 2, kTrXDigits);
      tc_proxy_fence();   // the digit rows are read by the tensor core
      consumer_sync();
      if (ct == 0 && ready >= 2) INK_TRACE(ready - 2, kTrXVisible);
      if (cw < 4) tc_upload_scales(tmem, sub, &sh.sfbx[0][0], 256, kTcDigits, D / 64, lane);
      consumer_sync();
      if (ct == 0) {
        __threadfence_block();
        sh.x_ready = ready;
      }
    };

    // ---- first activation vector
    {
      uint4 xb[VG];
      uint32_t amax_bits = 0;
#pragma unroll
      for (int g = 0; g < VG; ++g) {
        xb[g] = holder ? reinterpret_cast<const uint4*>(a.x)[g * VT + ct] : make_uint4(0, 0, 0, 0);
        const uint32_t w4[4] = {xb[g].x, xb[g].y, xb[g].z, xb[g].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) amax_bits = max(amax_bits, max(w4[k] & 0x7fffu, (w4[k] >> 16) & 0x7fffu));
      }
      float amax = bf16_to_f32(amax_bits);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (lane == 0) sh.red[cw][0] = amax;
      consumer_sync();
      amax = 0.f;
      for (int w = 0; w < kSC; ++w) amax = fmaxf(amax, sh.red[w][0]);
      stage(xb, amax, 1);
      consumer_sync();
    }

    for (int layer = 0; layer < a.n_layers; ++layer, base += plan.per_layer) {
      const uint16_t* norm_weight = a.layers[layer].norm_weight;
      unsigned* sync = a.sync + (size_t)layer * kSyncWordsPerLayer;
      const int par = layer & 1;
      const unsigned epoch1 = sh.epoch1;
      // slot of the ranks' deliveries: alternates with every block of every launch
      const int xpar = (int)(((epoch1 - 1u) * (unsigned)a.n_layers + (unsigned)layer) & 1u);
      const unsigned tag = layer_tag(epoch1, a.n_layers, layer);
      const float x_inverse = sh.x_inverse;
      const bool tracer = (ct == 0);
      if (tracer) INK_TRACE(layer, kTrLayerStart);
      // blocks that own no tile of a section still have to be counted
      if (ct == 0) {
        if (plan.n_sg == 0) red_release_add(sync + kShGuDone, 1u);
        if (plan.n_q == 0 && !tc) red_release_add(sync + kRtGuDone, 1u);   // (the tensor-core path counts tiles)
      }
      // ------------------------------------------------ router rows
      if (plan.n_r > 0) wait_flag(&sh.consts_layers, layer, &sh, lane);   // the layer's biases (loaded a layer ahead)
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
          if (lane == 0) {   // one word per row: the routing warps of all blocks poll for them
            const float l = round_bf16(acc);
            const float score = row < a.experts ? round_bf16(1.f / (1.f + __expf(-l))) + sh.consts.bias[row] : 0.f;
            unsigned long long* at = a.scores + (size_t)par * total_rows + row;
            asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(at), "l"(router_word(score, l, router_tag(tag))) : "memory");
          }
        } else {
          release(slot);
        }
      }
      if (tracer) INK_TRACE(layer, kTrRouterDone);
      if (tracer) INK_TRACE_VALUE(layer, kTrWaitRouter, (unsigned long long)waited);
      waited = busy = 0;
      // ------------------------------------------------ shared gate/up
      {
        float g[S::SG_PAIRS], u[S::SG_PAIRS];
        for (int t = first_of(plan.s_sg); t < plan.s_qg; t += kSC) {
          const unsigned char* src;
          int slot;
          if (!take(t, src, slot)) break;
          const int i = t - plan.s_sg;
          const int h = (i / kSC) % S::SG_SPLIT, blk = i / (kSC * S::SG_SPLIT);
          const int unit = blk * kSC + i % kSC;
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
          if (t + kSC >= plan.s_qg && warp_done(layer, 0, min(kSC, plan.n_sg), true) && lane == 0) red_release_add(sync + kShGuDone, 1u);
        }
      }
      if (tracer) INK_TRACE(layer, kTrShGuDone);
      if (tracer) INK_TRACE_VALUE(layer, kTrWaitShGu, (unsigned long long)waited);
      if (tracer) INK_TRACE_VALUE(layer, kTrBusyShGu, (unsigned long long)busy);
      waited = busy = 0;
      if (tc) {
        // this block is done with the BF16 copy of x: the tensor-core warps may overwrite it later on
        consumer_sync();
        if (ct == 0) {
          __threadfence_block();
          sh.sg_done = layer + 1;
        }
      }
      // ------------------------------------------------ routed gate/up
      if constexpr (!tc) {
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
            // every lane accumulates its columns of all rows of the tile, then ONE multi-row reduction
            // (QG_ROWS/2 + ... shuffles instead of five per row) leaves row r's total in its owner lane
            float acc[S::QG_ROWS];
#pragma unroll
            for (int row = 0; row < S::QG_ROWS; ++row) {
              const unsigned char* codes = src + (size_t)row * (D / 2) + lane * 16;
              const unsigned char* scales = src + S::QG_CODES + (size_t)row * (D / 16) + lane * 2;
              float sum = 0.f;
#pragma unroll
              for (int j = 0; j < S::QG_CPL; ++j)
                sum += dot32(*reinterpret_cast<const uint4*>(codes + j * 512), *reinterpret_cast<const uint16_t*>(scales + j * 64), xr[j]);
              acc[row] = sum;
            }
            release(slot);
            const float mine = multi_reduce<S::QG_ROWS>(acc, lane) * scale;
            // even rows are gate, odd rows up: the owner of an even row fetches the odd row next to it
            constexpr int kOwnerStride = 32 / S::QG_ROWS;
            const float up = __shfl_down_sync(0xffffffffu, mine, kOwnerStride);
            const int row = reduced_row<S::QG_ROWS>(lane);
            if (reduced_owner<S::QG_ROWS>(lane) && (row & 1) == 0) y[row >> 1] = (uint16_t)f32_to_bf16_bits(silu_mul(mine, up));
          } else {
            release(slot);
          }
          if (t + kSC >= plan.s_sd && warp_done(layer, 1, min(kSC, plan.n_q), true) && lane == 0) red_release_add(sync + kRtGuDone, 1u);
        }
      }
      if (tracer) INK_TRACE(layer, kTrRtGuDone);
      if (tracer) INK_TRACE_VALUE(layer, kTrWaitRtGu, (unsigned long long)waited);
      if (tracer) INK_TRACE_VALUE(layer, kTrBusyRtGu, (unsigned long long)busy);
      waited = busy = 0;
      // The phases that follow are not separated by block-wide barriers: a warp that is done with its gate/up
      // tiles goes on with its down tiles, and waits only for the staging flag of the vector it needs. Only
      // where the shared experts' staging area overlaps the x staging (narrow experts) must every warp be
      // past its gate/up tiles first.
      if (!tc && kSMaxTopK * F * 2 < D * 4) consumer_sync();
      // ------------------------------------------------ shared down
      if (tc) {
        if (lane == 0) wait_global(sync + kShGuDone, epoch1 * gridDim.x, &sh);
      } else {
        wait_flag(&sh.seen[0], layer, &sh, lane);
      }
      if (lane == 0) wait_routing(layer, &sh);
      __syncwarp();
      if (tracer) INK_TRACE(layer, kTrShGuAll);
      for (int e = cw; e < a.n_shared; e += kSC) {   // warp e stages shared expert e: act * gamma, BF16
        if (!sh.failed) {
          const uint4* src = reinterpret_cast<const uint4*>(a.shared_activated + ((size_t)par * a.n_shared + e) * F);
          const float gamma = sh.routes[par].gamma[e];
          uint4* dst = reinterpret_cast<uint4*>(s_sact + (size_t)e * F);
          constexpr int N = F / 256;
          uint4 v[N];
#pragma unroll
          for (int n = 0; n < N; ++n) v[n] = __ldcg(src + n * 32 + lane);
#pragma unroll
          for (int n = 0; n < N; ++n) {
            uint4 o;
            o.x = f32_to_bf16_bits(bf16lo(v[n].x) * gamma) | (f32_to_bf16_bits(bf16hi(v[n].x) * gamma) << 16);
            o.y = f32_to_bf16_bits(bf16lo(v[n].y) * gamma) | (f32_to_bf16_bits(bf16hi(v[n].y) * gamma) << 16);
            o.z = f32_to_bf16_bits(bf16lo(v[n].z) * gamma) | (f32_to_bf16_bits(bf16hi(v[n].z) * gamma) << 16);
            o.w = f32_to_bf16_bits(bf16lo(v[n].w) * gamma) | (f32_to_bf16_bits(bf16hi(v[n].w) * gamma) << 16);
            dst[n * 32 + lane] = o;
          }
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          sh.sact_flag[e] = layer + 1;
        }
      }
      unsigned sact_seen = 0;
      bool last_of_block = false;   // this warp reported the block's last down tile (CUDA-core variant)
      for (int t = first_of(plan.s_sd); t < plan.s_qd; t += kSC) {
        const unsigned char* src;
        int slot;
        if (!take(t, src, slot)) break;
        const int i = t - plan.s_sd;
        if (i >= plan.n_sd_real) {   // the padding tile of the tensor-core variant
          release(slot);
          continue;
        }
        const int per_e = plan.n_g * S::SD_PER_GROUP;
        const int e = i / per_e, rem = i % per_e;
        const int local0 = (rem / S::SD_PER_GROUP) * S::RT + (rem % S::SD_PER_GROUP) * S::SD_ROWS;
        if (!((sact_seen >> e) & 1u)) {   // once per layer and shared expert
          wait_flag(&sh.sact_flag[e], layer, &sh, lane);
          sact_seen |= 1u << e;
        }
        const uint4* xs = reinterpret_cast<const uint4*>(s_sact + (size_t)e * F);
        float acc[S::SD_ROWS];
#pragma unroll
        for (int row = 0; row < S::SD_ROWS; ++row) {
          float sum = 0.f;
#pragma unroll 2
          for (int c = 0; c < S::SD_CPL; ++c) {
            const int chunk = c * 32 + lane;
            sum = dot8(*reinterpret_cast<const uint4*>(src + (size_t)row * F * 2 + chunk * 16), xs[chunk], sum);
          }
          acc[row] = sum;
        }
        {
          const float total = multi_reduce<S::SD_ROWS>(acc, lane);   // one reduction for all rows of the tile
          if (reduced_owner<S::SD_ROWS>(lane)) {
            const int row = reduced_row<S::SD_ROWS>(lane);
            if (tc) a.sd_out[((size_t)par * a.n_shared + e) * D + (size_t)plan.g0 * S::RT + local0 + row] = round_bf16(total);
            else sh.contrib[a.top_k + e][local0 + row] = round_bf16(total);
          }
        }
        release(slot);
        if (!tc) {
          // the warps are counted once for all their down tiles (shared + routed): here only by a warp without routed ones
          if (t + kSC >= plan.s_pad && warp_done(layer, 2, min(kSC, plan.n_sd + plan.n_qd), false)) last_of_block = true;
        } else if (section_done(layer, 2, plan.n_sd_real, t + kSC >= plan.s_sd + plan.n_sd_real) && !sh.failed) {
          // the block's shared-expert rows are in global memory: count the block at every 128-row tile it
          // touches; whoever completes a tile (this warp or a tensor-core epilogue) sums and delivers it
          const int row_a = plan.g0 * S::RT, row_b = (plan.g0 + plan.n_g) * S::RT - 1;
          for (int tile = row_a / kTcRows; tile <= row_b / kTcRows; ++tile) {
            int last = 0;
            if (lane == 0)
              last = atomicAdd(a.tilesync + (size_t)layer * kTileCountersPerLayer + kSMaxTopK * 32 + tile, 1u) + 1u ==
                     epoch1 * sh.dn_target[tile];
            if (__shfl_sync(0xffffffffu, last, 0)) {
              __threadfence();
              finish_row_tile<D, F>(a, &sh, layer, par, xpar, tile, lane, 32);
              __syncwarp();   // (the lanes waited for different rows)
            }
          }
        }
      }
      if (tracer) INK_TRACE(layer, kTrShDownDone);
      if (tracer) INK_TRACE_VALUE(layer, kTrWaitShDown, (unsigned long long)waited);
      waited = 0;
      if constexpr (!tc) {
      // ------------------------------------------------ routed down
      wait_flag(&sh.seen[1], layer, &sh, lane);
      if (tracer) INK_TRACE(layer, kTrRtGuAll);
      for (int job = cw; job < a.top_k; job += kSC) {   // warp j stages route j
        if (!sh.failed) {
          const float inverse = warp_stage_f16<F>(a.activated + ((size_t)par * a.top_k + job) * F, s_act + (size_t)job * F, lane);
          if (lane == 0) sh.inverse[job] = inverse;
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          sh.act_flag[job] = layer + 1;
        }
      }
      if (tracer) INK_TRACE(layer, kTrActStaged);
      {
        const int sl = lane % S::LPR, rp = lane / S::LPR;
        uint32_t xr[S::QD_CPL][16];
        int loaded = -1;
        for (int t = first_of(plan.s_qd); t < plan.s_pad; t += kSC) {
          const unsigned char* src;
          int slot;
          if (!take(t, src, slot)) break;
          const int i = t - plan.s_qd;
          const int choice = i / plan.n_gt, first_group = (i % plan.n_gt) * S::QD_PAIR;
          const int groups_here = min(S::QD_PAIR, plan.n_g - first_group);
          const RouteEntry r = sh.routes[par].route[choice];
          if (r.dn_codes) {
            if (loaded != choice) {
              loaded = choice;
              wait_flag(&sh.act_flag[choice], layer, &sh, lane);
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
            const unsigned char* tile = src;
#pragma unroll 1
            for (int sub = 0; sub < groups_here; ++sub) {
            const int local0 = (first_group + sub) * S::RT;
            const unsigned char* src = tile + (size_t)sub * S::QD_CODES;                                  // this group's codes
            const unsigned char* src_scales = tile + S::QD_PAIR * S::QD_CODES + (size_t)sub * S::QD_SCALES;   // and scales
            if constexpr (S::LPR == 32) {
              // a row spans the warp: every lane accumulates its columns of all RT rows, one multi-row reduction
              float acc[S::RT];
#pragma unroll
              for (int row = 0; row < S::RT; ++row) {
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < S::QD_CPL; ++j) {
                  const int chunk = j * 32 + lane;
                  sum += dot32(*reinterpret_cast<const uint4*>(src + (size_t)row * (F / 2) + chunk * 16),
                               *reinterpret_cast<const uint16_t*>(src_scales + (size_t)row * (F / 16) + chunk * 2), xr[j]);
                }
                acc[row] = sum;
              }
              const float total = multi_reduce<S::RT>(acc, lane);
              if (reduced_owner<S::RT>(lane)) {
                const float down = round_bf16(total * scale);
                sh.contrib[choice][local0 + reduced_row<S::RT>(lane)] = round_bf16(down * r.weight);
              }
            } else {
#pragma unroll 1
              for (int p = 0; p < S::PASSES; ++p) {
                const int row = p * S::RPP + rp;
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < S::QD_CPL; ++j) {
                  const int chunk = j * S::LPR + sl;
                  acc += dot32(*reinterpret_cast<const uint4*>(src + (size_t)row * (F / 2) + chunk * 16),
                               *reinterpret_cast<const uint16_t*>(src_scales + (size_t)row * (F / 16) + chunk * 2), xr[j]);
                }
#pragma unroll
                for (int o = S::LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (sl == 0) {
                  const float down = round_bf16(acc * scale);
                  sh.contrib[choice][local0 + row] = round_bf16(down * r.weight);
                }
              }
            }
            }   // row groups of the tile
            release(slot);
          } else {
            release(slot);
          }
          if (t + kSC >= plan.s_pad && warp_done(layer, 2, min(kSC, plan.n_sd + plan.n_qd), false)) last_of_block = true;
        }
        // The warp that finished the block's last down tile sums the contributions in a
        // fixed order (routes in choice order, then the shared experts) and publishes them.
        // (Routed-down tiles start only after every shared-down tile of the block is done, so
        // the last tile is always a routed one.)
        if (last_of_block && !sh.failed) {
          __syncwarp();
          // hand this block's rows over (to every rank, itself included), then sum what the ranks sent for them
          if (a.world == 1) {
            for (int row = lane; row < plan.n_g * S::RT; row += 32) {
              float total = 0.f;
              for (int j = 0; j < n_jobs; ++j) total += sh.contrib[j][row];
              send_row<D>(a, xpar, tag, plan.g0 * S::RT + row, total);
            }
          } else {
            // to the peers two rows at a time (the block's rows start at a multiple of RT, RT is even): half as
            // many packets on the links
            for (int pair = lane; pair < plan.n_g * S::RT / 2; pair += 32) {
              float t0 = 0.f, t1 = 0.f;
              for (int j = 0; j < n_jobs; ++j) {
                t0 += sh.contrib[j][2 * pair];
                t1 += sh.contrib[j][2 * pair + 1];
              }
              const size_t at = ((size_t)xpar * a.world + a.rank) * D + (size_t)plan.g0 * S::RT + 2 * pair;
              for (int r = 0; r < a.world; ++r) st_tagged2_sys(a.peer_inbox[r] + at, t0, t1, tag);
            }
          }
          if (lane == 0) INK_TRACE(layer, kTrRowsSent);
          if (a.world > 1)
            for (int row = lane; row < plan.n_g * S::RT; row += 32) gather_row<D>(a, &sh, xpar, tag, plan.g0 * S::RT + row);
          __syncwarp();   // the lanes waited for different rows: together again before anything warp-wide
        }
      }
      }   // CUDA-core routed down
      // padding tiles at the end of the layer
      for (int t = first_of(plan.s_pad); t < plan.per_layer; t += kSC) {
        const unsigned char* src;
        int slot;
        if (!take(t, src, slot)) break;
        release(slot);
      }
      if (tracer) INK_TRACE(layer, kTrRtDownDone);
      if (tracer) INK_TRACE_VALUE(layer, kTrWaitRtDown, (unsigned long long)waited);
      waited = 0;
      const unsigned long long* summed = a.summed + (size_t)xpar * D;
      if (!a.glue) {
        // one block only: each block writes its own rows, summed over the ranks, as they arrive
        for (int row = ct; row < plan.n_g * S::RT; row += kSC * 32) {
          const size_t i = (size_t)plan.g0 * S::RT + row;
          a.partial[i] = wait_tagged(summed + i, tag, &sh);
        }
        break;
      }
      // the other set of activation maxima is free (its readers finished before this layer's deliveries
      // completed) and is needed clean by the next layer
      if (tc && blockIdx.x == 0 && ct < kSMaxTopK) a.act_amax[((layer + 1) & 1) * kSMaxTopK + ct] = 0u;
      // ------------------------------------------------ residual add + RMS norm (every block, redundantly)
      {
        const uint16_t* res_in = a.residual + (size_t)par * D;
        uint16_t* res_out = a.residual + (size_t)(par ^ 1) * D;
        float sumsq = 0.f, amax_h = 0.f, amax_w = 0.f;
        // all loads first (they are independent), arithmetic after: one L2 round trip; 16-byte loads of eight
        // consecutive elements keep both the loads and the code that follows short
        // (one answer per warp: what follows synchronises the warp, so its lanes must not disagree about a
        // failure that another warp reports while they read the flag)
        __syncwarp();
        const bool live = !__any_sync(0xffffffffu, sh.failed != 0) && holder;
        uint4 res[VG], nw[VG];
        float part[VG][8];
#pragma unroll
        for (int g = 0; g < VG; ++g) {
          const int group = g * VT + ct;
          res[g] = live ? __ldcg(reinterpret_cast<const uint4*>(res_in) + group) : make_uint4(0, 0, 0, 0);
          nw[g] = live ? reinterpret_cast<const uint4*>(norm_weight)[group] : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int k = 0; k < 8; ++k) part[g][k] = 0.f;
        }
        // The layer's output rows, summed over the ranks, as their owners publish them: every thread polls the
        // tagged words of its own elements (all of a round in flight together), so a block goes on as soon as
        // the last row it needs is there -- no counter, no fence.
        if (live) {
          unsigned long long w[VG][8];
          // Polling has to be gentle: every block polls the same 32 KB, and on B200 the polls delay the very stores
          // they wait for (a round of everything from every thread costs the L2 more than the rows take to arrive).
          // So ONE warp of the block watches one word per sending block -- the last row of its slice -- with a pause
          // between rounds, and raises a flag for the other warps ...
          if (cw == 0) {
            const int groups = D / S::RT;
            const long long t0 = clock64();
            for (;;) {
              bool there = true;
              for (int b = lane; b < (int)gridDim.x; b += 32) {
                const int first = (int)((long long)b * groups / gridDim.x), end = (int)((long long)(b + 1) * groups / gridDim.x);
                if (end > first) there = there && has_tag(ld_tagged(summed + (size_t)end * S::RT - 1), tag);
              }
              if (__all_sync(0xffffffffu, there) || sh.failed) break;
              if (clock64() - t0 > sh.limit) sh.failed = 1;
              __nanosleep(sh.pause);
            }
            __syncwarp();
            if (lane == 0) {
              __threadfence_block();
              sh.rows_seen = layer + 1;
            }
          } else {
            wait_flag(&sh.rows_seen, layer, &sh, lane);
          }
          // ... then every thread loads its own elements; a sender's other rows may be a moment behind its last one
          bool all = true;
#pragma unroll
          for (int g = 0; g < VG; ++g) {
            const unsigned long long* src = summed + (size_t)(g * VT + ct) * 8;
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
              unsigned long long pair[2];
              ld_tagged2(src + k, pair);
              w[g][k] = pair[0];
              w[g][k + 1] = pair[1];
              all = all && has_tag(pair[0], tag) && has_tag(pair[1], tag);
            }
          }
          const long long t0 = clock64();
          while (!all && !sh.failed) {
            __nanosleep(sh.pause);
            all = true;
#pragma unroll
            for (int g = 0; g < VG; ++g) {
              const unsigned long long* src = summed + (size_t)(g * VT + ct) * 8;
#pragma unroll
              for (int k = 0; k < 8; k += 2) {
                if (!has_tag(w[g][k], tag) || !has_tag(w[g][k + 1], tag)) {
                  unsigned long long pair[2];
                  ld_tagged2(src + k, pair);
                  w[g][k] = pair[0];
                  w[g][k + 1] = pair[1];
                  all = all && has_tag(pair[0], tag) && has_tag(pair[1], tag);
                }
              }
            }
            if (clock64() - t0 > sh.limit) sh.failed = 1;
          }
#pragma unroll
          for (int g = 0; g < VG; ++g)
#pragma unroll
            for (int k = 0; k < 8; ++k) part[g][k] = sh.failed ? 0.f : value_of(w[g][k]);
        }
        if (tracer) INK_TRACE(layer, kTrDownAll);
        float h[VG][8];
#pragma unroll
        for (int g = 0; g < VG; ++g) {
          const uint32_t r4[4] = {res[g].x, res[g].y, res[g].z, res[g].w}, w4[4] = {nw[g].x, nw[g].y, nw[g].z, nw[g].w};
          uint32_t packed[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float lo = round_bf16(bf16lo(r4[k]) + round_bf16(part[g][2 * k]));
            const float hi = round_bf16(bf16hi(r4[k]) + round_bf16(part[g][2 * k + 1]));
            h[g][2 * k] = lo;
            h[g][2 * k + 1] = hi;
            sumsq = fmaf(lo, lo, fmaf(hi, hi, sumsq));
            amax_h = fmaxf(amax_h, fmaxf(fabsf(lo), fabsf(hi)));
            amax_w = fmaxf(amax_w, fmaxf(fabsf(bf16lo(w4[k])), fabsf(bf16hi(w4[k]))));
            packed[k] = f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
          }
          if (blockIdx.x == 0 && live) {
            const int group = g * VT + ct;
            reinterpret_cast<uint4*>(res_out)[group] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            if (layer + 1 == a.n_layers) {
              float4* out = reinterpret_cast<float4*>(a.partial) + (size_t)group * 2;
              out[0] = make_float4(part[g][0], part[g][1], part[g][2], part[g][3]);
              out[1] = make_float4(part[g][4], part[g][5], part[g][6], part[g][7]);
            }
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
        if (tracer) INK_TRACE(layer, kTrNormReduced);
        sumsq = 0.f;
        amax_h = 0.f;
        amax_w = 0.f;
        for (int w = 0; w < kSC; ++w) {
          sumsq += sh.red[w][0];
          amax_h = fmaxf(amax_h, sh.red[w][1]);
          amax_w = fmaxf(amax_w, sh.red[w][2]);
        }
        const float scale = rsqrtf(sumsq / (float)D + a.eps);
        uint4 xb[VG];
#pragma unroll
        for (int g = 0; g < VG; ++g) {
          const uint32_t w4[4] = {nw[g].x, nw[g].y, nw[g].z, nw[g].w};
          uint32_t packed[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float lo = round_bf16(h[g][2 * k] * scale) * bf16lo(w4[k]);
            const float hi = round_bf16(h[g][2 * k + 1] * scale) * bf16hi(w4[k]);
            packed[k] = f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
          }
          xb[g] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
        if (layer + 1 == a.n_layers) {
          if (blockIdx.x == 0 && live) {
#pragma unroll
            for (int g = 0; g < VG; ++g) reinterpret_cast<uint4*>(a.normed_out)[g * VT + ct] = xb[g];
          }
        } else {
          stage(xb, amax_h * scale * amax_w, layer + 2);
          // contributions of inactive routes must read as zero in the next layer too
          for (int i = ct; i < (kSMaxTopK + kSMaxShared) * kSMaxRows; i += kSC * 32) (&sh.contrib[0][0])[i] = 0.f;
          if (ct < 3) sh.done[par ^ 1][ct] = 0;
        }
        consumer_sync();
        if (tracer) INK_TRACE(layer, kTrNormDone);
      }
    }
  } else if constexpr (TC) {
    // =========================================================== tensor-core warps
    // Warps 0..3 of the group move the weight scales of every unit from shared to tensor memory,
    // warps 4..7 read the accumulators; all eight turn the routed activations into digit rows.
    const int tw = warp - (kSC + 2), tt = threadIdx.x - (kSC + 2) * 32, et = tt - 128;
    const int sub = warp & 3;                                   // the tensor-memory subpartition this warp can reach
    const uint32_t lane_base = (uint32_t)(sub * 32) << 16;
    const int row = sub * 32 + lane;                            // accumulator row of this thread
    long long base = 0, qseq = 0, dseq = 0;                     // ring index of the layer's first tile; units, tile segments so far
    // weight scales of `n_units` units whose first ring slots are first_tile, first_tile + 2, ...
    auto scales_loop = [&](int first_tile, int n_units) {
      for (int i = 0; i < n_units; ++i) {
        const long long t = base + first_tile + 2 * i;
        const int slot = (int)(t % kSStages), sfs = (int)(qseq % kTcSfSlots);
        bool ok = lane != 0 || tc_wait_issued(t, &sh);   // one lane polls the issue count
        ok = __all_sync(0xffffffffu, ok) && tc_wait(&sh.full[slot], (uint32_t)(t / kSStages) & 1u, &sh);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        // lane = row % 32, column = row / 32, four scale bytes (one 64-column MMA step) per column
        const unsigned char* sc = slots + (size_t)slot * kSSlot + kTcCodeBytes;
        const uint4 r0 = *reinterpret_cast<const uint4*>(sc + lane * 16);
        const uint4 r1 = *reinterpret_cast<const uint4*>(sc + (lane + 32) * 16);
        const uint4 r2 = *reinterpret_cast<const uint4*>(sc + (lane + 64) * 16);
        const uint4 r3 = *reinterpret_cast<const uint4*>(sc + (lane + 96) * 16);
        ok = tc_wait(&sh.sf_empty[sfs], (uint32_t)((qseq / kTcSfSlots) & 1) ^ 1u, &sh);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t w[16] = {r0.x, r1.x, r2.x, r3.x, r0.y, r1.y, r2.y, r3.y, r0.z, r1.z, r2.z, r3.z, r0.w, r1.w, r2.w, r3.w};
        tc_st16(tmem + lane_base + kTcColSfa + sfs * 16, w);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.sf_full[sfs]);
        ++qseq;
      }
    };
    // sum of the four digit columns starting at `column` of the next tile segment's accumulator
    // (after a failed wait the four warps still walk the same barriers: nobody is left behind at one)
    auto read_segment = [&](int column) -> float {
      const int dbuf = (int)(dseq & 1);
      bool ok = tc_wait(&sh.d_full[dbuf], (uint32_t)((dseq >> 1) & 1), &sh);
      ok = __all_sync(0xffffffffu, ok);
      float sum = 0.f;
      if (ok) {
        tc_fence_after();
        float v[4];
        tc_ld4(tmem + lane_base + kTcColD + dbuf * 32 + column, v);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.d_empty[dbuf]);
        sum = (v[0] + v[1]) + (v[2] + v[3]);
      }
      ++dseq;
      return sum;
    };

    // the split of this block's tile segments is the same in every layer: work it out once (64-bit
    // divisions), not in the hand-over at the end of every segment
    if (tt < 2) {
      const int chunks = tt == 0 ? S::GU_CHUNKS : S::DN_CHUNKS;
      const long long total = (long long)a.top_k * (tt == 0 ? S::GU_TILES : S::DN_TILES) * chunks;
      int u = tt == 0 ? plan.qu0 : plan.du0;
      const int end = u + (tt == 0 ? plan.n_qu : plan.n_du);
      for (int seg = 0; seg < 8 && u < end; ++seg) {
        const int tg = u / chunks;
        int index;
        sh.seg_parts[tt][seg] = (uint8_t)tc_split((long long)tg * chunks, (long long)tg * chunks + chunks - 1, total, gridDim.x, blockIdx.x, &index);
        sh.seg_index[tt][seg] = (uint8_t)index;
        u = min(end, (tg + 1) * chunks);
      }
    }
    tc_group_sync();
    auto split_of = [&](int kind, int seg, int tg, int chunks, long long total, int* index) -> int {
      if (seg < 8) {
        *index = sh.seg_index[kind][seg];
        return sh.seg_parts[kind][seg];
      }
      return tc_split((long long)tg * chunks, (long long)tg * chunks + chunks - 1, total, gridDim.x, blockIdx.x, index);
    };

    for (int layer = 0; layer < a.n_layers; ++layer, base += plan.per_layer) {
      unsigned* sync = a.sync + (size_t)layer * kSyncWordsPerLayer;
      unsigned* tile_count = a.tilesync + (size_t)layer * kTileCountersPerLayer;
      const int par = layer & 1;
      const unsigned epoch1 = sh.epoch1;
      const int xpar = (int)(((epoch1 - 1u) * (unsigned)a.n_layers + (unsigned)layer) & 1u);
      const bool tracer = (et == 0);
      // ------------------------------------------------ routed gate/up
      if (tw < 4) {
        scales_loop(plan.s_qg, plan.n_qu);
        if (tt == 0) INK_TRACE(layer, kTrScalesGuEnd);
      } else {
        // SwiGLU where the tile is complete in this block; otherwise the part goes to global memory
        // and the block that stores the last part of the tile finishes it
        const long long total = (long long)a.top_k * S::GU_TILES * S::GU_CHUNKS;
        int u = plan.qu0;
        const int end = plan.qu0 + plan.n_qu;
        for (int seg = 0; u < end; ++seg) {
          const int tg = u / S::GU_CHUNKS;
          float sum = read_segment(0);
          int index;
          const int parts = split_of(0, seg, tg, S::GU_CHUNKS, total, &index);
          // A split tile is finished by the block that holds its first units: that block reaches the tile
          // last (end of its range), the others first (start of theirs), so their parts are long there.
          bool finish = true;
          if (parts > 1) {
            float* part = a.gu_part + (size_t)tg * S::GU_CHUNKS * kTcRows;
            if (index > 0) {
              part[(size_t)index * kTcRows + row] = sum;
              __threadfence();   // every writer pushes its own store out before the count moves
              epilogue_sync();
              if (et == 0) red_release_add(tile_count + tg, 1u);
              finish = false;
            } else {
              if (et == 0) wait_global(tile_count + tg, epoch1 * (unsigned)(parts - 1), &sh);
              epilogue_sync();
              __threadfence();
              for (int p = 1; p < parts; ++p) sum += __ldcg(part + (size_t)p * kTcRows + row);   // fixed order
            }
          }
          if (finish) {
            const int choice = tg / S::GU_TILES, tile = tg % S::GU_TILES;
            const RouteEntry r = sh.routes[par].route[choice];
            const float mine = sum * (r.gu_scale2 * sh.x_inverse);
            const float up = __shfl_xor_sync(0xffffffffu, mine, 1);   // even rows are gate, odd rows up
            uint32_t bits = 0;
            if ((lane & 1) == 0) {
              bits = r.gu_codes ? f32_to_bf16_bits(silu_mul(mine, up)) : 0u;
              a.activated[((size_t)par * a.top_k + choice) * F + tile * (kTcRows / 2) + (row >> 1)] = (uint16_t)bits;
            }
            // largest magnitude of the route's activations, for the normaliser of their digit rows
            bits &= 0x7fffu;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
            if (lane == 0) atomicMax(a.act_amax + par * kSMaxTopK + choice, bits);
            __threadfence();
            epilogue_sync();
            if (et == 0) red_release_add(sync + kRtGuDone, 1u);   // every writer fenced its own stores above
          }
          u = min(end, (tg + 1) * S::GU_CHUNKS);
        }
      }
      if (tracer) INK_TRACE(layer, kTrRtGuDone);
      // ------------------------------------------------ routed activations -> digit rows (all eight warps)
      if (lane == 0) {
        wait_global(sync + kRtGuDone, epoch1 * (unsigned)(a.top_k * S::GU_TILES), &sh);
        wait_routing(layer, &sh);
        const long long t0 = clock64();
        while (sh.sg_done <= layer && !sh.failed)
          if (clock64() - t0 > sh.limit) sh.failed = 1;
        __threadfence_block();
      }
      __syncwarp();
      if (tracer) INK_TRACE(layer, kTrRtGuAll);
      {
        // groups of 8 consecutive activations, consecutive groups to consecutive threads; a rolled loop
        // with the next group's load in flight
        constexpr int kGroups = F / 8;   // per route
        const int total = a.top_k * kGroups;
        const bool live = !sh.failed;
        const uint4* src = reinterpret_cast<const uint4*>(a.activated + (size_t)par * a.top_k * F);
        uint4 ahead = (live && tt < total) ? __ldcg(src + tt) : make_uint4(0, 0, 0, 0);
#pragma unroll 1
        for (int g = tt; g < total; g += 256) {
          const uint4 raw = ahead;
          if (g + 256 < total) ahead = live ? __ldcg(src + g + 256) : make_uint4(0, 0, 0, 0);
          const int j = g / kGroups;
          float inverse;
          const float scale = 512.f * pow2_normaliser(__ldcg(a.act_amax + par * kSMaxTopK + j), &inverse);   // below 1024
          tc_stage8(raw, scale, s_adig, 32, 4 * j, (g % kGroups) * 8, &sh.sfba[0][0], 128);
        }
      }
      tc_proxy_fence();   // the digit rows are read by the tensor core
      tc_group_sync();
      if (tw < 4) tc_upload_scales(tmem, sub, &sh.sfba[0][0], 128, 4 * a.top_k, F / 64, lane);
      tc_group_sync();
      if (tt == 0) {
        __threadfence_block();
        sh.act_ready = layer + 1;
      }
      if (tracer) INK_TRACE(layer, kTrActStaged);
      // ------------------------------------------------ routed down
      if (tw < 4) {
        scales_loop(plan.s_qd, plan.n_du);
        if (tt == 0) INK_TRACE(layer, kTrScalesDownEnd);
      } else {
        const long long total = (long long)a.top_k * S::DN_TILES * S::DN_CHUNKS;
        int u = plan.du0;
        const int end = plan.du0 + plan.n_du;
        for (int seg = 0; u < end; ++seg) {
          const int tg = u / S::DN_CHUNKS;
          const int j = tg / S::DN_TILES, tile = tg % S::DN_TILES;
          const float sum = read_segment(4 * j);
          int index;
          split_of(1, seg, tg, S::DN_CHUNKS, total, &index);
          a.dn_part[((size_t)tg * S::DN_CHUNKS + index) * kTcRows + row] = sum;
          __threadfence();
          epilogue_sync();
          if (et == 0) {
            __threadfence();
            sh.finisher = atomicAdd(tile_count + kSMaxTopK * 32 + tile, 1u) + 1u == epoch1 * sh.dn_target[tile];
          }
          epilogue_sync();
          if (sh.finisher) {   // every part of the row tile is in: sum and deliver it
            __threadfence();
            finish_row_tile<D, F>(a, &sh, layer, par, xpar, tile, et, 128);
          }
          u = min(end, (tg + 1) * S::DN_CHUNKS);
        }
      }
      if (tracer) INK_TRACE(layer, kTrRtDownDone);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tc && warp == kSC + 1) tc_dealloc(tmem, 512);
  if (threadIdx.x == 0 && sh.failed && a.status) atomicOr(a.status, kFlagWaitTimedOut);
  // Every block read the epoch before it could pass any counter, and block 0 gets here only after
  // the last counter of the launch, so this store cannot be seen by a block of the same launch.
  if (threadIdx.x == 0 && blockIdx.x == 0) *a.epoch = sh.epoch1;
}

// ------------------------------------------------------------------- host side
template <int D, int F, bool TC>
static int launch_stack(const StackArgs& a, cudaStream_t stream) {
  using S = StackShape<D, F>;
  constexpr int threads = TC ? kSThreadsTc : kSThreads;
  // The shared-memory opt-in, the cooperative-launch check and the SM count belong to a device, not to
  // the process: one record per device ordinal (a process may drive several GPUs).
  constexpr int kMaxDevices = 64;
  static int sms_of[kMaxDevices] = {};   // 0 = this device is not configured yet
  int device = 0;
  cudaGetDevice(&device);
  INK_REQUIRE(device >= 0 && device < kMaxDevices, kLaunchFailed, "moe_stack: device ordinal %d", device);
  if (sms_of[device] == 0) {
    cudaError_t e = cudaFuncSetAttribute(moe_stack_kernel<D, F, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "moe_stack: %d bytes of shared memory refused: %s", S::SMEM,
                cudaGetErrorString(e));
    cudaFuncSetAttribute(moe_stack_kernel<D, F, TC>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         (int)cudaSharedmemCarveoutMaxShared);
    int coop = 0, per_sm = 0, count = 0;
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
    INK_REQUIRE(coop, kLaunchFailed, "moe_stack: the device cannot launch cooperative kernels");
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_stack_kernel<D, F, TC>, threads, S::SMEM);
    INK_REQUIRE(e == cudaSuccess && per_sm >= 1 && count >= 1, kLaunchFailed, "moe_stack: the kernel does not fit on an SM");
    sms_of[device] = count;
  }
  const int sms = sms_of[device];
  const int groups = D / S::RT;
  const int rows_per_block = ((groups + sms - 1) / sms) * S::RT;
  INK_REQUIRE(rows_per_block <= kSMaxRows, kUnsupportedShape, "moe_stack: %d output rows per block", rows_per_block);
  StackArgs args = a;
  void* params[] = {&args};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)moe_stack_kernel<D, F, TC>, dim3(sms), dim3(threads), params,
                                              (size_t)S::SMEM, stream);
  INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "moe_stack: launch failed: %s", cudaGetErrorString(e));
  return kOk;
}

}  // namespace ink

using namespace ink;

extern "C" size_t ink_moe_stack_layer_bytes(void) { return sizeof(StackLayer); }

// ---- TMA descriptors of a layer's banks (driver entry point resolved at first use; no link to libcuda)
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (TensorMapEncodeFn)p;
  }
  return fn;
}
// bytes [row_bytes] x rows x experts, box of `box_bytes` x 128 rows x 1 expert
static int encode_bank(CUtensorMap* out, const void* base, uint64_t expert_stride, int experts, int rows, int row_bytes,
                       int box_bytes, bool swizzle) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  INK_REQUIRE(enc != nullptr, kLaunchFailed, "encode_banks: the driver has no cuTensorMapEncodeTiled");
  INK_REQUIRE(base != nullptr && aligned16(base) && expert_stride % 16 == 0 && expert_stride >= (uint64_t)rows * row_bytes,
              kBadArgument, "encode_banks: bank at %p with expert stride %llu", base, (unsigned long long)expert_stride);
  cuuint64_t dims[3] = {(cuuint64_t)row_bytes, (cuuint64_t)rows, (cuuint64_t)experts};
  cuuint64_t strides[2] = {(cuuint64_t)row_bytes, (cuuint64_t)expert_stride};
  cuuint32_t box[3] = {(cuuint32_t)box_bytes, (cuuint32_t)kTcRows, 1}, elem[3] = {1, 1, 1};
  const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  INK_REQUIRE(r == CUDA_SUCCESS, kBadArgument, "encode_banks: cuTensorMapEncodeTiled returned %d", (int)r);
  return kOk;
}

extern "C" int ink_moe_stack_encode_banks(void* out_host_512, const void* gate_up_codes, uint64_t gate_up_codes_stride,
                                          const void* gate_up_scales, uint64_t gate_up_scales_stride, const void* down_codes,
                                          uint64_t down_codes_stride, const void* down_scales, uint64_t down_scales_stride,
                                          int experts, int hidden, int intermediate) {
  INK_REQUIRE(out_host_512 != nullptr && experts >= 1, kBadArgument, "encode_banks: null output or no experts");
  INK_REQUIRE(hidden % kTcChunkK == 0 && intermediate % kTcChunkK == 0 && (2 * intermediate) % kTcRows == 0 &&
                  hidden % kTcRows == 0,
              kUnsupportedShape, "encode_banks: hidden=%d intermediate=%d do not tile by 128 rows x 256 columns", hidden,
              intermediate);
  CUtensorMap maps[4];
  int rc = encode_bank(&maps[0], gate_up_codes, gate_up_codes_stride, experts, 2 * intermediate, hidden / 2, 128, true);
  if (rc == kOk) rc = encode_bank(&maps[1], gate_up_scales, gate_up_scales_stride, experts, 2 * intermediate, hidden / 16, 16, false);
  if (rc == kOk) rc = encode_bank(&maps[2], down_codes, down_codes_stride, experts, hidden, intermediate / 2, 128, true);
  if (rc == kOk) rc = encode_bank(&maps[3], down_scales, down_scales_stride, experts, hidden, intermediate / 16, 16, false);
  if (rc != kOk) return rc;
  static_assert(sizeof(CUtensorMap) == 128, "a TMA descriptor is 128 bytes");
  memcpy(out_host_512, maps, sizeof(maps));
  return kOk;
}

static size_t pad256(size_t n) { return (n + 255) / 256 * 256; }
constexpr int kTileCounters = kTileCountersPerLayer;
static size_t dn_part_bytes(int hidden, int intermediate, int top_k) {
  return sizeof(float) * kTcRows * (size_t)top_k * (size_t)((hidden + kTcRows - 1) / kTcRows) *
         (size_t)((intermediate + kTcChunkK - 1) / kTcChunkK);
}
static size_t gu_part_bytes(int hidden, int intermediate, int top_k) {
  return sizeof(float) * kTcRows * (size_t)top_k * (size_t)((2 * intermediate + kTcRows - 1) / kTcRows) *
         (size_t)((hidden + kTcChunkK - 1) / kTcChunkK);
}

// The region other ranks write into: two sets (alternating from layer to layer) of one slot of
// `hidden` tagged 8-byte words per rank.
extern "C" size_t ink_moe_stack_symmetric_bytes(int n_layers, int hidden, int world) {
  (void)n_layers;
  return pad256(sizeof(unsigned long long) * 2 * (size_t)world * hidden);
}

// SM clocks a wait inside the one-launch kernel may take before the launch gives up (default: about a
// tenth of a second). A diagnostic knob: tests shorten it to see the give-up path without waiting.
static long long g_stack_wait_limit = kWaitLimitCycles;
extern "C" int ink_moe_stack_set_wait_limit(long long cycles) {
  INK_REQUIRE(cycles >= 1000, kBadArgument, "moe_stack: a wait limit of %lld clocks is too short", cycles);
  g_stack_wait_limit = cycles;
  return kOk;
}

extern "C" size_t ink_moe_stack_scratch_bytes(int n_layers, int hidden, int intermediate, int experts, int n_shared,
                                              int top_k) {
  size_t bytes = 0;
  bytes += pad256(sizeof(unsigned) * kSyncWordsPerLayer * (size_t)n_layers);   // sync
  bytes += pad256(sizeof(unsigned));                                            // epoch
  bytes += pad256(sizeof(RouteTable) * (size_t)n_layers);                       // routes
  bytes += pad256(gu_part_bytes(hidden, intermediate, top_k));                  // parts of split gate/up tiles
  bytes += pad256(dn_part_bytes(hidden, intermediate, top_k));                  // parts of split down tiles
  bytes += pad256(sizeof(float) * 2 * (size_t)n_shared * hidden);               // shared experts' down rows
  bytes += pad256(sizeof(unsigned) * 2 * kSMaxTopK);                            // activation maxima
  bytes += pad256(sizeof(unsigned) * kTileCounters * (size_t)n_layers);         // tile counters
  bytes += pad256(sizeof(unsigned long long) * 2 * (size_t)(experts + n_shared));   // router words
  bytes += pad256(2 * 2 * (size_t)top_k * intermediate);                        // activated
  bytes += pad256(2 * 2 * (size_t)n_shared * intermediate);                     // shared activated
  bytes += pad256(2 * 2 * (size_t)hidden);                                      // residual double buffer
  bytes += pad256(sizeof(unsigned long long) * 2 * (size_t)hidden);             // rows summed over the ranks (tagged)
  bytes += pad256(sizeof(unsigned long long) * (size_t)n_layers * kTraceBlocks * kTraceSlots);   // phase stamps (tracing)
  return bytes;
}

extern "C" size_t ink_moe_stack_trace_offset(int n_layers, int hidden, int intermediate, int experts,
                                             int n_shared, int top_k) {
  return ink_moe_stack_scratch_bytes(n_layers, hidden, intermediate, experts, n_shared, top_k) -
         pad256(sizeof(unsigned long long) * (size_t)n_layers * kTraceBlocks * kTraceSlots);
}

static int stack_decode(const void* layers, int n_layers, const void* x, void* residual_io, void* normed_out,
                        float* partial_out, int flags, float eps, int hidden, int intermediate, int experts,
                        int n_shared, int top_k, void* scratch, size_t scratch_bytes, int rank, int world,
                        const uint64_t* peer_regions, int32_t* status, ink_stream_t stream) {
  INK_REQUIRE(layers && x && partial_out && scratch, kBadArgument, "moe_stack: null pointer argument");
  INK_REQUIRE(flags >= 0 && flags <= 3, kBadArgument, "moe_stack: flags=%d", flags);
  const int glue = flags & 1;
  const bool banks_mapped = (flags & 2) != 0;   // every layer carries the TMA descriptors of its banks
  INK_REQUIRE(n_layers >= 1, kBadArgument, "moe_stack: n_layers=%d", n_layers);
  INK_REQUIRE(glue || n_layers == 1, kBadArgument, "moe_stack: without the glue only one block can run");
  INK_REQUIRE(!glue || (residual_io && normed_out), kBadArgument, "moe_stack: glue mode needs residual and normed buffers");
  INK_REQUIRE(top_k >= 1 && top_k <= kSMaxTopK && n_shared >= 0 && n_shared <= kSMaxShared && experts >= top_k &&
                  experts <= kSMaxExperts && top_k + n_shared <= 32,
              kUnsupportedShape, "moe_stack: experts=%d top_k=%d n_shared=%d unsupported", experts, top_k, n_shared);
  INK_REQUIRE(world >= 1 && world <= kSMaxWorld && rank >= 0 && rank < world && (world == 1 || peer_regions), kBadArgument,
              "moe_stack: rank=%d world=%d", rank, world);
  INK_REQUIRE(scratch_bytes >= ink_moe_stack_scratch_bytes(n_layers, hidden, intermediate, experts, n_shared, top_k),
              kBadArgument, "moe_stack: scratch of %zu bytes is too small", scratch_bytes);
  INK_REQUIRE(aligned16(x) && aligned16(scratch) && aligned16(partial_out) && aligned16(residual_io) && aligned16(normed_out),
              kMisaligned, "moe_stack: misaligned buffer (x, scratch, partial, residual and normed need 16-byte alignment)");
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
  a.gu_part = (float*)take(gu_part_bytes(hidden, intermediate, top_k));
  a.dn_part = (float*)take(dn_part_bytes(hidden, intermediate, top_k));
  a.sd_out = (float*)take(sizeof(float) * 2 * (size_t)n_shared * hidden);
  a.act_amax = (unsigned*)take(sizeof(unsigned) * 2 * kSMaxTopK);
  a.tilesync = (unsigned*)take(sizeof(unsigned) * kTileCounters * (size_t)n_layers);
  a.scores = (unsigned long long*)take(sizeof(unsigned long long) * 2 * (size_t)(experts + n_shared));
  a.activated = (uint16_t*)take(2 * 2 * (size_t)top_k * intermediate);
  a.shared_activated = (uint16_t*)take(2 * 2 * (size_t)n_shared * intermediate);
  a.residual = (uint16_t*)take(2 * 2 * (size_t)hidden);
  a.summed = (unsigned long long*)take(sizeof(unsigned long long) * 2 * (size_t)hidden);
  a.wait_limit = g_stack_wait_limit;
  {
    const char* pause = getenv("INKLING_STACK_POLL_PAUSE_NS");
    a.poll_pause_ns = pause ? (unsigned)atoi(pause) : 500u;   // measured on B200: 250..2000 ns are equally good, 64 ns costs 4 us per block
    if (a.poll_pause_ns > 100000u) a.poll_pause_ns = 500u;
  }
  for (int r = 0; r < kSMaxWorld; ++r) a.peer_inbox[r] = nullptr;
  for (int r = 0; r < world && world > 1; ++r) {
    char* region = (char*)(uintptr_t)peer_regions[r];
    INK_REQUIRE(region != nullptr && aligned16(region), kBadArgument, "moe_stack: bad region for rank %d", r);
    a.peer_inbox[r] = (unsigned long long*)region;
  }
  a.inbox = world > 1 ? a.peer_inbox[rank] : nullptr;
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
    rc = banks_mapped ? launch_stack<DD, FF, true>(a, s) : launch_stack<DD, FF, false>(a, s); \
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
                                    void* normed_out, float* partial_out, int flags, float eps, int hidden,
                                    int intermediate, int experts, int n_shared, int top_k, void* scratch,
                                    size_t scratch_bytes, int32_t* status, ink_stream_t stream) {
  return stack_decode(layers, n_layers, x, residual_io, normed_out, partial_out, flags, eps, hidden, intermediate,
                      experts, n_shared, top_k, scratch, scratch_bytes, 0, 1, nullptr, status, stream);
}

extern "C" int ink_moe_stack_decode_tp(const void* layers, int n_layers, const void* x, void* residual_io,
                                       void* normed_out, float* partial_out, int flags, float eps, int hidden,
                                       int intermediate, int experts, int n_shared, int top_k, void* scratch,
                                       size_t scratch_bytes, int rank, int world, const uint64_t* peer_regions,
                                       int32_t* status, ink_stream_t stream) {
  return stack_decode(layers, n_layers, x, residual_io, normed_out, partial_out, flags, eps, hidden, intermediate,
                      experts, n_shared, top_k, scratch, scratch_bytes, rank, world, peer_regions, status, stream);
}

// Streaming form of the decode-time expert projections for the production widths
// (hidden 1024..4096, intermediate 256..4096): persistent blocks, one per SM, each with
// a producer warp that streams its share of the weight bytes through a shared-memory
// ring with bulk asynchronous copies and eleven consumer warps that take ring slots in
// order, dequantise in registers and reduce with shuffles. No weight byte is read twice
// and the copies in flight do not depend on how fast any one warp computes. In the down
// kernel lane s of the producer warp owns ring slot s: one thread issues only about two
// tiles per microsecond (a barrier wait, the transaction count and two bulk copies, each a
// long-latency instruction), a third of what a block's share of the HBM bandwidth needs at
// its 4.6 KB tiles; the gate/up kernel's 18 KB tiles are fed by one lane.
#include "../../include/inkling_b200.h"
#include "common.cuh"
#include "decode_args.cuh"
#include "pipe.cuh"
#include "stream_math.cuh"

namespace ink {

// Consumer c takes tiles c, c + kConsumers, ... of its block and the ring depth is a
// multiple of kConsumers, so the tile that last used a slot was always finished by the
// very warp that now waits on it: a parity wait can then never be a whole phase behind.
constexpr int kConsumers = 11;
constexpr int kStreamThreads = (kConsumers + 1) * 32;  // warp 0 produces
constexpr int kMaxJobs = 16;                           // top_k + n_shared handled by the streaming kernels

__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");
}

struct Ring {
  static constexpr int kMaxStages = 2 * kConsumers;
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  int failed;     // a bounded wait gave up
};

__device__ __forceinline__ void ring_init(Ring* ring, int stages) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&ring->full[s], 1);
      mbar_init(&ring->empty[s], 1);
    }
    ring->failed = 0;
    mbar_init_fence();
  }
}

// ====================================================================== gate / up
template <int K>
struct GateUpStream {
  static constexpr int CPL = K / 1024;                // 16-byte chunks per lane per NVFP4 row
  static constexpr int Q_ROWS = 16384 / (K / 2);      // NVFP4 rows per tile: 8 / 16 / 32
  static constexpr int Q_PAIRS = Q_ROWS / 2;
  static constexpr int Q_CODES = 16384;
  static constexpr int Q_SCALES = Q_ROWS * (K / 16);  // 2048
  static constexpr int S_PAIRS = 16384 / (4 * K);     // BF16 (gate, up) pairs per tile: 1 / 2 / 4
  static constexpr int S_HALF = S_PAIRS * K * 2;      // bytes of the gate rows (= of the up rows)
  static constexpr int SLOT = Q_CODES + Q_SCALES;     // 18432 >= 2 * S_HALF
  static constexpr int B_CPL = K / 256;               // 16-byte chunks per lane per BF16 row
};

struct GateUpJob {   // routed job as the producer and the consumers see it
  const uint8_t* codes;
  const uint8_t* scales;
  float scale2;
};

template <int K>
__global__ void __launch_bounds__(kStreamThreads, 1) gate_up_stream_kernel(DecodeArgs a, int stages) {
  using G = GateUpStream<K>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ Ring ring;
  __shared__ GateUpJob s_job[kMaxJobs];
  __shared__ float s_inverse;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.y;
  const int f = a.intermediate;
  unsigned char* slots = smem;
  uint16_t* s_x16 = reinterpret_cast<uint16_t*>(smem + (size_t)stages * G::SLOT);  // FP16, normalised
  uint16_t* s_xbf = s_x16 + K;                                                        // BF16, as given

  // tiles of this token: shared experts first (they do not depend on the routing), then routes
  const int s_tiles_per_job = f / G::S_PAIRS, q_tiles_per_job = 2 * f / G::Q_ROWS;
  const int n_s = a.n_shared * s_tiles_per_job, total = n_s + a.top_k * q_tiles_per_job;
  const int first = (int)((long long)blockIdx.x * total / gridDim.x);
  const int last = (int)((long long)(blockIdx.x + 1) * total / gridDim.x);
  const int n_tiles = last - first;
  if (n_tiles <= 0) return;

  ring_init(&ring, stages);
  if (threadIdx.x < a.top_k) {
    const int64_t expert = a.indices[token * a.top_k + threadIdx.x];
    GateUpJob job{nullptr, nullptr, 0.f};
    if (expert < 0 || expert > a.max_expert) {
      if (a.status && blockIdx.x == 0) atomicOr(a.status, kFlagExpertOutOfRange);
    } else {
      const int64_t* entry = a.pointers + expert * kBank;
      job.codes = reinterpret_cast<const uint8_t*>(entry[0]);
      if (job.codes) {
        job.scales = reinterpret_cast<const uint8_t*>(entry[1]);
        job.scale2 = *reinterpret_cast<const float*>(entry[2]);
      }
    }
    s_job[threadIdx.x] = job;
  }
  __syncthreads();

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {   // (18 KB tiles: one lane keeps up, and measured slightly faster than a lane per slot)
      for (int i = 0; i < n_tiles; ++i) {
        const int slot = i % stages;
        if (i >= stages && !mbar_wait(&ring.empty[slot], ((i / stages) - 1) & 1)) {
          atomicExch(&ring.failed, 1);
          break;
        }
        unsigned char* dst = slots + (size_t)slot * G::SLOT;
        const int t = first + i;
        if (t < n_s) {
          const int e = t / s_tiles_per_job, pair0 = (t % s_tiles_per_job) * G::S_PAIRS;
          const size_t row = ((size_t)e * f + pair0) * K;
          mbar_expect_tx(&ring.full[slot], 2 * G::S_HALF);
          bulk_g2s(dst, a.shared_gate + row, G::S_HALF, &ring.full[slot]);
          bulk_g2s(dst + G::S_HALF, a.shared_up + row, G::S_HALF, &ring.full[slot]);
        } else {
          const int q = t - n_s, choice = q / q_tiles_per_job, row0 = (q % q_tiles_per_job) * G::Q_ROWS;
          const GateUpJob job = s_job[choice];
          if (job.codes) {
            mbar_expect_tx(&ring.full[slot], G::Q_CODES + G::Q_SCALES);
            bulk_g2s(dst, job.codes + (size_t)row0 * (K / 2), G::Q_CODES, &ring.full[slot]);
            bulk_g2s(dst + G::Q_CODES, job.scales + (size_t)row0 * (K / 16), G::Q_SCALES, &ring.full[slot]);
          } else {
            mbar_expect_tx(&ring.full[slot], 0);  // inactive expert: an empty slot keeps the order
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    const int cw = warp - 1;
    const uint16_t* x = a.x + (size_t)token * K;
    if (cw == 0) {
      const float inverse = warp_stage_f16<K>(x, s_x16, lane);
      if (lane == 0) s_inverse = inverse;
    }
    for (int i = threadIdx.x - 32; i < K / 8; i += kConsumers * 32)
      reinterpret_cast<uint4*>(s_xbf)[i] = reinterpret_cast<const uint4*>(x)[i];
    consumer_barrier();
    uint32_t xr[G::CPL][16];
#pragma unroll
    for (int j = 0; j < G::CPL; ++j) {
      const uint4* p = reinterpret_cast<const uint4*>(s_x16 + (j * 32 + lane) * 32);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const uint4 t4 = p[v];
        xr[j][4 * v + 0] = t4.x; xr[j][4 * v + 1] = t4.y; xr[j][4 * v + 2] = t4.z; xr[j][4 * v + 3] = t4.w;
      }
    }
    const float inverse = s_inverse;
    for (int i = cw; i < n_tiles; i += kConsumers) {
      const int slot = i % stages;
      if (!mbar_wait(&ring.full[slot], (i / stages) & 1)) {
        atomicExch(&ring.failed, 1);
        break;
      }
      const unsigned char* src = slots + (size_t)slot * G::SLOT;
      const int t = first + i;
      if (t < n_s) {
        // BF16 (gate, up) pairs of a shared expert
        const int e = t / s_tiles_per_job, pair0 = (t % s_tiles_per_job) * G::S_PAIRS;
        float g[G::S_PAIRS], u[G::S_PAIRS];
#pragma unroll
        for (int p = 0; p < G::S_PAIRS; ++p) {
          g[p] = 0.f;
          u[p] = 0.f;
#pragma unroll
          for (int c = 0; c < G::B_CPL; ++c) {
            const int chunk = c * 32 + lane;
            const uint4 xv = reinterpret_cast<const uint4*>(s_xbf)[chunk];
            g[p] = dot8(*reinterpret_cast<const uint4*>(src + (size_t)p * K * 2 + chunk * 16), xv, g[p]);
            u[p] = dot8(*reinterpret_cast<const uint4*>(src + G::S_HALF + (size_t)p * K * 2 + chunk * 16), xv, u[p]);
          }
        }
        float gate = multi_reduce<G::S_PAIRS>(g, lane);
        float up = multi_reduce<G::S_PAIRS>(u, lane);
        if (reduced_owner<G::S_PAIRS>(lane)) {
          // the reference's BF16 tensor ops: both bmm outputs, silu and the product round to BF16
          gate = round_bf16(gate);
          up = round_bf16(up);
          const float act = round_bf16(gate / (1.f + expf(-gate)));
          a.shared_activated[(size_t)(token * a.n_shared + e) * f + pair0 + reduced_row<G::S_PAIRS>(lane)] =
              (uint16_t)f32_to_bf16_bits(act * up);
        }
      } else {
        const int q = t - n_s, choice = q / q_tiles_per_job, row0 = (q % q_tiles_per_job) * G::Q_ROWS;
        const GateUpJob job = s_job[choice];
        if (job.codes) {
          float g[G::Q_PAIRS], u[G::Q_PAIRS];
#pragma unroll
          for (int p = 0; p < G::Q_PAIRS; ++p) {
            float acc_g = 0.f, acc_u = 0.f;
#pragma unroll
            for (int j = 0; j < G::CPL; ++j) {
              const int chunk = j * 32 + lane;
              const unsigned char* rg = src + (size_t)(2 * p) * (K / 2) + chunk * 16;
              const unsigned char* sg = src + G::Q_CODES + (size_t)(2 * p) * (K / 16) + chunk * 2;
              acc_g += dot32(*reinterpret_cast<const uint4*>(rg), *reinterpret_cast<const uint16_t*>(sg), xr[j]);
              acc_u += dot32(*reinterpret_cast<const uint4*>(rg + K / 2),
                             *reinterpret_cast<const uint16_t*>(sg + K / 16), xr[j]);
            }
            g[p] = acc_g;
            u[p] = acc_u;
          }
          const float gate = multi_reduce<G::Q_PAIRS>(g, lane) * (job.scale2 * inverse);
          const float up = multi_reduce<G::Q_PAIRS>(u, lane) * (job.scale2 * inverse);
          if (reduced_owner<G::Q_PAIRS>(lane))
            a.activated[(size_t)(token * a.top_k + choice) * f + row0 / 2 + reduced_row<G::Q_PAIRS>(lane)] =
                (uint16_t)f32_to_bf16_bits(silu_mul(gate, up));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ring.empty[slot]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && ring.failed && a.status) atomicOr(a.status, kFlagWaitTimedOut);
}

// =========================================================================== down
template <int K>
struct DownStream {
  static constexpr int CH = K / 32;
  static constexpr int LPR = CH < 32 ? CH : 32;
  static constexpr int CPL = CH / LPR;
  static constexpr int RPP = 32 / LPR;
  static constexpr int RT = K >= 2048 ? 4 : 8192 / K;      // output rows per row group
  static constexpr int PASSES = RT / RPP;
  static constexpr int Q_CODES = RT * (K / 2);
  static constexpr int Q_SCALES = RT * (K / 16);
  static constexpr int S_ROWS = RT / 2;                    // BF16 rows per tile (two tiles per group)
  static constexpr int S_BYTES = S_ROWS * K * 2;
  static constexpr int SLOT = (Q_CODES + Q_SCALES) > S_BYTES ? (Q_CODES + Q_SCALES) : S_BYTES;
  static constexpr int B_CPL = K / 256;                    // 16-byte chunks per lane per BF16 row
  static constexpr int MAX_ROWS = 64;                      // output rows one block may own
};

struct DownJob {
  const uint8_t* codes;
  const uint8_t* scales;
  float scale;      // scale2 * inverse of the activation normaliser
  float weight;     // router weight of the route
};

template <int K>
__global__ void __launch_bounds__(kStreamThreads, 1) down_stream_kernel(DecodeArgs a, int stages) {
  using D = DownStream<K>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ Ring ring;
  __shared__ DownJob s_job[kMaxJobs];
  __shared__ float s_contrib[kMaxJobs][D::MAX_ROWS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.y;
  const int d = a.hidden;
  const int jobs = a.top_k + a.n_shared;
  unsigned char* slots = smem;
  uint16_t* s_act = reinterpret_cast<uint16_t*>(smem + (size_t)stages * D::SLOT);  // [top_k][K] FP16 normalised
  uint16_t* s_shared = s_act + (size_t)a.top_k * K;                                  // [n_shared][K] BF16 (act*gamma)

  const int n_groups = d / D::RT;
  const int g0 = (int)((long long)blockIdx.x * n_groups / gridDim.x);
  const int g1 = (int)((long long)(blockIdx.x + 1) * n_groups / gridDim.x);
  const int groups = g1 - g0;
  if (groups <= 0) return;
  const int n_q = a.top_k * groups, n_tiles = n_q + a.n_shared * 2 * groups;

  ring_init(&ring, stages);
  for (int i = threadIdx.x; i < kMaxJobs * D::MAX_ROWS; i += blockDim.x) (&s_contrib[0][0])[i] = 0.f;
  if (threadIdx.x < a.top_k) {
    const int route = token * a.top_k + threadIdx.x;
    const int64_t expert = a.indices[route];
    DownJob job{nullptr, nullptr, 0.f, 0.f};
    if (expert < 0 || expert > a.max_expert) {
      if (a.status && blockIdx.x == 0) atomicOr(a.status, kFlagExpertOutOfRange);
    } else {
      const int64_t* entry = a.pointers + expert * kBank + 3;
      job.codes = reinterpret_cast<const uint8_t*>(entry[0]);
      if (job.codes) {
        job.scales = reinterpret_cast<const uint8_t*>(entry[1]);
        job.scale = *reinterpret_cast<const float*>(entry[2]);
        job.weight = bf16_to_f32(a.weights[route]);
      }
    }
    s_job[threadIdx.x] = job;
  }
  __syncthreads();

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane < stages) {
      const int slot = lane;
      for (int i = lane; i < n_tiles; i += stages) {
        if (i >= stages && !mbar_wait(&ring.empty[slot], ((i / stages) - 1) & 1)) {
          atomicExch(&ring.failed, 1);
          break;
        }
        unsigned char* dst = slots + (size_t)slot * D::SLOT;
        if (i < n_q) {
          const int choice = i / groups, row0 = (g0 + i % groups) * D::RT;
          const DownJob job = s_job[choice];
          if (job.codes) {
            mbar_expect_tx(&ring.full[slot], D::Q_CODES + D::Q_SCALES);
            bulk_g2s(dst, job.codes + (size_t)row0 * (K / 2), D::Q_CODES, &ring.full[slot]);
            bulk_g2s(dst + D::Q_CODES, job.scales + (size_t)row0 * (K / 16), D::Q_SCALES, &ring.full[slot]);
          } else {
            mbar_expect_tx(&ring.full[slot], 0);
          }
        } else {
          const int s = i - n_q, e = s / (2 * groups), rem = s % (2 * groups);
          const int row0 = (g0 + rem / 2) * D::RT + (rem & 1) * D::S_ROWS;
          mbar_expect_tx(&ring.full[slot], D::S_BYTES);
          bulk_g2s(dst, a.shared_down + ((size_t)e * d + row0) * K, D::S_BYTES, &ring.full[slot]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    const int cw = warp - 1;
    for (int job = cw; job < jobs; job += kConsumers) {
      if (job < a.top_k) {
        const float inverse = warp_stage_f16<K>(a.activated + (size_t)(token * a.top_k + job) * K,
                                                s_act + (size_t)job * K, lane);
        if (lane == 0) s_job[job].scale *= inverse;
      } else {
        const int e = job - a.top_k;
        const uint16_t* src = a.shared_activated + (size_t)(token * a.n_shared + e) * K;
        const float gamma = bf16_to_f32(a.gammas[token * a.n_shared + e]);
        uint32_t* dst = reinterpret_cast<uint32_t*>(s_shared + (size_t)e * K);
        for (int i = lane; i < K / 2; i += 32) {
          const uint32_t v = reinterpret_cast<const uint32_t*>(src)[i];
          // gamma multiplies the activation before the down projection, rounded to BF16
          dst[i] = f32_to_bf16_bits(bf16lo(v) * gamma) | (f32_to_bf16_bits(bf16hi(v) * gamma) << 16);
        }
      }
    }
    consumer_barrier();
    const int sl = lane % D::LPR, rp = lane / D::LPR;
    uint32_t xr[D::CPL][16];
    int loaded = -1;
    for (int i = cw; i < n_tiles; i += kConsumers) {
      const int slot = i % stages;
      if (!mbar_wait(&ring.full[slot], (i / stages) & 1)) {
        atomicExch(&ring.failed, 1);
        break;
      }
      const unsigned char* src = slots + (size_t)slot * D::SLOT;
      if (i < n_q) {
        const int choice = i / groups, local0 = (i % groups) * D::RT;
        const DownJob job = s_job[choice];
        if (job.codes) {
          if (loaded != choice) {
            loaded = choice;
#pragma unroll
            for (int j = 0; j < D::CPL; ++j) {
              const uint4* p = reinterpret_cast<const uint4*>(s_act + (size_t)choice * K + (j * D::LPR + sl) * 32);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const uint4 t4 = p[v];
                xr[j][4 * v + 0] = t4.x; xr[j][4 * v + 1] = t4.y; xr[j][4 * v + 2] = t4.z; xr[j][4 * v + 3] = t4.w;
              }
            }
          }
          float r[D::PASSES];
#pragma unroll
          for (int p = 0; p < D::PASSES; ++p) {
            const int row = p * D::RPP + rp;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < D::CPL; ++j) {
              const int chunk = j * D::LPR + sl;
              acc += dot32(*reinterpret_cast<const uint4*>(src + (size_t)row * (K / 2) + chunk * 16),
                           *reinterpret_cast<const uint16_t*>(src + D::Q_CODES + (size_t)row * (K / 16) + chunk * 2),
                           xr[j]);
            }
            r[p] = acc;
          }
          if constexpr (D::LPR == 32) {
            const float total = multi_reduce<D::PASSES>(r, lane);
            if (reduced_owner<D::PASSES>(lane)) {
              const float down = round_bf16(total * job.scale);
              s_contrib[choice][local0 + reduced_row<D::PASSES>(lane)] = round_bf16(down * job.weight);
            }
          } else {
#pragma unroll
            for (int p = 0; p < D::PASSES; ++p) {
              float v = r[p];
#pragma unroll
              for (int o = D::LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
              if (sl == 0) {
                const float down = round_bf16(v * job.scale);
                s_contrib[choice][local0 + p * D::RPP + rp] = round_bf16(down * job.weight);
              }
            }
          }
        }
      } else {
        const int s = i - n_q, e = s / (2 * groups), rem = s % (2 * groups);
        const int local0 = (rem / 2) * D::RT + (rem & 1) * D::S_ROWS;
        const uint16_t* xs = s_shared + (size_t)e * K;
        float r[D::S_ROWS];
#pragma unroll
        for (int row = 0; row < D::S_ROWS; ++row) {
          float acc = 0.f;
#pragma unroll
          for (int c = 0; c < D::B_CPL; ++c) {
            const int chunk = c * 32 + lane;
            acc = dot8(*reinterpret_cast<const uint4*>(src + (size_t)row * K * 2 + chunk * 16),
                       reinterpret_cast<const uint4*>(xs)[chunk], acc);
          }
          r[row] = acc;
        }
        const float total = multi_reduce<D::S_ROWS>(r, lane);
        if (reduced_owner<D::S_ROWS>(lane))
          s_contrib[a.top_k + e][local0 + reduced_row<D::S_ROWS>(lane)] = round_bf16(total);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ring.empty[slot]);
    }
  }
  __syncthreads();
  // fixed summation order: routes in choice order, then the shared experts
  for (int r = threadIdx.x; r < groups * D::RT; r += blockDim.x) {
    float total = 0.f;
    for (int j = 0; j < jobs; ++j) total += s_contrib[j][r];
    a.output[(size_t)token * d + (size_t)g0 * D::RT + r] = total;
  }
  if (threadIdx.x == 0 && ring.failed && a.status) atomicOr(a.status, kFlagWaitTimedOut);
}

// ---------------------------------------------------------------------- launchers
static int sm_count() {
  static int cached = 0;
  if (cached == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) cached = 148;
  }
  return cached;
}

constexpr size_t kSmemBudget = 220 * 1024;

// largest multiple of kConsumers slots that fits (at most Ring::kMaxStages)
static int ring_depth(size_t bytes, size_t slot) {
  int stages = (int)(bytes / slot);
  if (stages > Ring::kMaxStages) stages = Ring::kMaxStages;
  return stages / kConsumers * kConsumers;
}

template <int K>
static int launch_gate_up_stream(const DecodeArgs& a, cudaStream_t stream) {
  using G = GateUpStream<K>;
  const size_t staging = (size_t)K * 4;
  const int stages = ring_depth(kSmemBudget - staging, G::SLOT);
  INK_REQUIRE(stages > 0, kUnsupportedShape, "gate_up: no room for the ring in shared memory");
  const size_t smem = (size_t)stages * G::SLOT + staging;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gate_up_stream_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBudget);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "gate_up: shared memory opt-in refused: %s", cudaGetErrorString(e));
    INK_PREFER_MAX_SMEM(gate_up_stream_kernel<K>);
    configured = true;
  }
  gate_up_stream_kernel<K><<<dim3(sm_count(), a.tokens), kStreamThreads, smem, stream>>>(a, stages);
  INK_CHECK_LAUNCH("gate_up (streaming)");
  return kOk;
}

template <int K>
static int launch_down_stream(const DecodeArgs& a, cudaStream_t stream) {
  using D = DownStream<K>;
  const size_t staging = (size_t)(a.top_k + a.n_shared) * K * 2;
  const int stages = ring_depth(kSmemBudget - staging, D::SLOT);
  INK_REQUIRE(stages > 0, kUnsupportedShape, "down: no room for the ring in shared memory");
  const size_t smem = (size_t)stages * D::SLOT + staging;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(down_stream_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBudget);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "down: shared memory opt-in refused: %s", cudaGetErrorString(e));
    INK_PREFER_MAX_SMEM(down_stream_kernel<K>);
    configured = true;
  }
  down_stream_kernel<K><<<dim3(sm_count(), a.tokens), kStreamThreads, smem, stream>>>(a, stages);
  INK_CHECK_LAUNCH("down (streaming)");
  return kOk;
}

// Shapes the streaming kernels take; everything else goes to the narrow-width kernels.
bool stream_gate_up_supported(const DecodeArgs& a) {
  const int k = a.hidden, f = a.intermediate;
  return (k == 1024 || k == 2048 || k == 4096) && f >= 256 && f % 64 == 0 && a.top_k + a.n_shared <= kMaxJobs &&
         a.tokens <= 65535;
}
bool stream_down_supported(const DecodeArgs& a) {
  const int k = a.intermediate, d = a.hidden;
  const bool width = k == 256 || k == 512 || k == 1024 || k == 2048 || k == 4096;
  if (!width) return false;
  const int rt = k >= 2048 ? 4 : 8192 / k;
  const int per_block = ((d / rt) + sm_count() - 1) / sm_count() * rt;
  return d % rt == 0 && per_block <= 64 && a.top_k + a.n_shared <= kMaxJobs && a.tokens <= 65535 &&
         (size_t)(a.top_k + a.n_shared) * k * 2 + (size_t)kConsumers * (k == 4096 ? 16384 : 8192) <= kSmemBudget;
}

int dispatch_gate_up_stream(const DecodeArgs& a, cudaStream_t stream) {
  switch (a.hidden) {
    case 1024: return launch_gate_up_stream<1024>(a, stream);
    case 2048: return launch_gate_up_stream<2048>(a, stream);
    case 4096: return launch_gate_up_stream<4096>(a, stream);
    default: break;
  }
  set_error("gate_up (streaming): hidden=%d unsupported", a.hidden);
  return kUnsupportedShape;
}

int dispatch_down_stream(const DecodeArgs& a, cudaStream_t stream) {
  switch (a.intermediate) {
    case 256: return launch_down_stream<256>(a, stream);
    case 512: return launch_down_stream<512>(a, stream);
    case 1024: return launch_down_stream<1024>(a, stream);
    case 2048: return launch_down_stream<2048>(a, stream);
    case 4096: return launch_down_stream<4096>(a, stream);
    default: break;
  }
  set_error("down (streaming): intermediate=%d unsupported", a.intermediate);
  return kUnsupportedShape;
}

}  // namespace ink

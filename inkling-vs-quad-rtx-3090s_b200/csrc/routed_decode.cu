// Decode-time expert projections: one matrix-vector product per route, NVFP4 weights
// streamed from HBM and dequantised in registers (cvt e2m1x2 -> f16x2, HFMA2 against
// activations normalised into FP16, FP32 accumulation across 16-column blocks), the
// two shared BF16 experts folded in as extra jobs of the same launches.
//
//   gate_up_kernel : activated[route] = bf16(silu(gate) * up)
//   down_kernel    : output[token]    = sum_routes bf16(bf16(down) * w) + sum_shared bf16(down)
#include "../../include/inkling_b200.h"
#include "common.cuh"
#include "decode_args.cuh"
// this file stages its activations itself, in natural order: every word decoded with the conversion instruction
#define INK_E2M1_ON_ALU 0
#include "stream_math.cuh"

namespace ink {

// Geometry of one NVFP4 row of K columns seen by a warp: a row is K/32 chunks of 16
// bytes (32 weights, two scale bytes); LPR lanes share a row, each lane owns CPL chunks,
// and a warp covers RPP rows per pass.
template <int K>
struct RowMap {
  static constexpr int CH = K / 32;
  static constexpr int LPR = CH < 32 ? CH : 32;
  static constexpr int CPL = CH / LPR;
  static constexpr int RPP = 32 / LPR;
  static constexpr int PASSES = (kBatchLoads / CPL) > 0 ? (kBatchLoads / CPL) : 1;  // passes per batch
  static constexpr int ROWS_PER_BATCH = PASSES * RPP;
};

// 8 BF16 weights x 8 FP32 activations
__device__ __forceinline__ float dot8_bf16(const uint4& q, const float4& xa, const float4& xb, float acc) {
  acc = fmaf(bf16lo(q.x), xa.x, acc); acc = fmaf(bf16hi(q.x), xa.y, acc);
  acc = fmaf(bf16lo(q.y), xa.z, acc); acc = fmaf(bf16hi(q.y), xa.w, acc);
  acc = fmaf(bf16lo(q.z), xb.x, acc); acc = fmaf(bf16hi(q.z), xb.y, acc);
  acc = fmaf(bf16lo(q.w), xb.z, acc); acc = fmaf(bf16hi(q.w), xb.w, acc);
  return acc;
}

// Sum over the LPR lanes that share a row; every lane of the group gets the total.
template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Whole block: vector of K BF16 values -> FP16 in shared memory, scaled by a power of
// two so that the largest magnitude is in [1, 2). Returns the inverse scale.
template <int K>
__device__ __forceinline__ float stage_normalised_f16(const uint16_t* src, uint16_t* dst, float* s_red) {
  const int tid = threadIdx.x;
  uint32_t amax = 0;
  for (int i = tid; i < K / 2; i += blockDim.x) {
    const uint32_t v = reinterpret_cast<const uint32_t*>(src)[i];
    amax = max(amax, max(v & 0x7fffu, (v >> 16) & 0x7fffu));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((tid & 31) == 0) s_red[tid >> 5] = __uint_as_float(amax);
  __syncthreads();
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) amax = max(amax, __float_as_uint(s_red[w]));
  float inverse;
  const float scale = pow2_normaliser(amax, &inverse);
  for (int i = tid; i < K / 2; i += blockDim.x) {
    const uint32_t v = reinterpret_cast<const uint32_t*>(src)[i];
    reinterpret_cast<uint32_t*>(dst)[i] = f32x2_to_f16x2(bf16lo(v) * scale, bf16hi(v) * scale);
  }
  __syncthreads();
  return inverse;
}

// One warp: dot products of `rows` consecutive NVFP4 rows starting at row0 (rows beyond
// n_rows are skipped) against the lane's activation registers. After the call lane
// groups hold their row totals (unscaled) in result[pass].
template <int K>
__device__ __forceinline__ void warp_rows_nvfp4(const uint8_t* __restrict__ W, const uint8_t* __restrict__ S,
                                                int row0, int n_rows, const uint32_t (&xr)[RowMap<K>::CPL][16],
                                                float (&result)[RowMap<K>::PASSES]) {
  using M = RowMap<K>;
  const int lane = threadIdx.x & 31, sl = lane % M::LPR, rp = lane / M::LPR;
  uint4 q[M::PASSES][M::CPL];
  uint32_t sc[M::PASSES][M::CPL];
#pragma unroll
  for (int p = 0; p < M::PASSES; ++p) {
    const int row = row0 + p * M::RPP + rp;
    const bool ok = row < n_rows;
#pragma unroll
    for (int j = 0; j < M::CPL; ++j) {
      const int chunk = j * M::LPR + sl;
      if (ok) {
        q[p][j] = ldg_stream_16(W + (size_t)row * (K / 2) + chunk * 16);
        sc[p][j] = ldg_stream_u16(S + (size_t)row * (K / 16) + chunk * 2);
      } else {
        q[p][j] = make_uint4(0, 0, 0, 0);
        sc[p][j] = 0;
      }
    }
  }
#pragma unroll
  for (int p = 0; p < M::PASSES; ++p) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < M::CPL; ++j) acc += dot32(q[p][j], sc[p][j], xr[j]);
    result[p] = group_sum<M::LPR>(acc);
  }
}

template <int K>
__device__ __forceinline__ void load_x_registers(const uint16_t* s_x, uint32_t (&xr)[RowMap<K>::CPL][16]) {
  using M = RowMap<K>;
  const int sl = (threadIdx.x & 31) % M::LPR;
#pragma unroll
  for (int j = 0; j < M::CPL; ++j) {
    const uint4* p = reinterpret_cast<const uint4*>(s_x + (j * M::LPR + sl) * 32);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const uint4 t = p[v];
      xr[j][4 * v + 0] = t.x; xr[j][4 * v + 1] = t.y; xr[j][4 * v + 2] = t.z; xr[j][4 * v + 3] = t.w;
    }
  }
}

// One warp: dot product of one BF16 row of K columns with FP32 activations in shared
// memory; all lanes return the total.
template <int K>
__device__ __forceinline__ float warp_row_bf16(const uint16_t* __restrict__ row, const float* s_x) {
  constexpr int CHUNKS = K / 8;
  constexpr int PER_LANE = (CHUNKS + 31) / 32;
  const int lane = threadIdx.x & 31;
  float acc = 0.f;
#pragma unroll
  for (int base = 0; base < PER_LANE; base += kBatchLoads) {
    uint4 q[kBatchLoads];
#pragma unroll
    for (int i = 0; i < kBatchLoads; ++i) {
      const int c = (base + i) * 32 + lane;
      q[i] = (base + i < PER_LANE && c < CHUNKS) ? ldg_stream_16(row + c * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kBatchLoads; ++i) {
      const int c = (base + i) * 32 + lane;
      if (base + i < PER_LANE && c < CHUNKS) {
        const float4 xa = *reinterpret_cast<const float4*>(s_x + c * 8);
        const float4 xb = *reinterpret_cast<const float4*>(s_x + c * 8 + 4);
        acc = dot8_bf16(q[i], xa, xb, acc);
      }
    }
  }
  return warp_sum(acc);
}

// gate and up rows of a BF16 pair, loads of both rows in flight together
template <int K>
__device__ __forceinline__ void warp_pair_bf16(const uint16_t* __restrict__ gate_row,
                                               const uint16_t* __restrict__ up_row, const float* s_x,
                                               float* gate, float* up) {
  constexpr int CHUNKS = K / 8;
  constexpr int PER_LANE = (CHUNKS + 31) / 32;
  constexpr int HALF = kBatchLoads / 2;
  const int lane = threadIdx.x & 31;
  float g = 0.f, u = 0.f;
#pragma unroll
  for (int base = 0; base < PER_LANE; base += HALF) {
    uint4 qg[HALF], qu[HALF];
#pragma unroll
    for (int i = 0; i < HALF; ++i) {
      const int c = (base + i) * 32 + lane;
      const bool ok = base + i < PER_LANE && c < CHUNKS;
      qg[i] = ok ? ldg_stream_16(gate_row + c * 8) : make_uint4(0, 0, 0, 0);
      qu[i] = ok ? ldg_stream_16(up_row + c * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < HALF; ++i) {
      const int c = (base + i) * 32 + lane;
      if (base + i < PER_LANE && c < CHUNKS) {
        const float4 xa = *reinterpret_cast<const float4*>(s_x + c * 8);
        const float4 xb = *reinterpret_cast<const float4*>(s_x + c * 8 + 4);
        g = dot8_bf16(qg[i], xa, xb, g);
        u = dot8_bf16(qu[i], xa, xb, u);
      }
    }
  }
  *gate = warp_sum(g);
  *up = warp_sum(u);
}

// ============================================================== gate / up
constexpr int kGateUpThreads = 256;
constexpr int kGateUpWarps = kGateUpThreads / 32;
constexpr int kGateUpBatches = 4;       // NVFP4 batches a warp runs through
constexpr int kSharedPairsPerWarp = 1;  // BF16 (gate, up) pairs a warp runs through

template <int K>
struct GateUpTile {
  static constexpr int Q_ROWS = kGateUpWarps * kGateUpBatches * RowMap<K>::ROWS_PER_BATCH;  // NVFP4 rows per block
  static constexpr int S_PAIRS = kGateUpWarps * kSharedPairsPerWarp;                        // BF16 pairs per block
};

template <int K>
__global__ void __launch_bounds__(kGateUpThreads) gate_up_kernel(DecodeArgs a, int q_tiles, int s_tiles) {
  using M = RowMap<K>;
  __shared__ __align__(16) unsigned char s_x_raw[K * 4];
  __shared__ float s_red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int routes = a.tokens * a.top_k;
  const int f = a.intermediate;
  int block = blockIdx.x;
  if (block < routes * q_tiles) {
    // ------------------------------------------------ routed NVFP4 job
    const int route = block / q_tiles, tile = block % q_tiles;
    const int64_t expert = a.indices[route];
    if (expert < 0 || expert > a.max_expert) {
      if (threadIdx.x == 0 && a.status) atomicOr(a.status, kFlagExpertOutOfRange);
      return;
    }
    const int64_t* entry = a.pointers + expert * kBank;
    const uint8_t* W = reinterpret_cast<const uint8_t*>(entry[0]);
    if (W == nullptr) return;
    const uint8_t* S = reinterpret_cast<const uint8_t*>(entry[1]);
    const float scale2 = *reinterpret_cast<const float*>(entry[2]);
    uint16_t* s_x = reinterpret_cast<uint16_t*>(s_x_raw);
    const float inverse = stage_normalised_f16<K>(a.x + (size_t)(route / a.top_k) * K, s_x, s_red);
    uint32_t xr[M::CPL][16];
    load_x_registers<K>(s_x, xr);
    const float scale = scale2 * inverse;
    const int n_rows = 2 * f;
    const int sl = lane % M::LPR, rp = lane / M::LPR;
    const int warp_row0 = tile * GateUpTile<K>::Q_ROWS + warp * kGateUpBatches * M::ROWS_PER_BATCH;
    uint16_t* y = a.activated + (size_t)route * f;
#pragma unroll 1
    for (int b = 0; b < kGateUpBatches; ++b) {
      const int row0 = warp_row0 + b * M::ROWS_PER_BATCH;
      if (row0 >= n_rows) break;
      float r[M::PASSES];
      warp_rows_nvfp4<K>(W, S, row0, n_rows, xr, r);
      if constexpr (M::RPP == 1) {
        // even pass = gate row, odd pass = up row
#pragma unroll
        for (int p = 0; p + 1 < M::PASSES; p += 2) {
          const int row = row0 + p;
          if (lane == 0 && row + 1 < n_rows)
            y[row / 2] = (uint16_t)f32_to_bf16_bits(silu_mul(r[p] * scale, r[p + 1] * scale));
        }
      } else {
        // neighbouring lane groups hold gate (even row) and up (odd row)
#pragma unroll
        for (int p = 0; p < M::PASSES; ++p) {
          const float other = __shfl_xor_sync(0xffffffffu, r[p], M::LPR);
          const int row = row0 + p * M::RPP + rp;
          if (sl == 0 && (rp & 1) == 0 && row + 1 < n_rows)
            y[row / 2] = (uint16_t)f32_to_bf16_bits(silu_mul(r[p] * scale, other * scale));
        }
      }
    }
    return;
  }
  // ---------------------------------------------------- shared BF16 job
  block -= routes * q_tiles;
  const int job = block / s_tiles, tile = block % s_tiles;  // job = token * n_shared + e
  const int token = job / a.n_shared, e = job % a.n_shared;
  float* s_x = reinterpret_cast<float*>(s_x_raw);
  const uint16_t* x = a.x + (size_t)token * K;
  for (int i = threadIdx.x; i < K / 2; i += blockDim.x) {
    const uint32_t v = reinterpret_cast<const uint32_t*>(x)[i];
    s_x[2 * i] = bf16lo(v);
    s_x[2 * i + 1] = bf16hi(v);
  }
  __syncthreads();
  const uint16_t* Wg = a.shared_gate + (size_t)e * f * K;
  const uint16_t* Wu = a.shared_up + (size_t)e * f * K;
  uint16_t* y = a.shared_activated + (size_t)job * f;
#pragma unroll 1
  for (int i = 0; i < kSharedPairsPerWarp; ++i) {
    const int j = tile * GateUpTile<K>::S_PAIRS + warp * kSharedPairsPerWarp + i;
    if (j >= f) break;
    float g, u;
    warp_pair_bf16<K>(Wg + (size_t)j * K, Wu + (size_t)j * K, s_x, &g, &u);
    if (lane == 0) {
      // the reference's BF16 tensor ops: bmm outputs, silu, product each round to BF16
      g = round_bf16(g);
      u = round_bf16(u);
      const float act = round_bf16(g / (1.f + expf(-g)));
      y[j] = (uint16_t)f32_to_bf16_bits(act * u);
    }
  }
}

// ================================================================= down
constexpr int kDownThreads = 128;
constexpr int kDownWarps = kDownThreads / 32;

template <int K>
struct DownTile {
  static constexpr int ROWS_PER_WARP = RowMap<K>::ROWS_PER_BATCH;   // NVFP4 rows a warp owns
  static constexpr int ROWS = kDownWarps * ROWS_PER_WARP;          // output rows per block
};

// dynamic shared memory: top_k FP16 vectors of K, then n_shared FP32 vectors of K
template <int K>
__global__ void __launch_bounds__(kDownThreads) down_kernel(DecodeArgs a, int tiles) {
  using M = RowMap<K>;
  using T = DownTile<K>;
  extern __shared__ __align__(16) unsigned char s_dyn[];
  __shared__ float s_inverse[32];
  __shared__ float s_total[kDownWarps][T::ROWS_PER_WARP];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x / tiles, tile = blockIdx.x % tiles;
  const int d = a.hidden;
  uint16_t* s_act = reinterpret_cast<uint16_t*>(s_dyn);                         // [top_k][K] FP16
  float* s_shared = reinterpret_cast<float*>(s_dyn + (size_t)a.top_k * K * 2);  // [n_shared][K] FP32
  // ---- stage the activations of every job of this token; one warp per job
  const int jobs = a.top_k + a.n_shared;
  for (int job = warp; job < jobs; job += kDownWarps) {
    if (job < a.top_k) {
      const uint16_t* src = a.activated + (size_t)(token * a.top_k + job) * K;
      uint32_t amax = 0;
      for (int i = lane; i < K / 2; i += 32) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(src)[i];
        amax = max(amax, max(v & 0x7fffu, (v >> 16) & 0x7fffu));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      float inverse;
      const float scale = pow2_normaliser(amax, &inverse);
      if (lane == 0) s_inverse[job] = inverse;
      uint32_t* dst = reinterpret_cast<uint32_t*>(s_act + (size_t)job * K);
      for (int i = lane; i < K / 2; i += 32) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(src)[i];
        dst[i] = f32x2_to_f16x2(bf16lo(v) * scale, bf16hi(v) * scale);
      }
    } else {
      const int e = job - a.top_k;
      const uint16_t* src = a.shared_activated + (size_t)(token * a.n_shared + e) * K;
      const float gamma = bf16_to_f32(a.gammas[token * a.n_shared + e]);
      float* dst = s_shared + (size_t)e * K;
      for (int i = lane; i < K / 2; i += 32) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(src)[i];
        // gamma multiplies the activation before the down projection, rounded to BF16
        dst[2 * i] = round_bf16(bf16lo(v) * gamma);
        dst[2 * i + 1] = round_bf16(bf16hi(v) * gamma);
      }
    }
  }
  for (int i = lane; i < T::ROWS_PER_WARP; i += 32) s_total[warp][i] = 0.f;
  __syncthreads();
  const int warp_row0 = tile * T::ROWS + warp * T::ROWS_PER_WARP;
  const int sl = lane % M::LPR, rp = lane / M::LPR;
  // ---- routed jobs, in choice order
#pragma unroll 1
  for (int choice = 0; choice < a.top_k; ++choice) {
    const int route = token * a.top_k + choice;
    const int64_t expert = a.indices[route];
    if (expert < 0 || expert > a.max_expert) {
      if (threadIdx.x == 0 && tile == 0 && a.status) atomicOr(a.status, kFlagExpertOutOfRange);
      continue;
    }
    const int64_t* entry = a.pointers + expert * kBank + 3;
    const uint8_t* W = reinterpret_cast<const uint8_t*>(entry[0]);
    if (W == nullptr) continue;
    const uint8_t* S = reinterpret_cast<const uint8_t*>(entry[1]);
    const float scale = *reinterpret_cast<const float*>(entry[2]) * s_inverse[choice];
    const float w = bf16_to_f32(a.weights[route]);
    uint32_t xr[M::CPL][16];
    load_x_registers<K>(s_act + (size_t)choice * K, xr);
    float r[M::PASSES];
    warp_rows_nvfp4<K>(W, S, warp_row0, d, xr, r);
#pragma unroll
    for (int p = 0; p < M::PASSES; ++p) {
      if (sl == 0) {
        const float down = round_bf16(r[p] * scale);
        s_total[warp][p * M::RPP + rp] += round_bf16(down * w);
      }
    }
    __syncwarp();
  }
  // ---- shared jobs: BF16 rows, one row per warp pass
#pragma unroll 1
  for (int e = 0; e < a.n_shared; ++e) {
    const uint16_t* Wd = a.shared_down + (size_t)e * d * K;
#pragma unroll 1
    for (int i = 0; i < T::ROWS_PER_WARP; ++i) {
      const int row = warp_row0 + i;
      if (row >= d) break;
      const float v = warp_row_bf16<K>(Wd + (size_t)row * K, s_shared + (size_t)e * K);
      if (lane == 0) s_total[warp][i] += round_bf16(v);
    }
    __syncwarp();
  }
  __syncwarp();
  for (int i = lane; i < T::ROWS_PER_WARP; i += 32)
    if (warp_row0 + i < d) a.output[(size_t)token * d + warp_row0 + i] = s_total[warp][i];
}

// ============================================== BF16 expert banks (pointer stride 2)
// The unquantised expert layer (the reference's routed_decode.cu built with QUANT=0, :85-101):
// the same two kernels over BF16 rows, no scales. A route's table row is (gate_up_proj, down_proj).
constexpr int kBankBf16 = 2;
constexpr int kBf16PairsPerWarp = 2;

template <int K>
__global__ void __launch_bounds__(kGateUpThreads) gate_up_bf16_kernel(DecodeArgs a, int tiles) {
  __shared__ __align__(16) float s_x[K];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int route = blockIdx.x / tiles, tile = blockIdx.x % tiles;
  const int f = a.intermediate;
  const int64_t expert = a.indices[route];
  if (expert < 0 || expert > a.max_expert) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, kFlagExpertOutOfRange);
    return;
  }
  const uint16_t* W = reinterpret_cast<const uint16_t*>(a.pointers[expert * kBankBf16]);
  if (W == nullptr) return;
  const uint16_t* x = a.x + (size_t)(route / a.top_k) * K;
  for (int i = threadIdx.x; i < K / 2; i += blockDim.x) {
    const uint32_t v = reinterpret_cast<const uint32_t*>(x)[i];
    s_x[2 * i] = bf16lo(v);
    s_x[2 * i + 1] = bf16hi(v);
  }
  __syncthreads();
  uint16_t* y = a.activated + (size_t)route * f;
#pragma unroll 1
  for (int i = 0; i < kBf16PairsPerWarp; ++i) {
    const int j = (tile * kGateUpWarps + warp) * kBf16PairsPerWarp + i;
    if (j >= f) break;
    float g, u;
    // rows interleave: gate = row 2j, up = row 2j + 1
    warp_pair_bf16<K>(W + (size_t)(2 * j) * K, W + (size_t)(2 * j + 1) * K, s_x, &g, &u);
    if (lane == 0) y[j] = (uint16_t)f32_to_bf16_bits(silu_mul(g, u));
  }
}

// dynamic shared memory: top_k FP32 vectors of K
template <int K>
__global__ void __launch_bounds__(kDownThreads) down_bf16_kernel(DecodeArgs a, int tiles, int rows_per_warp) {
  extern __shared__ __align__(16) unsigned char s_dyn[];
  float* s_act = reinterpret_cast<float*>(s_dyn);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x / tiles, tile = blockIdx.x % tiles;
  const int d = a.hidden;
  for (int i = threadIdx.x; i < a.top_k * (K / 2); i += blockDim.x) {
    const uint32_t v = reinterpret_cast<const uint32_t*>(a.activated + (size_t)token * a.top_k * K)[i];
    s_act[2 * i] = bf16lo(v);
    s_act[2 * i + 1] = bf16hi(v);
  }
  __syncthreads();
  const int row0 = (tile * kDownWarps + warp) * rows_per_warp;
#pragma unroll 1
  for (int i = 0; i < rows_per_warp; ++i) {
    const int row = row0 + i;
    if (row >= d) break;
    float total = 0.f;
#pragma unroll 1
    for (int choice = 0; choice < a.top_k; ++choice) {
      const int route = token * a.top_k + choice;
      const int64_t expert = a.indices[route];
      if (expert < 0 || expert > a.max_expert) {
        if (lane == 0 && row == 0 && a.status) atomicOr(a.status, kFlagExpertOutOfRange);
        continue;
      }
      const uint16_t* W = reinterpret_cast<const uint16_t*>(a.pointers[expert * kBankBf16 + 1]);
      if (W == nullptr) continue;
      const float down = round_bf16(warp_row_bf16<K>(W + (size_t)row * K, s_act + (size_t)choice * K));
      total += round_bf16(down * bf16_to_f32(a.weights[route]));
    }
    if (lane == 0) a.output[(size_t)token * d + row] = total;
  }
}

template <int K>
static int launch_gate_up_bf16(const DecodeArgs& a, cudaStream_t stream) {
  const int per_block = kGateUpWarps * kBf16PairsPerWarp;
  const int tiles = (a.intermediate + per_block - 1) / per_block;
  gate_up_bf16_kernel<K><<<(unsigned)(a.tokens * a.top_k * tiles), kGateUpThreads, 0, stream>>>(a, tiles);
  INK_CHECK_LAUNCH("gate_up (BF16 banks)");
  return kOk;
}

template <int K>
static int launch_down_bf16(const DecodeArgs& a, cudaStream_t stream) {
  const int rows_per_warp = 4, per_block = kDownWarps * rows_per_warp;
  const int tiles = (a.hidden + per_block - 1) / per_block;
  const size_t smem = (size_t)a.top_k * K * 4;
  static thread_local size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(down_bf16_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "down (BF16 banks): %zu bytes of shared memory refused: %s", smem,
                cudaGetErrorString(e));
    configured = smem;
  }
  down_bf16_kernel<K><<<(unsigned)(a.tokens * tiles), kDownThreads, smem, stream>>>(a, tiles, rows_per_warp);
  INK_CHECK_LAUNCH("down (BF16 banks)");
  return kOk;
}

// ---------------------------------------------------------------- launchers
template <int K>
static int launch_gate_up(const DecodeArgs& a, cudaStream_t stream) {
  const int routes = a.tokens * a.top_k;
  const int q_tiles = (2 * a.intermediate + GateUpTile<K>::Q_ROWS - 1) / GateUpTile<K>::Q_ROWS;
  const int s_tiles = (a.intermediate + GateUpTile<K>::S_PAIRS - 1) / GateUpTile<K>::S_PAIRS;
  const long long blocks = (long long)routes * q_tiles + (long long)a.tokens * a.n_shared * s_tiles;
  if (blocks == 0) return kOk;
  INK_PREFER_MAX_SMEM(gate_up_kernel<K>);
  gate_up_kernel<K><<<(unsigned)blocks, kGateUpThreads, 0, stream>>>(a, q_tiles, s_tiles);
  INK_CHECK_LAUNCH("gate_up");
  return kOk;
}

template <int K>
static int launch_down(const DecodeArgs& a, cudaStream_t stream) {
  const int tiles = (a.hidden + DownTile<K>::ROWS - 1) / DownTile<K>::ROWS;
  const size_t smem = (size_t)a.top_k * K * 2 + (size_t)a.n_shared * K * 4;
  static thread_local size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(down_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "down: %zu bytes of shared memory refused: %s", smem,
                cudaGetErrorString(e));
    configured = smem;
  }
  INK_PREFER_MAX_SMEM(down_kernel<K>);
  down_kernel<K><<<(unsigned)(a.tokens * tiles), kDownThreads, smem, stream>>>(a, tiles);
  INK_CHECK_LAUNCH("down");
  return kOk;
}

#define INK_DISPATCH_WIDTH(width, call)                     \
  switch (width) {                                          \
    case 64: return call<64>(a, stream);                    \
    case 128: return call<128>(a, stream);                  \
    case 256: return call<256>(a, stream);                  \
    case 512: return call<512>(a, stream);                  \
    case 1024: return call<1024>(a, stream);                \
    case 2048: return call<2048>(a, stream);                \
    case 4096: return call<4096>(a, stream);                \
    default: break;                                         \
  }

static int dispatch_gate_up(const DecodeArgs& a, cudaStream_t stream) {
  INK_DISPATCH_WIDTH(a.hidden, launch_gate_up)
  set_error("gate_up: hidden=%d unsupported (power of two, 64..4096)", a.hidden);
  return kUnsupportedShape;
}
static int dispatch_down(const DecodeArgs& a, cudaStream_t stream) {
  INK_DISPATCH_WIDTH(a.intermediate, launch_down)
  set_error("down: intermediate=%d unsupported (power of two, 64..4096)", a.intermediate);
  return kUnsupportedShape;
}
static int dispatch_gate_up_bf16(const DecodeArgs& a, cudaStream_t stream) {
  INK_DISPATCH_WIDTH(a.hidden, launch_gate_up_bf16)
  set_error("gate_up (BF16 banks): hidden=%d unsupported (power of two, 64..4096)", a.hidden);
  return kUnsupportedShape;
}
static int dispatch_down_bf16(const DecodeArgs& a, cudaStream_t stream) {
  INK_DISPATCH_WIDTH(a.intermediate, launch_down_bf16)
  set_error("down (BF16 banks): intermediate=%d unsupported (power of two, 64..4096)", a.intermediate);
  return kUnsupportedShape;
}

static int check_decode(const DecodeArgs& a, bool with_shared) {
  INK_REQUIRE(a.tokens >= 0 && a.top_k >= 1 && a.top_k <= 30 && a.max_expert >= 0, kBadArgument,
              "decode: tokens=%d top_k=%d max_expert=%d", a.tokens, a.top_k, a.max_expert);
  if (a.tokens == 0) return kOk;  // nothing to read or write: pointers may be null
  INK_REQUIRE(a.x && a.indices && a.weights && a.pointers && a.activated && a.output, kBadArgument,
              "decode: null pointer argument");
  INK_REQUIRE(aligned16(a.x) && aligned16(a.indices) && aligned16(a.weights) && aligned16(a.activated) &&
                  aligned16(a.output),
              kMisaligned, "decode: buffers must be 16-byte aligned");
  if (with_shared && a.n_shared > 0) {
    INK_REQUIRE(a.shared_gate && a.shared_up && a.shared_down && a.gammas && a.shared_activated, kBadArgument,
                "moe_decode: null shared-expert argument");
    INK_REQUIRE(aligned16(a.shared_gate) && aligned16(a.shared_up) && aligned16(a.shared_down) &&
                    aligned16(a.shared_activated),
                kMisaligned, "moe_decode: shared-expert buffers must be 16-byte aligned");
    INK_REQUIRE(a.n_shared <= 8, kUnsupportedShape, "moe_decode: n_shared=%d (at most 8)", a.n_shared);
  }
  return kOk;
}

// streaming kernels for the production widths (stream_decode.cu)
bool stream_gate_up_supported(const DecodeArgs& a);
bool stream_down_supported(const DecodeArgs& a);
int dispatch_gate_up_stream(const DecodeArgs& a, cudaStream_t stream);
int dispatch_down_stream(const DecodeArgs& a, cudaStream_t stream);

}  // namespace ink

using namespace ink;

static DecodeArgs make_decode_args(const void* x, const int64_t* indices, const void* weights,
                                   const int64_t* pointers, void* activated, const void* shared_gate,
                                   const void* shared_up, const void* shared_down, const void* gammas,
                                   void* shared_activated, float* output, int tokens, int top_k, int n_shared,
                                   int hidden, int intermediate, int max_expert, int32_t* status) {
  DecodeArgs a;
  a.x = (const uint16_t*)x;
  a.indices = indices;
  a.weights = (const uint16_t*)weights;
  a.pointers = pointers;
  a.activated = (uint16_t*)activated;
  a.shared_gate = (const uint16_t*)shared_gate;
  a.shared_up = (const uint16_t*)shared_up;
  a.shared_down = (const uint16_t*)shared_down;
  a.gammas = (const uint16_t*)gammas;
  a.shared_activated = (uint16_t*)shared_activated;
  a.output = output;
  a.tokens = tokens;
  a.top_k = top_k;
  a.n_shared = n_shared;
  a.hidden = hidden;
  a.intermediate = intermediate;
  a.max_expert = max_expert;
  a.status = status;
  return a;
}

#define INK_MOE_PARAMS                                                                                       \
  const void *x, const int64_t *indices, const void *weights, const int64_t *pointers, void *activated,      \
      const void *shared_gate, const void *shared_up, const void *shared_down, const void *gammas,           \
      void *shared_activated, float *output, int tokens, int top_k, int n_shared, int hidden,                \
      int intermediate, int max_expert, int32_t *status, ink_stream_t stream
#define INK_MOE_ARGS                                                                                          \
  x, indices, weights, pointers, activated, shared_gate, shared_up, shared_down, gammas, shared_activated,   \
      output, tokens, top_k, n_shared, hidden, intermediate, max_expert, status

extern "C" int ink_moe_gate_up(INK_MOE_PARAMS) {
  DecodeArgs a = make_decode_args(INK_MOE_ARGS);
  if (int rc = check_decode(a, true)) return rc;
  if (tokens == 0) return kOk;
  if (stream_gate_up_supported(a)) return dispatch_gate_up_stream(a, (cudaStream_t)stream);
  return dispatch_gate_up(a, (cudaStream_t)stream);
}

extern "C" int ink_moe_down(INK_MOE_PARAMS) {
  DecodeArgs a = make_decode_args(INK_MOE_ARGS);
  if (int rc = check_decode(a, true)) return rc;
  if (tokens == 0) return kOk;
  if (stream_down_supported(a)) return dispatch_down_stream(a, (cudaStream_t)stream);
  return dispatch_down(a, (cudaStream_t)stream);
}

extern "C" int ink_moe_decode(INK_MOE_PARAMS) {
  if (int rc = ink_moe_gate_up(INK_MOE_ARGS, stream)) return rc;
  return ink_moe_down(INK_MOE_ARGS, stream);
}

extern "C" int ink_routed_decode(const void* x, const int64_t* indices, const void* weights,
                                 const int64_t* pointers, void* activated, float* output, int tokens, int top_k,
                                 int hidden, int intermediate, int max_expert, int quantized, int32_t* status,
                                 ink_stream_t stream) {
  INK_REQUIRE(quantized == 0 || quantized == 1, kBadArgument, "routed_decode: quantized=%d", quantized);
  if (quantized == 0) {
    // BF16 banks: pointer table [expert][2] = (gate_up_proj BF16 [2f, d], down_proj BF16 [d, f])
    DecodeArgs a = make_decode_args(x, indices, weights, pointers, activated, nullptr, nullptr, nullptr, nullptr, nullptr,
                                    output, tokens, top_k, 0, hidden, intermediate, max_expert, status);
    if (int rc = check_decode(a, false)) return rc;
    if (tokens == 0) return kOk;
    if (int rc = dispatch_gate_up_bf16(a, (cudaStream_t)stream)) return rc;
    return dispatch_down_bf16(a, (cudaStream_t)stream);
  }
  return ink_moe_decode(x, indices, weights, pointers, activated, nullptr, nullptr, nullptr, nullptr, nullptr,
                        output, tokens, top_k, 0, hidden, intermediate, max_expert, status, stream);
}

// Grouped expert projections on the block-scaled tensor-core path: the packed NVFP4 codes of an
// expert's 128-row weight tile are the M operand of tcgen05.mma.kind::mxf4nvf4.block_scale.block16
// straight from the checkpoint layout (tiled TMA into a ring of 18 KB units: 128 rows x 256 columns of
// codes and their E4M3 block scales), nothing is converted on the CUDA cores; the tokens routed to the
// expert are the N operand, each as four E2M1 digit rows with power-of-two block scales (tc_path.cuh),
// up to eight tokens (N = 32) per pass. Every active expert's bytes cross HBM once per eight of its
// tokens; accumulators live in tensor memory and are read back once per tile. The digit rows of every
// input row are made ONCE, by a small kernel in front, as ready-to-use pieces of the swizzled operand
// (a piece's swizzle depends on whether its token sits in an even or an odd slot of the batch, so both
// are kept); the main kernel only copies the pieces of a batch's tokens into place. (Making them per
// work item -- thirty-two tiles per expert need the same rows -- cost two thirds of the kernel's time.)
//
// Persistent blocks, one per SM. A work item is (expert group, batch of <= 8 routes, 128-row tile), tile
// fastest; every block takes a contiguous run of items, so it stages the activations of only one or two
// batches (the tiles of a batch share them). Warp 0 lane 0 streams weight units (it runs ahead of everything
// else: addresses do not depend on activations), warp 1 lane 0 issues the MMAs, warps 2..5 move each
// unit's weight scales from shared to tensor memory, warps 6..9 read the accumulators and write the
// outputs; warps 2..9 together turn the batch's activations into digit rows before its first MMA.
// Every wait is bounded; a wait that gives up sets kFlagWaitTimedOut and the block drains.
#include <stdlib.h>

#include "../../include/inkling_b200.h"
#include "common.cuh"
#include "decode_args.cuh"
#include "pipe.cuh"
#include "tc_path.cuh"

namespace ink {

constexpr int kGtBatch = 8;                      // routes per pass (x 4 digit rows = MMA N 32)
constexpr int kGtN = kGtBatch * kTcDigits;       // 32
constexpr int kGtUnits = 7;                      // ring depth, units of kTcUnitBytes
constexpr int kGtThreads = 320;
constexpr int kGtWorkers = 256;                  // warps 2..9
constexpr int kGtMaxGroups = 1024;
constexpr int kGtMaxK = 4096;                    // activation scales of a whole row must fit the tensor-memory columns

struct GemmTcArgs {
  const uint16_t* X;            // BF16 [*, K]
  const unsigned char* maps;    // the layer's four TMA descriptors (gate/up codes, scales, down codes, scales)
  const int64_t* pointers;      // [(max_expert + 1) * 6]: scale2 is read through it, a zero row is an inactive expert
  const int32_t* experts;       // [groups]
  const int32_t* rows;          // [groups, capacity]
  const int32_t* counts;        // [groups]
  uint16_t* Y;
  const float2* row_scale;      // per row of X: {power-of-two multiplier, its inverse}
  const unsigned char* digits;  // per row of X: [K/256 chunks][slot parity][4 digit rows][128 B], swizzled as the operand wants them
  const unsigned char* digit_scales;   // per row of X: [4 digit rows][kGtMaxK / 16] E4M3 block scales
  int capacity, n, k, top_k, groups, start;
  int32_t* status;
  long long* prof;              // optional [blocks][8] clock totals per phase (INKLING_GROUPED_PROFILE=1)
};

struct GtShared {
  uint64_t full[kGtUnits], empty[kGtUnits];
  uint64_t sf_full[kTcSfSlots], sf_empty[kTcSfSlots];
  uint64_t d_full[2], d_empty[2];      // two accumulators: the next tile's MMAs run while this one is read
  uint32_t tmem_base;
  volatile int staged;                 // items whose activations are staged as digit rows
  volatile int failed;
  int first_item[kGtMaxGroups + 1];    // items before each group
  int route[kGtBatch];
  float out_scale[kGtBatch];
  uint8_t sfb[kGtN][kGtMaxK / 16];     // block scales of the digit rows
};

__device__ __forceinline__ bool gt_wait(uint64_t* bar, uint32_t parity, GtShared* sh) {
  if (sh->failed) return false;
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (sh->failed) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      sh->failed = 1;
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void gt_worker_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }

// batches of a group (0: nothing to do for it)
__device__ __forceinline__ int gt_batches(const GemmTcArgs& a, int g, int bank) {
  const int count = a.counts[g], expert = a.experts[g];
  if (count <= 0 || expert < 0) return 0;
  if (a.pointers[(size_t)expert * kBank + bank] == 0) return 0;
  return (count + kGtBatch - 1) / kGtBatch;
}

struct GtItem { int group, batch, tile, batches; };
__device__ __forceinline__ GtItem gt_item(const GtShared& sh, int groups, int tiles, int index) {
  int lo = 0, hi = groups;   // largest g with first_item[g] <= index
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sh.first_item[mid] <= index) lo = mid;
    else hi = mid;
  }
  GtItem it;
  it.group = lo;
  it.batches = (sh.first_item[lo + 1] - sh.first_item[lo]) / tiles;
  const int local = index - sh.first_item[lo];
  it.batch = local / tiles;
  it.tile = local % tiles;
  return it;
}

template <int PROJ>
__global__ void __launch_bounds__(kGtThreads, 1) expert_gemm_tc_kernel(GemmTcArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ GtShared sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char* units = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles: 1024-byte aligned
  unsigned char* s_b = units + (size_t)kGtUnits * kTcUnitBytes;                          // [K/256][32 rows][128 B] digit rows
  const int K = a.k, chunks = K / kTcChunkK, tiles = a.n / kTcRows;
  const int bank = PROJ ? 3 : 0;
  const unsigned char* map_codes = a.maps + (PROJ ? 256 : 0);
  const unsigned char* map_scales = map_codes + 128;

  // ---- items before each group: all threads fetch the groups' sizes, one warp adds them up
  for (int g = threadIdx.x; g < a.groups; g += kGtThreads) sh.first_item[g + 1] = gt_batches(a, g, bank) * tiles;
  __syncthreads();
  if (warp == 0) {
    const int per_lane = (a.groups + 31) / 32;
    int mine = 0;
    for (int i = 0; i < per_lane; ++i) {
      const int g = lane * per_lane + i;
      if (g < a.groups) mine += sh.first_item[g + 1];
    }
    int before = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, before, o);
      if (lane >= o) before += v;
    }
    before -= mine;
    for (int i = 0; i < per_lane; ++i) {
      const int g = lane * per_lane + i;
      if (g < a.groups) {
        before += sh.first_item[g + 1];
        sh.first_item[g + 1] = before;   // items up to and including group g
      }
    }
    if (lane == 0) sh.first_item[0] = 0;
    if (lane == 0) {
      for (int s = 0; s < kGtUnits; ++s) {
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
      sh.staged = 0;
      sh.failed = 0;
      mbar_init_fence();
    }
  }
  __syncthreads();
  const int total = sh.first_item[a.groups];
  const int item_lo = (int)((long long)blockIdx.x * total / gridDim.x), item_hi = (int)((long long)(blockIdx.x + 1) * total / gridDim.x);
  if (item_hi <= item_lo) return;   // (before any tensor memory is taken)
  if (warp == 1) tc_alloc(&sh.tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_base;

  if (warp == 0) {
    // =========================================================== producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(map_codes) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(map_scales) : "memory");
      long long seq = 0;
      for (int index = item_lo; index < item_hi && !sh.failed; ++index) {
        const GtItem it = gt_item(sh, a.groups, tiles, index);
        const int z = a.experts[it.group] - a.start;
        for (int c = 0; c < chunks; ++c, ++seq) {
          const int u = (int)(seq % kGtUnits);
          if (seq >= kGtUnits && !gt_wait(&sh.empty[u], (uint32_t)((seq / kGtUnits) - 1) & 1u, &sh)) break;
          unsigned char* dst = units + (size_t)u * kTcUnitBytes;
          mbar_expect_tx(&sh.full[u], kTcUnitBytes);
          tc_tma_3d(dst, map_codes, c * 128, it.tile * kTcRows, z, &sh.full[u]);
          tc_tma_3d(dst + kTcCodeBytes, map_scales, c * 16, it.tile * kTcRows, z, &sh.full[u]);
        }
      }
    }
  } else if (warp == 1) {
    // =========================================================== MMA issue
    if (lane == 0) {
      long long seq = 0;
      int item_count = 0;
      long long t_wait_staged = 0, t_loop = 0;
      const uint32_t idesc = tc_idesc(kGtN);
      int stagings = 0;
      for (int index = item_lo; index < item_hi && !sh.failed; ++index, ++item_count) {
        const long long t_a = clock64();
        const GtItem it = gt_item(sh, a.groups, tiles, index);
        if (index == item_lo || it.tile == 0) {   // a new batch: its digit rows and their scales must be in place
          const long long t0 = clock64();
          while (sh.staged <= stagings && !sh.failed)
            if (clock64() - t0 > kWaitLimitCycles) sh.failed = 1;
          __threadfence_block();
          ++stagings;
        }
        const long long t_b = clock64();
        t_wait_staged += t_b - t_a;
        const int dbuf = item_count & 1;
        if (!gt_wait(&sh.d_empty[dbuf], (uint32_t)((item_count >> 1) & 1) ^ 1u, &sh)) break;   // this accumulator's previous tile has been read
        tc_fence_after();
        for (int c = 0; c < chunks; ++c, ++seq) {
          const int u = (int)(seq % kGtUnits), sfs = (int)(seq % kTcSfSlots);
          if (!gt_wait(&sh.full[u], (uint32_t)(seq / kGtUnits) & 1u, &sh)) break;
          if (!gt_wait(&sh.sf_full[sfs], (uint32_t)(seq / kTcSfSlots) & 1u, &sh)) break;
          tc_fence_after();
          const uint64_t ad = tc_desc_sw128(smem_u32(units + (size_t)u * kTcUnitBytes));
          const uint64_t bd = tc_desc_sw128(smem_u32(s_b + (size_t)c * kGtN * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma(tmem + kTcColD + dbuf * kGtN, ad + 2 * k, bd + 2 * k, idesc, (c == 0 && k == 0) ? 0u : 1u,
                   tmem + kTcColSfa + sfs * 16 + k * 4, tmem + kTcColSfb + (c * 4 + k) * 4);
          tc_commit(&sh.empty[u]);
          tc_commit(&sh.sf_empty[sfs]);
          if (c == chunks - 1) tc_commit(&sh.d_full[dbuf]);
        }
        t_loop += clock64() - t_b;
      }
      if (a.prof) {
        a.prof[blockIdx.x * 8 + 4] = t_wait_staged;
        a.prof[blockIdx.x * 8 + 5] = t_loop;
      }
    }
  } else {
    // =========================================================== workers: warps 2..5 scales, 6..9 accumulators
    const int wt = threadIdx.x - 64;
    const bool scale_warp = warp < 6;
    const int sub = warp & 3;                                   // the tensor-memory subpartition this warp reaches
    const uint32_t lane_base = (uint32_t)(sub * 32) << 16;
    long long seq = 0;
    int item_count = 0;
    long long t_stage = 0, t_upload = 0, t_main = 0;
    const long long t_begin = clock64();
    int stagings = 0;
    long long t_1 = 0, t_2 = 0;
    for (int index = item_lo; index < item_hi; ++index, ++item_count) {
      const long long t_0 = clock64();
      const GtItem it = gt_item(sh, a.groups, tiles, index);
      const bool fresh = index == item_lo || it.tile == 0;                        // a new batch: stage its activations
      const bool last_of_batch = index + 1 == item_hi || it.tile + 1 == tiles;   // the next item (if any) stages again
      t_1 = t_2 = t_0;
      if (fresh) {
      const int expert = a.experts[it.group];
      const int count = a.counts[it.group];
      // ---- the batch's routes
      if (wt < kGtBatch) {
        const int at = it.batch * kGtBatch + wt;
        int route = -1;
        float out_scale = 0.f;
        if (at < count) {
          route = a.rows[(size_t)it.group * a.capacity + at];
          const int in_row = PROJ == 0 ? route / a.top_k : route;
          const float scale2 = *reinterpret_cast<const float*>(a.pointers[(size_t)expert * kBank + bank + 2]);
          out_scale = scale2 * a.row_scale[in_row].y * (1.f / 512.f);
        }
        sh.route[wt] = route;
        sh.out_scale[wt] = out_scale;
      }
      gt_worker_sync();
      // ---- the digit rows of the batch's tokens into place: 16-byte pieces, consecutive pieces to consecutive threads,
      // eight loads in flight per thread
      {
        const int pieces_per_route = chunks * 32;   // 512 bytes per chunk
        const int n_pieces = kGtBatch * pieces_per_route;
#pragma unroll 1
        for (int p0 = wt; p0 < n_pieces; p0 += 8 * kGtWorkers) {
          uint4 v[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int p = p0 + q * kGtWorkers;
            v[q] = make_uint4(0, 0, 0, 0);
            if (p < n_pieces) {
              const int j = p / pieces_per_route, rem = p % pieces_per_route, c = rem >> 5, piece = rem & 31;
              const int route = sh.route[j];
              if (route >= 0) {
                const int in_row = PROJ == 0 ? route / a.top_k : route;
                v[q] = __ldg(reinterpret_cast<const uint4*>(a.digits + (((size_t)in_row * chunks + c) * 2 + (j & 1)) * 512) + piece);
              }
            }
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int p = p0 + q * kGtWorkers;
            if (p < n_pieces) {
              const int j = p / pieces_per_route, rem = p % pieces_per_route, c = rem >> 5, piece = rem & 31;
              *reinterpret_cast<uint4*>(s_b + (size_t)c * kGtN * 128 + (size_t)j * 512 + piece * 16) = v[q];
            }
          }
        }
        constexpr int kScalePieces = kTcDigits * (kGtMaxK / 16) / 16;   // 16-byte pieces of a token's scale rows: 64
        for (int p = wt; p < kGtBatch * kScalePieces; p += kGtWorkers) {
          const int j = p / kScalePieces, piece = p % kScalePieces;
          const int route = sh.route[j];
          uint4 v = make_uint4(0, 0, 0, 0);
          if (route >= 0) {
            const int in_row = PROJ == 0 ? route / a.top_k : route;
            v = __ldg(reinterpret_cast<const uint4*>(a.digit_scales + (size_t)in_row * kTcDigits * (kGtMaxK / 16)) + piece);
          }
          reinterpret_cast<uint4*>(&sh.sfb[kTcDigits * j][0])[piece] = v;
        }
      }
      tc_proxy_fence();   // the digit rows are read by the tensor core
      gt_worker_sync();
      t_1 = clock64();
      if (scale_warp) tc_upload_scales(tmem, sub, &sh.sfb[0][0], kGtMaxK / 16, kGtN, K / 64, lane);
      gt_worker_sync();
      t_2 = clock64();
      if (wt == 0) {
        __threadfence_block();
        sh.staged = ++stagings;
      }
      }   // fresh
      if (scale_warp) {
        // ---- weight scales of every unit: shared -> tensor memory (lane = row % 32, column = row / 32)
        for (int c = 0; c < chunks; ++c, ++seq) {
          const int u = (int)(seq % kGtUnits), sfs = (int)(seq % kTcSfSlots);
          bool ok = gt_wait(&sh.full[u], (uint32_t)(seq / kGtUnits) & 1u, &sh);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) continue;
          const unsigned char* sc = units + (size_t)u * kTcUnitBytes + kTcCodeBytes;
          const uint4 r0 = *reinterpret_cast<const uint4*>(sc + lane * 16);
          const uint4 r1 = *reinterpret_cast<const uint4*>(sc + (lane + 32) * 16);
          const uint4 r2 = *reinterpret_cast<const uint4*>(sc + (lane + 64) * 16);
          const uint4 r3 = *reinterpret_cast<const uint4*>(sc + (lane + 96) * 16);
          ok = gt_wait(&sh.sf_empty[sfs], (uint32_t)((seq / kTcSfSlots) & 1) ^ 1u, &sh);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) continue;
          tc_fence_after();
          const uint32_t w[16] = {r0.x, r1.x, r2.x, r3.x, r0.y, r1.y, r2.y, r3.y, r0.z, r1.z, r2.z, r3.z, r0.w, r1.w, r2.w, r3.w};
          tc_st16(tmem + lane_base + kTcColSfa + sfs * 16, w);
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh.sf_full[sfs]);
        }
      } else {
        // ---- the tile's accumulator: row = tensor-memory lane, four digit columns per route
        const int dbuf = item_count & 1;
        bool ok = gt_wait(&sh.d_full[dbuf], (uint32_t)((item_count >> 1) & 1), &sh);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
          tc_fence_after();
          float v[kGtN];
          tc_ld32(tmem + lane_base + kTcColD + dbuf * kGtN, v);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh.d_empty[dbuf]);
          const int r = it.tile * kTcRows + sub * 32 + lane;
#pragma unroll
          for (int j = 0; j < kGtBatch; ++j) {
            const int route = sh.route[j];
            const float mine = ((v[4 * j] + v[4 * j + 1]) + (v[4 * j + 2] + v[4 * j + 3])) * sh.out_scale[j];
            if (PROJ == 0) {
              const float up = __shfl_xor_sync(0xffffffffu, mine, 1);   // even rows are gate, odd rows up
              if (route >= 0 && (lane & 1) == 0)
                a.Y[(size_t)route * (a.n / 2) + (r >> 1)] = (uint16_t)f32_to_bf16_bits(mine / (1.f + __expf(-mine)) * up);
            } else {
              if (route >= 0) a.Y[(size_t)route * a.n + r] = (uint16_t)f32_to_bf16_bits(mine);
            }
          }
        }
      }
      // before the next batch is staged every MMA of this one must be done: the accumulator warps have seen the last
      // tile's accumulator complete, which the tensor core signals only after all earlier MMAs
      if (last_of_batch) gt_worker_sync();
      t_stage += t_1 - t_0;
      t_upload += t_2 - t_1;
      t_main += clock64() - t_2;
    }
    if (a.prof && wt == 0) {
      a.prof[blockIdx.x * 8 + 0] = t_stage;
      a.prof[blockIdx.x * 8 + 1] = t_upload;
      a.prof[blockIdx.x * 8 + 2] = t_main;
      a.prof[blockIdx.x * 8 + 3] = clock64() - t_begin;
      a.prof[blockIdx.x * 8 + 6] = item_count;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tc_dealloc(tmem, 512);
  if (threadIdx.x == 0 && sh.failed && a.status) atomicOr(a.status, kFlagWaitTimedOut);
}

// One block per row of X: its power-of-two normaliser, its four E2M1 digit rows as 512-byte pieces of the swizzled
// operand (per 256-column chunk, once for an even and once for an odd slot of a batch), and their block scales.
__global__ void __launch_bounds__(256) digit_rows_kernel(const uint16_t* __restrict__ X, int k, float2* row_scale,
                                                         unsigned char* digits, unsigned char* digit_scales) {
  extern __shared__ __align__(1024) unsigned char image[];   // [k/256][8 rows][128 B]: rows 0..3 even slot, 4..7 odd slot
  __shared__ __align__(16) uint8_t sf[8][kGtMaxK / 16];
  __shared__ uint32_t s_amax[8];
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint4* x = reinterpret_cast<const uint4*>(X + (size_t)row * k);
  uint32_t amax = 0;
  for (int g = threadIdx.x; g < k / 8; g += 256) {
    const uint4 v = x[g];
    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = max(amax, max(w4[j] & 0x7fffu, (w4[j] >> 16) & 0x7fffu));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) s_amax[warp] = amax;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < 8; ++w) amax = max(amax, s_amax[w]);
  float inverse;
  const float scale = pow2_normaliser(amax, &inverse);
  if (threadIdx.x == 0) row_scale[row] = make_float2(scale, inverse);
  for (int g = threadIdx.x; g < k / 8; g += 256) {   // (k / 8 is a multiple of 32: whole warps stay in the call)
    const uint4 v = x[g];
    tc_stage8(v, 512.f * scale, image, 8, 0, g * 8, &sf[0][0], kGtMaxK / 16);
    tc_stage8(v, 512.f * scale, image, 8, 4, g * 8, &sf[0][0], kGtMaxK / 16);
  }
  __syncthreads();
  uint4* out = reinterpret_cast<uint4*>(digits + (size_t)row * k * 4);
  for (int i = threadIdx.x; i < k * 4 / 16; i += 256) out[i] = reinterpret_cast<const uint4*>(image)[i];
  uint4* out_sf = reinterpret_cast<uint4*>(digit_scales + (size_t)row * kTcDigits * (kGtMaxK / 16));
  for (int i = threadIdx.x; i < kTcDigits * (kGtMaxK / 16) / 16; i += 256) out_sf[i] = reinterpret_cast<const uint4*>(&sf[0][0])[i];
}

}  // namespace ink

using namespace ink;

static size_t gt_pad256(size_t n) { return (n + 255) / 256 * 256; }
// row scales, digit-row pieces (4 k bytes per row) and their block scales (4 x 256 bytes per row)
extern "C" size_t ink_expert_gemm_tc_scratch_bytes(int input_rows, int k) {
  const size_t rows = input_rows > 0 ? (size_t)input_rows : 0;
  return gt_pad256(sizeof(float2) * rows) + gt_pad256(rows * (size_t)k * 4) + gt_pad256(rows * kTcDigits * (kGtMaxK / 16)) +
         8 * 8 * 256;   // (+ the optional per-block phase clocks)
}

extern "C" int ink_expert_gemm_tc(const void* x, int input_rows, const void* bank_maps, const int64_t* pointers,
                                  const int32_t* experts, const int32_t* rows, const int32_t* counts, void* y, int capacity,
                                  int n, int k, int top_k, int projection, int groups, int start, void* scratch,
                                  size_t scratch_bytes, int32_t* status, ink_stream_t stream) {
  INK_REQUIRE(x && bank_maps && pointers && experts && rows && counts && y && scratch, kBadArgument,
              "expert_gemm_tc: null pointer argument");
  INK_REQUIRE(projection == 0 || projection == 1, kBadArgument, "expert_gemm_tc: projection=%d", projection);
  INK_REQUIRE(k % kTcChunkK == 0 && k >= kTcChunkK && k <= kGtMaxK && n % kTcRows == 0 && n > 0, kUnsupportedShape,
              "expert_gemm_tc: n=%d k=%d unsupported (n a multiple of %d, k a multiple of %d up to %d)", n, k, kTcRows,
              kTcChunkK, kGtMaxK);
  INK_REQUIRE(groups >= 0 && groups <= kGtMaxGroups && capacity >= 1 && top_k >= 1 && input_rows >= 0 && start >= 0, kBadArgument,
              "expert_gemm_tc: bad sizes (groups=%d, at most %d)", groups, kGtMaxGroups);
  INK_REQUIRE(scratch_bytes >= ink_expert_gemm_tc_scratch_bytes(input_rows, k), kBadArgument,
              "expert_gemm_tc: scratch of %zu bytes, %zu needed", scratch_bytes, ink_expert_gemm_tc_scratch_bytes(input_rows, k));
  INK_REQUIRE(aligned16(x) && aligned16(y) && aligned16(scratch) && (reinterpret_cast<uintptr_t>(bank_maps) & 127u) == 0,
              kMisaligned, "expert_gemm_tc: misaligned buffer (the descriptors need 128-byte alignment)");
  if (groups == 0 || input_rows == 0) return kOk;
  cudaStream_t s = (cudaStream_t)stream;
  unsigned char* digits = (unsigned char*)scratch + gt_pad256(sizeof(float2) * (size_t)input_rows);
  unsigned char* digit_scales = digits + gt_pad256((size_t)input_rows * k * 4);
  digit_rows_kernel<<<input_rows, 256, (size_t)k * 4, s>>>((const uint16_t*)x, k, (float2*)scratch, digits, digit_scales);
  INK_CHECK_LAUNCH("expert_gemm_tc (digit rows)");
  GemmTcArgs a;
  a.X = (const uint16_t*)x;
  a.maps = (const unsigned char*)bank_maps;
  a.pointers = pointers;
  a.experts = experts;
  a.rows = rows;
  a.counts = counts;
  a.Y = (uint16_t*)y;
  a.row_scale = (const float2*)scratch;
  a.digits = digits;
  a.digit_scales = digit_scales;
  a.capacity = capacity;
  a.n = n;
  a.k = k;
  a.top_k = top_k;
  a.groups = groups;
  a.start = start;
  a.status = status;
  a.prof = nullptr;
  {
    // INKLING_GROUPED_PROFILE=1: the tail of the scratch (8 x 8 bytes per block after the row scales) gets per-phase clock totals
    const char* on = getenv("INKLING_GROUPED_PROFILE");
    if (on && on[0] == '1') a.prof = (long long*)((char*)scratch + ink_expert_gemm_tc_scratch_bytes(input_rows, k) - 8 * 8 * 256);
  }
  const size_t smem = (size_t)kGtUnits * kTcUnitBytes + (size_t)k * 16 + 1024;
  constexpr int kMaxDevices = 64;
  static int sms_of[2][kMaxDevices] = {};
  int device = 0;
  cudaGetDevice(&device);
  INK_REQUIRE(device >= 0 && device < kMaxDevices, kLaunchFailed, "expert_gemm_tc: device ordinal %d", device);
  if (sms_of[projection][device] == 0) {
    const size_t most = (size_t)kGtUnits * kTcUnitBytes + (size_t)kGtMaxK * 16 + 1024;
    cudaError_t e = projection == 0
                        ? cudaFuncSetAttribute(expert_gemm_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most)
                        : cudaFuncSetAttribute(expert_gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "expert_gemm_tc: %zu bytes of shared memory refused: %s", most, cudaGetErrorString(e));
    int count = 0;
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    INK_REQUIRE(count >= 1, kLaunchFailed, "expert_gemm_tc: no multiprocessors reported");
    sms_of[projection][device] = count;
  }
  const int blocks = sms_of[projection][device];
  if (projection == 0) expert_gemm_tc_kernel<0><<<blocks, kGtThreads, smem, s>>>(a);
  else expert_gemm_tc_kernel<1><<<blocks, kGtThreads, smem, s>>>(a);
  INK_CHECK_LAUNCH("expert_gemm_tc");
  return kOk;
}

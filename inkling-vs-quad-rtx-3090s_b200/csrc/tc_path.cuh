// NVFP4 weights on the tcgen05 tensor cores without converting them: the packed E2M1
// codes are the M = 128 operand of tcgen05.mma.kind::mxf4nvf4.block_scale straight from
// their checkpoint layout (tiled TMA, 128-byte swizzle), their E4M3 block scales go to
// tensor memory with tcgen05.st, and the BF16 activations become the N operand as four
// E2M1 "digit" rows per vector with power-of-two E4M3 block scales:
//     x[i] * 2^g  ~=  sum_t digit_t[i] * 2^(e_block - 3 t),   digit_t in {-4..4},
// exact to 2^-9 of four times the block's power-of-two scale. The MMA applies both scale
// sets and accumulates the four digit rows in FP32; the caller adds the four columns.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "pipe.cuh"

namespace ink {

constexpr int kTcRows = 128;                 // weight rows per tile (MMA M)
constexpr int kTcChunkK = 256;               // K elements per unit: one 128-byte swizzle row
constexpr int kTcCodeBytes = kTcRows * kTcChunkK / 2;    // 16384
constexpr int kTcScaleBytes = kTcRows * kTcChunkK / 16;  // 2048
constexpr int kTcUnitBytes = kTcCodeBytes + kTcScaleBytes;
constexpr int kTcSfSlots = 8;                // units whose weight scales sit in tensor memory
// tensor memory columns (512 allocated): two accumulators, the weight-scale ring, the activation scales
constexpr int kTcColD = 0, kTcColSfa = 64, kTcColSfb = 256;
constexpr int kTcDigits = 4;

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_alloc(uint32_t* dst_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart; the
// tile starts on a 1024-byte boundary and a K step of 64 elements advances the start by 32 bytes
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// E2M1 x E2M1, UE4M3 scales per 16 elements, FP32 accumulate, M = 128
__host__ __device__ constexpr uint32_t tc_idesc(int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t ad, uint64_t bd, uint32_t idesc, uint32_t accumulate, uint32_t sfa,
                                       uint32_t sfb) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(d),
      "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// 3-D tiled load: {byte in row, row, expert}
__device__ __forceinline__ void tc_tma_3d(void* dst, const void* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
// this warp's 32 lanes x 16 columns
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_ld4(uint32_t taddr, float (&v)[4]) {
  uint32_t r[4];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, "
      "%19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 2^p as an E4M3 byte, -9 <= p <= 8 (the three lowest are subnormals)
__device__ __forceinline__ uint32_t tc_e4m3_pow2(int p) { return p >= -6 ? (uint32_t)(p + 7) << 3 : (uint32_t)(4 >> (-7 - p)); }
// Eight consecutive elements k0 .. k0+7 (k0 a multiple of 8) of a BF16 vector whose largest
// magnitude `scale` brings into [512, 1024): their digit codes go to rows row0 .. row0+3 of a
// [K/256][rows][128 B] swizzled N operand, one 32-bit store per row, and the block's four scale
// bytes to sf[(row0 + t) * sf_pitch + k0 / 16]. A 16-element block is two such groups held by
// the lanes 2m and 2m+1 of a warp (the caller deals consecutive groups to consecutive lanes and
// keeps the whole warp in the call). Per element: q = round(v * 2^(9-e)) lies in [-2048, 2048];
// adding 4 * (512 + 64 + 8 + 1) turns its balanced base-8 digits (-4..3, the leading one up to 4)
// into plain ones, which index a table of E2M1 codes.
__device__ __forceinline__ void tc_stage8(uint4 raw, float scale, unsigned char* operand, int rows, int row0, int k0, uint8_t* sf,
                                          int sf_pitch) {
  const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(in[i] << 16) * scale;
    v[2 * i + 1] = __uint_as_float(in[i] & 0xffff0000u) * scale;
    m = fmaxf(m, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
  }
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  int e = (int)((__float_as_uint(m) >> 23) & 0xffu) - 128;   // floor(log2 of the block's largest magnitude) - 1
  e = e < 0 ? 0 : (e > 8 ? 8 : e);
  const float mult = __uint_as_float((uint32_t)(127 + 9 - e) << 23);
  constexpr uint32_t kCodes = 0x5420ACDEu;   // E2M1 codes of -4, -3, -2, -1, 0, 1, 2, 3
  uint32_t w0 = 0, w1 = 0, w2 = 0, w3 = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int q = __float2int_rn(v[i] * mult);
    q = q > 2048 ? 2048 : (q < -2048 ? -2048 : q);
    const uint32_t u = (uint32_t)(q + 2340);
    const uint32_t lead = u >> 9;   // 0..8
    w0 |= (lead == 8u ? 6u : (kCodes >> (4u * lead)) & 15u) << (4 * i);
    w1 |= ((kCodes >> (4u * ((u >> 6) & 7u))) & 15u) << (4 * i);
    w2 |= ((kCodes >> (4u * ((u >> 3) & 7u))) & 15u) << (4 * i);
    w3 |= ((kCodes >> (4u * (u & 7u))) & 15u) << (4 * i);
  }
  const int chunk = k0 >> 8, in256 = k0 & 255, unit = in256 >> 5, byte = (in256 & 31) >> 1;
  unsigned char* at = operand + (size_t)chunk * rows * 128 + byte;
  *reinterpret_cast<uint32_t*>(at + (row0 + 0) * 128 + ((unit ^ ((row0 + 0) & 7)) << 4)) = w0;
  *reinterpret_cast<uint32_t*>(at + (row0 + 1) * 128 + ((unit ^ ((row0 + 1) & 7)) << 4)) = w1;
  *reinterpret_cast<uint32_t*>(at + (row0 + 2) * 128 + ((unit ^ ((row0 + 2) & 7)) << 4)) = w2;
  *reinterpret_cast<uint32_t*>(at + (row0 + 3) * 128 + ((unit ^ ((row0 + 3) & 7)) << 4)) = w3;
  if ((k0 & 8) == 0) {
#pragma unroll
    for (int t = 0; t < kTcDigits; ++t) sf[(row0 + t) * sf_pitch + (k0 >> 4)] = (uint8_t)tc_e4m3_pow2(e - 3 * t);
  }
}

// Block scales of `rows` digit rows (`bytes_per_row` each, row r at table + r * pitch) into the
// activation-scale columns of tensor memory, 4 columns per 64-element step. Four warps, one per
// tensor-memory subpartition, write the same words.
__device__ __forceinline__ void tc_upload_scales(uint32_t tmem, int subpartition, const uint8_t* table, int pitch, int rows, int steps,
                                                 int lane) {
  const uint32_t base = tmem + ((uint32_t)(subpartition * 32) << 16) + kTcColSfb;
#pragma unroll 1
  for (int s0 = 0; s0 < steps; s0 += 4) {
    uint32_t r[16];
#pragma unroll
    for (int j = 0; j < 16; ++j)
      r[j] = ((j & 3) == 0 && lane < rows) ? *reinterpret_cast<const uint32_t*>(table + (size_t)lane * pitch + (s0 + (j >> 2)) * 4) : 0u;
    tc_st16(base + s0 * 4, r);
  }
  tc_wait_st();
  tc_fence_before();
}

// owner of item x when `total` items are dealt to `parts` blocks as [total*b/parts, total*(b+1)/parts)
__device__ __forceinline__ int tc_owner(long long x, long long total, long long parts) { return (int)(((x + 1) * parts - 1) / total); }

}  // namespace ink

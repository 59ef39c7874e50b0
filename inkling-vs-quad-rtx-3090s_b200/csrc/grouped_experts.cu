// Grouped expert projections for more than a handful of tokens: one 128-row weight tile
// of one active expert against all tokens routed to that expert, on the tcgen05 tensor
// cores. NVFP4 codes stream from HBM through a small bulk-copy ring, are expanded in
// shared memory to FP16 (E2M1 value x E4M3 block scale is exact in FP16) in the K-major
// core-matrix layout the MMA reads, the tokens' activations are gathered next to them,
// and tcgen05.mma (kind::f16, M = 128, N = tokens, FP32 accumulators in tensor memory)
// does the contraction. The per-bank FP32 scale and the activations' power-of-two
// normaliser are applied to the accumulator in the epilogue, which also fuses SwiGLU
// for the gate/up projection.
#include "../../include/inkling_b200.h"
#include "common.cuh"
#include "decode_args.cuh"
#include "pipe.cuh"

namespace ink {

constexpr int kGM = 128;        // weight rows per tile (MMA M)
constexpr int kGN = 128;        // tokens per pass (MMA N, padded to a multiple of 16)
constexpr int kGKC = 128;       // K elements per chunk
constexpr int kGThreads = 256;
constexpr int kGRaw = 4;        // raw-code stages in flight
constexpr int kGRawBytes = kGM * kGKC / 2;   // 8192

struct GemmArgs {
  const uint16_t* X;            // BF16 [*, K]
  const int64_t* pointers;      // [(max_expert + 1) * 6]
  const int32_t* experts;       // [groups] expert of each active group, -1 after
  const int32_t* rows;          // [groups, capacity] routes of each group
  const int32_t* counts;        // [groups]
  uint16_t* Y;                  // BF16 [capacity, n or n / 2]
  const float2* row_scale;      // per row of X: {power-of-two multiplier, its inverse}
  int capacity, n, k, top_k, projection;
  int32_t* status;
};

// ---- tcgen05 plumbing ---------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// K-major operand without swizzle: 8-row x 16-byte core matrices, rows 16 bytes apart,
// 8-row groups `sbo` bytes apart, the two 16-byte K slabs of one MMA `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version of this architecture
  return d;
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// this warp's 32 lanes x 16 consecutive FP32 columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- per-row power-of-two normaliser of the activations -----------------------------
__global__ void __launch_bounds__(256) row_scale_kernel(const uint16_t* __restrict__ X, int rows, int k, float2* out) {
  const int lane = threadIdx.x & 31, row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint32_t* p = reinterpret_cast<const uint32_t*>(X + (size_t)row * k);
  uint32_t amax = 0;
  for (int i = lane; i < k / 2; i += 32) {
    const uint32_t v = p[i];
    amax = max(amax, max(v & 0x7fffu, (v >> 16) & 0x7fffu));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) {
    float inverse;
    const float scale = pow2_normaliser(amax, &inverse);
    out[row] = make_float2(scale, inverse);
  }
}

// ---- the grouped GEMM -----------------------------------------------------------------
struct GemmShared {
  uint64_t raw_full[kGRaw];
  uint64_t mma_done;
  uint32_t tmem_base;
  int failed;
};

template <int PROJ>
__global__ void __launch_bounds__(kGThreads, 1) expert_gemm_kernel(GemmArgs a) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ GemmShared sh;
  __shared__ int s_route[kGN];
  __shared__ float s_out_scale[kGN];
  const int tid = threadIdx.x, warp = tid >> 5;
  const int group = blockIdx.y, m0 = blockIdx.x * kGM;
  const int count = a.counts[group];
  if (count <= 0) return;
  const int expert = a.experts[group];
  if (expert < 0) return;
  const int64_t* entry = a.pointers + (size_t)expert * kBank + (PROJ ? 3 : 0);
  const uint8_t* W = reinterpret_cast<const uint8_t*>(entry[0]);
  if (W == nullptr) return;
  const uint8_t* S = reinterpret_cast<const uint8_t*>(entry[1]);
  const float scale2 = *reinterpret_cast<const float*>(entry[2]);
  const int K = a.k, n_chunks = K / kGKC, srow = K / 16;

  unsigned char* s_a = smem;                                  // [16 slabs][128 rows][16 B]   32 KB
  unsigned char* s_b = s_a + kGM * kGKC * 2;                  // [16 slabs][Npad rows][16 B] <= 32 KB
  unsigned char* s_raw = s_b + kGN * kGKC * 2;                // kGRaw x 8 KB
  unsigned char* s_scales = s_raw + kGRaw * kGRawBytes;       // [128][K / 16]

  if (tid == 0) {
    for (int s = 0; s < kGRaw; ++s) mbar_init(&sh.raw_full[s], 1);
    mbar_init(&sh.mma_done, 1);
    sh.failed = 0;
    mbar_init_fence();
  }
  __syncthreads();
  if (warp == 0) tmem_alloc(&sh.tmem_base, kGN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_base;

  // block scales of the whole tile (row-major, K/16 bytes per row); ordinary loads
  for (int i = tid; i < kGM * srow / 4; i += kGThreads) {
    const int r = i / (srow / 4), c = i % (srow / 4);
    reinterpret_cast<uint32_t*>(s_scales)[i] =
        m0 + r < a.n ? *reinterpret_cast<const uint32_t*>(S + (size_t)(m0 + r) * srow + c * 4) : 0u;
  }

  uint32_t raw_parity = 0, mma_phase = 0;   // raw_parity: bit s = parity the next wait on stage s uses
  auto issue_raw = [&](int chunk) {
    // one 64-byte copy per weight row, all onto the stage's barrier
    const int stage = chunk % kGRaw;
    if (tid == 0) mbar_expect_tx(&sh.raw_full[stage], kGRawBytes);
    if (tid < kGM) {
      const int row = m0 + tid < a.n ? m0 + tid : a.n - 1;   // rows past the end repeat the last one, never stored
      bulk_g2s(s_raw + stage * kGRawBytes + tid * (kGKC / 2), W + (size_t)row * (K / 2) + (size_t)chunk * (kGKC / 2),
               kGKC / 2, &sh.raw_full[stage]);
    }
  };

  for (int n0 = 0; n0 < count; n0 += kGN) {
    const int n_here = min(kGN, count - n0);
    const int n_pad = (n_here + 15) / 16 * 16;
    __syncthreads();
    for (int n = tid; n < kGN; n += kGThreads) {
      int route = -1;
      float out_scale = 0.f;
      if (n < n_here) {
        route = a.rows[(size_t)group * a.capacity + n0 + n];
        const int in_row = PROJ == 0 ? route / a.top_k : route;
        out_scale = scale2 * a.row_scale[in_row].y;
      }
      s_route[n] = route;
      s_out_scale[n] = out_scale;
    }
    __syncthreads();
    const uint32_t idesc = (1u << 4) | ((uint32_t)(n_pad >> 3) << 17) | ((uint32_t)(kGM >> 4) << 24);
    for (int c = 0; c < kGRaw && c < n_chunks; ++c) issue_raw(c);

    for (int chunk = 0; chunk < n_chunks; ++chunk) {
      const int stage = chunk % kGRaw;
      bool ok = !sh.failed && mbar_wait(&sh.raw_full[stage], (raw_parity >> stage) & 1);
      raw_parity ^= 1u << stage;
      if (ok && (chunk > 0 || n0 > 0)) {
        ok = mbar_wait(&sh.mma_done, (mma_phase - 1) & 1);   // operands of the previous MMAs are free
      }
      if (!ok) sh.failed = 1;
      if (ok) {
        // ---- expand 128 rows x 128 codes to FP16 core matrices
        {
          const int r = tid >> 1, h = tid & 1;
          const uint4* src = reinterpret_cast<const uint4*>(s_raw + stage * kGRawBytes + r * (kGKC / 2) + h * 32);
          const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(s_scales + r * srow + chunk * (kGKC / 16) + h * 4);
          const uint32_t s01 = e4m3x2_to_f16x2((uint16_t)(sc4 & 0xffffu)), s23 = e4m3x2_to_f16x2((uint16_t)(sc4 >> 16));
          const uint32_t block_scale[4] = {__byte_perm(s01, 0, 0x1010), __byte_perm(s01, 0, 0x3232),
                                           __byte_perm(s23, 0, 0x1010), __byte_perm(s23, 0, 0x3232)};
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const uint4 codes = src[q];
            const uint32_t w4[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t hv[4];
              e2m1x8_to_f16x2(w4[j], hv);
              const uint32_t bs = block_scale[q * 2 + j / 2];
              const uint4 out = make_uint4(hmul2(hv[0], bs), hmul2(hv[1], bs), hmul2(hv[2], bs), hmul2(hv[3], bs));
              const int slab = h * 8 + q * 4 + j;
              *reinterpret_cast<uint4*>(s_a + slab * (kGM * 16) + r * 16) = out;
            }
          }
        }
        // ---- gather the tokens' activations for this K chunk
        for (int p = tid; p < n_pad * (kGKC / 8); p += kGThreads) {
          const int n = p % n_pad, slab = p / n_pad;
          uint4 out = make_uint4(0, 0, 0, 0);
          const int route = n < n_here ? s_route[n] : -1;
          if (route >= 0) {
            const int in_row = PROJ == 0 ? route / a.top_k : route;
            const float scale = a.row_scale[in_row].x;
            const uint4 v = *reinterpret_cast<const uint4*>(a.X + (size_t)in_row * K + (size_t)chunk * kGKC + slab * 8);
            out.x = f32x2_to_f16x2(bf16lo(v.x) * scale, bf16hi(v.x) * scale);
            out.y = f32x2_to_f16x2(bf16lo(v.y) * scale, bf16hi(v.y) * scale);
            out.z = f32x2_to_f16x2(bf16lo(v.z) * scale, bf16hi(v.z) * scale);
            out.w = f32x2_to_f16x2(bf16lo(v.w) * scale, bf16hi(v.w) * scale);
          }
          *reinterpret_cast<uint4*>(s_b + slab * (n_pad * 16) + n * 16) = out;
        }
        proxy_fence_async();   // generic-proxy writes above must be visible to the tensor core's reads
      }
      tc_fence_before();
      __syncthreads();
      if (sh.failed) break;
      if (tid == 0) {
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kGKC / 16; ++kk) {
          const uint64_t da = umma_desc(smem_u32(s_a) + kk * 2 * (kGM * 16), kGM * 16, 128);
          const uint64_t db = umma_desc(smem_u32(s_b) + kk * 2 * (n_pad * 16), n_pad * 16, 128);
          umma_f16(tmem, da, db, idesc, chunk > 0 || kk > 0);
        }
        tc_commit(&sh.mma_done);
      }
      ++mma_phase;
      if (chunk + kGRaw < n_chunks) issue_raw(chunk + kGRaw);
    }
    if (sh.failed) break;
    // ---- epilogue: row r of the tile sits in tensor-memory lane r
    if (!mbar_wait(&sh.mma_done, (mma_phase - 1) & 1)) sh.failed = 1;
    tc_fence_after();
    if (warp < 4 && !sh.failed) {
      const int r = tid;   // 0..127
      const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
      for (int c0 = 0; c0 < n_pad; c0 += 16) {
        float v[16];
        tmem_ld16(lane_base + c0, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int n = c0 + j;
          const float mine = v[j] * s_out_scale[n < kGN ? n : 0];
          if (PROJ == 0) {
            const float other = __shfl_down_sync(0xffffffffu, mine, 1);   // odd row = up
            if ((r & 1) == 0 && n < n_here && m0 + r + 1 < a.n)
              a.Y[(size_t)s_route[n] * (a.n / 2) + (m0 + r) / 2] = (uint16_t)f32_to_bf16_bits(mine / (1.f + __expf(-mine)) * other);
          } else {
            if (n < n_here && m0 + r < a.n) a.Y[(size_t)s_route[n] * a.n + m0 + r] = (uint16_t)f32_to_bf16_bits(mine);
          }
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kGN);
  if (tid == 0 && sh.failed && a.status) atomicOr(a.status, kFlagWaitTimedOut);
}

// ---- weighted sum of the routes' down rows per token (kernels/grouped_experts.py:152-186)
__global__ void __launch_bounds__(256) expert_reduce_kernel(const uint16_t* __restrict__ down,
                                                             const int64_t* __restrict__ indices,
                                                             const uint16_t* __restrict__ weights,
                                                             const int64_t* __restrict__ pointers, float* output,
                                                             int width, int top_k, int stride, int max_expert) {
  const int token = blockIdx.x;
  const int col = blockIdx.y * blockDim.x + threadIdx.x;
  if (col >= width) return;
  float acc = 0.f;
  for (int choice = 0; choice < top_k; ++choice) {
    const int route = token * top_k + choice;
    const int64_t expert = indices[route];
    const bool active = expert >= 0 && expert <= max_expert && pointers[expert * stride] != 0;
    const float value = active ? bf16_to_f32(down[(size_t)route * width + col]) : 0.f;
    acc += round_bf16(value * bf16_to_f32(weights[route]));
  }
  output[(size_t)token * width + col] += acc;
}

}  // namespace ink

using namespace ink;

extern "C" size_t ink_expert_gemm_scratch_bytes(int input_rows) { return sizeof(float2) * (size_t)(input_rows > 0 ? input_rows : 0); }

extern "C" int ink_expert_gemm(const void* x, int input_rows, const int64_t* pointers, const int32_t* experts,
                               const int32_t* rows, const int32_t* counts, void* y, int capacity, int n, int k,
                               int top_k, int projection, int quantized, int groups, void* scratch,
                               size_t scratch_bytes, int32_t* status, ink_stream_t stream) {
  INK_REQUIRE(quantized == 1, kUnsupportedShape, "expert_gemm: only NVFP4 banks (quantized=1) are built");
  INK_REQUIRE(x && pointers && experts && rows && counts && y && scratch, kBadArgument, "expert_gemm: null pointer argument");
  INK_REQUIRE(projection == 0 || projection == 1, kBadArgument, "expert_gemm: projection=%d", projection);
  INK_REQUIRE(k % kGKC == 0 && k >= kGKC && k <= 8192 && n % 2 == 0 && n > 0 && (k / 16) % 4 == 0, kUnsupportedShape,
              "expert_gemm: n=%d k=%d unsupported (k a multiple of %d up to 8192)", n, k, kGKC);
  INK_REQUIRE(groups >= 0 && capacity >= 1 && top_k >= 1 && input_rows >= 0, kBadArgument, "expert_gemm: bad sizes");
  INK_REQUIRE(scratch_bytes >= ink_expert_gemm_scratch_bytes(input_rows), kBadArgument, "expert_gemm: scratch too small");
  INK_REQUIRE(aligned16(x) && aligned16(y) && aligned16(scratch), kMisaligned, "expert_gemm: misaligned buffer");
  if (groups == 0 || input_rows == 0) return kOk;
  cudaStream_t s = (cudaStream_t)stream;
  INK_PREFER_MAX_SMEM(row_scale_kernel);
  row_scale_kernel<<<(input_rows + 7) / 8, 256, 0, s>>>((const uint16_t*)x, input_rows, k, (float2*)scratch);
  INK_CHECK_LAUNCH("expert_gemm (row scales)");
  GemmArgs a;
  a.X = (const uint16_t*)x;
  a.pointers = pointers;
  a.experts = experts;
  a.rows = rows;
  a.counts = counts;
  a.Y = (uint16_t*)y;
  a.row_scale = (const float2*)scratch;
  a.capacity = capacity;
  a.n = n;
  a.k = k;
  a.top_k = top_k;
  a.projection = projection;
  a.status = status;
  const size_t smem = (size_t)kGM * kGKC * 2 + (size_t)kGN * kGKC * 2 + (size_t)kGRaw * kGRawBytes + (size_t)kGM * (k / 16);
  static size_t configured[2] = {0, 0};
  if (smem > configured[projection]) {
    cudaError_t e = projection == 0
                        ? cudaFuncSetAttribute(expert_gemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                        : cudaFuncSetAttribute(expert_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    INK_REQUIRE(e == cudaSuccess, kLaunchFailed, "expert_gemm: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    configured[projection] = smem;
  }
  const dim3 grid((n + kGM - 1) / kGM, groups);
  if (projection == 0) {
    INK_PREFER_MAX_SMEM(expert_gemm_kernel<0>);
    expert_gemm_kernel<0><<<grid, kGThreads, smem, s>>>(a);
  } else {
    INK_PREFER_MAX_SMEM(expert_gemm_kernel<1>);
    expert_gemm_kernel<1><<<grid, kGThreads, smem, s>>>(a);
  }
  INK_CHECK_LAUNCH("expert_gemm");
  return kOk;
}

extern "C" int ink_expert_reduce(const void* down, const int64_t* indices, const void* weights, const int64_t* pointers,
                                 float* output, int tokens, int width, int top_k, int pointer_stride, int max_expert,
                                 ink_stream_t stream) {
  INK_REQUIRE(down && indices && weights && pointers && output, kBadArgument, "expert_reduce: null pointer argument");
  INK_REQUIRE(tokens >= 0 && width > 0 && top_k >= 1 && pointer_stride >= 1, kBadArgument, "expert_reduce: bad sizes");
  if (tokens == 0) return kOk;
  INK_PREFER_MAX_SMEM(expert_reduce_kernel);
  expert_reduce_kernel<<<dim3(tokens, (width + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint16_t*)down, indices, (const uint16_t*)weights, pointers, output, width, top_k, pointer_stride, max_expert);
  INK_CHECK_LAUNCH("expert_reduce");
  return kOk;
}

// Execution shim that lets the reference's CUDA C file kernels/routed_decode.cu be
// compiled by g++ and run on the CPU, unmodified and from where it lies, so that its
// outputs can pin the oracle. Test infrastructure only.
//
// One CUDA thread = one OS thread; one block runs at a time, so function-local
// `static` storage stands in for __shared__. __syncthreads is a block-wide barrier and
// __shfl_xor_sync an exchange through a per-block slot array bracketed by two barriers
// (valid because every thread of a block executes the same sequence of shuffles in
// this file).
#pragma once
#include <barrier>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

// the .cu file typedefs these itself; keep them apart from <cstdint>'s
#define uint8_t ref_u8
#define uint16_t ref_u16
#define uint32_t ref_u32
#define int64_t ref_i64

#define __global__
#define __device__
#define __forceinline__ inline
#define __restrict__
#define __shared__ static

struct ref_dim3 { int x, y, z; };
struct uint4 { unsigned x, y, z, w; };
static thread_local ref_dim3 threadIdx, blockIdx;
static std::barrier<>* ref_block_barrier = nullptr;
static float ref_slots[1024];

static inline void __syncthreads() { ref_block_barrier->arrive_and_wait(); }
static inline float __shfl_xor_sync(unsigned, float value, int offset) {
  ref_slots[threadIdx.x] = value;
  ref_block_barrier->arrive_and_wait();
  const float other = ref_slots[threadIdx.x ^ offset];
  ref_block_barrier->arrive_and_wait();
  return other;
}
static inline float __uint_as_float(unsigned bits) { float f; std::memcpy(&f, &bits, 4); return f; }
static inline unsigned __float_as_uint(float f) { unsigned b; std::memcpy(&b, &f, 4); return b; }

template <class Body>
static void ref_launch(int grid_x, int grid_y, int threads, Body body) {
  for (int by = 0; by < grid_y; ++by)
    for (int bx = 0; bx < grid_x; ++bx) {
      std::barrier<> barrier(threads);
      ref_block_barrier = &barrier;
      std::vector<std::thread> pool;
      pool.reserve(threads);
      for (int t = 0; t < threads; ++t)
        pool.emplace_back([=] {
          threadIdx = {t, 0, 0};
          blockIdx = {bx, by, 0};
          body();
        });
      for (auto& th : pool) th.join();
    }
}

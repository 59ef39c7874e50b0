// Host launcher around the reference's kernels/routed_decode.cu compiled for the CPU
// (see ref_cpu_shim.h). Built once per (K, QUANT) by oracle/build_ref.py with
//   g++ -std=c++20 -O1 -DK=<width> -DQUANT=<0|1> -DREF_CU='"<path>/kernels/routed_decode.cu"'
// The grids are the ones kernels/routed_decode.py:56-80 launches.
#include "ref_cpu_shim.h"
#include REF_CU

extern "C" void ref_launch_gate_up(const void* X, const void* indices, const void* pointers, void* Y,
                                   int top_k, int max_expert, int N, int rows, int routes) {
  ref_launch(N / rows, routes, THREADS, [=] {
    gate_up((const uint16_t*)X, (const int64_t*)indices, (const int64_t*)pointers, (uint16_t*)Y,
            top_k, max_expert, N, rows);
  });
}

extern "C" void ref_launch_down_reduce(const void* A, const void* indices, const void* weights,
                                       const void* pointers, void* out, int top_k, int max_expert,
                                       int N, int rows, int tokens) {
  ref_launch(N / rows, tokens, THREADS, [=] {
    down_reduce((const uint16_t*)A, (const int64_t*)indices, (const uint16_t*)weights,
                (const int64_t*)pointers, (float*)out, top_k, max_expert, N, rows);
  });
}

// Arguments shared by the decode-time expert kernels.
#pragma once
#include <stdint.h>

namespace ink {

constexpr int kBank = 6;            // pointer-table entries per NVFP4 expert
constexpr int kBatchLoads = 8;      // 16-byte weight loads a lane keeps in flight

struct DecodeArgs {
  const uint16_t* x;                // [tokens, hidden] BF16
  const int64_t* indices;           // [tokens * top_k]
  const uint16_t* weights;          // [tokens * top_k] BF16
  const int64_t* pointers;          // [(max_expert + 1) * 6]
  uint16_t* activated;              // [tokens * top_k, intermediate] BF16
  const uint16_t* shared_gate;      // [n_shared, intermediate, hidden] BF16
  const uint16_t* shared_up;
  const uint16_t* shared_down;      // [n_shared, hidden, intermediate] BF16
  const uint16_t* gammas;           // [tokens, n_shared] BF16
  uint16_t* shared_activated;       // [tokens * n_shared, intermediate] BF16
  float* output;                    // [tokens, hidden] FP32
  int tokens, top_k, n_shared, hidden, intermediate, max_expert;
  int32_t* status;
};


}  // namespace ink

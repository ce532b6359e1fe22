// Tensor maps (TMA descriptors) of 2-byte element tensors, encoded once and kept.
#pragma once

#include "aps_common.cuh"

#include <cuda.h>

namespace aps {

// A tiled tensor map with 128-byte swizzle over fp16 / bf16 data.  dims / box: innermost
// first; strides_bytes[i] = byte stride of dimension i + 1.  rank 2 or 3.
struct TensorMapSpec {
  const void* base;
  int dtype;                  // APS_F16 / APS_BF16
  int rank;
  uint64_t dims[3];
  uint64_t strides_bytes[2];
  uint32_t box[3];
};

// A tensor map is a pure function of its spec: the encoded maps are kept in a small per-thread
// table (the library has one calling thread), so a layer that is called every step with the
// same caches and weights encodes each of its maps once.
int cached_tensor_map(CUtensorMap* out, const TensorMapSpec& spec, const char* what);

}  // namespace aps

// Encoding and caching of tensor maps (see tensor_maps.cuh).  cuTensorMapEncodeTiled is
// resolved through the runtime's driver entry point query, so the library does not link
// against libcuda.
#include "tensor_maps.cuh"

#include <string.h>

namespace aps {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

struct MapSlot { TensorMapSpec spec; CUtensorMap map; bool used; };
constexpr int kMapSlots = 32;

bool same_spec(const TensorMapSpec& a, const TensorMapSpec& b) {
  if (a.base != b.base || a.dtype != b.dtype || a.rank != b.rank) return false;
  for (int i = 0; i < a.rank; ++i)
    if (a.dims[i] != b.dims[i] || a.box[i] != b.box[i]) return false;
  for (int i = 0; i + 1 < a.rank; ++i)
    if (a.strides_bytes[i] != b.strides_bytes[i]) return false;
  return true;
}

}  // namespace

int cached_tensor_map(CUtensorMap* out, const TensorMapSpec& spec, const char* what) {
  static thread_local MapSlot slots[kMapSlots] = {};
  static thread_local unsigned next_slot = 0;
  APS_REQUIRE(spec.rank == 2 || spec.rank == 3, APS_ERR_SHAPE, "tensor map (%s): rank %d not supported", what, spec.rank);
  for (int i = 0; i < kMapSlots; ++i)
    if (slots[i].used && same_spec(slots[i].spec, spec)) { *out = slots[i].map; return APS_OK; }
  EncodeTiledFn fn = encode_fn();
  APS_REQUIRE(fn != nullptr, APS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const CUtensorMapDataType dt = spec.dtype == APS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[3] = {spec.dims[0], spec.dims[1], spec.rank > 2 ? spec.dims[2] : 1};
  cuuint64_t strides[2] = {spec.strides_bytes[0], spec.rank > 2 ? spec.strides_bytes[1] : 0};
  cuuint32_t box[3] = {spec.box[0], spec.box[1], spec.rank > 2 ? spec.box[2] : 1};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult r = fn(out, dt, (cuuint32_t)spec.rank, const_cast<void*>(spec.base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  APS_REQUIRE(r == CUDA_SUCCESS, APS_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  MapSlot& s = slots[next_slot++ % kMapSlots];
  s.spec = spec; s.map = *out; s.used = true;
  return APS_OK;
}

}  // namespace aps

// Paged cache writes of the hybrid-cache path: pure data movement, HBM-bound.
//
// Every op moves whole rows (one token's K or V row, or one token's hidden row)
// between a packed tensor and a paged cache, driven by a slot mapping.  One CTA
// moves one row with the widest vector access the pointers, strides and row
// length allow (16 bytes in every layout the reference's cache engine produces);
// loads of a row are issued in batches of four before the stores so that each
// thread keeps 64 bytes in flight.  Results are bit-exact copies.
//
// Semantics follow the reference's additional_designs/mixed_cache_kernels/
// mixed_cache.cu (kernels at :6-28, :31-53, :56-116) and the call sites of the
// third-party reshape_and_cache_flash / copy_blocks in additional_designs/
// attention/backends/aptserve_flash_attn.py:58-65, 338-385.

#include "aps_common.cuh"

#include <initializer_list>
#include <stdlib.h>

namespace aps {
namespace {

constexpr int kCopyThreads = 256;

template <typename V>
__device__ __forceinline__ void copy_row(V* __restrict__ dst, const V* __restrict__ src, int n_vec) {
  const int bd = blockDim.x;
  int i = threadIdx.x;
  for (; i + 3 * bd < n_vec; i += 4 * bd) {
    V a = src[i], b = src[i + bd], c = src[i + 2 * bd], d = src[i + 3 * bd];
    dst[i] = a; dst[i + bd] = b; dst[i + 2 * bd] = c; dst[i + 3 * bd] = d;
  }
  for (; i < n_vec; i += bd) dst[i] = src[i];
}

template <typename V>
__device__ __forceinline__ void copy_row2(V* __restrict__ dst0, V* __restrict__ dst1,
                                          const V* __restrict__ src, int n_vec) {
  const int bd = blockDim.x;
  int i = threadIdx.x;
  for (; i + 3 * bd < n_vec; i += 4 * bd) {
    V a = src[i], b = src[i + bd], c = src[i + 2 * bd], d = src[i + 3 * bd];
    dst0[i] = a; dst0[i + bd] = b; dst0[i + 2 * bd] = c; dst0[i + 3 * bd] = d;
    dst1[i] = a; dst1[i + bd] = b; dst1[i + 2 * bd] = c; dst1[i + 3 * bd] = d;
  }
  for (; i < n_vec; i += bd) { V a = src[i]; dst0[i] = a; dst1[i] = a; }
}

// All byte offsets below are multiples of sizeof(V) (checked on the host).
template <typename V>
__global__ void __launch_bounds__(kCopyThreads)
reshape_and_cache_kernel(const char* __restrict__ key, const char* __restrict__ value,
                         char* __restrict__ key_cache, char* __restrict__ value_cache,
                         const int64_t* __restrict__ slot_mapping, int64_t num_tokens,
                         int64_t key_stride_b, int64_t value_stride_b, int64_t block_stride_b,
                         int64_t row_bytes, int block_size) {
  for (int64_t t = blockIdx.x; t < num_tokens; t += gridDim.x) {
    const int64_t slot = slot_mapping[t];
    if (slot < 0) continue;
    const int64_t off = (slot / block_size) * block_stride_b + (slot % block_size) * row_bytes;
    const int n_vec = static_cast<int>(row_bytes / sizeof(V));
    if (blockIdx.y == 0)
      copy_row(reinterpret_cast<V*>(key_cache + off),
               reinterpret_cast<const V*>(key + t * key_stride_b), n_vec);
    else
      copy_row(reinterpret_cast<V*>(value_cache + off),
               reinterpret_cast<const V*>(value + t * value_stride_b), n_vec);
  }
}

template <typename V>
__global__ void __launch_bounds__(kCopyThreads)
hidden_to_cache_kernel(const char* __restrict__ hidden, char* __restrict__ paged_cache,
                       const int64_t* __restrict__ slot_mapping, const int64_t* __restrict__ src_idx,
                       const int64_t* __restrict__ target_slot_idx, int64_t n,
                       int64_t hidden_stride_b, int64_t slot_stride_b, int64_t row_bytes) {
  for (int64_t i = blockIdx.x; i < n; i += gridDim.x) {
    const int64_t slot = slot_mapping[target_slot_idx[i]];
    if (slot < 0) continue;
    copy_row(reinterpret_cast<V*>(paged_cache + slot * slot_stride_b),
             reinterpret_cast<const V*>(hidden + src_idx[i] * hidden_stride_b),
             static_cast<int>(row_bytes / sizeof(V)));
  }
}

template <typename V>
__global__ void __launch_bounds__(kCopyThreads)
cache_to_hidden_kernel(char* __restrict__ hidden, const char* __restrict__ paged_cache,
                       const int64_t* __restrict__ slot_mapping, const int64_t* __restrict__ dst_idx,
                       int64_t n, int64_t hidden_stride_b, int64_t slot_stride_b, int64_t row_bytes) {
  for (int64_t i = blockIdx.x; i < n; i += gridDim.x) {
    const int64_t t = dst_idx[i];
    const int64_t slot = slot_mapping[t];
    if (slot < 0) continue;
    copy_row(reinterpret_cast<V*>(hidden + t * hidden_stride_b),
             reinterpret_cast<const V*>(paged_cache + slot * slot_stride_b),
             static_cast<int>(row_bytes / sizeof(V)));
  }
}

// Prefill cache write in one pass over the packed prompt tokens, as a flat list of row
// copies: jobs [0, 2 n_kv) copy the K row (even job) or the V row (odd job) of token
// kv_rows[job / 2] into the K / V plane; jobs [2 n_kv, 2 n_kv + n_hidden) copy the
// layer-input row of token hidden_rows[j] into the flat hidden rows.  Every token's slot is
// slot_mapping[token].
template <typename V>
__global__ void __launch_bounds__(kCopyThreads)
prefill_write_kernel(const char* __restrict__ key, const char* __restrict__ value,
                     const char* __restrict__ hidden, char* __restrict__ key_cache,
                     char* __restrict__ value_cache, char* __restrict__ hidden_cache,
                     const int64_t* __restrict__ slot_mapping, const int64_t* __restrict__ kv_rows,
                     int64_t n_kv, const int64_t* __restrict__ hidden_rows, int64_t n_hidden,
                     int64_t key_stride_b, int64_t value_stride_b, int64_t hidden_stride_b,
                     int64_t block_stride_b, int64_t slot_stride_b, int64_t kv_row_bytes,
                     int64_t hidden_row_bytes, int block_size) {
  for (int64_t job = blockIdx.x; job < 2 * n_kv + n_hidden; job += gridDim.x) {
    if (job < 2 * n_kv) {
      const int64_t tok = kv_rows[job >> 1];
      const int64_t slot = slot_mapping[tok];
      if (slot < 0) continue;
      const int64_t off = (slot / block_size) * block_stride_b + (slot % block_size) * kv_row_bytes;
      const int n_vec = static_cast<int>(kv_row_bytes / sizeof(V));
      if ((job & 1) == 0)
        copy_row(reinterpret_cast<V*>(key_cache + off), reinterpret_cast<const V*>(key + tok * key_stride_b), n_vec);
      else
        copy_row(reinterpret_cast<V*>(value_cache + off), reinterpret_cast<const V*>(value + tok * value_stride_b), n_vec);
    } else {
      const int64_t tok = hidden_rows[job - 2 * n_kv];
      const int64_t slot = slot_mapping[tok];
      if (slot < 0) continue;
      copy_row(reinterpret_cast<V*>(hidden_cache + slot * slot_stride_b),
               reinterpret_cast<const V*>(hidden + tok * hidden_stride_b),
               static_cast<int>(hidden_row_bytes / sizeof(V)));
    }
  }
}

// Jobs [0, n_kv): a K/V request's new token goes to the private cache and, at
// the same slot, to the shared cache (one read, two writes).  Jobs
// [n_kv, n_kv + n_hidden): a hidden request's re-projected token goes to the
// shared cache at slot_mapping_shared[j].  blockIdx.y selects K or V.
template <typename V>
__global__ void __launch_bounds__(kCopyThreads)
mixed_kv_to_cache_kernel(const char* __restrict__ key, const char* __restrict__ value,
                         char* __restrict__ k_cache, char* __restrict__ v_cache,
                         char* __restrict__ shared_k, char* __restrict__ shared_v,
                         const int64_t* __restrict__ slot_mapping,
                         const int64_t* __restrict__ slot_mapping_shared,
                         const int64_t* __restrict__ kv_cache_use_tot,
                         const int64_t* __restrict__ hidden_cache_use_tot, int64_t n_kv,
                         int64_t n_hidden, int64_t key_stride_b, int64_t value_stride_b,
                         int64_t block_stride_b, int64_t shared_block_stride_b,
                         int64_t row_bytes, int block_size) {
  const bool is_v = blockIdx.y != 0;
  const char* src_base = is_v ? value : key;
  const int64_t src_stride = is_v ? value_stride_b : key_stride_b;
  char* priv = is_v ? v_cache : k_cache;
  char* shar = is_v ? shared_v : shared_k;
  const int n_vec = static_cast<int>(row_bytes / sizeof(V));
  for (int64_t job = blockIdx.x; job < n_kv + n_hidden; job += gridDim.x) {
    if (job < n_kv) {
      const int64_t tok = kv_cache_use_tot[job];
      const int64_t slot = slot_mapping[tok];
      if (slot < 0) continue;
      const int64_t blk = slot / block_size, in_blk = (slot % block_size) * row_bytes;
      copy_row2(reinterpret_cast<V*>(priv + blk * block_stride_b + in_blk),
                reinterpret_cast<V*>(shar + blk * shared_block_stride_b + in_blk),
                reinterpret_cast<const V*>(src_base + tok * src_stride), n_vec);
    } else {
      const int64_t j = job - n_kv;
      const int64_t tok = hidden_cache_use_tot[j];
      const int64_t slot = slot_mapping_shared[j];
      if (slot < 0) continue;
      const int64_t blk = slot / block_size, in_blk = (slot % block_size) * row_bytes;
      copy_row(reinterpret_cast<V*>(shar + blk * shared_block_stride_b + in_blk),
               reinterpret_cast<const V*>(src_base + tok * src_stride), n_vec);
    }
  }
}

constexpr int kMaxLayersPerLaunch = 64;
struct LayerPtrs {
  char* k[kMaxLayersPerLaunch];
  char* v[kMaxLayersPerLaunch];
};

// grid = (pairs, layers, 2 planes); a block of one plane is split over
// gridDim-independent loops of 16-byte (or narrower) vectors.
template <typename V>
__global__ void __launch_bounds__(kCopyThreads)
copy_blocks_kernel(LayerPtrs ptrs, const int64_t* __restrict__ block_mapping, int64_t num_pairs,
                   int64_t block_bytes) {
  char* base = blockIdx.z == 0 ? ptrs.k[blockIdx.y] : ptrs.v[blockIdx.y];
  for (int64_t p = blockIdx.x; p < num_pairs; p += gridDim.x) {
    const int64_t src = block_mapping[2 * p], dst = block_mapping[2 * p + 1];
    copy_row(reinterpret_cast<V*>(base + dst * block_bytes),
             reinterpret_cast<const V*>(base + src * block_bytes),
             static_cast<int>(block_bytes / sizeof(V)));
  }
}

// Widest power-of-two vector (<= 16 bytes) dividing every quantity given.
inline int common_vector_bytes(std::initializer_list<uint64_t> values) {
  int v = 16;
  for (uint64_t x : values)
    while (v > 1 && (x % v) != 0) v >>= 1;
  return v;
}

// Rows are taken grid-stride by persistent CTAs: at most APS_COPY_CTAS_PER_SM (default 8,
// i.e. 2048 resident threads) per SM, so that large prefill writes do not pay a CTA launch
// per 10 KB row.
inline unsigned grid_for(int64_t rows) {
  static int per_sm = 0;
  if (per_sm == 0) {
    const char* v = getenv("APS_COPY_CTAS_PER_SM");
    per_sm = v != nullptr && atoi(v) > 0 ? atoi(v) : 8;
  }
  const int64_t cap = (int64_t)sm_count() * per_sm;
  return static_cast<unsigned>(rows < cap ? rows : cap);
}

inline int threads_for(int64_t n_vec) {
  int64_t t = (n_vec + 31) / 32 * 32;
  if (t < 32) t = 32;
  if (t > kCopyThreads) t = kCopyThreads;
  return static_cast<int>(t);
}

#define APS_DISPATCH_VEC(vec_bytes, ...)                                              \
  switch (vec_bytes) {                                                                \
    case 16: { using V = uint4; __VA_ARGS__; break; }                                 \
    case 8:  { using V = uint2; __VA_ARGS__; break; }                                 \
    case 4:  { using V = uint32_t; __VA_ARGS__; break; }                              \
    default: { using V = uint16_t; __VA_ARGS__; break; }                              \
  }

}  // namespace
}  // namespace aps

using namespace aps;

extern "C" int aps_reshape_and_cache(const void* key, const void* value, void* key_cache,
                                     void* value_cache, const int64_t* slot_mapping,
                                     int64_t num_tokens, int num_heads, int head_size,
                                     int block_size, int64_t key_stride, int64_t value_stride,
                                     int64_t block_stride, int dtype, void* stream) {
  const int es = dtype_size(dtype);
  APS_REQUIRE(es != 0, APS_ERR_DTYPE, "reshape_and_cache: unsupported dtype %d", dtype);
  APS_REQUIRE(num_tokens >= 0 && num_heads > 0 && head_size > 0 && block_size > 0, APS_ERR_SHAPE,
              "reshape_and_cache: bad sizes (tokens=%lld heads=%d head_size=%d block_size=%d)",
              (long long)num_tokens, num_heads, head_size, block_size);
  if (num_tokens == 0) return APS_OK;
  APS_REQUIRE(key && value && key_cache && value_cache && slot_mapping, APS_ERR_NULL_POINTER,
              "reshape_and_cache: null pointer");
  const int64_t row = (int64_t)num_heads * head_size;
  APS_REQUIRE(key_stride >= row && value_stride >= row && block_stride >= row * block_size,
              APS_ERR_SHAPE, "reshape_and_cache: strides smaller than a row / block");
  APS_REQUIRE(aligned_to(key, es) && aligned_to(value, es) && aligned_to(key_cache, es) &&
                  aligned_to(value_cache, es) && aligned_to(slot_mapping, 8),
              APS_ERR_MISALIGNED, "reshape_and_cache: pointer not aligned to its element size");
  const int vb = common_vector_bytes({(uint64_t)(uintptr_t)key, (uint64_t)(uintptr_t)value,
                                      (uint64_t)(uintptr_t)key_cache, (uint64_t)(uintptr_t)value_cache,
                                      (uint64_t)row * es, (uint64_t)key_stride * es,
                                      (uint64_t)value_stride * es, (uint64_t)block_stride * es});
  dim3 grid(grid_for(num_tokens), 2);
  APS_DISPATCH_VEC(vb, reshape_and_cache_kernel<V><<<grid, threads_for(row * es / vb), 0,
                                                   (cudaStream_t)stream>>>(
      (const char*)key, (const char*)value, (char*)key_cache, (char*)value_cache, slot_mapping,
      num_tokens, key_stride * es, value_stride * es, block_stride * es, row * es, block_size));
  return launch_status("reshape_and_cache_kernel");
}

extern "C" int aps_hidden_to_cache(const void* hidden, void* paged_cache,
                                   const int64_t* slot_mapping, const int64_t* src_idx,
                                   const int64_t* target_slot_idx, int64_t n, int hidden_size,
                                   int64_t hidden_stride, int64_t slot_stride, int dtype,
                                   void* stream) {
  const int es = dtype_size(dtype);
  APS_REQUIRE(es != 0, APS_ERR_DTYPE, "hidden_to_cache: unsupported dtype %d", dtype);
  APS_REQUIRE(n >= 0 && hidden_size > 0, APS_ERR_SHAPE, "hidden_to_cache: bad sizes");
  if (n == 0) return APS_OK;
  APS_REQUIRE(hidden && paged_cache && slot_mapping && src_idx && target_slot_idx,
              APS_ERR_NULL_POINTER, "hidden_to_cache: null pointer");
  APS_REQUIRE(hidden_stride >= hidden_size && slot_stride > 0, APS_ERR_SHAPE,
              "hidden_to_cache: bad strides (hidden_stride=%lld slot_stride=%lld)",
              (long long)hidden_stride, (long long)slot_stride);
  APS_REQUIRE(aligned_to(hidden, es) && aligned_to(paged_cache, es), APS_ERR_MISALIGNED,
              "hidden_to_cache: pointer not aligned to its element size");
  const int vb = common_vector_bytes({(uint64_t)(uintptr_t)hidden, (uint64_t)(uintptr_t)paged_cache,
                                      (uint64_t)hidden_size * es, (uint64_t)hidden_stride * es,
                                      (uint64_t)slot_stride * es});
  APS_DISPATCH_VEC(vb, hidden_to_cache_kernel<V><<<grid_for(n), threads_for((int64_t)hidden_size * es / vb),
                                                 0, (cudaStream_t)stream>>>(
      (const char*)hidden, (char*)paged_cache, slot_mapping, src_idx, target_slot_idx, n,
      hidden_stride * es, slot_stride * es, (int64_t)hidden_size * es));
  return launch_status("hidden_to_cache_kernel");
}

extern "C" int aps_cache_to_hidden(void* hidden, const void* paged_cache,
                                   const int64_t* slot_mapping, const int64_t* dst_idx, int64_t n,
                                   int hidden_size, int64_t hidden_stride, int64_t slot_stride,
                                   int dtype, void* stream) {
  const int es = dtype_size(dtype);
  APS_REQUIRE(es != 0, APS_ERR_DTYPE, "cache_to_hidden: unsupported dtype %d", dtype);
  APS_REQUIRE(n >= 0 && hidden_size > 0, APS_ERR_SHAPE, "cache_to_hidden: bad sizes");
  if (n == 0) return APS_OK;
  APS_REQUIRE(hidden && paged_cache && slot_mapping && dst_idx, APS_ERR_NULL_POINTER,
              "cache_to_hidden: null pointer");
  APS_REQUIRE(hidden_stride >= hidden_size && slot_stride > 0, APS_ERR_SHAPE,
              "cache_to_hidden: bad strides");
  APS_REQUIRE(aligned_to(hidden, es) && aligned_to(paged_cache, es), APS_ERR_MISALIGNED,
              "cache_to_hidden: pointer not aligned to its element size");
  const int vb = common_vector_bytes({(uint64_t)(uintptr_t)hidden, (uint64_t)(uintptr_t)paged_cache,
                                      (uint64_t)hidden_size * es, (uint64_t)hidden_stride * es,
                                      (uint64_t)slot_stride * es});
  APS_DISPATCH_VEC(vb, cache_to_hidden_kernel<V><<<grid_for(n), threads_for((int64_t)hidden_size * es / vb),
                                                 0, (cudaStream_t)stream>>>(
      (char*)hidden, (const char*)paged_cache, slot_mapping, dst_idx, n, hidden_stride * es,
      slot_stride * es, (int64_t)hidden_size * es));
  return launch_status("cache_to_hidden_kernel");
}

extern "C" int aps_mixed_kv_to_cache(const void* key, const void* value, void* k_cache,
                                     void* v_cache, void* shared_k_cache, void* shared_v_cache,
                                     const int64_t* slot_mapping,
                                     const int64_t* slot_mapping_shared,
                                     const int64_t* kv_cache_use_tot,
                                     const int64_t* hidden_cache_use_tot, int64_t n_kv,
                                     int64_t n_hidden, int num_heads, int head_size,
                                     int block_size, int64_t key_stride, int64_t value_stride,
                                     int64_t block_stride, int64_t shared_block_stride, int dtype,
                                     void* stream) {
  const int es = dtype_size(dtype);
  APS_REQUIRE(es != 0, APS_ERR_DTYPE, "mixed_kv_to_cache: unsupported dtype %d", dtype);
  APS_REQUIRE(n_kv >= 0 && n_hidden >= 0 && num_heads > 0 && head_size > 0 && block_size > 0,
              APS_ERR_SHAPE, "mixed_kv_to_cache: bad sizes");
  if (n_kv + n_hidden == 0) return APS_OK;
  APS_REQUIRE(key && value && shared_k_cache && shared_v_cache, APS_ERR_NULL_POINTER,
              "mixed_kv_to_cache: null pointer");
  APS_REQUIRE(n_kv == 0 || (k_cache && v_cache && slot_mapping && kv_cache_use_tot),
              APS_ERR_NULL_POINTER, "mixed_kv_to_cache: null pointer (K/V request arguments)");
  APS_REQUIRE(n_hidden == 0 || (slot_mapping_shared && hidden_cache_use_tot),
              APS_ERR_NULL_POINTER, "mixed_kv_to_cache: null pointer (hidden request arguments)");
  const int64_t row = (int64_t)num_heads * head_size;
  APS_REQUIRE(key_stride >= row && value_stride >= row && block_stride >= row * block_size &&
                  shared_block_stride >= row * block_size,
              APS_ERR_SHAPE, "mixed_kv_to_cache: strides smaller than a row / block");
  const int vb = common_vector_bytes(
      {(uint64_t)(uintptr_t)key, (uint64_t)(uintptr_t)value, (uint64_t)(uintptr_t)k_cache,
       (uint64_t)(uintptr_t)v_cache, (uint64_t)(uintptr_t)shared_k_cache,
       (uint64_t)(uintptr_t)shared_v_cache, (uint64_t)row * es, (uint64_t)key_stride * es,
       (uint64_t)value_stride * es, (uint64_t)block_stride * es,
       (uint64_t)shared_block_stride * es});
  APS_REQUIRE(vb >= es, APS_ERR_MISALIGNED, "mixed_kv_to_cache: pointer not aligned to its element size");
  dim3 grid(grid_for(n_kv + n_hidden), 2);
  APS_DISPATCH_VEC(vb, mixed_kv_to_cache_kernel<V><<<grid, threads_for(row * es / vb), 0,
                                                   (cudaStream_t)stream>>>(
      (const char*)key, (const char*)value, (char*)k_cache, (char*)v_cache, (char*)shared_k_cache,
      (char*)shared_v_cache, slot_mapping, slot_mapping_shared, kv_cache_use_tot,
      hidden_cache_use_tot, n_kv, n_hidden, key_stride * es, value_stride * es, block_stride * es,
      shared_block_stride * es, row * es, block_size));
  return launch_status("mixed_kv_to_cache_kernel");
}

extern "C" int aps_prefill_cache_write(const void* key, const void* value, const void* hidden,
                                       void* key_cache, void* value_cache, void* hidden_cache,
                                       const int64_t* slot_mapping, const int64_t* kv_rows,
                                       int64_t n_kv, const int64_t* hidden_rows, int64_t n_hidden,
                                       int num_heads, int head_size, int hidden_size, int block_size,
                                       int64_t key_stride, int64_t value_stride, int64_t hidden_stride,
                                       int64_t block_stride, int64_t slot_stride, int dtype,
                                       void* stream) {
  const int es = dtype_size(dtype);
  APS_REQUIRE(es != 0, APS_ERR_DTYPE, "prefill_cache_write: unsupported dtype %d", dtype);
  APS_REQUIRE(n_kv >= 0 && n_hidden >= 0 && num_heads > 0 && head_size > 0 && hidden_size > 0 &&
                  block_size > 0,
              APS_ERR_SHAPE, "prefill_cache_write: bad sizes");
  if (n_kv + n_hidden == 0) return APS_OK;
  APS_REQUIRE(slot_mapping != nullptr, APS_ERR_NULL_POINTER, "prefill_cache_write: null pointer");
  APS_REQUIRE(n_kv == 0 || (key && value && key_cache && value_cache && kv_rows), APS_ERR_NULL_POINTER,
              "prefill_cache_write: null pointer (K/V arguments)");
  APS_REQUIRE(n_hidden == 0 || (hidden && hidden_cache && hidden_rows), APS_ERR_NULL_POINTER,
              "prefill_cache_write: null pointer (hidden arguments)");
  const int64_t row = (int64_t)num_heads * head_size;
  APS_REQUIRE(n_kv == 0 || (key_stride >= row && value_stride >= row && block_stride >= row * block_size),
              APS_ERR_SHAPE, "prefill_cache_write: K/V strides smaller than a row / block");
  APS_REQUIRE(n_hidden == 0 || (hidden_stride >= hidden_size && slot_stride > 0), APS_ERR_SHAPE,
              "prefill_cache_write: bad hidden strides");
  int vb = 16;
  if (n_kv > 0)
    vb = common_vector_bytes({(uint64_t)(uintptr_t)key, (uint64_t)(uintptr_t)value,
                              (uint64_t)(uintptr_t)key_cache, (uint64_t)(uintptr_t)value_cache,
                              (uint64_t)row * es, (uint64_t)key_stride * es, (uint64_t)value_stride * es,
                              (uint64_t)block_stride * es});
  if (n_hidden > 0) {
    const int vh = common_vector_bytes({(uint64_t)(uintptr_t)hidden, (uint64_t)(uintptr_t)hidden_cache,
                                        (uint64_t)hidden_size * es, (uint64_t)hidden_stride * es,
                                        (uint64_t)slot_stride * es});
    vb = vh < vb ? vh : vb;
  }
  APS_REQUIRE(vb >= es, APS_ERR_MISALIGNED, "prefill_cache_write: pointer not aligned to its element size");
  const unsigned grid = grid_for(2 * n_kv + n_hidden);
  const int64_t widest = row > hidden_size ? row : hidden_size;
  APS_DISPATCH_VEC(vb, prefill_write_kernel<V><<<grid, threads_for(widest * es / vb), 0, (cudaStream_t)stream>>>(
      (const char*)key, (const char*)value, (const char*)hidden, (char*)key_cache, (char*)value_cache,
      (char*)hidden_cache, slot_mapping, kv_rows, n_kv, hidden_rows, n_hidden, key_stride * es,
      value_stride * es, hidden_stride * es, block_stride * es, slot_stride * es, row * es,
      (int64_t)hidden_size * es, block_size));
  return launch_status("prefill_write_kernel");
}

extern "C" int aps_copy_blocks(void* const* key_cache_ptrs, void* const* value_cache_ptrs,
                               int num_layers, const int64_t* block_mapping, int64_t num_pairs,
                               int64_t block_bytes, void* stream) {
  APS_REQUIRE(num_layers >= 0 && num_pairs >= 0 && block_bytes > 0, APS_ERR_SHAPE,
              "copy_blocks: bad sizes");
  if (num_layers == 0 || num_pairs == 0) return APS_OK;
  APS_REQUIRE(key_cache_ptrs && value_cache_ptrs && block_mapping, APS_ERR_NULL_POINTER,
              "copy_blocks: null pointer");
  uint64_t bits = (uint64_t)block_bytes;
  for (int l = 0; l < num_layers; ++l) {
    APS_REQUIRE(key_cache_ptrs[l] && value_cache_ptrs[l], APS_ERR_NULL_POINTER,
                "copy_blocks: null cache pointer for layer %d", l);
    bits |= (uint64_t)(uintptr_t)key_cache_ptrs[l] | (uint64_t)(uintptr_t)value_cache_ptrs[l];
  }
  int vb = 16;
  while (vb > 1 && (bits % vb) != 0) vb >>= 1;
  APS_REQUIRE(vb >= 2, APS_ERR_MISALIGNED, "copy_blocks: caches must be at least 2-byte aligned");
  for (int l0 = 0; l0 < num_layers; l0 += kMaxLayersPerLaunch) {
    const int nl = num_layers - l0 < kMaxLayersPerLaunch ? num_layers - l0 : kMaxLayersPerLaunch;
    LayerPtrs ptrs;
    for (int l = 0; l < nl; ++l) {
      ptrs.k[l] = (char*)key_cache_ptrs[l0 + l];
      ptrs.v[l] = (char*)value_cache_ptrs[l0 + l];
    }
    dim3 grid(grid_for(num_pairs > 65535 ? 65535 : num_pairs), nl, 2);
    APS_DISPATCH_VEC(vb, copy_blocks_kernel<V><<<grid, kCopyThreads, 0, (cudaStream_t)stream>>>(
                             ptrs, block_mapping, num_pairs, block_bytes));
    int st = launch_status("copy_blocks_kernel");
    if (st != APS_OK) return st;
  }
  return APS_OK;
}

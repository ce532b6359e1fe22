// Paged cache writes of the hybrid-cache path: pure data movement, HBM-bound.
//
// Every op moves whole rows (one token's K or V row, or one token's hidden row)
// between a packed tensor and a paged cache, driven by a slot mapping.  Results are
// bit-exact copies.  Two ways of moving a row:
//
//   bulk   (pointers, strides and row length all multiples of 16 bytes: every layout the
//          reference's cache engine produces)  One-warp CTAs, persistent.  The lanes
//          resolve the next 32 rows' addresses through the index tensors in parallel; one
//          lane then moves each row global -> shared -> global with two bulk-copy
//          instructions (cp.async.bulk, completion on an mbarrier on the way in, a bulk
//          group on the way out) through two buffers: the next row's load is in flight
//          while this row is stored.  One instruction per 10 KB instead of one load/store
//          pair per 16 bytes.  What a CTA spends per row is a chain of round trips counted
//          in SM cycles, so the number of CTAs per SM is what matters at the ~1 GHz SM clock
//          the power cap leaves inside a decode step: two buffers of one row each let ten
//          CTAs share an SM for 10 KB rows (measured inside the loaded step on OPT-13B
//          prefill rows: 5.4 TB/s read + write; deeper rings with fewer CTAs 3.0 - 4.0 TB/s,
//          the vector kernels 3.9 TB/s).
//   vector (anything else)  One CTA moves one row with the widest vector access the
//          alignment allows; loads of a row are issued in batches of four before the
//          stores so that each thread keeps 64 bytes in flight.
//
// Semantics follow the reference's additional_designs/mixed_cache_kernels/
// mixed_cache.cu (kernels at :6-28, :31-53, :56-116) and the call sites of the
// third-party reshape_and_cache_flash / copy_blocks in additional_designs/
// attention/backends/aptserve_flash_attn.py:58-65, 338-385.

#include "attention_common.cuh"   // NewTokenWrite

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


// ---- bulk-copy path -------------------------------------------------------------------
// ring depth, load look-ahead and CTAs per SM can be overridden at compile time for sweeps
#ifndef APS_BULK_STAGES
#define APS_BULK_STAGES 2
#endif
#ifndef APS_BULK_LOOK
#define APS_BULK_LOOK 1
#endif
#ifndef APS_BULK_MAX_CTAS
#define APS_BULK_MAX_CTAS 16
#endif
constexpr int kBulkStages = APS_BULK_STAGES;   // ring of row buffers per CTA
constexpr int kBulkLook = APS_BULK_LOOK;       // loads run this many rows ahead of the stores
static_assert(kBulkLook >= 1 && kBulkLook < kBulkStages, "look-ahead must leave one buffer to the stores");
#ifndef APS_BULK_MAX_PIECE
#define APS_BULK_MAX_PIECE 16384
#endif
constexpr uint32_t kBulkMaxPiece = APS_BULK_MAX_PIECE;   // rows longer than this are moved in equal pieces
constexpr long long kBulkWaitBudget = 2000000000LL;  // clock cycles before a wait gives up

// Set when a bulk-copy wait ran out (it never should: a bulk load completes unless its
// address faults); read back by aps_cache_ops_status.
__device__ int g_copy_status = 0;

struct BulkJob { const char* src; char* dst0; char* dst1; uint32_t bytes; };   // bytes == 0: skip

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Row pieces: a row of `row` bytes is cut into `pieces` runs of `piece` bytes (a multiple of
// 16; the last run is shorter).
struct Pieces {
  uint32_t pieces, piece;
  __host__ __device__ uint32_t offset(uint32_t i) const { return i * piece; }
  __host__ __device__ uint32_t length(uint32_t i, uint32_t row) const {
    const uint32_t o = i * piece;
    return o >= row ? 0u : (row - o < piece ? row - o : piece);
  }
};
inline Pieces pieces_for(uint64_t row_bytes) {
  Pieces p;
  p.pieces = (uint32_t)((row_bytes + kBulkMaxPiece - 1) / kBulkMaxPiece);
  if (p.pieces == 0) p.pieces = 1;
  p.piece = (uint32_t)(((row_bytes + p.pieces - 1) / p.pieces + 15) / 16 * 16);
  return p;
}

template <class Resolver>
__global__ void __launch_bounds__(32)
bulk_copy_kernel(const Resolver R, int64_t n_jobs, uint32_t stage_bytes) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t bars[kBulkStages];
  const int lane = threadIdx.x;
  if ((int64_t)blockIdx.x >= n_jobs) return;
  const int64_t n_my = (n_jobs - blockIdx.x + gridDim.x - 1) / gridDim.x;   // jobs blockIdx.x + k * gridDim.x
  if (lane == 0) {
    for (int s = 0; s < kBulkStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  auto resolve = [&](int64_t batch) {
    const int64_t k = batch * 32 + lane;
    BulkJob j{nullptr, nullptr, nullptr, 0u};
    if (k < n_my) j = R(blockIdx.x + k * (int64_t)gridDim.x);
    return j;
  };
  BulkJob cur = resolve(0), nxt = resolve(1);
  auto job_at = [&](int64_t k, int64_t cur_batch) {
    const bool in_cur = (k >> 5) == cur_batch;
    const int l = (int)(k & 31);
    BulkJob j;
    j.src = reinterpret_cast<const char*>(__shfl_sync(0xffffffffu, (unsigned long long)(in_cur ? cur.src : nxt.src), l));
    j.dst0 = reinterpret_cast<char*>(__shfl_sync(0xffffffffu, (unsigned long long)(in_cur ? cur.dst0 : nxt.dst0), l));
    j.dst1 = reinterpret_cast<char*>(__shfl_sync(0xffffffffu, (unsigned long long)(in_cur ? cur.dst1 : nxt.dst1), l));
    j.bytes = __shfl_sync(0xffffffffu, in_cur ? cur.bytes : nxt.bytes, l);
    return j;
  };
  uint32_t n_loaded = 0, n_stored = 0;   // rows actually moved (lane 0's view; skipped rows take no buffer)
  bool ok = true;
  int64_t cur_batch = 0;
  for (int64_t k = -kBulkLook; k < n_my; ++k) {
    const int64_t kl = k + kBulkLook;
    if (kl < n_my) {
      const BulkJob j = job_at(kl, cur_batch);
      if (lane == 0 && j.bytes != 0 && ok) {
        const uint32_t stage = n_loaded % kBulkStages;
        // the store that last read this buffer is at least (stages - look-ahead) bulk groups back
        asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kBulkStages - kBulkLook - 1) : "memory");
        const uint32_t bar = smem_addr(&bars[stage]), dst = smem_addr(ring + (size_t)stage * stage_bytes);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(j.bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst), "l"(j.src), "r"(j.bytes), "r"(bar) : "memory");
        ++n_loaded;
      }
    }
    if (k >= 0) {
      const BulkJob j = job_at(k, cur_batch);
      if (lane == 0 && j.bytes != 0 && ok) {
        const uint32_t stage = n_stored % kBulkStages, parity = (n_stored / kBulkStages) & 1u;
        const uint32_t bar = smem_addr(&bars[stage]), src = smem_addr(ring + (size_t)stage * stage_bytes);
        uint32_t done = 0;
        const long long t0 = clock64();
        for (int spins = 0; !done; ++spins) {
          asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                       : "=r"(done) : "r"(bar), "r"(parity) : "memory");
          if (!done && (spins & 255) == 255 && clock64() - t0 > kBulkWaitBudget) { ok = false; g_copy_status = 1; break; }
        }
        if (ok) {
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(j.dst0), "r"(src), "r"(j.bytes) : "memory");
          if (j.dst1 != nullptr)
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(j.dst1), "r"(src), "r"(j.bytes) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          ++n_stored;
        }
      }
      if ((k & 31) == 31) { cur = nxt; ++cur_batch; nxt = resolve(cur_batch + 1); }
    }
  }
  // the buffers must outlive the stores that read them; after a wait that gave up, a bounded
  // pause lets the loads still in flight land before the CTA's shared memory is released
  if (lane == 0) {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (!ok) { const long long t0 = clock64(); while (clock64() - t0 < 2000000LL) { } }
  }
  __syncwarp();
}

// One-warp CTAs, all resident: as many per SM as the occupancy query grants for this ring size
// with the shared-memory carve-out at its maximum (at most 16).
template <class Resolver>
int launch_bulk(const Resolver& R, int64_t n_jobs, uint32_t stage_bytes, cudaStream_t stream, const char* what) {
  static bool attr_set[64] = {false};
  const size_t smem = (size_t)kBulkStages * stage_bytes;
  int dev = 0;
  APS_CUDA(cudaGetDevice(&dev));
  APS_REQUIRE(dev >= 0 && dev < 64, APS_ERR_CUDA, "device index %d out of range", dev);
  if (!attr_set[dev]) {
    APS_CUDA(cudaFuncSetAttribute(bulk_copy_kernel<Resolver>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)(kBulkStages * kBulkMaxPiece)));
    APS_CUDA(cudaFuncSetAttribute(bulk_copy_kernel<Resolver>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  cudaSharedmemCarveoutMaxShared));
    attr_set[dev] = true;
  }
  int per_sm = 0;
  APS_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, bulk_copy_kernel<Resolver>, 32, smem));
  if (per_sm > APS_BULK_MAX_CTAS) per_sm = APS_BULK_MAX_CTAS;
  if (per_sm < 1) per_sm = 1;
  const int64_t cap = (int64_t)sm_count() * per_sm;
  const unsigned grid = (unsigned)(n_jobs < cap ? n_jobs : cap);
  bulk_copy_kernel<Resolver><<<grid, 32, smem, stream>>>(R, n_jobs, stage_bytes);
  return launch_status(what);
}

// rows shorter than this go through the vector kernels (one instruction pair per row piece
// is no gain when the pieces are tiny)
constexpr int64_t kBulkMinRowBytes = 512;

struct ReshapeJobs {   // job = (token * 2 + plane) * pieces + piece
  const char* key; const char* value; char* key_cache; char* value_cache; const int64_t* slot_mapping;
  int64_t key_stride_b, value_stride_b, block_stride_b, row_bytes; int block_size; Pieces pc;
  __device__ BulkJob operator()(int64_t job) const {
    const uint32_t piece = (uint32_t)(job % pc.pieces);
    const int64_t tp = job / pc.pieces, t = tp >> 1;
    const bool is_v = (tp & 1) != 0;
    const int64_t slot = slot_mapping[t];
    BulkJob j{nullptr, nullptr, nullptr, 0u};
    if (slot < 0) return j;
    const int64_t off = (slot / block_size) * block_stride_b + (slot % block_size) * row_bytes + pc.offset(piece);
    j.src = (is_v ? value + t * value_stride_b : key + t * key_stride_b) + pc.offset(piece);
    j.dst0 = (is_v ? value_cache : key_cache) + off;
    j.bytes = pc.length(piece, (uint32_t)row_bytes);
    return j;
  }
};

struct HiddenToCacheJobs {
  const char* hidden; char* paged_cache; const int64_t* slot_mapping; const int64_t* src_idx;
  const int64_t* target_slot_idx; int64_t hidden_stride_b, slot_stride_b, row_bytes; Pieces pc;
  __device__ BulkJob operator()(int64_t job) const {
    const uint32_t piece = (uint32_t)(job % pc.pieces);
    const int64_t i = job / pc.pieces;
    const int64_t slot = slot_mapping[target_slot_idx[i]];
    BulkJob j{nullptr, nullptr, nullptr, 0u};
    if (slot < 0) return j;
    j.src = hidden + src_idx[i] * hidden_stride_b + pc.offset(piece);
    j.dst0 = paged_cache + slot * slot_stride_b + pc.offset(piece);
    j.bytes = pc.length(piece, (uint32_t)row_bytes);
    return j;
  }
};

struct CacheToHiddenJobs {
  char* hidden; const char* paged_cache; const int64_t* slot_mapping; const int64_t* dst_idx;
  int64_t hidden_stride_b, slot_stride_b, row_bytes; Pieces pc;
  __device__ BulkJob operator()(int64_t job) const {
    const uint32_t piece = (uint32_t)(job % pc.pieces);
    const int64_t t = dst_idx[job / pc.pieces];
    const int64_t slot = slot_mapping[t];
    BulkJob j{nullptr, nullptr, nullptr, 0u};
    if (slot < 0) return j;
    j.src = paged_cache + slot * slot_stride_b + pc.offset(piece);
    j.dst0 = hidden + t * hidden_stride_b + pc.offset(piece);
    j.bytes = pc.length(piece, (uint32_t)row_bytes);
    return j;
  }
};

struct MixedKvJobs {   // job = (row * 2 + plane) * pieces + piece; rows [0, n_kv) K/V requests, then hidden tokens
  const char* key; const char* value; char* k_cache; char* v_cache; char* shared_k; char* shared_v;
  const int64_t* slot_mapping; const int64_t* slot_mapping_shared; const int64_t* kv_cache_use_tot;
  const int64_t* hidden_cache_use_tot; int64_t n_kv;
  int64_t key_stride_b, value_stride_b, block_stride_b, shared_block_stride_b, row_bytes; int block_size; Pieces pc;
  __device__ BulkJob operator()(int64_t job) const {
    const uint32_t piece = (uint32_t)(job % pc.pieces);
    const int64_t rp = job / pc.pieces, row = rp >> 1;
    const bool is_v = (rp & 1) != 0;
    BulkJob j{nullptr, nullptr, nullptr, 0u};
    int64_t tok, slot;
    if (row < n_kv) { tok = kv_cache_use_tot[row]; slot = slot_mapping[tok]; }
    else { tok = hidden_cache_use_tot[row - n_kv]; slot = slot_mapping_shared[row - n_kv]; }
    if (slot < 0) return j;
    const int64_t blk = slot / block_size, in_blk = (slot % block_size) * row_bytes + pc.offset(piece);
    j.src = (is_v ? value + tok * value_stride_b : key + tok * key_stride_b) + pc.offset(piece);
    char* shar = (is_v ? shared_v : shared_k) + blk * shared_block_stride_b + in_blk;
    if (row < n_kv) { j.dst0 = (is_v ? v_cache : k_cache) + blk * block_stride_b + in_blk; j.dst1 = shar; }
    else j.dst0 = shar;
    j.bytes = pc.length(piece, (uint32_t)row_bytes);
    return j;
  }
};

struct PrefillJobs {   // rows [0, 2 n_kv): K (even) / V (odd) row of token kv_rows[row / 2]; then hidden rows
  const char* key; const char* value; const char* hidden; char* key_cache; char* value_cache; char* hidden_cache;
  const int64_t* slot_mapping; const int64_t* kv_rows; int64_t n_kv; const int64_t* hidden_rows;
  int64_t key_stride_b, value_stride_b, hidden_stride_b, block_stride_b, slot_stride_b, kv_row_bytes, hidden_row_bytes;
  int block_size; Pieces pc_kv, pc_hid; uint32_t pieces;   // pieces = max of the two counts
  __device__ BulkJob operator()(int64_t job) const {
    const uint32_t piece = (uint32_t)(job % pieces);
    const int64_t row = job / pieces;
    BulkJob j{nullptr, nullptr, nullptr, 0u};
    if (row < 2 * n_kv) {
      const int64_t tok = kv_rows[row >> 1], slot = slot_mapping[tok];
      if (slot < 0 || piece >= pc_kv.pieces) return j;
      const int64_t off = (slot / block_size) * block_stride_b + (slot % block_size) * kv_row_bytes + pc_kv.offset(piece);
      const bool is_v = (row & 1) != 0;
      j.src = (is_v ? value + tok * value_stride_b : key + tok * key_stride_b) + pc_kv.offset(piece);
      j.dst0 = (is_v ? value_cache : key_cache) + off;
      j.bytes = pc_kv.length(piece, (uint32_t)kv_row_bytes);
    } else {
      const int64_t tok = hidden_rows[row - 2 * n_kv], slot = slot_mapping[tok];
      if (slot < 0 || piece >= pc_hid.pieces) return j;
      j.src = hidden + tok * hidden_stride_b + pc_hid.offset(piece);
      j.dst0 = hidden_cache + slot * slot_stride_b + pc_hid.offset(piece);
      j.bytes = pc_hid.length(piece, (uint32_t)hidden_row_bytes);
    }
    return j;
  }
};

constexpr int kMaxLayersPerLaunch = 64;
struct LayerPtrs {
  char* k[kMaxLayersPerLaunch];
  char* v[kMaxLayersPerLaunch];
};

// job = ((pair * layers + layer) * 2 + plane) * pieces + piece
struct CopyBlocksJobs {
  LayerPtrs ptrs; const int64_t* block_mapping; int layers; int64_t block_bytes; Pieces pc;
  __device__ BulkJob operator()(int64_t job) const {
    const uint32_t piece = (uint32_t)(job % pc.pieces);
    int64_t r = job / pc.pieces;
    const bool is_v = (r & 1) != 0; r >>= 1;
    const int layer = (int)(r % layers);
    const int64_t pair = r / layers;
    char* base = is_v ? ptrs.v[layer] : ptrs.k[layer];
    BulkJob j;
    j.src = base + block_mapping[2 * pair] * block_bytes + pc.offset(piece);
    j.dst0 = base + block_mapping[2 * pair + 1] * block_bytes + pc.offset(piece);
    j.dst1 = nullptr;
    j.bytes = pc.length(piece, (uint32_t)block_bytes);
    return j;
  }
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

// Vector kernels: rows are taken grid-stride by persistent CTAs, at most 8 per SM (2048
// resident threads), so that large prefill writes do not pay a CTA launch per 10 KB row.
inline unsigned grid_for(int64_t rows) {
  const int64_t cap = (int64_t)sm_count() * 8;
  return static_cast<unsigned>(rows < cap ? rows : cap);
}

inline bool bulk_ok(int vector_bytes, int64_t row_bytes) {
#ifdef APS_BULK_DISABLE   // sweeps only: everything through the vector kernels
  return false;
#endif
  return vector_bytes == 16 && row_bytes >= kBulkMinRowBytes && row_bytes < (int64_t(1) << 31);
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

namespace aps {
namespace {

// New-token writes of a decode batch, addressed from the block tables: row r*2 is the K row
// (K/V-cached request) or the layer-input row (hidden-cached request) of request r, row
// r*2 + 1 its V row (K/V-cached requests only).  The token's position is seq_lens[r] - 1.
struct NewTokenJobs {
  const char* hidden; const char* key; const char* value; char* key_cache; char* value_cache; char* hidden_cache;
  const int32_t* block_tables; const int32_t* seq_lens; const int32_t* cache_type;
  int max_blocks, block_size;
  int64_t hidden_stride_b, key_stride_b, value_stride_b, block_stride_b, slot_stride_b, kv_row_bytes, hidden_row_bytes;
  Pieces pc_kv, pc_hid; uint32_t pieces;
  __device__ BulkJob operator()(int64_t job) const {
    const uint32_t piece = (uint32_t)(job % pieces);
    const int64_t row = job / pieces, r = row >> 1;
    const bool second = (row & 1) != 0;
    BulkJob j{nullptr, nullptr, nullptr, 0u};
    const int pos = min(seq_lens[r], max_blocks * block_size) - 1;
    if (pos < 0) return j;
    const int64_t blk = block_tables[r * max_blocks + pos / block_size];
    if (cache_type[r] != 0) {
      if (second || piece >= pc_hid.pieces || hidden == nullptr) return j;
      j.src = hidden + r * hidden_stride_b + pc_hid.offset(piece);
      j.dst0 = hidden_cache + (blk * block_size + pos % block_size) * slot_stride_b + pc_hid.offset(piece);
      j.bytes = pc_hid.length(piece, (uint32_t)hidden_row_bytes);
    } else {
      if (piece >= pc_kv.pieces || key == nullptr) return j;
      const int64_t off = blk * block_stride_b + (pos % block_size) * kv_row_bytes + pc_kv.offset(piece);
      j.src = (second ? value + r * value_stride_b : key + r * key_stride_b) + pc_kv.offset(piece);
      j.dst0 = (second ? value_cache : key_cache) + off;
      j.bytes = pc_kv.length(piece, (uint32_t)kv_row_bytes);
    }
    return j;
  }
};

}  // namespace

int launch_new_token_write(const NewTokenWrite& a, cudaStream_t stream) {
  const int es = dtype_size(a.dtype);
  const int64_t row = (int64_t)a.heads * a.head_size;
  const bool kv = a.key != nullptr, hid = a.hidden != nullptr;
  if (!kv && !hid) return APS_OK;
  APS_REQUIRE(!kv || (a.value && a.key_cache && a.value_cache), APS_ERR_NULL_POINTER,
              "decode_layer_step: new_key given without new_value / K/V cache");
  APS_REQUIRE(!hid || a.hidden_cache, APS_ERR_NULL_POINTER, "decode_layer_step: hidden_states given without hidden cache");
  int vb = 16;
  if (kv) vb = common_vector_bytes({(uint64_t)(uintptr_t)a.key, (uint64_t)(uintptr_t)a.value, (uint64_t)(uintptr_t)a.key_cache,
                                    (uint64_t)(uintptr_t)a.value_cache, (uint64_t)row * es, (uint64_t)a.key_stride * es,
                                    (uint64_t)a.value_stride * es, (uint64_t)a.block_stride * es});
  if (hid) {
    const int vh = common_vector_bytes({(uint64_t)(uintptr_t)a.hidden, (uint64_t)(uintptr_t)a.hidden_cache,
                                        (uint64_t)a.hidden_size * es, (uint64_t)a.hidden_stride * es,
                                        (uint64_t)a.slot_stride * es});
    vb = vh < vb ? vh : vb;
  }
  APS_REQUIRE(vb == 16, APS_ERR_MISALIGNED,
              "decode_layer_step: step inputs and caches must be 16-byte aligned with 16-byte rows and strides");
  const Pieces pk = pieces_for((uint64_t)row * es), ph = pieces_for((uint64_t)a.hidden_size * es);
  const uint32_t pieces = !kv ? ph.pieces : !hid ? pk.pieces : (pk.pieces > ph.pieces ? pk.pieces : ph.pieces);
  const uint32_t stage = !kv ? ph.piece : !hid ? pk.piece : (pk.piece > ph.piece ? pk.piece : ph.piece);
  NewTokenJobs R{(const char*)a.hidden, (const char*)a.key, (const char*)a.value, (char*)a.key_cache,
                 (char*)a.value_cache, (char*)a.hidden_cache, a.block_tables, a.seq_lens, a.cache_type,
                 a.max_blocks_per_seq, a.block_size, a.hidden_stride * es, a.key_stride * es, a.value_stride * es,
                 a.block_stride * es, a.slot_stride * es, row * es, (int64_t)a.hidden_size * es, pk, ph, pieces};
  return launch_bulk(R, (int64_t)a.batch * 2 * pieces, stage, stream, "new-token cache write (bulk copy)");
}

}  // namespace aps

using namespace aps;

extern "C" int aps_cache_ops_status(int* host_status, void* stream) {
  APS_REQUIRE(host_status != nullptr, APS_ERR_NULL_POINTER, "cache_ops_status: null pointer");
  void* addr = nullptr;
  APS_CUDA(cudaGetSymbolAddress(&addr, g_copy_status));
  APS_CUDA(cudaMemcpyAsync(host_status, addr, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  APS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return APS_OK;
}

// Block moves between one plane of a GPU cache and one plane of the pinned CPU cache (or
// between two device caches): plain copies on the stream, issued from a native loop, with
// every run of pairs whose source and destination blocks are both consecutive merged into
// one copy (a swapped-out request's blocks are mostly allocated in runs).
extern "C" int aps_swap_blocks(const void* src, void* dst, const int64_t* pairs_host, int64_t num_pairs,
                               int64_t block_bytes, int64_t src_block_stride_bytes,
                               int64_t dst_block_stride_bytes, int64_t src_num_blocks,
                               int64_t dst_num_blocks, int kind, int64_t* copies_issued, void* stream) {
  APS_REQUIRE(num_pairs >= 0 && block_bytes > 0, APS_ERR_SHAPE, "swap_blocks: bad sizes");
  if (copies_issued != nullptr) *copies_issued = 0;
  if (num_pairs == 0) return APS_OK;
  APS_REQUIRE(src != nullptr && dst != nullptr && pairs_host != nullptr, APS_ERR_NULL_POINTER,
              "swap_blocks: null pointer");
  APS_REQUIRE(src_block_stride_bytes >= block_bytes && dst_block_stride_bytes >= block_bytes, APS_ERR_SHAPE,
              "swap_blocks: block stride shorter than a block");
  cudaMemcpyKind k;
  switch (kind) {
    case 0: k = cudaMemcpyHostToDevice; break;
    case 1: k = cudaMemcpyDeviceToHost; break;
    case 2: k = cudaMemcpyDeviceToDevice; break;
    default: return fail(APS_ERR_SHAPE, "swap_blocks: kind must be 0 (host to device), 1 (device to host) or 2");
  }
  for (int64_t i = 0; i < num_pairs; ++i) {
    const int64_t sb = pairs_host[2 * i], db = pairs_host[2 * i + 1];
    APS_REQUIRE(sb >= 0 && sb < src_num_blocks && db >= 0 && db < dst_num_blocks, APS_ERR_SHAPE,
                "swap_blocks: pair %lld (%lld -> %lld) is outside the caches", (long long)i, (long long)sb,
                (long long)db);
  }
  // runs can only be merged when blocks lie back to back in both tensors
  const bool dense = src_block_stride_bytes == block_bytes && dst_block_stride_bytes == block_bytes;
  int64_t issued = 0;
  for (int64_t i = 0; i < num_pairs;) {
    int64_t run = 1;
    while (dense && i + run < num_pairs && pairs_host[2 * (i + run)] == pairs_host[2 * i] + run &&
           pairs_host[2 * (i + run) + 1] == pairs_host[2 * i + 1] + run)
      ++run;
    const char* s = static_cast<const char*>(src) + pairs_host[2 * i] * src_block_stride_bytes;
    char* d = static_cast<char*>(dst) + pairs_host[2 * i + 1] * dst_block_stride_bytes;
    APS_CUDA(cudaMemcpyAsync(d, s, (size_t)(run * block_bytes), k, (cudaStream_t)stream));
    ++issued;
    i += run;
  }
  if (copies_issued != nullptr) *copies_issued = issued;
  return APS_OK;
}

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
  if (bulk_ok(vb, row * es)) {
    const Pieces pc = pieces_for((uint64_t)row * es);
    ReshapeJobs R{(const char*)key, (const char*)value, (char*)key_cache, (char*)value_cache, slot_mapping,
                  key_stride * es, value_stride * es, block_stride * es, row * es, block_size, pc};
    return launch_bulk(R, num_tokens * 2 * pc.pieces, pc.piece, (cudaStream_t)stream, "reshape_and_cache (bulk copy)");
  }
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
  if (bulk_ok(vb, (int64_t)hidden_size * es)) {
    const Pieces pc = pieces_for((uint64_t)hidden_size * es);
    HiddenToCacheJobs R{(const char*)hidden, (char*)paged_cache, slot_mapping, src_idx, target_slot_idx,
                        hidden_stride * es, slot_stride * es, (int64_t)hidden_size * es, pc};
    return launch_bulk(R, n * pc.pieces, pc.piece, (cudaStream_t)stream, "hidden_to_cache (bulk copy)");
  }
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
  if (bulk_ok(vb, (int64_t)hidden_size * es)) {
    const Pieces pc = pieces_for((uint64_t)hidden_size * es);
    CacheToHiddenJobs R{(char*)hidden, (const char*)paged_cache, slot_mapping, dst_idx,
                        hidden_stride * es, slot_stride * es, (int64_t)hidden_size * es, pc};
    return launch_bulk(R, n * pc.pieces, pc.piece, (cudaStream_t)stream, "cache_to_hidden (bulk copy)");
  }
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
  if (bulk_ok(vb, row * es)) {
    const Pieces pc = pieces_for((uint64_t)row * es);
    MixedKvJobs R{(const char*)key, (const char*)value, (char*)k_cache, (char*)v_cache, (char*)shared_k_cache,
                  (char*)shared_v_cache, slot_mapping, slot_mapping_shared, kv_cache_use_tot, hidden_cache_use_tot,
                  n_kv, key_stride * es, value_stride * es, block_stride * es, shared_block_stride * es, row * es,
                  block_size, pc};
    return launch_bulk(R, (n_kv + n_hidden) * 2 * pc.pieces, pc.piece, (cudaStream_t)stream, "mixed_kv_to_cache (bulk copy)");
  }
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
  if (bulk_ok(vb, (n_kv > 0 ? row : hidden_size) * (int64_t)es) && bulk_ok(vb, (n_hidden > 0 ? hidden_size : row) * (int64_t)es)) {
    const Pieces pk = pieces_for((uint64_t)row * es), ph = pieces_for((uint64_t)hidden_size * es);
    const uint32_t pieces = n_kv == 0 ? ph.pieces : n_hidden == 0 ? pk.pieces : (pk.pieces > ph.pieces ? pk.pieces : ph.pieces);
    const uint32_t stage = n_kv == 0 ? ph.piece : n_hidden == 0 ? pk.piece : (pk.piece > ph.piece ? pk.piece : ph.piece);
    PrefillJobs R{(const char*)key, (const char*)value, (const char*)hidden, (char*)key_cache, (char*)value_cache,
                  (char*)hidden_cache, slot_mapping, kv_rows, n_kv, hidden_rows, key_stride * es, value_stride * es,
                  hidden_stride * es, block_stride * es, slot_stride * es, row * es, (int64_t)hidden_size * es,
                  block_size, pk, ph, pieces};
    return launch_bulk(R, (2 * n_kv + n_hidden) * pieces, stage, (cudaStream_t)stream, "prefill_cache_write (bulk copy)");
  }
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
    if (bulk_ok(vb, block_bytes)) {
      const Pieces pc = pieces_for((uint64_t)block_bytes);
      CopyBlocksJobs R{ptrs, block_mapping, nl, block_bytes, pc};
      int st = launch_bulk(R, num_pairs * nl * 2 * pc.pieces, pc.piece, (cudaStream_t)stream, "copy_blocks (bulk copy)");
      if (st != APS_OK) return st;
      continue;
    }
    dim3 grid(grid_for(num_pairs > 65535 ? 65535 : num_pairs), nl, 2);
    APS_DISPATCH_VEC(vb, copy_blocks_kernel<V><<<grid, kCopyThreads, 0, (cudaStream_t)stream>>>(
                             ptrs, block_mapping, num_pairs, block_bytes));
    int st = launch_status("copy_blocks_kernel");
    if (st != APS_OK) return st;
  }
  return APS_OK;
}

// Hidden-path decode attention: K/V re-projection on tcgen05 tensor cores fused
// with the decode softmax, plus the hybrid (K/V + hidden) entry point.
//
// What it replaces in the reference (paths under additional_designs/):
//   model_executor/models/aptserve_opt.py:111-124   zero-filled hidden_holder,
//       cache_to_hidden gather of every cached hidden row, kv_only projection
//       (model_executor/layers/aptserve_linear.py:123-130, a cuBLAS GEMM);
//   attention/backends/aptserve_flash_attn.py:356-387  scatter of the projected
//       K/V into the shared cache;  :462-473  paged attention re-reading them.
// Here the hidden rows go HBM -> shared memory (TMA) -> tensor cores -> TMEM ->
// registers -> softmax partial; K and V never exist in global memory.
//
// One M tile = 128 cached token rows, taken 16 at a time (one paged cache block each)
// from the hidden requests in batch order, so a tile can hold rows of several requests and
// only the last tile is partly empty.  For head h the tile's 128 x 256 block
// [K_h | V_h] = X_tile * [W_k,h ; W_v,h]^T is accumulated in fp32 in tensor memory.
// Warp roles in every CTA (320 threads):
//   warp 0, warps 6-9  TMA producers: per 64-element slab of the hidden dimension warp 0
//             posts the stage's byte count and issues the W boxes of head h, warps 6-9
//             issue two 16-row boxes (two cache blocks of the tile) each; 128-byte swizzle,
//             multi-stage ring.  One thread cannot issue ten tensor copies in the 512
//             cycles the tensor cores need for a slab, hence the split;
//   warp 1    tcgen05.mma issuer (K = 16 per instruction, 4 per slab): the whole warp
//             runs the loop in step and one elected lane issues, on warp-uniform
//             operands; the accumulator is double-buffered in the 512 TMEM columns, so
//             the main loop of item i+1 overlaps the epilogue of item i;
//   warps 2-5 epilogue: one thread per token row reads its K row from TMEM, adds
//             b_k, dots with its request's q (pre-scaled by scale*log2 e); maxima, sums
//             and the weighted V column sums are formed per 16-row block with half-warp
//             shuffles and merged per request segment; one (max, sum, acc[128]) partial
//             per (segment, head) goes to scratch.
//
// Main loop: two CTAs of a cluster (cta_group::2) work on two M tiles of the same head
// with one M256 N256 instruction stream issued by the even CTA: each CTA loads its own X
// tile and HALF of the W rows (even CTA: W_k,h, odd CTA: W_v,h), the tensor cores read both
// halves, 6 stages of 32 KB.  Loads carry no multicast: each CTA fetches what it needs
// itself; the two CTAs only exchange mbarrier arrivals.
// CTAs are persistent and walk the items in groups (a few M tiles x a few heads) so
// that hidden tiles and W slabs are shared through L2.
//
// The library reads no environment variable.  Building with -DAPS_TUNING adds one
// (APS_RASTER=units,heads: group sizes of the work order) for sweeps; the default build
// has none.
//
// Every mbarrier wait is bounded by a clock budget; a wait that runs out records
// a code in the plan's status word, tells the other warps through shared memory,
// and the CTA drains, frees its tensor memory and returns.

#include "attention_common.cuh"
#include "tensor_maps.cuh"

#include <cuda.h>
#include <stdlib.h>
#include <string.h>
#include <type_traits>

namespace aps {
namespace {

constexpr int kBM = 128;          // token rows per tile (per CTA)
constexpr int kBN = 256;          // K_h | V_h columns
constexpr int kHeadDim = 128;      // columns of K (and of V) in one tile: one head of 128, two of 64, four of 32
constexpr int kMaxHeadsPerTile = 4;
constexpr int kBKBytes = 128;     // one swizzle row = 64 two-byte elements
constexpr int kABytes = kBM * kBKBytes;          // 16 KB
constexpr int kSubRows = 16;                     // rows per TMA box of the hidden cache
constexpr int kSubBytes = kSubRows * kBKBytes;   // 2 KB
constexpr int kSubsPerTile = kBM / kSubRows;     // 8
constexpr int kThreads = 320;          // warps 0 and 6-9 TMA producers, 1 MMA issue, 2-5 epilogue
constexpr int kStages = 6;
constexpr int kBBytes = kBN / 2 * kBKBytes;      // 16 KB: this CTA's half of the W rows
constexpr int kStageBytes = kABytes + kBBytes;   // 32 KB
constexpr long long kWaitBudget = 4000000000LL;  // clock cycles (~2 s) before a wait gives up

struct SmemAux {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  // epilogue scratch.  A tile can hold rows of several requests: a SEGMENT is a run of
  // sub-blocks of one request; everything below is kept per sub-block or per segment.
  int2 sub_rec[kSubsPerTile];          // (request, first token) of each sub-block, (-1, 0) = none
  int sub_seg[kSubsPerTile];           // segment of each sub-block, -1 = none
  int seg_req[kSubsPerTile];           // request of each segment
  int n_seg;
  alignas(16) float q[kSubsPerTile][kHeadDim];   // per segment: query row of its request, pre-scaled
  float bk[kHeadDim];
  float bv[kHeadDim];
  float sub_max[kMaxHeadsPerTile][kSubsPerTile];   // per head of the tile (head sizes 64 / 32: 2 / 4 heads)
  float sub_sum[kMaxHeadsPerTile][kSubsPerTile];
  alignas(16) float red_acc[kSubsPerTile][kHeadDim];   // written as float2
};

constexpr size_t smem_bytes() {
  return 1024 /*alignment slack*/ + (size_t)kStages * kStageBytes + sizeof(SmemAux);
}

// ---- PTX wrappers --------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_addr(uint32_t bar_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_addr(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
// Arrive on a barrier given by its shared::cluster address (own CTA or the peer).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_addr(uint32_t bar_addr, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar_addr), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when it gave up (or another warp already did): the code goes
// to the CTA's abort flag and, first come first served, to the status word in global memory.
__device__ __forceinline__ bool mbar_wait_addr(uint32_t bar_addr, uint32_t parity, volatile int* abort_flag,
                                               int* status, int code, long long budget = kWaitBudget) {
  if (mbar_try_wait_addr(bar_addr, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait_addr(bar_addr, parity)) {
    if ((++spins & 255) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > budget) {
        *abort_flag = code;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  return mbar_wait_addr(smem_u32(bar), parity, abort_flag, status, code);
}
// The same for a whole converged warp: every lane tests the barrier once; if that fails
// lane 0 does the bounded wait and the others take its verdict.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar_addr, uint32_t parity, volatile int* abort_flag,
                                               int* status, int code, int lane) {
  if (__all_sync(0xffffffffu, mbar_try_wait_addr(bar_addr, parity))) return true;
  const bool got = lane != 0 || mbar_wait_addr(bar_addr, parity, abort_flag, status, code);
  return __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank`.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Tensor copy (TMA): a box of the tensor map lands in this CTA's shared memory, the bytes
// are counted on an mbarrier of the even CTA of the pair (given as a shared::cluster address).
// Destination and barrier are 32-bit shared addresses.  No multicast: one destination CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map,
                                            uint32_t bar_cluster_addr, int x, int y, uint64_t l2_policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(l2_policy) : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The barrier is named by a shared::cluster address (own CTA or peer).
__device__ __forceinline__ void tc_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// One M256 N256 K16 instruction of the CTA pair.  The operand descriptors are given as 32-bit
// halves (the high half is common to both operands): the issuing thread steps a descriptor
// with one 32-bit add.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier over the 128 epilogue threads that also ANDs a per-thread flag, so that
// all of them take the same decision after a bounded wait.
__device__ __forceinline__ bool epi_all(bool flag) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out) : "r"((uint32_t)flag) : "memory");
  return out != 0;
}

// Shared-memory operand descriptor of a K-major tile with 128-byte swizzle (rows of 128 bytes,
// 8-row groups 1024 bytes apart): low half = (address >> 4) | version 1 in bit 16, high half =
// stride byte offset 1024 >> 4, bit 14, layout type 2 (SWIZZLE_128B) in bits 29-31.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
}

// kind::f16 instruction descriptor: fp32 accumulate, A/B format fmt (0 = f16,
// 1 = bf16), both K-major, N = 256, M = m (128 for one CTA, 256 for a pair).
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, uint32_t m) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((kBN >> 3) << 17) | ((m >> 4) << 24);
}

// ---- work items -----------------------------------------------------------------
enum { kModeAttend = 0, kModeStore = 1 };

struct HiddenParams {
  // attend mode
  int* plan;
  const int* part_offset;
  const int2* hid_subs;       // per 16-row sub-block of the M tiles: (request, first token) / (-1, 0)
  const int* first_tile;      // [batch] first M tile a hidden request has rows in
  const int* hid_rows;        // per sub-block: its first row in the hidden cache
  float* part_ml;
  float* part_acc;
  const void* query;
  const int32_t* block_tables;
  const int32_t* seq_lens;
  int max_blocks_per_seq;
  int block_size;
  int64_t query_stride;
  float scale_log2;
  // store mode
  void* kv_out;
  const int32_t* block_ids;   // 16-row block ids of X, or nullptr for identity
  int64_t n_rows;
  int64_t kv_stride;
  int n_store_tiles;
  // common
  const void* b_k;
  const void* b_v;
  int heads;
  int k_slabs;                // ceil(hidden_size / 64)
  int raster_units;           // units per group of the work order (see item_of)
  int raster_heads;           // heads per group of the work order
  int dense_a;                // X rows of a tile are contiguous: map_x has a 128-row box
  int* status;
};

struct Item {
  int unit, head;     // unit = a pair of M tiles (2u, 2u + 1)
  bool last_head;     // the block's last head: the unit's hidden rows are not read again in this head group
};

// Work order.  Heads are taken in groups of `rh`; inside a head group the units (tile
// pairs) are taken in groups of `ru`; inside such a block the order is head-major.
// While a head group is being worked on its W rows (rh x 2 x 128 x E elements) stay hot in
// L2 across all unit groups, and the hidden rows of a unit group are fetched from HBM once
// per head group and reused from L2 by the group's other heads.
__device__ __forceinline__ Item item_of(int i, int n_units, int heads, int ru, int rh) {
  const int per_hg = n_units * rh;
  const int hg = i / per_hg;
  const int rem = i - hg * per_hg;
  const int hsz = min(rh, heads - hg * rh);
  const int per_block = ru * hsz;
  const int ug = rem / per_block;
  const int within = rem - ug * per_block;
  const int gm = min(ru, n_units - ug * ru);
  const int hl = within / gm;
  Item it;
  it.head = hg * rh + hl;
  it.unit = ug * ru + within - hl * gm;
  it.last_head = hl == hsz - 1;
  return it;
}

// Number of 16-row sub-blocks of M tile `tile` that hold rows (they are always the leading
// ones; 0 when the tile does not exist).
template <int MODE>
__device__ __forceinline__ int tile_n_sub(const HiddenParams& p, int tile, int n_tiles) {
  if (tile >= n_tiles) return 0;
  if (MODE == kModeAttend) {
    const int4* rec = reinterpret_cast<const int4*>(p.hid_subs + (int64_t)tile * kSubsPerTile);
    int n = 0;
#pragma unroll
    for (int j = 0; j < kSubsPerTile / 2; ++j) {
      const int4 r = rec[j];   // two (request, first token) records
      n += (r.x >= 0) + (r.z >= 0);
    }
    return n;
  }
  const int valid = (int)min((int64_t)kBM, p.n_rows - (int64_t)tile * kBM);
  return (valid + kSubRows - 1) / kSubRows;
}

// First hidden-cache row of each of the tile's leading n_sub sub-blocks.
template <int MODE>
__device__ __forceinline__ void tile_sub_rows(const HiddenParams& p, int tile, int n_sub, int* sub_row) {
  if (MODE == kModeAttend) {
#pragma unroll
    for (int j = 0; j < kSubsPerTile; ++j) {
      // resolved through the block tables by the plan kernel
      sub_row[j] = j < n_sub ? p.hid_rows[(int64_t)tile * kSubsPerTile + j] : 0;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kSubsPerTile; ++j) {
      if (j < n_sub)
        sub_row[j] = p.block_ids ? p.block_ids[tile * kSubsPerTile + j] * kSubRows
                                 : tile * kBM + j * kSubRows;
      else
        sub_row[j] = 0;
    }
  }
}

// Column sum inside each 16-lane half of the warp: on return v[0], v[1] of a lane hold,
// for columns 2*(lane%16) and 2*(lane%16)+1, the sum over the 16 lanes of its half.
__device__ __forceinline__ void half_warp_column_sum(float* v, int lane) {
#pragma unroll
  for (int step = 0; step < 4; ++step) {
    const int off = 8 >> step, half = 16 >> step;
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? v[i] : v[i + half];
      const float keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
}

// ---- epilogue (the 128 threads of warps 2..5) --------------------------------------
// Before the accumulator is ready: find the tile's segments, stage the query row of every
// segment's request (attend mode) and the biases of head `head`.
template <typename T, int MODE>
__device__ __forceinline__ void epilogue_stage_inputs(SmemAux* aux, const HiddenParams& p, int tile,
                                                      bool tile_ok, int head, int et) {
  const int hcol = head * kHeadDim;
  const T* bk = static_cast<const T*>(p.b_k);
  const T* bv = static_cast<const T*>(p.b_v);
  aux->bk[et] = bk ? Elem<T>::to_float(bk[hcol + et]) : 0.f;
  aux->bv[et] = bv ? Elem<T>::to_float(bv[hcol + et]) : 0.f;
  if (MODE == kModeAttend) {
    if (et < kSubsPerTile)
      aux->sub_rec[et] = tile_ok ? p.hid_subs[(int64_t)tile * kSubsPerTile + et] : make_int2(-1, 0);
    epi_barrier();
    if (et == 0) {
      int n = 0;
      for (int j = 0; j < kSubsPerTile; ++j) {
        const int r = aux->sub_rec[j].x;
        if (r < 0) { aux->sub_seg[j] = -1; continue; }
        if (n == 0 || aux->seg_req[n - 1] != r || aux->sub_seg[j - 1] < 0) aux->seg_req[n++] = r;
        aux->sub_seg[j] = n - 1;
      }
      aux->n_seg = n;
    }
    epi_barrier();
    const int n_seg = aux->n_seg;
    for (int sgm = 0; sgm < n_seg; ++sgm) {
      const T* q = static_cast<const T*>(p.query) + aux->seg_req[sgm] * p.query_stride + hcol;
      aux->q[sgm][et] = Elem<T>::to_float(q[et]) * p.scale_log2;
    }
  }
  epi_barrier();
}

// After the accumulator is ready.  `release()` is called once, when this thread's
// last TMEM read has completed.
template <typename T, int MODE, int NH, typename Release>
__device__ __forceinline__ void epilogue_compute(SmemAux* aux, const HiddenParams& p, uint32_t t_row,
                                                 int tile, bool tile_ok, int head, int quarter,
                                                 int lane, int et, Release release) {
  // `head` counts tiles of 128 K columns: NH heads of 128 / NH elements each, adjacent in W
  // and in the query row, so that the loads and the accumulator look the same for every NH.
  constexpr int kD = kHeadDim / NH;       // head size
  constexpr int kChunks = 4 / NH;         // 32-column TMEM chunks per head
  const int row = quarter * 32 + lane;
  const int hcol = head * kHeadDim;
  uint32_t r[32];

  if (MODE == kModeStore) {
    const int64_t out_row = (int64_t)tile * kBM + row;
    const bool valid = tile_ok && out_row < p.n_rows;
    T* dst_k = static_cast<T*>(p.kv_out) + out_row * p.kv_stride + hcol;
    T* dst_v = dst_k + (int64_t)p.heads * kHeadDim;
#pragma unroll 1
    for (int c = 0; c < 8; ++c) {
      tmem_ld32(t_row + c * 32, r);
      tmem_ld_wait();
      const float* bias = c < 4 ? aux->bk : aux->bv;
      T* dst = (c < 4 ? dst_k : dst_v) + (c & 3) * 32;
      if (valid) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          T tmp[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            tmp[e] = Elem<T>::from_float(__uint_as_float(r[j + e]) + bias[(c & 3) * 32 + j + e]);
          *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(tmp);
        }
      }
    }
    release();
    epi_barrier();  // the bias buffers are rewritten by the next item
    return;
  }

  // this thread's row: sub-block `sub` of the tile, row `row % 16` of it
  const int sub = row >> 4;
  const int2 rec = aux->sub_rec[sub];
  const int my_seg = aux->sub_seg[sub];
  bool valid = false;
  if (my_seg >= 0) {
    const int seq = min(p.seq_lens[rec.x], p.max_blocks_per_seq * p.block_size);
    valid = rec.y + (row & 15) < seq;
  }
  const float* qs = aux->q[my_seg >= 0 ? my_seg : 0];
  // ---- scores: s = q . (K_row + b_k) per head, already in the log2 domain ----
  float s[NH];
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    float acc = 0.f;
#pragma unroll 1
    for (int c = h * kChunks; c < (h + 1) * kChunks; ++c) {
      tmem_ld32(t_row + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        acc = fmaf(qs[c * 32 + j], __uint_as_float(r[j]) + aux->bk[c * 32 + j], acc);
    }
    s[h] = valid ? acc : -INFINITY;
    // max over the 16 rows of the sub-block
    float hm = s[h];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) hm = fmaxf(hm, __shfl_xor_sync(0xffffffffu, hm, o));
    if ((lane & 15) == 0) aux->sub_max[h][sub] = hm;
  }
  epi_barrier();
  float pr[NH];
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    // max over the sub-blocks of the segment
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kSubsPerTile; ++j)
      if (aux->sub_seg[j] == my_seg) mx = fmaxf(mx, aux->sub_max[h][j]);
    pr[h] = valid ? exp2f(s[h] - mx) : 0.f;
    float hs = pr[h];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) hs += __shfl_xor_sync(0xffffffffu, hs, o);
    if ((lane & 15) == 0) aux->sub_sum[h][sub] = hs;
  }

  // ---- weighted V rows, column sums over the 16 rows of the sub-block ----
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    const float w = pr[h];
#pragma unroll 1
    for (int c = h * kChunks; c < (h + 1) * kChunks; ++c) {
      tmem_ld32(t_row + kHeadDim + c * 32, r);
      tmem_ld_wait();
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j)
        v[j] = valid ? w * (__uint_as_float(r[j]) + aux->bv[c * 32 + j]) : 0.f;
      half_warp_column_sum(v, lane);
      *reinterpret_cast<float2*>(&aux->red_acc[sub][c * 32 + 2 * (lane & 15)]) = make_float2(v[0], v[1]);
    }
  }
  release();
  epi_barrier();
  // ---- one partial per segment and head: thread et owns column et of the tile ----
  const int n_seg = aux->n_seg;
  const int my_h = et / kD;
  for (int sgm = 0; sgm < n_seg; ++sgm) {
    float a = 0.f, m_seg = -INFINITY, l_seg = 0.f;
#pragma unroll
    for (int j = 0; j < kSubsPerTile; ++j)
      if (aux->sub_seg[j] == sgm) {
        a += aux->red_acc[j][et];
        m_seg = fmaxf(m_seg, aux->sub_max[my_h][j]);
        l_seg += aux->sub_sum[my_h][j];
      }
    const int req = aux->seg_req[sgm];
    // partial slots are laid out [slot][head][head size]; p.heads counts tiles of NH heads
    const int64_t slot = (int64_t)(p.part_offset[req] + tile - p.first_tile[req]) * p.heads + head;
    p.part_acc[slot * kHeadDim + et] = a;
    if (et % kD == 0) *reinterpret_cast<float2*>(p.part_ml + (slot * NH + my_h) * 2) = make_float2(m_seg, l_seg);
  }
  epi_barrier();  // the segment tables and reduction buffers are rewritten by the next item
}

// ---- TMA producer role -----------------------------------------------------------
// Issuing one tensor copy costs the issuing thread on the order of a hundred cycles
// whatever the size of the box, and a paged tile needs eight 16-row boxes plus the W
// box per 64-element slab: one thread cannot issue them within the 512 cycles the
// tensor cores need for the slab.  So the boxes of a stage are split over five producer
// threads in five warps.  Producer 0 (warp 0) posts the stage's byte count and issues the
// W box (and the one 128-row box of a dense X tile); producers 1..4 (warps 6..9) own two
// fixed block slots of the tile each, so a producer's loop holds at most two copy
// instructions (a copy that is predicated off still costs the thread some twenty cycles).
// Every producer waits for the stage to be free on its own.  Like the MMA issuer, a producer
// is one thread with a few hundred cycles per slab: addresses are stepped, not recomputed
// from the stage index.
template <typename T, int MODE>
__device__ __forceinline__ void tma_producer(const HiddenParams& p, SmemAux* aux, uint8_t* smem,
                                             const CUtensorMap& map_x, const CUtensorMap& map_wk,
                                             const CUtensorMap& map_wv, int prod, int n_tiles,
                                             int n_units, int n_items, int first, int stride,
                                             uint32_t rank) {
  volatile int* abort_flag = &aux->abort_flag;
  const bool leader = rank == 0;
  const bool dense = p.dense_a != 0;
  uint32_t stage = 0, phase = 0;
  bool ok = true;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full_base = smem_u32(&aux->full[0]);
  const uint32_t empty_base = smem_u32(&aux->empty[0]);
  const uint32_t bar_first = mapa_u32(full_base, 0);   // where the bytes are counted: the even CTA
  const int j0 = prod > 0 ? (prod - 1) * 2 : kSubsPerTile;   // producer 0 owns no block slot
  const uint32_t sub_off = (uint32_t)(j0 * kSubBytes);
  const CUtensorMap* w_map = leader ? &map_wk : &map_wv;
  // L2 eviction priorities.  The W rows of the head group being worked on are re-read by every
  // round of items and are asked to stay (evict_last: -1.6 % time on configuration 2).  The
  // hidden rows keep the normal priority while the block's other heads still have to read them
  // and are marked evict_first on their last read of the head group (the block's last head):
  // -10 % DRAM traffic at the same time.  Marking every read of them evict_first evicted them
  // before the other heads had read them (+2 % time).
  const uint64_t pol_w = l2_policy_evict_last(), pol_normal = l2_policy_evict_normal();
  const uint64_t pol_first = l2_policy_evict_first();
  for (int i = first; i < n_items && ok; i += stride) {
    const Item it = item_of(i, n_units, p.heads, p.raster_units, p.raster_heads);
    const int tile = it.unit * 2 + (int)rank;
    const int n_sub = tile_n_sub<MODE>(p, tile, n_tiles);
    const uint64_t pol_x = it.last_head ? pol_first : pol_normal;
    int sub_row[kSubsPerTile];
    tile_sub_rows<MODE>(p, n_sub > 0 ? tile : 0, n_sub, sub_row);
    // a dense X tile is one 128-row box (rows past the end are zero-filled and still
    // counted); a paged tile is one 16-row box per cache block in use
    uint32_t tx_bytes = (uint32_t)((dense ? (n_sub > 0 ? kABytes : 0) : n_sub * kSubBytes) + kBBytes);
    if (leader) {
      const int peer_sub = tile_n_sub<MODE>(p, tile + 1, n_tiles);
      tx_bytes += (uint32_t)((dense ? (peer_sub > 0 ? kABytes : 0) : peer_sub * kSubBytes) + kBBytes);
    }
    const bool do_w = prod == 0;
    const bool do_dense = dense && prod == 0 && n_sub > 0;
    const bool post = prod == 0 && leader;            // posts the stage's byte count
    const int hrow = it.head * kHeadDim;
    int r0 = 0, r1 = 0;
#pragma unroll
    for (int j = 0; j < kSubsPerTile; ++j) { if (j == j0) r0 = sub_row[j]; if (j == j0 + 1) r1 = sub_row[j]; }
    const bool has0 = !dense && j0 < n_sub, has1 = !dense && j0 + 1 < n_sub;
    uint32_t a_dst = smem_base + stage * kStageBytes, off8 = stage * 8;
    int x = 0;
    for (int ks = p.k_slabs; ks > 0; --ks) {
      if (!mbar_wait_addr(empty_base + off8, phase ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
      const uint32_t b_dst = a_dst + kABytes;
      const uint32_t bar = bar_first + off8;
      if (post) mbar_expect_tx_addr(full_base + off8, tx_bytes);
      if (do_dense) tma_load_2d(a_dst, &map_x, bar, x, tile * kBM, pol_x);
      if (has0) tma_load_2d(a_dst + sub_off, &map_x, bar, x, r0, pol_x);
      if (has1) tma_load_2d(a_dst + sub_off + kSubBytes, &map_x, bar, x, r1, pol_x);
      if (prod != 0) mbar_arrive_addr(full_base + off8);
      else if (!leader && !mbar_wait_addr(full_base + off8, phase, abort_flag, p.status, 6)) { ok = false; break; }
      if (do_w) tma_load_2d(b_dst, w_map, bar, x, hrow, pol_w);
      x += kBKBytes / (int)sizeof(T);
      a_dst += kStageBytes; off8 += 8;
      if (++stage == kStages) { stage = 0; phase ^= 1; a_dst = smem_base; off8 = 0; }
    }
  }
  if (!ok) {
    // another role gave up: let copies that are still in flight land (bounded)
    // before the CTA's shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
  }
}

// ---- the kernel ---------------------------------------------------------------------
template <typename T, int MODE, int NH>
__global__ void __launch_bounds__(kThreads, 1)
hidden_path_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wk,
                   const __grid_constant__ CUtensorMap map_wv, const HiddenParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemAux* aux = reinterpret_cast<SmemAux*>(smem + (size_t)kStages * kStageBytes);
  // the warp index is broadcast from lane 0 so that the compiler can tell that the role
  // branches below are uniform across a warp
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const long long kernel_begin = clock64();
  volatile int* abort_flag = &aux->abort_flag;
  const uint32_t rank = cluster_ctarank();   // position in the CTA pair
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    // full[s] of the even CTA: one arrival from its producer 0 (with the byte count of both
    // CTAs' boxes) plus one per slab from each of its producers 1..4.  The last are what keeps
    // a producer without boxes in this tile in step: a stage cannot fill, be consumed and be
    // freed again behind the back of a producer that is still waiting for it (a parity wait
    // that is lapped twice never returns).  In the odd CTA, whose bytes are counted on the even
    // CTA's barrier, full[s] takes only those four arrivals and its producer 0 waits for them
    // before it issues the stage's W box (an arrival on the peer's barrier per slab and
    // producer costs ~2000 cycles).
    const uint32_t full_count = leader ? 5u : 4u;
    for (int s = 0; s < kStages; ++s) { mbar_init(&aux->full[s], full_count); mbar_init(&aux->empty[s], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&aux->acc_full[b], 1);
      mbar_init(&aux->acc_empty[b], 8);   // one arrival per epilogue warp of both CTAs
    }
    aux->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&aux->tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = aux->tmem_base;

  const int n_tiles = MODE == kModeAttend ? p.plan[kPlanNumHidTiles] : p.n_store_tiles;
  const int n_units = (n_tiles + 1) / 2;
  const int n_items = n_units * p.heads;
  const int first = (int)(blockIdx.x >> 1);
  const int stride = (int)(gridDim.x >> 1);

  if (warp == 0) {
    // ===================== TMA producer 0 =====================
    if (lane == 0)
      tma_producer<T, MODE>(p, aux, smem, map_x, map_wk, map_wv, 0, n_tiles, n_units, n_items, first, stride, rank);
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer (the even CTA issues for both) =====================
    if (leader) {
      // The whole warp runs the loop (waits, address stepping) in step and one elected lane
      // issues the tensor-core instructions: their operands are then warp-uniform values the
      // compiler can keep in uniform registers.  The issuer has 512 cycles per slab and a
      // lone warp issues an instruction only every few cycles, so everything the loop needs
      // is a 32-bit register stepped by a constant (barrier addresses, the low halves of the
      // two operand descriptors) and nothing is recomputed from the stage index.
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc = instr_desc(fmt, 256u);
      constexpr uint32_t kDescStep = (uint32_t)kStageBytes >> 4, kDescB = (uint32_t)kABytes >> 4;
      const uint32_t a_lo_first = smem_desc_lo(smem_u32(smem));
      const uint32_t full_first = smem_u32(&aux->full[0]), full_end = full_first + kStages * 8;
      const uint32_t empty_own = mapa_u32(smem_u32(&aux->empty[0]), 0);
      const uint32_t peer_delta = mapa_u32(smem_u32(&aux->empty[0]), 1) - empty_own;
      uint32_t a_lo = a_lo_first, full_addr = full_first, empty_addr = empty_own, phase = 0, n_local = 0;
      bool ok = true;
      for (int i = first; i < n_items && ok; i += stride, ++n_local) {
        const uint32_t buf = n_local & 1u, use = n_local >> 1;
        if (!mbar_wait_warp(smem_u32(&aux->acc_empty[buf]), (use & 1u) ^ 1u, abort_flag, p.status, 2, lane)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kBN;
        uint32_t accumulate = 0;
        for (int ks = p.k_slabs; ks > 0; --ks) {
          if (!mbar_wait_warp(full_addr, phase, abort_flag, p.status, 3, lane)) { ok = false; break; }
          tc_fence_after();
          if (elect_one()) {
            const uint32_t b_lo = a_lo + kDescB;
            tc_mma_f16(d_tmem, a_lo, b_lo, kDescHi, idesc, accumulate);
            tc_mma_f16(d_tmem, a_lo + 2, b_lo + 2, kDescHi, idesc, 1u);
            tc_mma_f16(d_tmem, a_lo + 4, b_lo + 4, kDescHi, idesc, 1u);
            tc_mma_f16(d_tmem, a_lo + 6, b_lo + 6, kDescHi, idesc, 1u);
            tc_commit(empty_addr);                 // release the stage in both CTAs
            tc_commit(empty_addr + peer_delta);
          }
          __syncwarp();
          accumulate = 1u;
          a_lo += kDescStep; full_addr += 8; empty_addr += 8;
          if (full_addr == full_end) {
            a_lo = a_lo_first; full_addr = full_first; empty_addr = empty_own; phase ^= 1u;
          }
        }
        if (ok && elect_one()) {
          const uint32_t f = smem_u32(&aux->acc_full[buf]);
          tc_commit(mapa_u32(f, 0));
          tc_commit(mapa_u32(f, 1));
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ===================== TMA producers 1..4 (warps 6..9) =====================
    if (lane == 0)
      tma_producer<T, MODE>(p, aux, smem, map_x, map_wk, map_wv, warp - 5, n_tiles, n_units, n_items, first, stride, rank);
    __syncwarp();
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int quarter = warp & 3;               // TMEM lanes this warp may read
    const int et = threadIdx.x - 64;            // 0..127
    uint32_t n_local = 0;
    bool ok = true;
    for (int i = first; i < n_items && ok; i += stride, ++n_local) {
      const Item it = item_of(i, n_units, p.heads, p.raster_units, p.raster_heads);
      const int tile = it.unit * 2 + (int)rank;
      const bool tile_ok = tile < n_tiles;
      const uint32_t buf = n_local & 1u, use = n_local >> 1;
      epilogue_stage_inputs<T, MODE>(aux, p, tile, tile_ok, it.head, et);
      // one lane per warp polls the barrier; the other 124 threads wait in the hardware
      // barrier of epi_all (polling by every thread floods the SM's mbarrier unit and slows
      // the producer / MMA handshake down)
      const bool got = lane != 0 || mbar_wait(&aux->acc_full[buf], use & 1u, abort_flag, p.status, 4);
      if (!epi_all(got)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * kBN;
      uint64_t* acc_empty = &aux->acc_empty[buf];
      auto release = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(acc_empty), 0));
      };
      epilogue_compute<T, MODE, NH>(aux, p, t_row, tile, tile_ok, it.head, quarter, lane, et, release);
    }
  }

  tc_fence_before();
  __syncthreads();
  // SM cycles CTA 0 spent in the kernel (always recorded: two clock reads per launch)
  if (MODE == kModeAttend && blockIdx.x == 0 && threadIdx.x == 0)
    reinterpret_cast<unsigned long long*>(p.plan + kPlanStatsWord)[8] = (unsigned long long)(clock64() - kernel_begin);
  cluster_sync_all();   // nobody leaves while the peer may still read its memory or signal it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// A bounded wait that runs out, on purpose and harmlessly: one thread waits on an mbarrier
// nobody ever arrives on, for `budget` clock cycles, then records `code` in the status word
// like the waits of hidden_path_kernel do.  Used by the tests of the status handling.
__global__ void bounded_wait_selftest_kernel(int* status, long long budget, int code) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait_addr(smem_u32(&bar), 0, &abort_flag, status, code, budget);
  }
}

// ---- host side -----------------------------------------------------------------
// 2-D row-major matrix [rows, cols] of 2-byte elements, box [box_rows, 64 cols], 128-byte
// swizzle; encoded once per distinct (pointer, shape, stride, box) and kept (tensor_maps.cu).
int make_map(CUtensorMap* map, const void* base, int dtype, uint64_t cols, uint64_t rows,
             uint64_t row_stride_elems, uint32_t box_rows, const char* what) {
  TensorMapSpec spec{};
  spec.base = base; spec.dtype = dtype; spec.rank = 2;
  spec.dims[0] = cols; spec.dims[1] = rows;
  spec.strides_bytes[0] = row_stride_elems * 2;
  spec.box[0] = 64; spec.box[1] = box_rows;
  return cached_tensor_map(map, spec, what);
}

// Work-order group sizes (tile pairs x heads).  Every order costs the same cycles (the kernel is
// tensor-bound in all of them) and, at the power cap, the same time within a percent; what
// differs is how much of W and of the hidden rows L2 still holds when they are needed again, i.e.
// the DRAM traffic - and that differs more between GPUs than between orders (OPT-13B layer, ncu,
// same binary and inputs: 4 x 10 reads 7.6 GB per launch on one B200, 9.6 GB on a second, 13.0 GB
// on a third; 2 x 10 reads 5.8 GB on the first and 15.0 GB on the third).  About 60 MB of L2
// serve a working set that both dies read, and the live set here (the group's W rows, 26 MB, plus
// the rows of the tile pairs in flight, 20 - 30 MB) sits at that edge.  4 x 10 is the order all
// the published timings were taken with; orders with fewer heads per group (W smaller, rows
// re-read more often) or with all heads in one group (W no longer resident) read 1.5 - 2.5 x more.
void raster_sizes(int* units, int* heads) {
  *units = 4; *heads = 10;
#ifdef APS_TUNING
  const char* v = getenv("APS_RASTER");
  if (v != nullptr) {
    int a = 0, b = 0;
    if (sscanf(v, "%d,%d", &a, &b) == 2 && a > 0 && b > 0) { *units = a; *heads = b; }
  }
#endif
}

// Launch geometry: one CTA per SM, in pairs, as many pairs as the device keeps resident at
// once.  Looked up once per kernel instantiation and device (the library assumes one calling
// thread per process, like the reference's single-threaded worker).
template <typename T, int MODE, int NH>
int launch_hidden(const CUtensorMap& mx, const CUtensorMap& mk, const CUtensorMap& mv,
                  HiddenParams p, cudaStream_t stream) {
  static int grid_for_device[64] = {0};
  raster_sizes(&p.raster_units, &p.raster_heads);
  if (p.raster_heads > p.heads) p.raster_heads = p.heads;
  int dev = 0;
  APS_CUDA(cudaGetDevice(&dev));
  APS_REQUIRE(dev >= 0 && dev < 64, APS_ERR_CUDA, "device index %d out of range", dev);
  auto kernel = hidden_path_kernel<T, MODE, NH>;
  constexpr size_t smem = smem_bytes();
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (grid_for_device[dev] == 0) {
    APS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int sms = sm_count();
    cfg.gridDim = dim3((unsigned)(sms & ~1));
    int clusters = 0;
    APS_CUDA(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
    APS_REQUIRE(clusters > 0, APS_ERR_CUDA, "no CTA pair of the re-projection kernel fits on this device");
    grid_for_device[dev] = 2 * (clusters < sms / 2 ? clusters : sms / 2);
  }
  cfg.gridDim = dim3((unsigned)grid_for_device[dev]);
  {
    ScopedProfile prof(1, stream);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mx, mk, mv, p);
    if (e != cudaSuccess)
      return fail(APS_ERR_CUDA, "launch of hidden_path_kernel failed: %s", cudaGetErrorString(e));
  }
  return launch_status("hidden_path_kernel");
}

struct HiddenArgs {
  const void* hidden_cache; const void* w_k; const void* b_k; const void* w_v; const void* b_v;
  int heads, head_size, hidden_size;
  int64_t hidden_row_stride, num_hidden_rows, w_stride;
  int dtype;
};

// An accumulator tile holds 128 K columns and 128 V columns: one head of 128 elements, two
// adjacent heads of 64 or four of 32 (their W rows and their slices of the query row are
// adjacent, so only the softmax epilogue knows the difference).
bool tensor_head_shape_ok(int heads, int head_size) {
  return (head_size == 128 || head_size == 64 || head_size == 32) && heads > 0 &&
         (heads * head_size) % kHeadDim == 0;
}

int check_hidden_args(const char* op, const HiddenArgs& a) {
  APS_REQUIRE(a.dtype == APS_F16 || a.dtype == APS_BF16, APS_ERR_UNSUPPORTED,
              "%s: the tensor-core re-projection supports fp16 and bf16 only (dtype %d)", op, a.dtype);
  APS_REQUIRE(tensor_head_shape_ok(a.heads, a.head_size), APS_ERR_UNSUPPORTED,
              "%s: the tensor-core re-projection takes head sizes 128, 64 and 32 with heads x head size a "
              "multiple of 128 (got %d heads of %d)", op, a.heads, a.head_size);
  APS_REQUIRE(a.hidden_cache && a.w_k && a.w_v, APS_ERR_NULL_POINTER, "%s: null pointer", op);
  APS_REQUIRE(a.hidden_size > 0 && a.num_hidden_rows > 0 && a.hidden_row_stride >= a.hidden_size &&
                  a.w_stride >= a.hidden_size,
              APS_ERR_SHAPE, "%s: bad hidden sizes / strides", op);
  APS_REQUIRE(a.hidden_size % 8 == 0 && a.hidden_row_stride % 8 == 0 && a.w_stride % 8 == 0 &&
                  aligned_to(a.hidden_cache, 16) && aligned_to(a.w_k, 16) && aligned_to(a.w_v, 16),
              APS_ERR_MISALIGNED,
              "%s: hidden cache and weights must be 16-byte aligned with 16-byte row strides", op);
  return APS_OK;
}

int make_maps(const HiddenArgs& a, CUtensorMap* mx, CUtensorMap* mk, CUtensorMap* mv, bool dense_x = false) {
  int st;
  const uint64_t hd = (uint64_t)a.heads * a.head_size;
  if ((st = make_map(mx, a.hidden_cache, a.dtype, a.hidden_size, a.num_hidden_rows, a.hidden_row_stride,
                     dense_x ? kBM : kSubRows, "hidden cache")) != APS_OK) return st;
  if ((st = make_map(mk, a.w_k, a.dtype, a.hidden_size, hd, a.w_stride, kHeadDim, "W_k")) != APS_OK) return st;
  return make_map(mv, a.w_v, a.dtype, a.hidden_size, hd, a.w_stride, kHeadDim, "W_v");
}

}  // namespace

// The hybrid decode attention after its arguments have been checked: plan, K/V streaming,
// re-projection, combine, all on `cs`.
int enqueue_hybrid_attention(const HybridCall& c, cudaStream_t cs) {
  const AttnShape& s = c.shape;
  int st;
  HiddenArgs a{c.hidden_cache, c.w_k, c.b_k, c.w_v, c.b_v, s.heads, s.head_size, c.hidden_size,
               c.hidden_row_stride, c.num_hidden_rows, c.w_stride, s.dtype};
  // fp16 / bf16 run on the tensor cores (head sizes 128 / 64 / 32 with heads x head size a
  // multiple of 128); fp32 and the other head counts run the CUDA-core re-projection (same
  // partials, one request per tile)
  const bool tensor_path = (s.dtype == APS_F16 || s.dtype == APS_BF16) && tensor_head_shape_ok(s.heads, s.head_size);
  CUtensorMap mx, mk, mv;
  if (tensor_path) {
    if ((st = check_hidden_args("hybrid_decode_attention", a)) != APS_OK) return st;
    if ((st = make_maps(a, &mx, &mk, &mv)) != APS_OK) return st;
  } else {
    APS_REQUIRE(hidden_simt_supported(s.dtype, s.head_size), APS_ERR_UNSUPPORTED,
                "hybrid_decode_attention: head size %d / dtype %d has no re-projection kernel "
                "(tensor cores: fp16 or bf16, head sizes 32 / 64 / 128 with heads x head size a multiple "
                "of 128; CUDA cores: head sizes 32, 64, 128)",
                s.head_size, s.dtype);
    APS_REQUIRE(c.hidden_cache && c.w_k && c.w_v, APS_ERR_NULL_POINTER, "hybrid_decode_attention: null pointer");
    APS_REQUIRE(c.hidden_size > 0 && c.hidden_row_stride >= c.hidden_size && c.w_stride >= c.hidden_size,
                APS_ERR_SHAPE, "hybrid_decode_attention: bad hidden sizes / strides");
  }
  const WorkspaceLayout w = workspace_layout(s.batch, s.max_blocks_per_seq, s.block_size, s.heads, s.head_size);
  const WorkspacePtrs ws = workspace_ptrs(c.workspace, w);
  const bool have_kv = c.key_cache != nullptr && c.value_cache != nullptr;
  // the tensor-core kernel takes M tiles packed across requests, the CUDA-core kernel one
  // request per tile
  if ((st = launch_plan(ws, c.seq_lens, c.cache_type, c.block_tables, s.batch, s.max_blocks_per_seq,
                        s.block_size, tensor_path, have_kv, cs)) != APS_OK) return st;
  // K/V requests: on the call's stream before the re-projection kernel
  if (have_kv) {
    if ((st = launch_kv_attention(ws, c.query, c.key_cache, c.value_cache, c.block_tables, c.seq_lens, s, cs)) != APS_OK) return st;
  }
  if (!tensor_path) {
    SimtHiddenArgs sa{c.query, c.hidden_cache, c.w_k, c.b_k, c.w_v, c.b_v, c.block_tables, c.seq_lens,
                      s.max_blocks_per_seq, s.block_size, s.heads, s.head_size, c.hidden_size,
                      s.query_stride, c.hidden_row_stride, c.w_stride, s.scale, s.dtype};
    if ((st = launch_hidden_simt(ws, sa, cs)) != APS_OK) return st;
    return launch_combine(ws, c.out, c.seq_lens, s, cs);
  }
  HiddenParams p{};
  p.plan = ws.plan; p.part_offset = ws.part_offset; p.hid_subs = ws.hid_subs; p.first_tile = ws.first_tile; p.hid_rows = ws.hid_rows;
  p.part_ml = ws.part_ml; p.part_acc = ws.part_acc; p.query = c.query;
  p.block_tables = c.block_tables; p.seq_lens = c.seq_lens;
  p.max_blocks_per_seq = s.max_blocks_per_seq; p.block_size = s.block_size;
  p.query_stride = s.query_stride; p.scale_log2 = s.scale * 1.4426950408889634f;
  // the kernel counts tiles of 128 K columns where the caller counts heads
  p.b_k = c.b_k; p.b_v = c.b_v; p.heads = s.heads * s.head_size / kHeadDim; p.k_slabs = (c.hidden_size + 63) / 64;
  p.status = ws.plan + kPlanStatus;
  const bool bf16 = s.dtype == APS_BF16;
  switch (kHeadDim / s.head_size) {
    case 1: st = bf16 ? launch_hidden<__nv_bfloat16, kModeAttend, 1>(mx, mk, mv, p, cs)
                      : launch_hidden<__half, kModeAttend, 1>(mx, mk, mv, p, cs); break;
    case 2: st = bf16 ? launch_hidden<__nv_bfloat16, kModeAttend, 2>(mx, mk, mv, p, cs)
                      : launch_hidden<__half, kModeAttend, 2>(mx, mk, mv, p, cs); break;
    default: st = bf16 ? launch_hidden<__nv_bfloat16, kModeAttend, 4>(mx, mk, mv, p, cs)
                       : launch_hidden<__half, kModeAttend, 4>(mx, mk, mv, p, cs); break;
  }
  if (st != APS_OK) return st;
  return launch_combine(ws, c.out, c.seq_lens, s, cs);
}

int check_hybrid_call(const char* op, const HybridCall& c) {
  int st = check_attention_args(op, c.out, c.query, c.key_cache, c.value_cache, c.block_tables, c.seq_lens,
                                c.shape, c.workspace, c.workspace_bytes, false);
  if (st != APS_OK || c.shape.batch == 0) return st;
  APS_REQUIRE(c.cache_type != nullptr, APS_ERR_NULL_POINTER, "%s: cache_type is null", op);
  APS_REQUIRE((c.key_cache == nullptr) == (c.value_cache == nullptr), APS_ERR_NULL_POINTER,
              "%s: key_cache and value_cache must both be given or both be NULL", op);
  return APS_OK;
}

}  // namespace aps

using namespace aps;

extern "C" int aps_hybrid_decode_attention(void* out, const void* query, const void* key_cache,
                                           const void* value_cache, const void* hidden_cache,
                                           const void* w_k, const void* b_k, const void* w_v,
                                           const void* b_v, const int32_t* block_tables,
                                           const int32_t* seq_lens, const int32_t* cache_type,
                                           int batch, int max_blocks_per_seq, int num_heads,
                                           int head_size, int hidden_size, int block_size,
                                           int64_t query_stride, int64_t out_stride,
                                           int64_t block_stride, int64_t hidden_row_stride,
                                           int64_t num_hidden_rows, int64_t w_stride, float scale,
                                           void* workspace, size_t workspace_bytes, int dtype,
                                           void* stream) {
  HybridCall c{};
  c.shape = AttnShape{batch, max_blocks_per_seq, num_heads, head_size, block_size,
                      query_stride, out_stride, block_stride, scale, dtype};
  c.out = out; c.query = query; c.key_cache = key_cache; c.value_cache = value_cache;
  c.hidden_cache = hidden_cache; c.w_k = w_k; c.b_k = b_k; c.w_v = w_v; c.b_v = b_v;
  c.block_tables = block_tables; c.seq_lens = seq_lens; c.cache_type = cache_type;
  c.hidden_size = hidden_size; c.hidden_row_stride = hidden_row_stride;
  c.num_hidden_rows = num_hidden_rows; c.w_stride = w_stride;
  c.workspace = workspace; c.workspace_bytes = workspace_bytes;
  int st = check_hybrid_call("hybrid_decode_attention", c);
  if (st != APS_OK || batch == 0) return st;
  return enqueue_hybrid_attention(c, (cudaStream_t)stream);
}

extern "C" int aps_kv_reprojection(void* kv, const void* x, const int32_t* block_ids, int64_t n_rows,
                                   const void* w_k, const void* b_k, const void* w_v, const void* b_v,
                                   int num_heads, int head_size, int hidden_size, int64_t x_row_stride,
                                   int64_t num_x_rows, int64_t w_stride, int64_t kv_stride, int dtype,
                                   int* status_word, void* stream) {
  APS_REQUIRE(n_rows >= 0 && num_heads > 0, APS_ERR_SHAPE, "kv_reprojection: bad sizes");
  if (n_rows == 0) return APS_OK;
  APS_REQUIRE(kv != nullptr, APS_ERR_NULL_POINTER, "kv_reprojection: null pointer");
  HiddenArgs a{x, w_k, b_k, w_v, b_v, num_heads, head_size, hidden_size, x_row_stride, num_x_rows, w_stride, dtype};
  int st;
  if ((st = check_hidden_args("kv_reprojection", a)) != APS_OK) return st;
  APS_REQUIRE(kv_stride >= 2LL * num_heads * head_size && kv_stride % 8 == 0 && aligned_to(kv, 16),
              APS_ERR_MISALIGNED, "kv_reprojection: output must be 16-byte aligned with a 16-byte row stride");
  APS_REQUIRE((n_rows + kBM - 1) / kBM < (1LL << 24), APS_ERR_SHAPE, "kv_reprojection: too many rows");
  CUtensorMap mx, mk, mv;
  const bool dense = block_ids == nullptr;   // contiguous X rows: one 128-row box per tile
  if ((st = make_maps(a, &mx, &mk, &mv, dense)) != APS_OK) return st;
  HiddenParams p{};
  p.dense_a = dense ? 1 : 0;
  p.kv_out = kv; p.block_ids = block_ids; p.n_rows = n_rows; p.kv_stride = kv_stride;
  p.n_store_tiles = (int)((n_rows + kBM - 1) / kBM);
  // stored K | V rows are head-major, so heads smaller than 128 need nothing but the tile count
  p.b_k = b_k; p.b_v = b_v; p.heads = num_heads * head_size / kHeadDim; p.k_slabs = (hidden_size + 63) / 64;
  p.status = status_word;
  cudaStream_t cs = (cudaStream_t)stream;
  return dtype == APS_BF16 ? launch_hidden<__nv_bfloat16, kModeStore, 1>(mx, mk, mv, p, cs)
                           : launch_hidden<__half, kModeStore, 1>(mx, mk, mv, p, cs);
}

extern "C" int aps_selftest_bounded_wait(void* workspace, size_t workspace_bytes, long long budget_cycles,
                                         void* out, int batch, int max_blocks_per_seq, int num_heads,
                                         int head_size, int block_size, int64_t out_stride, int dtype,
                                         void* stream) {
  APS_REQUIRE(workspace != nullptr && out != nullptr, APS_ERR_NULL_POINTER, "selftest_bounded_wait: null pointer");
  APS_REQUIRE(budget_cycles > 0 && budget_cycles <= 100000000LL, APS_ERR_SHAPE,
              "selftest_bounded_wait: the budget must be between 1 and 1e8 clock cycles");
  APS_REQUIRE(batch > 0 && max_blocks_per_seq > 0 && num_heads > 0 && head_size > 0 && block_size > 0,
              APS_ERR_SHAPE, "selftest_bounded_wait: bad sizes");
  const WorkspaceLayout w = workspace_layout(batch, max_blocks_per_seq, block_size, num_heads, head_size);
  APS_REQUIRE(aligned_to(workspace, 256) && workspace_bytes >= w.total, APS_ERR_WORKSPACE,
              "selftest_bounded_wait: workspace too small for this shape");
  const WorkspacePtrs ws = workspace_ptrs(workspace, w);
  cudaStream_t cs = (cudaStream_t)stream;
  bounded_wait_selftest_kernel<<<1, 32, 0, cs>>>(ws.plan + kPlanStatus, budget_cycles, kStatusWaitLast);
  int st = launch_status("bounded_wait_selftest_kernel");
  if (st != APS_OK) return st;
  AttnShape s{batch, max_blocks_per_seq, num_heads, head_size, block_size, 0, out_stride, 0, 1.f, dtype};
  return launch_combine(ws, out, nullptr, s, cs);
}

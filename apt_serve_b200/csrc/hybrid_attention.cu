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
// One work item = (M tile of 128 cached tokens of one hidden request, head h).
// The CTA computes the 128 x 256 tile [K_h | V_h] = X_tile * [W_k,h ; W_v,h]^T
// with fp32 accumulation in tensor memory:
//   warp 0    TMA producer: per 64-element slab of the hidden dimension, one
//             16-row box per cache block of the tile (hidden blocks are paged)
//             and two 128-row boxes of W_k / W_v rows of head h, 128-byte swizzle,
//             4-stage ring of 48 KB stages;
//   warp 1    tcgen05.mma issuer (M=128, N=256, K=16 per instruction, 4 per
//             slab), accumulators double-buffered in the 512 TMEM columns, so
//             the main loop of item i+1 overlaps the epilogue of item i;
//   warps 2-5 epilogue: one thread per token row reads its K row from TMEM, adds
//             b_k, dots with q (pre-scaled by scale*log2 e), block-wide max, then
//             reads its V row, weighs it and column-sums over the 128 rows with a
//             shuffle butterfly; the (max, sum, acc[128]) partial goes to scratch.
// CTAs are persistent (one per SM) and walk the items in a rasterised order that
// keeps 16 M tiles x ~9 heads in flight, so W_k|W_v slabs and hidden tiles are
// shared through L2.  No cluster launch and no multicast: every CTA fetches its
// own operands.
//
// Every mbarrier wait is bounded by a clock budget; a wait that runs out records
// a code in the plan's status word, tells the other warps through shared memory,
// and the CTA drains, frees its tensor memory and returns.

#include "attention_common.cuh"

#include <cuda.h>
#include <type_traits>

namespace aps {
namespace {

constexpr int kBM = 128;          // token rows per tile
constexpr int kBN = 256;          // K_h | V_h columns
constexpr int kHeadDim = 128;
constexpr int kBKBytes = 128;     // one swizzle row
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBKBytes;          // 16 KB
constexpr int kBBytes = kBN * kBKBytes;          // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;   // 48 KB
constexpr int kSubRows = 16;                     // rows per TMA box of the hidden cache
constexpr int kSubBytes = kSubRows * kBKBytes;   // 2 KB
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kRasterTiles = 16;                 // M tiles per raster group
constexpr long long kWaitBudget = 4000000000LL;  // clock cycles (~2 s) before a wait gives up

struct SmemAux {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float q[kHeadDim];
  float bk[kHeadDim];
  float bv[kHeadDim];
  float red_max[4];
  float red_sum[4];
  float red_acc[4][kHeadDim];
};

constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + (size_t)kStages * kStageBytes + sizeof(SmemAux);

// ---- PTX wrappers --------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when it gave up (or another warp already did).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > kWaitBudget) {
        *abort_flag = code;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
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

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups
// 1024 bytes apart (SBO), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// kind::f16 instruction descriptor: fp32 accumulate, A/B format fmt (0 = f16,
// 1 = bf16), both K-major, N = 256, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24);
}

// ---- work items -----------------------------------------------------------------
enum { kModeAttend = 0, kModeStore = 1 };

struct HiddenParams {
  // attend mode
  int* plan;
  const int* part_offset;
  const int2* hid_tiles;
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
  int* status;
};

struct Item { int tile, head; };

__device__ __forceinline__ Item item_of(int i, int n_tiles, int heads) {
  const int per_group = kRasterTiles * heads;
  const int g = i / per_group, within = i - g * per_group;
  const int gm = min(kRasterTiles, n_tiles - g * kRasterTiles);
  Item it;
  it.head = within / gm;
  it.tile = g * kRasterTiles + within - it.head * gm;
  return it;
}

// Butterfly column sum: on return v[0] of lane L holds the sum over the warp's
// 32 lanes of their v[L].
__device__ __forceinline__ void warp_column_sum(float* v, int lane) {
#pragma unroll
  for (int step = 0; step < 5; ++step) {
    const int off = 16 >> step;
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float send = upper ? v[i] : v[i + off];
      const float keep = upper ? v[i + off] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
}

template <typename T, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
hidden_path_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wk,
                   const __grid_constant__ CUtensorMap map_wv, const HiddenParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemAux* aux = reinterpret_cast<SmemAux*>(smem + (size_t)kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &aux->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&aux->full[s], 1); mbar_init(&aux->empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&aux->acc_full[b], 1); mbar_init(&aux->acc_empty[b], 4); }
    aux->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&aux->tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = aux->tmem_base;

  const int n_tiles = MODE == kModeAttend ? p.plan[kPlanNumHidTiles] : p.n_store_tiles;
  const int n_items = n_tiles * p.heads;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int i = blockIdx.x; i < n_items && ok; i += gridDim.x) {
        const Item it = item_of(i, n_tiles, p.heads);
        int n_sub;
        int sub_row[kBM / kSubRows];
        if (MODE == kModeAttend) {
          const int2 rc = p.hid_tiles[it.tile];
          const int seq = min(p.seq_lens[rc.x], p.max_blocks_per_seq * p.block_size);
          const int tok0 = rc.y * kBM;
          const int valid = min(kBM, seq - tok0);
          n_sub = (valid + kSubRows - 1) / kSubRows;
          const int32_t* bt = p.block_tables + (int64_t)rc.x * p.max_blocks_per_seq;
#pragma unroll
          for (int j = 0; j < kBM / kSubRows; ++j) {
            const int tok = tok0 + j * kSubRows;
            sub_row[j] = j < n_sub ? bt[tok / p.block_size] * p.block_size + tok % p.block_size : 0;
          }
        } else {
          const int64_t row0 = (int64_t)it.tile * kBM;
          const int valid = (int)min((int64_t)kBM, p.n_rows - row0);
          n_sub = (valid + kSubRows - 1) / kSubRows;
#pragma unroll
          for (int j = 0; j < kBM / kSubRows; ++j) {
            if (j < n_sub)
              sub_row[j] = p.block_ids ? p.block_ids[it.tile * (kBM / kSubRows) + j] * kSubRows
                                       : (int)(row0 + j * kSubRows);
            else
              sub_row[j] = 0;
          }
        }
        const uint32_t tx_bytes = (uint32_t)(n_sub * kSubBytes + kBBytes);
        for (int ks = 0; ks < p.k_slabs; ++ks) {
          if (!mbar_wait(&aux->empty[stage], phase ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          uint8_t* a_dst = smem + (size_t)stage * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          mbar_expect_tx(&aux->full[stage], tx_bytes);
          const int x = ks * (kBKBytes / (int)sizeof(T));
#pragma unroll
          for (int j = 0; j < kBM / kSubRows; ++j)
            if (j < n_sub) tma_load_2d(a_dst + j * kSubBytes, &map_x, &aux->full[stage], x, sub_row[j]);
          tma_load_2d(b_dst, &map_wk, &aux->full[stage], x, it.head * kHeadDim);
          tma_load_2d(b_dst + kBBytes / 2, &map_wv, &aux->full[stage], x, it.head * kHeadDim);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // another role gave up: let copies that are still in flight land (bounded)
        // before the CTA's shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const uint32_t idesc = instr_desc(sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u);
      uint32_t stage = 0, phase = 0, n_local = 0;
      bool ok = true;
      for (int i = blockIdx.x; i < n_items && ok; i += gridDim.x, ++n_local) {
        const uint32_t buf = n_local & 1u, use = n_local >> 1;
        if (!mbar_wait(&aux->acc_empty[buf], (use & 1u) ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kBN;
        for (int ks = 0; ks < p.k_slabs; ++ks) {
          if (!mbar_wait(&aux->full[stage], phase, abort_flag, p.status, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)stage * kStageBytes);
          const uint64_t a_desc = smem_desc_sw128(a_addr);
          const uint64_t b_desc = smem_desc_sw128(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBKBytes / 32; ++k)
            tc_mma_f16(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc,
                       (ks | k) != 0 ? 1u : 0u);
          tc_commit(&aux->empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&aux->acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int quarter = warp & 3;               // TMEM lanes this warp may read
    const int row = quarter * 32 + lane;        // token row inside the tile
    const int et = threadIdx.x - 64;            // 0..127 (column owner in the final step)
    const T* bk = static_cast<const T*>(p.b_k);
    const T* bv = static_cast<const T*>(p.b_v);
    uint32_t n_local = 0;
    bool ok = true;
    for (int i = blockIdx.x; i < n_items && ok; i += gridDim.x, ++n_local) {
      const Item it = item_of(i, n_tiles, p.heads);
      const uint32_t buf = n_local & 1u, use = n_local >> 1;
      const int hcol = it.head * kHeadDim;
      bool valid;
      int req = 0, chunk = 0;
      int64_t out_row = 0;
      if (MODE == kModeAttend) {
        const int2 rc = p.hid_tiles[it.tile];
        req = rc.x; chunk = rc.y;
        const int seq = min(p.seq_lens[req], p.max_blocks_per_seq * p.block_size);
        valid = chunk * kBM + row < seq;
        const T* q = static_cast<const T*>(p.query) + req * p.query_stride + hcol;
        aux->q[et] = Elem<T>::to_float(q[et]) * p.scale_log2;
      } else {
        out_row = (int64_t)it.tile * kBM + row;
        valid = out_row < p.n_rows;
      }
      aux->bk[et] = bk ? Elem<T>::to_float(bk[hcol + et]) : 0.f;
      aux->bv[et] = bv ? Elem<T>::to_float(bv[hcol + et]) : 0.f;
      epi_barrier();

      if (!epi_all(mbar_wait(&aux->acc_full[buf], use & 1u, abort_flag, p.status, 4))) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * kBN;
      uint32_t r[32];

      if (MODE == kModeStore) {
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
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&aux->acc_empty[buf]);
        epi_barrier();  // bias buffers are rewritten by the next item
        continue;
      }

      // ---- scores: s = q . (K_row + b_k), already in the log2 domain ----
      float s = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          s = fmaf(aux->q[c * 32 + j], __uint_as_float(r[j]) + aux->bk[c * 32 + j], s);
      }
      s = valid ? s : -INFINITY;
      float wm = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
      if (lane == 0) aux->red_max[quarter] = wm;
      epi_barrier();
      const float mx = fmaxf(fmaxf(aux->red_max[0], aux->red_max[1]), fmaxf(aux->red_max[2], aux->red_max[3]));
      const float pr = valid ? exp2f(s - mx) : 0.f;
      float ws = pr;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
      if (lane == 0) aux->red_sum[quarter] = ws;

      // ---- weighted V rows, column sums over the warp's 32 rows ----
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld32(t_row + kHeadDim + c * 32, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          v[j] = valid ? pr * (__uint_as_float(r[j]) + aux->bv[c * 32 + j]) : 0.f;
        warp_column_sum(v, lane);
        aux->red_acc[quarter][c * 32 + lane] = v[0];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&aux->acc_empty[buf]);
      epi_barrier();
      {
        const float a = aux->red_acc[0][et] + aux->red_acc[1][et] + aux->red_acc[2][et] + aux->red_acc[3][et];
        const int64_t slot = (int64_t)(p.part_offset[req] + chunk) * p.heads + it.head;
        p.part_acc[slot * kHeadDim + et] = a;
        if (et == 0) {
          const float l = aux->red_sum[0] + aux->red_sum[1] + aux->red_sum[2] + aux->red_sum[3];
          *reinterpret_cast<float2*>(p.part_ml + slot * 2) = make_float2(mx, l);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ---- host side -----------------------------------------------------------------
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

// 2-D row-major matrix [rows, cols] of 2-byte elements, box [box_rows, 64 cols], 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int dtype, uint64_t cols, uint64_t rows,
             uint64_t row_stride_elems, uint32_t box_rows, const char* what) {
  EncodeTiledFn fn = encode_fn();
  APS_REQUIRE(fn != nullptr, APS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const CUtensorMapDataType dt = dtype == APS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  APS_REQUIRE(r == CUDA_SUCCESS, APS_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  return APS_OK;
}

template <typename T, int MODE>
int launch_hidden(const CUtensorMap& mx, const CUtensorMap& mk, const CUtensorMap& mv,
                  const HiddenParams& p, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  APS_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    APS_CUDA(cudaFuncSetAttribute(hidden_path_kernel<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kSmemBytes));
    configured[dev] = true;
  }
  {
    ScopedProfile prof(1, stream);
    hidden_path_kernel<T, MODE><<<sm_count(), kThreads, kSmemBytes, stream>>>(mx, mk, mv, p);
  }
  return launch_status("hidden_path_kernel");
}

struct HiddenArgs {
  const void* hidden_cache; const void* w_k; const void* b_k; const void* w_v; const void* b_v;
  int heads, head_size, hidden_size;
  int64_t hidden_row_stride, num_hidden_rows, w_stride;
  int dtype;
};

int check_hidden_args(const char* op, const HiddenArgs& a) {
  APS_REQUIRE(a.dtype == APS_F16 || a.dtype == APS_BF16, APS_ERR_UNSUPPORTED,
              "%s: the tensor-core re-projection supports fp16 and bf16 only (dtype %d)", op, a.dtype);
  APS_REQUIRE(a.head_size == kHeadDim, APS_ERR_UNSUPPORTED,
              "%s: the tensor-core re-projection supports head size 128 only (got %d)", op, a.head_size);
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

int make_maps(const HiddenArgs& a, CUtensorMap* mx, CUtensorMap* mk, CUtensorMap* mv) {
  int st;
  const uint64_t hd = (uint64_t)a.heads * a.head_size;
  if ((st = make_map(mx, a.hidden_cache, a.dtype, a.hidden_size, a.num_hidden_rows, a.hidden_row_stride,
                     kSubRows, "hidden cache")) != APS_OK) return st;
  if ((st = make_map(mk, a.w_k, a.dtype, a.hidden_size, hd, a.w_stride, kHeadDim, "W_k")) != APS_OK) return st;
  return make_map(mv, a.w_v, a.dtype, a.hidden_size, hd, a.w_stride, kHeadDim, "W_v");
}

}  // namespace
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
  AttnShape s{batch, max_blocks_per_seq, num_heads, head_size, block_size,
              query_stride, out_stride, block_stride, scale, dtype};
  int st = check_attention_args("hybrid_decode_attention", out, query, key_cache, value_cache,
                                block_tables, seq_lens, s, workspace, workspace_bytes, false);
  if (st != APS_OK || batch == 0) return st;
  APS_REQUIRE(cache_type != nullptr, APS_ERR_NULL_POINTER, "hybrid_decode_attention: cache_type is null");
  HiddenArgs a{hidden_cache, w_k, b_k, w_v, b_v, num_heads, head_size, hidden_size,
               hidden_row_stride, num_hidden_rows, w_stride, dtype};
  if ((st = check_hidden_args("hybrid_decode_attention", a)) != APS_OK) return st;
  CUtensorMap mx, mk, mv;
  if ((st = make_maps(a, &mx, &mk, &mv)) != APS_OK) return st;

  const WorkspaceLayout w = workspace_layout(batch, max_blocks_per_seq, block_size, num_heads, head_size);
  const WorkspacePtrs ws = workspace_ptrs(workspace, w);
  cudaStream_t cs = (cudaStream_t)stream;
  if ((st = launch_plan(ws, seq_lens, cache_type, batch, max_blocks_per_seq, block_size, cs)) != APS_OK) return st;
  if (key_cache != nullptr && value_cache != nullptr) {
    if ((st = launch_kv_attention(ws, query, key_cache, value_cache, block_tables, seq_lens, s, cs)) != APS_OK) return st;
  }
  HiddenParams p{};
  p.plan = ws.plan; p.part_offset = ws.part_offset; p.hid_tiles = ws.hid_tiles;
  p.part_ml = ws.part_ml; p.part_acc = ws.part_acc; p.query = query;
  p.block_tables = block_tables; p.seq_lens = seq_lens;
  p.max_blocks_per_seq = max_blocks_per_seq; p.block_size = block_size;
  p.query_stride = query_stride; p.scale_log2 = scale * 1.4426950408889634f;
  p.b_k = b_k; p.b_v = b_v; p.heads = num_heads; p.k_slabs = (hidden_size + 63) / 64;
  p.status = ws.plan + kPlanStatus;
  st = dtype == APS_BF16 ? launch_hidden<__nv_bfloat16, kModeAttend>(mx, mk, mv, p, cs)
                         : launch_hidden<__half, kModeAttend>(mx, mk, mv, p, cs);
  if (st != APS_OK) return st;
  return launch_combine(ws, out, seq_lens, s, cs);
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
  if ((st = make_maps(a, &mx, &mk, &mv)) != APS_OK) return st;
  HiddenParams p{};
  p.kv_out = kv; p.block_ids = block_ids; p.n_rows = n_rows; p.kv_stride = kv_stride;
  p.n_store_tiles = (int)((n_rows + kBM - 1) / kBM);
  p.b_k = b_k; p.b_v = b_v; p.heads = num_heads; p.k_slabs = (hidden_size + 63) / 64;
  p.status = status_word;
  cudaStream_t cs = (cudaStream_t)stream;
  return dtype == APS_BF16 ? launch_hidden<__nv_bfloat16, kModeStore>(mx, mk, mv, p, cs)
                           : launch_hidden<__half, kModeStore>(mx, mk, mv, p, cs);
}

// K/V-path decode attention: a pure HBM-streaming paged attention.
//
// Replaces the third-party flash_attn_with_kvcache call of the reference
// (additional_designs/attention/backends/aptserve_flash_attn.py:452-461) for
// one query token per request over caches laid out [NB, BS, H, D]
// (additional_designs/worker/aptserve_cache_engine.py:61-80).
//
// Work unit: one warp streams one head of one 128-token chunk, 16 tokens at a time; the
// softmax is the online (running max / running sum) form in the log2 domain.  Two kernels:
//
//   kv_attention_tma_kernel  (fp16 / bf16, head sizes 64 / 128, cache blocks laid out back to
//       back as the cache engine allocates them)  The 16-token groups of K and V arrive in
//       shared memory by tensor copies (cp.async.bulk.tensor, one elected lane per warp, a ring
//       of three groups per warp with mbarriers) and the two small products run on the tensor
//       cores as mma.sync m16n8k16 with the single query row in row 0 of the A operand, fed by
//       ldmatrix: no conversion, no shuffle reduction, no byte permutes, ~100 instructions per
//       16 tokens and warp.  The kernel is HBM-bound only while the SMs can take in the bytes,
//       and inside a decode step it runs at the ~1 GHz the board's power cap leaves next to the
//       re-projection kernel: loads through the load/store unit (16 bytes per lane, whatever the
//       arithmetic) top out near 29 bytes per SM clock there, tensor copies reach 38.
//   kv_attention_kernel      (fp32; head sizes 32 and 256; any other block stride)  CUDA-core
//       arithmetic: LPR = row bytes / 16 lanes cover a row with one 16-byte load each, scores
//       are reduced over those lanes with shuffles.
// CTAs are persistent; work is handed out through an atomic counter.

#include "attention_common.cuh"
#include "tensor_maps.cuh"

namespace aps {
namespace {

constexpr int kPlanThreads = 1024;
constexpr int kKvWarps = 8;
constexpr unsigned kFull = 0xffffffffu;

// ---- planning ------------------------------------------------------------------
// One CTA.  Thread t handles a contiguous run of requests; two block-wide prefix sums:
// first over (K/V chunks, hidden sub-blocks), which fixes where each hidden request's rows
// sit in the tile list, then over the number of softmax partials each request will leave.
__device__ __forceinline__ void block_scan2(int* sa, int* sb, int tid, int& a, int& b) {
  sa[tid] = a; sb[tid] = b;
  __syncthreads();
  for (int off = 1; off < kPlanThreads; off <<= 1) {
    int x = 0, y = 0;
    if (tid >= off) { x = sa[tid - off]; y = sb[tid - off]; }
    __syncthreads();
    sa[tid] += x; sb[tid] += y;
    __syncthreads();
  }
  a = sa[tid]; b = sb[tid];   // inclusive sums
}

__global__ void __launch_bounds__(kPlanThreads)
plan_kernel(int* __restrict__ plan, int* __restrict__ part_offset, int2* __restrict__ kv_chunks,
            int2* __restrict__ hid_tiles, int* __restrict__ first_tile, int2* __restrict__ hid_subs,
            int* __restrict__ hid_rows, const int32_t* __restrict__ seq_lens,
            const int32_t* __restrict__ cache_type, const int32_t* __restrict__ block_tables, int batch,
            int max_tokens, int max_blocks, int block_size, int pack_tiles, int kv_present) {
  __shared__ int sa[kPlanThreads], sb[kPlanThreads];
  __shared__ int s_kv_missing;
  const int tid = threadIdx.x;
  if (tid == 0) s_kv_missing = 0;
  __syncthreads();
  const int per = (batch + kPlanThreads - 1) / kPlanThreads;
  const int r0 = min(batch, tid * per), r1 = min(batch, r0 + per);
  auto seq_of = [&](int r) { return max(0, min(seq_lens[r], max_tokens)); };
  auto hidden = [&](int r) { return cache_type != nullptr && cache_type[r] != 0; };
  // without a K/V cache a K/V-cached request gets no chunks and no partials: its output row is zero
  auto chunks_of = [&](int s) { return kv_present ? (s + kChunkTokens - 1) / kChunkTokens : 0; };
  auto subs_of = [&](int s) {   // sub-blocks a hidden request of s tokens occupies in the tile list
    const int n = (s + kSubRowsPlan - 1) / kSubRowsPlan;
    return pack_tiles ? n : (n + 7) / 8 * 8;
  };
  // pass 1: K/V chunks and hidden sub-blocks
  int kv = 0, sub = 0;
  for (int r = r0; r < r1; ++r) {
    const int s = seq_of(r);
    if (hidden(r)) sub += subs_of(s);
    else { kv += chunks_of(s); if (!kv_present) s_kv_missing = 1; }
  }
  int kv_inc = kv, sub_inc = sub;
  block_scan2(sa, sb, tid, kv_inc, sub_inc);
  const int total_kv = sa[kPlanThreads - 1], total_sub = sb[kPlanThreads - 1];
  __syncthreads();
  int o_kv = kv_inc - kv, o_sub = sub_inc - sub;
  // pass 2: partial slots per request (K/V: one per chunk; hidden: one per tile it has rows in)
  int slots = 0, dummy = 0;
  {
    int g = o_sub;
    for (int r = r0; r < r1; ++r) {
      const int s = seq_of(r);
      if (hidden(r)) {
        const int n = subs_of(s), real = (s + kSubRowsPlan - 1) / kSubRowsPlan;
        if (real > 0) slots += (g + real - 1) / 8 - g / 8 + 1;
        g += n;
      } else {
        slots += chunks_of(s);
      }
    }
  }
  int slots_inc = slots;
  block_scan2(sa, sb, tid, slots_inc, dummy);
  const int total_slots = sa[kPlanThreads - 1];
  int o_slot = slots_inc - slots;
  // write-out.  The per-request words are written by the request's owner thread; the lists
  // (one entry per K/V chunk or per 16-row sub-block, up to 128 per request, each sub-block
  // with a block-table lookup) are filled by the whole CTA: in round k every thread posts its
  // k-th request in shared memory and warp w fills the lists of entries w, w + 32, ...
  __shared__ int q_req[kPlanThreads], q_at[kPlanThreads], q_n[kPlanThreads], q_real[kPlanThreads];
  const int warp = tid >> 5, lane = tid & 31;
  int g = o_sub;
  for (int k = 0; k < per; ++k) {
    const int r = r0 + k;
    q_n[tid] = 0;
    if (r < r1) {
      const int s = seq_of(r);
      part_offset[r] = o_slot;
      q_req[tid] = r;
      if (hidden(r)) {
        const int n = subs_of(s), real = (s + kSubRowsPlan - 1) / kSubRowsPlan;
        first_tile[r] = g / 8;
        q_at[tid] = g; q_n[tid] = n; q_real[tid] = real;
        if (real > 0) o_slot += (g + real - 1) / 8 - g / 8 + 1;
        g += n;
      } else {
        first_tile[r] = 0;
        const int c = chunks_of(s);
        q_at[tid] = o_kv; q_n[tid] = c; q_real[tid] = -1;   // -1 marks a K/V request
        o_kv += c;
        o_slot += c;
      }
    }
    __syncthreads();
    for (int e = warp; e < kPlanThreads; e += kPlanThreads / 32) {
      const int n = q_n[e];
      if (n == 0) continue;
      const int req = q_req[e], at = q_at[e], real = q_real[e];
      if (real < 0) {
        for (int j = lane; j < n; j += 32) kv_chunks[at + j] = make_int2(req, j);
      } else {
        const int32_t* bt = block_tables + (int64_t)req * max_blocks;
        for (int j0 = 0; j0 < n; j0 += 128) {
          int blk[4];   // four independent block-table loads per lane before the stores
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = j0 + lane + 32 * u;
            blk[u] = j < real ? bt[j * kSubRowsPlan / block_size] : 0;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = j0 + lane + 32 * u;
            if (j >= n) continue;
            const int tok = j * kSubRowsPlan;
            hid_subs[at + j] = j < real ? make_int2(req, tok) : make_int2(-1, 0);
            hid_rows[at + j] = j < real ? blk[u] * block_size + tok % block_size : 0;
            if (!pack_tiles && (j & 7) == 0) hid_tiles[(at + j) / 8] = make_int2(req, j / 8);
          }
        }
      }
    }
    __syncthreads();
  }
  if (tid == kPlanThreads - 1) {
    part_offset[batch] = total_slots;
    plan[kPlanNumKvChunks] = total_kv;
    plan[kPlanNumHidTiles] = (total_sub + 7) / 8;
    plan[kPlanNumHidSubs] = total_sub;
    plan[kPlanKvCounter] = 0;
    plan[kPlanHidCounter] = 0;
    plan[kPlanStatus] = s_kv_missing ? kStatusNoKvCache : kStatusOk;
    // entries between the last sub-block and the end of the last tile read as padding
    for (int j = total_sub; j < (total_sub + 7) / 8 * 8; ++j) hid_subs[j] = make_int2(-1, 0);
  }
  if (tid >= kPlanStatsWord && tid < kPlanStatsWord + 18) plan[tid] = 0;  // optional kernel counters
}

// ---- K/V streaming ---------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <typename T, int D>
struct KvCfg {
  static constexpr int EPL = 16 / sizeof(T);               // elements per lane
  static constexpr int LPR = D / EPL;                      // lanes per row
  static constexpr int TPW = 32 / LPR;                     // rows per warp-wide load
  static constexpr int GT = (TPW * 8 < 16) ? TPW * 8 : 16; // tokens per group
  static constexpr int NL = GT / TPW;                      // loads per lane per group
  static_assert(LPR >= 1 && LPR <= 32 && (LPR & (LPR - 1)) == 0, "unsupported head size");
};

template <typename T, int D>
__global__ void __launch_bounds__(kKvWarps * 32, 2)
kv_attention_kernel(int* __restrict__ plan, const int* __restrict__ part_offset,
                    const int2* __restrict__ kv_chunks, float* __restrict__ part_ml,
                    float* __restrict__ part_acc, const T* __restrict__ query,
                    const T* __restrict__ key_cache, const T* __restrict__ value_cache,
                    const int32_t* __restrict__ block_tables, const int32_t* __restrict__ seq_lens,
                    int max_blocks_per_seq, int heads, int block_size, int64_t query_stride,
                    int64_t block_stride, float scale_log2) {
  using C = KvCfg<T, D>;
  __shared__ int s_base;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % C::LPR, tsel = lane / C::LPR;
  const int total = plan[kPlanNumKvChunks] * heads;
  const int64_t row_stride = (int64_t)heads * D;

  while (true) {
    if (threadIdx.x == 0) s_base = atomicAdd(&plan[kPlanKvCounter], (int)(blockDim.x >> 5));
    __syncthreads();
    const int base = s_base;
    __syncthreads();
    if (base >= total) break;
    const int unit = base + warp;
    if (unit >= total) continue;

    const int2 rc = kv_chunks[unit / heads];
    const int h = unit % heads;
    const int req = rc.x;
    const int seq = min(seq_lens[req], max_blocks_per_seq * block_size);
    const int tok_begin = rc.y * kChunkTokens;
    const int tok_end = min(seq, tok_begin + kChunkTokens);
    const int32_t* bt = block_tables + (int64_t)req * max_blocks_per_seq;

    float qf[C::EPL];
    {
      const uint4 qv = *reinterpret_cast<const uint4*>(query + req * query_stride + h * D + sub * C::EPL);
      Vec16<T>::unpack(qv, qf);
#pragma unroll
      for (int e = 0; e < C::EPL; ++e) qf[e] *= scale_log2;
    }
    float acc[C::EPL];
#pragma unroll
    for (int e = 0; e < C::EPL; ++e) acc[e] = 0.f;
    float m = -INFINITY, l = 0.f;

    uint4 kreg[C::NL], vreg[C::NL];
    auto row_offset = [&](int tb) -> int64_t {
      const int blk = bt[tb / block_size];
      return (int64_t)blk * block_stride + (int64_t)(tb % block_size + tsel) * row_stride +
             h * D + sub * C::EPL;
    };
    auto load_group = [&](uint4* reg, const T* cache, int tb) {
      const int64_t off = row_offset(tb);
#pragma unroll
      for (int i = 0; i < C::NL; ++i) {
        const int tok = tb + i * C::TPW + tsel;
        reg[i] = tok < tok_end ? ld_stream16(cache + off + (int64_t)i * C::TPW * row_stride)
                               : make_uint4(0, 0, 0, 0);
      }
    };

    load_group(kreg, key_cache, tok_begin);
    for (int tb = tok_begin; tb < tok_end; tb += C::GT) {
      load_group(vreg, value_cache, tb);
      float s[C::NL];
#pragma unroll
      for (int i = 0; i < C::NL; ++i) {
        float kf[C::EPL];
        Vec16<T>::unpack(kreg[i], kf);
        float a = 0.f;
#pragma unroll
        for (int e = 0; e < C::EPL; ++e) a = fmaf(qf[e], kf[e], a);
#pragma unroll
        for (int o = C::LPR / 2; o > 0; o >>= 1) a += __shfl_xor_sync(kFull, a, o);
        s[i] = (tb + i * C::TPW + tsel) < tok_end ? a : -INFINITY;
      }
      if (tb + C::GT < tok_end) load_group(kreg, key_cache, tb + C::GT);
      float gm = s[0];
#pragma unroll
      for (int i = 1; i < C::NL; ++i) gm = fmaxf(gm, s[i]);
#pragma unroll
      for (int o = C::LPR; o < 32; o <<= 1) gm = fmaxf(gm, __shfl_xor_sync(kFull, gm, o));
      const float m_new = fmaxf(m, gm);  // finite: every group holds at least one valid token
      const float corr = exp2f(m - m_new);
      l *= corr;
#pragma unroll
      for (int e = 0; e < C::EPL; ++e) acc[e] *= corr;
#pragma unroll
      for (int i = 0; i < C::NL; ++i) {
        const float p = exp2f(s[i] - m_new);
        l += p;
        float vf[C::EPL];
        Vec16<T>::unpack(vreg[i], vf);
#pragma unroll
        for (int e = 0; e < C::EPL; ++e) acc[e] = fmaf(p, vf[e], acc[e]);
      }
      m = m_new;
    }
#pragma unroll
    for (int o = C::LPR; o < 32; o <<= 1) {
      l += __shfl_xor_sync(kFull, l, o);
#pragma unroll
      for (int e = 0; e < C::EPL; ++e) acc[e] += __shfl_xor_sync(kFull, acc[e], o);
    }
    const int64_t slot = (int64_t)(part_offset[req] + rc.y) * heads + h;
    if (tsel == 0) {
      float* dst = part_acc + slot * D + sub * C::EPL;
#pragma unroll
      for (int e = 0; e < C::EPL; e += 4)
        *reinterpret_cast<float4*>(dst + e) = make_float4(acc[e], acc[e + 1], acc[e + 2], acc[e + 3]);
      if (lane == 0) *reinterpret_cast<float2*>(part_ml + slot * 2) = make_float2(m, l);
    }
  }
}

// ---- K/V streaming, products on the tensor cores -------------------------------------
// mma.sync.m16n8k16 fragments (g = lane / 4, j = lane % 4):
//   A (16 x 16, row major)  a0 = (row g, k = 2j, 2j+1)   a2 = (row g, k = 2j+8, 2j+9)
//                           a1, a3 = the same for row g + 8
//   B (16 x 8, column major) b0 = (k = 2j, 2j+1, column g)  b1 = (k = 2j+8, 2j+9, column g)
//   C (16 x 8, fp32)         c0, c1 = (row g, columns 2j, 2j+1)   c2, c3 = row g + 8
// Only row 0 of A holds data (the one query row), so only lanes 0..3 hold results.
template <typename T> struct Mma16816;
template <> struct Mma16816<__half> {
  // d0, d1 accumulate in place; rows 8..15 (a1, a3, c2, c3) are zero on input and dropped on output
  static __device__ __forceinline__ void run(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float x2, x3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %5}, {%7, %8}, {%0, %1, %9, %9};"
                 : "+f"(d0), "+f"(d1), "=f"(x2), "=f"(x3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.f));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <> struct Mma16816<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float x2, x3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %5}, {%7, %8}, {%0, %1, %9, %9};"
                 : "+f"(d0), "+f"(d1), "=f"(x2), "=f"(x3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.f));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};

constexpr int kGroupTokens = 16;   // tokens per softmax step

// ---- K/V streaming fed by tensor copies -------------------------------------------------
// A register-staged version of this kernel (16-byte ld.global per lane, the loaded vectors used
// as MMA fragments directly) kept 98 KB of loads in flight per SM and every byte passed the
// load/store unit: inside a decode step, at the ~1 GHz SM clock the power cap leaves, that was
// worth ~29 bytes per SM clock (4.3 TB/s), while the tensor-copy (TMA) path of the re-projection
// kernel delivers 60.  Here the 16-token groups arrive by cp.async.bulk.tensor: the K (V) plane is a
// 3-D tensor [head-row halves of 64 elements][cache rows][64 elements], one box of
// (64, 16 rows, D/64 halves) = one cache block's 16 rows of one head lands in shared memory as
// [half][token][128 bytes] with the 128-byte swizzle, so that ldmatrix reads it without bank
// conflicts: plain ldmatrix gives the B fragments of Q K^T, ldmatrix.trans those of P V (no
// byte permutes).  One elected lane per warp issues two copies per group (K box, V box) on the
// warp's own ring of stages, each with its mbarrier; the stream of groups continues across
// work units.  Rows of the last cache block past the sequence length arrive too: their scores
// are masked and their V rows are zeroed in shared memory before use.
#ifndef APS_KV_WARPS
#define APS_KV_WARPS 8
#endif
#ifndef APS_KV_STAGES
#define APS_KV_STAGES 3
#endif
// 8 warps with a ring of 3 groups each (193 KB of shared memory at head size 128, one CTA per SM)
// measured best on OPT-13B rows: 6.57 TB/s alone, 5.7 - 5.8 TB/s inside the loaded step; 4 warps x 3
// x 2 CTAs: 5.9 / 5.2; 12 warps x 2: 4.9 / 4.3; 6 warps x 4: 6.1 / 4.4; 5 warps x 5: 6.0 / 4.0.
constexpr int kTmaWarps = APS_KV_WARPS;
constexpr int kStatusKvWait = 5;   // a bounded wait for a K/V tensor copy ran out
constexpr long long kKvWaitBudget = 2000000000LL;

template <int DS>
struct TmaUnit {
  int n_groups;              // 16-token groups (0 = no unit)
  int tok_begin, tok_end;
  int my_row;                // lane l: first cache row (block * block_size + offset) of the unit's group l
  int head_coord;            // h * (D / 64): coordinate of the head in the third tensor dimension
  int64_t slot;              // where the unit's partial goes
  uint32_t qa[DS][2];        // A fragments (a0, a2) of the query row per 16-element step (lanes 0..3)
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <typename T, int D, int S>
__global__ void __launch_bounds__(kTmaWarps * 32, (384 / (kTmaWarps * 32)) > 0 ? (384 / (kTmaWarps * 32)) : 1)
kv_attention_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        int* __restrict__ plan, const int* __restrict__ part_offset,
                        const int2* __restrict__ kv_chunks, float* __restrict__ part_ml,
                        float* __restrict__ part_acc, const T* __restrict__ query,
                        const int32_t* __restrict__ block_tables, const int32_t* __restrict__ seq_lens,
                        int max_blocks_per_seq, int heads, int block_size, int64_t query_stride,
                        float scale_log2) {
  static_assert(sizeof(T) == 2 && (D == 64 || D == 128), "2-byte types, head size 64 or 128");
  constexpr int DS = D / 16;                  // 16-element steps of the head dimension
  constexpr int kHalves = D / 64;
  constexpr int kTileBytes = 16 * D * 2;      // K (or V) of one group: [half][token][128 B]
  constexpr int kStageBytes = 2 * kTileBytes;
  using M = Mma16816<T>;
  using Unit = TmaUnit<DS>;
  extern __shared__ unsigned char ring_raw[];
  __shared__ uint64_t bars[kTmaWarps][S];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;
  const int total = plan[kPlanNumKvChunks] * heads;
  const uint32_t ring = (((uint32_t)__cvta_generic_to_shared(ring_raw) + 1023u) & ~1023u) + warp * (S * kStageBytes);
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&bars[warp][0]);
  if (lane == 0) {
    for (int st = 0; st < S; ++st)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + st * 8) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  auto next_index = [&]() {
    int idx = 0;
    if (lane == 0) idx = atomicAdd(&plan[kPlanKvCounter], 1);
    return __shfl_sync(kFull, idx, 0);
  };
  auto load_unit = [&](int idx) {
    Unit u;
    u.n_groups = 0; u.tok_begin = u.tok_end = 0; u.my_row = 0; u.head_coord = 0; u.slot = 0;
#pragma unroll
    for (int st = 0; st < DS; ++st) u.qa[st][0] = u.qa[st][1] = 0u;
    if (idx < total) {
      const int2 rc = kv_chunks[idx / heads];
      const int h = idx % heads, req = rc.x;
      const int seq = min(seq_lens[req], max_blocks_per_seq * block_size);
      u.tok_begin = rc.y * kChunkTokens;
      u.tok_end = min(seq, u.tok_begin + kChunkTokens);
      u.n_groups = (u.tok_end - u.tok_begin + kGroupTokens - 1) / kGroupTokens;
      if (lane < u.n_groups) {
        const int tb = u.tok_begin + lane * kGroupTokens;   // a group never straddles a cache block
        u.my_row = block_tables[(int64_t)req * max_blocks_per_seq + tb / block_size] * block_size + tb % block_size;
      }
      u.head_coord = h * kHalves;
      u.slot = (int64_t)(part_offset[req] + rc.y) * heads + h;
      if (g == 0) {
        const T* q = query + req * query_stride + h * D + 2 * j;
#pragma unroll
        for (int st = 0; st < DS; ++st) {
          u.qa[st][0] = *reinterpret_cast<const uint32_t*>(q + 16 * st);
          u.qa[st][1] = *reinterpret_cast<const uint32_t*>(q + 16 * st + 8);
        }
      }
    }
    return u;
  };
  // request group gi of unit u into ring stage `stage`: two boxes counted on the stage's barrier
  auto issue_group = [&](const Unit& u, int gi, uint32_t stage) {
    const int row = __shfl_sync(kFull, u.my_row, gi);
    if (lane == 0) {
      const uint32_t bar = bar0 + stage * 8, dst = ring + stage * kStageBytes;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kStageBytes) : "memory");
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                   ::"r"(dst), "l"(reinterpret_cast<uint64_t>(&map_k)), "r"(bar), "r"(0), "r"(row), "r"(u.head_coord) : "memory");
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                   ::"r"(dst + kTileBytes), "l"(reinterpret_cast<uint64_t>(&map_v)), "r"(bar), "r"(0), "r"(row), "r"(u.head_coord) : "memory");
    }
  };
  auto try_wait = [&](uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
  };
  // the whole warp tests once; if the data is not there lane 0 waits (bounded) and tells the others
  auto wait_stage = [&](uint32_t stage, uint32_t parity) {
    const uint32_t bar = bar0 + stage * 8;
    if (__all_sync(kFull, try_wait(bar, parity))) return true;
    bool got = true;
    if (lane == 0) {
      const long long t0 = clock64();
      int spins = 0;
      while (!try_wait(bar, parity)) {
        if ((++spins & 255) == 0 && clock64() - t0 > kKvWaitBudget) { got = false; break; }
      }
    }
    got = __shfl_sync(kFull, got ? 1 : 0, 0) != 0;
    if (got) (void)try_wait(bar, parity);   // every lane observes the completed phase itself
    return got;
  };

  Unit cur = load_unit(next_index());
  Unit nxt = load_unit(next_index());
  int issue_in_nxt = 0, issue_g = 0;       // the request cursor: unit (cur / nxt) and group
  uint32_t issued = 0, consumed = 0;       // groups requested / used so far (ring stage = count % S)
  auto refill = [&]() {
    while (issued - consumed < (uint32_t)S) {
      if (!issue_in_nxt && issue_g >= cur.n_groups) { issue_in_nxt = 1; issue_g = 0; }
      if (issue_in_nxt && issue_g >= nxt.n_groups) break;   // nothing known beyond the next unit yet
      if (issue_in_nxt) issue_group(nxt, issue_g, issued % S);
      else issue_group(cur, issue_g, issued % S);
      ++issue_g; ++issued;
    }
  };
  refill();

  // per-lane parts of the ldmatrix addresses (row inside an 8-row group, 16-byte piece)
  const int lrow = lane & 7, lmat = lane >> 3;
  bool ok = true;
  while (cur.n_groups > 0 && ok) {
    float acc[D / 8][2];
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) acc[nb][0] = acc[nb][1] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int gi = 0; gi < cur.n_groups; ++gi) {
      const uint32_t stage = consumed % S;
      if (!wait_stage(stage, (consumed / S) & 1u)) { ok = false; break; }
      const uint32_t ktile = ring + stage * kStageBytes, vtile = ktile + kTileBytes;
      const int tb = cur.tok_begin + gi * kGroupTokens;
      const int n_valid = min(kGroupTokens, cur.tok_end - tb);
      if (n_valid < kGroupTokens) {
        // rows past the sequence length hold whatever the cache block holds: zero them in V
        // (their scores are masked below, and 0 * garbage must stay 0)
        const int n_pieces = (kGroupTokens - n_valid) * kHalves * 8;
        for (int i = lane; i < n_pieces; i += 32) {
          const int r = n_valid + i / (kHalves * 8), rem = i % (kHalves * 8);
          const uint32_t a = vtile + (rem >> 3) * 2048 + r * 128 + (rem & 7) * 16;
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(a), "r"(0u) : "memory");
        }
        __syncwarp();
      }
      // ---- scores of the group's two 8-token blocks: row 0 of Q K^T ----
      float sc[2][2][2];   // [block][partial chain][column]
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        sc[b][0][0] = sc[b][0][1] = sc[b][1][0] = sc[b][1][1] = 0.f;
        const int r = b * 8 + lrow;
#pragma unroll
        for (int c4 = 0; c4 < D / 32; ++c4) {
          const int piece = 4 * c4 + lmat;
          uint32_t kf[4];
          ldmatrix_x4(ktile + (piece >> 3) * 2048 + r * 128 + (((piece & 7) ^ (r & 7)) << 4), kf);
          M::run(sc[b][0][0], sc[b][0][1], cur.qa[2 * c4][0], cur.qa[2 * c4][1], kf[0], kf[1]);
          M::run(sc[b][1][0], sc[b][1][1], cur.qa[2 * c4 + 1][0], cur.qa[2 * c4 + 1][1], kf[2], kf[3]);
        }
      }
      // ---- online softmax over the 16 tokens (lane j of row 0: tokens 2j, 2j+1 of each block) ----
      float s[2][2];
      float gm = -INFINITY;
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float v = (sc[b][0][i] + sc[b][1][i]) * scale_log2;
          s[b][i] = b * 8 + 2 * j + i < n_valid ? v : -INFINITY;
          gm = fmaxf(gm, s[b][i]);
        }
      gm = fmaxf(gm, __shfl_xor_sync(kFull, gm, 1));
      gm = fmaxf(gm, __shfl_xor_sync(kFull, gm, 2));
      const float m_new = fmaxf(m, gm);   // finite: every group holds at least one valid token
      const float corr = exp2f(m - m_new);
      m = m_new;
      float p[2][2];
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int i = 0; i < 2; ++i) p[b][i] = exp2f(s[b][i] - m_new);
      l = l * corr + (p[0][0] + p[0][1]) + (p[1][0] + p[1][1]);
      // the score fragment, rounded to the cache's type, is the A fragment of P V
      const uint32_t pa0 = M::pack(p[0][0], p[0][1]), pa2 = M::pack(p[1][0], p[1][1]);
      // ---- weighted V rows: row 0 of P V; one transposed ldmatrix per 16 head elements ----
      {
        const int r = (lmat & 1) * 8 + lrow;
#pragma unroll
        for (int n2 = 0; n2 < D / 16; ++n2) {
          const int piece = 2 * n2 + (lmat >> 1);
          uint32_t vf[4];
          ldmatrix_x4_trans(vtile + (piece >> 3) * 2048 + r * 128 + (((piece & 7) ^ (r & 7)) << 4), vf);
          acc[2 * n2][0] *= corr; acc[2 * n2][1] *= corr;
          acc[2 * n2 + 1][0] *= corr; acc[2 * n2 + 1][1] *= corr;
          M::run(acc[2 * n2][0], acc[2 * n2][1], pa0, pa2, vf[0], vf[1]);
          M::run(acc[2 * n2 + 1][0], acc[2 * n2 + 1][1], pa0, pa2, vf[2], vf[3]);
        }
      }
      // every lane's reads of the stage are done (their results fed MMAs): it can be refilled.
      // After the zero fill above the next tensor copy follows generic stores to the stage.
      __syncwarp();
      if (n_valid < kGroupTokens && lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      ++consumed;
      refill();
    }
    if (!ok) break;
    // ---- the partial: lanes 0..3 hold row 0 (lane j: head elements nb*8 + 2j, 2j + 1) ----
    l += __shfl_xor_sync(kFull, l, 1);
    l += __shfl_xor_sync(kFull, l, 2);
    if (g == 0) {
      float* dst = part_acc + cur.slot * D + 2 * j;
#pragma unroll
      for (int nb = 0; nb < D / 8; ++nb) *reinterpret_cast<float2*>(dst + nb * 8) = make_float2(acc[nb][0], acc[nb][1]);
      if (lane == 0) *reinterpret_cast<float2*>(part_ml + cur.slot * 2) = make_float2(m, l);
    }
    // the next unit becomes the current one; the request cursor keeps its place in it
    cur = nxt;
    if (issue_in_nxt) issue_in_nxt = 0; else issue_g = 0;
    nxt = load_unit(cur.n_groups > 0 ? next_index() : total);
    refill();
  }
  if (!ok) {
    // a copy never arrived: record it (the combine kernel then marks the output) and give the
    // copies still in flight a bounded time to land before the CTA's shared memory is released
    if (lane == 0) atomicCAS(&plan[kPlanStatus], 0, kStatusKvWait);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
  }
}

// ---- combine -------------------------------------------------------------------
// One warp per (request, head): merge the request's partials in chunk order.  When a bounded
// wait of the re-projection kernel ran out (status word 1..7) some partials were never
// written: the whole output is filled with NaN instead of numbers that look plausible.
template <typename T>
__global__ void __launch_bounds__(256)
combine_kernel(const int* __restrict__ plan, const int* __restrict__ part_offset, const float* __restrict__ part_ml,
               const float* __restrict__ part_acc, T* __restrict__ out, int batch, int heads,
               int head_size, int64_t out_stride) {
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= batch * heads) return;
  const int req = unit / heads, h = unit % heads;
  const int p0 = part_offset[req], p1 = part_offset[req + 1];
  T* dst = out + req * out_stride + (int64_t)h * head_size;
  const int status = plan[kPlanStatus];
  if (status >= kStatusWaitFirst && status <= kStatusWaitLast) {
    for (int d = lane; d < head_size; d += 32) dst[d] = Elem<T>::from_float(__int_as_float(0x7fc00000));
    return;
  }
  // the lanes share the request's partials for the maximum and the denominator (butterfly
  // reductions: the same order every time), then every lane owns four head elements and walks
  // the partials in chunk order with independent 16-byte loads
  float mx = -INFINITY;
  for (int p = p0 + lane; p < p1; p += 32) mx = fmaxf(mx, part_ml[((int64_t)p * heads + h) * 2]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, o));
  float denom = 0.f;
  for (int p = p0 + lane; p < p1; p += 32) {
    const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((int64_t)p * heads + h) * 2);
    denom += exp2f(ml.x - mx) * ml.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(kFull, denom, o);
  const float inv = (p1 > p0 && denom > 0.f) ? 1.f / denom : 0.f;
  for (int d = lane * 4; d < head_size; d += 128) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int p = p0; p < p1; ++p) {
      const int64_t slot = (int64_t)p * heads + h;
      const float w = exp2f(part_ml[slot * 2] - mx);
      const float4 v = *reinterpret_cast<const float4*>(part_acc + slot * head_size + d);
      a.x = fmaf(w, v.x, a.x); a.y = fmaf(w, v.y, a.y); a.z = fmaf(w, v.z, a.z); a.w = fmaf(w, v.w, a.w);
    }
    dst[d] = Elem<T>::from_float(a.x * inv);
    dst[d + 1] = Elem<T>::from_float(a.y * inv);
    dst[d + 2] = Elem<T>::from_float(a.z * inv);
    dst[d + 3] = Elem<T>::from_float(a.w * inv);
  }
}

// Tensor maps of the K and V planes for the tensor-copy kernel: [64 elements][cache rows][row
// halves of 64 elements], box (64, 16 rows, D / 64).  The number of cache rows is not part of the
// C ABI (block ids come from the block tables), so the row dimension is given the largest bound a
// 32-bit row coordinate can reach; the copies only ever name rows of blocks that the block tables hold.
template <int D>
int kv_plane_maps(const void* key_cache, const void* value_cache, const AttnShape& s, CUtensorMap* mk, CUtensorMap* mv) {
  TensorMapSpec spec{};
  spec.dtype = s.dtype; spec.rank = 3;
  spec.dims[0] = 64; spec.dims[1] = uint64_t(1) << 31; spec.dims[2] = (uint64_t)s.heads * D / 64;
  spec.strides_bytes[0] = (uint64_t)s.heads * D * 2; spec.strides_bytes[1] = 128;
  spec.box[0] = 64; spec.box[1] = 16; spec.box[2] = D / 64;
  spec.base = key_cache;
  int st = cached_tensor_map(mk, spec, "K plane");
  if (st != APS_OK) return st;
  spec.base = value_cache;
  return cached_tensor_map(mv, spec, "V plane");
}

template <typename T, int D>
int launch_kv_typed(const WorkspacePtrs& ws, const void* query, const void* key_cache,
                    const void* value_cache, const int32_t* block_tables, const int32_t* seq_lens,
                    const AttnShape& s, cudaStream_t stream) {
  const float scale_log2 = s.scale * 1.4426950408889634f;
  if constexpr (sizeof(T) == 2 && (D == 64 || D == 128)) {
    // blocks laid out back to back ([NB, BS, H, D] contiguous, what the cache engine allocates):
    // cache row = block * BS + offset, and the tensor-copy kernel applies
    if (s.block_stride == (int64_t)s.block_size * s.heads * D) {
      constexpr int kStages = APS_KV_STAGES;
      constexpr int kSmem = 1024 + kTmaWarps * kStages * (2 * 16 * D * 2);
      auto kernel = kv_attention_tma_kernel<T, D, kStages>;
      static bool attr_set[64] = {false};
      int dev = 0;
      APS_CUDA(cudaGetDevice(&dev));
      APS_REQUIRE(dev >= 0 && dev < 64, APS_ERR_CUDA, "device index %d out of range", dev);
      if (!attr_set[dev]) {
        APS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
        APS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        attr_set[dev] = true;
      }
      CUtensorMap mk, mv;
      int st = kv_plane_maps<D>(key_cache, value_cache, s, &mk, &mv);
      if (st != APS_OK) return st;
      ScopedProfile prof(0, stream);
      int per_sm = 0;
      APS_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kTmaWarps * 32, kSmem));
      APS_REQUIRE(per_sm > 0, APS_ERR_CUDA, "the K/V streaming kernel does not fit on this device");
      kernel<<<sm_count() * per_sm, kTmaWarps * 32, kSmem, stream>>>(
          mk, mv, ws.plan, ws.part_offset, ws.kv_chunks, ws.part_ml, ws.part_acc, (const T*)query, block_tables,
          seq_lens, s.max_blocks_per_seq, s.heads, s.block_size, s.query_stride, scale_log2);
      return launch_status("kv_attention_tma_kernel");
    }
  }
  ScopedProfile prof(0, stream);
  // CUDA-core arithmetic: 2 persistent CTAs of 8 warps per SM
  const int grid = sm_count() * 2;
  const int threads = kKvWarps * 32;
  kv_attention_kernel<T, D><<<grid, threads, 0, stream>>>(
      ws.plan, ws.part_offset, ws.kv_chunks, ws.part_ml, ws.part_acc, (const T*)query,
      (const T*)key_cache, (const T*)value_cache, block_tables, seq_lens, s.max_blocks_per_seq,
      s.heads, s.block_size, s.query_stride, s.block_stride, scale_log2);
  return launch_status("kv_attention_kernel");
}

template <typename T>
int launch_kv_by_head(const WorkspacePtrs& ws, const void* q, const void* kc, const void* vc,
                      const int32_t* bt, const int32_t* sl, const AttnShape& s, cudaStream_t st) {
  switch (s.head_size) {
    case 32: return launch_kv_typed<T, 32>(ws, q, kc, vc, bt, sl, s, st);
    case 64: return launch_kv_typed<T, 64>(ws, q, kc, vc, bt, sl, s, st);
    case 128: return launch_kv_typed<T, 128>(ws, q, kc, vc, bt, sl, s, st);
    case 256:
      if constexpr (sizeof(T) == 2) return launch_kv_typed<T, 256>(ws, q, kc, vc, bt, sl, s, st);
    default: break;
  }
  return fail(APS_ERR_UNSUPPORTED, "decode attention: head size %d not supported for this dtype",
              s.head_size);
}

}  // namespace

bool kv_attention_supported(int dtype, int head_size) {
  if (head_size == 32 || head_size == 64 || head_size == 128) return dtype_size(dtype) != 0;
  if (head_size == 256) return dtype == APS_F16 || dtype == APS_BF16;
  return false;
}

int launch_plan(const WorkspacePtrs& ws, const int32_t* seq_lens, const int32_t* cache_type,
                const int32_t* block_tables, int batch, int max_blocks_per_seq, int block_size,
                bool pack_tiles, bool kv_present, cudaStream_t stream) {
  plan_kernel<<<1, kPlanThreads, 0, stream>>>(ws.plan, ws.part_offset, ws.kv_chunks, ws.hid_tiles,
                                              ws.first_tile, ws.hid_subs, ws.hid_rows, seq_lens,
                                              cache_type, block_tables, batch,
                                              max_blocks_per_seq * block_size, max_blocks_per_seq,
                                              block_size, pack_tiles ? 1 : 0, kv_present ? 1 : 0);
  return launch_status("plan_kernel");
}

int launch_kv_attention(const WorkspacePtrs& ws, const void* query, const void* key_cache,
                        const void* value_cache, const int32_t* block_tables,
                        const int32_t* seq_lens, const AttnShape& s, cudaStream_t stream) {
  switch (s.dtype) {
    case APS_F32: return launch_kv_by_head<float>(ws, query, key_cache, value_cache, block_tables, seq_lens, s, stream);
    case APS_F16: return launch_kv_by_head<__half>(ws, query, key_cache, value_cache, block_tables, seq_lens, s, stream);
    case APS_BF16: return launch_kv_by_head<__nv_bfloat16>(ws, query, key_cache, value_cache, block_tables, seq_lens, s, stream);
    default: return fail(APS_ERR_DTYPE, "decode attention: unsupported dtype %d", s.dtype);
  }
}

int launch_combine(const WorkspacePtrs& ws, void* out, const int32_t* seq_lens, const AttnShape& s,
                   cudaStream_t stream) {
  (void)seq_lens;
  const int units = s.batch * s.heads;
  const int grid = (units + 7) / 8;
  switch (s.dtype) {
    case APS_F32:
      combine_kernel<float><<<grid, 256, 0, stream>>>(ws.plan, ws.part_offset, ws.part_ml, ws.part_acc,
                                                     (float*)out, s.batch, s.heads, s.head_size, s.out_stride);
      break;
    case APS_F16:
      combine_kernel<__half><<<grid, 256, 0, stream>>>(ws.plan, ws.part_offset, ws.part_ml, ws.part_acc,
                                                      (__half*)out, s.batch, s.heads, s.head_size, s.out_stride);
      break;
    case APS_BF16:
      combine_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(ws.plan, ws.part_offset, ws.part_ml, ws.part_acc,
                                                             (__nv_bfloat16*)out, s.batch, s.heads, s.head_size, s.out_stride);
      break;
    default: return fail(APS_ERR_DTYPE, "decode attention: unsupported dtype %d", s.dtype);
  }
  return launch_status("combine_kernel");
}

// Argument checks shared by the two attention entry points.
int check_attention_args(const char* op, const void* out, const void* query, const void* key_cache,
                         const void* value_cache, const int32_t* block_tables,
                         const int32_t* seq_lens, const AttnShape& s, const void* workspace,
                         size_t workspace_bytes, bool need_kv) {
  const int es = dtype_size(s.dtype);
  APS_REQUIRE(es != 0, APS_ERR_DTYPE, "%s: unsupported dtype %d", op, s.dtype);
  APS_REQUIRE(s.batch >= 0 && s.max_blocks_per_seq > 0 && s.heads > 0 && s.head_size > 0 &&
                  s.block_size > 0,
              APS_ERR_SHAPE, "%s: bad sizes", op);
  APS_REQUIRE(s.block_size % 16 == 0, APS_ERR_UNSUPPORTED,
              "%s: block size must be a multiple of 16 (got %d)", op, s.block_size);
  APS_REQUIRE(kv_attention_supported(s.dtype, s.head_size), APS_ERR_UNSUPPORTED,
              "%s: head size %d is not supported for dtype %d", op, s.head_size, s.dtype);
  if (s.batch == 0) return APS_OK;
  APS_REQUIRE(out && query && block_tables && seq_lens, APS_ERR_NULL_POINTER, "%s: null pointer", op);
  APS_REQUIRE(!need_kv || (key_cache && value_cache), APS_ERR_NULL_POINTER, "%s: null cache pointer", op);
  const int64_t row = (int64_t)s.heads * s.head_size;
  APS_REQUIRE(s.query_stride >= row && s.out_stride >= row &&
                  s.block_stride >= row * s.block_size,
              APS_ERR_SHAPE, "%s: strides smaller than a row / block", op);
  APS_REQUIRE(aligned_to(query, 16) && aligned_to(key_cache, 16) && aligned_to(value_cache, 16) &&
                  (s.query_stride * es) % 16 == 0 && (s.block_stride * es) % 16 == 0 &&
                  (row * es) % 16 == 0 && aligned_to(out, es),
              APS_ERR_MISALIGNED, "%s: query / caches must be 16-byte aligned with 16-byte strides", op);
  const WorkspaceLayout w = workspace_layout(s.batch, s.max_blocks_per_seq, s.block_size, s.heads, s.head_size);
  APS_REQUIRE(workspace != nullptr && aligned_to(workspace, 256) && workspace_bytes >= w.total,
              APS_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned and hold %zu bytes (got %zu)",
              op, w.total, workspace_bytes);
  return APS_OK;
}

}  // namespace aps

using namespace aps;

extern "C" size_t aps_attention_workspace_bytes(int batch, int max_blocks_per_seq, int block_size,
                                                int num_heads, int head_size) {
  if (batch <= 0 || max_blocks_per_seq <= 0 || block_size <= 0 || num_heads <= 0 || head_size <= 0)
    return 0;
  return workspace_layout(batch, max_blocks_per_seq, block_size, num_heads, head_size).total;
}

extern "C" int aps_paged_decode_attention(void* out, const void* query, const void* key_cache,
                                          const void* value_cache, const int32_t* block_tables,
                                          const int32_t* seq_lens, int batch,
                                          int max_blocks_per_seq, int num_heads, int head_size,
                                          int block_size, int64_t query_stride, int64_t out_stride,
                                          int64_t block_stride, float scale, void* workspace,
                                          size_t workspace_bytes, int dtype, void* stream) {
  AttnShape s{batch, max_blocks_per_seq, num_heads, head_size, block_size,
              query_stride, out_stride, block_stride, scale, dtype};
  int st = check_attention_args("paged_decode_attention", out, query, key_cache, value_cache,
                                block_tables, seq_lens, s, workspace, workspace_bytes, true);
  if (st != APS_OK || batch == 0) return st;
  const WorkspaceLayout w = workspace_layout(batch, max_blocks_per_seq, block_size, num_heads, head_size);
  const WorkspacePtrs ws = workspace_ptrs(workspace, w);
  cudaStream_t cs = (cudaStream_t)stream;
  if ((st = launch_plan(ws, seq_lens, nullptr, block_tables, batch, max_blocks_per_seq, block_size, false, true, cs)) != APS_OK) return st;
  if ((st = launch_kv_attention(ws, query, key_cache, value_cache, block_tables, seq_lens, s, cs)) != APS_OK) return st;
  return launch_combine(ws, out, seq_lens, s, cs);
}

extern "C" int aps_attention_status(const void* workspace, int* host_status, void* stream) {
  APS_REQUIRE(workspace != nullptr && host_status != nullptr, APS_ERR_NULL_POINTER,
              "attention_status: null pointer");
  const int* word = static_cast<const int*>(workspace) + kPlanStatus;
  APS_CUDA(cudaMemcpyAsync(host_status, word, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  APS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return APS_OK;
}

extern "C" int aps_reprojection_cycles(const void* workspace, unsigned long long* host_cycles, void* stream) {
  APS_REQUIRE(workspace != nullptr && host_cycles != nullptr, APS_ERR_NULL_POINTER,
              "reprojection_cycles: null pointer");
  const unsigned long long* word =
      reinterpret_cast<const unsigned long long*>(static_cast<const int*>(workspace) + kPlanStatsWord) + 8;
  APS_CUDA(cudaMemcpyAsync(host_cycles, word, sizeof(unsigned long long), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  APS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return APS_OK;
}

// ---- decode attention for callers that cannot allocate -----------------------------
// The scratch of aps_paged_decode_attention_static lives in this module's image: a
// fixed array in device memory that every GPU which loads the library holds until the
// process exits.  Host code may not pass the array's name to a kernel (on the host it
// is only a handle); the device address is looked up with cudaGetSymbolAddress, with the
// calling thread's device current, on EVERY call: the lookup is a table read once the
// module is loaded, and an address kept across calls would go stale when the host tears
// its CUDA context down and creates a new one (cudaDeviceReset, a driver-API host).
namespace aps {
namespace {

constexpr size_t kStaticScratchBytes = size_t(32) << 20;  // 32 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int static_scratch_address(void** out) {
  void* p = nullptr;
  APS_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
  APS_REQUIRE(p != nullptr && aligned_to(p, 256), APS_ERR_CUDA,
              "paged_decode_attention_static: built-in scratch has no usable device address");
  *out = p;
  return APS_OK;
}

}  // namespace
}  // namespace aps

extern "C" int aps_paged_decode_attention_static(void* out, const void* query, const void* key_cache,
                                                 const void* value_cache, const int32_t* block_tables,
                                                 const int32_t* seq_lens, int batch,
                                                 int max_blocks_per_seq, int num_heads, int head_size,
                                                 int block_size, int64_t query_stride,
                                                 int64_t out_stride, int64_t block_stride, float scale,
                                                 int dtype, void* stream) {
  APS_REQUIRE(batch >= 0 && max_blocks_per_seq > 0 && num_heads > 0 && head_size > 0 && block_size > 0,
              APS_ERR_SHAPE, "paged_decode_attention_static: bad sizes");
  const WorkspaceLayout w = workspace_layout(batch > 0 ? batch : 1, max_blocks_per_seq, block_size,
                                             num_heads, head_size);
  APS_REQUIRE(w.total <= kStaticScratchBytes, APS_ERR_WORKSPACE,
              "paged_decode_attention_static: this batch needs %zu bytes of scratch but the built-in "
              "scratch holds %zu (batch %d x %d blocks of %d tokens, %d heads x %d); use "
              "aps_paged_decode_attention with a caller-provided workspace",
              w.total, kStaticScratchBytes, batch, max_blocks_per_seq, block_size, num_heads, head_size);
  AttnShape s{batch, max_blocks_per_seq, num_heads, head_size, block_size,
              query_stride, out_stride, block_stride, scale, dtype};
  // argument checks that do not touch the device come first; the scratch check inside
  // check_attention_args is satisfied by construction
  alignas(256) static unsigned char dummy_ws[256];
  int st = check_attention_args("paged_decode_attention_static", out, query, key_cache, value_cache,
                                block_tables, seq_lens, s, dummy_ws, w.total, true);
  if (st != APS_OK || batch == 0) return st;
  void* scratch = nullptr;
  if ((st = static_scratch_address(&scratch)) != APS_OK) return st;
  const WorkspacePtrs ws = workspace_ptrs(scratch, w);
  cudaStream_t cs = (cudaStream_t)stream;
  // plan_kernel rewrites every word of the scratch header (work counter, status word,
  // list sizes) and every partial that the combine reads is rewritten by this call, so
  // nothing left over from the previous call is ever read
  if ((st = launch_plan(ws, seq_lens, nullptr, block_tables, batch, max_blocks_per_seq, block_size, false, true, cs)) != APS_OK) return st;
  if ((st = launch_kv_attention(ws, query, key_cache, value_cache, block_tables, seq_lens, s, cs)) != APS_OK) return st;
  return launch_combine(ws, out, seq_lens, s, cs);
}

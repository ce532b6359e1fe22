// K/V-path decode attention: a pure HBM-streaming paged attention.
//
// Replaces the third-party flash_attn_with_kvcache call of the reference
// (additional_designs/attention/backends/aptserve_flash_attn.py:452-461) for
// one query token per request over caches laid out [NB, BS, H, D]
// (additional_designs/worker/aptserve_cache_engine.py:61-80).
//
// Work unit: one warp streams one head of one 128-token chunk.  A K (or V) row
// of one head is D*sizeof(T) contiguous bytes; LPR = that / 16 lanes cover a row
// with one 16-byte load each, so a warp-wide load fetches 32/LPR whole rows.
// Scores are reduced over the LPR lanes with shuffles; the softmax is the
// online (running max / running sum) form in the log2 domain.  Loads for the
// next group of tokens are issued before the arithmetic of the current one, so
// every thread keeps 8..16 independent 16-byte loads in flight.
// CTAs are persistent and take 8 warp-units at a time from an atomic counter.

#include "attention_common.cuh"

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
            int max_tokens, int max_blocks, int block_size, int pack_tiles) {
  __shared__ int sa[kPlanThreads], sb[kPlanThreads];
  const int tid = threadIdx.x;
  const int per = (batch + kPlanThreads - 1) / kPlanThreads;
  const int r0 = min(batch, tid * per), r1 = min(batch, r0 + per);
  auto seq_of = [&](int r) { return max(0, min(seq_lens[r], max_tokens)); };
  auto hidden = [&](int r) { return cache_type != nullptr && cache_type[r] != 0; };
  auto subs_of = [&](int s) {   // sub-blocks a hidden request of s tokens occupies in the tile list
    const int n = (s + kSubRowsPlan - 1) / kSubRowsPlan;
    return pack_tiles ? n : (n + 7) / 8 * 8;
  };
  // pass 1: K/V chunks and hidden sub-blocks
  int kv = 0, sub = 0;
  for (int r = r0; r < r1; ++r) {
    const int s = seq_of(r);
    if (hidden(r)) sub += subs_of(s); else kv += (s + kChunkTokens - 1) / kChunkTokens;
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
        slots += (s + kChunkTokens - 1) / kChunkTokens;
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
        const int c = (s + kChunkTokens - 1) / kChunkTokens;
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
    plan[kPlanStatus] = 0;
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

// ---- combine -------------------------------------------------------------------
// One warp per (request, head): merge the request's partials in chunk order.
template <typename T>
__global__ void __launch_bounds__(256)
combine_kernel(const int* __restrict__ part_offset, const float* __restrict__ part_ml,
               const float* __restrict__ part_acc, T* __restrict__ out, int batch, int heads,
               int head_size, int64_t out_stride) {
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= batch * heads) return;
  const int req = unit / heads, h = unit % heads;
  const int p0 = part_offset[req], p1 = part_offset[req + 1];
  float mx = -INFINITY;
  for (int p = p0; p < p1; ++p) mx = fmaxf(mx, part_ml[((int64_t)p * heads + h) * 2]);
  float denom = 0.f;
  for (int p = p0; p < p1; ++p) {
    const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((int64_t)p * heads + h) * 2);
    denom += exp2f(ml.x - mx) * ml.y;
  }
  const float inv = (p1 > p0 && denom > 0.f) ? 1.f / denom : 0.f;
  T* dst = out + req * out_stride + (int64_t)h * head_size;
  for (int d = lane; d < head_size; d += 32) {
    float a = 0.f;
    for (int p = p0; p < p1; ++p) {
      const int64_t slot = (int64_t)p * heads + h;
      a = fmaf(exp2f(part_ml[slot * 2] - mx), part_acc[slot * head_size + d], a);
    }
    dst[d] = Elem<T>::from_float(a * inv);
  }
}

template <typename T, int D>
int launch_kv_typed(const WorkspacePtrs& ws, const void* query, const void* key_cache,
                    const void* value_cache, const int32_t* block_tables, const int32_t* seq_lens,
                    const AttnShape& s, cudaStream_t stream) {
  // 2 persistent CTAs of 8 warps per SM
  const int grid = sm_count() * 2;
  const int threads = kKvWarps * 32;
  const float scale_log2 = s.scale * 1.4426950408889634f;
  ScopedProfile prof(0, stream);
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
                bool pack_tiles, cudaStream_t stream) {
  plan_kernel<<<1, kPlanThreads, 0, stream>>>(ws.plan, ws.part_offset, ws.kv_chunks, ws.hid_tiles,
                                              ws.first_tile, ws.hid_subs, ws.hid_rows, seq_lens,
                                              cache_type, block_tables, batch,
                                              max_blocks_per_seq * block_size, max_blocks_per_seq,
                                              block_size, pack_tiles ? 1 : 0);
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
      combine_kernel<float><<<grid, 256, 0, stream>>>(ws.part_offset, ws.part_ml, ws.part_acc,
                                                     (float*)out, s.batch, s.heads, s.head_size, s.out_stride);
      break;
    case APS_F16:
      combine_kernel<__half><<<grid, 256, 0, stream>>>(ws.part_offset, ws.part_ml, ws.part_acc,
                                                      (__half*)out, s.batch, s.heads, s.head_size, s.out_stride);
      break;
    case APS_BF16:
      combine_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(ws.part_offset, ws.part_ml, ws.part_acc,
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
  if ((st = launch_plan(ws, seq_lens, nullptr, block_tables, batch, max_blocks_per_seq, block_size, false, cs)) != APS_OK) return st;
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

// ---- decode attention for callers that cannot allocate -----------------------------
// The scratch of aps_paged_decode_attention_static lives in this module's image: a
// fixed array in device memory that every GPU which loads the library holds until the
// process exits.  Host code may not pass the array's name to a kernel (on the host it
// is only a handle); the device address is looked up once per device with
// cudaGetSymbolAddress, with that device current, and cached.
namespace aps {
namespace {

constexpr size_t kStaticScratchBytes = size_t(32) << 20;  // 32 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
void* g_static_scratch_addr[64] = {nullptr};

int static_scratch_address(void** out) {
  int dev = 0;
  APS_CUDA(cudaGetDevice(&dev));
  APS_REQUIRE(dev >= 0 && dev < 64, APS_ERR_CUDA, "paged_decode_attention_static: device index %d out of range", dev);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    APS_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    APS_REQUIRE(p != nullptr && aligned_to(p, 256), APS_ERR_CUDA,
                "paged_decode_attention_static: built-in scratch has no usable device address");
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
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
  if ((st = launch_plan(ws, seq_lens, nullptr, block_tables, batch, max_blocks_per_seq, block_size, false, cs)) != APS_OK) return st;
  if ((st = launch_kv_attention(ws, query, key_cache, value_cache, block_tables, seq_lens, s, cs)) != APS_OK) return st;
  return launch_combine(ws, out, seq_lens, s, cs);
}

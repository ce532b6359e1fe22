// Hidden-path decode attention with the projections absorbed into the query and the
// output (no counterpart in the reference, which re-projects every cached hidden row:
// additional_designs/model_executor/models/aptserve_opt.py:111-124).
//
// For a hidden-cached request r and head h the score of cached token t is
//     q . (W_k,h x_t + b_k) = (W_k,h^T q) . x_t + const      (the constant leaves the softmax)
// and the attention output is
//     sum_t p_t (W_v,h x_t + b_v) = W_v,h (sum_t p_t x_t) + b_v.
// With qa[r][h] = scale * log2(e) * W_k,h^T q[r][h] (an E-vector, folded by the caller with one
// batched GEMM) the hidden rows are attended directly, K = V = X with a "head dimension" of
// E, and the caller unfolds z[r][h] = sum_t p_t x_t with W_v,h in a second batched GEMM.
// Three kernels, two of them streaming the hidden rows once:
//   scores_kernel        S[t][h] = x_t . qa[r][h] for every cached token of every hidden
//                        request: one CTA per 128-token tile (grid: tiles of the longest
//                        possible request x requests; CTAs past a request's end return),
//                        mma.sync m16n8k16 over E in 64-element chunks staged by cp.async
//                        (3 stages);
//   softmax_kernel       P[t][h] = softmax over the request's tokens of S[.][h], one CTA per
//                        request (the scores are L2-resident);
//   weighted_sum_kernel  z[r][h][e] = sum_t P[t][h] x_t[e]: one CTA per (request, 512-wide
//                        slice of E), 32-token sub-tiles staged by cp.async (3 stages), P and X
//                        both through ldmatrix.trans, accumulators in registers.
// The warp-level mma.sync is used on purpose: both products have a tiny N (the padded head
// count) and a few MMAs per 16 bytes of X loaded, so the kernels are bound by streaming X,
// not by the tensor pipe.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "aps_common.cuh"

namespace aps {
namespace {

constexpr int kScoreTile = 128;     // tokens per CTA of the scores kernel (8 warps x 16)
constexpr int kScoreThreads = 256;
constexpr int kChunk = 64;          // elements of E per pipeline stage of the scores kernel
constexpr int kScoreStages = 3;

constexpr int kSumSlice = 512;      // columns of E per CTA of the weighted-sum kernel
constexpr int kSumThreads = 256;    // 8 warps x 64 columns
constexpr int kSumTokens = 32;      // tokens per sub-tile
constexpr int kSumStages = 3;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// First hidden-cache row of token `tok` of a request (through its block-table row).
__device__ __forceinline__ int64_t token_row(const int32_t* bt, int tok, int block_size) {
  return (int64_t)bt[tok / block_size] * block_size + tok % block_size;
}

struct AbsorbedArgs {
  const void* x;               // hidden cache, flat rows of x_row_stride elements
  const void* qa;              // [heads_padded][n_req][hidden] absorbed queries (model dtype)
  float* scores;               // [total tokens][heads_padded]
  void* probs;                 // [total tokens][heads_padded] softmax weights (model dtype)
  void* z;                     // [heads_padded][n_req][hidden] (model dtype): the softmax-weighted sums of the hidden rows
  const int32_t* block_tables; // [batch][max_blocks] (all requests of the batch)
  const int32_t* seq_lens;     // [batch]
  const int32_t* req_rows;     // [n_req] batch row of every hidden request
  const int64_t* tok_offset;   // [n_req + 1] first row of every hidden request in `scores`
  int n_req, max_blocks, block_size, hidden, heads_padded;
  int64_t x_row_stride, num_x_rows;
};

// ---- scores -------------------------------------------------------------------------
// Shared memory per stage: X chunk [128 tokens][64 elements] and qa chunk [HP][64], rows of
// 128 bytes, the 16-byte piece j of row r stored at position j ^ (r % 8) (ldmatrix reads
// eight rows at one piece index: without the swizzle they would share their banks).
template <typename T, int HP>
__global__ void __launch_bounds__(kScoreThreads)
scores_kernel(const AbsorbedArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kXBytes = kScoreTile * kChunk * 2, kQBytes = HP * kChunk * 2, kStage = kXBytes + kQBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ri = blockIdx.y, tok0 = blockIdx.x * kScoreTile;
  const int req = a.req_rows[ri];
  const int seq = min(a.seq_lens[req], a.max_blocks * a.block_size);
  if (tok0 >= seq) return;   // the grid covers the longest possible request
  const int32_t* bt = a.block_tables + (int64_t)req * a.max_blocks;
  const T* x = static_cast<const T*>(a.x);
  const T* qa = static_cast<const T*>(a.qa) + (int64_t)ri * a.hidden;   // head h of this request: + h * n_req * hidden
  const int n_chunks = a.hidden / kChunk;

  // this thread's copies per stage: X pieces (128 rows x 8 pieces = 1024, 4 per thread) and
  // qa pieces (HP rows x 8 pieces)
  const T* x_src[4];
  uint32_t x_dst[4];
  bool x_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int piece = threadIdx.x + i * kScoreThreads, row = piece >> 3, j = piece & 7;
    const int tok = tok0 + row;
    const int64_t xr = tok < seq ? token_row(bt, tok, a.block_size) : 0;
    x_ok[i] = tok < seq && xr < a.num_x_rows;
    x_src[i] = x + xr * a.x_row_stride + j * 8;
    x_dst[i] = (uint32_t)(row * 128 + ((j ^ (row & 7)) << 4));
  }
  constexpr int kQPieces = (HP * 8 + kScoreThreads - 1) / kScoreThreads;
  static_assert(HP % 16 == 0, "padded head count must be a multiple of 16");
  const T* q_src[kQPieces];
  uint32_t q_dst[kQPieces];
  bool q_ok[kQPieces];
#pragma unroll
  for (int i = 0; i < kQPieces; ++i) {
    const int piece = threadIdx.x + i * kScoreThreads, j = piece & 7;
    q_ok[i] = piece < HP * 8;
    const int row = q_ok[i] ? piece >> 3 : 0;
    q_src[i] = qa + (int64_t)row * a.n_req * a.hidden + j * 8;
    q_dst[i] = (uint32_t)(kXBytes + row * 128 + ((j ^ (row & 7)) << 4));
  }
  const uint32_t base = smem_addr(smem);
  auto issue = [&](int chunk, int stage) {
    const uint32_t s = base + stage * kStage;
#pragma unroll
    for (int i = 0; i < 4; ++i) cp_async16(s + x_dst[i], x_src[i] + chunk * kChunk, x_ok[i]);
#pragma unroll
    for (int i = 0; i < kQPieces; ++i)
      if (q_ok[i]) cp_async16(s + q_dst[i], q_src[i] + chunk * kChunk, true);
  };

  float acc[HP / 8][4];
#pragma unroll
  for (int n = 0; n < HP / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;

#pragma unroll
  for (int s = 0; s < kScoreStages - 1; ++s) {
    if (s < n_chunks) issue(s, s);
    cp_async_commit();
  }
  // ldmatrix row / piece of this lane: A (16 tokens x 16 k): matrices (rows 0-7, k 0-7),
  // (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15); B (two 8-head tiles x 16 k):
  // (heads 0-7, k 0-7), (heads 0-7, k 8-15), (heads 8-15, k 0-7), (heads 8-15, k 8-15)
  const int a_row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, a_piece = lane >> 4;
  const int b_row = (lane & 7) + ((lane >> 4) & 1) * 8, b_piece = (lane >> 3) & 1;
  for (int c = 0; c < n_chunks; ++c) {
    cp_async_wait<kScoreStages - 2>();
    __syncthreads();
    if (c + kScoreStages - 1 < n_chunks) issue(c + kScoreStages - 1, (c + kScoreStages - 1) % kScoreStages);
    cp_async_commit();
    const uint32_t s = base + (c % kScoreStages) * kStage;
#pragma unroll
    for (int ks = 0; ks < kChunk / 16; ++ks) {
      uint32_t af[4];
      ldmatrix_x4(s + a_row * 128 + (((ks * 2 + a_piece) ^ (a_row & 7)) << 4), af);
#pragma unroll
      for (int np = 0; np < HP / 16; ++np) {
        uint32_t bf[4];
        const int row = np * 16 + b_row;
        ldmatrix_x4(s + kXBytes + row * 128 + (((ks * 2 + b_piece) ^ (row & 7)) << 4), bf);
        mma16816<T>(acc[np * 2], af, bf[0], bf[1]);
        mma16816<T>(acc[np * 2 + 1], af, bf[2], bf[3]);
      }
    }
  }
  cp_async_wait<0>();
  // C fragment: rows g and g + 8 of the warp's 16 tokens, columns 2c, 2c + 1 of every 8-head tile
  const int g = lane >> 2, cq = lane & 3;
  float* out = a.scores + (a.tok_offset[ri] + tok0) * HP;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = warp * 16 + g + half * 8;
    if (tok0 + row < seq) {
#pragma unroll
      for (int n = 0; n < HP / 8; ++n)
        *reinterpret_cast<float2*>(out + (int64_t)row * HP + n * 8 + cq * 2) =
            make_float2(acc[n][half * 2], acc[n][half * 2 + 1]);
    }
  }
}

// ---- softmax over a request's tokens ------------------------------------------------
// One CTA per hidden request: P[t][h] = 2^(S[t][h] - max_t S[.][h]) / sum_t 2^(...), written in
// the model dtype.  Thread (row group rg, column group cgp) walks rows rg, rg + R, ... with
// 16-byte loads, four rows in flight, keeping a running (max, sum) for its four heads; the R row
// groups are merged through shared memory; a second walk writes P.
template <typename T> struct Pack2;
template <> struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t two(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
};
template <> struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t two(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
};

template <typename T, int HP>
__global__ void __launch_bounds__(kSumThreads)
softmax_kernel(const AbsorbedArgs a) {
  constexpr int G = HP / 4, R = kSumThreads / G;
  __shared__ float s_red[R * HP * 2];
  __shared__ float s_max[HP], s_inv[HP];
  const int ri = blockIdx.x;
  const int req = a.req_rows[ri];
  const int seq = min(a.seq_lens[req], a.max_blocks * a.block_size);
  const float* sc = a.scores + a.tok_offset[ri] * HP;
  T* pr = static_cast<T*>(a.probs) + a.tok_offset[ri] * HP;
  const int cgp = threadIdx.x % G, rg = threadIdx.x / G;
  const float4* src = reinterpret_cast<const float4*>(sc) + cgp;
  float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l4[4] = {0.f, 0.f, 0.f, 0.f};
  if (rg < R) {
    for (int t = rg; t < seq; t += 4 * R) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = t + u * R < seq ? src[(int64_t)(t + u * R) * G]
                               : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float e4[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float mn = fmaxf(m4[c], e4[c]);
          if (mn > -INFINITY) l4[c] = l4[c] * exp2f(m4[c] - mn) + exp2f(e4[c] - mn);
          m4[c] = mn;
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      s_red[(rg * HP + cgp * 4 + c) * 2] = m4[c];
      s_red[(rg * HP + cgp * 4 + c) * 2 + 1] = l4[c];
    }
  }
  __syncthreads();
  if (threadIdx.x < HP) {
    float m = -INFINITY, l = 0.f;
    for (int r = 0; r < R; ++r) m = fmaxf(m, s_red[(r * HP + threadIdx.x) * 2]);
    for (int r = 0; r < R; ++r) {
      const float mr = s_red[(r * HP + threadIdx.x) * 2];
      if (mr > -INFINITY) l += s_red[(r * HP + threadIdx.x) * 2 + 1] * exp2f(mr - m);
    }
    s_max[threadIdx.x] = m;
    s_inv[threadIdx.x] = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  if (rg < R) {
    const float mx[4] = {s_max[cgp * 4], s_max[cgp * 4 + 1], s_max[cgp * 4 + 2], s_max[cgp * 4 + 3]};
    const float iv[4] = {s_inv[cgp * 4], s_inv[cgp * 4 + 1], s_inv[cgp * 4 + 2], s_inv[cgp * 4 + 3]};
    for (int t = rg; t < seq; t += R) {
      const float4 v = src[(int64_t)t * G];
      uint2 o;
      o.x = Pack2<T>::two(exp2f(v.x - mx[0]) * iv[0], exp2f(v.y - mx[1]) * iv[1]);
      o.y = Pack2<T>::two(exp2f(v.z - mx[2]) * iv[2], exp2f(v.w - mx[3]) * iv[3]);
      *reinterpret_cast<uint2*>(pr + (int64_t)t * HP + cgp * 4) = o;
    }
  }
}

// ---- weighted sums ------------------------------------------------------------------
// z[h][e] = sum_t P[t][h] x_t[e] for one request and one 512-wide slice of E.  Shared memory
// per stage: an X sub-tile [32 tokens][512 columns] (rows of 1 KB, the 16-byte piece j stored
// at (j & ~7) | ((j ^ row) & 7)) and the sub-tile's P rows [32][HP] (rows padded by 16 bytes).
// Both operands are read with ldmatrix.trans: the tokens are the rows of both tiles and the
// contraction runs over them.
template <typename T, int HP>
__global__ void __launch_bounds__(kSumThreads, HP <= 48 ? 2 : 1)
weighted_sum_kernel(const AbsorbedArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kXBytes = kSumTokens * kSumSlice * 2;          // 32 KB
  constexpr int kPRow = HP * 2 + 16;                           // bytes per P row in shared memory
  constexpr int kStage = kXBytes + kSumTokens * kPRow;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ri = blockIdx.y, slice = blockIdx.x;
  const int req = a.req_rows[ri];
  const int seq = min(a.seq_lens[req], a.max_blocks * a.block_size);
  const int32_t* bt = a.block_tables + (int64_t)req * a.max_blocks;
  const T* x = static_cast<const T*>(a.x) + (int64_t)slice * kSumSlice;
  const T* pr = static_cast<const T*>(a.probs) + a.tok_offset[ri] * HP;
  const int n_sub = (seq + kSumTokens - 1) / kSumTokens;

  const uint32_t base = smem_addr(smem);
  auto issue = [&](int sub, int stage) {
    const uint32_t s = base + stage * kStage;
    // X: 32 rows x 64 pieces = 2048 pieces, 8 per thread; a thread keeps one piece column
    // (threadIdx.x % 64) and walks the rows.  The block size is a multiple of 16, so the 16
    // tokens of each half of the sub-tile sit in one cache block: two block-table lookups.
    const int j = threadIdx.x & 63, r0 = threadIdx.x >> 6;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int tok_first = sub * kSumTokens + half * 16;
      const int64_t row_first = tok_first < seq ? token_row(bt, tok_first, a.block_size) : 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = half * 16 + r0 + i * 4;
        const int64_t xr = row_first + r0 + i * 4;
        const bool ok = sub * kSumTokens + row < seq && xr < a.num_x_rows;
        cp_async16(s + row * 1024 + (((j & ~7) | ((j ^ row) & 7)) << 4), x + (ok ? xr : 0) * a.x_row_stride + j * 8, ok);
      }
    }
    // P: 32 rows x HP / 8 pieces (rows past the end are zero-filled: they weigh nothing)
    constexpr int kPPieces = kSumTokens * (HP / 8);
    for (int pce = threadIdx.x; pce < kPPieces; pce += kSumThreads) {
      const int row = pce / (HP / 8), jj = pce % (HP / 8);
      const int tok = sub * kSumTokens + row;
      cp_async16(s + kXBytes + row * kPRow + jj * 16, pr + (int64_t)(tok < seq ? tok : 0) * HP + jj * 8, tok < seq);
    }
  };
#pragma unroll
  for (int s = 0; s < kSumStages - 1; ++s) {
    if (s < n_sub) issue(s, s);
    cp_async_commit();
  }
  float acc[HP / 16][8][4];
#pragma unroll
  for (int m = 0; m < HP / 16; ++m)
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[m][n][e] = 0.f;
  // A = P^T (16 heads x 16 tokens) through ldmatrix.trans from P[token][head]: matrices
  // (t 0-7, heads 0-7), (t 0-7, heads 8-15), (t 8-15, heads 0-7), (t 8-15, heads 8-15);
  // B through ldmatrix.trans from X[token][column]: (t 0-7, cols 0-7), (t 8-15, cols 0-7),
  // (t 0-7, cols 8-15), (t 8-15, cols 8-15)
  const int a_row = (lane & 7) + ((lane >> 4) & 1) * 8, a_piece = (lane >> 3) & 1;
  const int b_row = (lane & 7) + ((lane >> 3) & 1) * 8, b_piece = lane >> 4;
  for (int sub = 0; sub < n_sub; ++sub) {
    cp_async_wait<kSumStages - 2>();
    __syncthreads();   // the stage has landed; everyone is done with the stage refilled next
    if (sub + kSumStages - 1 < n_sub) issue(sub + kSumStages - 1, (sub + kSumStages - 1) % kSumStages);
    cp_async_commit();
    const uint32_t s = base + (sub % kSumStages) * kStage;
#pragma unroll
    for (int ks = 0; ks < kSumTokens / 16; ++ks) {
      uint32_t bfr[4][4];
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        const int row = ks * 16 + b_row;
        const int j = warp * 8 + np * 2 + b_piece;   // 16-byte piece of the 1 KB row
        ldmatrix_x4_trans(s + row * 1024 + (((j & ~7) | ((j ^ row) & 7)) << 4), bfr[np]);
      }
#pragma unroll
      for (int m = 0; m < HP / 16; ++m) {
        uint32_t af[4];
        ldmatrix_x4_trans(s + kXBytes + (ks * 16 + a_row) * kPRow + ((m * 2 + a_piece) << 4), af);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          mma16816<T>(acc[m][np * 2], af, bfr[np][0], bfr[np][1]);
          mma16816<T>(acc[m][np * 2 + 1], af, bfr[np][2], bfr[np][3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  // C fragment: heads g and g + 8 of every 16-head tile, columns 2c, 2c + 1 of every 8-column tile
  const int g = lane >> 2, cq = lane & 3;
  T* z = static_cast<T*>(a.z) + (int64_t)ri * a.hidden + (int64_t)slice * kSumSlice + warp * 64;
#pragma unroll
  for (int m = 0; m < HP / 16; ++m)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int h = m * 16 + g + half * 8;
#pragma unroll
      for (int n = 0; n < 8; ++n)
        *reinterpret_cast<uint32_t*>(z + (int64_t)h * a.n_req * a.hidden + n * 8 + cq * 2) =
            Pack2<T>::two(acc[m][n][half * 2], acc[m][n][half * 2 + 1]);
    }
}

template <typename T, int HP>
int launch_absorbed(const AbsorbedArgs& a, cudaStream_t stream) {
  {
    constexpr size_t smem1 = (size_t)kScoreStages * (kScoreTile * kChunk * 2 + HP * kChunk * 2);
    auto k1 = scores_kernel<T, HP>;
    APS_CUDA(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
    const int tiles = (a.max_blocks * a.block_size + kScoreTile - 1) / kScoreTile;
    k1<<<dim3(tiles, a.n_req), kScoreThreads, smem1, stream>>>(a);
    int st = launch_status("scores_kernel");
    if (st != APS_OK) return st;
  }
  softmax_kernel<T, HP><<<a.n_req, kSumThreads, 0, stream>>>(a);
  {
    int st = launch_status("softmax_kernel");
    if (st != APS_OK) return st;
  }
  constexpr size_t smem2 = (size_t)kSumStages * (kSumTokens * kSumSlice * 2 + kSumTokens * (HP * 2 + 16));
  auto k2 = weighted_sum_kernel<T, HP>;
  APS_CUDA(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
  // two CTAs per SM need the largest shared-memory carve-out
  APS_CUDA(cudaFuncSetAttribute(k2, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  k2<<<dim3(a.hidden / kSumSlice, a.n_req), kSumThreads, smem2, stream>>>(a);
  return launch_status("weighted_sum_kernel");
}

template <typename T>
int launch_absorbed_hp(const AbsorbedArgs& a, cudaStream_t stream) {
  switch (a.heads_padded) {
    case 16: return launch_absorbed<T, 16>(a, stream);
    case 32: return launch_absorbed<T, 32>(a, stream);
    case 48: return launch_absorbed<T, 48>(a, stream);
    case 80: return launch_absorbed<T, 80>(a, stream);
    default: return fail(APS_ERR_UNSUPPORTED, "absorbed attention: %d padded heads (16, 32, 48, 80)", a.heads_padded);
  }
}

}  // namespace
}  // namespace aps

extern "C" int aps_absorbed_hidden_attention(void* z, float* scores, void* probs, const void* hidden_cache,
                                             const void* absorbed_query, const int32_t* block_tables,
                                             const int32_t* seq_lens, const int32_t* req_rows,
                                             const int64_t* tok_offset,
                                             int n_req, int max_blocks_per_seq,
                                             int block_size, int hidden_size, int heads_padded,
                                             int64_t hidden_row_stride, int64_t num_hidden_rows,
                                             int dtype, void* stream) {
  using namespace aps;
  const char* op = "absorbed_hidden_attention";
  APS_REQUIRE(n_req >= 0 && n_req <= 65535, APS_ERR_SHAPE, "%s: 0..65535 hidden requests", op);
  if (n_req == 0) return APS_OK;
  APS_REQUIRE(z && scores && probs && hidden_cache && absorbed_query && block_tables && seq_lens && req_rows &&
                  tok_offset,
              APS_ERR_NULL_POINTER, "%s: null pointer", op);
  APS_REQUIRE(dtype == APS_F16 || dtype == APS_BF16, APS_ERR_DTYPE, "%s: fp16 or bf16 only", op);
  APS_REQUIRE(hidden_size > 0 && hidden_size % kSumSlice == 0, APS_ERR_UNSUPPORTED,
              "%s: hidden size %d must be a multiple of %d", op, hidden_size, kSumSlice);
  APS_REQUIRE(block_size > 0 && block_size % 16 == 0 && max_blocks_per_seq > 0, APS_ERR_UNSUPPORTED,
              "%s: block size %d", op, block_size);
  APS_REQUIRE(hidden_row_stride >= hidden_size && hidden_row_stride % 8 == 0 && aligned_to(hidden_cache, 16) &&
                  aligned_to(absorbed_query, 16) && aligned_to(z, 16) && aligned_to(scores, 16) && aligned_to(probs, 16),
              APS_ERR_MISALIGNED, "%s: rows must be 16-byte aligned", op);
  AbsorbedArgs a{hidden_cache, absorbed_query, scores, probs, z, block_tables, seq_lens, req_rows, tok_offset,
                 n_req, max_blocks_per_seq, block_size, hidden_size, heads_padded,
                 hidden_row_stride, num_hidden_rows};
  cudaStream_t cs = (cudaStream_t)stream;
  return dtype == APS_BF16 ? launch_absorbed_hp<__nv_bfloat16>(a, cs) : launch_absorbed_hp<__half>(a, cs);
}

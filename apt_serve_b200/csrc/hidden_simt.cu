// Hidden-path decode attention on the CUDA cores: the generic counterpart of the
// tcgen05 kernel for element types and head sizes the tensor-core path does not take
// (fp32, head sizes 32 / 64, fp16 / bf16 with a head size other than 128).
//
// Same work items and the same softmax partials as the tensor-core kernel: one item is
// (128 cached tokens of one hidden-cached request, head h); two threads share a token row,
// each owning half of the head's columns.  K_h and V_h are re-projected in two passes over
// the hidden dimension, 32 elements at a time: a thread holds its row's slab in registers
// (16-byte loads straight from the cache), the pass's W rows are staged in shared memory as
// fp32 and read as broadcast float4, the D / 2 running sums stay in registers.  After the K
// pass the two halves of a row's score are added, after the V pass the weighted V row is
// column-summed over the 128 rows.
// The re-projection it replaces in the reference: additional_designs/model_executor/
// models/aptserve_opt.py:120-124 -> layers/aptserve_linear.py:123-130.

#include "attention_common.cuh"

namespace aps {
namespace {

constexpr int kRows = 128;     // token rows per item
constexpr int kSplit = 2;      // threads per row: each owns D / 2 columns of K (and of V)
constexpr int kSimtThreads = kRows * kSplit;
constexpr int kEC = 32;        // hidden elements per slab

// 32 consecutive elements of a row as fp32, by 16-byte loads when the slab is whole and aligned.
template <typename T>
__device__ __forceinline__ void load_slab(const T* __restrict__ row, int e0, int hidden, bool vec_ok,
                                          bool valid, float* __restrict__ out) {
  if (!valid) {
#pragma unroll
    for (int e = 0; e < kEC; ++e) out[e] = 0.f;
    return;
  }
  if (vec_ok && e0 + kEC <= hidden) {
    constexpr int kPer = 16 / (int)sizeof(T);
    const uint4* src = reinterpret_cast<const uint4*>(row + e0);
#pragma unroll
    for (int v = 0; v < kEC / kPer; ++v) {
      const uint4 raw = src[v];
      const T* el = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < kPer; ++j) out[v * kPer + j] = Elem<T>::to_float(el[j]);
    }
  } else {
#pragma unroll 4
    for (int e = 0; e < kEC; ++e) out[e] = e0 + e < hidden ? Elem<T>::to_float(row[e0 + e]) : 0.f;
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kSimtThreads)
hidden_simt_kernel(const int* __restrict__ plan, const int* __restrict__ part_offset,
                   const int2* __restrict__ hid_tiles, float* __restrict__ part_ml,
                   float* __restrict__ part_acc, const T* __restrict__ query,
                   const T* __restrict__ x_base, const T* __restrict__ w_k, const T* __restrict__ b_k,
                   const T* __restrict__ w_v, const T* __restrict__ b_v,
                   const int32_t* __restrict__ block_tables, const int32_t* __restrict__ seq_lens,
                   int max_blocks_per_seq, int block_size, int heads, int hidden, int64_t query_stride,
                   int64_t x_row_stride, int64_t w_stride, float scale_log2, int vec_ok) {
  constexpr int DH = D / kSplit;                 // columns per thread
  __shared__ __align__(16) float ws[D][kEC];     // the pass's W rows of this slab; read as broadcast float4
  __shared__ float red[4][D];
  __shared__ float part_s[kSplit][kRows];
  __shared__ float red_s[kSplit][8];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int r = t % kRows, half = t / kRows;     // half is uniform across a warp
  const int d0 = half * DH;
  const int n_items = plan[kPlanNumHidTiles] * heads;

  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int tile = item / heads, h = item % heads;
    const int2 rc = hid_tiles[tile];
    const int req = rc.x, chunk = rc.y;
    const int seq = min(seq_lens[req], max_blocks_per_seq * block_size);
    const int tok = chunk * kRows + r;
    const bool valid = tok < seq;
    const int32_t* bt = block_tables + (int64_t)req * max_blocks_per_seq;
    const int64_t row = valid ? (int64_t)bt[tok / block_size] * block_size + tok % block_size : 0;
    const T* xrow = x_base + row * x_row_stride;
    const T* q = query + req * query_stride + h * D;

    float s = 0.f, mx = 0.f, pr = 0.f;
    for (int pass = 0; pass < 2; ++pass) {
      const T* w = (pass == 0 ? w_k : w_v) + (int64_t)h * D * w_stride;
      const T* bias = pass == 0 ? b_k : b_v;
      float acc[DH];
#pragma unroll
      for (int d = 0; d < DH; ++d) acc[d] = 0.f;
      for (int e0 = 0; e0 < hidden; e0 += kEC) {
        float xr[kEC];
        load_slab<T>(xrow, e0, hidden, vec_ok != 0, valid, xr);   // in flight while W is staged
        __syncthreads();
        for (int i = t; i < D * kEC; i += kSimtThreads) {
          const int d = i / kEC, e = i % kEC;
          ws[d][e] = e0 + e < hidden ? Elem<T>::to_float(w[(int64_t)d * w_stride + e0 + e]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int d = 0; d < DH; ++d) {
          float a = acc[d];
          const float4* wrow = reinterpret_cast<const float4*>(&ws[d0 + d][0]);
#pragma unroll
          for (int e = 0; e < kEC / 4; ++e) {
            const float4 w4 = wrow[e];
            a = fmaf(xr[4 * e], w4.x, a);
            a = fmaf(xr[4 * e + 1], w4.y, a);
            a = fmaf(xr[4 * e + 2], w4.z, a);
            a = fmaf(xr[4 * e + 3], w4.w, a);
          }
          acc[d] = a;
        }
      }
      if (pass == 0) {
        // this thread's half of the score; the row's score is the sum of its two halves
        float sp = 0.f;
#pragma unroll
        for (int d = 0; d < DH; ++d) {
          const float kd = acc[d] + (bias ? Elem<T>::to_float(bias[h * D + d0 + d]) : 0.f);
          sp = fmaf(Elem<T>::to_float(q[d0 + d]) * scale_log2, kd, sp);
        }
        __syncthreads();
        part_s[half][r] = sp;
        __syncthreads();
        s = valid ? part_s[0][r] + part_s[1][r] : -INFINITY;
        // block max and weight (both halves compute the same values from the same 128 scores)
        float wm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
        if (lane == 0) red_s[half][warp & 3] = wm;
        __syncthreads();
        mx = fmaxf(fmaxf(red_s[half][0], red_s[half][1]), fmaxf(red_s[half][2], red_s[half][3]));
        pr = valid ? exp2f(s - mx) : 0.f;
        float wsum = pr;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
        if (lane == 0) red_s[half][4 + (warp & 3)] = wsum;
      } else {
        // column sums of p * (V + b_v) over the 128 rows
#pragma unroll
        for (int d = 0; d < DH; ++d) {
          float v = valid ? pr * (acc[d] + (bias ? Elem<T>::to_float(bias[h * D + d0 + d]) : 0.f)) : 0.f;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) red[warp & 3][d0 + d] = v;
        }
        __syncthreads();
        const int64_t slot = (int64_t)(part_offset[req] + chunk) * heads + h;
        for (int d = t; d < D; d += kSimtThreads)
          part_acc[slot * D + d] = red[0][d] + red[1][d] + red[2][d] + red[3][d];
        if (t == 0)
          *reinterpret_cast<float2*>(part_ml + slot * 2) =
              make_float2(mx, red_s[0][4] + red_s[0][5] + red_s[0][6] + red_s[0][7]);
      }
    }
    __syncthreads();
  }
}

template <typename T, int D>
int launch_typed(const WorkspacePtrs& ws, const SimtHiddenArgs& a, cudaStream_t stream) {
  const int grid = sm_count() * 4;
  // 16-byte loads of the hidden rows need aligned rows
  const int vec_ok = (reinterpret_cast<uintptr_t>(a.x_base) % 16 == 0 &&
                      (a.x_row_stride * (int64_t)sizeof(T)) % 16 == 0) ? 1 : 0;
  hidden_simt_kernel<T, D><<<grid, kSimtThreads, 0, stream>>>(
      ws.plan, ws.part_offset, ws.hid_tiles, ws.part_ml, ws.part_acc, (const T*)a.query,
      (const T*)a.x_base, (const T*)a.w_k, (const T*)a.b_k, (const T*)a.w_v, (const T*)a.b_v,
      a.block_tables, a.seq_lens, a.max_blocks_per_seq, a.block_size, a.heads, a.hidden,
      a.query_stride, a.x_row_stride, a.w_stride, a.scale * 1.4426950408889634f, vec_ok);
  return launch_status("hidden_simt_kernel");
}

template <typename T>
int launch_by_head(const WorkspacePtrs& ws, const SimtHiddenArgs& a, cudaStream_t stream) {
  switch (a.head_size) {
    case 32: return launch_typed<T, 32>(ws, a, stream);
    case 64: return launch_typed<T, 64>(ws, a, stream);
    case 128: return launch_typed<T, 128>(ws, a, stream);
    default: break;
  }
  return fail(APS_ERR_UNSUPPORTED, "hybrid_decode_attention: head size %d is not supported by the "
              "CUDA-core re-projection (32, 64, 128)", a.head_size);
}

}  // namespace

bool hidden_simt_supported(int dtype, int head_size) {
  return dtype_size(dtype) != 0 && (head_size == 32 || head_size == 64 || head_size == 128);
}

int launch_hidden_simt(const WorkspacePtrs& ws, const SimtHiddenArgs& a, cudaStream_t stream) {
  ScopedProfile prof(1, stream);   // the same timing hook as the tensor-core re-projection
  switch (a.dtype) {
    case APS_F32: return launch_by_head<float>(ws, a, stream);
    case APS_F16: return launch_by_head<__half>(ws, a, stream);
    case APS_BF16: return launch_by_head<__nv_bfloat16>(ws, a, stream);
    default: return fail(APS_ERR_DTYPE, "hybrid_decode_attention: unsupported dtype %d", a.dtype);
  }
}

}  // namespace aps

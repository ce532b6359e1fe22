// Hidden-path decode attention on the CUDA cores: the generic counterpart of the
// tcgen05 kernel for element types and head sizes the tensor-core path does not take
// (fp32, head sizes 32 / 64, fp16 / bf16 with a head size other than 128).
//
// Same work items and the same softmax partials as the tensor-core kernel: one item is
// (128 cached tokens of one hidden-cached request, head h); thread t owns token row t.
// K_h and V_h are re-projected in two passes over the hidden dimension, 32 elements at a
// time: the X rows and the W rows of the pass are staged in shared memory as fp32, every
// thread keeps the D running sums of its row in registers.  After the K pass the thread
// has its score, after the V pass the weighted V row is column-summed over the 128 rows.
// The re-projection it replaces in the reference: additional_designs/model_executor/
// models/aptserve_opt.py:120-124 -> layers/aptserve_linear.py:123-130.

#include "attention_common.cuh"

namespace aps {
namespace {

constexpr int kRows = 128;     // token rows per item == threads per CTA
constexpr int kEC = 32;        // hidden elements per staged slab

template <typename T, int D>
__global__ void __launch_bounds__(kRows)
hidden_simt_kernel(const int* __restrict__ plan, const int* __restrict__ part_offset,
                   const int2* __restrict__ hid_tiles, float* __restrict__ part_ml,
                   float* __restrict__ part_acc, const T* __restrict__ query,
                   const T* __restrict__ x_base, const T* __restrict__ w_k, const T* __restrict__ b_k,
                   const T* __restrict__ w_v, const T* __restrict__ b_v,
                   const int32_t* __restrict__ block_tables, const int32_t* __restrict__ seq_lens,
                   int max_blocks_per_seq, int block_size, int heads, int hidden, int64_t query_stride,
                   int64_t x_row_stride, int64_t w_stride, float scale_log2) {
  __shared__ float xs[kRows][kEC + 1];
  __shared__ float ws[D][kEC + 1];
  __shared__ float red[4][D];
  __shared__ float red_s[8];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int n_items = plan[kPlanNumHidTiles] * heads;

  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int tile = item / heads, h = item % heads;
    const int2 rc = hid_tiles[tile];
    const int req = rc.x, chunk = rc.y;
    const int seq = min(seq_lens[req], max_blocks_per_seq * block_size);
    const int tok = chunk * kRows + t;
    const bool valid = tok < seq;
    const int32_t* bt = block_tables + (int64_t)req * max_blocks_per_seq;
    const int64_t row = valid ? (int64_t)bt[tok / block_size] * block_size + tok % block_size : 0;
    const T* xrow = x_base + row * x_row_stride;
    const T* q = query + req * query_stride + h * D;

    float s = 0.f, mx = 0.f, pr = 0.f;
    for (int pass = 0; pass < 2; ++pass) {
      const T* w = (pass == 0 ? w_k : w_v) + (int64_t)h * D * w_stride;
      const T* bias = pass == 0 ? b_k : b_v;
      float acc[D];
#pragma unroll
      for (int d = 0; d < D; ++d) acc[d] = 0.f;
      for (int e0 = 0; e0 < hidden; e0 += kEC) {
        __syncthreads();
        // stage X[128 x 32]: thread t copies its own row slab; W[D x 32]: strided over the CTA
#pragma unroll 4
        for (int e = 0; e < kEC; ++e)
          xs[t][e] = (valid && e0 + e < hidden) ? Elem<T>::to_float(xrow[e0 + e]) : 0.f;
        for (int i = t; i < D * kEC; i += kRows) {
          const int d = i / kEC, e = i % kEC;
          ws[d][e] = e0 + e < hidden ? Elem<T>::to_float(w[(int64_t)d * w_stride + e0 + e]) : 0.f;
        }
        __syncthreads();
        float xr[kEC];
#pragma unroll
        for (int e = 0; e < kEC; ++e) xr[e] = xs[t][e];
#pragma unroll
        for (int d = 0; d < D; ++d) {
          float a = acc[d];
#pragma unroll
          for (int e = 0; e < kEC; ++e) a = fmaf(xr[e], ws[d][e], a);
          acc[d] = a;
        }
      }
      if (pass == 0) {
        // score of this row, block max, weight
#pragma unroll
        for (int d = 0; d < D; ++d) {
          const float kd = acc[d] + (bias ? Elem<T>::to_float(bias[h * D + d]) : 0.f);
          s = fmaf(Elem<T>::to_float(q[d]) * scale_log2, kd, s);
        }
        s = valid ? s : -INFINITY;
        float wm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
        __syncthreads();
        if (lane == 0) red_s[warp] = wm;
        __syncthreads();
        mx = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
        pr = valid ? exp2f(s - mx) : 0.f;
        float wsum = pr;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
        if (lane == 0) red_s[4 + warp] = wsum;
      } else {
        // column sums of p * (V + b_v) over the 128 rows
#pragma unroll
        for (int d = 0; d < D; ++d) {
          float v = valid ? pr * (acc[d] + (bias ? Elem<T>::to_float(bias[h * D + d]) : 0.f)) : 0.f;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) red[warp][d] = v;
        }
        __syncthreads();
        const int64_t slot = (int64_t)(part_offset[req] + chunk) * heads + h;
        for (int d = t; d < D; d += kRows)
          part_acc[slot * D + d] = red[0][d] + red[1][d] + red[2][d] + red[3][d];
        if (t == 0)
          *reinterpret_cast<float2*>(part_ml + slot * 2) =
              make_float2(mx, red_s[4] + red_s[5] + red_s[6] + red_s[7]);
      }
    }
    __syncthreads();
  }
}

template <typename T, int D>
int launch_typed(const WorkspacePtrs& ws, const SimtHiddenArgs& a, cudaStream_t stream) {
  const int grid = sm_count() * 4;
  hidden_simt_kernel<T, D><<<grid, kRows, 0, stream>>>(
      ws.plan, ws.part_offset, ws.hid_tiles, ws.part_ml, ws.part_acc, (const T*)a.query,
      (const T*)a.x_base, (const T*)a.w_k, (const T*)a.b_k, (const T*)a.w_v, (const T*)a.b_v,
      a.block_tables, a.seq_lens, a.max_blocks_per_seq, a.block_size, a.heads, a.hidden,
      a.query_stride, a.x_row_stride, a.w_stride, a.scale * 1.4426950408889634f);
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

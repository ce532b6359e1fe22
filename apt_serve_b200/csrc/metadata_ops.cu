// Device-side construction of the decode batch's index tensors.
//
// The reference builds them on the host: for every hidden-cached request a Python loop
// over all of its positions appends two slot ids (additional_designs/worker/
// aptserve_model_runner.py:527-539), the boolean masks are turned into index tensors
// (:613-648) and everything is shipped to the device (and broadcast to the
// tensor-parallel workers) every step -- about 2 x 8 bytes per cached hidden token.
// Here the host ships the two block tables, the sequence lengths and the cache types
// (a few bytes per 16 tokens) and two small kernels expand them in place:
//   layout_kernel   one CTA: prefix sums over the requests -> where each request starts
//                   in the expanded token space, among the hidden tokens, and its ordinal
//                   among the K/V-cached / hidden-cached requests;
//   fill_kernel     one CTA per request: writes the request's entries of all eight tensors.
// Integer work only; results are bit-identical to the host construction.
//
// The caller sizes the outputs from its own view of the batch (num_tot_tokens,
// num_hidden_tokens) and may pass NULL for an output that is empty in that view.  The kernels
// trust neither: layout_kernel recomputes the four totals from the device-side seq_lens and
// cache_type, and fill_kernel writes nothing at all unless they equal the caller's claim;
// every store is bounded by its tensor's capacity besides.

#include "aps_common.cuh"

namespace aps {
namespace {

constexpr int kScanThreads = 1024;

struct MetaLayout {       // per request, in the caller's scratch; entry [B] of each = the total
  int* exp_off;           // [B + 1] start in the expanded token space
  int* hid_off;           // [B + 1] start among the hidden tokens
  int* kv_ord;            // [B + 1] ordinal among the K/V-cached requests
  int* hid_ord;           // [B + 1] ordinal among the hidden-cached requests
};

__global__ void __launch_bounds__(kScanThreads)
layout_kernel(MetaLayout L, const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ cache_type,
              int batch, int max_tokens, int64_t* __restrict__ counts) {
  __shared__ int s[4][kScanThreads];
  const int tid = threadIdx.x;
  const int per = (batch + kScanThreads - 1) / kScanThreads;
  const int r0 = min(batch, tid * per), r1 = min(batch, r0 + per);
  int v[4] = {0, 0, 0, 0};   // expanded tokens, hidden tokens, K/V requests, hidden requests
  for (int r = r0; r < r1; ++r) {
    const int len = max(1, min(seq_lens[r], max_tokens));
    if (cache_type[r] != 0) { v[0] += len; v[1] += len; v[3] += 1; }
    else { v[0] += 1; v[2] += 1; }
  }
  for (int k = 0; k < 4; ++k) s[k][tid] = v[k];
  __syncthreads();
  for (int off = 1; off < kScanThreads; off <<= 1) {
    int a[4] = {0, 0, 0, 0};
    if (tid >= off) for (int k = 0; k < 4; ++k) a[k] = s[k][tid - off];
    __syncthreads();
    for (int k = 0; k < 4; ++k) s[k][tid] += a[k];
    __syncthreads();
  }
  int o[4];
  for (int k = 0; k < 4; ++k) o[k] = s[k][tid] - v[k];
  for (int r = r0; r < r1; ++r) {
    const int len = max(1, min(seq_lens[r], max_tokens));
    L.exp_off[r] = o[0]; L.hid_off[r] = o[1]; L.kv_ord[r] = o[2]; L.hid_ord[r] = o[3];
    if (cache_type[r] != 0) { o[0] += len; o[1] += len; o[3] += 1; }
    else { o[0] += 1; o[2] += 1; }
  }
  if (tid == kScanThreads - 1) {
    L.exp_off[batch] = s[0][tid]; L.hid_off[batch] = s[1][tid];
    L.kv_ord[batch] = s[2][tid]; L.hid_ord[batch] = s[3][tid];
    if (counts != nullptr) { counts[0] = s[0][tid]; counts[1] = s[1][tid]; counts[2] = s[2][tid]; counts[3] = s[3][tid]; }
  }
}

struct MetaOut {
  int64_t* slot_mapping; int64_t* slot_mapping_shared; int64_t* hidden_cache_use_tot;
  int64_t* kv_cache_use_tot; int64_t* hidden_holder_upd; int64_t* hidden_holder_pull;
  int64_t* hidden_cache_store_tot; int64_t* hidden_cache_use_input;
  int64_t cap_tot, cap_hidden;   // capacities of the [N_tot] and [N_h] tensors (the caller's claim)
  int64_t cap_kv_req, cap_hid_req;   // capacities of the per-request lists [n_kv] and [n_h]
};

__global__ void __launch_bounds__(256)
fill_kernel(MetaLayout L, MetaOut O, const int32_t* __restrict__ block_tables,
            const int32_t* __restrict__ block_tables_shared, const int32_t* __restrict__ seq_lens,
            const int32_t* __restrict__ cache_type, int batch, int max_blocks, int block_size) {
  // the device-side totals must be what the caller sized (and NULL-ed) the outputs for
  if (L.exp_off[batch] != O.cap_tot || L.hid_off[batch] != O.cap_hidden ||
      L.kv_ord[batch] != O.cap_kv_req || L.hid_ord[batch] != O.cap_hid_req)
    return;
  for (int r = blockIdx.x; r < batch; r += gridDim.x) {
    const int len = max(1, min(seq_lens[r], max_blocks * block_size));
    const int64_t e0 = L.exp_off[r];
    const int32_t* priv = block_tables + (int64_t)r * max_blocks;
    if (cache_type[r] != 0) {
      const int64_t h0 = L.hid_off[r];
      const int32_t* shar = block_tables_shared + (int64_t)r * max_blocks;
      for (int j = threadIdx.x; j < len; j += blockDim.x) {
        const int b = j / block_size, o = j % block_size;
        if (e0 + j < O.cap_tot) O.slot_mapping[e0 + j] = (int64_t)priv[b] * block_size + o;
        if (h0 + j < O.cap_hidden) {
          O.slot_mapping_shared[h0 + j] = (int64_t)shar[b] * block_size + o;
          O.hidden_cache_use_tot[h0 + j] = e0 + j;
        }
        // every earlier request holds exactly one "current token" entry, and so far none of this one
        if (j < len - 1 && e0 + j - r >= 0 && e0 + j - r < O.cap_tot - batch) O.hidden_holder_pull[e0 + j - r] = e0 + j;
      }
      if (threadIdx.x == 0) {
        O.hidden_holder_upd[r] = e0 + len - 1;
        const int ord = L.hid_ord[r];
        if (ord < O.cap_hid_req) {
          O.hidden_cache_store_tot[ord] = e0 + len - 1;
          O.hidden_cache_use_input[ord] = r;
        }
      }
    } else if (threadIdx.x == 0) {
      const int j = len - 1;
      if (e0 < O.cap_tot) O.slot_mapping[e0] = (int64_t)priv[j / block_size] * block_size + j % block_size;
      if (L.kv_ord[r] < O.cap_kv_req) O.kv_cache_use_tot[L.kv_ord[r]] = e0;
      O.hidden_holder_upd[r] = e0;
    }
  }
}

}  // namespace
}  // namespace aps

using namespace aps;

extern "C" size_t aps_decode_metadata_scratch_bytes(int batch) {
  return batch <= 0 ? 0 : (size_t)(4 * (batch + 1)) * sizeof(int);
}

extern "C" int aps_expand_decode_metadata(const int32_t* block_tables, const int32_t* block_tables_shared,
                                          const int32_t* seq_lens, const int32_t* cache_type, int batch,
                                          int max_blocks_per_seq, int block_size, int64_t* slot_mapping,
                                          int64_t* slot_mapping_shared, int64_t* hidden_cache_use_tot,
                                          int64_t* kv_cache_use_tot, int64_t* hidden_holder_upd,
                                          int64_t* hidden_holder_pull, int64_t* hidden_cache_store_tot,
                                          int64_t* hidden_cache_use_input, int64_t num_tot_tokens,
                                          int64_t num_hidden_tokens, int64_t* counts, void* scratch,
                                          size_t scratch_bytes, void* stream) {
  APS_REQUIRE(batch >= 0 && max_blocks_per_seq > 0 && block_size > 0 && num_tot_tokens >= batch &&
                  num_hidden_tokens >= 0 && num_hidden_tokens <= num_tot_tokens &&
                  num_tot_tokens - num_hidden_tokens <= batch,
              APS_ERR_SHAPE, "expand_decode_metadata: bad sizes (N_tot = %lld, N_h = %lld, batch = %d)",
              (long long)num_tot_tokens, (long long)num_hidden_tokens, batch);
  if (batch == 0) return APS_OK;
  // outputs whose length is zero for this batch may be NULL (an empty tensor has no storage)
  APS_REQUIRE(block_tables && seq_lens && cache_type && slot_mapping && hidden_holder_upd,
              APS_ERR_NULL_POINTER, "expand_decode_metadata: null pointer");
  // every hidden request holds at least one token, so N_h == 0 means there is none
  APS_REQUIRE(num_hidden_tokens == 0 || (block_tables_shared && slot_mapping_shared &&
                                         hidden_cache_use_tot && hidden_cache_store_tot &&
                                         hidden_cache_use_input),
              APS_ERR_NULL_POINTER, "expand_decode_metadata: null pointer (hidden-request outputs)");
  APS_REQUIRE(num_tot_tokens == num_hidden_tokens || kv_cache_use_tot != nullptr, APS_ERR_NULL_POINTER,
              "expand_decode_metadata: null pointer (kv_cache_use_tot)");
  APS_REQUIRE(num_tot_tokens == batch || hidden_holder_pull != nullptr, APS_ERR_NULL_POINTER,
              "expand_decode_metadata: null pointer (hidden_holder_pull)");
  APS_REQUIRE(scratch != nullptr && aligned_to(scratch, 4) &&
                  scratch_bytes >= aps_decode_metadata_scratch_bytes(batch),
              APS_ERR_WORKSPACE, "expand_decode_metadata: scratch must hold %zu bytes",
              aps_decode_metadata_scratch_bytes(batch));
  int* sc = static_cast<int*>(scratch);
  MetaLayout L{sc, sc + (batch + 1), sc + 2 * (batch + 1), sc + 3 * (batch + 1)};
  MetaOut O{slot_mapping, slot_mapping_shared, hidden_cache_use_tot, kv_cache_use_tot,
            hidden_holder_upd, hidden_holder_pull, hidden_cache_store_tot, hidden_cache_use_input,
            num_tot_tokens, num_hidden_tokens, num_tot_tokens - num_hidden_tokens,
            batch - (num_tot_tokens - num_hidden_tokens)};
  cudaStream_t cs = (cudaStream_t)stream;
  layout_kernel<<<1, kScanThreads, 0, cs>>>(L, seq_lens, cache_type, batch,
                                            max_blocks_per_seq * block_size, counts);
  int st = launch_status("layout_kernel");
  if (st != APS_OK) return st;
  const int grid = batch < sm_count() * 8 ? batch : sm_count() * 8;
  fill_kernel<<<grid, 256, 0, cs>>>(L, O, block_tables, block_tables_shared, seq_lens, cache_type,
                                    batch, max_blocks_per_seq, block_size);
  return launch_status("fill_kernel");
}

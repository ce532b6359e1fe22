// One decode layer-step of the hybrid-cache path in one call.
//
// What the reference does between the projections and o_proj of a decode layer with
// hidden-cached requests (additional_designs/model_executor/models/aptserve_opt.py:99-134
// with additional_designs/attention/backends/aptserve_flash_attn.py:331-387, 449-475):
// write the new token's layer-input row for hidden-cached requests (hidden_to_cache), write
// the new token's K/V rows for K/V-cached requests (mixed_kv_to_cache / reshape_and_cache_flash),
// then attend.  Here that is one host call that enqueues three launches on the caller's
// stream: a bulk-copy launch for all new-token rows, addressed straight from the private
// block tables, the sequence lengths and the cache-type mask (no int64 index tensors), and
// the hybrid decode attention (plan, K/V streaming, re-projection, combine).

#include "attention_common.cuh"

using namespace aps;

extern "C" int aps_decode_layer_step(void* out, const void* query, const void* hidden_states,
                                     const void* new_key, const void* new_value, void* key_cache,
                                     void* value_cache, void* hidden_cache, const void* w_k,
                                     const void* b_k, const void* w_v, const void* b_v,
                                     const int32_t* block_tables, const int32_t* seq_lens,
                                     const int32_t* cache_type, int batch, int max_blocks_per_seq,
                                     int num_heads, int head_size, int hidden_size, int block_size,
                                     int64_t query_stride, int64_t out_stride, int64_t hidden_states_stride,
                                     int64_t new_key_stride, int64_t new_value_stride, int64_t block_stride,
                                     int64_t hidden_row_stride, int64_t num_hidden_rows, int64_t w_stride,
                                     float scale, void* workspace, size_t workspace_bytes, int dtype,
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
  int st = check_hybrid_call("decode_layer_step", c);
  if (st != APS_OK || batch == 0) return st;
  APS_REQUIRE(hidden_size > 0 && hidden_states_stride >= hidden_size, APS_ERR_SHAPE,
              "decode_layer_step: bad hidden_states stride");
  const int64_t row = (int64_t)num_heads * head_size;
  APS_REQUIRE(new_key == nullptr || (new_key_stride >= row && new_value_stride >= row), APS_ERR_SHAPE,
              "decode_layer_step: new_key / new_value strides smaller than a row");
  APS_REQUIRE(hidden_states == nullptr || hidden_row_stride >= hidden_size, APS_ERR_SHAPE,
              "decode_layer_step: hidden cache rows shorter than the hidden size");
  cudaStream_t cs = (cudaStream_t)stream;
  NewTokenWrite nw{hidden_states, new_key, new_value, key_cache, value_cache, hidden_cache,
                   block_tables, seq_lens, cache_type, batch, max_blocks_per_seq, block_size,
                   num_heads, head_size, hidden_size, hidden_states_stride, new_key_stride,
                   new_value_stride, block_stride, hidden_row_stride, dtype};
  if ((st = launch_new_token_write(nw, cs)) != APS_OK) return st;
  return enqueue_hybrid_attention(c, cs);
}

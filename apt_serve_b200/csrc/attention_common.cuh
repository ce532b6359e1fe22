// Work planning, scratch layout and launch declarations shared by the K/V-path
// and hidden-path decode attention kernels.
//
// A decode batch is cut into CHUNKS of kChunkTokens consecutive tokens of one
// request.  Every chunk of a K/V-cached request is streamed by warps of the
// K/V kernel (one warp per head); every chunk of a hidden-cached request is one
// 128-row M tile of the re-projection GEMM.  Each (chunk, head) leaves a softmax
// partial (running max and sum in the log2 domain, un-normalised fp32
// accumulator) in the scratch buffer; a combine kernel merges a request's
// partials in chunk order, so the result does not depend on scheduling.
#pragma once

#include "aps_common.cuh"

namespace aps {

constexpr int kChunkTokens = 128;
constexpr int kSubRowsPlan = 16;   // rows of one sub-block of a hidden request's tile list

// Header words at the start of the scratch buffer (device-written).
enum PlanWord {
  kPlanNumKvChunks = 0,   // chunks of K/V-cached requests
  kPlanNumHidTiles = 1,   // chunks (M tiles) of hidden-cached requests
  kPlanKvCounter = 2,     // dynamic work counter of the K/V kernel
  kPlanHidCounter = 3,    // reserved
  kPlanStatus = 4,        // device status of the last call that used this scratch (StatusCode)
  kPlanNumHidSubs = 5,    // 16-row sub-blocks in the hidden requests' tile list (incl. padding entries)
  kPlanStatsWord = 16,    // 8 x 64-bit cycle counters of the re-projection kernel (debug aid), then
                          // one more: SM cycles its CTA 0 spent in the last launch
  kPlanWords = 64
};

// Values of the status word.  1..7: a bounded mbarrier wait of the re-projection kernel ran
// out (the code names the waiting role); the combine kernel then fills the whole output with
// NaN.  8: the batch holds K/V-cached requests but the call was given no K/V cache; their
// output rows are zero, the hidden-cached requests' rows are valid.
enum StatusCode {
  kStatusOk = 0,
  kStatusWaitFirst = 1,
  kStatusWaitLast = 7,
  kStatusNoKvCache = 8
};

struct WorkspaceLayout {
  int batch, heads, head_size, max_chunks;  // max_chunks = batch * chunks per longest request
  size_t off_plan, off_part_offset, off_kv_chunks, off_hid_tiles, off_first_tile, off_hid_subs,
      off_hid_rows, off_ml, off_acc, total;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline WorkspaceLayout workspace_layout(int batch, int max_blocks_per_seq, int block_size,
                                        int heads, int head_size) {
  WorkspaceLayout w;
  w.batch = batch; w.heads = heads; w.head_size = head_size;
  const int64_t max_tokens = (int64_t)max_blocks_per_seq * block_size;
  const int64_t per_req = (max_tokens + kChunkTokens - 1) / kChunkTokens;
  // one partial per 128-token chunk; a hidden request whose tiles are packed across requests
  // can touch one tile more than it has chunks
  const int64_t mc = (int64_t)batch * ((per_req > 0 ? per_req : 1) + 1);
  const int64_t subs = (int64_t)batch * (((max_tokens + kSubRowsPlan - 1) / kSubRowsPlan + 7) / 8 * 8) + 8;
  w.max_chunks = (int)mc;
  size_t o = 0;
  w.off_plan = o;        o = align_up(o + kPlanWords * sizeof(int), 256);
  w.off_part_offset = o; o = align_up(o + (size_t)(batch + 1) * sizeof(int), 256);
  w.off_kv_chunks = o;   o = align_up(o + (size_t)mc * sizeof(int2), 256);
  w.off_hid_tiles = o;   o = align_up(o + (size_t)mc * sizeof(int2), 256);
  w.off_first_tile = o;  o = align_up(o + (size_t)(batch + 1) * sizeof(int), 256);
  w.off_hid_subs = o;    o = align_up(o + (size_t)subs * sizeof(int2), 256);
  w.off_hid_rows = o;    o = align_up(o + (size_t)subs * sizeof(int), 256);
  w.off_ml = o;          o = align_up(o + (size_t)mc * heads * 2 * sizeof(float), 256);
  w.off_acc = o;         o = align_up(o + (size_t)mc * heads * head_size * sizeof(float), 256);
  w.total = o;
  return w;
}

struct WorkspacePtrs {
  int* plan;
  int* part_offset;   // [batch + 1] first partial slot of each request
  int2* kv_chunks;    // (request, chunk) of K/V-cached requests, request order
  int2* hid_tiles;    // (request, chunk) of hidden-cached requests, request order (unpacked plan only)
  int* first_tile;    // [batch] first M tile a hidden request has rows in
  int2* hid_subs;     // per 16-row sub-block of the M tiles: (request, first token) or (-1, 0) padding
  int* hid_rows;      // per sub-block: first row in the hidden cache (through the block table)
  float* part_ml;     // [slot][head][2]
  float* part_acc;    // [slot][head][head_size]
};

inline WorkspacePtrs workspace_ptrs(void* base, const WorkspaceLayout& w) {
  char* b = static_cast<char*>(base);
  WorkspacePtrs p;
  p.plan = reinterpret_cast<int*>(b + w.off_plan);
  p.part_offset = reinterpret_cast<int*>(b + w.off_part_offset);
  p.kv_chunks = reinterpret_cast<int2*>(b + w.off_kv_chunks);
  p.hid_tiles = reinterpret_cast<int2*>(b + w.off_hid_tiles);
  p.first_tile = reinterpret_cast<int*>(b + w.off_first_tile);
  p.hid_subs = reinterpret_cast<int2*>(b + w.off_hid_subs);
  p.hid_rows = reinterpret_cast<int*>(b + w.off_hid_rows);
  p.part_ml = reinterpret_cast<float*>(b + w.off_ml);
  p.part_acc = reinterpret_cast<float*>(b + w.off_acc);
  return p;
}

struct AttnShape {
  int batch, max_blocks_per_seq, heads, head_size, block_size;
  int64_t query_stride, out_stride, block_stride;
  float scale;
  int dtype;
};

// cache_type may be NULL (all requests K/V-cached).  The M tiles of the hidden requests are
// described in 16-row sub-blocks (hid_subs, 8 per tile).  pack_tiles = false: every request
// starts a new tile (tile = 128-token chunk, hid_tiles is filled too); pack_tiles = true:
// the sub-blocks of consecutive hidden requests are packed back to back, so a tile can hold
// rows of several requests and only the last tile is partly empty.
// kv_present = false: the call has no K/V cache; K/V-cached requests then get no work and no
// partials (zero output rows) and the status word is set to kStatusNoKvCache.
int launch_plan(const WorkspacePtrs& ws, const int32_t* seq_lens, const int32_t* cache_type,
                const int32_t* block_tables, int batch, int max_blocks_per_seq, int block_size,
                bool pack_tiles, bool kv_present, cudaStream_t stream);

int launch_kv_attention(const WorkspacePtrs& ws, const void* query, const void* key_cache,
                        const void* value_cache, const int32_t* block_tables,
                        const int32_t* seq_lens, const AttnShape& s, cudaStream_t stream);

int launch_combine(const WorkspacePtrs& ws, void* out, const int32_t* seq_lens,
                   const AttnShape& s, cudaStream_t stream);

bool kv_attention_supported(int dtype, int head_size);

// Argument checks shared by the attention entry points.
int check_attention_args(const char* op, const void* out, const void* query, const void* key_cache,
                         const void* value_cache, const int32_t* block_tables,
                         const int32_t* seq_lens, const AttnShape& s, const void* workspace,
                         size_t workspace_bytes, bool need_kv);

// CUDA-core re-projection for the shapes the tensor-core kernel does not take.
struct SimtHiddenArgs {
  const void* query; const void* x_base; const void* w_k; const void* b_k; const void* w_v; const void* b_v;
  const int32_t* block_tables; const int32_t* seq_lens;
  int max_blocks_per_seq, block_size, heads, head_size, hidden;
  int64_t query_stride, x_row_stride, w_stride;
  float scale;
  int dtype;
};
bool hidden_simt_supported(int dtype, int head_size);
int launch_hidden_simt(const WorkspacePtrs& ws, const SimtHiddenArgs& a, cudaStream_t stream);

// One hybrid decode attention call (the arguments of aps_hybrid_decode_attention).
struct HybridCall {
  AttnShape shape;
  void* out; const void* query; const void* key_cache; const void* value_cache;
  const void* hidden_cache; const void* w_k; const void* b_k; const void* w_v; const void* b_v;
  const int32_t* block_tables; const int32_t* seq_lens; const int32_t* cache_type;
  int hidden_size;
  int64_t hidden_row_stride, num_hidden_rows, w_stride;
  void* workspace; size_t workspace_bytes;
};
// New-token cache writes of a decode batch addressed from the block tables (cache_ops.cu).
// key == NULL: no K/V rows are written; hidden == NULL: no hidden rows are written.
struct NewTokenWrite {
  const void* hidden; const void* key; const void* value; void* key_cache; void* value_cache; void* hidden_cache;
  const int32_t* block_tables; const int32_t* seq_lens; const int32_t* cache_type;
  int batch, max_blocks_per_seq, block_size, heads, head_size, hidden_size;
  int64_t hidden_stride, key_stride, value_stride, block_stride, slot_stride;
  int dtype;
};
int launch_new_token_write(const NewTokenWrite& a, cudaStream_t stream);

int check_hybrid_call(const char* op, const HybridCall& c);
int enqueue_hybrid_attention(const HybridCall& c, cudaStream_t stream);

}  // namespace aps

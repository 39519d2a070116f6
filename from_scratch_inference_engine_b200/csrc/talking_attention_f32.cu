// The mixed-heads attention for float32 pages (the kernels are in talking_attention.cuh), and
// the entry point that picks the storage type.
#include "talking_attention.cuh"

using namespace fsie;

extern "C" int fsie_talking_attention_bf16(TalkingArgs args, int num_tiles, cudaStream_t stream);

extern "C" {

// Consecutive tokens of one request in a block's tile: 8, 4, 2 or 1 as the heads grow (a warp
// owns heads / 8 heads, rounded up, times that many tokens: 8 rows at most); 0: too many heads.
int fsie_talking_attention_tile_tokens(int heads) {
    if (heads <= 0 || heads > TA_ROWS) return 0;
    return 8 / (heads <= 8 ? 1 : heads <= 16 ? 2 : heads <= 32 ? 4 : 8);
}

// Keys that a block takes at a time for these sizes (0: the sizes do not fit shared memory).
int fsie_talking_attention_key_tile(int heads, int kv_heads, int dim, int vdim, int dtype) {
    return talking_key_tile(heads, kv_heads, dim, vdim, dtype == DTYPE_F32 ? 4 : 2);
}

// nsplit > 1 splits every tile's keys over that many blocks and needs part_stats
// [tiles * nsplit * 64 * 2] and part_out [nsplit * tokens * heads * vdim] (float).
int fsie_talking_attention(const float* q, const void* k_pages, const void* v_pages,
                           long long page_stride, int page_size, const int* block_tables,
                           int table_stride, const int* tile_item, const int* tile_row0, int num_tiles,
                           const int* item_qstart, const int* item_qlen, const int* item_pos0,
                           const int* item_slots, const float* talk, void* out, int tokens, int heads,
                           int kv_heads, int dim, int vdim, int window, int keep_first, int tile_tokens,
                           float scale, int nsplit, float* part_stats, float* part_out, int dtype,
                           int* error, cudaStream_t stream) {
    TalkingArgs a = {q, k_pages, v_pages, page_stride, page_size, block_tables, table_stride,
                     tile_item, tile_row0, item_qstart, item_qlen, item_pos0, item_slots, talk, out,
                     heads, kv_heads, dim, vdim, window, keep_first, tile_tokens, scale, error,
                     nsplit, 0, part_stats, part_out, tokens};
    if (dtype == DTYPE_F32) return talking_attention_launch<float>(a, num_tiles, stream);
    return fsie_talking_attention_bf16(a, num_tiles, stream);
}

}  // extern "C"

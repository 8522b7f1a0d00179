// Argument blocks of mx_decode_fused (decode_fused.cu). Plain C layout: the Python side
// mirrors these with ctypes structures and checks the sizes with mx_decode_fused_sizes.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#define MX_DF_MAX_GROUPS 4

// One entry of the model's schedule: a pre-norm block of LayerNorm -> attention (fused QKV,
// NeoX rotation over the whole head, paged cache) -> LayerNorm -> up / GELU(tanh) / down.
struct MxDfLayer {
    const float* ln1_w;
    const float* ln1_b;            // may be null
    const float* ln2_w;
    const float* ln2_b;            // may be null
    const __nv_bfloat16* qkv_w;    // [(heads + 2 kv heads) * head_dim][hidden]
    const __nv_bfloat16* o_w;      // [hidden][heads * head_dim]
    const __nv_bfloat16* fc_w;     // [inter][hidden]
    const __nv_bfloat16* proj_w;   // [hidden][inter]
    const float* qkv_b;            // biases may be null
    const float* o_b;
    const float* fc_b;
    const float* proj_b;
    const float* inv_freq;         // [head_dim / 2]
    __nv_bfloat16* cache;          // [page][2][kv head][page_size * head_dim] of this entry
    // tensor maps (128 bytes each, in device memory) over the four matrices, boxes of 256 columns
    // by 8 rows (QKV: a unit is two groups of 8 rows) or 16 rows (the others)
    const void* qkv_map;
    const void* o_map;
    const void* fc_map;
    const void* proj_map;
    long long n_pages;
    float ln1_eps, ln2_eps;
    float scale_log2;              // softmax scale * log2(e)
    int window;                    // 0: every key
    int group;                     // which set of block tables / slots
    int writes_cache;              // 0: the entry reads another entry's pages
};

struct MxDfParams {
    const MxDfLayer* layers;       // device array
    const int* token_ids;          // [rows]
    const int* tok_seq;            // [rows] -1 marks a padding row
    const int* context_lens;       // [rows] tokens cached before this step = position of the new token
    const int* slots[MX_DF_MAX_GROUPS];          // [rows] cache slot of the new token, -1 for padding
    const int* block_tables[MX_DF_MAX_GROUPS];   // [rows][bt_stride]
    int bt_stride[MX_DF_MAX_GROUPS];
    const __nv_bfloat16* embedding;              // [vocab][hidden]
    const float* final_w;
    const float* final_b;          // may be null
    const __nv_bfloat16* head;     // [vocab][hidden]
    const void* head_map;          // tensor map over the head, boxes of 256 columns by 16 rows
    float* x;                      // [rows][hidden] residual stream
    __nv_bfloat16* xb;             // [rows][hidden] the same rounded to bfloat16: what the norms read
    __nv_bfloat16* q;              // [rows][heads * head_dim] rotated queries
    __nv_bfloat16* attn;           // [rows][heads * head_dim]
    __nv_bfloat16* mid;            // [rows][inter]
    float* part_o;                 // [rows][heads][splits][head_dim]
    float* part_ml;                // [rows][heads][splits][2]  (max in log2 units, sum)
    float* stats;                  // [16][grid rounded up to 32][4]  (count, mean, M2) per row and block
    float* logits;                 // [rows][vocab]
    unsigned* barrier;             // one counter, zero at launch
    int* status;
    float final_eps;
    int n_layers, rows, hidden, n_heads, n_kv_heads, head_dim, inter, vocab;
    int page_size, n_splits;
    int x_cols;                    // columns of the activation stage in shared memory
    int xs_bytes;                  // its size
    int ring_slots;
    int grid;
};

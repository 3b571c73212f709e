// Argument block shared by the attention launchers (attention.cu, attention_mma.cu); mirrors
// titan_b200.kernels.AttnArgs.
#pragma once
#include "common.cuh"
#include "qk_args.h"

// Where the tensor-core prompt kernels take keys and values from.
#define TB_KV_FROM_STEP 1      // the step's own rows: every sequence of the step starts at position 0
#define TB_KV_FROM_CACHE 2     // the cache's pages, where the step's own keys have been appended already

struct AttnArgs {
    const void* q; int q_stride;            // [T][q_stride], head h at h*hd
    const void* kv_new; int kv_stride;      // [T][kv_stride]: K heads then V heads of this step (may be null)
    void* out; int out_stride;              // [T][out_stride]
    TbKvView cache;                         // storage may be null when every key is in kv_new
    TbBatch batch;
    int nh; int nkv; int hd;
    int window;                             // 0: all keys
    float scale;
    int chunk;                              // decode: fewest keys per split (see tb_split_keys)
    int n_splits;                           // decode: grid.z, the most splits a sequence is cut into
    float* scratch;                         // decode: [B][nh][n_splits][hd + 2]
    // decode, optional: lengths that were final before the step's first kernel ran, so that a kernel may read
    // them without waiting for its predecessors.  early_mode 1: early_len[b] = batch.kv_len[b] (the same numbers,
    // put there by a copy, not by a kernel); 2: early_len[slot] + 1 = batch.kv_len[b] (the cache's committed
    // length of the slot, for steps whose kv_len a kernel of the step computes); 0 or a null pointer: none.
    const int* early_len; int early_mode;
    // decode on tensor cores, optional: the head norm / rotary / append step folded into the attention kernel.  The
    // queries and the new token's key and value then come as the projection's float32 sums (fused_qk->in, rows of
    // fused_qk->in_stride: Q heads, K heads, V heads), with the norm weights, the rotary block, the row scales and the
    // cache of *fused_qk; ``q`` is not read.  Null: queries are bfloat16 rows at ``q`` and the cache holds every key.
    const QkArgs* fused_qk;
};

// How decode attention cuts the keys of ONE sequence into splits: ``chunk`` keys each while ``n_splits`` of
// them cover the sequence, else ``n_splits`` equal parts of whole 64-key pages.  Split s takes keys
// [s * keys, (s + 1) * keys) below the length; splits that start at or beyond the length are empty.  The
// borders depend on the sequence's own length and on the launch's two numbers, never on the other sequences
// of the batch, on the longest context the engine allows or on where the sequence lies in the cache.
// (berniehans/titan: num_splits = min(32, ceil(S / 256)), engine/engine-cuda/src/paged_attention.rs:368-370.)
__host__ __device__ __forceinline__ int tb_split_keys(int len, int chunk, int n_splits) {
    if ((long long)chunk * n_splits >= len) return chunk;
    return (((len + n_splits - 1) / n_splits) + 63) & ~63;
}

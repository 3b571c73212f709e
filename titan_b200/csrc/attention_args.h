// Argument block shared by the attention launchers (attention.cu, attention_mma.cu); mirrors
// titan_b200.kernels.AttnArgs.
#pragma once
#include "common.cuh"

struct AttnArgs {
    const void* q; int q_stride;            // [T][q_stride], head h at h*hd
    const void* kv_new; int kv_stride;      // [T][kv_stride]: K heads then V heads of this step (may be null)
    void* out; int out_stride;              // [T][out_stride]
    TbKvView cache;                         // storage may be null when every key is in kv_new
    TbBatch batch;
    int nh; int nkv; int hd;
    int window;                             // 0: all keys
    float scale;
    int chunk;                              // decode: keys per split
    int n_splits;                           // decode: grid.z
    float* scratch;                         // decode: [B][nh][n_splits][hd + 2]
    // decode, optional: lengths that were final before the step's first kernel ran, so that a kernel may read
    // them without waiting for its predecessors.  early_mode 1: early_len[b] = batch.kv_len[b] (the same numbers,
    // put there by a copy, not by a kernel); 2: early_len[slot] + 1 = batch.kv_len[b] (the cache's committed
    // length of the slot, for steps whose kv_len a kernel of the step computes); 0 or a null pointer: none.
    const int* early_len; int early_mode;
};

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
};

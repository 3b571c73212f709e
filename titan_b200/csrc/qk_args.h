// Argument block of the Q/K head norm + rotary (+ cache append) step, shared by its own kernel
// (elementwise.cu) and by the matrix product that does the same in its epilogue (gemm_tc.cu); mirrors
// titan_b200.kernels.QkArgs.
#pragma once
#include "common.cuh"

struct QkArgs {
    const void* in; int in_stride;          // [T][in_stride]: Q | K | V
    void* q_out; int q_stride;              // [T][q_stride]
    void* k_out; int k_stride;              // [T][k_stride] (null: K goes to the cache only)
    const float* q_w; const float* k_w;     // [hd] or null
    const float* inv_freq;                  // [rot/2] or null (no rotation)
    float eps; int rot; int nh; int nkv; int hd;
    const int* pos_of; const int* seq_of; const int* slot_of_seq;
    TbKvView cache; int append; int T;
    int zero_in;                            // after reading a head, write zeros over it (an accumulation buffer is left clean)
    const int* kv_len;                      // [B] lengths after the step: in a ring, a row that a later token of the step reuses is not written
};

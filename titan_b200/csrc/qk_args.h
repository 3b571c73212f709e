// Argument block of the Q/K head norm + rotary (+ cache append) kernel (elementwise.cu); mirrors
// titan_b200.kernels.QkArgs.
#pragma once
#include "common.cuh"

// What a position encoding hands to the kernels (titan_b200.kernels.RotaryArgs): the mixer passes it on
// without looking inside.  angle_k(position) = (position + offset) * inv_freq[k]; the pair
// (k, k + rot/2) of a head is rotated by that angle and scaled by ``magnitude``.
struct TbRotary {
    const float* inv_freq;                  // [rot/2] or null (no rotation)
    int rot;                                // leading dims of a head that are rotated
    float offset;                           // added to every position (0 for plain rotary)
    float magnitude;                        // factor on cosines and sines (1 for plain rotary)
};

struct QkArgs {
    const void* in; int in_stride;          // [T][in_stride]: Q | K | V
    void* q_out; int q_stride;              // [T][q_stride]
    void* k_out; int k_stride;              // [T][k_stride] (null: K goes to the cache only)
    const float* q_w; const float* k_w;     // [hd] or null
    TbRotary rope;
    float eps; int nh; int nkv; int hd;
    const int* pos_of; const int* seq_of; const int* slot_of_seq;
    TbKvView cache; int append; int T;
    int zero_in;                            // after reading a head, write zeros over it (an accumulation buffer is left clean)
    const int* kv_len;                      // [B] lengths after the step: in a ring, a row that a later token of the step reuses is not written
    // The input rows are products of UNSCALED activations (the RMS norm before the projection was folded into the
    // product): row t is first multiplied by 1/sqrt(sum_z row_sumsq[z][t] / row_width + row_eps), the row_parts partial
    // sums [part][32] added in the order of the parts.  Null: the rows are as they should be.
    const float* row_sumsq; int row_parts; int row_width; float row_eps;
};

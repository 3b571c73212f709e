// Declaration of the one entry point of this library that never allocates device memory.
//
// This entry point has no counterpart in berniehans/titan: its decode attention keeps its split
// partials in a buffer that the driver object allocates when it is built
// (engine/engine-cuda/src/paged_attention.rs:110-122).
//
// Who needs it: a host program that may not call cudaMalloc once it is running.  Two such callers
// are a serving process that hands the whole device to its own memory pool at start-up, so that a
// later cudaMalloc by anyone else fails, and a control loop with a latency budget, for which the
// implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.  Everywhere else
// in this library the scratch of split-KV decode attention is a tensor that the caller (the Python
// engine) allocates; here it is a fixed array inside the library image.
//
// tb_attn_decode_noalloc computes exactly what tb_attn_decode computes (attention.cu): one query per
// sequence over its cached keys, cut into at most ``n_splits`` splits of ``chunk`` keys or more
// (tb_split_keys in attention_args.h), then the merge of the splits.  The caller passes the same argument block, inputs and outputs as for tb_attn_decode;
// the ``scratch`` field is ignored.
//
// Limits and rules
//   * The scratch is TB_NOALLOC_SCRATCH_FLOATS float32 values (8 MiB).  Every GPU that loads the
//     library holds that much until the process exits, used or not.  A call needs
//     B * query_heads * n_splits * (head_dim + 2) values and is refused, with a message that names
//     both numbers, if that is more.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) with that
//     device current and remembers it.  Make that first call before any stream capture begins.
//   * Every call uses the same array, which keeps what the last call left in it.  Nothing in it has
//     to start at zero: each chunk's partial result is written before the merge reads it, and the
//     merge reads only the chunks its sequence has.  Two calls that overlap on the GPU (different
//     streams, or graphs replayed concurrently) race on the array; run them one after the other.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any path.
#pragma once
#include <cuda_runtime.h>

#include "attention_args.h"

#define TB_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)

// dtype: TB_F32 or TB_BF16.  Returns 0, or non-zero with the reason in tb_last_error().
extern "C" int tb_attn_decode_noalloc(const AttnArgs* args, int dtype, cudaStream_t stream);

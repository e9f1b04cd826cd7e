// Argument block of the ring-attention forward.
//
// The first twelve fields are the reference's Ring_fwd_params (csrc/ring.h:5-19), same names, order
// and meaning, so code that fills the reference struct fills this one.  The fields after the marker
// are what the benchmark configurations need and the reference lacks (csrc/ring_attention.cu:422-426
// is single batch / single head, non-causal, no LSE output).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

struct Ring_fwd_params
{
    int mype;             // this rank
    int npes;             // ring size
    int *seqlen;          // unused by this implementation (the reference keeps a device copy here)
    int *h_seqlen;        // host: rows held by each rank (they may differ, as the reference's seqlen[] allows)
    int dim;              // head dimension (64 or 128)
    float softmax_scale;  // NATURAL-base scale s: weights = softmax(s * q.k).  (The reference stores 1.0
                          // and feeds it to exp2, csrc/ring_attention.cu:389,597; log2(e) is applied here.)
    void *q_ptr;          // [batch, heads, seqlen_local, dim] fp16, device
    void *k_ptr;          // same layout; this rank's shard
    void *v_ptr;
    void *out_ptr;        // [batch, heads, seqlen_local, dim] fp32, device
    void *k_buffer;       // unused: receive buffers belong to the context, not to the call
    void *v_buffer;
    // ---- extensions -------------------------------------------------------------------------
    int batch;            // B (reference: 1)
    int heads;            // H (reference: 1)
    void *lse_ptr;        // [batch, heads, seqlen_local] fp32 natural-log row LSE, device; may be null
    int causal;           // 0/1: mask k_global > q_global (contiguous sharding)
    int is_bf16;          // 0 = fp16 inputs, 1 = bf16 inputs
    cudaStream_t stream;  // compute stream; the call is asynchronous on it
};

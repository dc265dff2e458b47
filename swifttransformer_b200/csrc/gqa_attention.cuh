// What the grouped-attention kernels share: which keys a query sees, and the extra term of the softmax.
//
// Cache layout (one page of one cache entry), the one of the differential attention with one key map
// (DiffCache with kd = dim):
//   keys   [kv_head][position in page][dim]    at offset 0
//   values [kv_head][position in page][vd]     at offset nkv * page_size * dim
//
// Mask.  The query at position p sees key j when j <= p and (p - j < window or j < keep_first); window <= 0:
// every j <= p.  The seen keys are two ranges of positions: the kept first ones [0, head_end) with
// head_end = min(keep_first, lo), and the recent ones [lo, p] with lo = max(0, p - window + 1).
//
// Softmax.  With has_sink the denominator holds one more term exp(sink) that has no value row:
//   w_j = exp(s_j) / (exp(sink) + sum_i exp(s_i)).
#pragma once
#include "diff_attention.cuh"

struct GqaMask {
    int window, keep_first;
};

__device__ __forceinline__ int gqa_lo(int pos, const GqaMask& m) { return m.window > 0 ? max(0, pos - m.window + 1) : 0; }
__device__ __forceinline__ int gqa_head_end(int lo, const GqaMask& m) { return m.window > 0 ? min(m.keep_first, lo) : 0; }
__device__ __forceinline__ bool gqa_seen(int key, int pos, const GqaMask& m) {
    return key <= pos && (m.window <= 0 || pos - key < m.window || key < m.keep_first);
}

// What is done to a head's result before it is stored: times out_scale, and, with gate, times
// sigmoid(gate[token * gate_ld + head * vd + e]) (gate logits as a product left them, in the storage type).
// sinks: with has_sink, the extra term's logit of every head (float [heads]); null: the one `sink` for all heads.
struct GqaEpilogue {
    const void* gate;
    long long gate_ld;
    float out_scale;
    const float* sinks;
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }

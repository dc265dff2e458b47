// Attention with weights mixed over the heads (talk_attention.cu) for single tokens and short portions in
// bfloat16, as two kernels, so that a step of few tokens still fills many blocks:
//
//   talk_scores   grid (token, key/value head, run of TS_KEYS seen keys): a thread per key fetches the whole key row
//                 in 16-byte pieces and takes its dot products with the group's queries (scaled floats in shared
//                 memory); the raw scores go to a float scratch [token][head][number of the seen key].
//   talk_values   grid (token, key/value head): all heads' scores of the token into shared memory, a warp per head
//                 finds maximum and sum (the extra term joins) and normalises in place; a thread per key then forms
//                 the mixed weights of the block's own heads, P'_a = sum_b T[a][b] P_b; the warps share the keys,
//                 their lanes side by side along the value row (a 16-byte piece each), and the warps' sums meet in
//                 shared memory, where gate and out_scale are applied.
//
// The seen keys of a token are numbered in one run (the kept first ones, then the window up to the query), as in
// gqa_attention_single.  The scratch holds n_cap numbers per (token, head): n_cap is the most keys a token of the
// step sees, given by the caller.  All heads' weights of a token must fit in shared memory (heads * n_cap floats);
// st_talk_attention_single_applies says whether they do.
#include "gqa_attention.cuh"

#define TS_THREADS 256
#define TS_KEYS 256          // seen keys per block of talk_scores
#define TS_MAX_REP 8
#define TV_THREADS 256
#define TV_WARPS (TV_THREADS / 32)
#define TV_ROWS 4            // value rows a lane asks for at once

__global__ void __launch_bounds__(TS_THREADS)
talk_scores_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, DiffCache cache,
                   float* __restrict__ scores, int n_cap, const int* __restrict__ items,
                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                   const int* __restrict__ slots, const int* __restrict__ block_table, int nh, float scale,
                   GqaMask mask, int* __restrict__ status) {
    extern __shared__ float ts_q[];                     // [rep][dim] queries times scale
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x;
    if (t < 0) return;
    const int pos = positions[t];
    if (pos < 0) return;
    const int dim = cache.kd, ps = cache.page_size, nkv = cache.nkv;
    const int c = blockIdx.y, rep = nh / nkv, h0 = c * rep;
    const int lo = gqa_lo(pos, mask), head_end = gqa_head_end(lo, mask);
    const int total = head_end + pos + 1 - lo;
    const int i = blockIdx.z * TS_KEYS + threadIdx.x;
    if (blockIdx.z * TS_KEYS >= total) return;
    for (int x = threadIdx.x; x < rep * dim; x += TS_THREADS)
        ts_q[x] = load1_cg(q + ((size_t)t * nh + h0) * dim + x) * scale;
    __syncthreads();
    if (i >= total) return;
    const int key = i < head_end ? i : lo + (i - head_end);
    const int page = block_table[(size_t)slots[seq_of_token[t]] * cache.max_pages + key / ps];
    float* dst = scores + ((size_t)blockIdx.x * nh + h0) * n_cap + i;
    if (page < 0) {
        if (status) *status = 1;
        for (int r = 0; r < rep; ++r) dst[(size_t)r * n_cap] = -INFINITY;
        return;
    }
    const uint4* kp = reinterpret_cast<const uint4*>(cache_keys(pool, cache, page, c, key % ps));
    const int pieces = dim / 8;
    for (int r0 = 0; r0 < rep; r0 += TS_MAX_REP) {
        float s[TS_MAX_REP];
#pragma unroll
        for (int r = 0; r < TS_MAX_REP; ++r) s[r] = 0.f;
        for (int p = 0; p < pieces; ++p) {
            const uint4 kk = __ldcg(kp + p);
            const uint32_t w4[4] = {kk.x, kk.y, kk.z, kk.w};
            float kf[8];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                kf[2 * x] = __uint_as_float(w4[x] << 16);
                kf[2 * x + 1] = __uint_as_float(w4[x] & 0xffff0000u);
            }
#pragma unroll
            for (int r = 0; r < TS_MAX_REP; ++r) {
                if (r0 + r >= rep) break;
                const float* qr = ts_q + (r0 + r) * dim + p * 8;
                float d = s[r];
#pragma unroll
                for (int x = 0; x < 8; ++x) d = fmaf(qr[x], kf[x], d);
                s[r] = d;
            }
        }
#pragma unroll
        for (int r = 0; r < TS_MAX_REP; ++r)
            if (r0 + r < rep) dst[(size_t)(r0 + r) * n_cap] = s[r];
    }
}

template <int REP>
__global__ void __launch_bounds__(TV_THREADS)
talk_values_kernel(const float* __restrict__ scores, int n_cap, const bf16* __restrict__ pool, DiffCache cache,
                   bf16* __restrict__ out, const int* __restrict__ items, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                   const int* __restrict__ block_table, int nh, GqaMask mask, const float* __restrict__ talk,
                   int has_sink, GqaEpilogue epi, int gate_heads) {
    extern __shared__ __align__(16) float tv_smem[];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x;
    if (t < 0) return;
    const int pos = positions[t];
    if (pos < 0) return;
    const int vd = cache.vd, ps = cache.page_size, nkv = cache.nkv;
    const int c = blockIdx.y, rep = nh / nkv, h0 = c * rep;
    const int lo = gqa_lo(pos, mask), head_end = gqa_head_end(lo, mask);
    const int total = head_end + pos + 1 - lo;
    const int ld = (total + 3) & ~3;
    float* sp = tv_smem;                                 // [nh][ld] weights of all heads
    float* sw = sp + (size_t)nh * ld;                    // [REP][ld] mixed weights of the block's heads
    float* so = sw + (size_t)REP * ld;                   // [TV_WARPS][REP][vd]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* src = scores + (size_t)blockIdx.x * nh * n_cap;
    for (int h = warp; h < nh; h += TV_WARPS) {
        float m = -INFINITY;
        for (int j = lane; j < total; j += 32) {
            const float s = __ldcg(src + (size_t)h * n_cap + j);
            sp[(size_t)h * ld + j] = s;
            m = fmaxf(m, s);
        }
        m = warp_max(m);
        const float sk = has_sink ? epi.sinks[h] : -INFINITY;
        m = fmaxf(m, sk);
        float sum = 0.f;
        for (int j = lane; j < total; j += 32) {
            const float s = sp[(size_t)h * ld + j];
            const float p = s > -INFINITY ? expf(s - m) : 0.f;
            sp[(size_t)h * ld + j] = p;
            sum += p;
        }
        sum = warp_sum(sum) + (has_sink ? expf(sk - m) : 0.f);
        const float inv = sum > 0.f ? 1.f / sum : 0.f;
        for (int j = lane; j < total; j += 32) sp[(size_t)h * ld + j] *= inv;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < total; j += TV_THREADS) {
        float w[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) w[r] = 0.f;
        for (int b = 0; b < nh; ++b) {
            const float p = sp[(size_t)b * ld + j];
#pragma unroll
            for (int r = 0; r < REP; ++r)
                if (r < rep) w[r] = fmaf(talk ? talk[(size_t)(h0 + r) * nh + b] : (b == h0 + r ? 1.f : 0.f), p, w[r]);
        }
#pragma unroll
        for (int r = 0; r < REP; ++r) sw[(size_t)r * ld + j] = w[r];
    }
    __syncthreads();
    // values: rows of up to 128 elements take half a warp (a warp walks two keys at once), wider ones the whole warp
    const int* bt = block_table + (size_t)slots[seq_of_token[t]] * cache.max_pages;
    const bool wide = vd > 128;
    const int half = wide ? 0 : lane >> 4, per_step = wide ? 1 : 2;
    const int e_v = 8 * (wide ? lane : (lane & 15));
    float acc[REP][8];
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int x = 0; x < 8; ++x) acc[r][x] = 0.f;
    const int stride = TV_WARPS * per_step;
    for (int j0 = warp * per_step + half; j0 < total + half; j0 += stride * TV_ROWS) {
        uint4 raw[TV_ROWS];
        bool has[TV_ROWS];
#pragma unroll
        for (int b = 0; b < TV_ROWS; ++b) {
            const int j = j0 + b * stride;
            has[b] = false;
            raw[b] = make_uint4(0u, 0u, 0u, 0u);
            if (j < total && e_v < vd) {
                const int key = j < head_end ? j : lo + (j - head_end);
                const int page = bt[key / ps];
                if (page >= 0) {
                    has[b] = true;
                    raw[b] = __ldcg(reinterpret_cast<const uint4*>(cache_values(pool, cache, page, c, key % ps) + e_v));
                }
            }
        }
#pragma unroll
        for (int b = 0; b < TV_ROWS; ++b) {
            if (!has[b]) continue;
            const int j = j0 + b * stride;
            const uint32_t w4[4] = {raw[b].x, raw[b].y, raw[b].z, raw[b].w};
#pragma unroll
            for (int r = 0; r < REP; ++r) {
                const float w = sw[(size_t)r * ld + j];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    acc[r][2 * x] = fmaf(w, __uint_as_float(w4[x] << 16), acc[r][2 * x]);
                    acc[r][2 * x + 1] = fmaf(w, __uint_as_float(w4[x] & 0xffff0000u), acc[r][2 * x + 1]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        if (!wide) {
#pragma unroll
            for (int x = 0; x < 8; ++x) acc[r][x] += __shfl_xor_sync(0xffffffffu, acc[r][x], 16);
        }
        if (half == 0) {
            float* dst = so + ((size_t)warp * REP + r) * vd;
#pragma unroll
            for (int x = 0; x < 8; ++x)
                if (e_v + x < vd) dst[e_v + x] = acc[r][x];
        }
    }
    __syncthreads();
    const bf16* gate = reinterpret_cast<const bf16*>(epi.gate);
    for (int idx = threadIdx.x; idx < rep * vd; idx += TV_THREADS) {
        const int r = idx / vd, e = idx % vd, h = h0 + r;
        float o = 0.f;
        for (int w = 0; w < TV_WARPS; ++w) o += so[((size_t)w * REP + r) * vd + e];
        o *= epi.out_scale;
        if (gate) o *= sigmoidf_(load1_cg(gate + (size_t)t * epi.gate_ld + (gate_heads ? h : h * vd + e)));
        out[((size_t)t * nh + h) * vd + e] = __float2bfloat16_rn(o);
    }
}

static size_t talk_values_smem(int nh, int rep_t, int vd, int n_cap) {
    const size_t ld = ((size_t)n_cap + 3) & ~(size_t)3;
    return ((size_t)nh * ld + (size_t)rep_t * ld + (size_t)TV_WARPS * rep_t * vd) * sizeof(float);
}
static int talk_rep_t(int rep) { return rep <= 1 ? 1 : (rep <= 2 ? 2 : (rep <= 4 ? 4 : 8)); }

// n_cap: the most keys a token of the step sees
ST_EXPORT int st_talk_attention_single_applies(int nh, int nkv, int dim, int vd, int n_cap) {
    if (nh <= 0 || nkv <= 0 || nh % nkv || nh / nkv > TS_MAX_REP || dim <= 0 || vd <= 0 || dim % 8 || vd % 8 || vd > 256)
        return 0;
    return n_cap > 0 && talk_values_smem(nh, talk_rep_t(nh / nkv), vd, n_cap) <= 160 * 1024;
}

ST_EXPORT long long st_talk_attention_single_scratch(int n_tokens, int nh, int n_cap) {
    return (long long)n_tokens * nh * n_cap;
}

template <int REP>
static int launch_talk_values(const float* scores, int n_cap, const void* pool, const DiffCache& c, void* out,
                              const int* items, const int* positions, const int* seq_of_token, const int* slots,
                              const int* block_table, int n_tokens, int nh, const GqaMask& mask, const float* talk,
                              int has_sink, const GqaEpilogue& epi, int gate_heads, cudaStream_t s) {
    const size_t smem = talk_values_smem(nh, REP, c.vd, n_cap);
    auto kern = talk_values_kernel<REP>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return st_launch_pdl("talk_values", kern, dim3(n_tokens, c.nkv), dim3(TV_THREADS), smem, s, scores, n_cap,
                         (const bf16*)pool, c, (bf16*)out, items, positions, seq_of_token, slots, block_table, nh, mask,
                         talk, has_sink, epi, gate_heads);
}

// bfloat16 only; scratch: float, st_talk_attention_single_scratch(n_tokens, nh, n_cap) elements
ST_EXPORT int st_talk_attention_single(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                       void* out, const int* items, const int* positions, const int* seq_of_token,
                                       const int* slots, const int* block_table, int max_pages, int n_tokens, int nh,
                                       int nkv, int dim, int vd, int page_size, float scale, int window, int keep_first,
                                       const float* talk, const float* sinks, const void* gate, long long gate_ld,
                                       int gate_heads, float out_scale, float* scratch, int n_cap, int* status,
                                       void* stream) {
    if (n_tokens <= 0) return 0;
    if (page_size <= 0 || keep_first < 0 || !scratch) return ST_ERR_BAD_ARG;
    if (!st_talk_attention_single_applies(nh, nkv, dim, vd, n_cap)) return ST_ERR_BAD_SIZE;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const GqaMask mask = {window, keep_first};
    const GqaEpilogue epi = {gate, gate_ld, out_scale, sinks};
    cudaStream_t s = (cudaStream_t)stream;
    const int rep = nh / nkv;
    int rc = st_launch_pdl("talk_scores", talk_scores_kernel, dim3(n_tokens, nkv, (n_cap + TS_KEYS - 1) / TS_KEYS),
                           dim3(TS_THREADS), (size_t)rep * dim * sizeof(float), s, (const bf16*)q, (const bf16*)pool, c,
                           scratch, n_cap, items, positions, seq_of_token, slots, block_table, nh, scale, mask, status);
    if (rc) return rc;
#define TV_ARGS scratch, n_cap, pool, c, out, items, positions, seq_of_token, slots, block_table, n_tokens, nh, mask, talk, \
                sinks != nullptr, epi, gate_heads, s
    const int rt = talk_rep_t(rep);
    if (rt == 1) return launch_talk_values<1>(TV_ARGS);
    if (rt == 2) return launch_talk_values<2>(TV_ARGS);
    if (rt == 4) return launch_talk_values<4>(TV_ARGS);
    return launch_talk_values<8>(TV_ARGS);
#undef TV_ARGS
}

// Grouped-query attention whose softmax weights are mixed over the heads before they meet the values
// ("talking heads"), over the flat paged cache of gqa_attention.cuh.
//
//   s_a(j)  = scale * q_a . k_g(a)(j)             over the keys the query sees (GqaMask)
//   P_a(j)  = exp(s_a(j)) / (sum_i exp(s_a(i)) [+ exp(sink_a)])
//   P'_a(j) = sum_b T[a][b] * P_b(j)              T float [heads][heads]; the extra term's share is not mixed
//   o_a     = out_scale * sum_j P'_a(j) v_g(a)(j) [* sigmoid(gate logit of head a, or of (a, e))]
//
// The mixing needs every head's normalised weight of a key, so a query's heads are served together and the keys
// are walked twice: first for every head's maximum and denominator, then again for the weights themselves (the
// scores are computed anew, by the same thread in the same order, so they are the same numbers).
//
// talk_attention_plain: one block per query token, float arithmetic for either storage type, key tiles aligned
// to absolute positions: a row's result does not depend on how the request was cut or on the batch.
#include "gqa_attention.cuh"

#define TK 128            // keys per tile == threads per block
#define T_ACC 64          // outputs (head, value dimension) per thread: heads * vd <= T_ACC * TK

// gate_heads != 0: one gate logit per head at gate[token * gate_ld + head]; else one per (head, e).
template <typename T>
__global__ void __launch_bounds__(TK)
talk_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ pool, DiffCache cache, T* __restrict__ out,
                            const int* __restrict__ items, const int* __restrict__ positions,
                            const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                            const int* __restrict__ block_table, int nh, float scale, GqaMask mask,
                            const float* __restrict__ talk, int has_sink, GqaEpilogue epi, int gate_heads,
                            int* __restrict__ status) {
    extern __shared__ float smem[];
    const int dim = cache.kd, vd = cache.vd, nkv = cache.nkv, ps = cache.page_size;
    float* sq = smem;                    // [nh][dim]
    float* sp = sq + nh * dim;           // [nh][TK]   scores, then weights
    float* sw = sp + nh * TK;            // [nh][TK]   mixed weights
    float* st = sw + nh * TK;            // [nh][nh]   the mixing matrix
    float* sm = st + nh * nh;            // [nh] maxima
    float* sl = sm + nh;                 // [nh] denominators
    for (int i = threadIdx.x; i < nh * nh; i += TK) st[i] = talk ? talk[i] : (i / nh == i % nh ? 1.f : 0.f);
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x;
    if (t < 0) return;
    const int pos = positions[t];
    if (pos < 0) return;
    const int rep = nh / nkv;
    const int* bt = block_table + (size_t)slots[seq_of_token[t]] * cache.max_pages;
    for (int i = threadIdx.x; i < nh * dim; i += TK) sq[i] = load1_cg(q + (size_t)t * nh * dim + i);
    for (int h = threadIdx.x; h < nh; h += TK) { sm[h] = -INFINITY; sl[h] = 0.f; }
    __syncthreads();
    const int lo = gqa_lo(pos, mask), head_end = gqa_head_end(lo, mask), hi = pos + 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // scores of this thread's key of a tile for all heads -> sp[h][thread], -inf where the key is not seen
    auto scores = [&](int base) {
        const int j = base + threadIdx.x;
        const bool seen = j < hi && (j >= lo || j < head_end);
        int page = -1;
        if (seen) {
            page = bt[j / ps];
            if (page < 0 && status) *status = 1;
        }
        for (int g = 0; g < nkv; ++g) {
            const T* krow = page >= 0 ? cache_keys(pool, cache, page, g, j % ps) : nullptr;
            for (int r = 0; r < rep; ++r) {
                const int h = g * rep + r;
                float s = -INFINITY;
                if (krow) {
                    const float* qh = sq + h * dim;
                    float d = 0.f;
                    for (int e = 0; e < dim; ++e) d = fmaf(qh[e], load1_cg(krow + e), d);
                    s = d * scale;
                }
                sp[h * TK + threadIdx.x] = s;
            }
        }
    };

    // ---- first walk: maxima and denominators; warp w owns heads w, w + 4, ...
    for (int base = 0; base < hi; base += TK) {
        if (base >= head_end && base + TK <= lo) continue;
        scores(base);
        __syncthreads();
        for (int h = warp; h < nh; h += TK / 32) {
            float tm = -INFINITY;
            for (int jj = lane; jj < TK; jj += 32) tm = fmaxf(tm, sp[h * TK + jj]);
            tm = warp_max(tm);
            const float m_old = sm[h], m_new = fmaxf(m_old, tm);
            float sum = 0.f;
            if (m_new > -INFINITY)
                for (int jj = lane; jj < TK; jj += 32) {
                    const float s = sp[h * TK + jj];
                    if (s > -INFINITY) sum += expf(s - m_new);
                }
            sum = warp_sum(sum);
            __syncwarp();
            if (lane == 0) {
                sl[h] = (m_old == -INFINITY ? 0.f : sl[h] * expf(m_old - m_new)) + sum;
                sm[h] = m_new;
            }
        }
        __syncthreads();
    }
    if (has_sink) {
        for (int h = threadIdx.x; h < nh; h += TK) {
            const float sk = epi.sinks[h], m_old = sm[h], m_new = fmaxf(m_old, sk);
            sl[h] = (m_old == -INFINITY ? 0.f : sl[h] * expf(m_old - m_new)) + expf(sk - m_new);
            sm[h] = m_new;
        }
    }
    __syncthreads();

    // ---- second walk: weights, mixed over heads, times the values
    float acc[T_ACC];
#pragma unroll
    for (int c = 0; c < T_ACC; ++c) acc[c] = 0.f;
    const int n_out = nh * vd;
    for (int base = 0; base < hi; base += TK) {
        if (base >= head_end && base + TK <= lo) continue;
        scores(base);
        for (int h = 0; h < nh; ++h) {
            const float s = sp[h * TK + threadIdx.x];
            sp[h * TK + threadIdx.x] = (s > -INFINITY && sl[h] > 0.f) ? expf(s - sm[h]) / sl[h] : 0.f;
        }
        for (int h = 0; h < nh; ++h) {
            float w = 0.f;
            for (int b = 0; b < nh; ++b) w = fmaf(st[h * nh + b], sp[b * TK + threadIdx.x], w);
            sw[h * TK + threadIdx.x] = w;
        }
        __syncthreads();
        const int j_end = min(TK, hi - base);
#pragma unroll
        for (int c = 0; c < T_ACC; ++c) {
            const int idx = threadIdx.x + c * TK;
            if (idx >= n_out) continue;
            const int h = idx / vd, e = idx % vd, g = h / rep;
            float x = acc[c];
            for (int jj = 0; jj < j_end; ++jj) {
                const int key = base + jj;
                if (!(key >= lo || key < head_end)) continue;
                const int page = bt[key / ps];
                if (page < 0) continue;
                x = fmaf(sw[h * TK + jj], load1_cg(cache_values(pool, cache, page, g, key % ps) + e), x);
            }
            acc[c] = x;
        }
        __syncthreads();
    }
    const T* gate = reinterpret_cast<const T*>(epi.gate);
#pragma unroll
    for (int c = 0; c < T_ACC; ++c) {
        const int idx = threadIdx.x + c * TK;
        if (idx >= n_out) continue;
        const int h = idx / vd;
        float o = acc[c] * epi.out_scale;
        if (gate) o *= sigmoidf_(load1_cg(gate + (size_t)t * epi.gate_ld + (gate_heads ? h : idx)));
        out[(size_t)t * n_out + idx] = from_f32<T>(o);
    }
}

ST_EXPORT int st_talk_attention_plain(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                      void* out, const int* items, const int* positions, const int* seq_of_token,
                                      const int* slots, const int* block_table, int max_pages, int n_tokens, int nh,
                                      int nkv, int dim, int vd, int page_size, float scale, int window, int keep_first,
                                      const float* talk, const float* sinks, const void* gate, long long gate_ld,
                                      int gate_heads, float out_scale, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || dim <= 0 || vd <= 0 || page_size <= 0 || keep_first < 0) return ST_ERR_BAD_ARG;
    if ((long long)nh * vd > (long long)T_ACC * TK) return ST_ERR_TOO_LARGE;
    const size_t smem = ((size_t)nh * dim + 2 * (size_t)nh * TK + (size_t)nh * nh + 2 * (size_t)nh) * sizeof(float);
    if (smem > 200 * 1024) return ST_ERR_TOO_LARGE;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const GqaMask mask = {window, keep_first};
    const GqaEpilogue epi = {gate, gate_ld, out_scale, sinks};
    cudaStream_t s = (cudaStream_t)stream;
#define TALK_PLAIN(T)                                                                                                 \
    do {                                                                                                              \
        auto kern = talk_attention_plain_kernel<T>;                                                                   \
        if (smem > 48 * 1024) {                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
            if (e != cudaSuccess) return (int)e;                                                                      \
        }                                                                                                             \
        return st_launch_pdl("talk_plain", kern, dim3(n_tokens), dim3(TK), smem, s, (const T*)q, (const T*)pool, c,   \
                             (T*)out, items, positions, seq_of_token, slots, block_table, nh, scale, mask, talk,      \
                             sinks != nullptr, epi, gate_heads, status);                                              \
    } while (0)
    if (dtype == 0) TALK_PLAIN(float);
    if (dtype == 1) TALK_PLAIN(bf16);
#undef TALK_PLAIN
    return ST_ERR_BAD_DTYPE;
}

// Grouped-query attention whose keys and values have sizes of their own, over the flat paged cache: the
// preparation of queries, keys and values from a fused projection, and the plain attention kernel.
//
//   q, k   <- projection + bias; the first rot_dims dimensions of every head rotated by position, dimension i
//             paired with i + rot_dims/2 (float angle p * inv_freq[i], sincosf); q times the temperature
//             1 + coef * ln(floor((p + 1) / every) + 1)  (coef == 0: none)
//   s_j    = scale * q . k_j over the keys the query sees (gqa_attention.cuh: a window of recent keys plus the
//             first keep_first keys of the request, or all keys up to the query)
//   w_j    = exp(s_j) / (sum_i exp(s_i) [+ exp(sink)])
//   out    = out_scale * (sum_j w_j v_j) [* sigmoid(gate)]
//
// The plain kernel computes in float for either storage type with key tiles aligned to absolute positions, so
// a row's result does not depend on how the request was cut into steps or on what else is in the batch.  It is
// the 32-bit path and serves bfloat16 sizes that the tensor-core kernels do not take.
#include "gqa_attention.cuh"

#define GP_THREADS 256

// proj: [n_tokens, ld], queries at column q_off (nh * dim), keys at k_off (nkv * dim), values at v_off (nkv * vd);
// bias: float [ld], indexed like the projection's columns, or null.  write_kv == 0: a layer that reads another
// layer's keys and values prepares its queries only.
template <typename T>
__global__ void __launch_bounds__(GP_THREADS)
gqa_prepare_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ bias,
                   const float* __restrict__ inv_freq, int rot_dims, float temp_coef, int temp_every,
                   T* __restrict__ q_out, T* __restrict__ pool, DiffCache cache, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                   const int* __restrict__ block_table, int nh, int write_kv, int* __restrict__ status) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0) return;
    const int dim = cache.kd, vd = cache.vd, nkv = cache.nkv;
    const int qw = nh * dim, kw = write_kv ? nkv * dim : 0, vw = write_kv ? nkv * vd : 0;
    int page = -1;
    if (write_kv) {
        page = block_table[(size_t)slots[seq_of_token[t]] * cache.max_pages + pos / cache.page_size];
        if (page < 0 && status && threadIdx.x == 0 && blockIdx.y == 0) *status = 1;
    }
    const int pip = pos % cache.page_size;
    const int half = rot_dims / 2;
    const float temp = temp_coef != 0.f ? 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f) : 1.f;
    const T* row = proj + (size_t)t * ld;
    for (int c = blockIdx.y * GP_THREADS + threadIdx.x; c < qw + kw + vw; c += GP_THREADS * gridDim.y) {
        const bool is_q = c < qw, is_k = !is_q && c < qw + kw;
        if (!is_q && page < 0) continue;
        if (!is_q && !is_k) {
            const int cc = c - qw - kw, col = v_off + cc;
            const float x = load1_cg(row + col) + (bias ? bias[col] : 0.f);
            cache_values(pool, cache, page, cc / vd, pip)[cc % vd] = from_f32<T>(x);
            continue;
        }
        const int cc = is_q ? c : c - qw;
        const int head = cc / dim, e = cc % dim;
        const int col = (is_q ? q_off : k_off) + cc;
        float x = load1_cg(row + col) + (bias ? bias[col] : 0.f);
        if (e < rot_dims) {
            const bool low = e < half;
            const int pcol = low ? col + half : col - half;
            const float y = load1_cg(row + pcol) + (bias ? bias[pcol] : 0.f);
            float sn, cs;
            sincosf((float)pos * inv_freq[low ? e : e - half], &sn, &cs);
            x = low ? x * cs - y * sn : x * cs + y * sn;
        }
        if (is_q) q_out[(size_t)t * qw + cc] = from_f32<T>(x * temp);
        else cache_keys(pool, cache, page, head, pip)[e] = from_f32<T>(x);
    }
}

ST_EXPORT int st_gqa_prepare(const void* proj, int ld, int q_off, int k_off, int v_off, const float* bias,
                             const float* inv_freq, int rot_dims, float temp_coef, int temp_every, void* q_out,
                             void* pool, long long page_stride, long long entry_offset, const int* positions,
                             const int* seq_of_token, const int* slots, const int* block_table, int max_pages,
                             int n_tokens, int nh, int nkv, int dim, int vd, int page_size, int write_kv, int* status,
                             int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || dim <= 0 || vd <= 0 || page_size <= 0) return ST_ERR_BAD_ARG;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > dim || (rot_dims > 0 && !inv_freq)) return ST_ERR_BAD_ARG;
    if (temp_coef != 0.f && temp_every <= 0) return ST_ERR_BAD_ARG;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const int total = nh * dim + (write_kv ? nkv * (dim + vd) : 0);
    int gy = (total + GP_THREADS * 4 - 1) / (GP_THREADS * 4);
    if (gy > 64) gy = 64;
    dim3 grid(n_tokens, gy);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0)
        return st_launch_pdl("gqa_prepare", gqa_prepare_kernel<float>, grid, dim3(GP_THREADS), 0, s, (const float*)proj, ld,
                             q_off, k_off, v_off, bias, inv_freq, rot_dims, temp_coef, temp_every, (float*)q_out,
                             (float*)pool, c, positions, seq_of_token, slots, block_table, nh, write_kv, status);
    if (dtype == 1)
        return st_launch_pdl("gqa_prepare", gqa_prepare_kernel<bf16>, grid, dim3(GP_THREADS), 0, s, (const bf16*)proj, ld,
                             q_off, k_off, v_off, bias, inv_freq, rot_dims, temp_coef, temp_every, (bf16*)q_out,
                             (bf16*)pool, c, positions, seq_of_token, slots, block_table, nh, write_kv, status);
    return ST_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------------------
// Plain attention: one block per (query token, head); `items` lists the tokens to serve (n_tokens of them,
// -1: none), or is null for tokens 0..n_tokens-1.
#define GK 128          // keys per tile == threads per block
#define G_VPASS 4       // value dimensions per thread: vd <= G_VPASS * GK

template <typename T>
__global__ void __launch_bounds__(GK)
gqa_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ pool, DiffCache cache, T* __restrict__ out,
                           const int* __restrict__ items, const int* __restrict__ positions,
                           const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                           const int* __restrict__ block_table, int nh, float scale, GqaMask mask, int has_sink,
                           float sink, GqaEpilogue epi, int* __restrict__ status) {
    extern __shared__ float smem[];
    float* sq = smem;            // [dim]
    float* sp = smem + cache.kd; // [GK]
    __shared__ float scratch[32];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    if (t < 0) return;
    const int pos = positions[t];
    if (pos < 0) return;
    const int nkv = cache.nkv, vd = cache.vd, dim = cache.kd, ps = cache.page_size;
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)slots[seq_of_token[t]] * cache.max_pages;
    for (int e = threadIdx.x; e < dim; e += GK) sq[e] = load1_cg(q + ((size_t)t * nh + h) * dim + e);
    __syncthreads();
    const int lo = gqa_lo(pos, mask), head_end = gqa_head_end(lo, mask), hi = pos + 1;
    float acc[G_VPASS];
#pragma unroll
    for (int c = 0; c < G_VPASS; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int base = 0; base < hi; base += GK) {
        if (base >= head_end && base + GK <= lo) continue;      // a tile between the kept keys and the window
        const int j = base + threadIdx.x;
        const bool seen = j < hi && (j >= lo || j < head_end);
        float s = -INFINITY;
        if (seen) {
            const int page = bt[j / ps];
            if (page >= 0) {
                const T* krow = cache_keys(pool, cache, page, kvh, j % ps);
                float d = 0.f;
                for (int e = 0; e < dim; ++e) d = fmaf(sq[e], load1_cg(krow + e), d);
                s = d * scale;
            } else if (status) {
                *status = 1;
            }
        }
        const float n = fmaxf(m, block_max(s, scratch));
        const float p = s > -INFINITY ? expf(s - n) : 0.f;
        const float corr = m == -INFINITY ? 0.f : expf(m - n);
        l = l * corr + block_sum(p, scratch);
        m = n;
        sp[threadIdx.x] = p;
        __syncthreads();
        const int j_end = min(GK, hi - base);
#pragma unroll
        for (int c = 0; c < G_VPASS; ++c) {
            const int e = threadIdx.x + c * GK;
            if (e >= vd) continue;
            float x = acc[c] * corr;
            for (int jj = 0; jj < j_end; ++jj) {
                const float w = sp[jj];
                if (w == 0.f) continue;                          // not seen (uniform over the block)
                const int key = base + jj;
                const int page = bt[key / ps];
                if (page < 0) continue;
                x = fmaf(w, load1_cg(cache_values(pool, cache, page, kvh, key % ps) + e), x);
            }
            acc[c] = x;
        }
        __syncthreads();
    }
    if (has_sink) {
        const float n = fmaxf(m, sink);
        const float corr = m == -INFINITY ? 0.f : expf(m - n);
        l = l * corr + expf(sink - n);
#pragma unroll
        for (int c = 0; c < G_VPASS; ++c) acc[c] *= corr;
    }
    const float inv = l > 0.f ? epi.out_scale / l : 0.f;
    const T* gate = reinterpret_cast<const T*>(epi.gate);
#pragma unroll
    for (int c = 0; c < G_VPASS; ++c) {
        const int e = threadIdx.x + c * GK;
        if (e >= vd) continue;
        float o = acc[c] * inv;
        if (gate) o *= sigmoidf_(load1_cg(gate + (size_t)t * epi.gate_ld + h * vd + e));
        out[((size_t)t * nh + h) * vd + e] = from_f32<T>(o);
    }
}

ST_EXPORT int st_gqa_attention_plain(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                     void* out, const int* items, const int* positions, const int* seq_of_token,
                                     const int* slots, const int* block_table, int max_pages, int n_tokens, int nh,
                                     int nkv, int dim, int vd, int page_size, float scale, int window, int keep_first,
                                     int has_sink, float sink, const void* gate, long long gate_ld, float out_scale,
                                     int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || dim <= 0 || vd <= 0 || page_size <= 0 || keep_first < 0) return ST_ERR_BAD_ARG;
    if (vd > G_VPASS * GK || dim > 4096) return ST_ERR_TOO_LARGE;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const GqaMask mask = {window, keep_first};
    const GqaEpilogue epi = {gate, gate_ld, out_scale};
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, nh);
    const size_t smem = (size_t)(dim + GK) * sizeof(float);
    if (dtype == 0)
        return st_launch_pdl("gqa_plain", gqa_attention_plain_kernel<float>, grid, dim3(GK), smem, s, (const float*)q,
                             (const float*)pool, c, (float*)out, items, positions, seq_of_token, slots, block_table, nh,
                             scale, mask, has_sink, sink, epi, status);
    if (dtype == 1)
        return st_launch_pdl("gqa_plain", gqa_attention_plain_kernel<bf16>, grid, dim3(GK), smem, s, (const bf16*)q,
                             (const bf16*)pool, c, (bf16*)out, items, positions, seq_of_token, slots, block_table, nh,
                             scale, mask, has_sink, sink, epi, status);
    return ST_ERR_BAD_DTYPE;
}

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

// ------------------------------------------------------------------------------------------------
// Single tokens and short portions in bfloat16: one block per (token, key/value head) serves all REP query heads
// of the group, so a key or value row is fetched once for them.  The seen keys (the kept first ones, then the
// window up to the query) are numbered in one run; warp w takes keys w*GS_BATCH .. of every GS_WARPS*GS_BATCH,
// its lanes side by side along the row (four neighbouring elements each: dim <= 128, vd <= 128 * GS_VPASS).
// The rows of a batch of keys and values are asked for before the first is used.  Every warp runs its own
// softmax (maximum, sum and weighted value sum per head, the same in all its lanes); the warps' parts meet in
// shared memory in warp order, where the extra term joins, and a thread per (head, value dimension) scales,
// gates and stores.  What a warp adds up depends on the key's number only, so a token's result is the same
// whatever else the step holds.
#define GS_THREADS 256
#define GS_WARPS (GS_THREADS / 32)
#define GS_BATCH 4
#define GS_VPASS 2

template <int REP>
__global__ void __launch_bounds__(GS_THREADS)
gqa_attention_single_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, DiffCache cache,
                            bf16* __restrict__ out, const int* __restrict__ items, const int* __restrict__ positions,
                            const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                            const int* __restrict__ block_table, int nh, float scale, GqaMask mask, int has_sink,
                            float sink, GqaEpilogue epi, int* __restrict__ status) {
    extern __shared__ __align__(16) float gs_smem[];      // [GS_WARPS][REP][vd + 2]: weighted sums, maximum, sum
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x, kvh = blockIdx.y;
    if (t < 0) return;
    const int pos = positions[t];
    if (pos < 0) return;
    const int nkv = cache.nkv, vd = cache.vd, dim = cache.kd, ps = cache.page_size;
    const int rep = nh / nkv, h0 = kvh * rep;
    const int* bt = block_table + (size_t)slots[seq_of_token[t]] * cache.max_pages;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lo = gqa_lo(pos, mask), head_end = gqa_head_end(lo, mask);
    const int total = head_end + pos + 1 - lo;
    const int e_k = 4 * lane;
    float qr[REP][4];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rep && e_k < dim) v = load4_cg(q + ((size_t)t * nh + h0 + r) * dim + e_k);
        qr[r][0] = v.x * scale; qr[r][1] = v.y * scale; qr[r][2] = v.z * scale; qr[r][3] = v.w * scale;
    }
    float acc[REP][GS_VPASS][4], m[REP], l[REP];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int p = 0; p < GS_VPASS; ++p)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[r][p][x] = 0.f;
    }
    for (int i0 = warp * GS_BATCH; i0 < total; i0 += GS_WARPS * GS_BATCH) {
        float4 kk[GS_BATCH], vv[GS_BATCH][GS_VPASS];
        bool seen[GS_BATCH];
#pragma unroll
        for (int u = 0; u < GS_BATCH; ++u) {
            const int i = i0 + u;
            const int key = i < head_end ? i : lo + (i - head_end);
            int page = -1;
            if (i < total) {
                page = bt[key / ps];
                if (page < 0 && status) *status = 1;
            }
            seen[u] = page >= 0;
            kk[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int p = 0; p < GS_VPASS; ++p) vv[u][p] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (page >= 0) {
                if (e_k < dim) kk[u] = load4_cg(cache_keys(pool, cache, page, kvh, key % ps) + e_k);
                const bf16* vrow = cache_values(pool, cache, page, kvh, key % ps);
#pragma unroll
                for (int p = 0; p < GS_VPASS; ++p)
                    if (p * 128 + e_k < vd) vv[u][p] = load4_cg(vrow + p * 128 + e_k);
            }
        }
#pragma unroll
        for (int u = 0; u < GS_BATCH; ++u) {
            if (!seen[u]) continue;                        // (the same in all lanes of the warp)
#pragma unroll
            for (int r = 0; r < REP; ++r) {
                if (r >= rep) continue;
                float s = fmaf(qr[r][0], kk[u].x, fmaf(qr[r][1], kk[u].y, fmaf(qr[r][2], kk[u].z, qr[r][3] * kk[u].w)));
                s = warp_sum(s);
                const float n = fmaxf(m[r], s);
                const float c = m[r] == -INFINITY ? 0.f : expf(m[r] - n);
                const float w = expf(s - n);
                l[r] = fmaf(l[r], c, w);
                m[r] = n;
#pragma unroll
                for (int p = 0; p < GS_VPASS; ++p) {
                    acc[r][p][0] = fmaf(w, vv[u][p].x, acc[r][p][0] * c);
                    acc[r][p][1] = fmaf(w, vv[u][p].y, acc[r][p][1] * c);
                    acc[r][p][2] = fmaf(w, vv[u][p].z, acc[r][p][2] * c);
                    acc[r][p][3] = fmaf(w, vv[u][p].w, acc[r][p][3] * c);
                }
            }
        }
    }
    const int ld = vd + 2;
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        if (r >= rep) continue;
        float* dst = gs_smem + ((size_t)warp * REP + r) * ld;
#pragma unroll
        for (int p = 0; p < GS_VPASS; ++p)
#pragma unroll
            for (int x = 0; x < 4; ++x)
                if (p * 128 + e_k + x < vd) dst[p * 128 + e_k + x] = acc[r][p][x];
        if (lane == 0) { dst[vd] = m[r]; dst[vd + 1] = l[r]; }
    }
    __syncthreads();
    const bf16* gate = reinterpret_cast<const bf16*>(epi.gate);
    for (int idx = threadIdx.x; idx < rep * vd; idx += GS_THREADS) {
        const int r = idx / vd, e = idx % vd;
        float M = has_sink ? sink : -INFINITY;
        for (int w = 0; w < GS_WARPS; ++w) M = fmaxf(M, gs_smem[((size_t)w * REP + r) * ld + vd]);
        float L = has_sink ? expf(sink - M) : 0.f, O = 0.f;
        for (int w = 0; w < GS_WARPS; ++w) {
            const float* src = gs_smem + ((size_t)w * REP + r) * ld;
            const float mw = src[vd];
            if (mw == -INFINITY) continue;
            const float c = expf(mw - M);
            L = fmaf(src[vd + 1], c, L);
            O = fmaf(src[e], c, O);
        }
        float o = L > 0.f ? O * epi.out_scale / L : 0.f;
        const int h = h0 + r;
        if (gate) o *= sigmoidf_(load1_cg(gate + (size_t)t * epi.gate_ld + h * vd + e));
        out[((size_t)t * nh + h) * vd + e] = __float2bfloat16_rn(o);
    }
}

ST_EXPORT int st_gqa_attention_single_applies(int nh, int nkv, int dim, int vd) {
    return nh > 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= 8 && dim > 0 && vd > 0 && dim % 4 == 0 && vd % 4 == 0 &&
           dim <= 128 && vd <= 128 * GS_VPASS;
}

template <int REP>
static int launch_gqa_single(const void* q, const void* pool, const DiffCache& c, void* out, const int* items,
                             const int* positions, const int* seq_of_token, const int* slots, const int* block_table,
                             int n_tokens, int nh, float scale, const GqaMask& mask, int has_sink, float sink,
                             const GqaEpilogue& epi, int* status, cudaStream_t s) {
    const size_t smem = (size_t)GS_WARPS * REP * (c.vd + 2) * sizeof(float);
    auto kern = gqa_attention_single_kernel<REP>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return st_launch_pdl("gqa_single", kern, dim3(n_tokens, c.nkv), dim3(GS_THREADS), smem, s, (const bf16*)q,
                         (const bf16*)pool, c, (bf16*)out, items, positions, seq_of_token, slots, block_table, nh, scale,
                         mask, has_sink, sink, epi, status);
}

// bfloat16 only; `items` as for the plain kernel
ST_EXPORT int st_gqa_attention_single(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                      void* out, const int* items, const int* positions, const int* seq_of_token,
                                      const int* slots, const int* block_table, int max_pages, int n_tokens, int nh,
                                      int nkv, int dim, int vd, int page_size, float scale, int window, int keep_first,
                                      int has_sink, float sink, const void* gate, long long gate_ld, float out_scale,
                                      int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (page_size <= 0 || keep_first < 0) return ST_ERR_BAD_ARG;
    if (!st_gqa_attention_single_applies(nh, nkv, dim, vd)) return ST_ERR_BAD_SIZE;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const GqaMask mask = {window, keep_first};
    const GqaEpilogue epi = {gate, gate_ld, out_scale};
    cudaStream_t s = (cudaStream_t)stream;
    const int rep = nh / nkv;
#define GS_ARGS q, pool, c, out, items, positions, seq_of_token, slots, block_table, n_tokens, nh, scale, mask, has_sink, sink, \
                epi, status, s
    if (rep == 1) return launch_gqa_single<1>(GS_ARGS);
    if (rep == 2) return launch_gqa_single<2>(GS_ARGS);
    if (rep <= 4) return launch_gqa_single<4>(GS_ARGS);
    return launch_gqa_single<8>(GS_ARGS);
#undef GS_ARGS
}

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

// The same with every query and key head divided by its root mean square over dim after the rotation
// (x / sqrt(mean(x^2) + norm_eps), no weight): a warp per head, a lane holding dimensions lane, lane + 32, ...
#define GP_NORM_PASSES 8      // heads of up to 32 * GP_NORM_PASSES dimensions
template <typename T>
__global__ void __launch_bounds__(GP_THREADS)
gqa_prepare_norm_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                        const float* __restrict__ bias, const float* __restrict__ inv_freq, int rot_dims,
                        float temp_coef, int temp_every, float norm_eps, T* __restrict__ q_out, T* __restrict__ pool,
                        DiffCache cache, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                        const int* __restrict__ slots, const int* __restrict__ block_table, int nh, int write_kv,
                        int* __restrict__ status) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0) return;
    const int dim = cache.kd, vd = cache.vd, nkv = cache.nkv;
    int page = -1;
    if (write_kv) {
        page = block_table[(size_t)slots[seq_of_token[t]] * cache.max_pages + pos / cache.page_size];
        if (page < 0 && status && threadIdx.x == 0 && blockIdx.y == 0) *status = 1;
    }
    const int pip = pos % cache.page_size;
    const int half = rot_dims / 2;
    const float temp = temp_coef != 0.f ? 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f) : 1.f;
    const T* row = proj + (size_t)t * ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = GP_THREADS / 32;
    const int units = nh + (write_kv ? 2 * nkv : 0);            // query heads, key heads, value heads
    for (int u = blockIdx.y * nwarp + warp; u < units; u += nwarp * gridDim.y) {
        if (u >= nh && page < 0) continue;
        if (u >= nh + nkv) {
            const int head = u - nh - nkv;
            for (int e = lane; e < vd; e += 32) {
                const int col = v_off + head * vd + e;
                cache_values(pool, cache, page, head, pip)[e] = from_f32<T>(load1_cg(row + col) + (bias ? bias[col] : 0.f));
            }
            continue;
        }
        const bool is_q = u < nh;
        const int head = is_q ? u : u - nh;
        const int col0 = (is_q ? q_off : k_off) + head * dim;
        float x[GP_NORM_PASSES];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < GP_NORM_PASSES; ++r) {
            const int e = lane + 32 * r;
            x[r] = 0.f;
            if (e >= dim) continue;
            const int col = col0 + e;
            float v = load1_cg(row + col) + (bias ? bias[col] : 0.f);
            if (e < rot_dims) {
                const bool low = e < half;
                const int pcol = low ? col + half : col - half;
                const float y = load1_cg(row + pcol) + (bias ? bias[pcol] : 0.f);
                float sn, cs;
                sincosf((float)pos * inv_freq[low ? e : e - half], &sn, &cs);
                v = low ? v * cs - y * sn : v * cs + y * sn;
            }
            x[r] = v;
            ss = fmaf(v, v, ss);
        }
        const float mult = rsqrtf(warp_sum(ss) / (float)dim + norm_eps) * (is_q ? temp : 1.f);
#pragma unroll
        for (int r = 0; r < GP_NORM_PASSES; ++r) {
            const int e = lane + 32 * r;
            if (e >= dim) continue;
            if (is_q) q_out[((size_t)t * nh + head) * dim + e] = from_f32<T>(x[r] * mult);
            else cache_keys(pool, cache, page, head, pip)[e] = from_f32<T>(x[r] * mult);
        }
    }
}

ST_EXPORT int st_gqa_prepare(const void* proj, int ld, int q_off, int k_off, int v_off, const float* bias,
                             const float* inv_freq, int rot_dims, float temp_coef, int temp_every, void* q_out,
                             void* pool, long long page_stride, long long entry_offset, const int* positions,
                             const int* seq_of_token, const int* slots, const int* block_table, int max_pages,
                             int n_tokens, int nh, int nkv, int dim, int vd, int page_size, int write_kv, int* status,
                             int dtype, void* stream, float norm_eps) {
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
    if (norm_eps > 0.f) {
        if (dim > 32 * GP_NORM_PASSES) return ST_ERR_TOO_LARGE;
        const int units = nh + (write_kv ? 2 * nkv : 0), per = GP_THREADS / 32;
        int ny = (units + per - 1) / per;
        if (ny > 64) ny = 64;
        dim3 ngrid(n_tokens, ny);
        if (dtype == 0)
            return st_launch_pdl("gqa_prepare", gqa_prepare_norm_kernel<float>, ngrid, dim3(GP_THREADS), 0, s,
                                 (const float*)proj, ld, q_off, k_off, v_off, bias, inv_freq, rot_dims, temp_coef,
                                 temp_every, norm_eps, (float*)q_out, (float*)pool, c, positions, seq_of_token, slots,
                                 block_table, nh, write_kv, status);
        if (dtype == 1)
            return st_launch_pdl("gqa_prepare", gqa_prepare_norm_kernel<bf16>, ngrid, dim3(GP_THREADS), 0, s,
                                 (const bf16*)proj, ld, q_off, k_off, v_off, bias, inv_freq, rot_dims, temp_coef,
                                 temp_every, norm_eps, (bf16*)q_out, (bf16*)pool, c, positions, seq_of_token, slots,
                                 block_table, nh, write_kv, status);
        return ST_ERR_BAD_DTYPE;
    }
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
        if (epi.sinks) sink = epi.sinks[h];
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
                                     int* status, int dtype, void* stream, const float* sinks) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || dim <= 0 || vd <= 0 || page_size <= 0 || keep_first < 0) return ST_ERR_BAD_ARG;
    if (vd > G_VPASS * GK || dim > 4096) return ST_ERR_TOO_LARGE;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const GqaMask mask = {window, keep_first};
    const GqaEpilogue epi = {gate, gate_ld, out_scale, has_sink ? sinks : nullptr};
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
// window up to the query) are numbered in one run and taken GS_TILE at a time, in two phases:
//   scores   a thread per key: it looks the key's page up, asks for the whole key row in 16-byte pieces at once
//            (GS_TILE rows are on their way together) and takes the dot products with the group's queries, which
//            stand in shared memory as scaled floats; the tile's maximum per head is found over the block, and the
//            weights exp(s - m) go to shared memory with the address of the key's value row;
//   values   the warps share the tile's keys, their lanes side by side along the value row (a 16-byte piece of eight
//            elements each: vd <= 256; rows of up to 128 elements take half a warp, so a warp walks two keys at
//            once), many rows in flight.
// The running maximum is the block's, so the warps' sums only have to be added at the end, where the extra term
// joins and a thread per (head, value dimension) scales, gates and stores.  What is added in which order depends
// on the key's number and on the block's shape (which the launcher picks by the step's size), so a token's result
// does not depend on the other tokens of the step beyond the rounding of sums taken in another order.
// Threads of a block (= keys of a tile) and value rows a warp asks for at once, by the query heads a block serves:
// with one or two heads the registers allow sixteen warps, four per scheduler, which hide one another's waits.
template <int REP> struct GsShape {
    static constexpr int THREADS = REP <= 2 ? 512 : 256;
    static constexpr int VB = REP == 1 ? 16 : (REP <= 4 ? 8 : 4);
};
#define GS_KPIECES 8      // 16-byte pieces of a key row asked for at once (64 dimensions)

// every 128-byte line of a row of n bfloat16 elements
__device__ __forceinline__ void gs_prefetch_row(const bf16* row, int n) {
    const char* p = reinterpret_cast<const char*>(row);
    const char* last = p + 2 * n - 1;
    for (const char* a = p; a < last; a += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(last));
}

template <int REP>
__global__ void __launch_bounds__(GsShape<REP>::THREADS)
gqa_attention_single_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, DiffCache cache,
                            bf16* __restrict__ out, const int* __restrict__ items, const int* __restrict__ positions,
                            const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                            const int* __restrict__ block_table, int nh, int hb, float scale, GqaMask mask,
                            int has_sink, float sink, GqaEpilogue epi, int* __restrict__ status) {
    constexpr int GS_THREADS = GsShape<REP>::THREADS, GS_WARPS = GS_THREADS / 32, GS_TILE = GS_THREADS;
    extern __shared__ __align__(16) unsigned char gs_raw[];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x;
    if (t < 0) return;
    const int pos = positions[t];
    if (pos < 0) return;
    const int nkv = cache.nkv, vd = cache.vd, dim = cache.kd, ps = cache.page_size;
    // the block's query heads: hb neighbours of one group (hb divides the group's size, hb <= REP)
    const int rep = hb, h0 = blockIdx.y * hb, kvh = h0 / (nh / nkv);
    long long* srow = reinterpret_cast<long long*>(gs_raw);             // [GS_TILE] value rows (element offsets), -1: none
    float* sq = reinterpret_cast<float*>(srow + GS_TILE);               // [REP][dim] queries times scale
    float* sp = sq + REP * dim;                                         // [REP][GS_TILE] weights
    float* sred = sp + REP * GS_TILE;                                   // [REP][GS_WARPS]
    float* sl = sred + REP * GS_WARPS;                                  // [GS_WARPS][REP] sums of weights
    float* so = sl + GS_WARPS * REP;                                    // [GS_WARPS][REP][vd] weighted value sums
    const int* bt = block_table + (size_t)slots[seq_of_token[t]] * cache.max_pages;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lo = gqa_lo(pos, mask), head_end = gqa_head_end(lo, mask);
    const int total = head_end + pos + 1 - lo;
    for (int i = threadIdx.x; i < REP * dim; i += GS_THREADS) {
        const int r = i / dim;
        sq[i] = r < rep ? load1_cg(q + ((size_t)t * nh + h0) * dim + i) * scale : 0.f;
    }
    // value rows: a lane owns eight neighbouring dimensions (one 16-byte piece).  Rows of up to 128 dimensions take
    // half a warp, and the two halves walk different keys; wider rows (up to 256) take the whole warp.
    const bool wide = vd > 128;
    const int half = wide ? 0 : lane >> 4, keys_per_step = wide ? 1 : 2;
    const int e_v = 8 * (wide ? lane : (lane & 15));
    float acc[REP][8], m[REP], l[REP];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int x = 0; x < 8; ++x) acc[r][x] = 0.f;
    }
    __syncthreads();
    const int pieces = dim / 8;
    for (int i0 = 0; i0 < total; i0 += GS_TILE) {
        // ---- scores: this thread's key
        const int i = i0 + threadIdx.x;
        const int key = i < head_end ? i : lo + (i - head_end);
        int page = -1;
        if (i < total) {
            page = bt[key / ps];
            if (page < 0 && status) *status = 1;
        }
        float s[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) s[r] = 0.f;
        // Asked into the second-level cache now, so that they are near when their turn comes: this key's value row
        // (read in the second phase) and the key row this thread takes in the next tile.
        if (page >= 0) gs_prefetch_row(cache_values(pool, cache, page, kvh, key % ps), vd);
        if (i + GS_TILE < total) {
            const int i_n = i + GS_TILE;
            const int key_n = i_n < head_end ? i_n : lo + (i_n - head_end);
            const int page_n = bt[key_n / ps];
            if (page_n >= 0) gs_prefetch_row(cache_keys(pool, cache, page_n, kvh, key_n % ps), dim);
        }
        if (page >= 0) {
            const uint4* kp = reinterpret_cast<const uint4*>(cache_keys(pool, cache, page, kvh, key % ps));
            for (int c0 = 0; c0 < pieces; c0 += GS_KPIECES) {
                uint4 kk[GS_KPIECES];
#pragma unroll
                for (int c = 0; c < GS_KPIECES; ++c)
                    kk[c] = c0 + c < pieces ? __ldcg(kp + c0 + c) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int c = 0; c < GS_KPIECES; ++c) {
                    if (c0 + c >= pieces) continue;
                    const uint32_t w4[4] = {kk[c].x, kk[c].y, kk[c].z, kk[c].w};
                    float kf[8];
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        kf[2 * x] = __uint_as_float(w4[x] << 16);
                        kf[2 * x + 1] = __uint_as_float(w4[x] & 0xffff0000u);
                    }
#pragma unroll
                    for (int r = 0; r < REP; ++r) {
                        const float4 qa = *reinterpret_cast<const float4*>(sq + r * dim + (c0 + c) * 8);
                        const float4 qb = *reinterpret_cast<const float4*>(sq + r * dim + (c0 + c) * 8 + 4);
                        float d = s[r];
                        d = fmaf(qa.x, kf[0], d); d = fmaf(qa.y, kf[1], d); d = fmaf(qa.z, kf[2], d); d = fmaf(qa.w, kf[3], d);
                        d = fmaf(qb.x, kf[4], d); d = fmaf(qb.y, kf[5], d); d = fmaf(qb.z, kf[6], d); d = fmaf(qb.w, kf[7], d);
                        s[r] = d;
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            const float wm = warp_max(page >= 0 ? s[r] : -INFINITY);
            if (lane == 0) sred[r * GS_WARPS + warp] = wm;
        }
        __syncthreads();
        float corr[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            float tm = sred[r * GS_WARPS];
#pragma unroll
            for (int w = 1; w < GS_WARPS; ++w) tm = fmaxf(tm, sred[r * GS_WARPS + w]);
            const float n = fmaxf(m[r], tm);
            corr[r] = m[r] == -INFINITY ? 0.f : expf(m[r] - n);
            m[r] = n;
            sp[r * GS_TILE + threadIdx.x] = page >= 0 ? expf(s[r] - n) : 0.f;
        }
        srow[threadIdx.x] = page >= 0 ? (long long)(cache_values(pool, cache, page, kvh, key % ps) - pool) : -1;
        __syncthreads();
        // ---- values: this warp's keys of the tile
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            l[r] *= corr[r];
#pragma unroll
            for (int x = 0; x < 8; ++x) acc[r][x] *= corr[r];
        }
        const int tile_n = min(GS_TILE, total - i0);
        // a warp's keys go VB steps at a time: all their value rows are asked for before the first is used, so that
        // a block keeps tens of kilobytes on their way (the rows, not the arithmetic, set the pace)
        constexpr int VB = GsShape<REP>::VB;
        const int stride = GS_WARPS * keys_per_step;
        for (int j0 = warp * keys_per_step + half; j0 < tile_n + half; j0 += stride * VB) {
            uint4 raw[VB];
            bool has[VB];
#pragma unroll
            for (int b = 0; b < VB; ++b) {
                const int j = j0 + b * stride;
                const long long off = j < tile_n ? srow[j] : -1;
                has[b] = off >= 0;
                raw[b] = (has[b] && e_v < vd) ? __ldcg(reinterpret_cast<const uint4*>(pool + off + e_v))
                                              : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int b = 0; b < VB; ++b) {
                if (!has[b]) continue;
                const int j = j0 + b * stride;
                const uint32_t w4[4] = {raw[b].x, raw[b].y, raw[b].z, raw[b].w};
#pragma unroll
                for (int r = 0; r < REP; ++r) {
                    const float w = sp[r * GS_TILE + j];
                    l[r] += w;
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        acc[r][2 * x] = fmaf(w, __uint_as_float(w4[x] << 16), acc[r][2 * x]);
                        acc[r][2 * x + 1] = fmaf(w, __uint_as_float(w4[x] & 0xffff0000u), acc[r][2 * x + 1]);
                    }
                }
            }
        }
        // (the next tile's first barrier stands between these reads of sp and srow and their next writes)
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        if (!wide) {                                   // the two halves of the warp walked different keys
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 16);
#pragma unroll
            for (int x = 0; x < 8; ++x) acc[r][x] += __shfl_xor_sync(0xffffffffu, acc[r][x], 16);
        }
        float* dst = so + ((size_t)warp * REP + r) * vd;
        if (half == 0) {
#pragma unroll
            for (int x = 0; x < 8; ++x)
                if (e_v + x < vd) dst[e_v + x] = acc[r][x];
        }
        if (lane == 0) sl[warp * REP + r] = l[r];
    }
    __syncthreads();
    const bf16* gate = reinterpret_cast<const bf16*>(epi.gate);
    for (int idx = threadIdx.x; idx < rep * vd; idx += GS_THREADS) {
        const int r = idx / vd, e = idx % vd;
        // m[] is indexed by a runtime head here: every thread holds the same maxima, pick by comparison
        float mr = -INFINITY;
#pragma unroll
        for (int rr = 0; rr < REP; ++rr)
            if (rr == r) mr = m[rr];
        float L = 0.f, O = 0.f;
        for (int w = 0; w < GS_WARPS; ++w) {
            L += sl[w * REP + r];
            O += so[((size_t)w * REP + r) * vd + e];
        }
        const int h = h0 + r;
        if (has_sink) {
            const float sk = epi.sinks ? epi.sinks[h] : sink;
            const float n = fmaxf(mr, sk);
            const float c = mr == -INFINITY ? 0.f : expf(mr - n);
            L = fmaf(L, c, expf(sk - n));
            O *= c;
        }
        float o = L > 0.f ? O * epi.out_scale / L : 0.f;
        if (gate) o *= sigmoidf_(load1_cg(gate + (size_t)t * epi.gate_ld + h * vd + e));
        out[((size_t)t * nh + h) * vd + e] = __float2bfloat16_rn(o);
    }
}

static size_t gqa_single_smem(int rep_t, int threads, int dim, int vd) {
    const size_t tile = threads, warps = threads / 32;
    return tile * sizeof(long long) +
           ((size_t)rep_t * dim + (size_t)rep_t * tile + 2 * (size_t)rep_t * warps + warps * rep_t * vd) * sizeof(float);
}

ST_EXPORT int st_gqa_attention_single_applies(int nh, int nkv, int dim, int vd) {
    return nh > 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= 8 && dim > 0 && vd > 0 && dim % 8 == 0 && vd % 8 == 0 &&
           dim <= 128 && vd <= 256;
}

template <int REP>
static int launch_gqa_single(const void* q, const void* pool, const DiffCache& c, void* out, const int* items,
                             const int* positions, const int* seq_of_token, const int* slots, const int* block_table,
                             int n_tokens, int nh, int hb, float scale, const GqaMask& mask, int has_sink, float sink,
                             const GqaEpilogue& epi, int* status, cudaStream_t s) {
    const size_t smem = gqa_single_smem(REP, GsShape<REP>::THREADS, c.kd, c.vd);
    auto kern = gqa_attention_single_kernel<REP>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return st_launch_pdl("gqa_single", kern, dim3(n_tokens, nh / hb), dim3(GsShape<REP>::THREADS), smem, s, (const bf16*)q,
                         (const bf16*)pool, c, (bf16*)out, items, positions, seq_of_token, slots, block_table, nh, hb,
                         scale, mask, has_sink, sink, epi, status);
}

// bfloat16 only; `items` as for the plain kernel
ST_EXPORT int st_gqa_attention_single(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                      void* out, const int* items, const int* positions, const int* seq_of_token,
                                      const int* slots, const int* block_table, int max_pages, int n_tokens, int nh,
                                      int nkv, int dim, int vd, int page_size, float scale, int window, int keep_first,
                                      int has_sink, float sink, const void* gate, long long gate_ld, float out_scale,
                                      int* status, void* stream, const float* sinks) {
    if (n_tokens <= 0) return 0;
    if (page_size <= 0 || keep_first < 0) return ST_ERR_BAD_ARG;
    if (!st_gqa_attention_single_applies(nh, nkv, dim, vd)) return ST_ERR_BAD_SIZE;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const GqaMask mask = {window, keep_first};
    const GqaEpilogue epi = {gate, gate_ld, out_scale, has_sink ? sinks : nullptr};
    cudaStream_t s = (cudaStream_t)stream;
    // Query heads per block: the whole group when that gives blocks for three quarters of the device (a key or value
    // row is then fetched once for the group), else the largest part of the group that does, down to one head; the
    // other blocks of a group find the rows in the second-level cache.  A head's result differs between the cases only
    // in how its keys are dealt to warps, that is in the order of additions.
    const int rep = nh / nkv;
    int hb = 1;
    for (int d = rep; d >= 1; --d)
        if (rep % d == 0 && 4LL * n_tokens * (nh / d) >= 3LL * st_sm_count()) { hb = d; break; }
#define GS_ARGS q, pool, c, out, items, positions, seq_of_token, slots, block_table, n_tokens, nh, hb, scale, mask, has_sink, \
                sink, epi, status, s
    if (hb == 1) return launch_gqa_single<1>(GS_ARGS);
    if (hb == 2) return launch_gqa_single<2>(GS_ARGS);
    if (hb <= 4) return launch_gqa_single<4>(GS_ARGS);
    return launch_gqa_single<8>(GS_ARGS);
#undef GS_ARGS
}

// Routing of a mixture of experts: which experts a token uses, the tokens sorted by expert, and the weighted
// sum of the experts' results.
//
// moe_route:   z = W_r h (float, W_r float [experts, width]); s = softmax(z) over all experts; the `top` experts
//              with the largest s (ties: the lower index) and their s as weights (not renormalised, unless asked: then divided by their sum + 1e-20);
//              optionally g = sigmoid(w_g . h), one number per token (the gate of a shared expert).
//              A padding token (position < 0) gets expert -1.
// moe_sort:    the step's (token, choice) items grouped by expert: offsets[e]..offsets[e+1] are expert e's places
//              in `sorted` (item indices), `place[item]` the inverse, and a list of row tiles (expert, first place)
//              for the grouped products, padded with expert -1.  One block; items of one expert stand in no
//              particular order, which changes no result: every row of a product is computed on its own.
// moe_combine: out[t] = sum_k weight[t,k] * y[place[t,k]]  (+ g[t] * shared[t]), in float.
#include "common.cuh"

#define ROUTE_THREADS 256
#define ROUTE_MAX_EXPERTS 1024

template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const T* __restrict__ h, int width, const float* __restrict__ w_r, int n_experts, int top,
                 int renorm, const float* __restrict__ w_g, const int* __restrict__ positions,
                 int* __restrict__ experts, float* __restrict__ weights, float* __restrict__ gate, int vec) {
    __shared__ float z[ROUTE_MAX_EXPERTS + 1];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = ROUTE_THREADS / 32;
    if (positions && positions[t] < 0) {
        for (int k = threadIdx.x; k < top; k += ROUTE_THREADS) { experts[(size_t)t * top + k] = -1; weights[(size_t)t * top + k] = 0.f; }
        if (gate && threadIdx.x == 0) gate[t] = 0.f;
        return;
    }
    const T* row = h + (size_t)t * width;
    const int n_rows = n_experts + (w_g ? 1 : 0);
    for (int e = warp; e < n_rows; e += nwarp) {
        const float* wr = e < n_experts ? w_r + (size_t)e * width : w_g;
        float d = 0.f;
        if (vec) {
            // four at a time; a lane's partial sums run in the same order whatever the batch
            for (int i = lane * 4; i < width; i += 128) {
                const float4 a = load4_cg(row + i), c = *reinterpret_cast<const float4*>(wr + i);
                d = fmaf(a.x, c.x, fmaf(a.y, c.y, fmaf(a.z, c.z, fmaf(a.w, c.w, d))));
            }
        } else {
            for (int i = lane; i < width; i += 32) d = fmaf(load1_cg(row + i), wr[i], d);
        }
        d = warp_sum(d);
        if (lane == 0) z[e] = d;
    }
    __syncthreads();
    if (warp != 0) return;
    if (w_g && lane == 0) gate[t] = 1.f / (1.f + expf(-z[n_experts]));
    float m = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) {
        const float p = expf(z[e] - m);
        z[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    const float inv = 1.f / sum;
    float chosen_sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -1.f;
        int arg = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32)
            if (z[e] > best) { best = z[e]; arg = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        chosen_sum += best * inv;
        if (lane == 0) {
            experts[(size_t)t * top + k] = arg;
            weights[(size_t)t * top + k] = best * inv;
            z[arg] = -2.f;
        }
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] /= chosen_sum + 1e-20f;
}

ST_EXPORT int st_moe_route(const void* h, int n_tokens, int width, const float* w_r, int n_experts, int top, int renorm,
                           const float* w_g, const int* positions, int* experts, float* weights, float* gate, int dtype,
                           void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_experts <= 0 || top <= 0 || top > n_experts) return ST_ERR_BAD_ARG;
    if (n_experts > ROUTE_MAX_EXPERTS) return ST_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = width % 4 == 0 && aligned16(h) && aligned16(w_r) && (!w_g || aligned16(w_g));
    if (dtype == 0)
        return st_launch_pdl("moe_route", moe_route_kernel<float>, dim3(n_tokens), dim3(ROUTE_THREADS), 0, s, (const float*)h,
                             width, w_r, n_experts, top, renorm, w_g, positions, experts, weights, gate, vec);
    if (dtype == 1)
        return st_launch_pdl("moe_route", moe_route_kernel<bf16>, dim3(n_tokens), dim3(ROUTE_THREADS), 0, s, (const bf16*)h,
                             width, w_r, n_experts, top, renorm, w_g, positions, experts, weights, gate, vec);
    return ST_ERR_BAD_DTYPE;
}

#define SORT_THREADS 1024

// offsets [n_experts + 1]; sorted [n_items]; place [n_items]; tile_group / tile_row0 [tile_cap]
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(const int* __restrict__ experts, int n_items, int n_experts, int tile_rows, int tile_cap,
                int* __restrict__ offsets, int* __restrict__ sorted, int* __restrict__ place,
                int* __restrict__ tile_group, int* __restrict__ tile_row0) {
    __shared__ int count[ROUTE_MAX_EXPERTS + 1];
    __shared__ int cursor[ROUTE_MAX_EXPERTS];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    for (int e = threadIdx.x; e <= n_experts; e += SORT_THREADS) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_items; i += SORT_THREADS) {
        const int e = __ldcg(experts + i);
        if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int c = count[e];
            offsets[e] = run;
            cursor[e] = run;
            for (int r = 0; r < c && tile < tile_cap; r += tile_rows, ++tile) {
                tile_group[tile] = e;
                tile_row0[tile] = run + r;
            }
            run += c;
        }
        offsets[n_experts] = run;
        for (; tile < tile_cap; ++tile) { tile_group[tile] = -1; tile_row0[tile] = 0; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_items; i += SORT_THREADS) {
        const int e = __ldcg(experts + i);
        if (e >= 0 && e < n_experts) {
            const int p = atomicAdd(&cursor[e], 1);
            sorted[p] = i;
            place[i] = p;
        } else {
            place[i] = -1;
        }
    }
}

ST_EXPORT int st_moe_sort(const int* experts, int n_items, int n_experts, int tile_rows, int tile_cap, int* offsets,
                          int* sorted, int* place, int* tile_group, int* tile_row0, void* stream) {
    if (n_items <= 0) return 0;
    if (n_experts <= 0 || tile_rows <= 0) return ST_ERR_BAD_ARG;
    if (n_experts > ROUTE_MAX_EXPERTS) return ST_ERR_TOO_LARGE;
    if (tile_cap < (n_items + tile_rows - 1) / tile_rows + n_experts) return ST_ERR_BAD_SIZE;
    return st_launch_pdl("moe_sort", moe_sort_kernel, dim3(1), dim3(SORT_THREADS), 0, (cudaStream_t)stream, experts, n_items,
                         n_experts, tile_rows, tile_cap, offsets, sorted, place, tile_group, tile_row0);
}

template <typename T, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights, int top,
                   const T* __restrict__ shared, const float* __restrict__ gate, int width, TO* __restrict__ out) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    if (VEC) {
        for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const int p = __ldcg(place + (size_t)t * top + k);
                if (p < 0) continue;
                const float w = __ldcg(weights + (size_t)t * top + k);
                const float4 v = load4_cg(y + (size_t)p * width + e);
                acc = make_float4(fmaf(w, v.x, acc.x), fmaf(w, v.y, acc.y), fmaf(w, v.z, acc.z), fmaf(w, v.w, acc.w));
            }
            if (shared) {
                const float w = __ldcg(gate + t);
                const float4 v = load4_cg(shared + (size_t)t * width + e);
                acc = make_float4(fmaf(w, v.x, acc.x), fmaf(w, v.y, acc.y), fmaf(w, v.z, acc.z), fmaf(w, v.w, acc.w));
            }
            store4(out + (size_t)t * width + e, acc);
        }
    } else
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = __ldcg(place + (size_t)t * top + k);
            if (p >= 0) acc = fmaf(__ldcg(weights + (size_t)t * top + k), load1_cg(y + (size_t)p * width + e), acc);
        }
        if (shared) acc = fmaf(__ldcg(gate + t), load1_cg(shared + (size_t)t * width + e), acc);
        out[(size_t)t * width + e] = from_f32<TO>(acc);
    }
}

ST_EXPORT int st_moe_combine(const void* y, const int* place, const float* weights, int top, const void* shared,
                             const float* gate, int n_tokens, int width, void* out, int dtype, int out_f32, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = width % 4 == 0 && aligned16(y) && aligned16(out) && (!shared || aligned16(shared));
    int block = ((vec ? width / 4 : width) + 31) / 32 * 32;
    if (block > 256) block = 256;
#define MC_LAUNCH(T, TO, VEC)                                                                                           \
    return st_launch_pdl("moe_combine", moe_combine_kernel<T, TO, VEC>, dim3(n_tokens), dim3(block), 0, s, (const T*)y, \
                         place, weights, top, (const T*)shared, gate, width, (TO*)out)
    if (dtype == 0) {
        if (vec) MC_LAUNCH(float, float, true);
        MC_LAUNCH(float, float, false);
    }
    if (dtype != 1) return ST_ERR_BAD_DTYPE;
    if (out_f32) {
        if (vec) MC_LAUNCH(bf16, float, true);
        MC_LAUNCH(bf16, float, false);
    }
    if (vec) MC_LAUNCH(bf16, bf16, true);
    MC_LAUNCH(bf16, bf16, false);
#undef MC_LAUNCH
}

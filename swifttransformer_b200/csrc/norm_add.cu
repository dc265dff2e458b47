// Two elementwise kernels of blocks that normalise a sub-layer's OUTPUT before the residual sum, and of
// gated feed-forwards.
//
// norm_add:   x[r] += mult * gain * y[r] / sqrt(mean(y[r]^2) + eps)      (gain: one number, read from the device)
//             optionally act[r] = x[r] in the activation type, for the sub-layer that reads x next.
//             x is the float residual stream; statistics and the sum are float for every storage type.
// gated_act:  out[r][j] = act(gu[r][j]) * gu[r][inner + j]               (gu = the fused gate | up product)
#include "common.cuh"

template <typename T, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
norm_add_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ gain, float mult, float eps,
                int width, const int* __restrict__ positions, TO* __restrict__ act) {
    __shared__ float scratch[32];
    const float g = gain[0];                             // a weight: fetched before the wait
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int r = blockIdx.x;
    if (positions && positions[r] < 0) return;          // padding token of a fixed-shape step
    const T* yr = y + (size_t)r * width;
    float* xr = x + (size_t)r * width;
    float ss = 0.f;
    if (VEC) {
        for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
            const float4 v = load4_cg(yr + e);
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    } else {
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            const float v = load1_cg(yr + e);
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float k = rsqrtf(ss / (float)width + eps) * g * mult;
    if (VEC) {
        for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
            const float4 v = load4_cg(yr + e), o = load4_cg(xr + e);
            const float4 n = make_float4(o.x + k * v.x, o.y + k * v.y, o.z + k * v.z, o.w + k * v.w);
            store4(xr + e, n);
            if (act) store4(act + (size_t)r * width + e, n);
        }
    } else {
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            const float v = __ldcg(xr + e) + k * load1_cg(yr + e);
            xr[e] = v;
            if (act) act[(size_t)r * width + e] = from_f32<TO>(v);
        }
    }
}

ST_EXPORT int st_norm_add(float* x, const void* y, const float* gain, float mult, float eps, int n_rows, int width,
                          const int* positions, void* act, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return ST_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = width % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(act);
    int block = ((vec ? width / 4 : width) + 31) / 32 * 32;
    if (block > 256) block = 256;
#define NA_LAUNCH(T, VEC)                                                                                         \
    return st_launch_pdl("norm_add", norm_add_kernel<T, T, VEC>, dim3(n_rows), dim3(block), 0, s, x, (const T*)y, gain, \
                         mult, eps, width, positions, (T*)act)
    if (dtype == 0) {
        if (vec) NA_LAUNCH(float, true);
        NA_LAUNCH(float, false);
    } else if (dtype == 1) {
        if (vec) NA_LAUNCH(bf16, true);
        NA_LAUNCH(bf16, false);
    }
#undef NA_LAUNCH
    return ST_ERR_BAD_DTYPE;
}

// VEC: inner % 8 == 0 and 16-byte aligned rows: eight outputs per thread
template <typename T, bool VEC>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int inner, size_t total, int act) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (VEC) {
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < total; i += stride * 8) {
            const size_t r = i / inner, j = i % inner;
            const T* row = gu + r * 2 * inner + j;
            const float4 g0 = load4_cg(row), g1 = load4_cg(row + 4), u0 = load4_cg(row + inner), u1 = load4_cg(row + inner + 4);
            store4(out + i, make_float4(apply_act(g0.x, act) * u0.x, apply_act(g0.y, act) * u0.y,
                                        apply_act(g0.z, act) * u0.z, apply_act(g0.w, act) * u0.w));
            store4(out + i + 4, make_float4(apply_act(g1.x, act) * u1.x, apply_act(g1.y, act) * u1.y,
                                            apply_act(g1.z, act) * u1.z, apply_act(g1.w, act) * u1.w));
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            const size_t r = i / inner, j = i % inner;
            const T* row = gu + r * 2 * inner;
            out[i] = from_f32<T>(apply_act(load1_cg(row + j), act) * load1_cg(row + inner + j));
        }
    }
}

ST_EXPORT int st_gated_act(const void* gu, void* out, int n_rows, int inner, int act, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (inner <= 0 || act < 0 || act > 4) return ST_ERR_BAD_ARG;
    const size_t total = (size_t)n_rows * inner;
    const bool vec = inner % 8 == 0 && aligned16(gu) && aligned16(out);
    const size_t work = vec ? total / 8 : total;
    int grid = (int)((work + 255) / 256);
    if (grid > st_sm_count() * 16) grid = st_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
#define GA_LAUNCH(T, VEC)                                                                                         \
    return st_launch_pdl("gated_act", gated_act_kernel<T, VEC>, dim3(grid), dim3(256), 0, s, (const T*)gu, (T*)out, inner, \
                         total, act)
    if (dtype == 0) {
        if (vec) GA_LAUNCH(float, true);
        GA_LAUNCH(float, false);
    } else if (dtype == 1) {
        if (vec) GA_LAUNCH(bf16, true);
        GA_LAUNCH(bf16, false);
    }
#undef GA_LAUNCH
    return ST_ERR_BAD_DTYPE;
}

// The gated unit with limits, from the fused gate | up product gu [rows, 2 * inner] and its bias (float
// [2 * inner] or null):  g = min(gate + b_g, limit), u = clamp(up + b_u, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + shift).  limit <= 0: no limits.
__device__ __forceinline__ float gated_clamped_one(float g, float u, float limit, float alpha, float shift) {
    if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
    return g / (1.f + expf(-alpha * g)) * (u + shift);
}

// VEC: inner % 8 == 0 and 16-byte aligned rows: eight outputs per thread
template <typename T, bool VEC>
__global__ void gated_clamped_act_kernel(const T* __restrict__ gu, const float* __restrict__ bias, T* __restrict__ out,
                                         int inner, size_t total, float limit, float alpha, float shift) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (VEC) {
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < total; i += stride * 8) {
            const size_t r = i / inner, j = i % inner;
            const T* row = gu + r * 2 * inner + j;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float4 g = load4_cg(row + 4 * half), u = load4_cg(row + inner + 4 * half);
                if (bias) {
                    g = add4(g, load4(bias + j + 4 * half));
                    u = add4(u, load4(bias + inner + j + 4 * half));
                }
                store4(out + i + 4 * half, make_float4(gated_clamped_one(g.x, u.x, limit, alpha, shift),
                                                       gated_clamped_one(g.y, u.y, limit, alpha, shift),
                                                       gated_clamped_one(g.z, u.z, limit, alpha, shift),
                                                       gated_clamped_one(g.w, u.w, limit, alpha, shift)));
            }
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            const size_t r = i / inner, j = i % inner;
            const T* row = gu + r * 2 * inner;
            float g = load1_cg(row + j), u = load1_cg(row + inner + j);
            if (bias) { g += bias[j]; u += bias[inner + j]; }
            out[i] = from_f32<T>(gated_clamped_one(g, u, limit, alpha, shift));
        }
    }
}

ST_EXPORT int st_gated_clamped_act(const void* gu, const float* bias, void* out, int n_rows, int inner, float limit,
                                   float alpha, float shift, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (inner <= 0) return ST_ERR_BAD_ARG;
    const size_t total = (size_t)n_rows * inner;
    const bool vec = inner % 8 == 0 && aligned16(gu) && aligned16(out) && (!bias || aligned16(bias));
    const size_t work = vec ? total / 8 : total;
    int grid = (int)((work + 255) / 256);
    if (grid > st_sm_count() * 16) grid = st_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
#define GC_LAUNCH(T, VEC)                                                                                          \
    return st_launch_pdl("gated_clamped", gated_clamped_act_kernel<T, VEC>, dim3(grid), dim3(256), 0, s, (const T*)gu, \
                         bias, (T*)out, inner, total, limit, alpha, shift)
    if (dtype == 0) {
        if (vec) GC_LAUNCH(float, true);
        GC_LAUNCH(float, false);
    } else if (dtype == 1) {
        if (vec) GC_LAUNCH(bf16, true);
        GC_LAUNCH(bf16, false);
    }
#undef GC_LAUNCH
    return ST_ERR_BAD_DTYPE;
}

// Several copies of the residual stream ("hyper-connections"), and what stands around them.
//
// A model with n streams keeps lanes [n][tokens][width] in float.  A sub-layer reads one mixture of them and its
// result goes back into all of them:
//
//   u        = sum_s a[s] * lanes[s]                          h = u / sqrt(mean(u^2) + eps) * w      (hc_read_norm)
//   lanes[t] <- sum_s M[s][t] * lanes[s] + b[t] * y           all t at once from the old lanes        (hc_write)
//
// hc_write_read_norm does the update of one sub-layer and the read of the next in one pass over the copies (a block per
// token: the new values are written back and their mixture is normed while they are still in registers).
//
// hc_step_conv does all of that and the sub-layer's input convolution for steps in which every request brings one token.
//
// hc_spread makes the n copies of the embedding's rows, hc_sum adds them up at the end.  a, b [n] and M [n][n]
// (indexed [from][to]) are float vectors on the device.
//
// norm_pair_sum:  out = ca * wa * A / rms(A) + cb * wb * B / rms(B), row by row, float out: two sub-results that are
//                 normed over the model width before they meet.
// xielu:          z > 0: ap z^2 + z/2;  z <= 0: aq (exp(z) - 1 - z) + z/2, in place.
//
// All arithmetic is float; rows of tokens at a negative position (padding of a fixed-shape step) are skipped
// where a kernel is given the positions.
#include "common.cuh"

#define HC_MAX_STREAMS 8
#define HC_THREADS 256

__global__ void __launch_bounds__(HC_THREADS)
hc_spread_kernel(const float* __restrict__ x, float* __restrict__ lanes, long long n_elems, int n_streams) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const long long i = (long long)blockIdx.x * HC_THREADS + threadIdx.x;
    if (i >= n_elems) return;
    const float v = __ldcg(x + i);
    for (int s = 0; s < n_streams; ++s) lanes[(long long)s * n_elems + i] = v;
}

__global__ void __launch_bounds__(HC_THREADS)
hc_sum_kernel(const float* __restrict__ lanes, float* __restrict__ x, long long n_elems, int n_streams) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const long long i = (long long)blockIdx.x * HC_THREADS + threadIdx.x;
    if (i >= n_elems) return;
    float v = 0.f;
    for (int s = 0; s < n_streams; ++s) v += __ldcg(lanes + (long long)s * n_elems + i);
    x[i] = v;
}

// One block per token.  The mixture is written to `out` first and rescaled in place by the thread that wrote it,
// so a row of any width needs no staging.  out: float [tokens, width].
__global__ void __launch_bounds__(HC_THREADS)
hc_read_norm_kernel(const float* __restrict__ lanes, long long lane_stride, int n_streams,
                    const float* __restrict__ coef, const float* __restrict__ gain, float eps, int width,
                    float* __restrict__ out, const int* __restrict__ positions) {
    __shared__ float scratch[32];
    float a[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s) a[s] = s < n_streams ? coef[s] : 0.f;
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    if (positions && positions[t] < 0) return;
    const float* row = lanes + (size_t)t * width;
    float* dst = out + (size_t)t * width;
    float ss = 0.f;
    if ((width & 3) == 0) {
        for (int c = threadIdx.x * 4; c < width; c += HC_THREADS * 4) {
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s) {
                if (s >= n_streams) break;
                const float4 v = load4_cg(row + (size_t)s * lane_stride + c);
                u.x = fmaf(a[s], v.x, u.x); u.y = fmaf(a[s], v.y, u.y); u.z = fmaf(a[s], v.z, u.z); u.w = fmaf(a[s], v.w, u.w);
            }
            ss = fmaf(u.x, u.x, fmaf(u.y, u.y, fmaf(u.z, u.z, fmaf(u.w, u.w, ss))));
            store4(dst + c, u);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += HC_THREADS) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s) {
                if (s >= n_streams) break;
                u = fmaf(a[s], __ldcg(row + (size_t)s * lane_stride + c), u);
            }
            ss = fmaf(u, u, ss);
            dst[c] = u;
        }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
    if ((width & 3) == 0) {
        for (int c = threadIdx.x * 4; c < width; c += HC_THREADS * 4) {
            float4 u = load4(dst + c);
            const float4 g = *reinterpret_cast<const float4*>(gain + c);
            u.x *= inv * g.x; u.y *= inv * g.y; u.z *= inv * g.z; u.w *= inv * g.w;
            store4(dst + c, u);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += HC_THREADS) dst[c] = dst[c] * inv * gain[c];
    }
}

// A thread per (token, channel): reads the n old values, writes the n new ones.  y: float or the storage type.
template <typename TY>
__global__ void __launch_bounds__(HC_THREADS)
hc_write_kernel(float* __restrict__ lanes, long long lane_stride, int n_streams, const float* __restrict__ mix,
                const float* __restrict__ outc, const TY* __restrict__ y, long long n_elems) {
    __shared__ float m[HC_MAX_STREAMS * HC_MAX_STREAMS], b[HC_MAX_STREAMS];
    if (threadIdx.x < n_streams * n_streams) m[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < n_streams) b[threadIdx.x] = outc[threadIdx.x];
    __syncthreads();
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const long long i = (long long)blockIdx.x * HC_THREADS + threadIdx.x;
    if (i >= n_elems) return;
    float old[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s) old[s] = s < n_streams ? __ldcg(lanes + (long long)s * lane_stride + i) : 0.f;
    const float yv = load1_cg(y + i);
#pragma unroll
    for (int t = 0; t < HC_MAX_STREAMS; ++t) {
        if (t >= n_streams) break;
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < n_streams) v = fmaf(m[s * n_streams + t], old[s], v);
        lanes[(long long)t * lane_stride + i] = fmaf(b[t], yv, v);
    }
}

// The update of the sub-layer that just ran and the read of the next one, one block per token:
//   lanes[t] <- sum_s M[s][t] lanes[s] + b[t] y;   u = sum_t a[t] lanes[t];   out = u / rms(u) * gain
// V = 4: four neighbouring channels per thread (width % 4 == 0), V = 1: any width.
template <typename TY, int V>
__global__ void __launch_bounds__(HC_THREADS)
hc_write_read_norm_kernel(float* __restrict__ lanes, long long lane_stride, int n_streams,
                          const float* __restrict__ mix, const float* __restrict__ outc, const TY* __restrict__ y,
                          const float* __restrict__ coef, const float* __restrict__ gain, float eps, int width,
                          float* __restrict__ out, const int* __restrict__ positions) {
    __shared__ float m[HC_MAX_STREAMS * HC_MAX_STREAMS], b[HC_MAX_STREAMS], a[HC_MAX_STREAMS];
    __shared__ float scratch[32];
    if (threadIdx.x < n_streams * n_streams) m[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < n_streams) { b[threadIdx.x] = outc[threadIdx.x]; a[threadIdx.x] = coef[threadIdx.x]; }
    __syncthreads();
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    if (positions && positions[t] < 0) return;
    float* row = lanes + (size_t)t * width;
    const TY* yrow = y + (size_t)t * width;
    float* dst = out + (size_t)t * width;
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < width; c += HC_THREADS * V) {
        float old[HC_MAX_STREAMS][V], yv[V], u[V];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s) {
            if (s >= n_streams) break;
            if (V == 4) {
                const float4 v = load4_cg(row + (size_t)s * lane_stride + c);
                old[s][0] = v.x; old[s][1] = v.y; old[s][2] = v.z; old[s][V - 1] = v.w;
            } else {
                old[s][0] = __ldcg(row + (size_t)s * lane_stride + c);
            }
        }
        if (V == 4) {
            const float4 v = load4_cg(yrow + c);
            yv[0] = v.x; yv[1] = v.y; yv[2] = v.z; yv[V - 1] = v.w;
        } else {
            yv[0] = load1_cg(yrow + c);
        }
#pragma unroll
        for (int x = 0; x < V; ++x) u[x] = 0.f;
#pragma unroll 1
        for (int q = 0; q < n_streams; ++q) {
            float nv[V];
#pragma unroll
            for (int x = 0; x < V; ++x) {
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < HC_MAX_STREAMS; ++s)
                    if (s < n_streams) v = fmaf(m[s * n_streams + q], old[s][x], v);
                nv[x] = fmaf(b[q], yv[x], v);
                u[x] = fmaf(a[q], nv[x], u[x]);
            }
            if (V == 4) store4(row + (size_t)q * lane_stride + c, make_float4(nv[0], nv[1], nv[2], nv[V - 1]));
            else row[(size_t)q * lane_stride + c] = nv[0];
        }
#pragma unroll
        for (int x = 0; x < V; ++x) ss = fmaf(u[x], u[x], ss);
        if (V == 4) store4(dst + c, make_float4(u[0], u[1], u[2], u[V - 1]));
        else dst[c] = u[0];
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
    for (int c = threadIdx.x * V; c < width; c += HC_THREADS * V) {
        if (V == 4) {
            float4 u = load4(dst + c);
            const float4 g = *reinterpret_cast<const float4*>(gain + c);
            u.x *= inv * g.x; u.y *= inv * g.y; u.z *= inv * g.z; u.w *= inv * g.w;
            store4(dst + c, u);
        } else {
            dst[c] = dst[c] * inv * gain[c];
        }
    }
}

// y_dtype: 0 float, 1 bfloat16
ST_EXPORT int st_hc_write_read_norm(float* lanes, int n_streams, const float* mix, const float* outc, const void* y,
                                    int y_dtype, const float* coef, const float* gain, float eps, int n_tokens, int width,
                                    float* out, const int* positions, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_streams <= 0 || width <= 0) return ST_ERR_BAD_ARG;
    if (n_streams > HC_MAX_STREAMS) return ST_ERR_TOO_LARGE;
    const long long stride = (long long)n_tokens * width;
    const bool vec = width % 4 == 0 && aligned16(lanes) && aligned16(y) && aligned16(out) && aligned16(gain);
    cudaStream_t s = (cudaStream_t)stream;
#define HCWR(TY, V)                                                                                                   \
    return st_launch_pdl("hc_write_read", hc_write_read_norm_kernel<TY, V>, dim3(n_tokens), dim3(HC_THREADS), 0, s,   \
                         lanes, stride, n_streams, mix, outc, (const TY*)y, coef, gain, eps, width, out, positions)
    if (y_dtype == 0) { if (vec) HCWR(float, 4); HCWR(float, 1); }
    if (y_dtype == 1) { if (vec) HCWR(bf16, 4); HCWR(bf16, 1); }
#undef HCWR
    return ST_ERR_BAD_DTYPE;
}

// Steps in which every request brings one token: update (y != null), read, norm and the input convolution in one
// kernel, a block per token.  h = norm(u); out_act = h + sum_j w[c][j] * (the request's last taps - 1 inputs, h); the
// state moves on by h.  A thread owns its channels of the request's state: conv_state float [slots][taps - 1][width].
#define HC_MAX_TAPS 8
#define HC_STEP_THREADS 1024     // such a step has few tokens, so few blocks: a block's threads are its parallelism
template <typename TY, typename TO>
__global__ void __launch_bounds__(HC_STEP_THREADS)
hc_step_conv_kernel(float* __restrict__ lanes, long long lane_stride, int n_streams, const float* __restrict__ mix,
                    const float* __restrict__ outc, const TY* __restrict__ y, const float* __restrict__ coef,
                    const float* __restrict__ gain, float eps, int width, const float* __restrict__ conv_w, int taps,
                    float* __restrict__ conv_state, int write_state, float* __restrict__ tmp, TO* __restrict__ out_act,
                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                    const int* __restrict__ slots) {
    __shared__ float m[HC_MAX_STREAMS * HC_MAX_STREAMS], b[HC_MAX_STREAMS], a[HC_MAX_STREAMS];
    __shared__ float scratch[32];
    if (y && threadIdx.x < n_streams * n_streams) m[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < n_streams) { b[threadIdx.x] = y ? outc[threadIdx.x] : 0.f; a[threadIdx.x] = coef[threadIdx.x]; }
    __syncthreads();
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    if (positions[t] < 0) return;
    float* row = lanes + (size_t)t * width;
    float* dst = tmp + (size_t)t * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += HC_STEP_THREADS) {
        float old[HC_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s) old[s] = s < n_streams ? __ldcg(row + (size_t)s * lane_stride + c) : 0.f;
        float u = 0.f;
        if (y) {
            const float yv = load1_cg(y + (size_t)t * width + c);
#pragma unroll 1
            for (int q = 0; q < n_streams; ++q) {
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < HC_MAX_STREAMS; ++s)
                    if (s < n_streams) v = fmaf(m[s * n_streams + q], old[s], v);
                v = fmaf(b[q], yv, v);
                row[(size_t)q * lane_stride + c] = v;
                u = fmaf(a[q], v, u);
            }
        } else {
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < n_streams) u = fmaf(a[s], old[s], u);
        }
        ss = fmaf(u, u, ss);
        dst[c] = u;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
    const int keep = taps - 1;
    float* st = conv_state + (size_t)slots[seq_of_token[t]] * keep * width;
    for (int c = threadIdx.x; c < width; c += HC_STEP_THREADS) {
        const float h = dst[c] * inv * gain[c];
        float vv[HC_MAX_TAPS];
        float o = h;
        for (int j = 0; j < keep; ++j) {
            vv[j] = __ldcg(st + (size_t)j * width + c);
            o = fmaf(conv_w[(size_t)c * taps + j], vv[j], o);
        }
        o = fmaf(conv_w[(size_t)c * taps + keep], h, o);
        if (write_state) {
            for (int j = 0; j + 1 < keep; ++j) st[(size_t)j * width + c] = vv[j + 1];
            if (keep > 0) st[(size_t)(keep - 1) * width + c] = h;
        }
        out_act[(size_t)t * width + c] = from_f32<TO>(o);
    }
}

// y null: no update, read only.  y_dtype / out_dtype: 0 float, 1 bfloat16.  tmp: float [n_tokens][width] scratch.
ST_EXPORT int st_hc_step_conv(float* lanes, int n_streams, const float* mix, const float* outc, const void* y, int y_dtype,
                              const float* coef, const float* gain, float eps, int n_tokens, int width,
                              const float* conv_w, int taps, float* conv_state, int write_state, float* tmp,
                              void* out_act, int out_dtype, const int* positions, const int* seq_of_token,
                              const int* slots, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_streams <= 0 || width <= 0 || taps < 1 || !positions || !seq_of_token || !slots) return ST_ERR_BAD_ARG;
    if (n_streams > HC_MAX_STREAMS || taps > HC_MAX_TAPS) return ST_ERR_TOO_LARGE;
    const long long stride = (long long)n_tokens * width;
    cudaStream_t s = (cudaStream_t)stream;
#define HCSC(TY, TO)                                                                                                  \
    return st_launch_pdl("hc_step_conv", hc_step_conv_kernel<TY, TO>, dim3(n_tokens), dim3(HC_STEP_THREADS), 0, s, lanes, \
                         stride, n_streams, mix, outc, (const TY*)y, coef, gain, eps, width, conv_w, taps, conv_state, \
                         write_state, tmp, (TO*)out_act, positions, seq_of_token, slots)
    const int yd = y ? y_dtype : 0;
    if (yd == 0 && out_dtype == 0) HCSC(float, float);
    if (yd == 0 && out_dtype == 1) HCSC(float, bf16);
    if (yd == 1 && out_dtype == 0) HCSC(bf16, float);
    if (yd == 1 && out_dtype == 1) HCSC(bf16, bf16);
#undef HCSC
    return ST_ERR_BAD_DTYPE;
}

ST_EXPORT int st_hc_spread(const float* x, float* lanes, long long n_elems, int n_streams, void* stream) {
    if (n_elems <= 0) return 0;
    if (n_streams <= 0) return ST_ERR_BAD_ARG;
    return st_launch_pdl("hc_spread", hc_spread_kernel, dim3((unsigned)((n_elems + HC_THREADS - 1) / HC_THREADS)),
                         dim3(HC_THREADS), 0, (cudaStream_t)stream, x, lanes, n_elems, n_streams);
}

ST_EXPORT int st_hc_sum(const float* lanes, float* x, long long n_elems, int n_streams, void* stream) {
    if (n_elems <= 0) return 0;
    if (n_streams <= 0) return ST_ERR_BAD_ARG;
    return st_launch_pdl("hc_sum", hc_sum_kernel, dim3((unsigned)((n_elems + HC_THREADS - 1) / HC_THREADS)),
                         dim3(HC_THREADS), 0, (cudaStream_t)stream, lanes, x, n_elems, n_streams);
}

ST_EXPORT int st_hc_read_norm(const float* lanes, int n_streams, const float* coef, const float* gain, float eps,
                              int n_tokens, int width, float* out, const int* positions, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_streams <= 0 || width <= 0) return ST_ERR_BAD_ARG;
    if (n_streams > HC_MAX_STREAMS) return ST_ERR_TOO_LARGE;
    return st_launch_pdl("hc_read_norm", hc_read_norm_kernel, dim3(n_tokens), dim3(HC_THREADS), 0, (cudaStream_t)stream,
                         lanes, (long long)n_tokens * width, n_streams, coef, gain, eps, width, out, positions);
}

// y_dtype: 0 float, 1 bfloat16
ST_EXPORT int st_hc_write(float* lanes, int n_streams, const float* mix, const float* outc, const void* y, int y_dtype,
                          int n_tokens, int width, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_streams <= 0 || width <= 0) return ST_ERR_BAD_ARG;
    if (n_streams > HC_MAX_STREAMS) return ST_ERR_TOO_LARGE;
    const long long n = (long long)n_tokens * width;
    const dim3 grid((unsigned)((n + HC_THREADS - 1) / HC_THREADS));
    if (y_dtype == 0)
        return st_launch_pdl("hc_write", hc_write_kernel<float>, grid, dim3(HC_THREADS), 0, (cudaStream_t)stream, lanes, n,
                             n_streams, mix, outc, (const float*)y, n);
    if (y_dtype == 1)
        return st_launch_pdl("hc_write", hc_write_kernel<bf16>, grid, dim3(HC_THREADS), 0, (cudaStream_t)stream, lanes, n,
                             n_streams, mix, outc, (const bf16*)y, n);
    return ST_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------------------
template <typename TA, typename TB>
__global__ void __launch_bounds__(HC_THREADS)
norm_pair_sum_kernel(const TA* __restrict__ a, const float* __restrict__ wa, float ca, const TB* __restrict__ b,
                     const float* __restrict__ wb, float cb, float eps, int width, float* __restrict__ out,
                     const int* __restrict__ positions) {
    __shared__ float scratch[32];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    if (positions && positions[t] < 0) return;
    const TA* ra = a + (size_t)t * width;
    const TB* rb = b + (size_t)t * width;
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < width; c += HC_THREADS) {
        const float x = load1_cg(ra + c), y = load1_cg(rb + c);
        sa = fmaf(x, x, sa);
        sb = fmaf(y, y, sb);
    }
    const float ia = ca * rsqrtf(block_sum(sa, scratch) / (float)width + eps);
    const float ib = cb * rsqrtf(block_sum(sb, scratch) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += HC_THREADS)
        out[(size_t)t * width + c] = fmaf(load1_cg(ra + c) * ia, wa[c], load1_cg(rb + c) * ib * wb[c]);
}

// a_dtype / b_dtype: 0 float, 1 bfloat16
ST_EXPORT int st_norm_pair_sum(const void* a, int a_dtype, const float* wa, float ca, const void* b, int b_dtype,
                               const float* wb, float cb, float eps, int n_rows, int width, float* out,
                               const int* positions, void* stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return ST_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
#define NPS(TA, TB)                                                                                                   \
    return st_launch_pdl("norm_pair_sum", norm_pair_sum_kernel<TA, TB>, dim3(n_rows), dim3(HC_THREADS), 0, s,         \
                         (const TA*)a, wa, ca, (const TB*)b, wb, cb, eps, width, out, positions)
    if (a_dtype == 0 && b_dtype == 0) NPS(float, float);
    if (a_dtype == 1 && b_dtype == 0) NPS(bf16, float);
    if (a_dtype == 0 && b_dtype == 1) NPS(float, bf16);
    if (a_dtype == 1 && b_dtype == 1) NPS(bf16, bf16);
#undef NPS
    return ST_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float xielu_(float z, float ap, float aq) {
    return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(HC_THREADS)
xielu_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n, float ap, float aq) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const long long i = ((long long)blockIdx.x * HC_THREADS + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = load4_cg(in + i);
        store4(out + i, make_float4(xielu_(v.x, ap, aq), xielu_(v.y, ap, aq), xielu_(v.z, ap, aq), xielu_(v.w, ap, aq)));
    } else {
        for (long long j = i; j < n; ++j) out[j] = from_f32<TO>(xielu_(load1_cg(in + j), ap, aq));
    }
}

// in: float or the storage type `dtype` (in_f32); out: the storage type.  n must keep rows 4-element aligned for the
// vector path: the launcher checks the pointers and falls back to single elements by passing n as it is.
ST_EXPORT int st_xielu(const void* in, int in_f32, void* out, long long n, float ap, float aq, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (!aligned16(in) || !aligned16(out)) return ST_ERR_BAD_ARG;
    const dim3 grid((unsigned)((n + HC_THREADS * 4 - 1) / (HC_THREADS * 4)));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0)
        return st_launch_pdl("xielu", xielu_kernel<float, float>, grid, dim3(HC_THREADS), 0, s, (const float*)in, (float*)out, n, ap, aq);
    if (dtype == 1 && in_f32)
        return st_launch_pdl("xielu", xielu_kernel<float, bf16>, grid, dim3(HC_THREADS), 0, s, (const float*)in, (bf16*)out, n, ap, aq);
    if (dtype == 1)
        return st_launch_pdl("xielu", xielu_kernel<bf16, bf16>, grid, dim3(HC_THREADS), 0, s, (const bf16*)in, (bf16*)out, n, ap, aq);
    return ST_ERR_BAD_DTYPE;
}

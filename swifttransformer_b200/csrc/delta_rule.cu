// The gated delta rule: a linear recurrence whose state is corrected towards each token's value.
//
// Per value head h (G query/key heads serve H value heads: g = h / (H / G)), with S [dim, vd] zero when a
// request starts:
//
//   q, k, v  = silu(conv(projection))            short causal convolution over time, one filter per channel
//   q <- q / sqrt(sum q^2 + 1e-6) * dim^(-1/2),  k <- k / sqrt(sum k^2 + 1e-6)          per head
//   beta     = sigmoid(b)                                                              per head
//   decay_c  = exp(-exp(A_log_h) * softplus(sum_r a1_r * W_a2[h * dim + c, r] + dt_bias[h * dim + c]))
//   S <- diag(decay) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//   out      = out_scale * o / sqrt(mean(o^2) + eps) * w * sigmoid(sum_r g1_r * W_g2[h * vd + e, r])
//
// Two simpler forms of the same are taken by rank: with rank_a == 0 the projection holds one decay logit per head
// at a_off (dt_bias is then [H] and all key channels of a head decay alike); with rank_g == 0 it holds the output
// gate's logits themselves at g_off ([H * vd]).  gate_silu: the gate is z * sigmoid(z) instead of sigmoid(z).
//
// Three kernels.  delta_prepare turns a token's row of the float projection [q | k | v | b | a1 | g1] into a
// float row [q (G*dim) | k (G*dim) | v (H*vd) | decay (H*dim) | beta (H)]; delta_scan walks each request's
// tokens with the state's columns in registers (a column of S evolves on its own: its dot products with k and q
// are sums over dim, shared by the L lanes that hold the column) and the tokens' rows staged in shared memory; delta_output norms and gates each head's o.
// Everything here is float arithmetic; only the low-rank matrices and the result are in the storage type.
//
// Since (decay S + k u^T)^T q = (decay S)^T q + u (k . q), both dot products of a token are taken from the
// decayed state in one pass of shuffles.
#include "common.cuh"

#define DR_MAX_TAPS 8
#define DR_PREP_THREADS 256
#define DR_EARLY_TOKENS 128   // steps of at most this many tokens let the next kernel's blocks in early
#define DR_UNIT_PASSES 8      // a warp's lanes cover a head of up to 32 * DR_UNIT_PASSES channels

struct DeltaShape {
    int H, G, dim, vd;            // value heads, query/key heads, key size, value size
    int q_off, k_off, v_off, b_off, a_off, g_off;   // columns of the projection
    int rank_a, rank_g;           // 0: no low-rank pair, the projection holds the logits themselves (see below)
    int gate_silu;                // the output gate: 0 sigmoid(z), 1 z * sigmoid(z)
    // columns of a prepared row
    __host__ __device__ int pq() const { return 0; }
    __host__ __device__ int pk() const { return G * dim; }
    __host__ __device__ int pv() const { return 2 * G * dim; }
    __host__ __device__ int pd() const { return 2 * G * dim + H * vd; }
    __host__ __device__ int pb() const { return 2 * G * dim + H * vd + H * dim; }
    __host__ __device__ int row() const { return 2 * G * dim + H * vd + H * dim + H; }
};

__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.f + expf(-z)); }

// sum_r x[r] * w[r] in the order of r, the weights fetched in 16-byte pieces where the row allows it
#define DR_RANK_SMEM 256      // low-rank inputs of up to this many numbers wait in shared memory
template <typename TW>
__device__ __forceinline__ float lowrank_dot(const float* x, const TW* __restrict__ w, int rank) {
    float z = 0.f;
    if constexpr (sizeof(TW) == 2) {
        if ((rank & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
            for (int r = 0; r < rank; r += 8) {
                const uint4 u = __ldg(reinterpret_cast<const uint4*>(w + r));
                const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    z = fmaf(x[r + 2 * i], __uint_as_float(w4[i] << 16), z);
                    z = fmaf(x[r + 2 * i + 1], __uint_as_float(w4[i] & 0xffff0000u), z);
                }
            }
            return z;
        }
    } else {
        if ((rank & 3) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
            for (int r = 0; r < rank; r += 4) {
                const float4 u = __ldg(reinterpret_cast<const float4*>(w + r));
                z = fmaf(x[r], u.x, z); z = fmaf(x[r + 1], u.y, z); z = fmaf(x[r + 2], u.z, z); z = fmaf(x[r + 3], u.w, z);
            }
            return z;
        }
    }
    for (int r = 0; r < rank; ++r) z = fmaf(x[r], to_f32(w[r]), z);
    return z;
}

// conv_w: float [2*G*dim + H*vd, taps] in the projection's order q | k | v; state: [slots, taps-1, channels]
// float, the last taps-1 projected rows of every request (read here; with move_state, in steps where every request
// brings one token, also moved on here: the thread that reads a channel's state is the only one that writes it).
template <typename TW>
__global__ void __launch_bounds__(DR_PREP_THREADS)
delta_prepare_kernel(const float* __restrict__ proj, int ld, DeltaShape sh, const float* __restrict__ conv_w,
                     float* __restrict__ state, int move_state, int taps, const TW* __restrict__ w_a2,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ prep,
                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                     const int* __restrict__ q_start, const int* __restrict__ slots) {
    ST_PDL_WAIT();
    // In a step of few tokens the recurrence's blocks may come in at once.  In a long portion they come in when this
    // grid is all but done: let in early, they were placed on the few multiprocessors that had room beside this
    // grid's blocks, many to each, and the walk over 2048 tokens took nearly twice as long (measured).
    const bool early = gridDim.x <= DR_EARLY_TOKENS;
    if (early) ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0) return;
    const int b = seq_of_token[t];
    const int i = t - q_start[b];                         // the token's place in its portion
    const int H = sh.H, G = sh.G, dim = sh.dim, vd = sh.vd;
    const int channels = 2 * G * dim + H * vd;
    const int keep = taps - 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const float* row = proj + (size_t)t * ld;
    float* st = state + (size_t)slots[b] * keep * channels;
    float* dst = prep + (size_t)t * sh.row();
    const int units = 2 * G + H;
    for (int u = blockIdx.y * nwarp + warp; u < units; u += nwarp * gridDim.y) {
        const bool is_v = u >= 2 * G;
        const int width = is_v ? vd : dim;
        const int ch0 = is_v ? 2 * G * dim + (u - 2 * G) * vd : u * dim;     // q heads, then k heads, then v heads
        float x[DR_UNIT_PASSES];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < DR_UNIT_PASSES; ++r) {
            x[r] = 0.f;
            const int e = lane + 32 * r;
            if (e >= width) continue;
            const int c = ch0 + e;
            // the projection's columns q_off.. hold q | k | v in this order
            float y = 0.f, vv[DR_MAX_TAPS];
            for (int j = 0; j < taps; ++j) {
                const int back = keep - j;
                float v;
                if (back <= i) v = __ldcg(row - (size_t)back * ld + sh.q_off + c);
                else v = __ldcg(st + (size_t)(keep - (back - i)) * channels + c);    // zero before the request's start
                vv[j] = v;
                y = fmaf(conv_w[(size_t)c * taps + j], v, y);
            }
            if (move_state)
                for (int j = 0; j < keep; ++j) st[(size_t)j * channels + c] = vv[j + 1];
            y = siluf_(y);
            x[r] = y;
            ss = fmaf(y, y, ss);
        }
        float mult = 1.f;
        if (!is_v) {
            ss = warp_sum(ss);
            mult = rsqrtf(ss + 1e-6f);
            if (u < G) mult *= rsqrtf((float)dim);
        }
#pragma unroll
        for (int r = 0; r < DR_UNIT_PASSES; ++r) {
            const int e = lane + 32 * r;
            if (e < width) dst[ch0 + e] = x[r] * mult;       // the prepared row starts with q | k | v as well
        }
    }
    if (blockIdx.y == 0) {
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            dst[sh.pb() + h] = 1.f / (1.f + expf(-__ldcg(row + sh.b_off + h)));
    }
    // decays: the low-rank step size, one thread per (head, key channel)
    __shared__ float xs_a[DR_RANK_SMEM];
    const float* xa = row + sh.a_off;
    if (sh.rank_a > 0 && sh.rank_a <= DR_RANK_SMEM) {
        for (int r = threadIdx.x; r < sh.rank_a; r += blockDim.x) xs_a[r] = __ldcg(xa + r);
        __syncthreads();
        xa = xs_a;
    }
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H * dim; c += blockDim.x * gridDim.y) {
        float z, bias;
        if (sh.rank_a > 0) {
            z = lowrank_dot(xa, w_a2 + (size_t)c * sh.rank_a, sh.rank_a);
            bias = dt_bias[c];
        } else {
            z = __ldcg(xa + c / dim);
            bias = dt_bias[c / dim];
        }
        const float dt = softplusf_(z + bias);
        dst[sh.pd() + c] = expf(-expf(a_log[c / dim]) * dt);
    }
    if (!early) ST_PDL_TRIGGER();
}

// ------------------------------------------------------------------------------------------------
// The recurrence.  grid (requests of the step, H, column groups); a block of DS_THREADS threads holds
// DS_THREADS / L columns of one head's state, L lanes per column with R rows each (dim <= L * R); lane `sub` of a
// column holds rows sub * R .. sub * R + R - 1.
//
// A token's step is short (a few hundred cycles) and the next one cannot start before it ends, so a trip to
// memory per token would be most of the time.  The block therefore brings the prepared rows of DS_CHUNK tokens at
// a time into shared memory with asynchronous 4-byte copies, DS_STAGES chunks deep: per token the head's k, q and
// decays (dimension sub * R + r at r * L + sub, so that the lanes of a column read neighbouring banks and the
// columns of a warp the same word), the block's values and beta.  Every thread then reads its 3 R numbers of the
// next token from shared memory while this token's sums travel through the shuffles.
#define DS_THREADS 128
#define DS_CHUNK 8
#define DS_STAGES 3

__device__ __forceinline__ void cp_async4s(uint32_t dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void ds_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void ds_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <int L, int R>
struct DeltaScanSmem {
    static constexpr int COLS = DS_THREADS / L;
    static constexpr int DP = L * R;                     // padded key size
    static constexpr int ROW = 3 * DP + COLS + 1;        // k | q | decay | the block's values | beta
    static constexpr size_t BYTES = (size_t)DS_STAGES * DS_CHUNK * ROW * sizeof(float);
};

template <int L, int R>
__global__ void __launch_bounds__(DS_THREADS)
delta_scan_kernel(const float* __restrict__ prep, DeltaShape sh, float* __restrict__ state, int write_state,
                  float* __restrict__ o_out, const int* __restrict__ positions, const int* __restrict__ q_start,
                  const int* __restrict__ slots) {
    using M = DeltaScanSmem<L, R>;
    extern __shared__ __align__(16) float ds_smem[];
    ST_PDL_WAIT();
    const int b = blockIdx.x, h = blockIdx.y;
    const int first = q_start[b], n = q_start[b + 1] - first;
    if (n <= 0 || positions[first] < 0) return;            // padding of a fixed-shape step
    const int H = sh.H, dim = sh.dim, vd = sh.vd;
    const int g = h / (H / sh.G);
    const int sub = threadIdx.x % L;
    const int col0 = blockIdx.z * M::COLS;
    const int col = col0 + threadIdx.x / L;
    const bool live = col < vd;
    const int d0 = sub * R;
    float* S = state + (((size_t)slots[b] * H + h) * dim) * vd + col;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = (live && d0 + r < dim) ? S[(size_t)(d0 + r) * vd] : 0.f;
    const int row_len = sh.row();
    const float* p = prep + (size_t)first * row_len;
    // the padding of the staged rows (dimensions past dim, columns past vd) stays zero: nothing is copied there
    for (int i = threadIdx.x; i < DS_STAGES * DS_CHUNK * M::ROW; i += DS_THREADS) ds_smem[i] = 0.f;
    __syncthreads();
    const int n_chunks = (n + DS_CHUNK - 1) / DS_CHUNK;
    // What this thread copies for every token is fixed for the launch: JN key dimensions (their k, q and decay) and
    // one of the block's values or beta.  The places are worked out once; per token a copy is then an addition.
    constexpr int JN = (M::DP + DS_THREADS - 1) / DS_THREADS;
    int src_k[JN], src_q[JN], src_d[JN];
    uint32_t dst_at[JN];
    const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(ds_smem);
#pragma unroll
    for (int ji = 0; ji < JN; ++ji) {
        const int j = threadIdx.x + ji * DS_THREADS;
        src_k[ji] = j < dim ? sh.pk() + g * dim + j : -1;
        src_q[ji] = sh.pq() + g * dim + j;
        src_d[ji] = sh.pd() + h * dim + j;
        dst_at[ji] = (uint32_t)((j % R) * L + j / R) * 4u;
    }
    int src_x = -1;                                        // the value of one of the block's columns, or beta
    if (threadIdx.x < M::COLS) {
        if (col0 + threadIdx.x < vd) src_x = sh.pv() + h * vd + col0 + threadIdx.x;
    } else if (threadIdx.x == M::COLS) {
        src_x = sh.pb() + h;
    }
    const uint32_t dst_x = (uint32_t)(3 * M::DP + threadIdx.x) * 4u;
    auto stage_chunk = [&](int c) {
        uint32_t dst = smem0 + (uint32_t)((c % DS_STAGES) * DS_CHUNK * M::ROW) * 4u;
        const int t_end = min(DS_CHUNK, n - c * DS_CHUNK);
        const float* row = p + (size_t)(c * DS_CHUNK) * row_len;
#pragma unroll
        for (int t = 0; t < DS_CHUNK; ++t) {
            if (t < t_end) {
#pragma unroll
                for (int ji = 0; ji < JN; ++ji) {
                    if (src_k[ji] >= 0) {
                        cp_async4s(dst + dst_at[ji], row + src_k[ji]);
                        cp_async4s(dst + (uint32_t)M::DP * 4u + dst_at[ji], row + src_q[ji]);
                        cp_async4s(dst + (uint32_t)M::DP * 8u + dst_at[ji], row + src_d[ji]);
                    }
                }
                if (src_x >= 0) cp_async4s(dst + dst_x, row + src_x);
            }
            row += row_len;
            dst += (uint32_t)M::ROW * 4u;
        }
    };
#pragma unroll
    for (int c = 0; c < DS_STAGES - 1; ++c) {
        if (c < n_chunks) stage_chunk(c);
        ds_commit();
    }
    float* o_at = o_out + (size_t)first * H * vd + h * vd + col;
    const size_t o_step = (size_t)H * vd;
    const bool writes_o = live && sub == 0;
    float kq[R], qq[R], dd[R], v, beta;
    auto fetch = [&](const float* row) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            kq[r] = row[r * L + sub];
            qq[r] = row[M::DP + r * L + sub];
            dd[r] = row[2 * M::DP + r * L + sub];
        }
        v = row[3 * M::DP + threadIdx.x / L];
        beta = row[3 * M::DP + M::COLS];
    };
    for (int c = 0; c < n_chunks; ++c) {
        ds_wait<DS_STAGES - 2>();           // chunk c has landed (this thread's copies; the barrier makes it all threads')
        __syncthreads();                    // also: every thread is done with chunk c - 1, whose stage is filled next
        if (c + DS_STAGES - 1 < n_chunks) stage_chunk(c + DS_STAGES - 1);
        ds_commit();
        const float* rows = ds_smem + (size_t)(c % DS_STAGES) * DS_CHUNK * M::ROW;
        const int t_end = min(DS_CHUNK, n - c * DS_CHUNK);
        fetch(rows);
        for (int t = 0; t < t_end; ++t) {
            float k_[R];
            // partial sums in four lanes of arithmetic, so that the chain of additions is R / 4 long
            float sk4[4] = {0.f, 0.f, 0.f, 0.f}, sq4[4] = {0.f, 0.f, 0.f, 0.f}, kq4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < R; ++r) {
                k_[r] = kq[r];
                s[r] *= dd[r];
                sk4[r & 3] = fmaf(s[r], k_[r], sk4[r & 3]);
                sq4[r & 3] = fmaf(s[r], qq[r], sq4[r & 3]);
                kq4[r & 3] = fmaf(k_[r], qq[r], kq4[r & 3]);
            }
            float sk = (sk4[0] + sk4[1]) + (sk4[2] + sk4[3]);
            float sq = (sq4[0] + sq4[1]) + (sq4[2] + sq4[3]);
            float kdq = (kq4[0] + kq4[1]) + (kq4[2] + kq4[3]);
            const float v_now = v, beta_now = beta;
            if (t + 1 < t_end) fetch(rows + (t + 1) * M::ROW);      // the next token's numbers are on their way meanwhile
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) {
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
                kdq += __shfl_xor_sync(0xffffffffu, kdq, o);
            }
            const float u = beta_now * (v_now - sk);
#pragma unroll
            for (int r = 0; r < R; ++r) s[r] = fmaf(k_[r], u, s[r]);
            if (writes_o) *o_at = fmaf(u, kdq, sq);
            o_at += o_step;
        }
    }
    // The successor's blocks are let in only now: while they wait for this grid on the same multiprocessors, the
    // walk over a long portion was measured to take nearly twice as long.
    ST_PDL_TRIGGER();
    ds_wait<0>();
    if (write_state && live) {
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (d0 + r < dim) S[(size_t)(d0 + r) * vd] = s[r];
    }
}

// out[t, h, e] = out_scale * o / sqrt(mean_e o^2 + eps) * norm_w[e] * sigmoid(sum_r g1[t, r] * W_g2[h * vd + e, r])
template <typename T>
__global__ void __launch_bounds__(128)
delta_output_kernel(const float* __restrict__ o, const float* __restrict__ proj, int ld, DeltaShape sh,
                    const T* __restrict__ w_g2, const float* __restrict__ norm_w, float eps, float out_scale,
                    T* __restrict__ out, const int* __restrict__ positions) {
    __shared__ float scratch[32];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x, h = blockIdx.y;
    if (positions[t] < 0) return;
    const int vd = sh.vd;
    const float* orow = o + ((size_t)t * sh.H + h) * vd;
    float ss = 0.f;
    for (int e = threadIdx.x; e < vd; e += blockDim.x) {
        const float x = __ldcg(orow + e);
        ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)vd + eps) * out_scale;
    __shared__ float xs_g[DR_RANK_SMEM];
    const float* g1 = proj + (size_t)t * ld + sh.g_off;
    if (sh.rank_g > 0 && sh.rank_g <= DR_RANK_SMEM) {
        for (int r = threadIdx.x; r < sh.rank_g; r += blockDim.x) xs_g[r] = __ldcg(g1 + r);
        __syncthreads();
        g1 = xs_g;
    }
    for (int e = threadIdx.x; e < vd; e += blockDim.x) {
        const float z = sh.rank_g > 0 ? lowrank_dot(g1, w_g2 + (size_t)(h * vd + e) * sh.rank_g, sh.rank_g)
                                      : __ldcg(g1 + h * vd + e);
        const float gate = (sh.gate_silu ? z : 1.f) / (1.f + expf(-z));
        out[((size_t)t * sh.H + h) * vd + e] = from_f32<T>(__ldcg(orow + e) * inv * norm_w[e] * gate);
    }
}

// 0: the launcher chooses the lanes per column of the recurrence; 8 or 16: this many (for tests and tuning).
static int ds_forced_lanes = 0;
ST_EXPORT int st_delta_rule_set_lanes(int lanes) {
    if (lanes != 0 && lanes != 8 && lanes != 16) return ST_ERR_BAD_ARG;
    ds_forced_lanes = lanes;
    return 0;
}
ST_EXPORT long long st_delta_rule_scratch_floats(int n_tokens, int H, int G, int dim, int vd) {
    return (long long)n_tokens * ((long long)2 * G * dim + (long long)H * vd + (long long)H * dim + H + (long long)H * vd);
}

// proj: float [n_tokens, ld]; w_a2 [H*dim, rank_a], w_g2 [H*vd, rank_g] in the storage type `dtype`, as is out
// [n_tokens, H*vd]; conv_state float [slots, taps-1, 2*G*dim + H*vd]; state float [slots, H, dim, vd];
// scratch: float, st_delta_rule_scratch_floats elements.  write_state == 0: the states are read, not moved on.
ST_EXPORT int st_delta_rule(const float* proj, int ld, int q_off, int b_off, int a_off, int g_off, int rank_a,
                            int rank_g, const float* conv_w, int taps, float* conv_state, const void* w_a2,
                            const float* a_log, const float* dt_bias, const void* w_g2, const float* norm_w, float eps,
                            float out_scale, float* state, int write_state, int single_tokens, float* scratch,
                            void* out, const int* positions, const int* seq_of_token, const int* q_start,
                            const int* slots, int n_tokens, int n_seqs, int H, int G, int dim, int vd, int dtype,
                            void* stream, int gate_silu) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || dim <= 0 || vd <= 0 || taps < 1 || rank_a < 0 || rank_g < 0) return ST_ERR_BAD_ARG;
    if (taps > DR_MAX_TAPS || dim > 32 * DR_UNIT_PASSES || vd > 32 * DR_UNIT_PASSES) return ST_ERR_TOO_LARGE;
    if (dtype != 0 && dtype != 1) return ST_ERR_BAD_DTYPE;
    DeltaShape sh;
    sh.H = H; sh.G = G; sh.dim = dim; sh.vd = vd;
    sh.q_off = q_off; sh.k_off = q_off + G * dim; sh.v_off = q_off + 2 * G * dim;
    sh.b_off = b_off; sh.a_off = a_off; sh.g_off = g_off; sh.rank_a = rank_a; sh.rank_g = rank_g; sh.gate_silu = gate_silu;
    cudaStream_t s = (cudaStream_t)stream;
    float* prep = scratch;
    float* o = scratch + (size_t)n_tokens * sh.row();
    const int move = single_tokens && write_state && taps > 1;
    int rc;
    {
        const int units = 2 * G + H;
        int gy = (units + 7) / 8;
        if (gy > 16) gy = 16;
        dim3 grid(n_tokens, gy);
        if (dtype == 0)
            rc = st_launch_pdl("delta_prepare", delta_prepare_kernel<float>, grid, dim3(DR_PREP_THREADS), 0, s, proj, ld, sh,
                               conv_w, conv_state, move, taps, (const float*)w_a2, a_log, dt_bias, prep, positions,
                               seq_of_token, q_start, slots);
        else
            rc = st_launch_pdl("delta_prepare", delta_prepare_kernel<bf16>, grid, dim3(DR_PREP_THREADS), 0, s, proj, ld, sh,
                               conv_w, conv_state, move, taps, (const bf16*)w_a2, a_log, dt_bias, prep, positions,
                               seq_of_token, q_start, slots);
        if (rc) return rc;
    }
    {
#define DS_LAUNCH(L, R)                                                                                              \
    do {                                                                                                             \
        const size_t smem = DeltaScanSmem<L, R>::BYTES;                                                              \
        if (smem > 48 * 1024) {                                                                                      \
            cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<L, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                                         \
            if (e != cudaSuccess) return (int)e;                                                                     \
        }                                                                                                            \
        rc = st_launch_pdl("delta_scan", delta_scan_kernel<L, R>,                                                    \
                           dim3(n_seqs, H, (vd + DS_THREADS / L - 1) / (DS_THREADS / L)), dim3(DS_THREADS), smem, s, \
                           (const float*)prep, sh, state, write_state, o, positions, q_start, slots);                \
    } while (0)
        // Lanes per column.  A token's step is a chain of dependent instructions, so a launch is as fast as its
        // blocks are spread: when eight lanes per column give fewer blocks than the device has multiprocessors,
        // sixteen (fewer rows each, one more stage of shuffles) were measured faster, by a fifth for one request of
        // eight heads; for short columns (dim <= 32) and for steps of many requests eight are.  Thirty-two lanes
        // were measured too and never won.
        int lanes = ds_forced_lanes;
        if (!lanes) {
            const long long cols8 = (vd + DS_THREADS / 8 - 1) / (DS_THREADS / 8);
            lanes = (dim > 32 && (long long)n_seqs * H * cols8 < st_sm_count()) ? 16 : 8;
        }
        if (dim > 128) lanes = 16;
        if (lanes == 8) {
            if (dim <= 32) DS_LAUNCH(8, 4);
            else if (dim <= 64) DS_LAUNCH(8, 8);
            else DS_LAUNCH(8, 16);
        } else {
            if (dim <= 32) DS_LAUNCH(16, 2);
            else if (dim <= 64) DS_LAUNCH(16, 4);
            else if (dim <= 128) DS_LAUNCH(16, 8);
            else DS_LAUNCH(16, 16);
        }
#undef DS_LAUNCH
        if (rc) return rc;
    }
    dim3 grid(n_tokens, H);
    if (dtype == 0)
        return st_launch_pdl("delta_output", delta_output_kernel<float>, grid, dim3(128), 0, s, (const float*)o, proj, ld, sh,
                             (const float*)w_g2, norm_w, eps, out_scale, (float*)out, positions);
    return st_launch_pdl("delta_output", delta_output_kernel<bf16>, grid, dim3(128), 0, s, (const float*)o, proj, ld, sh,
                         (const bf16*)w_g2, norm_w, eps, out_scale, (bf16*)out, positions);
}

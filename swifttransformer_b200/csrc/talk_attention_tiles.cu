// Attention with weights mixed over the heads (talk_attention.cu) for prompt portions on the warp-level tensor
// cores (mma.sync m16n8k16, bfloat16 in, float accumulate): one block per 16 query rows of one request, all heads.
//
// The mixing needs every head's normalised weight of a (query, key) pair in one place, and a head's result needs
// room of its own: sixteen rows x all heads x vd floats is what the registers of one block hold.  So a block takes
// sixteen rows; its eight warps share the heads (warp w owns heads w, w + 8, ...: their queries, maxima, sums and
// results), and every key tile (32 keys of every key/value head, two stages of 16-byte asynchronous copies) is
// used by all of them.  The keys are walked twice:
//
//   first   S = Q K^T per owned head, the running maximum and sum; then the extra term joins the sum;
//   second  S again (the same products in the same order), P = exp2(S - m) / l, written to shared memory in the
//           layout of the product's accumulator (a lane's sixteen numbers of a head side by side); after a barrier
//           every warp forms P'_a = sum_b T[a][b] P_b for its heads, element by element in that same layout, in
//           float, packs it as the next product's row operand and adds P'_a V of its head's own key/value head.
//
// Mask, gate and extra term as in talk_attention.cu / gqa_attention.cuh.  Sizes are template arguments rounded up
// (dim and vd to 32/64/128) with the padding columns zero in shared memory; dim and vd themselves must be multiples
// of 8.  Scores, the softmax and the mixing are float; the exponentials use the fast exp2.
#include "gqa_attention.cuh"
#include "mma_sync.cuh"

#define TT_ROWS 16
#define TT_KEYS 32
#define TT_MAX_THREADS 512

template <int DIMT, int VDT>
struct TalkTileSmem {
    static constexpr int K_LD = DIMT + 8;
    static constexpr int V_LD = VDT + 8;
    __host__ __device__ static size_t stage_elems(int nkv) { return (size_t)nkv * TT_KEYS * (K_LD + V_LD); }
    static size_t bytes(int nh, int nkv) {
        return 2 * stage_elems(nkv) * sizeof(bf16) + ((size_t)nh * TT_KEYS * TT_ROWS + (size_t)nh * nh) * sizeof(float);
    }
};

// keys key0 .. key0 + 31 of every key/value head into a stage: keys [nkv][32][K_LD], then the block's part of the
// values (columns e0 .. e0 + vd_block - 1 of every row) [nkv][32][V_LD]
template <int DIMT, int VDT, int THREADS>
__device__ __forceinline__ void talk_load_kv_tile(bf16* stage, const bf16* __restrict__ pool, const DiffCache& cache,
                                                  const int* __restrict__ bt, int key0, int lo, int hi, int keep_first,
                                                  int e0, int vd_block, int* __restrict__ status) {
    using L = TalkTileSmem<DIMT, VDT>;
    constexpr int KC = DIMT / 8, VC = VDT / 8;
    const int nkv = cache.nkv, dim = cache.kd, ps = cache.page_size;
    bf16* sk = stage;
    bf16* sv = stage + (size_t)nkv * TT_KEYS * L::K_LD;
    // THREADS / 32 threads per key: one look-up of its page, then the pieces of its rows in every key/value head
    constexpr int PER = THREADS / TT_KEYS;
    const int row = threadIdx.x / PER, sub = threadIdx.x % PER;
    const int key = key0 + row;
    int page = -1;
    if (key <= hi && (key >= lo || key < keep_first)) {
        page = bt[key / ps];
        if (page < 0 && status) *status = 1;
    }
    const int pip = key % ps;
    for (int c = sub; c < nkv * (KC + VC); c += PER) {
        const int kvh = c / (KC + VC), p = c % (KC + VC);
        if (p < KC) {
            const int e = p * 8;
            bf16* dst = sk + ((size_t)kvh * TT_KEYS + row) * L::K_LD + e;
            if (page >= 0 && e < dim) cp_async16(dst, cache_keys(pool, cache, page, kvh, pip) + e, true);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        } else {
            const int e = (p - KC) * 8;
            bf16* dst = sv + ((size_t)kvh * TT_KEYS + row) * L::V_LD + e;
            if (page >= 0 && e < vd_block) cp_async16(dst, cache_values(pool, cache, page, kvh, pip) + e0 + e, true);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
}

template <int DIMT, int VDT, int HPW, int TT_WARPS>
__global__ void __launch_bounds__(TT_WARPS * 32)
talk_attention_tiles_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, DiffCache cache,
                            bf16* __restrict__ out, const int* __restrict__ tiles, int parts,
                            const int* __restrict__ q_start, const int* __restrict__ start_pos,
                            const int* __restrict__ slots, const int* __restrict__ block_table, int nh, float scale,
                            GqaMask mask, const float* __restrict__ talk, int has_sink, GqaEpilogue epi, int gate_heads,
                            int* __restrict__ status) {
    using L = TalkTileSmem<DIMT, VDT>;
    constexpr int TT_THREADS = TT_WARPS * 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int nkv = cache.nkv, vd = cache.vd, dim = cache.kd;
    bf16* stages = reinterpret_cast<bf16*>(smem_raw);
    const size_t stage_elems = L::stage_elems(nkv);
    float* sp = reinterpret_cast<float*>(stages + 2 * stage_elems);      // [nh][4 n-tiles][32 lanes][4]
    float* st = sp + (size_t)nh * TT_KEYS * TT_ROWS;                      // [nh][nh]
    for (int i = threadIdx.x; i < nh * nh; i += TT_THREADS) st[i] = talk ? talk[i] : (i / nh == i % nh ? 1.f : 0.f);
    ST_PDL_TRIGGER();
    const int tile = blockIdx.x / parts, part = blockIdx.x % parts;
    const int req = tiles[2 * tile], off = tiles[2 * tile + 1] + part * TT_ROWS;
    const int first = q_start[req], n_new = q_start[req + 1] - first;
    if (off >= n_new) return;
    const int rep = nh / nkv;
    // the value columns this block serves: a model whose heads x vd do not fit one block's registers is served by
    // gridDim.y blocks per sixteen rows, each with all the scores and weights and a part of every value row
    const int vd_block = vd / gridDim.y, e0 = blockIdx.y * vd_block;
    const int start = start_pos[req];
    const int* bt = block_table + (size_t)slots[req] * cache.max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int rows_here = min(TT_ROWS, n_new - off);
    const int p_first = start + off, hi = p_first + rows_here - 1;
    const int lo = gqa_lo(p_first, mask);
    const int keep = mask.window > 0 ? mask.keep_first : 0;
    int pos[2];
    bool live[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        live[r] = g + 8 * r < rows_here;
        pos[r] = p_first + g + 8 * r;
    }
    // the queries of this warp's heads (head warp + 8 i), as row operands
    uint32_t qa[HPW][DIMT / 16][4];
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = warp + TT_WARPS * i;
#pragma unroll
        for (int ks = 0; ks < DIMT / 16; ++ks)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int r = x & 1, col = ks * 16 + 2 * tq + 8 * (x >> 1);
                uint32_t v = 0;
                if (h < nh && live[r] && col < dim)
                    v = __ldcg(reinterpret_cast<const uint32_t*>(q + ((size_t)(first + off + g + 8 * r) * nh + h) * dim + col));
                qa[i][ks][x] = v;
            }
    }
    const float LOG2E = 1.4426950408889634f;
    const float scale_l2 = scale * LOG2E;
    float m[HPW][2], l[HPW][2];
#pragma unroll
    for (int i = 0; i < HPW; ++i) { m[i][0] = m[i][1] = -INFINITY; l[i][0] = l[i][1] = 0.f; }

    const int k_b = lo / TT_KEYS, kt_last = hi / TT_KEYS;
    const int head_end = min(keep, lo);
    const int n_a = min((head_end + TT_KEYS - 1) / TT_KEYS, k_b);
    const int n_t = n_a + kt_last - k_b + 1;
#define TT_TILE(i) ((i) < n_a ? (i) : k_b + (i) - n_a)

    // S of head (warp + 8 i) for the stage's 32 keys, masked, in units of log2(e)
    auto scores = [&](const bf16* stage, int i, int key0, bool inside, float (&s)[TT_KEYS / 8][4]) {
        const int h = warp + TT_WARPS * i;
        const bf16* sk = stage + (size_t)(h / rep) * TT_KEYS * L::K_LD;
#pragma unroll
        for (int nt = 0; nt < TT_KEYS / 8; ++nt) {
#pragma unroll
            for (int x = 0; x < 4; ++x) s[nt][x] = 0.f;
            // the column operand of two steps of k at once: four 8 x 8 pieces of the tile's rows nt * 8 .. + 7
#pragma unroll
            for (int ks = 0; ks < DIMT / 16; ks += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, sk + (nt * 8 + (lane & 7)) * L::K_LD + ks * 16 + (lane >> 3) * 8);
                mma_bf16(s[nt], qa[i][ks], b0, b1);
                mma_bf16(s[nt], qa[i][ks + 1], b2, b3);
            }
            if (inside) {
#pragma unroll
                for (int x = 0; x < 4; ++x) s[nt][x] *= scale_l2;
            } else {
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int r = x >> 1, key = key0 + nt * 8 + 2 * tq + (x & 1);
                    s[nt][x] = (live[r] && gqa_seen(key, pos[r], mask)) ? s[nt][x] * scale_l2 : -INFINITY;
                }
            }
        }
    };
    // a tile that every one of the block's sixteen rows sees whole takes no mask
    const int lo_last = gqa_lo(p_first + TT_ROWS - 1, mask);
    auto whole = [&](int key0) {
        return rows_here == TT_ROWS && key0 + TT_KEYS - 1 <= p_first &&
               (mask.window <= 0 || key0 >= lo_last || key0 + TT_KEYS <= keep);
    };

    // ---- first walk: maxima and sums.  One barrier per tile: behind it the tile has landed for every thread and
    // every warp is done with the tile before, whose stage the copies of the next tile may then fill.
    talk_load_kv_tile<DIMT, VDT, TT_THREADS>(stages, pool, cache, bt, TT_TILE(0) * TT_KEYS, lo, hi, keep, e0, vd_block, status);
    cp_async_commit();
    for (int t = 0; t < n_t; ++t) {
        const bf16* stage = stages + (t & 1) * stage_elems;
        cp_async_wait<0>();
        __syncthreads();
        // behind the last tile of this walk the first tile of the second walk is already asked for
        const int nxt = t + 1 < n_t ? t + 1 : 0;
        talk_load_kv_tile<DIMT, VDT, TT_THREADS>(stages + ((t + 1) & 1) * stage_elems, pool, cache, bt, TT_TILE(nxt) * TT_KEYS, lo, hi,
                                     keep, e0, vd_block, status);
        cp_async_commit();
        const int key0 = TT_TILE(t) * TT_KEYS;
        const bool inside = whole(key0);
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            if (warp + TT_WARPS * i >= nh) continue;
            float s[TT_KEYS / 8][4];
            scores(stage, i, key0, inside, s);
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < TT_KEYS / 8; ++nt)
#pragma unroll
                for (int x = 0; x < 4; ++x) tmax[x >> 1] = fmaxf(tmax[x >> 1], s[nt][x]);
            float tsum[2] = {0.f, 0.f}, m_new[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
                m_new[r] = fmaxf(m[i][r], tmax[r]);
            }
#pragma unroll
            for (int nt = 0; nt < TT_KEYS / 8; ++nt)
#pragma unroll
                for (int x = 0; x < 4; ++x)
                    if (s[nt][x] > -INFINITY) tsum[x >> 1] += fast_exp2(s[nt][x] - m_new[x >> 1]);
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tsum[r] += __shfl_xor_sync(0xffffffffu, tsum[r], 1);
                tsum[r] += __shfl_xor_sync(0xffffffffu, tsum[r], 2);
                l[i][r] = (m[i][r] == -INFINITY ? 0.f : l[i][r] * fast_exp2(m[i][r] - m_new[r])) + tsum[r];
                m[i][r] = m_new[r];
            }
        }
    }
    // the extra term; from here on l holds 1 / denominator
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = warp + TT_WARPS * i;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float ll = l[i][r];
            if (has_sink && h < nh) {
                const float s_l2 = epi.sinks[h] * LOG2E;
                const float m_new = fmaxf(m[i][r], s_l2);
                ll = (m[i][r] == -INFINITY ? 0.f : ll * fast_exp2(m[i][r] - m_new)) + fast_exp2(s_l2 - m_new);
                m[i][r] = m_new;
            }
            l[i][r] = ll > 0.f ? 1.f / ll : 0.f;
        }
    }

    // ---- second walk: weights, mixed, times the values
    float o[HPW][VDT / 8][4];
#pragma unroll
    for (int i = 0; i < HPW; ++i)
#pragma unroll
        for (int nt = 0; nt < VDT / 8; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x) o[i][nt][x] = 0.f;
    // (tile 0 of this walk is on its way into stage n_t & 1: the stages go on in turn)
    for (int t = 0; t < n_t; ++t) {
        const int u = n_t + t;
        const bf16* stage = stages + (u & 1) * stage_elems;
        cp_async_wait<0>();
        __syncthreads();            // the tile has landed; every warp is done with the tile before and its weights
        if (t + 1 < n_t)
            talk_load_kv_tile<DIMT, VDT, TT_THREADS>(stages + ((u + 1) & 1) * stage_elems, pool, cache, bt, TT_TILE(t + 1) * TT_KEYS, lo,
                                         hi, keep, e0, vd_block, status);
        cp_async_commit();
        const int key0 = TT_TILE(t) * TT_KEYS;
        const bool inside = whole(key0);
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int h = warp + TT_WARPS * i;
            if (h >= nh) continue;
            float s[TT_KEYS / 8][4];
            scores(stage, i, key0, inside, s);
#pragma unroll
            for (int nt = 0; nt < TT_KEYS / 8; ++nt) {
                float4 p;
                p.x = s[nt][0] > -INFINITY ? fast_exp2(s[nt][0] - m[i][0]) * l[i][0] : 0.f;
                p.y = s[nt][1] > -INFINITY ? fast_exp2(s[nt][1] - m[i][0]) * l[i][0] : 0.f;
                p.z = s[nt][2] > -INFINITY ? fast_exp2(s[nt][2] - m[i][1]) * l[i][1] : 0.f;
                p.w = s[nt][3] > -INFINITY ? fast_exp2(s[nt][3] - m[i][1]) * l[i][1] : 0.f;
                *reinterpret_cast<float4*>(sp + (((size_t)h * (TT_KEYS / 8) + nt) * 32 + lane) * 4) = p;
            }
        }
        __syncthreads();
        const bf16* sv_all = stage + (size_t)nkv * TT_KEYS * L::K_LD;
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int h = warp + TT_WARPS * i;
            if (h >= nh) continue;
            float4 w[TT_KEYS / 8];
#pragma unroll
            for (int nt = 0; nt < TT_KEYS / 8; ++nt) w[nt] = make_float4(0.f, 0.f, 0.f, 0.f);
            const float* trow = st + (size_t)h * nh;
            for (int b = 0; b < nh; ++b) {
                const float c = trow[b];
#pragma unroll
                for (int nt = 0; nt < TT_KEYS / 8; ++nt) {
                    const float4 p = *reinterpret_cast<const float4*>(sp + (((size_t)b * (TT_KEYS / 8) + nt) * 32 + lane) * 4);
                    w[nt].x = fmaf(c, p.x, w[nt].x); w[nt].y = fmaf(c, p.y, w[nt].y);
                    w[nt].z = fmaf(c, p.z, w[nt].z); w[nt].w = fmaf(c, p.w, w[nt].w);
                }
            }
            uint32_t pa[TT_KEYS / 16][4];
#pragma unroll
            for (int nt = 0; nt < TT_KEYS / 8; ++nt) {
                pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(w[nt].x, w[nt].y);
                pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(w[nt].z, w[nt].w);
            }
            const bf16* sv = sv_all + (size_t)(h / rep) * TT_KEYS * L::V_LD;
#pragma unroll
            for (int ks = 0; ks < TT_KEYS / 16; ++ks)
#pragma unroll
                for (int nt2 = 0; nt2 < VDT / 16; ++nt2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, sv + (ks * 16 + (lane & 15)) * L::V_LD + nt2 * 16 + (lane >> 4) * 8);
                    mma_bf16(o[i][2 * nt2], pa[ks], b0, b1);
                    mma_bf16(o[i][2 * nt2 + 1], pa[ks], b2, b3);
                }
        }
    }
#undef TT_TILE
    cp_async_wait<0>();
    const bf16* gate = reinterpret_cast<const bf16*>(epi.gate);
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = warp + TT_WARPS * i;
        if (h >= nh) continue;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (!live[r]) continue;
            const size_t t = (size_t)(first + off + g + 8 * r);
            bf16* orow = out + (t * nh + h) * vd + e0;
            float gh = epi.out_scale;
            if (gate && gate_heads) gh *= sigmoidf_(to_f32(gate[t * epi.gate_ld + h]));
            const bf16* grow = (gate && !gate_heads) ? gate + t * epi.gate_ld + (size_t)h * vd + e0 : nullptr;
#pragma unroll
            for (int nt = 0; nt < VDT / 8; ++nt) {
                const int e = nt * 8 + 2 * tq;
                if (e >= vd_block) continue;
                float a = o[i][nt][2 * r] * gh, b = o[i][nt][2 * r + 1] * gh;
                if (grow) {
                    a *= sigmoidf_(to_f32(grow[e]));
                    b *= sigmoidf_(to_f32(grow[e + 1]));
                }
                *reinterpret_cast<uint32_t*>(orow + e) = pack_bf16(a, b);
            }
        }
    }
}

static int talk_round(int n) { return n <= 32 ? 32 : (n <= 64 ? 64 : 128); }

// How a model's heads are laid over a block: blocks per sixteen rows (each with a part of every value row), warps per
// block, heads per warp.  Sixteen warps when the registers of 512 threads hold a warp's heads (its sums are heads x
// vd / 2 floats per lane): four warps per scheduler hide one another's waits (measured: a fifth faster than eight
// warps with two heads each); else eight warps with up to four heads each; else the value rows are cut in two or four.
#define TT_SMEM_LIMIT (224 * 1024)
static bool talk_split(int nh, int nkv, int dim, int vd, int* v_parts, int* warps, int* hpw) {
    const int dimt = talk_round(dim);
    for (int parts = 1; parts <= 4; parts *= 2) {
        if (vd % (8 * parts)) break;
        const int vdt = talk_round(vd / parts);
        const size_t smem = 2 * (size_t)nkv * TT_KEYS * (dimt + 8 + vdt + 8) * sizeof(bf16) +
                            ((size_t)nh * TT_KEYS * TT_ROWS + (size_t)nh * nh) * sizeof(float);
        if (smem > TT_SMEM_LIMIT) continue;
        const int h16 = (nh + 15) / 16, h8 = (nh + 7) / 8;
        if (h16 <= 2 && h16 * vdt <= 128 && h16 * dimt <= 128) { *v_parts = parts; *warps = 16; *hpw = h16; return true; }
        const int h8t = h8 <= 2 ? h8 : 4;
        if (h8 <= 4 && h8t * vdt <= 256 && h8t * dimt <= 256) { *v_parts = parts; *warps = 8; *hpw = h8t; return true; }
    }
    return false;
}

// bfloat16; dim and vd multiples of 8 up to 128; the heads within the registers of one block (with the value rows cut in
// up to four parts), the stages and the weights within shared memory
ST_EXPORT int st_talk_attention_tiles_applies(int nh, int nkv, int dim, int vd) {
    if (nh <= 0 || nkv <= 0 || nh % nkv || dim <= 0 || vd <= 0 || dim % 8 || vd % 8 || dim > 128 || vd > 128) return 0;
    int v_parts, warps, hpw;
    return talk_split(nh, nkv, dim, vd, &v_parts, &warps, &hpw) ? 1 : 0;
}

template <int DIMT, int VDT, int HPW, int WARPS>
static int launch_talk_tiles(const void* q, const void* pool, const DiffCache& c, void* out, const int* tiles, int n_tiles,
                             int tile_rows, const int* q_start, const int* start_pos, const int* slots,
                             const int* block_table, int nh, float scale, const GqaMask& mask, const float* talk,
                             int has_sink, const GqaEpilogue& epi, int gate_heads, int v_parts, int* status,
                             cudaStream_t s) {
    if constexpr (HPW * VDT > 256 || HPW * DIMT > 256 || (WARPS == 16 && (HPW > 2 || HPW * VDT > 128 || HPW * DIMT > 128))) {
        return ST_ERR_BAD_SIZE;
    } else {
        const size_t smem = TalkTileSmem<DIMT, VDT>::bytes(nh, c.nkv);
        if (smem > TT_SMEM_LIMIT) return ST_ERR_TOO_LARGE;
        auto kern = talk_attention_tiles_kernel<DIMT, VDT, HPW, WARPS>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        const int parts = (tile_rows + TT_ROWS - 1) / TT_ROWS;
        kern<<<dim3(n_tiles * parts, v_parts), WARPS * 32, smem, s>>>((const bf16*)q, (const bf16*)pool, c, (bf16*)out, tiles, parts,
                                                            q_start, start_pos, slots, block_table, nh, scale, mask, talk,
                                                            has_sink, epi, gate_heads, status);
        return st_launch_status();
    }
}

// tiles: int32 [n_tiles][2] = (request of the step, offset of the tile among its new tokens), tile_rows rows each;
// a tile whose offset lies past the request's tokens is padding.  gate: bfloat16 logits or null.
ST_EXPORT int st_talk_attention_tiles(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                      void* out, const int* tiles, int n_tiles, int tile_rows, const int* q_start,
                                      const int* start_pos, const int* slots, const int* block_table, int max_pages,
                                      int nh, int nkv, int dim, int vd, int page_size, float scale, int window,
                                      int keep_first, const float* talk, const float* sinks, const void* gate,
                                      long long gate_ld, int gate_heads, float out_scale, int* status, void* stream) {
    if (n_tiles <= 0) return 0;
    if (page_size <= 0 || keep_first < 0 || tile_rows <= 0 || tile_rows % TT_ROWS) return ST_ERR_BAD_ARG;
    if (!st_talk_attention_tiles_applies(nh, nkv, dim, vd)) return ST_ERR_BAD_SIZE;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const GqaMask mask = {window, keep_first};
    const GqaEpilogue epi = {gate, gate_ld, out_scale, sinks};
    cudaStream_t s = (cudaStream_t)stream;
    int v_parts, warps, hpw;
    if (!talk_split(nh, nkv, dim, vd, &v_parts, &warps, &hpw)) return ST_ERR_BAD_SIZE;
    const int dimt = talk_round(dim), vdt = talk_round(vd / v_parts);
#define TT_ARGS q, pool, c, out, tiles, n_tiles, tile_rows, q_start, start_pos, slots, block_table, nh, scale, mask, talk, \
                sinks != nullptr, epi, gate_heads, v_parts, status, s
#define TT_BY_HEADS(D, V)                                                          \
    do {                                                                           \
        if (warps == 16 && hpw == 1) return launch_talk_tiles<D, V, 1, 16>(TT_ARGS); \
        if (warps == 16) return launch_talk_tiles<D, V, 2, 16>(TT_ARGS);           \
        if (hpw == 1) return launch_talk_tiles<D, V, 1, 8>(TT_ARGS);               \
        if (hpw == 2) return launch_talk_tiles<D, V, 2, 8>(TT_ARGS);               \
        return launch_talk_tiles<D, V, 4, 8>(TT_ARGS);                             \
    } while (0)
#define TT_BY_V(D)                            \
    do {                                      \
        if (vdt == 32) TT_BY_HEADS(D, 32);    \
        if (vdt == 64) TT_BY_HEADS(D, 64);    \
        TT_BY_HEADS(D, 128);                  \
    } while (0)
    if (dimt == 32) TT_BY_V(32);
    if (dimt == 64) TT_BY_V(64);
    TT_BY_V(128);
#undef TT_BY_V
#undef TT_BY_HEADS
#undef TT_ARGS
}

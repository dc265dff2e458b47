// Grouped-query attention for prompt portions on the warp-level tensor cores (mma.sync m16n8k16, bfloat16 in,
// float accumulate): one block per (128 query rows of one request, query head).
//
// Eight warps carry sixteen query rows each.  All read the same key tile (64 keys) and value tile from shared
// memory, filled by 16-byte asynchronous copies from the pages (two stages: the next tile lands while this one
// is multiplied).  Each warp keeps S = Q K^T, the running maximum and sum and O = P V (16 x vd) in registers.
//
// Mask (gqa_attention.cuh): with a window the keys a block reads are two runs of tiles, those that hold the kept
// first keys of the request and those from the window of the block's first row up to its last row; the tiles
// between them are never touched (their pages may be gone).  A tile wholly inside the range of every row of a
// warp takes no mask.  The softmax's extra term joins the sum once, after the last tile.  The head's result is
// multiplied by out_scale and, with a gate, by sigmoid(gate logit) when it is stored.
//
// Sizes are template arguments rounded up (dim to 32/64/96/128, vd to 32/64/96/128/256) with the padding columns
// zero in shared memory; dim and vd themselves must be multiples of 8 (16-byte pieces).  Scores and the softmax
// are float; the weights' exponentials use the fast exp2.
#include "gqa_attention.cuh"
#include "mma_sync.cuh"

#define GT_ROWS 128     // query rows per block
#define GT_KEYS 64      // keys per tile
#define GT_THREADS 256

template <int DIMT, int VDT>
struct GqaTileSmem {
    static constexpr int K_LD = DIMT + 8;       // elements per key row, padded against bank conflicts
    static constexpr int V_LD = VDT + 8;
    static constexpr int STAGE = GT_KEYS * (K_LD + V_LD);
    static constexpr size_t BYTES = 2 * (size_t)STAGE * sizeof(bf16);
};

// keys key0 .. key0 + 63 of kv head kvh into a stage; a key the block's rows do not see (past `hi`, or between
// the kept first keys and `lo`) is zeros and its page is not looked up
template <int DIMT, int VDT>
__device__ __forceinline__ void gqa_load_kv_tile(bf16* stage, const bf16* __restrict__ pool, const DiffCache& cache,
                                                 const int* __restrict__ bt, int kvh, int key0, int lo, int hi,
                                                 int keep_first, int* __restrict__ status) {
    using L = GqaTileSmem<DIMT, VDT>;
    bf16* sk = stage;
    bf16* sv = stage + GT_KEYS * L::K_LD;
    constexpr int KC = DIMT / 8, VC = VDT / 8;      // 16-byte pieces per row
    const int dim = cache.kd, vd = cache.vd, ps = cache.page_size;
    // four threads per key row: one look-up of the row's page, then the row's pieces in turn
    const int row = threadIdx.x >> 2;
    const int key = key0 + row;
    int page = -1;
    if (key <= hi && (key >= lo || key < keep_first)) {
        page = bt[key / ps];
        if (page < 0 && status) *status = 1;            // a hole in the block table: the key counts as zeros
    }
    const bf16* krow = page >= 0 ? cache_keys(pool, cache, page, kvh, key % ps) : nullptr;
    const bf16* vrow = page >= 0 ? cache_values(pool, cache, page, kvh, key % ps) : nullptr;
    for (int c = threadIdx.x & 3; c < KC + VC; c += 4) {
        if (c < KC) {
            const int e = c * 8;
            bf16* dst = sk + row * L::K_LD + e;
            if (page >= 0 && e < dim) cp_async16(dst, krow + e, true);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        } else {
            const int e = (c - KC) * 8;
            bf16* dst = sv + row * L::V_LD + e;
            if (page >= 0 && e < vd) cp_async16(dst, vrow + e, true);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
}

template <int DIMT, int VDT>
__global__ void __launch_bounds__(GT_THREADS)
gqa_attention_tiles_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, DiffCache cache,
                           bf16* __restrict__ out, const int* __restrict__ tiles, int parts,
                           const int* __restrict__ q_start, const int* __restrict__ start_pos,
                           const int* __restrict__ slots, const int* __restrict__ block_table, int nh, float scale,
                           GqaMask mask, int has_sink, float sink, GqaEpilogue epi, int* __restrict__ status) {
    using L = GqaTileSmem<DIMT, VDT>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    ST_PDL_TRIGGER();
    const int tile = blockIdx.x / parts, part = blockIdx.x % parts;
    const int req = tiles[2 * tile], off = tiles[2 * tile + 1] + part * GT_ROWS;
    const int first = q_start[req], n_new = q_start[req + 1] - first;
    if (off >= n_new) return;                           // padding tile, or the part lies past the request's tokens
    const int h = blockIdx.y, nkv = cache.nkv, vd = cache.vd, dim = cache.kd;
    const int kvh = h / (nh / nkv);
    const int start = start_pos[req];
    const int* bt = block_table + (size_t)slots[req] * cache.max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int row0 = warp * 16;
    const int rows_here = min(GT_ROWS, n_new - off);
    const int p_first = start + off, hi = p_first + rows_here - 1;
    const int lo = gqa_lo(p_first, mask);
    const int keep = mask.window > 0 ? mask.keep_first : 0;

    // this thread's two query rows (g and g + 8 of the warp's sixteen)
    int pos[2];
    bool live[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + g + 8 * r;
        live[r] = row < rows_here;
        pos[r] = p_first + row;
    }
    // what decides whether a key tile needs a mask for this warp's sixteen rows
    const bool w_all_live = row0 + 15 < rows_here;
    const bool w_any_live = row0 < rows_here;
    const int w_pos_min = p_first + row0, w_lo_max = gqa_lo(p_first + row0 + 15, mask);
    // Q fragments, from global memory (once)
    uint32_t qa[DIMT / 16][4];
#pragma unroll
    for (int ks = 0; ks < DIMT / 16; ++ks)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int r = x & 1, col = ks * 16 + 2 * tq + 8 * (x >> 1);
            const int row = row0 + g + 8 * r;
            uint32_t v = 0;
            if (live[r] && col < dim)
                v = __ldcg(reinterpret_cast<const uint32_t*>(q + ((size_t)(first + off + row) * nh + h) * dim + col));
            qa[ks][x] = v;
        }

    float o[VDT / 8][4];
#pragma unroll
    for (int nt = 0; nt < VDT / 8; ++nt)
#pragma unroll
        for (int x = 0; x < 4; ++x) o[nt][x] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // scores are kept in units of log2(e), so that the weights are exp2
    const float LOG2E = 1.4426950408889634f;
    const float scale_l2 = scale * LOG2E;

    // the block's key tiles: n_a tiles from tile 0 on (kept first keys), then tiles k_b .. kt_last
    const int k_b = lo / GT_KEYS, kt_last = hi / GT_KEYS;
    const int head_end = min(keep, lo);
    const int n_a = min((head_end + GT_KEYS - 1) / GT_KEYS, k_b);
    const int n_t = n_a + kt_last - k_b + 1;
#define GT_TILE(i) ((i) < n_a ? (i) : k_b + (i) - n_a)
    gqa_load_kv_tile<DIMT, VDT>(smem, pool, cache, bt, kvh, GT_TILE(0) * GT_KEYS, lo, hi, keep, status);
    cp_async_commit();
    for (int i = 0; i < n_t; ++i) {
        bf16* stage = smem + (i & 1) * L::STAGE;
        if (i + 1 < n_t)
            gqa_load_kv_tile<DIMT, VDT>(smem + ((i + 1) & 1) * L::STAGE, pool, cache, bt, kvh, GT_TILE(i + 1) * GT_KEYS, lo,
                                        hi, keep, status);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* sk = stage;
        const bf16* sv = stage + GT_KEYS * L::K_LD;
        const int key0 = GT_TILE(i) * GT_KEYS;
        // a warp that has no rows, whose rows all lie before the tile's first key, or whose rows' windows all start
        // behind the tile's last key (and the tile holds no kept key) has nothing to do with it
        if (w_any_live && key0 <= min(p_first + row0 + 15, hi) &&
            !(mask.window > 0 && key0 >= keep && key0 + GT_KEYS - 1 < gqa_lo(w_pos_min, mask))) {
            // S = Q K^T for the tile's 64 keys
            float s[GT_KEYS / 8][4];
#pragma unroll
            for (int nt = 0; nt < GT_KEYS / 8; ++nt) {
#pragma unroll
                for (int x = 0; x < 4; ++x) s[nt][x] = 0.f;
#pragma unroll
                for (int ks = 0; ks < DIMT / 16; ++ks) {
                    const bf16* kp = sk + (nt * 8 + g) * L::K_LD + ks * 16 + 2 * tq;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kp);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kp + 8);
                    mma_bf16(s[nt], qa[ks], b0, b1);
                }
            }
            float tmax[2] = {-INFINITY, -INFINITY};
            const bool inside = w_all_live && key0 + GT_KEYS - 1 <= w_pos_min &&
                                (mask.window <= 0 || key0 >= w_lo_max || key0 + GT_KEYS <= keep);
            if (inside) {
#pragma unroll
                for (int nt = 0; nt < GT_KEYS / 8; ++nt)
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float v = s[nt][x] * scale_l2;
                        s[nt][x] = v;
                        tmax[x >> 1] = fmaxf(tmax[x >> 1], v);
                    }
            } else {
#pragma unroll
                for (int nt = 0; nt < GT_KEYS / 8; ++nt)
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const int r = x >> 1, key = key0 + nt * 8 + 2 * tq + (x & 1);
                        const float v = (live[r] && gqa_seen(key, pos[r], mask)) ? s[nt][x] * scale_l2 : -INFINITY;
                        s[nt][x] = v;
                        tmax[r] = fmaxf(tmax[r], v);
                    }
            }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
                const float m_new = fmaxf(m[r], tmax[r]);
                corr[r] = m[r] == -INFINITY ? 0.f : fast_exp2(m[r] - m_new);
                m[r] = m_new;
            }
            float tsum[2] = {0.f, 0.f};
            uint32_t pa[GT_KEYS / 16][4];
#pragma unroll
            for (int nt = 0; nt < GT_KEYS / 8; ++nt) {
                float p[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int r = x >> 1;
                    p[x] = s[nt][x] == -INFINITY ? 0.f : fast_exp2(s[nt][x] - m[r]);
                    tsum[r] += p[x];
                }
                pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
                pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tsum[r] += __shfl_xor_sync(0xffffffffu, tsum[r], 1);
                tsum[r] += __shfl_xor_sync(0xffffffffu, tsum[r], 2);
                l[r] = l[r] * corr[r] + tsum[r];
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {     // a maximum of the warp's rows moved
#pragma unroll
                for (int nt = 0; nt < VDT / 8; ++nt) {
                    o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
                    o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
                }
            }
            // O += P V: V [key][vd] is the k-major operand, read transposed
#pragma unroll
            for (int ks = 0; ks < GT_KEYS / 16; ++ks)
#pragma unroll
                for (int nt2 = 0; nt2 < VDT / 16; ++nt2) {
                    uint32_t b0, b1, b2, b3;
                    const bf16* vp = sv + (ks * 16 + (lane & 15)) * L::V_LD + nt2 * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b0, b1, b2, b3, vp);
                    mma_bf16(o[2 * nt2], pa[ks], b0, b1);
                    mma_bf16(o[2 * nt2 + 1], pa[ks], b2, b3);
                }
        }
        __syncthreads();            // the stage may be refilled
    }
#undef GT_TILE
    cp_async_wait<0>();
    // the extra term of the denominator, then scale, gate and store
    float inv[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float ll = l[r], c = 1.f;
        if (has_sink) {
            const float s_l2 = (epi.sinks ? epi.sinks[h] : sink) * LOG2E;
            const float m_new = fmaxf(m[r], s_l2);
            c = m[r] == -INFINITY ? 0.f : fast_exp2(m[r] - m_new);
            ll = ll * c + fast_exp2(s_l2 - m_new);
        }
        inv[r] = ll > 0.f ? c * epi.out_scale / ll : 0.f;
    }
    const bf16* gate = reinterpret_cast<const bf16*>(epi.gate);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (!live[r]) continue;
        const size_t t = (size_t)(first + off + row0 + g + 8 * r);
        bf16* orow = out + (t * nh + h) * vd;
        const bf16* grow = gate ? gate + t * epi.gate_ld + (size_t)h * vd : nullptr;
#pragma unroll
        for (int nt = 0; nt < VDT / 8; ++nt) {
            const int e = nt * 8 + 2 * tq;
            if (e >= vd) continue;
            float a = o[nt][2 * r] * inv[r], b = o[nt][2 * r + 1] * inv[r];
            if (grow) {
                const __nv_bfloat162 gg = *reinterpret_cast<const __nv_bfloat162*>(grow + e);
                a *= sigmoidf_(__low2float(gg));
                b *= sigmoidf_(__high2float(gg));
            }
            *reinterpret_cast<uint32_t*>(orow + e) = pack_bf16(a, b);
        }
    }
}

template <int DIMT, int VDT>
static int launch_gqa_tiles(const void* q, const void* pool, const DiffCache& c, void* out, const int* tiles, int n_tiles,
                            int tile_rows, const int* q_start, const int* start_pos, const int* slots,
                            const int* block_table, int nh, float scale, const GqaMask& mask, int has_sink, float sink,
                            const GqaEpilogue& epi, int* status, cudaStream_t s) {
    using L = GqaTileSmem<DIMT, VDT>;
    const size_t smem = L::BYTES;
    auto kern = gqa_attention_tiles_kernel<DIMT, VDT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int parts = (tile_rows + GT_ROWS - 1) / GT_ROWS;
    kern<<<dim3(n_tiles * parts, nh), GT_THREADS, smem, s>>>((const bf16*)q, (const bf16*)pool, c, (bf16*)out, tiles, parts,
                                                            q_start, start_pos, slots, block_table, nh, scale, mask,
                                                            has_sink, sink, epi, status);
    return st_launch_status();
}

ST_EXPORT int st_gqa_attention_tiles_applies(int dim, int vd) {
    return dim > 0 && vd > 0 && dim % 8 == 0 && vd % 8 == 0 && dim <= 128 && vd <= 256;
}

// tiles: int32 [n_tiles][2] = (request of the step, offset of a tile of `tile_rows` query rows among its new tokens);
// a tile whose offset lies past the request's tokens is padding.  gate: bfloat16 logits, the head's at
// gate[token * gate_ld + head * vd ...], or null; gate_ld even and the pointer 4-byte aligned.
ST_EXPORT int st_gqa_attention_tiles(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                     void* out, const int* tiles, int n_tiles, int tile_rows, const int* q_start,
                                     const int* start_pos, const int* slots, const int* block_table, int max_pages,
                                     int nh, int nkv, int dim, int vd, int page_size, float scale, int window,
                                     int keep_first, int has_sink, float sink, const void* gate, long long gate_ld,
                                     float out_scale, int* status, void* stream, const float* sinks) {
    if (n_tiles <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || tile_rows <= 0 || keep_first < 0) return ST_ERR_BAD_ARG;
    if (!st_gqa_attention_tiles_applies(dim, vd)) return ST_ERR_BAD_SIZE;
    if (gate && ((gate_ld & 1) || ((uintptr_t)gate & 3))) return ST_ERR_BAD_ARG;
    const DiffCache c = {max_pages, page_size, nkv, dim, vd, page_stride, entry_offset};
    const GqaMask mask = {window, keep_first};
    const GqaEpilogue epi = {gate, gate_ld, out_scale, has_sink ? sinks : nullptr};
    cudaStream_t s = (cudaStream_t)stream;
#define GT_ARGS q, pool, c, out, tiles, n_tiles, tile_rows, q_start, start_pos, slots, block_table, nh, scale, mask, has_sink, \
                sink, epi, status, s
#define GT_PICK_V(DIMT)                                                   \
    do {                                                                  \
        if (vd <= 32) return launch_gqa_tiles<DIMT, 32>(GT_ARGS);         \
        if (vd <= 64) return launch_gqa_tiles<DIMT, 64>(GT_ARGS);         \
        if (vd <= 96) return launch_gqa_tiles<DIMT, 96>(GT_ARGS);         \
        if (vd <= 128) return launch_gqa_tiles<DIMT, 128>(GT_ARGS);       \
        return launch_gqa_tiles<DIMT, 256>(GT_ARGS);                      \
    } while (0)
    if (dim <= 32) GT_PICK_V(32);
    if (dim <= 64) GT_PICK_V(64);
    if (dim <= 96) GT_PICK_V(96);
    GT_PICK_V(128);
#undef GT_PICK_V
#undef GT_ARGS
}

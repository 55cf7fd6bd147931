// Paged attention in its general form: keys and values of different widths, an optional
// distance bias per head, a sliding window and a chunk mask, float32 queries.
//
// What the kinds of attention that the head-size-specific kernels do not cover share:
//   * key rows `Dk` wide and value rows `Dv` wide, each with a row stride of its own, so that
//     the value may be a leading part of the cached key row (attention over a compressed
//     latent: key = [latent | rotated part], value = latent, one cached tensor);
//   * score = (q . k) * scale - slope[h] * (p - j) where `slopes` is given (a linear distance
//     bias; p the query's position, j the key's);
//   * visible keys lo .. p with lo the largest of 0, p - window + 1 (window > 0) and
//     floor(p / chunk) * chunk (chunk > 0; chunks are counted from position 0 of the sequence);
//     with keep_first > 0 the keys 0 .. keep_first - 1 stay visible below lo as well (at their true positions);
//   * with softcap > 0 the scaled score becomes softcap * tanh(score / softcap) (before the distance bias);
//   * with `sinks` [Hq] the softmax's denominator holds one more term per head, exp(sinks[h]), that has no value.
// Queries come in float32 (rotation and score are 32-bit arithmetic whatever the cache holds);
// scores, the running maximum, the sums and the output accumulate in float32 with expf.
//
// One block per (query token, query head); key tiles of 32 aligned to absolute key indices,
// tile i handled by warp i mod 4, warps combined in index order: the result at a position does
// not depend on how the tokens were cut into steps, on what else is in the batch or on which
// pages hold the keys.  Prompt portions and single decoded tokens take the same kernel.
//
// Layouts: q [N, Hq, Dk] float32; out [N, Hq, Dv] T (float32 with out_f32); pools [pages, Hkv, page_size, stride] T;
// block_table [S, table_stride]; cu_q [S+1]; kv_len [S] (after this step); seq_of_token [N].
//
// Also here: the kernel that splits a fused projection row [q | k | v] of such widths into float32
// queries and the pages.
#include "mma_common.cuh"

namespace {

using namespace pb;

constexpr int kWarps = 4;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int n = 8; };

__device__ __forceinline__ void load16(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

struct GeneralShape {
    int Hq, Hkv, Dk, Dv, k_stride, v_stride, page_size, window, chunk, table_stride;
    int k_vec;          // leading key elements that 16-byte loads may take (0 when rows are not 16-byte aligned)
    float scale;
    int keep_first;     // keys below this stay visible whatever the window or chunk says; 0: none
    float softcap;      // > 0: scaled scores are capped to softcap * tanh(score / softcap)
    int v_share;        // consecutive key heads that read one value head (the value pool has Hkv / v_share heads); 1: a value head per key head
    int out_f32;        // the output rows are float32 whatever the pools' type (what follows subtracts them from one another)
};

template <typename T>
__device__ __forceinline__ void store_out(T* out, size_t at, float v, int out_f32) {
    if (out_f32) reinterpret_cast<float*>(out)[at] = v;
    else out[at] = from_float<T>(v);
}

// Tiles of 32 keys that a query (or a block of queries) with lowest key `lo` walks over: the tiles that hold kept first
// keys and lie wholly below the tile of `lo`, then the tiles from that of `lo` on.  n_kept is the count of the former.
__device__ __forceinline__ int kept_tiles(int lo, int keep_first) {
    return min((keep_first + 31) >> 5, lo >> 5);
}
__device__ __forceinline__ float cap_score(float s, float softcap) {
    return softcap > 0.0f ? softcap * tanhf(s / softcap) : s;
}

template <typename T, int ACC>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_general_kernel(const float* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                               T* __restrict__ out, const int* __restrict__ block_table, const int* __restrict__ cu_q,
                               const int* __restrict__ kv_len, const int* __restrict__ seq_of_token,
                               const float* __restrict__ slopes, const float* __restrict__ sinks, const GeneralShape sh,
                               const PoolBounds bounds) {
    extern __shared__ float smem[];
    const int Dk = sh.Dk, Dv = sh.Dv;
    float* q_s = smem;                         // [Dk] query times scale
    float* p_s = q_s + Dk;                     // [kWarps][32]
    float* m_s = p_s + kWarps * 32;            // [kWarps]
    float* l_s = m_s + kWarps;                 // [kWarps]
    float* acc_s = l_s + kWarps;               // [kWarps][Dv]

    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = seq_of_token[t];
    const int q0 = cu_q[s], q1 = cu_q[s + 1];
    const int p = kv_len[s] - (q1 - q0) + (t - q0);
    int lo = 0;
    if (sh.window > 0 && p - sh.window + 1 > lo) lo = p - sh.window + 1;
    if (sh.chunk > 0 && (p / sh.chunk) * sh.chunk > lo) lo = (p / sh.chunk) * sh.chunk;
    const int g = h / (sh.Hq / sh.Hkv);
    const int* table = block_table + (size_t)s * sh.table_stride;
    const float slope = slopes ? slopes[h] : 0.0f;

    const float* qv = q + ((size_t)t * sh.Hq + h) * Dk;
    for (int i = threadIdx.x; i < Dk; i += blockDim.x) q_s[i] = qv[i] * sh.scale;
    __syncthreads();

    float m_run = -INFINITY, l_run = 0.0f;
    float acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.0f;

    const int first_tile = lo >> 5, last_tile = p >> 5;
    const int n_kept = kept_tiles(lo, sh.keep_first);
    const int n_walk = n_kept + last_tile - first_tile + 1;
    for (int idx = warp; idx < n_walk; idx += kWarps) {
        const int tile = idx < n_kept ? idx : first_tile + idx - n_kept;
        const int j = (tile << 5) + lane;
        const bool valid = j <= p && (j >= lo || j < sh.keep_first);
        float sc = -INFINITY;
        if (valid) {
            int page = table[j / sh.page_size];
            if (!page_ok(page, bounds)) page = 0;
            const T* kr = k_pool + (((size_t)page * sh.Hkv + g) * sh.page_size + j % sh.page_size) * sh.k_stride;
            float dot = 0.0f;
            int d = 0;
            for (; d < sh.k_vec; d += Vec<T>::n) {
                float kf[Vec<T>::n];
                load16(kr + d, kf);
#pragma unroll
                for (int e = 0; e < Vec<T>::n; ++e) dot = fmaf(q_s[d + e], kf[e], dot);
            }
            for (; d < Dk; ++d) dot = fmaf(q_s[d], to_float(kr[d]), dot);
            sc = cap_score(dot, sh.softcap) - slope * (float)(p - j);
        }
        const float m_new = fmaxf(m_run, warp_max(sc));      // finite: every tile in range has a visible key
        const float pv = valid ? expf(sc - m_new) : 0.0f;
        const float corr = expf(m_run - m_new);               // 0 on the first tile (m_run = -inf)
        l_run = l_run * corr + warp_sum(pv);
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] *= corr;
        __syncwarp();
        p_s[warp * 32 + lane] = pv;
        __syncwarp();
        const int j0 = tile << 5;
        const int k_end = (p - j0 < 31) ? p - j0 : 31;
        for (int kk = 0; kk <= k_end; ++kk) {
            const int jj = j0 + kk;
            if (jj < lo && jj >= sh.keep_first) continue;      // uniform over the warp
            int page = table[jj / sh.page_size];
            if (!page_ok(page, bounds)) page = 0;
            const T* vr = v_pool + (((size_t)page * (sh.Hkv / sh.v_share) + g / sh.v_share) * sh.page_size + jj % sh.page_size) * sh.v_stride;
            const float pk = p_s[warp * 32 + kk];
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < Dv) acc[i] = fmaf(pk, to_float(vr[d]), acc[i]);
            }
        }
    }

    if (lane == 0) { m_s[warp] = m_run; l_s[warp] = l_run; }
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < Dv) acc_s[warp * Dv + d] = acc[i];
    }
    __syncthreads();
    float m_all = m_s[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) m_all = fmaxf(m_all, m_s[w]);
    float l_all = 0.0f;
    float f[kWarps];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) { f[w] = (m_s[w] == -INFINITY) ? 0.0f : expf(m_s[w] - m_all); l_all += l_s[w] * f[w]; }
    if (sinks) l_all += expf(sinks[h] - m_all);
    const size_t ov = ((size_t)t * sh.Hq + h) * Dv;
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) o += acc_s[w * Dv + d] * f[w];
        store_out(out, ov + d, o / l_all, sh.out_f32);
    }
}

template <typename T, int ACC>
int launch_general(const float* q, const void* k_pool, const void* v_pool, void* out, const int* block_table, const int* cu_q,
                   const int* kv_len, const int* seq_of_token, const float* slopes, const float* sinks, int n_tokens,
                   const GeneralShape& sh, cudaStream_t stream) {
    const size_t smem = sizeof(float) * (sh.Dk + kWarps * 32 + 2 * kWarps + (size_t)kWarps * sh.Dv);
    dim3 grid(n_tokens, sh.Hq);
    paged_attention_general_kernel<T, ACC><<<grid, kWarps * 32, smem, stream>>>(q, (const T*)k_pool, (const T*)v_pool, (T*)out,
        block_table, cu_q, kv_len, seq_of_token, slopes, sinks, sh, pb::pool_bounds_now());
    return launch_status();
}

template <typename T>
int dispatch_general(const float* q, const void* k_pool, const void* v_pool, void* out, const int* block_table, const int* cu_q,
                     const int* kv_len, const int* seq_of_token, const float* slopes, const float* sinks, int n_tokens,
                     GeneralShape sh, cudaStream_t stream) {
    const bool aligned = ((uintptr_t)k_pool % 16 == 0) && ((size_t)sh.k_stride * sizeof(T)) % 16 == 0;
    sh.k_vec = aligned ? sh.Dk - sh.Dk % Vec<T>::n : 0;
#define PB_GENERAL(A) return launch_general<T, A>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, seq_of_token, slopes, sinks, n_tokens, sh, stream)
    if (sh.Dv <= 64) PB_GENERAL(2);
    if (sh.Dv <= 128) PB_GENERAL(4);
    if (sh.Dv <= 256) PB_GENERAL(8);
    if (sh.Dv <= 512) PB_GENERAL(16);
    PB_GENERAL(32);
#undef PB_GENERAL
}

// ---------------------------------------------------------------- the tiled form
// The same arithmetic with the keys and values of a tile staged in shared memory and shared by 16 query rows: the rows of
// a block are consecutive (token, head) pairs of one sequence and one key/value head (index = token * group + head in
// group), so a step of single tokens shares a tile among the heads of a group and a prompt portion among tokens as well.
// Warp w owns rows 4w .. 4w+3; its lane l scores key l of the tile against the four rows (the key's elements come from
// shared memory 16 bytes at a time, the queries by broadcast), the warp reduces maxima and sums over its lanes, and lane l
// then owns value columns l, l + 32, ... of the four rows' outputs.  Tiles of 32 keys are aligned to absolute key
// indices and taken in ascending order; a tile in which a row sees nothing leaves that row's state untouched, so a row's
// result depends on its own position alone.  With splits (grid z) each block takes a contiguous share of the tiles and
// writes (maximum, sum, unnormalised output) per row to a float32 workspace that general_combine_kernel merges in split
// order.  Needs key and value rows that are multiples of 16 bytes; other sizes take the kernel above.
constexpr int kRows = 16;
constexpr int kTile = 32;

struct TiledShape {
    GeneralShape g;
    int n_seqs, n_splits, k_row, v_row;      // rows of the staged tiles in elements (k_row padded; v_row = k_row when the value is part of the key row)
    int v_in_k;
};


template <typename T, int ACC>
__global__ void __launch_bounds__(128)
general_tiled_kernel(const float* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool, T* __restrict__ out,
                     float* __restrict__ partial, const int* __restrict__ block_table, const int* __restrict__ cu_q,
                     const int* __restrict__ kv_len, const float* __restrict__ slopes, const float* __restrict__ sinks,
                     const TiledShape ts, const PoolBounds bounds) {
    constexpr int V = Vec<T>::n;
    const GeneralShape& sh = ts.g;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int Dk = sh.Dk, Dv = sh.Dv, GH = sh.Hq / sh.Hkv;
    float* q_s = reinterpret_cast<float*>(smem_raw);                         // [kRows][Dk]
    float* p_s = q_s + kRows * Dk;                                            // [kRows][kTile]
    T* k_s = reinterpret_cast<T*>(p_s + kRows * kTile);                       // [kTile][k_row]
    T* v_s = ts.v_in_k ? k_s : k_s + (size_t)kTile * ts.k_row;                // [kTile][v_row]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = blockIdx.y, split = blockIdx.z;
    int tile = blockIdx.x, s = 0, q0 = 0, q_len = 0;
    for (; s < ts.n_seqs; ++s) {
        q0 = cu_q[s];
        q_len = cu_q[s + 1] - q0;
        const int nt = (q_len * GH + kRows - 1) / kRows;
        if (tile < nt) break;
        tile -= nt;
    }
    if (s >= ts.n_seqs) return;
    const int ctx0 = kv_len[s] - q_len;
    const int idx0 = tile * kRows;
    const int n_rows = min(kRows, q_len * GH - idx0);
    const int* table = block_table + (size_t)s * sh.table_stride;

    // the block's span of keys: from the lowest key any row sees to the highest
    int lo_blk = 0x7fffffff, hi_blk = 0;
    for (int r = 0; r < n_rows; ++r) {
        const int p = ctx0 + (idx0 + r) / GH;
        int lo = 0;
        if (sh.window > 0 && p - sh.window + 1 > lo) lo = p - sh.window + 1;
        if (sh.chunk > 0 && (p / sh.chunk) * sh.chunk > lo) lo = (p / sh.chunk) * sh.chunk;
        lo_blk = min(lo_blk, lo);
        hi_blk = max(hi_blk, p);
    }
    // the tiles the block walks over, in ascending order: those of kept first keys below the span, then the span's
    const int kt0 = lo_blk / kTile, n_kept = kept_tiles(lo_blk, sh.keep_first);
    const int n_tiles = n_kept + hi_blk / kTile - kt0 + 1;
    const int per = (n_tiles + ts.n_splits - 1) / ts.n_splits;
    const int t_begin = split * per, t_end = min(n_tiles, t_begin + per);

    // this thread's four rows
    int pos[4], lo_r[4], tok[4], head[4];
    float slope[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int row = warp * 4 + r;
        const bool on = row < n_rows;
        const int idx = idx0 + (on ? row : 0);
        tok[r] = q0 + idx / GH;
        head[r] = g * GH + idx % GH;
        pos[r] = on ? ctx0 + idx / GH : -1;                  // -1: sees no key
        int lo = 0;
        if (sh.window > 0 && pos[r] - sh.window + 1 > lo) lo = pos[r] - sh.window + 1;
        if (sh.chunk > 0 && pos[r] >= 0 && (pos[r] / sh.chunk) * sh.chunk > lo) lo = (pos[r] / sh.chunk) * sh.chunk;
        lo_r[r] = lo;
        slope[r] = slopes ? slopes[head[r]] : 0.0f;
    }
    // the rows' queries, 16 bytes at a time, all copies in flight at once (the scale enters with the scores)
    {
        const int q_chunks = Dk / 4;
        for (int c = threadIdx.x; c < kRows * q_chunks; c += blockDim.x) {
            const int row = c / q_chunks, part = c % q_chunks;
            const bool on = row < n_rows;
            const int idx = idx0 + (on ? row : 0);
            const float* src = q + ((size_t)(q0 + idx / GH) * sh.Hq + g * GH + idx % GH) * Dk + part * 4;
            cp_async16(smem_u32(q_s + (size_t)row * Dk + part * 4), src, on);
        }
        cp_async_commit();
    }

    float m_run[4], l_run[4], acc[4][ACC];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        m_run[r] = -INFINITY;
        l_run[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[r][i] = 0.0f;
    }

    const int k_chunks = Dk / V, v_chunks = Dv / V;
    for (int ti = t_begin; ti < t_end; ++ti) {
        const int kt = ti < n_kept ? ti : kt0 + ti - n_kept;
        const int j0 = kt * kTile;
        __syncthreads();                                   // the tile before is done with
        {
            // four threads per key: one look into the block table, then the row's 16-byte pieces, all in flight at once
            const int key = threadIdx.x >> 2, sub = threadIdx.x & 3;
            const int j = j0 + key;
            const bool ok = j <= hi_blk && (j >= lo_blk || j < sh.keep_first);   // rows outside the block's span are filled with zeros
            const T* k_src = k_pool;
            const T* v_src = v_pool;
            if (ok) {
                int page = table[j / sh.page_size];
                if (!page_ok(page, bounds)) page = 0;
                const size_t at = ((size_t)page * sh.Hkv + g) * sh.page_size + j % sh.page_size;
                const size_t v_at = ((size_t)page * (sh.Hkv / sh.v_share) + g / sh.v_share) * sh.page_size + j % sh.page_size;
                k_src = k_pool + at * sh.k_stride;
                v_src = v_pool + v_at * sh.v_stride;
            }
            for (int part = sub; part < k_chunks; part += 4)
                cp_async16(smem_u32(k_s + (size_t)key * ts.k_row + part * V), k_src + part * V, ok);
            if (!ts.v_in_k)
                for (int part = sub; part < v_chunks; part += 4)
                    cp_async16(smem_u32(v_s + (size_t)key * ts.v_row + part * V), v_src + part * V, ok);
            cp_async_commit();
            cp_async_wait<0>();
        }
        __syncthreads();

        if (warp * 4 >= n_rows) continue;                  // a warp without rows only helps to load (a step of single tokens: the group's heads are all the rows there are)
        // scores of key `lane` against the warp's four rows
        float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const T* kr = k_s + (size_t)lane * ts.k_row;
        const float* qr = q_s + (size_t)(warp * 4) * Dk;
        for (int d = 0; d < Dk; d += V) {
            float kf[V];
            load16(kr + d, kf);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
#pragma unroll
                for (int e = 0; e < V; e += 4) {
                    const float4 qv = *reinterpret_cast<const float4*>(qr + r * Dk + d + e);
                    sc[r] = fmaf(qv.x, kf[e], sc[r]);
                    sc[r] = fmaf(qv.y, kf[e + 1], sc[r]);
                    sc[r] = fmaf(qv.z, kf[e + 2], sc[r]);
                    sc[r] = fmaf(qv.w, kf[e + 3], sc[r]);
                }
            }
        }
        const int j = j0 + lane;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const bool vis = j <= pos[r] && (j >= lo_r[r] || j < sh.keep_first);
            const float v = vis ? (sh.softcap > 0.0f ? cap_score(sc[r] * sh.scale, sh.softcap) - slope[r] * (float)(pos[r] - j)
                                                     : fmaf(sc[r], sh.scale, -slope[r] * (float)(pos[r] - j)))
                                : -INFINITY;
            const float m_new = fmaxf(m_run[r], warp_max(v));
            float pv = 0.0f, corr = 1.0f;
            if (m_new != -INFINITY) {                       // uniform over the warp
                pv = vis ? expf(v - m_new) : 0.0f;
                corr = expf(m_run[r] - m_new);              // 0 while the row had seen nothing
            }
            l_run[r] = l_run[r] * corr + warp_sum(pv);
            m_run[r] = m_new;
            if (corr != 1.0f) {
#pragma unroll
                for (int i = 0; i < ACC; ++i) acc[r][i] *= corr;
            }
            p_s[(warp * 4 + r) * kTile + lane] = pv;
        }
        __syncwarp();
        // outputs: lane owns value columns lane + 32 i of the four rows
        const float* pr = p_s + (warp * 4) * kTile;
        for (int kk = 0; kk < kTile; kk += 4) {
            float4 pw[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) pw[r] = *reinterpret_cast<const float4*>(pr + r * kTile + kk);
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int c = lane + 32 * i;
                if (c < Dv) {
                    const float v0 = to_float(v_s[(size_t)(kk + 0) * ts.v_row + c]), v1 = to_float(v_s[(size_t)(kk + 1) * ts.v_row + c]);
                    const float v2 = to_float(v_s[(size_t)(kk + 2) * ts.v_row + c]), v3 = to_float(v_s[(size_t)(kk + 3) * ts.v_row + c]);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        acc[r][i] = fmaf(pw[r].x, v0, acc[r][i]);
                        acc[r][i] = fmaf(pw[r].y, v1, acc[r][i]);
                        acc[r][i] = fmaf(pw[r].z, v2, acc[r][i]);
                        acc[r][i] = fmaf(pw[r].w, v3, acc[r][i]);
                    }
                }
            }
        }
        __syncwarp();
    }

    cp_async_wait<0>();                                    // a block without tiles still has its queries on their way
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        if (warp * 4 + r >= n_rows) continue;
        const size_t row = (size_t)tok[r] * sh.Hq + head[r];
        if (ts.n_splits == 1) {
            const float inv = 1.0f / (sinks ? l_run[r] + expf(sinks[head[r]] - m_run[r]) : l_run[r]);
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int c = lane + 32 * i;
                if (c < Dv) store_out(out, row * Dv + c, acc[r][i] * inv, sh.out_f32);
            }
        } else {
            float* pp = partial + (row * ts.n_splits + split) * (Dv + 2);
            if (lane == 0) { pp[0] = m_run[r]; pp[1] = l_run[r]; }
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int c = lane + 32 * i;
                if (c < Dv) pp[2 + c] = acc[r][i];
            }
        }
    }
}

// out[row] = sum over the splits, in their order, of their partial outputs weighted by exp(m_split - m_all), over the
// weighted sum of their sums.  One block per (token, head).
template <typename T>
__global__ void general_combine_kernel(const float* __restrict__ partial, T* __restrict__ out, const float* __restrict__ sinks,
                                       int Hq, int n_splits, int Dv, int out_f32) {
    const size_t row = blockIdx.x;
    const float* pp = partial + row * n_splits * (Dv + 2);
    float m_all = -INFINITY;
    for (int z = 0; z < n_splits; ++z) m_all = fmaxf(m_all, pp[(size_t)z * (Dv + 2)]);
    float l_all = 0.0f;
    for (int z = 0; z < n_splits; ++z) {
        const float m = pp[(size_t)z * (Dv + 2)];
        if (m != -INFINITY) l_all += pp[(size_t)z * (Dv + 2) + 1] * expf(m - m_all);
    }
    if (sinks) l_all += expf(sinks[row % Hq] - m_all);
    for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
        float o = 0.0f;
        for (int z = 0; z < n_splits; ++z) {
            const float m = pp[(size_t)z * (Dv + 2)];
            if (m != -INFINITY) o += pp[(size_t)z * (Dv + 2) + 2 + c] * expf(m - m_all);
        }
        store_out(out, row * Dv + c, o / l_all, out_f32);
    }
}

template <typename T>
size_t tiled_smem(const TiledShape& ts) {
    return sizeof(float) * (kRows * ts.g.Dk + kRows * kTile) + sizeof(T) * kTile * ((size_t)ts.k_row + (ts.v_in_k ? 0 : ts.v_row));
}

template <typename T, int ACC>
int launch_tiled(const float* q, const void* k_pool, const void* v_pool, void* out, float* partial, const int* block_table,
                 const int* cu_q, const int* kv_len, const float* slopes, const float* sinks, int n_tokens, int row_tiles,
                 const TiledShape& ts, cudaStream_t stream) {
    const size_t smem = tiled_smem<T>(ts);
    static size_t allowed = 48 * 1024;                     // per instantiation
    if (smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(general_tiled_kernel<T, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    dim3 grid(row_tiles, ts.g.Hkv, ts.n_splits);
    general_tiled_kernel<T, ACC><<<grid, 128, smem, stream>>>(q, (const T*)k_pool, (const T*)v_pool, (T*)out, partial, block_table,
                                                              cu_q, kv_len, slopes, sinks, ts, pb::pool_bounds_now());
    int status = launch_status();
    if (status == 0 && ts.n_splits > 1) {
        int b = 32;
        while (b < ts.g.Dv && b < 256) b <<= 1;
        general_combine_kernel<T><<<n_tokens * ts.g.Hq, b, 0, stream>>>(partial, (T*)out, sinks, ts.g.Hq, ts.n_splits, ts.g.Dv, ts.g.out_f32);
        status = launch_status();
    }
    return status;
}

template <typename T>
bool tiled_shape(TiledShape& ts, const void* k_pool, const void* v_pool) {
    const GeneralShape& sh = ts.g;
    const size_t e = sizeof(T);
    if ((sh.Dk * e) % 16 || (sh.Dv * e) % 16 || (sh.k_stride * e) % 16 || (sh.v_stride * e) % 16) return false;
    if (((uintptr_t)k_pool | (uintptr_t)v_pool) % 16) return false;
    ts.v_in_k = (k_pool == v_pool && sh.k_stride == sh.v_stride && sh.Dv <= sh.Dk) ? 1 : 0;
    const int unit = 16 / (int)e;                           // elements in 16 bytes
    int k_units = sh.Dk / unit;
    if (k_units % 2 == 0) ++k_units;                        // rows an odd number of 16-byte units apart: lanes on different rows do not collide
    ts.k_row = k_units * unit;
    ts.v_row = ts.v_in_k ? ts.k_row : sh.Dv;
    return tiled_smem<T>(ts) <= 200 * 1024;
}

template <typename T>
int dispatch_tiled(const float* q, const void* k_pool, const void* v_pool, void* out, float* partial, const int* block_table,
                   const int* cu_q, const int* kv_len, const float* slopes, const float* sinks, int n_tokens, int row_tiles,
                   const TiledShape& ts, cudaStream_t stream) {
#define PB_TILED(A) return launch_tiled<T, A>(q, k_pool, v_pool, out, partial, block_table, cu_q, kv_len, slopes, sinks, n_tokens, row_tiles, ts, stream)
    if (ts.g.Dv <= 64) PB_TILED(2);
    if (ts.g.Dv <= 128) PB_TILED(4);
    if (ts.g.Dv <= 256) PB_TILED(8);
    PB_TILED(16);
#undef PB_TILED
}

// One warp per (token, head) of the fused projection row [q: Hq*Dk | k: Hk*Dk | v: Hv*Dv]:
// queries to float32 [N, Hq, Dk], keys and values into the pages of the token's slot (pools of Hk and of Hv heads).
// With temp_coef != 0 a query at position p is multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1).
template <typename T>
__global__ void qkv_split_write_kernel(const T* __restrict__ qkv, float* __restrict__ q_out, T* __restrict__ k_pool,
                                       T* __restrict__ v_pool, const int* __restrict__ slots, int Hq, int Hk, int Hv, int Dk, int Dv,
                                       int page_size, const int* __restrict__ positions, float temp_coef, int temp_every,
                                       const PoolBounds bounds) {
    pdl_wait();         // may have come onto the SMs while the product before it was ending: nothing is touched before that one is done
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (head >= Hq + Hk + Hv) return;
    const size_t row = (size_t)Hq * Dk + (size_t)Hk * Dk + (size_t)Hv * Dv;
    const T* base = qkv + (size_t)t * row;
    if (head < Hq) {
        const T* src = base + (size_t)head * Dk;
        float* dst = q_out + ((size_t)t * Hq + head) * Dk;
        float f = 1.0f;
        if (temp_coef != 0.0f) f = 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every + 1));
        for (int i = lane; i < Dk; i += 32) dst[i] = to_float(src[i]) * f;
        return;
    }
    const int slot = slots[t];
    if (slot < 0 || !slot_ok(slot, page_size, bounds)) return;
    const bool is_k = head < Hq + Hk;
    const int kvh = is_k ? head - Hq : head - Hq - Hk;
    const int D = is_k ? Dk : Dv, Hp = is_k ? Hk : Hv;
    const T* src = base + (size_t)Hq * Dk + (is_k ? (size_t)kvh * Dk : (size_t)Hk * Dk + (size_t)kvh * Dv);
    T* dst = (is_k ? k_pool : v_pool) + (((size_t)(slot / page_size) * Hp + kvh) * page_size + slot % page_size) * D;
    for (int i = lane; i < D; i += 32) dst[i] = src[i];
}

}  // namespace

PB_EXPORT int pb_paged_attention_general(int dtype, const float* q, const void* k_pool, const void* v_pool, void* out,
                                         const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                                         const int* seq_of_token, const float* slopes, int n_tokens, int Hq, int Hkv, int Dk,
                                         int Dv, int k_stride, int v_stride, int page_size, float scale, int window, int chunk,
                                         int keep_first, float softcap, const float* sinks, int v_share, int out_f32, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (Dk <= 0 || Dv <= 0 || Dk > 4096 || Dv > 1024 || Hkv <= 0 || Hq <= 0 || Hq % Hkv || page_size <= 0 || k_stride < Dk ||
        v_stride < Dv || window < 0 || chunk < 0 || keep_first < 0 || !(softcap >= 0.0f) || v_share <= 0 || Hkv % v_share)
        return PB_ERR_BAD_SIZE;
    if (Hq > 65535) return PB_ERR_TOO_LARGE;
    GeneralShape sh{Hq, Hkv, Dk, Dv, k_stride, v_stride, page_size, window, chunk, table_stride, 0, scale, keep_first, softcap, v_share,
                    out_f32 != 0};
    if (dtype == PB_F32)
        return dispatch_general<float>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, seq_of_token, slopes, sinks, n_tokens, sh,
                                       stream);
    if (dtype == PB_BF16)
        return dispatch_general<__nv_bfloat16>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, seq_of_token, slopes, sinks, n_tokens,
                                               sh, stream);
    return PB_ERR_BAD_DTYPE;
}

PB_EXPORT int pb_qkv_split_write(int dtype, const void* qkv, float* q_out, void* k_pool, void* v_pool, const int* slots,
                                 int n_tokens, int Hq, int Hk, int Hv, int Dk, int Dv, int page_size, const int* positions,
                                 float temp_coef, int temp_every, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (Hq <= 0 || Hk < 0 || Hv < 0 || Dk <= 0 || Dv <= 0 || page_size <= 0) return PB_ERR_BAD_SIZE;
    if (temp_coef != 0.0f && (positions == nullptr || temp_every <= 0)) return PB_ERR_BAD_SIZE;
    const int heads = Hq + Hk + Hv;
    dim3 grid(n_tokens, (heads + 3) / 4);
    if (dtype == PB_F32)
        launch_pdl(qkv_split_write_kernel<float>, grid, 128, 0, stream, (const float*)qkv, q_out, (float*)k_pool, (float*)v_pool, slots, Hq,
                                                                Hk, Hv, Dk, Dv, page_size, positions, temp_coef, temp_every, pb::pool_bounds_now());
    else if (dtype == PB_BF16)
        launch_pdl(qkv_split_write_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)qkv, q_out, (__nv_bfloat16*)k_pool,
                                                                        (__nv_bfloat16*)v_pool, slots, Hq, Hk, Hv, Dk, Dv, page_size,
                                                                        positions, temp_coef, temp_every, pb::pool_bounds_now());
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_attention_general_tiled_supported(int dtype, const void* k_pool, const void* v_pool, int Hq, int Hkv, int Dk, int Dv,
                                                   int k_stride, int v_stride) {
    if (Dk <= 0 || Dv <= 0 || Dv > 512 || Hkv <= 0 || Hq <= 0 || Hq % Hkv || k_stride < Dk || v_stride < Dv) return 0;
    TiledShape ts{};
    ts.g = GeneralShape{Hq, Hkv, Dk, Dv, k_stride, v_stride, 1, 0, 0, 0, 0, 1.0f, 0, 0.0f, 1};
    if (dtype == PB_F32) return tiled_shape<float>(ts, k_pool, v_pool) ? 1 : 0;
    if (dtype == PB_BF16) return tiled_shape<__nv_bfloat16>(ts, k_pool, v_pool) ? 1 : 0;
    return 0;
}

// The tiled form of pb_paged_attention_general.  row_tiles: the sum over the sequences of ceil(new tokens * (Hq / Hkv) / 16).
// n_splits > 1 needs `partial`: float32, n_tokens * Hq * n_splits * (Dv + 2) elements.
PB_EXPORT int pb_paged_attention_general_tiled(int dtype, const float* q, const void* k_pool, const void* v_pool, void* out,
                                               float* partial, const int* block_table, int table_stride, const int* cu_q,
                                               const int* kv_len, const float* slopes, int n_tokens, int n_seqs, int row_tiles,
                                               int n_splits, int Hq, int Hkv, int Dk, int Dv, int k_stride, int v_stride,
                                               int page_size, float scale, int window, int chunk, int keep_first, float softcap,
                                               const float* sinks, int v_share, int out_f32, cudaStream_t stream) {
    if (n_tokens <= 0 || row_tiles <= 0) return 0;
    if (v_share <= 0 || Hkv % v_share) return PB_ERR_BAD_SIZE;
    if (!pb_attention_general_tiled_supported(dtype, k_pool, v_pool, Hq, Hkv, Dk, Dv, k_stride, v_stride)) return PB_ERR_BAD_SIZE;
    if (page_size <= 0 || window < 0 || chunk < 0 || keep_first < 0 || !(softcap >= 0.0f) || n_splits < 1 || n_splits > 65535 ||
        (n_splits > 1 && partial == nullptr) || (uintptr_t)q % 16)
        return PB_ERR_BAD_SIZE;
    if (Hkv > 65535) return PB_ERR_TOO_LARGE;
    TiledShape ts{};
    ts.g = GeneralShape{Hq, Hkv, Dk, Dv, k_stride, v_stride, page_size, window, chunk, table_stride, 0, scale, keep_first, softcap, v_share,
                        out_f32 != 0};
    ts.n_seqs = n_seqs;
    ts.n_splits = n_splits;
    if (dtype == PB_F32) {
        tiled_shape<float>(ts, k_pool, v_pool);
        return dispatch_tiled<float>(q, k_pool, v_pool, out, partial, block_table, cu_q, kv_len, slopes, sinks, n_tokens, row_tiles, ts,
                                     stream);
    }
    tiled_shape<__nv_bfloat16>(ts, k_pool, v_pool);
    return dispatch_tiled<__nv_bfloat16>(q, k_pool, v_pool, out, partial, block_table, cu_q, kv_len, slopes, sinks, n_tokens, row_tiles,
                                         ts, stream);
}

// The general attention (float32 queries, key and value rows of different widths, distance bias, window,
// chunk mask) for prompt portions on the tensor cores, with both contractions at float32-like precision.
//
// mma.sync takes bfloat16 operands.  The cache holds bfloat16 keys and values, which are exact as they are; what
// must not be rounded to 16 bits are the queries (rotated in float32) and the softmax weights.  Each of them is
// split into two bfloat16 numbers, x = hi + lo with hi = bf16(x) and lo = bf16(x - hi) (16 bits of mantissa
// together), and every product is two MMAs into the same float32 accumulator: S = Q_hi K^T + Q_lo K^T,
// O += P_hi V + P_lo V.  Scores, maxima, exponentials (ex2.approx of the score times log2 e: relative error 2^-22)
// and sums are float32.
//
// One block of four warps per (64 query tokens of one sequence, query head); each warp owns 16 rows.  The split
// queries stay in shared memory; keys and values stream through a two-stage cp.async pipeline of 32-key tiles
// gathered row by row through the block table (any page size) into XOR-swizzled tiles.  Tiles are aligned to
// absolute key indices and taken in ascending order; a tile in which a row sees nothing leaves the row as it was.
// Kept first keys (keep_first > 0: keys 0 .. keep_first - 1 stay visible below the window), a cap on the scaled score
// (softcap > 0: softcap * tanh(score / softcap) in float32, through ex2.approx like the softmax's exponentials) and a
// sink per head (one more term exp(sinks[h]) in the softmax's denominator) as in the CUDA-core kernels.
#include "mma_common.cuh"

namespace {

using namespace pb;

constexpr int kBM = 64;          // query rows per block
constexpr int kBN = 32;          // keys per pipeline stage
constexpr int kWarps = 4;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// tanh(x) = 1 - 2 / (1 + e^(2x)) with the exponential from ex2.approx (relative error 2^-22) and an approximate division: the
// absolute error stays below 3e-7, which in a capped score (cap * tanh) is a few units in the last place of the cap.
__device__ __forceinline__ float tanh_ex2(float x) {
    return 1.0f - __fdividef(2.0f, 1.0f + ex2(x * (2.0f * kLog2e)));
}

__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

struct TcShape {
    int n_seqs, Hq, Hkv, k_stride, v_stride, page_size, window, chunk, table_stride;
    float scale;
    int keep_first;
    float softcap;
    int v_share;        // consecutive key heads that read one value head (the value pool has Hkv / v_share heads)
    int out_f32;        // the output rows are float32: the accumulators go out as they are, without the round to bfloat16
};

__device__ __forceinline__ int lowest_key(int pos, const TcShape& sh) {
    int lo = 0;
    if (sh.window > 0 && pos - sh.window + 1 > lo) lo = pos - sh.window + 1;
    if (sh.chunk > 0 && (pos / sh.chunk) * sh.chunk > lo) lo = (pos / sh.chunk) * sh.chunk;
    return lo;
}

template <int DK, int DV>
__global__ void __launch_bounds__(kWarps * 32, 2)
general_tc_kernel(const float* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                  bf16* __restrict__ out, const int* __restrict__ block_table, const int* __restrict__ cu_q,
                  const int* __restrict__ kv_len, const float* __restrict__ slopes, const float* __restrict__ sinks,
                  const TcShape sh, const PoolBounds bounds) {
    constexpr int kChunksK = DK / 8, kChunksV = DV / 8;
    constexpr int kQBytes = kBM * DK * 2;                    // one of the two query tiles
    constexpr int kKBytes = kBN * DK * 2, kVBytes = kBN * DV * 2;
    constexpr int kKSteps = DK / 16, kNTiles = DV / 8;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);               // [Q hi][Q lo][2 stages][K tile | V tile]
    const uint32_t stage_base = smem_base + 2 * kQBytes;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int head = blockIdx.y;
    const int kvh = head / (sh.Hq / sh.Hkv);

    int tile = gridDim.x - 1 - blockIdx.x;                   // heaviest first
    int s = 0, q0 = 0, q_len = 0;
    for (; s < sh.n_seqs; ++s) {
        q0 = cu_q[s];
        q_len = cu_q[s + 1] - q0;
        const int nt = (q_len + kBM - 1) / kBM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (s >= sh.n_seqs) return;
    const int m0 = tile * kBM;
    const int rows = min(kBM, q_len - m0);
    const int ctx0 = kv_len[s] - q_len;
    const int pos_first = ctx0 + m0, pos_last = ctx0 + m0 + rows - 1;
    const int lo_blk = lowest_key(pos_first, sh);            // the lowest key is no lower for a later position
    // the tiles the block walks over, in ascending order: those of kept first keys below the span, then the span's
    const int kt0 = lo_blk / kBN, n_kept = min((sh.keep_first + kBN - 1) / kBN, kt0);
    const int n_tiles = n_kept + pos_last / kBN - kt0 + 1;
    const int* table = block_table + (size_t)s * sh.table_stride;

    auto issue_kv = [&](int tile_index, int stage) {
        // four threads per key row: one look into the block table, then the row's 16-byte pieces of K and of V
        static_assert(kBN * 4 == kWarps * 32, "four threads per key row");
        const uint32_t k_dst = stage_base + stage * (kKBytes + kVBytes), v_dst = k_dst + kKBytes;
        const int row = tid >> 2, sub = tid & 3;
        const int key = (tile_index < n_kept ? tile_index : kt0 + tile_index - n_kept) * kBN + row;
        const bool ok = key <= pos_last && (key >= lo_blk || key < sh.keep_first);
        size_t k_at = 0, v_at = 0;
        if (ok) {
            int page = table[key / sh.page_size];
            if (!page_ok(page, bounds)) page = 0;
            const size_t at = ((size_t)page * sh.Hkv + kvh) * sh.page_size + key % sh.page_size;
            k_at = at * sh.k_stride;
            v_at = (((size_t)page * (sh.Hkv / sh.v_share) + kvh / sh.v_share) * sh.page_size + key % sh.page_size) * sh.v_stride;
        }
#pragma unroll
        for (int c = sub; c < kChunksK; c += 4) cp_async16(k_dst + tile_offset<DK>(row, c), k_pool + k_at + c * 8, ok);
#pragma unroll
        for (int c = sub; c < kChunksV; c += 4) cp_async16(v_dst + tile_offset<DV>(row, c), v_pool + v_at + c * 8, ok);
    };

    issue_kv(0, 0);
    cp_async_commit();
    // the query rows, split into their two halves
    for (int idx = tid; idx < kBM * kChunksK; idx += kWarps * 32) {
        const int row = idx / kChunksK, c = idx % kChunksK;
        uint4 hi = make_uint4(0, 0, 0, 0), lo = make_uint4(0, 0, 0, 0);
        if (row < rows) {
            const float4* src = reinterpret_cast<const float4*>(q + ((size_t)(q0 + m0 + row) * sh.Hq + head) * DK + c * 8);
            const float4 a = src[0], b = src[1];
            split_bf16(a.x, a.y, hi.x, lo.x);
            split_bf16(a.z, a.w, hi.y, lo.y);
            split_bf16(b.x, b.y, hi.z, lo.z);
            split_bf16(b.z, b.w, hi.w, lo.w);
        }
        *reinterpret_cast<uint4*>(smem + tile_offset<DK>(row, c)) = hi;
        *reinterpret_cast<uint4*>(smem + kQBytes + tile_offset<DK>(row, c)) = lo;
    }

    float o[kNTiles][4];
#pragma unroll
    for (int i = 0; i < kNTiles; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const float sl2 = sh.scale * kLog2e;
    const float cap_in = sh.softcap > 0.0f ? sh.scale / sh.softcap : 0.0f;
    const float slope2 = slopes ? slopes[head] * kLog2e : 0.0f;
    const int r0 = min(warp * 16 + g, rows - 1), r1 = min(warp * 16 + g + 8, rows - 1);
    const int pos0 = pos_first + r0, pos1 = pos_first + r1;
    const int lo0 = lowest_key(pos0, sh), lo1 = lowest_key(pos1, sh);
    const int wpos_first = pos_first + min(warp * 16, rows - 1), wpos_last = pos_first + min(warp * 16 + 15, rows - 1);
    const int wlo_first = lowest_key(wpos_first, sh);
    const int q_row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);

    for (int it = 0; it < n_tiles; ++it) {
        if (it + 1 < n_tiles) issue_kv(it + 1, (it + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();                                   // tile `it` has landed (and, the first time, the queries are written)

        const int stage = it & 1;
        const uint32_t k_s = stage_base + stage * (kKBytes + kVBytes), v_s = k_s + kKBytes;
        const int key0 = (it < n_kept ? it : kt0 + it - n_kept) * kBN;
        const bool active = warp * 16 < rows && key0 <= wpos_last && (key0 + kBN - 1 >= wlo_first || key0 < sh.keep_first);
        if (active) {
            float sc[kBN / 8][4];
#pragma unroll
            for (int n = 0; n < kBN / 8; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f; }
#pragma unroll
            for (int ks = 0; ks < kKSteps; ++ks) {
                uint32_t qh[4], ql[4];
                ldmatrix_x4(qh, smem_base + tile_offset<DK>(q_row, ks * 2 + (lane >> 4)));
                ldmatrix_x4(ql, smem_base + kQBytes + tile_offset<DK>(q_row, ks * 2 + (lane >> 4)));
                // both halves of the queries against the tile's four groups of eight keys: eight MMAs, each accumulator
                // used again only after three others
                uint32_t kb[kBN / 16][4];
#pragma unroll
                for (int nn = 0; nn < kBN / 16; ++nn) {
                    const int row = nn * 16 + (lane & 7) + ((lane >> 4) << 3);
                    ldmatrix_x4(kb[nn], k_s + tile_offset<DK>(row, ks * 2 + ((lane >> 3) & 1)));
                }
#pragma unroll
                for (int nn = 0; nn < kBN / 16; ++nn) {
                    mma_bf16(sc[2 * nn], qh, kb[nn][0], kb[nn][1]);
                    mma_bf16(sc[2 * nn + 1], qh, kb[nn][2], kb[nn][3]);
                }
#pragma unroll
                for (int nn = 0; nn < kBN / 16; ++nn) {
                    mma_bf16(sc[2 * nn], ql, kb[nn][0], kb[nn][1]);
                    mma_bf16(sc[2 * nn + 1], ql, kb[nn][2], kb[nn][3]);
                }
            }
            // scores in the exponent's units (times log2 e), with the distance bias; what a row does not see is -inf
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < kBN / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + n * 8 + 2 * t + (e & 1);
                    const int pos = (e >> 1) ? pos1 : pos0;
                    const int lo = (e >> 1) ? lo1 : lo0;
                    const bool vis = key <= pos && (key >= lo || key < sh.keep_first);
                    float v = -INFINITY;
                    if (vis) {
                        if (sh.softcap > 0.0f)
                            v = fmaf(sh.softcap * tanh_ex2(sc[n][e] * cap_in), kLog2e, -slope2 * (float)(pos - key));
                        else
                            v = fmaf(sc[n][e], sl2, -slope2 * (float)(pos - key));
                    }
                    sc[n][e] = v;
                    tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
                }
            float corr[2], m_safe[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float mx = tmax[r];
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[r], mx);
                m_safe[r] = (m_new == -INFINITY) ? 0.0f : m_new;             // a row that has seen no key yet
                corr[r] = ex2(m_run[r] - m_safe[r]);
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
                for (int i = 0; i < kNTiles; ++i) {
                    o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk) {
                uint32_t ph[4], pl[4];
                float pv[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        pv[n][e] = ex2(sc[2 * kk + n][e] - m_safe[e >> 1]);
                        l_run[e >> 1] += pv[n][e];
                    }
                split_bf16(pv[0][0], pv[0][1], ph[0], pl[0]);
                split_bf16(pv[0][2], pv[0][3], ph[1], pl[1]);
                split_bf16(pv[1][0], pv[1][1], ph[2], pl[2]);
                split_bf16(pv[1][2], pv[1][3], ph[3], pl[3]);
#pragma unroll
                for (int i = 0; i < kNTiles; i += 4) {
                    uint32_t va[4], vb[4];
                    const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldmatrix_x4_trans(va, v_s + tile_offset<DV>(row, i + (lane >> 4)));
                    ldmatrix_x4_trans(vb, v_s + tile_offset<DV>(row, i + 2 + (lane >> 4)));
                    mma_bf16(o[i], ph, va[0], va[1]);
                    mma_bf16(o[i + 1], ph, va[2], va[3]);
                    mma_bf16(o[i + 2], ph, vb[0], vb[1]);
                    mma_bf16(o[i + 3], ph, vb[2], vb[3]);
                    mma_bf16(o[i], pl, va[0], va[1]);
                    mma_bf16(o[i + 1], pl, va[2], va[3]);
                    mma_bf16(o[i + 2], pl, vb[0], vb[1]);
                    mma_bf16(o[i + 3], pl, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();                                   // everyone is done with this stage before it is refilled
    }
    cp_async_wait<0>();

    // Normalise, round, and store 16 bytes at a time through the warp's own rows of the first query tile.
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        if (sinks != nullptr && m_run[r] != -INFINITY) l_run[r] += ex2(fmaf(sinks[head], kLog2e, -m_run[r]));
    }
    const float inv0 = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, inv1 = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
    if (sh.out_f32) {
        // a lane's accumulators are pairs of neighbours in rows g and g + 8 of the warp's 16: 8 bytes a store, 32 in a row per quad
        float* out32 = reinterpret_cast<float*>(out);
        const int m_lo = warp * 16 + g, m_hi = m_lo + 8;
#pragma unroll
        for (int i = 0; i < kNTiles; ++i) {
            if (m_lo < rows)
                *reinterpret_cast<float2*>(out32 + ((size_t)(q0 + m0 + m_lo) * sh.Hq + head) * DV + 8 * i + 2 * t) =
                    make_float2(o[i][0] * inv0, o[i][1] * inv0);
            if (m_hi < rows)
                *reinterpret_cast<float2*>(out32 + ((size_t)(q0 + m0 + m_hi) * sh.Hq + head) * DV + 8 * i + 2 * t) =
                    make_float2(o[i][2] * inv1, o[i][3] * inv1);
        }
        return;
    }
    // (every warp has passed the loop's last barrier, so both query tiles are free: 2 * kBM * DK elements for kWarps * 16 * DV)
    unsigned char* w_s = smem + warp * 16 * (DV > DK ? DV : DK) * 2;     // [16 rows][DV] bf16, swizzled; DV <= 2 DK
#pragma unroll
    for (int i = 0; i < kNTiles; ++i) {
        const uint32_t lo_off = tile_offset<DV>(g, i) + (2 * t) * 2, hi_off = tile_offset<DV>(g + 8, i) + (2 * t) * 2;
        *reinterpret_cast<uint32_t*>(w_s + lo_off) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        *reinterpret_cast<uint32_t*>(w_s + hi_off) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 16 * kChunksV / 32; ++i) {
        const int idx = i * 32 + lane;
        const int row = idx / kChunksV, c = idx % kChunksV;
        const int m = warp * 16 + row;
        if (m < rows) {
            const uint4 v = *reinterpret_cast<const uint4*>(w_s + tile_offset<DV>(row, c));
            *reinterpret_cast<uint4*>(out + ((size_t)(q0 + m0 + m) * sh.Hq + head) * DV + c * 8) = v;
        }
    }
}

template <int DK, int DV>
int launch_general_tc(const float* q, const void* k_pool, const void* v_pool, void* out, const int* block_table, const int* cu_q,
                      const int* kv_len, const float* slopes, const float* sinks, int n_q_tiles, const TcShape& sh,
                      cudaStream_t stream) {
    static_assert(DV <= 2 * DK && DK % 16 == 0 && DV % 32 == 0 && DK >= 64 && DV >= 64, "tile shapes");
    constexpr int smem = 2 * kBM * DK * 2 + 2 * kBN * (DK + DV) * 2;
    static bool configured = false;
    if (!configured) {
        const cudaError_t rc = cudaFuncSetAttribute(general_tc_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (rc != cudaSuccess) return (int)rc;
        configured = true;
    }
    dim3 grid(n_q_tiles, sh.Hq);
    general_tc_kernel<DK, DV><<<grid, kWarps * 32, smem, stream>>>(q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, block_table,
                                                                   cu_q, kv_len, slopes, sinks, sh, pool_bounds_now());
    return launch_status();
}

}  // namespace

// Query rows per block: the caller sizes the grid as the sum over the sequences of ceil(new tokens / this).
PB_EXPORT int pb_attention_general_tc_tile(void) { return kBM; }

PB_EXPORT int pb_attention_general_tc_supported(int dtype, const void* q, const void* k_pool, const void* v_pool, int Hq, int Hkv,
                                                int Dk, int Dv, int k_stride, int v_stride) {
    if (dtype != PB_BF16 || Hkv <= 0 || Hq <= 0 || Hq % Hkv || Hq > 65535) return 0;
    if (!((Dk == 64 && Dv == 64) || (Dk == 64 && Dv == 128) || (Dk == 128 && Dv == 128) || (Dk == 192 && Dv == 128))) return 0;
    if (k_stride < Dk || v_stride < Dv || k_stride % 8 || v_stride % 8) return 0;       // rows start on 16-byte boundaries
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) % 16) return 0;
    return 1;
}

// q float32 [N, Hq, Dk]; out bfloat16 [N, Hq, Dv] (float32 with out_f32); pools bfloat16 [pages, Hkv, page_size, stride].
PB_EXPORT int pb_paged_attention_general_tc(int dtype, const float* q, const void* k_pool, const void* v_pool, void* out,
                                            const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                                            const float* slopes, int n_seqs, int n_q_tiles, int Hq, int Hkv, int Dk, int Dv,
                                            int k_stride, int v_stride, int page_size, float scale, int window, int chunk,
                                            int keep_first, float softcap, const float* sinks, int v_share, int out_f32, cudaStream_t stream) {
    if (n_seqs <= 0 || n_q_tiles <= 0) return 0;
    if (v_share <= 0 || Hkv % v_share) return PB_ERR_BAD_SIZE;
    if (!pb_attention_general_tc_supported(dtype, q, k_pool, v_pool, Hq, Hkv, Dk, Dv, k_stride, v_stride) || ((uintptr_t)out % 16))
        return PB_ERR_BAD_SIZE;
    if (page_size <= 0 || window < 0 || chunk < 0 || keep_first < 0 || !(softcap >= 0.0f)) return PB_ERR_BAD_SIZE;
    const TcShape sh{n_seqs, Hq, Hkv, k_stride, v_stride, page_size, window, chunk, table_stride, scale, keep_first, softcap, v_share,
                     out_f32 != 0};
    if (Dk == 64 && Dv == 128)
        return launch_general_tc<64, 128>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, slopes, sinks, n_q_tiles, sh, stream);
    if (Dk == 64)
        return launch_general_tc<64, 64>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, slopes, sinks, n_q_tiles, sh, stream);
    if (Dk == 128)
        return launch_general_tc<128, 128>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, slopes, sinks, n_q_tiles, sh, stream);
    return launch_general_tc<192, 128>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, slopes, sinks, n_q_tiles, sh, stream);
}

// The experts' products of a mixture of experts for steps of many tokens (bfloat16): the (token, chosen expert) pairs are
// sorted by expert on the device and every expert's rows run through tensor-core tiles against that expert's weights.
//
//   moe_sort        pairs p = token * top + slot, expert ids[p] -> offsets [E + 1] (where an expert's pairs start in the sorted
//                   order), sorted [P] (the pairs, grouped by expert), and the list of row tiles: tile t covers rows
//                   tile_row0[t] .. of expert tile_expert[t]; meta[0] = number of tiles.  One block; nothing returns to the host.
//   moe_grouped     mode 0: act[sorted row] = gated(h[token] Wg[e]^T, h[token] Wu[e]^T)   (rows gathered by pair / top)
//                   mode 1: y[sorted row] (float32) = act[sorted row] W_down[e]^T
//                   mma.sync m16n8k16, bfloat16 operands, float32 accumulators; tiles of 128 rows x 64 output columns
//                   (mode 0: 64 gate and the 64 up columns that go with them), K in steps of 64 through a three-stage cp.async
//                   pipeline.  The grid has as many row tiles as the worst case needs; blocks beyond meta[0] return at once.
//   moe_combine     out[n] = add[n] + sum over the slots, in their order, of weight[n, slot] * y[place of pair n * top + slot];
//                   float32 sums, one rounding.
// Where the sizes allow it (contraction widths that are multiples of 8, as for every tcgen05 product of this library) the two
// products run on the grouped form of the tcgen05 kernel instead (pb_gemm_tcgen05_grouped: TMA, tensor memory, the same tile
// list), with the tokens' rows gathered into sorted order first (moe_gather_rows); PULSAR_MOE_TCGEN05=0 keeps mma.sync.
// A row's result depends on that row and its expert's weights alone, so the order of the pairs inside an expert (which the
// sort leaves to the atomics) does not show in the output.
#include "mma_common.cuh"

namespace {

using namespace pb;

constexpr int kBM = 128, kBN = 64, kBK = 64, kPad = 8, kStages = 3, kThreads = 256;
constexpr int kRow = kBK + kPad;                       // shared-memory row stride in elements (144 bytes: eight rows fall on eight different 16-byte columns of the banks)

__global__ void moe_sort_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int* __restrict__ offsets,
                                int* __restrict__ sorted, int* __restrict__ place, int* __restrict__ tile_expert,
                                int* __restrict__ tile_row0, int* __restrict__ meta) {
    pdl_wait();
    extern __shared__ int sh[];                        // counts [E], cursor [E]
    int* counts = sh;
    int* cursor = sh + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&counts[ids[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < n_experts; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            for (int r = 0; r < counts[e]; r += kBM) {
                tile_expert[tiles] = e;
                tile_row0[tiles] = at + r;
                ++tiles;
            }
            at += counts[e];
        }
        offsets[n_experts] = at;
        meta[0] = tiles;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int at = atomicAdd(&cursor[ids[p]], 1);
        sorted[at] = p;
        place[p] = at;
    }
}

// rows[at] = h[sorted[at] / top]: the tokens' rows in the order of the sorted pairs, 16 bytes a thread.
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ h, const int* __restrict__ sorted, bf16* __restrict__ rows, int width,
                                       int top) {
    pdl_wait();
    const int at = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(sorted[at] / top) * width);
    uint4* dst = reinterpret_cast<uint4*>(rows + (size_t)at * width);
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src[i];
}

// MODE 0: gate/up with the gating; MODE 1: down.  Eight warps, four along the rows and two along the columns: a warp owns
// 32 rows x 32 output columns (mode 0: 32 gate columns and the 32 up columns that go with them).
template <int MODE>
__global__ void __launch_bounds__(kThreads)
moe_grouped_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, const int* __restrict__ offsets,
                   const int* __restrict__ sorted, const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                   const int* __restrict__ meta, bf16* __restrict__ act_out, float* __restrict__ y_out, int K, int n_out, int top,
                   const GatedInter gating, const float* __restrict__ in_weights) {
    pdl_wait();
    constexpr int kWRows = MODE == 0 ? 2 * kBN : kBN;
    constexpr int kParts = MODE == 0 ? 2 : 1;              // gate and up, or one
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* a_s = reinterpret_cast<bf16*>(smem_raw);                               // [stages][kBM][kRow]
    bf16* w_s = a_s + kStages * kBM * kRow;                                       // [stages][kWRows][kRow]
    __shared__ int src_row[kBM];
    const int tile = blockIdx.x;
    if (tile >= meta[0]) return;
    const int e = tile_expert[tile], row0 = tile_row0[tile];
    const int rows = min(kBM, offsets[e + 1] - row0);
    const int n0 = blockIdx.y * kBN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp >> 1, warp_n = warp & 1;
    if (tid < kBM) {
        int r = -1;
        if (tid < rows) r = MODE == 0 ? sorted[row0 + tid] / top : row0 + tid;
        src_row[tid] = r;
    }
    __syncthreads();
    const bf16* w_e = w + (size_t)e * (MODE == 0 ? 2 : 1) * n_out * K;

    auto issue = [&](int k0, int stage) {
        bf16* as = a_s + stage * kBM * kRow;
        bf16* ws = w_s + stage * kWRows * kRow;
        for (int c = tid; c < kBM * (kBK / 8); c += kThreads) {
            const int r = c / (kBK / 8), part = c % (kBK / 8);
            const int k = k0 + part * 8;
            const bool ok = src_row[r] >= 0 && k < K;
            cp_async16(smem_u32(as + r * kRow + part * 8), ok ? a + (size_t)src_row[r] * K + k : a, ok);
        }
        for (int c = tid; c < kWRows * (kBK / 8); c += kThreads) {
            const int r = c / (kBK / 8), part = c % (kBK / 8);
            const int k = k0 + part * 8;
            const int col = n0 + (r % kBN);
            const bool ok = col < n_out && k < K;
            const size_t wr = MODE == 0 ? (size_t)(r / kBN) * n_out + col : (size_t)col;      // up rows follow the gate rows
            cp_async16(smem_u32(ws + r * kRow + part * 8), ok ? w_e + wr * K + k : w_e, ok);
        }
    };

    float acc[2][4 * kParts][4];
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int i = 0; i < 4 * kParts; ++i) { acc[mi][i][0] = acc[mi][i][1] = acc[mi][i][2] = acc[mi][i][3] = 0.0f; }

    const int k_steps = (K + kBK - 1) / kBK;
#pragma unroll
    for (int st = 0; st < kStages - 1; ++st) {
        if (st < k_steps) issue(st * kBK, st);
        cp_async_commit();
    }
    for (int ks = 0; ks < k_steps; ++ks) {
        cp_async_wait<kStages - 2>();
        __syncthreads();                                   // stage ks has landed; everyone is done with stage ks - 1
        if (ks + kStages - 1 < k_steps) issue((ks + kStages - 1) * kBK, (ks + kStages - 1) % kStages);
        cp_async_commit();
        const bf16* as = a_s + (ks % kStages) * kBM * kRow;
        const bf16* ws = w_s + (ks % kStages) * kWRows * kRow;
        if (warp_m * 32 < rows) {
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk) {
                uint32_t af[2][4];
#pragma unroll
                for (int mi = 0; mi < 2; ++mi)
                    ldmatrix_x4(af[mi], smem_u32(as + (warp_m * 32 + mi * 16 + (lane & 15)) * kRow + kk * 16 + (lane >> 4) * 8));
#pragma unroll
                for (int part = 0; part < kParts; ++part)
#pragma unroll
                    for (int nn = 0; nn < 2; ++nn) {
                        uint32_t bfr[4];
                        const int r = part * kBN + warp_n * 32 + nn * 16 + (lane & 7) + ((lane >> 4) << 3);
                        ldmatrix_x4(bfr, smem_u32(ws + r * kRow + kk * 16 + ((lane >> 3) & 1) * 8));
#pragma unroll
                        for (int mi = 0; mi < 2; ++mi) {
                            mma_bf16(acc[mi][part * 4 + 2 * nn], af[mi], bfr[0], bfr[1]);
                            mma_bf16(acc[mi][part * 4 + 2 * nn + 1], af[mi], bfr[2], bfr[3]);
                        }
                    }
            }
        }
    }
    cp_async_wait<0>();

    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = warp_m * 32 + mi * 16 + g + half * 8;
            if (r >= rows) continue;
            if (MODE == 0) {
                bf16* dst = act_out + (size_t)(row0 + r) * n_out;
                const float ws = in_weights ? in_weights[sorted[row0 + r]] : 1.0f;     // the pair's weight on the expert's input
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int col = n0 + warp_n * 32 + j * 8 + 2 * t;
                    const float v0 = gated(ws * acc[mi][j][2 * half], ws * acc[mi][j + 4 * (kParts - 1)][2 * half], gating);
                    const float v1 = gated(ws * acc[mi][j][2 * half + 1], ws * acc[mi][j + 4 * (kParts - 1)][2 * half + 1], gating);
                    if (col + 1 < n_out && (n_out & 1) == 0) *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(v0, v1);
                    else {
                        if (col < n_out) dst[col] = __float2bfloat16_rn(v0);
                        if (col + 1 < n_out) dst[col + 1] = __float2bfloat16_rn(v1);
                    }
                }
            } else {
                float* dst = y_out + (size_t)(row0 + r) * n_out;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int col = n0 + warp_n * 32 + j * 8 + 2 * t;
                    if (col + 1 < n_out && (n_out & 1) == 0) *reinterpret_cast<float2*>(dst + col) = make_float2(acc[mi][j][2 * half], acc[mi][j][2 * half + 1]);
                    else {
                        if (col < n_out) dst[col] = acc[mi][j][2 * half];
                        if (col + 1 < n_out) dst[col + 1] = acc[mi][j][2 * half + 1];
                    }
                }
            }
        }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                   const bf16* __restrict__ add, const float* __restrict__ add_scale, bf16* __restrict__ out, int width,
                                   int top, size_t total) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / width, c = i % width;
        float sum = add ? __bfloat162float(add[i]) * (add_scale ? add_scale[n] : 1.0f) : 0.0f;
        for (int slot = 0; slot < top; ++slot)
            sum = fmaf(weights ? weights[n * top + slot] : 1.0f, y[(size_t)place[n * top + slot] * width + c], sum);
        out[i] = __float2bfloat16_rn(sum);
    }
}

}  // namespace

// Ints of the workspace that pb_moe_grouped needs for n tokens: offsets [E + 1], sorted [n * top], tile lists, meta.
PB_EXPORT int pb_moe_grouped_workspace(int n, int top, int n_experts) {
    const int pairs = n * top, tiles = (pairs + kBM - 1) / kBM + n_experts;
    return (n_experts + 1) + 2 * pairs + 2 * tiles + 4;
}

// 1 when the grouped products take these sizes: contraction widths that are multiples of 8 (16-byte rows).
PB_EXPORT int pb_moe_grouped_supported(int width, int ff, int n_experts) {
    return (width > 0 && ff > 0 && width % 8 == 0 && ff % 8 == 0 && n_experts > 0 && n_experts <= 4096) ? 1 : 0;
}

// h [n, width], w_gate_up [E, 2 ff, width], w_down [E, width, ff], add [n, width] or null, out [n, width]: bfloat16;
// ids int32 [n, top], weights float32 [n, top]; act bfloat16 [n * top, ff] and y float32 [n * top, width] scratch;
// work: int32 scratch of pb_moe_grouped_workspace(n, top, E) elements.  limit <= 0: no clamp.  gathered: bfloat16
// [n * top, width] scratch for the tcgen05 form, or null for the mma.sync form.
PB_EXPORT int pb_gemm_tcgen05_grouped(int mode, int out_dtype, const void* x, const void* w, void* out, int P, int N, int K,
                                      int n_groups, const int* offsets, const int* tile_group, const int* tile_row0, const int* meta,
                                      int max_row_tiles, float limit, float alpha, float shift, const int* row_pair,
                                      const float* pair_scale, cudaStream_t stream);

PB_EXPORT int pb_moe_grouped(const void* h, const void* w_gate_up, const void* w_down, const int* ids, const float* weights,
                             const void* add, void* act, float* y, void* out, int* work, void* gathered, int n, int width, int ff,
                             int n_experts, int top, float limit, float alpha, float shift, int weight_input, const float* add_scale,
                             cudaStream_t stream) {
    if (n <= 0) return 0;
    // weight_input: a pair's weight multiplies its expert's input (in the gate/up epilogue: W (w h) = w (W h)) and the sum
    // over a token's experts takes every pair once; add_scale (float32 [n] or null) multiplies `add`.
    const float* in_weights = weight_input ? weights : nullptr;
    const float* out_weights = weight_input ? nullptr : weights;
    if (!pb_moe_grouped_supported(width, ff, n_experts) || top <= 0 || top > n_experts) return PB_ERR_BAD_SIZE;
    const int pairs = n * top, tiles = (pairs + kBM - 1) / kBM + n_experts;
    if (tiles > 0x7fffffff / 2 || (ff + kBN - 1) / kBN > 65535 || (width + kBN - 1) / kBN > 65535) return PB_ERR_TOO_LARGE;
    int* offsets = work;
    int* sorted = offsets + n_experts + 1;
    int* place = sorted + pairs;
    int* tile_expert = place + pairs;
    int* tile_row0 = tile_expert + tiles;
    int* meta = tile_row0 + tiles;
    int rc = launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), sizeof(int) * 2 * n_experts, stream, ids, pairs, n_experts, offsets, sorted,
                        place, tile_expert, tile_row0, meta);
    if (rc != 0) return rc;
    const size_t total = (size_t)n * width;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (gathered != nullptr) {
        // the tcgen05 form: rows gathered into sorted order, then the two grouped products over the same tile list
        int threads = width / 8;
        threads = threads > 256 ? 256 : (threads + 31) / 32 * 32;
        rc = launch_pdl(moe_gather_rows_kernel, dim3(pairs), dim3(threads), 0, stream, (const bf16*)h, (const int*)sorted, (bf16*)gathered,
                        width, top);
        if (rc != 0) return rc;
        rc = pb_gemm_tcgen05_grouped(1, PB_BF16, gathered, w_gate_up, act, pairs, 2 * ff, width, n_experts, offsets, tile_expert, tile_row0,
                                     meta, tiles, limit, alpha, shift, sorted, in_weights, stream);
        if (rc != 0) return rc;
        rc = pb_gemm_tcgen05_grouped(0, PB_F32, act, w_down, y, pairs, width, ff, n_experts, offsets, tile_expert, tile_row0, meta, tiles,
                                     0.0f, 1.0f, 0.0f, nullptr, nullptr, stream);
        if (rc != 0) return rc;
        return launch_pdl(moe_combine_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)y, (const int*)place, out_weights,
                          (const bf16*)add, add_scale, (bf16*)out, width, top, total);
    }
    const GatedInter gating(ff, limit > 0.0f ? limit : __builtin_huge_valf(), alpha, shift);
    constexpr int smem0 = kStages * (kBM + 2 * kBN) * kRow * 2, smem1 = kStages * (kBM + kBN) * kRow * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t ce = cudaFuncSetAttribute(moe_grouped_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem0);
        if (ce == cudaSuccess) ce = cudaFuncSetAttribute(moe_grouped_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1);
        if (ce != cudaSuccess) return (int)ce;
        configured = true;
    }
    rc = launch_pdl(moe_grouped_kernel<0>, dim3(tiles, (ff + kBN - 1) / kBN), dim3(kThreads), smem0, stream, (const bf16*)h, (const bf16*)w_gate_up,
                    (const int*)offsets, (const int*)sorted, (const int*)tile_expert, (const int*)tile_row0, (const int*)meta, (bf16*)act,
                    (float*)nullptr, width, ff, top, gating, in_weights);
    if (rc != 0) return rc;
    rc = launch_pdl(moe_grouped_kernel<1>, dim3(tiles, (width + kBN - 1) / kBN), dim3(kThreads), smem1, stream, (const bf16*)act,
                    (const bf16*)w_down, (const int*)offsets, (const int*)sorted, (const int*)tile_expert, (const int*)tile_row0,
                    (const int*)meta, (bf16*)nullptr, y, ff, width, top, gating, (const float*)nullptr);
    if (rc != 0) return rc;
    return launch_pdl(moe_combine_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)y, (const int*)place, out_weights,
                      (const bf16*)add, add_scale, (bf16*)out, width, top, total);
}

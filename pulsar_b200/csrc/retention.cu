// Retention: linear attention with a fixed decay per head, a float32 state matrix per (sequence, head), no softmax.
//
//   S_t = decay_h S_(t-1) + k_t v_t^T        S [D, V] float32, kept per sequence in a state slot, zero at the start
//   o_t = S_t^T q_t                          [V]
//   y_t = o_t / sqrt(mean(o_t^2) + eps) * silu(g_t)      per head; written in the activation dtype
//
// `rows` float32 [N, stride] holds, per token, q (H*D) | k (H*D) | v (H*V) | g (H*V) as the fused projection left them.
//
//   retention_prepare   q and k of every (token, head): the first `rotary` dimensions turn in the rotate-half layout
//                       (element i pairs with element i + rotary/2) by cos/sin [N, rotary/2]; k is multiplied by k_scale
//                       afterwards; both go to float32 [N, H, D].
//   retention_step      token by token: a block per (head, sequence); thread (v, slice) holds the slice's rows of column v
//                       of S in registers, so a token costs one pass over the state.  Decoding and short portions.
//   retention_chunk_*   portions in chunks of kChunk tokens, parallel over chunks:
//                         state   U_c = sum_j decay^(n-1-j) k_j v_j^T over the chunk's n tokens          (per chunk, head)
//                         fold    S_in(c) = state entering chunk c; S <- decay^n S + U_c along a sequence  (per element)
//                         out     o_i = sum_(j<=i) decay^(i-j) (q_i . k_j) v_j + decay^(i+1) S_in^T q_i, then norm and gate
//                       A token's value differs from the token-by-token one by rounding only.
// All arithmetic is float32 on CUDA cores.
#include "common.cuh"

namespace {

using namespace pb;

constexpr int kChunk = 32;
constexpr int kPowers = kChunk + 4;        // room for decay^0 .. decay^kChunk, a multiple of four floats
constexpr int kStateRows = 32;           // rows of the entering state that a block stages at a time

__global__ void retention_prepare_kernel(const float* __restrict__ rows, long stride, const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t, float* __restrict__ q_out, float* __restrict__ k_out,
                                         int H, int D, int rotary, float k_scale) {
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int hh = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);          // query heads, then key heads
    if (hh >= 2 * H) return;
    const bool is_k = hh >= H;
    const float* src = rows + (size_t)t * stride + (size_t)hh * D;
    float* dst = (is_k ? k_out : q_out) + ((size_t)t * H + (is_k ? hh - H : hh)) * D;
    const float f = is_k ? k_scale : 1.0f;
    const int half = rotary >> 1;
    const float* c = cos_t + (size_t)t * half;
    const float* s = sin_t + (size_t)t * half;
    for (int i = lane; i < half; i += 32) {
        const float u = src[i], v = src[i + half];
        dst[i] = (u * c[i] - v * s[i]) * f;
        dst[i + half] = (v * c[i] + u * s[i]) * f;
    }
    for (int i = rotary + lane; i < D; i += 32) dst[i] = src[i] * f;
}

template <typename T, int PER, int THREADS>
__global__ void __launch_bounds__(THREADS) retention_step_kernel(const float* __restrict__ qr, const float* __restrict__ kr, const float* __restrict__ rows,
                                      long stride, int v_off, int g_off, const float* __restrict__ decay, float* __restrict__ state,
                                      long state_stride, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                      T* __restrict__ y, int H, int D, int V, int DS, float eps) {
    pdl_wait();
    extern __shared__ float smem[];
    float* qs = smem;                        // [D]
    float* ks = qs + D;                      // [D]
    float* part = ks + D;                    // [DS][V]
    float* red = part + (size_t)DS * V;      // [32]
    const int h = blockIdx.x, s = blockIdx.y, tid = threadIdx.x;
    const int v = tid % V, ds = tid / V;
    const bool on = ds < DS;
    const int d0 = ds * PER;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    const float dec = decay[h];
    float* kept = state + (size_t)state_slots[s] * state_stride + (size_t)h * D * V;
    float S[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) S[i] = (on && d0 + i < D) ? kept[(size_t)(d0 + i) * V + v] : 0.0f;
    for (int t = t0; t < t1; ++t) {
        const float* q_row = qr + ((size_t)t * H + h) * D;
        const float* k_row = kr + ((size_t)t * H + h) * D;
        for (int i = tid; i < D; i += blockDim.x) { qs[i] = q_row[i]; ks[i] = k_row[i]; }
        const float vv = on ? rows[(size_t)t * stride + v_off + (size_t)h * V + v] : 0.0f;
        __syncthreads();
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if (d0 + i < D) {
                S[i] = fmaf(dec, S[i], ks[d0 + i] * vv);
                acc = fmaf(S[i], qs[d0 + i], acc);
            }
        }
        if (on) part[ds * V + v] = acc;
        __syncthreads();
        float o = 0.0f;
        if (ds == 0)
            for (int k = 0; k < DS; ++k) o += part[k * V + v];
        const float ss = block_sum(o * o, red);
        if (ds == 0) {
            const float g = rows[(size_t)t * stride + g_off + (size_t)h * V + v];
            y[(size_t)t * H * V + (size_t)h * V + v] = from_float<T>(o * rsqrtf(ss / (float)V + eps) * (g / (1.0f + expf(-g))));
        }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i)
        if (on && d0 + i < D) kept[(size_t)(d0 + i) * V + v] = S[i];
}

// The chunk `chunk` of a step whose sequence s has ceil(q_len / kChunk) chunks: its sequence and tokens [t0, t1).
__device__ __forceinline__ bool find_chunk(const int* cu_q, int n_seqs, int chunk, int& s, int& t0, int& t1) {
    int base = 0;
    for (s = 0; s < n_seqs; ++s) {
        const int q0 = cu_q[s], len = cu_q[s + 1] - q0;
        const int nc = (len + kChunk - 1) / kChunk;
        if (chunk < base + nc) {
            t0 = q0 + (chunk - base) * kChunk;
            t1 = min(t0 + kChunk, q0 + len);
            return true;
        }
        base += nc;
    }
    return false;
}

// U [chunks, H, D, V]: what the chunk's own tokens leave in a state that was zero before them.
__global__ void retention_chunk_state_kernel(const float* __restrict__ kr, const float* __restrict__ rows, long stride, int v_off,
                                             const float* __restrict__ decay, const int* __restrict__ cu_q, int n_seqs,
                                             float* __restrict__ U, int H, int D, int V) {
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    const int Dp = (D + 3) & ~3, Vp = (V + 3) & ~3;
    float* ks = smem;                        // [kChunk][Dp], weighted
    float* vs = ks + kChunk * Dp;            // [kChunk][Vp]
    const int chunk = blockIdx.x, h = blockIdx.y;
    int s, t0, t1;
    if (!find_chunk(cu_q, n_seqs, chunk, s, t0, t1)) return;
    const int n = t1 - t0;
    const float dec = decay[h];
    for (int i = threadIdx.x; i < kChunk * Dp; i += blockDim.x) {
        const int j = i / Dp, d = i - j * Dp;
        ks[i] = (j < n && d < D) ? kr[((size_t)(t0 + j) * H + h) * D + d] * powf(dec, (float)(n - 1 - j)) : 0.0f;
    }
    for (int i = threadIdx.x; i < kChunk * Vp; i += blockDim.x) {
        const int j = i / Vp, v = i - j * Vp;
        vs[i] = (j < n && v < V) ? rows[(size_t)(t0 + j) * stride + v_off + (size_t)h * V + v] : 0.0f;
    }
    __syncthreads();
    float* out = U + ((size_t)chunk * H + h) * D * V;
    const int tiles_v = Vp >> 2, tiles = (Dp >> 2) * tiles_v;
    for (int tile = threadIdx.x; tile < tiles; tile += blockDim.x) {
        const int d = (tile / tiles_v) << 2, v = (tile % tiles_v) << 2;
        float acc[4][4] = {};
        for (int j = 0; j < n; ++j) {
            const float4 a = *reinterpret_cast<const float4*>(ks + j * Dp + d);
            const float4 b = *reinterpret_cast<const float4*>(vs + j * Vp + v);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int z = 0; z < 4; ++z) acc[x][z] = fmaf(av[x], bv[z], acc[x][z]);
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int z = 0; z < 4; ++z)
                if (d + x < D && v + z < V) out[(size_t)(d + x) * V + v + z] = acc[x][z];
    }
}

// Along a sequence's chunks: U_c is replaced by the state that enters chunk c; the state behind the last chunk is kept.
__global__ void retention_fold_kernel(float* __restrict__ U, const float* __restrict__ decay, float* __restrict__ state,
                                      long state_stride, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                      int H, int DV) {
    pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, s = blockIdx.z;
    if (e >= DV) return;
    int first = 0;
    for (int i = 0; i < s; ++i) first += (cu_q[i + 1] - cu_q[i] + kChunk - 1) / kChunk;
    const int len = cu_q[s + 1] - cu_q[s];
    const int nc = (len + kChunk - 1) / kChunk;
    const float dec = decay[h];
    const float full = powf(dec, (float)kChunk);
    float* kept = state + (size_t)state_slots[s] * state_stride + (size_t)h * DV + e;
    float S = *kept;
    float* u0 = U + ((size_t)first * H + h) * DV + e;
    const size_t step = (size_t)H * DV;
    constexpr int kAhead = 8;                // chunks whose own parts are in flight together: they do not depend on the fold
    for (int c0 = 0; c0 < nc; c0 += kAhead) {
        float own[kAhead];
#pragma unroll
        for (int k = 0; k < kAhead; ++k) own[k] = c0 + k < nc ? u0[(size_t)(c0 + k) * step] : 0.0f;
#pragma unroll
        for (int k = 0; k < kAhead; ++k) {
            if (c0 + k < nc) {
                u0[(size_t)(c0 + k) * step] = S;
                const int n = min(kChunk, len - (c0 + k) * kChunk);
                S = fmaf(n == kChunk ? full : powf(dec, (float)n), S, own[k]);
            }
        }
    }
    *kept = S;
}

template <typename T>
__global__ void retention_chunk_out_kernel(const float* __restrict__ qr, const float* __restrict__ kr, const float* __restrict__ rows,
                                           long stride, int v_off, int g_off, const float* __restrict__ decay,
                                           const int* __restrict__ cu_q, int n_seqs, const float* __restrict__ S_in,
                                           T* __restrict__ y, int H, int D, int V, float eps) {
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    const int Dp = (D + 3) & ~3, Vp = (V + 3) & ~3;
    const int Dq = Dp + 4;                   // row stride of q and k: rows a multiple of 32 floats apart would share their banks
    float* qs = smem;                        // [kChunk][Dq]
    float* ks = qs + kChunk * Dq;            // [kChunk][Dq]
    float* vs = ks + kChunk * Dq;            // [kChunk][Vp]
    float* os = vs + kChunk * Vp;            // [kChunk][Vp]
    float* A = os + kChunk * Vp;             // [kChunk][kChunk]
    float* pw = A + kChunk * kChunk;         // [kPowers]: decay^m, m <= kChunk
    float* st = pw + kPowers;                // [kStateRows][Vp]: rows of the entering state
    const int chunk = blockIdx.x, h = blockIdx.y;
    int s, t0, t1;
    if (!find_chunk(cu_q, n_seqs, chunk, s, t0, t1)) return;
    const int n = t1 - t0;
    const float dec = decay[h];
    for (int i = threadIdx.x; i <= kChunk; i += blockDim.x) pw[i] = powf(dec, (float)i);
    for (int i = threadIdx.x; i < kChunk * Dq; i += blockDim.x) {
        const int j = i / Dq, d = i - j * Dq;
        const bool in = j < n && d < D;
        qs[i] = in ? qr[((size_t)(t0 + j) * H + h) * D + d] : 0.0f;
        ks[i] = in ? kr[((size_t)(t0 + j) * H + h) * D + d] : 0.0f;
    }
    for (int i = threadIdx.x; i < kChunk * Vp; i += blockDim.x) {
        const int j = i / Vp, v = i - j * Vp;
        vs[i] = (j < n && v < V) ? rows[(size_t)(t0 + j) * stride + v_off + (size_t)h * V + v] : 0.0f;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < kChunk * kChunk; e += blockDim.x) {
        const int i = e / kChunk, j = e - i * kChunk;
        float dot = 0.0f;
        if (j <= i && i < n) {
            const float* a = qs + i * Dq;
            const float* b = ks + j * Dq;
            for (int d = 0; d < Dp; d += 4) {
                const float4 x = *reinterpret_cast<const float4*>(a + d), z = *reinterpret_cast<const float4*>(b + d);
                dot = fmaf(x.x, z.x, dot); dot = fmaf(x.y, z.y, dot); dot = fmaf(x.z, z.z, dot); dot = fmaf(x.w, z.w, dot);
            }
            dot *= pw[i - j];
        }
        A[e] = dot;
    }
    __syncthreads();
    const float* Sc = S_in + ((size_t)chunk * H + h) * D * V;
    const bool vec_s = (V & 3) == 0;
    const int tiles_v = Vp >> 2, tiles = (kChunk >> 2) * tiles_v;
    // A thread owns a 4 x 4 tile of the outputs (rows i0 .., columns v ..); where there are more tiles than threads the block
    // walks them in passes.  The entering state comes through shared memory, kStateRows rows at a time, fetched by the whole
    // block with all its loads in flight together, so its latency is paid once per group of rows.
    for (int pass = 0; pass * (int)blockDim.x < tiles; ++pass) {
        const int tile = pass * blockDim.x + threadIdx.x;
        const int i0 = (tile / tiles_v) << 2, v = (tile % tiles_v) << 2;
        const bool mine = tile < tiles && i0 < n;
        float inner[4][4] = {}, carried[4][4] = {};
        if (mine) {
            // four keys at a time: eight 16-byte loads feed 64 multiply-adds.  Scores of keys behind a query and rows behind
            // the chunk's last token are zero, so a group of four may reach past them.
            for (int j = 0; j < i0 + 4; j += 4) {
                float a[4][4], b[4][4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float4 t = *reinterpret_cast<const float4*>(A + (i0 + x) * kChunk + j);
                    a[x][0] = t.x; a[x][1] = t.y; a[x][2] = t.z; a[x][3] = t.w;
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float4 t = *reinterpret_cast<const float4*>(vs + (j + k) * Vp + v);
                    b[k][0] = t.x; b[k][1] = t.y; b[k][2] = t.z; b[k][3] = t.w;
                }
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                    for (int x = 0; x < 4; ++x)
#pragma unroll
                        for (int z = 0; z < 4; ++z) inner[x][z] = fmaf(a[x][k], b[k][z], inner[x][z]);
            }
        }
        for (int dt = 0; dt < D; dt += kStateRows) {
            __syncthreads();                 // the rows staged before have been read
            for (int i = threadIdx.x; i < kStateRows * tiles_v; i += blockDim.x) {
                const int r = i / tiles_v, c = (i - r * tiles_v) << 2;
                float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (dt + r < D) {
                    const float* src = Sc + (size_t)(dt + r) * V + c;
                    if (vec_s) {
                        t = *reinterpret_cast<const float4*>(src);
                    } else {
                        t.x = src[0];
                        if (c + 1 < V) t.y = src[1];
                        if (c + 2 < V) t.z = src[2];
                        if (c + 3 < V) t.w = src[3];
                    }
                }
                *reinterpret_cast<float4*>(st + r * Vp + c) = t;
            }
            __syncthreads();
            if (mine) {
                const int rows_here = min(kStateRows, Dp - dt);          // a multiple of four; q is zero from D on
                for (int d = 0; d < rows_here; d += 4) {
                    float a[4][4], b[4][4];
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float4 t = *reinterpret_cast<const float4*>(qs + (i0 + x) * Dq + dt + d);
                        a[x][0] = t.x; a[x][1] = t.y; a[x][2] = t.z; a[x][3] = t.w;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float4 t = *reinterpret_cast<const float4*>(st + (d + k) * Vp + v);
                        b[k][0] = t.x; b[k][1] = t.y; b[k][2] = t.z; b[k][3] = t.w;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k)
#pragma unroll
                        for (int x = 0; x < 4; ++x)
#pragma unroll
                            for (int z = 0; z < 4; ++z) carried[x][z] = fmaf(a[x][k], b[k][z], carried[x][z]);
                }
            }
        }
        if (mine) {
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int z = 0; z < 4; ++z) os[(i0 + x) * Vp + v + z] = fmaf(pw[i0 + x + 1], carried[x][z], inner[x][z]);
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = warp; i < n; i += warps) {
        float ss = 0.0f;
        for (int v = lane; v < V; v += 32) ss += os[i * Vp + v] * os[i * Vp + v];
        const float r = rsqrtf(warp_sum(ss) / (float)V + eps);
        const float* g_row = rows + (size_t)(t0 + i) * stride + g_off + (size_t)h * V;
        T* out = y + (size_t)(t0 + i) * H * V + (size_t)h * V;
        for (int v = lane; v < V; v += 32) {
            const float g = g_row[v];
            out[v] = from_float<T>(os[i * Vp + v] * r * (g / (1.0f + expf(-g))));
        }
    }
}

template <typename K>
int allow_smem(K kernel, size_t smem) {
    if (smem <= 48 * 1024) return 0;
    if (smem > 200 * 1024) return PB_ERR_TOO_LARGE;
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

template <typename T, int PER, int THREADS>
int launch_step(const float* qr, const float* kr, const float* rows, long stride, int v_off, int g_off, const float* decay,
                float* state, long state_stride, const int* cu_q, const int* state_slots, void* y, int n_seqs, int H, int D, int V,
                float eps, cudaStream_t stream) {
    const int DS = (D + PER - 1) / PER;
    const int threads = (V * DS + 31) / 32 * 32;
    const size_t smem = sizeof(float) * (2 * (size_t)D + (size_t)DS * V + 32);
    if (threads > THREADS) return PB_ERR_TOO_LARGE;
    const int rc = allow_smem(retention_step_kernel<T, PER, THREADS>, smem);
    if (rc != 0) return rc;
    return launch_pdl(retention_step_kernel<T, PER, THREADS>, dim3(H, n_seqs), dim3(threads), smem, stream, qr, kr, rows, stride, v_off, g_off,
                      decay, state, state_stride, cu_q, state_slots, (T*)y, H, D, V, DS, eps);
}

template <typename T>
int dispatch_step(const float* qr, const float* kr, const float* rows, long stride, int v_off, int g_off, const float* decay,
                  float* state, long state_stride, const int* cu_q, const int* state_slots, void* y, int n_seqs, int H, int D, int V,
                  float eps, cudaStream_t stream) {
    // the fewest rows of a column per thread that keep the block within 512 threads (256 where a thread holds 64 rows: the
    // registers of a block are 64 K)
#define PB_STEP(PER, THREADS) return launch_step<T, PER, THREADS>(qr, kr, rows, stride, v_off, g_off, decay, state, state_stride, cu_q, \
                                                                 state_slots, y, n_seqs, H, D, V, eps, stream)
    if (V * ((D + 7) / 8) <= 512) PB_STEP(8, 512);
    if (V * ((D + 15) / 16) <= 512) PB_STEP(16, 512);
    if (V * ((D + 31) / 32) <= 512) PB_STEP(32, 512);
    if (V * ((D + 63) / 64) <= 256) PB_STEP(64, 256);
#undef PB_STEP
    return PB_ERR_TOO_LARGE;
}

bool step_fits(int D, int V) { return V * ((D + 31) / 32) <= 512 || V * ((D + 63) / 64) <= 256; }

}  // namespace

PB_EXPORT int pb_retention_chunk() { return kChunk; }

// Whether the token-by-token kernel holds a head's state of these sizes in one block's registers; where it does not, every
// step takes the form in chunks (a single token is a chunk of one).
PB_EXPORT int pb_retention_step_supported(int D, int V) { return D > 0 && V > 0 && step_fits(D, V) ? 1 : 0; }

// rows float32 [n, stride]: q (H*D) | k (H*D) | v (H*V) | g (H*V); cos/sin float32 [n, rotary/2]; qr, kr float32 [n, H, D]
// (workspace); decay float32 [H]; state: float32 rows of state_stride elements per slot, the first H*D*V are this mixer's
// [H, D, V]; y [n, H*V] in `dtype`.  max_chunks > 0: the form that is parallel over chunks, with workspace U
// [max_chunks, H, D, V] float32 (max_chunks >= the sum over the step's sequences of ceil(q_len / pb_retention_chunk())).
PB_EXPORT int pb_retention(int dtype, const float* rows, long stride, const float* cos_t, const float* sin_t, float* qr, float* kr,
                           const float* decay, float* state, long state_stride, const int* cu_q, const int* state_slots, void* y,
                           int n, int n_seqs, int H, int D, int V, int rotary, float k_scale, float eps, int max_chunks, float* U,
                           cudaStream_t stream) {
    if (n <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || rotary < 0 || rotary > D || (rotary & 1) || stride < (long)2 * H * (D + V) ||
        state_stride < (long)H * D * V || (rotary > 0 && (cos_t == nullptr || sin_t == nullptr)))
        return PB_ERR_BAD_SIZE;
    if (dtype != PB_F32 && dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
    if (n_seqs > 65535 || H > 65535 || max_chunks > 65535 * 32) return PB_ERR_TOO_LARGE;
    const int v_off = 2 * H * D, g_off = 2 * H * D + H * V;
    const int warps = 4;
    int rc = launch_pdl(retention_prepare_kernel, dim3(n, (2 * H + warps - 1) / warps), dim3(warps * 32), 0, stream, rows, stride, cos_t,
                        sin_t, qr, kr, H, D, rotary, k_scale);
    if (rc != 0) return rc;
    if (max_chunks <= 0) {
        if (!step_fits(D, V)) return PB_ERR_TOO_LARGE;
        if (dtype == PB_F32)
            return dispatch_step<float>(qr, kr, rows, stride, v_off, g_off, decay, state, state_stride, cu_q, state_slots, y, n_seqs, H, D,
                                        V, eps, stream);
        return dispatch_step<__nv_bfloat16>(qr, kr, rows, stride, v_off, g_off, decay, state, state_stride, cu_q, state_slots, y, n_seqs,
                                            H, D, V, eps, stream);
    }
    if (U == nullptr) return PB_ERR_BAD_SIZE;
    const int Dp = (D + 3) & ~3, Vp = (V + 3) & ~3;
    const size_t smem_state = sizeof(float) * kChunk * ((size_t)Dp + Vp);
    rc = allow_smem(retention_chunk_state_kernel, smem_state);
    if (rc != 0) return rc;
    rc = launch_pdl(retention_chunk_state_kernel, dim3(max_chunks, H), dim3(256), smem_state, stream, (const float*)kr, rows, stride, v_off,
                    decay, cu_q, n_seqs, U, H, D, V);
    if (rc != 0) return rc;
    const int DV = D * V;
    rc = launch_pdl(retention_fold_kernel, dim3((DV + 255) / 256, H, n_seqs), dim3(256), 0, stream, U, decay, state, state_stride, cu_q,
                    state_slots, H, DV);
    if (rc != 0) return rc;
    const size_t smem_out = sizeof(float) * (kChunk * (2 * (size_t)(Dp + 4) + 2 * (size_t)Vp) + kChunk * kChunk + kPowers + kStateRows * (size_t)Vp);
    if (dtype == PB_F32) {
        rc = allow_smem(retention_chunk_out_kernel<float>, smem_out);
        if (rc != 0) return rc;
        return launch_pdl(retention_chunk_out_kernel<float>, dim3(max_chunks, H), dim3(256), smem_out, stream, (const float*)qr,
                          (const float*)kr, rows, stride, v_off, g_off, decay, cu_q, n_seqs, (const float*)U, (float*)y, H, D, V, eps);
    }
    rc = allow_smem(retention_chunk_out_kernel<__nv_bfloat16>, smem_out);
    if (rc != 0) return rc;
    return launch_pdl(retention_chunk_out_kernel<__nv_bfloat16>, dim3(max_chunks, H), dim3(256), smem_out, stream, (const float*)qr,
                      (const float*)kr, rows, stride, v_off, g_off, decay, cu_q, n_seqs, (const float*)U, (__nv_bfloat16*)y, H, D, V, eps);
}

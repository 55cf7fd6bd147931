// A mixture of gated experts: the router, and the experts' products for steps of a few tokens.
//
//   moe_route      z = W_r h in float32 (W_r float32 [E, width]; h in the activation dtype), s = sigmoid(z), the `top`
//                  largest s per token (ties: the lower index), weights s * scale, or with `renormalize` s / sum of the
//                  chosen s * scale.  ids int32 [N, top] in descending order of s, weights float32 [N, top].
//                  With `softmax` the scores are s = softmax(z) over all experts instead, and a renormalised weight is
//                  s / (sum of the chosen s + renorm_eps) * scale.
//   moe_gate_up    for every (token, chosen expert): g = W_gate[e] h, u = W_up[e] h (float32 sums), the gated unit
//                  out = g' * sigmoid(alpha * g') * (u' + shift) with g' = min(g, limit), u' = clamp(u, -limit, limit),
//                  one rounding on store: act [N * top, ff].  Weights [E, 2 ff, width]: an expert's gate rows, then
//                  its up rows.
//   moe_down       out[n] = add[n] + sum over the chosen experts, in the order of ids, of weight * (W_down[e] act[n, slot]);
//                  float32 sums, one rounding on store.  Weights [E, width, ff].  `add` (optional): what a shared
//                  expert contributed.
// A warp owns one output element and walks the contraction in a fixed order, so a token's result does not depend on
// what else is in the step.  These kernels read an expert's weights once per token that chose it: they are for steps
// of a few tokens (and for the float32 engine); larger steps sort the tokens by expert and take the grouped product.
#include "common.cuh"

namespace {

using namespace pb;

__device__ __forceinline__ void load_chunk(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void load_chunk(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
}
constexpr int kRouteRows = 4;            // router rows a warp walks side by side: their loads are in flight together

__device__ __forceinline__ void fma4(float& z, const float4& a, const float4& x) {
    z = fmaf(a.x, x.x, z); z = fmaf(a.y, x.y, z); z = fmaf(a.z, x.z, z); z = fmaf(a.w, x.w, z);
}

// One block per TOK tokens; a warp takes kRouteRows rows of the router at a time (groups strided over the warps), reads
// each once, 16 bytes a lane with two chunks per row in flight, and adds it up against each of the block's tokens, whose
// float32 rows sit in shared memory and are read once for the group's rows.  A token's sums run in an order that depends
// on the width alone, not on TOK or on which tokens share its block.
template <typename T, int TOK>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, int* __restrict__ ids,
                                 float* __restrict__ weights, int n, int width, int n_experts, int top, float scale,
                                 int renormalize, int n_extra, float* __restrict__ extra, int softmax, float renorm_eps) {
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    float* x = smem;                                     // [TOK][width]
    float* s = smem + (size_t)TOK * width;               // [TOK][n_experts + n_extra]
    const int n_rows = n_experts + n_extra;              // the rows behind the experts' compete for nothing: their sigmoids go to `extra`
    const int t0 = blockIdx.x * TOK, n_tok = min(TOK, n - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    constexpr int kPer = 16 / (int)sizeof(T);            // elements of a 16-byte load
    if (width % kPer == 0 && ((uintptr_t)h & 15) == 0) {
        const int chunks = width / kPer;
        for (int i = threadIdx.x; i < TOK * chunks; i += blockDim.x) {
            const int k = i / chunks, c = i - k * chunks;
            float f[kPer];
            if (k < n_tok) {
                load_chunk(h + (size_t)(t0 + k) * width + c * kPer, f);
            } else {
#pragma unroll
                for (int j = 0; j < kPer; ++j) f[j] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < kPer; j += 4)
                *reinterpret_cast<float4*>(x + k * width + c * kPer + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
        }
    } else {
#pragma unroll
        for (int k = 0; k < TOK; ++k)
            for (int i = threadIdx.x; i < width; i += blockDim.x)
                x[k * width + i] = k < n_tok ? to_float(h[(size_t)(t0 + k) * width + i]) : 0.0f;
    }
    __syncthreads();
    const bool vec = (width & 3) == 0 && ((uintptr_t)router & 15) == 0;
    const int n_groups = (n_rows + kRouteRows - 1) / kRouteRows;
    for (int grp = warp; grp < n_groups; grp += warps) {
        const int e0 = grp * kRouteRows;
        const float* w[kRouteRows];
#pragma unroll
        for (int r = 0; r < kRouteRows; ++r) w[r] = router + (size_t)min(e0 + r, n_rows - 1) * width;
        float z[kRouteRows][TOK];
#pragma unroll
        for (int r = 0; r < kRouteRows; ++r)
#pragma unroll
            for (int k = 0; k < TOK; ++k) z[r][k] = 0.0f;
        if (vec) {
            int i = lane * 4;
            for (; i + 128 < width; i += 256) {
                float4 a[kRouteRows], b[kRouteRows];
#pragma unroll
                for (int r = 0; r < kRouteRows; ++r) {
                    a[r] = *reinterpret_cast<const float4*>(w[r] + i);
                    b[r] = *reinterpret_cast<const float4*>(w[r] + i + 128);
                }
#pragma unroll
                for (int k = 0; k < TOK; ++k) {
                    const float4 xa = *reinterpret_cast<const float4*>(x + k * width + i);
                    const float4 xb = *reinterpret_cast<const float4*>(x + k * width + i + 128);
#pragma unroll
                    for (int r = 0; r < kRouteRows; ++r) { fma4(z[r][k], a[r], xa); fma4(z[r][k], b[r], xb); }
                }
            }
            if (i < width) {
                float4 a[kRouteRows];
#pragma unroll
                for (int r = 0; r < kRouteRows; ++r) a[r] = *reinterpret_cast<const float4*>(w[r] + i);
#pragma unroll
                for (int k = 0; k < TOK; ++k) {
                    const float4 xa = *reinterpret_cast<const float4*>(x + k * width + i);
#pragma unroll
                    for (int r = 0; r < kRouteRows; ++r) fma4(z[r][k], a[r], xa);
                }
            }
        } else {
            for (int i = lane; i < width; i += 32) {
                float a[kRouteRows];
#pragma unroll
                for (int r = 0; r < kRouteRows; ++r) a[r] = w[r][i];
#pragma unroll
                for (int k = 0; k < TOK; ++k) {
                    const float xv = x[k * width + i];
#pragma unroll
                    for (int r = 0; r < kRouteRows; ++r) z[r][k] = fmaf(a[r], xv, z[r][k]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < kRouteRows; ++r) {
#pragma unroll
            for (int k = 0; k < TOK; ++k) {
                const float zk = warp_sum(z[r][k]);
                if (lane == 0 && e0 + r < n_rows)
                    s[k * n_rows + e0 + r] = (softmax && e0 + r < n_experts) ? zk : 1.0f / (1.0f + expf(-zk));
            }
        }
    }
    __syncthreads();
    if (warp >= n_tok) return;                           // warp k picks for token k of the block
    float* sk = s + (size_t)warp * n_rows;
    const size_t t = (size_t)t0 + warp;
    for (int e = lane; e < n_extra; e += 32) extra[t * n_extra + e] = sk[n_experts + e];
    if (softmax) {                                       // the experts' entries hold logits: scores over all of them
        float top_z = -INFINITY;
        for (int e = lane; e < n_experts; e += 32) top_z = fmaxf(top_z, sk[e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) top_z = fmaxf(top_z, __shfl_xor_sync(0xffffffffu, top_z, o));
        float sum = 0.0f;
        for (int e = lane; e < n_experts; e += 32) { const float p = expf(sk[e] - top_z); sk[e] = p; sum += p; }
        sum = warp_sum(sum);
        for (int e = lane; e < n_experts; e += 32) sk[e] = sk[e] / sum;
        __syncwarp();
    }
    float total = 0.0f;
    for (int c = 0; c < top; ++c) {
        // the largest score left; among equals the lowest index
        float best = -1.0f;
        int arg = n_experts;
        for (int e = lane; e < n_experts; e += 32)
            if (sk[e] > best) { best = sk[e]; arg = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (lane == 0) {
            ids[t * top + c] = arg;
            weights[t * top + c] = best;
            sk[arg] = -2.0f;                 // taken
        }
        total += best;
        __syncwarp();
    }
    if (lane == 0) {
        const float f = renormalize ? scale / (total + renorm_eps) : scale;
        for (int c = 0; c < top; ++c) weights[t * top + c] *= f;
    }
}

template <typename T> struct Chunk;
template <> struct Chunk<float> { static constexpr int n = 4; };
template <> struct Chunk<__nv_bfloat16> { static constexpr int n = 8; };

// The warp's sum over i of w[i] * x[i] (x in shared memory, float32).  Rows that start on a 16-byte boundary and hold
// a whole number of 16-byte chunks are read 16 bytes a lane, four chunks in flight; the order of addition depends on
// the row's length and alignment alone.
template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    constexpr int V = Chunk<T>::n;
    constexpr int U = 4;                                 // chunks a lane has in flight
    float acc = 0.0f;
    if (n % V == 0 && ((uintptr_t)w & 15) == 0) {
        float part[U];
#pragma unroll
        for (int u = 0; u < U; ++u) part[u] = 0.0f;
        int i = lane * V;
        for (; i + (U - 1) * 32 * V < n; i += U * 32 * V) {
            float a[U][V];
#pragma unroll
            for (int u = 0; u < U; ++u) load_chunk(w + i + u * 32 * V, a[u]);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float xa[V];
#pragma unroll
                for (int e = 0; e < V; e += 4) load_chunk(x + i + u * 32 * V + e, *reinterpret_cast<float(*)[4]>(xa + e));
#pragma unroll
                for (int e = 0; e < V; ++e) part[u] = fmaf(a[u][e], xa[e], part[u]);
            }
        }
        for (; i < n; i += 32 * V) {
            float a[V], xa[V];
            load_chunk(w + i, a);
#pragma unroll
            for (int e = 0; e < V; e += 4) load_chunk(x + i + e, *reinterpret_cast<float(*)[4]>(xa + e));
#pragma unroll
            for (int e = 0; e < V; ++e) part[0] = fmaf(a[e], xa[e], part[0]);
        }
        return warp_sum((part[0] + part[1]) + (part[2] + part[3]));
    }
    for (int i = lane; i < n; i += 32) acc = fmaf(to_float(w[i]), x[i], acc);
    return warp_sum(acc);
}

template <typename T>
__global__ void moe_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gate_up, const int* __restrict__ ids,
                                   T* __restrict__ act, int width, int ff, int top, const GatedInter p,
                                   const float* __restrict__ in_weights) {
    pdl_wait();
    extern __shared__ __align__(16) float x[];             // [width]
    const int pair = blockIdx.x, t = pair / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < width; i += blockDim.x) x[i] = to_float(h[(size_t)t * width + i]);
    __syncthreads();
    const int e = ids[pair];
    const float ws = in_weights ? in_weights[pair] : 1.0f;      // the pair's weight on the expert's input: W (w h) = w (W h)
    const T* w = w_gate_up + (size_t)e * 2 * ff * width;
    for (int j = blockIdx.y * warps + warp; j < ff; j += gridDim.y * warps) {
        const float g = dot_row(w + (size_t)j * width, x, width, lane);
        const float u = dot_row(w + (size_t)(ff + j) * width, x, width, lane);
        if (lane == 0) act[(size_t)pair * ff + j] = from_float<T>(gated(ws * g, ws * u, p));
    }
}

template <typename T>
__global__ void moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ ids,
                                const float* __restrict__ weights, const T* __restrict__ add, const float* __restrict__ add_scale,
                                T* __restrict__ out, int width, int ff, int top) {
    pdl_wait();
    extern __shared__ __align__(16) float y[];             // [top][ff]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) y[i] = to_float(act[(size_t)t * top * ff + i]);
    __syncthreads();
    for (int c = blockIdx.y * warps + warp; c < width; c += gridDim.y * warps) {
        float sum = add ? to_float(add[(size_t)t * width + c]) * (add_scale ? add_scale[t] : 1.0f) : 0.0f;
        for (int slot = 0; slot < top; ++slot) {
            const int e = ids[(size_t)t * top + slot];
            const float d = dot_row(w_down + ((size_t)e * width + c) * ff, y + (size_t)slot * ff, ff, lane);
            sum = fmaf(weights ? weights[(size_t)t * top + slot] : 1.0f, d, sum);
        }
        if (lane == 0) out[(size_t)t * width + c] = from_float<T>(sum);
    }
}

template <typename T, int TOK>
int launch_route(const void* h, const float* router, int* ids, float* weights, int n, int width, int n_experts, int top, float scale,
                 int renormalize, int n_extra, float* extra, int softmax, float renorm_eps, cudaStream_t stream) {
    const size_t smem = sizeof(float) * TOK * ((size_t)width + n_experts + n_extra);
    if (smem > 200 * 1024) return PB_ERR_TOO_LARGE;
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        const cudaError_t ce = cudaFuncSetAttribute(moe_route_kernel<T, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce != cudaSuccess) return (int)ce;
        allowed = smem;
    }
    int warps = (n_experts + n_extra + kRouteRows - 1) / kRouteRows;      // a warp per group of rows where that fits a block
    if (warps > 16) warps = 16;
    if (warps < TOK) warps = TOK;                                         // warp k picks for token k
    return launch_pdl(moe_route_kernel<T, TOK>, dim3((n + TOK - 1) / TOK), dim3(32 * warps), smem, stream, (const T*)h, router, ids,
                      weights, n, width, n_experts, top, scale, renormalize, n_extra, extra, softmax, renorm_eps);
}

template <typename T>
int dispatch_route(const void* h, const float* router, int* ids, float* weights, int n, int width, int n_experts, int top, float scale,
                   int renormalize, int n_extra, float* extra, int softmax, float renorm_eps, cudaStream_t stream) {
    // tokens a block shares the router's rows among: one where the step is a few tokens (their blocks run side by side),
    // eight where their float32 rows leave room for three blocks on a SM, else four
    const size_t row = sizeof(float) * ((size_t)width + n_experts + n_extra);
#define PB_ROUTE(TOK) return launch_route<T, TOK>(h, router, ids, weights, n, width, n_experts, top, scale, renormalize, n_extra, extra, softmax, renorm_eps, stream)
    if (n <= 16) PB_ROUTE(1);
    if (8 * row <= 72 * 1024) PB_ROUTE(8);
    PB_ROUTE(4);
#undef PB_ROUTE
}

}  // namespace

// router [n_experts + n_extra, width]: the rows behind the experts' are scored too (sigmoid) and go to extra [n, n_extra].
PB_EXPORT int pb_moe_route(int dtype, const void* h, const float* router, int* ids, float* weights, int n, int width, int n_experts,
                           int top, float scale, int renormalize, int n_extra, float* extra, int softmax, float renorm_eps,
                           cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || n_experts <= 0 || top <= 0 || top > n_experts || n_extra < 0 || (n_extra > 0 && extra == nullptr)) return PB_ERR_BAD_SIZE;
    if (dtype == PB_F32) return dispatch_route<float>(h, router, ids, weights, n, width, n_experts, top, scale, renormalize, n_extra, extra, softmax, renorm_eps, stream);
    if (dtype == PB_BF16)
        return dispatch_route<__nv_bfloat16>(h, router, ids, weights, n, width, n_experts, top, scale, renormalize, n_extra, extra, softmax, renorm_eps, stream);
    return PB_ERR_BAD_DTYPE;
}

// in_weights (float32 [n * top] or null): a pair's weight multiplies the expert's input instead of its output.
PB_EXPORT int pb_moe_gate_up(int dtype, const void* h, const void* w_gate_up, const int* ids, void* act, int n, int width, int ff,
                             int top, float limit, float alpha, float shift, const float* in_weights, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || ff <= 0 || top <= 0) return PB_ERR_BAD_SIZE;
    const size_t smem = sizeof(float) * (size_t)width;
    if (smem > 48 * 1024) return PB_ERR_TOO_LARGE;
    const int warps = 8;
    int by = (ff + warps - 1) / warps;
    if (by > 64) by = 64;
    const GatedInter p(ff, limit > 0.0f ? limit : __builtin_huge_valf(), alpha, shift);
    dim3 grid(n * top, by);
    if (dtype == PB_F32)
        return launch_pdl(moe_gate_up_kernel<float>, grid, dim3(warps * 32), smem, stream, (const float*)h, (const float*)w_gate_up, ids,
                          (float*)act, width, ff, top, p, in_weights);
    if (dtype == PB_BF16)
        return launch_pdl(moe_gate_up_kernel<__nv_bfloat16>, grid, dim3(warps * 32), smem, stream, (const __nv_bfloat16*)h,
                          (const __nv_bfloat16*)w_gate_up, ids, (__nv_bfloat16*)act, width, ff, top, p, in_weights);
    return PB_ERR_BAD_DTYPE;
}

// weights null: every pair counts once (its weight went into the expert's input); add_scale (float32 [n] or null) multiplies `add`.
PB_EXPORT int pb_moe_down(int dtype, const void* act, const void* w_down, const int* ids, const float* weights, const void* add,
                          const float* add_scale, void* out, int n, int width, int ff, int top, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || ff <= 0 || top <= 0) return PB_ERR_BAD_SIZE;
    const size_t smem = sizeof(float) * (size_t)top * ff;
    if (smem > 48 * 1024) return PB_ERR_TOO_LARGE;
    const int warps = 8;
    int by = (width + warps - 1) / warps;
    if (by > 64) by = 64;
    dim3 grid(n, by);
    if (dtype == PB_F32)
        return launch_pdl(moe_down_kernel<float>, grid, dim3(warps * 32), smem, stream, (const float*)act, (const float*)w_down, ids,
                          weights, (const float*)add, add_scale, (float*)out, width, ff, top);
    if (dtype == PB_BF16)
        return launch_pdl(moe_down_kernel<__nv_bfloat16>, grid, dim3(warps * 32), smem, stream, (const __nv_bfloat16*)act,
                          (const __nv_bfloat16*)w_down, ids, weights, (const __nv_bfloat16*)add, add_scale, (__nv_bfloat16*)out, width, ff, top);
    return PB_ERR_BAD_DTYPE;
}

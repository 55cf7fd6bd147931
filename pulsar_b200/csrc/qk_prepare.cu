// What stands between the fused q | k (| gate) projection and the general attention kernels when the heads are
// rotated and normed without a weight, and what stands behind those kernels when the heads are gated.
//
//   qk_prepare     per (token, head) of a projection row [q: Hq*D | k: Hkv*D | ...] (float32 or T, row stride given):
//                    x = row + bias                                     (bias float32, optional)
//                    weighted norm (pre_eps >= 0): x / sqrt(mean(x^2) + pre_eps) * w, w float32 [D], one for the query
//                    heads and one for the key heads, before the rotation
//                    key heads with values_from_keys: x, as it is now, goes to the value pool
//                    the first `rotary` dimensions turn in the rotate-half layout: element i pairs with element
//                    i + rotary/2, (u, v) -> (u cos - v sin, v cos + u sin), cos/sin [N, rotary/2] float32
//                    unit norm (eps >= 0): x / sqrt(mean(x^2) + eps) over the head, no weight
//                  queries to float32 [N, Hq, D], keys to the key pool (T).  All arithmetic is float32; the pools
//                  take one rounding.  Hv > 0: Hv value heads of Dv behind the key heads in the row go to the value
//                  pool as they are.
//   add_bias       x[n, c] += bias[c] (bias float32): a projection's bias where no kernel behind the product takes it along.
//   sigmoid_gate_strided   x[n, c] *= sigmoid(gate[n, c / group]) with float32 arithmetic; gate float32 or T, a column slice
//                  of a wider row; `group` columns of x share a gate column (a gate per head).
#include "common.cuh"

namespace {

using namespace pb;

constexpr int kMaxPerLane = 16;          // head sizes up to 512

template <typename TIn, typename T>
__global__ void qk_prepare_kernel(const TIn* __restrict__ rows, long row_stride, const float* __restrict__ q_bias,
                                  const float* __restrict__ k_bias, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  float* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                  const int* __restrict__ slots, int Hq, int Hkv, int D, int rotary, float eps, int unit_norm,
                                  int values_from_keys, int page_size, const float* __restrict__ q_norm_w,
                                  const float* __restrict__ k_norm_w, float pre_eps, int Hv, int Dv, const PoolBounds bounds) {
    pdl_wait();
    extern __shared__ float smem[];                      // [warps][D]
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    if (head >= Hq + Hkv + Hv) return;
    if (head >= Hq + Hkv) {                              // a value head: copied to its page
        const int hv = head - Hq - Hkv;
        const int slot = slots[t];
        if (slot < 0 || !slot_ok(slot, page_size, bounds)) return;
        const TIn* src = rows + (size_t)t * row_stride + (size_t)(Hq + Hkv) * D + (size_t)hv * Dv;
        T* dst = v_pool + (((size_t)(slot / page_size) * Hv + hv) * page_size + slot % page_size) * Dv;
        for (int i = lane; i < Dv; i += 32) dst[i] = from_float<T>(to_float(src[i]));
        return;
    }
    float* x = smem + (size_t)warp * D;
    const bool is_q = head < Hq;
    const TIn* src = rows + (size_t)t * row_stride + (size_t)head * D;       // key heads follow the query heads
    const float* bias = is_q ? (q_bias ? q_bias + (size_t)head * D : nullptr) : (k_bias ? k_bias + (size_t)(head - Hq) * D : nullptr);
    for (int i = lane; i < D; i += 32) x[i] = to_float(src[i]) + (bias ? bias[i] : 0.0f);
    __syncwarp();
    int slot = -1;
    size_t at = 0;
    if (!is_q) {
        slot = slots[t];
        if (slot < 0 || !slot_ok(slot, page_size, bounds)) return;           // uniform over the warp
        at = (((size_t)(slot / page_size) * Hkv + (head - Hq)) * page_size + slot % page_size) * D;
        if (values_from_keys)
            for (int i = lane; i < D; i += 32) v_pool[at + i] = from_float<T>(x[i]);
    }
    const float* pre_w = is_q ? q_norm_w : k_norm_w;
    if (pre_w != nullptr) {
        float ss = 0.0f;
        for (int i = lane; i < D; i += 32) ss += x[i] * x[i];
        const float r = rsqrtf(warp_sum(ss) / (float)D + pre_eps);
        for (int i = lane; i < D; i += 32) x[i] = x[i] * r * pre_w[i];
        __syncwarp();
    }
    const int half = rotary >> 1;
    const float* c = cos_t + (size_t)t * half;
    const float* s = sin_t + (size_t)t * half;
    for (int i = lane; i < half; i += 32) {
        const float u = x[i], v = x[i + half];
        x[i] = u * c[i] - v * s[i];
        x[i + half] = v * c[i] + u * s[i];
    }
    __syncwarp();
    float inv = 1.0f;
    if (unit_norm) {
        float ss = 0.0f;
        for (int i = lane; i < D; i += 32) ss += x[i] * x[i];
        inv = rsqrtf(warp_sum(ss) / (float)D + eps);
    }
    if (is_q) {
        float* dst = q_out + ((size_t)t * Hq + head) * D;
        for (int i = lane; i < D; i += 32) dst[i] = x[i] * inv;
    } else {
        for (int i = lane; i < D; i += 32) k_pool[at + i] = from_float<T>(x[i] * inv);
    }
}

template <typename T, typename TG>
__global__ void sigmoid_gate_strided_kernel(T* __restrict__ x, const TG* __restrict__ gate, long gate_stride, int width, int group,
                                            size_t total) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / width, col = i % width;
        const float g = to_float(gate[row * gate_stride + col / group]);
        x[i] = from_float<T>(to_float(x[i]) / (1.0f + expf(-g)));
    }
}

template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int width, size_t total) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = from_float<T>(to_float(x[i]) + bias[i % width]);
}

template <typename TIn, typename T>
int launch_prepare(const void* rows, long row_stride, const float* q_bias, const float* k_bias, const float* cos_t, const float* sin_t,
                   float* q_out, void* k_pool, void* v_pool, const int* slots, int n, int Hq, int Hkv, int D, int rotary, float eps,
                   int unit_norm, int values_from_keys, int page_size, const float* q_norm_w, const float* k_norm_w, float pre_eps,
                   int Hv, int Dv, cudaStream_t stream) {
    const int warps = 4;
    dim3 grid(n, (Hq + Hkv + Hv + warps - 1) / warps);
    return launch_pdl(qk_prepare_kernel<TIn, T>, grid, dim3(warps * 32), sizeof(float) * warps * D, stream, (const TIn*)rows, row_stride,
                      q_bias, k_bias, cos_t, sin_t, q_out, (T*)k_pool, (T*)v_pool, slots, Hq, Hkv, D, rotary, eps, unit_norm,
                      values_from_keys, page_size, q_norm_w, k_norm_w, pre_eps, Hv, Dv, pool_bounds_now());
}

}  // namespace

// rows [n, row_stride] of dtype in_dtype (query heads, then key heads, D wide each); pools of dtype `dtype`
// [pages, Hkv, page_size, D]; q_out float32 [n, Hq, D]; cos/sin float32 [n, rotary / 2]; eps < 0: no unit norm.
// Hkv 0: the rows hold queries only (pools and slots unused).  pre_eps >= 0: the weighted norm before the rotation with
// q_norm_w / k_norm_w float32 [D].  Hv > 0: value heads of Dv behind the key heads; v_pool is [pages, Hv, page_size, Dv].
PB_EXPORT int pb_qk_prepare(int in_dtype, int dtype, const void* rows, long row_stride, const float* q_bias, const float* k_bias,
                            const float* cos_t, const float* sin_t, float* q_out, void* k_pool, void* v_pool, const int* slots,
                            int n, int Hq, int Hkv, int D, int rotary, float eps, int values_from_keys, int page_size,
                            const float* q_norm_w, const float* k_norm_w, float pre_eps, int Hv, int Dv, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (Hv < 0 || (Hv > 0 && (Dv <= 0 || v_pool == nullptr || slots == nullptr || values_from_keys)) ||
        row_stride < (long)(Hq + Hkv) * D + (long)Hv * Dv || (pre_eps >= 0.0f && q_norm_w == nullptr) ||
        (pre_eps >= 0.0f && Hkv > 0 && k_norm_w == nullptr))
        return PB_ERR_BAD_SIZE;
    if (pre_eps < 0.0f) q_norm_w = k_norm_w = nullptr;
    if (Hq <= 0 || Hkv < 0 || D <= 0 || D > 32 * kMaxPerLane * 4 || rotary < 0 || rotary > D || rotary % 2 || page_size <= 0 ||
        row_stride < (long)(Hq + Hkv) * D || (Hkv > 0 && (k_pool == nullptr || slots == nullptr)) ||
        (values_from_keys && Hkv > 0 && v_pool == nullptr) || (rotary > 0 && (cos_t == nullptr || sin_t == nullptr)))
        return PB_ERR_BAD_SIZE;
    if ((Hq + Hkv + Hv + 3) / 4 > 65535) return PB_ERR_TOO_LARGE;
    const int unit = eps >= 0.0f ? 1 : 0;
#define PB_PREP(TI, T) return launch_prepare<TI, T>(rows, row_stride, q_bias, k_bias, cos_t, sin_t, q_out, k_pool, v_pool, slots, n, Hq, \
                                                    Hkv, D, rotary, eps, unit, values_from_keys, page_size, q_norm_w, k_norm_w, pre_eps, Hv, Dv, stream)
    if (in_dtype == PB_F32 && dtype == PB_F32) PB_PREP(float, float);
    if (in_dtype == PB_F32 && dtype == PB_BF16) PB_PREP(float, __nv_bfloat16);
    if (in_dtype == PB_BF16 && dtype == PB_BF16) PB_PREP(__nv_bfloat16, __nv_bfloat16);
    if (in_dtype == PB_BF16 && dtype == PB_F32) PB_PREP(__nv_bfloat16, float);
#undef PB_PREP
    return PB_ERR_BAD_DTYPE;
}

// x [n, width] (dtype) *= sigmoid(gate[n, c / group]) where gate rows are gate_stride elements apart (gate_dtype): `group`
// neighbouring columns of x share one gate column (1: a gate per element; a head's width: a gate per head).
PB_EXPORT int pb_sigmoid_gate_strided(int dtype, int gate_dtype, void* x, const void* gate, long gate_stride, int n, int width,
                                      int group, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || group <= 0 || width % group || gate_stride < width / group) return PB_ERR_BAD_SIZE;
    const size_t total = (size_t)n * width;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
#define PB_GATE(T, TG) return launch_pdl(sigmoid_gate_strided_kernel<T, TG>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)x, \
                                         (const TG*)gate, gate_stride, width, group, total)
    if (dtype == PB_F32 && gate_dtype == PB_F32) PB_GATE(float, float);
    if (dtype == PB_BF16 && gate_dtype == PB_F32) PB_GATE(__nv_bfloat16, float);
    if (dtype == PB_BF16 && gate_dtype == PB_BF16) PB_GATE(__nv_bfloat16, __nv_bfloat16);
    if (dtype == PB_F32 && gate_dtype == PB_BF16) PB_GATE(float, __nv_bfloat16);
#undef PB_GATE
    return PB_ERR_BAD_DTYPE;
}

// x [n, width] (dtype) += bias [width] (float32).
PB_EXPORT int pb_add_bias(int dtype, void* x, const float* bias, int n, int width, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || bias == nullptr) return PB_ERR_BAD_SIZE;
    const size_t total = (size_t)n * width;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == PB_F32) return launch_pdl(add_bias_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (float*)x, bias, width, total);
    if (dtype == PB_BF16)
        return launch_pdl(add_bias_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, bias, width, total);
    return PB_ERR_BAD_DTYPE;
}

// Small kernels around composite mixers and repeated walks over a run of layers.
//
//   scaled_sum       out[i] = a * x[i] + b * y[i] (float32 arithmetic, one rounding on store): two mixers side by side whose
//                    outputs join with a weight each.  x and y are of one dtype, out of its own.
//   concat_streams   out[n] = [ residual[n] (+ delta[n]) | origin[n] ] in the activation dtype: the operand of the product that
//                    opens a walk, x <- W [x ; x0].  residual and origin are float32 [N, width]; delta (optional) is what the
//                    layer before left pending.
#include "common.cuh"

namespace {

using namespace pb;

template <typename TIn, typename T>
__global__ void scaled_sum_kernel(const TIn* __restrict__ x, const TIn* __restrict__ y, T* __restrict__ out, float a, float b, size_t total) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_float<T>(fmaf(a, to_float(x[i]), b * to_float(y[i])));
}

template <typename T>
__global__ void concat_streams_kernel(const float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ origin,
                                      T* __restrict__ out, int width, size_t total) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / width, col = i % width;
        const float x = residual[i] + (delta != nullptr ? to_float(delta[i]) : 0.0f);
        out[row * 2 * width + col] = from_float<T>(x);
        out[row * 2 * width + width + col] = from_float<T>(origin[i]);
    }
}

unsigned blocks_for(size_t total) {
    size_t blocks = (total + 255) / 256;
    return (unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks);
}

}  // namespace

PB_EXPORT int pb_scaled_sum(int in_dtype, int dtype, const void* x, const void* y, void* out, float a, float b, long long total,
                            cudaStream_t stream) {
    if (total <= 0) return 0;
#define PB_SUM(TI, T) return launch_pdl(scaled_sum_kernel<TI, T>, dim3(blocks_for(total)), dim3(256), 0, stream, (const TI*)x, \
                                        (const TI*)y, (T*)out, a, b, (size_t)total)
    if (in_dtype == PB_F32 && dtype == PB_F32) PB_SUM(float, float);
    if (in_dtype == PB_F32 && dtype == PB_BF16) PB_SUM(float, __nv_bfloat16);
    if (in_dtype == PB_BF16 && dtype == PB_BF16) PB_SUM(__nv_bfloat16, __nv_bfloat16);
    if (in_dtype == PB_BF16 && dtype == PB_F32) PB_SUM(__nv_bfloat16, float);
#undef PB_SUM
    return PB_ERR_BAD_DTYPE;
}

PB_EXPORT int pb_concat_streams(int dtype, const float* residual, const void* delta, const float* origin, void* out, int n, int width,
                                cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0) return PB_ERR_BAD_SIZE;
    const size_t total = (size_t)n * width;
    if (dtype == PB_F32)
        return launch_pdl(concat_streams_kernel<float>, dim3(blocks_for(total)), dim3(256), 0, stream, residual, (const float*)delta, origin,
                          (float*)out, width, total);
    if (dtype == PB_BF16)
        return launch_pdl(concat_streams_kernel<__nv_bfloat16>, dim3(blocks_for(total)), dim3(256), 0, stream, residual,
                          (const __nv_bfloat16*)delta, origin, (__nv_bfloat16*)out, width, total);
    return PB_ERR_BAD_DTYPE;
}

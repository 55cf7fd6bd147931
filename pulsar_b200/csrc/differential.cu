// Differential attention: what follows the two softmax maps of a head.
//
//   diff_combine   maps [N, 2 H, Dv] holds, for every token, the outputs of both maps of every head over the same values,
//                  ordered so that the query heads of one key head are neighbours: with R = H / G query heads per key/value
//                  head, head h = g R + r has its first map at row (2 g) R + r and its second at row (2 g + 1) R + r.
//                  o = a1 - lambda * a2, divided by its root mean square over the head's Dv values (eps inside the root),
//                  times `gain`: out [N, H, Dv].  float32 arithmetic, one rounding on store.  A warp per (token, head).
#include "common.cuh"

namespace {

using namespace pb;

template <typename In, typename Out>
__global__ void diff_combine_kernel(const In* __restrict__ maps, Out* __restrict__ out, int n, int H, int R, int Dv, float lambda,
                                    float eps, float gain) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= (long long)n * H) return;
    const int t = (int)(pair / H), h = (int)(pair % H);
    const int g = h / R, r = h % R;
    const In* a1 = maps + ((size_t)t * 2 * H + (size_t)(2 * g) * R + r) * Dv;
    const In* a2 = maps + ((size_t)t * 2 * H + (size_t)(2 * g + 1) * R + r) * Dv;
    constexpr int kKeep = 8;                    // values a lane keeps in registers (Dv up to 256); beyond that they are read again
    float o[kKeep];
    float ss = 0.0f;
    int k = 0;
    for (int i = lane; i < Dv; i += 32, ++k) {
        const float v = to_float(a1[i]) - lambda * to_float(a2[i]);
        if (k < kKeep) o[k] = v;
        ss += v * v;
    }
    const float f = rsqrtf(warp_sum(ss) / (float)Dv + eps) * gain;
    Out* dst = out + ((size_t)t * H + h) * Dv;
    k = 0;
    for (int i = lane; i < Dv; i += 32, ++k) {
        const float v = k < kKeep ? o[k] : to_float(a1[i]) - lambda * to_float(a2[i]);
        dst[i] = from_float<Out>(v * f);
    }
}

}  // namespace

PB_EXPORT int pb_diff_combine(int in_dtype, int out_dtype, const void* maps, void* out, int n, int H, int G, int Dv, float lambda,
                              float eps, float gain, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || Dv <= 0) return PB_ERR_BAD_SIZE;
    const int warps = 4;
    const long long pairs = (long long)n * H;
    const dim3 grid((unsigned)((pairs + warps - 1) / warps)), block(warps * 32);
    const int R = H / G;
#define PB_DIFF(In, Out) return launch_pdl(diff_combine_kernel<In, Out>, grid, block, 0, stream, (const In*)maps, (Out*)out, n, H, R, Dv, lambda, eps, gain)
    if (in_dtype == PB_F32 && out_dtype == PB_F32) PB_DIFF(float, float);
    if (in_dtype == PB_F32 && out_dtype == PB_BF16) PB_DIFF(float, __nv_bfloat16);
    if (in_dtype == PB_BF16 && out_dtype == PB_BF16) PB_DIFF(__nv_bfloat16, __nv_bfloat16);
#undef PB_DIFF
    return PB_ERR_BAD_DTYPE;
}

// Memory-bound kernels of layers whose two sublayers read one norm's output side by side, with a blend of neighbouring
// tokens in front of the mixer.
//
//   norm_shift     h = rmsnorm(x) * w (float32 sums; w [width] float32), hs = h + (h' - h) * shift with h' the h of the token
//                  before in the same sequence: the row above when that token is part of the step, else the sequence's kept
//                  row (`state`, float32, one row per state slot; zeros for a fresh sequence).  h goes to the feed-forward,
//                  hs to the mixer, both rounded once to the activation dtype.  A sequence's last token of the step leaves
//                  its float32 h in `pending` [sequences, width]; parallel_add moves it into the kept row, after every
//                  reader of the old one is done.  Without `shift` the kernel is a plain norm (hs is not written).
//   parallel_add   x += m * (a + b) in float32 on the float32 stream (b optional), and the move of `pending` into the kept
//                  rows.  With `next`: also the norm_shift of the layer that follows, on the stream as it then stands; the
//                  new stream goes to `x_out`, another buffer than `x`, because a row's blend reads the row above as it was.
//   activation     out = act(in) element by element, in [N, F] float32 or the activation dtype: 0 gelu (erf), 1 gelu (tanh
//                  form), 2 silu, 3 relu.  float32 arithmetic, one rounding on store.
#include "common.cuh"

#include <stdint.h>

namespace {

using namespace pb;

struct ShiftArgs {
    const float* weight;        // [width] norm weight
    const float* shift;         // [width] or null
    const float* state;         // kept rows, read
    long state_stride;
    const int* seq_of_token;    // [N]
    const int* cu_q;            // [S + 1]
    const int* state_slots;     // [S]
    float* pending;             // [S, width]
    float eps;
};

// Row t of the stream as `cur` (and the row above as `prev`, only read when t is not its sequence's first token of the step):
// callers give functors so that the fused form can hand in rows that exist nowhere in memory yet.
template <typename T, typename Row>
__device__ __forceinline__ void norm_shift_row(const Row& row, int t, const ShiftArgs& p, T* __restrict__ h_out,
                                               T* __restrict__ hs_out, int width, float* scratch) {
    const int s = p.seq_of_token[t];
    const int first = p.cu_q[s], last = p.cu_q[s + 1] - 1;
    const bool has_prev = p.shift != nullptr && t > first;
    float ss = 0.0f, ssp = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = row(t, i);
        ss += x * x;
        if (has_prev) { const float xp = row(t - 1, i); ssp += xp * xp; }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + p.eps);
    const float invp = has_prev ? rsqrtf(block_sum(ssp, scratch) / (float)width + p.eps) : 0.0f;    // has_prev is uniform over the block
    const float* kept = p.state + (size_t)p.state_slots[s] * p.state_stride;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float w = p.weight[i];
        const float h = row(t, i) * inv * w;
        h_out[(size_t)t * width + i] = from_float<T>(h);
        if (p.shift != nullptr) {
            const float hp = has_prev ? row(t - 1, i) * invp * w : kept[i];
            hs_out[(size_t)t * width + i] = from_float<T>(h + (hp - h) * p.shift[i]);
            if (t == last) p.pending[(size_t)s * width + i] = h;
        }
    }
}

struct PlainRow {
    const float* x;
    int width;
    __device__ __forceinline__ float operator()(int t, int i) const { return x[(size_t)t * width + i]; }
};

template <typename T>
__global__ void norm_shift_kernel(const float* __restrict__ x, const ShiftArgs p, T* __restrict__ h_out, T* __restrict__ hs_out,
                                  int width) {
    pdl_wait();
    __shared__ float scratch[32];
    norm_shift_row<T>(PlainRow{x, width}, blockIdx.x, p, h_out, hs_out, width, scratch);
}

template <typename T>
struct SumRow {
    const float* x;
    const T* a;
    const T* b;
    float m;
    int width;
    __device__ __forceinline__ float operator()(int t, int i) const {
        const size_t at = (size_t)t * width + i;
        const float d = to_float(a[at]) + (b != nullptr ? to_float(b[at]) : 0.0f);
        return x[at] + m * d;
    }
};

// commit: kept row of the sequence whose last token of the step is t <- pending (of the layer that ends here)
struct CommitArgs {
    const float* pending;
    float* state;
    long state_stride;
    const int* seq_of_token;
    const int* cu_q;
    const int* state_slots;
};

template <typename T>
__global__ void parallel_add_kernel(const float* __restrict__ x, const T* __restrict__ a, const T* __restrict__ b, float m,
                                    float* __restrict__ x_out, const CommitArgs c, const ShiftArgs next, T* __restrict__ h_out,
                                    T* __restrict__ hs_out, int width) {
    pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const SumRow<T> row{x, a, b, m, width};
    for (int i = threadIdx.x; i < width; i += blockDim.x) x_out[(size_t)t * width + i] = row(t, i);
    if (c.pending != nullptr) {
        const int s = c.seq_of_token[t];
        if (t == c.cu_q[s + 1] - 1) {
            float* kept = c.state + (size_t)c.state_slots[s] * c.state_stride;
            for (int i = threadIdx.x; i < width; i += blockDim.x) kept[i] = c.pending[(size_t)s * width + i];
        }
    }
    if (next.weight != nullptr) norm_shift_row<T>(row, t, next, h_out, hs_out, width, scratch);
}

__device__ __forceinline__ float act_value(float z, int kind) {
    if (kind == 0) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    if (kind == 1) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    if (kind == 2) return z / (1.0f + expf(-z));
    return fmaxf(z, 0.0f);
}

template <typename In, typename Out>
__global__ void activation_kernel(const In* __restrict__ in, Out* __restrict__ out, size_t total, int kind) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_float<Out>(act_value(to_float(in[i]), kind));
}

int row_threads(int width) {
    int threads = (width + 3) / 4;
    threads = (threads + 31) / 32 * 32;
    return threads > 512 ? 512 : (threads < 32 ? 32 : threads);
}

}  // namespace

// x [n, width] float32; weight [width]; shift [width] or null (then hs, state, pending and the index arrays are unused);
// state: float32 rows of `state_stride` elements, one per state slot; h, hs [n, width] in `dtype`; pending [n_seqs, width].
PB_EXPORT int pb_norm_shift(int dtype, const float* x, const float* weight, float eps, const float* shift, const float* state,
                            long state_stride, const int* seq_of_token, const int* cu_q, const int* state_slots, void* h, void* hs,
                            float* pending, int n, int width, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || seq_of_token == nullptr || cu_q == nullptr) return PB_ERR_BAD_SIZE;
    if (shift != nullptr && (state == nullptr || state_slots == nullptr || pending == nullptr || hs == nullptr)) return PB_ERR_BAD_SIZE;
    const ShiftArgs p{weight, shift, state, state_stride, seq_of_token, cu_q, state_slots, pending, eps};
    if (dtype == PB_F32)
        return launch_pdl(norm_shift_kernel<float>, dim3(n), dim3(row_threads(width)), 0, stream, x, p, (float*)h, (float*)hs, width);
    if (dtype == PB_BF16)
        return launch_pdl(norm_shift_kernel<__nv_bfloat16>, dim3(n), dim3(row_threads(width)), 0, stream, x, p, (__nv_bfloat16*)h,
                          (__nv_bfloat16*)hs, width);
    return PB_ERR_BAD_DTYPE;
}

// x_out = x + m * (a + b) (b may be null; x_out may be x itself only without `next_weight`); pending (or null) -> the kept
// rows of `state`; with next_weight: the following layer's norm_shift on x_out's rows (next_shift may be null: a plain norm).
PB_EXPORT int pb_parallel_add(int dtype, const float* x, const void* a, const void* b, float m, float* x_out, const float* pending,
                              float* state, long state_stride, const int* seq_of_token, const int* cu_q, const int* state_slots,
                              const float* next_weight, float next_eps, const float* next_shift, const float* next_state,
                              long next_state_stride, float* next_pending, void* h, void* hs, int n, int width, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || a == nullptr) return PB_ERR_BAD_SIZE;
    if ((pending != nullptr || next_weight != nullptr) && (seq_of_token == nullptr || cu_q == nullptr || state_slots == nullptr))
        return PB_ERR_BAD_SIZE;
    if (next_weight != nullptr && (x_out == x || h == nullptr)) return PB_ERR_BAD_SIZE;
    if (next_shift != nullptr && (next_state == nullptr || next_pending == nullptr || hs == nullptr || next_pending == pending))
        return PB_ERR_BAD_SIZE;
    const CommitArgs c{pending, state, state_stride, seq_of_token, cu_q, state_slots};
    const ShiftArgs nx{next_weight, next_shift, next_state, next_state_stride, seq_of_token, cu_q, state_slots, next_pending, next_eps};
    if (dtype == PB_F32)
        return launch_pdl(parallel_add_kernel<float>, dim3(n), dim3(row_threads(width)), 0, stream, x, (const float*)a, (const float*)b, m,
                          x_out, c, nx, (float*)h, (float*)hs, width);
    if (dtype == PB_BF16)
        return launch_pdl(parallel_add_kernel<__nv_bfloat16>, dim3(n), dim3(row_threads(width)), 0, stream, x, (const __nv_bfloat16*)a,
                          (const __nv_bfloat16*)b, m, x_out, c, nx, (__nv_bfloat16*)h, (__nv_bfloat16*)hs, width);
    return PB_ERR_BAD_DTYPE;
}

// in [total] (in_dtype) -> out [total] (out_dtype); kind: 0 gelu (erf), 1 gelu (tanh form), 2 silu, 3 relu.
PB_EXPORT int pb_activation(int in_dtype, int out_dtype, const void* in, void* out, long long total, int kind, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (kind < 0 || kind > 3) return PB_ERR_BAD_SIZE;
    size_t blocks = ((size_t)total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const dim3 grid((unsigned)blocks), block(256);
    if (in_dtype == PB_F32 && out_dtype == PB_F32)
        return launch_pdl(activation_kernel<float, float>, grid, block, 0, stream, (const float*)in, (float*)out, (size_t)total, kind);
    if (in_dtype == PB_F32 && out_dtype == PB_BF16)
        return launch_pdl(activation_kernel<float, __nv_bfloat16>, grid, block, 0, stream, (const float*)in, (__nv_bfloat16*)out,
                          (size_t)total, kind);
    if (in_dtype == PB_BF16 && out_dtype == PB_BF16)
        return launch_pdl(activation_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)in,
                          (__nv_bfloat16*)out, (size_t)total, kind);
    return PB_ERR_BAD_DTYPE;
}

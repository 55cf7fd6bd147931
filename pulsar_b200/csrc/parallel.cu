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
//                  Both kernels have a form that moves four elements at a time and keeps a token's row (and the row above)
//                  in registers between the sum of squares and the output; it takes widths that are multiples of four up
//                  to 8192 with 16-byte aligned rows, the plain form everything else.  A layer's two ends always take the
//                  same form, so the fused boundary and the two separate kernels give the same bits.
//   activation     out = act(in) element by element, in [N, F] float32 or the activation dtype: 0 gelu (erf), 1 gelu (tanh
//                  form), 2 silu, 3 relu.  float32 arithmetic, one rounding on store.
#include "common.cuh"

#include <stdint.h>

#include <initializer_list>

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

// ---- four elements at a time
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&lo);
    raw.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float dot4(float4 v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }

// two sums over the block with one pair of barriers; each is added up in block_sum's order.  `scratch` needs 64 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();   // scratch may still be read from an earlier call
    if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; }
    __syncthreads();
    a = warp_sum(lane < nwarps ? scratch[lane] : 0.0f);
    b = warp_sum(lane < nwarps ? scratch[32 + lane] : 0.0f);
}

constexpr int kVecIters = 4;            // a thread holds up to 4 x 4 elements of a row: widths up to 4 * 512 * 4.  The kernels take
                                        // the count as ITERS (1, 2 or 4, by the width) so that narrow rows cost few registers.

// norm_shift_row with the row in registers.  `cur` holds the thread's part of row t on entry (the caller loaded it, and may
// have stored it as the new stream); the row above is loaded here through `row.at4`.
template <typename T, int ITERS, typename Row>
__device__ __forceinline__ void norm_shift_row4(const Row& row, int t, const float4 (&cur)[ITERS], const ShiftArgs& p,
                                                T* __restrict__ h_out, T* __restrict__ hs_out, int width, float* scratch) {
    const int s = p.seq_of_token[t];
    const int first = p.cu_q[s], last = p.cu_q[s + 1] - 1;
    const bool has_prev = p.shift != nullptr && t > first;
    const int quads = width >> 2;
    float4 prev[ITERS];
    float ss = 0.0f, ssp = 0.0f;
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int q = threadIdx.x + k * blockDim.x;
        if (q < quads) {
            ss += dot4(cur[k]);
            if (has_prev) { prev[k] = row.at4(t - 1, q); ssp += dot4(prev[k]); }
        }
    }
    block_sum2(ss, ssp, scratch);
    const float inv = rsqrtf(ss / (float)width + p.eps);
    const float invp = has_prev ? rsqrtf(ssp / (float)width + p.eps) : 0.0f;
    const float* kept = p.state + (size_t)p.state_slots[s] * p.state_stride;
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int q = threadIdx.x + k * blockDim.x;
        if (q < quads) {
            const size_t at = (size_t)t * width + 4 * q;
            const float4 w = load4(p.weight + 4 * q);
            const float4 h = make_float4(cur[k].x * inv * w.x, cur[k].y * inv * w.y, cur[k].z * inv * w.z, cur[k].w * inv * w.w);
            store4(h_out + at, h);
            if (p.shift != nullptr) {
                float4 hp;
                if (has_prev) hp = make_float4(prev[k].x * invp * w.x, prev[k].y * invp * w.y, prev[k].z * invp * w.z, prev[k].w * invp * w.w);
                else hp = load4(kept + 4 * q);
                const float4 m = load4(p.shift + 4 * q);
                store4(hs_out + at, make_float4(h.x + (hp.x - h.x) * m.x, h.y + (hp.y - h.y) * m.y, h.z + (hp.z - h.z) * m.z,
                                                h.w + (hp.w - h.w) * m.w));
                if (t == last) store4(p.pending + (size_t)s * width + 4 * q, h);
            }
        }
    }
}

struct PlainRow {
    const float* x;
    int width;
    __device__ __forceinline__ float operator()(int t, int i) const { return x[(size_t)t * width + i]; }
    __device__ __forceinline__ float4 at4(int t, int q) const { return load4(x + (size_t)t * width + 4 * q); }
};

template <typename T>
__global__ void norm_shift_kernel(const float* __restrict__ x, const ShiftArgs p, T* __restrict__ h_out, T* __restrict__ hs_out,
                                  int width) {
    pdl_wait();
    __shared__ float scratch[32];
    norm_shift_row<T>(PlainRow{x, width}, blockIdx.x, p, h_out, hs_out, width, scratch);
}

template <typename T, int ITERS>
__global__ void norm_shift4_kernel(const float* __restrict__ x, const ShiftArgs p, T* __restrict__ h_out, T* __restrict__ hs_out,
                                   int width) {
    pdl_wait();
    __shared__ float scratch[64];
    const PlainRow row{x, width};
    float4 cur[ITERS];
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int q = threadIdx.x + k * blockDim.x;
        if (q < (width >> 2)) cur[k] = row.at4(blockIdx.x, q);
    }
    norm_shift_row4<T, ITERS>(row, blockIdx.x, cur, p, h_out, hs_out, width, scratch);
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
    __device__ __forceinline__ float4 at4(int t, int q) const {
        const size_t at = (size_t)t * width + 4 * q;
        const float4 xv = load4(x + at), av = load4(a + at);
        float4 d = av;
        if (b != nullptr) { const float4 bv = load4(b + at); d = make_float4(av.x + bv.x, av.y + bv.y, av.z + bv.z, av.w + bv.w); }
        return make_float4(xv.x + m * d.x, xv.y + m * d.y, xv.z + m * d.z, xv.w + m * d.w);
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

template <typename T, int ITERS>
__global__ void parallel_add4_kernel(const float* __restrict__ x, const T* __restrict__ a, const T* __restrict__ b, float m,
                                     float* __restrict__ x_out, const CommitArgs c, const ShiftArgs next, T* __restrict__ h_out,
                                     T* __restrict__ hs_out, int width) {
    pdl_wait();
    __shared__ float scratch[64];
    const int t = blockIdx.x, quads = width >> 2;
    const SumRow<T> row{x, a, b, m, width};
    float4 cur[ITERS];
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int q = threadIdx.x + k * blockDim.x;
        if (q < quads) {
            cur[k] = row.at4(t, q);
            store4(x_out + (size_t)t * width + 4 * q, cur[k]);
        }
    }
    if (c.pending != nullptr) {
        const int s = c.seq_of_token[t];
        if (t == c.cu_q[s + 1] - 1) {
            float* kept = c.state + (size_t)c.state_slots[s] * c.state_stride;
            for (int q = threadIdx.x; q < quads; q += blockDim.x) store4(kept + 4 * q, load4(c.pending + (size_t)s * width + 4 * q));
        }
    }
    if (next.weight != nullptr) norm_shift_row4<T, ITERS>(row, t, cur, next, h_out, hs_out, width, scratch);
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

// quads of a row that a thread of the four-at-a-time form holds: 1, 2 or kVecIters
int vector_iters(int width, int threads) {
    const int per_thread = ((width >> 2) + threads - 1) / threads;
    return per_thread <= 1 ? 1 : (per_thread <= 2 ? 2 : kVecIters);
}

bool aligned16(const void* p) { return p == nullptr || ((uintptr_t)p & 15) == 0; }

// whether the four-at-a-time form takes these rows: `wide` pointers hold float32 rows, `narrow` ones rows of the activation
// dtype (8-byte steps of four bfloat16 elements need 8-byte alignment; 16 is asked of all)
bool vector_rows(int width, long stride_a, long stride_b, std::initializer_list<const void*> pointers) {
    if (width % 4 != 0 || width > 4 * 512 * kVecIters || stride_a % 4 != 0 || stride_b % 4 != 0) return false;
    for (const void* p : pointers)
        if (!aligned16(p)) return false;
    return true;
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
    if (vector_rows(width, state_stride, 0, {x, weight, shift, state, h, hs, pending})) {
        const int threads = row_threads(width), iters = vector_iters(width, threads);
#define PB_SHIFT4(T, ITERS) return launch_pdl(norm_shift4_kernel<T, ITERS>, dim3(n), dim3(threads), 0, stream, x, p, (T*)h, (T*)hs, width)
#define PB_SHIFT4_BY_ITERS(T) do { if (iters == 1) PB_SHIFT4(T, 1); if (iters == 2) PB_SHIFT4(T, 2); PB_SHIFT4(T, kVecIters); } while (0)
        if (dtype == PB_F32) PB_SHIFT4_BY_ITERS(float);
        if (dtype == PB_BF16) PB_SHIFT4_BY_ITERS(__nv_bfloat16);
#undef PB_SHIFT4_BY_ITERS
#undef PB_SHIFT4
        return PB_ERR_BAD_DTYPE;
    }
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
    if (vector_rows(width, state_stride, next_state_stride, {x, a, b, x_out, pending, state, next_weight, next_shift, next_state,
                                                             next_pending, h, hs})) {
        const int threads = row_threads(width), iters = vector_iters(width, threads);
#define PB_ADD4(T, ITERS) \
    return launch_pdl(parallel_add4_kernel<T, ITERS>, dim3(n), dim3(threads), 0, stream, x, (const T*)a, (const T*)b, m, x_out, c, nx, \
                      (T*)h, (T*)hs, width)
#define PB_ADD4_BY_ITERS(T) do { if (iters == 1) PB_ADD4(T, 1); if (iters == 2) PB_ADD4(T, 2); PB_ADD4(T, kVecIters); } while (0)
        if (dtype == PB_F32) PB_ADD4_BY_ITERS(float);
        if (dtype == PB_BF16) PB_ADD4_BY_ITERS(__nv_bfloat16);
#undef PB_ADD4_BY_ITERS
#undef PB_ADD4
        return PB_ERR_BAD_DTYPE;
    }
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

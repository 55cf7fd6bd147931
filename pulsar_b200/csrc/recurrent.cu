// Gated recurrences whose gates read the current token only (float32 state, one row per state slot).
//
//   min_gru        proj [N, 3 W] float32 holds, per token, the pre-activations z | u | g of W channels each (biases of z and u
//                  are added here).  z' = sigmoid(z + bz); u' = u + bx; candidate c = u' + 1/2 where u' >= 0, sigmoid(u')
//                  below; S <- (1 - z') S + z' c per channel, token by token from the sequence's kept state; the kernel
//                  writes y = S * silu(g) in the activation dtype and leaves the last S in the kept state.  A thread owns a
//                  channel of a sequence and walks the sequence's tokens of the step in order; the loads of the tokens ahead
//                  do not depend on the recurrence and are kept in flight eight at a time.
//   min_gru_chunked  the same for long portions, parallel over tokens: a portion is cut into runs of kRun tokens; pass 1
//                  gives every (run, channel) its decay product A = prod (1 - z') and its contribution B (the state the run
//                  would leave from zero); pass 2 folds a sequence's runs in order (in segments, a warp each, joined through
//                  shared memory), keeps S_in(run) per run and leaves the final state; pass 3 walks every run again from
//                  its S_in and writes y.  The state entering a run is A * S + B folded over the runs before it, so a
//                  token's value differs from the token-by-token one by rounding only.
#include "common.cuh"

namespace {

using namespace pb;

// FAST (the bfloat16 engine): exponential and reciprocal from the special-function unit (ex2.approx of v log2 e and
// rcp.approx: a few units in the last place of a float32 each, and exactly 0 or 1 where e^-v leaves its range); the kernels
// below spend most of their instructions on these.  The float32 engine keeps the library's exponential and a true division.
template <bool FAST>
__device__ __forceinline__ float sigmoid_of(float v) {
    if (FAST) return __fdividef(1.0f, 1.0f + __expf(-v));
    return 1.0f / (1.0f + expf(-v));
}

template <bool FAST>
__device__ __forceinline__ void gru_gates(float z, float u, float bz, float bx, float& zz, float& cand) {
    zz = sigmoid_of<FAST>(z + bz);
    const float uu = u + bx;
    cand = uu >= 0.0f ? uu + 0.5f : sigmoid_of<FAST>(uu);
}

template <typename T> struct Fast { static constexpr bool value = false; };
template <> struct Fast<__nv_bfloat16> { static constexpr bool value = true; };

template <typename T>
__global__ void min_gru_kernel(const float* __restrict__ proj, const float* __restrict__ bz, const float* __restrict__ bx,
                               float* __restrict__ state, long state_stride, const int* __restrict__ cu_q,
                               const int* __restrict__ state_slots, T* __restrict__ y, int W) {
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (c >= W) return;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    float* kept = state + (size_t)state_slots[s] * state_stride + c;
    float S = *kept;
    const float b_z = bz[c], b_x = bx[c];
    constexpr int U = 8;
    for (int t = t0; t < t1; t += U) {
        float z[U], u[U], g[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const bool on = t + k < t1;
            const float* p = proj + (size_t)(on ? t + k : t) * 3 * W + c;
            z[k] = p[0]; u[k] = p[W]; g[k] = p[2 * W];
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (t + k < t1) {
                float zz, cand;
                gru_gates<Fast<T>::value>(z[k], u[k], b_z, b_x, zz, cand);
                S = (1.0f - zz) * S + zz * cand;
                y[(size_t)(t + k) * W + c] = from_float<T>(S * (g[k] * sigmoid_of<Fast<T>::value>(g[k])));
            }
        }
    }
    *kept = S;
}

constexpr int kRun = 16;

// runs of a step: sequence s has ceil(q_len / kRun) of them; run_seq / run_first list them (built on the device by pass 1's
// first block would need a scan; the host gives an upper bound and every block finds its run by walking cu_q).
__device__ __forceinline__ bool find_run(const int* cu_q, int n_seqs, int run, int& s, int& t0, int& t1, int& index) {
    for (s = 0; s < n_seqs; ++s) {
        const int q0 = cu_q[s], q_len = cu_q[s + 1] - q0;
        const int runs = (q_len + kRun - 1) / kRun;
        if (run < runs) {
            index = run;
            t0 = q0 + run * kRun;
            t1 = min(t0 + kRun, q0 + q_len);
            return true;
        }
        run -= runs;
    }
    return false;
}

template <bool FAST>
__global__ void min_gru_runs_kernel(const float* __restrict__ proj, const float* __restrict__ bz, const float* __restrict__ bx,
                                    const int* __restrict__ cu_q, int n_seqs, float* __restrict__ run_a, float* __restrict__ run_b,
                                    int W) {
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    int s, t0, t1, index;
    if (!find_run(cu_q, n_seqs, blockIdx.y, s, t0, t1, index) || c >= W) return;
    const float b_z = bz[c], b_x = bx[c];
    float A = 1.0f, B = 0.0f;
    constexpr int U = 8;
    for (int t = t0; t < t1; t += U) {
        float z[U], u[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const float* p = proj + (size_t)(t + k < t1 ? t + k : t) * 3 * W + c;
            z[k] = p[0]; u[k] = p[W];
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (t + k < t1) {
                float zz, cand;
                gru_gates<FAST>(z[k], u[k], b_z, b_x, zz, cand);
                A = (1.0f - zz) * A;
                B = (1.0f - zz) * B + zz * cand;
            }
        }
    }
    run_a[(size_t)blockIdx.y * W + c] = A;
    run_b[(size_t)blockIdx.y * W + c] = B;
}

// per (sequence, channel): the state that enters each of the sequence's runs (written over run_b), and the final state.
// A block takes 32 channels (a lane each) and cuts the sequence's runs into kCarryWarps segments, a warp each: the warp
// folds its segment from (1, 0) with all its loads in flight, the segments' products meet in shared memory, every warp
// folds the ones before it onto the kept state, and walks its segment again from there.  The first kCarryKeep runs of a
// segment stay in registers between the two walks (portions up to kCarryWarps * kCarryKeep runs: all of them).
constexpr int kCarryWarps = 8, kCarryKeep = 16;

__global__ void __launch_bounds__(kCarryWarps * 32)
min_gru_carry_kernel(const float* __restrict__ run_a, float* __restrict__ run_b, float* __restrict__ state, long state_stride,
                     const int* __restrict__ cu_q, const int* __restrict__ state_slots, int W) {
    pdl_wait();
    __shared__ float As[kCarryWarps][32], Bs[kCarryWarps][32];
    const int lane = threadIdx.x & 31, j = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane, s = blockIdx.y;
    const bool on = c < W;
    int run0 = 0;
    for (int k = 0; k < s; ++k) run0 += (cu_q[k + 1] - cu_q[k] + kRun - 1) / kRun;
    const int runs = (cu_q[s + 1] - cu_q[s] + kRun - 1) / kRun;
    const int seg = (runs + kCarryWarps - 1) / kCarryWarps;
    const int r0 = min(j * seg, runs), r1 = min(r0 + seg, runs);
    float* kept = state + (size_t)state_slots[s] * state_stride + c;
    float A[kCarryKeep], B[kCarryKeep];
    float a_seg = 1.0f, b_seg = 0.0f, S = 0.0f;
    if (on) {
        S = *kept;
#pragma unroll
        for (int k = 0; k < kCarryKeep; ++k) {
            if (r0 + k < r1) {
                const size_t at = (size_t)(run0 + r0 + k) * W + c;
                A[k] = run_a[at]; B[k] = run_b[at];
            }
        }
#pragma unroll
        for (int k = 0; k < kCarryKeep; ++k)
            if (r0 + k < r1) { a_seg *= A[k]; b_seg = A[k] * b_seg + B[k]; }
#pragma unroll 4
        for (int r = r0 + kCarryKeep; r < r1; ++r) {
            const size_t at = (size_t)(run0 + r) * W + c;
            const float a = run_a[at], b = run_b[at];
            a_seg *= a; b_seg = a * b_seg + b;
        }
    }
    As[j][lane] = a_seg; Bs[j][lane] = b_seg;
    __syncthreads();                                       // every warp has read the kept state by now
    if (!on) return;
    for (int jj = 0; jj < j; ++jj) S = As[jj][lane] * S + Bs[jj][lane];
#pragma unroll
    for (int k = 0; k < kCarryKeep; ++k) {
        if (r0 + k < r1) {
            run_b[(size_t)(run0 + r0 + k) * W + c] = S;
            S = A[k] * S + B[k];
        }
    }
    for (int r = r0 + kCarryKeep; r < r1; ++r) {
        const size_t at = (size_t)(run0 + r) * W + c;
        const float a = run_a[at], b = run_b[at];
        run_b[at] = S;
        S = a * S + b;
    }
    if (j == kCarryWarps - 1) *kept = S;                   // the last warp's walk ends at the sequence's end, whatever its share
}

template <typename T>
__global__ void min_gru_outputs_kernel(const float* __restrict__ proj, const float* __restrict__ bz, const float* __restrict__ bx,
                                       const int* __restrict__ cu_q, int n_seqs, const float* __restrict__ run_in,
                                       T* __restrict__ y, int W) {
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    int s, t0, t1, index;
    if (!find_run(cu_q, n_seqs, blockIdx.y, s, t0, t1, index) || c >= W) return;
    const float b_z = bz[c], b_x = bx[c];
    float S = run_in[(size_t)blockIdx.y * W + c];
    constexpr int U = 8;
    for (int t = t0; t < t1; t += U) {
        float z[U], u[U], g[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const float* p = proj + (size_t)(t + k < t1 ? t + k : t) * 3 * W + c;
            z[k] = p[0]; u[k] = p[W]; g[k] = p[2 * W];
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (t + k < t1) {
                float zz, cand;
                gru_gates<Fast<T>::value>(z[k], u[k], b_z, b_x, zz, cand);
                S = (1.0f - zz) * S + zz * cand;
                y[(size_t)(t + k) * W + c] = from_float<T>(S * (g[k] * sigmoid_of<Fast<T>::value>(g[k])));
            }
        }
    }
}

}  // namespace

PB_EXPORT int pb_min_gru_run() { return kRun; }

// proj [n, 3 W] float32; bz, bx [W] float32; state: float32 rows of state_stride elements, the first W of a row are this
// recurrence's; y [n, W] in `dtype`.  max_runs > 0: the form that is parallel over tokens, with workspace run_a / run_b
// [max_runs, W] float32 (max_runs >= the step's number of runs, sum over its sequences of ceil(q_len / pb_min_gru_run())).
PB_EXPORT int pb_min_gru(int dtype, const float* proj, const float* bz, const float* bx, float* state, long state_stride,
                         const int* cu_q, const int* state_slots, void* y, int n, int n_seqs, int W, int max_runs, float* run_a,
                         float* run_b, cudaStream_t stream) {
    if (n <= 0 || n_seqs <= 0) return 0;
    if (W <= 0 || state_stride < W) return PB_ERR_BAD_SIZE;
    if (dtype != PB_F32 && dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
    if (n_seqs > 65535 || max_runs > 65535) return PB_ERR_TOO_LARGE;
    const int threads = W >= 128 ? 128 : (W + 31) / 32 * 32;
    const dim3 block(threads), grid_s((W + threads - 1) / threads, n_seqs);
    if (max_runs <= 0) {
        if (dtype == PB_F32)
            return launch_pdl(min_gru_kernel<float>, grid_s, block, 0, stream, proj, bz, bx, state, state_stride, cu_q, state_slots, (float*)y, W);
        return launch_pdl(min_gru_kernel<__nv_bfloat16>, grid_s, block, 0, stream, proj, bz, bx, state, state_stride, cu_q, state_slots,
                          (__nv_bfloat16*)y, W);
    }
    if (run_a == nullptr || run_b == nullptr) return PB_ERR_BAD_SIZE;
    const dim3 grid_r((W + threads - 1) / threads, max_runs);
    int rc = dtype == PB_F32 ? launch_pdl(min_gru_runs_kernel<false>, grid_r, block, 0, stream, proj, bz, bx, cu_q, n_seqs, run_a, run_b, W)
                             : launch_pdl(min_gru_runs_kernel<true>, grid_r, block, 0, stream, proj, bz, bx, cu_q, n_seqs, run_a, run_b, W);
    if (rc != 0) return rc;
    rc = launch_pdl(min_gru_carry_kernel, dim3((W + 31) / 32, n_seqs), dim3(kCarryWarps * 32), 0, stream, (const float*)run_a, run_b, state,
                    state_stride, cu_q, state_slots, W);
    if (rc != 0) return rc;
    if (dtype == PB_F32)
        return launch_pdl(min_gru_outputs_kernel<float>, grid_r, block, 0, stream, proj, bz, bx, cu_q, n_seqs, (const float*)run_b, (float*)y, W);
    return launch_pdl(min_gru_outputs_kernel<__nv_bfloat16>, grid_r, block, 0, stream, proj, bz, bx, cu_q, n_seqs, (const float*)run_b,
                      (__nv_bfloat16*)y, W);
}

// Selective scan (Mamba): a diagonal state space per channel whose step size and input and
// output maps depend on the token.  Per channel c and state index n, S a float32 state carried
// from token to token in the request's slot [rows, inner, states]:
//   dt = softplus(dt_raw[c] + dt_bias[c])
//   S[c][n] = exp(dt * A[c][n]) * S[c][n] + dt * x[c] * B[n],      A = -exp(A_log)
//   y[c] = sum_n S[c][n] * C[n] + D[c] * x[c]
//   out[c] = y[c] * silu(z[c])
// Step sizes, decays, exponentials and the state are float32; x, z, B and C come in the model dtype.
//
// A block serves some channels of one request and walks its tokens of the step in order; TS
// threads share a channel (thread l owns states l, l + TS, ...) and add their parts of y by
// shuffles in a fixed order.  B and C of a few tokens at a time go through shared memory.
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

constexpr int THREADS = 128;
constexpr int TOKENS = 16;       // tokens whose B and C are staged (and whose dt, x, z are loaded) at once
constexpr int NPT = 8;           // states per thread at most

struct ScanArgs {
    const void* x;           // [N, x_stride] in T, channel c at column c
    long long x_stride;
    const void* z;           // [N, z_stride] in T
    long long z_stride;
    const float* dt_raw;     // [N, inner]
    const float* dt_bias;    // [inner]
    const void* bc;          // [N, bc_stride] in T: B (states) | C (states)
    long long bc_stride;
    const float* A_log;      // [inner, states]
    const float* D;          // [inner]
    float* state;            // [rows, inner, states]
    void* out;               // [N, inner] in T
    const int* seq_starts;
    const int* seq_rows;
    int inner, states, TS;
};

template <typename T>
__global__ void __launch_bounds__(THREADS) selective_scan_kernel(ScanArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ float bcs[];          // TOKENS * 2 * states
    const int TS = a.TS, states = a.states;
    const int tid = threadIdx.x;
    const int l = tid % TS;
    const int c = blockIdx.x * (THREADS / TS) + tid / TS;
    const bool live = c < a.inner;
    const int r = blockIdx.y;
    float A[NPT], S[NPT];
#pragma unroll
    for (int e = 0; e < NPT; ++e) {
        const int n = l + e * TS;
        A[e] = (live && n < states) ? -expf(a.A_log[(size_t)c * states + n]) : 0.f;
    }
    const float bias = live ? a.dt_bias[c] : 0.f;
    const float Dc = live ? a.D[c] : 0.f;
    sb::pdl_wait();
    const int n0 = a.seq_starts[r], n1 = a.seq_starts[r + 1];
    const int row = a.seq_rows[r];
    float* st = a.state + ((size_t)row * a.inner + (live ? c : 0)) * states;
#pragma unroll
    for (int e = 0; e < NPT; ++e) {
        const int n = l + e * TS;
        S[e] = (live && n < states) ? st[n] : 0.f;
    }
    const T* xs = (const T*)a.x;
    const T* zs = (const T*)a.z;
    const T* bc = (const T*)a.bc;
    for (int t0 = n0; t0 < n1; t0 += TOKENS) {
        const int nt = min(TOKENS, n1 - t0);
        __syncthreads();
        for (int i = tid; i < nt * 2 * states; i += THREADS) {
            const int t = i / (2 * states), k = i - t * 2 * states;
            bcs[i] = to_float(bc[(size_t)(t0 + t) * a.bc_stride + k]);
        }
        __syncthreads();
        // the tokens' own values: all loads go out before the first is used (one round trip for the batch)
        float raws[TOKENS], xvs[TOKENS], zvs[TOKENS];
#pragma unroll
        for (int t = 0; t < TOKENS; ++t) {
            raws[t] = xvs[t] = zvs[t] = 0.f;
            if (live && t < nt) {
                const int n = t0 + t;
                raws[t] = a.dt_raw[(size_t)n * a.inner + c];
                xvs[t] = to_float(xs[(size_t)n * a.x_stride + c]);
                if (l == 0) zvs[t] = to_float(zs[(size_t)n * a.z_stride + c]);
            }
        }
#pragma unroll
        for (int t = 0; t < TOKENS; ++t) {
            if (t >= nt) break;
            const int n = t0 + t;
            const float raw = raws[t] + bias;
            const float dt = live ? (raw > 20.f ? raw : log1pf(expf(raw))) : 0.f;
            const float xv = xvs[t];
            const float* Bt = bcs + t * 2 * states;
            const float* Ct = Bt + states;
            const float dx = dt * xv;
            float y = 0.f;
#pragma unroll
            for (int e = 0; e < NPT; ++e) {
                const int k = l + e * TS;
                if (k < states) {
                    S[e] = fmaf(expf(dt * A[e]), S[e], dx * Bt[k]);
                    y = fmaf(S[e], Ct[k], y);
                }
            }
            for (int o = TS >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (live && l == 0) {
                y += Dc * xv;
                const float zv = zvs[t];
                ((T*)a.out)[(size_t)n * a.inner + c] = from_float<T>(y * (zv / (1.0f + expf(-zv))));
            }
        }
    }
    if (live) {
#pragma unroll
        for (int e = 0; e < NPT; ++e) {
            const int n = l + e * TS;
            if (n < states) st[n] = S[e];
        }
    }
}

}  // namespace

extern "C" int sb_selective_scan(const void* x, long long x_stride, const void* z, long long z_stride,
                                 const float* dt_raw, const float* dt_bias, const void* bc, long long bc_stride,
                                 const float* A_log, const float* D, float* state, void* out,
                                 const int* seq_starts, const int* seq_rows, int R, int inner, int states,
                                 int dtype, cudaStream_t stream) {
    SB_REQUIRE(R >= 0 && inner > 0 && states > 0 && states <= 32 * NPT,
               "selective_scan: bad sizes R=%d inner=%d states=%d (at most %d)", R, inner, states, 32 * NPT);
    SB_REQUIRE(R <= 65535, "selective_scan: %d requests exceed one launch", R);
    if (R == 0) return 0;
    int TS = 1;
    while (TS < 32 && TS * 2 <= states) TS *= 2;          // threads a channel: a power of two, at most the states
    while (TS * NPT < states) TS *= 2;
    ScanArgs a;
    a.x = x; a.x_stride = x_stride; a.z = z; a.z_stride = z_stride; a.dt_raw = dt_raw; a.dt_bias = dt_bias;
    a.bc = bc; a.bc_stride = bc_stride; a.A_log = A_log; a.D = D; a.state = state; a.out = out;
    a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.inner = inner; a.states = states; a.TS = TS;
    const int per_block = THREADS / TS;
    dim3 grid((inner + per_block - 1) / per_block, R);
    const size_t smem = (size_t)TOKENS * 2 * states * sizeof(float);
    if (dtype == SB_F32) sb::launch(selective_scan_kernel<float>, grid, dim3(THREADS), smem, stream, a);
    else if (dtype == SB_BF16) sb::launch(selective_scan_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream, a);
    else SB_REQUIRE(false, "selective_scan: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

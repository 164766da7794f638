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
    extern __shared__ float bcs[];          // TOKENS * 2 * states, then (dt, dt*x, D*x, silu(z)) per channel and token
    float* tok = bcs + TOKENS * 2 * a.states;
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
        // The tokens' own values, made once per channel: lane l of a channel's group takes the tokens
        // t = l, l + TS, ... (loads first, all in flight), computes the step size, its product with x and
        // the output gate, and leaves them in shared memory for the group.
        {
            float raws[TOKENS], xv[TOKENS], zv[TOKENS];
#pragma unroll
            for (int k = 0; k < TOKENS; ++k) {
                const int t = l + k * TS;
                raws[k] = xv[k] = zv[k] = 0.f;
                if (live && t < nt) {
                    const int n = t0 + t;
                    raws[k] = a.dt_raw[(size_t)n * a.inner + c];
                    xv[k] = to_float(xs[(size_t)n * a.x_stride + c]);
                    zv[k] = to_float(zs[(size_t)n * a.z_stride + c]);
                }
            }
#pragma unroll
            for (int k = 0; k < TOKENS; ++k) {
                const int t = l + k * TS;
                if (t < nt) {
                    const float raw = raws[k] + bias;
                    const float dt = raw > 20.f ? raw : log1pf(expf(raw));
                    float* o = tok + ((tid / TS) * TOKENS + t) * 4;
                    o[0] = dt;
                    o[1] = dt * xv[k];
                    o[2] = Dc * xv[k];
                    o[3] = zv[k] / (1.0f + expf(-zv[k]));
                }
            }
        }
        __syncwarp();
#pragma unroll 4
        for (int t = 0; t < nt; ++t) {
            const float4 v = *reinterpret_cast<const float4*>(tok + ((tid / TS) * TOKENS + t) * 4);
            const float dt = v.x, dx = v.y;
            const float* Bt = bcs + t * 2 * states;
            const float* Ct = Bt + states;
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
            if (live && l == 0) ((T*)a.out)[(size_t)(t0 + t) * a.inner + c] = from_float<T>((y + v.z) * v.w);
        }
        __syncwarp();
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
    // threads a channel: a power of two, as few as hold the states at NPT each (what a thread does per token
    // beside its states is the same for every thread of a channel), but four where the states allow it
    int TS = 1;
    while (TS * NPT < states) TS *= 2;
    while (TS < 4 && TS * 2 <= states) TS *= 2;
    ScanArgs a;
    a.x = x; a.x_stride = x_stride; a.z = z; a.z_stride = z_stride; a.dt_raw = dt_raw; a.dt_bias = dt_bias;
    a.bc = bc; a.bc_stride = bc_stride; a.A_log = A_log; a.D = D; a.state = state; a.out = out;
    a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.inner = inner; a.states = states; a.TS = TS;
    const int per_block = THREADS / TS;
    dim3 grid((inner + per_block - 1) / per_block, R);
    const size_t smem = ((size_t)TOKENS * 2 * states + (size_t)per_block * TOKENS * 4) * sizeof(float);
    if (dtype == SB_F32) sb::launch(selective_scan_kernel<float>, grid, dim3(THREADS), smem, stream, a);
    else if (dtype == SB_BF16) sb::launch(selective_scan_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream, a);
    else SB_REQUIRE(false, "selective_scan: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

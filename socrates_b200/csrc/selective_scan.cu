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

// exp of a decay's exponent (dt * A <= 0).  The float32 engine uses expf; in the bfloat16 engine, whose
// activations carry 8 bits, the hardware exponential (a relative error near 1e-6) is far below what the
// activations' rounding leaves, and the kernel is bound by these instructions.
template <typename T> __device__ __forceinline__ float decay_exp(float x) { return expf(x); }
template <> __device__ __forceinline__ float decay_exp<__nv_bfloat16>(float x) { return __expf(x); }

constexpr int THREADS = 128;
constexpr int TOKENS = 16;       // tokens whose B and C are staged (and whose dt, x, z are loaded) at once
constexpr int NPT = 8;           // states per thread at most
constexpr int SEGMENT = 128;     // tokens per segment of the three-launch form (a multiple of TOKENS)

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
    int R, seg;              // requests of the step; tokens per segment of the three-launch form
    float* seg_state;        // [segments of the step, inner, states]
    float* seg_dt;           // [segments of the step, inner]: the sum of the step sizes in the segment
};

// The segments of a step in one list: request 0's, then request 1's, ...  Finds segment g's request and its
// number within the request; false if the step has fewer segments.
__device__ __forceinline__ bool find_segment(int g, const int* seq_starts, int R, int len, int& r, int& si) {
    for (r = 0; r < R; ++r) {
        const int ns = (seq_starts[r + 1] - seq_starts[r] + len - 1) / len;
        if (g < ns) { si = g; return true; }
        g -= ns;
    }
    return false;
}

// MODE 0: a block walks all tokens of its request (decode steps; many requests).  One long prompt has too
// few channels to fill the GPU that way (a warp per scheduler, every step's latency exposed), so it runs as
// three launches over segments of `seg` tokens, each segment a block row of its own:
// MODE 1: the segment from a zero state: its final state and the sum of its step sizes, to scratch;
// (selective_scan_join_kernel walks a request's segments: S <- exp(A * sum dt) S + contribution, and leaves
//  the state BEFORE each segment in scratch and the state after the last in the request's slot;)
// MODE 2: the segment again from the state before it, this time writing the outputs.
template <typename T, int MODE>
__global__ void __launch_bounds__(THREADS) selective_scan_kernel(ScanArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ float bcs[];          // TOKENS * 2 * states, then (dt, dt*x, D*x, silu(z)) per channel and token
    float* tok = bcs + TOKENS * 2 * a.states;
    const int TS = a.TS, states = a.states;
    const int tid = threadIdx.x;
    const int l = tid % TS;
    const int c = blockIdx.x * (THREADS / TS) + tid / TS;
    const bool live = c < a.inner;
    int r = blockIdx.y, si = 0;
    float A[NPT], S[NPT];
#pragma unroll
    for (int e = 0; e < NPT; ++e) {
        const int n = l + e * TS;
        A[e] = (live && n < states) ? -expf(a.A_log[(size_t)c * states + n]) : 0.f;
    }
    const float bias = live ? a.dt_bias[c] : 0.f;
    const float Dc = live ? a.D[c] : 0.f;
    sb::pdl_wait();
    if (MODE != 0 && !find_segment(blockIdx.y, a.seq_starts, a.R, a.seg, r, si)) return;
    const int n0 = MODE == 0 ? a.seq_starts[r] : a.seq_starts[r] + si * a.seg;
    const int n1 = MODE == 0 ? a.seq_starts[r + 1] : min(a.seq_starts[r + 1], n0 + a.seg);
    const int row = a.seq_rows[r];
    float* st = MODE == 0 ? a.state + ((size_t)row * a.inner + (live ? c : 0)) * states
                          : a.seg_state + ((size_t)blockIdx.y * a.inner + (live ? c : 0)) * states;
#pragma unroll
    for (int e = 0; e < NPT; ++e) {
        const int n = l + e * TS;
        S[e] = (MODE != 1 && live && n < states) ? st[n] : 0.f;
    }
    float dt_sum = 0.f;
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
                    dt_sum += dt;
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
                    S[e] = fmaf(decay_exp<T>(dt * A[e]), S[e], dx * Bt[k]);
                    y = fmaf(S[e], Ct[k], y);
                }
            }
            if (MODE != 1) {
                for (int o = TS >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                if (live && l == 0) ((T*)a.out)[(size_t)(t0 + t) * a.inner + c] = from_float<T>((y + v.z) * v.w);
            }
        }
        __syncwarp();
    }
    if (MODE == 1) {
        for (int o = TS >> 1; o > 0; o >>= 1) dt_sum += __shfl_xor_sync(0xffffffffu, dt_sum, o);
        if (live && l == 0) a.seg_dt[(size_t)blockIdx.y * a.inner + c] = dt_sum;
    }
    if (live && MODE != 2) {
#pragma unroll
        for (int e = 0; e < NPT; ++e) {
            const int n = l + e * TS;
            if (n < states) st[n] = S[e];
        }
    }
}

// Between MODE 1 and MODE 2: one thread per (channel, state) of a request walks its segments.
__global__ void __launch_bounds__(256) selective_scan_join_kernel(ScanArgs a) {
    sb::pdl_launch_dependents();
    const int i = blockIdx.x * 256 + threadIdx.x, r = blockIdx.y;
    const int size = a.inner * a.states;
    const float A = i < size ? -expf(a.A_log[i]) : 0.f;
    sb::pdl_wait();
    if (i >= size) return;
    int base = 0;
    for (int q = 0; q < r; ++q) base += (a.seq_starts[q + 1] - a.seq_starts[q] + a.seg - 1) / a.seg;
    const int ns = (a.seq_starts[r + 1] - a.seq_starts[r] + a.seg - 1) / a.seg;
    const int c = i / a.states;
    float* slot = a.state + (size_t)a.seq_rows[r] * size + i;
    float s = *slot;
    for (int g0 = 0; g0 < ns; g0 += 8) {                         // eight segments' loads in flight
        float u[8], d[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (g0 + k < ns) {
                u[k] = a.seg_state[(size_t)(base + g0 + k) * size + i];
                d[k] = a.seg_dt[(size_t)(base + g0 + k) * a.inner + c];
            }
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (g0 + k < ns) {
                a.seg_state[(size_t)(base + g0 + k) * size + i] = s;
                s = fmaf(expf(A * d[k]), s, u[k]);
            }
    }
    *slot = s;
}

}  // namespace

extern "C" int sb_selective_scan(const void* x, long long x_stride, const void* z, long long z_stride,
                                 const float* dt_raw, const float* dt_bias, const void* bc, long long bc_stride,
                                 const float* A_log, const float* D, float* state, void* out,
                                 const int* seq_starts, const int* seq_rows, int R, int inner, int states, int N,
                                 float* scratch, long long scratch_floats, int dtype, cudaStream_t stream) {
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
    SB_REQUIRE(dtype == SB_F32 || dtype == SB_BF16, "selective_scan: unknown dtype %d", dtype);
    // few requests with long portions: segments in parallel (three launches) if the caller lent scratch
    const int segs = (N + SEGMENT - 1) / SEGMENT + R;
    const bool spread = scratch != nullptr && (int)grid.x * R < 4 * 148 && segs > 2 * R &&
                        (long long)segs * inner * (states + 1) <= scratch_floats;
    a.R = R; a.seg = SEGMENT; a.seg_state = scratch; a.seg_dt = scratch ? scratch + (size_t)segs * inner * states : nullptr;
    if (!spread) {
        if (dtype == SB_F32) sb::launch(selective_scan_kernel<float, 0>, grid, dim3(THREADS), smem, stream, a);
        else sb::launch(selective_scan_kernel<__nv_bfloat16, 0>, grid, dim3(THREADS), smem, stream, a);
        SB_LAUNCH_CHECK();
    }
    dim3 sgrid(grid.x, segs), jgrid((inner * states + 255) / 256, R);
    if (dtype == SB_F32) {
        sb::launch(selective_scan_kernel<float, 1>, sgrid, dim3(THREADS), smem, stream, a);
        sb::launch(selective_scan_join_kernel, jgrid, dim3(256), 0, stream, a);
        sb::launch(selective_scan_kernel<float, 2>, sgrid, dim3(THREADS), smem, stream, a);
    } else {
        sb::launch(selective_scan_kernel<__nv_bfloat16, 1>, sgrid, dim3(THREADS), smem, stream, a);
        sb::launch(selective_scan_join_kernel, jgrid, dim3(256), 0, stream, a);
        sb::launch(selective_scan_kernel<__nv_bfloat16, 2>, sgrid, dim3(THREADS), smem, stream, a);
    }
    SB_LAUNCH_CHECK();
}

// float32 elements of scratch with which a step of N tokens of R requests can run its segments in parallel.
extern "C" long long sb_selective_scan_scratch(int N, int R, int inner, int states) {
    return (long long)((N + SEGMENT - 1) / SEGMENT + R) * inner * (states + 1);
}

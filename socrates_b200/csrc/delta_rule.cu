// Gated delta rule: a recurrent mixer whose state is a matrix per head that is decayed, corrected
// towards the new value along the new key, and read with the query.
//
//   q_t = unit(q_t) * D^-1/2 ,  k_t = unit(k_t)            unit(x) = x / sqrt(sum(x^2) + 1e-6)
//   beta_t = sigmoid(b_t) ,  g_t = exp(-exp(A_log) * softplus(a_t + dt_bias))        (per head)
//   S <- g_t S ;  u = beta_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
//   y_t = o_t / sqrt(mean(o_t^2) + eps) * w * silu(gate_t)
//
// Value head h uses query/key head h / (H / G).  The state S [D, Dv] is float32 and lives in the
// request's state slot; everything above is float32, only q, k, v, gate, a, b arrive in the model
// dtype (they are matrix products and convolutions) and y leaves in it.
//
// A block serves one (request, value head) and walks the request's tokens of the step in order.
// Thread j owns column j of S (Dv columns, D rows in registers): the columns of S never mix, so
// the only exchange between threads is the sum of o^2 for the norm.  q_t and k_t sit in the lanes
// of every warp (lane l holds dims l, l + 32, ...) and are handed round by shuffles.
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

struct DeltaArgs {
    const void* qkv;       // [N, qkv_stride] in T: q at q_off, k at k_off (G heads of D), v at v_off (H heads of Dv)
    long long qkv_stride;
    int q_off, k_off, v_off;
    const void* proj;      // [N, proj_stride] in T: gate at gate_off (H*Dv), b at b_off (H), a at a_off (H)
    long long proj_stride;
    int gate_off, b_off, a_off;
    const float* A_log;    // [H]
    const float* dt_bias;  // [H]
    const float* norm_w;   // [Dv]
    float* state;          // [rows, H, D, Dv]
    void* out;             // [N, H*Dv] in T
    const int* seq_starts; // [R + 1]
    const int* seq_rows;   // [R]
    int H, G, D, Dv;
    float eps, q_scale;
};

__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T, int DC>
__global__ void __launch_bounds__(256) delta_rule_kernel(DeltaArgs a) {
    sb::pdl_launch_dependents();
    __shared__ float red[2][8];
    const int h = blockIdx.x, r = blockIdx.y;
    const int j = threadIdx.x, lane = j & 31, warp = j >> 5, nwarps = blockDim.x >> 5;
    const int D = a.D, Dv = a.Dv;
    const int kh = h / (a.H / a.G);
    const bool col = j < Dv;
    const float neg_rate = -expf(a.A_log[h]);
    const float dt_bias = a.dt_bias[h];
    const float w = col ? a.norm_w[j] : 0.f;
    sb::pdl_wait();
    const int t0 = a.seq_starts[r], t1 = a.seq_starts[r + 1];
    if (t0 >= t1) return;
    float* sp = a.state + ((size_t)a.seq_rows[r] * a.H + h) * D * Dv + j;
    float S[DC * 32];
#pragma unroll
    for (int i = 0; i < DC * 32; ++i) S[i] = (col && i < D) ? sp[(size_t)i * Dv] : 0.f;

    const T* qkv = (const T*)a.qkv;
    const T* proj = (const T*)a.proj;
    for (int t = t0; t < t1; ++t) {
        const T* xr = qkv + (size_t)t * a.qkv_stride;
        const T* pr = proj + (size_t)t * a.proj_stride;
        float kreg[DC], qreg[DC];
        float kss = 0.f, qss = 0.f;
#pragma unroll
        for (int c = 0; c < DC; ++c) {
            const int d = c * 32 + lane;
            kreg[c] = d < D ? to_float(xr[a.k_off + kh * D + d]) : 0.f;
            qreg[c] = d < D ? to_float(xr[a.q_off + kh * D + d]) : 0.f;
            kss += kreg[c] * kreg[c];
            qss += qreg[c] * qreg[c];
        }
        const float v = col ? to_float(xr[a.v_off + h * Dv + j]) : 0.f;
        const float gate = col ? to_float(pr[a.gate_off + h * Dv + j]) : 0.f;
        const float beta = 1.0f / (1.0f + expf(-to_float(pr[a.b_off + h])));
        const float decay = expf(neg_rate * softplus(to_float(pr[a.a_off + h]) + dt_bias));
        kss = warp_sum(kss);
        qss = warp_sum(qss);
        const float kinv = 1.0f / sqrtf(kss + 1e-6f), qinv = a.q_scale / sqrtf(qss + 1e-6f);
#pragma unroll
        for (int c = 0; c < DC; ++c) { kreg[c] *= kinv; qreg[c] *= qinv; }
        // what the decayed state already answers along k
        float rk = 0.f;
#pragma unroll
        for (int c = 0; c < DC; ++c)
#pragma unroll
            for (int l = 0; l < 32; ++l) rk = fmaf(S[c * 32 + l], __shfl_sync(0xffffffffu, kreg[c], l), rk);
        const float u = beta * (v - decay * rk);
        float o = 0.f;
#pragma unroll
        for (int c = 0; c < DC; ++c)
#pragma unroll
            for (int l = 0; l < 32; ++l) {
                const float s = fmaf(__shfl_sync(0xffffffffu, kreg[c], l), u, decay * S[c * 32 + l]);
                S[c * 32 + l] = s;
                o = fmaf(s, __shfl_sync(0xffffffffu, qreg[c], l), o);
            }
        // the head's root mean square over the value dims: a sum over the block's warps
        float ss = warp_sum(col ? o * o : 0.f);
        if (nwarps > 1) {
            float* rd = red[(t - t0) & 1];
            if (lane == 0) rd[warp] = ss;
            __syncthreads();
            ss = 0.f;
            for (int x = 0; x < nwarps; ++x) ss += rd[x];
        }
        const float rinv = 1.0f / sqrtf(ss / (float)Dv + a.eps);
        if (col)
            ((T*)a.out)[(size_t)t * a.H * Dv + h * Dv + j] = from_float<T>(o * rinv * w * (gate / (1.0f + expf(-gate))));
    }
#pragma unroll
    for (int i = 0; i < DC * 32; ++i)
        if (col && i < D) sp[(size_t)i * Dv] = S[i];
}

template <typename T>
int launch_delta(const DeltaArgs& a, int R, cudaStream_t stream) {
    const int threads = ((a.Dv + 31) / 32) * 32;
    const dim3 grid(a.H, R);
    switch ((a.D + 31) / 32) {
        case 1: sb::launch(delta_rule_kernel<T, 1>, grid, dim3(threads), 0, stream, a); break;
        case 2: sb::launch(delta_rule_kernel<T, 2>, grid, dim3(threads), 0, stream, a); break;
        case 3: sb::launch(delta_rule_kernel<T, 3>, grid, dim3(threads), 0, stream, a); break;
        default: sb::launch(delta_rule_kernel<T, 4>, grid, dim3(threads), 0, stream, a); break;
    }
    SB_LAUNCH_CHECK();
}

}  // namespace

// Largest key and value head sizes the kernel takes.
extern "C" int sb_delta_rule_supports(int D, int Dv) { return D >= 1 && D <= 128 && Dv >= 1 && Dv <= 256; }

extern "C" int sb_delta_rule(void* out, const void* qkv, long long qkv_stride, int q_off, int k_off, int v_off,
                             const void* proj, long long proj_stride, int gate_off, int b_off, int a_off,
                             const float* A_log, const float* dt_bias, const float* norm_w, float* state,
                             const int* seq_starts, const int* seq_rows, int R, int H, int G, int D, int Dv,
                             float eps, float q_scale, int dtype, cudaStream_t stream) {
    SB_REQUIRE(R >= 0 && H > 0 && G > 0 && H % G == 0, "delta_rule: %d value heads are no multiple of %d key heads", H, G);
    SB_REQUIRE(sb_delta_rule_supports(D, Dv), "delta_rule: heads of %d (keys, at most 128) and %d (values, at most 256) dims", D, Dv);
    SB_REQUIRE(R <= 65535, "delta_rule: %d requests exceed one launch", R);
    if (R == 0) return 0;
    DeltaArgs a;
    a.qkv = qkv; a.qkv_stride = qkv_stride; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.proj = proj; a.proj_stride = proj_stride; a.gate_off = gate_off; a.b_off = b_off; a.a_off = a_off;
    a.A_log = A_log; a.dt_bias = dt_bias; a.norm_w = norm_w; a.state = state; a.out = out;
    a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.H = H; a.G = G; a.D = D; a.Dv = Dv;
    a.eps = eps; a.q_scale = q_scale;
    if (dtype == SB_F32) return launch_delta<float>(a, R, stream);
    if (dtype == SB_BF16) return launch_delta<__nv_bfloat16>(a, R, stream);
    SB_REQUIRE(false, "delta_rule: unknown dtype %d", dtype);
}

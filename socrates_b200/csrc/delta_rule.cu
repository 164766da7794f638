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
// A block serves 8 columns of the state of one (request, value head) and walks the request's tokens
// of the step in order.  The columns of S never mix, so blocks need nothing from one another; the
// sum of o^2 over a head's columns, the norm and the gate are a second, elementwise kernel that
// reads the raw o.  Sixteen neighbouring threads share a column (a sixteenth of the D rows each, in
// registers; four shuffles join their partial dot products).  Tokens are staged eight at a time
// by four more warps of the block: they load q and k, make them unit vectors and leave them in
// shared memory with beta, the decay and the values beside them, into one of two buffers while the
// walking warps are busy with the other, so the serial walk waits neither for a global load nor for
// a norm, an exponential or a logarithm.
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
    float* raw_o;          // [N, H*Dv]: o before the norm and the gate
    const int* seq_starts; // [R + 1]
    const int* seq_rows;   // [R]
    int H, G, D, Dv;
    float eps, q_scale;
};

__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

constexpr int RG = 16;                // threads that share a column of the state
constexpr int COLS = 8;               // columns of a block
constexpr int TB = 8;                 // tokens staged at a time
constexpr int WALKERS = COLS * RG;    // 128 threads walk the tokens ...
constexpr int STAGERS = 128;          // ... and 128 prepare the next ones meanwhile
constexpr int THREADS = WALKERS + STAGERS;
constexpr int TPW = TB / (STAGERS / 32);     // tokens a staging warp prepares

// DR rows of the state per thread (D <= RG * DR); in shared memory the sixteen parts of a q or k
// vector are 12 floats apart, so that the 16-byte reads of eight neighbouring parts fall into different
// banks.  (The walk is bound by how fast ONE warp issues dependent instructions, about 4.8 clocks each:
// with four threads a column and 32 rows a thread a token cost 136 instructions, 655 clocks; sixteen
// threads a column halve the instructions and double the blocks, so that SMs interleave two blocks' warps.)
template <typename T, int DR>
__global__ void __launch_bounds__(THREADS) delta_rule_kernel(DeltaArgs a) {
    sb::pdl_launch_dependents();
    constexpr int ST = DR <= 8 ? 12 : DR + 4;         // floats from one part to the next: an odd number of 16-byte pieces
    constexpr int PITCH = RG * ST;
    constexpr int DC = (RG * DR + 31) / 32;          // values of a vector per lane while staging
    __shared__ __align__(16) float ks[2][TB][PITCH];
    __shared__ __align__(16) float qs[2][TB][PITCH];
    __shared__ float vs[2][TB][COLS], beta_s[2][TB], decay_s[2][TB], os[TB][COLS];
    const int h = blockIdx.x, r = blockIdx.y, c0 = blockIdx.z * COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool walker = tid < WALKERS;
    const int D = a.D, Dv = a.Dv, H = a.H;
    const int kh = h / (H / a.G);
    const float neg_rate = -expf(a.A_log[h]);
    const float dt_bias = a.dt_bias[h];
    sb::pdl_wait();
    const int t0 = a.seq_starts[r], t1 = a.seq_starts[r + 1];
    if (t0 >= t1) return;
    const T* qkv = (const T*)a.qkv;
    const T* proj = (const T*)a.proj;

    // ---- staging warps: tokens tc + sw, tc + sw + 4, ... of a chunk become unit q and k, beta, the decay
    // and the block's columns of v in buffer `buf`
    auto stage = [&](int tc, int buf) {
        const int sw = warp - WALKERS / 32;
#pragma unroll
        for (int m = 0; m < TPW; ++m) {
            const int tt = sw + (STAGERS / 32) * m, t = tc + tt;
            if (t >= t1) break;
            const T* xr = qkv + (size_t)t * a.qkv_stride;
            const T* pr = proj + (size_t)t * a.proj_stride;
            float kv[DC], qv[DC], kss = 0.f, qss = 0.f;
#pragma unroll
            for (int c = 0; c < DC; ++c) {
                const int d = c * 32 + lane;
                kv[c] = d < D ? to_float(xr[a.k_off + kh * D + d]) : 0.f;
                qv[c] = d < D ? to_float(xr[a.q_off + kh * D + d]) : 0.f;
                kss += kv[c] * kv[c];
                qss += qv[c] * qv[c];
            }
            const float v = (lane < COLS && c0 + lane < Dv) ? to_float(xr[a.v_off + h * Dv + c0 + lane]) : 0.f;
            const float bz = to_float(pr[a.b_off + h]), az = to_float(pr[a.a_off + h]);
            kss = warp_sum(kss);
            qss = warp_sum(qss);
            const float kinv = 1.0f / sqrtf(kss + 1e-6f), qinv = a.q_scale / sqrtf(qss + 1e-6f);
#pragma unroll
            for (int c = 0; c < DC; ++c) {
                const int d = c * 32 + lane;
                if (d < RG * DR) {
                    const int at = (d / DR) * ST + d % DR;
                    ks[buf][tt][at] = kv[c] * kinv;
                    qs[buf][tt][at] = qv[c] * qinv;
                }
            }
            if (lane < COLS) vs[buf][tt][lane] = v;
            if (lane == 0) {
                beta_s[buf][tt] = 1.0f / (1.0f + expf(-bz));
                decay_s[buf][tt] = expf(neg_rate * softplus(az + dt_bias));
            }
        }
    };

    const int rg = tid & (RG - 1), cj = (tid / RG) & (COLS - 1), j = c0 + cj;
    const bool col = walker && j < Dv;
    float* sp = a.state + ((size_t)a.seq_rows[r] * H + h) * D * Dv + j;
    float S[DR];
    if (walker) {
#pragma unroll
        for (int ii = 0; ii < DR; ++ii) {
            const int i = rg * DR + ii;
            S[ii] = (col && i < D) ? sp[(size_t)i * Dv] : 0.f;
        }
    } else {
        stage(t0, 0);
    }
    __syncthreads();
    int buf = 0;
    for (int tc = t0; tc < t1; tc += TB, buf ^= 1) {
        const int nt = min(TB, t1 - tc);
        if (!walker) {
            if (tc + TB < t1) stage(tc + TB, buf ^ 1);        // while the walkers are busy with this chunk
        } else {
            for (int tt = 0; tt < nt; ++tt) {
                const float4* k4 = reinterpret_cast<const float4*>(&ks[buf][tt][rg * ST]);
                const float4* q4 = reinterpret_cast<const float4*>(&qs[buf][tt][rg * ST]);
                const float decay = decay_s[buf][tt], beta = beta_s[buf][tt], v = vs[buf][tt][cj];
                float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;      // what the state already answers along k
                float4 kk[DR / 4];
#pragma unroll
                for (int x = 0; x < DR / 4; ++x) kk[x] = k4[x];
#pragma unroll
                for (int x = 0; x < DR / 4; ++x) {
                    const float4 k = kk[x];
                    r0 = fmaf(S[4 * x], k.x, r0); r1 = fmaf(S[4 * x + 1], k.y, r1);
                    r2 = fmaf(S[4 * x + 2], k.z, r2); r3 = fmaf(S[4 * x + 3], k.w, r3);
                }
                float rk = (r0 + r1) + (r2 + r3);
#pragma unroll
                for (int sh = 1; sh < RG; sh <<= 1) rk += __shfl_xor_sync(0xffffffffu, rk, sh);
                const float u = beta * (v - decay * rk);
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
                for (int x = 0; x < DR / 4; ++x) {
                    const float4 k = kk[x], q = q4[x];
                    S[4 * x] = fmaf(k.x, u, decay * S[4 * x]);         o0 = fmaf(S[4 * x], q.x, o0);
                    S[4 * x + 1] = fmaf(k.y, u, decay * S[4 * x + 1]); o1 = fmaf(S[4 * x + 1], q.y, o1);
                    S[4 * x + 2] = fmaf(k.z, u, decay * S[4 * x + 2]); o2 = fmaf(S[4 * x + 2], q.z, o2);
                    S[4 * x + 3] = fmaf(k.w, u, decay * S[4 * x + 3]); o3 = fmaf(S[4 * x + 3], q.w, o3);
                }
                float o = (o0 + o1) + (o2 + o3);
#pragma unroll
                for (int sh = 1; sh < RG; sh <<= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
                if (rg == 0) os[tt][cj] = o;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(WALKERS) : "memory");      // the walkers only
            for (int tt = warp; tt < nt; tt += WALKERS / 32)
                if (lane < COLS && c0 + lane < Dv) a.raw_o[(size_t)(tc + tt) * H * Dv + h * Dv + c0 + lane] = os[tt][lane];
        }
        __syncthreads();
    }
    if (walker) {
#pragma unroll
        for (int ii = 0; ii < DR; ++ii) {
            const int i = rg * DR + ii;
            if (col && i < D) sp[(size_t)i * Dv] = S[ii];
        }
    }
}

// y = o / sqrt(mean(o^2) + eps) * w * silu(gate), a warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128) delta_out_kernel(DeltaArgs a, int N) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= N * a.H) return;
    const int t = item / a.H, h = item - t * a.H, Dv = a.Dv;
    const float* o = a.raw_o + (size_t)t * a.H * Dv + h * Dv;
    const T* gate = (const T*)a.proj + (size_t)t * a.proj_stride + a.gate_off + h * Dv;
    float ss = 0.f;
    for (int j = lane; j < Dv; j += 32) ss += o[j] * o[j];
    ss = warp_sum(ss);
    const float rinv = 1.0f / sqrtf(ss / (float)Dv + a.eps);
    T* y = (T*)a.out + (size_t)t * a.H * Dv + h * Dv;
    for (int j = lane; j < Dv; j += 32) {
        const float g = to_float(gate[j]);
        y[j] = from_float<T>(o[j] * rinv * a.norm_w[j] * (g / (1.0f + expf(-g))));
    }
}

template <typename T>
int launch_delta(const DeltaArgs& a, int R, int N, cudaStream_t stream) {
    const dim3 grid(a.H, R, (a.Dv + COLS - 1) / COLS);
    if (a.D <= RG * 4) sb::launch(delta_rule_kernel<T, 4>, grid, dim3(THREADS), 0, stream, a);     // rows per thread
    else if (a.D <= RG * 8) sb::launch(delta_rule_kernel<T, 8>, grid, dim3(THREADS), 0, stream, a);
    else sb::launch(delta_rule_kernel<T, 16>, grid, dim3(THREADS), 0, stream, a);
    sb::launch(delta_out_kernel<T>, dim3((N * a.H + 3) / 4), dim3(128), 0, stream, a, N);
    SB_LAUNCH_CHECK();
}

}  // namespace

// Largest key and value head sizes the kernel takes.
extern "C" int sb_delta_rule_supports(int D, int Dv) { return D >= 1 && D <= 256 && Dv >= 1 && Dv <= 1024; }

extern "C" int sb_delta_rule(void* out, const void* qkv, long long qkv_stride, int q_off, int k_off, int v_off,
                             const void* proj, long long proj_stride, int gate_off, int b_off, int a_off,
                             const float* A_log, const float* dt_bias, const float* norm_w, float* state,
                             const int* seq_starts, const int* seq_rows, int R, int H, int G, int D, int Dv,
                             float eps, float q_scale, int dtype, float* raw_o, int N, cudaStream_t stream) {
    SB_REQUIRE(R >= 0 && H > 0 && G > 0 && H % G == 0, "delta_rule: %d value heads are no multiple of %d key heads", H, G);
    SB_REQUIRE(sb_delta_rule_supports(D, Dv), "delta_rule: heads of %d (keys, at most 256) and %d (values, at most 1024) dims", D, Dv);
    SB_REQUIRE(R <= 65535 && (Dv + COLS - 1) / COLS <= 65535, "delta_rule: %d requests exceed one launch", R);
    SB_REQUIRE(raw_o != nullptr && N >= 0, "delta_rule: scratch for %d tokens is missing", N);
    if (R == 0 || N == 0) return 0;
    DeltaArgs a;
    a.qkv = qkv; a.qkv_stride = qkv_stride; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.proj = proj; a.proj_stride = proj_stride; a.gate_off = gate_off; a.b_off = b_off; a.a_off = a_off;
    a.A_log = A_log; a.dt_bias = dt_bias; a.norm_w = norm_w; a.state = state; a.out = out;
    a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.H = H; a.G = G; a.D = D; a.Dv = Dv;
    a.eps = eps; a.q_scale = q_scale; a.raw_o = raw_o;
    if (dtype == SB_F32) return launch_delta<float>(a, R, N, stream);
    if (dtype == SB_BF16) return launch_delta<__nv_bfloat16>(a, R, N, stream);
    SB_REQUIRE(false, "delta_rule: unknown dtype %d", dtype);
}

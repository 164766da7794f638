// Retention: linear attention with one fixed decay per head, no softmax and no denominator.
//
// Per head, with S a [dk, dv] float32 state carried from token to token in the request's slot:
//   q_t, k_t  <- rotate(q_t), rotate(k_t) * k_scale         (angles float32(position) * inv_freq)
//   S_t = decay * S_{t-1} + k_t v_t^T
//   o_t = S_t^T q_t
//   out_t = o_t / sqrt(mean(o_t^2) + eps) * silu(g_t)
//
// One block per (request, head) walks the request's tokens of the step in order, the state in
// registers: thread (slice s, column j) owns rows s, s + P, ... of column j.  The same kernel
// serves a prompt's portion and a single decoded token, so a position's numbers do not depend on
// how the tokens were cut into steps.
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

struct RetArgs {
    const void* qkvg;          // [N, stride] in T: q | k | v | g
    long long stride;
    int q_off, k_off, v_off, g_off;
    float* state;              // [rows, H, dk, dv]
    const float* decay;        // [H]
    const float* inv_freq;     // [rot/2]
    int rot;
    void* out;                 // [N, H*dv] in T
    const int* seq_starts;
    const int* seq_rows;
    const int* seq_first_pos;
    int H, dk, dv, P;
    float eps, k_scale;
};

template <typename T, int RPT>
__global__ void __launch_bounds__(RPT > 32 ? 256 : 512) retention_kernel(RetArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv, P = a.P;
    float* qs = sm;                    // dk
    float* ks = qs + dk;               // dk
    float* red = ks + dk;              // P * dv
    __shared__ float scratch[33];
    const int r = blockIdx.y, h = blockIdx.x;
    const int tid = threadIdx.x;
    const int j = tid % dv, s = tid / dv;
    const bool active = s < P;         // the block is rounded up to whole warps
    const float decay = a.decay[h];
    const int half = a.rot / 2;
    sb::pdl_wait();
    const int n0 = a.seq_starts[r], n1 = a.seq_starts[r + 1];
    const int row = a.seq_rows[r], first = a.seq_first_pos[r];
    float* S = a.state + (((size_t)row * a.H + h) * dk) * dv;
    float st[RPT];
#pragma unroll
    for (int e = 0; e < RPT; ++e) {
        const int i = s + e * P;
        st[e] = (active && i < dk) ? S[(size_t)i * dv + j] : 0.f;
    }
    const T* in = (const T*)a.qkvg;
    for (int n = n0; n < n1; ++n) {
        const T* tok = in + (size_t)n * a.stride;
        const float pos = (float)(first + (n - n0));
        // rotated q and k of this token, one dim per thread
        for (int i = tid; i < dk; i += blockDim.x) {
            float qv = to_float(tok[a.q_off + h * dk + i]);
            float kv = to_float(tok[a.k_off + h * dk + i]);
            if (i < a.rot) {
                const int f = i < half ? i : i - half;
                const float ang = pos * a.inv_freq[f];
                const float c = cosf(ang), sn = sinf(ang);
                const int other = i < half ? i + half : i - half;
                const float qo = to_float(tok[a.q_off + h * dk + other]);
                const float ko = to_float(tok[a.k_off + h * dk + other]);
                // dim i < half: u cos - v sin; its partner: v cos + u sin
                qv = i < half ? qv * c - qo * sn : qv * c + qo * sn;
                kv = i < half ? kv * c - ko * sn : kv * c + ko * sn;
            }
            qs[i] = qv;
            ks[i] = kv * a.k_scale;
        }
        const float v = active ? to_float(tok[a.v_off + h * dv + j]) : 0.f;
        __syncthreads();
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < RPT; ++e) {
            const int i = s + e * P;
            if (i < dk) {
                st[e] = fmaf(decay, st[e], ks[i] * v);
                part = fmaf(st[e], qs[i], part);
            }
        }
        if (active) red[s * dv + j] = part;
        __syncthreads();
        float o = 0.f;
        if (s == 0)
            for (int p = 0; p < P; ++p) o += red[p * dv + j];
        const float total = block_sum(s == 0 ? o * o : 0.f, scratch);
        if (s == 0) {
            const float rinv = 1.0f / sqrtf(total / (float)dv + a.eps);
            const float g = to_float(tok[a.g_off + h * dv + j]);
            ((T*)a.out)[((size_t)n * a.H + h) * dv + j] = from_float<T>(o * rinv * (g / (1.0f + expf(-g))));
        }
    }
#pragma unroll
    for (int e = 0; e < RPT; ++e) {
        const int i = s + e * P;
        if (active && i < dk) S[(size_t)i * dv + j] = st[e];
    }
}

template <typename T>
int launch_retention(const RetArgs& a, int R, int threads, int rpt, size_t smem, cudaStream_t stream) {
    dim3 grid(a.H, R);
#define SB_RET(N_)                                                                              \
    if (rpt <= N_) {                                                                             \
        sb::launch(retention_kernel<T, N_>, grid, dim3(threads), smem, stream, a);              \
        return 0;                                                                                \
    }
    SB_RET(4) SB_RET(8) SB_RET(16) SB_RET(32) SB_RET(64) SB_RET(128)
#undef SB_RET
    return 1;
}

}  // namespace

extern "C" int sb_retention(const void* qkvg, long long stride, int q_off, int k_off, int v_off, int g_off,
                            float* state, const float* decay, const float* inv_freq, int rot, void* out,
                            const int* seq_starts, const int* seq_rows, const int* seq_first_pos, int R, int H,
                            int dk, int dv, float eps, float k_scale, int dtype, cudaStream_t stream) {
    SB_REQUIRE(R >= 0 && H > 0 && dk > 0 && dv > 0 && dv <= 512, "retention: bad sizes R=%d H=%d dk=%d dv=%d", R, H, dk, dv);
    SB_REQUIRE(rot >= 0 && rot <= dk && rot % 2 == 0, "retention: %d rotating dims of %d", rot, dk);
    SB_REQUIRE(R <= 65535, "retention: %d requests exceed one launch", R);
    if (R == 0) return 0;
    int P = 256 / dv;
    if (P < 1) P = 1;
    if (P > dk) P = dk;
    const int threads = (P * dv + 31) / 32 * 32;
    const int rpt = (dk + P - 1) / P;
    SB_REQUIRE(rpt <= 128 && threads <= (rpt > 32 ? 256 : 512),
               "retention: a head of %d x %d does not fit a block's registers", dk, dv);
    RetArgs a;
    a.qkvg = qkvg; a.stride = stride; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off;
    a.state = state; a.decay = decay; a.inv_freq = inv_freq; a.rot = rot; a.out = out;
    a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.seq_first_pos = seq_first_pos;
    a.H = H; a.dk = dk; a.dv = dv; a.P = P; a.eps = eps; a.k_scale = k_scale;
    const size_t smem = (size_t)(2 * dk + P * dv) * sizeof(float);
    int bad;
    if (dtype == SB_F32) bad = launch_retention<float>(a, R, threads, rpt, smem, stream);
    else if (dtype == SB_BF16) bad = launch_retention<__nv_bfloat16>(a, R, threads, rpt, smem, stream);
    else SB_REQUIRE(false, "retention: unknown dtype %d", dtype);
    SB_REQUIRE(!bad, "retention: no kernel for %d state rows per thread", rpt);
    SB_LAUNCH_CHECK();
}

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

// cos and sin of position * frequency.  With `lo` (the part of the frequency below float32) the angle is
// carried as a float32 product plus its exact rounding error and the low part's share, so that a position in
// the thousands costs no accuracy: cos(p + e) = cos p - e sin p, sin(p + e) = sin p + e cos p for a tiny e.
__device__ __forceinline__ void angle_cos_sin(float pos, float f, const float* lo, int i, float& c, float& s) {
    const float p = pos * f;
    c = cosf(p);
    s = sinf(p);
    if (lo != nullptr) {
        const float e = fmaf(pos, f, -p) + pos * lo[i];
        const float c0 = c;
        c = fmaf(-e, s, c);
        s = fmaf(e, c0, s);
    }
}

struct RetArgs {
    const void* qkvg;          // [N, stride] in T: q | k | v | g
    long long stride;
    int q_off, k_off, v_off, g_off;
    float* state;              // [rows, H, dk, dv]
    const float* decay;        // [H]
    const float* inv_freq;     // [rot/2]
    const float* inv_freq_lo;  // [rot/2] or null: what float32 rounding took from each frequency
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
                float c, sn;
                angle_cos_sin(pos, a.inv_freq[f], a.inv_freq_lo, f, c, sn);
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


// ----------------------------------------------------------------------------------------
// The same recurrence for prompt portions, a chunk of C tokens at a time.  With S0 the state
// before the chunk and t, s counting tokens inside it:
//   o_t = decay^(t+1) * S0^T q_t + sum_{s<=t} decay^(t-s) (q_t . k_s) v_s
//   S_C = decay^C * S0 + sum_s decay^(C-1-s) k_s v_s^T
// so the tokens of a chunk are independent of one another and a block of 256 threads works on
// all of them at once; chunks follow one another through the state, which stays in shared
// memory.  Scores, decays and sums are float32 on the CUDA cores.  One block per (request, head).
// Warp w owns the tokens t = w, w + 8, ... of a chunk (and the state rows i = w, w + 8, ... in the
// update); lane l owns the value columns j = l, l + 32, ...
struct RetChunkArgs {
    RetArgs r;
    int C;               // tokens per chunk: 16, 32 or 64
    int R;               // requests of the step
    float* scratch;      // [chunks of the step, H, dk, dv], for the three-launch form (see below)
};

// The chunks of a step in one list: request 0's, then request 1's, ...  Finds chunk g's request and its
// number within the request; false if the step has fewer chunks.
__device__ __forceinline__ bool find_chunk(int g, const int* seq_starts, int R, int C, int& r, int& ci) {
    for (r = 0; r < R; ++r) {
        const int nc = (seq_starts[r + 1] - seq_starts[r] + C - 1) / C;
        if (g < nc) { ci = g; return true; }
        g -= nc;
    }
    return false;
}

// rows x cols of T from global memory (row stride `src_stride` elements) to float32 shared memory (row
// stride `dst_stride`), by the 256 threads of a block; 16-byte loads where the rows allow them.
template <typename T>
__device__ __forceinline__ void copy_rows(float* dst, int dst_stride, const T* src, long long src_stride, int rows,
                                          int cols, int tid) {
    constexpr int VEC = Vec16<T>::N;
    if (cols % VEC == 0 && src_stride % VEC == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const int per_row = cols / VEC, total = rows * per_row;
#pragma unroll 4
        for (int idx = tid; idx < total; idx += 256) {
            const int t = idx / per_row, v = idx - t * per_row;
            Vec16<T> x;
            x.load(src + (size_t)t * src_stride + v * VEC);
#pragma unroll
            for (int e = 0; e < VEC; ++e) dst[t * dst_stride + v * VEC + e] = x.get(e);
        }
    } else {
#pragma unroll 4
        for (int idx = tid; idx < rows * cols; idx += 256) {
            const int t = idx / cols, i = idx - t * cols;
            dst[t * dst_stride + i] = to_float(src[(size_t)t * src_stride + i]);
        }
    }
}

constexpr int TB = 4;      // tokens (or state rows) a warp works on at once

// MODE 0: one block per (request, head) walks the request's chunks in order (enough blocks when many
// requests bring portions).  A single long prompt would leave most SMs idle that way, so it runs as three
// launches instead, every chunk a block of its own:
// MODE 1: each chunk's own contribution to the state, sum_s decay^(len-1-s) k_s v_s^T, to scratch;
// (retention_state_scan_kernel then walks the chunks of a request: the state BEFORE each chunk replaces the
//  chunk's contribution in scratch, and the request's slot gets the state after the last one;)
// MODE 2: each chunk's outputs from the state before it.
template <typename T, int JJ, int MODE>
__global__ void __launch_bounds__(256) retention_chunk_kernel(RetChunkArgs ca) {
    sb::pdl_launch_dependents();
    const RetArgs& a = ca.r;
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv, C = ca.C, kst = dk + 1;
    float* Ss = sm;                         // [dk][dv]   the state
    float* Qs = Ss + dk * dv;               // [C][dk]
    float* Ks = Qs + C * dk;                // [C][dk+1]
    float* Vs = Ks + C * kst;               // [C][dv]
    float* As = Vs + C * dv;                // [C][C]     decayed scores
    float* pw = As + C * C;                 // [C+1]      powers of the decay
    const int h = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float decay = a.decay[h];
    const int half = a.rot / 2;
    if (tid == 0) {
        float p = 1.f;
        for (int n = 0; n <= C; ++n) { pw[n] = p; p *= decay; }
    }
    sb::pdl_wait();
    int r = blockIdx.y, ci = 0;
    if (MODE != 0 && !find_chunk(blockIdx.y, a.seq_starts, ca.R, C, r, ci)) return;
    const int n0 = a.seq_starts[r], n1 = a.seq_starts[r + 1];
    const int row = a.seq_rows[r], first = a.seq_first_pos[r];
    // MODE 0: the request's slot.  Else this chunk's place in scratch: written in MODE 1, read in MODE 2.
    float* S = MODE == 0 ? a.state + (((size_t)row * a.H + h) * dk) * dv
                         : ca.scratch + (((size_t)blockIdx.y * a.H + h) * dk) * dv;
    for (int i = tid; i < dk * dv; i += 256) Ss[i] = MODE == 1 ? 0.f : S[i];
    const T* in = (const T*)a.qkvg;
    const int c_first = MODE == 0 ? n0 : n0 + ci * C, c_end = MODE == 0 ? n1 : min(n1, c_first + C);
    for (int c0 = c_first; c0 < c_end; c0 += C) {
        const int len = min(C, n1 - c0);
        __syncthreads();                    // the last chunk's readers are done with Q, K, V and A
        // ---- this chunk's q, k and v as they come from the projection (copies with many loads in
        // flight: nothing here depends on a loaded value), then q and k rotated in place and k scaled
        if (MODE != 1) copy_rows(Qs, dk, in + (size_t)c0 * a.stride + a.q_off + h * dk, a.stride, len, dk, tid);
        copy_rows(Ks, kst, in + (size_t)c0 * a.stride + a.k_off + h * dk, a.stride, len, dk, tid);
        copy_rows(Vs, dv, in + (size_t)c0 * a.stride + a.v_off + h * dv, a.stride, len, dv, tid);
        __syncthreads();
        for (int idx = tid; idx < len * dk; idx += 256) {
            const int t = idx / dk, i = idx - t * dk;
            if (i < half) {                 // this thread owns the pair (i, i + half) of token t
                float c, sn;
                angle_cos_sin((float)(first + (c0 - n0) + t), a.inv_freq[i], a.inv_freq_lo, i, c, sn);
                if (MODE != 1) {
                    const float qu = Qs[t * dk + i], qv = Qs[t * dk + i + half];
                    Qs[t * dk + i] = qu * c - qv * sn;
                    Qs[t * dk + i + half] = qv * c + qu * sn;
                }
                const float ku = Ks[t * kst + i], kv = Ks[t * kst + i + half];
                Ks[t * kst + i] = (ku * c - kv * sn) * a.k_scale;
                Ks[t * kst + i + half] = (kv * c + ku * sn) * a.k_scale;
            } else if (i >= a.rot) {
                Ks[t * kst + i] *= a.k_scale;
            }
        }
        __syncthreads();
        // ---- decayed scores A[t][s] = (q_t . k_s) decay^(t-s) for s <= t, zero above the diagonal
        for (int t = warp; t < (MODE == 1 ? 0 : len); t += 8) {
            for (int s0 = 0; s0 < C; s0 += 32) {
                const int s = s0 + lane;
                float dot = 0.f;
                if (s <= t) {
                    const float* qr = Qs + t * dk;
                    const float* kr = Ks + s * kst;
                    for (int i = 0; i < dk; ++i) dot = fmaf(qr[i], kr[i], dot);
                    dot *= pw[t - s];
                }
                if (s < C) As[t * C + s] = dot;
            }
        }
        __syncthreads();
        // ---- outputs, four tokens of the warp at a time (a value of the state or of v serves all four)
        for (int t0 = warp; t0 < (MODE == 1 ? 0 : len); t0 += 8 * TB) {
            float acc[TB][JJ], inter[TB][JJ];
#pragma unroll
            for (int k = 0; k < TB; ++k)
#pragma unroll
                for (int jj = 0; jj < JJ; ++jj) acc[k][jj] = inter[k][jj] = 0.f;
            int tk[TB];
#pragma unroll
            for (int k = 0; k < TB; ++k) tk[k] = min(t0 + 8 * k, len - 1);      // rows past the end repeat the last one and are not written
            for (int i = 0; i < dk; ++i) {
                float qi[TB];
#pragma unroll
                for (int k = 0; k < TB; ++k) qi[k] = Qs[tk[k] * dk + i];
#pragma unroll
                for (int jj = 0; jj < JJ; ++jj) {
                    const int j = lane + 32 * jj;
                    const float sv = j < dv ? Ss[i * dv + j] : 0.f;
#pragma unroll
                    for (int k = 0; k < TB; ++k) inter[k][jj] = fmaf(qi[k], sv, inter[k][jj]);
                }
            }
            const int last = tk[TB - 1];
            for (int s = 0; s <= last; ++s) {
                float w[TB];
#pragma unroll
                for (int k = 0; k < TB; ++k) w[k] = As[tk[k] * C + s];
#pragma unroll
                for (int jj = 0; jj < JJ; ++jj) {
                    const int j = lane + 32 * jj;
                    const float vv = j < dv ? Vs[s * dv + j] : 0.f;
#pragma unroll
                    for (int k = 0; k < TB; ++k) acc[k][jj] = fmaf(w[k], vv, acc[k][jj]);
                }
            }
#pragma unroll
            for (int k = 0; k < TB; ++k) {
                const int t = t0 + 8 * k;
                if (t >= len) break;
                float ss = 0.f;
#pragma unroll
                for (int jj = 0; jj < JJ; ++jj) {
                    acc[k][jj] = fmaf(pw[t + 1], inter[k][jj], acc[k][jj]);
                    if (lane + 32 * jj < dv) ss += acc[k][jj] * acc[k][jj];
                }
                ss = warp_sum(ss);
                const float rinv = 1.0f / sqrtf(ss / (float)dv + a.eps);
                const T* tok = in + (size_t)(c0 + t) * a.stride;
#pragma unroll
                for (int jj = 0; jj < JJ; ++jj) {
                    const int j = lane + 32 * jj;
                    if (j < dv) {
                        const float g = to_float(tok[a.g_off + h * dv + j]);
                        ((T*)a.out)[((size_t)(c0 + t) * a.H + h) * dv + j] =
                            from_float<T>(acc[k][jj] * rinv * (g / (1.0f + expf(-g))));
                    }
                }
            }
        }
        __syncthreads();                    // every reader of the old state is done
        // ---- the state moves on by the chunk, four rows of the warp at a time
        for (int i0 = warp; i0 < (MODE == 2 ? 0 : dk); i0 += 8 * TB) {
            float acc[TB][JJ];
#pragma unroll
            for (int k = 0; k < TB; ++k)
#pragma unroll
                for (int jj = 0; jj < JJ; ++jj) acc[k][jj] = 0.f;
            int ik[TB];
#pragma unroll
            for (int k = 0; k < TB; ++k) ik[k] = min(i0 + 8 * k, dk - 1);
            for (int s = 0; s < len; ++s) {
                const float p = pw[len - 1 - s];
                float w[TB];
#pragma unroll
                for (int k = 0; k < TB; ++k) w[k] = Ks[s * kst + ik[k]] * p;
#pragma unroll
                for (int jj = 0; jj < JJ; ++jj) {
                    const int j = lane + 32 * jj;
                    const float vv = j < dv ? Vs[s * dv + j] : 0.f;
#pragma unroll
                    for (int k = 0; k < TB; ++k) acc[k][jj] = fmaf(w[k], vv, acc[k][jj]);
                }
            }
#pragma unroll
            for (int k = 0; k < TB; ++k) {
                const int i = i0 + 8 * k;
                if (i >= dk) break;
#pragma unroll
                for (int jj = 0; jj < JJ; ++jj) {
                    const int j = lane + 32 * jj;
                    if (j < dv) Ss[i * dv + j] = fmaf(pw[len], Ss[i * dv + j], acc[k][jj]);
                }
            }
        }
    }
    __syncthreads();
    if (MODE != 2)
        for (int i = tid; i < dk * dv; i += 256) S[i] = Ss[i];
}

// Between MODE 1 and MODE 2: for every (request, head) the chunks in order; scratch holds each chunk's own
// contribution and receives the state before that chunk; the slot receives the state after the last.
__global__ void __launch_bounds__(256) retention_state_scan_kernel(RetChunkArgs ca) {
    sb::pdl_launch_dependents();
    const RetArgs& a = ca.r;
    const int h = blockIdx.x, r = blockIdx.y, C = ca.C;
    const float decay = a.decay[h];
    sb::pdl_wait();
    int base = 0;
    for (int q = 0; q < r; ++q) base += (a.seq_starts[q + 1] - a.seq_starts[q] + C - 1) / C;
    const int len_all = a.seq_starts[r + 1] - a.seq_starts[r];
    const int nc = (len_all + C - 1) / C;
    float pw_full = 1.f, pw_last = 1.f;
    for (int n = 0; n < C; ++n) pw_full *= decay;
    for (int n = 0; n < len_all - (nc - 1) * C; ++n) pw_last *= decay;
    const int size = a.dk * a.dv;
    float* S = a.state + ((size_t)a.seq_rows[r] * a.H + h) * size;
    // the elements of a state are independent: blockIdx.z takes every gridDim.z-th group of 256
    for (int i = blockIdx.z * 256 + threadIdx.x; i < size; i += 256 * gridDim.z) {
        float s = S[i];
        for (int c0 = 0; c0 < nc; c0 += 8) {                     // eight chunks' loads in flight
            float u[8];
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (c0 + k < nc) u[k] = ca.scratch[((size_t)(base + c0 + k) * a.H + h) * size + i];
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (c0 + k < nc) {
                    ca.scratch[((size_t)(base + c0 + k) * a.H + h) * size + i] = s;
                    s = fmaf(c0 + k == nc - 1 ? pw_last : pw_full, s, u[k]);
                }
        }
        S[i] = s;
    }
}

template <typename T, int JJ, int MODE>
void launch_chunk_mode(const RetChunkArgs& ca, dim3 grid, size_t smem, cudaStream_t stream) {
    static sb::OncePerDevice once;
    if (!once.flag()) {
        cudaFuncSetAttribute(retention_chunk_kernel<T, JJ, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        once.flag() = true;
    }
    sb::launch(retention_chunk_kernel<T, JJ, MODE>, grid, dim3(256), smem, stream, ca);
}

// chunks: an upper bound of the step's chunks (ceil(N / C) + R); scratch null: one launch, a block per request.
template <typename T, int JJ>
void launch_retention_chunked_jj(const RetChunkArgs& ca, int chunks, size_t smem, cudaStream_t stream) {
    if (ca.scratch == nullptr) {
        launch_chunk_mode<T, JJ, 0>(ca, dim3(ca.r.H, ca.R), smem, stream);
        return;
    }
    launch_chunk_mode<T, JJ, 1>(ca, dim3(ca.r.H, chunks), smem, stream);
    int slices = (ca.r.dk * ca.r.dv + 255) / 256;
    if (slices > 16) slices = 16;
    sb::launch(retention_state_scan_kernel, dim3(ca.r.H, ca.R, slices), dim3(256), 0, stream, ca);
    launch_chunk_mode<T, JJ, 2>(ca, dim3(ca.r.H, chunks), smem, stream);
}

template <typename T>
int launch_retention_chunked(const RetArgs& a, int R, int C, int chunks, float* scratch, size_t smem, cudaStream_t stream) {
    RetChunkArgs ca;
    ca.r = a;
    ca.C = C;
    ca.R = R;
    ca.scratch = scratch;
    if (a.dv <= 64) launch_retention_chunked_jj<T, 2>(ca, chunks, smem, stream);
    else if (a.dv <= 128) launch_retention_chunked_jj<T, 4>(ca, chunks, smem, stream);
    else if (a.dv <= 256) launch_retention_chunked_jj<T, 8>(ca, chunks, smem, stream);
    else return 1;
    return 0;
}

}  // namespace

extern "C" int sb_retention(const void* qkvg, long long stride, int q_off, int k_off, int v_off, int g_off,
                            float* state, const float* decay, const float* inv_freq, const float* inv_freq_lo, int rot,
                            void* out,
                            const int* seq_starts, const int* seq_rows, const int* seq_first_pos, int R, int H,
                            int dk, int dv, float eps, float k_scale, int chunked, int N, float* scratch,
                            long long scratch_floats, int dtype, cudaStream_t stream) {
    SB_REQUIRE(R >= 0 && H > 0 && dk > 0 && dv > 0 && dv <= 512, "retention: bad sizes R=%d H=%d dk=%d dv=%d", R, H, dk, dv);
    SB_REQUIRE(rot >= 0 && rot <= dk && rot % 2 == 0, "retention: %d rotating dims of %d", rot, dk);
    SB_REQUIRE(R <= 65535, "retention: %d requests exceed one launch", R);
    if (R == 0) return 0;
    if (chunked) {
        // prompt portions: chunks of as many tokens as fit a block's shared memory beside the state
        RetArgs a;
        a.qkvg = qkvg; a.stride = stride; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off;
        a.state = state; a.decay = decay; a.inv_freq = inv_freq; a.inv_freq_lo = inv_freq_lo; a.rot = rot; a.out = out;
        a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.seq_first_pos = seq_first_pos;
        a.H = H; a.dk = dk; a.dv = dv; a.P = 1; a.eps = eps; a.k_scale = k_scale;
        int C = 64;
        auto need = [&](int c) { return (size_t)(dk * dv + c * dk + c * (dk + 1) + c * dv + c * c + c + 1) * sizeof(float); };
        while (C > 16 && need(C) > 200 * 1024) C /= 2;
        if (need(C) <= 200 * 1024 && dv <= 256) {
            // one launch while the requests' heads alone fill the GPU, else a block per chunk in three launches
            const int chunks = (N + C - 1) / C + R;
            const bool spread = scratch != nullptr && R * H < 132 && chunks > 2 * R &&
                                (long long)chunks * H * dk * dv <= scratch_floats;
            int bad = 1;
            if (dtype == SB_F32) bad = launch_retention_chunked<float>(a, R, C, chunks, spread ? scratch : nullptr, need(C), stream);
            else if (dtype == SB_BF16)
                bad = launch_retention_chunked<__nv_bfloat16>(a, R, C, chunks, spread ? scratch : nullptr, need(C), stream);
            SB_REQUIRE(!bad, "retention: no chunked kernel for dv=%d or dtype %d", dv, dtype);
            SB_LAUNCH_CHECK();
        }
        // a head too large for shared memory falls through to the token-by-token kernel
    }
    int P = 256 / dv;
    if (P < 1) P = 1;
    if (P > dk) P = dk;
    const int threads = (P * dv + 31) / 32 * 32;
    const int rpt = (dk + P - 1) / P;
    SB_REQUIRE(rpt <= 128 && threads <= (rpt > 32 ? 256 : 512),
               "retention: a head of %d x %d does not fit a block's registers", dk, dv);
    RetArgs a;
    a.qkvg = qkvg; a.stride = stride; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off;
    a.state = state; a.decay = decay; a.inv_freq = inv_freq; a.inv_freq_lo = inv_freq_lo; a.rot = rot; a.out = out;
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

// Tokens per chunk of the chunked kernels for a head of dk x dv (0: the head does not fit shared memory).
extern "C" int sb_retention_chunk(int dk, int dv) {
    int C = 64;
    auto need = [&](int c) { return (size_t)(dk * dv + c * dk + c * (dk + 1) + c * dv + c * c + c + 1) * sizeof(float); };
    while (C > 16 && need(C) > 200 * 1024) C /= 2;
    return (need(C) <= 200 * 1024 && dv <= 256) ? C : 0;
}

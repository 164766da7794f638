// Short causal convolution over time, per channel, of a step's flat batch.
//
//   u_t = in_t + in_bias                          (the projected values, the projection's bias included)
//   y_t = act(sum_j taps[c][j] * u_{t-K+1+j} + conv_bias)      zeros before a sequence's start
//
// A request's tokens may arrive in portions: the last K-1 values of u of each sequence live in
// its state slot `tail` [rows, K-1, C] (float32) and stand in for the tokens before the portion.
// `short_conv` reads the tail as earlier steps left it; `short_conv_tail` then moves it on.
// The two are separate launches because every token of a portion may read the old tail.
//
// Channels are cut into up to three column ranges with a destination each: a dense matrix in the
// model dtype, or a paged pool [pages, heads, page_size, head_dim] written at the token's slot.
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

constexpr int MAX_TAPS = 16;

struct ConvSeg {
    int begin, end;        // channels [begin, end)
    int paged;             // 0: dense [N, stride]; 1: paged pool
    void* dst;
    long long stride;      // dense: elements per row
    int heads, head_dim;   // paged
};

struct ConvArgs {
    const void* in;        // [N, in_stride] in T, channel c at column c
    long long in_stride;
    const float* in_bias;  // [C] or null
    const float* taps;     // [C, K]
    const float* conv_bias;   // [C] or null
    int act;               // 0 none, 1 silu
    const float* tail;     // [rows, K-1, C]
    int C, K, N;
    const int* token_rows;
    const int* positions;
    const int* block_table;
    int table_width, page_size;
    ConvSeg seg[3];
    int nseg;
};

template <typename T>
__global__ void __launch_bounds__(256) short_conv_kernel(ConvArgs a) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int n = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int row = a.token_rows[n], pos = a.positions[n];
    const int K = a.K;
    // how many tokens directly before this one belong to the same request (at most K-1 matter)
    int same = 0;
    for (int b = 1; b < K; ++b) {
        if (n - b >= 0 && a.token_rows[n - b] == row) same = b;
        else break;
    }
    const T* in = (const T*)a.in;
    const float bias = a.in_bias ? a.in_bias[c] : 0.f;
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
        const int back = K - 1 - j;
        if (pos - back < 0) continue;                       // before the sequence's start
        float u;
        if (back <= same) u = to_float(in[(size_t)(n - back) * a.in_stride + c]) + bias;
        else u = a.tail[((size_t)row * (K - 1) + (K - 1 - back + same)) * a.C + c];
        acc = fmaf(a.taps[(size_t)c * K + j], u, acc);
    }
    if (a.conv_bias) acc += a.conv_bias[c];
    if (a.act == 1) acc = acc / (1.0f + expf(-acc));
    for (int s = 0; s < a.nseg; ++s) {
        const ConvSeg& g = a.seg[s];
        if (c < g.begin || c >= g.end) continue;
        const int e = c - g.begin;
        if (!g.paged) {
            ((T*)g.dst)[(size_t)n * g.stride + e] = from_float<T>(acc);
        } else {
            const int head = e / g.head_dim, x = e - head * g.head_dim;
            const int page = a.block_table[(size_t)row * a.table_width + pos / a.page_size];
            ((T*)g.dst)[(((size_t)page * g.heads + head) * a.page_size + pos % a.page_size) * g.head_dim + x] =
                from_float<T>(acc);
        }
    }
}

// One thread per (request, channel): the new tail is the last K-1 values of (old tail, this portion).
template <typename T>
__global__ void __launch_bounds__(256) short_conv_tail_kernel(float* __restrict__ tail, const T* __restrict__ in,
                                                              long long in_stride, const float* __restrict__ in_bias,
                                                              int C, int K, const int* __restrict__ seq_starts,
                                                              const int* __restrict__ seq_rows) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int n0 = seq_starts[r], n1 = seq_starts[r + 1], len = n1 - n0;
    const int row = seq_rows[r];
    const float bias = in_bias ? in_bias[c] : 0.f;
    float* t = tail + (size_t)row * (K - 1) * C + c;
    float v[MAX_TAPS];
#pragma unroll
    for (int i = 0; i < MAX_TAPS; ++i) {
        if (i >= K - 1) break;
        const int from_end = K - 1 - i;                     // this entry is the from_end-th value from the end
        if (from_end <= len) v[i] = to_float(in[(size_t)(n1 - from_end) * in_stride + c]) + bias;
        else v[i] = t[(size_t)(i + len) * C];
    }
#pragma unroll
    for (int i = 0; i < MAX_TAPS; ++i) {
        if (i >= K - 1) break;
        t[(size_t)i * C] = v[i];
    }
}

}  // namespace

// seg_*: arrays of `nseg` entries describing the destinations (see ConvSeg).
extern "C" int sb_short_conv(const void* in, long long in_stride, const float* in_bias, const float* taps,
                             const float* conv_bias, int act, const float* tail, int C, int K, int N,
                             const int* token_rows, const int* positions, const int* block_table,
                             int table_width, int page_size, int nseg, const int* seg_begin, const int* seg_end,
                             const int* seg_paged, void* const* seg_dst, const long long* seg_stride,
                             const int* seg_heads, const int* seg_head_dim, int dtype, cudaStream_t stream) {
    SB_REQUIRE(C > 0 && N >= 0 && K >= 1 && K <= MAX_TAPS, "short_conv: bad sizes C=%d N=%d taps=%d (at most %d)", C, N, K,
               MAX_TAPS);
    SB_REQUIRE(nseg >= 1 && nseg <= 3, "short_conv: %d destinations (1 to 3)", nseg);
    SB_REQUIRE(K == 1 || tail != nullptr, "short_conv: %d taps need a tail state", K);
    SB_REQUIRE(N <= 65535, "short_conv: %d tokens exceed one launch", N);
    if (N == 0) return 0;
    ConvArgs a;
    a.in = in; a.in_stride = in_stride; a.in_bias = in_bias; a.taps = taps; a.conv_bias = conv_bias; a.act = act;
    a.tail = tail; a.C = C; a.K = K; a.N = N; a.token_rows = token_rows; a.positions = positions;
    a.block_table = block_table; a.table_width = table_width; a.page_size = page_size; a.nseg = nseg;
    for (int s = 0; s < nseg; ++s) {
        a.seg[s].begin = seg_begin[s]; a.seg[s].end = seg_end[s]; a.seg[s].paged = seg_paged[s];
        a.seg[s].dst = seg_dst[s]; a.seg[s].stride = seg_stride[s]; a.seg[s].heads = seg_heads[s];
        a.seg[s].head_dim = seg_head_dim[s];
        SB_REQUIRE(!a.seg[s].paged || (block_table != nullptr && page_size > 0 && a.seg[s].head_dim > 0),
                   "short_conv: a paged destination needs a block table");
    }
    dim3 grid((C + 255) / 256, N);
    if (dtype == SB_F32) sb::launch(short_conv_kernel<float>, grid, dim3(256), 0, stream, a);
    else if (dtype == SB_BF16) sb::launch(short_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, a);
    else SB_REQUIRE(false, "short_conv: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

extern "C" int sb_short_conv_tail(float* tail, const void* in, long long in_stride, const float* in_bias, int C,
                                  int K, const int* seq_starts, const int* seq_rows, int R, int dtype,
                                  cudaStream_t stream) {
    SB_REQUIRE(C > 0 && R >= 0 && K >= 1 && K <= MAX_TAPS, "short_conv_tail: bad sizes C=%d R=%d taps=%d", C, R, K);
    if (R == 0 || K == 1) return 0;
    dim3 grid((C + 255) / 256, R);
    if (dtype == SB_F32)
        sb::launch(short_conv_tail_kernel<float>, grid, dim3(256), 0, stream, tail, (const float*)in, in_stride, in_bias,
                   C, K, seq_starts, seq_rows);
    else if (dtype == SB_BF16)
        sb::launch(short_conv_tail_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, tail, (const __nv_bfloat16*)in,
                   in_stride, in_bias, C, K, seq_starts, seq_rows);
    else
        SB_REQUIRE(false, "short_conv_tail: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

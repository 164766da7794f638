// Norm kernels of blocks that norm a branch BEFORE it joins the residual stream, and the
// small elementwise steps beside them.  All arithmetic is float32.
//
//   fold_rmsnorm:   b = sum_s delta[s][r] + branch_bias            (the branch's output)
//                   b = b / sqrt(mean(b^2) + branch_eps) * branch_gain      (if branch_gain)
//                   v = residual[r] + b + add_rows[r] + add_vec
//                   residual[r] = v ;  out[m] = v / sqrt(mean(v^2) + eps) * gain    (if out)
//                   (out with a null gain: out[m] = v, the stream itself in the model dtype, for
//                   blocks whose branches read the stream without a norm in front)
//   normed_mean:    out[r] = scale * sum_t unit_rms(sum_s x_t[s][r]) * gain_t       (t < 2)
//   bias_act:       out[r][f] = act(sum_s in[s][r][f] + bias[f])
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

struct FoldArgs {
    float* residual;
    const float* delta;        // [S, rows, d] or null
    int S;
    size_t delta_stride;
    const float* branch_bias;  // [d] or null
    const float* branch_gain;  // [d] or null: the branch joins as it is
    float branch_eps;
    const float* add_rows;     // [rows, d] or null
    const float* add_vec;      // [d] or null
    const float* gain;         // [d]; used with out; null: out is the unnormed row
    void* out;                 // [M, d] in T, or null
    const int* row_index;      // [M] or null
    int d;
    float eps;
    int write_residual;
};

template <typename T>
__global__ void __launch_bounds__(256) fold_rmsnorm_kernel(FoldArgs a) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    extern __shared__ float row[];          // d floats
    __shared__ float scratch[33];
    const int m = blockIdx.x, d = a.d;
    const int r = a.row_index ? a.row_index[m] : m;
    const bool branch = a.S > 0 || a.branch_bias != nullptr;
    float binv = 1.f;
    if (branch) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float b = 0.f;
            for (int s0 = 0; s0 < a.S; s0 += 16) {              // sixteen loads in flight, added in order
                float p[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (s0 + j < a.S) p[j] = __ldg(a.delta + (size_t)(s0 + j) * a.delta_stride + (size_t)r * d + i);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (s0 + j < a.S) b += p[j];
            }
            if (a.branch_bias) b += a.branch_bias[i];
            row[i] = b;
            ss += b * b;
        }
        if (a.branch_gain) {
            const float total = block_sum(ss, scratch);
            binv = 1.0f / sqrtf(total / (float)d + a.branch_eps);
        }
    }
    float* res = a.residual + (size_t)r * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = res[i];
        if (branch) v += a.branch_gain ? row[i] * binv * a.branch_gain[i] : row[i];
        if (a.add_rows) v += a.add_rows[(size_t)r * d + i];
        if (a.add_vec) v += a.add_vec[i];
        row[i] = v;
        if (a.write_residual) res[i] = v;
        ss += v * v;
    }
    if (a.out == nullptr) return;
    T* o = (T*)a.out + (size_t)m * d;
    if (a.gain == nullptr) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<T>(row[i]);
        return;
    }
    const float total = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(total / (float)d + a.eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<T>(row[i] * rinv * a.gain[i]);
}

// The same with 16-byte accesses (d a multiple of 4, aligned rows) and every partial sum of a column
// in flight at once: with few rows (a decode step) the kernel is one or two round trips to L2 per
// phase instead of one per partial sum and column.
template <typename T>
__global__ void __launch_bounds__(512) fold_rmsnorm_vec_kernel(FoldArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ float row[];          // d floats
    __shared__ float scratch[33];
    const int m = blockIdx.x, d4 = a.d / 4;
    sb::pdl_wait();
    const int r = a.row_index ? a.row_index[m] : m;
    const bool branch = a.S > 0 || a.branch_bias != nullptr;
    float4* row4 = reinterpret_cast<float4*>(row);
    const size_t stride4 = a.delta_stride / 4;
    float binv = 1.f;
    if (branch) {
        float ss = 0.f;
        const float4* del4 = reinterpret_cast<const float4*>(a.delta) + (size_t)r * d4;
        for (int i = threadIdx.x; i < d4; i += blockDim.x) {
            float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s0 = 0; s0 < a.S; s0 += 16) {
                float4 p[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (s0 + j < a.S) p[j] = __ldg(del4 + (size_t)(s0 + j) * stride4 + i);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (s0 + j < a.S) { b.x += p[j].x; b.y += p[j].y; b.z += p[j].z; b.w += p[j].w; }
            }
            if (a.branch_bias) {
                const float4 c = __ldg(reinterpret_cast<const float4*>(a.branch_bias) + i);
                b.x += c.x; b.y += c.y; b.z += c.z; b.w += c.w;
            }
            row4[i] = b;
            ss += b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
        }
        if (a.branch_gain) {
            const float total = block_sum(ss, scratch);
            binv = 1.0f / sqrtf(total / (float)a.d + a.branch_eps);
        }
    }
    float4* res4 = reinterpret_cast<float4*>(a.residual + (size_t)r * a.d);
    float ss = 0.f;
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        float4 v = res4[i];
        if (branch) {
            float4 b = row4[i];
            if (a.branch_gain) {
                const float4 g = __ldg(reinterpret_cast<const float4*>(a.branch_gain) + i);
                b.x *= binv * g.x; b.y *= binv * g.y; b.z *= binv * g.z; b.w *= binv * g.w;
            }
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        }
        if (a.add_rows) {
            const float4 c = reinterpret_cast<const float4*>(a.add_rows + (size_t)r * a.d)[i];
            v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
        }
        if (a.add_vec) {
            const float4 c = __ldg(reinterpret_cast<const float4*>(a.add_vec) + i);
            v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
        }
        row4[i] = v;
        if (a.write_residual) res4[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (a.out == nullptr) return;
    const bool normed = a.gain != nullptr;
    const float rinv = normed ? 1.0f / sqrtf(block_sum(ss, scratch) / (float)a.d + a.eps) : 1.0f;
    T* o = (T*)a.out + (size_t)m * a.d;
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        const float4 v = row4[i];
        const float4 g = normed ? __ldg(reinterpret_cast<const float4*>(a.gain) + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float x0 = v.x * rinv * g.x, x1 = v.y * rinv * g.y, x2 = v.z * rinv * g.z, x3 = v.w * rinv * g.w;
        if constexpr (sizeof(T) == 2) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(x0, x1), hi = __floats2bfloat162_rn(x2, x3);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(o + 4 * i) = pk;
        } else {
            *reinterpret_cast<float4*>(o + 4 * i) = make_float4(x0, x1, x2, x3);
        }
    }
}

struct MeanArgs {
    const float* x[2];
    int S[2];
    size_t stride[2];
    const float* gain[2];
    float* out;
    int d;
    float eps, scale;
};

__global__ void __launch_bounds__(256) normed_mean_kernel(MeanArgs a) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    extern __shared__ float rows[];         // 2 * d floats
    __shared__ float scratch[33];
    const int r = blockIdx.x, d = a.d;
    float inv[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float b = 0.f;
            for (int s0 = 0; s0 < a.S[t]; s0 += 16) {          // sixteen loads in flight, added in order
                float p[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (s0 + j < a.S[t]) p[j] = __ldg(a.x[t] + (size_t)(s0 + j) * a.stride[t] + (size_t)r * d + i);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (s0 + j < a.S[t]) b += p[j];
            }
            rows[t * d + i] = b;
            ss += b * b;
        }
        const float total = block_sum(ss, scratch);
        inv[t] = 1.0f / sqrtf(total / (float)d + a.eps);
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        a.out[(size_t)r * d + i] =
            a.scale * (rows[i] * inv[0] * a.gain[0][i] + rows[d + i] * inv[1] * a.gain[1][i]);
}

__device__ __forceinline__ float activation(float z, int act) {
    switch (act) {
        case 1: { const float p = fmaxf(z, 0.f); return p * p; }                       // relu squared
        case 2: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));   // gelu (tanh form)
        case 3: return z / (1.0f + expf(-z));                                          // silu
        default: return z;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) bias_act_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                       const float* __restrict__ parts, int S, size_t part_stride,
                                                       const float* __restrict__ bias, int F, size_t total, int act) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float z = 0.f;
        if (parts) {
            for (int s = 0; s < S; ++s) z += parts[s * part_stride + i];
        } else {
            z = to_float(in[i]);
        }
        if (bias) z += bias[i % F];
        out[i] = from_float<T>(activation(z, act));
    }
}

}  // namespace

// out_dtype: element type of `out` (float32 also in the bfloat16 engine, for a normed row that
// becomes a residual itself).
extern "C" int sb_fold_rmsnorm(float* residual, const float* delta, int S, long long delta_stride,
                               const float* branch_bias, const float* branch_gain, float branch_eps,
                               const float* add_rows, const float* add_vec, const float* gain, void* out,
                               const int* row_index, int M, int d, float eps, int out_dtype,
                               cudaStream_t stream) {
    SB_REQUIRE(M >= 0 && d > 0 && S >= 0, "fold_rmsnorm: bad sizes M=%d d=%d S=%d", M, d, S);
    SB_REQUIRE(S == 0 || delta != nullptr, "fold_rmsnorm: S=%d partial sums but no buffer", S);
    if (M == 0) return 0;
    const size_t smem = (size_t)d * sizeof(float);
    SB_REQUIRE(smem <= 200 * 1024, "fold_rmsnorm: width %d does not fit one block's shared memory", d);
    FoldArgs a;
    a.residual = residual; a.delta = delta; a.S = S; a.delta_stride = (size_t)delta_stride;
    a.branch_bias = branch_bias; a.branch_gain = branch_gain; a.branch_eps = branch_eps;
    a.add_rows = add_rows; a.add_vec = add_vec; a.gain = gain; a.out = out; a.row_index = row_index;
    a.d = d; a.eps = eps;
    a.write_residual = row_index == nullptr &&
                       (S > 0 || branch_bias != nullptr || add_rows != nullptr || add_vec != nullptr);
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = d % 4 == 0 && delta_stride % 4 == 0 && aligned(residual) && aligned(delta) && aligned(branch_bias) &&
                     aligned(branch_gain) && aligned(add_rows) && aligned(add_vec) && aligned(gain) && aligned(out);
    if (vec) {
        int threads = ((d / 4 + 31) / 32) * 32;
        if (threads > 512) threads = 512;
        if (M > 512 && threads > 256) threads = 256;
        if (out_dtype == SB_F32) {
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(fold_rmsnorm_vec_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            sb::launch(fold_rmsnorm_vec_kernel<float>, dim3(M), dim3(threads), smem, stream, a);
        } else if (out_dtype == SB_BF16) {
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(fold_rmsnorm_vec_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            sb::launch(fold_rmsnorm_vec_kernel<__nv_bfloat16>, dim3(M), dim3(threads), smem, stream, a);
        } else {
            SB_REQUIRE(false, "fold_rmsnorm: unknown dtype %d", out_dtype);
        }
        SB_LAUNCH_CHECK();
    }
    if (out_dtype == SB_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(fold_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        sb::launch(fold_rmsnorm_kernel<float>, dim3(M), dim3(256), smem, stream, a);
    } else if (out_dtype == SB_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(fold_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        sb::launch(fold_rmsnorm_kernel<__nv_bfloat16>, dim3(M), dim3(256), smem, stream, a);
    } else {
        SB_REQUIRE(false, "fold_rmsnorm: unknown dtype %d", out_dtype);
    }
    SB_LAUNCH_CHECK();
}

extern "C" int sb_normed_mean(float* out, const float* x0, int S0, long long stride0, const float* gain0,
                              const float* x1, int S1, long long stride1, const float* gain1, int N, int d,
                              float eps, float scale, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && d > 0 && S0 > 0 && S1 > 0, "normed_mean: bad sizes N=%d d=%d S=%d,%d", N, d, S0, S1);
    if (N == 0) return 0;
    const size_t smem = 2 * (size_t)d * sizeof(float);
    SB_REQUIRE(smem <= 200 * 1024, "normed_mean: width %d does not fit one block's shared memory", d);
    MeanArgs a;
    a.x[0] = x0; a.S[0] = S0; a.stride[0] = (size_t)stride0; a.gain[0] = gain0;
    a.x[1] = x1; a.S[1] = S1; a.stride[1] = (size_t)stride1; a.gain[1] = gain1;
    a.out = out; a.d = d; a.eps = eps; a.scale = scale;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(normed_mean_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch(normed_mean_kernel, dim3(N), dim3(256), smem, stream, a);
    SB_LAUNCH_CHECK();
}

// in: [N, F] in the model dtype, or (parts != null) float32 partial sums [S, N, F].
extern "C" int sb_bias_act(void* out, const void* in, const float* parts, int S, long long part_stride,
                           const float* bias, int N, int F, int act, int dtype, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && F > 0 && act >= 0 && act <= 3, "bias_act: bad sizes N=%d F=%d or activation %d", N, F, act);
    SB_REQUIRE((in != nullptr) != (parts != nullptr), "bias_act: one input, a matrix or partial sums");
    if (N == 0) return 0;
    const size_t total = (size_t)N * F;
    const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
    if (dtype == SB_F32)
        sb::launch(bias_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, (const float*)in, parts, S,
                   (size_t)part_stride, bias, F, total, act);
    else if (dtype == SB_BF16)
        sb::launch(bias_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)in, parts, S, (size_t)part_stride, bias, F, total, act);
    else
        SB_REQUIRE(false, "bias_act: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

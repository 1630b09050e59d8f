// Row kernels of designs that norm after the sum, gate a mixer's output element by element, or average two
// normed branches.  Statistics and products are float; a row is one block's, and the order of its sums depends
// on the row's width alone (never on how many rows a step has).
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

static inline int row_threads(int width) { return width <= 256 ? 64 : (width <= 2048 ? 128 : 256); }

// res <- norm(alpha * res + branch); y (optional) the same rows in another type
template <typename TB, typename TY>
__global__ void postnorm_kernel(float* __restrict__ res, const TB* __restrict__ branch, float alpha, const void* __restrict__ w,
                                int w_dtype, float eps, float off, TY* __restrict__ y, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    float* r = res + (long long)blockIdx.x * width;
    const TB* b = branch + (long long)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float h = fmaf(alpha, r[i], to_float(b[i]));
        r[i] = h;                     // this thread reads it back below
        ss = fmaf(h, h, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = r[i] * inv * (rdl_load(w, i, w_dtype) + off);
        r[i] = v;
        if (y) y[(long long)blockIdx.x * width + i] = from_float<TY>(v);
    }
}

extern "C" int rdl_postnorm(float* res, const void* branch, int branch_dtype, float alpha, const void* w, int w_dtype, float eps,
                            float off, void* y, int y_dtype, int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(branch_dtype) && rdl_valid_dtype(w_dtype) && rdl_valid_dtype(y_dtype), "postnorm: bad dtype");
    RDL_REQUIRE(res && branch && w && n_rows >= 0 && width > 0, "postnorm: missing rows or weight");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(n_rows), block(row_threads(width));
    cudaError_t e;
    if (branch_dtype == RDL_BF16) {
        if (y_dtype == RDL_BF16)
            e = rdl_launch(postnorm_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, st, res, (const __nv_bfloat16*)branch, alpha, w,
                           w_dtype, eps, off, (__nv_bfloat16*)y, width);
        else
            e = rdl_launch(postnorm_kernel<__nv_bfloat16, float>, grid, block, 0, st, res, (const __nv_bfloat16*)branch, alpha, w, w_dtype,
                           eps, off, (float*)y, width);
    } else {
        if (y_dtype == RDL_BF16)
            e = rdl_launch(postnorm_kernel<float, __nv_bfloat16>, grid, block, 0, st, res, (const float*)branch, alpha, w, w_dtype, eps,
                           off, (__nv_bfloat16*)y, width);
        else
            e = rdl_launch(postnorm_kernel<float, float>, grid, block, 0, st, res, (const float*)branch, alpha, w, w_dtype, eps, off,
                           (float*)y, width);
    }
    RDL_CHECK_EX(e, "postnorm");
    return 0;
}

// out = c (norm(a; wa) + norm(b; wb))
template <typename T>
__global__ void norm_pair_kernel(float* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, const void* __restrict__ wa,
                                 const void* __restrict__ wb, int w_dtype, float eps, float c, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const T* ra = a + (long long)blockIdx.x * width;
    const T* rb = b + (long long)blockIdx.x * width;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = to_float(ra[i]), z = to_float(rb[i]);
        sa = fmaf(x, x, sa);
        sb = fmaf(z, z, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = 1.0f / sqrtf(sa / (float)width + eps), ib = 1.0f / sqrtf(sb / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = to_float(ra[i]) * ia * rdl_load(wa, i, w_dtype);
        const float z = to_float(rb[i]) * ib * rdl_load(wb, i, w_dtype);
        out[(long long)blockIdx.x * width + i] = c * (x + z);
    }
}

extern "C" int rdl_norm_pair(float* out, const void* a, const void* b, int dtype, const void* wa, const void* wb, int w_dtype,
                             float eps, float c, int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype) && rdl_valid_dtype(w_dtype), "norm_pair: bad dtype");
    RDL_REQUIRE(out && a && b && wa && wb && n_rows >= 0 && width > 0, "norm_pair: missing rows or weights");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == RDL_BF16)
        e = rdl_launch(norm_pair_kernel<__nv_bfloat16>, dim3(n_rows), dim3(row_threads(width)), 0, st, out, (const __nv_bfloat16*)a,
                       (const __nv_bfloat16*)b, wa, wb, w_dtype, eps, c, width);
    else
        e = rdl_launch(norm_pair_kernel<float>, dim3(n_rows), dim3(row_threads(width)), 0, st, out, (const float*)a, (const float*)b, wa,
                       wb, w_dtype, eps, c, width);
    RDL_CHECK_EX(e, "norm_pair");
    return 0;
}

__device__ __forceinline__ float gate_value(float g, int act) {
    const float s = 1.0f / (1.0f + expf(-g));
    return act == RDL_GATE_SILU ? g * s : s;
}

template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ x, long long x_stride,
                                const T* __restrict__ g, long long g_stride, int act, int n_rows, int width) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const long long total = (long long)n_rows * width;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / width;
        const int i = (int)(idx - t * width);
        out[t * out_stride + i] = from_float<T>(to_float(x[t * x_stride + i]) * gate_value(to_float(g[t * g_stride + i]), act));
    }
}

extern "C" int rdl_gate_mul(void* out, long long out_stride, const void* x, long long x_stride, const void* g, long long g_stride,
                            int dtype, int gate_act, int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "gate_mul: bad dtype %d", dtype);
    RDL_REQUIRE(gate_act == RDL_GATE_SIGMOID || gate_act == RDL_GATE_SILU, "gate_mul: unknown gate %d", gate_act);
    RDL_REQUIRE(out && x && g && n_rows >= 0 && width > 0 && out_stride >= width && x_stride >= width && g_stride >= width,
                "gate_mul: missing rows or strides below the width");
    if (n_rows == 0) return 0;
    const long long total = (long long)n_rows * width;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == RDL_BF16)
        e = rdl_launch(gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st, (__nv_bfloat16*)out, out_stride,
                       (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)g, g_stride, gate_act, n_rows, width);
    else
        e = rdl_launch(gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, st, (float*)out, out_stride, (const float*)x, x_stride,
                       (const float*)g, g_stride, gate_act, n_rows, width);
    RDL_CHECK_EX(e, "gate_mul");
    return 0;
}

// float rows normed group by group, times an optional weight and an optional gate
template <typename TO>
__global__ void group_norm_gate_kernel(TO* __restrict__ out, const float* __restrict__ x, int groups, int group, const void* __restrict__ w,
                                       int w_dtype, float eps, const void* __restrict__ g, long long g_stride, int g_dtype, int act) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x, gi = blockIdx.y;
    const long long base = ((long long)t * groups + gi) * group;
    const int col0 = gi * group;
    float ss = 0.f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const float v = x[base + i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)group + eps);
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        float v = x[base + i] * inv;
        if (w) v *= rdl_load(w, col0 + i, w_dtype);
        if (g) v *= gate_value(rdl_load(g, (long long)t * g_stride + col0 + i, g_dtype), act);
        out[base + i] = from_float<TO>(v);
    }
}

extern "C" int rdl_group_norm_gate(void* out, int out_dtype, const float* x, int n_rows, int groups, int group, const void* w,
                                   int w_dtype, float eps, const void* g, long long g_stride, int g_dtype, int gate_act, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(out_dtype) && rdl_valid_dtype(w_dtype) && rdl_valid_dtype(g_dtype), "group_norm_gate: bad dtype");
    RDL_REQUIRE(out && x && n_rows >= 0 && groups > 0 && groups <= 65535 && group > 0, "group_norm_gate: bad sizes");
    RDL_REQUIRE(gate_act == RDL_GATE_SIGMOID || gate_act == RDL_GATE_SILU, "group_norm_gate: unknown gate %d", gate_act);
    RDL_REQUIRE(!g || g_stride >= (long long)groups * group, "group_norm_gate: the gate's rows are narrower than the groups");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(n_rows, groups), block(group <= 64 ? 32 : row_threads(group));
    cudaError_t e;
    if (out_dtype == RDL_BF16)
        e = rdl_launch(group_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, st, (__nv_bfloat16*)out, x, groups, group, w, w_dtype, eps, g,
                       g_stride, g_dtype, gate_act);
    else
        e = rdl_launch(group_norm_gate_kernel<float>, grid, block, 0, st, (float*)out, x, groups, group, w, w_dtype, eps, g, g_stride,
                       g_dtype, gate_act);
    RDL_CHECK_EX(e, "group_norm_gate");
    return 0;
}

// Routed feed-forward (mixture of experts): the router, and the experts for few rows.
//
// Router, per row x (float arithmetic throughout):
//   z = W_r x,  s = softmax(z) over all experts (identity experts included),
//   choice = s + correction;  the `top` largest choices are taken (ties: the lower index),
//   their weights are s itself (not renormalised).
// An expert e < n_real is a gated feed-forward, y = W_down act(W_gate x, W_up x); an expert e >= n_real is
// an identity expert whose output is x.  The row's result is sum_k weight_k y_k in the order of the choice.
//
// Few rows (single-token steps, the 32-bit path): every (row, choice) pair streams its expert's
// matrices, a warp per output value (rdl_moe_gate_up, rdl_moe_down_combine); the sums run lane by lane
// over k in an order that depends on k alone.  Many rows are sorted by expert and go through the tiled
// product with one expert per row tile (rdl_moe_align, rdl_moe_gather, rdl_gemm_tc_grouped, rdl_moe_combine).
#include "activations.cuh"
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int ROUTE_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_kernel(const T* __restrict__ x, const float* __restrict__ w_router,
                                                                  const float* __restrict__ correction, int n_experts, int width, int top,
                                                                  int* __restrict__ sel, float* __restrict__ sel_w) {
    extern __shared__ float zs[];              // [n_experts] logits, then scores; [n_experts] choice
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* row = x + (long long)t * width;
    for (int e = warp; e < n_experts; e += ROUTE_THREADS / 32) {
        const float* w = w_router + (long long)e * width;
        float acc = 0.f;
        for (int k = lane; k < width; k += 32) acc = fmaf(w[k], to_float(row[k]), acc);
        acc = warp_sum(acc);
        if (lane == 0) zs[e] = acc;
    }
    __syncthreads();
    if (warp != 0) return;
    float* choice = zs + n_experts;
    float m = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) m = fmaxf(m, zs[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) {
        const float p = expf(zs[e] - m);
        zs[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < n_experts; e += 32) {
        const float s = zs[e] / sum;
        zs[e] = s;
        choice[e] = s + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; best_e = e; }       // lanes see their experts in rising order: the lower index wins a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = 0;              // only if every remaining choice is NaN or -inf
        if (lane == 0) {
            sel[(long long)t * top + k] = best_e;
            sel_w[(long long)t * top + k] = zs[best_e];
            choice[best_e] = -INFINITY;
        }
        __syncwarp();
    }
}

constexpr int PAIR_WARPS = 8;

// mid[p, j] = act(W_gate[e] x, W_up[e] x)[j] for pair p = (row t, choice k) with expert e = sel[p] < n_real.
// w: [n_real][2 ff][width], an expert's gate rows followed by its up rows.  A warp per (pair, j).
template <typename T>
__global__ void __launch_bounds__(PAIR_WARPS * 32) moe_gate_up_kernel(T* __restrict__ mid, const T* __restrict__ x, const T* __restrict__ w,
                                                                      const int* __restrict__ sel, int top, int n_real, int ff, int width,
                                                                      int activation, float act_param) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int p = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = sel[p];
    if (e < 0 || e >= n_real) return;
    const int j = blockIdx.x * PAIR_WARPS + warp;
    if (j >= ff) return;
    const T* row = x + (long long)(p / top) * width;
    const T* wg = w + ((long long)e * 2 * ff + j) * width;
    const T* wu = wg + (long long)ff * width;
    float g = 0.f, u = 0.f;
    for (int k = lane; k < width; k += 32) {
        const float xv = to_float(row[k]);
        g = fmaf(to_float(wg[k]), xv, g);
        u = fmaf(to_float(wu[k]), xv, u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) mid[(long long)p * ff + j] = from_float<T>(rdl_gated(g, u, activation, act_param));
}

// out[t, n] = sum_k sel_w[t, k] * (expert k real ? W_down[e_k][n, :] . mid[(t, k), :] : x[t, n]), k in rising order.
template <typename T>
__global__ void __launch_bounds__(PAIR_WARPS * 32) moe_down_combine_kernel(T* __restrict__ out, const T* __restrict__ mid, const T* __restrict__ x,
                                                                           const T* __restrict__ w_down, const int* __restrict__ sel,
                                                                           const float* __restrict__ sel_w, int top, int n_real, int ff,
                                                                           int width) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * PAIR_WARPS + warp;
    if (n >= width) return;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const int p = t * top + k;
        const int e = sel[p];
        const float wk = sel_w[p];
        float y;
        if (e >= n_real) {
            y = to_float(x[(long long)t * width + n]);
        } else {
            const T* w = w_down + ((long long)e * width + n) * ff;
            const T* m = mid + (long long)p * ff;
            float acc = 0.f;
            for (int i = lane; i < ff; i += 32) acc = fmaf(to_float(w[i]), to_float(m[i]), acc);
            y = warp_sum(acc);
        }
        total = fmaf(wk, y, total);
    }
    if (lane == 0) out[(long long)t * width + n] = from_float<T>(total);
}

}  // namespace

extern "C" int rdl_moe_route(const void* x, int dtype, const float* w_router, const float* correction, int n_rows, int n_experts,
                             int width, int top, int* sel, float* sel_w, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "moe_route: bad dtype %d", dtype);
    RDL_REQUIRE(x && w_router && sel && sel_w && n_experts > 0 && width > 0, "moe_route: bad arguments");
    RDL_REQUIRE(top >= 1 && top <= n_experts, "moe_route: %d of %d experts cannot be chosen", top, n_experts);
    RDL_REQUIRE(n_experts <= 4096, "moe_route: %d experts exceed the 4,096 the router kernel holds", n_experts);
    if (n_rows == 0) return 0;
    const size_t smem = 2 * (size_t)n_experts * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(moe_route_kernel<__nv_bfloat16>, dim3(n_rows), dim3(ROUTE_THREADS), smem, st, (const __nv_bfloat16*)x, w_router,
                                correction, n_experts, width, top, sel, sel_w), "moe_route");
    else
        RDL_CHECK_EX(rdl_launch(moe_route_kernel<float>, dim3(n_rows), dim3(ROUTE_THREADS), smem, st, (const float*)x, w_router, correction,
                                n_experts, width, top, sel, sel_w), "moe_route");
    return 0;
}

extern "C" int rdl_moe_gate_up(void* mid, int dtype, const void* x, const void* w_gate_up, const int* sel, int n_rows, int top, int n_real,
                               int ff, int width, int activation, float act_param, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "moe_gate_up: bad dtype %d", dtype);
    RDL_REQUIRE(mid && x && sel && (w_gate_up || n_real == 0) && top > 0 && ff > 0 && width > 0, "moe_gate_up: bad arguments");
    RDL_REQUIRE(rdl_gated_known(activation), "moe_gate_up: unknown activation %d", activation);
    if (n_rows == 0 || n_real == 0) return 0;
    RDL_REQUIRE((long long)n_rows * top <= 65535, "moe_gate_up: %d rows x %d choices exceed the grid limit", n_rows, top);
    const dim3 grid((ff + PAIR_WARPS - 1) / PAIR_WARPS, n_rows * top);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(moe_gate_up_kernel<__nv_bfloat16>, grid, dim3(PAIR_WARPS * 32), 0, st, (__nv_bfloat16*)mid, (const __nv_bfloat16*)x,
                                (const __nv_bfloat16*)w_gate_up, sel, top, n_real, ff, width, activation, act_param), "moe_gate_up");
    else
        RDL_CHECK_EX(rdl_launch(moe_gate_up_kernel<float>, grid, dim3(PAIR_WARPS * 32), 0, st, (float*)mid, (const float*)x, (const float*)w_gate_up,
                                sel, top, n_real, ff, width, activation, act_param), "moe_gate_up");
    return 0;
}

extern "C" int rdl_moe_down_combine(void* out, int dtype, const void* mid, const void* x, const void* w_down, const int* sel,
                                    const float* sel_w, int n_rows, int top, int n_real, int ff, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "moe_down_combine: bad dtype %d", dtype);
    RDL_REQUIRE(out && x && sel && sel_w && ((mid && w_down) || n_real == 0) && top > 0 && width > 0, "moe_down_combine: bad arguments");
    if (n_rows == 0) return 0;
    RDL_REQUIRE(n_rows <= 65535, "moe_down_combine: %d rows exceed the grid limit", n_rows);
    const dim3 grid((width + PAIR_WARPS - 1) / PAIR_WARPS, n_rows);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(moe_down_combine_kernel<__nv_bfloat16>, grid, dim3(PAIR_WARPS * 32), 0, st, (__nv_bfloat16*)out,
                                (const __nv_bfloat16*)mid, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_down, sel, sel_w, top, n_real, ff, width),
                     "moe_down_combine");
    else
        RDL_CHECK_EX(rdl_launch(moe_down_combine_kernel<float>, grid, dim3(PAIR_WARPS * 32), 0, st, (float*)out, (const float*)mid, (const float*)x,
                                (const float*)w_down, sel, sel_w, top, n_real, ff, width), "moe_down_combine");
    return 0;
}

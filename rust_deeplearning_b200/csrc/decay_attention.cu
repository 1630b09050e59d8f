// Linear attention with a fixed decay per head: per sequence and head a state S [dim][vdim] in float,
//   S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,
// kept per slot between steps.  Before they enter the recurrence q and k may be rotated (half-split pairs, float
// tables), q, k and v may go through SiLU and k is multiplied by a constant - all in float, from the rows as the
// input projection left them.
//
// decay_scan_kernel walks a sequence token by token.  A block owns 32 columns of one head's state (a column j of S
// decides o[j] alone, so the columns of a head can be shared out between blocks): thread (j, r) holds S[i][j] for the
// RPT rows i of slice r in registers.  Per token every thread updates its rows and forms its part of o[j]; the parts
// are added by the column's first thread in the order of the slices.  Nothing depends on how many tokens a step
// brings or on what else is in the batch, so a sequence's results are the same bits however it is cut into steps.
// It serves the 32-bit path, single-token steps (a step reads and writes the state once: the memory's rate), and is
// the reference of the chunked kernel.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

#define DA_COLS 32          // columns of the state a block owns
#define DA_MAX_PREFETCH 2   // raw values of q and of k a thread brings for the next token

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename T, int RPT>
__global__ void __launch_bounds__(256) decay_scan_kernel(DecayAttentionArgs a) {
    extern __shared__ float sm[];
    const int dim = a.dim, vdim = a.vdim;
    float* q_raw = sm;                       // [2][dim]
    float* k_raw = q_raw + 2 * dim;          // [2][dim]
    float* v_in = k_raw + 2 * dim;           // [2][DA_COLS]
    float* q_s = v_in + 2 * DA_COLS;         // [dim]
    float* k_s = q_s + dim;                  // [dim]
    float* part = k_s + dim;                 // [slices][DA_COLS]
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DA_COLS;
    const int row0 = a.seq_start[seq], n = a.seq_start[seq + 1] - row0;
    if (n <= 0) return;
    if (a.tok_pos[row0] < 0) return;         // a padding sequence of a fixed-size batch
    const int tid = threadIdx.x, j = tid & 31, r = tid >> 5, n_thr = blockDim.x;
    const int col = c0 + j;
    const bool col_ok = col < vdim;
    const int i0 = r * RPT;
    const float decay = a.decay[h];
    float* S = a.state + (((long long)a.slots[seq] * a.n_heads + h) * dim) * vdim;
    float s_reg[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) s_reg[i] = (col_ok && i0 + i < dim) ? S[(long long)(i0 + i) * vdim + col] : 0.f;

    const T* rows = (const T*)a.rows;
    const int half = a.rot_n >> 1;
    float pq[DA_MAX_PREFETCH], pk[DA_MAX_PREFETCH], pv = 0.f;
    auto fetch = [&](int t) {
        const T* row = rows + (long long)(row0 + t) * a.row_stride;
#pragma unroll
        for (int u = 0; u < DA_MAX_PREFETCH; ++u) {
            const int i = tid + u * n_thr;
            pq[u] = i < dim ? to_float(row[a.q_col + h * dim + i]) : 0.f;
            pk[u] = i < dim ? to_float(row[a.k_col + h * dim + i]) : 0.f;
        }
        pv = (r == 0 && col_ok) ? to_float(row[a.v_col + h * vdim + col]) : 0.f;
    };
    auto stage = [&](int b) {
#pragma unroll
        for (int u = 0; u < DA_MAX_PREFETCH; ++u) {
            const int i = tid + u * n_thr;
            if (i < dim) { q_raw[b * dim + i] = pq[u]; k_raw[b * dim + i] = pk[u]; }
        }
        if (r == 0) v_in[b * DA_COLS + j] = a.silu ? silu_f(pv) : pv;
    };
    fetch(0);
    stage(0);
    __syncthreads();
    for (int t = 0; t < n; ++t) {
        const int b = t & 1;
        if (t + 1 < n) fetch(t + 1);
        // q and k of this token as they enter the recurrence
        const int pos = a.tok_pos[row0 + t];
        for (int i = tid; i < dim; i += n_thr) {
            float qv, kv;
            if (i < 2 * half) {
                const int f = i < half ? i : i - half;
                const float cs = a.cos_t[(long long)pos * half + f], sn = a.sin_t[(long long)pos * half + f];
                const float q1 = q_raw[b * dim + f], q2 = q_raw[b * dim + f + half];
                const float k1 = k_raw[b * dim + f], k2 = k_raw[b * dim + f + half];
                qv = i < half ? q1 * cs - q2 * sn : q2 * cs + q1 * sn;
                kv = i < half ? k1 * cs - k2 * sn : k2 * cs + k1 * sn;
            } else {
                qv = q_raw[b * dim + i];
                kv = k_raw[b * dim + i];
            }
            if (a.silu) { qv = silu_f(qv); kv = silu_f(kv); }
            q_s[i] = qv;
            k_s[i] = kv * a.k_scale;
        }
        __syncthreads();
        const float v = v_in[b * DA_COLS + j];
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            if (i0 + i < dim) {
                s_reg[i] = fmaf(decay, s_reg[i], k_s[i0 + i] * v);
                acc = fmaf(s_reg[i], q_s[i0 + i], acc);
            }
        }
        part[r * DA_COLS + j] = acc;
        if (t + 1 < n) stage(b ^ 1);
        __syncthreads();
        if (r == 0 && col_ok) {
            float o = 0.f;
            const int slices = (dim + RPT - 1) / RPT;
            for (int s = 0; s < slices; ++s) o += part[s * DA_COLS + j];
            a.out[(long long)(row0 + t) * a.n_heads * vdim + (long long)h * vdim + col] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i)
        if (col_ok && i0 + i < dim) S[(long long)(i0 + i) * vdim + col] = s_reg[i];
}

static int check_decay_args(const DecayAttentionArgs* a, const char* who) {
    RDL_REQUIRE(rdl_valid_dtype(a->dtype), "%s: bad dtype %d", who, a->dtype);
    RDL_REQUIRE(a->n_tokens >= 0 && a->n_seqs >= 0 && a->n_heads > 0 && a->dim > 0 && a->vdim > 0, "%s: bad sizes", who);
    RDL_REQUIRE(a->rows && a->decay && a->tok_pos && a->seq_start && a->slots && a->state && a->out, "%s: missing rows, decay, batch description, state or output", who);
    RDL_REQUIRE(a->rot_n >= 0 && a->rot_n % 2 == 0 && a->rot_n <= a->dim && (a->rot_n == 0 || (a->cos_t && a->sin_t)),
                "%s: the rotated dimensions (%d) must be even, at most dim (%d) and come with tables", who, a->rot_n, a->dim);
    RDL_REQUIRE(a->n_heads <= 65535 && (a->vdim + DA_COLS - 1) / DA_COLS <= 65535, "%s: too many heads or columns for one grid", who);
    return 0;
}

template <typename T>
static int launch_scan(const DecayAttentionArgs* a, cudaStream_t st) {
    const int dim = a->dim;
    // rows a thread keeps: the fewest that let eight slices cover dim
    int rpt = 4;
    while (rpt < 64 && (dim + rpt - 1) / rpt > 8) rpt *= 2;
    const int slices = (dim + rpt - 1) / rpt;
    RDL_REQUIRE(slices <= 8, "decay_attention_scan: dim %d exceeds 512", dim);
    const int threads = 32 * slices;
    RDL_REQUIRE(dim <= DA_MAX_PREFETCH * threads, "decay_attention_scan: dim %d is too large for %d threads", dim, threads);
    const size_t smem = (size_t)(6 * dim + 2 * DA_COLS + slices * DA_COLS) * sizeof(float);
    const dim3 grid(a->n_seqs, a->n_heads, (a->vdim + DA_COLS - 1) / DA_COLS), block(threads);
    cudaError_t e;
    switch (rpt) {
        case 4: e = rdl_launch(decay_scan_kernel<T, 4>, grid, block, smem, st, *a); break;
        case 8: e = rdl_launch(decay_scan_kernel<T, 8>, grid, block, smem, st, *a); break;
        case 16: e = rdl_launch(decay_scan_kernel<T, 16>, grid, block, smem, st, *a); break;
        case 32: e = rdl_launch(decay_scan_kernel<T, 32>, grid, block, smem, st, *a); break;
        default: e = rdl_launch(decay_scan_kernel<T, 64>, grid, block, smem, st, *a); break;
    }
    RDL_CHECK_EX(e, "decay_attention_scan");
    return 0;
}

extern "C" int rdl_decay_attention_scan(const DecayAttentionArgs* a, void* stream) {
    if (int e = check_decay_args(a, "decay_attention_scan")) return e;
    if (a->n_tokens == 0 || a->n_seqs == 0) return 0;
    return a->dtype == RDL_BF16 ? launch_scan<__nv_bfloat16>(a, (cudaStream_t)stream) : launch_scan<float>(a, (cudaStream_t)stream);
}

extern "C" int rdl_decay_attention_chunked(const DecayAttentionArgs* a, void* stream) {
    (void)stream;
    if (int e = check_decay_args(a, "decay_attention_chunked")) return e;
    RDL_REQUIRE(false, "decay_attention_chunked: not available");
    return 0;
}

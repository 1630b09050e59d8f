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

// ---- the chunked form, for many tokens in bfloat16 ----
//
// With chunks of C = 64 tokens, S the state before a chunk's first token, L the chunk's tokens and i, j places inside it:
//   o_i   = sum_{j <= i} d^(i-j) (q_i . k_j) v_j  +  d^(i+1) S^T q_i
//   S'    = d^L S + U,   U = sum_j d^(L-1-j) k_j v_j^T.
// U needs nothing of the chunks before, and o needs of them only S, so the work is parallel over chunks in three launches:
//   1. decay_chunk_kernel<false>: a block per (chunk, head, 64 state columns) forms U = K^T V_d on tensor cores, with k and
//      v as they enter the recurrence (rotation, SiLU and k's constant in float, rounded to bfloat16 once) and
//      V_d[j] = v_j d^(L-1-j), into a float work buffer [chunk][head][dim][vdim];
//   2. decay_chunk_scan_kernel: a thread per state element walks its sequence's chunks, S' = d^L S + U in float, leaving
//      in the work buffer the state BEFORE each chunk and in the cache the state after the last;
//   3. decay_chunk_kernel<true>: a block per (chunk, head, 64 columns): P = (Q K^T) * d^(i-j) (16 rows a warp; the powers of
//      d applied to the float sums), O = P V, and O += d^(i+1) (Q S) with the float S as two bfloat16 terms (its rounding
//      and the remainder's), so that the state's 24 bits are not cut to 8 on the way.  Eight warps: two share a group of
//      16 rows and take 32 columns each, so that a block keeps twice the loads in flight while it fills shared memory.
// The powers d^n are exp2(n log2 d) in float (d^0 = 1 also for d = 0).  Chunks are numbered over the step's sequences in
// order; a block finds its sequence by walking the sequences' chunk counts.
#define DC_CHUNK 64
#define DC_COLS 64
#define DC_THREADS 256
#define DC_PAD 8            // bfloat16 values between rows in shared memory: ldmatrix reads eight rows without bank conflicts

__device__ __forceinline__ uint32_t dc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dc_ldm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void dc_ldm4t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void dc_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dc_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void dc_load8(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h2[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}
__device__ __forceinline__ void dc_load8(const float* p, float (&f)[8]) {
    const float4 lo = __ldg(reinterpret_cast<const float4*>(p)), hi = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w; f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
}
__device__ __forceinline__ void dc_store8(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 raw;
    raw.x = dc_pack(f[0], f[1]); raw.y = dc_pack(f[2], f[3]); raw.z = dc_pack(f[4], f[5]); raw.w = dc_pack(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// chunk number `idx` of the step -> its sequence and its first token there; false beyond the step's last chunk
__device__ __forceinline__ bool dc_find_chunk(const DecayAttentionArgs& a, int idx, int& seq, int& t0) {
    for (int s = 0; s < a.n_seqs; ++s) {
        const int n = a.seq_start[s + 1] - a.seq_start[s];
        const int nc = (n > 0 && a.tok_pos[a.seq_start[s]] >= 0) ? (n + DC_CHUNK - 1) / DC_CHUNK : 0;
        if (idx < nc) { seq = s; t0 = idx * DC_CHUNK; return true; }
        idx -= nc;
    }
    return false;
}

template <bool OUTPUT>
__global__ void __launch_bounds__(DC_THREADS) decay_chunk_kernel(DecayAttentionArgs a, float* __restrict__ work, int vec) {
    extern __shared__ __align__(16) unsigned char dc_raw[];
    const int dim = a.dim, vdim = a.vdim;
    const int h = blockIdx.y, c0 = blockIdx.z * DC_COLS;
    const int nv = min(DC_COLS, vdim - c0);              // columns of this block (a multiple of 16)
    const int qs = dim + DC_PAD, vs = DC_COLS + DC_PAD;   // row strides in shared memory, in values
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(dc_raw);     // [64][qs]
    __nv_bfloat16* Vs = Ks + DC_CHUNK * qs;                             // [64][vs]  v (OUTPUT) or v times d^(L-1-j)
    __nv_bfloat16* Qs = Vs + DC_CHUNK * vs;                             // [64][qs]   OUTPUT only, like the two below
    __nv_bfloat16* Sh = Qs + DC_CHUNK * qs;                             // [dim][vs] the state, rounded
    __nv_bfloat16* Sl = Sh + dim * vs;                                  // [dim][vs] what the rounding left
    __shared__ float pw[DC_CHUNK + 1];                                  // d^n
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    int seq, t0;
    if (!dc_find_chunk(a, blockIdx.x, seq, t0)) return;
    const int row0 = a.seq_start[seq], n = a.seq_start[seq + 1] - row0;
    const int L = min(DC_CHUNK, n - t0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const float decay = a.decay[h];
    const float lg = decay > 0.f ? log2f(decay) : 0.f;
    for (int d = tid; d <= DC_CHUNK; d += DC_THREADS) pw[d] = d == 0 ? 1.f : (decay > 0.f ? exp2f((float)d * lg) : 0.f);
    const int ksteps = dim >> 4, n_mt = dim >> 4, nt_count = nv >> 3;
    float* W = work + (((long long)blockIdx.x * a.n_heads + h) * dim) * vdim + c0;     // this chunk's U, then the state before it
    const __nv_bfloat16* rows = (const __nv_bfloat16*)a.rows;
    const int half = a.rot_n >> 1;
    __syncthreads();        // pw

    // ---- q, k, v as they enter the recurrence: rotated pairs first, then the values that only pass ----
    if (vec) {
        // 16 bytes a load, and a thread's loads of several items asked for before any is used
        const int hg = half >> 3;
#pragma unroll 2
        for (int idx = tid; idx < DC_CHUNK * hg; idx += DC_THREADS) {
            const int j = idx / hg, f = (idx - j * hg) << 3;
            float k_lo[8], k_hi[8], q_lo[8], q_hi[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) k_lo[e] = k_hi[e] = q_lo[e] = q_hi[e] = 0.f;
            if (j < L) {
                const __nv_bfloat16* row = rows + (long long)(row0 + t0 + j) * a.row_stride;
                const int pos = a.tok_pos[row0 + t0 + j];
                float cs[8], sn[8], x1[8], x2[8];
                dc_load8(a.cos_t + (long long)pos * half + f, cs);
                dc_load8(a.sin_t + (long long)pos * half + f, sn);
                dc_load8(row + a.k_col + h * dim + f, x1);
                dc_load8(row + a.k_col + h * dim + f + half, x2);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    k_lo[e] = x1[e] * cs[e] - x2[e] * sn[e];
                    k_hi[e] = x2[e] * cs[e] + x1[e] * sn[e];
                    if (a.silu) { k_lo[e] = silu_f(k_lo[e]); k_hi[e] = silu_f(k_hi[e]); }
                    k_lo[e] *= a.k_scale; k_hi[e] *= a.k_scale;
                }
                if (OUTPUT) {
                    dc_load8(row + a.q_col + h * dim + f, x1);
                    dc_load8(row + a.q_col + h * dim + f + half, x2);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        q_lo[e] = x1[e] * cs[e] - x2[e] * sn[e];
                        q_hi[e] = x2[e] * cs[e] + x1[e] * sn[e];
                        if (a.silu) { q_lo[e] = silu_f(q_lo[e]); q_hi[e] = silu_f(q_hi[e]); }
                    }
                }
            }
            dc_store8(Ks + j * qs + f, k_lo);
            dc_store8(Ks + j * qs + f + half, k_hi);
            if (OUTPUT) { dc_store8(Qs + j * qs + f, q_lo); dc_store8(Qs + j * qs + f + half, q_hi); }
        }
        const int rg = (dim - 2 * half) >> 3;     // groups of eight values that do not rotate
#pragma unroll 2
        for (int idx = tid; idx < DC_CHUNK * rg; idx += DC_THREADS) {
            const int j = idx / rg, i = 2 * half + ((idx - j * rg) << 3);
            float kv[8], qv[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) kv[e] = qv[e] = 0.f;
            if (j < L) {
                const __nv_bfloat16* row = rows + (long long)(row0 + t0 + j) * a.row_stride;
                dc_load8(row + a.k_col + h * dim + i, kv);
                if (OUTPUT) dc_load8(row + a.q_col + h * dim + i, qv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    if (a.silu) { kv[e] = silu_f(kv[e]); qv[e] = silu_f(qv[e]); }
                    kv[e] *= a.k_scale;
                }
            }
            dc_store8(Ks + j * qs + i, kv);
            if (OUTPUT) dc_store8(Qs + j * qs + i, qv);
        }
        const int vg = nv >> 3;
#pragma unroll 2
        for (int idx = tid; idx < DC_CHUNK * vg; idx += DC_THREADS) {
            const int j = idx / vg, c = (idx - j * vg) << 3;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
            if (j < L) {
                dc_load8(rows + (long long)(row0 + t0 + j) * a.row_stride + a.v_col + h * vdim + c0 + c, v);
                const float wj = OUTPUT ? 1.f : pw[L - 1 - j];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = (a.silu ? silu_f(v[e]) : v[e]) * wj;
            }
            dc_store8(Vs + j * vs + c, v);
        }
    } else {
    for (int idx = tid; idx < DC_CHUNK * half; idx += DC_THREADS) {
        const int j = idx / half, f = idx - j * half;
        float q_lo = 0.f, q_hi = 0.f, k_lo = 0.f, k_hi = 0.f;
        if (j < L) {
            const __nv_bfloat16* row = rows + (long long)(row0 + t0 + j) * a.row_stride;
            const int pos = a.tok_pos[row0 + t0 + j];
            const float cs = a.cos_t[(long long)pos * half + f], sn = a.sin_t[(long long)pos * half + f];
            const __nv_bfloat16* kr = row + a.k_col + h * dim;
            const float k1 = __bfloat162float(kr[f]), k2 = __bfloat162float(kr[f + half]);
            k_lo = k1 * cs - k2 * sn; k_hi = k2 * cs + k1 * sn;
            if (a.silu) { k_lo = silu_f(k_lo); k_hi = silu_f(k_hi); }
            k_lo *= a.k_scale; k_hi *= a.k_scale;
            if (OUTPUT) {
                const __nv_bfloat16* qr = row + a.q_col + h * dim;
                const float q1 = __bfloat162float(qr[f]), q2 = __bfloat162float(qr[f + half]);
                q_lo = q1 * cs - q2 * sn; q_hi = q2 * cs + q1 * sn;
                if (a.silu) { q_lo = silu_f(q_lo); q_hi = silu_f(q_hi); }
            }
        }
        Ks[j * qs + f] = __float2bfloat16_rn(k_lo);
        Ks[j * qs + f + half] = __float2bfloat16_rn(k_hi);
        if (OUTPUT) { Qs[j * qs + f] = __float2bfloat16_rn(q_lo); Qs[j * qs + f + half] = __float2bfloat16_rn(q_hi); }
    }
    {
        const int rest = dim - 2 * half;     // values of a head that do not rotate
        for (int idx = tid; idx < DC_CHUNK * rest; idx += DC_THREADS) {
            const int j = idx / rest, i = 2 * half + idx - j * rest;
            float qv = 0.f, kv = 0.f;
            if (j < L) {
                const __nv_bfloat16* row = rows + (long long)(row0 + t0 + j) * a.row_stride;
                kv = __bfloat162float(row[a.k_col + h * dim + i]);
                if (a.silu) kv = silu_f(kv);
                kv *= a.k_scale;
                if (OUTPUT) {
                    qv = __bfloat162float(row[a.q_col + h * dim + i]);
                    if (a.silu) qv = silu_f(qv);
                }
            }
            Ks[j * qs + i] = __float2bfloat16_rn(kv);
            if (OUTPUT) Qs[j * qs + i] = __float2bfloat16_rn(qv);
        }
    }
    for (int idx = tid; idx < DC_CHUNK * (nv >> 1); idx += DC_THREADS) {
        const int j = idx / (nv >> 1), c = 2 * (idx - j * (nv >> 1));
        float v0 = 0.f, v1 = 0.f;
        if (j < L) {
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(
                rows + (long long)(row0 + t0 + j) * a.row_stride + a.v_col + h * vdim + c0 + c));
            v0 = a.silu ? silu_f(v.x) : v.x;
            v1 = a.silu ? silu_f(v.y) : v.y;
            if (!OUTPUT) { v0 *= pw[L - 1 - j]; v1 *= pw[L - 1 - j]; }
        }
        *reinterpret_cast<__nv_bfloat162*>(Vs + j * vs + c) = __floats2bfloat162_rn(v0, v1);
    }
    }
    if (OUTPUT) {
        // the state before this chunk as two bfloat16 terms
#pragma unroll 4
        for (int idx = tid; idx < dim * (nv >> 2); idx += DC_THREADS) {       // vdim and the block's first column are multiples of 16
            const int r = idx / (nv >> 2), c = 4 * (idx - r * (nv >> 2));
            const float4 sv = __ldcg(reinterpret_cast<const float4*>(W + (long long)r * vdim + c));
            const __nv_bfloat162 h0 = __floats2bfloat162_rn(sv.x, sv.y), h1 = __floats2bfloat162_rn(sv.z, sv.w);
            const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
            uint2 hi, lo;
            hi.x = *reinterpret_cast<const uint32_t*>(&h0); hi.y = *reinterpret_cast<const uint32_t*>(&h1);
            lo.x = dc_pack(sv.x - f0.x, sv.y - f0.y); lo.y = dc_pack(sv.z - f1.x, sv.w - f1.y);
            *reinterpret_cast<uint2*>(Sh + r * vs + c) = hi;
            *reinterpret_cast<uint2*>(Sl + r * vs + c) = lo;
        }
    }
    __syncthreads();

    if (!OUTPUT) {
        // ---- U = K^T V_d: rows 16 warp .. + 15 of the state are this warp's ----
        if (warp < n_mt) {
            const int m0 = warp * 16;
            float u[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) u[nt][0] = u[nt][1] = u[nt][2] = u[nt][3] = 0.f;
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                uint32_t ka[4];
                dc_ldm4t(ka, dc_smem(Ks + (kb * 16 + ((lane >> 4) << 3) + (lane & 7)) * qs + m0 + (((lane >> 3) & 1) << 3)));
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    if (2 * nb >= nt_count) continue;
                    uint32_t bf[4];
                    dc_ldm4t(bf, dc_smem(Vs + (kb * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * vs + nb * 16 + ((lane >> 4) << 3)));
                    dc_mma(u[2 * nb], ka, bf[0], bf[1]);
                    dc_mma(u[2 * nb + 1], ka, bf[2], bf[3]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                if (nt >= nt_count) continue;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    *reinterpret_cast<float2*>(W + (long long)(m0 + g + 8 * hh) * vdim + nt * 8 + 2 * tq) = make_float2(u[nt][2 * hh], u[nt][2 * hh + 1]);
            }
        }
        return;
    }

    // ---- P = (Q K^T) d^(i-j), rows 16 warp .. + 15 ----
    // warps rw and rw + 4 share the rows 16 rw .. + 15 (each forms P for itself) and take 32 of the block's 64 columns each
    const int rw = warp & 3, cw = warp >> 2;
    const int i_hi = rw * 16 + g + 8;       // this thread's rows of the chunk: i_hi - 8 and i_hi
    uint32_t qf[8][4];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
        if (kk < ksteps) dc_ldm4(qf[kk], dc_smem(Qs + (rw * 16 + (lane & 15)) * qs + kk * 16 + 8 * (lane >> 4)));
    float p[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) p[nt][0] = p[nt][1] = p[nt][2] = p[nt][3] = 0.f;
#pragma unroll
    for (int np = 0; np < 4; ++np) {
        if (np > rw) continue;            // keys after this warp's last row
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            if (kk >= ksteps) continue;
            uint32_t bf[4];
            dc_ldm4(bf, dc_smem(Ks + (np * 16 + ((lane >> 4) << 3) + (lane & 7)) * qs + kk * 16 + (((lane >> 3) & 1) << 3)));
            dc_mma(p[2 * np], qf[kk], bf[0], bf[1]);
            dc_mma(p[2 * np + 1], qf[kk], bf[2], bf[3]);
        }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = i_hi - 8 + 8 * (e >> 1), j = nt * 8 + 2 * tq + (e & 1);
            p[nt][e] = j <= i ? p[nt][e] * pw[i - j] : 0.f;
        }
    }
    // ---- O = P V + d^(i+1) Q S ----
    float o[4][4], o2[4][4];          // column tiles 4 cw .. 4 cw + 3 of the block
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; o2[nt][0] = o2[nt][1] = o2[nt][2] = o2[nt][3] = 0.f; }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
        if (kb > rw) continue;
        uint32_t pa[4] = {dc_pack(p[2 * kb][0], p[2 * kb][1]), dc_pack(p[2 * kb][2], p[2 * kb][3]),
                          dc_pack(p[2 * kb + 1][0], p[2 * kb + 1][1]), dc_pack(p[2 * kb + 1][2], p[2 * kb + 1][3])};
#pragma unroll
        for (int nl = 0; nl < 2; ++nl) {
            const int nb = 2 * cw + nl;
            if (2 * nb >= nt_count) continue;
            uint32_t bf[4];
            dc_ldm4t(bf, dc_smem(Vs + (kb * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * vs + nb * 16 + ((lane >> 4) << 3)));
            dc_mma(o[2 * nl], pa, bf[0], bf[1]);
            dc_mma(o[2 * nl + 1], pa, bf[2], bf[3]);
        }
    }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        if (kk >= ksteps) continue;
#pragma unroll
        for (int nl = 0; nl < 2; ++nl) {
            const int nb = 2 * cw + nl;
            if (2 * nb >= nt_count) continue;
            const int off = (kk * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * vs + nb * 16 + ((lane >> 4) << 3);
            uint32_t bh[4], bl[4];
            dc_ldm4t(bh, dc_smem(Sh + off));
            dc_ldm4t(bl, dc_smem(Sl + off));
            dc_mma(o2[2 * nl], qf[kk], bh[0], bh[1]);
            dc_mma(o2[2 * nl + 1], qf[kk], bh[2], bh[3]);
            dc_mma(o2[2 * nl], qf[kk], bl[0], bl[1]);
            dc_mma(o2[2 * nl + 1], qf[kk], bl[2], bl[3]);
        }
    }
    const float w_lo = pw[i_hi - 8 + 1], w_hi = pw[i_hi + 1];
    float* out_lo = a.out + (long long)(row0 + t0 + i_hi - 8) * a.n_heads * vdim + (long long)h * vdim + c0;
    float* out_hi = out_lo + 8LL * a.n_heads * vdim;
#pragma unroll
    for (int nl = 0; nl < 4; ++nl) {
        const int nt = 4 * cw + nl;
        if (nt >= nt_count) continue;
        const int c = nt * 8 + 2 * tq;
        if (i_hi - 8 < L) *reinterpret_cast<float2*>(out_lo + c) = make_float2(fmaf(w_lo, o2[nl][0], o[nl][0]), fmaf(w_lo, o2[nl][1], o[nl][1]));
        if (i_hi < L) *reinterpret_cast<float2*>(out_hi + c) = make_float2(fmaf(w_hi, o2[nl][2], o[nl][2]), fmaf(w_hi, o2[nl][3], o[nl][3]));
    }
}

// S' = d^L S + U over a sequence's chunks, a thread per four state elements; the work buffer keeps the state before each chunk
__global__ void __launch_bounds__(256) decay_chunk_scan_kernel(DecayAttentionArgs a, float* __restrict__ work) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int row0 = a.seq_start[seq], n = a.seq_start[seq + 1] - row0;
    if (n <= 0 || a.tok_pos[row0] < 0) return;
    int first = 0;                                  // the step's chunks before this sequence's
    for (int s = 0; s < seq; ++s) {
        const int m = a.seq_start[s + 1] - a.seq_start[s];
        if (m > 0 && a.tok_pos[a.seq_start[s]] >= 0) first += (m + DC_CHUNK - 1) / DC_CHUNK;
    }
    const long long per = (long long)a.dim * a.vdim;          // a multiple of 4 (both sizes are multiples of 16)
    const long long e = 4 * ((long long)blockIdx.z * blockDim.x + threadIdx.x);
    if (e >= per) return;
    const float decay = a.decay[h];
    const float full = decay > 0.f ? exp2f((float)DC_CHUNK * log2f(decay)) : 0.f;
    float4* S = reinterpret_cast<float4*>(a.state + ((long long)a.slots[seq] * a.n_heads + h) * per + e);
    float4 s = *S;
    const int chunks = (n + DC_CHUNK - 1) / DC_CHUNK;
    float4* w = reinterpret_cast<float4*>(work + ((long long)first * a.n_heads + h) * per + e);
    const long long step = (long long)a.n_heads * per / 4;
    // four chunks' values are asked for while the four before them are summed and stored: loads stay in flight throughout
    float4 u[4], nx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) u[i] = i < chunks ? __ldcg(w + i * step) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = 0; c < chunks; c += 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) nx[i] = c + 4 + i < chunks ? __ldcg(w + (4 + i) * step) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (c + i < chunks) {
                __stcg(w + i * step, s);
                const int L = min(DC_CHUNK, n - (c + i) * DC_CHUNK);
                const float dl = L == DC_CHUNK ? full : (decay > 0.f ? exp2f((float)L * log2f(decay)) : 0.f);
                s.x = fmaf(dl, s.x, u[i].x); s.y = fmaf(dl, s.y, u[i].y); s.z = fmaf(dl, s.z, u[i].z); s.w = fmaf(dl, s.w, u[i].w);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = nx[i];
        w += 4 * step;
    }
    *S = s;
}

extern "C" int rdl_decay_attention_chunked(const DecayAttentionArgs* a, void* work, long long work_bytes, void* stream) {
    if (int e = check_decay_args(a, "decay_attention_chunked")) return e;
    RDL_REQUIRE(a->dtype == RDL_BF16, "decay_attention_chunked: bfloat16 rows only");
    RDL_REQUIRE(a->dim % 16 == 0 && a->dim <= 128 && a->vdim % 16 == 0, "decay_attention_chunked: dim %d and vdim %d must be multiples of 16, dim at most 128",
                a->dim, a->vdim);
    RDL_REQUIRE(((uintptr_t)a->out & 7) == 0 && ((uintptr_t)a->state & 15) == 0 && ((uintptr_t)work & 15) == 0,
                "decay_attention_chunked: the output must be 8-byte aligned, state and work buffer 16-byte aligned");
    RDL_REQUIRE((a->v_col % 2) == 0 && (a->row_stride % 2) == 0 && ((uintptr_t)a->rows & 3) == 0,
                "decay_attention_chunked: the value heads must start at an even column of 4-byte aligned rows");
    if (a->n_tokens == 0 || a->n_seqs == 0) return 0;
    const int max_chunks = rdl_decay_attention_chunks(a->n_tokens, a->n_seqs);
    RDL_REQUIRE(work && work_bytes >= (long long)max_chunks * a->n_heads * a->dim * a->vdim * (long long)sizeof(float),
                "decay_attention_chunked: the work buffer is too small");
    const int qs = a->dim + DC_PAD, vs = DC_COLS + DC_PAD;
    const size_t smem_u = (size_t)(DC_CHUNK * qs + DC_CHUNK * vs) * 2;
    const size_t smem_o = (size_t)(2 * DC_CHUNK * qs + DC_CHUNK * vs + 2 * a->dim * vs) * 2;
    static bool opted = false;
    if (!opted) {
        RDL_CUDA(cudaFuncSetAttribute(decay_chunk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024), "decay_attention_chunked");
        opted = true;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(max_chunks, a->n_heads, (a->vdim + DC_COLS - 1) / DC_COLS);
    // 16-byte loads where every head starts on a 16-byte boundary and the rotated half is a whole number of them
    const int vec = ((uintptr_t)a->rows & 15) == 0 && a->row_stride % 8 == 0 && a->q_col % 8 == 0 && a->k_col % 8 == 0 && a->v_col % 8 == 0 &&
                    (a->rot_n / 2) % 8 == 0 && (a->rot_n == 0 || ((((uintptr_t)a->cos_t) | ((uintptr_t)a->sin_t)) & 15) == 0);
    RDL_CHECK_EX(rdl_launch(decay_chunk_kernel<false>, grid, dim3(DC_THREADS), smem_u, st, *a, (float*)work, vec), "decay_attention_chunked (chunk states)");
    const long long per = (long long)a->dim * a->vdim;
    RDL_CHECK_EX(rdl_launch(decay_chunk_scan_kernel, dim3(a->n_seqs, a->n_heads, (unsigned)((per / 4 + 127) / 128)), dim3(128), 0, st, *a, (float*)work),
                 "decay_attention_chunked (scan)");
    RDL_CHECK_EX(rdl_launch(decay_chunk_kernel<true>, grid, dim3(DC_THREADS), smem_o, st, *a, (float*)work, vec), "decay_attention_chunked (outputs)");
    return 0;
}

// chunks a step of n_tokens rows in n_seqs sequences can have at most (every sequence may end in a partial chunk)
extern "C" int rdl_decay_attention_chunks(int n_tokens, int n_seqs) {
    const int by_tokens = n_tokens / DC_CHUNK + n_seqs;
    return by_tokens < n_tokens ? by_tokens : n_tokens;
}

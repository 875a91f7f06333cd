// Kernels of two more recurrent mixers and of the parts that stand around them, beside ops_cells.cu:
//   * linear attention with a fixed decay per head:  S <- decay_h S + k v^T,  o = S^T q  (q, k, v under silu), and
//     the RMS norm of the concatenated heads under a sigmoid gate;
//   * the real-gated linear recurrent unit:  gates from square blocks of the convolved input,
//     a = exp(-c r softplus(lam)),  S <- a S + sqrt(1 - a^2) (i u),  output S gelu(y);
//   * a gate per head on attention outputs, a weighted sum of two branches, relu(z)^2, and the weighted sum of the
//     chosen experts' outputs with experts that hand their input on and a gated shared expert.
// Everything a recurrence touches, every norm and gate is float32; T is the compute type of projections and
// activations (bfloat16 or float32).
//
// Batch layout as everywhere: token-major rows; q_start[r] .. q_start[r + 1] are the rows of request r, seq_lens[r]
// its cached length after the step.  A request with seq_lens[r] <= 0 is padding of a captured step and is skipped,
// and so are rows at or beyond q_start[R].  The arithmetic behind a token is the same however its request was cut.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

}  // namespace

// ---------------------------------------------------------------- linear attention with a decay per head
//
// proj row: [q: heads * dim | k: heads * dim | v: heads * vdim | ...] (pre-activations).  Per request and head, token
// by token:  S <- decay S + silu(k) silu(v)^T,  o = S^T silu(q).  state: float32 [slots][heads][dim][vdim];
// out: float32 [rows][heads * vdim].
//
// A block of DA_WARPS warps takes one head of one request and DA_COLS value columns.  A lane is a column; warp w holds rows
// w RMAX .. (w + 1) RMAX - 1 of every column in registers, so that q and k are read from shared memory as broadcasts,
// sixteen bytes a load, and nothing is exchanged between lanes: a warp leaves its part of a token's dot products in
// shared memory, and after a batch of DA_BATCH tokens the parts are added in the order of the warps.  Tokens are
// staged a batch at a time with their activation applied.
// FAST (the bfloat16 rows): the activation with the approximate exponential and division, whose error is far below
// the rounding of the projected values.  VEC (bfloat16 rows whose sizes and addresses are in steps of 8 elements):
// a batch's values are fetched sixteen bytes a load into registers while the batch in front is computed, so that no
// token waits for memory; otherwise a thread has four loads in flight while it stages.
#define DA_WARPS 16
#define DA_COLS 32
#define DA_BATCH 16
#define DA_MAX_DIM 256
#define DA_MAX_VEC 3  // 16-byte loads a thread issues for one batch: 16 * (2 * 256 / 8 + 32 / 8) / 512, rounded up

template <bool FAST>
__device__ __forceinline__ float silu_act(float z) {
    return FAST ? __fdividef(z, 1.0f + __expf(-z)) : z / (1.0f + expf(-z));
}

template <int RMAX>
constexpr int da_smem_bytes() { return (2 * DA_BATCH * DA_WARPS * RMAX + DA_BATCH * DA_COLS + DA_WARPS * DA_BATCH * DA_COLS) * 4; }

template <typename T, int RMAX, bool FAST, bool VEC>
__global__ void __launch_bounds__(DA_WARPS * 32)
decay_attention_kernel(const T* __restrict__ proj, int64_t stride, const float* __restrict__ decay, float* __restrict__ state,
                       float* __restrict__ out, const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                       const int32_t* __restrict__ slots, int heads, int dim, int vdim, int n_slots, int* err) {
    constexpr int GROUPS = RMAX / 4, W = DA_WARPS * RMAX;  // W: rows of shared memory a token's q (or k) takes
    const int col_blocks = (vdim + DA_COLS - 1) / DA_COLS;
    const int h = blockIdx.x / col_blocks, cb = blockIdx.x % col_blocks, r = blockIdx.y;
    const float d = decay[h];
    pdl_wait();
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    extern __shared__ __align__(16) float da_smem[];
    float* qs = da_smem;                       // [DA_BATCH][W]
    float* ks = qs + DA_BATCH * W;             // [DA_BATCH][W]
    float* vs = ks + DA_BATCH * W;             // [DA_BATCH][DA_COLS]
    float* red = vs + DA_BATCH * DA_COLS;      // [DA_WARPS][DA_BATCH][DA_COLS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, j = cb * DA_COLS + lane;
    const bool live = j < vdim;
    const int row0 = warp * RMAX;
    if (dim < W)  // rows behind the head's last one stay zero
        for (int i = tid; i < 2 * DA_BATCH * (W - dim); i += blockDim.x) qs[(i / (W - dim)) * W + dim + i % (W - dim)] = 0.f;
    float* sp = state + ((int64_t)slot * heads + h) * dim * vdim + (live ? j : 0);  // a row's columns lie side by side
    float S[RMAX];
#pragma unroll
    for (int i = 0; i < RMAX; ++i) S[i] = (live && row0 + i < dim) ? sp[(int64_t)(row0 + i) * vdim] : 0.f;
    const int64_t k_off = (int64_t)heads * dim + (int64_t)h * dim, v_off = 2 * (int64_t)heads * dim + (int64_t)h * vdim;
    // VEC: the items of a batch are 16-byte pieces, per token dim / 8 of q, dim / 8 of k and DA_COLS / 8 of v
    const int dim8 = dim >> 3, ipt = 2 * dim8 + DA_COLS / 8;
    uint4 raw[DA_MAX_VEC];
    auto issue = [&](int t0, int nb) {
#pragma unroll
        for (int w = 0; w < DA_MAX_VEC; ++w) {
            const int i = tid + w * DA_WARPS * 32;
            raw[w] = make_uint4(0u, 0u, 0u, 0u);
            if (i < nb * ipt) {
                const int t = i / ipt, c = i - t * ipt;
                const bf16* row = reinterpret_cast<const bf16*>(proj) + (int64_t)(q0 + t0 + t) * stride;
                const bf16* src = c < dim8 ? row + (int64_t)h * dim + c * 8
                                : c < 2 * dim8 ? row + k_off + (c - dim8) * 8 : row + v_off + cb * DA_COLS + (c - 2 * dim8) * 8;
                if (c < 2 * dim8 || cb * DA_COLS + (c - 2 * dim8) * 8 < vdim) raw[w] = *reinterpret_cast<const uint4*>(src);
            }
        }
    };
    auto deposit = [&](int nb) {
#pragma unroll
        for (int w = 0; w < DA_MAX_VEC; ++w) {
            const int i = tid + w * DA_WARPS * 32;
            if (i < nb * ipt) {
                const int t = i / ipt, c = i - t * ipt;
                float* dst = c < dim8 ? qs + t * W + c * 8 : c < 2 * dim8 ? ks + t * W + (c - dim8) * 8 : vs + t * DA_COLS + (c - 2 * dim8) * 8;
                const uint32_t q[4] = {raw[w].x, raw[w].y, raw[w].z, raw[w].w};
                float f[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    f[2 * e] = silu_act<FAST>(__uint_as_float(q[e] << 16));
                    f[2 * e + 1] = silu_act<FAST>(__uint_as_float(q[e] & 0xffff0000u));
                }
                *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
            }
        }
    };
    if (VEC) issue(0, min(DA_BATCH, q_len));
    for (int t0 = 0; t0 < q_len; t0 += DA_BATCH) {
        const int nb = min(DA_BATCH, q_len - t0);
        __syncthreads();  // the batch in front is done with shared memory (and, the first time, the zeros are in place)
        if (VEC) {
            deposit(nb);
            __syncthreads();
            if (t0 + DA_BATCH < q_len) issue(t0 + DA_BATCH, min(DA_BATCH, q_len - t0 - DA_BATCH));  // in flight while this batch is computed
        } else {
            const int n_qk = nb * dim, n_all = n_qk + nb * DA_COLS;
            for (int i0 = tid; i0 < n_all; i0 += 4 * blockDim.x) {  // four loads (pairs, for q and k) in flight
                float a[4], b[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int i = i0 + w * blockDim.x;
                    a[w] = b[w] = 0.f;
                    if (i < n_qk) {
                        const int t = i / dim, e = i - t * dim;
                        const T* row = proj + (int64_t)(q0 + t0 + t) * stride;
                        a[w] = to_float(row[(int64_t)h * dim + e]);
                        b[w] = to_float(row[k_off + e]);
                    } else if (i < n_all) {
                        const int t = (i - n_qk) / DA_COLS, e = (i - n_qk) - t * DA_COLS;
                        if (cb * DA_COLS + e < vdim) a[w] = to_float(proj[(int64_t)(q0 + t0 + t) * stride + v_off + cb * DA_COLS + e]);
                    }
                }
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int i = i0 + w * blockDim.x;
                    if (i < n_qk) {
                        const int t = i / dim, e = i - t * dim;
                        qs[t * W + e] = silu_act<FAST>(a[w]);
                        ks[t * W + e] = silu_act<FAST>(b[w]);
                    } else if (i < n_all) {
                        const int t = (i - n_qk) / DA_COLS, e = (i - n_qk) - t * DA_COLS;
                        vs[t * DA_COLS + e] = silu_act<FAST>(a[w]);  // silu(0) = 0 behind the last column
                    }
                }
            }
            __syncthreads();
        }
        if (row0 < dim) {  // (a warp whose rows lie behind the head's last one has nothing to add)
            for (int t = 0; t < nb; t += 2) {  // two tokens' loads in flight; their updates in order
                const int t1 = min(t + 1, nb - 1);
                const float v0 = vs[t * DA_COLS + lane], v1 = vs[t1 * DA_COLS + lane];
                float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
                for (int g = 0; g < GROUPS; ++g) {
                    const float4 k4 = *reinterpret_cast<const float4*>(ks + t * W + row0 + 4 * g);
                    const float4 q4 = *reinterpret_cast<const float4*>(qs + t * W + row0 + 4 * g);
                    const float4 k5 = *reinterpret_cast<const float4*>(ks + t1 * W + row0 + 4 * g);
                    const float4 q5 = *reinterpret_cast<const float4*>(qs + t1 * W + row0 + 4 * g);
                    S[4 * g + 0] = fmaf(k4.x, v0, d * S[4 * g + 0]);
                    S[4 * g + 1] = fmaf(k4.y, v0, d * S[4 * g + 1]);
                    S[4 * g + 2] = fmaf(k4.z, v0, d * S[4 * g + 2]);
                    S[4 * g + 3] = fmaf(k4.w, v0, d * S[4 * g + 3]);
                    a0 = fmaf(S[4 * g + 0], q4.x, a0);
                    a1 = fmaf(S[4 * g + 1], q4.y, a1);
                    a0 = fmaf(S[4 * g + 2], q4.z, a0);
                    a1 = fmaf(S[4 * g + 3], q4.w, a1);
                    if (t + 1 < nb) {
                        S[4 * g + 0] = fmaf(k5.x, v1, d * S[4 * g + 0]);
                        S[4 * g + 1] = fmaf(k5.y, v1, d * S[4 * g + 1]);
                        S[4 * g + 2] = fmaf(k5.z, v1, d * S[4 * g + 2]);
                        S[4 * g + 3] = fmaf(k5.w, v1, d * S[4 * g + 3]);
                        b0 = fmaf(S[4 * g + 0], q5.x, b0);
                        b1 = fmaf(S[4 * g + 1], q5.y, b1);
                        b0 = fmaf(S[4 * g + 2], q5.z, b0);
                        b1 = fmaf(S[4 * g + 3], q5.w, b1);
                    }
                }
                red[(warp * DA_BATCH + t) * DA_COLS + lane] = a0 + a1;
                if (t + 1 < nb) red[(warp * DA_BATCH + t + 1) * DA_COLS + lane] = b0 + b1;
            }
        }
        __syncthreads();
        const int n_warps = min(DA_WARPS, (dim + RMAX - 1) / RMAX);  // warps that hold rows of the head
        for (int i = tid; i < nb * DA_COLS; i += blockDim.x) {
            const int t = i / DA_COLS, c = i - t * DA_COLS;
            if (cb * DA_COLS + c >= vdim) continue;
            float sum = 0.f;
            for (int w = 0; w < n_warps; ++w) sum += red[(w * DA_BATCH + t) * DA_COLS + c];
            out[(int64_t)(q0 + t0 + t) * heads * vdim + (int64_t)h * vdim + cb * DA_COLS + c] = sum;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < RMAX; ++i)
            if (row0 + i < dim) sp[(int64_t)(row0 + i) * vdim] = S[i];
    }
}

template <typename T, int RMAX, bool FAST, bool VEC>
static int launch_decay_attention(const void* proj, int64_t stride, const float* decay, float* state, float* out,
                                  const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int R, int heads,
                                  int dim, int vdim, int n_slots, int* err, cudaStream_t stream) {
    constexpr int smem = da_smem_bytes<RMAX>();
    static SsPerDevice opted;
    if (int rc = ss_opt_in_smem(decay_attention_kernel<T, RMAX, FAST, VEC>, smem, opted)) return rc;
    const dim3 grid(heads * ((vdim + DA_COLS - 1) / DA_COLS), R), block(DA_WARPS * 32);
    ss_launch(decay_attention_kernel<T, RMAX, FAST, VEC>, grid, block, smem, stream, (const T*)proj, stride, decay, state, out,
              q_start, seq_lens, slots, heads, dim, vdim, n_slots, err);
    return SS_LAUNCH_CHECK();
}

extern "C" int ss_decay_attention(const void* proj, int64_t stride, const float* decay, float* state, float* out,
                                  const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int R, int heads,
                                  int dim, int vdim, int n_slots, int dtype, int* err, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (heads < 1 || dim < 1 || dim > DA_MAX_DIM || vdim < 1) return (int)cudaErrorInvalidValue;
#define DA_GO(T, RMAX, FAST, VEC)                                                                                         \
    return launch_decay_attention<T, RMAX, FAST, VEC>(proj, stride, decay, state, out, q_start, seq_lens, slots, R, heads, \
                                                      dim, vdim, n_slots, err, stream)
#define DA_PICK(T, FAST, VEC)                                                                                           \
    do {                                                                                                                \
        if (dim <= 4 * DA_WARPS) DA_GO(T, 4, FAST, VEC);                                                                \
        else if (dim <= 8 * DA_WARPS) DA_GO(T, 8, FAST, VEC);                                                           \
        else DA_GO(T, 16, FAST, VEC);                                                                                   \
    } while (0)
    const bool vec = dtype == SS_BF16 && dim % 8 == 0 && vdim % 8 == 0 && stride % 8 == 0 && ((uintptr_t)proj & 15) == 0;
    if (dtype == SS_BF16) {
        if (vec) DA_PICK(bf16, true, true); else DA_PICK(bf16, true, false);
    } else {
        DA_PICK(float, false, false);
    }
#undef DA_PICK
#undef DA_GO
    return 0;
}

// ---------------------------------------------------------------- RMS norm of a row under a sigmoid gate
//
// out[row][c] = x[row][c] / sqrt(mean(x[row]^2) + eps) * weight[c] * sigmoid(gate[row][c]); x float32 [rows][C], gate
// a view with rows gate_stride apart, weight float32.  A block per row.
template <typename T>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ x, const T* __restrict__ gate, int64_t gate_stride,
                     const float* __restrict__ weight, T* __restrict__ out, int C, float eps) {
    pdl_wait();
    __shared__ float scratch[33];
    const float* xr = x + (int64_t)blockIdx.x * C;
    const T* gr = gate + (int64_t)blockIdx.x * gate_stride;
    float ss = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)C + eps);
    for (int c = threadIdx.x; c < C; c += blockDim.x)
        out[(int64_t)blockIdx.x * C + c] = from_float<T>(xr[c] * rstd * weight[c] * sigmoid_f(to_float(gr[c])));
}

extern "C" int ss_gated_rmsnorm(const float* x, const void* gate, int64_t gate_stride, const float* weight, void* out,
                                int n_rows, int C, float eps, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (dtype == SS_BF16)
        ss_launch(gated_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, x, (const bf16*)gate, gate_stride, weight,
                  (bf16*)out, C, eps);
    else
        ss_launch(gated_rmsnorm_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, (const float*)gate, gate_stride, weight,
                  (float*)out, C, eps);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- gates from square blocks of the input
//
// u [rows][blocks * bs] (row stride u_stride); W [blocks][2 bs][bs]: per block the rows of the first gate, then those
// of the second; bias float32 [blocks][2 bs] or null.  pre[b][row][o] = bias[b][o] + sum_i W[b][o][i] u[row][b bs + i],
// float32 [blocks][rows][2 bs], accumulated in float32 in a fixed order.  A block of threads takes 32 rows and 64
// outputs of one block of the input.
#define BG_ROWS 32
#define BG_OUT 64
#define BG_K 32
template <typename T>
__global__ void __launch_bounds__(256)
block_gates_kernel(const T* __restrict__ u, int64_t u_stride, const T* __restrict__ W, const float* __restrict__ bias,
                   float* __restrict__ pre, int n_rows, int bs) {
    pdl_wait();
    __shared__ float Us[BG_ROWS][BG_K + 1], Ws[BG_OUT][BG_K + 1];
    const int b = blockIdx.z, row0 = blockIdx.x * BG_ROWS, o0 = blockIdx.y * BG_OUT, n_out = 2 * bs;
    const int tid = threadIdx.x, tx = tid % BG_OUT, ty = tid / BG_OUT;  // ty: 0..3, eight rows each
    const T* Wb = W + (int64_t)b * n_out * bs;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k0 = 0; k0 < bs; k0 += BG_K) {
        for (int i = tid; i < BG_ROWS * BG_K; i += 256) {
            const int rr = i / BG_K, kk = i % BG_K;
            Us[rr][kk] = (row0 + rr < n_rows && k0 + kk < bs) ? to_float(u[(int64_t)(row0 + rr) * u_stride + (int64_t)b * bs + k0 + kk]) : 0.f;
        }
        for (int i = tid; i < BG_OUT * BG_K; i += 256) {
            const int oo = i / BG_K, kk = i % BG_K;
            Ws[oo][kk] = (o0 + oo < n_out && k0 + kk < bs) ? to_float(Wb[(int64_t)(o0 + oo) * bs + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < BG_K; ++kk) {
            const float w = Ws[tx][kk];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(Us[ty * 8 + i][kk], w, acc[i]);
        }
        __syncthreads();
    }
    const int o = o0 + tx;
    if (o >= n_out) return;
    const float bv = bias ? bias[(int64_t)b * n_out + o] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = row0 + ty * 8 + i;
        if (row < n_rows) pre[((int64_t)b * n_rows + row) * n_out + o] = acc[i] + bv;
    }
}

extern "C" int ss_block_gates(const void* u, int64_t u_stride, const void* W, const float* bias, float* pre, int n_rows,
                              int blocks, int bs, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (blocks < 1 || bs < 1) return (int)cudaErrorInvalidValue;
    const dim3 grid((n_rows + BG_ROWS - 1) / BG_ROWS, (2 * bs + BG_OUT - 1) / BG_OUT, blocks);
    if (dtype == SS_BF16)
        ss_launch(block_gates_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)u, u_stride, (const bf16*)W, bias, pre, n_rows, bs);
    else
        ss_launch(block_gates_kernel<float>, grid, dim3(256), 0, stream, (const float*)u, u_stride, (const float*)W, bias, pre, n_rows, bs);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- the real-gated linear recurrence
//
// Per request and channel c = b bs + o, token by token, with pre[b][row] = [first gate: bs | second gate: bs] (float32;
// their biases are added here where `bias` is given):
//   r = sigmoid(pre1),  i = sigmoid(pre2),  a = exp(-rate r softplus(lam[c])),  S <- a S + sqrt(1 - a^2) i u,
//   out = S * gelu_tanh(y)            (y: a view of the projection, rows y_stride apart; u [rows][C])
// state float32 [slots][C].
//
// A block takes one request and 32 neighbouring channels (a lane each, so that a warp reads whole lines) and cuts the
// request's rows of this step into one segment per warp.  The recurrence is linear in S: a warp first walks its segment
// from S = 0, which gives the segment's map S -> A S + B (and leaves every token's a and b in place of its two gate
// values); the maps of the segments in front, applied in order to the request's state, give the warp its start; the
// second walk is the recurrence as written and writes the outputs.  With one warp (a decode step) the first walk
// starts from the state itself.  The same algebra however a request is cut; the roundings differ with the segments.
#define GL_MAX_SEGS 16
template <typename T>
__global__ void __launch_bounds__(32 * GL_MAX_SEGS)
gated_linear_recurrence_kernel(float* __restrict__ pre, const float* __restrict__ bias, const T* __restrict__ u,
                               const T* __restrict__ y, int64_t y_stride, const float* __restrict__ lam, float rate,
                               float* __restrict__ state, T* __restrict__ out, const int32_t* __restrict__ q_start,
                               const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ slots, int n_rows, int C,
                               int bs, int n_slots, int* err) {
    const int lane = threadIdx.x & 31, seg = threadIdx.x >> 5, n_segs = blockDim.x >> 5;
    const int c = blockIdx.x * 32 + lane, r = blockIdx.y;
    const bool live = c < C;
    const int b = live ? c / bs : 0, o = live ? c - b * bs : 0;
    const float neg = live ? -rate * softplus_f(lam[c]) : 0.f;
    const float b1 = (bias && live) ? bias[(int64_t)b * 2 * bs + o] : 0.f, b2 = (bias && live) ? bias[(int64_t)b * 2 * bs + bs + o] : 0.f;
    pdl_wait();
    __shared__ float seg_a[GL_MAX_SEGS][32], seg_b[GL_MAX_SEGS][32];
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    const int per = (q_len + n_segs - 1) / n_segs;
    const int t0 = min(q_len, seg * per), t1 = min(q_len, t0 + per);
    float* p = pre + ((int64_t)b * n_rows + q0) * 2 * bs + o;
    const float s_init = live ? state[(int64_t)slot * C + c] : 0.f;
    float A = 1.f, S = n_segs == 1 ? s_init : 0.f;
    if (live) {
        for (int t = t0; t < t1; t += 4) {  // the loads of four tokens are in flight together
            float z1[4], z2[4], uv[4], yv[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int tt = min(t + w, t1 - 1);
                z1[w] = p[(int64_t)tt * 2 * bs];
                z2[w] = p[(int64_t)tt * 2 * bs + bs];
                uv[w] = to_float(u[(int64_t)(q0 + tt) * C + c]);
                yv[w] = n_segs == 1 ? to_float(y[(int64_t)(q0 + tt) * y_stride + c]) : 0.f;
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                if (t + w >= t1) break;
                const float g1 = sigmoid_f(z1[w] + b1), g2 = sigmoid_f(z2[w] + b2);
                const float la = neg * g1;
                const float a = expf(la);
                const float add = sqrtf(-expm1f(2.0f * la)) * (g2 * uv[w]);  // 1 - a^2 without cancellation where a is close to one
                S = fmaf(a, S, add);
                if (n_segs == 1) {
                    out[(int64_t)(q0 + t + w) * C + c] = from_float<T>(S * gelu_tanh_f(yv[w]));
                } else {
                    p[(int64_t)(t + w) * 2 * bs] = a;
                    p[(int64_t)(t + w) * 2 * bs + bs] = add;
                    A *= a;
                }
            }
        }
    }
    if (n_segs == 1) {
        if (live) state[(int64_t)slot * C + c] = S;
        return;
    }
    seg_a[seg][lane] = A;
    seg_b[seg][lane] = S;
    __syncthreads();
    S = s_init;
    for (int v = 0; v < seg; ++v) S = fmaf(seg_a[v][lane], S, seg_b[v][lane]);
    if (!live) return;
    for (int t = t0; t < t1; t += 4) {
        float av[4], bv[4], yv[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int tt = min(t + w, t1 - 1);
            av[w] = p[(int64_t)tt * 2 * bs];
            bv[w] = p[(int64_t)tt * 2 * bs + bs];
            yv[w] = to_float(y[(int64_t)(q0 + tt) * y_stride + c]);
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            if (t + w >= t1) break;
            S = fmaf(av[w], S, bv[w]);
            out[(int64_t)(q0 + t + w) * C + c] = from_float<T>(S * gelu_tanh_f(yv[w]));
        }
    }
    // the warp with the request's last token leaves the state
    if (t1 == q_len && t0 < t1) state[(int64_t)slot * C + c] = S;
}

extern "C" int ss_gated_linear_recurrence(float* pre, const float* bias, const void* u, const void* y, int64_t y_stride,
                                          const float* lam, float rate, float* state, void* out, const int32_t* q_start,
                                          const int32_t* seq_lens, const int32_t* slots, int R, int n_rows, int C, int bs,
                                          int n_slots, int dtype, int* err, cudaStream_t stream, int segments) {
    if (R <= 0 || n_rows <= 0) return 0;
    if (C < 1 || bs < 1 || C % bs || segments < 1 || segments > GL_MAX_SEGS) return (int)cudaErrorInvalidValue;
    const dim3 grid((C + 31) / 32, R), block(32 * segments);
    if (dtype == SS_BF16)
        ss_launch(gated_linear_recurrence_kernel<bf16>, grid, block, 0, stream, pre, bias, (const bf16*)u, (const bf16*)y,
                  y_stride, lam, rate, state, (bf16*)out, q_start, seq_lens, slots, n_rows, C, bs, n_slots, err);
    else
        ss_launch(gated_linear_recurrence_kernel<float>, grid, block, 0, stream, pre, bias, (const float*)u,
                  (const float*)y, y_stride, lam, rate, state, (float*)out, q_start, seq_lens, slots, n_rows, C, bs, n_slots, err);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- a gate per head
//
// x[row][h * D + d] *= sigmoid(gate[row][h]): x [rows][heads * D] contiguous, gate a view with rows gate_stride apart.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const T* __restrict__ gate, int64_t gate_stride, int64_t n, int heads, int D) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int64_t row = idx / ((int64_t)heads * D);
    const int h = (int)((idx - row * heads * D) / D);
    x[idx] = from_float<T>(to_float(x[idx]) * sigmoid_f(to_float(gate[row * gate_stride + h])));
}

extern "C" int ss_head_gate(void* x, const void* gate, int64_t gate_stride, int n_rows, int heads, int D, int dtype,
                            cudaStream_t stream) {
    const int64_t n = (int64_t)n_rows * heads * D;
    if (n <= 0) return 0;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == SS_BF16)
        ss_launch(head_gate_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)x, (const bf16*)gate, gate_stride, n, heads, D);
    else
        ss_launch(head_gate_kernel<float>, grid, dim3(256), 0, stream, (float*)x, (const float*)gate, gate_stride, n, heads, D);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- out = sa * a + sb * b, element by element
template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, float sa, const T* __restrict__ b, float sb, T* __restrict__ out, int64_t n) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) out[idx] = from_float<T>(fmaf(sa, to_float(a[idx]), sb * to_float(b[idx])));
}

extern "C" int ss_scaled_sum(const void* a, float sa, const void* b, float sb, void* out, int64_t n, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == SS_BF16)
        ss_launch(scaled_sum_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)a, sa, (const bf16*)b, sb, (bf16*)out, n);
    else
        ss_launch(scaled_sum_kernel<float>, grid, dim3(256), 0, stream, (const float*)a, sa, (const float*)b, sb, (float*)out, n);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- relu(z)^2 over the first `cols` columns of rows
template <typename T>
__global__ void relu_square_kernel(const T* in, int64_t in_stride, T* out, int64_t n, int cols) {  // in may be out
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int64_t row = idx / cols;
    const float z = to_float(in[row * in_stride + (idx - row * cols)]);
    out[idx] = from_float<T>(z > 0.f ? z * z : 0.f);
}

// bfloat16 with columns, row stride and both addresses in steps of 8 elements: sixteen bytes a load and a store
__global__ void relu_square_bf16x8_kernel(const bf16* in, int64_t in_stride, bf16* out, int64_t n8, int cols8) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n8) return;
    const int64_t row = idx / cols8;
    const uint4 raw = *reinterpret_cast<const uint4*>(in + row * in_stride + (idx - row * cols8) * 8);
    const uint32_t q[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float lo = __uint_as_float(q[e] << 16), hi = __uint_as_float(q[e] & 0xffff0000u);
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(lo > 0.f ? lo * lo : 0.f, hi > 0.f ? hi * hi : 0.f);
        o[e] = *reinterpret_cast<const uint32_t*>(&h2);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

extern "C" int ss_relu_square(const void* in, int64_t in_stride, void* out, int n_rows, int cols, int dtype, cudaStream_t stream) {
    const int64_t n = (int64_t)n_rows * cols;
    if (n <= 0) return 0;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == SS_BF16 && cols % 8 == 0 && in_stride % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0)
        ss_launch(relu_square_bf16x8_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, stream, (const bf16*)in, in_stride,
                  (bf16*)out, n / 8, cols / 8);
    else if (dtype == SS_BF16)
        ss_launch(relu_square_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)in, in_stride, (bf16*)out, n, cols);
    else
        ss_launch(relu_square_kernel<float>, grid, dim3(256), 0, stream, (const float*)in, in_stride, (float*)out, n, cols);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- weighted sum of the chosen experts' outputs
//
// out[t][i] = round_T(sum_k w[t][k] term(t, k)[i] + g[t] shared[t][i]), float32 arithmetic in the order of the choices:
// term(t, k) is the output of expert ids[t][k], either y[t][k] (float32 rows in the order of the choices) or
// sorted[place[t * top + k]] (bfloat16 rows in the plan's order), or, for an expert from `real` on, which has no
// weights and hands its input on, x[t].  w null: ones.  g[t] = sigmoid(gate[t * gate_stride]) (null: one).
template <typename T>
__global__ void moe_mix_kernel(const float* __restrict__ y, const bf16* __restrict__ sorted, const int32_t* __restrict__ place,
                               const int32_t* __restrict__ ids, const float* __restrict__ w, int real, const T* __restrict__ x,
                               const T* __restrict__ shared, const float* __restrict__ gate, int64_t gate_stride,
                               T* __restrict__ out, int64_t n, int hidden, int top) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int64_t t = idx / hidden;
    const int i = (int)(idx - t * hidden);
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
        const int64_t a = t * top + k;
        float term;
        if (ids[a] >= real) term = to_float(x[idx]);
        else term = sorted ? to_float(sorted[(int64_t)place[a] * hidden + i]) : y[a * hidden + i];
        v = fmaf(w ? w[a] : 1.f, term, v);
    }
    if (shared) v = fmaf(gate ? sigmoid_f(gate[t * gate_stride]) : 1.f, to_float(shared[idx]), v);
    out[idx] = from_float<T>(v);
}

extern "C" int ss_moe_mix(const float* y, const void* sorted, const int32_t* place, const int32_t* ids, const float* w,
                          int real, const void* x, const void* shared, const float* gate, int64_t gate_stride, void* out,
                          int n_tokens, int hidden, int top, int dtype, cudaStream_t stream) {
    const int64_t n = (int64_t)n_tokens * hidden;
    if (n <= 0) return 0;
    if (!ids || !x || (!y && !(sorted && place))) return (int)cudaErrorInvalidValue;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == SS_BF16)
        ss_launch(moe_mix_kernel<bf16>, grid, dim3(256), 0, stream, y, (const bf16*)sorted, place, ids, w, real, (const bf16*)x,
                  (const bf16*)shared, gate, gate_stride, (bf16*)out, n, hidden, top);
    else
        ss_launch(moe_mix_kernel<float>, grid, dim3(256), 0, stream, y, (const bf16*)nullptr, (const int32_t*)nullptr, ids, w, real,
                  (const float*)x, (const float*)shared, gate, gate_stride, (float*)out, n, hidden, top);
    return SS_LAUNCH_CHECK();
}

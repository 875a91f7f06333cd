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
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

}  // namespace

// ---------------------------------------------------------------- linear attention with a decay per head
//
// proj row: [q: heads * dim | k: heads * dim | v: heads * vdim | ...] (pre-activations).  Per request and head, token
// by token:  S <- decay S + silu(k) silu(v)^T,  o = S^T silu(q).  state: float32 [slots][heads][vdim][dim];
// out: float32 [rows][heads * vdim].  A block takes one head of one request and DA_COLS value columns; a column is
// held by DA_LANES lanes, each with every DA_LANES-th row of it in registers; tokens are staged DA_BATCH at a time.
#define DA_LANES 8
#define DA_COLS 32
#define DA_BATCH 16
#define DA_MAX_DIM 256

template <typename T, int RMAX>
__global__ void __launch_bounds__(DA_LANES * DA_COLS)
decay_attention_kernel(const T* __restrict__ proj, int64_t stride, const float* __restrict__ decay, float* __restrict__ state,
                       float* __restrict__ out, const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                       const int32_t* __restrict__ slots, int heads, int dim, int vdim, int n_slots, int* err) {
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
    __shared__ float qs[DA_BATCH][DA_MAX_DIM], ks[DA_BATCH][DA_MAX_DIM], vs[DA_BATCH][DA_COLS];
    const int tid = threadIdx.x, sub = tid % DA_LANES, col = tid / DA_LANES, j = cb * DA_COLS + col;
    const bool live = j < vdim;
    float* sp = state + (((int64_t)slot * heads + h) * vdim + (live ? j : 0)) * dim;
    float S[RMAX];
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
        const int row = sub + i * DA_LANES;
        S[i] = (live && row < dim) ? sp[row] : 0.f;
    }
    const int64_t k_off = (int64_t)heads * dim + (int64_t)h * dim, v_off = 2 * (int64_t)heads * dim + (int64_t)h * vdim;
    for (int t0 = 0; t0 < q_len; t0 += DA_BATCH) {
        const int nb = min(DA_BATCH, q_len - t0);
        __syncthreads();
        for (int i = tid; i < nb * dim; i += blockDim.x) {
            const int t = i / dim, e = i - t * dim;
            const T* row = proj + (int64_t)(q0 + t0 + t) * stride;
            qs[t][e] = silu_f(to_float(row[(int64_t)h * dim + e]));
            ks[t][e] = silu_f(to_float(row[k_off + e]));
        }
        for (int i = tid; i < nb * DA_COLS; i += blockDim.x) {
            const int t = i / DA_COLS, e = i - t * DA_COLS;
            vs[t][e] = cb * DA_COLS + e < vdim ? silu_f(to_float(proj[(int64_t)(q0 + t0 + t) * stride + v_off + cb * DA_COLS + e])) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nb; ++t) {
            const float v = vs[t][col];
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < RMAX; ++i) {
                const int row = sub + i * DA_LANES;
                if (row < dim) {
                    S[i] = fmaf(ks[t][row], v, d * S[i]);
                    acc = fmaf(S[i], qs[t][row], acc);
                }
            }
#pragma unroll
            for (int o = DA_LANES / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (sub == 0 && live) out[(int64_t)(q0 + t0 + t) * heads * vdim + (int64_t)h * vdim + j] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < RMAX; ++i) {
            const int row = sub + i * DA_LANES;
            if (row < dim) sp[row] = S[i];
        }
    }
}

extern "C" int ss_decay_attention(const void* proj, int64_t stride, const float* decay, float* state, float* out,
                                  const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int R, int heads,
                                  int dim, int vdim, int n_slots, int dtype, int* err, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (heads < 1 || dim < 1 || dim > DA_MAX_DIM || vdim < 1) return (int)cudaErrorInvalidValue;
    const dim3 grid(heads * ((vdim + DA_COLS - 1) / DA_COLS), R), block(DA_LANES * DA_COLS);
#define DA_GO(T, RMAX)                                                                                                  \
    ss_launch(decay_attention_kernel<T, RMAX>, grid, block, 0, stream, (const T*)proj, stride, decay, state, out, q_start, \
              seq_lens, slots, heads, dim, vdim, n_slots, err)
#define DA_PICK(T)                                                                                                      \
    do {                                                                                                                \
        if (dim <= 8 * DA_LANES) DA_GO(T, 8);                                                                           \
        else if (dim <= 16 * DA_LANES) DA_GO(T, 16);                                                                    \
        else DA_GO(T, 32);                                                                                              \
    } while (0)
    if (dtype == SS_BF16) DA_PICK(bf16); else DA_PICK(float);
#undef DA_PICK
#undef DA_GO
    return SS_LAUNCH_CHECK();
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
// Per request and channel c = b bs + o, token by token, with pre[b][row] = [first gate: bs | second gate: bs] (float32,
// their biases added where `bias` is given):
//   r = sigmoid(pre1),  i = sigmoid(pre2),  a = exp(-rate r softplus(lam[c])),  S <- a S + sqrt(1 - a^2) i u,
//   out = S * gelu_tanh(y)            (y: a view of the projection, rows y_stride apart; u [rows][C])
// state float32 [slots][C].  A thread per request and channel.
template <typename T>
__global__ void __launch_bounds__(128)
gated_linear_recurrence_kernel(const float* __restrict__ pre, const float* __restrict__ bias, const T* __restrict__ u,
                               const T* __restrict__ y, int64_t y_stride, const float* __restrict__ lam, float rate,
                               float* __restrict__ state, T* __restrict__ out, const int32_t* __restrict__ q_start,
                               const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ slots, int n_rows, int C,
                               int bs, int n_slots, int* err) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    const int b = c < C ? c / bs : 0, o = c < C ? c - b * bs : 0;
    const float neg = c < C ? -rate * softplus_f(lam[c]) : 0.f;
    const float b1 = (bias && c < C) ? bias[(int64_t)b * 2 * bs + o] : 0.f, b2 = (bias && c < C) ? bias[(int64_t)b * 2 * bs + bs + o] : 0.f;
    pdl_wait();
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (c >= C || q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    float S = state[(int64_t)slot * C + c];
    const float* p = pre + ((int64_t)b * n_rows + q0) * 2 * bs + o;
    for (int t = 0; t < q_len; ++t) {
        const float g1 = sigmoid_f(p[(int64_t)t * 2 * bs] + b1), g2 = sigmoid_f(p[(int64_t)t * 2 * bs + bs] + b2);
        const float uv = to_float(u[(int64_t)(q0 + t) * C + c]);
        const float la = neg * g1;
        const float a = expf(la);
        // 1 - a^2 without cancellation where a is close to one
        const float keep = sqrtf(-expm1f(2.0f * la));
        S = fmaf(a, S, keep * (g2 * uv));
        out[(int64_t)(q0 + t) * C + c] = from_float<T>(S * gelu_tanh_f(to_float(y[(int64_t)(q0 + t) * y_stride + c])));
    }
    state[(int64_t)slot * C + c] = S;
}

extern "C" int ss_gated_linear_recurrence(const float* pre, const float* bias, const void* u, const void* y, int64_t y_stride,
                                          const float* lam, float rate, float* state, void* out, const int32_t* q_start,
                                          const int32_t* seq_lens, const int32_t* slots, int R, int n_rows, int C, int bs,
                                          int n_slots, int dtype, int* err, cudaStream_t stream) {
    if (R <= 0 || n_rows <= 0) return 0;
    if (C < 1 || bs < 1 || C % bs) return (int)cudaErrorInvalidValue;
    const dim3 grid((C + 127) / 128, R);
    if (dtype == SS_BF16)
        ss_launch(gated_linear_recurrence_kernel<bf16>, grid, dim3(128), 0, stream, pre, bias, (const bf16*)u, (const bf16*)y,
                  y_stride, lam, rate, state, (bf16*)out, q_start, seq_lens, slots, n_rows, C, bs, n_slots, err);
    else
        ss_launch(gated_linear_recurrence_kernel<float>, grid, dim3(128), 0, stream, pre, bias, (const float*)u,
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
__global__ void relu_square_kernel(const T* __restrict__ in, int64_t in_stride, T* __restrict__ out, int64_t n, int cols) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int64_t row = idx / cols;
    const float z = to_float(in[row * in_stride + (idx - row * cols)]);
    out[idx] = from_float<T>(z > 0.f ? z * z : 0.f);
}

extern "C" int ss_relu_square(const void* in, int64_t in_stride, void* out, int n_rows, int cols, int dtype, cudaStream_t stream) {
    const int64_t n = (int64_t)n_rows * cols;
    if (n <= 0) return 0;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == SS_BF16)
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

// Kernels of recurrent cells with per-request state and of latent attention, beside the parts of ops_mixers.cu:
//   * an embedding that is a sum of three rows (token table, a hashed table of (previous, current) token pairs,
//     a learned position table), written once per residual stream; the previous token is per-request state;
//   * the matrix-memory cell (mLSTM): S <- keep S + take k v^T with exponential gates and a running maximum,
//     and the per-head output norm with its gate;
//   * a gated recurrence per channel (minGRU) with its output gate;
//   * the xIELU activation of a feed-forward without a gate branch;
//   * latent attention: the norms of the two latents, rotation and page write of (rotated shared key | latent),
//     queries carried into the latent space head by head, and the heads' outputs carried up to values.
// Everything a recurrence touches, every norm, angle and gate is float32; T is the compute type of projections
// and activations (bfloat16 or float32).
//
// Batch layout as everywhere: token-major rows; q_start[r] .. q_start[r + 1] are the rows of request r, seq_lens[r]
// its cached length after the step.  A request with seq_lens[r] <= 0 is padding of a captured step and is skipped,
// and so are rows at or beyond q_start[R].  The arithmetic behind a token is the same however its request was cut.
#include "common.cuh"

namespace {

__device__ __forceinline__ int request_of_row(const int32_t* __restrict__ q_start, int R, int row) {
    if (row >= q_start[R]) return -1;
    int lo = 0, hi = R - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (q_start[mid] <= row) lo = mid; else hi = mid - 1;
    }
    return lo;
}

__device__ __forceinline__ float sigmoid_exact(float z) { return 1.0f / (1.0f + expf(-z)); }
// log(sigmoid(z)) without cancellation at either end
__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

}  // namespace

// ---------------------------------------------------------------- embedding as a sum of rows
//
// out[row][copy][:] = scale * table[token] + pair[hash] + pos_table[position], float32, every copy alike.
// hash = (previous * mul_prev + token * mul_cur) mod buckets; a request's first token takes row `buckets`.  The
// previous token of a step's first row is the request's state last_token[slot]; the block of that row also
// leaves the step's last token there (it reads before it writes, so no other block touches the entry).
template <typename T>
__global__ void __launch_bounds__(128)
embed_sum_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ positions, const T* __restrict__ table,
                 const T* __restrict__ pair, const T* __restrict__ pos_table, float* __restrict__ out,
                 int32_t* __restrict__ last_token, const int32_t* __restrict__ q_start,
                 const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ slots, int R, int hidden, int vocab,
                 int copies, int buckets, long long mul_prev, long long mul_cur, int n_positions, int n_slots, float scale,
                 int* err) {
    pdl_wait();
    const int row = blockIdx.x;
    const int token = tokens[row];
    const int r = request_of_row(q_start, R, row);
    const bool live = r >= 0 && seq_lens[r] > 0;
    __shared__ int prev_s;
    if (threadIdx.x == 0) {
        int prev = -1;
        if (live) {
            const int slot = slots[r];
            const bool has_slot = slot >= 0 && slot < n_slots;
            const bool first_row = row == q_start[r];
            if (pair && !has_slot) atomicOr(err, SS_ERR_SLOT_RANGE);
            if (positions[row] > 0) prev = !first_row ? tokens[row - 1] : (pair && has_slot ? last_token[slot] : -1);
            if (pair && has_slot && first_row) last_token[slot] = tokens[q_start[r + 1] - 1];
        }
        prev_s = prev;
    }
    __syncthreads();
    float* dst = out + (int64_t)row * copies * hidden;
    if (token < 0 || token >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_TOKEN_RANGE);
        for (int i = threadIdx.x; i < copies * hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const int p = live ? positions[row] : 0;
    const T* pair_row = nullptr;
    if (pair && live) {
        const int prev = prev_s;
        long long h = buckets;
        if (p > 0 && prev >= 0 && prev < vocab) h = ((long long)prev * mul_prev + (long long)token * mul_cur) % buckets;
        pair_row = pair + h * hidden;
    }
    const T* pos_row = nullptr;
    if (pos_table && live) {
        if (p >= 0 && p < n_positions) pos_row = pos_table + (int64_t)p * hidden;
        else if (threadIdx.x == 0) atomicOr(err, SS_ERR_TOKEN_RANGE);
    }
    const T* tok_row = table + (int64_t)token * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = to_float(tok_row[i]) * scale;
        if (pair_row) v += to_float(pair_row[i]);
        if (pos_row) v += to_float(pos_row[i]);
        for (int c = 0; c < copies; ++c) dst[(int64_t)c * hidden + i] = v;
    }
}

extern "C" int ss_embed_sum(const int32_t* tokens, const int32_t* positions, const void* table, const void* pair,
                            const void* pos_table, float* out, int32_t* last_token, const int32_t* q_start,
                            const int32_t* seq_lens, const int32_t* slots, int R, int n_rows, int hidden, int vocab, int copies,
                            int buckets, long long mul_prev, long long mul_cur, int n_positions, int n_slots, float scale,
                            int dtype, int* err, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (dtype == SS_BF16)
        ss_launch(embed_sum_kernel<bf16>, dim3(n_rows), dim3(128), 0, stream, tokens, positions, (const bf16*)table,
                  (const bf16*)pair, (const bf16*)pos_table, out, last_token, q_start, seq_lens, slots, R, hidden, vocab, copies,
                  buckets, mul_prev, mul_cur, n_positions, n_slots, scale, err);
    else
        ss_launch(embed_sum_kernel<float>, dim3(n_rows), dim3(128), 0, stream, tokens, positions, (const float*)table,
                  (const float*)pair, (const float*)pos_table, out, last_token, q_start, seq_lens, slots, R, hidden, vocab,
                  copies, buckets, mul_prev, mul_cur, n_positions, n_slots, scale, err);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- the matrix-memory cell
//
// Per head, with raw gate values a_t (input) and b_t (forget), biases included:
//   i_t = cap tanh(a_t / cap),  f_t = log sigmoid(cap tanh(b_t / cap)),  m_t = max(f_t + m_{t-1}, i_t),
//   keep_t = exp(f_t + m_{t-1} - m_t),  take_t = exp(i_t - m_t),
//   S_t = keep_t S_{t-1} + take_t k_t v_t^T   [D x V],   n_t = keep_t n_{t-1} + take_t k_t.
// The kernel treats n as one more column of S (the column of a value that is always 1) and writes, per token,
// the numerators S_t^T q_t [V], the scalar n_t . q_t and m_t; the norm kernel behind it divides.
// State: memory [slot][H][V + 1][D] float32 (column-major, column V is n), peak [slot][H] (m, starts at 0).
// A block: one request, one head, MC_COLS columns; a column is shared by MC_LANES lanes, lane j holding rows
// d = i * MC_LANES + j.  Tokens are staged MC_TOKENS at a time in shared memory as float32.
#define MC_LANES 8
#define MC_COLS 16
#define MC_TOKENS 16
#define MC_THREADS (MC_LANES * MC_COLS)

template <typename T, int DPL>
__global__ void __launch_bounds__(MC_THREADS)
matrix_cell_kernel(const T* __restrict__ qkv, int64_t stride, const float* __restrict__ gates, int64_t gate_stride,
                   const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap, float q_scale,
                   float* __restrict__ memory, float* __restrict__ peak, float* __restrict__ num, float* __restrict__ nq,
                   float* __restrict__ peaks_out, const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                   const int32_t* __restrict__ slots, int H, int D, int V, int n_slots, int* err) {
    pdl_wait();
    extern __shared__ float cell_smem[];
    float* qs = cell_smem;                       // [MC_TOKENS][D]
    float* ks = qs + MC_TOKENS * D;              // [MC_TOKENS][D]
    float* vs = ks + MC_TOKENS * D;              // [MC_TOKENS][MC_COLS]
    float* gi = vs + MC_TOKENS * MC_COLS;        // [MC_TOKENS] each: i, f, keep, take, m
    float* gf = gi + MC_TOKENS;
    float* keep_s = gf + MC_TOKENS;
    float* take_s = keep_s + MC_TOKENS;
    float* m_s = take_s + MC_TOKENS;

    const int tid = threadIdx.x, j = tid & (MC_LANES - 1), col_here = tid / MC_LANES;
    const int h = blockIdx.y, r = blockIdx.z;
    const int col = blockIdx.x * MC_COLS + col_here;  // V: the column of n
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (tid == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    const bool col_ok = col <= V;
    float* mem = memory + (((int64_t)slot * H + h) * (V + 1) + (col_ok ? col : 0)) * D;
    float S[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = i * MC_LANES + j;
        S[i] = (col_ok && d < D) ? mem[d] : 0.f;
    }
    float m_prev = peak[(int64_t)slot * H + h];
    const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;

    for (int t0 = 0; t0 < q_len; t0 += MC_TOKENS) {
        const int n = min(MC_TOKENS, q_len - t0);
        __syncthreads();  // the batch before has been used
        for (int idx = tid; idx < n * D; idx += MC_THREADS) {
            const int t = idx / D, d = idx - t * D;
            const T* src = qkv + (int64_t)(q0 + t0 + t) * stride + (int64_t)h * D + d;
            qs[t * D + d] = to_float(src[0]) * q_scale;
            ks[t * D + d] = to_float(src[(int64_t)H * D]);
        }
        for (int idx = tid; idx < n * MC_COLS; idx += MC_THREADS) {
            const int t = idx / MC_COLS, c = idx - t * MC_COLS, gc = blockIdx.x * MC_COLS + c;
            vs[idx] = gc < V ? to_float(qkv[(int64_t)(q0 + t0 + t) * stride + 2 * (int64_t)H * D + (int64_t)h * V + gc])
                             : (gc == V ? 1.f : 0.f);
        }
        if (tid < n) {
            const float* g = gates + (int64_t)(q0 + t0 + tid) * gate_stride;
            gi[tid] = cap * tanhf((g[h] + bi) / cap);
            gf[tid] = log_sigmoid(cap * tanhf((g[H + h] + bf) / cap));
        }
        __syncthreads();
        if (tid == 0) {  // the running maximum is a chain; everything else of the gates is not
            float m = m_prev;
            for (int t = 0; t < n; ++t) {
                const float carried = gf[t] + m;
                const float m_new = fmaxf(carried, gi[t]);
                keep_s[t] = expf(carried - m_new);
                take_s[t] = expf(gi[t] - m_new);
                m_s[t] = m_new;
                m = m_new;
            }
        }
        __syncthreads();
        m_prev = m_s[n - 1];
        if (blockIdx.x == 0 && tid < n) peaks_out[(int64_t)(q0 + t0 + tid) * H + h] = m_s[tid];
        for (int t = 0; t < n; ++t) {
            const float keep = keep_s[t];
            const float tv = take_s[t] * vs[t * MC_COLS + col_here];
            const float* kt = ks + t * D;
            const float* qt = qs + t * D;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = i * MC_LANES + j;
                if (d < D) {
                    S[i] = fmaf(keep, S[i], kt[d] * tv);
                    acc = fmaf(S[i], qt[d], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (j == 0 && col_ok) {
                const int64_t row = q0 + t0 + t;
                if (col < V) num[row * H * V + (int64_t)h * V + col] = acc;
                else nq[row * H + h] = acc;
            }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = i * MC_LANES + j;
            if (d < D) mem[d] = S[i];
        }
    }
    if (blockIdx.x == 0 && tid == 0) peak[(int64_t)slot * H + h] = m_prev;
}

template <typename T>
static int launch_matrix_cell(const void* qkv, int64_t stride, const float* gates, int64_t gate_stride, const float* bias_i,
                              const float* bias_f, float cap, float q_scale, float* memory, float* peak, float* num, float* nq,
                              float* peaks_out, const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int R,
                              int H, int D, int V, int n_slots, int* err, cudaStream_t stream) {
    const dim3 grid((V + 1 + MC_COLS - 1) / MC_COLS, H, R);
    const int smem = (2 * MC_TOKENS * D + MC_TOKENS * MC_COLS + 5 * MC_TOKENS) * 4;
#define CELL_LAUNCH(DPL)                                                                                                   \
    ss_launch(matrix_cell_kernel<T, DPL>, grid, dim3(MC_THREADS), smem, stream, (const T*)qkv, stride, gates, gate_stride,  \
              bias_i, bias_f, cap, q_scale, memory, peak, num, nq, peaks_out, q_start, seq_lens, slots, H, D, V, n_slots, err)
    if (D <= 8 * MC_LANES) CELL_LAUNCH(8);
    else if (D <= 16 * MC_LANES) CELL_LAUNCH(16);
    else CELL_LAUNCH(32);
#undef CELL_LAUNCH
    return SS_LAUNCH_CHECK();
}

extern "C" int ss_matrix_cell(const void* qkv, int64_t stride, const float* gates, int64_t gate_stride, const float* bias_i,
                              const float* bias_f, float cap, float q_scale, float* memory, float* peak, float* num, float* nq,
                              float* peaks_out, const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int R,
                              int H, int D, int V, int n_slots, int dtype, int* err, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (D < 1 || D > 32 * MC_LANES || V < 1 || !(cap > 0.f)) return (int)cudaErrorInvalidValue;
    if (dtype == SS_BF16)
        return launch_matrix_cell<bf16>(qkv, stride, gates, gate_stride, bias_i, bias_f, cap, q_scale, memory, peak, num, nq,
                                        peaks_out, q_start, seq_lens, slots, R, H, D, V, n_slots, err, stream);
    return launch_matrix_cell<float>(qkv, stride, gates, gate_stride, bias_i, bias_f, cap, q_scale, memory, peak, num, nq,
                                     peaks_out, q_start, seq_lens, slots, R, H, D, V, n_slots, err, stream);
}

// The cell's output: o = num / (max(|n . q|, exp(-m)) + 1e-6), each head divided by its root mean square, times a
// weight over all heads' elements, times sigmoid(gate).  A warp per (row, head); gate: [rows][gate_stride] in T.
template <typename T>
__global__ void __launch_bounds__(128)
cell_output_kernel(const float* __restrict__ num, const float* __restrict__ nq, const float* __restrict__ peaks,
                   const float* __restrict__ weight, const T* __restrict__ gate, int64_t gate_stride, T* __restrict__ out,
                   int n_rows, int H, int V, float eps) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t pair = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (pair >= (int64_t)n_rows * H) return;
    const int64_t row = pair / H;
    const int h = (int)(pair - row * H);
    const float den = fmaxf(fabsf(nq[pair]), expf(-peaks[pair])) + 1e-6f;
    const float* src = num + pair * V;
    float ss = 0.f;
    for (int v = lane; v < V; v += 32) {
        const float o = src[v] / den;
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + eps);
    for (int v = lane; v < V; v += 32) {
        const float o = src[v] / den * inv * weight[h * V + v];
        const float g = to_float(gate[row * gate_stride + (int64_t)h * V + v]);
        out[pair * V + v] = from_float<T>(o * sigmoid_exact(g));
    }
}

extern "C" int ss_cell_output(const float* num, const float* nq, const float* peaks, const float* weight, const void* gate,
                              int64_t gate_stride, void* out, int n_rows, int H, int V, float eps, int dtype,
                              cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const dim3 grid((unsigned)(((int64_t)n_rows * H + 3) / 4));
    if (dtype == SS_BF16)
        ss_launch(cell_output_kernel<bf16>, grid, dim3(128), 0, stream, num, nq, peaks, weight, (const bf16*)gate, gate_stride,
                  (bf16*)out, n_rows, H, V, eps);
    else
        ss_launch(cell_output_kernel<float>, grid, dim3(128), 0, stream, num, nq, peaks, weight, (const float*)gate,
                  gate_stride, (float*)out, n_rows, H, V, eps);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- gated recurrence per channel
//
// proj row: [z: W | u: W | g: W]; `bias` (float32 [2 W] or null) is added to z and u in float32.  z' = sigmoid(z);
// candidate = u + 1/2 where u >= 0, sigmoid(u) below; S <- (1 - z') S + z' candidate; out = S silu(g).  State [slot][W] float32.
// A thread per (request, channel) walks the request's rows in order.
template <typename T>
__global__ void __launch_bounds__(128)
gated_recurrence_kernel(const T* __restrict__ proj, int64_t stride, const float* __restrict__ bias,
                        float* __restrict__ state, T* __restrict__ out,
                        const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                        const int32_t* __restrict__ slots, int W, int n_slots, int* err) {
    pdl_wait();
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    if (c >= W) return;
    float S = state[(int64_t)slot * W + c];
    const float bz = bias ? bias[c] : 0.f, bu = bias ? bias[W + c] : 0.f;
    const T* src = proj + (int64_t)q0 * stride + c;
    constexpr int AHEAD = 4;  // rows whose loads are in flight while one is used
    float zb[AHEAD], ub[AHEAD], gb[AHEAD];
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
        const bool ok = a < q_len;
        zb[a] = ok ? to_float(src[(int64_t)a * stride]) : 0.f;
        ub[a] = ok ? to_float(src[(int64_t)a * stride + W]) : 0.f;
        gb[a] = ok ? to_float(src[(int64_t)a * stride + 2 * W]) : 0.f;
    }
    for (int t0 = 0; t0 < q_len; t0 += AHEAD) {
#pragma unroll
        for (int a = 0; a < AHEAD; ++a) {
            const int t = t0 + a;
            if (t >= q_len) break;
            const float z = sigmoid_exact(zb[a] + bz), u = ub[a] + bu, g = gb[a];
            const int nx = t + AHEAD;
            if (nx < q_len) {
                zb[a] = to_float(src[(int64_t)nx * stride]);
                ub[a] = to_float(src[(int64_t)nx * stride + W]);
                gb[a] = to_float(src[(int64_t)nx * stride + 2 * W]);
            }
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_exact(u);
            S = fmaf(z, cand, (1.0f - z) * S);
            out[(int64_t)(q0 + t) * W + c] = from_float<T>(S * (g / (1.0f + expf(-g))));
        }
    }
    state[(int64_t)slot * W + c] = S;
}

extern "C" int ss_gated_recurrence(const void* proj, int64_t stride, const float* bias, float* state, void* out,
                                   const int32_t* q_start,
                                   const int32_t* seq_lens, const int32_t* slots, int R, int W, int n_slots, int dtype, int* err,
                                   cudaStream_t stream) {
    if (R <= 0 || W <= 0) return 0;
    const dim3 grid((W + 127) / 128, R);
    if (dtype == SS_BF16)
        ss_launch(gated_recurrence_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)proj, stride, bias, state,
                  (bf16*)out, q_start, seq_lens, slots, W, n_slots, err);
    else
        ss_launch(gated_recurrence_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, stride, bias, state,
                  (float*)out, q_start, seq_lens, slots, W, n_slots, err);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- xIELU
//
// z > 0: a z^2 + z / 2;  z <= 0: b (exp(z) - 1 - z) + z / 2, with a = softplus(p) and b = 1/2 + softplus(q) formed
// on the host.  In place or into `out`.
template <typename T>
__global__ void __launch_bounds__(256)
xielu_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t n, float a, float b) {
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float z = to_float(in[i]);
        const float y = z > 0.f ? fmaf(a * z, z, 0.5f * z) : fmaf(b, expm1f(z) - z, 0.5f * z);
        out[i] = from_float<T>(y);
    }
}

// bfloat16, eight elements a thread (n a multiple of 8, both pointers on 16-byte boundaries)
__global__ void __launch_bounds__(256)
xielu_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int64_t n8, float a, float b) {
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 raw = in[i];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float z0 = __uint_as_float(w[e] << 16), z1 = __uint_as_float(w[e] & 0xffff0000u);
            const float y0 = z0 > 0.f ? fmaf(a * z0, z0, 0.5f * z0) : fmaf(b, expm1f(z0) - z0, 0.5f * z0);
            const float y1 = z1 > 0.f ? fmaf(a * z1, z1, 0.5f * z1) : fmaf(b, expm1f(z1) - z1, 0.5f * z1);
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(y0, y1);
            o[e] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

extern "C" int ss_xielu(const void* in, void* out, int64_t n, float a, float b, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == SS_BF16 && n % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const int blocks = (int)((n / 8 + 255) / 256 < 148 * 16 ? (n / 8 + 255) / 256 : 148 * 16);
        ss_launch(xielu_bf16x8_kernel, dim3(blocks), dim3(256), 0, stream, (const uint4*)in, (uint4*)out, n / 8, a, b);
        return SS_LAUNCH_CHECK();
    }
    const int blocks = (int)((n + 255) / 256 < 148 * 32 ? (n + 255) / 256 : 148 * 32);
    if (dtype == SS_BF16)
        ss_launch(xielu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)in, (bf16*)out, n, a, b);
    else
        ss_launch(xielu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)in, (float*)out, n, a, b);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- latent attention: latents, rotation, page write
//
// A row of the down projection: [query latent: QR | key/value latent: KR | shared key part: RD | ...].
//   cq = rmsnorm(query latent) * wq                                    -> cq_out [rows][QR]
//   c  = rmsnorm(key/value latent) * wkv;  s = rotate(shared key part) (pairs (i, i + RD / 2), angle p * freq[i],
//        cosines and sines times mscale)
//   key page row   [s: RD | c: KR | zeros to DP],  value page row [c: KR | zeros to DP]   at slot_mapping[row]
// With KR = 0 (a layer that reads another layer's pages) only cq is formed.  A block per row.
template <typename T>
__global__ void __launch_bounds__(128)
latent_rows_kernel(const T* __restrict__ down, int64_t stride, const int32_t* __restrict__ positions,
                   const int32_t* __restrict__ slot_mapping, const float* __restrict__ wq, const float* __restrict__ wkv,
                   const float* __restrict__ freq, float mscale, T* __restrict__ cq_out, T* __restrict__ kv, int QR, int KR,
                   int RD, int DP, int page_size, int64_t num_pages, float eps, int* err) {
    pdl_wait();
    __shared__ float scratch[33];
    const int row = blockIdx.x, tid = threadIdx.x;
    const T* src = down + (int64_t)row * stride;
    float ss = 0.f;
    for (int i = tid; i < QR; i += blockDim.x) {
        const float v = to_float(src[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv_q = 1.0f / sqrtf(ss / (float)QR + eps);
    for (int i = tid; i < QR; i += blockDim.x) cq_out[(int64_t)row * QR + i] = from_float<T>(to_float(src[i]) * inv_q * wq[i]);
    if (KR <= 0 || kv == nullptr) return;
    const int slot = slot_mapping[row];
    if (slot < 0) return;  // a padding row of a captured step
    const int64_t page = slot / page_size;
    if (page >= num_pages) {
        if (tid == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    float s2 = 0.f;
    for (int i = tid; i < KR; i += blockDim.x) {
        const float v = to_float(src[QR + i]);
        s2 = fmaf(v, v, s2);
    }
    s2 = block_sum(s2, scratch);
    const float inv_c = 1.0f / sqrtf(s2 / (float)KR + eps);
    const int off = slot - (int)page * page_size;
    T* krow = kv + (((page * 2 + 0) * page_size) + off) * (int64_t)DP;
    T* vrow = kv + (((page * 2 + 1) * page_size) + off) * (int64_t)DP;
    const float p = (float)positions[row];
    const int half = RD / 2;
    for (int i = tid; i < half; i += blockDim.x) {
        const float a = to_float(src[QR + KR + i]), b = to_float(src[QR + KR + half + i]);
        float c = 1.f, s = 0.f;
        if (freq) {
            const float angle = p * freq[i];
            c = cosf(angle) * mscale;
            s = sinf(angle) * mscale;
        }
        krow[i] = from_float<T>(a * c - b * s);
        krow[half + i] = from_float<T>(b * c + a * s);
    }
    for (int i = tid; i < KR; i += blockDim.x) {
        const T c = from_float<T>(to_float(src[QR + i]) * inv_c * wkv[i]);
        krow[RD + i] = c;
        vrow[i] = c;
    }
    for (int i = RD + KR + tid; i < DP; i += blockDim.x) krow[i] = from_float<T>(0.f);
    for (int i = KR + tid; i < DP; i += blockDim.x) vrow[i] = from_float<T>(0.f);
}

extern "C" int ss_latent_rows(const void* down, int64_t stride, const int32_t* positions, const int32_t* slot_mapping,
                              const float* wq, const float* wkv, const float* freq, float mscale, void* cq_out, void* kv,
                              int n_rows, int QR, int KR, int RD, int DP, int page_size, int64_t num_pages, float eps, int dtype,
                              int* err, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (RD % 2 || (KR > 0 && RD + KR > DP)) return (int)cudaErrorInvalidValue;
    if (dtype == SS_BF16)
        ss_launch(latent_rows_kernel<bf16>, dim3(n_rows), dim3(128), 0, stream, (const bf16*)down, stride, positions,
                  slot_mapping, wq, wkv, freq, mscale, (bf16*)cq_out, (bf16*)kv, QR, KR, RD, DP, page_size, num_pages, eps, err);
    else
        ss_launch(latent_rows_kernel<float>, dim3(n_rows), dim3(128), 0, stream, (const float*)down, stride, positions,
                  slot_mapping, wq, wkv, freq, mscale, (float*)cq_out, (float*)kv, QR, KR, RD, DP, page_size, num_pages, eps,
                  err);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- a product per head
//
// out[row][h][o] = f(row, h) * sum_i x[row][h][i] * w[h][i][o]   for o < O, with x rows x_stride apart and heads
// x_head apart, out rows out_stride apart and heads out_head apart; float32 accumulation in the order of i.
// `turn` > 0: out[row][h][0 .. turn) takes the `turn` elements x[row][h][I .. I + turn) rotated by the row's position
// (pairs (i, i + turn / 2)); the product's outputs start at column `turn`, and columns from turn + O to `pad_to`
// are zeroed.  `scale_col` >= 0: f = sigmoid(gates[row][scale_col + h]).
// A block: HP_ROWS rows of one head; threads over o.
#define HP_ROWS 8

template <typename T>
__global__ void __launch_bounds__(128)
head_product_kernel(const T* __restrict__ x, int64_t x_stride, int x_head, const T* __restrict__ w, T* __restrict__ out,
                    int64_t out_stride, int out_head, int n_rows, int I, int O, int turn, int pad_to,
                    const int32_t* __restrict__ positions, const float* __restrict__ freq, float mscale,
                    const T* __restrict__ gates, int64_t gate_stride, int scale_col) {
    pdl_wait();
    extern __shared__ float hp_smem[];  // [HP_ROWS][I + turn]
    const int h = blockIdx.y, row0 = blockIdx.x * HP_ROWS, tid = threadIdx.x;
    const int rows = min(HP_ROWS, n_rows - row0);
    const int width = I + turn;
    for (int idx = tid; idx < HP_ROWS * width; idx += blockDim.x) {
        const int rr = idx / width, i = idx - rr * width;
        hp_smem[idx] = rr < rows ? to_float(x[(int64_t)(row0 + rr) * x_stride + (int64_t)h * x_head + i]) : 0.f;
    }
    __syncthreads();
    const T* wh = w + (int64_t)h * I * O;
    for (int o = tid; o < O; o += blockDim.x) {
        float acc[HP_ROWS];
#pragma unroll
        for (int rr = 0; rr < HP_ROWS; ++rr) acc[rr] = 0.f;
        for (int i = 0; i < I; ++i) {
            const float wv = to_float(wh[(int64_t)i * O + o]);
#pragma unroll
            for (int rr = 0; rr < HP_ROWS; ++rr) acc[rr] = fmaf(hp_smem[rr * width + i], wv, acc[rr]);
        }
#pragma unroll
        for (int rr = 0; rr < HP_ROWS; ++rr) {
            if (rr >= rows) break;
            float f = 1.f;
            if (scale_col >= 0) f = sigmoid_exact(to_float(gates[(int64_t)(row0 + rr) * gate_stride + scale_col + h]));
            out[(int64_t)(row0 + rr) * out_stride + (int64_t)h * out_head + turn + o] = from_float<T>(acc[rr] * f);
        }
    }
    const int half = turn / 2;
    for (int idx = tid; idx < rows * half; idx += blockDim.x) {
        const int rr = idx / half, i = idx - rr * half;
        const float a = hp_smem[rr * width + I + i], b = hp_smem[rr * width + I + half + i];
        float c = 1.f, s = 0.f;
        if (freq) {
            const float angle = (float)positions[row0 + rr] * freq[i];
            c = cosf(angle) * mscale;
            s = sinf(angle) * mscale;
        }
        T* dst = out + (int64_t)(row0 + rr) * out_stride + (int64_t)h * out_head;
        dst[i] = from_float<T>(a * c - b * s);
        dst[half + i] = from_float<T>(b * c + a * s);
    }
    for (int idx = tid; idx < rows * (pad_to - turn - O); idx += blockDim.x) {
        const int span = pad_to - turn - O;
        const int rr = idx / span, i = idx - rr * span;
        out[(int64_t)(row0 + rr) * out_stride + (int64_t)h * out_head + turn + O + i] = from_float<T>(0.f);
    }
}

extern "C" int ss_head_product(const void* x, int64_t x_stride, int x_head, const void* w, void* out, int64_t out_stride,
                               int out_head, int n_rows, int H, int I, int O, int turn, int pad_to, const int32_t* positions,
                               const float* freq, float mscale, const void* gates, int64_t gate_stride, int scale_col, int dtype,
                               cudaStream_t stream) {
    if (n_rows <= 0 || H <= 0) return 0;
    if (turn % 2 || pad_to < turn + O) return (int)cudaErrorInvalidValue;
    const dim3 grid((n_rows + HP_ROWS - 1) / HP_ROWS, H);
    const int smem = HP_ROWS * (I + turn) * 4;
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (dtype == SS_BF16)
        ss_launch(head_product_kernel<bf16>, grid, dim3(128), smem, stream, (const bf16*)x, x_stride, x_head, (const bf16*)w,
                  (bf16*)out, out_stride, out_head, n_rows, I, O, turn, pad_to, positions, freq, mscale, (const bf16*)gates,
                  gate_stride, scale_col);
    else
        ss_launch(head_product_kernel<float>, grid, dim3(128), smem, stream, (const float*)x, x_stride, x_head, (const float*)w,
                  (float*)out, out_stride, out_head, n_rows, I, O, turn, pad_to, positions, freq, mscale, (const float*)gates,
                  gate_stride, scale_col);
    return SS_LAUNCH_CHECK();
}

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
//
// A block: one request, one head, MC_WARPS * 4 * CPT columns.  A compute warp holds four groups of CPT columns; a group
// is shared by MC_LANES lanes, lane j holding rows d = i * 4 MC_LANES + 4 j + (0 .. 3), i < NI, of each of its columns
// in registers (a lane reads q and k as 16-byte words that neighbouring lanes continue).  Three more warps stage the
// next MC_TOKENS tokens as float32 in the other half of shared memory (one q, scaled; one k; one the block's values
// and the gates with their chain m) while the compute warps walk the staged ones; rows past the last token
// are staged as k = q = 0 with keep = 1 and take = 0, so that a group of MC_GROUP tokens is always walked whole.  The
// dot products of a group of tokens are reduced together: a lane hands half of its columns' partial sums to its
// partner at each step.
#define MC_LANES 8
#define MC_TOKENS 32  // a lane of the staging warp a token
#define MC_GROUP 4
#define MC_WARPS 4
#define MC_THREADS ((MC_WARPS + 3) * 32)
static_assert(MC_TOKENS == 32 && MC_TOKENS % MC_GROUP == 0, "the gates of a batch are one warp wide");

// 16 bytes of T as floats
__device__ __forceinline__ void unpack16(const uint4& raw, float (&v)[8], bf16) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        v[2 * e] = __uint_as_float(w[e] << 16);
        v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
}
__device__ __forceinline__ void unpack16(const uint4& raw, float (&v)[4], float) {
    v[0] = __uint_as_float(raw.x); v[1] = __uint_as_float(raw.y); v[2] = __uint_as_float(raw.z); v[3] = __uint_as_float(raw.w);
}

// The sum over a group's 8 lanes of CPT values each; lane j ends with the sum of column `column_of_lane<CPT>(j)`.
template <int CPT> __device__ __forceinline__ int column_of_lane(int j) {
    return CPT == 4 ? ((j >> 2) & 1) * 2 + ((j >> 1) & 1) : (j >> 2) & 1;
}
template <int CPT> __device__ __forceinline__ float sum_columns(const float (&a)[CPT], int j) {
    float x;
    const bool up = j & 4;
    if constexpr (CPT == 4) {
        float x0 = up ? a[2] : a[0], x1 = up ? a[3] : a[1];
        x0 += __shfl_xor_sync(0xffffffffu, up ? a[0] : a[2], 4);
        x1 += __shfl_xor_sync(0xffffffffu, up ? a[1] : a[3], 4);
        const bool mid = j & 2;
        x = mid ? x1 : x0;
        x += __shfl_xor_sync(0xffffffffu, mid ? x0 : x1, 2);
    } else {
        static_assert(CPT == 2, "two or four columns a lane");
        x = up ? a[1] : a[0];
        x += __shfl_xor_sync(0xffffffffu, up ? a[0] : a[1], 4);
        x += __shfl_xor_sync(0xffffffffu, x, 2);
    }
    return x + __shfl_xor_sync(0xffffffffu, x, 1);
}

template <typename T, int NI, int CPT>
__global__ void __launch_bounds__(MC_THREADS)
matrix_cell_kernel(const T* __restrict__ qkv, int64_t stride, const float* __restrict__ gates, int64_t gate_stride,
                   const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap, float q_scale,
                   float* __restrict__ memory, float* __restrict__ peak, float* __restrict__ num, float* __restrict__ nq,
                   float* __restrict__ peaks_out, const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                   const int32_t* __restrict__ slots, int H, int D, int V, int n_slots, int wide_loads, int* err) {
    pdl_wait();
    constexpr int DP = NI * 4 * MC_LANES;            // rows as staged: zeros from D on
    constexpr int COLS = MC_WARPS * 4 * CPT;         // columns of a block
    constexpr int HALF = 2 * MC_TOKENS * DP + MC_TOKENS * COLS + 5 * MC_TOKENS;
    constexpr int VEC = 16 / (int)sizeof(T);
    extern __shared__ __align__(16) float cell_smem[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, r = blockIdx.z;
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (tid == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    const int n_batches = (q_len + MC_TOKENS - 1) / MC_TOKENS;
    const bool stager = warp >= MC_WARPS, stages_gates = warp == MC_WARPS + 2;

    // ---- the staging warps: one for q, one for k, one for the values and the gates
    float m_prev = stages_gates ? peak[(int64_t)slot * H + h] : 0.f;
    const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
    auto stage = [&](int batch) {
        float* half = cell_smem + (batch & 1) * HALF;
        float* vs = half + 2 * MC_TOKENS * DP;     // [MC_TOKENS][COLS], behind q and k [MC_TOKENS][DP] each
        float* gi = vs + MC_TOKENS * COLS;         // [MC_TOKENS] each: i, f, keep, take, m
        float* gf = gi + MC_TOKENS;
        float* keep_s = gf + MC_TOKENS;
        float* take_s = keep_s + MC_TOKENS;
        float* m_s = take_s + MC_TOKENS;
        const int t0 = batch * MC_TOKENS, n = min(MC_TOKENS, q_len - t0);
        const T* base = qkv + (int64_t)(q0 + t0) * stride;
        if (!stages_gates) {
            const bool is_k = warp == MC_WARPS + 1;
            float* dst = half + (is_k ? MC_TOKENS * DP : 0);
            const T* rows = base + (is_k ? (int64_t)H * D : 0) + (int64_t)h * D;
            const float factor = is_k ? 1.f : q_scale;
            if (wide_loads) {
                constexpr int PER_ROW = DP / VEC;
#pragma unroll 8
                for (int idx = lane; idx < MC_TOKENS * PER_ROW; idx += 32) {
                    const int t = idx / PER_ROW, d = (idx - t * PER_ROW) * VEC;
                    float v[VEC];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) v[e] = 0.f;
                    if (t < n && d < D)  // D is a multiple of VEC here
                        unpack16(*reinterpret_cast<const uint4*>(rows + (int64_t)t * stride + d), v, T());
#pragma unroll
                    for (int e = 0; e < VEC; e += 4)
                        *reinterpret_cast<float4*>(dst + t * DP + d + e) =
                            make_float4(v[e] * factor, v[e + 1] * factor, v[e + 2] * factor, v[e + 3] * factor);
                }
            } else {
#pragma unroll 8
                for (int idx = lane; idx < MC_TOKENS * DP; idx += 32) {
                    const int t = idx / DP, d = idx - t * DP;
                    dst[idx] = (t < n && d < D) ? to_float(rows[(int64_t)t * stride + d]) * factor : 0.f;
                }
            }
            return;
        }
        float a = 0.f, b = 0.f;  // a lane a token
        if (lane < n) {
            const float* g = gates + (int64_t)(q0 + t0 + lane) * gate_stride;
            a = cap * tanhf((g[h] + bi) / cap);
            b = log_sigmoid(cap * tanhf((g[H + h] + bf) / cap));
        }
        gi[lane] = a;
        gf[lane] = b;
        const T* vals = base + 2 * (int64_t)H * D + (int64_t)h * V;
        const int c0 = blockIdx.x * COLS;
        if (wide_loads) {
            constexpr int PER_ROW = COLS / VEC;
#pragma unroll
            for (int idx = lane; idx < MC_TOKENS * PER_ROW; idx += 32) {
                const int t = idx / PER_ROW, c = (idx - t * PER_ROW) * VEC;
                float v[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) v[e] = 0.f;
                if (t < n && c0 + c < V)  // V is a multiple of VEC here
                    unpack16(*reinterpret_cast<const uint4*>(vals + (int64_t)t * stride + c0 + c), v, T());
                if (c0 + c == V) v[0] = 1.f;
#pragma unroll
                for (int e = 0; e < VEC; e += 4)
                    *reinterpret_cast<float4*>(vs + t * COLS + c + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
            }
        } else {
#pragma unroll 8
            for (int idx = lane; idx < MC_TOKENS * COLS; idx += 32) {
                const int t = idx / COLS, gc = c0 + idx - t * COLS;
                float v = gc == V ? 1.f : 0.f;
                if (t < n && gc < V) v = to_float(vals[(int64_t)t * stride + gc]);
                vs[idx] = v;
            }
        }
        __syncwarp();
        if (lane == 0) {  // the running maximum is a chain; everything else of the gates is not
            float m = m_prev;
            for (int t = 0; t < n; ++t) {
                m = fmaxf(gf[t] + m, gi[t]);
                m_s[t] = m;
            }
        }
        __syncwarp();
        float keep = 1.f, take = 0.f;
        if (lane < n) {
            const float before = lane ? m_s[lane - 1] : m_prev, now = m_s[lane];
            keep = expf(b + before - now);
            take = expf(a - now);
            if (blockIdx.x == 0) peaks_out[(int64_t)(q0 + t0 + lane) * H + h] = now;
        }
        keep_s[lane] = keep;
        take_s[lane] = take;
        m_prev = m_s[n - 1];
    };

    // ---- the compute warps
    const int j = lane & (MC_LANES - 1), group = warp * 4 + (lane >> 3);
    const int col0 = blockIdx.x * COLS + group * CPT;  // this lane's columns: col0 .. col0 + CPT - 1; V is the column of n
    float S[CPT][NI * 4];
    const bool rows_of_4 = (D & 3) == 0;
    if (!stager) {
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const bool col_ok = col0 + c <= V;
            const float* mem = memory + (((int64_t)slot * H + h) * (V + 1) + (col_ok ? col0 + c : 0)) * D;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int d = i * 4 * MC_LANES + 4 * j;
                if (col_ok && rows_of_4 && d < D) {
                    const float4 w = *reinterpret_cast<const float4*>(mem + d);
                    S[c][4 * i] = w.x; S[c][4 * i + 1] = w.y; S[c][4 * i + 2] = w.z; S[c][4 * i + 3] = w.w;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[c][4 * i + e] = (col_ok && d + e < D) ? mem[d + e] : 0.f;
                }
            }
        }
    }

    if (stager) stage(0);
    __syncthreads();
    for (int batch = 0; batch < n_batches; ++batch) {
        if (stager) {
            if (batch + 1 < n_batches) stage(batch + 1);
        } else {
            const float* half = cell_smem + (batch & 1) * HALF;
            const float4* qs4 = reinterpret_cast<const float4*>(half);
            const float4* ks4 = reinterpret_cast<const float4*>(half + MC_TOKENS * DP);
            const float* vs = half + 2 * MC_TOKENS * DP;
            const float* keep_s = vs + MC_TOKENS * COLS + 2 * MC_TOKENS;
            const float* take_s = keep_s + MC_TOKENS;
            const int t0 = batch * MC_TOKENS, n = min(MC_TOKENS, q_len - t0);
            for (int tg = 0; tg < n; tg += MC_GROUP) {
                float acc[MC_GROUP][CPT];
#pragma unroll
                for (int g = 0; g < MC_GROUP; ++g) {
                    const int t = tg + g;
                    const float keep = keep_s[t], take = take_s[t];
                    float tv[CPT];
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        tv[c] = take * vs[t * COLS + group * CPT + c];
                        acc[g][c] = 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        const float4 k4 = ks4[t * (DP / 4) + i * MC_LANES + j], q4 = qs4[t * (DP / 4) + i * MC_LANES + j];
                        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                        for (int c = 0; c < CPT; ++c) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                S[c][4 * i + e] = fmaf(keep, S[c][4 * i + e], kk[e] * tv[c]);
                                acc[g][c] = fmaf(S[c][4 * i + e], qq[e], acc[g][c]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int g = 0; g < MC_GROUP; ++g) {
                    const float total = sum_columns<CPT>(acc[g], j);
                    const int col = col0 + column_of_lane<CPT>(j);
                    const bool writer = CPT == 4 ? (j & 1) == 0 : (j & 3) == 0;
                    if (writer && tg + g < n && col <= V) {
                        const int64_t row = q0 + t0 + tg + g;
                        if (col < V) num[row * H * V + (int64_t)h * V + col] = total;
                        else nq[row * H + h] = total;
                    }
                }
            }
        }
        __syncthreads();
    }

    if (stager) {
        if (stages_gates && blockIdx.x == 0 && lane == 0) peak[(int64_t)slot * H + h] = m_prev;
        return;
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        if (col0 + c > V) continue;
        float* mem = memory + (((int64_t)slot * H + h) * (V + 1) + col0 + c) * D;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = i * 4 * MC_LANES + 4 * j;
            if (rows_of_4 && d < D) {
                *reinterpret_cast<float4*>(mem + d) = make_float4(S[c][4 * i], S[c][4 * i + 1], S[c][4 * i + 2], S[c][4 * i + 3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (d + e < D) mem[d + e] = S[c][4 * i + e];
            }
        }
    }
}

template <typename T, int NI, int CPT>
static int launch_matrix_cell_as(const void* qkv, int64_t stride, const float* gates, int64_t gate_stride, const float* bias_i,
                                 const float* bias_f, float cap, float q_scale, float* memory, float* peak, float* num,
                                 float* nq, float* peaks_out, const int32_t* q_start, const int32_t* seq_lens,
                                 const int32_t* slots, int R, int H, int D, int V, int n_slots, int* err, cudaStream_t stream) {
    constexpr int COLS = MC_WARPS * 4 * CPT, VEC = 16 / (int)sizeof(T);
    constexpr int smem = 2 * (2 * MC_TOKENS * NI * 4 * MC_LANES + MC_TOKENS * COLS + 5 * MC_TOKENS) * 4;
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(matrix_cell_kernel<T, NI, CPT>, smem, opted)) return rc_smem;
    // rows of q, k and v are fetched 16 bytes at a time where every head's rows start on such a boundary
    const int wide = D % VEC == 0 && V % VEC == 0 && stride % VEC == 0 && ((uintptr_t)qkv & 15) == 0;
    const dim3 grid((V + 1 + COLS - 1) / COLS, H, R);
    ss_launch(matrix_cell_kernel<T, NI, CPT>, grid, dim3(MC_THREADS), smem, stream, (const T*)qkv, stride, gates, gate_stride,
              bias_i, bias_f, cap, q_scale, memory, peak, num, nq, peaks_out, q_start, seq_lens, slots, H, D, V, n_slots, wide,
              err);
    return SS_LAUNCH_CHECK();
}

template <typename T>
static int launch_matrix_cell(const void* qkv, int64_t stride, const float* gates, int64_t gate_stride, const float* bias_i,
                              const float* bias_f, float cap, float q_scale, float* memory, float* peak, float* num, float* nq,
                              float* peaks_out, const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int R,
                              int H, int D, int V, int n_slots, int* err, cudaStream_t stream) {
#define CELL_LAUNCH(NI, CPT)                                                                                                \
    return launch_matrix_cell_as<T, NI, CPT>(qkv, stride, gates, gate_stride, bias_i, bias_f, cap, q_scale, memory, peak, num, \
                                             nq, peaks_out, q_start, seq_lens, slots, R, H, D, V, n_slots, err, stream)
    const int rows = 4 * MC_LANES;  // rows of one step over a column's lanes
    if (D <= rows) CELL_LAUNCH(1, 2);
    if (D <= 2 * rows) CELL_LAUNCH(2, 2);
    if (D <= 3 * rows) CELL_LAUNCH(3, 2);
    if (D <= 4 * rows) CELL_LAUNCH(4, 2);
    if (D <= 6 * rows) CELL_LAUNCH(6, 2);
    CELL_LAUNCH(8, 2);
#undef CELL_LAUNCH
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

// The same recurrence over prompt portions, cut in time as well.  S_t = (1 - z_t) S_{t-1} + z_t c_t is linear in S, so a
// segment of tokens acts on the state it meets as S -> A S + B with A the product of its (1 - z_t) and B its result from
// zero.  A block: one request, 32 channels (the lanes) and GR_SEGS warps; a tile is GR_SEGS segments of GR_LEN tokens.
// Every warp loads its segment once (all loads in flight together, a tile ahead of their use) and forms (A, B); each thread then chains the
// segments' (A, B) in order from the state the tile met, which gives it the state in front of its own segment and the
// state behind the tile; then it walks its segment again from registers with the recurrence as written, and writes.
// Tokens past the request's end act as A = 1, B = 0.
#define GR_SEGS 16
#define GR_LEN 8

template <typename T>
__global__ void __launch_bounds__(GR_SEGS * 32)
gated_recurrence_portions_kernel(const T* __restrict__ proj, int64_t stride, const float* __restrict__ bias,
                                 float* __restrict__ state, T* __restrict__ out, const int32_t* __restrict__ q_start,
                                 const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ slots, int W, int n_slots,
                                 int* err) {
    pdl_wait();
    __shared__ float As[2][GR_SEGS][32], Bs[2][GR_SEGS][32];
    const int lane = threadIdx.x & 31, seg = threadIdx.x >> 5;
    const int r = blockIdx.y, c = blockIdx.x * 32 + lane;
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    const bool live = c < W;
    float S_tile = live ? state[(int64_t)slot * W + c] : 0.f;
    const float bz = (bias && live) ? bias[c] : 0.f, bu = (bias && live) ? bias[W + c] : 0.f;
    const T* src = proj + (int64_t)q0 * stride + (live ? c : 0);
    int parity = 0;
    float zr[GR_LEN], ur[GR_LEN], gr[GR_LEN];
    auto fetch = [&](int first, float (&z)[GR_LEN], float (&u)[GR_LEN], float (&g)[GR_LEN]) {
#pragma unroll
        for (int a = 0; a < GR_LEN; ++a) {
            const bool ok = live && first + a < q_len;
            const T* p = src + (int64_t)(first + a) * stride;
            z[a] = ok ? to_float(p[0]) : 0.f;
            u[a] = ok ? to_float(p[W]) : 0.f;
            g[a] = ok ? to_float(p[2 * W]) : 0.f;
        }
    };
    fetch(seg * GR_LEN, zr, ur, gr);
    for (int tile0 = 0; tile0 < q_len; tile0 += GR_SEGS * GR_LEN, parity ^= 1) {
        const int first = tile0 + seg * GR_LEN;
        float zn[GR_LEN], un[GR_LEN], gn[GR_LEN];  // the next tile's rows are fetched while this one is walked
        fetch(first + GR_SEGS * GR_LEN, zn, un, gn);
        float A = 1.f, B = 0.f;
#pragma unroll
        for (int a = 0; a < GR_LEN; ++a) {
            const bool ok = first + a < q_len;
            const float z = ok ? sigmoid_exact(zr[a] + bz) : 0.f, u = ur[a] + bu;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_exact(u);
            zr[a] = z;
            ur[a] = cand;
            A *= 1.0f - z;
            B = fmaf(z, cand, (1.0f - z) * B);
        }
        As[parity][seg][lane] = A;
        Bs[parity][seg][lane] = B;
        __syncthreads();  // one barrier a tile: the next tile writes the other pair of tables
        float S = S_tile, S_in = S_tile;
#pragma unroll
        for (int s = 0; s < GR_SEGS; ++s) {
            if (s == seg) S_in = S;
            S = fmaf(As[parity][s][lane], S, Bs[parity][s][lane]);
        }
        S_tile = S;
        S = S_in;
#pragma unroll
        for (int a = 0; a < GR_LEN; ++a) {
            if (!live || first + a >= q_len) break;
            S = fmaf(zr[a], ur[a], (1.0f - zr[a]) * S);
            const float g = gr[a];
            out[(int64_t)(q0 + first + a) * W + c] = from_float<T>(S * (g / (1.0f + expf(-g))));
        }
#pragma unroll
        for (int a = 0; a < GR_LEN; ++a) {
            zr[a] = zn[a];
            ur[a] = un[a];
            gr[a] = gn[a];
        }
    }
    if (live && seg == 0) state[(int64_t)slot * W + c] = S_tile;
}

extern "C" int ss_gated_recurrence(const void* proj, int64_t stride, const float* bias, float* state, void* out,
                                   const int32_t* q_start,
                                   const int32_t* seq_lens, const int32_t* slots, int R, int W, int n_slots, int dtype, int* err,
                                   cudaStream_t stream, int portions) {
    if (R <= 0 || W <= 0) return 0;
    if (portions) {  // some request brings more than a few tokens
        const dim3 tiles((W + 31) / 32, R);
        if (dtype == SS_BF16)
            ss_launch(gated_recurrence_portions_kernel<bf16>, tiles, dim3(GR_SEGS * 32), 0, stream, (const bf16*)proj, stride,
                      bias, state, (bf16*)out, q_start, seq_lens, slots, W, n_slots, err);
        else
            ss_launch(gated_recurrence_portions_kernel<float>, tiles, dim3(GR_SEGS * 32), 0, stream, (const float*)proj, stride,
                      bias, state, (float*)out, q_start, seq_lens, slots, W, n_slots, err);
        return SS_LAUNCH_CHECK();
    }
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

// exp(z) - 1 - z for z <= 0, to a few 1e-7 of max(z^2 / 2, 1e-7): a series near zero, where the subtraction would
// cancel, and the fast exponential elsewhere.  For results that are rounded to bfloat16.
__device__ __forceinline__ float exp_tail(float z) {
    const float series = z * z * fmaf(z, fmaf(z, fmaf(z, fmaf(z, 1.f / 720.f, 1.f / 120.f), 1.f / 24.f), 1.f / 6.f), 0.5f);
    return z > -0.25f ? series : (__expf(z) - 1.f) - z;
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
            const float y0 = z0 > 0.f ? fmaf(a * z0, z0, 0.5f * z0) : fmaf(b, exp_tail(z0), 0.5f * z0);
            const float y1 = z1 > 0.f ? fmaf(a * z1, z1, 0.5f * z1) : fmaf(b, exp_tail(z1), 0.5f * z1);
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
// are zeroed.  `scale_col` >= 0: f = sigmoid(gates[row][scale_col + h]).  With w null the product is already in
// `out` (a library's batched product wrote it): the kernel rotates, zeroes the padding and multiplies by f in place.
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
    if (w == nullptr && scale_col >= 0) {
        for (int idx = tid; idx < rows * O; idx += blockDim.x) {
            const int rr = idx / O, o = idx - rr * O;
            const float f = sigmoid_exact(to_float(gates[(int64_t)(row0 + rr) * gate_stride + scale_col + h]));
            T* dst = out + (int64_t)(row0 + rr) * out_stride + (int64_t)h * out_head + turn + o;
            *dst = from_float<T>(to_float(*dst) * f);
        }
    }
    const T* wh = w + (int64_t)h * I * O;
    for (int o = tid; w != nullptr && o < O; o += blockDim.x) {
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

// Kernels of the parts beside plain attention and the dense feed-forward: a grouped RMS norm on a branch's output,
// a state-space mixer (short causal convolution and the diagonal recurrence, both with per-request state), routed
// experts (router, plan, grouped products), weighted query/key norms in front of the rotation with rotated
// values, the turn back of the heads' outputs, and a soft cap.  Everything the recurrence touches, every norm and
// every router score is float32; T is the compute type of projections and activations (bfloat16 or float32).
//
// Batch layout as everywhere: token-major rows; q_start[r] .. q_start[r + 1] are the rows of request r, seq_lens[r]
// its cached length after the step.  A request with seq_lens[r] <= 0 is padding of a captured step and is skipped,
// and so are rows at or beyond q_start[R].
#include "common.cuh"

// The request whose rows hold `row`: the last r with q_start[r] <= row (requests without rows are passed over);
// -1 when the row lies beyond the last request.
__device__ __forceinline__ int request_of_row(const int32_t* __restrict__ q_start, int R, int row) {
    if (row >= q_start[R]) return -1;
    int lo = 0, hi = R - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (q_start[mid] <= row) lo = mid; else hi = mid - 1;
    }
    return lo;
}

__device__ __forceinline__ float silu_exact(float z) { return z / (1.0f + expf(-z)); }

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// ---------------------------------------------------------------- grouped RMS norm
//
// x_i = sum_{k < terms} in[row][k * hidden + i]  (+ extra[row][i])  (* silu(gate[row][i]))
// the row in `groups` equal consecutive parts; y_i = x_i / sqrt(mean(part^2) + eps) * weight[i]
// residual given: residual[row][i] += y_i and out (if given) = residual; else out = y.
// rows given: source row of output row m is rows[m].
// term_rows given: term k of row r is row term_rows[r * terms + k] of `in` ([.][hidden]) instead.
// A block per output row; a group is summed by GW warps in a fixed order that depends on the sizes only.
template <typename TI>
__device__ __forceinline__ float term_at(const TI* __restrict__ in, const TI* __restrict__ src,
                                         const int32_t* __restrict__ term_rows, int64_t row, int terms, int hidden, int k, int i) {
    if (term_rows) return to_float(in[(int64_t)term_rows[row * terms + k] * hidden + i]);
    return to_float(src[(int64_t)k * hidden + i]);
}

// MODE 0: one term, no index, nothing added, no gate (a branch's output as it is); 1: one term under a gate; 2: the
// general form.  Each a kernel of its own, so that the simple forms ask nothing per element.
template <typename TI, typename TG, typename TO, int MODE>
__global__ void __launch_bounds__(256)
group_norm_kernel(const TI* __restrict__ in, int64_t in_stride, int terms, const TO* __restrict__ extra,
                  const TG* __restrict__ gate, int64_t gate_stride, const float* __restrict__ weight,
                  float* __restrict__ residual, TO* __restrict__ out, const int32_t* __restrict__ rows, int hidden,
                  int groups, float eps, const int32_t* __restrict__ term_rows) {
    pdl_wait();
    __shared__ float part[8];
    const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = rows ? rows[m] : m;
    const int gs = hidden / groups;
    const int gw = groups >= 8 ? 1 : 8 / groups;  // warps that share a group
    const int at_once = 8 / gw;                   // groups the block holds at a time
    const TI* src = in + row * in_stride;
    // where the terms of this row start: looked up once, not per element
    constexpr int MAXT = MODE == 2 ? 8 : 1;
    const TI* tp[MAXT];
#pragma unroll
    for (int k = 0; k < MAXT; ++k)
        tp[k] = (MODE == 2 && k < terms) ? (term_rows ? in + (int64_t)term_rows[row * terms + k] * hidden : src + (int64_t)k * hidden) : src;
    auto value_at = [&](int i) -> float {
        if (MODE == 0) return to_float(src[i]);
        if (MODE == 1) return to_float(src[i]) * silu_exact(to_float(gate[row * gate_stride + i]));
        float x;
        if (terms <= MAXT) {
            x = to_float(tp[0][i]);
#pragma unroll
            for (int k = 1; k < MAXT; ++k)
                if (k < terms) x += to_float(tp[k][i]);
        } else {
            x = term_at(in, src, term_rows, row, terms, hidden, 0, i);
            for (int k = 1; k < terms; ++k) x += term_at(in, src, term_rows, row, terms, hidden, k, i);
        }
        if (extra) x += to_float(extra[row * hidden + i]);
        if (gate) x *= silu_exact(to_float(gate[row * gate_stride + i]));
        return x;
    };
    for (int g0 = 0; g0 < groups; g0 += at_once) {
        const int g = g0 + warp / gw, wi = warp % gw;
        const bool on = g < groups && warp < at_once * gw;
        float ss = 0.f;
        if (on) {
#pragma unroll 4
            for (int j = wi * 32 + lane; j < gs; j += gw * 32) {
                const float x = value_at(g * gs + j);
                ss = fmaf(x, x, ss);
            }
            ss = warp_sum(ss);
        }
        __syncthreads();
        if (lane == 0) part[warp] = on ? ss : 0.f;
        __syncthreads();
        if (on) {
            float total = 0.f;
            for (int k = 0; k < gw; ++k) total += part[(warp / gw) * gw + k];
            const float rstd = 1.0f / sqrtf(total / (float)gs + eps);
#pragma unroll 4
            for (int j = wi * 32 + lane; j < gs; j += gw * 32) {
                const int i = g * gs + j;
                float y = value_at(i) * rstd * weight[i];
                if (residual) {
                    y += residual[row * hidden + i];
                    residual[row * hidden + i] = y;
                }
                if (out) out[(int64_t)m * hidden + i] = from_float<TO>(y);
            }
        }
    }
}

// in_type: 0 the compute type, 1 float32.  dtype: the compute type (of out, extra and gate).
extern "C" int ss_group_norm(const void* in, int in_f32, int64_t in_stride, int terms, const void* extra, const void* gate,
                             int64_t gate_stride, const float* weight, float* residual, void* out, const int32_t* rows,
                             int n_out, int hidden, int groups, float eps, int dtype, cudaStream_t stream,
                             const int32_t* term_rows) {
    if (n_out <= 0) return 0;
    if (groups < 1 || hidden % groups || terms < 1) return (int)cudaErrorInvalidValue;
    const int mode = (terms == 1 && !term_rows && !extra) ? (gate ? 1 : 0) : 2;
#define GN_LAUNCH(TI, T, MODE)                                                                                        \
    ss_launch(group_norm_kernel<TI, T, T, MODE>, dim3(n_out), dim3(256), 0, stream, (const TI*)in, in_stride, terms,  \
              (const T*)extra, (const T*)gate, gate_stride, weight, residual, (T*)out, rows, hidden, groups, eps, term_rows)
#define GN_GO(TI, T)                                                                                                  \
    if (mode == 0) GN_LAUNCH(TI, T, 0);                                                                               \
    else if (mode == 1) GN_LAUNCH(TI, T, 1);                                                                          \
    else GN_LAUNCH(TI, T, 2)
    if (dtype == SS_F32) { GN_GO(float, float); }
    else if (in_f32) { GN_GO(float, bf16); }
    else { GN_GO(bf16, bf16); }
#undef GN_LAUNCH
#undef GN_GO
    return SS_LAUNCH_CHECK();
}

// The float32 stream rounded to the compute type (what a branch reads).
__global__ void round_stream_kernel(const float* __restrict__ in, bf16* __restrict__ out, int64_t n) {
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}

extern "C" int ss_round_stream(const float* in, void* out, int64_t n, cudaStream_t stream) {
    if (n <= 0) return 0;
    ss_launch(round_stream_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, in, (bf16*)out, n);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- short causal convolution with state
//
// in: channel c of token `row` is proj[row * stride + col0 + c].  out[row][c] = silu(bias[c] + sum_j taps[c][j] *
// input(t - (T - 1 - j))), where inputs in front of the step's first row come from the request's state
// [slot][T - 1][C] (float32; index T - 2 is the newest) and inputs in front of the request's first token are the
// zeros a fresh state holds.  `fused_update`: every request brings one token and the thread that read the state
// also shifts it; otherwise conv_state_kernel does that in a launch of its own, behind this one.  `plus_input` 1: the
// result is input + (bias +) convolution with no activation instead (a convolution on a branch's input); 2: bias +
// convolution with no activation.
#define CONV_MAX_TAPS 8
#define CONV_ROWS 32
// A thread takes one channel over CONV_ROWS consecutive rows and keeps the channel's last T - 1 inputs in
// registers, so every input is read once (and the few in front of the tile once more).
template <typename T>
__global__ void __launch_bounds__(128)
conv_silu_kernel(const T* __restrict__ proj, int64_t stride, int col0, const float* __restrict__ taps,
                 const float* __restrict__ bias, float* __restrict__ state, T* __restrict__ out,
                 const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                 const int32_t* __restrict__ slots, int R, int n_rows, int C, int n_taps, int n_slots, int fused_update,
                 int* err, int plus_input) {
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float w[CONV_MAX_TAPS], x[CONV_MAX_TAPS];  // x[j]: the input T - 1 - j tokens back; x[T - 1]: the current one
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        w[j] = j < n_taps ? taps[(int64_t)c * n_taps + j] : 0.f;
        x[j] = 0.f;
    }
    const float b = bias ? bias[c] : 0.f;
    const int back = n_taps - 1;
    const int row_end = min(n_rows, (blockIdx.x + 1) * CONV_ROWS);
    int r = -1, r_end = -1;  // the request of the rows in front of r_end
    bool on = false;
    float* st = state;
    const int row_first = blockIdx.x * CONV_ROWS;
    for (int row = row_first; row < row_end; ++row) {
        bool fresh = row == blockIdx.x * CONV_ROWS;
        if (row >= r_end) {
            r = request_of_row(q_start, R, row);
            if (r < 0) break;
            r_end = q_start[r + 1];
            const int slot = slots[r];
            on = seq_lens[r] > 0 && slot >= 0 && slot < n_slots;
            if (seq_lens[r] > 0 && !on && threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
            st = state + (int64_t)(on ? slot : 0) * back * C + c;
            fresh = true;
        }
        if (!on) continue;
        if (fresh) {  // the window in front of this row: earlier rows of the step, or the request's state
            const int i = row - q_start[r];
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
                if (j >= back) break;
                const int src = i - (back - j);
                x[j] = src >= 0 ? to_float(proj[(int64_t)(row - (back - j)) * stride + col0 + c]) : st[(int64_t)(back + src) * C];
            }
        }
        const float cur = to_float(proj[(int64_t)row * stride + col0 + c]);
        float acc = b;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)  // (no register array is indexed by a run-time value)
            if (j <= back) acc = fmaf(w[j], j < back ? x[j] : cur, acc);
        out[(int64_t)row * C + c] = from_float<T>(plus_input == 1 ? cur + acc : (plus_input == 2 ? acc : silu_exact(acc)));
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < back) x[j] = j + 1 < back ? x[j + 1] : cur;
        if (fused_update) {
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
                if (j < back) st[(int64_t)j * C] = x[j];
        }
    }
}

// The same for bfloat16 with channels in steps of 8 (and the projection's rows and the first channel on 16-byte
// boundaries) and at most 4 taps: a thread takes 8 neighbouring channels, 16 bytes a load and a store, over
// CONV_ROWS rows.  The window of a row that is not a request's first in this tile is already in registers.
__global__ void __launch_bounds__(128)
conv_silu_bf16x8_kernel(const bf16* __restrict__ proj, int64_t stride, int col0, const float* __restrict__ taps,
                        const float* __restrict__ bias, float* __restrict__ state, bf16* __restrict__ out,
                        const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                        const int32_t* __restrict__ slots, int R, int n_rows, int C, int n_taps, int n_slots,
                        int fused_update, int* err, int plus_input) {
    pdl_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    constexpr int MAXB = 3;  // taps - 1 at most
    const int back = n_taps - 1;
    float w[8][MAXB + 1], x[8][MAXB], b[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        b[e] = bias ? bias[c + e] : 0.f;
#pragma unroll
        for (int j = 0; j <= MAXB; ++j) w[e][j] = j < n_taps ? taps[(int64_t)(c + e) * n_taps + j] : 0.f;
#pragma unroll
        for (int j = 0; j < MAXB; ++j) x[e][j] = 0.f;
    }
    auto widen = [](const uint4& raw, float (&v)[8]) {
        const uint32_t q[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { v[2 * e] = __uint_as_float(q[e] << 16); v[2 * e + 1] = __uint_as_float(q[e] & 0xffff0000u); }
    };
    const int row_first = blockIdx.x * CONV_ROWS, row_end = min(n_rows, row_first + CONV_ROWS);
    int r = -1, r_end = -1;
    bool on = false;
    float* st = state;
    for (int row = row_first; row < row_end; ++row) {
        bool fresh = row == row_first;
        if (row >= r_end) {
            r = request_of_row(q_start, R, row);
            if (r < 0) break;
            r_end = q_start[r + 1];
            const int slot = slots[r];
            on = seq_lens[r] > 0 && slot >= 0 && slot < n_slots;
            if (seq_lens[r] > 0 && !on && threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
            st = state + (int64_t)(on ? slot : 0) * back * C + c;
            fresh = true;
        }
        if (!on) continue;
        if (fresh) {
            const int i = row - q_start[r];
#pragma unroll
            for (int j = 0; j < MAXB; ++j) {
                if (j >= back) break;
                const int src = i - (back - j);
                float v[8];
                if (src >= 0) {
                    widen(*reinterpret_cast<const uint4*>(proj + (int64_t)(row - (back - j)) * stride + col0 + c), v);
                } else {
                    const float4 lo = *reinterpret_cast<const float4*>(st + (int64_t)(back + src) * C);
                    const float4 hi = *reinterpret_cast<const float4*>(st + (int64_t)(back + src) * C + 4);
                    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e][j] = v[e];
            }
        }
        float cur[8];
        widen(*reinterpret_cast<const uint4*>(proj + (int64_t)row * stride + col0 + c), cur);
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            float o2[2];
#pragma unroll
            for (int d = 0; d < 2; ++d) {
                float acc = b[e + d];
#pragma unroll
                for (int j = 0; j <= MAXB; ++j)
                    if (j <= back) acc = fmaf(w[e + d][j], j < back ? x[e + d][j < MAXB ? j : 0] : cur[e + d], acc);
                o2[d] = plus_input == 1 ? cur[e + d] + acc : (plus_input == 2 ? acc : silu_exact(acc));
            }
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(o2[0], o2[1]);
            packed[e >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        *reinterpret_cast<uint4*>(out + (int64_t)row * C + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
            for (int j = 0; j < MAXB; ++j)
                if (j < back) x[e][j] = (j + 1 < back) ? x[e][j + 1 < MAXB ? j + 1 : 0] : cur[e];
        if (fused_update) {
#pragma unroll
            for (int j = 0; j < MAXB; ++j)
                if (j < back) {
                    *reinterpret_cast<float4*>(st + (int64_t)j * C) = make_float4(x[0][j], x[1][j], x[2][j], x[3][j]);
                    *reinterpret_cast<float4*>(st + (int64_t)j * C + 4) = make_float4(x[4][j], x[5][j], x[6][j], x[7][j]);
                }
        }
    }
}

// The state after the step: the last T - 1 inputs of each request, old ones kept where the step brought fewer.
template <typename T>
__global__ void __launch_bounds__(128)
conv_state_kernel(const T* __restrict__ proj, int64_t stride, int col0, float* __restrict__ state,
                  const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                  const int32_t* __restrict__ slots, int C, int n_taps, int n_slots) {
    pdl_wait();
    const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (c >= C || q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) return;
    const int back = n_taps - 1;
    float* st = state + (int64_t)slot * back * C + c;
    for (int s = 0; s < back; ++s) {  // ascending: an old value is read before its place is written
        const int i = q_len - back + s;
        st[(int64_t)s * C] = i >= 0 ? to_float(proj[(int64_t)(q0 + i) * stride + col0 + c]) : st[(int64_t)(s + q_len) * C];
    }
}

extern "C" int ss_conv_silu(const void* proj, int64_t stride, int col0, const float* taps, const float* bias, float* state,
                            void* out, const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int R,
                            int n_rows, int C, int n_taps, int n_slots, int fused_update, int dtype, int* err,
                            cudaStream_t stream, int plus_input) {
    if (n_rows <= 0 || R <= 0) return 0;
    if (n_taps < 1 || n_taps > CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
    const dim3 grid((n_rows + CONV_ROWS - 1) / CONV_ROWS, (C + 127) / 128);
    if (dtype == SS_BF16 && !fused_update && n_taps <= 4 && C % 8 == 0 && col0 % 8 == 0 && stride % 8 == 0 && ((uintptr_t)proj & 15) == 0 &&
        ((uintptr_t)out & 15) == 0 && ((uintptr_t)state & 15) == 0) {
        const dim3 grid8((n_rows + CONV_ROWS - 1) / CONV_ROWS, (C / 8 + 127) / 128);
        ss_launch(conv_silu_bf16x8_kernel, grid8, dim3(128), 0, stream, (const bf16*)proj, stride, col0, taps, bias, state,
                  (bf16*)out, q_start, seq_lens, slots, R, n_rows, C, n_taps, n_slots, fused_update, err, plus_input);
    } else if (dtype == SS_BF16)
        ss_launch(conv_silu_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)proj, stride, col0, taps, bias, state,
                  (bf16*)out, q_start, seq_lens, slots, R, n_rows, C, n_taps, n_slots, fused_update, err, plus_input);
    else
        ss_launch(conv_silu_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, stride, col0, taps, bias, state,
                  (float*)out, q_start, seq_lens, slots, R, n_rows, C, n_taps, n_slots, fused_update, err, plus_input);
    if (!fused_update && n_taps > 1) {
        const dim3 grid2(R, (C + 127) / 128);
        if (dtype == SS_BF16)
            ss_launch(conv_state_kernel<bf16>, grid2, dim3(128), 0, stream, (const bf16*)proj, stride, col0, state, q_start,
                      seq_lens, slots, C, n_taps, n_slots);
        else
            ss_launch(conv_state_kernel<float>, grid2, dim3(128), 0, stream, (const float*)proj, stride, col0, state, q_start,
                      seq_lens, slots, C, n_taps, n_slots);
    }
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- the diagonal state-space recurrence
//
// Per request, head h (group g = h / (heads / groups)) and token t, with x_t [P], B_t and C_t [N] (the convolution's
// output: x at column 0, B at heads * P, C behind B), raw step dt_t (a column of the input projection):
//   dt = softplus(dt_t + dt_bias[h]);  S <- exp(-exp(A_log[h]) dt) S + dt B_t x_t^T;  y_t = S^T C_t + D[h] x_t.
// S is float32 [N x P] per (slot, head), stored [slot][head][P][N], carried across steps.  A block per (request,
// head, tile of PT <= 32 columns p); 4 neighbouring lanes share a column, each holding PER consecutive n in registers
// (N <= 4 PER: many independent chains a thread, few shuffles a token); tokens run one after the other, staged SCAN_TB at a time through shared memory, where a
// lane's PER values of B and of C stand together (and 4 floats apart from the next lane's, so that the 16-byte
// loads of the 8 lanes fall on different banks).  The order of the arithmetic behind an output does not depend on
// how the request was cut into steps.
#define SCAN_NS 4
#define SCAN_PT 32
template <typename T, int PER>
__global__ void __launch_bounds__(SCAN_PT * SCAN_NS)
ssm_scan_kernel(const T* __restrict__ xbc, int C, const T* __restrict__ dt_raw, int64_t dt_stride,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, float* __restrict__ y, const int32_t* __restrict__ q_start,
                const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ slots, int heads, int groups, int P,
                int N, int PT, int n_slots, int* err) {
    pdl_wait();
    constexpr int SCAN_TB = PER >= 64 ? 16 : 32;  // tokens staged at a time (the widest state: fewer, to stay in 48 KB)
    constexpr int SEG = PER + 4, ROW = SCAN_NS * SEG;  // a lane's segment, a token's row of B (or C)
    extern __shared__ __align__(16) float sm[];
    float* Bs = sm;                      // [TB][ROW]
    float* Cs = Bs + SCAN_TB * ROW;      // [TB][ROW]
    float* xs = Cs + SCAN_TB * ROW;      // [TB][PT]
    float* dts = xs + SCAN_TB * PT;      // [TB]
    float* decs = dts + SCAN_TB;         // [TB]
    const int r = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * PT;
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    const int tid = threadIdx.x, pl = tid / SCAN_NS, ns = tid % SCAN_NS;
    const int p = p0 + pl, n0 = ns * PER;
    const bool valid = p < P;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    float* st = state + (((int64_t)slot * heads + h) * P + (valid ? p : 0)) * N;
    float S[PER];
    const bool vec = (N & 3) == 0;  // then a lane's values are whole 16-byte pieces
#pragma unroll
    for (int i = 0; i < PER; i += 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid && vec && n0 + i < N) v = *reinterpret_cast<const float4*>(st + n0 + i);
        if (valid && !vec) {
            if (n0 + i < N) v.x = st[n0 + i];
            if (n0 + i + 1 < N) v.y = st[n0 + i + 1];
            if (n0 + i + 2 < N) v.z = st[n0 + i + 2];
            if (n0 + i + 3 < N) v.w = st[n0 + i + 3];
        }
        S[i] = v.x; S[i + 1] = v.y; S[i + 2] = v.z; S[i + 3] = v.w;
    }
    const float rate = expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];
    // bfloat16 rows whose B and C parts start on 16-byte boundaries are staged 8 values a load
    const bool vec8 = sizeof(T) == 2 && (C & 7) == 0 && (inner & 7) == 0 && (N & 7) == 0 && (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
    if (vec8 && N < SCAN_NS * PER) {  // the places behind N are never written by that path: zeros, which leave their S at zero
        const int used = min(SCAN_TB, q_len) * ROW;
        for (int i = tid; i < used; i += blockDim.x) Bs[i] = Cs[i] = 0.f;
    }
    for (int t0 = 0; t0 < q_len; t0 += SCAN_TB) {
        const int nt = min(SCAN_TB, q_len - t0);
        __syncthreads();
        if (vec8) {  // 16 bytes (8 values of B or of C) a load, all of a thread's loads in flight together
            const int chunks = N >> 3;
#pragma unroll 4
            for (int idx = tid; idx < nt * 2 * chunks; idx += blockDim.x) {
                const int tt = idx / (2 * chunks), rem = idx - tt * 2 * chunks;
                const int which = rem >= chunks, n = (rem - which * chunks) << 3;
                const uint4 raw = *reinterpret_cast<const uint4*>(xbc + (int64_t)(q0 + t0 + tt) * C + inner + which * groups * N + g * N + n);
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
                float* dst = (which ? Cs : Bs) + tt * ROW + (n / PER) * SEG + n % PER;  // PER is a multiple of 8
                reinterpret_cast<float4*>(dst)[0] = make_float4(__low2float(h2[0]), __high2float(h2[0]), __low2float(h2[1]), __high2float(h2[1]));
                reinterpret_cast<float4*>(dst)[1] = make_float4(__low2float(h2[2]), __high2float(h2[2]), __low2float(h2[3]), __high2float(h2[3]));
            }
        } else {
#pragma unroll 4
            for (int idx = tid; idx < nt * SCAN_NS * PER; idx += blockDim.x) {
                const int tt = idx / (SCAN_NS * PER), n = idx - tt * (SCAN_NS * PER);
                const T* row = xbc + (int64_t)(q0 + t0 + tt) * C + inner + g * N;
                const int at = tt * ROW + (n / PER) * SEG + n % PER;
                Bs[at] = n < N ? to_float(row[n]) : 0.f;  // n beyond N: zeros, which leave their S at zero
                Cs[at] = n < N ? to_float(row[groups * N + n]) : 0.f;
            }
        }
#pragma unroll 4
        for (int idx = tid; idx < nt * PT; idx += blockDim.x) {
            const int tt = idx / PT, j = idx - tt * PT;
            xs[idx] = (p0 + j < P) ? to_float(xbc[(int64_t)(q0 + t0 + tt) * C + h * P + p0 + j]) : 0.f;
        }
        if (tid < nt) {
            const float z = to_float(dt_raw[(int64_t)(q0 + t0 + tid) * dt_stride + h]) + bias;
            const float dt = z > 20.f ? z : log1pf(expf(z));
            dts[tid] = dt;
            decs[tid] = expf(-rate * dt);
        }
        __syncthreads();
        float* yp = y + (int64_t)(q0 + t0) * inner + h * P + p;
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt, yp += inner) {
            const float dec = decs[tt], xv = xs[tt * PT + pl];
            const float dx = dts[tt] * xv;
            const float4* b4 = reinterpret_cast<const float4*>(Bs + tt * ROW + ns * SEG);
            const float4* c4 = reinterpret_cast<const float4*>(Cs + tt * ROW + ns * SEG);
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i += 4) {
                const float4 b = b4[i >> 2], c = c4[i >> 2];
                S[i] = fmaf(dec, S[i], dx * b.x);
                S[i + 1] = fmaf(dec, S[i + 1], dx * b.y);
                S[i + 2] = fmaf(dec, S[i + 2], dx * b.z);
                S[i + 3] = fmaf(dec, S[i + 3], dx * b.w);
                acc0 = fmaf(S[i], c.x, acc0);
                acc1 = fmaf(S[i + 1], c.y, acc1);
                acc0 = fmaf(S[i + 2], c.z, acc0);
                acc1 = fmaf(S[i + 3], c.w, acc1);
            }
            float acc = acc0 + acc1;
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (ns == 0 && valid) *yp = fmaf(skip, xv, acc);
        }
    }
    if (valid) {
#pragma unroll
        for (int i = 0; i < PER; i += 4) {
            if (vec) {
                if (n0 + i < N) *reinterpret_cast<float4*>(st + n0 + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (n0 + i + e < N) st[n0 + i + e] = S[i + e];
            }
        }
    }
}

// The same recurrence for bfloat16 rows whose parts start on 16-byte boundaries: the tokens' B, C and x are copied
// to shared memory as they are (cp.async, 16 bytes a copy) one batch of tokens ahead of the arithmetic, into two
// buffers that take turns, and widened to float32 as they are read (8 values a 16-byte load).
__device__ __forceinline__ void cp_async_16_on(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
template <int PER>
__global__ void __launch_bounds__(SCAN_PT * SCAN_NS)
ssm_scan_bf16_kernel(const bf16* __restrict__ xbc, int C, const bf16* __restrict__ dt_raw, int64_t dt_stride,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                     const float* __restrict__ d_skip, float* __restrict__ state, float* __restrict__ y,
                     const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                     const int32_t* __restrict__ slots, int heads, int groups, int P, int N, int PT, int n_slots,
                     int* err) {
    pdl_wait();
    constexpr int TB = PER >= 64 ? 16 : 32;
    constexpr int SEGB = PER * 2 + 16, ROWB = SCAN_NS * SEGB;  // bytes: a lane's segment (16 apart from the next), a token's row
    extern __shared__ __align__(16) unsigned char raw_sm[];
    // per stage: B rows, C rows, x rows; behind both stages: the step sizes and decays of both
    const int stage_bytes = 2 * TB * ROWB + TB * PT * 2;
    float* dts = reinterpret_cast<float*>(raw_sm + 2 * stage_bytes);  // [2][TB]
    float* decs = dts + 2 * TB;                                        // [2][TB]
    const int r = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * PT;
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    if (q_len <= 0 || seq_lens[r] <= 0) return;
    const int slot = slots[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        return;
    }
    const int tid = threadIdx.x, pl = tid / SCAN_NS, ns = tid % SCAN_NS;
    const int p = p0 + pl, n0 = ns * PER;
    const bool valid = p < P;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    float* st = state + (((int64_t)slot * heads + h) * P + (valid ? p : 0)) * N;
    float S[PER];
#pragma unroll
    for (int i = 0; i < PER; i += 4) {  // N is a multiple of 8 here
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid && n0 + i < N) v = *reinterpret_cast<const float4*>(st + n0 + i);
        S[i] = v.x; S[i + 1] = v.y; S[i + 2] = v.z; S[i + 3] = v.w;
    }
    const float rate = expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];
    for (int i = tid * 16; i < 2 * stage_bytes; i += blockDim.x * 16)  // what no copy writes (n beyond N) stays zero
        *reinterpret_cast<uint4*>(raw_sm + i) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const int chunks = N >> 3, x_chunks = PT >> 3;
    auto issue = [&](int stage, int t0, int nt) {
        unsigned char* base = raw_sm + stage * stage_bytes;
        for (int idx = tid; idx < nt * 2 * chunks; idx += blockDim.x) {
            const int tt = idx / (2 * chunks), rem = idx - tt * 2 * chunks;
            const int which = rem >= chunks, n = (rem - which * chunks) << 3;
            cp_async_16_on(base + which * TB * ROWB + tt * ROWB + (n / PER) * SEGB + (n % PER) * 2,
                           xbc + (int64_t)(q0 + t0 + tt) * C + inner + which * groups * N + g * N + n);
        }
        for (int idx = tid; idx < nt * x_chunks; idx += blockDim.x) {
            const int tt = idx / x_chunks, c = idx - tt * x_chunks;
            if (p0 + 8 * c < P)
                cp_async_16_on(base + 2 * TB * ROWB + (tt * PT + 8 * c) * 2, xbc + (int64_t)(q0 + t0 + tt) * C + h * P + p0 + 8 * c);
        }
    };
    const int n_batches = (q_len + TB - 1) / TB;
    issue(0, 0, min(TB, q_len));
    cp_async_commit();
    float dt_next = (tid < min(TB, q_len)) ? to_float(dt_raw[(int64_t)(q0 + tid) * dt_stride + h]) : 0.f;
    for (int k = 0; k < n_batches; ++k) {
        const int t0 = k * TB, nt = min(TB, q_len - t0), buf = k & 1;
        if (tid < nt) {
            const float z = dt_next + bias;
            const float dt = z > 20.f ? z : log1pf(expf(z));
            dts[buf * TB + tid] = dt;
            decs[buf * TB + tid] = expf(-rate * dt);
        }
        if (k + 1 < n_batches) {
            const int nt1 = min(TB, q_len - t0 - TB);
            issue(buf ^ 1, t0 + TB, nt1);
            if (tid < nt1) dt_next = to_float(dt_raw[(int64_t)(q0 + t0 + TB + tid) * dt_stride + h]);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* base = raw_sm + buf * stage_bytes;
        const bf16* xs = reinterpret_cast<const bf16*>(base + 2 * TB * ROWB);
        float* yp = y + (int64_t)(q0 + t0) * inner + h * P + p;
#pragma unroll 2
        for (int tt = 0; tt < nt; ++tt, yp += inner) {
            const float dec = decs[buf * TB + tt], xv = to_float(xs[tt * PT + pl]);
            const float dx = dts[buf * TB + tt] * xv;
            const uint4* b8 = reinterpret_cast<const uint4*>(base + tt * ROWB + ns * SEGB);
            const uint4* c8 = reinterpret_cast<const uint4*>(base + TB * ROWB + tt * ROWB + ns * SEGB);
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i += 8) {
                const uint4 bw = b8[i >> 3], cw = c8[i >> 3];
                const uint32_t bb[4] = {bw.x, bw.y, bw.z, bw.w}, cc[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float b_lo = __uint_as_float(bb[e] << 16), b_hi = __uint_as_float(bb[e] & 0xffff0000u);
                    const float c_lo = __uint_as_float(cc[e] << 16), c_hi = __uint_as_float(cc[e] & 0xffff0000u);
                    S[i + 2 * e] = fmaf(dec, S[i + 2 * e], dx * b_lo);
                    S[i + 2 * e + 1] = fmaf(dec, S[i + 2 * e + 1], dx * b_hi);
                    acc0 = fmaf(S[i + 2 * e], c_lo, acc0);
                    acc1 = fmaf(S[i + 2 * e + 1], c_hi, acc1);
                }
            }
            float acc = acc0 + acc1;
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (ns == 0 && valid) *yp = fmaf(skip, xv, acc);
        }
        __syncthreads();  // the buffer is free for the copies of the batch after next
    }
    cp_async_wait<0>();
    if (valid) {
#pragma unroll
        for (int i = 0; i < PER; i += 4)
            if (n0 + i < N) *reinterpret_cast<float4*>(st + n0 + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    }
}

extern "C" int ss_ssm_scan(const void* xbc, int C, const void* dt_raw, int64_t dt_stride, const float* dt_bias,
                           const float* a_log, const float* d_skip, float* state, float* y, const int32_t* q_start,
                           const int32_t* seq_lens, const int32_t* slots, int R, int heads, int groups, int P, int N,
                           int n_slots, int dtype, int* err, cudaStream_t stream, int long_rows) {
    if (R <= 0) return 0;
    if (N < 1 || N > 256 || P < 1 || groups < 1 || heads % groups) return (int)cudaErrorInvalidValue;
    const int PT = P >= SCAN_PT ? SCAN_PT : (P + 7) / 8 * 8;  // a block of PT * 4 threads: whole warps
    const dim3 grid(R, heads, (P + PT - 1) / PT), block(PT * SCAN_NS);
    const int per = N <= 32 ? 8 : (N <= 64 ? 16 : (N <= 128 ? 32 : 64));
    const int tb = per >= 64 ? 16 : 32;
    const int smem = (2 * tb * SCAN_NS * (per + 4) + tb * PT + 2 * tb) * 4;
    if (long_rows && dtype == SS_BF16 && C % 8 == 0 && (heads * P) % 8 == 0 && N % 8 == 0 && P % 8 == 0 && ((uintptr_t)xbc & 15) == 0 &&
        ((uintptr_t)state & 15) == 0) {
        const int stage = 2 * tb * SCAN_NS * (per * 2 + 16) + tb * PT * 2;
        const int smem16 = 2 * stage + 4 * tb * 4;
#define SCAN16_GO(PER)                                                                                                  \
    ss_launch(ssm_scan_bf16_kernel<PER>, grid, block, smem16, stream, (const bf16*)xbc, C, (const bf16*)dt_raw, dt_stride,  \
              dt_bias, a_log, d_skip, state, y, q_start, seq_lens, slots, heads, groups, P, N, PT, n_slots, err)
        if (per == 8) SCAN16_GO(8);
        else if (per == 16) SCAN16_GO(16);
        else if (per == 32) SCAN16_GO(32);
        else SCAN16_GO(64);
#undef SCAN16_GO
        return SS_LAUNCH_CHECK();
    }
#define SCAN_GO(T, PER)                                                                                                 \
    ss_launch(ssm_scan_kernel<T, PER>, grid, block, smem, stream, (const T*)xbc, C, (const T*)dt_raw, dt_stride, dt_bias,     \
              a_log, d_skip, state, y, q_start, seq_lens, slots, heads, groups, P, N, PT, n_slots, err)
#define SCAN_PICK(T)                                                                                                    \
    if (per == 8) SCAN_GO(T, 8);                                                                                        \
    else if (per == 16) SCAN_GO(T, 16);                                                                                 \
    else if (per == 32) SCAN_GO(T, 32);                                                                                 \
    else SCAN_GO(T, 64)
    if (dtype == SS_BF16) { SCAN_PICK(bf16); }
    else { SCAN_PICK(float); }
#undef SCAN_PICK
#undef SCAN_GO
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- router of the routed experts
//
// z = W_router x in float32 (x and W in the compute type); scores s = sigmoid(z), or, with `softmax`, the softmax of
// z over all experts; choice scores c = s + correction (no correction: c = s).  With `groups` > 1 the experts form
// that many equal groups of neighbours, a group's score is its largest choice score, and only experts of the `keep`
// best groups can be chosen (the others' choice scores count as -infinity).  The `top` largest choice scores are
// chosen (ties: the lower index); ids[token][k] the chosen expert, w[token][k] = its score s (without the
// correction), or, with `renormalize`, that divided by the sum over the chosen.  `extra` more rows of W behind the
// experts' ride along in the product: their logits leave raw in extra_out[token][extra] (a gate that reads the
// same input, say).  A block per token.
#define ROUTER_MAX_EXPERTS 1024
#define ROUTER_THREADS 256
// A lane's part of w . x (x in shared memory as float32).  bfloat16 rows of a length in steps of 8 (their starts are
// then on 16-byte boundaries when the matrix is): sixteen bytes a load, four loads in flight.
__device__ __forceinline__ float router_dot(const float* __restrict__ w, const float* __restrict__ xs, int hidden, int lane) {
    float acc = 0.f;
    for (int i = lane; i < hidden; i += 32) acc = fmaf(w[i], xs[i], acc);
    return acc;
}
__device__ __forceinline__ float router_dot(const bf16* __restrict__ w, const float* __restrict__ xs, int hidden, int lane) {
    float acc = 0.f;
    if ((hidden & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
#pragma unroll 4
        for (int i = lane * 8; i < hidden; i += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
            const float4 a = *reinterpret_cast<const float4*>(xs + i), b = *reinterpret_cast<const float4*>(xs + i + 4);
            acc = fmaf(__uint_as_float(raw.x << 16), a.x, acc);
            acc = fmaf(__uint_as_float(raw.x & 0xffff0000u), a.y, acc);
            acc = fmaf(__uint_as_float(raw.y << 16), a.z, acc);
            acc = fmaf(__uint_as_float(raw.y & 0xffff0000u), a.w, acc);
            acc = fmaf(__uint_as_float(raw.z << 16), b.x, acc);
            acc = fmaf(__uint_as_float(raw.z & 0xffff0000u), b.y, acc);
            acc = fmaf(__uint_as_float(raw.w << 16), b.z, acc);
            acc = fmaf(__uint_as_float(raw.w & 0xffff0000u), b.w, acc);
        }
        return acc;
    }
    for (int i = lane; i < hidden; i += 32) acc = fmaf(to_float(w[i]), xs[i], acc);
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_kernel(const T* __restrict__ x, const T* __restrict__ w_router, int32_t* __restrict__ ids,
              float* __restrict__ weights, int hidden, int experts, int top, int renormalize, int softmax,
              const float* __restrict__ correction, int groups, int keep, float* __restrict__ extra_out, int extra) {
    pdl_wait();
    extern __shared__ __align__(16) float rsm[];
    float* xs = rsm;                  // [hidden] (rounded up to a multiple of 4)
    float* z = rsm + ((hidden + 3) & ~3);  // [experts] scores
    float* c = z + experts;           // [experts] choice scores
    float* gb = c + experts;          // [groups] the groups' scores
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < hidden; i += blockDim.x) xs[i] = to_float(x[(int64_t)t * hidden + i]);
    __syncthreads();
    const int n_warps = blockDim.x >> 5;
    for (int e = warp; e < experts + extra; e += n_warps) {
        const T* w = w_router + (int64_t)e * hidden;
        float acc = router_dot(w, xs, hidden, lane);
        acc = warp_sum(acc);
        if (lane == 0) {
            if (e >= experts) extra_out[(int64_t)t * extra + (e - experts)] = acc;
            else z[e] = softmax ? acc : 1.0f / (1.0f + expf(-acc));  // the choice below is among scores
        }
    }
    __syncthreads();
    if (warp != 0) return;
    if (softmax) {
        float mx = -INFINITY;
        for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < experts; e += 32) {
            const float p = expf(z[e] - mx);
            z[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) z[e] = z[e] / sum;
    }
    for (int e = lane; e < experts; e += 32) c[e] = z[e] + (correction ? correction[e] : 0.f);
    __syncwarp();
    if (groups > 1) {
        const int per = experts / groups;
        for (int g = lane; g < groups; g += 32) {
            float m = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, c[e]);
            gb[g] = m;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {  // the best group that is left, `keep` times; a kept group is marked by NaN
            float best = -INFINITY;
            int at = groups;
            for (int g = lane; g < groups; g += 32) {
                const float v = gb[g];
                if (v == v && (v > best || at == groups)) { best = v; at = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (oa < groups && (at == groups || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
            }
            if (lane == 0 && at < groups) gb[at] = __int_as_float(0x7fc00000);
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32) {
            const float mark = gb[e / per];
            if (mark == mark) c[e] = -INFINITY;  // its group was not kept
        }
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = experts;
        for (int e = lane; e < experts; e += 32) {
            const float v = c[e];
            if (v > best) { best = v; at = e; }  // ascending e: the lower index stays on a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        const float s = at < experts ? z[at] : 0.f;
        total += s;
        if (lane == 0) {
            ids[(int64_t)t * top + k] = at < experts ? at : 0;
            weights[(int64_t)t * top + k] = s;
            if (at < experts) c[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (renormalize && lane == 0)
        for (int k = 0; k < top; ++k) weights[(int64_t)t * top + k] /= total;
}

extern "C" int ss_router(const void* x, const void* w_router, int32_t* ids, float* weights, int n_tokens, int hidden,
                         int experts, int top, int renormalize, int dtype, cudaStream_t stream, int softmax,
                         const float* correction, int groups, int keep, float* extra_out, int extra) {
    if (n_tokens <= 0) return 0;
    if (experts < 1 || experts > ROUTER_MAX_EXPERTS || top < 1 || top > experts) return (int)cudaErrorInvalidValue;
    if (groups < 1 || experts % groups || keep < 1 || keep > groups || extra < 0 || (extra > 0 && !extra_out))
        return (int)cudaErrorInvalidValue;
    const int smem = (((hidden + 3) & ~3) + 2 * experts + groups) * 4;
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (dtype == SS_BF16)
        ss_launch(router_kernel<bf16>, dim3(n_tokens), dim3(ROUTER_THREADS), smem, stream, (const bf16*)x, (const bf16*)w_router, ids,
                  weights, hidden, experts, top, renormalize, softmax, correction, groups, keep, extra_out, extra);
    else
        ss_launch(router_kernel<float>, dim3(n_tokens), dim3(ROUTER_THREADS), smem, stream, (const float*)x, (const float*)w_router,
                  ids, weights, hidden, experts, top, renormalize, softmax, correction, groups, keep, extra_out, extra);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- plan of the grouped products
//
// A = tokens * top assignments (token t, choice k) -> a = t * top + k.  The plan sorts them by expert:
// perm[s] = the assignment at sorted place s; an expert's places are consecutive and cut into tiles of `tile`
// rows: tile_expert[i] (or -1 for a tile that holds nothing), tile_row0[i], tile_rows[i].  The lists have
// ceil(A / tile) + experts entries, the most any routing needs, so the launch that walks them is the same every
// step.  One block.  Places within an expert follow the order in which threads arrive; no result depends on it,
// since every row of a product is computed by itself.  Experts from `real` on have no weights (experts that hand their
// input on): their assignments are sorted like the others, their tiles are marked as holding nothing.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ perm, int32_t* __restrict__ tile_expert,
                int32_t* __restrict__ tile_row0, int32_t* __restrict__ tile_rows, int A, int experts, int tile,
                int max_tiles, int32_t* __restrict__ place, int real) {
    pdl_wait();
    __shared__ int count[ROUTER_MAX_EXPERTS], start[ROUTER_MAX_EXPERTS], first_tile[ROUTER_MAX_EXPERTS + 1];
    const int tid = threadIdx.x;
    for (int e = tid; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int a = tid; a < A; a += blockDim.x) atomicAdd(&count[ids[a]], 1);
    __syncthreads();
    if (tid == 0) {
        int rows = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = rows;
            first_tile[e] = tiles;
            rows += count[e];
            tiles += (count[e] + tile - 1) / tile;
        }
        first_tile[experts] = tiles;
    }
    __syncthreads();
    for (int e = tid; e < experts; e += blockDim.x) {
        const int n = count[e];
        for (int i = 0; i * tile < n; ++i) {
            const int at = first_tile[e] + i;
            tile_expert[at] = e < real ? e : -1;  // an expert without weights: its rows keep their places, no product runs
            tile_row0[at] = start[e] + i * tile;
            tile_rows[at] = min(tile, n - i * tile);
        }
        count[e] = 0;  // from here on: places handed out
    }
    for (int i = first_tile[experts] + tid; i < max_tiles; i += blockDim.x) {
        tile_expert[i] = -1;
        tile_row0[i] = 0;
        tile_rows[i] = 0;
    }
    __syncthreads();
    for (int a = tid; a < A; a += blockDim.x) {
        const int e = ids[a];
        const int at = start[e] + atomicAdd(&count[e], 1);
        perm[at] = a;
        if (place) place[a] = at;  // the inverse: where assignment a stands in sorted order
    }
}

extern "C" int ss_moe_plan(const int32_t* ids, int32_t* perm, int32_t* tile_expert, int32_t* tile_row0, int32_t* tile_rows,
                           int A, int experts, int tile, int max_tiles, int32_t* place, cudaStream_t stream, int real) {
    if (A <= 0) return 0;
    if (experts < 1 || experts > ROUTER_MAX_EXPERTS || tile < 1 || max_tiles < (A + tile - 1) / tile + experts)
        return (int)cudaErrorInvalidValue;
    ss_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, ids, perm, tile_expert, tile_row0, tile_rows, A, experts, tile,
              max_tiles, place, real > 0 ? real : experts);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- grouped products on CUDA cores
//
// UP:   hidden[s][n] = silu(g) * u,  g = sum_k a_k Wgu[e][n][k],  u = sum_k a_k Wgu[e][ff + n][k],
//       a = round_T(w[perm[s]] * x[perm[s] / top])   (the weight is on the expert's input; no weights: a = x)
// DOWN: y[perm[s]][n] = sum_k hidden[s][k] Wd[e][n][k]   (float32 out, one row per assignment)
// `single` (with the DOWN form, for experts without a gate branch): hidden[s][n] = relu(z)^2, z = sum_k a_k W[e][n][k]
// for the rows s of the plan's tile blockIdx.x (expert e) and the 64 columns n of blockIdx.y.  float32
// accumulation in a fixed order.
__device__ __forceinline__ float relu_square(float z) { return z > 0.f ? z * z : 0.f; }
#define MG_M 64
#define MG_N 64
#define MG_K 16
template <typename T, bool UP>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ x, const float* __restrict__ weights, const T* __restrict__ W,
                const int32_t* __restrict__ perm, const int32_t* __restrict__ tile_expert,
                const int32_t* __restrict__ tile_row0, const int32_t* __restrict__ tile_rows, T* __restrict__ hidden,
                float* __restrict__ y, int top, int K, int n_out, int run, int single) {
    pdl_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int row0 = tile_row0[blockIdx.x], rows = tile_rows[blockIdx.x];
    const bool first = UP || single;  // the product that reads the tokens' rows and writes the hidden rows
    __shared__ float As[MG_K][MG_M + 4];
    __shared__ float Ws[UP ? 2 : 1][MG_K][MG_N + 4];
    __shared__ int src_row[MG_M];
    __shared__ float src_w[MG_M];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.y * MG_N;
    if (tid < MG_M) {
        const int a = tid < rows ? perm[row0 + tid] : -1;
        src_row[tid] = a;
        src_w[tid] = (first && a >= 0 && weights) ? weights[a] : 1.f;
    }
    __syncthreads();
    // UP: W is [experts][2 n_out][K]; DOWN: [experts][n_out][K]
    const T* We = W + (int64_t)e * (UP ? 2 : 1) * n_out * K;
    float acc[UP ? 2 : 1][4][4];
#pragma unroll
    for (int u = 0; u < (UP ? 2 : 1); ++u)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[u][i][j] = 0.f;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += MG_K) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            float a = 0.f;
            if (lr < rows && k < K) {
                if (first) a = to_float(from_float<T>(src_w[lr] * to_float(x[(int64_t)(src_row[lr] / top) * K + k])));
                else a = to_float(x[(int64_t)(row0 + lr) * K + k]);
            }
            As[lk + q][lr] = a;
            const int wn = n0 + lr;
            // UP: gate and up rows alternate in runs of `run` (run = n_out: all gate rows, then all up rows)
            const int64_t wrow = UP ? (int64_t)(wn / run) * 2 * run + wn % run : wn;
            Ws[0][lk + q][lr] = (wn < n_out && k < K) ? to_float(We[wrow * K + k]) : 0.f;
            if (UP) Ws[1][lk + q][lr] = (wn < n_out && k < K) ? to_float(We[(wrow + run) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MG_K; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int u = 0; u < (UP ? 2 : 1); ++u) {
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] = Ws[u][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[u][i][j] = fmaf(a[i], w[j], acc[u][i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = ty * 4 + i;
        if (m >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= n_out) continue;
            if (UP) hidden[(int64_t)(row0 + m) * n_out + n] = from_float<T>(silu_mul<false>(acc[0][i][j], acc[UP ? 1 : 0][i][j]));
            else if (single) hidden[(int64_t)(row0 + m) * n_out + n] = from_float<T>(relu_square(acc[0][i][j]));
            else y[(int64_t)src_row[m] * n_out + n] = acc[0][i][j];
        }
    }
}

extern "C" int ss_moe_gemm(const void* x, const float* weights, const void* W, const int32_t* perm,
                           const int32_t* tile_expert, const int32_t* tile_row0, const int32_t* tile_rows, void* hidden,
                           float* y, int top, int K, int n_out, int max_tiles, int up, int dtype, int run, cudaStream_t stream,
                           int single) {
    if (max_tiles <= 0) return 0;
    if (up && (run < 1 || n_out % run)) return (int)cudaErrorInvalidValue;
    if (single && (up || !hidden)) return (int)cudaErrorInvalidValue;
    const dim3 grid(max_tiles, (n_out + MG_N - 1) / MG_N);
#define MG_GO(T, UP)                                                                                                    \
    ss_launch(moe_gemm_kernel<T, UP>, grid, dim3(256), 0, stream, (const T*)x, weights, (const T*)W, perm, tile_expert,       \
              tile_row0, tile_rows, (T*)hidden, y, top, K, n_out, run, single)
    if (dtype == SS_BF16) { if (up) MG_GO(bf16, true); else MG_GO(bf16, false); }
    else { if (up) MG_GO(float, true); else MG_GO(float, false); }
#undef MG_GO
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- grouped products on the tensor cores (bfloat16)
//
// The same two products with mma.sync.m16n8k16 tiles fed by ldmatrix from a three-stage cp.async ring.  The rows of an
// expert are contiguous in sorted order, so the activations are first gathered into that order (and, for the up
// product, multiplied by the router's score and rounded) by moe_gather_kernel; a block then takes one tile of BM
// sorted rows (the plan's tile size) and 64 output columns: for UP the 64 gate rows and the 64 matching up rows of
// the expert's stacked weight, whose accumulators meet in the epilogue as silu(g) * u.  K and n_out are multiples of 8.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool on) {
    const int bytes = on ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void ldsm_x4(uint32_t r[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// sorted[s][k] = round(w[perm[s]] * x[perm[s] / top][k]) for the `total` assignments (8 elements a thread).
__global__ void moe_gather_kernel(const bf16* __restrict__ x, const float* __restrict__ weights,
                                  const int32_t* __restrict__ perm, bf16* __restrict__ sorted, int total, int top, int K) {
    pdl_wait();
    const int chunks = K / 8;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)total * chunks) return;
    const int s = (int)(idx / chunks), c = (int)(idx - (int64_t)s * chunks);
    const int a = perm[s];
    const float w = weights ? weights[a] : 1.f;
    const uint4 raw = *reinterpret_cast<const uint4*>(x + (int64_t)(a / top) * K + c * 8);
    const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t out[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&in[e]);
        const __nv_bfloat162 r = __floats2bfloat162_rn(w * __low2float(v), w * __high2float(v));
        out[e] = *reinterpret_cast<const uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(sorted + (int64_t)s * K + c * 8) = make_uint4(out[0], out[1], out[2], out[3]);
}

// MM_BK: columns of K a stage holds; MM_STAGES: stages of the ring.  Tiles of few rows (decode steps) stream an
// expert's weights once and are bound by the bytes in flight: deeper and wider stages; tiles of 128 rows are bound by
// the tensor pipe and keep more blocks on an SM with smaller ones.
template <int BM, bool UP, int MM_BK, int MM_STAGES>
constexpr int moe_mma_smem() { return MM_STAGES * (BM + (UP ? 128 : 64)) * (MM_BK + 8) * 2; }

template <int BM, int WARPS_M, bool UP, int MM_BK, int MM_STAGES>
__global__ void __launch_bounds__(256)
moe_gemm_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, const int32_t* __restrict__ perm,
                    const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ tile_row0,
                    const int32_t* __restrict__ tile_rows, bf16* __restrict__ hidden, float* __restrict__ y, int K,
                    int n_out, int run) {
    constexpr int WARPS_N = 8 / WARPS_M, TM = BM / WARPS_M, TN = 64 / WARPS_N, MT = TM / 16, NT = TN / 8;
    constexpr int NB = UP ? 128 : 64, U = UP ? 2 : 1, MM_STR = MM_BK + 8, CPR = MM_BK / 8;  // 16-byte chunks a row
    static_assert(TM % 16 == 0 && TN % 16 == 0, "a warp's tile is whole m16 x n16 pieces");
    pdl_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int row0 = tile_row0[blockIdx.x], rows = tile_rows[blockIdx.x], n0 = blockIdx.y * 64;
    extern __shared__ __align__(16) unsigned char mm_raw[];
    bf16* As = reinterpret_cast<bf16*>(mm_raw);                 // [stage][BM][MM_STR]
    bf16* Bs = As + MM_STAGES * BM * MM_STR;                    // [stage][NB][MM_STR]
    const bf16* We = W + (int64_t)e * U * n_out * K;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WARPS_N, wn = warp % WARPS_N;

    auto load_stage = [&](int stage, int k0) {
        bf16* as = As + stage * BM * MM_STR;
        bf16* bs = Bs + stage * NB * MM_STR;
        for (int c = tid; c < BM * CPR; c += 256) {
            const int r = c / CPR, kc = (c % CPR) * 8;
            const bool on = r < rows && k0 + kc < K;
            cp_async_16(as + r * MM_STR + kc, A + (on ? (int64_t)(row0 + r) * K + k0 + kc : 0), on);
        }
        for (int c = tid; c < NB * CPR; c += 256) {
            const int r = c / CPR, kc = (c % CPR) * 8;
            const int n = n0 + (r & 63);
            const bool on = n < n_out && k0 + kc < K;
            // UP: gate and up rows alternate in runs of `run`; rows 0..63 of the tile are gate rows, 64..127 the up rows
            const int64_t wrow = UP ? (int64_t)(n / run) * 2 * run + n % run + (r >= 64 ? run : 0) : n;
            cp_async_16(bs + r * MM_STR + kc, We + (on ? wrow * K + k0 + kc : 0), on);
        }
    };

    float acc[U][MT][NT][4];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j) acc[u][i][j][0] = acc[u][i][j][1] = acc[u][i][j][2] = acc[u][i][j][3] = 0.f;

    const int k_steps = (K + MM_BK - 1) / MM_BK;
#pragma unroll
    for (int s = 0; s < MM_STAGES - 1; ++s) {
        if (s < k_steps) load_stage(s, s * MM_BK);
        cp_async_commit();
    }
    for (int ks = 0; ks < k_steps; ++ks) {
        cp_async_wait<MM_STAGES - 2>();
        __syncthreads();
        if (ks + MM_STAGES - 1 < k_steps) load_stage((ks + MM_STAGES - 1) % MM_STAGES, (ks + MM_STAGES - 1) * MM_BK);
        cp_async_commit();
        const bf16* as = As + (ks % MM_STAGES) * BM * MM_STR;
        const bf16* bs = Bs + (ks % MM_STAGES) * NB * MM_STR;
#pragma unroll
        for (int kk = 0; kk < MM_BK; kk += 16) {
            uint32_t af[MT][4];
#pragma unroll
            for (int i = 0; i < MT; ++i)
                ldsm_x4(af[i], as + (wm * TM + i * 16 + (lane & 15)) * MM_STR + kk + ((lane >> 4) << 3));
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    uint32_t b[4];
                    const int brow = u * 64 + wn * TN + j * 8 + (lane & 7) + ((lane >> 4) << 3);
                    ldsm_x4(b, bs + brow * MM_STR + kk + (((lane >> 3) & 1) << 3));
#pragma unroll
                    for (int i = 0; i < MT; ++i) {
                        mma_16816(acc[u][i][j], af[i], b[0], b[1]);
                        mma_16816(acc[u][i][j + 1], af[i], b[2], b[3]);
                    }
                }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = wm * TM + i * 16 + (lane >> 2) + half * 8;
            if (m >= rows) continue;
            const bool squared = !UP && hidden != nullptr;  // an expert without a gate branch: relu(z)^2 into the hidden rows
            const int64_t out_row = (UP || squared) ? (int64_t)(row0 + m) : (int64_t)perm[row0 + m];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int n = n0 + wn * TN + j * 8 + ((lane & 3) << 1);
                if (n >= n_out) continue;  // n_out is even: a pair is in or out together
                if (UP) {
                    const float h0 = silu_mul<true>(acc[0][i][j][half * 2], acc[U - 1][i][j][half * 2]);
                    const float h1 = silu_mul<true>(acc[0][i][j][half * 2 + 1], acc[U - 1][i][j][half * 2 + 1]);
                    *reinterpret_cast<__nv_bfloat162*>(hidden + out_row * n_out + n) = __floats2bfloat162_rn(h0, h1);
                } else if (squared) {
                    *reinterpret_cast<__nv_bfloat162*>(hidden + out_row * n_out + n) =
                        __floats2bfloat162_rn(relu_square(acc[0][i][j][half * 2]), relu_square(acc[0][i][j][half * 2 + 1]));
                } else {
                    *reinterpret_cast<float2*>(y + out_row * n_out + n) = make_float2(acc[0][i][j][half * 2], acc[0][i][j][half * 2 + 1]);
                }
            }
        }
}

template <int BM, int WARPS_M, bool UP, int MM_BK, int MM_STAGES>
static int launch_moe_mma(const void* A, const void* W, const int32_t* perm, const int32_t* tile_expert,
                          const int32_t* tile_row0, const int32_t* tile_rows, void* hidden, float* y, int K, int n_out,
                          int max_tiles, int run, cudaStream_t stream) {
    constexpr int smem = moe_mma_smem<BM, UP, MM_BK, MM_STAGES>();
    static SsPerDevice opted;
    if (int rc = ss_opt_in_smem(moe_gemm_mma_kernel<BM, WARPS_M, UP, MM_BK, MM_STAGES>, smem, opted)) return rc;
    ss_launch(moe_gemm_mma_kernel<BM, WARPS_M, UP, MM_BK, MM_STAGES>, dim3(max_tiles, (n_out + 63) / 64), dim3(256), smem, stream,
              (const bf16*)A, (const bf16*)W, perm, tile_expert, tile_row0, tile_rows, (bf16*)hidden, y, K, n_out, run);
    return SS_LAUNCH_CHECK();
}

// tile: the plan's tile size, 128 or 32.  up: A is the gathered activations, the output the hidden rows; else A the
// hidden rows and the output one float32 row per assignment.
extern "C" int ss_moe_gemm_mma(const void* A, const void* W, const int32_t* perm, const int32_t* tile_expert,
                               const int32_t* tile_row0, const int32_t* tile_rows, void* hidden, float* y, int K, int n_out,
                               int max_tiles, int tile, int up, int run, int wide_stages, cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    if (up && (run < 1 || n_out % run)) return (int)cudaErrorInvalidValue;
    if (K % 8 || n_out % 8 || (tile != 128 && tile != 32) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15))
        return (int)cudaErrorInvalidValue;
    if (tile == 128)
        return up ? launch_moe_mma<128, 4, true, 32, 3>(A, W, perm, tile_expert, tile_row0, tile_rows, hidden, y, K, n_out, max_tiles, run, stream)
                  : launch_moe_mma<128, 4, false, 32, 3>(A, W, perm, tile_expert, tile_row0, tile_rows, hidden, y, K, n_out, max_tiles, run, stream);
    // few pairs (one or two requests) touch few experts, whose few blocks want as many bytes in flight each as they can
    // hold: 128-wide stages (2 experts: 97 against 160 us); more experts fill the SMs with blocks of 64-wide stages
    // (6 experts: 180 against 204 us)
    if (wide_stages)
        return up ? launch_moe_mma<32, 2, true, 128, 3>(A, W, perm, tile_expert, tile_row0, tile_rows, hidden, y, K, n_out, max_tiles, run, stream)
                  : launch_moe_mma<32, 2, false, 128, 3>(A, W, perm, tile_expert, tile_row0, tile_rows, hidden, y, K, n_out, max_tiles, run, stream);
    return up ? launch_moe_mma<32, 2, true, 64, 3>(A, W, perm, tile_expert, tile_row0, tile_rows, hidden, y, K, n_out, max_tiles, run, stream)
              : launch_moe_mma<32, 2, false, 64, 4>(A, W, perm, tile_expert, tile_row0, tile_rows, hidden, y, K, n_out, max_tiles, run, stream);
}

extern "C" int ss_moe_gather(const void* x, const float* weights, const int32_t* perm, void* sorted, int total, int top,
                             int K, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (K % 8) return (int)cudaErrorInvalidValue;
    const int64_t n = (int64_t)total * (K / 8);
    ss_launch(moe_gather_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const bf16*)x, weights, perm,
              (bf16*)sorted, total, top, K);
    return SS_LAUNCH_CHECK();
}

// out[t][i] = round_T(sum_k y[t * top + k][i] + shared[t][i]): the chosen experts' outputs in the order of the
// choices, then the shared expert's.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ shared, T* __restrict__ out,
                                   int64_t n, int hidden, int top, const bf16* __restrict__ sorted,
                                   const int32_t* __restrict__ place) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int64_t t = idx / hidden;
    const int i = (int)(idx - t * hidden);
    float v = 0.f;
    for (int k = 0; k < top; ++k)  // float32 rows in the order of the choices, or bfloat16 rows in sorted order
        v += sorted ? to_float(sorted[(int64_t)place[t * top + k] * hidden + i]) : y[(t * top + k) * hidden + i];
    if (shared) v += to_float(shared[idx]);
    out[idx] = from_float<T>(v);
}

extern "C" int ss_moe_combine(const float* y, const void* shared, void* out, int n_tokens, int hidden, int top, int dtype,
                              const void* sorted, const int32_t* place, cudaStream_t stream) {
    const int64_t n = (int64_t)n_tokens * hidden;
    if (n <= 0) return 0;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == SS_BF16)
        ss_launch(moe_combine_kernel<bf16>, grid, dim3(256), 0, stream, y, (const bf16*)shared, (bf16*)out, n, hidden, top, (const bf16*)sorted, place);
    else
        ss_launch(moe_combine_kernel<float>, grid, dim3(256), 0, stream, y, (const float*)shared, (float*)out, n, hidden, top, (const bf16*)nullptr, (const int32_t*)nullptr);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- query/key norm, rotation of q, k and v, page write
//
// A token's row holds n_q query heads, n_kv key heads and n_kv value heads of D elements.  Queries and keys: an
// RMS norm over the head's first norm_dim elements with a weight shared by all heads (q_weight / k_weight, float32
// [norm_dim]; norm_dim 0: none), then the rotation of the first rot_dim elements by position * inv_freq[i].
// Values (v_rot_dim > 0): the first v_rot_dim elements rotated by position * v_inv_freq[m].  Pairs are (i, i + dims/2)
// or, `interleaved`, (2i, 2i + 1).  Queries are written in place, keys and values to their page (in place when the
// token has no slot).  A warp per head.  kv: [page][2][kv head][offset][D].
template <typename T>
__global__ void __launch_bounds__(256)
norm_rope_cache_kernel(T* __restrict__ rows, int64_t row_stride, const int32_t* __restrict__ positions,
                       const int32_t* __restrict__ slots, const float* __restrict__ inv_freq,
                       const float* __restrict__ v_inv_freq, const float* __restrict__ q_weight,
                       const float* __restrict__ k_weight, T* __restrict__ kv, int n_q, int n_kv, int D, int rot_dim,
                       int v_rot_dim, int interleaved, int norm_dim, float eps, int page_size, int64_t pool_slots,
                       int* err) {
    pdl_wait();
    __shared__ float cos_s[128], sin_s[128], vcos_s[128], vsin_s[128];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < rot_dim / 2; i += blockDim.x) sincosf(__fmul_rn(pos, inv_freq[i]), &sin_s[i], &cos_s[i]);
    for (int i = threadIdx.x; i < v_rot_dim / 2; i += blockDim.x) sincosf(__fmul_rn(pos, v_inv_freq[i]), &vsin_s[i], &vcos_s[i]);
    int64_t slot = (slots && kv) ? (int64_t)slots[t] : -1;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        slot = -1;
    }
    const int64_t page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? (int)(slot % page_size) : 0;
    __syncthreads();
    for (int h = blockIdx.y * n_warps + warp; h < n_q + 2 * n_kv; h += gridDim.y * n_warps) {
        T* src = rows + (int64_t)t * row_stride + (int64_t)h * D;
        const bool is_v = h >= n_q + n_kv, is_k = !is_v && h >= n_q;
        T* dst = src;
        if (slot >= 0 && is_k) dst = kv + ((((page * 2 + 0) * n_kv + (h - n_q)) * page_size + off) * (int64_t)D);
        if (slot >= 0 && is_v) dst = kv + ((((page * 2 + 1) * n_kv + (h - n_q - n_kv)) * page_size + off) * (int64_t)D);
        const int dims = is_v ? v_rot_dim : rot_dim, half = dims >> 1;
        const float* cs = is_v ? vcos_s : cos_s;
        const float* sn = is_v ? vsin_s : sin_s;
        const bool normed = !is_v && norm_dim > 0;
        const float* w = is_k ? k_weight : q_weight;
        // a lane holds up to 4 rotated pairs (u, v) and up to 8 elements behind the rotated part
        constexpr int PPL = 4, TPL = 8;
        float u[PPL], v[PPL], tail[TPL];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < PPL; ++c) {
            const int i = lane + 32 * c;
            u[c] = v[c] = 0.f;
            if (i < half) {
                const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
                u[c] = to_float(src[iu]);
                v[c] = to_float(src[iv]);
                if (iu < norm_dim) ss = fmaf(u[c], u[c], ss);
                if (iv < norm_dim) ss = fmaf(v[c], v[c], ss);
            }
        }
#pragma unroll
        for (int c = 0; c < TPL; ++c) {
            const int d = dims + lane + 32 * c;
            tail[c] = d < D ? to_float(src[d]) : 0.f;
            if (d < norm_dim) ss = fmaf(tail[c], tail[c], ss);
        }
        float rstd = 1.f;
        if (normed) rstd = 1.0f / sqrtf(warp_sum(ss) / (float)norm_dim + eps);
#pragma unroll
        for (int c = 0; c < PPL; ++c) {
            const int i = lane + 32 * c;
            if (i >= half) break;
            const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
            float a = u[c], b = v[c];
            if (normed) {
                a = iu < norm_dim ? a * rstd * w[iu] : 0.f;
                b = iv < norm_dim ? b * rstd * w[iv] : 0.f;
            }
            // (u, v) -> (u c - v s, v c + u s)
            dst[iu] = from_float<T>(__fadd_rn(__fmul_rn(a, cs[i]), __fmul_rn(-b, sn[i])));
            dst[iv] = from_float<T>(__fadd_rn(__fmul_rn(b, cs[i]), __fmul_rn(a, sn[i])));
        }
#pragma unroll
        for (int c = 0; c < TPL; ++c) {
            const int d = dims + lane + 32 * c;
            if (d >= D) break;
            float a = tail[c];
            if (normed) a = d < norm_dim ? a * rstd * w[d] : 0.f;
            dst[d] = from_float<T>(a);
        }
    }
}

// The same for bfloat16 heads that are rotated whole in half-split pairs (rot_dim = D, values rotated whole or not
// at all, the norm over the whole head or none, D a multiple of 16): LPH = D / 16 lanes share a head, each with 8
// elements of the first half and the 8 they pair with, 16 bytes a load and a store.  A block per token.
template <int LPH>
__global__ void __launch_bounds__(256)
norm_rope_cache_bf16x8_kernel(bf16* __restrict__ rows, int64_t row_stride, const int32_t* __restrict__ positions,
                              const int32_t* __restrict__ slots, const float* __restrict__ inv_freq,
                              const float* __restrict__ v_inv_freq, const float* __restrict__ q_weight,
                              const float* __restrict__ k_weight, bf16* __restrict__ kv, int n_q, int n_kv, int D,
                              int rotate_v, int normed, float eps, int page_size, int64_t pool_slots, int* err) {
    pdl_wait();
    __shared__ float cos_s[128], sin_s[128], vcos_s[128], vsin_s[128];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int half = D >> 1;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        sincosf(__fmul_rn(pos, inv_freq[i]), &sin_s[i], &cos_s[i]);
        if (rotate_v) sincosf(__fmul_rn(pos, v_inv_freq[i]), &vsin_s[i], &vcos_s[i]);
    }
    int64_t slot = (slots && kv) ? (int64_t)slots[t] : -1;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        slot = -1;
    }
    const int64_t page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? (int)(slot % page_size) : 0;
    bf16* row = rows + (int64_t)t * row_stride;
    __syncthreads();
    constexpr int HPW = 32 / LPH;
    const int sub = lane / LPH, l = lane % LPH;
    const int heads = n_q + 2 * n_kv;
    for (int hb = warp * HPW; hb < heads; hb += n_warps * HPW) {  // the same trips for every lane of a warp (shuffles below)
        const int h = hb + sub;
        const bool on = h < heads;
        const bool is_v = h >= n_q + n_kv, is_k = !is_v && h >= n_q;
        float u[8], v[8];
        float ss = 0.f;
        if (on) {
            const uint4 ru = *reinterpret_cast<const uint4*>(row + (int64_t)h * D + 8 * l);
            const uint4 rv = *reinterpret_cast<const uint4*>(row + (int64_t)h * D + half + 8 * l);
            const uint32_t wu[4] = {ru.x, ru.y, ru.z, ru.w}, wv[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                u[2 * e] = __uint_as_float(wu[e] << 16); u[2 * e + 1] = __uint_as_float(wu[e] & 0xffff0000u);
                v[2 * e] = __uint_as_float(wv[e] << 16); v[2 * e + 1] = __uint_as_float(wv[e] & 0xffff0000u);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(u[e], u[e], fmaf(v[e], v[e], ss));
        }
        if (normed) {  // the whole warp takes part in the shuffles
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        }
        if (!on) continue;
        if (normed && !is_v) {
            const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
            const float* w = is_k ? k_weight : q_weight;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                u[e] = u[e] * rstd * w[8 * l + e];
                v[e] = v[e] * rstd * w[half + 8 * l + e];
            }
        }
        if (!is_v || rotate_v) {
            const float* cs = is_v ? vcos_s : cos_s;
            const float* sn = is_v ? vsin_s : sin_s;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float c = cs[8 * l + e], s_ = sn[8 * l + e];
                const float a = u[e], b = v[e];
                u[e] = __fadd_rn(__fmul_rn(a, c), __fmul_rn(-b, s_));
                v[e] = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s_));
            }
        }
        bf16* dst = row + (int64_t)h * D;
        if (slot >= 0 && is_k) dst = kv + ((((page * 2 + 0) * n_kv + (h - n_q)) * page_size + off) * (int64_t)D);
        if (slot >= 0 && is_v) dst = kv + ((((page * 2 + 1) * n_kv + (h - n_q - n_kv)) * page_size + off) * (int64_t)D);
        uint32_t ou[4], ov[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 a = __floats2bfloat162_rn(u[2 * e], u[2 * e + 1]), b = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
            ou[e] = *reinterpret_cast<const uint32_t*>(&a);
            ov[e] = *reinterpret_cast<const uint32_t*>(&b);
        }
        *reinterpret_cast<uint4*>(dst + 8 * l) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
        *reinterpret_cast<uint4*>(dst + half + 8 * l) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
    }
}

extern "C" int ss_norm_rope_cache(void* rows, int64_t row_stride, const int32_t* positions, const int32_t* slots,
                                  const float* inv_freq, const float* v_inv_freq, const float* q_weight,
                                  const float* k_weight, void* kv, int n_tokens, int n_q, int n_kv, int D, int rot_dim,
                                  int v_rot_dim, int interleaved, int norm_dim, float eps, int page_size,
                                  int64_t num_pages, int dtype, int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D < 2 || D > 256 || rot_dim < 0 || rot_dim > D || rot_dim % 2 || v_rot_dim < 0 || v_rot_dim > D || v_rot_dim % 2 ||
        norm_dim < 0 || norm_dim > D || (rot_dim > 0 && !inv_freq) || (v_rot_dim > 0 && !v_inv_freq) ||
        (norm_dim > 0 && (!q_weight || (n_kv > 0 && !k_weight))))
        return (int)cudaErrorInvalidValue;
    const int heads = n_q + 2 * n_kv;
    const int warps = heads >= 8 ? 8 : (heads >= 4 ? 4 : 2);
    const dim3 grid(n_tokens, (heads + warps - 1) / warps);
    const int64_t pool = num_pages * page_size;
    if (dtype == SS_BF16 && !interleaved && D % 16 == 0 && rot_dim == D && (v_rot_dim == 0 || v_rot_dim == D) &&
        (norm_dim == 0 || norm_dim == D) && row_stride % 8 == 0 && ((uintptr_t)rows & 15) == 0 && ((uintptr_t)kv & 15) == 0) {
        const int lph = D / 16;  // 1 .. 16 lanes a head; the kernel takes powers of two
#define NR8_GO(LPH)                                                                                                     \
    ss_launch(norm_rope_cache_bf16x8_kernel<LPH>, dim3(n_tokens), dim3(256), 0, stream, (bf16*)rows, row_stride, positions,   \
              slots, inv_freq, v_inv_freq, q_weight, k_weight, (bf16*)kv, n_q, n_kv, D, (int)(v_rot_dim == D),            \
              (int)(norm_dim == D), eps, page_size, pool, err)
        if (lph == 1) { NR8_GO(1); return SS_LAUNCH_CHECK(); }
        if (lph == 2) { NR8_GO(2); return SS_LAUNCH_CHECK(); }
        if (lph == 4) { NR8_GO(4); return SS_LAUNCH_CHECK(); }
        if (lph == 8) { NR8_GO(8); return SS_LAUNCH_CHECK(); }
        if (lph == 16) { NR8_GO(16); return SS_LAUNCH_CHECK(); }
#undef NR8_GO
    }
    if (dtype == SS_BF16)
        ss_launch(norm_rope_cache_kernel<bf16>, grid, dim3(warps * 32), 0, stream, (bf16*)rows, row_stride, positions, slots,
                  inv_freq, v_inv_freq, q_weight, k_weight, (bf16*)kv, n_q, n_kv, D, rot_dim, v_rot_dim, interleaved,
                  norm_dim, eps, page_size, pool, err);
    else
        ss_launch(norm_rope_cache_kernel<float>, grid, dim3(warps * 32), 0, stream, (float*)rows, row_stride, positions,
                  slots, inv_freq, v_inv_freq, q_weight, k_weight, (float*)kv, n_q, n_kv, D, rot_dim, v_rot_dim, interleaved,
                  norm_dim, eps, page_size, pool, err);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- turning the heads' outputs back
//
// x: [tokens][heads * D] in place; the first `dims` elements of every head are rotated by sign * position *
// inv_freq[m], pairs as above.  A thread per pair.
template <typename T>
__global__ void turn_heads_kernel(T* __restrict__ x, const int32_t* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int64_t n_pairs, int heads, int D, int dims,
                                  int interleaved, float sign) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_pairs) return;
    const int half = dims >> 1;
    const int m = (int)(idx % half);
    const int64_t th = idx / half;  // token * heads + head
    const int64_t t = th / heads;
    float sn, cs;
    sincosf(__fmul_rn((float)positions[t], inv_freq[m]), &sn, &cs);
    sn *= sign;
    T* head = x + th * D;
    const int i0 = interleaved ? 2 * m : m, i1 = interleaved ? 2 * m + 1 : m + half;
    const float u = to_float(head[i0]), v = to_float(head[i1]);
    head[i0] = from_float<T>(__fadd_rn(__fmul_rn(u, cs), __fmul_rn(-v, sn)));
    head[i1] = from_float<T>(__fadd_rn(__fmul_rn(v, cs), __fmul_rn(u, sn)));
}

extern "C" int ss_turn_heads(void* x, const int32_t* positions, const float* inv_freq, int n_tokens, int heads, int D,
                             int dims, int interleaved, float sign, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || dims <= 0) return 0;
    if (dims % 2 || dims > D) return (int)cudaErrorInvalidValue;
    const int64_t n_pairs = (int64_t)n_tokens * heads * (dims / 2);
    const dim3 grid((unsigned)((n_pairs + 255) / 256));
    if (dtype == SS_BF16)
        ss_launch(turn_heads_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)x, positions, inv_freq, n_pairs, heads, D, dims,
                  interleaved, sign);
    else
        ss_launch(turn_heads_kernel<float>, grid, dim3(256), 0, stream, (float*)x, positions, inv_freq, n_pairs, heads, D,
                  dims, interleaved, sign);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- soft cap:  x <- cap * tanh(scale * x / cap)
// (cap 0: x <- scale * x)
__global__ void soft_cap_kernel(float* __restrict__ x, int64_t n, float cap, float scale) {
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i] * scale;
    x[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

extern "C" int ss_soft_cap(float* x, int64_t n, float cap, cudaStream_t stream, float scale) {
    if (n <= 0) return 0;
    ss_launch(soft_cap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, cap, scale);
    return SS_LAUNCH_CHECK();
}

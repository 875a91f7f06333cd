// Row-wise kernels for decoders that keep several residual streams and shape queries and keys after their
// rotation: the hyper-connection step (write a branch's output into the streams, read the next branch's input out
// of them, RMS norm) in one launch, rotation of neighbouring or half-split pairs with scaled sines, a unit RMS norm
// per head and the key/value page write in one launch, a gated linear unit with a steeper sigmoid and clamped
// inputs, and an element-wise sigmoid gate.  All sizes and constants are run-time parameters.  Everything the
// formulas below name is float32; inputs and outputs are float32 or bfloat16.

#include "common.cuh"

// None of these kernels lets the kernel behind it start early (griddepcontrol.launch_dependents): each is short, and
// with the early start a prompt step of 2,048 tokens at a width of 5,120 (every second launch a two-SM tcgen05
// product or the tcgen05 attention, which take tensor memory before they wait for the kernel in front) stopped
// making progress about three times in four; with the kernels of this file in stream order it did not in any run.
// They still wait for the kernel in front (griddepcontrol.wait), which may have started them early.

// ---------------------------------------------------------------- hyper-connections
//
// A token has S streams x_0 .. x_{S-1} of `hidden` floats (streams: [tokens][S][hidden]).  One launch does, per token,
//   write:  x_t <- sum_s mix[s][t] x_s + w_out[t] * y          (all t from the old streams; skipped when y is null;
//           with y2, two branches that read the same input, y stands for y + y2, added in float32)
//   read:   u = sum_t w_in[t] x_t
//   norm:   out = u / sqrt(mean(u^2) + eps) * weight            (rounded once, to the output type)
// With `rows`, output row i is token rows[i] and the streams stay as they are (the write is only applied on the way
// to u).  S = 1 with mix = out = in = 1 is the ordinary residual add in front of a norm.  A block per output row; a
// row is walked twice (the second walk re-reads what the first wrote, or repeats its arithmetic), so the additions
// behind one value never depend on the batch.
#define HC_MAX_STREAMS 8

template <typename T, int SMAX>
__global__ void hc_norm_kernel(float* __restrict__ streams, const T* __restrict__ y, const T* __restrict__ y2,
                               const float* __restrict__ mix,
                               const float* __restrict__ w_out, const float* __restrict__ w_in,
                               const void* __restrict__ weight, int w_f32, T* __restrict__ out,
                               const int32_t* __restrict__ rows, int S, int hidden, float eps) {
    // the connection weights are constants of the model: read before the wait for the kernel in front
    float m[SMAX][SMAX], wo[SMAX], wi[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
        wo[s] = (y != nullptr && s < S) ? w_out[s] : 0.f;
        wi[s] = s < S ? (w_in ? w_in[s] : 1.f) : 0.f;
#pragma unroll
        for (int t = 0; t < SMAX; ++t) m[s][t] = (y != nullptr && s < S && t < S) ? mix[s * S + t] : 0.f;
    }
    pdl_wait();
    __shared__ float scratch[33];
    const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* base = streams + src * (int64_t)S * hidden;
    const T* yr = y ? y + src * (int64_t)hidden : nullptr;
    const T* y2r = (y && y2) ? y2 + src * (int64_t)hidden : nullptr;  // a second output of the same branch point
    const bool write_back = rows == nullptr && y != nullptr;

    float ss = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float x[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) x[s] = s < S ? base[(int64_t)s * hidden + j] : 0.f;
        float u = 0.f;
        if (yr) {
            const float yv = y2r ? to_float(yr[j]) + to_float(y2r[j]) : to_float(yr[j]);
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
                if (t >= S) break;
                float v = __fmul_rn(wo[t], yv);
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) v = fmaf(m[s][t], x[s], v);
                if (write_back) base[(int64_t)t * hidden + j] = v;
                u = fmaf(wi[t], v, u);
            }
        } else {
#pragma unroll
            for (int t = 0; t < SMAX; ++t)
                if (t < S) u = fmaf(wi[t], x[t], u);
        }
        ss = fmaf(u, u, ss);
    }
    ss = block_sum(ss, scratch);  // its barriers also order the writes above before the reads below
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* o = out + (int64_t)blockIdx.x * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float x[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) x[s] = s < S ? base[(int64_t)s * hidden + j] : 0.f;
        float u = 0.f;
        if (yr && !write_back) {
            const float yv = y2r ? to_float(yr[j]) + to_float(y2r[j]) : to_float(yr[j]);
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
                if (t >= S) break;
                float v = __fmul_rn(wo[t], yv);
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) v = fmaf(m[s][t], x[s], v);
                u = fmaf(wi[t], v, u);
            }
        } else {
#pragma unroll
            for (int t = 0; t < SMAX; ++t)
                if (t < S) u = fmaf(wi[t], x[t], u);
        }
        o[j] = from_float<T>(u * rstd * load_vec<T>(weight, j, w_f32));
    }
}

// Four consecutive elements with one access.
__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ld4(const bf16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x), b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void st4(bf16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const uint32_t*>(&a);
    t.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}

// The same step with 16-byte accesses and the row walked ONCE (hidden a multiple of 4, at most 16 * blockDim): a
// thread keeps its up to NV groups of four values of u in registers between the sum of squares and the output.  The
// arithmetic behind every value is the kernel's above, operation for operation.
#define HC_NV 4
template <typename T, int SMAX>
__global__ void hc_norm_vec_kernel(float* __restrict__ streams, const T* __restrict__ y, const T* __restrict__ y2,
                                   const float* __restrict__ mix,
                                   const float* __restrict__ w_out, const float* __restrict__ w_in,
                                   const void* __restrict__ weight, int w_f32, T* __restrict__ out,
                                   const int32_t* __restrict__ rows, int S, int hidden, float eps) {
    float m[SMAX][SMAX], wo[SMAX], wi[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
        wo[s] = (y != nullptr && s < S) ? w_out[s] : 0.f;
        wi[s] = s < S ? (w_in ? w_in[s] : 1.f) : 0.f;
#pragma unroll
        for (int t = 0; t < SMAX; ++t) m[s][t] = (y != nullptr && s < S && t < S) ? mix[s * S + t] : 0.f;
    }
    pdl_wait();
    __shared__ float scratch[33];
    const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* base = streams + src * (int64_t)S * hidden;
    const T* yr = y ? y + src * (int64_t)hidden : nullptr;
    const T* y2r = (y && y2) ? y2 + src * (int64_t)hidden : nullptr;  // a second output of the same branch point
    const bool write_back = rows == nullptr && y != nullptr;
    float u[HC_NV][4];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < HC_NV; ++it) {
        const int j = (threadIdx.x + it * blockDim.x) * 4;
        if (j >= hidden) break;
        float x[SMAX][4];
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
            if (s < S) ld4(base + (int64_t)s * hidden + j, x[s]);
        u[it][0] = u[it][1] = u[it][2] = u[it][3] = 0.f;
        if (yr) {
            float yv[4];
            ld4(yr + j, yv);
            if (y2r) {
                float y2v[4];
                ld4(y2r + j, y2v);
#pragma unroll
                for (int e = 0; e < 4; ++e) yv[e] += y2v[e];
            }
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
                if (t >= S) break;
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = __fmul_rn(wo[t], yv[e]);
#pragma unroll
                for (int s = 0; s < SMAX; ++s) {
                    if (s < S) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = fmaf(m[s][t], x[s][e], v[e]);
                    }
                }
                if (write_back) st4(base + (int64_t)t * hidden + j, v);
#pragma unroll
                for (int e = 0; e < 4; ++e) u[it][e] = fmaf(wi[t], v[e], u[it][e]);
            }
        } else {
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
                if (t < S) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) u[it][e] = fmaf(wi[t], x[t][e], u[it][e]);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) ss = fmaf(u[it][e], u[it][e], ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* o = out + (int64_t)blockIdx.x * hidden;
#pragma unroll
    for (int it = 0; it < HC_NV; ++it) {
        const int j = (threadIdx.x + it * blockDim.x) * 4;
        if (j >= hidden) break;
        float r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) r[e] = u[it][e] * rstd * load_vec<T>(weight, j + e, w_f32);
        st4(o + j, r);
    }
}

template <typename T>
static int launch_hc_norm(float* streams, const void* y, const void* y2, const float* mix, const float* w_out, const float* w_in,
                          const void* weight, int w_f32, void* out, const int32_t* rows, int n_rows, int S, int hidden,
                          float eps, cudaStream_t stream) {
    if (hidden % 4 == 0 && hidden <= 16 * 512 && S <= 4) {
        int vthreads = ((hidden / 4 + HC_NV - 1) / HC_NV + 31) / 32 * 32;
        vthreads = vthreads < 64 ? 64 : vthreads;
#define HC_VEC(SMAX)                                                                                                     \
    ss_launch(hc_norm_vec_kernel<T, SMAX>, dim3(n_rows), dim3(vthreads), 0, stream, streams, (const T*)y, (const T*)y2, mix, w_out, w_in, \
              weight, w_f32, (T*)out, rows, S, hidden, eps)
        if (S == 1) HC_VEC(1);
        else if (S == 2) HC_VEC(2);
        else HC_VEC(4);
#undef HC_VEC
        return SS_LAUNCH_CHECK();
    }
    const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
#define HC_GO(SMAX)                                                                                                   \
    ss_launch(hc_norm_kernel<T, SMAX>, dim3(n_rows), dim3(threads), 0, stream, streams, (const T*)y, (const T*)y2, mix, w_out, w_in, \
              weight, w_f32, (T*)out, rows, S, hidden, eps)
    if (S == 1) HC_GO(1);
    else if (S == 2) HC_GO(2);
    else if (S <= 4) HC_GO(4);
    else HC_GO(HC_MAX_STREAMS);
#undef HC_GO
    return SS_LAUNCH_CHECK();
}

// streams: float32 [tokens][S][hidden]; y: [tokens][hidden] or null; mix [S][S] (from, to), w_out [S], w_in [S] (null:
// ones) float32 on the device; weight [hidden] in the output type or float32; rows: int32 [n_rows] or null.
extern "C" int ss_hc_norm(float* streams, const void* y, const float* mix, const float* w_out, const float* w_in,
                          const void* weight, int w_f32, void* out, const int32_t* rows, int n_rows, int S, int hidden,
                          float eps, int dtype, cudaStream_t stream, const void* y2) {
    if (n_rows <= 0) return 0;
    if (S < 1 || S > HC_MAX_STREAMS || (y != nullptr && (!mix || !w_out))) return (int)cudaErrorInvalidValue;
    if (dtype == SS_BF16)
        return launch_hc_norm<bf16>(streams, y, y2, mix, w_out, w_in, weight, w_f32, out, rows, n_rows, S, hidden, eps, stream);
    return launch_hc_norm<float>(streams, y, y2, mix, w_out, w_in, weight, w_f32, out, rows, n_rows, S, hidden, eps, stream);
}

// ---------------------------------------------------------------- rotation, unit norm, page write
//
// A token's row holds n_q query heads, then (has_kv) n_kv key heads and n_kv value heads, D elements each, at
// `row_stride` (even) elements from the next token's.  A warp takes one head at a time:
//   rotation of the first rot_dim elements by angle = position * inv_freq[i]:
//       pairs (2i, 2i+1) when `interleaved`, else (i, i + rot_dim/2);
//       (a, b) -> (a c - b s, b c + a s) with c = mscale cos(angle), s = mscale sin(angle);
//   then (norm_dim > 0) the head is divided by sqrt(sum(x^2) / norm_dim + eps): a unit RMS norm over the head's
//   norm_dim real elements (elements beyond them are padding and zero);
//   queries are written back in place, keys to their page (or in place when the token has no slot), values are
//   copied to their page as they are.
// kv layout: [page][2][kv head][offset in page][D].  D even, at most 256.
// Two neighbouring elements with one load or store.
__device__ __forceinline__ void load_pair(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
}
__device__ __forceinline__ void load_pair(const bf16* p, float& a, float& b) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
    a = __low2float(v); b = __high2float(v);
}
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// A block per token and group of heads (grid.y), a warp per head: every head's loads are in flight at once, and the
// token's sines and cosines are formed once per block.
template <typename T>
__global__ void __launch_bounds__(256)
rope_norm_cache_kernel(T* __restrict__ rows, int64_t row_stride, const int32_t* __restrict__ positions,
                       const int32_t* __restrict__ slots, const float* __restrict__ inv_freq, float mscale,
                       T* __restrict__ kv, int n_q, int n_kv, int D, int rot_dim, int interleaved, int norm_dim,
                       float eps, int page_size, int64_t pool_slots, int write_cache, int* err) {
    pdl_wait();
    __shared__ float cos_s[128], sin_s[128];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int half = rot_dim >> 1, pairs = D >> 1;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(__fmul_rn(pos, inv_freq[i]), &sn, &cs);
        sin_s[i] = sn * mscale;
        cos_s[i] = cs * mscale;
    }
    int64_t slot = (write_cache && slots) ? (int64_t)slots[t] : -1;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        slot = -1;
    }
    const int64_t page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? (int)(slot % page_size) : 0;
    __syncthreads();
    for (int h = blockIdx.y * n_warps + warp; h < n_q + 2 * n_kv; h += gridDim.y * n_warps) {
        T* src = rows + (int64_t)t * row_stride + (int64_t)h * D;
        if (h >= n_q + n_kv) {  // a value head: copied to its page as it is
            if (slot < 0) continue;
            T* dst = kv + ((((page * 2 + 1) * n_kv + (h - n_q - n_kv)) * page_size + off) * (int64_t)D);
            if ((D * sizeof(T)) % 16 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
                for (int c = lane; c < (int)(D * sizeof(T) / 16); c += 32)
                    reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
            } else {
                for (int d = lane; d < D; d += 32) dst[d] = src[d];
            }
            continue;
        }
        T* dst = (h < n_q || slot < 0) ? src : kv + ((((page * 2 + 0) * n_kv + (h - n_q)) * page_size + off) * (int64_t)D);
        constexpr int PPL = 4;  // pairs per lane: D <= 256
        float a[PPL], b[PPL];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < PPL; ++c) {
            const int p = lane + 32 * c;
            if (p >= pairs) break;
            float x1, x2;
            if (p < half && !interleaved) {  // element p with element p + rot_dim / 2
                x1 = to_float(src[p]);
                x2 = to_float(src[p + half]);
            } else {  // neighbours: a rotated pair (2p, 2p + 1), or two elements beyond the rotated part
                load_pair(src + (p < half ? 2 * p : rot_dim + 2 * (p - half)), x1, x2);
            }
            if (p < half) {
                const float cs = cos_s[p], sn = sin_s[p];
                const float r1 = __fadd_rn(__fmul_rn(x1, cs), __fmul_rn(-x2, sn));
                const float r2 = __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
                x1 = r1;
                x2 = r2;
            }
            a[c] = x1;
            b[c] = x2;
            ss = fmaf(x1, x1, ss);
            ss = fmaf(x2, x2, ss);
        }
        float scale = 1.f;
        if (norm_dim > 0) {
            ss = warp_sum(ss);
            scale = 1.0f / sqrtf(ss / (float)norm_dim + eps);
        }
#pragma unroll
        for (int c = 0; c < PPL; ++c) {
            const int p = lane + 32 * c;
            if (p >= pairs) break;
            if (p < half && !interleaved) {
                dst[p] = from_float<T>(a[c] * scale);
                dst[p + half] = from_float<T>(b[c] * scale);
            } else {
                store_pair(dst + (p < half ? 2 * p : rot_dim + 2 * (p - half)), a[c] * scale, b[c] * scale);
            }
        }
    }
}

// bfloat16 with 16-byte accesses (neighbouring pairs, D a multiple of 8, 16-byte aligned rows): LPH lanes share a
// head, 8 elements (4 pairs) each, so a warp holds 32 / LPH heads at a time and two such sets are in flight per
// thread; value heads are copied 16 bytes a thread.  A block per token.
template <int LPH>
__global__ void __launch_bounds__(256)
rope_norm_cache_bf16x8_kernel(bf16* __restrict__ rows, int64_t row_stride, const int32_t* __restrict__ positions,
                              const int32_t* __restrict__ slots, const float* __restrict__ inv_freq, float mscale,
                              bf16* __restrict__ kv, int n_q, int n_kv, int D, int rot_dim, int norm_dim, float eps,
                              int page_size, int64_t pool_slots, int write_cache, int* err) {
    pdl_wait();
    __shared__ float cos_s[128], sin_s[128];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int half = rot_dim >> 1;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(__fmul_rn(pos, inv_freq[i]), &sn, &cs);
        sin_s[i] = sn * mscale;
        cos_s[i] = cs * mscale;
    }
    int64_t slot = (write_cache && slots) ? (int64_t)slots[t] : -1;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        slot = -1;
    }
    const int64_t page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? (int)(slot % page_size) : 0;
    bf16* row = rows + (int64_t)t * row_stride;
    // values first: their copies are in flight while the sines are formed
    if (slot >= 0) {
        const int cpr = D / 8;
        for (int idx = threadIdx.x; idx < n_kv * cpr; idx += blockDim.x) {
            const int h = idx / cpr, c = idx - h * cpr;
            reinterpret_cast<uint4*>(kv + (((page * 2 + 1) * n_kv + h) * page_size + off) * (int64_t)D)[c] =
                reinterpret_cast<const uint4*>(row + (int64_t)(n_q + n_kv + h) * D)[c];
        }
    }
    __syncthreads();
    constexpr int HPW = 32 / LPH, U = 2;
    const int sub = lane / LPH, l = lane % LPH;
    const bool lane_on = l * 8 < D;
    const int heads = n_q + n_kv, stride = n_warps * HPW;
    for (int hb = warp * HPW; hb < heads; hb += stride * U) {  // the same trips for every lane of a warp (shuffles below)
        const int h0 = hb + sub;
        uint4 raw[U];
        bool on[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int h = h0 + u * stride;
            on[u] = lane_on && h < heads;
            if (on[u]) raw[u] = *reinterpret_cast<const uint4*>(row + (int64_t)h * D + l * 8);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int h = h0 + u * stride;
            float x[8];
            float ss = 0.f;
            if (on[u]) {
                const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
                    float x1 = __low2float(v), x2 = __high2float(v);
                    const int p = l * 4 + e;
                    if (p < half) {
                        const float cs = cos_s[p], sn = sin_s[p];
                        const float r1 = __fadd_rn(__fmul_rn(x1, cs), __fmul_rn(-x2, sn));
                        const float r2 = __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
                        x1 = r1;
                        x2 = r2;
                    }
                    x[2 * e] = x1;
                    x[2 * e + 1] = x2;
                    ss = fmaf(x1, x1, ss);
                    ss = fmaf(x2, x2, ss);
                }
            }
            float scale = 1.f;
            if (norm_dim > 0) {  // the whole warp takes part in the shuffles
#pragma unroll
                for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                scale = 1.0f / sqrtf(ss / (float)norm_dim + eps);
            }
            if (on[u]) {
                bf16* dst = (h < n_q || slot < 0) ? row + (int64_t)h * D
                                                  : kv + ((((page * 2 + 0) * n_kv + (h - n_q)) * page_size + off) * (int64_t)D);
                uint32_t o4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __nv_bfloat162 v = __floats2bfloat162_rn(x[2 * e] * scale, x[2 * e + 1] * scale);
                    o4[e] = *reinterpret_cast<const uint32_t*>(&v);
                }
                *reinterpret_cast<uint4*>(dst + l * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
        }
    }
}

extern "C" int ss_rope_norm_cache(void* rows, int64_t row_stride, const int32_t* positions, const int32_t* slots,
                                  const float* inv_freq, float mscale, void* kv, int n_tokens, int n_q, int n_kv,
                                  int D, int rot_dim, int interleaved, int norm_dim, float eps, int page_size,
                                  int64_t num_pages, int write_cache, int dtype, int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D < 2 || D > 256 || D % 2 || rot_dim < 0 || rot_dim > D || rot_dim % 2 || (rot_dim > 0 && !inv_freq) ||
        row_stride % 2 || ((uintptr_t)rows & 7) || ((uintptr_t)kv & 7))
        return (int)cudaErrorInvalidValue;
    const int heads = n_q + 2 * n_kv;
    const int warps = heads >= 8 ? 8 : (heads >= 4 ? 4 : 2);
    const dim3 grid(n_tokens, (heads + warps - 1) / warps);
    const int64_t pool = num_pages * page_size;
    if (dtype == SS_BF16 && (interleaved || rot_dim == 0) && D % 8 == 0 && row_stride % 8 == 0 && rot_dim <= 256 &&
        ((uintptr_t)rows & 15) == 0 && ((uintptr_t)kv & 15) == 0) {
        const int lph = D <= 32 ? 4 : (D <= 64 ? 8 : (D <= 128 ? 16 : 32));
#define RN_GO(LPH)                                                                                                      \
    ss_launch(rope_norm_cache_bf16x8_kernel<LPH>, dim3(n_tokens), dim3(256), 0, stream, (bf16*)rows, row_stride, positions, \
              slots, inv_freq, mscale, (bf16*)kv, n_q, n_kv, D, rot_dim, norm_dim, eps, page_size, pool, write_cache, err)
        if (lph == 4) RN_GO(4);
        else if (lph == 8) RN_GO(8);
        else if (lph == 16) RN_GO(16);
        else RN_GO(32);
#undef RN_GO
        return SS_LAUNCH_CHECK();
    }
    if (dtype == SS_BF16)
        ss_launch(rope_norm_cache_kernel<bf16>, grid, dim3(warps * 32), 0, stream, (bf16*)rows, row_stride,
                  positions, slots, inv_freq, mscale, (bf16*)kv, n_q, n_kv, D, rot_dim, interleaved, norm_dim, eps,
                  page_size, pool, write_cache, err);
    else
        ss_launch(rope_norm_cache_kernel<float>, grid, dim3(warps * 32), 0, stream, (float*)rows, row_stride,
                  positions, slots, inv_freq, mscale, (float*)kv, n_q, n_kv, D, rot_dim, interleaved, norm_dim, eps,
                  page_size, pool, write_cache, err);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- gated linear unit with limits
//
// in: [n][2 * inter], gate and up features alternating in runs of `block` as in the SwiGLU kernel.
//   g = min(gate, limit), u = clamp(up, -limit, limit)       (limit <= 0: no clamping)
//   out = g * sigmoid(alpha * g) * (u + shift)
// alpha = 1, shift = 0 and no limit is silu(gate) * up.  The expression is common.cuh's glu_mul, which the matrix
// product's fused epilogue uses too: a value does not depend on which of them ran.
template <typename T>
__global__ void glu_limited_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t n, int inter, int block,
                                   float alpha, float limit, float shift) {
    pdl_wait();
    const int64_t total = n * inter;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / inter;
        const int c = (int)(idx - r * inter);
        const T* gp = in + r * 2 * inter + (int64_t)(c / block) * 2 * block + (c % block);
        out[idx] = from_float<T>(glu_mul<sizeof(T) == 2>(to_float(gp[0]), to_float(gp[block]), alpha, limit, shift));
    }
}

// bfloat16, 8 gate and the 8 matching up features per thread (block % 8 == 0, 16-byte aligned rows).
__global__ void glu_limited_bf16x8_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int64_t n, int inter,
                                          int block, float alpha, float limit, float shift) {
    pdl_wait();
    const int per_row = inter / 8;
    const int64_t total = n * per_row;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / per_row;
        const int c = (int)(idx - r * per_row) * 8;
        const bf16* gp = in + r * 2 * inter + (int64_t)(c / block) * 2 * block + (c % block);
        const uint4 gv = *reinterpret_cast<const uint4*>(gp);
        const uint4 uv = *reinterpret_cast<const uint4*>(gp + block);
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t ow[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(&gw[e]);
            const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(&uw[e]);
            const __nv_bfloat162 o2 = __floats2bfloat162_rn(
                glu_mul<true>(__low2float(g2), __low2float(u2), alpha, limit, shift),
                glu_mul<true>(__high2float(g2), __high2float(u2), alpha, limit, shift));
            ow[e] = *reinterpret_cast<const uint32_t*>(&o2);
        }
        *reinterpret_cast<uint4*>(out + r * inter + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

extern "C" int ss_glu_limited(const void* in, void* out, int64_t n, int inter, int block, float alpha, float limit,
                              float shift, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (block <= 0 || inter % block != 0) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    if (dtype == SS_BF16 && inter % 8 == 0 && block % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        int64_t blocks = (n * (inter / 8) + threads - 1) / threads;
        if (blocks > ss_sm_count() * 16) blocks = ss_sm_count() * 16;
        ss_launch(glu_limited_bf16x8_kernel, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)in, (bf16*)out, n,
                  inter, block, alpha, limit, shift);
        return SS_LAUNCH_CHECK();
    }
    int64_t blocks = (n * inter + threads - 1) / threads;
    if (blocks > ss_sm_count() * 32) blocks = ss_sm_count() * 32;
    if (dtype == SS_BF16)
        ss_launch(glu_limited_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)in, (bf16*)out, n, inter,
                  block, alpha, limit, shift);
    else
        ss_launch(glu_limited_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)in, (float*)out, n,
                  inter, block, alpha, limit, shift);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- sigmoid gate
//
// x[t][c] *= sigmoid(gate[t][c]) for c < width; x rows are x_stride apart, gate rows gate_stride.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, int64_t x_stride, const T* __restrict__ gate, int64_t gate_stride,
                                    int64_t n, int width) {
    pdl_wait();
    const int64_t total = n * width;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / width;
        const int c = (int)(idx - r * width);
        const float g = to_float(gate[r * gate_stride + c]);
        T* p = x + r * x_stride + c;
        *p = from_float<T>(to_float(*p) / (1.0f + expf(-g)));
    }
}

extern "C" int ss_sigmoid_gate(void* x, int64_t x_stride, const void* gate, int64_t gate_stride, int64_t n, int width,
                               int dtype, cudaStream_t stream) {
    if (n <= 0 || width <= 0) return 0;
    const int threads = 256;
    int64_t blocks = (n * width + threads - 1) / threads;
    if (blocks > ss_sm_count() * 32) blocks = ss_sm_count() * 32;
    if (dtype == SS_BF16)
        ss_launch(sigmoid_gate_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (bf16*)x, x_stride, (const bf16*)gate,
                  gate_stride, n, width);
    else
        ss_launch(sigmoid_gate_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (float*)x, x_stride,
                  (const float*)gate, gate_stride, n, width);
    return SS_LAUNCH_CHECK();
}

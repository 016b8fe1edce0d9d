// A residual stream kept as n copies per token ("hyper-connections"), rows of n * width floats, copy s at columns
// s * width .. (s + 1) * width.  A sublayer reads one weighted sum of the copies and its output goes back into every
// copy, while the copies themselves are mixed by an n x n matrix:
//
//   u = sum_s a[s] x_s;   h = u / rms(u) * w        (streams_norm: the sublayer's input, in the activation dtype)
//   x'_t = sum_s M[s, t] x_s + b[t] y               (streams_mix_add: all copies at once from the old ones)
//
//  (1) streams_norm: a block per output row; a = null counts every copy once (the sum of the copies, as the model's
//      last norm reads it); rows picks input rows.
//  (2) streams_mix_add: a block per row; with the next sublayer's (a', w', eps') it also leaves that sublayer's
//      input, so the stream is read and written once between two sublayers.
//  (3) embed_copies: the embedding row times a factor, plus (optionally) a learned vector of the token's position that
//      is not scaled, written into all n copies.
// Everything is 32-bit; sums over s run in the order s = 0, 1, ...; a row's result depends on that row alone.
#include "common.cuh"

namespace imparo {

constexpr int HC_MAX = 8;

template <typename TOut>
__global__ void streams_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows, int n,
                                    const float* __restrict__ a, const float* __restrict__ w, float eps,
                                    TOut* __restrict__ out, int width) {
    extern __shared__ float u_s[];
    __shared__ float scratch[33];
    pdl_trigger();
    float coef[HC_MAX];
#pragma unroll
    for (int s = 0; s < HC_MAX; ++s) coef[s] = (s < n) ? (a ? a[s] : 1.0f) : 0.f;
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * n * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float u = coef[0] * xr[i];
#pragma unroll
        for (int s = 1; s < HC_MAX; ++s)
            if (s < n) u += coef[s] * xr[(size_t)s * width + i];
        u_s[i] = u;
        ss += u * u;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TOut* o = out + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TOut>(u_s[i] * scale * w[i]);
}

// V: columns per thread and access (4: 16-byte loads and stores, for widths that are multiples of four; 1: any width).
// Every element's sums run in the same order either way.
template <typename TOut, int V>
__global__ void streams_mix_add_kernel(float* __restrict__ x, int n, const float* __restrict__ mix,
                                       const float* __restrict__ b, const float* __restrict__ y,
                                       const float* __restrict__ na, const float* __restrict__ nw, float neps,
                                       TOut* __restrict__ nout, int width) {
    extern __shared__ float u_s[];
    __shared__ float scratch[33];
    __shared__ float m_s[HC_MAX * HC_MAX], b_s[HC_MAX], a_s[HC_MAX];
    pdl_trigger();
    for (int i = threadIdx.x; i < n * n; i += blockDim.x) m_s[i] = mix[i];
    for (int i = threadIdx.x; i < n; i += blockDim.x) { b_s[i] = b[i]; a_s[i] = (nw && na) ? na[i] : 1.0f; }
    __syncthreads();
    pdl_wait();
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * n * width;
    const float* yr = y + (size_t)r * width;
    float ss = 0.f;
    for (int i = threadIdx.x * V; i < width; i += blockDim.x * V) {
        float old[HC_MAX][V], yv[V], u[V];
#pragma unroll
        for (int s = 0; s < HC_MAX; ++s) {
            if (V == 4) {
                const float4 q = s < n ? *reinterpret_cast<const float4*>(xr + (size_t)s * width + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                old[s][0] = q.x; old[s][1 % V] = q.y; old[s][2 % V] = q.z; old[s][3 % V] = q.w;
            } else {
                old[s][0] = s < n ? xr[(size_t)s * width + i] : 0.f;
            }
        }
        if (V == 4) {
            const float4 q = *reinterpret_cast<const float4*>(yr + i);
            yv[0] = q.x; yv[1 % V] = q.y; yv[2 % V] = q.z; yv[3 % V] = q.w;
        } else {
            yv[0] = yr[i];
        }
#pragma unroll
        for (int e = 0; e < V; ++e) u[e] = 0.f;
#pragma unroll
        for (int t = 0; t < HC_MAX; ++t) {
            if (t < n) {
                float v[V];
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float acc = m_s[t] * old[0][e];                     // mix[s, t] at s * n + t
#pragma unroll
                    for (int s = 1; s < HC_MAX; ++s)
                        if (s < n) acc += m_s[s * n + t] * old[s][e];
                    acc += b_s[t] * yv[e];
                    v[e] = acc;
                    u[e] = t == 0 ? a_s[0] * acc : u[e] + a_s[t] * acc;
                }
                if (V == 4) *reinterpret_cast<float4*>(xr + (size_t)t * width + i) = make_float4(v[0], v[1 % V], v[2 % V], v[3 % V]);
                else xr[(size_t)t * width + i] = v[0];
            }
        }
        if (nw) {
#pragma unroll
            for (int e = 0; e < V; ++e) { u_s[i + e] = u[e]; ss += u[e] * u[e]; }
        }
    }
    if (!nw) return;
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + neps);
    TOut* o = nout + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TOut>(u_s[i] * scale * nw[i]);
}

template <typename T>
__global__ void embed_copies_kernel(const T* __restrict__ table, const int* __restrict__ ids, float scale, int copies,
                                    const T* __restrict__ pos_table, const int* __restrict__ positions, int n_positions,
                                    float* __restrict__ out, int width, int vocab, int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report(status, IMPARO_ST_TOKEN_RANGE, 71, t, id);
        id = 0;
    }
    const T* row = table + (size_t)id * width;
    const T* prow = nullptr;
    if (pos_table) {
        int p = positions[t];
        if (p < 0 || p >= n_positions) {
            if (threadIdx.x == 0) report(status, IMPARO_ST_TOKEN_RANGE, 72, t, p);
            p = 0;
        }
        prow = pos_table + (size_t)p * width;
    }
    float* o = out + (size_t)t * copies * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = to_f32(row[i]) * scale;
        if (prow) v += to_f32(prow[i]);
        for (int s = 0; s < copies; ++s) o[(size_t)s * width + i] = v;
    }
}

}  // namespace imparo

using namespace imparo;

static inline int hc_threads(int width) { return width >= 2048 ? 512 : (width >= 512 ? 256 : 128); }

// x: float32 [*, n * width]; rows: int32 input row per output row, or null; a: float32 [n] or null (ones).
extern "C" int imparo_streams_norm(const float* x, const int* rows, int n, const float* a, const float* w, float eps,
                                   void* out, int out_dtype, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n < 1 || n > HC_MAX) return -2;
    if ((size_t)width * sizeof(float) > 96 * 1024) return -3;
    const size_t smem = (size_t)width * sizeof(float);
    if (out_dtype == IMPARO_DT_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(streams_norm_kernel<float>, dim3(n_rows), dim3(hc_threads(width)), smem, stream, x, rows, n, a, w, eps, (float*)out, width);
    } else if (out_dtype == IMPARO_DT_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(streams_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(hc_threads(width)), smem, stream, x, rows, n, a, w, eps,
               (__nv_bfloat16*)out, width);
    } else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// x: float32 [n_rows, n * width], updated in place; mix: float32 [n, n] indexed [from, to]; b: float32 [n]; y: float32
// [n_rows, width].  nw != null: also nout[r] = rms-norm of sum_t na[t] x'_t (na null: ones) times nw, in out_dtype.
extern "C" int imparo_streams_mix_add(float* x, int n, const float* mix, const float* b, const float* y, const float* na,
                                      const float* nw, float neps, void* nout, int out_dtype, int n_rows, int width,
                                      cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n < 1 || n > HC_MAX) return -2;
    if ((size_t)width * sizeof(float) > 96 * 1024) return -3;
    const size_t smem = nw ? (size_t)width * sizeof(float) : 0;
    const bool vec = width % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0;
#define IMPARO_MIX(T_, V_) do { \
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_mix_add_kernel<T_, V_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch(streams_mix_add_kernel<T_, V_>, dim3(n_rows), dim3(hc_threads(width / (V_))), smem, stream, x, n, mix, b, y, na, nw, neps, \
               (T_*)nout, width); } while (0)
    if (!nw || out_dtype == IMPARO_DT_F32) {
        if (vec) IMPARO_MIX(float, 4); else IMPARO_MIX(float, 1);
    } else if (out_dtype == IMPARO_DT_BF16) {
        if (vec) IMPARO_MIX(__nv_bfloat16, 4); else IMPARO_MIX(__nv_bfloat16, 1);
    } else return -1;
#undef IMPARO_MIX
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// pos_table: [n_positions, width] in the table's dtype with positions int32 [n_tok], or null (no position vectors).
extern "C" int imparo_embed_copies(const void* table, int table_dtype, const int* ids, float scale, int copies,
                                   const void* pos_table, const int* positions, int n_positions, float* out,
                                   int n_tok, int width, int vocab, int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (copies < 1 || copies > HC_MAX) return -2;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == IMPARO_DT_F32)
        launch(embed_copies_kernel<float>, dim3(n_tok), dim3(threads), 0, stream, (const float*)table, ids, scale, copies,
               (const float*)pos_table, positions, n_positions, out, width, vocab, status);
    else if (table_dtype == IMPARO_DT_BF16)
        launch(embed_copies_kernel<__nv_bfloat16>, dim3(n_tok), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, scale, copies,
               (const __nv_bfloat16*)pos_table, positions, n_positions, out, width, vocab, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

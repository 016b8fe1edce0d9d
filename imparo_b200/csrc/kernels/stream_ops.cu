// Row-wise kernels around the 32-bit residual stream that arrangements other than the plain
// pre-norm block need: activations on their own, an RMS norm multiplied by a sigmoid gate, the
// mean of several RMS-normed branches added into the stream with a factor, a scaled add, a
// vector (and optionally the tokens' embedding rows) added to the stream, a soft cap on logits.
//
// All sums of squares are fixed trees over blockDim threads (common.cuh block_sum), so a row's
// result never depends on which other rows are in the launch.  Norms, gates and the stream are
// 32-bit in both precisions; only stored activations take the path's dtype.
#include "common.cuh"

namespace imparo {

#define IMPARO_ACT_RELU2 0
#define IMPARO_ACT_GELU_TANH 1
#define IMPARO_ACT_SILU 2

__device__ __forceinline__ float act_apply(float z, int kind) {
    if (kind == IMPARO_ACT_RELU2) { const float r = fmaxf(z, 0.f); return r * r; }
    if (kind == IMPARO_ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return silu(z);
}

// out[i] = act(x[i]); x and out may be the same buffer
template <typename T>
__global__ void act_rows_kernel(const T* x, T* out, size_t n, int kind) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(act_apply(to_f32(x[i]), kind));
}

// the same 16 bytes at a time (n a multiple of the vector, both pointers 16-byte aligned)
template <typename T>
__global__ void act_rows_vec_kernel(const T* x, T* out, size_t n_vec, int kind) {
    constexpr int N = 16 / sizeof(T);
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        uint4 raw = reinterpret_cast<const uint4*>(x)[i];
        T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int u = 0; u < N; ++u) e[u] = from_f32<T>(act_apply(to_f32(e[u]), kind));
        reinterpret_cast<uint4*>(out)[i] = raw;
    }
}

// out[r, :] = act(x[r, :]) for rows of x that are a stretch of wider rows (x_stride elements apart); out is dense.
// VEC: 16 bytes at a time (width and x_stride multiples of the vector, both pointers 16-byte aligned)
template <typename T, bool VEC>
__global__ void act_rows_strided_kernel(const T* __restrict__ x, size_t x_stride, T* __restrict__ out, int n_rows, int width, int kind) {
    constexpr int N = VEC ? 16 / (int)sizeof(T) : 1;
    pdl_trigger();
    pdl_wait();
    const int per_row = width / N;
    const size_t total = (size_t)n_rows * per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / per_row;
        const int c = (int)(i - r * per_row) * N;
        if (VEC) {
            uint4 raw = *reinterpret_cast<const uint4*>(x + r * x_stride + c);
            T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
            for (int u = 0; u < N; ++u) e[u] = from_f32<T>(act_apply(to_f32(e[u]), kind));
            *reinterpret_cast<uint4*>(out + r * width + c) = raw;
        } else {
            out[r * width + c] = from_f32<T>(act_apply(to_f32(x[r * x_stride + c]), kind));
        }
    }
}

// out[r, :] = o[r, :] / rms(o[r, :]) * w * sigmoid(gate[r, :]);  o is 32-bit, gate rows have their own stride
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                                     const T* __restrict__ gate, size_t gate_stride, T* __restrict__ out, int width, int vec) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* orow = o + (size_t)r * width;
    const T* g = gate + (size_t)r * gate_stride;
    float ss = 0.f;
    if (vec) {                                     // width a multiple of 4, rows 16-byte aligned (8-byte for the gate and out in bfloat16)
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(orow + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)width + eps);
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(orow + i);
            const float4 ww = *reinterpret_cast<const float4*>(w + i);
            float gv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) gv[u] = 1.0f / (1.0f + expf(-to_f32(g[i + u])));
            T* dst = out + (size_t)r * width + i;
            dst[0] = from_f32<T>(v.x * scale * ww.x * gv[0]); dst[1] = from_f32<T>(v.y * scale * ww.y * gv[1]);
            dst[2] = from_f32<T>(v.z * scale * ww.z * gv[2]); dst[3] = from_f32<T>(v.w * scale * ww.w * gv[3]);
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = orow[i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float gv = to_f32(g[i]);
        out[(size_t)r * width + i] = from_f32<T>(orow[i] * scale * w[i] * (1.0f / (1.0f + expf(-gv))));
    }
}

// x[r, :] += coef * sum_b rms(branch_b[r, :]) * w_b  +  extra_coef * extra[r, :]
struct Branches {
    const float* b[4];
    const float* w[4];
};

__global__ void norm_mean_add_kernel(float* __restrict__ x, Branches br, int n_branches, float eps, float coef,
                                     const float* __restrict__ extra, float extra_coef, int width, int vec) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    float scale[4] = {0.f, 0.f, 0.f, 0.f};
    float* xr = x + (size_t)r * width;
    if (vec) {                                     // width a multiple of 4 and every row 16-byte aligned
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (b < n_branches) {
                    const float4 v = *reinterpret_cast<const float4*>(br.b[b] + (size_t)r * width + i);
                    ss[b] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 4; ++b)
            if (b < n_branches) scale[b] = coef / sqrtf(block_sum(ss[b], scratch) / (float)width + eps);
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 acc = *reinterpret_cast<const float4*>(xr + i);
            if (extra) {
                const float4 e = *reinterpret_cast<const float4*>(extra + (size_t)r * width + i);
                acc.x += extra_coef * e.x; acc.y += extra_coef * e.y; acc.z += extra_coef * e.z; acc.w += extra_coef * e.w;
            }
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (b < n_branches) {
                    const float4 v = *reinterpret_cast<const float4*>(br.b[b] + (size_t)r * width + i);
                    const float4 ww = *reinterpret_cast<const float4*>(br.w[b] + i);
                    s.x += v.x * scale[b] * ww.x; s.y += v.y * scale[b] * ww.y; s.z += v.z * scale[b] * ww.z; s.w += v.w * scale[b] * ww.w;
                }
            }
            acc.x += s.x; acc.y += s.y; acc.z += s.z; acc.w += s.w;
            *reinterpret_cast<float4*>(xr + i) = acc;
        }
        return;
    }
    for (int b = 0; b < n_branches; ++b) {
        const float* row = br.b[b] + (size_t)r * width;
        float ss = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = row[i]; ss += v * v; }
        ss = block_sum(ss, scratch);
        scale[b] = coef / sqrtf(ss / (float)width + eps);
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float s = 0.f;
        for (int b = 0; b < n_branches; ++b) s += br.b[b][(size_t)r * width + i] * scale[b] * br.w[b][i];
        float v = s;
        if (extra) v += extra_coef * extra[(size_t)r * width + i];
        xr[i] += v;
    }
}

// The same, and then the RMS norm of the updated row with weight nw into out (the next layer's normed input): the
// stream is read and written once for both.  A thread norms the elements it wrote itself.
template <typename TOut>
__global__ void norm_mean_add_rmsnorm_kernel(float* __restrict__ x, Branches br, int n_branches, float eps, float coef,
                                             const float* __restrict__ extra, float extra_coef, int width, int vec,
                                             const float* __restrict__ nw, float neps, TOut* __restrict__ out) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    float scale[4] = {0.f, 0.f, 0.f, 0.f};
    float* xr = x + (size_t)r * width;
    TOut* orow = out + (size_t)r * width;
    const int step = vec ? 4 : 1;
    {
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i = threadIdx.x * step; i < width; i += blockDim.x * step) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (b < n_branches) {
                    const float* p = br.b[b] + (size_t)r * width + i;
                    if (vec) { const float4 v = *reinterpret_cast<const float4*>(p); ss[b] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
                    else ss[b] += p[0] * p[0];
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 4; ++b)
            if (b < n_branches) scale[b] = coef / sqrtf(block_sum(ss[b], scratch) / (float)width + eps);
    }
    float ss2 = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 acc = *reinterpret_cast<const float4*>(xr + i);
            if (extra) {
                const float4 e = *reinterpret_cast<const float4*>(extra + (size_t)r * width + i);
                acc.x += extra_coef * e.x; acc.y += extra_coef * e.y; acc.z += extra_coef * e.z; acc.w += extra_coef * e.w;
            }
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (b < n_branches) {
                    const float4 v = *reinterpret_cast<const float4*>(br.b[b] + (size_t)r * width + i);
                    const float4 ww = *reinterpret_cast<const float4*>(br.w[b] + i);
                    s.x += v.x * scale[b] * ww.x; s.y += v.y * scale[b] * ww.y; s.z += v.z * scale[b] * ww.z; s.w += v.w * scale[b] * ww.w;
                }
            }
            acc.x += s.x; acc.y += s.y; acc.z += s.z; acc.w += s.w;
            *reinterpret_cast<float4*>(xr + i) = acc;
            ss2 += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
        }
        const float nscale = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)width + neps);
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xr + i);
            const float4 g = *reinterpret_cast<const float4*>(nw + i);
            TOut* o = orow + i;
            o[0] = from_f32<TOut>(v.x * nscale * g.x); o[1] = from_f32<TOut>(v.y * nscale * g.y);
            o[2] = from_f32<TOut>(v.z * nscale * g.z); o[3] = from_f32<TOut>(v.w * nscale * g.w);
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float acc = xr[i];
        if (extra) acc += extra_coef * extra[(size_t)r * width + i];
        float sum = 0.f;
        for (int b = 0; b < n_branches; ++b) sum += br.b[b][(size_t)r * width + i] * scale[b] * br.w[b][i];
        acc += sum;
        xr[i] = acc;
        ss2 += acc * acc;
    }
    const float nscale = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)width + neps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) orow[i] = from_f32<TOut>(xr[i] * nscale * nw[i]);
}

__global__ void add_scaled_kernel(float* __restrict__ x, const float* __restrict__ y, float coef, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] += coef * y[i];
}

// x += sum_b coef[b] * y_b for up to four float32 sources of x's shape, in the order b = 0, 1, ...
__global__ void add_weighted_kernel(float* __restrict__ x, Branches br, int n_branches, float c0, float c1, float c2, float c3,
                                    size_t n) {
    pdl_trigger();
    pdl_wait();
    const float c[4] = {c0, c1, c2, c3};
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b)
            if (b < n_branches) acc += c[b] * br.b[b][i];
        x[i] += acc;
    }
}

// x[t, :] += (table[ids[t], :] if table) + (vec[:] if vec)
template <typename T>
__global__ void stream_inject_kernel(float* __restrict__ x, const T* __restrict__ table, const int* __restrict__ ids,
                                     const float* __restrict__ vec, int width, int vocab, int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = nullptr;
    if (table) {
        int id = ids[t];
        if (id < 0 || id >= vocab) {
            if (threadIdx.x == 0) report(status, IMPARO_ST_TOKEN_RANGE, 40, t, id);
            id = 0;
        }
        row = table + (size_t)id * width;
    }
    float* xr = x + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = xr[i];
        if (row) v += to_f32(row[i]);
        if (vec) v += vec[i];
        xr[i] = v;
    }
}

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    pdl_trigger();
    pdl_wait();
    const float inv = 1.0f / cap;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

// x[r, :] += y[r, :] / rms(y[r, :]) * w  (a norm on a sublayer's OUTPUT, then the residual add); when `copy` is given,
// the updated row is also stored there in the activation dtype, which is what the next sublayer's products read.
template <typename TOut>
__global__ void __launch_bounds__(256)
out_norm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, float eps, int width,
                    TOut* __restrict__ copy, int vec) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* yr = y + (size_t)r * width;
    float* xr = x + (size_t)r * width;
    float ss = 0.f;
    if (vec) {                                     // width a multiple of 4 and every row 16-byte aligned
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(yr + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)width + eps);
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(yr + i);
            const float4 ww = *reinterpret_cast<const float4*>(w + i);
            float4 o = *reinterpret_cast<const float4*>(xr + i);
            o.x += v.x * scale * ww.x; o.y += v.y * scale * ww.y; o.z += v.z * scale * ww.z; o.w += v.w * scale * ww.w;
            *reinterpret_cast<float4*>(xr + i) = o;
            if (copy) {
                TOut* c = copy + (size_t)r * width + i;
                c[0] = from_f32<TOut>(o.x); c[1] = from_f32<TOut>(o.y); c[2] = from_f32<TOut>(o.z); c[3] = from_f32<TOut>(o.w);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = yr[i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i] + yr[i] * scale * w[i];
        xr[i] = v;
        if (copy) copy[(size_t)r * width + i] = from_f32<TOut>(v);
    }
}

// out[i] = x[i] in another dtype
template <typename TOut>
__global__ void cast_rows_kernel(const float* __restrict__ x, TOut* __restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TOut>(x[i]);
}

__global__ void scale_rows_kernel(float* x, size_t n, float factor) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] *= factor;
}

}  // namespace imparo


using namespace imparo;

static inline unsigned flat_grid(size_t n) {
    const size_t b = (n + 255) / 256;
    return (unsigned)(b < 1 ? 1 : (b > 65535 ? 65535 : b));
}

extern "C" int imparo_act_rows(const void* x, void* out, int dtype, long long n, int kind, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind < 0 || kind > 2) return -22;
    const bool aligned = (((uintptr_t)x | (uintptr_t)out) & 15) == 0;
    if (dtype == IMPARO_DT_F32) {
        if (aligned && n % 4 == 0)
            launch(act_rows_vec_kernel<float>, dim3(flat_grid(n / 4)), dim3(256), 0, stream, (const float*)x, (float*)out, (size_t)(n / 4), kind);
        else
            launch(act_rows_kernel<float>, dim3(flat_grid(n)), dim3(256), 0, stream, (const float*)x, (float*)out, (size_t)n, kind);
    } else if (dtype == IMPARO_DT_BF16) {
        if (aligned && n % 8 == 0)
            launch(act_rows_vec_kernel<__nv_bfloat16>, dim3(flat_grid(n / 8)), dim3(256), 0, stream, (const __nv_bfloat16*)x,
                   (__nv_bfloat16*)out, (size_t)(n / 8), kind);
        else
            launch(act_rows_kernel<__nv_bfloat16>, dim3(flat_grid(n)), dim3(256), 0, stream, (const __nv_bfloat16*)x,
                   (__nv_bfloat16*)out, (size_t)n, kind);
    } else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_act_rows_strided(const void* x, long long x_stride, void* out, int dtype, int n_rows, int width, int kind,
                                       cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    if (kind < 0 || kind > 2) return -22;
    if (x_stride < width) return -2;
    const int es = dtype == IMPARO_DT_F32 ? 4 : 2, nvec = 16 / es;
    const bool vec = width % nvec == 0 && x_stride % nvec == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0;
    const size_t total = (size_t)n_rows * (vec ? width / nvec : width);
#define IMPARO_ACT(T_, V_) launch(act_rows_strided_kernel<T_, V_>, dim3(flat_grid(total)), dim3(256), 0, stream, (const T_*)x, \
        (size_t)x_stride, (T_*)out, n_rows, width, kind)
    if (dtype == IMPARO_DT_F32) { if (vec) IMPARO_ACT(float, true); else IMPARO_ACT(float, false); }
    else if (dtype == IMPARO_DT_BF16) { if (vec) IMPARO_ACT(__nv_bfloat16, true); else IMPARO_ACT(__nv_bfloat16, false); }
    else return -1;
#undef IMPARO_ACT
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_gated_rmsnorm(const float* o, const float* w, float eps, const void* gate, long long gate_stride,
                                    void* out, int dtype, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    const int vec = (width % 4 == 0 && (((uintptr_t)o | (uintptr_t)w) & 15) == 0) ? 1 : 0;
    if (dtype == IMPARO_DT_F32)
        launch(gated_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, o, w, eps, (const float*)gate,
               (size_t)gate_stride, (float*)out, width, vec);
    else if (dtype == IMPARO_DT_BF16)
        launch(gated_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, o, w, eps,
               (const __nv_bfloat16*)gate, (size_t)gate_stride, (__nv_bfloat16*)out, width, vec);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_norm_mean_add(float* x, int n_branches, const float* const* branches, const float* const* weights,
                                    float eps, float coef, const float* extra, float extra_coef, int n_rows, int width,
                                    cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_branches < 0 || n_branches > 4) return -2;
    Branches br = {};
    uintptr_t all = (uintptr_t)x | (uintptr_t)extra;
    for (int b = 0; b < n_branches; ++b) { br.b[b] = branches[b]; br.w[b] = weights[b]; all |= (uintptr_t)branches[b] | (uintptr_t)weights[b]; }
    const int vec = (width % 4 == 0 && (all & 15) == 0) ? 1 : 0;
    launch(norm_mean_add_kernel, dim3(n_rows), dim3(width >= 1024 ? 256 : 128), 0, stream, x, br, n_branches, eps, coef, extra,
           extra_coef, width, vec);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_norm_mean_add_rmsnorm(float* x, int n_branches, const float* const* branches, const float* const* weights,
                                            float eps, float coef, const float* extra, float extra_coef, const float* nw,
                                            float neps, void* out, int out_dtype, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_branches < 0 || n_branches > 4) return -2;
    Branches br = {};
    uintptr_t all = (uintptr_t)x | (uintptr_t)extra;
    for (int b = 0; b < n_branches; ++b) { br.b[b] = branches[b]; br.w[b] = weights[b]; all |= (uintptr_t)branches[b] | (uintptr_t)weights[b]; }
    const int vec = (width % 4 == 0 && (all & 15) == 0) ? 1 : 0;
    const dim3 block(width >= 1024 ? 256 : 128);
    if (out_dtype == IMPARO_DT_F32)
        launch(norm_mean_add_rmsnorm_kernel<float>, dim3(n_rows), block, 0, stream, x, br, n_branches, eps, coef, extra, extra_coef,
               width, vec, nw, neps, (float*)out);
    else if (out_dtype == IMPARO_DT_BF16)
        launch(norm_mean_add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), block, 0, stream, x, br, n_branches, eps, coef, extra,
               extra_coef, width, vec, nw, neps, (__nv_bfloat16*)out);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_add_scaled(float* x, const float* y, float coef, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    launch(add_scaled_kernel, dim3(flat_grid(n)), dim3(256), 0, stream, x, y, coef, (size_t)n);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// ys: up to four float32 device pointers of n floats each (null beyond n_branches); coefs: their factors.
extern "C" int imparo_add_weighted(float* x, const float* y0, const float* y1, const float* y2, const float* y3, int n_branches,
                                   float c0, float c1, float c2, float c3, long long n, cudaStream_t stream) {
    if (n <= 0 || n_branches <= 0) return 0;
    if (n_branches > 4) return -2;
    Branches br;
    br.b[0] = y0; br.b[1] = y1; br.b[2] = y2; br.b[3] = y3;
    launch(add_weighted_kernel, dim3(flat_grid(n)), dim3(256), 0, stream, x, br, n_branches, c0, c1, c2, c3, (size_t)n);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_stream_inject(float* x, const void* table, int dtype, const int* ids, const float* vec, int n_tok,
                                    int width, int vocab, int* status, cudaStream_t stream) {
    if (n_tok <= 0 || (!table && !vec)) return 0;
    if (dtype == IMPARO_DT_F32)
        launch(stream_inject_kernel<float>, dim3(n_tok), dim3(128), 0, stream, x, (const float*)table, ids, vec, width, vocab, status);
    else if (dtype == IMPARO_DT_BF16)
        launch(stream_inject_kernel<__nv_bfloat16>, dim3(n_tok), dim3(128), 0, stream, x, (const __nv_bfloat16*)table, ids, vec,
               width, vocab, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return -2;
    launch(softcap_kernel, dim3(flat_grid(n)), dim3(256), 0, stream, x, (size_t)n, cap);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// x float32 [rows, width] += rms-normed y * w; copy (or null): [rows, width] in copy_dtype, the updated rows
extern "C" int imparo_out_norm_add(float* x, const float* y, const float* w, float eps, void* copy, int copy_dtype, int rows,
                                   int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int vec = width % 4 == 0 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)copy) & 15) == 0;
    if (copy != nullptr && copy_dtype == IMPARO_DT_BF16)
        launch(out_norm_add_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, x, y, w, eps, width, (__nv_bfloat16*)copy, vec);
    else if (copy == nullptr || copy_dtype == IMPARO_DT_F32)
        launch(out_norm_add_kernel<float>, dim3(rows), dim3(256), 0, stream, x, y, w, eps, width, (float*)copy, vec);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_cast_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256 > 8192 ? 8192 : (n + 255) / 256);
    if (out_dtype == IMPARO_DT_BF16)
        launch(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x, (__nv_bfloat16*)out, (size_t)n);
    else if (out_dtype == IMPARO_DT_F32)
        launch(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (float*)out, (size_t)n);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_scale_rows(float* x, long long n, float factor, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256 > 8192 ? 8192 : (n + 255) / 256);
    launch(scale_rows_kernel, dim3(blocks), dim3(256), 0, stream, x, (size_t)n, factor);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// Attention over the paged cache for shapes and variants the specialised kernels do not take:
// any head size up to 256 with a value size of its own, rotation of interleaved pairs (2i, 2i+1)
// or of half-split pairs (i, i + n_rot/2) over the first n_rot dimensions with a magnitude on the
// sines and cosines, an explicit score scale, a window, and a softmax whose denominator counts one
// more term of score 0 that has no value ("sink": p_j = exp(s_j) / (1 + sum exp(s_j))).
//
//  (1) qkv_rotate_store: rows [q heads * hd | kv heads * hd | kv heads * vd] -> rotated queries,
//      rotated keys and plain values written into their pages (K rows kv*hd wide, V rows kv*vd wide).
//  (2) attention_any: one warp per (token, head); keys walked 32 at a time in position order, every
//      lane scores one key; running max and sum in 32-bit; then the lanes accumulate the values, each
//      owning dimensions lane, lane+32, ...  The walk depends only on (position, window).
//      With a sink the running max starts at 0 and the running sum at 1: the extra term is a key
//      of score 0 seen before all others; with sink values (one number per head) the extra term is exp(value) instead of 1:
//      the running max starts at the head's value.  With a soft cap c the scaled score becomes c * tanh(score / c).
//      Heads up to 640 wide (a cache of latent vectors that every head reads is one wide key/value head).
//  (3) qkv_prepare_store: the same rows as a 32-bit product, for variants that work on whole heads in 32-bit before
//      anything is rounded: biases added, half-split rotation, then q and k divided by their own root mean square
//      per head (a norm without a weight), values optionally blended with the values another layer made for the
//      same rows (v = (1 - lambda) v + lambda v_other, lambda a device scalar) and optionally saved for that use.
//      v_from_k: the row has no value columns; a value head is the key head of the same number as it stands before the
//      rotation (keys that are their own values).
#include "common.cuh"

namespace imparo {

constexpr int ANY_MAX_HEAD = 256;
constexpr int ANY_WARPS = 4;
constexpr int ANY_ATT_MAX_HEAD = 640;          // attention_any alone takes heads this wide

template <typename T>
__global__ void __launch_bounds__(ANY_WARPS * 32)
qkv_rotate_store_kernel(const T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ item_of_token,
                        const float* __restrict__ inv_freq, int n_rot, int interleaved, float magnitude,
                        T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                        const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                        int nh, int nkv, int hd, int vd, size_t in_width, int* status) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hh = blockIdx.y * ANY_WARPS + warp;
    const int total = nh + 2 * nkv;
    if (hh >= total) return;
    const int pos = positions[t];
    const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
    const T* src;
    T* dst = nullptr;
    int bad_page = 0;
    int n;                                                       // this head's size
    if (is_q) {
        src = qkv + (size_t)t * in_width + (size_t)hh * hd;
        dst = q_out + ((size_t)t * nh + hh) * hd;
        n = hd;
    } else {
        const int kvh = is_k ? hh - nh : hh - nh - nkv;
        n = is_k ? hd : vd;
        src = qkv + (size_t)t * in_width + (size_t)nh * hd + (is_k ? (size_t)kvh * hd : (size_t)nkv * hd + (size_t)kvh * vd);
        const int blk = pos / page_size;
        int page = -1;
        if (blk < max_blocks) page = table[(size_t)item_of_token[t] * max_blocks + blk];
        if (page < 0 || page >= n_pages) {
            bad_page = page;
        } else {
            const size_t r = (size_t)page * page_size + (pos % page_size);
            dst = is_k ? k_cache + r * ((size_t)nkv * hd) + (size_t)kvh * hd : v_cache + r * ((size_t)nkv * vd) + (size_t)kvh * vd;
        }
    }
    pdl_wait();
    if (dst == nullptr) {
        if (lane == 0) report(status, IMPARO_ST_PAGE_RANGE, 41, t, bad_page);
        return;
    }
    const int half = n_rot >> 1;
    if ((is_q || is_k) && inv_freq && half > 0) {
        for (int i = lane; i < half; i += 32) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            sn *= magnitude; cs *= magnitude;
            const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
            const float u = to_f32(src[a]), v = to_f32(src[b]);
            dst[a] = from_f32<T>(u * cs - v * sn);
            dst[b] = from_f32<T>(v * cs + u * sn);
        }
        for (int d = n_rot + lane; d < n; d += 32) dst[d] = src[d];
    } else {
        for (int d = lane; d < n; d += 32) dst[d] = src[d];
    }
}

// Many tokens (a prompt portion), interleaved pairs, even head and value sizes, rows whose pairs are aligned: a block owns
// one token; the position's sines and cosines are computed once and shared by all of the token's heads (the kernel above
// computes them per head), and a lane moves a pair (2i, 2i+1) as one 4- or 8-byte word.
template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; };
__device__ __forceinline__ float2 pair_f32(float2 v) { return v; }
__device__ __forceinline__ float2 pair_f32(__nv_bfloat162 v) { return __bfloat1622float2(v); }
template <typename P> __device__ __forceinline__ P pair_from(float a, float b);
template <> __device__ __forceinline__ float2 pair_from<float2>(float a, float b) { return make_float2(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 pair_from<__nv_bfloat162>(float a, float b) { return __floats2bfloat162_rn(a, b); }

template <typename T>
__global__ void __launch_bounds__(ANY_WARPS * 32)
qkv_rotate_store_token_kernel(const T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ item_of_token,
                              const float* __restrict__ inv_freq, int n_rot, float magnitude,
                              T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                              const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                              int nh, int nkv, int hd, int vd, size_t in_width, int* status) {
    using P = typename Pair<T>::type;
    __shared__ float sn_s[ANY_MAX_HEAD / 2], cs_s[ANY_MAX_HEAD / 2];
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int half = inv_freq ? (n_rot >> 1) : 0;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        sn_s[i] = sn * magnitude; cs_s[i] = cs * magnitude;
    }
    size_t cache_row = 0;
    int page = 0;
    if (nkv > 0) {
        const int blk = pos / page_size;
        page = blk < max_blocks ? table[(size_t)item_of_token[t] * max_blocks + blk] : -1;
        if (page >= 0 && page < n_pages) cache_row = (size_t)page * page_size + (pos % page_size);
    }
    __syncthreads();
    pdl_wait();
    if (nkv > 0 && (page < 0 || page >= n_pages) && threadIdx.x == 0)
        report(status, IMPARO_ST_PAGE_RANGE, 41, t, page);           // the token's keys and values are skipped, its queries written
    const int total = nh + 2 * nkv;
    const T* row = qkv + (size_t)t * in_width;
    for (int hh = warp; hh < total; hh += ANY_WARPS) {
        const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
        const T* src;
        T* dst;
        int n;
        if (is_q) {
            src = row + (size_t)hh * hd;
            dst = q_out + ((size_t)t * nh + hh) * hd;
            n = hd;
        } else {
            if (page < 0 || page >= n_pages) continue;
            const int kvh = is_k ? hh - nh : hh - nh - nkv;
            n = is_k ? hd : vd;
            src = row + (size_t)nh * hd + (is_k ? (size_t)kvh * hd : (size_t)nkv * hd + (size_t)kvh * vd);
            dst = is_k ? k_cache + cache_row * ((size_t)nkv * hd) + (size_t)kvh * hd : v_cache + cache_row * ((size_t)nkv * vd) + (size_t)kvh * vd;
        }
        const int turn = (is_q || is_k) ? half : 0;
        for (int i = lane; i < n / 2; i += 32) {
            const float2 v = pair_f32(reinterpret_cast<const P*>(src)[i]);
            float a = v.x, b = v.y;
            if (i < turn) { a = v.x * cs_s[i] - v.y * sn_s[i]; b = v.y * cs_s[i] + v.x * sn_s[i]; }
            reinterpret_cast<P*>(dst)[i] = pair_from<P>(a, b);
        }
    }
}


// One warp per (token, head) of a 32-bit product row; the head passes through shared memory so that a rotation pair and
// the head's sum of squares are at hand.  unit_eps < 0: q and k keep their length.
template <typename T>
__global__ void __launch_bounds__(ANY_WARPS * 32)
qkv_prepare_store_kernel(const float* __restrict__ qkv, size_t in_width, const float* __restrict__ bias,
                         const int* __restrict__ positions, const int* __restrict__ item_of_token,
                         const float* __restrict__ inv_freq, int n_rot, float unit_eps,
                         const T* __restrict__ v_other, const float* __restrict__ v_lambda, T* __restrict__ v_save,
                         T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                         const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                         int nh, int nkv, int hd, int vd, int v_from_k, int* status) {
    __shared__ float head[ANY_WARPS][ANY_MAX_HEAD];
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hh = blockIdx.y * ANY_WARPS + warp;
    const int total = nh + 2 * nkv;
    if (hh >= total) return;
    const int pos = positions[t];
    const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
    const int kvh = is_q ? 0 : (is_k ? hh - nh : hh - nh - nkv);
    const int n = (is_q || is_k) ? hd : vd;
    const size_t col = is_q ? (size_t)hh * hd
                            : (size_t)nh * hd + ((is_k || v_from_k) ? (size_t)kvh * hd : (size_t)nkv * hd + (size_t)kvh * vd);
    T* dst = nullptr;
    int bad_page = 0;
    if (is_q) {
        dst = q_out + ((size_t)t * nh + hh) * hd;
    } else {
        const int blk = pos / page_size;
        int page = -1;
        if (blk < max_blocks) page = table[(size_t)item_of_token[t] * max_blocks + blk];
        if (page < 0 || page >= n_pages) {
            bad_page = page;
        } else {
            const size_t r = (size_t)page * page_size + (pos % page_size);
            dst = is_k ? k_cache + r * ((size_t)nkv * hd) + (size_t)kvh * hd : v_cache + r * ((size_t)nkv * vd) + (size_t)kvh * vd;
        }
    }
    pdl_wait();
    if (dst == nullptr) {
        if (lane == 0) report(status, IMPARO_ST_PAGE_RANGE, 43, t, bad_page);
        return;
    }
    const float* src = qkv + (size_t)t * in_width + col;
    float* hv = head[warp];
    for (int d = lane; d < n; d += 32) hv[d] = src[d] + (bias ? bias[col + d] : 0.f);
    __syncwarp();
    if (!is_q && !is_k) {                                           // a value head
        const size_t at = (size_t)t * nkv * vd + (size_t)kvh * vd;
        const float lam = (v_other && v_lambda) ? *v_lambda : 0.f;
        for (int d = lane; d < n; d += 32) {
            float v = hv[d];
            if (v_save) v_save[at + d] = from_f32<T>(v);
            if (v_other) v = (1.0f - lam) * v + lam * to_f32(v_other[at + d]);
            dst[d] = from_f32<T>(v);
        }
        return;
    }
    const int half = inv_freq ? (n_rot >> 1) : 0;
    float ss = 0.f;
    constexpr int PER = ANY_MAX_HEAD / 32;
    float val[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        float v = 0.f;
        if (d < n) {
            v = hv[d];
            if (d < 2 * half) {
                const int pair = d < half ? d : d - half;
                float sn, cs;
                sincosf((float)pos * inv_freq[pair], &sn, &cs);
                v = d < half ? hv[d] * cs - hv[d + half] * sn : hv[d] * cs + hv[d - half] * sn;
            }
        }
        val[i] = v;
        ss += v * v;
    }
    float scale = 1.0f;
    if (unit_eps >= 0.f) scale = 1.0f / sqrtf(warp_sum(ss) / (float)n + unit_eps);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        if (d < n) dst[d] = from_f32<T>(val[i] * scale);
    }
}

template <typename T>
__global__ void __launch_bounds__(ANY_WARPS * 32)
attention_any_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                     const int* __restrict__ positions, const int* __restrict__ item_of_token,
                     const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                     int window, float scale, int sink, const float* __restrict__ sink_values, float softcap,
                     T* __restrict__ out, int nh, int nkv, int hd, int vd, int* status) {
    __shared__ float qbuf[ANY_WARPS][ANY_ATT_MAX_HEAD];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * ANY_WARPS + warp;
    if (h >= nh) return;
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* tab = table + (size_t)item_of_token[t] * max_blocks;
    const size_t kw = (size_t)nkv * hd, vw = (size_t)nkv * vd;
    float* qs = qbuf[warp];
    const T* qrow = q + ((size_t)t * nh + h) * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32(qrow[d]);
    __syncwarp();

    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    constexpr int PER = ANY_ATT_MAX_HEAD / 32;
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    float m = sink ? (sink_values ? sink_values[h] : 0.f) : -INFINITY, l = sink ? 1.f : 0.f;

    for (int base = lo; base <= pos; base += 32) {
        const int j = base + lane;
        float s = -INFINITY;
        int rowi = -1;
        if (j <= pos) {
            const int blk = j / page_size;
            const int page = blk < max_blocks ? tab[blk] : -1;
            if (page < 0 || page >= n_pages) {
                report(status, IMPARO_ST_PAGE_RANGE, 42, t, page);
            } else {
                rowi = page * page_size + (j % page_size);
                const T* kp = k_cache + (size_t)rowi * kw + (size_t)kvh * hd;
                float d = 0.f;
                for (int c = 0; c < hd; ++c) d += to_f32(kp[c]) * qs[c];
                s = d * scale;
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float p = (rowi >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] *= corr;
        m = m_new;
        const int cnt = min(32, pos - base + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int rj = __shfl_sync(0xffffffffu, rowi, jj);
            if (rj < 0) continue;
            const T* vp = v_cache + (size_t)rj * vw + (size_t)kvh * vd;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + 32 * i;
                if (d < vd) acc[i] += pj * to_f32(vp[d]);
            }
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* orow = out + ((size_t)t * nh + h) * vd;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace imparo

using namespace imparo;

// qkv: [n_tok, nh*hd + nkv*hd + nkv*vd] in rows of row_stride elements (a stretch of a wider product).  nkv == 0: queries only.
extern "C" int imparo_qkv_rotate_store(const void* qkv, int dtype, const int* positions, const int* item_of_token,
                                       const float* inv_freq, int n_rot, int interleaved, float magnitude,
                                       void* q_out, void* k_cache, void* v_cache,
                                       const int* table, int max_blocks, int page_size, int n_pages,
                                       int n_tok, int nh, int nkv, int hd, int vd, long long row_stride, int* status,
                                       cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (hd < 1 || hd > ANY_MAX_HEAD || vd < 1 || vd > ANY_MAX_HEAD) return -3;
    if (n_rot < 0 || n_rot > hd || (n_rot & 1)) return -4;
    if (row_stride < (long long)(nh + nkv) * hd + (long long)nkv * vd) return -2;
    {
        // a prompt portion with interleaved pairs (or no rotation) whose pairs can be moved as words: a block per token
        const int es = dtype == IMPARO_DT_F32 ? 4 : 2;
        const bool words = hd % 2 == 0 && vd % 2 == 0 && row_stride % 2 == 0 &&
                           (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & (uintptr_t)(2 * es - 1)) == 0;
        if (n_tok >= 256 && words && (interleaved || inv_freq == nullptr || n_rot == 0)) {
            if (dtype == IMPARO_DT_F32)
                launch(qkv_rotate_store_token_kernel<float>, dim3(n_tok), dim3(ANY_WARPS * 32), 0, stream, (const float*)qkv, positions,
                       item_of_token, inv_freq, n_rot, magnitude, (float*)q_out, (float*)k_cache, (float*)v_cache, table, max_blocks,
                       page_size, n_pages, nh, nkv, hd, vd, (size_t)row_stride, status);
            else if (dtype == IMPARO_DT_BF16)
                launch(qkv_rotate_store_token_kernel<__nv_bfloat16>, dim3(n_tok), dim3(ANY_WARPS * 32), 0, stream, (const __nv_bfloat16*)qkv,
                       positions, item_of_token, inv_freq, n_rot, magnitude, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
                       (__nv_bfloat16*)v_cache, table, max_blocks, page_size, n_pages, nh, nkv, hd, vd, (size_t)row_stride, status);
            else return -1;
            IMPARO_CHECK_LAUNCH();
            return 0;
        }
    }
    dim3 grid(n_tok, (nh + 2 * nkv + ANY_WARPS - 1) / ANY_WARPS);
    if (dtype == IMPARO_DT_F32)
        launch(qkv_rotate_store_kernel<float>, grid, dim3(ANY_WARPS * 32), 0, stream, (const float*)qkv, positions, item_of_token,
               inv_freq, n_rot, interleaved, magnitude, (float*)q_out, (float*)k_cache, (float*)v_cache, table, max_blocks,
               page_size, n_pages, nh, nkv, hd, vd, (size_t)row_stride, status);
    else if (dtype == IMPARO_DT_BF16)
        launch(qkv_rotate_store_kernel<__nv_bfloat16>, grid, dim3(ANY_WARPS * 32), 0, stream, (const __nv_bfloat16*)qkv, positions,
               item_of_token, inv_freq, n_rot, interleaved, magnitude, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
               (__nv_bfloat16*)v_cache, table, max_blocks, page_size, n_pages, nh, nkv, hd, vd, (size_t)row_stride, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_attention_any(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                    const int* positions, const int* item_of_token,
                                    const int* table, int max_blocks, int page_size, int n_pages,
                                    int window, float scale, int sink, const float* sink_values, float softcap, void* out,
                                    int n_tok, int nh, int nkv, int hd, int vd, int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (hd < 1 || hd > ANY_ATT_MAX_HEAD || vd < 1 || vd > ANY_ATT_MAX_HEAD) return -3;
    if (nkv <= 0 || nh % nkv != 0) return -5;
    dim3 grid(n_tok, (nh + ANY_WARPS - 1) / ANY_WARPS);
    if (dtype == IMPARO_DT_F32)
        launch(attention_any_kernel<float>, grid, dim3(ANY_WARPS * 32), 0, stream,
               (const float*)q, (const float*)k_cache, (const float*)v_cache, positions, item_of_token, table,
               max_blocks, page_size, n_pages, window, scale, sink, sink_values, softcap, (float*)out, nh, nkv, hd, vd, status);
    else if (dtype == IMPARO_DT_BF16)
        launch(attention_any_kernel<__nv_bfloat16>, grid, dim3(ANY_WARPS * 32), 0, stream,
               (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, positions,
               item_of_token, table, max_blocks, page_size, n_pages, window, scale, sink, sink_values, softcap, (__nv_bfloat16*)out, nh, nkv, hd,
               vd, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// qkv: float32 [n_tok, nh*hd + nkv*hd + nkv*vd] in rows of row_stride floats; bias float32 over the same columns or null;
// unit_eps < 0: no unit norm; v_other / v_save: [n_tok, nkv*vd] in dtype or null; v_lambda: a float on the device.
extern "C" int imparo_qkv_prepare_store(const float* qkv, long long row_stride, const float* bias, int dtype, const int* positions,
                                        const int* item_of_token, const float* inv_freq, int n_rot, float unit_eps,
                                        const void* v_other, const float* v_lambda, void* v_save,
                                        void* q_out, void* k_cache, void* v_cache, const int* table, int max_blocks,
                                        int page_size, int n_pages, int n_tok, int nh, int nkv, int hd, int vd, int v_from_k,
                                        int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (hd < 1 || hd > ANY_MAX_HEAD || vd < 1 || vd > ANY_MAX_HEAD) return -3;
    if (n_rot < 0 || n_rot > hd || (n_rot & 1)) return -4;
    if (v_from_k && vd != hd) return -6;
    if (row_stride < (long long)(nh + nkv) * hd + (v_from_k ? 0 : (long long)nkv * vd)) return -2;
    dim3 grid(n_tok, (nh + 2 * nkv + ANY_WARPS - 1) / ANY_WARPS);
    if (dtype == IMPARO_DT_F32)
        launch(qkv_prepare_store_kernel<float>, grid, dim3(ANY_WARPS * 32), 0, stream, qkv, (size_t)row_stride, bias, positions,
               item_of_token, inv_freq, n_rot, unit_eps, (const float*)v_other, v_lambda, (float*)v_save, (float*)q_out,
               (float*)k_cache, (float*)v_cache, table, max_blocks, page_size, n_pages, nh, nkv, hd, vd, v_from_k, status);
    else if (dtype == IMPARO_DT_BF16)
        launch(qkv_prepare_store_kernel<__nv_bfloat16>, grid, dim3(ANY_WARPS * 32), 0, stream, qkv, (size_t)row_stride, bias, positions,
               item_of_token, inv_freq, n_rot, unit_eps, (const __nv_bfloat16*)v_other, v_lambda, (__nv_bfloat16*)v_save,
               (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, table, max_blocks, page_size, n_pages, nh, nkv,
               hd, vd, v_from_k, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// Pieces of an attention whose keys and values are made from one small latent vector per token, which is all the
// cache keeps.  With per-head matrices U_k [dim, rank] and U_v [vdim, rank] and the cached latent c_j,
//   q . (U_k c_j) = (U_k^T q) . c_j      and      sum_j p_j (U_v c_j) = U_v (sum_j p_j c_j),
// so the attention itself runs over the latents with every head sharing the one cached row per token: queries are
// taken into the latent space before it and the result is taken out of it after it.
//
//  (1) latent_norm_store: per row of a 32-bit product [.. q latent .. | .. kv latent ..], each stretch divided by its
//      root mean square times a weight; the query latent goes to an activation tensor, the kv latent into its page.
//  (1b) latent_rot_store: the form with a rotated part beside the latent.  Per row of a 32-bit product
//      [q: heads x (dim plain | rot rotated) | c_raw: rank | kr: rot]: the page row becomes [rms(c_raw) * w | turn(kr)]
//      (rank + rot wide; kr is one key part that all heads share); every head's plain query dimensions go to q_plain
//      [T, heads * dim] and its rotated ones, turned by the position, to the last rot entries of the head's latent-space
//      query q_lat [T, heads * (rank + rot)] (the first rank entries are U_k^T q_plain, made by heads_linear).  The turn: of the
//      first n_rot of the rot dimensions, i pairs with i + n_rot/2, angle = position * inv_freq[i] in 32-bit.  Two CTAs per
//      token: one for the queries, one for the cached row.
//  (2) heads_linear: out[t, h, :] = W[h] x[t, h, :] for every head h (W [heads, out, in]), optionally times
//      sigmoid(gate[t, h, :]) (a 32-bit product's columns).  A warp per output feature of a head and tile of eight rows;
//      32-bit sums (for steps of few rows: many rows go to the library's batched product).
#include "common.cuh"

namespace imparo {

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_store_kernel(const float* __restrict__ proj, size_t stride, int q_off, int q_rank, int c_off, int c_rank,
                         const float* __restrict__ wq, const float* __restrict__ wc, float eps,
                         const int* __restrict__ positions, const int* __restrict__ item_of_token,
                         T* __restrict__ q_out, T* __restrict__ cache, const int* __restrict__ table, int max_blocks,
                         int page_size, int n_pages, int* status) {
    __shared__ float scratch[33];
    pdl_trigger();
    const int t = blockIdx.x;
    const bool is_q = blockIdx.y == 0;
    T* dst = nullptr;
    int bad_page = 0;
    if (is_q) {
        dst = q_out + (size_t)t * q_rank;
    } else {
        const int pos = positions[t];
        const int blk = pos / page_size;
        int page = -1;
        if (blk < max_blocks) page = table[(size_t)item_of_token[t] * max_blocks + blk];
        if (page < 0 || page >= n_pages) bad_page = page;
        else dst = cache + ((size_t)page * page_size + (pos % page_size)) * c_rank;
    }
    pdl_wait();
    const int n = is_q ? q_rank : c_rank;
    const float* src = proj + (size_t)t * stride + (is_q ? q_off : c_off);
    const float* w = is_q ? wq : wc;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += src[i] * src[i];
    ss = block_sum(ss, scratch);
    if (dst == nullptr) {
        if (threadIdx.x == 0) report(status, IMPARO_ST_PAGE_RANGE, 74, t, bad_page);
        return;
    }
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = from_f32<T>(src[i] * scale * w[i]);
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_rot_store_kernel(const float* __restrict__ proj, size_t stride, int heads, int dim, int rot, int rank,
                        const float* __restrict__ wc, float eps, const float* __restrict__ inv_freq, int n_rot,
                        const int* __restrict__ positions, const int* __restrict__ item_of_token,
                        T* __restrict__ q_plain, T* __restrict__ q_lat, T* __restrict__ cache, const int* __restrict__ table,
                        int max_blocks, int page_size, int n_pages, int* status) {
    __shared__ float scratch[33];
    __shared__ float cs_s[256], sn_s[256];         // the position's cosines and sines, once for all heads (n_rot <= 512)
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int blk = pos / page_size;
    int page = -1;
    if (blk < max_blocks) page = table[(size_t)item_of_token[t] * max_blocks + blk];
    const int q_width = heads * (dim + rot), row_w = rank + rot, half = n_rot / 2;
    const float fpos = (float)pos;
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(fpos * inv_freq[j], &sn_s[j], &cs_s[j]);
    pdl_wait();
    __syncthreads();
    const float* row = proj + (size_t)t * stride;
    if (blockIdx.y == 0) {
        // queries: plain dimensions as they are, rotated ones turned
        for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
            const int h = i / dim, d = i % dim;
            q_plain[(size_t)t * heads * dim + i] = from_f32<T>(row[(size_t)h * (dim + rot) + d]);
        }
        for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
            const int h = i / rot, d = i % rot;
            const float* qr = row + (size_t)h * (dim + rot) + dim;
            float v = qr[d];
            if (d < n_rot) {
                const int j = d < half ? d : d - half;
                const float sn = sn_s[j], cs = cs_s[j];
                v = d < half ? qr[d] * cs - qr[d + half] * sn : qr[d] * cs + qr[d - half] * sn;
            }
            q_lat[((size_t)t * heads + h) * row_w + rank + d] = from_f32<T>(v);
        }
        return;
    }
    // the cached row
    const float* c = row + q_width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss += c[i] * c[i];
    ss = block_sum(ss, scratch);
    if (page < 0 || page >= n_pages) {
        if (threadIdx.x == 0) report(status, IMPARO_ST_PAGE_RANGE, 75, t, page);
        return;
    }
    T* dst = cache + ((size_t)page * page_size + (pos % page_size)) * row_w;
    const float scale = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>(c[i] * scale * wc[i]);
    const float* kr = c + rank;
    for (int d = threadIdx.x; d < rot; d += blockDim.x) {
        float v = kr[d];
        if (d < n_rot) {
            const int j = d < half ? d : d - half;
            const float sn = sn_s[j], cs = cs_s[j];
            v = d < half ? kr[d] * cs - kr[d + half] * sn : kr[d] * cs + kr[d - half] * sn;
        }
        dst[rank + d] = from_f32<T>(v);
    }
}

constexpr int HL_ROWS = 8;

// A warp per (head, output feature) and tile of HL_ROWS rows: the lanes stride over the head's inputs (the matrix row is
// read once, coalesced), every row's sum is finished by a warp sum in a fixed order.
template <typename T>
__global__ void __launch_bounds__(128)
heads_linear_kernel(const T* __restrict__ x, size_t x_stride, const T* __restrict__ w, const float* __restrict__ gate,
                    size_t gate_stride, T* __restrict__ out, size_t out_stride, int n_tok, int n_in, int n_out,
                    int x_head, int out_head, int gate_per_head) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y;
    const int o = blockIdx.x * 4 + warp;
    const int t0 = blockIdx.z * HL_ROWS;
    if (o >= n_out) return;
    const int rows = min(HL_ROWS, n_tok - t0);
    const T* wr = w + ((size_t)h * n_out + o) * n_in;
    const T* xh = x + (size_t)t0 * x_stride + (size_t)h * x_head;
    float acc[HL_ROWS];
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r) acc[r] = 0.f;
    for (int i = lane; i < n_in; i += 32) {
        const float wv = to_f32(wr[i]);
#pragma unroll
        for (int r = 0; r < HL_ROWS; ++r)
            if (r < rows) acc[r] += wv * to_f32(xh[(size_t)r * x_stride + i]);
    }
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && r < rows) {
            float res = v;
            if (gate) res *= 1.0f / (1.0f + expf(-gate[(size_t)(t0 + r) * gate_stride + (gate_per_head ? (size_t)h : (size_t)h * n_out + o)]));
            out[(size_t)(t0 + r) * out_stride + (size_t)h * out_head + o] = from_f32<T>(res);
        }
    }
}

// x[t, c] *= sigmoid(gate[t, c / group]) in place (gate: columns of a 32-bit product; group 1: a gate per element, group g: a
// gate per stretch of g columns, e.g. per head)
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ x, size_t x_stride, const float* __restrict__ gate, size_t gate_stride, int n_tok, int width,
                    int group) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    T* xr = x + (size_t)t * x_stride;
    const float* gr = gate + (size_t)t * gate_stride;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x)
        xr[c] = from_f32<T>(to_f32(xr[c]) * (1.0f / (1.0f + expf(-gr[group > 1 ? c / group : c]))));
}

}  // namespace imparo

using namespace imparo;

// x: rows of x_stride elements (width used), bfloat16 or float32; gate: float32 rows of gate_stride floats.
extern "C" int imparo_sigmoid_gate(void* x, long long x_stride, const float* gate, long long gate_stride, int dtype, int n_tok,
                                   int width, int group, cudaStream_t stream) {
    if (n_tok <= 0 || width <= 0) return 0;
    if (group < 1) return -2;
    const dim3 grid((width + 255) / 256 > 8 ? 8 : (width + 255) / 256, n_tok);
    if (dtype == IMPARO_DT_F32)
        launch(sigmoid_gate_kernel<float>, grid, dim3(256), 0, stream, (float*)x, (size_t)x_stride, gate, (size_t)gate_stride, n_tok, width, group);
    else if (dtype == IMPARO_DT_BF16)
        launch(sigmoid_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)x, (size_t)x_stride, gate,
               (size_t)gate_stride, n_tok, width, group);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// proj: float32 rows of `stride` floats; q_out: [n_tok, q_rank] and cache pages of c_rank per position, both in dtype.
extern "C" int imparo_latent_norm_store(const float* proj, long long stride, int q_off, int q_rank, int c_off, int c_rank,
                                        const float* wq, const float* wc, float eps, const int* positions,
                                        const int* item_of_token, void* q_out, void* cache, int dtype, const int* table,
                                        int max_blocks, int page_size, int n_pages, int n_tok, int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (q_rank < 1 || c_rank < 1 || stride < q_off + q_rank || stride < c_off + c_rank) return -2;
    if (dtype == IMPARO_DT_F32)
        launch(latent_norm_store_kernel<float>, dim3(n_tok, 2), dim3(128), 0, stream, proj, (size_t)stride, q_off, q_rank, c_off, c_rank,
               wq, wc, eps, positions, item_of_token, (float*)q_out, (float*)cache, table, max_blocks, page_size, n_pages, status);
    else if (dtype == IMPARO_DT_BF16)
        launch(latent_norm_store_kernel<__nv_bfloat16>, dim3(n_tok, 2), dim3(128), 0, stream, proj, (size_t)stride, q_off, q_rank, c_off,
               c_rank, wq, wc, eps, positions, item_of_token, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, table, max_blocks,
               page_size, n_pages, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// proj: float32 rows of `stride` floats = [heads * (dim + rot) | rank | rot | ...]; q_plain [n_tok, heads * dim], q_lat
// [n_tok, heads * (rank + rot)] and cache pages of rank + rot per position, all in dtype; inv_freq float32 [n_rot / 2] (null
// with n_rot 0).
extern "C" int imparo_latent_rot_store(const float* proj, long long stride, int heads, int dim, int rot, int rank, const float* wc,
                                       float eps, const float* inv_freq, int n_rot, const int* positions, const int* item_of_token,
                                       void* q_plain, void* q_lat, void* cache, int dtype, const int* table, int max_blocks,
                                       int page_size, int n_pages, int n_tok, int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (heads < 1 || dim < 1 || rot < 0 || rank < 1 || n_rot < 0 || n_rot > rot || n_rot > 512 || n_rot % 2 || (n_rot > 0 && inv_freq == nullptr)
        || stride < (long long)heads * (dim + rot) + rank + rot) return -2;
    if (dtype == IMPARO_DT_F32)
        launch(latent_rot_store_kernel<float>, dim3(n_tok, 2), dim3(128), 0, stream, proj, (size_t)stride, heads, dim, rot, rank, wc, eps,
               inv_freq, n_rot, positions, item_of_token, (float*)q_plain, (float*)q_lat, (float*)cache, table, max_blocks, page_size,
               n_pages, status);
    else if (dtype == IMPARO_DT_BF16)
        launch(latent_rot_store_kernel<__nv_bfloat16>, dim3(n_tok, 2), dim3(128), 0, stream, proj, (size_t)stride, heads, dim, rot, rank, wc,
               eps, inv_freq, n_rot, positions, item_of_token, (__nv_bfloat16*)q_plain, (__nv_bfloat16*)q_lat, (__nv_bfloat16*)cache,
               table, max_blocks, page_size, n_pages, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// x: rows of x_stride elements in which head h's n_in inputs start at h * x_head; w: [heads, n_out, n_in]; gate: float32 rows
// (heads * n_out used, or `heads` with gate_per_head) or null; out: rows of out_stride elements in which head h's n_out
// outputs start at h * out_head.  x, w and out share the dtype.
extern "C" int imparo_heads_linear(const void* x, long long x_stride, const void* w, const float* gate, long long gate_stride,
                                   void* out, long long out_stride, int dtype, int n_tok, int heads, int n_in, int n_out,
                                   int x_head, int out_head, int gate_per_head, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (heads < 1 || n_in < 1 || n_out < 1 || x_head < n_in || out_head < n_out) return -2;
    const size_t smem = 0;
    const int tiles = (n_tok + HL_ROWS - 1) / HL_ROWS;
    if (tiles > 65535 || heads > 65535) return -2;
    const dim3 grid((n_out + 3) / 4, heads, tiles);
    if (dtype == IMPARO_DT_F32)
        launch(heads_linear_kernel<float>, grid, dim3(128), smem, stream, (const float*)x, (size_t)x_stride, (const float*)w, gate,
               (size_t)gate_stride, (float*)out, (size_t)out_stride, n_tok, n_in, n_out, x_head, out_head, gate_per_head);
    else if (dtype == IMPARO_DT_BF16)
        launch(heads_linear_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)x, (size_t)x_stride,
               (const __nv_bfloat16*)w, gate, (size_t)gate_stride, (__nv_bfloat16*)out, (size_t)out_stride, n_tok, n_in, n_out, x_head,
               out_head, gate_per_head);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

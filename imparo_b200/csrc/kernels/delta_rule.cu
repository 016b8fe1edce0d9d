// The gated delta rule with one decay per head and key channel, over ragged batches, state in the request's slot.
//
// Per value head h (its query/key head is h / (heads / kv_heads)) a request keeps S [dim, vdim] in 32-bit:
//   S <- g * S (row d times g[d]);   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q        (in this order)
//
//  (1) delta_prepare: per row, in 32-bit: q and k of every query/key head divided by sqrt(sum of squares + unit_eps)
//      (q also times q_scale), beta = sigmoid(b), g = exp(-exp(A_log[h]) * softplus(a + dt_bias)) written over a.
//  (2) delta_scan: the value columns of S are independent of one another, so a lane owns a stretch of DPT key
//      channels of one column p: LPC lanes share a column (dim <= DPT * LPC), a warp walks a request's rows in order
//      with its 32 / LPC columns in registers.  The row's q, k and g pass through shared memory (the next row is
//      fetched while the current one is computed); the two sums over the key channels are finished by shuffles among
//      the LPC lanes.  The additions' order depends on (dim, LPC) only.
//  (3) head_norm_gate: every head's output divided by its root mean square over vdim, times a weight [vdim] shared
//      by the heads, times sigmoid(gate).
#include "common.cuh"

namespace imparo {

__device__ __forceinline__ float dr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---- (1) ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ qkv, size_t qkv_stride, int q_off, int k_off, const float* __restrict__ bproj,
                     size_t b_stride, int b_off, float* __restrict__ a, const float* __restrict__ A_log,
                     const float* __restrict__ dt_bias, float* __restrict__ beta, int heads, int kv_heads, int dim,
                     float unit_eps, float q_scale) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int task = warp; task < 2 * kv_heads; task += nw) {
        const bool is_q = task < kv_heads;
        float* v = qkv + (size_t)t * qkv_stride + (is_q ? q_off + task * dim : k_off + (task - kv_heads) * dim);
        float ss = 0.f;
        for (int d = lane; d < dim; d += 32) ss += v[d] * v[d];
        ss = warp_sum(ss);
        const float f = (1.0f / sqrtf(ss + unit_eps)) * (is_q ? q_scale : 1.0f);
        for (int d = lane; d < dim; d += 32) v[d] *= f;
    }
    float* ar = a + (size_t)t * heads * dim;
    for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
        const float rate = expf(A_log[i / dim]);
        ar[i] = expf(-rate * dr_softplus(ar[i] + dt_bias[i]));
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x)
        beta[(size_t)t * heads + h] = 1.0f / (1.0f + expf(-bproj[(size_t)t * b_stride + b_off + h]));
}

// ---- (2) ------------------------------------------------------------------------------------------------------
constexpr int DR_WARPS = 4;

template <int DPT, int LPC>
__global__ void __launch_bounds__(DR_WARPS * 32)
delta_scan_kernel(const float* __restrict__ qkv, size_t qkv_stride, int q_off, int k_off, int v_off,
                  const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ state,
                  const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_slots,
                  float* __restrict__ out, int heads, int kv_heads, int dim, int vdim, int* status) {
    constexpr int DP = DPT * LPC;                   // padded key size
    constexpr int CPW = 32 / LPC;                   // columns per warp
    __shared__ __align__(16) float buf[DR_WARPS][2][3 * DP];
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int item = blockIdx.z, h = blockIdx.y;
    const int col = (blockIdx.x * DR_WARPS + warp) * CPW + lane / LPC;
    const int part = lane % LPC;
    const int first = item_row_start[item], n = item_row_start[item + 1] - first;
    const int slot = item_slot[item];
    pdl_wait();
    if ((blockIdx.x * DR_WARPS + warp) * CPW >= vdim) return;            // a warp without columns
    if (slot < 0 || slot >= n_slots) {
        if (lane == 0 && blockIdx.x == 0 && warp == 0) report(status, IMPARO_ST_SLOT_RANGE, 73, item, slot);
        return;
    }
    const bool live = col < vdim;
    const int kvh = h / (heads / kv_heads);
    float* Sg = state + (((size_t)slot * heads + h) * dim) * vdim;
    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = part * DPT + i;
        S[i] = (live && d < dim) ? Sg[(size_t)d * vdim + col] : 0.f;
    }
    // a row's q, k and g of this head: 3 * DP floats, fetched by the warp's lanes a row ahead
    constexpr int PER = (3 * DP + 31) / 32;
    float ahead[PER];
    auto fetch = [&](int t) {
        const float* row = qkv + (size_t)t * qkv_stride;
        const float* gr = g + ((size_t)t * heads + h) * dim;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = lane + 32 * i;
            const int which = e / DP, d = e % DP;
            float v = 0.f;
            if (e < 3 * DP && d < dim)
                v = which == 0 ? row[q_off + kvh * dim + d] : (which == 1 ? row[k_off + kvh * dim + d] : gr[d]);
            ahead[i] = v;
        }
    };
    auto stash = [&](int b) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = lane + 32 * i;
            if (e < 3 * DP) buf[warp][b][e] = ahead[i];
        }
    };
    if (n > 0) { fetch(first); stash(0); }
    __syncwarp();
    float v_next = 0.f, b_next = 0.f;
    if (n > 0) {
        v_next = live ? qkv[(size_t)first * qkv_stride + v_off + h * vdim + col] : 0.f;
        b_next = beta[(size_t)first * heads + h];
    }
    for (int j = 0; j < n; ++j) {
        const int t = first + j;
        const float vv = v_next, bb = b_next;
        if (j + 1 < n) {
            fetch(t + 1);
            v_next = live ? qkv[(size_t)(t + 1) * qkv_stride + v_off + h * vdim + col] : 0.f;
            b_next = beta[(size_t)(t + 1) * heads + h];
        }
        const float* qs = buf[warp][j & 1] + part * DPT;
        const float* ks = qs + DP;
        const float* gs = ks + DP;
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
            const float4 g4 = *reinterpret_cast<const float4*>(gs + i);
            const float4 k4 = *reinterpret_cast<const float4*>(ks + i);
            S[i] *= g4.x; S[i + 1] *= g4.y; S[i + 2] *= g4.z; S[i + 3] *= g4.w;
            r0 += S[i] * k4.x; r1 += S[i + 1] * k4.y; r2 += S[i + 2] * k4.z; r3 += S[i + 3] * k4.w;
        }
        float r = (r0 + r1) + (r2 + r3);
#pragma unroll
        for (int o = LPC / 2; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        const float u = bb * (vv - r);
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(ks + i);
            const float4 q4 = *reinterpret_cast<const float4*>(qs + i);
            S[i] += k4.x * u; S[i + 1] += k4.y * u; S[i + 2] += k4.z * u; S[i + 3] += k4.w * u;
            o0 += S[i] * q4.x; o1 += S[i + 1] * q4.y; o2 += S[i + 2] * q4.z; o3 += S[i + 3] * q4.w;
        }
        float o = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int s = LPC / 2; s > 0; s >>= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
        if (live && part == 0) out[((size_t)t * heads + h) * vdim + col] = o;
        if (j + 1 < n) stash((j + 1) & 1);
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = part * DPT + i;
        if (live && d < dim) Sg[(size_t)d * vdim + col] = S[i];
    }
}

// ---- (3) ------------------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, const float* __restrict__ gate,
                      size_t gate_stride, TOut* __restrict__ out, int heads, int vdim) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int h = blockIdx.y * nw + warp; h < heads; h += gridDim.y * nw) {
        const float* orow = o + ((size_t)t * heads + h) * vdim;
        const float* grow = gate + (size_t)t * gate_stride + (size_t)h * vdim;
        float ss = 0.f;
        for (int p = lane; p < vdim; p += 32) ss += orow[p] * orow[p];
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)vdim + eps);
        TOut* dst = out + ((size_t)t * heads + h) * vdim;
        for (int p = lane; p < vdim; p += 32)
            dst[p] = from_f32<TOut>(orow[p] * scale * w[p] * (1.0f / (1.0f + expf(-grow[p]))));
    }
}

}  // namespace imparo

using namespace imparo;

// qkv: float32 rows (q heads at q_off, k heads at k_off: kv_heads * dim each), normed in place; bproj: float32 rows with the
// heads' beta inputs at b_off; a: float32 [n_tok, heads * dim], overwritten by the decays; beta: float32 [n_tok, heads].
extern "C" int imparo_delta_prepare(float* qkv, long long qkv_stride, int q_off, int k_off, const float* bproj, long long b_stride,
                                    int b_off, float* a, const float* A_log, const float* dt_bias, float* beta, int n_tok,
                                    int heads, int kv_heads, int dim, float unit_eps, float q_scale, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads) return -2;
    launch(delta_prepare_kernel, dim3(n_tok), dim3(128), 0, stream, qkv, (size_t)qkv_stride, q_off, k_off, bproj, (size_t)b_stride,
           b_off, a, A_log, dt_bias, beta, heads, kv_heads, dim, unit_eps, q_scale);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// state: float32 [n_slots, heads, dim, vdim]; out: float32 [n_tok, heads * vdim].
extern "C" int imparo_delta_scan(const float* qkv, long long qkv_stride, int q_off, int k_off, int v_off, const float* g,
                                 const float* beta, float* state, const int* item_row_start, const int* item_slot, int n_slots,
                                 int n_items, float* out, int heads, int kv_heads, int dim, int vdim, int* status,
                                 cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || dim > 256 || vdim < 1) return -2;
#define IMPARO_DS(DPT_, LPC_) do { \
        const int cpw = 32 / (LPC_); \
        const int warps = (vdim + cpw - 1) / cpw; \
        launch(delta_scan_kernel<DPT_, LPC_>, dim3((warps + DR_WARPS - 1) / DR_WARPS, heads, n_items), dim3(DR_WARPS * 32), 0, stream, \
               qkv, (size_t)qkv_stride, q_off, k_off, v_off, g, beta, state, item_row_start, item_slot, n_slots, out, heads, \
               kv_heads, dim, vdim, status); } while (0)
    if (dim <= 16) IMPARO_DS(16, 1);
    else if (dim <= 32) IMPARO_DS(32, 1);
    else if (dim <= 64) IMPARO_DS(32, 2);
    else if (dim <= 128) IMPARO_DS(32, 4);
    else IMPARO_DS(32, 8);
#undef IMPARO_DS
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// o: float32 [n_tok, heads * vdim]; w: float32 [vdim]; gate: float32 rows of gate_stride floats (heads * vdim used).
extern "C" int imparo_head_norm_gate(const float* o, const float* w, float eps, const float* gate, long long gate_stride,
                                     void* out, int out_dtype, int n_tok, int heads, int vdim, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    const dim3 grid(n_tok, (heads + 15) / 16 > 0 ? (heads + 15) / 16 : 1);
    if (out_dtype == IMPARO_DT_F32)
        launch(head_norm_gate_kernel<float>, grid, dim3(128), 0, stream, o, w, eps, gate, (size_t)gate_stride, (float*)out, heads, vdim);
    else if (out_dtype == IMPARO_DT_BF16)
        launch(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, o, w, eps, gate, (size_t)gate_stride,
               (__nv_bfloat16*)out, heads, vdim);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// The gated delta rule with one decay per head and key channel, over ragged batches, state in the request's slot.
//
// Per value head h (its query/key head is h / (heads / kv_heads)) a request keeps S [dim, vdim] in 32-bit:
//   S <- g * S (row d times g[d]);   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q        (in this order)
//
//  (1) delta_prepare: per row, in 32-bit: q and k of every query/key head divided by sqrt(sum of squares + unit_eps)
//      (q also times q_scale), beta = sigmoid(b), g = exp(-exp(A_log[h]) * softplus(a + dt_bias)) written over a.
//  (2) delta_scan: the value columns of S are independent of one another, so a lane owns a stretch of 4 (8 beyond key
//      size 128) key channels of one column p: LPC lanes share a column, a warp walks a request's rows in order with its
//      32 / LPC columns in registers.  The rows' q, k, g, v and beta pass through shared memory in blocks of four rows
//      that the CTA copies asynchronously two blocks ahead; the two sums over the key channels are finished by shuffles
//      among the LPC lanes, the read-out's off the recurrence's chain.  The additions' order depends on the key size only.
//  (3) head_norm_gate: every head's output divided by its root mean square over vdim, times a weight ([vdim] shared
//      by the heads, or [heads * vdim] with each head's own), times sigmoid(gate).
#include "common.cuh"
#include <type_traits>

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
constexpr int DR_RB = 4;        // rows per staged block
constexpr int DR_ST = 3;        // blocks in flight or in use per warp

__device__ __forceinline__ void dr_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void dr_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// N consecutive floats from shared memory into registers: 16-byte reads where N allows
template <int N>
__device__ __forceinline__ void dr_ld(const float* p, float (&v)[N]) {
    if constexpr (N % 4 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            const float4 q = *reinterpret_cast<const float4*>(p + i);
            v[i] = q.x; v[i + 1] = q.y; v[i + 2] = q.z; v[i + 3] = q.w;
        }
    } else if constexpr (N == 2) {
        const float2 q = *reinterpret_cast<const float2*>(p);
        v[0] = q.x; v[1] = q.y;
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = p[i];
    }
}

__host__ __device__ constexpr int dr_row_floats(int dp, int cols) { return (3 * dp + cols + 1 + 3) & ~3; }   // q | k | g | v of the CTA's columns | beta

// LPC lanes share a value column (dim <= DPT * LPC); a warp has 32 / LPC columns, a CTA DR_WARPS times as many, all of one
// request and head.  The rows' q, k, g, v and beta come through shared memory in blocks of DR_RB rows that the CTA's
// threads copy asynchronously, two blocks ahead of the one in use, so that the walk over a request's rows never waits for
// the memory's latency.  VEC: 16-byte copies (dim, offsets and strides multiples of four floats, 16-byte aligned bases);
// else 4-byte copies.  The additions' order depends on (dim, DPT, LPC) only.
template <int DPT, int LPC, bool VEC>
__global__ void __launch_bounds__(DR_WARPS * 32)
delta_scan_kernel(const float* __restrict__ qkv, size_t qkv_stride, int q_off, int k_off, int v_off,
                  const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ state,
                  const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_slots,
                  float* __restrict__ out, int heads, int kv_heads, int dim, int vdim, int* status) {
    constexpr int DP = DPT * LPC;                   // padded key size
    constexpr int CPW = 32 / LPC;                   // columns per warp
    constexpr int VC = DR_WARPS * CPW;              // columns per CTA
    constexpr int ROWF = dr_row_floats(DP, VC);
    constexpr int THREADS = DR_WARPS * 32;
    extern __shared__ __align__(16) float stage[];  // [DR_ST][DR_RB][ROWF]
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int item = blockIdx.z, h = blockIdx.y;
    const int cta_col0 = blockIdx.x * VC;
    const int col = cta_col0 + warp * CPW + lane / LPC;
    const int part = lane % LPC;
    const int first = item_row_start[item], n = item_row_start[item + 1] - first;
    const int slot = item_slot[item];
    pdl_wait();
    if (slot < 0 || slot >= n_slots) {                                   // (uniform over the CTA)
        if (tid == 0 && blockIdx.x == 0) report(status, IMPARO_ST_SLOT_RANGE, 73, item, slot);
        return;
    }
    const bool live = col < vdim;
    const bool busy = cta_col0 + warp * CPW < vdim;                      // a warp without columns only copies and waits
    const int kvh = h / (heads / kv_heads);
    float* Sg = state + (((size_t)slot * heads + h) * dim) * vdim;
    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = part * DPT + i;
        S[i] = (live && d < dim) ? Sg[(size_t)d * vdim + col] : 0.f;
    }
    const int n_blocks = (n + DR_RB - 1) / DR_RB;
    // FAST (16-byte copies and dim > 32): a thread copies the same pieces of every block, so where they come from and go
    // to is worked out once: ITEMS 16-byte groups of q | k | g (an offset from the block's first row; the row and the place
    // in the stage packed into one word) and VB values or betas.  Stretches beyond dim and vdim stay zero from the start.
    constexpr bool FAST = VEC && DP >= 64;
    constexpr int GROUPS = DR_RB * 3 * DP / 4;                           // 16-byte groups of a block
    constexpr int ITEMS = FAST ? (GROUPS + THREADS - 1) / THREADS : 1;
    constexpr int VB = FAST ? (DR_RB * (VC + 1) + THREADS - 1) / THREADS : 1;
    int f_off[ITEMS], f_key[ITEMS];                  // key: place in the stage | row << 24 | from g << 28; -1: nothing
    const float* vb_ptr[VB];
    size_t vb_step[VB];
    int vb_key[VB];
    if (FAST) {
        constexpr int VPS = DP / 4, VPR = 3 * VPS;
        for (int e = tid; e < DR_ST * DR_RB * ROWF; e += THREADS) stage[e] = 0.f;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int e = tid + THREADS * i;
            const int r = e / VPR, c = e % VPR;
            const int which = c / VPS, d = (c % VPS) * 4;
            f_off[i] = which == 2 ? (r * heads + h) * dim + d : r * (int)qkv_stride + (which == 0 ? q_off : k_off) + kvh * dim + d;
            f_key[i] = (e < GROUPS && d < dim) ? ((r * ROWF + which * DP + d) | (r << 24) | ((which == 2) << 28)) : -1;
        }
#pragma unroll
        for (int j = 0; j < VB; ++j) {
            const int e = tid + THREADS * j;
            const int r = e / (VC + 1), c = e % (VC + 1);
            vb_ptr[j] = nullptr; vb_step[j] = 0; vb_key[j] = -1;
            if (e < DR_RB * (VC + 1)) {
                if (c == VC) {
                    vb_ptr[j] = beta + (size_t)(first + r) * heads + h;
                    vb_step[j] = (size_t)DR_RB * heads;
                    vb_key[j] = (r * ROWF + 3 * DP + c) | (r << 24);
                } else if (cta_col0 + c < vdim) {
                    vb_ptr[j] = qkv + (size_t)(first + r) * qkv_stride + v_off + h * vdim + cta_col0 + c;
                    vb_step[j] = (size_t)DR_RB * qkv_stride;
                    vb_key[j] = (r * ROWF + 3 * DP + c) | (r << 24);
                }
            }
        }
        __syncthreads();
    }
    auto issue = [&](int b) {
        if (b < n_blocks) {
            float* dst = stage + (b % DR_ST) * DR_RB * ROWF;
            const int t0 = first + b * DR_RB, nb = min(DR_RB, n - b * DR_RB);
            if (FAST) {
                const float* base_q = qkv + (size_t)t0 * qkv_stride;
                const float* base_g = g + (size_t)t0 * heads * dim;
#pragma unroll
                for (int i = 0; i < ITEMS; ++i) {
                    const int key = f_key[i];
                    if (key >= 0 && ((key >> 24) & 15) < nb) dr_cp16(dst + (key & 0xffffff), ((key >> 28) & 1 ? base_g : base_q) + f_off[i]);
                }
#pragma unroll
                for (int j = 0; j < VB; ++j) {
                    if (vb_key[j] >= 0 && (vb_key[j] >> 24) < nb) dr_cp4(dst + (vb_key[j] & 0xffffff), vb_ptr[j]);
                    vb_ptr[j] += vb_step[j];
                }
            } else {
                for (int e = tid; e < nb * 3 * DP; e += THREADS) {
                    const int r = e / (3 * DP), c = e % (3 * DP);
                    const int which = c / DP, d = c % DP;
                    float* to = dst + r * ROWF + c;
                    if (d < dim) {
                        const float* src = which == 2 ? g + ((size_t)(t0 + r) * heads + h) * dim + d
                                                      : qkv + (size_t)(t0 + r) * qkv_stride + (which == 0 ? q_off : k_off) + kvh * dim + d;
                        dr_cp4(to, src);
                    } else {
                        *to = 0.f;
                    }
                }
                for (int e = tid; e < nb * (VC + 1); e += THREADS) {     // the values of this CTA's columns, and beta
                    const int r = e / (VC + 1), c = e % (VC + 1);
                    float* to = dst + r * ROWF + 3 * DP + c;
                    if (c == VC) dr_cp4(to, beta + (size_t)(t0 + r) * heads + h);
                    else if (cta_col0 + c < vdim) dr_cp4(to, qkv + (size_t)(t0 + r) * qkv_stride + v_off + h * vdim + cta_col0 + c);
                    else *to = 0.f;
                }
            }
        }
        dr_commit();                                                     // (an empty group keeps the count in step)
    };
    issue(0);
    issue(1);
    for (int b = 0; b < n_blocks; ++b) {
        dr_wait1();                                                      // this thread's copies of block b are done
        __syncthreads();                                                 // ... and everybody's; block b - 1 is no longer read
        issue(b + 2);                                                    // into the stage that block b - 1 has left
        if (!busy) continue;
        const float* src = stage + (b % DR_ST) * DR_RB * ROWF;
        const int nb = min(DR_RB, n - b * DR_RB);
        float o_part[DR_RB];
        auto rows = [&](auto whole) {                                    // whole: the block has all its rows, nothing to test
#pragma unroll
        for (int r = 0; r < DR_RB; ++r) {
            o_part[r] = 0.f;
            if (decltype(whole)::value || r < nb) {
                const float* row = src + r * ROWF;
                const float vv = row[3 * DP + warp * CPW + lane / LPC], bb = row[3 * DP + VC];
                float gv[DPT], kv[DPT], qv[DPT];
                dr_ld<DPT>(row + 2 * DP + part * DPT, gv);
                dr_ld<DPT>(row + DP + part * DPT, kv);
                dr_ld<DPT>(row + part * DPT, qv);
                float rp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    S[i] *= gv[i];
                    rp[i & 3] += S[i] * kv[i];
                }
                float rs = (rp[0] + rp[1]) + (rp[2] + rp[3]);
#pragma unroll
                for (int o = LPC / 2; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
                const float u = bb * (vv - rs);
                float op[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    S[i] += kv[i] * u;
                    op[i & 3] += S[i] * qv[i];
                }
                o_part[r] = (op[0] + op[1]) + (op[2] + op[3]);
            }
        }
        };
        if (nb == DR_RB) rows(std::true_type{}); else rows(std::false_type{});
        // the read-outs' sums over the lanes of a column: off the recurrence's chain, the block's rows side by side
#pragma unroll
        for (int s2 = LPC / 2; s2 > 0; s2 >>= 1) {
#pragma unroll
            for (int r = 0; r < DR_RB; ++r) o_part[r] += __shfl_xor_sync(0xffffffffu, o_part[r], s2);
        }
        if (live && part == 0) {
#pragma unroll
            for (int r = 0; r < DR_RB; ++r)
                if (r < nb) out[((size_t)(first + b * DR_RB + r) * heads + h) * vdim + col] = o_part[r];
        }
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
                      size_t gate_stride, TOut* __restrict__ out, int heads, int vdim, int w_head_stride) {
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
        const float* wh = w + (size_t)h * w_head_stride;
        for (int p = lane; p < vdim; p += 32)
            dst[p] = from_f32<TOut>(orow[p] * scale * wh[p] * (1.0f / (1.0f + expf(-grow[p]))));
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
    const bool vec = dim % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && qkv_stride % 4 == 0 &&
                     (((uintptr_t)qkv | (uintptr_t)g) & 15) == 0;
    cudaError_t e = cudaSuccess;
#define IMPARO_DS(DPT_, LPC_, VEC_) do { \
        constexpr int cols = DR_WARPS * (32 / (LPC_)); \
        constexpr size_t smem = (size_t)DR_ST * DR_RB * dr_row_floats((DPT_) * (LPC_), cols) * sizeof(float); \
        static bool configured = false; \
        if (!configured) { \
            e = cudaFuncSetAttribute(delta_scan_kernel<DPT_, LPC_, VEC_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; \
        } \
        launch(delta_scan_kernel<DPT_, LPC_, VEC_>, dim3((vdim + cols - 1) / cols, heads, n_items), dim3(DR_WARPS * 32), smem, stream, \
               qkv, (size_t)qkv_stride, q_off, k_off, v_off, g, beta, state, item_row_start, item_slot, n_slots, out, heads, \
               kv_heads, dim, vdim, status); } while (0)
#define IMPARO_DS2(DPT_, LPC_) do { if (vec) IMPARO_DS(DPT_, LPC_, true); else IMPARO_DS(DPT_, LPC_, false); } while (0)
    // four key channels per lane (measured at key size 64 and 2,048 rows: 8 per lane 560 us, 4 per lane 415 us, 2 per lane
    // 520 us), eight where a column would need more than a warp
    if (dim <= 4) IMPARO_DS2(4, 1);
    else if (dim <= 8) IMPARO_DS2(4, 2);
    else if (dim <= 16) IMPARO_DS2(4, 4);
    else if (dim <= 32) IMPARO_DS2(4, 8);
    else if (dim <= 64) IMPARO_DS2(4, 16);
    else if (dim <= 128) IMPARO_DS2(4, 32);
    else IMPARO_DS2(8, 32);
#undef IMPARO_DS2
#undef IMPARO_DS
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// o: float32 [n_tok, heads * vdim]; w: float32 [vdim] (w_head_stride 0) or [heads * vdim] (w_head_stride vdim); gate: float32
// rows of gate_stride floats (heads * vdim used).
extern "C" int imparo_head_norm_gate(const float* o, const float* w, float eps, const float* gate, long long gate_stride,
                                     void* out, int out_dtype, int n_tok, int heads, int vdim, int w_head_stride,
                                     cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    const dim3 grid(n_tok, (heads + 15) / 16 > 0 ? (heads + 15) / 16 : 1);
    if (out_dtype == IMPARO_DT_F32)
        launch(head_norm_gate_kernel<float>, grid, dim3(128), 0, stream, o, w, eps, gate, (size_t)gate_stride, (float*)out, heads, vdim, w_head_stride);
    else if (out_dtype == IMPARO_DT_BF16)
        launch(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, o, w, eps, gate, (size_t)gate_stride,
               (__nv_bfloat16*)out, heads, vdim, w_head_stride);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

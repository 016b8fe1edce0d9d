// A routed feed-forward (mixture of experts) over the rows of a step.
//
//  (1) moe_route: router logits z = W_r h in 32-bit (a warp per expert, four rows per block), then a warp per row picks the
//      `top` largest (by logit: the scores sigmoid(z) or softmax(z) are monotone in it; ties: the lower expert), optionally
//      renormalised to sum 1.  Leaves expert ids [rows, top] and weights [rows, top].
//  (2) moe_rows_*: each (row, choice) pair on its own: the expert's gate and up rows times the (optionally weighted)
//      input, silu(gate) * up, then the expert's down rows; the choices of a row are added in order.  Weights are
//      streamed once per pair: the form for steps of few rows.
//  (3) moe_group_*: pairs sorted by expert (a counting sort whose order inside an expert is the row order, so the
//      result does not depend on what else is in the step), tiles of 32 pairs x 64 outputs per CTA: bfloat16 on
//      tensor cores (mma.sync through wmma fragments, 32-bit accumulation), 32-bit with FFMA.  The tile list is made
//      on the device from the counts; CTAs beyond it leave at once, so the launch depends on (rows, top, experts)
//      only.
//
// Expert e's matrices: w_gu[e] = [gate; up] ([2 ff, width]), w_down[e] ([width, ff]).  The weight multiplies the
// expert's input (weight_input = 1) or its output (0).
#include "common.cuh"
#include <mma.h>

namespace imparo {

// A warp's dot product of a matrix row with a vector in shared memory (32-bit).  When the row is 16 bytes wide per
// lane and turn (VEC), lanes read 16 bytes at a time, four loads in flight; the order of additions is fixed either way.
template <typename T> struct Vec16 { static constexpr int N = 16 / (int)sizeof(T); };

template <typename T>
__device__ __forceinline__ float dot16(const uint4 raw, const float* __restrict__ x) {
    float a = 0.f;
    if constexpr (sizeof(T) == 2) {
        const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float2 f = __bfloat1622float2(v[u]);
            a = fmaf(f.x, x[2 * u], a);
            a = fmaf(f.y, x[2 * u + 1], a);
        }
    } else {
        const float* v = reinterpret_cast<const float*>(&raw);
#pragma unroll
        for (int u = 0; u < 4; ++u) a = fmaf(v[u], x[u], a);
    }
    return a;
}

template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ x, int n, bool vec, int lane) {
    float acc = 0.f;
    if (vec) {
        constexpr int PER = Vec16<T>::N;
        const uint4* w4 = reinterpret_cast<const uint4*>(w);
        const int n4 = n / PER;
        int i = lane;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (; i + 96 < n4; i += 128) {
            const uint4 r0 = w4[i], r1 = w4[i + 32], r2 = w4[i + 64], r3 = w4[i + 96];
            a0 += dot16<T>(r0, x + (size_t)i * PER);
            a1 += dot16<T>(r1, x + (size_t)(i + 32) * PER);
            a2 += dot16<T>(r2, x + (size_t)(i + 64) * PER);
            a3 += dot16<T>(r3, x + (size_t)(i + 96) * PER);
        }
        for (; i < n4; i += 32) a0 += dot16<T>(w4[i], x + (size_t)i * PER);
        acc = (a0 + a1) + (a2 + a3);
    } else {
        for (int i = lane; i < n; i += 32) acc += to_f32(w[i]) * x[i];
    }
    return warp_sum(acc);
}

// ---- (1) router -------------------------------------------------------------------------------------------------
// Logits: a block takes up to four rows (a router row read once serves them all) and eight experts, a warp each; grid
// (row blocks, ceil(experts / 8)).  A dot product always adds in the same order, whatever else the launch holds.
template <typename T>
__global__ void __launch_bounds__(256)
moe_logits_kernel(const T* __restrict__ h, const float* __restrict__ w_r, int n_rows, int width, int experts, int rows_per_block,
                  float* __restrict__ logits) {
    extern __shared__ __align__(16) float route_smem[];  // [rows][width] the rows in 32-bit
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = blockIdx.x * rows_per_block;
    const int R = min(rows_per_block, n_rows - r0);
    float* rows = route_smem;
    for (int i = threadIdx.x; i < R * width; i += blockDim.x) rows[i] = to_f32(h[(size_t)r0 * width + i]);
    __syncthreads();
    const int e = blockIdx.y * 8 + warp;
    if (e >= experts) return;
    const float* wr = w_r + (size_t)e * width;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (width % 4 == 0) {
        const float4* w4 = reinterpret_cast<const float4*>(wr);
        const int n4 = width / 4;
        int i = lane;
        for (; i + 96 < n4; i += 128) {                      // four loads in flight
            float4 u[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) u[k] = w4[i + 32 * k];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (r < R) {
                    const float* x = rows + (size_t)r * width + 4 * i;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        acc[r] += u[k].x * x[128 * k] + u[k].y * x[128 * k + 1] + u[k].z * x[128 * k + 2] + u[k].w * x[128 * k + 3];
                }
            }
        }
        for (; i < n4; i += 32) {
            const float4 u = w4[i];
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (r < R) {
                    const float* x = rows + (size_t)r * width + 4 * i;
                    acc[r] += u.x * x[0] + u.y * x[1] + u.z * x[2] + u.w * x[3];
                }
        }
    } else {
        for (int i = lane; i < width; i += 32) {
            const float u = wr[i];
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (r < R) acc[r] += u * rows[(size_t)r * width + i];
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && r < R) logits[(size_t)(r0 + r) * experts + e] = v;
    }
}

// The choice: a warp per row, four rows per block
// logits: [n_rows, parts * experts]; a logit is the sum of its `parts` entries, experts apart, added in order (parts > 1:
// the router matrix was cut into bfloat16 pieces whose sum is the 32-bit matrix to its last bit, see imparo_moe_pick)
__global__ void __launch_bounds__(128)
moe_pick_kernel(const float* __restrict__ logits, int n_rows, int experts, int parts, int top, int softmax_scores, int renormalise,
                int groups, int keep, float renorm_eps, float weight_scale, int out_stride, int* __restrict__ ids,
                float* __restrict__ wts) {
    extern __shared__ __align__(16) float pick_smem[];   // [4][experts] scores, then [4][groups] maxima of the groups
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x * 4 + warp;
    if (r >= n_rows) return;
    float* s = pick_smem + (size_t)warp * experts;
    for (int e = lane; e < experts; e += 32) {
        const float* l = logits + (size_t)r * parts * experts + e;
        float v = l[0];
        for (int k = 1; k < parts; ++k) v += l[(size_t)k * experts];
        s[e] = v;
    }
    __syncwarp();
    // The choice goes by the logits: scores are monotone in them, and a sigmoid that has reached 1 in 32-bit would tie.
    float m = -INFINITY, l = 1.f;
    if (softmax_scores) {
        for (int e = lane; e < experts; e += 32) m = fmaxf(m, s[e]);
        m = warp_max(m);
        l = 0.f;
        for (int e = lane; e < experts; e += 32) l += expf(s[e] - m);
        l = warp_sum(l);
    }
    // Experts in `groups` equal groups of neighbours: a group's score is its largest, and only the `keep` best groups'
    // experts stay candidates (ties: the lower group).  The others leave the candidates; the softmax above counted them.
    if (groups > 1 && keep < groups) {
        const int per = experts / groups;
        // every group's maximum first (a lane per group), then a lane per group counts the groups that beat its own: a group
        // is kept when fewer than `keep` do.  All verdicts are in before any score is masked.
        float* gmax = pick_smem + (size_t)4 * experts + (size_t)warp * groups;
        for (int g = lane; g < groups; g += 32) {
            float mx = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) mx = fmaxf(mx, s[e]);
            gmax[g] = mx;
        }
        __syncwarp();
        for (int g = lane; g < groups; g += 32) {
            const float mine = gmax[g];
            int beaten = 0;
            for (int o = 0; o < groups; ++o) {
                const float other = gmax[o];
                if (other > mine || (other == mine && o < g)) ++beaten;
            }
            if (beaten >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) s[e] = -INFINITY;
        }
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = s[e];
            if (v > best) { best = v; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        const float score = softmax_scores ? expf(best - m) / l : 1.0f / (1.0f + expf(-best));
        if (lane == 0) {
            ids[(size_t)r * out_stride + k] = arg;
            wts[(size_t)r * out_stride + k] = score;
            s[arg] = -INFINITY;
        }
        total += score;
        __syncwarp();
    }
    if (renormalise && lane < top) wts[(size_t)r * out_stride + lane] = wts[(size_t)r * out_stride + lane] / (total + renorm_eps) * weight_scale;
    else if (weight_scale != 1.0f && lane < top) wts[(size_t)r * out_stride + lane] *= weight_scale;
    // choices beyond `top` (out_stride > top) are experts every row uses with weight 1: numbers experts, experts + 1, ...
    for (int k = top + lane; k < out_stride; k += 32) {
        ids[(size_t)r * out_stride + k] = experts + (k - top);
        wts[(size_t)r * out_stride + k] = 1.0f;
    }
}

// ---- (2) pair by pair ---------------------------------------------------------------------------------------------
// two rows against the same vector at once: eight loads in flight
template <typename T>
__device__ __forceinline__ void warp_dot2(const T* __restrict__ w0, const T* __restrict__ w1, const float* __restrict__ x, int n,
                                          bool vec, int lane, float& r0, float& r1) {
    if (!vec) {
        r0 = warp_dot<T>(w0, x, n, false, lane);
        r1 = warp_dot<T>(w1, x, n, false, lane);
        return;
    }
    constexpr int PER = Vec16<T>::N;
    const uint4* p0 = reinterpret_cast<const uint4*>(w0);
    const uint4* p1 = reinterpret_cast<const uint4*>(w1);
    const int n4 = n / PER;
    int i = lane;
    float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
    for (; i + 96 < n4; i += 128) {
        uint4 u[4], v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) { u[k] = p0[i + 32 * k]; v[k] = p1[i + 32 * k]; }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            a[k] += dot16<T>(u[k], x + (size_t)(i + 32 * k) * PER);
            b[k] += dot16<T>(v[k], x + (size_t)(i + 32 * k) * PER);
        }
    }
    for (; i < n4; i += 32) {
        a[0] += dot16<T>(p0[i], x + (size_t)i * PER);
        b[0] += dot16<T>(p1[i], x + (size_t)i * PER);
    }
    r0 = warp_sum((a[0] + a[1]) + (a[2] + a[3]));
    r1 = warp_sum((b[0] + b[1]) + (b[2] + b[3]));
}

// grid (rows * top, ceil(ff / 32)); 8 warps, each 4 features
template <typename T>
__global__ void __launch_bounds__(256)
moe_rows_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gu, const int* __restrict__ ids, const float* __restrict__ wts,
                   int width, int ff, int top, int experts, int weight_input, int act, float limit, T* __restrict__ mid) {
    extern __shared__ __align__(16) float up_smem[];
    pdl_trigger();
    pdl_wait();
    const int pair = blockIdx.x, r = pair / top;
    const int e = ids[pair];
    if (e < 0 || e >= experts) return;
    const float wt = weight_input ? wts[pair] : 1.0f;
    const T* hr = h + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) up_smem[i] = to_f32(from_f32<T>(wt * to_f32(hr[i])));
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* base = w_gu + (size_t)e * 2 * ff * width;
    const bool vec = width % Vec16<T>::N == 0 && ((uintptr_t)w_gu & 15) == 0;
    for (int j = 0; j < 4; ++j) {
        const int f = blockIdx.y * 32 + warp * 4 + j;
        if (f >= ff) break;
        float ag, au;
        warp_dot2<T>(base + (size_t)f * width, base + (size_t)(ff + f) * width, up_smem, width, vec, lane, ag, au);
        if (lane == 0) mid[(size_t)pair * ff + f] = from_f32<T>(gated_act(act, limit, ag, au));
    }
}

// grid (rows, ceil(width / 32)); 8 warps, each 4 outputs; out float32 [rows, width] is overwritten
template <typename T>
__global__ void __launch_bounds__(256)
moe_rows_down_kernel(const T* __restrict__ mid, const T* __restrict__ w_down, const int* __restrict__ ids,
                     const float* __restrict__ wts, int width, int ff, int top, int experts, int weight_input,
                     float* __restrict__ out) {
    extern __shared__ __align__(16) float down_smem[];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool vec = ff % Vec16<T>::N == 0 && ((uintptr_t)w_down & 15) == 0;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top; ++k) {
        const int pair = r * top + k;
        const int e = ids[pair];
        __syncthreads();
        for (int i = threadIdx.x; i < ff; i += blockDim.x) down_smem[i] = to_f32(mid[(size_t)pair * ff + i]);
        __syncthreads();
        if (e < 0 || e >= experts) continue;
        const float wt = weight_input ? 1.0f : wts[pair];
        for (int j = 0; j < 4; ++j) {
            const int o = blockIdx.y * 32 + warp * 4 + j;
            if (o >= width) break;
            acc[j] += wt * warp_dot<T>(w_down + ((size_t)e * width + o) * ff, down_smem, ff, vec, lane);
        }
    }
    if (lane == 0)
        for (int j = 0; j < 4; ++j) {
            const int o = blockIdx.y * 32 + warp * 4 + j;
            if (o < width) out[(size_t)r * width + o] = acc[j];
        }
}

// ---- (3) grouped by expert ----------------------------------------------------------------------------------------
constexpr int GM = 32, GN = 64, GK = 32;          // tile: pairs x outputs, K step

// One block: counts per expert, offsets, the sorted pair list (stable: by expert, then by pair index) and the tile list.
// plan: [0] number of tiles; tile_expert[t], tile_first[t] (index into sorted), tile_rows[t]
__global__ void __launch_bounds__(1024)
moe_group_plan_kernel(const int* __restrict__ ids, int n_pairs, int experts, int* __restrict__ sorted,
                      int* __restrict__ expert_start, int* __restrict__ plan, int max_tiles) {
    extern __shared__ int plan_smem[];               // experts + 1 offsets
    pdl_trigger();
    pdl_wait();
    int* start = plan_smem;
    const int tid = threadIdx.x;
    // thread e counts its expert's pairs and then writes them in pair order: the order inside an expert is by row
    for (int e = tid; e <= experts; e += blockDim.x) start[e] = 0;
    __syncthreads();
    for (int e = tid; e < experts; e += blockDim.x) {
        int c = 0;
        for (int i = 0; i < n_pairs; ++i) c += ids[i] == e;
        start[e + 1] = c;
    }
    __syncthreads();
    if (tid == 0) {
        int tiles = 0;
        for (int e = 0; e < experts; ++e) {
            const int c = start[e + 1];
            start[e + 1] = start[e] + c;
            for (int lo = 0; lo < c && tiles < max_tiles; lo += GM) {
                plan[1 + 3 * tiles] = e;
                plan[2 + 3 * tiles] = start[e] + lo;
                plan[3 + 3 * tiles] = min(GM, c - lo);
                ++tiles;
            }
        }
        plan[0] = tiles;
    }
    __syncthreads();
    for (int e = tid; e < experts; e += blockDim.x) {
        int at = start[e];
        expert_start[e] = at;
        for (int i = 0; i < n_pairs; ++i)
            if (ids[i] == e) sorted[at++] = i;
    }
    if (tid == 0) expert_start[experts] = start[experts];
}

// A[m, k]: row `pair_of[m]` of the operand (times its weight when asked), B[n, k]: the expert's matrix rows.
// bfloat16: wmma 16x16x16, 8 warps as 2 (m) x 4 (n); float32: each thread a 2 x 4 patch with FFMA.
template <typename T> struct GroupTile;

template <> struct __align__(32) GroupTile<__nv_bfloat16> {
    using T = __nv_bfloat16;
    static constexpr int LDS = GK + 8;
    T a[GM][LDS];
    T b[GN][LDS];
    float c[GM][GN + 4];
};
template <> struct __align__(32) GroupTile<float> {
    static constexpr int LDS = GK + 1;
    float a[GM][LDS];
    float b[GN][LDS];
    float c[GM][GN + 4];
};

// acc tile = A (GM x K) * B^T (GN x K); result left in sm.c
template <typename T, typename LoadA>
__device__ __forceinline__ void group_tile_product(GroupTile<T>& sm, LoadA load_a, const T* __restrict__ bmat, int n0, int n_rows_b,
                                                   int K, int rows) {
    const int tid = threadIdx.x;
    if constexpr (sizeof(T) == 2) {
        using namespace nvcuda;
        const int warp = tid >> 5, wm = warp >> 2, wn = warp & 3;
        wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
        wmma::fill_fragment(acc, 0.f);
        for (int k0 = 0; k0 < K; k0 += GK) {
            __syncthreads();
            for (int i = tid; i < GM * GK; i += 256) {
                const int m = i / GK, k = i % GK;
                sm.a[m][k] = (m < rows && k0 + k < K) ? load_a(m, k0 + k) : from_f32<T>(0.f);
            }
            for (int i = tid; i < GN * GK; i += 256) {
                const int n = i / GK, k = i % GK;
                sm.b[n][k] = (n0 + n < n_rows_b && k0 + k < K) ? bmat[(size_t)(n0 + n) * K + k0 + k] : from_f32<T>(0.f);
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < GK; kk += 16) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
                wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
                wmma::load_matrix_sync(fa, &sm.a[wm * 16][kk], GroupTile<T>::LDS);
                wmma::load_matrix_sync(fb, &sm.b[wn * 16][kk], GroupTile<T>::LDS);
                wmma::mma_sync(acc, fa, fb, acc);
            }
        }
        wmma::store_matrix_sync(&sm.c[wm * 16][wn * 16], acc, GN + 4, wmma::mem_row_major);
        __syncthreads();
    } else {
        const int tm = (tid >> 4) * 2, tn = (tid & 15) * 4;      // 16 x 16 threads, 2 x 4 each
        float acc[2][4] = {};
        for (int k0 = 0; k0 < K; k0 += GK) {
            __syncthreads();
            for (int i = tid; i < GM * GK; i += 256) {
                const int m = i / GK, k = i % GK;
                sm.a[m][k] = (m < rows && k0 + k < K) ? load_a(m, k0 + k) : 0.f;
            }
            for (int i = tid; i < GN * GK; i += 256) {
                const int n = i / GK, k = i % GK;
                sm.b[n][k] = (n0 + n < n_rows_b && k0 + k < K) ? bmat[(size_t)(n0 + n) * K + k0 + k] : 0.f;
            }
            __syncthreads();
            const int kn = min(GK, K - k0);
            for (int k = 0; k < kn; ++k) {
                float av[2], bv[4];
#pragma unroll
                for (int i = 0; i < 2; ++i) av[i] = sm.a[tm + i][k];
#pragma unroll
                for (int j = 0; j < 4; ++j) bv[j] = sm.b[tn + j][k];
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) sm.c[tm + i][tn + j] = acc[i][j];
        __syncthreads();
    }
}

// grid (max_tiles, ceil(ff / 64)): mid[pair, f] = silu(gate) * up for the tile's pairs; gate and up as two products
template <typename T>
__global__ void __launch_bounds__(256)
moe_group_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gu, const int* __restrict__ sorted, const int* __restrict__ plan,
                    const float* __restrict__ wts, int width, int ff, int top, int weight_input, int act, float limit,
                    T* __restrict__ mid) {
    __shared__ GroupTile<T> sm;
    __shared__ int pair_of[GM];
    __shared__ float wt_of[GM];
    __shared__ float gate_c[GM][GN];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int e = plan[1 + 3 * tile], first = plan[2 + 3 * tile], rows = plan[3 + 3 * tile];
    if (threadIdx.x < GM) {
        const int p = threadIdx.x < rows ? sorted[first + threadIdx.x] : -1;
        pair_of[threadIdx.x] = p;
        wt_of[threadIdx.x] = (p >= 0 && weight_input) ? wts[p] : 1.0f;
    }
    __syncthreads();
    const int n0 = blockIdx.y * GN;
    auto load_a = [&](int m, int k) -> T {
        return from_f32<T>(wt_of[m] * to_f32(h[(size_t)(pair_of[m] / top) * width + k]));
    };
    const T* base = w_gu + (size_t)e * 2 * ff * width;
    group_tile_product<T>(sm, load_a, base, n0, ff, width, rows);
    for (int i = threadIdx.x; i < GM * GN; i += 256) gate_c[i / GN][i % GN] = sm.c[i / GN][i % GN];
    group_tile_product<T>(sm, load_a, base + (size_t)ff * width, n0, ff, width, rows);
    for (int i = threadIdx.x; i < GM * GN; i += 256) {
        const int m = i / GN, n = i % GN;
        if (m < rows && n0 + n < ff) mid[(size_t)pair_of[m] * ff + n0 + n] = from_f32<T>(gated_act(act, limit, gate_c[m][n], sm.c[m][n]));
    }
}

// grid (max_tiles, ceil(width / 64)): pair_out[pair, o] = down row o . mid[pair]  (times the weight when it is on the output)
template <typename T>
__global__ void __launch_bounds__(256)
moe_group_down_kernel(const T* __restrict__ mid, const T* __restrict__ w_down, const int* __restrict__ sorted,
                      const int* __restrict__ plan, const float* __restrict__ wts, int width, int ff, int weight_input,
                      float* __restrict__ pair_out) {
    __shared__ GroupTile<T> sm;
    __shared__ int pair_of[GM];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int e = plan[1 + 3 * tile], first = plan[2 + 3 * tile], rows = plan[3 + 3 * tile];
    if (threadIdx.x < GM) pair_of[threadIdx.x] = threadIdx.x < rows ? sorted[first + threadIdx.x] : -1;
    __syncthreads();
    const int n0 = blockIdx.y * GN;
    auto load_a = [&](int m, int k) -> T { return mid[(size_t)pair_of[m] * ff + k]; };
    group_tile_product<T>(sm, load_a, w_down + (size_t)e * width * ff, n0, width, ff, rows);
    for (int i = threadIdx.x; i < GM * GN; i += 256) {
        const int m = i / GN, n = i % GN;
        if (m < rows && n0 + n < width) {
            const float wt = weight_input ? 1.0f : wts[pair_of[m]];
            pair_out[(size_t)pair_of[m] * width + n0 + n] = wt * sm.c[m][n];
        }
    }
}

// out[r, :] = sum over the row's choices, in order
__global__ void __launch_bounds__(256)
moe_sum_pairs_kernel(const float* __restrict__ pair_out, int n_rows, int width, int top, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)n_rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width, c = i - r * width;
        float a = 0.f;
        for (int k = 0; k < top; ++k) a += pair_out[(r * top + k) * width + c];
        out[i] = a;
    }
}

// ---- (4) sorted into tiles of 128 rows for the tensor-memory product (gemm_prefill.cu, grouped) --------------------------
// One block.  Every pair gets a row in a buffer in which each expert's rows start at a multiple of 128: slot_of_pair[p];
// tile_group[t] names the expert of row tile t, -1 beyond the last used tile.  Inside an expert the rows keep the pairs'
// order.  Shared memory: (32 + 2) * experts ints.
constexpr int TILE_ROWS = 128;

__global__ void __launch_bounds__(1024)
moe_tile_plan_kernel(const int* __restrict__ ids, int n_pairs, int experts, int* __restrict__ slot_of_pair,
                     int* __restrict__ tile_group, int max_tiles) {
    extern __shared__ int tp_smem[];
    int* warp_counts = tp_smem;                          // [32][experts]
    int* base = tp_smem + 32 * experts;                  // [experts] pairs seen so far
    int* start_row = base + experts;                     // [experts] first row of the expert's stretch
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = tid; e < experts; e += blockDim.x) base[e] = 0;
    for (int p0 = 0; p0 < n_pairs; p0 += 1024) {
        for (int i = tid; i < 32 * experts; i += blockDim.x) warp_counts[i] = 0;
        __syncthreads();
        const int p = p0 + tid;
        int e = p < n_pairs ? ids[p] : -1;
        if (e >= experts) e = -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        if (e >= 0 && rank == 0) warp_counts[warp * experts + e] = __popc(same);
        __syncthreads();
        for (int x = tid; x < experts; x += blockDim.x) {
            int run = base[x];
            for (int w = 0; w < 32; ++w) {
                const int c = warp_counts[w * experts + x];
                warp_counts[w * experts + x] = run;
                run += c;
            }
            base[x] = run;
        }
        __syncthreads();
        if (p < n_pairs) slot_of_pair[p] = e >= 0 ? warp_counts[warp * experts + e] + rank : -1;
        __syncthreads();
    }
    if (tid == 0) {
        int t = 0;
        for (int e = 0; e < experts; ++e) {
            start_row[e] = t * TILE_ROWS;
            const int n = (base[e] + TILE_ROWS - 1) / TILE_ROWS;
            for (int i = 0; i < n && t < max_tiles; ++i) tile_group[t++] = e;
        }
        for (; t < max_tiles; ++t) tile_group[t] = -1;
    }
    __syncthreads();
    for (int p = tid; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < experts && slot_of_pair[p] >= 0) slot_of_pair[p] += start_row[e];
    }
}

// xg[slot_of_pair[p], :] = bfloat16(weight * h[p / top, :]); a block per pair, 16 bytes per thread and turn
__global__ void __launch_bounds__(128)
moe_tile_gather_kernel(const __nv_bfloat16* __restrict__ h, const int* __restrict__ slot_of_pair, const float* __restrict__ wts,
                       int width, int top, int weight_input, __nv_bfloat16* __restrict__ xg) {
    pdl_trigger();
    pdl_wait();
    const int p = blockIdx.x;
    const int slot = slot_of_pair[p];
    if (slot < 0) return;
    const float wt = weight_input ? wts[p] : 1.0f;
    const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(p / top) * width);
    uint4* dst = reinterpret_cast<uint4*>(xg + (size_t)slot * width);
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) {
        uint4 raw = src[i];
        if (weight_input) {
            __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float2 f = __bfloat1622float2(v[u]);
                v[u] = __floats2bfloat162_rn(wt * f.x, wt * f.y);
            }
        }
        dst[i] = raw;
    }
}

// out[r, :] = sum over the row's choices, in order, of out_g[slot_of_pair[r * top + k], :]  (times the weight when it
// multiplies the output); width a multiple of 4
__global__ void __launch_bounds__(256)
moe_tile_sum_kernel(const float* __restrict__ out_g, const int* __restrict__ slot_of_pair, const float* __restrict__ wts,
                    int width, int top, int weight_input, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < top; ++k) {
            const int slot = slot_of_pair[r * top + k];
            if (slot < 0) continue;
            const float wt = weight_input ? 1.0f : wts[r * top + k];
            const float4 v = *reinterpret_cast<const float4*>(out_g + (size_t)slot * width + c);
            a.x += wt * v.x; a.y += wt * v.y; a.z += wt * v.z; a.w += wt * v.w;
        }
        *reinterpret_cast<float4*>(out + (size_t)r * width + c) = a;
    }
}

}  // namespace imparo

using namespace imparo;

// logits: float32 scratch [n_rows, experts].  Two launches.
// The choice's further parameters (both entry points): groups, keep (experts in `groups` equal groups of neighbours, only the
// `keep` best groups' experts may be chosen; groups <= 1: all), renorm_eps (added to the chosen scores' sum before the
// division when renormalise is set), weight_scale (a factor on the weights), out_stride (ids and wts have out_stride >= top
// entries per row: the entries beyond `top` name experts every row uses with weight 1, numbered from `experts` on).
static inline size_t pick_smem_bytes(int experts, int groups) {
    return (size_t)4 * (experts + (groups > 1 ? groups : 0)) * sizeof(float);
}

static inline bool pick_args_ok(int experts, int top, int groups, int keep, int out_stride) {
    if (pick_smem_bytes(experts, groups) > 48 * 1024) return false;
    if (top < 1 || top > experts || top > 32 || experts > 2048 || out_stride < top || out_stride > top + 32) return false;
    if (groups > 1 && (experts % groups != 0 || keep < 1 || keep > groups || keep * (experts / groups) < top)) return false;
    return true;
}

extern "C" int imparo_moe_route(const void* h, int dtype, const float* w_r, int n_rows, int width, int experts, int top,
                                int softmax_scores, int renormalise, int groups, int keep, float renorm_eps, float weight_scale,
                                int out_stride, float* logits, int* ids, float* wts, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!pick_args_ok(experts, top, groups, keep, out_stride) || logits == nullptr) return -2;
    int per = 4;
    if ((size_t)4 * width * sizeof(float) > 48 * 1024) per = 1;
    const size_t smem = (size_t)per * width * sizeof(float);
    if (smem > 48 * 1024) return -25;
    dim3 grid((n_rows + per - 1) / per, (experts + 7) / 8);
    if (dtype == IMPARO_DT_F32)
        launch(moe_logits_kernel<float>, grid, dim3(256), smem, stream, (const float*)h, w_r, n_rows, width, experts, per, logits);
    else if (dtype == IMPARO_DT_BF16)
        launch(moe_logits_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)h, w_r, n_rows, width, experts,
               per, logits);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    launch(moe_pick_kernel, dim3((n_rows + 3) / 4), dim3(128), pick_smem_bytes(experts, groups), stream, (const float*)logits, n_rows,
           experts, 1, top, softmax_scores, renormalise, groups, keep, renorm_eps, weight_scale, out_stride, ids, wts);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// The choice alone, from logits that a product has made: [n_rows, parts * experts] float32.  With bfloat16 rows h (exact in
// 32-bit) and the 32-bit router matrix cut into three bfloat16 pieces (w1 = W rounded, w2 = W - w1 rounded, w3 the rest
// rounded: 8 + 8 + 8 bits of mantissa, their sum is W to its last bit), the
// tensor-core product h [w1; w2; w3]^T has exact products and 32-bit sums: the router's logits in 32-bit, at the product's speed.
extern "C" int imparo_moe_pick(const float* logits, int n_rows, int experts, int parts, int top, int softmax_scores, int renormalise,
                               int groups, int keep, float renorm_eps, float weight_scale, int out_stride, int* ids, float* wts,
                               cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!pick_args_ok(experts, top, groups, keep, out_stride) || parts < 1 || parts > 4) return -2;
    launch(moe_pick_kernel, dim3((n_rows + 3) / 4), dim3(128), pick_smem_bytes(experts, groups), stream, logits, n_rows, experts,
           parts, top, softmax_scores, renormalise, groups, keep, renorm_eps, weight_scale, out_stride, ids, wts);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// mid: [n_rows * top, ff] in dtype; out float32 [n_rows, width].  Two launches.
extern "C" int imparo_moe_rows(const void* h, const void* w_gu, const void* w_down, int dtype, const int* ids, const float* wts,
                               int n_rows, int width, int ff, int top, int experts, int weight_input, int act, float limit,
                               void* mid, float* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if ((size_t)width * 4 > 48 * 1024 || (size_t)ff * 4 > 48 * 1024) return -25;
    dim3 g1(n_rows * top, (ff + 31) / 32), g2(n_rows, (width + 31) / 32);
    if (dtype == IMPARO_DT_F32) {
        launch(moe_rows_up_kernel<float>, g1, dim3(256), (size_t)width * 4, stream, (const float*)h, (const float*)w_gu, ids, wts, width,
               ff, top, experts, weight_input, act, limit, (float*)mid);
        IMPARO_CHECK_LAUNCH();
        launch(moe_rows_down_kernel<float>, g2, dim3(256), (size_t)ff * 4, stream, (const float*)mid, (const float*)w_down, ids, wts,
               width, ff, top, experts, weight_input, out);
    } else if (dtype == IMPARO_DT_BF16) {
        launch(moe_rows_up_kernel<__nv_bfloat16>, g1, dim3(256), (size_t)width * 4, stream, (const __nv_bfloat16*)h,
               (const __nv_bfloat16*)w_gu, ids, wts, width, ff, top, experts, weight_input, act, limit, (__nv_bfloat16*)mid);
        IMPARO_CHECK_LAUNCH();
        launch(moe_rows_down_kernel<__nv_bfloat16>, g2, dim3(256), (size_t)ff * 4, stream, (const __nv_bfloat16*)mid,
               (const __nv_bfloat16*)w_down, ids, wts, width, ff, top, experts, weight_input, out);
    } else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// scratch_i: int32 [n_pairs + experts + 1 + 1 + 3 * max_tiles], max_tiles = n_pairs / 32 + experts; pair_out float32
// [n_pairs, width]; mid [n_pairs, ff] in dtype; out float32 [n_rows, width].  Four launches.
extern "C" int imparo_moe_grouped(const void* h, const void* w_gu, const void* w_down, int dtype, const int* ids, const float* wts,
                                  int n_rows, int width, int ff, int top, int experts, int weight_input, int act, float limit,
                                  void* mid, float* pair_out, int* scratch_i, float* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int n_pairs = n_rows * top;
    const int max_tiles = n_pairs / GM + experts;
    if (experts > 4096) return -25;
    int* sorted = scratch_i;
    int* expert_start = scratch_i + n_pairs;
    int* plan = expert_start + experts + 1;
    launch(moe_group_plan_kernel, dim3(1), dim3(1024), (size_t)(experts + 1) * sizeof(int), stream, ids, n_pairs, experts, sorted,
           expert_start, plan, max_tiles);
    IMPARO_CHECK_LAUNCH();
    dim3 g1(max_tiles, (ff + GN - 1) / GN), g2(max_tiles, (width + GN - 1) / GN);
    if (dtype == IMPARO_DT_F32) {
        launch(moe_group_up_kernel<float>, g1, dim3(256), 0, stream, (const float*)h, (const float*)w_gu, (const int*)sorted,
               (const int*)plan, wts, width, ff, top, weight_input, act, limit, (float*)mid);
        IMPARO_CHECK_LAUNCH();
        launch(moe_group_down_kernel<float>, g2, dim3(256), 0, stream, (const float*)mid, (const float*)w_down, (const int*)sorted,
               (const int*)plan, wts, width, ff, weight_input, pair_out);
    } else if (dtype == IMPARO_DT_BF16) {
        launch(moe_group_up_kernel<__nv_bfloat16>, g1, dim3(256), 0, stream, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_gu,
               (const int*)sorted, (const int*)plan, wts, width, ff, top, weight_input, act, limit, (__nv_bfloat16*)mid);
        IMPARO_CHECK_LAUNCH();
        launch(moe_group_down_kernel<__nv_bfloat16>, g2, dim3(256), 0, stream, (const __nv_bfloat16*)mid, (const __nv_bfloat16*)w_down,
               (const int*)sorted, (const int*)plan, wts, width, ff, weight_input, pair_out);
    } else return -1;
    IMPARO_CHECK_LAUNCH();
    const size_t total = (size_t)n_rows * width;
    launch(moe_sum_pairs_kernel, dim3((unsigned)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256)), dim3(256), 0, stream,
           (const float*)pair_out, n_rows, width, top, out);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_gemm_prefill_grouped(const void* x, int ldx, const void* w, int n_groups, void* out, int ldo, int m_tiles,
                                           int N, int K, int epilogue, int act, float limit, const int* tile_group, int* status,
                                           cudaStream_t stream);

// bfloat16, width and ff multiples of 8, at most 256 experts: rows sorted into tiles of 128 per expert and both products on
// the tensor-memory kernel (SwiGLU in the first one's epilogue).  m_tiles = n_pairs / 128 + experts; xg bfloat16
// [m_tiles * 128, width]; mid_g bfloat16 [m_tiles * 128, ff]; out_g float32 [m_tiles * 128, width]; scratch_i int32
// [n_pairs + m_tiles]; out float32 [n_rows, width].  Five launches.  -25: not a case for this path.
extern "C" int imparo_moe_tiles(const void* h, const void* w_gu, const void* w_down, const int* ids, const float* wts, int n_rows,
                                int width, int ff, int top, int experts, int weight_input, int act, float limit, void* xg, void* mid_g,
                                float* out_g, int* scratch_i, float* out, int* status, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width % 8 != 0 || ff % 8 != 0 || experts > 256) return -25;
    const int n_pairs = n_rows * top;
    const int m_tiles = n_pairs / TILE_ROWS + experts;
    int* slot_of_pair = scratch_i;
    int* tile_group = scratch_i + n_pairs;
    launch(moe_tile_plan_kernel, dim3(1), dim3(1024), (size_t)34 * experts * sizeof(int), stream, ids, n_pairs, experts, slot_of_pair,
           tile_group, m_tiles);
    IMPARO_CHECK_LAUNCH();
    launch(moe_tile_gather_kernel, dim3(n_pairs), dim3(128), 0, stream, (const __nv_bfloat16*)h, (const int*)slot_of_pair, wts, width,
           top, weight_input, (__nv_bfloat16*)xg);
    IMPARO_CHECK_LAUNCH();
    int rc = imparo_gemm_prefill_grouped(xg, width, w_gu, experts, mid_g, ff, m_tiles, ff, width, 3, act, limit, tile_group, status, stream);
    if (rc) return rc;
    rc = imparo_gemm_prefill_grouped(mid_g, ff, w_down, experts, out_g, width, m_tiles, width, ff, 1, 0, 0.f, tile_group, status, stream);
    if (rc) return rc;
    launch(moe_tile_sum_kernel, dim3(n_rows), dim3(256), 0, stream, (const float*)out_g, (const int*)slot_of_pair, wts, width, top,
           weight_input, out);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

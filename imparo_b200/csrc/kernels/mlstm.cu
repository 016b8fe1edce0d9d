// A matrix memory with exponential gates (the mLSTM recurrence), over a fixed-size state per request and head:
//
//     a_t = cap * tanh((x_i + b_i) / cap)                         log input gate
//     f_t = log sigmoid(cap * tanh((x_f + b_f) / cap))            log forget gate
//     m_t = max(f_t + m_(t-1), a_t)                               running maximum, m_0 = 0
//     S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T        S: [dim, vdim], S_0 = 0
//     n_t = exp(f_t + m_(t-1) - m_t) n_(t-1) + exp(a_t - m_t) k_t              n: [dim],       n_0 = 0
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),     q_t already times q_scale
//
// for ragged batches: a request's rows are walked in order from what its slot holds (S, n, m in three state tensors,
// all zero for a fresh request), and the slot is written back at the end, so a prompt cut into portions, or decoded
// token by token, runs the same sequence of operations as the whole prompt.  q, k, v and the gates' pre-activations are
// columns of one 32-bit product; everything here is 32-bit.
//
//  (1) mlstm_recurrent: one warp per (request, head, 32 value columns), up to four warps of one head in a CTA.  A lane owns
//      one column of S in registers (dim values); n is spread over the lanes (entry d with lane d % 32) and m is kept by
//      every lane; the rows' k, q, v and gate inputs are copied asynchronously into shared memory a stage of 8 or 16 rows
//      ahead, k and q once for the CTA's warps.  Every warp of a head repeats n and m and keeps a copy of its own in the
//      slot (n is [heads, vblocks, dim], m [heads, vblocks], vblocks = ceil(vdim / 32)): no CTA reads what another one
//      writes.  Key sizes above 64: two lanes share a value column, each with half of the key dimension, so that a lane
//      keeps at most 128 state entries in registers; a warp then owns 16 columns and two warps of a CTA share a copy.
//  (2) long portions in chunks of `chunk` rows that run side by side, in three launches.  With b_t the sum of the log
//      forget gates from the chunk's first row to row t, the recurrence unrolls to
//          m_t = max(b_t + m_in, max_(s<=t) (b_t - b_s + a_s))
//          S_t = exp(b_t + m_in - m_t) S_in + sum_(s<=t) exp(b_t - b_s + a_s - m_t) k_s v_s^T        (n_t alike)
//      with (S_in, n_in, m_in) the state the chunk starts from, and every exponent is <= 0.  So
//        local: every chunk alone from the empty state (m_in = -inf: S = 0 carries no maximum): its (S, n, m) and total b
//        scan:  per request over its chunks in order: the state each chunk starts from, combined as
//               m' = max(b + m_in, m_loc), S' = exp(b + m_in - m') S_in + exp(m_loc - m') S_loc; the slot's S and n at the end
//        out:   every chunk alone from its starting state: the outputs of its rows (the row walk of (1))
//      The chunk walk is the same arithmetic as the row walk; results differ by the order of additions only.
#include "common.cuh"

namespace imparo {

__device__ __forceinline__ float ml_log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

struct MlstmCols {
    const float* proj;      // float32 rows
    size_t stride;
    int q_off, k_off, v_off, i_off, f_off;
    const float* i_bias;    // [heads]
    const float* f_bias;    // [heads]
    float cap, q_scale;
};

// A CTA is NW warps: warp w owns value columns [(blockIdx.z * NW + w) * 32, +32) of one (request or chunk, head).  The rows'
// k, q, v and gate inputs pass through shared memory in stages of ST rows that all threads copy asynchronously (cp.async, 4
// bytes each) one stage ahead of the one being walked; k and q are shared by the CTA's warps.
template <int DMAX> struct MlStage { static constexpr int ROWS = DMAX <= 64 ? 16 : 8; };

template <int DMAX, int NW>
struct MlSmem {
    static constexpr int ST = MlStage<DMAX>::ROWS;
    float k[2][ST][DMAX];
    float q[2][ST][DMAX];
    float v[2][ST][NW * 32];
    float x[2][ST][2];          // the gates' inputs as the product left them
    float g[ST][2];             // log input gate, log forget gate
};

__device__ __forceinline__ void ml_cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ml_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ml_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Rows [r_begin, r_end) of one request and head.  S: this lane's column of the state; nl: this lane's entries of n
// (d = lane, lane + 32, ...); m: the running maximum (-INFINITY: an empty state).  OUT: the rows' outputs are wanted (else
// only the state, and q is not read).  Every thread of the CTA calls this with the same rows; `live`: this lane has a column.
template <int DMAX, int NW, int SPLIT, bool OUT>
__device__ __forceinline__ void ml_walk(const MlstmCols& c, MlSmem<DMAX, NW>& sm, float (&S)[DMAX / SPLIT], float (&nl)[DMAX / 32], float& m,
                                        int r_begin, int r_end, float* __restrict__ out, int h, int heads, int dim, int vdim,
                                        int v0, int col, bool live, float* total_f) {
    constexpr int ST = MlSmem<DMAX, NW>::ST;
    constexpr int DL = DMAX / SPLIT;                   // state entries per lane
    constexpr int WCOLS = 32 / SPLIT;                  // value columns per warp
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = NW * 32;
    const int dofs = (lane / WCOLS) * DL;              // this lane's stretch of the key dimension
    const int vcols = min(NW * WCOLS, vdim - v0);
    // columns no copy writes: zero once
    for (int i = tid; i < 2 * ST * DMAX; i += nthreads) {
        const int d = i % DMAX;
        if (d >= dim || !OUT) (&sm.q[0][0][0])[i] = 0.f;
        if (d >= dim) (&sm.k[0][0][0])[i] = 0.f;
    }
    for (int i = tid; i < 2 * ST * NW * 32; i += nthreads)
        if (i % (NW * 32) >= vcols) (&sm.v[0][0][0])[i] = 0.f;
    const int per_row = dim + (OUT ? dim : 0) + vcols + 2;
    auto issue = [&](int base, int n, int buf) {
        for (int e = tid; e < n * per_row; e += nthreads) {
            const int r = e / per_row;
            int cidx = e - r * per_row;
            const float* row = c.proj + (size_t)(base + r) * c.stride;
            if (cidx < dim) { ml_cp_async4(&sm.k[buf][r][cidx], row + c.k_off + (size_t)h * dim + cidx); continue; }
            cidx -= dim;
            if (OUT) {
                if (cidx < dim) { ml_cp_async4(&sm.q[buf][r][cidx], row + c.q_off + (size_t)h * dim + cidx); continue; }
                cidx -= dim;
            }
            if (cidx < vcols) { ml_cp_async4(&sm.v[buf][r][cidx], row + c.v_off + (size_t)h * vdim + v0 + cidx); continue; }
            cidx -= vcols;
            ml_cp_async4(&sm.x[buf][r][cidx], row + (cidx == 0 ? c.i_off : c.f_off) + h);
        }
        ml_cp_commit();
    };
    float fsum = 0.f;
    const int total = r_end - r_begin;
    const int n_stages = (total + ST - 1) / ST;
    if (n_stages > 0) issue(r_begin, min(ST, total), 0);
    const float bi = c.i_bias[h], bf = c.f_bias[h];
    for (int s = 0; s < n_stages; ++s) {
        const int base = r_begin + s * ST, n = min(ST, r_end - base), buf = s & 1;
        if (s + 1 < n_stages) {
            issue(base + ST, min(ST, r_end - base - ST), buf ^ 1);
            ml_cp_wait<1>();
        } else {
            ml_cp_wait<0>();
        }
        __syncthreads();
        if (tid < n) {
            sm.g[tid][0] = c.cap * tanhf((sm.x[buf][tid][0] + bi) / c.cap);
            sm.g[tid][1] = ml_log_sigmoid(c.cap * tanhf((sm.x[buf][tid][1] + bf) / c.cap));
        }
        __syncthreads();
        for (int r = 0; r < n; ++r) {
            const float a = sm.g[r][0], f = sm.g[r][1];
            fsum += f;
            const float m_new = fmaxf(f + m, a);
            const float keep = expf(f + m - m_new);       // an empty state (m = -inf) keeps nothing: exp(-inf) = 0
            const float put = expf(a - m_new);
            m = m_new;
            const float pv = put * sm.v[buf][r][warp * WCOLS + (lane % WCOLS)];
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f, nq = 0.f;
#pragma unroll
            for (int d = 0; d < DL; d += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&sm.k[buf][r][dofs + d]);
                S[d] = keep * S[d] + k4.x * pv;
                S[d + 1] = keep * S[d + 1] + k4.y * pv;
                S[d + 2] = keep * S[d + 2] + k4.z * pv;
                S[d + 3] = keep * S[d + 3] + k4.w * pv;
                if (OUT) {
                    const float4 q4 = *reinterpret_cast<const float4*>(&sm.q[buf][r][dofs + d]);
                    o0 += S[d] * q4.x; o1 += S[d + 1] * q4.y; o2 += S[d + 2] * q4.z; o3 += S[d + 3] * q4.w;
                }
            }
#pragma unroll
            for (int j = 0; j < DMAX / 32; ++j) {
                nl[j] = keep * nl[j] + put * sm.k[buf][r][j * 32 + lane];
                if (OUT) nq += nl[j] * sm.q[buf][r][j * 32 + lane];
            }
            if (OUT) {
                nq = warp_sum(nq) * c.q_scale;
                const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
                float o = (o0 + o1) + (o2 + o3);
                if (SPLIT == 2) o += __shfl_xor_sync(0xffffffffu, o, 16);        // the other half of the key dimension
                if (live && lane < WCOLS) out[(size_t)(base + r) * ((size_t)heads * vdim) + (size_t)h * vdim + col] = o * c.q_scale / den;
            }
        }
        __syncthreads();          // the stage after the next one is copied into this buffer
    }
    if (total_f) *total_f = fsum;
}

// SPLIT = 2 (key sizes above 64): two lanes share a value column, each with half of the key dimension in registers; a warp
// then owns 16 value columns and a CTA 16 * NW.
template <int DMAX, int NW, int SPLIT>
__global__ void __launch_bounds__(NW * 32)
mlstm_recurrent_kernel(MlstmCols c, float* __restrict__ state_S, float* __restrict__ state_n, float* __restrict__ state_m,
                       const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_slots,
                       float* __restrict__ out, int heads, int dim, int vdim, int vblocks, int* status) {
    __shared__ __align__(16) MlSmem<DMAX, NW> sm;
    pdl_trigger();
    constexpr int DL = DMAX / SPLIT, WCOLS = 32 / SPLIT;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int item = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * NW * WCOLS, wcol = v0 + warp * WCOLS, col = wcol + (lane % WCOLS);
    const int vb = wcol / 32, dofs = (lane / WCOLS) * DL;
    const int r0 = item_row_start[item], r1 = item_row_start[item + 1];
    const int slot = item_slot[item];
    pdl_wait();
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) report(status, IMPARO_ST_SLOT_RANGE, 81, item, slot);
        return;
    }
    const bool live = col < vdim, mine = wcol < vdim;
    float* sp = state_S + (((size_t)slot * heads + h) * dim) * vdim + col;
    const size_t copy = ((size_t)slot * heads + h) * vblocks + (mine ? vb : 0);
    float* np = state_n + copy * dim;
    float* mp = state_m + copy;
    float S[DL], nl[DMAX / 32];
#pragma unroll
    for (int d = 0; d < DL; ++d) S[d] = (live && dofs + d < dim) ? sp[(size_t)(dofs + d) * vdim] : 0.f;
#pragma unroll
    for (int j = 0; j < DMAX / 32; ++j) nl[j] = (j * 32 + lane < dim) ? np[j * 32 + lane] : 0.f;
    float m = *mp;
    ml_walk<DMAX, NW, SPLIT, true>(c, sm, S, nl, m, r0, r1, out, h, heads, dim, vdim, v0, col, live, nullptr);
    if (live) {
#pragma unroll
        for (int d = 0; d < DL; ++d) if (dofs + d < dim) sp[(size_t)(dofs + d) * vdim] = S[d];
    }
    __syncthreads();          // warps that share a copy of n and m have all read it
    if (mine) {
#pragma unroll
        for (int j = 0; j < DMAX / 32; ++j) if (j * 32 + lane < dim) np[j * 32 + lane] = nl[j];
        if (lane == 0) *mp = m;
    }
}

// ---- long portions in chunks ---------------------------------------------------------------------------------------
// The chunks of all requests of the launch are numbered in order (chunk c of a request: rows r0 + c * chunk ...).  The
// grid's x extent is an upper bound of their number (rows / chunk + requests); blocks beyond it return.
__device__ __forceinline__ bool ml_find_chunk(const int* __restrict__ item_row_start, int n_items, int chunk, int g,
                                              int& item, int& r_begin, int& r_end, int& first_of_item) {
    int basec = 0;
    for (int i = 0; i < n_items; ++i) {
        const int r0 = item_row_start[i], r1 = item_row_start[i + 1];
        const int nc = (r1 - r0 + chunk - 1) / chunk;
        if (g < basec + nc) {
            item = i;
            r_begin = r0 + (g - basec) * chunk;
            r_end = min(r_begin + chunk, r1);
            first_of_item = basec;
            return true;
        }
        basec += nc;
    }
    return false;
}

// chunk_S [chunks, heads, dim, vdim], chunk_n [chunks, heads, vblocks, dim], chunk_mb [chunks, heads, vblocks, 3] = (the
// chunk's own maximum, its total b, the maximum it starts from).  The out pass of a request's last chunk leaves the slot's
// maximum.
template <int DMAX, int NW, int SPLIT, bool OUT>
__global__ void __launch_bounds__(NW * 32)
mlstm_chunk_kernel(MlstmCols c, float* __restrict__ chunk_S, float* __restrict__ chunk_n, float* __restrict__ chunk_mb,
                   const int* __restrict__ item_row_start, int n_items, int chunk, float* __restrict__ out, int heads, int dim,
                   int vdim, int vblocks, const int* __restrict__ item_slot, int n_slots, float* __restrict__ state_m) {
    __shared__ __align__(16) MlSmem<DMAX, NW> sm;
    pdl_trigger();
    constexpr int DL = DMAX / SPLIT, WCOLS = 32 / SPLIT;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * NW * WCOLS, wcol = v0 + warp * WCOLS, col = wcol + (lane % WCOLS);
    const int vb = wcol / 32, dofs = (lane / WCOLS) * DL;
    int item, r_begin, r_end, first;
    const bool found = ml_find_chunk(item_row_start, n_items, chunk, g, item, r_begin, r_end, first);
    pdl_wait();
    if (!found) return;
    const bool live = col < vdim, mine = wcol < vdim;
    float* sp = chunk_S + (((size_t)g * heads + h) * dim) * vdim + col;
    const size_t copy = ((size_t)g * heads + h) * vblocks + (mine ? vb : 0);
    float* np = chunk_n + copy * dim;
    float* mb = chunk_mb + copy * 3;
    float S[DL], nl[DMAX / 32];
    float m, total;
    if (OUT) {                  // from the state the scan left for this chunk
#pragma unroll
        for (int d = 0; d < DL; ++d) S[d] = (live && dofs + d < dim) ? sp[(size_t)(dofs + d) * vdim] : 0.f;
#pragma unroll
        for (int j = 0; j < DMAX / 32; ++j) nl[j] = (j * 32 + lane < dim) ? np[j * 32 + lane] : 0.f;
        m = mb[2];
        ml_walk<DMAX, NW, SPLIT, true>(c, sm, S, nl, m, r_begin, r_end, out, h, heads, dim, vdim, v0, col, live, nullptr);
        if (mine && lane == 0 && r_end == item_row_start[item + 1]) {
            const int slot = item_slot[item];
            if (slot >= 0 && slot < n_slots) state_m[((size_t)slot * heads + h) * vblocks + vb] = m;
        }
        return;
    }
#pragma unroll
    for (int d = 0; d < DL; ++d) S[d] = 0.f;
#pragma unroll
    for (int j = 0; j < DMAX / 32; ++j) nl[j] = 0.f;
    m = -INFINITY;
    ml_walk<DMAX, NW, SPLIT, false>(c, sm, S, nl, m, r_begin, r_end, nullptr, h, heads, dim, vdim, v0, col, live, &total);
    if (live) {
#pragma unroll
        for (int d = 0; d < DL; ++d) if (dofs + d < dim) sp[(size_t)(dofs + d) * vdim] = S[d];
    }
    if (mine) {
#pragma unroll
        for (int j = 0; j < DMAX / 32; ++j) if (j * 32 + lane < dim) np[j * 32 + lane] = nl[j];
        if (lane == 0) { mb[0] = m; mb[1] = total; mb[2] = 0.f; }
    }
}

// grid (requests, heads, ceil((dim * vdim + vblocks * dim) / 256)): a thread per entry of S (and of every copy of n), walking
// the request's chunks.  The slot's maximum is only read here (every copy holds the same number).
__global__ void __launch_bounds__(256)
mlstm_chunk_scan_kernel(float* __restrict__ chunk_S, float* __restrict__ chunk_n, float* __restrict__ chunk_mb,
                        float* __restrict__ state_S, float* __restrict__ state_n, const float* __restrict__ state_m,
                        const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_slots, int chunk,
                        int heads, int dim, int vdim, int vblocks, int* status) {
    pdl_trigger();
    const int item = blockIdx.x, h = blockIdx.y;
    int first = 0;
    for (int i = 0; i < item; ++i) first += (item_row_start[i + 1] - item_row_start[i] + chunk - 1) / chunk;
    const int nc = (item_row_start[item + 1] - item_row_start[item] + chunk - 1) / chunk;
    const int slot = item_slot[item];
    pdl_wait();
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0 && blockIdx.z == 0) report(status, IMPARO_ST_SLOT_RANGE, 82, item, slot);
        return;
    }
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int n_S = dim * vdim;
    if (e >= n_S + vblocks * dim) return;
    const bool is_n = e >= n_S;
    const size_t sh = (size_t)slot * heads + h;
    float* sv = is_n ? state_n + sh * vblocks * dim + (e - n_S) : state_S + sh * n_S + e;
    float val = *sv, m = state_m[sh * vblocks];
    const size_t per_chunk = is_n ? (size_t)heads * vblocks * dim : (size_t)heads * n_S;
    float* lv0 = is_n ? chunk_n + ((size_t)first * heads + h) * vblocks * dim + (e - n_S) : chunk_S + ((size_t)first * heads + h) * n_S + e;
    for (int c0 = 0; c0 < nc; c0 += 4) {
        // four chunks' loads at once (they depend on nothing), then the four dependent steps
        float local[4], m_loc[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (c0 + u < nc) {
                const size_t g = (size_t)(first + c0 + u) * heads + h;
                local[u] = lv0[(size_t)(c0 + u) * per_chunk];
                m_loc[u] = chunk_mb[g * vblocks * 3];
                b[u] = chunk_mb[g * vblocks * 3 + 1];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (c0 + u < nc) {
                const size_t g = (size_t)(first + c0 + u) * heads + h;
                lv0[(size_t)(c0 + u) * per_chunk] = val;                          // the state this chunk starts from
                if (e < vblocks) chunk_mb[(g * vblocks + e) * 3 + 2] = m;         // and its maximum (an entry no thread reads here)
                const float m_new = fmaxf(b[u] + m, m_loc[u]);
                val = expf(b[u] + m - m_new) * val + expf(m_loc[u] - m_new) * local[u];
                m = m_new;
            }
        }
    }
    *sv = val;
}

}  // namespace imparo

using namespace imparo;

template <int DMAX, int NW, int SPLIT>
static int mlstm_launch_nw(const MlstmCols& c, float* S, float* n, float* m, const int* item_row_start, const int* item_slot, int n_slots,
                           int n_items, int n_tok, float* out, int heads, int dim, int vdim, int chunk, float* chunk_S, float* chunk_n,
                           float* chunk_mb, int* status, cudaStream_t stream) {
    const int vblocks = (vdim + 31) / 32;
    const int zb = (vdim + NW * (32 / SPLIT) - 1) / (NW * (32 / SPLIT));
    if (chunk <= 0) {
        launch(mlstm_recurrent_kernel<DMAX, NW, SPLIT>, dim3(n_items, heads, zb), dim3(NW * 32), 0, stream, c, S, n, m, item_row_start, item_slot,
               n_slots, out, heads, dim, vdim, vblocks, status);
        IMPARO_CHECK_LAUNCH();
        return 0;
    }
    const int most = n_tok / chunk + n_items;
    launch(mlstm_chunk_kernel<DMAX, NW, SPLIT, false>, dim3(most, heads, zb), dim3(NW * 32), 0, stream, c, chunk_S, chunk_n, chunk_mb,
           item_row_start, n_items, chunk, (float*)nullptr, heads, dim, vdim, vblocks, item_slot, n_slots, m);
    IMPARO_CHECK_LAUNCH();
    const int entries = dim * vdim + vblocks * dim;
    launch(mlstm_chunk_scan_kernel, dim3(n_items, heads, (entries + 255) / 256), dim3(256), 0, stream, chunk_S, chunk_n, chunk_mb, S, n,
           (const float*)m, item_row_start, item_slot, n_slots, chunk, heads, dim, vdim, vblocks, status);
    IMPARO_CHECK_LAUNCH();
    launch(mlstm_chunk_kernel<DMAX, NW, SPLIT, true>, dim3(most, heads, zb), dim3(NW * 32), 0, stream, c, chunk_S, chunk_n, chunk_mb,
           item_row_start, n_items, chunk, out, heads, dim, vdim, vblocks, item_slot, n_slots, m);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// the warps of a CTA share the staged keys and queries: as many as the head's value columns fill, up to four; key sizes above 64
// are split over two lanes per column
template <int DMAX>
static int mlstm_launch(const MlstmCols& c, float* S, float* n, float* m, const int* item_row_start, const int* item_slot, int n_slots,
                        int n_items, int n_tok, float* out, int heads, int dim, int vdim, int chunk, float* chunk_S, float* chunk_n,
                        float* chunk_mb, int* status, cudaStream_t stream) {
    constexpr int SPLIT = DMAX > 64 ? 2 : 1;
    const int wblocks = (vdim + 32 / SPLIT - 1) / (32 / SPLIT);          // warps a head's value columns fill
    if (wblocks >= 3)
        return mlstm_launch_nw<DMAX, 4, SPLIT>(c, S, n, m, item_row_start, item_slot, n_slots, n_items, n_tok, out, heads, dim, vdim, chunk,
                                               chunk_S, chunk_n, chunk_mb, status, stream);
    if (wblocks == 2)
        return mlstm_launch_nw<DMAX, 2, SPLIT>(c, S, n, m, item_row_start, item_slot, n_slots, n_items, n_tok, out, heads, dim, vdim, chunk,
                                               chunk_S, chunk_n, chunk_mb, status, stream);
    return mlstm_launch_nw<DMAX, 1, SPLIT>(c, S, n, m, item_row_start, item_slot, n_slots, n_items, n_tok, out, heads, dim, vdim, chunk,
                                           chunk_S, chunk_n, chunk_mb, status, stream);
}

// proj: float32 rows of `stride` floats with q and k (heads * dim each), v (heads * vdim) and the two gates' pre-activations
// (heads each) at the given column offsets; i_bias, f_bias float32 [heads]; with vblocks = ceil(vdim / 32): state_S float32
// [n_slots, heads, dim, vdim], state_n [n_slots, heads, vblocks, dim], state_m [n_slots, heads, vblocks]; out float32
// [n_tok, heads * vdim].  chunk > 0: the chunked form, with chunk_S float32 [(n_tok / chunk + n_items), heads, dim, vdim],
// chunk_n [.., heads, vblocks, dim], chunk_mb [.., heads, vblocks, 3].  n_items <= 65535, heads <= 65535.
extern "C" int imparo_mlstm_scan(const float* proj, long long stride, int q_off, int k_off, int v_off, int i_off, int f_off,
                                 const float* i_bias, const float* f_bias, float cap, float q_scale, float* state_S, float* state_n,
                                 float* state_m, const int* item_row_start, const int* item_slot, int n_slots, int n_items,
                                 int n_tok, float* out, int heads, int dim, int vdim, int chunk, float* chunk_S, float* chunk_n,
                                 float* chunk_mb, int* status, cudaStream_t stream) {
    if (n_items <= 0 || n_tok <= 0) return 0;
    if (heads < 1 || dim < 1 || dim > 256 || vdim < 1 || n_items > 65535 || heads > 65535 || !(cap > 0.f)) return -2;
    if (chunk > 0 && (chunk_S == nullptr || chunk_n == nullptr || chunk_mb == nullptr)) return -2;
    MlstmCols c;
    c.proj = proj; c.stride = (size_t)stride;
    c.q_off = q_off; c.k_off = k_off; c.v_off = v_off; c.i_off = i_off; c.f_off = f_off;
    c.i_bias = i_bias; c.f_bias = f_bias; c.cap = cap; c.q_scale = q_scale;
    if (dim <= 32)
        return mlstm_launch<32>(c, state_S, state_n, state_m, item_row_start, item_slot, n_slots, n_items, n_tok, out, heads, dim, vdim,
                                chunk, chunk_S, chunk_n, chunk_mb, status, stream);
    if (dim <= 64)
        return mlstm_launch<64>(c, state_S, state_n, state_m, item_row_start, item_slot, n_slots, n_items, n_tok, out, heads, dim, vdim,
                                chunk, chunk_S, chunk_n, chunk_mb, status, stream);
    if (dim <= 128)
        return mlstm_launch<128>(c, state_S, state_n, state_m, item_row_start, item_slot, n_slots, n_items, n_tok, out, heads, dim, vdim,
                                 chunk, chunk_S, chunk_n, chunk_mb, status, stream);
    return mlstm_launch<256>(c, state_S, state_n, state_m, item_row_start, item_slot, n_slots, n_items, n_tok, out, heads, dim, vdim,
                             chunk, chunk_S, chunk_n, chunk_mb, status, stream);
}

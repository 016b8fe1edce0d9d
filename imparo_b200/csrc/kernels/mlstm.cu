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
//  (1) mlstm_recurrent: one warp per (request, head, 32 value columns).  A lane owns one column of S in registers (dim
//      values); n is spread over the lanes (entry d with lane d % 32) and m is kept by every lane; the rows are staged 16
//      at a time in shared memory.  Every warp of a head repeats n and m and keeps a copy of its own in the slot (n is
//      [heads, vblocks, dim], m [heads, vblocks], vblocks = ceil(vdim / 32)): no warp reads what another one writes.
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

constexpr int ML_STAGE = 16;

__device__ __forceinline__ float ml_log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

struct MlstmCols {
    const float* proj;      // float32 rows
    size_t stride;
    int q_off, k_off, v_off, i_off, f_off;
    const float* i_bias;    // [heads]
    const float* f_bias;    // [heads]
    float cap, q_scale;
};

// Rows [r_begin, r_end) of one request and head, for the 32 value columns of this warp.  S: this lane's column of the
// state; nl: this lane's entries of n (d = lane, lane + 32, ...); m: the running maximum (-INFINITY: an empty state).
// out: null when only the state is wanted.
template <int DMAX>
__device__ __forceinline__ void ml_walk(const MlstmCols& c, float (&S)[DMAX], float (&nl)[DMAX / 32], float& m, int r_begin, int r_end,
                                        float* __restrict__ out, int h, int heads, int dim, int vdim, int col, bool live,
                                        float (*qs)[DMAX], float (*ks)[DMAX], float (*vs)[32], float (*gs)[2], float* total_f) {
    const int lane = threadIdx.x;
    float fsum = 0.f;
    for (int base = r_begin; base < r_end; base += ML_STAGE) {
        const int n = min(ML_STAGE, r_end - base);
        __syncwarp();
        for (int r = 0; r < n; ++r) {
            const float* row = c.proj + (size_t)(base + r) * c.stride;
            const float* qr = row + c.q_off + (size_t)h * dim;
            const float* kr = row + c.k_off + (size_t)h * dim;
            for (int d = lane; d < DMAX; d += 32) {
                qs[r][d] = (d < dim && out) ? qr[d] * c.q_scale : 0.f;
                ks[r][d] = d < dim ? kr[d] : 0.f;
            }
            vs[r][lane] = live ? row[c.v_off + (size_t)h * vdim + col] : 0.f;
        }
        if (lane < n) {
            const float* row = c.proj + (size_t)(base + lane) * c.stride;
            const float xi = row[c.i_off + h] + c.i_bias[h], xf = row[c.f_off + h] + c.f_bias[h];
            gs[lane][0] = c.cap * tanhf(xi / c.cap);
            gs[lane][1] = ml_log_sigmoid(c.cap * tanhf(xf / c.cap));
        }
        __syncwarp();
        for (int r = 0; r < n; ++r) {
            const float a = gs[r][0], f = gs[r][1];
            fsum += f;
            const float m_new = fmaxf(f + m, a);
            const float keep = expf(f + m - m_new);       // an empty state (m = -inf) keeps nothing: exp(-inf) = 0
            const float put = expf(a - m_new);
            m = m_new;
            const float pv = put * vs[r][lane];
            float o = 0.f, nq = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; d += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&ks[r][d]);
                const float4 q4 = *reinterpret_cast<const float4*>(&qs[r][d]);
                S[d] = keep * S[d] + k4.x * pv;         o += S[d] * q4.x;
                S[d + 1] = keep * S[d + 1] + k4.y * pv; o += S[d + 1] * q4.y;
                S[d + 2] = keep * S[d + 2] + k4.z * pv; o += S[d + 2] * q4.z;
                S[d + 3] = keep * S[d + 3] + k4.w * pv; o += S[d + 3] * q4.w;
            }
#pragma unroll
            for (int j = 0; j < DMAX / 32; ++j) {
                nl[j] = keep * nl[j] + put * ks[r][j * 32 + lane];
                nq += nl[j] * qs[r][j * 32 + lane];
            }
            if (out) {
                nq = warp_sum(nq);
                const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
                if (live) out[(size_t)(base + r) * ((size_t)heads * vdim) + (size_t)h * vdim + col] = o / den;
            }
        }
    }
    if (total_f) *total_f = fsum;
}

template <int DMAX>
__global__ void __launch_bounds__(32)
mlstm_recurrent_kernel(MlstmCols c, float* __restrict__ state_S, float* __restrict__ state_n, float* __restrict__ state_m,
                       const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_slots,
                       float* __restrict__ out, int heads, int dim, int vdim, int* status) {
    __shared__ __align__(16) float qs[ML_STAGE][DMAX], ks[ML_STAGE][DMAX], vs[ML_STAGE][32], gs[ML_STAGE][2];
    pdl_trigger();
    const int item = blockIdx.x, h = blockIdx.y, col = blockIdx.z * 32 + threadIdx.x;
    const int lane = threadIdx.x;
    const int r0 = item_row_start[item], r1 = item_row_start[item + 1];
    const int slot = item_slot[item];
    pdl_wait();
    if (slot < 0 || slot >= n_slots) {
        if (lane == 0) report(status, IMPARO_ST_SLOT_RANGE, 81, item, slot);
        return;
    }
    const bool live = col < vdim;
    float* sp = state_S + (((size_t)slot * heads + h) * dim) * vdim + col;
    const size_t copy = ((size_t)slot * heads + h) * gridDim.z + blockIdx.z;
    float* np = state_n + copy * dim;
    float* mp = state_m + copy;
    float S[DMAX], nl[DMAX / 32];
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = (live && d < dim) ? sp[(size_t)d * vdim] : 0.f;
#pragma unroll
    for (int j = 0; j < DMAX / 32; ++j) nl[j] = (j * 32 + lane < dim) ? np[j * 32 + lane] : 0.f;
    float m = *mp;
    ml_walk<DMAX>(c, S, nl, m, r0, r1, out, h, heads, dim, vdim, col, live, qs, ks, vs, gs, nullptr);
    if (live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d) if (d < dim) sp[(size_t)d * vdim] = S[d];
    }
#pragma unroll
    for (int j = 0; j < DMAX / 32; ++j) if (j * 32 + lane < dim) np[j * 32 + lane] = nl[j];
    if (lane == 0) *mp = m;
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
template <int DMAX, bool OUT>
__global__ void __launch_bounds__(32)
mlstm_chunk_kernel(MlstmCols c, float* __restrict__ chunk_S, float* __restrict__ chunk_n, float* __restrict__ chunk_mb,
                   const int* __restrict__ item_row_start, int n_items, int chunk, float* __restrict__ out, int heads, int dim,
                   int vdim, const int* __restrict__ item_slot, int n_slots, float* __restrict__ state_m) {
    __shared__ __align__(16) float qs[ML_STAGE][DMAX], ks[ML_STAGE][DMAX], vs[ML_STAGE][32], gs[ML_STAGE][2];
    pdl_trigger();
    const int g = blockIdx.x, h = blockIdx.y, col = blockIdx.z * 32 + threadIdx.x;
    const int lane = threadIdx.x;
    int item, r_begin, r_end, first;
    const bool found = ml_find_chunk(item_row_start, n_items, chunk, g, item, r_begin, r_end, first);
    pdl_wait();
    if (!found) return;
    const bool live = col < vdim;
    float* sp = chunk_S + (((size_t)g * heads + h) * dim) * vdim + col;
    const size_t copy = ((size_t)g * heads + h) * gridDim.z + blockIdx.z;
    float* np = chunk_n + copy * dim;
    float* mb = chunk_mb + copy * 3;
    float S[DMAX], nl[DMAX / 32];
    float m, total;
    if (OUT) {                  // from the state the scan left for this chunk
#pragma unroll
        for (int d = 0; d < DMAX; ++d) S[d] = (live && d < dim) ? sp[(size_t)d * vdim] : 0.f;
#pragma unroll
        for (int j = 0; j < DMAX / 32; ++j) nl[j] = (j * 32 + lane < dim) ? np[j * 32 + lane] : 0.f;
        m = mb[2];
        ml_walk<DMAX>(c, S, nl, m, r_begin, r_end, out, h, heads, dim, vdim, col, live, qs, ks, vs, gs, nullptr);
        if (lane == 0 && r_end == item_row_start[item + 1]) {
            const int slot = item_slot[item];
            if (slot >= 0 && slot < n_slots) state_m[((size_t)slot * heads + h) * gridDim.z + blockIdx.z] = m;
        }
        return;
    }
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = 0.f;
#pragma unroll
    for (int j = 0; j < DMAX / 32; ++j) nl[j] = 0.f;
    m = -INFINITY;
    ml_walk<DMAX>(c, S, nl, m, r_begin, r_end, nullptr, h, heads, dim, vdim, col, live, qs, ks, vs, gs, &total);
    if (live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d) if (d < dim) sp[(size_t)d * vdim] = S[d];
    }
#pragma unroll
    for (int j = 0; j < DMAX / 32; ++j) if (j * 32 + lane < dim) np[j * 32 + lane] = nl[j];
    if (lane == 0) { mb[0] = m; mb[1] = total; mb[2] = 0.f; }
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
    for (int cidx = 0; cidx < nc; ++cidx) {
        const size_t g = (size_t)(first + cidx) * heads + h;
        float* lv = is_n ? chunk_n + g * vblocks * dim + (e - n_S) : chunk_S + g * n_S + e;
        const float m_loc = chunk_mb[g * vblocks * 3], b = chunk_mb[g * vblocks * 3 + 1];
        const float local = *lv;
        *lv = val;                                             // the state this chunk starts from
        if (e < vblocks) chunk_mb[(g * vblocks + e) * 3 + 2] = m;      // and its maximum (an entry no thread reads here)
        const float m_new = fmaxf(b + m, m_loc);
        val = expf(b + m - m_new) * val + expf(m_loc - m_new) * local;
        m = m_new;
    }
    *sv = val;
}

}  // namespace imparo

using namespace imparo;

template <int DMAX>
static int mlstm_launch(const MlstmCols& c, float* S, float* n, float* m, const int* item_row_start, const int* item_slot, int n_slots,
                        int n_items, int n_tok, float* out, int heads, int dim, int vdim, int chunk, float* chunk_S, float* chunk_n,
                        float* chunk_mb, int* status, cudaStream_t stream) {
    const int vblocks = (vdim + 31) / 32;
    if (chunk <= 0) {
        launch(mlstm_recurrent_kernel<DMAX>, dim3(n_items, heads, vblocks), dim3(32), 0, stream, c, S, n, m, item_row_start, item_slot,
               n_slots, out, heads, dim, vdim, status);
        IMPARO_CHECK_LAUNCH();
        return 0;
    }
    const int most = n_tok / chunk + n_items;
    launch(mlstm_chunk_kernel<DMAX, false>, dim3(most, heads, vblocks), dim3(32), 0, stream, c, chunk_S, chunk_n, chunk_mb,
           item_row_start, n_items, chunk, (float*)nullptr, heads, dim, vdim, item_slot, n_slots, m);
    IMPARO_CHECK_LAUNCH();
    const int entries = dim * vdim + vblocks * dim;
    launch(mlstm_chunk_scan_kernel, dim3(n_items, heads, (entries + 255) / 256), dim3(256), 0, stream, chunk_S, chunk_n, chunk_mb, S, n,
           (const float*)m, item_row_start, item_slot, n_slots, chunk, heads, dim, vdim, vblocks, status);
    IMPARO_CHECK_LAUNCH();
    launch(mlstm_chunk_kernel<DMAX, true>, dim3(most, heads, vblocks), dim3(32), 0, stream, c, chunk_S, chunk_n, chunk_mb,
           item_row_start, n_items, chunk, out, heads, dim, vdim, item_slot, n_slots, m);
    IMPARO_CHECK_LAUNCH();
    return 0;
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

// A short causal convolution over time on every channel of a stretch of a 32-bit product, for ragged batches, with the
// last taps-1 inputs of each request kept in its state slot:
//
//   y[t, c] = act( sum_j w[c, j] * u[t - taps + 1 + j, c] ),   u = product column (+ bias[c]),  zeros before the sequence
//
//  (1) channel_conv: a thread per (row, channel); inputs before the portion's first row come from the slot (oldest first),
//      which is all zeros for a fresh request.  act 0: none, 1: silu.
//  (2) channel_conv_state: moves the slot on by the portion's rows; it runs after every reader of the old state.
// The bias belongs to the product (a projection with a bias): the slot keeps biased values, and positions before the
// sequence count as zero, not as the bias.
#include "common.cuh"

namespace imparo {

constexpr int CC_MAX_TAPS = 17;

__global__ void __launch_bounds__(256)
channel_conv_kernel(const float* __restrict__ in, size_t stride, int col0, int channels, int taps,
                    const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state,
                    const int* __restrict__ item_row_start, const int* __restrict__ item_of_token,
                    const int* __restrict__ item_slot, int n_slots, int act, float* __restrict__ out, size_t out_stride,
                    int* status) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int item = item_of_token[t];
    const int first = item_row_start[item];
    const int slot = item_slot[item];
    float wt[CC_MAX_TAPS];
    if (c < channels)
        for (int k = 0; k < taps; ++k) wt[k] = w[(size_t)c * taps + k];
    const float bv = (bias && c < channels) ? bias[c] : 0.f;
    pdl_wait();
    if (c >= channels) return;
    if (slot < 0 || slot >= n_slots) {
        if (c == 0) report(status, IMPARO_ST_SLOT_RANGE, 72, t, slot);
        return;
    }
    const float* st = state + (size_t)slot * (taps - 1) * channels;
    const int j = t - first;                                      // row within the portion
    float acc = 0.f;
    for (int k = 0; k < taps; ++k) {
        const int src = j - (taps - 1 - k);
        const float u = src >= 0 ? in[(size_t)(first + src) * stride + col0 + c] + bv
                                 : st[(size_t)(taps - 1 + src) * channels + c];
        acc += wt[k] * u;
    }
    out[(size_t)t * out_stride + c] = act == 1 ? silu(acc) : acc;
}

__global__ void __launch_bounds__(256)
channel_conv_state_kernel(const float* __restrict__ in, size_t stride, int col0, int channels, int taps,
                          const float* __restrict__ bias, float* __restrict__ state,
                          const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_slots) {
    pdl_trigger();
    const int item = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int first = item_row_start[item], n = item_row_start[item + 1] - first;
    const int slot = item_slot[item];
    pdl_wait();
    if (c >= channels || slot < 0 || slot >= n_slots) return;
    float* st = state + (size_t)slot * (taps - 1) * channels;
    const int keep = taps - 1;
    const float bv = bias ? bias[c] : 0.f;
    // entry i of the new state is input number (n - keep + i) of the portion; negative numbers are old entries
    float moved[CC_MAX_TAPS];
    for (int i = 0; i < keep; ++i) {
        const int src = n - keep + i;
        moved[i] = src >= 0 ? in[(size_t)(first + src) * stride + col0 + c] + bv : st[(size_t)(keep + src) * channels + c];
    }
    for (int i = 0; i < keep; ++i) st[(size_t)i * channels + c] = moved[i];
}

}  // namespace imparo

using namespace imparo;

// in: float32 rows of `stride` floats, the convolved stretch at columns col0 .. col0 + channels; w: float32 [channels, taps];
// bias: float32 [channels] or null; state: float32 [n_slots, taps - 1, channels]; out: float32 rows of out_stride floats.
extern "C" int imparo_channel_conv(const float* in, long long stride, int col0, int channels, int taps, const float* w,
                                   const float* bias, const float* state, const int* item_row_start, const int* item_of_token,
                                   const int* item_slot, int n_slots, int act, float* out, long long out_stride, int n_tok,
                                   int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (taps < 1 || taps > CC_MAX_TAPS) return -2;
    if (channels < 1 || stride < col0 + channels || out_stride < channels) return -3;
    launch(channel_conv_kernel, dim3(n_tok, (channels + 255) / 256), dim3(256), 0, stream, in, (size_t)stride, col0, channels, taps,
           w, bias, state, item_row_start, item_of_token, item_slot, n_slots, act, out, (size_t)out_stride, status);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_channel_conv_state(const float* in, long long stride, int col0, int channels, int taps, const float* bias,
                                         float* state, const int* item_row_start, const int* item_slot, int n_slots, int n_items,
                                         cudaStream_t stream) {
    if (n_items <= 0 || taps <= 1) return 0;
    if (taps > CC_MAX_TAPS) return -2;
    launch(channel_conv_state_kernel, dim3(n_items, (channels + 255) / 256), dim3(256), 0, stream, in, (size_t)stride, col0, channels,
           taps, bias, state, item_row_start, item_slot, n_slots);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// A short causal convolution over time on every channel of a row buffer, with the rolling inputs of every
// request kept between steps:
//
//     y[t][c] = sum_j taps[c][j] * u[t - n + 1 + j][c],   j = 0 .. n - 1,
//
// where u before the start of a sequence is zero.  A step brings segments (runs of consecutive tokens of
// one request); the n - 1 inputs in front of a segment come from the request's state slot, which holds
// the last n - 1 inputs of the sequence so far (oldest first, zero when the request starts).
//
//   fwb_causal_conv:  out <- conv(in) for the columns [col0, col0 + C) of every row (other columns are
//                     not touched; `in` and `out` are different buffers of one shape), then the state of
//                     every segment's slot moves on to the segment's last n - 1 inputs.
// Two launches: the convolution reads the old state, the second kernel writes the new one.  All
// arithmetic is fp32, taps applied in the order j = 0 .. n - 1 whatever the step's cut.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* __restrict__ in, T* __restrict__ out, long long ld, int col0, int C,
                   const float* __restrict__ taps, int n, const float* __restrict__ state, long long slot_stride,
                   const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
                   const int* __restrict__ seg_slot) {
    fwb::pdl_entry();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seg = tok_seg[t];
    const int local = t - seg_start[seg];                 // tokens of this segment in front of t
    const float* slot = state + (size_t)seg_slot[seg] * slot_stride;
    float acc = 0.0f;
    for (int j = 0; j < n; ++j) {
        const int back = n - 1 - j;                        // how far behind t this tap reads
        float u;
        if (back <= local) u = to_f32<T>(in[(size_t)(t - back) * ld + col0 + c]);
        else u = slot[(size_t)(n - 1 + local - back) * C + c];   // state row n-1-(back-local)
        acc = fmaf(taps[(size_t)c * n + j], u, acc);
    }
    out[(size_t)t * ld + col0 + c] = from_f32<T>(acc);
}

// One thread per (segment, channel): the new state rows are the segment's last n - 1 inputs, or, for a
// segment shorter than that, the old rows moved up with the segment's inputs behind them.
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_advance_kernel(const T* __restrict__ in, long long ld, int col0, int C, int n,
                           float* __restrict__ state, long long slot_stride, const int* __restrict__ seg_start,
                           const int* __restrict__ seg_slot) {
    fwb::pdl_entry();
    const int seg = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = seg_start[seg], len = seg_start[seg + 1] - first;
    float* slot = state + (size_t)seg_slot[seg] * slot_stride;
    const int keep = n - 1;
    float rows[MAX_TAPS];
    for (int k = 0; k < keep; ++k) {
        const int at = len - keep + k;                     // index inside the segment (negative: older)
        rows[k] = at >= 0 ? to_f32<T>(in[(size_t)(first + at) * ld + col0 + c]) : slot[(size_t)(keep + at) * C + c];
    }
    for (int k = 0; k < keep; ++k) slot[(size_t)k * C + c] = rows[k];
}

template <typename T>
int launch(const void* in, void* out, long long ld, int col0, int C, const float* taps, int n, float* state,
           long long slot_stride, const int* tok_seg, const int* seg_start, const int* seg_slot, int T_tokens,
           int S, cudaStream_t stream) {
    const dim3 grid(T_tokens, (C + 255) / 256);
    fwb::pdl(causal_conv_kernel<T>, grid, 256, 0, stream)((const T*)in, (T*)out, ld, col0, C, taps, n, state,
                                                          slot_stride, tok_seg, seg_start, seg_slot);
    if (n > 1) {
        const dim3 grid2(S, (C + 255) / 256);
        fwb::pdl(causal_conv_advance_kernel<T>, grid2, 256, 0, stream)((const T*)in, ld, col0, C, n, state,
                                                                       slot_stride, seg_start, seg_slot);
    }
    return fwb_launch_status();
}

}  // namespace

// in, out: [T][ld] fp32 or bf16 (both of one type, different buffers); taps: [C][n] fp32; state: fp32, slot s
// at state + s * slot_stride, [n - 1][C] (may be null when n == 1); tok_seg: [T]; seg_start: [S + 1];
// seg_slot: [S].
FWB_API int fwb_causal_conv(const void* in, void* out, int is_bf16, long long ld, int col0, int C,
                            const float* taps, int n, float* state, long long slot_stride, const int* tok_seg,
                            const int* seg_start, const int* seg_slot, int T, int S, cudaStream_t stream) {
    if (T <= 0 || C <= 0) return FWB_OK;
    if (!in || !out || in == out || !taps || !tok_seg || !seg_start || !seg_slot || n < 1 || S <= 0 || col0 < 0 ||
        ld < col0 + C || (n > 1 && !state))
        return FWB_BAD_ARGUMENT;
    if (n > MAX_TAPS || (C + 255) / 256 > 65535) return FWB_TOO_LARGE;
    return is_bf16 ? launch<__nv_bfloat16>(in, out, ld, col0, C, taps, n, state, slot_stride, tok_seg, seg_start,
                                           seg_slot, T, S, stream)
                   : launch<float>(in, out, ld, col0, C, taps, n, state, slot_stride, tok_seg, seg_start, seg_slot,
                                   T, S, stream);
}

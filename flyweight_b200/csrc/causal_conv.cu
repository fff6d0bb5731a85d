// A short causal convolution over time on every channel of a row buffer, with the rolling inputs of every
// request kept between steps:
//
//     y[t][c] = sum_j taps[c][j] * u[t - n + 1 + j][c],   j = 0 .. n - 1,
//
// where u before the start of a sequence is zero.  A step brings segments (runs of consecutive tokens of
// one request); the n - 1 inputs in front of a segment come from the request's state slot, which holds
// the last n - 1 inputs of the sequence so far (oldest first, zero when the request starts).
//
//   fwb_causal_conv:  out[t][0 .. C) <- conv of the columns [col0, col0 + C) of `in` (rows `ld` entries apart;
//                     `out` is another buffer whose rows are `out_ld` apart), then the state of every
//                     segment's slot moves on to the segment's last n - 1 inputs.  With norm ranges (one or
//                     two column ranges of the output, each with a weight): every range of a row is brought to
//                     unit root mean square over `count` of its channels and multiplied by its weight before
//                     it is written, in the same launch (a block per token keeps the row in shared memory).
// Two launches: the convolution reads the old state, the second kernel writes the new one.  All
// arithmetic is fp32, taps applied in the order j = 0 .. n - 1 whatever the step's cut, and a row's sums of
// squares are added in an order the block size alone fixes.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int MAX_TAPS = 16;

struct ConvNormRange {
    int col0, width, count;
    const float* weight;
};

// One output: the taps in the order j = 0 .. n - 1 over the token's own row and the rows before it, which lie
// in this step's buffer (`local` tokens of the segment precede the token) or in the request's slot.
template <typename T>
__device__ __forceinline__ float conv_one(const T* __restrict__ in, size_t at, long long ld, const float* __restrict__ taps,
                                          int n, int c, int C, int local, const float* __restrict__ slot) {
    float acc = 0.0f;
    for (int j = 0; j < n; ++j) {
        const int back = n - 1 - j;                        // how far behind the token this tap reads
        const float u = back <= local ? to_f32<T>(in[at - (size_t)back * ld])
                                      : slot[(size_t)(n - 1 + local - back) * C + c];
        acc = fmaf(taps[(size_t)c * n + j], u, acc);
    }
    return acc;
}

// Four consecutive channels of one row as fp32 (16 bytes of fp32, 8 of bfloat16).
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&lo);
    raw.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// Two sums over a block at once; every thread gets both.  The order of additions is fixed by the block size.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* scratch /* 66 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) {
        scratch[warp] = a;
        scratch[33 + warp] = b;
    }
    __syncthreads();
    if (warp == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        const float ta = warp_sum(lane < warps ? scratch[lane] : 0.0f);
        const float tb = warp_sum(lane < warps ? scratch[33 + lane] : 0.0f);
        if (lane == 0) {
            scratch[32] = ta;
            scratch[65] = tb;
        }
    }
    __syncthreads();
    return make_float2(scratch[32], scratch[65]);
}

// One block per token, four channels a thread and turn (16-byte loads), NT taps held in registers: the
// convolved row stays in shared memory while the sums of squares of its one or two norm ranges are reduced,
// then every entry leaves scaled (entries outside the ranges, or all of them when there is no range, leave as
// they are).  C, ld, out_ld, col0 and the ranges' borders are multiples of four.
template <typename T, int NT>
__global__ void __launch_bounds__(256, 6)
causal_conv_norm_vec_kernel(const T* __restrict__ in, T* __restrict__ out, long long ld, long long out_ld, int col0,
                            int C, const float* __restrict__ taps, const float* __restrict__ state,
                            long long slot_stride, const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
                            const int* __restrict__ seg_slot, ConvNormRange r0, ConvNormRange r1, float eps) {
    fwb::pdl_entry();
    extern __shared__ float4 row4[];               // [C / 4]
    __shared__ float scratch[66];
    const int t = blockIdx.x;
    const int seg = tok_seg[t];
    const int local = t - seg_start[seg];
    const float* slot = state + (size_t)seg_slot[seg] * slot_stride;
    const T* mine = in + (size_t)t * ld + col0;
    float ss0 = 0.0f, ss1 = 0.0f;
    for (int c = 4 * threadIdx.x; c < C; c += 4 * blockDim.x) {
        float w[4 * NT];                           // taps of channels c .. c+3: [channel][tap]
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const float4 piece = *reinterpret_cast<const float4*>(taps + (size_t)c * NT + 4 * i);
            w[4 * i] = piece.x, w[4 * i + 1] = piece.y, w[4 * i + 2] = piece.z, w[4 * i + 3] = piece.w;
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int back = NT - 1 - j;
            const float4 u = back <= local ? load4<T>(mine + c - (size_t)back * ld)
                                           : *reinterpret_cast<const float4*>(slot + (size_t)(NT - 1 + local - back) * C + c);
            acc.x = fmaf(w[j], u.x, acc.x), acc.y = fmaf(w[NT + j], u.y, acc.y);
            acc.z = fmaf(w[2 * NT + j], u.z, acc.z), acc.w = fmaf(w[3 * NT + j], u.w, acc.w);
        }
        row4[c >> 2] = acc;
        const float sq = fmaf(acc.x, acc.x, fmaf(acc.y, acc.y, fmaf(acc.z, acc.z, acc.w * acc.w)));
        if (c >= r0.col0 && c < r0.col0 + r0.width) ss0 += sq;
        else if (c >= r1.col0 && c < r1.col0 + r1.width) ss1 += sq;
    }
    float inv0 = 0.0f, inv1 = 0.0f;
    if (r0.width > 0) {
        const float2 sums = block_sum2(ss0, ss1, scratch);
        inv0 = rsqrtf(sums.x / (float)(r0.count > 0 ? r0.count : 1) + eps);
        inv1 = rsqrtf(sums.y / (float)(r1.count > 0 ? r1.count : 1) + eps);
    }
    T* dst = out + (size_t)t * out_ld;
    for (int c = 4 * threadIdx.x; c < C; c += 4 * blockDim.x) {
        float4 v = row4[c >> 2];                   // (written by this very thread)
        if (c >= r0.col0 && c < r0.col0 + r0.width) {
            const float4 g = *reinterpret_cast<const float4*>(r0.weight + (c - r0.col0));
            v.x = (v.x * inv0) * g.x, v.y = (v.y * inv0) * g.y, v.z = (v.z * inv0) * g.z, v.w = (v.w * inv0) * g.w;
        } else if (c >= r1.col0 && c < r1.col0 + r1.width) {
            const float4 g = *reinterpret_cast<const float4*>(r1.weight + (c - r1.col0));
            v.x = (v.x * inv1) * g.x, v.y = (v.y * inv1) * g.y, v.z = (v.z * inv1) * g.z, v.w = (v.w * inv1) * g.w;
        }
        store4<T>(dst + c, v);
    }
}

// One block per token: the convolved row stays in shared memory while the sums of squares of its one or two
// norm ranges are reduced, then every entry leaves scaled (entries outside the ranges leave as they are).
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_norm_kernel(const T* __restrict__ in, T* __restrict__ out, long long ld, long long out_ld, int col0, int C,
                        const float* __restrict__ taps, int n, const float* __restrict__ state, long long slot_stride,
                        const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
                        const int* __restrict__ seg_slot, ConvNormRange r0, ConvNormRange r1, float eps) {
    fwb::pdl_entry();
    extern __shared__ float row[];                 // [C]
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int seg = tok_seg[t];
    const int local = t - seg_start[seg];
    const float* slot = state + (size_t)seg_slot[seg] * slot_stride;
    float ss0 = 0.0f, ss1 = 0.0f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float v = conv_one<T>(in, (size_t)t * ld + col0 + c, ld, taps, n, c, C, local, slot);
        row[c] = v;
        if (c >= r0.col0 && c < r0.col0 + r0.width) ss0 = fmaf(v, v, ss0);
        else if (c >= r1.col0 && c < r1.col0 + r1.width) ss1 = fmaf(v, v, ss1);
    }
    const float inv0 = rsqrtf(block_sum(ss0, scratch) / (float)(r0.count > 0 ? r0.count : 1) + eps);
    const float inv1 = r1.width > 0 ? rsqrtf(block_sum(ss1, scratch) / (float)(r1.count > 0 ? r1.count : 1) + eps) : 0.0f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float v = row[c];
        if (c >= r0.col0 && c < r0.col0 + r0.width) v = (v * inv0) * r0.weight[c - r0.col0];
        else if (c >= r1.col0 && c < r1.col0 + r1.width) v = (v * inv1) * r1.weight[c - r1.col0];
        out[(size_t)t * out_ld + c] = from_f32<T>(v);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* __restrict__ in, T* __restrict__ out, long long ld, long long out_ld, int col0, int C,
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
    const float acc = conv_one<T>(in, (size_t)t * ld + col0 + c, ld, taps, n, c, C, local, slot);
    out[(size_t)t * out_ld + c] = from_f32<T>(acc);
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
int launch(const void* in, void* out, long long ld, long long out_ld, int col0, int C, const float* taps, int n,
           float* state, long long slot_stride, const int* tok_seg, const int* seg_start, const int* seg_slot,
           int T_tokens, int S, ConvNormRange r0, ConvNormRange r1, float eps, cudaStream_t stream) {
    const bool by_four = n <= 4 && C % 4 == 0 && ld % 4 == 0 && out_ld % 4 == 0 && col0 % 4 == 0 && r0.col0 % 4 == 0 &&
                         r0.width % 4 == 0 && r1.col0 % 4 == 0 && r1.width % 4 == 0 && (size_t)C * sizeof(float) <= 160 * 1024 &&
                         (((uintptr_t)in | (uintptr_t)out | (uintptr_t)taps | (uintptr_t)state | (uintptr_t)r0.weight |
                           (uintptr_t)r1.weight) & 15) == 0 && (slot_stride % 4 == 0);
    if (by_four) {
        const size_t smem = (size_t)C * sizeof(float);
#define FWB_CONV_VEC(NT)                                                                                          \
    do {                                                                                                          \
        if (smem > 48 * 1024)                                                                                     \
            cudaFuncSetAttribute(causal_conv_norm_vec_kernel<T, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                                      \
        fwb::pdl(causal_conv_norm_vec_kernel<T, NT>, T_tokens, 256, smem, stream)(                                \
            (const T*)in, (T*)out, ld, out_ld, col0, C, taps, state, slot_stride, tok_seg, seg_start, seg_slot,  \
            r0, r1, eps);                                                                                         \
    } while (0)
        switch (n) {
            case 1: FWB_CONV_VEC(1); break;
            case 2: FWB_CONV_VEC(2); break;
            case 3: FWB_CONV_VEC(3); break;
            default: FWB_CONV_VEC(4); break;
        }
#undef FWB_CONV_VEC
    } else if (r0.width > 0) {
        const size_t smem = (size_t)C * sizeof(float);
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(causal_conv_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fwb::pdl(causal_conv_norm_kernel<T>, T_tokens, 256, smem, stream)(
            (const T*)in, (T*)out, ld, out_ld, col0, C, taps, n, state, slot_stride, tok_seg, seg_start, seg_slot, r0,
            r1, eps);
    } else {
        const dim3 grid(T_tokens, (C + 255) / 256);
        fwb::pdl(causal_conv_kernel<T>, grid, 256, 0, stream)((const T*)in, (T*)out, ld, out_ld, col0, C, taps, n,
                                                              state, slot_stride, tok_seg, seg_start, seg_slot);
    }
    if (n > 1) {
        const dim3 grid2(S, (C + 255) / 256);
        fwb::pdl(causal_conv_advance_kernel<T>, grid2, 256, 0, stream)((const T*)in, ld, col0, C, n, state,
                                                                       slot_stride, seg_start, seg_slot);
    }
    return fwb_launch_status();
}

}  // namespace

// in: [T][ld], out: [T][out_ld], fp32 or bf16 (both of one type, different buffers); taps: [C][n] fp32; state: fp32,
// slot s at state + s * slot_stride, [n - 1][C] (may be null when n == 1); tok_seg: [T]; seg_start: [S + 1];
// seg_slot: [S].  Norm ranges (width0 == 0: none; width1 == 0: one): columns [c0, c0 + width) of the output, the
// mean of squares over `count` channels, weights fp32 [width].
FWB_API int fwb_causal_conv(const void* in, void* out, int is_bf16, long long ld, long long out_ld, int col0, int C,
                            const float* taps, int n, float* state, long long slot_stride, const int* tok_seg,
                            const int* seg_start, const int* seg_slot, int T, int S, int norm_col0, int norm_width0,
                            int norm_count0, const float* norm_w0, int norm_col1, int norm_width1, int norm_count1,
                            const float* norm_w1, float eps, cudaStream_t stream) {
    if (T <= 0 || C <= 0) return FWB_OK;
    if (!in || !out || in == out || !taps || !tok_seg || !seg_start || !seg_slot || n < 1 || S <= 0 || col0 < 0 ||
        ld < col0 + C || out_ld < C || (n > 1 && !state))
        return FWB_BAD_ARGUMENT;
    if (n > MAX_TAPS || (C + 255) / 256 > 65535) return FWB_TOO_LARGE;
    ConvNormRange r0{norm_col0, norm_width0, norm_count0, norm_w0}, r1{norm_col1, norm_width1, norm_count1, norm_w1};
    if (r0.width > 0) {
        if (!r0.weight || r0.col0 < 0 || r0.col0 + r0.width > C || (r1.width > 0 && (!r1.weight || r1.col0 < 0 ||
                                                                                      r1.col0 + r1.width > C)))
            return FWB_BAD_ARGUMENT;
        if ((size_t)C * sizeof(float) > 160 * 1024) return FWB_TOO_LARGE;
    } else if (r1.width > 0) {
        return FWB_BAD_ARGUMENT;
    }
    return is_bf16 ? launch<__nv_bfloat16>(in, out, ld, out_ld, col0, C, taps, n, state, slot_stride, tok_seg, seg_start,
                                           seg_slot, T, S, r0, r1, eps, stream)
                   : launch<float>(in, out, ld, out_ld, col0, C, taps, n, state, slot_stride, tok_seg, seg_start,
                                   seg_slot, T, S, r0, r1, eps, stream);
}

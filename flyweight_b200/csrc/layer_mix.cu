// Small kernels of layers whose mixer and feed-forward read one norm side by side, with a scale per
// channel on each result, a token-indexed side input, gates on attention outputs and values mixed
// between layers.  All arithmetic is fp32; stores round to the buffer's type.
//
//   fwb_rmsnorm_ranges:     in place, per row and per column range r: buf[c0_r .. c0_r+n_r) <- w_r * unit(.)
//                           with the mean of squares divided by count_r (zero padding inside a range does
//                           not count)
//   fwb_value_mix:          save: first[t][:] = rows[t][c0 .. c0+n);  mix: rows[t][c0+i] <- (1-lam) rows + lam first
//   fwb_sigmoid_gate_mul:   y[t][h][c] *= sigmoid(gate[t][h*gw + (gw == 1 ? 0 : c)])
//   fwb_scaled_add:         x[t][c] += s1[c] a[t][c] (+ s2[c] b[t][c])                        (fp32; a bf16 copy on request)
//   fwb_unary_act:          out = act(in), act = relu squared | silu | sigmoid | gelu (tanh form)
//   fwb_side_gate:          out[t][c] = gelu(g[t][c]) * table[token[t]][c0 + c]
//   fwb_scale:              x *= s                                                            (fp32)
//   fwb_pair_norm_mean:     y = 0.5 (wa unit(a) + wb unit(b))                                 (fp32)
//   fwb_gated_rmsnorm:      out[t][:] = w unit(o[t][:]) * sigmoid(gate[t][:])
#include "common.cuh"

using namespace fwb;

namespace {

__device__ __forceinline__ float sigmoid_f32(float g) {
    const float e = expf(-fabsf(g));
    return g >= 0.0f ? 1.0f / (1.0f + e) : e / (1.0f + e);
}

struct NormRange {
    int col0, width, count;
    const float* weight;
};

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_ranges_kernel(T* __restrict__ buf, long long row_stride, NormRange r0, NormRange r1, float eps) {
    fwb::pdl_entry();
    __shared__ float scratch[33];
    const NormRange r = blockIdx.y == 0 ? r0 : r1;
    T* row = buf + (size_t)blockIdx.x * row_stride + r.col0;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < r.width; i += blockDim.x) {
        const float v = to_f32<T>(row[i]);
        ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)r.count + eps);
    for (int i = threadIdx.x; i < r.width; i += blockDim.x)
        row[i] = from_f32<T>((to_f32<T>(row[i]) * inv) * r.weight[i]);
}

template <typename T>
__global__ void value_mix_kernel(T* __restrict__ rows, long long row_stride, int col0, int width,
                                 T* __restrict__ first, const float* __restrict__ lam, int n_rows, int mix) {
    fwb::pdl_entry();
    const size_t n = (size_t)n_rows * width;
    const float l = mix ? lam[0] : 0.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width, c = i - t * width;
        T* at = rows + t * row_stride + col0 + c;
        if (mix) *at = from_f32<T>((1.0f - l) * to_f32<T>(*at) + l * to_f32<T>(first[i]));
        else first[i] = *at;
    }
}

// gate rows are `gate_stride` entries apart (heads * gate_width of them in use)
template <typename T, typename TG>
__global__ void sigmoid_gate_mul_kernel(T* __restrict__ y, const TG* __restrict__ gate, long long gate_stride,
                                        int n_rows, int heads, int head_dim, int gate_width) {
    fwb::pdl_entry();
    const size_t n = (size_t)n_rows * heads * head_dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t th = i / head_dim;
        const int c = (int)(i - th * head_dim);
        const size_t t = th / heads;
        const int h = (int)(th - t * heads);
        const float g = to_f32<TG>(gate[t * gate_stride + (size_t)h * gate_width + (gate_width == 1 ? 0 : c)]);
        y[i] = from_f32<T>(to_f32<T>(y[i]) * sigmoid_f32(g));
    }
}

__global__ void scaled_add_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ s1,
                                  const float* __restrict__ b, const float* __restrict__ s2, __nv_bfloat16* __restrict__ copy,
                                  int n_rows, int H) {
    fwb::pdl_entry();
    const size_t n = (size_t)n_rows * H;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % H);
        float d = (s1 ? s1[c] : 1.0f) * a[i];
        if (b) d += (s2 ? s2[c] : 1.0f) * b[i];
        const float sum = x[i] + d;
        x[i] = sum;
        if (copy) copy[i] = __float2bfloat16_rn(sum);
    }
}

__device__ __forceinline__ float unary_f32(float v, int act) {
    switch (act) {
        case 0: { const float r = fmaxf(v, 0.0f); return r * r; }
        case 1: return silu_f32(v);
        case 2: return sigmoid_f32(v);
        default: return gelu_tanh_f32(v);
    }
}

template <typename TI, typename TO>
__global__ void unary_act_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n, int act) {
    fwb::pdl_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(unary_f32(to_f32<TI>(in[i]), act));
}

// bfloat16 to bfloat16, eight entries (16 bytes) a thread and turn
__global__ void unary_act_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, size_t groups, int act) {
    fwb::pdl_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
        uint4 v = in[i];
        __nv_bfloat162* pair = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(pair[j]);
            pair[j] = __floats2bfloat162_rn(unary_f32(f.x, act), unary_f32(f.y, act));
        }
        out[i] = v;
    }
}

template <typename TI, typename TT, typename TO>
__global__ void side_gate_kernel(const TI* __restrict__ g, const TT* __restrict__ table, int table_width, int col0,
                                 const int* __restrict__ tokens, int vocab, TO* __restrict__ out, int n_rows, int dim) {
    fwb::pdl_entry();
    const size_t n = (size_t)n_rows * dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / dim;
        const int c = (int)(i - t * dim);
        int token = tokens[t];
        token = token < 0 ? 0 : (token >= vocab ? vocab - 1 : token);     // (a bad id was flagged by the embedding)
        const float e = to_f32<TT>(table[(size_t)token * table_width + col0 + c]);
        out[i] = from_f32<TO>(gelu_tanh_f32(to_f32<TI>(g[i])) * e);
    }
}

__global__ void scale_kernel(float* __restrict__ x, size_t n, float s) {
    fwb::pdl_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] *= s;
}

__global__ void __launch_bounds__(256)
pair_norm_mean_kernel(const float* __restrict__ a, const float* __restrict__ wa, const float* __restrict__ b,
                      const float* __restrict__ wb, float eps, float* __restrict__ y, int H) {
    fwb::pdl_entry();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * H;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float u = a[base + i], v = b[base + i];
        sa = fmaf(u, u, sa);
        sb = fmaf(v, v, sb);
    }
    const float ia = rsqrtf(block_sum(sa, scratch) / (float)H + eps);
    const float ib = rsqrtf(block_sum(sb, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        y[base + i] = 0.5f * ((a[base + i] * ia) * wa[i] + (b[base + i] * ib) * wb[i]);
}

template <typename TG, typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ o, const TG* __restrict__ gate, long long gate_stride,
                     const float* __restrict__ w, float eps, TO* __restrict__ out, int H) {
    fwb::pdl_entry();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * H;
    const TG* g = gate + (size_t)blockIdx.x * gate_stride;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(o[base + i], o[base + i], ss);
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[base + i] = from_f32<TO>(((o[base + i] * inv) * w[i]) * sigmoid_f32(to_f32<TG>(g[i])));
}

inline int blocks_for(size_t n) { return (int)((n + 255) / 256 > 8192 ? 8192 : (n + 255) / 256); }

}  // namespace

using bf = __nv_bfloat16;

// buf: [T][row_stride] fp32 or bf16.  Up to two column ranges per row (width1 == 0: one): each is brought
// to unit root mean square over `count` of its channels and multiplied by its weight (fp32 [width]).
FWB_API int fwb_rmsnorm_ranges(void* buf, int is_bf16, long long row_stride, int T, int col0, int width0, int count0,
                               const float* w0, int col1, int width1, int count1, const float* w1, float eps,
                               cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!buf || !w0 || width0 <= 0 || count0 <= 0 || col0 < 0 || col0 + width0 > row_stride) return FWB_BAD_ARGUMENT;
    if (width1 > 0 && (!w1 || count1 <= 0 || col1 < 0 || col1 + width1 > row_stride)) return FWB_BAD_ARGUMENT;
    const NormRange r0{col0, width0, count0, w0}, r1{col1, width1, count1 > 0 ? count1 : 1, w1};
    const dim3 grid(T, width1 > 0 ? 2 : 1);
    if (is_bf16) fwb::pdl(rmsnorm_ranges_kernel<bf>, grid, 256, 0, stream)((bf*)buf, row_stride, r0, r1, eps);
    else fwb::pdl(rmsnorm_ranges_kernel<float>, grid, 256, 0, stream)((float*)buf, row_stride, r0, r1, eps);
    return fwb_launch_status();
}

// rows: [T][row_stride]; first: [T][width], both of one type.  mix == 0: first <- the columns; mix == 1: the
// columns <- (1 - lam) columns + lam first, lam one fp32 number on the device.
FWB_API int fwb_value_mix(void* rows, int is_bf16, long long row_stride, int col0, int width, void* first,
                          const float* lam, int T, int mix, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!rows || !first || width <= 0 || col0 < 0 || col0 + width > row_stride || (mix && !lam)) return FWB_BAD_ARGUMENT;
    const int blocks = blocks_for((size_t)T * width);
    if (is_bf16) fwb::pdl(value_mix_kernel<bf>, blocks, 256, 0, stream)((bf*)rows, row_stride, col0, width, (bf*)first, lam, T, mix);
    else fwb::pdl(value_mix_kernel<float>, blocks, 256, 0, stream)((float*)rows, row_stride, col0, width, (float*)first, lam, T, mix);
    return fwb_launch_status();
}

// y: [T][heads][head_dim], gate: [T][heads][gate_width] with gate_width 1 (a gate per head) or head_dim.
FWB_API int fwb_sigmoid_gate_mul(void* y, const void* gate, int is_bf16, int T, int heads, int head_dim,
                                 int gate_width, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!y || !gate || heads <= 0 || head_dim <= 0 || (gate_width != 1 && gate_width != head_dim)) return FWB_BAD_ARGUMENT;
    const int blocks = blocks_for((size_t)T * heads * head_dim);
    const long long stride = (long long)heads * gate_width;
    if (is_bf16) fwb::pdl(sigmoid_gate_mul_kernel<bf, bf>, blocks, 256, 0, stream)((bf*)y, (const bf*)gate, stride, T, heads, head_dim, gate_width);
    else fwb::pdl(sigmoid_gate_mul_kernel<float, float>, blocks, 256, 0, stream)((float*)y, (const float*)gate, stride, T, heads, head_dim, gate_width);
    return fwb_launch_status();
}

// bfloat16 rows, eight entries (16 bytes) a thread and turn, a gate per head: one sigmoid for the eight.
template <typename TG>
__global__ void sigmoid_head_gate_mul_bf16x8_kernel(uint4* __restrict__ y, const TG* __restrict__ gate, long long gate_stride,
                                                    size_t n8, int heads, int head_dim8) {
    fwb::pdl_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t th = i / head_dim8;
        const size_t t = th / heads;
        const float s = sigmoid_f32(to_f32<TG>(gate[t * gate_stride + (th - t * heads)]));
        uint4 raw = y[i];
        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(pairs[j]);
            pairs[j] = __floats2bfloat162_rn(v.x * s, v.y * s);
        }
        y[i] = raw;
    }
}

// The same with the gate inside the rows of another buffer (some columns of a fused projection): `gate` points at
// the first gate entry of row 0, rows are `gate_stride` entries apart, and its type may differ from y's.
FWB_API int fwb_sigmoid_gate_mul_strided(void* y, int y_bf16, const void* gate, int gate_bf16, long long gate_stride,
                                         int T, int heads, int head_dim, int gate_width, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!y || !gate || heads <= 0 || head_dim <= 0 || (gate_width != 1 && gate_width != head_dim) ||
        gate_stride < (long long)heads * gate_width)
        return FWB_BAD_ARGUMENT;
    const int blocks = blocks_for((size_t)T * heads * head_dim);
    if (y_bf16 && gate_width == 1 && head_dim % 8 == 0 && ((uintptr_t)y & 15) == 0) {
        const size_t n8 = (size_t)T * heads * (head_dim / 8);
        if (gate_bf16)
            fwb::pdl(sigmoid_head_gate_mul_bf16x8_kernel<bf>, blocks_for(n8), 256, 0, stream)((uint4*)y, (const bf*)gate, gate_stride, n8, heads, head_dim / 8);
        else
            fwb::pdl(sigmoid_head_gate_mul_bf16x8_kernel<float>, blocks_for(n8), 256, 0, stream)((uint4*)y, (const float*)gate, gate_stride, n8, heads, head_dim / 8);
        return fwb_launch_status();
    }
    if (y_bf16 && gate_bf16)
        fwb::pdl(sigmoid_gate_mul_kernel<bf, bf>, blocks, 256, 0, stream)((bf*)y, (const bf*)gate, gate_stride, T, heads, head_dim, gate_width);
    else if (y_bf16)
        fwb::pdl(sigmoid_gate_mul_kernel<bf, float>, blocks, 256, 0, stream)((bf*)y, (const float*)gate, gate_stride, T, heads, head_dim, gate_width);
    else if (!gate_bf16)
        fwb::pdl(sigmoid_gate_mul_kernel<float, float>, blocks, 256, 0, stream)((float*)y, (const float*)gate, gate_stride, T, heads, head_dim, gate_width);
    else
        return FWB_UNSUPPORTED;
    return fwb_launch_status();
}

// x, a, b: [T][H] fp32 (b may be null); s1, s2: [H] fp32 or null (no scale); copy_bf16: [T][H] bfloat16 or null
// (the new stream once more, rounded, for a product that reads it next).
FWB_API int fwb_scaled_add(float* x, const float* a, const float* s1, const float* b, const float* s2, void* copy_bf16,
                           int T, int H, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!x || !a || H <= 0) return FWB_BAD_ARGUMENT;
    fwb::pdl(scaled_add_kernel, blocks_for((size_t)T * H), 256, 0, stream)(x, a, s1, b, s2, (__nv_bfloat16*)copy_bf16, T, H);
    return fwb_launch_status();
}

// act: 0 relu squared, 1 silu, 2 sigmoid, 3 gelu (tanh form).  `out` may be `in`.
FWB_API int fwb_unary_act(const void* in, int in_bf16, void* out, int out_bf16, long long n, int act, cudaStream_t stream) {
    if (n <= 0) return FWB_OK;
    if (!in || !out || act < 0 || act > 3) return FWB_BAD_ARGUMENT;
    const int blocks = blocks_for((size_t)n);
    if (in_bf16 && out_bf16 && n % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0)
        fwb::pdl(unary_act_bf16x8_kernel, blocks_for((size_t)n / 8), 256, 0, stream)((const uint4*)in, (uint4*)out, (size_t)n / 8, act);
    else if (in_bf16 && out_bf16) fwb::pdl(unary_act_kernel<bf, bf>, blocks, 256, 0, stream)((const bf*)in, (bf*)out, (size_t)n, act);
    else if (!in_bf16 && out_bf16) fwb::pdl(unary_act_kernel<float, bf>, blocks, 256, 0, stream)((const float*)in, (bf*)out, (size_t)n, act);
    else if (!in_bf16 && !out_bf16) fwb::pdl(unary_act_kernel<float, float>, blocks, 256, 0, stream)((const float*)in, (float*)out, (size_t)n, act);
    else return FWB_UNSUPPORTED;
    return fwb_launch_status();
}

// g: [T][dim]; table: [vocab][table_width] (fp32 or bf16); out: [T][dim] = gelu(g) * table[token][col0 + c].
FWB_API int fwb_side_gate(const void* g, int g_bf16, const void* table, int table_bf16, int table_width, int col0,
                          const int* tokens, int vocab, void* out, int out_bf16, int T, int dim, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!g || !table || !tokens || !out || dim <= 0 || col0 < 0 || col0 + dim > table_width || vocab <= 0) return FWB_BAD_ARGUMENT;
    const int blocks = blocks_for((size_t)T * dim);
    if (g_bf16 && table_bf16 && out_bf16)
        fwb::pdl(side_gate_kernel<bf, bf, bf>, blocks, 256, 0, stream)((const bf*)g, (const bf*)table, table_width, col0, tokens, vocab, (bf*)out, T, dim);
    else if (!g_bf16 && !table_bf16 && !out_bf16)
        fwb::pdl(side_gate_kernel<float, float, float>, blocks, 256, 0, stream)((const float*)g, (const float*)table, table_width, col0, tokens, vocab, (float*)out, T, dim);
    else if (!g_bf16 && table_bf16 && out_bf16)
        fwb::pdl(side_gate_kernel<float, bf, bf>, blocks, 256, 0, stream)((const float*)g, (const bf*)table, table_width, col0, tokens, vocab, (bf*)out, T, dim);
    else return FWB_UNSUPPORTED;
    return fwb_launch_status();
}

FWB_API int fwb_scale(float* x, long long n, float s, cudaStream_t stream) {
    if (n <= 0) return FWB_OK;
    if (!x) return FWB_BAD_ARGUMENT;
    fwb::pdl(scale_kernel, blocks_for((size_t)n), 256, 0, stream)(x, (size_t)n, s);
    return fwb_launch_status();
}

// a, b, y: [T][H] fp32; wa, wb: [H] fp32.
FWB_API int fwb_pair_norm_mean(const float* a, const float* wa, const float* b, const float* wb, float eps, float* y,
                               int T, int H, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!a || !wa || !b || !wb || !y || H <= 0) return FWB_BAD_ARGUMENT;
    fwb::pdl(pair_norm_mean_kernel, T, 256, 0, stream)(a, wa, b, wb, eps, y, H);
    return fwb_launch_status();
}

// o: [T][H] fp32; gate: rows of H entries, `gate_stride` entries apart (fp32 or bf16); w: [H]; out: [T][H].
FWB_API int fwb_gated_rmsnorm(const float* o, const void* gate, int gate_bf16, long long gate_stride, const float* w,
                              float eps, void* out, int out_bf16, int T, int H, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!o || !gate || !w || !out || H <= 0 || gate_stride < H) return FWB_BAD_ARGUMENT;
    if (gate_bf16 && out_bf16)
        fwb::pdl(gated_rmsnorm_kernel<bf, bf>, T, 256, 0, stream)(o, (const bf*)gate, gate_stride, w, eps, (bf*)out, H);
    else if (!gate_bf16 && !out_bf16)
        fwb::pdl(gated_rmsnorm_kernel<float, float>, T, 256, 0, stream)(o, (const float*)gate, gate_stride, w, eps, (float*)out, H);
    else if (!gate_bf16 && out_bf16)
        fwb::pdl(gated_rmsnorm_kernel<float, bf>, T, 256, 0, stream)(o, (const float*)gate, gate_stride, w, eps, (bf*)out, H);
    else return FWB_UNSUPPORTED;
    return fwb_launch_status();
}

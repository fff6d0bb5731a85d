// Kernels for layers that put a weighted RMS norm on a sublayer's output before the residual sum, and
// the gated product of a feed-forward with a choice of activation.
//
//   fwb_rmsnorm_add:   x[t] += w * y[t] / sqrt(mean(y[t]^2) + eps)                 (fp32, in place)
//                      and, when a second weight is given, the norm that the next sublayer reads,
//                      h[t] = w2 * x[t] / sqrt(mean(x[t]^2) + eps2), from the new x in the same pass
//   fwb_gate_act_mul:  out[t][f] = act(gu[t][f]) * gu[t][F + f],  act = silu | gelu (tanh form); or the clamped
//                      swish, min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1)
// All arithmetic is fp32; a row is summed in an order that depends on its length alone.
#include "common.cuh"

using namespace fwb;

namespace {

template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, float eps,
                   const float* __restrict__ w2, float eps2, TO* __restrict__ h, int H) {
    fwb::pdl_entry();
    extern __shared__ float row[];            // the new x of this row
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = y[base + i];
        ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
    float sx = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = x[base + i] + (y[base + i] * inv) * w[i];
        x[base + i] = v;
        if (w2) {
            row[i] = v;
            sx = fmaf(v, v, sx);
        }
    }
    if (!w2) return;
    const float inv2 = rsqrtf(block_sum(sx, scratch) / (float)H + eps2);
    for (int i = threadIdx.x; i < H; i += blockDim.x) h[base + i] = from_f32<TO>((row[i] * inv2) * w2[i]);
}

template <typename TI, typename TO>
__global__ void gate_act_mul_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int T, int F, int act,
                                    float limit) {
    fwb::pdl_entry();
    const size_t n = (size_t)T * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / F, f = i - t * F;
        const float g = to_f32<TI>(gu[t * 2 * F + f]);
        const float u = to_f32<TI>(gu[t * 2 * F + F + f]);
        out[i] = from_f32<TO>(gated_f32(act, limit, g, u));
    }
}

}  // namespace

// x, y: [T][H] fp32; w: [H] fp32.  w2 (may be null), eps2, h ([T][H], fp32 or bf16): the next norm.
FWB_API int fwb_rmsnorm_add(float* x, const float* y, const float* w, float eps, const float* w2, float eps2,
                            void* h, int h_bf16, int T, int H, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!x || !y || !w || H <= 0 || (w2 && !h)) return FWB_BAD_ARGUMENT;
    const size_t smem = w2 ? (size_t)H * sizeof(float) : 0;
    if (smem > 160 * 1024) return FWB_TOO_LARGE;
    if (h_bf16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(rmsnorm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fwb::pdl(rmsnorm_add_kernel<__nv_bfloat16>, T, 256, smem, stream)(x, y, w, eps, w2, eps2, (__nv_bfloat16*)h, H);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(rmsnorm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fwb::pdl(rmsnorm_add_kernel<float>, T, 256, smem, stream)(x, y, w, eps, w2, eps2, (float*)h, H);
    }
    return fwb_launch_status();
}

// gu: [T][2F] (gate columns, then up columns); out: [T][F].  act: 0 silu, 1 gelu (tanh form), 2 the clamped
// swish with its `limit`.
FWB_API int fwb_gate_act_mul(const void* gu, int in_bf16, void* out, int out_bf16, int T, int F, int act,
                             float limit, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!gu || !out || F <= 0 || act < 0 || act > 2) return FWB_BAD_ARGUMENT;
    const size_t n = (size_t)T * F;
    const int blocks = (int)((n + 255) / 256 > 8192 ? 8192 : (n + 255) / 256);
    if (in_bf16 && out_bf16)
        fwb::pdl(gate_act_mul_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 256, 0, stream)(
            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F, act, limit);
    else if (!in_bf16 && out_bf16)
        fwb::pdl(gate_act_mul_kernel<float, __nv_bfloat16>, blocks, 256, 0, stream)(
            (const float*)gu, (__nv_bfloat16*)out, T, F, act, limit);
    else if (!in_bf16 && !out_bf16)
        fwb::pdl(gate_act_mul_kernel<float, float>, blocks, 256, 0, stream)((const float*)gu, (float*)out, T, F, act, limit);
    else
        return FWB_UNSUPPORTED;
    return fwb_launch_status();
}

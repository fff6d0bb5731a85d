// Linear attention with a fixed decay per head: a recurrence whose state is one [dim][vdim] matrix per
// head and request, kept in fp32 in the request's slot.
//
//   S_t = decay_h S_(t-1) + k_t v_t^T;     o_t = S_t^T q_t
//
// q, k (heads x dim) and v (heads x vdim) are columns of one fp32 projection row per token; with
// `act_silu` they pass silu on the way in.  One block owns 32 columns of one head's state for one
// segment of the step and walks the segment's tokens in order; the state's rows are cut over the
// block's warps, 16 rows a thread, in registers.  Tokens are staged 16 at a time in shared memory, so the
// walk itself reads no global memory; the partial read-outs of the warps are summed in warp order when
// a stage is done.  A token's arithmetic is the same whatever the cut of the sequence into steps, so a
// prompt in one piece, in portions or token by token gives the same bits.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int COLS = 32;      // state columns per block (one per lane)
constexpr int ROWS = 16;      // state rows per thread
constexpr int STAGE = 16;     // tokens staged at a time
constexpr int MAX_SPLITS = 32;

__global__ void __launch_bounds__(COLS * MAX_SPLITS)
decay_scan_kernel(const float* __restrict__ p, long long row_stride, int q_col, int k_col, int v_col, int act_silu,
                  const float* __restrict__ decay, float* __restrict__ state, long long slot_stride,
                  const int* __restrict__ seg_start, const int* __restrict__ seg_slot, float* __restrict__ o,
                  int H, int d, int e) {
    fwb::pdl_entry();
    extern __shared__ float smem[];
    const int splits = blockDim.x / COLS, dpad = splits * ROWS;
    float* qs = smem;                          // [STAGE][dpad]
    float* ks = qs + STAGE * dpad;             // [STAGE][dpad]
    float* vs = ks + STAGE * dpad;             // [STAGE][COLS]
    float* part = vs + STAGE * COLS;           // [splits][STAGE][COLS]
    const int seg = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * COLS;
    const int el = threadIdx.x & (COLS - 1), ds = threadIdx.x / COLS;
    const int col = e0 + el;
    const bool live = col < e;
    const int first = seg_start[seg], last = seg_start[seg + 1];
    const float g = decay[h];
    float* mine = state + (size_t)seg_slot[seg] * slot_stride + (size_t)h * d * e;

    float s[ROWS];
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
        const int row = ds * ROWS + j;
        s[j] = (live && row < d) ? mine[(size_t)row * e + col] : 0.0f;
    }
    for (int t0 = first; t0 < last; t0 += STAGE) {
        const int n = last - t0 < STAGE ? last - t0 : STAGE;
        __syncthreads();
        for (int i = threadIdx.x; i < STAGE * dpad; i += blockDim.x) {
            const int tok = i / dpad, row = i - tok * dpad;
            float qv = 0.0f, kv = 0.0f;
            if (tok < n && row < d) {
                const float* src = p + (size_t)(t0 + tok) * row_stride + (size_t)h * d + row;
                qv = src[q_col];
                kv = src[k_col];
                if (act_silu) {
                    qv = silu_f32(qv);
                    kv = silu_f32(kv);
                }
            }
            qs[i] = qv;
            ks[i] = kv;
        }
        for (int i = threadIdx.x; i < STAGE * COLS; i += blockDim.x) {
            const int tok = i / COLS, c = e0 + (i - tok * COLS);
            float v = 0.0f;
            if (tok < n && c < e) {
                v = p[(size_t)(t0 + tok) * row_stride + v_col + (size_t)h * e + c];
                if (act_silu) v = silu_f32(v);
            }
            vs[i] = v;
        }
        __syncthreads();
        for (int tok = 0; tok < n; ++tok) {
            const float v = vs[tok * COLS + el];
            const float* kr = ks + tok * dpad + ds * ROWS;
            const float* qr = qs + tok * dpad + ds * ROWS;
            float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
            for (int j = 0; j < ROWS; j += 2) {
                s[j] = fmaf(g, s[j], kr[j] * v);
                s[j + 1] = fmaf(g, s[j + 1], kr[j + 1] * v);
                a0 = fmaf(s[j], qr[j], a0);
                a1 = fmaf(s[j + 1], qr[j + 1], a1);
            }
            part[(ds * STAGE + tok) * COLS + el] = a0 + a1;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n * COLS; i += blockDim.x) {
            const int tok = i / COLS, c = i - tok * COLS;
            if (e0 + c >= e) continue;
            float sum = 0.0f;
            for (int w = 0; w < splits; ++w) sum += part[(w * STAGE + tok) * COLS + c];
            o[(size_t)(t0 + tok) * H * e + (size_t)h * e + e0 + c] = sum;
        }
    }
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
        const int row = ds * ROWS + j;
        if (live && row < d) mine[(size_t)row * e + col] = s[j];
    }
}

}  // namespace

// p: fp32 rows of `row_stride` entries, one per token, that hold q [H][d] from column q_col, k [H][d] from
// k_col and v [H][e] from v_col.  decay: fp32 [H].  state: fp32, a request's slot `slot_stride` entries after
// the one before, [H][d][e] at its head (read at the head of every segment and advanced).  seg_start [S+1],
// seg_slot [S]: the step's segments.  o: fp32 [T][H][e].
FWB_API int fwb_decay_scan(const float* p, long long row_stride, int q_col, int k_col, int v_col, int act_silu,
                           const float* decay, float* state, long long slot_stride, const int* seg_start,
                           const int* seg_slot, float* o, int T, int S, int H, int d, int e, cudaStream_t stream) {
    if (T <= 0 || S <= 0) return FWB_OK;
    if (!p || !decay || !state || !seg_start || !seg_slot || !o) return FWB_BAD_ARGUMENT;
    if (H <= 0 || d <= 0 || e <= 0 || q_col < 0 || k_col < 0 || v_col < 0) return FWB_BAD_ARGUMENT;
    if (row_stride < (long long)H * d || slot_stride < (long long)H * d * e) return FWB_BAD_ARGUMENT;
    const int splits = (d + ROWS - 1) / ROWS;
    if (splits > MAX_SPLITS || H > 65535) return FWB_TOO_LARGE;
    const int tiles = (e + COLS - 1) / COLS;
    if (tiles > 65535) return FWB_TOO_LARGE;
    const size_t smem = ((size_t)2 * STAGE * splits * ROWS + (size_t)STAGE * COLS + (size_t)splits * STAGE * COLS) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(decay_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    fwb::pdl(decay_scan_kernel, dim3(S, H, tiles), COLS * splits, smem, stream)(
        p, row_stride, q_col, k_col, v_col, act_silu, decay, state, slot_stride, seg_start, seg_slot, o, H, d, e);
    return fwb_launch_status();
}

// Mixture of experts: the router, the sorting of (token, expert) pairs by expert, the experts'
// gated products over the sorted rows, and the weighted sum.
//
//   route    scores s = softmax(router h) over all N router outputs (fp32).  The choice is made on
//            s + correction: the outputs form n_groups runs of N / n_groups neighbours, a run's value
//            is its largest choice value, only the `keep` best runs stay in the race (the others count
//            as minus infinity), and the `top` largest survivors are chosen.  The weights are the plain
//            s of the chosen, not renormalised.  Ties go to the lower index.
//   sort     pairs whose output is a real expert (index < E) are counted per expert, the counts are
//            scanned, every pair gets its row among its expert's rows, and the row tiles of the two
//            products are listed.  Outputs from E on are identity experts: they have no row.
//   gemm     one CTA per (row tile of one expert, tile of output features): rows gathered through the
//            sorted list, fp32 FMA accumulation over k in order.  Form 1: act(x gate^T) * (x up^T) for
//            the stacked matrix [gate rows | up rows]; form 0: the plain product in fp32.
//   gather   the sorted rows' inputs side by side, for the grouped tensor-core product (bfloat16)
//   combine  out[t] = sum over the token's pairs, in slot order, of weight * (expert row | h[t] itself
//            for an identity expert); alone, or followed in the same kernel by a weighted RMS norm of
//            the sum and the residual sum, x[t] += w * unit(out[t]).
// A pair's row is a sum over k in a fixed order whatever else is in the step, and a token's pairs are
// added in slot order, so a token's result does not depend on the batch.  Grids are sized for the
// worst case from the step's static sizes (every kernel reads the counts on the device), so a step
// can be captured in a CUDA graph.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int TM = 64, TN = 64, TK = 16;       // tile of the experts' products

template <typename TH>
__global__ void __launch_bounds__(512)
moe_route_kernel(const TH* __restrict__ h, const float* __restrict__ router, const float* __restrict__ correction,
                 int* __restrict__ ids, float* __restrict__ weights, int T, int W, int N, int n_groups, int keep,
                 int top, int vec) {
    fwb::pdl_entry();
    // One block per token.  Its warps share the router's outputs between them (output n: lanes stride
    // over k with sixteen sums in flight, added in one fixed order); warp 0 then chooses.
    extern __shared__ float shared[];             // s[N], choice[N], group value[n_groups]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    float* s = shared;
    float* choice = s + N;
    float* best = choice + N;
    const TH* row = h + (size_t)t * W;
    const int warps = blockDim.x >> 5;
    if (vec) {
        // K is cut over the warps, 128 entries a warp and turn (four a lane: one 16-byte piece of every
        // output's weights, all in flight together); a warp leaves one partial sum per output and turn
        // in shared memory, and warp 0 adds them in warp order
        float* partial = best + n_groups;          // [warps][N]
        for (int i = threadIdx.x; i < warps * N; i += blockDim.x) partial[i] = 0.0f;
        __syncthreads();
        for (int k0 = warp * 128; k0 < W; k0 += warps * 128) {
            const int k = k0 + lane * 4;
            const bool in = k < W;
            float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (in) {
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] = to_f32<TH>(row[k + j]);
            }
            for (int n0 = 0; n0 < N; n0 += 16) {
                float4 w[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    w[j] = (in && n0 + j < N) ? *reinterpret_cast<const float4*>(router + (size_t)(n0 + j) * W + k)
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float v = fmaf(x[3], w[j].w, fmaf(x[2], w[j].z, fmaf(x[1], w[j].y, x[0] * w[j].x)));
                    v = warp_sum(v);
                    if (lane == 0 && n0 + j < N) partial[warp * N + n0 + j] += v;
                }
            }
        }
        __syncthreads();
        if (warp == 0)
            for (int n = lane; n < N; n += 32) {
                float acc = 0.0f;
                for (int w = 0; w < warps; ++w) acc += partial[w * N + n];
                s[n] = acc;
            }
        __syncwarp();
    } else {
    for (int n = 2 * warp; n < N; n += 2 * warps) {
        // two outputs at a time: their weights and the token's row, sixteen strides of 32 each, in flight together
        const bool two = n + 1 < N;
        const float* w0 = router + (size_t)n * W;
        const float* w1 = router + (size_t)(two ? n + 1 : n) * W;
        float p0[16], p1[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) p0[j] = p1[j] = 0.0f;
        int k = lane;
        for (; k + 15 * 32 < W; k += 16 * 32) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float x = to_f32<TH>(row[k + 32 * j]);
                p0[j] = fmaf(x, w0[k + 32 * j], p0[j]);
                p1[j] = fmaf(x, w1[k + 32 * j], p1[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (k + 32 * j < W) {
                const float x = to_f32<TH>(row[k + 32 * j]);
                p0[j] = fmaf(x, w0[k + 32 * j], p0[j]);
                p1[j] = fmaf(x, w1[k + 32 * j], p1[j]);
            }
#pragma unroll
        for (int step = 8; step > 0; step >>= 1)
#pragma unroll
            for (int j = 0; j < step; ++j) {
                p0[j] += p0[j + step];
                p1[j] += p1[j + step];
            }
        const float a0 = warp_sum(p0[0]), a1 = warp_sum(p1[0]);
        if (lane == 0) {
            s[n] = a0;
            if (two) s[n + 1] = a1;
        }
    }
    }
    __syncthreads();
    if (warp != 0) return;
    float m = -INFINITY;
    for (int n = lane; n < N; n += 32) m = fmaxf(m, s[n]);
    m = warp_max(m);
    float sum = 0.0f;
    for (int n = lane; n < N; n += 32) sum += expf(s[n] - m);
    sum = warp_sum(sum);
    for (int n = lane; n < N; n += 32) {
        const float v = expf(s[n] - m) / sum;
        s[n] = v;
        choice[n] = v + correction[n];
    }
    __syncwarp();
    const int per = N / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
        float v = -INFINITY;
        for (int j = 0; j < per; ++j) v = fmaxf(v, choice[g * per + j]);
        best[g] = v;
    }
    __syncwarp();
    // the (n_groups - keep) weakest runs leave the race, weakest first; ties: the higher index leaves
    for (int out = 0; out < n_groups - keep; ++out) {
        float v = INFINITY;
        int at = -1;
        for (int g = lane; g < n_groups; g += 32)
            if (best[g] != INFINITY && (best[g] < v || (best[g] == v && g > at))) {
                v = best[g];
                at = g;
            }
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, offset);
            const int oat = __shfl_xor_sync(0xffffffffu, at, offset);
            if (oat >= 0 && (at < 0 || ov < v || (ov == v && oat > at))) {
                v = ov;
                at = oat;
            }
        }
        if (at < 0) break;
        __syncwarp();
        if (lane == 0) best[at] = INFINITY;        // marks a run that is out
        for (int j = lane; j < per; j += 32) choice[at * per + j] = -INFINITY;
        __syncwarp();
    }
    // the `top` largest choice values, largest first; ties: the lower index
    for (int slot = 0; slot < top; ++slot) {
        float v = -INFINITY;
        int at = -1;
        for (int n = lane; n < N; n += 32)
            if (choice[n] > v || at < 0) {
                if (choice[n] > v || at < 0) {
                    v = choice[n];
                    at = n;
                }
            }
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, offset);
            const int oat = __shfl_xor_sync(0xffffffffu, at, offset);
            if (oat >= 0 && (at < 0 || ov > v || (ov == v && oat < at))) {
                v = ov;
                at = oat;
            }
        }
        __syncwarp();
        if (lane == 0) {
            ids[(size_t)t * top + slot] = at;
            weights[(size_t)t * top + slot] = s[at];
            choice[at] = -INFINITY;
        }
        __syncwarp();
    }
}

// A router that is a table: token id -> its `top` experts, each with weight 1 / top.
__global__ void __launch_bounds__(256)
moe_route_table_kernel(const int* __restrict__ token_ids, const int* __restrict__ table, int vocab, int top, int T,
                       int* __restrict__ ids, float* __restrict__ weights) {
    fwb::pdl_entry();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * top) return;
    const int t = i / top, slot = i - t * top;
    int token = token_ids[t];
    token = token < 0 ? 0 : (token >= vocab ? vocab - 1 : token);   // (the embedding flags such an id)
    ids[i] = table[(size_t)token * top + slot];
    weights[i] = 1.0f / (float)top;
}

// One block.  ids: [A] router outputs of the pairs (A = tokens * top).  Writes
//   offsets[E + 1]   first row of every expert among the sorted rows
//   row_token[A]     token of every sorted row
//   pair_row[A]      sorted row of every pair (-1: an identity expert)
//   tiles[0]         number of row tiles (of tile_rows rows at most, none across two experts);
//                    tiles[1 + 2 i], tiles[2 + 2 i]: expert and first row of tile i
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int A, int top, int E, int tile_rows, int* __restrict__ offsets,
                int* __restrict__ row_token, int* __restrict__ pair_row, int* __restrict__ tiles) {
    fwb::pdl_entry();
    extern __shared__ int counts[];               // [E] counts, then [E] cursors
    int* cursor = counts + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = ids[a];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, n_tiles = 0;
        for (int e = 0; e < E; ++e) {
            const int n = counts[e];
            offsets[e] = at;
            cursor[e] = at;
            for (int row = 0; row < n; row += tile_rows) {
                tiles[1 + 2 * n_tiles] = e;
                tiles[2 + 2 * n_tiles] = at + row;
                ++n_tiles;
            }
            at += n;
        }
        offsets[E] = at;
        tiles[0] = n_tiles;
    }
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = ids[a];
        int row = -1;
        if (e >= 0 && e < E) {
            row = atomicAdd(&cursor[e], 1);
            row_token[row] = a / top;
        }
        pair_row[a] = row;
    }
}

__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const uint4* __restrict__ h, const int* __restrict__ row_token, const int* __restrict__ offsets,
                       int E, uint4* __restrict__ out, int pieces) {
    fwb::pdl_entry();
    const int row = blockIdx.x;
    if (row >= offsets[E]) return;            // rows behind the last expert's belong to nobody
    const uint4* src = h + (size_t)row_token[row] * pieces;
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) out[(size_t)row * pieces + i] = src[i];
}

// FORM 1: out[row][f] = act(x . gate_f) * (x . up_f), w: [E][2F][K] (gate rows, then up rows), N = F.
// FORM 0: out[row][n] = x . w_n, w: [E][N][K], fp32 out.
// x rows: FORM 1 gathers token rows through row_token; FORM 0 reads sorted rows directly.
template <typename TX, typename TW, typename TO, int FORM>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                const int* __restrict__ offsets, const int* __restrict__ row_token, const int* __restrict__ tiles,
                int N, int K, int act, float limit) {
    fwb::pdl_entry();
    const int tile = blockIdx.y;
    if (tile >= tiles[0]) return;
    const int expert = tiles[1 + 2 * tile], row0 = tiles[2 + 2 * tile];
    const int row_end = offsets[expert + 1];
    const int n0 = blockIdx.x * TN;
    __shared__ float xs[TK][TM + 1];
    __shared__ float ws[FORM ? 2 : 1][TK][TN + 1];
    __shared__ int src_row[TM];
    if (threadIdx.x < TM) {
        const int row = row0 + threadIdx.x;
        src_row[threadIdx.x] = row < row_end ? (FORM ? row_token[row] : row) : -1;
    }
    __syncthreads();
    const TW* w_gate = w + (size_t)expert * (FORM ? 2 : 1) * N * K;
    const TW* w_up = w_gate + (size_t)N * K;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;      // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4] = {}, acc2[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int i = threadIdx.x; i < TM * TK; i += 256) {
            const int r = i / TK, k = i - r * TK;
            const int src = src_row[r];
            xs[k][r] = (src >= 0 && k0 + k < K) ? to_f32<TX>(x[(size_t)src * K + k0 + k]) : 0.0f;
        }
        for (int i = threadIdx.x; i < TN * TK; i += 256) {
            const int n = i / TK, k = i - n * TK;
            const bool in = n0 + n < N && k0 + k < K;
            ws[0][k][n] = in ? to_f32<TW>(w_gate[(size_t)(n0 + n) * K + k0 + k]) : 0.0f;
            if (FORM) ws[1][k][n] = in ? to_f32<TW>(w_up[(size_t)(n0 + n) * K + k0 + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b[j] = ws[0][k][tx * 4 + j];
                if (FORM) b2[j] = ws[1][k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (FORM) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + ty * 4 + i;
        if (row >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (FORM) v = gated_f32(act, limit, v, acc2[i][j]);
            out[(size_t)row * N + n] = from_f32<TO>(v);
        }
    }
}

template <typename TH>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const TH* __restrict__ h, const int* __restrict__ pair_row,
                   const int* __restrict__ ids, const float* __restrict__ weights, float* __restrict__ out, int W,
                   int top, int E) {
    fwb::pdl_entry();
    constexpr int MAX_TOP = 64;
    __shared__ int rows[MAX_TOP];                 // the sorted row of every slot; -1: identity; -2: nothing
    __shared__ float wts[MAX_TOP];
    const int t = blockIdx.x;
    if (threadIdx.x < top) {
        const int a = t * top + threadIdx.x;
        const int row = pair_row[a];
        rows[threadIdx.x] = row >= 0 ? row : (ids[a] >= E ? -1 : -2);
        wts[threadIdx.x] = weights[a];
    }
    __syncthreads();
    if ((W & 3) == 0 && sizeof(TH) == 4) {
        // rows of 16-byte pieces (the fp32 path's h as well as y)
        const float4* y4 = reinterpret_cast<const float4*>(y);
        const float4* h4 = reinterpret_cast<const float4*>(h);
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int slot = 0; slot < top; ++slot) {
                const int row = rows[slot];
                if (row == -2) continue;
                const float4 v = row >= 0 ? y4[(size_t)row * (W / 4) + i] : h4[(size_t)t * (W / 4) + i];
                const float wt = wts[slot];
                acc.x = fmaf(wt, v.x, acc.x), acc.y = fmaf(wt, v.y, acc.y);
                acc.z = fmaf(wt, v.z, acc.z), acc.w = fmaf(wt, v.w, acc.w);
            }
            reinterpret_cast<float4*>(out)[(size_t)t * (W / 4) + i] = acc;
        }
        return;
    }
    if ((W & 3) == 0) {
        const float4* y4 = reinterpret_cast<const float4*>(y);
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int slot = 0; slot < top; ++slot) {
                const int row = rows[slot];
                if (row == -2) continue;
                float4 v;
                if (row >= 0) {
                    v = y4[(size_t)row * (W / 4) + i];
                } else {
                    const TH* own = h + (size_t)t * W + 4 * i;
                    v = make_float4(to_f32<TH>(own[0]), to_f32<TH>(own[1]), to_f32<TH>(own[2]), to_f32<TH>(own[3]));
                }
                const float wt = wts[slot];
                acc.x = fmaf(wt, v.x, acc.x), acc.y = fmaf(wt, v.y, acc.y);
                acc.z = fmaf(wt, v.z, acc.z), acc.w = fmaf(wt, v.w, acc.w);
            }
            reinterpret_cast<float4*>(out)[(size_t)t * (W / 4) + i] = acc;
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float acc = 0.0f;
        float own = 0.0f;
        bool have = false;
        for (int slot = 0; slot < top; ++slot) {
            const int row = rows[slot];
            float v = 0.0f;
            if (row >= 0) {
                v = y[(size_t)row * W + i];
            } else if (row == -1) {
                if (!have) {
                    own = to_f32<TH>(h[(size_t)t * W + i]);
                    have = true;
                }
                v = own;
            }
            acc = fmaf(wts[slot], v, acc);
        }
        out[(size_t)t * W + i] = acc;
    }
}

// The weighted sum of a token's expert rows, the weighted RMS norm of that sum and the residual sum in
// one pass: x[t] += w * y / sqrt(mean(y^2) + eps) with y as moe_combine_kernel makes it (same order of
// additions), kept in shared memory between the two passes.
template <typename TH>
__global__ void __launch_bounds__(256)
moe_combine_norm_add_kernel(const float* __restrict__ y, const TH* __restrict__ h, const int* __restrict__ pair_row,
                            const int* __restrict__ ids, const float* __restrict__ weights, float* __restrict__ x,
                            const float* __restrict__ norm_w, float eps, int W, int top, int E,
                            const float* __restrict__ extra) {
    fwb::pdl_entry();
    constexpr int MAX_TOP = 64;
    extern __shared__ float sum_row[];            // [W]
    __shared__ int rows[MAX_TOP];
    __shared__ float wts[MAX_TOP];
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    if (threadIdx.x < top) {
        const int a = t * top + threadIdx.x;
        const int row = pair_row[a];
        rows[threadIdx.x] = row >= 0 ? row : (ids[a] >= E ? -1 : -2);
        wts[threadIdx.x] = weights[a];
    }
    __syncthreads();
    float ss = 0.0f;
    if ((W & 3) == 0) {
        // rows of 16-byte pieces; every element is still its own sum over the slots, in slot order
        const float4* y4 = reinterpret_cast<const float4*>(y);
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
            const TH* mine = h + (size_t)t * W + 4 * i;
            const float4 own = make_float4(to_f32<TH>(mine[0]), to_f32<TH>(mine[1]), to_f32<TH>(mine[2]), to_f32<TH>(mine[3]));
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int slot = 0; slot < top; ++slot) {
                const int row = rows[slot];
                const float4 v = row >= 0 ? y4[(size_t)row * (W / 4) + i] : (row == -1 ? own : make_float4(0.f, 0.f, 0.f, 0.f));
                const float wt = wts[slot];
                acc.x = fmaf(wt, v.x, acc.x), acc.y = fmaf(wt, v.y, acc.y);
                acc.z = fmaf(wt, v.z, acc.z), acc.w = fmaf(wt, v.w, acc.w);
            }
            if (extra) {                               // (what every token gets besides its experts: added last)
                const float4 more = reinterpret_cast<const float4*>(extra)[(size_t)t * (W / 4) + i];
                acc.x += more.x, acc.y += more.y, acc.z += more.z, acc.w += more.w;
            }
            reinterpret_cast<float4*>(sum_row)[i] = acc;
            ss = fmaf(acc.x, acc.x, fmaf(acc.y, acc.y, fmaf(acc.z, acc.z, fmaf(acc.w, acc.w, ss))));
        }
    } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            float acc = 0.0f;
            const float own = to_f32<TH>(h[(size_t)t * W + i]);
            for (int slot = 0; slot < top; ++slot) {
                const int row = rows[slot];
                const float v = row >= 0 ? y[(size_t)row * W + i] : (row == -1 ? own : 0.0f);
                acc = fmaf(wts[slot], v, acc);
            }
            if (extra) acc += extra[(size_t)t * W + i];
            sum_row[i] = acc;
            ss = fmaf(acc, acc, ss);
        }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) x[(size_t)t * W + i] += (sum_row[i] * inv) * norm_w[i];
}

}  // namespace

// h: [T][W] fp32 or bf16; router: [N][W] fp32; correction: [N] fp32; ids, weights: [T][top].
FWB_API int fwb_moe_route(const void* h, int h_bf16, const float* router, const float* correction, int* ids,
                          float* weights, int T, int W, int N, int n_groups, int keep, int top,
                          cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!h || !router || !correction || !ids || !weights) return FWB_BAD_ARGUMENT;
    if (W <= 0 || N <= 0 || n_groups <= 0 || N % n_groups || keep <= 0 || keep > n_groups || top <= 0 ||
        top > keep * (N / n_groups))
        return FWB_BAD_ARGUMENT;
    const int blocks = T;
    // Few tokens (a decode step): a CTA's life is what counts, so K is cut over sixteen warps and every
    // output's weights are in flight at once (8 tokens, 32 outputs of 2,048: 27 -> 11 us).  Many tokens fill
    // the GPU and throughput counts: two outputs a warp at a time, one reduction an output (2,048 tokens:
    // 115 us against 155 the other way).
    const int vec = (W % 4 == 0 && ((uintptr_t)router & 15) == 0 && W >= 512 && T < 256) ? 1 : 0;
    const int threads = vec ? 512 : (N >= 32 ? 512 : (N >= 16 ? 256 : 128));
    const size_t smem = (size_t)(2 * N + n_groups + (vec ? (threads / 32) * N : 0)) * sizeof(float);
    if (smem > 48 * 1024) return FWB_TOO_LARGE;
    if (h_bf16)
        fwb::pdl(moe_route_kernel<__nv_bfloat16>, blocks, threads, smem, stream)(
            (const __nv_bfloat16*)h, router, correction, ids, weights, T, W, N, n_groups, keep, top, vec);
    else
        fwb::pdl(moe_route_kernel<float>, blocks, threads, smem, stream)((const float*)h, router, correction, ids,
                                                                          weights, T, W, N, n_groups, keep, top, vec);
    return fwb_launch_status();
}

// token_ids: [T] int32; table: [vocab][top] int32; ids, weights: [T][top].
FWB_API int fwb_moe_route_table(const int* token_ids, const int* table, int vocab, int top, int T, int* ids,
                                float* weights, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!token_ids || !table || !ids || !weights || vocab <= 0 || top <= 0) return FWB_BAD_ARGUMENT;
    fwb::pdl(moe_route_table_kernel, (T * top + 255) / 256, 256, 0, stream)(token_ids, table, vocab, top, T, ids, weights);
    return fwb_launch_status();
}

// ids: [A]; offsets: [E + 1]; row_token, pair_row: [A]; tiles: [1 + 2 (A / tile_rows + E + 1)].
// tile_rows: rows of a tile of the products that follow (TM = 64 for fwb_moe_gemm).
FWB_API int fwb_moe_sort(const int* ids, int A, int top, int E, int tile_rows, int* offsets, int* row_token,
                         int* pair_row, int* tiles, cudaStream_t stream) {
    if (A <= 0) return FWB_OK;
    if (!ids || !offsets || !row_token || !pair_row || !tiles || top <= 0 || E < 0 || tile_rows <= 0)
        return FWB_BAD_ARGUMENT;
    if (E > 4096) return FWB_TOO_LARGE;
    fwb::pdl(moe_sort_kernel, 1, 1024, (size_t)(2 * E + 1) * sizeof(int), stream)(ids, A, top, E, tile_rows, offsets,
                                                                                  row_token, pair_row, tiles);
    return fwb_launch_status();
}

// out[row] = h[row_token[row]] for the sorted rows (16-byte pieces): the experts' first product then
// reads its rows side by side.  h: [T][W] bf16, W a multiple of 8; out: [A][W].
FWB_API int fwb_moe_gather_rows(const void* h, const int* row_token, const int* offsets, int E, void* out, int A,
                                int W, cudaStream_t stream) {
    if (A <= 0) return FWB_OK;
    if (!h || !row_token || !offsets || !out || W <= 0 || (W & 7)) return FWB_BAD_ARGUMENT;
    fwb::pdl(moe_gather_rows_kernel, A, 128, 0, stream)((const uint4*)h, row_token, offsets, E, (uint4*)out, W / 8);
    return fwb_launch_status();
}

// form 1: x [T][K] (rows gathered by row_token), w [E][2N][K], out [A][N] in the dtype of x.
// form 0: x [A][K] sorted rows, w [E][N][K], out [A][N] fp32.
// x and w are both fp32 or both bf16.  max_tiles: the most tiles the sorted list can hold (the grid).
FWB_API int fwb_moe_gemm(const void* x, const void* w, int bf16, void* out, const int* offsets,
                         const int* row_token, const int* tiles, int max_tiles, int N, int K, int form, int act,
                         float limit, cudaStream_t stream) {
    if (max_tiles <= 0) return FWB_OK;
    if (!x || !w || !out || !offsets || !row_token || !tiles || N <= 0 || K <= 0 || form < 0 || form > 1 ||
        act < 0 || act > 2)
        return FWB_BAD_ARGUMENT;
    if (max_tiles > 65535) return FWB_TOO_LARGE;
    const dim3 grid((N + TN - 1) / TN, max_tiles);
    using bf = __nv_bfloat16;
    if (form == 1 && bf16)
        fwb::pdl(moe_gemm_kernel<bf, bf, bf, 1>, grid, 256, 0, stream)((const bf*)x, (const bf*)w, (bf*)out, offsets,
                                                                       row_token, tiles, N, K, act, limit);
    else if (form == 1)
        fwb::pdl(moe_gemm_kernel<float, float, float, 1>, grid, 256, 0, stream)(
            (const float*)x, (const float*)w, (float*)out, offsets, row_token, tiles, N, K, act, limit);
    else if (bf16)
        fwb::pdl(moe_gemm_kernel<bf, bf, float, 0>, grid, 256, 0, stream)((const bf*)x, (const bf*)w, (float*)out,
                                                                          offsets, row_token, tiles, N, K, act, limit);
    else
        fwb::pdl(moe_gemm_kernel<float, float, float, 0>, grid, 256, 0, stream)(
            (const float*)x, (const float*)w, (float*)out, offsets, row_token, tiles, N, K, act, limit);
    return fwb_launch_status();
}

// y: [A][W] fp32 sorted rows; h: [T][W]; out: [T][W] fp32.
FWB_API int fwb_moe_combine(const float* y, const void* h, int h_bf16, const int* pair_row, const int* ids,
                            const float* weights, float* out, int T, int W, int top, int E, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!y || !h || !pair_row || !ids || !weights || !out || W <= 0 || top <= 0) return FWB_BAD_ARGUMENT;
    if (top > 64) return FWB_TOO_LARGE;
    if (h_bf16)
        fwb::pdl(moe_combine_kernel<__nv_bfloat16>, T, 256, 0, stream)(y, (const __nv_bfloat16*)h, pair_row, ids,
                                                                       weights, out, W, top, E);
    else
        fwb::pdl(moe_combine_kernel<float>, T, 256, 0, stream)(y, (const float*)h, pair_row, ids, weights, out, W,
                                                               top, E);
    return fwb_launch_status();
}

// The same sum (plus row t of `extra`, fp32 [T][W] or null: what every token gets besides its experts), then
// x[t] += norm_w * sum / sqrt(mean(sum^2) + eps) in place (x: [T][W] fp32).
FWB_API int fwb_moe_combine_norm_add(const float* y, const void* h, int h_bf16, const int* pair_row, const int* ids,
                                     const float* weights, float* x, const float* norm_w, float eps, int T, int W,
                                     int top, int E, const float* extra, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!y || !h || !pair_row || !ids || !weights || !x || !norm_w || W <= 0 || top <= 0) return FWB_BAD_ARGUMENT;
    if (top > 64) return FWB_TOO_LARGE;
    const size_t smem = (size_t)W * sizeof(float);
    if (smem > 160 * 1024) return FWB_TOO_LARGE;
    if (h_bf16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(moe_combine_norm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fwb::pdl(moe_combine_norm_add_kernel<__nv_bfloat16>, T, 256, smem, stream)(
            y, (const __nv_bfloat16*)h, pair_row, ids, weights, x, norm_w, eps, W, top, E, extra);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(moe_combine_norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fwb::pdl(moe_combine_norm_add_kernel<float>, T, 256, smem, stream)(y, (const float*)h, pair_row, ids, weights, x,
                                                                           norm_w, eps, W, top, E, extra);
    }
    return fwb_launch_status();
}

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


// ---------------------------------------------------------------------------------------------------
// The same recurrence over portions of prompts, 64 tokens at a time on tensor cores (the serving path in
// bfloat16).  With S the state in front of a run of n tokens and g the head's decay, token i of the run
// (counted from 0) reads
//
//   o_i = g^(i+1) S^T q_i + sum_{j <= i} g^(i-j) (q_i . k_j) v_j
//
// and the run leaves  S' = g^n S + sum_j g^(n-1-j) k_j v_j^T.  One block owns 32 columns of one head's
// state for one piece of a segment and walks its runs in order; a warp owns 16 tokens of the run and 16 columns.  q, k and v enter
// the products as bfloat16 (silu of the fp32 projection, rounded once); everything else -- the state, the
// powers of the decay, the decayed scores -- is fp32, and wherever an fp32 quantity is an operand of a
// tensor-core product (the state in q.S, the decayed scores in P.V, the decayed values in k v^T) it enters as
// the sum of two bfloat16 numbers (the value rounded, and what the rounding left), two products into one
// fp32 accumulator, so that no more than about 2^-17 of it is lost.
//
// A long segment is cut into pieces of `piece_len` tokens (a multiple of RUN) that run side by side: a first
// launch sums what each piece alone adds to the state (from zero), a small kernel chains those sums into
// the state in front of every piece, and the main launch then walks every piece from its own start.  Only
// a segment's last piece writes the slot.  Segments of one piece skip the first two launches' work.
constexpr int RUN = 64;        // tokens per run
constexpr int CT = 32;         // state columns per block
constexpr int PAD = 8;         // bf16 entries behind every shared row (rows then start 4 banks apart)
constexpr int SF = CT + 4;     // fp32 entries per row of the state's master copy
constexpr int THREADS = 256;   // eight warps: four bands of 16 tokens by two halves of the columns

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ld32(const __nv_bfloat16* at) { return *reinterpret_cast<const uint32_t*>(at); }
// x = hi + lo with hi = bf16(x): the two halves of an fp32 operand
__device__ __forceinline__ void split_bf16(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(x);
    lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}
__device__ __forceinline__ void split_pair(float x, float y, uint32_t& hi, uint32_t& lo) {
    __nv_bfloat16 xh, xl, yh, yl;
    split_bf16(x, xh, xl);
    split_bf16(y, yh, yl);
    __nv_bfloat162 h2(xh, yh), l2(xl, yl);
    hi = *reinterpret_cast<uint32_t*>(&h2);
    lo = *reinterpret_cast<uint32_t*>(&l2);
}
__device__ __forceinline__ float silu_quick(float x) { return x * __frcp_rn(1.0f + __expf(-x)); }

// four 8x8 tiles of bfloat16, each transposed on the way: lane l gives the address of row l % 8 of tile l / 8
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const __nv_bfloat16* row) {
    const uint32_t at = (uint32_t)__cvta_generic_to_shared(row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(at));
}
// four consecutive floats of which `left` exist (VEC: one 16-byte load; the caller has checked the alignment)
template <bool VEC>
__device__ __forceinline__ float4 take4(const float* at, int left) {
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (left <= 0) return v;
    if (VEC) return *reinterpret_cast<const float4*>(at);
    v.x = at[0];
    if (left > 1) v.y = at[1];
    if (left > 2) v.z = at[2];
    if (left > 3) v.w = at[3];
    return v;
}
__device__ __forceinline__ float4 silu4(float4 v) {
    return make_float4(silu_quick(v.x), silu_quick(v.y), silu_quick(v.z), silu_quick(v.w));
}
__device__ __forceinline__ uint2 pack4(float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    return make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

// SUMS: the first launch (what a piece adds to a zero state, written to `scratch`; no read-out).
// Shared rows are [token][channel] throughout; the products that want them the other way round (keys as
// rows of k v^T, values as columns of P.V) take them through transposing ldmatrix loads.  The decay of the
// state's update rides on the values: S' = g^n S + sum_j k_j (g^(n-1-j) v_j)^T, so the keys enter exactly.
template <bool SUMS, bool VEC>
__global__ void __launch_bounds__(THREADS, 2)
decay_runs_kernel(const float* __restrict__ p, long long row_stride, int q_col, int k_col, int v_col, int act_silu,
                  const float* __restrict__ decay, float* __restrict__ state, long long slot_stride,
                  const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                  const int* __restrict__ piece_seg, const int* __restrict__ piece_tok0, int piece_len,
                  float* __restrict__ scratch, float* __restrict__ o, int H, int d, int e, int DP) {
    fwb::pdl_entry();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int QS = DP + PAD;                           // entries per row of the [token][channel] arrays
    constexpr int VS = CT + PAD;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [RUN][QS]
    __nv_bfloat16* Ks = Qs + RUN * QS;                                  // [RUN][QS]
    __nv_bfloat16* Vs = Ks + RUN * QS;                                  // [RUN][VS]  values
    __nv_bfloat16* Vdhi = Vs + RUN * VS;                                // [RUN][VS]  values times g^(n-1-token)
    __nv_bfloat16* Vdlo = Vdhi + RUN * VS;
    __nv_bfloat16* SThi = Vdlo + RUN * VS;                              // [CT][QS]   the state, by column
    __nv_bfloat16* STlo = SThi + CT * QS;
    float* Sf = reinterpret_cast<float*>(STlo + CT * QS);               // [DP][SF]   the state itself
    float* pw = Sf + DP * SF;                                           // [RUN + 1]  powers of the decay

    const int piece = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * CT;
    const int seg = piece_seg[piece], first = piece_tok0[piece], seg_end = seg_start[seg + 1];
    const int last = first + piece_len < seg_end ? first + piece_len : seg_end;
    const bool head = first == seg_start[seg], tail = last == seg_end;
    if (SUMS && tail) return;                          // nothing follows this piece: its sum is not needed
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int dp16 = DP >> 4, d4 = DP >> 2;
    const size_t head_at = (size_t)h * d * e;
    float* mine = state + (size_t)seg_slot[seg] * slot_stride + head_at;
    float* held = scratch ? scratch + (size_t)piece * H * d * e + head_at : nullptr;
    // the state in front of the piece: the slot's for a segment of one piece, else what the chain left (also
    // for a first piece, since the last piece of its segment writes the slot in the same launch)
    const float* front = SUMS ? nullptr : (head && tail ? mine : held);
    float* behind = SUMS ? held : (tail ? mine : nullptr);

    for (int i = tid; i <= RUN; i += blockDim.x) pw[i] = (float)pow((double)decay[h], (double)i);
    for (int i = tid; i < DP * CT; i += blockDim.x) {
        const int r = i / CT, c = i - r * CT;
        Sf[r * SF + c] = (front && r < d && e0 + c < e) ? front[(size_t)r * e + e0 + c] : 0.0f;
    }

    for (int t0 = first; t0 < last; t0 += RUN) {
        const int n = last - t0 < RUN ? last - t0 : RUN;
        __syncthreads();                                   // the run before is done with the shared rows
        // q and k: four channels a thread and four such groups in flight
        for (int base = tid; base < RUN * d4; base += 4 * THREADS) {
            float4 qv[4], kv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * THREADS, tok = i / d4, r = (i - tok * d4) << 2;
                const int left = (i < RUN * d4 && tok < n) ? d - r : 0;
                const float* src = p + (size_t)(t0 + tok) * row_stride + (size_t)h * d + r;
                qv[u] = SUMS ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : take4<VEC>(src + q_col, left);
                kv[u] = take4<VEC>(src + k_col, left);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * THREADS, tok = i / d4, r = (i - tok * d4) << 2;
                if (i >= RUN * d4) break;
                if (!SUMS) *reinterpret_cast<uint2*>(Qs + tok * QS + r) = pack4(act_silu ? silu4(qv[u]) : qv[u]);
                *reinterpret_cast<uint2*>(Ks + tok * QS + r) = pack4(act_silu ? silu4(kv[u]) : kv[u]);
            }
        }
        {   // v: the rounded value, and the rounded value times g^(n-1-token) in two halves
            float4 vv[RUN * CT / 4 / THREADS];
#pragma unroll
            for (int u = 0; u < RUN * CT / 4 / THREADS; ++u) {
                const int i = tid + u * THREADS, tok = i / (CT / 4), c = (i % (CT / 4)) << 2;
                vv[u] = take4<VEC>(p + (size_t)(t0 + tok) * row_stride + v_col + (size_t)h * e + e0 + c,
                                   tok < n ? e - (e0 + c) : 0);
            }
#pragma unroll
            for (int u = 0; u < RUN * CT / 4 / THREADS; ++u) {
                const int i = tid + u * THREADS, tok = i / (CT / 4), c = (i % (CT / 4)) << 2;
                const uint2 packed = pack4(act_silu ? silu4(vv[u]) : vv[u]);
                if (!SUMS) *reinterpret_cast<uint2*>(Vs + tok * VS + c) = packed;
                const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&packed.x);
                const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&packed.y);
                const float w = tok < n ? pw[n - 1 - tok] : 0.0f;
                uint2 dh, dl;
                split_pair(__low2float(lo2) * w, __high2float(lo2) * w, dh.x, dl.x);
                split_pair(__low2float(hi2) * w, __high2float(hi2) * w, dh.y, dl.y);
                *reinterpret_cast<uint2*>(Vdhi + tok * VS + c) = dh;
                *reinterpret_cast<uint2*>(Vdlo + tok * VS + c) = dl;
            }
        }
        for (int i = tid; !SUMS && i < DP * CT; i += blockDim.x) {
            const int r = i / CT, c = i - r * CT;
            __nv_bfloat16 hi, lo;
            split_bf16(Sf[r * SF + c], hi, lo);
            SThi[c * QS + r] = hi;
            STlo[c * QS + r] = lo;
        }
        __syncthreads();

        // a warp owns 16 tokens of the run (row0 .. row0 + 15) and one half of the block's columns
        const int band = warp & 3, row0 = band * 16, half_at = warp >> 2;
        // the address this lane gives to a transposing load of values: 16 tokens by 16 columns
        const int v_lane = (lane & 15) * VS + ((lane >> 4) << 3);
        if (!SUMS && row0 < n) {
            const __nv_bfloat16* qa = Qs + (row0 + g) * QS + 2 * t;
            float acc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[nt][j] = 0.0f;
            // what the state in front of the run gives: (q . S) g^(i+1)
            for (int ks = 0; ks < dp16; ++ks) {
                uint32_t a[4] = {ld32(qa + ks * 16), ld32(qa + 8 * QS + ks * 16), ld32(qa + ks * 16 + 8),
                                 ld32(qa + 8 * QS + ks * 16 + 8)};
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int at = (half_at * 16 + nt * 8 + g) * QS + ks * 16 + 2 * t;
                    mma_bf16(acc[nt], a, ld32(SThi + at), ld32(SThi + at + 8));
                    mma_bf16(acc[nt], a, ld32(STlo + at), ld32(STlo + at + 8));
                }
            }
            const float up = pw[row0 + g + 1], down = pw[row0 + g + 9];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                acc[nt][0] *= up;
                acc[nt][1] *= up;
                acc[nt][2] *= down;
                acc[nt][3] *= down;
            }
            // the run's own keys, 16 at a time up to this warp's last token: decayed scores, then P.V
            for (int kk = 0; kk <= band; ++kk) {
                float sc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
                for (int ks = 0; ks < dp16; ++ks) {
                    uint32_t a[4] = {ld32(qa + ks * 16), ld32(qa + 8 * QS + ks * 16), ld32(qa + ks * 16 + 8),
                                     ld32(qa + 8 * QS + ks * 16 + 8)};
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int at = (kk * 16 + half * 8 + g) * QS + ks * 16 + 2 * t;
                        mma_bf16(sc[half], a, ld32(Ks + at), ld32(Ks + at + 8));
                    }
                }
                uint32_t ahi[4], alo[4];
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const int i = row0 + g + 8 * rr, j = kk * 16 + half * 8 + 2 * t;
                        const float w0 = j <= i ? sc[half][2 * rr] * pw[i - j] : 0.0f;
                        const float w1 = j + 1 <= i ? sc[half][2 * rr + 1] * pw[i - j - 1] : 0.0f;
                        split_pair(w0, w1, ahi[2 * half + rr], alo[2 * half + rr]);
                    }
                uint32_t b[4];
                ldsm4t(b, Vs + kk * 16 * VS + half_at * 16 + v_lane);
                mma_bf16(acc[0], ahi, b[0], b[1]);
                mma_bf16(acc[0], alo, b[0], b[1]);
                mma_bf16(acc[1], ahi, b[2], b[3]);
                mma_bf16(acc[1], alo, b[2], b[3]);
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = row0 + g + 8 * (j >> 1), c = e0 + half_at * 16 + nt * 8 + 2 * t + (j & 1);
                    if (i < n && c < e) o[(size_t)(t0 + i) * H * e + (size_t)h * e + c] = acc[nt][j];
                }
        }
        // the state behind the run: 16 of its rows at a time, a warp each
        const float shrink = pw[n];
        const int steps = (n + 15) >> 4;
        // this lane's address in a transposing load of keys: 16 tokens by 16 channels
        const int k_lane = ((lane & 7) + ((lane >> 4) << 3)) * QS + (((lane >> 3) & 1) << 3);
        for (int mt = warp; mt < dp16; mt += THREADS / 32) {
            float* srow = Sf + (mt * 16 + g) * SF + 2 * t;
            float acc[CT / 8][4];
#pragma unroll
            for (int nt = 0; nt < CT / 8; ++nt) {
                acc[nt][0] = srow[nt * 8] * shrink;
                acc[nt][1] = srow[nt * 8 + 1] * shrink;
                acc[nt][2] = srow[8 * SF + nt * 8] * shrink;
                acc[nt][3] = srow[8 * SF + nt * 8 + 1] * shrink;
            }
            for (int ks = 0; ks < steps; ++ks) {
                uint32_t a[4];
                ldsm4t(a, Ks + ks * 16 * QS + mt * 16 + k_lane);
#pragma unroll
                for (int np = 0; np < CT / 16; ++np) {
                    uint32_t bh[4], bl[4];
                    ldsm4t(bh, Vdhi + ks * 16 * VS + np * 16 + v_lane);
                    ldsm4t(bl, Vdlo + ks * 16 * VS + np * 16 + v_lane);
                    mma_bf16(acc[2 * np], a, bh[0], bh[1]);
                    mma_bf16(acc[2 * np], a, bl[0], bl[1]);
                    mma_bf16(acc[2 * np + 1], a, bh[2], bh[3]);
                    mma_bf16(acc[2 * np + 1], a, bl[2], bl[3]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < CT / 8; ++nt) {
                srow[nt * 8] = acc[nt][0];
                srow[nt * 8 + 1] = acc[nt][1];
                srow[8 * SF + nt * 8] = acc[nt][2];
                srow[8 * SF + nt * 8 + 1] = acc[nt][3];
            }
        }
    }
    __syncthreads();
    for (int i = tid; behind && i < DP * CT; i += blockDim.x) {
        const int r = i / CT, c = i - r * CT;
        if (r < d && e0 + c < e) behind[(size_t)r * e + e0 + c] = Sf[r * SF + c];
    }
}

// Chains the pieces' sums: walking a segment's pieces in order, every piece's entry of `scratch` (what the
// piece alone adds) is replaced by the state in front of that piece.  One thread per state entry; blocks of
// pieces that are not the first of a segment of several pieces have nothing to do.
__global__ void __launch_bounds__(256)
decay_chain_kernel(const float* __restrict__ decay, const float* __restrict__ state, long long slot_stride,
                   const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                   const int* __restrict__ piece_seg, const int* __restrict__ piece_tok0, int piece_len,
                   float* __restrict__ scratch, int H, int d, int e) {
    fwb::pdl_entry();
    const int piece = blockIdx.x;
    const int seg = piece_seg[piece], first = piece_tok0[piece], seg_end = seg_start[seg + 1];
    if (first != seg_start[seg] || first + piece_len >= seg_end) return;
    const size_t size = (size_t)H * d * e;
    const size_t at = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
    if (at >= size) return;
    const int h = (int)(at / ((size_t)d * e));
    const float shrink = (float)pow((double)decay[h], (double)piece_len);
    float run = state[(size_t)seg_slot[seg] * slot_stride + at];
    for (int c = piece;; ++c) {
        float* cell = scratch + (size_t)c * size + at;
        if (piece_tok0[c] + piece_len >= seg_end) {        // the segment's last piece
            *cell = run;
            break;
        }
        const float sum = *cell;
        *cell = run;
        run = shrink * run + sum;
    }
}

size_t decay_runs_smem(int DP) {
    const size_t QS = DP + PAD, VS = CT + PAD;
    return (2 * RUN * QS + 3 * RUN * VS + 2 * CT * QS) * sizeof(__nv_bfloat16)
           + ((size_t)DP * SF + RUN + 1) * sizeof(float);
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

// The same operation, 64 tokens of a segment at a time on tensor cores: q, k and v enter as bfloat16, the
// state, the decay's powers and every sum stay fp32.  For steps that bring portions of prompts; heads of up
// to 256 channels (FWB_UNSUPPORTED beyond: the token-by-token form takes those).  The segments come cut into
// `P` pieces of at most `piece_len` tokens (a multiple of 64): piece_seg, piece_tok0.  `scratch`: fp32
// [P][H d e], needed when some segment has more than one piece (`chained` != 0), else it may be null.
FWB_API int fwb_decay_runs(const float* p, long long row_stride, int q_col, int k_col, int v_col, int act_silu,
                           const float* decay, float* state, long long slot_stride, const int* seg_start,
                           const int* seg_slot, const int* piece_seg, const int* piece_tok0, int piece_len,
                           int chained, float* scratch, float* o, int T, int S, int P, int H, int d, int e,
                           cudaStream_t stream) {
    if (T <= 0 || S <= 0 || P <= 0) return FWB_OK;
    if (!p || !decay || !state || !seg_start || !seg_slot || !piece_seg || !piece_tok0 || !o) return FWB_BAD_ARGUMENT;
    if (H <= 0 || d <= 0 || e <= 0 || q_col < 0 || k_col < 0 || v_col < 0) return FWB_BAD_ARGUMENT;
    if (piece_len <= 0 || piece_len % RUN != 0 || (chained && !scratch)) return FWB_BAD_ARGUMENT;
    if (row_stride < (long long)H * d || slot_stride < (long long)H * d * e) return FWB_BAD_ARGUMENT;
    if (d > 256) return FWB_UNSUPPORTED;
    const int tiles = (e + CT - 1) / CT;
    const size_t size = (size_t)H * d * e;
    if (H > 65535 || tiles > 65535 || (size + 255) / 256 > 65535) return FWB_TOO_LARGE;
    const int DP = (d + 15) / 16 * 16;
    const size_t smem = decay_runs_smem(DP);
    // 16-byte loads where every group of four channels starts on such a border
    const bool vec = d % 4 == 0 && e % 4 == 0 && row_stride % 4 == 0 && q_col % 4 == 0 && k_col % 4 == 0
                     && v_col % 4 == 0 && reinterpret_cast<uintptr_t>(p) % 16 == 0;
    auto sums = vec ? decay_runs_kernel<true, true> : decay_runs_kernel<true, false>;
    auto walk = vec ? decay_runs_kernel<false, true> : decay_runs_kernel<false, false>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(sums, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(walk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    if (chained) {
        fwb::pdl(sums, dim3(P, H, tiles), THREADS, smem, stream)(
            p, row_stride, q_col, k_col, v_col, act_silu, decay, state, slot_stride, seg_start, seg_slot, piece_seg,
            piece_tok0, piece_len, scratch, o, H, d, e, DP);
        int status = fwb_launch_status();
        if (status != FWB_OK) return status;
        fwb::pdl(decay_chain_kernel, dim3(P, (unsigned)((size + 255) / 256)), 256, 0, stream)(
            decay, state, slot_stride, seg_start, seg_slot, piece_seg, piece_tok0, piece_len, scratch, H, d, e);
        status = fwb_launch_status();
        if (status != FWB_OK) return status;
    }
    fwb::pdl(walk, dim3(P, H, tiles), THREADS, smem, stream)(
        p, row_stride, q_col, k_col, v_col, act_silu, decay, state, slot_stride, seg_start, seg_slot, piece_seg,
        piece_tok0, piece_len, chained ? scratch : nullptr, o, H, d, e, DP);
    return fwb_launch_status();
}

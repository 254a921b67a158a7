// gtb_seq_kernels.cuh -- device side of the layer-list sequence models (include/gten_b200_seq.h).
//
// One pass = R rows (tokens) of S segments; segment s continues slot seg_slot[s] for seg_len[s] rows starting at row seg_row0[s].
// Everything the kernels need to know about a row sits in the device-side PassTables, so a pass is a fixed launch
// sequence whatever the positions are (CUDA-graph replay for decode steps).
//
// Precision: the residual stream, norms, convolution, attention scores and weights, the recurrent state and everything that
// enters the recurrence are fp32 in both compute modes.  OT is the type of matrix-product operands and of the K/V cache:
// __nv_bfloat16 (products on bf16 operands with fp32 accumulation) or float (true fp32, FFMA only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gtb {
namespace seq {

typedef __nv_bfloat16 bf16;

struct SlotState {
    int pos;          // tokens held
    int prev;         // last token fed (-1: none)
    int pending;      // last sampled token: what the next device-driven decode step feeds
    int stopped;      // sampled the end-of-sequence id
};

struct PassTables {
    // per segment
    const int* seg_slot;
    const int* seg_row0;
    const int* seg_len;
    // per row
    const int* row_seg;
    int* tok;          // token ids (host-fed, or written by k_plan from SlotState::pending)
    int* row_pos;      // written by k_plan
    int* row_prev;     // previous token of the row, -1 for a sequence's first token; written by k_plan
    SlotState* slots;
};

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ T cvt(float v);
template <> __device__ __forceinline__ float cvt<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 cvt<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// sum over the block; every thread gets the result.  red: 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // red may still be read from a previous call
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// dot of a shared-memory fp32 vector with a cached key row; `vec`: the row is 16-byte aligned and n a multiple of 8 (4 for fp32)
__device__ __forceinline__ float key_dot(const float* __restrict__ q, const bf16* __restrict__ k, int n, bool vec) {
    float s = 0.0f;
    if (vec) {
        for (int i = 0; i < n; i += 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(k + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                s = fmaf(q[i + 2 * j], __uint_as_float(w[j] << 16), s);
                s = fmaf(q[i + 2 * j + 1], __uint_as_float(w[j] & 0xffff0000u), s);
            }
        }
    } else {
        for (int i = 0; i < n; i++) s = fmaf(q[i], __bfloat162float(k[i]), s);
    }
    return s;
}
__device__ __forceinline__ float key_dot(const float* __restrict__ q, const float* __restrict__ k, int n, bool vec) {
    float s = 0.0f;
    if (vec) {
        for (int i = 0; i < n; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(k + i);
            s = fmaf(q[i], v.x, s); s = fmaf(q[i + 1], v.y, s); s = fmaf(q[i + 2], v.z, s); s = fmaf(q[i + 3], v.w, s);
        }
    } else {
        for (int i = 0; i < n; i++) s = fmaf(q[i], k[i], s);
    }
    return s;
}
__device__ __forceinline__ float gelu_tanh(float z) {
    const float c = 0.7978845608028654f;      // sqrt(2/pi)
    return 0.5f * z * (1.0f + tanhf(c * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------------------------------------ plan / commit
// row tables of a pass from the slots' device-side state.  from_pending: rows take their token from the slot (decode loop).
__global__ void k_plan(PassTables t, int R, int from_pending) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    const int s = t.row_seg[r], slot = t.seg_slot[s], row0 = t.seg_row0[s];
    const SlotState st = t.slots[slot];
    if (from_pending) t.tok[r] = st.pending;
    const int pos = st.pos + (r - row0);
    t.row_pos[r] = pos;
    t.row_prev[r] = (r > row0) ? (from_pending ? st.pending : t.tok[r - 1]) : (pos == 0 ? -1 : st.prev);
}
__global__ void k_commit(PassTables t, int S) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= S) return;
    SlotState& st = t.slots[t.seg_slot[s]];
    if (st.stopped) return;
    st.pos += t.seg_len[s];
    st.prev = t.tok[t.seg_row0[s] + t.seg_len[s] - 1];
}

// ------------------------------------------------------------------------------------------------ embedding
// x = scale * embed[tok] (+ bigram[(prev * mul_prev + tok * mul_cur) mod buckets], row `buckets` for a sequence's first token); x0 = x;
// op (optional): x again as the operand of the first matrix product, for models whose first layer reads the stream itself
template <typename OT>
__global__ void k_embed(PassTables t, const bf16* __restrict__ embed, const bf16* __restrict__ bigram, int buckets, int mul_prev,
                        int mul_cur, int width, float scale, float* __restrict__ x, float* __restrict__ x0, OT* __restrict__ op, int ld_op) {
    const int r = blockIdx.x;
    const int tok = t.tok[r], prev = t.row_prev[r];
    long long row = buckets;
    if (prev >= 0) row = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = __bfloat162float(embed[(size_t)tok * width + c]) * scale;
        if (buckets > 0) v += __bfloat162float(bigram[(size_t)row * width + c]);
        x[(size_t)r * width + c] = v;
        if (x0) x0[(size_t)r * width + c] = v;
        if (op) op[(size_t)r * ld_op + c] = cvt<OT>(v);
    }
}

// ------------------------------------------------------------------------------------------------ norm with one gain
// h = x / sqrt(mean(x^2) + eps) * g, g a single number.  rows: optional gather (row index per output row).
template <typename OUT>
__global__ void k_rmsnorm_scalar(const float* __restrict__ x, int width, float eps, const float* __restrict__ g, const int* __restrict__ rows,
                                 OUT* __restrict__ out, int ld_out) {
    __shared__ float red[33];
    const int o = blockIdx.x, r = rows ? rows[o] : o;
    const float* xr = x + (size_t)r * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = xr[c]; ss += v * v; }
    ss = block_sum(ss, red);
    const float sc = (1.0f / sqrtf(ss / (float)width + eps)) * g[0];
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)o * ld_out + c] = cvt<OUT>(xr[c] * sc);
}

// ------------------------------------------------------------------------------------------------ input convolution
// out_a = h + conv_a(h), out_b = h + conv_b(h); conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j).  Rows before the segment come from the
// slot's history `tail` [n_slots][taps - 1][width] (zeros after a reset = zeros before the sequence's start).
template <typename OT>
__global__ void k_canon(PassTables t, const float* __restrict__ h, int width, int taps, const bf16* __restrict__ wa, const bf16* __restrict__ wb,
                        const float* __restrict__ tail, OT* __restrict__ out_a, OT* __restrict__ out_b, int ld_out) {
    const int r = blockIdx.x;
    const int s = t.row_seg[r], row0 = t.seg_row0[s], slot = t.seg_slot[s];
    const float* tl = tail + (size_t)slot * (taps - 1) * width;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
        float a = 0.0f, b = 0.0f;
        for (int j = 0; j < taps; j++) {
            const int src = r - (taps - 1) + j;
            const float v = (src >= row0) ? h[(size_t)src * width + c] : tl[(size_t)(src - row0 + taps - 1) * width + c];
            a += __bfloat162float(wa[(size_t)c * taps + j]) * v;
            if (wb) b += __bfloat162float(wb[(size_t)c * taps + j]) * v;
        }
        const float hc = h[(size_t)r * width + c];
        out_a[(size_t)r * ld_out + c] = cvt<OT>(hc + a);
        if (out_b) out_b[(size_t)r * ld_out + c] = cvt<OT>(hc + b);
    }
}
// Norm and convolution in one kernel: a CTA owns row r; its warps first compute 1 / rms of the `taps` rows the convolution reaches
// back to (those inside the segment), then every thread forms h of its channels for those rows on the fly.  h of the row itself
// is also written out (the history update reads it).
template <typename OT>
__global__ void __launch_bounds__(256) k_norm_canon(PassTables t, const float* __restrict__ x, int width, float eps, const float* __restrict__ g, int taps,
                                                    const bf16* __restrict__ wa, const bf16* __restrict__ wb, const float* __restrict__ tail,
                                                    float* __restrict__ h, OT* __restrict__ out_a, OT* __restrict__ out_b, int ld_out) {
    __shared__ float inv[32];
    const int r = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int s = t.row_seg[r], row0 = t.seg_row0[s], slot = t.seg_slot[s];
    const float gain = g[0];
    for (int j = wid; j < taps; j += nw) {
        const int src = r - (taps - 1) + j;
        if (src < row0) continue;                          // warp-uniform
        const float* xr = x + (size_t)src * width;
        float ss = 0.0f;
        for (int c = lane; c < width; c += 32) { const float v = xr[c]; ss += v * v; }
        ss = warp_sum(ss);
        if (lane == 0) inv[j] = (1.0f / sqrtf(ss / (float)width + eps)) * gain;
    }
    __syncthreads();
    const float* tl = tail + (size_t)slot * (taps - 1) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float a = 0.0f, b = 0.0f, hc = 0.0f;
        for (int j = 0; j < taps; j++) {
            const int src = r - (taps - 1) + j;
            const float v = (src >= row0) ? x[(size_t)src * width + c] * inv[j] : tl[(size_t)(src - row0 + taps - 1) * width + c];
            a += __bfloat162float(wa[(size_t)c * taps + j]) * v;
            if (wb) b += __bfloat162float(wb[(size_t)c * taps + j]) * v;
            hc = v;
        }
        h[(size_t)r * width + c] = hc;
        out_a[(size_t)r * ld_out + c] = cvt<OT>(hc + a);
        if (out_b) out_b[(size_t)r * ld_out + c] = cvt<OT>(hc + b);
    }
}
// no convolution configured: the operand is h itself
template <typename OT>
__global__ void k_copy_operand(const float* __restrict__ h, int width, OT* __restrict__ out_a, OT* __restrict__ out_b, int ld_out) {
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const OT v = cvt<OT>(h[(size_t)r * width + c]);
        out_a[(size_t)r * ld_out + c] = v;
        if (out_b) out_b[(size_t)r * ld_out + c] = v;
    }
}
// history <- the last taps - 1 values of h of each segment's sequence.  One thread per channel walks k upwards: entry k is written
// after every entry it is read for (k + len > k).
__global__ void k_canon_tail(PassTables t, const float* __restrict__ h, int width, int taps, float* __restrict__ tail) {
    const int s = blockIdx.x;
    const int row0 = t.seg_row0[s], len = t.seg_len[s], slot = t.seg_slot[s];
    if (t.slots[slot].stopped) return;
    float* tl = tail + (size_t)slot * (taps - 1) * width;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x)
        for (int k = 0; k < taps - 1; k++) {
            const int off = len - (taps - 1) + k;          // offset inside the segment of the row that lands in entry k
            tl[(size_t)k * width + c] = (off >= 0) ? h[(size_t)(row0 + off) * width + c] : tl[(size_t)(k + len) * width + c];
        }
}

// ------------------------------------------------------------------------------------------------ matrix product (SIMT)
// C[M][N] = (acc ? C : 0) + bias + A[M][K] . W[N][K]^T with fp32 accumulation on FFMA: the true-fp32 product, and the bf16 product of
// passes too small for the tensor-core kernel.  K is a multiple of 16 (operands are zero-padded to a multiple of 64).
constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16;
template <typename AT>
__global__ void __launch_bounds__(256) k_gemm_simt(const AT* __restrict__ A, int lda, const bf16* __restrict__ W, int ldw, float* __restrict__ C, int ldc,
                                                   int M, int N, int K, const float* __restrict__ bias, int accumulate) {
    __shared__ float sa[SG_BK][SG_BM + 4];
    __shared__ float sw[SG_BK][SG_BN + 4];
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = threadIdx.x + i * 256;          // 64 rows x 16 k
            const int rr = e >> 4, kk = e & 15;
            sa[kk][rr] = (m0 + rr < M) ? ldf<AT>(A + (size_t)(m0 + rr) * lda + k0 + kk) : 0.0f;
            sw[kk][rr] = (n0 + rr < N) ? __bfloat162float(W[(size_t)(n0 + rr) * ldw + k0 + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; kk++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = sa[kk][ty * 4 + i]; w[i] = sw[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            if (accumulate) v += C[(size_t)m * ldc + n];
            C[(size_t)m * ldc + n] = v;
        }
    }
}

// Few rows (decode): the weight matrix is streamed exactly once for all M <= MR rows.  A CTA owns NC output columns and its 8 warps
// split K; a lane takes 8 consecutive k per step (one 16-byte weight load per column, all of them issued before the first use; the
// rows of A come through L1 as 16-byte loads too), the lanes' partial sums meet in a shuffle reduction and the warps' in shared memory.
template <typename AT> __device__ __forceinline__ void load8(const AT* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float (&v)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <typename AT, int MR, int NC>
__global__ void __launch_bounds__(256) k_gemv_rows(const AT* __restrict__ A, int lda, const bf16* __restrict__ W, int ldw, float* __restrict__ C, int ldc,
                                                   int M, int N, int K, const float* __restrict__ bias, int accumulate) {
    __shared__ float red[8][MR * NC];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n0 = blockIdx.x * NC;
    float acc[MR][NC];
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
        for (int c = 0; c < NC; c++) acc[m][c] = 0.0f;
    // K % 64 == 0 and every row is 16-byte aligned: steps of 8 elements never straddle the end
#pragma unroll 2
    for (int k = (warp * 32 + lane) * 8; k < K; k += 2048) {
        uint4 wv[NC];
#pragma unroll
        for (int c = 0; c < NC; c++)
            wv[c] = (n0 + c < N) ? __ldg(reinterpret_cast<const uint4*>(W + (size_t)(n0 + c) * ldw + k)) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int m = 0; m < MR; m++) {
            if (m >= M) break;
            float av[8];
            load8<AT>(A + (size_t)m * lda + k, av);
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const uint32_t ww[4] = {wv[c].x, wv[c].y, wv[c].z, wv[c].w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    acc[m][c] = fmaf(av[2 * i], __uint_as_float(ww[i] << 16), acc[m][c]);
                    acc[m][c] = fmaf(av[2 * i + 1], __uint_as_float(ww[i] & 0xffff0000u), acc[m][c]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
        for (int c = 0; c < NC; c++) {
            const float v = warp_sum(acc[m][c]);
            if (lane == 0) red[warp][m * NC + c] = v;
        }
    __syncthreads();
    if (threadIdx.x < MR * NC) {
        const int m = threadIdx.x / NC, c = threadIdx.x % NC;
        if (m < M && n0 + c < N) {
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; w++) o += red[w][threadIdx.x];
            if (bias) o += bias[n0 + c];
            if (accumulate) o += C[(size_t)m * ldc + n0 + c];
            C[(size_t)m * ldc + n0 + c] = o;
        }
    }
}

// ------------------------------------------------------------------------------------------------ sigmoid attention
struct AttnBranch {
    int heads, kv_heads, dim, vdim;
    float scale, eps, out_scale;
    int qk_norm;
    int q_off, k_off, v_off;     // column offsets of q | k | v in the projection buffer
    int a_off;                   // column offset of this branch's output in the out-projection operand
    const float* pb;             // [heads] or null
    int max_ctx;
};
// q (and k) to unit RMS per head in place; k, v of every row appended to the slot's cache [n_slots][max_ctx][kv_heads * dim|vdim].
template <typename OT>
__global__ void k_attn_prep(PassTables t, AttnBranch b, float* __restrict__ P, int ldp, OT* __restrict__ kc, OT* __restrict__ vc) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int slot = t.seg_slot[t.row_seg[r]], pos = t.row_pos[r];
    float* p = P + (size_t)r * ldp;
    const size_t crow = (size_t)slot * b.max_ctx + pos;
    for (int u = blockIdx.y * nw + wid; u < b.heads + 2 * b.kv_heads; u += gridDim.y * nw) {
        if (u < b.heads + b.kv_heads) {
            const bool is_q = u < b.heads;
            float* v = p + (is_q ? b.q_off + u * b.dim : b.k_off + (u - b.heads) * b.dim);
            float sc = 1.0f;
            if (b.qk_norm) {
                float ss = 0.0f;
                for (int i = lane; i < b.dim; i += 32) ss += v[i] * v[i];
                ss = warp_sum(ss);
                sc = 1.0f / sqrtf(ss / (float)b.dim + b.eps);
            }
            if (is_q) { for (int i = lane; i < b.dim; i += 32) v[i] *= sc; }
            else {
                OT* dst = kc + crow * (size_t)(b.kv_heads * b.dim) + (size_t)(u - b.heads) * b.dim;
                for (int i = lane; i < b.dim; i += 32) dst[i] = cvt<OT>(v[i] * sc);
            }
        } else {
            const int g = u - b.heads - b.kv_heads;
            const float* v = p + b.v_off + g * b.vdim;
            OT* dst = vc + crow * (size_t)(b.kv_heads * b.vdim) + (size_t)g * b.vdim;
            for (int i = lane; i < b.vdim; i += 32) dst[i] = cvt<OT>(v[i]);
        }
    }
}
// one CTA per (row, query head): out = out_scale * sum_{j <= pos} sigmoid(scale q.k_j + pb) v_j, keys in tiles of blockDim.x.
// A thread scores one key of the tile, then the threads turn to the value channels.  vdim <= 4 * blockDim.x.
template <typename OT>
__global__ void __launch_bounds__(128) k_sigattn(PassTables t, AttnBranch b, const float* __restrict__ P, int ldp, const OT* __restrict__ kc,
                                                 const OT* __restrict__ vc, OT* __restrict__ out, int ld_out) {
    extern __shared__ float sm[];
    float* sq = sm;                 // [dim]
    float* swt = sm + b.dim;        // [blockDim.x]
    const int r = blockIdx.x, h = blockIdx.y, g = h / (b.heads / b.kv_heads);
    const int slot = t.seg_slot[t.row_seg[r]], pos = t.row_pos[r];
    const float* q = P + (size_t)r * ldp + b.q_off + h * b.dim;
    for (int i = threadIdx.x; i < b.dim; i += blockDim.x) sq[i] = q[i];
    const float bias = b.pb ? b.pb[h] : 0.0f;
    const size_t kld = (size_t)b.kv_heads * b.dim, vld = (size_t)b.kv_heads * b.vdim;
    const OT* kbase = kc + (size_t)slot * b.max_ctx * kld + (size_t)g * b.dim;
    const OT* vbase = vc + (size_t)slot * b.max_ctx * vld + (size_t)g * b.vdim;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const bool kvec = b.dim % 8 == 0;            // rows of the cache start on 16-byte boundaries then
    __syncthreads();
    for (int j0 = 0; j0 <= pos; j0 += blockDim.x) {
        const int j = j0 + threadIdx.x;
        float w = 0.0f;
        if (j <= pos) {
            w = sigmoidf_(key_dot(sq, kbase + (size_t)j * kld, b.dim, kvec) * b.scale + bias);
        }
        swt[threadIdx.x] = w;
        __syncthreads();
        const int nj = min((int)blockDim.x, pos + 1 - j0);
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            const int c = threadIdx.x + cc * blockDim.x;
            if (c < b.vdim) {
                float a = acc[cc];
                const OT* vr = vbase + (size_t)j0 * vld + c;
                for (int jj = 0; jj < nj; jj++) a = fmaf(swt[jj], ldf<OT>(vr + (size_t)jj * vld), a);
                acc[cc] = a;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
        const int c = threadIdx.x + cc * blockDim.x;
        if (c < b.vdim) out[(size_t)r * ld_out + b.a_off + h * b.vdim + c] = cvt<OT>(acc[cc] * b.out_scale);
    }
}

// Decode rows at long contexts: the keys of a (row, head) are split over gridDim.z CTAs; each writes its partial sum to
// part [split][R][heads * vdim] (zeros for an empty range), k_sigattn_join adds the splits in order.  Nothing is normalised over keys,
// so the partial sums simply add.
template <typename OT>
__global__ void __launch_bounds__(128) k_sigattn_split(PassTables t, AttnBranch b, const float* __restrict__ P, int ldp, const OT* __restrict__ kc,
                                                       const OT* __restrict__ vc, float* __restrict__ part, int R) {
    extern __shared__ float sm[];
    float* sq = sm;
    float* swt = sm + b.dim;
    const int r = blockIdx.x, h = blockIdx.y, g = h / (b.heads / b.kv_heads);
    const int slot = t.seg_slot[t.row_seg[r]], pos = t.row_pos[r];
    const int per = ((pos + 1 + (int)gridDim.z - 1) / (int)gridDim.z + 127) / 128 * 128;
    const int lo = blockIdx.z * per, hi = min(pos + 1, lo + per);
    const float* q = P + (size_t)r * ldp + b.q_off + h * b.dim;
    for (int i = threadIdx.x; i < b.dim; i += blockDim.x) sq[i] = q[i];
    const float bias = b.pb ? b.pb[h] : 0.0f;
    const size_t kld = (size_t)b.kv_heads * b.dim, vld = (size_t)b.kv_heads * b.vdim;
    const OT* kbase = kc + (size_t)slot * b.max_ctx * kld + (size_t)g * b.dim;
    const OT* vbase = vc + (size_t)slot * b.max_ctx * vld + (size_t)g * b.vdim;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const int kg = b.vdim <= 32 ? 4 : b.vdim <= 64 ? 2 : 1, cw = 128 / kg;      // key groups of the value phase and their width
    const bool kvec = b.dim % 8 == 0;            // rows of the cache start on 16-byte boundaries then
    __syncthreads();
    for (int j0 = lo; j0 < hi; j0 += blockDim.x) {
        const int j = j0 + threadIdx.x;
        float w = 0.0f;
        if (j < hi) {
            w = sigmoidf_(key_dot(sq, kbase + (size_t)j * kld, b.dim, kvec) * b.scale + bias);
        }
        swt[threadIdx.x] = w;
        __syncthreads();
        const int nj = min((int)blockDim.x, hi - j0);
        if (kg > 1) {                                    // narrow heads: kg thread groups take every kg-th key of the tile
            const int c = threadIdx.x % cw, grp = threadIdx.x / cw;
            if (c < b.vdim) {
                float a = acc[0];
                const OT* vr = vbase + (size_t)j0 * vld + c;
#pragma unroll 4
                for (int jj = grp; jj < nj; jj += kg) a = fmaf(swt[jj], ldf<OT>(vr + (size_t)jj * vld), a);
                acc[0] = a;
            }
        } else {
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                const int c = threadIdx.x + cc * blockDim.x;
                if (c < b.vdim) {
                    float a = acc[cc];
                    const OT* vr = vbase + (size_t)j0 * vld + c;
                    for (int jj = 0; jj < nj; jj++) a = fmaf(swt[jj], ldf<OT>(vr + (size_t)jj * vld), a);
                    acc[cc] = a;
                }
            }
        }
        __syncthreads();
    }
    if (kg > 1) {                                        // the groups' partial sums meet in shared memory, group 0 stores
        swt[threadIdx.x] = acc[0];
        __syncthreads();
        const int c = threadIdx.x;
        if (c < b.vdim) {
            float a = 0.0f;
            for (int q = 0; q < kg; q++) a += swt[q * cw + c];
            part[((size_t)blockIdx.z * R + r) * (b.heads * b.vdim) + h * b.vdim + c] = a;
        }
        return;
    }
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
        const int c = threadIdx.x + cc * blockDim.x;
        if (c < b.vdim) part[((size_t)blockIdx.z * R + r) * (b.heads * b.vdim) + h * b.vdim + c] = acc[cc];
    }
}
template <typename OT>
__global__ void k_sigattn_join(AttnBranch b, const float* __restrict__ part, int R, int splits, OT* __restrict__ out, int ld_out) {
    const int r = blockIdx.x, n = b.heads * b.vdim;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
        float a = 0.0f;
        for (int k = 0; k < splits; k++) a += part[((size_t)k * R + r) * n + c];
        out[(size_t)r * ld_out + b.a_off + c] = cvt<OT>(a * b.out_scale);
    }
}

// ------------------------------------------------------------------------------------------------ retention
struct RetBranch {
    int heads, dim, vdim;
    float scale, eps, out_scale;
    int rot_dims;
    const float* inv_freq;       // [rot_dims / 2]
    const float* decay;          // [heads]
    int out_norm, gated;
    int q_off, k_off, v_off, g_off;
    int a_off;
};
// One CTA per (segment, head, slice of value channels) walks the segment's rows in order: S <- decay S + k v^T, o = S^T q.  The columns of
// the state are independent of each other, so a CTA keeps only its slice [dim][vs] in shared memory for the walk (thread x = value
// channel; row groups of the state are split over the y dimension of the CTA and summed through shared memory); it starts from and
// returns to the slot's state in HBM.  q and k are rotated (pairs i, i + rot_dims/2) and k scaled here.
// raw o goes to O [R][heads * vdim] (fp32); normalisation and the gate follow in k_ret_post.
__global__ void k_retention(PassTables t, RetBranch b, const float* __restrict__ P, int ldp, float* __restrict__ state, float* __restrict__ O, int vs) {
    extern __shared__ float sm[];
    const int s = blockIdx.x, h = blockIdx.y;
    const int slot = t.seg_slot[s], row0 = t.seg_row0[s], len = t.seg_len[s];
    const int ny = blockDim.y, ty = threadIdx.y, jl = threadIdx.x;        // blockDim.x >= vs
    const int j = blockIdx.z * vs + jl;                                   // value channel
    const bool jok = jl < vs && j < b.vdim;
    const int tid = ty * blockDim.x + jl, nt = blockDim.x * ny;
    float* S = sm;                                   // [dim][vs]
    float* sq = S + (size_t)b.dim * vs;              // [2][dim]
    float* sk = sq + 2 * b.dim;                      // [2][dim]
    float* part = sk + 2 * b.dim;                    // [ny][vs]
    float* gs = state + ((size_t)slot * b.heads + h) * (size_t)b.dim * b.vdim;
    const bool live = !t.slots[slot].stopped;
    for (int e = tid; e < b.dim * vs; e += nt) {
        const int i = e / vs, c = blockIdx.z * vs + e % vs;
        S[e] = c < b.vdim ? gs[(size_t)i * b.vdim + c] : 0.0f;
    }
    const float decay = b.decay[h];
    const int half = b.rot_dims / 2;
    const int i0 = (int)(((long long)b.dim * ty) / ny), i1 = (int)(((long long)b.dim * (ty + 1)) / ny);
    for (int n = 0; n < len; n++) {
        const int r = row0 + n, buf = n & 1;
        const float* p = P + (size_t)r * ldp;
        const float pos = (float)t.row_pos[r];
        for (int i = tid; i < b.dim; i += nt) {
            float qv = p[b.q_off + h * b.dim + i], kv = p[b.k_off + h * b.dim + i];
            if (i < b.rot_dims) {
                const int f = i < half ? i : i - half;
                float sn, cs;
                sincosf(pos * b.inv_freq[f], &sn, &cs);
                const int o = i < half ? i + half : i - half;
                const float qo = p[b.q_off + h * b.dim + o], ko = p[b.k_off + h * b.dim + o];
                // pair (u, v) = (x_i, x_(i + half)): u' = u cos - v sin, v' = v cos + u sin
                qv = i < half ? qv * cs - qo * sn : qv * cs + qo * sn;
                kv = i < half ? kv * cs - ko * sn : kv * cs + ko * sn;
            }
            sq[buf * b.dim + i] = qv;
            sk[buf * b.dim + i] = kv * b.scale;
        }
        __syncthreads();
        if (jok) {
            const float v = p[b.v_off + h * b.vdim + j];
            float o = 0.0f;
            for (int i = i0; i < i1; i++) {
                const float sv = fmaf(decay, S[(size_t)i * vs + jl], sk[buf * b.dim + i] * v);
                S[(size_t)i * vs + jl] = sv;
                o = fmaf(sv, sq[buf * b.dim + i], o);
            }
            part[ty * vs + jl] = o;
        }
        __syncthreads();
        if (ty == 0 && jok) {
            float o = 0.0f;
            for (int y = 0; y < ny; y++) o += part[y * vs + jl];
            O[(size_t)r * (b.heads * b.vdim) + h * b.vdim + j] = o;
        }
    }
    __syncthreads();
    if (live)
        for (int e = tid; e < b.dim * vs; e += nt) {
            const int i = e / vs, c = blockIdx.z * vs + e % vs;
            if (c < b.vdim) gs[(size_t)i * b.vdim + c] = S[e];
        }
}
// per (row, head): o / rms(o) (optional), * silu(gate) (optional), * out_scale -> operand of the out projection
template <typename OT>
__global__ void k_ret_post(RetBranch b, const float* __restrict__ O, const float* __restrict__ P, int ldp, OT* __restrict__ out, int ld_out) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int h = blockIdx.y * nw + wid; h < b.heads; h += gridDim.y * nw) {
        const float* o = O + (size_t)r * (b.heads * b.vdim) + h * b.vdim;
        float sc = b.out_scale;
        if (b.out_norm) {
            float ss = 0.0f;
            for (int i = lane; i < b.vdim; i += 32) ss += o[i] * o[i];
            ss = warp_sum(ss);
            sc *= 1.0f / sqrtf(ss / (float)b.vdim + b.eps);
        }
        for (int i = lane; i < b.vdim; i += 32) {
            float v = o[i] * sc;
            if (b.gated) { const float g = P[(size_t)r * ldp + b.g_off + h * b.vdim + i]; v *= g * sigmoidf_(g); }
            out[(size_t)r * ld_out + b.a_off + h * b.vdim + i] = cvt<OT>(v);
        }
    }
}

// ------------------------------------------------------------------------------------------------ feed-forward activation, glue
// act = gelu_tanh(gate) * up from G [R][2 ff] into the out-projection operand at column a_off.  Columns of G: gate | up, or
// (interleaved) groups of 32 gate columns each followed by its 32 up columns.
template <typename OT>
__global__ void k_geglu(const float* __restrict__ G, int ff, OT* __restrict__ out, int ld_out, int a_off, int R, int interleaved) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * ff) return;
    const int r = (int)(i / ff), c = (int)(i % ff);
    const int gc = interleaved ? (c >> 5) * 64 + (c & 31) : c, uc = interleaved ? gc + 32 : ff + c;
    out[(size_t)r * ld_out + a_off + c] = cvt<OT>(gelu_tanh(G[(size_t)r * 2 * ff + gc]) * G[(size_t)r * 2 * ff + uc]);
}
// C[r][c] += Y[r][c] for an [M][N] block (N contiguous in Y)
__global__ void k_add_block(float* __restrict__ C, int ldc, const float* __restrict__ Y, int N, int M) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * N) return;
    const size_t r = i / N, c = i % N;
    C[r * ldc + c] += Y[i];
}
// operand [x | x0] of the loop's entry projection
template <typename OT>
__global__ void k_concat2(const float* __restrict__ x, const float* __restrict__ x0, int width, OT* __restrict__ out, int ld_out) {
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        out[(size_t)r * ld_out + c] = cvt<OT>(x[(size_t)r * width + c]);
        out[(size_t)r * ld_out + width + c] = cvt<OT>(x0[(size_t)r * width + c]);
    }
}

// ------------------------------------------------------------------------------------------------ sampling
// first maximum of each logits row (lowest index wins ties, like the greedy loop of the single-model engine); the token becomes the
// slot's pending token and lands in hist[row][step]; a slot that samples eos_id stops.
__global__ void __launch_bounds__(1024) k_argmax_rows(const float* __restrict__ logits, int n, PassTables t, int eos_id, int* __restrict__ out,
                                                       int out_ld, int out_col) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const int s = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const float* lg = logits + (size_t)s * n;
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int j = tid; j < n; j += blockDim.x) {
        const float v = lg[j];
        if (v > best) { best = v; arg = j; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
    }
    if (lane == 0) { sv[wid] = best; si[wid] = arg; }
    __syncthreads();
    if (wid == 0) {
        best = sv[lane]; arg = si[lane];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
        }
        if (lane == 0) {
            if (arg == 0x7fffffff) arg = 0;
            SlotState& st = t.slots[t.seg_slot[s]];
            if (st.stopped) arg = st.pending;
            st.pending = arg;
            if (eos_id >= 0 && arg == eos_id) st.stopped = 1;
            out[(size_t)s * out_ld + out_col] = arg;
        }
    }
}

// ================================================================================================ chunked retention (prompt portions)
// The recurrence S_t = g S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over a chunk of L rows that starts from state S0 is
//     o_a   = g^(a+1) S0^T q_a + sum_{b <= a} g^(a-b) (q_a . k_b) v_b
//     S_end = g^L S0 + sum_b g^(L-1-b) k_b v_b^T
// so the rows of a chunk are matrix products, and only a cheap scan over the chunks' [dim][vdim] contributions is sequential:
//   k_ret_rotate     rotary positions on q and k, k scaled (in place, fp32)
//   k_ret_chunk_kv   U_c = sum_b g^(L-1-b) k_b v_b^T for every chunk, all chunks in parallel
//   k_ret_scan       per (segment, head): walks the chunks, leaves the state BEFORE each chunk in its U_c slot, writes the slot's state
//   k_ret_chunk_out  o of every row from its chunk's q, k, v and the state before the chunk, all chunks in parallel
// All of it is fp32 FFMA in both compute modes: state, decay powers and everything that enters the recurrence stay in 32-bit.
__device__ __forceinline__ bool ret_find_chunk(const PassTables& t, int S, int C, int idx, int& seg, int& c) {
    for (int s = 0; s < S; s++) {
        const int n = (t.seg_len[s] + C - 1) / C;
        if (idx < n) { seg = s; c = idx; return true; }
        idx -= n;
    }
    return false;
}

__global__ void k_ret_rotate(PassTables t, RetBranch b, float* __restrict__ P, int ldp) {
    const int r = blockIdx.x;
    float* p = P + (size_t)r * ldp;
    const float pos = (float)t.row_pos[r];
    const int half = b.rot_dims / 2;
    for (int e = threadIdx.x; e < b.heads * b.dim; e += blockDim.x) {
        const int h = e / b.dim, i = e % b.dim;
        if (i < half) {
            float sn, cs;
            sincosf(pos * b.inv_freq[i], &sn, &cs);
            float* q = p + b.q_off + h * b.dim;
            float* k = p + b.k_off + h * b.dim;
            const float qu = q[i], qv = q[i + half], ku = k[i], kv = k[i + half];
            q[i] = qu * cs - qv * sn; q[i + half] = qv * cs + qu * sn;
            k[i] = (ku * cs - kv * sn) * b.scale; k[i + half] = (kv * cs + ku * sn) * b.scale;
        } else if (i >= b.rot_dims) {
            p[b.k_off + h * b.dim + i] *= b.scale;
        }
    }
}

// grid (chunks, heads, value slices); U [chunk][head][dim][vdim].  Shared memory: k' [C][dp] (k times g^(L-1-b)), v [C][vsp]; a thread
// accumulates 4 x 4 tiles of U from float4 reads (dp, vsp: dim and the slice width rounded up to 4, zero-filled).
__global__ void __launch_bounds__(256) k_ret_chunk_kv(PassTables t, RetBranch b, const float* __restrict__ P, int ldp, int S, int C, int vs,
                                                      float* __restrict__ U) {
    extern __shared__ __align__(16) float sm[];
    int seg, c;
    if (!ret_find_chunk(t, S, C, blockIdx.x, seg, c)) return;
    const int h = blockIdx.y, j0 = blockIdx.z * vs, nv = min(vs, b.vdim - j0);
    const int row0 = t.seg_row0[seg] + c * C, L = min(C, t.seg_len[seg] - c * C);
    const int dp = (b.dim + 3) & ~3, vsp = (vs + 3) & ~3;
    float* sk = sm;                 // [C][dp]
    float* sv = sm + C * dp;        // [C][vsp]
    const float lg = logf(b.decay[h]);
    for (int e = threadIdx.x; e < C * dp; e += blockDim.x) {
        const int bb = e / dp, i = e % dp;
        sk[e] = (bb < L && i < b.dim) ? P[(size_t)(row0 + bb) * ldp + b.k_off + h * b.dim + i] * expf(lg * (float)(L - 1 - bb)) : 0.0f;
    }
    for (int e = threadIdx.x; e < C * vsp; e += blockDim.x) {
        const int bb = e / vsp, j = e % vsp;
        sv[e] = (bb < L && j < nv) ? P[(size_t)(row0 + bb) * ldp + b.v_off + h * b.vdim + j0 + j] : 0.0f;
    }
    __syncthreads();
    float* u = U + (((size_t)blockIdx.x * b.heads + h) * b.dim) * b.vdim;
    const int tj = vsp / 4, ti = dp / 4;
    for (int tile = threadIdx.x; tile < ti * tj; tile += blockDim.x) {
        const int i4 = (tile / tj) * 4, j4 = (tile % tj) * 4;
        float acc[4][4] = {};
        for (int bb = 0; bb < L; bb++) {
            const float4 k4 = *reinterpret_cast<const float4*>(sk + bb * dp + i4);
            const float4 v4 = *reinterpret_cast<const float4*>(sv + bb * vsp + j4);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int x = 0; x < 4; x++)
#pragma unroll
                for (int y = 0; y < 4; y++) acc[x][y] = fmaf(kk[x], vv[y], acc[x][y]);
        }
#pragma unroll
        for (int x = 0; x < 4; x++)
#pragma unroll
            for (int y = 0; y < 4; y++)
                if (i4 + x < b.dim && j4 + y < nv) u[(size_t)(i4 + x) * b.vdim + j0 + j4 + y] = acc[x][y];
    }
}

// grid (segments, heads, blocks of state elements): every state element walks the segment's chunks on its own
__global__ void __launch_bounds__(256) k_ret_scan(PassTables t, RetBranch b, int S, int C, float* __restrict__ U, float* __restrict__ state) {
    const int seg = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= b.dim * b.vdim) return;
    int first = 0;
    for (int s = 0; s < seg; s++) first += (t.seg_len[s] + C - 1) / C;
    const int len = t.seg_len[seg], nchunk = (len + C - 1) / C, slot = t.seg_slot[seg];
    float* gs = state + ((size_t)slot * b.heads + h) * (size_t)b.dim * b.vdim;
    const float lg = logf(b.decay[h]);
    const float gc = expf(lg * (float)C);
    float s0 = gs[e];
    float* u = U + (((size_t)first * b.heads + h) * b.dim) * b.vdim + e;
    const size_t stride = (size_t)b.heads * b.dim * b.vdim;
    // batches of 16 chunks: all of a batch's loads are issued before the dependent chain of multiply-adds starts
    for (int c0 = 0; c0 < nchunk; c0 += 16) {
        float add[16];
#pragma unroll
        for (int i = 0; i < 16; i++) add[i] = (c0 + i < nchunk) ? u[(size_t)(c0 + i) * stride] : 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++)
            if (c0 + i < nchunk) {
                u[(size_t)(c0 + i) * stride] = s0;
                const int Lc = min(C, len - (c0 + i) * C);
                s0 = fmaf(Lc == C ? gc : expf(lg * (float)Lc), s0, add[i]);
            }
    }
    if (!t.slots[slot].stopped) gs[e] = s0;
}

// grid (chunks, heads, value slices); Sb [chunk][head][dim][vdim] = state before the chunk; O [R][heads * vdim].
// Shared memory, all zero-filled beyond the chunk's rows and the slice's columns: qT, kT [dim][C] (position-minor, so that four rows
// are one float4), v [C][vsp], aT [C keys][C rows] = g^(a-b) q_a.k_b for b <= a, s0 [dim][vsp].  Three products on 4 x 4 register tiles.
__global__ void __launch_bounds__(256) k_ret_chunk_out(PassTables t, RetBranch b, const float* __restrict__ P, int ldp, int S, int C, int vs,
                                                       const float* __restrict__ Sb, float* __restrict__ O) {
    extern __shared__ __align__(16) float sm[];
    int seg, c;
    if (!ret_find_chunk(t, S, C, blockIdx.x, seg, c)) return;
    const int h = blockIdx.y, j0 = blockIdx.z * vs, nv = min(vs, b.vdim - j0);
    const int row0 = t.seg_row0[seg] + c * C, L = min(C, t.seg_len[seg] - c * C);
    const int vsp = (vs + 3) & ~3;
    const int CP = C + 4;                 // row pitch of the transposed operands: float4 reads stay aligned, transposing stores hit 8 banks
    float* sq = sm;                       // [dim][CP]
    float* sk = sq + b.dim * CP;          // [dim][CP]; the same space holds s0 [dim][vsp] once the key products are done (vsp <= C)
    float* sv = sk + b.dim * CP;          // [C][vsp]
    float* sa = sv + C * vsp;             // [C][C]
    float* s0 = sk;
    const float lg = logf(b.decay[h]);
    for (int e = threadIdx.x; e < C * b.dim; e += blockDim.x) {      // a warp reads 32 consecutive dims of one row
        const int i = e % b.dim, bb = e / b.dim;
        float qv = 0.0f, kv = 0.0f;
        if (bb < L) {
            const float* p = P + (size_t)(row0 + bb) * ldp;
            qv = p[b.q_off + h * b.dim + i];
            kv = p[b.k_off + h * b.dim + i];
        }
        sq[i * CP + bb] = qv;
        sk[i * CP + bb] = kv;
    }
    for (int e = threadIdx.x; e < C * vsp; e += blockDim.x) {
        const int bb = e / vsp, j = e % vsp;
        sv[e] = (bb < L && j < nv) ? P[(size_t)(row0 + bb) * ldp + b.v_off + h * b.vdim + j0 + j] : 0.0f;
    }
    __syncthreads();
    const int tc = C / 4;
    for (int tile = threadIdx.x; tile < tc * tc; tile += blockDim.x) {
        const int a4 = (tile / tc) * 4, b4 = (tile % tc) * 4;
        float acc[4][4] = {};                           // [key][row]
        if (b4 <= a4 + 3 && a4 < L) {
            for (int i = 0; i < b.dim; i++) {
                const float4 q4 = *reinterpret_cast<const float4*>(sq + i * CP + a4);
                const float4 k4 = *reinterpret_cast<const float4*>(sk + i * CP + b4);
                const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                for (int y = 0; y < 4; y++)
#pragma unroll
                    for (int x = 0; x < 4; x++) acc[y][x] = fmaf(kk[y], qq[x], acc[y][x]);
            }
        }
#pragma unroll
        for (int y = 0; y < 4; y++)
#pragma unroll
            for (int x = 0; x < 4; x++) {
                const int a = a4 + x, bb = b4 + y;
                sa[bb * C + a] = (bb <= a) ? acc[y][x] * expf(lg * (float)(a - bb)) : 0.0f;
            }
    }
    __syncthreads();
    const float* sb = Sb + (((size_t)blockIdx.x * b.heads + h) * b.dim) * b.vdim;
    for (int e = threadIdx.x; e < b.dim * vsp; e += blockDim.x) {
        const int i = e / vsp, j = e % vsp;
        s0[e] = j < nv ? sb[(size_t)i * b.vdim + j0 + j] : 0.0f;
    }
    __syncthreads();
    const int tj = vsp / 4;
    for (int tile = threadIdx.x; tile < tc * tj; tile += blockDim.x) {
        const int a4 = (tile / tj) * 4, j4 = (tile % tj) * 4;
        if (a4 >= L) continue;
        float intra[4][4] = {}, inter[4][4] = {};       // [row][channel]
        const int bmax = min(L, a4 + 4);
        for (int bb = 0; bb < bmax; bb++) {
            const float4 w4 = *reinterpret_cast<const float4*>(sa + bb * C + a4);
            const float4 v4 = *reinterpret_cast<const float4*>(sv + bb * vsp + j4);
            const float ww[4] = {w4.x, w4.y, w4.z, w4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int x = 0; x < 4; x++)
#pragma unroll
                for (int y = 0; y < 4; y++) intra[x][y] = fmaf(ww[x], vv[y], intra[x][y]);
        }
        for (int i = 0; i < b.dim; i++) {
            const float4 q4 = *reinterpret_cast<const float4*>(sq + i * CP + a4);
            const float4 z4 = *reinterpret_cast<const float4*>(s0 + i * vsp + j4);
            const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, zz[4] = {z4.x, z4.y, z4.z, z4.w};
#pragma unroll
            for (int x = 0; x < 4; x++)
#pragma unroll
                for (int y = 0; y < 4; y++) inter[x][y] = fmaf(qq[x], zz[y], inter[x][y]);
        }
#pragma unroll
        for (int x = 0; x < 4; x++) {
            if (a4 + x >= L) continue;
            const float ga = expf(lg * (float)(a4 + x + 1));
#pragma unroll
            for (int y = 0; y < 4; y++)
                if (j4 + y < nv) O[(size_t)(row0 + a4 + x) * (b.heads * b.vdim) + h * b.vdim + j0 + j4 + y] = fmaf(ga, inter[x][y], intra[x][y]);
        }
    }
}

// ================================================================================================ sigmoid attention on tensor cores
// Prompt portions in bf16 mode: a CTA owns 64 consecutive rows of one segment and one query head (4 warps x 16 rows) and sweeps the
// slot's cache in tiles of 64 keys up to its last row's position: S = Q K^T on mma.sync m16n8k16 (bf16 operands, fp32 accumulators),
// weight = sigmoid(scale S + pb) in fp32 under the causal mask, O += W V with the weights as bf16 A fragments taken straight from
// the accumulator registers.  No running maximum and no rescaling: the weights are not normalised.  DP / VP: head sizes padded to
// 32, 64 or 128 with zero columns in shared memory.
__device__ __forceinline__ void sa_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void sa_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void sa_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sa_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// sigmoid from the special-function unit's exp2 and reciprocal: relative error of a few ulp also for tiny weights (the weights are
// rounded to bf16 right after)
__device__ __forceinline__ float sa_sigmoid(float z) { return __fdividef(1.0f, 1.0f + __expf(-z)); }
__device__ __forceinline__ bool sa_find_tile(const PassTables& t, int S, int idx, int& seg, int& q0) {
    for (int s = 0; s < S; s++) {
        const int n = (t.seg_len[s] + 63) / 64;
        if (idx < n) { seg = s; q0 = (n - 1 - idx) * 64; return true; }      // a segment's last tiles sweep the most keys: they start first
        idx -= n;
    }
    return false;
}

// 16-byte asynchronous copy global -> shared; !valid: the destination is filled with zeros
__device__ __forceinline__ void sa_cp16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

template <int DP, int VP, int HPC>
__global__ void __launch_bounds__(128 * HPC) k_sigattn_mma(PassTables t, AttnBranch b, int S, const float* __restrict__ P, int ldp, const bf16* __restrict__ kc,
                                                     const bf16* __restrict__ vc, bf16* __restrict__ out, int ld_out) {
    constexpr int LQ = DP + 8, LV = VP + 8;
    extern __shared__ __align__(16) unsigned char sa_raw[];
    bf16* sq = reinterpret_cast<bf16*>(sa_raw);          // [HPC][64][LQ]: the CTA's query heads share one K/V head
    bf16* sk0 = sq + HPC * 64 * LQ;                     // [2][64][LQ]: key tiles, double-buffered
    bf16* sv0 = sk0 + 2 * 64 * LQ;                      // [2][64][LV]
    int seg, q0;
    if (!sa_find_tile(t, S, blockIdx.x, seg, q0)) return;
    constexpr int NT = 128 * HPC;
    const int hsub = (threadIdx.x >> 7);                 // which of the CTA's heads this warp works for
    const int h = blockIdx.y * HPC + hsub, g = h / (b.heads / b.kv_heads);
    const int slot = t.seg_slot[seg], row0 = t.seg_row0[seg] + q0, nq = min(64, t.seg_len[seg] - q0);
    const int pos0 = t.row_pos[row0];                    // position of the tile's first row; row i sits at pos0 + i
    const int warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    for (int e = threadIdx.x; e < HPC * 64 * DP; e += NT) {
        const int hh = e / (64 * DP), r = (e / DP) % 64, i = e % DP;
        sq[(hh * 64 + r) * LQ + i] = __float2bfloat16_rn((r < nq && i < b.dim) ? P[(size_t)(row0 + r) * ldp + b.q_off + (blockIdx.y * HPC + hh) * b.dim + i] : 0.0f);
    }
    const float bias = b.pb ? b.pb[h] : 0.0f;
    const size_t kld = (size_t)b.kv_heads * b.dim, vld = (size_t)b.kv_heads * b.vdim;
    const bf16* kbase = kc + (size_t)slot * b.max_ctx * kld + (size_t)g * b.dim;
    const bf16* vbase = vc + (size_t)slot * b.max_ctx * vld + (size_t)g * b.vdim;
    const bool vec = (b.dim % 8 == 0) && (b.vdim % 8 == 0);
    float o[VP / 8][4];
#pragma unroll
    for (int n = 0; n < VP / 8; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    const int last = pos0 + nq - 1;                      // last key any row of the tile sees
    const uint32_t sq_a = (uint32_t)__cvta_generic_to_shared(sq + hsub * 64 * LQ);
    // tile j0 -> stage st: asynchronous 16-byte copies when the cache rows are 16-byte aligned, plain loads otherwise
    auto load_tile = [&](int st, int j0) {
        bf16* sk = sk0 + st * 64 * LQ;
        bf16* sv = sv0 + st * 64 * LV;
        const int nk = min(64, last + 1 - j0);
        if (vec) {
            const uint32_t ka = (uint32_t)__cvta_generic_to_shared(sk), va = (uint32_t)__cvta_generic_to_shared(sv);
            for (int e = threadIdx.x; e < 64 * (DP / 8); e += NT) {
                const int r = e / (DP / 8), c8 = (e % (DP / 8)) * 8;
                const bool ok = r < nk && c8 < b.dim;
                sa_cp16(ka + (uint32_t)((r * LQ + c8) * 2), ok ? (const void*)(kbase + (size_t)(j0 + r) * kld + c8) : (const void*)kbase, ok);
            }
            for (int e = threadIdx.x; e < 64 * (VP / 8); e += NT) {
                const int r = e / (VP / 8), c8 = (e % (VP / 8)) * 8;
                const bool ok = r < nk && c8 < b.vdim;
                sa_cp16(va + (uint32_t)((r * LV + c8) * 2), ok ? (const void*)(vbase + (size_t)(j0 + r) * vld + c8) : (const void*)vbase, ok);
            }
        } else {
            for (int e = threadIdx.x; e < 64 * DP; e += NT) {
                const int r = e / DP, i = e % DP;
                sk[r * LQ + i] = (r < nk && i < b.dim) ? kbase[(size_t)(j0 + r) * kld + i] : __float2bfloat16_rn(0.0f);
            }
            for (int e = threadIdx.x; e < 64 * VP; e += NT) {
                const int r = e / VP, i = e % VP;
                sv[r * LV + i] = (r < nk && i < b.vdim) ? vbase[(size_t)(j0 + r) * vld + i] : __float2bfloat16_rn(0.0f);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_tile(0, 0);
    int it = 0;
    for (int j0 = 0; j0 <= last; j0 += 64, it++) {
        const int st = it & 1;
        const bool more = j0 + 64 <= last;
        if (more) load_tile(st ^ 1, j0 + 64);            // its previous reader passed the barrier at the end of the last iteration
        if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const uint32_t sk_a = (uint32_t)__cvta_generic_to_shared(sk0 + st * 64 * LQ), sv_a = (uint32_t)__cvta_generic_to_shared(sv0 + st * 64 * LV);
        if (j0 > pos0 + warp * 16 + 15) { __syncthreads(); continue; }        // every key of the tile lies after this warp's rows
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; n++) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f; }
#pragma unroll
        for (int kk = 0; kk < DP / 16; kk++) {
            uint32_t a[4];
            sa_ldsm_x4(sq_a + (uint32_t)(((warp * 16 + (lane & 15)) * LQ + kk * 16 + (lane >> 4) * 8) * 2), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int n2 = 0; n2 < 4; n2++) {
                uint32_t b0, b1, b2, b3;
                sa_ldsm_x4(sk_a + (uint32_t)(((n2 * 16 + (lane & 7) + (lane >> 4) * 8) * LQ + kk * 16 + ((lane >> 3) & 1) * 8) * 2), b0, b1, b2, b3);
                sa_mma(sc[2 * n2], a, b0, b1);
                sa_mma(sc[2 * n2 + 1], a, b2, b3);
            }
        }
        // weights: rows gq and gq + 8 of the warp's 16, keys j0 + 8 n + 2 tq (+1)
        const int p_lo = pos0 + warp * 16 + gq, p_hi = p_lo + 8;
        uint32_t w[8][2];
#pragma unroll
        for (int n = 0; n < 8; n++) {
            const int key = j0 + n * 8 + tq * 2;
            const float w0 = key <= p_lo ? sa_sigmoid(sc[n][0] * b.scale + bias) : 0.0f;
            const float w1 = key + 1 <= p_lo ? sa_sigmoid(sc[n][1] * b.scale + bias) : 0.0f;
            const float w2 = key <= p_hi ? sa_sigmoid(sc[n][2] * b.scale + bias) : 0.0f;
            const float w3 = key + 1 <= p_hi ? sa_sigmoid(sc[n][3] * b.scale + bias) : 0.0f;
            w[n][0] = sa_pack(w0, w1);
            w[n][1] = sa_pack(w2, w3);
        }
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {                 // 16 keys per step
            const uint32_t a[4] = {w[2 * kk][0], w[2 * kk][1], w[2 * kk + 1][0], w[2 * kk + 1][1]};
#pragma unroll
            for (int n2 = 0; n2 < VP / 16; n2++) {
                uint32_t b0, b1, b2, b3;
                sa_ldsm_x4_t(sv_a + (uint32_t)(((kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LV + n2 * 16 + (lane >> 4) * 8) * 2), b0, b1, b2, b3);
                sa_mma(o[2 * n2], a, b0, b1);
                sa_mma(o[2 * n2 + 1], a, b2, b3);
            }
        }
        __syncthreads();                                 // this stage may be refilled from the next iteration on
    }
    const int r_lo = warp * 16 + gq, r_hi = r_lo + 8;
#pragma unroll
    for (int n = 0; n < VP / 8; n++) {
        const int c = n * 8 + tq * 2;
#pragma unroll
        for (int x = 0; x < 2; x++) {
            if (c + x >= b.vdim) continue;
            if (r_lo < nq) out[(size_t)(row0 + r_lo) * ld_out + b.a_off + h * b.vdim + c + x] = __float2bfloat16_rn(o[n][x] * b.out_scale);
            if (r_hi < nq) out[(size_t)(row0 + r_hi) * ld_out + b.a_off + h * b.vdim + c + x] = __float2bfloat16_rn(o[n][2 + x] * b.out_scale);
        }
    }
}

}  // namespace seq
}  // namespace gtb

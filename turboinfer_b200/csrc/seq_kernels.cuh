// seq_kernels.cuh -- kernels of the layered sequence engine (seq_engine.cu): a decoder described layer by layer (windowed
// rotary attention with unit-RMS queries / keys and a per-head output gate, token-shifted linear recurrence with a
// data-dependent decay, gated feed-forward, scalar-gain RMS norms before and after every sublayer, a looped block of
// layers) stepping a RAGGED batch: the rows of a step are the new tokens of several sequences, portions of prompts next
// to single decoded tokens.  Every row carries (sequence entry, position); attention reads a paged key/value cache through
// the sequence's page table, the recurrence reads and writes the sequence's state slot.
//
// Number formats.  The residual stream, norms, rotary angles, attention scores and weights, the recurrent state, decays,
// gates of the recurrence and unit norms are fp32 in both modes.  WT = __nv_bfloat16: matrix products take bf16 weights and
// bf16-rounded activations with fp32 accumulation (tensor cores); WT = float: true fp32 FMA products (no TF32).
#pragma once
#include <cuda_bf16.h>
#include <cstdint>
#include "kernels.cuh"

namespace tib {
namespace seq {

constexpr int kPageTokens = 64;

// what a step's kernels need to find a row's sequence: all arrays live in one device buffer uploaded once per step
struct StepMeta {
    const int* tok;        // [T] token id of every row
    const int* row_ent;    // [T] entry (sequence of this step) of every row
    const int* row_pos;    // [T] position of the row's token in its sequence
    const int* ent_row0;   // [E + 1] first row of every entry
    const int* ent_slot;   // [E] state slot / page-table row of every entry
    const int* ent_pos0;   // [E] position of the entry's first row (tokens already cached)
    const int* page_table; // [slots][table_stride] physical page of every logical page
    int table_stride;
    int T, E;
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
// activation as the matrix product sees it: rounded to the weight type
template <typename WT> __device__ __forceinline__ float act_round(float v);
template <> __device__ __forceinline__ float act_round<float>(float v) { return v; }
template <> __device__ __forceinline__ float act_round<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// sum over the block (blockDim.x a multiple of 32, <= 1024); `red` holds 32 floats; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float s = (l < nw) ? red[l] : 0.f;
    s = warp_sum(s);
    return s;
}

// ---- embedding -----------------------------------------------------------------------------------------------------
// x[t] = embed[tok[t]] (+ the sinusoidal position vector: entry 2i = sin(pos * pos_freq[i]), entry 2i + 1 = cos of the same angle,
// angle and functions in fp32); x0 (optional) keeps the embedding output for the looped block's input projection; copies > 1: the row
// is written that many times in a row (x [T][copies][D]: the streams of hyper-connections all start from the embedding output)
template <typename WT>
__global__ void embed_rows_kernel(const WT* emb, StepMeta m, int D, float* x, float* x0, const float* pos_freq, int copies) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    const int t = blockIdx.x;
    const WT* e = emb + (size_t)m.tok[t] * D;
    const float pos = pos_freq ? (float)m.row_pos[t] : 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = to_f32(e[d]);
        if (pos_freq) {
            const float ang = pos * pos_freq[d >> 1];
            v += (d & 1) ? cosf(ang) : sinf(ang);
        }
        for (int c = 0; c < copies; ++c) x[((size_t)t * copies + c) * D + d] = v;
        if (x0) x0[(size_t)t * D + d] = v;
    }
}
// xc[t] = [x[t]; x0[t]]
__global__ void concat_rows_kernel(const float* x, const float* x0, int D, float* xc) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        xc[(size_t)t * 2 * D + d] = x[(size_t)t * D + d];
        xc[(size_t)t * 2 * D + D + d] = x0[(size_t)t * D + d];
    }
}

// ---- RMS norms -------------------------------------------------------------------------------------------------------------
// The gain is one number for all coordinates (gvec = 0: gain[0]) or one per coordinate (gvec = 1: gain[d]; a design that stores
// its gains around zero and applies 1 + w has them converted once when the model is finalized).
// y[t] = x[row(t)] / sqrt(mean(x^2) + eps) * gain; rows (optional) gathers (the rows whose logits are wanted); ldx = row stride of x
// (a slice of a wider projection output)
__global__ void rmsnorm_kernel(const float* x, int ldx, const int* rows, int D, const float* gain, int gvec, float eps, float* y) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    __shared__ float red[32];
    const int t = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[t] : t) * ldx;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) ss += xr[d] * xr[d];
    ss = block_sum(ss, red);
    const float sc = 1.f / sqrtf(ss / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) y[(size_t)t * D + d] = xr[d] * sc * gain[gvec ? d : 0];
}
// The end of a sublayer: x[t] += norm(m[t]) with m = the sublayer's result, optionally
//   * multiplied first by sigmoid(gate[t][d] + gate_bias[d]) (a gated residual: `gate` is a slice of the sublayer's fused input
//     projection, row stride gate_ld), and
//   * with idw[t] * hin[t][d] added before that (experts that return their input, weighted by the router),
// and with gain2 != null the next sublayer's input y[t] = x[t] / rms(x[t]) * gain2 is written in the same pass.
struct PostArgs {
    float* x;              // [T][D] residual stream, updated in place
    float* mo;             // [T][D] sublayer result (overwritten with the gated value when a gate is given)
    const float* gain;     // norm behind the sublayer
    const float* gain2;    // norm in front of the next sublayer (null: none)
    float* y;              // [T][D] next sublayer's input
    const float* gate;     // null: no gate
    const float* gate_bias;
    const float* idw;      // [T] null: none
    const float* hin;      // [T][D]
    int gate_ld, D, gvec, gvec2;
    float eps;
};
__global__ void postnorm_residual_kernel(PostArgs a) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    __shared__ float red[32];
    const int t = blockIdx.x, D = a.D;
    float* mr = a.mo + (size_t)t * D;
    float* xr = a.x + (size_t)t * D;
    float ss = 0.f;
    if (a.gate || a.idw) {
        const float wi = a.idw ? a.idw[t] : 0.f;
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float v = mr[d];
            if (a.idw) v = fmaf(wi, a.hin[(size_t)t * D + d], v);
            if (a.gate) v *= 1.f / (1.f + expf(-(a.gate[(size_t)t * a.gate_ld + d] + a.gate_bias[d])));
            mr[d] = v;
            ss += v * v;
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) ss += mr[d] * mr[d];
    }
    ss = block_sum(ss, red);
    const float sc = 1.f / sqrtf(ss / (float)D + a.eps);
    float s2 = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = xr[d] + mr[d] * sc * a.gain[a.gvec ? d : 0];
        xr[d] = v;
        s2 += v * v;
    }
    if (a.gain2) {
        s2 = block_sum(s2, red);
        const float sc2 = 1.f / sqrtf(s2 / (float)D + a.eps);
        for (int d = threadIdx.x; d < D; d += blockDim.x) a.y[(size_t)t * D + d] = xr[d] * sc2 * a.gain2[a.gvec2 ? d : 0];
    }
}

// ---- matrix products: C[M, N] = epi(A[M, K] . W[N, K]^T) ----------------------------------------------------------------
enum {
    EPI_NONE = 0, EPI_TANH = 1, EPI_SCALE = 2, EPI_SILU = 3, EPI_SOFTCAP = 4 /* alpha * tanh(v / alpha) */, EPI_GELU_TANH = 5,
    EPI_XIELU = 6 /* alpha v^2 + v / 2 for v > 0, beta (exp(v) - 1 - v) + v / 2 otherwise */, EPI_MAX0 = 7
};
__device__ __forceinline__ float xielu(float v, float a_pos, float a_neg) {
    return v > 0.f ? fmaf(a_pos * v, v, 0.5f * v) : fmaf(a_neg, expm1f(v) - v, 0.5f * v);
}
__device__ __forceinline__ float epi_apply(float v, int epi, float alpha, float beta = 0.f) {
    if (epi == EPI_XIELU) return xielu(v, alpha, beta);
    if (epi == EPI_MAX0) return fmaxf(v, 0.f);
    if (epi == EPI_TANH) return tanhf(v);
    if (epi == EPI_SCALE) return v * alpha;
    if (epi == EPI_SILU) return v / (1.f + expf(-v));
    if (epi == EPI_SOFTCAP) return alpha * tanhf(v / alpha);
    if (epi == EPI_GELU_TANH) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

// true fp32: 64 x 64 tile, 16-deep k-steps, 256 threads with 4 x 4 outputs each
// (grid.z > 1: a batch of products, number z reads A + z * za, W + z * zw and writes C + z * zc -- one small matrix per head)
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* A, int lda, const float* W, float* C, int ldc, int M, int N, int K,
                                                        int epi, float alpha, float beta, size_t za, size_t zw, size_t zc) {
    __shared__ float As[16][64 + 4], Ws[16][64 + 4];
    A += blockIdx.z * za;
    W += blockIdx.z * zw;
    C += blockIdx.z * zc;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, c = i & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
            if (gm < M && gn < N) C[(size_t)gm * ldc + gn] = epi_apply(acc[i][j], epi, alpha, beta);
        }
}

// bf16 x bf16 -> fp32 on the warp-level tensor path (mma.sync m16n8k16): 64 x 64 tile, 32-deep k-steps, 4 warps of 32 x 32.
// A is fp32 in memory and rounded to bf16 while it is staged; any M, N, K (edges are zero-filled).
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// (grid.z > 1: a batch of products, as in gemm_f32_kernel)
__global__ void __launch_bounds__(128) gemm_bf16_kernel(const float* A, int lda, const __nv_bfloat16* W, float* C, int ldc, int M, int N,
                                                         int K, int epi, float alpha, float beta, size_t za, size_t zw, size_t zc) {
    constexpr int BM = 64, BN = 64, BK = 32, LD = BK + 8;
    __shared__ __align__(16) __nv_bfloat16 As[BM * LD], Ws[BN * LD];
    A += blockIdx.z * za;
    W += blockIdx.z * zw;
    C += blockIdx.z * zc;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const bool vecA = (lda % 4 == 0) && (K % BK == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    const bool vecW = (K % BK == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
    float acc[2][4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        if (vecA) {
            for (int i = threadIdx.x; i < BM * (BK / 4); i += 128) {
                const int r = i / (BK / 4), c = (i % (BK / 4)) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (m0 + r < M) v = *reinterpret_cast<const float4*>(A + (size_t)(m0 + r) * lda + k0 + c);
                __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(&As[r * LD + c]);
                d[0] = __floats2bfloat162_rn(v.x, v.y);
                d[1] = __floats2bfloat162_rn(v.z, v.w);
            }
        } else {
            for (int i = threadIdx.x; i < BM * BK; i += 128) {
                const int r = i / BK, c = i % BK;
                As[r * LD + c] = __float2bfloat16_rn((m0 + r < M && k0 + c < K) ? A[(size_t)(m0 + r) * lda + k0 + c] : 0.f);
            }
        }
        if (vecW) {
            for (int i = threadIdx.x; i < BN * (BK / 8); i += 128) {
                const int r = i / (BK / 8), c = (i % (BK / 8)) * 8;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (n0 + r < N) v = *reinterpret_cast<const uint4*>(W + (size_t)(n0 + r) * K + k0 + c);
                *reinterpret_cast<uint4*>(&Ws[r * LD + c]) = v;
            }
        } else {
            for (int i = threadIdx.x; i < BN * BK; i += 128) {
                const int r = i / BK, c = i % BK;
                Ws[r * LD + c] = (n0 + r < N && k0 + c < K) ? W[(size_t)(n0 + r) * K + k0 + c] : __float2bfloat16_rn(0.f);
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            uint32_t a[2][4], b[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const __nv_bfloat16* p = &As[(wm + i * 16 + g) * LD + kk + 2 * t4];
                a[i][0] = *reinterpret_cast<const uint32_t*>(p);
                a[i][1] = *reinterpret_cast<const uint32_t*>(p + 8 * LD);
                a[i][2] = *reinterpret_cast<const uint32_t*>(p + 8);
                a[i][3] = *reinterpret_cast<const uint32_t*>(p + 8 * LD + 8);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat16* p = &Ws[(wn + j * 8 + g) * LD + kk + 2 * t4];
                b[j][0] = *reinterpret_cast<const uint32_t*>(p);
                b[j][1] = *reinterpret_cast<const uint32_t*>(p + 8);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], a[i], b[j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int gm = m0 + wm + i * 16 + g + (e >> 1) * 8, gn = n0 + wn + j * 8 + 2 * t4 + (e & 1);
                if (gm < M && gn < N) C[(size_t)gm * ldc + gn] = epi_apply(acc[i][j][e], epi, alpha, beta);
            }
}

// few rows (M <= 8, the decode step): the weights are streamed once with 16-byte loads, one warp per output column; the rows
// sit in shared memory.  Fused in front: the scalar-gain RMS norm of the rows (norm_gain != null).  Fused behind: an activation
// or scale, or the gated feed-forward's act(gate) * up over the row pair (n, n + glu_ff) of the fused [gate | up] matrix.
// Bound by the weight bytes.
constexpr int kRowGemvMaxRows = 8;
constexpr int kRowGemvThreads = 256;
__device__ __forceinline__ float ff_act(float z, int act);
// eight consecutive weights as they lie in memory (kept packed while the loads are in flight) and as fp32
template <typename WT> struct Raw8;
template <> struct Raw8<float> { float4 a, b; };
template <> struct Raw8<__nv_bfloat16> { uint4 v; };
__device__ __forceinline__ void load_raw8(const float* p, Raw8<float>& r) {
    r.a = *reinterpret_cast<const float4*>(p);
    r.b = *reinterpret_cast<const float4*>(p + 4);
}
__device__ __forceinline__ void load_raw8(const __nv_bfloat16* p, Raw8<__nv_bfloat16>& r) { r.v = *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void unpack8(const Raw8<float>& r, float (&w)[8]) {
    w[0] = r.a.x; w[1] = r.a.y; w[2] = r.a.z; w[3] = r.a.w; w[4] = r.b.x; w[5] = r.b.y; w[6] = r.b.z; w[7] = r.b.w;
}
__device__ __forceinline__ void unpack8(const Raw8<__nv_bfloat16>& r, float (&w)[8]) {
    const uint32_t u[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        w[2 * i] = __uint_as_float(u[i] << 16);
        w[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
    }
}
template <typename WT>
__device__ __forceinline__ void gemv_row_dot(const WT* w, const float* xs, int M, int K, bool vec, int lane, float (&acc)[kRowGemvMaxRows]) {
#pragma unroll
    for (int r = 0; r < kRowGemvMaxRows; ++r) acc[r] = 0.f;
    if (vec) {
        constexpr int UNR = 32 / (int)sizeof(Raw8<WT>) * 4;   // 16-byte loads a lane has in flight before it multiplies: 8 (bf16), 4 (fp32)
        for (int k0 = lane * 8; k0 < K; k0 += 256 * UNR) {
            Raw8<WT> raw[UNR];
#pragma unroll
            for (int q = 0; q < UNR; ++q)
                if (k0 + 256 * q < K) load_raw8(w + k0 + 256 * q, raw[q]);
#pragma unroll
            for (int q = 0; q < UNR; ++q) {
                const int k = k0 + 256 * q;
                if (k < K) {
                    float wv[8];
                    unpack8(raw[q], wv);
#pragma unroll
                    for (int r = 0; r < kRowGemvMaxRows; ++r)
                        if (r < M) {
                            const float4 a = *reinterpret_cast<const float4*>(xs + r * K + k), b = *reinterpret_cast<const float4*>(xs + r * K + k + 4);
                            acc[r] = fmaf(a.x, wv[0], fmaf(a.y, wv[1], fmaf(a.z, wv[2], fmaf(a.w, wv[3], acc[r]))));
                            acc[r] = fmaf(b.x, wv[4], fmaf(b.y, wv[5], fmaf(b.z, wv[6], fmaf(b.w, wv[7], acc[r]))));
                        }
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = to_f32(w[k]);
#pragma unroll
            for (int r = 0; r < kRowGemvMaxRows; ++r)
                if (r < M) acc[r] = fmaf(xs[r * K + k], wv, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < kRowGemvMaxRows; ++r)
        if (r < M) acc[r] = warp_sum(acc[r]);
}
// Launched with programmatic stream serialization: the block asks L2 for its first weight rows while the kernel before it is
// still running, and only then waits for that kernel's results (the rows).
template <typename WT>
__global__ void __launch_bounds__(kRowGemvThreads, 2) gemv_rows_kernel(const float* A, int lda, const WT* W, float* C, int ldc, int M, int N, int K, int epi,
                                                                  float alpha, float beta, const float* norm_gain, float eps, int glu_ff, int glu_act, int gvec) {
    extern __shared__ __align__(16) float xs[];   // [M][K]
    __shared__ float rss[kRowGemvMaxRows][kRowGemvThreads / 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    pdl_launch_dependents();
    {   // the weights do not depend on the rows: ask L2 for this warp's first column(s) before the rows are there
        const int n = blockIdx.x * nw + warp;
        const size_t row_bytes = (size_t)K * sizeof(WT);
        if (n < N) {
            const char* w = reinterpret_cast<const char*>(W + (size_t)n * K);
            for (size_t o = (size_t)lane * 128; o < row_bytes; o += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(w + o));
            if (glu_ff > 0) {
                const char* w2 = reinterpret_cast<const char*>(W + (size_t)(n + glu_ff) * K);
                for (size_t o = (size_t)lane * 128; o < row_bytes; o += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(w2 + o));
            }
        }
    }
    pdl_wait_prior_grid();
    // rows -> shared memory (rounded to the weight type when no norm comes first), sums of squares on the way
    const bool vec4 = (K % 4 == 0) && (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    for (int r = 0; r < M; ++r) {
        const float* ar = A + (size_t)r * lda;
        float* xr = xs + (size_t)r * K;
        float ss = 0.f;
        if (vec4) {
            for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
                float4 v = *reinterpret_cast<const float4*>(ar + k);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                if (!norm_gain) { v.x = act_round<WT>(v.x); v.y = act_round<WT>(v.y); v.z = act_round<WT>(v.z); v.w = act_round<WT>(v.w); }
                *reinterpret_cast<float4*>(xr + k) = v;
            }
        } else {
            for (int k = threadIdx.x; k < K; k += blockDim.x) {
                const float v = ar[k];
                ss += v * v;
                xr[k] = norm_gain ? v : act_round<WT>(v);
            }
        }
        if (norm_gain) {
            ss = warp_sum(ss);
            if (lane == 0) rss[r][warp] = ss;
        }
    }
    __syncthreads();
    if (norm_gain) {
        for (int r = 0; r < M; ++r) {
            float ss = 0.f;
            for (int w = 0; w < nw; ++w) ss += rss[r][w];
            const float sc = 1.f / sqrtf(ss / (float)K + eps);
            float* xr = xs + (size_t)r * K;
            for (int k = threadIdx.x; k < K; k += blockDim.x) xr[k] = act_round<WT>(xr[k] * sc * norm_gain[gvec ? k : 0]);
        }
        __syncthreads();
    }
    const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
    float acc[kRowGemvMaxRows], acc2[kRowGemvMaxRows];
    for (int n = blockIdx.x * nw + warp; n < N; n += gridDim.x * nw) {
        gemv_row_dot<WT>(W + (size_t)n * K, xs, M, K, vec, lane, acc);
        if (glu_ff > 0) gemv_row_dot<WT>(W + (size_t)(n + glu_ff) * K, xs, M, K, vec, lane, acc2);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < kRowGemvMaxRows; ++r)
                if (r < M) C[(size_t)r * ldc + n] = glu_ff > 0 ? ff_act(acc[r], glu_act) * acc2[r] : epi_apply(acc[r], epi, alpha, beta);
        }
    }
}

// Few rows, one small matrix per head: C[r][h * c_stride + n] = sum_k A[r][h * a_stride + k] * W[h][n][k] (W: [heads][N][K]).
// grid (column groups, heads); the head's slice of the rows sits in shared memory, one warp per output column.
template <typename WT>
__global__ void __launch_bounds__(kRowGemvThreads) gemv_heads_rows_kernel(const float* A, int lda, int a_stride, const WT* W, float* C, int ldc, int c_stride, int M, int N,
                                                                           int K) {
    extern __shared__ __align__(16) float xs[];   // [M][K]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, h = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    for (int i = threadIdx.x; i < M * K; i += blockDim.x) xs[i] = act_round<WT>(A[(size_t)(i / K) * lda + (size_t)h * a_stride + i % K]);
    __syncthreads();
    const WT* Wh = W + (size_t)h * N * K;
    const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(Wh) & 15) == 0);
    float acc[kRowGemvMaxRows];
    for (int n = blockIdx.x * nw + warp; n < N; n += gridDim.x * nw) {
        gemv_row_dot<WT>(Wh + (size_t)n * K, xs, M, K, vec, lane, acc);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < kRowGemvMaxRows; ++r)
                if (r < M) C[(size_t)r * ldc + (size_t)h * c_stride + n] = acc[r];
        }
    }
}

// The same few-row product on the warp-level tensor cores (bf16 weights, bf16-rounded rows, fp32 accumulators): the cost of a
// weight byte no longer grows with the number of rows.  A block owns 16 output columns, its 8 warps split K; a lane (g = lane / 4,
// t = lane % 4) reads 16 bytes of column g and of column g + 8 straight from global memory and 16 bytes of row g from shared
// memory at the same 8 consecutive k -- the k order inside an m16n8k16 step is permuted the same way for both operands, which
// a dot product does not mind -- and issues two MMAs per 32 k.  The warps' partial tiles are summed through shared memory in warp
// order.  Needs K % 32 == 0 and 16-byte aligned weight rows.  Row stride in shared memory: K + 32 elements (rows of a quarter
// warp fall into different banks).
constexpr int kMmaCols = 16;
// Routed experts on few rows: the stacked matrices hold every expert's rows, the step's tokens chose only some.  Output columns
// (front product) or k (down product) in [first + e * group, first + (e + 1) * group) belong to expert e < count; a column tile or
// k chunk whose experts were chosen by no row is not read (its outputs are never used / its activations are exactly zero).
struct ExpertSkip {
    const int* used;   // [count] 0 / 1; null: nothing is skipped
    int first, group, count;
};
__device__ __forceinline__ bool expert_range_used(const ExpertSkip& s, int lo, int hi) {   // does [lo, hi] touch a used expert or leave the experts' range?
    if (!s.used) return true;
    if (lo < s.first) return true;
    const int e0 = (lo - s.first) / s.group, e1 = (hi - s.first) / s.group;
    for (int e = e0; e <= e1; ++e)
        if (e >= s.count || s.used[e]) return true;
    return false;
}
__host__ __device__ inline size_t gemv_mma_smem_bytes(int M, int K) { return (size_t)M * (K + 32) * 2 + 8 * 2 * 128 * sizeof(float); }
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <bool GLU>
__global__ void __launch_bounds__(256) gemv_rows_mma_kernel(const float* A, int lda, const __nv_bfloat16* W, float* C, int ldc, int M, int N, int K, int epi,
                                                           float alpha, float beta, const float* norm_gain, float eps, int glu_ff, int glu_act, int gvec, ExpertSkip nskip,
                                                           ExpertSkip kskip) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int Kp = K + 32;
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smraw);                       // [M][Kp]
    float* red = reinterpret_cast<float*>(smraw + (size_t)M * Kp * 2);                  // [8 warps][2][128]
    __shared__ float rss[kRowGemvMaxRows][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int NC = K / 32, c_begin = warp * NC / 8, c_end = (warp + 1) * NC / 8;   // this warp's 32-k chunks
    pdl_launch_dependents();
    {   // ask L2 for this warp's slice of the block's first 16 (32 with the gate's partner) weight rows
        const int n = min((int)blockIdx.x * kMmaCols + (lane & 15), N - 1);
        const char* w = reinterpret_cast<const char*>(W + (size_t)n * K + (size_t)c_begin * 32);
        const size_t bytes = (size_t)(c_end - c_begin) * 64;
        for (size_t o = (size_t)(lane >> 4) * 128; o < bytes; o += 256) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(w + o));
            if (GLU) asm volatile("prefetch.global.L2 [%0];" ::"l"(w + o + (size_t)glu_ff * K * 2));
        }
    }
    pdl_wait_prior_grid();
    // rows -> shared memory as bf16, behind the scalar-gain RMS norm when one is fused in front; 16-byte loads, several in flight
    // (every block stages all rows, so this prologue is on the critical path of the launch)
    const bool v4 = (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);   // K is a multiple of 32
    if (norm_gain) {
        for (int r = 0; r < M; ++r) {
            const float* ar = A + (size_t)r * lda;
            float ss = 0.f;
            if (v4) {
#pragma unroll 4
                for (int k = threadIdx.x * 4; k < K; k += 1024) {
                    const float4 v = *reinterpret_cast<const float4*>(ar + k);
                    ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
                }
            } else {
                for (int k = threadIdx.x; k < K; k += blockDim.x) ss += ar[k] * ar[k];
            }
            ss = warp_sum(ss);
            if (lane == 0) rss[r][warp] = ss;
        }
        __syncthreads();
    }
    for (int r = 0; r < M; ++r) {
        float sc = 1.f;
        if (norm_gain) {
            float ss = 0.f;
            for (int w = 0; w < 8; ++w) ss += rss[r][w];
            sc = (gvec ? 1.f : norm_gain[0]) / sqrtf(ss / (float)K + eps);
        }
        const bool gv = norm_gain && gvec;
        const float* ar = A + (size_t)r * lda;
        __nv_bfloat16* xr = xs + (size_t)r * Kp;
        if (v4) {
#pragma unroll 4
            for (int k = threadIdx.x * 4; k < K; k += 1024) {
                float4 v = *reinterpret_cast<const float4*>(ar + k);
                if (gv) {
                    const float4 gn = *reinterpret_cast<const float4*>(norm_gain + k);
                    v.x *= gn.x; v.y *= gn.y; v.z *= gn.z; v.w *= gn.w;
                }
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * sc, v.y * sc), hi = __floats2bfloat162_rn(v.z * sc, v.w * sc);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(xr + k) = pk;
            }
        } else {
            for (int k = threadIdx.x; k < K; k += blockDim.x) xr[k] = __float2bfloat16_rn(ar[k] * (gv ? norm_gain[k] : 1.f) * sc);
        }
    }
    __syncthreads();
    constexpr int UNR = GLU ? 4 : 8;   // chunks whose weight loads are in flight together (16-byte loads a lane: 2 or 4 a chunk)
    // when chunks may be skipped the warps take the chunks in turn (every warp gets its share of every expert) instead of one range each
    const int cstep = kskip.used ? 8 : 1, c0 = kskip.used ? warp : c_begin, c1 = kskip.used ? NC : c_end;
    for (int n0 = blockIdx.x * kMmaCols; n0 < N; n0 += gridDim.x * kMmaCols) {
        if (!expert_range_used(nskip, n0, min(n0 + kMmaCols, N) - 1)) continue;   // (uniform over the block)
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
        const __nv_bfloat16* w0 = W + (size_t)min(n0 + g, N - 1) * K + 8 * t;
        const __nv_bfloat16* w1 = W + (size_t)min(n0 + g + 8, N - 1) * K + 8 * t;
        const size_t up = (size_t)glu_ff * K;
        const __nv_bfloat16* xr = xs + (size_t)g * Kp + 8 * t;
        for (int c = c0; c < c1; c += UNR * cstep) {
            uint4 ra[UNR], rb[UNR], ua[GLU ? UNR : 1], ub[GLU ? UNR : 1];
            bool on[UNR];
#pragma unroll
            for (int q = 0; q < UNR; ++q) {
                const int cc = c + q * cstep;
                on[q] = cc < c1 && expert_range_used(kskip, cc * 32, cc * 32 + 31);
                if (on[q]) {
                    const int k = cc * 32;
                    ra[q] = *reinterpret_cast<const uint4*>(w0 + k);
                    rb[q] = *reinterpret_cast<const uint4*>(w1 + k);
                    if (GLU) {
                        ua[q] = *reinterpret_cast<const uint4*>(w0 + up + k);
                        ub[q] = *reinterpret_cast<const uint4*>(w1 + up + k);
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < UNR; ++q)
                if (on[q]) {
                    uint4 x = make_uint4(0u, 0u, 0u, 0u);
                    if (g < M) x = *reinterpret_cast<const uint4*>(xr + (c + q * cstep) * 32);
                    mma_bf16_16816(acc, ra[q].x, rb[q].x, ra[q].y, rb[q].y, x.x, x.y);
                    mma_bf16_16816(acc, ra[q].z, rb[q].z, ra[q].w, rb[q].w, x.z, x.w);
                    if (GLU) {
                        mma_bf16_16816(acc2, ua[q].x, ub[q].x, ua[q].y, ub[q].y, x.x, x.y);
                        mma_bf16_16816(acc2, ua[q].z, ub[q].z, ua[q].w, ub[q].w, x.z, x.w);
                    }
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            red[(warp * 2 + 0) * 128 + lane * 4 + i] = acc[i];
            if (GLU) red[(warp * 2 + 1) * 128 + lane * 4 + i] = acc2[i];
        }
        __syncthreads();
        if (threadIdx.x < 128) {   // element (tile column j, row r) sits in lane (j % 8) * 4 + r / 2, register (j / 8) * 2 + r % 2
            const int j = threadIdx.x >> 3, r = threadIdx.x & 7;
            const int src = (((j & 7) << 2) + (r >> 1)) * 4 + ((j >> 3) << 1) + (r & 1);
            float v = 0.f, v2 = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                v += red[(w * 2 + 0) * 128 + src];
                if (GLU) v2 += red[(w * 2 + 1) * 128 + src];
            }
            if (r < M && n0 + j < N) C[(size_t)r * ldc + n0 + j] = GLU ? ff_act(v, glu_act) * v2 : epi_apply(v, epi, alpha, beta);
        }
        __syncthreads();
    }
}

// The five input products of the wkv mixer for few rows in ONE launch: r, k, v, g and the decay's first matrix each read their
// own token-shift mix x_s = h + (prev - h) * mu_s, so a block works on one of the five products, builds that product's mix of
// the rows in shared memory (no mixes in global memory) and streams its share of that product's weight rows.
struct WkvFrontArgs {
    const float* h;      // [T][D] mixer input rows
    const float* mu;     // [5][D]: r, k, v, g, w
    const float* prev;   // [slots][D]: the mixer input of each sequence's last row of the step before
    const void* W[5];
    float* out[5];       // [T][N[s]]
    int N[5], epi[5];
    int blk0[6];         // blocks blk0[s] .. blk0[s + 1] - 1 work on product s
    int D;
};
template <typename WT>
__global__ void __launch_bounds__(kRowGemvThreads, 2) wkv_front_rows_kernel(WkvFrontArgs a, StepMeta m) {
    extern __shared__ __align__(16) float xs[];   // [T][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    pdl_launch_dependents();
    int s = 0;
    while (s < 4 && (int)blockIdx.x >= a.blk0[s + 1]) ++s;
    const int b = blockIdx.x - a.blk0[s], nb = a.blk0[s + 1] - a.blk0[s];
    const WT* W = reinterpret_cast<const WT*>(a.W[s]);
    const int N = a.N[s], K = a.D, M = m.T;
    {
        const int n = b * nw + warp;
        if (n < N) {
            const char* w = reinterpret_cast<const char*>(W + (size_t)n * K);
            for (size_t o = (size_t)lane * 128; o < (size_t)K * sizeof(WT); o += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(w + o));
        }
    }
    pdl_wait_prior_grid();
    const float* mu = a.mu + (size_t)s * K;
    for (int r = 0; r < M; ++r) {
        const int e = m.row_ent[r];
        const bool first = (r == m.ent_row0[e]);
        const float* pr = first ? (m.ent_pos0[e] > 0 ? a.prev + (size_t)m.ent_slot[e] * K : nullptr) : a.h + (size_t)(r - 1) * K;
        const float* hr = a.h + (size_t)r * K;
        if (K % 4 == 0) {   // (all row bases are 16-byte aligned then: allocations, and rows K floats apart)
#pragma unroll 2
            for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
                const float4 hv = *reinterpret_cast<const float4*>(hr + k), mv = *reinterpret_cast<const float4*>(mu + k);
                const float4 pv = pr ? *reinterpret_cast<const float4*>(pr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 o;
                o.x = act_round<WT>(fmaf(pv.x - hv.x, mv.x, hv.x));
                o.y = act_round<WT>(fmaf(pv.y - hv.y, mv.y, hv.y));
                o.z = act_round<WT>(fmaf(pv.z - hv.z, mv.z, hv.z));
                o.w = act_round<WT>(fmaf(pv.w - hv.w, mv.w, hv.w));
                *reinterpret_cast<float4*>(xs + (size_t)r * K + k) = o;
            }
        } else {
            for (int k = threadIdx.x; k < K; k += blockDim.x) {
                const float hv = hr[k];
                const float df = (pr ? pr[k] : 0.f) - hv;
                xs[(size_t)r * K + k] = act_round<WT>(fmaf(df, mu[k], hv));
            }
        }
    }
    __syncthreads();
    const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
    float acc[kRowGemvMaxRows];
    for (int n = b * nw + warp; n < N; n += nb * nw) {
        gemv_row_dot<WT>(W + (size_t)n * K, xs, M, K, vec, lane, acc);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < kRowGemvMaxRows; ++r)
                if (r < M) a.out[s][(size_t)r * N + n] = epi_apply(acc[r], a.epi[s], 1.f);
        }
    }
}

// ---- attention -------------------------------------------------------------------------------------------------------
struct AttnShape {
    int heads, kv_heads, dim, vdim;   // H, G, d, dv
    int window;                       // a row at position p sees positions p - window + 1 .. p (0: all of 0 .. p)
    int rot_dims;                     // leading coordinates of a head that are rotated, in pairs (2i, 2i + 1)
    int qk_norm, out_gate;
    float scale, eps;
    int ld;                           // row stride of the fused projection output [q | k | v | gate]
    int v_ld;                         // token stride of the value pool; 0: kv_heads * vdim.  A cache whose values are the leading
                                      // coordinates of its key rows passes the key pool as the value pool and the key stride here.
    const float* sink;                // [heads] or null: the softmax denominator gains exp(sink[h]), a term without key or value
    // read by the head-mixing kernel only (seq_headmix.cuh); the step sends a layer there when one of them is set
    float softcap;                    // > 0: score <- cap * tanh(score / cap) after scaling
    int keep_first;                   // with a window: keys at positions < keep_first stay visible
    const float* talk;                // [heads][heads] or null: score_h <- sum_g talk[h][g] score_g before masking
    // read by attn_prepare_kernel: what happens to the projections before they are used / cached
    int rot_half;                     // 1: rotated coordinate i pairs with i + rot_dims / 2 instead of (2 i, 2 i + 1)
    int v_norm;                       // 1: every value head is divided by its RMS (no weight) before it is cached
    const float* bias;                // [ld columns of q | k | v] or null: added to the projections first
    const float* temp;                // [heads] or null: query head h is multiplied by temp[h] (a per-head factor of its scores)
    // the output gate's pre-activations when they are not part of the fused projection: gate[t * gate_ld + h] (null: behind q | k | v)
    const float* gate;
    int gate_ld;
};
// sigmoid output gate of (row t, head h), 1 without a gate
__device__ __forceinline__ float attn_gate(const AttnShape& s, const float* qkvg, int t, int h) {
    if (!s.out_gate) return 1.f;
    const float z = s.gate ? s.gate[(size_t)t * s.gate_ld + h]
                           : qkvg[(size_t)t * s.ld + (size_t)(s.heads + s.kv_heads) * s.dim + (size_t)s.kv_heads * s.vdim + h];
    return 1.f / (1.f + expf(-z));
}
__device__ __forceinline__ size_t attn_vstride(const AttnShape& s) { return s.v_ld ? (size_t)s.v_ld : (size_t)s.kv_heads * s.vdim; }
// the end of a softmax with a sink: (max, sum) -> the factor for the accumulated weighted values
__device__ __forceinline__ float attn_finish_factor(const AttnShape& s, int h, float mx, float l) {
    if (!s.sink) return 1.f / l;
    const float sk = s.sink[h], m2 = fmaxf(mx, sk), c = expf(mx - m2);
    return c / (l * c + expf(sk - m2));
}
// Biases, rotation of q and k, unit RMS per head, the per-head query factor, unit-RMS values and the cache append: one block per
// row.  q is rewritten in place; k and v go to the row's page.  inv_freq[rot_dims / 2] holds the (scaled) frequencies; the angle is
// position * frequency in fp32.  Pair i of the rotated coordinates is (2 i, 2 i + 1) or, with rot_half, (i, i + rot_dims / 2).
__global__ void attn_prepare_kernel(float* qkvg, StepMeta m, AttnShape s, const float* inv_freq, float* k_pool, float* v_pool) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    const int t = blockIdx.x;
    const int pos = m.row_pos[t];
    const int slot = m.ent_slot[m.row_ent[t]];
    const int page = m.page_table[(size_t)slot * m.table_stride + pos / kPageTokens];
    const size_t tok_off = (size_t)page * kPageTokens + pos % kPageTokens;
    float* row = qkvg + (size_t)t * s.ld;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int nqk = s.heads + s.kv_heads, half = s.rot_dims / 2;
    for (int h = warp; h < nqk; h += nw) {
        float* v = row + (size_t)h * s.dim;   // q heads first, k heads right behind them
        const float* b = s.bias ? s.bias + (size_t)h * s.dim : nullptr;
        float ss = 0.f;
        for (int i = lane; i < half; i += 32) {
            const int i0 = s.rot_half ? i : 2 * i, i1 = s.rot_half ? i + half : 2 * i + 1;
            const float a = v[i0] + (b ? b[i0] : 0.f), c = v[i1] + (b ? b[i1] : 0.f);
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            const float ra = a * cs - c * sn, rc = c * cs + a * sn;
            v[i0] = ra;
            v[i1] = rc;
            ss += ra * ra + rc * rc;
        }
        for (int i = 2 * half + lane; i < s.dim; i += 32) {
            const float a = v[i] + (b ? b[i] : 0.f);
            v[i] = a;
            ss += a * a;
        }
        ss = warp_sum(ss);
        float sc = s.qk_norm ? 1.f / sqrtf(ss / (float)s.dim + s.eps) : 1.f;
        __syncwarp();
        if (h < s.heads) {
            if (s.temp) sc *= s.temp[h];
            if (s.qk_norm || s.temp)
                for (int i = lane; i < s.dim; i += 32) v[i] *= sc;
        } else {
            float* kd = k_pool + tok_off * (size_t)(s.kv_heads * s.dim) + (size_t)(h - s.heads) * s.dim;
            for (int i = lane; i < s.dim; i += 32) kd[i] = v[i] * sc;
        }
    }
    const float* vs = row + (size_t)nqk * s.dim;
    const float* vb = s.bias ? s.bias + (size_t)nqk * s.dim : nullptr;
    float* vd = v_pool + tok_off * (size_t)(s.kv_heads * s.vdim);
    if (s.v_norm) {
        for (int g = warp; g < s.kv_heads; g += nw) {
            float ss = 0.f;
            for (int i = lane; i < s.vdim; i += 32) {
                const float a = vs[g * s.vdim + i] + (vb ? vb[g * s.vdim + i] : 0.f);
                ss += a * a;
            }
            const float sc = 1.f / sqrtf(warp_sum(ss) / (float)s.vdim + s.eps);
            for (int i = lane; i < s.vdim; i += 32) vd[g * s.vdim + i] = (vs[g * s.vdim + i] + (vb ? vb[g * s.vdim + i] : 0.f)) * sc;
        }
    } else {
        for (int i = threadIdx.x; i < s.kv_heads * s.vdim; i += blockDim.x) vd[i] = vs[i] + (vb ? vb[i] : 0.f);
    }
}

// Softmax attention of one (row, query head) over the keys its window allows, read from the paged cache: 4 warps share the
// keys, a lane owns coordinates lane, lane + 32, ...; online softmax per warp, merged through shared memory.  The output is
// multiplied by sigmoid(gate) of its head.  out[t][h * dv ..].
constexpr int kAttnWarps = 4;
constexpr int kAttnMaxPerLane = 8;   // head sizes up to 256
constexpr int kAttnWidePerLane = 20; // the wide instantiation: head sizes up to 640 (a low-rank cache row with its rotated part)
template <int PL>
__global__ void __launch_bounds__(kAttnWarps * 32) window_attention_kernel(const float* qkvg, StepMeta m, AttnShape s, const int* rows,
                                                                            const float* k_pool, const float* v_pool, float* out) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    extern __shared__ float sm[];   // [kAttnWarps][dv] partial outputs, then [kAttnWarps] max, [kAttnWarps] sum
    const int t = rows ? rows[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = m.row_pos[t];
    const int slot = m.ent_slot[m.row_ent[t]];
    const int* table = m.page_table + (size_t)slot * m.table_stride;
    const int g = h / (s.heads / s.kv_heads);
    const float* q = qkvg + (size_t)t * s.ld + (size_t)h * s.dim;
    float qr[PL], o[PL];
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < s.dim ? q[d] : 0.f;
        o[i] = 0.f;
    }
    const int lo = (s.window > 0 && pos - s.window + 1 > 0) ? pos - s.window + 1 : 0;
    float mx = -INFINITY, l = 0.f;
    const size_t kstride = (size_t)s.kv_heads * s.dim, vstride = attn_vstride(s);
    for (int j = lo + warp; j <= pos; j += kAttnWarps) {
        const size_t off = (size_t)table[j / kPageTokens] * kPageTokens + j % kPageTokens;
        const float* kr = k_pool + off * kstride + (size_t)g * s.dim;
        float sc = 0.f;
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int d = lane + 32 * i;
            if (d < s.dim) sc = fmaf(qr[i], kr[d], sc);
        }
        sc = warp_sum(sc) * s.scale;
        const float nm = fmaxf(mx, sc);
        const float corr = expf(mx - nm), p = expf(sc - nm);
        l = l * corr + p;
        const float* vr = v_pool + off * vstride + (size_t)g * s.vdim;
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int d = lane + 32 * i;
            if (d < s.vdim) o[i] = fmaf(p, vr[d], o[i] * corr);
        }
        mx = nm;
    }
    float* po = sm;
    float* pm = sm + kAttnWarps * s.vdim;
    float* pl = pm + kAttnWarps;
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int d = lane + 32 * i;
        if (d < s.vdim) po[warp * s.vdim + d] = o[i];
    }
    if (lane == 0) {
        pm[warp] = mx;
        pl[warp] = l;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, pm[w]);
    float L = 0.f, f[kAttnWarps];
    for (int w = 0; w < kAttnWarps; ++w) {
        f[w] = (pm[w] == -INFINITY) ? 0.f : expf(pm[w] - M);
        L += pl[w] * f[w];
    }
    const float fin = attn_finish_factor(s, h, M, L) * attn_gate(s, qkvg, t, h);
    for (int d = threadIdx.x; d < s.vdim; d += blockDim.x) {
        float acc = 0.f;
        for (int w = 0; w < kAttnWarps; ++w) acc += po[w * s.vdim + d] * f[w];
        out[(size_t)t * (s.heads * s.vdim) + (size_t)h * s.vdim + d] = acc * fin;
    }
}

// The same attention for prompt portions: a block owns up to 64 consecutive rows of ONE sequence and one query head, walks the
// key pages its rows can see (a page = a 64-key tile, fetched once per block), and does both products as register-tiled fp32
// loops out of shared memory: S = Q K^T (4 x 4 scores a thread), masking and online softmax per row across the 16 threads that
// share it, O += P V.  Head sizes must be multiples of 4; tiles[2 i] = first row, tiles[2 i + 1] = row count.
constexpr int kAttnTile = 64;
template <int DV4>   // float4 column groups of the output a thread owns: ceil(dv / 64)
__global__ void __launch_bounds__(256) window_attention_tiled_kernel(const float* qkvg, StepMeta m, AttnShape s, const int* tiles,
                                                                      const float* k_pool, const float* v_pool, float* out) {
    extern __shared__ __align__(16) float smt[];
    const int d = s.dim, dv = s.vdim, ldq = d + 4, ldp = kAttnTile + 4;
    // a cache whose values are the leading coordinates of its key rows (one key/value head): the value tile IS the key tile
    const bool v_in_k = (v_pool == k_pool) && s.kv_heads == 1 && s.v_ld == s.dim && dv <= d;
    const int ldvs = v_in_k ? ldq : dv;
    float* Qs = smt;
    float* Ks = Qs + kAttnTile * ldq;
    float* Vs = v_in_k ? Ks : Ks + kAttnTile * ldq;
    float* Ps = Vs + (v_in_k ? kAttnTile * ldq : kAttnTile * dv);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int row0 = tiles[2 * blockIdx.x], n = tiles[2 * blockIdx.x + 1], h = blockIdx.y;
    const int p0 = m.row_pos[row0];
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[row0]] * m.table_stride;
    const int g = h / (s.heads / s.kv_heads);
    for (int i = tid; i < kAttnTile * d; i += 256) {
        const int r = i / d, k = i % d;
        Qs[r * ldq + k] = r < n ? qkvg[(size_t)(row0 + r) * s.ld + (size_t)h * d + k] : 0.f;
    }
    const int lo = (s.window > 0 && p0 - s.window + 1 > 0) ? p0 - s.window + 1 : 0, hi = p0 + n - 1;
    float mrow[4], lrow[4], acc[4][DV4 * 4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        mrow[i] = -INFINITY;
        lrow[i] = 0.f;
#pragma unroll
        for (int j = 0; j < DV4 * 4; ++j) acc[i][j] = 0.f;
    }
    const size_t kstride = (size_t)s.kv_heads * d, vstride = attn_vstride(s);
    for (int pg = lo / kPageTokens; pg <= hi / kPageTokens; ++pg) {
        __syncthreads();
        const size_t tok0 = (size_t)table[pg] * kPageTokens;
        const float* kb = k_pool + tok0 * kstride + (size_t)g * d;
        const float* vb = v_pool + tok0 * vstride + (size_t)g * dv;
        for (int i = tid; i < kAttnTile * (d / 4); i += 256) {
            const int c = i / (d / 4), k4 = (i % (d / 4)) * 4, key = pg * kPageTokens + c;
            const float4 v = (key >= lo && key <= hi) ? *reinterpret_cast<const float4*>(kb + (size_t)c * kstride + k4) : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(&Ks[c * ldq + k4]) = v;
        }
        for (int i = tid; i < (v_in_k ? 0 : kAttnTile * (dv / 4)); i += 256) {
            const int c = i / (dv / 4), k4 = (i % (dv / 4)) * 4, key = pg * kPageTokens + c;
            const float4 v = (key >= lo && key <= hi) ? *reinterpret_cast<const float4*>(vb + (size_t)c * vstride + k4) : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(&Vs[c * dv + k4]) = v;
        }
        __syncthreads();
        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
        for (int k = 0; k < d; k += 4) {
            float4 qa[4], kk[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qa[i] = *reinterpret_cast<const float4*>(&Qs[(ty + 16 * i) * ldq + k]);
#pragma unroll
            for (int j = 0; j < 4; ++j) kk[j] = *reinterpret_cast<const float4*>(&Ks[(tx + 16 * j) * ldq + k]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    sc[i][j] = fmaf(qa[i].x, kk[j].x, fmaf(qa[i].y, kk[j].y, fmaf(qa[i].z, kk[j].z, fmaf(qa[i].w, kk[j].w, sc[i][j]))));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = ty + 16 * i, pos = p0 + r;
            bool ok[4];
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int key = pg * kPageTokens + tx + 16 * j;
                ok[j] = r < n && key <= pos && (s.window <= 0 || key > pos - s.window);
                sc[i][j] = ok[j] ? sc[i][j] * s.scale : -INFINITY;
                tmax = fmaxf(tmax, sc[i][j]);
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, o));
            const float nm = fmaxf(mrow[i], tmax);
            const float corr = (nm == -INFINITY) ? 1.f : expf(mrow[i] - nm);
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float pj = ok[j] ? expf(sc[i][j] - nm) : 0.f;
                Ps[r * ldp + tx + 16 * j] = pj;
                psum += pj;
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) psum += __shfl_xor_sync(0xFFFFFFFFu, psum, o);
            lrow[i] = lrow[i] * corr + psum;
            mrow[i] = nm;
#pragma unroll
            for (int j = 0; j < DV4 * 4; ++j) acc[i][j] *= corr;
        }
        __syncthreads();
        for (int c = 0; c < kAttnTile; c += 4) {
            float4 pr[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pr[i] = *reinterpret_cast<const float4*>(&Ps[(ty + 16 * i) * ldp + c]);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
                for (int jj = 0; jj < DV4; ++jj) {
                    const int col = tx * 4 + 64 * jj;
                    if (col < dv) {
                        const float4 v = *reinterpret_cast<const float4*>(&Vs[(c + cc) * ldvs + col]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float p = cc == 0 ? pr[i].x : cc == 1 ? pr[i].y : cc == 2 ? pr[i].z : pr[i].w;
                            acc[i][jj * 4 + 0] = fmaf(p, v.x, acc[i][jj * 4 + 0]);
                            acc[i][jj * 4 + 1] = fmaf(p, v.y, acc[i][jj * 4 + 1]);
                            acc[i][jj * 4 + 2] = fmaf(p, v.z, acc[i][jj * 4 + 2]);
                            acc[i][jj * 4 + 3] = fmaf(p, v.w, acc[i][jj * 4 + 3]);
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty + 16 * i;
        if (r >= n) continue;
        const int t = row0 + r;
        const float f = attn_gate(s, qkvg, t, h) * attn_finish_factor(s, h, mrow[i], lrow[i]);
#pragma unroll
        for (int jj = 0; jj < DV4; ++jj) {
            const int col = tx * 4 + 64 * jj;
            if (col < dv) {
                float* o = out + (size_t)t * (s.heads * dv) + (size_t)h * dv + col;
                o[0] = acc[i][jj * 4 + 0] * f;
                o[1] = acc[i][jj * 4 + 1] * f;
                o[2] = acc[i][jj * 4 + 2] * f;
                o[3] = acc[i][jj * 4 + 3] * f;
            }
        }
    }
}
inline size_t attn_tiled_smem_bytes(int d, int dv, bool v_in_k = false) {
    return sizeof(float) * ((size_t)2 * kAttnTile * (d + 4) + (v_in_k ? 0 : (size_t)kAttnTile * dv) + (size_t)kAttnTile * (kAttnTile + 4));
}

// ---- gated feed-forward: act(gate) * up over the fused projection output [gate | up] ------------------------------------
enum { ACT_RELU = 0, ACT_SILU = 1, ACT_GELU_TANH = 2 };
__device__ __forceinline__ float ff_act(float z, int act) {
    if (act == 0 /*ACT_RELU*/) return fmaxf(z, 0.f);
    if (act == 1 /*ACT_SILU*/) return z / (1.f + expf(-z));
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__global__ void glu_kernel(const float* gu, int ff, int act, float* y, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / ff, c = i % ff;
        y[i] = ff_act(gu[t * 2 * ff + c], act) * gu[t * 2 * ff + ff + c];
    }
}

// ---- token-shifted linear recurrence (wkv) ----------------------------------------------------------------------------
// mixes[s][t] = h[t] + (prev[t] - h[t]) * mu[s], s = r, k, v, g, w; prev is the row before within the entry, the slot's
// saved row for an entry's first row, zeros at position 0.
__global__ void wkv_mix_kernel(const float* h, StepMeta m, int D, const float* mu /*[5][D]*/, const float* prev_state /*[slots][D]*/,
                               float* mixes /*[5][T][D]*/) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    const int t = blockIdx.x;
    const int e = m.row_ent[t];
    const bool first = (t == m.ent_row0[e]);
    const float* pr = first ? (m.ent_pos0[e] > 0 ? prev_state + (size_t)m.ent_slot[e] * D : nullptr) : h + (size_t)(t - 1) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float hv = h[(size_t)t * D + d];
        const float df = (pr ? pr[d] : 0.f) - hv;
#pragma unroll
        for (int s = 0; s < 5; ++s) mixes[((size_t)s * m.T + t) * D + d] = fmaf(df, mu[(size_t)s * D + d], hv);
    }
}
// the slot keeps the mixer input of the entry's last row for the next step
__global__ void wkv_save_prev_kernel(const float* h, StepMeta m, int D, float* prev_state) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    const int e = blockIdx.x;
    const int t = m.ent_row0[e + 1] - 1;
    for (int d = threadIdx.x; d < D; d += blockDim.x) prev_state[(size_t)m.ent_slot[e] * D + d] = h[(size_t)t * D + d];
}
// The recurrence of one (entry, head), token by token: thread j owns column j of the state S [d][d] (key channel i, value
// channel j).  o_j = sum_i r_i (S_ij + u_i k_i v_j); S_ij <- w_i S_ij + k_i v_j with w = exp(-exp(z + w0)).  The raw o goes to
// `out`; wkv_finish_kernel divides every head's o by its RMS and applies channel weights and gate (that reduction is
// independent of the scan, so it stays out of the sequential loop).
struct WkvArgs {
    const float *r, *k, *v, *z;           // [T][H * d] each
    const float *w0, *u;                  // [H * d]
    float* state;                         // [slots][H][d][d]
    float* out;                           // [T][H * d] raw o
    int heads, dim;
    int s_in_smem;
};
// any head size: S in shared memory while the entry's rows run (in global memory directly when it does not fit)
__global__ void wkv_scan_kernel(WkvArgs a, StepMeta m) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    extern __shared__ float sm[];
    const int e = blockIdx.x, hd = blockIdx.y, d = a.dim, j = threadIdx.x;
    const int C = a.heads * d;
    float* rs = sm;            // r_i
    float* ks = rs + d;        // k_i
    float* ws = ks + d;        // decay_i
    float* us = ws + d;        // u_i * k_i
    float* Sg = a.state + ((size_t)m.ent_slot[e] * a.heads + hd) * (size_t)d * d;
    float* S = a.s_in_smem ? us + d : Sg;
    const bool fresh = (m.ent_pos0[e] == 0);
    if (j < d) {
        if (a.s_in_smem)
            for (int i = 0; i < d; ++i) S[i * d + j] = fresh ? 0.f : Sg[i * d + j];
        else if (fresh)
            for (int i = 0; i < d; ++i) S[i * d + j] = 0.f;
    }
    const int t0 = m.ent_row0[e], t1 = m.ent_row0[e + 1];
    for (int t = t0; t < t1; ++t) {
        const size_t base = (size_t)t * C + (size_t)hd * d;
        __syncthreads();
        if (j < d) {
            const float kv = a.k[base + j];
            rs[j] = a.r[base + j];
            ks[j] = kv;
            ws[j] = expf(-expf(a.z[base + j] + a.w0[hd * d + j]));
            us[j] = a.u[hd * d + j] * kv;
        }
        __syncthreads();
        if (j < d) {
            float acc = 0.f;
            const float vj = a.v[base + j];
            for (int i = 0; i < d; ++i) {
                const float s = S[i * d + j];
                acc = fmaf(rs[i], fmaf(us[i], vj, s), acc);
                S[i * d + j] = fmaf(ws[i], s, ks[i] * vj);
            }
            a.out[base + j] = acc;
        }
    }
    if (a.s_in_smem && j < d) {
        __syncthreads();
        for (int i = 0; i < d; ++i) Sg[i * d + j] = S[i * d + j];
    }
}
// head sizes 32 / 64 / 128: a BLOCK owns 32 value columns of a head (grid z = column group); its NW warps split the key
// channels, so a lane keeps D / NW entries of its state column in registers and a token costs D / NW multiply-adds a lane
// instead of D.  Tokens are taken CH at a time: the block puts the chunk's r / k / decay / u k vectors and its v columns into
// shared memory (decays and u k computed there once), requests the NEXT chunk's operands from memory, and then every warp runs
// the chunk's tokens back to back over its key channels and leaves a partial output per token; the partials of the NW warps
// are summed (in warp order, so the result does not depend on timing) while the next chunk is staged.  Two block barriers a chunk.
template <int D, int CH, int NW>
__global__ void __launch_bounds__(32 * NW) wkv_scan_split_kernel(WkvArgs a, StepMeta m) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    constexpr int RP = D / NW;          // key channels a warp owns
    constexpr int NT = 32 * NW;
    constexpr int PER = CH * D / NT;    // operands of each kind a thread stages per chunk
    constexpr int VPER = (CH * 32 + NT - 1) / NT;
    static_assert(D % NW == 0 && RP % 4 == 0 && (CH * D) % NT == 0, "chunk staging must divide evenly");
    __shared__ __align__(16) float buf[CH][4][D];
    __shared__ float vbuf[CH][32];
    __shared__ float part[NW][CH][32];
    const int e = blockIdx.x, hd = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col0 = blockIdx.z * 32, j = col0 + lane;
    const int C = a.heads * D;
    float* Sg = a.state + ((size_t)m.ent_slot[e] * a.heads + hd) * (size_t)D * D;
    float S[RP];
    const bool fresh = (m.ent_pos0[e] == 0);
#pragma unroll
    for (int i = 0; i < RP; ++i) S[i] = fresh ? 0.f : Sg[(size_t)(warp * RP + i) * D + j];
    float w0[PER], u[PER];
#pragma unroll
    for (int p = 0; p < PER; ++p) {
        const int i = (tid + NT * p) % D;
        w0[p] = a.w0[hd * D + i];
        u[p] = a.u[hd * D + i];
    }
    const int t0 = m.ent_row0[e], t1 = m.ent_row0[e + 1];
    float nr[PER], nk[PER], nz[PER], nv[VPER];
    auto fetch = [&](int tc) {
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int q = tid + NT * p, c = q / D, i = q % D;
            const size_t base = (size_t)min(tc + c, t1 - 1) * C + (size_t)hd * D + i;
            nr[p] = a.r[base];
            nk[p] = a.k[base];
            nz[p] = a.z[base];
        }
#pragma unroll
        for (int p = 0; p < VPER; ++p) {
            const int q = tid + NT * p, c = q >> 5, l = q & 31;
            nv[p] = c < CH ? a.v[(size_t)min(tc + c, t1 - 1) * C + (size_t)hd * D + col0 + l] : 0.f;
        }
    };
    auto emit = [&](int tc) {   // out[t][j] = sum over the warps' partials, chunk starting at row tc
        for (int q = tid; q < CH * 32; q += NT) {
            const int c = q >> 5, l = q & 31;
            if (tc + c < t1) {
                float s = part[0][c][l];
#pragma unroll
                for (int w = 1; w < NW; ++w) s += part[w][c][l];
                a.out[(size_t)(tc + c) * C + (size_t)hd * D + col0 + l] = s;
            }
        }
    };
    fetch(t0);
    for (int tc = t0; tc < t1; tc += CH) {
        if (tc > t0) emit(tc - CH);
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int q = tid + NT * p, c = q / D, i = q % D;
            buf[c][0][i] = nr[p];
            buf[c][1][i] = nk[p];
            buf[c][2][i] = expf(-expf(nz[p] + w0[p]));
            buf[c][3][i] = u[p] * nk[p];
        }
#pragma unroll
        for (int p = 0; p < VPER; ++p) {
            const int q = tid + NT * p;
            if (q < CH * 32) vbuf[q >> 5][q & 31] = nv[p];
        }
        __syncthreads();
        if (tc + CH < t1) fetch(tc + CH);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            if (tc + c < t1) {
                float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
                const float v = vbuf[c][lane];
#pragma unroll
                for (int i = 0; i < RP; i += 4) {
                    const int ch = warp * RP + i;
                    const float4 r4 = *reinterpret_cast<const float4*>(&buf[c][0][ch]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&buf[c][1][ch]);
                    const float4 w4 = *reinterpret_cast<const float4*>(&buf[c][2][ch]);
                    const float4 u4 = *reinterpret_cast<const float4*>(&buf[c][3][ch]);
                    acc0 = fmaf(r4.x, fmaf(u4.x, v, S[i]), acc0);
                    S[i] = fmaf(w4.x, S[i], k4.x * v);
                    acc1 = fmaf(r4.y, fmaf(u4.y, v, S[i + 1]), acc1);
                    S[i + 1] = fmaf(w4.y, S[i + 1], k4.y * v);
                    acc2 = fmaf(r4.z, fmaf(u4.z, v, S[i + 2]), acc2);
                    S[i + 2] = fmaf(w4.z, S[i + 2], k4.z * v);
                    acc3 = fmaf(r4.w, fmaf(u4.w, v, S[i + 3]), acc3);
                    S[i + 3] = fmaf(w4.w, S[i + 3], k4.w * v);
                }
                part[warp][c][lane] = (acc0 + acc1) + (acc2 + acc3);
            }
        }
        __syncthreads();
    }
    emit(t0 + (t1 - t0 - 1) / CH * CH);
#pragma unroll
    for (int i = 0; i < RP; ++i) Sg[(size_t)(warp * RP + i) * D + j] = S[i];
}
// o[t, head] / rms(o[t, head]) * normw * gate, in place: one warp per (row, head).  d = the head's output size; normw is
// [heads][d] (w_heads = 1) or one [d] vector shared by the heads (w_heads = 0); gate (optional) has row stride gate_ld and is
// used as it is (gate_silu = 0) or through z * sigmoid(z) (gate_silu = 1).
__global__ void head_rmsnorm_gate_kernel(float* o, const float* gate, int gate_ld, int gate_silu, const float* normw, int w_heads, int T, int heads, int d,
                                         float eps) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T * heads) return;
    const int hd = warp % heads, t = warp / heads;
    const size_t base = (size_t)t * heads * d + (size_t)hd * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss += o[base + i] * o[base + i];
    ss = warp_sum(ss);
    const float sc = 1.f / sqrtf(ss / (float)d + eps);
    for (int i = lane; i < d; i += 32) {
        float g = 1.f;
        if (gate) {
            g = gate[(size_t)t * gate_ld + (size_t)hd * d + i];
            if (gate_silu) g = g / (1.f + expf(-g));
        }
        o[base + i] = o[base + i] * sc * normw[(w_heads ? hd * d : 0) + i] * g;
    }
}

// ---- helpers -----------------------------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* x, const int* rows, int D, float* y) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) y[(size_t)t * D + d] = x[(size_t)rows[t] * D + d];
}
// A[M][lda] (fp32) -> Y[M][K] (bf16, dense rows), four elements a thread; K a multiple of 4
__global__ void rows_to_bf16_kernel(const float* A, int lda, int M, int K, __nv_bfloat16* y) {
    const size_t n4 = (size_t)M * (K / 4);
    const bool vec = (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / (K / 4), c = (i % (K / 4)) * 4;
        const float* src = A + r * lda + c;
        float4 v;
        if (vec) v = *reinterpret_cast<const float4*>(src);
        else v = make_float4(src[0], src[1], src[2], src[3]);
        __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(y + r * K + c);
        d[0] = __floats2bfloat162_rn(v.x, v.y);
        d[1] = __floats2bfloat162_rn(v.z, v.w);
    }
}
__global__ void f32_to_bf16_kernel(const float* x, __nv_bfloat16* y, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) y[i] = __float2bfloat16_rn(x[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* x, float* y, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) y[i] = __bfloat162float(x[i]);
}

}  // namespace seq
}  // namespace tib

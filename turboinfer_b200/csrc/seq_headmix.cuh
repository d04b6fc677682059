// seq_headmix.cuh -- attention of the layered sequence engine whose scores are worked on between the dot product and the
// softmax, and the small stateful pieces that come with such layers:
//
//   * whole-projection query / key norm: q (all heads at once) and k are divided by the RMS over the WHOLE projection and
//     multiplied by a plain per-coordinate weight, then k and v are appended to the row's page (attn_prepare_whole_kernel);
//   * capped, head-mixed, windowed attention with kept first keys and a sink (the mix_* kernels, three passes):
//         s_h(i, j)  = cap * tanh(scale * q_h(i) . k_g(h)(j) / cap)                  (cap <= 0: no cap)
//         s'_h(i, j) = sum_g T[h][g] s_g(i, j)                                       (T null: no mixing)
//         row i sees key j  <=>  j <= i and (window <= 0 or i - j < window or j < keep_first)
//         p_h(i, j)  = exp(s'_h(i, j)) / (sum over seen j' of exp(s'_h(i, j')) + exp(sink_h))   (sink null: no extra term)
//     The mixing needs the scores of ALL heads of a (query, key) pair at once, unlike the per-head kernels of seq_kernels.cuh /
//     seq_attn_tc.cuh, whose softmax runs along with the scores;
//   * a causal depth-wise short convolution over time in front of a mixer, y_t = x_t + sum_j w[:, j] x_(t - taps + 1 + j), whose
//     last taps - 1 inputs are sequence state (short_conv_kernel, short_conv_save_kernel).
//
// Everything here is fp32 in both compute modes: scores, cap, mixing, softmax and the weighted sum of values (in bf16 mode the two
// products of prompt tiles run on the tensor cores over fp16 hi / lo halves of their fp32 operands, which keeps fp32 accuracy).
#pragma once
#include "prefill.cuh"
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

// ---- short convolution ------------------------------------------------------------------------------------------------------------
// state [slots][taps - 1][D]: the inputs at positions len - (taps - 1) .. len - 1 of the slot's sequence, oldest first.  Entries
// for positions before 0 are never read (a slot that is used again needs no clearing).
// An entry that brings ONE row (a decoded token) also shifts its slot's state here: the thread that read a coordinate's old entries
// writes its new ones (short_conv_save_kernel then skips that entry).
template <int V> __device__ __forceinline__ void conv_load(const float* p, float (&v)[V]) {
    if constexpr (V == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
        v[0] = *p;
    }
}
template <int V> __device__ __forceinline__ void conv_store(float* p, const float (&v)[V]) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else *p = v[0];
}
// V = 4: a thread takes four neighbouring coordinates with 16-byte loads and stores (D in whole fours); V = 1: one coordinate at a time.
template <int V>
__global__ void short_conv_kernel(const float* x, StepMeta m, int D, int taps, const float* w, float* state, float* y) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    constexpr int CH = V == 4 ? 4 : 8;   // taps whose inputs are requested together
    const int t = blockIdx.x, e = m.row_ent[t], i = t - m.ent_row0[e], pos0 = m.ent_pos0[e];
    float* st = state + (size_t)m.ent_slot[e] * (taps - 1) * D;
    const bool alone = m.ent_row0[e + 1] - m.ent_row0[e] == 1;
    for (int d = (blockIdx.y * blockDim.x + threadIdx.x) * V; d < D; d += gridDim.y * blockDim.x * V) {
        float xv[V], acc[V];
        conv_load<V>(x + (size_t)t * D + d, xv);
#pragma unroll
        for (int c = 0; c < V; ++c) acc[c] = xv[c];
        // the taps' inputs are requested together (CH at a time), then multiplied in ascending order of the tap
        for (int j0 = 0; j0 < taps; j0 += CH) {
            float v[CH][V], wv[CH][V];
#pragma unroll
            for (int q = 0; q < CH; ++q) {
                const int j = j0 + q, back = taps - 1 - j;
                const bool in_step = i - back >= 0;
                const bool ok = j < taps && (in_step || pos0 + i - back >= 0);
                const float* src = in_step ? x + (size_t)(t - back) * D + d : st + (size_t)(taps - 1 + i - back) * D + d;
                if (ok) conv_load<V>(src, v[q]);
#pragma unroll
                for (int c = 0; c < V; ++c) {
                    if (!ok) v[q][c] = 0.f;
                    wv[q][c] = j < taps ? w[(size_t)(d + c) * taps + j] : 0.f;
                }
            }
#pragma unroll
            for (int q = 0; q < CH; ++q)
                if (j0 + q < taps) {
#pragma unroll
                    for (int c = 0; c < V; ++c) acc[c] = fmaf(wv[q][c], v[q][c], acc[c]);
                }
        }
        conv_store<V>(y + (size_t)t * D + d, acc);
        if (alone) {
            for (int s = 0; s + 2 < taps; ++s) {
                float o[V];
                conv_load<V>(st + (size_t)(s + 1) * D + d, o);
                conv_store<V>(st + (size_t)s * D + d, o);
            }
            if (taps > 1) conv_store<V>(st + (size_t)(taps - 2) * D + d, xv);
        }
    }
}
// Many rows (prompt portions): a block takes R consecutive rows and a thread four neighbouring coordinates (D in whole fours), whose
// weights (taps <= KT) it reads ONCE and keeps in registers, the tap that reaches `back` rows back in entry KT - 1 - back.
// Rows that all lie in one entry, taps - 1 rows or more behind its first: their inputs and those of the taps - 1 rows in front are
// requested together, each once (no state is read or shifted).  Other blocks (an entry's first rows, entries of few rows) go row by
// row.  The arithmetic of a coordinate is that of short_conv_kernel either way: acc = x, then the taps from the oldest input on.
template <int R, int KT>
__global__ void __launch_bounds__(128) short_conv_rows_kernel(const float* __restrict__ x, StepMeta m, int T, int D, int taps, const float* __restrict__ w, float* state, float* __restrict__ y) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int d = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (d >= D) return;
    const int skip = KT - taps;   // entries below it hold no tap
    float wv[KT][4];
#pragma unroll
    for (int q = 0; q < KT; ++q)
#pragma unroll
        for (int c = 0; c < 4; ++c) wv[q][c] = q >= skip ? w[(size_t)(d + c) * taps + q - skip] : 0.f;
    const int t0 = blockIdx.x * R, t1 = min(T, t0 + R);
    const int e0 = m.row_ent[t0];
    if (e0 == m.row_ent[t1 - 1] && t0 - m.ent_row0[e0] >= taps - 1) {
        float xs[R + KT - 1][4];   // rows t0 - (KT - 1) .. t0 + R - 1
#pragma unroll
        for (int r = 0; r < R + KT - 1; ++r) {
            const int t = t0 - (KT - 1) + r;
            if (r >= skip && t < t1) conv_load<4>(x + (size_t)t * D + d, xs[r]);
            else xs[r][0] = xs[r][1] = xs[r][2] = xs[r][3] = 0.f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (t0 + r < t1) {
                float acc[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[c] = xs[r + KT - 1][c];
#pragma unroll
                for (int q = 0; q < KT; ++q)
                    if (q >= skip) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[c] = fmaf(wv[q][c], xs[r + q][c], acc[c]);
                    }
                conv_store<4>(y + (size_t)(t0 + r) * D + d, acc);
            }
        return;
    }
    for (int t = t0; t < t1; ++t) {
        const int e = m.row_ent[t], i = t - m.ent_row0[e], pos0 = m.ent_pos0[e];
        float* st = state + (size_t)m.ent_slot[e] * (taps - 1) * D;
        const bool alone = m.ent_row0[e + 1] - m.ent_row0[e] == 1;
        float xv[4], acc[4], v[KT][4];
        conv_load<4>(x + (size_t)t * D + d, xv);
#pragma unroll
        for (int q = 0; q < KT; ++q) {
            const int back = KT - 1 - q;
            const bool in_step = i - back >= 0;
            const bool ok = q >= skip && (in_step || pos0 + i - back >= 0);
            const float* src = in_step ? x + (size_t)(t - back) * D + d : st + (size_t)(taps - 1 + i - back) * D + d;
            if (ok) conv_load<4>(src, v[q]);
            else v[q][0] = v[q][1] = v[q][2] = v[q][3] = 0.f;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[c] = xv[c];
#pragma unroll
        for (int q = 0; q < KT; ++q)
            if (q >= skip) {
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[c] = fmaf(wv[q][c], v[q][c], acc[c]);
            }
        conv_store<4>(y + (size_t)t * D + d, acc);
        if (alone) {
            for (int s = 0; s + 2 < taps; ++s) {
                float o[4];
                conv_load<4>(st + (size_t)(s + 1) * D + d, o);
                conv_store<4>(st + (size_t)s * D + d, o);
            }
            if (taps > 1) conv_store<4>(st + (size_t)(taps - 2) * D + d, xv);
        }
    }
}
// after all rows of the step have read the old state: the slot keeps the last taps - 1 inputs of its sequence
__global__ void short_conv_save_kernel(const float* x, StepMeta m, int D, int taps, float* state) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int e = blockIdx.x, row0 = m.ent_row0[e], n = m.ent_row0[e + 1] - row0;
    if (n == 1) return;   // (saved by short_conv_kernel)
    float* st = state + (size_t)m.ent_slot[e] * (taps - 1) * D;
    for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x)
        for (int s = 0; s < taps - 1; ++s) {   // ascending: entry n + s is still the old one when it is read
            const int i = n - (taps - 1) + s;
            st[(size_t)s * D + d] = i >= 0 ? x[(size_t)(row0 + i) * D + d] : st[(size_t)(n + s) * D + d];
        }
}

// ---- whole-projection query / key norm and the cache append ------------------------------------------------------------------
// One block per row of the fused projection [q | k | v]: q is rewritten in place, k and v go to the row's page.
__global__ void attn_prepare_whole_kernel(float* qkv, StepMeta m, AttnShape s, const float* qw, const float* kw, float* k_pool, float* v_pool) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    __shared__ float red[32];
    const int t = blockIdx.x, pos = m.row_pos[t];
    const int page = m.page_table[(size_t)m.ent_slot[m.row_ent[t]] * m.table_stride + pos / kPageTokens];
    const size_t tok = (size_t)page * kPageTokens + pos % kPageTokens;
    const int nq = s.heads * s.dim, nk = s.kv_heads * s.dim, nv = s.kv_heads * s.vdim;
    float* q = qkv + (size_t)t * s.ld;
    const float* k = q + nq;
    const float* v = k + nk;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) sq += q[i] * q[i];
    for (int i = threadIdx.x; i < nk; i += blockDim.x) sk += k[i] * k[i];
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float cq = 1.f / sqrtf(sq / (float)nq + s.eps), ck = 1.f / sqrtf(sk / (float)nk + s.eps);
    for (int i = threadIdx.x; i < nq; i += blockDim.x) q[i] = q[i] * cq * (qw ? qw[i] : 1.f);
    float* kd = k_pool + tok * (size_t)nk;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) kd[i] = k[i] * ck * (kw ? kw[i] : 1.f);
    float* vd = v_pool + tok * (size_t)nv;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) vd[i] = v[i];
}

// ---- capped, head-mixed attention ------------------------------------------------------------------------------------------------
// The mixing needs the scores of ALL heads of a (query, key) pair before any head's softmax can start, so the attention runs as
// three passes over a score scratch in global memory (sized to stay in L2):
//   1  scores: S[row][head][u] = cap * tanh(scale * q . k / cap) for every key u of the row's band -- register-tiled fp32 products of
//      64 rows x 64 keys per block for prompt portions (mix_scores_tiles_kernel), one warp per key for single rows
//      (mix_scores_rows_kernel);
//   2  one block per row: the H scores of every key are mixed through T, the mask is applied, and every head's softmax (with the
//      sink in the denominator) turns its scores into weights in place (mix_softmax_kernel);
//   3  weighted values: out[row][head] = sum_u P[row][head][u] v(u) -- again 64 x 64 tiles for prompt portions
//      (mix_values_tiles_kernel) and a split of the keys over the warps of a block for single rows (mix_values_rows_kernel).
// Every entry of the step is cut into tiles of up to 64 rows of one sequence (`tiles`: first row, row count); tiles with fewer than
// `small` rows go through the row kernels.  The keys a tile can see form its BAND, one list for all its rows: the kept first keys
// that lie below the window of the tile's first row, then the range from that window's start to the tile's last row; u indexes
// this list, and the mask of pass 2 removes what a single row must not see.
struct MixBand {
    int lo, nA, total;
    __device__ __forceinline__ int key(int u) const { return u < nA ? u : lo + (u - nA); }
};
__host__ __device__ inline MixBand mix_band(int p0, int n, int window, int keep_first) {
    MixBand b;
    b.lo = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
    b.nA = window > 0 ? (keep_first < b.lo ? keep_first : b.lo) : 0;
    b.total = b.nA + (p0 + n - 1 - b.lo + 1);
    return b;
}
struct MixArgs {
    const int* tiles;      // [n tiles][2]
    const int* row_tile;   // [T] the tile of every row of the step
    int tile0, row_base;   // first tile and first row of the batch the scratch holds (scratch row = row - row_base)
    int ldu;               // keys the scratch holds per (row, head)
    int small;             // tiles with fewer rows take the row kernels
    float* S;              // [rows][H][ldu] scores, then weights
    float* inv_den;        // [rows][H] 1 / softmax denominator
};
__device__ __forceinline__ float mix_cap(float v, const AttnShape& s) {
    v *= s.scale;
    return s.softcap > 0.f ? s.softcap * tanhf(v / s.softcap) : v;
}
__device__ __forceinline__ size_t mix_token(const int* table, int j) { return (size_t)table[j / kPageTokens] * kPageTokens + j % kPageTokens; }

// pass 1, prompt portions: grid (groups of the band's 64-key tiles, tiles of the batch, heads).  TC (bf16 mode, head size in whole 16-element
// steps): the product runs on the warp-level tensor cores at fp32 accuracy, the split-half scheme of window_attention_h3_kernel --
// every fp32 operand is split into two fp16 halves (x = hi + lo) as it is staged, and lo*hi + hi*lo + hi*hi is accumulated in fp32
// by mma.sync m16n8k16; a warp owns 16 rows x 32 keys.  Otherwise true fp32 multiply-adds, 4 rows x 4 keys a thread.
template <bool TC>
__global__ void __launch_bounds__(256) mix_scores_tiles_kernel(const float* qkv, StepMeta m, AttnShape s, MixArgs a, const float* k_pool) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ __align__(16) float mixsm[];
    const int tile = a.tile0 + blockIdx.y, row0 = a.tiles[2 * tile], n = a.tiles[2 * tile + 1];
    if (n < a.small) return;
    const int p0 = m.row_pos[row0];
    const MixBand b = mix_band(p0, n, s.window, s.keep_first);
    if ((int)blockIdx.x * 64 >= b.total) return;
    const int d = s.dim, d4 = (d + 3) / 4 * 4, ldq = d4 + 4, h = blockIdx.z, g = h / (s.heads / s.kv_heads);
    float* Qs = mixsm;
    float* Ks = Qs + 64 * ldq;
    // TC: four fp16 images [64][d + 8] (hi and lo halves of the queries and of the keys) in the same bytes
    const int LD = d + 8;
    __half* Qh = reinterpret_cast<__half*>(mixsm);
    __half* Ql = Qh + 64 * LD;
    __half* Kh = Ql + 64 * LD;
    __half* Kl = Kh + 64 * LD;
    const auto store_split4 = [](const float4& v, __half* hi, __half* lo) {
        __half x[4], y[4];
        split_h(v.x, x[0], y[0]); split_h(v.y, x[1], y[1]); split_h(v.z, x[2], y[2]); split_h(v.w, x[3], y[3]);
        *reinterpret_cast<uint2*>(hi) = make_uint2(pack_h2(x[0], x[1]), pack_h2(x[2], x[3]));
        *reinterpret_cast<uint2*>(lo) = make_uint2(pack_h2(y[0], y[1]), pack_h2(y[2], y[3]));
    };
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[row0]] * m.table_stride;
    const size_t kstride = (size_t)s.kv_heads * d;
    const bool vec = (d % 4 == 0) && (s.ld % 4 == 0);
    // the query tile is staged (and split) once; the block then walks the band's key tiles blockIdx.x, blockIdx.x + gridDim.x, ...
    for (int i = tid; i < 64 * (d4 / 4); i += 256) {
        const int r = i / (d4 / 4), k4 = (i % (d4 / 4)) * 4;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < n) {
            const float* src = qkv + (size_t)(row0 + r) * s.ld + (size_t)h * d + k4;
            if (vec) q = *reinterpret_cast<const float4*>(src);
            else { q.x = src[0]; if (k4 + 1 < d) q.y = src[1]; if (k4 + 2 < d) q.z = src[2]; if (k4 + 3 < d) q.w = src[3]; }
        }
        if constexpr (TC) store_split4(q, Qh + r * LD + k4, Ql + r * LD + k4);
        else *reinterpret_cast<float4*>(&Qs[r * ldq + k4]) = q;
    }
    for (int u0 = blockIdx.x * 64; u0 < b.total; u0 += gridDim.x * 64) {
        __syncthreads();   // (the key tile of the round before has been read)
        for (int i = tid; i < 64 * (d4 / 4); i += 256) {
            const int r = i / (d4 / 4), k4 = (i % (d4 / 4)) * 4;
            float4 k = make_float4(0.f, 0.f, 0.f, 0.f);
            if (u0 + r < b.total) {
                const float* src = k_pool + mix_token(table, b.key(u0 + r)) * kstride + (size_t)g * d + k4;
                if (vec) k = *reinterpret_cast<const float4*>(src);
                else { k.x = src[0]; if (k4 + 1 < d) k.y = src[1]; if (k4 + 2 < d) k.z = src[2]; if (k4 + 3 < d) k.w = src[3]; }
            }
            if constexpr (TC) store_split4(k, Kh + r * LD + k4, Kl + r * LD + k4);
            else *reinterpret_cast<float4*>(&Ks[r * ldq + k4]) = k;
        }
        __syncthreads();
        if constexpr (TC) {
            const int warp = tid >> 5, lane = tid & 31, gg = lane >> 2, t = lane & 3, rg = warp & 3, kh = warp >> 2;
            float c[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
            const uint32_t* qh_row = reinterpret_cast<const uint32_t*>(Qh + (16 * rg + gg) * LD) + t;
            const uint32_t* ql_row = reinterpret_cast<const uint32_t*>(Ql + (16 * rg + gg) * LD) + t;
            const int lm = lane >> 3, lr = lane & 7;
            const uint32_t k_ld = (uint32_t)(((lr + 8 * (lm >> 1)) * LD + 8 * (lm & 1)) * 2);
            const uint32_t kh_s = smem_u32(Kh), kl_s = smem_u32(Kl);
            for (int ks = 0; ks < d / 16; ++ks) {
                const uint32_t ah[4] = {qh_row[8 * ks], qh_row[8 * ks + 4 * LD], qh_row[8 * ks + 4], qh_row[8 * ks + 4 * LD + 4]};
                const uint32_t al[4] = {ql_row[8 * ks], ql_row[8 * ks + 4 * LD], ql_row[8 * ks + 4], ql_row[8 * ks + 4 * LD + 4]};
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {
                    uint32_t bh[4], bl[4];
                    const uint32_t off = (uint32_t)(((32 * kh + 16 * jp) * LD + 16 * ks) * 2) + k_ld;
                    ldsm_x4(bh, kh_s + off);
                    ldsm_x4(bl, kl_s + off);
                    mma_f16(c[2 * jp], al, bh[0], bh[1]);
                    mma_f16(c[2 * jp + 1], al, bh[2], bh[3]);
                    mma_f16(c[2 * jp], ah, bl[0], bl[1]);
                    mma_f16(c[2 * jp + 1], ah, bl[2], bl[3]);
                    mma_f16(c[2 * jp], ah, bh[0], bh[1]);
                    mma_f16(c[2 * jp + 1], ah, bh[2], bh[3]);
                }
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = 16 * rg + gg + 8 * half;
                if (r >= n) continue;
                float* dst = a.S + ((size_t)(row0 + r - a.row_base) * s.heads + h) * a.ldu + u0;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int key = 32 * kh + 8 * nt + 2 * t;
                    if (u0 + key < b.total) dst[key] = mix_cap(c[nt][2 * half], s);
                    if (u0 + key + 1 < b.total) dst[key + 1] = mix_cap(c[nt][2 * half + 1], s);
                }
            }
            continue;
        }
        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
        for (int k = 0; k < d4; k += 4) {
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
            const int r = ty + 16 * i;
            if (r >= n) continue;
            float* dst = a.S + ((size_t)(row0 + r - a.row_base) * s.heads + h) * a.ldu + u0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (u0 + tx + 16 * j < b.total) dst[tx + 16 * j] = mix_cap(sc[i][j], s);
        }
    }
}

// pass 1, single rows: grid (chunks of 64 keys, rows of the batch, key/value heads); a warp takes 8 keys, a lane the coordinates
// lane, lane + 32, ...; the row's query heads of the group wait in shared memory
template <int PL>   // coordinates of a head a lane owns: head sizes up to 32 * PL
__global__ void __launch_bounds__(256) mix_scores_rows_kernel(const float* qkv, StepMeta m, AttnShape s, MixArgs a, const float* k_pool) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ __align__(16) float mixsm[];   // [H / G][d]
    const int row = a.row_base + blockIdx.y, tile = a.row_tile[row], row0 = a.tiles[2 * tile], n = a.tiles[2 * tile + 1];
    if (n >= a.small) return;
    const MixBand b = mix_band(m.row_pos[row0], n, s.window, s.keep_first);
    const int u0 = blockIdx.x * 64;
    if (u0 >= b.total) return;
    const int d = s.dim, HG = s.heads / s.kv_heads, g = blockIdx.z, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < HG * d; i += 256) mixsm[i] = qkv[(size_t)row * s.ld + (size_t)g * HG * d + i];
    __syncthreads();
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[row0]] * m.table_stride;
    const size_t kstride = (size_t)s.kv_heads * d;
    // the warp's 8 key rows are requested together (PL coordinates a lane each), then multiplied with four query heads at a time
    float kv[8][PL];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const int u = min(u0 + warp * 8 + c, b.total - 1);
        const float* kr = k_pool + mix_token(table, b.key(u)) * kstride + (size_t)g * d;
#pragma unroll
        for (int i = 0; i < PL; ++i) kv[c][i] = lane + 32 * i < d ? kr[lane + 32 * i] : 0.f;
    }
    for (int hl0 = 0; hl0 < HG; hl0 += 4) {
        float qv[4][PL];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < PL; ++i) qv[q][i] = (hl0 + q < HG && lane + 32 * i < d) ? mixsm[(hl0 + q) * d + lane + 32 * i] : 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int u = u0 + warp * 8 + c;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < PL; ++i)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[q] = fmaf(qv[q][i], kv[c][i], acc[q]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float v = warp_sum(acc[q]);
                if (lane == 0 && hl0 + q < HG && u < b.total) a.S[((size_t)(row - a.row_base) * s.heads + g * HG + hl0 + q) * a.ldu + u] = mix_cap(v, s);
            }
        }
    }
}

// pass 2: grid (64, tiles of the batch); block (r, tile) owns row r of the tile and all heads: every key's H scores are mixed in
// registers and masked, then every head's weights exp(s - max) replace its scores and 1 / (their sum + exp(sink - max)) is kept
template <int HP, int NT>   // NT threads: 512 where the heads' registers allow it (more of a row's loads in flight), else 256
__global__ void __launch_bounds__(NT, (HP <= 16 && NT == 256) ? 3 : 1) mix_softmax_kernel(StepMeta m, AttnShape s, MixArgs a, int in_smem) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ __align__(16) float mixsm[];   // in_smem: [H][ldu] the row's mixed scores between the two sweeps
    __shared__ __align__(16) float Tm[HP * HP];
    __shared__ float red[NT / 32][HP];
    __shared__ float top[HP];
    const int tile = a.tile0 + blockIdx.y, row0 = a.tiles[2 * tile], n = a.tiles[2 * tile + 1], r = blockIdx.x;
    if (r >= n) return;
    const int H = s.heads, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p0 = m.row_pos[row0], pos = p0 + r;
    const MixBand b = mix_band(p0, n, s.window, s.keep_first);
    if (s.talk)
        for (int i = tid; i < HP * HP; i += NT) Tm[i] = (i / HP < H && i % HP < H) ? s.talk[(i / HP) * H + i % HP] : 0.f;
    __syncthreads();
    float* base = a.S + (size_t)(row0 + r - a.row_base) * H * a.ldu;
    float mx[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) mx[h] = -INFINITY;
    for (int u = tid; u < b.total; u += NT) {
        const int j = b.key(u);
        const bool seen = j <= pos && (s.window <= 0 || pos - j < s.window || j < s.keep_first);
        float sv[HP];
#pragma unroll
        for (int h = 0; h < HP; ++h) sv[h] = h < H ? base[(size_t)h * a.ldu + u] : 0.f;
#pragma unroll
        for (int h = 0; h < HP; ++h) {
            if (h >= H) break;
            float v = sv[h];
            if (s.talk) {
                v = 0.f;
#pragma unroll
                for (int g = 0; g < HP; g += 4) {
                    const float4 tv = *reinterpret_cast<const float4*>(&Tm[h * HP + g]);
                    v = fmaf(tv.x, sv[g], fmaf(tv.y, sv[g + 1], fmaf(tv.z, sv[g + 2], fmaf(tv.w, sv[g + 3], v))));
                }
            }
            v = seen ? v : -INFINITY;
            if (in_smem) mixsm[(size_t)h * a.ldu + u] = v;
            else base[(size_t)h * a.ldu + u] = v;
            mx[h] = fmaxf(mx[h], v);
        }
    }
#pragma unroll
    for (int h = 0; h < HP; ++h) {
        const float v = warp_max(mx[h]);
        if (lane == 0) red[warp][h] = v;
    }
    __syncthreads();
    if (tid < HP) {
        float v = red[0][tid];
        for (int w = 1; w < NT / 32; ++w) v = fmaxf(v, red[w][tid]);
        if (s.sink && tid < H) v = fmaxf(v, s.sink[tid]);
        top[tid] = v;
    }
    __syncthreads();
    float sum[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) sum[h] = 0.f;
    for (int u = tid; u < b.total; u += NT) {   // (each thread reads back what it wrote itself)
#pragma unroll
        for (int h = 0; h < HP; ++h) {
            if (h >= H) break;
            const float v = in_smem ? mixsm[(size_t)h * a.ldu + u] : base[(size_t)h * a.ldu + u];
            const float e = v == -INFINITY ? 0.f : expf(v - top[h]);
            base[(size_t)h * a.ldu + u] = e;
            sum[h] += e;
        }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < HP; ++h) {
        const float v = warp_sum(sum[h]);
        if (lane == 0) red[warp][h] = v;
    }
    __syncthreads();
    if (tid < H) {
        float v = 0.f;
        for (int w = 0; w < NT / 32; ++w) v += red[w][tid];
        if (s.sink) v += expf(s.sink[tid] - top[tid]);
        a.inv_den[(size_t)(row0 + r - a.row_base) * H + tid] = 1.f / v;
    }
}

// pass 2 for many heads (more than 16: the register form above would hold 32 or 64 scores, maxima and sums a thread): the row's scores
// of all heads are copied to shared memory [H][ldu] first; then four lanes share a group of FOUR neighbouring keys, each mixing a
// quarter of the heads (QW = 8 or 16 of them) from the H scores of those keys in shared memory (T transposed, so that a lane's heads
// are contiguous: one score vector and QW / 4 vectors of T a step for 4 QW multiply-adds) and writing them back in place once all
// four have read (they sit in one warp); then one warp per head takes the maximum, writes exp(s - max) to the scratch and keeps
// 1 / (sum + exp(sink - max)).  grid (64, tiles of the batch), 512 threads.
constexpr int kMixWideThreads = 512;
__host__ __device__ inline size_t mix_softmax_wide_smem_bytes(int H, int ldu) { return ((size_t)H * ldu + (size_t)H * 64) * sizeof(float); }
template <int QW>   // heads a lane mixes: up to 4 x QW heads
__global__ void __launch_bounds__(kMixWideThreads) mix_softmax_wide_kernel(StepMeta m, AttnShape s, MixArgs a) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ __align__(16) float mixsm[];
    const int tile = a.tile0 + blockIdx.y, row0 = a.tiles[2 * tile], n = a.tiles[2 * tile + 1], r = blockIdx.x;
    if (r >= n) return;
    const int H = s.heads, HQ = (H + 3) / 4, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, ldu = a.ldu;
    constexpr int NW = kMixWideThreads / 32, LT = 4 * QW;
    float* R = mixsm;                 // [H][ldu]
    float* Tt = R + (size_t)H * ldu;  // [H (g)][LT]: Tt[g][q * QW + k] = T[q * HQ + k][g] (identity without a mixing matrix)
    const int p0 = m.row_pos[row0], pos = p0 + r;
    const MixBand b = mix_band(p0, n, s.window, s.keep_first);
    float* base = a.S + (size_t)(row0 + r - a.row_base) * H * ldu;
    for (int i = tid; i < H * LT; i += kMixWideThreads) {
        const int g = i / LT, q = (i % LT) / QW, k = i % QW, h = q * HQ + k;
        Tt[i] = (k < HQ && h < H) ? (s.talk ? s.talk[h * H + g] : (h == g ? 1.f : 0.f)) : 0.f;
    }
    for (int i = tid; i < H * (ldu / 4); i += kMixWideThreads) {   // (whole vectors of the scratch: what lies beyond the band is never used)
        const int h = i / (ldu / 4), u4 = (i % (ldu / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (u4 < b.total) v = *reinterpret_cast<const float4*>(base + (size_t)h * ldu + u4);
        *reinterpret_cast<float4*>(R + (size_t)h * ldu + u4) = v;
    }
    __syncthreads();
    const int q = lane >> 3;   // this lane's quarter of the heads: q * HQ .. q * HQ + HQ - 1
    for (int u = warp * 32 + 4 * (lane & 7); u < (b.total + 31) / 32 * 32; u += NW * 32) {   // (whole groups of 32 keys: a warp stays together)
        const bool in = u < b.total;
        float acc[4][QW];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int k = 0; k < QW; ++k) acc[c][k] = 0.f;
        if (in)
            for (int g = 0; g < H; ++g) {
                const float4 sv = *reinterpret_cast<const float4*>(R + (size_t)g * ldu + u);
                const float4* tr = reinterpret_cast<const float4*>(Tt + g * LT + q * QW);
#pragma unroll
                for (int k4 = 0; k4 < QW / 4; ++k4) {
                    const float4 tv = tr[k4];
                    const float t4[4] = {tv.x, tv.y, tv.z, tv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        acc[0][4 * k4 + e] = fmaf(t4[e], sv.x, acc[0][4 * k4 + e]);
                        acc[1][4 * k4 + e] = fmaf(t4[e], sv.y, acc[1][4 * k4 + e]);
                        acc[2][4 * k4 + e] = fmaf(t4[e], sv.z, acc[2][4 * k4 + e]);
                        acc[3][4 * k4 + e] = fmaf(t4[e], sv.w, acc[3][4 * k4 + e]);
                    }
                }
            }
        __syncwarp();   // the four lanes of a key group have read its scores
        if (in) {
            bool seen[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = b.key(min(u + c, b.total - 1));
                seen[c] = u + c < b.total && j <= pos && (s.window <= 0 || pos - j < s.window || j < s.keep_first);
            }
#pragma unroll
            for (int k = 0; k < QW; ++k)
                if (k < HQ && q * HQ + k < H)
                    *reinterpret_cast<float4*>(R + (size_t)(q * HQ + k) * ldu + u) =
                        make_float4(seen[0] ? acc[0][k] : -INFINITY, seen[1] ? acc[1][k] : -INFINITY, seen[2] ? acc[2][k] : -INFINITY, seen[3] ? acc[3][k] : -INFINITY);
        }
    }
    __syncthreads();
    for (int h = warp; h < H; h += NW) {
        const float* rr = R + (size_t)h * ldu;
        float mx = -INFINITY;
        for (int u = lane; u < b.total; u += 32) mx = fmaxf(mx, rr[u]);
        mx = warp_max(mx);
        if (s.sink) mx = fmaxf(mx, s.sink[h]);
        float sum = 0.f;
        for (int u = lane; u < b.total; u += 32) {
            const float v = rr[u];
            const float e = v == -INFINITY ? 0.f : expf(v - mx);
            base[(size_t)h * ldu + u] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        if (lane == 0) a.inv_den[(size_t)(row0 + r - a.row_base) * H + h] = 1.f / (sum + (s.sink ? expf(s.sink[h] - mx) : 0.f));
    }
}

// pass 3, prompt portions: grid (tiles of the batch, heads, groups of 64 value columns); O[64 rows][64 columns] = sum over the band's
// 64-key tiles of P V, 4 rows x 4 columns a thread -- or, TC (bf16 mode), split-half tensor-core products as in pass 1 (the value tile
// is read through transposing matrix loads), a warp owning 16 rows x 32 columns
template <bool TC>
__global__ void __launch_bounds__(256, 3) mix_values_tiles_kernel(StepMeta m, AttnShape s, MixArgs a, const float* v_pool, float* out) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ __align__(16) float mixsm[];
    const int tile = a.tile0 + blockIdx.x, row0 = a.tiles[2 * tile], n = a.tiles[2 * tile + 1];
    if (n < a.small) return;
    const int H = s.heads, dv = s.vdim, h = blockIdx.y, g = h / (H / s.kv_heads), ldp = 64 + 4;
    float* Ps = mixsm;             // [64 rows][ldp]
    constexpr int ldv = 64;
    float* Vs = Ps + 64 * ldp;     // [64 keys][ldv]
    // TC: four fp16 images [64][72] (hi and lo halves of the weights and of the values)
    constexpr int LH = 72;
    __half* Ph = reinterpret_cast<__half*>(mixsm);
    __half* Pl = Ph + 64 * LH;
    __half* Vh = Pl + 64 * LH;
    __half* Vl = Vh + 64 * LH;
    const auto store_split4 = [](const float4& v, __half* hi, __half* lo) {
        __half x[4], y[4];
        split_h(v.x, x[0], y[0]); split_h(v.y, x[1], y[1]); split_h(v.z, x[2], y[2]); split_h(v.w, x[3], y[3]);
        *reinterpret_cast<uint2*>(hi) = make_uint2(pack_h2(x[0], x[1]), pack_h2(x[2], x[3]));
        *reinterpret_cast<uint2*>(lo) = make_uint2(pack_h2(y[0], y[1]), pack_h2(y[2], y[3]));
    };
    const int col0 = blockIdx.z * 64;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int warp = tid >> 5, lane = tid & 31, gg = lane >> 2, t4 = lane & 3, rg = warp & 3, ch = warp >> 2;
    const MixBand b = mix_band(m.row_pos[row0], n, s.window, s.keep_first);
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[row0]] * m.table_stride;
    const size_t vstride = (size_t)s.kv_heads * dv;
    const bool vec = dv % 4 == 0, vecp = a.ldu % 4 == 0;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    // the next key tile's weights and values are requested while the current one is multiplied (four 16-byte loads of each a thread)
    float4 np[4], nv[4];
    const auto fetch = [&](int u0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int i = tid + 256 * q, r = i >> 4, c4 = (i & 15) * 4;
            float4 p = make_float4(0.f, 0.f, 0.f, 0.f), v = p;
            if (r < n) {
                const float* src = a.S + ((size_t)(row0 + r - a.row_base) * H + h) * a.ldu + u0 + c4;
                if (vecp && u0 + c4 + 3 < b.total) p = *reinterpret_cast<const float4*>(src);
                else {
                    if (u0 + c4 < b.total) p.x = src[0];
                    if (u0 + c4 + 1 < b.total) p.y = src[1];
                    if (u0 + c4 + 2 < b.total) p.z = src[2];
                    if (u0 + c4 + 3 < b.total) p.w = src[3];
                }
            }
            const int k4 = col0 + c4;   // (r is the key of the tile here)
            if (u0 + r < b.total && k4 < dv) {
                const float* src = v_pool + mix_token(table, b.key(u0 + r)) * vstride + (size_t)g * dv + k4;
                if (vec) v = *reinterpret_cast<const float4*>(src);
                else { v.x = src[0]; if (k4 + 1 < dv) v.y = src[1]; if (k4 + 2 < dv) v.z = src[2]; if (k4 + 3 < dv) v.w = src[3]; }
            }
            np[q] = p;
            nv[q] = v;
        }
    };
    fetch(0);
    for (int u0 = 0; u0 < b.total; u0 += 64) {
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int i = tid + 256 * q, r = i >> 4, c4 = (i & 15) * 4;
            if constexpr (TC) {
                store_split4(np[q], Ph + r * LH + c4, Pl + r * LH + c4);
                store_split4(nv[q], Vh + r * LH + c4, Vl + r * LH + c4);
            } else {
                *reinterpret_cast<float4*>(&Ps[r * ldp + c4]) = np[q];
                *reinterpret_cast<float4*>(&Vs[r * ldv + c4]) = nv[q];
            }
        }
        __syncthreads();
        if (u0 + 64 < b.total) fetch(u0 + 64);
        if constexpr (TC) {
            const uint32_t* ph_row = reinterpret_cast<const uint32_t*>(Ph + (16 * rg + gg) * LH) + t4;
            const uint32_t* pl_row = reinterpret_cast<const uint32_t*>(Pl + (16 * rg + gg) * LH) + t4;
            const int lm = lane >> 3, lr = lane & 7;
            const uint32_t v_ld = (uint32_t)(((lr + 8 * (lm & 1)) * LH + 8 * (lm >> 1)) * 2);
            const uint32_t vh_s = smem_u32(Vh), vl_s = smem_u32(Vl);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t ah[4] = {ph_row[8 * kk], ph_row[8 * kk + 4 * LH], ph_row[8 * kk + 4], ph_row[8 * kk + 4 * LH + 4]};
                const uint32_t al[4] = {pl_row[8 * kk], pl_row[8 * kk + 4 * LH], pl_row[8 * kk + 4], pl_row[8 * kk + 4 * LH + 4]};
#pragma unroll
                for (int np2 = 0; np2 < 2; ++np2) {
                    uint32_t bh[4], bl[4];
                    const uint32_t off = (uint32_t)((16 * kk * LH + 32 * ch + 16 * np2) * 2) + v_ld;
                    ldsm_x4_trans(bh, vh_s + off);
                    ldsm_x4_trans(bl, vl_s + off);
                    mma_f16(acc[2 * np2], al, bh[0], bh[1]);
                    mma_f16(acc[2 * np2 + 1], al, bh[2], bh[3]);
                    mma_f16(acc[2 * np2], ah, bl[0], bl[1]);
                    mma_f16(acc[2 * np2 + 1], ah, bl[2], bl[3]);
                    mma_f16(acc[2 * np2], ah, bh[0], bh[1]);
                    mma_f16(acc[2 * np2 + 1], ah, bh[2], bh[3]);
                }
            }
            continue;
        }
        for (int c = 0; c < 64; c += 4) {
            float4 pr[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pr[i] = *reinterpret_cast<const float4*>(&Ps[(ty + 16 * i) * ldp + c]);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const float4 v = *reinterpret_cast<const float4*>(&Vs[(c + cc) * ldv + tx * 4]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float p = cc == 0 ? pr[i].x : cc == 1 ? pr[i].y : cc == 2 ? pr[i].z : pr[i].w;
                    acc[i][0] = fmaf(p, v.x, acc[i][0]);
                    acc[i][1] = fmaf(p, v.y, acc[i][1]);
                    acc[i][2] = fmaf(p, v.z, acc[i][2]);
                    acc[i][3] = fmaf(p, v.w, acc[i][3]);
                }
            }
        }
    }
    if constexpr (TC) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = 16 * rg + gg + 8 * half;
            if (r >= n) continue;
            const float f = a.inv_den[(size_t)(row0 + r - a.row_base) * H + h];
            float* o = out + (size_t)(row0 + r) * ((size_t)H * dv) + (size_t)h * dv;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int col = col0 + 32 * ch + 8 * nt + 2 * t4;
                if (col < dv) o[col] = acc[nt][2 * half] * f;
                if (col + 1 < dv) o[col + 1] = acc[nt][2 * half + 1] * f;
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty + 16 * i;
        if (r >= n) continue;
        const float f = a.inv_den[(size_t)(row0 + r - a.row_base) * H + h];
        float* o = out + (size_t)(row0 + r) * ((size_t)H * dv) + (size_t)h * dv;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = col0 + tx * 4 + e;
            if (col < dv) o[col] = acc[i][e] * f;
        }
    }
}

// pass 3, single rows: grid (rows of the batch, heads); 32 warps split the band's keys (four keys in flight a warp), a lane owns the
// value coordinates lane, lane + 32, ...; the warps' sums are added in warp order
constexpr int kMixRowWarps = 32;
template <int PL>
__global__ void __launch_bounds__(kMixRowWarps * 32) mix_values_rows_kernel(StepMeta m, AttnShape s, MixArgs a, const float* v_pool, float* out) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ __align__(16) float mixsm[];   // [warps][dv]
    const int row = a.row_base + blockIdx.x, tile = a.row_tile[row], row0 = a.tiles[2 * tile], n = a.tiles[2 * tile + 1];
    if (n >= a.small) return;
    const int H = s.heads, dv = s.vdim, h = blockIdx.y, g = h / (H / s.kv_heads), warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const MixBand b = mix_band(m.row_pos[row0], n, s.window, s.keep_first);
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[row0]] * m.table_stride;
    const size_t vstride = (size_t)s.kv_heads * dv;
    const float* P = a.S + ((size_t)(row - a.row_base) * H + h) * a.ldu;
    const int chunk = (b.total + kMixRowWarps - 1) / kMixRowWarps, ub = warp * chunk, ue = min(b.total, ub + chunk);
    float o[PL];
#pragma unroll
    for (int i = 0; i < PL; ++i) o[i] = 0.f;
    for (int u = ub; u < ue; u += 4) {
        float p[4];
        const float* vr[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int uu = min(u + q, ue - 1);
            p[q] = u + q < ue ? P[uu] : 0.f;
            vr[q] = v_pool + mix_token(table, b.key(uu)) * vstride + (size_t)g * dv;
        }
        float vv[4][PL];
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int c = lane + 32 * i;
#pragma unroll
            for (int q = 0; q < 4; ++q) vv[q][i] = c < dv ? vr[q][c] : 0.f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < PL; ++i) o[i] = fmaf(p[q], vv[q][i], o[i]);
    }
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) mixsm[warp * dv + c] = o[i];
    }
    __syncthreads();
    const float f = a.inv_den[(size_t)(row - a.row_base) * H + h];
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float acc = 0.f;
        for (int w = 0; w < kMixRowWarps; ++w) acc += mixsm[w * dv + c];
        out[(size_t)row * ((size_t)H * dv) + (size_t)h * dv + c] = acc * f;
    }
}

}  // namespace seq
}  // namespace tib

// seq_headmix.cuh -- attention of the layered sequence engine whose scores are worked on between the dot product and the
// softmax, and the small stateful pieces that come with such layers:
//
//   * whole-projection query / key norm: q (all heads at once) and k are divided by the RMS over the WHOLE projection and
//     multiplied by a plain per-coordinate weight, then k and v are appended to the row's page (attn_prepare_whole_kernel);
//   * capped, head-mixed, windowed attention with kept first keys and a sink (heads_mixed_attention_kernel):
//         s_h(i, j)  = cap * tanh(scale * q_h(i) . k_g(h)(j) / cap)                  (cap <= 0: no cap)
//         s'_h(i, j) = sum_g T[h][g] s_g(i, j)                                       (T null: no mixing)
//         row i sees key j  <=>  j <= i and (window <= 0 or i - j < window or j < keep_first)
//         p_h(i, j)  = exp(s'_h(i, j)) / (sum over seen j' of exp(s'_h(i, j')) + exp(sink_h))   (sink null: no extra term)
//     The mixing needs the scores of ALL heads of a (query, key) pair at once, so a block owns rows of one sequence and every
//     head, unlike the per-head kernels of seq_kernels.cuh / seq_attn_tc.cuh;
//   * a causal depth-wise short convolution over time in front of a mixer, y_t = x_t + sum_j w[:, j] x_(t - taps + 1 + j), whose
//     last taps - 1 inputs are sequence state (short_conv_kernel, short_conv_save_kernel).
//
// Everything here is fp32 in both compute modes: scores, cap, mixing, softmax and the weighted sum of values.
#pragma once
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

// ---- short convolution ------------------------------------------------------------------------------------------------------------
// state [slots][taps - 1][D]: the inputs at positions len - (taps - 1) .. len - 1 of the slot's sequence, oldest first.  Entries
// for positions before 0 are never read (a slot that is used again needs no clearing).
__global__ void short_conv_kernel(const float* x, StepMeta m, int D, int taps, const float* w, const float* state, float* y) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int t = blockIdx.x, e = m.row_ent[t], i = t - m.ent_row0[e], pos0 = m.ent_pos0[e];
    const float* st = state + (size_t)m.ent_slot[e] * (taps - 1) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float xv = x[(size_t)t * D + d];
        float acc = xv;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;
            float v = 0.f;
            if (back == 0) v = xv;
            else if (i - back >= 0) v = x[(size_t)(t - back) * D + d];
            else if (pos0 + i - back >= 0) v = st[(size_t)(taps - 1 + i - back) * D + d];
            acc = fmaf(w[(size_t)d * taps + j], v, acc);
        }
        y[(size_t)t * D + d] = acc;
    }
}
// after all rows of the step have read the old state: the slot keeps the last taps - 1 inputs of its sequence
__global__ void short_conv_save_kernel(const float* x, StepMeta m, int D, int taps, float* state) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int e = blockIdx.x, row0 = m.ent_row0[e], n = m.ent_row0[e + 1] - row0;
    float* st = state + (size_t)m.ent_slot[e] * (taps - 1) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x)
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
// A block owns up to R consecutive rows of ONE sequence and ALL query heads.  The keys its rows can see are the kept first ones
// below the window and the window's range, walked as one list in tiles of 64 keys.  Per key tile:
//   A  for every key/value head g: its key tile and the query vectors of its heads go to shared memory, scores (2 queries x 4 keys
//      a thread), scale and cap -> S[head * R + row][key]
//   B  one thread per (row, key) column: the H scores are mixed through T (registers), the mask is applied (-inf)
//   C  one warp per S row: running maximum and sum, S <- exp(S - max), the factor for what was accumulated before
//   D  for every key/value head g: its value tile to shared memory, O[head * R + row] <- O * factor + P V (O in shared memory,
//      a tile's sum in registers)
// Two forms of the grid.  Prompt portions: `tiles` lists (first row, rows <= 64) pairs; block b takes rows [sub_i * R, ...) of tile
// b / sub, finishes the softmax (sink included) and writes out[t][h * dv ..].  Single rows: `rows` lists rows, blockIdx.y is one of
// `splits` chunks of the row's key list; the block leaves (max, sum, unnormalised O) per head in `part`
// [row index][head][split][dv + 2], which attention_merge_kernel combines.
constexpr int kMixKT = 64;
struct MixLayout {   // shared memory, in floats
    int R, d4, dv4, ldq, ldkv, ldS, HP;
    int off_T, off_Q, off_KV, off_S, off_O, off_stat, total;
};
__host__ __device__ inline MixLayout mix_layout(int H, int G, int d, int dv, int R, int HP, bool talk) {
    MixLayout L;
    L.R = R; L.HP = HP;
    L.d4 = (d + 3) / 4 * 4; L.dv4 = (dv + 3) / 4 * 4;
    L.ldq = L.d4 + 4; L.ldkv = (L.d4 > L.dv4 ? L.d4 : L.dv4) + 4; L.ldS = kMixKT + 4;
    int o = 0;
    L.off_T = o; o += talk ? H * HP : 0;
    L.off_Q = o; o += (H / G) * R * L.ldq;
    L.off_KV = o; o += kMixKT * L.ldkv;
    L.off_S = o; o += H * R * L.ldS;
    L.off_O = o; o += H * R * L.dv4;
    L.off_stat = o; o += 3 * H * R;
    L.total = o;
    return L;
}
__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
    return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, acc))));
}
template <int HP>
__global__ void __launch_bounds__(256) heads_mixed_attention_kernel(const float* qkv, StepMeta m, AttnShape s, const int* tiles, int R, int sub, const int* rows,
                                                                    int splits, const float* k_pool, const float* v_pool, float* out, float* part) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ __align__(16) float mixsm[];
    const int H = s.heads, G = s.kv_heads, HG = H / G, d = s.dim, dv = s.vdim;
    const MixLayout L = mix_layout(H, G, d, dv, R, HP, s.talk != nullptr);
    float* Tm = mixsm + L.off_T;
    float* Qg = mixsm + L.off_Q;
    float* KV = mixsm + L.off_KV;
    float* S = mixsm + L.off_S;
    float* O = mixsm + L.off_O;
    float* mrow = mixsm + L.off_stat;
    float* lrow = mrow + H * R;
    float* crow = lrow + H * R;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, tx = tid & 15, ty = tid >> 4;
    int row0, n, z = 0;
    if (rows) {
        row0 = rows[blockIdx.x];
        n = 1;
        z = blockIdx.y;
    } else {
        const int tile = blockIdx.x / sub, si = blockIdx.x % sub;
        row0 = tiles[2 * tile] + si * R;
        n = min(R, tiles[2 * tile + 1] - si * R);
        if (n <= 0) return;
    }
    const int p0 = m.row_pos[row0], hi = p0 + n - 1;
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[row0]] * m.table_stride;
    const int lo = (s.window > 0 && p0 - s.window + 1 > 0) ? p0 - s.window + 1 : 0;
    const int nA = s.window > 0 ? min(s.keep_first, lo) : 0;   // kept first keys below the window's range
    const int total = nA + (hi - lo + 1);
    int u_begin = 0, u_end = total;
    if (rows && splits > 1) {
        const int chunk = (total + splits - 1) / splits;
        u_begin = min(total, z * chunk);
        u_end = min(total, u_begin + chunk);
    }
    if (s.talk)
        for (int i = tid; i < H * HP; i += 256) Tm[i] = (i % HP) < H ? s.talk[(i / HP) * H + i % HP] : 0.f;
    for (int i = tid; i < H * R; i += 256) { mrow[i] = -INFINITY; lrow[i] = 0.f; }
    for (int i = tid; i < H * R * L.dv4; i += 256) O[i] = 0.f;
    const size_t kstride = (size_t)G * d, vstride = (size_t)G * dv;
    const bool vecq = (d % 4 == 0) && (s.ld % 4 == 0), veck = d % 4 == 0, vecv = dv % 4 == 0;
    const float inv_cap = s.softcap > 0.f ? 1.f / s.softcap : 0.f;
    const int QV = HG * R;
    for (int u0 = u_begin; u0 < u_end; u0 += kMixKT) {
        const int kc = min(kMixKT, u_end - u0);
        // ---- A: scores of every head ----
        for (int g = 0; g < G; ++g) {
            __syncthreads();
            for (int i = tid; i < kMixKT * (L.d4 / 4); i += 256) {
                const int c = i / (L.d4 / 4), k4 = (i % (L.d4 / 4)) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < kc) {
                    const int u = u0 + c, j = u < nA ? u : lo + (u - nA);
                    const float* src = k_pool + ((size_t)table[j / kPageTokens] * kPageTokens + j % kPageTokens) * kstride + (size_t)g * d + k4;
                    if (veck) v = *reinterpret_cast<const float4*>(src);
                    else {
                        v.x = src[0];
                        if (k4 + 1 < d) v.y = src[1];
                        if (k4 + 2 < d) v.z = src[2];
                        if (k4 + 3 < d) v.w = src[3];
                    }
                }
                *reinterpret_cast<float4*>(&KV[c * L.ldkv + k4]) = v;
            }
            for (int i = tid; i < QV * (L.d4 / 4); i += 256) {
                const int qv = i / (L.d4 / 4), k4 = (i % (L.d4 / 4)) * 4, hl = qv / R, r = qv % R;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < n) {
                    const float* src = qkv + (size_t)(row0 + r) * s.ld + (size_t)(g * HG + hl) * d + k4;
                    if (vecq) v = *reinterpret_cast<const float4*>(src);
                    else {
                        v.x = src[0];
                        if (k4 + 1 < d) v.y = src[1];
                        if (k4 + 2 < d) v.z = src[2];
                        if (k4 + 3 < d) v.w = src[3];
                    }
                }
                *reinterpret_cast<float4*>(&Qg[qv * L.ldq + k4]) = v;
            }
            __syncthreads();
            for (int qp = ty; 2 * qp < QV; qp += 16) {
                const int q0 = 2 * qp, q1 = min(q0 + 1, QV - 1);
                const float* qa = Qg + q0 * L.ldq;
                const float* qb = Qg + q1 * L.ldq;
                float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                for (int k = 0; k < L.d4; k += 4) {
                    const float4 a = *reinterpret_cast<const float4*>(qa + k), b = *reinterpret_cast<const float4*>(qb + k);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const float4 kk = *reinterpret_cast<const float4*>(&KV[(tx + 16 * jj) * L.ldkv + k]);
                        sc[0][jj] = dot4(a, kk, sc[0][jj]);
                        sc[1][jj] = dot4(b, kk, sc[1][jj]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int qv = q0 + i;
                    if (qv < QV) {
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            float v = sc[i][jj] * s.scale;
                            if (s.softcap > 0.f) v = s.softcap * tanhf(v * inv_cap);
                            S[(size_t)(g * QV + qv) * L.ldS + tx + 16 * jj] = v;
                        }
                    }
                }
            }
        }
        __syncthreads();
        // ---- B: mixing across the heads, mask ----
        for (int col = tid; col < R * kMixKT; col += 256) {
            const int r = col / kMixKT, c = col % kMixKT;
            bool seen = false;
            if (r < n && c < kc) {
                const int u = u0 + c, j = u < nA ? u : lo + (u - nA), pos = p0 + r;
                seen = j <= pos && (s.window <= 0 || pos - j < s.window || j < s.keep_first);
            }
            float* sp = S + (size_t)r * L.ldS + c;
            const size_t hs = (size_t)R * L.ldS;
            if (!seen) {
                for (int h = 0; h < H; ++h) sp[h * hs] = -INFINITY;
            } else if (s.talk) {
                float sv[HP];
#pragma unroll
                for (int g = 0; g < HP; ++g) sv[g] = g < H ? sp[g * hs] : 0.f;
                for (int h = 0; h < H; ++h) {
                    float acc = 0.f;
#pragma unroll
                    for (int g = 0; g < HP; g += 4) {
                        const float4 tv = *reinterpret_cast<const float4*>(&Tm[h * HP + g]);
                        acc = fmaf(tv.x, sv[g], fmaf(tv.y, sv[g + 1], fmaf(tv.z, sv[g + 2], fmaf(tv.w, sv[g + 3], acc))));
                    }
                    sp[h * hs] = acc;
                }
            }
        }
        __syncthreads();
        // ---- C: running softmax statistics of every (head, row) ----
        for (int hr = warp; hr < H * R; hr += 8) {
            float* sp = S + (size_t)hr * L.ldS;
            const float v0 = sp[lane], v1 = sp[lane + 32];
            const float tmax = warp_max(fmaxf(v0, v1));
            const float mo = mrow[hr], nm = fmaxf(mo, tmax);
            float e0 = 0.f, e1 = 0.f, corr = 1.f;
            if (nm != -INFINITY) {
                e0 = expf(v0 - nm);
                e1 = expf(v1 - nm);
                corr = expf(mo - nm);
            }
            sp[lane] = e0;
            sp[lane + 32] = e1;
            const float ps = warp_sum(e0 + e1);
            if (lane == 0) {
                lrow[hr] = lrow[hr] * corr + ps;
                mrow[hr] = nm;
                crow[hr] = corr;
            }
        }
        // ---- D: weighted values ----
        for (int g = 0; g < G; ++g) {
            __syncthreads();
            for (int i = tid; i < kMixKT * (L.dv4 / 4); i += 256) {
                const int c = i / (L.dv4 / 4), k4 = (i % (L.dv4 / 4)) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < kc) {
                    const int u = u0 + c, j = u < nA ? u : lo + (u - nA);
                    const float* src = v_pool + ((size_t)table[j / kPageTokens] * kPageTokens + j % kPageTokens) * vstride + (size_t)g * dv + k4;
                    if (vecv) v = *reinterpret_cast<const float4*>(src);
                    else {
                        v.x = src[0];
                        if (k4 + 1 < dv) v.y = src[1];
                        if (k4 + 2 < dv) v.z = src[2];
                        if (k4 + 3 < dv) v.w = src[3];
                    }
                }
                *reinterpret_cast<float4*>(&KV[c * L.ldkv + k4]) = v;
            }
            __syncthreads();
            const int ncx = L.dv4 / 4, items = ((QV + 1) / 2) * ncx;
            for (int item = tid; item < items; item += 256) {
                const int cx = item % ncx, qp = item / ncx;
                const int hr0 = g * QV + 2 * qp, hr1 = g * QV + min(2 * qp + 1, QV - 1);
                const float* pa = S + (size_t)hr0 * L.ldS;
                const float* pb = S + (size_t)hr1 * L.ldS;
                float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
                for (int c = 0; c < kc; ++c) {
                    const float4 v = *reinterpret_cast<const float4*>(&KV[c * L.ldkv + 4 * cx]);
                    const float x0 = pa[c], x1 = pb[c];
                    a0.x = fmaf(x0, v.x, a0.x); a0.y = fmaf(x0, v.y, a0.y); a0.z = fmaf(x0, v.z, a0.z); a0.w = fmaf(x0, v.w, a0.w);
                    a1.x = fmaf(x1, v.x, a1.x); a1.y = fmaf(x1, v.y, a1.y); a1.z = fmaf(x1, v.z, a1.z); a1.w = fmaf(x1, v.w, a1.w);
                }
                float4* o0 = reinterpret_cast<float4*>(&O[(size_t)hr0 * L.dv4 + 4 * cx]);
                const float c0 = crow[hr0];
                float4 w = *o0;
                w.x = fmaf(w.x, c0, a0.x); w.y = fmaf(w.y, c0, a0.y); w.z = fmaf(w.z, c0, a0.z); w.w = fmaf(w.w, c0, a0.w);
                *o0 = w;
                if (2 * qp + 1 < QV) {
                    float4* o1 = reinterpret_cast<float4*>(&O[(size_t)hr1 * L.dv4 + 4 * cx]);
                    const float c1 = crow[hr1];
                    w = *o1;
                    w.x = fmaf(w.x, c1, a1.x); w.y = fmaf(w.y, c1, a1.y); w.z = fmaf(w.z, c1, a1.z); w.w = fmaf(w.w, c1, a1.w);
                    *o1 = w;
                }
            }
        }
    }
    __syncthreads();
    if (rows && part) {
        const size_t ps = (size_t)dv + 2;
        for (int i = tid; i < H * (dv + 2); i += 256) {
            const int h = i / (dv + 2), c = i % (dv + 2);
            const int hr = h * R;
            float* dst = part + (((size_t)blockIdx.x * H + h) * splits + z) * ps;
            dst[c] = c == 0 ? mrow[hr] : c == 1 ? lrow[hr] : O[(size_t)hr * L.dv4 + c - 2];
        }
    } else {
        for (int i = tid; i < H * n * dv; i += 256) {
            const int c = i % dv, r = (i / dv) % n, h = i / (dv * n);
            const int hr = h * R + r;
            out[(size_t)(row0 + r) * ((size_t)H * dv) + (size_t)h * dv + c] = O[(size_t)hr * L.dv4 + c] * attn_finish_factor(s, h, mrow[hr], lrow[hr]);
        }
    }
}

}  // namespace seq
}  // namespace tib

// seq_attn_tc.cuh -- attention of the layered sequence engine for prompt portions on the warp-level tensor cores, at fp32
// accuracy: the split-half scheme of the library's prefill attention (prefill.cuh: every fp32 operand x = hi + lo with two fp16
// halves, 22 mantissa bits, and hi*hi + hi*lo + lo*hi accumulated in fp32 by mma.sync m16n8k16), generalised to
//   - ragged steps: a block owns up to 128 consecutive rows of ONE sequence (tiles[2 i] = first row, tiles[2 i + 1] = count),
//   - grouped key/value heads, a sliding window (only the pages the tile's rows can see are visited),
//   - the per-head sigmoid output gate and the sink term of the softmax denominator.
// Scores, softmax and the running sums are fp32.  Head sizes 64 and 128 with dim == vdim; other shapes use the fp32 tiled kernel.
// Also here: the split-key attention of decode rows (flash-decoding: key chunks in parallel, then a merge).
#pragma once
#include "prefill.cuh"
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

constexpr int kAttnTcTile = kTcQ;   // 128 rows a block

template <int DH>
__global__ void __launch_bounds__(kTcThreads, 1) window_attention_h3_kernel(const float* qkvg, StepMeta m, AttnShape s, const int* tiles,
                                                                             const float* k_pool, const float* v_pool, float* out) {
    constexpr int LD = DH + 8, KS = DH / 16, NT = DH / 8;
    extern __shared__ __align__(16) __half h3w_smem[];
    __half* Qh = h3w_smem;                 // [128][LD]
    __half* Ql = Qh + kTcQ * LD;
    __half* Kh = Ql + kTcQ * LD;           // [64][LD]
    __half* Kl = Kh + kTcKT * LD;
    __half* Vh = Kl + kTcKT * LD;
    __half* Vl = Vh + kTcKT * LD;
    const int row0 = tiles[2 * blockIdx.x], M = tiles[2 * blockIdx.x + 1], h = blockIdx.y;
    const int pos0 = m.row_pos[row0];
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[row0]] * m.table_stride;
    const int gkv = h / (s.heads / s.kv_heads);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int r0 = 16 * warp + g, r1 = r0 + 8;
    auto store_split4 = [](const float4& v, __half* hi, __half* lo) {
        __half a[4], b[4];
        split_h(v.x, a[0], b[0]); split_h(v.y, a[1], b[1]); split_h(v.z, a[2], b[2]); split_h(v.w, a[3], b[3]);
        *reinterpret_cast<uint2*>(hi) = make_uint2(pack_h2(a[0], a[1]), pack_h2(a[2], a[3]));
        *reinterpret_cast<uint2*>(lo) = make_uint2(pack_h2(b[0], b[1]), pack_h2(b[2], b[3]));
    };
    for (int i = tid; i < kTcQ * (DH / 4); i += kTcThreads) {
        const int q = i / (DH / 4), d4 = (i % (DH / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q < M) {
            const float* src = qkvg + (size_t)(row0 + q) * s.ld + (size_t)h * DH + d4;   // (the row pitch need not be a multiple of 4)
            v = make_float4(src[0], src[1], src[2], src[3]);
        }
        store_split4(v, Qh + q * LD + d4, Ql + q * LD + d4);
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int last_pos = pos0 + M - 1;
    const int lo = (s.window > 0 && pos0 - s.window + 1 > 0) ? pos0 - s.window + 1 : 0;
    const int warp_first = pos0 + 16 * warp, warp_last = pos0 + min(16 * warp + 15, M - 1);
    const int warp_lo = (s.window > 0 && warp_first - s.window + 1 > 0) ? warp_first - s.window + 1 : 0;
    const uint32_t* qh_row = reinterpret_cast<const uint32_t*>(Qh + (16 * warp + g) * LD) + t;
    const uint32_t* ql_row = reinterpret_cast<const uint32_t*>(Ql + (16 * warp + g) * LD) + t;
    const int lm = lane >> 3, lr = lane & 7;
    const uint32_t k_ld = (uint32_t)(((lr + 8 * (lm >> 1)) * LD + 8 * (lm & 1)) * 2);
    const uint32_t v_ld = (uint32_t)(((lr + 8 * (lm & 1)) * LD + 8 * (lm >> 1)) * 2);
    const uint32_t kh_s = smem_u32(Kh), kl_s = smem_u32(Kl), vh_s = smem_u32(Vh), vl_s = smem_u32(Vl);
    const size_t pitch = (size_t)s.kv_heads * DH;
    for (int t0 = lo / kPageTokens * kPageTokens; t0 <= last_pos; t0 += kTcKT) {   // a key tile = a page
        __syncthreads();
        const size_t tok0 = (size_t)table[t0 / kPageTokens] * kPageTokens;
        for (int i = tid; i < kTcKT * (DH / 4); i += kTcThreads) {
            const int kk = i / (DH / 4), d4 = (i % (DH / 4)) * 4, tk = t0 + kk;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (tk >= lo && tk <= last_pos) {
                const size_t row = (tok0 + kk) * pitch + (size_t)gkv * DH + d4;
                kv = *reinterpret_cast<const float4*>(k_pool + row);
                vv = *reinterpret_cast<const float4*>(v_pool + row);
            }
            store_split4(kv, Kh + kk * LD + d4, Kl + kk * LD + d4);
            store_split4(vv, Vh + kk * LD + d4, Vl + kk * LD + d4);
        }
        __syncthreads();
        if (t0 > warp_last || t0 + kTcKT - 1 < warp_lo || 16 * warp >= M) continue;   // nothing of this page is visible to the warp's rows
        float sc[kTcKT / 8][4];
#pragma unroll
        for (int j = 0; j < kTcKT / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const uint32_t ah[4] = {qh_row[8 * ks], qh_row[8 * ks + 4 * LD], qh_row[8 * ks + 4], qh_row[8 * ks + 4 * LD + 4]};
            const uint32_t al[4] = {ql_row[8 * ks], ql_row[8 * ks + 4 * LD], ql_row[8 * ks + 4], ql_row[8 * ks + 4 * LD + 4]};
#pragma unroll
            for (int jp = 0; jp < kTcKT / 16; ++jp) {
                uint32_t bh[4], bl[4];
                const uint32_t off = (uint32_t)((16 * jp * LD + 16 * ks) * 2) + k_ld;
                ldsm_x4(bh, kh_s + off);
                ldsm_x4(bl, kl_s + off);
                mma_f16(sc[2 * jp], al, bh[0], bh[1]);
                mma_f16(sc[2 * jp + 1], al, bh[2], bh[3]);
                mma_f16(sc[2 * jp], ah, bl[0], bl[1]);
                mma_f16(sc[2 * jp + 1], ah, bl[2], bl[3]);
                mma_f16(sc[2 * jp], ah, bh[0], bh[1]);
                mma_f16(sc[2 * jp + 1], ah, bh[2], bh[3]);
            }
        }
        const int qp0 = pos0 + r0, qp1 = pos0 + r1;
        const int w = s.window > 0 ? s.window : 0x3FFFFFFF;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < kTcKT / 8; ++j) {
            const int key = t0 + 8 * j + 2 * t;
            sc[j][0] = (key <= qp0 && key > qp0 - w && r0 < M) ? sc[j][0] * s.scale : -INFINITY;
            sc[j][1] = (key + 1 <= qp0 && key + 1 > qp0 - w && r0 < M) ? sc[j][1] * s.scale : -INFINITY;
            sc[j][2] = (key <= qp1 && key > qp1 - w && r1 < M) ? sc[j][2] * s.scale : -INFINITY;
            sc[j][3] = (key + 1 <= qp1 && key + 1 > qp1 - w && r1 < M) ? sc[j][3] * s.scale : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
            mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int j = 0; j < kTcKT / 8; ++j) {
            sc[j][0] = mn0 == -INFINITY ? 0.f : expf(sc[j][0] - mn0);
            sc[j][1] = mn0 == -INFINITY ? 0.f : expf(sc[j][1] - mn0);
            sc[j][2] = mn1 == -INFINITY ? 0.f : expf(sc[j][2] - mn1);
            sc[j][3] = mn1 == -INFINITY ? 0.f : expf(sc[j][3] - mn1);
            rs0 += sc[j][0] + sc[j][1];
            rs1 += sc[j][2] + sc[j][3];
        }
        rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1); rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
        rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1); rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
        const float c0 = mn0 == -INFINITY ? 1.f : expf(m0 - mn0), c1 = mn1 == -INFINITY ? 1.f : expf(m1 - mn1);
        l0 = l0 * c0 + rs0;
        l1 = l1 * c1 + rs1;
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int n = 0; n < NT; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
#pragma unroll
        for (int jp = 0; jp < kTcKT / 16; ++jp) {
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x = sc[2 * jp + (i >> 1)][2 * (i & 1)], y = sc[2 * jp + (i >> 1)][2 * (i & 1) + 1];
                __half xh, xl, yh, yl;
                split_h(x, xh, xl);
                split_h(y, yh, yl);
                ph[i] = pack_h2(xh, yh);
                pl[i] = pack_h2(xl, yl);
            }
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t bh[4], bl[4];
                const uint32_t off = (uint32_t)((16 * jp * LD + 16 * np) * 2) + v_ld;
                ldsm_x4_trans(bh, vh_s + off);
                ldsm_x4_trans(bl, vl_s + off);
                mma_f16(o[2 * np], pl, bh[0], bh[1]);
                mma_f16(o[2 * np + 1], pl, bh[2], bh[3]);
                mma_f16(o[2 * np], ph, bl[0], bl[1]);
                mma_f16(o[2 * np + 1], ph, bl[2], bl[3]);
                mma_f16(o[2 * np], ph, bh[0], bh[1]);
                mma_f16(o[2 * np + 1], ph, bh[2], bh[3]);
            }
        }
    }
    float i0 = 0.f, i1 = 0.f;
    if (r0 < M) i0 = attn_gate(s, qkvg, row0 + r0, h) * attn_finish_factor(s, h, m0, l0);
    if (r1 < M) i1 = attn_gate(s, qkvg, row0 + r1, h) * attn_finish_factor(s, h, m1, l1);
    const size_t opitch = (size_t)s.heads * DH;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        if (r0 < M) *reinterpret_cast<float2*>(out + (size_t)(row0 + r0) * opitch + (size_t)h * DH + 8 * n + 2 * t) = make_float2(o[n][0] * i0, o[n][1] * i0);
        if (r1 < M) *reinterpret_cast<float2*>(out + (size_t)(row0 + r1) * opitch + (size_t)h * DH + 8 * n + 2 * t) = make_float2(o[n][2] * i1, o[n][3] * i1);
    }
}

// ---- decode rows with long windows: key chunks in parallel -----------------------------------------------------------------
// grid (rows, heads, splits): split z of a (row, head) takes keys lo + z * chunk .. and leaves its partial (max, sum, o[dv]) in
// `part`; attention_merge_kernel combines the splits and applies the gate.  chunk = ceil(visible keys / splits).
template <int PL>
__global__ void __launch_bounds__(kAttnWarps * 32) window_attention_split_kernel(const float* qkvg, StepMeta m, AttnShape s, const int* rows, int splits,
                                                                                  const float* k_pool, const float* v_pool, float* part) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    extern __shared__ float sm[];
    const int bx = blockIdx.x, t = rows ? rows[bx] : bx, h = blockIdx.y, z = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = m.row_pos[t];
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[t]] * m.table_stride;
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
    const int chunk = (pos - lo + 1 + splits - 1) / splits;
    const int j0 = lo + z * chunk, j1 = min(pos, j0 + chunk - 1);
    float mx = -INFINITY, l = 0.f;
    const size_t kstride = (size_t)s.kv_heads * s.dim, vstride = attn_vstride(s);
    // a warp takes its keys four at a time: the four K rows (and then the four V rows) are requested together
    for (int jb = j0 + 4 * warp; jb <= j1; jb += 4 * kAttnWarps) {
        size_t off[4];
        float sc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = min(jb + u, j1);
            off[u] = (size_t)table[j / kPageTokens] * kPageTokens + j % kPageTokens;
            sc[u] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int d = lane + 32 * i;
            if (d < s.dim) {
#pragma unroll
                for (int u = 0; u < 4; ++u) sc[u] = fmaf(qr[i], k_pool[off[u] * kstride + (size_t)g * s.dim + d], sc[u]);
            }
        }
        float vv[4][PL];
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int d = lane + 32 * i;
#pragma unroll
            for (int u = 0; u < 4; ++u) vv[u][i] = d < s.vdim ? v_pool[off[u] * vstride + (size_t)g * s.vdim + d] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float su = warp_sum(sc[u]) * s.scale;
            if (jb + u <= j1) {
                const float nm = fmaxf(mx, su);
                const float corr = expf(mx - nm), p = expf(su - nm);
                l = l * corr + p;
#pragma unroll
                for (int i = 0; i < PL; ++i) o[i] = fmaf(p, vv[u][i], o[i] * corr);
                mx = nm;
            }
        }
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
    float Mx = -INFINITY;
    for (int w = 0; w < kAttnWarps; ++w) Mx = fmaxf(Mx, pm[w]);
    float L = 0.f, f[kAttnWarps];
    for (int w = 0; w < kAttnWarps; ++w) {
        f[w] = (pm[w] == -INFINITY) ? 0.f : expf(pm[w] - Mx);
        L += pl[w] * f[w];
    }
    float* dst = part + (((size_t)bx * s.heads + h) * splits + z) * (size_t)(s.vdim + 2);
    for (int d = threadIdx.x; d < s.vdim; d += blockDim.x) {
        float acc = 0.f;
        for (int w = 0; w < kAttnWarps; ++w) acc += po[w * s.vdim + d] * f[w];
        dst[2 + d] = acc;
    }
    if (threadIdx.x == 0) {
        dst[0] = Mx;
        dst[1] = L;
    }
}
// one warp per (row, head): lane z holds split z's (max, sum); the output coordinates are spread over the lanes
__global__ void attention_merge_kernel(const float* part, const float* qkvg, StepMeta m, AttnShape s, const int* rows, int n_rows, int splits, float* out) {
    pdl_launch_dependents();   // the kernel behind this one may be scheduled (and a few-row product may fetch its weights) ...
    pdl_wait_prior_grid();     // ... while this one waits here for the kernel before it, when it was launched ahead of its end
    const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wid >= n_rows * s.heads) return;
    const int bx = wid / s.heads, h = wid % s.heads, t = rows ? rows[bx] : bx;
    const size_t ps = (size_t)(s.vdim + 2);
    const float* p = part + ((size_t)bx * s.heads + h) * splits * ps;
    const float mz = lane < splits ? p[(size_t)lane * ps] : -INFINITY;
    const float lz = lane < splits ? p[(size_t)lane * ps + 1] : 0.f;
    const float Mx = warp_max(mz);
    const float fz = mz == -INFINITY ? 0.f : expf(mz - Mx);
    const float L = warp_sum(lz * fz);
    const float fin = attn_finish_factor(s, h, Mx, L) * attn_gate(s, qkvg, t, h);
    // every split's factor in registers first, so that the loads of a coordinate's partials do not wait on one another
    constexpr int kMaxSplits = 32;   // (a lane holds a split's statistics)
    float fs[kMaxSplits];
#pragma unroll
    for (int z = 0; z < kMaxSplits; ++z) fs[z] = __shfl_sync(0xFFFFFFFFu, fz, z);
    for (int d0 = 0; d0 < s.vdim; d0 += 32) {
        const int d = d0 + lane;
        float acc = 0.f;
#pragma unroll
        for (int z = 0; z < kMaxSplits; ++z)
            if (z < splits && d < s.vdim) acc = fmaf(p[(size_t)z * ps + 2 + d], fs[z], acc);
        if (d < s.vdim) out[(size_t)t * (s.heads * s.vdim) + (size_t)h * s.vdim + d] = acc * fin;
    }
}

}  // namespace seq
}  // namespace tib

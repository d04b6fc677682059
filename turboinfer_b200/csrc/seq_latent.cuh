// seq_latent.cuh -- latent attention of the layered sequence engine: softmax attention whose per-head keys and values are
// linear images (Uk, Uv) of ONE cached low-rank vector c per token, plus one rotated key part shared by all heads.
//
// The cache holds, per token, the row [c (rank) | rotated key part (rot)] in fp32 -- nothing per head.  The per-head products
// are moved to the query side and behind the weighted sum, which is the same arithmetic re-associated:
//     score_h(i, j) = (q_h . Uk_h c_j + qr_h . kr_j) * scale = ((Uk_h^T q_h) . c_j + qr_h . kr_j) * scale
//     out_h(i)      = sum_j p_h(i, j) Uv_h c_j                = Uv_h (sum_j p_h(i, j) c_j)
// so the attention itself is one key/value head of size rank + rot (values = the first rank coordinates of the key row) shared
// by all query heads, and runs on the paged attention kernels of seq_kernels.cuh / seq_attn_tc.cuh (value pool = key pool; a
// sliding window, a sink term and a per-head output gate -- one number a head, so it commutes with Uv -- are the layer's choice).  This file holds what is special: the cache append and the query's rotated part.
#pragma once
#include "seq_attn_tc.cuh"
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

struct LatentShape {
    int heads, dim, rot, rank;   // per head: `dim` unrotated and `rot` rotated query coordinates; cached row = rank + rot
    int ld;                      // row stride of the fused projection [q | dkv | ...]
    int off_q, off_dkv;          // column of q (heads * (dim + rot)) and of the down projection (rank + rot); off_dkv < 0: the layer
                                 // reads another layer's cache and appends nothing
    float eps;
    int rot_half;                // 1: rotated coordinate i pairs with i + rot / 2 instead of (2 i, 2 i + 1)
};
// One block per row.  Own cache: c = dkv[:rank] / rms * cnorm -> page row; rotated key part -> behind it.  Every head's rotated
// query part -> qabs[t][h][rank ...] (the absorbed part [0, rank) is written by the product with Uk^T).  Pair i of the rotated
// parts -- (2i, 2i + 1), or (i, i + rot / 2) with rot_half -- turns by position * inv_freq[i], angle in fp32.
__global__ void latent_prepare_kernel(const float* proj, StepMeta m, LatentShape s, const float* inv_freq, const float* cnorm, float* pool, float* qabs) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    __shared__ float red[32];
    const int t = blockIdx.x, pos = m.row_pos[t];
    const float* row = proj + (size_t)t * s.ld;
    const int kd = s.rank + s.rot;
    if (s.off_dkv >= 0) {
        const int slot = m.ent_slot[m.row_ent[t]];
        const int page = m.page_table[(size_t)slot * m.table_stride + pos / kPageTokens];
        float* dst = pool + ((size_t)page * kPageTokens + pos % kPageTokens) * kd;
        const float* src = row + s.off_dkv;
        float ss = 0.f;
        for (int i = threadIdx.x; i < s.rank; i += blockDim.x) ss += src[i] * src[i];
        ss = block_sum(ss, red);
        const float sc = 1.f / sqrtf(ss / (float)s.rank + s.eps);
        for (int i = threadIdx.x; i < s.rank; i += blockDim.x) dst[i] = src[i] * sc * cnorm[i];
        for (int i = threadIdx.x; i < s.rot / 2; i += blockDim.x) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            const int i0 = s.rot_half ? i : 2 * i, i1 = s.rot_half ? i + s.rot / 2 : 2 * i + 1;
            const float a = src[s.rank + i0], b = src[s.rank + i1];
            dst[s.rank + i0] = a * cs - b * sn;
            dst[s.rank + i1] = b * cs + a * sn;
        }
    }
    for (int x = threadIdx.x; x < s.heads * (s.rot / 2); x += blockDim.x) {
        const int h = x / (s.rot / 2), i = x % (s.rot / 2);
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        const float* q = row + s.off_q + (size_t)h * (s.dim + s.rot) + s.dim;
        float* dst = qabs + ((size_t)t * s.heads + h) * kd + s.rank;
        const int i0 = s.rot_half ? i : 2 * i, i1 = s.rot_half ? i + s.rot / 2 : 2 * i + 1;
        const float a = q[i0], b = q[i1];
        dst[i0] = a * cs - b * sn;
        dst[i1] = b * cs + a * sn;
    }
}
// Uk [heads * dim][rank] -> per head its transpose [heads][rank][dim]: the weight of the query-side product
template <typename WT>
__global__ void transpose_heads_kernel(const WT* uk, int heads, int dim, int rank, WT* out) {
    const size_t n = (size_t)heads * dim * rank;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t h = i / ((size_t)dim * rank), r = (i / dim) % rank, d = i % dim;
        out[i] = uk[(h * dim + d) * rank + r];
    }
}

// Prompt portions of latent attention on the warp-level tensor cores at fp32 accuracy (bf16 mode): the split-half scheme of
// window_attention_h3_kernel (x = hi + lo with two fp16 halves, hi*hi + hi*lo + lo*hi accumulated in fp32 by mma.sync m16n8k16;
// scores, softmax with the sink and running sums in fp32) for ONE shared key/value head whose values are the leading DV
// coordinates of its DK-wide key rows -- so the key tile in shared memory is also the value tile and nothing is loaded twice.
// A block owns up to 64 consecutive rows of one sequence and one query head; its 8 warps are 4 row groups x 2 halves of the
// value columns: both warps of a row group compute the 16 x 64 scores of a key tile (the softmax needs whole rows), each
// accumulates its half of the DV output columns -- a DV-wide output tile of 16 rows does not fit one warp's registers.
// tiles[2 i] = first row, tiles[2 i + 1] = row count; q = absorbed queries [T][heads][DK]; pool = [pages * 64][DK].
constexpr int kLatQ = 64;
template <int DK> constexpr size_t latent_h3_smem_bytes() { return ((size_t)2 * kLatQ + 2 * kTcKT) * (DK + 8) * sizeof(__half); }
template <int DK, int DV>
__global__ void __launch_bounds__(256, 1) latent_attention_h3_kernel(const float* q, StepMeta m, AttnShape s, const int* tiles, const float* pool, float* out) {
    constexpr int LD = DK + 8, KS = DK / 16, NTH = DV / 16;   // NTH: 8-column output tiles a warp owns = (DV / 2) / 8
    static_assert(DK % 16 == 0 && DV % 32 == 0 && DV <= DK, "tile sizes");
    extern __shared__ __align__(16) __half lat_smem[];
    __half* Qh = lat_smem;                 // [64][LD]
    __half* Ql = Qh + kLatQ * LD;
    __half* Kh = Ql + kLatQ * LD;          // [64][LD]: keys, and in their leading DV columns the values
    __half* Kl = Kh + kTcKT * LD;
    const int row0 = tiles[2 * blockIdx.x], M = tiles[2 * blockIdx.x + 1], h = blockIdx.y;
    const int pos0 = m.row_pos[row0];
    const int* table = m.page_table + (size_t)m.ent_slot[m.row_ent[row0]] * m.table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int rg = warp & 3, vh = warp >> 2;
    const int r0 = 16 * rg + g, r1 = r0 + 8;
    auto store_split4 = [](const float4& v, __half* hi, __half* lo) {
        __half a[4], b[4];
        split_h(v.x, a[0], b[0]); split_h(v.y, a[1], b[1]); split_h(v.z, a[2], b[2]); split_h(v.w, a[3], b[3]);
        *reinterpret_cast<uint2*>(hi) = make_uint2(pack_h2(a[0], a[1]), pack_h2(a[2], a[3]));
        *reinterpret_cast<uint2*>(lo) = make_uint2(pack_h2(b[0], b[1]), pack_h2(b[2], b[3]));
    };
    for (int i = tid; i < kLatQ * (DK / 4); i += 256) {
        const int qi = i / (DK / 4), d4 = (i % (DK / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (qi < M) {
            const float* src = q + (size_t)(row0 + qi) * s.ld + (size_t)h * DK + d4;
            v = make_float4(src[0], src[1], src[2], src[3]);
        }
        store_split4(v, Qh + qi * LD + d4, Ql + qi * LD + d4);
    }
    float o[NTH][4];
#pragma unroll
    for (int n = 0; n < NTH; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int last_pos = pos0 + M - 1;
    const int lo = (s.window > 0 && pos0 - s.window + 1 > 0) ? pos0 - s.window + 1 : 0;   // first key any row of the tile sees
    const int warp_first = pos0 + 16 * rg, warp_last = pos0 + min(16 * rg + 15, M - 1);
    const int warp_lo = (s.window > 0 && warp_first - s.window + 1 > 0) ? warp_first - s.window + 1 : 0;
    const uint32_t* qh_row = reinterpret_cast<const uint32_t*>(Qh + (16 * rg + g) * LD) + t;
    const uint32_t* ql_row = reinterpret_cast<const uint32_t*>(Ql + (16 * rg + g) * LD) + t;
    const int lm = lane >> 3, lr = lane & 7;
    const uint32_t k_ld = (uint32_t)(((lr + 8 * (lm >> 1)) * LD + 8 * (lm & 1)) * 2);
    const uint32_t v_ld = (uint32_t)(((lr + 8 * (lm & 1)) * LD + 8 * (lm >> 1)) * 2);
    const uint32_t kh_s = smem_u32(Kh), kl_s = smem_u32(Kl);
    for (int t0 = lo / kPageTokens * kPageTokens; t0 <= last_pos; t0 += kTcKT) {   // a key tile = a page; pages below the window are not visited
        __syncthreads();
        const size_t tok0 = (size_t)table[t0 / kPageTokens] * kPageTokens;
        for (int i = tid; i < kTcKT * (DK / 4); i += 256) {
            const int kk = i / (DK / 4), d4 = (i % (DK / 4)) * 4;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t0 + kk >= lo && t0 + kk <= last_pos) kv = *reinterpret_cast<const float4*>(pool + (tok0 + kk) * (size_t)DK + d4);
            store_split4(kv, Kh + kk * LD + d4, Kl + kk * LD + d4);
        }
        __syncthreads();
        if (t0 > warp_last || t0 + kTcKT - 1 < warp_lo || 16 * rg >= M) continue;   // nothing of this page is visible to the warp's rows
        float sc[kTcKT / 8][4];
#pragma unroll
        for (int j = 0; j < kTcKT / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll 4
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
        for (int n = 0; n < NTH; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
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
            for (int np = 0; np < NTH / 2; ++np) {
                uint32_t bh[4], bl[4];
                const uint32_t off = (uint32_t)((16 * jp * LD + vh * (DV / 2) + 16 * np) * 2) + v_ld;
                ldsm_x4_trans(bh, kh_s + off);
                ldsm_x4_trans(bl, kl_s + off);
                mma_f16(o[2 * np], pl, bh[0], bh[1]);
                mma_f16(o[2 * np + 1], pl, bh[2], bh[3]);
                mma_f16(o[2 * np], ph, bl[0], bl[1]);
                mma_f16(o[2 * np + 1], ph, bl[2], bl[3]);
                mma_f16(o[2 * np], ph, bh[0], bh[1]);
                mma_f16(o[2 * np + 1], ph, bh[2], bh[3]);
            }
        }
    }
    const float i0 = r0 < M ? attn_finish_factor(s, h, m0, l0) * attn_gate(s, q, row0 + r0, h) : 0.f;
    const float i1 = r1 < M ? attn_finish_factor(s, h, m1, l1) * attn_gate(s, q, row0 + r1, h) : 0.f;
    const size_t opitch = (size_t)s.heads * DV;
#pragma unroll
    for (int n = 0; n < NTH; ++n) {
        const size_t col = (size_t)h * DV + vh * (DV / 2) + 8 * n + 2 * t;
        if (r0 < M) *reinterpret_cast<float2*>(out + (size_t)(row0 + r0) * opitch + col) = make_float2(o[n][0] * i0, o[n][1] * i0);
        if (r1 < M) *reinterpret_cast<float2*>(out + (size_t)(row0 + r1) * opitch + col) = make_float2(o[n][2] * i1, o[n][3] * i1);
    }
}

}  // namespace seq
}  // namespace tib

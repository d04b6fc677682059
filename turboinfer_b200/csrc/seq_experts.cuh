// seq_experts.cuh -- feed-forward forms of the layered sequence engine beside the gated one of seq_kernels.cuh: the polynomial
// norm activation of a dense feed-forward, and routed experts (router, group-limited choice, identity experts, shared expert).
//
// Routed experts run as two products over stacked weights: [gate_0; up_0; gate_1; up_1; ...; shared gate; shared up] in front and
// the down matrices side by side along K behind, with the routing weight (zero for an expert the token did not choose) folded
// into the activation between them: sum_e w_e Down_e a_e = [Down_0 | Down_1 | ...] [w_0 a_0; w_1 a_1; ...].  Router logits,
// softmax, choice and weights are fp32.
#pragma once
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

// y[t] = a N(z) + b N(z^2) + c N(z^3) + e with N(u) = u / sqrt(mean(u^2) + eps) over the F coordinates of row t; coef = (a, b, c, e)
__global__ void polynorm_kernel(const float* z, int ld, int F, const float* coef, float eps, float* y) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    __shared__ float red[32];
    const int t = blockIdx.x;
    const float* zr = z + (size_t)t * ld;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        s2 += v2;
        s4 += v2 * v2;
        s6 += v2 * v2 * v2;
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    const float r1 = coef[0] / sqrtf(s2 / (float)F + eps), r2 = coef[1] / sqrtf(s4 / (float)F + eps), r3 = coef[2] / sqrtf(s6 / (float)F + eps);
    const float e = coef[3];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        y[(size_t)t * F + i] = fmaf(v, r1, fmaf(v2, r2, fmaf(v2 * v, r3, e)));
    }
}

struct RouteShape {
    int n_real, n_id;    // experts with weights, identity experts behind them (router outputs = n_real + n_id)
    int top;             // experts a token uses
    int groups, keep;    // equal groups of neighbouring router outputs; only the `keep` groups with the largest member can be chosen
    int by_logits;       // 1: `correction` is a bias added to the logits, the `top` largest biased logits are chosen and the weights are
                         // the softmax over the chosen ones (no groups)
};
// One warp per row.  s = softmax(logits); choice = s + correction; the best `keep` groups by their largest choice score stay, the
// `top` largest choice scores among them are picked (first index wins a tie); weights = s over the picked ones / (their sum + 1e-20).
// wdense[t][e] = weight of real expert e or 0; idw[t] = sum of the weights of picked identity experts.
// Shared memory per warp: s[n], choice[n], group score[groups], group kept[groups].
// used (optional; the grid is then ONE block that holds all rows): used[e] = 1 when some row picked real expert e, else 0.
__global__ void moe_route_kernel(const float* proj, int ld, int off, RouteShape r, const float* correction, int T, float* wdense, float* idw, int* used) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ float rsm[];
    const int n = r.n_real + r.n_id, per = 2 * n + 2 * r.groups;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t < T) {
    float* s = rsm + (size_t)warp * per;
    float* ch = s + n;
    float* gs = ch + n;
    float* kept = gs + r.groups;
    const float* z = proj + (size_t)t * ld + off;
    float mx = -INFINITY;
    for (int i = lane; i < n; i += 32) mx = fmaxf(mx, z[i] + (r.by_logits ? correction[i] : 0.f));
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) {
        const float e = expf(z[i] + (r.by_logits ? correction[i] : 0.f) - mx);
        s[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    for (int i = lane; i < n; i += 32) {
        // by logits: the choice is made among the biased logits, and exp(. - max) of a chosen one over the chosen ones' sum is the
        // softmax over the chosen logits (the largest logit is always among them, so nothing underflows that matters)
        if (r.by_logits) { ch[i] = z[i] + correction[i]; s[i] = fmaxf(s[i], 1e-37f); }
        else { s[i] = s[i] / sum; ch[i] = s[i] + correction[i]; }
    }
    __syncwarp();
    const int size = n / r.groups;
    for (int g = lane; g < r.groups; g += 32) {
        float b = -INFINITY;
        for (int i = g * size; i < (g + 1) * size; ++i) b = fmaxf(b, ch[i]);
        gs[g] = b;
        kept[g] = 0.f;
    }
    __syncwarp();
    // keep the best groups: a group outside them has its members' choice scores set to -inf
    if (r.keep < r.groups) {
        for (int k = 0; k < r.keep; ++k) {
            float b = -INFINITY;
            int bi = 0x7FFFFFFF;
            for (int g = lane; g < r.groups; g += 32)
                if (gs[g] > b) { b = gs[g]; bi = g; }      // (ascending g within a lane: the first maximum stays)
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xFFFFFFFFu, b, o);
                const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
                if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
            }
            if (lane == 0 && bi != 0x7FFFFFFF) {
                kept[bi] = 1.f;
                gs[bi] = -INFINITY;   // not to be found again
            }
            __syncwarp();
        }
        for (int i = lane; i < n; i += 32)
            if (kept[i / size] == 0.f) ch[i] = -INFINITY;
        __syncwarp();
    }
    for (int i = lane; i < r.n_real; i += 32) wdense[(size_t)t * r.n_real + i] = 0.f;
    __syncwarp();
    float tot = 0.f;
    int picked[8];   // up to 8 picks are remembered in registers per pass; more picks run in further passes over `done` marks
    // picks are marked by moving their choice score to NaN-free -inf after remembering them in `s` order: weights need s only
    // first pass: find the picks and their sum
    const int top = min(r.top, n);
    for (int k0 = 0; k0 < top; k0 += 8) {
        const int kn = min(8, top - k0);
        for (int k = 0; k < kn; ++k) {
            float b = -INFINITY;
            int bi = 0x7FFFFFFF;
            for (int i = lane; i < n; i += 32)
                if (ch[i] > b) { b = ch[i]; bi = i; }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xFFFFFFFFu, b, o);
                const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
                if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
            }
            picked[k] = bi;
            if (bi != 0x7FFFFFFF) {
                tot += s[bi];
                if (lane == 0) ch[bi] = -INFINITY;
            }
            __syncwarp();
        }
        // remember the picks of this pass: negative s marks a pick (s > 0 always), so that the weights can be written once tot is known
        if (lane == 0)
            for (int k = 0; k < kn; ++k)
                if (picked[k] != 0x7FFFFFFF) s[picked[k]] = -s[picked[k]];
        __syncwarp();
    }
    const float inv = 1.f / (tot + 1e-20f);
    float wi = 0.f;
    for (int i = lane; i < n; i += 32)
        if (s[i] < 0.f) {
            const float w = -s[i] * inv;
            if (i < r.n_real) wdense[(size_t)t * r.n_real + i] = w;
            else wi += w;
        }
    wi = warp_sum(wi);
    if (lane == 0) idw[t] = wi;
    }
    if (used) {
        __syncthreads();
        for (int e = threadIdx.x; e < r.n_real; e += blockDim.x) {
            int u = 0;
            for (int x = 0; x < T; ++x) u |= wdense[(size_t)x * r.n_real + e] != 0.f;
            used[e] = u;
        }
    }
}

// act[t][e * F + c] = wdense[t][e] * silu(gate_e[c]) * up_e[c] (0 without reading when the weight is 0), and behind the experts
// act[t][E * F + c] = sigmoid(proj[t][off_sg]) * silu(gate_s[c]) * up_s[c] for the shared expert (Fs = 0: none).
// Expert e's [gate | up] block starts at proj column off_gu + e * 2F, the shared expert's at off_sh.
__global__ void moe_act_kernel(const float* proj, int ld, int off_gu, int E, int F, const float* wdense, int off_sh, int Fs, int off_sg, float* act, int T) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int W = E * F + Fs;
    const size_t n = (size_t)T * W;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / W;
        const int x = (int)(i % W);
        const float* row = proj + t * ld;
        float v = 0.f;
        if (x < E * F) {
            const int e = x / F, c = x % F;
            const float w = wdense[t * E + e];
            if (w != 0.f) {
                const float g = row[off_gu + (size_t)e * 2 * F + c], u = row[off_gu + (size_t)e * 2 * F + F + c];
                v = w * (g / (1.f + expf(-g))) * u;
            }
        } else {
            const int c = x - E * F;
            const float g = row[off_sh + c], u = row[off_sh + Fs + c];
            v = (g / (1.f + expf(-g))) * u;
            if (off_sg >= 0) v /= 1.f + expf(-row[off_sg]);
        }
        act[i] = v;
    }
}

// per-token side input: g[t][j] = g[t][j] * side_embed[tok[t]][layer * ds + j]   (g holds gelu_tanh(side.gate x) on entry)
template <typename WT>
__global__ void side_mul_kernel(float* g, StepMeta m, const WT* side_embed, int row_len, int layer, int ds) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const size_t n = (size_t)m.T * ds;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / ds, j = i % ds;
        g[i] *= to_f32(side_embed[(size_t)m.tok[t] * row_len + (size_t)layer * ds + j]);
    }
}

}  // namespace seq
}  // namespace tib

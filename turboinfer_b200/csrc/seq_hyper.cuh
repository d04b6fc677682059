// seq_hyper.cuh -- hyper-connections of the layered sequence engine: the residual is S copies ("streams") X_0 .. X_(S-1) of the
// embedding output instead of one vector.  A sublayer reads one mixture of them and writes into all of them:
//     u = sum_s in[s] X_s,   y = sublayer(norm(u)),   X_t <- sum_s mix[s][t] X_s + out[t] y   (all t at once, from the old copies)
// and the model's output is sum_s X_s.  One stream with in = mix = out = 1 is the ordinary pre-norm residual x <- x + y, which is
// how the engine runs models with norms in front of the sublayers only.
//
// hyper_kernel closes one sublayer and opens the next in a single pass over a row (as postnorm_residual_kernel does for norms
// around the sublayers): the update with the finished sublayer's result (+ its output bias), the sum of the streams (what a layer
// run leaves, and what the head reads), and the next sublayer's input norm(sum_s in'[s] X_s) * gain.  Everything is fp32.
#pragma once
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

constexpr int kMaxStreams = 16;

struct HyperArgs {
    float* X;               // [T][S][D], updated in place
    const float* y;         // [T][D] result of the sublayer that ends here; null: nothing ends (the first sublayer of a step)
    const float* bias;      // [D] or null: added to y
    const float* mix;       // [S][S], indexed [from][to]
    const float* out;       // [S]
    const float* in_next;   // [S] or null: no sublayer follows (the head reads `sum`)
    const float* gain;      // norm in front of the next sublayer: [D], or one number when gvec = 0
    float* h;               // [T][D] the next sublayer's input
    float* sum;             // [T][D] or null: sum of the streams after the update
    int S, D, gvec;
    float eps;
};

__global__ void __launch_bounds__(256) hyper_kernel(HyperArgs a) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    __shared__ float red[32];
    __shared__ float s_mix[kMaxStreams * kMaxStreams], s_out[kMaxStreams], s_in[kMaxStreams];
    const int t = blockIdx.x, S = a.S, D = a.D;
    if (a.y)
        for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = a.mix[i];
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = a.y ? a.out[threadIdx.x] : 0.f;
        s_in[threadIdx.x] = a.in_next ? a.in_next[threadIdx.x] : 0.f;
    }
    __syncthreads();
    float* xr = a.X + (size_t)t * S * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float x[kMaxStreams];
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s) x[s] = s < S ? xr[(size_t)s * D + d] : 0.f;
        if (a.y) {
            const float yv = a.y[(size_t)t * D + d] + (a.bias ? a.bias[d] : 0.f);
            float n[kMaxStreams];
#pragma unroll
            for (int to = 0; to < kMaxStreams; ++to) {
                if (to >= S) continue;
                float acc = 0.f;
#pragma unroll
                for (int s = 0; s < kMaxStreams; ++s)
                    if (s < S) acc = fmaf(s_mix[s * S + to], x[s], acc);
                n[to] = fmaf(s_out[to], yv, acc);
            }
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < S) {
                    x[s] = n[s];
                    xr[(size_t)s * D + d] = n[s];
                }
        }
        if (a.sum) {
            float tot = 0.f;
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < S) tot += x[s];
            a.sum[(size_t)t * D + d] = tot;
        }
        if (a.in_next) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < S) u = fmaf(s_in[s], x[s], u);
            a.h[(size_t)t * D + d] = u;   // (the thread that wrote it scales it below)
            ss += u * u;
        }
    }
    if (!a.in_next) return;
    ss = block_sum(ss, red);
    const float sc = 1.f / sqrtf(ss / (float)D + a.eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) a.h[(size_t)t * D + d] *= sc * a.gain[a.gvec ? d : 0];
}

}  // namespace seq
}  // namespace tib

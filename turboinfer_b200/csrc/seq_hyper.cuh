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
    // a step whose entries all bring ONE row (decoding): the next sublayer's short convolution h + conv(h) rides along -- it reads
    // the slot's state only -- and the slot's state is shifted here (the layout of short_conv_kernel); null: the step runs that kernel
    const float* conv_w;    // [D][taps]
    float* conv_state;      // [slots][taps - 1][D]
    float* hc;              // [T][D]
    int taps;
};

// NS > 0: the number of streams, known when the kernel is compiled (the copies of a coordinate live in registers);
// NS = 0: any number up to kMaxStreams (small arrays indexed at run time).  V = 4: a thread takes four neighbouring coordinates with
// 16-byte loads and stores (D in whole fours), V = 1: one coordinate at a time.
// A step of few rows is a handful of blocks whose time is the latency of their loads, one after the other: it is launched with as many
// threads a row as the registers allow (hyper_max_threads), so that a thread meets one or two coordinates; many rows run 256 a row.
template <int NS> constexpr int hyper_max_threads() { return NS == 0 ? 256 : NS <= 4 ? 1024 : 512; }
template <int V> __device__ __forceinline__ void hyper_load(const float* p, float (&v)[V]) {
    if constexpr (V == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
        v[0] = *p;
    }
}
template <int V> __device__ __forceinline__ void hyper_store(float* p, const float (&v)[V]) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else *p = v[0];
}
template <int NS, int V>
__global__ void __launch_bounds__(V == 4 ? 256 : hyper_max_threads<NS>()) hyper_kernel(HyperArgs a, StepMeta m) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    constexpr int CAP = NS > 0 ? NS : kMaxStreams;
    __shared__ float red[32];
    __shared__ float s_mix[kMaxStreams * kMaxStreams], s_out[kMaxStreams], s_in[kMaxStreams];
    const int t = blockIdx.x, S = NS > 0 ? NS : a.S, D = a.D;
    if (a.y)
        for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = a.mix[i];
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = a.y ? a.out[threadIdx.x] : 0.f;
        s_in[threadIdx.x] = a.in_next ? a.in_next[threadIdx.x] : 0.f;
    }
    __syncthreads();
    float* xr = a.X + (size_t)t * S * D;
    float ss = 0.f;
    for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
        float x[CAP][V];
#pragma unroll
        for (int s = 0; s < CAP; ++s)
            if (s < S) hyper_load<V>(xr + (size_t)s * D + d, x[s]);
        if (a.y) {
            float yv[V], bv[V];
            hyper_load<V>(a.y + (size_t)t * D + d, yv);
            if (a.bias) {
                hyper_load<V>(a.bias + d, bv);
#pragma unroll
                for (int v = 0; v < V; ++v) yv[v] += bv[v];
            }
            float n[CAP][V];
#pragma unroll
            for (int to = 0; to < CAP; ++to)
                if (to < S) {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        float acc = 0.f;
#pragma unroll
                        for (int s = 0; s < CAP; ++s)
                            if (s < S) acc = fmaf(s_mix[s * S + to], x[s][v], acc);
                        n[to][v] = fmaf(s_out[to], yv[v], acc);
                    }
                }
#pragma unroll
            for (int s = 0; s < CAP; ++s)
                if (s < S) {
#pragma unroll
                    for (int v = 0; v < V; ++v) x[s][v] = n[s][v];
                    hyper_store<V>(xr + (size_t)s * D + d, x[s]);
                }
        }
        if (a.sum) {
            float tot[V];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                tot[v] = 0.f;
#pragma unroll
                for (int s = 0; s < CAP; ++s)
                    if (s < S) tot[v] += x[s][v];
            }
            hyper_store<V>(a.sum + (size_t)t * D + d, tot);
        }
        if (a.in_next) {
            float u[V];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                u[v] = 0.f;
#pragma unroll
                for (int s = 0; s < CAP; ++s)
                    if (s < S) u[v] = fmaf(s_in[s], x[s][v], u[v]);
                ss += u[v] * u[v];
            }
            hyper_store<V>(a.h + (size_t)t * D + d, u);   // (the thread that wrote it scales it below)
        }
    }
    if (!a.in_next) return;
    ss = block_sum(ss, red);
    const float sc = 1.f / sqrtf(ss / (float)D + a.eps);
    if (!a.conv_w) {
        for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
            float u[V];
            hyper_load<V>(a.h + (size_t)t * D + d, u);
#pragma unroll
            for (int v = 0; v < V; ++v) u[v] *= sc * a.gain[a.gvec ? d + v : 0];
            hyper_store<V>(a.h + (size_t)t * D + d, u);
        }
        return;
    }
    const int e = m.row_ent[t], pos = m.ent_pos0[e], taps = a.taps;
    float* st = a.conv_state + (size_t)m.ent_slot[e] * (taps - 1) * D;
    for (int d0 = threadIdx.x * V; d0 < D; d0 += blockDim.x * V)
        for (int d = d0; d < d0 + V; ++d) {
            const float hv = a.h[(size_t)t * D + d] * (sc * a.gain[a.gvec ? d : 0]);
            float acc = fmaf(a.conv_w[(size_t)d * taps + taps - 1], hv, hv);
            for (int j = 0; j + 1 < taps; ++j) {   // state entry j holds the input at position pos - (taps - 1) + j
                const float v = pos - (taps - 1) + j >= 0 ? st[(size_t)j * D + d] : 0.f;
                acc = fmaf(a.conv_w[(size_t)d * taps + j], v, acc);
                if (j > 0) st[(size_t)(j - 1) * D + d] = v;
            }
            if (taps > 1) st[(size_t)(taps - 2) * D + d] = hv;
            a.hc[(size_t)t * D + d] = acc;
        }
}

}  // namespace seq
}  // namespace tib

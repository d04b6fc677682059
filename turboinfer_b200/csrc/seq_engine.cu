// seq_engine.cu -- implementation of include/ti_b200_seq.h: the layered sequence engine (sm_100a).
//
// Host side: model description and named tensors, the page pool / state-slot manager, the ragged step, the
// continuous-batching generation loop and the sampler launch.  Device side: seq_kernels.cuh (+ sampling.cuh, the sampler the
// rest of the library uses).  One library stream; a step is enqueued without host synchronisation until its results are read.
#include "../../include/ti_b200_seq.h"

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "seq_kernels.cuh"
#include "seq_gemm_tc.cuh"
#include "seq_attn_tc.cuh"
#include "seq_recurrent.cuh"
#include "seq_latent.cuh"
#include "seq_experts.cuh"
#include "seq_headmix.cuh"
#include "seq_hyper.cuh"
#include "sampling.cuh"

using namespace tib;
using namespace tib::seq;

namespace {

thread_local std::string g_err;
int g_device = -1, g_num_sms = 0;
cudaStream_t g_stream = nullptr;
uint64_t g_launches = 0;
size_t g_smem_optin = 0;
bool g_use_tiled_attn = true;   // TURBOINFER_B200_SEQ_TILED_ATTN=0: every row goes through the row-at-a-time attention kernel
constexpr int kAttnTiledMinRows = 8;
constexpr int kAttnMaxSplits = 16;    // key chunks of a decode row's attention   // portions at least this long are cut into attention tiles
bool g_use_pdl = true;  // TURBOINFER_B200_SEQ_PDL=0: the few-row products wait for their predecessor before they start (A/B measurements)
bool g_use_row_mma = true;   // TURBOINFER_B200_SEQ_ROW_MMA=0: few-row products stay on the fp32 multiply-add kernel (A/B measurements)
bool g_use_tc = true;   // TURBOINFER_B200_SEQ_TC=0: prompt-side products stay on the warp-level tensor path (A/B measurements)

int fail(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_err = buf;
    return 1;
}
#define CK(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) return fail("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)
#define TRY(expr)            \
    do {                     \
        int rc_ = (expr);    \
        if (rc_ != 0) return rc_; \
    } while (0)
#define LAUNCHED()     \
    do {               \
        ++g_launches;  \
        CK(cudaGetLastError()); \
    } while (0)

template <typename T>
struct DevBuf {
    T* p = nullptr;
    size_t n = 0;
    DevBuf() = default;
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    DevBuf(DevBuf&& o) noexcept : p(o.p), n(o.n) { o.p = nullptr; o.n = 0; }
    DevBuf& operator=(DevBuf&& o) noexcept {
        if (this != &o) { release(); p = o.p; n = o.n; o.p = nullptr; o.n = 0; }
        return *this;
    }
    ~DevBuf() { release(); }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        n = 0;
    }
    int alloc(size_t count) {
        release();
        if (count == 0) return 0;
        cudaError_t e = cudaMalloc(&p, count * sizeof(T));
        if (e != cudaSuccess) return fail("cudaMalloc(%zu bytes) failed: %s", count * sizeof(T), cudaGetErrorString(e));
        n = count;
        return 0;
    }
    int ensure(size_t count) { return count <= n ? 0 : alloc(count); }
};

int grid_for(size_t n, int block = 256) {
    size_t g = (n + block - 1) / block;
    return (int)std::max<size_t>(1, std::min(g, (size_t)g_num_sms * 8));
}

// ---- tensors ---------------------------------------------------------------------------------------------------------
// a matrix is kept in the model's weight type (bf16 or fp32), everything else (gains, mixing vectors, decay offsets) in fp32
struct Tensor {
    std::vector<int64_t> shape;
    bool matrix = false;
    bool set = false;
    DevBuf<uint8_t> data;
    size_t count() const {
        size_t c = 1;
        for (auto s : shape) c *= (size_t)s;
        return c;
    }
};

__global__ void synth_fill_f32_kernel(float* out, size_t n, uint64_t seed, float amp, float offset) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = synth_uniform(seed, i, amp) + offset;
}
// first maximum of every row (temperature 0); its log-probability under softmax(logits) when asked for
__global__ void argmax_rows_kernel(const float* logits, int V, int ld, int* tok, float* logprob) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    __shared__ float bv[32];
    __shared__ int bi[32];
    __shared__ float red[32];
    const float* r = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int idx = 0x7FFFFFFF;
    const int bd = blockDim.x;
    for (int i = threadIdx.x; i < V; i += 4 * bd) {   // four independent loads a pass, compared in ascending index order
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = i + q * bd < V ? r[i + q * bd] : -INFINITY;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (v[q] > best) { best = v[q]; idx = i + q * bd; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    best = bv[0];
    idx = bi[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
        if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += 4 * bd) {
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = i + q * bd < V ? r[i + q * bd] : -INFINITY;
        s += (expf(v[0] - best) + expf(v[1] - best)) + (expf(v[2] - best) + expf(v[3] - best));
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) {
        tok[blockIdx.x] = idx == 0x7FFFFFFF ? 0 : idx;
        if (logprob) logprob[blockIdx.x] = -logf(s);
    }
}

struct LayerW {
    ti_seq_layer_desc d{};
    // attention: fused [q | k | v | gate] rows, output projection, frequencies
    const void *qkvg = nullptr, *o = nullptr;
    int n_qkvg = 0;
    DevBuf<uint8_t> qkvg_buf;
    DevBuf<float> inv_freq;
    // wkv
    const void *r = nullptr, *k = nullptr, *v = nullptr, *g = nullptr, *w1 = nullptr, *w2 = nullptr;
    DevBuf<float> mu;   // [5][D]: r, k, v, g, w
    const float *w0 = nullptr, *u = nullptr, *normw = nullptr;
    // feed-forward: fused [gate | up] rows, down
    const void *gateup = nullptr, *down = nullptr;
    DevBuf<uint8_t> gateup_buf;
    const float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr;
    // gla / hgrn2 / latent attention: ONE fused input projection [q | k or f | v | gate | decay-in | down-kv | residual gate] (the parts
    // the mixer has), its width and the column where each part starts (-1: the mixer has no such part)
    const void* front = nullptr;
    DevBuf<uint8_t> front_buf;
    int n_front = 0, off_q = -1, off_k = -1, off_v = -1, off_g = -1, off_a1 = -1, off_dkv = -1, off_rg1 = -1;
    const void *a2 = nullptr, *uv = nullptr;
    DevBuf<uint8_t> ukT;                       // latent attention: per head the transpose of the key up-projection [heads][rank][dim]
    const float *a2b = nullptr, *fb = nullptr, *lower = nullptr, *cnorm = nullptr, *sink = nullptr;
    // feed-forward forms with a fused front [router | shared scale | residual gate | up or experts' gate, up | shared gate, up]
    const void* ffront = nullptr;
    DevBuf<uint8_t> ffront_buf, down_buf;      // down_buf: experts' (and the shared expert's) down matrices side by side along K
    int n_ffront = 0, off_router = -1, off_sg = -1, off_rg2 = -1, off_up = -1, off_sh = -1, ff_width = 0;
    const float *poly = nullptr, *correction = nullptr;
    const void *rg1 = nullptr, *rg2 = nullptr; // residual gates that are not part of a fused front (products of their own)
    const float *rg1b = nullptr, *rg2b = nullptr;
    // per-token side input
    const void *side_gate = nullptr, *side_proj = nullptr;
    const float* side_norm = nullptr;
    // attention with a whole-projection q / k norm, mixed heads; the short convolution in front of the mixer; a dense feed-forward's
    // activation numbers (xielu: softplus(act[0]), 1/2 + softplus(act[1])); the router's bias
    const float *qnorm = nullptr, *knorm = nullptr, *talk = nullptr, *canon = nullptr, *route_bias = nullptr;
    float act_a = 0.f, act_b = 0.f;
    // attention with biased projections / a per-head score factor / a fixed sink; latent attention with low-rank queries; a second
    // convolution in front of the feed-forward; hyper-connections (index 0: mixer, 1: feed-forward)
    DevBuf<float> qkv_bias, sink_zero;         // biases of the fused [q | k | v] product side by side; zeros [heads]
    const float *o_bias = nullptr, *temp = nullptr, *canon2 = nullptr, *dqnorm = nullptr;
    const void* uq = nullptr;
    int off_dq = -1, ld_front = 0;             // ld_front: row stride of the fused front product's output (>= n_front: room for q behind it)
    const float *hc_in[2] = {nullptr, nullptr}, *hc_out[2] = {nullptr, nullptr}, *hc_mix[2] = {nullptr, nullptr};
    int mix_HP = 0;   // > 0: the layer's attention is the head-mixing one; register bound of its head count (8 / 16 / 32 / 64)
};

// one execution of a layer: a looped layer runs several times, every run with its own cache or state
struct Run {
    int layer = 0;
    bool enters_pass = false;   // the looped block's input projection comes right before this run
    DevBuf<float> k_pool, v_pool;          // attention: [pages * 64][G * d], [pages * 64][G * dv]; latent attention: k_pool [pages * 64][rank + rot]
    DevBuf<float> state, prev;             // wkv: [slots][H][d][d], [slots][D]; gla / hgrn2: state [slots][H][dk][dv]
    int kv_run = -1;                       // latent attention reading another layer's cache: the run that owns it
    DevBuf<float> conv_state;              // short convolution: [slots][taps - 1][D], the last inputs of every sequence
    DevBuf<float> conv_state2;             // the same for the convolution in front of the feed-forward
};

struct SeqState {
    bool live = false;
    int len = 0;
    std::vector<int> pages;
};

struct Model {
    ti_seq_model_desc d{};
    std::vector<LayerW> layers;
    std::vector<Run> runs;
    std::map<std::string, Tensor> tensors;
    std::vector<std::string> order;   // required tensors in a fixed order
    bool finalized = false;
    size_t wsize = 2;                 // bytes per matrix element
    const void *embed = nullptr, *loop_in = nullptr, *head = nullptr, *side_embed = nullptr;
    const float* final_norm = nullptr;
    DevBuf<float> pos_freq;           // sinusoidal positions: [ceil(width / 2)] frequencies
    int n_streams = 0;                // copies of the residual the step keeps (norms in front only: >= 1)
    DevBuf<float> xs, ones;           // [rows][streams][D]; ones: in / mix / out of the one-stream residual x <- x + y
    int gvec = 0;                     // 1: the norms around the sublayers have one gain per coordinate
    // cache manager
    int num_pages = 0;
    std::vector<int> free_pages;
    std::vector<SeqState> seqs;
    // step scratch
    int cap_rows = 0, cap_want = 0;
    DevBuf<float> x, x0, xc, h, hc, proj, mixes, att, mo, act, lora, hn, logits, logprobs;   // hc: the mixer input behind a short convolution
    bool any_conv = false;
    DevBuf<float> aux, aux2, route, rgbuf;   // decays / absorbed queries, weighted latent sums, routing weights, unfused residual gates
    int max_aux = 0, max_aux2 = 0, max_route = 0;
    bool any_rgbuf = false;
    DevBuf<int> meta, picks;
    DevBuf<__nv_bfloat16> abf;   // bf16 copy of a product's activations for the tcgen05 path: [rows][max_k]
    DevBuf<float> attn_part;     // split-key attention partials: [rows][heads][splits][vdim + 2]
    DevBuf<float> mix_S, mix_den; // head-mixing attention: scores / weights [rows of a batch][heads][keys], 1 / denominators [rows][heads]
    bool any_mixed = false;
    int max_heads_v = 0;         // max over attention layers of heads * (vdim + 2)
    DevBuf<int> err;             // device flag: a bounded wait in a kernel ran out
    int max_k = 0;
    int* meta_host = nullptr;
    size_t meta_host_cap = 0;
    int max_proj = 0, max_att = 0, max_ff = 0, max_rank = 0;
    bool any_wkv = false;
    // debug
    bool dbg = false;
    DevBuf<float> dbg_buf;
    int dbg_rows = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.f;
    ~Model() {
        if (meta_host) cudaFreeHost(meta_host);
        if (ev0) cudaEventDestroy(ev0);
        if (ev1) cudaEventDestroy(ev1);
    }
};

std::mutex g_mu;
std::vector<std::unique_ptr<Model>> g_models;
Model* get_model(ti_seq_model_t h) {
    if (h == 0 || h > g_models.size()) return nullptr;
    return g_models[h - 1].get();
}

void require(Model& m, const std::string& name, std::vector<int64_t> shape, bool matrix) {
    Tensor t;
    t.shape = std::move(shape);
    t.matrix = matrix;
    m.tensors[name] = std::move(t);
    m.order.push_back(name);
}

bool is_recurrent(int mixer) { return mixer == TI_SEQ_MIXER_WKV || mixer == TI_SEQ_MIXER_GLA || mixer == TI_SEQ_MIXER_HGRN2; }

int describe_tensors(Model& m) {
    const int64_t D = m.d.width, V = m.d.vocab;
    if (m.d.norm_kind != TI_SEQ_NORM_SCALAR && m.d.norm_kind != TI_SEQ_NORM_ONE_PLUS && m.d.norm_kind != TI_SEQ_NORM_VECTOR) return fail("norm kind %d", m.d.norm_kind);
    const std::vector<int64_t> gain_shape = m.d.norm_kind != TI_SEQ_NORM_SCALAR ? std::vector<int64_t>{D} : std::vector<int64_t>{};
    const bool front = m.d.norm_place == TI_SEQ_NORMS_FRONT;
    if (m.d.streams < 0 || m.d.streams > kMaxStreams) return fail("%d residual streams (at most %d)", m.d.streams, kMaxStreams);
    if (m.d.streams > 0 && !front) return fail("hyper-connections are built for norms in front of the sublayers only");
    require(m, "embed", {V, D}, true);
    if (m.d.side_dim > 0) require(m, "side.embed", {V, (int64_t)m.d.side_dim * m.d.n_layers}, true);
    if (m.d.loop_times > 0 && !m.d.loop_plain) require(m, "loop.in", {D, 2 * D}, true);
    for (int i = 0; i < m.d.n_layers; ++i) {
        const ti_seq_layer_desc& L = m.layers[i].d;
        const std::string p = "l" + std::to_string(i) + ".";
        const bool behind = m.d.norm_place == TI_SEQ_NORMS_BEHIND;
        require(m, p + "norm1", gain_shape, false);
        if (!behind && !front) require(m, p + "norm1b", gain_shape, false);
        if (front && (L.res_gate || L.layer_scale || (L.mixer != TI_SEQ_MIXER_ATTENTION && L.mixer != TI_SEQ_MIXER_LATENT) || (L.ff > 0 && L.ff_kind != TI_SEQ_FF_GLU)))
            return fail("layer %d: norms in front of the sublayers only are built for attention / latent attention layers with a gated feed-forward, without residual gates and layer scale", i);
        for (int q = 1; q <= (m.d.streams > 0 ? (L.ff > 0 ? 2 : 1) : 0); ++q) {
            const std::string hc = p + "hc" + std::to_string(q) + ".";
            require(m, hc + "in", {(int64_t)m.d.streams}, false);
            require(m, hc + "out", {(int64_t)m.d.streams}, false);
            require(m, hc + "mix", {(int64_t)m.d.streams, (int64_t)m.d.streams}, false);
        }
        if (L.layer_scale) {
            require(m, p + "ls1", {D}, false);
            if (L.ff > 0) require(m, p + "ls2", {D}, false);
        }
        if (L.conv_taps >= 1 && L.mixer != TI_SEQ_MIXER_ATTENTION && L.mixer != TI_SEQ_MIXER_LATENT) return fail("layer %d: the short convolution is built in front of attention and latent attention mixers", i);
        if (L.conv_taps >= 1) require(m, p + "canon1", {D, (int64_t)L.conv_taps}, false);
        else if (L.conv_taps < 0) return fail("layer %d: %d convolution taps", i, L.conv_taps);
        if (L.conv_ff && L.conv_taps < 1) return fail("layer %d: a convolution in front of the feed-forward without taps", i);
        if (L.conv_ff && L.ff > 0) require(m, p + "canon2", {D, (int64_t)L.conv_taps}, false);
        if (L.sink != TI_SEQ_SINK_NONE && L.sink != TI_SEQ_SINK_LEARNED && L.sink != TI_SEQ_SINK_ZERO) return fail("layer %d: sink kind %d", i, L.sink);
        if (L.rot_linear < 0.f) return fail("layer %d: frequency divisor %g", i, L.rot_linear);
        if (behind && (L.res_gate || L.mixer != TI_SEQ_MIXER_ATTENTION)) return fail("layer %d: norms behind the sublayers only are built for attention layers without residual gates", i);
        if (L.mixer == TI_SEQ_MIXER_ATTENTION) {
            if (L.heads <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads) return fail("layer %d: heads %d / kv_heads %d", i, L.heads, L.kv_heads);
            if (L.dim <= 0 || L.vdim <= 0 || L.dim > 32 * kAttnMaxPerLane || L.vdim > 32 * kAttnMaxPerLane)
                return fail("layer %d: head sizes %d / %d outside 1..%d", i, L.dim, L.vdim, 32 * kAttnMaxPerLane);
            if (L.rot_dims < 0 || L.rot_dims > L.dim || (L.rot_dims & 1)) return fail("layer %d: rot dims %d of %d", i, L.rot_dims, L.dim);
            require(m, p + "mix.q", {(int64_t)L.heads * L.dim, D}, true);
            require(m, p + "mix.k", {(int64_t)L.kv_heads * L.dim, D}, true);
            require(m, p + "mix.v", {(int64_t)L.kv_heads * L.vdim, D}, true);
            if (L.out_gate) require(m, p + "mix.g", {(int64_t)L.heads, D}, true);
            require(m, p + "mix.o", {D, (int64_t)L.heads * L.vdim}, true);
            if (L.qk_norm == TI_SEQ_QK_NORM_WHOLE) {
                if (L.rot_dims > 0 || L.out_gate) return fail("layer %d: the whole-projection q / k norm is built without rotation and output gate", i);
                require(m, p + "mix.q.norm", {(int64_t)L.heads * L.dim}, false);
                require(m, p + "mix.k.norm", {(int64_t)L.kv_heads * L.dim}, false);
            } else if (L.qk_norm != TI_SEQ_QK_NORM_NONE && L.qk_norm != TI_SEQ_QK_NORM_HEAD) return fail("layer %d: q / k norm kind %d", i, L.qk_norm);
            if (L.talk) require(m, p + "mix.talk", {(int64_t)L.heads, (int64_t)L.heads}, false);
            if (L.sink == TI_SEQ_SINK_LEARNED) require(m, p + "mix.sink", {(int64_t)L.heads}, false);
            if (L.proj_bias) {
                require(m, p + "mix.q.b", {(int64_t)L.heads * L.dim}, false);
                require(m, p + "mix.k.b", {(int64_t)L.kv_heads * L.dim}, false);
                require(m, p + "mix.v.b", {(int64_t)L.kv_heads * L.vdim}, false);
                require(m, p + "mix.o.b", {D}, false);
                if (!front) return fail("layer %d: the output projection's bias is built with norms in front of the sublayers only", i);
            }
            if (L.head_temp) require(m, p + "mix.temp", {(int64_t)L.heads}, false);
            if ((L.proj_bias || L.head_temp || L.v_norm || L.rot_half) && L.qk_norm == TI_SEQ_QK_NORM_WHOLE)
                return fail("layer %d: biases, per-head score factors, value norms and half-split rotation are built without the whole-projection q / k norm", i);
            if (L.keep_first < 0 || L.softcap < 0.f) return fail("layer %d: keep_first %d softcap %g", i, L.keep_first, L.softcap);
            if (L.talk || L.softcap > 0.f || L.keep_first > 0) {   // the head-mixing kernel takes the layer
                if (L.out_gate || L.qk_norm == TI_SEQ_QK_NORM_HEAD || L.rot_dims > 0) return fail("layer %d: capped / mixed scores and kept first keys are built without rotation, per-head norm and output gate", i);
                if (L.heads > 64) return fail("layer %d: %d heads exceed the 64 the head-mixing attention holds in registers", i, L.heads);
            }
        } else if (L.mixer == TI_SEQ_MIXER_WKV) {
            if (L.heads <= 0 || L.dim <= 0 || L.dim > 1024 || L.decay_rank <= 0) return fail("layer %d: wkv heads %d dim %d rank %d", i, L.heads, L.dim, L.decay_rank);
            const int64_t C = (int64_t)L.heads * L.dim;
            for (const char* s : {"r", "k", "v", "g", "w"}) require(m, p + "mix.mu." + s, {D}, false);
            for (const char* s : {"r", "k", "v", "g"}) require(m, p + "mix." + s, {C, D}, true);
            require(m, p + "mix.w1", {(int64_t)L.decay_rank, D}, true);
            require(m, p + "mix.w2", {C, (int64_t)L.decay_rank}, true);
            require(m, p + "mix.w0", {C}, false);
            require(m, p + "mix.u", {(int64_t)L.heads, (int64_t)L.dim}, false);
            require(m, p + "mix.norm", {C}, false);
            require(m, p + "mix.o", {D, C}, true);
        } else if (L.mixer == TI_SEQ_MIXER_GLA || L.mixer == TI_SEQ_MIXER_HGRN2) {
            if (L.heads <= 0 || L.dim <= 0 || L.vdim <= 0 || L.dim > 4096 || L.vdim > 65535 * 128)
                return fail("layer %d: recurrence heads %d dim %d vdim %d", i, L.heads, L.dim, L.vdim);
            const int64_t C = (int64_t)L.heads * L.dim, Cv = (int64_t)L.heads * L.vdim;
            require(m, p + "mix.q", {C, D}, true);
            if (L.mixer == TI_SEQ_MIXER_GLA) {
                if (L.decay_rank <= 0 || !(L.decay_tau > 0.f)) return fail("layer %d: gla decay rank %d tau %g", i, L.decay_rank, L.decay_tau);
                require(m, p + "mix.k", {C, D}, true);
                require(m, p + "mix.v", {Cv, D}, true);
                require(m, p + "mix.g", {Cv, D}, true);
                require(m, p + "mix.a1", {(int64_t)L.decay_rank, D}, true);
                require(m, p + "mix.a2", {C, (int64_t)L.decay_rank}, true);
                require(m, p + "mix.a2.b", {C}, false);
            } else {
                require(m, p + "mix.f", {C, D}, true);
                require(m, p + "mix.f.b", {C}, false);
                require(m, p + "mix.lower", {C}, false);
                require(m, p + "mix.v", {Cv, D}, true);
            }
            require(m, p + "mix.norm", {(int64_t)L.vdim}, false);
            require(m, p + "mix.o", {D, Cv}, true);
        } else if (L.mixer == TI_SEQ_MIXER_LATENT) {
            if (L.heads <= 0 || L.dim <= 0 || L.vdim <= 0 || L.kv_rank <= 0 || L.rot_dims < 0 || (L.rot_dims & 1))
                return fail("layer %d: latent attention heads %d dim %d rot %d vdim %d rank %d", i, L.heads, L.dim, L.rot_dims, L.vdim, L.kv_rank);
            if (L.kv_rank + L.rot_dims > 32 * kAttnWidePerLane) return fail("layer %d: cached row of %d + %d exceeds %d", i, L.kv_rank, L.rot_dims, 32 * kAttnWidePerLane);
            if (L.kv_from >= 0) {
                if (L.kv_from >= i) return fail("layer %d: reads the cache of layer %d, which does not run before it", i, L.kv_from);
                const ti_seq_layer_desc& S = m.layers[L.kv_from].d;
                if (S.mixer != TI_SEQ_MIXER_LATENT || S.kv_from >= 0 || S.kv_rank != L.kv_rank || S.rot_dims != L.rot_dims || S.rot_base != L.rot_base)
                    return fail("layer %d: layer %d has no cache of its own with the same rank, rotated size and rotation", i, L.kv_from);
            }
            if (L.q_rank > 0) {
                require(m, p + "mix.dq", {(int64_t)L.q_rank, D}, true);
                require(m, p + "mix.dq.norm", {(int64_t)L.q_rank}, false);
                require(m, p + "mix.uq", {(int64_t)L.heads * (L.dim + L.rot_dims), (int64_t)L.q_rank}, true);
            } else if (L.q_rank == 0) {
                require(m, p + "mix.q", {(int64_t)L.heads * (L.dim + L.rot_dims), D}, true);
            } else return fail("layer %d: query rank %d", i, L.q_rank);
            if (L.window < 0) return fail("layer %d: window %d", i, L.window);
            if (L.out_gate) require(m, p + "mix.g", {(int64_t)L.heads, D}, true);
            if (L.kv_from < 0) {
                require(m, p + "mix.dkv", {(int64_t)L.kv_rank + L.rot_dims, D}, true);
                require(m, p + "mix.dkv.norm", {(int64_t)L.kv_rank}, false);
            }
            require(m, p + "mix.uk", {(int64_t)L.heads * L.dim, (int64_t)L.kv_rank}, true);
            require(m, p + "mix.uv", {(int64_t)L.heads * L.vdim, (int64_t)L.kv_rank}, true);
            if (L.sink == TI_SEQ_SINK_LEARNED) require(m, p + "mix.sink", {(int64_t)L.heads}, false);
            require(m, p + "mix.o", {D, (int64_t)L.heads * L.vdim}, true);
        } else {
            return fail("layer %d: unknown mixer %d", i, L.mixer);
        }
        if (L.res_gate) {
            require(m, p + "rg1", {D, D}, true);
            require(m, p + "rg1.b", {D}, false);
        }
        if (L.ff > 0) {
            require(m, p + "norm2", gain_shape, false);
            if (!behind && !front) require(m, p + "norm2b", gain_shape, false);
            if (behind && L.ff_kind != TI_SEQ_FF_DENSE && L.ff_kind != TI_SEQ_FF_EXPERTS) return fail("layer %d: norms behind the sublayers only are built for the dense and the routed feed-forward", i);
            if (L.ff_kind == TI_SEQ_FF_DENSE) {
                if (L.ff_act != TI_SEQ_ACT_XIELU && L.ff_act != TI_SEQ_ACT_RELU && L.ff_act != TI_SEQ_ACT_SILU && L.ff_act != TI_SEQ_ACT_GELU_TANH)
                    return fail("layer %d: activation %d", i, L.ff_act);
                require(m, p + "mlp.up", {(int64_t)L.ff, D}, true);
                require(m, p + "mlp.down", {D, (int64_t)L.ff}, true);
                if (L.ff_act == TI_SEQ_ACT_XIELU) require(m, p + "mlp.act", {2}, false);
            } else if (L.ff_kind == TI_SEQ_FF_GLU) {
                require(m, p + "mlp.gate", {(int64_t)L.ff, D}, true);
                require(m, p + "mlp.up", {(int64_t)L.ff, D}, true);
                require(m, p + "mlp.down", {D, (int64_t)L.ff}, true);
            } else if (L.ff_kind == TI_SEQ_FF_POLYNORM) {
                require(m, p + "mlp.up", {(int64_t)L.ff, D}, true);
                require(m, p + "mlp.down", {D, (int64_t)L.ff}, true);
                require(m, p + "mlp.act", {4}, false);
            } else if (L.ff_kind == TI_SEQ_FF_EXPERTS) {
                const int n = L.experts + L.identity;
                if (L.experts < 0 || L.identity < 0 || n <= 0 || L.top <= 0 || L.top > n || L.groups <= 0 || n % L.groups || L.groups_keep <= 0 || L.groups_keep > L.groups)
                    return fail("layer %d: %d experts + %d identity, top %d, %d groups keep %d", i, L.experts, L.identity, L.top, L.groups, L.groups_keep);
                for (int e = 0; e < L.experts; ++e) {
                    const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                    require(m, q + "gate", {(int64_t)L.ff, D}, true);
                    require(m, q + "up", {(int64_t)L.ff, D}, true);
                    require(m, q + "down", {D, (int64_t)L.ff}, true);
                }
                require(m, p + "mlp.router", {(int64_t)n, D}, true);
                if (L.route_kind == TI_SEQ_ROUTE_TOP_LOGITS) {
                    if (L.groups != 1 || L.groups_keep != 1) return fail("layer %d: the choice by logits has no groups", i);
                    require(m, p + "mlp.router.b", {(int64_t)n}, false);
                } else if (L.route_kind == TI_SEQ_ROUTE_SOFTMAX_ALL) {
                    require(m, p + "mlp.correction", {(int64_t)n}, false);
                } else return fail("layer %d: router kind %d", i, L.route_kind);
                if (L.shared_ff > 0) {
                    require(m, p + "mlp.shared.gate", {(int64_t)L.shared_ff, D}, true);
                    require(m, p + "mlp.shared.up", {(int64_t)L.shared_ff, D}, true);
                    require(m, p + "mlp.shared.down", {D, (int64_t)L.shared_ff}, true);
                    if (!L.shared_plain) require(m, p + "mlp.shared.sg", {1, D}, true);
                }
            } else {
                return fail("layer %d: unknown feed-forward kind %d", i, L.ff_kind);
            }
            if (L.res_gate) {
                require(m, p + "rg2", {D, D}, true);
                require(m, p + "rg2.b", {D}, false);
            }
        }
        if (m.d.side_dim > 0) {
            require(m, p + "side.gate", {(int64_t)m.d.side_dim, D}, true);
            require(m, p + "side.proj", {D, (int64_t)m.d.side_dim}, true);
            require(m, p + "side.norm", {D}, false);
        }
    }
    require(m, "final.norm", gain_shape, false);
    if (!m.d.tied_head) require(m, "head", {V, D}, true);
    if (m.d.norm_place != TI_SEQ_NORMS_AROUND && m.d.norm_place != TI_SEQ_NORMS_BEHIND && !front) return fail("norm placement %d", m.d.norm_place);
    if (front && (m.d.side_dim > 0 || (m.d.loop_times > 0 && !m.d.loop_plain))) return fail("norms in front of the sublayers only are built without side input and without a projection between the passes of a looped block");
    if (m.d.norm_place == TI_SEQ_NORMS_BEHIND && (m.d.loop_times > 0 || m.d.side_dim > 0)) return fail("norms behind the sublayers only are built without a looped block and side input");
    return 0;
}

// store `n` source elements (fp32 on the device) into the tensor's own format
int store_from_f32(Model& m, Tensor& t, const float* src_dev, size_t n) {
    if (t.matrix && m.d.mode == TI_SEQ_BF16) {
        TRY(t.data.alloc(n * 2));
        f32_to_bf16_kernel<<<grid_for(n), 256, 0, g_stream>>>(src_dev, reinterpret_cast<__nv_bfloat16*>(t.data.p), n);
        LAUNCHED();
    } else {
        TRY(t.data.alloc(n * 4));
        CK(cudaMemcpyAsync(t.data.p, src_dev, n * 4, cudaMemcpyDeviceToDevice, g_stream));
    }
    CK(cudaStreamSynchronize(g_stream));
    t.set = true;
    return 0;
}

std::vector<float> rotary_frequencies(const ti_seq_layer_desc& L) {
    std::vector<float> f((size_t)L.rot_dims / 2);
    const double two_pi = 6.283185307179586476925286766559;
    for (size_t i = 0; i < f.size(); ++i) {
        double fi = std::pow((double)L.rot_base, -2.0 * (double)i / (double)L.rot_dims);
        if (L.rot_scaled) {
            const double wl = two_pi / fi, orig = L.rot_original;
            if (wl > orig / L.rot_low) fi = fi / L.rot_factor;
            else if (!(wl < orig / L.rot_high)) {
                const double s = (orig / wl - L.rot_low) / ((double)L.rot_high - L.rot_low);
                fi = (1.0 - s) * fi / L.rot_factor + s * fi;
            }
        }
        if (L.rot_linear > 0.f) fi /= (double)L.rot_linear;
        f[i] = (float)fi;
    }
    return f;
}

int concat_rows(Model& m, const std::vector<const Tensor*>& parts, DevBuf<uint8_t>& out, int* rows, std::vector<int>* offsets = nullptr) {
    size_t bytes = 0;
    int n = 0;
    for (const Tensor* t : parts) {
        if (offsets) offsets->push_back(t ? n : -1);
        if (!t) continue;
        bytes += t->data.n;
        n += (int)t->shape[0];
    }
    TRY(out.alloc(bytes));
    size_t off = 0;
    for (const Tensor* t : parts) {
        if (!t) continue;
        CK(cudaMemcpyAsync(out.p + off, t->data.p, t->data.n, cudaMemcpyDeviceToDevice, g_stream));
        off += t->data.n;
    }
    CK(cudaStreamSynchronize(g_stream));
    *rows = n;
    (void)m;
    return 0;
}

// matrices [rows][cols_i] side by side along the columns: out [rows][sum cols_i]
int concat_cols(Model& m, const std::vector<const Tensor*>& parts, DevBuf<uint8_t>& out, int* cols) {
    int64_t rows = -1, total = 0;
    for (const Tensor* t : parts) {
        if (!t) continue;
        if (rows >= 0 && t->shape[0] != rows) return fail("internal: column concatenation of matrices with different row counts");
        rows = t->shape[0];
        total += t->shape[1];
    }
    TRY(out.alloc((size_t)rows * total * m.wsize));
    size_t off = 0;
    for (const Tensor* t : parts) {
        if (!t) continue;
        const size_t w = (size_t)t->shape[1] * m.wsize;
        CK(cudaMemcpy2DAsync(out.p + off, (size_t)total * m.wsize, t->data.p, w, w, (size_t)rows, cudaMemcpyDeviceToDevice, g_stream));
        off += w;
    }
    CK(cudaStreamSynchronize(g_stream));
    *cols = (int)total;
    return 0;
}
__global__ void mul_vec_kernel(float* w, const float* v, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) w[i] *= v[i];
}
__global__ void add_one_kernel(float* w, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) w[i] += 1.f;
}

// ---- tensor maps for the tcgen05 path: a bf16 matrix [rows][cols], cols contiguous, boxes of 64 x 128 with the 128-byte swizzle ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr));
        if (!p || qr != cudaDriverEntryPointSuccess) return fail("cuTensorMapEncodeTiled is not available in this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kSgBK, (cuuint32_t)kSgBM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed (%d)", (int)r);
    return 0;
}

// ---- matrix product dispatch ----------------------------------------------------------------------------------------------
// Fusion a caller may ask for; it happens inside the product when the step is a decode step (few rows) and the caller does the
// separate kernel otherwise (gemm() says which through the return of fused()).
// Launch of a kernel of the step with programmatic stream serialization: it may be scheduled while the kernel before it is still
// running and parks in griddepcontrol.wait (the first statement of every kernel launched through here) until that one has
// completed, so the launch latency of the many small kernels of a decode step overlaps the kernel in front.
template <typename... KArgs, typename... Args>
int launch_dep(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = g_stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    CK(cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...));
    return 0;   // (the caller counts the launch)
}

struct Fuse {
    const float* norm_gain = nullptr;   // RMS norm of the input rows in front of the product (gvec: one gain per coordinate)
    int gvec = 0;
    float eps = 0.f;
    int glu_ff = 0, glu_act = 0;        // act(gate) * up behind a fused [gate | up] product: N is then the inner size
    ExpertSkip nskip{}, kskip{};        // few rows over stacked expert matrices: column tiles / k chunks of experts no row chose are not read
};
bool few_rows(int M, int K) { return M <= kRowGemvMaxRows && (size_t)M * K * sizeof(float) <= g_smem_optin; }

int gemm(Model& m, const float* A, int lda, const void* W, float* C, int ldc, int M, int N, int K, int epi = EPI_NONE, float alpha = 1.f,
         const Fuse* fuse = nullptr, float beta = 0.f) {
    if (M <= 0 || N <= 0) return 0;
    const size_t xs_bytes = (size_t)M * K * sizeof(float);
    // few rows of a very long K that do not fit shared memory together (the side-by-side down matrices of many experts): in halves,
    // rather than on the tile kernels, which would run a handful of blocks over the whole K
    const size_t mma_bytes = gemv_mma_smem_bytes(M, K);
    // bf16 weights with K in whole 32-element chunks: the tensor-core form (a weight byte costs the same for 1 and for 8 rows; rows staged as bf16)
    const bool mma_ok = M <= kRowGemvMaxRows && m.d.mode == TI_SEQ_BF16 && g_use_row_mma && K % 32 == 0 && K >= 256 && (reinterpret_cast<uintptr_t>(W) & 15) == 0 &&
                        mma_bytes <= g_smem_optin;
    const bool plain = !fuse || (!fuse->norm_gain && !fuse->glu_ff);   // (a request to skip unused experts' rows is only a permission)
    if (plain && M > 1 && M <= kRowGemvMaxRows && !mma_ok && !few_rows(M, K) && few_rows(1, K)) {
        const int half = M / 2;
        TRY(gemm(m, A, lda, W, C, ldc, half, N, K, epi, alpha, fuse, beta));
        return gemm(m, A + (size_t)half * lda, lda, W, C + (size_t)half * ldc, ldc, M - half, N, K, epi, alpha, fuse, beta);
    }
    if (mma_ok || few_rows(M, K)) {
        const int warps = kRowGemvThreads / 32;
        // enough resident blocks to keep the memory system busy, few enough that staging the rows in every block stays small
        // beside the weight bytes: 2 blocks an SM (their registers allow no more) as far as their shared memory allows, columns looped inside
        const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(2, (200u << 10) / std::max<size_t>(xs_bytes, 1)));
        const int grid = std::max(1, std::min((N + warps - 1) / warps, g_num_sms * per_sm));
        const Fuse f = fuse ? *fuse : Fuse{};
        if (mma_ok) {
            const int fit = (int)std::max<size_t>(1, std::min<size_t>(2, (200u << 10) / mma_bytes));
            const int blocks = std::max(1, std::min((N + kMmaCols - 1) / kMmaCols, g_num_sms * fit));
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(blocks);
            cfg.blockDim = dim3(256);
            cfg.dynamicSmemBytes = mma_bytes;
            cfg.stream = g_stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = g_use_pdl ? 1 : 0;
            if (f.glu_ff > 0)
                CK(cudaLaunchKernelEx(&cfg, gemv_rows_mma_kernel<true>, A, lda, (const __nv_bfloat16*)W, C, ldc, M, N, K, epi, alpha, beta, f.norm_gain, f.eps, f.glu_ff,
                                      f.glu_act, f.gvec, f.nskip, f.kskip));
            else
                CK(cudaLaunchKernelEx(&cfg, gemv_rows_mma_kernel<false>, A, lda, (const __nv_bfloat16*)W, C, ldc, M, N, K, epi, alpha, beta, f.norm_gain, f.eps, f.glu_ff,
                                      f.glu_act, f.gvec, f.nskip, f.kskip));
            LAUNCHED();
            return 0;
        }
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kRowGemvThreads);
        cfg.dynamicSmemBytes = xs_bytes;
        cfg.stream = g_stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_use_pdl ? 1 : 0;
        if (m.d.mode == TI_SEQ_BF16)
            CK(cudaLaunchKernelEx(&cfg, gemv_rows_kernel<__nv_bfloat16>, A, lda, (const __nv_bfloat16*)W, C, ldc, M, N, K, epi, alpha, beta, f.norm_gain, f.eps,
                                  f.glu_ff, f.glu_act, f.gvec));
        else
            CK(cudaLaunchKernelEx(&cfg, gemv_rows_kernel<float>, A, lda, (const float*)W, C, ldc, M, N, K, epi, alpha, beta, f.norm_gain, f.eps, f.glu_ff,
                                  f.glu_act, f.gvec));
        LAUNCHED();
        return 0;
    }
    if (!plain) return fail("internal: a fused product was asked for on the many-row path");
    // prompt-sized products in bf16 mode: tcgen05 (TMA wants 16-byte row pitches and bases)
    if (m.d.mode == TI_SEQ_BF16 && g_use_tc && M > 32 && N >= 64 && K >= 64 && K % 8 == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0 && m.abf.p &&
        (size_t)M * K <= m.abf.n) {
        rows_to_bf16_kernel<<<grid_for((size_t)M * K / 4), 256, 0, g_stream>>>(A, lda, M, K, m.abf.p);
        LAUNCHED();
        CUtensorMap ma, mw;
        TRY(make_tmap_bf16(&ma, m.abf.p, (uint64_t)K, (uint64_t)M));
        TRY(make_tmap_bf16(&mw, W, (uint64_t)K, (uint64_t)N));
        TcArgs g{};
        g.M = M; g.N = N; g.K = K; g.C = C; g.ldc = ldc; g.epi = epi; g.alpha = alpha; g.beta = beta; g.err = m.err.p;
        gemm_bf16_tc_kernel<<<dim3((N + kSgBN - 1) / kSgBN, (M + kSgBM - 1) / kSgBM), kSgThreads, kSgSmemBytes, g_stream>>>(ma, mw, g);
        LAUNCHED();
        return 0;
    }
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (m.d.mode == TI_SEQ_BF16) gemm_bf16_kernel<<<grid, 128, 0, g_stream>>>(A, lda, (const __nv_bfloat16*)W, C, ldc, M, N, K, epi, alpha, beta, 0, 0, 0);
    else gemm_f32_kernel<<<grid, 256, 0, g_stream>>>(A, lda, (const float*)W, C, ldc, M, N, K, epi, alpha, beta, 0, 0, 0);
    LAUNCHED();
    return 0;
}

// one small product per head: C[r][h * c_stride + n] = sum_k A[r][h * a_stride + k] W[h][n][k]; few rows in one launch, else a product per head
int gemm_heads(Model& m, const float* A, int lda, int a_stride, const void* W, float* C, int ldc, int c_stride, int heads, int M, int N, int K) {
    if (M <= kRowGemvMaxRows && (size_t)M * K * sizeof(float) <= 48 * 1024) {
        const int warps = kRowGemvThreads / 32;
        const dim3 grid(std::max(1, std::min((N + warps - 1) / warps, std::max(1, 4 * g_num_sms / heads))), heads);
        if (m.d.mode == TI_SEQ_BF16)
            TRY(launch_dep(gemv_heads_rows_kernel<__nv_bfloat16>, grid, dim3(kRowGemvThreads), (size_t)M * K * sizeof(float), A, lda, a_stride, (const __nv_bfloat16*)W, C, ldc, c_stride, M, N, K));
        else
            TRY(launch_dep(gemv_heads_rows_kernel<float>, grid, dim3(kRowGemvThreads), (size_t)M * K * sizeof(float), A, lda, a_stride, (const float*)W, C, ldc, c_stride, M, N, K));
        LAUNCHED();
        return 0;
    }
    // many rows: all heads in one launch of the tile kernels (a head's product is too small to fill the GPU by itself)
    const dim3 grid((N + 63) / 64, (M + 63) / 64, heads);
    if (heads <= 65535 && grid.y <= 65535) {
        if (m.d.mode == TI_SEQ_BF16)
            gemm_bf16_kernel<<<grid, 128, 0, g_stream>>>(A, lda, (const __nv_bfloat16*)W, C, ldc, M, N, K, EPI_NONE, 1.f, 0.f, (size_t)a_stride, (size_t)N * K, (size_t)c_stride);
        else
            gemm_f32_kernel<<<grid, 256, 0, g_stream>>>(A, lda, (const float*)W, C, ldc, M, N, K, EPI_NONE, 1.f, 0.f, (size_t)a_stride, (size_t)N * K, (size_t)c_stride);
        LAUNCHED();
        return 0;
    }
    for (int h = 0; h < heads; ++h)
        TRY(gemm(m, A + (size_t)h * a_stride, lda, (const uint8_t*)W + (size_t)h * N * K * m.wsize, C + (size_t)h * c_stride, ldc, M, N, K));
    return 0;
}

int ensure_scratch(Model& m, int rows, int want) {
    if (rows > m.cap_rows) {
        const size_t R = (size_t)std::max(rows, 64), D = m.d.width;
        TRY(m.x.alloc(R * D));
        if (m.n_streams > 0) TRY(m.xs.alloc(R * (size_t)m.n_streams * D));
        TRY(m.x0.alloc(R * D));
        if (m.d.loop_times > 0) TRY(m.xc.alloc(R * 2 * D));
        TRY(m.h.alloc(R * D));
        if (m.any_conv) TRY(m.hc.alloc(R * D));
        TRY(m.proj.alloc(R * (size_t)m.max_proj));
        if (m.any_wkv) TRY(m.mixes.alloc(5 * R * D));
        TRY(m.att.alloc(R * (size_t)m.max_att));
        TRY(m.mo.alloc(R * D));
        if (m.max_ff) TRY(m.act.alloc(R * (size_t)m.max_ff));
        if (m.max_rank) TRY(m.lora.alloc(R * (size_t)m.max_rank));
        if (m.max_aux) TRY(m.aux.alloc(R * (size_t)m.max_aux));
        if (m.max_aux2) TRY(m.aux2.alloc(R * (size_t)m.max_aux2));
        if (m.max_route) TRY(m.route.alloc(R * (size_t)m.max_route));
        if (m.any_rgbuf) TRY(m.rgbuf.alloc(R * D));
        if (m.dbg) TRY(m.dbg_buf.alloc(m.runs.size() * R * D));
        if (m.d.mode == TI_SEQ_BF16 && g_use_tc) TRY(m.abf.alloc(R * (size_t)m.max_k));
        if (m.max_heads_v) TRY(m.attn_part.alloc(R * (size_t)m.max_heads_v * kAttnMaxSplits));
        m.cap_rows = (int)R;
    }
    if (want > m.cap_want) {
        const size_t W = (size_t)std::max(want, 8);
        TRY(m.hn.alloc(W * m.d.width));
        TRY(m.logits.alloc(W * m.d.vocab));
        TRY(m.logprobs.alloc(W));
        TRY(m.picks.alloc(W));
        m.cap_want = (int)W;
    }
    return 0;
}

// ---- the step ----------------------------------------------------------------------------------------------------------------
// few rows: the wkv mixer's r / k / v / g / decay-input products with their mixes built in the prologue (one launch)
int wkv_front(Model& m, LayerW& L, Run& R, const StepMeta& sm, int T, float* pr, float* pk, float* pv, float* pg, float* lora) {
    const int D = m.d.width, C = L.d.heads * L.d.dim, rank = L.d.decay_rank;
    WkvFrontArgs a{};
    a.h = m.h.p; a.mu = L.mu.p; a.prev = R.prev.p; a.D = D;
    const void* W[5] = {L.r, L.k, L.v, L.g, L.w1};
    float* out[5] = {pr, pk, pv, pg, lora};
    const int N[5] = {C, C, C, C, rank}, epi[5] = {EPI_NONE, EPI_NONE, EPI_NONE, EPI_SILU, EPI_TANH};
    const int warps = kRowGemvThreads / 32, budget = 2 * g_num_sms;
    const long total = 4L * C + rank;
    a.blk0[0] = 0;
    for (int s = 0; s < 5; ++s) {
        a.W[s] = W[s]; a.out[s] = out[s]; a.N[s] = N[s]; a.epi[s] = epi[s];
        const int want = (N[s] + warps - 1) / warps;
        const int share = (int)std::max<long>(1, (long)budget * N[s] / total);
        a.blk0[s + 1] = a.blk0[s] + std::max(1, std::min(want, share));
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(a.blk0[5]);
    cfg.blockDim = dim3(kRowGemvThreads);
    cfg.dynamicSmemBytes = (size_t)T * D * sizeof(float);
    cfg.stream = g_stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    if (m.d.mode == TI_SEQ_BF16) CK(cudaLaunchKernelEx(&cfg, wkv_front_rows_kernel<__nv_bfloat16>, a, sm));
    else CK(cudaLaunchKernelEx(&cfg, wkv_front_rows_kernel<float>, a, sm));
    LAUNCHED();
    return 0;
}

struct SampleSpec {
    bool on = false;
    float temperature = 0.f, top_p = 1.f;
    int top_k = 0;
    uint64_t seed = 0;
    const int32_t* index = nullptr;
    int32_t* out_tokens = nullptr;
    float* out_logprobs = nullptr;
};

int run_step(Model& m, int E, const int32_t* seqs, const int32_t* counts, const int32_t* tokens, int n_want, const int32_t* want_rows,
             float* logits_host, const SampleSpec& smp) {
    if (!m.finalized) return fail("model not finalized");
    if (E <= 0) return 0;
    const int D = m.d.width, V = m.d.vocab;
    int T = 0;
    for (int e = 0; e < E; ++e) {
        if (seqs[e] < 0 || seqs[e] >= (int)m.seqs.size() || !m.seqs[seqs[e]].live) return fail("step: sequence %d is not open", seqs[e]);
        for (int f = 0; f < e; ++f)
            if (seqs[f] == seqs[e]) return fail("step: sequence %d appears twice", seqs[e]);
        if (counts[e] <= 0) return fail("step: entry %d brings no tokens", e);
        T += counts[e];
    }
    for (int i = 0; i < T; ++i)
        if (tokens[i] < 0 || tokens[i] >= V) return fail("step: token id %d outside the vocabulary", tokens[i]);
    for (int i = 0; i < n_want; ++i)
        if (want_rows[i] < 0 || want_rows[i] >= T) return fail("step: wanted row %d outside the step", want_rows[i]);
    // pages for the new tokens (all or nothing)
    int need = 0;
    for (int e = 0; e < E; ++e) {
        const SeqState& s = m.seqs[seqs[e]];
        need += (s.len + counts[e] + kPageTokens - 1) / kPageTokens - (int)s.pages.size();
    }
    if (need > (int)m.free_pages.size()) return fail("step: page pool exhausted (%d pages needed, %zu free)", need, m.free_pages.size());
    for (int e = 0; e < E; ++e) {
        SeqState& s = m.seqs[seqs[e]];
        const int np = (s.len + counts[e] + kPageTokens - 1) / kPageTokens;
        while ((int)s.pages.size() < np) {
            s.pages.push_back(m.free_pages.back());
            m.free_pages.pop_back();
        }
    }
    const int n_out = smp.on ? E : n_want;
    TRY(ensure_scratch(m, T, std::max(n_out, 1)));
    // meta buffer: tok | row_ent | row_pos | ent_row0 | ent_slot | ent_pos0 | out rows | page table
    const int stride = m.num_pages;
    // attention work lists: prompt portions are cut into tiles of up to 64 rows of one sequence, the other rows go one by one
    std::vector<int> tiles, tiles128, small_rows;
    {
        int r0 = 0;
        for (int e = 0; e < E; ++e) {
            if (counts[e] >= kAttnTiledMinRows) {
                for (int o = 0; o < counts[e]; o += kAttnTile) { tiles.push_back(r0 + o); tiles.push_back(std::min(kAttnTile, counts[e] - o)); }
                for (int o = 0; o < counts[e]; o += kAttnTcTile) { tiles128.push_back(r0 + o); tiles128.push_back(std::min(kAttnTcTile, counts[e] - o)); }
            } else
                for (int o = 0; o < counts[e]; ++o) small_rows.push_back(r0 + o);
            r0 += counts[e];
        }
    }
    const int n_tiles = (int)tiles.size() / 2, n_tiles128 = (int)tiles128.size() / 2, n_small = (int)small_rows.size();
    // the head-mixing attention cuts EVERY entry into tiles of up to 64 rows and wants the tile of every row
    std::vector<int> mtiles, row_tile;
    if (m.any_mixed) {
        row_tile.resize(T);
        int r0 = 0;
        for (int e = 0; e < E; ++e) {
            for (int o = 0; o < counts[e]; o += kAttnTile) {
                const int nrow = std::min(kAttnTile, counts[e] - o);
                for (int r = 0; r < nrow; ++r) row_tile[r0 + o + r] = (int)mtiles.size() / 2;
                mtiles.push_back(r0 + o);
                mtiles.push_back(nrow);
            }
            r0 += counts[e];
        }
    }
    const int n_mtiles = (int)mtiles.size() / 2;
    const size_t n_meta = (size_t)3 * T + (size_t)(E + 1) + 2 * (size_t)E + (size_t)std::max(n_out, 1) + (size_t)m.seqs.size() * stride +
                          (size_t)3 * T + 4 + mtiles.size() + row_tile.size();
    if (n_meta > m.meta_host_cap) {
        if (m.meta_host) cudaFreeHost(m.meta_host);
        m.meta_host = nullptr;
        m.meta_host_cap = 0;
        CK(cudaMallocHost(&m.meta_host, n_meta * 2 * sizeof(int)));
        m.meta_host_cap = n_meta * 2;
    }
    TRY(m.meta.ensure(m.meta_host_cap));
    int* hp = m.meta_host;
    int *h_tok = hp, *h_ent = h_tok + T, *h_pos = h_ent + T, *h_row0 = h_pos + T, *h_slot = h_row0 + E + 1, *h_pos0 = h_slot + E,
        *h_out = h_pos0 + E, *h_table = h_out + std::max(n_out, 1);
    int row = 0;
    for (int e = 0; e < E; ++e) {
        const SeqState& s = m.seqs[seqs[e]];
        h_row0[e] = row;
        h_slot[e] = seqs[e];
        h_pos0[e] = s.len;
        for (int i = 0; i < counts[e]; ++i, ++row) {
            h_tok[row] = tokens[row];
            h_ent[row] = e;
            h_pos[row] = s.len + i;
        }
        if (smp.on) h_out[e] = row - 1;
    }
    h_row0[E] = row;
    int max_pos = 0;
    for (int e = 0; e < E; ++e) max_pos = std::max(max_pos, m.seqs[seqs[e]].len + counts[e] - 1);
    if (!smp.on)
        for (int i = 0; i < n_want; ++i) h_out[i] = want_rows[i];
    for (size_t s = 0; s < m.seqs.size(); ++s)
        for (int p = 0; p < stride; ++p) h_table[s * stride + p] = p < (int)m.seqs[s].pages.size() ? m.seqs[s].pages[p] : 0;
    int* h_tiles = h_table + m.seqs.size() * stride;
    int* h_small = h_tiles + tiles.size();
    std::copy(tiles.begin(), tiles.end(), h_tiles);
    std::copy(small_rows.begin(), small_rows.end(), h_small);
    int* h_tiles128 = h_small + small_rows.size();
    std::copy(tiles128.begin(), tiles128.end(), h_tiles128);
    int* h_mtiles = h_tiles128 + tiles128.size();
    std::copy(mtiles.begin(), mtiles.end(), h_mtiles);
    int* h_row_tile = h_mtiles + mtiles.size();
    std::copy(row_tile.begin(), row_tile.end(), h_row_tile);
    // the previous step's copy out of this pinned buffer has completed: every step ends with a stream synchronisation
    CK(cudaMemcpyAsync(m.meta.p, hp, n_meta * sizeof(int), cudaMemcpyHostToDevice, g_stream));
    StepMeta sm{};
    sm.tok = m.meta.p;
    sm.row_ent = sm.tok + T;
    sm.row_pos = sm.row_ent + T;
    sm.ent_row0 = sm.row_pos + T;
    sm.ent_slot = sm.ent_row0 + E + 1;
    sm.ent_pos0 = sm.ent_slot + E;
    const int* d_out = sm.ent_pos0 + E;
    sm.page_table = d_out + std::max(n_out, 1);
    const int* d_tiles = sm.page_table + m.seqs.size() * stride;
    const int* d_small = d_tiles + tiles.size();
    const int* d_tiles128 = d_small + small_rows.size();
    const int* d_mtiles = d_tiles128 + tiles128.size();
    const int* d_row_tile = d_mtiles + mtiles.size();
    sm.table_stride = stride;
    sm.T = T;
    sm.E = E;

    CK(cudaEventRecord(m.ev0, g_stream));
    const bool bf = m.d.mode == TI_SEQ_BF16;
    const int nt = 256;
    const bool front = m.d.norm_place == TI_SEQ_NORMS_FRONT;   // norms in front of the sublayers only: the residual lives in m.xs (one or more streams)
    float* emb_out = front ? m.xs.p : m.x.p;
    const int emb_copies = front ? m.n_streams : 1;
    if (bf) TRY(launch_dep(embed_rows_kernel<__nv_bfloat16>, dim3(T), dim3(nt), 0, (const __nv_bfloat16*)m.embed, sm, D, emb_out, m.loop_in ? m.x0.p : nullptr, (const float*)m.pos_freq.p, emb_copies));
    else TRY(launch_dep(embed_rows_kernel<float>, dim3(T), dim3(nt), 0, (const float*)m.embed, sm, D, emb_out, m.loop_in ? m.x0.p : nullptr, (const float*)m.pos_freq.p, emb_copies));
    LAUNCHED();
    const float eps = m.d.norm_eps;
    const int gv = m.gvec;
    // the end of a sublayer: (identity experts) -> (gate) -> norm behind the sublayer -> residual sum (-> the next sublayer's input)
    auto post = [&](const float* gain, int gain_vec, const float* gain2, const float* gate, int gate_ld, const float* gate_bias, const float* idw) -> int {
        PostArgs a{};
        a.x = m.x.p; a.mo = m.mo.p; a.gain = gain; a.gain2 = gain2; a.y = m.h.p; a.gate = gate; a.gate_bias = gate_bias; a.idw = idw; a.hin = m.h.p;
        a.gate_ld = gate_ld; a.D = D; a.gvec = gain_vec; a.gvec2 = gv; a.eps = eps;
        TRY(launch_dep(postnorm_residual_kernel, dim3(T), dim3(nt), 0, a));
        LAUNCHED();
        return 0;
    };
    // norms in front only: sublayer `q` (0: mixer, 1: feed-forward) of layer run `ri` ends with its result in m.mo -- every stream is
    // rewritten, and the input of the sublayer that follows (the same run's feed-forward or the next run's mixer) goes to m.h; the last
    // sublayer of a run leaves the sum of the streams in m.x.  q < 0: nothing ends, the first sublayer of the step is opened.
    bool all_single = true;   // a decoding step: every entry brings one row, and a sublayer's convolution reads its slot's state only
    for (int e = 0; e < E; ++e) all_single = all_single && counts[e] == 1;
    auto hyper = [&](size_t ri, int q) -> int {
        const LayerW& L = m.layers[m.runs[ri].layer];
        HyperArgs a{};
        a.X = m.xs.p; a.S = m.n_streams; a.D = D; a.gvec = gv; a.eps = eps; a.h = m.h.p;
        const LayerW* next = nullptr;
        int nq = 0;
        size_t nri = ri;
        if (q < 0) next = &L;
        else {
            a.y = m.mo.p; a.mix = L.hc_mix[q]; a.out = L.hc_out[q];
            a.bias = q == 0 ? L.o_bias : nullptr;
            if (q == 0 && L.d.ff > 0) { next = &L; nq = 1; }
            else {
                a.sum = m.x.p;
                if (ri + 1 < m.runs.size()) { nri = ri + 1; next = &m.layers[m.runs[nri].layer]; }
            }
        }
        if (next) {
            a.in_next = next->hc_in[nq]; a.gain = nq == 0 ? next->norm1 : next->norm2;
            const float* cw = nq == 0 ? next->canon : next->canon2;
            if (all_single && cw) {   // the next sublayer's convolution rides along
                a.conv_w = cw; a.conv_state = nq == 0 ? m.runs[nri].conv_state.p : m.runs[nri].conv_state2.p; a.hc = m.hc.p; a.taps = next->d.conv_taps;
            }
        }
        // few rows: more threads a row, one coordinate each; many rows: 256 threads with four neighbouring coordinates each (D in fours)
        const bool few = T <= 2 * g_num_sms;
        const bool v4 = !few && D % 4 == 0;
#define TI_HYPER_CASE(N)                                                                                                                              \
    case N:                                                                                                                                           \
        if (v4) TRY(launch_dep(hyper_kernel<N, 4>, dim3(T), dim3(nt), 0, a, sm));                                                                     \
        else TRY(launch_dep(hyper_kernel<N, 1>, dim3(T), dim3(few ? std::min(hyper_max_threads<N>(), std::max(nt, (D + 31) / 32 * 32)) : nt), 0, a, sm)); \
        break;
        switch (m.n_streams) {
            TI_HYPER_CASE(1) TI_HYPER_CASE(2) TI_HYPER_CASE(3) TI_HYPER_CASE(4) TI_HYPER_CASE(5) TI_HYPER_CASE(6) TI_HYPER_CASE(7) TI_HYPER_CASE(8)
            default: TRY(launch_dep(hyper_kernel<0, 1>, dim3(T), dim3(nt), 0, a, sm)); break;
        }
#undef TI_HYPER_CASE
        LAUNCHED();
        return 0;
    };
    // the short convolution in front of a sublayer: y = x + conv(x) over the sequence's last inputs; the slot then keeps the newest ones
    auto short_conv = [&](const float* in, const float* w, int taps, float* state, float* out) -> int {
        constexpr int kConvRows = 8;   // rows a block of the many-rows kernel takes
        const dim3 rows_grid((T + kConvRows - 1) / kConvRows, (D / 4 + 127) / 128);
        if (T > 64 && D % 4 == 0 && taps <= 4) TRY(launch_dep(short_conv_rows_kernel<kConvRows, 4>, rows_grid, dim3(128), 0, in, sm, T, D, taps, w, state, out));
        else if (T > 64 && D % 4 == 0 && taps <= 8) TRY(launch_dep(short_conv_rows_kernel<kConvRows, 8>, rows_grid, dim3(128), 0, in, sm, T, D, taps, w, state, out));
        else if (T > 64 && D % 4 == 0) TRY(launch_dep(short_conv_kernel<4>, dim3(T), dim3(std::min(nt, (D / 4 + 31) / 32 * 32)), 0, in, sm, D, taps, w, state, out));
        else TRY(launch_dep(short_conv_kernel<1>, dim3(T, T <= 64 ? (D + nt - 1) / nt : 1), dim3(nt), 0, in, sm, D, taps, w, state, out));
        LAUNCHED();
        bool many = false;   // (an entry of one row has shifted its state in the kernel above)
        for (int e = 0; e < E; ++e) many = many || counts[e] > 1;
        if (taps > 1 && many) {
            TRY(launch_dep(short_conv_save_kernel, dim3(E, (D + nt - 1) / nt), dim3(nt), 0, in, sm, D, taps, state));
            LAUNCHED();
        }
        return 0;
    };
    if (front) TRY(hyper(0, -1));
    // paged softmax attention of all rows of the step (prompt portions in tiles, the other rows one by one or split over their keys)
    auto attention = [&](const AttnShape& s, const float* q, const float* kp, const float* vp, float* out) -> int {
        const bool wide = std::max(s.dim, s.vdim) > 32 * kAttnMaxPerLane;
        const size_t smem = ((size_t)kAttnWarps * s.vdim + 2 * kAttnWarps) * sizeof(float);
        const bool v_in_k = kp == vp && s.kv_heads == 1 && s.v_ld == s.dim && s.vdim <= s.dim;
        const size_t tsmem = attn_tiled_smem_bytes(s.dim, s.vdim, v_in_k);
        const bool tiled_ok = g_use_tiled_attn && n_tiles > 0 && s.dim % 4 == 0 && s.vdim % 4 == 0 && s.vdim <= 512 && tsmem <= g_smem_optin && (s.v_ld % 4 == 0);
        // bf16 mode, head sizes 64 / 128: the split-half tensor-core kernel (fp32-accurate); fp32 mode keeps true fp32 arithmetic
        const bool h3_ok = g_use_tiled_attn && g_use_tc && bf && n_tiles128 > 0 && s.dim == s.vdim && (s.dim == 64 || s.dim == 128) &&
                           (s.kv_heads * s.dim) % 4 == 0 && s.v_ld == 0;
        // bf16 mode, a shared key/value head with the values inside the key rows (latent attention), instantiated sizes: tensor cores
        const bool lat_size = (s.dim == 320 && s.vdim == 256) || (s.dim == 192 && s.vdim == 128) || (s.dim == 160 && s.vdim == 128);
        const bool lat_ok = g_use_tiled_attn && g_use_tc && bf && n_tiles > 0 && v_in_k && (!s.out_gate || s.gate) && !s.qk_norm && lat_size;
        const int* rest = (tiled_ok || h3_ok || lat_ok) ? d_small : nullptr;
        const int n_rest = (tiled_ok || h3_ok || lat_ok) ? n_small : T;
        if (lat_ok) {
            const dim3 grid(n_tiles, s.heads);
            if (s.dim == 320) latent_attention_h3_kernel<320, 256><<<grid, 256, latent_h3_smem_bytes<320>(), g_stream>>>(q, sm, s, d_tiles, kp, out);
            else if (s.dim == 192) latent_attention_h3_kernel<192, 128><<<grid, 256, latent_h3_smem_bytes<192>(), g_stream>>>(q, sm, s, d_tiles, kp, out);
            else latent_attention_h3_kernel<160, 128><<<grid, 256, latent_h3_smem_bytes<160>(), g_stream>>>(q, sm, s, d_tiles, kp, out);
            LAUNCHED();
        } else if (h3_ok) {
            const dim3 grid(n_tiles128, s.heads);
            if (s.dim == 64) window_attention_h3_kernel<64><<<grid, kTcThreads, attn_h3_smem_bytes<64>(), g_stream>>>(q, sm, s, d_tiles128, kp, vp, out);
            else window_attention_h3_kernel<128><<<grid, kTcThreads, attn_h3_smem_bytes<128>(), g_stream>>>(q, sm, s, d_tiles128, kp, vp, out);
            LAUNCHED();
        } else if (tiled_ok) {
            const dim3 grid(n_tiles, s.heads);
            if (s.vdim <= 64) window_attention_tiled_kernel<1><<<grid, 256, tsmem, g_stream>>>(q, sm, s, d_tiles, kp, vp, out);
            else if (s.vdim <= 128) window_attention_tiled_kernel<2><<<grid, 256, tsmem, g_stream>>>(q, sm, s, d_tiles, kp, vp, out);
            else if (s.vdim <= 256) window_attention_tiled_kernel<4><<<grid, 256, tsmem, g_stream>>>(q, sm, s, d_tiles, kp, vp, out);
            else window_attention_tiled_kernel<8><<<grid, 256, tsmem, g_stream>>>(q, sm, s, d_tiles, kp, vp, out);
            LAUNCHED();
        }
        if (n_rest > 0) {
            // single rows: key chunks in parallel (a row-at-a-time walk is one memory round trip a key) unless the rows alone fill the GPU
            const int span = s.window > 0 ? std::min(s.window, max_pos + 1) : max_pos + 1;
            int splits = 1;
            if (span >= 32) splits = std::max(1, std::min({(span + 15) / 16, kAttnMaxSplits, (2 * g_num_sms) / std::max(1, n_rest * s.heads)}));
            if (splits > 1 && m.attn_part.p) {
                if (wide) TRY(launch_dep(window_attention_split_kernel<kAttnWidePerLane>, dim3(n_rest, s.heads, splits), dim3(kAttnWarps * 32), smem, q, sm, s, rest, splits, kp, vp, m.attn_part.p));
                else TRY(launch_dep(window_attention_split_kernel<kAttnMaxPerLane>, dim3(n_rest, s.heads, splits), dim3(kAttnWarps * 32), smem, q, sm, s, rest, splits, kp, vp, m.attn_part.p));
                LAUNCHED();
                TRY(launch_dep(attention_merge_kernel, dim3((n_rest * s.heads + 7) / 8), dim3(256), 0, (const float*)m.attn_part.p, q, sm, s, rest, n_rest, splits, out));
                LAUNCHED();
            } else {
                if (wide) TRY(launch_dep(window_attention_kernel<kAttnWidePerLane>, dim3(n_rest, s.heads), dim3(kAttnWarps * 32), smem, q, sm, s, rest, kp, vp, out));
                else TRY(launch_dep(window_attention_kernel<kAttnMaxPerLane>, dim3(n_rest, s.heads), dim3(kAttnWarps * 32), smem, q, sm, s, rest, kp, vp, out));
                LAUNCHED();
            }
        }
        return 0;
    };
    // attention whose scores are capped / mixed across the heads / see kept first keys: three passes over a score scratch, in batches
    // of tiles whose scratch stays within L2 (every entry is cut into tiles; short ones take the row kernels of each pass)
    auto mixed_attention = [&](const AttnShape& s, const LayerW& L, const float* q, const float* kp, const float* vp, float* out) -> int {
        const int H = s.heads, HG = s.heads / s.kv_heads;
        int max_total = 1;
        for (int t = 0; t < n_mtiles; ++t) max_total = std::max(max_total, mix_band(h_pos[mtiles[2 * t]], mtiles[2 * t + 1], s.window, s.keep_first).total);
        const int ldu = (max_total + 63) / 64 * 64;
        const size_t per_row = (size_t)H * ldu;
        const size_t budget_rows = std::min<size_t>(32768, std::max<size_t>(kAttnTile, ((size_t)24 << 20) / per_row));   // 96 MiB of scores: most of them stay in L2 between the passes, and a launch fills the GPU
        for (int t0 = 0; t0 < n_mtiles;) {
            int t1 = t0, rows = 0;
            bool big = false, small = false;
            while (t1 < n_mtiles && (t1 == t0 || (size_t)(rows + mtiles[2 * t1 + 1]) <= budget_rows)) {
                rows += mtiles[2 * t1 + 1];
                (mtiles[2 * t1 + 1] >= kAttnTiledMinRows ? big : small) = true;
                ++t1;
            }
            TRY(m.mix_S.ensure((size_t)rows * per_row));
            TRY(m.mix_den.ensure((size_t)rows * H));
            MixArgs a{};
            a.tiles = d_mtiles; a.row_tile = d_row_tile; a.tile0 = t0; a.row_base = mtiles[2 * t0]; a.ldu = ldu; a.small = kAttnTiledMinRows;
            a.S = m.mix_S.p; a.inv_den = m.mix_den.p;
            const int nt_b = t1 - t0, d4 = (s.dim + 3) / 4 * 4, dv4 = (s.vdim + 3) / 4 * 4;
            if (big) {
                // bf16 mode: split-half tensor-core products (fp32-accurate); fp32 mode keeps true fp32 arithmetic
                if (bf && g_use_tc && s.dim % 16 == 0) TRY(launch_dep(mix_scores_tiles_kernel<true>, dim3((ldu / 64 + 2) / 3, nt_b, H), dim3(256), (size_t)2 * 64 * (d4 + 8) * sizeof(float), q, sm, s, a, kp));
                else TRY(launch_dep(mix_scores_tiles_kernel<false>, dim3((ldu / 64 + 2) / 3, nt_b, H), dim3(256), (size_t)2 * 64 * (d4 + 8) * sizeof(float), q, sm, s, a, kp));
                LAUNCHED();
            }
            if (small) {
                TRY(launch_dep(mix_scores_rows_kernel<kAttnMaxPerLane>, dim3(ldu / 64, rows, s.kv_heads), dim3(256), (size_t)HG * s.dim * sizeof(float), q, sm, s, a, kp));
                LAUNCHED();
            }
            const dim3 g2(big ? kAttnTile : kAttnTiledMinRows - 1, nt_b);
            // a row's mixed scores wait in shared memory between the two sweeps when they fit (three blocks an SM), else in the scratch
            const size_t row_bytes = per_row * sizeof(float);
            const int in_smem = row_bytes <= 72 * 1024 ? 1 : 0;
            const size_t sm2 = in_smem ? row_bytes : 0;
            // more than 16 heads: the form that mixes out of shared memory, when a row's scores of all heads fit there
            if (L.mix_HP >= 32 && mix_softmax_wide_smem_bytes(H, ldu) <= g_smem_optin) {
                if (H <= 32) TRY(launch_dep(mix_softmax_wide_kernel<8>, g2, dim3(kMixWideThreads), mix_softmax_wide_smem_bytes(H, ldu), sm, s, a));
                else TRY(launch_dep(mix_softmax_wide_kernel<16>, g2, dim3(kMixWideThreads), mix_softmax_wide_smem_bytes(H, ldu), sm, s, a));
                LAUNCHED();
            } else {
            // (few rows: 512 threads a row have more of its loads in flight; many rows fill the GPU better with 256)
            if (L.mix_HP == 8 && !big) TRY(launch_dep(mix_softmax_kernel<8, 512>, g2, dim3(512), sm2, sm, s, a, in_smem));
            else if (L.mix_HP == 16 && !big) TRY(launch_dep(mix_softmax_kernel<16, 512>, g2, dim3(512), sm2, sm, s, a, in_smem));
            else if (L.mix_HP == 8) TRY(launch_dep(mix_softmax_kernel<8, 256>, g2, dim3(256), sm2, sm, s, a, in_smem));
            else if (L.mix_HP == 16) TRY(launch_dep(mix_softmax_kernel<16, 256>, g2, dim3(256), sm2, sm, s, a, in_smem));
            else if (L.mix_HP == 32) TRY(launch_dep(mix_softmax_kernel<32, 256>, g2, dim3(256), sm2, sm, s, a, in_smem));
            else TRY(launch_dep(mix_softmax_kernel<64, 256>, g2, dim3(256), sm2, sm, s, a, in_smem));
            LAUNCHED();
            }
            if (big) {
                if (bf && g_use_tc) TRY(launch_dep(mix_values_tiles_kernel<true>, dim3(nt_b, H, (dv4 + 63) / 64), dim3(256), (size_t)4 * 64 * 72 * sizeof(__half), sm, s, a, vp, out));
                else TRY(launch_dep(mix_values_tiles_kernel<false>, dim3(nt_b, H, (dv4 + 63) / 64), dim3(256), (size_t)64 * (68 + 64) * sizeof(float), sm, s, a, vp, out));
                LAUNCHED();
            }
            if (small) {
                TRY(launch_dep(mix_values_rows_kernel<kAttnMaxPerLane>, dim3(rows, H), dim3(kMixRowWarps * 32), (size_t)kMixRowWarps * s.vdim * sizeof(float), sm, s, a, vp, out));
                LAUNCHED();
            }
            t0 = t1;
        }
        return 0;
    };
    for (size_t ri = 0; ri < m.runs.size(); ++ri) {
        Run& R = m.runs[ri];
        LayerW& L = m.layers[R.layer];
        if (R.enters_pass) {
            TRY(launch_dep(concat_rows_kernel, dim3(T), dim3(nt), 0, m.x.p, m.x0.p, D, m.xc.p));
            LAUNCHED();
            TRY(gemm(m, m.xc.p, 2 * D, m.loop_in, m.x.p, D, T, D, 2 * D));
        }
        const int mixer = L.d.mixer;
        const bool attn = mixer == TI_SEQ_MIXER_ATTENTION;
        // decode steps (few rows) fuse the norm in front of the attention projections into the product's prologue
        const bool behind = m.d.norm_place == TI_SEQ_NORMS_BEHIND;   // the sublayers read the residual stream itself
        const bool fuse_rows = few_rows(T, D) && !L.d.res_gate && !behind && !front && L.d.conv_taps < 1;
        // the mixers with ONE fused input projection (residual gate included) take the norm into that product's prologue as well
        const bool fuse_front = few_rows(T, D) && (mixer == TI_SEQ_MIXER_GLA || mixer == TI_SEQ_MIXER_HGRN2 || mixer == TI_SEQ_MIXER_LATENT) && !L.rg1 && !front && L.d.conv_taps < 1;
        Fuse ff1;
        ff1.norm_gain = L.norm1; ff1.eps = eps; ff1.gvec = gv;
        const Fuse* front_fuse = fuse_front ? &ff1 : nullptr;
        if (!(fuse_rows && attn) && !fuse_front && !behind && !front) {   // (with norms in front only, the sublayer before this one has left the input in m.h)
            TRY(launch_dep(rmsnorm_kernel, dim3(T), dim3(nt), 0, (const float*)m.x.p, D, (const int*)nullptr, D, L.norm1, gv, eps, m.h.p));
            LAUNCHED();
        }
        const float* mix_in = behind ? m.x.p : m.h.p;   // what the mixer reads
        if (L.d.conv_taps >= 1) {   // ... with the short convolution over the sequence's last inputs added (decoding with norms in front: done already)
            if (!(front && all_single)) TRY(short_conv(mix_in, L.canon, L.d.conv_taps, R.conv_state.p, m.hc.p));
            mix_in = m.hc.p;
        }
        const float* front_in = fuse_front ? m.x.p : mix_in;
        const float* gate1 = nullptr;   // residual gate of the mixer: pre-activations and their row stride
        int gate1_ld = 0;
        if (L.d.res_gate && L.rg1) {
            TRY(gemm(m, m.h.p, D, L.rg1, m.rgbuf.p, D, T, D, D));
            gate1 = m.rgbuf.p;
            gate1_ld = D;
        } else if (L.d.res_gate) {
            gate1 = m.proj.p + L.off_rg1;
            gate1_ld = L.ld_front;
        }
        if (attn) {
            AttnShape s{};
            s.heads = L.d.heads; s.kv_heads = L.d.kv_heads; s.dim = L.d.dim; s.vdim = L.d.vdim;
            s.window = L.d.window; s.rot_dims = L.d.rot_dims; s.qk_norm = L.d.qk_norm; s.out_gate = L.d.out_gate;
            s.scale = L.d.scale; s.eps = eps; s.ld = L.n_qkvg;
            if (fuse_rows) {
                Fuse f;
                f.norm_gain = L.norm1; f.eps = eps; f.gvec = gv;
                TRY(gemm(m, m.x.p, D, L.qkvg, m.proj.p, L.n_qkvg, T, L.n_qkvg, D, EPI_NONE, 1.f, &f));
            } else {
                TRY(gemm(m, mix_in, D, L.qkvg, m.proj.p, L.n_qkvg, T, L.n_qkvg, D));
            }
            s.sink = L.sink; s.softcap = L.d.softcap; s.keep_first = L.d.keep_first; s.talk = L.talk;
            s.rot_half = L.d.rot_half; s.v_norm = L.d.v_norm; s.bias = L.qkv_bias.p; s.temp = L.temp;
            if (L.d.qk_norm == TI_SEQ_QK_NORM_WHOLE) TRY(launch_dep(attn_prepare_whole_kernel, dim3(T), dim3(256), 0, m.proj.p, sm, s, L.qnorm, L.knorm, R.k_pool.p, R.v_pool.p));
            else TRY(launch_dep(attn_prepare_kernel, dim3(T), dim3(128), 0, m.proj.p, sm, s, L.inv_freq.p, R.k_pool.p, R.v_pool.p));
            LAUNCHED();
            if (L.mix_HP > 0) TRY(mixed_attention(s, L, m.proj.p, R.k_pool.p, R.v_pool.p, m.att.p));
            else TRY(attention(s, m.proj.p, R.k_pool.p, R.v_pool.p, m.att.p));
            TRY(gemm(m, m.att.p, s.heads * s.vdim, L.o, m.mo.p, D, T, D, s.heads * s.vdim));
        } else if (mixer == TI_SEQ_MIXER_WKV) {
            const int C = L.d.heads * L.d.dim, d = L.d.dim, rank = L.d.decay_rank;
            const size_t TD = (size_t)T * D, TC = (size_t)T * C;
            float *pr = m.proj.p, *pk = pr + TC, *pv = pk + TC, *pg = pv + TC, *pz = pg + TC;
            if (fuse_rows) {   // the five input products and their token-shift mixes in one launch
                TRY(wkv_front(m, L, R, sm, T, pr, pk, pv, pg, m.lora.p));
                TRY(launch_dep(wkv_save_prev_kernel, dim3(E), dim3(nt), 0, m.h.p, sm, D, R.prev.p));
                LAUNCHED();
            } else {
                TRY(launch_dep(wkv_mix_kernel, dim3(T), dim3(nt), 0, m.h.p, sm, D, L.mu.p, R.prev.p, m.mixes.p));
                LAUNCHED();
                TRY(launch_dep(wkv_save_prev_kernel, dim3(E), dim3(nt), 0, m.h.p, sm, D, R.prev.p));
                LAUNCHED();
                TRY(gemm(m, m.mixes.p + 0 * TD, D, L.r, pr, C, T, C, D));
                TRY(gemm(m, m.mixes.p + 1 * TD, D, L.k, pk, C, T, C, D));
                TRY(gemm(m, m.mixes.p + 2 * TD, D, L.v, pv, C, T, C, D));
                TRY(gemm(m, m.mixes.p + 3 * TD, D, L.g, pg, C, T, C, D, EPI_SILU));
                TRY(gemm(m, m.mixes.p + 4 * TD, D, L.w1, m.lora.p, rank, T, rank, D, EPI_TANH));
            }
            TRY(gemm(m, m.lora.p, rank, L.w2, pz, C, T, C, rank));
            WkvArgs a{};
            a.r = pr; a.k = pk; a.v = pv; a.z = pz;
            a.w0 = L.w0; a.u = L.u;
            a.state = R.state.p; a.out = m.att.p; a.heads = L.d.heads; a.dim = d;
            const dim3 grid(E, L.d.heads);
            if (d == 32) TRY(launch_dep(wkv_scan_split_kernel<32, 8, 4>, dim3(E, L.d.heads, 1), dim3(128), 0, a, sm));
            else if (d == 64) TRY(launch_dep(wkv_scan_split_kernel<64, 8, 8>, dim3(E, L.d.heads, 2), dim3(256), 0, a, sm));
            else if (d == 128) TRY(launch_dep(wkv_scan_split_kernel<128, 4, 16>, dim3(E, L.d.heads, 4), dim3(512), 0, a, sm));
            else {
                const size_t small = 4 * (size_t)d * sizeof(float), full = small + (size_t)d * d * sizeof(float);
                a.s_in_smem = full <= g_smem_optin ? 1 : 0;
                TRY(launch_dep(wkv_scan_kernel, dim3(grid), dim3((d + 31) / 32 * 32), a.s_in_smem ? full : small, a, sm));
            }
            LAUNCHED();
            TRY(launch_dep(head_rmsnorm_gate_kernel, dim3((T * L.d.heads + 7) / 8), dim3(256), 0, m.att.p, (const float*)pg, C, 0, L.normw, 1, T, L.d.heads, d, eps));
            LAUNCHED();
            TRY(gemm(m, m.att.p, C, L.o, m.mo.p, D, T, D, C));
        } else if (mixer == TI_SEQ_MIXER_GLA || mixer == TI_SEQ_MIXER_HGRN2) {
            const bool gla = mixer == TI_SEQ_MIXER_GLA;
            const int H = L.d.heads, dk = L.d.dim, dv = L.d.vdim, C = H * dk, Cv = H * dv, nf = L.n_front;
            TRY(gemm(m, front_in, D, L.front, m.proj.p, nf, T, nf, D, EPI_NONE, 1.f, front_fuse));
            LinScanArgs a{};
            a.q = m.proj.p + L.off_q; a.ldq = nf;
            a.v = m.proj.p + L.off_v; a.ldv = nf;
            if (gla) {   // decay = sigmoid(A2 (A1 h) + b)^(1 / tau): the scan turns the second product's output into decays as it stages them
                TRY(gemm(m, m.proj.p + L.off_a1, nf, L.a2, m.aux.p, C, T, C, L.d.decay_rank));
                a.k = m.proj.p + L.off_k; a.ldk = nf;
                a.a = m.aux.p; a.lda = C;
                a.qscale = 1.f / sqrtf((float)dk);
                a.gates = LIN_GATES_GLA; a.bias = L.a2b; a.lower = nullptr; a.inv_tau = 1.f / L.d.decay_tau;
            } else {     // q = silu(.), forget gate f = lower + (1 - lower) sigmoid(. + b) is the decay, 1 - f is written (all inside the scan)
                a.k = nullptr; a.ldk = 0;
                a.a = m.proj.p + L.off_k; a.lda = nf;
                a.qscale = 1.f;
                a.gates = LIN_GATES_HGRN2; a.bias = L.fb; a.lower = L.lower; a.inv_tau = 1.f;
            }
            a.state = R.state.p; a.out = m.att.p; a.heads = H; a.dk = dk; a.dv = dv;
            const int threads = std::min(128, (dv + 31) / 32 * 32);
            const dim3 grid(E, H, (dv + threads - 1) / threads);
            const int zg = (dv + 31) / 32;
            if (dk == 32) TRY(launch_dep(linear_scan_split_kernel<32, 8, 4>, dim3(E, H, zg), dim3(128), 0, a, sm));
            else if (dk == 64) TRY(launch_dep(linear_scan_split_kernel<64, 8, 8>, dim3(E, H, zg), dim3(256), 0, a, sm));
            else if (dk == 128) TRY(launch_dep(linear_scan_split_kernel<128, 4, 16>, dim3(E, H, zg), dim3(512), 0, a, sm));
            else if (dk <= 32) TRY(launch_dep(linear_scan_kernel<32>, grid, dim3(threads), linear_scan_smem_bytes(dk, threads, false), a, sm));
            else if (dk <= 64) TRY(launch_dep(linear_scan_kernel<64>, grid, dim3(threads), linear_scan_smem_bytes(dk, threads, false), a, sm));
            else if (dk <= 128) TRY(launch_dep(linear_scan_kernel<128>, grid, dim3(threads), linear_scan_smem_bytes(dk, threads, false), a, sm));
            else {
                const int th = linear_scan_smem_bytes(dk, threads, true) <= g_smem_optin ? threads : 32;
                const dim3 g2(E, H, (dv + th - 1) / th);
                if (linear_scan_smem_bytes(dk, th, true) > g_smem_optin) return fail("layer %d: %d key channels do not fit the recurrence kernel", R.layer, dk);
                TRY(launch_dep(linear_scan_kernel<0>, g2, dim3(th), linear_scan_smem_bytes(dk, th, true), a, sm));
            }
            LAUNCHED();
            TRY(launch_dep(head_rmsnorm_gate_kernel, dim3((T * H + 7) / 8), dim3(256), 0, m.att.p, gla ? (const float*)(m.proj.p + L.off_g) : (const float*)nullptr, nf, 1,
                           L.normw, 0, T, H, dv, eps));
            LAUNCHED();
            TRY(gemm(m, m.att.p, Cv, L.o, m.mo.p, D, T, D, Cv));
        } else {   // latent attention
            const int H = L.d.heads, d = L.d.dim, dr = L.d.rot_dims, dv = L.d.vdim, rank = L.d.kv_rank, kd = rank + dr, nf = L.ld_front;
            TRY(gemm(m, front_in, D, L.front, m.proj.p, nf, T, L.n_front, D, EPI_NONE, 1.f, front_fuse));
            if (L.d.q_rank > 0) {   // q = Uq norm(Dq h): the norm rides in the second product's prologue when the rows are few
                const int qr = L.d.q_rank, nq = H * (d + dr);
                if (few_rows(T, qr)) {
                    Fuse f;
                    f.norm_gain = L.dqnorm; f.eps = eps; f.gvec = 1;
                    TRY(gemm(m, m.proj.p + L.off_dq, nf, L.uq, m.proj.p + L.off_q, nf, T, nq, qr, EPI_NONE, 1.f, &f));
                } else {
                    TRY(launch_dep(rmsnorm_kernel, dim3(T), dim3(nt), 0, (const float*)(m.proj.p + L.off_dq), nf, (const int*)nullptr, qr, L.dqnorm, 1, eps, m.lora.p));
                    LAUNCHED();
                    TRY(gemm(m, m.lora.p, qr, L.uq, m.proj.p + L.off_q, nf, T, nq, qr));
                }
            }
            float* pool = R.kv_run >= 0 ? m.runs[R.kv_run].k_pool.p : R.k_pool.p;
            LatentShape ls{};
            ls.heads = H; ls.dim = d; ls.rot = dr; ls.rank = rank; ls.ld = nf; ls.off_q = L.off_q; ls.off_dkv = L.off_dkv; ls.eps = eps;
            ls.rot_half = L.d.rot_half;
            TRY(launch_dep(latent_prepare_kernel, dim3(T), dim3(128), 0, (const float*)m.proj.p, sm, ls, (const float*)L.inv_freq.p, L.cnorm, pool, m.aux.p));
            LAUNCHED();
            // the key up-projection moves to the query: qabs[t][h][0 .. rank) = Uk_h^T q_h
            TRY(gemm_heads(m, m.proj.p + L.off_q, nf, d + dr, L.ukT.p, m.aux.p, H * kd, kd, H, T, rank, d));
            AttnShape s{};
            s.heads = H; s.kv_heads = 1; s.dim = kd; s.vdim = rank; s.window = L.d.window; s.rot_dims = 0; s.qk_norm = 0;
            s.scale = L.d.scale; s.eps = eps; s.ld = H * kd; s.v_ld = kd; s.sink = L.sink;
            // (the gate is one number a head: it commutes with the value up-projection behind the weighted sum)
            s.out_gate = L.d.out_gate; s.gate = L.d.out_gate ? m.proj.p + L.off_g : nullptr; s.gate_ld = nf;
            TRY(attention(s, m.aux.p, pool, pool, m.aux2.p));
            // ... and the value up-projection behind the weighted sum: att[t][h] = Uv_h (sum_j p_j c_j)
            TRY(gemm_heads(m, m.aux2.p, H * rank, rank, L.uv, m.att.p, H * dv, dv, H, T, dv, rank));
            TRY(gemm(m, m.att.p, H * dv, L.o, m.mo.p, D, T, D, H * dv));
        }
        if (L.d.ff > 0) {
            const bool fuse_ff = fuse_rows && L.d.ff_kind == TI_SEQ_FF_GLU;
            if (front) TRY(hyper(ri, 0));
            else TRY(post(L.norm1b, gv, (fuse_ff || behind) ? nullptr : L.norm2, gate1, gate1_ld, L.rg1b, nullptr));
            const float* ff_in = behind ? m.x.p : m.h.p;   // what the feed-forward reads
            if (L.canon2) {
                if (!(front && all_single)) TRY(short_conv(ff_in, L.canon2, L.d.conv_taps, R.conv_state2.p, m.hc.p));
                ff_in = m.hc.p;
            }
            const float* gate2 = nullptr;
            int gate2_ld = 0;
            if (L.d.res_gate && L.rg2) {
                TRY(gemm(m, m.h.p, D, L.rg2, m.rgbuf.p, D, T, D, D));
                gate2 = m.rgbuf.p;
                gate2_ld = D;
            } else if (L.d.res_gate) {
                gate2 = m.proj.p + L.off_rg2;
                gate2_ld = L.n_ffront;
            }
            const float* idw = nullptr;
            bool down_done = false;
            const int F = L.d.ff;
            if (L.d.ff_kind == TI_SEQ_FF_DENSE) {   // the activation rides in the up product's epilogue
                const int epi = L.d.ff_act == TI_SEQ_ACT_XIELU ? EPI_XIELU : L.d.ff_act == TI_SEQ_ACT_SILU ? EPI_SILU : L.d.ff_act == TI_SEQ_ACT_GELU_TANH ? EPI_GELU_TANH : EPI_MAX0;
                TRY(gemm(m, ff_in, D, L.ffront, m.act.p, F, T, F, D, epi, L.act_a, nullptr, L.act_b));
            } else if (L.d.ff_kind == TI_SEQ_FF_GLU) {
                if (fuse_ff) {   // norm -> [gate | up] -> act(gate) * up in one launch
                    Fuse f;
                    f.norm_gain = L.norm2; f.eps = eps; f.gvec = gv; f.glu_ff = F; f.glu_act = L.d.ff_act;
                    TRY(gemm(m, m.x.p, D, L.gateup, m.act.p, F, T, F, D, EPI_NONE, 1.f, &f));
                } else if (few_rows(T, D)) {   // [gate | up] -> act(gate) * up in one launch
                    Fuse f;
                    f.glu_ff = F; f.glu_act = L.d.ff_act;
                    TRY(gemm(m, ff_in, D, L.gateup, m.act.p, F, T, F, D, EPI_NONE, 1.f, &f));
                } else {
                    TRY(gemm(m, ff_in, D, L.gateup, m.proj.p, 2 * F, T, 2 * F, D));
                    glu_kernel<<<grid_for((size_t)T * F), 256, 0, g_stream>>>(m.proj.p, F, L.d.ff_act, m.act.p, (size_t)T * F);
                    LAUNCHED();
                }
            } else if (L.d.ff_kind == TI_SEQ_FF_POLYNORM) {
                TRY(gemm(m, m.h.p, D, L.ffront, m.proj.p, L.n_ffront, T, L.n_ffront, D));
                TRY(launch_dep(polynorm_kernel, dim3(T), dim3(nt), 0, (const float*)(m.proj.p + L.off_up), L.n_ffront, F, L.poly, eps, m.act.p));
                LAUNCHED();
            } else {
                const int nfw = L.n_ffront, Ex = L.d.experts;
                RouteShape r{};
                r.n_real = Ex; r.n_id = L.d.identity; r.top = L.d.top; r.groups = L.d.groups; r.keep = L.d.groups_keep;
                r.by_logits = L.d.route_kind == TI_SEQ_ROUTE_TOP_LOGITS ? 1 : 0;
                const float* route_vec = r.by_logits ? L.route_bias : L.correction;
                float* wdense = m.route.p;
                float* idw_buf = m.route.p + (size_t)T * std::max(Ex, 1);
                const size_t rper = (size_t)(2 * (Ex + L.d.identity) + 2 * L.d.groups) * sizeof(float);
                // few rows: [router | shared scale | residual gate] first, then the experts' rows with the ones nobody chose left out
                const bool sparse = few_rows(T, D) && bf && Ex > 0 && L.off_up > 0 && T * rper <= 40 * 1024;
                if (sparse) {
                    int* used = reinterpret_cast<int*>(idw_buf + T);
                    TRY(gemm(m, ff_in, D, L.ffront, m.proj.p, nfw, T, L.off_up, D));
                    TRY(launch_dep(moe_route_kernel, dim3(1), dim3(T * 32), T * rper, (const float*)m.proj.p, nfw, L.off_router, r, route_vec, T, wdense, idw_buf, used));
                    LAUNCHED();
                    Fuse f;
                    f.nskip = ExpertSkip{used, 0, 2 * F, Ex};
                    TRY(gemm(m, ff_in, D, (const uint8_t*)L.ffront + (size_t)L.off_up * D * m.wsize, m.proj.p + L.off_up, nfw, T, nfw - L.off_up, D, EPI_NONE, 1.f, &f));
                } else {
                    TRY(gemm(m, ff_in, D, L.ffront, m.proj.p, nfw, T, nfw, D));
                    const int rw = 4;
                    TRY(launch_dep(moe_route_kernel, dim3((T + rw - 1) / rw), dim3(rw * 32), rw * rper, (const float*)m.proj.p, nfw, L.off_router, r, route_vec, T, wdense, idw_buf,
                                   (int*)nullptr));
                    LAUNCHED();
                }
                if (L.ff_width > 0) {
                    TRY(launch_dep(moe_act_kernel, dim3(grid_for((size_t)T * L.ff_width)), dim3(256), 0, (const float*)m.proj.p, nfw, L.off_up, Ex, F, (const float*)wdense, L.off_sh,
                                   L.d.shared_ff, L.off_sg, m.act.p, T));
                    LAUNCHED();
                }
                if (sparse) {
                    Fuse f;
                    f.kskip = ExpertSkip{reinterpret_cast<const int*>(idw_buf + T), 0, F, Ex};
                    TRY(gemm(m, m.act.p, L.ff_width, L.down, m.mo.p, D, T, D, L.ff_width, EPI_NONE, 1.f, &f));
                    down_done = true;
                }
                if (L.d.identity > 0) idw = idw_buf;
            }
            if (down_done) {}
            else if (L.ff_width > 0) TRY(gemm(m, m.act.p, L.ff_width, L.down, m.mo.p, D, T, D, L.ff_width));
            else CK(cudaMemsetAsync(m.mo.p, 0, (size_t)T * D * sizeof(float), g_stream));
            if (front) TRY(hyper(ri, 1));
            else TRY(post(L.norm2b, gv, nullptr, gate2, gate2_ld, L.rg2b, idw));
        } else if (front) {
            TRY(hyper(ri, 0));
        } else {
            TRY(post(L.norm1b, gv, nullptr, gate1, gate1_ld, L.rg1b, nullptr));
        }
        if (m.d.side_dim > 0) {   // per-token side input: x += plain_norm(P (gelu_tanh(G x) * side_embedding[token, layer slice]))
            const int ds = m.d.side_dim;
            TRY(gemm(m, m.x.p, D, L.side_gate, m.aux2.p, ds, T, ds, D, EPI_GELU_TANH));
            if (bf) TRY(launch_dep(side_mul_kernel<__nv_bfloat16>, dim3(grid_for((size_t)T * ds)), dim3(256), 0, m.aux2.p, sm, (const __nv_bfloat16*)m.side_embed, ds * m.d.n_layers, R.layer, ds));
            else TRY(launch_dep(side_mul_kernel<float>, dim3(grid_for((size_t)T * ds)), dim3(256), 0, m.aux2.p, sm, (const float*)m.side_embed, ds * m.d.n_layers, R.layer, ds));
            LAUNCHED();
            TRY(gemm(m, m.aux2.p, ds, L.side_proj, m.mo.p, D, T, D, ds));
            TRY(post(L.side_norm, 1, nullptr, nullptr, 0, nullptr, nullptr));
        }
        if (m.dbg) CK(cudaMemcpyAsync(m.dbg_buf.p + ri * (size_t)T * D, m.x.p, (size_t)T * D * sizeof(float), cudaMemcpyDeviceToDevice, g_stream));
    }
    m.dbg_rows = T;
    if (n_out > 0) {
        // logits: scaled, or capped through cap * tanh(. / cap)
        const int head_epi = m.d.logit_softcap > 0.f ? EPI_SOFTCAP : EPI_SCALE;
        const float head_alpha = m.d.logit_softcap > 0.f ? m.d.logit_softcap : m.d.logit_scale;
        if (few_rows(n_out, D)) {
            TRY(launch_dep(gather_rows_kernel, dim3(n_out), dim3(nt), 0, m.x.p, d_out, D, m.hn.p));
            LAUNCHED();
            Fuse f;
            f.norm_gain = m.final_norm; f.eps = eps; f.gvec = m.gvec;
            TRY(gemm(m, m.hn.p, D, m.head, m.logits.p, V, n_out, V, D, head_epi, head_alpha, &f));
        } else {
            TRY(launch_dep(rmsnorm_kernel, dim3(n_out), dim3(nt), 0, (const float*)m.x.p, D, d_out, D, m.final_norm, m.gvec, eps, m.hn.p));
            LAUNCHED();
            TRY(gemm(m, m.hn.p, D, m.head, m.logits.p, V, n_out, V, D, head_epi, head_alpha));
        }
    }
    if (smp.on) {
        const bool greedy = !(smp.temperature > 0.f) || smp.top_k == 1;
        if (greedy) {
            TRY(launch_dep(argmax_rows_kernel, dim3(E), dim3(1024), 0, m.logits.p, V, V, m.picks.p, m.logprobs.p));
            LAUNCHED();
        } else {
            const size_t row_smem = sample_row_smem_bytes(V);
            for (int e = 0; e < E; ++e) {   // one launch per sequence: every sequence has its own RNG stream and counter
                SampleArgs a{};
                a.logits = m.logits.p + (size_t)e * V; a.V = V; a.ld = V;
                a.temperature = smp.temperature; a.top_k = smp.top_k; a.top_p = smp.top_p;
                a.seed = smp.seed + 0x9E3779B97F4A7C15ull * (uint64_t)(uint32_t)seqs[e];
                a.step = smp.index ? smp.index[e] : 0;
                a.token_out = m.picks.p + e; a.logprob_out = m.logprobs.p + e;
                a.staged = row_smem ? 1 : 0;
                if (sample_keys_in_registers(V)) sample_kernel<32><<<1, kSampleThreads, row_smem, g_stream>>>(a);
                else sample_kernel<0><<<1, kSampleThreads, row_smem, g_stream>>>(a);
                LAUNCHED();
            }
        }
    }
    CK(cudaEventRecord(m.ev1, g_stream));
    if (smp.on) {
        CK(cudaMemcpyAsync(smp.out_tokens, m.picks.p, (size_t)E * sizeof(int), cudaMemcpyDeviceToHost, g_stream));
        if (smp.out_logprobs) CK(cudaMemcpyAsync(smp.out_logprobs, m.logprobs.p, (size_t)E * sizeof(float), cudaMemcpyDeviceToHost, g_stream));
    } else if (n_want > 0 && logits_host) {
        CK(cudaMemcpyAsync(logits_host, m.logits.p, (size_t)n_want * V * sizeof(float), cudaMemcpyDeviceToHost, g_stream));
    }
    int kerr = 0;
    CK(cudaMemcpyAsync(&kerr, m.err.p, sizeof(int), cudaMemcpyDeviceToHost, g_stream));
    CK(cudaStreamSynchronize(g_stream));
    if (kerr) return fail("step: a bounded wait inside a kernel ran out (tensor-core product pipeline)");
    CK(cudaEventElapsedTime(&m.last_ms, m.ev0, m.ev1));
    for (int e = 0; e < E; ++e) m.seqs[seqs[e]].len += counts[e];
    return 0;
}

int open_seq(Model& m, int32_t* seq) {
    for (size_t s = 0; s < m.seqs.size(); ++s)
        if (!m.seqs[s].live) {
            m.seqs[s].live = true;
            m.seqs[s].len = 0;
            m.seqs[s].pages.clear();
            *seq = (int32_t)s;
            return 0;
        }
    return fail("no free state slot (%zu sequences live)", m.seqs.size());
}
int close_seq(Model& m, int32_t seq) {
    if (seq < 0 || seq >= (int)m.seqs.size() || !m.seqs[seq].live) return fail("close: sequence %d is not open", seq);
    SeqState& s = m.seqs[seq];
    for (int p : s.pages) m.free_pages.push_back(p);
    s.pages.clear();
    s.len = 0;
    s.live = false;
    return 0;
}

}  // namespace

extern "C" {

const char* ti_seq_last_error(void) { return g_err.c_str(); }
uint64_t ti_seq_launch_count(void) { return g_launches; }

int ti_seq_init(int device) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return fail("ti_seq_init: no CUDA device (this engine has no CPU fallback)");
    if (device < 0 || device >= n) return fail("ti_seq_init: device %d of %d", device, n);
    CK(cudaSetDevice(device));
    cudaDeviceProp p{};
    CK(cudaGetDeviceProperties(&p, device));
    if (p.major < 10) return fail("ti_seq_init: device %d is sm_%d%d; this library is built for sm_100a only", device, p.major, p.minor);
    g_num_sms = p.multiProcessorCount;
    g_smem_optin = std::min<size_t>(p.sharedMemPerBlockOptin, 200 * 1024);
    if (!g_stream) CK(cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking));
    CK(cudaFuncSetAttribute(gemv_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(gemv_rows_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(gemv_rows_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(wkv_front_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(wkv_front_rows_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(gemv_rows_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(gemm_bf16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSgSmemBytes));
    if (const char* e = getenv("TURBOINFER_B200_SEQ_TC")) g_use_tc = atoi(e) != 0;
    if (const char* e = getenv("TURBOINFER_B200_SEQ_PDL")) g_use_pdl = atoi(e) != 0;
    if (const char* e = getenv("TURBOINFER_B200_SEQ_ROW_MMA")) g_use_row_mma = atoi(e) != 0;
    if (const char* e = getenv("TURBOINFER_B200_SEQ_TILED_ATTN")) g_use_tiled_attn = atoi(e) != 0;
    CK(cudaFuncSetAttribute(window_attention_h3_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_h3_smem_bytes<64>()));
    CK(cudaFuncSetAttribute(window_attention_h3_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_h3_smem_bytes<128>()));
    CK(cudaFuncSetAttribute(window_attention_tiled_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(window_attention_tiled_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(window_attention_tiled_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(wkv_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(window_attention_tiled_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(linear_scan_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(latent_attention_h3_kernel<320, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)latent_h3_smem_bytes<320>()));
    CK(cudaFuncSetAttribute(latent_attention_h3_kernel<192, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)latent_h3_smem_bytes<192>()));
    CK(cudaFuncSetAttribute(latent_attention_h3_kernel<160, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)latent_h3_smem_bytes<160>()));
    CK(cudaFuncSetAttribute(mix_scores_tiles_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(mix_scores_tiles_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(mix_scores_rows_kernel<kAttnMaxPerLane>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(mix_softmax_kernel<8, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    CK(cudaFuncSetAttribute(mix_softmax_kernel<16, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    CK(cudaFuncSetAttribute(mix_softmax_wide_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(mix_softmax_wide_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_smem_optin));
    CK(cudaFuncSetAttribute(mix_softmax_kernel<8, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    CK(cudaFuncSetAttribute(mix_softmax_kernel<16, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    CK(cudaFuncSetAttribute(mix_softmax_kernel<32, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    CK(cudaFuncSetAttribute(mix_softmax_kernel<64, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    CK(cudaFuncSetAttribute(sample_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 176 * 1024));
    CK(cudaFuncSetAttribute(sample_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 176 * 1024));
    g_device = device;
    return 0;
}

int ti_seq_model_new(const ti_seq_model_desc* desc, const ti_seq_layer_desc* layers, ti_seq_model_t* out) {
    if (g_device < 0) return fail("ti_seq: not initialised -- call ti_seq_init(device) first (no CPU fallback exists)");
    if (!desc || !layers || !out) return fail("model_new: null argument");
    if (desc->vocab <= 0 || desc->width <= 0 || desc->n_layers <= 0) return fail("model_new: vocab %d width %d layers %d", desc->vocab, desc->width, desc->n_layers);
    if (desc->mode != TI_SEQ_BF16 && desc->mode != TI_SEQ_F32) return fail("model_new: mode %d", desc->mode);
    if (desc->max_tokens <= 0 || desc->max_seqs <= 0) return fail("model_new: max_tokens %d max_seqs %d", desc->max_tokens, desc->max_seqs);
    if (desc->loop_times > 0 && (desc->loop_start < 0 || desc->loop_stop > desc->n_layers || desc->loop_start >= desc->loop_stop))
        return fail("model_new: looped block [%d, %d) of %d layers", desc->loop_start, desc->loop_stop, desc->n_layers);
    auto m = std::make_unique<Model>();
    m->d = *desc;
    m->wsize = desc->mode == TI_SEQ_BF16 ? 2 : 4;
    m->layers.resize(desc->n_layers);
    for (int i = 0; i < desc->n_layers; ++i) m->layers[i].d = layers[i];
    TRY(describe_tensors(*m));
    // the order of layer runs
    auto add_run = [&](int layer, bool enters) {
        m->runs.emplace_back();
        m->runs.back().layer = layer;
        m->runs.back().enters_pass = enters;
    };
    if (desc->loop_times > 0) {
        for (int i = 0; i < desc->loop_start; ++i) add_run(i, false);
        for (int t = 0; t < desc->loop_times; ++t)
            for (int i = desc->loop_start; i < desc->loop_stop; ++i) add_run(i, i == desc->loop_start && !desc->loop_plain);
        for (int i = desc->loop_stop; i < desc->n_layers; ++i) add_run(i, false);
    } else {
        for (int i = 0; i < desc->n_layers; ++i) add_run(i, false);
    }
    std::lock_guard<std::mutex> lk(g_mu);
    g_models.push_back(std::move(m));
    *out = g_models.size();
    return 0;
}

int ti_seq_model_tensor_count(ti_seq_model_t h, int32_t* n) {
    Model* m = get_model(h);
    if (!m) return fail("bad model handle");
    *n = (int32_t)m->order.size();
    return 0;
}
int ti_seq_model_tensor_info(ti_seq_model_t h, int32_t i, char* name, size_t cap, int64_t* shape, int32_t* ndim) {
    Model* m = get_model(h);
    if (!m) return fail("bad model handle");
    if (i < 0 || i >= (int)m->order.size()) return fail("tensor index %d", i);
    const std::string& nm = m->order[i];
    snprintf(name, cap, "%s", nm.c_str());
    const Tensor& t = m->tensors[nm];
    *ndim = (int32_t)t.shape.size();
    for (size_t k = 0; k < t.shape.size(); ++k) shape[k] = t.shape[k];
    return 0;
}

static int check_shape(const Tensor& t, const char* name, const int64_t* shape, int32_t ndim) {
    bool ok = (size_t)ndim == t.shape.size();
    for (int k = 0; ok && k < ndim; ++k) ok = shape[k] == t.shape[k];
    if (!ok) {
        std::string want, got;
        for (auto s : t.shape) want += std::to_string(s) + " ";
        for (int k = 0; k < ndim; ++k) got += std::to_string(shape[k]) + " ";
        return fail("tensor %s: shape [ %s] given, [ %s] expected", name, got.c_str(), want.c_str());
    }
    return 0;
}

int ti_seq_model_set_tensor(ti_seq_model_t h, const char* name, int32_t dtype, const void* data, const int64_t* shape, int32_t ndim) {
    Model* m = get_model(h);
    if (!m) return fail("bad model handle");
    if (m->finalized) return fail("set_tensor after finalize");
    auto it = m->tensors.find(name);
    if (it == m->tensors.end()) return fail("tensor %s is not part of this model", name);
    Tensor& t = it->second;
    TRY(check_shape(t, name, shape, ndim));
    const size_t n = t.count();
    if (dtype == TI_SEQ_BF16 && t.matrix && m->d.mode == TI_SEQ_BF16) {   // stays as it is
        TRY(t.data.alloc(n * 2));
        CK(cudaMemcpyAsync(t.data.p, data, n * 2, cudaMemcpyHostToDevice, g_stream));
        CK(cudaStreamSynchronize(g_stream));
        t.set = true;
        return 0;
    }
    DevBuf<float> f;
    TRY(f.alloc(n));
    if (dtype == TI_SEQ_BF16) {
        DevBuf<__nv_bfloat16> b;
        TRY(b.alloc(n));
        CK(cudaMemcpyAsync(b.p, data, n * 2, cudaMemcpyHostToDevice, g_stream));
        bf16_to_f32_kernel<<<grid_for(n), 256, 0, g_stream>>>(b.p, f.p, n);
        LAUNCHED();
        CK(cudaStreamSynchronize(g_stream));
    } else if (dtype == TI_SEQ_F32) {
        CK(cudaMemcpyAsync(f.p, data, n * 4, cudaMemcpyHostToDevice, g_stream));
    } else {
        return fail("tensor %s: element type %d", name, dtype);
    }
    return store_from_f32(*m, t, f.p, n);
}

int ti_seq_model_set_tensor_synthetic(ti_seq_model_t h, const char* name, const int64_t* shape, int32_t ndim, uint64_t seed, float amp, float offset) {
    Model* m = get_model(h);
    if (!m) return fail("bad model handle");
    if (m->finalized) return fail("set_tensor after finalize");
    auto it = m->tensors.find(name);
    if (it == m->tensors.end()) return fail("tensor %s is not part of this model", name);
    Tensor& t = it->second;
    TRY(check_shape(t, name, shape, ndim));
    const size_t n = t.count();
    DevBuf<float> f;
    TRY(f.alloc(n));
    synth_fill_f32_kernel<<<grid_for(n), 256, 0, g_stream>>>(f.p, n, seed, amp, offset);
    LAUNCHED();
    return store_from_f32(*m, t, f.p, n);
}

int ti_seq_model_finalize(ti_seq_model_t h) {
    Model* mp = get_model(h);
    if (!mp) return fail("bad model handle");
    Model& m = *mp;
    if (m.finalized) return 0;
    for (const auto& nm : m.order)
        if (!m.tensors[nm].set) return fail("finalize: tensor %s was not given", nm.c_str());
    auto T = [&](const std::string& nm) -> Tensor* {
        auto it = m.tensors.find(nm);
        return it == m.tensors.end() ? nullptr : &it->second;
    };
    auto F = [&](const std::string& nm) -> const float* { return reinterpret_cast<const float*>(T(nm)->data.p); };
    auto P = [&](const std::string& nm) -> const void* { return T(nm)->data.p; };
    const int D = m.d.width;
    m.embed = P("embed");
    m.head = m.d.tied_head ? m.embed : P("head");
    const bool behind = m.d.norm_place == TI_SEQ_NORMS_BEHIND;
    if (m.d.pos_base > 0.f) {   // frequencies in double, rounded once
        std::vector<float> f((size_t)(D + 1) / 2);
        for (size_t i = 0; i < f.size(); ++i) f[i] = (float)std::pow((double)m.d.pos_base, -2.0 * (double)i / (double)D);
        TRY(m.pos_freq.alloc(f.size()));
        CK(cudaMemcpy(m.pos_freq.p, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    if (m.d.side_dim > 0) m.side_embed = P("side.embed");
    if (m.d.loop_times > 0 && !m.d.loop_plain) m.loop_in = P("loop.in");
    m.gvec = m.d.norm_kind != TI_SEQ_NORM_SCALAR ? 1 : 0;
    const bool front = m.d.norm_place == TI_SEQ_NORMS_FRONT;
    if (front) {   // one stream with in = mix = out = 1 is the plain residual x <- x + y
        m.n_streams = std::max(1, m.d.streams);
        const float one[1] = {1.f};
        TRY(m.ones.alloc(1));
        CK(cudaMemcpy(m.ones.p, one, sizeof(one), cudaMemcpyHostToDevice));
    }
    if (m.d.norm_kind == TI_SEQ_NORM_ONE_PLUS) {   // gains stored around zero and applied as 1 + w: converted once
        std::vector<std::string> names{"final.norm"};
        for (int i = 0; i < m.d.n_layers; ++i)
            for (const char* sfx : {"norm1", "norm1b", "norm2", "norm2b"}) names.push_back("l" + std::to_string(i) + "." + sfx);
        for (const auto& nm : names)
            if (Tensor* t = T(nm)) {
                add_one_kernel<<<grid_for(t->count()), 256, 0, g_stream>>>(reinterpret_cast<float*>(t->data.p), t->count());
                LAUNCHED();
            }
        CK(cudaStreamSynchronize(g_stream));
    }
    // layer scale: the gain of the norm behind a sublayer and the scale behind that norm are one multiplication per coordinate
    for (int i = 0; i < m.d.n_layers; ++i) {
        if (!m.layers[i].d.layer_scale) continue;
        if (!m.gvec) return fail("finalize: layer scale needs norms with one gain per coordinate");
        const std::string p = "l" + std::to_string(i) + ".";
        for (int k = 1; k <= 2; ++k) {
            Tensor* ls = T(p + "ls" + std::to_string(k));
            Tensor* g = T(p + "norm" + std::to_string(k) + (behind ? "" : "b"));
            if (!ls || !g) continue;
            mul_vec_kernel<<<grid_for(g->count()), 256, 0, g_stream>>>(reinterpret_cast<float*>(g->data.p), reinterpret_cast<const float*>(ls->data.p), g->count());
            LAUNCHED();
        }
        CK(cudaStreamSynchronize(g_stream));
    }
    m.final_norm = F("final.norm");
    m.max_k = 2 * D;
    auto note_k = [&](int k) { m.max_k = std::max(m.max_k, k); };
    auto release = [&](const std::string& nm) {
        if (Tensor* t = T(nm)) t->data.release();
    };
    for (int i = 0; i < m.d.n_layers; ++i) {
        LayerW& L = m.layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        if (behind) L.norm1b = F(p + "norm1");   // the only norm of the sublayer sits behind it
        else if (front) L.norm1 = F(p + "norm1");
        else { L.norm1 = F(p + "norm1"); L.norm1b = F(p + "norm1b"); }
        if (L.d.conv_taps >= 1) { L.canon = F(p + "canon1"); m.any_conv = true; }
        if (L.d.conv_ff && L.d.ff > 0) L.canon2 = F(p + "canon2");
        for (int q = 0; q < 2 && front; ++q) {
            if (q == 1 && L.d.ff <= 0) break;
            const std::string hc = p + "hc" + std::to_string(q + 1) + ".";
            L.hc_in[q] = m.d.streams > 0 ? F(hc + "in") : m.ones.p;
            L.hc_out[q] = m.d.streams > 0 ? F(hc + "out") : m.ones.p;
            L.hc_mix[q] = m.d.streams > 0 ? F(hc + "mix") : m.ones.p;
        }
        if (L.d.sink == TI_SEQ_SINK_ZERO) {
            TRY(L.sink_zero.alloc((size_t)L.d.heads));
            CK(cudaMemset(L.sink_zero.p, 0, (size_t)L.d.heads * sizeof(float)));
            L.sink = L.sink_zero.p;
        }
        bool rg1_fused = false, rg2_fused = false;
        if (L.d.mixer == TI_SEQ_MIXER_ATTENTION) {
            TRY(concat_rows(m, {T(p + "mix.q"), T(p + "mix.k"), T(p + "mix.v"), L.d.out_gate ? T(p + "mix.g") : nullptr}, L.qkvg_buf, &L.n_qkvg));
            L.qkvg = L.qkvg_buf.p;
            for (const char* s : {"mix.q", "mix.k", "mix.v", "mix.g"}) release(p + s);
            L.o = P(p + "mix.o");
            const std::vector<float> f = rotary_frequencies(L.d);
            TRY(L.inv_freq.alloc(std::max<size_t>(1, f.size())));
            if (!f.empty()) CK(cudaMemcpy(L.inv_freq.p, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice));
            m.max_proj = std::max(m.max_proj, L.n_qkvg);
            m.max_att = std::max(m.max_att, L.d.heads * L.d.vdim);
            m.max_heads_v = std::max(m.max_heads_v, L.d.heads * (L.d.vdim + 2));
            if (L.d.qk_norm == TI_SEQ_QK_NORM_WHOLE) { L.qnorm = F(p + "mix.q.norm"); L.knorm = F(p + "mix.k.norm"); }
            if (L.d.talk) L.talk = F(p + "mix.talk");
            if (L.d.sink == TI_SEQ_SINK_LEARNED) L.sink = F(p + "mix.sink");
            if (L.d.head_temp) L.temp = F(p + "mix.temp");
            if (L.d.proj_bias) {   // the three biases side by side, as the fused product lays its columns out
                const size_t nq = (size_t)L.d.heads * L.d.dim, nk = (size_t)L.d.kv_heads * L.d.dim, nv = (size_t)L.d.kv_heads * L.d.vdim;
                TRY(L.qkv_bias.alloc(nq + nk + nv));
                CK(cudaMemcpy(L.qkv_bias.p, F(p + "mix.q.b"), nq * sizeof(float), cudaMemcpyDeviceToDevice));
                CK(cudaMemcpy(L.qkv_bias.p + nq, F(p + "mix.k.b"), nk * sizeof(float), cudaMemcpyDeviceToDevice));
                CK(cudaMemcpy(L.qkv_bias.p + nq + nk, F(p + "mix.v.b"), nv * sizeof(float), cudaMemcpyDeviceToDevice));
                L.o_bias = F(p + "mix.o.b");
            }
            if (L.d.talk || L.d.softcap > 0.f || L.d.keep_first > 0) {
                const int H = L.d.heads, d4 = (L.d.dim + 3) / 4 * 4, dv4 = (L.d.vdim + 3) / 4 * 4;
                L.mix_HP = H <= 8 ? 8 : H <= 16 ? 16 : H <= 32 ? 32 : 64;
                (void)dv4;
                if ((size_t)2 * 64 * (d4 + 8) * sizeof(float) > g_smem_optin)
                    return fail("finalize: layer %d: head sizes %d / %d do not fit the head-mixing attention's shared memory", i, L.d.dim, L.d.vdim);
                m.any_mixed = true;
            }
        } else if (L.d.mixer == TI_SEQ_MIXER_WKV) {
            const int C = L.d.heads * L.d.dim;
            L.r = P(p + "mix.r"); L.k = P(p + "mix.k"); L.v = P(p + "mix.v"); L.g = P(p + "mix.g");
            L.w1 = P(p + "mix.w1"); L.w2 = P(p + "mix.w2"); L.o = P(p + "mix.o");
            L.w0 = F(p + "mix.w0"); L.u = F(p + "mix.u"); L.normw = F(p + "mix.norm");
            TRY(L.mu.alloc(5 * (size_t)D));
            int k = 0;
            for (const char* s : {"r", "k", "v", "g", "w"})
                CK(cudaMemcpy(L.mu.p + (size_t)(k++) * D, F(p + "mix.mu." + s), (size_t)D * sizeof(float), cudaMemcpyDeviceToDevice));
            m.max_proj = std::max(m.max_proj, 5 * C);
            m.max_att = std::max(m.max_att, C);
            m.max_rank = std::max(m.max_rank, L.d.decay_rank);
            m.any_wkv = true;
        } else if (L.d.mixer == TI_SEQ_MIXER_GLA || L.d.mixer == TI_SEQ_MIXER_HGRN2) {
            const bool gla = L.d.mixer == TI_SEQ_MIXER_GLA;
            const int C = L.d.heads * L.d.dim, Cv = L.d.heads * L.d.vdim;
            std::vector<int> off;
            TRY(concat_rows(m, {T(p + "mix.q"), T(p + (gla ? "mix.k" : "mix.f")), T(p + "mix.v"), gla ? T(p + "mix.g") : nullptr, gla ? T(p + "mix.a1") : nullptr,
                                L.d.res_gate ? T(p + "rg1") : nullptr}, L.front_buf, &L.n_front, &off));
            L.front = L.front_buf.p;
            L.off_q = off[0]; L.off_k = off[1]; L.off_v = off[2]; L.off_g = off[3]; L.off_a1 = off[4]; L.off_rg1 = off[5];
            rg1_fused = L.d.res_gate != 0;
            for (const char* s : {"mix.q", "mix.k", "mix.f", "mix.v", "mix.g", "mix.a1", "rg1"}) release(p + s);
            if (gla) {
                L.a2 = P(p + "mix.a2");
                L.a2b = F(p + "mix.a2.b");
                note_k(L.d.decay_rank);
                m.max_aux = std::max(m.max_aux, C);
            } else {
                L.fb = F(p + "mix.f.b");
                L.lower = F(p + "mix.lower");
            }
            L.normw = F(p + "mix.norm");
            L.o = P(p + "mix.o");
            L.ld_front = L.n_front;
            m.max_proj = std::max(m.max_proj, L.n_front);
            m.max_att = std::max(m.max_att, Cv);
        } else {   // latent attention
            const int H = L.d.heads, kd = L.d.kv_rank + L.d.rot_dims;
            std::vector<int> off;
            TRY(concat_rows(m, {T(p + (L.d.q_rank > 0 ? "mix.dq" : "mix.q")), L.d.kv_from < 0 ? T(p + "mix.dkv") : nullptr, L.d.res_gate ? T(p + "rg1") : nullptr,
                                L.d.out_gate ? T(p + "mix.g") : nullptr}, L.front_buf, &L.n_front, &off));
            L.front = L.front_buf.p;
            L.off_q = off[0]; L.off_dkv = off[1]; L.off_rg1 = off[2]; L.off_g = off[3];
            L.ld_front = L.n_front;
            if (L.d.q_rank > 0) {   // the queries come from a second product and sit behind the first one's columns
                L.off_dq = off[0];
                L.off_q = L.n_front;
                L.ld_front = L.n_front + H * (L.d.dim + L.d.rot_dims);
                L.uq = P(p + "mix.uq");
                L.dqnorm = F(p + "mix.dq.norm");
                note_k(L.d.q_rank);
                m.max_rank = std::max(m.max_rank, L.d.q_rank);
            }
            rg1_fused = L.d.res_gate != 0;
            for (const char* s : {"mix.q", "mix.dq", "mix.dkv", "rg1", "mix.g"}) release(p + s);
            if (L.d.kv_from < 0) L.cnorm = F(p + "mix.dkv.norm");
            if (L.d.sink == TI_SEQ_SINK_LEARNED) L.sink = F(p + "mix.sink");
            TRY(L.ukT.alloc((size_t)H * L.d.dim * L.d.kv_rank * m.wsize));
            const size_t n = (size_t)H * L.d.dim * L.d.kv_rank;
            if (m.d.mode == TI_SEQ_BF16)
                transpose_heads_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, g_stream>>>((const __nv_bfloat16*)P(p + "mix.uk"), H, L.d.dim, L.d.kv_rank, (__nv_bfloat16*)L.ukT.p);
            else
                transpose_heads_kernel<float><<<grid_for(n), 256, 0, g_stream>>>((const float*)P(p + "mix.uk"), H, L.d.dim, L.d.kv_rank, (float*)L.ukT.p);
            LAUNCHED();
            CK(cudaStreamSynchronize(g_stream));
            release(p + "mix.uk");
            L.uv = P(p + "mix.uv");
            L.o = P(p + "mix.o");
            ti_seq_layer_desc rd = L.d;   // frequencies of the rotated part: every pair of it turns
            rd.rot_scaled = 0;
            const std::vector<float> f = rotary_frequencies(rd);
            TRY(L.inv_freq.alloc(std::max<size_t>(1, f.size())));
            if (!f.empty()) CK(cudaMemcpy(L.inv_freq.p, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice));
            note_k(L.d.dim);
            note_k(L.d.kv_rank);
            m.max_proj = std::max(m.max_proj, L.ld_front);
            m.max_att = std::max(m.max_att, H * L.d.vdim);
            m.max_aux = std::max(m.max_aux, H * kd);
            m.max_aux2 = std::max(m.max_aux2, H * L.d.kv_rank);
            m.max_heads_v = std::max(m.max_heads_v, H * (L.d.kv_rank + 2));
        }
        if (L.d.res_gate) {
            L.rg1b = F(p + "rg1.b");
            if (!rg1_fused) { L.rg1 = P(p + "rg1"); m.any_rgbuf = true; }
        }
        if (L.d.ff > 0) {
            if (behind) L.norm2b = F(p + "norm2");
            else if (front) L.norm2 = F(p + "norm2");
            else { L.norm2 = F(p + "norm2"); L.norm2b = F(p + "norm2b"); }
            if (L.d.ff_kind == TI_SEQ_FF_DENSE) {
                L.ffront = P(p + "mlp.up");
                L.n_ffront = L.d.ff;
                L.off_up = 0;
                L.down = P(p + "mlp.down");
                L.ff_width = L.d.ff;
                if (L.d.ff_act == TI_SEQ_ACT_XIELU) {
                    float a[2];
                    CK(cudaMemcpy(a, F(p + "mlp.act"), sizeof(a), cudaMemcpyDeviceToHost));
                    const auto softplus = [](double z) { return z > 30.0 ? z : std::log1p(std::exp(z)); };
                    L.act_a = (float)softplus(a[0]);
                    L.act_b = (float)(0.5 + softplus(a[1]));
                }
                m.max_proj = std::max(m.max_proj, L.d.ff);
            } else if (L.d.ff_kind == TI_SEQ_FF_GLU) {
                int rows = 0;
                TRY(concat_rows(m, {T(p + "mlp.gate"), T(p + "mlp.up")}, L.gateup_buf, &rows));
                L.gateup = L.gateup_buf.p;
                release(p + "mlp.gate");
                release(p + "mlp.up");
                L.down = P(p + "mlp.down");
                L.ff_width = L.d.ff;
                m.max_proj = std::max(m.max_proj, 2 * L.d.ff);
            } else if (L.d.ff_kind == TI_SEQ_FF_POLYNORM) {
                std::vector<int> off;
                TRY(concat_rows(m, {T(p + "mlp.up"), L.d.res_gate ? T(p + "rg2") : nullptr}, L.ffront_buf, &L.n_ffront, &off));
                L.ffront = L.ffront_buf.p;
                L.off_up = off[0]; L.off_rg2 = off[1];
                rg2_fused = L.d.res_gate != 0;
                release(p + "mlp.up");
                release(p + "rg2");
                L.poly = F(p + "mlp.act");
                L.down = P(p + "mlp.down");
                L.ff_width = L.d.ff;
                m.max_proj = std::max(m.max_proj, L.n_ffront);
            } else {
                const int E = L.d.experts;
                std::vector<const Tensor*> parts{T(p + "mlp.router"), L.d.shared_ff > 0 && !L.d.shared_plain ? T(p + "mlp.shared.sg") : nullptr, L.d.res_gate ? T(p + "rg2") : nullptr};
                std::vector<const Tensor*> downs;
                for (int e = 0; e < E; ++e) {
                    const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                    parts.push_back(T(q + "gate"));
                    parts.push_back(T(q + "up"));
                    downs.push_back(T(q + "down"));
                }
                if (L.d.shared_ff > 0) {
                    parts.push_back(T(p + "mlp.shared.gate"));
                    parts.push_back(T(p + "mlp.shared.up"));
                    downs.push_back(T(p + "mlp.shared.down"));
                }
                std::vector<int> off;
                TRY(concat_rows(m, parts, L.ffront_buf, &L.n_ffront, &off));
                L.ffront = L.ffront_buf.p;
                L.off_router = off[0]; L.off_sg = off[1]; L.off_rg2 = off[2];
                L.off_up = E > 0 ? off[3] : -1;
                L.off_sh = L.d.shared_ff > 0 ? off[3 + 2 * E] : -1;
                rg2_fused = L.d.res_gate != 0;
                L.ff_width = E * L.d.ff + L.d.shared_ff;
                if (L.ff_width > 0) {
                    int cols = 0;
                    TRY(concat_cols(m, downs, L.down_buf, &cols));
                    L.down = L.down_buf.p;
                }
                for (int e = 0; e < E; ++e)
                    for (const char* s : {"gate", "up", "down"}) release(p + "mlp.e" + std::to_string(e) + "." + s);
                for (const char* s : {"mlp.router", "mlp.shared.sg", "mlp.shared.gate", "mlp.shared.up", "mlp.shared.down", "rg2"}) release(p + s);
                if (L.d.route_kind == TI_SEQ_ROUTE_TOP_LOGITS) L.route_bias = F(p + "mlp.router.b");
                else L.correction = F(p + "mlp.correction");
                m.max_proj = std::max(m.max_proj, L.n_ffront);
                m.max_route = std::max(m.max_route, 2 * std::max(E, 1) + 1);   // weights, identity weight, and (few rows) the experts' used flags
            }
            m.max_ff = std::max(m.max_ff, L.ff_width);
            if (L.d.res_gate) {
                L.rg2b = F(p + "rg2.b");
                if (!rg2_fused) { L.rg2 = P(p + "rg2"); m.any_rgbuf = true; }
            }
        }
        if (m.d.side_dim > 0) {
            L.side_gate = P(p + "side.gate");
            L.side_proj = P(p + "side.proj");
            L.side_norm = F(p + "side.norm");
            m.max_aux2 = std::max(m.max_aux2, m.d.side_dim);
            note_k(m.d.side_dim);
        }
    }
    // cache pools and state slots: one of each per layer RUN
    m.num_pages = (m.d.max_tokens + kPageTokens - 1) / kPageTokens;
    for (int p = m.num_pages - 1; p >= 0; --p) m.free_pages.push_back(p);
    m.seqs.resize(m.d.max_seqs);
    for (size_t ri = 0; ri < m.runs.size(); ++ri) {
        Run& R = m.runs[ri];
        const ti_seq_layer_desc& L = m.layers[R.layer].d;
        if (L.mixer == TI_SEQ_MIXER_ATTENTION) {
            TRY(R.k_pool.alloc((size_t)m.num_pages * kPageTokens * L.kv_heads * L.dim));
            TRY(R.v_pool.alloc((size_t)m.num_pages * kPageTokens * L.kv_heads * L.vdim));
        } else if (L.mixer == TI_SEQ_MIXER_LATENT) {
            if (L.kv_from < 0) {
                TRY(R.k_pool.alloc((size_t)m.num_pages * kPageTokens * (L.kv_rank + L.rot_dims)));
            } else {   // the latest earlier run of the layer whose cache this one reads
                for (size_t rj = 0; rj < ri; ++rj)
                    if (m.runs[rj].layer == L.kv_from) R.kv_run = (int)rj;
                if (R.kv_run < 0) return fail("finalize: layer %d reads the cache of layer %d, which has not run before it", R.layer, L.kv_from);
            }
        } else if (L.mixer == TI_SEQ_MIXER_WKV) {
            TRY(R.state.alloc((size_t)m.d.max_seqs * L.heads * L.dim * L.dim));
            TRY(R.prev.alloc((size_t)m.d.max_seqs * D));
            CK(cudaMemset(R.state.p, 0, R.state.n * sizeof(float)));
            CK(cudaMemset(R.prev.p, 0, R.prev.n * sizeof(float)));
        } else {
            TRY(R.state.alloc((size_t)m.d.max_seqs * L.heads * L.dim * L.vdim));
            CK(cudaMemset(R.state.p, 0, R.state.n * sizeof(float)));
        }
        if (L.conv_taps > 1) {
            TRY(R.conv_state.alloc((size_t)m.d.max_seqs * (L.conv_taps - 1) * D));
            CK(cudaMemset(R.conv_state.p, 0, R.conv_state.n * sizeof(float)));
            if (L.conv_ff && L.ff > 0) {
                TRY(R.conv_state2.alloc((size_t)m.d.max_seqs * (L.conv_taps - 1) * D));
                CK(cudaMemset(R.conv_state2.p, 0, R.conv_state2.n * sizeof(float)));
            }
        }
    }
    m.max_k = std::max({m.max_k, 2 * D, m.max_att, m.max_ff, m.max_rank, D});
    TRY(m.err.alloc(1));
    CK(cudaMemset(m.err.p, 0, sizeof(int)));
    CK(cudaEventCreate(&m.ev0));
    CK(cudaEventCreate(&m.ev1));
    m.finalized = true;
    return 0;
}

int ti_seq_model_free(ti_seq_model_t h) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (h == 0 || h > g_models.size() || !g_models[h - 1]) return fail("bad model handle");
    cudaStreamSynchronize(g_stream);
    g_models[h - 1].reset();
    return 0;
}

int ti_seq_open(ti_seq_model_t h, int32_t* seq) {
    Model* m = get_model(h);
    if (!m || !m->finalized) return fail("bad model handle");
    return open_seq(*m, seq);
}
int ti_seq_close(ti_seq_model_t h, int32_t seq) {
    Model* m = get_model(h);
    if (!m || !m->finalized) return fail("bad model handle");
    return close_seq(*m, seq);
}
int ti_seq_length(ti_seq_model_t h, int32_t seq, int32_t* tokens) {
    Model* m = get_model(h);
    if (!m || !m->finalized) return fail("bad model handle");
    if (seq < 0 || seq >= (int)m->seqs.size() || !m->seqs[seq].live) return fail("sequence %d is not open", seq);
    *tokens = m->seqs[seq].len;
    return 0;
}
int ti_seq_pool_info(ti_seq_model_t h, int32_t* free_pages, int32_t* total_pages, int32_t* free_slots, int32_t* page_tokens) {
    Model* m = get_model(h);
    if (!m || !m->finalized) return fail("bad model handle");
    int fs = 0;
    for (const auto& s : m->seqs) fs += !s.live;
    if (free_pages) *free_pages = (int32_t)m->free_pages.size();
    if (total_pages) *total_pages = m->num_pages;
    if (free_slots) *free_slots = fs;
    if (page_tokens) *page_tokens = kPageTokens;
    return 0;
}
int ti_seq_pages(ti_seq_model_t h, int32_t seq, int32_t* pages, int32_t cap, int32_t* n) {
    Model* m = get_model(h);
    if (!m || !m->finalized) return fail("bad model handle");
    if (seq < 0 || seq >= (int)m->seqs.size() || !m->seqs[seq].live) return fail("sequence %d is not open", seq);
    const auto& pg = m->seqs[seq].pages;
    *n = (int32_t)pg.size();
    for (int i = 0; i < (int)pg.size() && i < cap; ++i) pages[i] = pg[i];
    return 0;
}

int ti_seq_step(ti_seq_model_t h, int32_t n_entries, const int32_t* seqs, const int32_t* counts, const int32_t* tokens, int32_t n_want,
                const int32_t* want_rows, float* logits_host) {
    Model* m = get_model(h);
    if (!m) return fail("bad model handle");
    return run_step(*m, n_entries, seqs, counts, tokens, n_want, want_rows, logits_host, SampleSpec{});
}

int ti_seq_step_sample(ti_seq_model_t h, int32_t n_entries, const int32_t* seqs, const int32_t* counts, const int32_t* tokens, float temperature,
                       int32_t top_k, float top_p, uint64_t seed, const int32_t* sample_index, int32_t* out_tokens, float* out_logprobs) {
    Model* m = get_model(h);
    if (!m) return fail("bad model handle");
    if (!out_tokens) return fail("step_sample: out_tokens is null");
    SampleSpec s;
    s.on = true; s.temperature = temperature; s.top_k = top_k; s.top_p = top_p; s.seed = seed; s.index = sample_index;
    s.out_tokens = out_tokens; s.out_logprobs = out_logprobs;
    return run_step(*m, n_entries, seqs, counts, tokens, 0, nullptr, nullptr, s);
}

// The generation loop: continuous batching over the step above.  Waiting requests are admitted in order while a state slot is
// free and the pool has pages for the whole request (prompt + max_new, so that a running request never stalls); a step takes
// one decode token from every running request whose prompt is done, then prompt portions (oldest first) until `step_tokens`
// rows are filled.
int ti_seq_generate(ti_seq_model_t h, int32_t n_req, const int32_t* prompts, const int32_t* lens, int32_t max_new, int32_t step_tokens,
                    float temperature, int32_t top_k, float top_p, uint64_t seed, int32_t eos, int32_t* out_tokens, int32_t* out_lens) {
    Model* mp = get_model(h);
    if (!mp || !mp->finalized) return fail("bad model handle");
    Model& m = *mp;
    if (n_req <= 0 || max_new <= 0) return fail("generate: n_req %d max_new %d", n_req, max_new);
    if (step_tokens <= 0) step_tokens = 512;
    struct Req { int id, seq, fed, n_out, last, reserved; const int32_t* prompt; int len; };
    std::vector<size_t> start(n_req + 1, 0);
    for (int i = 0; i < n_req; ++i) {
        if (lens[i] <= 0) return fail("generate: request %d has an empty prompt", i);
        start[i + 1] = start[i] + lens[i];
    }
    const auto pages_for = [](int tokens) { return (tokens + kPageTokens - 1) / kPageTokens; };
    for (int i = 0; i < n_req; ++i)
        if (pages_for(lens[i] + max_new) > m.num_pages) return fail("generate: request %d (%d + %d tokens) exceeds the page pool", i, lens[i], max_new);
    std::vector<Req> running;
    int next = 0, done = 0, reserved_pages = 0;
    for (int i = 0; i < n_req; ++i) out_lens[i] = 0;
    std::vector<int32_t> seqs, counts, toks, sidx, picks;
    while (done < n_req) {
        // admission
        while (next < n_req) {
            const int need = pages_for(lens[next] + max_new);
            int live_pages = 0;
            for (const auto& s : m.seqs) live_pages += s.live ? (int)s.pages.size() : 0;
            (void)live_pages;
            if (reserved_pages + need > m.num_pages) break;
            int32_t s = -1;
            if (open_seq(m, &s) != 0) break;
            running.push_back(Req{next, s, 0, 0, 0, need, prompts + start[next], lens[next]});
            reserved_pages += need;
            ++next;
        }
        if (running.empty()) return fail("generate: nothing can be admitted");
        seqs.clear(); counts.clear(); toks.clear(); sidx.clear();
        int budget = step_tokens;
        std::vector<int> in_step;
        for (size_t i = 0; i < running.size(); ++i)   // decode tokens first
            if (running[i].fed == running[i].len && budget > 0) {
                seqs.push_back(running[i].seq); counts.push_back(1); toks.push_back(running[i].last); sidx.push_back(running[i].n_out);
                in_step.push_back((int)i);
                --budget;
            }
        for (size_t i = 0; i < running.size() && budget > 0; ++i)
            if (running[i].fed < running[i].len) {
                const int c = std::min(budget, running[i].len - running[i].fed);
                seqs.push_back(running[i].seq); counts.push_back(c); sidx.push_back(0);
                toks.insert(toks.end(), running[i].prompt + running[i].fed, running[i].prompt + running[i].fed + c);
                in_step.push_back((int)i);
                budget -= c;
            }
        picks.resize(seqs.size());
        SampleSpec s;
        s.on = true; s.temperature = temperature; s.top_k = top_k; s.top_p = top_p; s.seed = seed; s.index = sidx.data(); s.out_tokens = picks.data();
        TRY(run_step(m, (int)seqs.size(), seqs.data(), counts.data(), toks.data(), 0, nullptr, nullptr, s));
        std::vector<size_t> finished;
        for (size_t k = 0; k < in_step.size(); ++k) {
            Req& r = running[in_step[k]];
            const bool was_decode = r.fed == r.len;
            if (!was_decode) r.fed += counts[k];
            if (r.fed < r.len) continue;   // the pick behind an unfinished prompt portion is not used
            r.last = picks[k];
            out_tokens[(size_t)r.id * max_new + r.n_out] = picks[k];
            ++r.n_out;
            out_lens[r.id] = r.n_out;
            if (r.n_out >= max_new || (eos >= 0 && picks[k] == eos)) finished.push_back(in_step[k]);
        }
        std::sort(finished.rbegin(), finished.rend());
        for (size_t i : finished) {
            TRY(close_seq(m, running[i].seq));
            reserved_pages -= running[i].reserved;
            running.erase(running.begin() + i);
            ++done;
        }
    }
    return 0;
}

int ti_seq_debug_layers(ti_seq_model_t h, int32_t enable) {
    Model* m = get_model(h);
    if (!m) return fail("bad model handle");
    m->dbg = enable != 0;
    m->cap_rows = 0;   // scratch is laid out again on the next step
    return 0;
}
int ti_seq_debug_layers_read(ti_seq_model_t h, float* out, size_t cap_floats, int32_t* runs, int32_t* rows) {
    Model* m = get_model(h);
    if (!m || !m->dbg || !m->dbg_buf.p) return fail("debug layers are not enabled");
    const size_t n = m->runs.size() * (size_t)m->dbg_rows * m->d.width;
    if (n > cap_floats) return fail("debug buffer too small: %zu floats needed", n);
    CK(cudaMemcpy(out, m->dbg_buf.p, n * sizeof(float), cudaMemcpyDeviceToHost));
    *runs = (int32_t)m->runs.size();
    *rows = m->dbg_rows;
    return 0;
}
int ti_seq_flush_l2(void) {
    static DevBuf<uint8_t> buf;
    const size_t bytes = (size_t)256 << 20;
    if (g_device < 0) return fail("ti_seq: not initialised");
    TRY(buf.ensure(bytes));
    CK(cudaMemsetAsync(buf.p, 1, bytes, g_stream));
    CK(cudaStreamSynchronize(g_stream));
    return 0;
}
int ti_seq_last_step_ms(ti_seq_model_t h, float* ms) {
    Model* m = get_model(h);
    if (!m) return fail("bad model handle");
    *ms = m->last_ms;
    return 0;
}
int ti_seq_model_bytes(ti_seq_model_t h, double* weight_bytes, double* kv_bytes_per_token, double* state_bytes_per_seq) {
    Model* m = get_model(h);
    if (!m || !m->finalized) return fail("bad model handle");
    double w = 0, kv = 0, st = 0;
    const double D = m->d.width, ws = (double)m->wsize;
    if (m->d.loop_times > 0 && !m->d.loop_plain) w += 2 * D * D * ws * m->d.loop_times;
    for (const Run& R : m->runs) {
        const ti_seq_layer_desc& L = m->layers[R.layer].d;
        if (L.mixer == TI_SEQ_MIXER_ATTENTION) {
            w += ((double)L.heads * L.dim + (double)L.kv_heads * (L.dim + L.vdim) + (L.out_gate ? L.heads : 0) + (double)L.heads * L.vdim) * D * ws;
            kv += (double)L.kv_heads * (L.dim + L.vdim) * 4;
        } else if (L.mixer == TI_SEQ_MIXER_WKV) {
            const double C = (double)L.heads * L.dim;
            w += (5 * C * D + (double)L.decay_rank * (D + C)) * ws;
            st += ((double)L.heads * L.dim * L.dim + D) * 4;
        } else if (L.mixer == TI_SEQ_MIXER_GLA || L.mixer == TI_SEQ_MIXER_HGRN2) {
            const double C = (double)L.heads * L.dim, Cv = (double)L.heads * L.vdim;
            w += (2 * C * D + 2 * Cv * D) * ws;   // q, k or f, v, o
            if (L.mixer == TI_SEQ_MIXER_GLA) w += (Cv * D + (double)L.decay_rank * (D + C)) * ws;
            st += (double)L.heads * L.dim * L.vdim * 4;
        } else {
            const double H = L.heads;
            w += (H * (L.dim + L.vdim) * L.kv_rank + H * L.vdim * D + (L.out_gate ? H * D : 0.0)) * ws;
            w += (L.q_rank > 0 ? (double)L.q_rank * (D + H * (L.dim + L.rot_dims)) : H * (L.dim + L.rot_dims) * D) * ws;
            if (L.kv_from < 0) {
                w += (double)(L.kv_rank + L.rot_dims) * D * ws;
                kv += (double)(L.kv_rank + L.rot_dims) * 4;
            }
        }
        if (L.conv_taps > 1) st += (double)(L.conv_taps - 1) * D * 4 * (L.conv_ff && L.ff > 0 ? 2 : 1);
        if (L.res_gate) w += (L.ff > 0 ? 2.0 : 1.0) * D * D * ws;
        if (L.ff > 0) {
            // routed experts: the stacked products read every expert's weights whatever the tokens chose
            if (L.ff_kind == TI_SEQ_FF_GLU) w += 3.0 * L.ff * D * ws;
            else if (L.ff_kind == TI_SEQ_FF_POLYNORM || L.ff_kind == TI_SEQ_FF_DENSE) w += 2.0 * L.ff * D * ws;
            else w += (3.0 * ((double)L.experts * L.ff + L.shared_ff) + L.experts + L.identity + (L.shared_ff > 0 && !L.shared_plain ? 1 : 0)) * D * ws;
        }
        if (m->d.side_dim > 0) w += 2.0 * m->d.side_dim * D * ws;
    }
    w += (double)m->d.vocab * D * ws;   // the head (the embedding table itself when the two are tied)
    if (weight_bytes) *weight_bytes = w;
    if (kv_bytes_per_token) *kv_bytes_per_token = kv;
    if (state_bytes_per_seq) *state_bytes_per_seq = st;
    return 0;
}

}  // extern "C"

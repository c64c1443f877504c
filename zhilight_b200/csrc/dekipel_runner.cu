// Host-side driver of the Dekipel model family: weights, slot caches and states, the per-step kernel chain and its
// CUDA graph.  Same driver shape as llama_runner.cu (task slots, host tokens in, logits / greedy picks out), built
// from the shared pieces of runner_common.cuh.
//
// A layer: x += norm1b(mixer(conv1(norm1(x)))), x += norm2b(ff(conv2(norm2(x)))) with x in fp32, every norm an RMS
// norm in groups, conv = the input plus a short causal convolution of it over the positions of the sequence.
// The mixer is latent attention (latent_attn.cu): q = W_uq rms(W_dq u), c = rms(W_dkv u) cached per position (or
// another layer's cache), absorbed attention with a sink, heads gated by sigmoid(W_g u), W_o.  The feed-forward is
// W_down relu(W_up u)^2.  One step takes T rows (token, slot, position) in any mix of prompt portions and single
// decode tokens; the kernels index caches and convolution rings by (slot, position), so the same chain serves both.
#include "runner_common.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace {

using namespace zl;

struct DLayer {
    zl_dekipel_layer_t c{};
    float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr;
    float *canon1 = nullptr, *canon2 = nullptr, *dq_norm = nullptr, *dkv_norm = nullptr, *sink = nullptr;
    void* w_in = nullptr;   // rows: W_dq (q_rank) | W_dkv (kv_rank, own latents only) | W_g (heads * vdim); (n_in, width)
    int n_in = 0, c_off = 0, g_off = 0;
    void* uq = nullptr;     // (heads * dim, q_rank)
    void* uk_t = nullptr;   // (heads, kv_rank, dim): W_uk of each head transposed, so that the absorption is an NT GEMM
    void* uv = nullptr;     // (heads * vdim, kv_rank)
    void* o = nullptr;      // (width, heads * vdim)
    void *up = nullptr, *down = nullptr;
    SlotCache latents;      // own latents: (slots, max_seq, kv_rank) in the activation dtype
    void** lat_addrs = nullptr;   // this layer's or its source layer's table
    SlotCache ring1, ring2;       // convolution inputs: (slots, taps - 1, width) fp32
    bool ready = false;
};

}  // namespace

struct zl_dekipel {
    zl_dekipel_config_t cfg{};
    cudaStream_t stream = nullptr;
    StagedMap staged;
    std::vector<DLayer> layers;
    void *embed = nullptr, *head = nullptr;
    float* final_norm = nullptr;
    bool finalized = false;
    int esz = 2;   // bytes of an activation / weight element
    int tcap = 0;
    float *x = nullptr, *hbuf = nullptr, *proj = nullptr, *qa = nullptr, *y = nullptr, *xw = nullptr, *logits = nullptr;
    void *ubuf = nullptr, *cq = nullptr, *q = nullptr, *olat = nullptr, *og = nullptr, *act = nullptr, *xn = nullptr;
    int32_t *d_tokens = nullptr, *d_slots = nullptr, *d_pos = nullptr, *d_want = nullptr, *d_next = nullptr;
    int32_t* h_stage = nullptr;   // pinned: tokens | slots | pos | want | next
    void* attn_ws = nullptr;
    size_t attn_ws_bytes = 0;
    void* argmax_ws = nullptr;
    float* layer_dump = nullptr;   // (num_layers, tcap, width) when capture is on
    bool capture = false;
    std::map<long long, cudaGraphExec_t> graphs;
    int cur_max_len = 0;   // device-resident decode loop: host-side bound of positions + 1
    double weight_bytes = 0;
    int kernels_per_step = 0;
};

namespace {

constexpr int kDefaultPdlMask = 1;

int fail(int line, const std::string& msg, int code = ZL_ERR_STATE) {
    zl_set_last_error(__FILE__, line, msg.c_str());
    return code;
}

// src (heads * dim, R) -> dst (heads, R, dim)
template <typename TS, typename TD>
__global__ void k_convert_head_transpose(const TS* __restrict__ src, TD* __restrict__ dst, int heads, int dim, int R) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)heads * dim * R) return;
    const int d = (int)(i % dim), r = (int)((i / dim) % R), h = (int)(i / ((size_t)dim * R));
    dst[i] = from_f32<TD>(to_f32<TS>(src[((size_t)h * dim + d) * R + r]));
}
int finalize_layer(zl_dekipel* m, int l) {
    const auto& c = m->cfg;
    DLayer& L = m->layers[l];
    const auto& lc = L.c;
    const std::string p = "l" + std::to_string(l) + ".";
    const int D = c.width, H = lc.heads, R = lc.kv_rank, own = lc.kv_from < 0;
    RCHECK(take_f32(m, p + "norm1", 1, D, &L.norm1));
    RCHECK(take_f32(m, p + "norm1b", 1, D, &L.norm1b));
    RCHECK(take_f32(m, p + "canon1", D, c.canon_taps, &L.canon1));
    RCHECK(take_f32(m, p + "mix.dq.norm", 1, lc.q_rank, &L.dq_norm));
    RCHECK(take_f32(m, p + "mix.sink", 1, H, &L.sink));
    L.c_off = lc.q_rank;
    L.g_off = lc.q_rank + (own ? R : 0);
    L.n_in = L.g_off + H * lc.vdim;
    RCHECK(dmalloc(&L.w_in, (size_t)L.n_in * D * m->esz));
    RCHECK(put_weight(m, p + "mix.dq", lc.q_rank, D, L.w_in, 0));
    if (own) {
        RCHECK(put_weight(m, p + "mix.dkv", R, D, L.w_in, (size_t)L.c_off * D));
        RCHECK(take_f32(m, p + "mix.dkv.norm", 1, R, &L.dkv_norm));
    }
    RCHECK(put_weight(m, p + "mix.g", H * lc.vdim, D, L.w_in, (size_t)L.g_off * D));
    RCHECK(take_weight(m, p + "mix.uq", H * lc.dim, lc.q_rank, &L.uq));
    {
        const Staged* s = need(m, p + "mix.uk", H * lc.dim, R);
        if (!s) return ZL_ERR_STATE;
        const size_t n = (size_t)H * lc.dim * R;
        RCHECK(dmalloc(&L.uk_t, n * m->esz));
        const unsigned blocks = (unsigned)((n + 255) / 256);
        if (c.dtype == ZL_F32) {
            if (s->elem == 2)
                k_convert_head_transpose<<<blocks, 256, 0, m->stream>>>(static_cast<const __nv_bfloat16*>(s->ptr),
                                                                         static_cast<float*>(L.uk_t), H, lc.dim, R);
            else
                k_convert_head_transpose<<<blocks, 256, 0, m->stream>>>(static_cast<const float*>(s->ptr),
                                                                         static_cast<float*>(L.uk_t), H, lc.dim, R);
        } else {
            if (s->elem == 2)
                k_convert_head_transpose<<<blocks, 256, 0, m->stream>>>(static_cast<const __nv_bfloat16*>(s->ptr),
                                                                         static_cast<__nv_bfloat16*>(L.uk_t), H, lc.dim, R);
            else
                k_convert_head_transpose<<<blocks, 256, 0, m->stream>>>(static_cast<const float*>(s->ptr),
                                                                         static_cast<__nv_bfloat16*>(L.uk_t), H, lc.dim, R);
        }
        ZL_CHECK_LAUNCH();
        ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
        staged_drop(m->staged, p + "mix.uk");
        m->weight_bytes += (double)n * m->esz;
    }
    RCHECK(take_weight(m, p + "mix.uv", H * lc.vdim, R, &L.uv));
    RCHECK(take_weight(m, p + "mix.o", D, H * lc.vdim, &L.o));
    if (lc.ff > 0) {
        RCHECK(take_f32(m, p + "norm2", 1, D, &L.norm2));
        RCHECK(take_f32(m, p + "norm2b", 1, D, &L.norm2b));
        RCHECK(take_f32(m, p + "canon2", D, c.canon_taps, &L.canon2));
        RCHECK(take_weight(m, p + "mlp.up", lc.ff, D, &L.up));
        RCHECK(take_weight(m, p + "mlp.down", D, lc.ff, &L.down));
    }
    L.ready = true;
    return ZL_OK;
}

// attention split counts are baked into a graph: one graph per length bucket
int len_bucket(const zl_dekipel* m, int max_len) {
    int b = 256;
    while (b < max_len) b <<= 1;
    return b < m->cfg.max_seq ? b : (m->cfg.max_seq > 256 ? m->cfg.max_seq : 256);
}

int alloc_runtime(zl_dekipel* m) {
    const auto& c = m->cfg;
    const int D = c.width, T = m->tcap, B = c.max_batch, keep = c.canon_taps - 1;
    size_t n_in = 0, qr = 0, hd = 0, hr = 0, hv = 0, ff = 0;
    for (auto& L : m->layers) {
        const auto& lc = L.c;
        if (lc.kv_from < 0) {
            RCHECK(L.latents.create(B, (size_t)c.max_seq * lc.kv_rank * m->esz, m->stream));
            L.lat_addrs = L.latents.addrs;
        }
        if (keep > 0) {
            RCHECK(L.ring1.create(B, (size_t)keep * D * 4, m->stream));
            if (lc.ff > 0) RCHECK(L.ring2.create(B, (size_t)keep * D * 4, m->stream));
        }
        RCHECK(zl_latent_attention_prepare(lc.heads, lc.kv_rank, c.dtype));
        n_in = std::max(n_in, (size_t)L.n_in);
        qr = std::max(qr, (size_t)lc.q_rank);
        hd = std::max(hd, (size_t)lc.heads * lc.dim);
        hr = std::max(hr, (size_t)lc.heads * lc.kv_rank);
        hv = std::max(hv, (size_t)lc.heads * lc.vdim);
        ff = std::max(ff, (size_t)lc.ff);
        for (int b = 1; b <= T; ++b) {   // the split count falls as the rows grow: size for the worst product
            const int s = zl_latent_attention_splits(b, lc.heads, lc.kv_rank, len_bucket(m, c.max_seq));
            m->attn_ws_bytes = std::max(m->attn_ws_bytes, zl_latent_attention_workspace_bytes(b, lc.heads, lc.kv_rank, s));
            if (s == 1) break;
        }
    }
    for (auto& L : m->layers)
        if (L.c.kv_from >= 0) L.lat_addrs = m->layers[L.c.kv_from].latents.addrs;
    const size_t e = m->esz;
    RCHECK(dmalloc((void**)&m->x, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->hbuf, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->y, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->proj, (size_t)T * n_in * 4));
    RCHECK(dmalloc((void**)&m->qa, (size_t)T * hr * 4));
    RCHECK(dmalloc((void**)&m->xw, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->logits, (size_t)T * c.vocab * 4));
    RCHECK(dmalloc(&m->ubuf, (size_t)T * D * e));
    RCHECK(dmalloc(&m->cq, (size_t)T * qr * e));
    RCHECK(dmalloc(&m->q, (size_t)T * hd * e));
    RCHECK(dmalloc(&m->olat, (size_t)T * hr * e));
    RCHECK(dmalloc(&m->og, (size_t)T * hv * e));
    RCHECK(dmalloc(&m->act, (size_t)T * (ff ? ff : 1) * e));
    RCHECK(dmalloc(&m->xn, (size_t)T * D * e));
    RCHECK(dmalloc((void**)&m->d_tokens, (size_t)T * 4));
    RCHECK(dmalloc((void**)&m->d_slots, (size_t)T * 4));
    RCHECK(dmalloc((void**)&m->d_pos, (size_t)T * 4));
    RCHECK(dmalloc((void**)&m->d_want, (size_t)T * 4));
    RCHECK(dmalloc((void**)&m->d_next, (size_t)T * 4));
    RCHECK(dmalloc(&m->attn_ws, m->attn_ws_bytes));
    RCHECK(dmalloc(&m->argmax_ws, zl_argmax_workspace_bytes(T)));
    ZL_CHECK_CUDA(cudaMallocHost((void**)&m->h_stage, sizeof(int32_t) * 5 * (size_t)T));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

// Which kernels of the step are launched with a programmatic dependency (they may start while their predecessor drains
// and wait inside): 1 skinny Linears, 2 tiled / per-head GEMMs, 4 norm / convolution / residual rows, 8 attention,
// 16 the tail (gather, final norm, head, pick).  Measured on B200 (1 and 32 rows, two layer sizes): only the skinny
// Linears of steps with few rows gain (their first weight loads fly before the wait); early-started CTAs of the row
// kernels and GEMMs take SM slots from the kernel they wait for and cost up to 50 % of a 32-row step.
// ZL_DEKIPEL_PDL_MASK overrides the default.
int pdl_mask() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("ZL_DEKIPEL_PDL_MASK");
        v = e ? atoi(e) : kDefaultPdlMask;
    }
    return v;
}
int pdl_for(const zl_dekipel* m, int bit) { return (m->cfg.use_pdl && (pdl_mask() & bit)) ? 1 : 0; }

// y (M, N) = x (M, K) @ w (N, K)^T.  Decode-sized 16-bit products whose K suits it stream the weights once through the
// framework's skinny kernel; everything else goes through the tiled kernel.
int linear(zl_dekipel* m, const void* x, int K, const void* w, int N, void* y, int M, int out_dtype, int epi) {
    const auto& c = m->cfg;
    static const bool no_skinny = getenv("ZL_DEKIPEL_NO_SKINNY") != nullptr;
    if (!no_skinny && c.dtype != ZL_F32 && epi != ZL_GEMM_EPI_SIGMOID_GATE && M <= 32 && K % 32 == 0 && N >= 64 &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0)
        return zl_dense_gemm_skinny_act(x, K, w, nullptr, y, M, N, K, c.dtype, out_dtype, epi == ZL_GEMM_EPI_RELU2 ? 1 : 0,
                                        M <= 8 ? pdl_for(m, 1) : 0, m->stream);
    return zl_gemm_nt(x, K, 0, w, K, 0, y, N, 0, M, N, K, 1, c.dtype, out_dtype, epi, nullptr, 0, 0, pdl_for(m, 2), m->stream);
}

int enqueue_step(zl_dekipel* m, int T, int n_want, int max_len) {
    const auto& c = m->cfg;
    const int D = c.width, dt = c.dtype, G = c.norm_groups, taps = c.canon_taps;
    const int pdl_gemm = pdl_for(m, 2), pdl_row = pdl_for(m, 4), pdl_attn = pdl_for(m, 8), pdl_tail = pdl_for(m, 16);
    cudaStream_t st = m->stream;
    // ZL_DEKIPEL_UNFUSED=1: one kernel per operator (pre-norm and convolution apart), for A/B and bring-up
    static const bool fuse = getenv("ZL_DEKIPEL_UNFUSED") == nullptr;
    if (dt == ZL_F32)
        ZL_CHECK_CUDA(launch(k_embed_f32<float>, dim3(T), dim3(128), 0, st, false, (const int32_t*)m->d_tokens,
                             (const float*)m->embed, m->x, D, c.vocab, 1.0f));
    else
        ZL_CHECK_CUDA(launch(k_embed_f32<__nv_bfloat16>, dim3(T), dim3(128), 0, st, false, (const int32_t*)m->d_tokens,
                             (const __nv_bfloat16*)m->embed, m->x, D, c.vocab, 1.0f));
    for (int l = 0; l < c.num_layers; ++l) {
        DLayer& L = m->layers[l];
        const auto& lc = L.c;
        const int H = lc.heads, R = lc.kv_rank, own = lc.kv_from < 0;
        // mixer sublayer
        if (fuse) {
            RCHECK(zl_group_norm_conv(m->x, D, L.norm1, L.canon1, m->d_slots, m->d_pos, (const float*)L.ring1.buf, m->hbuf, m->ubuf,
                                      T, D, G, taps, c.eps, dt, pdl_row, st));
        } else {
            RCHECK(zl_group_rmsnorm(m->x, D, L.norm1, m->hbuf, D, T, D, G, c.eps, ZL_F32, pdl_row, st));
            RCHECK(zl_causal_conv_mix(m->hbuf, D, L.canon1, m->d_slots, m->d_pos, (const float*)L.ring1.buf, m->ubuf, D, T, D,
                                      taps, dt, pdl_row, st));
        }
        RCHECK(linear(m, m->ubuf, D, L.w_in, L.n_in, m->proj, T, ZL_F32, ZL_GEMM_EPI_NONE));
        RCHECK(zl_latent_norm_append(m->proj, L.n_in, 0, lc.q_rank, L.dq_norm, m->cq, L.c_off, R, own ? L.dkv_norm : nullptr,
                                     L.lat_addrs, m->d_slots, m->d_pos, T, c.eps, dt, pdl_row, st));
        RCHECK(linear(m, m->cq, lc.q_rank, L.uq, H * lc.dim, m->q, T, dt, ZL_GEMM_EPI_NONE));
        RCHECK(zl_gemm_nt(m->q, (long long)H * lc.dim, lc.dim, L.uk_t, lc.dim, (long long)R * lc.dim, m->qa, (long long)H * R, R,
                          T, R, lc.dim, H, dt, ZL_F32, ZL_GEMM_EPI_NONE, nullptr, 0, 0, pdl_gemm, st));
        const int splits = zl_latent_attention_splits(T, H, R, max_len);
        RCHECK(zl_latent_attention(m->qa, L.lat_addrs, m->d_slots, m->d_pos, L.sink, lc.scale, m->olat, T, H, R, splits,
                                   m->attn_ws, m->attn_ws_bytes, dt, pdl_attn, st));
        RCHECK(zl_gemm_nt(m->olat, (long long)H * R, R, L.uv, R, (long long)lc.vdim * R, m->og, (long long)H * lc.vdim, lc.vdim, T,
                          lc.vdim, R, H, dt, dt, ZL_GEMM_EPI_SIGMOID_GATE, m->proj + L.g_off, L.n_in, lc.vdim, pdl_gemm, st));
        RCHECK(linear(m, m->og, H * lc.vdim, L.o, D, m->y, T, ZL_F32, ZL_GEMM_EPI_NONE));
        RCHECK(zl_group_rmsnorm_residual(m->y, D, L.norm1b, m->x, D, T, D, G, c.eps, m->hbuf, D, m->d_slots, m->d_pos,
                                         (float*)L.ring1.buf, taps, pdl_row, st));
        if (lc.ff > 0) {
            if (fuse) {
                RCHECK(zl_group_norm_conv(m->x, D, L.norm2, L.canon2, m->d_slots, m->d_pos, (const float*)L.ring2.buf, m->hbuf,
                                          m->ubuf, T, D, G, taps, c.eps, dt, pdl_row, st));
            } else {
                RCHECK(zl_group_rmsnorm(m->x, D, L.norm2, m->hbuf, D, T, D, G, c.eps, ZL_F32, pdl_row, st));
                RCHECK(zl_causal_conv_mix(m->hbuf, D, L.canon2, m->d_slots, m->d_pos, (const float*)L.ring2.buf, m->ubuf, D, T, D,
                                          taps, dt, pdl_row, st));
            }
            RCHECK(linear(m, m->ubuf, D, L.up, lc.ff, m->act, T, dt, ZL_GEMM_EPI_RELU2));
            RCHECK(linear(m, m->act, lc.ff, L.down, D, m->y, T, ZL_F32, ZL_GEMM_EPI_NONE));
            RCHECK(zl_group_rmsnorm_residual(m->y, D, L.norm2b, m->x, D, T, D, G, c.eps, m->hbuf, D, m->d_slots, m->d_pos,
                                             (float*)L.ring2.buf, taps, pdl_row, st));
        }
        if (m->capture && m->layer_dump)
            ZL_CHECK_CUDA(cudaMemcpyAsync(m->layer_dump + (size_t)l * m->tcap * D, m->x, (size_t)T * D * 4,
                                          cudaMemcpyDeviceToDevice, st));
    }
    if (n_want > 0) {
        ZL_CHECK_CUDA(launch(k_gather_rows_f32, dim3(n_want), dim3(128), 0, st, false, (const float*)m->x,
                             (const int32_t*)m->d_want, m->xw, D));
        RCHECK(zl_group_rmsnorm(m->xw, D, m->final_norm, m->xn, D, n_want, D, G, c.eps, dt, pdl_tail, st));
        RCHECK(linear(m, m->xn, D, m->head, c.vocab, m->logits, n_want, ZL_F32, ZL_GEMM_EPI_NONE));
        RCHECK(zl_argmax(m->logits, m->d_next, n_want, c.vocab, m->argmax_ws, zl_argmax_workspace_bytes(n_want), pdl_tail, st));
    }
    return ZL_OK;
}

// decode-sized steps replay a CUDA graph per (rows, wanted rows, length bucket); prompt portions are enqueued directly
int run_step(zl_dekipel* m, int T, int n_want, int max_len) {
    const int bucket = len_bucket(m, max_len);
    if (!m->cfg.use_graph || T > m->cfg.max_batch || m->capture) return enqueue_step(m, T, n_want, bucket);
    const long long key = ((long long)T << 40) | ((long long)n_want << 24) | (long long)(bucket >> 8);
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        cudaGraph_t graph = nullptr;
        ZL_CHECK_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_step(m, T, n_want, bucket);
        const cudaError_t ce = cudaStreamEndCapture(m->stream, &graph);
        if (rc != ZL_OK) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        ZL_CHECK_CUDA(ce);
        cudaGraphExec_t exec = nullptr;
        ZL_CHECK_CUDA(cudaGraphInstantiate(&exec, graph, 0));
        size_t n_nodes = 0;
        cudaGraphGetNodes(graph, nullptr, &n_nodes);
        m->kernels_per_step = (int)n_nodes;
        cudaGraphDestroy(graph);
        it = m->graphs.emplace(key, exec).first;
    }
    ZL_CHECK_CUDA(cudaGraphLaunch(it->second, m->stream));
    return ZL_OK;
}

}  // namespace

extern "C" int zl_dekipel_create(const zl_dekipel_config_t* cfg, const zl_dekipel_layer_t* layers, zl_dekipel_t** out) {
    ZL_CHECK_ARG(cfg && layers && out);
    ZL_CHECK_ARG(cfg->num_layers > 0 && cfg->width > 0 && cfg->vocab > 0 && cfg->max_batch > 0 && cfg->max_seq > 0);
    ZL_CHECK_ARG(cfg->norm_groups > 0 && cfg->width % cfg->norm_groups == 0 && cfg->canon_taps >= 1 && cfg->eps >= 0.f);
    ZL_CHECK_SUPPORTED(cfg->dtype == ZL_BF16 || cfg->dtype == ZL_F32);
    ZL_CHECK_ARG(cfg->max_step_tokens >= 0 && cfg->max_step_tokens <= 65535);
    for (int l = 0; l < cfg->num_layers; ++l) {
        const auto& lc = layers[l];
        ZL_CHECK_ARG(lc.heads > 0 && lc.dim > 0 && lc.vdim > 0 && lc.q_rank > 0 && lc.kv_rank > 0 && lc.ff >= 0);
        if (lc.kv_from >= 0) {
            // the source layer runs earlier in the step, owns its latents, and has the same latent size
            ZL_CHECK_ARG(lc.kv_from < l && layers[lc.kv_from].kv_from < 0 && layers[lc.kv_from].kv_rank == lc.kv_rank);
        }
    }
    zl_dekipel* m = new zl_dekipel();
    m->cfg = *cfg;
    m->esz = cfg->dtype == ZL_F32 ? 4 : 2;
    m->tcap = cfg->max_step_tokens > cfg->max_batch ? cfg->max_step_tokens : cfg->max_batch;
    m->layers.resize(cfg->num_layers);
    for (int l = 0; l < cfg->num_layers; ++l) m->layers[l].c = layers[l];
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete m;
        zl_set_last_error(__FILE__, __LINE__, "cudaStreamCreate failed (no CUDA device? there is no CPU fallback)");
        return ZL_ERR_CUDA;
    }
    *out = m;
    return ZL_OK;
}

extern "C" void zl_dekipel_destroy(zl_dekipel_t* m) {
    if (!m) return;
    cudaStreamSynchronize(m->stream);
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
    for (auto& s : m->staged) cudaFree(s.second.ptr);
    for (auto& L : m->layers) {
        for (void* p : {(void*)L.norm1, (void*)L.norm1b, (void*)L.norm2, (void*)L.norm2b, (void*)L.canon1, (void*)L.canon2,
                        (void*)L.dq_norm, (void*)L.dkv_norm, (void*)L.sink, L.w_in, L.uq, L.uk_t, L.uv, L.o, L.up, L.down})
            if (p) cudaFree(p);
        L.latents.destroy();
        L.ring1.destroy();
        L.ring2.destroy();
    }
    for (void* p : {m->embed, m->head, (void*)m->final_norm, (void*)m->x, (void*)m->hbuf, (void*)m->proj, (void*)m->qa,
                    (void*)m->y, (void*)m->xw, (void*)m->logits, m->ubuf, m->cq, m->q, m->olat, m->og, m->act, m->xn,
                    (void*)m->d_tokens, (void*)m->d_slots, (void*)m->d_pos, (void*)m->d_want, (void*)m->d_next, m->attn_ws,
                    m->argmax_ws, (void*)m->layer_dump})
        if (p) cudaFree(p);
    if (m->h_stage) cudaFreeHost(m->h_stage);
    cudaStreamDestroy(m->stream);
    delete m;
}

extern "C" int zl_dekipel_load_tensor(zl_dekipel_t* m, const char* name, const void* data_host, int rows, int cols,
                                      int elem_bytes) {
    ZL_CHECK_ARG(m && name && data_host && rows > 0 && cols > 0 && (elem_bytes == 2 || elem_bytes == 4));
    if (m->finalized) return fail(__LINE__, "model already finalized");
    return staged_load(m->staged, name, data_host, rows, cols, elem_bytes, m->stream);
}

extern "C" int zl_dekipel_finalize(zl_dekipel_t* m) {
    ZL_CHECK_ARG(m);
    if (m->finalized) return ZL_OK;
    for (int l = 0; l < m->cfg.num_layers; ++l)
        if (!m->layers[l].ready) RCHECK(finalize_layer(m, l));
    RCHECK(take_weight(m, "embed", m->cfg.vocab, m->cfg.width, &m->embed));
    m->weight_bytes -= (double)m->cfg.vocab * m->cfg.width * m->esz;   // gathered, not streamed
    RCHECK(take_weight(m, "head", m->cfg.vocab, m->cfg.width, &m->head));
    RCHECK(take_f32(m, "final.norm", 1, m->cfg.width, &m->final_norm));
    RCHECK(alloc_runtime(m));
    m->finalized = true;
    return ZL_OK;
}

extern "C" int zl_dekipel_init_synthetic(zl_dekipel_t* m, uint64_t seed) {
    ZL_CHECK_ARG(m);
    if (m->finalized) return fail(__LINE__, "model already finalized");
    const auto& c = m->cfg;
    const int D = c.width;
    auto lin = [&](const std::string& name, int n, int k) {
        const float a = sqrtf(3.0f / (float)k);   // unit-variance outputs for unit-variance inputs
        return stage_random(m, name, n, k, -a, a, seed);
    };
    for (int l = 0; l < c.num_layers; ++l) {
        const auto& lc = m->layers[l].c;
        const std::string p = "l" + std::to_string(l) + ".";
        const int H = lc.heads, R = lc.kv_rank;
        for (const char* n : {"norm1", "norm1b"}) RCHECK(stage_random(m, p + n, 1, D, 0.9f, 1.1f, seed));
        RCHECK(stage_random(m, p + "canon1", D, c.canon_taps, -0.3f, 0.3f, seed));
        RCHECK(lin(p + "mix.dq", lc.q_rank, D));
        RCHECK(stage_random(m, p + "mix.dq.norm", 1, lc.q_rank, 0.9f, 1.1f, seed));
        RCHECK(lin(p + "mix.uq", H * lc.dim, lc.q_rank));
        if (lc.kv_from < 0) {
            RCHECK(lin(p + "mix.dkv", R, D));
            RCHECK(stage_random(m, p + "mix.dkv.norm", 1, R, 0.9f, 1.1f, seed));
        }
        RCHECK(lin(p + "mix.uk", H * lc.dim, R));
        RCHECK(lin(p + "mix.uv", H * lc.vdim, R));
        RCHECK(stage_random(m, p + "mix.sink", 1, H, -1.0f, 1.0f, seed));
        RCHECK(lin(p + "mix.g", H * lc.vdim, D));
        RCHECK(lin(p + "mix.o", D, H * lc.vdim));
        if (lc.ff > 0) {
            for (const char* n : {"norm2", "norm2b"}) RCHECK(stage_random(m, p + n, 1, D, 0.9f, 1.1f, seed));
            RCHECK(stage_random(m, p + "canon2", D, c.canon_taps, -0.3f, 0.3f, seed));
            RCHECK(lin(p + "mlp.up", lc.ff, D));
            RCHECK(lin(p + "mlp.down", D, lc.ff));
        }
        RCHECK(finalize_layer(m, l));   // bound the staging memory to one layer
    }
    RCHECK(stage_random(m, "embed", c.vocab, D, -1.7f, 1.7f, seed));
    RCHECK(lin("head", c.vocab, D));
    RCHECK(stage_random(m, "final.norm", 1, D, 0.9f, 1.1f, seed));
    return zl_dekipel_finalize(m);
}

extern "C" int zl_dekipel_step(zl_dekipel_t* m, const int32_t* tokens_host, const int32_t* slots_host,
                               const int32_t* positions_host, int T, const int32_t* want_rows_host, int n_want,
                               float* logits_host, int32_t* next_host) {
    ZL_CHECK_ARG(m && tokens_host && slots_host && positions_host && T > 0 && n_want >= 0);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    ZL_CHECK_ARG(T <= m->tcap && n_want <= T && (n_want == 0 || want_rows_host));
    const auto& c = m->cfg;
    int32_t* hs = m->h_stage;
    int max_len = 0;
    for (int i = 0; i < T; ++i) {
        ZL_CHECK_ARG(tokens_host[i] >= 0 && tokens_host[i] < c.vocab);
        ZL_CHECK_ARG(slots_host[i] >= 0 && slots_host[i] < c.max_batch);
        ZL_CHECK_ARG(positions_host[i] >= 0 && positions_host[i] < c.max_seq);
        // rows of one slot are consecutive and at consecutive positions; a slot appears in one run only
        if (i > 0 && slots_host[i] == slots_host[i - 1]) ZL_CHECK_ARG(positions_host[i] == positions_host[i - 1] + 1);
        hs[i] = tokens_host[i];
        hs[T + i] = slots_host[i];
        hs[2 * T + i] = positions_host[i];
        if (positions_host[i] + 1 > max_len) max_len = positions_host[i] + 1;
    }
    for (int i = 0; i < n_want; ++i) {
        ZL_CHECK_ARG(want_rows_host[i] >= 0 && want_rows_host[i] < T);
        hs[3 * T + i] = want_rows_host[i];
    }
    cudaStream_t st = m->stream;
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_tokens, hs, (size_t)T * 4, cudaMemcpyHostToDevice, st));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_slots, hs + T, (size_t)T * 4, cudaMemcpyHostToDevice, st));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_pos, hs + 2 * T, (size_t)T * 4, cudaMemcpyHostToDevice, st));
    if (n_want) ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_want, hs + 3 * T, (size_t)n_want * 4, cudaMemcpyHostToDevice, st));
    RCHECK(run_step(m, T, n_want, max_len));
    if (n_want && next_host) ZL_CHECK_CUDA(cudaMemcpyAsync(hs + 4 * T, m->d_next, (size_t)n_want * 4, cudaMemcpyDeviceToHost, st));
    if (n_want && logits_host)
        ZL_CHECK_CUDA(cudaMemcpyAsync(logits_host, m->logits, (size_t)n_want * c.vocab * 4, cudaMemcpyDeviceToHost, st));
    ZL_CHECK_CUDA(cudaStreamSynchronize(st));
    if (n_want && next_host)
        for (int i = 0; i < n_want; ++i) next_host[i] = hs[4 * T + i];
    if (max_len > m->cur_max_len) m->cur_max_len = max_len;
    return ZL_OK;
}

extern "C" int zl_dekipel_set_state(zl_dekipel_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B) {
    ZL_CHECK_ARG(m && tokens_host && positions_host && B > 0 && B <= m->cfg.max_batch);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));   // the staging buffer is free again
    int32_t* hs = m->h_stage;
    int mx = 0;
    for (int i = 0; i < B; ++i) {
        ZL_CHECK_ARG(tokens_host[i] >= 0 && tokens_host[i] < m->cfg.vocab);
        ZL_CHECK_ARG(positions_host[i] >= 0 && positions_host[i] < m->cfg.max_seq);
        hs[i] = tokens_host[i];
        hs[B + i] = positions_host[i];
        if (positions_host[i] + 1 > mx) mx = positions_host[i] + 1;
    }
    m->cur_max_len = mx;
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_tokens, hs, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_pos, hs + B, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    k_iota_i32<<<cdiv(B, 256), 256, 0, m->stream>>>(m->d_slots, m->d_want, B);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" int zl_dekipel_step_device(zl_dekipel_t* m, int B) {
    ZL_CHECK_ARG(m && B > 0 && B <= m->cfg.max_batch);
    if (m->cur_max_len >= m->cfg.max_seq) return fail(__LINE__, "latent caches full (max_seq reached)");
    RCHECK(run_step(m, B, B, m->cur_max_len));
    k_decode_advance<<<cdiv(B, 64), 64, 0, m->stream>>>(m->d_tokens, m->d_pos, m->d_next, B);
    ZL_CHECK_LAUNCH();
    m->cur_max_len += 1;
    return ZL_OK;
}

extern "C" int zl_dekipel_sync(zl_dekipel_t* m) {
    ZL_CHECK_ARG(m);
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" zl_stream_t zl_dekipel_stream(zl_dekipel_t* m) { return m ? (zl_stream_t)m->stream : nullptr; }

extern "C" int zl_dekipel_capture_layers(zl_dekipel_t* m, int on) {
    ZL_CHECK_ARG(m);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    if (on && !m->layer_dump)
        RCHECK(dmalloc((void**)&m->layer_dump, (size_t)m->cfg.num_layers * m->tcap * m->cfg.width * 4));
    m->capture = on != 0;
    return ZL_OK;
}

extern "C" int zl_dekipel_read_layers(zl_dekipel_t* m, float* out_host, int T) {
    ZL_CHECK_ARG(m && out_host && T > 0 && T <= m->tcap);
    if (!m->layer_dump) return fail(__LINE__, "layer capture was not switched on");
    const size_t row = (size_t)m->cfg.width * 4;
    ZL_CHECK_CUDA(cudaMemcpy2DAsync(out_host, (size_t)T * row, m->layer_dump, (size_t)m->tcap * row, (size_t)T * row,
                                    m->cfg.num_layers, cudaMemcpyDeviceToHost, m->stream));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" int zl_dekipel_stats(zl_dekipel_t* m, double* weight_bytes, int* kernels_per_step) {
    ZL_CHECK_ARG(m);
    if (weight_bytes) *weight_bytes = m->weight_bytes;
    if (kernels_per_step) *kernels_per_step = m->kernels_per_step;
    return ZL_OK;
}

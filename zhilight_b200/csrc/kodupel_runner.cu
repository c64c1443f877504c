// Host-side driver of the Kodupel model family: weights, slot caches and recurrent states, the per-step kernel chain and
// its CUDA graph.  Same driver shape as dekipel_runner.cu (task slots, host (token, slot, position) rows in, logits /
// greedy picks out), built from the shared pieces of runner_common.cuh.
//
// x = scale * embed[token] in fp32.  A layer: x += norm1(mixer(x)), x += norm2(experts(x)); the sublayers read x itself
// (rounded to the activation dtype for the Linears), the norms are RMS norms with weight 1 + w on the outputs only.
//   attention mixer:  one fused projection [W_q; W_k; W_v; W_g] with biases -> per-head norms, rotation, append to the
//                     slot's key / value caches (mixer_rows.cu) -> attention with a unit sink and a gate per head
//                     (sink_attn.cu) -> W_o with bias.  A layer with kv_from reads another layer's caches.
//   delta-rule mixer: one fused projection [W_r; W_k; W_v; W_a; W_g], the decay logits W_w2 tanh(W_w1 x) + w0 -> the
//                     recurrence over the slot's state (delta_rule.cu) -> per-head RMS norm, weight, gate -> W_o.
//   experts:          routing on the device (moe_route.cu) -> two grouped GEMMs over the (token, choice) pairs sorted by
//                     expert (gemm_tiled.cu), the clamped gated unit as the first one's epilogue -> weighted sum of a
//                     token's pairs inside the norm + residual kernel.
// One step takes T rows in any mix of prompt portions and single decode tokens; every kernel indexes caches and states
// by (slot, position), and the recurrence walks each run of rows (one slot, consecutive positions) in order.
#include "runner_common.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace {

using namespace zl;

struct KLayer {
    zl_kodupel_layer_t c{};
    float *norm1 = nullptr, *norm2 = nullptr;   // 1 + w
    void* w_in = nullptr;                       // fused input projection (n_in, width)
    float* b_in = nullptr;                      // its bias, fp32 (zeros where a part has none)
    void* b_in_act = nullptr;                   // the same in the activation dtype (skinny kernel)
    int n_in = 0, q_off = 0, k_off = -1, v_off = 0, g_off = 0, a_off = 0;   // attention: q | k | v | g; delta: r | k | v | a | g
    void* o = nullptr;                          // (width, heads * vdim)
    float* o_b = nullptr;
    void* o_b_act = nullptr;
    // attention
    float *q_norm = nullptr, *k_norm = nullptr;
    double* inv_freq = nullptr;
    float mscale = 1.f;
    SlotCache kcache, vcache;
    void **k_addrs = nullptr, **v_addrs = nullptr;   // own or the source layer's
    // delta rule
    void *w1 = nullptr, *w2 = nullptr;
    float *w0 = nullptr, *out_norm = nullptr;
    void* w0_act = nullptr;
    SlotCache state;                            // (slots, heads, dim, dim) fp32
    // experts
    float *router = nullptr, *correction = nullptr;   // fp32 (experts, width), (experts)
    void* w_gu = nullptr;                       // (experts, 2 * ff, width): rows 2j / 2j+1 = gate_j / up_j
    void* w_down = nullptr;                     // (experts, width, ff)
    bool ready = false;
};

}  // namespace

struct zl_kodupel {
    zl_kodupel_config_t cfg{};
    cudaStream_t stream = nullptr;
    StagedMap staged;
    std::vector<KLayer> layers;
    void *embed = nullptr, *head = nullptr;
    float* final_norm = nullptr;
    bool finalized = false;
    int esz = 2;
    int tcap = 0;
    float *x = nullptr, *proj = nullptr, *dlog = nullptr, *orec = nullptr, *y = nullptr, *ypair = nullptr, *xw = nullptr,
          *logits = nullptr, *top_w = nullptr;
    void *xa = nullptr, *q = nullptr, *att = nullptr, *z1 = nullptr, *act = nullptr, *xn = nullptr;
    int32_t *d_tokens = nullptr, *d_slots = nullptr, *d_pos = nullptr, *d_want = nullptr, *d_next = nullptr;
    int32_t *d_run0 = nullptr, *d_runlen = nullptr, *top_e = nullptr, *grp_off = nullptr, *list_token = nullptr,
            *list_pair = nullptr;
    int32_t* h_stage = nullptr;   // pinned: tokens | slots | pos | want | next | run0 | runlen
    void* attn_ws = nullptr;
    size_t attn_ws_bytes = 0;
    void* delta_ws = nullptr;
    size_t delta_ws_bytes = 0;
    void* argmax_ws = nullptr;
    float* layer_dump = nullptr;
    bool capture = false;
    std::map<long long, cudaGraphExec_t> graphs;
    int cur_max_len = 0;
    double weight_bytes = 0;
    int kernels_per_step = 0;
};

namespace {

int fail(int line, const std::string& msg, int code = ZL_ERR_STATE) {
    zl_set_last_error(__FILE__, line, msg.c_str());
    return code;
}

// x[t] = scale * embed[token[t]] in fp32 and the same rounded to the activation dtype (what the first Linears read)
__global__ void k_embed_scaled_pair(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table, float* __restrict__ x,
                                    __nv_bfloat16* __restrict__ xa, int D, int vocab, float scale) {
    pdl_trigger();
    pdl_wait();
    int id = ids[blockIdx.x];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = __bfloat162float(table[(size_t)id * D + i]) * scale;
        x[(size_t)blockIdx.x * D + i] = v;
        xa[(size_t)blockIdx.x * D + i] = __float2bfloat16_rn(v);
    }
}

__global__ void k_add_one(float* w, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) w[i] += 1.0f;
}
// dst rows 2j / 2j+1 of expert e <- gate / up row j of expert e; src are (ff, D) each
template <typename TS, typename TD>
__global__ void k_interleave_rows(const TS* __restrict__ gate, const TS* __restrict__ up, TD* __restrict__ dst, int ff, int D) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)ff * D) return;
    const size_t j = i / D, c = i % D;
    dst[(2 * j) * D + c] = from_f32<TD>(to_f32<TS>(gate[i]));
    dst[(2 * j + 1) * D + c] = from_f32<TD>(to_f32<TS>(up[i]));
}

// checkpoint norm tensor w -> fp32 array of the multipliers 1 + w
int take_norm(zl_kodupel* m, const std::string& name, int n, float** out) {
    RCHECK(take_f32(m, name, 1, n, out));
    k_add_one<<<cdiv(n, 256), 256, 0, m->stream>>>(*out, n);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

// bias segment `name` (n) -> fp32 bias array at offset off
int put_bias(zl_kodupel* m, const std::string& name, int n, float* dst, int off) {
    const Staged* s = need(m, name, 1, n);
    if (!s) return ZL_ERR_STATE;
    RCHECK(convert_to<float>(m, s, dst + off, (size_t)n));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, name);
    return ZL_OK;
}

// fp32 bias -> a copy in the activation dtype (bf16 mode; the checkpoint's biases are bfloat16, so nothing is lost)
int bias_act_copy(zl_kodupel* m, const float* src, int n, void** out) {
    if (m->cfg.dtype == ZL_F32) return ZL_OK;
    RCHECK(dmalloc(out, (size_t)n * 2));
    k_convert<float, __nv_bfloat16><<<cdiv(n, 256), 256, 0, m->stream>>>(src, static_cast<__nv_bfloat16*>(*out), (size_t)n);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

int finalize_experts(zl_kodupel* m, int l) {
    KLayer& L = m->layers[l];
    const auto& lc = L.c;
    const int D = m->cfg.width, E = lc.experts, F = lc.ff;
    const std::string p = "l" + std::to_string(l) + ".mlp.";
    RCHECK(take_f32(m, p + "router", E, D, &L.router));
    RCHECK(take_f32(m, p + "correction", 1, E, &L.correction));
    RCHECK(dmalloc(&L.w_gu, (size_t)E * 2 * F * D * m->esz));
    RCHECK(dmalloc(&L.w_down, (size_t)E * D * F * m->esz));
    for (int e = 0; e < E; ++e) {
        const std::string pe = p + "e" + std::to_string(e) + ".";
        const Staged* g = need(m, pe + "gate", F, D);
        const Staged* u = need(m, pe + "up", F, D);
        if (!g || !u) return ZL_ERR_STATE;
        if (g->elem != u->elem) return fail(__LINE__, "gate and up of an expert differ in dtype");
        const size_t n = (size_t)F * D, off = (size_t)e * 2 * n;
        const unsigned blocks = (unsigned)((n + 255) / 256);
        if (m->cfg.dtype == ZL_F32) {
            if (g->elem == 2)
                k_interleave_rows<<<blocks, 256, 0, m->stream>>>((const __nv_bfloat16*)g->ptr, (const __nv_bfloat16*)u->ptr,
                                                                 (float*)L.w_gu + off, F, D);
            else
                k_interleave_rows<<<blocks, 256, 0, m->stream>>>((const float*)g->ptr, (const float*)u->ptr, (float*)L.w_gu + off, F, D);
        } else {
            if (g->elem == 2)
                k_interleave_rows<<<blocks, 256, 0, m->stream>>>((const __nv_bfloat16*)g->ptr, (const __nv_bfloat16*)u->ptr,
                                                                 (__nv_bfloat16*)L.w_gu + off, F, D);
            else
                k_interleave_rows<<<blocks, 256, 0, m->stream>>>((const float*)g->ptr, (const float*)u->ptr,
                                                                 (__nv_bfloat16*)L.w_gu + off, F, D);
        }
        ZL_CHECK_LAUNCH();
        ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
        staged_drop(m->staged, pe + "gate");
        staged_drop(m->staged, pe + "up");
        m->weight_bytes += 2.0 * n * m->esz;
        RCHECK(put_weight(m, pe + "down", D, F, L.w_down, (size_t)e * D * F));
    }
    return ZL_OK;
}

int finalize_layer(zl_kodupel* m, int l) {
    const auto& c = m->cfg;
    KLayer& L = m->layers[l];
    const auto& lc = L.c;
    const std::string p = "l" + std::to_string(l) + ".", mx = p + "mix.";
    const int D = c.width, H = lc.heads;
    RCHECK(take_norm(m, p + "norm1", D, &L.norm1));
    if (lc.type == ZL_MIXER_ATTENTION) {
        const int G = lc.kv_heads, d = lc.dim, vd = lc.vdim, own = lc.kv_from < 0;
        L.q_off = 0;
        L.k_off = own ? H * d : -1;
        L.v_off = own ? H * d + G * d : 0;
        L.g_off = H * d + (own ? G * (d + vd) : 0);
        L.n_in = L.g_off + H;
        RCHECK(dmalloc(&L.w_in, (size_t)L.n_in * D * m->esz));
        RCHECK(dmalloc((void**)&L.b_in, (size_t)L.n_in * 4));
        ZL_CHECK_CUDA(cudaMemsetAsync(L.b_in, 0, (size_t)L.n_in * 4, m->stream));
        RCHECK(put_weight(m, mx + "q", H * d, D, L.w_in, 0));
        RCHECK(put_bias(m, mx + "q.b", H * d, L.b_in, 0));
        RCHECK(take_f32(m, mx + "q.norm", 1, d, &L.q_norm));
        if (own) {
            RCHECK(put_weight(m, mx + "k", G * d, D, L.w_in, (size_t)L.k_off * D));
            RCHECK(put_bias(m, mx + "k.b", G * d, L.b_in, L.k_off));
            RCHECK(put_weight(m, mx + "v", G * vd, D, L.w_in, (size_t)L.v_off * D));
            RCHECK(put_bias(m, mx + "v.b", G * vd, L.b_in, L.v_off));
            RCHECK(take_f32(m, mx + "k.norm", 1, d, &L.k_norm));
        }
        RCHECK(put_weight(m, mx + "g", H, D, L.w_in, (size_t)L.g_off * D));
        RCHECK(take_weight(m, mx + "o", D, H * vd, &L.o));
        RCHECK(take_f32(m, mx + "o.b", 1, D, &L.o_b));
        RCHECK(bias_act_copy(m, L.o_b, D, &L.o_b_act));
        if (lc.rot_dims > 0) {
            std::vector<double> f(lc.rot_dims / 2);
            RCHECK(zl_rope_inv_freq_yarn(lc.rot_base, lc.rot_dims, lc.yarn_factor, lc.yarn_original, lc.yarn_fast, lc.yarn_slow,
                                         f.data(), &L.mscale));
            RCHECK(dmalloc((void**)&L.inv_freq, f.size() * 8));
            ZL_CHECK_CUDA(cudaMemcpy(L.inv_freq, f.data(), f.size() * 8, cudaMemcpyHostToDevice));
        }
    } else {
        const int d = lc.dim, hd = H * d, R = lc.decay_rank;
        L.q_off = 0;          // r
        L.k_off = hd;
        L.v_off = 2 * hd;
        L.a_off = 3 * hd;
        L.g_off = 4 * hd;
        L.n_in = 5 * hd;
        RCHECK(dmalloc(&L.w_in, (size_t)L.n_in * D * m->esz));
        RCHECK(dmalloc((void**)&L.b_in, (size_t)L.n_in * 4));
        ZL_CHECK_CUDA(cudaMemsetAsync(L.b_in, 0, (size_t)L.n_in * 4, m->stream));
        RCHECK(put_weight(m, mx + "r", hd, D, L.w_in, 0));
        RCHECK(put_weight(m, mx + "k", hd, D, L.w_in, (size_t)L.k_off * D));
        RCHECK(put_weight(m, mx + "v", hd, D, L.w_in, (size_t)L.v_off * D));
        RCHECK(put_weight(m, mx + "a", hd, D, L.w_in, (size_t)L.a_off * D));
        RCHECK(put_bias(m, mx + "a.b", hd, L.b_in, L.a_off));
        RCHECK(put_weight(m, mx + "g", hd, D, L.w_in, (size_t)L.g_off * D));
        RCHECK(take_weight(m, mx + "w1", R, D, &L.w1));
        RCHECK(take_weight(m, mx + "w2", hd, R, &L.w2));
        RCHECK(take_f32(m, mx + "w0", 1, hd, &L.w0));
        RCHECK(bias_act_copy(m, L.w0, hd, &L.w0_act));
        RCHECK(take_f32(m, mx + "norm", 1, hd, &L.out_norm));
        RCHECK(take_weight(m, mx + "o", D, hd, &L.o));
    }
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    RCHECK(bias_act_copy(m, L.b_in, L.n_in, &L.b_in_act));
    if (lc.experts > 0) {
        RCHECK(take_norm(m, p + "norm2", D, &L.norm2));
        RCHECK(finalize_experts(m, l));
    }
    L.ready = true;
    return ZL_OK;
}

int len_bucket(const zl_kodupel* m, int max_len) {
    int b = 256;
    while (b < max_len) b <<= 1;
    return b < m->cfg.max_seq ? b : (m->cfg.max_seq > 256 ? m->cfg.max_seq : 256);
}

int alloc_runtime(zl_kodupel* m) {
    const auto& c = m->cfg;
    const int D = c.width, T = m->tcap, B = c.max_batch;
    size_t n_in = 1, hd = 1, hv = 1, rank = 1, pairs_ff = 1, top = 1, experts = 1;
    for (auto& L : m->layers) {
        const auto& lc = L.c;
        if (lc.type == ZL_MIXER_ATTENTION) {
            if (lc.kv_from < 0) {
                RCHECK(L.kcache.create(B, (size_t)c.max_seq * lc.kv_heads * lc.dim * m->esz, m->stream));
                RCHECK(L.vcache.create(B, (size_t)c.max_seq * lc.kv_heads * lc.vdim * m->esz, m->stream));
                L.k_addrs = L.kcache.addrs;
                L.v_addrs = L.vcache.addrs;
            }
            for (int b = 1; b <= T; ++b) {
                const int s = zl_sink_attention_splits(b, lc.heads, lc.kv_heads, len_bucket(m, c.max_seq));
                m->attn_ws_bytes = std::max(m->attn_ws_bytes, zl_sink_attention_workspace_bytes(b, lc.heads, lc.vdim, s));
                if (s == 1) break;
            }
            hv = std::max(hv, (size_t)lc.heads * lc.vdim);
        } else {
            RCHECK(zl_delta_rule_prepare(lc.dim, lc.dim));
            RCHECK(L.state.create(B, (size_t)lc.heads * lc.dim * lc.dim * 4, m->stream));
            m->delta_ws_bytes = std::max(m->delta_ws_bytes, zl_delta_rule_workspace_bytes(T, lc.heads, lc.dim, lc.dim));
            rank = std::max(rank, (size_t)lc.decay_rank);
            hv = std::max(hv, (size_t)lc.heads * lc.dim);
        }
        n_in = std::max(n_in, (size_t)L.n_in);
        hd = std::max(hd, (size_t)lc.heads * lc.dim);
        pairs_ff = std::max(pairs_ff, (size_t)lc.top * lc.ff);
        top = std::max(top, (size_t)lc.top);
        experts = std::max(experts, (size_t)lc.experts);
    }
    for (auto& L : m->layers)
        if (L.c.type == ZL_MIXER_ATTENTION && L.c.kv_from >= 0) {
            L.k_addrs = m->layers[L.c.kv_from].kcache.addrs;
            L.v_addrs = m->layers[L.c.kv_from].vcache.addrs;
        }
    const size_t e = m->esz;
    RCHECK(dmalloc((void**)&m->x, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->proj, (size_t)T * n_in * 4));
    RCHECK(dmalloc((void**)&m->dlog, (size_t)T * hd * 4));
    RCHECK(dmalloc((void**)&m->orec, (size_t)T * hd * 4));
    RCHECK(dmalloc((void**)&m->y, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->ypair, (size_t)T * top * D * 4));
    RCHECK(dmalloc((void**)&m->xw, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->logits, (size_t)T * c.vocab * 4));
    RCHECK(dmalloc((void**)&m->top_w, (size_t)T * top * 4));
    RCHECK(dmalloc(&m->xa, (size_t)T * D * e));
    RCHECK(dmalloc(&m->q, (size_t)T * hd * e));
    RCHECK(dmalloc(&m->att, (size_t)T * hv * e));
    RCHECK(dmalloc(&m->z1, (size_t)T * rank * e));
    RCHECK(dmalloc(&m->act, (size_t)T * pairs_ff * e));
    RCHECK(dmalloc(&m->xn, (size_t)T * D * e));
    for (int32_t** p : {&m->d_tokens, &m->d_slots, &m->d_pos, &m->d_want, &m->d_next, &m->d_run0, &m->d_runlen})
        RCHECK(dmalloc((void**)p, (size_t)T * 4));
    RCHECK(dmalloc((void**)&m->top_e, (size_t)T * top * 4));
    RCHECK(dmalloc((void**)&m->list_token, (size_t)T * top * 4));
    RCHECK(dmalloc((void**)&m->list_pair, (size_t)T * top * 4));
    RCHECK(dmalloc((void**)&m->grp_off, (experts + 1) * 4));
    RCHECK(dmalloc(&m->attn_ws, m->attn_ws_bytes));
    RCHECK(dmalloc(&m->delta_ws, m->delta_ws_bytes));
    RCHECK(dmalloc(&m->argmax_ws, zl_argmax_workspace_bytes(T)));
    ZL_CHECK_CUDA(cudaMallocHost((void**)&m->h_stage, sizeof(int32_t) * 7 * (size_t)T));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

// Which kernels of a step of at most 8 rows are launched with a programmatic dependency: 1 skinny Linears, 2 other GEMMs
// (tanh, grouped), 4 row kernels (norms, combine, head prep, router, plan), 8 attention, 16 recurrence, 32 the tail.
// Larger steps use none (early CTAs of a dependent kernel take SM slots from the kernel they wait for).
// ZL_KODUPEL_PDL_MASK overrides the default.
constexpr int kDefaultPdlMask = 1;
int pdl_mask() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("ZL_KODUPEL_PDL_MASK");
        v = e ? atoi(e) : kDefaultPdlMask;
    }
    return v;
}
int pdl_for(const zl_kodupel* m, int bit, int T) { return (m->cfg.use_pdl && T <= 8 && (pdl_mask() & bit)) ? 1 : 0; }

// y (M, N) = x (M, K) @ w (N, K)^T + bias, optional tanh.  bias_f32 / bias_act are the same numbers in two types.
int linear(zl_kodupel* m, const void* x, int K, const void* w, int N, const float* bias_f32, const void* bias_act, void* y,
           int M, int out_dtype, int epi) {
    const auto& c = m->cfg;
    static const bool no_skinny = getenv("ZL_KODUPEL_NO_SKINNY") != nullptr;
    if (!no_skinny && c.dtype != ZL_F32 && epi == ZL_GEMM_EPI_NONE && M <= 32 && K % 32 == 0 && N >= 64 && (!bias_f32 || bias_act) &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0)
        return zl_dense_gemm_skinny_act(x, K, w, bias_act, y, M, N, K, c.dtype, out_dtype, 0, pdl_for(m, 1, M), m->stream);
    return zl_gemm_nt_bias(x, K, w, K, bias_f32, y, N, M, N, K, c.dtype, out_dtype, epi, pdl_for(m, 2, M), m->stream);
}

int enqueue_step(zl_kodupel* m, int T, int n_want, int n_runs, int max_run, int max_len) {
    const auto& c = m->cfg;
    const int D = c.width, dt = c.dtype;
    cudaStream_t st = m->stream;
    const int pg = pdl_for(m, 2, T), pr = pdl_for(m, 4, T), pa = pdl_for(m, 8, T), pd = pdl_for(m, 16, T), pt = pdl_for(m, 32, T);
    const void* xin = dt == ZL_F32 ? (const void*)m->x : (const void*)m->xa;   // what the Linears read
    void* xa_out = dt == ZL_F32 ? nullptr : m->xa;
    if (dt == ZL_F32) {
        ZL_CHECK_CUDA(launch(k_embed_f32<float>, dim3(T), dim3(128), 0, st, false, (const int32_t*)m->d_tokens,
                             (const float*)m->embed, m->x, D, c.vocab, c.embed_scale));
    } else {
        ZL_CHECK_CUDA(launch(k_embed_scaled_pair, dim3(T), dim3(128), 0, st, false, (const int32_t*)m->d_tokens,
                             (const __nv_bfloat16*)m->embed, m->x, (__nv_bfloat16*)m->xa, D, c.vocab, c.embed_scale));
    }
    for (int l = 0; l < c.num_layers; ++l) {
        KLayer& L = m->layers[l];
        const auto& lc = L.c;
        const int H = lc.heads;
        RCHECK(linear(m, xin, D, L.w_in, L.n_in, L.b_in, L.b_in_act, m->proj, T, ZL_F32, ZL_GEMM_EPI_NONE));
        if (lc.type == ZL_MIXER_ATTENTION) {
            RCHECK(zl_qkv_headnorm_rope_append(m->proj, L.n_in, L.q_off, L.k_off, L.v_off, H, lc.kv_heads, lc.dim, lc.vdim,
                                               L.q_norm, L.k_norm, L.inv_freq, lc.rot_dims, L.mscale, c.eps, m->q, L.k_addrs,
                                               L.v_addrs, m->d_slots, m->d_pos, T, dt, pr, st));
            const int splits = zl_sink_attention_splits(T, H, lc.kv_heads, max_len);
            RCHECK(zl_sink_attention(m->q, L.k_addrs, L.v_addrs, m->d_slots, m->d_pos, nullptr, m->proj + L.g_off, L.n_in,
                                     lc.scale, m->att, T, H, lc.kv_heads, lc.dim, lc.vdim, splits, m->attn_ws, m->attn_ws_bytes,
                                     m->d_run0, m->d_runlen, n_runs, max_run, dt, pa, st));
            RCHECK(linear(m, m->att, H * lc.vdim, L.o, D, L.o_b, L.o_b_act, m->y, T, ZL_F32, ZL_GEMM_EPI_NONE));
        } else {
            const int hd = H * lc.dim;
            RCHECK(linear(m, xin, D, L.w1, lc.decay_rank, nullptr, nullptr, m->z1, T, dt, ZL_GEMM_EPI_TANH));
            RCHECK(linear(m, m->z1, lc.decay_rank, L.w2, hd, L.w0, L.w0_act, m->dlog, T, ZL_F32, ZL_GEMM_EPI_NONE));
            RCHECK(zl_delta_rule(m->proj + L.q_off, L.n_in, m->proj + L.k_off, L.n_in, m->proj + L.v_off, L.n_in,
                                 m->proj + L.a_off, L.n_in, m->dlog, hd, expf(-0.5f), 1e-6f, m->d_run0, m->d_runlen, n_runs,
                                 m->d_slots, m->d_pos, L.state.addrs, m->orec, hd, H, lc.dim, lc.dim, T, m->delta_ws, m->delta_ws_bytes, pd, st));
            RCHECK(zl_head_rmsnorm_gate(m->orec, hd, L.out_norm, m->proj + L.g_off, L.n_in, m->att, hd, T, H, lc.dim, c.eps, dt,
                                        pr, st));
            RCHECK(linear(m, m->att, hd, L.o, D, nullptr, nullptr, m->y, T, ZL_F32, ZL_GEMM_EPI_NONE));
        }
        RCHECK(zl_rmsnorm_residual_combine(m->y, D, nullptr, 1, L.norm1, m->x, D, xa_out, dt, T, D, c.eps, pr, st));
        if (lc.experts > 0) {
            const int E = lc.experts, top = lc.top, F = lc.ff;
            RCHECK(zl_moe_route(m->x, D, L.router, L.correction, m->top_e, m->top_w, m->grp_off, m->list_token, m->list_pair,
                                T, D, E, top, ZL_MOE_SCORE_SIGMOID, 0, pr, st));
            RCHECK(zl_gemm_nt_grouped(xin, D, m->list_token, L.w_gu, D, (long long)2 * F * D, m->act, F, nullptr, m->grp_off, E,
                                      T, 2 * F, D, dt, dt, ZL_GEMM_EPI_GLU_CLAMP, lc.limit, 1.702f, 1.0f, pg, st));
            RCHECK(zl_gemm_nt_grouped(m->act, F, nullptr, L.w_down, F, (long long)D * F, m->ypair, D, m->list_pair, m->grp_off,
                                      E, T, D, F, dt, ZL_F32, ZL_GEMM_EPI_NONE, 0.f, 1.f, 0.f, pg, st));
            RCHECK(zl_rmsnorm_residual_combine(m->ypair, D, m->top_w, top, L.norm2, m->x, D, xa_out, dt, T, D, c.eps, pr, st));
        }
        if (m->capture && m->layer_dump)
            ZL_CHECK_CUDA(cudaMemcpyAsync(m->layer_dump + (size_t)l * m->tcap * D, m->x, (size_t)T * D * 4,
                                          cudaMemcpyDeviceToDevice, st));
    }
    if (n_want > 0) {
        ZL_CHECK_CUDA(launch(k_gather_rows_f32, dim3(n_want), dim3(128), 0, st, false, (const float*)m->x,
                             (const int32_t*)m->d_want, m->xw, D));
        RCHECK(zl_group_rmsnorm(m->xw, D, m->final_norm, m->xn, D, n_want, D, 1, c.eps, dt, pt, st));
        RCHECK(linear(m, m->xn, D, m->head, c.vocab, nullptr, nullptr, m->logits, n_want, ZL_F32, ZL_GEMM_EPI_NONE));
        RCHECK(zl_argmax(m->logits, m->d_next, n_want, c.vocab, m->argmax_ws, zl_argmax_workspace_bytes(n_want), pt, st));
    }
    return ZL_OK;
}

// decode-sized steps replay a CUDA graph per (rows, wanted rows, runs, length bucket); prompt portions are enqueued directly
// (max_run: the longest run; a captured step is sized for the longest run its row count allows)
int run_step(zl_kodupel* m, int T, int n_want, int n_runs, int max_run, int max_len) {
    const int bucket = len_bucket(m, max_len);
    if (!m->cfg.use_graph || T > m->cfg.max_batch || m->capture) return enqueue_step(m, T, n_want, n_runs, max_run, bucket);
    const long long key = ((long long)T << 48) | ((long long)n_want << 32) | ((long long)n_runs << 16) | (long long)(bucket >> 8);
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        cudaGraph_t graph = nullptr;
        ZL_CHECK_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_step(m, T, n_want, n_runs, T - n_runs + 1, bucket);
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

extern "C" int zl_kodupel_create(const zl_kodupel_config_t* cfg, const zl_kodupel_layer_t* layers, zl_kodupel_t** out) {
    ZL_CHECK_ARG(cfg && layers && out);
    ZL_CHECK_ARG(cfg->num_layers > 0 && cfg->width > 0 && cfg->vocab > 0 && cfg->max_batch > 0 && cfg->max_seq > 0);
    ZL_CHECK_ARG(cfg->eps >= 0.f);
    ZL_CHECK_SUPPORTED(cfg->dtype == ZL_BF16 || cfg->dtype == ZL_F32);
    ZL_CHECK_ARG(cfg->max_step_tokens >= 0 && cfg->max_step_tokens <= 65535);
    for (int l = 0; l < cfg->num_layers; ++l) {
        const auto& lc = layers[l];
        ZL_CHECK_ARG(lc.heads > 0 && lc.dim > 0 && lc.experts >= 0);
        if (lc.type == ZL_MIXER_ATTENTION) {
            ZL_CHECK_ARG(lc.kv_heads > 0 && lc.heads % lc.kv_heads == 0 && lc.vdim > 0);
            ZL_CHECK_ARG(lc.rot_dims >= 0 && lc.rot_dims <= lc.dim && lc.rot_dims % 2 == 0);
            ZL_CHECK_ARG(lc.rot_dims == 0 || lc.rot_base > 1.f);
            if (lc.kv_from >= 0) {
                // the source layer runs earlier in the step, owns its caches, and has the same key / value shape
                const auto& sc = layers[lc.kv_from < l ? lc.kv_from : 0];
                ZL_CHECK_ARG(lc.kv_from < l && sc.type == ZL_MIXER_ATTENTION && sc.kv_from < 0 && sc.kv_heads == lc.kv_heads &&
                             sc.dim == lc.dim && sc.vdim == lc.vdim);
            }
        } else {
            ZL_CHECK_ARG(lc.type == ZL_MIXER_GENERAL_DELTA && lc.decay_rank > 0);
        }
        if (lc.experts > 0) ZL_CHECK_ARG(lc.top > 0 && lc.top <= lc.experts && lc.ff > 0 && lc.limit > 0.f);
    }
    zl_kodupel* m = new zl_kodupel();
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

extern "C" void zl_kodupel_destroy(zl_kodupel_t* m) {
    if (!m) return;
    cudaStreamSynchronize(m->stream);
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
    for (auto& s : m->staged) cudaFree(s.second.ptr);
    for (auto& L : m->layers) {
        for (void* p : {(void*)L.norm1, (void*)L.norm2, L.w_in, (void*)L.b_in, L.b_in_act, L.o, (void*)L.o_b, L.o_b_act,
                        (void*)L.q_norm, (void*)L.k_norm, (void*)L.inv_freq, L.w1, L.w2, (void*)L.w0, L.w0_act, (void*)L.out_norm,
                        (void*)L.router, (void*)L.correction, L.w_gu, L.w_down})
            if (p) cudaFree(p);
        L.kcache.destroy();
        L.vcache.destroy();
        L.state.destroy();
    }
    for (void* p : {m->embed, m->head, (void*)m->final_norm, (void*)m->x, (void*)m->proj, (void*)m->dlog, (void*)m->orec,
                    (void*)m->y, (void*)m->ypair, (void*)m->xw, (void*)m->logits, (void*)m->top_w, m->xa, m->q, m->att, m->z1,
                    m->act, m->xn, (void*)m->d_tokens, (void*)m->d_slots, (void*)m->d_pos, (void*)m->d_want, (void*)m->d_next,
                    (void*)m->d_run0, (void*)m->d_runlen, (void*)m->top_e, (void*)m->grp_off, (void*)m->list_token,
                    (void*)m->list_pair, m->attn_ws, m->delta_ws, m->argmax_ws, (void*)m->layer_dump})
        if (p) cudaFree(p);
    if (m->h_stage) cudaFreeHost(m->h_stage);
    cudaStreamDestroy(m->stream);
    delete m;
}

extern "C" int zl_kodupel_load_tensor(zl_kodupel_t* m, const char* name, const void* data_host, int rows, int cols,
                                      int elem_bytes) {
    ZL_CHECK_ARG(m && name && data_host && rows > 0 && cols > 0 && (elem_bytes == 2 || elem_bytes == 4));
    if (m->finalized) return fail(__LINE__, "model already finalized");
    return staged_load(m->staged, name, data_host, rows, cols, elem_bytes, m->stream);
}

extern "C" int zl_kodupel_finalize(zl_kodupel_t* m) {
    ZL_CHECK_ARG(m);
    if (m->finalized) return ZL_OK;
    for (int l = 0; l < m->cfg.num_layers; ++l)
        if (!m->layers[l].ready) RCHECK(finalize_layer(m, l));
    RCHECK(take_weight(m, "embed", m->cfg.vocab, m->cfg.width, &m->embed));
    m->weight_bytes -= (double)m->cfg.vocab * m->cfg.width * m->esz;   // gathered, not streamed
    RCHECK(take_weight(m, "head", m->cfg.vocab, m->cfg.width, &m->head));
    RCHECK(take_norm(m, "final.norm", m->cfg.width, &m->final_norm));
    RCHECK(alloc_runtime(m));
    m->finalized = true;
    return ZL_OK;
}

extern "C" int zl_kodupel_init_synthetic(zl_kodupel_t* m, uint64_t seed) {
    ZL_CHECK_ARG(m);
    if (m->finalized) return fail(__LINE__, "model already finalized");
    const auto& c = m->cfg;
    const int D = c.width;
    auto lin = [&](const std::string& name, int n, int k) {
        const float a = sqrtf(3.0f / (float)k);   // unit-variance outputs for unit-variance inputs
        return stage_random(m, name, n, k, -a, a, seed);
    };
    auto small = [&](const std::string& name, int n, float a) { return stage_random(m, name, 1, n, -a, a, seed); };
    for (int l = 0; l < c.num_layers; ++l) {
        const auto& lc = m->layers[l].c;
        const std::string p = "l" + std::to_string(l) + ".", mx = p + "mix.";
        const int H = lc.heads;
        RCHECK(small(p + "norm1", D, 0.1f));
        if (lc.type == ZL_MIXER_ATTENTION) {
            RCHECK(lin(mx + "q", H * lc.dim, D));
            RCHECK(small(mx + "q.b", H * lc.dim, 0.1f));
            RCHECK(stage_random(m, mx + "q.norm", 1, lc.dim, 0.9f, 1.1f, seed));
            if (lc.kv_from < 0) {
                RCHECK(lin(mx + "k", lc.kv_heads * lc.dim, D));
                RCHECK(small(mx + "k.b", lc.kv_heads * lc.dim, 0.1f));
                RCHECK(lin(mx + "v", lc.kv_heads * lc.vdim, D));
                RCHECK(small(mx + "v.b", lc.kv_heads * lc.vdim, 0.1f));
                RCHECK(stage_random(m, mx + "k.norm", 1, lc.dim, 0.9f, 1.1f, seed));
            }
            RCHECK(lin(mx + "g", H, D));
            RCHECK(lin(mx + "o", D, H * lc.vdim));
            RCHECK(small(mx + "o.b", D, 0.1f));
        } else {
            const int hd = H * lc.dim;
            for (const char* n : {"r", "k", "v", "a", "g"}) RCHECK(lin(mx + n, hd, D));
            RCHECK(small(mx + "a.b", hd, 0.5f));
            RCHECK(lin(mx + "w1", lc.decay_rank, D));
            RCHECK(lin(mx + "w2", hd, lc.decay_rank));
            RCHECK(small(mx + "w0", hd, 1.0f));
            RCHECK(stage_random(m, mx + "norm", 1, hd, 0.9f, 1.1f, seed));
            RCHECK(lin(mx + "o", D, hd));
        }
        if (lc.experts > 0) {
            RCHECK(small(p + "norm2", D, 0.1f));
            RCHECK(lin(p + "mlp.router", lc.experts, D));
            RCHECK(small(p + "mlp.correction", lc.experts, 0.2f));
            for (int e = 0; e < lc.experts; ++e) {
                const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
                RCHECK(lin(pe + "gate", lc.ff, D));
                RCHECK(lin(pe + "up", lc.ff, D));
                RCHECK(lin(pe + "down", D, lc.ff));
            }
        }
        RCHECK(finalize_layer(m, l));   // bound the staging memory to one layer
    }
    RCHECK(stage_random(m, "embed", c.vocab, D, -1.7f, 1.7f, seed));
    RCHECK(lin("head", c.vocab, D));
    RCHECK(small("final.norm", D, 0.1f));
    return zl_kodupel_finalize(m);
}

extern "C" int zl_kodupel_step(zl_kodupel_t* m, const int32_t* tokens_host, const int32_t* slots_host,
                               const int32_t* positions_host, int T, const int32_t* want_rows_host, int n_want,
                               float* logits_host, int32_t* next_host) {
    ZL_CHECK_ARG(m && tokens_host && slots_host && positions_host && T > 0 && n_want >= 0);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    ZL_CHECK_ARG(T <= m->tcap && n_want <= T && (n_want == 0 || want_rows_host));
    const auto& c = m->cfg;
    int32_t* hs = m->h_stage;
    int max_len = 0, n_runs = 0, max_run = 1;
    for (int i = 0; i < T; ++i) {
        ZL_CHECK_ARG(tokens_host[i] >= 0 && tokens_host[i] < c.vocab);
        ZL_CHECK_ARG(slots_host[i] >= 0 && slots_host[i] < c.max_batch);
        ZL_CHECK_ARG(positions_host[i] >= 0 && positions_host[i] < c.max_seq);
        // rows of one slot are consecutive and at consecutive positions; a slot appears in one run only
        if (i > 0 && slots_host[i] == slots_host[i - 1]) {
            ZL_CHECK_ARG(positions_host[i] == positions_host[i - 1] + 1);
            hs[6 * T + n_runs - 1] += 1;
            if (hs[6 * T + n_runs - 1] > max_run) max_run = hs[6 * T + n_runs - 1];
        } else {
            hs[5 * T + n_runs] = i;
            hs[6 * T + n_runs] = 1;
            ++n_runs;
        }
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
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_run0, hs + 5 * T, (size_t)n_runs * 4, cudaMemcpyHostToDevice, st));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_runlen, hs + 6 * T, (size_t)n_runs * 4, cudaMemcpyHostToDevice, st));
    if (n_want) ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_want, hs + 3 * T, (size_t)n_want * 4, cudaMemcpyHostToDevice, st));
    RCHECK(run_step(m, T, n_want, n_runs, max_run, max_len));
    if (n_want && next_host) ZL_CHECK_CUDA(cudaMemcpyAsync(hs + 4 * T, m->d_next, (size_t)n_want * 4, cudaMemcpyDeviceToHost, st));
    if (n_want && logits_host)
        ZL_CHECK_CUDA(cudaMemcpyAsync(logits_host, m->logits, (size_t)n_want * c.vocab * 4, cudaMemcpyDeviceToHost, st));
    ZL_CHECK_CUDA(cudaStreamSynchronize(st));
    if (n_want && next_host)
        for (int i = 0; i < n_want; ++i) next_host[i] = hs[4 * T + i];
    if (max_len > m->cur_max_len) m->cur_max_len = max_len;
    return ZL_OK;
}

extern "C" int zl_kodupel_set_state(zl_kodupel_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B) {
    ZL_CHECK_ARG(m && tokens_host && positions_host && B > 0 && B <= m->cfg.max_batch);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));   // the staging buffer is free again
    int32_t* hs = m->h_stage;
    const int T = m->tcap;
    int mx = 0;
    for (int i = 0; i < B; ++i) {
        ZL_CHECK_ARG(tokens_host[i] >= 0 && tokens_host[i] < m->cfg.vocab);
        ZL_CHECK_ARG(positions_host[i] >= 0 && positions_host[i] < m->cfg.max_seq);
        hs[i] = tokens_host[i];
        hs[T + i] = positions_host[i];
        hs[2 * T + i] = 1;
        if (positions_host[i] + 1 > mx) mx = positions_host[i] + 1;
    }
    m->cur_max_len = mx;
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_tokens, hs, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_pos, hs + T, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_runlen, hs + 2 * T, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    k_iota_i32<<<cdiv(B, 256), 256, 0, m->stream>>>(m->d_slots, m->d_want, B);
    k_iota_i32<<<cdiv(B, 256), 256, 0, m->stream>>>(m->d_run0, m->d_want, B);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" int zl_kodupel_step_device(zl_kodupel_t* m, int B) {
    ZL_CHECK_ARG(m && B > 0 && B <= m->cfg.max_batch);
    if (m->cur_max_len >= m->cfg.max_seq) return fail(__LINE__, "caches full (max_seq reached)");
    RCHECK(run_step(m, B, B, B, 1, m->cur_max_len));
    k_decode_advance<<<cdiv(B, 64), 64, 0, m->stream>>>(m->d_tokens, m->d_pos, m->d_next, B);
    ZL_CHECK_LAUNCH();
    m->cur_max_len += 1;
    return ZL_OK;
}

extern "C" int zl_kodupel_sync(zl_kodupel_t* m) {
    ZL_CHECK_ARG(m);
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" zl_stream_t zl_kodupel_stream(zl_kodupel_t* m) { return m ? (zl_stream_t)m->stream : nullptr; }

extern "C" int zl_kodupel_capture_layers(zl_kodupel_t* m, int on) {
    ZL_CHECK_ARG(m);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    if (on && !m->layer_dump)
        RCHECK(dmalloc((void**)&m->layer_dump, (size_t)m->cfg.num_layers * m->tcap * m->cfg.width * 4));
    m->capture = on != 0;
    return ZL_OK;
}

extern "C" int zl_kodupel_read_layers(zl_kodupel_t* m, float* out_host, int T) {
    ZL_CHECK_ARG(m && out_host && T > 0 && T <= m->tcap);
    if (!m->layer_dump) return fail(__LINE__, "layer capture was not switched on");
    const size_t row = (size_t)m->cfg.width * 4;
    ZL_CHECK_CUDA(cudaMemcpy2DAsync(out_host, (size_t)T * row, m->layer_dump, (size_t)m->tcap * row, (size_t)T * row,
                                    m->cfg.num_layers, cudaMemcpyDeviceToHost, m->stream));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" int zl_kodupel_read_state(zl_kodupel_t* m, int layer, int slot, float* out_host) {
    ZL_CHECK_ARG(m && out_host && layer >= 0 && layer < m->cfg.num_layers && slot >= 0 && slot < m->cfg.max_batch);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    const KLayer& L = m->layers[layer];
    ZL_CHECK_ARG(L.c.type == ZL_MIXER_GENERAL_DELTA);
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    ZL_CHECK_CUDA(cudaMemcpy(out_host, (const char*)L.state.buf + (size_t)slot * L.state.slot_bytes, L.state.slot_bytes,
                             cudaMemcpyDeviceToHost));
    return ZL_OK;
}

extern "C" int zl_kodupel_stats(zl_kodupel_t* m, double* weight_bytes, int* kernels_per_step) {
    ZL_CHECK_ARG(m);
    if (weight_bytes) *weight_bytes = m->weight_bytes;
    if (kernels_per_step) *kernels_per_step = m->kernels_per_step;
    return ZL_OK;
}

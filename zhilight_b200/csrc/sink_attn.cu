// Causal attention over per-slot key and value caches with grouped key/value heads, a softmax whose denominator holds
// one extra term exp(sink) that has no value (sink = 0 adds exactly one), and an optional sigmoid gate per head on
// the output.  Token t of the step sees rows 0 .. pos[t] of the caches of slot[t]; the step's own keys and values are
// appended before this runs, so prompts, portions of prompts and single decode tokens are the same case.
//
// k_sink_attn: any head sizes up to 256 and any dtype; scores, softmax and the weighted sum in fp32 FMAs.  One CTA per
// (token, query head); its 8 warps take the keys j = warp, warp + 8, ... (a fixed assignment: the result of a token
// does not depend on the step it is computed in) with an online softmax each, merged in warp order with the sink term.
#include "common.cuh"

namespace zl {

constexpr int kSaWarps = 8, kSaMaxPerLane = 8;

struct SinkAttnP {
    const void* q;             // (T, H * d)
    void* const* k_addrs;      // slot -> (max_seq, G, d)
    void* const* v_addrs;      // slot -> (max_seq, G, vd)
    const int32_t *slot, *pos;
    const float* sink;         // (H) or null: sink 0
    const float* gate;         // gate[t * ldg + h] logits or null
    long long ldg;
    void* out;                 // (T, H * vd)
    int H, G, d, vd;
    float scale;
    int splits;
    float* ws;                 // splits > 1: (T, H, splits, 2 + vd) partial (max, sum, weighted values)
};

template <typename T>
__global__ void __launch_bounds__(kSaWarps * 32) k_sink_attn(SinkAttnP p) {
    extern __shared__ float ssm[];
    float* sq = ssm;                        // d
    float* sm_m = ssm + p.d;                // kSaWarps
    float* sm_l = sm_m + kSaWarps;          // kSaWarps
    float* sm_acc = sm_l + kSaWarps;        // kSaWarps * vd
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.x, t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = h / (p.H / p.G), pos = p.pos[t], sl = p.slot[t];
    const T* q = static_cast<const T*>(p.q) + ((size_t)t * p.H + h) * p.d;
    for (int c = threadIdx.x; c < p.d; c += blockDim.x) sq[c] = to_f32<T>(q[c]) * p.scale;
    __syncthreads();
    const T* kc = static_cast<const T*>(p.k_addrs[sl]) + (size_t)g * p.d;
    const T* vc = static_cast<const T*>(p.v_addrs[sl]) + (size_t)g * p.vd;
    const size_t kst = (size_t)p.G * p.d, vst = (size_t)p.G * p.vd;
    float m = -INFINITY, l = 0.f, acc[kSaMaxPerLane];
#pragma unroll
    for (int i = 0; i < kSaMaxPerLane; ++i) acc[i] = 0.f;
    // keys of this split: a range of whole groups of kSaWarps keys
    int j_lo = 0, j_hi = pos + 1;
    if (p.splits > 1) {
        const int per = cdiv(cdiv(pos + 1, p.splits), kSaWarps) * kSaWarps;
        j_lo = blockIdx.z * per;
        j_hi = min(pos + 1, j_lo + per);
    }
    for (int j = j_lo + warp; j < j_hi; j += kSaWarps) {
        const T* kr = kc + (size_t)j * kst;
        float s = 0.f;
        for (int c = lane; c < p.d; c += 32) s = fmaf(sq[c], to_f32<T>(kr[c]), s);
        s = warp_sum(s);
        const float mn = fmaxf(m, s), corr = expf(m - mn), w = expf(s - mn);
        l = fmaf(l, corr, w);
        const T* vr = vc + (size_t)j * vst;
#pragma unroll
        for (int i = 0; i < kSaMaxPerLane; ++i) {
            const int c = lane + 32 * i;
            if (c < p.vd) acc[i] = fmaf(acc[i], corr, w * to_f32<T>(vr[c]));
        }
        m = mn;
    }
    if (lane == 0) sm_m[warp] = m, sm_l[warp] = l;
#pragma unroll
    for (int i = 0; i < kSaMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < p.vd) sm_acc[(size_t)warp * p.vd + c] = acc[i];
    }
    __syncthreads();
    if (p.splits > 1) {   // partial result of this range, without the sink
        float M = -INFINITY;
        for (int w = 0; w < kSaWarps; ++w) M = fmaxf(M, sm_m[w]);
        float L = 0.f;
        for (int w = 0; w < kSaWarps; ++w) L = fmaf(sm_l[w], sm_m[w] == -INFINITY ? 0.f : expf(sm_m[w] - M), L);
        float* part = p.ws + (((size_t)t * p.H + h) * p.splits + blockIdx.z) * (2 + p.vd);
        if (threadIdx.x == 0) part[0] = M, part[1] = L;
        for (int c = threadIdx.x; c < p.vd; c += blockDim.x) {
            float o = 0.f;
            for (int w = 0; w < kSaWarps; ++w)
                o = fmaf(sm_acc[(size_t)w * p.vd + c], sm_m[w] == -INFINITY ? 0.f : expf(sm_m[w] - M), o);
            part[2 + c] = o;
        }
        return;
    }
    const float sink = p.sink ? p.sink[h] : 0.f;
    float M = sink;
    for (int w = 0; w < kSaWarps; ++w) M = fmaxf(M, sm_m[w]);
    float L = expf(sink - M);
    for (int w = 0; w < kSaWarps; ++w) L = fmaf(sm_l[w], expf(sm_m[w] - M), L);
    float gate = 1.0f;
    if (p.gate) gate = 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.ldg + h]));
    T* out = static_cast<T*>(p.out) + ((size_t)t * p.H + h) * p.vd;
    for (int c = threadIdx.x; c < p.vd; c += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < kSaWarps; ++w) o = fmaf(sm_acc[(size_t)w * p.vd + c], expf(sm_m[w] - M), o);
        out[c] = from_f32<T>(o / L * gate);
    }
}

// merge of the splits with the sink term and the gate; one warp per (token, head), grid (ceil(H / 4), T)
template <typename T>
__global__ void __launch_bounds__(128) k_sink_attn_merge(SinkAttnP p) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= p.H) return;
    const float* part = p.ws + ((size_t)t * p.H + h) * p.splits * (2 + p.vd);
    const float sink = p.sink ? p.sink[h] : 0.f;
    float M = sink;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, part[(size_t)s * (2 + p.vd)]);
    float L = expf(sink - M);
    for (int s = 0; s < p.splits; ++s) {
        const float ms = part[(size_t)s * (2 + p.vd)];
        L = fmaf(part[(size_t)s * (2 + p.vd) + 1], ms == -INFINITY ? 0.f : expf(ms - M), L);
    }
    float gate = 1.0f;
    if (p.gate) gate = 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.ldg + h]));
    T* out = static_cast<T*>(p.out) + ((size_t)t * p.H + h) * p.vd;
    for (int c = lane; c < p.vd; c += 32) {
        float o = 0.f;
        for (int s = 0; s < p.splits; ++s) {
            const float ms = part[(size_t)s * (2 + p.vd)];
            o = fmaf(part[(size_t)s * (2 + p.vd) + 2 + c], ms == -INFINITY ? 0.f : expf(ms - M), o);
        }
        out[c] = from_f32<T>(o / L * gate);
    }
}

}  // namespace zl

using namespace zl;

extern "C" size_t zl_sink_attention_workspace_bytes(int T, int heads, int vdim, int splits) {
    return splits > 1 ? (size_t)T * heads * splits * (2 + vdim) * sizeof(float) : 0;
}

// enough CTAs for two waves of the SMs, no split shorter than 256 keys, at most 32
extern "C" int zl_sink_attention_splits(int T, int heads, int kv_heads, int max_len) {
    (void)kv_heads;
    const int want = cdiv(2 * device_sm_count(), T * heads > 0 ? T * heads : 1);
    const int cap = max_len / 256 > 0 ? max_len / 256 : 1;
    int s = want < cap ? want : cap;
    if (s > 32) s = 32;
    return s < 1 ? 1 : s;
}

extern "C" int zl_sink_attention(const void* q, void* const* k_addrs, void* const* v_addrs, const int32_t* slot,
                                 const int32_t* pos, const float* sink, const float* gate, long long ldg, float scale, void* out,
                                 int T, int heads, int kv_heads, int dim, int vdim, int splits, void* workspace,
                                 size_t workspace_bytes, int dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(q && k_addrs && v_addrs && slot && pos && out && T > 0 && T <= 65535 && heads > 0 && kv_heads > 0);
    ZL_CHECK_ARG(heads % kv_heads == 0 && dim > 0 && vdim > 0);
    ZL_CHECK_SUPPORTED(vdim <= 32 * kSaMaxPerLane);
    ZL_CHECK_ARG(dtype == ZL_F16 || dtype == ZL_BF16 || dtype == ZL_F32);
    ZL_CHECK_ARG(splits >= 1 && splits <= 65535);
    ZL_CHECK_ARG(splits == 1 || (workspace && workspace_bytes >= zl_sink_attention_workspace_bytes(T, heads, vdim, splits)));
    SinkAttnP p{q, k_addrs, v_addrs, slot, pos, sink, gate, ldg, out, heads, kv_heads, dim, vdim, scale, splits,
                static_cast<float*>(workspace)};
    const dim3 grid(heads, T, splits), block(kSaWarps * 32);
    const size_t smem = ((size_t)dim + 2 * kSaWarps + (size_t)kSaWarps * vdim) * sizeof(float);
    cudaError_t e;
    if (dtype == ZL_F32) e = launch(k_sink_attn<float>, grid, block, smem, stream, pdl != 0, p);
    else if (dtype == ZL_BF16) e = launch(k_sink_attn<__nv_bfloat16>, grid, block, smem, stream, pdl != 0, p);
    else e = launch(k_sink_attn<__half>, grid, block, smem, stream, pdl != 0, p);
    ZL_CHECK_CUDA(e);
    if (splits > 1) {
        const dim3 mg(cdiv(heads, 4), T), mb(128);
        if (dtype == ZL_F32) e = launch(k_sink_attn_merge<float>, mg, mb, 0, stream, pdl != 0, p);
        else if (dtype == ZL_BF16) e = launch(k_sink_attn_merge<__nv_bfloat16>, mg, mb, 0, stream, pdl != 0, p);
        else e = launch(k_sink_attn_merge<__half>, mg, mb, 0, stream, pdl != 0, p);
        ZL_CHECK_CUDA(e);
    }
    return ZL_OK;
}

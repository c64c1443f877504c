// Attention over a cache of low-rank key-value latents, in the absorbed form, with a per-head softmax sink.
//
// A layer of this kind caches one latent row c_j (kv_rank numbers) per position; keys and values of head h are
// W_uk,h c_j and W_uv,h c_j.  Instead of expanding the cache, the query is pulled through W_uk,h once
// (qa_h = W_uk,h^T q_h, a per-head GEMM before this kernel), so that score_h(i, j) = scale * qa_h(i) . c_j, and the
// probabilities are applied to the latents themselves (o_h = sum_j p_j c_j); W_uv,h follows as a per-head GEMM.  All
// heads of a token read the same latent rows: multi-query attention with head size kv_rank whose K and V are one array.
// The softmax denominator of head h additionally holds exp(sink_h): a term with no key and no value, not scaled.  It
// enters the running (max, sum) pair as its initial value (max = sink_h, sum = 1), or in the merge when the keys of a
// token are split over several CTAs.  Scores, probabilities and the accumulation are fp32.
//
// Token t of a step sees the rows 0 .. pos[t] of its slot; the step's own latents are appended before this kernel, so
// one kernel serves prompt portions (consecutive positions of one slot) and decode batches (one token per slot).
#include "common.cuh"

#include <math.h>

namespace zl {

constexpr int kLaThreads = 128;
constexpr int kLaKeys = 32;         // keys per tile: one per lane in the score phase
constexpr int kLaMaxElems = 4096;   // (heads per CTA) x kv_rank accumulators, 32 per thread at most

template <typename TC>
struct LaParams {
    const float* qa;       // (T, H, R)
    void* const* slot_addrs;
    const int32_t* slot;
    const int32_t* pos;
    const float* sink;     // (H)
    void* out;             // (T, H, R) activation dtype
    float* part_acc;       // (T, H, S, R)
    float* part_ml;        // (T, H, S, 2)
    float scale;
    int H, R, HG, S;
};

template <typename TC, int EPT>
__global__ void __launch_bounds__(kLaThreads) k_latent_attn(LaParams<TC> p) {
    extern __shared__ float smem[];
    const int R = p.R, RP = R + 1;
    float* sq = smem;                       // [HG][R]
    float* sc = sq + p.HG * R;              // [32][R + 1]
    float* sp = sc + kLaKeys * RP;          // [HG][32]
    float* sm = sp + p.HG * kLaKeys;        // [HG] running max
    float* sl = sm + p.HG;                  // [HG] running sum
    float* scorr = sl + p.HG;               // [HG]
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, h0 = blockIdx.y * p.HG, split = blockIdx.z;
    const int hg = min(p.HG, p.H - h0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int len = p.pos[t] + 1;
    const TC* cache = static_cast<const TC*>(p.slot_addrs[p.slot[t]]);
    int lo = 0, hi = len;
    if (p.S > 1) {
        const int per = cdiv(cdiv(len, p.S), kLaKeys) * kLaKeys;
        lo = split * per;
        hi = min(len, lo + per);
    }
    for (int i = tid; i < hg * R; i += kLaThreads) sq[i] = p.qa[((size_t)t * p.H + h0) * R + i];
    if (tid < hg) {
        sm[tid] = p.S > 1 ? -INFINITY : p.sink[h0 + tid];
        sl[tid] = p.S > 1 ? 0.f : 1.f;
    }
    float acc[EPT];
#pragma unroll
    for (int k = 0; k < EPT; ++k) acc[k] = 0.f;

    for (int j0 = lo; j0 < hi; j0 += kLaKeys) {
        __syncthreads();   // previous tile fully consumed (and sq / sm / sl initialised)
        for (int i = tid; i < kLaKeys * R; i += kLaThreads) {
            const int j = i / R, r = i - j * R;
            sc[j * RP + r] = (j0 + j < hi) ? to_f32<TC>(cache[(size_t)(j0 + j) * R + r]) : 0.f;
        }
        __syncthreads();
        for (int hh = warp; hh < hg; hh += kLaThreads / 32) {
            const float* q = sq + hh * R;
            const float* c = sc + lane * RP;
            float s = 0.f;
            for (int r = 0; r < R; ++r) s = fmaf(q[r], c[r], s);
            const bool valid = j0 + lane < hi;
            s = valid ? s * p.scale : -INFINITY;
            const float m_old = sm[hh];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float pj = valid ? expf(s - m_new) : 0.f;
            const float ps = warp_sum(pj);
            sp[hh * kLaKeys + lane] = pj;
            __syncwarp();
            if (lane == 0) {
                const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                scorr[hh] = corr;
                sl[hh] = sl[hh] * corr + ps;
                sm[hh] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int e = tid + k * kLaThreads;
            if (e < hg * R) {
                const int hh = e / R, r = e - hh * R;
                float a = acc[k] * scorr[hh];
                const float* pr = sp + hh * kLaKeys;
#pragma unroll 8
                for (int j = 0; j < kLaKeys; ++j) a = fmaf(pr[j], sc[j * RP + r], a);
                acc[k] = a;
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int e = tid + k * kLaThreads;
        if (e < hg * R) {
            const int hh = e / R, r = e - hh * R;
            const size_t th = (size_t)t * p.H + h0 + hh;
            if (p.S > 1) p.part_acc[(th * p.S + split) * R + r] = acc[k];
            else static_cast<TC*>(p.out)[th * R + r] = from_f32<TC>(acc[k] / sl[hh]);
        }
    }
    if (p.S > 1 && tid < hg) {
        const size_t th = (size_t)t * p.H + h0 + tid;
        p.part_ml[(th * p.S + split) * 2 + 0] = sm[tid];
        p.part_ml[(th * p.S + split) * 2 + 1] = sl[tid];
    }
}

// grid (H, T): merge the S partial (max, sum, accumulator) triples of one (token, head) and the sink
template <typename TC>
__global__ void k_latent_attn_merge(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    const float* __restrict__ sink, TC* __restrict__ out, int H, int R, int S) {
    pdl_trigger();
    pdl_wait();
    const size_t th = (size_t)blockIdx.y * H + blockIdx.x;
    const float* ml = part_ml + th * S * 2;
    float M = sink[blockIdx.x];
    for (int s = 0; s < S; ++s) M = fmaxf(M, ml[2 * s]);
    float L = expf(sink[blockIdx.x] - M);
    for (int s = 0; s < S; ++s)
        if (ml[2 * s] != -INFINITY) L += ml[2 * s + 1] * expf(ml[2 * s] - M);
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < S; ++s)
            if (ml[2 * s] != -INFINITY) a += part_acc[(th * S + s) * R + r] * expf(ml[2 * s] - M);
        out[th * R + r] = from_f32<TC>(a / L);
    }
}

static int la_heads_per_cta(int H, int R) {
    int hg = kLaMaxElems / R;
    if (hg < 1) hg = 1;
    return hg < H ? hg : H;
}
static size_t la_smem_bytes(int HG, int R) {
    return sizeof(float) * ((size_t)HG * R + (size_t)kLaKeys * (R + 1) + (size_t)HG * kLaKeys + 3 * (size_t)HG);
}

template <typename TC>
static int la_launch(LaParams<TC> p, int T, bool pdl, cudaStream_t st) {
    const size_t smem = la_smem_bytes(p.HG, p.R);
    const int ept = cdiv(p.HG * p.R, kLaThreads);
    const dim3 grid(T, cdiv(p.H, p.HG), p.S), block(kLaThreads);
#define ZL_LA_CASE(E)                                                                                        \
    {                                                                                                        \
        ZL_CHECK_CUDA(launch(k_latent_attn<TC, E>, grid, block, smem, st, pdl, p));                           \
    }
    if (ept <= 4) ZL_LA_CASE(4)
    else if (ept <= 8) ZL_LA_CASE(8)
    else if (ept <= 16) ZL_LA_CASE(16)
    else ZL_LA_CASE(32)
#undef ZL_LA_CASE
    if (p.S > 1)
        ZL_CHECK_CUDA(launch(k_latent_attn_merge<TC>, dim3(p.H, T), dim3(128), 0, st, pdl, (const float*)p.part_acc,
                             (const float*)p.part_ml, p.sink, static_cast<TC*>(p.out), p.H, p.R, p.S));
    return ZL_OK;
}

}  // namespace zl

using namespace zl;

extern "C" size_t zl_latent_attention_workspace_bytes(int T, int heads, int kv_rank, int splits) {
    if (splits <= 1) return 0;
    return sizeof(float) * (size_t)T * heads * splits * ((size_t)kv_rank + 2);
}

template <typename TC>
static int la_prepare(size_t smem) {
    ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn<TC, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn<TC, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn<TC, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn<TC, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return ZL_OK;
}

// how many CTAs share one token's keys: enough to fill the GPU when the step has few (token, head group) pairs
extern "C" int zl_latent_attention_splits(int T, int heads, int kv_rank, int max_len) {
    if (T <= 0 || heads <= 0 || kv_rank <= 0 || kv_rank > kLaMaxElems) return 1;
    const int ctas = T * cdiv(heads, la_heads_per_cta(heads, kv_rank));
    const int want = 2 * device_sm_count();
    if (ctas >= want || max_len <= 4 * kLaKeys) return 1;
    int s = cdiv(want, ctas);
    const int by_len = cdiv(max_len, 4 * kLaKeys);
    if (s > by_len) s = by_len;
    return s < 1 ? 1 : (s > 64 ? 64 : s);
}

// opt-in shared memory of the kernel for this shape; call once outside any stream capture
extern "C" int zl_latent_attention_prepare(int heads, int kv_rank, int dtype) {
    ZL_CHECK_ARG(heads > 0 && kv_rank > 0);
    ZL_CHECK_SUPPORTED(kv_rank <= kLaMaxElems);
    const size_t smem = la_smem_bytes(la_heads_per_cta(heads, kv_rank), kv_rank);
    ZL_CHECK_SUPPORTED(smem <= 200 * 1024);
    if (smem <= 48 * 1024) return ZL_OK;
    if (dtype == ZL_F32) return la_prepare<float>(smem);
    if (dtype == ZL_BF16) return la_prepare<__nv_bfloat16>(smem);
    return la_prepare<__half>(smem);
}

extern "C" int zl_latent_attention(const float* q_absorbed, void* const* slot_addrs, const int32_t* slot, const int32_t* pos,
                                   const float* sink, float scale, void* out, int T, int heads, int kv_rank, int splits,
                                   void* workspace, size_t workspace_bytes, int dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(q_absorbed && slot_addrs && slot && pos && sink && out && T > 0 && heads > 0 && kv_rank > 0);
    ZL_CHECK_ARG(dtype == ZL_F16 || dtype == ZL_BF16 || dtype == ZL_F32);
    ZL_CHECK_ARG(splits >= 1 && splits <= 65535 && heads <= 65535);
    ZL_CHECK_SUPPORTED(kv_rank <= kLaMaxElems);
    ZL_CHECK_ARG(workspace_bytes >= zl_latent_attention_workspace_bytes(T, heads, kv_rank, splits) && (splits == 1 || workspace));
    const int HG = la_heads_per_cta(heads, kv_rank);
    ZL_CHECK_SUPPORTED(la_smem_bytes(HG, kv_rank) <= 200 * 1024);
    float* part_acc = static_cast<float*>(workspace);
    float* part_ml = splits > 1 ? part_acc + (size_t)T * heads * splits * kv_rank : nullptr;
    if (dtype == ZL_F32) {
        LaParams<float> p{q_absorbed, slot_addrs, slot, pos, sink, out, part_acc, part_ml, scale, heads, kv_rank, HG, splits};
        return la_launch<float>(p, T, pdl != 0, stream);
    }
    if (dtype == ZL_BF16) {
        LaParams<__nv_bfloat16> p{q_absorbed, slot_addrs, slot, pos, sink, out, part_acc, part_ml, scale, heads, kv_rank, HG, splits};
        return la_launch<__nv_bfloat16>(p, T, pdl != 0, stream);
    }
    LaParams<__half> p{q_absorbed, slot_addrs, slot, pos, sink, out, part_acc, part_ml, scale, heads, kv_rank, HG, splits};
    return la_launch<__half>(p, T, pdl != 0, stream);
}

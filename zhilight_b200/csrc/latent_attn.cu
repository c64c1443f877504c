// Attention over a cache of low-rank key-value latents, in the absorbed form, with a per-head softmax sink.
//
// A layer of this kind caches one latent row c_j (kv_rank numbers) per position; keys and values of head h are
// W_uk,h c_j and W_uv,h c_j.  Instead of expanding the cache, the query is pulled through W_uk,h once
// (qa_h = W_uk,h^T q_h, a per-head GEMM before this kernel), so that score_h(i, j) = scale * qa_h(i) . c_j, and the
// probabilities are applied to the latents themselves (o_h = sum_j p_j c_j); W_uv,h follows as a per-head GEMM.  All
// heads of a token read the same latent rows: multi-query attention with head size kv_rank whose K and V are one array.
// The softmax normaliser of head h has one extra term, exp(sink_h), that belongs to no position: it adds to the sum only,
// unscaled, once per head and query.  It enters the running (max, sum) pair as its initial value (max = sink_h, sum = 1),
// or in the merge when the keys of a token are split over several CTAs.  Scores, probabilities and the accumulation are fp32.
//
// Token t of a step sees the rows 0 .. pos[t] of its slot; the step's own latents are appended before this kernel, so
// one kernel serves prompt portions (consecutive positions of one slot) and decode batches (one token per slot).
#include "common.cuh"

#include <math.h>
#include <stdlib.h>

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

// grid (H, T): merge the S <= 64 partial (max, sum, accumulator) triples of one (token, head) and the sink
template <typename TC>
__global__ void k_latent_attn_merge(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    const float* __restrict__ sink, TC* __restrict__ out, int H, int R, int S) {
    __shared__ float wgt[64];
    pdl_trigger();
    pdl_wait();
    const size_t th = (size_t)blockIdx.y * H + blockIdx.x;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float* ml = part_ml + th * S * 2;
        const float sk = sink[blockIdx.x];
        const float m0 = lane < S ? ml[2 * lane] : -INFINITY, m1 = lane + 32 < S ? ml[2 * (lane + 32)] : -INFINITY;
        const float l0 = lane < S ? ml[2 * lane + 1] : 0.f, l1 = lane + 32 < S ? ml[2 * (lane + 32) + 1] : 0.f;
        const float M = fmaxf(sk, warp_max(fmaxf(m0, m1)));
        const float e0 = m0 == -INFINITY ? 0.f : expf(m0 - M), e1 = m1 == -INFINITY ? 0.f : expf(m1 - M);
        const float L = expf(sk - M) + warp_sum(l0 * e0 + l1 * e1);
        wgt[lane] = e0 / L;
        wgt[lane + 32] = e1 / L;
    }
    __syncthreads();
    const float* pa = part_acc + th * S * R;
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        float a = 0.f;
#pragma unroll 4
        for (int s = 0; s < S; ++s) a = fmaf(pa[(size_t)s * R + r], wgt[s], a);
        out[th * R + r] = from_f32<TC>(a);
    }
}

// ---- tensor-core variant (bfloat16 caches, kv_rank a multiple of 64 up to 512) -------------------------------------------
// One CTA = one token x 16 heads x one key range; 4 warps.  The 32-key latent tile is staged once in shared memory
// (cp.async, three tiles in flight) and serves both products: S = Qa C^T (contraction over kv_rank, split in quarters over the
// warps, the partial 16 x 32 score tiles summed through shared memory in a fixed order) and O += P C (each warp owns a
// quarter of the kv_rank output columns; C is read through ldmatrix.trans).  Scores, softmax and O are fp32; Qa and P
// enter the MMAs as bfloat16.
constexpr int kLmKeys = 32;
constexpr int kLmRows = 16;
constexpr int kLmStages = 3;   // latent tiles in flight per CTA

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}

template <int NK>   // kv_rank = 64 * NK: every warp contracts over 16 * NK and owns 16 * NK output columns
__global__ void __launch_bounds__(128) k_latent_attn_mma(LaParams<__nv_bfloat16> p) {
    constexpr int RQ = 16 * NK, R = 4 * RQ, RP = R + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sc = reinterpret_cast<__nv_bfloat16*>(smem_raw);                       // [stages][32][RP]
    float* ss = reinterpret_cast<float*>(smem_raw + (size_t)kLmStages * kLmKeys * RP * 2);   // [4][16][34]
    pdl_trigger();
    pdl_wait();
    const int h0 = blockIdx.x * kLmRows, t = blockIdx.y, split = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q4 = lane & 3;
    const int len = p.pos[t] + 1;
    const __nv_bfloat16* cache = static_cast<const __nv_bfloat16*>(p.slot_addrs[p.slot[t]]);
    int lo = 0, hi = len;
    if (p.S > 1) {
        const int per = cdiv(cdiv(len, p.S), kLmKeys) * kLmKeys;
        lo = split * per;
        hi = min(len, lo + per);
    }
    const int ha = h0 + g, hb = h0 + g + 8;   // the two heads (rows) this lane holds
    // query fragments of this warp's contraction quarter
    uint32_t qf[NK][4];
    {
        const float* qa = p.qa + ((size_t)t * p.H) * R + warp * RQ;
#pragma unroll
        for (int ks = 0; ks < NK; ++ks) {
            const int k = ks * 16 + 2 * q4;
            const float2 z = make_float2(0.f, 0.f);
            const float2 a0 = ha < p.H ? *reinterpret_cast<const float2*>(qa + (size_t)ha * R + k) : z;
            const float2 a1 = hb < p.H ? *reinterpret_cast<const float2*>(qa + (size_t)hb * R + k) : z;
            const float2 a2 = ha < p.H ? *reinterpret_cast<const float2*>(qa + (size_t)ha * R + k + 8) : z;
            const float2 a3 = hb < p.H ? *reinterpret_cast<const float2*>(qa + (size_t)hb * R + k + 8) : z;
            qf[ks][0] = pack_bf16(a0.x, a0.y), qf[ks][1] = pack_bf16(a1.x, a1.y);
            qf[ks][2] = pack_bf16(a2.x, a2.y), qf[ks][3] = pack_bf16(a3.x, a3.y);
        }
    }
    float m_run[2], l_run[2];
    m_run[0] = p.S > 1 ? -INFINITY : (ha < p.H ? p.sink[ha] : 0.f);
    m_run[1] = p.S > 1 ? -INFINITY : (hb < p.H ? p.sink[hb] : 0.f);
    l_run[0] = l_run[1] = p.S > 1 ? 0.f : 1.f;
    float o[2 * NK][4];
#pragma unroll
    for (int i = 0; i < 2 * NK; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[i][c] = 0.f;

    auto stage = [&](int j0, int buf) {   // 32 keys x R bf16 in 16-byte pieces; keys past `hi` are zero rows
        __nv_bfloat16* dst = sc + (size_t)buf * kLmKeys * RP;
        for (int i = tid; i < kLmKeys * (R / 8); i += 128) {
            const int j = i / (R / 8), c8 = (i - j * (R / 8)) * 8;
            if (j0 + j < hi) cp_async16(dst + j * RP + c8, cache + (size_t)(j0 + j) * R + c8);
            else *reinterpret_cast<uint4*>(dst + j * RP + c8) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    };
    const int n_tiles = hi > lo ? cdiv(hi - lo, kLmKeys) : 0;
    if (n_tiles > 0) stage(lo, 0);
    if (n_tiles > 1) stage(lo + kLmKeys, 1);
    else cp_async_commit();
    for (int it = 0; it < n_tiles; ++it) {
        const int j0 = lo + it * kLmKeys, buf = it % kLmStages;
        cp_async_wait<1>();   // all but the youngest group: tile `it` has landed
        __syncthreads();      // ... for every thread; every warp is done with round it - 1 (its buffer, the score tiles)
        if (it + 2 < n_tiles) stage(j0 + 2 * kLmKeys, (it + 2) % kLmStages);   // two tiles ahead of the math
        else cp_async_commit();
        const __nv_bfloat16* ct = sc + (size_t)buf * kLmKeys * RP;
        // partial scores over this warp's quarter of kv_rank
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) s[nt][c] = 0.f;
            const __nv_bfloat16* krow = ct + (nt * 8 + g) * RP + warp * RQ + 2 * q4;
#pragma unroll
            for (int ks = 0; ks < NK; ++ks) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + ks * 16);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + ks * 16 + 8);
                mma_16816_bf16(s[nt], qf[ks], b0, b1, s[nt]);
            }
        }
        float* mine = ss + warp * (kLmRows * 34);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            *reinterpret_cast<float2*>(mine + g * 34 + nt * 8 + 2 * q4) = make_float2(s[nt][0], s[nt][1]);
            *reinterpret_cast<float2*>(mine + (g + 8) * 34 + nt * 8 + 2 * q4) = make_float2(s[nt][2], s[nt][3]);
        }
        __syncthreads();
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float2 ra = make_float2(0.f, 0.f), rb = make_float2(0.f, 0.f);
#pragma unroll
            for (int w = 0; w < 4; ++w) {   // same order in every warp: identical sums
                const float2 xa = *reinterpret_cast<const float2*>(ss + w * (kLmRows * 34) + g * 34 + nt * 8 + 2 * q4);
                const float2 xb = *reinterpret_cast<const float2*>(ss + w * (kLmRows * 34) + (g + 8) * 34 + nt * 8 + 2 * q4);
                ra.x += xa.x, ra.y += xa.y, rb.x += xb.x, rb.y += xb.y;
            }
            const int j = j0 + nt * 8 + 2 * q4;
            s[nt][0] = j < hi ? ra.x * p.scale : -INFINITY;
            s[nt][1] = j + 1 < hi ? ra.y * p.scale : -INFINITY;
            s[nt][2] = j < hi ? rb.x * p.scale : -INFINITY;
            s[nt][3] = j + 1 < hi ? rb.y * p.scale : -INFINITY;
            mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
        }
        float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            corr[r] = expf(m_run[r] - m_use);
            m_run[r] = m_new;
            mx[r] = m_use;
        }
        uint32_t pf[2][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float p0 = expf(s[nt][0] - mx[0]), p1 = expf(s[nt][1] - mx[0]);
            const float p2 = expf(s[nt][2] - mx[1]), p3 = expf(s[nt][3] - mx[1]);
            sum[0] += p0 + p1;
            sum[1] += p2 + p3;
            pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
            l_run[r] = l_run[r] * corr[r] + sum[r];
        }
        // O (16 x RQ columns of this warp) = O * corr + P (16 x 32 keys) C (32 keys x RQ)
#pragma unroll
        for (int nt = 0; nt < 2 * NK; ++nt) {
            o[nt][0] *= corr[0], o[nt][1] *= corr[0], o[nt][2] *= corr[1], o[nt][3] *= corr[1];
            uint32_t bv[4];
            ldmatrix_x4_trans(bv, ct + lane * RP + warp * RQ + nt * 8);
            mma_16816_bf16(o[nt], pf[0], bv[0], bv[1], o[nt]);
            mma_16816_bf16(o[nt], pf[1], bv[2], bv[3], o[nt]);
        }
    }
    const size_t tha = (size_t)t * p.H + ha, thb = (size_t)t * p.H + hb;
#pragma unroll
    for (int nt = 0; nt < 2 * NK; ++nt) {
        const int col = warp * RQ + nt * 8 + 2 * q4;
        if (p.S > 1) {
            if (ha < p.H) *reinterpret_cast<float2*>(p.part_acc + (tha * p.S + split) * R + col) = make_float2(o[nt][0], o[nt][1]);
            if (hb < p.H) *reinterpret_cast<float2*>(p.part_acc + (thb * p.S + split) * R + col) = make_float2(o[nt][2], o[nt][3]);
        } else {
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
            if (ha < p.H)
                *reinterpret_cast<uint32_t*>(out + tha * R + col) = pack_bf16(o[nt][0] / l_run[0], o[nt][1] / l_run[0]);
            if (hb < p.H)
                *reinterpret_cast<uint32_t*>(out + thb * R + col) = pack_bf16(o[nt][2] / l_run[1], o[nt][3] / l_run[1]);
        }
    }
    if (p.S > 1 && warp == 0 && q4 == 0) {
        if (ha < p.H) p.part_ml[(tha * p.S + split) * 2] = m_run[0], p.part_ml[(tha * p.S + split) * 2 + 1] = l_run[0];
        if (hb < p.H) p.part_ml[(thb * p.S + split) * 2] = m_run[1], p.part_ml[(thb * p.S + split) * 2 + 1] = l_run[1];
    }
}

static bool lm_eligible(int dtype, int R) {
    static const bool off = getenv("ZL_LATENT_ATTN_NO_MMA") != nullptr;
    return !off && dtype == ZL_BF16 && R % 64 == 0 && R >= 64 && R <= 512;
}
static size_t lm_smem_bytes(int R) { return (size_t)kLmStages * kLmKeys * (R + 8) * 2 + (size_t)4 * kLmRows * 34 * 4; }

static int lm_launch(const LaParams<__nv_bfloat16>& p, int T, bool pdl, cudaStream_t st) {
    const size_t smem = lm_smem_bytes(p.R);
    const dim3 grid(cdiv(p.H, kLmRows), T, p.S), block(128);
    switch (p.R / 64) {
        case 1: ZL_CHECK_CUDA(launch(k_latent_attn_mma<1>, grid, block, smem, st, pdl, p)); break;
        case 2: ZL_CHECK_CUDA(launch(k_latent_attn_mma<2>, grid, block, smem, st, pdl, p)); break;
        case 3: ZL_CHECK_CUDA(launch(k_latent_attn_mma<3>, grid, block, smem, st, pdl, p)); break;
        case 4: ZL_CHECK_CUDA(launch(k_latent_attn_mma<4>, grid, block, smem, st, pdl, p)); break;
        case 5: ZL_CHECK_CUDA(launch(k_latent_attn_mma<5>, grid, block, smem, st, pdl, p)); break;
        case 6: ZL_CHECK_CUDA(launch(k_latent_attn_mma<6>, grid, block, smem, st, pdl, p)); break;
        case 7: ZL_CHECK_CUDA(launch(k_latent_attn_mma<7>, grid, block, smem, st, pdl, p)); break;
        default: ZL_CHECK_CUDA(launch(k_latent_attn_mma<8>, grid, block, smem, st, pdl, p)); break;
    }
    if (p.S > 1)
        ZL_CHECK_CUDA(launch(k_latent_attn_merge<__nv_bfloat16>, dim3(p.H, T), dim3(128), 0, st, pdl, (const float*)p.part_acc,
                             (const float*)p.part_ml, p.sink, static_cast<__nv_bfloat16*>(p.out), p.H, p.R, p.S));
    return ZL_OK;
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
    const int ctas = T * cdiv(heads, lm_eligible(ZL_BF16, kv_rank) ? kLmRows : la_heads_per_cta(heads, kv_rank));
    const int want = 2 * device_sm_count();
    if (ctas >= want || max_len <= 4 * kLaKeys) return 1;
    int s = want / ctas;   // rounded down: one wave of CTAs, no tail
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
    if (lm_eligible(dtype, kv_rank) && lm_smem_bytes(kv_rank) > 48 * 1024) {
        const int b = (int)lm_smem_bytes(kv_rank);
        ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn_mma<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
        ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn_mma<5>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
        ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn_mma<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
        ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn_mma<7>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
        ZL_CHECK_CUDA(cudaFuncSetAttribute(k_latent_attn_mma<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    }
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
        if (lm_eligible(dtype, kv_rank) && (reinterpret_cast<uintptr_t>(q_absorbed) & 7) == 0) return lm_launch(p, T, pdl != 0, stream);
        return la_launch<__nv_bfloat16>(p, T, pdl != 0, stream);
    }
    LaParams<__half> p{q_absorbed, slot_addrs, slot, pos, sink, out, part_acc, part_ml, scale, heads, kv_rank, HG, splits};
    return la_launch<__half>(p, T, pdl != 0, stream);
}

// Generalized delta rule: a recurrent mixer whose state per head is a (dk, dv) fp32 matrix S carried from token to token,
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,      o_t = S_t^T r_t,
// with u_t = k_t / sqrt(sum(k_t^2) + unit_eps), a decay w_t = exp(-decay_scale * sigmoid(decay_logit_t)) and a removal
// rate a_t = sigmoid(rate_logit_t) per key channel; both subtracted terms read S_(t-1).
//
// The columns of S (one per value channel) never meet: S_t[:, j] depends on S_(t-1)[:, j] and on the token's vectors
// only.  A thread owns one column and walks the tokens of its sequence in order, so the result of a token does not
// depend on how the sequence was cut into steps or on the other sequences of the step.  A CTA owns `cols` columns of
// one head of one run (the consecutive rows of one slot in the step); the token vectors (u, a*u, w, k, r) of a chunk of
// tokens are prepared by the whole CTA in shared memory, then every thread updates its column for the chunk without
// any barrier.  The column lives in registers when dk is one of the compiled sizes, in shared memory otherwise.
// A run that starts at position 0 starts from a zero state (a slot given to a new sequence needs no clearing); the
// final state goes back to the slot.  Everything is fp32.
#include "common.cuh"

#include <cstdlib>

namespace zl {

constexpr int kDrChunk = 8;   // tokens prepared at a time

struct DeltaP {
    const float *r, *k, *v, *rate_logit, *decay_logit;   // (T, H * dk) / v: (T, H * dv), row strides below
    long long ld_r, ld_k, ld_v, ld_a, ld_w;
    const int32_t *run_row0, *run_len;   // per run: first row of the step, rows
    const int32_t *slot, *pos;
    void* const* state_addrs;            // slot -> (H, dk, dv) fp32
    float* o;                            // (T, H * dv)
    long long ld_o;
    int H, dk, dv, cols;
    float decay_scale, unit_eps;
};

// grid (dv / cols rounded up, H, runs); block = cols rounded up to a warp.  DK > 0: the column in registers.
template <int DK>
__global__ void k_delta_rule(DeltaP p) {
    extern __shared__ float dsm[];
    const int dk = DK > 0 ? DK : p.dk;
    float* tok = dsm;                                   // [kDrChunk][5][dk]: u, a*u, w, k, r
    float* scol = dsm + (size_t)kDrChunk * 5 * dk;      // DK == 0: [dk][blockDim] the columns of this CTA
    pdl_trigger();
    pdl_wait();
    const int run = blockIdx.z, h = blockIdx.y, tid = threadIdx.x, nth = blockDim.x;
    const int warp = tid >> 5, lane = tid & 31, nw = nth >> 5;
    const int row0 = p.run_row0[run], len = p.run_len[run];
    if (len <= 0) return;
    const int j = blockIdx.x * p.cols + tid;            // my value channel
    const bool mine = tid < p.cols && j < p.dv;
    float* sg = static_cast<float*>(p.state_addrs[p.slot[row0]]) + (size_t)h * dk * p.dv;
    const bool fresh = p.pos[row0] == 0;
    float S[DK > 0 ? DK : 1];
    if (mine) {
        if constexpr (DK > 0) {
#pragma unroll
            for (int i = 0; i < DK; ++i) S[i] = fresh ? 0.f : sg[(size_t)i * p.dv + j];
        } else {
            for (int i = 0; i < dk; ++i) scol[(size_t)i * nth + tid] = fresh ? 0.f : sg[(size_t)i * p.dv + j];
        }
    }
    for (int c0 = 0; c0 < len; c0 += kDrChunk) {
        const int cn = min(kDrChunk, len - c0);
        __syncthreads();   // the previous chunk's vectors are no longer read
        for (int tt = warp; tt < cn; tt += nw) {
            const size_t t = (size_t)(row0 + c0 + tt);
            const float* kr = p.k + t * p.ld_k + (size_t)h * dk;
            float ss = 0.f;
            for (int i = lane; i < dk; i += 32) ss = fmaf(kr[i], kr[i], ss);
            const float inv = 1.0f / sqrtf(warp_sum(ss) + p.unit_eps);
            float* tv = tok + (size_t)tt * 5 * dk;
            for (int i = lane; i < dk; i += 32) {
                const float kk = kr[i], u = kk * inv;
                const float a = 1.0f / (1.0f + expf(-p.rate_logit[t * p.ld_a + (size_t)h * dk + i]));
                const float sg_w = 1.0f / (1.0f + expf(-p.decay_logit[t * p.ld_w + (size_t)h * dk + i]));
                tv[i] = u;
                tv[dk + i] = a * u;
                tv[2 * dk + i] = expf(-p.decay_scale * sg_w);
                tv[3 * dk + i] = kk;
                tv[4 * dk + i] = p.r[t * p.ld_r + (size_t)h * dk + i];
            }
        }
        __syncthreads();
        if (!mine) continue;
        for (int tt = 0; tt < cn; ++tt) {
            const size_t t = (size_t)(row0 + c0 + tt);
            const float* tv = tok + (size_t)tt * 5 * dk;
            const float vj = p.v[t * p.ld_v + (size_t)h * p.dv + j];
            float dot = 0.f, out = 0.f;
            if constexpr (DK > 0) {
#pragma unroll
                for (int i = 0; i < DK; ++i) dot = fmaf(tv[i], S[i], dot);
#pragma unroll
                for (int i = 0; i < DK; ++i) {
                    const float s = fmaf(tv[3 * DK + i], vj, fmaf(-tv[DK + i], dot, tv[2 * DK + i] * S[i]));
                    S[i] = s;
                    out = fmaf(s, tv[4 * DK + i], out);
                }
            } else {
                for (int i = 0; i < dk; ++i) dot = fmaf(tv[i], scol[(size_t)i * nth + tid], dot);
                for (int i = 0; i < dk; ++i) {
                    const float s = fmaf(tv[3 * dk + i], vj, fmaf(-tv[dk + i], dot, tv[2 * dk + i] * scol[(size_t)i * nth + tid]));
                    scol[(size_t)i * nth + tid] = s;
                    out = fmaf(s, tv[4 * dk + i], out);
                }
            }
            p.o[t * p.ld_o + (size_t)h * p.dv + j] = out;
        }
    }
    if (mine) {
        if constexpr (DK > 0) {
#pragma unroll
            for (int i = 0; i < DK; ++i) sg[(size_t)i * p.dv + j] = S[i];
        } else {
            for (int i = 0; i < dk; ++i) sg[(size_t)i * p.dv + j] = scol[(size_t)i * nth + tid];
        }
    }
}

template <int DK>
static int launch_delta(const DeltaP& p, int runs, int block, bool pdl, cudaStream_t st) {
    size_t smem = (size_t)kDrChunk * 5 * p.dk * sizeof(float);
    if (DK == 0) smem += (size_t)p.dk * block * sizeof(float);
    if (smem > 48 * 1024) {
        static size_t set_for = 0;
        if (smem > set_for) {
            ZL_CHECK_CUDA(cudaFuncSetAttribute(k_delta_rule<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            set_for = smem;
        }
    }
    ZL_CHECK_CUDA(launch(k_delta_rule<DK>, dim3(cdiv(p.dv, p.cols), p.H, runs), dim3(block), smem, st, pdl, p));
    return ZL_OK;
}

}  // namespace zl

using namespace zl;

extern "C" int zl_delta_rule_prepare(int dim_k, int dim_v) {
    ZL_CHECK_ARG(dim_k > 0 && dim_v > 0);
    // the generic kernel keeps its columns in shared memory: a warp of columns must fit beside the token vectors
    const size_t smem = ((size_t)kDrChunk * 5 * dim_k + (size_t)dim_k * 32) * sizeof(float);
    ZL_CHECK_SUPPORTED(smem <= 200 * 1024);
    return ZL_OK;
}

extern "C" int zl_delta_rule(const float* r, long long ld_r, const float* k, long long ld_k, const float* v, long long ld_v,
                             const float* rate_logit, long long ld_a, const float* decay_logit, long long ld_w,
                             float decay_scale, float unit_eps, const int32_t* run_row0, const int32_t* run_len, int runs,
                             const int32_t* slot, const int32_t* pos, void* const* state_addrs, float* o, long long ld_o,
                             int heads, int dim_k, int dim_v, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(r && k && v && rate_logit && decay_logit && run_row0 && run_len && slot && pos && state_addrs && o);
    ZL_CHECK_ARG(runs > 0 && runs <= 65535 && heads > 0 && heads <= 65535 && dim_k > 0 && dim_v > 0);
    DeltaP p{r, k, v, rate_logit, decay_logit, ld_r, ld_k, ld_v, ld_a, ld_w, run_row0, run_len, slot, pos, state_addrs, o, ld_o,
             heads, dim_k, dim_v, 0, decay_scale, unit_eps};
    // a warp of columns per CTA spreads one sequence over heads * dv / 32 CTAs
    p.cols = 32;
    const int block = 32;
    static const bool no_reg = getenv("ZL_DELTA_NO_REG") != nullptr;
    if (!no_reg && dim_k == 32) return launch_delta<32>(p, runs, block, pdl != 0, stream);
    if (!no_reg && dim_k == 64) return launch_delta<64>(p, runs, block, pdl != 0, stream);
    if (!no_reg && dim_k == 128) return launch_delta<128>(p, runs, block, pdl != 0, stream);
    if (zl_delta_rule_prepare(dim_k, dim_v) != ZL_OK) return ZL_ERR_UNSUPPORTED;
    return launch_delta<0>(p, runs, block, pdl != 0, stream);
}

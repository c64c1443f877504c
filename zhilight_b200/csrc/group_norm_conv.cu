// Token-wise pieces around the Linears of a layer that keeps its residual stream in fp32:
//   * RMS norm in groups: the vector is cut into `groups` equal consecutive parts, each divided by its own
//     sqrt(mean(part^2) + eps), the whole multiplied by a weight (groups == 1 is the plain RMSNorm of norm_rope.cu,
//     here with fp32 input);
//   * the same norm applied to a sublayer's output and added to the residual stream (post-norm);
//   * a short causal convolution over time, per channel, added to its own input, whose last taps-1 inputs per
//     sequence live in a per-slot ring next to the KV slots (the part of a sequence's state that is not attention);
//   * plain RMS norm of the low-rank query / key-value latents with the append of the latter to the slot's cache.
// Everything is computed in fp32; only the stores round to the activation dtype.
#include "common.cuh"

namespace zl {

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();   // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];   // same order in every thread: identical result
    return s;
}

// grid (groups, T)
template <typename TO>
__global__ void k_group_rmsnorm(const float* __restrict__ x, long long ldx, const float* __restrict__ w,
                                TO* __restrict__ y, long long ldy, int gs, float eps) {
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int c0 = blockIdx.x * gs;
    const float* xr = x + (size_t)blockIdx.y * ldx + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)gs + eps);
    TO* yr = y + (size_t)blockIdx.y * ldy + c0;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) yr[i] = from_f32<TO>(xr[i] * r * w[c0 + i]);
}

// 1 / sqrt(mean(row[g*gs .. +gs)^2) + eps), computed by the whole CTA (the same order of sums in every CTA)
__device__ __forceinline__ float group_inv_rms(const float* __restrict__ row, int g, int gs, float eps, float* red) {
    const float* xr = row + (size_t)g * gs;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    return 1.0f / sqrtf(block_sum(ss, red) / (float)gs + eps);
}

// x[t] += gnorm(y[t]) * w; optionally h[t] -> ring[slot][pos % (taps-1)] for the rows that are among the last taps-1 of
// their sequence in this step (rows of one sequence are consecutive, so row t + taps-1 tells).
// grid (ceil(D / blockDim), T): a CTA owns blockDim channels and computes the sums of the groups they lie in itself.
__global__ void k_group_rmsnorm_residual(const float* __restrict__ y, long long ldy, const float* __restrict__ w,
                                         float* __restrict__ x, long long ldx, int gs, float eps,
                                         const float* __restrict__ h, long long ldh, const int32_t* __restrict__ slot,
                                         const int32_t* __restrict__ pos, float* __restrict__ ring, int keep, int T, int D) {
    __shared__ float red[32];
    extern __shared__ float inv[];   // one per group that meets this CTA's channels
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, c0 = blockIdx.x * blockDim.x, c = c0 + threadIdx.x;
    const int g_lo = c0 / gs, g_hi = min(D - 1, c0 + (int)blockDim.x - 1) / gs;
    const float* yr = y + (size_t)t * ldy;
    for (int g = g_lo; g <= g_hi; ++g) {
        const float r = group_inv_rms(yr, g, gs, eps, red);
        if (threadIdx.x == 0) inv[g - g_lo] = r;
    }
    __syncthreads();
    if (c >= D) return;
    x[(size_t)t * ldx + c] += yr[c] * inv[c / gs - g_lo] * w[c];
    if (ring && keep > 0) {
        const int s = slot[t];
        const bool later = t + keep < T && slot[t + keep] == s;   // a row of this sequence keep steps on overwrites it
        if (!later) ring[((size_t)s * keep + (pos[t] % keep)) * D + c] = h[(size_t)t * ldh + c];
    }
}

// u[t] = h[t] + sum_j wt[c][j] * h_at(pos[t] - (taps-1) + j); the input at an earlier position comes from this step's
// rows when the sequence brought it in this step, from the slot's ring otherwise, and is zero before the sequence's start.
template <typename TO>
__global__ void k_causal_conv_mix(const float* __restrict__ h, long long ldh, const float* __restrict__ wt,
                                  const int32_t* __restrict__ slot, const int32_t* __restrict__ pos,
                                  const float* __restrict__ ring, TO* __restrict__ u, long long ldu, int D, int taps) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= D) return;
    const int s = slot[t], p = pos[t], keep = taps - 1;
    const float cur = h[(size_t)t * ldh + c];
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = keep - j, q = p - back;
        float v;
        if (back == 0) v = cur;
        else if (q < 0) v = 0.f;
        else if (t - back >= 0 && slot[t - back] == s && pos[t - back] == q) v = h[(size_t)(t - back) * ldh + c];
        else v = ring[((size_t)s * keep + (q % keep)) * D + c];
        acc = fmaf(wt[(size_t)c * taps + j], v, acc);
    }
    u[(size_t)t * ldu + c] = from_f32<TO>(cur + acc);
}


// The pre-norm and the convolution in one pass: h[t] = gnorm(x[t]) * w, u[t] = h[t] + conv.  The norm is per row, so the
// earlier rows the convolution needs are normalised again here when they are rows of this step (the same arithmetic as
// in their own CTA, hence the same values); otherwise they come from the slot's ring.
// grid (ceil(D / blockDim), T); dynamic shared memory: taps * (groups that meet the CTA's channels) inverse RMS values.
template <typename TO>
__global__ void k_group_norm_conv(const float* __restrict__ x, long long ldx, const float* __restrict__ w,
                                  const float* __restrict__ wt, const int32_t* __restrict__ slot,
                                  const int32_t* __restrict__ pos, const float* __restrict__ ring, float* __restrict__ h,
                                  TO* __restrict__ u, int D, int gs, int taps, float eps) {
    __shared__ float red[32];
    extern __shared__ float inv[];   // [taps][ng]; entry < 0: that row is not in this step
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, s = slot[t], p = pos[t], keep = taps - 1;
    const int c0 = blockIdx.x * blockDim.x, c = c0 + threadIdx.x;
    const int g_lo = c0 / gs, g_hi = min(D - 1, c0 + (int)blockDim.x - 1) / gs, ng = g_hi - g_lo + 1;
    for (int back = 0; back < taps; ++back) {
        const bool here = back == 0 || (t - back >= 0 && slot[t - back] == s && pos[t - back] == p - back);   // CTA-uniform
        for (int g = g_lo; g <= g_hi; ++g) {
            const float r = here ? group_inv_rms(x + (size_t)(t - back) * ldx, g, gs, eps, red) : -1.f;
            if (threadIdx.x == 0) inv[back * ng + g - g_lo] = r;
        }
    }
    __syncthreads();
    if (c >= D) return;
    const int g = c / gs - g_lo;
    const float wc = w[c];
    const float cur = x[(size_t)t * ldx + c] * inv[g] * wc;
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = keep - j, q = p - back;
        float v;
        if (back == 0) v = cur;
        else if (q < 0) v = 0.f;
        else if (inv[back * ng + g] >= 0.f) v = x[(size_t)(t - back) * ldx + c] * inv[back * ng + g] * wc;
        else v = ring[((size_t)s * keep + (q % keep)) * D + c];
        acc = fmaf(wt[(size_t)c * taps + j], v, acc);
    }
    h[(size_t)t * D + c] = cur;
    u[(size_t)t * D + c] = from_f32<TO>(cur + acc);
}

// grid (2, T): part 0 = query latent -> cq[t]; part 1 = key-value latent -> cache row (slot[t], pos[t])
template <typename TO>
__global__ void k_latent_norm_append(const float* __restrict__ proj, long long ldp, int q_off, int q_rank,
                                     const float* __restrict__ wq, TO* __restrict__ cq, int c_off, int kv_rank,
                                     const float* __restrict__ wkv, void* const* __restrict__ slot_addrs,
                                     const int32_t* __restrict__ slot, const int32_t* __restrict__ pos, float eps) {
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const bool kv = blockIdx.x == 1;
    if (kv && !wkv) return;
    const int n = kv ? kv_rank : q_rank;
    const float* src = proj + (size_t)t * ldp + (kv ? c_off : q_off);
    const float* w = kv ? wkv : wq;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = src[i];
        ss = fmaf(v, v, ss);
    }
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    TO* dst = kv ? static_cast<TO*>(slot_addrs[slot[t]]) + (size_t)pos[t] * kv_rank : cq + (size_t)t * q_rank;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = from_f32<TO>(src[i] * r * w[i]);
}

// channels per CTA of the row-parallel kernels: a row is spread over several CTAs so that a decode step of one token
// still fills more than one SM
static int row_chunk(int D) { return D >= 2048 ? 256 : (D >= 256 ? 128 : 64); }

static int norm_threads(int n) {
    int th = 32;
    while (th < 256 && th * 4 < n) th <<= 1;
    return th;
}

}  // namespace zl

using namespace zl;

extern "C" int zl_group_rmsnorm(const float* x, long long ldx, const float* weight, void* y, long long ldy, int T, int D,
                                int groups, float eps, int out_dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(x && weight && y && T > 0 && D > 0 && groups > 0 && D % groups == 0 && T <= 65535);
    ZL_CHECK_ARG(out_dtype == ZL_F16 || out_dtype == ZL_BF16 || out_dtype == ZL_F32);
    const int gs = D / groups;
    const dim3 grid(groups, T), block(norm_threads(gs));
    cudaError_t e;
    if (out_dtype == ZL_F32)
        e = launch(k_group_rmsnorm<float>, grid, block, 0, stream, pdl != 0, x, ldx, weight, static_cast<float*>(y), ldy, gs, eps);
    else if (out_dtype == ZL_BF16)
        e = launch(k_group_rmsnorm<__nv_bfloat16>, grid, block, 0, stream, pdl != 0, x, ldx, weight,
                   static_cast<__nv_bfloat16*>(y), ldy, gs, eps);
    else
        e = launch(k_group_rmsnorm<__half>, grid, block, 0, stream, pdl != 0, x, ldx, weight, static_cast<__half*>(y), ldy, gs, eps);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_group_rmsnorm_residual(const float* y, long long ldy, const float* weight, float* x, long long ldx, int T,
                                         int D, int groups, float eps, const float* conv_in, long long ld_conv_in,
                                         const int32_t* slot, const int32_t* pos, float* ring, int taps, int pdl,
                                         zl_stream_t stream) {
    ZL_CHECK_ARG(y && weight && x && T > 0 && D > 0 && groups > 0 && D % groups == 0 && T <= 65535);
    ZL_CHECK_ARG(!ring || (conv_in && slot && pos && taps >= 1));
    const int gs = D / groups, th = row_chunk(D);
    const size_t smem = sizeof(float) * (size_t)((th - 1) / gs + 2);
    ZL_CHECK_CUDA(launch(k_group_rmsnorm_residual, dim3(cdiv(D, th), T), dim3(th), smem, stream, pdl != 0, y, ldy, weight, x, ldx,
                         gs, eps, conv_in, ld_conv_in, slot, pos, ring, ring ? taps - 1 : 0, T, D));
    return ZL_OK;
}

extern "C" int zl_causal_conv_mix(const float* h, long long ldh, const float* taps_weight, const int32_t* slot,
                                  const int32_t* pos, const float* ring, void* u, long long ldu, int T, int D, int taps,
                                  int out_dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(h && taps_weight && slot && pos && u && T > 0 && D > 0 && taps >= 1 && T <= 65535);
    ZL_CHECK_ARG(taps == 1 || ring);
    ZL_CHECK_ARG(out_dtype == ZL_F16 || out_dtype == ZL_BF16 || out_dtype == ZL_F32);
    const dim3 grid(cdiv(D, 128), T), block(128);
    cudaError_t e;
    if (out_dtype == ZL_F32)
        e = launch(k_causal_conv_mix<float>, grid, block, 0, stream, pdl != 0, h, ldh, taps_weight, slot, pos, ring,
                   static_cast<float*>(u), ldu, D, taps);
    else if (out_dtype == ZL_BF16)
        e = launch(k_causal_conv_mix<__nv_bfloat16>, grid, block, 0, stream, pdl != 0, h, ldh, taps_weight, slot, pos, ring,
                   static_cast<__nv_bfloat16*>(u), ldu, D, taps);
    else
        e = launch(k_causal_conv_mix<__half>, grid, block, 0, stream, pdl != 0, h, ldh, taps_weight, slot, pos, ring,
                   static_cast<__half*>(u), ldu, D, taps);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_group_norm_conv(const float* x, long long ldx, const float* norm_weight, const float* taps_weight,
                                  const int32_t* slot, const int32_t* pos, const float* ring, float* h, void* u, int T, int D,
                                  int groups, int taps, float eps, int out_dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(x && norm_weight && taps_weight && slot && pos && h && u && T > 0 && D > 0 && taps >= 1);
    ZL_CHECK_ARG(groups > 0 && D % groups == 0 && (taps == 1 || ring));
    ZL_CHECK_ARG(out_dtype == ZL_F16 || out_dtype == ZL_BF16 || out_dtype == ZL_F32);
    const int gs = D / groups, th = row_chunk(D);
    const size_t smem = sizeof(float) * (size_t)taps * ((th - 1) / gs + 2);
    ZL_CHECK_SUPPORTED(smem <= 40 * 1024 && T <= 65535);
    const dim3 grid(cdiv(D, th), T), block(th);
    cudaError_t e;
    if (out_dtype == ZL_F32)
        e = launch(k_group_norm_conv<float>, grid, block, smem, stream, pdl != 0, x, ldx, norm_weight, taps_weight, slot, pos,
                   ring, h, static_cast<float*>(u), D, gs, taps, eps);
    else if (out_dtype == ZL_BF16)
        e = launch(k_group_norm_conv<__nv_bfloat16>, grid, block, smem, stream, pdl != 0, x, ldx, norm_weight, taps_weight, slot,
                   pos, ring, h, static_cast<__nv_bfloat16*>(u), D, gs, taps, eps);
    else
        e = launch(k_group_norm_conv<__half>, grid, block, smem, stream, pdl != 0, x, ldx, norm_weight, taps_weight, slot, pos,
                   ring, h, static_cast<__half*>(u), D, gs, taps, eps);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_latent_norm_append(const float* proj, long long ldp, int q_off, int q_rank, const float* q_weight, void* cq,
                                     int c_off, int kv_rank, const float* kv_weight, void* const* slot_addrs,
                                     const int32_t* slot, const int32_t* pos, int T, float eps, int dtype, int pdl,
                                     zl_stream_t stream) {
    ZL_CHECK_ARG(proj && q_weight && cq && q_rank > 0 && T > 0 && T <= 65535);
    ZL_CHECK_ARG(!kv_weight || (slot_addrs && slot && pos && kv_rank > 0));
    ZL_CHECK_ARG(dtype == ZL_F16 || dtype == ZL_BF16 || dtype == ZL_F32);
    const int big = q_rank > kv_rank ? q_rank : kv_rank;
    const dim3 grid(kv_weight ? 2 : 1, T), block(norm_threads(big));
    cudaError_t e;
    if (dtype == ZL_F32)
        e = launch(k_latent_norm_append<float>, grid, block, 0, stream, pdl != 0, proj, ldp, q_off, q_rank, q_weight,
                   static_cast<float*>(cq), c_off, kv_rank, kv_weight, slot_addrs, slot, pos, eps);
    else if (dtype == ZL_BF16)
        e = launch(k_latent_norm_append<__nv_bfloat16>, grid, block, 0, stream, pdl != 0, proj, ldp, q_off, q_rank, q_weight,
                   static_cast<__nv_bfloat16*>(cq), c_off, kv_rank, kv_weight, slot_addrs, slot, pos, eps);
    else
        e = launch(k_latent_norm_append<__half>, grid, block, 0, stream, pdl != 0, proj, ldp, q_off, q_rank, q_weight,
                   static_cast<__half*>(cq), c_off, kv_rank, kv_weight, slot_addrs, slot, pos, eps);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

// Token-wise pieces of mixers that work per head, all in fp32 (rotation angles in double) with stores rounded to the
// activation dtype:
//   * the step from a fused q | k | v projection row to attention operands: RMS norm per head over the head size with a
//     weight shared by the heads (queries, keys), a weightless RMS norm of every value head, a rotation of the first
//     `rot_dims` dimensions of queries and keys in adjacent pairs (2i, 2i+1) by pos * inv_freq[i] with cos / sin scaled
//     by `mscale` (the frequencies are a table, so any scaling rule is the caller's), and the append of keys and values
//     to the slot's caches;
//   * RMS norm per head of a mixer's output with a full-width weight and a sigmoid gate;
//   * the weighted sum of several parts per token (the chosen experts' outputs), RMS norm, residual add.
#include "common.cuh"

#include <cmath>

namespace zl {

struct QkvPrepP {
    const float* proj;
    long long ldp;
    int q_off, k_off, v_off;   // k_off < 0: the layer has no keys / values of its own
    int H, G, d, vd, rot_dims;
    const float *q_w, *k_w;
    const double* inv_freq;
    float mscale, eps;
    void* q_out;               // (T, H * d)
    void* const* k_addrs;      // slot -> (max_seq, G, d)
    void* const* v_addrs;      // slot -> (max_seq, G, vd)
    const int32_t *slot, *pos;
};

// one warp per (token, unit); units: H query heads, then G key heads, then G value heads.  grid (ceil(units / 4), T)
template <typename TO>
__global__ void __launch_bounds__(128) k_qkv_headnorm_rope_append(QkvPrepP p) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + warp;
    const int units = p.H + (p.k_off >= 0 ? 2 * p.G : 0);
    if (unit >= units) return;
    const float* row = p.proj + (size_t)t * p.ldp;
    const int pos = p.pos[t];
    const float* src;
    const float* w;
    TO* dst;
    int n;
    bool rotate;
    if (unit < p.H) {
        src = row + p.q_off + (size_t)unit * p.d;
        w = p.q_w;
        n = p.d;
        rotate = true;
        dst = static_cast<TO*>(p.q_out) + ((size_t)t * p.H + unit) * p.d;
    } else if (unit < p.H + p.G) {
        const int g = unit - p.H;
        src = row + p.k_off + (size_t)g * p.d;
        w = p.k_w;
        n = p.d;
        rotate = true;
        dst = static_cast<TO*>(p.k_addrs[p.slot[t]]) + ((size_t)pos * p.G + g) * p.d;
    } else {
        const int g = unit - p.H - p.G;
        src = row + p.v_off + (size_t)g * p.vd;
        w = nullptr;
        n = p.vd;
        rotate = false;
        dst = static_cast<TO*>(p.v_addrs[p.slot[t]]) + ((size_t)pos * p.G + g) * p.vd;
    }
    float ss = 0.f;
    for (int c = lane; c < n; c += 32) ss = fmaf(src[c], src[c], ss);
    const float r = 1.0f / sqrtf(warp_sum(ss) / (float)n + p.eps);
    const int rot = rotate ? p.rot_dims : 0;
    // rotated pairs: lane handles pair i = (2i, 2i + 1)
    for (int i = lane; 2 * i < rot; i += 32) {
        const float u = src[2 * i] * r * w[2 * i], v = src[2 * i + 1] * r * w[2 * i + 1];
        // the angle and its cos / sin in double: at position 1000 a float angle is already off by 3e-5 rad, which a sharp
        // score multiplies; rot_dims / 2 evaluations per head cost nothing beside the projections
        double sd, cd;
        sincos((double)pos * p.inv_freq[i], &sd, &cd);
        const float cs = (float)(cd * (double)p.mscale), sn = (float)(sd * (double)p.mscale);
        dst[2 * i] = from_f32<TO>(u * cs - v * sn);
        dst[2 * i + 1] = from_f32<TO>(v * cs + u * sn);
    }
    for (int c = rot + lane; c < n; c += 32) dst[c] = from_f32<TO>(src[c] * r * (w ? w[c] : 1.0f));
}

// y[t][h*dv + c] = o / sqrt(mean_c(o^2) + eps) * w[h*dv + c] * sigmoid(gate[t][h*dv + c]); one warp per (token, head)
template <typename TO>
__global__ void __launch_bounds__(128) k_head_rmsnorm_gate(const float* __restrict__ o, long long ldo,
                                                           const float* __restrict__ w, const float* __restrict__ gate,
                                                           long long ldg, TO* __restrict__ y, long long ldy, int H, int dv,
                                                           float eps) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= H) return;
    const float* src = o + (size_t)t * ldo + (size_t)h * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(src[c], src[c], ss);
    const float r = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        float v = src[c] * r;
        if (w) v *= w[(size_t)h * dv + c];
        if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + (size_t)h * dv + c]));
        y[(size_t)t * ldy + (size_t)h * dv + c] = from_f32<TO>(v);
    }
}

// x[t] += w * s / sqrt(mean(s^2) + eps) with s = sum_p coef[t][p] * parts[t * n_parts + p]; the parts are added in the
// order of p; the new x also goes out rounded to the activation dtype for the next Linear.  One CTA per token.
template <typename TO>
__global__ void __launch_bounds__(256) k_rmsnorm_residual_combine(const float* __restrict__ parts, long long ldp,
                                                                  const float* __restrict__ coef, int n_parts,
                                                                  const float* __restrict__ w, float* __restrict__ x,
                                                                  long long ldx, TO* __restrict__ x_act, int D, float eps,
                                                                  int vec) {
    __shared__ float red[8];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float* pr = parts + (size_t)t * n_parts * ldp;
    const float* cf = coef ? coef + (size_t)t * n_parts : nullptr;
    // vec: D % 4 == 0, D <= 4096, 16-byte aligned rows: every thread keeps its (up to four) 4-channel sums in registers
    float4 keep[4];
    float ss = 0.f;
    if (vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c4 = threadIdx.x + i * 256;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c4 * 4 < D)
                for (int q = 0; q < n_parts; ++q) {
                    const float a = cf ? cf[q] : 1.0f;
                    const float4 v = *reinterpret_cast<const float4*>(pr + (size_t)q * ldp + c4 * 4);
                    s.x = fmaf(a, v.x, s.x), s.y = fmaf(a, v.y, s.y), s.z = fmaf(a, v.z, s.z), s.w = fmaf(a, v.w, s.w);
                }
            keep[i] = s;
            ss = fmaf(s.x, s.x, fmaf(s.y, s.y, fmaf(s.z, s.z, fmaf(s.w, s.w, ss))));
        }
    } else {
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            float s = 0.f;
            for (int q = 0; q < n_parts; ++q) s = fmaf(cf ? cf[q] : 1.0f, pr[(size_t)q * ldp + c], s);
            ss = fmaf(s, s, ss);
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
    const float r = 1.0f / sqrtf(tot / (float)D + eps);
    if (vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = (threadIdx.x + i * 256) * 4;
            if (c >= D) continue;
            const float4 wv = *reinterpret_cast<const float4*>(w + c);
            float4 xv = *reinterpret_cast<float4*>(x + (size_t)t * ldx + c);
            xv.x += keep[i].x * r * wv.x, xv.y += keep[i].y * r * wv.y, xv.z += keep[i].z * r * wv.z, xv.w += keep[i].w * r * wv.w;
            *reinterpret_cast<float4*>(x + (size_t)t * ldx + c) = xv;
            if (x_act) {
                x_act[(size_t)t * D + c] = from_f32<TO>(xv.x), x_act[(size_t)t * D + c + 1] = from_f32<TO>(xv.y);
                x_act[(size_t)t * D + c + 2] = from_f32<TO>(xv.z), x_act[(size_t)t * D + c + 3] = from_f32<TO>(xv.w);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float s = 0.f;
        for (int q = 0; q < n_parts; ++q) s = fmaf(cf ? cf[q] : 1.0f, pr[(size_t)q * ldp + c], s);
        const float nx = x[(size_t)t * ldx + c] + s * r * w[c];
        x[(size_t)t * ldx + c] = nx;
        if (x_act) x_act[(size_t)t * D + c] = from_f32<TO>(nx);
    }
}

}  // namespace zl

using namespace zl;

extern "C" int zl_qkv_headnorm_rope_append(const float* proj, long long ldp, int q_off, int k_off, int v_off, int heads,
                                           int kv_heads, int dim, int vdim, const float* q_weight, const float* k_weight,
                                           const double* inv_freq, int rot_dims, float mscale, float eps, void* q_out,
                                           void* const* k_addrs, void* const* v_addrs, const int32_t* slot,
                                           const int32_t* pos, int T, int dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(proj && q_weight && q_out && slot && pos && T > 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0);
    ZL_CHECK_ARG(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq));
    ZL_CHECK_ARG(k_off < 0 || (k_weight && k_addrs && v_addrs && v_off >= 0));
    ZL_CHECK_ARG(dtype == ZL_F16 || dtype == ZL_BF16 || dtype == ZL_F32);
    QkvPrepP p{proj, ldp, q_off, k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, q_weight, k_weight, inv_freq,
               mscale, eps, q_out, k_addrs, v_addrs, slot, pos};
    const int units = heads + (k_off >= 0 ? 2 * kv_heads : 0);
    const dim3 grid(cdiv(units, 4), T), block(128);
    cudaError_t e;
    if (dtype == ZL_F32) e = launch(k_qkv_headnorm_rope_append<float>, grid, block, 0, stream, pdl != 0, p);
    else if (dtype == ZL_BF16) e = launch(k_qkv_headnorm_rope_append<__nv_bfloat16>, grid, block, 0, stream, pdl != 0, p);
    else e = launch(k_qkv_headnorm_rope_append<__half>, grid, block, 0, stream, pdl != 0, p);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_head_rmsnorm_gate(const float* o, long long ldo, const float* weight, const float* gate, long long ldg,
                                    void* y, long long ldy, int T, int heads, int vdim, float eps, int out_dtype, int pdl,
                                    zl_stream_t stream) {
    ZL_CHECK_ARG(o && y && T > 0 && heads > 0 && vdim > 0);
    ZL_CHECK_ARG(out_dtype == ZL_F16 || out_dtype == ZL_BF16 || out_dtype == ZL_F32);
    const dim3 grid(cdiv(heads, 4), T), block(128);
    cudaError_t e;
    if (out_dtype == ZL_F32)
        e = launch(k_head_rmsnorm_gate<float>, grid, block, 0, stream, pdl != 0, o, ldo, weight, gate, ldg, (float*)y, ldy, heads,
                   vdim, eps);
    else if (out_dtype == ZL_BF16)
        e = launch(k_head_rmsnorm_gate<__nv_bfloat16>, grid, block, 0, stream, pdl != 0, o, ldo, weight, gate, ldg,
                   (__nv_bfloat16*)y, ldy, heads, vdim, eps);
    else
        e = launch(k_head_rmsnorm_gate<__half>, grid, block, 0, stream, pdl != 0, o, ldo, weight, gate, ldg, (__half*)y, ldy,
                   heads, vdim, eps);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_rmsnorm_residual_combine(const float* parts, long long ldp, const float* coef, int n_parts,
                                           const float* weight, float* x, long long ldx, void* x_act, int act_dtype, int T,
                                           int D, float eps, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(parts && weight && x && n_parts > 0 && T > 0 && D > 0 && ldp >= D && ldx >= D);
    ZL_CHECK_ARG(!x_act || act_dtype == ZL_F16 || act_dtype == ZL_BF16);
    cudaError_t e;
    const int vec = D % 4 == 0 && D <= 4096 && ldp % 4 == 0 && ldx % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(parts) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight)) & 15) == 0;
    if (x_act && act_dtype == ZL_F16)
        e = launch(k_rmsnorm_residual_combine<__half>, dim3(T), dim3(256), 0, stream, pdl != 0, parts, ldp, coef, n_parts, weight,
                   x, ldx, (__half*)x_act, D, eps, vec);
    else
        e = launch(k_rmsnorm_residual_combine<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, pdl != 0, parts, ldp, coef, n_parts,
                   weight, x, ldx, (__nv_bfloat16*)x_act, D, eps, vec);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_rope_inv_freq_yarn(double base, int dims, double factor, double original, double fast, double slow,
                                     double* out, float* mscale) {
    ZL_CHECK_ARG(base > 1.0 && dims >= 0 && dims % 2 == 0 && (dims == 0 || out));
    const int half = dims / 2;
    const double kPi = 3.14159265358979323846;
    double lo = 0, hi = 0;
    if (factor > 0) {
        ZL_CHECK_ARG(original > 0 && fast > 0 && slow > 0);
        auto dim_of = [&](double turns) { return dims * log(original / (2 * kPi * turns)) / (2 * log(base)); };
        lo = fmax(floor(dim_of(fast)), 0.0);
        hi = fmin(ceil(dim_of(slow)), (double)(dims - 1));
    }
    for (int i = 0; i < half; ++i) {
        double f = pow(base, -2.0 * i / dims);
        if (factor > 0) {
            const double ramp = fmin(fmax((i - lo) / fmax(hi - lo, 0.001), 0.0), 1.0);
            f = f / factor * ramp + f * (1 - ramp);
        }
        out[i] = f;
    }
    if (mscale) *mscale = factor > 0 ? (float)(0.1 * log(factor) + 1.0) : 1.0f;
    return ZL_OK;
}

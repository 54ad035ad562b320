// Token-wise pieces of mixers that work per head, all in fp32 (rotation angles in double) with stores rounded to the
// activation dtype:
//   * the step from a fused q | k | v projection row to attention operands: RMS norm per head over the head size with a
//     weight shared by the heads (queries, keys), a weightless RMS norm of every value head, a rotation of the first
//     `rot_dims` dimensions of queries and keys in adjacent pairs (2i, 2i+1) by pos * inv_freq[i] with cos / sin scaled
//     by `mscale` (the frequencies are a table, so any scaling rule is the caller's), and the append of keys and values
//     to the slot's caches;
//   * RMS norm per head of a mixer's output with a full-width weight and a sigmoid gate;
//   * the weighted sum of several parts per token (the chosen experts' outputs), RMS norm, residual add;
//   * RMS norm of queries and keys over the whole projection (all heads at once, a weight of that size), the unnormed key
//     projection kept as the value, and the append to the slot's caches;
//   * the mixes of a token with its predecessor, x + (x_prev - x) * mu_s for several coefficient vectors mu_s at once (the
//     predecessor is the previous row of the run or the slot's stored last token);
//   * norm after the sum: x <- w * rms(alpha x + c_a a + c_b b);
//   * rotations from a per-step (cos, sin) table: queries and keys over their first rot_dims dimensions and values over
//     all of theirs, pairs in halves or adjacent, no norms, with the append to the slot's caches;
//   * the residual update of a parallel layer: both sublayers' results times a layer scale and a sigmoid gate per channel,
//     the second a weighted sum of parts of which some may be the sublayers' input itself, then the next layer's norm.
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

// y[t][h*dv + c] = o / sqrt(mean_c(o^2) + eps) * w[h*w_stride + c] * f(gate[t][h*dv + c]); f = sigmoid, or silu (gate_silu);
// one warp per (token, head)
template <typename TO>
__global__ void __launch_bounds__(128) k_head_rmsnorm_gate(const float* __restrict__ o, long long ldo,
                                                           const float* __restrict__ w, const float* __restrict__ gate,
                                                           long long ldg, TO* __restrict__ y, long long ldy, int H, int dv,
                                                           float eps, int w_stride, int gate_silu) {
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
        if (w) v *= w[(size_t)h * w_stride + c];
        if (gate) {
            const float gl = gate[(size_t)t * ldg + (size_t)h * dv + c], sg = 1.0f / (1.0f + expf(-gl));
            v *= gate_silu ? gl * sg : sg;
        }
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

// grid (T, 2).  CTA (t, 0): q <- rms(q over all H*d) * q_w -> q_out.  CTA (t, 1): k <- rms(k over all G*d) * k_w -> key cache
// row; the projected k itself -> value cache row.  A thread keeps up to 8 of its values in registers between the two passes.
template <typename TO>
__global__ void __launch_bounds__(512) k_qk_fullnorm_append(const float* __restrict__ proj, long long ldp, int q_off, int k_off,
                                                            int nq, int nk, const float* __restrict__ q_w,
                                                            const float* __restrict__ k_w, float eps, TO* __restrict__ q_out,
                                                            void* const* k_addrs, void* const* v_addrs,
                                                            const int32_t* __restrict__ slot, const int32_t* __restrict__ pos) {
    __shared__ float red[16];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const bool keys = blockIdx.y == 1;
    const int n = keys ? nk : nq;
    const float* src = proj + (size_t)t * ldp + (keys ? k_off : q_off);
    const float* w = keys ? k_w : q_w;
    float keep[8], ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * 512;
        keep[i] = c < n ? src[c] : 0.f;
        ss = fmaf(keep[i], keep[i], ss);
    }
    for (int c = threadIdx.x + 8 * 512; c < n; c += 512) ss = fmaf(src[c], src[c], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < 16; ++i) tot += red[i];
    const float r = 1.0f / sqrtf(tot / (float)n + eps);
    TO* dst = keys ? static_cast<TO*>(k_addrs[slot[t]]) + (size_t)pos[t] * nk : q_out + (size_t)t * nq;
    TO* vd = keys ? static_cast<TO*>(v_addrs[slot[t]]) + (size_t)pos[t] * nk : nullptr;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * 512;
        if (c < n) {
            dst[c] = from_f32<TO>(keep[i] * r * w[c]);
            if (keys) vd[c] = from_f32<TO>(keep[i]);
        }
    }
    for (int c = threadIdx.x + 8 * 512; c < n; c += 512) {
        dst[c] = from_f32<TO>(src[c] * r * w[c]);
        if (keys) vd[c] = from_f32<TO>(src[c]);
    }
}

// out[s][t] = x[t] + (prev - x[t]) * mu[s], s < n_mix; prev = x[t - 1] when that row belongs to the same sequence, zeros at
// position 0, else the slot's stored last token.  store_state: every row is a run of its own, so the kernel also stores
// x[t] as the slot's last token (otherwise the caller stores the runs' tails afterwards).  grid (T, ceil(D / (256 * V)));
// a thread owns V consecutive channels (V = 4 when the rows are 16-byte aligned), read once and written n_mix times.
template <typename TO, int V>
__global__ void __launch_bounds__(256) k_token_shift_mix(const float* __restrict__ x, long long ldx, const float* __restrict__ mu,
                                                         int n_mix, void* const* state_addrs, const int32_t* __restrict__ slot,
                                                         const int32_t* __restrict__ pos, TO* __restrict__ out, long long out_stride,
                                                         int D, int store_state) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, sl = slot[t], c = (blockIdx.y * 256 + threadIdx.x) * V;
    if (c >= D) return;
    const bool in_step = t > 0 && slot[t - 1] == sl, first = pos[t] == 0;
    float* st = static_cast<float*>(state_addrs[sl]);
    const float* xr = x + (size_t)t * ldx;
    float cur[V], dx[V];
    if constexpr (V == 4) {
        const float4 cv = *reinterpret_cast<const float4*>(xr + c);
        float4 pv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in_step) pv = *reinterpret_cast<const float4*>(xr + c - ldx);
        else if (!first) pv = *reinterpret_cast<const float4*>(st + c);
        cur[0] = cv.x, cur[1] = cv.y, cur[2] = cv.z, cur[3] = cv.w;
        dx[0] = pv.x - cv.x, dx[1] = pv.y - cv.y, dx[2] = pv.z - cv.z, dx[3] = pv.w - cv.w;
        if (store_state) *reinterpret_cast<float4*>(st + c) = cv;
    } else {
        cur[0] = xr[c];
        dx[0] = (in_step ? xr[c - ldx] : (first ? 0.f : st[c])) - cur[0];
        if (store_state) st[c] = cur[0];
    }
#pragma unroll 5
    for (int s = 0; s < n_mix; ++s) {
        TO* o = out + (size_t)s * out_stride + (size_t)t * D + c;
        if constexpr (V == 4) {
            const float4 m = *reinterpret_cast<const float4*>(mu + (size_t)s * D + c);
            o[0] = from_f32<TO>(fmaf(dx[0], m.x, cur[0])), o[1] = from_f32<TO>(fmaf(dx[1], m.y, cur[1]));
            o[2] = from_f32<TO>(fmaf(dx[2], m.z, cur[2])), o[3] = from_f32<TO>(fmaf(dx[3], m.w, cur[3]));
        } else {
            o[0] = from_f32<TO>(fmaf(dx[0], mu[(size_t)s * D + c], cur[0]));
        }
    }
}

// one CTA per token: x <- w * s / sqrt(mean(s^2) + eps), s = alpha x + ca a + cb b (b may be null); also x rounded to TO.
// vec: D % 4 == 0, D <= 4096, 16-byte aligned rows: every thread keeps its (up to four) 4-channel sums in registers;
// otherwise the sums wait in shared memory (D floats).
template <typename TO>
__global__ void __launch_bounds__(256) k_postnorm_combine(float* __restrict__ x, long long ldx, float alpha,
                                                          const float* __restrict__ a, long long lda, float ca,
                                                          const float* __restrict__ b, long long ldb, float cb,
                                                          const float* __restrict__ w, TO* __restrict__ x_act, int D, float eps,
                                                          int vec) {
    extern __shared__ float psm[];   // D when !vec
    __shared__ float red[8];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    float ss = 0.f;
    float4 keep[4];
    if (vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = (threadIdx.x + i * 256) * 4;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < D) {
                const float4 xv = *reinterpret_cast<const float4*>(x + (size_t)t * ldx + c);
                const float4 av = *reinterpret_cast<const float4*>(a + (size_t)t * lda + c);
                s.x = fmaf(ca, av.x, alpha * xv.x), s.y = fmaf(ca, av.y, alpha * xv.y);
                s.z = fmaf(ca, av.z, alpha * xv.z), s.w = fmaf(ca, av.w, alpha * xv.w);
                if (b) {
                    const float4 bv = *reinterpret_cast<const float4*>(b + (size_t)t * ldb + c);
                    s.x = fmaf(cb, bv.x, s.x), s.y = fmaf(cb, bv.y, s.y), s.z = fmaf(cb, bv.z, s.z), s.w = fmaf(cb, bv.w, s.w);
                }
            }
            keep[i] = s;
            ss = fmaf(s.x, s.x, fmaf(s.y, s.y, fmaf(s.z, s.z, fmaf(s.w, s.w, ss))));
        }
    } else {
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            float s = fmaf(ca, a[(size_t)t * lda + c], alpha * x[(size_t)t * ldx + c]);
            if (b) s = fmaf(cb, b[(size_t)t * ldb + c], s);
            psm[c] = s;
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
            const float4 nx = make_float4(keep[i].x * r * wv.x, keep[i].y * r * wv.y, keep[i].z * r * wv.z, keep[i].w * r * wv.w);
            *reinterpret_cast<float4*>(x + (size_t)t * ldx + c) = nx;
            if (x_act) {
                x_act[(size_t)t * D + c] = from_f32<TO>(nx.x), x_act[(size_t)t * D + c + 1] = from_f32<TO>(nx.y);
                x_act[(size_t)t * D + c + 2] = from_f32<TO>(nx.z), x_act[(size_t)t * D + c + 3] = from_f32<TO>(nx.w);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float nx = psm[c] * r * w[c];
        x[(size_t)t * ldx + c] = nx;
        if (x_act) x_act[(size_t)t * D + c] = from_f32<TO>(nx);
    }
}

// table[t][i] = (cos, sin)(pos[t] * inv_freq[i]): the angle and its functions in double (at position 1000 a float angle is
// already off by 3e-5 rad), once per step for every kernel that turns by these angles
__global__ void __launch_bounds__(256) k_rope_table(const int32_t* __restrict__ pos, const double* __restrict__ inv_freq,
                                                    float2* __restrict__ table, int T, int half) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * half) return;
    const int t = i / half;
    double sd, cd;
    sincos((double)pos[t] * inv_freq[i - t * half], &sd, &cd);
    table[i] = make_float2((float)cd, (float)sd);
}

struct QkvRopeP {
    const float* proj;
    long long ldp;
    int q_off, k_off, v_off;   // k_off < 0: the layer has no keys / values of its own
    int H, G, d, vd, rot_dims, layout;
    const float2* qk_table;    // (T, rot_dims / 2)
    const float2* v_table;     // (T, vd / 2) or null: values are stored as projected
    void* q_out;               // (T, H * d)
    void* const* k_addrs;      // slot -> (max_seq, G, d)
    void* const* v_addrs;      // slot -> (max_seq, G, vd)
    const int32_t *slot, *pos;
};

// one warp per (token, unit); units: H query heads, then G key heads, then G value heads.  grid (ceil(units / 4), T).
// No norms: the unit's first `rot` channels turn pair by pair by the token's table row, the rest pass.
template <typename TO>
__global__ void __launch_bounds__(128) k_qkv_rope_append(QkvRopeP p) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + warp;
    const int units = p.H + (p.k_off >= 0 ? 2 * p.G : 0);
    if (unit >= units) return;
    const float* row = p.proj + (size_t)t * p.ldp;
    const float* src;
    const float2* tab;
    TO* dst;
    int n, rot;
    if (unit < p.H) {
        src = row + p.q_off + (size_t)unit * p.d;
        n = p.d, rot = p.rot_dims;
        tab = p.qk_table + (size_t)t * (p.rot_dims >> 1);
        dst = static_cast<TO*>(p.q_out) + ((size_t)t * p.H + unit) * p.d;
    } else if (unit < p.H + p.G) {
        const int g = unit - p.H;
        src = row + p.k_off + (size_t)g * p.d;
        n = p.d, rot = p.rot_dims;
        tab = p.qk_table + (size_t)t * (p.rot_dims >> 1);
        dst = static_cast<TO*>(p.k_addrs[p.slot[t]]) + ((size_t)p.pos[t] * p.G + g) * p.d;
    } else {
        const int g = unit - p.H - p.G;
        src = row + p.v_off + (size_t)g * p.vd;
        n = p.vd, rot = p.v_table ? p.vd : 0;
        tab = p.v_table + (size_t)t * (p.vd >> 1);
        dst = static_cast<TO*>(p.v_addrs[p.slot[t]]) + ((size_t)p.pos[t] * p.G + g) * p.vd;
    }
    const int half = rot >> 1;
    for (int i = lane; i < half; i += 32) {
        const int c1 = p.layout == ZL_ROT_ADJACENT ? 2 * i : i, c2 = p.layout == ZL_ROT_ADJACENT ? 2 * i + 1 : i + half;
        const float u = src[c1], v = src[c2];
        const float2 cs = tab[i];
        dst[c1] = from_f32<TO>(u * cs.x - v * cs.y);
        dst[c2] = from_f32<TO>(v * cs.x + u * cs.y);
    }
    for (int c = rot + lane; c < n; c += 32) dst[c] = from_f32<TO>(src[c]);
}

struct GatedCombineP {
    float* x;
    long long ldx;
    float mult;
    const float* gates;        // gate logits of both sublayers in one row: [ga_off .. + D), [gf_off .. + D)
    long long ldg;
    const float* a;            // first sublayer's result (T, D)
    long long lda;
    int ga_off;
    const float* scale_a;
    const float* parts;        // second sublayer: n_parts rows per token, or null
    long long ldp;
    const float* coef;         // (T, n_parts) or null: ones
    const int32_t* choice;     // (T, n_parts) or null; entries >= n_real stand for the sublayers' input itself
    int n_parts, n_real;
    const float* f_dense;      // one more row per token added to the second sublayer's sum, or null
    long long ldf;
    int gf_off;
    const float* scale_f;
    const float* norm_w;       // multipliers of the norm the sublayers read (for the handed-through input)
    const float* next_w;       // multipliers of the next norm, or null
    void* h_next;
    int D;
    float eps;
};

__device__ __forceinline__ float block_sum_256(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();   // red may still be read from an earlier sum
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    return tot;
}

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <typename TO>
__device__ __forceinline__ void store4(TO* dst, float a, float b, float c, float d) {
    if constexpr (sizeof(TO) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
    } else {
        TO v[4] = {from_f32<TO>(a), from_f32<TO>(b), from_f32<TO>(c), from_f32<TO>(d)};
        *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(v);
    }
}

// x[t] += mult * (scale_a sigmoid(g_a) a[t] + scale_f sigmoid(g_f) f[t]), f[t] = sum_p coef_p * (part_p or the sublayers'
// input norm_w * rms(x_old)) + f_dense[t], the parts added in the order of p; then the next layer's norm of the new x.
// One CTA per token.  vec (D % 4 == 0, D <= 4096, every row 16-byte aligned): a thread keeps its (up to four) 4-channel
// pieces of x in registers and every load of a piece is independent of the others; otherwise channel by channel with the
// new x in dynamic shared memory (D floats) between the two passes.
template <typename TO>
__global__ void __launch_bounds__(256) k_gated_parallel_combine(GatedCombineP p, int vec) {
    extern __shared__ float gsx[];
    __shared__ float red[8];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, D = p.D;
    float* xr = p.x + (size_t)t * p.ldx;
    const float* gr = p.gates + (size_t)t * p.ldg;
    const float* ar = p.a + (size_t)t * p.lda;
    const bool second = p.parts || p.f_dense;
    const int32_t* ch = p.choice ? p.choice + (size_t)t * p.n_parts : nullptr;
    const float* cf = p.coef ? p.coef + (size_t)t * p.n_parts : nullptr;
    bool through = false;
    if (p.parts && ch)
        for (int q = 0; q < p.n_parts; ++q) through |= ch[q] >= p.n_real;
    TO* h = p.next_w ? static_cast<TO*>(p.h_next) + (size_t)t * D : nullptr;
    if (vec) {
        float4 xv[4];
        float so = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = (threadIdx.x + i * 256) * 4;
            xv[i] = c < D ? ld4(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            so = fmaf(xv[i].x, xv[i].x, fmaf(xv[i].y, xv[i].y, fmaf(xv[i].z, xv[i].z, fmaf(xv[i].w, xv[i].w, so))));
        }
        float r_old = 0.f;
        if (through) r_old = 1.0f / sqrtf(block_sum_256(so, red) / (float)D + p.eps);   // uniform over the CTA
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = (threadIdx.x + i * 256) * 4;
            if (c >= D) continue;
            const float4 sa = ld4(p.scale_a + c), ga = ld4(gr + p.ga_off + c), av = ld4(ar + c);
            float4 s = make_float4(sa.x * sigmoid_f(ga.x) * av.x, sa.y * sigmoid_f(ga.y) * av.y, sa.z * sigmoid_f(ga.z) * av.z,
                                   sa.w * sigmoid_f(ga.w) * av.w);
            if (second) {
                const float4 sf = ld4(p.scale_f + c), gf = ld4(gr + p.gf_off + c);
                float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
                if (p.parts) {
                    float4 hv = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (through) {
                        const float4 nw = ld4(p.norm_w + c);
                        hv = make_float4(xv[i].x * r_old * nw.x, xv[i].y * r_old * nw.y, xv[i].z * r_old * nw.z, xv[i].w * r_old * nw.w);
                    }
#pragma unroll 4
                    for (int q = 0; q < p.n_parts; ++q) {
                        const float4 v = (ch && ch[q] >= p.n_real) ? hv : ld4(p.parts + ((size_t)t * p.n_parts + q) * p.ldp + c);
                        const float w = cf ? cf[q] : 1.0f;
                        f.x = fmaf(w, v.x, f.x), f.y = fmaf(w, v.y, f.y), f.z = fmaf(w, v.z, f.z), f.w = fmaf(w, v.w, f.w);
                    }
                }
                if (p.f_dense) {
                    const float4 fd = ld4(p.f_dense + (size_t)t * p.ldf + c);
                    f.x += fd.x, f.y += fd.y, f.z += fd.z, f.w += fd.w;
                }
                s.x = fmaf(sf.x * sigmoid_f(gf.x), f.x, s.x), s.y = fmaf(sf.y * sigmoid_f(gf.y), f.y, s.y);
                s.z = fmaf(sf.z * sigmoid_f(gf.z), f.z, s.z), s.w = fmaf(sf.w * sigmoid_f(gf.w), f.w, s.w);
            }
            const float4 nx = make_float4(fmaf(p.mult, s.x, xv[i].x), fmaf(p.mult, s.y, xv[i].y), fmaf(p.mult, s.z, xv[i].z),
                                          fmaf(p.mult, s.w, xv[i].w));
            *reinterpret_cast<float4*>(xr + c) = nx;
            xv[i] = nx;
            ss = fmaf(nx.x, nx.x, fmaf(nx.y, nx.y, fmaf(nx.z, nx.z, fmaf(nx.w, nx.w, ss))));
        }
        if (!h) return;
        const float r = 1.0f / sqrtf(block_sum_256(ss, red) / (float)D + p.eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = (threadIdx.x + i * 256) * 4;
            if (c >= D) continue;
            const float4 nw = ld4(p.next_w + c);
            store4<TO>(h + c, xv[i].x * r * nw.x, xv[i].y * r * nw.y, xv[i].z * r * nw.z, xv[i].w * r * nw.w);
        }
        return;
    }
    float r_old = 0.f;
    if (through) {   // uniform over the CTA
        float so = 0.f;
        for (int c = threadIdx.x; c < D; c += 256) so = fmaf(xr[c], xr[c], so);
        r_old = 1.0f / sqrtf(block_sum_256(so, red) / (float)D + p.eps);
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < D; c += 256) {
        const float xv = xr[c];
        float s = p.scale_a[c] * sigmoid_f(gr[p.ga_off + c]) * ar[c];
        if (second) {
            float f = 0.f;
            if (p.parts)
                for (int q = 0; q < p.n_parts; ++q) {
                    const float v = (ch && ch[q] >= p.n_real) ? xv * r_old * p.norm_w[c] : p.parts[((size_t)t * p.n_parts + q) * p.ldp + c];
                    f = fmaf(cf ? cf[q] : 1.0f, v, f);
                }
            if (p.f_dense) f += p.f_dense[(size_t)t * p.ldf + c];
            s = fmaf(p.scale_f[c] * sigmoid_f(gr[p.gf_off + c]), f, s);
        }
        const float nx = fmaf(p.mult, s, xv);
        xr[c] = nx;
        gsx[c] = nx;
        ss = fmaf(nx, nx, ss);
    }
    if (!h) return;
    const float r = 1.0f / sqrtf(block_sum_256(ss, red) / (float)D + p.eps);
    for (int c = threadIdx.x; c < D; c += 256) h[c] = from_f32<TO>(gsx[c] * r * p.next_w[c]);
}

}  // namespace zl

using namespace zl;

extern "C" int zl_rope_table(const int32_t* pos, int T, const double* inv_freq, int half, float* table, int pdl,
                             zl_stream_t stream) {
    ZL_CHECK_ARG(pos && inv_freq && table && T > 0 && half > 0 && (reinterpret_cast<uintptr_t>(table) & 7) == 0);
    ZL_CHECK_CUDA(launch(k_rope_table, dim3(cdiv(T * half, 256)), dim3(256), 0, stream, pdl != 0, pos, inv_freq,
                         reinterpret_cast<float2*>(table), T, half));
    return ZL_OK;
}

extern "C" int zl_qkv_table_rope_append(const float* proj, long long ldp, int q_off, int k_off, int v_off, int heads, int kv_heads,
                                  int dim, int vdim, const float* qk_table, int rot_dims, const float* v_table, int layout,
                                  void* q_out, void* const* k_addrs, void* const* v_addrs, const int32_t* slot,
                                  const int32_t* pos, int T, int dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(proj && q_out && slot && pos && T > 0 && T <= 65535 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0);
    ZL_CHECK_ARG(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || qk_table));
    ZL_CHECK_ARG(k_off < 0 || (k_addrs && v_addrs && (!v_table || vdim % 2 == 0)));
    ZL_CHECK_ARG(layout == ZL_ROT_HALVES || layout == ZL_ROT_ADJACENT);
    ZL_CHECK_ARG(dtype == ZL_F16 || dtype == ZL_BF16 || dtype == ZL_F32);
    QkvRopeP p{proj, ldp, q_off, k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, layout,
               reinterpret_cast<const float2*>(qk_table), reinterpret_cast<const float2*>(v_table), q_out, k_addrs, v_addrs, slot, pos};
    const int units = heads + (k_off >= 0 ? 2 * kv_heads : 0);
    const dim3 grid(cdiv(units, 4), T), block(128);
    cudaError_t e;
    if (dtype == ZL_F32) e = launch(k_qkv_rope_append<float>, grid, block, 0, stream, pdl != 0, p);
    else if (dtype == ZL_BF16) e = launch(k_qkv_rope_append<__nv_bfloat16>, grid, block, 0, stream, pdl != 0, p);
    else e = launch(k_qkv_rope_append<__half>, grid, block, 0, stream, pdl != 0, p);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_gated_parallel_combine(float* x, long long ldx, float mult, const float* gates, long long ldg, const float* a,
                                         long long lda, int ga_off, const float* scale_a, const float* parts, long long ldp,
                                         const float* coef, const int32_t* choice, int n_parts, int n_real, const float* f_dense,
                                         long long ldf, int gf_off, const float* scale_f, const float* norm_w,
                                         const float* next_w, void* h_next, int act_dtype, int T, int D, float eps, int pdl,
                                         zl_stream_t stream) {
    ZL_CHECK_ARG(x && gates && a && scale_a && T > 0 && D > 0 && ldx >= D && lda >= D && ga_off >= 0);
    ZL_CHECK_ARG(!parts || (n_parts > 0 && ldp >= D && (!choice || norm_w)));
    ZL_CHECK_ARG(!(parts || f_dense) || (scale_f && gf_off >= 0));
    ZL_CHECK_ARG(!f_dense || ldf >= D);
    ZL_CHECK_ARG(!next_w || (h_next && (act_dtype == ZL_F16 || act_dtype == ZL_BF16 || act_dtype == ZL_F32)));
    GatedCombineP p{x, ldx, mult, gates, ldg, a, lda, ga_off, scale_a, parts, ldp, coef, choice, n_parts, n_real, f_dense, ldf,
                    gf_off, scale_f, norm_w, next_w, h_next, D, eps};
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    const int vec = D % 4 == 0 && D <= 4096 && ldx % 4 == 0 && ldg % 4 == 0 && lda % 4 == 0 && ga_off % 4 == 0 && al16(x) &&
                    al16(gates) && al16(a) && al16(scale_a) &&
                    (!(parts || f_dense) || (gf_off % 4 == 0 && al16(scale_f))) &&
                    (!parts || (ldp % 4 == 0 && al16(parts) && (!choice || al16(norm_w)))) &&
                    (!f_dense || (ldf % 4 == 0 && al16(f_dense))) && (!next_w || (al16(next_w) && al16(h_next)));
    const size_t smem = vec ? 0 : (size_t)D * sizeof(float);
    ZL_CHECK_SUPPORTED(smem <= 200 * 1024);
    cudaError_t e = cudaSuccess;
    static size_t set_for[3] = {0, 0, 0};
    const int ti = act_dtype == ZL_F32 ? 0 : (act_dtype == ZL_BF16 ? 1 : 2);
    if (smem > 48 * 1024 && smem > set_for[ti]) {
        if (ti == 0) e = cudaFuncSetAttribute(k_gated_parallel_combine<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        else if (ti == 1) e = cudaFuncSetAttribute(k_gated_parallel_combine<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        else e = cudaFuncSetAttribute(k_gated_parallel_combine<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ZL_CHECK_CUDA(e);
        set_for[ti] = smem;
    }
    if (ti == 0) e = launch(k_gated_parallel_combine<float>, dim3(T), dim3(256), smem, stream, pdl != 0, p, vec);
    else if (ti == 1) e = launch(k_gated_parallel_combine<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, pdl != 0, p, vec);
    else e = launch(k_gated_parallel_combine<__half>, dim3(T), dim3(256), smem, stream, pdl != 0, p, vec);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_qk_fullnorm_append(const float* proj, long long ldp, int q_off, int k_off, int heads, int kv_heads, int dim,
                                     const float* q_weight, const float* k_weight, float eps, void* q_out, void* const* k_addrs,
                                     void* const* v_addrs, const int32_t* slot, const int32_t* pos, int T, int dtype, int pdl,
                                     zl_stream_t stream) {
    ZL_CHECK_ARG(proj && q_weight && k_weight && q_out && k_addrs && v_addrs && slot && pos && T > 0);
    ZL_CHECK_ARG(heads > 0 && kv_heads > 0 && dim > 0 && q_off >= 0 && k_off >= 0);
    ZL_CHECK_ARG(dtype == ZL_F16 || dtype == ZL_BF16 || dtype == ZL_F32);
    const int nq = heads * dim, nk = kv_heads * dim;
    cudaError_t e;
    if (dtype == ZL_F32)
        e = launch(k_qk_fullnorm_append<float>, dim3(T, 2), dim3(512), 0, stream, pdl != 0, proj, ldp, q_off, k_off, nq, nk, q_weight,
                   k_weight, eps, (float*)q_out, k_addrs, v_addrs, slot, pos);
    else if (dtype == ZL_BF16)
        e = launch(k_qk_fullnorm_append<__nv_bfloat16>, dim3(T, 2), dim3(512), 0, stream, pdl != 0, proj, ldp, q_off, k_off, nq, nk,
                   q_weight, k_weight, eps, (__nv_bfloat16*)q_out, k_addrs, v_addrs, slot, pos);
    else
        e = launch(k_qk_fullnorm_append<__half>, dim3(T, 2), dim3(512), 0, stream, pdl != 0, proj, ldp, q_off, k_off, nq, nk, q_weight,
                   k_weight, eps, (__half*)q_out, k_addrs, v_addrs, slot, pos);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_token_shift_mix(const float* x, long long ldx, const float* mu, int n_mix, void* const* state_addrs,
                                  const int32_t* slot, const int32_t* pos, void* out, long long out_stride, int T, int D,
                                  int store_state, int out_dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(x && mu && state_addrs && slot && pos && out && n_mix > 0 && T > 0 && D > 0 && ldx >= D);
    ZL_CHECK_ARG(out_stride >= (long long)T * D);
    ZL_CHECK_ARG(out_dtype == ZL_F16 || out_dtype == ZL_BF16 || out_dtype == ZL_F32);
    // 4 channels per thread when every row (x, the stored tokens, mu, out) starts on a 16-byte boundary
    const bool v4 = D % 4 == 0 && ldx % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(mu)) & 15) == 0;
    const dim3 grid(T, cdiv(D, 256 * (v4 ? 4 : 1))), block(256);
    cudaError_t e;
#define ZL_TSM(TO, V)                                                                                                       \
    launch(k_token_shift_mix<TO, V>, grid, block, 0, stream, pdl != 0, x, ldx, mu, n_mix, state_addrs, slot, pos, (TO*)out, \
           out_stride, D, store_state)
    if (out_dtype == ZL_F32) e = v4 ? ZL_TSM(float, 4) : ZL_TSM(float, 1);
    else if (out_dtype == ZL_BF16) e = v4 ? ZL_TSM(__nv_bfloat16, 4) : ZL_TSM(__nv_bfloat16, 1);
    else e = v4 ? ZL_TSM(__half, 4) : ZL_TSM(__half, 1);
#undef ZL_TSM
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_postnorm_combine(float* x, long long ldx, float alpha, const float* a, long long lda, float coef_a,
                                   const float* b, long long ldb, float coef_b, const float* weight, void* x_act, int act_dtype,
                                   int T, int D, float eps, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(x && a && weight && T > 0 && D > 0 && ldx >= D && lda >= D && (!b || ldb >= D));
    ZL_CHECK_ARG(!x_act || act_dtype == ZL_F16 || act_dtype == ZL_BF16);
    const int vec = D % 4 == 0 && D <= 4096 && ldx % 4 == 0 && lda % 4 == 0 && (!b || ldb % 4 == 0) &&
                    ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                      reinterpret_cast<uintptr_t>(weight)) & 15) == 0;
    ZL_CHECK_SUPPORTED(vec || (size_t)D * 4 <= 48 * 1024);
    cudaError_t e;
    const size_t smem = vec ? 0 : (size_t)D * 4;
    if (x_act && act_dtype == ZL_F16)
        e = launch(k_postnorm_combine<__half>, dim3(T), dim3(256), smem, stream, pdl != 0, x, ldx, alpha, a, lda, coef_a, b, ldb,
                   coef_b, weight, (__half*)x_act, D, eps, vec);
    else
        e = launch(k_postnorm_combine<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, pdl != 0, x, ldx, alpha, a, lda, coef_a, b,
                   ldb, coef_b, weight, (__nv_bfloat16*)x_act, D, eps, vec);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_head_rmsnorm_gate_fn(const float* o, long long ldo, const float* weight, int weight_head_stride,
                                       const float* gate, long long ldg, int gate_fn, void* y, long long ldy, int T, int heads,
                                       int vdim, float eps, int out_dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(o && y && T > 0 && heads > 0 && vdim > 0 && (gate_fn == ZL_GATE_SIGMOID || gate_fn == ZL_GATE_SILU));
    ZL_CHECK_ARG(weight_head_stride == 0 || weight_head_stride >= vdim);
    ZL_CHECK_ARG(out_dtype == ZL_F16 || out_dtype == ZL_BF16 || out_dtype == ZL_F32);
    const dim3 grid(cdiv(heads, 4), T), block(128);
    const int silu = gate_fn == ZL_GATE_SILU;
    cudaError_t e;
    if (out_dtype == ZL_F32)
        e = launch(k_head_rmsnorm_gate<float>, grid, block, 0, stream, pdl != 0, o, ldo, weight, gate, ldg, (float*)y, ldy, heads,
                   vdim, eps, weight_head_stride, silu);
    else if (out_dtype == ZL_BF16)
        e = launch(k_head_rmsnorm_gate<__nv_bfloat16>, grid, block, 0, stream, pdl != 0, o, ldo, weight, gate, ldg,
                   (__nv_bfloat16*)y, ldy, heads, vdim, eps, weight_head_stride, silu);
    else
        e = launch(k_head_rmsnorm_gate<__half>, grid, block, 0, stream, pdl != 0, o, ldo, weight, gate, ldg, (__half*)y, ldy,
                   heads, vdim, eps, weight_head_stride, silu);
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

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
    return zl_head_rmsnorm_gate_fn(o, ldo, weight, vdim, gate, ldg, ZL_GATE_SIGMOID, y, ldy, T, heads, vdim, eps, out_dtype, pdl,
                                   stream);
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

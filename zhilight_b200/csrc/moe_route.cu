// Routing of a mixture of experts, on the device from the router's input to the index lists of the grouped GEMMs:
//   * k_moe_route: logits z = W_router x in fp32 (x is the fp32 residual stream), a score per expert (sigmoid or
//     softmax over the experts), the `top` experts with the largest score + correction (ties: the lower index), their
//     weights = the scores without the correction, optionally renormalised to sum 1.  The logits may also arrive ready
//     (columns of a fused projection).  Restricted choice: the experts form equal groups of neighbours, a group ranks by
//     its largest score + correction, and only experts of the `keep` best groups can be chosen;
//   * k_moe_plan: the (token, choice) pairs sorted by expert: group offsets, and for every list entry the token row it
//     reads and the pair row it writes.  The order inside a group is arbitrary (no row's result depends on it).
// Nothing returns to the host, so a step with routing can be captured in a CUDA graph.
#include "common.cuh"

namespace zl {

constexpr int kRouteWarps = 16;

// row . row with independent 16-byte loads in flight (both rows 16-byte aligned, D % 4 == 0), else element by element
__device__ __forceinline__ float route_dot(const float* __restrict__ a, const float* __restrict__ b, int D, int lane, bool vec) {
    float acc0 = 0.f, acc1 = 0.f;
    if (vec) {
        const float4* a4 = reinterpret_cast<const float4*>(a);
        const float4* b4 = reinterpret_cast<const float4*>(b);
        const int n4 = D >> 2;
        int c = lane;
        for (; c + 32 < n4; c += 64) {
            const float4 x0 = a4[c], y0 = b4[c], x1 = a4[c + 32], y1 = b4[c + 32];
            acc0 = fmaf(x0.x, y0.x, fmaf(x0.y, y0.y, fmaf(x0.z, y0.z, fmaf(x0.w, y0.w, acc0))));
            acc1 = fmaf(x1.x, y1.x, fmaf(x1.y, y1.y, fmaf(x1.z, y1.z, fmaf(x1.w, y1.w, acc1))));
        }
        for (; c < n4; c += 32) {
            const float4 x0 = a4[c], y0 = b4[c];
            acc0 = fmaf(x0.x, y0.x, fmaf(x0.y, y0.y, fmaf(x0.z, y0.z, fmaf(x0.w, y0.w, acc0))));
        }
    } else {
        for (int c = lane; c < D; c += 32) acc0 = fmaf(a[c], b[c], acc0);
    }
    return warp_sum(acc0 + acc1);
}

// grid (T), 16 warps; dynamic shared memory (2 * E + groups) floats.  w_router null: x[t] holds the E logits.
__global__ void __launch_bounds__(kRouteWarps * 32) k_moe_route(const float* __restrict__ x, long long ldx,
                                                   const float* __restrict__ w_router, const float* __restrict__ correction,
                                                   int32_t* __restrict__ top_e, float* __restrict__ top_w, int D, int E,
                                                   int top, int score_fn, int renorm, int groups, int keep, float renorm_eps) {
    extern __shared__ float sm[];
    float* score = sm;        // s_e
    float* choice = sm + E;   // s_e + correction_e; taken experts drop to -inf
    float* gbest = sm + 2 * E;   // largest choice value of every group; a kept group is marked +inf
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* xr = x + (size_t)t * ldx;
    if (w_router) {
        const bool vec = (D & 3) == 0 && (ldx & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_router)) & 15) == 0;
        for (int e = warp; e < E; e += kRouteWarps) {
            const float acc = route_dot(xr, w_router + (size_t)e * D, D, lane, vec);
            if (lane == 0) score[e] = acc;
        }
    } else {
        for (int e = threadIdx.x; e < E; e += blockDim.x) score[e] = xr[e];
    }
    __syncthreads();
    if (warp != 0) return;
    if (score_fn == ZL_MOE_SCORE_SOFTMAX) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, score[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(score[e] - mx);
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) score[e] = expf(score[e] - mx) / sum;
    } else {
        for (int e = lane; e < E; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
    }
    for (int e = lane; e < E; e += 32) choice[e] = score[e] + (correction ? correction[e] : 0.f);
    __syncwarp();
    if (groups > 1 && keep < groups) {
        // the `keep` groups with the largest member survive (ties: the lower group); the others' members drop to -inf
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY;
            for (int i = 0; i < per; ++i) b = fmaxf(b, choice[g * per + i]);
            gbest[g] = b;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gbest[g];
                if (v != INFINITY && (v > bv || bi == 0x7fffffff)) bv = v, bi = g;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) bv = ov, bi = oi;
            }
            if (lane == 0 && bi < groups) gbest[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gbest[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = choice[e];
            if (v > bv) bv = v, bi = e;   // ascending e: the lower index wins a tie inside a lane
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
        if (bi >= E) bi = k < E ? k : 0;   // only when every score is NaN / -inf
        if (lane == 0) {
            top_e[(size_t)t * top + k] = bi;
            top_w[(size_t)t * top + k] = score[bi];
            choice[bi] = -INFINITY;
        }
        wsum += score[bi];
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int k = 0; k < top; ++k) top_w[(size_t)t * top + k] /= wsum + renorm_eps;
}

// one CTA; dynamic shared memory 2 * (E + 1) ints
__global__ void __launch_bounds__(1024) k_moe_plan(const int32_t* __restrict__ top_e, int pairs, int E, int top,
                                                   int32_t* __restrict__ grp_off, int32_t* __restrict__ list_token,
                                                   int32_t* __restrict__ list_pair) {
    extern __shared__ int ism[];
    int* cnt = ism;            // E + 1
    int* cur = ism + E + 1;    // E + 1
    pdl_trigger();
    pdl_wait();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&cnt[top_e[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int c = cnt[e];
            cur[e] = run;
            grp_off[e] = run;
            run += c;
        }
        grp_off[E] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int at = atomicAdd(&cur[top_e[i]], 1);
        list_token[at] = i / top;
        list_pair[at] = i;
    }
}

}  // namespace zl

using namespace zl;

extern "C" int zl_moe_route(const float* x, long long ldx, const float* w_router, const float* correction, int32_t* top_experts,
                            float* top_weights, int32_t* group_offsets, int32_t* list_token, int32_t* list_pair, int T, int D,
                            int experts, int top, int score_fn, int renormalize, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(x && w_router && top_experts && top_weights && group_offsets && list_token && list_pair);
    ZL_CHECK_ARG(T > 0 && D > 0 && experts > 0 && top > 0 && top <= experts && experts <= 4096);
    ZL_CHECK_ARG(score_fn == ZL_MOE_SCORE_SIGMOID || score_fn == ZL_MOE_SCORE_SOFTMAX);
    return zl_moe_route_grouped(x, ldx, w_router, correction, top_experts, top_weights, group_offsets, list_token, list_pair, T, D,
                                experts, top, 1, 1, score_fn, renormalize, 0.f, pdl, stream);
}

extern "C" int zl_moe_route_grouped(const float* x, long long ldx, const float* w_router, const float* correction,
                                    int32_t* top_experts, float* top_weights, int32_t* group_offsets, int32_t* list_token,
                                    int32_t* list_pair, int T, int D, int slots, int top, int groups, int keep, int score_fn,
                                    int renormalize, float renorm_eps, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(x && top_experts && top_weights && group_offsets && list_token && list_pair);
    ZL_CHECK_ARG(T > 0 && (D > 0 || !w_router) && slots > 0 && top > 0 && top <= slots && slots <= 4096);
    ZL_CHECK_ARG(w_router || ldx >= slots);
    ZL_CHECK_ARG(groups >= 1 && slots % groups == 0 && keep >= 1 && keep <= groups && keep * (slots / groups) >= top);
    ZL_CHECK_ARG(score_fn == ZL_MOE_SCORE_SIGMOID || score_fn == ZL_MOE_SCORE_SOFTMAX);
    // with ready logits only the choosing warp has work
    ZL_CHECK_CUDA(launch(k_moe_route, dim3(T), dim3(w_router ? kRouteWarps * 32 : 32), (size_t)(2 * slots + groups) * sizeof(float), stream,
                         pdl != 0, x, ldx, w_router, correction, top_experts, top_weights, D, slots, top, score_fn, renormalize,
                         groups, keep, renorm_eps));
    ZL_CHECK_CUDA(launch(k_moe_plan, dim3(1), dim3(1024), (size_t)2 * (slots + 1) * sizeof(int), stream, pdl != 0,
                         (const int32_t*)top_experts, T * top, slots, top, group_offsets, list_token, list_pair));
    return ZL_OK;
}

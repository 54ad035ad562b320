// Causal attention over per-slot key and value caches with grouped key/value heads, a softmax whose denominator holds
// one extra term exp(sink) that has no value (sink = 0 adds exactly one), and an optional sigmoid gate per head on
// the output.  Token t of the step sees rows 0 .. pos[t] of the caches of slot[t]; the step's own keys and values are
// appended before this runs, so prompts, portions of prompts and single decode tokens are the same case.
// Two optional restrictions of the general form: with chunk > 0 a token sees only the keys of its own block of `chunk`
// positions (blocks counted from position 0 of the sequence), and with a distance table the score of (token, key)
// gets dist_bias[h][min(pos - key, n_dist - 1)] added after the scale.  Two more options: no sink at all (an ordinary
// softmax), and an output rotation: values that were cached turned by their own position give a sum that is turned back
// by the query's position, pair by pair from a (cos, sin) table, in fp32 before the store.
//
// k_sink_attn_mma (16-bit caches, head sizes that are multiples of 16, values up to 128 wide, at most 16 query heads per
// key/value head): a CTA owns up to 64 rows = (consecutive tokens of one run) x (the query heads of one key/value
// head), so prompts fill the tile with tokens and decode steps with the heads that share the cached bytes.  Keys and
// values come in tiles of 64 rows (cp.async, double buffered); S = Q K^T and O += P V on mma.sync.m16n8k16 with fp32
// accumulators, the scores' scale, mask and online softmax in fp32 registers.  The probabilities enter the second
// product as a bfloat16 pair hi + lo (two MMAs), so that no weight is rounded to 8 bits.  The sink is the initial
// (max, sum) = (sink, 1) of every row; with key splits it is added by the merge kernel instead.
// k_sink_attn: any head sizes up to 256 and any dtype; scores, softmax and the weighted sum in fp32 FMAs.  One CTA per
// (token, query head); its 8 warps take the keys j = warp, warp + 8, ... (a fixed assignment: the result of a token
// does not depend on the step it is computed in) with an online softmax each, merged in warp order with the sink term.
#include "common.cuh"

#include <cmath>
#include <cstdlib>
#include <type_traits>

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
    int chunk = 0;             // > 0: keys below (pos / chunk) * chunk are not seen
    const float* dist_bias = nullptr;   // (H, n_dist) added to the scaled score by distance, or null
    int n_dist = 0;
    int no_sink = 0;           // the denominator holds the keys only
    const float* out_table = nullptr;   // (T, vd / 2) pairs (cos, sin): the output of token t is turned back by these angles
    int out_layout = 0;        // ZL_ROT_HALVES: pair (m, m + vd / 2); ZL_ROT_ADJACENT: pair (2m, 2m + 1)
};

// the two channels of pair m
__device__ __forceinline__ void sa_pair(const SinkAttnP& p, int m, int& c1, int& c2) {
    if (p.out_layout == ZL_ROT_ADJACENT) c1 = 2 * m, c2 = 2 * m + 1;
    else c1 = m, c2 = m + (p.vd >> 1);
}
// (u, v) turned by minus the angle of (cos, sin) = cs, times `mul`, stored
template <typename T>
__device__ __forceinline__ void sa_store_unrotated(T* out, int c1, int c2, float u, float v, float2 cs, float mul) {
    out[c1] = from_f32<T>((u * cs.x + v * cs.y) * mul);
    out[c2] = from_f32<T>((v * cs.x - u * cs.y) * mul);
}

// first key a token at `pos` sees
__device__ __forceinline__ int sa_first_key(const SinkAttnP& p, int pos) { return p.chunk > 0 ? (pos / p.chunk) * p.chunk : 0; }

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
    int j_lo = sa_first_key(p, pos), j_hi = pos + 1;
    if (p.splits > 1) {
        const int per = cdiv(cdiv(pos + 1 - j_lo, p.splits), kSaWarps) * kSaWarps;
        j_lo += blockIdx.z * per;
        j_hi = min(pos + 1, j_lo + per);
    }
    const float* bias = p.dist_bias ? p.dist_bias + (size_t)h * p.n_dist : nullptr;
    for (int j = j_lo + warp; j < j_hi; j += kSaWarps) {
        const T* kr = kc + (size_t)j * kst;
        float s = 0.f;
        for (int c = lane; c < p.d; c += 32) s = fmaf(sq[c], to_f32<T>(kr[c]), s);
        s = warp_sum(s);
        if (bias) s += bias[min(pos - j, p.n_dist - 1)];
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
    const float sink = p.no_sink ? -INFINITY : (p.sink ? p.sink[h] : 0.f);
    float M = sink;
    for (int w = 0; w < kSaWarps; ++w) M = fmaxf(M, sm_m[w]);
    float L = expf(sink - M);   // 0 without a sink: the token's own key keeps M finite
    for (int w = 0; w < kSaWarps; ++w) L = fmaf(sm_l[w], expf(sm_m[w] - M), L);
    float gate = 1.0f;
    if (p.gate) gate = 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.ldg + h]));
    T* out = static_cast<T*>(p.out) + ((size_t)t * p.H + h) * p.vd;
    if (p.out_table) {
        const float2* tab = reinterpret_cast<const float2*>(p.out_table) + (size_t)t * (p.vd >> 1);
        for (int mi = threadIdx.x; mi < (p.vd >> 1); mi += blockDim.x) {
            int c1, c2;
            sa_pair(p, mi, c1, c2);
            float o1 = 0.f, o2 = 0.f;
            for (int w = 0; w < kSaWarps; ++w) {
                const float e = expf(sm_m[w] - M);
                o1 = fmaf(sm_acc[(size_t)w * p.vd + c1], e, o1);
                o2 = fmaf(sm_acc[(size_t)w * p.vd + c2], e, o2);
            }
            sa_store_unrotated<T>(out, c1, c2, o1, o2, tab[mi], gate / L);
        }
        return;
    }
    for (int c = threadIdx.x; c < p.vd; c += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < kSaWarps; ++w) o = fmaf(sm_acc[(size_t)w * p.vd + c], expf(sm_m[w] - M), o);
        out[c] = from_f32<T>(o / L * gate);
    }
}

// ---- tensor-core kernel ----------------------------------------------------------------------------------------------
struct SinkAttnMmaP {
    SinkAttnP a;
    const int32_t *run_row0, *run_len;
};

constexpr int kTq = 64, kTk = 64;

__device__ __forceinline__ void sa_cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void sa_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void sa_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void sa_ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void sa_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
template <typename T>
__device__ __forceinline__ void sa_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void sa_mma<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    mma_16816_f16(d, a, b0, b1, d);
}
template <>
__device__ __forceinline__ void sa_mma<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    mma_16816_bf16(d, a, b0, b1, d);
}
template <typename T>
__device__ __forceinline__ uint32_t sa_pack(float x, float y) {
    T a = from_f32<T>(x), b = from_f32<T>(y);
    return (uint32_t) * reinterpret_cast<uint16_t*>(&a) | ((uint32_t) * reinterpret_cast<uint16_t*>(&b) << 16);
}

// grid (ceil(longest run / tokens per tile), G, runs * splits); 4 warps.  NV: 8-column value tiles per warp.
// DEC = false: a tile of 64 rows, 16 per warp, every warp over all 64 keys of a key tile.
// DEC = true (the rows of a tile fit 16: decode steps): every warp holds the same 16 rows and takes 16 of the 64 keys
// of a key tile with a softmax state of its own; the four states are merged through shared memory at the end.
template <typename T, int NV, bool DEC>
__global__ void __launch_bounds__(128) k_sink_attn_mma(SinkAttnMmaP pp) {
    extern __shared__ __align__(16) unsigned char sa_raw[];
    const SinkAttnP& p = pp.a;
    constexpr int QR = DEC ? 16 : kTq;      // rows of the query tile
    constexpr int NS = DEC ? 2 : 8;         // 8-key score tiles per warp and key tile
    const int DP = p.d + 8, VP = NV * 8 + 8;
    T* sQ = reinterpret_cast<T*>(sa_raw);   // [QR][DP]
    T* sK = sQ + QR * DP;                   // [2][kTk][DP]
    T* sV = sK + 2 * kTk * DP;              // [2][kTk][VP]
    pdl_trigger();
    pdl_wait();
    const int run = blockIdx.z / p.splits, split = blockIdx.z % p.splits, g = blockIdx.y;
    const int R = p.H / p.G, nq = QR / R;
    const int len = pp.run_len[run], t0 = blockIdx.x * nq;
    if (t0 >= len) return;
    const int ntok = min(nq, len - t0), row0 = pp.run_row0[run] + t0;
    const int sl = p.slot[row0], pos0 = p.pos[row0];
    const int n_keys = pos0 + ntok;
    // key tiles start at multiples of kTk from key 0 whatever the step, so a token's sums do not depend on the cut
    int k_lo = (sa_first_key(p, pos0) / kTk) * kTk, k_hi = n_keys;
    if (p.splits > 1) {
        const int per = cdiv(cdiv(n_keys - k_lo, p.splits), kTk) * kTk;
        k_lo += split * per;
        k_hi = min(n_keys, k_lo + per);
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
    const int d8 = p.d >> 3, v8 = p.vd >> 3;
    const T* kc = static_cast<const T*>(p.k_addrs[sl]) + (size_t)g * p.d;
    const T* vc = static_cast<const T*>(p.v_addrs[sl]) + (size_t)g * p.vd;
    const size_t kst = (size_t)p.G * p.d, vst = (size_t)p.G * p.vd;

    auto load_kv = [&](int buf, int k0) {
        T* dk = sK + (size_t)buf * kTk * DP;
        T* dv = sV + (size_t)buf * kTk * VP;
        for (int i = tid; i < kTk * d8; i += 128) {
            const int r = i / d8, c = i - r * d8, kj = k0 + r;
            if (kj < k_hi) sa_cp_async16(dk + (size_t)r * DP + c * 8, kc + (size_t)kj * kst + c * 8);
            else *reinterpret_cast<uint4*>(dk + (size_t)r * DP + c * 8) = make_uint4(0, 0, 0, 0);
        }
        for (int i = tid; i < kTk * (NV + 0); i += 128) {
            const int r = i / NV, c = i - r * NV, kj = k0 + r;
            if (kj < k_hi && c < v8) sa_cp_async16(dv + (size_t)r * VP + c * 8, vc + (size_t)kj * vst + c * 8);
            else *reinterpret_cast<uint4*>(dv + (size_t)r * VP + c * 8) = make_uint4(0, 0, 0, 0);
        }
    };
    // rows of this thread: wrow + gq and + 8; row -> (token, head in the group).  kb: the warp's first key in a key tile
    const int wrow = DEC ? 0 : warp * 16, kb = DEC ? warp * 16 : 0;
    int tok_of[2], pos_of[2], head_of[2], first_of[2];
    bool row_ok[2];
    const float* bias_of[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = wrow + gq + hh * 8;
        tok_of[hh] = r / R;
        head_of[hh] = g * R + (r - tok_of[hh] * R);
        row_ok[hh] = tok_of[hh] < ntok;
        pos_of[hh] = pos0 + tok_of[hh];
        first_of[hh] = sa_first_key(p, pos_of[hh]);
        bias_of[hh] = p.dist_bias ? p.dist_bias + (size_t)(head_of[hh] < p.H ? head_of[hh] : 0) * p.n_dist : nullptr;
    }
    float m_run[2], l_run[2], O[NV][4];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const float sink = p.sink ? p.sink[head_of[hh] < p.H ? head_of[hh] : 0] : 0.f;
        m_run[hh] = (DEC || p.splits > 1 || p.no_sink) ? -1e30f : sink;
        l_run[hh] = (DEC || p.splits > 1 || p.no_sink || tq != 0) ? 0.f : 1.f;   // the sink's exp(sink - m) = 1, held by one thread of the quad
    }
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) O[j][c] = 0.f;

    if (k_lo < k_hi) {
        // the query tile
        for (int i = tid; i < QR * d8; i += 128) {
            const int r = i / d8, c = i - r * d8, tk = r / R;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tk < ntok)
                v = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + ((size_t)(row0 + tk) * p.H + g * R + (r - tk * R)) * p.d + c * 8);
            *reinterpret_cast<uint4*>(sQ + (size_t)r * DP + c * 8) = v;
        }
        load_kv(0, k_lo);
        sa_cp_commit();
        int buf = 0;
        for (int k0 = k_lo; k0 < k_hi; k0 += kTk, buf ^= 1) {
            sa_cp_wait<0>();
            __syncthreads();   // tile k0 (and the query tile) is in shared memory; every warp is done with the other buffer
            if (k0 + kTk < k_hi) load_kv(buf ^ 1, k0 + kTk);
            sa_cp_commit();
            const T* tK = sK + (size_t)buf * kTk * DP;
            const T* tV = sV + (size_t)buf * kTk * VP;
            float S[NS][4];
#pragma unroll
            for (int j = 0; j < NS; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) S[j][c] = 0.f;
            for (int kk = 0; kk < p.d; kk += 16) {
                uint32_t a[4];
                sa_ldmatrix_x4(a, sQ + (size_t)(wrow + (lane & 15)) * DP + kk + (lane >> 4) * 8);
#pragma unroll
                for (int jj = 0; jj < NS / 2; ++jj) {
                    uint32_t b[4];
                    sa_ldmatrix_x4(b, tK + (size_t)(kb + jj * 16 + (lane & 7) + (lane >> 4) * 8) * DP + kk + ((lane >> 3) & 1) * 8);
                    sa_mma<T>(S[2 * jj], a, b[0], b[1]);
                    sa_mma<T>(S[2 * jj + 1], a, b[2], b[3]);
                }
            }
            // scale, mask, online softmax (rows gq and gq + 8 of the warp's 16)
            float mx[2] = {-1e30f, -1e30f};
#pragma unroll
            for (int j = 0; j < NS; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int hh = c >> 1, key = k0 + kb + 8 * j + 2 * tq + (c & 1);
                    const bool ok = row_ok[hh] && key < k_hi && key <= pos_of[hh] && key >= first_of[hh];
                    float sc = S[j][c] * p.scale;
                    if (ok && bias_of[hh]) sc += bias_of[hh][min(pos_of[hh] - key, p.n_dist - 1)];
                    S[j][c] = ok ? sc : -1e30f;
                    mx[hh] = fmaxf(mx[hh], S[j][c]);
                }
            float corr[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
                const float mn = fmaxf(m_run[hh], mx[hh]);
                corr[hh] = expf(m_run[hh] - mn);
                m_run[hh] = mn;
                l_run[hh] *= corr[hh];
            }
#pragma unroll
            for (int j = 0; j < NS; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int hh = c >> 1;
                    const float pr = S[j][c] > -1e29f ? expf(S[j][c] - m_run[hh]) : 0.f;
                    S[j][c] = pr;
                    l_run[hh] += pr;
                }
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                O[j][0] *= corr[0], O[j][1] *= corr[0];
                O[j][2] *= corr[1], O[j][3] *= corr[1];
            }
            // O += P V, 16 keys at a time
#pragma unroll
            for (int k2 = 0; k2 < NS / 2; ++k2) {
                uint32_t ah[4], al[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float x = S[2 * k2 + (r >> 1)][(r & 1) * 2], y = S[2 * k2 + (r >> 1)][(r & 1) * 2 + 1];
                    ah[r] = sa_pack<T>(x, y);
                    if constexpr (sizeof(T) == 2 && !std::is_same<T, __half>::value) {
                        const float xh = round_to<T>(x), yh = round_to<T>(y);
                        al[r] = sa_pack<T>(x - xh, y - yh);
                    }
                }
#pragma unroll
                for (int nn = 0; nn < NV / 2; ++nn) {
                    uint32_t b[4];
                    sa_ldmatrix_x4_trans(b, tV + (size_t)(kb + k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VP + nn * 16 + (lane >> 4) * 8);
                    sa_mma<T>(O[2 * nn], ah, b[0], b[1]);
                    sa_mma<T>(O[2 * nn + 1], ah, b[2], b[3]);
                    if constexpr (!std::is_same<T, __half>::value) {
                        sa_mma<T>(O[2 * nn], al, b[0], b[1]);
                        sa_mma<T>(O[2 * nn + 1], al, b[2], b[3]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
    if constexpr (DEC) {
        // the four warps' states of the same 16 rows -> one, through shared memory (the key tiles are no longer needed)
        __syncthreads();
        float* mm = reinterpret_cast<float*>(sa_raw);   // [4][16] max, [4][16] sum, [4][16][NV * 8] values
        float* ml = mm + 64;
        float* mo = ml + 64;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int r = gq + hh * 8;
            if (tq == 0) mm[warp * 16 + r] = m_run[hh], ml[warp * 16 + r] = l_run[hh];
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                mo[((size_t)warp * 16 + r) * (NV * 8) + 8 * j + 2 * tq] = O[j][hh * 2];
                mo[((size_t)warp * 16 + r) * (NV * 8) + 8 * j + 2 * tq + 1] = O[j][hh * 2 + 1];
            }
        }
        __syncthreads();
        const int r = tid >> 3, tk = r / R;   // 8 threads per row
        if (tk >= ntok) return;
        const int t = row0 + tk, h = g * R + (r - tk * R);
        const float sink = p.sink ? p.sink[h] : 0.f;
        const bool with_sink = p.splits == 1 && !p.no_sink;
        float M = with_sink ? sink : -1e30f;
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * 16 + r]);
        float L = with_sink ? expf(sink - M) : 0.f, wgt[4];
        for (int w = 0; w < 4; ++w) {
            wgt[w] = ml[w * 16 + r] > 0.f ? expf(mm[w * 16 + r] - M) : 0.f;
            L = fmaf(ml[w * 16 + r], wgt[w], L);
        }
        if (p.splits > 1) {
            float* part = p.ws + (((size_t)t * p.H + h) * p.splits + split) * (2 + p.vd);
            if ((tid & 7) == 0) part[0] = L > 0.f ? M : -INFINITY, part[1] = L;
            for (int c = tid & 7; c < p.vd; c += 8) {
                float o = 0.f;
                for (int w = 0; w < 4; ++w) o = fmaf(mo[((size_t)w * 16 + r) * (NV * 8) + c], wgt[w], o);
                part[2 + c] = o;
            }
        } else {
            float gate = 1.0f;
            if (p.gate) gate = 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.ldg + h]));
            const float inv = gate / L;
            T* out = static_cast<T*>(p.out) + ((size_t)t * p.H + h) * p.vd;
            if (p.out_table) {
                const float2* tab = reinterpret_cast<const float2*>(p.out_table) + (size_t)t * (p.vd >> 1);
                for (int mi = tid & 7; mi < (p.vd >> 1); mi += 8) {
                    int c1, c2;
                    sa_pair(p, mi, c1, c2);
                    float o1 = 0.f, o2 = 0.f;
                    for (int w = 0; w < 4; ++w) {
                        o1 = fmaf(mo[((size_t)w * 16 + r) * (NV * 8) + c1], wgt[w], o1);
                        o2 = fmaf(mo[((size_t)w * 16 + r) * (NV * 8) + c2], wgt[w], o2);
                    }
                    sa_store_unrotated<T>(out, c1, c2, o1, o2, tab[mi], inv);
                }
            } else
            for (int c = tid & 7; c < p.vd; c += 8) {
                float o = 0.f;
                for (int w = 0; w < 4; ++w) o = fmaf(mo[((size_t)w * 16 + r) * (NV * 8) + c], wgt[w], o);
                out[c] = from_f32<T>(o * inv);
            }
        }
    } else {
    if (p.out_table && p.splits == 1) {
        // the tile's normalised rows go through shared memory (the key tiles are no longer needed): the two channels of a
        // pair sit in different threads
        __syncthreads();
        float* so = reinterpret_cast<float*>(sa_raw);   // [kTq][vd + 1]
        const int SP = p.vd + 1, half = p.vd >> 1;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            if (!row_ok[hh]) continue;
            float gate = 1.0f;
            if (p.gate) gate = 1.0f / (1.0f + expf(-p.gate[(size_t)(row0 + tok_of[hh]) * p.ldg + head_of[hh]]));
            const float inv = gate / l_run[hh];
            float* sr = so + (size_t)(wrow + gq + hh * 8) * SP;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int c = 8 * j + 2 * tq;
                if (c < p.vd) sr[c] = O[j][hh * 2] * inv, sr[c + 1] = O[j][hh * 2 + 1] * inv;
            }
        }
        __syncthreads();
        for (int i = tid; i < kTq * half; i += 128) {
            const int r = i / half, mi = i - r * half, tk = r / R;
            if (tk >= ntok) continue;
            const int t = row0 + tk, h = g * R + (r - tk * R);
            int c1, c2;
            sa_pair(p, mi, c1, c2);
            const float2 cs = reinterpret_cast<const float2*>(p.out_table)[(size_t)t * half + mi];
            sa_store_unrotated<T>(static_cast<T*>(p.out) + ((size_t)t * p.H + h) * p.vd, c1, c2, so[(size_t)r * SP + c1],
                                  so[(size_t)r * SP + c2], cs, 1.0f);
        }
        return;
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        if (!row_ok[hh]) continue;
        const int t = row0 + tok_of[hh], h = head_of[hh];
        if (p.splits > 1) {
            float* part = p.ws + (((size_t)t * p.H + h) * p.splits + split) * (2 + p.vd);
            const bool empty = l_run[hh] <= 0.f;
            if (tq == 0) part[0] = empty ? -INFINITY : m_run[hh], part[1] = empty ? 0.f : l_run[hh];
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int c = 8 * j + 2 * tq;
                if (c < p.vd) part[2 + c] = O[j][hh * 2], part[2 + c + 1] = O[j][hh * 2 + 1];
            }
        } else {
            float gate = 1.0f;
            if (p.gate) gate = 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.ldg + h]));
            const float inv = gate / l_run[hh];
            T* out = static_cast<T*>(p.out) + ((size_t)t * p.H + h) * p.vd;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int c = 8 * j + 2 * tq;
                if (c < p.vd) {
                    out[c] = from_f32<T>(O[j][hh * 2] * inv);
                    out[c + 1] = from_f32<T>(O[j][hh * 2 + 1] * inv);
                }
            }
        }
    }
    }
}

template <typename T, int NV, bool DEC>
static cudaError_t launch_sink_mma(const SinkAttnMmaP& pp, int runs, int max_run_len, bool pdl, cudaStream_t st) {
    const SinkAttnP& p = pp.a;
    const int qr = DEC ? 16 : kTq, nq = qr / (p.H / p.G);
    size_t smem = ((size_t)qr * (p.d + 8) + 2 * (size_t)kTk * (p.d + 8) + 2 * (size_t)kTk * (NV * 8 + 8)) * sizeof(T);
    if (DEC && smem < (size_t)(128 + 64 * NV * 8) * sizeof(float)) smem = (size_t)(128 + 64 * NV * 8) * sizeof(float);
    if (!DEC && p.out_table && smem < (size_t)kTq * (p.vd + 1) * sizeof(float)) smem = (size_t)kTq * (p.vd + 1) * sizeof(float);
    static size_t set_for = 0;
    if (smem > 48 * 1024 && smem > set_for) {
        const cudaError_t e = cudaFuncSetAttribute(k_sink_attn_mma<T, NV, DEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        set_for = smem;
    }
    return launch(k_sink_attn_mma<T, NV, DEC>, dim3(cdiv(max_run_len, nq), p.G, runs * p.splits), dim3(128), smem, st, pdl, pp);
}
template <typename T, int NV>
static cudaError_t launch_sink_mma_d(const SinkAttnMmaP& pp, int runs, int max_run_len, bool pdl, cudaStream_t st) {
    // the rows of the longest run fit one 16-row tile: the decode form
    if (max_run_len * (pp.a.H / pp.a.G) <= 16) return launch_sink_mma<T, NV, true>(pp, runs, max_run_len, pdl, st);
    return launch_sink_mma<T, NV, false>(pp, runs, max_run_len, pdl, st);
}
template <typename T>
static cudaError_t launch_sink_mma_t(const SinkAttnMmaP& pp, int runs, int max_run_len, bool pdl, cudaStream_t st) {
    if (pp.a.vd <= 32) return launch_sink_mma_d<T, 4>(pp, runs, max_run_len, pdl, st);
    if (pp.a.vd <= 64) return launch_sink_mma_d<T, 8>(pp, runs, max_run_len, pdl, st);
    return launch_sink_mma_d<T, 16>(pp, runs, max_run_len, pdl, st);
}

// merge of the splits (at most 32) with the sink term and the gate; one warp per (token, head), grid (ceil(H / 4), T).
// Lane s holds the (max, sum) of split s, so the weights of all splits come from one round of loads.
template <typename T>
__global__ void __launch_bounds__(128) k_sink_attn_merge(SinkAttnP p) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= p.H) return;
    const int stride = 2 + p.vd;
    const float* part = p.ws + ((size_t)t * p.H + h) * p.splits * stride;
    const float sink = p.no_sink ? -INFINITY : (p.sink ? p.sink[h] : 0.f);
    const float ms = lane < p.splits ? part[(size_t)lane * stride] : -INFINITY;
    const float ls = lane < p.splits ? part[(size_t)lane * stride + 1] : 0.f;
    const float M = fmaxf(sink, warp_max(ms));
    const float wgt = ms == -INFINITY ? 0.f : expf(ms - M);
    // the sum over the splits in the order of the splits, the same in every lane
    float L = expf(sink - M);
    for (int s = 0; s < p.splits; ++s) L = fmaf(__shfl_sync(0xffffffffu, ls, s), __shfl_sync(0xffffffffu, wgt, s), L);
    float gate = 1.0f;
    if (p.gate) gate = 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.ldg + h]));
    T* out = static_cast<T*>(p.out) + ((size_t)t * p.H + h) * p.vd;
    float wv[32];   // every split's weight in every lane: the loads below do not wait for shuffles
#pragma unroll
    for (int s = 0; s < 32; ++s) wv[s] = __shfl_sync(0xffffffffu, wgt, s);
    if (p.out_table) {
        const float2* tab = reinterpret_cast<const float2*>(p.out_table) + (size_t)t * (p.vd >> 1);
        for (int mi = lane; mi < (p.vd >> 1); mi += 32) {
            int c1, c2;
            sa_pair(p, mi, c1, c2);
            float v1[32], v2[32];
#pragma unroll
            for (int s = 0; s < 32; ++s) {
                v1[s] = s < p.splits ? part[(size_t)s * stride + 2 + c1] : 0.f;
                v2[s] = s < p.splits ? part[(size_t)s * stride + 2 + c2] : 0.f;
            }
            float o1 = 0.f, o2 = 0.f;
#pragma unroll
            for (int s = 0; s < 32; ++s) o1 = fmaf(v1[s], wv[s], o1), o2 = fmaf(v2[s], wv[s], o2);
            sa_store_unrotated<T>(out, c1, c2, o1, o2, tab[mi], gate / L);
        }
        return;
    }
    for (int c = lane; c < p.vd; c += 32) {
        float v[32];
#pragma unroll
        for (int s = 0; s < 32; ++s) v[s] = s < p.splits ? part[(size_t)s * stride + 2 + c] : 0.f;   // all loads in flight
        float o = 0.f;
#pragma unroll
        for (int s = 0; s < 32; ++s) o = fmaf(v[s], wv[s], o);   // splits in order; absent ones add 0 * 0
        out[c] = from_f32<T>(o / L * gate);
    }
}

}  // namespace zl

using namespace zl;

extern "C" size_t zl_sink_attention_workspace_bytes(int T, int heads, int vdim, int splits) {
    return splits > 1 ? (size_t)T * heads * splits * (2 + vdim) * sizeof(float) : 0;
}

// enough CTAs for four per SM (a CTA of the tensor-core kernel serves one key/value head of up to 64 / group rows), no
// split shorter than 128 keys, at most 32
extern "C" int zl_sink_attention_splits(int T, int heads, int kv_heads, int max_len) {
    (void)heads;
    const int ctas = T * kv_heads > 0 ? T * kv_heads : 1;
    const int want = cdiv(4 * device_sm_count(), ctas);
    const int cap = max_len / 128 > 0 ? max_len / 128 : 1;
    int s = want < cap ? want : cap;
    if (s > 32) s = 32;
    return s < 1 ? 1 : s;
}

extern "C" int zl_sink_attention(const void* q, void* const* k_addrs, void* const* v_addrs, const int32_t* slot,
                                 const int32_t* pos, const float* sink, const float* gate, long long ldg, float scale, void* out,
                                 int T, int heads, int kv_heads, int dim, int vdim, int splits, void* workspace,
                                 size_t workspace_bytes, const int32_t* run_row0, const int32_t* run_len, int runs,
                                 int max_run_len, int dtype, int pdl, zl_stream_t stream) {
    return zl_sink_attention_ex(q, k_addrs, v_addrs, slot, pos, sink, 0, gate, ldg, scale, 0, nullptr, 0, nullptr, 0, out, T, heads,
                                kv_heads, dim, vdim, splits, workspace, workspace_bytes, run_row0, run_len, runs, max_run_len,
                                dtype, pdl, stream);
}

extern "C" int zl_distance_bias_table(const float* table_host, int rows, int heads, double far, int n_dist, float* out_host) {
    ZL_CHECK_ARG(table_host && out_host && rows > 0 && heads > 0 && n_dist > 0);
    const int half = rows / 2;
    ZL_CHECK_ARG(rows == 1 || (half > 0 && far > (double)half));
    for (int n = 0; n < n_dist; ++n) {
        int b = n;
        if (n >= half) {
            b = rows == 1 ? 0 : half + (int)floor(log((double)n / half) / log(far / half) * (double)(rows - half));
            if (b > rows - 1) b = rows - 1;
        }
        for (int h = 0; h < heads; ++h) out_host[(size_t)h * n_dist + n] = table_host[(size_t)b * heads + h];
    }
    return ZL_OK;
}

extern "C" int zl_sink_attention_local(const void* q, void* const* k_addrs, void* const* v_addrs, const int32_t* slot,
                                       const int32_t* pos, const float* sink, const float* gate, long long ldg, float scale,
                                       int chunk, const float* dist_bias, int n_dist, void* out, int T, int heads, int kv_heads,
                                       int dim, int vdim, int splits, void* workspace, size_t workspace_bytes,
                                       const int32_t* run_row0, const int32_t* run_len, int runs, int max_run_len, int dtype,
                                       int pdl, zl_stream_t stream) {
    return zl_sink_attention_ex(q, k_addrs, v_addrs, slot, pos, sink, 0, gate, ldg, scale, chunk, dist_bias, n_dist, nullptr, 0, out,
                                T, heads, kv_heads, dim, vdim, splits, workspace, workspace_bytes, run_row0, run_len, runs,
                                max_run_len, dtype, pdl, stream);
}

extern "C" int zl_sink_attention_ex(const void* q, void* const* k_addrs, void* const* v_addrs, const int32_t* slot,
                                    const int32_t* pos, const float* sink, int no_sink, const float* gate, long long ldg,
                                    float scale, int chunk, const float* dist_bias, int n_dist, const float* out_table,
                                    int out_layout, void* out, int T, int heads, int kv_heads, int dim, int vdim, int splits,
                                    void* workspace, size_t workspace_bytes, const int32_t* run_row0, const int32_t* run_len,
                                    int runs, int max_run_len, int dtype, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(chunk >= 0 && (!dist_bias || n_dist > 0));
    ZL_CHECK_ARG(!out_table || (vdim % 2 == 0 && (out_layout == ZL_ROT_HALVES || out_layout == ZL_ROT_ADJACENT) &&
                                (reinterpret_cast<uintptr_t>(out_table) & 7) == 0));
    ZL_CHECK_ARG(q && k_addrs && v_addrs && slot && pos && out && T > 0 && T <= 65535 && heads > 0 && kv_heads > 0);
    ZL_CHECK_ARG(heads % kv_heads == 0 && dim > 0 && vdim > 0);
    ZL_CHECK_SUPPORTED(vdim <= 32 * kSaMaxPerLane);
    ZL_CHECK_ARG(dtype == ZL_F16 || dtype == ZL_BF16 || dtype == ZL_F32);
    ZL_CHECK_ARG(splits >= 1 && splits <= 32);
    ZL_CHECK_ARG(splits == 1 || (workspace && workspace_bytes >= zl_sink_attention_workspace_bytes(T, heads, vdim, splits)));
    SinkAttnP p{q, k_addrs, v_addrs, slot, pos, sink, gate, ldg, out, heads, kv_heads, dim, vdim, scale, splits,
                static_cast<float*>(workspace)};
    p.chunk = chunk;
    p.dist_bias = dist_bias;
    p.n_dist = n_dist;
    p.no_sink = no_sink != 0;
    p.out_table = out_table;
    p.out_layout = out_layout;
    const dim3 grid(heads, T, splits), block(kSaWarps * 32);
    const size_t smem = ((size_t)dim + 2 * kSaWarps + (size_t)kSaWarps * vdim) * sizeof(float);
    cudaError_t e;
    static const bool no_mma = getenv("ZL_SINK_ATTN_NO_MMA") != nullptr;
    const bool mma = !no_mma && run_row0 && run_len && runs > 0 && max_run_len > 0 && dtype != ZL_F32 && dim % 16 == 0 &&
                     vdim % 8 == 0 && vdim <= 128 && dim <= 256 && heads / kv_heads <= 16 && 16 % (heads / kv_heads) == 0;
    if (mma) {
        ZL_CHECK_ARG((long long)runs * splits <= 65535 && kv_heads <= 65535);
        SinkAttnMmaP pp{p, run_row0, run_len};
        e = dtype == ZL_BF16 ? launch_sink_mma_t<__nv_bfloat16>(pp, runs, max_run_len, pdl != 0, stream)
                             : launch_sink_mma_t<__half>(pp, runs, max_run_len, pdl != 0, stream);
    } else if (dtype == ZL_F32) e = launch(k_sink_attn<float>, grid, block, smem, stream, pdl != 0, p);
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

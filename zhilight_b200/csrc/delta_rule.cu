// Generalized delta rule: a recurrent mixer whose state per head is a (dk, dv) fp32 matrix S carried from token to token,
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,      o_t = S_t^T r_t,
// with u_t = k_t / sqrt(sum(k_t^2) + unit_eps), a decay w_t = exp(-decay_scale * sigmoid(decay_logit_t)) and a removal
// rate a_t = sigmoid(rate_logit_t) per key channel; both subtracted terms read S_(t-1).
//
// The columns of S (one per value channel) never meet: S_t[:, j] depends on S_(t-1)[:, j] and on the token's vectors
// only.  A column is walked through the tokens of its sequence in order, so the result of a token does not depend on
// how the sequence was cut into steps or on the other sequences of the step.  A CTA owns 32 columns of one head of one
// run (the consecutive rows of one slot in the step).  The token vectors (u, a*u, w, k, r, v) are prepared for all
// tokens at once by a kernel of their own; the recurrence stages them chunk by chunk in shared memory ahead of use.
// For the compiled key sizes (32, 64, 128) a column lives in the registers of four adjacent lanes (k_delta_rule_quad;
// ZL_DELTA_NO_QUAD: of one thread, k_delta_rule), for other sizes in shared memory, one thread per column.
// A run that starts at position 0 starts from a zero state (a slot given to a new sequence needs no clearing); the
// final state goes back to the slot.  Everything is fp32.
//
// Two more recurrences run on the same column kernels, each with a preparation kernel of its own that writes the same
// six token vectors:
//   * gated delta rule:  S <- g S;  e = beta (v - S^T k);  S <- S + k e^T;  o = S^T q, with a scalar decay g and a
//     scalar rate beta per head and unit q, k.  Expanded, S_t = g S_(t-1) - (g beta k)(k^T S_(t-1)) + (beta k) v^T: the
//     general form with u = k, a*u = g beta k, w = g in every channel and beta k as the written key.  Its q, k, v first
//     pass a short causal convolution per channel (the last taps - 1 inputs of a sequence are kept per slot) and silu.
//   * decay with a bonus for the current token:  o_t = (S_(t-1) + diag(b) k_t v_t^T)^T r_t;  S_t = diag(w_t) S_(t-1) + k_t v_t^T.
//     The read-out comes before the write: o_t[j] = r_t . S_(t-1)[:, j] + (sum_i r_i b_i k_i) v_t[j], so the column
//     kernel's dot product runs over r and the scalar in front of v_t[j] is prepared per (token, head) (READ_FIRST).
#include "common.cuh"

#include <cstdlib>

namespace zl {

constexpr int kDrChunk = 16;   // tokens staged at a time (fewer when a head's vectors are too large for two such buffers)

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
    float* prep;                         // (T, H, 5 * dk + dv): u, a*u, w, k, r, v of every token and head
    int chunk;                           // tokens staged at a time
};

// The token vectors of the recurrence, for all tokens at once: one warp per (token, head).  grid (ceil(H / 4), T)
__global__ void __launch_bounds__(128) k_delta_prep(DeltaP p) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= p.H) return;
    const int dk = p.dk;
    const float* kr = p.k + (size_t)t * p.ld_k + (size_t)h * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss = fmaf(kr[i], kr[i], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) + p.unit_eps);
    float* tv = p.prep + ((size_t)t * p.H + h) * (5 * dk + p.dv);
    for (int i = lane; i < dk; i += 32) {
        const float kk = kr[i], u = kk * inv;
        const float a = 1.0f / (1.0f + expf(-p.rate_logit[(size_t)t * p.ld_a + (size_t)h * dk + i]));
        const float sg_w = 1.0f / (1.0f + expf(-p.decay_logit[(size_t)t * p.ld_w + (size_t)h * dk + i]));
        tv[i] = u;
        tv[dk + i] = a * u;
        tv[2 * dk + i] = expf(-p.decay_scale * sg_w);
        tv[3 * dk + i] = kk;
        tv[4 * dk + i] = p.r[(size_t)t * p.ld_r + (size_t)h * dk + i];
    }
    for (int j = lane; j < p.dv; j += 32) tv[5 * dk + j] = p.v[(size_t)t * p.ld_v + (size_t)h * p.dv + j];
}

__device__ __forceinline__ void dr_cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void dr_cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void dr_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void dr_cp_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// grid (dv / cols rounded up, H, runs); block = cols rounded up to a warp.  DK > 0: the column in registers.
// The prepared vectors of the next chunk of tokens fly into the other half of the shared buffer (cp.async) while the
// threads update their columns for the current chunk, so that no load sits on the chain from token to token.
template <int DK, bool READ_FIRST>
__global__ void k_delta_rule(DeltaP p) {
    extern __shared__ __align__(16) float dsm[];
    const int dk = DK > 0 ? DK : p.dk;
    const int per = 5 * dk + p.dv;                      // floats per (token, head)
    float* tok = dsm;                                   // [2][kDrChunk][per]
    float* scol = dsm + (size_t)2 * p.chunk * per;      // DK == 0: [dk][blockDim] the columns of this CTA
    pdl_trigger();
    pdl_wait();
    const int run = blockIdx.z, h = blockIdx.y, tid = threadIdx.x, nth = blockDim.x;
    const int row0 = p.run_row0[run], len = p.run_len[run];
    if (len <= 0) return;
    const int j = blockIdx.x * p.cols + tid;            // my value channel
    const bool mine = tid < p.cols && j < p.dv;
    float* sg = static_cast<float*>(p.state_addrs[p.slot[row0]]) + (size_t)h * dk * p.dv;
    const bool fresh = p.pos[row0] == 0;
    const bool vec = (per & 3) == 0;
    auto stage = [&](int buf, int c0) {
        const int cn = min(p.chunk, len - c0);
        float* dst = tok + (size_t)buf * p.chunk * per;
        for (int tt = 0; tt < cn; ++tt) {
            const float* src = p.prep + ((size_t)(row0 + c0 + tt) * p.H + h) * per;
            if (vec)
                for (int i = tid * 4; i < per; i += nth * 4) dr_cp_async16(dst + (size_t)tt * per + i, src + i);
            else
                for (int i = tid; i < per; i += nth) dr_cp_async4(dst + (size_t)tt * per + i, src + i);
        }
    };
    stage(0, 0);
    dr_cp_commit();
    float S[DK > 0 ? DK : 1];
    if (mine) {
        if constexpr (DK > 0) {
#pragma unroll
            for (int i = 0; i < DK; ++i) S[i] = fresh ? 0.f : sg[(size_t)i * p.dv + j];
        } else {
            for (int i = 0; i < dk; ++i) scol[(size_t)i * nth + tid] = fresh ? 0.f : sg[(size_t)i * p.dv + j];
        }
    }
    int buf = 0;
    for (int c0 = 0; c0 < len; c0 += p.chunk, buf ^= 1) {
        const int cn = min(p.chunk, len - c0);
        dr_cp_wait_all();
        __syncthreads();   // this chunk has landed for every thread; the other half is no longer read
        if (c0 + p.chunk < len) stage(buf ^ 1, c0 + p.chunk);
        dr_cp_commit();
        if (!mine) continue;
        for (int tt = 0; tt < cn; ++tt) {
            const size_t t = (size_t)(row0 + c0 + tt);
            const float* tv = tok + ((size_t)buf * p.chunk + tt) * per;
            const float vj = tv[5 * dk + blockIdx.x * p.cols + tid];
            float out = 0.f;
            if constexpr (DK > 0) {
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;   // four chains; added in a fixed order
#pragma unroll
                for (int i = 0; i < DK; i += 4) {
                    const float4 u = *reinterpret_cast<const float4*>(tv + i);
                    d0 = fmaf(u.x, S[i], d0), d1 = fmaf(u.y, S[i + 1], d1), d2 = fmaf(u.z, S[i + 2], d2), d3 = fmaf(u.w, S[i + 3], d3);
                }
                const float dot = (d0 + d1) + (d2 + d3);
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
                if constexpr (READ_FIRST) {
#pragma unroll
                    for (int i = 0; i < DK; i += 4) {
                        const float4 w = *reinterpret_cast<const float4*>(tv + 2 * DK + i);
                        const float4 kk = *reinterpret_cast<const float4*>(tv + 3 * DK + i);
                        S[i] = fmaf(kk.x, vj, w.x * S[i]);
                        S[i + 1] = fmaf(kk.y, vj, w.y * S[i + 1]);
                        S[i + 2] = fmaf(kk.z, vj, w.z * S[i + 2]);
                        S[i + 3] = fmaf(kk.w, vj, w.w * S[i + 3]);
                    }
                    out = fmaf(tv[4 * DK], vj, dot);
                } else {
#pragma unroll
                for (int i = 0; i < DK; i += 4) {
                    const float4 au = *reinterpret_cast<const float4*>(tv + DK + i);
                    const float4 w = *reinterpret_cast<const float4*>(tv + 2 * DK + i);
                    const float4 kk = *reinterpret_cast<const float4*>(tv + 3 * DK + i);
                    const float4 rr = *reinterpret_cast<const float4*>(tv + 4 * DK + i);
                    S[i] = fmaf(kk.x, vj, fmaf(-au.x, dot, w.x * S[i]));
                    S[i + 1] = fmaf(kk.y, vj, fmaf(-au.y, dot, w.y * S[i + 1]));
                    S[i + 2] = fmaf(kk.z, vj, fmaf(-au.z, dot, w.z * S[i + 2]));
                    S[i + 3] = fmaf(kk.w, vj, fmaf(-au.w, dot, w.w * S[i + 3]));
                    o0 = fmaf(S[i], rr.x, o0), o1 = fmaf(S[i + 1], rr.y, o1), o2 = fmaf(S[i + 2], rr.z, o2), o3 = fmaf(S[i + 3], rr.w, o3);
                }
                out = (o0 + o1) + (o2 + o3);
                }
            } else {
                float dot = 0.f;
                for (int i = 0; i < dk; ++i) dot = fmaf(tv[i], scol[(size_t)i * nth + tid], dot);
                if constexpr (READ_FIRST) {
                    for (int i = 0; i < dk; ++i)
                        scol[(size_t)i * nth + tid] = fmaf(tv[3 * dk + i], vj, tv[2 * dk + i] * scol[(size_t)i * nth + tid]);
                    out = fmaf(tv[4 * dk], vj, dot);
                } else {
                    for (int i = 0; i < dk; ++i) {
                        const float s = fmaf(tv[3 * dk + i], vj, fmaf(-tv[dk + i], dot, tv[2 * dk + i] * scol[(size_t)i * nth + tid]));
                        scol[(size_t)i * nth + tid] = s;
                        out = fmaf(s, tv[4 * dk + i], out);
                    }
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

// tokens per staging buffer: kDrChunk, or as many as keep the two buffers within 96 KB (at least one)
static int delta_chunk(int dk, int dv) {
    const size_t per = (size_t)(5 * dk + dv) * sizeof(float);
    size_t c = (96 * 1024) / (2 * per);
    return c >= (size_t)kDrChunk ? kDrChunk : (c < 1 ? 1 : (int)c);
}
static size_t delta_smem(int DK, int dk, int dv, int block) {
    size_t smem = (size_t)2 * delta_chunk(dk, dv) * (5 * dk + dv) * sizeof(float);
    if (DK == 0) smem += (size_t)dk * block * sizeof(float);
    return smem;
}

template <int DK, bool READ_FIRST>
static int launch_delta(const DeltaP& p, int runs, int block, bool pdl, cudaStream_t st) {
    const size_t smem = delta_smem(DK, p.dk, p.dv, block);
    if (smem > 48 * 1024) {
        static size_t set_for = 0;
        if (smem > set_for) {
            ZL_CHECK_CUDA(cudaFuncSetAttribute(k_delta_rule<DK, READ_FIRST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            set_for = smem;
        }
    }
    ZL_CHECK_CUDA(launch(k_delta_rule<DK, READ_FIRST>, dim3(cdiv(p.dv, p.cols), p.H, runs), dim3(block), smem, st, pdl, p));
    return ZL_OK;
}

// The same recurrence with a column of S spread over LANES adjacent lanes: a lane holds DK / LANES entries of its column in
// registers -- the 4-element pieces f = LANES i + q of the key dimension, so that the lanes' 16-byte reads of a staged
// vector fall into different banks -- and the dot products are finished with log2(LANES) shuffles.  A head then occupies
// LANES warps per 32 columns instead of one: a prompt of one sequence runs on heads * dv / 32 CTAs only, each token is a
// dependent chain, and one warp per scheduler issues an instruction every 4 - 5 cycles; more warps with fewer instructions
// each is what shortens it.  The sums are taken in an order fixed by the token (piece by piece, then over the lanes),
// whatever the step.  grid (dv / 32 rounded up, H, runs); block 32 * LANES.
template <int DK, int LANES, bool READ_FIRST>
__global__ void __launch_bounds__(32 * LANES) k_delta_rule_quad(DeltaP p) {
    extern __shared__ __align__(16) float dsm[];
    constexpr int Q = DK / LANES, NT = 32 * LANES;      // entries per lane (a multiple of 4), threads
    static_assert(Q % 4 == 0 && Q >= 4, "a lane holds whole 4-element pieces");
    const int per = 5 * DK + p.dv;
    float* tok = dsm;                                   // [2][chunk][per]
    pdl_trigger();
    pdl_wait();
    const int run = blockIdx.z, h = blockIdx.y, tid = threadIdx.x;
    const int row0 = p.run_row0[run], len = p.run_len[run];
    if (len <= 0) return;
    const int q = tid % LANES, col = tid / LANES;       // my share of the keys, my column inside the CTA
    const int j = blockIdx.x * 32 + col;                // my value channel
    const bool mine = j < p.dv;                         // the lanes of a column agree
    float* sg = static_cast<float*>(p.state_addrs[p.slot[row0]]) + (size_t)h * DK * p.dv;
    const bool fresh = p.pos[row0] == 0;
    auto stage = [&](int buf, int c0) {
        const int cn = min(p.chunk, len - c0);
        float* dst = tok + (size_t)buf * p.chunk * per;
        const float* src = p.prep + ((size_t)(row0 + c0) * p.H + h) * per;
        for (int tt = 0; tt < cn; ++tt, dst += per, src += (size_t)p.H * per)
            for (int i = tid * 4; i < per; i += NT * 4) dr_cp_async16(dst + i, src + i);
    };
    stage(0, 0);
    dr_cp_commit();
    // S[4 i + c] is key (LANES i + q) * 4 + c of my column
    float S[Q];
#pragma unroll
    for (int m = 0; m < Q; ++m) S[m] = (fresh || !mine) ? 0.f : sg[(size_t)((LANES * (m >> 2) + q) * 4 + (m & 3)) * p.dv + j];
    float* optr = p.o + (size_t)row0 * p.ld_o + (size_t)h * p.dv + j;
    const int vcol = 5 * DK + (mine ? j : 0);
    int buf = 0;
    for (int c0 = 0; c0 < len; c0 += p.chunk, buf ^= 1) {
        const int cn = min(p.chunk, len - c0);
        dr_cp_wait_all();
        __syncthreads();   // this chunk has landed for every thread; the other half is no longer read
        if (c0 + p.chunk < len) stage(buf ^ 1, c0 + p.chunk);
        dr_cp_commit();
        const float* tv = tok + (size_t)buf * p.chunk * per;
        for (int tt = 0; tt < cn; ++tt, tv += per, optr += p.ld_o) {
            const float vj = mine ? tv[vcol] : 0.f;
            const float4* mq = reinterpret_cast<const float4*>(tv) + q;   // piece i of a vector at DK/4 * vector + LANES * i
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int i = 0; i < Q / 4; ++i) {
                const float4 u = mq[LANES * i];
                d0 = fmaf(u.x, S[4 * i], d0), d1 = fmaf(u.y, S[4 * i + 1], d1), d2 = fmaf(u.z, S[4 * i + 2], d2), d3 = fmaf(u.w, S[4 * i + 3], d3);
            }
            float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
            for (int x = 1; x < LANES; x <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, x);
            float out;
            if constexpr (READ_FIRST) {
#pragma unroll
                for (int i = 0; i < Q / 4; ++i) {
                    const float4 w = mq[2 * (DK / 4) + LANES * i];
                    const float4 kk = mq[3 * (DK / 4) + LANES * i];
                    S[4 * i] = fmaf(kk.x, vj, w.x * S[4 * i]);
                    S[4 * i + 1] = fmaf(kk.y, vj, w.y * S[4 * i + 1]);
                    S[4 * i + 2] = fmaf(kk.z, vj, w.z * S[4 * i + 2]);
                    S[4 * i + 3] = fmaf(kk.w, vj, w.w * S[4 * i + 3]);
                }
                out = fmaf(tv[4 * DK], vj, dot);
            } else {
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
                for (int i = 0; i < Q / 4; ++i) {
                    const float4 au = mq[(DK / 4) + LANES * i];
                    const float4 w = mq[2 * (DK / 4) + LANES * i];
                    const float4 kk = mq[3 * (DK / 4) + LANES * i];
                    const float4 rr = mq[4 * (DK / 4) + LANES * i];
                    S[4 * i] = fmaf(kk.x, vj, fmaf(-au.x, dot, w.x * S[4 * i]));
                    S[4 * i + 1] = fmaf(kk.y, vj, fmaf(-au.y, dot, w.y * S[4 * i + 1]));
                    S[4 * i + 2] = fmaf(kk.z, vj, fmaf(-au.z, dot, w.z * S[4 * i + 2]));
                    S[4 * i + 3] = fmaf(kk.w, vj, fmaf(-au.w, dot, w.w * S[4 * i + 3]));
                    o0 = fmaf(S[4 * i], rr.x, o0), o1 = fmaf(S[4 * i + 1], rr.y, o1), o2 = fmaf(S[4 * i + 2], rr.z, o2), o3 = fmaf(S[4 * i + 3], rr.w, o3);
                }
                out = (o0 + o1) + (o2 + o3);
#pragma unroll
                for (int x = 1; x < LANES; x <<= 1) out += __shfl_xor_sync(0xffffffffu, out, x);
            }
            if (mine && q == 0) *optr = out;
        }
    }
    if (mine) {
#pragma unroll
        for (int m = 0; m < Q; ++m) sg[(size_t)((LANES * (m >> 2) + q) * 4 + (m & 3)) * p.dv + j] = S[m];
    }
}

template <int DK, int LANES, bool READ_FIRST>
static int launch_delta_quad(const DeltaP& p, int runs, bool pdl, cudaStream_t st) {
    const size_t smem = delta_smem(DK, p.dk, p.dv, 32 * LANES);
    if (smem > 48 * 1024) {
        static size_t set_for = 0;
        if (smem > set_for) {
            ZL_CHECK_CUDA(cudaFuncSetAttribute(k_delta_rule_quad<DK, LANES, READ_FIRST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            set_for = smem;
        }
    }
    ZL_CHECK_CUDA(launch(k_delta_rule_quad<DK, LANES, READ_FIRST>, dim3(cdiv(p.dv, 32), p.H, runs), dim3(32 * LANES), smem, st, pdl, p));
    return ZL_OK;
}

// the column kernel over prepared token vectors: registers for the compiled key sizes, shared memory otherwise
template <bool READ_FIRST>
static int run_columns(DeltaP& p, int runs, bool pdl, cudaStream_t st) {
    // a warp of columns per CTA spreads one sequence over heads * dv / 32 CTAs
    p.cols = 32;
    const int block = 32;
    static const bool no_reg_env = getenv("ZL_DELTA_NO_REG") != nullptr;
    static const bool no_quad = getenv("ZL_DELTA_NO_QUAD") != nullptr;
    const bool no_reg = no_reg_env || (5 * p.dk + p.dv) % 4 != 0;   // the register kernel reads the staged vectors 16 bytes at a time
    static const int lanes_env = getenv("ZL_DELTA_LANES") ? atoi(getenv("ZL_DELTA_LANES")) : 4;
    if (!no_reg && !no_quad) {   // a column over 4 or 8 adjacent lanes
        if (lanes_env == 4) {
            if (p.dk == 32) return launch_delta_quad<32, 4, READ_FIRST>(p, runs, pdl, st);
            if (p.dk == 64) return launch_delta_quad<64, 4, READ_FIRST>(p, runs, pdl, st);
            if (p.dk == 128) return launch_delta_quad<128, 4, READ_FIRST>(p, runs, pdl, st);
        } else {
            if (p.dk == 32) return launch_delta_quad<32, 8, READ_FIRST>(p, runs, pdl, st);
            if (p.dk == 64) return launch_delta_quad<64, 8, READ_FIRST>(p, runs, pdl, st);
            if (p.dk == 128) return launch_delta_quad<128, 8, READ_FIRST>(p, runs, pdl, st);
        }
    }
    if (!no_reg && p.dk == 32) return launch_delta<32, READ_FIRST>(p, runs, block, pdl, st);
    if (!no_reg && p.dk == 64) return launch_delta<64, READ_FIRST>(p, runs, block, pdl, st);
    if (!no_reg && p.dk == 128) return launch_delta<128, READ_FIRST>(p, runs, block, pdl, st);
    if (zl_delta_rule_prepare(p.dk, p.dv) != ZL_OK) return ZL_ERR_UNSUPPORTED;
    return launch_delta<0, READ_FIRST>(p, runs, block, pdl, st);
}

// ---- gated delta rule with short convolutions --------------------------------------------------------------------------
struct GatedPrepP {
    const float* proj;          // (T, ld): q | k | v at col_qkv (G*dk, G*dk, H*dv channels), rate logits (H) at col_b, decay inputs (H) at col_a
    long long ld;
    int col_qkv, col_b, col_a;
    int H, G, dk, dv, taps;
    const float* conv_w;        // (C, taps), C = 2 G dk + H dv, the last tap is the current token's
    const float *a_log, *dt_bias;   // (H)
    void* const* ring_addrs;    // slot -> (taps - 1, C) fp32: input at position p sits in entry p % (taps - 1)
    const int32_t *slot, *pos;
    float unit_eps, q_scale;
    int store_ring;             // every row is a run of its own: the kernel also stores its input into the ring
    float* prep;
};

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// One CTA per (token, q / k head): convolution + silu of that head's q and k channels and of the v channels of the value
// heads that use it into shared memory, then a warp per value head writes the token vectors.  No channel is shared between
// CTAs, so a channel's ring entries are read and (store_ring) overwritten by one thread.  grid (T, G)
__global__ void __launch_bounds__(128) k_gated_delta_prep(GatedPrepP p) {
    extern __shared__ float gsm[];   // q (dk) | k (dk) | v (rep * dv)
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dk = p.dk, rep = p.H / p.G, nr = p.taps - 1;
    const int C = 2 * p.G * dk + p.H * p.dv, n_mine = 2 * dk + rep * p.dv;
    const int sl = p.slot[t], pos = p.pos[t];
    const float* row = p.proj + (size_t)t * p.ld + p.col_qkv;
    float* ring = nr > 0 ? static_cast<float*>(p.ring_addrs[sl]) : nullptr;
    // how many earlier rows of this step belong to the same sequence (at most taps - 1 matter)
    int back = 0;
    while (back < nr && t - back - 1 >= 0 && p.slot[t - back - 1] == sl) ++back;
    for (int i = threadIdx.x; i < n_mine; i += blockDim.x) {
        // local index -> channel among q | k | v of all heads
        const int c = i < dk ? g * dk + i : (i < 2 * dk ? p.G * dk + g * dk + (i - dk) : 2 * p.G * dk + g * rep * p.dv + (i - 2 * dk));
        const float* w = p.conv_w + (size_t)c * p.taps;
        const float cur = row[c];
        float acc = w[nr] * cur;
        for (int j = 1; j <= nr; ++j) {   // the input j positions back
            const int pj = pos - j;
            if (pj < 0) break;
            const float xin = j <= back ? row[c - (long long)j * p.ld] : ring[(size_t)(pj % nr) * C + c];
            acc = fmaf(w[nr - j], xin, acc);
        }
        if (p.store_ring && nr > 0) ring[(size_t)(pos % nr) * C + c] = cur;
        gsm[i] = silu_f(acc);
    }
    __syncthreads();
    const float* q = gsm;
    const float* k = gsm + dk;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < dk; i += 32) sq = fmaf(q[i], q[i], sq), sk = fmaf(k[i], k[i], sk);
    const float iq = p.q_scale / sqrtf(warp_sum(sq) + p.unit_eps), ik = 1.0f / sqrtf(warp_sum(sk) + p.unit_eps);
    const float* prow = p.proj + (size_t)t * p.ld;
    for (int hh = warp; hh < rep; hh += (int)(blockDim.x >> 5)) {
        const int h = g * rep + hh;
        const float* v = gsm + 2 * dk + (size_t)hh * p.dv;
        const float beta = 1.0f / (1.0f + expf(-prow[p.col_b + h]));
        const float decay = expf(-expf(p.a_log[h]) * softplus_f(prow[p.col_a + h] + p.dt_bias[h]));
        float* tv = p.prep + ((size_t)t * p.H + h) * (5 * dk + p.dv);
        for (int i = lane; i < dk; i += 32) {
            const float u = k[i] * ik;
            tv[i] = u;
            tv[dk + i] = decay * beta * u;
            tv[2 * dk + i] = decay;
            tv[3 * dk + i] = beta * u;
            tv[4 * dk + i] = q[i] * iq;
        }
        for (int j = lane; j < p.dv; j += 32) tv[5 * dk + j] = v[j];
    }
}

// The last n_tail rows of every run of a (T, ld) fp32 matrix, columns col .. col + C, into the slots' rings
// (slot -> (n_tail, C)): the row at position p goes to entry p % n_tail.  grid (runs, n_tail)
__global__ void __launch_bounds__(256) k_store_run_tails(const float* __restrict__ src, long long ld, int col, int C, int n_tail,
                                                         const int32_t* __restrict__ run_row0, const int32_t* __restrict__ run_len,
                                                         const int32_t* __restrict__ slot, const int32_t* __restrict__ pos,
                                                         void* const* ring_addrs) {
    pdl_trigger();
    pdl_wait();
    const int run = blockIdx.x, j = blockIdx.y, len = run_len[run];
    if (j >= len) return;
    const int row = run_row0[run] + len - 1 - j;
    float* dst = static_cast<float*>(ring_addrs[slot[row]]) + (size_t)(pos[row] % n_tail) * C;
    const float* s = src + (size_t)row * ld + col;
    for (int c = threadIdx.x; c < C; c += blockDim.x) dst[c] = s[c];
}

// ---- decay with a bonus for the current token ---------------------------------------------------------------------------
struct BonusPrepP {
    const float *r, *k, *v, *decay_logit;   // (T, H * dk) / v (T, H * dv)
    long long ld_r, ld_k, ld_v, ld_w;
    const float* bonus;                     // (H, dk)
    int H, dk, dv;
    float* prep;
};
// one warp per (token, head).  grid (ceil(H / 4), T).  w = exp(-exp(decay_logit))
__global__ void __launch_bounds__(128) k_bonus_decay_prep(BonusPrepP p) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= p.H) return;
    const int dk = p.dk;
    const float* rr = p.r + (size_t)t * p.ld_r + (size_t)h * dk;
    const float* kr = p.k + (size_t)t * p.ld_k + (size_t)h * dk;
    const float* wr = p.decay_logit + (size_t)t * p.ld_w + (size_t)h * dk;
    const float* bo = p.bonus + (size_t)h * dk;
    float* tv = p.prep + ((size_t)t * p.H + h) * (5 * dk + p.dv);
    float s = 0.f;
    for (int i = lane; i < dk; i += 32) {
        const float r = rr[i], k = kr[i];
        s = fmaf(r * bo[i], k, s);
        tv[i] = r;
        tv[dk + i] = 0.f;
        tv[2 * dk + i] = expf(-expf(wr[i]));
        tv[3 * dk + i] = k;
        if (i > 0) tv[4 * dk + i] = 0.f;
    }
    s = warp_sum(s);
    if (lane == 0) tv[4 * dk] = s;
    for (int j = lane; j < p.dv; j += 32) tv[5 * dk + j] = p.v[(size_t)t * p.ld_v + (size_t)h * p.dv + j];
}

}  // namespace zl

using namespace zl;

extern "C" int zl_delta_rule_prepare(int dim_k, int dim_v) {
    ZL_CHECK_ARG(dim_k > 0 && dim_v > 0);
    // the general kernel keeps its columns in shared memory: a warp of columns must fit beside the staged token vectors
    ZL_CHECK_SUPPORTED(delta_smem(0, dim_k, dim_v, 32) <= 200 * 1024);
    return ZL_OK;
}

extern "C" size_t zl_delta_rule_workspace_bytes(int T, int heads, int dim_k, int dim_v) {
    return (size_t)T * heads * (5 * dim_k + dim_v) * sizeof(float);
}

extern "C" int zl_delta_rule(const float* r, long long ld_r, const float* k, long long ld_k, const float* v, long long ld_v,
                             const float* rate_logit, long long ld_a, const float* decay_logit, long long ld_w,
                             float decay_scale, float unit_eps, const int32_t* run_row0, const int32_t* run_len, int runs,
                             const int32_t* slot, const int32_t* pos, void* const* state_addrs, float* o, long long ld_o,
                             int heads, int dim_k, int dim_v, int T, void* workspace, size_t workspace_bytes, int pdl,
                             zl_stream_t stream) {
    ZL_CHECK_ARG(r && k && v && rate_logit && decay_logit && run_row0 && run_len && slot && pos && state_addrs && o);
    ZL_CHECK_ARG(runs > 0 && runs <= 65535 && heads > 0 && heads <= 65535 && dim_k > 0 && dim_v > 0);
    ZL_CHECK_ARG(T > 0 && T <= 65535 && workspace && workspace_bytes >= zl_delta_rule_workspace_bytes(T, heads, dim_k, dim_v));
    DeltaP p{r, k, v, rate_logit, decay_logit, ld_r, ld_k, ld_v, ld_a, ld_w, run_row0, run_len, slot, pos, state_addrs, o, ld_o,
             heads, dim_k, dim_v, 0, decay_scale, unit_eps, static_cast<float*>(workspace), delta_chunk(dim_k, dim_v)};
    ZL_CHECK_CUDA(launch(k_delta_prep, dim3(cdiv(heads, 4), T), dim3(128), 0, stream, pdl != 0, p));
    return run_columns<false>(p, runs, pdl != 0, stream);
}

extern "C" int zl_store_run_tails(const float* src, long long ld, int col, int channels, int n_tail, const int32_t* run_row0,
                                  const int32_t* run_len, int runs, const int32_t* slot, const int32_t* pos,
                                  void* const* ring_addrs, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(src && run_row0 && run_len && slot && pos && ring_addrs && channels > 0 && n_tail > 0 && n_tail <= 65535);
    ZL_CHECK_ARG(runs > 0 && col >= 0 && ld >= col + channels);
    ZL_CHECK_CUDA(launch(k_store_run_tails, dim3(runs, n_tail), dim3(256), 0, stream, pdl != 0, src, ld, col, channels, n_tail,
                         run_row0, run_len, slot, pos, ring_addrs));
    return ZL_OK;
}

extern "C" int zl_gated_delta_rule(const float* proj, long long ld, int col_qkv, int col_rate, int col_decay,
                                   const float* conv_weight, int taps, const float* a_log, const float* dt_bias, float unit_eps,
                                   float q_scale, void* const* ring_addrs, const int32_t* run_row0, const int32_t* run_len,
                                   int runs, const int32_t* slot, const int32_t* pos, void* const* state_addrs, float* o,
                                   long long ld_o, int heads, int kv_heads, int dim_k, int dim_v, int T, void* workspace,
                                   size_t workspace_bytes, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(proj && conv_weight && a_log && dt_bias && run_row0 && run_len && slot && pos && state_addrs && o);
    ZL_CHECK_ARG(taps >= 1 && (taps == 1 || ring_addrs) && heads > 0 && kv_heads > 0 && heads % kv_heads == 0);
    ZL_CHECK_ARG(runs > 0 && runs <= 65535 && heads <= 65535 && dim_k > 0 && dim_v > 0);
    ZL_CHECK_ARG(T > 0 && T <= 65535 && workspace && workspace_bytes >= zl_delta_rule_workspace_bytes(T, heads, dim_k, dim_v));
    const int C = 2 * kv_heads * dim_k + heads * dim_v, n_cta = 2 * dim_k + heads / kv_heads * dim_v;
    ZL_CHECK_SUPPORTED((size_t)n_cta * 4 <= 200 * 1024 && kv_heads <= 65535);
    GatedPrepP g{proj, ld, col_qkv, col_rate, col_decay, heads, kv_heads, dim_k, dim_v, taps, conv_weight, a_log, dt_bias,
                 ring_addrs, slot, pos, unit_eps, q_scale, runs == T ? 1 : 0, static_cast<float*>(workspace)};
    const size_t smem = (size_t)n_cta * 4;
    if (smem > 48 * 1024) {
        static size_t set_for = 0;
        if (smem > set_for) {
            ZL_CHECK_CUDA(cudaFuncSetAttribute(k_gated_delta_prep, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            set_for = smem;
        }
    }
    ZL_CHECK_CUDA(launch(k_gated_delta_prep, dim3(T, kv_heads), dim3(128), smem, stream, pdl != 0, g));
    if (runs != T && taps > 1)   // rows of a run read ring entries that its last rows overwrite: stored afterwards
        if (int rc_ = (zl_store_run_tails(proj, ld, col_qkv, C, taps - 1, run_row0, run_len, runs, slot, pos, ring_addrs, pdl, stream))) return rc_;
    DeltaP p{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, run_row0, run_len, slot, pos, state_addrs, o, ld_o,
             heads, dim_k, dim_v, 0, 0.f, 0.f, static_cast<float*>(workspace), delta_chunk(dim_k, dim_v)};
    return run_columns<false>(p, runs, pdl != 0, stream);
}

extern "C" int zl_bonus_decay_scan(const float* r, long long ld_r, const float* k, long long ld_k, const float* v, long long ld_v,
                                   const float* decay_logit, long long ld_w, const float* bonus, const int32_t* run_row0,
                                   const int32_t* run_len, int runs, const int32_t* slot, const int32_t* pos,
                                   void* const* state_addrs, float* o, long long ld_o, int heads, int dim_k, int dim_v, int T,
                                   void* workspace, size_t workspace_bytes, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(r && k && v && decay_logit && bonus && run_row0 && run_len && slot && pos && state_addrs && o);
    ZL_CHECK_ARG(runs > 0 && runs <= 65535 && heads > 0 && heads <= 65535 && dim_k > 0 && dim_v > 0);
    ZL_CHECK_ARG(T > 0 && T <= 65535 && workspace && workspace_bytes >= zl_delta_rule_workspace_bytes(T, heads, dim_k, dim_v));
    BonusPrepP b{r, k, v, decay_logit, ld_r, ld_k, ld_v, ld_w, bonus, heads, dim_k, dim_v, static_cast<float*>(workspace)};
    ZL_CHECK_CUDA(launch(k_bonus_decay_prep, dim3(cdiv(heads, 4), T), dim3(128), 0, stream, pdl != 0, b));
    DeltaP p{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, run_row0, run_len, slot, pos, state_addrs, o, ld_o,
             heads, dim_k, dim_v, 0, 0.f, 0.f, static_cast<float*>(workspace), delta_chunk(dim_k, dim_v)};
    return run_columns<true>(p, runs, pdl != 0, stream);
}

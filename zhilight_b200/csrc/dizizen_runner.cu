// Host-side driver of the Dizizen model family: weights, slot caches, the per-step kernel chain and its CUDA graph.
// Same driver shape as kodupel_runner.cu (task slots, host (token, slot, position) rows in, logits / greedy picks out),
// built from the shared pieces of runner_common.cuh.
//
// x = scale * embed[token] in fp32 (the embedding kernel also writes the first layer's normed input).  A layer is parallel: h = norm1(x) (weight 1 + w) feeds both sublayers and
//   x += mult * (ls1 * sigmoid(W_rg1 h + b) * mixer(h) + ls2 * sigmoid(W_rg2 h + b) * ff(h)).
// Everything that is a Linear of h without an activation is ONE projection [W_q; W_k; W_v; W_rg1; W_rg2; W_router] with one
// bias vector and fp32 output: the attention operands, both gates' logits and the router's logits are columns of it.
//   attention:  rotation tables of the step (mixer_rows.cu: one (cos, sin) table per distinct (base, size), angles in
//               double) -> q, k turned in halves over rot_dims, v turned over all of vdim, appended to the slot's caches
//               -> causal softmax attention whose epilogue turns every head's sum back by the query's position
//               (sink_attn.cu) -> W_o with bias.  A layer with kv_from reads another layer's caches.
//   dense ff:   [W_gate; W_up] with rows interleaved and the clamped gated unit as the epilogue, then W_down with bias.
//   experts:    routing on the device from the projection's logit columns (moe_route.cu: softmax scores, choice inside the
//               best groups, identity slots sorted behind the experts) -> two grouped GEMMs over the (token, choice)
//               pairs of real experts, relu^2 as the first one's epilogue -> the shared expert as two plain GEMMs.
//   combine:    one kernel per layer takes both results, the gates' logits, the layer scales, the routing weights (pairs
//               of identity slots read norm1(x) recomputed in place), updates x and writes the next layer's h.
// One step takes T rows in any mix of prompt portions and single decode tokens; every kernel indexes caches by
// (slot, position).
#include "runner_common.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace {

using namespace zl;

struct DLayer {
    zl_dizizen_layer_t c{};
    float* norm1 = nullptr;                      // 1 + w
    float *ls1 = nullptr, *ls2 = nullptr;
    void* w_in = nullptr;                        // fused projection (n_in, width)
    float* b_in = nullptr;                       // its bias, fp32 (zeros for the router's rows)
    void* b_in_act = nullptr;                    // the same in the activation dtype (skinny kernel)
    int n_in = 0, q_off = 0, k_off = -1, v_off = 0, g1_off = 0, g2_off = -1, r_off = -1;
    void* o = nullptr;                           // (width, heads * vdim)
    float* o_b = nullptr;
    void* o_b_act = nullptr;
    int qk_rot = -1, v_rot = -1;                 // indices into the model's rotation tables
    SlotCache kcache, vcache;
    void **k_addrs = nullptr, **v_addrs = nullptr;   // own or the source layer's
    // dense feed-forward
    void* w_gu = nullptr;                        // (2 * ff, width): rows 2j / 2j+1 = gate_j / up_j
    float* b_gu = nullptr;                       // (2 * ff) interleaved alike
    void* w_down = nullptr;                      // dense: (width, ff); experts: (experts, width, ff)
    float* b_down = nullptr;
    void* b_down_act = nullptr;
    // experts
    float* correction = nullptr;                 // (experts + identity)
    void* w_up = nullptr;                        // (experts, ff, width)
    void *s_up = nullptr, *s_down = nullptr;     // shared expert (shared_ff, width), (width, shared_ff)
    bool ready = false;
};

// one (cos, sin) table per distinct (base, rotated size): filled once per step from the rows' positions
struct RotTable {
    double base = 0;
    int dims = 0;
    double* inv_freq = nullptr;   // device (dims / 2)
    float* table = nullptr;       // device (tcap, dims / 2) float pairs
};

}  // namespace

struct zl_dizizen {
    zl_dizizen_config_t cfg{};
    cudaStream_t stream = nullptr;
    cudaStream_t side = nullptr;                 // the feed-forward branch of a layer runs here beside the mixer
    std::vector<cudaEvent_t> ev_h, ev_proj, ev_ff;   // per layer: h ready, projection ready (main) / feed-forward done (side)
    StagedMap staged;
    std::vector<DLayer> layers;
    std::vector<RotTable> rots;
    void *embed = nullptr, *head = nullptr;
    float* final_norm = nullptr;
    bool finalized = false;
    int esz = 2;
    int tcap = 0;
    float *x = nullptr, *proj = nullptr, *ya = nullptr, *yf = nullptr, *ypair = nullptr, *xw = nullptr, *logits = nullptr,
          *top_w = nullptr;
    void *h = nullptr, *q = nullptr, *att = nullptr, *act = nullptr, *act_s = nullptr, *xn = nullptr;
    int32_t *d_tokens = nullptr, *d_slots = nullptr, *d_pos = nullptr, *d_want = nullptr, *d_next = nullptr;
    int32_t *d_run0 = nullptr, *d_runlen = nullptr, *top_e = nullptr, *grp_off = nullptr, *list_token = nullptr,
            *list_pair = nullptr;
    int32_t* h_stage = nullptr;   // pinned: tokens | slots | pos | want | next | run0 | runlen
    void* attn_ws = nullptr;
    size_t attn_ws_bytes = 0;
    void* argmax_ws = nullptr;
    float* layer_dump = nullptr;
    bool capture = false;
    std::map<long long, cudaGraphExec_t> graphs;
    int cur_max_len = 0;
    double weight_bytes = 0;
    int kernels_per_step = 0;
};

namespace {

int fail(int line, const std::string& msg, int code = ZL_ERR_STATE) {
    zl_set_last_error(__FILE__, line, msg.c_str());
    return code;
}

int rot_index(zl_dizizen* m, double base, int dims) {
    for (size_t i = 0; i < m->rots.size(); ++i)
        if (m->rots[i].base == base && m->rots[i].dims == dims) return (int)i;
    RotTable r;
    r.base = base;
    r.dims = dims;
    m->rots.push_back(r);
    return (int)m->rots.size() - 1;
}

// x[t] = scale * embed[token[t]] in fp32 and the first layer's input h[t] = w * x[t] / sqrt(mean(x[t]^2) + eps) in the
// activation dtype; one CTA per token, the row in registers for widths up to 8 * 256
template <typename TW, typename TO>
__global__ void __launch_bounds__(256) k_embed_scaled_norm(const int32_t* __restrict__ ids, const TW* __restrict__ table,
                                                           const float* __restrict__ w, float* __restrict__ x, TO* __restrict__ h,
                                                           int D, int vocab, float scale, float eps) {
    __shared__ float red[8];
    int id = ids[blockIdx.x];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const TW* src = table + (size_t)id * D;
    float* xr = x + (size_t)blockIdx.x * D;
    float keep[8], ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * 256;
        keep[i] = c < D ? to_f32<TW>(src[c]) * scale : 0.f;
        if (c < D) xr[c] = keep[i];
        ss = fmaf(keep[i], keep[i], ss);
    }
    for (int c = threadIdx.x + 2048; c < D; c += 256) {
        const float v = to_f32<TW>(src[c]) * scale;
        xr[c] = v;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float r = 1.0f / sqrtf(tot / (float)D + eps);
    TO* hr = h + (size_t)blockIdx.x * D;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < D) hr[c] = from_f32<TO>(keep[i] * r * w[c]);
    }
    for (int c = threadIdx.x + 2048; c < D; c += 256) hr[c] = from_f32<TO>(xr[c] * r * w[c]);
}

int finalize_ff(zl_dizizen* m, int l) {
    DLayer& L = m->layers[l];
    const auto& lc = L.c;
    const int D = m->cfg.width, F = lc.ff;
    const std::string p = "l" + std::to_string(l) + ".mlp.";
    if (lc.ff_kind == ZL_FF_DENSE) {
        RCHECK(dmalloc(&L.w_gu, (size_t)2 * F * D * m->esz));
        RCHECK(put_interleaved(m, p + "gate", p + "up", F, D, L.w_gu, 0, false));
        RCHECK(dmalloc((void**)&L.b_gu, (size_t)2 * F * 4));
        RCHECK(put_interleaved(m, p + "gate.b", p + "up.b", F, 1, L.b_gu, 0, true));
        RCHECK(take_weight(m, p + "down", D, F, &L.w_down));
        RCHECK(take_f32(m, p + "down.b", 1, D, &L.b_down));
        RCHECK(bias_copy_act(m, L.b_down, D, &L.b_down_act));
        return ZL_OK;
    }
    const int E = lc.experts;
    RCHECK(take_f32(m, p + "correction", 1, E + lc.identity, &L.correction));
    RCHECK(dmalloc(&L.w_up, (size_t)std::max(E, 1) * F * D * m->esz));
    RCHECK(dmalloc(&L.w_down, (size_t)std::max(E, 1) * D * F * m->esz));
    for (int e = 0; e < E; ++e) {
        const std::string pe = p + "e" + std::to_string(e) + ".";
        RCHECK(put_weight(m, pe + "up", F, D, L.w_up, (size_t)e * F * D));
        RCHECK(put_weight(m, pe + "down", D, F, L.w_down, (size_t)e * D * F));
    }
    if (lc.shared_ff > 0) {
        RCHECK(take_weight(m, p + "shared.up", lc.shared_ff, D, &L.s_up));
        RCHECK(take_weight(m, p + "shared.down", D, lc.shared_ff, &L.s_down));
    }
    return ZL_OK;
}

int finalize_layer(zl_dizizen* m, int l) {
    const auto& c = m->cfg;
    DLayer& L = m->layers[l];
    const auto& lc = L.c;
    const std::string p = "l" + std::to_string(l) + ".", mx = p + "mix.";
    const int D = c.width, H = lc.heads, G = lc.kv_heads, d = lc.dim, vd = lc.vdim;
    const bool own = lc.kv_from < 0, ff = lc.ff_kind != ZL_FF_NONE, moe = lc.ff_kind == ZL_FF_MOE;
    const int slots = lc.experts + lc.identity;
    RCHECK(take_norm_plus_one(m, p + "norm1", D, &L.norm1));
    L.q_off = 0;
    L.k_off = own ? H * d : -1;
    L.v_off = own ? H * d + G * d : 0;
    // the gates' columns start at a multiple of 4 and the row has a multiple of 8 columns (rows of zeros in between), so that
    // the combine kernel reads its logits in 16-byte pieces whatever the head and slot counts are
    L.g1_off = (H * d + (own ? G * (d + vd) : 0) + 3) & ~3;
    L.g2_off = ff ? L.g1_off + D : -1;
    L.r_off = moe ? L.g1_off + 2 * D : -1;
    L.n_in = (L.g1_off + D + (ff ? D : 0) + (moe ? slots : 0) + 7) & ~7;
    RCHECK(dmalloc(&L.w_in, (size_t)L.n_in * D * m->esz));
    ZL_CHECK_CUDA(cudaMemsetAsync(L.w_in, 0, (size_t)L.n_in * D * m->esz, m->stream));
    RCHECK(dmalloc((void**)&L.b_in, (size_t)L.n_in * 4));
    ZL_CHECK_CUDA(cudaMemsetAsync(L.b_in, 0, (size_t)L.n_in * 4, m->stream));
    RCHECK(put_weight(m, mx + "q", H * d, D, L.w_in, 0));
    RCHECK(put_bias_f32(m, mx + "q.b", H * d, L.b_in, 0));
    if (own) {
        RCHECK(put_weight(m, mx + "k", G * d, D, L.w_in, (size_t)L.k_off * D));
        RCHECK(put_bias_f32(m, mx + "k.b", G * d, L.b_in, L.k_off));
        RCHECK(put_weight(m, mx + "v", G * vd, D, L.w_in, (size_t)L.v_off * D));
        RCHECK(put_bias_f32(m, mx + "v.b", G * vd, L.b_in, L.v_off));
    }
    RCHECK(put_weight(m, p + "rg1", D, D, L.w_in, (size_t)L.g1_off * D));
    RCHECK(put_bias_f32(m, p + "rg1.b", D, L.b_in, L.g1_off));
    RCHECK(take_f32(m, p + "ls1", 1, D, &L.ls1));
    if (ff) {
        RCHECK(put_weight(m, p + "rg2", D, D, L.w_in, (size_t)L.g2_off * D));
        RCHECK(put_bias_f32(m, p + "rg2.b", D, L.b_in, L.g2_off));
        RCHECK(take_f32(m, p + "ls2", 1, D, &L.ls2));
    }
    if (moe) RCHECK(put_weight(m, p + "mlp.router", slots, D, L.w_in, (size_t)L.r_off * D));
    RCHECK(take_weight(m, mx + "o", D, H * vd, &L.o));
    RCHECK(take_f32(m, mx + "o.b", 1, D, &L.o_b));
    RCHECK(bias_copy_act(m, L.o_b, D, &L.o_b_act));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    RCHECK(bias_copy_act(m, L.b_in, L.n_in, &L.b_in_act));
    if (ff) RCHECK(finalize_ff(m, l));
    L.qk_rot = lc.rot_dims > 0 ? rot_index(m, lc.rot_base, lc.rot_dims) : -1;
    L.v_rot = rot_index(m, lc.rot_base, vd);
    L.ready = true;
    return ZL_OK;
}

int len_bucket(const zl_dizizen* m, int max_len) {
    int b = 256;
    while (b < max_len) b <<= 1;
    return b < m->cfg.max_seq ? b : (m->cfg.max_seq > 256 ? m->cfg.max_seq : 256);
}

int alloc_runtime(zl_dizizen* m) {
    const auto& c = m->cfg;
    const int D = c.width, T = m->tcap, B = c.max_batch;
    size_t n_in = 1, hd = 1, hv = 1, ffw = 1, pairs_ff = 1, top = 1, slots = 1, sff = 1;
    for (auto& L : m->layers) {
        const auto& lc = L.c;
        if (lc.kv_from < 0) {
            RCHECK(L.kcache.create(B, (size_t)c.max_seq * lc.kv_heads * lc.dim * m->esz, m->stream));
            RCHECK(L.vcache.create(B, (size_t)c.max_seq * lc.kv_heads * lc.vdim * m->esz, m->stream));
            L.k_addrs = L.kcache.addrs;
            L.v_addrs = L.vcache.addrs;
        }
        for (int b = 1; b <= T; ++b) {
            const int s = zl_sink_attention_splits(b, lc.heads, lc.kv_heads, len_bucket(m, c.max_seq));
            m->attn_ws_bytes = std::max(m->attn_ws_bytes, zl_sink_attention_workspace_bytes(b, lc.heads, lc.vdim, s));
            if (s == 1) break;
        }
        n_in = std::max(n_in, (size_t)L.n_in);
        hd = std::max(hd, (size_t)lc.heads * lc.dim);
        hv = std::max(hv, (size_t)lc.heads * lc.vdim);
        if (lc.ff_kind == ZL_FF_DENSE) ffw = std::max(ffw, (size_t)lc.ff);
        if (lc.ff_kind == ZL_FF_MOE) {
            pairs_ff = std::max(pairs_ff, (size_t)lc.top * lc.ff);
            top = std::max(top, (size_t)lc.top);
            slots = std::max(slots, (size_t)(lc.experts + lc.identity));
            sff = std::max(sff, (size_t)lc.shared_ff);
        }
    }
    for (auto& L : m->layers)
        if (L.c.kv_from >= 0) {
            L.k_addrs = m->layers[L.c.kv_from].kcache.addrs;
            L.v_addrs = m->layers[L.c.kv_from].vcache.addrs;
        }
    for (auto& r : m->rots) {
        const int half = r.dims / 2;
        std::vector<double> f(half);
        for (int i = 0; i < half; ++i) f[i] = pow(r.base, -2.0 * i / r.dims);
        RCHECK(dmalloc((void**)&r.inv_freq, (size_t)half * 8));
        ZL_CHECK_CUDA(cudaMemcpy(r.inv_freq, f.data(), (size_t)half * 8, cudaMemcpyHostToDevice));
        RCHECK(dmalloc((void**)&r.table, (size_t)T * half * 8));
    }
    const size_t e = m->esz;
    RCHECK(dmalloc((void**)&m->x, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->proj, (size_t)T * n_in * 4));
    RCHECK(dmalloc((void**)&m->ya, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->yf, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->ypair, (size_t)T * top * D * 4));
    RCHECK(dmalloc((void**)&m->xw, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->logits, (size_t)T * c.vocab * 4));
    RCHECK(dmalloc((void**)&m->top_w, (size_t)T * top * 4));
    RCHECK(dmalloc(&m->h, (size_t)T * D * e));
    RCHECK(dmalloc(&m->q, (size_t)T * hd * e));
    RCHECK(dmalloc(&m->att, (size_t)T * hv * e));
    RCHECK(dmalloc(&m->act, (size_t)T * std::max(pairs_ff, ffw) * e));
    RCHECK(dmalloc(&m->act_s, (size_t)T * sff * e));
    RCHECK(dmalloc(&m->xn, (size_t)T * D * e));
    for (int32_t** p : {&m->d_tokens, &m->d_slots, &m->d_pos, &m->d_want, &m->d_next, &m->d_run0, &m->d_runlen})
        RCHECK(dmalloc((void**)p, (size_t)T * 4));
    RCHECK(dmalloc((void**)&m->top_e, (size_t)T * top * 4));
    RCHECK(dmalloc((void**)&m->list_token, (size_t)T * top * 4));
    RCHECK(dmalloc((void**)&m->list_pair, (size_t)T * top * 4));
    RCHECK(dmalloc((void**)&m->grp_off, (slots + 1) * 4));
    RCHECK(dmalloc(&m->attn_ws, m->attn_ws_bytes));
    RCHECK(dmalloc(&m->argmax_ws, zl_argmax_workspace_bytes(T)));
    ZL_CHECK_CUDA(cudaMallocHost((void**)&m->h_stage, sizeof(int32_t) * 7 * (size_t)T));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

// Which kernels of a step of at most 8 rows are launched with a programmatic dependency: 1 skinny Linears, 2 other GEMMs,
// 4 row kernels, 8 attention, 32 the tail.  Larger steps use none.  ZL_DIZIZEN_PDL_MASK overrides the default.
constexpr int kDefaultPdlMask = 1;
int pdl_mask() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("ZL_DIZIZEN_PDL_MASK");
        v = e ? atoi(e) : kDefaultPdlMask;
    }
    return v;
}
int pdl_for(const zl_dizizen* m, int bit, int T) { return (m->cfg.use_pdl && T <= 8 && (pdl_mask() & bit)) ? 1 : 0; }

// y (M, N) = x (M, K) @ w (N, K)^T + bias, optional relu^2.  bias_f32 / bias_act are the same numbers in two types.
int linear(zl_dizizen* m, cudaStream_t st, const void* x, int K, const void* w, int N, const float* bias_f32,
           const void* bias_act, void* y, int M, int out_dtype, int epi) {
    const auto& c = m->cfg;
    if (c.dtype != ZL_F32 && epi == ZL_GEMM_EPI_NONE && M <= 32 && K % 32 == 0 && N >= 64 && (!bias_f32 || bias_act) &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0)
        return zl_dense_gemm_skinny_act(x, K, w, bias_act, y, M, N, K, c.dtype, out_dtype, 0, pdl_for(m, 1, M), st);
    return zl_gemm_nt_bias(x, K, w, K, bias_f32, y, N, M, N, K, c.dtype, out_dtype, epi, pdl_for(m, 2, M), st);
}

int enqueue_step(zl_dizizen* m, int T, int n_want, int n_runs, int max_run, int max_len) {
    const auto& c = m->cfg;
    const int D = c.width, dt = c.dtype;
    cudaStream_t st = m->stream;
    const int pg = pdl_for(m, 2, T), pr = pdl_for(m, 4, T), pa = pdl_for(m, 8, T), pt = pdl_for(m, 32, T);
    if (dt == ZL_F32)
        ZL_CHECK_CUDA(launch(k_embed_scaled_norm<float, float>, dim3(T), dim3(256), 0, st, false, (const int32_t*)m->d_tokens,
                             (const float*)m->embed, (const float*)m->layers[0].norm1, m->x, (float*)m->h, D, c.vocab,
                             c.embed_scale, c.eps));
    else
        ZL_CHECK_CUDA(launch(k_embed_scaled_norm<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), 0, st, false,
                             (const int32_t*)m->d_tokens, (const __nv_bfloat16*)m->embed, (const float*)m->layers[0].norm1, m->x,
                             (__nv_bfloat16*)m->h, D, c.vocab, c.embed_scale, c.eps));
    for (auto& r : m->rots) RCHECK(zl_rope_table(m->d_pos, T, r.inv_freq, r.dims / 2, r.table, pr, st));
    // The two sublayers of a layer read the same h and meet only in the combine kernel: the feed-forward runs on a second
    // stream beside the mixer (fork after h, join before the combine; inside a captured step the events become graph edges).
    // A routed feed-forward needs the projection's logit columns, its shared expert does not.  ZL_DIZIZEN_ONE_STREAM=1: all
    // kernels on one stream in the order mixer, feed-forward.
    static const bool one_stream = getenv("ZL_DIZIZEN_ONE_STREAM") != nullptr;
    for (int l = 0; l < c.num_layers; ++l) {
        DLayer& L = m->layers[l];
        const auto& lc = L.c;
        const int H = lc.heads;
        const bool fork = !one_stream && lc.ff_kind != ZL_FF_NONE;
        cudaStream_t sf = fork ? m->side : st;
        if (fork) {
            ZL_CHECK_CUDA(cudaEventRecord(m->ev_h[l], st));
            ZL_CHECK_CUDA(cudaStreamWaitEvent(sf, m->ev_h[l], 0));
        }
        RCHECK(linear(m, st, m->h, D, L.w_in, L.n_in, L.b_in, L.b_in_act, m->proj, T, ZL_F32, ZL_GEMM_EPI_NONE));
        if (fork && lc.ff_kind == ZL_FF_MOE) ZL_CHECK_CUDA(cudaEventRecord(m->ev_proj[l], st));
        const float* vtab = m->rots[L.v_rot].table;
        RCHECK(zl_qkv_table_rope_append(m->proj, L.n_in, L.q_off, L.k_off, L.v_off, H, lc.kv_heads, lc.dim, lc.vdim,
                                        L.qk_rot >= 0 ? m->rots[L.qk_rot].table : nullptr, lc.rot_dims, vtab, ZL_ROT_HALVES, m->q,
                                        L.k_addrs, L.v_addrs, m->d_slots, m->d_pos, T, dt, pr, st));
        const int splits = zl_sink_attention_splits(T, H, lc.kv_heads, max_len);
        RCHECK(zl_sink_attention_ex(m->q, L.k_addrs, L.v_addrs, m->d_slots, m->d_pos, nullptr, 1, nullptr, 0, lc.scale, 0, nullptr,
                                    0, vtab, ZL_ROT_HALVES, m->att, T, H, lc.kv_heads, lc.dim, lc.vdim, splits, m->attn_ws,
                                    m->attn_ws_bytes, m->d_run0, m->d_runlen, n_runs, max_run, dt, pa, st));
        RCHECK(linear(m, st, m->att, H * lc.vdim, L.o, D, L.o_b, L.o_b_act, m->ya, T, ZL_F32, ZL_GEMM_EPI_NONE));
        const float *parts = nullptr, *f_dense = nullptr;
        if (lc.ff_kind == ZL_FF_DENSE) {
            RCHECK(zl_gemm_nt_glu_clamp(m->h, D, L.w_gu, D, L.b_gu, m->act, lc.ff, T, 2 * lc.ff, D, dt, dt, lc.limit, 1.702f, 1.0f,
                                        pg, sf));
            RCHECK(linear(m, sf, m->act, lc.ff, L.w_down, D, L.b_down, L.b_down_act, m->yf, T, ZL_F32, ZL_GEMM_EPI_NONE));
            f_dense = m->yf;
        } else if (lc.ff_kind == ZL_FF_MOE) {
            const int E = lc.experts, F = lc.ff;
            if (lc.shared_ff > 0) {
                RCHECK(linear(m, sf, m->h, D, L.s_up, lc.shared_ff, nullptr, nullptr, m->act_s, T, dt, ZL_GEMM_EPI_RELU2));
                RCHECK(linear(m, sf, m->act_s, lc.shared_ff, L.s_down, D, nullptr, nullptr, m->yf, T, ZL_F32, ZL_GEMM_EPI_NONE));
                f_dense = m->yf;
            }
            if (fork) ZL_CHECK_CUDA(cudaStreamWaitEvent(sf, m->ev_proj[l], 0));
            RCHECK(zl_moe_route_grouped(m->proj + L.r_off, L.n_in, nullptr, L.correction, m->top_e, m->top_w, m->grp_off,
                                        m->list_token, m->list_pair, T, D, E + lc.identity, lc.top, lc.groups, lc.keep,
                                        ZL_MOE_SCORE_SOFTMAX, 1, 1e-20f, pr, sf));
            if (E > 0) {
                RCHECK(zl_gemm_nt_grouped(m->h, D, m->list_token, L.w_up, D, (long long)F * D, m->act, F, nullptr, m->grp_off, E,
                                          T, F, D, dt, dt, ZL_GEMM_EPI_RELU2, 0.f, 1.f, 0.f, pg, sf));
                RCHECK(zl_gemm_nt_grouped(m->act, F, nullptr, L.w_down, F, (long long)D * F, m->ypair, D, m->list_pair,
                                          m->grp_off, E, T, D, F, dt, ZL_F32, ZL_GEMM_EPI_NONE, 0.f, 1.f, 0.f, pg, sf));
            }
            parts = m->ypair;
        }
        if (fork) {
            ZL_CHECK_CUDA(cudaEventRecord(m->ev_ff[l], sf));
            ZL_CHECK_CUDA(cudaStreamWaitEvent(st, m->ev_ff[l], 0));
        }
        const float* next_w = l + 1 < c.num_layers ? m->layers[l + 1].norm1 : nullptr;
        RCHECK(zl_gated_parallel_combine(m->x, D, c.residual_mult, m->proj, L.n_in, m->ya, D, L.g1_off, L.ls1, parts, D, m->top_w,
                                         m->top_e, lc.top, lc.experts, f_dense, D, L.g2_off, L.ls2, L.norm1, next_w, m->h, dt, T,
                                         D, c.eps, pr, st));
        if (m->capture && m->layer_dump)
            ZL_CHECK_CUDA(cudaMemcpyAsync(m->layer_dump + (size_t)l * m->tcap * D, m->x, (size_t)T * D * 4,
                                          cudaMemcpyDeviceToDevice, st));
    }
    if (n_want > 0) {
        ZL_CHECK_CUDA(launch(k_gather_rows_f32, dim3(n_want), dim3(128), 0, st, false, (const float*)m->x,
                             (const int32_t*)m->d_want, m->xw, D));
        RCHECK(zl_group_rmsnorm(m->xw, D, m->final_norm, m->xn, D, n_want, D, 1, c.eps, dt, pt, st));
        RCHECK(linear(m, st, m->xn, D, m->head, c.vocab, nullptr, nullptr, m->logits, n_want, ZL_F32, ZL_GEMM_EPI_NONE));
        RCHECK(zl_argmax(m->logits, m->d_next, n_want, c.vocab, m->argmax_ws, zl_argmax_workspace_bytes(n_want), pt, st));
    }
    return ZL_OK;
}

// decode-sized steps replay a CUDA graph per (rows, wanted rows, runs, length bucket); prompt portions are enqueued directly
// (max_run: the longest run; a captured step is sized for the longest run its row count allows)
int run_step(zl_dizizen* m, int T, int n_want, int n_runs, int max_run, int max_len) {
    const int bucket = len_bucket(m, max_len);
    if (!m->cfg.use_graph || T > m->cfg.max_batch || m->capture) return enqueue_step(m, T, n_want, n_runs, max_run, bucket);
    const long long key = ((long long)T << 48) | ((long long)n_want << 32) | ((long long)n_runs << 16) | (long long)(bucket >> 8);
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        cudaGraph_t graph = nullptr;
        ZL_CHECK_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_step(m, T, n_want, n_runs, T - n_runs + 1, bucket);
        const cudaError_t ce = cudaStreamEndCapture(m->stream, &graph);
        if (rc != ZL_OK) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        ZL_CHECK_CUDA(ce);
        cudaGraphExec_t exec = nullptr;
        ZL_CHECK_CUDA(cudaGraphInstantiate(&exec, graph, 0));
        size_t n_nodes = 0;
        cudaGraphGetNodes(graph, nullptr, &n_nodes);
        m->kernels_per_step = (int)n_nodes;
        cudaGraphDestroy(graph);
        it = m->graphs.emplace(key, exec).first;
    }
    ZL_CHECK_CUDA(cudaGraphLaunch(it->second, m->stream));
    return ZL_OK;
}

}  // namespace

extern "C" int zl_dizizen_create(const zl_dizizen_config_t* cfg, const zl_dizizen_layer_t* layers, zl_dizizen_t** out) {
    ZL_CHECK_ARG(cfg && layers && out);
    ZL_CHECK_ARG(cfg->num_layers > 0 && cfg->width > 0 && cfg->vocab > 0 && cfg->max_batch > 0 && cfg->max_seq > 0);
    ZL_CHECK_ARG(cfg->eps >= 0.f);
    ZL_CHECK_SUPPORTED(cfg->dtype == ZL_BF16 || cfg->dtype == ZL_F32);
    ZL_CHECK_ARG(cfg->max_step_tokens >= 0 && cfg->max_step_tokens <= 65535);
    for (int l = 0; l < cfg->num_layers; ++l) {
        const auto& lc = layers[l];
        ZL_CHECK_ARG(lc.heads > 0 && lc.dim > 0 && lc.kv_heads > 0 && lc.heads % lc.kv_heads == 0 && lc.vdim > 0 && lc.vdim % 2 == 0);
        ZL_CHECK_ARG(lc.rot_dims >= 0 && lc.rot_dims <= lc.dim && lc.rot_dims % 2 == 0 && lc.rot_base > 1.f);
        if (lc.kv_from >= 0) {
            // the source layer runs earlier in the step, owns its caches, and has the same key / value shape
            const auto& sc = layers[lc.kv_from < l ? lc.kv_from : 0];
            ZL_CHECK_ARG(lc.kv_from < l && sc.kv_from < 0 && sc.kv_heads == lc.kv_heads && sc.dim == lc.dim && sc.vdim == lc.vdim);
        }
        ZL_CHECK_ARG(lc.ff_kind == ZL_FF_NONE || lc.ff_kind == ZL_FF_DENSE || lc.ff_kind == ZL_FF_MOE);
        if (lc.ff_kind == ZL_FF_DENSE) ZL_CHECK_ARG(lc.ff > 0 && lc.limit > 0.f);
        if (lc.ff_kind == ZL_FF_MOE) {
            const int slots = lc.experts + lc.identity;
            ZL_CHECK_ARG(lc.experts >= 0 && lc.identity >= 0 && slots > 0 && lc.top > 0 && lc.top <= slots && lc.shared_ff >= 0);
            ZL_CHECK_ARG(lc.experts == 0 || lc.ff > 0);
            ZL_CHECK_ARG(lc.groups >= 1 && slots % lc.groups == 0 && lc.keep >= 1 && lc.keep <= lc.groups &&
                         lc.keep * (slots / lc.groups) >= lc.top);
        }
    }
    zl_dizizen* m = new zl_dizizen();
    m->cfg = *cfg;
    m->esz = cfg->dtype == ZL_F32 ? 4 : 2;
    m->tcap = cfg->max_step_tokens > cfg->max_batch ? cfg->max_step_tokens : cfg->max_batch;
    m->layers.resize(cfg->num_layers);
    for (int l = 0; l < cfg->num_layers; ++l) m->layers[l].c = layers[l];
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete m;
        zl_set_last_error(__FILE__, __LINE__, "cudaStreamCreate failed (no CUDA device? there is no CPU fallback)");
        return ZL_ERR_CUDA;
    }
    bool ok = cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking) == cudaSuccess;
    for (auto* evs : {&m->ev_h, &m->ev_proj, &m->ev_ff}) {
        evs->assign(cfg->num_layers, nullptr);
        for (auto& e : *evs) ok = ok && cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) {
        zl_dizizen_destroy(m);
        zl_set_last_error(__FILE__, __LINE__, "creating the side stream or its events failed");
        return ZL_ERR_CUDA;
    }
    *out = m;
    return ZL_OK;
}

extern "C" void zl_dizizen_destroy(zl_dizizen_t* m) {
    if (!m) return;
    cudaStreamSynchronize(m->stream);
    if (m->side) cudaStreamSynchronize(m->side);
    for (auto* evs : {&m->ev_h, &m->ev_proj, &m->ev_ff})
        for (auto e : *evs)
            if (e) cudaEventDestroy(e);
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
    for (auto& s : m->staged) cudaFree(s.second.ptr);
    for (auto& L : m->layers) {
        for (void* p : {(void*)L.norm1, (void*)L.ls1, (void*)L.ls2, L.w_in, (void*)L.b_in, L.b_in_act, L.o, (void*)L.o_b, L.o_b_act,
                        L.w_gu, (void*)L.b_gu, L.w_down, (void*)L.b_down, L.b_down_act, (void*)L.correction, L.w_up, L.s_up,
                        L.s_down})
            if (p) cudaFree(p);
        L.kcache.destroy();
        L.vcache.destroy();
    }
    for (auto& r : m->rots)
        for (void* p : {(void*)r.inv_freq, (void*)r.table})
            if (p) cudaFree(p);
    for (void* p : {m->embed, m->head, (void*)m->final_norm, (void*)m->x, (void*)m->proj, (void*)m->ya, (void*)m->yf,
                    (void*)m->ypair, (void*)m->xw, (void*)m->logits, (void*)m->top_w, m->h, m->q, m->att, m->act, m->act_s,
                    m->xn, (void*)m->d_tokens, (void*)m->d_slots, (void*)m->d_pos, (void*)m->d_want, (void*)m->d_next,
                    (void*)m->d_run0, (void*)m->d_runlen, (void*)m->top_e, (void*)m->grp_off, (void*)m->list_token,
                    (void*)m->list_pair, m->attn_ws, m->argmax_ws, (void*)m->layer_dump})
        if (p) cudaFree(p);
    if (m->h_stage) cudaFreeHost(m->h_stage);
    if (m->side) cudaStreamDestroy(m->side);
    cudaStreamDestroy(m->stream);
    delete m;
}

extern "C" int zl_dizizen_load_tensor(zl_dizizen_t* m, const char* name, const void* data_host, int rows, int cols,
                                      int elem_bytes) {
    ZL_CHECK_ARG(m && name && data_host && rows > 0 && cols > 0 && (elem_bytes == 2 || elem_bytes == 4));
    if (m->finalized) return fail(__LINE__, "model already finalized");
    return staged_load(m->staged, name, data_host, rows, cols, elem_bytes, m->stream);
}

extern "C" int zl_dizizen_finalize(zl_dizizen_t* m) {
    ZL_CHECK_ARG(m);
    if (m->finalized) return ZL_OK;
    for (int l = 0; l < m->cfg.num_layers; ++l)
        if (!m->layers[l].ready) RCHECK(finalize_layer(m, l));
    RCHECK(take_weight(m, "embed", m->cfg.vocab, m->cfg.width, &m->embed));
    m->weight_bytes -= (double)m->cfg.vocab * m->cfg.width * m->esz;   // gathered, not streamed
    RCHECK(take_weight(m, "head", m->cfg.vocab, m->cfg.width, &m->head));
    RCHECK(take_norm_plus_one(m, "final.norm", m->cfg.width, &m->final_norm));
    RCHECK(alloc_runtime(m));
    m->finalized = true;
    return ZL_OK;
}

extern "C" int zl_dizizen_init_synthetic(zl_dizizen_t* m, uint64_t seed) {
    ZL_CHECK_ARG(m);
    if (m->finalized) return fail(__LINE__, "model already finalized");
    const auto& c = m->cfg;
    const int D = c.width;
    auto lin = [&](const std::string& name, int n, int k) {
        const float a = sqrtf(3.0f / (float)k);   // unit-variance outputs for unit-variance inputs
        return stage_random(m, name, n, k, -a, a, seed);
    };
    auto small = [&](const std::string& name, int n, float a) { return stage_random(m, name, 1, n, -a, a, seed); };
    for (int l = 0; l < c.num_layers; ++l) {
        const auto& lc = m->layers[l].c;
        const std::string p = "l" + std::to_string(l) + ".", mx = p + "mix.", ml = p + "mlp.";
        const int H = lc.heads;
        RCHECK(small(p + "norm1", D, 0.1f));
        RCHECK(lin(mx + "q", H * lc.dim, D));
        RCHECK(small(mx + "q.b", H * lc.dim, 0.1f));
        if (lc.kv_from < 0) {
            RCHECK(lin(mx + "k", lc.kv_heads * lc.dim, D));
            RCHECK(small(mx + "k.b", lc.kv_heads * lc.dim, 0.1f));
            RCHECK(lin(mx + "v", lc.kv_heads * lc.vdim, D));
            RCHECK(small(mx + "v.b", lc.kv_heads * lc.vdim, 0.1f));
        }
        RCHECK(lin(mx + "o", D, H * lc.vdim));
        RCHECK(small(mx + "o.b", D, 0.1f));
        RCHECK(lin(p + "rg1", D, D));
        RCHECK(small(p + "rg1.b", D, 0.1f));
        RCHECK(stage_random(m, p + "ls1", 1, D, 0.5f, 1.0f, seed));
        if (lc.ff_kind != ZL_FF_NONE) {
            RCHECK(lin(p + "rg2", D, D));
            RCHECK(small(p + "rg2.b", D, 0.1f));
            RCHECK(stage_random(m, p + "ls2", 1, D, 0.5f, 1.0f, seed));
        }
        if (lc.ff_kind == ZL_FF_DENSE) {
            RCHECK(lin(ml + "gate", lc.ff, D));
            RCHECK(small(ml + "gate.b", lc.ff, 0.1f));
            RCHECK(lin(ml + "up", lc.ff, D));
            RCHECK(small(ml + "up.b", lc.ff, 0.1f));
            RCHECK(lin(ml + "down", D, lc.ff));
            RCHECK(small(ml + "down.b", D, 0.1f));
        } else if (lc.ff_kind == ZL_FF_MOE) {
            RCHECK(lin(ml + "router", lc.experts + lc.identity, D));
            RCHECK(small(ml + "correction", lc.experts + lc.identity, 0.02f));
            for (int e = 0; e < lc.experts; ++e) {
                const std::string pe = ml + "e" + std::to_string(e) + ".";
                RCHECK(lin(pe + "up", lc.ff, D));
                RCHECK(lin(pe + "down", D, lc.ff));
            }
            if (lc.shared_ff > 0) {
                RCHECK(lin(ml + "shared.up", lc.shared_ff, D));
                RCHECK(lin(ml + "shared.down", D, lc.shared_ff));
            }
        }
        RCHECK(finalize_layer(m, l));   // bound the staging memory to one layer
    }
    RCHECK(stage_random(m, "embed", c.vocab, D, -1.7f, 1.7f, seed));
    RCHECK(lin("head", c.vocab, D));
    RCHECK(small("final.norm", D, 0.1f));
    return zl_dizizen_finalize(m);
}

extern "C" int zl_dizizen_step(zl_dizizen_t* m, const int32_t* tokens_host, const int32_t* slots_host,
                               const int32_t* positions_host, int T, const int32_t* want_rows_host, int n_want,
                               float* logits_host, int32_t* next_host) {
    ZL_CHECK_ARG(m && tokens_host && slots_host && positions_host && T > 0 && n_want >= 0);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    ZL_CHECK_ARG(T <= m->tcap && n_want <= T && (n_want == 0 || want_rows_host));
    const auto& c = m->cfg;
    int32_t* hs = m->h_stage;
    int max_len = 0, n_runs = 0, max_run = 1;
    for (int i = 0; i < T; ++i) {
        ZL_CHECK_ARG(tokens_host[i] >= 0 && tokens_host[i] < c.vocab);
        ZL_CHECK_ARG(slots_host[i] >= 0 && slots_host[i] < c.max_batch);
        ZL_CHECK_ARG(positions_host[i] >= 0 && positions_host[i] < c.max_seq);
        // rows of one slot are consecutive and at consecutive positions; a slot appears in one run only
        if (i > 0 && slots_host[i] == slots_host[i - 1]) {
            ZL_CHECK_ARG(positions_host[i] == positions_host[i - 1] + 1);
            hs[6 * T + n_runs - 1] += 1;
            if (hs[6 * T + n_runs - 1] > max_run) max_run = hs[6 * T + n_runs - 1];
        } else {
            hs[5 * T + n_runs] = i;
            hs[6 * T + n_runs] = 1;
            ++n_runs;
        }
        hs[i] = tokens_host[i];
        hs[T + i] = slots_host[i];
        hs[2 * T + i] = positions_host[i];
        if (positions_host[i] + 1 > max_len) max_len = positions_host[i] + 1;
    }
    for (int i = 0; i < n_want; ++i) {
        ZL_CHECK_ARG(want_rows_host[i] >= 0 && want_rows_host[i] < T);
        hs[3 * T + i] = want_rows_host[i];
    }
    cudaStream_t st = m->stream;
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_tokens, hs, (size_t)T * 4, cudaMemcpyHostToDevice, st));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_slots, hs + T, (size_t)T * 4, cudaMemcpyHostToDevice, st));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_pos, hs + 2 * T, (size_t)T * 4, cudaMemcpyHostToDevice, st));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_run0, hs + 5 * T, (size_t)n_runs * 4, cudaMemcpyHostToDevice, st));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_runlen, hs + 6 * T, (size_t)n_runs * 4, cudaMemcpyHostToDevice, st));
    if (n_want) ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_want, hs + 3 * T, (size_t)n_want * 4, cudaMemcpyHostToDevice, st));
    RCHECK(run_step(m, T, n_want, n_runs, max_run, max_len));
    if (n_want && next_host) ZL_CHECK_CUDA(cudaMemcpyAsync(hs + 4 * T, m->d_next, (size_t)n_want * 4, cudaMemcpyDeviceToHost, st));
    if (n_want && logits_host)
        ZL_CHECK_CUDA(cudaMemcpyAsync(logits_host, m->logits, (size_t)n_want * c.vocab * 4, cudaMemcpyDeviceToHost, st));
    ZL_CHECK_CUDA(cudaStreamSynchronize(st));
    if (n_want && next_host)
        for (int i = 0; i < n_want; ++i) next_host[i] = hs[4 * T + i];
    if (max_len > m->cur_max_len) m->cur_max_len = max_len;
    return ZL_OK;
}

extern "C" int zl_dizizen_set_state(zl_dizizen_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B) {
    ZL_CHECK_ARG(m && tokens_host && positions_host && B > 0 && B <= m->cfg.max_batch);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));   // the staging buffer is free again
    int32_t* hs = m->h_stage;
    const int T = m->tcap;
    int mx = 0;
    for (int i = 0; i < B; ++i) {
        ZL_CHECK_ARG(tokens_host[i] >= 0 && tokens_host[i] < m->cfg.vocab);
        ZL_CHECK_ARG(positions_host[i] >= 0 && positions_host[i] < m->cfg.max_seq);
        hs[i] = tokens_host[i];
        hs[T + i] = positions_host[i];
        hs[2 * T + i] = 1;
        if (positions_host[i] + 1 > mx) mx = positions_host[i] + 1;
    }
    m->cur_max_len = mx;
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_tokens, hs, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_pos, hs + T, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    ZL_CHECK_CUDA(cudaMemcpyAsync(m->d_runlen, hs + 2 * T, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    k_iota_i32<<<cdiv(B, 256), 256, 0, m->stream>>>(m->d_slots, m->d_want, B);
    k_iota_i32<<<cdiv(B, 256), 256, 0, m->stream>>>(m->d_run0, m->d_want, B);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" int zl_dizizen_step_device(zl_dizizen_t* m, int B) {
    ZL_CHECK_ARG(m && B > 0 && B <= m->cfg.max_batch);
    if (m->cur_max_len >= m->cfg.max_seq) return fail(__LINE__, "caches full (max_seq reached)");
    RCHECK(run_step(m, B, B, B, 1, m->cur_max_len));
    k_decode_advance<<<cdiv(B, 64), 64, 0, m->stream>>>(m->d_tokens, m->d_pos, m->d_next, B);
    ZL_CHECK_LAUNCH();
    m->cur_max_len += 1;
    return ZL_OK;
}

extern "C" int zl_dizizen_sync(zl_dizizen_t* m) {
    ZL_CHECK_ARG(m);
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" zl_stream_t zl_dizizen_stream(zl_dizizen_t* m) { return m ? (zl_stream_t)m->stream : nullptr; }

extern "C" int zl_dizizen_capture_layers(zl_dizizen_t* m, int on) {
    ZL_CHECK_ARG(m);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    if (on && !m->layer_dump)
        RCHECK(dmalloc((void**)&m->layer_dump, (size_t)m->cfg.num_layers * m->tcap * m->cfg.width * 4));
    m->capture = on != 0;
    return ZL_OK;
}

extern "C" int zl_dizizen_read_layers(zl_dizizen_t* m, float* out_host, int T) {
    ZL_CHECK_ARG(m && out_host && T > 0 && T <= m->tcap);
    if (!m->layer_dump) return fail(__LINE__, "layer capture was not switched on");
    const size_t row = (size_t)m->cfg.width * 4;
    ZL_CHECK_CUDA(cudaMemcpy2DAsync(out_host, (size_t)T * row, m->layer_dump, (size_t)m->tcap * row, (size_t)T * row,
                                    m->cfg.num_layers, cudaMemcpyDeviceToHost, m->stream));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" int zl_dizizen_read_cache(zl_dizizen_t* m, int layer, int slot, int n_rows, float* keys_host, float* values_host) {
    ZL_CHECK_ARG(m && keys_host && values_host && layer >= 0 && layer < m->cfg.num_layers && slot >= 0 && slot < m->cfg.max_batch);
    ZL_CHECK_ARG(n_rows > 0 && n_rows <= m->cfg.max_seq);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    const DLayer& L = m->layers[layer];
    ZL_CHECK_ARG(L.c.kv_from < 0);
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    const SlotCache* cs[2] = {&L.kcache, &L.vcache};
    float* outs[2] = {keys_host, values_host};
    const size_t ns[2] = {(size_t)n_rows * L.c.kv_heads * L.c.dim, (size_t)n_rows * L.c.kv_heads * L.c.vdim};
    for (int i = 0; i < 2; ++i) {
        const char* src = (const char*)cs[i]->buf + (size_t)slot * cs[i]->slot_bytes;
        if (m->cfg.dtype == ZL_F32) {
            ZL_CHECK_CUDA(cudaMemcpy(outs[i], src, ns[i] * 4, cudaMemcpyDeviceToHost));
        } else {
            std::vector<uint16_t> tmp(ns[i]);
            ZL_CHECK_CUDA(cudaMemcpy(tmp.data(), src, ns[i] * 2, cudaMemcpyDeviceToHost));
            for (size_t j = 0; j < ns[i]; ++j) {
                const uint32_t u = (uint32_t)tmp[j] << 16;
                memcpy(outs[i] + j, &u, 4);
            }
        }
    }
    return ZL_OK;
}

extern "C" int zl_dizizen_stats(zl_dizizen_t* m, double* weight_bytes, int* kernels_per_step) {
    ZL_CHECK_ARG(m);
    if (weight_bytes) *weight_bytes = m->weight_bytes;
    if (kernels_per_step) *kernels_per_step = m->kernels_per_step;
    return ZL_OK;
}

// Host-side driver of the Lagelorn model family: weights, slot caches and recurrent states, the per-step kernel chain and
// its CUDA graph.  Same driver shape as kodupel_runner.cu (task slots, host (token, slot, position) rows in, logits /
// greedy picks out), built from the shared pieces of runner_common.cuh.
//
// x = embed[token] + pos[position] in fp32.  A layer is norm after the sum: x <- norm1(alpha x + mixer(x)),
// x <- norm2(alpha x + ff(x)) (RMS norms with plain weights; a layer may have no feed-forward), then the layer's slice e
// of a second token embedding enters: y = W_proj (gelu_tanh(W_gate x) * e), x <- x + norm(y).  The sublayers read x itself
// (rounded to the activation dtype for the Linears).
//   delta layer:     one fused projection [W_q; W_k; W_v; W_b; W_a; W_g] -> short convolutions, silu, unit q / k, rate and
//                    decay, the gated delta rule over the slot's state (delta_rule.cu) -> per-head RMS norm, weight,
//                    silu gate (mixer_rows.cu) -> W_o.
//   parallel layer:  left_scale * A(x) + right_scale * R(x).
//     A: one projection [W_q; W_k] with biases -> norms over the whole projection, append of the normed keys (keys) and the
//        projected keys (values) to the slot's caches (mixer_rows.cu) -> attention inside blocks of positions with a
//        distance bias and a sink (sink_attn.cu) -> W_o.
//     R: five mixes of the token with its predecessor (mixer_rows.cu) -> a batch of four projections r, k, v, g and the
//        decay path W_w2 tanh(W_w1 .) + w0 -> the decaying state with a bonus for the current token (delta_rule.cu) ->
//        per-head RMS norm, weight, silu gate -> W_o.
//   feed-forward:    [W_gate; W_up] with rows interleaved and gelu_tanh(gate) * up as the epilogue, then W_down.
// One step takes T rows in any mix of prompt portions and single decode tokens; every kernel indexes caches and states
// by (slot, position), and the recurrences walk each run of rows (one slot, consecutive positions) in order.
#include "runner_common.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace {

using namespace zl;

struct GLayer {
    zl_lagelorn_layer_t c{};
    float *norm1 = nullptr, *norm2 = nullptr;
    // delta: fused projection q | k | v | b | a | g; parallel: the attention's q | k
    void* w_in = nullptr;
    float* b_in = nullptr;
    void* b_in_act = nullptr;
    int n_in = 0, q_off = 0, k_off = 0, v_off = 0, b_off = 0, a_off = 0, g_off = 0;
    void* o = nullptr;                           // delta (width, heads * vdim); parallel: attention (width, l_heads * l_dim)
    // delta
    float *conv_w = nullptr, *a_log = nullptr, *dt_bias = nullptr, *out_norm = nullptr;
    SlotCache state, ring;                       // (heads, dim, vdim) fp32; (conv - 1, channels) fp32
    // parallel, attention
    float *q_norm = nullptr, *k_norm = nullptr, *dist_bias = nullptr, *sink = nullptr;
    int n_dist = 0;
    SlotCache kcache, vcache;
    // parallel, decaying state
    float* mu = nullptr;                         // (5, width): r, k, v, g, w
    void* w_rkvg = nullptr;                      // (4, r_heads * r_dim, width)
    void *w1 = nullptr, *w2 = nullptr, *r_o = nullptr;
    float *w0 = nullptr, *bonus = nullptr, *r_norm = nullptr;
    void* w0_act = nullptr;
    SlotCache r_state, shift;                    // (r_heads, r_dim, r_dim) fp32; (width) fp32: the slot's last token
    // feed-forward
    void *w_gu = nullptr, *w_down = nullptr;     // (2 ff, width): rows 2j / 2j+1 = gate_j / up_j; (width, ff)
    float *b_gu = nullptr, *b_down = nullptr;
    void* b_down_act = nullptr;
    // token side input
    void *s_gate = nullptr, *s_proj = nullptr;
    float* s_norm = nullptr;
    bool ready = false;
};

}  // namespace

struct zl_lagelorn {
    zl_lagelorn_config_t cfg{};
    cudaStream_t stream = nullptr;
    StagedMap staged;
    std::vector<GLayer> layers;
    void *embed = nullptr, *pos_table = nullptr, *side_embed = nullptr, *head = nullptr;
    float* final_norm = nullptr;
    bool finalized = false;
    int esz = 2;
    int tcap = 0;
    float *x = nullptr, *proj = nullptr, *rkvg = nullptr, *dlog = nullptr, *orec = nullptr, *y = nullptr, *y2 = nullptr,
          *side = nullptr, *xw = nullptr, *logits = nullptr;
    void *xa = nullptr, *mix = nullptr, *q = nullptr, *att = nullptr, *z1 = nullptr, *act = nullptr, *sg = nullptr, *xn = nullptr;
    int32_t *d_tokens = nullptr, *d_slots = nullptr, *d_pos = nullptr, *d_want = nullptr, *d_next = nullptr;
    int32_t *d_run0 = nullptr, *d_runlen = nullptr;
    int32_t* h_stage = nullptr;   // pinned: tokens | slots | pos | want | next | run0 | runlen
    void* attn_ws = nullptr;
    size_t attn_ws_bytes = 0;
    void* delta_ws = nullptr;
    size_t delta_ws_bytes = 0;
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

// x[t] = embed[token[t]] + pos_table[pos[t]] in fp32, the same rounded to the activation dtype, and the token's row of the
// second embedding (all layers' slices) in fp32
template <typename TW>
__global__ void k_embed_pos_side(const int32_t* __restrict__ ids, const int32_t* __restrict__ pos, const TW* __restrict__ table,
                                 const TW* __restrict__ pos_table, const TW* __restrict__ side_table, float* __restrict__ x,
                                 TW* __restrict__ xa, float* __restrict__ side, int D, int S, int vocab, int max_pos) {
    pdl_trigger();
    pdl_wait();
    int id = ids[blockIdx.x], p = pos[blockIdx.x];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    if (blockIdx.y == 1) {   // grid (T, 2): the second CTA of a token gathers the side row
        for (int i = threadIdx.x; i < S; i += blockDim.x) side[(size_t)blockIdx.x * S + i] = to_f32<TW>(side_table[(size_t)id * S + i]);
        return;
    }
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = to_f32<TW>(table[(size_t)id * D + i]) + to_f32<TW>(pos_table[(size_t)p * D + i]);
        x[(size_t)blockIdx.x * D + i] = v;
        if (xa) xa[(size_t)blockIdx.x * D + i] = from_f32<TW>(v);
    }
}

// dst rows 2j / 2j+1 <- gate / up row j; src are (ff, D) each
template <typename TS, typename TD>
__global__ void k_interleave_rows2(const TS* __restrict__ gate, const TS* __restrict__ up, TD* __restrict__ dst, int ff, int D) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)ff * D) return;
    const size_t j = i / D, c = i % D;
    dst[(2 * j) * D + c] = from_f32<TD>(to_f32<TS>(gate[i]));
    dst[(2 * j + 1) * D + c] = from_f32<TD>(to_f32<TS>(up[i]));
}

// segment `name` (n values) -> fp32 array at offset off
int put_f32(zl_lagelorn* m, const std::string& name, int n, float* dst, size_t off) {
    const Staged* s = need(m, name, 1, n);
    if (!s) return ZL_ERR_STATE;
    RCHECK(convert_to<float>(m, s, dst + off, (size_t)n));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, name);
    return ZL_OK;
}
// (rows, cols) matrix -> fp32 array at offset off
int put_f32_2d(zl_lagelorn* m, const std::string& name, int rows, int cols, float* dst, size_t off) {
    const Staged* s = need(m, name, rows, cols);
    if (!s) return ZL_ERR_STATE;
    RCHECK(convert_to<float>(m, s, dst + off, (size_t)rows * cols));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, name);
    return ZL_OK;
}

// fp32 bias -> a copy in the activation dtype (bf16 mode; the checkpoint's biases are bfloat16, so nothing is lost)
int bias_act_copy(zl_lagelorn* m, const float* src, int n, void** out) {
    if (m->cfg.dtype == ZL_F32) return ZL_OK;
    RCHECK(dmalloc(out, (size_t)n * 2));
    k_convert<float, __nv_bfloat16><<<cdiv(n, 256), 256, 0, m->stream>>>(src, static_cast<__nv_bfloat16*>(*out), (size_t)n);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

int finalize_ff(zl_lagelorn* m, int l) {
    GLayer& L = m->layers[l];
    const int D = m->cfg.width, F = L.c.ff;
    const std::string p = "l" + std::to_string(l) + ".mlp.";
    const Staged* g = need(m, p + "gate", F, D);
    const Staged* u = need(m, p + "up", F, D);
    if (!g || !u) return ZL_ERR_STATE;
    if (g->elem != u->elem) return fail(__LINE__, "gate and up of a feed-forward differ in dtype");
    RCHECK(dmalloc(&L.w_gu, (size_t)2 * F * D * m->esz));
    const size_t n = (size_t)F * D;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (m->cfg.dtype == ZL_F32) {
        if (g->elem == 2)
            k_interleave_rows2<<<blocks, 256, 0, m->stream>>>((const __nv_bfloat16*)g->ptr, (const __nv_bfloat16*)u->ptr, (float*)L.w_gu, F, D);
        else
            k_interleave_rows2<<<blocks, 256, 0, m->stream>>>((const float*)g->ptr, (const float*)u->ptr, (float*)L.w_gu, F, D);
    } else {
        if (g->elem == 2)
            k_interleave_rows2<<<blocks, 256, 0, m->stream>>>((const __nv_bfloat16*)g->ptr, (const __nv_bfloat16*)u->ptr,
                                                              (__nv_bfloat16*)L.w_gu, F, D);
        else
            k_interleave_rows2<<<blocks, 256, 0, m->stream>>>((const float*)g->ptr, (const float*)u->ptr, (__nv_bfloat16*)L.w_gu, F, D);
    }
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, p + "gate");
    staged_drop(m->staged, p + "up");
    m->weight_bytes += 2.0 * n * m->esz;
    // the two biases interleaved like the rows
    const Staged* gb = need(m, p + "gate.b", 1, F);
    const Staged* ub = need(m, p + "up.b", 1, F);
    if (!gb || !ub) return ZL_ERR_STATE;
    if (gb->elem != ub->elem) return fail(__LINE__, "gate and up biases differ in dtype");
    RCHECK(dmalloc((void**)&L.b_gu, (size_t)2 * F * 4));
    if (gb->elem == 2)
        k_interleave_rows2<<<cdiv(F, 256), 256, 0, m->stream>>>((const __nv_bfloat16*)gb->ptr, (const __nv_bfloat16*)ub->ptr, L.b_gu, F, 1);
    else
        k_interleave_rows2<<<cdiv(F, 256), 256, 0, m->stream>>>((const float*)gb->ptr, (const float*)ub->ptr, L.b_gu, F, 1);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, p + "gate.b");
    staged_drop(m->staged, p + "up.b");
    RCHECK(take_weight(m, p + "down", D, F, &L.w_down));
    RCHECK(take_f32(m, p + "down.b", 1, D, &L.b_down));
    RCHECK(bias_act_copy(m, L.b_down, D, &L.b_down_act));
    return ZL_OK;
}

int finalize_layer(zl_lagelorn* m, int l) {
    const auto& c = m->cfg;
    GLayer& L = m->layers[l];
    const auto& lc = L.c;
    const std::string p = "l" + std::to_string(l) + ".", mx = p + "mix.";
    const int D = c.width;
    RCHECK(take_f32(m, p + "norm1", 1, D, &L.norm1));
    if (lc.type == ZL_LAYER_DELTA) {
        const int H = lc.heads, G = lc.kv_heads, d = lc.dim, vd = lc.vdim;
        L.q_off = 0;
        L.k_off = G * d;
        L.v_off = 2 * G * d;
        L.b_off = L.v_off + H * vd;
        L.a_off = L.b_off + H;
        L.g_off = L.a_off + H;
        L.n_in = L.g_off + H * vd;
        const int C = L.b_off;   // channels that pass the convolution
        RCHECK(dmalloc(&L.w_in, (size_t)L.n_in * D * m->esz));
        RCHECK(put_weight(m, mx + "q", G * d, D, L.w_in, 0));
        RCHECK(put_weight(m, mx + "k", G * d, D, L.w_in, (size_t)L.k_off * D));
        RCHECK(put_weight(m, mx + "v", H * vd, D, L.w_in, (size_t)L.v_off * D));
        RCHECK(put_weight(m, mx + "b", H, D, L.w_in, (size_t)L.b_off * D));
        RCHECK(put_weight(m, mx + "a", H, D, L.w_in, (size_t)L.a_off * D));
        RCHECK(put_weight(m, mx + "g", H * vd, D, L.w_in, (size_t)L.g_off * D));
        RCHECK(dmalloc((void**)&L.conv_w, (size_t)C * lc.conv * 4));
        RCHECK(put_f32_2d(m, mx + "q.conv", G * d, lc.conv, L.conv_w, 0));
        RCHECK(put_f32_2d(m, mx + "k.conv", G * d, lc.conv, L.conv_w, (size_t)L.k_off * lc.conv));
        RCHECK(put_f32_2d(m, mx + "v.conv", H * vd, lc.conv, L.conv_w, (size_t)L.v_off * lc.conv));
        RCHECK(take_f32(m, mx + "A_log", 1, H, &L.a_log));
        RCHECK(take_f32(m, mx + "dt_bias", 1, H, &L.dt_bias));
        RCHECK(take_f32(m, mx + "norm", 1, vd, &L.out_norm));
        RCHECK(take_weight(m, mx + "o", D, H * vd, &L.o));
    } else {
        const std::string lf = mx + "left.", rt = mx + "right.";
        const int H = lc.l_heads, G = lc.l_kv_heads, d = lc.l_dim;
        L.q_off = 0;
        L.k_off = H * d;
        L.n_in = (H + G) * d;
        RCHECK(dmalloc(&L.w_in, (size_t)L.n_in * D * m->esz));
        RCHECK(dmalloc((void**)&L.b_in, (size_t)L.n_in * 4));
        RCHECK(put_weight(m, lf + "q", H * d, D, L.w_in, 0));
        RCHECK(put_weight(m, lf + "k", G * d, D, L.w_in, (size_t)L.k_off * D));
        RCHECK(put_f32(m, lf + "q.b", H * d, L.b_in, 0));
        RCHECK(put_f32(m, lf + "k.b", G * d, L.b_in, L.k_off));
        RCHECK(bias_act_copy(m, L.b_in, L.n_in, &L.b_in_act));
        RCHECK(take_f32(m, lf + "q.norm", 1, H * d, &L.q_norm));
        RCHECK(take_f32(m, lf + "k.norm", 1, G * d, &L.k_norm));
        RCHECK(take_f32(m, lf + "sink", 1, H, &L.sink));
        RCHECK(take_weight(m, lf + "o", D, H * d, &L.o));
        {   // the distance table, one entry per distance a token can see
            float* rel = nullptr;
            RCHECK(take_f32(m, lf + "rel", lc.l_rel_rows, H, &rel));
            std::vector<float> host((size_t)lc.l_rel_rows * H);
            ZL_CHECK_CUDA(cudaMemcpy(host.data(), rel, host.size() * 4, cudaMemcpyDeviceToHost));
            cudaFree(rel);
            L.n_dist = lc.l_chunk > 0 ? std::min(lc.l_chunk, c.max_seq) : c.max_seq;
            std::vector<float> table((size_t)H * L.n_dist);
            RCHECK(zl_distance_bias_table(host.data(), lc.l_rel_rows, H, (double)lc.l_bias_max, L.n_dist, table.data()));
            RCHECK(dmalloc((void**)&L.dist_bias, table.size() * 4));
            ZL_CHECK_CUDA(cudaMemcpy(L.dist_bias, table.data(), table.size() * 4, cudaMemcpyHostToDevice));
        }
        const int RH = lc.r_heads, rd = lc.r_dim, hd = RH * rd, R = lc.r_decay_rank;
        RCHECK(dmalloc((void**)&L.mu, (size_t)5 * D * 4));
        const char* mixes[5] = {"r", "k", "v", "g", "w"};
        for (int i = 0; i < 5; ++i) RCHECK(put_f32(m, rt + "mu." + mixes[i], D, L.mu, (size_t)i * D));
        RCHECK(dmalloc(&L.w_rkvg, (size_t)4 * hd * D * m->esz));
        for (int i = 0; i < 4; ++i) RCHECK(put_weight(m, rt + mixes[i], hd, D, L.w_rkvg, (size_t)i * hd * D));
        RCHECK(take_weight(m, rt + "w1", R, D, &L.w1));
        RCHECK(take_weight(m, rt + "w2", hd, R, &L.w2));
        RCHECK(take_f32(m, rt + "w0", 1, hd, &L.w0));
        RCHECK(bias_act_copy(m, L.w0, hd, &L.w0_act));
        RCHECK(take_f32(m, rt + "u", RH, rd, &L.bonus));
        RCHECK(take_f32(m, rt + "norm", 1, hd, &L.r_norm));
        RCHECK(take_weight(m, rt + "o", D, hd, &L.r_o));
    }
    if (lc.ff > 0) {
        RCHECK(take_f32(m, p + "norm2", 1, D, &L.norm2));
        RCHECK(finalize_ff(m, l));
    }
    RCHECK(take_weight(m, p + "side.gate", c.side_dim, D, &L.s_gate));
    RCHECK(take_weight(m, p + "side.proj", D, c.side_dim, &L.s_proj));
    RCHECK(take_f32(m, p + "side.norm", 1, D, &L.s_norm));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    L.ready = true;
    return ZL_OK;
}

int len_bucket(const zl_lagelorn* m, int max_len) {
    int b = 256;
    while (b < max_len) b <<= 1;
    return b < m->cfg.max_seq ? b : (m->cfg.max_seq > 256 ? m->cfg.max_seq : 256);
}
// the longest key range a token of this layer can see
int attn_span(const GLayer& L, int max_len) { return L.c.l_chunk > 0 ? std::min(L.c.l_chunk, max_len) : max_len; }

int alloc_runtime(zl_lagelorn* m) {
    const auto& c = m->cfg;
    const int D = c.width, T = m->tcap, B = c.max_batch;
    size_t n_in = 1, hd = 1, hq = 1, hv = 1, rank = 1, ff = 1;
    for (auto& L : m->layers) {
        const auto& lc = L.c;
        if (lc.type == ZL_LAYER_DELTA) {
            RCHECK(zl_delta_rule_prepare(lc.dim, lc.vdim));
            RCHECK(L.state.create(B, (size_t)lc.heads * lc.dim * lc.vdim * 4, m->stream));
            if (lc.conv > 1) RCHECK(L.ring.create(B, (size_t)(lc.conv - 1) * L.b_off * 4, m->stream));
            m->delta_ws_bytes = std::max(m->delta_ws_bytes, zl_delta_rule_workspace_bytes(T, lc.heads, lc.dim, lc.vdim));
            hv = std::max(hv, (size_t)lc.heads * lc.vdim);
        } else {
            RCHECK(L.kcache.create(B, (size_t)c.max_seq * lc.l_kv_heads * lc.l_dim * m->esz, m->stream));
            RCHECK(L.vcache.create(B, (size_t)c.max_seq * lc.l_kv_heads * lc.l_dim * m->esz, m->stream));
            for (int b = 1; b <= T; ++b) {
                const int s = zl_sink_attention_splits(b, lc.l_heads, lc.l_kv_heads, attn_span(L, len_bucket(m, c.max_seq)));
                m->attn_ws_bytes = std::max(m->attn_ws_bytes, zl_sink_attention_workspace_bytes(b, lc.l_heads, lc.l_dim, s));
                if (s == 1) break;
            }
            RCHECK(zl_delta_rule_prepare(lc.r_dim, lc.r_dim));
            RCHECK(L.r_state.create(B, (size_t)lc.r_heads * lc.r_dim * lc.r_dim * 4, m->stream));
            RCHECK(L.shift.create(B, (size_t)D * 4, m->stream));
            m->delta_ws_bytes = std::max(m->delta_ws_bytes, zl_delta_rule_workspace_bytes(T, lc.r_heads, lc.r_dim, lc.r_dim));
            hq = std::max(hq, (size_t)lc.l_heads * lc.l_dim);
            hv = std::max(hv, std::max((size_t)lc.l_heads * lc.l_dim, (size_t)lc.r_heads * lc.r_dim));
            hd = std::max(hd, (size_t)lc.r_heads * lc.r_dim);
            rank = std::max(rank, (size_t)lc.r_decay_rank);
        }
        n_in = std::max(n_in, (size_t)L.n_in);
        ff = std::max(ff, (size_t)lc.ff);
    }
    const size_t e = m->esz, S = (size_t)c.num_layers * c.side_dim;
    RCHECK(dmalloc((void**)&m->x, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->proj, (size_t)T * n_in * 4));
    RCHECK(dmalloc((void**)&m->rkvg, (size_t)4 * T * hd * 4));
    RCHECK(dmalloc((void**)&m->dlog, (size_t)T * hd * 4));
    RCHECK(dmalloc((void**)&m->orec, (size_t)T * hv * 4));
    RCHECK(dmalloc((void**)&m->y, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->y2, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->side, (size_t)T * S * 4));
    RCHECK(dmalloc((void**)&m->xw, (size_t)T * D * 4));
    RCHECK(dmalloc((void**)&m->logits, (size_t)T * c.vocab * 4));
    RCHECK(dmalloc(&m->xa, (size_t)T * D * e));
    RCHECK(dmalloc(&m->mix, (size_t)5 * T * D * e));
    RCHECK(dmalloc(&m->q, (size_t)T * hq * e));
    RCHECK(dmalloc(&m->att, (size_t)T * hv * e));
    RCHECK(dmalloc(&m->z1, (size_t)T * rank * e));
    RCHECK(dmalloc(&m->act, (size_t)T * ff * e));
    RCHECK(dmalloc(&m->sg, (size_t)T * c.side_dim * e));
    RCHECK(dmalloc(&m->xn, (size_t)T * D * e));
    for (int32_t** p : {&m->d_tokens, &m->d_slots, &m->d_pos, &m->d_want, &m->d_next, &m->d_run0, &m->d_runlen})
        RCHECK(dmalloc((void**)p, (size_t)T * 4));
    RCHECK(dmalloc(&m->attn_ws, m->attn_ws_bytes));
    RCHECK(dmalloc(&m->delta_ws, m->delta_ws_bytes));
    RCHECK(dmalloc(&m->argmax_ws, zl_argmax_workspace_bytes(T)));
    ZL_CHECK_CUDA(cudaMallocHost((void**)&m->h_stage, sizeof(int32_t) * 7 * (size_t)T));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

// Which kernels of a step of at most 8 rows are launched with a programmatic dependency: 1 skinny Linears, 2 other GEMMs,
// 4 row kernels (norms, mixes, head prep), 8 attention, 16 recurrences, 32 the tail.  Larger steps use none.
// ZL_LAGELORN_PDL_MASK overrides the default.
constexpr int kDefaultPdlMask = 1;
int pdl_mask() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("ZL_LAGELORN_PDL_MASK");
        v = e ? atoi(e) : kDefaultPdlMask;
    }
    return v;
}
int pdl_for(const zl_lagelorn* m, int bit, int T) { return (m->cfg.use_pdl && T <= 8 && (pdl_mask() & bit)) ? 1 : 0; }

// y (M, N) = x (M, K) @ w (N, K)^T + bias, optional epilogue.  bias_f32 / bias_act are the same numbers in two types.
int linear(zl_lagelorn* m, const void* x, int K, const void* w, int N, const float* bias_f32, const void* bias_act, void* y,
           int M, int out_dtype, int epi) {
    const auto& c = m->cfg;
    static const bool no_skinny = getenv("ZL_LAGELORN_NO_SKINNY") != nullptr;
    // the skinny kernel: plain Linears of up to 32 rows, and the narrow tanh projection of 9 .. 32 rows (a tile kernel would
    // put one CTA on its 64 columns; up to 8 rows the streamed few-rows kernel inside zl_gemm_nt_bias is the faster one)
    const bool skinny_epi = epi == ZL_GEMM_EPI_NONE || (epi == ZL_GEMM_EPI_TANH && M > 8);
    if (!no_skinny && c.dtype != ZL_F32 && skinny_epi && M <= 32 && K % 32 == 0 && N >= 64 && (!bias_f32 || bias_act) &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0)
        return zl_dense_gemm_skinny_act(x, K, w, bias_act, y, M, N, K, c.dtype, out_dtype, epi == ZL_GEMM_EPI_TANH ? 2 : 0,
                                        pdl_for(m, 1, M), m->stream);
    return zl_gemm_nt_bias(x, K, w, K, bias_f32, y, N, M, N, K, c.dtype, out_dtype, epi, pdl_for(m, 2, M), m->stream);
}

int enqueue_step(zl_lagelorn* m, int T, int n_want, int n_runs, int max_run, int max_len) {
    const auto& c = m->cfg;
    const int D = c.width, dt = c.dtype, S = c.num_layers * c.side_dim;
    cudaStream_t st = m->stream;
    const int pg = pdl_for(m, 2, T), pr = pdl_for(m, 4, T), pa = pdl_for(m, 8, T), pd = pdl_for(m, 16, T), pt = pdl_for(m, 32, T);
    const void* xin = dt == ZL_F32 ? (const void*)m->x : (const void*)m->xa;   // what the Linears read
    void* xa_out = dt == ZL_F32 ? nullptr : m->xa;
    const bool single = n_runs == T;   // every row is a run of its own
    if (dt == ZL_F32) {
        ZL_CHECK_CUDA(launch(k_embed_pos_side<float>, dim3(T, 2), dim3(256), 0, st, false, (const int32_t*)m->d_tokens,
                             (const int32_t*)m->d_pos, (const float*)m->embed, (const float*)m->pos_table,
                             (const float*)m->side_embed, m->x, (float*)nullptr, m->side, D, S, c.vocab, c.max_positions));
    } else {
        ZL_CHECK_CUDA(launch(k_embed_pos_side<__nv_bfloat16>, dim3(T, 2), dim3(256), 0, st, false, (const int32_t*)m->d_tokens,
                             (const int32_t*)m->d_pos, (const __nv_bfloat16*)m->embed, (const __nv_bfloat16*)m->pos_table,
                             (const __nv_bfloat16*)m->side_embed, m->x, (__nv_bfloat16*)m->xa, m->side, D, S, c.vocab,
                             c.max_positions));
    }
    for (int l = 0; l < c.num_layers; ++l) {
        GLayer& L = m->layers[l];
        const auto& lc = L.c;
        if (lc.type == ZL_LAYER_DELTA) {
            const int H = lc.heads, hv = H * lc.vdim;
            RCHECK(linear(m, xin, D, L.w_in, L.n_in, nullptr, nullptr, m->proj, T, ZL_F32, ZL_GEMM_EPI_NONE));
            RCHECK(zl_gated_delta_rule(m->proj, L.n_in, L.q_off, L.b_off, L.a_off, L.conv_w, lc.conv, L.a_log, L.dt_bias, 1e-6f,
                                       1.0f / sqrtf((float)lc.dim), L.ring.addrs, m->d_run0, m->d_runlen, n_runs, m->d_slots,
                                       m->d_pos, L.state.addrs, m->orec, hv, H, lc.kv_heads, lc.dim, lc.vdim, T, m->delta_ws,
                                       m->delta_ws_bytes, pd, st));
            RCHECK(zl_head_rmsnorm_gate_fn(m->orec, hv, L.out_norm, 0, m->proj + L.g_off, L.n_in, ZL_GATE_SILU, m->att, hv, T, H,
                                           lc.vdim, c.eps, dt, pr, st));
            RCHECK(linear(m, m->att, hv, L.o, D, nullptr, nullptr, m->y, T, ZL_F32, ZL_GEMM_EPI_NONE));
            RCHECK(zl_postnorm_combine(m->x, D, c.postln_alpha, m->y, D, 1.0f, nullptr, 0, 0.f, L.norm1, xa_out, dt, T, D, c.eps,
                                       pr, st));
        } else {
            const int H = lc.l_heads, G = lc.l_kv_heads, d = lc.l_dim, RH = lc.r_heads, rd = lc.r_dim, hd = RH * rd;
            const size_t esz = m->esz;
            // the mixes of the decaying-state mixer (they read x before anything of this layer changes it)
            RCHECK(zl_token_shift_mix(m->x, D, L.mu, 5, L.shift.addrs, m->d_slots, m->d_pos, m->mix, (long long)T * D, T, D,
                                      single ? 1 : 0, dt, pr, st));
            if (!single) RCHECK(zl_store_run_tails(m->x, D, 0, D, 1, m->d_run0, m->d_runlen, n_runs, m->d_slots, m->d_pos,
                                                   L.shift.addrs, pr, st));
            // attention
            RCHECK(linear(m, xin, D, L.w_in, L.n_in, L.b_in, L.b_in_act, m->proj, T, ZL_F32, ZL_GEMM_EPI_NONE));
            RCHECK(zl_qk_fullnorm_append(m->proj, L.n_in, L.q_off, L.k_off, H, G, d, L.q_norm, L.k_norm, c.eps, m->q, L.kcache.addrs,
                                         L.vcache.addrs, m->d_slots, m->d_pos, T, dt, pr, st));
            const int splits = zl_sink_attention_splits(T, H, G, attn_span(L, max_len));
            RCHECK(zl_sink_attention_local(m->q, L.kcache.addrs, L.vcache.addrs, m->d_slots, m->d_pos, L.sink, nullptr, 0, lc.l_scale,
                                           lc.l_chunk, L.dist_bias, L.n_dist, m->att, T, H, G, d, d, splits, m->attn_ws,
                                           m->attn_ws_bytes, m->d_run0, m->d_runlen, n_runs, max_run, dt, pa, st));
            RCHECK(linear(m, m->att, H * d, L.o, D, nullptr, nullptr, m->y, T, ZL_F32, ZL_GEMM_EPI_NONE));
            // decaying state
            RCHECK(zl_gemm_nt(m->mix, D, (long long)T * D, L.w_rkvg, D, (long long)hd * D, m->rkvg, hd, (long long)T * hd, T, hd, D,
                              4, dt, ZL_F32, ZL_GEMM_EPI_NONE, nullptr, 0, 0, pg, st));
            RCHECK(linear(m, (const char*)m->mix + (size_t)4 * T * D * esz, D, L.w1, lc.r_decay_rank, nullptr, nullptr, m->z1, T, dt,
                          ZL_GEMM_EPI_TANH));
            RCHECK(linear(m, m->z1, lc.r_decay_rank, L.w2, hd, L.w0, L.w0_act, m->dlog, T, ZL_F32, ZL_GEMM_EPI_NONE));
            const float* rk = m->rkvg;
            RCHECK(zl_bonus_decay_scan(rk, hd, rk + (size_t)T * hd, hd, rk + (size_t)2 * T * hd, hd, m->dlog, hd, L.bonus, m->d_run0,
                                       m->d_runlen, n_runs, m->d_slots, m->d_pos, L.r_state.addrs, m->orec, hd, RH, rd, rd, T,
                                       m->delta_ws, m->delta_ws_bytes, pd, st));
            RCHECK(zl_head_rmsnorm_gate_fn(m->orec, hd, L.r_norm, rd, rk + (size_t)3 * T * hd, hd, ZL_GATE_SILU, m->att, hd, T, RH, rd,
                                           c.eps, dt, pr, st));
            RCHECK(linear(m, m->att, hd, L.r_o, D, nullptr, nullptr, m->y2, T, ZL_F32, ZL_GEMM_EPI_NONE));
            RCHECK(zl_postnorm_combine(m->x, D, c.postln_alpha, m->y, D, lc.left_scale, m->y2, D, lc.right_scale, L.norm1, xa_out, dt,
                                       T, D, c.eps, pr, st));
        }
        if (lc.ff > 0) {
            RCHECK(zl_gemm_nt_fused(xin, D, L.w_gu, D, L.b_gu, m->act, lc.ff, T, 2 * lc.ff, D, dt, dt, ZL_GEMM_EPI_GEGLU_TANH, nullptr,
                                    0, 0.f, pg, st));
            RCHECK(linear(m, m->act, lc.ff, L.w_down, D, L.b_down, L.b_down_act, m->y, T, ZL_F32, ZL_GEMM_EPI_NONE));
            RCHECK(zl_postnorm_combine(m->x, D, c.postln_alpha, m->y, D, 1.0f, nullptr, 0, 0.f, L.norm2, xa_out, dt, T, D, c.eps, pr,
                                       st));
        }
        // the layer's slice of the token's second embedding
        if (dt != ZL_F32 && T > 8 && T <= 32 && D % 32 == 0 && c.side_dim >= 64 && (reinterpret_cast<uintptr_t>(L.s_gate) & 15) == 0)
            RCHECK(zl_dense_gemm_skinny_mul(xin, D, L.s_gate, nullptr, m->sg, T, c.side_dim, D, dt, dt, 3,
                                            m->side + (size_t)l * c.side_dim, S, pdl_for(m, 1, T), st));
        else
            RCHECK(zl_gemm_nt_fused(xin, D, L.s_gate, D, nullptr, m->sg, c.side_dim, T, c.side_dim, D, dt, dt,
                                    ZL_GEMM_EPI_GELU_TANH_MUL, m->side + (size_t)l * c.side_dim, S, 0.f, pg, st));
        RCHECK(linear(m, m->sg, c.side_dim, L.s_proj, D, nullptr, nullptr, m->y, T, ZL_F32, ZL_GEMM_EPI_NONE));
        RCHECK(zl_rmsnorm_residual_combine(m->y, D, nullptr, 1, L.s_norm, m->x, D, xa_out, dt, T, D, c.eps, pr, st));
        if (m->capture && m->layer_dump)
            ZL_CHECK_CUDA(cudaMemcpyAsync(m->layer_dump + (size_t)l * m->tcap * D, m->x, (size_t)T * D * 4,
                                          cudaMemcpyDeviceToDevice, st));
    }
    if (n_want > 0) {
        ZL_CHECK_CUDA(launch(k_gather_rows_f32, dim3(n_want), dim3(128), 0, st, false, (const float*)m->x,
                             (const int32_t*)m->d_want, m->xw, D));
        RCHECK(zl_group_rmsnorm(m->xw, D, m->final_norm, m->xn, D, n_want, D, 1, c.eps, dt, pt, st));
        RCHECK(zl_gemm_nt_fused(m->xn, D, m->head, D, nullptr, m->logits, c.vocab, n_want, c.vocab, D, dt, ZL_F32, ZL_GEMM_EPI_SOFTCAP,
                                nullptr, 0, c.logit_softcap, pg, st));
        RCHECK(zl_argmax(m->logits, m->d_next, n_want, c.vocab, m->argmax_ws, zl_argmax_workspace_bytes(n_want), pt, st));
    }
    return ZL_OK;
}

// decode-sized steps replay a CUDA graph per (rows, wanted rows, runs, length bucket); prompt portions are enqueued directly
// (max_run: the longest run; a captured step is sized for the longest run its row count allows)
int run_step(zl_lagelorn* m, int T, int n_want, int n_runs, int max_run, int max_len) {
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

extern "C" int zl_lagelorn_create(const zl_lagelorn_config_t* cfg, const zl_lagelorn_layer_t* layers, zl_lagelorn_t** out) {
    ZL_CHECK_ARG(cfg && layers && out);
    ZL_CHECK_ARG(cfg->num_layers > 0 && cfg->width > 0 && cfg->vocab > 0 && cfg->max_batch > 0 && cfg->max_seq > 0);
    ZL_CHECK_ARG(cfg->max_positions >= cfg->max_seq && cfg->side_dim > 0 && cfg->eps >= 0.f && cfg->logit_softcap > 0.f);
    ZL_CHECK_SUPPORTED(cfg->dtype == ZL_BF16 || cfg->dtype == ZL_F32);
    ZL_CHECK_ARG(cfg->max_step_tokens >= 0 && cfg->max_step_tokens <= 65535);
    for (int l = 0; l < cfg->num_layers; ++l) {
        const auto& lc = layers[l];
        ZL_CHECK_ARG(lc.ff >= 0);
        if (lc.type == ZL_LAYER_DELTA) {
            ZL_CHECK_ARG(lc.heads > 0 && lc.kv_heads > 0 && lc.heads % lc.kv_heads == 0 && lc.dim > 0 && lc.vdim > 0 && lc.conv >= 1);
        } else {
            ZL_CHECK_ARG(lc.type == ZL_LAYER_PARALLEL);
            ZL_CHECK_ARG(lc.l_heads > 0 && lc.l_kv_heads > 0 && lc.l_heads % lc.l_kv_heads == 0 && lc.l_dim > 0);
            ZL_CHECK_ARG(lc.l_chunk >= 0 && lc.l_rel_rows > 0 && (lc.l_rel_rows == 1 || lc.l_bias_max > (float)(lc.l_rel_rows / 2)));
            ZL_CHECK_ARG(lc.r_heads > 0 && lc.r_dim > 0 && lc.r_decay_rank > 0);
        }
    }
    zl_lagelorn* m = new zl_lagelorn();
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
    *out = m;
    return ZL_OK;
}

extern "C" void zl_lagelorn_destroy(zl_lagelorn_t* m) {
    if (!m) return;
    cudaStreamSynchronize(m->stream);
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
    for (auto& s : m->staged) cudaFree(s.second.ptr);
    for (auto& L : m->layers) {
        for (void* p : {(void*)L.norm1, (void*)L.norm2, L.w_in, (void*)L.b_in, L.b_in_act, L.o, (void*)L.conv_w, (void*)L.a_log,
                        (void*)L.dt_bias, (void*)L.out_norm, (void*)L.q_norm, (void*)L.k_norm, (void*)L.dist_bias, (void*)L.sink,
                        (void*)L.mu, L.w_rkvg, L.w1, L.w2, L.r_o, (void*)L.w0, (void*)L.bonus, (void*)L.r_norm, L.w0_act, L.w_gu,
                        L.w_down, (void*)L.b_gu, (void*)L.b_down, L.b_down_act, L.s_gate, L.s_proj, (void*)L.s_norm})
            if (p) cudaFree(p);
        for (SlotCache* sc : {&L.state, &L.ring, &L.kcache, &L.vcache, &L.r_state, &L.shift}) sc->destroy();
    }
    for (void* p : {m->embed, m->pos_table, m->side_embed, m->head, (void*)m->final_norm, (void*)m->x, (void*)m->proj, (void*)m->rkvg,
                    (void*)m->dlog, (void*)m->orec, (void*)m->y, (void*)m->y2, (void*)m->side, (void*)m->xw, (void*)m->logits, m->xa,
                    m->mix, m->q, m->att, m->z1, m->act, m->sg, m->xn, (void*)m->d_tokens, (void*)m->d_slots, (void*)m->d_pos,
                    (void*)m->d_want, (void*)m->d_next, (void*)m->d_run0, (void*)m->d_runlen, m->attn_ws, m->delta_ws, m->argmax_ws,
                    (void*)m->layer_dump})
        if (p) cudaFree(p);
    if (m->h_stage) cudaFreeHost(m->h_stage);
    cudaStreamDestroy(m->stream);
    delete m;
}

extern "C" int zl_lagelorn_load_tensor(zl_lagelorn_t* m, const char* name, const void* data_host, int rows, int cols,
                                       int elem_bytes) {
    ZL_CHECK_ARG(m && name && data_host && rows > 0 && cols > 0 && (elem_bytes == 2 || elem_bytes == 4));
    if (m->finalized) return fail(__LINE__, "model already finalized");
    return staged_load(m->staged, name, data_host, rows, cols, elem_bytes, m->stream);
}

extern "C" int zl_lagelorn_finalize(zl_lagelorn_t* m) {
    ZL_CHECK_ARG(m);
    if (m->finalized) return ZL_OK;
    const auto& c = m->cfg;
    for (int l = 0; l < c.num_layers; ++l)
        if (!m->layers[l].ready) RCHECK(finalize_layer(m, l));
    RCHECK(take_weight(m, "embed", c.vocab, c.width, &m->embed));
    RCHECK(take_weight(m, "pos", c.max_positions, c.width, &m->pos_table));
    RCHECK(take_weight(m, "side.embed", c.vocab, c.num_layers * c.side_dim, &m->side_embed));
    // gathered, not streamed
    m->weight_bytes -= ((double)c.vocab * c.width + (double)c.max_positions * c.width + (double)c.vocab * c.num_layers * c.side_dim) * m->esz;
    RCHECK(take_weight(m, "head", c.vocab, c.width, &m->head));
    RCHECK(take_f32(m, "final.norm", 1, c.width, &m->final_norm));
    RCHECK(alloc_runtime(m));
    m->finalized = true;
    return ZL_OK;
}

extern "C" int zl_lagelorn_init_synthetic(zl_lagelorn_t* m, uint64_t seed) {
    ZL_CHECK_ARG(m);
    if (m->finalized) return fail(__LINE__, "model already finalized");
    const auto& c = m->cfg;
    const int D = c.width;
    auto lin = [&](const std::string& name, int n, int k) {
        const float a = sqrtf(3.0f / (float)k);   // unit-variance outputs for unit-variance inputs
        return stage_random(m, name, n, k, -a, a, seed);
    };
    auto small = [&](const std::string& name, int n, float a) { return stage_random(m, name, 1, n, -a, a, seed); };
    auto around = [&](const std::string& name, int n, float mid, float a) { return stage_random(m, name, 1, n, mid - a, mid + a, seed); };
    for (int l = 0; l < c.num_layers; ++l) {
        const auto& lc = m->layers[l].c;
        const std::string p = "l" + std::to_string(l) + ".", mx = p + "mix.";
        RCHECK(around(p + "norm1", D, 1.0f, 0.1f));
        if (lc.type == ZL_LAYER_DELTA) {
            const int H = lc.heads, G = lc.kv_heads, d = lc.dim, vd = lc.vdim;
            RCHECK(lin(mx + "q", G * d, D));
            RCHECK(lin(mx + "k", G * d, D));
            RCHECK(lin(mx + "v", H * vd, D));
            RCHECK(lin(mx + "b", H, D));
            RCHECK(lin(mx + "a", H, D));
            RCHECK(lin(mx + "g", H * vd, D));
            RCHECK(stage_random(m, mx + "q.conv", G * d, lc.conv, -0.6f, 0.6f, seed));
            RCHECK(stage_random(m, mx + "k.conv", G * d, lc.conv, -0.6f, 0.6f, seed));
            RCHECK(stage_random(m, mx + "v.conv", H * vd, lc.conv, -0.6f, 0.6f, seed));
            RCHECK(small(mx + "A_log", H, 1.0f));
            RCHECK(small(mx + "dt_bias", H, 1.0f));
            RCHECK(around(mx + "norm", vd, 1.0f, 0.1f));
            RCHECK(lin(mx + "o", D, H * vd));
        } else {
            const std::string lf = mx + "left.", rt = mx + "right.";
            const int H = lc.l_heads, G = lc.l_kv_heads, d = lc.l_dim, hd = lc.r_heads * lc.r_dim;
            RCHECK(lin(lf + "q", H * d, D));
            RCHECK(small(lf + "q.b", H * d, 0.1f));
            RCHECK(lin(lf + "k", G * d, D));
            RCHECK(small(lf + "k.b", G * d, 0.1f));
            RCHECK(around(lf + "q.norm", H * d, 1.0f, 0.1f));
            RCHECK(around(lf + "k.norm", G * d, 1.0f, 0.1f));
            RCHECK(stage_random(m, lf + "rel", lc.l_rel_rows, H, -1.0f, 1.0f, seed));
            RCHECK(small(lf + "sink", H, 1.0f));
            RCHECK(lin(lf + "o", D, H * d));
            for (const char* n : {"r", "k", "v", "g", "w"}) RCHECK(around(rt + "mu." + n, D, 0.5f, 0.5f));
            for (const char* n : {"r", "k", "v", "g"}) RCHECK(lin(rt + n, hd, D));
            RCHECK(lin(rt + "w1", lc.r_decay_rank, D));
            RCHECK(lin(rt + "w2", hd, lc.r_decay_rank));
            RCHECK(around(rt + "w0", hd, -2.0f, 1.5f));
            RCHECK(stage_random(m, rt + "u", lc.r_heads, lc.r_dim, -0.5f, 0.5f, seed));
            RCHECK(around(rt + "norm", hd, 1.0f, 0.1f));
            RCHECK(lin(rt + "o", D, hd));
        }
        if (lc.ff > 0) {
            RCHECK(around(p + "norm2", D, 1.0f, 0.1f));
            RCHECK(lin(p + "mlp.gate", lc.ff, D));
            RCHECK(small(p + "mlp.gate.b", lc.ff, 0.1f));
            RCHECK(lin(p + "mlp.up", lc.ff, D));
            RCHECK(small(p + "mlp.up.b", lc.ff, 0.1f));
            RCHECK(lin(p + "mlp.down", D, lc.ff));
            RCHECK(small(p + "mlp.down.b", D, 0.1f));
        }
        RCHECK(lin(p + "side.gate", c.side_dim, D));
        RCHECK(lin(p + "side.proj", D, c.side_dim));
        RCHECK(around(p + "side.norm", D, 0.3f, 0.1f));
        RCHECK(finalize_layer(m, l));   // bound the staging memory to one layer
    }
    RCHECK(stage_random(m, "embed", c.vocab, D, -1.7f, 1.7f, seed));
    RCHECK(stage_random(m, "pos", c.max_positions, D, -0.5f, 0.5f, seed));
    RCHECK(stage_random(m, "side.embed", c.vocab, c.num_layers * c.side_dim, -1.7f, 1.7f, seed));
    RCHECK(lin("head", c.vocab, D));
    RCHECK(around("final.norm", D, 1.0f, 0.1f));
    return zl_lagelorn_finalize(m);
}

extern "C" int zl_lagelorn_step(zl_lagelorn_t* m, const int32_t* tokens_host, const int32_t* slots_host,
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
            for (int j = 0; j < n_runs; ++j) ZL_CHECK_ARG(slots_host[hs[5 * T + j]] != slots_host[i]);
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

extern "C" int zl_lagelorn_set_state(zl_lagelorn_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B) {
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

extern "C" int zl_lagelorn_step_device(zl_lagelorn_t* m, int B) {
    ZL_CHECK_ARG(m && B > 0 && B <= m->cfg.max_batch);
    if (m->cur_max_len >= m->cfg.max_seq) return fail(__LINE__, "caches full (max_seq reached)");
    RCHECK(run_step(m, B, B, B, 1, m->cur_max_len));
    k_decode_advance<<<cdiv(B, 64), 64, 0, m->stream>>>(m->d_tokens, m->d_pos, m->d_next, B);
    ZL_CHECK_LAUNCH();
    m->cur_max_len += 1;
    return ZL_OK;
}

extern "C" int zl_lagelorn_sync(zl_lagelorn_t* m) {
    ZL_CHECK_ARG(m);
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" zl_stream_t zl_lagelorn_stream(zl_lagelorn_t* m) { return m ? (zl_stream_t)m->stream : nullptr; }

extern "C" int zl_lagelorn_capture_layers(zl_lagelorn_t* m, int on) {
    ZL_CHECK_ARG(m);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    if (on && !m->layer_dump)
        RCHECK(dmalloc((void**)&m->layer_dump, (size_t)m->cfg.num_layers * m->tcap * m->cfg.width * 4));
    m->capture = on != 0;
    return ZL_OK;
}

extern "C" int zl_lagelorn_read_layers(zl_lagelorn_t* m, float* out_host, int T) {
    ZL_CHECK_ARG(m && out_host && T > 0 && T <= m->tcap);
    if (!m->layer_dump) return fail(__LINE__, "layer capture was not switched on");
    const size_t row = (size_t)m->cfg.width * 4;
    ZL_CHECK_CUDA(cudaMemcpy2DAsync(out_host, (size_t)T * row, m->layer_dump, (size_t)m->tcap * row, (size_t)T * row,
                                    m->cfg.num_layers, cudaMemcpyDeviceToHost, m->stream));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

extern "C" int zl_lagelorn_read_state(zl_lagelorn_t* m, int layer, int slot, float* out_host) {
    ZL_CHECK_ARG(m && out_host && layer >= 0 && layer < m->cfg.num_layers && slot >= 0 && slot < m->cfg.max_batch);
    if (!m->finalized) return fail(__LINE__, "model not finalized");
    const GLayer& L = m->layers[layer];
    const SlotCache& sc = L.c.type == ZL_LAYER_DELTA ? L.state : L.r_state;
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    ZL_CHECK_CUDA(cudaMemcpy(out_host, (const char*)sc.buf + (size_t)slot * sc.slot_bytes, sc.slot_bytes, cudaMemcpyDeviceToHost));
    return ZL_OK;
}

extern "C" int zl_lagelorn_stats(zl_lagelorn_t* m, double* weight_bytes, int* kernels_per_step) {
    ZL_CHECK_ARG(m);
    if (weight_bytes) *weight_bytes = m->weight_bytes;
    if (kernels_per_step) *kernels_per_step = m->kernels_per_step;
    return ZL_OK;
}

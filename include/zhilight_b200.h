/*
 * zhilight_b200 -- C-ABI of the B200-native (sm_100a) quantized-decode hot path of ZhiLight.
 *
 * Every entry point replaces one reference operator (cited as file:line under /root/reference).
 * Conventions:
 *   - plain pointers + sizes, no C++/torch types; all data pointers are DEVICE pointers unless
 *     the name ends in _host;
 *   - stream-ordered on `stream`, no allocation, no host sync inside (except zl_llama_* which
 *     owns its buffers);
 *   - returns ZL_OK (0) or a negative error code; zl_last_error() gives the message of the last
 *     failure on the calling thread.  The C++ mirror (zhilight_b200/host) turns codes into the
 *     reference's BMEngineException behaviour;
 *   - re-entrant per device; no global mutable state besides per-device symmetric buffers
 *     created by zl_comm_*.
 *
 * dtype codes follow bmengine core::DataType ordering where they overlap
 * (3rd/bmengine/bmengine/include/bmengine/core/dtype.h).
 */
#ifndef ZHILIGHT_B200_H_
#define ZHILIGHT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* zl_stream_t; /* == cudaStream_t */

enum {
    ZL_OK = 0,
    ZL_ERR_INVALID_ARG = -1,
    ZL_ERR_UNSUPPORTED = -2,
    ZL_ERR_CUDA = -3,
    ZL_ERR_STATE = -4
};

enum { ZL_F16 = 0, ZL_BF16 = 1, ZL_F32 = 2 };

/* epilogues of zl_w4a16_gemm */
enum {
    ZL_EPI_NONE = 0,     /* y = acc (+bias)                                                     */
    ZL_EPI_SWIGLU = 1,   /* packed rows interleave gate/up; y[:, n] = silu(T(gate)) * T(up)      */
    ZL_EPI_RESIDUAL = 2, /* y = T(T(acc (+bias)) + residual)   (block_kernel.cu:7-17)           */
    ZL_EPI_QKV_ROPE = 3  /* fused qkv: split + RoPE(q,k) + KV append (zl_w4a16_gemm_fused only)    */
};

const char* zl_last_error(void);
int zl_version(void);
/* number of kernel launches issued by this library on the calling thread since the last reset */
long long zl_launch_count(int reset);
/* one-time per-device kernel attribute setup (opt-in shared memory); called by zl_llama_create and lazily
 * by the ops; must not first happen inside a stream capture. */
int zl_prepare(void);

/* ------------------------------------------------------------------------------------------ *
 * Load-time integer layout transforms (bit-exact with the reference)
 * ------------------------------------------------------------------------------------------ */
/* nn::gptq::gptq_shuffle  (src/nn/quant/gptq/q_gemm.cu:778-872, qdq_4.cuh:16-35).
 * qweight (K/8, N) int32 in place.  q_perm (K) int32 or NULL; scratch (K/8*N words) required iff q_perm. */
int zl_gptq_shuffle(uint32_t* qweight, const int32_t* q_perm, uint32_t* scratch, int K, int N,
                    zl_stream_t stream);
/* nn::gptq::increase_zero (src/nn/quant/gptq/utils.cu:61-88): each nibble (z+1)&15, in place. */
int zl_gptq_increase_zero(uint32_t* qzeros, size_t n_words, zl_stream_t stream);
/* nn::gptq::subtract8 (utils.cu:91-118). */
int zl_gptq_subtract8(uint32_t* words, size_t n_words, zl_stream_t stream);
/* nn::gptq::q4_to_q8 (utils.cu:177-214): (R, C/8) int32 -> (R, C) uint8. */
int zl_q4_to_q8(const uint32_t* in, uint8_t* out, size_t n_words, zl_stream_t stream);
/* nn::gptq::un_shuffle (utils.cu:25-58): AWQ zero de-interleave in place, (rows, cols) words. */
int zl_awq_un_shuffle(uint32_t* qzeros, int rows, int cols, zl_stream_t stream);
/* nn::gptq::shuffle_awq (utils.cu:121-174): (K, N/8) -> (K/8, N). */
int zl_awq_shuffle(const uint32_t* in, uint32_t* out, int K, int N, int use_exllama, zl_stream_t stream);
/* functions::Transpose for 2-D tensors of 1/2/4-byte elements: (rows, cols) -> (cols, rows). */
int zl_transpose_2d(const void* in, void* out, int rows, int cols, int elem_bytes, zl_stream_t stream);
/* nn::gptq::dequant_k_major out_type 0 (q_gemm_k_major.cu:843-905): W16[n,k] = half(q-z)*half(s). */
int zl_gptq_dequant_k_major(const uint32_t* qweight_km, const uint8_t* qzeros_km, const void* scales_km,
                            void* out_f16, int N, int K, int group_size, zl_stream_t stream);

/* ------------------------------------------------------------------------------------------ *
 * ZLW4: the B200 tile-packed W4 layout consumed by zl_w4a16_gemm.
 * Built once at load from the reference k-major tensors
 * (Int4GPTQ::preprocess_weight, src/nn/linear/linear.cpp:1139-1160).
 * ------------------------------------------------------------------------------------------ */
size_t zl_w4_packed_bytes(int N, int K, int group_size);
/* qweight_km (N_src, K/8) u32 shuffled, qzeros_km (N_src, K/g) u8 (NULL or sym!=0 -> zero 8),
 * scales_km (N_src, K/g) f16.  row_map (N) int32 or NULL: packed row p takes source row row_map[p]. */
int zl_w4_pack(const uint32_t* qweight_km, const uint8_t* qzeros_km, const void* scales_km,
               const int32_t* row_map, void* packed, int N, int K, int group_size, int sym,
               zl_stream_t stream);
/* variant 0: ZLW4 (fp16 HMMA kernels); variant 1: ZLW4I (exact-integer IMMA kernel, zl_w4a16_gemm_fused with
 * args.variant = 1).  zl_w4_pack == variant 0. */
int zl_w4_pack_v(const uint32_t* qweight_km, const uint8_t* qzeros_km, const void* scales_km,
                 const int32_t* row_map, void* packed, int N, int K, int group_size, int sym, int variant,
                 zl_stream_t stream);
int zl_w4_unpack_v(const void* packed, uint32_t* qweight_km, uint8_t* qzeros_km, void* scales_km, int N, int K,
                   int group_size, int variant, zl_stream_t stream);
/* inverse (tests): recover k-major nibbles/zeros/scales from the packed form. */
int zl_w4_unpack(const void* packed, uint32_t* qweight_km, uint8_t* qzeros_km, void* scales_km, int N, int K,
                 int group_size, zl_stream_t stream);

/* nn::gptq::gptq_gemm_k_major / KERNEL_gemm_warp_reduce / gemm_fuse_gate_in
 * (src/nn/quant/gptq/q_gemm_k_major.cu:957-1116, 176-237, 529-578):
 * y[m,n] = sum_k x[m,k] * (q[n,k]-z[n,k/g]) * s[n,k/g] (+bias[n]), fp16 in/out, fp32 accumulate.
 * x (M, K) f16 row stride ldx; y (M, N_out) f16 where N_out = N (NONE/RESIDUAL) or N/2 (SWIGLU).
 * Any M >= 1 (weights are re-streamed per 32-token chunk).  pdl != 0 -> programmatic dependent launch. */
int zl_w4a16_gemm(const void* x, int ldx, const void* packed, const void* bias, const void* residual,
                  void* y, int M, int N, int K, int group_size, int epilogue, int pdl, zl_stream_t stream);

/* The same GEMM with the neighbouring operators of the decode layer folded in:
 *   ln_weight != NULL : nn::LayerNorm (rms, layernorm.cu:9-42) of x is fused into the prologue:
 *                       y = rsqrt(mean(x^2)+eps) * (W . (x*ln_weight)) (+bias);
 *   epilogue ZL_EPI_QKV_ROPE: W is the fused qkv weight packed with zl_qkv_rope_row_map; the epilogue applies
 *                       rope_qk_cache (rotary_embedding_fuse_cache.cu:23-63) and copy_to_rag_buffer2
 *                       (ragged_buffer_kernel.cu:194-222, BSHD) and writes q (M, num_heads*dim_head).
 *   tp_mode (tensor parallel, integer kernel only; replaces ModelContext::reduce_sum + element_add_scale between a
 *                       row-parallel Linear and the next column-parallel one, model_context.cpp:203-243, block.cpp:123-141):
 *                       2 on the row-parallel GEMM (o_proj / w_out, epilogue NONE, y unused): the fp16 partial tile is
 *                       stored straight into every rank's NVLink-mapped inbox of tp_comm as 8-byte words {2 x fp16, tag}
 *                       (valid on arrival: no flags, no fences);
 *                       1 on the next GEMM: its activation row becomes T(T(sum_r partial_r) + x), x = residual stream,
 *                       reduced in rank order while the activations are staged (the staging loop polls the words' tags);
 *                       the sum is also stored to tp_h_out (M, K; must not alias x).  0: off.
 *                       tp_index: index of the exchange within the step (0 .. 511, consecutive, the same on producer and
 *                       consumer), | 512 when the step has an ODD number of exchanges (the two slots must alternate across
 *                       step boundaries too); zl_comm_ll_begin_step(tp_comm) must be enqueued once per step before the
 *                       first such GEMM, on every rank.
 * bias is indexed by PACKED row. */
typedef struct zl_comm zl_comm_t;
typedef struct zl_w4_fused_args {
    const void* x; int ldx; const void* packed; const void* bias; const void* residual; void* y;
    int M, N, K, group_size, epilogue, pdl;
    const void* ln_weight; float eps;
    const float* cos; const float* sin; void* q_out;
    const int32_t* token_batch; const int32_t* placement; void* const* k_addrs; void* const* v_addrs;
    int num_heads, num_kv_heads, dim_head;
    const void* prefetch_ptr; size_t prefetch_bytes; /* next kernel's weights: pulled into L2 as this one drains (may be NULL) */
    int variant; /* layout of `packed`: 0 ZLW4, 1 ZLW4I (integer kernel; needs the staged activations to fit smem) */
    zl_comm_t* tp_comm; int tp_mode; void* tp_h_out; int tp_index;
} zl_w4_fused_args_t;
int zl_w4a16_gemm_fused(const zl_w4_fused_args_t* args, zl_stream_t stream);
/* 1 if the exact-integer kernel (variant 1, M <= 16) can run this shape: its staged activations must fit shared memory. */
int zl_w4_int_kernel_fits(int M, int N, int K);
/* which kernel serves (M, N, K) on the ZLW4I layout (variant 1): 3 = exact-integer mma.sync kernel, 4 = tcgen05 / TMEM /
 * TMA kernel (any M, N % 128 == 0, no fused RMSNorm prologue), 0 = neither (pack variant 0 and use the fp16 mma.sync kernel). */
int zl_w4_int_layout_route(int M, int N, int K);
/* last watchdog code published by a tcgen05 kernel on the current device (0 = none); a bounded mbarrier wait that expires
 * records which pipeline barrier starved and traps instead of hanging the GPU. */
unsigned zl_w4_tc_watchdog(void);
/* debug / tests: at least `splits` pieces per weight-row tile in the tcgen05 kernel's stream-k schedule (0 = automatic; also
 * ZL_TC_SPLITS). */
int zl_w4_tc_set_splits(int splits);
/* tests: host view of the tcgen05 kernel's stream-k schedule (the kernel's own scheduling code): pieces of CTA `cta` of `ctas`
 * for n_tiles x G (tile, group) units; out[5 i ..] = tile, g0, g1, pieces of that tile, workspace slot (-1: whole tile);
 * returns the number of pieces. */
int zl_w4_tc_schedule(int n_tiles, int G, int ctas, int cta, int* out, int max_pieces);
/* debug: with ZL_TC_DBG & 16, CTA 0 of the tcgen05 kernel stamps its pipeline hand-overs with clock64; copies
 * [11 roles][64 stages][4 events] of the last launch to `out` (n <= 2816 values). */
int zl_w4_tc_read_trace(long long* out, int n);
/* debug: device buffer of grid*16 uint64 globaltimer samples written by the integer kernel (NULL = off). */
int zl_w4_set_trace(void* buf);
/* row_map (n_heads_total*dim_head) for zl_w4_pack so that RoPE partners (c, c+d/2) share an MMA tile. */
int zl_qkv_rope_row_map(int32_t* row_map, int n_heads_total, int dim_head, zl_stream_t stream);
/* dst[i] = src[map[i]] for 16-bit elements (bias permutation to packed-row order). */
int zl_gather_rows_16(const void* src, const int32_t* map, void* dst, int n, zl_stream_t stream);

/* ---- W8A8 Linear: SmoothQuant INT8 (Int8Linear, src/nn/linear/linear.cpp:432-636) and per-tensor FP8 e4m3
 * (Fp8Linear, linear.cpp:1612-1695) ---------------------------------------------------------------------- */
enum { ZL_W8_INT8 = 0, ZL_W8_FP8 = 1, ZL_W8_FP8_ROWS = 2 /* fp8 with one f32 weight scale per output row */ };
/* int8_op::quant_calc_scale (src/nn/quant/int8/quant_kernel.cu:15-103): per-token absmax quantisation,
 * scale[m] = absmax/127, q = int8(nearbyint(x * (127/absmax))).  x (M,K) f16/bf16 row stride ldx; q (M,K) int8. */
int zl_int8_quant_per_token(const void* x, int ldx, void* q, float* scale, int M, int K, int dtype, int pdl,
                            zl_stream_t stream);
/* int8_op::layernorm_quant (quant_kernel.cu:106-227): y = RMSNorm(x)*w/scale in T plus the int8 twin q with
 * qscale[t] = absmax(x*w) * rsqrt / 127. */
int zl_rmsnorm_quant(const void* x, const void* weight, void* y, void* q, float* qscale, int T, int D, float eps,
                     float scale, int dtype, int pdl, zl_stream_t stream);
/* nn::fp8::dynamic_scaled_quant (src/nn/quant/fp8/fp8_util.cu:110-228): *scale = absmax/448 over all n elements,
 * q = e4m3(sat(x * (1/scale))) with the reference's fp16 product rounding.  n <= 4 Mi elements (decode sizes). */
int zl_fp8_quant_per_tensor(const void* x, void* q, float* scale, size_t n, int dtype, int pdl, zl_stream_t stream);
/* Int8Linear::forward GEMM + int8_op::quant_scale_back (+add_bias), or Fp8Linear::forward's scaled fp8 GEMM, as ONE
 * kernel: y(M,N) = T(acc * x_scale * w_scale) (+bias).  xq (M,K) int8/e4m3; w (N,K) int8/e4m3 row-major (the
 * reference's parameter layout); kind ZL_W8_INT8: x_scale (M) f32, w_scale (N) of w_scale_dtype (ZL_F32 or dtype);
 * kind ZL_W8_FP8: both scales one f32.  INT8 results are bit-identical to the reference's three-kernel path. */
/* int8_op::quant_scale_back (quant_kernel.cu:231-306) stand-alone: y = T(float(acc) * x_scale[m] * w_scale[n]). */
int zl_int8_scale_back(const int32_t* acc, const float* x_scale, const void* w_scale, int w_scale_dtype, void* y, int M,
                       int N, int dtype, zl_stream_t stream);
int zl_w8a8_gemm(const void* xq, const float* x_scale, const void* w, const void* w_scale, int w_scale_dtype,
                 const void* bias, void* y, int M, int N, int K, int kind, int dtype, int pdl, zl_stream_t stream);

/* functions::Gemm / NormalLinear for skinny M (lm_head, bf16 models; src/nn/linear/linear.cpp:150-430,
 * src/nn/embedding/embedding.cu:353-392): y(M,N) = x(M,K) @ W(N,K)^T (+bias), dtype f16/bf16,
 * out_dtype f16/bf16/f32. */
int zl_dense_gemm_skinny(const void* x, int ldx, const void* w, const void* bias, void* y, int M, int N, int K,
                         int dtype, int out_dtype, int pdl, zl_stream_t stream);
/* the same with an activation on the output: act 0 none, 1 relu(v)^2, 2 tanh(v) */
int zl_dense_gemm_skinny_act(const void* x, int ldx, const void* w, const void* bias, void* y, int M, int N, int K, int dtype,
                             int out_dtype, int act, int pdl, zl_stream_t stream);
/* act 0 none, 1 relu(v)^2, 2 tanh(v), 3 gelu_tanh(v) * mul[m * ld_mul + n] (mul fp32, device) */
int zl_dense_gemm_skinny_mul(const void* x, int ldx, const void* w, const void* bias, void* y, int M, int N, int K, int dtype,
                             int out_dtype, int act, const float* mul, int ld_mul, int pdl, zl_stream_t stream);

/* ------------------------------------------------------------------------------------------ *
 * Norm / residual / activation
 * ------------------------------------------------------------------------------------------ */
/* nn::LayerNorm::forward, rms (src/nn/layernorm/layernorm.cu:9-42): y = T(x*rsqrt(mean(x^2)+eps)*w/scale). */
int zl_rmsnorm(const void* x, const void* weight, void* y, int T, int D, float eps, float scale, int dtype,
               int pdl, zl_stream_t stream);
/* Residual + RMSNorm.  mode 0: block.cpp:124-131 order -- out_sum = T(a+b) (block_kernel.cu:7-17),
 * y = rmsnorm(out_sum);  mode 1: LayerNorm::fuse_add (layernorm.cu:28-41) -- y normalises the unrounded sum.
 * b may be NULL (then out_sum = a).  out_sum may alias a. */
int zl_add_rmsnorm(const void* a, const void* b, const void* weight, void* out_sum, void* y, int T, int D,
                   float eps, float scale, int mode, int dtype, int pdl, zl_stream_t stream);
/* nn::element_add_scale (src/nn/block/block_kernel.cu:7-17), scale_residual=false:
 * c = T(a + T(b*scale))  computed in T. */
int zl_element_add_scale(const void* a, const void* b, void* c, size_t n, float scale, int dtype,
                         zl_stream_t stream);
/* nn::gate_mul_inplace (src/nn/linear/activation_kernel.cu:55-106): out = T(act(float(gate))*float(up));
 * act 0 = silu, 1 = gelu.  gate/up (T, F) with row strides.  up == NULL: out = T(act(gate)), the activation
 * Linear::activate applies (src/nn/linear/linear.cpp activate(), activation_kernel.cu). */
int zl_gate_mul(const void* gate, int ld_gate, const void* up, int ld_up, void* out, int ld_out, int T, int F,
                int act, int dtype, zl_stream_t stream);

/* ------------------------------------------------------------------------------------------ *
 * RoPE + KV append
 * ------------------------------------------------------------------------------------------ */
/* RopePreparer (src/nn/position/rope_preparer.cu:49-161): cos/sin fp32 (T, d).
 * llama3_factor <= 0 -> plain rope. */
int zl_rope_cos_sin(const int32_t* pos, float* cos_out, float* sin_out, int T, int dim_head, float theta,
                    float llama3_factor, float low_freq_factor, float high_freq_factor, float old_context_len,
                    int neox, zl_stream_t stream);
/* nn::rope_qk_cache (src/nn/position/rotary_embedding_fuse_cache.cu:23-125): split fused qkv and rotate q,k. */
int zl_rope_qk_cache(const float* cos, const float* sin, const void* qkv, void* q, void* k, void* v, int T,
                     int num_heads, int num_kv_heads, int dim_head, int neox, int dtype, zl_stream_t stream);
/* nn copy_to_rag_buffer2 (src/kvcache/ragged_buffer_kernel.cu:194-300). */
int zl_copy_to_rag_buffer2(const int32_t* placement, const int32_t* buf_lens, const void* k_src,
                           const void* v_src, void* const* k_addrs, void* const* v_addrs, int B, int len_q,
                           int num_kv_heads, int dim_head, int bshd, int dtype, zl_stream_t stream);
/* Fused: split qkv (+bias already applied) + RoPE(q,k) + append K/V rows at placement into the per-task
 * buffers + write rotated q.  Replaces rope_qk_cache + copy_to_rag_buffer2 (attention.cpp:865-898, 636-676).
 * token_batch (T) int32: task index of each token; placement (T) int32 (<0: skip append). */
int zl_qkv_rope_append(const float* cos, const float* sin, const void* qkv, void* q_out,
                       const int32_t* token_batch, const int32_t* placement, void* const* k_addrs,
                       void* const* v_addrs, int T, int num_heads, int num_kv_heads, int dim_head, int neox,
                       int bshd, const int32_t* buf_lens, int dtype, int pdl, zl_stream_t stream);

/* ------------------------------------------------------------------------------------------ *
 * Decode attention over per-task ragged KV buffers
 * nn::multi_query_attention_rag_buffer (src/nn/attention/attention_kernel.cu:1252-1457)
 * ------------------------------------------------------------------------------------------ */
/* one-shot hint: the NEXT zl_decode_attention call on this thread also prefetches [ptr, ptr+bytes) into L2
 * (weights of a later GEMM; attention leaves HBM idle at small batch). */
int zl_decode_attention_set_prefetch(const void* ptr, size_t bytes);
size_t zl_decode_attention_workspace_bytes(int B, int len_q, int num_heads, int dim_head, int max_len_buf);
/* q (B, len_q, H_q, d); buf_lens (B); k_addrs/v_addrs (B) device arrays of device pointers;
 * mask int8 ragged concat of (len_q, len_buf_b); out (B, len_q, H_q, d).  bshd: (len_buf, H_kv, d) else
 * (H_kv, len_buf, d). */
int zl_decode_attention(const void* q, const int32_t* buf_lens, void* const* k_addrs, void* const* v_addrs,
                        const int8_t* mask, float scale, int max_len_buf, void* out, int B, int len_q,
                        int num_heads, int num_kv_heads, int dim_head, int bshd, void* workspace,
                        size_t workspace_bytes, int dtype, int pdl, zl_stream_t stream);

/* int8 KV cache (KV_CACHE_DTYPE=int8 of the reference): KERNEL_mqa_rag_buffer_split_kv_quant
 * (src/nn/attention/attention_kernel.cu:804-880, src/nn/attention/quant_attention.cuh:10-123).  K / V buffers per task are
 * (len_buf, H_kv, d) uint8 = round(x * 127 / absmax) + 128, scale buffers (len_buf, H_kv) fp32 = absmax / 127 (BSHD only,
 * like the reference); q is fp16; out in out_dtype.  Any max_len_buf (the reference only takes this path above
 * ATTN_SPLIT_KV_THRES = 1024).  workspace as zl_decode_attention_workspace_bytes. */
int zl_decode_attention_kv8(const void* q, const int32_t* buf_lens, void* const* k_addrs, void* const* v_addrs,
                            void* const* scale_k_addrs, void* const* scale_v_addrs, const int8_t* mask, float scale,
                            int max_len_buf, void* out, int B, int len_q, int num_heads, int num_kv_heads, int dim_head,
                            void* workspace, size_t workspace_bytes, int out_dtype, int pdl, zl_stream_t stream);
/* cache side of the same contract: int8_op::quant_calc_scale(x, 127, 128) per (token, kv head) row
 * (src/nn/quant/int8/quant_kernel.cu:15-47) + copy_to_rag_buffer2 of the codes and of the scales
 * (src/nn/attention/attention.cpp:656-676): k_src / v_src (T, H_kv, d), token t goes to row placement[t] of task
 * token_batch[t] (placement < 0: skipped). */
/* the same quantisation on dense rows: x (M, K) -> q (M, K) uint8, scale (M) fp32 (quant_calc_scale(x, 127, 128)). */
int zl_int8_quant_rows_u8(const void* x, void* q, float* scale, int M, int K, int dtype, zl_stream_t stream);
int zl_kv_int8_quant_append(const void* k_src, const void* v_src, const int32_t* token_batch, const int32_t* placement,
                            void* const* k_addrs, void* const* v_addrs, void* const* scale_k_addrs,
                            void* const* scale_v_addrs, int T, int num_kv_heads, int dim_head, int dtype, int pdl,
                            zl_stream_t stream);

/* ------------------------------------------------------------------------------------------ *
 * Decode-step helpers around the layers
 * ------------------------------------------------------------------------------------------ */
/* nn::Embedding lookup (src/nn/embedding/embedding.cu:20-60): out[t,:] = table[ids[t],:]. */
int zl_embedding(const int32_t* ids, const void* table, void* out, int T, int D, int vocab, int dtype, int pdl,
                 zl_stream_t stream);
/* greedy pick (generator/batch_generator.cpp:1762-1884 with beam 1): argmax over fp32 logits (T, V). */
size_t zl_argmax_workspace_bytes(int T);
int zl_argmax(const float* logits, int32_t* out, int T, int V, void* workspace, size_t workspace_bytes, int pdl,
              zl_stream_t stream);
/* vocab-parallel pick: per-token {float value, int global index} candidate of one logits shard (T, V), and the
 * merge over the all-gathered candidates [ranks][stride] (embedding.cu:353-392 gathers the logits instead). */
int zl_argmax_candidates(const float* logits, void* cand_out, int T, int V, int idx_offset, void* workspace,
                         size_t workspace_bytes, int pdl, zl_stream_t stream);
int zl_argmax_merge(const void* cand_all, int32_t* out, int T, int ranks, int stride, int pdl, zl_stream_t stream);
/* synthetic-checkpoint generators (bench / tests): counter-based hash RNG, reproducible per seed. */
int zl_fill_random_u32(uint32_t* p, size_t n, uint64_t seed, zl_stream_t stream);
int zl_fill_const_u32(uint32_t* p, size_t n, uint32_t value, zl_stream_t stream);
int zl_fill_uniform(void* p, size_t n, float lo, float hi, uint64_t seed, int dtype, zl_stream_t stream);

/* ------------------------------------------------------------------------------------------ *
 * Tensor-parallel exchange over NVLink peer memory (one process per GPU, one node)
 * Replaces ModelContext::reduce_sum / reduce_sum2 / reduce_tp_int8 (src/model/model_context.cpp:203-326) and
 * the c10d NCCL wrappers it calls (3rd/bmengine/bmengine/c10d/c10d.cpp:42-136) on the decode path.
 * ------------------------------------------------------------------------------------------ */
/* Allocates this rank's symmetric buffer (inboxes for world_size sources x 2 parities of max_elems 16-bit values). */
int zl_comm_create(int rank, int world_size, size_t max_elems_16bit, zl_comm_t** out);
void zl_comm_destroy(zl_comm_t* c);
int zl_comm_rank(zl_comm_t* c);
int zl_comm_world_size(zl_comm_t* c);
/* CUDA IPC handle of the symmetric buffer (zl_comm_ipc_handle_bytes() bytes); exchange them out of band
 * (torch.distributed all_gather in zhilight_b200/dist.py) and hand all of them (index = rank) to open_peers. */
int zl_comm_ipc_handle_bytes(void);
int zl_comm_get_ipc_handle(zl_comm_t* c, void* handle_out);
int zl_comm_open_peers(zl_comm_t* c, const void* handles_all);
/* once per decode step that uses the exchange fused into the W4 GEMMs (tp_mode of zl_w4a16_gemm_fused), before the first
 * such GEMM of the step and on every rank: advances the step counter the word tags are derived from. */
int zl_comm_ll_begin_step(zl_comm_t* c, zl_stream_t stream);
/* out = T(T(sum over ranks of partial) + residual); n % 32 == 0; residual may be NULL; out may alias residual.
 * int8_payload != 0: peers' contributions travel as int8 + one T scale per 32 values (the reference's group-32
 * format, int8/quant_reduce_kernel.cu:14-38); deterministic rank-ordered fp32 reduction either way. */
int zl_allreduce_one_shot(zl_comm_t* c, const void* partial, const void* residual, void* out, size_t n, int dtype,
                          int int8_payload, int pdl, zl_stream_t stream);
/* out[r*bytes ..] = `in` of rank r (bytes % 16 == 0, small: one CTA). */
int zl_allgather_small(zl_comm_t* c, const void* in, void* out, size_t bytes, int pdl, zl_stream_t stream);
/* int8_op::quant_group_32 / dequant_sum_quant_g32 / dequant_group_32 / dequant_group_fuse_add
 * (src/nn/quant/int8/quant_reduce_kernel.cu:14-38, 243-322, 105-140, 201-240); M = number of 32-groups. */
int zl_quant_group_32(const void* in, int8_t* out_q, void* out_scale, size_t M, int dtype, zl_stream_t stream);
int zl_dequant_sum_quant_g32(const void* my, const int8_t* q_others, const void* scale_others, int8_t* out_q,
                             void* out_scale, size_t M, int world_size, int dtype, zl_stream_t stream);
/* add != NULL: dequant_group_fuse_add (out = q*s + add). */
int zl_dequant_group_32(const int8_t* q, const void* scale, const void* add, void* out, size_t M, int dtype,
                        zl_stream_t stream);

/* ------------------------------------------------------------------------------------------ *
 * Decode driver: the model::LLaMA::encode + get_logits + greedy pick stand-in
 * (src/model/llama.cpp:75-165, src/nn/block/block.cpp:86-143, src/nn/attention/attention.cpp:846-964,
 *  src/nn/feedforward/feedforward.cpp:113-137) for len_q = 1 dynamic-batch steps.  The reference keeps
 * its scheduler (src/generator) above this; here the caller supplies (token, position) per task.
 * One CUDA graph per batch size, all kernels chained with programmatic dependent launch.
 * ------------------------------------------------------------------------------------------ */
typedef struct zl_llama zl_llama_t;
typedef struct zl_llama_config {
    int num_layers, dim_model, num_heads, num_kv_heads, dim_head, dim_ff, vocab_size;
    float eps, rope_theta;
    float rope_llama3_factor; /* <= 0: plain rope */
    float rope_low_freq_factor, rope_high_freq_factor, rope_orig_ctx;
    int quant_type; /* model_config.hpp:132-144 QuantType: 0 none, 2 AutoInt8 (fp weights quantised per row at load),
                     * 5 GPTQ, 6 AWQ, 7 FP8 (e4m3 weights + per-tensor weight_scale), 8 GPTQ_Marlin (= 5 with sym) */
    int group_size, sym;
    int dtype; /* ZL_F16 / ZL_BF16 (W4 paths are fp16-only like the reference, q_gemm_k_major.cu:989) */
    int max_batch, max_seq;
    int tp_rank, tp_size;
    int use_pdl, use_graph;
    int tp_int8; /* TP all-reduce payload: 0 = activation dtype, 1 = int8 group-32 (REDUCE_TP_INT8 of the reference) */
    int fuse; /* 0: one kernel per reference operator; 1: RMSNorm folded into the W4 GEMMs; 2 (3 is accepted as 2):
               * + qkv RoPE/KV-append epilogue.  Launches with more than 16 tokens run zl_rmsnorm + the tcgen05 GEMM. */
    int prefill_chunk; /* 0: decode only.  1..2048: zl_llama_prefill processes a prompt in chunks of this many tokens
                        * (chunked prefill, zhilight/config/adapter.py:47-48) */
    int qkv_bias; /* zl_llama_init_synthetic: also create q/k/v biases (Qwen2: attention.cpp:105-109); loaded checkpoints
                   * carry their ".bias" tensors regardless of this flag */
} zl_llama_config_t;

int zl_llama_create(const zl_llama_config_t* cfg, zl_llama_t** out);
/* tensor parallel: hand the driver its exchange object (zl_comm_create + open_peers) before the first step. */
int zl_llama_set_comm(zl_llama_t* m, zl_comm_t* comm);
void zl_llama_destroy(zl_llama_t* m);
/* Stage one checkpoint tensor (HOST pointer, row-major (rows, cols)); names as produced by
 * zhilight/loader.py:250-358 without the "llama." prefix, e.g. "layers.0.attn.project_q.qweight". */
int zl_llama_load_tensor(zl_llama_t* m, const char* name, const void* data_host, int rows, int cols,
                         int elem_bytes);
/* Fill every tensor of the configured architecture with reproducible random data ON DEVICE
 * (HF-GPTQ layout for quantized linears) and run the load pipeline layer by layer. */
int zl_llama_init_synthetic(zl_llama_t* m, uint64_t seed);
/* Run the load pipeline (Int4GPTQ::preprocess_weight + fusion + ZLW4 pack) on the staged tensors. */
int zl_llama_finalize(zl_llama_t* m);
/* One decode step for B tasks.  tokens_host/positions_host (B) int32; task b owns KV slot b.
 * next_tokens_host (B) int32 greedy picks; logits_host NULL or (B, vocab) fp32.  Synchronous. */
int zl_llama_decode(zl_llama_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B,
                    int32_t* next_tokens_host, float* logits_host);
/* Device-resident variant: stage tokens/positions once, then each call replays the step, feeds the picked
 * tokens back and advances positions on the device; no host sync. */
int zl_llama_set_state(zl_llama_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B);
int zl_llama_step_device(zl_llama_t* m, int B);
/* read back the device-resident (token, position) state; synchronous. */
int zl_llama_get_state(zl_llama_t* m, int32_t* tokens_host, int32_t* positions_host, int B);
int zl_llama_sync(zl_llama_t* m);
/* Chunked prefill of ONE task (SearchTask prompt, src/generator/batch_generator.cpp:1576): appends tokens_host[0..n) at
 * positions pos0.. to the task's KV buffers through the same kernels (M = chunk GEMMs, causal len_q = chunk attention)
 * and returns the greedy next token (and optionally the last position's logits, vocab/tp floats).  Synchronous. */
/* Prefill keeps its own token / position staging on the device: the (token, position) state of the decode tasks set by
 * zl_llama_set_state survives a prefill issued between two zl_llama_step_device calls (continuous batching).  It
 * overwrites the next-token / logits row 0 outputs, which zl_llama_step_device consumes before it returns. */
int zl_llama_prefill(zl_llama_t* m, int task, const int32_t* tokens_host, int n, int pos0, int32_t* next_token_host,
                     float* logits_host);
zl_stream_t zl_llama_stream(zl_llama_t* m);
/* bytes the step must read from HBM per rank (weights + lm_head + norms), kernel launches per step. */
int zl_llama_stats(zl_llama_t* m, int B, double* weight_bytes, int* kernels_per_step);
/* Roofline probe for the dominant kernel: enqueue only the W4A16 (or dense) GEMMs of one decode step
 * (every layer's own weights, same PDL chain) `iters` times between CUDA events on the driver's stream.
 * Returns total milliseconds, the number of GEMM launches and their algorithmic bytes. */
int zl_llama_bench_gemms(zl_llama_t* m, int B, int iters, float* ms, int* launches, double* bytes);

/* ------------------------------------------------------------------------------------------ *
 * Building blocks of layers with an fp32 residual stream, grouped norms, short convolutions and latent attention
 * ------------------------------------------------------------------------------------------ */
enum {
    ZL_GEMM_EPI_NONE = 0,
    ZL_GEMM_EPI_RELU2 = 1 /* max(v,0)^2 */,
    ZL_GEMM_EPI_SIGMOID_GATE = 2 /* v * sigmoid(gate) */,
    ZL_GEMM_EPI_TANH = 3,
    ZL_GEMM_EPI_GLU_CLAMP = 4 /* columns 2j, 2j+1 = gate, up -> column j: g = min(gate, limit), u = clamp(up, +-limit),
                                 g * sigmoid(alpha * g) * (u + beta); grouped call only */,
    ZL_GEMM_EPI_GEGLU_TANH = 5 /* columns 2j, 2j+1 = gate, up -> column j: gelu_tanh(gate) * up, with
                                  gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) */,
    ZL_GEMM_EPI_GELU_TANH_MUL = 6 /* gelu_tanh(v) * mul[m][n] */,
    ZL_GEMM_EPI_SOFTCAP = 7 /* limit * tanh(v / limit) */
};
/* y[b](M,N) = epi(x[b](M,K) @ w[b](N,K)^T), b < batch, element strides per batch entry; any M, N, K.  in_dtype
 * ZL_F16 / ZL_BF16 (tensor cores, fp32 accumulation) or ZL_F32 (plain fp32 FMAs, no reduced-precision mode);
 * out_dtype = in_dtype or ZL_F32; gate (fp32, same indexing as y with ldg / gate_batch_stride) for the gate epilogue. */
int zl_gemm_nt(const void* x, long long ldx, long long x_batch_stride, const void* w, long long ldw,
               long long w_batch_stride, void* y, long long ldy, long long y_batch_stride, int M, int N, int K, int batch,
               int in_dtype, int out_dtype, int epilogue, const float* gate, long long ldg, long long gate_batch_stride,
               int pdl, zl_stream_t stream);
/* One problem with a per-column fp32 bias (NULL: none) added before the epilogue (none, relu^2 or tanh). */
int zl_gemm_nt_bias(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y, long long ldy,
                    int M, int N, int K, int in_dtype, int out_dtype, int epilogue, int pdl, zl_stream_t stream);
/* One problem with a per-column fp32 bias (NULL: none) and any epilogue but the clamped unit: none, relu^2, tanh, sigmoid
 * gate / gelu_tanh times multiplier (mul fp32 (M, N), row stride ld_mul), gelu_tanh(gate) * up over column pairs (the
 * bias has N entries, y has N / 2 columns), soft cap at `limit`. */
int zl_gemm_nt_fused(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y, long long ldy,
                     int M, int N, int K, int in_dtype, int out_dtype, int epilogue, const float* mul, long long ld_mul,
                     float limit, int pdl, zl_stream_t stream);
/* Grouped problems for mixtures of experts.  A list of rows sorted by group: group g owns the list entries
 * group_offsets[g] .. group_offsets[g+1] (device, groups + 1 ints) and the weight block w + g * w_group_stride (N, K).
 * List entry i reads row x_rows[i] of x (NULL: row i) and writes row y_rows[i] of y (NULL: row i).  max_rows bounds the
 * rows of any group (the step's row count); the offsets are read on the device, so the call can be captured in a graph.
 * Epilogue none, relu^2, or the clamped gated unit over column pairs (y has N / 2 columns). */
int zl_gemm_nt_grouped(const void* x, long long ldx, const int32_t* x_rows, const void* w, long long ldw,
                       long long w_group_stride, void* y, long long ldy, const int32_t* y_rows, const int32_t* group_offsets,
                       int groups, int max_rows, int N, int K, int in_dtype, int out_dtype, int epilogue, float limit,
                       float alpha, float beta, int pdl, zl_stream_t stream);
/* One problem with the clamped gated unit over column pairs and a per-column fp32 bias (NULL: none; 2 entries per output
 * column, added before the unit): y (M, N / 2) = g sigmoid(alpha g) (u + beta), g = min(gate, limit), u = clamp(up, +-limit). */
int zl_gemm_nt_glu_clamp(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y, long long ldy,
                         int M, int N, int K, int in_dtype, int out_dtype, float limit, float alpha, float beta, int pdl,
                         zl_stream_t stream);
/* y[t] = w * x[t] / sqrt(mean(x[t]^2 over each of `groups` equal consecutive parts) + eps); x fp32, y out_dtype. */
int zl_group_rmsnorm(const float* x, long long ldx, const float* weight, void* y, long long ldy, int T, int D, int groups,
                     float eps, int out_dtype, int pdl, zl_stream_t stream);
/* x[t] += the same norm of y[t] (fp32).  With ring != NULL also stores conv_in[t] into the convolution ring
 * ring[slot[t]][pos[t] % (taps-1)][D] for the rows that are among the last taps-1 of their sequence in this step. */
int zl_group_rmsnorm_residual(const float* y, long long ldy, const float* weight, float* x, long long ldx, int T, int D,
                              int groups, float eps, const float* conv_in, long long ld_conv_in, const int32_t* slot,
                              const int32_t* pos, float* ring, int taps, int pdl, zl_stream_t stream);
/* u[t] = h[t] + sum_j taps_weight[c][j] * h(pos[t] - taps + 1 + j): per-channel causal convolution over the positions of
 * a sequence; earlier inputs come from this step's rows (rows of a sequence are consecutive) or from the slot's ring,
 * zeros before position 0.  taps_weight fp32 (D, taps). */
int zl_causal_conv_mix(const float* h, long long ldh, const float* taps_weight, const int32_t* slot, const int32_t* pos,
                       const float* ring, void* u, long long ldu, int T, int D, int taps, int out_dtype, int pdl,
                       zl_stream_t stream);
/* zl_group_rmsnorm (-> h, fp32, kept for the ring update) and zl_causal_conv_mix (-> u) in one kernel. */
int zl_group_norm_conv(const float* x, long long ldx, const float* norm_weight, const float* taps_weight, const int32_t* slot,
                       const int32_t* pos, const float* ring, float* h, void* u, int T, int D, int groups, int taps, float eps,
                       int out_dtype, int pdl, zl_stream_t stream);
/* plain RMS norms of the two low-rank latents inside a fused projection row: proj[t][q_off .. +q_rank) -> cq (T, q_rank)
 * and, when kv_weight != NULL, proj[t][c_off .. +kv_rank) -> row pos[t] of the latent cache of slot[t]. */
int zl_latent_norm_append(const float* proj, long long ldp, int q_off, int q_rank, const float* q_weight, void* cq, int c_off,
                          int kv_rank, const float* kv_weight, void* const* slot_addrs, const int32_t* slot,
                          const int32_t* pos, int T, float eps, int dtype, int pdl, zl_stream_t stream);
/* Absorbed attention over cached latents with a softmax sink.  q_absorbed (T, heads, kv_rank) fp32 = W_uk,h^T q_h;
 * token t sees rows 0..pos[t] of slot_addrs[slot[t]] ((max_seq, kv_rank) of `dtype`); out (T, heads, kv_rank) of `dtype`
 * = sum_j softmax_with_sink(scale * q_absorbed . c_j) c_j; the denominator holds exp(sink[h]) once.  splits > 1 cuts
 * every token's keys over that many CTAs (workspace of zl_latent_attention_workspace_bytes). */
size_t zl_latent_attention_workspace_bytes(int T, int heads, int kv_rank, int splits);
int zl_latent_attention_prepare(int heads, int kv_rank, int dtype);
int zl_latent_attention_splits(int T, int heads, int kv_rank, int max_len);
int zl_latent_attention(const float* q_absorbed, void* const* slot_addrs, const int32_t* slot, const int32_t* pos,
                        const float* sink, float scale, void* out, int T, int heads, int kv_rank, int splits, void* workspace,
                        size_t workspace_bytes, int dtype, int pdl, zl_stream_t stream);

/* ------------------------------------------------------------------------------------------ *
 * Dekipel: decoder-only model of latent-attention layers (queries and key-values through low-rank latents, no
 * positional rotation, causal softmax with a per-head sink, sigmoid output gate, optional sharing of another layer's
 * latent cache), each sublayer between a pre- and a post-norm (RMS norm in groups), reading its input through a short
 * causal convolution, with a relu^2 feed-forward.  Same driver shape as zl_llama_*: task slots with per-slot caches,
 * host (token, slot, position) in, logits / greedy picks out.
 * ------------------------------------------------------------------------------------------ */
typedef struct zl_dekipel zl_dekipel_t;
typedef struct zl_dekipel_layer {
    int heads, dim, vdim, q_rank, kv_rank;
    int kv_from; /* -1: own key-value latents; j: reads layer j's latent cache */
    int ff;      /* 0: no feed-forward sublayer */
    float scale;
} zl_dekipel_layer_t;
typedef struct zl_dekipel_config {
    int num_layers, width, vocab;
    int norm_groups, canon_taps;
    float eps;
    int dtype; /* ZL_BF16: 16-bit Linears with fp32 accumulation; ZL_F32: everything in fp32 */
    int max_batch /* slots */, max_seq /* rows per slot */, max_step_tokens /* tokens per step */;
    int use_pdl, use_graph;
} zl_dekipel_config_t;

int zl_dekipel_create(const zl_dekipel_config_t* cfg, const zl_dekipel_layer_t* layers, zl_dekipel_t** out);
void zl_dekipel_destroy(zl_dekipel_t* m);
/* Stage one checkpoint tensor (HOST pointer, row-major (rows, cols); elem_bytes 2 = bfloat16, 4 = float32 / int32). */
int zl_dekipel_load_tensor(zl_dekipel_t* m, const char* name, const void* data_host, int rows, int cols, int elem_bytes);
int zl_dekipel_init_synthetic(zl_dekipel_t* m, uint64_t seed);
int zl_dekipel_finalize(zl_dekipel_t* m);
/* One step over T tokens: token t belongs to slot slots[t] at position positions[t]; the rows of one slot are consecutive
 * with consecutive positions (a prompt portion), or every row is another slot (a decode batch), or any mix.  Appends to
 * the slots' caches and states.  want_rows (n_want indices into the step's rows): their logits go to logits_host
 * (n_want, vocab) fp32 and their greedy picks to next_host (n_want); either may be NULL.  Synchronous. */
int zl_dekipel_step(zl_dekipel_t* m, const int32_t* tokens_host, const int32_t* slots_host, const int32_t* positions_host,
                    int T, const int32_t* want_rows_host, int n_want, float* logits_host, int32_t* next_host);
/* Device-resident decode loop (bench): set the (token, position) of slots 0..B-1 once, then every call runs one step,
 * feeds the greedy picks back and advances the positions on the device; no host sync. */
int zl_dekipel_set_state(zl_dekipel_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B);
int zl_dekipel_step_device(zl_dekipel_t* m, int B);
int zl_dekipel_sync(zl_dekipel_t* m);
zl_stream_t zl_dekipel_stream(zl_dekipel_t* m);
/* residual stream after every layer of the last step, (num_layers, T, width) fp32, when capture was switched on */
int zl_dekipel_capture_layers(zl_dekipel_t* m, int on);
int zl_dekipel_read_layers(zl_dekipel_t* m, float* out_host, int T);
int zl_dekipel_stats(zl_dekipel_t* m, double* weight_bytes, int* kernels_per_step);

/* ------------------------------------------------------------------------------------------ *
 * Building blocks of layers with per-head norms, rotated and cached keys, recurrent state and routed experts
 * ------------------------------------------------------------------------------------------ */
/* Rotation frequencies f_i = base^(-2i/dims), i < dims/2, with YaRN scaling when factor > 0: with
 * dim(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dims-1) and
 * ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is f_i / factor * ramp_i + f_i (1 - ramp_i), and
 * cos / sin are scaled by mscale = 0.1 ln(factor) + 1 (1 without scaling).  Host function; out (dims/2) doubles. */
int zl_rope_inv_freq_yarn(double base, int dims, double factor, double original, double fast, double slow, double* out,
                          float* mscale);
/* From a fused projection row proj[t] (fp32) to attention operands: per query head RMS norm over `dim` times q_weight
 * (dim), rotation of the first rot_dims dimensions in adjacent pairs (2i, 2i+1) by pos[t] * inv_freq[i] (cos, sin times
 * mscale), -> q_out (T, heads * dim) of `dtype`; when k_off >= 0 the same for the key heads (k_weight) -> row pos[t] of
 * k_addrs[slot[t]] ((max_seq, kv_heads, dim)), and every value head divided by its RMS over `vdim` -> row pos[t] of
 * v_addrs[slot[t]] ((max_seq, kv_heads, vdim)). */
int zl_qkv_headnorm_rope_append(const float* proj, long long ldp, int q_off, int k_off, int v_off, int heads, int kv_heads,
                                int dim, int vdim, const float* q_weight, const float* k_weight, const double* inv_freq,
                                int rot_dims, float mscale, float eps, void* q_out, void* const* k_addrs,
                                void* const* v_addrs, const int32_t* slot, const int32_t* pos, int T, int dtype, int pdl,
                                zl_stream_t stream);
/* Causal attention over the slots' caches: query head h uses key/value head h / (heads / kv_heads);
 * p_j = exp(s_j) / (exp(sink_h) + sum_i exp(s_i)) with s = scale * q . k (sink NULL: every sink is 0, the
 * extra term is then exactly 1); out (T, heads * vdim) of `dtype`, head h times sigmoid(gate[t * ldg + h]) when gate != NULL.
 * splits > 1 cuts the keys of every token over that many CTAs (decode with long contexts); workspace of
 * zl_sink_attention_workspace_bytes.  With the runs of the step (run i = rows run_row0[i] .. + run_len[i]: one slot,
 * consecutive positions; max_run_len bounds run_len) 16-bit caches go through the tensor-core kernel, which tiles
 * the tokens of a run; run_row0 NULL: the general kernel, one CTA per (token, head). */
size_t zl_sink_attention_workspace_bytes(int T, int heads, int vdim, int splits);
int zl_sink_attention_splits(int T, int heads, int kv_heads, int max_len);
int zl_sink_attention(const void* q, void* const* k_addrs, void* const* v_addrs, const int32_t* slot, const int32_t* pos,
                      const float* sink, const float* gate, long long ldg, float scale, void* out, int T, int heads,
                      int kv_heads, int dim, int vdim, int splits, void* workspace, size_t workspace_bytes,
                      const int32_t* run_row0, const int32_t* run_len, int runs, int max_run_len, int dtype, int pdl,
                      zl_stream_t stream);
/* The same with two restrictions a design may add.  chunk > 0: token t sees only the keys from (pos[t] / chunk) * chunk
 * on (blocks of `chunk` positions counted from position 0 of the sequence).  dist_bias != NULL (device, fp32
 * (heads, n_dist)): dist_bias[h][min(pos[t] - j, n_dist - 1)] is added to the scaled score of key j; the sink gets none.
 * max_len passed to zl_sink_attention_splits may be the chunk size when chunk > 0. */
int zl_sink_attention_local(const void* q, void* const* k_addrs, void* const* v_addrs, const int32_t* slot,
                            const int32_t* pos, const float* sink, const float* gate, long long ldg, float scale, int chunk,
                            const float* dist_bias, int n_dist, void* out, int T, int heads, int kv_heads, int dim, int vdim,
                            int splits, void* workspace, size_t workspace_bytes, const int32_t* run_row0,
                            const int32_t* run_len, int runs, int max_run_len, int dtype, int pdl, zl_stream_t stream);
/* Host helper: a learned table (rows, heads) indexed by a bucket of the distance n -> out_host (heads, n_dist), entry
 * [h][n] = table[bucket(n)][h] with bucket(n) = n below half = rows / 2 and
 * min(rows - 1, half + floor(ln(n / half) / ln(far / half) * (rows - half))) from there on (evaluated in double). */
int zl_distance_bias_table(const float* table_host, int rows, int heads, double far, int n_dist, float* out_host);
/* y[t][h] = o[t][h] / sqrt(mean(o[t][h]^2 over vdim) + eps) * weight[h * vdim + c] * sigmoid(gate[t * ldg + h * vdim + c]);
 * weight and gate may be NULL. */
int zl_head_rmsnorm_gate(const float* o, long long ldo, const float* weight, const float* gate, long long ldg, void* y,
                         long long ldy, int T, int heads, int vdim, float eps, int out_dtype, int pdl, zl_stream_t stream);
/* The same with the weight's stride between heads given (0: one weight of vdim shared by the heads) and the gate's
 * function chosen: sigmoid(g) or silu(g) = g sigmoid(g). */
enum { ZL_GATE_SIGMOID = 0, ZL_GATE_SILU = 1 };
int zl_head_rmsnorm_gate_fn(const float* o, long long ldo, const float* weight, int weight_head_stride, const float* gate,
                            long long ldg, int gate_fn, void* y, long long ldy, int T, int heads, int vdim, float eps,
                            int out_dtype, int pdl, zl_stream_t stream);
/* Queries and keys normed over the whole projection: from a projection row proj[t] (fp32), q = proj[q_off .. + heads * dim)
 * divided by its RMS over all heads * dim entries, times q_weight (heads * dim) -> q_out (T, heads * dim) of `dtype`; the
 * same for k = proj[k_off .. + kv_heads * dim) with k_weight -> row pos[t] of k_addrs[slot[t]]; the projected k itself
 * (no norm) -> row pos[t] of v_addrs[slot[t]]: the values are the keys. */
int zl_qk_fullnorm_append(const float* proj, long long ldp, int q_off, int k_off, int heads, int kv_heads, int dim,
                          const float* q_weight, const float* k_weight, float eps, void* q_out, void* const* k_addrs,
                          void* const* v_addrs, const int32_t* slot, const int32_t* pos, int T, int dtype, int pdl,
                          zl_stream_t stream);
/* Mixes of a token with its predecessor: out[s] (T, D) of out_dtype at out + s * out_stride elements,
 * out[s][t] = x[t] + (prev - x[t]) * mu[s], mu fp32 (n_mix, D); prev = x[t - 1] when row t - 1 is of the same slot,
 * zeros at position 0, else state_addrs[slot[t]] ((D) fp32, the slot's last token).  store_state != 0 (only when no two
 * rows share a slot): x[t] also becomes the slot's last token; otherwise call zl_store_run_tails(x, ...) afterwards. */
int zl_token_shift_mix(const float* x, long long ldx, const float* mu, int n_mix, void* const* state_addrs,
                       const int32_t* slot, const int32_t* pos, void* out, long long out_stride, int T, int D,
                       int store_state, int out_dtype, int pdl, zl_stream_t stream);
/* Norm after the sum: x[t] <- weight * s / sqrt(mean(s^2) + eps), s = alpha x[t] + coef_a a[t] + coef_b b[t] (b NULL: no
 * third term); x fp32; x_act != NULL also receives the new x[t] rounded to act_dtype. */
int zl_postnorm_combine(float* x, long long ldx, float alpha, const float* a, long long lda, float coef_a, const float* b,
                        long long ldb, float coef_b, const float* weight, void* x_act, int act_dtype, int T, int D, float eps,
                        int pdl, zl_stream_t stream);
/* x[t] += weight * s / sqrt(mean(s^2) + eps), s = sum_p coef[t * n_parts + p] * parts[(t * n_parts + p) * ldp ..] (coef
 * NULL: ones); x fp32.  x_act != NULL also receives the new x[t] rounded to act_dtype (the next Linear's input). */
int zl_rmsnorm_residual_combine(const float* parts, long long ldp, const float* coef, int n_parts, const float* weight,
                                float* x, long long ldx, void* x_act, int act_dtype, int T, int D, float eps, int pdl,
                                zl_stream_t stream);
/* Generalized delta rule over the runs of a step (run i = rows run_row0[i] .. + run_len[i], one slot, consecutive
 * positions): per head a (dim_k, dim_v) fp32 state S in state_addrs[slot] ((heads, dim_k, dim_v)), zero at position 0,
 * S <- diag(w) S - (a * u)(u^T S) + k v^T, o = S^T r, with u = k / sqrt(sum(k^2) + unit_eps),
 * w = exp(-decay_scale * sigmoid(decay_logit)), a = sigmoid(rate_logit).  All inputs fp32 (T, heads * dim); T rows in
 * the step; workspace of zl_delta_rule_workspace_bytes. */
int zl_delta_rule_prepare(int dim_k, int dim_v);
size_t zl_delta_rule_workspace_bytes(int T, int heads, int dim_k, int dim_v);
int zl_delta_rule(const float* r, long long ld_r, const float* k, long long ld_k, const float* v, long long ld_v,
                  const float* rate_logit, long long ld_a, const float* decay_logit, long long ld_w, float decay_scale,
                  float unit_eps, const int32_t* run_row0, const int32_t* run_len, int runs, const int32_t* slot,
                  const int32_t* pos, void* const* state_addrs, float* o, long long ld_o, int heads, int dim_k, int dim_v,
                  int T, void* workspace, size_t workspace_bytes, int pdl, zl_stream_t stream);
/* The last n_tail rows of every run of src (T, ld) fp32, columns col .. col + channels, into per-slot rings
 * ring_addrs[slot] ((n_tail, channels) fp32): the row at position p goes to entry p % n_tail. */
int zl_store_run_tails(const float* src, long long ld, int col, int channels, int n_tail, const int32_t* run_row0,
                       const int32_t* run_len, int runs, const int32_t* slot, const int32_t* pos, void* const* ring_addrs,
                       int pdl, zl_stream_t stream);
/* Gated delta rule over the runs of a step, per head a (dim_k, dim_v) fp32 state in state_addrs[slot] (zero at position
 * 0):  S <- g S;  e = beta (v - S^T k);  S <- S + k e^T;  o = S^T q.  proj (T, ld) fp32 holds, from column col_qkv, the
 * projections q | k (kv_heads * dim_k each; head h uses q / k head h / (heads / kv_heads)) | v (heads * dim_v), at col_rate
 * the logits of beta = sigmoid(.) (heads) and at col_decay the inputs of g = exp(-exp(a_log[h]) softplus(. + dt_bias[h])).
 * q | k | v first pass a causal convolution per channel (conv_weight fp32 (channels, taps), last tap = the current token,
 * zeros before position 0; the last taps - 1 inputs of a sequence live in ring_addrs[slot] ((taps - 1, channels) fp32, position
 * p in entry p % (taps - 1)) and are updated by this call) and silu; then q, k <- x / sqrt(sum(x^2) + unit_eps) per head
 * and q times q_scale.  Workspace of zl_delta_rule_workspace_bytes. */
int zl_gated_delta_rule(const float* proj, long long ld, int col_qkv, int col_rate, int col_decay, const float* conv_weight,
                        int taps, const float* a_log, const float* dt_bias, float unit_eps, float q_scale,
                        void* const* ring_addrs, const int32_t* run_row0, const int32_t* run_len, int runs, const int32_t* slot,
                        const int32_t* pos, void* const* state_addrs, float* o, long long ld_o, int heads, int kv_heads,
                        int dim_k, int dim_v, int T, void* workspace, size_t workspace_bytes, int pdl, zl_stream_t stream);
/* Decaying state with a bonus for the current token, same state layout:  o_t = (S + diag(bonus[h]) k_t v_t^T)^T r_t, then
 * S <- diag(w_t) S + k_t v_t^T with w_t = exp(-exp(decay_logit_t)) per head and key channel.  Inputs fp32 (T, heads * dim),
 * bonus fp32 (heads, dim_k).  Workspace of zl_delta_rule_workspace_bytes. */
int zl_bonus_decay_scan(const float* r, long long ld_r, const float* k, long long ld_k, const float* v, long long ld_v,
                        const float* decay_logit, long long ld_w, const float* bonus, const int32_t* run_row0,
                        const int32_t* run_len, int runs, const int32_t* slot, const int32_t* pos, void* const* state_addrs,
                        float* o, long long ld_o, int heads, int dim_k, int dim_v, int T, void* workspace,
                        size_t workspace_bytes, int pdl, zl_stream_t stream);
/* Routing of a mixture of experts: logits W_router x[t] (fp32), scores (sigmoid, or softmax over the experts), the
 * `top` largest of score + correction (NULL: none), weights = their scores (renormalize: divided by their sum) ->
 * top_experts / top_weights (T, top); and the (token, choice) pairs sorted by expert for zl_gemm_nt_grouped:
 * group_offsets (experts + 1), list_token / list_pair (T * top). */
enum { ZL_MOE_SCORE_SIGMOID = 0, ZL_MOE_SCORE_SOFTMAX = 1 };
int zl_moe_route(const float* x, long long ldx, const float* w_router, const float* correction, int32_t* top_experts,
                 float* top_weights, int32_t* group_offsets, int32_t* list_token, int32_t* list_pair, int T, int D,
                 int experts, int top, int score_fn, int renormalize, int pdl, zl_stream_t stream);

/* The same from the router's input x (w_router != NULL) or from ready logits (w_router NULL: x is (T, slots) fp32 with row
 * stride ldx), with restricted choice: the `slots` router outputs form `groups` equal groups of neighbours, a group ranks
 * by its largest score + correction, and only slots of the `keep` best groups can be chosen (ties: the lower index).  The
 * weights are the chosen scores, divided by (their sum + renorm_eps) when renormalize != 0.  Slots from `experts` on have
 * no weights (a caller's identity slots): the lists are sorted over all `slots` groups, group_offsets has slots + 1
 * entries, and a grouped GEMM over the first `experts` groups skips them. */
int zl_moe_route_grouped(const float* x, long long ldx, const float* w_router, const float* correction, int32_t* top_experts,
                         float* top_weights, int32_t* group_offsets, int32_t* list_token, int32_t* list_pair, int T, int D,
                         int slots, int top, int groups, int keep, int score_fn, int renormalize, float renorm_eps, int pdl,
                         zl_stream_t stream);
/* cos / sin of pos[t] * inv_freq[i] (double angles, evaluated in double) -> table (T, half) of float pairs (cos, sin). */
int zl_rope_table(const int32_t* pos, int T, const double* inv_freq, int half, float* table, int pdl, zl_stream_t stream);
enum { ZL_ROT_HALVES = 0 /* pair (i, i + n / 2) */, ZL_ROT_ADJACENT = 1 /* pair (2i, 2i + 1) */ };
/* From a fused projection row proj[t] (fp32) to attention operands with tables of zl_rope_table: the first rot_dims
 * dimensions of every query head turn by qk_table[t] (rot_dims / 2 pairs in `layout`) -> q_out (T, heads * dim) of `dtype`;
 * when k_off >= 0 the same for the key heads -> row pos[t] of k_addrs[slot[t]], and every value head -> row pos[t] of
 * v_addrs[slot[t]], turned over all vdim dimensions by v_table[t] (vdim / 2 pairs) when v_table != NULL. */
int zl_qkv_table_rope_append(const float* proj, long long ldp, int q_off, int k_off, int v_off, int heads, int kv_heads, int dim,
                       int vdim, const float* qk_table, int rot_dims, const float* v_table, int layout, void* q_out,
                       void* const* k_addrs, void* const* v_addrs, const int32_t* slot, const int32_t* pos, int T, int dtype,
                       int pdl, zl_stream_t stream);
/* zl_sink_attention_local with two more options.  no_sink != 0: an ordinary softmax (no extra term in the denominator;
 * `sink` is ignored).  out_table != NULL (a table of zl_rope_table, (T, vdim / 2)): every head's output at token t is
 * turned back by the table's angles (pair (u, v) -> (u cos + v sin, v cos - u sin), pairs over vdim in out_layout) in
 * fp32 before it is stored: the inverse of a rotation the cached values carry. */
int zl_sink_attention_ex(const void* q, void* const* k_addrs, void* const* v_addrs, const int32_t* slot, const int32_t* pos,
                         const float* sink, int no_sink, const float* gate, long long ldg, float scale, int chunk,
                         const float* dist_bias, int n_dist, const float* out_table, int out_layout, void* out, int T, int heads,
                         int kv_heads, int dim, int vdim, int splits, void* workspace, size_t workspace_bytes,
                         const int32_t* run_row0, const int32_t* run_len, int runs, int max_run_len, int dtype, int pdl,
                         zl_stream_t stream);
/* The residual update of a layer whose sublayers read one norm of x and are gated per channel:
 *   x[t] += mult * (scale_a * sigmoid(gates[t][ga_off + c]) * a[t] + scale_f * sigmoid(gates[t][gf_off + c]) * f[t]),
 *   f[t] = sum_p coef[t][p] * (choice[t][p] < n_real ? parts[t * n_parts + p] : h[t]) + f_dense[t]
 * with h[t] = norm_w * x[t] / sqrt(mean(x[t]^2) + eps) of the x before the update (the sublayers' input, recomputed for
 * choices that hand it through).  a, parts, f_dense fp32 (T or T * n_parts rows of D); parts / f_dense may be NULL (no
 * such term; both NULL: no second sublayer); choice NULL: every part is real.  next_w != NULL: the next layer's input
 * next_w * x[t] / sqrt(mean(x[t]^2) + eps) of the new x -> h_next (T, D) of act_dtype. */
int zl_gated_parallel_combine(float* x, long long ldx, float mult, const float* gates, long long ldg, const float* a,
                              long long lda, int ga_off, const float* scale_a, const float* parts, long long ldp,
                              const float* coef, const int32_t* choice, int n_parts, int n_real, const float* f_dense,
                              long long ldf, int gf_off, const float* scale_f, const float* norm_w, const float* next_w,
                              void* h_next, int act_dtype, int T, int D, float eps, int pdl, zl_stream_t stream);
/* ------------------------------------------------------------------------------------------ *
 * Kodupel: decoder-only model whose layers are listed one by one: the mixer is attention (grouped key/value heads,
 * biased projections, per-head query / key RMS norm, partial rotation in adjacent pairs with YaRN frequencies, value
 * heads of unit RMS, a softmax whose denominator holds an extra 1, one sigmoid gate per head, optionally another
 * layer's key/value cache) or a generalized delta rule (a recurrent per-head state); the feed-forward is a mixture
 * of clamped gated experts chosen by sigmoid scores plus a correction; RMS norms with weight 1 + w sit on the
 * sublayers' outputs only; the residual stream is fp32.  Same driver shape as zl_dekipel_*.
 * ------------------------------------------------------------------------------------------ */
enum { ZL_MIXER_ATTENTION = 0, ZL_MIXER_GENERAL_DELTA = 1 };
typedef struct zl_kodupel zl_kodupel_t;
typedef struct zl_kodupel_layer {
    int type;              /* ZL_MIXER_* */
    int heads, kv_heads, dim, vdim;
    int kv_from;           /* attention: -1 own keys and values; j: reads layer j's caches */
    int rot_dims;          /* attention: rotated dimensions of every head (even, <= dim; 0: none) */
    float rot_base, yarn_factor /* 0: no scaling */, yarn_original, yarn_fast, yarn_slow;
    float scale;           /* attention: score scale */
    int decay_rank;        /* delta rule: inner size of the decay's two-matrix path */
    int experts, top, ff;  /* experts 0: no feed-forward sublayer */
    float limit;           /* clamp of the experts' gate and up projections */
} zl_kodupel_layer_t;
typedef struct zl_kodupel_config {
    int num_layers, width, vocab;
    float eps, embed_scale;
    int dtype; /* ZL_BF16 or ZL_F32 */
    int max_batch, max_seq, max_step_tokens;
    int use_pdl, use_graph;
} zl_kodupel_config_t;
int zl_kodupel_create(const zl_kodupel_config_t* cfg, const zl_kodupel_layer_t* layers, zl_kodupel_t** out);
void zl_kodupel_destroy(zl_kodupel_t* m);
int zl_kodupel_load_tensor(zl_kodupel_t* m, const char* name, const void* data_host, int rows, int cols, int elem_bytes);
int zl_kodupel_init_synthetic(zl_kodupel_t* m, uint64_t seed);
int zl_kodupel_finalize(zl_kodupel_t* m);
/* Same contract as zl_dekipel_step. */
int zl_kodupel_step(zl_kodupel_t* m, const int32_t* tokens_host, const int32_t* slots_host, const int32_t* positions_host,
                    int T, const int32_t* want_rows_host, int n_want, float* logits_host, int32_t* next_host);
int zl_kodupel_set_state(zl_kodupel_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B);
int zl_kodupel_step_device(zl_kodupel_t* m, int B);
int zl_kodupel_sync(zl_kodupel_t* m);
zl_stream_t zl_kodupel_stream(zl_kodupel_t* m);
int zl_kodupel_capture_layers(zl_kodupel_t* m, int on);
int zl_kodupel_read_layers(zl_kodupel_t* m, float* out_host, int T);
int zl_kodupel_stats(zl_kodupel_t* m, double* weight_bytes, int* kernels_per_step);
/* Copies one slot's recurrent state of layer `layer` ((heads, dim, dim) fp32) to the host (tests). */
int zl_kodupel_read_state(zl_kodupel_t* m, int layer, int slot, float* out_host);

/* ------------------------------------------------------------------------------------------ *
 * Lagelorn: decoder-only model with learned positions and norm after the sum, x <- norm(alpha x + sublayer(x)) on an
 * fp32 residual stream, whose layers are listed one by one.  A "delta" layer's mixer is a gated delta rule behind
 * short convolutions; a "parallel" layer's mixer is the weighted sum of two mixers that read the same input: attention
 * within blocks of positions (queries and keys normed over the whole projection, values = the projected keys, a
 * learned bias by bucketed distance, a learned sink per head) and a decaying per-head state with a bonus for the
 * current token whose inputs are mixes of the token with its predecessor.  The feed-forward, where a layer has one,
 * is W_down (gelu_tanh(W_gate x) * (W_up x)) with biases.  After every layer a per-layer token embedding enters through
 * a small gated projection and a norm.  The logits are soft-capped.  Same driver shape as zl_kodupel_*.
 * ------------------------------------------------------------------------------------------ */
enum { ZL_LAYER_DELTA = 0, ZL_LAYER_PARALLEL = 1 };
typedef struct zl_lagelorn zl_lagelorn_t;
typedef struct zl_lagelorn_layer {
    int type;                              /* ZL_LAYER_* */
    int heads, kv_heads, dim, vdim, conv;  /* delta: value heads, q / k heads, key size, value size, convolution taps */
    int l_heads, l_kv_heads, l_dim;        /* parallel, attention: query heads, key heads, head size (values = keys) */
    int l_chunk, l_rel_rows;               /* block of positions a token sees (0: all), rows of the distance table */
    float l_bias_max, l_scale;             /* distance of the table's last logarithmic step, scale of q . k */
    int r_heads, r_dim, r_decay_rank;      /* parallel, decaying state: heads, head size, inner size of the decay path */
    float left_scale, right_scale;
    int ff;                                /* feed-forward inner size, 0: none */
} zl_lagelorn_layer_t;
typedef struct zl_lagelorn_config {
    int num_layers, width, vocab, max_positions, side_dim;
    float eps, postln_alpha, logit_softcap;
    int dtype;                             /* ZL_BF16 or ZL_F32 */
    int max_batch, max_seq, max_step_tokens, use_pdl, use_graph;
} zl_lagelorn_config_t;
int zl_lagelorn_create(const zl_lagelorn_config_t* cfg, const zl_lagelorn_layer_t* layers, zl_lagelorn_t** out);
void zl_lagelorn_destroy(zl_lagelorn_t* m);
int zl_lagelorn_load_tensor(zl_lagelorn_t* m, const char* name, const void* data_host, int rows, int cols, int elem_bytes);
int zl_lagelorn_init_synthetic(zl_lagelorn_t* m, uint64_t seed);
int zl_lagelorn_finalize(zl_lagelorn_t* m);
/* Same contract as zl_dekipel_step. */
int zl_lagelorn_step(zl_lagelorn_t* m, const int32_t* tokens_host, const int32_t* slots_host, const int32_t* positions_host,
                     int T, const int32_t* want_rows_host, int n_want, float* logits_host, int32_t* next_host);
int zl_lagelorn_set_state(zl_lagelorn_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B);
int zl_lagelorn_step_device(zl_lagelorn_t* m, int B);
int zl_lagelorn_sync(zl_lagelorn_t* m);
zl_stream_t zl_lagelorn_stream(zl_lagelorn_t* m);
int zl_lagelorn_capture_layers(zl_lagelorn_t* m, int on);
int zl_lagelorn_read_layers(zl_lagelorn_t* m, float* out_host, int T);
int zl_lagelorn_stats(zl_lagelorn_t* m, double* weight_bytes, int* kernels_per_step);
/* Copies one slot's recurrent state of layer `layer` ((heads, dim_k, dim_v) fp32) to the host (tests). */
int zl_lagelorn_read_state(zl_lagelorn_t* m, int layer, int slot, float* out_host);

/* ------------------------------------------------------------------------------------------ *
 * Dizizen: decoder-only model of parallel layers on an fp32 residual stream: one RMS norm (weight 1 + w) feeds the
 * mixer and the feed-forward, each result is scaled per channel (layer scale) and gated by sigmoid(W h + b), and the
 * sum enters the stream times residual_mult.  The mixer is attention with grouped key/value heads, biased
 * projections, rotation of queries and keys in halves, values rotated by their own position (cached so) whose summed
 * output is turned back by the query's position, an ordinary causal softmax, optionally another layer's caches.  The
 * feed-forward is absent, a dense clamped gated unit with biases, or a mixture of relu^2 experts chosen by softmax
 * scores plus a correction inside the best groups of router slots, with identity slots that hand the input through
 * and a shared expert.  Same driver shape as zl_kodupel_*.
 * ------------------------------------------------------------------------------------------ */
enum { ZL_FF_NONE = 0, ZL_FF_DENSE = 1, ZL_FF_MOE = 2 };
typedef struct zl_dizizen zl_dizizen_t;
typedef struct zl_dizizen_layer {
    int heads, kv_heads, dim, vdim;
    int kv_from;           /* -1 own keys and values; j: reads layer j's caches */
    int rot_dims;          /* rotated dimensions of every query / key head (even, <= dim; 0: none) */
    float rot_base, scale; /* frequencies base^(-2i/n) for queries / keys (n = rot_dims) and values (n = vdim); score scale */
    int ff_kind;           /* ZL_FF_* */
    int ff;                /* inner size of the dense feed-forward or of one expert */
    float limit;           /* dense: clamp of the gate and up projections */
    int experts, identity, top, groups, keep; /* router slots = experts + identity, in `groups` groups of which `keep` count */
    int shared_ff;         /* inner size of the shared expert, 0: none */
} zl_dizizen_layer_t;
typedef struct zl_dizizen_config {
    int num_layers, width, vocab;
    float eps, embed_scale, residual_mult;
    int dtype; /* ZL_BF16 or ZL_F32 */
    int max_batch, max_seq, max_step_tokens;
    int use_pdl, use_graph;
} zl_dizizen_config_t;
int zl_dizizen_create(const zl_dizizen_config_t* cfg, const zl_dizizen_layer_t* layers, zl_dizizen_t** out);
void zl_dizizen_destroy(zl_dizizen_t* m);
int zl_dizizen_load_tensor(zl_dizizen_t* m, const char* name, const void* data_host, int rows, int cols, int elem_bytes);
int zl_dizizen_init_synthetic(zl_dizizen_t* m, uint64_t seed);
int zl_dizizen_finalize(zl_dizizen_t* m);
/* Same contract as zl_dekipel_step. */
int zl_dizizen_step(zl_dizizen_t* m, const int32_t* tokens_host, const int32_t* slots_host, const int32_t* positions_host,
                    int T, const int32_t* want_rows_host, int n_want, float* logits_host, int32_t* next_host);
int zl_dizizen_set_state(zl_dizizen_t* m, const int32_t* tokens_host, const int32_t* positions_host, int B);
int zl_dizizen_step_device(zl_dizizen_t* m, int B);
int zl_dizizen_sync(zl_dizizen_t* m);
zl_stream_t zl_dizizen_stream(zl_dizizen_t* m);
int zl_dizizen_capture_layers(zl_dizizen_t* m, int on);
int zl_dizizen_read_layers(zl_dizizen_t* m, float* out_host, int T);
int zl_dizizen_stats(zl_dizizen_t* m, double* weight_bytes, int* kernels_per_step);
/* Copies rows 0 .. n_rows of one slot's key and value caches of a layer that owns them to the host as fp32:
 * keys (n_rows, kv_heads * dim), values (n_rows, kv_heads * vdim) (tests). */
int zl_dizizen_read_cache(zl_dizizen_t* m, int layer, int slot, int n_rows, float* keys_host, float* values_host);
#ifdef __cplusplus
}
#endif
#endif /* ZHILIGHT_B200_H_ */

"""Torch-tensor front end of the C-ABI (plumbing only: torch supplies device memory and streams).

Every function takes CUDA tensors, passes raw pointers to libzhilight_b200.so on the current stream and
returns torch tensors.  Names / argument meaning mirror the reference operator each one replaces.
"""
import ctypes

import torch

from . import _lib

F16, BF16, F32 = 0, 1, 2
EPI_NONE, EPI_SWIGLU, EPI_RESIDUAL, EPI_QKV_ROPE = 0, 1, 2, 3


def _dt(t):
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise _lib.ZLError(-2, "unsupported dtype %s" % t.dtype)


def _p(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise _lib.ZLError(-1, "zhilight_b200 ops need CUDA tensors (no CPU fallback)")
    if not t.is_contiguous():
        raise _lib.ZLError(-1, "tensor must be contiguous")
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# ------------------------------------------------------------------ load-time transforms
def gptq_shuffle(qweight, q_perm=None):
    """nn::gptq::gptq_shuffle -- in place on (K/8, N) int32."""
    k8, n = qweight.shape
    scratch = torch.empty_like(qweight) if q_perm is not None else None
    _lib.call("zl_gptq_shuffle", _p(qweight), _p(q_perm), _p(scratch), k8 * 8, n, _stream())
    return qweight


def gptq_increase_zero(qzeros):
    _lib.call("zl_gptq_increase_zero", _p(qzeros), qzeros.numel(), _stream())
    return qzeros


def gptq_subtract8(words):
    _lib.call("zl_gptq_subtract8", _p(words), words.numel(), _stream())
    return words


def q4_to_q8(qzeros):
    r, c8 = qzeros.shape
    out = torch.empty((r, c8 * 8), dtype=torch.uint8, device=qzeros.device)
    _lib.call("zl_q4_to_q8", _p(qzeros), _p(out), qzeros.numel(), _stream())
    return out


def awq_un_shuffle(qzeros):
    _lib.call("zl_awq_un_shuffle", _p(qzeros), qzeros.shape[0], qzeros.shape[1], _stream())
    return qzeros


def awq_shuffle(qweight, use_exllama=True):
    k, n8 = qweight.shape
    out = torch.empty((k // 8, n8 * 8), dtype=qweight.dtype, device=qweight.device)
    _lib.call("zl_awq_shuffle", _p(qweight), _p(out), k, n8 * 8, int(use_exllama), _stream())
    return out


def transpose_2d(x):
    r, c = x.shape
    out = torch.empty((c, r), dtype=x.dtype, device=x.device)
    _lib.call("zl_transpose_2d", _p(x), _p(out), r, c, x.element_size(), _stream())
    return out


def gptq_to_k_major(qweight, qzeros, scales, is_awq=False):
    """Int4GPTQ::preprocess_weight + transpose_weight (linear.cpp:1139-1160, 1085-1099) on device.
    Consumes copies of the HF tensors; returns (qweight_km (N,K/8) i32, qzeros_km (N,G) u8, scales_km (N,G) f16)."""
    if is_awq:
        qw = awq_shuffle(qweight.contiguous(), True)
        qz = awq_un_shuffle(qzeros.clone())
    else:
        qw = gptq_shuffle(qweight.clone())
        qz = gptq_increase_zero(qzeros.clone())
    z8 = q4_to_q8(qz)
    return transpose_2d(qw), transpose_2d(z8), transpose_2d(scales.contiguous())


def gptq_dequant_k_major(qweight_km, qzeros_km, scales_km):
    n, k8 = qweight_km.shape
    g = scales_km.shape[1]
    out = torch.empty((n, k8 * 8), dtype=torch.float16, device=qweight_km.device)
    _lib.call("zl_gptq_dequant_k_major", _p(qweight_km), _p(qzeros_km), _p(scales_km), _p(out), n, k8 * 8,
              (k8 * 8) // g, _stream())
    return out


def w4_pack(qweight_km, qzeros_km, scales_km, group_size=128, sym=False, row_map=None, variant=0):
    n_src, k8 = qweight_km.shape
    n = n_src if row_map is None else row_map.numel()
    k = k8 * 8
    nbytes = _lib.load().zl_w4_packed_bytes(n, k, group_size)
    if nbytes == 0:
        raise _lib.ZLError(-2, "unsupported ZLW4 shape N=%d K=%d group=%d" % (n, k, group_size))
    packed = torch.empty(nbytes, dtype=torch.uint8, device=qweight_km.device)
    _lib.call("zl_w4_pack_v", _p(qweight_km), _p(qzeros_km), _p(scales_km), _p(row_map), _p(packed), n, k, group_size,
              int(sym), int(variant), _stream())
    return packed


def w4_unpack(packed, n, k, group_size=128, variant=0):
    dev = packed.device
    qw = torch.empty((n, k // 8), dtype=torch.int32, device=dev)
    qz = torch.empty((n, k // group_size), dtype=torch.uint8, device=dev)
    sc = torch.empty((n, k // group_size), dtype=torch.float16, device=dev)
    _lib.call("zl_w4_unpack_v", _p(packed), _p(qw), _p(qz), _p(sc), n, k, group_size, int(variant), _stream())
    return qw, qz, sc


def swiglu_row_map(f, device):
    p = torch.arange(2 * f, device=device, dtype=torch.int32)
    tile, r = p // 16, p % 16
    return torch.where(r < 8, tile * 8 + r, f + tile * 8 + (r - 8)).to(torch.int32).contiguous()


# ------------------------------------------------------------------ compute
def w4a16_gemm(x, packed, n, k, group_size=128, bias=None, residual=None, epilogue=EPI_NONE, pdl=False, out=None):
    """nn::gptq::gptq_gemm_k_major (GEMV path) on the ZLW4 layout."""
    if x.dtype != torch.float16:
        raise _lib.ZLError(-2, "A must be half")      # q_gemm_k_major.cu:989
    m = x.shape[0]
    n_out = n // 2 if epilogue == EPI_SWIGLU else n
    if out is None:
        out = torch.empty((m, n_out), dtype=torch.float16, device=x.device)
    _lib.call("zl_w4a16_gemm", _p(x), x.stride(0), _p(packed), _p(bias), _p(residual), _p(out), m, n, k, group_size,
              epilogue, int(pdl), _stream())
    return out


def _dp(t):
    return t.data_ptr() if t is not None else None


def qkv_rope_row_map(n_heads_total, dim_head, device):
    m = torch.empty(n_heads_total * dim_head, dtype=torch.int32, device=device)
    _lib.call("zl_qkv_rope_row_map", _p(m), n_heads_total, dim_head, _stream())
    return m


def gather_rows_16(src, row_map):
    dst = torch.empty(row_map.numel(), dtype=src.dtype, device=src.device)
    _lib.call("zl_gather_rows_16", _p(src), _p(row_map), _p(dst), row_map.numel(), _stream())
    return dst


def w4a16_gemm_fused(x, packed, n, k, group_size=128, bias=None, residual=None, epilogue=EPI_NONE, pdl=False, out=None,
                     ln_weight=None, eps=1e-5, rope=None, variant=0):
    """zl_w4a16_gemm_fused.  rope = dict(cos, sin, token_batch, placement, k_bufs, v_bufs, num_heads, num_kv_heads,
    dim_head) for EPI_QKV_ROPE (returns q); bias must be in packed-row order."""
    if x.dtype != torch.float16:
        raise _lib.ZLError(-2, "A must be half")
    m = x.shape[0]
    a = _lib.W4FusedArgs()
    a.x, a.ldx, a.packed, a.bias, a.residual = x.data_ptr(), x.stride(0), packed.data_ptr(), _dp(bias), _dp(residual)
    a.M, a.N, a.K, a.group_size, a.epilogue, a.pdl = m, n, k, group_size, epilogue, int(pdl)
    a.ln_weight, a.eps = _dp(ln_weight), eps
    a.variant = int(variant)
    keep = []
    if epilogue == EPI_QKV_ROPE:
        r = rope
        q = torch.empty((m, r["num_heads"] * r["dim_head"]), dtype=torch.float16, device=x.device)
        ka, va = _ptr_table(r["k_bufs"], x.device), _ptr_table(r["v_bufs"], x.device)
        keep += [ka, va]
        a.cos, a.sin, a.q_out = r["cos"].data_ptr(), r["sin"].data_ptr(), q.data_ptr()
        a.token_batch, a.placement = r["token_batch"].data_ptr(), r["placement"].data_ptr()
        a.k_addrs, a.v_addrs = ka.data_ptr(), va.data_ptr()
        a.num_heads, a.num_kv_heads, a.dim_head = r["num_heads"], r["num_kv_heads"], r["dim_head"]
        ret = q
    else:
        n_out = n // 2 if epilogue == EPI_SWIGLU else n
        if out is None:
            out = torch.empty((m, n_out), dtype=torch.float16, device=x.device)
        a.y = out.data_ptr()
        ret = out
    _lib.call("zl_w4a16_gemm_fused", ctypes.byref(a), _stream())
    if keep:
        torch.cuda.current_stream().synchronize()
    return ret


def dense_gemm_skinny(x, w, bias=None, out_dtype=None, pdl=False):
    m, k = x.shape
    n = w.shape[0]
    od = x.dtype if out_dtype is None else out_dtype
    out = torch.empty((m, n), dtype=od, device=x.device)
    _lib.call("zl_dense_gemm_skinny", _p(x), x.stride(0), _p(w), _p(bias), _p(out), m, n, k, _dt(x), _dt(out),
              int(pdl), _stream())
    return out


W8_INT8, W8_FP8 = 0, 1


def int8_quant_per_token(x, pdl=False):
    """int8_op::quant_calc_scale: returns (q int8 (M,K), scale f32 (M))."""
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    scale = torch.empty((m,), dtype=torch.float32, device=x.device)
    _lib.call("zl_int8_quant_per_token", _p(x), x.stride(0), _p(q), _p(scale), m, k, _dt(x), int(pdl), _stream())
    return q, scale


def rmsnorm_quant(x, weight, eps, scale=1.0, pdl=False):
    """int8_op::layernorm_quant: returns (y, q int8, qscale f32 (T))."""
    t, d = x.shape
    y = torch.empty_like(x)
    q = torch.empty((t, d), dtype=torch.int8, device=x.device)
    qs = torch.empty((t,), dtype=torch.float32, device=x.device)
    _lib.call("zl_rmsnorm_quant", _p(x), _p(weight), _p(y), _p(q), _p(qs), t, d, eps, scale, _dt(x), int(pdl),
              _stream())
    return y, q, qs


def fp8_quant_per_tensor(x, pdl=False):
    """nn::fp8::dynamic_scaled_quant: returns (q uint8 holding e4m3 bits, scale f32 (1))."""
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty((1,), dtype=torch.float32, device=x.device)
    _lib.call("zl_fp8_quant_per_tensor", _p(x), _p(q), _p(scale), x.numel(), _dt(x), int(pdl), _stream())
    return q, scale


def w8a8_gemm(xq, x_scale, w, w_scale, out_dtype, kind=W8_INT8, bias=None, pdl=False):
    m, k = xq.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device=xq.device)
    ws_dt = 2 if w_scale.dtype == torch.float32 else _dt(w_scale)
    _lib.call("zl_w8a8_gemm", _p(xq), _p(x_scale), _p(w), _p(w_scale), ws_dt, _p(bias), _p(y), m, n, k, kind,
              _dt(y), int(pdl), _stream())
    return y


def int8_linear(x, w_q, w_scale, bias=None, pdl=False):
    """Int8Linear::forward (linear.cpp:560-636) in two launches instead of three."""
    q, s = int8_quant_per_token(x, pdl)
    return w8a8_gemm(q, s, w_q, w_scale, x.dtype, W8_INT8, bias, pdl)


def fp8_linear(x, w_fp8, w_scale, bias=None, pdl=False):
    """Fp8Linear::forward (linear.cpp:1660-1695)."""
    q, s = fp8_quant_per_tensor(x, pdl)
    return w8a8_gemm(q, s, w_fp8, w_scale, x.dtype, W8_FP8, bias, pdl)


def rmsnorm(x, weight, eps, scale=1.0, pdl=False):
    t, d = x.shape
    y = torch.empty_like(x)
    _lib.call("zl_rmsnorm", _p(x), _p(weight), _p(y), t, d, eps, scale, _dt(x), int(pdl), _stream())
    return y


def add_rmsnorm(a, b, weight, eps, scale=1.0, mode=0, pdl=False):
    t, d = a.shape
    out_sum = torch.empty_like(a)
    y = torch.empty_like(a)
    _lib.call("zl_add_rmsnorm", _p(a), _p(b), _p(weight), _p(out_sum), _p(y), t, d, eps, scale, mode, _dt(a),
              int(pdl), _stream())
    return out_sum, y


def element_add_scale(a, b, scale=1.0):
    c = torch.empty_like(a)
    _lib.call("zl_element_add_scale", _p(a), _p(b), _p(c), a.numel(), scale, _dt(a), _stream())
    return c


def gate_mul(gate, up, act="silu"):
    t, f = gate.shape
    out = torch.empty((t, f), dtype=gate.dtype, device=gate.device)
    # strided views are fine here: the C entry point takes row strides
    _lib.call("zl_gate_mul", ctypes.c_void_p(gate.data_ptr()), gate.stride(0),
              ctypes.c_void_p(up.data_ptr()) if up is not None else None, up.stride(0) if up is not None else 0, _p(out), f, t, f, 0 if act == "silu" else 1, _dt(gate), _stream())
    return out


def activation(x, act):
    """Linear::activate: silu / gelu in fp32, rounded to T."""
    return gate_mul(x, None, act)


def rope_cos_sin(pos, dim_head, theta, llama3=None, neox=True):
    t = pos.numel()
    cos = torch.empty((t, dim_head), dtype=torch.float32, device=pos.device)
    sin = torch.empty_like(cos)
    l3 = llama3 or {}
    _lib.call("zl_rope_cos_sin", _p(pos), _p(cos), _p(sin), t, dim_head, float(theta),
              float(l3.get("factor", 0.0)), float(l3.get("low", 1.0)), float(l3.get("high", 4.0)),
              float(l3.get("orig", 8192.0)), int(neox), _stream())
    return cos, sin


def rope_qk_cache(cos, sin, qkv, num_heads, num_kv_heads, dim_head, neox=True):
    t = qkv.shape[0]
    q = torch.empty((t, num_heads * dim_head), dtype=qkv.dtype, device=qkv.device)
    k = torch.empty((t, num_kv_heads * dim_head), dtype=qkv.dtype, device=qkv.device)
    v = torch.empty_like(k)
    _lib.call("zl_rope_qk_cache", _p(cos), _p(sin), _p(qkv), _p(q), _p(k), _p(v), t, num_heads, num_kv_heads,
              dim_head, int(neox), _dt(qkv), _stream())
    return q, k, v


def _ptr_table(tensors, device):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=device)


def copy_to_rag_buffer2(placement, buf_lens, k_src, v_src, k_bufs, v_bufs, bshd=True):
    b, len_q, hkv, d = k_src.shape
    ka, va = _ptr_table(k_bufs, k_src.device), _ptr_table(v_bufs, k_src.device)
    _lib.call("zl_copy_to_rag_buffer2", _p(placement), _p(buf_lens), _p(k_src), _p(v_src), _p(ka), _p(va), b, len_q,
              hkv, d, int(bshd), _dt(k_src), _stream())
    torch.cuda.current_stream().synchronize()      # keep the pointer tables alive until the copy ran


def qkv_rope_append(cos, sin, qkv, token_batch, placement, k_bufs, v_bufs, num_heads, num_kv_heads, dim_head,
                    buf_lens=None, neox=True, bshd=True, pdl=False):
    t = qkv.shape[0]
    q = torch.empty((t, num_heads * dim_head), dtype=qkv.dtype, device=qkv.device)
    ka, va = _ptr_table(k_bufs, qkv.device), _ptr_table(v_bufs, qkv.device)
    _lib.call("zl_qkv_rope_append", _p(cos), _p(sin), _p(qkv), _p(q), _p(token_batch), _p(placement), _p(ka), _p(va),
              t, num_heads, num_kv_heads, dim_head, int(neox), int(bshd), _p(buf_lens), _dt(qkv), int(pdl), _stream())
    torch.cuda.current_stream().synchronize()
    return q


def decode_attention(q, buf_lens, k_bufs, v_bufs, mask, scale, max_len_buf, num_kv_heads, bshd=True, pdl=False):
    """nn::multi_query_attention_rag_buffer: q (B, len_q, H_q, d); k_bufs/v_bufs lists of per-task tensors."""
    b, len_q, hq, d = q.shape
    out = torch.empty_like(q)
    ws_bytes = _lib.load().zl_decode_attention_workspace_bytes(b, len_q, hq, d, max_len_buf)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    ka, va = _ptr_table(k_bufs, q.device), _ptr_table(v_bufs, q.device)
    _lib.call("zl_decode_attention", _p(q), _p(buf_lens), _p(ka), _p(va), _p(mask), float(scale), max_len_buf,
              _p(out), b, len_q, hq, num_kv_heads, d, int(bshd), _p(ws), ws_bytes, _dt(q), int(pdl), _stream())
    torch.cuda.current_stream().synchronize()
    return out


def decode_attention_kv8(q, buf_lens, k_bufs, v_bufs, sk_bufs, sv_bufs, mask, scale, max_len_buf, num_kv_heads, out_dtype=None,
                         pdl=False):
    """int8 KV cache attention: q (B, len_q, H_q, d) f16; k/v lists of (len_buf, H_kv, d) uint8; sk/sv lists of
    (len_buf, H_kv) fp32 scales."""
    b, len_q, hq, d = q.shape
    out = torch.empty(q.shape, dtype=out_dtype or q.dtype, device=q.device)
    ws_bytes = _lib.load().zl_decode_attention_workspace_bytes(b, len_q, hq, d, max_len_buf)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    tabs = [_ptr_table(x, q.device) for x in (k_bufs, v_bufs, sk_bufs, sv_bufs)]
    _lib.call("zl_decode_attention_kv8", _p(q), _p(buf_lens), _p(tabs[0]), _p(tabs[1]), _p(tabs[2]), _p(tabs[3]), _p(mask),
              float(scale), max_len_buf, _p(out), b, len_q, hq, num_kv_heads, d, _p(ws), ws_bytes, _dt(out), int(pdl),
              _stream())
    torch.cuda.current_stream().synchronize()
    return out


def kv_int8_quant_append(k_src, v_src, token_batch, placement, k_bufs, v_bufs, sk_bufs, sv_bufs):
    """k_src / v_src (T, H_kv, d) -> uint8 codes + fp32 scales scattered into the per-task caches."""
    t, hkv, d = k_src.shape
    tabs = [_ptr_table(x, k_src.device) for x in (k_bufs, v_bufs, sk_bufs, sv_bufs)]
    _lib.call("zl_kv_int8_quant_append", _p(k_src), _p(v_src), _p(token_batch), _p(placement), _p(tabs[0]), _p(tabs[1]),
              _p(tabs[2]), _p(tabs[3]), t, hkv, d, _dt(k_src), 0, _stream())
    torch.cuda.current_stream().synchronize()


def embedding(ids, table):
    t = ids.numel()
    out = torch.empty((t, table.shape[1]), dtype=table.dtype, device=table.device)
    _lib.call("zl_embedding", _p(ids), _p(table), _p(out), t, table.shape[1], table.shape[0], _dt(table), 0, _stream())
    return out


def argmax(logits):
    t, v = logits.shape
    out = torch.empty(t, dtype=torch.int32, device=logits.device)
    nb = _lib.load().zl_argmax_workspace_bytes(t)
    ws = torch.empty(nb, dtype=torch.uint8, device=logits.device)
    _lib.call("zl_argmax", _p(logits), _p(out), t, v, _p(ws), nb, 0, _stream())
    return out


# ------------------------------------------------------------------ fp32-residual layers: grouped norm, conv, latents
GEMM_EPI_NONE, GEMM_EPI_RELU2, GEMM_EPI_SIGMOID_GATE = 0, 1, 2


def gemm_nt(x, w, out_dtype=None, epilogue=GEMM_EPI_NONE, gate=None):
    """y = epi(x @ w^T).  x (M, K) with w (N, K), or batched x (B, M, K) with w (B, N, K); any sizes.  gate (fp32, shape of
    y) for GEMM_EPI_SIGMOID_GATE."""
    batched = x.dim() == 3
    xb, wb = (x, w) if batched else (x[None], w[None])
    b, m, k = xb.shape
    n = wb.shape[1]
    od = out_dtype or x.dtype
    y = torch.empty((b, m, n), dtype=od, device=x.device)
    _lib.call("zl_gemm_nt", _p(xb), k, m * k, _p(wb), k, n * k, _p(y), n, m * n, m, n, k, b, _dt(x), _dt(y), epilogue,
              _p(gate), n, m * n, 0, _stream())
    return y if batched else y[0]


def group_rmsnorm(x, weight, groups, eps, out_dtype=torch.float32):
    """x (T, D) fp32, weight (D) fp32 -> (T, D): RMS norm over each of `groups` equal consecutive parts."""
    t, d = x.shape
    y = torch.empty((t, d), dtype=out_dtype, device=x.device)
    _lib.call("zl_group_rmsnorm", _p(x), d, _p(weight), _p(y), d, t, d, groups, eps, _dt(y), 0, _stream())
    return y


def group_rmsnorm_residual(y, weight, x, groups, eps, conv_in=None, slot=None, pos=None, ring=None, taps=1):
    """x += group_rmsnorm(y) in place; with ring (slots, taps-1, D) also stores conv_in rows into the slots' rings."""
    t, d = x.shape
    _lib.call("zl_group_rmsnorm_residual", _p(y), d, _p(weight), _p(x), d, t, d, groups, eps, _p(conv_in), d, _p(slot),
              _p(pos), _p(ring), taps, 0, _stream())
    return x


def causal_conv_mix(h, taps_weight, slot, pos, ring, out_dtype=torch.float32):
    """u = h + causal conv of h over each sequence's positions; h (T, D) fp32, taps_weight (D, taps) fp32,
    ring (slots, taps-1, D) fp32 or None when taps == 1."""
    t, d = h.shape
    u = torch.empty((t, d), dtype=out_dtype, device=h.device)
    _lib.call("zl_causal_conv_mix", _p(h), d, _p(taps_weight), _p(slot), _p(pos), _p(ring), _p(u), d, t, d,
              taps_weight.shape[1], _dt(u), 0, _stream())
    return u


def slot_table(cache):
    """cache (slots, rows, width) -> int64 tensor of the slots' base addresses (a device pointer table)."""
    step = cache.stride(0) * cache.element_size()
    return torch.tensor([cache.data_ptr() + i * step for i in range(cache.shape[0])], dtype=torch.int64, device=cache.device)


def latent_norm_append(proj, q_off, q_weight, c_off, kv_weight, cache, table, slot, pos, eps):
    """RMS norms of the query latent (-> returned (T, q_rank)) and of the key-value latent (-> cache rows (slot, pos))."""
    t, ldp = proj.shape
    q_rank = q_weight.numel()
    cq = torch.empty((t, q_rank), dtype=cache.dtype, device=proj.device)
    _lib.call("zl_latent_norm_append", _p(proj), ldp, q_off, q_rank, _p(q_weight), _p(cq), c_off,
              cache.shape[2], _p(kv_weight), _p(table), _p(slot), _p(pos), t, eps, _dt(cache), 0, _stream())
    return cq


def latent_attention(q_absorbed, cache, table, slot, pos, sink, scale, splits=1):
    """q_absorbed (T, H, R) fp32, cache (slots, rows, R) -> (T, H, R) of the cache dtype."""
    t, h, r = q_absorbed.shape
    lib = _lib.load()
    _lib.check(lib.zl_latent_attention_prepare(h, r, _dt(cache)))
    nbytes = lib.zl_latent_attention_workspace_bytes(t, h, r, splits)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=cache.device)
    out = torch.empty((t, h, r), dtype=cache.dtype, device=cache.device)
    _lib.call("zl_latent_attention", _p(q_absorbed), _p(table), _p(slot), _p(pos), _p(sink), scale, _p(out), t, h, r, splits,
              _p(ws), nbytes, _dt(cache), 0, _stream())
    return out


def group_norm_conv(x, norm_weight, taps_weight, slot, pos, ring, groups, eps, out_dtype=torch.float32):
    """Fused pre-norm + causal convolution: returns (h = group_rmsnorm(x), u = h + conv(h))."""
    t, d = x.shape
    h = torch.empty((t, d), dtype=torch.float32, device=x.device)
    u = torch.empty((t, d), dtype=out_dtype, device=x.device)
    _lib.call("zl_group_norm_conv", _p(x), d, _p(norm_weight), _p(taps_weight), _p(slot), _p(pos), _p(ring), _p(h), _p(u), t, d,
              groups, taps_weight.shape[1], eps, _dt(u), 0, _stream())
    return h, u


# ------------------------------------------------------------------ per-head norms, rotation, sink attention, delta rule, experts
GEMM_EPI_TANH, GEMM_EPI_GLU_CLAMP = 3, 4
MOE_SCORE_SIGMOID, MOE_SCORE_SOFTMAX = 0, 1


def gemm_nt_bias(x, w, bias=None, out_dtype=None, epilogue=GEMM_EPI_NONE):
    """y = epi(x @ w^T + bias); x (M, K), w (N, K), bias (N) fp32 or None; epilogue none, relu^2 or tanh."""
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=out_dtype or x.dtype, device=x.device)
    _lib.call("zl_gemm_nt_bias", _p(x), k, _p(w), k, _p(bias), _p(y), n, m, n, k, _dt(x), _dt(y), epilogue, 0, _stream())
    return y


def gemm_nt_grouped(x, w, group_offsets, rows_out, x_rows=None, y_rows=None, out_dtype=None, epilogue=GEMM_EPI_NONE, limit=0.0,
                    alpha=1.0, beta=0.0):
    """Grouped y = epi(x[x_rows] @ w[g]^T) scattered to y[y_rows]; w (G, N, K); group_offsets (G + 1) int32 over a list
    sorted by group; y has `rows_out` rows of N (N / 2 with the gated-unit epilogue) columns, zero where nothing lands."""
    g, n, k = w.shape
    n_out = n // 2 if epilogue == GEMM_EPI_GLU_CLAMP else n
    y = torch.zeros((rows_out, n_out), dtype=out_dtype or x.dtype, device=x.device)
    total = (x_rows if x_rows is not None else y_rows if y_rows is not None else x).shape[0]
    _lib.call("zl_gemm_nt_grouped", _p(x), x.shape[1], _p(x_rows), _p(w), k, n * k, _p(y), n_out, _p(y_rows), _p(group_offsets),
              g, total, n, k, _dt(x), _dt(y), epilogue, limit, alpha, beta, 0, _stream())
    return y


def rope_inv_freq_yarn(base, dims, factor=0.0, original=0.0, fast=0.0, slow=0.0):
    """-> (frequencies (dims / 2) float64 numpy array, cos / sin scale)."""
    import numpy as np
    out = np.zeros(max(dims // 2, 1), dtype=np.float64)
    ms = ctypes.c_float()
    _lib.call("zl_rope_inv_freq_yarn", float(base), dims, float(factor), float(original), float(fast), float(slow),
              out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)), ctypes.cast(ctypes.byref(ms), ctypes.c_void_p))
    return out[:dims // 2], ms.value


def qkv_headnorm_rope_append(proj, q_off, k_off, v_off, heads, kv_heads, dim, vdim, q_weight, k_weight, inv_freq, rot_dims,
                             mscale, eps, k_cache, v_cache, k_table, v_table, slot, pos, dtype):
    """proj (T, ld) fp32, inv_freq (rot_dims / 2) float64 -> q (T, heads * dim) of `dtype`; keys / values go to rows (slot, pos) of the caches
    (slots, rows, kv_heads * dim) / (slots, rows, kv_heads * vdim) unless k_off < 0."""
    t, ldp = proj.shape
    q = torch.empty((t, heads * dim), dtype=dtype, device=proj.device)
    _lib.call("zl_qkv_headnorm_rope_append", _p(proj), ldp, q_off, k_off, v_off, heads, kv_heads, dim, vdim, _p(q_weight),
              _p(k_weight), ctypes.cast(_p(inv_freq), ctypes.POINTER(ctypes.c_double)), rot_dims, mscale, eps, _p(q), _p(k_table), _p(v_table), _p(slot), _p(pos), t, _dt(q),
              0, _stream())
    return q


def sink_attention(q, k_table, v_table, slot, pos, scale, heads, kv_heads, dim, vdim, sink=None, gate=None, splits=1,
                   run_row0=None, run_len=None, max_run_len=0):
    """q (T, heads * dim) -> (T, heads * vdim); gate (T, ld) fp32 logits whose first `heads` columns gate the heads.
    run_row0 / run_len (int32 device tensors) describe the step's runs and select the tensor-core kernel."""
    t = q.shape[0]
    lib = _lib.load()
    nbytes = lib.zl_sink_attention_workspace_bytes(t, heads, vdim, splits)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    out = torch.empty((t, heads * vdim), dtype=q.dtype, device=q.device)
    _lib.call("zl_sink_attention", _p(q), _p(k_table), _p(v_table), _p(slot), _p(pos), _p(sink), _p(gate),
              gate.shape[1] if gate is not None else 0, scale, _p(out), t, heads, kv_heads, dim, vdim, splits, _p(ws), nbytes,
              _p(run_row0), _p(run_len), run_row0.numel() if run_row0 is not None else 0, max_run_len, _dt(q), 0, _stream())
    return out


def head_rmsnorm_gate(o, heads, vdim, eps, weight=None, gate=None, out_dtype=torch.float32):
    """o (T, heads * vdim) fp32: each head divided by its RMS, times weight (heads * vdim), times sigmoid(gate) (same shape)."""
    t = o.shape[0]
    y = torch.empty((t, heads * vdim), dtype=out_dtype, device=o.device)
    _lib.call("zl_head_rmsnorm_gate", _p(o), heads * vdim, _p(weight), _p(gate), heads * vdim, _p(y), heads * vdim, t, heads,
              vdim, eps, _dt(y), 0, _stream())
    return y


def rmsnorm_residual_combine(parts, coef, weight, x, eps, act_dtype=None):
    """x (T, D) fp32 += weight * rmsnorm(sum_p coef[t, p] * parts[t, p]); parts (T, n_parts, D) fp32, coef (T, n_parts) or None.
    Returns the new x rounded to act_dtype when that is given."""
    t, n_parts, d = parts.shape
    xa = torch.empty((t, d), dtype=act_dtype, device=x.device) if act_dtype is not None else None
    _lib.call("zl_rmsnorm_residual_combine", _p(parts), d, _p(coef), n_parts, _p(weight), _p(x), d, _p(xa),
              _dt(xa) if xa is not None else BF16, t, d, eps, 0, _stream())
    return xa


def delta_rule(r, k, v, rate_logit, decay_logit, decay_scale, unit_eps, run_row0, run_len, slot, pos, state, state_table, heads,
               dim_k, dim_v):
    """All inputs (T, heads * dim) fp32; state (slots, heads, dim_k, dim_v) fp32 is updated in place.  -> o (T, heads * dim_v)."""
    t = r.shape[0]
    o = torch.empty((t, heads * dim_v), dtype=torch.float32, device=r.device)
    nbytes = _lib.load().zl_delta_rule_workspace_bytes(t, heads, dim_k, dim_v)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=r.device)
    _lib.call("zl_delta_rule", _p(r), heads * dim_k, _p(k), heads * dim_k, _p(v), heads * dim_v, _p(rate_logit), heads * dim_k,
              _p(decay_logit), heads * dim_k, decay_scale, unit_eps, _p(run_row0), _p(run_len), run_row0.numel(), _p(slot),
              _p(pos), _p(state_table), _p(o), heads * dim_v, heads, dim_k, dim_v, t, _p(ws), nbytes, 0, _stream())
    return o


def moe_route(x, w_router, correction, top, score_fn=MOE_SCORE_SIGMOID, renormalize=False):
    """x (T, D) fp32, w_router (E, D) fp32 -> (experts (T, top) int32, weights (T, top) fp32, group offsets (E + 1),
    list_token (T * top), list_pair (T * top))."""
    t, d = x.shape
    e = w_router.shape[0]
    dev = x.device
    te = torch.empty((t, top), dtype=torch.int32, device=dev)
    tw = torch.empty((t, top), dtype=torch.float32, device=dev)
    off = torch.empty(e + 1, dtype=torch.int32, device=dev)
    lt = torch.empty(t * top, dtype=torch.int32, device=dev)
    lp = torch.empty(t * top, dtype=torch.int32, device=dev)
    _lib.call("zl_moe_route", _p(x), d, _p(w_router), _p(correction), _p(te), _p(tw), _p(off), _p(lt), _p(lp), t, d, e, top,
              score_fn, int(renormalize), 0, _stream())
    return te, tw, off, lt, lp


# ------------------------------------------------------------------ block attention with distance bias, predecessor mixes,
# norm after the sum, gated delta rule, decaying state with a bonus
GEMM_EPI_GEGLU_TANH, GEMM_EPI_GELU_TANH_MUL, GEMM_EPI_SOFTCAP = 5, 6, 7
GATE_SIGMOID, GATE_SILU = 0, 1


def gemm_nt_fused(x, w, bias=None, out_dtype=None, epilogue=GEMM_EPI_NONE, mul=None, limit=0.0):
    """y = epi(x @ w^T + bias); epilogue none / relu^2 / tanh / gelu_tanh(v) * mul (mul (M, N) fp32) / gelu_tanh(gate) * up over
    column pairs (y has N / 2 columns) / soft cap at `limit`."""
    m, k = x.shape
    n = w.shape[0]
    n_out = n // 2 if epilogue == GEMM_EPI_GEGLU_TANH else n
    y = torch.empty((m, n_out), dtype=out_dtype or x.dtype, device=x.device)
    _lib.call("zl_gemm_nt_fused", _p(x), k, _p(w), k, _p(bias), _p(y), n_out, m, n, k, _dt(x), _dt(y), epilogue, _p(mul),
              mul.shape[1] if mul is not None else 0, limit, 0, _stream())
    return y


def dense_gemm_skinny_mul(x, w, act, mul=None, out_dtype=None):
    """Skinny Linear with an activation on the output: act 0 none, 1 relu^2, 2 tanh, 3 gelu_tanh(v) * mul[m, n] (mul fp32)."""
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=out_dtype or x.dtype, device=x.device)
    _lib.call("zl_dense_gemm_skinny_mul", _p(x), k, _p(w), None, _p(y), m, n, k, _dt(x), _dt(y), act, _p(mul),
              mul.shape[1] if mul is not None else 0, 0, _stream())
    return y


def distance_bias_table(table, far, n_dist):
    """table (rows, heads) numpy float32 -> (heads, n_dist) numpy float32: the table's row for every distance below n_dist."""
    import numpy as np
    t = np.ascontiguousarray(table, dtype=np.float32)
    out = np.zeros((t.shape[1], n_dist), dtype=np.float32)
    _lib.call("zl_distance_bias_table", t.ctypes.data_as(ctypes.c_void_p), t.shape[0], t.shape[1], float(far), n_dist,
              out.ctypes.data_as(ctypes.c_void_p))
    return out


def sink_attention_local(q, k_table, v_table, slot, pos, scale, heads, kv_heads, dim, vdim, sink=None, chunk=0, dist_bias=None,
                         splits=1, run_row0=None, run_len=None, max_run_len=0):
    """sink_attention restricted to blocks of `chunk` positions (0: none) and with dist_bias (heads, n_dist) fp32 added to the
    scaled scores by distance."""
    t = q.shape[0]
    lib = _lib.load()
    nbytes = lib.zl_sink_attention_workspace_bytes(t, heads, vdim, splits)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    out = torch.empty((t, heads * vdim), dtype=q.dtype, device=q.device)
    _lib.call("zl_sink_attention_local", _p(q), _p(k_table), _p(v_table), _p(slot), _p(pos), _p(sink), None, 0, scale, chunk,
              _p(dist_bias), dist_bias.shape[1] if dist_bias is not None else 0, _p(out), t, heads, kv_heads, dim, vdim, splits,
              _p(ws), nbytes, _p(run_row0), _p(run_len), run_row0.numel() if run_row0 is not None else 0, max_run_len, _dt(q), 0,
              _stream())
    return out


def qk_fullnorm_append(proj, q_off, k_off, heads, kv_heads, dim, q_weight, k_weight, eps, k_table, v_table, slot, pos, dtype):
    """proj (T, ld) fp32 -> q (T, heads * dim) of `dtype`, normed over the whole projection; the normed k goes to the key
    cache rows (slot, pos), the projected k itself to the value cache rows."""
    t, ldp = proj.shape
    q = torch.empty((t, heads * dim), dtype=dtype, device=proj.device)
    _lib.call("zl_qk_fullnorm_append", _p(proj), ldp, q_off, k_off, heads, kv_heads, dim, _p(q_weight), _p(k_weight), eps, _p(q),
              _p(k_table), _p(v_table), _p(slot), _p(pos), t, _dt(q), 0, _stream())
    return q


def token_shift_mix(x, mu, state_table, slot, pos, store_state, out_dtype=torch.float32):
    """x (T, D) fp32, mu (n, D) fp32 -> (n, T, D): x + (x_prev - x) * mu[s]; state (slots, D) fp32 through its pointer table."""
    t, d = x.shape
    n = mu.shape[0]
    out = torch.empty((n, t, d), dtype=out_dtype, device=x.device)
    _lib.call("zl_token_shift_mix", _p(x), d, _p(mu), n, _p(state_table), _p(slot), _p(pos), _p(out), t * d, t, d,
              int(store_state), _dt(out), 0, _stream())
    return out


def store_run_tails(src, col, channels, n_tail, run_row0, run_len, slot, pos, ring_table):
    _lib.call("zl_store_run_tails", _p(src), src.shape[1], col, channels, n_tail, _p(run_row0), _p(run_len), run_row0.numel(),
              _p(slot), _p(pos), _p(ring_table), 0, _stream())


def postnorm_combine(x, alpha, a, coef_a, weight, eps, b=None, coef_b=0.0, act_dtype=None):
    """x (T, D) fp32 <- weight * rms(alpha x + coef_a a + coef_b b) in place; returns the new x rounded to act_dtype if given."""
    t, d = x.shape
    xa = torch.empty((t, d), dtype=act_dtype, device=x.device) if act_dtype is not None else None
    _lib.call("zl_postnorm_combine", _p(x), d, alpha, _p(a), d, coef_a, _p(b), d, coef_b, _p(weight), _p(xa),
              _dt(xa) if xa is not None else BF16, t, d, eps, 0, _stream())
    return xa


def head_rmsnorm_gate_fn(o, heads, vdim, eps, weight=None, weight_head_stride=0, gate=None, gate_fn=GATE_SIGMOID,
                         out_dtype=torch.float32):
    t = o.shape[0]
    y = torch.empty((t, heads * vdim), dtype=out_dtype, device=o.device)
    _lib.call("zl_head_rmsnorm_gate_fn", _p(o), heads * vdim, _p(weight), weight_head_stride, _p(gate), heads * vdim, gate_fn, _p(y),
              heads * vdim, t, heads, vdim, eps, _dt(y), 0, _stream())
    return y


def gated_delta_rule(proj, col_qkv, col_rate, col_decay, conv_weight, a_log, dt_bias, unit_eps, q_scale, ring_table, run_row0,
                     run_len, slot, pos, state_table, heads, kv_heads, dim_k, dim_v):
    """proj (T, ld) fp32 (q | k | v from col_qkv, rate logits, decay inputs); states and rings are updated in place through
    their pointer tables.  -> o (T, heads * dim_v) fp32."""
    t, ld = proj.shape
    o = torch.empty((t, heads * dim_v), dtype=torch.float32, device=proj.device)
    nbytes = _lib.load().zl_delta_rule_workspace_bytes(t, heads, dim_k, dim_v)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=proj.device)
    _lib.call("zl_gated_delta_rule", _p(proj), ld, col_qkv, col_rate, col_decay, _p(conv_weight), conv_weight.shape[1], _p(a_log),
              _p(dt_bias), unit_eps, q_scale, _p(ring_table), _p(run_row0), _p(run_len), run_row0.numel(), _p(slot), _p(pos),
              _p(state_table), _p(o), heads * dim_v, heads, kv_heads, dim_k, dim_v, t, _p(ws), nbytes, 0, _stream())
    return o


def bonus_decay_scan(r, k, v, decay_logit, bonus, run_row0, run_len, slot, pos, state_table, heads, dim_k, dim_v):
    """r, k, decay_logit (T, heads * dim_k), v (T, heads * dim_v) fp32, bonus (heads, dim_k) fp32 -> o (T, heads * dim_v)."""
    t = r.shape[0]
    o = torch.empty((t, heads * dim_v), dtype=torch.float32, device=r.device)
    nbytes = _lib.load().zl_delta_rule_workspace_bytes(t, heads, dim_k, dim_v)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=r.device)
    _lib.call("zl_bonus_decay_scan", _p(r), heads * dim_k, _p(k), heads * dim_k, _p(v), heads * dim_v, _p(decay_logit),
              heads * dim_k, _p(bonus), _p(run_row0), _p(run_len), run_row0.numel(), _p(slot), _p(pos), _p(state_table), _p(o),
              heads * dim_v, heads, dim_k, dim_v, t, _p(ws), nbytes, 0, _stream())
    return o


# ------------------------------------------------------------------ parallel gated layers, rotated values, grouped routing
ROT_HALVES, ROT_ADJACENT = 0, 1


def gemm_nt_glu_clamp(x, w, bias=None, out_dtype=None, limit=1.0, alpha=1.0, beta=0.0):
    """y (M, N / 2) = g sigmoid(alpha g) (u + beta) over the column pairs (gate, up) of x @ w^T + bias, g = min(gate, limit),
    u = clamp(up, +-limit); w (N, K) with gate / up rows interleaved, bias (N) fp32 or None."""
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n // 2), dtype=out_dtype or x.dtype, device=x.device)
    _lib.call("zl_gemm_nt_glu_clamp", _p(x), k, _p(w), k, _p(bias), _p(y), n // 2, m, n, k, _dt(x), _dt(y), limit, alpha, beta, 0,
              _stream())
    return y


def moe_route_grouped(x, w_router, correction, top, groups=1, keep=1, score_fn=MOE_SCORE_SOFTMAX, renormalize=True,
                      renorm_eps=0.0):
    """moe_route with the choice restricted to the `keep` best of `groups` groups of neighbouring slots.  w_router None:
    x (T, slots) already holds the logits."""
    t, d = x.shape
    e = w_router.shape[0] if w_router is not None else d
    dev = x.device
    te = torch.empty((t, top), dtype=torch.int32, device=dev)
    tw = torch.empty((t, top), dtype=torch.float32, device=dev)
    off = torch.empty(e + 1, dtype=torch.int32, device=dev)
    lt = torch.empty(t * top, dtype=torch.int32, device=dev)
    lp = torch.empty(t * top, dtype=torch.int32, device=dev)
    _lib.call("zl_moe_route_grouped", _p(x), d, _p(w_router), _p(correction), _p(te), _p(tw), _p(off), _p(lt), _p(lp), t, d, e,
              top, groups, keep, score_fn, int(renormalize), renorm_eps, 0, _stream())
    return te, tw, off, lt, lp


def rope_table(pos, inv_freq):
    """pos (T) int32, inv_freq (half) float64 device tensors -> (T, half, 2) fp32 (cos, sin) of pos * inv_freq."""
    t, half = pos.numel(), inv_freq.numel()
    out = torch.empty((t, half, 2), dtype=torch.float32, device=pos.device)
    _lib.call("zl_rope_table", _p(pos), t, ctypes.cast(_p(inv_freq), ctypes.POINTER(ctypes.c_double)), half, _p(out), 0, _stream())
    return out


def qkv_table_rope_append(proj, q_off, k_off, v_off, heads, kv_heads, dim, vdim, qk_table, rot_dims, v_table, layout, k_slots,
                          v_slots, slot, pos, dtype):
    """proj (T, ld) fp32 -> q (T, heads * dim) of `dtype` turned by qk_table; keys (turned alike) and values (turned over vdim
    by v_table, None: as projected) go to rows (slot, pos) of the caches behind the slot tables unless k_off < 0."""
    t, ldp = proj.shape
    q = torch.empty((t, heads * dim), dtype=dtype, device=proj.device)
    _lib.call("zl_qkv_table_rope_append", _p(proj), ldp, q_off, k_off, v_off, heads, kv_heads, dim, vdim, _p(qk_table), rot_dims,
              _p(v_table), layout, _p(q), _p(k_slots), _p(v_slots), _p(slot), _p(pos), t, _dt(q), 0, _stream())
    return q


def sink_attention_ex(q, k_table, v_table, slot, pos, scale, heads, kv_heads, dim, vdim, sink=None, no_sink=False, gate=None,
                      chunk=0, dist_bias=None, out_table=None, out_layout=ROT_HALVES, splits=1, run_row0=None, run_len=None,
                      max_run_len=0):
    """sink_attention_local with an ordinary softmax (no_sink) and / or every head's output turned back by out_table
    ((T, vdim / 2, 2) fp32 from rope_table)."""
    t = q.shape[0]
    lib = _lib.load()
    nbytes = lib.zl_sink_attention_workspace_bytes(t, heads, vdim, splits)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    out = torch.empty((t, heads * vdim), dtype=q.dtype, device=q.device)
    _lib.call("zl_sink_attention_ex", _p(q), _p(k_table), _p(v_table), _p(slot), _p(pos), _p(sink), int(no_sink), _p(gate),
              gate.shape[1] if gate is not None else 0, scale, chunk, _p(dist_bias),
              dist_bias.shape[1] if dist_bias is not None else 0, _p(out_table), out_layout, _p(out), t, heads, kv_heads, dim, vdim,
              splits, _p(ws), nbytes, _p(run_row0), _p(run_len), run_row0.numel() if run_row0 is not None else 0, max_run_len,
              _dt(q), 0, _stream())
    return out


def gated_parallel_combine(x, mult, gates, ga_off, a, scale_a, eps, parts=None, coef=None, choice=None, n_real=0, f_dense=None,
                           gf_off=0, scale_f=None, norm_w=None, next_w=None, act_dtype=torch.float32):
    """x (T, D) fp32 += mult * (scale_a sigmoid(gates[:, ga_off:ga_off + D]) a + scale_f sigmoid(gates[:, gf_off:gf_off + D]) f),
    f = sum_p coef[:, p] * (parts[:, p], or norm_w * rms(x) where choice[:, p] >= n_real) + f_dense; parts (T, P, D) fp32.
    Returns next_w * rms(new x) in act_dtype when next_w is given."""
    t, d = x.shape
    n_parts = parts.shape[1] if parts is not None else 0
    h = torch.empty((t, d), dtype=act_dtype, device=x.device) if next_w is not None else None
    _lib.call("zl_gated_parallel_combine", _p(x), d, mult, _p(gates), gates.shape[1], _p(a), d, ga_off, _p(scale_a), _p(parts), d,
              _p(coef), _p(choice), n_parts, n_real, _p(f_dense), d, gf_off, _p(scale_f), _p(norm_w), _p(next_w), _p(h),
              _dt(h) if h is not None else F32, t, d, eps, 0, _stream())
    return h

// Host-side pieces shared by the model drivers (llama_runner.cu, dekipel_runner.cu, kodupel_runner.cu, ...): staged checkpoint tensors,
// device allocation helpers, and the slot cache -- the per-task, per-layer row buffers every driver appends to and
// its kernels reach through a device table of slot base pointers (the reference's per-task buffer tables,
// src/model/rag_buffer_context.h:141-181).
#pragma once
#include "common.cuh"

#include <cmath>
#include <map>
#include <string>
#include <vector>

namespace zl {

#define RCHECK(...)                   \
    do {                              \
        int _rc = (__VA_ARGS__);           \
        if (_rc != ZL_OK) return _rc; \
    } while (0)

inline int dmalloc(void** p, size_t bytes) {
    ZL_CHECK_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    return ZL_OK;
}

// a checkpoint tensor staged on the device until the load pipeline consumes it
struct Staged {
    void* ptr = nullptr;
    int rows = 0, cols = 0, elem = 0;
};
using StagedMap = std::map<std::string, Staged>;

inline const Staged* staged_find(const StagedMap& m, const std::string& name) {
    auto it = m.find(name);
    return it == m.end() ? nullptr : &it->second;
}
inline void staged_drop(StagedMap& m, const std::string& name) {
    auto it = m.find(name);
    if (it != m.end()) {
        cudaFree(it->second.ptr);
        m.erase(it);
    }
}
// copy a host tensor to the device and register it under `name` (replacing an earlier one); synchronous
inline int staged_load(StagedMap& m, const char* name, const void* data_host, int rows, int cols, int elem_bytes,
                       cudaStream_t stream) {
    Staged s;
    s.rows = rows;
    s.cols = cols;
    s.elem = elem_bytes;
    const size_t bytes = (size_t)rows * cols * elem_bytes;
    RCHECK(dmalloc(&s.ptr, bytes));
    ZL_CHECK_CUDA(cudaMemcpyAsync(s.ptr, data_host, bytes, cudaMemcpyHostToDevice, stream));
    ZL_CHECK_CUDA(cudaStreamSynchronize(stream));
    staged_drop(m, name);
    m[name] = s;
    return ZL_OK;
}

// frees device temporaries on every exit path of a load helper
struct DevTmp {
    std::vector<void*> ptrs;
    ~DevTmp() {
        for (void* p : ptrs)
            if (p) cudaFree(p);
    }
    int alloc(void** p, size_t bytes) {
        int rc = dmalloc(p, bytes);
        if (rc == ZL_OK) ptrs.push_back(*p);
        return rc;
    }
};

static __global__ void k_slot_table(void** tab, char* base, size_t stride, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) tab[i] = base + (size_t)i * stride;
}

// One row buffer per slot: (slots, rows_per_slot, row_bytes) in one allocation, zero-filled (rows never written must
// be finite: a masked key still meets an exact 0 weight), plus the device table of the slots' base pointers.  A slot
// that is given to a new sequence needs no clearing: a position is written before any token may see it.
struct SlotCache {
    void* buf = nullptr;
    void** addrs = nullptr;   // device (slots)
    size_t slot_bytes = 0;
    int slots = 0;
    int create(int n_slots, size_t bytes_per_slot, cudaStream_t stream) {
        slots = n_slots;
        slot_bytes = bytes_per_slot;
        RCHECK(dmalloc(&buf, slot_bytes * n_slots));
        ZL_CHECK_CUDA(cudaMemsetAsync(buf, 0, slot_bytes * n_slots, stream));
        RCHECK(dmalloc((void**)&addrs, sizeof(void*) * n_slots));
        k_slot_table<<<cdiv(n_slots, 256), 256, 0, stream>>>(addrs, (char*)buf, slot_bytes, n_slots);
        ZL_CHECK_LAUNCH();
        return ZL_OK;
    }
    void destroy() {
        if (buf) cudaFree(buf);
        if (addrs) cudaFree((void*)addrs);
        buf = nullptr;
        addrs = nullptr;
    }
};

// ---- pieces of a driver with an fp32 residual stream ------------------------------------------------------------------
// M is the driver's model struct: it has `staged`, `stream`, `weight_bytes`, `esz` (bytes of a weight element) and
// `cfg.dtype`.  The embedding gather multiplies by `scale` (1 for models without an embedding scale).
template <typename TS, typename TD>
__global__ void k_convert(const TS* __restrict__ src, TD* __restrict__ dst, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = from_f32<TD>(to_f32<TS>(src[i]));
}
template <typename TW>
__global__ void k_embed_f32(const int32_t* __restrict__ ids, const TW* __restrict__ table, float* __restrict__ out, int D,
                            int vocab, float scale) {
    pdl_trigger();
    pdl_wait();
    int id = ids[blockIdx.x];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int i = threadIdx.x; i < D; i += blockDim.x) out[(size_t)blockIdx.x * D + i] = to_f32<TW>(table[(size_t)id * D + i]) * scale;
}
static __global__ void k_gather_rows_f32(const float* __restrict__ src, const int32_t* __restrict__ rows, float* __restrict__ dst,
                                  int D) {
    pdl_trigger();
    pdl_wait();
    const float* s = src + (size_t)rows[blockIdx.x] * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[(size_t)blockIdx.x * D + i] = s[i];
}
static __global__ void k_decode_advance(int32_t* __restrict__ tokens, int32_t* __restrict__ pos, const int32_t* __restrict__ next,
                                 int B) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) {
        tokens[i] = next[i];
        pos[i] += 1;
    }
}
static __global__ void k_iota_i32(int32_t* a, int32_t* b, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = b[i] = i;
}

// staged (rows, cols) tensor of bfloat16 (elem 2) or float32 (elem 4) -> new device array of float / the activation type
template <typename TD, typename M>
int convert_to(M* m, const Staged* s, TD* dst, size_t n) {
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (s->elem == 2)
        k_convert<__nv_bfloat16, TD><<<blocks, 256, 0, m->stream>>>(static_cast<const __nv_bfloat16*>(s->ptr), dst, n);
    else
        k_convert<float, TD><<<blocks, 256, 0, m->stream>>>(static_cast<const float*>(s->ptr), dst, n);
    ZL_CHECK_LAUNCH();
    return ZL_OK;
}

template <typename M>
const Staged* need(M* m, const std::string& name, int rows, int cols) {
    const Staged* s = staged_find(m->staged, name);
    if (!s || (size_t)s->rows * s->cols != (size_t)rows * cols || (s->elem != 2 && s->elem != 4) ||
        (s->rows != rows && !(rows == 1 || cols == 1))) {
        zl_set_last_error(__FILE__, __LINE__, ("missing or ill-shaped tensor " + name).c_str());
        return nullptr;
    }
    return s;
}

template <typename M>
int take_f32(M* m, const std::string& name, int rows, int cols, float** out) {
    const Staged* s = need(m, name, rows, cols);
    if (!s) return ZL_ERR_STATE;
    const size_t n = (size_t)rows * cols;
    RCHECK(dmalloc((void**)out, n * 4));
    RCHECK(convert_to<float>(m, s, *out, n));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, name);
    m->weight_bytes += (double)n * 4;
    return ZL_OK;
}

// convert into dst (activation dtype) at element offset `off`
template <typename M>
int put_weight(M* m, const std::string& name, int rows, int cols, void* dst, size_t off) {
    const Staged* s = need(m, name, rows, cols);
    if (!s) return ZL_ERR_STATE;
    const size_t n = (size_t)rows * cols;
    if (m->cfg.dtype == ZL_F32)
        RCHECK(convert_to<float>(m, s, static_cast<float*>(dst) + off, n));
    else
        RCHECK(convert_to<__nv_bfloat16>(m, s, static_cast<__nv_bfloat16*>(dst) + off, n));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, name);
    m->weight_bytes += (double)n * m->esz;
    return ZL_OK;
}

template <typename M>
int take_weight(M* m, const std::string& name, int rows, int cols, void** out) {
    RCHECK(dmalloc(out, (size_t)rows * cols * m->esz));
    return put_weight(m, name, rows, cols, *out, 0);
}

template <typename M>
int stage_random(M* m, const std::string& name, int rows, int cols, float lo, float hi, uint64_t seed) {
    Staged s;
    s.rows = rows;
    s.cols = cols;
    s.elem = 2;
    const size_t n = (size_t)rows * cols;
    RCHECK(dmalloc(&s.ptr, n * 2));
    uint64_t h = seed;
    for (char ch : name) h = h * 1099511628211ull + (unsigned char)ch;
    RCHECK(zl_fill_uniform(s.ptr, n, lo, hi, h, ZL_BF16, m->stream));
    staged_drop(m->staged, name);
    m->staged[name] = s;
    return ZL_OK;
}


// ---- load helpers of drivers whose checkpoints keep norm weights around zero, biases per projection and gate / up pairs ---
static __global__ void k_add_const(float* w, int n, float v) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) w[i] += v;
}
// dst rows 2j / 2j+1 <- a row j / b row j; a, b are (rows, cols) each
template <typename TS, typename TD>
__global__ void k_interleave_pair_rows(const TS* __restrict__ a, const TS* __restrict__ b, TD* __restrict__ dst, int rows, int cols) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    const size_t j = i / cols, c = i % cols;
    dst[(2 * j) * cols + c] = from_f32<TD>(to_f32<TS>(a[i]));
    dst[(2 * j + 1) * cols + c] = from_f32<TD>(to_f32<TS>(b[i]));
}

// checkpoint norm tensor w -> fp32 array of the multipliers 1 + w
template <typename M>
int take_norm_plus_one(M* m, const std::string& name, int n, float** out) {
    RCHECK(take_f32(m, name, 1, n, out));
    k_add_const<<<cdiv(n, 256), 256, 0, m->stream>>>(*out, n, 1.0f);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

// bias segment `name` (n) -> fp32 bias array at offset off
template <typename M>
int put_bias_f32(M* m, const std::string& name, int n, float* dst, int off) {
    const Staged* s = need(m, name, 1, n);
    if (!s) return ZL_ERR_STATE;
    RCHECK(convert_to<float>(m, s, dst + off, (size_t)n));
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, name);
    return ZL_OK;
}

// fp32 bias -> a copy in the activation dtype (16-bit modes; checkpoint biases are 16-bit, so nothing is lost)
template <typename M>
int bias_copy_act(M* m, const float* src, int n, void** out) {
    if (m->cfg.dtype == ZL_F32) return ZL_OK;
    RCHECK(dmalloc(out, (size_t)n * 2));
    k_convert<float, __nv_bfloat16><<<cdiv(n, 256), 256, 0, m->stream>>>(src, static_cast<__nv_bfloat16*>(*out), (size_t)n);
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    return ZL_OK;
}

// tensors `a` and `b` (rows, cols) -> dst (2 * rows, cols) at element offset off with their rows interleaved (a gated unit's
// gate / up pairs as the GEMM epilogues want them); dst_f32: dst is fp32 whatever the activation dtype (biases)
template <typename M>
int put_interleaved(M* m, const std::string& a, const std::string& b, int rows, int cols, void* dst, size_t off, bool dst_f32) {
    const Staged* sa = need(m, a, rows, cols);
    const Staged* sb = need(m, b, rows, cols);
    if (!sa || !sb) return ZL_ERR_STATE;
    if (sa->elem != sb->elem) {
        zl_set_last_error(__FILE__, __LINE__, ("tensors of a pair differ in dtype: " + a).c_str());
        return ZL_ERR_STATE;
    }
    const size_t n = (size_t)rows * cols;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    const bool f32 = dst_f32 || m->cfg.dtype == ZL_F32;
    if (f32) {
        if (sa->elem == 2)
            k_interleave_pair_rows<<<blocks, 256, 0, m->stream>>>((const __nv_bfloat16*)sa->ptr, (const __nv_bfloat16*)sb->ptr,
                                                                  (float*)dst + off, rows, cols);
        else
            k_interleave_pair_rows<<<blocks, 256, 0, m->stream>>>((const float*)sa->ptr, (const float*)sb->ptr, (float*)dst + off, rows, cols);
    } else {
        if (sa->elem == 2)
            k_interleave_pair_rows<<<blocks, 256, 0, m->stream>>>((const __nv_bfloat16*)sa->ptr, (const __nv_bfloat16*)sb->ptr,
                                                                  (__nv_bfloat16*)dst + off, rows, cols);
        else
            k_interleave_pair_rows<<<blocks, 256, 0, m->stream>>>((const float*)sa->ptr, (const float*)sb->ptr,
                                                                  (__nv_bfloat16*)dst + off, rows, cols);
    }
    ZL_CHECK_LAUNCH();
    ZL_CHECK_CUDA(cudaStreamSynchronize(m->stream));
    staged_drop(m->staged, a);
    staged_drop(m->staged, b);
    if (!dst_f32) m->weight_bytes += 2.0 * n * m->esz;
    return ZL_OK;
}

}  // namespace zl

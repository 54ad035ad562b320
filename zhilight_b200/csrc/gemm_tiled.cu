// General tiled GEMM y[b](M,N) = epi(x[b](M,K) @ w[b](N,K)^T) for any M, N, K, with a batch of strided problems
// (one per attention head) and small fused epilogues: a per-column bias, relu^2, tanh, a sigmoid gate, the tanh form of
// gelu times a per-element multiplier, a tanh soft cap, and gated units over column pairs (columns 2j / 2j+1 hold
// gate / up, output column j): the clamped unit of expert feed-forwards and gelu_tanh(gate) * up.  Grouped mode serves
// mixtures of experts: problem b owns the rows grp_off[b] .. grp_off[b+1] of a list sorted by expert, input rows are
// gathered and output rows scattered through index lists, so one launch covers every expert of a step whatever
// the routing turned out to be (the counts stay on the device: the launch can sit in a CUDA graph).
//
// The decode-sized dense Linear of the framework (dense_gemm.cu) wants K % 32 == 0 and M <= 32 per pass and re-streams
// the weights for every 32 rows; models whose projection ranks are not multiples of 32, prompt-sized M, and per-head
// weight blocks go through this kernel instead.  16-bit inputs: 64 x 64 x 32 tiles, mma.sync.m16n8k16 with fp32
// accumulation, a three-stage cp.async pipeline, fragments through ldmatrix.  fp32 inputs: 64 x 64 x 16 tiles of plain FMAs (no TF32), every
// product and sum in IEEE fp32.
#include "common.cuh"

#include <cstdlib>

namespace zl {

struct GemmP {
    const void* x;
    const void* w;
    void* y;
    const float* gate;
    long long ldx, xb, ldw, wb, ldy, yb, ldg, gb;
    int M, N, K;
    const float* bias = nullptr;      // (batch, N) fp32, added before the epilogue
    long long bb = 0;
    const int32_t* grp_off = nullptr; // grouped mode: rows grp_off[b] .. grp_off[b+1] of the sorted list belong to problem b
    const int32_t* x_rows = nullptr;  // sorted index -> row of x (identity when null)
    const int32_t* y_rows = nullptr;  // sorted index -> row of y (identity when null)
    int act_tanh = 0;                 // few-rows kernel without the gated unit: tanh of the (biased) sum
    float limit = 0.f, alpha = 1.f, beta = 0.f;   // gated unit: g = min(gate, limit), u = clamp(up, +-limit), g sigmoid(alpha g) (u + beta)
                                      // soft cap: limit * tanh(v / limit)
    int pair_gelu = 0;                // few-rows kernel with a gated unit: gelu_tanh(gate) * up instead of the clamped unit
    int act_gelu_mul = 0;             // few-rows kernel without the gated unit: gelu_tanh of the (biased) sum times gate[m][n]
    int act_relu2 = 0;                // few-rows kernel without the gated unit: max(sum, 0)^2
};

__host__ __device__ constexpr bool epi_pairs(int epi) { return epi == ZL_GEMM_EPI_GLU_CLAMP || epi == ZL_GEMM_EPI_GEGLU_TANH; }


// rows of problem b and the place of its first row in the sorted list
__device__ __forceinline__ void gemm_rows_of(const GemmP& p, int b, int& rows, int& first) {
    if (p.grp_off) {
        first = p.grp_off[b];
        rows = p.grp_off[b + 1] - first;
    } else {
        first = 0;
        rows = p.M;
    }
}
__device__ __forceinline__ float glu_clamp(float gate, float up, const GemmP& p) {
    const float g = fminf(gate, p.limit), u = fminf(fmaxf(up, -p.limit), p.limit);
    return g * (1.0f / (1.0f + expf(-p.alpha * g))) * (u + p.beta);
}

template <int EPI>
__device__ __forceinline__ float pair_unit(float gate, float up, const GemmP& p) {
    if constexpr (EPI == ZL_GEMM_EPI_GEGLU_TANH) return gelu_f(gate) * up;
    else return glu_clamp(gate, up, p);
}

template <int EPI>
__device__ __forceinline__ float gemm_epilogue(float v, const GemmP& p, int b, int m, int n) {
    if constexpr (EPI == ZL_GEMM_EPI_RELU2) {
        const float r = fmaxf(v, 0.f);
        return r * r;
    } else if constexpr (EPI == ZL_GEMM_EPI_SIGMOID_GATE) {
        const float g = p.gate[(size_t)b * p.gb + (size_t)m * p.ldg + n];
        return v * (1.0f / (1.0f + expf(-g)));
    } else if constexpr (EPI == ZL_GEMM_EPI_TANH) {
        return tanhf(v);
    } else if constexpr (EPI == ZL_GEMM_EPI_GELU_TANH_MUL) {
        return gelu_f(v) * p.gate[(size_t)b * p.gb + (size_t)m * p.ldg + n];
    } else if constexpr (EPI == ZL_GEMM_EPI_SOFTCAP) {
        return p.limit * tanhf(v / p.limit);
    } else {
        return v;
    }
}

// ---- 16-bit inputs -------------------------------------------------------------------------------------------------
constexpr int kGB = 64, kGK = 32, kGPad = 8;

template <typename T>
__device__ __forceinline__ uint4 load8(const T* base, long long ld, int row, int rows, int k, int K, bool vec) {
    uint4 r = make_uint4(0, 0, 0, 0);
    if (row >= rows || k >= K) return r;
    const T* p = base + (size_t)row * ld + k;
    if (vec) return *reinterpret_cast<const uint4*>(p);   // vec implies K % 8 == 0: the 8 elements are inside the row
    T* e = reinterpret_cast<T*>(&r);
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (k + i < K) e[i] = p[i];
    return r;
}

template <typename T>
__device__ __forceinline__ void mma_in(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_in<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    mma_16816_f16(d, a, b0, b1, d);
}
template <>
__device__ __forceinline__ void mma_in<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    mma_16816_bf16(d, a, b0, b1, d);
}

constexpr int kGStages = 3;

__device__ __forceinline__ void g_cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void g_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void g_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void g_ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}

// one 64 x 32 tile into shared memory from the two row pointers of this thread (null: a row beyond the matrix): 16-byte
// cp.async pieces when the layout allows, guarded element loads otherwise; rows / k beyond the matrix become zeros
template <typename T>
__device__ __forceinline__ void stage_tile(T (*dst)[kGK + kGPad], const T* const (&rowp)[2], int k0, int K, bool vec, int lr,
                                           int lc) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = lr + half * 32, k = k0 + lc;
        if (vec && rowp[half] && k < K) g_cp_async16(&dst[r][lc], rowp[half] + k);
        else *reinterpret_cast<uint4*>(&dst[r][lc]) = load8(rowp[half], 0, 0, rowp[half] ? 1 : 0, k, K, false);
    }
}

template <typename T, typename TO, int EPI>
__global__ void __launch_bounds__(128) k_gemm_mma(GemmP p, int vec_x, int vec_w) {
    __shared__ __align__(16) T sA[kGStages][kGB][kGK + kGPad];
    __shared__ __align__(16) T sB[kGStages][kGB][kGK + kGPad];
    pdl_trigger();
    const int b = blockIdx.z;
    const T* x = static_cast<const T*>(p.x) + (size_t)b * p.xb;
    const T* w = static_cast<const T*>(p.w) + (size_t)b * p.wb;
    const int m0 = blockIdx.y * kGB, n0 = blockIdx.x * kGB;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int lr = tid >> 2, lc = (tid & 3) * 8;   // this thread's 8-element pieces: rows lr and lr + 32
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const T* wrow[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) wrow[half] = n0 + lr + half * 32 < p.N ? w + (size_t)(n0 + lr + half * 32) * p.ldw : nullptr;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

    const int steps = cdiv(p.K, kGK);
    pdl_wait();
    int M, first;
    gemm_rows_of(p, b, M, first);   // the index lists are a predecessor's output: read after the wait
    if (m0 >= M) return;
    const T* xrow[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int m = m0 + lr + half * 32;
        xrow[half] = m < M ? x + (size_t)(p.x_rows ? p.x_rows[first + m] : first + m) * p.ldx : nullptr;
    }
    for (int s = 0; s < kGStages - 1; ++s) {
        if (s < steps) {
            stage_tile<T>(sA[s], xrow, s * kGK, p.K, vec_x, lr, lc);
            stage_tile<T>(sB[s], wrow, s * kGK, p.K, vec_w, lr, lc);
        }
        g_cp_commit();
    }
    for (int s = 0; s < steps; ++s) {
        const int buf = s % kGStages;
        g_cp_wait<kGStages - 2>();   // tile s has landed (one younger group may still fly)
        __syncthreads();             // ... for every thread; and every warp is done with tile s - 1, whose buffer is refilled now
        if (s + kGStages - 1 < steps) {
            const int nb = (s + kGStages - 1) % kGStages, k0 = (s + kGStages - 1) * kGK;
            stage_tile<T>(sA[nb], xrow, k0, p.K, vec_x, lr, lc);
            stage_tile<T>(sB[nb], wrow, k0, p.K, vec_w, lr, lc);
        }
        g_cp_commit();
#pragma unroll
        for (int kk = 0; kk < kGK; kk += 16) {
            uint32_t a[2][4], bq[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) g_ldmatrix_x4(a[i], &sA[buf][wm + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj)   // two 8-column tiles per ldmatrix: {b0, b1} of tile 2jj, {b0, b1} of tile 2jj + 1
                g_ldmatrix_x4(bq[jj], &sB[buf][wn + jj * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                mma_in<T>(acc[0][j], a[0], bq[j >> 1][(j & 1) * 2], bq[j >> 1][(j & 1) * 2 + 1]);
                mma_in<T>(acc[1][j], a[1], bq[j >> 1][(j & 1) * 2], bq[j >> 1][(j & 1) * 2 + 1]);
            }
        }
    }
    TO* y = static_cast<TO*>(p.y) + (size_t)b * p.yb;
    const float* bias = p.bias ? p.bias + (size_t)b * p.bb : nullptr;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int m = m0 + wm + i * 16 + g + hh * 8;
            if (m >= M) continue;
            const size_t yr = (size_t)(p.y_rows ? p.y_rows[first + m] : first + m) * p.ldy;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + wn + j * 8 + 2 * t;
                float v0 = acc[i][j][hh * 2], v1 = acc[i][j][hh * 2 + 1];
                if (bias) {
                    if (n < p.N) v0 += bias[n];
                    if (n + 1 < p.N) v1 += bias[n + 1];
                }
                if constexpr (epi_pairs(EPI)) {
                    if (n + 1 < p.N) y[yr + (n >> 1)] = from_f32<TO>(pair_unit<EPI>(v0, v1, p));
                } else {
                    if (n < p.N) y[yr + n] = from_f32<TO>(gemm_epilogue<EPI>(v0, p, b, m, n));
                    if (n + 1 < p.N) y[yr + n + 1] = from_f32<TO>(gemm_epilogue<EPI>(v1, p, b, m, n + 1));
                }
            }
        }
}


// ---- decode-sized M, 16-bit inputs -----------------------------------------------------------------------------------
// y[b](M <= 8, N) for many small per-head weight blocks: one warp per output column n streams w[b][n][:] once with
// 16-byte loads and multiplies it with all M rows of x[b], which the CTA holds in shared memory.  fp32 accumulation,
// warp-shuffle reduction.  grid (ceil(N / 32), batch), 8 warps, 4 columns per warp.
constexpr int kSmCols = 32;

template <typename T, typename TO, int EPI, int MT>
__global__ void __launch_bounds__(256) k_gemm_small_m(GemmP p) {
    extern __shared__ __align__(16) unsigned char sx_raw[];
    T* sx = reinterpret_cast<T*>(sx_raw);   // [M][K]
    pdl_trigger();
    const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* w = static_cast<const T*>(p.w) + (size_t)b * p.wb;
    const T* x = static_cast<const T*>(p.x) + (size_t)b * p.xb;
    const int K = p.K, K8 = K / 8;
    pdl_wait();
    for (int i = threadIdx.x; i < p.M * K8; i += blockDim.x) {
        const int m = i / K8, k8 = i - m * K8;
        *reinterpret_cast<uint4*>(sx + (size_t)m * K + k8 * 8) = *reinterpret_cast<const uint4*>(x + (size_t)m * p.ldx + k8 * 8);
    }
    __syncthreads();
    for (int n = blockIdx.x * kSmCols + warp; n < min(p.N, (int)(blockIdx.x + 1) * kSmCols); n += 8) {
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.f;
        const T* wr = w + (size_t)n * p.ldw;
        for (int k8 = lane; k8 < K8; k8 += 128) {   // four 16-byte loads of the weight row in flight per lane
            uint4 wq[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) wq[u] = k8 + 32 * u < K8 ? ld_nc_na_u4(wr + (size_t)(k8 + 32 * u) * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (k8 + 32 * u >= K8) break;
                float wf[8];
                unpack8<T>(wq[u], wf);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    if (m < p.M) {
                        float xf[8];
                        unpack8<T>(*reinterpret_cast<const uint4*>(sx + (size_t)m * K + (size_t)(k8 + 32 * u) * 8), xf);
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[m] = fmaf(wf[e], xf[e], acc[m]);
                    }
                }
            }
        }
        float mine = 0.f;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float v = warp_sum(acc[m]);
            if (lane == m) mine = v;
        }
        if (lane < p.M) {
            TO* y = static_cast<TO*>(p.y) + (size_t)b * p.yb;
            if (p.bias) mine += p.bias[(size_t)b * p.bb + n];
            y[(size_t)lane * p.ldy + n] = from_f32<TO>(gemm_epilogue<EPI>(mine, p, b, lane, n));
        }
    }
}

template <typename T, typename TO, int EPI>
static cudaError_t launch_small_m_mt(const GemmP& p, int batch, bool pdl, cudaStream_t st) {
    const dim3 grid(cdiv(p.N, kSmCols), batch), block(256);
    const size_t smem = (size_t)p.M * p.K * sizeof(T);
    if (p.M <= 2) return launch(k_gemm_small_m<T, TO, EPI, 2>, grid, block, smem, st, pdl, p);
    if (p.M <= 4) return launch(k_gemm_small_m<T, TO, EPI, 4>, grid, block, smem, st, pdl, p);
    return launch(k_gemm_small_m<T, TO, EPI, 8>, grid, block, smem, st, pdl, p);
}
template <typename T, typename TO>
static cudaError_t launch_small_m(const GemmP& p, int batch, int epi, bool pdl, cudaStream_t st) {
    if (epi == ZL_GEMM_EPI_RELU2) return launch_small_m_mt<T, TO, ZL_GEMM_EPI_RELU2>(p, batch, pdl, st);
    if (epi == ZL_GEMM_EPI_SIGMOID_GATE) return launch_small_m_mt<T, TO, ZL_GEMM_EPI_SIGMOID_GATE>(p, batch, pdl, st);
    if (epi == ZL_GEMM_EPI_TANH) return launch_small_m_mt<T, TO, ZL_GEMM_EPI_TANH>(p, batch, pdl, st);
    if (epi == ZL_GEMM_EPI_GELU_TANH_MUL) return launch_small_m_mt<T, TO, ZL_GEMM_EPI_GELU_TANH_MUL>(p, batch, pdl, st);
    if (epi == ZL_GEMM_EPI_SOFTCAP) return launch_small_m_mt<T, TO, ZL_GEMM_EPI_SOFTCAP>(p, batch, pdl, st);
    return launch_small_m_mt<T, TO, ZL_GEMM_EPI_NONE>(p, batch, pdl, st);
}

// ---- grouped problems with few rows each (decode steps of a mixture of experts) ----------------------------------------
// One CTA = 8 output columns of one group with the gated unit, 16 without, one or two per warp; the group's rows (gathered
// through x_rows) sit in shared memory eight at a time, and a warp streams two weight rows at once -- the gate and the up
// row of its column, or the rows of its two columns -- once per eight rows with four 16-byte loads per row in flight.
// Groups without rows cost an early exit.
constexpr int kGrpCols = 8;

template <typename T, typename TO, bool GLU>
__global__ void __launch_bounds__(256) k_gemm_grouped_small(GemmP p) {
    extern __shared__ __align__(16) unsigned char sx_raw[];
    T* sx = reinterpret_cast<T*>(sx_raw);   // [8][K]
    pdl_trigger();
    const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* w = static_cast<const T*>(p.w) + (size_t)b * p.wb;
    const T* x = static_cast<const T*>(p.x);
    TO* y = static_cast<TO*>(p.y);
    const int K = p.K, K8 = K / 8, n_out = GLU ? p.N / 2 : p.N;
    // a warp streams two weight rows at once: gate and up of its column (gated unit), or the rows of two columns
    // (8 apart) otherwise, so that eight 16-byte loads per lane are in flight either way
    constexpr int kCols = GLU ? kGrpCols : 2 * kGrpCols;
    const int n = blockIdx.x * kCols + warp, n2 = GLU ? n : n + kGrpCols;
    const bool has1 = n < n_out, has2 = GLU ? has1 : n2 < n_out;
    pdl_wait();
    int M, first;
    gemm_rows_of(p, b, M, first);
    for (int m0 = 0; m0 < M; m0 += 8) {
        const int mc = min(8, M - m0);
        __syncthreads();   // the previous eight rows are no longer read
        for (int i = threadIdx.x; i < mc * K8; i += blockDim.x) {
            const int m = i / K8, k8 = i - m * K8;
            const size_t row = p.x_rows ? p.x_rows[first + m0 + m] : first + m0 + m;
            *reinterpret_cast<uint4*>(sx + (size_t)m * K + k8 * 8) = *reinterpret_cast<const uint4*>(x + row * p.ldx + k8 * 8);
        }
        __syncthreads();
        if (!has1) continue;
        float acc[8], acc2[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) acc[m] = acc2[m] = 0.f;
        const T* wr = w + (size_t)(GLU ? 2 * n : n) * p.ldw;
        const T* wr2 = GLU ? wr + p.ldw : w + (size_t)(has2 ? n2 : n) * p.ldw;
        for (int k8 = lane; k8 < K8; k8 += 128) {
            uint4 wq[4], wq2[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const bool in = k8 + 32 * u < K8;
                wq[u] = in ? ld_nc_na_u4(wr + (size_t)(k8 + 32 * u) * 8) : make_uint4(0, 0, 0, 0);
                wq2[u] = (in && has2) ? ld_nc_na_u4(wr2 + (size_t)(k8 + 32 * u) * 8) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (k8 + 32 * u >= K8) break;
                float wf[8], wf2[8];
                unpack8<T>(wq[u], wf);
                unpack8<T>(wq2[u], wf2);
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    if (m < mc) {
                        float xf[8];
                        unpack8<T>(*reinterpret_cast<const uint4*>(sx + (size_t)m * K + (size_t)(k8 + 32 * u) * 8), xf);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            acc[m] = fmaf(wf[e], xf[e], acc[m]);
                            acc2[m] = fmaf(wf2[e], xf[e], acc2[m]);
                        }
                    }
                }
            }
        }
        float mine = 0.f, mine2 = 0.f;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            float v = warp_sum(acc[m]), v2 = warp_sum(acc2[m]);
            if (GLU) {
                if (p.bias) v += p.bias[(size_t)b * p.bb + 2 * n], v2 += p.bias[(size_t)b * p.bb + 2 * n + 1];
                v = p.pair_gelu ? gelu_f(v) * v2 : glu_clamp(v, v2, p);
            } else {
                if (p.bias) v += p.bias[(size_t)b * p.bb + n], v2 += has2 ? p.bias[(size_t)b * p.bb + n2] : 0.f;
                if (p.act_tanh) v = tanhf(v), v2 = tanhf(v2);
                if (p.act_relu2) v = fmaxf(v, 0.f), v *= v, v2 = fmaxf(v2, 0.f), v2 *= v2;
                if (p.act_gelu_mul && m < mc) {
                    const float* gr = p.gate + (size_t)(first + m0 + m) * p.ldg;
                    v = gelu_f(v) * gr[n];
                    v2 = has2 ? gelu_f(v2) * gr[n2] : 0.f;
                }
            }
            if (lane == m) mine = v, mine2 = v2;
        }
        if (lane < mc) {
            const size_t yr = (size_t)(p.y_rows ? p.y_rows[first + m0 + lane] : first + m0 + lane) * p.ldy;
            y[yr + n] = from_f32<TO>(mine);
            if (!GLU && has2) y[yr + n2] = from_f32<TO>(mine2);
        }
    }
}

template <typename T, typename TO>
static cudaError_t launch_grouped_small(const GemmP& p, int groups, bool glu, bool pdl, cudaStream_t st) {
    const dim3 grid(glu ? cdiv(p.N / 2, kGrpCols) : cdiv(p.N, 2 * kGrpCols), groups), block(256);
    const size_t smem = (size_t)8 * p.K * sizeof(T);
    cudaError_t e = cudaSuccess;
    static size_t set_glu = 0, set_plain = 0;
    size_t& set_for = glu ? set_glu : set_plain;
    if (smem > 48 * 1024 && smem > set_for) {
        e = glu ? cudaFuncSetAttribute(k_gemm_grouped_small<T, TO, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                : cudaFuncSetAttribute(k_gemm_grouped_small<T, TO, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        set_for = smem;
    }
    return glu ? launch(k_gemm_grouped_small<T, TO, true>, grid, block, smem, st, pdl, p)
               : launch(k_gemm_grouped_small<T, TO, false>, grid, block, smem, st, pdl, p);
}

// ---- fp32 inputs ---------------------------------------------------------------------------------------------------
constexpr int kFK = 16;

__device__ __forceinline__ float4 load4f(const float* rowp, int k, int K, bool vec) {
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!rowp || k >= K) return r;
    const float* p = rowp + k;
    if (vec) return *reinterpret_cast<const float4*>(p);
    r.x = p[0];
    if (k + 1 < K) r.y = p[1];
    if (k + 2 < K) r.z = p[2];
    if (k + 3 < K) r.w = p[3];
    return r;
}

template <int EPI>
__global__ void __launch_bounds__(256) k_gemm_f32(GemmP p, int vec_x, int vec_w) {
    __shared__ float sA[kFK][kGB + 4];   // k-major: the inner product walks k, 4 rows / columns per thread
    __shared__ float sB[kFK][kGB + 4];
    pdl_trigger();
    const int b = blockIdx.z;
    const float* x = static_cast<const float*>(p.x) + (size_t)b * p.xb;
    const float* w = static_cast<const float*>(p.w) + (size_t)b * p.wb;
    const int m0 = blockIdx.y * kGB, n0 = blockIdx.x * kGB;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int lr = tid >> 2, lc = (tid & 3) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const float* wrow = n0 + lr < p.N ? w + (size_t)(n0 + lr) * p.ldw : nullptr;
    float4 rw = load4f(wrow, lc, p.K, vec_w);
    pdl_wait();
    int M, first;
    gemm_rows_of(p, b, M, first);
    if (m0 >= M) return;
    const float* xrow = m0 + lr < M ? x + (size_t)(p.x_rows ? p.x_rows[first + m0 + lr] : first + m0 + lr) * p.ldx : nullptr;
    float4 rx = load4f(xrow, lc, p.K, vec_x);
    const int steps = cdiv(p.K, kFK);
    for (int s = 0; s < steps; ++s) {
        __syncthreads();   // the previous step's reads are done
        sA[lc + 0][lr] = rx.x, sA[lc + 1][lr] = rx.y, sA[lc + 2][lr] = rx.z, sA[lc + 3][lr] = rx.w;
        sB[lc + 0][lr] = rw.x, sB[lc + 1][lr] = rw.y, sB[lc + 2][lr] = rw.z, sB[lc + 3][lr] = rw.w;
        __syncthreads();
        if (s + 1 < steps) {
            const int k = (s + 1) * kFK + lc;
            rx = load4f(xrow, k, p.K, vec_x);
            rw = load4f(wrow, k, p.K, vec_w);
        }
#pragma unroll
        for (int k = 0; k < kFK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&sA[k][ty * 4]);
            const float4 bb = *reinterpret_cast<const float4*>(&sB[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
    float* y = static_cast<float*>(p.y) + (size_t)b * p.yb;
    const float* bias = p.bias ? p.bias + (size_t)b * p.bb : nullptr;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
        const size_t yr = (size_t)(p.y_rows ? p.y_rows[first + m] : first + m) * p.ldy;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (bias && n < p.N) acc[i][j] += bias[n];
        }
        if constexpr (epi_pairs(EPI)) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < p.N) y[yr + (n >> 1)] = pair_unit<EPI>(acc[i][j], acc[i][j + 1], p);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + tx * 4 + j;
                if (n < p.N) y[yr + n] = gemm_epilogue<EPI>(acc[i][j], p, b, m, n);
            }
        }
    }
}

template <typename T, typename TO>
static cudaError_t launch_mma(const GemmP& p, int batch, int epi, bool vx, bool vw, bool pdl, cudaStream_t st) {
    const dim3 grid(cdiv(p.N, kGB), cdiv(p.M, kGB), batch), block(128);
    if (epi == ZL_GEMM_EPI_RELU2) return launch(k_gemm_mma<T, TO, ZL_GEMM_EPI_RELU2>, grid, block, 0, st, pdl, p, (int)vx, (int)vw);
    if (epi == ZL_GEMM_EPI_SIGMOID_GATE)
        return launch(k_gemm_mma<T, TO, ZL_GEMM_EPI_SIGMOID_GATE>, grid, block, 0, st, pdl, p, (int)vx, (int)vw);
    if (epi == ZL_GEMM_EPI_TANH) return launch(k_gemm_mma<T, TO, ZL_GEMM_EPI_TANH>, grid, block, 0, st, pdl, p, (int)vx, (int)vw);
    if (epi == ZL_GEMM_EPI_GLU_CLAMP)
        return launch(k_gemm_mma<T, TO, ZL_GEMM_EPI_GLU_CLAMP>, grid, block, 0, st, pdl, p, (int)vx, (int)vw);
    if (epi == ZL_GEMM_EPI_GEGLU_TANH)
        return launch(k_gemm_mma<T, TO, ZL_GEMM_EPI_GEGLU_TANH>, grid, block, 0, st, pdl, p, (int)vx, (int)vw);
    if (epi == ZL_GEMM_EPI_GELU_TANH_MUL)
        return launch(k_gemm_mma<T, TO, ZL_GEMM_EPI_GELU_TANH_MUL>, grid, block, 0, st, pdl, p, (int)vx, (int)vw);
    if (epi == ZL_GEMM_EPI_SOFTCAP)
        return launch(k_gemm_mma<T, TO, ZL_GEMM_EPI_SOFTCAP>, grid, block, 0, st, pdl, p, (int)vx, (int)vw);
    return launch(k_gemm_mma<T, TO, ZL_GEMM_EPI_NONE>, grid, block, 0, st, pdl, p, (int)vx, (int)vw);
}

static bool aligned_for(const void* ptr, long long ld, long long bstride, int K, int elem, int batch) {
    const int per16 = 16 / elem;
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && ld % per16 == 0 && K % per16 == 0 &&
           (batch == 1 || bstride % per16 == 0);
}

}  // namespace zl

using namespace zl;

// row count of a step up to which grouped problems take the few-rows kernel (ZL_GEMM_GROUPED_SMALL_MAX overrides)
static int grouped_small_max() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("ZL_GEMM_GROUPED_SMALL_MAX");
        v = e ? atoi(e) : 8;
    }
    return v;
}

static int gemm_dispatch(GemmP p, int batch, int in_dtype, int out_dtype, int epilogue, int pdl, cudaStream_t stream) {
    const int M = p.M, N = p.N, K = p.K;
    const bool grouped = p.grp_off != nullptr, pairs = epi_pairs(epilogue);
    ZL_CHECK_ARG(p.x && p.w && p.y && M > 0 && N > 0 && K > 0 && batch > 0 && batch <= 65535);
    ZL_CHECK_ARG(p.ldx >= K && p.ldw >= K && p.ldy >= (pairs ? N / 2 : N));
    ZL_CHECK_ARG(in_dtype == ZL_F16 || in_dtype == ZL_BF16 || in_dtype == ZL_F32);
    ZL_CHECK_ARG(out_dtype == in_dtype || out_dtype == ZL_F32);
    ZL_CHECK_ARG(epilogue >= ZL_GEMM_EPI_NONE && epilogue <= ZL_GEMM_EPI_SOFTCAP);
    const bool gated = epilogue == ZL_GEMM_EPI_SIGMOID_GATE || epilogue == ZL_GEMM_EPI_GELU_TANH_MUL;
    ZL_CHECK_ARG(!gated || (p.gate && p.ldg >= N && !grouped));
    ZL_CHECK_ARG(epilogue != ZL_GEMM_EPI_SOFTCAP || p.limit > 0.f);
    ZL_CHECK_ARG(!pairs || N % 2 == 0);
    ZL_CHECK_ARG(grouped || (!p.x_rows && !p.y_rows));
    ZL_CHECK_ARG(cdiv(M, kGB) <= 65535 && cdiv(N, kSmCols) <= 2147483647);
    const int elem = in_dtype == ZL_F32 ? 4 : 2;
    // gathered rows start at any multiple of ldx: the batch stride plays no part in their alignment
    const bool vx = aligned_for(p.x, p.ldx, p.xb, K, elem, batch), vw = aligned_for(p.w, p.ldw, p.wb, K, elem, batch);
    cudaError_t e;
    if (in_dtype == ZL_F32) {
        const dim3 grid(cdiv(N, kGB), cdiv(M, kGB), batch), block(256);
        if (epilogue == ZL_GEMM_EPI_RELU2)
            e = launch(k_gemm_f32<ZL_GEMM_EPI_RELU2>, grid, block, 0, stream, pdl != 0, p, (int)vx, (int)vw);
        else if (epilogue == ZL_GEMM_EPI_SIGMOID_GATE)
            e = launch(k_gemm_f32<ZL_GEMM_EPI_SIGMOID_GATE>, grid, block, 0, stream, pdl != 0, p, (int)vx, (int)vw);
        else if (epilogue == ZL_GEMM_EPI_TANH)
            e = launch(k_gemm_f32<ZL_GEMM_EPI_TANH>, grid, block, 0, stream, pdl != 0, p, (int)vx, (int)vw);
        else if (epilogue == ZL_GEMM_EPI_GLU_CLAMP)
            e = launch(k_gemm_f32<ZL_GEMM_EPI_GLU_CLAMP>, grid, block, 0, stream, pdl != 0, p, (int)vx, (int)vw);
        else if (epilogue == ZL_GEMM_EPI_GEGLU_TANH)
            e = launch(k_gemm_f32<ZL_GEMM_EPI_GEGLU_TANH>, grid, block, 0, stream, pdl != 0, p, (int)vx, (int)vw);
        else if (epilogue == ZL_GEMM_EPI_GELU_TANH_MUL)
            e = launch(k_gemm_f32<ZL_GEMM_EPI_GELU_TANH_MUL>, grid, block, 0, stream, pdl != 0, p, (int)vx, (int)vw);
        else if (epilogue == ZL_GEMM_EPI_SOFTCAP)
            e = launch(k_gemm_f32<ZL_GEMM_EPI_SOFTCAP>, grid, block, 0, stream, pdl != 0, p, (int)vx, (int)vw);
        else
            e = launch(k_gemm_f32<ZL_GEMM_EPI_NONE>, grid, block, 0, stream, pdl != 0, p, (int)vx, (int)vw);
    } else if (grouped && M <= grouped_small_max() && vx && vw && K % 8 == 0 && (size_t)8 * K * 2 <= 160 * 1024 &&
               (epilogue == ZL_GEMM_EPI_NONE || epilogue == ZL_GEMM_EPI_RELU2 || pairs)) {   // a decode step's experts: a handful of rows per group
        p.act_relu2 = epilogue == ZL_GEMM_EPI_RELU2;
        if (in_dtype == ZL_BF16)
            e = out_dtype == ZL_F32 ? launch_grouped_small<__nv_bfloat16, float>(p, batch, pairs, pdl != 0, stream)
                                    : launch_grouped_small<__nv_bfloat16, __nv_bfloat16>(p, batch, pairs, pdl != 0, stream);
        else
            e = out_dtype == ZL_F32 ? launch_grouped_small<__half, float>(p, batch, pairs, pdl != 0, stream)
                                    : launch_grouped_small<__half, __half>(p, batch, pairs, pdl != 0, stream);
    } else if (!grouped && pairs && batch == 1 && M <= 8 && vx && vw && K % 8 == 0 &&
               (size_t)8 * K * 2 <= 160 * 1024) {   // a dense gated feed-forward of a decode step: gate and up rows streamed together
        p.pair_gelu = epilogue == ZL_GEMM_EPI_GEGLU_TANH;
        if (in_dtype == ZL_BF16)
            e = out_dtype == ZL_F32 ? launch_grouped_small<__nv_bfloat16, float>(p, 1, true, pdl != 0, stream)
                                    : launch_grouped_small<__nv_bfloat16, __nv_bfloat16>(p, 1, true, pdl != 0, stream);
        else
            e = out_dtype == ZL_F32 ? launch_grouped_small<__half, float>(p, 1, true, pdl != 0, stream)
                                    : launch_grouped_small<__half, __half>(p, 1, true, pdl != 0, stream);
    } else if (!grouped && (epilogue == ZL_GEMM_EPI_TANH || epilogue == ZL_GEMM_EPI_GELU_TANH_MUL) && batch == 1 &&
               M <= 8 && vx && vw && K % 8 == 0 && (size_t)8 * K * 2 <= 160 * 1024) {
        // a narrow tanh / gelu-times-multiplier projection of a decode step: one column per warp, loads in flight.  (With more
        // than 8 rows the kernel re-streams the weights per 8 rows and measured slower than the tile kernel.)
        p.act_tanh = epilogue == ZL_GEMM_EPI_TANH;
        p.act_gelu_mul = epilogue == ZL_GEMM_EPI_GELU_TANH_MUL;
        if (in_dtype == ZL_BF16)
            e = out_dtype == ZL_F32 ? launch_grouped_small<__nv_bfloat16, float>(p, 1, false, pdl != 0, stream)
                                    : launch_grouped_small<__nv_bfloat16, __nv_bfloat16>(p, 1, false, pdl != 0, stream);
        else
            e = out_dtype == ZL_F32 ? launch_grouped_small<__half, float>(p, 1, false, pdl != 0, stream)
                                    : launch_grouped_small<__half, __half>(p, 1, false, pdl != 0, stream);
    } else if (!grouped && !pairs && M <= 8 && vx && vw && (size_t)M * K * 2 <= 48 * 1024) {   // few rows: stream the weights once per column
        if (in_dtype == ZL_BF16)
            e = out_dtype == ZL_F32 ? launch_small_m<__nv_bfloat16, float>(p, batch, epilogue, pdl != 0, stream)
                                    : launch_small_m<__nv_bfloat16, __nv_bfloat16>(p, batch, epilogue, pdl != 0, stream);
        else
            e = out_dtype == ZL_F32 ? launch_small_m<__half, float>(p, batch, epilogue, pdl != 0, stream)
                                    : launch_small_m<__half, __half>(p, batch, epilogue, pdl != 0, stream);
    } else if (in_dtype == ZL_BF16) {
        e = out_dtype == ZL_F32 ? launch_mma<__nv_bfloat16, float>(p, batch, epilogue, vx, vw, pdl != 0, stream)
                                : launch_mma<__nv_bfloat16, __nv_bfloat16>(p, batch, epilogue, vx, vw, pdl != 0, stream);
    } else {
        e = out_dtype == ZL_F32 ? launch_mma<__half, float>(p, batch, epilogue, vx, vw, pdl != 0, stream)
                                : launch_mma<__half, __half>(p, batch, epilogue, vx, vw, pdl != 0, stream);
    }
    ZL_CHECK_CUDA(e);
    return ZL_OK;
}

extern "C" int zl_gemm_nt(const void* x, long long ldx, long long x_batch_stride, const void* w, long long ldw,
                          long long w_batch_stride, void* y, long long ldy, long long y_batch_stride, int M, int N, int K,
                          int batch, int in_dtype, int out_dtype, int epilogue, const float* gate, long long ldg,
                          long long gate_batch_stride, int pdl, zl_stream_t stream) {
    ZL_CHECK_ARG(!epi_pairs(epilogue) && epilogue != ZL_GEMM_EPI_SOFTCAP);
    GemmP p{x, w, y, gate, ldx, x_batch_stride, ldw, w_batch_stride, ldy, y_batch_stride, ldg, gate_batch_stride, M, N, K};
    return gemm_dispatch(p, batch, in_dtype, out_dtype, epilogue, pdl, stream);
}

extern "C" int zl_gemm_nt_fused(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y,
                                long long ldy, int M, int N, int K, int in_dtype, int out_dtype, int epilogue,
                                const float* mul, long long ld_mul, float limit, int pdl, zl_stream_t stream) {
    GemmP p{x, w, y, mul, ldx, 0, ldw, 0, ldy, 0, ld_mul, 0, M, N, K};
    p.bias = bias;
    p.limit = limit;
    ZL_CHECK_ARG(epilogue != ZL_GEMM_EPI_GLU_CLAMP);
    return gemm_dispatch(p, 1, in_dtype, out_dtype, epilogue, pdl, stream);
}

extern "C" int zl_gemm_nt_bias(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y,
                               long long ldy, int M, int N, int K, int in_dtype, int out_dtype, int epilogue, int pdl,
                               zl_stream_t stream) {
    ZL_CHECK_ARG(epilogue == ZL_GEMM_EPI_NONE || epilogue == ZL_GEMM_EPI_RELU2 || epilogue == ZL_GEMM_EPI_TANH);
    GemmP p{x, w, y, nullptr, ldx, 0, ldw, 0, ldy, 0, 0, 0, M, N, K};
    p.bias = bias;
    return gemm_dispatch(p, 1, in_dtype, out_dtype, epilogue, pdl, stream);
}

extern "C" int zl_gemm_nt_glu_clamp(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y,
                                    long long ldy, int M, int N, int K, int in_dtype, int out_dtype, float limit, float alpha,
                                    float beta, int pdl, zl_stream_t stream) {
    GemmP p{x, w, y, nullptr, ldx, 0, ldw, 0, ldy, 0, 0, 0, M, N, K};
    p.bias = bias;
    p.limit = limit;
    p.alpha = alpha;
    p.beta = beta;
    return gemm_dispatch(p, 1, in_dtype, out_dtype, ZL_GEMM_EPI_GLU_CLAMP, pdl, stream);
}

extern "C" int zl_gemm_nt_grouped(const void* x, long long ldx, const int32_t* x_rows, const void* w, long long ldw,
                                  long long w_group_stride, void* y, long long ldy, const int32_t* y_rows,
                                  const int32_t* group_offsets, int groups, int max_rows, int N, int K, int in_dtype,
                                  int out_dtype, int epilogue, float limit, float alpha, float beta, int pdl,
                                  zl_stream_t stream) {
    ZL_CHECK_ARG(group_offsets && (epilogue == ZL_GEMM_EPI_NONE || epilogue == ZL_GEMM_EPI_RELU2 || epilogue == ZL_GEMM_EPI_GLU_CLAMP));
    GemmP p{x, w, y, nullptr, ldx, 0, ldw, w_group_stride, ldy, 0, 0, 0, max_rows, N, K};
    p.grp_off = group_offsets;
    p.x_rows = x_rows;
    p.y_rows = y_rows;
    p.limit = limit;
    p.alpha = alpha;
    p.beta = beta;
    return gemm_dispatch(p, groups, in_dtype, out_dtype, epilogue, pdl, stream);
}

// Row-wise pieces of a hybrid decoder layer: embedding into an fp32 residual stream, the residual update fused with a
// weight-only layer norm, RMS norm of a projection output, and the feed-forward activations.
#include "mix_common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) embed_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table,
                                                            float* __restrict__ out, T* __restrict__ copy, int width, int64_t vocab) {
    B200_PDL_SYNC();
    const int row = blockIdx.x;
    int64_t id = ids[row];
    if (id < 0 || id >= vocab) id = 0;
    const T* src = table + id * width;
    float* dst = out + (int64_t)row * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const T v = src[c];
        dst[c] = ldf(&v);
        if (copy) copy[(int64_t)row * width + c] = v;
    }
}

// Norm on a sublayer's OUTPUT, then the residual update:  x[row] += mult * y[row] / sqrt(mean(y^2) + eps) * (w_offset + w).
// y is the branch output in the activation type, or (y32) in fp32.  `copy`, when given, receives the updated row in the
// activation type: the operand of the next sublayer's projections, which read the stream itself.  `out_next`, when given,
// receives the RMS norm of the updated row with the next sublayer's input weight, x / sqrt(mean(x^2) + eps) * (next_offset +
// w_next): layers that norm a sublayer on both sides do the closing norm, the update and the opening norm in one pass.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) add_normed_kernel(float* __restrict__ x, const T* __restrict__ y,
                                                                 const float* __restrict__ y32, const T* __restrict__ w, float mult,
                                                                 float w_offset, T* __restrict__ copy, const T* __restrict__ w_next,
                                                                 float next_offset, T* __restrict__ out_next, int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = y32 ? y32[base + c] : ldf(y + base + c);
        q = fmaf(v, v, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    float q2 = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = y32 ? y32[base + c] : ldf(y + base + c);
        const float r = fmaf(mult, v * rstd * (w_offset + ldf(w + c)), x[base + c]);
        x[base + c] = r;
        q2 = fmaf(r, r, q2);
        if (copy) stf(copy + base + c, r);
    }
    if (out_next == nullptr) return;
    const float rstd2 = 1.0f / sqrtf(block_sum(q2, red) / (float)cols + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x)      // the same thread wrote these elements: no fence needed
        stf(out_next + base + c, x[base + c] * rstd2 * (next_offset + ldf(w_next + c)));
}

// Token embedding scaled by a constant, plus a hashed embedding of the (previous token, token) pair:
//     x = table[id] * scale + pair[(prev * mul_prev + id * mul_cur) mod buckets],   row `buckets` of pair for a sequence's first token.
// The previous token of a portion's first token comes from the sequence's state slot (prev_tok, int64 [slots]); afterwards
// token_state_update_kernel leaves the portion's last token there.  One CTA per (token of a portion, sequence).
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) embed_pair_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table, float scale,
                                                                 const T* __restrict__ pair, int64_t buckets, int64_t mul_prev,
                                                                 int64_t mul_cur, const int64_t* __restrict__ prev_tok,
                                                                 const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
                                                                 const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens,
                                                                 float* __restrict__ out, T* __restrict__ copy, int width, int64_t vocab) {
    B200_PDL_SYNC();
    const int s = blockIdx.y, i = blockIdx.x;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (cu_q == nullptr && sp.qlen == 0) {                 // padding row of a captured single-token step: defined, unused
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            out[(int64_t)s * width + c] = 0.f;
            if (copy) stf(copy + (int64_t)s * width + c, 0.f);
        }
        return;
    }
    if (i >= sp.qlen) return;
    const int64_t row = sp.q0 + i;
    const int pos = sp.klen - sp.qlen + i;
    int64_t id = ids[row];
    if (id < 0 || id >= vocab) id = 0;
    const T* src = table + id * width;
    const T* src2 = nullptr;
    if (pair != nullptr) {
        int64_t prow = buckets;
        if (pos > 0) {
            int64_t prev = i > 0 ? ids[row - 1] : prev_tok[state_slots[s]];
            if (prev < 0 || prev >= vocab) prev = 0;
            prow = (prev * mul_prev + id * mul_cur) % buckets;
            if (prow < 0) prow += buckets;
        }
        src2 = pair + prow * width;
    }
    float* dst = out + row * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = ldf(src + c) * scale;
        if (src2) v += ldf(src2 + c);
        dst[c] = v;
        if (copy) stf(copy + row * width + c, v);
    }
}

__global__ void token_state_update_kernel(const int64_t* __restrict__ ids, int64_t* __restrict__ prev_tok,
                                          const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
                                          const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens, int num_seqs) {
    B200_PDL_SYNC();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= num_seqs) return;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen > 0) prev_tok[state_slots[s]] = ids[sp.q0 + sp.qlen - 1];
}

// out[i] = x[row] / sqrt(mean(x[row]^2) + eps) * (w_offset + w) for row = rows_idx[i] (or i) of an fp32 stream.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows_idx,
                                                                   const T* __restrict__ w, float w_offset, T* __restrict__ out,
                                                                   int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const int64_t row = rows_idx ? rows_idx[blockIdx.x] : blockIdx.x;
    const float* xr = x + row * cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) q = fmaf(xr[c], xr[c], q);
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    T* o = out + (int64_t)blockIdx.x * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) stf(o + c, xr[c] * rstd * (w_offset + ldf(w + c)));
}

// x[row] += (a[row] + b[row] + b32[row])  (each term optional), then out[i] = LN(x[row]) * w, where the statistics are the
// mean and the mean of squared deviations of the updated row.  rows_idx (optional) names the rows to normalise: the
// update is then skipped (it must have happened already) and out has one row per index.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) add_layernorm_kernel(float* __restrict__ x, const T* __restrict__ a,
                                                                    const T* __restrict__ b, const float* __restrict__ b32,
                                                                    const T* __restrict__ w, T* __restrict__ out,
                                                                    const int32_t* __restrict__ rows_idx, int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const int orow = blockIdx.x;
    const int64_t row = rows_idx ? rows_idx[orow] : orow;
    float* xr = x + row * cols;
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float v = xr[c];
        if (!rows_idx && (a || b || b32)) {
            float d = 0.f;
            if (a) d += ldf(a + row * cols + c);
            if (b) d += ldf(b + row * cols + c);
            if (b32) d += b32[row * cols + c];
            v += d;
            xr[c] = v;
        }
        s += v;
    }
    if (out == nullptr) return;
    const float mean = block_sum(s, red) / (float)cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {      // same thread wrote these elements: no fence needed
        const float d = xr[c] - mean;
        q = fmaf(d, d, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    T* o = out + (int64_t)orow * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) stf(o + c, (xr[c] - mean) * rstd * ldf(w + c));
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_any_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ w,
                                                                  T* __restrict__ out, int64_t out_stride, int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const T* xr = x + (int64_t)blockIdx.x * x_stride;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = ldf(xr + c);
        q = fmaf(v, v, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    T* o = out + (int64_t)blockIdx.x * out_stride;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) stf(o + c, ldf(xr + c) * rstd * ldf(w + c));
}

__device__ __forceinline__ float gelu_tanh_(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// kind 0: x = [gate | up] per row, out = gelu_tanh(gate) * up;  kind 1: out = relu(x)^2 (no second half);
// kind 2: x = [gate | up], out = silu(gate) * up;  kind 3: out = gelu_tanh(x) (no second half)
template <typename T>
__global__ void ff_act_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int n, int kind) {
    B200_PDL_SYNC();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * n) return;
    const int64_t r = i / n;
    const int c = (int)(i - r * n);
    if (kind == 1) {
        const float v = fmaxf(ldf(x + i), 0.f);
        stf(out + i, v * v);
    } else if (kind == 3) {
        stf(out + i, gelu_tanh_(ldf(x + i)));
    } else {
        const float g = ldf(x + r * 2 * n + c), u = ldf(x + r * 2 * n + n + c);
        stf(out + i, (kind == 0 ? gelu_tanh_(g) : siluf_(g)) * u);
    }
}

// bf16 rows whose halves are multiples of 8: 8 columns per thread, 128-bit accesses, one row per blockIdx.y
__global__ void __launch_bounds__(256) ff_act_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int n, int kind) {
    B200_PDL_SYNC();
    const int c = (blockIdx.x * 256 + threadIdx.x) << 3;
    if (c >= n) return;
    const int64_t r = blockIdx.y;
    float o[8];
    if (kind == 1 || kind == 3) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(x + r * n + c), v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float t = fmaxf(v[e], 0.f);
            o[e] = kind == 1 ? t * t : gelu_tanh_(v[e]);
        }
    } else {
        float gt[8], up[8];
        unpack8(*reinterpret_cast<const uint4*>(x + r * 2 * n + c), gt);
        unpack8(*reinterpret_cast<const uint4*>(x + r * 2 * n + n + c), up);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (kind == 0 ? gelu_tanh_(gt[e]) : siluf_(gt[e])) * up[e];
    }
    *reinterpret_cast<uint4*>(out + r * n + c) = pack8(o);
}

// Gated unit with clamped branches: x = [gate | up] per row, g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + 1).
__device__ __forceinline__ float glu_clamped_(float g, float u, float limit, float alpha) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoidf_(alpha * g) * (u + 1.0f);
}

template <typename T>
__global__ void ff_glu_clamped_kernel(const T* __restrict__ x, int64_t x_stride, T* __restrict__ out, int64_t rows, int n, float limit,
                                      float alpha) {
    B200_PDL_SYNC();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * n) return;
    const int64_t r = i / n;
    const int c = (int)(i - r * n);
    stf(out + i, glu_clamped_(ldf(x + r * x_stride + c), ldf(x + r * x_stride + n + c), limit, alpha));
}

__global__ void __launch_bounds__(256) ff_glu_clamped_vec_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_stride, __nv_bfloat16* __restrict__ out, int n,
                                                                 float limit, float alpha) {
    B200_PDL_SYNC();
    const int c = (blockIdx.x * 256 + threadIdx.x) << 3;
    if (c >= n) return;
    const int64_t r = blockIdx.y;
    float gt[8], up[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(x + r * x_stride + c), gt);
    unpack8(*reinterpret_cast<const uint4*>(x + r * x_stride + n + c), up);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = glu_clamped_(gt[e], up[e], limit, alpha);
    *reinterpret_cast<uint4*>(out + r * n + c) = pack8(o);
}

// A sublayer's close in a layer that gates, norms and column-scales the sublayer's result:
//     t = y * sigmoid(gate);  x += t / sqrt(mean(t^2) + eps) * w_out;  out_next = x / sqrt(mean(x^2) + eps) * next_scale * w_next.
// The gated row stays in registers between the statistic and the update (PER elements per thread; wider rows are recomputed).
template <typename T, int PER>
__global__ void __launch_bounds__(ROW_THREADS) gated_add_normed_kernel(float* __restrict__ x, const T* __restrict__ y,
                                                                       const float* __restrict__ y32, const T* __restrict__ gate,
                                                                       int64_t gate_stride, const float* __restrict__ w_out,
                                                                       const float* __restrict__ w_next, float next_scale,
                                                                       T* __restrict__ out_next, int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * cols;
    const T* grow = gate ? gate + (int64_t)blockIdx.x * gate_stride : nullptr;
    auto gated = [&](int c) {
        const float v = y32 ? y32[base + c] : ldf(y + base + c);
        return grow ? v * sigmoidf_(ldf(grow + c)) : v;
    };
    float t[PER];
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = threadIdx.x + k * ROW_THREADS;
        t[k] = c < cols ? gated(c) : 0.f;
        q = fmaf(t[k], t[k], q);
    }
    for (int c = threadIdx.x + PER * ROW_THREADS; c < cols; c += ROW_THREADS) {
        const float v = gated(c);
        q = fmaf(v, v, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    float q2 = 0.f;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = threadIdx.x + k * ROW_THREADS;
        if (c < cols) {
            t[k] = fmaf(t[k] * rstd, w_out[c], x[base + c]);
            x[base + c] = t[k];
            q2 = fmaf(t[k], t[k], q2);
        }
    }
    for (int c = threadIdx.x + PER * ROW_THREADS; c < cols; c += ROW_THREADS) {
        const float r = fmaf(gated(c) * rstd, w_out[c], x[base + c]);
        x[base + c] = r;
        q2 = fmaf(r, r, q2);
    }
    if (out_next == nullptr) return;
    const float rstd2 = next_scale / sqrtf(block_sum(q2, red) / (float)cols + eps);
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = threadIdx.x + k * ROW_THREADS;
        if (c < cols) stf(out_next + base + c, t[k] * rstd2 * (w_next ? w_next[c] : 1.0f));
    }
    for (int c = threadIdx.x + PER * ROW_THREADS; c < cols; c += ROW_THREADS)      // the same thread wrote these elements
        stf(out_next + base + c, x[base + c] * rstd2 * (w_next ? w_next[c] : 1.0f));
}

__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ x, int64_t n, float cap) {
    B200_PDL_SYNC();
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        float4 v = *reinterpret_cast<float4*>(x + i);
        v.x = cap * tanhf(v.x / cap), v.y = cap * tanhf(v.y / cap), v.z = cap * tanhf(v.z / cap), v.w = cap * tanhf(v.w / cap);
        *reinterpret_cast<float4*>(x + i) = v;
    } else {
        for (int64_t j = i; j < n && j < i + 4; ++j) x[j] = cap * tanhf(x[j] / cap);
    }
}

}  // namespace

extern "C" int b200m_abi_version(void) { return 4; }

extern "C" int b200m_ff_glu_clamped(const void* x, int64_t x_stride, void* out, int64_t rows, int n, float limit, float alpha, int is32,
                                    void* stream) {
    if (!x || !out || rows < 0 || n <= 0 || x_stride < 2 * (int64_t)n) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!is32 && n % 8 == 0 && x_stride % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        for (int64_t r0 = 0; r0 < rows; r0 += 65535) {             // grid.y limit
            const int64_t nr = rows - r0 < 65535 ? rows - r0 : 65535;
            B200_LAUNCH((ff_glu_clamped_vec_kernel), dim3((n / 8 + 255) / 256, (unsigned)nr), 256, 0, st,
                        static_cast<const __nv_bfloat16*>(x) + r0 * x_stride, x_stride, static_cast<__nv_bfloat16*>(out) + r0 * n, n, limit, alpha);
        }
        return b200_launch_status(nullptr);
    }
    const int64_t total = rows * n;
    B200M_DISPATCH(is32, B200_LAUNCH((ff_glu_clamped_kernel<T>), (unsigned)((total + 255) / 256), 256, 0, st, static_cast<const T*>(x),
                                     x_stride, static_cast<T*>(out), rows, n, limit, alpha));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_gated_add_normed_norm(float* x, const void* y, const float* y32, const void* gate, int64_t gate_stride,
                                           const float* w_out, const float* w_next, float next_scale, void* out_next, int rows,
                                           int cols, float eps, int is32, void* stream) {
    if (!x || (!y && !y32) || !w_out || rows < 0 || cols <= 0) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cols <= 4 * ROW_THREADS) {
        B200M_DISPATCH(is32, B200_LAUNCH((gated_add_normed_kernel<T, 4>), rows, ROW_THREADS, 0, st, x, static_cast<const T*>(y), y32,
                                         static_cast<const T*>(gate), gate_stride, w_out, w_next, next_scale, static_cast<T*>(out_next),
                                         cols, eps));
    } else {
        B200M_DISPATCH(is32, B200_LAUNCH((gated_add_normed_kernel<T, 16>), rows, ROW_THREADS, 0, st, x, static_cast<const T*>(y), y32,
                                         static_cast<const T*>(gate), gate_stride, w_out, w_next, next_scale, static_cast<T*>(out_next),
                                         cols, eps));
    }
    return b200_launch_status(nullptr);
}

extern "C" int b200m_softcap(float* x, int64_t n, float cap, void* stream) {
    if (!x || n < 0 || !(cap > 0.f)) return B200_EINVAL;
    if (n == 0) return B200_OK;
    B200_LAUNCH((softcap_kernel), (unsigned)((n + 1023) / 1024), 256, 0, static_cast<cudaStream_t>(stream), x, n, cap);
    return b200_launch_status(nullptr);
}

extern "C" int b200m_embed(const int64_t* ids, const void* table, float* out, void* copy, int n, int width, int64_t vocab, int is32,
                           void* stream) {
    if (!ids || !table || !out || n < 0 || width <= 0 || vocab <= 0) return B200_EINVAL;
    if (n == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((embed_kernel<T>), n, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), ids,
                                     static_cast<const T*>(table), out, static_cast<T*>(copy), width, vocab));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_add_normed(float* x, const void* y, const float* y32, const void* w, float mult, float w_offset, void* copy,
                                int rows, int cols, float eps, int is32, void* stream) {
    if (!x || (!y && !y32) || !w || rows < 0 || cols <= 0) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((add_normed_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), x,
                                     static_cast<const T*>(y), y32, static_cast<const T*>(w), mult, w_offset,
                                     static_cast<T*>(copy), static_cast<const T*>(nullptr), 0.f, static_cast<T*>(nullptr), cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_add_normed_norm(float* x, const void* y, const float* y32, const void* w, float mult, float w_offset, void* copy,
                                     const void* w_next, float next_offset, void* out_next, int rows, int cols, float eps, int is32,
                                     void* stream) {
    if (!x || (!y && !y32) || !w || rows < 0 || cols <= 0 || (out_next && !w_next)) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((add_normed_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), x,
                                     static_cast<const T*>(y), y32, static_cast<const T*>(w), mult, w_offset,
                                     static_cast<T*>(copy), static_cast<const T*>(w_next), next_offset, static_cast<T*>(out_next),
                                     cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_embed_pair(const int64_t* ids, const void* table, float scale, const void* pair, int64_t buckets, int64_t mul_prev,
                                int64_t mul_cur, int64_t* prev_tok, const int32_t* state_slots, const int32_t* cu_q,
                                const int32_t* cu_k, const int32_t* ctx_lens, float* out, void* copy, int num_seqs, int max_q, int width,
                                int64_t vocab, int is32, void* stream) {
    if (!ids || !table || !out || width <= 0 || vocab <= 0) return B200_EINVAL;
    if (pair && (buckets <= 0 || !prev_tok || !state_slots)) return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (num_seqs <= 0 || max_q <= 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B200M_DISPATCH(is32, B200_LAUNCH((embed_pair_kernel<T>), dim3(max_q, num_seqs), ROW_THREADS, 0, st, ids, static_cast<const T*>(table),
                                     scale, static_cast<const T*>(pair), buckets, mul_prev, mul_cur, prev_tok, state_slots, cu_q, cu_k,
                                     ctx_lens, out, static_cast<T*>(copy), width, vocab));
    int rc = b200_launch_status(nullptr);
    if (rc != B200_OK || !pair) return rc;
    B200_LAUNCH((token_state_update_kernel), (num_seqs + 127) / 128, 128, 0, st, ids, prev_tok, state_slots, cu_q, cu_k, ctx_lens, num_seqs);
    return b200_launch_status(nullptr);
}

extern "C" int b200m_rmsnorm_rows(const float* x, const int32_t* rows_idx, const void* w, float w_offset, void* out, int rows,
                                  int cols, float eps, int is32, void* stream) {
    if (!x || !w || !out || rows < 0 || cols <= 0) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((rmsnorm_rows_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), x, rows_idx,
                                     static_cast<const T*>(w), w_offset, static_cast<T*>(out), cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_add_layernorm(float* x, const void* a, const void* b, const float* b32, const void* w, void* out,
                                   const int32_t* rows_idx, int rows, int cols, float eps, int is32, void* stream) {
    if (!x || rows < 0 || cols <= 0 || (out && !w)) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((add_layernorm_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), x,
                                     static_cast<const T*>(a), static_cast<const T*>(b), b32, static_cast<const T*>(w),
                                     static_cast<T*>(out), rows_idx, cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_rmsnorm(const void* x, int64_t x_stride, const void* w, void* out, int64_t out_stride, int rows, int cols,
                             float eps, int is32, void* stream) {
    if (!x || !w || !out || rows < 0 || cols <= 0) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((rmsnorm_any_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream),
                                     static_cast<const T*>(x), x_stride, static_cast<const T*>(w), static_cast<T*>(out),
                                     out_stride, cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_ff_act(const void* x, void* out, int64_t rows, int n, int kind, int is32, void* stream) {
    if (!x || !out || rows < 0 || n <= 0 || kind < 0 || kind > 3) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    if (!is32 && n % 8 == 0 && rows <= 65535 * 32 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        for (int64_t r0 = 0; r0 < rows; r0 += 65535) {             // grid.y limit
            const int64_t nr = rows - r0 < 65535 ? rows - r0 : 65535;
            const int64_t in_row = (kind == 1 || kind == 3) ? n : 2 * (int64_t)n;
            B200_LAUNCH((ff_act_vec_kernel), dim3((n / 8 + 255) / 256, (unsigned)nr), 256, 0, static_cast<cudaStream_t>(stream),
                        static_cast<const __nv_bfloat16*>(x) + r0 * in_row, static_cast<__nv_bfloat16*>(out) + r0 * n, n, kind);
        }
        return b200_launch_status(nullptr);
    }
    const int64_t total = rows * n;
    B200M_DISPATCH(is32, B200_LAUNCH((ff_act_kernel<T>), (unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream),
                                     static_cast<const T*>(x), static_cast<T*>(out), rows, n, kind));
    return b200_launch_status(nullptr);
}

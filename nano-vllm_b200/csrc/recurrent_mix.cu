// Linear recurrences with per-sequence state slots: a gated diagonal recurrence and the gated delta rule.
//
// Everything that enters a recurrence (gates, decays, step sizes, unit norms, the state) is fp32 in both element types; the
// activation type T only names what the projections and convolutions in front left in memory and what the result is rounded to.
// A step whose sequence has no tokens behind it starts from zeros whatever the slot holds, so a slot needs no clearing when
// it changes hands.
//
// Gated diagonal recurrence (one scalar state per channel):
//     r = sigmoid(gr + br), i = sigmoid(gi + bi)          gr, gi: block-diagonal maps of u, computed by the caller (fp32)
//     a = exp(rate * r)                                   rate = -c softplus(lambda) <= 0, per channel
//     S <- a S + sqrt(1 - a^2) (i u)                      out = S * gelu_tanh(y)
//   diag_scan_kernel<MODE 0>  whole portions, one thread per channel walking the tokens (single-token steps included)
//   diag_scan_kernel<MODE 1>, diag_carry_kernel, diag_scan_kernel<MODE 3>: long portions as chunks in parallel -- every chunk from
//   zero keeping (product of a, end state), a serial pass over the chunk summaries that leaves every chunk's start state, and
//   every chunk again from its start state writing the output.
//
// Gated delta rule (per head a matrix state S [dim, vdim]; query/key head h / (H / G)):
//     q <- q / sqrt(|q|^2 + 1e-6) * q_scale,  k <- k / sqrt(|k|^2 + 1e-6)
//     g = exp(rate_h softplus(a_t + dt_bias_h)),  beta = sigmoid(b_t)
//     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   Columns of S are independent, so a thread group of four lanes owns one column (dim / 4 state elements per lane in
//   registers) and walks the tokens; a CTA covers 32 columns of one (sequence, head).  The decay folds into the update:
//   d = S_old^T k;  u = beta (v - g d);  S_new = g S_old + k u.  Tokens are staged through shared memory a chunk ahead.
#include "mix_common.cuh"

namespace {

__device__ __forceinline__ float softplus_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float gelu_tanh1_(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

// gates: fp32 [blocks, rows, 2 * cb]: for block b and token row t the cb pre-activations of r, then those of i.
template <typename T, int MODE>
__global__ void __launch_bounds__(128) diag_scan_kernel(const T* __restrict__ u, int64_t u_stride, const float* __restrict__ gates, int64_t rows,
                                                        const float* __restrict__ gate_bias, const float* __restrict__ rate,
                                                        const T* __restrict__ y, int64_t y_stride, float* __restrict__ state,
                                                        const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
                                                        const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens,
                                                        T* __restrict__ out, int channels, int cb, int chunk_len, int nchunks,
                                                        float* __restrict__ ws) {
    B200_PDL_SYNC();
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int i_begin = MODE == 0 ? 0 : blockIdx.z * chunk_len;
    if (i_begin >= sp.qlen) return;
    const int i_end = MODE == 0 ? sp.qlen : min(sp.qlen, i_begin + chunk_len);
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int b = c / cb, j = c - b * cb;
    const float br = gate_bias[(int64_t)b * 2 * cb + j], bi = gate_bias[(int64_t)b * 2 * cb + cb + j], rt = rate[c];
    const float* gb = gates + (int64_t)b * rows * 2 * cb + j;
    float* st = state + (int64_t)state_slots[s] * channels + c;
    float* wsp = ws ? ws + (((int64_t)s * nchunks + blockIdx.z) * channels + c) * 2 : nullptr;
    float S = 0.f, P = 1.f;
    if (MODE == 0) S = (sp.klen - sp.qlen > 0) ? *st : 0.f;
    if (MODE == 3) S = wsp[0];
    constexpr int TB = 4;                                    // tokens whose operands are fetched before their (serial) arithmetic
    for (int i0 = i_begin; i0 < i_end; i0 += TB) {
        float uu[TB], gr[TB], gi[TB], yy[TB];
#pragma unroll
        for (int k = 0; k < TB; ++k) {
            const int64_t row = sp.q0 + min(i0 + k, i_end - 1);
            uu[k] = ldf(u + row * u_stride + c);
            gr[k] = gb[row * 2 * cb];
            gi[k] = gb[row * 2 * cb + cb];
            yy[k] = MODE == 1 ? 0.f : ldf(y + row * y_stride + c);
        }
#pragma unroll
        for (int k = 0; k < TB; ++k) {
            if (i0 + k >= i_end) break;
            const float la = rt * sigmoidf_(gr[k] + br);     // log a <= 0
            const float a = expf(la);
            const float drive = sqrtf(-expm1f(2.0f * la)) * sigmoidf_(gi[k] + bi) * uu[k];
            S = fmaf(a, S, drive);
            if (MODE == 1) P *= a;
            else stf(out + (int64_t)(sp.q0 + i0 + k) * channels + c, S * gelu_tanh1_(yy[k]));
        }
    }
    if (MODE == 0) *st = S;
    if (MODE == 1) {
        wsp[0] = P;
        wsp[1] = S;
    }
}

// ws[s, z, c] = (product of a over chunk z, end state of chunk z from zero) -> ws[s, z, c, 0] = state at the start of chunk z
__global__ void __launch_bounds__(128) diag_carry_kernel(float* __restrict__ ws, float* __restrict__ state, const int32_t* __restrict__ state_slots,
                                                         const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k,
                                                         const int32_t* __restrict__ ctx_lens, int channels, int chunk_len, int nchunks) {
    B200_PDL_SYNC();
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float* st = state + (int64_t)state_slots[s] * channels + c;
    float S = (sp.klen - sp.qlen > 0) ? *st : 0.f;
    const int used = (sp.qlen + chunk_len - 1) / chunk_len;
    for (int z = 0; z < used; ++z) {
        float* w = ws + (((int64_t)s * nchunks + z) * channels + c) * 2;
        const float P = w[0], E = w[1];
        w[0] = S;
        S = fmaf(P, S, E);
    }
    *st = S;
}

constexpr int GD_LANES = 4;            // lanes that share one column of the state
constexpr int GD_COLS = 32;            // columns per CTA (128 threads)

// DPL state rows per lane: lane `sub` of a column's group owns rows sub * DPL .. sub * DPL + DPL - 1 (zero beyond dim).
// state: [slots, H, vdim, dim] (a column's rows are contiguous).
// Tokens are staged through shared memory TB at a time, as fp32: the chunk after the current one is fetched into registers
// before the current one is worked on and stored afterwards (two buffers), so the serial walk never waits for global memory.
// A staged key or query row is four lane segments of DPL floats, each padded by four: 128-bit reads without bank conflicts.
// After a chunk lands, 128 / TB threads per token form its unit-norm factors, write strength and decay once for the CTA.
template <typename T, int DPL>
__global__ void __launch_bounds__(GD_LANES * GD_COLS) gated_delta_kernel(
    const T* __restrict__ x, int64_t stride, int q_off, int k_off, int v_off,     // per token: q, k [G, dim], v [H, vdim] (convolved, activated)
    const float* __restrict__ ba, int64_t ba_stride,                              // per token: H write strengths, then H decay inputs (pre-activation)
    const float* __restrict__ rate, const float* __restrict__ dt_bias,            // [H]: rate = -exp(A_log)
    float* __restrict__ state, const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
    const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens, float* __restrict__ out,      // [n, H, vdim] fp32
    int H, int G, int dim, int vdim, float q_scale) {
    B200_PDL_SYNC();
    constexpr int NT = GD_LANES * GD_COLS;
    constexpr int TB = DPL >= 64 ? 8 : 16;
    constexpr int SEG = DPL + 4, ROW = GD_LANES * SEG, DP = GD_LANES * DPL;
    constexpr int PF = (TB * DP) / NT;                     // key (and query) elements a thread fetches per chunk
    constexpr int PV = (TB * GD_COLS) / NT;                // value elements a thread fetches per chunk
    constexpr int TPT = NT / TB;                           // threads that share one token's factors
    __shared__ __align__(16) float ks[2][TB][ROW];
    __shared__ __align__(16) float qs[2][TB][ROW];
    __shared__ float vs[2][TB][GD_COLS];
    __shared__ float sc[2][TB][4];                         // key normaliser, query normaliser * scale, write strength, decay
    const int h = blockIdx.x, s = blockIdx.y, tid = threadIdx.x;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int sub = tid % GD_LANES;
    const int col0 = blockIdx.z * GD_COLS, col = col0 + tid / GD_LANES;
    const bool live = col < vdim;
    const int cc = live ? col : vdim - 1;
    const int g = h / (H / G);
    float* st = state + (((int64_t)state_slots[s] * H + h) * vdim + cc) * dim + sub * DPL;
    const bool has_hist = sp.klen - sp.qlen > 0;
    const bool vec_state = dim == GD_LANES * DPL;           // whole lane segments (then 16-byte aligned too): 128-bit state accesses
    float S[DPL];
    if (has_hist && vec_state) {
#pragma unroll
        for (int k = 0; k < DPL / 4; ++k) {
            const float4 f = reinterpret_cast<const float4*>(st)[k];
            S[4 * k] = f.x, S[4 * k + 1] = f.y, S[4 * k + 2] = f.z, S[4 * k + 3] = f.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < DPL; ++k) S[k] = (has_hist && sub * DPL + k < dim) ? st[k] : 0.f;
    }
    const float rt = rate[h], db = dt_bias[h];
    const T* qp = x + q_off + (int64_t)g * dim;
    const T* kp = x + k_off + (int64_t)g * dim;
    const T* vp = x + v_off + (int64_t)h * vdim + col0;
    float fk[PF], fq[PF], fv[PV], fb = 0.f, fa = 0.f;      // the next chunk, in flight
    auto fetch = [&](int i0) {
#pragma unroll
        for (int j = 0; j < PF; ++j) {
            const int e = tid + NT * j, t = e / DP, d = e - t * DP;
            const bool ok = i0 + t < sp.qlen && d < dim;
            const int64_t row = sp.q0 + i0 + t;
            fk[j] = ok ? ldf(kp + row * stride + d) : 0.f;
            fq[j] = ok ? ldf(qp + row * stride + d) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < PV; ++j) {
            const int e = tid + NT * j, t = e / GD_COLS, c = e - t * GD_COLS;
            fv[j] = (i0 + t < sp.qlen && col0 + c < vdim) ? ldf(vp + (int64_t)(sp.q0 + i0 + t) * stride + c) : 0.f;
        }
        if (tid < TB && i0 + tid < sp.qlen) {
            fb = ba[(int64_t)(sp.q0 + i0 + tid) * ba_stride + h];
            fa = ba[(int64_t)(sp.q0 + i0 + tid) * ba_stride + H + h];
        }
    };
    auto land = [&](int buf) {                             // registers -> shared memory
#pragma unroll
        for (int j = 0; j < PF; ++j) {
            const int e = tid + NT * j, t = e / DP, d = e - t * DP;
            const int at = (d / DPL) * SEG + (d % DPL);
            ks[buf][t][at] = fk[j];
            qs[buf][t][at] = fq[j];
        }
#pragma unroll
        for (int j = 0; j < PV; ++j) {
            const int e = tid + NT * j;
            vs[buf][e / GD_COLS][e % GD_COLS] = fv[j];
        }
        if (tid < TB) {
            sc[buf][tid][2] = sigmoidf_(fb);
            sc[buf][tid][3] = expf(rt * softplus_(fa + db));
        }
    };
    auto factors = [&](int buf) {                          // after a barrier: the unit-norm factors of the chunk's tokens
        const int t = tid / TPT, j = tid % TPT;
        float ssk = 0.f, ssq = 0.f;
        for (int d = j; d < DP; d += TPT) {
            const int at = (d / DPL) * SEG + (d % DPL);
            const float a = ks[buf][t][at], b = qs[buf][t][at];
            ssk = fmaf(a, a, ssk);
            ssq = fmaf(b, b, ssq);
        }
#pragma unroll
        for (int o = 1; o < TPT; o <<= 1) {
            ssk += __shfl_xor_sync(0xffffffffu, ssk, o);
            ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        }
        if (j == 0) {
            sc[buf][t][0] = 1.0f / sqrtf(ssk + 1e-6f);
            sc[buf][t][1] = q_scale / sqrtf(ssq + 1e-6f);
        }
    };
    fetch(0);
    land(0);
    __syncthreads();
    factors(0);
    __syncthreads();
    for (int i0 = 0, buf = 0; i0 < sp.qlen; i0 += TB, buf ^= 1) {
        const bool more = i0 + TB < sp.qlen;
        if (more) fetch(i0 + TB);
        const int nt = min(TB, sp.qlen - i0);
        for (int t = 0; t < nt; ++t) {
            const float4* kr = reinterpret_cast<const float4*>(&ks[buf][t][sub * SEG]);
            const float4* qr = reinterpret_cast<const float4*>(&qs[buf][t][sub * SEG]);
            float4 kk[DPL / 4];
            float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < DPL / 4; ++k) {
                kk[k] = kr[k];
                d4[0] = fmaf(S[4 * k], kk[k].x, d4[0]);
                d4[1] = fmaf(S[4 * k + 1], kk[k].y, d4[1]);
                d4[2] = fmaf(S[4 * k + 2], kk[k].z, d4[2]);
                d4[3] = fmaf(S[4 * k + 3], kk[k].w, d4[3]);
            }
            float dk = (d4[0] + d4[1]) + (d4[2] + d4[3]);
#pragma unroll
            for (int o = 1; o < GD_LANES; o <<= 1) dk += __shfl_xor_sync(0xffffffffu, dk, o);
            const float rk = sc[buf][t][0], rq = sc[buf][t][1], beta = sc[buf][t][2], gdec = sc[buf][t][3];
            const float v = vs[buf][t][tid / GD_LANES];
            const float uw = beta * (v - gdec * dk * rk) * rk;   // u times the key's normaliser: S += (k rk) u
            float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < DPL / 4; ++k) {
                const float4 qq = qr[k];
                S[4 * k] = fmaf(kk[k].x, uw, gdec * S[4 * k]);
                S[4 * k + 1] = fmaf(kk[k].y, uw, gdec * S[4 * k + 1]);
                S[4 * k + 2] = fmaf(kk[k].z, uw, gdec * S[4 * k + 2]);
                S[4 * k + 3] = fmaf(kk[k].w, uw, gdec * S[4 * k + 3]);
                o4[0] = fmaf(S[4 * k], qq.x, o4[0]);
                o4[1] = fmaf(S[4 * k + 1], qq.y, o4[1]);
                o4[2] = fmaf(S[4 * k + 2], qq.z, o4[2]);
                o4[3] = fmaf(S[4 * k + 3], qq.w, o4[3]);
            }
            float oq = (o4[0] + o4[1]) + (o4[2] + o4[3]);
#pragma unroll
            for (int o = 1; o < GD_LANES; o <<= 1) oq += __shfl_xor_sync(0xffffffffu, oq, o);
            if (live && sub == 0) out[((int64_t)(sp.q0 + i0 + t) * H + h) * vdim + col] = oq * rq;
        }
        if (more) {
            land(buf ^ 1);                                 // its last readers passed the barrier that closed the previous chunk
            __syncthreads();
            factors(buf ^ 1);
            __syncthreads();
        }
    }
    if (live && vec_state) {
#pragma unroll
        for (int k = 0; k < DPL / 4; ++k) reinterpret_cast<float4*>(st)[k] = make_float4(S[4 * k], S[4 * k + 1], S[4 * k + 2], S[4 * k + 3]);
    } else if (live) {
#pragma unroll
        for (int k = 0; k < DPL; ++k)
            if (sub * DPL + k < dim) st[k] = S[k];
    }
}

// out[t, h, :] = c * o / sqrt(mean(o^2) + eps) * w * act(gate[t, h, :]) for o = x[t, h, :] (fp32), one warp per (token, head).
// act 0: sigmoid, 1: silu.  w (optional): [vdim], shared by the heads.
template <typename T>
__global__ void __launch_bounds__(128) head_rmsnorm_gate_kernel(const float* __restrict__ x, const T* __restrict__ w, const T* __restrict__ gate,
                                                                int64_t gate_stride, int act, T* __restrict__ out, int64_t out_stride,
                                                                float out_scale, int64_t rows, int H, int vdim, float eps) {
    B200_PDL_SYNC();
    const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const int64_t t = r / H;
    const int h = (int)(r - t * H);
    const float* o = x + r * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss = fmaf(o[c], o[c], ss);
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    for (int c = lane; c < vdim; c += 32) {
        float v = o[c] * rstd;
        if (w) v *= ldf(w + c);
        if (gate) {
            const float z = ldf(gate + t * gate_stride + (int64_t)h * vdim + c);
            v *= act ? siluf_(z) : sigmoidf_(z);
        }
        stf(out + t * out_stride + (int64_t)h * vdim + c, v * out_scale);
    }
}

}  // namespace

extern "C" int b200m_diag_scan(const void* u, int64_t u_stride, const float* gates, int64_t rows, const float* gate_bias, const float* rate,
                               const void* y, int64_t y_stride, float* state, const int32_t* state_slots, const int32_t* cu_q,
                               const int32_t* cu_k, const int32_t* ctx_lens, void* out, int num_seqs, int max_q, int channels,
                               int block_channels, int chunk_len, float* ws, int is32, void* stream) {
    if (!u || !gates || !gate_bias || !rate || !y || !state || !state_slots || !out) return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (channels <= 0 || block_channels <= 0 || channels % block_channels) return B200_EINVAL;
    if (num_seqs <= 0 || max_q <= 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool chunked = ws != nullptr && chunk_len > 0 && max_q > chunk_len;
    const int nchunks = chunked ? (max_q + chunk_len - 1) / chunk_len : 1;
    const int bx = (channels + 127) / 128;
#define DIAG_GO(MODE, GZ)                                                                                                          \
    B200M_DISPATCH(is32, B200_LAUNCH((diag_scan_kernel<T, MODE>), dim3(bx, num_seqs, GZ), 128, 0, st, static_cast<const T*>(u), u_stride, \
                                     gates, rows, gate_bias, rate, static_cast<const T*>(y), y_stride, state, state_slots, cu_q, cu_k,    \
                                     ctx_lens, static_cast<T*>(out), channels, block_channels, chunk_len, nchunks, ws))
    if (!chunked) {
        DIAG_GO(0, 1);
        return b200_launch_status(nullptr);
    }
    DIAG_GO(1, nchunks);
    int rc = b200_launch_status(nullptr);
    if (rc != B200_OK) return rc;
    B200_LAUNCH((diag_carry_kernel), dim3(bx, num_seqs), 128, 0, st, ws, state, state_slots, cu_q, cu_k, ctx_lens, channels, chunk_len, nchunks);
    rc = b200_launch_status(nullptr);
    if (rc != B200_OK) return rc;
    DIAG_GO(3, nchunks);
#undef DIAG_GO
    return b200_launch_status(nullptr);
}

extern "C" int b200m_gated_delta(const void* x, int64_t stride, int q_off, int k_off, int v_off, const float* ba, int64_t ba_stride,
                                 const float* rate, const float* dt_bias, float* state, const int32_t* state_slots, const int32_t* cu_q,
                                 const int32_t* cu_k, const int32_t* ctx_lens, float* out, int num_seqs, int num_heads, int num_kv_heads,
                                 int dim, int vdim, float q_scale, int is32, void* stream) {
    if (!x || !ba || !rate || !dt_bias || !state || !state_slots || !out) return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || dim <= 0 || vdim <= 0) return B200_EINVAL;
    if (dim > 64 * GD_LANES) return B200_EUNSUPPORTED;
    if (num_seqs <= 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(num_heads, num_seqs, (vdim + GD_COLS - 1) / GD_COLS);
#define GD_GO(N)                                                                                                                   \
    B200M_DISPATCH(is32, B200_LAUNCH((gated_delta_kernel<T, N>), grid, GD_LANES * GD_COLS, 0, st, static_cast<const T*>(x), stride, q_off, \
                                     k_off, v_off, ba, ba_stride, rate, dt_bias, state, state_slots, cu_q, cu_k, ctx_lens, out, num_heads, \
                                     num_kv_heads, dim, vdim, q_scale))
    const int dpl = (dim + GD_LANES - 1) / GD_LANES;
    if (dpl <= 4) GD_GO(4);
    else if (dpl <= 8) GD_GO(8);
    else if (dpl <= 16) GD_GO(16);
    else if (dpl <= 32) GD_GO(32);
    else GD_GO(64);
#undef GD_GO
    return b200_launch_status(nullptr);
}

extern "C" int b200m_head_rmsnorm_gate(const float* x, const void* w, const void* gate, int64_t gate_stride, int act, void* out,
                                       int64_t out_stride, float out_scale, int n, int num_heads, int vdim, float eps, int is32,
                                       void* stream) {
    if (!x || !out || n < 0 || num_heads <= 0 || vdim <= 0) return B200_EINVAL;
    if (n == 0) return B200_OK;
    const int64_t rows = (int64_t)n * num_heads;
    B200M_DISPATCH(is32, B200_LAUNCH((head_rmsnorm_gate_kernel<T>), (unsigned)((rows + 3) / 4), 128, 0, static_cast<cudaStream_t>(stream), x,
                                     static_cast<const T*>(w), static_cast<const T*>(gate), gate_stride, act, static_cast<T*>(out),
                                     out_stride, out_scale, rows, num_heads, vdim, eps));
    return b200_launch_status(nullptr);
}

// Selective-scan (Mamba-1) recurrence with per-sequence state slots.
//
// Per channel c and state n, with u the convolved + SiLU'd input, dt = softplus(dt_raw + bias), A = -exp(A_log) (given):
//     S[c, n] <- exp(dt_c * A[c, n]) * S[c, n] + dt_c * u_c * B_n ;   y_c = sum_n S[c, n] * C_n + D_c * u_c ;   out = y * silu(z)
// A sequence owns one slot: its fp32 state S [channels, state] and the last (taps - 1) inputs of the causal convolution.
// A step whose sequence has no tokens behind it starts from zeros whatever the slot holds, so a slot needs no clearing
// when it changes hands.
//
//   causal_conv_kernel      : depthwise causal convolution + bias (+ SiLU) over a varlen batch, history taken from the slot
//   conv_state_update_kernel: the slot's history after the step (run after the convolution: it overwrites what that reads)
//   selective_scan_kernel   : the recurrence, serial over a sequence's tokens, 4 lanes per channel holding the state in
//                             registers; one token per sequence is the decode case of the same kernel.  Long portions run
//                             it three times over chunks of tokens: (1) every chunk from a zero state, keeping its end state
//                             and sum of step sizes; (2) scan_carry_kernel chains the chunks, S_in[z+1] = exp(A sum_dt[z])
//                             S_in[z] + S_end[z]; (3) every chunk again from its true start state, now writing y
#include "mix_common.cuh"

namespace {

constexpr int CONV_MAX_TAPS = 8;

// conv_state: [slots, taps - 1, channels] fp32, row taps-2 is the newest input.
template <typename T>
__global__ void __launch_bounds__(256) causal_conv_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ w,
                                                          const T* __restrict__ bias, const float* __restrict__ conv_state,
                                                          const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
                                                          const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens,
                                                          T* __restrict__ out, int channels, int taps, int tok_tile, int act) {
    B200_PDL_SYNC();
    const int s = blockIdx.z;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    const int i0 = blockIdx.y * tok_tile;
    if (i0 >= sp.qlen) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const bool has_hist = sp.klen - sp.qlen > 0;
    const float* hist = conv_state + (int64_t)state_slots[s] * (taps - 1) * channels;
    const float b = bias ? ldf(bias + c) : 0.f;
    const int i1 = min(sp.qlen, i0 + tok_tile);
    auto input = [&](int m) -> float {                     // input at local index m of the portion (negative: before it)
        if (m >= 0) return ldf(x + (int64_t)(sp.q0 + m) * x_stride + c);
        return has_hist ? hist[(int64_t)(taps - 1 + m) * channels + c] : 0.f;
    };
    if (taps <= CONV_MAX_TAPS) {
        // weights and a sliding window of the last taps inputs live in registers: one load per token
        float wr[CONV_MAX_TAPS], win[CONV_MAX_TAPS];
#pragma unroll
        for (int k = 0; k < CONV_MAX_TAPS; ++k) {
            wr[k] = k < taps ? ldf(w + (int64_t)c * taps + (taps - 1 - k)) : 0.f;      // wr[k]: weight of the input k tokens back
            win[k] = (k >= 1 && k < taps) ? input(i0 - k) : 0.f;                         // win[k]: input k tokens back (win[0] set below)
        }
        for (int i = i0; i < i1; ++i) {
            win[0] = ldf(x + (int64_t)(sp.q0 + i) * x_stride + c);
            float a = b;
#pragma unroll
            for (int k = 0; k < CONV_MAX_TAPS; ++k) a = fmaf(wr[k], win[k], a);
            stf(out + (int64_t)(sp.q0 + i) * channels + c, act ? siluf_(a) : a);
#pragma unroll
            for (int k = CONV_MAX_TAPS - 1; k >= 1; --k) win[k] = win[k - 1];
        }
        return;
    }
    for (int i = i0; i < i1; ++i) {
        float a = b;
        for (int k = 0; k < taps; ++k) a = fmaf(ldf(w + (int64_t)c * taps + k), input(i - (taps - 1 - k)), a);
        stf(out + (int64_t)(sp.q0 + i) * channels + c, act ? siluf_(a) : a);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) conv_state_update_kernel(const T* __restrict__ x, int64_t x_stride, float* __restrict__ conv_state,
                                                                const int32_t* __restrict__ state_slots,
                                                                const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k,
                                                                const int32_t* __restrict__ ctx_lens, int channels, int taps) {
    B200_PDL_SYNC();
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const bool has_hist = sp.klen - sp.qlen > 0;
    float* hist = conv_state + (int64_t)state_slots[s] * (taps - 1) * channels;
    for (int j = 0; j < taps - 1; ++j) {                   // ascending: row j reads row j + qlen > j of the old history
        const int m = sp.qlen - (taps - 1) + j;
        float v = 0.f;
        if (m >= 0) v = ldf(x + (int64_t)(sp.q0 + m) * x_stride + c);
        else if (has_hist) v = hist[(int64_t)(taps - 1 + m) * channels + c];
        hist[(int64_t)j * channels + c] = v;
    }
}

__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

constexpr int SCAN_LANES = 4;          // lanes that share one channel's state
constexpr int SCAN_CH = 32;            // channels per CTA (128 threads)

// NPL states per lane: state n = k * SCAN_LANES + sub, k < NPL.
// MODE 0: whole portion, slot to slot.  1: chunk from zero, end state and sum of dt to the workspace.  3: chunk from the
// workspace's start state, y out.
template <typename T, int NPL, int MODE>
__global__ void __launch_bounds__(SCAN_LANES * SCAN_CH) selective_scan_kernel(
    const T* __restrict__ u,            // [n, channels]
    const T* __restrict__ dt_raw,       // [n, channels]
    const T* __restrict__ dt_bias,      // [channels]
    const float* __restrict__ A,        // [channels, nstate]  (negative)
    const T* __restrict__ Bm, const T* __restrict__ Cm, int64_t bc_stride,   // [n, nstate] with a row stride
    const T* __restrict__ Dv,           // [channels]
    const T* __restrict__ z, int64_t z_stride,                               // [n, channels] with a row stride
    float* __restrict__ state,          // [slots, channels, nstate]
    const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k,
    const int32_t* __restrict__ ctx_lens, T* __restrict__ y, int channels, int nstate, int chunk_len, int nchunks,
    float* __restrict__ ws_state, float* __restrict__ ws_sumdt) {
    B200_PDL_SYNC();
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int i_begin = MODE == 0 ? 0 : blockIdx.z * chunk_len;
    if (i_begin >= sp.qlen) return;
    const int i_end = MODE == 0 ? sp.qlen : min(sp.qlen, i_begin + chunk_len);
    const int sub = threadIdx.x % SCAN_LANES;
    const int c = blockIdx.x * SCAN_CH + threadIdx.x / SCAN_LANES;
    const bool live = c < channels;
    const int cc = live ? c : channels - 1;
    float* st = state + ((int64_t)state_slots[s] * channels + cc) * nstate;
    const bool has_hist = sp.klen - sp.qlen > 0;
    float S[NPL], a[NPL];
#pragma unroll
    for (int k = 0; k < NPL; ++k) {
        const int n = k * SCAN_LANES + sub;
        if (MODE == 0) S[k] = (has_hist && n < nstate) ? st[n] : 0.f;
        else if (MODE == 1) S[k] = 0.f;
        else S[k] = n < nstate ? ws_state[(((int64_t)s * nchunks + blockIdx.z) * channels + cc) * nstate + n] : 0.f;
        a[k] = n < nstate ? A[(int64_t)cc * nstate + n] : 0.f;
    }
    const float bias = ldf(dt_bias + cc), dskip = ldf(Dv + cc);
    // Tokens in groups of TB: all loads of a group are issued before its (serial) arithmetic, so the recurrence waits for
    // memory once per group instead of once per token.
    constexpr int TB = NPL <= 4 ? 8 : (NPL <= 8 ? 4 : 2);
    float sumdt = 0.f;
    for (int i0 = i_begin; i0 < i_end; i0 += TB) {
        float uu[TB], dr[TB], zz[TB], bb[TB][NPL], cv[TB][NPL];
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            if (i0 + j >= i_end) {                          // past the portion: nothing to fetch (a single-token step has one row)
                uu[j] = dr[j] = zz[j] = 0.f;
#pragma unroll
                for (int k = 0; k < NPL; ++k) bb[j][k] = cv[j][k] = 0.f;
                continue;
            }
            const int64_t t = sp.q0 + i0 + j;
            uu[j] = ldf(u + t * channels + cc);
            dr[j] = ldf(dt_raw + t * channels + cc);
            zz[j] = ldf(z + t * z_stride + cc);
#pragma unroll
            for (int k = 0; k < NPL; ++k) {
                const int n = min(k * SCAN_LANES + sub, nstate - 1);
                bb[j][k] = ldf(Bm + t * bc_stride + n);
                cv[j][k] = ldf(Cm + t * bc_stride + n);
            }
        }
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            if (i0 + j < i_end) {
                const float dt = softplusf_(dr[j] + bias);
                sumdt += dt;
                const float du = dt * uu[j];
                float part = 0.f;
#pragma unroll
                for (int k = 0; k < NPL; ++k) {
                    if (k * SCAN_LANES + sub < nstate) {
                        S[k] = fmaf(expf(dt * a[k]), S[k], du * bb[j][k]);
                        part = fmaf(S[k], cv[j][k], part);
                    }
                }
                if (MODE == 1) continue;
                part += __shfl_xor_sync(0xffffffffu, part, 1);
                part += __shfl_xor_sync(0xffffffffu, part, 2);
                if (live && sub == 0) stf(y + (sp.q0 + i0 + j) * (int64_t)channels + cc, (part + dskip * uu[j]) * siluf_(zz[j]));
            }
        }
    }
    if (MODE == 3) return;
    if (MODE == 1) {
        st = ws_state + (((int64_t)s * nchunks + blockIdx.z) * channels + cc) * nstate;
        if (live && sub == 0) ws_sumdt[((int64_t)s * nchunks + blockIdx.z) * channels + cc] = sumdt;
    }
    if (live) {
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const int n = k * SCAN_LANES + sub;
            if (n < nstate) st[n] = S[k];
        }
    }
}

template <typename T>
__device__ __forceinline__ float decay_exp(float x);
template <>
__device__ __forceinline__ float decay_exp<float>(float x) { return expf(x); }
template <>
__device__ __forceinline__ float decay_exp<__nv_bfloat16>(float x) { return __expf(x); }     // x <= 0; the fast form is exact to ~2 ulp there

// One thread per channel with all NS (>= nstate) states in registers: the form for the usual small states (<= 32).  B and C of
// a group of 8 tokens are staged in shared memory once per CTA (every channel reads the same values); u, dt and z are read
// coalesced across the CTA's 128 channels.  Same MODEs as above.
constexpr int SCH_TB = 8;
template <typename T, int NS, int MODE>
__global__ void __launch_bounds__(128) selective_scan_ch_kernel(
    const T* __restrict__ u, const T* __restrict__ dt_raw, const T* __restrict__ dt_bias, const float* __restrict__ A,
    const T* __restrict__ Bm, const T* __restrict__ Cm, int64_t bc_stride, const T* __restrict__ Dv, const T* __restrict__ z,
    int64_t z_stride, float* __restrict__ state, const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
    const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens, T* __restrict__ y, int channels, int nstate,
    int chunk_len, int nchunks, float* __restrict__ ws_state, float* __restrict__ ws_sumdt) {
    B200_PDL_SYNC();
    __shared__ float sB[SCH_TB][NS], sC[SCH_TB][NS];
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int i_begin = MODE == 0 ? 0 : blockIdx.z * chunk_len;
    if (i_begin >= sp.qlen) return;
    const int i_end = MODE == 0 ? sp.qlen : min(sp.qlen, i_begin + chunk_len);
    const int c = blockIdx.x * 128 + threadIdx.x;
    const bool live = c < channels;
    const int cc = live ? c : channels - 1;
    float* st = state + ((int64_t)state_slots[s] * channels + cc) * nstate;
    const bool has_hist = sp.klen - sp.qlen > 0;
    float S[NS], a[NS];
#pragma unroll
    for (int n = 0; n < NS; ++n) {
        const bool in = n < nstate;
        if (MODE == 0) S[n] = (has_hist && in) ? st[n] : 0.f;
        else if (MODE == 1) S[n] = 0.f;
        else S[n] = in ? ws_state[(((int64_t)s * nchunks + blockIdx.z) * channels + cc) * nstate + n] : 0.f;
        a[n] = in ? A[(int64_t)cc * nstate + n] : 0.f;
    }
    const float bias = ldf(dt_bias + cc), dskip = ldf(Dv + cc);
    float sumdt = 0.f;
    for (int i0 = i_begin; i0 < i_end; i0 += SCH_TB) {
        __syncthreads();
        for (int e = threadIdx.x; e < SCH_TB * NS * 2; e += 128) {
            const int j = e / (2 * NS), r = e - j * 2 * NS, n = r % NS;
            float v = 0.f;
            if (i0 + j < i_end && n < nstate) v = ldf((r < NS ? Bm : Cm) + (int64_t)(sp.q0 + i0 + j) * bc_stride + n);
            (r < NS ? sB : sC)[j][n] = v;
        }
        float uu[SCH_TB], dr[SCH_TB], zz[SCH_TB];
#pragma unroll
        for (int j = 0; j < SCH_TB; ++j) {
            const bool in = i0 + j < i_end;
            const int64_t t = sp.q0 + (in ? i0 + j : i_begin);
            uu[j] = in ? ldf(u + t * channels + cc) : 0.f;
            dr[j] = in ? ldf(dt_raw + t * channels + cc) : 0.f;
            zz[j] = (in && MODE != 1) ? ldf(z + t * z_stride + cc) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < SCH_TB; ++j) {
            if (i0 + j < i_end) {
                const float dt = softplusf_(dr[j] + bias);
                const float du = dt * uu[j];
                sumdt += dt;
                float part = 0.f;
#pragma unroll
                for (int n = 0; n < NS; ++n) {
                    S[n] = fmaf(decay_exp<T>(dt * a[n]), S[n], du * sB[j][n]);
                    part = fmaf(S[n], sC[j][n], part);
                }
                if (MODE != 1 && live) stf(y + (sp.q0 + i0 + j) * (int64_t)channels + cc, (part + dskip * uu[j]) * siluf_(zz[j]));
            }
        }
    }
    if (MODE == 3 || !live) return;
    if (MODE == 1) {
        st = ws_state + (((int64_t)s * nchunks + blockIdx.z) * channels + cc) * nstate;
        ws_sumdt[((int64_t)s * nchunks + blockIdx.z) * channels + cc] = sumdt;
    }
#pragma unroll
    for (int n = 0; n < NS; ++n)
        if (n < nstate) st[n] = S[n];
}

// Chains the chunks of every sequence: ws_state[z] goes from "end state of chunk z started at zero" to "state at the start
// of chunk z"; the slot receives the state after the last chunk.
__global__ void __launch_bounds__(256) scan_carry_kernel(const float* __restrict__ A, float* __restrict__ state,
                                                         const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
                                                         const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens, int channels,
                                                         int nstate, int chunk_len, int nchunks, float* __restrict__ ws_state,
                                                         const float* __restrict__ ws_sumdt) {
    B200_PDL_SYNC();
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (int64_t)channels * nstate) return;
    const int c = (int)(e / nstate);
    float* slot = state + (int64_t)state_slots[s] * channels * nstate + e;
    float carry = (sp.klen - sp.qlen > 0) ? *slot : 0.f;
    const float a = A[e];
    const int used = (sp.qlen + chunk_len - 1) / chunk_len;
    for (int z = 0; z < used; ++z) {
        float* w = ws_state + ((int64_t)s * nchunks + z) * channels * nstate + e;
        const float end = *w;
        *w = carry;
        carry = fmaf(expf(a * ws_sumdt[((int64_t)s * nchunks + z) * channels + c]), carry, end);
    }
    *slot = carry;
}

}  // namespace

extern "C" int b200m_causal_conv(const void* x, int64_t x_stride, const void* w, const void* bias, float* conv_state,
                                 const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens,
                                 void* out, int num_seqs, int max_q, int channels, int taps, int act, int is32, void* stream) {
    if (!x || !w || !conv_state || !state_slots || !out || channels <= 0 || taps <= 0) return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (num_seqs <= 0 || max_q <= 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int tok_tile = 64;
    dim3 grid((channels + 255) / 256, (max_q + tok_tile - 1) / tok_tile, num_seqs);
    B200M_DISPATCH(is32, B200_LAUNCH((causal_conv_kernel<T>), grid, 256, 0, st, static_cast<const T*>(x), x_stride,
                                     static_cast<const T*>(w), static_cast<const T*>(bias), conv_state, state_slots, cu_q, cu_k,
                                     ctx_lens, static_cast<T*>(out), channels, taps, tok_tile, act));
    int rc = b200_launch_status(nullptr);
    if (rc != B200_OK || taps == 1) return rc;
    dim3 grid2((channels + 255) / 256, num_seqs);
    B200M_DISPATCH(is32, B200_LAUNCH((conv_state_update_kernel<T>), grid2, 256, 0, st, static_cast<const T*>(x), x_stride,
                                     conv_state, state_slots, cu_q, cu_k, ctx_lens, channels, taps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_selective_scan(const void* u, const void* dt_raw, const void* dt_bias, const float* A, const void* Bm,
                                    const void* Cm, int64_t bc_stride, const void* Dv, const void* z, int64_t z_stride,
                                    float* state, const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k,
                                    const int32_t* ctx_lens, void* y, int num_seqs, int channels, int nstate, int chunk_len, int max_q,
                                    float* ws, int is32, void* stream) {
    if (!u || !dt_raw || !dt_bias || !A || !Bm || !Cm || !Dv || !z || !state || !state_slots || !y) return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (channels <= 0 || nstate <= 0) return B200_EINVAL;
    if (nstate > 32 * SCAN_LANES) return B200_EUNSUPPORTED;
    if (num_seqs <= 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool chunked = ws != nullptr && chunk_len > 0 && max_q > chunk_len;
    const int nchunks = chunked ? (max_q + chunk_len - 1) / chunk_len : 1;
    float* ws_state = ws;
    float* ws_sumdt = ws ? ws + (int64_t)num_seqs * nchunks * channels * nstate : nullptr;
    dim3 grid((channels + SCAN_CH - 1) / SCAN_CH, num_seqs, 1);
#define SCAN_GO(N, MODE)                                                                                                       \
    B200M_DISPATCH(is32, B200_LAUNCH((selective_scan_kernel<T, N, MODE>), grid, SCAN_LANES * SCAN_CH, 0, st,                    \
                                     static_cast<const T*>(u), static_cast<const T*>(dt_raw), static_cast<const T*>(dt_bias), A, \
                                     static_cast<const T*>(Bm), static_cast<const T*>(Cm), bc_stride, static_cast<const T*>(Dv), \
                                     static_cast<const T*>(z), z_stride, state, state_slots, cu_q, cu_k, ctx_lens,             \
                                     static_cast<T*>(y), channels, nstate, chunk_len, nchunks, ws_state, ws_sumdt))
#define SCH_GO(N, MODE)                                                                                                        \
    B200M_DISPATCH(is32, B200_LAUNCH((selective_scan_ch_kernel<T, N, MODE>), gridc, 128, 0, st, static_cast<const T*>(u),       \
                                     static_cast<const T*>(dt_raw), static_cast<const T*>(dt_bias), A, static_cast<const T*>(Bm), \
                                     static_cast<const T*>(Cm), bc_stride, static_cast<const T*>(Dv), static_cast<const T*>(z),  \
                                     z_stride, state, state_slots, cu_q, cu_k, ctx_lens, static_cast<T*>(y), channels, nstate,  \
                                     chunk_len, nchunks, ws_state, ws_sumdt))
#define SCAN_ALL(MODE)                  \
    do {                                \
        if (nstate <= 8) SCH_GO(8, MODE);        \
        else if (nstate <= 16) SCH_GO(16, MODE); \
        else if (nstate <= 32) SCH_GO(32, MODE); \
        else if (npl <= 2) SCAN_GO(2, MODE);  \
        else if (npl <= 4) SCAN_GO(4, MODE);  \
        else if (npl <= 8) SCAN_GO(8, MODE);  \
        else if (npl <= 16) SCAN_GO(16, MODE); \
        else SCAN_GO(32, MODE);               \
    } while (0)
    const int npl = (nstate + SCAN_LANES - 1) / SCAN_LANES;
    dim3 gridc((channels + 127) / 128, num_seqs, chunked ? nchunks : 1);
    if (!chunked) {
        SCAN_ALL(0);
        return b200_launch_status(nullptr);
    }
    grid.z = nchunks;
    SCAN_ALL(1);
    int rc = b200_launch_status(nullptr);
    if (rc != B200_OK) return rc;
    const int64_t cn = (int64_t)channels * nstate;
    B200_LAUNCH((scan_carry_kernel), dim3((unsigned)((cn + 255) / 256), num_seqs), 256, 0, st, A, state, state_slots, cu_q, cu_k, ctx_lens,
                channels, nstate, chunk_len, nchunks, ws_state, (const float*)ws_sumdt);
    rc = b200_launch_status(nullptr);
    if (rc != B200_OK) return rc;
    SCAN_ALL(3);
#undef SCAN_ALL
#undef SCH_GO
#undef SCAN_GO
    return b200_launch_status(nullptr);
}

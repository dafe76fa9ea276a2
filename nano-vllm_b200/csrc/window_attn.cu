// Grouped-query attention with a sliding window and a linear distance bias over a paged key/value cache.
//
// Per token the cache holds one row [k (G * dim) | v (G * vdim)] per layer that owns a key/value projection; query head h
// reads key/value head h / (H / G).  There is no rotation: position enters through the bias and the window only.
//     s_ij = (q_i . k_j) * scale - slope[h] * (i - j),   visible: 0 <= i - j < window or j < keep_first   (window <= 0: every j <= i)
//     p = softmax over the visible j,   out_i = sum_j p_ij v_j
// The kernels read whatever the cache rows hold: a design that rotates its keys stores them rotated (headnorm_rope_store_kernel).
// Softmax statistics and the output accumulate in fp32 in both element types.
//
//   qk_norm_store_kernel : RMS norm of the WHOLE query projection and of the whole key projection (one statistic per token
//                          over all heads, weight per column), queries normalised in place, keys and values scattered to the
//                          token's cache slot
//   window_attn_kernel   : any mix of prompt portions and single tokens on the fp32 FMA pipe (one warp per (token, head),
//                          key/value tiles shared by the warps of a CTA through shared memory)
//   window_attn_mma_kernel (bf16): the same on the tensor cores, 64 (token, head) rows x 64-key tiles, double-buffered
//                          asynchronous copies; single-token steps may split a long window over several CTAs
#include "mix_common.cuh"

namespace {

constexpr int WA_WARPS = 8;
constexpr int WA_TILE = 32;

template <typename T>
__global__ void __launch_bounds__(256) qk_norm_store_kernel(T* __restrict__ qkv, int64_t stride, int q_cols, int k_cols, int v_cols,
                                                            const T* __restrict__ wq, const T* __restrict__ wk,
                                                            const int32_t* __restrict__ slots, T* __restrict__ cache, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[8];
    const int t = blockIdx.x;
    T* x = qkv + (int64_t)t * stride;
    if (wq != nullptr) {
        float q = 0.f;
        for (int c = threadIdx.x; c < q_cols; c += blockDim.x) {
            const float v = ldf(x + c);
            q = fmaf(v, v, q);
        }
        const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)q_cols + eps);
        for (int c = threadIdx.x; c < q_cols; c += blockDim.x) stf(x + c, ldf(x + c) * rstd * ldf(wq + c));
    }
    if (k_cols + v_cols == 0) return;
    const int slot = slots[t];
    if (slot < 0) return;                                  // block-uniform
    T* dst = cache + (int64_t)slot * (k_cols + v_cols);
    const T* k = x + q_cols;
    float rstd = 1.0f;
    if (wk != nullptr) {
        float q = 0.f;
        for (int c = threadIdx.x; c < k_cols; c += blockDim.x) {
            const float v = ldf(k + c);
            q = fmaf(v, v, q);
        }
        rstd = 1.0f / sqrtf(block_sum(q, red) / (float)k_cols + eps);
    }
    for (int c = threadIdx.x; c < k_cols; c += blockDim.x) stf(dst + c, wk ? ldf(k + c) * rstd * ldf(wk + c) : ldf(k + c));
    for (int c = threadIdx.x; c < v_cols; c += blockDim.x) dst[k_cols + c] = k[k_cols + c];
}

// bf16 rows whose three parts are multiples of 8 columns: 128-bit accesses, 8 columns per thread and step
__global__ void __launch_bounds__(256) qk_norm_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, int64_t stride, int q_cols, int k_cols,
                                                                int v_cols, const __nv_bfloat16* __restrict__ wq,
                                                                const __nv_bfloat16* __restrict__ wk, const int32_t* __restrict__ slots,
                                                                __nv_bfloat16* __restrict__ cache, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[8];
    const int t = blockIdx.x;
    __nv_bfloat16* x = qkv + (int64_t)t * stride;
    auto sum_sq = [&](const __nv_bfloat16* p, int cols) {
        float q = 0.f;
        for (int c = threadIdx.x * 8; c < cols; c += 256 * 8) {
            float f[8];
            unpack8(*reinterpret_cast<const uint4*>(p + c), f);
#pragma unroll
            for (int e = 0; e < 8; ++e) q = fmaf(f[e], f[e], q);
        }
        return block_sum(q, red);
    };
    auto scaled = [&](const __nv_bfloat16* p, const __nv_bfloat16* w, float rstd, int c) {
        float f[8], g[8];
        unpack8(*reinterpret_cast<const uint4*>(p + c), f);
        unpack8(*reinterpret_cast<const uint4*>(w + c), g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = f[e] * rstd * g[e];
        return pack8(f);
    };
    if (wq != nullptr) {
        const float rstd = 1.0f / sqrtf(sum_sq(x, q_cols) / (float)q_cols + eps);
        for (int c = threadIdx.x * 8; c < q_cols; c += 256 * 8) *reinterpret_cast<uint4*>(x + c) = scaled(x, wq, rstd, c);
    }
    if (k_cols + v_cols == 0) return;
    const int slot = slots[t];
    if (slot < 0) return;                                  // block-uniform
    __nv_bfloat16* dst = cache + (int64_t)slot * (k_cols + v_cols);
    const __nv_bfloat16* k = x + q_cols;
    const float rstd = wk ? 1.0f / sqrtf(sum_sq(k, k_cols) / (float)k_cols + eps) : 1.0f;
    for (int c = threadIdx.x * 8; c < k_cols + v_cols; c += 256 * 8)
        *reinterpret_cast<uint4*>(dst + c) = (c < k_cols && wk) ? scaled(k, wk, rstd, c) : *reinterpret_cast<const uint4*>(k + c);
}

// One warp per (token, head-in-group) pair; a CTA covers WA_WARPS consecutive pairs of one sequence and one key/value head.
// OACC = ceil(vdim / 32): output accumulators per lane.
// keep_first > 0 (with a window): the first keep_first tokens of a sequence stay visible to every later token; the CTA walks
// those keys first, then the keys of its window.  vsets > 1: every query head's weights are applied to the values of each of
// the vsets (= G) value heads in turn (blockIdx.z names the pair), giving out [total_q, H, vsets, vdim]: what a mixing of the
// heads' weight matrices after the softmax needs.  out32 != nullptr: the result is written there in fp32 instead.
template <typename T, int OACC>
__global__ void __launch_bounds__(WA_WARPS * 32) window_attn_kernel(
    const T* __restrict__ q, int64_t q_stride,        // [total_q, >= H * dim]
    const T* __restrict__ cache, int row_elems, int v_off,
    const int32_t* __restrict__ block_tables, int bt_stride, int block_size,
    const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens,
    const float* __restrict__ slopes, int window, int keep_first, int vsets,
    T* __restrict__ out, float* __restrict__ out32,   // [total_q, H * vsets * vdim]
    int H, int G, int dim, int vdim, float scale) {
    B200_PDL_SYNC();
    extern __shared__ float smem[];
    const int D = dim + vdim;
    const int DS = D | 1;                                  // odd row stride: lanes reading one column of 32 rows hit 32 banks
    float* tile = smem;                                    // [WA_TILE][DS]: k (dim) | v (vdim) of one key/value head
    float* qs = tile + WA_TILE * DS;                       // [WA_WARPS][dim]
    float* pb = qs + WA_WARPS * dim;                       // [WA_WARPS][WA_TILE]
    const int s = blockIdx.y, g = blockIdx.z / vsets, rep = H / G;
    const int vs = blockIdx.z - g * vsets, vh = vsets > 1 ? vs : g;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npairs = sp.qlen * rep;
    const int pair0 = blockIdx.x * WA_WARPS;
    if (pair0 >= npairs) return;
    const int pair = pair0 + warp;
    const bool active = pair < npairs;
    const int i = active ? pair / rep : 0, h = g * rep + (active ? pair % rep : 0);
    const int first = sp.klen - sp.qlen;                   // position of this step's first token
    const int pos = first + i;
    const int i_lo = pair0 / rep, i_hi = min(sp.qlen - 1, (pair0 + WA_WARPS - 1) / rep);
    const int kmax = first + i_hi + 1;                     // keys any warp of this CTA may see: [0, nkeep) and [kmin, kmax)
    const int kmin = window > 0 ? max(0, first + i_lo - window + 1) : 0;
    const int nkeep = min(keep_first, kmin);
    const int my_lo = window > 0 ? max(0, pos - window + 1) : 0;
    float* myq = qs + warp * dim;
    if (active) {
        const T* qr = q + (int64_t)(sp.q0 + i) * q_stride + (int64_t)h * dim;
        for (int c = lane; c < dim; c += 32) myq[c] = ldf(qr + c) * scale;
    }
    const float slope = (active && slopes) ? slopes[h] : 0.f;
    float m = -INFINITY, l = 0.f;
    float acc[OACC];
#pragma unroll
    for (int k = 0; k < OACC; ++k) acc[k] = 0.f;
    const int32_t* bt = block_tables + (int64_t)s * bt_stride;
    const int nwalk = nkeep + (kmax - kmin);               // walked keys: index u < nkeep is key u, else key kmin + (u - nkeep)
    for (int u0 = 0; u0 < nwalk; u0 += WA_TILE) {
        __syncthreads();                                   // previous tile consumed (and the queries written)
        const int rows = min(WA_TILE, nwalk - u0);
        for (int e = threadIdx.x; e < rows * D; e += blockDim.x) {
            const int r = e / D, c = e - r * D;
            const int u = u0 + r;
            const int j = u < nkeep ? u : kmin + (u - nkeep);
            const int64_t slot = (int64_t)bt[j / block_size] * block_size + (j % block_size);
            const T* src = cache + slot * row_elems;
            tile[r * DS + c] = ldf(c < dim ? src + (int64_t)g * dim + c : src + v_off + (int64_t)vh * vdim + (c - dim));
        }
        __syncthreads();
        const int u = u0 + lane;
        const int j = u < nkeep ? u : kmin + (u - nkeep);
        const bool valid = active && lane < rows && j <= pos && (j >= my_lo || j < keep_first);
        if (__any_sync(0xffffffffu, valid)) {              // the tile holds at least one key this row sees
            float sc = -INFINITY;
            if (valid) {
                const float* kr = tile + lane * DS;
                float a = 0.f;
                for (int c = 0; c < dim; ++c) a = fmaf(myq[c], kr[c], a);
                sc = a - slope * (float)(pos - j);
            }
            const float m_new = fmaxf(m, warp_max(sc));
            const float alpha = expf(m - m_new);
            const float p = valid ? expf(sc - m_new) : 0.f;
            l = l * alpha + warp_sum(p);
            m = m_new;
            pb[warp * WA_TILE + lane] = p;
            __syncwarp();
#pragma unroll
            for (int k = 0; k < OACC; ++k) {
                const int c = lane + 32 * k;
                float a = acc[k] * alpha;
                if (c < vdim)
                    for (int r = 0; r < rows; ++r) a = fmaf(pb[warp * WA_TILE + r], tile[r * DS + dim + c], a);
                acc[k] = a;
            }
            __syncwarp();
        }
    }
    if (active) {
        const float inv = 1.0f / l;
        const int64_t o = (((int64_t)(sp.q0 + i) * H + h) * vsets + vs) * vdim;
#pragma unroll
        for (int k = 0; k < OACC; ++k) {
            const int c = lane + 32 * k;
            if (c < vdim) {
                if (out32) out32[o + c] = acc[k] * inv;
                else stf(out + o + c, acc[k] * inv);
            }
        }
    }
}

template <typename K>
int wa_ensure_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return B200_OK;
    if (bytes > 227 * 1024) return B200_EUNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
        b200_tls_cuda_error() = cudaGetErrorString(e);
        return B200_ECUDA;
    }
    return B200_OK;
}

template <typename T, int OACC>
int launch_window_fma(const void* q, int64_t q_stride, const void* cache, int row_elems, int v_off, const int32_t* block_tables,
                      int bt_stride, int block_size, const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens,
                      const float* slopes, int window, int keep_first, int vsets, void* out, bool out_f32, int num_seqs, int max_q,
                      int H, int G, int dim, int vdim, float scale, cudaStream_t stream) {
    const int D = dim + vdim;
    const size_t smem = sizeof(float) * ((size_t)WA_TILE * (D | 1) + (size_t)WA_WARPS * dim + WA_WARPS * WA_TILE);
    int rc = wa_ensure_smem(window_attn_kernel<T, OACC>, smem);
    if (rc != B200_OK) return rc;
    dim3 grid((max_q * (H / G) + WA_WARPS - 1) / WA_WARPS, num_seqs, G * vsets);
    B200_LAUNCH((window_attn_kernel<T, OACC>), grid, WA_WARPS * 32, smem, stream, static_cast<const T*>(q), q_stride,
                static_cast<const T*>(cache), row_elems, v_off, block_tables, bt_stride, block_size, cu_q, cu_k, ctx_lens, slopes,
                window, keep_first, vsets, out_f32 ? nullptr : static_cast<T*>(out), out_f32 ? static_cast<float*>(out) : nullptr, H,
                G, dim, vdim, scale);
    return b200_launch_status(nullptr);
}


// ---------------------------------------------------------------------------------------------------------------------------
// Tensor-core form (bf16).  The 64 rows of a CTA are (token, head-in-group) pairs of one sequence and one key/value head, 16 per
// warp; key tiles of 64 cache rows (keys DK wide, values DV wide) arrive by 16-byte asynchronous copies into a two-deep ring, the
// next tile in flight while the current one is multiplied.  S = Q K^T and O += P V are mma.sync m16n8k16 with fp32 accumulators
// in registers; scale, distance bias, window and causal mask are applied to the S fragments; the softmax runs in base 2.
// Tiles start at multiples of 64 keys; rows past the last visible key are zero-filled (never read: their page may be absent).
// splits > 1 (single-token steps): blockIdx.z also names a share of the key tiles and the CTA leaves unnormalised partials.
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int WM_BM = 64;
constexpr float WM_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void wm_cp16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void wm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void wm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void wm_ldsm(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void wm_ldsm_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void wm_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float wm_ex2(float x) {       // 2^x on the special-function unit; -inf -> 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t wm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// KS (single-token steps with at most 16 query heads per key/value head): the CTA's 16 rows are shared by its four warps, each
// of which takes 16 of a tile's 64 keys with its own running (max, sum, O); the four are merged through shared memory at the end.
template <int DK, int DV, bool KS, bool QREG, int BN>
__global__ void __launch_bounds__(128) window_attn_mma_kernel(
    const __nv_bfloat16* __restrict__ q, int64_t q_stride, const __nv_bfloat16* __restrict__ cache, int row_elems, int v_off,
    const int32_t* __restrict__ block_tables, int bt_stride, int block_size, int bs_shift, const int32_t* __restrict__ cu_q,
    const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens, const float* __restrict__ slopes, int window,
    int keep_first, int vsets, __nv_bfloat16* __restrict__ out, float* __restrict__ out32, int H, int G, float scale, int splits,
    float* __restrict__ part) {
    static_assert(!KS || BN == 64, "the key-sharing form shares out 64-key tiles");
    B200_PDL_SYNC();
    constexpr int KSTR = DK + 8, VSTR = DV + 8;           // row strides: 16-byte multiples, odd in 16-byte units (conflict-free ldmatrix)
    constexpr int BM = KS ? 16 : WM_BM;                   // rows of the CTA
    constexpr int WK = KS ? 16 : BN;                   // keys of a tile one warp multiplies
    extern __shared__ __align__(16) unsigned char wm_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(wm_smem);       // [BM][KSTR]
    __nv_bfloat16* Ks = Qs + BM * KSTR;                                  // [2][64][KSTR]
    __nv_bfloat16* Vs = Ks + 2 * BN * KSTR;                           // [2][64][VSTR]
    const int s = blockIdx.y, rep = H / G;
    const int gz = blockIdx.z / splits, split = blockIdx.z - gz * splits;
    const int g = gz / vsets, vs = gz - g * vsets, vh = vsets > 1 ? vs : g;     // key head, value set, value head
    const int HV = H * vsets;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    const int nrows = sp.qlen * rep;
    const int row0 = (gridDim.x - 1 - blockIdx.x) * BM;                  // the last rows of a portion see the most keys: launched first
    if (row0 >= nrows) return;
    const int first = sp.klen - sp.qlen;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t4 = lane & 3;
    const int i_lo = row0 / rep, i_hi = min(sp.qlen - 1, (row0 + BM - 1) / rep);
    const int kmax = first + i_hi + 1;
    const int kmin = window > 0 ? max(0, first + i_lo - window + 1) : 0;
    const int t_lo = kmin / BN, t_hi = (kmax + BN - 1) / BN;    // key tiles of the window: [t_lo, t_hi)
    // kept first tokens: their tiles below the window's are walked first.  Walked tile u is key tile u when u < n_keep, else
    // key tile t_lo + (u - n_keep).
    const int n_keep = (window > 0 && keep_first > 0) ? min((keep_first + BN - 1) / BN, t_lo) : 0;
    int u_lo = 0, u_hi = n_keep + (t_hi - t_lo);
    if (splits > 1) {
        const int nt = u_hi;
        u_lo = (int)(((int64_t)nt * split) / splits);
        u_hi = (int)(((int64_t)nt * (split + 1)) / splits);
    }
    auto tile_of = [&](int u) { return u < n_keep ? u : t_lo + (u - n_keep); };
    const int32_t* bt = block_tables + (int64_t)s * bt_stride;

    // a tile's rows: eight lanes copy one cache row (128 contiguous bytes per step), sixteen rows per pass.  The page numbers of a
    // tile are looked up one tile ahead of its copies, so that the table read never stands between a warp and its next MMAs.
    const int lr = tid >> 3, lc = tid & 7;
    auto lookup = [&](int u, int (&pg)[BN / 16]) {
        const int t = tile_of(u);
#pragma unroll
        for (int p = 0; p < BN / 16; ++p) {
            const int j = t * BN + p * 16 + lr;
            pg[p] = (u < u_hi && j < kmax) ? bt[bs_shift >= 0 ? j >> bs_shift : j / block_size] : -1;
        }
    };
    auto load_tile = [&](int buf, int u, const int (&pg)[BN / 16]) {
        const int j0 = tile_of(u) * BN;
        __nv_bfloat16* kd = Ks + buf * BN * KSTR;
        __nv_bfloat16* vd = Vs + buf * BN * VSTR;
        constexpr int KC = DK / 8, VC = DV / 8;
#pragma unroll
        for (int p = 0; p < BN / 16; ++p) {
            const int r = p * 16 + lr;
            const int j = j0 + r;
            const bool ok = pg[p] >= 0;
            const int in_page = bs_shift >= 0 ? j & (block_size - 1) : j % block_size;
            const __nv_bfloat16* src = ok ? cache + ((int64_t)pg[p] * block_size + in_page) * row_elems : cache;
            const int nb = ok ? 16 : 0;
#pragma unroll
            for (int c = lc; c < KC; c += 8) wm_cp16(smem_u32(kd + r * KSTR + c * 8), ok ? src + g * DK + c * 8 : src, nb);
#pragma unroll
            for (int c = lc; c < VC; c += 8) wm_cp16(smem_u32(vd + r * VSTR + c * 8), ok ? src + v_off + vh * DV + c * 8 : src, nb);
        }
        wm_commit();
    };
    int pg[BN / 16];
    lookup(u_lo, pg);
    if (u_lo < u_hi) load_tile(0, u_lo, pg);
    lookup(u_lo + 1, pg);

    // queries of this CTA's rows (plain loads; visible after the loop's first barrier)
    for (int e = tid; e < BM * (DK / 8); e += 128) {
        const int r = e / (DK / 8), c = e - r * (DK / 8);
        const int rr = row0 + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (rr < nrows) {
            const int i = rr / rep, h = g * rep + (rr - i * rep);
            v = *reinterpret_cast<const uint4*>(q + (int64_t)(sp.q0 + i) * q_stride + (int64_t)h * DK + c * 8);
        }
        *reinterpret_cast<uint4*>(Qs + r * KSTR + c * 8) = v;
    }

    // this thread's two rows: (warp * 16 +) gq and + 8
    const int wrow = KS ? 0 : warp * 16;                  // first row of this warp within the CTA
    const int wkey = KS ? warp * 16 : 0;                  // first key of this warp within a tile
    int pos_r[2];
    float slope2[2];
    bool live[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int rr = row0 + wrow + gq + 8 * hh;
        live[hh] = rr < nrows;
        const int i = live[hh] ? rr / rep : 0;
        pos_r[hh] = first + i;
        slope2[hh] = (live[hh] && slopes) ? slopes[g * rep + (rr - i * rep)] * WM_LOG2E : 0.f;
    }
    // keys any row of this warp sees: [w_lo, w_hi]; keys every row of this warp sees: [f_lo, f_hi] (empty unless all 16 rows are live)
    const int wr0 = row0 + wrow, wr1 = min(nrows - 1, wr0 + 15);
    const int w_hi = wr0 < nrows ? first + wr1 / rep : -1;
    const int w_lo = window > 0 ? max(0, first + wr0 / rep - window + 1) : 0;
    const int f_hi = wr0 + 15 < nrows ? first + wr0 / rep : -1;
    const int f_lo = window > 0 ? max(0, first + wr1 / rep - window + 1) : 0;
    const float scale2 = scale * WM_LOG2E;

    __syncthreads();                                                     // the queries are staged: keep this warp's fragments in registers
    const uint32_t a_base = smem_u32(Qs + (wrow + (lane & 15)) * KSTR + ((lane >> 4) << 3));
    uint32_t qf[QREG ? DK / 16 : 1][4];
    if constexpr (QREG) {
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) wm_ldsm(a_base + kk * 32, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    for (int u = u_lo; u < u_hi; ++u) {
        const int buf = (u - u_lo) & 1;
        if (u + 1 < u_hi) {
            load_tile(buf ^ 1, u + 1, pg);
            lookup(u + 2, pg);
            wm_wait<1>();
        } else {
            wm_wait<0>();
        }
        __syncthreads();
        const int j0 = tile_of(u) * BN + wkey;                        // first key this warp multiplies
        if (w_hi >= j0 && (w_lo < j0 + WK || j0 < keep_first)) {         // warp-uniform: some row of this warp sees some key of its share
            const __nv_bfloat16* kt = Ks + buf * BN * KSTR + wkey * KSTR;
            const __nv_bfloat16* vt = Vs + buf * BN * VSTR + wkey * VSTR;
            float sc[WK / 8][4];
#pragma unroll
            for (int n = 0; n < WK / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
            const uint32_t b_base = smem_u32(kt + ((lane & 7) + ((lane >> 4) << 3)) * KSTR + (((lane >> 3) & 1) << 3));
            {   // S = Q K^T; the next key fragment is loaded before the current one is multiplied
                constexpr int NP = WK / 16, STEPS = (DK / 16) * NP;
                uint32_t bc[4], bn[4] = {0, 0, 0, 0}, ac[4] = {0, 0, 0, 0};
                wm_ldsm(b_base, bc[0], bc[1], bc[2], bc[3]);
#pragma unroll
                for (int st = 0; st < STEPS; ++st) {
                    const int kk = st / NP, np = st % NP;
                    if (!QREG && np == 0) wm_ldsm(a_base + kk * 32, ac[0], ac[1], ac[2], ac[3]);
                    if (st + 1 < STEPS) {
                        const int kn = (st + 1) / NP, nn = (st + 1) % NP;
                        wm_ldsm(b_base + (nn * 16 * KSTR + kn * 16) * 2, bn[0], bn[1], bn[2], bn[3]);
                    }
                    if constexpr (QREG) {
                        wm_mma(sc[2 * np], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], bc[0], bc[1]);
                        wm_mma(sc[2 * np + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], bc[2], bc[3]);
                    } else {
                        wm_mma(sc[2 * np], ac[0], ac[1], ac[2], ac[3], bc[0], bc[1]);
                        wm_mma(sc[2 * np + 1], ac[0], ac[1], ac[2], ac[3], bc[2], bc[3]);
                    }
#pragma unroll
                    for (int x = 0; x < 4; ++x) bc[x] = bn[x];
                }
            }
            // scale, bias, mask; running maximum.  Inside the window of every row of the warp no mask is needed: two FMAs per score.
            float m_new[2] = {m_run[0], m_run[1]};
            if (j0 + WK - 1 <= f_hi && j0 >= f_lo) {
                const float base0 = -slope2[0] * (float)(pos_r[0] - j0 - 2 * t4), base1 = -slope2[1] * (float)(pos_r[1] - j0 - 2 * t4);
#pragma unroll
                for (int n = 0; n < WK / 8; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int hh = e >> 1;
                        const float v = fmaf(sc[n][e], scale2, fmaf(slope2[hh], (float)(n * 8 + (e & 1)), hh ? base1 : base0));
                        sc[n][e] = v;
                        m_new[hh] = fmaxf(m_new[hh], v);
                    }
            } else {
#pragma unroll
                for (int n = 0; n < WK / 8; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int hh = e >> 1;
                        const int jj = j0 + n * 8 + 2 * t4 + (e & 1);
                        const int dist = pos_r[hh] - jj;
                        const bool ok = live[hh] && dist >= 0 && (window <= 0 || dist < window || jj < keep_first);
                        const float v = ok ? fmaf(sc[n][e], scale2, -slope2[hh] * (float)dist) : -INFINITY;
                        sc[n][e] = v;
                        m_new[hh] = fmaxf(m_new[hh], v);
                    }
            }
            float alpha[2], m_use[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                m_new[hh] = fmaxf(m_new[hh], __shfl_xor_sync(0xffffffffu, m_new[hh], 1));
                m_new[hh] = fmaxf(m_new[hh], __shfl_xor_sync(0xffffffffu, m_new[hh], 2));
                m_use[hh] = m_new[hh] == -INFINITY ? 0.f : m_new[hh];    // a row that has seen nothing yet
                alpha[hh] = wm_ex2(m_run[hh] - m_use[hh]);
                m_run[hh] = m_new[hh];
                l_run[hh] *= alpha[hh];
            }
#pragma unroll
            for (int n = 0; n < WK / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = wm_ex2(sc[n][e] - m_use[e >> 1]);
                    sc[n][e] = p;
                    l_run[e >> 1] += p;
                }
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) {
                o[n][0] *= alpha[0];
                o[n][1] *= alpha[0];
                o[n][2] *= alpha[1];
                o[n][3] *= alpha[1];
            }
            // O += P V: P from the S fragments, V through transposing loads
            const uint32_t v_base = smem_u32(vt + ((lane & 7) + (((lane >> 3) & 1) << 3)) * VSTR + ((lane >> 4) << 3));
            {
                constexpr int NP = DV / 16, STEPS = (WK / 16) * NP;
                uint32_t bc[4], bn[4] = {0, 0, 0, 0}, pa[4] = {0, 0, 0, 0};
                wm_ldsm_t(v_base, bc[0], bc[1], bc[2], bc[3]);
#pragma unroll
                for (int st = 0; st < STEPS; ++st) {
                    const int kk = st / NP, np = st % NP;
                    if (np == 0) {
                        pa[0] = wm_pack(sc[2 * kk][0], sc[2 * kk][1]);
                        pa[1] = wm_pack(sc[2 * kk][2], sc[2 * kk][3]);
                        pa[2] = wm_pack(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                        pa[3] = wm_pack(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
                    }
                    if (st + 1 < STEPS) {
                        const int kn = (st + 1) / NP, nn = (st + 1) % NP;
                        wm_ldsm_t(v_base + (kn * 16 * VSTR + nn * 16) * 2, bn[0], bn[1], bn[2], bn[3]);
                    }
                    wm_mma(o[2 * np], pa[0], pa[1], pa[2], pa[3], bc[0], bc[1]);
                    wm_mma(o[2 * np + 1], pa[0], pa[1], pa[2], pa[3], bc[2], bc[3]);
#pragma unroll
                    for (int x = 0; x < 4; ++x) bc[x] = bn[x];
                }
            }
        }
        __syncthreads();                                                 // the tile is consumed: its buffer may be refilled
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
    if constexpr (KS) {
        // merge the four warps' partials of the 16 rows through shared memory (the value buffers: all tiles are consumed)
        float* scr = reinterpret_cast<float*>(Vs);                       // [4][16][DV + 2]: max, sum, O
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float* pr = scr + ((size_t)warp * 16 + gq + 8 * hh) * (DV + 2);
            if (t4 == 0) {
                pr[0] = m_run[hh];
                pr[1] = l_run[hh];
            }
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) {
                pr[2 + n * 8 + 2 * t4] = o[n][2 * hh];
                pr[2 + n * 8 + 2 * t4 + 1] = o[n][2 * hh + 1];
            }
        }
        __syncthreads();
        for (int e = tid; e < 16 * DV; e += 128) {
            const int r = e / DV, c = e - r * DV;
            const int rr = row0 + r;
            if (rr >= nrows) continue;
            const float* pr = scr + (size_t)r * (DV + 2);
            constexpr int WSTEP = 16 * (DV + 2);
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) M = fmaxf(M, pr[w * WSTEP]);
            float L = 0.f, a = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = pr[w * WSTEP];
                if (mw != -INFINITY) {
                    const float f = exp2f(mw - M);
                    L = fmaf(pr[w * WSTEP + 1], f, L);
                    a = fmaf(pr[w * WSTEP + 2 + c], f, a);
                }
            }
            const int i = rr / rep, hv = (g * rep + (rr - i * rep)) * vsets + vs;
            if (splits > 1) {
                float* pp = part + (((int64_t)s * splits + split) * HV + hv) * (DV + 2);
                if (c == 0) {
                    pp[0] = M;
                    pp[1] = L;
                }
                pp[2 + c] = a;
            } else if (out32) {
                out32[((int64_t)(sp.q0 + i) * HV + hv) * DV + c] = a / L;
            } else {
                out[((int64_t)(sp.q0 + i) * HV + hv) * DV + c] = __float2bfloat16_rn(a / L);
            }
        }
    } else {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int rr = row0 + warp * 16 + gq + 8 * hh;
        if (rr >= nrows) continue;
        const int i = rr / rep, hv = (g * rep + (rr - i * rep)) * vsets + vs;
        if (splits > 1) {                                                // decode rows only (one token per sequence): i == 0
            float* pp = part + (((int64_t)s * splits + split) * HV + hv) * (DV + 2);
            if (t4 == 0) {
                pp[0] = m_run[hh];
                pp[1] = l_run[hh];
            }
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) {
                pp[2 + n * 8 + 2 * t4] = o[n][2 * hh];
                pp[2 + n * 8 + 2 * t4 + 1] = o[n][2 * hh + 1];
            }
        } else {
            const float inv = 1.0f / l_run[hh];
            const int64_t ob = ((int64_t)(sp.q0 + i) * HV + hv) * DV;
            if (out32) {
#pragma unroll
                for (int n = 0; n < DV / 8; ++n)
                    *reinterpret_cast<float2*>(out32 + ob + n * 8 + 2 * t4) = make_float2(o[n][2 * hh] * inv, o[n][2 * hh + 1] * inv);
            } else {
#pragma unroll
                for (int n = 0; n < DV / 8; ++n)
                    *reinterpret_cast<uint32_t*>(out + ob + n * 8 + 2 * t4) = wm_pack(o[n][2 * hh] * inv, o[n][2 * hh + 1] * inv);
            }
        }
    }
    }
}

// out[s, h, :] = sum_k acc_k 2^(m_k - M) / sum_k l_k 2^(m_k - M) over the `splits` partials of a decode row
__global__ void window_merge_kernel(const float* __restrict__ part, const int32_t* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out,
                                    float* __restrict__ out32, int H, int vdim, int splits) {
    B200_PDL_SYNC();
    const int s = blockIdx.x, h = blockIdx.y;
    if (ctx_lens[s] <= 0) return;
    const float* base = part + ((int64_t)s * splits * H + h) * (vdim + 2);
    const int64_t step = (int64_t)H * (vdim + 2);
    float M = -INFINITY;
    for (int k = 0; k < splits; ++k) M = fmaxf(M, base[k * step]);
    float L = 0.f;
    for (int k = 0; k < splits; ++k) L += base[k * step + 1] * exp2f(base[k * step] - M);
    const float inv = 1.0f / L;
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
        float a = 0.f;
        for (int k = 0; k < splits; ++k) {
            const float mk = base[k * step];
            if (mk != -INFINITY) a = fmaf(base[k * step + 2 + c], exp2f(mk - M), a);
        }
        if (out32) out32[((int64_t)s * H + h) * vdim + c] = a * inv;
        else out[((int64_t)s * H + h) * vdim + c] = __float2bfloat16_rn(a * inv);
    }
}

template <int DK, int DV, bool KS, bool QREG, int BN>
int launch_window_mma_as(const void* q, int64_t q_stride, const void* cache, int row_elems, int v_off, const int32_t* block_tables,
                         int bt_stride, int block_size, const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens,
                         const float* slopes, int window, int keep_first, int vsets, void* out, bool out_f32, int num_seqs, int max_q,
                         int H, int G, float scale, int splits, float* part, cudaStream_t stream) {
    using bf = __nv_bfloat16;
    constexpr int BM = KS ? 16 : WM_BM;
    const size_t smem = sizeof(bf) * ((size_t)BM * (DK + 8) + 2 * (size_t)BN * (DK + 8) + 2 * (size_t)BN * (DV + 8));
    int rc = wa_ensure_smem(window_attn_mma_kernel<DK, DV, KS, QREG, BN>, smem);
    if (rc != B200_OK) return rc;
    int bs_shift = -1;
    if ((block_size & (block_size - 1)) == 0)
        for (bs_shift = 0; (1 << bs_shift) < block_size; ++bs_shift) {}
    dim3 grid((max_q * (H / G) + BM - 1) / BM, num_seqs, G * vsets * splits);
    bf* out16 = out_f32 ? nullptr : static_cast<bf*>(out);
    float* out32 = out_f32 ? static_cast<float*>(out) : nullptr;
    B200_LAUNCH((window_attn_mma_kernel<DK, DV, KS, QREG, BN>), grid, 128, smem, stream, static_cast<const bf*>(q), q_stride,
                static_cast<const bf*>(cache), row_elems, v_off, block_tables, bt_stride, block_size, bs_shift, cu_q, cu_k, ctx_lens,
                slopes, window, keep_first, vsets, out16, out32, H, G, scale, splits, part);
    rc = b200_launch_status(nullptr);
    if (rc != B200_OK || splits <= 1) return rc;
    B200_LAUNCH((window_merge_kernel), dim3(num_seqs, H * vsets), DV < 64 ? 32 : 64, 0, stream, part, ctx_lens, out16, out32, H * vsets, DV,
                splits);
    return b200_launch_status(nullptr);
}

template <int DK, int DV>
int launch_window_mma(const void* q, int64_t q_stride, const void* cache, int row_elems, int v_off, const int32_t* block_tables,
                      int bt_stride, int block_size, const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens,
                      const float* slopes, int window, int keep_first, int vsets, void* out, bool out_f32, int num_seqs, int max_q, int H,
                      int G, float scale, int splits, float* part, cudaStream_t stream) {
    if (cu_q == nullptr && H / G <= 16)                   // single-token step: the four warps share every key tile
        return launch_window_mma_as<DK, DV, true, true, 64>(q, q_stride, cache, row_elems, v_off, block_tables, bt_stride, block_size, cu_q, cu_k,
                                                  ctx_lens, slopes, window, keep_first, vsets, out, out_f32, num_seqs, max_q, H, G, scale, splits, part, stream);
    // row-tiled form: query fragments are re-read from shared memory per key tile (measured faster than 32 more live registers)
    // (32-key tiles, which let four CTAs instead of two share an SM at 128-wide heads, were measured and are not faster)
    return launch_window_mma_as<DK, DV, false, false, 64>(q, q_stride, cache, row_elems, v_off, block_tables, bt_stride, block_size, cu_q, cu_k,
                                                          ctx_lens, slopes, window, keep_first, vsets, out, out_f32, num_seqs, max_q, H, G, scale, splits, part, stream);
}

}  // namespace

extern "C" int b200m_qk_norm_store(void* qkv, int64_t stride, int q_cols, int k_cols, int v_cols, const void* q_norm_w,
                                   const void* k_norm_w, const int32_t* slots, void* cache, int n, float eps, int is32,
                                   void* stream) {
    if (!qkv || n < 0 || q_cols < 0 || k_cols < 0 || v_cols < 0 || stride < q_cols + k_cols + v_cols) return B200_EINVAL;
    if (k_cols + v_cols > 0 && (!slots || !cache)) return B200_EINVAL;
    if (n == 0) return B200_OK;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(q_norm_w) |
                           reinterpret_cast<uintptr_t>(k_norm_w);
    if (!is32 && ptrs % 16 == 0 && stride % 8 == 0 && q_cols % 8 == 0 && k_cols % 8 == 0 && v_cols % 8 == 0) {
        using bf = __nv_bfloat16;
        B200_LAUNCH((qk_norm_store_vec_kernel), n, 256, 0, static_cast<cudaStream_t>(stream), static_cast<bf*>(qkv), stride, q_cols, k_cols,
                    v_cols, static_cast<const bf*>(q_norm_w), static_cast<const bf*>(k_norm_w), slots, static_cast<bf*>(cache), eps);
        return b200_launch_status(nullptr);
    }
    B200M_DISPATCH(is32, B200_LAUNCH((qk_norm_store_kernel<T>), n, 256, 0, static_cast<cudaStream_t>(stream), static_cast<T*>(qkv),
                                     stride, q_cols, k_cols, v_cols, static_cast<const T*>(q_norm_w),
                                     static_cast<const T*>(k_norm_w), slots, static_cast<T*>(cache), eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_window_attention(const void* q, int64_t q_stride, const void* cache, int row_elems, int v_off,
                                      const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q,
                                      const int32_t* cu_k, const int32_t* ctx_lens, const float* slopes, int window, int keep_first,
                                      int all_values, void* out, int total_q, int num_seqs, int max_q, int num_heads, int num_kv_heads,
                                      int dim, int vdim, float scale, int is32, int flags, int splits, float* part, void* stream) {
    if (!q || !cache || !block_tables || !out || total_q < 0 || num_seqs < 0 || num_heads <= 0 || num_kv_heads <= 0 ||
        num_heads % num_kv_heads || dim <= 0 || vdim <= 0 || block_size <= 0 || keep_first < 0)
        return B200_EINVAL;
    const int vsets = all_values ? num_kv_heads : 1;
    const bool out_f32 = (flags & 2) != 0 && !is32;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (total_q == 0 || num_seqs == 0 || max_q <= 0) return B200_OK;
    if (vdim > 512) return B200_EUNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache)) % 16 == 0) && q_stride % 8 == 0 &&
                         row_elems % 8 == 0 && v_off % 8 == 0;
    if (!is32 && !(flags & 1) && aligned && (dim == 32 || dim == 64 || dim == 128) && (vdim == 32 || vdim == 64 || vdim == 128)) {
        if (cu_q != nullptr || splits < 1) splits = 1;                  // keys are split for single-token steps only
        if (splits > 1 && !part) return B200_EINVAL;
#define WA_MMA(DK, DV)                                                                                                           \
    if (dim == DK && vdim == DV)                                                                                                 \
        return launch_window_mma<DK, DV>(q, q_stride, cache, row_elems, v_off, block_tables, bt_stride, block_size, cu_q, cu_k,  \
                                         ctx_lens, slopes, window, keep_first, vsets, out, out_f32, num_seqs, max_q, num_heads,  \
                                         num_kv_heads, scale, splits, part, st)
        WA_MMA(32, 32);
        WA_MMA(32, 64);
        WA_MMA(32, 128);
        WA_MMA(64, 32);
        WA_MMA(64, 64);
        WA_MMA(64, 128);
        WA_MMA(128, 32);
        WA_MMA(128, 64);
        WA_MMA(128, 128);
#undef WA_MMA
    }
#define WA_FMA(OACC)                                                                                                             \
    B200M_DISPATCH(is32, return (launch_window_fma<T, OACC>(q, q_stride, cache, row_elems, v_off, block_tables, bt_stride,       \
                                                            block_size, cu_q, cu_k, ctx_lens, slopes, window, keep_first, vsets, \
                                                            out, out_f32, num_seqs, max_q, num_heads, num_kv_heads, dim, vdim,   \
                                                            scale, st)))
    const int oacc = (vdim + 31) / 32;
    if (oacc <= 1) WA_FMA(1);
    if (oacc <= 2) WA_FMA(2);
    if (oacc <= 4) WA_FMA(4);
    if (oacc <= 8) WA_FMA(8);
    WA_FMA(16);
#undef WA_FMA
    return B200_EUNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------------------------------------
// Per-head query/key norm with a partial pair rotation, unit-RMS values, and the mixing of the heads' attention weights.
//
//   headnorm_rope_store_kernel : per token and head, q <- rms_norm(q) * wq (one weight vector of `dim` elements shared by all
//                                heads), the pairs (2i, 2i + 1), i < rope_dims / 2, turned by the token's position, in place;
//                                keys the same with wk and scattered to the token's cache row; values divided by their root mean
//                                square (no weight) and scattered next to the keys.  One warp per head, fp32 throughout, one
//                                rounding at the store.
//   head_mix_gate_kernel       : out[t, h, :] = c * gate(t, h, :) * sum_g mix[h, g] * acc[t, g, h / (H / G), :], where acc[t, g, v, :]
//                                is head g's softmax weights applied to the values of value head v (window attention with
//                                all_values): mixing the weight matrices of the heads after the softmax is linear in them, so
//                                it commutes with the product by the values.  gate = sigmoid of a projection column.
// ---------------------------------------------------------------------------------------------------------------------------
namespace {

template <typename T>
__global__ void __launch_bounds__(128) headnorm_rope_store_kernel(T* __restrict__ x, int64_t stride, int q_off, int k_off, int v_off, int H,
                                                                  int G, int dim, int vdim, const T* __restrict__ wq,
                                                                  const T* __restrict__ wk, int v_unit, const float* __restrict__ cos_sin,
                                                                  int rope_dims, const float* __restrict__ v_cos_sin, int v_rope_dims,
                                                                  const int64_t* __restrict__ positions,
                                                                  const int32_t* __restrict__ slots, T* __restrict__ cache, float eps) {
    B200_PDL_SYNC();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    T* row = x + (int64_t)t * stride;
    const int slot = slots ? slots[t] : -1;
    const float* cs = cos_sin ? cos_sin + positions[t] * rope_dims : nullptr;
    const float* vcs = v_cos_sin ? v_cos_sin + positions[t] * v_rope_dims : nullptr;
    T* crow = (cache && slot >= 0) ? cache + (int64_t)slot * ((int64_t)G * (dim + vdim)) : nullptr;
    for (int r = warp; r < H + 2 * G; r += nw) {
        const bool is_q = r < H, is_k = !is_q && r < H + G;
        const int d = (is_q || is_k) ? dim : vdim;
        const T* src = is_q ? row + q_off + (int64_t)r * dim : is_k ? row + k_off + (int64_t)(r - H) * dim : row + v_off + (int64_t)(r - H - G) * vdim;
        T* dst = is_q ? row + q_off + (int64_t)r * dim
                      : (crow ? (is_k ? crow + (int64_t)(r - H) * dim : crow + (int64_t)G * dim + (int64_t)(r - H - G) * vdim) : nullptr);
        if (dst == nullptr) continue;                      // keys and values of a token without a cache slot
        const T* w = is_q ? wq : is_k ? wk : nullptr;
        const bool normed = is_q ? wq != nullptr : is_k ? wk != nullptr : v_unit != 0;
        float rstd = 1.0f;
        if (normed) {
            float ss = 0.f;
            for (int c = lane; c < d; c += 32) {
                const float v = ldf(src + c);
                ss = fmaf(v, v, ss);
            }
            rstd = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
        }
        // queries and keys turn by one table, values (when asked for) by their own, over their own width
        const float* rcs = (is_q || is_k) ? cs : vcs;
        const bool rot = rcs != nullptr;
        const int half = ((is_q || is_k) ? rope_dims : v_rope_dims) / 2;
        for (int c = 2 * lane; c < d; c += 64) {           // a lane owns whole pairs
            float a = ldf(src + c) * rstd, b = c + 1 < d ? ldf(src + c + 1) * rstd : 0.f;
            if (w) {
                a *= ldf(w + c);
                if (c + 1 < d) b *= ldf(w + c + 1);
            }
            const int i = c >> 1;
            if (rot && i < half) {
                const float co = rcs[i], si = rcs[half + i];
                const float ra = a * co - b * si, rb = b * co + a * si;
                a = ra;
                b = rb;
            }
            stf(dst + c, a);
            if (c + 1 < d) stf(dst + c + 1, b);
        }
    }
}

// out[t, h, :] = rotate(acc[t, h, :], sign * position) * sigmoid(gate[t, h, :]): a thread per pair of elements of a head.
template <typename T, typename A>
__global__ void __launch_bounds__(256) head_rotate_gate_kernel(const A* __restrict__ acc, int64_t acc_tok_stride, int64_t acc_head_stride,
                                                               const float* __restrict__ cos_sin, int rope_dims, int layout, float sign,
                                                               const int64_t* __restrict__ positions, const T* __restrict__ gate,
                                                               int64_t gate_stride, T* __restrict__ out, int64_t out_stride, int H, int vdim) {
    B200_PDL_SYNC();
    const int64_t t = blockIdx.x;
    const int half = rope_dims / 2, pairs = (vdim + 1) / 2;
    const float* cs = cos_sin ? cos_sin + positions[t] * rope_dims : nullptr;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < H * pairs; e += gridDim.y * blockDim.x) {
        const int h = e / pairs, p = e - h * pairs;
        // pair p of the head: rotated pairs first (p < half), then the elements past rope_dims two at a time
        int e0, e1;
        if (p < half) {
            e0 = layout ? p : 2 * p;
            e1 = layout ? p + half : 2 * p + 1;
        } else {
            e0 = rope_dims + 2 * (p - half);
            e1 = e0 + 1;
        }
        const A* a = acc + t * acc_tok_stride + (int64_t)h * acc_head_stride;
        float u = ldf(a + e0), v = e1 < vdim ? ldf(a + e1) : 0.f;
        if (cs != nullptr && p < half) {
            const float co = cs[p], si = sign * cs[half + p];
            const float ru = u * co - v * si, rv = v * co + u * si;
            u = ru;
            v = rv;
        }
        const int64_t o = (int64_t)h * vdim;
        if (gate) {
            u *= sigmoidf_(ldf(gate + t * gate_stride + o + e0));
            if (e1 < vdim) v *= sigmoidf_(ldf(gate + t * gate_stride + o + e1));
        }
        stf(out + t * out_stride + o + e0, u);
        if (e1 < vdim) stf(out + t * out_stride + o + e1, v);
    }
}

}  // namespace

extern "C" int b200m_head_rotate_gate(const void* acc, int acc_f32, int64_t acc_tok_stride, int64_t acc_head_stride, const float* cos_sin,
                                      int rope_dims, int layout, float sign, const int64_t* positions, const void* gate, int64_t gate_stride,
                                      void* out, int64_t out_stride, int n, int num_heads, int vdim, int is32, void* stream) {
    if (!acc || !out || n < 0 || num_heads <= 0 || vdim <= 0 || rope_dims < 0 || rope_dims > vdim || (rope_dims & 1)) return B200_EINVAL;
    if (cos_sin && rope_dims > 0 && !positions) return B200_EINVAL;
    if (n == 0) return B200_OK;
    if (rope_dims == 0) cos_sin = nullptr;
    if (cos_sin == nullptr) rope_dims = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int work = num_heads * ((vdim + 1) / 2);
    dim3 grid(n, (unsigned)((work + 1023) / 1024));                 // up to four pairs per thread
    if (is32 || acc_f32) {
        B200M_DISPATCH(is32, B200_LAUNCH((head_rotate_gate_kernel<T, float>), grid, 256, 0, st, static_cast<const float*>(acc), acc_tok_stride,
                                         acc_head_stride, cos_sin, rope_dims, layout, sign, positions, static_cast<const T*>(gate), gate_stride,
                                         static_cast<T*>(out), out_stride, num_heads, vdim));
    } else {
        B200_LAUNCH((head_rotate_gate_kernel<__nv_bfloat16, __nv_bfloat16>), grid, 256, 0, st, static_cast<const __nv_bfloat16*>(acc),
                    acc_tok_stride, acc_head_stride, cos_sin, rope_dims, layout, sign, positions, static_cast<const __nv_bfloat16*>(gate),
                    gate_stride, static_cast<__nv_bfloat16*>(out), out_stride, num_heads, vdim);
    }
    return b200_launch_status(nullptr);
}

namespace {

// One thread per (value head v, VEC columns) of a token: it reads head g's accumulator for that value head once and feeds the
// H / G output heads that own value head v (eight at a time), so every accumulator element is read once.  The mixing matrix
// sits in shared memory.  VEC = 4 (fp32 accumulators, vdim a multiple of four): 128-bit accumulator reads.
template <typename T, typename A, int VEC>
__global__ void __launch_bounds__(256) head_mix_gate_kernel(const A* __restrict__ acc, const float* __restrict__ mix, const T* __restrict__ gate,
                                                            int64_t gate_stride, T* __restrict__ out, int64_t out_stride, float out_scale,
                                                            int H, int G, int vdim) {
    B200_PDL_SYNC();
    constexpr int RB = 8;
    extern __shared__ float hm_mix[];                      // [H][H]
    for (int e = threadIdx.x; e < H * H; e += blockDim.x) hm_mix[e] = mix[e];
    __syncthreads();
    const int64_t t = blockIdx.x;
    const int rep = H / G, vq = vdim / VEC;
    const A* a = acc + t * (int64_t)H * G * vdim;
    for (int e = threadIdx.x; e < G * vq; e += blockDim.x) {
        const int v = e / vq, c = (e - v * vq) * VEC;
        for (int r0 = 0; r0 < rep; r0 += RB) {
            float sum[RB][VEC];
#pragma unroll
            for (int r = 0; r < RB; ++r)
#pragma unroll
                for (int x = 0; x < VEC; ++x) sum[r][x] = 0.f;
            const float* m = hm_mix + (v * rep + r0) * H;
            for (int g = 0; g < H; ++g) {
                float xv[VEC];
                const A* src = a + ((int64_t)g * G + v) * vdim + c;
                if constexpr (VEC == 4) {
                    const float4 f = *reinterpret_cast<const float4*>(src);
                    xv[0] = f.x, xv[1] = f.y, xv[2] = f.z, xv[3] = f.w;
                } else {
                    xv[0] = ldf(src);
                }
#pragma unroll
                for (int r = 0; r < RB; ++r)
                    if (r0 + r < rep) {
                        const float w = m[r * H + g];
#pragma unroll
                        for (int x = 0; x < VEC; ++x) sum[r][x] = fmaf(w, xv[x], sum[r][x]);
                    }
            }
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                if (r0 + r >= rep) break;
                const int o = (v * rep + r0 + r) * vdim + c;
#pragma unroll
                for (int x = 0; x < VEC; ++x) {
                    const float z = gate ? sigmoidf_(ldf(gate + t * gate_stride + o + x)) : 1.0f;
                    stf(out + t * out_stride + o + x, sum[r][x] * z * out_scale);
                }
            }
        }
    }
}

}  // namespace

extern "C" int b200m_headnorm_rope_store(void* x, int64_t stride, int q_off, int k_off, int v_off, int num_heads, int num_kv_heads, int dim,
                                         int vdim, const void* q_norm_w, const void* k_norm_w, int v_unit_norm, const float* cos_sin,
                                         int rope_dims, const float* v_cos_sin, int v_rope_dims, const int64_t* positions,
                                         const int32_t* slots, void* cache, int n, float eps, int is32, void* stream) {
    if (!x || n < 0 || num_heads <= 0 || num_kv_heads <= 0 || dim <= 0 || vdim <= 0 || rope_dims < 0 || rope_dims > dim || (rope_dims & 1))
        return B200_EINVAL;
    if ((cos_sin && rope_dims > 0 && !positions) || (cache && !slots)) return B200_EINVAL;
    if (v_rope_dims < 0 || v_rope_dims > vdim || (v_rope_dims & 1) || (v_cos_sin && v_rope_dims > 0 && !positions)) return B200_EINVAL;
    if (v_rope_dims == 0) v_cos_sin = nullptr;
    if (n == 0) return B200_OK;
    if (rope_dims == 0) cos_sin = nullptr;
    B200M_DISPATCH(is32, B200_LAUNCH((headnorm_rope_store_kernel<T>), n, 128, 0, static_cast<cudaStream_t>(stream), static_cast<T*>(x), stride,
                                     q_off, k_off, v_off, num_heads, num_kv_heads, dim, vdim, static_cast<const T*>(q_norm_w),
                                     static_cast<const T*>(k_norm_w), v_unit_norm, cos_sin, rope_dims, v_cos_sin, v_rope_dims, positions, slots,
                                     static_cast<T*>(cache), eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_head_mix_gate(const void* acc, int acc_f32, const float* mix, const void* gate, int64_t gate_stride, void* out,
                                   int64_t out_stride, float out_scale, int n, int num_heads, int num_kv_heads, int vdim, int is32,
                                   void* stream) {
    if (!acc || !mix || !out || n < 0 || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || vdim <= 0) return B200_EINVAL;
    if (n == 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = sizeof(float) * (size_t)num_heads * num_heads;
    if (smem > 48 * 1024) return B200_EUNSUPPORTED;
    const bool vec = (is32 || acc_f32) && vdim % 4 == 0 && reinterpret_cast<uintptr_t>(acc) % 16 == 0;
    if (vec) {
        B200M_DISPATCH(is32, B200_LAUNCH((head_mix_gate_kernel<T, float, 4>), n, 256, smem, st, static_cast<const float*>(acc), mix,
                                         static_cast<const T*>(gate), gate_stride, static_cast<T*>(out), out_stride, out_scale, num_heads,
                                         num_kv_heads, vdim));
    } else if (is32 || acc_f32) {
        B200M_DISPATCH(is32, B200_LAUNCH((head_mix_gate_kernel<T, float, 1>), n, 256, smem, st, static_cast<const float*>(acc), mix,
                                         static_cast<const T*>(gate), gate_stride, static_cast<T*>(out), out_stride, out_scale, num_heads,
                                         num_kv_heads, vdim));
    } else {
        using bf = __nv_bfloat16;
        B200_LAUNCH((head_mix_gate_kernel<bf, bf, 1>), n, 256, smem, st, static_cast<const bf*>(acc), mix, static_cast<const bf*>(gate),
                    gate_stride, static_cast<bf*>(out), out_stride, out_scale, num_heads, num_kv_heads, vdim);
    }
    return b200_launch_status(nullptr);
}

// Latent attention over a paged cache of compressed keys.
//
// Per token the cache holds one row [c (kv_rank, RMS-normed) | k_rot (rot_dim, rotated)] shared by all heads.  With the
// key/value up-projections folded into the query and the output (q_lat[h] = W_uk[h]^T q_nope[h]; head output =
// W_uv[h] * sum_j p_j c_j) attention is multi-query over those rows:
//     s_j = (q_lat[h] . c_j + q_rot[h] . k_rot_j) * scale,   p = softmax over {s_j, j <= pos} and a per-head sink logit
// The sink takes part in the maximum and the denominator only: it is a key with a fixed score and a zero value; without one
// (sink == NULL) the softmax is the ordinary one.  window > 0 hides the keys with pos - j >= window; key tiles wholly below
// every row's window are never staged.  The rotated parts pair (2i, 2i+1) (layout 0) or (i, i + rope_dims/2) (layout 1).
//
//   latent_store_kernel : RMS norm of the latent, rotation of the shared key part, scatter to the token's cache slot
//   latent_attn_kernel  : any mix of prompt portions and single tokens (one warp per (token, head), key tiles shared
//                         by the warps of a CTA through shared memory)
//   latent_decode_kernel: one token per sequence, keys split over CTAs, partial (max, sum, acc) merged by the last CTA
#include "mix_common.cuh"

namespace {

constexpr int LA_WARPS = 8;
constexpr int LA_TILE = 32;

// interleaved rotation of `dims` leading elements of a rot_dim-long vector; cs = [cos (dims/2) | sin (dims/2)] of the position
__device__ __forceinline__ void rotate_pair(float u, float v, float c, float s, float& ou, float& ov) {
    ou = u * c - v * s;
    ov = v * c + u * s;
}
// elements of pair i: (2i, 2i+1) in the interleaved layout, (i, i + half) in the halves layout
__device__ __forceinline__ int pair_lo(int i, int half, int layout) { return layout ? i : 2 * i; }
__device__ __forceinline__ int pair_hi(int i, int half, int layout) { return layout ? i + half : 2 * i + 1; }

template <typename T>
__global__ void __launch_bounds__(128) latent_store_kernel(const T* __restrict__ dkv, int64_t stride, const T* __restrict__ w,
                                                           const float* __restrict__ cos_sin, int rope_dims,
                                                           const int64_t* __restrict__ positions, const int32_t* __restrict__ slots,
                                                           T* __restrict__ cache, int rank, int rot_dim, float eps, int layout) {
    B200_PDL_SYNC();
    __shared__ float red[4];
    const int t = blockIdx.x;
    const int slot = slots[t];
    if (slot < 0) return;
    const T* x = dkv + (int64_t)t * stride;
    T* dst = cache + (int64_t)slot * (rank + rot_dim);
    float q = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float v = ldf(x + c);
        q = fmaf(v, v, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)rank + eps);
    for (int c = threadIdx.x; c < rank; c += blockDim.x) stf(dst + c, ldf(x + c) * rstd * ldf(w + c));
    const float* cs = cos_sin + positions[t] * rope_dims;
    const int half = rope_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float a, b;
        const int e0 = rank + pair_lo(i, half, layout), e1 = rank + pair_hi(i, half, layout);
        rotate_pair(ldf(x + e0), ldf(x + e1), cs[i], cs[half + i], a, b);
        stf(dst + e0, a);
        stf(dst + e1, b);
    }
    for (int c = rope_dims + threadIdx.x; c < rot_dim; c += blockDim.x) stf(dst + rank + c, ldf(x + rank + c));
}

// q for one (token, head) into shared memory: [q_lat (rank) | rotated q_rot (rot_dim)], fp32, pre-multiplied by scale
template <typename T>
__device__ __forceinline__ void load_query(float* qs, const T* q_lat, const T* q_rot, const float* cs, int rank, int rot_dim,
                                           int rope_dims, float scale, int lane, int layout) {
    for (int c = lane; c < rank; c += 32) qs[c] = ldf(q_lat + c) * scale;
    const int half = rope_dims / 2;
    for (int i = lane; i < half; i += 32) {
        float a, b;
        const int e0 = pair_lo(i, half, layout), e1 = pair_hi(i, half, layout);
        rotate_pair(ldf(q_rot + e0), ldf(q_rot + e1), cs[i], cs[half + i], a, b);
        qs[rank + e0] = a * scale;
        qs[rank + e1] = b * scale;
    }
    for (int c = rope_dims + lane; c < rot_dim; c += 32) qs[rank + c] = ldf(q_rot + c) * scale;
}

// OACC = ceil(rank / 32): output accumulators per lane.
template <typename T, int OACC>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attn_kernel(
    const T* __restrict__ q_lat,        // [H, total_q, rank]
    const T* __restrict__ q_raw,        // token t, head h at t * q_tok_stride + h * q_head_stride; the rotated part starts at q_rot_off of each head
    int64_t q_tok_stride, int q_head_stride, int q_rot_off,
    const T* __restrict__ cache,        // [slots, rank + rot_dim]
    const int32_t* __restrict__ block_tables, int bt_stride, int block_size,
    const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens,
    const float* __restrict__ sink,     // [H]
    const float* __restrict__ cos_sin, int rope_dims,
    T* __restrict__ out,                // [H, total_q, rank]
    int total_q, int H, int rank, int rot_dim, float scale, int window, int layout) {
    B200_PDL_SYNC();
    extern __shared__ float smem[];
    const int D = rank + rot_dim;
    const int DS = D | 1;                                  // odd row stride: lanes reading one column of 32 rows hit 32 banks
    float* tile = smem;                                    // [LA_TILE][DS]
    float* qs = tile + LA_TILE * DS;                       // [LA_WARPS][D]
    float* pb = qs + LA_WARPS * D;                         // [LA_WARPS][LA_TILE]
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair0 = blockIdx.x * LA_WARPS;
    if (pair0 >= sp.qlen * H) return;
    const int pair = pair0 + warp;
    const bool active = pair < sp.qlen * H;
    const int i = active ? pair / H : 0, h = active ? pair % H : 0;
    const int first = sp.klen - sp.qlen;                   // position of this step's first token
    const int pos = first + i;
    const int i_hi = min(sp.qlen - 1, (pair0 + LA_WARPS - 1) / H);
    const int kmax = first + i_hi + 1;                     // keys any warp of this CTA may see
    float* myq = qs + warp * D;
    if (active) {
        const int64_t row = sp.q0 + i;
        load_query(myq, q_lat + ((int64_t)h * total_q + row) * rank, q_raw + row * q_tok_stride + (int64_t)h * q_head_stride + q_rot_off,
                   cos_sin + (int64_t)pos * rope_dims, rank, rot_dim, rope_dims, scale, lane, layout);
    }
    float m = (active && sink) ? sink[h] : -1e30f, l = sink ? 1.0f : 0.f;      // the sink: score sink[h], weight exp(0) = 1, no value
    float acc[OACC];
#pragma unroll
    for (int k = 0; k < OACC; ++k) acc[k] = 0.f;
    const int32_t* bt = block_tables + (int64_t)s * bt_stride;
    // the first tile any row of this CTA sees: the lowest row's window start
    const int j_first = window > 0 ? (max(first + pair0 / H - window + 1, 0) / LA_TILE) * LA_TILE : 0;
    for (int j0 = j_first; j0 < kmax; j0 += LA_TILE) {
        __syncthreads();                                   // previous tile consumed (and the queries written)
        const int rows = min(LA_TILE, kmax - j0);
        for (int e = threadIdx.x; e < rows * D; e += blockDim.x) {
            const int r = e / D, c = e - r * D;
            const int j = j0 + r;
            const int64_t slot = (int64_t)bt[j / block_size] * block_size + (j % block_size);
            tile[r * DS + c] = ldf(cache + slot * D + c);
        }
        __syncthreads();
        if (active && j0 <= pos && (window <= 0 || j0 + LA_TILE > pos - window + 1)) {
            const bool valid = lane < rows && j0 + lane <= pos && (window <= 0 || pos - (j0 + lane) < window);
            float sc = -INFINITY;
            if (valid) {
                const float* kr = tile + lane * DS;
                float a = 0.f;
                for (int c = 0; c < D; ++c) a = fmaf(myq[c], kr[c], a);
                sc = a;
            }
            const float m_new = fmaxf(m, warp_max(sc));
            const float alpha = expf(m - m_new);
            const float p = valid ? expf(sc - m_new) : 0.f;
            l = l * alpha + warp_sum(p);
            m = m_new;
            pb[warp * LA_TILE + lane] = p;
            __syncwarp();
            const int nk = min(rows, pos - j0 + 1);
#pragma unroll
            for (int k = 0; k < OACC; ++k) {
                const int c = lane + 32 * k;
                float a = acc[k] * alpha;
                if (c < rank)
                    for (int j = 0; j < nk; ++j) a = fmaf(pb[warp * LA_TILE + j], tile[j * DS + c], a);
                acc[k] = a;
            }
            __syncwarp();
        }
    }
    if (active) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = out + ((int64_t)h * total_q + sp.q0 + i) * rank;
#pragma unroll
        for (int k = 0; k < OACC; ++k) {
            const int c = lane + 32 * k;
            if (c < rank) stf(o + c, acc[k] * inv);
        }
    }
}

template <typename K>
int ensure_smem(K kernel, size_t bytes) {
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
int launch_attn(const void* q_lat, const void* q_raw, int64_t q_tok_stride, int q_head_stride, int q_rot_off, const void* cache,
                const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q, const int32_t* cu_k,
                const int32_t* ctx_lens, const float* sink, const float* cos_sin, int rope_dims, void* out, int total_q,
                int num_seqs, int max_q, int H, int rank, int rot_dim, float scale, int window, int layout, cudaStream_t stream) {
    const int D = rank + rot_dim;
    const size_t smem = sizeof(float) * ((size_t)LA_TILE * (D | 1) + (size_t)LA_WARPS * D + LA_WARPS * LA_TILE);
    int rc = ensure_smem(latent_attn_kernel<T, OACC>, smem);
    if (rc != B200_OK) return rc;
    dim3 grid((max_q * H + LA_WARPS - 1) / LA_WARPS, num_seqs);
    B200_LAUNCH((latent_attn_kernel<T, OACC>), grid, LA_WARPS * 32, smem, stream, static_cast<const T*>(q_lat),
                static_cast<const T*>(q_raw), q_tok_stride, q_head_stride, q_rot_off, static_cast<const T*>(cache), block_tables, bt_stride,
                block_size, cu_q, cu_k, ctx_lens, sink, cos_sin, rope_dims, static_cast<T*>(out), total_q, H, rank, rot_dim,
                scale, window, layout);
    return b200_launch_status(nullptr);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Tensor-core form (bf16): rows of a tile are (token, head) pairs of one sequence, 16 per warp, 4 warps; key tiles of 64 cache
// rows are staged once per CTA and serve as B operand of S = Q K^T (row-major [key][dim]) and, through transposing loads, of
// O += P V over their first `rank` columns.  One CTA covers at most MMA_OC output columns (grid.z walks wider latents and
// recomputes S).  Scores, softmax statistics and O accumulate in fp32 registers; the sink seeds the running maximum and sum.
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int MMA_BM = 64;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__host__ __device__ inline int mma_row_stride(int D) {
    const int Dp = (D + 15) & ~15;
    return Dp + (((Dp >> 3) & 1) ? 16 : 8);          // stride / 8 odd: the 8 rows of an ldmatrix hit 8 different 16-byte bank groups
}

// WS (single-token steps with at most 16 heads): the four warps share the 16 query rows and each takes 16 of a tile's 64 keys,
// leaving one partial per (split, warp).  Only those 16 query rows are staged, and the room that saves holds a second key
// tile: the next tile's asynchronous copies are in flight while the current one is multiplied.
// BN: keys per staged tile (64; 32 for wide rows, so that two CTAs still fit in an SM's shared memory).
template <int NT_O, bool WS, int BN>
__global__ void __launch_bounds__(128) latent_attn_mma_kernel(
    const __nv_bfloat16* __restrict__ q_lat, const __nv_bfloat16* __restrict__ q_raw, int64_t q_tok_stride, int q_head_stride, int q_rot_off,
    const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_tables, int bt_stride, int block_size,
    const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens,
    const float* __restrict__ sink, const float* __restrict__ cos_sin, int rope_dims, __nv_bfloat16* __restrict__ out,
    int total_q, int H, int rank, int rot_dim, float scale, int window, int layout, int splits, float* __restrict__ part) {
    B200_PDL_SYNC();
    constexpr int MMA_BN = BN;
    static_assert(!WS || BN == 64, "the warp-split form shares out 64-key tiles");
    extern __shared__ __align__(16) unsigned char smraw[];
    const int D = rank + rot_dim, Dp = (D + 15) & ~15, DS = mma_row_stride(D);
    constexpr int QR = WS ? 16 : MMA_BM;                  // staged query rows
    constexpr int NBUF = WS ? 2 : 1;                      // staged key tiles
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);
    __nv_bfloat16* Ks = Qs + QR * DS;
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    // the last row tiles of a portion see the most keys: they are launched first
    const int nrows = sp.qlen * H, row0 = (gridDim.x - 1 - blockIdx.x) * MMA_BM;
    if (row0 >= nrows) return;
    // grid.z = (column chunk, key split): with splits > 1 (single-token steps) every CTA covers a contiguous share of the
    // key tiles and leaves unnormalised (acc, max, sum) partials for latent_merge_kernel
    const int split = blockIdx.z % splits;
    const int rc0 = (blockIdx.z / splits) * (NT_O * 8);
    const int first = sp.klen - sp.qlen;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);

    // ---- stage Q (rotating its last rot_dim elements), zero the padding of both tiles: a warp per row, lanes over columns ----
    for (int r = warp; r < QR; r += 4) {
        const int rr = row0 + r;
        const bool live_row = rr < nrows;
        const int i = live_row ? rr / H : 0, h = live_row ? rr - i * H : 0;
        const int64_t tok = sp.q0 + i;
        const __nv_bfloat16* ql = q_lat + ((int64_t)h * total_q + tok) * rank;
        const __nv_bfloat16* qr = q_raw + tok * q_tok_stride + (int64_t)h * q_head_stride + q_rot_off;
        const float* cs = cos_sin + (int64_t)(first + i) * rope_dims;
        const int half = rope_dims >> 1;
        for (int c = lane; c < DS; c += 32) {
            __nv_bfloat16 v = zero;
            if (live_row && c < D) {
                if (c < rank) {
                    v = ql[c];
                } else {
                    const int cr = c - rank;
                    if (cr < rope_dims) {
                        const int p = layout ? (cr < half ? cr : cr - half) : cr >> 1;
                        const bool second = layout ? cr >= half : (cr & 1);
                        const float u = __bfloat162float(qr[pair_lo(p, half, layout)]), w = __bfloat162float(qr[pair_hi(p, half, layout)]);
                        v = __float2bfloat16_rn(second ? (w * cs[p] + u * cs[half + p]) : (u * cs[p] - w * cs[half + p]));
                    } else {
                        v = qr[cr];
                    }
                }
            }
            Qs[r * DS + c] = v;
        }
    }
    for (int r = warp; r < NBUF * MMA_BN; r += 4)
        for (int c = Dp + lane; c < DS; c += 32) Ks[r * DS + c] = zero;
    // rows of this warp: g and g + 8 of its 16
    constexpr int NKT = WS ? 2 : BN / 8;                  // 8-key tiles of S per warp
    const int rwarp = WS ? 0 : warp;                      // which 16 rows of the tile this warp owns
    const int koff = WS ? warp * 16 : 0;                  // first key of the tile this warp looks at
    float m_run[2], l_run[2];
    int pos_row[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int rr = row0 + rwarp * 16 + g + 8 * k;
        const bool live = rr < nrows;
        const int i = live ? rr / H : 0;
        pos_row[k] = live ? first + i : -1;
        m_run[k] = live ? (sink ? sink[rr - i * H] : -1e30f) : 0.f;
        l_run[k] = (sink || !live) ? 1.0f : 0.f;
        if (split > 0 || (WS && warp > 0)) {              // the sink is counted once, by the first partial
            m_run[k] = -1e30f;
            l_run[k] = 0.f;
        }
    }
    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const int np_used = min(NT_O / 2, (rank - rc0 + 15) / 16);       // pairs of 8-column tiles that hold real output columns
    const int i_hi = min(sp.qlen - 1, (row0 + MMA_BM - 1) / H);
    const int kmax = first + i_hi + 1;
    const int warp_pos_max = first + min(sp.qlen - 1, (row0 + rwarp * 16 + 15) / H);
    const bool warp_live = row0 + rwarp * 16 < nrows;
    // smallest position among this warp's live rows (a dead row sees nothing, so the masked path handles warps that have one)
    const int warp_pos_min = (row0 + rwarp * 16 + 15 < nrows) ? first + (row0 + rwarp * 16) / H : -1;
    const int32_t* bt = block_tables + (int64_t)s * bt_stride;
    const uint32_t qs_base = smem_u32(Qs), ks_base = smem_u32(Ks);
    const bool vec = (D & 7) == 0;
    // with a window the walk starts at the tile that holds the first key the CTA's lowest row sees
    const int t_lo = window > 0 ? max(first + row0 / H - window + 1, 0) / MMA_BN : 0;
    const int warp_pos_lo = first + (row0 + rwarp * 16) / H;      // smallest position among this warp's rows
    int j_begin = t_lo * MMA_BN, j_end = kmax;
    if (splits > 1) {
        const int tiles = (kmax + MMA_BN - 1) / MMA_BN - t_lo, per = (tiles + splits - 1) / splits;
        j_begin = (t_lo + split * per) * MMA_BN;
        j_end = min(kmax, (t_lo + (split + 1) * per) * MMA_BN);
    }
    // ---- stage one tile of cache rows: a warp per row (one page lookup), lanes over 16-byte pieces ----
    // a tile that lies inside one page (pages are multiples of the tile, tiles start at multiples of it) needs one lookup
    const bool one_page = (block_size % MMA_BN) == 0;
    auto stage = [&](int j0, int buf) {
        __nv_bfloat16* Kb = Ks + buf * MMA_BN * DS;
        const uint32_t kb = ks_base + (uint32_t)(buf * MMA_BN * DS * 2);
        const __nv_bfloat16* page0 = cache;
        if (one_page) page0 = cache + ((int64_t)bt[j0 / block_size] * block_size + (j0 % block_size)) * D;
        if (one_page && vec && j0 + MMA_BN <= kmax) {
            // the usual tile: whole, inside one page, rows of whole 16-byte pieces.  A lane owns the same pieces of every row
            // of its warp, so a copy costs a pointer step and nothing else.
            for (int c = lane << 3; c < Dp; c += 256) {
                const bool col = c < D;                  // pieces past the row's end are zero-filled (nothing is read)
                const __nv_bfloat16* src = col ? page0 + (int64_t)warp * D + c : cache;
                const int64_t step = col ? 4 * (int64_t)D : 0;
                const uint32_t nbytes = col ? 16u : 0u;
                uint32_t dst = kb + (uint32_t)((warp * DS + c) * 2);
#pragma unroll
                for (int r = 0; r < MMA_BN / 4; ++r) {
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"((const void*)src), "r"(nbytes) : "memory");
                    src += step;
                    dst += (uint32_t)(4 * DS * 2);
                }
            }
            return;
        }
        for (int r = warp; r < MMA_BN; r += 4) {
            const int j = j0 + r;
            const bool in = j < kmax;
            const __nv_bfloat16* src = cache;
            if (in) src = one_page ? page0 + (int64_t)r * D : cache + ((int64_t)bt[j / block_size] * block_size + (j % block_size)) * D;
            if (vec) {                                    // asynchronous 16-byte copies (zero-filled outside the row): all in flight at once
                for (int c = lane << 3; c < Dp; c += 256) {
                    const bool ok = in && c < D;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kb + (uint32_t)((r * DS + c) * 2)),
                                 "l"(ok ? (const void*)(src + c) : (const void*)cache), "r"(ok ? 16 : 0) : "memory");
                }
            } else {
                for (int c = lane; c < Dp; c += 32) Kb[r * DS + c] = (in && c < D) ? src[c] : zero;
            }
        }
    };
    const bool pipelined = NBUF == 2 && vec;              // rows that are not whole 16-byte pieces are staged by plain stores, one tile at a time
    if (pipelined && j_begin < j_end) {
        stage(j_begin, 0);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    int it = 0;
    for (int j0 = j_begin; j0 < j_end; j0 += MMA_BN, ++it) {
        int buf = 0;
        __syncthreads();                                  // the tile of the last iteration is consumed (and Q is written)
        if (pipelined) {
            buf = it & 1;
            if (j0 + MMA_BN < j_end) {                    // the next tile goes into the other buffer while this one is used
                stage(j0 + MMA_BN, buf ^ 1);
                asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
        } else {
            stage(j0, 0);
            asm volatile("cp.async.wait_all;" ::: "memory");
        }
        __syncthreads();
        const uint32_t kt_base = ks_base + (uint32_t)(buf * MMA_BN * DS * 2);
        if (!warp_live || j0 + koff > warp_pos_max) continue;
        if (window > 0 && j0 + koff + NKT * 8 - 1 <= warp_pos_lo - window) continue;      // below every row's window
        // ---- S = Q K^T (16 rows x NKT * 8 keys per warp) ----
        float sc[NKT][4];
#pragma unroll
        for (int n = 0; n < NKT; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
        const uint32_t a_addr = qs_base + (uint32_t)(((rwarp * 16 + (lane & 15)) * DS + ((lane >> 4) << 3)) * 2);
        const uint32_t b_addr = kt_base + (uint32_t)(((koff + (lane & 7) + ((lane >> 4) << 3)) * DS + (((lane >> 3) & 1) << 3)) * 2);
#pragma unroll 4
        for (int kk = 0; kk < Dp; kk += 16) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(a_addr + kk * 2, a0, a1, a2, a3);
#pragma unroll
            for (int np = 0; np < NKT / 2; ++np) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b_addr + (uint32_t)((np * 16 * DS + kk) * 2), b0, b1, b2, b3);
                mma_bf16(sc[2 * np], a0, a1, a2, a3, b0, b1);
                mma_bf16(sc[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // ---- mask, online softmax ----
        float mx[2] = {m_run[0], m_run[1]};
        // tiles wholly behind every row of this warp (the bulk of a long portion) need no mask
        const bool all_visible = j0 + koff + NKT * 8 - 1 <= warp_pos_min && (window <= 0 || j0 + koff > warp_pos_max - window);
        if (all_visible) {
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    sc[n][e] *= scale;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sc[n][e]);
                }
        } else {
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = j0 + koff + n * 8 + 2 * t4 + (e & 1);
                    const int k = e >> 1;
                    const float v = (key <= pos_row[k] && (window <= 0 || pos_row[k] - key < window)) ? sc[n][e] * scale : -INFINITY;
                    sc[n][e] = v;
                    mx[k] = fmaxf(mx[k], v);
                }
        }
        float alpha[2], psum[2] = {0.f, 0.f};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 1));
            mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 2));
            alpha[k] = __expf(m_run[k] - mx[k]);
            m_run[k] = mx[k];
        }
        uint32_t pa[NKT / 2][4];
#pragma unroll
        for (int n = 0; n < NKT; ++n) {
            const float p0 = __expf(sc[n][0] - mx[0]), p1 = __expf(sc[n][1] - mx[0]);
            const float p2 = __expf(sc[n][2] - mx[1]), p3 = __expf(sc[n][3] - mx[1]);
            psum[0] += p0 + p1;
            psum[1] += p2 + p3;
            pa[n >> 1][(n & 1) * 2] = pack_bf16x2(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(p2, p3);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            psum[k] += __shfl_xor_sync(0xffffffffu, psum[k], 1);
            psum[k] += __shfl_xor_sync(0xffffffffu, psum[k], 2);
            l_run[k] = l_run[k] * alpha[k] + psum[k];
        }
        if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {      // the running maxima settle early in a long row
#pragma unroll
            for (int n = 0; n < NT_O; ++n) {
                o[n][0] *= alpha[0];
                o[n][1] *= alpha[0];
                o[n][2] *= alpha[1];
                o[n][3] *= alpha[1];
            }
        }
        // ---- O += P V ----
        const uint32_t v_addr = kt_base + (uint32_t)(((koff + (lane & 7) + (((lane >> 3) & 1) << 3)) * DS + rc0 + ((lane >> 4) << 3)) * 2);
        if (np_used == NT_O / 2) {                        // the usual case, without predicates: loads run ahead of the products
#pragma unroll
            for (int kk = 0; kk < NKT / 2; ++kk) {
#pragma unroll
                for (int np = 0; np < NT_O / 2; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(v_addr + (uint32_t)((kk * 16 * DS + np * 16) * 2), b0, b1, b2, b3);
                    mma_bf16(o[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    mma_bf16(o[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
        } else {
#pragma unroll
            for (int kk = 0; kk < NKT / 2; ++kk) {
#pragma unroll
                for (int np = 0; np < NT_O / 2; ++np) {
                    if (np < np_used) {
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4_t(v_addr + (uint32_t)((kk * 16 * DS + np * 16) * 2), b0, b1, b2, b3);
                        mma_bf16(o[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                        mma_bf16(o[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                    }
                }
            }
        }
    }
    // ---- write ----
    if (splits > 1) {                                     // rows are heads here (one token per sequence)
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int rr = row0 + rwarp * 16 + g + 8 * k;
            if (rr >= nrows) continue;
            const int np = WS ? splits * 4 : splits, pi = WS ? split * 4 + warp : split;
            float* dst = part + (((int64_t)s * np + pi) * H + rr) * (rank + 2);
#pragma unroll
            for (int n = 0; n < NT_O; ++n) {
                const int c = rc0 + n * 8 + 2 * t4;
                if (c < rank) dst[c] = o[n][2 * k];
                if (c + 1 < rank) dst[c + 1] = o[n][2 * k + 1];
            }
            if (rc0 == 0 && t4 == 0) {
                dst[rank] = m_run[k];
                dst[rank + 1] = l_run[k];
            }
        }
        return;
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int rr = row0 + warp * 16 + g + 8 * k;
        if (rr >= nrows) continue;
        const int i = rr / H, h = rr - i * H;
        const float inv = l_run[k] > 0.f ? 1.0f / l_run[k] : 0.f;
        __nv_bfloat16* dst = out + ((int64_t)h * total_q + sp.q0 + i) * rank;
#pragma unroll
        for (int n = 0; n < NT_O; ++n) {
            const int c = rc0 + n * 8 + 2 * t4;
            if (c < rank) dst[c] = __float2bfloat16_rn(o[n][2 * k] * inv);
            if (c + 1 < rank) dst[c + 1] = __float2bfloat16_rn(o[n][2 * k + 1] * inv);
        }
    }
}

// out[h, s, :] = sum_p e^(m_p - M) acc_p / sum_p e^(m_p - M) l_p over the key splits of a single-token step
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ part, const int32_t* __restrict__ ctx_lens, int splits,
                                                           int H, int rank, int total_q, __nv_bfloat16* __restrict__ out) {
    B200_PDL_SYNC();
    const int s = blockIdx.x, h = blockIdx.y;
    if (ctx_lens[s] <= 0) return;
    const float* base = part + ((int64_t)s * splits * H + h) * (rank + 2);
    const int64_t step = (int64_t)H * (rank + 2);
    float M = -1e30f;
    for (int p = 0; p < splits; ++p) M = fmaxf(M, base[p * step + rank]);
    float L = 0.f;
    for (int p = 0; p < splits; ++p) L += __expf(base[p * step + rank] - M) * base[p * step + rank + 1];
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float a = 0.f;
        for (int p = 0; p < splits; ++p) a = fmaf(__expf(base[p * step + rank] - M), base[p * step + c], a);
        out[((int64_t)h * total_q + s) * rank + c] = __float2bfloat16_rn(a * inv);
    }
}

template <int NT_O, bool WS, int BN>
int launch_attn_mma_bn(const void* q_lat, const void* q_raw, int64_t q_tok_stride, int q_head_stride, int q_rot_off, const void* cache,
                    const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q, const int32_t* cu_k,
                    const int32_t* ctx_lens, const float* sink, const float* cos_sin, int rope_dims, void* out, int total_q,
                    int num_seqs, int max_q, int H, int rank, int rot_dim, float scale, int window, int layout, int splits, float* part, cudaStream_t stream) {
    const int DS = mma_row_stride(rank + rot_dim);
    if (splits < 1 || max_q != 1 || cu_q != nullptr || part == nullptr || H > MMA_BM) splits = 1;
    const size_t smem = (size_t)(WS ? 16 + 2 * BN : MMA_BM + BN) * DS * sizeof(__nv_bfloat16);       // as the kernel lays it out
    int rc = ensure_smem(latent_attn_mma_kernel<NT_O, WS, BN>, smem);
    if (rc != B200_OK) return rc;
    dim3 grid((max_q * H + MMA_BM - 1) / MMA_BM, num_seqs, ((rank + NT_O * 8 - 1) / (NT_O * 8)) * splits);
    using bf = __nv_bfloat16;
    B200_LAUNCH((latent_attn_mma_kernel<NT_O, WS, BN>), grid, 128, smem, stream, static_cast<const bf*>(q_lat), static_cast<const bf*>(q_raw),
                q_tok_stride, q_head_stride, q_rot_off, static_cast<const bf*>(cache), block_tables, bt_stride, block_size, cu_q, cu_k, ctx_lens,
                sink, cos_sin, rope_dims, static_cast<bf*>(out), total_q, H, rank, rot_dim, scale, window, layout, splits, part);
    rc = b200_launch_status(nullptr);
    if (rc != B200_OK || splits == 1) return rc;
    B200_LAUNCH((latent_merge_kernel), dim3(num_seqs, H), 128, 0, stream, (const float*)part, ctx_lens, WS ? splits * 4 : splits, H, rank,
                total_q, static_cast<bf*>(out));
    return b200_launch_status(nullptr);
}

template <int NT_O, bool WS>
int launch_attn_mma_ws(const void* q_lat, const void* q_raw, int64_t q_tok_stride, int q_head_stride, int q_rot_off, const void* cache,
                       const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q, const int32_t* cu_k,
                       const int32_t* ctx_lens, const float* sink, const float* cos_sin, int rope_dims, void* out, int total_q,
                       int num_seqs, int max_q, int H, int rank, int rot_dim, float scale, int window, int layout, int splits, float* part, cudaStream_t stream) {
    // 64-key tiles while two CTAs of (64 + 64) staged rows fit in an SM; 32-key tiles for wider rows
    const bool narrow = !WS && (size_t)(MMA_BM + 64) * mma_row_stride(rank + rot_dim) * sizeof(__nv_bfloat16) > 112 * 1024;
    if (narrow)
        return launch_attn_mma_bn<NT_O, false, 32>(q_lat, q_raw, q_tok_stride, q_head_stride, q_rot_off, cache, block_tables, bt_stride, block_size, cu_q, cu_k,
                                                   ctx_lens, sink, cos_sin, rope_dims, out, total_q, num_seqs, max_q, H, rank, rot_dim, scale,
                                                   window, layout, splits, part, stream);
    return launch_attn_mma_bn<NT_O, WS, 64>(q_lat, q_raw, q_tok_stride, q_head_stride, q_rot_off, cache, block_tables, bt_stride, block_size, cu_q, cu_k,
                                            ctx_lens, sink, cos_sin, rope_dims, out, total_q, num_seqs, max_q, H, rank, rot_dim, scale, window, layout,
                                            splits, part, stream);
}

template <int NT_O>
int launch_attn_mma(const void* q_lat, const void* q_raw, int64_t q_tok_stride, int q_head_stride, int q_rot_off, const void* cache,
                    const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q, const int32_t* cu_k,
                    const int32_t* ctx_lens, const float* sink, const float* cos_sin, int rope_dims, void* out, int total_q,
                    int num_seqs, int max_q, int H, int rank, int rot_dim, float scale, int window, int layout, int splits, float* part, cudaStream_t stream) {
    if (splits > 1 && max_q == 1 && cu_q == nullptr && part != nullptr && H <= 16)
        return launch_attn_mma_ws<NT_O, true>(q_lat, q_raw, q_tok_stride, q_head_stride, q_rot_off, cache, block_tables, bt_stride, block_size, cu_q, cu_k,
                                              ctx_lens, sink, cos_sin, rope_dims, out, total_q, num_seqs, max_q, H, rank, rot_dim, scale,
                                              window, layout, splits, part, stream);
    return launch_attn_mma_ws<NT_O, false>(q_lat, q_raw, q_tok_stride, q_head_stride, q_rot_off, cache, block_tables, bt_stride, block_size, cu_q, cu_k,
                                           ctx_lens, sink, cos_sin, rope_dims, out, total_q, num_seqs, max_q, H, rank, rot_dim, scale,
                                           window, layout, splits, part, stream);
}

}  // namespace

extern "C" int b200m_latent_store(const void* dkv, int64_t stride, const void* norm_w, const float* cos_sin, int rope_dims,
                                  const int64_t* positions, const int32_t* slots, void* cache, int n, int rank, int rot_dim,
                                  float eps, int layout, int is32, void* stream) {
    if (!dkv || !norm_w || !cos_sin || !positions || !slots || !cache || n < 0 || rank <= 0 || rot_dim < 0) return B200_EINVAL;
    if (rope_dims < 0 || rope_dims > rot_dim || (rope_dims & 1)) return B200_EINVAL;
    if (n == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((latent_store_kernel<T>), n, 128, 0, static_cast<cudaStream_t>(stream),
                                     static_cast<const T*>(dkv), stride, static_cast<const T*>(norm_w), cos_sin, rope_dims,
                                     positions, slots, static_cast<T*>(cache), rank, rot_dim, eps, layout));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_latent_attention(const void* q_lat, const void* q_raw, int64_t q_tok_stride, int q_head_stride, int q_rot_off, const void* cache,
                                      const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q,
                                      const int32_t* cu_k, const int32_t* ctx_lens, const float* sink, const float* cos_sin,
                                      int rope_dims, void* out, int total_q, int num_seqs, int max_q, int num_heads, int rank,
                                      int rot_dim, float scale, int window, int layout, int is32, int flags, int splits, float* part,
                                      void* stream) {
    if (!q_lat || !q_raw || !cache || !block_tables || !cos_sin || !out) return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (total_q < 0 || num_seqs < 0 || num_heads <= 0 || rank <= 0 || rot_dim < 0 || block_size <= 0) return B200_EINVAL;
    if (rope_dims < 0 || rope_dims > rot_dim || (rope_dims & 1)) return B200_EINVAL;
    if (rank > 512) return B200_EUNSUPPORTED;
    if (total_q == 0 || num_seqs == 0 || max_q <= 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!is32 && !(flags & 1)) {         // bf16: tensor cores; 128 output columns per CTA when the latent fits, else 256 per pass
        if (rank <= 128)
            return launch_attn_mma<16>(q_lat, q_raw, q_tok_stride, q_head_stride, q_rot_off, cache, block_tables, bt_stride, block_size, cu_q, cu_k,
                                       ctx_lens, sink, cos_sin, rope_dims, out, total_q, num_seqs, max_q, num_heads, rank, rot_dim, scale, window, layout, splits, part, st);
        return launch_attn_mma<32>(q_lat, q_raw, q_tok_stride, q_head_stride, q_rot_off, cache, block_tables, bt_stride, block_size, cu_q, cu_k,
                                   ctx_lens, sink, cos_sin, rope_dims, out, total_q, num_seqs, max_q, num_heads, rank, rot_dim, scale, window, layout, splits, part, st);
    }
#define LA_GO(N)                                                                                                              \
    B200M_DISPATCH(is32, return (launch_attn<T, N>(q_lat, q_raw, q_tok_stride, q_head_stride, q_rot_off, cache, block_tables, bt_stride,     \
                                                   block_size, cu_q, cu_k, ctx_lens, sink, cos_sin, rope_dims, out, total_q,  \
                                                   num_seqs, max_q, num_heads, rank, rot_dim, scale, window, layout, st)))
    if (rank <= 128) LA_GO(4);
    if (rank <= 256) LA_GO(8);
    LA_GO(16);
#undef LA_GO
    return B200_EINVAL;
}

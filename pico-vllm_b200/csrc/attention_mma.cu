// Paged causal attention for bfloat16 on tensor cores: one kernel for portions of prompts
// ("prefill") and one for single tokens over a long cache ("decode").  Both keep the query
// heads that share a key/value head in ONE tile (row = token * g + head of the group), so each
// key and value is read once per group, stage keys and values of 64 cache positions at a time in
// shared memory with cp.async (double buffered; rows are found through the block table, so any
// page size works), multiply with mma.sync m16n8k16 (bf16 in, float32 accumulate) and keep the
// running max / sum softmax in float32 registers.  The decode kernel cuts a token's key range
// into n_splits parts (grid.x) and, inside a block, gives each of its 4 warps a quarter of every
// 64-key tile; the four partial results are merged in shared memory, the splits by the combine
// kernel of attention_generic.cu.
//
// Restated from the reference: query head j reads key/value head j / g
// (pico_vllm/kernels/attention.py:31,139); scores * hd^-1/2 (attention.py:92,231); key n visible to
// the query at position p iff n <= p (attention.py:193-198) - and n > p - window when the layer
// has a window; online softmax in float32 (attention.py:189-213); p is rounded to bfloat16 before
// p.v as in the reference's prefill kernel (attention.py:206).  The reference runs one program
// per query head with 16x16 tiles and walks every page of the context, masked or not
// (attention.py:167-169); here tiles beyond the last visible key are never loaded.
#include "common.cuh"

#include "mma_helpers.cuh"

// How a block's threads share the 16-byte pieces of a tile: a power-of-two number of threads per
// row (at least hd/8 pieces), so that no division is needed per piece.  page_shift >= 0 when the
// page size is a power of two.
struct TileMap {
    int chunks;        // 16-byte pieces per row (hd / 8)
    int c;             // this thread's piece of a row (may be >= chunks: the thread then idles)
    int row0, rstep;   // first row and row step of this thread
    int page_shift, page_size;
};
__device__ __forceinline__ TileMap make_tile_map(int hd, int page_size) {
    TileMap tm;
    tm.chunks = hd >> 3;
    int sh = 1;
    while ((1 << sh) < tm.chunks) ++sh;             // threads per row = 2^sh (2 .. 32)
    tm.c = threadIdx.x & ((1 << sh) - 1);
    tm.row0 = threadIdx.x >> sh;
    tm.rstep = MMA_THREADS >> sh;
    tm.page_size = page_size;
    tm.page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    return tm;
}

// Loads keys (or values) of cache positions n0 .. n0+MMA_BN-1 of one key/value head into a
// shared tile [MMA_BN][ld] (ld = hd + 8 elements: the 16 bytes of padding make ldmatrix free of
// bank conflicts for every hd that is a multiple of 16).  Positions outside [n_lo, n_hi) are
// filled with zeros and their pages are not touched.
__device__ __forceinline__ void load_kv_tile(bf16* tile, const bf16* __restrict__ pages, const int* __restrict__ table,
                                             int n0, int n_lo, int n_hi, int kh, int nkv, int hd, int ld,
                                             const TileMap& tm) {
    if (tm.c >= tm.chunks) return;
    for (int key = tm.row0; key < MMA_BN; key += tm.rstep) {
        const int n = n0 + key;
        const bool ok = n >= n_lo && n < n_hi;
        const bf16* src = pages;
        if (ok) {
            int page, off;
            if (tm.page_shift >= 0) {
                page = table[n >> tm.page_shift];
                off = n & (tm.page_size - 1);
            } else {
                const int blk = n / tm.page_size;
                page = table[blk];
                off = n - blk * tm.page_size;
            }
            src = pages + (((size_t)page * nkv + kh) * tm.page_size + off) * hd + tm.c * 8;
        }
        cp_async_16(smem_u32(tile + key * ld + tm.c * 8), src, ok);
    }
}

// One 16-row tile of queries against NT 8-key n-tiles of a shared K tile: s[j] += Q K^T.
template <int HD_MAX, int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const bf16* q_rows, const bf16* k_rows, int hd, int ld,
                                        int lane) {
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int k0 = 0; k0 < HD_MAX; k0 += 16) {
        if (k0 < hd) {
            uint32_t a[4];
            ldmatrix_x4(a, smem_u32(q_rows + a_row * ld + k0 + a_col));
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, smem_u32(k_rows + (j * 8 + b_row) * ld + k0 + b_col));
                mma_bf16(s[j], a, b[0], b[1]);
                mma_bf16(s[j + 1], a, b[2], b[3]);
            }
        }
    }
}

// o[16 x hd] += P[16 x NT*8 keys] V, with P taken from the score registers (rounded to bf16).
template <int HD_MAX, int NT>
__device__ __forceinline__ void pv_tile(float (&o)[HD_MAX / 8][4], const float (&p)[NT][4], const bf16* v_rows, int hd,
                                        int ld, int lane) {
    const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_col = (lane >> 4) * 8;
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {       // 16 keys per step
        uint32_t a[4];
        a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
        a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
        a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
        a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
        for (int d0 = 0; d0 < HD_MAX; d0 += 16) {
            if (d0 < hd) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, smem_u32(v_rows + (kk * 16 + v_row) * ld + d0 + v_col));
                mma_bf16(o[d0 / 8], a, b[0], b[1]);
                mma_bf16(o[d0 / 8 + 1], a, b[2], b[3]);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------ prefill
// grid: (tiles of tokens, kv heads, listed segments).  A block takes `tpt` = 64 / g tokens of one
// segment and the g query heads of one kv head: 64 rows, 16 per warp.
template <int HD_MAX>
__global__ void __launch_bounds__(MMA_THREADS)
paged_prefill_mma_kernel(const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ k_pages,
                         const bf16* __restrict__ v_pages, bf16* __restrict__ out, const int* __restrict__ seg_list,
                         const int* __restrict__ cu_q, const int* __restrict__ positions,
                         const int* __restrict__ block_table, int table_stride, int nh, int nkv, int hd,
                         int page_size, int window, float scale_log2) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int g = nh / nkv;
    const int tpt = 64 / g;                         // tokens per tile (g <= 64)
    const int seg = seg_list ? seg_list[blockIdx.z] : blockIdx.z;
    const int q0 = cu_q[seg], qlen = cu_q[seg + 1] - q0;
    const int tok0 = blockIdx.x * tpt;
    if (tok0 >= qlen) return;
    const int ntok = min(tpt, qlen - tok0);
    const int kh = blockIdx.y;
    const int pos0 = positions[q0] + tok0;          // position of the tile's first token
    const int hi = pos0 + ntok;                     // one past the last visible key of the tile
    const int lo = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int ld = hd + 8;
    const TileMap tm = make_tile_map(hd, page_size);
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);              // [64][ld]
    bf16* k_s = q_s + 64 * ld;                                  // [2][MMA_BN][ld]
    bf16* v_s = k_s + 2 * MMA_BN * ld;                          // [2][MMA_BN][ld]
    const int* table = block_table + (size_t)seg * table_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // queries of the tile -> shared memory (rows beyond the tile's tokens are zero)
    const int chunks = hd >> 3;
    for (int idx = threadIdx.x; idx < 64 * chunks; idx += MMA_THREADS) {
        const int r = idx / chunks, c = idx - r * chunks;
        const int tok = r / g, head = r - tok * g;
        const bool ok = tok < ntok;
        const bf16* src = q + (size_t)(q0 + tok0 + (ok ? tok : 0)) * q_row_stride + (size_t)(kh * g + head) * hd + c * 8;
        cp_async_16(smem_u32(q_s + r * ld + c * 8), src, ok);
    }
    const int ntiles = (hi - lo + MMA_BN - 1) / MMA_BN;
    load_kv_tile(k_s, k_pages, table, lo, lo, hi, kh, nkv, hd, ld, tm);
    load_kv_tile(v_s, v_pages, table, lo, lo, hi, kh, nkv, hd, ld, tm);
    cp_async_commit();

    float o[HD_MAX / 8][4];
#pragma unroll
    for (int i = 0; i < HD_MAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // positions of the two rows this thread holds
    int row_pos[2], row_lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        const int tok = row / g;
        row_pos[r] = tok < ntok ? pos0 + tok : -1;             // -1: a padding row sees nothing
        row_lo[r] = (window > 0 && row_pos[r] + 1 > window) ? row_pos[r] + 1 - window : 0;
    }
    // the last key any row of this warp sees: later tiles are skipped by this warp
    const int warp_last_tok = min(ntok - 1, (warp * 16 + 15) / g);
    const int warp_hi = (warp * 16) / g < ntok ? pos0 + warp_last_tok + 1 : lo;

    for (int t = 0; t < ntiles; ++t) {
        const int n0 = lo + t * MMA_BN;
        const int buf = t & 1;
        if (t + 1 < ntiles) {
            load_kv_tile(k_s + (buf ^ 1) * MMA_BN * ld, k_pages, table, n0 + MMA_BN, lo, hi, kh, nkv, hd, ld, tm);
            load_kv_tile(v_s + (buf ^ 1) * MMA_BN * ld, v_pages, table, n0 + MMA_BN, lo, hi, kh, nkv, hd, ld, tm);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (n0 < warp_hi) {
            float s[MMA_BN / 8][4];
#pragma unroll
            for (int j = 0; j < MMA_BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            qk_tile<HD_MAX, MMA_BN / 8>(s, q_s + warp * 16 * ld, k_s + buf * MMA_BN * ld, hd, ld, lane);
#pragma unroll
            for (int j = 0; j < MMA_BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int n = n0 + j * 8 + (lane & 3) * 2 + (e & 1);
                    const int r = e >> 1;
                    const bool vis = n <= row_pos[r] && n >= row_lo[r];
                    s[j][e] = vis ? s[j][e] * scale_log2 : -INFINITY;
                }
            }
            online_softmax<HD_MAX, MMA_BN / 8>(s, m, l, o);
            pv_tile<HD_MAX, MMA_BN / 8>(o, s, v_s + buf * MMA_BN * ld, hd, ld, lane);
        }
        __syncthreads();      // the buffer is overwritten by the load of tile t+2
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        const int tok = row / g, head = row - tok * g;
        if (tok >= ntok) continue;
        const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
        bf16* dst = out + ((size_t)(q0 + tok0 + tok) * nh + kh * g + head) * hd + (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < HD_MAX / 8; ++i)
            if (i * 8 < hd)
                *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
}

// ------------------------------------------------------------------------------------------ decode
// grid: (splits, kv heads, listed tokens).  One token, the g (<= 16) query heads of one kv head:
// a single 16-row tile.  Warp w takes cache positions 16w .. 16w+15 of every 64-position tile.
template <int HD_MAX>
__global__ void __launch_bounds__(MMA_THREADS)
paged_decode_mma_kernel(const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ k_pages,
                        const bf16* __restrict__ v_pages, bf16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, const int* __restrict__ tok_list,
                        const int* __restrict__ tok_seg, const int* __restrict__ positions,
                        const int* __restrict__ block_table, int table_stride, int nh, int nkv, int hd,
                        int page_size, int window, float scale_log2, int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int g = nh / nkv;
    const int t = tok_list ? tok_list[blockIdx.z] : blockIdx.z;
    const int kh = blockIdx.y, sp = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int hi = pos + 1;                         // pos = -1 (padding): no keys at all
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const int ntiles_all = (hi - lo + MMA_BN - 1) / MMA_BN;
    const int per = (ntiles_all + n_splits - 1) / n_splits;
    const int begin = lo + sp * per * MMA_BN;
    const int end = min(hi, begin + per * MMA_BN);
    const int ntiles = end > begin ? (end - begin + MMA_BN - 1) / MMA_BN : 0;
    const int ld = hd + 8;
    const TileMap tm = make_tile_map(hd, page_size);
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);              // [16][ld]
    bf16* k_s = q_s + 16 * ld;                                  // [DEC_STAGES][MMA_BN][ld]
    bf16* v_s = k_s + DEC_STAGES * MMA_BN * ld;
    const int* table = block_table + (size_t)tok_seg[t] * table_stride;

    const int chunks = hd >> 3;
    for (int idx = threadIdx.x; idx < 16 * chunks; idx += MMA_THREADS) {
        const int r = idx / chunks, c = idx - r * chunks;
        const bool ok = r < g;
        const bf16* src = q + (size_t)t * q_row_stride + (size_t)(kh * g + (ok ? r : 0)) * hd + c * 8;
        cp_async_16(smem_u32(q_s + r * ld + c * 8), src, ok);
    }
    // the first DEC_STAGES-1 tiles are requested at once; queries ride with the first group
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
        if (st < ntiles) {
            load_kv_tile(k_s + st * MMA_BN * ld, k_pages, table, begin + st * MMA_BN, begin, end, kh, nkv, hd, ld, tm);
            load_kv_tile(v_s + st * MMA_BN * ld, v_pages, table, begin + st * MMA_BN, begin, end, kh, nkv, hd, ld, tm);
        }
        cp_async_commit();
    }

    float o[HD_MAX / 8][4];
#pragma unroll
    for (int i = 0; i < HD_MAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int it = 0; it < ntiles; ++it) {
        const int n0 = begin + it * MMA_BN;
        const int buf = it % DEC_STAGES;
        cp_async_wait<DEC_STAGES - 2>();
        __syncthreads();                                // tile `it` has landed; everyone is done with tile it-1
        {
            const int nx = it + DEC_STAGES - 1;         // goes into the buffer tile it-1 used
            if (nx < ntiles) {
                const int nb = nx % DEC_STAGES;
                load_kv_tile(k_s + nb * MMA_BN * ld, k_pages, table, begin + nx * MMA_BN, begin, end, kh, nkv, hd, ld, tm);
                load_kv_tile(v_s + nb * MMA_BN * ld, v_pages, table, begin + nx * MMA_BN, begin, end, kh, nkv, hd, ld, tm);
            }
            cp_async_commit();
        }
        const int w0 = n0 + warp * 16;              // this warp's 16 positions of the tile
        if (w0 < end) {
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            qk_tile<HD_MAX, 2>(s, q_s, k_s + (buf * MMA_BN + warp * 16) * ld, hd, ld, lane);
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int n = w0 + j * 8 + (lane & 3) * 2 + (e & 1);
                    s[j][e] = n < end ? s[j][e] * scale_log2 : -INFINITY;
                }
            online_softmax<HD_MAX, 2>(s, m, l, o);
            pv_tile<HD_MAX, 2>(o, s, v_s + (buf * MMA_BN + warp * 16) * ld, hd, ld, lane);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    // merge the four warps: (m, l, o) of each warp -> shared memory (the tile buffers are free now)
    float* mo = reinterpret_cast<float*>(k_s);                  // [4 warps][16 rows][hd]
    float* mml = mo + 4 * 16 * hd;                              // [4][16][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + r * 8;
        if ((lane & 3) == 0) {
            mml[(warp * 16 + row) * 2] = m[r];
            mml[(warp * 16 + row) * 2 + 1] = l[r];
        }
#pragma unroll
        for (int i = 0; i < HD_MAX / 8; ++i)
            if (i * 8 < hd) {
                const int d = i * 8 + (lane & 3) * 2;
                mo[(warp * 16 + row) * hd + d] = o[i][2 * r];
                mo[(warp * 16 + row) * hd + d + 1] = o[i][2 * r + 1];
            }
    }
    __syncthreads();
    const float LN2 = 0.6931471805599453f;
    for (int idx = threadIdx.x; idx < g * hd; idx += MMA_THREADS) {
        const int row = idx / hd, d = idx - row * hd;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * 16 + row) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = mml[(w * 16 + row) * 2];
            if (mw != -INFINITY) {
                const float f = exp2f(mw - M);
                L += mml[(w * 16 + row) * 2 + 1] * f;
                acc += mo[(w * 16 + row) * hd + d] * f;
            }
        }
        const int h = kh * g + row;
        if (n_splits == 1) {
            out[((size_t)t * nh + h) * hd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            const size_t slot = ((size_t)t * nh + h) * n_splits + sp;
            part_o[slot * hd + d] = acc;
            if (d == 0) {
                part_ml[slot * 2] = M == -INFINITY ? -INFINITY : M * LN2;   // natural-log units for the combine kernel
                part_ml[slot * 2 + 1] = L;
            }
        }
    }
}

// out[t, h, :] = sum_i o_i e^(m_i - M) / sum_i l_i e^(m_i - M) over the splits i of a listed token.
// One block per (token, head): the first warp turns the splits' (m, l) into weights e^(m_i - M) / L,
// then every thread sums its head dimensions over the splits (independent, coalesced loads).
#define COMBINE_MAX_SPLITS 64
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      bf16* __restrict__ out, const int* __restrict__ tok_list, int nh, int hd,
                                      int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float wgt[COMBINE_MAX_SPLITS];
    const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x;
    const size_t th = (size_t)t * nh + blockIdx.y;
    const float* ml = part_ml + th * n_splits * 2;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float m0 = lane < n_splits ? ml[2 * lane] : -INFINITY;
        const float m1 = lane + 32 < n_splits ? ml[2 * (lane + 32)] : -INFINITY;
        const float l0 = lane < n_splits ? ml[2 * lane + 1] : 0.f;
        const float l1 = lane + 32 < n_splits ? ml[2 * (lane + 32) + 1] : 0.f;
        const float M = warp_max(fmaxf(m0, m1));
        const float e0 = m0 == -INFINITY ? 0.f : expf(m0 - M), e1 = m1 == -INFINITY ? 0.f : expf(m1 - M);
        const float L = warp_sum(l0 * e0 + l1 * e1);
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        wgt[lane] = e0 * inv;
        wgt[lane + 32] = e1 * inv;
    }
    __syncthreads();
    const float* po = part_o + th * n_splits * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int i = 0; i < n_splits; ++i) acc += po[(size_t)i * hd + d] * wgt[i];
        out[th * hd + d] = __float2bfloat16_rn(acc);
    }
}

int pico_launch_decode_combine(const float* part_o, const float* part_ml, void* out, const int* tok_list, int n_tok,
                               int nh, int hd, int n_splits, cudaStream_t stream) {
    pico_launch(decode_combine_kernel, dim3(dim3(n_tok, nh)), dim3(hd >= 128 ? 128 : 64), 0, stream, part_o, part_ml, (bf16*)out, tok_list,
                                                                           nh, hd, n_splits);
    return pico_launch_status();
}

static size_t prefill_smem(int hd) { return (size_t)(64 + 4 * MMA_BN) * (hd + 8) * sizeof(bf16); }
static size_t decode_smem(int hd) {
    const size_t tiles = (size_t)(16 + 2 * DEC_STAGES * MMA_BN) * (hd + 8) * sizeof(bf16);
    const size_t merge = (size_t)16 * (hd + 8) * sizeof(bf16) + (size_t)4 * 16 * (hd + 2) * sizeof(float);
    return tiles > merge ? tiles : merge;
}

// Prompt portions.  seg_list: [n_segs] segments to run (null: 0 .. n_segs-1); cu_q: first token of
// each segment; max_q_len: most tokens any listed segment brings.  Tokens of a segment have
// consecutive positions.  out rows of tokens in other segments are not touched.
PICO_API int pico_paged_prefill_mma(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                    void* out, const int* seg_list, int n_segs, const int* cu_q, int max_q_len,
                                    const int* positions, const int* block_table, int table_stride, int nh,
                                    int nkv, int hd, int page_size, int window, float scale, cudaStream_t stream) {
    if (n_segs <= 0 || max_q_len <= 0) return 0;
    if (hd % 16 != 0 || hd < 16 || hd > 256 || nkv <= 0 || nh % nkv != 0) return PICO_ERR_SIZE;
    const int g = nh / nkv;
    if (g > 64 || nkv > 65535 || n_segs > 65535) return PICO_ERR_SIZE;
    if (q_row_stride % 8 != 0) return PICO_ERR_ALIGN;
    const int tpt = 64 / g;
    const dim3 grid((max_q_len + tpt - 1) / tpt, nkv, n_segs);
    const size_t smem = prefill_smem(hd);
    const float scale_log2 = scale * 1.4426950408889634f;
#define LAUNCH_PREFILL(HD)                                                                                          \
    do {                                                                                                            \
        cudaFuncSetAttribute(paged_prefill_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        pico_launch((paged_prefill_mma_kernel<HD>), dim3(grid), dim3(MMA_THREADS), smem, stream,                                           \
            (const bf16*)q, q_row_stride, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, seg_list, cu_q,   \
            positions, block_table, table_stride, nh, nkv, hd, page_size, window, scale_log2);                      \
    } while (0)
    if (hd <= 64) LAUNCH_PREFILL(64);
    else if (hd <= 128) LAUNCH_PREFILL(128);
    else LAUNCH_PREFILL(256);
#undef LAUNCH_PREFILL
    return pico_launch_status();
}

// Single tokens.  tok_list: [n_tok] tokens to run (null: 0 .. n_tok-1).  part_o / part_ml: scratch for
// n_splits > 1, indexed by the token's number in the whole batch: [T_total * nh * n_splits * hd] and
// [T_total * nh * n_splits * 2] floats.
PICO_API int pico_paged_decode_mma(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                   void* out, float* part_o, float* part_ml, const int* tok_list, int n_tok,
                                   const int* tok_seg, const int* positions, const int* block_table,
                                   int table_stride, int nh, int nkv, int hd, int page_size, int window,
                                   float scale, int n_splits, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (hd % 16 != 0 || hd < 16 || hd > 256 || nkv <= 0 || nh % nkv != 0) return PICO_ERR_SIZE;
    const int g = nh / nkv;
    if (g > 16 || nkv > 65535 || n_tok > 65535 || n_splits < 1 || n_splits > COMBINE_MAX_SPLITS) return PICO_ERR_SIZE;
    if (n_splits > 1 && (!part_o || !part_ml)) return PICO_ERR_SIZE;
    if (q_row_stride % 8 != 0) return PICO_ERR_ALIGN;
    const dim3 grid(n_splits, nkv, n_tok);
    const size_t smem = decode_smem(hd);
    const float scale_log2 = scale * 1.4426950408889634f;
#define LAUNCH_DECODE(HD)                                                                                          \
    do {                                                                                                           \
        cudaFuncSetAttribute(paged_decode_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        pico_launch((paged_decode_mma_kernel<HD>), dim3(grid), dim3(MMA_THREADS), smem, stream,                                           \
            (const bf16*)q, q_row_stride, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, part_o, part_ml, \
            tok_list, tok_seg, positions, block_table, table_stride, nh, nkv, hd, page_size, window, scale_log2,   \
            n_splits);                                                                                             \
    } while (0)
    if (hd <= 64) LAUNCH_DECODE(64);
    else if (hd <= 128) LAUNCH_DECODE(128);
    else LAUNCH_DECODE(256);
#undef LAUNCH_DECODE
    if (n_splits > 1) return pico_launch_decode_combine(part_o, part_ml, out, tok_list, n_tok, nh, hd, n_splits, stream);
    return pico_launch_status();
}

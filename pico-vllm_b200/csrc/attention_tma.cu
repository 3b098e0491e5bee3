// Single-token ("decode") paged attention for bfloat16 with the cache pages brought in by TMA.
//
// A cache page of one key/value head is a contiguous [page_size, head_dim] block, so a tile of 64
// cache positions is 64 / page_size boxes of a 2-D tensor map over the layer's pages
// ([pages * kv_heads * page_size rows, head_dim]); one box is a whole page of one head and lands in
// shared memory in the 128-byte swizzle, which ldmatrix then reads with few bank conflicts.  A
// producer warp issues the copies (cp.async.bulk.tensor.3d, completion on an mbarrier) while four
// consumer warps multiply, so neither the per-16-byte address arithmetic of a cp.async pipeline -
// which made the earlier kernel instruction-bound - nor the issue of the copies sits in the
// consumers' way; full/empty mbarriers per stage replace block-wide barriers.  The products are
// mma.sync m16n8k16 with float32 accumulation, with the 16 cache positions of a warp as the rows and
// the g <= 16 query heads of a key/value head as the 8-wide columns; running max/sum softmax in
// float32; the key range of a token is cut into n_splits parts, which for 2, 4, 8 or 16 parts form a
// thread-block cluster that adds its partial results through distributed shared memory (otherwise a
// second kernel combines them).
//
// Formulas restated from the reference as cited in attention_mma.cu
// (pico_vllm/kernels/attention.py:31, 67-82, 92).  Every wait on an mbarrier is bounded: after
// TMA_WAIT_LIMIT polls the block records an error in a status word, stops issuing copies and
// leaves (its results are then invalid; the host reads the word with pico_tma_status).
#include <cuda.h>
#include "mma_helpers.cuh"

#define TMA_STAGES_MANY 3      // stages of 32 KB: small enough that the next kernel's blocks fit beside a block
#define TMA_WAIT_LIMIT (1 << 15)     // polls of a barrier (some microseconds each) before a thread gives up
#ifndef TMA_L2_PROMO
#define TMA_L2_PROMO CU_TENSOR_MAP_L2_PROMOTION_L2_256B
#endif
#define TMA_TABLE_CACHE 256        // block-table entries of a block's key range kept in shared memory

__device__ int g_tma_status = 0;     // 0 = fine; 1 = a wait on a TMA copy ran out

PICO_API int pico_tma_status(int* out) {
    return (int)cudaMemcpyFromSymbol(out, g_tma_status, sizeof(int), 0, cudaMemcpyDeviceToHost);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < TMA_WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}
// thread-block cluster: barrier over all threads of all blocks, and loads from another block's shared memory
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void st_cluster_f32(float* local, int rank, float v) {
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(raddr), "f"(v) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

template <int NTHREADS> __device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;\n" ::"n"(NTHREADS) : "memory");
}

// A tile is 64 cache positions = 64 / page_size pages, and a page arrives as one TMA box
// [HD / 64 blocks of 64 dims][page_size positions][128 bytes] in the 128-byte swizzle: inside a block the
// 16-byte piece c of position r sits at piece c ^ (r & 7) (a block starts on a multiple of 1024 bytes, since
// page_size >= 8).  Consecutive positions are consecutive 128-byte rows, so the eight rows an ldmatrix reads
// fall into eight different bank groups (with rows of HD * 2 bytes, position after position, they fell into four:
// half of the shared-memory wavefronts of the kernel were bank conflicts).
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int key, int dim, int page_size) {
    const int pg = key / page_size, r = key - pg * page_size;
    const int chunk = (dim & 63) >> 3;
    return (uint32_t)(pg * page_size * HD * 2 + (dim >> 6) * page_size * 128 + r * 128 + ((chunk ^ (r & 7)) << 4));
}

// 4 consumer warps (multiply) + 1 producer warp (one lane issues the TMA copies).  full[s]: the
// copies of stage s have landed (transaction count); empty[s]: the four consumer warps are done
// with stage s.
// CW consumer warps in groups of four: group i takes tiles i, i + CW/4, ... (a group multiplies one tile,
// 16 cache positions per warp); one group is what the launcher uses.
template <int HD, int TMA_STAGES, int CW, int NT>     // head size 64 or 128; stages; consumer warps (4 or 8); 8-head tiles (g <= 8 NT)
__global__ void __launch_bounds__((CW + 1) * 32)
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                        const bf16* __restrict__ q, int q_row_stride, bf16* __restrict__ out,
                        float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ tok_list,
                        const int* __restrict__ tok_seg, const int* __restrict__ positions,
                        const int* __restrict__ block_table, int table_stride, int nh, int nkv, int page_size,
                        int window, float scale_log2, int n_splits, int cluster_reduce) {
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_dyn[];
    constexpr int TILE_BYTES = MMA_BN * HD * 2;                  // one K or V tile
    constexpr int QLD = HD + 8;
    // the swizzle pattern follows shared-memory address bits 7..9: tiles start on 1024 bytes
    unsigned char* smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    // [stages][K tile | V tile], then the queries, the barriers, the block-table entries
    unsigned char* tiles = smem_raw;
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw + TMA_STAGES * 2 * TILE_BYTES);     // [16][QLD]
    uint64_t* full = reinterpret_cast<uint64_t*>(q_s + 16 * QLD);                    // [stages]
    uint64_t* empty = full + TMA_STAGES;                                             // [stages]
    volatile int* abort_s = reinterpret_cast<volatile int*>(empty + TMA_STAGES);
    int* tbl_s = const_cast<int*>(abort_s) + 2;                                      // [TMA_TABLE_CACHE]
    float* recv_o = reinterpret_cast<float*>(tbl_s + TMA_TABLE_CACHE);               // [splits][share]: what the cluster's blocks push here
    const int g = nh / nkv;
    float* recv_ml = recv_o + n_splits * ((g * HD + n_splits - 1) / n_splits);       // [splits][16 rows][max, sum]
    const int kh = blockIdx.y, sp = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < TMA_STAGES; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 4);
        }
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    // Token lists, positions and block tables come from the host copy at the start of the step and
    // the cache of earlier positions from earlier steps: all of that may be read now.  What the
    // kernel before this one wrote - the queries, and the key/value of the token's own position -
    // is read only after pdl_wait(): by the consumers before they load the queries, by the producer
    // before it copies the tile that holds the token's own position.
    const int t = tok_list ? tok_list[blockIdx.z] : blockIdx.z;
    const int pos = positions[t];
    const int hi = pos + 1;                                      // pos = -1 (padding): no keys at all
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    // tiles are aligned to multiples of 64 cache positions, so that a tile is whole pages
    const int tile_lo = lo / MMA_BN, tile_hi = (hi + MMA_BN - 1) / MMA_BN;
    const int per = (tile_hi - tile_lo + n_splits - 1) / n_splits;
    const int t_begin = tile_lo + sp * per;
    const int t_end = min(tile_hi, t_begin + per);
    const int ntiles = t_end > t_begin ? t_end - t_begin : 0;
    const int* table = block_table + (size_t)tok_seg[t] * table_stride;
    const int ppt = MMA_BN / page_size;                          // pages per tile
    {   // the block-table entries of this block's range, read once and together
        const int first_entry = t_begin * ppt;
        const int n_entries = min(ntiles * ppt, TMA_TABLE_CACHE);
        for (int i = threadIdx.x; i < n_entries; i += (CW + 1) * 32)
            tbl_s[i] = first_entry + i < table_stride ? table[first_entry + i] : 0;
    }
    __syncthreads();                                             // barriers are initialised, the table is there

    if (warp == CW) {
        // ---------------------------------------------------------------- producer
        // One copy costs its issuing thread a few hundred cycles, so the copies of a tile are issued
        // by different lanes: lane 2*pg copies page pg of the keys, lane 2*pg+1 of the values.
        bool waited = false;
        for (int it = 0; it < ntiles; ++it) {
            const int s = it % TMA_STAGES;
            if (it >= TMA_STAGES && !mbar_wait(empty + s, ((it / TMA_STAGES) - 1) & 1)) {
                g_tma_status = 1;
                *abort_s = 1;
            }
            __syncwarp();
            if (*abort_s) break;
            const int n0 = (t_begin + it) * MMA_BN;
            if (!waited && n0 + MMA_BN > pos) {      // this tile holds the token's own key and value
                pdl_wait();
                waited = true;
            }
            unsigned char* kt = tiles + (size_t)s * 2 * TILE_BYTES;
            // pages wholly outside [lo, hi) are skipped: they may have been given back (a window) or
            // not exist yet
            int first = 0, last = ppt;
            while (first < last && n0 + (first + 1) * page_size <= lo) ++first;
            while (last > first && n0 + (last - 1) * page_size >= hi) --last;
            if (lane == 0) mbar_expect_tx(full + s, (uint32_t)((last - first) * page_size * HD * 2 * 2));
            __syncwarp();
            const int pg = lane >> 1;
            if (pg >= first && pg < last) {
                const int e = it * ppt + pg;
                const int page = e < TMA_TABLE_CACHE ? tbl_s[e] : table[n0 / page_size + pg];
                const int row = (page * nkv + kh) * page_size;
                tma_load_3d(kt + (lane & 1) * TILE_BYTES + pg * page_size * HD * 2, (lane & 1) ? &v_map : &k_map, 0, row, 0,
                            full + s);
            }
        }
        if (cluster_reduce) cluster_sync_all();     // every thread of the cluster takes part in its barrier
        return;
    }
    // -------------------------------------------------------------------- consumers (warps 0..CW-1)
    constexpr int NG = CW / 4;                                   // consumer groups
    const int grp = warp >> 2, wq = warp & 3;
    pdl_wait();                                                  // the queries come from the kernel before
    for (int idx = threadIdx.x; idx < 16 * (HD / 8); idx += CW * 32) {
        const int r = idx / (HD / 8), c = idx - r * (HD / 8);
        const bool ok = r < g;
        const bf16* src = q + (size_t)t * q_row_stride + (size_t)(kh * g + (ok ? r : 0)) * HD + c * 8;
        cp_async_16(smem_u32(q_s + r * QLD + c * 8), src, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    consumer_sync<CW * 32>();                                             // the queries are in shared memory

    // The products are taken the other way round than in a prompt kernel: the 16 cache positions of a
    // warp are the 16 ROWS of the tensor-core tile and the query heads its 8 columns, because a token
    // brings at most 16 heads (NT tiles of 8) and a tile of 8 columns costs half the instructions of two:
    //   S^T [16 keys x 8 heads] = K [16 keys x hd] Q^T;   O^T [hd x 8 heads] += V^T [hd x 16 keys] P^T.
    // A thread then holds, of S^T and P^T, keys lane/4 and lane/4 + 8 and heads 2 (lane%4), + 1; the
    // maxima and sums of a head run over the 8 lanes with the same lane%4.
    float o[NT][HD / 16][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) o[nt][i][0] = o[nt][i][1] = o[nt][i][2] = o[nt][i][3] = 0.f;
    float m[NT][2], l[NT][2];          // per head column of the thread: running maximum (all keys so far, log2 units), this thread's part of the sum
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) m[nt][0] = m[nt][1] = -INFINITY, l[nt][0] = l[nt][1] = 0.f;
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;       // K as the 16-row operand
    const int b_row = lane & 7, b_col = ((lane >> 3) & 1) * 8;                           // Q rows as the 8-column operand
    const int v_row = (lane & 7) + (lane >> 4) * 8, v_col = ((lane >> 3) & 1) * 8;       // V^T through the transposing load
    // the queries are the same for every tile: their fragments stay in registers
    uint32_t qf[NT][HD / 16][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int k0 = 0; k0 < HD; k0 += 16) ldmatrix_x2(qf[nt][k0 / 16], smem_u32(q_s + (nt * 8 + b_row) * QLD + k0 + b_col));

    // where this lane's rows of a tile sit does not change from tile to tile
    const int kw = wq * 16;                                      // this warp's 16 positions of the tile
    uint32_t k_off[HD / 16], v_off[HD / 16];
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) {
        k_off[i] = tile_off<HD>(kw + a_row, i * 16 + a_col, page_size);
        v_off[i] = tile_off<HD>(kw + v_row, i * 16 + v_col, page_size);
    }
    for (int it = grp; it < ntiles; it += NG) {
        const int s = it % TMA_STAGES;
        const int n0 = (t_begin + it) * MMA_BN;
        if (!mbar_wait(full + s, (it / TMA_STAGES) & 1)) {
            g_tma_status = 1;
            *abort_s = 1;
        }
        if (*abort_s) break;
        const uint32_t kt = smem_u32(tiles + (size_t)s * 2 * TILE_BYTES);
        const uint32_t vt = kt + TILE_BYTES;
        const int w0 = n0 + kw;
        if (w0 < hi && w0 + 16 > lo) {
            // q.k: four independent accumulators per head tile (a tensor-core instruction waits more
            // than a hundred clocks for the one before it when both add into the same registers)
            float sc[NT][4][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[nt][c][0] = sc[nt][c][1] = sc[nt][c][2] = sc[nt][c][3] = 0.f;
#pragma unroll
            for (int k0 = 0; k0 < HD; k0 += 16) {
                uint32_t a[4];
                ldmatrix_x4(a, kt + k_off[k0 / 16]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16(sc[nt][(k0 / 16) & 3], a, qf[nt][k0 / 16][0], qf[nt][k0 / 16][1]);
            }
            const int key_a = w0 + (lane >> 2), key_b = key_a + 8;                   // the thread's two cache positions
            const bool vis_a = key_a >= lo && key_a < hi, vis_b = key_b >= lo && key_b < hi;
            const bool warp_edge = __any_sync(0xffffffffu, !(vis_a && vis_b));
            uint32_t pb[NT][2];                                  // P^T as the 8-column operand: keys 0-7 and 8-15 of the warp
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float x[4];                                      // [key a: head 0, 1; key b: head 0, 1]
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = (sc[nt][0][e] + sc[nt][1][e]) + (sc[nt][2][e] + sc[nt][3][e]);
                    x[e] = ((e < 2) ? vis_a : vis_b) ? v * scale_log2 : -INFINITY;
                }
                float p[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float mx = fmaxf(x[h], x[2 + h]);
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    const float m_new = fmaxf(m[nt][h], mx);
                    const float corr = m_new == -INFINITY ? 1.f : fast_exp2(m[nt][h] - m_new);
                    const float sub = m_new == -INFINITY ? 0.f : m_new;
                    p[h] = fast_exp2(x[h] - sub);
                    p[2 + h] = fast_exp2(x[2 + h] - sub);
                    l[nt][h] = l[nt][h] * corr + p[h] + p[2 + h];
                    m[nt][h] = m_new;
#pragma unroll
                    for (int i = 0; i < HD / 16; ++i) {
                        o[nt][i][h] *= corr;
                        o[nt][i][2 + h] *= corr;
                    }
                }
                // [key][head pair] -> [head][key pair]: the 8 x 8 transpose between the layout a product
                // leaves and the layout the next one reads as its 8-column operand
                const uint32_t pa = pack_bf16(p[0], p[1]), pc = pack_bf16(p[2], p[3]);
                asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(pb[nt][0]) : "r"(pa));
                asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(pb[nt][1]) : "r"(pc));
            }
            // p.v: invisible positions have p = 0 exactly, but their value rows may hold anything
            // (another request's data, or not-a-number): they are read as zero
#pragma unroll
            for (int d0 = 0; d0 < HD; d0 += 16) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, vt + v_off[d0 / 16]);
                if (warp_edge) {
                    // register j of lane L holds dims d0 + L/4 (+ 8 for odd j) of cache positions
                    // w0 + (j / 2) * 8 + (L % 4) * 2 + {0, 1} (low and high half): clear by position
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int key0 = w0 + (j >> 1) * 8 + (lane & 3) * 2;
                        const bool ok0 = key0 >= lo && key0 < hi, ok1 = key0 + 1 >= lo && key0 + 1 < hi;
                        a[j] &= (ok0 ? 0x0000ffffu : 0u) | (ok1 ? 0xffff0000u : 0u);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16(o[nt][d0 / 16], a, pb[nt][0], pb[nt][1]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);                   // this warp is done with the stage
    }
    // the sums of a head: over the 8 lanes that hold its keys
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float v = l[nt][h];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            l[nt][h] = v;
        }
    consumer_sync<CW * 32>();
    const bool dead = *abort_s != 0;
    if (dead && !cluster_reduce) return;
    // merge the four warps: (m, l, o) of each warp -> shared memory (all copies have landed and been used)
    constexpr int MO_LD = HD + 4;                               // padded rows: the four head rows of a lane group fall into different banks
    float* mo = reinterpret_cast<float*>(tiles);                // [CW warps][16 rows][MO_LD]
    float* mml = mo + CW * 16 * MO_LD;                          // [CW][16][2]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = nt * 8 + (lane & 3) * 2 + h;         // query head of the group
            if ((lane >> 2) == 0) {
                mml[(warp * 16 + row) * 2] = m[nt][h];
                mml[(warp * 16 + row) * 2 + 1] = l[nt][h];
            }
#pragma unroll
            for (int i = 0; i < HD / 16; ++i) {
                const int d = i * 16 + (lane >> 2);
                mo[(warp * 16 + row) * MO_LD + d] = o[nt][i][h];
                mo[(warp * 16 + row) * MO_LD + d + 8] = o[nt][i][2 + h];
            }
        }
    consumer_sync<CW * 32>();
    const float LN2 = 0.6931471805599453f;
    // With a cluster, block sp adds output elements [sp * share, (sp + 1) * share) of the g * HD over all
    // blocks: every block PUSHES what it has of another block's share (and its maxima and sums) into
    // that block's receive area through distributed shared memory, one cluster barrier follows, and
    // each block then adds from its own shared memory - nobody reads remote memory after the barrier,
    // so blocks may leave at once.
    const int total = g * HD;
    const int share = (total + n_splits - 1) / n_splits;
    for (int idx = threadIdx.x; idx < total; idx += CW * 32) {
        const int row = idx / HD, d = idx - row * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < CW; ++w) M = fmaxf(M, mml[(w * 16 + row) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < CW; ++w) {
            const float mw = mml[(w * 16 + row) * 2];
            if (mw != -INFINITY) {
                const float f = fast_exp2(mw - M);
                L += mml[(w * 16 + row) * 2 + 1] * f;
                acc += mo[(w * 16 + row) * MO_LD + d] * f;
            }
        }
        const int h = kh * g + row;
        if (n_splits == 1) {
            out[((size_t)t * nh + h) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else if (cluster_reduce) {
            const int r = idx / share;
            st_cluster_f32(recv_o + sp * share + (idx - r * share), r, acc);
            if (d == 0) {
                for (int rr = 0; rr < n_splits; ++rr) {
                    st_cluster_f32(recv_ml + (sp * 16 + row) * 2, rr, M);
                    st_cluster_f32(recv_ml + (sp * 16 + row) * 2 + 1, rr, L);
                }
            }
        } else {
            const size_t slot = ((size_t)t * nh + h) * n_splits + sp;
            part_o[slot * HD + d] = acc;
            if (d == 0) {
                part_ml[slot * 2] = M == -INFINITY ? -INFINITY : M * LN2;   // natural-log units for the combine kernel
                part_ml[slot * 2 + 1] = L;
            }
        }
    }
    if (!cluster_reduce || n_splits == 1) return;
    cluster_sync_all();
    {
        const int lo_i = sp * share, hi_i = min(total, lo_i + share);
        for (int idx = lo_i + (int)threadIdx.x; idx < hi_i; idx += CW * 32) {
            const int row = idx / HD, d = idx - row * HD;
            float M = -INFINITY;
            for (int r = 0; r < n_splits; ++r) M = fmaxf(M, recv_ml[(r * 16 + row) * 2]);
            float L = 0.f, acc = 0.f;
            for (int r = 0; r < n_splits; ++r) {
                const float mr = recv_ml[(r * 16 + row) * 2];
                if (mr != -INFINITY) {
                    const float f = fast_exp2(mr - M);
                    L += recv_ml[(r * 16 + row) * 2 + 1] * f;
                    acc += recv_o[r * share + (idx - lo_i)] * f;
                }
            }
            out[((size_t)t * nh + kh * g + row) * HD + d] = __float2bfloat16_rn((L > 0.f && !dead) ? acc / L : 0.f);
        }
    }
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) == cudaSuccess &&
            st == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Fills `map_out` (128 bytes, 64-byte aligned host memory) with a tensor map over the cache pages of
// one layer: a [rows, hd] bfloat16 matrix (rows = pages * kv_heads * page_size) read in boxes of
// [page_size rows, hd elements] (one page of one head) with the 128-byte swizzle, the 64-element blocks of the
// rows one after the other in shared memory.  Returns 0, or PICO_ERR_SIZE for sizes
// the TMA kernels do not take, or -7 when the driver refuses.
PICO_API int pico_make_kv_tensor_map(void* map_out, const void* base, long long rows, int hd, int page_size) {
    if (hd % 64 != 0 || hd < 64 || hd > 256 || page_size < 8 || page_size > MMA_BN || MMA_BN % page_size != 0 ||
        (page_size & 7) != 0 || ((uintptr_t)base & 15) != 0)
        return PICO_ERR_SIZE;
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return -7;
    // dimensions: 64 elements of a 128-byte segment, the rows, the hd/64 segments of a row; one box is a
    // whole page of one key/value head and arrives as [segment][row][128 bytes]
    const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(hd / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)hd * 2, 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)page_size, (cuuint32_t)(hd / 64)};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          TMA_L2_PROMO, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -7;
}

__global__ void decode_combine_kernel(const float*, const float*, bf16*, const int*, int, int, int);
int pico_launch_decode_combine(const float* part_o, const float* part_ml, void* out, const int* tok_list, int n_tok,
                               int nh, int hd, int n_splits, cudaStream_t stream);

// Can clusters of `size` blocks of the decode kernel run here?  (Asked once per configuration.)
template <int HD, int ST, int CW, int NT>
static bool tma_cluster_query(int size, size_t smem) {
    if (size > 8 && cudaFuncSetAttribute(paged_decode_tma_kernel<HD, ST, CW, NT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) !=
                        cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    cudaFuncSetAttribute(paged_decode_tma_kernel<HD, ST, CW, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(size, 1, 1);
    cfg.blockDim = dim3((CW + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, paged_decode_tma_kernel<HD, ST, CW, NT>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return n > 0;
}
static bool tma_cluster_ok(int hd, int size, int nt, size_t smem) {
    static int cache[2][2][5];      // [hd 64/128][head tiles - 1][log2 size]: 0 unknown, 1 yes, 2 no
    int lg = 0;
    while ((1 << lg) < size) ++lg;
    int& c = cache[hd == 128 ? 1 : 0][nt - 1][lg];
    if (c == 0) {
        bool ok;
        if (hd == 128) ok = nt == 1 ? tma_cluster_query<128, TMA_STAGES_MANY, 4, 1>(size, smem) : tma_cluster_query<128, TMA_STAGES_MANY, 4, 2>(size, smem);
        else ok = nt == 1 ? tma_cluster_query<64, TMA_STAGES_MANY, 4, 1>(size, smem) : tma_cluster_query<64, TMA_STAGES_MANY, 4, 2>(size, smem);
        c = ok ? 1 : 2;
    }
    return c == 1;
}

// Single tokens with TMA-fed tiles.  k_map / v_map: tensor maps made by pico_make_kv_tensor_map (host
// pointers; they are copied into the kernel's parameters).  Other arguments as pico_paged_decode_mma.
PICO_API int pico_paged_decode_tma(const void* k_map, const void* v_map, const void* q, int q_row_stride, void* out,
                                   float* part_o, float* part_ml, const int* tok_list, int n_tok, const int* tok_seg,
                                   const int* positions, const int* block_table, int table_stride, int nh, int nkv,
                                   int hd, int page_size, int window, float scale, int n_splits,
                                   cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv != 0) return PICO_ERR_SIZE;
    const int g = nh / nkv;
    if (g > 16 || nkv > 65535 || n_tok > 65535 || n_splits < 1 || n_splits > 64) return PICO_ERR_SIZE;
    if (page_size < 8 || MMA_BN % page_size != 0) return PICO_ERR_SIZE;
    if (q_row_stride % 8 != 0) return PICO_ERR_ALIGN;
    const dim3 grid(n_splits, nkv, n_tok);
    const float scale_log2 = scale * 1.4426950408889634f;
    // (one block per SM with more stages or eight consumer warps was measured slower: it keeps the next
    // kernel's blocks, which prefetch under programmatic launch, off the SM)
    const int stages = TMA_STAGES_MANY;
    const int nt = g <= 8 ? 1 : 2;                               // tiles of 8 query heads
    const size_t smem = (size_t)stages * 2 * MMA_BN * hd * 2 + (size_t)16 * (hd + 8) * 2 + 2 * stages * 8 + 8 +
                        TMA_TABLE_CACHE * 4 + 1024 +
                        (n_splits > 1 ? (size_t)(n_splits * ((g * hd + n_splits - 1) / n_splits) + n_splits * 32) * 4 : 0);
    CUtensorMap km, vm;
    memcpy(&km, k_map, sizeof(CUtensorMap));
    memcpy(&vm, v_map, sizeof(CUtensorMap));
    // 2, 4, 8 or 16 splits: the splits of one (token, kv head) run as one thread-block cluster and are
    // added through distributed shared memory; otherwise through scratch and the combine kernel
    int cluster = 0;
    if (n_splits == 2 || n_splits == 4 || n_splits == 8 || n_splits == 16) cluster = tma_cluster_ok(hd, n_splits, nt, smem) ? 1 : 0;
    if (n_splits > 1 && !cluster && (!part_o || !part_ml)) return PICO_ERR_SIZE;
#define LAUNCH_TMA(HD, NT)                                                                                              \
    do {                                                                                                                \
        cudaFuncSetAttribute(paged_decode_tma_kernel<HD, TMA_STAGES_MANY, 4, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                             (int)smem);                                                                                \
        pico_launch_cluster((paged_decode_tma_kernel<HD, TMA_STAGES_MANY, 4, NT>), grid, dim3(5 * 32), smem, stream,    \
                            cluster ? n_splits : 1, km, vm, (const bf16*)q, q_row_stride, (bf16*)out, part_o,           \
                            part_ml, tok_list, tok_seg, positions, block_table, table_stride, nh, nkv, page_size,       \
                            window, scale_log2, n_splits, cluster);                                                     \
    } while (0)
    if (hd == 64) {
        if (nt == 1) LAUNCH_TMA(64, 1); else LAUNCH_TMA(64, 2);
    } else {
        if (nt == 1) LAUNCH_TMA(128, 1); else LAUNCH_TMA(128, 2);
    }
#undef LAUNCH_TMA
    if (n_splits > 1 && !cluster)
        return pico_launch_decode_combine(part_o, part_ml, out, tok_list, n_tok, nh, hd, n_splits, stream);
    return pico_launch_status();
}

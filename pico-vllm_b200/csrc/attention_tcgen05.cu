// Paged causal attention for portions of prompts ("prefill") on the 5th-generation tensor cores.
//
// A block takes 128 rows of queries - 128 / g tokens of one segment times the g query heads that
// share a key/value head - and walks the visible cache positions 64 at a time:
//   warps 0, 13   issue the TMA copies of the pages of a tile, lane = box: warp 0 the keys ([page rows, 64
//               dims] boxes, one per page and 64-dim block), warp 13 the values (one box per page with all
//               its 64-dim blocks), 128-byte swizzle, separate rings for keys and values: a key stage is
//               free once S = Q K^T has read it, a value stage once O += P V has;
//   warps 1, 10-12  one lane each issues tcgen05.mma: S = Q K^T (M 128, N 64, Q from tensor memory - the
//               softmax warps of pipeline 0 put their rows there once -, K from shared memory,
//               accumulator S in tensor memory) for pipeline 0 (warp 1) and 1 (warp 10); O += P V (M 128,
//               N head_dim, P read from tensor memory, V from shared memory as an MN-major operand,
//               accumulator O in tensor memory) for pipeline 0 (warp 11) and 1 (warp 12).  A tcgen05.mma
//               costs its issuing thread about a hundred clocks whatever its size (measured), so one
//               issuing thread would be the bottleneck; tcgen05.commit signals mbarriers;
//   warps 2-9   softmax, two groups of four warps: thread = row.  tcgen05.ld of the row's 64 scores,
//               mask, running max and sum in float32 (exp2 on scores scaled to log2 units, packed
//               two-lane fma / add), probabilities as bfloat16 pairs back into tensor memory
//               (tcgen05.st); the O accumulator is rescaled in tensor memory only when a row's maximum
//               has grown by more than 2^8 since the value in use, which is exact because the same
//               maximum is used for the sum.
// Even tiles go through pipeline 0 (its own S, P, O columns and softmax group), odd tiles through
// pipeline 1, so that one tile's softmax runs beside the other's and beside the products; at the end
// the two partial results (O, maximum, sum) are merged and divided by the sum.
// Rules restated from the reference: query head j reads key/value head j / g
// (pico_vllm/kernels/attention.py:139); scores * hd^-1/2 (attention.py:231); key n visible to the
// query at position p iff n <= p (attention.py:193-198) - and n > p - window with a window; online
// softmax in float32, p rounded to the cache type before p.v (attention.py:189-213).
// Every mbarrier wait is bounded (status word pico_tca_status); tensor memory is freed on every path.
#include <cuda.h>
#include "common.cuh"

#define TCA_BM 128
#define TCA_BN 64
#define TCA_THREADS 448
#define TCA_STAGES 4
#define TCA_WAIT_LIMIT (1 << 14)     // polls of a barrier (some microseconds each) before a thread gives up
#define TCA_TABLE_CACHE 1024
#define TCA_RESCALE_AT 8.0f     // log2 units: rescale the accumulator when the maximum grew by more than this

__device__ int g_tca_status = 0;

PICO_API int pico_tca_status(int* out) {
    return (int)cudaMemcpyFromSymbol(out, g_tca_status, sizeof(int), 0, cudaMemcpyDeviceToHost);
}

__device__ __forceinline__ uint32_t tca_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tca_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tca_u32(bar)), "r"(count));
}
__device__ __forceinline__ void tca_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tca_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tca_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tca_u32(bar)) : "memory");
}
__device__ __forceinline__ bool tca_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < TCA_WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(tca_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tca_tma_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(tca_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(tca_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tca_tma_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
        ::"r"(tca_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(tca_u32(bar))
        : "memory");
}
// K-major operand [rows][64 bf16] in the 128-byte swizzle (rows 128 bytes, 8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t tca_desc_k(uint32_t tile, int k16) {
    const uint32_t addr = tile + k16 * 32;
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// MN-major operand: values [keys][head dims], head dims contiguous.  A value tile is stored page by page,
// each page as its 64-dim blocks one after the other ([block][page rows][128 bytes], 128-byte swizzle):
// `addr` is the first of 16 keys, 64-dim blocks are `block_bytes` apart (leading byte offset) and the two
// groups of 8 keys `group_bytes` apart (stride byte offset: 1024 inside a page).
__device__ __forceinline__ uint64_t tca_desc_mn(uint32_t addr, uint32_t block_bytes, uint32_t group_bytes) {
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)((block_bytes >> 4) & 0x3fff) << 16) |
           ((uint64_t)((group_bytes >> 4) & 0x3fff) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tca_mma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(zero) : "memory");
}
__device__ __forceinline__ void tca_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tca_u32(bar)) : "memory");
}
__device__ __forceinline__ void tca_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tca_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float tca_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tca_fence_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void tca_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t acc) {
    const uint32_t zero = 0;       // the a operand is read from tensor memory
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(acc), "r"(zero) : "memory");
}
__device__ __forceinline__ float tca_max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
// two float32 lanes in one 64-bit register: the packed forms of fma and add halve the instruction count
__device__ __forceinline__ uint64_t tca_pack(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void tca_unpack(uint64_t r, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(r));
}
__device__ __forceinline__ uint64_t tca_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t tca_add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ void tca_softmax_sync() { asm volatile("bar.sync 2, 256;\n" ::: "memory"); }

// Tensor-memory columns of a block (512 allocated): scores of the two pipelines, their probabilities
// (bfloat16 pairs, the a operand of p.v), their output accumulators.
#define TCA_COL_S 0
#define TCA_COL_P 128
#define TCA_COL_O 192
#define TCA_COL_Q 448          // the queries as a tensor-memory operand: 64 columns of bfloat16 pairs at head size 128

template <int HD>      // head size, a multiple of 64 up to 128
__global__ void __launch_bounds__(TCA_THREADS)
paged_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                             const bf16* __restrict__ q, int q_row_stride, bf16* __restrict__ out,
                             const int* __restrict__ seg_list, const int* __restrict__ cu_q,
                             const int* __restrict__ positions, const int* __restrict__ block_table, int table_stride,
                             int nh, int nkv, int page_size, int window, float scale_log2,
                             float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                             size_t n_rows, int n_parts, int split_min) {
    pdl_launch_dependents();
    extern __shared__ unsigned char tca_dyn[];
    constexpr int NH = HD / 64;                              // 64-dim blocks of a head
    constexpr int SUB = TCA_BN * 128;                        // bytes of one [64 keys][64 dims] block
    constexpr int KV_BYTES = NH * SUB;                       // one K (or V) tile
    unsigned char* smem = tca_dyn + ((1024u - (tca_u32(tca_dyn) & 1023u)) & 1023u);
    unsigned char* k_s = smem;                               // [stages] K tiles: a stage is free once S = Q K^T has read it
    unsigned char* v_s = k_s + TCA_STAGES * KV_BYTES;        // [stages] V tiles: free once O += P V has read it, two tiles later
    uint64_t* k_full = reinterpret_cast<uint64_t*>(v_s + TCA_STAGES * KV_BYTES);
    uint64_t* k_empty = k_full + TCA_STAGES;
    uint64_t* v_full = k_empty + TCA_STAGES;
    uint64_t* v_empty = v_full + TCA_STAGES;
    uint64_t* s_full = v_empty + TCA_STAGES;                 // [2] the scores of a tile are in tensor memory
    uint64_t* s_empty = s_full + 2;                          // [2] the softmax warps have read them
    uint64_t* p_full = s_empty + 2;                          // [2] the probabilities are in tensor memory (and O is rescaled)
    uint64_t* pv_done = p_full + 2;                          // [2] the p.v products of a tile are done
    uint64_t* q_ready = pv_done + 2;                         // the queries are in tensor memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float2* ml_s = reinterpret_cast<float2*>(const_cast<int*>(abort_s) + 3);   // [2][128] maximum in use and sum of a row
    int* tbl_s = reinterpret_cast<int*>(ml_s + 2 * TCA_BM);  // [TCA_TABLE_CACHE]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = nh / nkv;
    const int tpt = TCA_BM / g;
    const int kh = blockIdx.y;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TCA_STAGES; ++s) {
            tca_mbar_init(k_full + s, 1);
            tca_mbar_init(k_empty + s, 1);
            tca_mbar_init(v_full + s, 1);
            tca_mbar_init(v_empty + s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            tca_mbar_init(s_full + i, 1);
            tca_mbar_init(s_empty + i, 4);
            tca_mbar_init(p_full + i, 4);
            tca_mbar_init(pv_done + i, 1);
        }
        tca_mbar_init(q_ready, 4);
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        tca_fence_async();
    }
    if (warp == 1) {       // all 512 columns of tensor memory (448 used at head size 128)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tca_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    pdl_wait();
    const int seg = seg_list ? seg_list[blockIdx.z] : blockIdx.z;
    const int q0 = cu_q[seg], qlen = cu_q[seg + 1] - q0;
    // the tiles with the most keys (the last tokens) are launched first, so that they do not form the tail
    // With n_parts = 2 a query tile has two blocks, neighbours in the grid: when the tile sees split_min key
    // tiles or more, each takes half of them and the one that finishes last adds the two partial results;
    // otherwise the first block takes all and the second has nothing to do.
    const int n_qt = (int)gridDim.x / n_parts;
    const int qt = (int)blockIdx.x / n_parts, part = (int)blockIdx.x - qt * n_parts;
    const int tok0 = (n_qt - 1 - qt) * tpt;
    const bool tile_ok = tok0 < qlen;                        // uniform for the block
    const int ntok = tile_ok ? min(tpt, qlen - tok0) : 0;
    const int pos0 = tile_ok ? positions[q0] + tok0 : 0;     // position of the tile's first token
    const int hi = pos0 + ntok;                              // one past the last visible key of the tile
    const int lo = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    int t_begin = lo / TCA_BN, t_end = tile_ok ? (hi + TCA_BN - 1) / TCA_BN : 0;
    const bool split = n_parts == 2 && tile_ok && t_end - t_begin >= split_min;
    if (split) {
        const int half = (t_end - t_begin + 1) / 2;
        if (part == 0) t_end = t_begin + half;
        else t_begin += half;
    }
    const bool active = tile_ok && (part == 0 || split);
    const int ntiles = active ? t_end - t_begin : 0;
    const int* table = block_table + (size_t)seg * table_stride;
    const int ppt = TCA_BN / page_size;
    if (active) {
        const int first_entry = t_begin * ppt;
        const int n_entries = min(ntiles * ppt, TCA_TABLE_CACHE);
        for (int i = threadIdx.x; i < n_entries; i += TCA_THREADS)
            tbl_s[i] = first_entry + i < table_stride ? table[first_entry + i] : 0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 || warp == 13) {
        // ---------------------------------------------------------------- producers: warp 0 copies keys, warp 13 values
        // keys: one box per (page, 64-dim block), [block][64 keys][128 bytes]; values: one box per page with
        // all its 64-dim blocks, [page][block][page rows][128 bytes].  Lane = box.
        const int kv = warp == 13;
        const int jobs = kv ? ppt : ppt * NH;
        const int h = kv ? 0 : lane % NH, pg = kv ? lane : lane / NH;
        const CUtensorMap* map = kv ? &v_map : &k_map;
        unsigned char* ring = (kv ? v_s : k_s) + (kv ? pg * page_size * (NH * 128) : h * SUB + pg * page_size * 128);
        uint64_t* full_b = kv ? v_full : k_full;
        uint64_t* empty_b = kv ? v_empty : k_empty;
        const int row_mul = nkv * page_size, row_add = kh * page_size;
        for (int it = 0; it < ntiles; ++it) {
            const int s = it % TCA_STAGES;
            if (it >= TCA_STAGES && !tca_wait(empty_b + s, ((it / TCA_STAGES) - 1) & 1)) {
                g_tca_status = 1;
                *abort_s = 1;
            }
            if (__any_sync(0xffffffffu, *abort_s != 0)) break;
            const int n0 = (t_begin + it) * TCA_BN;
            int first = 0, last = ppt;            // pages wholly outside [lo, hi) are not copied
            if (n0 < lo || n0 + TCA_BN > hi) {
                while (first < last && n0 + (first + 1) * page_size <= lo) ++first;
                while (last > first && n0 + (last - 1) * page_size >= hi) --last;
            }
            if (lane == 0) tca_expect_tx(full_b + s, (uint32_t)((last - first) * page_size * HD * 2));
            __syncwarp();
            if (lane < jobs && pg >= first && pg < last) {
                const int e = it * ppt + pg;
                const int page = e < TCA_TABLE_CACHE ? tbl_s[e] : table[n0 / page_size + pg];
                const int row = page * row_mul + row_add;
                if (kv) tca_tma_3d(ring + (size_t)s * KV_BYTES, map, 0, row, 0, full_b + s);
                else tca_tma_2d(ring + (size_t)s * KV_BYTES, map, h * 64, row, full_b + s);
            }
            __syncwarp();
        }
    } else if (warp == 1 || (warp >= 10 && warp <= 12)) {
        // ---------------------------------------------------------------- tensor-core issue
        // Two pipelines: even tiles use S, P, O number 0, odd tiles number 1, so that one tile's softmax
        // runs beside the other's; the two partial outputs are added at the end.  A tcgen05.mma costs its
        // issuing thread about a hundred clocks whatever its size, so four threads issue: warps 1 and 10
        // the S = Q K^T products of pipelines 0 and 1, warps 11 and 12 their O += P V products.
        const int pipe = (warp == 1 || warp == 11) ? 0 : 1;
        const bool is_pv = warp >= 11;
        if (lane == 0 && ntiles > pipe) {
            // float32 accumulate, bfloat16 operands; S: N = 64, both K-major; O: N = HD, b MN-major
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TCA_BN >> 3) << 17) | ((uint32_t)(TCA_BM >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TCA_BM >> 4) << 24);
            bool ok = true;
            // every descriptor is made once: per tile only the stage's offset (in 16-byte units) is added
            if (!is_pv) {
                uint64_t k_desc[NH * 4];
                const uint32_t k0 = tca_u32(k_s);
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16) k_desc[h * 4 + k16] = tca_desc_k(k0 + h * SUB, k16);
                const uint32_t ts = tmem_base + TCA_COL_S + pipe * TCA_BN, tq = tmem_base + TCA_COL_Q;
                ok = tca_wait(q_ready, 0);
                int j = 0;
                for (int it = pipe; ok && it < ntiles; it += 2, ++j) {
                    const int s = it % TCA_STAGES;
                    if (!tca_wait(k_full + s, (it / TCA_STAGES) & 1) || (j > 0 && !tca_wait(s_empty + pipe, (j - 1) & 1))) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint64_t stage = (uint64_t)(s * (KV_BYTES >> 4));
#pragma unroll
                    for (int i = 0; i < NH * 4; ++i) tca_mma_ts(ts, tq + i * 8, k_desc[i] + stage, idesc_s, i ? 1u : 0u);
                    tca_commit(k_empty + s);           // the keys of the stage have been read
                    tca_commit(s_full + pipe);
                }
            } else {
                uint64_t v_desc[4];
                // 16 keys per product: they lie in one page (two pages of 8 rows), 64-dim blocks page_size rows apart
                const uint32_t v0 = tca_u32(v_s), page_bytes = (uint32_t)(page_size * NH * 128);
                const uint32_t group_bytes = page_size >= 16 ? 1024u : page_bytes;
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16) {
                    const int key = k16 * 16;
                    v_desc[k16] = tca_desc_mn(v0 + (uint32_t)(key / page_size) * page_bytes + (uint32_t)(key % page_size) * 128u,
                                              (uint32_t)page_size * 128u, group_bytes);
                }
                const uint32_t tp = tmem_base + TCA_COL_P + pipe * (TCA_BN / 2), to = tmem_base + TCA_COL_O + pipe * HD;
                int j = 0;
                for (int it = pipe; it < ntiles; it += 2, ++j) {
                    const int s = it % TCA_STAGES;
                    if (!tca_wait(v_full + s, (it / TCA_STAGES) & 1) || !tca_wait(p_full + pipe, j & 1)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint64_t stage = (uint64_t)(s * (KV_BYTES >> 4));
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16) tca_mma_ts(to, tp + k16 * 8, v_desc[k16] + stage, idesc_o, (j | k16) ? 1u : 0u);
                    tca_commit(v_empty + s);           // the values of the stage have been read
                    tca_commit(pv_done + pipe);        // P may be overwritten, O holds this tile
                }
            }
            if (!ok) {
                g_tca_status = 1;
                *abort_s = 1;
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax warps: thread = row
        const int pipe = (warp - 2) >> 2;                    // warps 2-5: even tiles, warps 6-9: odd tiles
        const int qtr = warp & 3;
        const int r = qtr * 32 + lane;                       // row of the tile = tensor-memory lane
        const int tok = r / g, head = r - tok * g;
        const bool row_ok = tok < ntok;
        const int row_pos = row_ok ? pos0 + tok : -1;
        const int row_lo = (window > 0 && row_pos + 1 > window) ? row_pos + 1 - window : 0;
        const uint32_t lane_off = (uint32_t)(qtr * 32) << 16;
        const uint32_t tmem_s = tmem_base + TCA_COL_S + pipe * TCA_BN + lane_off;
        const uint32_t tmem_p = tmem_base + TCA_COL_P + pipe * (TCA_BN / 2) + lane_off;
        const uint32_t tmem_o = tmem_base + TCA_COL_O + pipe * HD + lane_off;
        if (pipe == 0) {
            // this thread's query row -> tensor memory, as the a operand of S = Q K^T: column i of the row holds
            // dims 2i and 2i + 1 (rows beyond the tile's tokens are zero)
            const bf16* qrow = q + (size_t)(q0 + tok0 + (row_ok ? tok : 0)) * q_row_stride + (size_t)(kh * g + head) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 2; c += 32) {
                uint32_t qv[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 v = row_ok ? *reinterpret_cast<const uint4*>(qrow + c * 2 + i * 8) : make_uint4(0u, 0u, 0u, 0u);
                    qv[4 * i] = v.x; qv[4 * i + 1] = v.y; qv[4 * i + 2] = v.z; qv[4 * i + 3] = v.w;
                }
                tca_st32(tmem_base + TCA_COL_Q + lane_off + c, qv);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tca_arrive(q_ready);
        }
        float m_use = -INFINITY, l = 0.f;                    // maximum in use (log2 units), running sum
        bool dead = false;
        const uint64_t scale2 = tca_pack(scale_log2, scale_log2);
        int j = 0;
        for (int it = pipe; it < ntiles; it += 2, ++j) {
            const int n0 = (t_begin + it) * TCA_BN;
            const int s = it % TCA_STAGES;
            bool waited = tca_wait(s_full + pipe, j & 1);
            if (!waited) {
                g_tca_status = 1;
                *abort_s = 1;
            }
            if (__any_sync(0xffffffffu, !waited || *abort_s != 0)) { dead = true; break; }      // the warp leaves together
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            uint32_t sv[64];
            tca_ld32(tmem_s, *reinterpret_cast<uint32_t(*)[32]>(sv));
            tca_ld32(tmem_s + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tca_arrive(s_empty + pipe);       // this pipeline's next scores may be written
            if (n0 + TCA_BN - 1 > pos0 || n0 < row_lo || n0 < lo) {      // some key may be hidden from some row
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int n = n0 + c;
                    if (!(n <= row_pos && n >= row_lo)) sv[c] = 0xff800000u;     // -inf
                }
            }
            // the maximum of the raw scores (the scale is positive), four chains of three-input maxima
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 64; c += 8) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    mx4[i] = tca_max3(mx4[i], __uint_as_float(sv[c + 2 * i]), __uint_as_float(sv[c + 2 * i + 1]));
            }
            const float mx = fmaxf(tca_max3(mx4[0], mx4[1], mx4[2]), mx4[3]) * scale_log2;
            // the maximum in use moves only when the true one has grown by more than 2^8: the same
            // value is used for the probabilities and for the sum, so the result is exact
            const bool grow = mx > m_use + TCA_RESCALE_AT;
            const float m_new = grow ? mx : m_use;
            const bool need = grow && m_use != -INFINITY;    // O holds something that has to be rescaled
            const float corr = need ? tca_exp2(m_use - m_new) : 1.0f;
            m_use = m_new;
            const float neg_m = m_use == -INFINITY ? 0.f : -m_use;
            const uint64_t neg_m2 = tca_pack(neg_m, neg_m);
            uint64_t sum2[2] = {0ull, 0ull};
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
                float x0, x1;
                tca_unpack(tca_fma2(tca_pack(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, neg_m2), x0, x1);
                const float p0 = tca_exp2(x0), p1 = tca_exp2(x1);
                sum2[(c >> 1) & 1] = tca_add2(sum2[(c >> 1) & 1], tca_pack(p0, p1));
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h2);
            }
            float sa, sb;
            tca_unpack(tca_add2(sum2[0], sum2[1]), sa, sb);
            l = l * corr + (sa + sb);
            // P and O of this pipeline's tile before must have been consumed / completed
            waited = j == 0 || tca_wait(pv_done + pipe, (j - 1) & 1);
            if (!waited) {
                g_tca_status = 1;
                *abort_s = 1;
            }
            if (__any_sync(0xffffffffu, !waited || *abort_s != 0)) { dead = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t ov[32];
                    tca_ld32(tmem_o + c, ov);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    tca_st32(tmem_o + c, ov);
                }
            }
            // probabilities -> tensor memory: column i of the row holds keys 2i (low half) and 2i + 1
            tca_st32(tmem_p, pk);
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            // value rows outside [lo, hi) may hold anything (pages given back, what lies beyond the
            // request's last token): they are cleared before the tensor core multiplies them by zero
            if (n0 < lo || n0 + TCA_BN > hi) {
                if (!tca_wait(v_full + s, (it / TCA_STAGES) & 1)) {
                    g_tca_status = 1;
                    *abort_s = 1;
                }
                unsigned char* vt = v_s + (size_t)s * KV_BYTES;
                const int key = r & 63;
                const int n = n0 + key;
                if (n < lo || n >= hi) {
                    for (int h = r >> 6; h < NH; h += 2) {
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(vt + ((key / page_size) * NH + h) * (page_size * 128) + (key % page_size) * 128 + c * 16) =
                                make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                tca_fence_async();
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tca_arrive(p_full + pipe);
        }
        // this pipeline's last p.v
        if (!dead && j > 0 && !tca_wait(pv_done + pipe, (j - 1) & 1)) {
            g_tca_status = 1;
            *abort_s = 1;
        }
        ml_s[pipe * TCA_BM + r] = make_float2(m_use, l);
        // one thread's view of the error flag, so that all 256 take the same way through the barriers below
        if (r == 0 && pipe == 0) const_cast<int*>(abort_s)[2] = *abort_s;
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        tca_softmax_sync();              // every softmax thread comes here
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (ntiles > 0 && !abort_s[2]) {
            // out = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)); each pipeline's
            // warps write half of the head's dims.  A pipeline without tiles holds nothing that may be read.
            const bool two = ntiles > 1;
            const float2 a = ml_s[r], b = two ? ml_s[TCA_BM + r] : make_float2(-INFINITY, 0.f);
            const float m = fmaxf(a.x, b.x);
            const float fa = a.x == -INFINITY ? 0.f : tca_exp2(a.x - m), fb = b.x == -INFINITY ? 0.f : tca_exp2(b.x - m);
            const float den = a.y * fa + b.y * fb;
            const uint32_t o_a = tmem_base + TCA_COL_O + lane_off, o_b = o_a + HD;
            const size_t orow = (size_t)(q0 + tok0 + (row_ok ? tok : 0)) * nh + kh * g + head;
            bf16* dst = out + orow * HD;
            float wa = fa, wb = fb, w_other = 0.f;            // weights of this block's two sums and of the other block's
            const float* other_o = nullptr;
            bool write_out = true;
            if (split) {
                // this block's sum, not yet divided, and its maximum and denominator go to scratch; the block of
                // the pair that gets there last reads the other's and writes the result.  The sum below is the same
                // whichever of the two comes last.
                float* my_o = part_o + ((size_t)part * n_rows + orow) * HD;
#pragma unroll 1
                for (int c = pipe * (HD / 2); c < (pipe + 1) * (HD / 2); c += 32) {
                    uint32_t ov[32], ow[32];
                    tca_ld32(o_a + c, ov);
                    if (two) tca_ld32(o_b + c, ow);          // a pipeline without tiles holds nothing that may be read
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float4 y;
                            y.x = __uint_as_float(ov[i]) * fa;
                            y.y = __uint_as_float(ov[i + 1]) * fa;
                            y.z = __uint_as_float(ov[i + 2]) * fa;
                            y.w = __uint_as_float(ov[i + 3]) * fa;
                            if (two) {
                                y.x += __uint_as_float(ow[i]) * fb;
                                y.y += __uint_as_float(ow[i + 1]) * fb;
                                y.z += __uint_as_float(ow[i + 2]) * fb;
                                y.w += __uint_as_float(ow[i + 3]) * fb;
                            }
                            *reinterpret_cast<float4*>(my_o + c + i) = y;
                        }
                    }
                }
                if (pipe == 0 && row_ok)
                    *reinterpret_cast<float2*>(part_ml + ((size_t)part * n_rows + orow) * 2) = make_float2(m, den);
                __threadfence();
                tca_softmax_sync();
                if (r == 0 && pipe == 0) {
                    int* cnt = counters + ((size_t)blockIdx.z * nkv + kh) * n_qt + qt;
                    const int before = atomicAdd(cnt, 1);
                    if (before == 1) *cnt = 0;                 // both have arrived: ready for the next launch
                    const_cast<int*>(abort_s)[1] = before;
                }
                tca_softmax_sync();
                write_out = abort_s[1] == 1;
                if (write_out) {
                    __threadfence();
                    other_o = part_o + ((size_t)(1 - part) * n_rows + orow) * HD;
                    const float2 o_ml = row_ok ? __ldcg(reinterpret_cast<const float2*>(part_ml + ((size_t)(1 - part) * n_rows + orow) * 2))
                                               : make_float2(-INFINITY, 0.f);
                    const float mm = fmaxf(m, o_ml.x);
                    const float f1 = m == -INFINITY ? 0.f : tca_exp2(m - mm), f2 = o_ml.x == -INFINITY ? 0.f : tca_exp2(o_ml.x - mm);
                    const float dd = den * f1 + o_ml.y * f2;
                    const float inv2 = dd > 0.f ? 1.0f / dd : 0.f;
                    wa = fa * f1 * inv2;
                    wb = fb * f1 * inv2;
                    w_other = f2 * inv2;
                }
            } else {
                const float inv = den > 0.f ? 1.0f / den : 0.f;
                wa = fa * inv;
                wb = fb * inv;
            }
            if (write_out) {
#pragma unroll 1
            for (int c = pipe * (HD / 2); c < (pipe + 1) * (HD / 2); c += 32) {
                uint32_t ov[32], ow[32];
                tca_ld32(o_a + c, ov);
                if (two) tca_ld32(o_b + c, ow);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 o4;
                        uint32_t* o32 = reinterpret_cast<uint32_t*>(&o4);
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            float y0 = __uint_as_float(ov[i + e]) * wa, y1 = __uint_as_float(ov[i + e + 1]) * wa;
                            if (two) {
                                y0 += __uint_as_float(ow[i + e]) * wb;
                                y1 += __uint_as_float(ow[i + e + 1]) * wb;
                            }
                            if (other_o) {
                                const float2 t2 = __ldcg(reinterpret_cast<const float2*>(other_o + c + i + e));
                                y0 += t2.x * w_other;
                                y1 += t2.y * w_other;
                            }
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(y0, y1);
                            o32[e / 2] = *reinterpret_cast<uint32_t*>(&h2);
                        }
                        *reinterpret_cast<uint4*>(dst + c + i) = o4;
                    }
                }
            }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*TcaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TcaEncodeFn tca_encode_fn() {
    static TcaEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) == cudaSuccess &&
            st == cudaDriverEntryPointSuccess)
            fn = (TcaEncodeFn)p;
    }
    return fn;
}

// Tensor map over the cache pages of one layer ([rows, hd] bfloat16, rows = pages * kv_heads * page_size)
// read in boxes of [page_size rows, 64 dims] with the 128-byte swizzle: the operand layout of tcgen05.mma.
// With `all_blocks` (the values) a box holds all 64-dim blocks of the page rows, one block after the other.
PICO_API int pico_make_kv_tensor_map_2d(void* map_out, const void* base, long long rows, int hd, int page_size, int all_blocks) {
    if (hd % 64 != 0 || hd < 64 || hd > 128 || page_size < 8 || page_size > TCA_BN || TCA_BN % page_size != 0 ||
        (page_size & 7) != 0 || ((uintptr_t)base & 15) != 0)
        return PICO_ERR_SIZE;
    TcaEncodeFn fn = tca_encode_fn();
    if (!fn) return -7;
    if (all_blocks) {
        const cuuint64_t dims3[3] = {64, (cuuint64_t)rows, (cuuint64_t)(hd / 64)};
        const cuuint64_t strides3[2] = {(cuuint64_t)hd * 2, 128};
        const cuuint32_t box3[3] = {64, (cuuint32_t)page_size, (cuuint32_t)(hd / 64)};
        const cuuint32_t estr3[3] = {1, 1, 1};
        const CUresult r3 = fn((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims3,
                               strides3, box3, estr3, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r3 == CUDA_SUCCESS ? 0 : -7;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -7;
}

// Prompt portions on tcgen05; arguments as pico_paged_prefill_mma, with the 2-D tensor maps above.
// pair_min_keys > 0: every query tile gets two blocks, and a tile that sees at least that many keys is shared by
// them.  This pays when a few long tiles would otherwise set the kernel's time (a portion late in a long context:
// 286 instead of 331 us for 2,048 tokens after 14,336); a pair costs ~10 us for its second prologue, the partial
// results through scratch and their sum, so short tiles lose (2,048 tokens from the start: 57 instead of 30 us when
// tiles from 512 keys on are shared).  scratch: float32 [2][n_tokens][nh][hd + 2]; counters: n_counters int32,
// zero before the first launch (the kernel leaves them zero).
PICO_API int pico_paged_prefill_tcgen05(const void* k_map, const void* v_map, const void* q, int q_row_stride, void* out,
                                        const int* seg_list, int n_segs, const int* cu_q, int max_q_len,
                                        const int* positions, const int* block_table, int table_stride, int nh, int nkv,
                                        int hd, int page_size, int window, float scale, int pair_min_keys, float* scratch,
                                        int n_tokens, int* counters, int n_counters, cudaStream_t stream) {
    if (n_segs <= 0 || max_q_len <= 0) return 0;
    if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv != 0) return PICO_ERR_SIZE;
    const int g = nh / nkv;
    if (g > TCA_BM || nkv > 65535 || n_segs > 65535) return PICO_ERR_SIZE;
    if (page_size < 8 || TCA_BN % page_size != 0) return PICO_ERR_SIZE;
    if (q_row_stride % 8 != 0) return PICO_ERR_ALIGN;
    const int tpt = TCA_BM / g;
    const int n_qt = (max_q_len + tpt - 1) / tpt;
    const int n_parts = (pair_min_keys > 0 && scratch && counters && (long long)n_qt * nkv * n_segs <= n_counters && n_tokens > 0) ? 2 : 1;
    const size_t n_rows = (size_t)n_tokens * nh;
    const int split_min = pair_min_keys / TCA_BN > 2 ? pair_min_keys / TCA_BN : 2;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + 2 * n_rows * hd : nullptr;
    const dim3 grid(n_qt * n_parts, nkv, n_segs);
    const float scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = (size_t)TCA_STAGES * 2 * TCA_BN * hd * 2 + (4 * TCA_STAGES + 9) * 8 + 16 + 2 * TCA_BM * 8 + TCA_TABLE_CACHE * 4 + 1024;
    CUtensorMap km, vm;
    memcpy(&km, k_map, sizeof(CUtensorMap));
    memcpy(&vm, v_map, sizeof(CUtensorMap));
#define LAUNCH_TCA(HD)                                                                                                   \
    do {                                                                                                                 \
        cudaFuncSetAttribute(paged_prefill_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        pico_launch((paged_prefill_tcgen05_kernel<HD>), grid, dim3(TCA_THREADS), smem, stream, km, vm, (const bf16*)q,   \
                    q_row_stride, (bf16*)out, seg_list, cu_q, positions, block_table, table_stride, nh, nkv, page_size,  \
                    window, scale_log2, part_o, part_ml, counters, n_rows, n_parts, split_min);                          \
    } while (0)
    if (hd == 64) LAUNCH_TCA(64);
    else LAUNCH_TCA(128);
#undef LAUNCH_TCA
    return pico_launch_status();
}

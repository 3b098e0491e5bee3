// Paged causal attention for portions of prompts ("prefill") on the 5th-generation tensor cores.
//
// A block takes 128 rows of queries - 128 / g tokens of one segment times the g query heads that
// share a key/value head - and walks the visible cache positions 64 at a time:
//   warp 0      issues the TMA copies of the pages of a tile (keys and values, [page rows, 64 dims]
//               boxes in the 128-byte swizzle, several lanes issuing in parallel);
//   warp 1      one lane issues tcgen05.mma: S = Q K^T (M 128, N 64, accumulator S in tensor memory)
//               and, once the probabilities are ready, O += P V (M 128, N head_dim, V as an MN-major
//               operand, accumulator O in tensor memory); tcgen05.commit signals mbarriers;
//   warps 2-5   softmax: thread = row.  tcgen05.ld of the row's 64 scores, mask, running max and sum in
//               float32 (exp2 on scores scaled to log2 units), probabilities as bfloat16 into shared
//               memory in the operand layout; the O accumulator is rescaled in tensor memory
//               (tcgen05.ld / st) only when a row's maximum has grown by more than 2^8 since the value in
//               use, which is exact because the same maximum is used for the sum; at the end O / sum.
// Rules restated from the reference: query head j reads key/value head j / g
// (pico_vllm/kernels/attention.py:139); scores * hd^-1/2 (attention.py:231); key n visible to the
// query at position p iff n <= p (attention.py:193-198) - and n > p - window with a window; online
// softmax in float32, p rounded to the cache type before p.v (attention.py:189-213).
// Every mbarrier wait is bounded (status word pico_tca_status); tensor memory is freed on every path.
#include <cuda.h>
#include "common.cuh"

#define TCA_BM 128
#define TCA_BN 64
#define TCA_THREADS 192
#define TCA_STAGES 3
#define TCA_WAIT_LIMIT (1 << 20)
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
// K-major operand [rows][64 bf16] in the 128-byte swizzle (rows 128 bytes, 8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t tca_desc_k(uint32_t tile, int k16) {
    const uint32_t addr = tile + k16 * 32;
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// MN-major operand: values [keys][head dims], head dims contiguous, stored as blocks of [64 keys][64 dims]
// (128-byte rows, 128-byte swizzle): 8-key groups 1024 bytes apart (stride byte offset), 64-dim blocks
// `block_bytes` apart (leading byte offset).  k16 selects 16 keys.
__device__ __forceinline__ uint64_t tca_desc_mn(uint32_t tile, int k16, uint32_t block_bytes) {
    const uint32_t addr = tile + k16 * 16 * 128;
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)((block_bytes >> 4) & 0x3fff) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
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
__device__ __forceinline__ void tca_sm_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

template <int HD>      // head size, a multiple of 64 up to 128
__global__ void __launch_bounds__(TCA_THREADS)
paged_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                             const bf16* __restrict__ q, int q_row_stride, bf16* __restrict__ out,
                             const int* __restrict__ seg_list, const int* __restrict__ cu_q,
                             const int* __restrict__ positions, const int* __restrict__ block_table, int table_stride,
                             int nh, int nkv, int page_size, int window, float scale_log2) {
    pdl_launch_dependents();
    extern __shared__ unsigned char tca_dyn[];
    constexpr int NH = HD / 64;                              // 64-dim blocks of a head
    constexpr int SUB = TCA_BN * 128;                        // bytes of one [64 keys][64 dims] block
    constexpr int KV_BYTES = NH * SUB;                       // one K (or V) tile
    constexpr int QSUB = TCA_BM * 128;                       // bytes of one [128 rows][64 dims] block of Q
    unsigned char* smem = tca_dyn + ((1024u - (tca_u32(tca_dyn) & 1023u)) & 1023u);
    unsigned char* q_s = smem;                               // [NH][128 rows][128 B]
    unsigned char* p_s = q_s + NH * QSUB;                    // [128 rows][128 B]: probabilities of 64 keys
    unsigned char* kv_s = p_s + QSUB;                        // [stages][K tile | V tile]
    uint64_t* kv_full = reinterpret_cast<uint64_t*>(kv_s + TCA_STAGES * 2 * KV_BYTES);
    uint64_t* kv_empty = kv_full + TCA_STAGES;
    uint64_t* s_full = kv_empty + TCA_STAGES;                // the scores of a tile are in tensor memory
    uint64_t* s_empty = s_full + 1;                          // the softmax warps have read them
    uint64_t* p_full = s_empty + 1;                          // the probabilities are in shared memory (and O is rescaled)
    uint64_t* pv_done = p_full + 1;                          // the p.v products of a tile are done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* tbl_s = const_cast<int*>(abort_s) + 2;              // [TCA_TABLE_CACHE]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = nh / nkv;
    const int tpt = TCA_BM / g;
    const int kh = blockIdx.y;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TCA_STAGES; ++s) {
            tca_mbar_init(kv_full + s, 1);
            tca_mbar_init(kv_empty + s, 1);
        }
        tca_mbar_init(s_full, 1);
        tca_mbar_init(s_empty, 4);
        tca_mbar_init(p_full, 4);
        tca_mbar_init(pv_done, 1);
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        tca_fence_async();
    }
    if (warp == 1) {       // tensor memory: 64 columns of scores + HD columns of output (256 allocated)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tca_u32(tmem_slot)), "r"(256));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    pdl_wait();
    const int seg = seg_list ? seg_list[blockIdx.z] : blockIdx.z;
    const int q0 = cu_q[seg], qlen = cu_q[seg + 1] - q0;
    // the tiles with the most keys (the last tokens) are launched first, so that they do not form the tail
    const int tok0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * tpt;
    const bool active = tok0 < qlen;                         // uniform for the block
    const int ntok = active ? min(tpt, qlen - tok0) : 0;
    const int pos0 = active ? positions[q0] + tok0 : 0;      // position of the tile's first token
    const int hi = pos0 + ntok;                              // one past the last visible key of the tile
    const int lo = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int t_begin = lo / TCA_BN, t_end = active ? (hi + TCA_BN - 1) / TCA_BN : 0;
    const int ntiles = active ? t_end - t_begin : 0;
    const int* table = block_table + (size_t)seg * table_stride;
    const int ppt = TCA_BN / page_size;
    if (active) {
        const int first_entry = t_begin * ppt;
        const int n_entries = min(ntiles * ppt, TCA_TABLE_CACHE);
        for (int i = threadIdx.x; i < n_entries; i += TCA_THREADS)
            tbl_s[i] = first_entry + i < table_stride ? table[first_entry + i] : 0;
        // queries -> shared memory in the operand layout: row r = token * g + head, 16-byte piece c of
        // block h at q_s + h * QSUB + r * 128 + ((c ^ (r & 7)) << 4); rows beyond the tile are zero
        for (int idx = threadIdx.x; idx < TCA_BM * (HD / 8); idx += TCA_THREADS) {
            const int r = idx / (HD / 8), c = idx - r * (HD / 8);
            const int tok = r / g, head = r - tok * g;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (tok < ntok)
                v = *reinterpret_cast<const uint4*>(q + (size_t)(q0 + tok0 + tok) * q_row_stride + (size_t)(kh * g + head) * HD + c * 8);
            *reinterpret_cast<uint4*>(q_s + (c >> 3) * QSUB + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
        }
        tca_fence_async();       // the tensor core reads Q through the async proxy
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + TCA_BN;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer: lane 2*(pg*NH+h) + {0: K, 1: V}
        for (int it = 0; it < ntiles; ++it) {
            const int s = it % TCA_STAGES;
            if (it >= TCA_STAGES && !tca_wait(kv_empty + s, ((it / TCA_STAGES) - 1) & 1)) {
                g_tca_status = 1;
                *abort_s = 1;
            }
            __syncwarp();
            if (*abort_s) break;
            const int n0 = (t_begin + it) * TCA_BN;
            unsigned char* kt = kv_s + (size_t)s * 2 * KV_BYTES;
            int first = 0, last = ppt;        // pages wholly outside [lo, hi) are not copied
            while (first < last && n0 + (first + 1) * page_size <= lo) ++first;
            while (last > first && n0 + (last - 1) * page_size >= hi) --last;
            if (lane == 0) tca_expect_tx(kv_full + s, (uint32_t)((last - first) * page_size * HD * 2 * 2));
            __syncwarp();
            for (int job = lane; job < ppt * NH * 2; job += 32) {
                const int kv = job & 1, h = (job >> 1) % NH, pg = (job >> 1) / NH;
                if (pg >= first && pg < last) {
                    const int e = it * ppt + pg;
                    const int page = e < TCA_TABLE_CACHE ? tbl_s[e] : table[n0 / page_size + pg];
                    const int row = (page * nkv + kh) * page_size;
                    tca_tma_2d(kt + kv * KV_BYTES + h * SUB + pg * page_size * 128, kv ? &v_map : &k_map, h * 64, row,
                               kv_full + s);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- tensor-core issue
        if (lane == 0 && ntiles > 0) {
            // float32 accumulate, bfloat16 operands; S: N = 64, both K-major; O: N = HD, b MN-major
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TCA_BN >> 3) << 17) | ((uint32_t)(TCA_BM >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TCA_BM >> 4) << 24);
            const uint32_t qa = tca_u32(q_s), pa = tca_u32(p_s);
            auto issue_qk = [&](int it) -> bool {
                const int s = it % TCA_STAGES;
                if (!tca_wait(kv_full + s, (it / TCA_STAGES) & 1)) return false;
                if (it > 0 && !tca_wait(s_empty, (it - 1) & 1)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t kt = tca_u32(kv_s + (size_t)s * 2 * KV_BYTES);
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)
                        tca_mma(tmem_s, tca_desc_k(qa + h * QSUB, k16), tca_desc_k(kt + h * SUB, k16), idesc_s, (h | k16) ? 1u : 0u);
                tca_commit(s_full);
                return true;
            };
            bool ok = issue_qk(0);
            for (int it = 0; ok && it < ntiles; ++it) {
                if (it + 1 < ntiles) ok = issue_qk(it + 1);           // the next tile's scores while this tile's softmax runs
                if (!ok) break;
                if (!tca_wait(p_full, it & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const int s = it % TCA_STAGES;
                const uint32_t vt = tca_u32(kv_s + (size_t)s * 2 * KV_BYTES + KV_BYTES);
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)
                    tca_mma(tmem_o, tca_desc_k(pa, k16), tca_desc_mn(vt, k16, SUB), idesc_o, (it | k16) ? 1u : 0u);
                tca_commit(kv_empty + s);      // keys and values of the stage have been read
                tca_commit(pv_done);           // P may be overwritten, O holds this tile
            }
            if (!ok) {
                g_tca_status = 1;
                *abort_s = 1;
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax warps: thread = row
        const int qtr = warp & 3;
        const int r = qtr * 32 + lane;                       // row of the tile = tensor-memory lane
        const int tok = r / g, head = r - tok * g;
        const bool row_ok = tok < ntok;
        const int row_pos = row_ok ? pos0 + tok : -1;
        const int row_lo = (window > 0 && row_pos + 1 > window) ? row_pos + 1 - window : 0;
        const uint32_t lane_off = (uint32_t)(qtr * 32) << 16;
        float m_use = -INFINITY, l = 0.f;                    // maximum in use (log2 units), running sum
        bool dead = false;
        for (int it = 0; it < ntiles; ++it) {
            const int n0 = (t_begin + it) * TCA_BN;
            const int s = it % TCA_STAGES;
            if (!tca_wait(s_full, it & 1)) {
                g_tca_status = 1;
                *abort_s = 1;
            }
            if (*abort_s) { dead = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            uint32_t sv[64];
            tca_ld32(tmem_s + lane_off, *reinterpret_cast<uint32_t(*)[32]>(sv));
            tca_ld32(tmem_s + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tca_arrive(s_empty);              // the next tile's scores may be written
            const bool edge = n0 + TCA_BN - 1 > pos0 || n0 < row_lo || n0 < lo;       // some key may be hidden from some row
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 64; ++c) {
                float x = __uint_as_float(sv[c]) * scale_log2;
                if (edge) {
                    const int n = n0 + c;
                    if (!(n <= row_pos && n >= row_lo)) x = -INFINITY;
                }
                sv[c] = __float_as_uint(x);
                mx = fmaxf(mx, x);
            }
            // the maximum in use moves only when the true one has grown by more than 2^8: the same
            // value is used for the probabilities and for the sum, so the result is exact
            const bool grow = mx > m_use + TCA_RESCALE_AT;
            const float m_new = grow ? mx : m_use;
            const float corr = (grow && m_use != -INFINITY) ? tca_exp2(m_use - m_new) : 1.0f;
            const bool need = grow && m_use != -INFINITY;    // O holds something that has to be rescaled
            m_use = m_new;
            const float m_sub = m_use == -INFINITY ? 0.f : m_use;
            float sum = 0.f;
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
                const float p0 = tca_exp2(__uint_as_float(sv[c]) - m_sub), p1 = tca_exp2(__uint_as_float(sv[c + 1]) - m_sub);
                sum += p0 + p1;
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h2);
            }
            l = l * corr + sum;
            // P and O of the tile before must have been consumed / completed
            if (it > 0 && !tca_wait(pv_done, (it - 1) & 1)) {
                g_tca_status = 1;
                *abort_s = 1;
            }
            if (*abort_s) { dead = true; break; }
            if (__any_sync(0xffffffffu, need)) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t ov[32];
                    tca_ld32(tmem_o + lane_off + c, ov);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * corr);
                    tca_st32(tmem_o + lane_off + c, ov);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            // probabilities -> shared memory, operand layout
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(p_s + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            // value rows outside [lo, hi) may hold anything (pages given back, what lies beyond the
            // request's last token): they are cleared before the tensor core multiplies them by zero
            if (n0 < lo || n0 + TCA_BN > hi) {
                if (!tca_wait(kv_full + s, (it / TCA_STAGES) & 1)) {
                    g_tca_status = 1;
                    *abort_s = 1;
                }
                unsigned char* vt = kv_s + (size_t)s * 2 * KV_BYTES + KV_BYTES;
                const int key = r & 63;
                const int n = n0 + key;
                if (n < lo || n >= hi) {
                    for (int h = r >> 6; h < NH; h += 2) {
#pragma unroll
                        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(vt + h * SUB + key * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            tca_fence_async();
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tca_arrive(p_full);
        }
        if (!dead && ntiles > 0) {
            if (!tca_wait(pv_done, (ntiles - 1) & 1)) {
                g_tca_status = 1;
                *abort_s = 1;
                dead = true;
            }
        }
        if (!dead && ntiles > 0 && !*abort_s) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = out + ((size_t)(q0 + tok0 + (row_ok ? tok : 0)) * nh + kh * g + head) * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t ov[32];
                tca_ld32(tmem_o + lane_off + c, ov);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 o4;
                        uint32_t* ow = reinterpret_cast<uint32_t*>(&o4);
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(ov[j + e]) * inv, __uint_as_float(ov[j + e + 1]) * inv);
                            ow[e / 2] = *reinterpret_cast<uint32_t*>(&h2);
                        }
                        *reinterpret_cast<uint4*>(dst + c + j) = o4;
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(256));
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
PICO_API int pico_make_kv_tensor_map_2d(void* map_out, const void* base, long long rows, int hd, int page_size) {
    if (hd % 64 != 0 || hd < 64 || hd > 128 || page_size < 8 || page_size > TCA_BN || TCA_BN % page_size != 0 ||
        (page_size & 7) != 0 || ((uintptr_t)base & 15) != 0)
        return PICO_ERR_SIZE;
    TcaEncodeFn fn = tca_encode_fn();
    if (!fn) return -7;
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
PICO_API int pico_paged_prefill_tcgen05(const void* k_map, const void* v_map, const void* q, int q_row_stride, void* out,
                                        const int* seg_list, int n_segs, const int* cu_q, int max_q_len,
                                        const int* positions, const int* block_table, int table_stride, int nh, int nkv,
                                        int hd, int page_size, int window, float scale, cudaStream_t stream) {
    if (n_segs <= 0 || max_q_len <= 0) return 0;
    if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv != 0) return PICO_ERR_SIZE;
    const int g = nh / nkv;
    if (g > TCA_BM || nkv > 65535 || n_segs > 65535) return PICO_ERR_SIZE;
    if (page_size < 8 || TCA_BN % page_size != 0) return PICO_ERR_SIZE;
    if (q_row_stride % 8 != 0) return PICO_ERR_ALIGN;
    const int tpt = TCA_BM / g;
    const dim3 grid((max_q_len + tpt - 1) / tpt, nkv, n_segs);
    const float scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = (size_t)(hd / 64 + 1) * TCA_BM * 128 + (size_t)TCA_STAGES * 2 * TCA_BN * hd * 2 +
                        (2 * TCA_STAGES + 4) * 8 + 16 + TCA_TABLE_CACHE * 4 + 1024;
    CUtensorMap km, vm;
    memcpy(&km, k_map, sizeof(CUtensorMap));
    memcpy(&vm, v_map, sizeof(CUtensorMap));
#define LAUNCH_TCA(HD)                                                                                                   \
    do {                                                                                                                 \
        cudaFuncSetAttribute(paged_prefill_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        pico_launch((paged_prefill_tcgen05_kernel<HD>), grid, dim3(TCA_THREADS), smem, stream, km, vm, (const bf16*)q,   \
                    q_row_stride, (bf16*)out, seg_list, cu_q, positions, block_table, table_stride, nh, nkv, page_size,  \
                    window, scale_log2);                                                                                 \
    } while (0)
    if (hd == 64) LAUNCH_TCA(64);
    else LAUNCH_TCA(128);
#undef LAUNCH_TCA
    return pico_launch_status();
}

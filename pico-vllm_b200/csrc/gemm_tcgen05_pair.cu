// Matrix products for many tokens (prefill) on the 5th-generation tensor cores, two SMs per tile:
// y[m, n] = sum_k x[m, k] w[n, k], bfloat16 in, float32 accumulate in tensor memory.
//
// A cluster of two blocks computes a 256 x BN tile of y with tcgen05.mma.cta_group::2 (M 256, N BN,
// K 16): each block holds 128 rows of x and HALF of the w rows of the tile in its shared memory, the
// instruction reads both halves, and each block's tensor memory receives its own 128 rows of the
// accumulator.  Compared with one block per tile this halves the shared-memory bytes a product reads
// for w, which is what bounds the one-block form (measured: 171 clocks per 128 x 256 x 16 product from
// shared memory against 136 at the tensor cores' rate).  Roles by warp, in both blocks unless said:
//   warp 0   one lane issues the TMA copies (128-byte swizzle) of its block's x tile [128 rows, 64 k]
//            and its half of the w tile [BN / 2 rows, 64 k]; the copies of both blocks complete on the
//            full barrier of block 0, whose producer posts the expected bytes of both;
//   warp 1   allocates tensor memory (2 x BN columns, with the pair's other block); in block 0 one
//            lane issues the products and tcgen05.commit with cluster multicast, which frees the
//            stage in both blocks and, after the last k-block, tells both epilogues;
//   warps 2-5  epilogue of the block's 128 rows: tcgen05.ld, epilogue, store; then an arrival on
//            block 0's acc_empty barrier (a remote arrival from block 1).
// Epilogues as in gemm_tcgen05.cu: STORE (bfloat16), RESIDUAL (float32 x_res += y, in place), SWIGLU
// (block 0 loads gate rows n0.., block 1 the same features' up rows I + n0..; out = silu(gate) * up).
// Nothing here is multicast by TMA: each block copies what it alone needs.
//
// The reference runs these products as cuBLAS nn.Linear calls and a separate SwiGLU
// (pico_vllm/model.py:200-225, 309-318); silu(g) = g * sigmoid(g) (pico_vllm/kernels/swiglu.py:36-41).
// Every mbarrier wait is bounded; a block that gives up sets the status word read by
// pico_tp_status, still meets its partner at the cluster barrier and frees its tensor memory.
#include <cuda.h>
#include "common.cuh"

#define TP_BM 128              // rows of x per block (256 per pair)
#define TP_BK 64
#define TP_THREADS 192
#define TP_WAIT_LIMIT (1 << 14)      // polls of a barrier (some microseconds each) before a thread gives up

enum { TP_STORE = 0, TP_RESIDUAL = 1, TP_SWIGLU = 2 };

__device__ int g_tp_status = 0;
PICO_API int pico_tp_status(int* out) {
    return (int)cudaMemcpyFromSymbol(out, g_tp_status, sizeof(int), 0, cudaMemcpyDeviceToHost);
}

__device__ __forceinline__ uint32_t tp_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tp_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tp_u32(bar)), "r"(count));
}
__device__ __forceinline__ void tp_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tp_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tp_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < TP_WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(tp_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// The copy lands in this block's shared memory; its bytes are counted on the barrier at the same
// offset in the pair's even block (bit 24 of a shared::cluster address is the block's rank in the pair).
__device__ __forceinline__ void tp_tma_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(tp_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(tp_u32(bar) & 0xFEFFFFFFu)
        : "memory");
}
__device__ __forceinline__ uint64_t tp_desc(uint32_t tile_addr, int k16) {
    const uint32_t addr = tile_addr + k16 * 32;
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tp_mma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(zero) : "memory");
}
// arrives on the barrier at this offset in both blocks of the pair when the products issued so far are done
__device__ __forceinline__ void tp_commit_both(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(tp_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void tp_arrive_rank0(uint64_t* bar) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(tp_u32(bar)), "r"(0));
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(remote) : "memory");
}
__device__ __forceinline__ void tp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tp_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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

struct TpArgs {
    int M, N, K;              // N: rows of w (SWIGLU: 2 * I)
    bf16* out;                // STORE: [M, N]; SWIGLU: [M, N / 2]
    float* resid;             // RESIDUAL: [M, N]
};

__device__ __forceinline__ void tp_st32(void* p, const uint32_t (&r)[8]) {      // one 32-byte store (a whole sector)
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n"
                 ::"l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tp_ld8(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "l"(p));
}
// silu(g) * u = g * u / (1 + 2^(-g log2 e)) in float32 with the fast exponential and reciprocal
__device__ __forceinline__ float tp_silu_mul(float g, float u) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(g * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(1.0f + e));
    return g * r * u;
}
__device__ __forceinline__ uint32_t tp_pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Pairs are persistent: pair c computes tiles c, c + pairs, ... (tile t = n-block t / m_tiles, m-block
// t % m_tiles of MB * 256 rows).  MB = 1: a block holds 128 rows of x and the accumulator is
// double-buffered in tensor memory (the epilogue of a tile runs beside the products of the next).
// MB = 2: a block holds 256 rows (two products per k step share its half of the w tile, which cuts
// the bytes that come from L2 per product by a quarter - at these sizes the copies, not the tensor
// cores, set the pace), the two accumulators fill tensor memory, and eight epilogue warps drain them.
template <int BN, int EPI, int STAGES, int MB>
__global__ void __launch_bounds__(64 + 128 * MB)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map, const TpArgs p,
                         int m_tiles, int n_tiles) {
    pdl_launch_dependents();
    extern __shared__ unsigned char tp_dyn[];
    unsigned char* smem = tp_dyn + ((1024u - (tp_u32(tp_dyn) & 1023u)) & 1023u);
    constexpr int ROWS = MB * TP_BM;                           // rows of x per block
    constexpr int NBUF = MB == 1 ? 2 : 1;                      // accumulator buffers (of MB accumulators each)
    constexpr int A_BLOCK = TP_BM * TP_BK * 2, A_BYTES = MB * A_BLOCK, B_BYTES = (BN / 2) * TP_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int COLS = EPI == TP_SWIGLU ? BN / 2 : BN;       // output columns of a tile
    constexpr int TMEM_COLS = 512;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);      // used in block 0: both blocks' copies landed
    uint64_t* empty = full + STAGES;                           // the products have read the stage (both blocks)
    uint64_t* acc_full = empty + STAGES;                       // [NBUF]: the products of a tile are done (both blocks)
    uint64_t* acc_empty = acc_full + 2;                        // [NBUF], used in block 0: both epilogues have read the buffer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int nkb = (p.K + TP_BK - 1) / TP_BK;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tp_mbar_init(full + s, 1);
            tp_mbar_init(empty + s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            tp_mbar_init(acc_full + i, 1);
            tp_mbar_init(acc_empty + i, 8 * MB);               // one arrival per epilogue warp of both blocks
        }
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tp_u32(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    tp_cluster_sync();          // both blocks' barriers are initialised before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                 // x comes from the kernel before

    if (warp == 0) {
        if (lane == 0) {
            int step = 0;
            for (int t = pair; t < total_tiles && !*abort_s; t += n_pairs) {
                const int m0 = (t % m_tiles) * 2 * ROWS + (int)rank * ROWS, n0 = (t / m_tiles) * COLS;
                const int w_row = EPI == TP_SWIGLU ? (rank ? p.N / 2 + n0 : n0) : n0 + (int)rank * (BN / 2);
                for (int kb = 0; kb < nkb; ++kb, ++step) {
                    const int s = step % STAGES;
                    if (step >= STAGES && !tp_wait(empty + s, ((step / STAGES) - 1) & 1)) {
                        g_tp_status = 1;
                        *abort_s = 1;
                    }
                    if (*abort_s) break;
                    unsigned char* a = smem + s * STAGE_BYTES;
                    if (rank == 0) tp_expect_tx(full + s, 2 * STAGE_BYTES);
                    tp_tma_2d(a, &x_map, kb * TP_BK, m0, full + s);
                    tp_tma_2d(a + A_BYTES, &w_map, kb * TP_BK, w_row, full + s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // instruction descriptor: float32 accumulate, bfloat16 a and b, both K-major, N = BN, M = 256 (the pair)
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int step = 0, it = 0;
            for (int t = pair; t < total_tiles && !*abort_s; t += n_pairs, ++it) {
                const int buf = it % NBUF, use = it / NBUF;    // use: how often this buffer has been filled before
                if (use >= 1 && !tp_wait(acc_empty + buf, (use - 1) & 1)) {      // both epilogues have read it
                    g_tp_status = 1;
                    *abort_s = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t acc = tmem_base + buf * MB * BN;
                for (int kb = 0; kb < nkb; ++kb, ++step) {
                    const int s = step % STAGES;
                    if (!tp_wait(full + s, (step / STAGES) & 1)) {
                        g_tp_status = 1;
                        *abort_s = 1;
                    }
                    if (*abort_s) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a = tp_u32(smem + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
                    for (int k16 = 0; k16 < TP_BK / 16; ++k16) {
                        const uint64_t bd = tp_desc(b, k16);
#pragma unroll
                        for (int j = 0; j < MB; ++j)
                            tp_mma(acc + j * BN, tp_desc(a + j * A_BLOCK, k16), bd, idesc, (kb > 0 || k16 > 0) ? 1u : 0u);
                    }
                    tp_commit_both(empty + s);     // the stage is free in both blocks when these products have read it
                }
                tp_commit_both(acc_full + buf);    // and the accumulators are complete when all of them are done
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps 2 .. 2 + 4 MB - 1:
        // warp w drains tensor-memory lanes 32 (w % 4) .. of accumulator (w - 2) / 4: 32 rows of this block
        const int q = warp & 3, j = (warp - 2) >> 2;
        int it = 0;
        for (int t = pair; t < total_tiles; t += n_pairs, ++it) {
            const int buf = it % NBUF, use = it / NBUF;
            const int m0 = (t % m_tiles) * 2 * ROWS + (int)rank * ROWS + j * TP_BM, n0 = (t / m_tiles) * COLS;
            const int row = m0 + q * 32 + lane;
            bool ok = tp_wait(acc_full + buf, use & 1);
            if (!ok) {
                g_tp_status = 1;
                *abort_s = 1;
            }
            if (__any_sync(0xffffffffu, !ok || *abort_s != 0)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t taddr = tmem_base + (buf * MB + j) * BN + ((uint32_t)(q * 32) << 16);
            if (EPI == TP_SWIGLU) {
                const int I = p.N / 2;
                const bool wide = (I & 15) == 0;               // rows of out start on 32 bytes
#pragma unroll 1
                for (int c = 0; c < BN / 2; c += 32) {
                    uint32_t g[32], u[32];
                    tp_ld32(taddr + c, g);
                    tp_ld32(taddr + BN / 2 + c, u);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (row < p.M) {
                        bf16* dst = p.out + (size_t)row * I + n0 + c;
#pragma unroll
                        for (int i = 0; i < 32; i += 16) {
                            uint32_t pk[8];
#pragma unroll
                            for (int e = 0; e < 16; e += 2)
                                pk[e / 2] = tp_pack(tp_silu_mul(__uint_as_float(g[i + e]), __uint_as_float(u[i + e])),
                                                    tp_silu_mul(__uint_as_float(g[i + e + 1]), __uint_as_float(u[i + e + 1])));
                            if (wide && n0 + c + i + 16 <= I) {
                                tp_st32(dst + i, pk);
                            } else {
                                if (n0 + c + i < I) *reinterpret_cast<uint4*>(dst + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                                if (n0 + c + i + 8 < I) *reinterpret_cast<uint4*>(dst + i + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                            }
                        }
                    }
                }
            } else if (EPI == TP_RESIDUAL) {
                const bool wide = (p.N & 7) == 0;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t v[32];
                    tp_ld32(taddr + c, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (row < p.M) {
                        float* dst = p.resid + (size_t)row * p.N + n0 + c;
                        if (wide && n0 + c + 32 <= p.N) {
                            uint32_t r[4][8];
#pragma unroll
                            for (int i = 0; i < 4; ++i) tp_ld8(dst + i * 8, r[i]);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
#pragma unroll
                                for (int e = 0; e < 8; ++e) r[i][e] = __float_as_uint(__uint_as_float(r[i][e]) + __uint_as_float(v[i * 8 + e]));
                                tp_st32(dst + i * 8, r[i]);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                if (n0 + c + i < p.N) {
                                    float4 r = *reinterpret_cast<float4*>(dst + i);
                                    r.x += __uint_as_float(v[i]);
                                    r.y += __uint_as_float(v[i + 1]);
                                    r.z += __uint_as_float(v[i + 2]);
                                    r.w += __uint_as_float(v[i + 3]);
                                    *reinterpret_cast<float4*>(dst + i) = r;
                                }
                            }
                        }
                    }
                }
            } else {
                const bool wide = (p.N & 15) == 0;
#pragma unroll 1
                for (int c = 0; c < BN; c += 64) {
                    uint32_t v[64];
                    tp_ld32(taddr + c, *reinterpret_cast<uint32_t(*)[32]>(v));
                    tp_ld32(taddr + c + 32, *reinterpret_cast<uint32_t(*)[32]>(v + 32));
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (row < p.M) {
                        bf16* dst = p.out + (size_t)row * p.N + n0 + c;
#pragma unroll
                        for (int i = 0; i < 64; i += 16) {
                            uint32_t pk[8];
#pragma unroll
                            for (int e = 0; e < 16; e += 2) pk[e / 2] = tp_pack(__uint_as_float(v[i + e]), __uint_as_float(v[i + e + 1]));
                            if (wide && n0 + c + i + 16 <= p.N) {
                                tp_st32(dst + i, pk);
                            } else {
                                if (n0 + c + i < p.N) *reinterpret_cast<uint4*>(dst + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                                if (n0 + c + i + 8 < p.N) *reinterpret_cast<uint4*>(dst + i + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                            }
                        }
                    }
                }
            }
            // this warp has read its part of the buffer: the tile that uses it next may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tp_arrive_rank0(acc_empty + buf);
        }
    }
    // nobody leaves while its partner may still signal its barriers or read its shared memory
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    tp_cluster_sync();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*TpEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TpEncodeFn tp_encode_fn() {
    static TpEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) == cudaSuccess &&
            st == cudaDriverEntryPointSuccess)
            fn = (TpEncodeFn)p;
    }
    return fn;
}

// A tensor map over a row-major bfloat16 matrix [rows, K] (row stride ld elements) read in boxes of
// [box_rows rows, 64 elements] with the 128-byte swizzle; what lies outside the matrix reads as zero.
static int tp_make_map(CUtensorMap* map, const void* base, long long rows, int K, long long ld, int box_rows) {
    TpEncodeFn fn = tp_encode_fn();
    if (!fn) return -7;
    if (((uintptr_t)base & 15) != 0 || (ld * 2) % 16 != 0 || box_rows > 256) return PICO_ERR_ALIGN;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {TP_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -7;
}

static int tp_num_sms() { return pico_num_sms(); }

template <int BN, int EPI, int MB>
static int tp_launch(const void* x, int ldx, const void* w, const TpArgs& a, cudaStream_t stream) {
    constexpr int STAGE_BYTES = (MB * TP_BM + BN / 2) * TP_BK * 2;
    constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 8 ? 8 : (200 * 1024) / STAGE_BYTES;
    CUtensorMap xm, wm;
    int rc = tp_make_map(&xm, x, a.M, a.K, ldx, MB * TP_BM);
    if (rc) return rc;
    rc = tp_make_map(&wm, w, a.N, a.K, a.K, BN / 2);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16 + 1024;
    cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN, EPI, STAGES, MB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int n_out = EPI == TP_SWIGLU ? a.N / 2 : a.N;
    const int cols = EPI == TP_SWIGLU ? BN / 2 : BN;
    const int n_tiles = (n_out + cols - 1) / cols, m_tiles = (a.M + 2 * MB * TP_BM - 1) / (2 * MB * TP_BM);
    const int max_pairs = tp_num_sms() / 2;
    const int pairs = n_tiles * m_tiles < max_pairs ? n_tiles * m_tiles : max_pairs;
    pico_launch_cluster((gemm_tcgen05_pair_kernel<BN, EPI, STAGES, MB>), dim3(2 * pairs), dim3(64 + 128 * MB), smem, stream, 2,
                        xm, wm, a, m_tiles, n_tiles);
    return pico_launch_status();
}

// The tile (columns of w, and 256 or 512 rows of x per pair) that needs the least time: rounds of the
// pairs over the tiles times the work of a tile plus a fixed part; the tall form where it fills the pairs.
static void tp_pick(int M, int n_out, bool swiglu, int force_mb, int& bn_out, int& mb_out) {
    const int pairs = tp_num_sms() / 2;
    long long best_cost = -1;
    const int widths[3] = {256, 192, 128};
    for (int mb = 2; mb >= 1; --mb) {
        if (force_mb && mb != force_mb) continue;
        const int m_tiles = (M + 2 * mb * TP_BM - 1) / (2 * mb * TP_BM);
        for (int i = 0; i < 3; ++i) {
            const int bn = widths[i], cols = swiglu ? bn / 2 : bn;
            if (mb == 2 && bn != 256) continue;
            const long long tiles = (long long)m_tiles * ((n_out + cols - 1) / cols);
            // per tile: the products (a quarter cheaper per row in the tall form) plus a fixed part
            const long long cost = ((tiles + pairs - 1) / pairs) * (mb == 2 ? (long long)(bn * 3 / 2 + 40) : (long long)(bn + 16));
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                bn_out = bn;
                mb_out = mb;
            }
        }
    }
}

// epi: 0 = out[M, N] = x w^T (bfloat16); 1 = resid[M, N] (float32) += x w^T; 2 = out[M, N/2] =
// silu(x wg^T) * (x wu^T) with w = [wg; wu].  x: [M, K] bfloat16 with row stride ldx; w: [N, K] contiguous.
// rows_per_pair: 0 = chosen here, 256 or 512.
PICO_API int pico_gemm_tcgen05_pair(const void* x, int ldx, const void* w, void* out, float* resid, int M, int N, int K,
                                    int epi, int rows_per_pair, cudaStream_t stream) {
    if (M < 1 || N < 16 || K < 16 || K % 8 != 0 || ldx % 8 != 0) return PICO_ERR_SIZE;
    if (epi == TP_SWIGLU && (N % 2 != 0 || (N / 2) % 8 != 0)) return PICO_ERR_SIZE;
    if (epi != TP_SWIGLU && N % 8 != 0) return PICO_ERR_SIZE;
    if (rows_per_pair != 0 && rows_per_pair != 256 && rows_per_pair != 512) return PICO_ERR_SIZE;
    TpArgs a;
    a.M = M; a.N = N; a.K = K; a.out = (bf16*)out; a.resid = resid;
    int bn = 256, mb = 1;
    tp_pick(M, epi == TP_SWIGLU ? N / 2 : N, epi == TP_SWIGLU, rows_per_pair / 256, bn, mb);
#define TP_CASE(BN, MB)                                                                       \
    if (bn == BN && mb == MB) {                                                               \
        if (epi == TP_STORE) return tp_launch<BN, TP_STORE, MB>(x, ldx, w, a, stream);        \
        if (epi == TP_RESIDUAL) return tp_launch<BN, TP_RESIDUAL, MB>(x, ldx, w, a, stream);  \
        if (epi == TP_SWIGLU) return tp_launch<BN, TP_SWIGLU, MB>(x, ldx, w, a, stream);      \
    }
    TP_CASE(256, 2)
    TP_CASE(256, 1)
    TP_CASE(192, 1)
    TP_CASE(128, 1)
#undef TP_CASE
    return PICO_ERR_SIZE;
}

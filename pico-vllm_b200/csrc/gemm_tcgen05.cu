// Matrix products for many tokens (prefill) on the 5th-generation tensor cores:
// y[m, n] = sum_k x[m, k] w[n, k], bfloat16 in, float32 accumulate in tensor memory.
//
// One block computes a 128 x BN tile of y.  Roles by warp:
//   warp 0   one lane issues the TMA copies (cp.async.bulk.tensor.2d, 128-byte swizzle) of the
//            x tile [128 rows, 64 k] and the w tile [BN rows, 64 k] of every k-block into a ring
//            of shared-memory stages (full/empty mbarriers);
//   warp 1   allocates BN columns of tensor memory; one lane issues tcgen05.mma (M 128, N BN, K 16,
//            operands by shared-memory descriptors, accumulator in tensor memory) four times per
//            k-block and tcgen05.commit, which frees the stage when the products have read it and,
//            after the last k-block, tells the epilogue that the accumulator is complete;
//   warps 2-5  epilogue: each reads its 32 rows of the accumulator with tcgen05.ld, applies the
//            epilogue and stores.
// Epilogues: STORE (bfloat16), RESIDUAL (float32 x_res += y, in place), SWIGLU (the tile's first
// BN/2 columns are gate features n0.., the second BN/2 the same features' up rows: the w tile is
// two boxes, rows [n0, n0 + BN/2) and [I + n0, I + n0 + BN/2); out = silu(gate) * up, bfloat16).
//
// The reference runs these products as cuBLAS nn.Linear calls and a separate SwiGLU
// (pico_vllm/model.py:309-318); the formulas are the same (silu(g) = g * sigmoid(g),
// pico_vllm/kernels/swiglu.py:36-41).  Every mbarrier wait is bounded; a block that gives up sets
// the status word read by pico_tc_status and still frees its tensor memory.
#include <cuda.h>
#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_WAIT_LIMIT (1 << 18)

enum { TC_STORE = 0, TC_RESIDUAL = 1, TC_SWIGLU = 2 };

__device__ int g_tc_status = 0;
PICO_API int pico_tc_status(int* out) {
    return (int)cudaMemcpyFromSymbol(out, g_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost);
}

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tc_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < TC_WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(tc_smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tc_tma_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(tc_smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(tc_smem_u32(bar))
        : "memory");
}
// Shared-memory matrix descriptor of a K-major tile [rows][64 bf16] stored by TMA with the 128-byte
// swizzle: rows are 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset), version 1
// (Blackwell), layout type 2 (128-byte swizzle).  k16 selects the 16-element (32-byte) step inside the row.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t tile_addr, int k16) {
    const uint32_t addr = tile_addr + k16 * 32;
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);            // start address
    d |= (uint64_t)1 << 16;                           // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset
    d |= (uint64_t)1 << 46;                           // descriptor version
    d |= (uint64_t)2 << 61;                           // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;      // no output lane is disabled
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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

struct TcArgs {
    int M, N, K;              // N: rows of w (SWIGLU: 2 * I)
    bf16* out;                // STORE: [M, N]; SWIGLU: [M, N / 2]
    float* resid;             // RESIDUAL: [M, N]
};

// Blocks are persistent: block b computes tiles b, b + gridDim.x, ... (tile t = n-block t / m_tiles,
// m-block t % m_tiles, so that blocks running together share a w tile in L2).  The accumulator is
// double-buffered in tensor memory (2 x BN columns): the epilogue of one tile runs while the next
// tile's products are issued.
template <int BN, int EPI, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map, const TcArgs p,
                    int m_tiles, int n_tiles) {
    pdl_launch_dependents();
    extern __shared__ unsigned char tc_dyn[];
    unsigned char* smem = tc_dyn + ((1024u - (tc_smem_u32(tc_dyn) & 1023u)) & 1023u);
    constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int COLS = EPI == TC_SWIGLU ? BN / 2 : BN;       // output columns of a tile
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;                       // [2]: the products of a tile are done
    uint64_t* acc_empty = acc_full + 2;                        // [2]: the epilogue has read the buffer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (p.K + TC_BK - 1) / TC_BK;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc_mbar_init(full + s, 1);
            tc_mbar_init(empty + s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(acc_full + i, 1);
            tc_mbar_init(acc_empty + i, 4);                    // one arrival per epilogue warp
        }
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {       // tensor memory for two accumulators: 2 x BN columns of 128 lanes x 32 bits
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(tmem_slot)), "r"(2 * BN));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();            // x comes from the kernel before

    if (warp == 0) {
        if (lane == 0) {
            int step = 0;                                      // k-blocks issued so far, over all tiles
            for (int t = blockIdx.x; t < total_tiles && !*abort_s; t += gridDim.x) {
                const int m0 = (t % m_tiles) * TC_BM, n0 = (t / m_tiles) * COLS;
                for (int kb = 0; kb < nkb; ++kb, ++step) {
                    const int s = step % STAGES;
                    if (step >= STAGES && !tc_mbar_wait(empty + s, ((step / STAGES) - 1) & 1)) {
                        g_tc_status = 1;
                        *abort_s = 1;
                    }
                    if (*abort_s) break;
                    unsigned char* a = smem + s * STAGE_BYTES;
                    unsigned char* b = a + A_BYTES;
                    tc_mbar_expect_tx(full + s, STAGE_BYTES);
                    tc_tma_2d(a, &x_map, kb * TC_BK, m0, full + s);
                    if (EPI == TC_SWIGLU) {
                        tc_tma_2d(b, &w_map, kb * TC_BK, n0, full + s);
                        tc_tma_2d(b + B_BYTES / 2, &w_map, kb * TC_BK, p.N / 2 + n0, full + s);
                    } else {
                        tc_tma_2d(b, &w_map, kb * TC_BK, n0, full + s);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: float32 accumulate, bfloat16 a and b, both K-major, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            int step = 0, it = 0;
            for (int t = blockIdx.x; t < total_tiles && !*abort_s; t += gridDim.x, ++it) {
                const int buf = it & 1;
                if (it >= 2 && !tc_mbar_wait(acc_empty + buf, ((it >> 1) - 1) & 1)) {      // the epilogue has read it
                    g_tc_status = 1;
                    *abort_s = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t acc = tmem_base + buf * BN;
                for (int kb = 0; kb < nkb; ++kb, ++step) {
                    const int s = step % STAGES;
                    if (!tc_mbar_wait(full + s, (step / STAGES) & 1)) {
                        g_tc_status = 1;
                        *abort_s = 1;
                    }
                    if (*abort_s) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a = tc_smem_u32(smem + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
                    for (int k16 = 0; k16 < TC_BK / 16; ++k16)
                        tc_mma(acc, tc_smem_desc(a, k16), tc_smem_desc(b, k16), idesc, (kb > 0 || k16 > 0) ? 1u : 0u);
                    tc_commit(empty + s);      // the stage is free when these products have read it
                }
                tc_commit(acc_full + buf);     // and the accumulator is complete when all of them are done
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps 2..5
        const int q = warp & 3;                // the quarter of the 128 tensor-memory lanes this warp may read
        int it = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++it) {
            const int buf = it & 1;
            const int m0 = (t % m_tiles) * TC_BM, n0 = (t / m_tiles) * COLS;
            const int row = m0 + q * 32 + lane;
            if (!tc_mbar_wait(acc_full + buf, (it >> 1) & 1)) {
                g_tc_status = 1;
                *abort_s = 1;
            }
            if (*abort_s) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
            if (EPI == TC_SWIGLU) {
                const int I = p.N / 2;
#pragma unroll 1
                for (int c = 0; c < BN / 2; c += 32) {
                    uint32_t g[32], u[32];
                    tc_ld32(taddr + c, g);
                    tc_ld32(taddr + BN / 2 + c, u);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (row < p.M) {
                        bf16* dst = p.out + (size_t)row * I + n0 + c;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (n0 + c + j < I) {
                                uint4 pk;
                                uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                                for (int e = 0; e < 8; e += 2) {
                                    const float g0 = __uint_as_float(g[j + e]), g1 = __uint_as_float(g[j + e + 1]);
                                    const float a0 = g0 / (1.0f + expf(-g0)) * __uint_as_float(u[j + e]);
                                    const float a1 = g1 / (1.0f + expf(-g1)) * __uint_as_float(u[j + e + 1]);
                                    __nv_bfloat162 h = __floats2bfloat162_rn(a0, a1);
                                    pw[e / 2] = *reinterpret_cast<uint32_t*>(&h);
                                }
                                *reinterpret_cast<uint4*>(dst + j) = pk;
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t v[32];
                    tc_ld32(taddr + c, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (row < p.M) {
                        if (EPI == TC_RESIDUAL) {
                            float* dst = p.resid + (size_t)row * p.N + n0 + c;
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                if (n0 + c + j < p.N) {
                                    float4 r = *reinterpret_cast<float4*>(dst + j);
                                    r.x += __uint_as_float(v[j]);
                                    r.y += __uint_as_float(v[j + 1]);
                                    r.z += __uint_as_float(v[j + 2]);
                                    r.w += __uint_as_float(v[j + 3]);
                                    *reinterpret_cast<float4*>(dst + j) = r;
                                }
                            }
                        } else {
                            bf16* dst = p.out + (size_t)row * p.N + n0 + c;
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                if (n0 + c + j < p.N) {
                                    uint4 pk;
                                    uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                                    for (int e = 0; e < 8; e += 2) {
                                        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[j + e]), __uint_as_float(v[j + e + 1]));
                                        pw[e / 2] = *reinterpret_cast<uint32_t*>(&h);
                                    }
                                    *reinterpret_cast<uint4*>(dst + j) = pk;
                                }
                            }
                        }
                    }
                }
            }
            // this warp has read its part of the buffer: the next tile but one may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(acc_empty + buf)) : "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * BN));
    }
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*TcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TcEncodeFn tc_encode_fn() {
    static TcEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) == cudaSuccess &&
            st == cudaDriverEntryPointSuccess)
            fn = (TcEncodeFn)p;
    }
    return fn;
}

// A tensor map over a row-major bfloat16 matrix [rows, K] (row stride ld elements) read in boxes of
// [box_rows rows, 64 elements] with the 128-byte swizzle; what lies outside the matrix reads as zero.
static int tc_make_map(CUtensorMap* map, const void* base, long long rows, int K, long long ld, int box_rows) {
    TcEncodeFn fn = tc_encode_fn();
    if (!fn) return -7;
    if (((uintptr_t)base & 15) != 0 || (ld * 2) % 16 != 0 || box_rows > 256) return PICO_ERR_ALIGN;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -7;
}

template <int BN, int EPI>
static int tc_launch(const void* x, int ldx, const void* w, const TcArgs& a, cudaStream_t stream) {
    constexpr int STAGES = BN == 256 ? 4 : 6;
    CUtensorMap xm, wm;
    int rc = tc_make_map(&xm, x, a.M, a.K, ldx, TC_BM);
    if (rc) return rc;
    rc = tc_make_map(&wm, w, a.N, a.K, a.K, EPI == TC_SWIGLU ? BN / 2 : BN);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * (TC_BM + BN) * TC_BK * 2 + (2 * STAGES + 4) * 8 + 16 + 1024;
    cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int n_out = EPI == TC_SWIGLU ? a.N / 2 : a.N;
    const int cols = EPI == TC_SWIGLU ? BN / 2 : BN;
    const int n_tiles = (n_out + cols - 1) / cols, m_tiles = (a.M + TC_BM - 1) / TC_BM;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const int grid = n_tiles * m_tiles < sms ? n_tiles * m_tiles : sms;
    pico_launch((gemm_tcgen05_kernel<BN, EPI, STAGES>), dim3(grid), dim3(TC_THREADS), smem, stream, xm, wm, a, m_tiles,
                n_tiles);
    return pico_launch_status();
}

// epi: 0 = out[M, N] = x w^T (bfloat16); 1 = resid[M, N] (float32) += x w^T; 2 = out[M, N/2] =
// silu(x wg^T) * (x wu^T) with w = [wg; wu].  x: [M, K] bfloat16 with row stride ldx; w: [N, K] contiguous.
PICO_API int pico_gemm_tcgen05(const void* x, int ldx, const void* w, void* out, float* resid, int M, int N, int K,
                               int epi, cudaStream_t stream) {
    if (M < 1 || N < 16 || K < 16 || K % 8 != 0 || ldx % 8 != 0) return PICO_ERR_SIZE;
    if (epi == TC_SWIGLU && (N % 2 != 0 || (N / 2) % 8 != 0)) return PICO_ERR_SIZE;
    if (epi != TC_SWIGLU && N % 8 != 0) return PICO_ERR_SIZE;
    TcArgs a;
    a.M = M; a.N = N; a.K = K; a.out = (bf16*)out; a.resid = resid;
    if (epi == TC_STORE) return tc_launch<256, TC_STORE>(x, ldx, w, a, stream);
    if (epi == TC_RESIDUAL) return tc_launch<256, TC_RESIDUAL>(x, ldx, w, a, stream);
    if (epi == TC_SWIGLU) return tc_launch<256, TC_SWIGLU>(x, ldx, w, a, stream);
    return PICO_ERR_SIZE;
}

// Matrix products for a handful of tokens (decode): y[m, n] = sum_k x[m, k] w[n, k], bfloat16 in,
// float32 accumulate, for M <= 16 tokens.  At this size the product is a stream of the weight
// matrix from HBM, so the kernel is built around that stream: one block owns 16 output features
// for ALL tokens over the WHOLE of K (no split-K, hence no second pass and a fixed summation
// order), its 4 warps take alternate 64-wide slices of K, weights and activations come in through
// a deep cp.async pipeline (8 KB of weights per stage; 8 stages with two blocks per SM, or 16
// stages with one block per SM when there are few tiles), the products run on tensor cores with
// the weights as the 16-row operand (mma.sync m16n8k16: rows = output features, columns = tokens),
// and the four warps' sums are added in shared memory.  Blocks are persistent: a block walks tiles
// blockIdx.x, blockIdx.x + gridDim.x, ... and its pipeline runs on across tile boundaries, so the
// weight stream never drains.  The 16 features of a tile are two runs of 8 consecutive rows of w,
// which lets the epilogue see pairs that belong together:
//
//   STORE     y = (sum + bias) as bfloat16 or float32                       (plain projection, head)
//   RESIDUAL  x_res[m, n] += sum, float32 in place                          (o_proj, down_proj)
//   SWIGLU    a[m, i] = silu(gate_i) * up_i; rows i (gate) and I + i (up)   (gate_up, no 2I buffer)
//   ROPE      q/k heads: rows d and d + hd/2 of a head: bias, rotation by the token's position,
//             q to the query buffer, k and v straight into their cache pages   (qkv projection)
//   ARGMAX    token[m] = the first n with the largest sum: every block keeps the best of its own tiles, the
//             block that finishes last picks among the blocks' bests (greedy head: the [M, N] logits are
//             never written; the reference computes them all and calls argmax, pico_vllm/model.py:445,
//             pico_vllm/sampler.py:3-8)
//
// The reference runs these as cuBLAS nn.Linear calls followed by separate kernels
// (pico_vllm/model.py:200-225, 290-295, 326-332; pico_vllm/kernels/swiglu.py,
// pico_vllm/kernels/fused_rope_kvcache_store.py); the formulas are the same: silu(g) = g * sigmoid(g)
// (swiglu.py:36-41), x1' = x1 c - x2 s, x2' = x2 c + x1 s with angle = position * theta^(-2i/hd)
// (fused_rope_kvcache_store.py:60-65; model.py:80-86), cache row = page * page_size + offset
// (store_kvcache.py:24-50).
#include "common.cuh"

#ifndef SG_WARPS
#define SG_WARPS 8           // warps per block; each takes every SG_WARPS-th 64-wide slice of K
#endif
#define SG_THREADS (32 * SG_WARPS)
#define SG_KW 64               // K per pipeline step of one warp
#define SG_LD (SG_KW + 8)      // padded row of a stage in shared memory (elements): 144 bytes, conflict-free ldmatrix

#ifndef SG_ST_XPRE
#define SG_ST_XPRE 4           // pipeline depth when the activations sit in shared memory
#endif
#ifndef SG_ST_STREAM
#define SG_ST_STREAM 4         // ... when they are streamed beside the weights
#endif
#ifndef SG_ST_DEEP
#define SG_ST_DEEP 8          // ... when there are fewer tiles than SMs (one block per SM)
#endif
#define SG_NORM_CACHE 12       // float4 per lane of a row kept in registers by the norm prologue (rows up to 1536 wide)
#ifndef SG_CTAS_PER_SM
#define SG_CTAS_PER_SM 2
#endif

enum { SG_STORE = 0, SG_RESIDUAL = 1, SG_SWIGLU = 2, SG_ROPE = 3, SG_ARGMAX = 4 };

// ARGMAX: what each block found, and how many blocks have reported (reset by the block that reports last, so
// launches on one stream need no clearing in between; launches that overlap on the GPU would mix their entries)
#define SG_ARGMAX_MAX_GRID 1024
__device__ float g_sg_best_v[SG_ARGMAX_MAX_GRID * 16];
__device__ int g_sg_best_i[SG_ARGMAX_MAX_GRID * 16];
__device__ unsigned int g_sg_reported = 0;

struct SkinnyArgs {
    const bf16* w;            // [N, K]
    const bf16* x;            // [M, K] (row stride ldx)
    int ldx;
    // or, instead of x: the float32 residual stream, to be RMS-normed on the way in (needs the
    // activations-in-shared-memory mode): x[m, :] = xf[rows ? rows[m] : m, :] * rsqrt(mean(xf^2) + eps) * norm_w
    const float* xf;          // [*, K]
    const float* norm_w;      // [K]
    const int* x_rows;        // [M] or null
    float eps;
    int M, N, K;
    // STORE
    void* out;                // [M, ld_out] bf16 or float32
    int ld_out;
    int out_f32;
    const float* bias;        // [N] or null (STORE and ROPE)
    // RESIDUAL
    float* resid;             // [M, N]
    // SWIGLU: N = 2 * I; out = [M, I] bf16 in `out`
    // ROPE
    int nh, nkv, hd, rot_half, page_size;
    const int* positions;     // [M]
    const int* slots;         // [M] or null
    const float* inv_freq;    // [rot_half]
    bf16* q_out;              // [M, nh * hd]
    bf16* k_pages;
    bf16* v_pages;
    // ARGMAX
    int* tokens;              // [M]
};

__device__ __forceinline__ uint32_t sg_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sg_cp16(uint32_t dst, const void* src, bool pred) {
    const int n = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void sg_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void sg_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void sg_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sg_ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void sg_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The two runs of 8 weight rows a block owns.
template <int EPI>
__device__ __forceinline__ void sg_rows(const SkinnyArgs& p, int tile, int& row_a, int& row_b) {
    if (EPI == SG_SWIGLU) {
        row_a = tile * 8;                  // gate rows
        row_b = p.N / 2 + tile * 8;        // the same features' up rows
    } else if (EPI == SG_ROPE) {
        const int per_head = p.hd / 16;    // tiles per head
        const int rot_heads = p.nh + p.nkv;
        const int head = tile / per_head, j = tile - head * per_head;
        if (head < rot_heads) {            // q or k head: dims 8j.. and hd/2 + 8j..
            row_a = head * p.hd + j * 8;
            row_b = row_a + p.hd / 2;
        } else {                           // v head: 16 consecutive dims
            row_a = head * p.hd + j * 16;
            row_b = row_a + 8;
        }
    } else {
        row_a = tile * 16;
        row_b = row_a + 8;
    }
}

template <int XR>
__device__ __forceinline__ float sg_sum(const float* red, int f, int t) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < SG_WARPS; ++w) v += red[(w * 16 + f) * XR + t];
    return v;
}

template <int MT, int EPI>
__device__ __forceinline__ void sg_epilogue(const SkinnyArgs& p, const float* red, int row_a, int row_b, float* best_v,
                                            int* best_i) {
    constexpr int XR = MT * 8;
    if (EPI == SG_ARGMAX) {
        // one thread per token: the tile's 16 features in rising order of n, so that the first of equals wins
        const int t = threadIdx.x;
        if (t < p.M) {
            float bv = best_v[t];
            int bi = best_i[t];
#pragma unroll
            for (int f = 0; f < 16; ++f) {
                const float v = sg_sum<XR>(red, f, t);
                const int n = (f < 8 ? row_a + f : row_b + f - 8);
                if (v > bv || (v == bv && n < bi)) { bv = v; bi = n; }
            }
            best_v[t] = bv;
            best_i[t] = bi;
        }
    } else if (EPI == SG_STORE || EPI == SG_RESIDUAL) {
        for (int idx = threadIdx.x; idx < 16 * XR; idx += SG_THREADS) {
            const int t = idx / 16, f = idx - t * 16;          // consecutive threads: consecutive features
            if (t >= p.M) continue;
            const float v = sg_sum<XR>(red, f, t);
            const int n = (f < 8 ? row_a + f : row_b + f - 8);
            if (EPI == SG_RESIDUAL) {
                p.resid[(size_t)t * p.N + n] += v;
            } else {
                const float y = v + (p.bias ? p.bias[n] : 0.f);
                if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)t * p.ld_out + n] = y;
                else reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ld_out + n] = __float2bfloat16_rn(y);
            }
        }
    } else if (EPI == SG_SWIGLU) {
        for (int idx = threadIdx.x; idx < 8 * XR; idx += SG_THREADS) {
            const int t = idx / 8, f = idx - t * 8;
            if (t >= p.M) continue;
            const float gte = sg_sum<XR>(red, f, t);
            const int fu = f + 8;
            const float up = sg_sum<XR>(red, fu, t);
            const float sl = gte / (1.0f + expf(-gte));
            reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ld_out + row_a + f] = __float2bfloat16_rn(sl * up);
        }
    } else {    // SG_ROPE
        const int rot_heads = p.nh + p.nkv;
        const int head = row_a / p.hd;
        if (head < rot_heads) {
            const int d0 = row_a - head * p.hd;                 // first dim of the lower half (8j)
            for (int idx = threadIdx.x; idx < 8 * XR; idx += SG_THREADS) {
                const int t = idx / 8, f = idx - t * 8;
                if (t >= p.M) continue;
                float x1 = sg_sum<XR>(red, f, t);
                const int fu = f + 8;
                float x2 = sg_sum<XR>(red, fu, t);
                if (p.bias) { x1 += p.bias[row_a + f]; x2 += p.bias[row_b + f]; }
                float y1 = x1, y2 = x2;
                const int i = d0 + f;                           // pair index
                if (i < p.rot_half) {
                    float s, c;
                    sincosf((float)p.positions[t] * p.inv_freq[i], &s, &c);
                    y1 = x1 * c - x2 * s;
                    y2 = x2 * c + x1 * s;
                }
                if (head < p.nh) {
                    bf16* dst = p.q_out + (size_t)t * p.nh * p.hd + row_a + f;
                    dst[0] = __float2bfloat16_rn(y1);
                    dst[p.hd / 2] = __float2bfloat16_rn(y2);
                } else if (p.slots && p.slots[t] >= 0) {
                    const int slot = p.slots[t], kh = head - p.nh;
                    bf16* dst = p.k_pages + (((size_t)(slot / p.page_size) * p.nkv + kh) * p.page_size + slot % p.page_size) * p.hd + i;
                    dst[0] = __float2bfloat16_rn(y1);
                    dst[p.hd / 2] = __float2bfloat16_rn(y2);
                }
            }
        } else {
            const int kh = head - rot_heads;
            const int d0 = row_a - head * p.hd;
            for (int idx = threadIdx.x; idx < 16 * XR; idx += SG_THREADS) {
                const int t = idx / 16, f = idx - t * 16;
                if (t >= p.M || !p.slots || p.slots[t] < 0) continue;
                float v = sg_sum<XR>(red, f, t);
                if (p.bias) v += p.bias[row_a + f];
                const int slot = p.slots[t];
                p.v_pages[(((size_t)(slot / p.page_size) * p.nkv + kh) * p.page_size + slot % p.page_size) * p.hd + d0 + f] =
                    __float2bfloat16_rn(v);
            }
        }
    }
}

// XPRE: the activations of all of K are put into shared memory once per block (they are the same
// for every tile); otherwise each warp streams its slices of them beside the weights.
template <int MT, int EPI, int STAGES, bool XPRE>     // MT: tokens padded to 8 * MT
__global__ void __launch_bounds__(SG_THREADS) skinny_gemm_kernel(const SkinnyArgs p, int n_tiles, int x_ld) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char sg_smem[];
    constexpr int XR = MT * 8;                               // token rows
    constexpr int STAGE_ROWS = XPRE ? 16 : 16 + XR;
    constexpr int STAGE_ELEMS = STAGE_ROWS * SG_LD;          // one warp's stage: rows of 64 + 8 elements
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    bf16* ring = reinterpret_cast<bf16*>(sg_smem) + (size_t)warp * STAGES * STAGE_ELEMS;
    bf16* x_all = reinterpret_cast<bf16*>(sg_smem) + (size_t)SG_WARPS * STAGES * STAGE_ELEMS;     // XPRE: [XR][x_ld]
    float* red = reinterpret_cast<float*>(x_all + (XPRE ? (size_t)XR * x_ld : 0));          // [warps][16][XR]
    float* best_v = red + SG_WARPS * 16 * XR;                                                // ARGMAX: [XR], [XR]
    int* best_i = reinterpret_cast<int*>(best_v + XR);
    if (EPI == SG_ARGMAX && threadIdx.x < XR) {
        best_v[threadIdx.x] = -INFINITY;
        best_i[threadIdx.x] = 0x7fffffff;
    }
    const int nk64 = (p.K + SG_KW - 1) / SG_KW;
    const int nkw = nk64 > warp ? (nk64 - warp + SG_WARPS - 1) / SG_WARPS : 0;     // 64-wide slices of K this warp takes per tile
    const int my_tiles = (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_tiles * nkw;                            // this warp's pipeline steps

    // one pipeline step of this warp: 16 weight rows x 64 k (and, when they are streamed, the
    // activations of the same k) into the step's stage
    auto load_step = [&](int it, bool weights, bool acts) {
        const int li = it / nkw, j = it - li * nkw;
        bf16* ws = ring + (it % STAGES) * STAGE_ELEMS;
        const int k0 = (warp + SG_WARPS * j) * SG_KW;
        if (weights) {
            int ra, rb;
            sg_rows<EPI>(p, blockIdx.x + li * gridDim.x, ra, rb);
#pragma unroll
            for (int q = 0; q < 4; ++q) {                        // 16 rows x 8 chunks of 16 bytes
                const int idx = lane + 32 * q;
                const int r = idx >> 3, c = idx & 7;
                const int k = k0 + c * 8;
                const int row = (r < 8 ? ra + r : rb + r - 8);
                const bool ok = k < p.K;
                sg_cp16(sg_smem_u32(ws + r * SG_LD + c * 8), p.w + (size_t)row * p.K + (ok ? k : 0), ok);
            }
        }
        if (!XPRE && acts) {
            bf16* xs = ws + 16 * SG_LD;
#pragma unroll
            for (int q = 0; q < MT * 2; ++q) {                   // XR rows x 8 chunks
                const int idx = lane + 32 * q;
                const int r = idx >> 3, c = idx & 7;
                const int k = k0 + c * 8;
                const bool ok = k < p.K && r < p.M;
                sg_cp16(sg_smem_u32(xs + r * SG_LD + c * 8), p.x + (size_t)(ok ? r : 0) * p.ldx + (ok ? k : 0), ok);
            }
        }
    };

    if (XPRE) {
        // the weights do not depend on the kernel before this one: their stream starts at once,
        // and only then does the block wait for that kernel's output, the activations
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < total) load_step(s, true, false);
            sg_commit();
        }
        // the norm weights do not depend on the kernel before either: a lane's share of them (K up to
        // SG_NORM_CACHE * 128) is in registers before the wait
        float4 nw[SG_NORM_CACHE];
        const bool cached = p.xf != nullptr && p.K <= SG_NORM_CACHE * 128 && p.K % 4 == 0;
        if (cached) {
#pragma unroll
            for (int i = 0; i < SG_NORM_CACHE; ++i) {
                const int k = lane * 4 + i * 128;
                nw[i] = k < p.K ? *reinterpret_cast<const float4*>(p.norm_w + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        pdl_wait();
        if (p.xf) {
            // RMS norm of the residual stream on the way in, float32, one warp per token row
            // (y = x * rsqrt(mean(x^2) + eps) * w, pico_vllm/RMSNorm.py:22-34)
            const int kpad = nk64 * SG_KW;
            for (int r = warp; r < XR; r += SG_WARPS) {
                bf16* dst = x_all + r * x_ld;
                if (r >= p.M) {
                    for (int k = lane * 2; k < kpad; k += 64) *reinterpret_cast<uint32_t*>(dst + k) = 0u;
                    continue;
                }
                const float* src = p.xf + (size_t)(p.x_rows ? p.x_rows[r] : r) * p.K;
                if (cached) {
                    // one pass: the row is read once into registers, summed, scaled and stored
                    float4 xv[SG_NORM_CACHE];
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < SG_NORM_CACHE; ++i) {
                        const int k = lane * 4 + i * 128;
                        xv[i] = k < p.K ? *reinterpret_cast<const float4*>(src + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int i = 0; i < SG_NORM_CACHE; ++i) ss += xv[i].x * xv[i].x + xv[i].y * xv[i].y + xv[i].z * xv[i].z + xv[i].w * xv[i].w;
                    ss = warp_sum(ss);
                    const float inv = 1.0f / sqrtf(ss / (float)p.K + p.eps);
#pragma unroll
                    for (int i = 0; i < SG_NORM_CACHE; ++i) {
                        const int k = lane * 4 + i * 128;
                        if (k < kpad) {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(xv[i].x * inv * nw[i].x, xv[i].y * inv * nw[i].y);
                            __nv_bfloat162 hi = __floats2bfloat162_rn(xv[i].z * inv * nw[i].z, xv[i].w * inv * nw[i].w);
                            uint2 pk;
                            pk.x = *reinterpret_cast<uint32_t*>(&lo);
                            pk.y = *reinterpret_cast<uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(dst + k) = pk;
                        }
                    }
                    continue;
                }
                float ss = 0.f;
                for (int k = lane * 4; k < p.K; k += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(src + k);
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / (float)p.K + p.eps);
                for (int k = lane * 4; k < kpad; k += 128) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f), w = v;
                    if (k < p.K) {
                        v = *reinterpret_cast<const float4*>(src + k);
                        w = *reinterpret_cast<const float4*>(p.norm_w + k);
                    }
                    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * inv * w.x, v.y * inv * w.y);
                    __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * inv * w.z, v.w * inv * w.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<uint32_t*>(&lo);
                    pk.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst + k) = pk;
                }
            }
        } else {
            const int chunks = (nk64 * SG_KW) >> 3;              // per row, K rounded up to 64
            for (int idx = threadIdx.x; idx < XR * chunks; idx += SG_THREADS) {
                const int r = idx / chunks, c = idx - r * chunks;
                const int k = c * 8;
                const bool ok = k < p.K && r < p.M;
                sg_cp16(sg_smem_u32(x_all + r * x_ld + k), p.x + (size_t)(ok ? r : 0) * p.ldx + (ok ? k : 0), ok);
            }
        }
        sg_commit();
        sg_wait<0>();            // once per block: the activations (and the first weight stages) have landed
        __syncthreads();
    } else {
        // the same here: the weights of the first stages are asked for before the wait, the
        // activations that go with them after it
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s)
            if (s < total) load_step(s, true, false);
        pdl_wait();
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < total) load_step(s, false, true);
            sg_commit();
        }
    }
    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_row = lane & 7, b_col = ((lane >> 3) & 1) * 8;
    int it = 0;
    for (int li = 0; li < my_tiles; ++li) {
        for (int j = 0; j < nkw; ++j, ++it) {
            sg_wait<STAGES - 2>();
            __syncwarp();
            if (it + STAGES - 1 < total) load_step(it + STAGES - 1, true, true);
            sg_commit();
            const bf16* ws = ring + (it % STAGES) * STAGE_ELEMS;
            const bf16* xs = XPRE ? x_all + (warp + SG_WARPS * j) * SG_KW : ws + 16 * SG_LD;
            const int xld = XPRE ? x_ld : SG_LD;
#pragma unroll
            for (int ks = 0; ks < SG_KW; ks += 16) {
                uint32_t a[4];
                sg_ldmatrix_x4(a, sg_smem_u32(ws + a_row * SG_LD + ks + a_col));
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    uint32_t b[2];
                    sg_ldmatrix_x2(b, sg_smem_u32(xs + (nt * 8 + b_row) * xld + ks + b_col));
                    sg_mma(acc[nt], a, b[0], b[1]);
                }
            }
        }
        // the tile is complete: add the four warps' sums (red[warp][feature 0..15][token 0..XR-1])
        int row_a, row_b;
        sg_rows<EPI>(p, blockIdx.x + li * gridDim.x, row_a, row_b);
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int f = (lane >> 2) + (e >> 1) * 8;
                const int t = nt * 8 + (lane & 3) * 2 + (e & 1);
                red[(warp * 16 + f) * XR + t] = acc[nt][e];
                acc[nt][e] = 0.f;
            }
        }
        __syncthreads();
        sg_epilogue<MT, EPI>(p, red, row_a, row_b, best_v, best_i);
        __syncthreads();         // red is written again at the end of the next tile
    }
    sg_wait<0>();
    if (EPI == SG_ARGMAX) {
        // this block's bests go to its row of the global table; the block that reports last reads all rows
        __shared__ unsigned int ticket;
        if (threadIdx.x < XR) {
            g_sg_best_v[blockIdx.x * 16 + threadIdx.x] = best_v[threadIdx.x];
            g_sg_best_i[blockIdx.x * 16 + threadIdx.x] = best_i[threadIdx.x];
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) ticket = atomicAdd(&g_sg_reported, 1u);
        __syncthreads();
        if (ticket == gridDim.x - 1) {
            __threadfence();
            // a warp per token: lanes take blocks lane, lane + 32, ...; the smaller index wins among equals
            for (int t = warp; t < p.M; t += SG_WARPS) {
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                for (int b = lane; b < (int)gridDim.x; b += 32) {
                    const float v = __ldcg(&g_sg_best_v[b * 16 + t]);
                    const int n = __ldcg(&g_sg_best_i[b * 16 + t]);
                    if (v > bv || (v == bv && n < bi)) { bv = v; bi = n; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float v = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int n = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (v > bv || (v == bv && n < bi)) { bv = v; bi = n; }
                }
                if (lane == 0) p.tokens[t] = bi == 0x7fffffff ? 0 : bi;
            }
            if (threadIdx.x == 0) g_sg_reported = 0;
        }
    }
}

// Do the activations of all of K fit in shared memory beside the weight rings (two blocks per SM)?
static bool sg_xpre(int mt, int K) { return (size_t)mt * 8 * (K + 72) * sizeof(bf16) <= (mt == 1 ? 34 : 52) * 1024; }

static int sg_num_sms() { return pico_num_sms(); }

template <int MT, int EPI, int STAGES, bool XPRE>
static void sg_launch_one(const SkinnyArgs& a, int tiles, int grid, cudaStream_t stream) {
    const int x_ld = ((a.K + SG_KW - 1) / SG_KW) * SG_KW + 8;
    const size_t smem = (size_t)SG_WARPS * STAGES * (XPRE ? 16 : 16 + MT * 8) * SG_LD * sizeof(bf16) +
                        (XPRE ? (size_t)MT * 8 * x_ld * sizeof(bf16) : 0) + (size_t)SG_WARPS * 16 * MT * 8 * sizeof(float) +
                        (EPI == SG_ARGMAX ? (size_t)2 * MT * 8 * sizeof(float) : 0);
    cudaFuncSetAttribute(skinny_gemm_kernel<MT, EPI, STAGES, XPRE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pico_launch((skinny_gemm_kernel<MT, EPI, STAGES, XPRE>), dim3(grid), dim3(SG_THREADS), smem, stream, a, tiles, x_ld);
}

template <int EPI>
static int sg_launch(const SkinnyArgs& a, int tiles, cudaStream_t stream) {
    const int mt = (a.M + 7) / 8;
    const int sms = sg_num_sms();
    // persistent blocks, SG_CTAS_PER_SM per SM
    int grid = tiles < SG_CTAS_PER_SM * sms ? tiles : SG_CTAS_PER_SM * sms;
    if (EPI == SG_ARGMAX && grid > SG_ARGMAX_MAX_GRID) grid = SG_ARGMAX_MAX_GRID;
    // the activations of all of K stay in shared memory when they fit beside the weight rings
    const bool xpre = sg_xpre(mt, a.K);
    if (a.xf && !xpre) return PICO_ERR_SIZE;
    // fewer tiles than SMs and a long K: one block per SM has to keep enough bytes in flight alone
    const bool deep = !xpre && tiles <= sms;
    if (mt == 1) {
        if (xpre) sg_launch_one<1, EPI, SG_ST_XPRE, true>(a, tiles, grid, stream);
        else if (deep) sg_launch_one<1, EPI, SG_ST_DEEP, false>(a, tiles, grid, stream);
        else sg_launch_one<1, EPI, SG_ST_STREAM, false>(a, tiles, grid, stream);
    } else if (mt == 2) {
        if (xpre) sg_launch_one<2, EPI, SG_ST_XPRE - 1, true>(a, tiles, grid, stream);
        else if (deep) sg_launch_one<2, EPI, SG_ST_DEEP * 3 / 4, false>(a, tiles, grid, stream);
        else sg_launch_one<2, EPI, SG_ST_STREAM * 3 / 4, false>(a, tiles, grid, stream);
    } else
        return PICO_ERR_SIZE;
    return pico_launch_status();
}

static int sg_check(int M, int N, int K, int ldx) {
    if (M < 1 || M > 16 || K < 16 || K % 16 != 0 || N < 16 || ldx % 8 != 0) return PICO_ERR_SIZE;
    return 0;
}

// Says whether the norm-on-the-way-in form takes these sizes (M tokens, inner size K).
PICO_API int pico_skinny_norm_fits(int M, int K) {
    return M >= 1 && M <= 16 && K % 16 == 0 && sg_xpre((M + 7) / 8, K) ? 1 : 0;
}

static void sg_set_x(SkinnyArgs& a, const void* x, int ldx, const float* norm_w, float eps, const int* x_rows) {
    if (norm_w) {            // x is the float32 residual stream
        a.xf = (const float*)x;
        a.norm_w = norm_w;
        a.eps = eps;
        a.x_rows = x_rows;
        a.x = nullptr;
        a.ldx = 8;
    } else {
        a.x = (const bf16*)x;
        a.ldx = ldx;
    }
}

// y = x w^T (+ bias): out [M, ld_out] bfloat16 (out_f32 = 0) or float32 (1).  N % 16 == 0.
// With norm_w: x is the float32 residual stream [*, K] (rows x_rows[m] or m) and is RMS-normed on the way in.
PICO_API int pico_skinny_linear(const void* x, int ldx, const void* w, const float* bias, void* out, int ld_out,
                                int out_f32, int M, int N, int K, const float* norm_w, float eps, const int* x_rows,
                                cudaStream_t stream) {
    if (sg_check(M, N, K, norm_w ? 8 : ldx) || N % 16 != 0) return PICO_ERR_SIZE;
    SkinnyArgs a = {};
    a.w = (const bf16*)w; sg_set_x(a, x, ldx, norm_w, eps, x_rows); a.M = M; a.N = N; a.K = K;
    a.out = out; a.ld_out = ld_out; a.out_f32 = out_f32; a.bias = bias;
    return sg_launch<SG_STORE>(a, N / 16, stream);
}

// resid[M, N] (float32) += x w^T.  N % 16 == 0.
PICO_API int pico_skinny_linear_residual(const void* x, int ldx, const void* w, float* resid, int M, int N, int K,
                                         cudaStream_t stream) {
    if (sg_check(M, N, K, ldx) || N % 16 != 0) return PICO_ERR_SIZE;
    SkinnyArgs a = {};
    a.w = (const bf16*)w; a.x = (const bf16*)x; a.ldx = ldx; a.M = M; a.N = N; a.K = K; a.resid = resid;
    return sg_launch<SG_RESIDUAL>(a, N / 16, stream);
}

// out[M, I] = silu(x wg^T) * (x wu^T) with w = [wg; wu] of shape [2I, K].  I % 8 == 0.
PICO_API int pico_skinny_gate_up_swiglu(const void* x, int ldx, const void* w, void* out, int M, int I, int K,
                                        const float* norm_w, float eps, cudaStream_t stream) {
    if (sg_check(M, 2 * I, K, norm_w ? 8 : ldx) || I % 8 != 0) return PICO_ERR_SIZE;
    SkinnyArgs a = {};
    a.w = (const bf16*)w; sg_set_x(a, x, ldx, norm_w, eps, nullptr); a.M = M; a.N = 2 * I; a.K = K;
    a.out = out; a.ld_out = I;
    return sg_launch<SG_SWIGLU>(a, I / 8, stream);
}

// qkv projection with bias, rotary encoding and cache store fused: q_out [M, nh*hd] gets the rotated
// queries, rotated keys and the values go to their cache rows (slots[m], -1 or null = no store).
// w: [(nh + 2 nkv) * hd, K], rows ordered q heads, k heads, v heads.  hd % 16 == 0.
PICO_API int pico_skinny_qkv_rope_store(const void* x, int ldx, const void* w, const float* bias, void* q_out,
                                        const int* positions, const float* inv_freq, int rot_dim, const int* slots,
                                        void* k_pages, void* v_pages, int M, int K, int nh, int nkv, int hd,
                                        int page_size, const float* norm_w, float eps, cudaStream_t stream) {
    const int N = (nh + 2 * nkv) * hd;
    if (sg_check(M, N, K, norm_w ? 8 : ldx) || hd % 16 != 0 || rot_dim % 2 != 0 || rot_dim > hd) return PICO_ERR_SIZE;
    SkinnyArgs a = {};
    a.w = (const bf16*)w; sg_set_x(a, x, ldx, norm_w, eps, nullptr); a.M = M; a.N = N; a.K = K; a.bias = bias;
    a.nh = nh; a.nkv = nkv; a.hd = hd; a.rot_half = rot_dim / 2; a.page_size = page_size;
    a.positions = positions; a.slots = slots; a.inv_freq = inv_freq;
    a.q_out = (bf16*)q_out; a.k_pages = (bf16*)k_pages; a.v_pages = (bf16*)v_pages;
    return sg_launch<SG_ROPE>(a, N / 16, stream);
}

// tokens[m] = the first n that maximises (x w^T)[m, n]: the greedy choice of the head without the logits.
// With norm_w: x is the float32 residual stream [*, K] (rows x_rows[m] or m), RMS-normed on the way in.  N % 16 == 0.
// Its launches must follow one another on one stream (they share the table of the blocks' bests).
PICO_API int pico_skinny_argmax(const void* x, int ldx, const void* w, int* tokens, int M, int N, int K, const float* norm_w,
                                float eps, const int* x_rows, cudaStream_t stream) {
    if (sg_check(M, N, K, norm_w ? 8 : ldx) || N % 16 != 0 || !tokens) return PICO_ERR_SIZE;
    SkinnyArgs a = {};
    a.w = (const bf16*)w; sg_set_x(a, x, ldx, norm_w, eps, x_rows); a.M = M; a.N = N; a.K = K; a.tokens = tokens;
    return sg_launch<SG_ARGMAX>(a, N / 16, stream);
}

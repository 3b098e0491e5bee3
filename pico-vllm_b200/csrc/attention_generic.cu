// Paged causal attention with grouped heads, for any head size that is a multiple of 16 up to
// 256, float32 or bfloat16 storage, float32 arithmetic.  One block per (query token, key/value
// head, split of the key range); each warp takes query heads of the group in turn, walks the
// visible keys 32 at a time (one key per lane for q.k, one head dimension per lane for p.v)
// with a running max and sum, and either writes the output or, with more than one split, a
// partial (max, sum, unnormalised output) that a second kernel combines.  This is the kernel
// of the 32-bit path and the fallback of the bfloat16 path.
//
// Restated from the reference: query head j uses key/value head j / g
// (pico_vllm/kernels/attention.py:31,139); scores scaled by hd^-1/2 (attention.py:92,231);
// key n is visible to the query at position p iff n <= p (attention.py:193-198); running
// max/sum softmax in float32 (attention.py:67-82, 189-213); pages found through the block table
// (attention.py:47-52, 172-176).  The window rule (only the last W keys) is the meaning of the
// architecture's sliding_window key; the reference has none.  Unlike the reference's prefill
// kernel, p is not rounded to the cache type before p.v, and keys beyond the query are never read.
#include "common.cuh"

#define ATT_MAX_DPL 8  // head dimensions per lane: hd <= 256

template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<bf16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int hd) {
    float acc = 0.f;
    for (int d = 0; d < hd; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + d);
        acc += q[d] * kv.x;
        acc += q[d + 1] * kv.y;
        acc += q[d + 2] * kv.z;
        acc += q[d + 3] * kv.w;
    }
    return acc;
}
template <>
__device__ __forceinline__ float dot_row<bf16>(const float* __restrict__ q, const bf16* __restrict__ k, int hd) {
    float acc = 0.f;
    for (int d = 0; d < hd; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p[j]);
            acc += q[d + 2 * j] * f.x;
            acc += q[d + 2 * j + 1] * f.y;
        }
    }
    return acc;
}

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    const int* __restrict__ tok_seg, const int* __restrict__ positions, const int* __restrict__ block_table,
    int table_stride, int nh, int nkv, int hd, int page_size, int window, float scale, int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float q_s[];  // [warps][hd]
    const int t = blockIdx.x, kh = blockIdx.y, sp = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int g = nh / nkv;
    const int seg = tok_seg[t];
    const int pos = positions[t];
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    // this split's part of [lo, hi), in whole tiles of 32 keys counted from lo
    const int ntiles = (hi - lo + 31) / 32;
    const int per = (ntiles + n_splits - 1) / n_splits;
    const int begin = lo + sp * per * 32;
    int end = begin + per * 32;
    if (end > hi) end = hi;
    const int* table = block_table + (size_t)seg * table_stride;
    float* qw = q_s + warp * hd;

    for (int hq = warp; hq < g; hq += nwarps) {
        const int h = kh * g + hq;
        const T* qp = q + (size_t)t * q_row_stride + (size_t)h * hd;
        __syncwarp();
        for (int d = lane; d < hd; d += 32) qw[d] = to_f32(qp[d]) * scale;
        __syncwarp();
        float m = -INFINITY, l = 0.f;
        float o[ATT_MAX_DPL];
#pragma unroll
        for (int j = 0; j < ATT_MAX_DPL; ++j) o[j] = 0.f;

        for (int n0 = begin; n0 < end; n0 += 32) {
            const int n = n0 + lane;
            const bool valid = n < end;
            long long row = 0;
            float s = -INFINITY;
            if (valid) {
                const int page = table[n / page_size];
                row = (((long long)page * nkv + kh) * page_size + (n % page_size)) * hd;
                s = dot_row<T>(qw, k_pages + row, hd);
            }
            const float m_new = fmaxf(m, warp_max(s));
            const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
            const float p = valid ? expf(s - m_new) : 0.f;
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int j = 0; j < ATT_MAX_DPL; ++j) o[j] *= corr;
            m = m_new;
            const int cnt = min(32, end - n0);
            for (int j = 0; j < cnt; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
                const long long rj = __shfl_sync(0xffffffffu, row, j);
                const T* vp = v_pages + rj;
#pragma unroll
                for (int jj = 0; jj < ATT_MAX_DPL; ++jj) {
                    const int d = lane + 32 * jj;
                    if (d < hd) o[jj] += pj * to_f32(vp[d]);
                }
            }
        }
        if (n_splits == 1) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            T* op = out + ((size_t)t * nh + h) * hd;
#pragma unroll
            for (int jj = 0; jj < ATT_MAX_DPL; ++jj) {
                const int d = lane + 32 * jj;
                if (d < hd) op[d] = from_f32<T>(o[jj] * inv);
            }
        } else {
            const size_t slot = ((size_t)t * nh + h) * n_splits + sp;
            float* po = part_o + slot * hd;
#pragma unroll
            for (int jj = 0; jj < ATT_MAX_DPL; ++jj) {
                const int d = lane + 32 * jj;
                if (d < hd) po[d] = o[jj];
            }
            if (lane == 0) {
                part_ml[slot * 2] = m;
                part_ml[slot * 2 + 1] = l;
            }
        }
    }
}

// out[t, h, :] = sum_i o_i exp(m_i - M) / sum_i l_i exp(m_i - M) over the splits i.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         T* __restrict__ out, int hd, int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t th = blockIdx.x;  // t * nh + h
    const float* ml = part_ml + th * n_splits * 2;
    float M = -INFINITY;
    for (int i = 0; i < n_splits; ++i) M = fmaxf(M, ml[2 * i]);
    float L = 0.f;
    for (int i = 0; i < n_splits; ++i) {
        const float mi = ml[2 * i];
        if (mi != -INFINITY) L += ml[2 * i + 1] * expf(mi - M);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < n_splits; ++i) {
            const float mi = ml[2 * i];
            if (mi != -INFINITY) acc += part_o[(th * n_splits + i) * hd + d] * expf(mi - M);
        }
        out[th * hd + d] = from_f32<T>(acc * inv);
    }
}

// q: rows of q_row_stride elements, head h at column h*hd.  out: [T, nh*hd].
// part_o: [T*nh*n_splits*hd] floats and part_ml: [T*nh*n_splits*2] floats of scratch, needed
// only when n_splits > 1.  block_table: [segments, table_stride] page numbers.
PICO_API int pico_paged_attention_generic(const void* q, int q_row_stride, const void* k_pages,
                                          const void* v_pages, void* out, float* part_o, float* part_ml,
                                          const int* tok_seg, const int* positions, const int* block_table,
                                          int table_stride, int T, int nh, int nkv, int hd, int page_size,
                                          int window, float scale, int n_splits, int act_dtype,
                                          cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd % 16 != 0 || hd < 16 || hd > 32 * ATT_MAX_DPL) return PICO_ERR_SIZE;
    if (nkv <= 0 || nh % nkv != 0 || n_splits < 1 || n_splits > 65535 || nkv > 65535) return PICO_ERR_SIZE;
    if (n_splits > 1 && (!part_o || !part_ml)) return PICO_ERR_SIZE;
    const int g = nh / nkv;
    const int warps = g < 4 ? g : 4;
    const dim3 grid(T, nkv, n_splits);
    const size_t smem = (size_t)warps * hd * sizeof(float);
    if (act_dtype == PICO_F32) {
        if ((q_row_stride % 4) != 0) return PICO_ERR_ALIGN;
        pico_launch((paged_attention_generic_kernel<float>), dim3(grid), dim3(warps * 32), smem, stream, 
            (const float*)q, q_row_stride, (const float*)k_pages, (const float*)v_pages, (float*)out, part_o,
            part_ml, tok_seg, positions, block_table, table_stride, nh, nkv, hd, page_size, window, scale, n_splits);
        if (n_splits > 1)
            pico_launch((attention_combine_kernel<float>), dim3(T * nh), dim3(64), 0, stream, part_o, part_ml, (float*)out, hd, n_splits);
    } else if (act_dtype == PICO_BF16) {
        pico_launch((paged_attention_generic_kernel<bf16>), dim3(grid), dim3(warps * 32), smem, stream, 
            (const bf16*)q, q_row_stride, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, part_o, part_ml,
            tok_seg, positions, block_table, table_stride, nh, nkv, hd, page_size, window, scale, n_splits);
        if (n_splits > 1)
            pico_launch((attention_combine_kernel<bf16>), dim3(T * nh), dim3(64), 0, stream, part_o, part_ml, (bf16*)out, hd, n_splits);
    } else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// ---------------------------------------------------------------------------------------------
// The entry point that allocates nothing (declared and documented in pico_noalloc.h; it has no
// counterpart in the reference).  Its scratch is this file-scope device array.  In host code the
// name g_noalloc_scratch is only a stand-in for the symbol, not a device address: the address
// the kernels get comes from cudaGetSymbolAddress, looked up once per device below.
#include "pico_noalloc.h"
#include <stdio.h>

#define PICO_ERR_SCRATCH (-5)
#define PICO_ERR_SYMBOL (-6)
#define PICO_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) float g_noalloc_scratch[PICO_NOALLOC_SCRATCH_FLOATS];
static float* g_noalloc_scratch_ptr[PICO_NOALLOC_MAX_DEVICES];   // device address, per device; 0 = not looked up

static int noalloc_fail(int code, char* err, int err_len, const char* msg) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, "pico_paged_attention_noalloc: %s", msg);
    return code;
}

PICO_API int pico_paged_attention_noalloc(const void* q, int q_row_stride, const void* k_pages,
                                          const void* v_pages, void* out, const int* tok_seg,
                                          const int* positions, const int* block_table, int table_stride,
                                          int T, int nh, int nkv, int hd, int page_size, int window, float scale,
                                          int n_splits, int act_dtype, cudaStream_t stream, char* err,
                                          int err_len) {
    if (err && err_len > 0) err[0] = 0;
    if (T <= 0) return 0;
    // the same limits as pico_paged_attention_generic, checked first so that the product below cannot wrap
    if (nh <= 0 || nkv <= 0 || nkv > 65535 || nh % nkv != 0 || hd % 16 != 0 || hd < 16 || hd > 32 * ATT_MAX_DPL ||
        n_splits < 1 || n_splits > 65535)
        return noalloc_fail(PICO_ERR_SIZE, err, err_len, "a size the attention kernels do not take");
    // one part per token needs no scratch at all: the kernel writes its result straight to out
    const long long need = n_splits == 1 ? 0 : (long long)T * nh * n_splits * (hd + 2);
    if (need > (long long)PICO_NOALLOC_SCRATCH_FLOATS) {
        char msg[200];
        snprintf(msg, sizeof msg,
                 "T*nh*n_splits*(hd+2) = %lld float32 of scratch wanted, the built-in array holds %d "
                 "(use fewer splits or tokens, or pico_paged_attention_generic with your own buffer)",
                 need, (int)PICO_NOALLOC_SCRATCH_FLOATS);
        return noalloc_fail(PICO_ERR_SCRATCH, err, err_len, msg);
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PICO_NOALLOC_MAX_DEVICES)
        return noalloc_fail(PICO_ERR_SYMBOL, err, err_len, "cannot tell the current device");
    if (!g_noalloc_scratch_ptr[dev]) {
        // set-up, once per device, with that device current
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            char msg[160];
            snprintf(msg, sizeof msg, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return noalloc_fail(PICO_ERR_SYMBOL, err, err_len, msg);
        }
        g_noalloc_scratch_ptr[dev] = p;
    }
    float* part_o = g_noalloc_scratch_ptr[dev];
    float* part_ml = part_o + (size_t)T * nh * n_splits * hd;
    const int rc = pico_paged_attention_generic(q, q_row_stride, k_pages, v_pages, out, part_o, part_ml, tok_seg,
                                                positions, block_table, table_stride, T, nh, nkv, hd, page_size,
                                                window, scale, n_splits, act_dtype, stream);
    if (rc == PICO_ERR_SIZE) return noalloc_fail(rc, err, err_len, "a size the attention kernels do not take");
    if (rc == PICO_ERR_DTYPE) return noalloc_fail(rc, err, err_len, "act_dtype must be 0 (float32) or 1 (bfloat16)");
    if (rc == PICO_ERR_ALIGN) return noalloc_fail(rc, err, err_len, "q_row_stride must be a multiple of 4 for float32");
    if (rc != 0) return noalloc_fail(rc, err, err_len, "kernel launch failed");
    return 0;
}

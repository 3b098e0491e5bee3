// Bias add + rotary position encoding of q and k + store of k and v into cache pages,
// one kernel.  The query part of the qkv buffer is rotated in place; k (rotated) and v
// go straight to their pages and are not written back to the buffer.
//
// Restated from the reference: rotation of the half-split pairs (d, d + hd/2),
// x1' = x1 c - x2 s, x2' = x2 c + x1 s (pico_vllm/model.py:116-124); angle = position *
// theta^(-2i/hd) (pico_vllm/model.py:80-86); cache row of a token = page * page_size +
// offset inside [pages, kv_heads, page_size, hd] (pico_vllm/kernels/store_kvcache.py:24-50);
// the fused decode form is pico_vllm/kernels/fused_rope_kvcache_store.py:5-163.  Unlike
// the reference, which rotates in bfloat16 from a bfloat16 table, angles, sines and the
// rotation are float32 here, and the bias is added in float32 before rotating.
#include "common.cuh"

template <typename TA>
__global__ void rope_store_kernel(TA* __restrict__ qkv, int row_stride, const float* __restrict__ bias,
                                  const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  const int* __restrict__ slots, TA* __restrict__ k_pages,
                                  TA* __restrict__ v_pages, int nh, int nkv, int hd, int rot_half,
                                  int page_size) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float cs[];  // cos[rot_half], sin[rot_half]
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < rot_half; i += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[rot_half + i] = s;
    }
    __syncthreads();
    TA* row = qkv + (size_t)t * row_stride;
    const int slot = slots ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    const int half = hd / 2;  // pairs are (d, d + hd/2); the first rot_half pairs are rotated
    const int n_rot_heads = nh + (slot >= 0 ? nkv : 0);
    for (int idx = threadIdx.x; idx < n_rot_heads * half; idx += blockDim.x) {
        const int head = idx / half, i = idx - head * half;
        const int c0 = head * hd + i, c1 = c0 + half;
        float x1 = to_f32(row[c0]), x2 = to_f32(row[c1]);
        if (bias) { x1 += bias[c0]; x2 += bias[c1]; }
        float y1 = x1, y2 = x2;
        if (i < rot_half) {
            const float c = cs[i], s = cs[rot_half + i];
            y1 = x1 * c - x2 * s;
            y2 = x2 * c + x1 * s;
        }
        if (head < nh) {
            row[c0] = from_f32<TA>(y1);
            row[c1] = from_f32<TA>(y2);
        } else {
            const int kh = head - nh;
            TA* dst = k_pages + (((size_t)page * nkv + kh) * page_size + off) * hd;
            dst[i] = from_f32<TA>(y1);
            dst[i + half] = from_f32<TA>(y2);
        }
    }
    if (slot >= 0) {
        const int v0 = (nh + nkv) * hd;
        for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
            const int kh = idx / hd, d = idx - kh * hd;
            float v = to_f32(row[v0 + idx]);
            if (bias) v += bias[v0 + idx];
            v_pages[(((size_t)page * nkv + kh) * page_size + off) * hd + d] = from_f32<TA>(v);
        }
    }
}

// The same for bfloat16 with 16-byte accesses: a thread takes 8 consecutive pairs (dims i..i+7 and
// i + hd/2 .. of one head) or 8 consecutive dims of a value head; a block takes `tpb` tokens (as many as
// give it about 256 threads' worth of work; one token with 160 threads at 12 + 2 heads of 128, which
// measured fastest of the block shapes tried).
// Needs hd % 16 == 0, rot_half % 8 == 0, row_stride % 8 == 0 and 16-byte aligned buffers.
#define ROPE_MAX_TPB 8
__device__ __forceinline__ void rope_unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 p = __bfloat1622float2(h[i]);
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
    }
}
__device__ __forceinline__ uint4 rope_pack8(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}
__device__ __forceinline__ void rope_add_bias8(const float* __restrict__ b, float (&f)[8]) {
    const float4 b0 = *reinterpret_cast<const float4*>(b), b1 = *reinterpret_cast<const float4*>(b + 4);
    f[0] += b0.x; f[1] += b0.y; f[2] += b0.z; f[3] += b0.w;
    f[4] += b1.x; f[5] += b1.y; f[6] += b1.z; f[7] += b1.w;
}

__global__ void __launch_bounds__(256)
rope_store_bf16x8_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ bias,
                         const int* __restrict__ positions, const float* __restrict__ inv_freq,
                         const int* __restrict__ slots, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, int T,
                         int nh, int nkv, int hd, int rot_half, int page_size, int tpb) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float cs[];  // [tpb][cos[rot_half], sin[rot_half]]
    const int t0 = blockIdx.x * tpb;
    for (int idx = threadIdx.x; idx < tpb * rot_half; idx += blockDim.x) {
        const int tt = idx / rot_half, i = idx - tt * rot_half;
        if (t0 + tt < T) {
            float s, c;
            sincosf((float)positions[t0 + tt] * inv_freq[i], &s, &c);
            cs[tt * 2 * rot_half + i] = c;
            cs[tt * 2 * rot_half + rot_half + i] = s;
        }
    }
    __syncthreads();
    const int half = hd / 2, gph = half / 8;               // groups of 8 pairs per head
    const int rot_items = (nh + nkv) * gph, v_items = nkv * (hd / 8), items = rot_items + v_items;
    for (int idx = threadIdx.x; idx < tpb * items; idx += blockDim.x) {
        const int tt = idx / items, w = idx - tt * items;
        const int t = t0 + tt;
        if (t >= T) break;
        bf16* row = qkv + (size_t)t * row_stride;
        const int slot = slots ? slots[t] : -1;
        const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
        if (w < rot_items) {
            const int head = w / gph, i = (w - head * gph) * 8;
            if (head >= nh && slot < 0) continue;            // keys of a token that is not stored
            const int c0 = head * hd + i, c1 = c0 + half;
            float x1[8], x2[8];
            rope_unpack8(*reinterpret_cast<const uint4*>(row + c0), x1);
            rope_unpack8(*reinterpret_cast<const uint4*>(row + c1), x2);
            if (bias) {
                rope_add_bias8(bias + c0, x1);
                rope_add_bias8(bias + c1, x2);
            }
            if (i < rot_half) {
                const float* cp = cs + tt * 2 * rot_half + i;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float c = cp[e], sn = cp[rot_half + e];
                    const float y1 = x1[e] * c - x2[e] * sn, y2 = x2[e] * c + x1[e] * sn;
                    x1[e] = y1;
                    x2[e] = y2;
                }
            }
            bf16* dst = head < nh ? row + c0 : k_pages + (((size_t)page * nkv + (head - nh)) * page_size + off) * hd + i;
            *reinterpret_cast<uint4*>(dst) = rope_pack8(x1);
            *reinterpret_cast<uint4*>(dst + half) = rope_pack8(x2);
        } else if (slot >= 0) {
            const int j = (w - rot_items) * 8;               // 8 dims of the value part
            const int kh = j / hd, d = j - kh * hd;
            const int c = (nh + nkv) * hd + j;
            float v[8];
            rope_unpack8(*reinterpret_cast<const uint4*>(row + c), v);
            if (bias) rope_add_bias8(bias + c, v);
            *reinterpret_cast<uint4*>(v_pages + (((size_t)page * nkv + kh) * page_size + off) * hd + d) = rope_pack8(v);
        }
    }
}

// qkv: [T, row_stride] with columns q heads, k heads, v heads.  slots may be null (a layer that
// reads another layer's cache rotates its queries only); a slot of -1 skips that token's store.
PICO_API int pico_rope_store(void* qkv, int row_stride, const float* bias, const int* positions,
                             const float* inv_freq, const int* slots, void* k_pages, void* v_pages, int T,
                             int nh, int nkv, int hd, int rot_dim, int page_size, int act_dtype,
                             cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd % 2 != 0 || rot_dim % 2 != 0 || rot_dim > hd || rot_dim < 0) return PICO_ERR_SIZE;
    const int rot_half = rot_dim / 2;
    const size_t smem = (size_t)2 * rot_half * sizeof(float);
    if (smem > 48 * 1024) return PICO_ERR_SIZE;
    const int work = (nh + nkv) * (hd / 2);
    const int threads = work >= 512 ? 256 : (work >= 128 ? 128 : 64);
    const bool vec = act_dtype == PICO_BF16 && hd % 16 == 0 && rot_half % 8 == 0 && row_stride % 8 == 0 &&
                     ((uintptr_t)qkv & 15) == 0 && (!bias || ((uintptr_t)bias & 15) == 0) &&
                     (!slots || (((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0)) &&
                     (size_t)ROPE_MAX_TPB * smem <= 48 * 1024;
    if (vec) {
        const int items = (nh + nkv) * (hd / 16) + nkv * (hd / 8);      // 16-byte pieces of work per token
        int tpb = 256 / items;
        tpb = tpb < 1 ? 1 : (tpb > ROPE_MAX_TPB ? ROPE_MAX_TPB : tpb);
        int vthreads = (tpb * items + 31) / 32 * 32;
        vthreads = vthreads > 256 ? 256 : vthreads;
        pico_launch(rope_store_bf16x8_kernel, dim3((T + tpb - 1) / tpb), dim3(vthreads), (size_t)tpb * smem, stream,
                    (bf16*)qkv, row_stride, bias, positions, inv_freq, slots, (bf16*)k_pages, (bf16*)v_pages, T, nh, nkv, hd,
                    rot_half, page_size, tpb);
    } else if (act_dtype == PICO_F32)
        pico_launch((rope_store_kernel<float>), dim3(T), dim3(threads), smem, stream, (float*)qkv, row_stride, bias, positions, inv_freq,
                                                               slots, (float*)k_pages, (float*)v_pages, nh, nkv, hd,
                                                               rot_half, page_size);
    else if (act_dtype == PICO_BF16)
        pico_launch((rope_store_kernel<bf16>), dim3(T), dim3(threads), smem, stream, (bf16*)qkv, row_stride, bias, positions, inv_freq,
                                                              slots, (bf16*)k_pages, (bf16*)v_pages, nh, nkv, hd,
                                                              rot_half, page_size);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

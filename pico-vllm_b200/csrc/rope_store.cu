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
    if (act_dtype == PICO_F32)
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

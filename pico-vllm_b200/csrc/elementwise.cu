// Embedding gather, residual-add + RMSNorm, SwiGLU.  Memory-bound row kernels; all
// arithmetic in float32, storage in the activation type (float or bfloat16).
//
// Formulas restated from the reference: embedding pico_vllm/model.py:405,427; RMSNorm
// y = x * rsqrt(mean(x^2)+eps) * w in float32, pico_vllm/RMSNorm.py:22-34; the residual
// add fused before the norm as in pico_vllm/kernels/fused_add_norm.py:6-59 (which the
// reference defines but never calls); silu(g)*u in float32, pico_vllm/kernels/swiglu.py:28-44.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// An id below zero stands for "the token chosen in the step before": id = -(j + 1) takes
// feedback[j], the j-th token the sampling kernel wrote, so that a step can be launched before the
// host has read the last step's tokens.
template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int H, int V, const int* __restrict__ feedback) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    int id = ids[row];
    if (id < 0 && feedback) id = feedback[-id - 1];
    const bool ok = id >= 0 && id < V;
    const TW* src = table + (size_t)(ok ? id : 0) * H;
    float* dst = out + (size_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? to_f32(src[i]) : 0.f;
}

PICO_API int pico_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H,
                            int V, const int* feedback, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == PICO_F32)
        pico_launch((embedding_kernel<float>), dim3(T), dim3(threads), 0, stream, ids, (const float*)table, out, H, V, feedback);
    else if (table_dtype == PICO_BF16)
        pico_launch((embedding_kernel<bf16>), dim3(T), dim3(threads), 0, stream, ids, (const bf16*)table, out, H, V, feedback);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// ---------------------------------------------------------------- residual add + RMSNorm
// x: float32 residual stream [*, H].  delta (optional): what the previous part produced.
// rows == nullptr: row r of the grid is row r of x; x[r] += delta[r] is written back and
// out[r] = norm(x[r]).  rows != nullptr: out[r] = norm(x[rows[r]] + delta[rows[r]]) and x
// is left alone (used for the last norm, on the rows whose logits are wanted).
template <typename TA> struct Delta4;
template <> struct Delta4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Delta4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// VEC4: H is a multiple of 4; every access is 4 elements wide.
template <typename TA, bool VEC4>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ delta,
                                   const float* __restrict__ weight, TA* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float vals[];  // H floats, then 33 of scratch
    float* scratch = vals + H;
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    float ss = 0.f;
    if (VEC4) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(x + src + i);
            if (delta) {
                const float4 d = Delta4<TA>::load(delta + src + i);
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                if (!rows) *reinterpret_cast<float4*>(x + src + i) = v;
            }
            *reinterpret_cast<float4*>(vals + i) = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = x[src + i];
            if (delta) {
                v += to_f32(delta[src + i]);
                if (!rows) x[src + i] = v;
            }
            vals[i] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TA* dst = out + (size_t)r * H;
    if (VEC4) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(vals + i);
            const float4 w = *reinterpret_cast<const float4*>(weight + i);
            Delta4<TA>::store(dst + i, make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w));
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f32<TA>(vals[i] * inv * weight[i]);
    }
}

PICO_API int pico_add_rmsnorm(float* x, const void* delta, const float* weight, void* out, const int* rows,
                              int R, int H, float eps, int act_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) return PICO_ERR_SIZE;
    int threads = 256;
    if (H <= 256) threads = 64;
    else if (H <= 2048) threads = 128;       // 128 threads were faster than 192, 256 and 384 at 2048 rows of 1536
    else if (H > 4096) threads = 512;
#define LAUNCH_NORM(TA, V4)                                                                                          \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(add_rmsnorm_kernel<TA, V4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        pico_launch((add_rmsnorm_kernel<TA, V4>), dim3(R), dim3(threads), smem, stream, x, (const TA*)delta, weight,  \
                    (TA*)out, rows, H, eps);                                                                         \
    } while (0)
    const bool v4 = H % 4 == 0;
    if (act_dtype == PICO_F32) {
        if (v4) LAUNCH_NORM(float, true); else LAUNCH_NORM(float, false);
    } else if (act_dtype == PICO_BF16) {
        if (v4) LAUNCH_NORM(bf16, true); else LAUNCH_NORM(bf16, false);
    } else
        return PICO_ERR_DTYPE;
#undef LAUNCH_NORM
    return pico_launch_status();
}

// ---------------------------------------------------------------- SwiGLU
// gate_up: [T, 2*I] with the gate columns first; out[t, i] = silu(gate) * up.
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gate_up, TA* __restrict__ out, int I, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float g = to_f32(gate_up[t * 2 * (size_t)I + i]);
        const float u = to_f32(gate_up[t * 2 * (size_t)I + I + i]);
        const float s = g / (1.0f + expf(-g));
        out[idx] = from_f32<TA>(s * u);
    }
}

// bfloat16, I a multiple of 8: 16-byte loads and stores, 8 features per thread
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int I, size_t total8) {
    pdl_launch_dependents();
    pdl_wait();
    const int I8 = I >> 3;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I8;
        const int i = (int)(idx - t * I8) << 3;
        const uint4 g4 = *reinterpret_cast<const uint4*>(gate_up + t * 2 * (size_t)I + i);
        const uint4 u4 = *reinterpret_cast<const uint4*>(gate_up + t * 2 * (size_t)I + I + i);
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 o4;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(gp[j]), u = __bfloat1622float2(up[j]);
            op[j] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + t * (size_t)I + i) = o4;
    }
}

PICO_API int pico_swiglu(const void* gate_up, void* out, int T, int I, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (act_dtype == PICO_BF16 && I % 8 == 0) {
        const size_t total8 = (size_t)T * (I / 8);
        size_t want8 = (total8 + 255) / 256;
        const long long cap = 16LL * pico_num_sms();
        const int blocks8 = (int)((long long)want8 > cap ? cap : (long long)want8);
        pico_launch(swiglu_bf16x8_kernel, dim3(blocks8), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out, I, total8);
        return pico_launch_status();
    }
    const size_t total = (size_t)T * I;
    const int threads = 256;
    size_t want = (total + threads - 1) / threads;
    const long long cap1 = 16LL * pico_num_sms();
    const int blocks = (int)((long long)want > cap1 ? cap1 : (long long)want);
    if (act_dtype == PICO_F32)
        pico_launch((swiglu_kernel<float>), dim3(blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, I, total);
    else if (act_dtype == PICO_BF16)
        pico_launch((swiglu_kernel<bf16>), dim3(blocks), dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, I, total);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

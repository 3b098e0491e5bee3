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
template <typename TA>
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
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[src + i];
        if (delta) {
            v += to_f32(delta[src + i]);
            if (!rows) x[src + i] = v;
        }
        vals[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TA* dst = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f32<TA>(vals[i] * inv * weight[i]);
}

PICO_API int pico_add_rmsnorm(float* x, const void* delta, const float* weight, void* out, const int* rows,
                              int R, int H, float eps, int act_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) return PICO_ERR_SIZE;
    int threads = 256;
    if (H <= 256) threads = 64;
    else if (H <= 1024) threads = 128;
    else if (H > 4096) threads = 512;
    if (act_dtype == PICO_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        pico_launch((add_rmsnorm_kernel<float>), dim3(R), dim3(threads), smem, stream, x, (const float*)delta, weight, (float*)out, rows, H, eps);
    } else if (act_dtype == PICO_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        pico_launch((add_rmsnorm_kernel<bf16>), dim3(R), dim3(threads), smem, stream, x, (const bf16*)delta, weight, (bf16*)out, rows, H, eps);
    } else
        return PICO_ERR_DTYPE;
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

PICO_API int pico_swiglu(const void* gate_up, void* out, int T, int I, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t total = (size_t)T * I;
    const int threads = 256;
    size_t want = (total + threads - 1) / threads;
    const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    if (act_dtype == PICO_F32)
        pico_launch((swiglu_kernel<float>), dim3(blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, I, total);
    else if (act_dtype == PICO_BF16)
        pico_launch((swiglu_kernel<bf16>), dim3(blocks), dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, I, total);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// Next-token choice from float32 logits: argmax (temperature 0), temperature sampling, and nucleus
// (top-p) sampling, by inverse CDF with one uniform number per row that the host supplies.  The
// maximum of a row and its first index are found by several blocks (a vocabulary of 150 k entries is
// 600 KB per row: one block per row took 63 us for 8 rows); the block that finishes a row last adds
// up the partial results - in the order of the parts, so the result does not depend on which block
// that is - and, for a row that is sampled, goes on alone with the passes over the row.
//
// Restated from the reference: temperature 0 means argmax (pico_vllm/sampler.py:3-8,62-63);
// otherwise probabilities are softmax(logits / temperature) (sampler.py:16); top-p keeps, in
// descending order of probability, every token whose higher-ranked tokens hold less than top_p
// of the mass, and renormalises (sampler.py:26-33); top_p >= 1 turns it off (sampler.py:64).
// The reference draws with torch.multinomial from torch's global generator; here the draw is the
// first token, in vocabulary order, at which the running sum of kept probabilities passes
// uniform * kept mass, so a row's result depends only on its logits, parameters and uniform.
// The kept set is found without sorting: token i is kept iff the mass of tokens with a larger
// weight is < top_p * total, and the smallest kept weight is found by bisection on the float
// bit pattern (equal weights are kept or dropped together).
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ float block_excl_scan(float v, float* scratch, float* total) {
    // exclusive prefix sum over threads in thread order; scratch: 33 floats
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    float inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nwarps ? scratch[lane] : 0.f;
        float winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        scratch[lane] = winc - w;  // exclusive over warps
        if (lane == 31) scratch[32] = winc;
    }
    __syncthreads();
    const float res = scratch[warp] + inc - v;
    *total = scratch[32];
    return res;
}

#define SAMPLE_MAX_PARTS 64
#define SAMPLE_MAX_ROWS 1024
__device__ float g_sample_part_max[SAMPLE_MAX_ROWS * SAMPLE_MAX_PARTS];
__device__ int g_sample_part_arg[SAMPLE_MAX_ROWS * SAMPLE_MAX_PARTS];
__device__ int g_sample_arrived[SAMPLE_MAX_ROWS];

// grid (parts, rows): block (p, r) takes elements [p * per, (p + 1) * per) of row r
__global__ void sample_kernel(const float* __restrict__ logits, int row_stride, int V,
                              const float* __restrict__ temperature, const float* __restrict__ top_p,
                              const float* __restrict__ uniform, int* __restrict__ out, int per) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    __shared__ int iscratch[33];
    const int r = blockIdx.y, parts = gridDim.x;
    const float* x = logits + (size_t)r * row_stride;
    const int tid = threadIdx.x;

    // max and its first index, of this block's part
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    {
        const int p0 = min(V, (int)blockIdx.x * per), p1 = min(V, p0 + per);
        for (int i = p0 + tid; i < p1; i += blockDim.x) {
            const float v = x[i];
            if (v > best) { best = v; best_i = i; }
        }
    }
    if (parts > 1) {
        const float pm = block_max(best, scratch);
        int pc = (best == pm) ? best_i : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pc = min(pc, __shfl_xor_sync(0xffffffffu, pc, o));
        __syncthreads();
        if ((tid & 31) == 0) iscratch[tid >> 5] = pc;
        __syncthreads();
        if (tid == 0) {
            int c = 0x7fffffff;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) c = min(c, iscratch[w]);
            g_sample_part_max[r * SAMPLE_MAX_PARTS + blockIdx.x] = pm;
            g_sample_part_arg[r * SAMPLE_MAX_PARTS + blockIdx.x] = c;
            __threadfence();
            iscratch[32] = atomicAdd(&g_sample_arrived[r], 1) == parts - 1;
        }
        __syncthreads();
        if (!iscratch[32]) return;                  // another block finishes this row
        __threadfence();
        if (tid == 0) g_sample_arrived[r] = 0;       // for the next launch
        // the parts in their order: the first index of the maximum stays the first
        best = -INFINITY;
        best_i = 0x7fffffff;
        if (tid < parts) {
            best = __ldcg(&g_sample_part_max[r * SAMPLE_MAX_PARTS + tid]);
            best_i = __ldcg(&g_sample_part_arg[r * SAMPLE_MAX_PARTS + tid]);
        }
        __syncthreads();
    }
    const float mx = block_max(best, scratch);
    int cand = (best == mx) ? best_i : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if ((tid & 31) == 0) iscratch[tid >> 5] = cand;
    __syncthreads();
    if (tid < 32) {
        int c = tid < (blockDim.x >> 5) ? iscratch[tid] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c = min(c, __shfl_xor_sync(0xffffffffu, c, o));
        if (tid == 0) iscratch[32] = c;
    }
    __syncthreads();
    const int arg = iscratch[32];
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 0.f) || arg == 0x7fffffff) {  // greedy, or a row without a finite maximum
        if (tid == 0) out[r] = arg == 0x7fffffff ? 0 : arg;
        return;
    }
    const float inv_t = 1.0f / temp;
    const float tp = top_p ? top_p[r] : 1.f;

    // contiguous chunk of the vocabulary per thread, so that the scan runs in vocabulary order
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int c0 = min(V, tid * chunk), c1 = min(V, c0 + chunk);

    float zsum = 0.f;
    for (int i = c0; i < c1; ++i) zsum += expf((x[i] - mx) * inv_t);
    const float Z = block_sum(zsum, scratch);

    float thresh = 0.f;  // keep weights >= thresh
    if (tp < 1.f) {
        const float limit = tp * Z;
        unsigned lo = 0u, hi = __float_as_uint(1.0f);  // f(hi) is true: no weight exceeds 1
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            const float tau = __uint_as_float(mid);
            float above = 0.f;
            for (int i = c0; i < c1; ++i) {
                const float w = expf((x[i] - mx) * inv_t);
                if (w > tau) above += w;
            }
            above = block_sum(above, scratch);
            if (above < limit) hi = mid; else lo = mid + 1;
        }
        thresh = __uint_as_float(lo);
    }

    float mine = 0.f;
    for (int i = c0; i < c1; ++i) {
        const float w = expf((x[i] - mx) * inv_t);
        if (w >= thresh) mine += w;
    }
    float kept;
    const float before = block_excl_scan(mine, scratch, &kept);
    const float target = uniform[r] * kept;

    // the last thread, in order, whose chunk is not empty and starts at or below the target
    int who = (mine > 0.f && before <= target) ? tid : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) who = max(who, __shfl_xor_sync(0xffffffffu, who, o));
    __syncthreads();
    if ((tid & 31) == 0) iscratch[tid >> 5] = who;
    __syncthreads();
    if (tid < 32) {
        int c = tid < (blockDim.x >> 5) ? iscratch[tid] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c = max(c, __shfl_xor_sync(0xffffffffu, c, o));
        if (tid == 0) iscratch[32] = c;
    }
    __syncthreads();
    const int winner = iscratch[32];
    if (winner < 0) {
        if (tid == 0) out[r] = arg;
        return;
    }
    if (tid == winner) {
        float acc = before;
        int pick = -1, last = -1;
        for (int i = c0; i < c1; ++i) {
            const float w = expf((x[i] - mx) * inv_t);
            if (w >= thresh) {
                acc += w;
                last = i;
                if (acc > target) { pick = i; break; }
            }
        }
        out[r] = pick >= 0 ? pick : last;
    }
}

// logits: [R, row_stride] float32, the first V columns are used.  temperature, top_p, uniform:
// [R] float32 (temperature/top_p may be null: greedy / no nucleus).  out: [R] int32.
PICO_API int pico_sample(const float* logits, int row_stride, int R, int V, const float* temperature,
                         const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return PICO_ERR_SIZE;
    if (temperature && !uniform) return PICO_ERR_SIZE;
    // parts of at least 2048 entries, as many as give every SM a block or two
    int parts = 1;
    if (R <= SAMPLE_MAX_ROWS) {
        while (parts < SAMPLE_MAX_PARTS && parts * 2 * 2048 <= V && parts * R < 296) parts *= 2;
    }
    const int per = (V + parts - 1) / parts;
    pico_launch(sample_kernel, dim3(parts, R), dim3(SAMPLE_THREADS), 0, stream, logits, row_stride, V, temperature, top_p, uniform,
                out, per);
    return pico_launch_status();
}

// float32 copy of bfloat16 rows (logits of the bfloat16 path are handed out as float32)
__global__ void bf16_to_f32_kernel(const bf16* __restrict__ in, float* __restrict__ out, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __bfloat162float(in[i]);
}
PICO_API int pico_bf16_to_f32(const void* in, float* out, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    long long want = (n + 255) / 256;
    const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    pico_launch(bf16_to_f32_kernel, dim3(blocks), dim3(256), 0, stream, (const bf16*)in, out, (size_t)n);
    return pico_launch_status();
}

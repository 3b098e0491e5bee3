// Next-token choice from float32 logits: argmax (temperature 0), temperature sampling, and nucleus
// (top-p) sampling, by inverse CDF with one uniform number per row that the host supplies.
//
// Restated from the reference: temperature 0 means argmax (pico_vllm/sampler.py:3-8,62-63);
// otherwise probabilities are softmax(logits / temperature) (sampler.py:16); top-p keeps, in
// descending order of probability, every token whose higher-ranked tokens hold less than top_p
// of the mass, and renormalises (sampler.py:26-33); top_p >= 1 turns it off (sampler.py:64).
// The reference draws with torch.multinomial from torch's global generator; here the draw is the
// first token, in vocabulary order, at which the running sum of kept probabilities passes
// uniform * kept mass, so a row's result depends only on its logits, parameters and uniform.
//
// A vocabulary of 150 k entries is 600 KB per row, so every pass over a row is made by several
// blocks (grid: parts x rows), and the block that arrives last at the row's counter finishes the
// pass.  Masses are summed as 32.32 fixed-point integers (weight = exp((x - max) / T) <= 1), so that
// sums do not depend on the order in which blocks and threads add: the choice is reproducible.
//   1. maximum and its first index (greedy rows end here);
//   2. the kept set without sorting: token i is kept iff the mass of tokens with a larger weight is
//      < top_p * total.  The smallest kept weight is found by its bit pattern, 11 + 11 + 10 bits at a
//      time: a histogram of mass per value of the next bits among the weights that share the bits
//      found so far, then the lowest bin whose mass above is still below the limit (equal weights
//      are kept or dropped together);
//   3. kept mass per part, the part and then the token at which the running sum passes the target.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_MAX_PARTS 64
#define SAMPLE_ROWS 128          // rows per round of launches
#define SAMPLE_BINS 2048

typedef unsigned long long u64;

struct SampleRow {
    float mx, inv_t;
    int arg, sampled;            // sampled: 0 = done (greedy), 1 = goes through steps 2 and 3
    int resolved;                // the smallest kept weight is known (top_p >= 1, or all bits found)
    unsigned prefix, thresh;     // bits of the smallest kept weight found so far; its whole pattern
    u64 total, limit, above;     // sum of all weights; top_p * total; mass above the bits found so far
    int arrived[5];              // blocks that have finished each pass
};
__device__ SampleRow g_sample_rows[SAMPLE_ROWS];
__device__ float g_sample_part_max[SAMPLE_ROWS * SAMPLE_MAX_PARTS];
__device__ int g_sample_part_arg[SAMPLE_ROWS * SAMPLE_MAX_PARTS];
__device__ u64 g_sample_part_kept[SAMPLE_ROWS * SAMPLE_MAX_PARTS];
__device__ u64 g_sample_hist[SAMPLE_ROWS * SAMPLE_BINS];

__device__ __forceinline__ float sample_weight(float x, float mx, float inv_t) { return expf((x - mx) * inv_t); }
__device__ __forceinline__ u64 sample_fixed(float w) { return __float2ull_rz(w * 4294967296.0f); }

// sums and exclusive prefix sums of 64-bit integers over the block, in thread order; scratch: 33 entries
__device__ __forceinline__ u64 block_excl_scan_u64(u64 v, u64* scratch, u64* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    u64 inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        const u64 w = lane < nwarps ? scratch[lane] : 0ull;
        u64 winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        scratch[lane] = winc - w;
        if (lane == 31) scratch[32] = winc;
    }
    __syncthreads();
    const u64 res = scratch[warp] + inc - v;
    *total = scratch[32];
    return res;
}
__device__ __forceinline__ int block_min_int(int v, int* scratch) {       // scratch: 33 ints
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        int c = threadIdx.x < (blockDim.x >> 5) ? scratch[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c = min(c, __shfl_xor_sync(0xffffffffu, c, o));
        if (threadIdx.x == 0) scratch[32] = c;
    }
    __syncthreads();
    return scratch[32];
}
// true in every thread of the one block that arrives last at the counter (which it then resets)
__device__ __forceinline__ bool sample_last_block(int* counter, int blocks, int* flag) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int last = atomicAdd(counter, 1) == blocks - 1;
        if (last) *counter = 0;
        *flag = last;
    }
    __syncthreads();
    const bool last = *flag != 0;
    if (last) __threadfence();
    return last;
}

// Step 1.  grid (parts, rows): block (p, r) takes elements [p * per, (p + 1) * per) of row r.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_max_kernel(const float* __restrict__ logits, int row_stride, int V, const float* __restrict__ temperature,
                  int* __restrict__ out, int per) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    __shared__ int iscratch[33];
    __shared__ int flag;
    const int r = blockIdx.y, parts = gridDim.x, tid = threadIdx.x;
    const float* x = logits + (size_t)r * row_stride;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    {
        const int p0 = min(V, (int)blockIdx.x * per), p1 = min(V, p0 + per);
        for (int i = p0 + tid; i < p1; i += blockDim.x) {
            const float v = x[i];
            if (v > best) { best = v; best_i = i; }
        }
    }
    const float pm = block_max(best, scratch);
    const int pc = block_min_int(best == pm ? best_i : 0x7fffffff, iscratch);
    if (tid == 0) {
        g_sample_part_max[r * SAMPLE_MAX_PARTS + blockIdx.x] = pm;
        g_sample_part_arg[r * SAMPLE_MAX_PARTS + blockIdx.x] = pc;
    }
    SampleRow& row = g_sample_rows[r];
    if (!sample_last_block(&row.arrived[0], parts, &flag)) return;
    // the parts in their order: the first index of the maximum stays the first
    best = -INFINITY;
    best_i = 0x7fffffff;
    if (tid < parts) {
        best = __ldcg(&g_sample_part_max[r * SAMPLE_MAX_PARTS + tid]);
        best_i = __ldcg(&g_sample_part_arg[r * SAMPLE_MAX_PARTS + tid]);
    }
    const float mx = block_max(best, scratch);
    const int arg = block_min_int(best == mx ? best_i : 0x7fffffff, iscratch);
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp > 0.f) || arg == 0x7fffffff;       // or a row without a finite maximum
    for (int b = tid; b < SAMPLE_BINS; b += blockDim.x) g_sample_hist[r * SAMPLE_BINS + b] = 0ull;
    if (tid == 0) {
        if (greedy) out[r] = arg == 0x7fffffff ? 0 : arg;
        row.mx = mx;
        row.arg = arg == 0x7fffffff ? 0 : arg;
        row.inv_t = greedy ? 0.f : 1.0f / temp;
        row.sampled = greedy ? 0 : 1;
        row.resolved = 0;
        row.prefix = 0u;
        row.thresh = 0u;
        row.total = row.limit = row.above = 0ull;
    }
}

// Step 2, LEVEL 0, 1, 2: mass per value of the next 11, 11, 10 bits of the weight's pattern.
template <int LEVEL>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_hist_kernel(const float* __restrict__ logits, int row_stride, int V, const float* __restrict__ top_p, int per) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ u64 sh[SAMPLE_BINS];
    __shared__ u64 scratch[33];
    __shared__ int iscratch[33];
    __shared__ int flag;
    const int r = blockIdx.y, parts = gridDim.x, tid = threadIdx.x;
    SampleRow& row = g_sample_rows[r];
    if (!row.sampled || row.resolved) return;          // written by an earlier kernel: the same for every block of the row
    constexpr int NB = LEVEL == 2 ? 1024 : SAMPLE_BINS;
    const float* x = logits + (size_t)r * row_stride;
    const float mx = row.mx, inv_t = row.inv_t;
    const unsigned prefix = row.prefix;
    for (int b = tid; b < NB; b += blockDim.x) sh[b] = 0ull;
    __syncthreads();
    u64 zsum = 0ull;
    {
        const int p0 = min(V, (int)blockIdx.x * per), p1 = min(V, p0 + per);
        for (int i = p0 + tid; i < p1; i += blockDim.x) {
            const float w = sample_weight(x[i], mx, inv_t);
            const unsigned pat = __float_as_uint(w);
            const u64 fx = sample_fixed(w);
            if (LEVEL == 0) {
                zsum += fx;
                atomicAdd(&sh[pat >> 21], fx);
            } else if (LEVEL == 1) {
                if ((pat >> 21) == prefix) atomicAdd(&sh[(pat >> 10) & 0x7ffu], fx);
            } else {
                if ((pat >> 10) == prefix) atomicAdd(&sh[pat & 0x3ffu], fx);
            }
        }
    }
    __syncthreads();
    for (int b = tid; b < NB; b += blockDim.x)
        if (sh[b]) atomicAdd(&g_sample_hist[r * SAMPLE_BINS + b], sh[b]);
    if (LEVEL == 0) {
        u64 tot;
        block_excl_scan_u64(zsum, scratch, &tot);
        if (tid == 0) atomicAdd(&row.total, tot);
    }
    if (!sample_last_block(&row.arrived[1 + LEVEL], parts, &flag)) return;
    // the lowest bin whose mass above (in higher bins, and above the bits found before) is below the limit
    u64 limit = row.limit, base = row.above;
    bool all = false;
    if (LEVEL == 0) {
        const u64 total = __ldcg(&row.total);
        const float tp = top_p ? top_p[r] : 1.f;
        all = !(tp < 1.f);
        limit = (u64)((double)tp * (double)total);
    }
    // thread t takes bins NB - 1 - 2t and NB - 2 - 2t: descending, so that a prefix sum is the mass above
    const int hi_bin = NB - 1 - 2 * tid, lo_bin = hi_bin - 1;
    const u64 h_hi = hi_bin >= 0 ? __ldcg(&g_sample_hist[r * SAMPLE_BINS + hi_bin]) : 0ull;
    const u64 h_lo = lo_bin >= 0 ? __ldcg(&g_sample_hist[r * SAMPLE_BINS + lo_bin]) : 0ull;
    u64 tot;
    const u64 before = base + block_excl_scan_u64(h_hi + h_lo, scratch, &tot);
    int cand = 0x7fffffff;
    if (hi_bin >= 0 && before < limit) cand = hi_bin;
    if (lo_bin >= 0 && before + h_hi < limit) cand = lo_bin;
    const int bin = block_min_int(cand, iscratch);
    for (int b = tid; b < SAMPLE_BINS; b += blockDim.x) g_sample_hist[r * SAMPLE_BINS + b] = 0ull;      // for the next pass
    if (all) {
        if (tid == 0) { row.limit = limit; row.thresh = 0u; row.resolved = 1; }
        return;
    }
    if (bin == 0x7fffffff) {          // a limit of zero: only the largest weight (1.0) is kept
        if (tid == 0) { row.limit = limit; row.thresh = __float_as_uint(1.0f); row.resolved = 1; }
        return;
    }
    // the mass above the chosen bin: this thread knows it if the bin is one of its two
    if (bin == hi_bin || bin == lo_bin) {
        row.limit = limit;
        row.above = bin == hi_bin ? before : before + h_hi;
        if (LEVEL == 0) row.prefix = (unsigned)bin;
        else if (LEVEL == 1) row.prefix = (prefix << 11) | (unsigned)bin;
        else {
            row.thresh = (prefix << 10) | (unsigned)bin;
            row.resolved = 1;
        }
    }
}

// Step 3.  Kept mass per part; the last block finds the part and the token where the running sum passes the target.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_pick_kernel(const float* __restrict__ logits, int row_stride, int V, const float* __restrict__ uniform,
                   int* __restrict__ out, int per) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ u64 scratch[33];
    __shared__ int iscratch[33];
    __shared__ int flag;
    __shared__ u64 sh_before;
    const int r = blockIdx.y, parts = gridDim.x, tid = threadIdx.x;
    SampleRow& row = g_sample_rows[r];
    if (!row.sampled) return;
    const float* x = logits + (size_t)r * row_stride;
    const float mx = row.mx, inv_t = row.inv_t;
    const unsigned thresh = row.thresh;
    u64 mine = 0ull;
    {
        const int p0 = min(V, (int)blockIdx.x * per), p1 = min(V, p0 + per);
        for (int i = p0 + tid; i < p1; i += blockDim.x) {
            const float w = sample_weight(x[i], mx, inv_t);
            if (__float_as_uint(w) >= thresh) mine += sample_fixed(w);
        }
    }
    u64 part_kept;
    block_excl_scan_u64(mine, scratch, &part_kept);
    if (tid == 0) g_sample_part_kept[r * SAMPLE_MAX_PARTS + blockIdx.x] = part_kept;
    if (!sample_last_block(&row.arrived[4], parts, &flag)) return;
    // the parts in vocabulary order: the last part that is not empty and starts at or below the target
    const u64 pk = tid < parts ? __ldcg(&g_sample_part_kept[r * SAMPLE_MAX_PARTS + tid]) : 0ull;
    u64 kept;
    const u64 pbefore = block_excl_scan_u64(pk, scratch, &kept);
    const u64 target = (u64)((double)uniform[r] * (double)kept);
    const int winner = -block_min_int((tid < parts && pk > 0ull && pbefore <= target) ? -tid : 1, iscratch);
    if (winner < 0) {                 // nothing was kept (cannot happen with a finite maximum)
        if (tid == 0) out[r] = row.arg;
        return;
    }
    if (tid == winner) sh_before = pbefore;
    __syncthreads();
    // the winning part, a contiguous chunk per thread so that the scan runs in vocabulary order
    const int p0 = min(V, winner * per), p1 = min(V, p0 + per);
    const int chunk = (p1 - p0 + (int)blockDim.x - 1) / (int)blockDim.x;
    const int c0 = min(p1, p0 + tid * chunk), c1 = min(p1, c0 + chunk);
    u64 cmine = 0ull;
    for (int i = c0; i < c1; ++i) {
        const float w = sample_weight(x[i], mx, inv_t);
        if (__float_as_uint(w) >= thresh) cmine += sample_fixed(w);
    }
    u64 unused;
    const u64 cbefore = sh_before + block_excl_scan_u64(cmine, scratch, &unused);
    const int who = -block_min_int((cmine > 0ull && cbefore <= target) ? -tid : 1, iscratch);
    if (who < 0) {
        if (tid == 0) out[r] = row.arg;
        return;
    }
    if (tid == who) {
        u64 acc = cbefore;
        int pick = -1, last = -1;
        for (int i = c0; i < c1; ++i) {
            const float w = sample_weight(x[i], mx, inv_t);
            if (__float_as_uint(w) >= thresh) {
                const u64 fx = sample_fixed(w);
                if (fx == 0ull) continue;
                acc += fx;
                last = i;
                if (acc > target) { pick = i; break; }
            }
        }
        out[r] = pick >= 0 ? pick : (last >= 0 ? last : row.arg);
    }
}

// logits: [R, row_stride] float32, the first V columns are used.  temperature, top_p, uniform:
// [R] float32 (temperature/top_p may be null: greedy / no nucleus).  out: [R] int32.
PICO_API int pico_sample(const float* logits, int row_stride, int R, int V, const float* temperature,
                         const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return PICO_ERR_SIZE;
    if (temperature && !uniform) return PICO_ERR_SIZE;
    const int wave = 2 * pico_num_sms();
    for (int r0 = 0; r0 < R; r0 += SAMPLE_ROWS) {
        const int rows = R - r0 < SAMPLE_ROWS ? R - r0 : SAMPLE_ROWS;
        // parts of at least 2048 entries, as many as give every SM a block or two
        int parts = 1;
        while (parts < SAMPLE_MAX_PARTS && parts * 2 * 2048 <= V && parts * rows < wave) parts *= 2;
        const int per = (V + parts - 1) / parts;
        const float* lg = logits + (size_t)r0 * row_stride;
        const dim3 grid(parts, rows), block(SAMPLE_THREADS);
        pico_launch(sample_max_kernel, grid, block, 0, stream, lg, row_stride, V, temperature ? temperature + r0 : nullptr,
                    out + r0, per);
        if (temperature) {
            const float* tp = top_p ? top_p + r0 : nullptr;
            pico_launch(sample_hist_kernel<0>, grid, block, 0, stream, lg, row_stride, V, tp, per);
            if (top_p) {
                pico_launch(sample_hist_kernel<1>, grid, block, 0, stream, lg, row_stride, V, tp, per);
                pico_launch(sample_hist_kernel<2>, grid, block, 0, stream, lg, row_stride, V, tp, per);
            }
            pico_launch(sample_pick_kernel, grid, block, 0, stream, lg, row_stride, V, uniform + r0, out + r0, per);
        }
    }
    return pico_launch_status();
}

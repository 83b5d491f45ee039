// Token choice from float32 logits, one block per row.
//
// argmax: the largest logit, lowest token id on ties (the reference's reducers do the
// same, thinruntime/triton_kernels.py:2249-2250, 2470-2471; torch.argmax of the float
// logits at thinruntime/gpu_runtime.py:11204).
//
// sample: scores = logits / temperature; tokens below the k-th largest score are
// dropped (ties with it stay); then the nucleus: a token is dropped when the
// probability of all tokens with a larger score already exceeds top_p; the survivors'
// softmax is sampled by inverse CDF in token-id order at a uniform number that is a
// function of (seed, request, step) only.  The distribution is the one of
// scripts/stress_validate_thin.py:840-856 (its sampler runs on the host with
// torch.multinomial); the k-th value and the nucleus edge are found without sorting,
// by bisection on the bit pattern of the scores.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned order_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float <=> larger key
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, long long ld, int vocab, int* __restrict__ out) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float x = row[j];
        if (x > v || (x == v && j < idx) || idx == 0x7fffffff) { v = x; idx = j; }
    }
    // NaN logits never compare greater; a row of NaN yields its first visited ids.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int warps = blockDim.x >> 5;
        v = lane < warps ? best_v[lane] : -INFINITY;
        idx = lane < warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx;
    }
}

// Two stages for large vocabularies: ARGMAX_CHUNKS blocks per row each reduce a slice to
// (value, id) in `scratch`, then one warp per row reduces those; the comparison rule
// (larger value, lower id on ties) is the same at every level.
#define ARGMAX_CHUNKS 32

__global__ void __launch_bounds__(256)
argmax_stage1_kernel(const float* __restrict__ logits, long long ld, int vocab, float* __restrict__ scratch_v,
                     int* __restrict__ scratch_i) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    const float* row = logits + (size_t)blockIdx.y * ld;
    const int per = (vocab + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int lo = blockIdx.x * per, hi = min(vocab, lo + per);
    float v = -INFINITY;
    int idx = 0x7fffffff;
    if ((((uintptr_t)(row + lo)) & 15) == 0) {
        // four 16-byte loads per thread in flight together (one load per loop turn, each waiting for the one before
        // through the comparison, cost a round trip to the L2 per element: 11 us for 4,008 elements a block)
        const float4* row4 = reinterpret_cast<const float4*>(row + lo);
        const int quads = (hi - lo) >> 2;
        for (int base = 0; base < quads; base += 4 * 256) {
            float4 x[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int q = base + k * 256 + threadIdx.x;
                if (q < quads) x[k] = __ldg(row4 + q);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int q = base + k * 256 + threadIdx.x;
                if (q < quads) {
                    const int j = lo + 4 * q;
                    if (idx == 0x7fffffff || x[k].x > v) { v = x[k].x; idx = j; }
                    if (x[k].y > v) { v = x[k].y; idx = j + 1; }
                    if (x[k].z > v) { v = x[k].z; idx = j + 2; }
                    if (x[k].w > v) { v = x[k].w; idx = j + 3; }
                }
            }
        }
        for (int j = lo + 4 * quads + threadIdx.x; j < hi; j += blockDim.x) {       // at most three numbers at the end
            const float x = row[j];
            if (idx == 0x7fffffff || x > v || (x == v && j < idx)) { v = x; idx = j; }
        }
    } else {
        for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) {
            const float x = row[j];
            if (idx == 0x7fffffff || x > v) { v = x; idx = j; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < 8 ? best_v[lane] : -INFINITY;
        idx = lane < 8 ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
        }
        if (lane == 0) {
            scratch_v[blockIdx.y * ARGMAX_CHUNKS + blockIdx.x] = v;
            scratch_i[blockIdx.y * ARGMAX_CHUNKS + blockIdx.x] = idx;
        }
    }
}

__global__ void argmax_stage2_kernel(const float* __restrict__ scratch_v, const int* __restrict__ scratch_i, int n_rows,
                                     int* __restrict__ out) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    float v = scratch_v[row * ARGMAX_CHUNKS + lane];
    int idx = scratch_i[row * ARGMAX_CHUNKS + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
    }
    if (lane == 0) out[row] = idx == 0x7fffffff ? 0 : idx;
}

// scratch: room for n_rows * 32 floats and n_rows * 32 ints (may be null: one block per row then).
extern "C" int tt_argmax_rows(const float* logits, long long ld, int n_rows, int vocab, int* out, float* scratch_v,
                              int* scratch_i, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return (int)cudaErrorInvalidValue;
    if (scratch_v && scratch_i && vocab >= 8192 && n_rows <= 65535) {
        tt_launch_pdl(argmax_stage1_kernel, dim3(dim3(ARGMAX_CHUNKS, n_rows)), dim3(256), 0, stream, logits, ld, vocab, scratch_v, scratch_i);
        tt_launch_pdl(argmax_stage2_kernel, dim3((n_rows + 3) / 4), dim3(128), 0, stream, scratch_v, scratch_i, n_rows, out);
        TT_LAUNCH_CHECK();
    }
    tt_launch_pdl(argmax_rows_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, vocab, out);
    TT_LAUNCH_CHECK();
}

// splitmix64 finaliser
__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

// uniform in [0, 1) from (seed, request, step): 24 bits
__device__ __forceinline__ float counter_uniform(unsigned long long seed, unsigned long long request, unsigned long long step) {
    unsigned long long x = mix64(seed + 0x9E3779B97F4A7C15ull);
    x = mix64(x ^ (request * 0xD1B54A32D192ED03ull));
    x = mix64(x ^ (step * 0x8CB92BA72F3D8DD7ull));
    return (float)(x >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ int block_count(int v, int* shared32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) shared32[warp] = v;
    __syncthreads();
    int total = lane < (int)(blockDim.x >> 5) ? shared32[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    return total;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, long long ld, int vocab, float temperature, int top_k,
                   float top_p, unsigned long long seed, const int* __restrict__ request,
                   const int* __restrict__ step, int* __restrict__ out) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    __shared__ float red[32];
    __shared__ int redi[32];
    __shared__ float prefix[SAMPLE_THREADS];
    const float* row = logits + (size_t)blockIdx.x * ld;
    const float inv_t = 1.0f / temperature;

    float mx = -INFINITY;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) mx = fmaxf(mx, row[j]);
    mx = tt_block_max(mx, red);

    // the k-th largest score, as an order key: the largest key with count(keys >= key) >= k
    unsigned floor_key = 0u;
    if (top_k > 0 && top_k < vocab) {
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = floor_key | (1u << bit);
            int c = 0;
            for (int j = threadIdx.x; j < vocab; j += blockDim.x) c += order_key(row[j]) >= cand;
            if (block_count(c, redi) >= top_k) floor_key = cand;
        }
    }

    // nucleus edge: the smallest key v with mass(keys > v) <= top_p * mass(all kept)
    if (top_p < 1.0f) {
        float z = 0.0f;
        for (int j = threadIdx.x; j < vocab; j += blockDim.x)
            if (order_key(row[j]) >= floor_key) z += expf((row[j] - mx) * inv_t);
        z = tt_block_sum(z, red);
        const float limit = top_p * z;
        // largest key w with mass(keys > w) > limit; the edge is w + 1
        unsigned w = 0u;
        bool any = false;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = w | (1u << bit);
            float above = 0.0f;
            for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
                const unsigned key = order_key(row[j]);
                if (key >= floor_key && key > cand) above += expf((row[j] - mx) * inv_t);
            }
            above = tt_block_sum(above, red);
            if (above > limit) { w = cand; any = true; }
        }
        if (!any) {
            // is even key 0 past the limit?
            float above = 0.0f;
            for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
                const unsigned key = order_key(row[j]);
                if (key >= floor_key && key > 0u) above += expf((row[j] - mx) * inv_t);
            }
            above = tt_block_sum(above, red);
            any = above > limit;
        }
        if (any) {
            const unsigned edge = w + 1u;
            if (edge > floor_key) floor_key = edge;
        }
    }

    // inverse CDF in token-id order; thread i owns ids [i * chunk, (i + 1) * chunk)
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * chunk, hi = min(vocab, lo + chunk);
    float mine = 0.0f;
    for (int j = lo; j < hi; ++j)
        if (order_key(row[j]) >= floor_key) mine += expf((row[j] - mx) * inv_t);
    prefix[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float run = 0.0f;
        for (int i = 0; i < (int)blockDim.x; ++i) { run += prefix[i]; prefix[i] = run; }
    }
    __syncthreads();
    const float total = prefix[blockDim.x - 1];
    const float u = counter_uniform(seed, (unsigned long long)(unsigned)request[blockIdx.x], (unsigned long long)(unsigned)step[blockIdx.x]);
    const float target = u * total;
    const float before = threadIdx.x ? prefix[threadIdx.x - 1] : 0.0f;
    const float after = prefix[threadIdx.x];
    // exactly one thread has before <= target < after (prefix is non-decreasing and target < total)
    if (before <= target && target < after) {
        float run = before;
        int pick = -1, last = -1;
        for (int j = lo; j < hi; ++j) {
            if (order_key(row[j]) < floor_key) continue;
            last = j;
            run += expf((row[j] - mx) * inv_t);
            if (run > target) { pick = j; break; }
        }
        out[blockIdx.x] = pick >= 0 ? pick : last;
    }
    if (!(total > 0.0f) && threadIdx.x == 0) out[blockIdx.x] = 0;  // a row without finite logits
}

extern "C" int tt_sample_rows(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k,
                              float top_p, unsigned long long seed, const int* request, const int* step, int* out,
                              cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || !(temperature > 0.0f) || !(top_p > 0.0f)) return (int)cudaErrorInvalidValue;
    tt_launch_pdl(sample_rows_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, vocab, temperature, top_k, top_p, seed, request, step, out);
    TT_LAUNCH_CHECK();
}

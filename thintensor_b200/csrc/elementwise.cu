// Memory-bound kernels between the matrix products: embedding gather, residual add
// fused with RMSNorm, rotary encoding fused with the cache append, SwiGLU, and the
// length bookkeeping of a step.  All statistics, angles and sums are float32.
//
// Counterparts in random-unknown-username/Thintensor (Triton, one token per launch):
// _copy_embed_token thinruntime/gpu_runtime.py:11396-11427; _rms_norm_kernel and
// _add_rms_norm_kernel thinruntime/triton_kernels.py:2561-2614; _rope_qk_inplace_kernel
// thinruntime/triton_kernels.py:2637-2687 with PagedKVCache._store_token
// thinruntime/gpu_runtime.py:4530-4556; _silu_mul_kernel thinruntime/triton_kernels.py:2760-2774.
#include "common.cuh"

// ------------------------------------------------------------------------------------
// embedding gather: residual[t, :] = table[token[t], :] * scale   (float32 out)
// ------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ residual, int hidden, int vocab, float scale,
                                    unsigned* status) {
    // The first kernel of every step waits before it lets its dependents start: whatever a
    // later kernel of this step reads ahead of its own wait (lengths, tables, cache blocks of
    // earlier steps) is then complete, because no kernel of this step starts before the
    // previous step's last kernel has finished.
    tt_pdl_wait();
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    int id = tokens[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, TT_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) residual[(size_t)t * hidden + j] = 0.0f;
        return;
    }
    const TW* row = table + (size_t)id * hidden;
    float* out = residual + (size_t)t * hidden;
    if constexpr (sizeof(TW) == 2) {
        // rows of whole 16-byte pieces: eight numbers a load, two 16-byte stores
        if ((hidden & 7) == 0 && (((uintptr_t)table | (uintptr_t)residual) & 15) == 0) {
            for (int j = 8 * threadIdx.x; j < hidden; j += 8 * blockDim.x) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + j));
                const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 a = __bfloat1622float2(pairs[0]), b = __bfloat1622float2(pairs[1]);
                const float2 c = __bfloat1622float2(pairs[2]), d = __bfloat1622float2(pairs[3]);
                *reinterpret_cast<float4*>(out + j) = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
                *reinterpret_cast<float4*>(out + j + 4) = make_float4(c.x * scale, c.y * scale, d.x * scale, d.y * scale);
            }
            return;
        }
    }
    for (int j = threadIdx.x; j < hidden; j += blockDim.x)
        out[j] = tt_to_float(row[j]) * scale;
}

extern "C" int tt_embed_gather(const void* table, int table_dtype, const int* tokens, float* residual, int n_tokens,
                               int hidden, int vocab, float scale, unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == TT_F32)
        tt_launch_pdl(embed_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, tokens, residual, hidden, vocab, scale, status);
    else
        tt_launch_pdl(embed_gather_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)table, tokens, residual, hidden, vocab, scale, status);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// residual add + RMSNorm.
//   x = residual[r] + delta[0][r] + delta[1][r] + ...      (fixed order)
//   residual[r] = x                                        (only when rows == nullptr)
//   out[i] = x * rsqrt(mean(x^2) + eps) * (weight + weight_offset)
// One block per output row; the row is kept in shared memory between the two passes.
// With `rows`, output row i is taken from residual row rows[i] and nothing is written
// back (the final norm at the wanted positions).
// ------------------------------------------------------------------------------------
template <typename TOut>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const float* __restrict__ delta, int splits,
                                   size_t split_stride, const float* __restrict__ weight, float weight_offset,
                                   float eps, TOut* __restrict__ out, const int* __restrict__ rows, int hidden,
                                   int row_cache) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float row_shared[];  // row_cache floats, then 32 for the reduction
    float* reduce = row_shared + row_cache;
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* res = residual + (size_t)r * hidden;
    const float* del = delta ? delta + (size_t)r * hidden : nullptr;
    float sumsq = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float x = res[j];
        for (int s = 0; s < splits; ++s) x += del[(size_t)s * split_stride + j];
        if (j < row_cache) row_shared[j] = x;
        if (!rows && splits > 0) res[j] = x;
        sumsq += x * x;
    }
    const float total = tt_block_sum(sumsq, reduce);
    const float rstd = rsqrtf(total / (float)hidden + eps);
    TOut* o = out + (size_t)i * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float x;
        if (j < row_cache) {
            x = row_shared[j];
        } else if (!rows) {
            x = res[j];  // written back above by this same thread
        } else {
            x = res[j];
            for (int s = 0; s < splits; ++s) x += del[(size_t)s * split_stride + j];
        }
        o[j] = tt_from_float<TOut>(x * rstd * (weight[j] + weight_offset));
    }
}

// four consecutive outputs as one store (the row start is 16-byte aligned and j counts groups of four)
__device__ __forceinline__ void tt_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void tt_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&lo);
    v.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// The same for hidden sizes that are multiples of 4 up to 16384: every thread keeps its
// (up to four) float4 pieces of the row in registers, all loads of the k-slices are
// independent, and the order of additions is the one of the kernel above.
#define NORM_VEC_MAX 4
// PIECES: float4 pieces of a row per thread: 1 when the block is as wide as the row (few rows: decoding), else up to
// NORM_VEC_MAX (prompts).  BATCH: how many k-slices' loads are in flight together.
template <typename TOut, int PIECES, int BATCH>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const float* __restrict__ delta, int splits, size_t split_stride,
                       const float* __restrict__ weight, float weight_offset, float eps, TOut* __restrict__ out,
                       const int* __restrict__ rows, int hidden) {
    tt_pdl_launch_dependents();
    __shared__ float reduce[32];
    const int i = blockIdx.x;
    const int quads = hidden >> 2;
    // the norm's weight is written by no kernel: it is fetched while the previous kernel still runs
    const float4* w4 = reinterpret_cast<const float4*>(weight);
    float4 w[PIECES];
#pragma unroll
    for (int v = 0; v < PIECES; ++v) {
        const int j = threadIdx.x + v * blockDim.x;
        if (j < quads) w[v] = __ldg(w4 + j);
    }
    tt_pdl_wait();
    const int r = rows ? rows[i] : i;
    float4* res = reinterpret_cast<float4*>(residual + (size_t)r * hidden);
    const float4* del = delta ? reinterpret_cast<const float4*>(delta + (size_t)r * hidden) : nullptr;
    const size_t stride4 = split_stride >> 2;
    float4 x[PIECES];
    float sumsq = 0.0f;
#pragma unroll
    for (int v = 0; v < PIECES; ++v) {
        const int j = threadIdx.x + v * blockDim.x;
        if (j < quads) {
            float4 a = res[j];
            // BATCH slices' loads are in flight together (one after the other they cost a round trip to the L2
            // each: a decode step's norm after a product of 16 k-slices); the additions keep the slices' order
            for (int s0 = 0; s0 < splits; s0 += BATCH) {
                float4 d[BATCH];
#pragma unroll
                for (int i = 0; i < BATCH; ++i)
                    if (s0 + i < splits) d[i] = __ldg(del + (size_t)(s0 + i) * stride4 + j);
#pragma unroll
                for (int i = 0; i < BATCH; ++i)
                    if (s0 + i < splits) { a.x += d[i].x; a.y += d[i].y; a.z += d[i].z; a.w += d[i].w; }
            }
            if (!rows && splits > 0) res[j] = a;
            x[v] = a;
            sumsq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    const float total = tt_block_sum(sumsq, reduce);
    const float rstd = rsqrtf(total / (float)hidden + eps);
    TOut* o = out + (size_t)i * hidden;
#pragma unroll
    for (int v = 0; v < PIECES; ++v) {
        const int j = threadIdx.x + v * blockDim.x;
        if (j < quads) {
            const float y0 = x[v].x * rstd * (w[v].x + weight_offset), y1 = x[v].y * rstd * (w[v].y + weight_offset);
            const float y2 = x[v].z * rstd * (w[v].z + weight_offset), y3 = x[v].w * rstd * (w[v].w + weight_offset);
            tt_store4(o + 4 * j, y0, y1, y2, y3);
        }
    }
}

extern "C" int tt_add_rmsnorm(float* residual, const float* delta, int splits, long long split_stride,
                              const float* weight, float weight_offset, float eps, void* out, int out_dtype,
                              const int* rows, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!delta) splits = 0;
    if (hidden % 4 == 0 && hidden <= 4096 * NORM_VEC_MAX && split_stride % 4 == 0 && ((uintptr_t)residual & 15) == 0 &&
        ((uintptr_t)delta & 15) == 0 && ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        int threads = ((hidden / 4 + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        if (n_rows >= 1024) {
            // prompts: up to four pieces of the row per thread (fewer, fatter blocks: measured 5.33 -> 5.20 ms for a
            // 2,048-token prefill of the 1B shape)
            const int fewest = (((hidden / 4 + NORM_VEC_MAX - 1) / NORM_VEC_MAX + 31) / 32) * 32;
            threads = fewest < 128 ? 128 : fewest;
            if (threads > 1024) threads = 1024;
        }
        const bool one_piece = threads * 4 >= hidden;         // the block covers the row: one piece per thread, eight slices at a time
#define TT_NORM(T, P, B) tt_launch_pdl(add_rmsnorm_vec_kernel<T, P, B>, dim3(n_rows), dim3(threads), 0, stream, residual, delta, splits, (size_t)split_stride, weight, weight_offset, eps, (T*)out, rows, hidden)
        if (out_dtype == TT_F32) { if (one_piece) TT_NORM(float, 1, 8); else TT_NORM(float, NORM_VEC_MAX, 2); }
        else { if (one_piece) TT_NORM(__nv_bfloat16, 1, 8); else TT_NORM(__nv_bfloat16, NORM_VEC_MAX, 2); }
#undef TT_NORM
        TT_LAUNCH_CHECK();
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int row_cache = hidden <= 11264 ? hidden : 11264;  // 44 KB of the default 48 KB
    const size_t shared = (size_t)(row_cache + 32) * sizeof(float);
    if (out_dtype == TT_F32)
        tt_launch_pdl(add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), shared, stream, residual, delta, splits, (size_t)split_stride, weight, weight_offset, eps, (float*)out, rows, hidden, row_cache);
    else
        tt_launch_pdl(add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), shared, stream, residual, delta, splits, (size_t)split_stride, weight, weight_offset, eps, (__nv_bfloat16*)out, rows, hidden, row_cache);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// rotary encoding + cache append.
// qkv: float32 [splits][tokens][q_cols + 2 * kv_cols] partial sums of the projection.
// For token t of sequence b at position p = len_before[b] + (t - cu[b]):
//   q' -> q_out[t] (activation dtype), k' -> key pool at p, v -> value pool at p
//   (values are stored transposed inside a block, see common.cuh).
// Rotation on the first rotary_dim numbers of each head, halves convention:
//   a' = a cos - b sin, b' = b cos + a sin, angle = inv_freq[i] * float(p) in float32.
// kv_cols == 0: the projection holds queries only and nothing is appended (a layer that
// reads another layer's cache).
// ------------------------------------------------------------------------------------
// sum of one element over the k-slices of a projection: independent loads, fixed order of additions
__device__ __forceinline__ float sum_slices(const float* __restrict__ p, int splits, size_t split_stride) {
    float total = 0.0f;
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
        const float a = __ldg(p + (size_t)s * split_stride), b = __ldg(p + (size_t)(s + 1) * split_stride);
        const float c = __ldg(p + (size_t)(s + 2) * split_stride), d = __ldg(p + (size_t)(s + 3) * split_stride);
        total = (((total + a) + b) + c) + d;
    }
    for (; s < splits; ++s) total += __ldg(p + (size_t)s * split_stride);
    return total;
}

// One thread per item of a token: a rotated pair of q or k, a number beyond the rotary
// part, or a value.  grid = (tokens, ceil(items / blockDim.x)).
template <typename TAct>
__global__ void rope_append_kernel(const float* __restrict__ qkv, int splits, size_t split_stride,
                                   const float* __restrict__ inv_freq,
                                   int rotary_dim, float attention_scaling, TAct* __restrict__ q_out,
                                   TAct* __restrict__ k_pool, TAct* __restrict__ v_pool,
                                   const int* __restrict__ table, int table_width, int pool_blocks,
                                   const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                   int heads, int kv_heads, int head_dim, int write_cache, unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int half = rotary_dim >> 1;
    const int q_cols = heads * head_dim;
    const int kv_cols = write_cache ? kv_heads * head_dim : 0;
    const int cols = q_cols + 2 * kv_cols;
    const float* row = qkv + (size_t)t * cols;
    const int* table_row = table + (size_t)b * table_width;
    const int rot_heads = heads + (write_cache ? kv_heads : 0);
    const int pass = head_dim - rotary_dim;  // numbers of a head that are not rotated
    const int n_rot = rot_heads * half, n_pass = rot_heads * pass;
    int w = blockIdx.y * blockDim.x + threadIdx.x;
    if (w < n_rot) {
        const int head = w / half, i = w - head * half;
        const int col = head * head_dim + i;  // k heads follow q heads in the row
        const float a = sum_slices(row + col, splits, split_stride);
        const float c2 = sum_slices(row + col + half, splits, split_stride);
        float si, co;
        sincosf(inv_freq[i] * (float)pos, &si, &co);
        co *= attention_scaling;
        si *= attention_scaling;
        const float ra = a * co - c2 * si, rb = c2 * co + a * si;
        if (head < heads) {
            q_out[(size_t)t * q_cols + col] = tt_from_float<TAct>(ra);
            q_out[(size_t)t * q_cols + col + half] = tt_from_float<TAct>(rb);
        } else {
            const long long off = tt_cache_offset(table_row, pos, head - heads, kv_heads, head_dim, pool_blocks, status);
            if (off >= 0) {
                k_pool[off + i] = tt_from_float<TAct>(ra);
                k_pool[off + i + half] = tt_from_float<TAct>(rb);
            }
        }
        return;
    }
    w -= n_rot;
    if (w < n_pass) {
        const int head = w / pass, i = rotary_dim + (w - head * pass);
        const int col = head * head_dim + i;
        const float a = sum_slices(row + col, splits, split_stride);
        if (head < heads) {
            q_out[(size_t)t * q_cols + col] = tt_from_float<TAct>(a);
        } else {
            const long long off = tt_cache_offset(table_row, pos, head - heads, kv_heads, head_dim, pool_blocks, status);
            if (off >= 0) k_pool[off + i] = tt_from_float<TAct>(a);
        }
        return;
    }
    w -= n_pass;
    if (w < kv_cols) {
        const int kh = w / head_dim, i = w - kh * head_dim;
        const float a = sum_slices(row + q_cols + kv_cols + w, splits, split_stride);
        const long long off = tt_value_offset(table_row, pos, kh, kv_heads, head_dim, pool_blocks, status);
        if (off >= 0) v_pool[off + (long long)i * TT_BLOCK_TOKENS] = tt_from_float<TAct>(a);
    }
}

// The same with four neighbouring items per thread (float4 loads, 8-byte stores of q and k): used
// when the rotary part and the rest of a head are multiples of 8 and 4 numbers.
__device__ __forceinline__ float4 sum_slices4(const float* __restrict__ p, int splits, size_t split_stride) {
    float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < splits; ++s) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p + (size_t)s * split_stride));
        total.x += v.x; total.y += v.y; total.z += v.z; total.w += v.w;
    }
    return total;
}

constexpr int ROPE_MAX_HALF = 128;          // half of the largest rotary part (head sizes go up to 256)

template <typename TAct>
__global__ void rope_append_vec_kernel(const float* __restrict__ qkv, int splits, size_t split_stride,
                                       const float* __restrict__ inv_freq, int rotary_dim, float attention_scaling,
                                       TAct* __restrict__ q_out, TAct* __restrict__ k_pool, TAct* __restrict__ v_pool,
                                       const int* __restrict__ table, int table_width, int pool_blocks,
                                       const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                       int heads, int kv_heads, int head_dim, int write_cache, unsigned* status) {
    tt_pdl_launch_dependents();
    // Lengths, offsets and tables were written before the step's first kernel started: the token's sequence, position,
    // cache block and angles are found ahead of the wait for the qkv product (five dependent round trips to the L2 that
    // would otherwise follow it); only the product's slices are read after it.
    const int t = blockIdx.x;
    // one token per sequence (a decode step): token t is sequence t, which two independent loads confirm
    const int b = (sequences == (int)gridDim.x && cu[t] == t && cu[t + 1] == t + 1) ? t : tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int half = rotary_dim >> 1, half4 = half >> 2;
    const int q_cols = heads * head_dim;
    const int kv_cols = write_cache ? kv_heads * head_dim : 0;
    const int cols = q_cols + 2 * kv_cols;
    const float* row = qkv + (size_t)t * cols;
    const int* table_row = table + (size_t)b * table_width;
    const int rot_heads = heads + (write_cache ? kv_heads : 0);
    const int pass4 = (head_dim - rotary_dim) >> 2;
    const int n_rot = rot_heads * half4, n_pass = rot_heads * pass4;
    // the angles depend on the position only: one table per block instead of one sincosf per head and pair
    __shared__ float cos_sh[ROPE_MAX_HALF], sin_sh[ROPE_MAX_HALF];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(__ldg(inv_freq + i) * (float)pos, &sin_sh[i], &cos_sh[i]);
    // the token's cache block, looked up once: -1 where the table entry lies outside the pool (reported when a write needs it)
    int block = -1;
    if (write_cache) {
        block = table_row[pos / TT_BLOCK_TOKENS];
        if (block < 0 || block >= pool_blocks) block = -1;
    }
    const int slot = pos % TT_BLOCK_TOKENS;
    auto key_offset = [&](int kv_head) -> long long {
        if (block < 0) { atomicOr(status, TT_STATUS_BAD_BLOCK); return -1; }
        return (((long long)block * kv_heads + kv_head) * TT_BLOCK_TOKENS + slot) * head_dim;
    };
    auto value_offset = [&](int kv_head) -> long long {
        if (block < 0) { atomicOr(status, TT_STATUS_BAD_BLOCK); return -1; }
        return ((long long)block * kv_heads + kv_head) * head_dim * TT_BLOCK_TOKENS + slot;
    };
    __syncthreads();
    tt_pdl_wait();
    const int n_val = kv_cols >> 2;
    // the token's blocks (one when there are many tokens, several when there are few) walk over its items
    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_rot + n_pass + n_val; item += gridDim.y * blockDim.x) {
        int w = item;
        if (w < n_rot) {
            const int head = w / half4, i = (w - head * half4) * 4;
            const int col = head * head_dim + i;
            const float4 a = sum_slices4(row + col, splits, split_stride);
            const float4 c = sum_slices4(row + col + half, splits, split_stride);
            const float s0 = sin_sh[i], c0 = cos_sh[i], s1 = sin_sh[i + 1], c1 = cos_sh[i + 1];
            const float s2 = sin_sh[i + 2], c2 = cos_sh[i + 2], s3 = sin_sh[i + 3], c3 = cos_sh[i + 3];
            const float k = attention_scaling;
            const float ra0 = (a.x * c0 - c.x * s0) * k, rb0 = (c.x * c0 + a.x * s0) * k;
            const float ra1 = (a.y * c1 - c.y * s1) * k, rb1 = (c.y * c1 + a.y * s1) * k;
            const float ra2 = (a.z * c2 - c.z * s2) * k, rb2 = (c.z * c2 + a.z * s2) * k;
            const float ra3 = (a.w * c3 - c.w * s3) * k, rb3 = (c.w * c3 + a.w * s3) * k;
            TAct* dst;
            if (head < heads) {
                dst = q_out + (size_t)t * q_cols + col;
            } else {
                const long long off = key_offset(head - heads);
                if (off < 0) continue;
                dst = k_pool + off + i;
            }
            tt_store4(dst, ra0, ra1, ra2, ra3);
            tt_store4(dst + half, rb0, rb1, rb2, rb3);
            continue;
        }
        w -= n_rot;
        if (w < n_pass) {
            const int head = w / pass4, i = rotary_dim + (w - head * pass4) * 4;
            const int col = head * head_dim + i;
            const float4 a = sum_slices4(row + col, splits, split_stride);
            if (head < heads) {
                tt_store4(q_out + (size_t)t * q_cols + col, a.x, a.y, a.z, a.w);
            } else {
                const long long off = key_offset(head - heads);
                if (off >= 0) tt_store4(k_pool + off + i, a.x, a.y, a.z, a.w);
            }
            continue;
        }
        w -= n_pass;
        const int e = w * 4, kh = e / head_dim, i = e - kh * head_dim;
        const float4 a = sum_slices4(row + q_cols + kv_cols + e, splits, split_stride);
        const long long off = value_offset(kh);
        if (off >= 0) {
            TAct* dst = v_pool + off + (long long)i * TT_BLOCK_TOKENS;      // values lie transposed: one number per 64-token row
            dst[0] = tt_from_float<TAct>(a.x);
            dst[TT_BLOCK_TOKENS] = tt_from_float<TAct>(a.y);
            dst[2 * TT_BLOCK_TOKENS] = tt_from_float<TAct>(a.z);
            dst[3 * TT_BLOCK_TOKENS] = tt_from_float<TAct>(a.w);
        }
    }
}

extern "C" int tt_rope_append(const float* qkv, int splits, long long split_stride,
                              const float* inv_freq, int rotary_dim, float attention_scaling, void* q_out,
                              void* k_pool, void* v_pool, int act_dtype, const int* table, int table_width,
                              int pool_blocks, const int* cu, const int* len_before, int sequences, int n_tokens,
                              int heads, int kv_heads, int head_dim, int write_cache, unsigned* status,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return (int)cudaErrorInvalidValue;
    const int rot_heads = heads + (write_cache ? kv_heads : 0);
    if (rotary_dim % 8 == 0 && rotary_dim / 2 <= ROPE_MAX_HALF && (head_dim - rotary_dim) % 4 == 0 && split_stride % 4 == 0 && ((uintptr_t)qkv & 15) == 0 &&
        ((uintptr_t)inv_freq & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)k_pool & 15) == 0) {
        const int items4 = rot_heads * (rotary_dim / 8) + rot_heads * ((head_dim - rotary_dim) / 4) + (write_cache ? kv_heads * head_dim / 4 : 0);
        // prompts: one block per token (fewer blocks, each with more loads in flight); few tokens: a block per 128 items
        const int threads4 = n_tokens >= 1024 ? (items4 >= 256 ? 256 : (items4 >= 128 ? 128 : 64)) : 128;
        const dim3 grid4(n_tokens, n_tokens >= 1024 ? 1 : (items4 + threads4 - 1) / threads4);
        if (act_dtype == TT_F32)
            tt_launch_pdl(rope_append_vec_kernel<float>, grid4, dim3(threads4), 0, stream, qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (float*)q_out, (float*)k_pool, (float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
        else
            tt_launch_pdl(rope_append_vec_kernel<__nv_bfloat16>, grid4, dim3(threads4), 0, stream, qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
        TT_LAUNCH_CHECK();
    }
    const int items = rot_heads * (rotary_dim / 2) + rot_heads * (head_dim - rotary_dim) + (write_cache ? kv_heads * head_dim : 0);
    const int threads = 128;
    const dim3 grid(n_tokens, (items + threads - 1) / threads);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    if (act_dtype == TT_F32)
        tt_launch_pdl(rope_append_kernel<float>, dim3(grid), dim3(threads), 0, stream, qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (float*)q_out, (float*)k_pool, (float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
    else
        tt_launch_pdl(rope_append_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// What every layer's rotation of a step has in common, computed once per step: for packed token t
// its position p = len_before[b] + (t - cu[b]), its sequence b, and cos and sin of inv_freq[i] * p
// (float32 angle, as in the kernels above).  The tensor-core qkv product's epilogue reads these
// instead of finding the sequence and calling sincosf again in each of the model's layers.
//   cos_sin: float2 [tokens][half]; where: int2 [tokens] = (position, sequence)
// ------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, int half, const int* __restrict__ cu,
                                  const int* __restrict__ len_before, int sequences, float2* __restrict__ cos_sin,
                                  int2* __restrict__ where) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    if (threadIdx.x == 0) where[t] = make_int2(pos, b);
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float si, co;
        sincosf(__ldg(inv_freq + i) * (float)pos, &si, &co);
        cos_sin[(size_t)t * half + i] = make_float2(co, si);
    }
}

extern "C" int tt_rope_table(const float* inv_freq, int half, const int* cu, const int* len_before, int sequences, int n_tokens,
                             void* cos_sin, void* where, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (half <= 0) return (int)cudaErrorInvalidValue;
    const int threads = half >= 64 ? 64 : 32;
    tt_launch_pdl(rope_table_kernel, dim3(n_tokens), dim3(threads), 0, stream, inv_freq, half, cu, len_before, sequences, (float2*)cos_sin, (int2*)where);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// SwiGLU: act[t, j] = silu(gate[t, j]) * up[t, j], silu(g) = g / (1 + exp(-g)).
// gate_up: float32 [splits][tokens][2 * inter], gate columns first.
// ------------------------------------------------------------------------------------
template <typename TAct>
__global__ void swiglu_kernel(const float* __restrict__ gate_up, int splits, size_t split_stride,
                              TAct* __restrict__ act, int inter, size_t total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    const float* row = gate_up + t * (size_t)(2 * inter);
    float g = 0.0f, u = 0.0f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {                  // gate and up of up to four slices in flight together
        g += __ldg(row + s * split_stride + j);
        u += __ldg(row + s * split_stride + inter + j);
    }
    act[idx] = tt_from_float<TAct>(g / (1.0f + expf(-g)) * u);
}

extern "C" int tt_swiglu(const float* gate_up, int splits, long long split_stride, void* act,
                         int act_dtype, int n_tokens, int inter, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * inter;
    if (total == 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (act_dtype == TT_F32)
        tt_launch_pdl(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, gate_up, splits, (size_t)split_stride, (float*)act, inter, total);
    else
        tt_launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, gate_up, splits, (size_t)split_stride, (__nv_bfloat16*)act, inter, total);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// after a step: len[b] += cu[b + 1] - cu[b]; counters[b] += 1 where the caller keeps a count of
// the steps each sequence has taken (the sampler's random numbers are indexed by it)
// ------------------------------------------------------------------------------------
__global__ void advance_lengths_kernel(int* __restrict__ len, const int* __restrict__ cu, int* __restrict__ counters, int sequences) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < sequences) {
        len[b] += cu[b + 1] - cu[b];
        if (counters) counters[b] += 1;
    }
}

extern "C" int tt_advance_lengths(int* len, const int* cu, int* counters, int sequences, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    tt_launch_pdl(advance_lengths_kernel, dim3((sequences + 127) / 128), dim3(128), 0, stream, len, cu, counters, sequences);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// A few int32 numbers between device memory and pinned host memory that the device can
// address (token ids in, sampled ids out): as a kernel in the chain of a step this costs
// a fraction of a copy node in a CUDA graph.  Host memory is read and written uncached.
// ------------------------------------------------------------------------------------
__global__ void copy_int32_kernel(int* __restrict__ dst, const int* __restrict__ src, int n, const int* __restrict__ extra) {
    tt_pdl_wait();
    tt_pdl_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) __stcg(dst + i, __ldcv(src + i));
    if (extra && i == n) __stcg(dst + n, __ldcv(extra));
}

// extra: one more int32 (the device status word, say) that is copied to dst[n]; may be null.
extern "C" int tt_copy_int32(int* dst, const int* src, int n, const int* extra, cudaStream_t stream) {
    if (n <= 0) return 0;
    tt_launch_pdl(copy_int32_kernel, dim3((n + 1 + 127) / 128), dim3(128), 0, stream, dst, src, n, extra);
    TT_LAUNCH_CHECK();
}

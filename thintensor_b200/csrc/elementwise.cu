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
    const int t = blockIdx.x;
    int id = tokens[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, TT_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) residual[(size_t)t * hidden + j] = 0.0f;
        return;
    }
    const TW* row = table + (size_t)id * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x)
        residual[(size_t)t * hidden + j] = tt_to_float(row[j]) * scale;
}

extern "C" int tt_embed_gather(const void* table, int table_dtype, const int* tokens, float* residual, int n_tokens,
                               int hidden, int vocab, float scale, unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == TT_F32)
        embed_gather_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)table, tokens, residual, hidden, vocab, scale, status);
    else
        embed_gather_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>((const __nv_bfloat16*)table, tokens, residual, hidden, vocab, scale, status);
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

extern "C" int tt_add_rmsnorm(float* residual, const float* delta, int splits, long long split_stride,
                              const float* weight, float weight_offset, float eps, void* out, int out_dtype,
                              const int* rows, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int row_cache = hidden <= 11264 ? hidden : 11264;  // 44 KB of the default 48 KB
    const size_t shared = (size_t)(row_cache + 32) * sizeof(float);
    if (!delta) splits = 0;
    if (out_dtype == TT_F32)
        add_rmsnorm_kernel<float><<<n_rows, threads, shared, stream>>>(residual, delta, splits, (size_t)split_stride, weight, weight_offset, eps, (float*)out, rows, hidden, row_cache);
    else
        add_rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, shared, stream>>>(residual, delta, splits, (size_t)split_stride, weight, weight_offset, eps, (__nv_bfloat16*)out, rows, hidden, row_cache);
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
template <typename TAct>
__global__ void rope_append_kernel(const float* __restrict__ qkv, int splits, size_t split_stride,
                                   const float* __restrict__ inv_freq,
                                   int rotary_dim, float attention_scaling, TAct* __restrict__ q_out,
                                   TAct* __restrict__ k_pool, TAct* __restrict__ v_pool,
                                   const int* __restrict__ table, int table_width, int pool_blocks,
                                   const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                   int heads, int kv_heads, int head_dim, int write_cache, unsigned* status) {
    extern __shared__ float cs[];  // cos[rotary_dim / 2], sin[rotary_dim / 2]
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int half = rotary_dim >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = inv_freq[i] * (float)pos;
        float s, c;
        sincosf(angle, &s, &c);
        cs[i] = c * attention_scaling;
        cs[half + i] = s * attention_scaling;
    }
    __syncthreads();
    const int q_cols = heads * head_dim;
    const int kv_cols = write_cache ? kv_heads * head_dim : 0;
    const int cols = q_cols + 2 * kv_cols;
    const float* row = qkv + (size_t)t * cols;
    const int* table_row = table + (size_t)b * table_width;
    const int rot_heads = heads + (write_cache ? kv_heads : 0);
    const int pass = head_dim - rotary_dim;  // numbers of a head that are not rotated
    // rotated pairs of q and k
    for (int w = threadIdx.x; w < rot_heads * half; w += blockDim.x) {
        const int head = w / half, i = w - head * half;
        const int col = head * head_dim + i;  // k heads follow q heads in the row
        float a = 0.0f, c2 = 0.0f;
        for (int s = 0; s < splits; ++s) {
            a += row[s * split_stride + col];
            c2 += row[s * split_stride + col + half];
        }
        const float co = cs[i], si = cs[half + i];
        const float ra = a * co - c2 * si, rb = c2 * co + a * si;
        if (head < heads) {
            q_out[(size_t)t * q_cols + col] = tt_from_float<TAct>(ra);
            q_out[(size_t)t * q_cols + col + half] = tt_from_float<TAct>(rb);
        } else {
            const int kh = head - heads;
            const long long off = tt_cache_offset(table_row, pos, kh, kv_heads, head_dim, pool_blocks, status);
            if (off >= 0) {
                k_pool[off + i] = tt_from_float<TAct>(ra);
                k_pool[off + i + half] = tt_from_float<TAct>(rb);
            }
        }
    }
    // numbers beyond the rotary part pass through
    for (int w = threadIdx.x; w < rot_heads * pass; w += blockDim.x) {
        const int head = w / pass, i = rotary_dim + (w - head * pass);
        const int col = head * head_dim + i;
        float a = 0.0f;
        for (int s = 0; s < splits; ++s) a += row[s * split_stride + col];
        if (head < heads) {
            q_out[(size_t)t * q_cols + col] = tt_from_float<TAct>(a);
        } else {
            const long long off = tt_cache_offset(table_row, pos, head - heads, kv_heads, head_dim, pool_blocks, status);
            if (off >= 0) k_pool[off + i] = tt_from_float<TAct>(a);
        }
    }
    // values
    for (int w = threadIdx.x; w < kv_cols; w += blockDim.x) {
        const int kh = w / head_dim, i = w - kh * head_dim;
        const int col = q_cols + kv_cols + w;
        float a = 0.0f;
        for (int s = 0; s < splits; ++s) a += row[s * split_stride + col];
        const long long off = tt_value_offset(table_row, pos, kh, kv_heads, head_dim, pool_blocks, status);
        if (off >= 0) v_pool[off + (long long)i * TT_BLOCK_TOKENS] = tt_from_float<TAct>(a);
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
    const int work = (heads + kv_heads) * head_dim / 2;
    const int threads = work >= 512 ? 256 : 128;
    const size_t shared = (size_t)(rotary_dim > 0 ? rotary_dim : 2) * sizeof(float);
    if (act_dtype == TT_F32)
        rope_append_kernel<float><<<n_tokens, threads, shared, stream>>>(qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (float*)q_out, (float*)k_pool, (float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
    else
        rope_append_kernel<__nv_bfloat16><<<n_tokens, threads, shared, stream>>>(qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// SwiGLU: act[t, j] = silu(gate[t, j]) * up[t, j], silu(g) = g / (1 + exp(-g)).
// gate_up: float32 [splits][tokens][2 * inter], gate columns first.
// ------------------------------------------------------------------------------------
template <typename TAct>
__global__ void swiglu_kernel(const float* __restrict__ gate_up, int splits, size_t split_stride,
                              TAct* __restrict__ act, int inter, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    const float* row = gate_up + t * (size_t)(2 * inter);
    float g = 0.0f, u = 0.0f;
    for (int s = 0; s < splits; ++s) {
        g += row[s * split_stride + j];
        u += row[s * split_stride + inter + j];
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
        swiglu_kernel<float><<<blocks, threads, 0, stream>>>(gate_up, splits, (size_t)split_stride, (float*)act, inter, total);
    else
        swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(gate_up, splits, (size_t)split_stride, (__nv_bfloat16*)act, inter, total);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// after a step: len[b] += cu[b + 1] - cu[b]
// ------------------------------------------------------------------------------------
__global__ void advance_lengths_kernel(int* __restrict__ len, const int* __restrict__ cu, int sequences) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < sequences) len[b] += cu[b + 1] - cu[b];
}

extern "C" int tt_advance_lengths(int* len, const int* cu, int sequences, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    advance_lengths_kernel<<<(sequences + 127) / 128, 128, 0, stream>>>(len, cu, sequences);
    TT_LAUNCH_CHECK();
}

// Causal grouped-query attention over the block cache, for any head size that is a
// multiple of 16 up to 256, in float32 or bfloat16 storage with float32 arithmetic.
// One kernel serves prompts and decoding: a warp owns one (token, query head, split)
// and walks that token's visible keys 32 at a time with a running softmax; with more
// than one split the partial (max, sum, accumulator) triples are merged by a second
// kernel.  This is the exact path (every product and sum in float32 FMA) and the
// fallback of the tensor-core kernels for head sizes they do not take.
//
// Counterparts in random-unknown-username/Thintensor: _single_token_gqa_attention_kernel
// thinruntime/triton_kernels.py:14-109 and the split pair
// _split_gqa_attention_partial_kernel / _reduce_kernel thinruntime/triton_kernels.py:112-245
// (one token, one sequence); the formula is thinruntime/gpu_runtime.py:8913-8961.
#include "attention_kernels.cuh"

// part_acc: float32 [tokens * heads * splits * head_dim], part_ml: float32
// [tokens * heads * splits * 2]; both may be null when splits == 1.
extern "C" int tt_attention(const void* q, const void* k_pool, const void* v_pool, int dtype, const int* table,
                            int table_width, int pool_blocks, const int* cu, const int* len_before, int sequences,
                            int n_tokens, int heads, int kv_heads, int head_dim, float scale, int window, int splits,
                            void* out, float* part_acc, float* part_ml, unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim % 16 || head_dim > ATTN_MAX_HEAD_DIM || heads % kv_heads || splits < 1 || splits > 65535)
        return (int)cudaErrorInvalidValue;
    if (splits > 1 && (!part_acc || !part_ml)) return (int)cudaErrorInvalidValue;
    const long long rows = (long long)n_tokens * heads;
    const dim3 grid((unsigned)((rows + ATTN_WARPS - 1) / ATTN_WARPS), (unsigned)splits);
    const size_t shared = (size_t)ATTN_WARPS * head_dim * sizeof(float);
    if (dtype == TT_F32) {
        attention_rows_kernel<float><<<grid, ATTN_WARPS * 32, shared, stream>>>((const float*)q, (const float*)k_pool, (const float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, scale, window, splits, (float*)out, part_acc, part_ml, status);
        if (splits > 1)
            attention_merge_kernel<float><<<grid.x, ATTN_WARPS * 32, 0, stream>>>(part_acc, part_ml, splits, head_dim, rows, (float*)out);
    } else {
        attention_rows_kernel<__nv_bfloat16><<<grid, ATTN_WARPS * 32, shared, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, scale, window, splits, (__nv_bfloat16*)out, part_acc, part_ml, status);
        if (splits > 1)
            attention_merge_kernel<__nv_bfloat16><<<grid.x, ATTN_WARPS * 32, 0, stream>>>(part_acc, part_ml, splits, head_dim, rows, (__nv_bfloat16*)out);
    }
    TT_LAUNCH_CHECK();
}

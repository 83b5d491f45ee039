// tt_attention_decode_static: the split-key attention of attention.cu with its scratch in
// a file-scope device array instead of caller-provided memory.  It calls no cudaMalloc,
// cudaFree or any routine that allocates.  Read attention_static_scratch.h for whom it is
// meant, its fixed limit, and the rule that calls must not overlap on the GPU.
#include "attention_static_scratch.h"

#include <mutex>
#include <stdio.h>

#include "attention_kernels.cuh"

// The scratch itself.  In host code this name is only a handle for the symbol lookup
// below: it is NOT a device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char tt_static_scratch[TT_STATIC_SCRATCH_BYTES];

#define TT_STATIC_MAX_DEVICES 64
static float* scratch_address[TT_STATIC_MAX_DEVICES];   // device address of the array, per device
static std::mutex scratch_mutex;
static thread_local char last_error[256] = "no error";

extern "C" const char* tt_attention_static_last_error(void) { return last_error; }

// Bytes of scratch for these sizes, or ~0ull when a size is not positive or the count is beyond
// 2^40 entries (65,000 times the array).  Every multiplication is preceded by a division that shows
// it cannot pass that bound, so no product can wrap around and come back small enough to be accepted.
extern "C" unsigned long long tt_attention_static_bytes_needed(int n_tokens, int heads, int head_dim, int splits) {
    const unsigned long long never = ~0ull;
    const unsigned long long limit = 1ull << 40;
    if (n_tokens <= 0 || heads <= 0 || head_dim <= 0 || splits <= 0) return never;
    unsigned long long slots = (unsigned long long)n_tokens;
    if (slots > limit / (unsigned long long)heads) return never;
    slots *= (unsigned long long)heads;
    if (slots > limit / (unsigned long long)splits) return never;
    slots *= (unsigned long long)splits;
    if (slots > limit / (unsigned long long)head_dim) return never;
    // accumulators, then (max, sum) pairs, the second part starting on a 256-byte boundary
    const unsigned long long acc = (slots * (unsigned long long)head_dim * sizeof(float) + 255ull) & ~255ull;
    return acc + slots * 2 * sizeof(float);
}

// The device address of the array on the current device; looked up once per device, with
// that device current.
static int scratch_for_current_device(float** out) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        snprintf(last_error, sizeof(last_error), "cudaGetDevice failed: %s", cudaGetErrorString(err));
        return (int)err;
    }
    if (device < 0 || device >= TT_STATIC_MAX_DEVICES) {
        snprintf(last_error, sizeof(last_error), "device index %d is beyond the %d this entry point keeps addresses for", device, TT_STATIC_MAX_DEVICES);
        return TT_STATIC_NO_SYMBOL;
    }
    std::lock_guard<std::mutex> guard(scratch_mutex);
    if (!scratch_address[device]) {
        void* address = nullptr;
        err = cudaGetSymbolAddress(&address, tt_static_scratch);
        if (err != cudaSuccess || !address) {
            snprintf(last_error, sizeof(last_error), "cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(err));
            return TT_STATIC_NO_SYMBOL;
        }
        scratch_address[device] = (float*)address;
    }
    *out = scratch_address[device];
    return TT_STATIC_OK;
}

extern "C" int tt_attention_decode_static(const void* q, const void* k_pool, const void* v_pool, int dtype,
                                          const int* table, int table_width, int pool_blocks, const int* cu,
                                          const int* len_before, int sequences, int n_tokens, int heads, int kv_heads,
                                          int head_dim, float scale, int window, int splits, void* out,
                                          unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return TT_STATIC_OK;
    if (sequences <= 0 || table_width <= 0 || pool_blocks <= 0 || head_dim <= 0 || head_dim % 16 || head_dim > ATTN_MAX_HEAD_DIM || heads <= 0 || kv_heads <= 0 ||
        heads % kv_heads || splits < 1 || splits > 65535 || (dtype != TT_F32 && dtype != TT_BF16)) {
        snprintf(last_error, sizeof(last_error), "sizes not taken: head_dim %d (multiples of 16 up to %d), heads %d, kv_heads %d, splits %d, dtype %d",
                 head_dim, ATTN_MAX_HEAD_DIM, heads, kv_heads, splits, dtype);
        return TT_STATIC_BAD_SIZE;
    }
    const unsigned long long need = tt_attention_static_bytes_needed(n_tokens, heads, head_dim, splits);
    if (need > TT_STATIC_SCRATCH_BYTES) {
        snprintf(last_error, sizeof(last_error), "%d tokens x %d heads x %d splits x head size %d need %llu bytes of scratch; the static array holds %u",
                 n_tokens, heads, splits, head_dim, need, TT_STATIC_SCRATCH_BYTES);
        return TT_STATIC_TOO_LARGE;
    }
    float* scratch = nullptr;
    const int found = scratch_for_current_device(&scratch);
    if (found != TT_STATIC_OK) return found;
    const unsigned long long slots = (unsigned long long)n_tokens * heads * splits;
    float* part_acc = scratch;
    float* part_ml = (float*)((unsigned char*)scratch + ((slots * head_dim * sizeof(float) + 255ull) & ~255ull));

    const long long rows = (long long)n_tokens * heads;
    const dim3 grid((unsigned)((rows + ATTN_WARPS - 1) / ATTN_WARPS), (unsigned)splits);
    const size_t shared = (size_t)ATTN_WARPS * head_dim * sizeof(float);
    // with one split the first kernel writes `out` directly and the scratch is not touched
    if (dtype == TT_F32) {
        attention_rows_kernel<float><<<grid, ATTN_WARPS * 32, shared, stream>>>((const float*)q, (const float*)k_pool, (const float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, scale, window, splits, (float*)out, part_acc, part_ml, status);
        if (splits > 1)
            attention_merge_kernel<float><<<grid.x, ATTN_WARPS * 32, 0, stream>>>(part_acc, part_ml, splits, head_dim, rows, (float*)out);
    } else {
        attention_rows_kernel<__nv_bfloat16><<<grid, ATTN_WARPS * 32, shared, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, scale, window, splits, (__nv_bfloat16*)out, part_acc, part_ml, status);
        if (splits > 1)
            attention_merge_kernel<__nv_bfloat16><<<grid.x, ATTN_WARPS * 32, 0, stream>>>(part_acc, part_ml, splits, head_dim, rows, (__nv_bfloat16*)out);
    }
    const cudaError_t launched = cudaGetLastError();
    if (launched != cudaSuccess) snprintf(last_error, sizeof(last_error), "launch failed: %s", cudaGetErrorString(launched));
    return (int)launched;
}

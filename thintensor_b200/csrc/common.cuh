// Shared helpers of the sm_100a kernels: element types, conversions, reductions and
// the status word.  Every entry point is extern "C", takes raw device pointers and a
// stream, allocates nothing, and returns a cudaError_t value as int (0 = launched).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Element type codes used across the C interface.
#define TT_F32 0
#define TT_BF16 1

// Tokens of one cache block; block tables index blocks of this many tokens.
#define TT_BLOCK_TOKENS 64

// Bits of the device status word.  A kernel that meets one of these conditions sets
// the bit, skips the access and carries on; the host reads the word after the step.
#define TT_STATUS_BAD_TOKEN 1u      // token id outside the embedding table
#define TT_STATUS_BAD_BLOCK 2u      // block table entry outside the pool
#define TT_STATUS_WAIT_EXPIRED 4u   // a bounded wait on an mbarrier ran out
#define TT_STATUS_BAD_SHAPE 8u      // a size the kernel cannot take reached the device

#define TT_LAUNCH_CHECK() return (int)cudaGetLastError()

// Programmatic dependent launch.  A kernel started through tt_launch_pdl may begin while
// the kernel before it in the stream is still running; it must call tt_pdl_wait() before
// it touches anything that kernel (or any earlier one) wrote, and it calls
// tt_pdl_launch_dependents() as early as it can so that the kernel after it may in turn
// start its own preamble (for a matrix product: fetching weights, which no kernel of the
// step writes).  tt_pdl_wait() returns only when every earlier kernel has finished and
// its writes are visible, so the chain of dependencies stays intact.  Both are no-ops in
// a kernel that was launched the ordinary way.
__device__ __forceinline__ void tt_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void tt_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename Kernel, typename... Args>
static inline cudaError_t tt_launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t shared, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, args...);
}

// The same with the grid's z dimension grouped into thread-block clusters of cluster_z CTAs.
template <typename Kernel, typename... Args>
static inline cudaError_t tt_launch_pdl_cluster(Kernel kernel, dim3 grid, dim3 block, size_t shared, cudaStream_t stream,
                                                unsigned cluster_z, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = 1;
    attribute[1].val.clusterDim.y = 1;
    attribute[1].val.clusterDim.z = cluster_z;
    config.attrs = attribute;
    config.numAttrs = 2;
    return cudaLaunchKernelEx(&config, kernel, args...);
}

template <typename T> __device__ __forceinline__ float tt_to_float(T v);
template <> __device__ __forceinline__ float tt_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float tt_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T tt_from_float(float v);
template <> __device__ __forceinline__ float tt_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 tt_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float tt_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float tt_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// the additions depends only on the block size, never on the data or the grid.
__device__ __forceinline__ float tt_block_sum(float v, float* shared32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = tt_warp_sum(v);
    __syncthreads();
    if (lane == 0) shared32[warp] = v;
    __syncthreads();
    float total = (lane < warps) ? shared32[lane] : 0.0f;
    total = tt_warp_sum(total);
    return total;
}

__device__ __forceinline__ float tt_block_max(float v, float* shared32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = tt_warp_max(v);
    __syncthreads();
    if (lane == 0) shared32[warp] = v;
    __syncthreads();
    float total = (lane < warps) ? shared32[lane] : -INFINITY;
    total = tt_warp_max(total);
    return total;
}

// The sequence of a packed token: the b with cu[b] <= t < cu[b + 1].
__device__ __forceinline__ int tt_find_sequence(const int* __restrict__ cu, int sequences, int t) {
    int lo = 0, hi = sequences;  // invariant: cu[lo] <= t < cu[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

// The cache of one layer is two block pools.  Keys:   [block][kv_head][TT_BLOCK_TOKENS][head_dim]
// (a token's head vector is contiguous).  Values: [block][kv_head][head_dim][TT_BLOCK_TOKENS]
// (transposed: the 64 tokens of one head dimension are contiguous, which is the operand
// order the P @ V tensor-core product reads straight from global memory).
//
// tt_cache_offset: element offset of a key vector; tt_value_offset: element offset of
// value dimension 0 of a token, dimension d lies d * TT_BLOCK_TOKENS elements further.
// Both return -1 and raise the status bit when the table entry is outside the pool.
__device__ __forceinline__ long long tt_cache_offset(const int* __restrict__ table_row, int position, int kv_head,
                                                     int kv_heads, int head_dim, int pool_blocks,
                                                     unsigned* status) {
    const int block = table_row[position / TT_BLOCK_TOKENS];
    if (block < 0 || block >= pool_blocks) {
        if (status) atomicOr(status, TT_STATUS_BAD_BLOCK);
        return -1;
    }
    return (((long long)block * kv_heads + kv_head) * TT_BLOCK_TOKENS + (position % TT_BLOCK_TOKENS)) * head_dim;
}

__device__ __forceinline__ long long tt_value_offset(const int* __restrict__ table_row, int position, int kv_head,
                                                     int kv_heads, int head_dim, int pool_blocks,
                                                     unsigned* status) {
    const int block = table_row[position / TT_BLOCK_TOKENS];
    if (block < 0 || block >= pool_blocks) {
        if (status) atomicOr(status, TT_STATUS_BAD_BLOCK);
        return -1;
    }
    return ((long long)block * kv_heads + kv_head) * head_dim * TT_BLOCK_TOKENS + (position % TT_BLOCK_TOKENS);
}

// Kernel templates of the exact attention path, shared by the entry points that launch
// them (attention.cu, attention_static_scratch.cu).  See attention.cu for what they compute.
#pragma once
#include "common.cuh"


#define ATTN_WARPS 4
#define ATTN_MAX_HEAD_DIM 256

template <typename T> struct Vec16;  // 16 bytes of T
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ float dot16(const T* __restrict__ krow, const float* __restrict__ q, int head_dim);

template <>
__device__ __forceinline__ float dot16<float>(const float* __restrict__ krow, const float* __restrict__ q, int head_dim) {
    float acc = 0.0f;
    for (int d = 0; d < head_dim; d += 4) {
        const float4 k = *reinterpret_cast<const float4*>(krow + d);
        acc = fmaf(k.x, q[d], acc);
        acc = fmaf(k.y, q[d + 1], acc);
        acc = fmaf(k.z, q[d + 2], acc);
        acc = fmaf(k.w, q[d + 3], acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot16<__nv_bfloat16>(const __nv_bfloat16* __restrict__ krow, const float* __restrict__ q, int head_dim) {
    float acc = 0.0f;
    for (int d = 0; d < head_dim; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p[i]);
            acc = fmaf(f.x, q[d + 2 * i], acc);
            acc = fmaf(f.y, q[d + 2 * i + 1], acc);
        }
    }
    return acc;
}

// window <= 0: all keys 0..pos.  window > 0: keys pos - window + 1 .. pos.
template <typename T>
__global__ void attention_rows_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                      const T* __restrict__ v_pool, const int* __restrict__ table, int table_width,
                                      int pool_blocks, const int* __restrict__ cu, const int* __restrict__ len_before,
                                      int sequences, int n_tokens, int heads, int kv_heads, int head_dim, float scale,
                                      int window, int splits, T* __restrict__ out, float* __restrict__ part_acc,
                                      float* __restrict__ part_ml, unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float q_shared[];  // ATTN_WARPS * head_dim
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * ATTN_WARPS + warp;  // (token, head)
    if (row >= (long long)n_tokens * heads) return;
    const int t = (int)(row / heads), h = (int)(row - (long long)t * heads);
    const int split = blockIdx.y;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int kh = h / (heads / kv_heads);
    const int* table_row = table + (size_t)b * table_width;

    float* qs = q_shared + warp * head_dim;
    for (int d = lane; d < head_dim; d += 32) qs[d] = tt_to_float(q[((size_t)t * heads + h) * head_dim + d]) * scale;
    __syncwarp();

    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos - first + 1;
    int per = (n_keys + splits - 1) / splits;
    per = (per + 31) & ~31;
    const int begin = first + split * per;
    const int end = min(begin + per, pos + 1);

    float m_run = -INFINITY, l_run = 0.0f;
    float acc[ATTN_MAX_HEAD_DIM / 32];
#pragma unroll
    for (int i = 0; i < ATTN_MAX_HEAD_DIM / 32; ++i) acc[i] = 0.0f;

    for (int base = begin; base < end; base += 32) {
        const int key = base + lane;
        long long off = -1, voff = -1;
        float score = -INFINITY;
        if (key < end) {
            off = tt_cache_offset(table_row, key, kh, kv_heads, head_dim, pool_blocks, status);
            if (off >= 0) {
                score = dot16<T>(k_pool + off, qs, head_dim);
                voff = tt_value_offset(table_row, key, kh, kv_heads, head_dim, pool_blocks, nullptr);
            }
        }
        const float m_tile = tt_warp_max(score);
        if (m_tile == -INFINITY) continue;  // nothing readable in this tile
        const float m_new = fmaxf(m_run, m_tile);
        const float corr = expf(m_run - m_new);  // 0 on the first tile
        const float p = (score == -INFINITY) ? 0.0f : expf(score - m_new);
        l_run = l_run * corr + tt_warp_sum(p);
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < ATTN_MAX_HEAD_DIM / 32; ++i) acc[i] *= corr;
        const int count = min(32, end - base);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long oj = __shfl_sync(0xffffffffu, voff, j);
            if (oj < 0) continue;
            const T* vcol = v_pool + oj;               // dimension d of this key lies d * 64 elements on
#pragma unroll
            for (int i = 0; i < ATTN_MAX_HEAD_DIM / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, tt_to_float(vcol[(size_t)d * TT_BLOCK_TOKENS]), acc[i]);
            }
        }
    }

    if (splits == 1) {
        const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll
        for (int i = 0; i < ATTN_MAX_HEAD_DIM / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) out[((size_t)t * heads + h) * head_dim + d] = tt_from_float<T>(acc[i] * inv);
        }
    } else {
        const size_t slot = ((size_t)t * heads + h) * splits + split;
#pragma unroll
        for (int i = 0; i < ATTN_MAX_HEAD_DIM / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) part_acc[slot * head_dim + d] = acc[i];
        }
        if (lane == 0) {
            part_ml[slot * 2] = m_run;
            part_ml[slot * 2 + 1] = l_run;
        }
    }
}

// out[t, h, :] = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M), M = max_s m_s.
// One warp per row.  Lanes first take one slice each to find M and the weights, then all
// lanes walk the slices' accumulators with independent loads; the additions run in slice
// order, so the result does not depend on the grid.
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                       int splits, int head_dim, long long rows, T* __restrict__ out) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * ATTN_WARPS + warp;
    if (row >= rows) return;
    const float* ml = part_ml + (size_t)row * splits * 2;
    float m = -INFINITY;
    for (int s = lane; s < splits; s += 32) m = fmaxf(m, __ldg(ml + 2 * s));
    m = tt_warp_max(m);
    float l = 0.0f;
    float acc[ATTN_MAX_HEAD_DIM / 32];
#pragma unroll
    for (int i = 0; i < ATTN_MAX_HEAD_DIM / 32; ++i) acc[i] = 0.0f;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        // this lane's slice of the group of 32: its weight and its share of the denominator
        const int mine = s0 + lane;
        float w_mine = 0.0f, l_mine = 0.0f;
        if (mine < splits) {
            const float ms = __ldg(ml + 2 * mine);
            if (ms != -INFINITY) { w_mine = expf(ms - m); l_mine = __ldg(ml + 2 * mine + 1) * w_mine; }
        }
        const int count = min(32, splits - s0);
        for (int j = 0; j < count; ++j) l += __shfl_sync(0xffffffffu, l_mine, j);
#pragma unroll 4
        for (int j = 0; j < count; ++j) {
            const float w = __shfl_sync(0xffffffffu, w_mine, j);
            const float* a = part_acc + ((size_t)row * splits + s0 + j) * head_dim;
#pragma unroll
            for (int i = 0; i < ATTN_MAX_HEAD_DIM / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(__ldg(a + d), w, acc[i]);
            }
        }
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < ATTN_MAX_HEAD_DIM / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) out[(size_t)row * head_dim + d] = tt_from_float<T>(acc[i] * inv);
    }
}

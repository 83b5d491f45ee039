// Causal grouped-query attention over the block cache on tensor cores (mma.sync), bfloat16,
// for head sizes 32, 64, 96 and 128 and up to 16 query heads per key/value head: the decode
// kernel of every such model, and the prompt kernel for the head sizes the tcgen05 kernel
// does not take.
//
// A warp owns a tile of 16 query rows that share one sequence and one key/value head:
// rows are (token, head of the group) pairs, 16 / group tokens by `group` heads, so every
// key and value is read once for the whole group.  The warp walks the sequence's cache
// blocks (64 keys each) within its slice of the keys; per block S = Q K^T and O += P V run
// as m16n8k16 mma.sync with a running softmax in float32.  A decode step has only `group`
// rows per tile, so its products are transposed (16 keys on the rows, the group's queries on
// the 8 columns: key_tile_math), which halves the products and the exponentials.
//
// No ldmatrix and no transposes: both products take their B operand as 16-byte pieces of
// cache rows.  That works because (1) a dot product does not care in which order its terms
// are added, so the k index of each product is permuted such that a thread's four fragment
// registers are 16 contiguous bytes of a cache row (for Q K^T the head dimension is
// permuted identically in Q and K; for P V the key index is permuted identically in P's
// columns and V's rows, by choosing which key each score column stands for), and (2)
// values are stored transposed inside a cache block ([head_dim][64 tokens], see
// common.cuh), which is the "k contiguous" order P V needs.
//
// Two kernels share the per-block arithmetic (block_math).
// Prompts (attention_mma_kernel): the four warps of a CTA hold 64 query rows of one
// sequence and one key/value head; each block's K and V tiles are copied once per CTA into
// shared memory with cp.async, two or three blocks ahead, and every warp takes its
// fragments from there.
// Decoding (attention_decode_kernel): one token per sequence, a tile is one CTA; its warps
// split the tile's blocks of keys among themselves (warp w takes blocks w, w + WARPS, ...).
// The step is bound by reading the cache once.  A block's keys of one head are 8 to 16 KB of
// contiguous memory and so are its values, so a warp asks the copy engine for both
// (cp.async.bulk, completion on an mbarrier per stage) into its own ring of shared-memory
// stages, a block ahead of the arithmetic, and every thread reads its fragments as 16-byte
// pieces of the tiles' rows; copies of blocks that the step does not write start before the
// wait for the previous kernel.  The warps' (max, sum, accumulator) meet in shared memory at
// the end.  grid.z may cut the keys into slices as well: up to 8 slices form a thread-block
// cluster and are combined over distributed shared memory, more leave partial results in
// scratch for the CTA that finishes last (or for attention_merge_kernel).  For head size 64
// the kernel can also do what comes before attention in a step: rotate q and k and write the
// new key and value into the cache (DecodeRope).
//
// Counterparts in random-unknown-username/Thintensor: _single_token_gqa_attention_kernel and
// the split pair, thinruntime/triton_kernels.py:14-245 (one token, one program per query
// head, SIMT); prompts are fed token by token there.
#include "attention_kernels.cuh"
#include "tcgen05.cuh"

#include <cooperative_groups.h>
namespace cg = cooperative_groups;

// Tests of the failure path only: every decode warp's first stage expects this many bytes more than its copies bring, so its
// barrier never completes and the bounded wait has to run out (0 in every real run; handed to the kernel as an argument).
static int decode_undelivered_bytes_for_tests = 0;

namespace {

constexpr int MMA_WARPS = 4;          // warps of a CTA of the prompt kernel

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ uint4 load16(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }

// 2^x on the special-function unit; exact enough for probabilities that are rounded to bfloat16
// (relative error about 2^-22), and 2^-inf = 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Which key of a 64-key block score column n of score tile j stands for (see the header).
__device__ __forceinline__ int key_of(int j, int n) { return 32 * (j >> 2) + 8 * (n >> 1) + 2 * (j & 3) + (n & 1); }

// The rows a thread owns (g and g + 8 of a 16-row tile) and the running softmax state.
template <int HD> struct TileState {
    static constexpr int KC = HD / 32;   // 32-wide chunks of the head dimension
    static constexpr int NT = HD / 8;    // 8-wide output tiles
    uint32_t qa[KC][4], qb[KC][4];       // Q fragments of rows g and g + 8, head dimension permuted
    float o[NT][4];
    float m_run[2], l_run[2];
    int row_pos[2], row_first[2];
};

// One block of 64 keys: S = Q K^T, scale, mask, running softmax, O += P V.
// load_k(j, c) returns the 16 bytes of key key_of(j, g) at dims 32c + 8t .. + 7;
// load_v(n, half) returns the 16 bytes of value dimension 8n + g at keys 32 * half + 8t .. + 7.
template <int HD, typename LoadK, typename LoadV>
__device__ __forceinline__ void block_math(TileState<HD>& st, int key_base, int t, float scale_log2, LoadK load_k, LoadV load_v) {
    constexpr int KC = TileState<HD>::KC, NT = TileState<HD>::NT;
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int c = 0; c < KC; ++c) {
            const uint4 kr = load_k(j, c);
            mma_bf16(s[j], st.qa[c][0], st.qb[c][0], st.qa[c][1], st.qb[c][1], kr.x, kr.y);
            mma_bf16(s[j], st.qa[c][2], st.qb[c][2], st.qa[c][3], st.qb[c][3], kr.z, kr.w);
        }
    }
    // a block whose every key is visible to both rows needs no mask
    const int lo = min(st.row_pos[0], st.row_pos[1]), first = max(st.row_first[0], st.row_first[1]);
    const bool all_visible = key_base + TT_BLOCK_TOKENS - 1 <= lo && key_base >= first;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float mx = -INFINITY;
        if (all_visible) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float v = s[j][2 * i + e] * scale_log2;
                    s[j][2 * i + e] = v;
                    mx = fmaxf(mx, v);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key_base + key_of(j, 2 * t + e);
                    const bool seen = key <= st.row_pos[i] && key >= st.row_first[i];
                    const float v = seen ? s[j][2 * i + e] * scale_log2 : -INFINITY;
                    s[j][2 * i + e] = v;
                    mx = fmaxf(mx, v);
                }
            }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(st.m_run[i], mx);
        const float corr = (m_new == -INFINITY) ? 1.0f : fast_exp2(st.m_run[i] - m_new);
        const float base = (m_new == -INFINITY) ? 0.0f : m_new;
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float p = fast_exp2(s[j][2 * i + e] - base);
                s[j][2 * i + e] = p;
                sum += p;
            }
        }
        st.l_run[i] = st.l_run[i] * corr + sum;
        st.m_run[i] = m_new;
#pragma unroll
        for (int n = 0; n < NT; ++n) { st.o[n][2 * i] *= corr; st.o[n][2 * i + 1] *= corr; }
    }
    uint32_t pa[4][4];
#pragma unroll
    for (int mm = 0; mm < 4; ++mm) {
        pa[mm][0] = pack_bf16(s[2 * mm][0], s[2 * mm][1]);
        pa[mm][1] = pack_bf16(s[2 * mm][2], s[2 * mm][3]);
        pa[mm][2] = pack_bf16(s[2 * mm + 1][0], s[2 * mm + 1][1]);
        pa[mm][3] = pack_bf16(s[2 * mm + 1][2], s[2 * mm + 1][3]);
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint4 vr = load_v(n, half);
            mma_bf16(st.o[n], pa[2 * half][0], pa[2 * half][1], pa[2 * half][2], pa[2 * half][3], vr.x, vr.y);
            mma_bf16(st.o[n], pa[2 * half + 1][0], pa[2 * half + 1][1], pa[2 * half + 1][2], pa[2 * half + 1][3], vr.z, vr.w);
        }
    }
}

// ------------------------------------------------------------------ one token per sequence: keys on the 16-row side
// A decode step has `group` query rows per key/value head (4 in the Llama shapes), so a 16-row tile of queries is
// mostly padding, and mma.sync runs at a small fraction of the tensor cores' rate on this architecture (8 cycles per
// m16n8k16 per SM, measured): with queries on the rows the products of a 64-key block keep the tensor pipe busy for
// 512 cycles per SM, which bounds the step at about 5 TB/s.  Here the products are transposed: S^T = K Q^T has 16 keys
// on the rows and 8 queries on the columns (NQ column tiles for groups of more than 8), O^T = V^T P^T has 16 head
// dimensions on the rows; a block then takes half the products and half the exponentials.  K and V pieces are the
// very same 16 bytes per thread as in block_math (key tile mt, rows g and g + 8, are load_k(2 mt, c) and
// load_k(2 mt + 1, c); dimension tile dt, rows g and g + 8, are load_v(2 dt, half) and load_v(2 dt + 1, half)), so the
// copies into shared memory do not change.  P^T reaches the second product's B operand through movmatrix (an 8 x 8
// transpose across the warp), the one step that the other orientation gets for free.
__device__ __forceinline__ uint32_t transpose_8x8(uint32_t v) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(v));
    return d;
}

template <int HD, int NQ> struct KeyTileState {
    static constexpr int KC = HD / 32, DT = HD / 16;
    uint32_t q[NQ][KC][4];              // this lane's query (8 nq + g), 16 bytes per 32-wide chunk of the head dimension
    float o[DT][NQ][4];                 // [0], [1]: dimension 16 dt + g, queries 8 nq + 2 t and + 1; [2], [3]: dimension + 8
    float m_run[NQ][2], l_run[NQ][2];   // queries 8 nq + 2 t + e; l is this lane's share (its keys) until finish_sums
    int pos, first;                     // the step's token sees keys first .. pos
};

template <int HD, int NQ>
__device__ __forceinline__ void start_queries(KeyTileState<HD, NQ>& st, const __nv_bfloat16* rows, int row_stride, int group, int g, int t,
                                              int pos, int first) {
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq) {
        const int query = 8 * nq + g;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            const uint4 v = query < group ? *reinterpret_cast<const uint4*>(rows + (size_t)query * row_stride + 32 * c + 8 * t) : make_uint4(0, 0, 0, 0);
            st.q[nq][c][0] = v.x; st.q[nq][c][1] = v.y; st.q[nq][c][2] = v.z; st.q[nq][c][3] = v.w;
        }
#pragma unroll
        for (int dt = 0; dt < HD / 16; ++dt) st.o[dt][nq][0] = st.o[dt][nq][1] = st.o[dt][nq][2] = st.o[dt][nq][3] = 0.0f;
        st.m_run[nq][0] = st.m_run[nq][1] = -INFINITY;
        st.l_run[nq][0] = st.l_run[nq][1] = 0.0f;
    }
    st.pos = pos;
    st.first = first;
}

// One block of 64 keys, as four key tiles of 16; load_k and load_v as in block_math.
template <int HD, int NQ, typename LoadK, typename LoadV>
__device__ __forceinline__ void key_tile_math(KeyTileState<HD, NQ>& st, int key_base, int g, int t, float scale_log2,
                                              LoadK load_k, LoadV load_v) {
    constexpr int KC = HD / 32, DT = HD / 16, N_MT = TT_BLOCK_TOKENS / 16;
    float s[N_MT][NQ][4];
#pragma unroll
    for (int m = 0; m < N_MT; ++m) {
#pragma unroll
        for (int nq = 0; nq < NQ; ++nq) s[m][nq][0] = s[m][nq][1] = s[m][nq][2] = s[m][nq][3] = 0.0f;
#pragma unroll
        for (int c = 0; c < KC; ++c) {
            const uint4 ka = load_k(2 * m, c), kb = load_k(2 * m + 1, c);
#pragma unroll
            for (int nq = 0; nq < NQ; ++nq) {
                mma_bf16(s[m][nq], ka.x, kb.x, ka.y, kb.y, st.q[nq][c][0], st.q[nq][c][1]);
                mma_bf16(s[m][nq], ka.z, kb.z, ka.w, kb.w, st.q[nq][c][2], st.q[nq][c][3]);
            }
        }
    }
    if (!(key_base + TT_BLOCK_TOKENS - 1 <= st.pos && key_base >= st.first)) {     // a sequence's end or a window's edge: key by key
#pragma unroll
        for (int m = 0; m < N_MT; ++m)
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) {
                const int key = key_base + key_of(2 * m + hi, g);
                if (!(key <= st.pos && key >= st.first)) {
#pragma unroll
                    for (int nq = 0; nq < NQ; ++nq) s[m][nq][2 * hi] = s[m][nq][2 * hi + 1] = -INFINITY;
                }
            }
    }
    float corr[NQ][2];
    bool grew = false;
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float mx = -INFINITY;
#pragma unroll
            for (int m = 0; m < N_MT; ++m) mx = fmaxf(mx, fmaxf(s[m][nq][e], s[m][nq][2 + e]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(st.m_run[nq][e], mx * scale_log2);     // the scale is positive
            corr[nq][e] = (m_new == -INFINITY) ? 1.0f : fast_exp2(st.m_run[nq][e] - m_new);
            grew = grew || corr[nq][e] != 1.0f;
            const float nbase = (m_new == -INFINITY) ? 0.0f : -m_new;
            float sum = 0.0f;
#pragma unroll
            for (int m = 0; m < N_MT; ++m)
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    const float p = fast_exp2(fmaf(s[m][nq][2 * hi + e], scale_log2, nbase));
                    s[m][nq][2 * hi + e] = p;
                    sum += p;
                }
            st.l_run[nq][e] = st.l_run[nq][e] * corr[nq][e] + sum;
            st.m_run[nq][e] = m_new;
        }
    // the accumulator is rescaled only where some query's maximum has grown (after a sequence's first blocks it rarely does)
    if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
        for (int dt = 0; dt < DT; ++dt)
#pragma unroll
            for (int nq = 0; nq < NQ; ++nq) {
                st.o[dt][nq][0] *= corr[nq][0]; st.o[dt][nq][1] *= corr[nq][1];
                st.o[dt][nq][2] *= corr[nq][0]; st.o[dt][nq][3] *= corr[nq][1];
            }
    }
    uint32_t pb[N_MT][NQ][2];           // P^T as the second product's B operand: keys 2 t, 2 t + 1 (and + 8) of the tile, query g
#pragma unroll
    for (int m = 0; m < N_MT; ++m)
#pragma unroll
        for (int nq = 0; nq < NQ; ++nq) {
            pb[m][nq][0] = transpose_8x8(pack_bf16(s[m][nq][0], s[m][nq][1]));
            pb[m][nq][1] = transpose_8x8(pack_bf16(s[m][nq][2], s[m][nq][3]));
        }
#pragma unroll
    for (int dt = 0; dt < DT; ++dt)
#pragma unroll
        for (int half = 0; half < N_MT / 2; ++half) {
            const uint4 va = load_v(2 * dt, half), vb = load_v(2 * dt + 1, half);
#pragma unroll
            for (int nq = 0; nq < NQ; ++nq) {
                mma_bf16(st.o[dt][nq], va.x, vb.x, va.y, vb.y, pb[2 * half][nq][0], pb[2 * half][nq][1]);
                mma_bf16(st.o[dt][nq], va.z, vb.z, va.w, vb.w, pb[2 * half + 1][nq][0], pb[2 * half + 1][nq][1]);
            }
        }
}

// Every lane's share of the row sums becomes the whole sum (the lanes of one t hold the same queries).
template <int HD, int NQ>
__device__ __forceinline__ void finish_sums(KeyTileState<HD, NQ>& st) {
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float l = st.l_run[nq][e];
            l += __shfl_xor_sync(0xffffffffu, l, 4);
            l += __shfl_xor_sync(0xffffffffu, l, 8);
            l += __shfl_xor_sync(0xffffffffu, l, 16);
            st.l_run[nq][e] = l;
        }
}

template <int HD>
__device__ __forceinline__ void load_queries(TileState<HD>& st, const __nv_bfloat16* __restrict__ q, const size_t (&row_q)[2],
                                             const bool (&row_ok)[2], int t) {
#pragma unroll
    for (int c = 0; c < TileState<HD>::KC; ++c) {
        const uint4 zero = make_uint4(0, 0, 0, 0);
        const uint4 va = row_ok[0] ? load16(q + row_q[0] + 32 * c + 8 * t) : zero;
        const uint4 vb = row_ok[1] ? load16(q + row_q[1] + 32 * c + 8 * t) : zero;
        st.qa[c][0] = va.x; st.qa[c][1] = va.y; st.qa[c][2] = va.z; st.qa[c][3] = va.w;
        st.qb[c][0] = vb.x; st.qb[c][1] = vb.y; st.qb[c][2] = vb.z; st.qb[c][3] = vb.w;
    }
#pragma unroll
    for (int n = 0; n < TileState<HD>::NT; ++n) { st.o[n][0] = st.o[n][1] = st.o[n][2] = st.o[n][3] = 0.0f; }
    st.m_run[0] = st.m_run[1] = -INFINITY;
    st.l_run[0] = st.l_run[1] = 0.0f;
}

// ------------------------------------------------------------------------------ prompts
// Four warps = 64 query rows (16 rows each) of one sequence and one key/value head share
// every block of keys: the block's K and V tiles are copied once per CTA into shared
// memory with cp.async, two or three blocks ahead, and every warp reads its fragments
// from there with 16-byte loads.  A tile row of 128 bytes or a multiple covers all 32
// banks, so the two rows that a quarter-warp touches together would collide; the 16-byte
// chunk index is therefore XOR-ed with 4 on odd rows when it is written and when it is read.
// Heavy tiles (late tokens, many keys) are scheduled first.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// One contiguous piece of global memory into shared memory by the copy engine (both 16-byte aligned, a multiple of 16
// bytes); its bytes are counted on the mbarrier.
__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int HD> struct PromptShape {
    static constexpr int K_ROW = HD * 2;                       // bytes of one key row
    static constexpr bool K_SWIZZLE = (K_ROW % 128) == 0;      // rows that start on the same bank
    static constexpr int TILE_BYTES = 64 * HD * 2;             // one K tile = one V tile
    static constexpr int STAGES = HD <= 64 ? 3 : 2;
};

template <int HD>
__global__ void __launch_bounds__(MMA_WARPS * 32)
attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                     const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ table, int table_width,
                     int pool_blocks, const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                     int heads, int kv_heads, float scale_log2, int window, int tokens_per_tile, int cta_tiles,
                     __nv_bfloat16* __restrict__ out, unsigned* status) {
    using P = PromptShape<HD>;
    constexpr int NT = HD / 8, STAGES = P::STAGES;
    extern __shared__ uint4 stage_mem[];                       // [STAGES][K tile, V tile]
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kh = blockIdx.x;                  // heads on x, tiles on y: every head's heavy tiles are handed out before anybody's light ones
    const int group = heads / kv_heads;
    const int tokens_per_cta = tokens_per_tile * MMA_WARPS;

    // which sequence and which of its CTA tiles: lanes look at 32 sequences at a time, a warp
    // scan of their tile counts finds the owner.  Late tiles of a sequence come first.
    int tile = cta_tiles - 1 - (int)blockIdx.y;
    int b = -1;
    for (int base = 0; base < sequences && b < 0; base += 32) {
        const int mine = base + lane;
        const int count = mine < sequences ? (cu[mine + 1] - cu[mine] + tokens_per_cta - 1) / tokens_per_cta : 0;
        int prefix = count;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, prefix, o);
            if (lane >= o) prefix += up;
        }
        const unsigned owner = __ballot_sync(0xffffffffu, tile < prefix);
        if (owner) {
            const int first = __ffs(owner) - 1;
            b = base + first;
            tile -= __shfl_sync(0xffffffffu, prefix - count, first);
        } else {
            tile -= __shfl_sync(0xffffffffu, prefix, 31);
        }
    }
    if (b < 0) return;                 // a spare CTA (the grid is an upper bound): all its warps leave together
    const int seq_begin = cu[b], seq_new = cu[b + 1] - seq_begin, before = len_before[b];
    const int cta_tok0 = tile * tokens_per_cta;
    const int cta_tokens = min(tokens_per_cta, seq_new - cta_tok0);
    const int tok0 = cta_tok0 + warp * tokens_per_tile;                          // this warp's first token
    const int tile_tokens = max(0, min(tokens_per_tile, seq_new - tok0));       // 0: the warp only helps copying

    TileState<HD> st;
    size_t row_q[2];
    bool row_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        const int local = r / group;
        row_ok[i] = local < tile_tokens;
        const int token = seq_begin + tok0 + local, head = kh * group + (r - local * group);
        row_q[i] = ((size_t)token * heads + head) * HD;
        st.row_pos[i] = row_ok[i] ? before + tok0 + local : -1;
        st.row_first[i] = (window > 0 && st.row_pos[i] - window + 1 > 0) ? st.row_pos[i] - window + 1 : 0;
    }
    load_queries<HD>(st, q, row_q, row_ok, t);

    // blocks of keys: the CTA walks from the first block any of its rows sees to the last; a warp
    // skips the arithmetic of blocks beyond its own last position
    const int cta_lo = before + cta_tok0, cta_hi = before + cta_tok0 + cta_tokens - 1;
    const int lo_key = (window > 0 && cta_lo - window + 1 > 0) ? cta_lo - window + 1 : 0;
    const int block0 = lo_key / TT_BLOCK_TOKENS, block1 = cta_hi / TT_BLOCK_TOKENS;
    const int n_blocks = block1 - block0 + 1;
    const int my_hi = tile_tokens > 0 ? before + tok0 + tile_tokens - 1 : -1;
    const int my_lo = before + tok0;
    const int my_lo_key = (window > 0 && my_lo - window + 1 > 0) ? my_lo - window + 1 : 0;
    const int* table_row = table + (size_t)b * table_width;
    uint8_t* stages = reinterpret_cast<uint8_t*>(stage_mem);
    unsigned bad = 0;                                            // bit i % 32: block i has no usable data

    auto issue = [&](int i) {                                    // all threads: copy block block0 + i into its stage
        if (i < n_blocks) {
            const int block = table_row[block0 + i];
            if (block >= 0 && block < pool_blocks) {
                const uint8_t* ksrc = reinterpret_cast<const uint8_t*>(k_pool + ((size_t)block * kv_heads + kh) * TT_BLOCK_TOKENS * HD);
                const uint8_t* vsrc = reinterpret_cast<const uint8_t*>(v_pool + ((size_t)block * kv_heads + kh) * HD * TT_BLOCK_TOKENS);
                uint8_t* kdst = stages + (size_t)(i % STAGES) * 2 * P::TILE_BYTES;
                uint8_t* vdst = kdst + P::TILE_BYTES;
                constexpr int K_CHUNKS = P::K_ROW / 16;          // 16-byte chunks per key row
                for (int c = threadIdx.x; c < P::TILE_BYTES / 16; c += MMA_WARPS * 32) {
                    const int row = c / K_CHUNKS, ch = c - row * K_CHUNKS;
                    const int to = P::K_SWIZZLE ? (ch ^ ((row & 1) << 2)) : ch;
                    cp_async16(kdst + row * P::K_ROW + to * 16, ksrc + (size_t)c * 16);
                }
                for (int c = threadIdx.x; c < P::TILE_BYTES / 16; c += MMA_WARPS * 32) {
                    const int row = c >> 3, ch = c & 7;          // a value row is 64 tokens = 8 chunks
                    cp_async16(vdst + row * 128 + ((ch ^ ((row & 1) << 2)) * 16), vsrc + (size_t)c * 16);
                }
                bad &= ~(1u << (i & 31));
            } else {
                bad |= 1u << (i & 31);
                if (threadIdx.x == 0) atomicOr(status, TT_STATUS_BAD_BLOCK);
            }
        }
        cp_async_commit();
    };

#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) issue(i);
    for (int i = 0; i < n_blocks; ++i) {
        cp_async_wait<STAGES - 2>();          // this thread's copies of block i are done ...
        __syncthreads();                      // ... and so are everybody's; the stage of block i - 1 is free again
        issue(i + STAGES - 1);
        const int kb = block0 + i;
        if ((bad >> (i & 31)) & 1u) continue;
        if (kb * TT_BLOCK_TOKENS > my_hi || (kb + 1) * TT_BLOCK_TOKENS <= my_lo_key) continue;   // nothing for this warp here
        const uint8_t* ktile = stages + (size_t)(i % STAGES) * 2 * P::TILE_BYTES;
        const uint8_t* vtile = ktile + P::TILE_BYTES;
        block_math<HD>(st, kb * TT_BLOCK_TOKENS, t, scale_log2,
                       [&](int j, int c) {
                           const int row = key_of(j, g), ch = 4 * c + t;
                           const int at = P::K_SWIZZLE ? (ch ^ ((row & 1) << 2)) : ch;
                           return *reinterpret_cast<const uint4*>(ktile + row * P::K_ROW + at * 16);
                       },
                       [&](int n, int half) {
                           const int row = 8 * n + g, ch = 4 * half + t;
                           return *reinterpret_cast<const uint4*>(vtile + row * 128 + ((ch ^ ((row & 1) << 2)) * 16));
                       });
    }
    cp_async_wait<0>();

    // row sums live spread over the four threads of a quad
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        st.l_run[i] += __shfl_xor_sync(0xffffffffu, st.l_run[i], 1);
        st.l_run[i] += __shfl_xor_sync(0xffffffffu, st.l_run[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!row_ok[i]) continue;
        const float inv = st.l_run[i] > 0.0f ? 1.0f / st.l_run[i] : 0.0f;
        __nv_bfloat16* dst = out + row_q[i] + 2 * t;
#pragma unroll
        for (int n = 0; n < NT; ++n)
            *reinterpret_cast<uint32_t*>(dst + 8 * n) = pack_bf16(st.o[n][2 * i] * inv, st.o[n][2 * i + 1] * inv);
    }
}

// ----------------------------------------------------------------------------- decoding

// How many warps share a tile and how many blocks each keeps in flight.  ONE_PER_SM: the slots
// fill an SM, warps * stages * (HD * 256 bytes) <= 192 KB; for grids of at most one CTA per SM.
// Measured on a B200 for head size 64: 6 warps with 2 blocks each beat 4 warps with 3 (more warps
// hide more of the arithmetic's latency; 7 warps gain nothing further).  TWO_PER_SM: half the
// warps and half the shared memory, so that one CTA's start and end run under the other's
// streaming; faster when the grid has several waves, slower when not.  THREE_PER_SM: for grids of
// more than two and at most three CTAs per SM, which then run as one wave instead of two (384
// CTAs of 32 blocks: 1780 -> 1558 us per decode step of the 1B shape).  Other shapes measured for
// the grids of several waves, us per step with 3 x 2 / 2 x 3 / 2 x 2 / 1 x 3 warps x stages: 512
// CTAs 1841 / 1796 / 1865 / 1804; 1,024 CTAs 2913 / 2870 / 2795 / 2855; 256 CTAs of 128 blocks
// 2281 / 2175 / 2658 / 3661 (none better throughout).  Head size 128 with
// one warp per CTA (2 or 3 CTAs per SM) was 18 to 30 % slower per step than one CTA per SM.
constexpr int DECODE_TABLE_CACHE = 1024;     // table entries (64 K tokens) a decode CTA keeps in shared memory
constexpr int ONE_PER_SM = 0, TWO_PER_SM = 1, THREE_PER_SM = 2;
template <int HD, int SHAPE> struct DecodeShape;
template <> struct DecodeShape<32, ONE_PER_SM> { static constexpr int WARPS = 8, STAGES = 3; };
template <> struct DecodeShape<64, ONE_PER_SM> { static constexpr int WARPS = 6, STAGES = 2; };
template <> struct DecodeShape<64, TWO_PER_SM> { static constexpr int WARPS = 3, STAGES = 2; };
template <> struct DecodeShape<64, THREE_PER_SM> { static constexpr int WARPS = 2, STAGES = 2; };
template <> struct DecodeShape<96, ONE_PER_SM> { static constexpr int WARPS = 4, STAGES = 2; };
template <> struct DecodeShape<128, ONE_PER_SM> { static constexpr int WARPS = 3, STAGES = 2; };
template <int HD> constexpr bool decode_has_small_shapes = HD == 64;

// What the fused form of the decode kernel does before attention: the step's q, k and v
// come as float32 slices of the qkv product ([splits][sequences][(heads + 2 kv_heads) * HD]);
// q and k are rotated (all HD numbers of a head, pairs d and d + HD / 2), and the CTA that
// holds a sequence's last block writes k and v into the cache before it reads that block.
struct DecodeRope {
    const float* qkv;
    int splits;
    size_t split_stride;
    const float* inv_freq;
    float attention_scaling;
    int write_cache;
};

// More key slices than a cluster holds: every CTA of a (sequence, kv head) has left its partial result in scratch
// memory; the one that finishes last combines them all, in slice order, so that no merge kernel has to be launched
// and waited for.  A CTA's stores are fenced before it draws its ticket, and the last CTA fences again before it
// reads the others': the usual last-block reduction, without any waiting.
template <int HD>
__device__ __noinline__ void combine_by_last_cta(unsigned* __restrict__ tickets, const float* __restrict__ part_acc,
                                                 const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int b, int kh,
                                                 int heads, int kv_heads, int group, int splits, int threads) {
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* ticket = tickets + (size_t)b * kv_heads + kh;
        const unsigned drawn = atomicAdd(ticket, 1u);
        is_last = drawn == (unsigned)splits - 1u;
        if (is_last) *ticket = 0u;                      // nobody else touches it any more: ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < group * (HD / 2); idx += threads) {
        const int r = idx / (HD / 2), d = 2 * (idx - r * (HD / 2));
        const size_t row_index = (size_t)b * heads + kh * group + r;
        const float* ml = part_ml + row_index * splits * 2;
        const float* acc = part_acc + row_index * splits * HD + d;
        float m = -INFINITY;
#pragma unroll 8
        for (int sl = 0; sl < splits; ++sl) m = fmaxf(m, __ldcg(ml + 2 * sl));
        float l = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
        if (m != -INFINITY) {
#pragma unroll 8
            for (int sl = 0; sl < splits; ++sl) {
                const float2 state = __ldcg(reinterpret_cast<const float2*>(ml + 2 * sl));     // (maximum in natural units, sum)
                const float2 o = __ldcg(reinterpret_cast<const float2*>(acc + (size_t)sl * HD));
                const float weight = state.x == -INFINITY ? 0.0f : expf(state.x - m);
                l = fmaf(state.y, weight, l);
                acc0 = fmaf(o.x, weight, acc0);
                acc1 = fmaf(o.y, weight, acc1);
            }
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        *reinterpret_cast<__nv_bfloat162*>(out + row_index * HD + d) = __floats2bfloat162_rn(acc0 * inv, acc1 * inv);
    }
}

// TICKETS: the instance that can combine more slices than a cluster holds by itself (see combine_by_last_cta).  It
// is a kernel of its own because the mere presence of that path cost the others' main loop 8 to 28 % (measured on a
// B200: 0.853 -> 0.92 ms per step at batch 8, 2.09 -> 2.65 ms with 32,768 cached tokens), whether inlined or not.
template <int HD, bool ROPE, int SHAPE, bool TICKETS = false, int NQ = 1>
__global__ void __launch_bounds__(DecodeShape<HD, SHAPE>::WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, DecodeRope rope, __nv_bfloat16* __restrict__ k_pool,
                        __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ table, int table_width,
                        int pool_blocks, const int* __restrict__ len_before, int heads, int kv_heads, float scale_log2,
                        int window, int splits, int cluster_merge, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ part_acc, float* __restrict__ part_ml, unsigned* __restrict__ tickets, int undelivered_bytes,
                        unsigned* status) {
    constexpr int WARPS = DecodeShape<HD, SHAPE>::WARPS, STAGES = DecodeShape<HD, SHAPE>::STAGES;
    constexpr int TILE = TT_BLOCK_TOKENS * HD * 2;     // bytes of a block's keys of one head, and of its values
    extern __shared__ __align__(128) uint4 slots[];   // [WARPS][STAGES]: a K tile [64 keys][HD], then a V tile [HD][64 keys], as they lie in the cache
    __shared__ uint64_t landed[WARPS][STAGES];        // a stage's two copies have arrived
    tt_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int b = blockIdx.x, kh = blockIdx.y, split = blockIdx.z;
    if (threadIdx.x == 0) {
        for (int w = 0; w < WARPS; ++w)
            for (int s = 0; s < STAGES; ++s) tc::mbar_init(tc::smem_u32(&landed[w][s]), 1);
        tc::fence_barrier_init();
    }
    const int group = heads / kv_heads;
    // Lengths and tables were written before this step's first kernel started (by the step
    // before, or by the host), so they may be read ahead of the wait; so may every block but
    // the one that this step's token goes into.  The sequence's table row goes to shared memory
    // while the length is still on its way, so that no copy has to wait for a table entry.
    __shared__ int table_sh[DECODE_TABLE_CACHE];
    const int* table_row = table + (size_t)b * table_width;
    for (int i = threadIdx.x; i < min(table_width, DECODE_TABLE_CACHE); i += WARPS * 32) table_sh[i] = table_row[i];
    const int pos = len_before[b];                    // position of this step's token = keys 0 .. pos
    __syncthreads();
    const int lo_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int block0 = lo_key / TT_BLOCK_TOKENS, block1 = pos / TT_BLOCK_TOKENS;
    const int per = (block1 - block0 + 1 + splits - 1) / splits;
    const int my_begin = block0 + split * per, my_end = min(block1 + 1, my_begin + per);
    const int n_mine = my_begin + warp < my_end ? (my_end - my_begin - warp + WARPS - 1) / WARPS : 0;   // blocks of this warp
    // block1, if it is this warp's, is its last; it is copied only after the wait
    const int n_early = (n_mine > 0 && my_begin + warp + (n_mine - 1) * WARPS == block1) ? n_mine - 1 : n_mine;
    char* my_slots = reinterpret_cast<char*>(slots) + (size_t)warp * STAGES * 2 * TILE;
    // this lane's 16-byte pieces inside the tiles: key_of(j, g) = key_of(0, g) + 32 (j >> 2) + 2 (j & 3), so every piece
    // lies at a compile-time distance from one address per tile
    const int k_lane = (key_of(0, g) * HD + 8 * t) * 2, v_lane = TILE + (g * TT_BLOCK_TOKENS + 8 * t) * 2;
    unsigned valid = 0;                                // bit i % 32: block i of this warp has usable data
    int issued = 0;                                    // blocks of this warp whose copies have started
    bool waits_ok = true;

    // A block's keys of one head are contiguous in the cache and so are its values: one lane asks the copy engine for
    // both, no thread computes an address per piece, and the load/store unit is left to the fragment reads.
    auto issue_next = [&]() {
        const int i = issued++;
        const int kb = my_begin + warp + i * WARPS;
        const int block = kb < DECODE_TABLE_CACHE ? table_sh[kb] : table_row[kb];
        const bool good = block >= 0 && block < pool_blocks;
        __syncwarp();                                  // every lane has read what the stage held before
        if (lane == 0) {
            const uint32_t bar = tc::smem_u32(&landed[warp][i % STAGES]);
            if (good) {
                const size_t tile = ((size_t)block * kv_heads + kh) * (TT_BLOCK_TOKENS * HD);     // a K tile and a V tile have the same size
                char* dst = my_slots + (size_t)(i % STAGES) * 2 * TILE;
                tc::mbar_expect_tx(bar, 2 * TILE + (i == 0 ? undelivered_bytes : 0));
                bulk_copy(dst, k_pool + tile, TILE, bar);
                bulk_copy(dst + TILE, v_pool + tile, TILE, bar);
            } else {
                tc::mbar_arrive(bar);                  // the stage's phase still ends, so the parities stay in step
                atomicOr(status, TT_STATUS_BAD_BLOCK);
            }
        }
        if (good) valid |= 1u << (i & 31); else valid &= ~(1u << (i & 31));
    };

    while (issued < min(STAGES - 1, n_early)) issue_next();
    tt_pdl_wait();                                     // the queries (or the qkv product) come from the previous kernel

    KeyTileState<HD, NQ> st;
    if constexpr (ROPE) {
        // All threads share the work: one item is a rotated pair (d, d + HD / 2) of a query head
        // or of the new key, or one number of the new value.  Queries go to shared memory, from
        // where every warp takes its fragments; key and value go to the cache.
        constexpr int HALF = HD / 2, PITCH_Q = HD + 8;
        __shared__ __align__(16) __nv_bfloat16 q_sh[16 * PITCH_Q];
        const int q_cols = heads * HD, kv_cols = rope.write_cache ? kv_heads * HD : 0;
        const float* row = rope.qkv + (size_t)b * (q_cols + 2 * kv_cols);
        const bool append = rope.write_cache && my_begin <= block1 && block1 < my_end;   // this CTA reads the new key
        const int pair_rows = group + (append ? 1 : 0);
        const int items = pair_rows * HALF + (append ? HALF : 0);      // the value's numbers go two to an item, like the pairs
        // two numbers HALF apart, each summed over the product's k-slices in slice order; the loads of both and of
        // up to eight slices are in flight together (one loop per number cost a second round trip to the L2)
        auto sum_slices_pair = [&](const float* p, float& first, float& second) {
            float x = 0.0f, y = 0.0f;
#pragma unroll 8
            for (int s = 0; s < rope.splits; ++s) {
                x += __ldg(p + (size_t)s * rope.split_stride);
                y += __ldg(p + HALF + (size_t)s * rope.split_stride);
            }
            first = x;
            second = y;
        };
        long long k_off = -1, v_off = -1;
        if (append) {
            k_off = tt_cache_offset(table_row, pos, kh, kv_heads, HD, pool_blocks, status);
            v_off = tt_value_offset(table_row, pos, kh, kv_heads, HD, pool_blocks, status);
        }
        for (int item = threadIdx.x; item < items; item += WARPS * 32) {
            if (item < pair_rows * HALF) {
                const int r = item / HALF, i = item - r * HALF;
                const float* p = r < group ? row + (size_t)(kh * group + r) * HD + i : row + q_cols + (size_t)kh * HD + i;
                float a, bb;
                sum_slices_pair(p, a, bb);
                float si, co;
                sincosf(rope.inv_freq[i] * (float)pos, &si, &co);
                co *= rope.attention_scaling;
                si *= rope.attention_scaling;
                const __nv_bfloat16 lo = __float2bfloat16_rn(a * co - bb * si), hi = __float2bfloat16_rn(bb * co + a * si);
                if (r < group) {
                    q_sh[r * PITCH_Q + i] = lo;
                    q_sh[r * PITCH_Q + i + HALF] = hi;
                } else if (k_off >= 0) {
                    k_pool[k_off + i] = lo;
                    k_pool[k_off + i + HALF] = hi;
                }
            } else {
                const int d = item - pair_rows * HALF;
                const float* p = row + q_cols + kv_cols + (size_t)kh * HD + d;
                float a, bb;
                sum_slices_pair(p, a, bb);
                if (v_off >= 0) {
                    v_pool[v_off + (long long)d * TT_BLOCK_TOKENS] = __float2bfloat16_rn(a);
                    v_pool[v_off + (long long)(d + HALF) * TT_BLOCK_TOKENS] = __float2bfloat16_rn(bb);
                }
            }
        }
        if (append) {                                  // key and value are in memory, and visible to the copy engine, before their block is copied
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");
        }
        __syncthreads();
        start_queries<HD, NQ>(st, q_sh, PITCH_Q, group, g, t, pos, lo_key);
    } else {
        start_queries<HD, NQ>(st, q + ((size_t)b * heads + kh * group) * HD, HD, group, g, t, pos, lo_key);
    }

    int waited = 0;                                    // blocks of this warp whose copies have been waited for
    for (int i = 0; i < n_mine; ++i) {
        while (issued < min(n_mine, i + STAGES)) issue_next();     // block i and up to STAGES - 1 beyond it
        if (waits_ok && !tc::mbar_wait(tc::smem_u32(&landed[warp][i % STAGES]), (uint32_t)((i / STAGES) & 1))) {
            if (lane == 0) atomicOr(status, TT_STATUS_WAIT_EXPIRED);
            waits_ok = false;
        }
        waited = i + 1;
        if (!waits_ok) break;
        if (!((valid >> (i & 31)) & 1u)) continue;
        const char* src = my_slots + (size_t)(i % STAGES) * 2 * TILE;
        const int kb = my_begin + warp + i * WARPS;
        key_tile_math<HD, NQ>(st, kb * TT_BLOCK_TOKENS, g, t, scale_log2,
                              [&](int j, int c) { return *reinterpret_cast<const uint4*>(src + k_lane + ((32 * (j >> 2) + 2 * (j & 3)) * HD * 2 + 64 * c)); },
                              [&](int n, int half) { return *reinterpret_cast<const uint4*>(src + v_lane + (n * 8 * TT_BLOCK_TOKENS * 2 + 64 * half)); });
    }
    // after a wait that ran out: the copies still under way get one more bounded wait each before shared memory is reused
    for (int i = waited; i < issued; ++i) tc::mbar_wait(tc::smem_u32(&landed[warp][i % STAGES]), (uint32_t)((i / STAGES) & 1));
    finish_sums<HD, NQ>(st);

    // the warps' partial results meet in shared memory (the slots are free now)
    __syncthreads();
    constexpr int PITCH = HD + 4;
    float* sh_o = reinterpret_cast<float*>(slots);     // [WARPS][16][PITCH]
    float* sh_m = sh_o + WARPS * 16 * PITCH;           // [WARPS][16]
    float* sh_l = sh_m + WARPS * 16;
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = 8 * nq + 2 * t + e;
            float* dst = sh_o + ((size_t)warp * 16 + r) * PITCH + g;
#pragma unroll
            for (int dt = 0; dt < HD / 16; ++dt) { dst[16 * dt] = st.o[dt][nq][e]; dst[16 * dt + 8] = st.o[dt][nq][2 + e]; }
            if (g == 0) { sh_m[warp * 16 + r] = st.m_run[nq][e]; sh_l[warp * 16 + r] = st.l_run[nq][e]; }
        }
    __syncthreads();
    // cluster_merge: the slices of a (sequence, kv head) form a thread-block cluster; each leaves its
    // result in its own shared memory and the CTAs combine them over distributed shared memory
    float* cta_acc = sh_l + WARPS * 16;                // [16][HD]
    float* cta_ml = cta_acc + 16 * HD;                 // [16][2]
    // one item = two neighbouring numbers of one row
    for (int idx = threadIdx.x; idx < group * (HD / 2); idx += WARPS * 32) {
        const int r = idx / (HD / 2), d = 2 * (idx - r * (HD / 2));
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sh_m[w * 16 + r]);
        float l = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
        if (m != -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float weight = exp2f(sh_m[w * 16 + r] - m);       // 0 for a warp that saw no key
                const float2 o = *reinterpret_cast<const float2*>(sh_o + ((size_t)w * 16 + r) * PITCH + d);
                l = fmaf(sh_l[w * 16 + r], weight, l);
                acc0 = fmaf(o.x, weight, acc0);
                acc1 = fmaf(o.y, weight, acc1);
            }
        }
        const size_t row_index = (size_t)b * heads + kh * group + r;
        if (splits == 1) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            *reinterpret_cast<__nv_bfloat162*>(out + row_index * HD + d) = __floats2bfloat162_rn(acc0 * inv, acc1 * inv);
        } else if (cluster_merge) {
            *reinterpret_cast<float2*>(cta_acc + r * HD + d) = make_float2(acc0, acc1);
            if (d == 0) { cta_ml[2 * r] = m; cta_ml[2 * r + 1] = l; }
        } else {
            const size_t slot = row_index * splits + split;
            *reinterpret_cast<float2*>(part_acc + slot * HD + d) = make_float2(acc0, acc1);
            if (d == 0) {
                part_ml[slot * 2] = m * 0.6931471805599453f;            // the merge works with natural exponents
                part_ml[slot * 2 + 1] = l;
            }
        }
    }
    if constexpr (TICKETS) {
        if (splits > 1 && !cluster_merge && tickets)
            combine_by_last_cta<HD>(tickets, part_acc, part_ml, out, b, kh, heads, kv_heads, group, splits, WARPS * 32);
    }
    if (splits > 1 && cluster_merge) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                                // every slice's result is in its shared memory
        // every CTA of the cluster combines the rows rank, rank + splits, ... and stores them
        const int rank = (int)cluster.block_rank();
        const int my_rows = rank < group ? (group - rank + splits - 1) / splits : 0;
        for (int idx = threadIdx.x; idx < my_rows * (HD / 2); idx += WARPS * 32) {
            const int r = rank + (idx / (HD / 2)) * splits, d = 2 * (idx % (HD / 2));
            float m = -INFINITY;
            for (int s = 0; s < splits; ++s) m = fmaxf(m, cluster.map_shared_rank(cta_ml, s)[2 * r]);
            float l = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
            if (m != -INFINITY) {
                for (int s = 0; s < splits; ++s) {
                    const float* ml = cluster.map_shared_rank(cta_ml, s);
                    const float weight = exp2f(ml[2 * r] - m);         // 0 for a slice that saw no key
                    const float2 o = *reinterpret_cast<const float2*>(cluster.map_shared_rank(cta_acc, s) + r * HD + d);
                    l = fmaf(ml[2 * r + 1], weight, l);
                    acc0 = fmaf(o.x, weight, acc0);
                    acc1 = fmaf(o.y, weight, acc1);
                }
            }
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)b * heads + kh * group + r) * HD + d) = __floats2bfloat162_rn(acc0 * inv, acc1 * inv);
        }
        cluster.sync();                                // no slice leaves while its shared memory is being read
    }
}

// Up to 8 slices (the portable cluster size) are combined inside the decode kernel by a
// thread-block cluster; more go through scratch memory and the merge kernel.
inline bool slices_form_cluster(int splits) { return splits > 1 && splits <= 8; }

// The decode kernel, plain (ROPE = false: rotated queries in q, the cache already holds the
// step's keys and values) or fused with the rotation and the cache write.
template <int HD, bool ROPE, int SHAPE, int NQ>
cudaError_t launch_decode_tiles(const void* q, const DecodeRope& rope, void* k_pool, void* v_pool, const int* table, int table_width,
                                int pool_blocks, const int* len_before, int sequences, int heads, int kv_heads, float scale_log2,
                                int window, int splits, void* out, float* part_acc, float* part_ml, unsigned* tickets, unsigned* status,
                                cudaStream_t stream) {
    using D = DecodeShape<HD, SHAPE>;
    constexpr int shared = D::WARPS * D::STAGES * (8 * (HD / 32) + (HD / 8) * 2) * 32 * 16;
    static_assert(shared >= D::WARPS * 16 * (HD + 6) * 4 + 16 * (HD + 2) * 4, "the slots must also hold the warps' and the CTA's partial results");
    if constexpr (SHAPE == ONE_PER_SM) {
        if (tickets && splits > 1 && !slices_form_cluster(splits)) {
            static bool configured_tickets = false;
            auto with_tickets = attention_decode_kernel<HD, ROPE, SHAPE, true, NQ>;
            if (!configured_tickets) {
                const cudaError_t err = cudaFuncSetAttribute(with_tickets, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
                if (err != cudaSuccess) return err;
                configured_tickets = true;
            }
            return tt_launch_pdl(with_tickets, dim3(sequences, kv_heads, splits), dim3(D::WARPS * 32), shared, stream,
                (const __nv_bfloat16*)q, rope, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks,
                len_before, heads, kv_heads, scale_log2, window, splits, 0, (__nv_bfloat16*)out, part_acc, part_ml, tickets, decode_undelivered_bytes_for_tests, status);
        }
    }
    static bool configured = false;
    auto kernel = attention_decode_kernel<HD, ROPE, SHAPE, false, NQ>;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
        if (err != cudaSuccess) return err;
        configured = true;
    }
    if (slices_form_cluster(splits))
        return tt_launch_pdl_cluster(kernel, dim3(sequences, kv_heads, splits), dim3(D::WARPS * 32), shared, stream, (unsigned)splits,
            (const __nv_bfloat16*)q, rope, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks,
            len_before, heads, kv_heads, scale_log2, window, splits, 1, (__nv_bfloat16*)out, part_acc, part_ml, tickets, decode_undelivered_bytes_for_tests, status);
    return tt_launch_pdl(kernel, dim3(sequences, kv_heads, splits), dim3(D::WARPS * 32), shared, stream,
        (const __nv_bfloat16*)q, rope, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks,
        len_before, heads, kv_heads, scale_log2, window, splits, 0, (__nv_bfloat16*)out, part_acc, part_ml, tickets, decode_undelivered_bytes_for_tests, status);
}

// One column tile of 8 queries serves groups of up to 8 query heads per key/value head, two serve up to 16.
template <int HD, bool ROPE, int SHAPE = ONE_PER_SM>
cudaError_t launch_decode(const void* q, const DecodeRope& rope, void* k_pool, void* v_pool, const int* table, int table_width,
                          int pool_blocks, const int* len_before, int sequences, int heads, int kv_heads, float scale_log2,
                          int window, int splits, void* out, float* part_acc, float* part_ml, unsigned* tickets, unsigned* status,
                          cudaStream_t stream) {
    if (heads / kv_heads > 8)
        return launch_decode_tiles<HD, ROPE, SHAPE, 2>(q, rope, k_pool, v_pool, table, table_width, pool_blocks, len_before, sequences, heads,
                                                       kv_heads, scale_log2, window, splits, out, part_acc, part_ml, tickets, status, stream);
    return launch_decode_tiles<HD, ROPE, SHAPE, 1>(q, rope, k_pool, v_pool, table, table_width, pool_blocks, len_before, sequences, heads,
                                                   kv_heads, scale_log2, window, splits, out, part_acc, part_ml, tickets, status, stream);
}

template <int HD>
int merge_slices(int n_rows_tokens, int heads, int splits, void* out, float* part_acc, float* part_ml, cudaStream_t stream,
                 bool inside_kernel = false) {
    if (splits > 1 && !inside_kernel) {
        const long long rows = (long long)n_rows_tokens * heads;
        tt_launch_pdl(attention_merge_kernel<__nv_bfloat16>, dim3((unsigned)((rows + ATTN_WARPS - 1) / ATTN_WARPS)), dim3(ATTN_WARPS * 32), 0, stream,
            part_acc, part_ml, splits, HD, rows, (__nv_bfloat16*)out);
    }
    return (int)cudaGetLastError();
}

template <int HD>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* table, int table_width, int pool_blocks,
           const int* cu, const int* len_before, int sequences, int n_tokens, int heads, int kv_heads, float scale,
           int window, int splits, int one_token_each, void* out, float* part_acc, float* part_ml, unsigned* tickets, unsigned* status,
           cudaStream_t stream) {
    const int group = heads / kv_heads;
    const float scale_log2 = scale * 1.4426950408889634f;
    cudaError_t err;
    if (one_token_each) {
        static int sm_count = 0;
        if (sm_count == 0) {
            int device = 0;
            if ((err = cudaGetDevice(&device)) != cudaSuccess) return (int)err;
            if ((err = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return (int)err;
        }
        const long long ctas = (long long)sequences * kv_heads * splits;
        if (ctas > sm_count) tickets = nullptr;         // several CTAs per SM: the variants without tickets, and the merge kernel
        bool done = false;
        if constexpr (decode_has_small_shapes<HD>) {
            if (ctas > 2 * sm_count && ctas <= 3 * sm_count) {          // one wave of three CTAs per SM
                err = launch_decode<HD, false, THREE_PER_SM>(q, DecodeRope{}, const_cast<void*>(k_pool), const_cast<void*>(v_pool), table,
                                                             table_width, pool_blocks, len_before, sequences, heads, kv_heads, scale_log2,
                                                             window, splits, out, part_acc, part_ml, tickets, status, stream);
                done = true;
            } else if (ctas > sm_count) {                               // several waves
                err = launch_decode<HD, false, TWO_PER_SM>(q, DecodeRope{}, const_cast<void*>(k_pool), const_cast<void*>(v_pool), table,
                                                           table_width, pool_blocks, len_before, sequences, heads, kv_heads, scale_log2,
                                                           window, splits, out, part_acc, part_ml, tickets, status, stream);
                done = true;
            }
        }
        if (!done)
            err = launch_decode<HD, false>(q, DecodeRope{}, const_cast<void*>(k_pool), const_cast<void*>(v_pool), table, table_width,
                                           pool_blocks, len_before, sequences, heads, kv_heads, scale_log2, window, splits, out,
                                           part_acc, part_ml, tickets, status, stream);
    } else {
        // packed prompts: keys are not sliced (a prompt has tiles enough); a CTA is 64 query rows
        if (splits != 1) return (int)cudaErrorInvalidValue;
        using P = PromptShape<HD>;
        constexpr int shared = P::STAGES * 2 * P::TILE_BYTES;
        static bool configured = false;
        auto kernel = attention_mma_kernel<HD>;
        if (!configured) {
            err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
            if (err != cudaSuccess) return (int)err;
            configured = true;
        }
        const int tokens_per_tile = 16 / group;
        const int tokens_per_cta = tokens_per_tile * MMA_WARPS;
        const int cta_tiles = (n_tokens + tokens_per_cta - 1) / tokens_per_cta + sequences;   // upper bound; spare CTAs leave at once
        if (cta_tiles > 65535) return (int)cudaErrorInvalidValue;                             // the grid's y extent; steps are cut into pieces long before
        err = tt_launch_pdl(kernel, dim3(kv_heads, cta_tiles, 1), dim3(MMA_WARPS * 32), shared, stream,
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu,
            len_before, sequences, heads, kv_heads, scale_log2, window, tokens_per_tile, cta_tiles, (__nv_bfloat16*)out, status);
    }
    if (err != cudaSuccess) return (int)err;
    return merge_slices<HD>(n_tokens, heads, splits, out, part_acc, part_ml, stream, one_token_each && (slices_form_cluster(splits) || tickets));
}

}  // namespace

// For tests of the failure path, never for serving: the limit of the decode kernel's bounded waits (0: the default of two
// seconds) and bytes that every warp's first stage expects beyond what its copies bring (0: normal operation).
extern "C" int tt_attention_mma_failure_drill(unsigned long long wait_limit_ns, int undelivered_bytes) {
    const int code = tc::set_wait_limit_ns(wait_limit_ns);
    if (code != 0) return code;
    decode_undelivered_bytes_for_tests = undelivered_bytes < 0 ? 0 : undelivered_bytes;
    return 0;
}

// one_token_each: 0 = packed prompts (any number of tokens per sequence); 1 = every
// sequence brings exactly one token (n_tokens == sequences) and the decode kernel runs.
// tickets: null, or sequences * kv_heads words that are zero (and are zero again when the kernel is done): with
// more slices than a cluster holds, the CTA that finishes last for a (sequence, kv head) then combines the
// slices itself and no merge kernel is launched.
// 1 if this kernel takes the sizes, 0 if the exact kernel has to serve them.
extern "C" int tt_attention_mma_supports(int heads, int kv_heads, int head_dim) {
    if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16) return 0;
    return head_dim == 32 || head_dim == 64 || head_dim == 96 || head_dim == 128;
}

extern "C" int tt_attention_mma(const void* q, const void* k_pool, const void* v_pool, const int* table, int table_width,
                                int pool_blocks, const int* cu, const int* len_before, int sequences, int n_tokens,
                                int heads, int kv_heads, int head_dim, float scale, int window, int splits,
                                int one_token_each, void* out, float* part_acc, float* part_ml, unsigned* tickets, unsigned* status,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!tt_attention_mma_supports(heads, kv_heads, head_dim) || splits < 1 || splits > 65535 || kv_heads > 65535)
        return (int)cudaErrorInvalidValue;
    if (splits > 1 && (!part_acc || !part_ml)) return (int)cudaErrorInvalidValue;
#define TT_LAUNCH(HD) return launch<HD>(q, k_pool, v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, scale, window, splits, one_token_each, out, part_acc, part_ml, tickets, status, stream)
    switch (head_dim) {
        case 32: TT_LAUNCH(32);
        case 64: TT_LAUNCH(64);
        case 96: TT_LAUNCH(96);
        default: TT_LAUNCH(128);
    }
#undef TT_LAUNCH
}

// Decoding with the rotation and the cache write inside the attention kernel: takes the
// float32 slices of the qkv product instead of rotated queries.  For bfloat16 caches, head
// size 64 rotated whole (rotary_dim == head_dim), one token per sequence.  (Head size 128 was
// measured slower this way than with the separate kernel: its CTAs have 96 threads for the
// rotation, and the copies in flight leave no room for more.)
// write_cache = 0: the product holds queries only and the cache is read as it is.
// 1 if the sizes are taken, 0 if rope_append and the plain kernel have to serve them.
extern "C" int tt_attention_decode_rope_supports(int heads, int kv_heads, int head_dim, int rotary_dim) {
    if (!tt_attention_mma_supports(heads, kv_heads, head_dim)) return 0;
    return head_dim == 64 && rotary_dim == head_dim;
}

extern "C" int tt_attention_decode_rope(const float* qkv, int qkv_splits, long long split_stride, const float* inv_freq,
                                        int rotary_dim, float attention_scaling, int write_cache, void* k_pool, void* v_pool,
                                        const int* table, int table_width, int pool_blocks, const int* len_before,
                                        int sequences, int heads, int kv_heads, int head_dim, float scale, int window,
                                        int splits, void* out, float* part_acc, float* part_ml, unsigned* tickets, unsigned* status,
                                        cudaStream_t stream) {
    if (sequences <= 0) return 0;
    if (!tt_attention_decode_rope_supports(heads, kv_heads, head_dim, rotary_dim) || splits < 1 || splits > 65535 || kv_heads > 65535 ||
        qkv_splits < 1 || split_stride % 4 != 0 || ((uintptr_t)qkv & 15) != 0)
        return (int)cudaErrorInvalidValue;
    if (splits > 1 && (!part_acc || !part_ml)) return (int)cudaErrorInvalidValue;
    const DecodeRope rope{qkv, qkv_splits, (size_t)split_stride, inv_freq, attention_scaling, write_cache};
    const float scale_log2 = scale * 1.4426950408889634f;
    const cudaError_t err = launch_decode<64, true>(nullptr, rope, k_pool, v_pool, table, table_width, pool_blocks, len_before, sequences,
                                                    heads, kv_heads, scale_log2, window, splits, out, part_acc, part_ml, tickets, status, stream);
    if (err != cudaSuccess) return (int)err;
    return merge_slices<64>(sequences, heads, splits, out, part_acc, part_ml, stream, slices_form_cluster(splits) || tickets);
}

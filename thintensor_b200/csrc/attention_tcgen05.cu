// Causal grouped-query attention for prompts on the 5th-generation tensor cores: both
// products of every block of 64 keys (S = Q K^T and O += P V) are tcgen05.mma with their
// accumulators in tensor memory, operands arrive by TMA, and the softmax between them runs
// in registers with one thread per query row.  bfloat16, head size 64 or 128.
//
// A CTA owns 128 query rows of one sequence and one key/value head: 128 / group tokens by
// `group` heads, fetched as one 3-D TMA box from q [token][head][dim].  Per block of keys:
//   warp 0 (one thread)  looks the block up in the table and issues TMA loads of the K tile
//                        [64 keys][dim] and of the V tile, which the cache stores transposed
//                        ([dim][64 keys], see common.cuh): both are "k contiguous" B operands
//                        exactly as they lie in the cache;
//   warp 1 (one thread)  issues S_i = Q K_i^T (M 128, N 64) into one of two S accumulators as
//                        soon as K_i has landed, and O += P_i V_i (M 128, N dim, A operand in
//                        tensor memory) once the softmax warps have written P_i, so S_{i+1} is
//                        computed while softmax_i runs and P_i V_i while softmax_{i+1} runs;
//   warps 2-5 (2-9)      read a row of S per thread (tcgen05.ld, no shuffles needed for the
//                        row maximum and sum; head size 128: two threads per row, 32 scores each,
//                        which exchange their maxima), scale, mask the diagonal blocks, exponentiate,
//                        and write P back to tensor memory as bfloat16 pairs (tcgen05.st), one
//                        of two buffers: P never passes through shared memory, which took a
//                        third of a block's time when it did (stores, proxy fence).  O stays
//                        in tensor memory; it is rescaled only when a row's maximum has grown
//                        by more than 2^8 since the scale in use (then the warp reads, scales
//                        and writes back its 32 rows of O), otherwise the old scale stays.
// At the end every thread divides its row of O by the row sum and stores it.
// Every wait is bounded as in gemm_tcgen05.cu.
//
// The reference has no counterpart: it feeds prompts token by token through its
// single-token attention (thinruntime/cli.py:2802-2807, thinruntime/triton_kernels.py:14-109).
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int ROWS = 128;            // query rows of a CTA
constexpr int KEYS = TT_BLOCK_TOKENS;
constexpr int KV_STAGES = 3;
constexpr float RESCALE_THRESHOLD = 8.0f;     // in log2 units

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two float32 numbers in one 64-bit register and the packed arithmetic of sm_100 on them: one issue slot for two
// results.  The softmax threads' time goes to issue slots and to the special-function unit, not to anything else.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

template <int HD> struct Layout {
    // Threads per query row in the softmax.  Head size 128 leaves room for one CTA per SM only, and
    // four softmax warps cannot hide their own latencies: two threads per row (8 warps) are 10 %
    // faster there.  Head size 64 runs two CTAs per SM and is bound elsewhere: one thread per row.
    static constexpr int SPLIT = HD == 128 ? 2 : 1;
    static constexpr int THREADS = 64 + SPLIT * ROWS;
    static constexpr int CHUNKS = HD / 64;                      // 64-wide slices of the head dimension
    static constexpr int Q_BYTES = ROWS * HD * 2;
    static constexpr int K_BYTES = KEYS * HD * 2;               // = V tile
    static constexpr int STAGE_BYTES = 2 * K_BYTES;
    static constexpr int SMEM = Q_BYTES + KV_STAGES * STAGE_BYTES + 1024;
    static constexpr int O_COL = 128;                           // S: 2 x 64 columns, then O: HD, then P: 2 x 32 (bfloat16 pairs)
    static constexpr int P_COL = O_COL + HD;
    static constexpr int TMEM_COLS = HD == 64 ? 256 : 512;
};

struct Args {
    const int* table;
    int table_width, pool_blocks;
    const int* cu;
    const int* len_before;
    int sequences, heads, kv_heads, group, tokens_per_tile, cta_tiles;
    float scale_log2;
    int window;
    __nv_bfloat16* out;
    unsigned* status;
};

template <int HD>
__global__ void __launch_bounds__(Layout<HD>::THREADS, HD == 64 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const Args args) {
    using L = Layout<HD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem;
    uint8_t* kv_smem = q_smem + L::Q_BYTES;
    __shared__ uint64_t q_full, kv_full[KV_STAGES], kv_empty[KV_STAGES], s_full[2], p_ready[2], pv_done[2];
    __shared__ uint32_t tmem_base_shared;
    __shared__ int tile_info[2];                                  // sequence, tile within the sequence
    __shared__ float pair_max[2][2][ROWS];

    tt_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The grid is (kv heads, tiles) and blocks are handed out with x running fastest: the heaviest tile of every
    // head comes first, then the next heaviest of every head, so the CTAs that start last are the lightest ones
    // (with the heads on y, whole heads, heavy tiles included, started behind others' light tiles).
    const int kh = blockIdx.x;

    if (warp == 0) {
        // which sequence and which of its tiles (late tiles, which see most keys, first)
        int tile = args.cta_tiles - 1 - (int)blockIdx.y;
        int b = -1;
        for (int base = 0; base < args.sequences && b < 0; base += 32) {
            const int mine = base + lane;
            const int count = mine < args.sequences ? (args.cu[mine + 1] - args.cu[mine] + args.tokens_per_tile - 1) / args.tokens_per_tile : 0;
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
        if (lane == 0) { tile_info[0] = b; tile_info[1] = tile; }
    }
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), 1);
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(smem_u32(&kv_full[s]), 1); mbar_init(smem_u32(&kv_empty[s]), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&s_full[i]), 1); mbar_init(smem_u32(&p_ready[i]), 4 * L::SPLIT); mbar_init(smem_u32(&pv_done[i]), 1); }
        fence_barrier_init();
    }
    __syncthreads();
    const int b = tile_info[0], tile = tile_info[1];
    if (b < 0) return;                                            // a spare CTA: everybody leaves before tensor memory is touched
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_shared), L::TMEM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_shared;

    // offsets and lengths were written before the step's first kernel started: the tile's place is found ahead of the wait
    const int seq_begin = args.cu[b], seq_new = args.cu[b + 1] - seq_begin, before = args.len_before[b];
    const int tok0 = tile * args.tokens_per_tile;
    const int tile_tokens = min(args.tokens_per_tile, seq_new - tok0);
    const int lo_pos = before + tok0, hi_pos = before + tok0 + tile_tokens - 1;
    const int lo_key = (args.window > 0 && lo_pos - args.window + 1 > 0) ? lo_pos - args.window + 1 : 0;
    const int block0 = lo_key / KEYS, block1 = hi_pos / KEYS;
    const int n_blocks = block1 - block0 + 1;
    tt_pdl_wait();                                                // queries and this step's keys come from the previous kernel

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint32_t qbar = smem_u32(&q_full);
            // the box holds group * tokens_per_tile rows (128, or a few less when the group does not divide 128)
            mbar_expect_tx(qbar, (uint32_t)(L::CHUNKS * args.group * args.tokens_per_tile * 128));
#pragma unroll
            for (int c = 0; c < L::CHUNKS; ++c)
                tma_load_3d(smem_u32(q_smem + c * ROWS * 128), &map_q, c * 64, kh * args.group, seq_begin + tok0, qbar);
            const int* table_row = args.table + (size_t)b * args.table_width;
            int issued = 0;
            for (int i = 0; i < n_blocks; ++i) {
                const int s = i % KV_STAGES;
                if (i >= KV_STAGES && !mbar_wait(smem_u32(&kv_empty[s]), (uint32_t)(((i / KV_STAGES) & 1) ^ 1))) {
                    atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); break;
                }
                int block = table_row[block0 + i];
                if (block < 0 || block >= args.pool_blocks) { atomicOr(args.status, TT_STATUS_BAD_BLOCK); block = 0; }
                const uint32_t bar = smem_u32(&kv_full[s]);
                mbar_expect_tx(bar, L::STAGE_BYTES);
                uint8_t* stage = kv_smem + (size_t)s * L::STAGE_BYTES;
                const int k_row = (block * args.kv_heads + kh) * KEYS, v_row = (block * args.kv_heads + kh) * HD;
#pragma unroll
                for (int c = 0; c < L::CHUNKS; ++c) tma_load_2d(smem_u32(stage + c * KEYS * 128), &map_k, c * 64, k_row, bar);
                tma_load_2d(smem_u32(stage + L::K_BYTES), &map_v, 0, v_row, bar);
                ++issued;
            }
            for (int i = max(0, issued - KV_STAGES); i < issued; ++i)       // drain before shared memory is given up
                if (!mbar_wait(smem_u32(&kv_full[i % KV_STAGES]), (uint32_t)((i / KV_STAGES) & 1))) { atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); break; }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc(ROWS, KEYS), idesc_o = instr_desc(ROWS, HD);
            bool ok = mbar_wait(smem_u32(&q_full), 0);
            if (!ok) atomicOr(args.status, TT_STATUS_WAIT_EXPIRED);
            auto issue_s = [&](int i) {                           // S_i = Q K_i^T into S accumulator i & 1
                const int s = i % KV_STAGES;
                if (!mbar_wait(smem_u32(&kv_full[s]), (uint32_t)((i / KV_STAGES) & 1))) { atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; return; }
                fence_after_sync();
                const uint32_t q_addr = smem_u32(q_smem), k_addr = smem_u32(kv_smem + (size_t)s * L::STAGE_BYTES);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t off_q = (kk / 4) * ROWS * 128 + (kk % 4) * 32, off_k = (kk / 4) * KEYS * 128 + (kk % 4) * 32;
                    umma_bf16(tmem_base + (i & 1) * 64, smem_desc(q_addr + off_q), smem_desc(k_addr + off_k), idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(smem_u32(&s_full[i & 1]));
            };
            if (ok) issue_s(0);
            if (ok && n_blocks > 1) issue_s(1);
            for (int i = 0; i < n_blocks && ok; ++i) {
                // O += P_i V_i once the softmax warps have written P_i
                if (!mbar_wait(smem_u32(&p_ready[i & 1]), (uint32_t)((i >> 1) & 1))) { atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; break; }
                fence_after_sync();
                const int s = i % KV_STAGES;
                const uint32_t p_tmem = tmem_base + L::P_COL + (i & 1) * 32;
                const uint32_t v_addr = smem_u32(kv_smem + (size_t)s * L::STAGE_BYTES + L::K_BYTES);
#pragma unroll
                for (int kk = 0; kk < KEYS / 16; ++kk)
                    umma_bf16_a_in_tmem(tmem_base + L::O_COL, p_tmem + kk * 8, smem_desc(v_addr + kk * 32), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(smem_u32(&kv_empty[s]));              // K_i and V_i are free once these products are done
                umma_commit(smem_u32(&pv_done[i & 1]));
                if (i + 2 < n_blocks) issue_s(i + 2);             // its S accumulator was read before P_i was announced
            }
        }
    } else {
        // ------------------------------------------------------------ softmax: SPLIT threads per query row
        // With two: warps 2-5 take keys 0..31 of a block, warps 6-9 keys 32..63; the two threads of a row
        // sit in warps with the same index modulo 4 (the tensor-memory lanes a warp may read), exchange
        // their maxima through shared memory at a named barrier of their own, keep separate sums, and
        // share the columns of O between them.  After a failed wait a thread keeps walking through the
        // barriers (without waiting for anything else), so its partner is never left alone at one.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const int local = r / args.group;
        const bool row_ok = local < tile_tokens;
        const int pos = row_ok ? before + tok0 + local : -1;
        const int first = (args.window > 0 && pos - args.window + 1 > 0) ? pos - args.window + 1 : 0;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        constexpr int SPLIT = L::SPLIT, HALF_KEYS = KEYS / SPLIT, O_COLS = HD / SPLIT;   // what one thread of a row handles
        float m_used = -INFINITY, l = 0.0f;                       // the scale in use (log2 units) and this thread's part of the sum
        bool ok = true;
        auto pair_barrier = [&]() { if (SPLIT == 2) asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); };
        auto expired = [&]() { if (lane == 0) atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; };
        for (int i = 0; i < n_blocks; ++i) {
            if (ok && !mbar_wait(smem_u32(&s_full[i & 1]), (uint32_t)((i >> 1) & 1))) expired();
            fence_after_sync();
            float s[HALF_KEYS];
            {
                // both halves of the row are asked for before either is waited for (one round trip to tensor memory, not two)
                uint32_t raw[HALF_KEYS / 32][32];
#pragma unroll
                for (int c = 0; c < HALF_KEYS / 32; ++c) tmem_load32_issue(lane_base + (i & 1) * 64 + half * HALF_KEYS + 32 * c, raw[c]);
                tmem_load_wait();
#pragma unroll
                for (int c = 0; c < HALF_KEYS / 32; ++c)
#pragma unroll
                    for (int j = 0; j < 32; ++j) s[32 * c + j] = tmem_loaded(raw[c][j]);
            }
            const int key_base = (block0 + i) * KEYS + half * HALF_KEYS;
            const bool all_visible = __all_sync(0xffffffffu, key_base + HALF_KEYS - 1 <= pos && key_base >= first);
            if (!all_visible) {
#pragma unroll
                for (int j = 0; j < HALF_KEYS; ++j) {
                    const int key = key_base + j;
                    s[j] = (key <= pos && key >= first) ? s[j] : -INFINITY;
                }
            }
            float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;   // four chains of three-input maxima
#pragma unroll
            for (int j = 0; j < HALF_KEYS; j += 8) {
                mxa = max3(mxa, s[j], s[j + 1]);
                mxb = max3(mxb, s[j + 2], s[j + 3]);
                mxc = max3(mxc, s[j + 4], s[j + 5]);
                mxd = max3(mxd, s[j + 6], s[j + 7]);
            }
            float mx = fmaxf(max3(mxa, mxb, mxc), mxd);
            if (SPLIT == 2) {
                pair_max[i & 1][half][r] = mx;
                pair_barrier();
                mx = fmaxf(mx, pair_max[i & 1][half ^ 1][r]);
            }
            mx *= args.scale_log2;
            const bool grow = mx > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && mx != -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? mx : m_used;
                const float corr = (m_used == -INFINITY) ? 0.0f : fast_exp2(m_used - m_new);
                if (i > 0) {
                    if (ok && !mbar_wait(smem_u32(&pv_done[(i - 1) & 1]), (uint32_t)(((i - 1) >> 1) & 1))) expired();
                    fence_after_sync();
#pragma unroll
                    for (int c = 0; c < O_COLS; c += 32) {
                        float o[32];
                        tmem_load32(lane_base + L::O_COL + half * O_COLS + c, o);
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] *= corr;
                        tmem_store32(lane_base + L::O_COL + half * O_COLS + c, o);
                    }
                }
                l *= corr;
                m_used = m_new;
            }
            const float base = (m_used == -INFINITY) ? 0.0f : m_used;
            // p = 2^(s * scale - base), two at a time: packed multiply-add, two exponentials, packed sum, one conversion
            // per pair.  (Making a quarter or half of the pairs by a cubic on the floating-point pipes instead of the
            // special-function unit was measured slower: 168 -> 193 and 221 ms for a 32,768-token prompt.)
            const uint64_t scale2 = pack2(args.scale_log2, args.scale_log2), nbase2 = pack2(-base, -base);
            uint64_t sum_a = pack2(0.0f, 0.0f), sum_b = sum_a;
            uint32_t packed[HALF_KEYS / 2];
#pragma unroll
            for (int j = 0; j < HALF_KEYS; j += 2) {
                const uint64_t t = fma2(pack2(s[j], s[j + 1]), scale2, nbase2);
                float t0, t1;
                unpack2(t, t0, t1);
                const uint64_t p = pack2(fast_exp2(t0), fast_exp2(t1));
                if ((j >> 1) & 1) sum_b = add2(sum_b, p); else sum_a = add2(sum_a, p);
                float p0, p1;
                unpack2(p, p0, p1);
                const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                packed[j / 2] = *reinterpret_cast<const uint32_t*>(&h);
            }
            {
                float a0, a1;
                unpack2(add2(sum_a, sum_b), a0, a1);
                l += a0 + a1;
            }
            // P_i goes to buffer i & 1, which the products of block i - 2 must have finished reading.  They have: the
            // issuing thread asked for them before it asked for S_i, its products complete in the order it issues them, and
            // this thread has seen S_i complete.  (A wait of its own on pv_done here cost 160 cycles of 1,500 a block.)
            if (SPLIT == 2) tmem_store16(lane_base + L::P_COL + (i & 1) * 32 + half * 16, packed);
            else tmem_store32(lane_base + L::P_COL + (i & 1) * 32, reinterpret_cast<const float*>(packed));
            fence_before_sync();
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(smem_u32(&p_ready[i & 1]));
        }
        if (ok) {
            const int last = n_blocks - 1;
            if (!mbar_wait(smem_u32(&pv_done[last & 1]), (uint32_t)((last >> 1) & 1))) expired();
        }
        if (SPLIT == 2) {               // the row sum is the two threads' sums together (both rescaled to the same maximum)
            pair_max[n_blocks & 1][half][r] = l;
            pair_barrier();
            l += pair_max[n_blocks & 1][half ^ 1][r];
        }
        if (ok) {
            fence_after_sync();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const int token = seq_begin + tok0 + local, head = kh * args.group + (r - local * args.group);
            __nv_bfloat16* dst = args.out + ((size_t)token * args.heads + head) * HD + half * O_COLS;
#pragma unroll
            for (int c = 0; c < O_COLS; c += 32) {
                float o[32];
                tmem_load32(lane_base + L::O_COL + half * O_COLS + c, o);
                if (row_ok) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 v;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(o[e] * inv, o[e + 1] * inv), h1 = __floats2bfloat162_rn(o[e + 2] * inv, o[e + 3] * inv);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(o[e + 4] * inv, o[e + 5] * inv), h3 = __floats2bfloat162_rn(o[e + 6] * inv, o[e + 7] * inv);
                        v.x = *reinterpret_cast<uint32_t*>(&h0); v.y = *reinterpret_cast<uint32_t*>(&h1);
                        v.z = *reinterpret_cast<uint32_t*>(&h2); v.w = *reinterpret_cast<uint32_t*>(&h3);
                        *reinterpret_cast<uint4*>(dst + c + e) = v;
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, L::TMEM_COLS);
}

template <int HD>
int launch(const void* q, const void* k_pool, const void* v_pool, const Args& args, int n_tokens, cudaStream_t stream) {
    using L = Layout<HD>;
    CUtensorMap map_q, map_k, map_v;
    {   // q [token][head][dim]: a box of 64 dims x group heads x tokens_per_tile tokens = up to 128 rows of 128 bytes
        const cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)args.heads, (cuuint64_t)n_tokens};
        const cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)args.heads * HD * 2};
        const cuuint32_t box[3] = {64, (cuuint32_t)args.group, (cuuint32_t)args.tokens_per_tile};
        if (!tc::make_map(&map_q, q, 3, dims, strides, box)) return -1;
    }
    {   // keys [block * kv_head * 64 tokens][dim]
        const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)args.pool_blocks * args.kv_heads * KEYS};
        const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        const cuuint32_t box[2] = {64, KEYS};
        if (!tc::make_map(&map_k, k_pool, 2, dims, strides, box)) return -1;
    }
    {   // values [block * kv_head * dim][64 tokens]
        const cuuint64_t dims[2] = {(cuuint64_t)KEYS, (cuuint64_t)args.pool_blocks * args.kv_heads * HD};
        const cuuint64_t strides[1] = {(cuuint64_t)KEYS * 2};
        const cuuint32_t box[2] = {KEYS, (cuuint32_t)HD};
        if (!tc::make_map(&map_v, v_pool, 2, dims, strides, box)) return -1;
    }
    static bool configured = false;
    auto kernel = attention_tcgen05_kernel<HD>;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM);
        if (err != cudaSuccess) return (int)err;
        configured = true;
    }
    tt_launch_pdl(kernel, dim3(args.kv_heads, args.cta_tiles), dim3(L::THREADS), (size_t)L::SMEM, stream, map_q, map_k, map_v, args);
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" int tt_attention_tcgen05_supports(int heads, int kv_heads, int head_dim) {
    if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16) return 0;
    return head_dim == 64 || head_dim == 128;
}

// Packed prompts (any number of tokens per sequence) attending over the block cache; the
// new tokens' keys and values are already in the cache.  Returns a cudaError_t value, or -1
// if the tensor maps could not be made.
extern "C" int tt_attention_tcgen05(const void* q, const void* k_pool, const void* v_pool, const int* table, int table_width,
                                    int pool_blocks, const int* cu, const int* len_before, int sequences, int n_tokens,
                                    int heads, int kv_heads, int head_dim, float scale, int window, void* out,
                                    unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!tt_attention_tcgen05_supports(heads, kv_heads, head_dim) || ((uintptr_t)q & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))
        return (int)cudaErrorInvalidValue;
    Args args;
    args.table = table; args.table_width = table_width; args.pool_blocks = pool_blocks; args.cu = cu; args.len_before = len_before;
    args.sequences = sequences; args.heads = heads; args.kv_heads = kv_heads; args.group = heads / kv_heads;
    args.tokens_per_tile = ROWS / args.group;
    args.cta_tiles = (n_tokens + args.tokens_per_tile - 1) / args.tokens_per_tile + sequences;   // upper bound; spare CTAs leave at once
    if (args.cta_tiles > 65535) return (int)cudaErrorInvalidValue;                               // the grid's y extent; steps are cut into pieces long before
    args.scale_log2 = scale * 1.4426950408889634f; args.window = window; args.out = (__nv_bfloat16*)out; args.status = status;
    if (head_dim == 64) return launch<64>(q, k_pool, v_pool, args, n_tokens, stream);
    return launch<128>(q, k_pool, v_pool, args, n_tokens, stream);
}

// bfloat16 matrix products on the 5th-generation tensor cores of sm_100a:
//   out = x @ w^T,  x [tokens, k] and w [features, k] both bfloat16 with k contiguous,
// accumulated in float32 in tensor memory.
//
// One CTA computes one 128-row accumulator tile.  Operand tiles of 64 k-elements (128
// bytes per row) travel global -> shared memory by TMA (cp.async.bulk.tensor, 128-byte
// swizzle) through a ring of stages guarded by full/empty mbarriers; one elected thread
// issues tcgen05.mma (M = 128, K = 16 per instruction) on shared-memory descriptors;
// tcgen05.commit releases stages and finally signals the epilogue warps, which read the
// accumulator with tcgen05.ld and store.  Warp 0 loads, warp 1 owns tensor memory and
// issues, warps 2-5 are the epilogue (each reads the 32 lanes its warp index allows).
//
// Four forms:
//   TOKENS_ON_M            tile = 128 tokens x BN features; float32 partial sums
//                          out[split][token][feature] (+ bias in split 0).  Prompts.
//   TOKENS_ON_M + SWIGLU   the weight holds gate rows then up rows; each k-block issues
//                          two products (gate tile, up tile) into two column ranges and
//                          the epilogue writes silu(gate) * up in bfloat16.
//   FEATURES_ON_M          tile = 128 features x BN tokens (BN = 16..128): the weights sit
//                          on the 128-row side so that a decode step with few tokens
//                          wastes no tensor-core rows and streams each weight exactly
//                          once; the output is written transposed.  k may be cut into
//                          `splits` slices (grid.z) so that few output tiles still fill
//                          148 SMs; consumers sum the slices.
//   FEATURES_ON_M + SWIGLU the 128 rows of a tile are 64 gate rows over the 64 up rows of the
//                          same features (two TMA boxes per stage); the up half of the
//                          accumulator crosses to the gate half's threads through shared
//                          memory and silu(gate) * up is stored in bfloat16.  k is not cut.
//
// Prompts with enough tiles to fill the GPU run the persistent kernel further down: one
// CTA per SM walks over 128 x 256 tiles (or 128 x 128 gate + 128 x 128 up), with two
// accumulators in tensor memory so that the epilogue of one tile runs under the products
// of the next.  From 2,048 tokens on (SwiGLU: 512) its CTA-pair form takes over:
// tcgen05.mma.cta_group::2 on tiles of 256 tokens, each CTA fetching only half of the weights.
//
// Every wait is bounded: when one runs out the kernel raises TT_STATUS_WAIT_EXPIRED,
// drains its outstanding copies, frees its tensor memory and returns.
//
// Counterparts in random-unknown-username/Thintensor: the Triton matvec kernels
// thinruntime/triton_kernels.py:484-535, 2074-2185 (multi_matvec), 3022-3083 (split-k)
// and _fused_gate_up_silu_kernel :3155-3239; all SIMT, one token.
#include "tcgen05.cuh"

#include <cooperative_groups.h>
namespace cg = cooperative_groups;

namespace {

constexpr int BM = 128;          // accumulator rows (UMMA M)
constexpr int BK = 64;           // k elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

enum Form { TOKENS_ON_M = 0, TOKENS_ON_M_SWIGLU = 1, FEATURES_ON_M = 2, FEATURES_ON_M_SWIGLU = 3, TOKENS_ON_M_QKV = 4 };

using namespace tc;

template <int FORM, int BN> struct Shape {
    static constexpr bool dual = FORM == TOKENS_ON_M_SWIGLU;
    static constexpr int a_bytes = BM * BK * 2;
    static constexpr int b_bytes = BN * BK * 2 * (dual ? 2 : 1);
    static constexpr int stage_bytes = a_bytes + b_bytes;
    static constexpr int acc_cols = BN * (dual ? 2 : 1);
    static constexpr int tmem_cols = acc_cols < 32 ? 32 : acc_cols;
};

// Where the qkv form of the prompt kernels sends its output instead of a float32 matrix: the columns
// are q heads, then k heads, then v heads of head_dim numbers each; q and k are rotated (all of a head,
// halves convention) with the step's table of cosines and sines, q goes to q_out in bfloat16 and k and v
// into the block cache at the token's position (values transposed inside a block, see common.cuh).
struct QkvRope {
    __nv_bfloat16* q_out;    // [tokens][q_cols]
    __nv_bfloat16* k_pool;
    __nv_bfloat16* v_pool;
    const float2* cos_sin;   // [tokens][head_dim / 2]: (cos, sin) of inv_freq[i] * position
    const int2* where;       // [tokens]: (position, sequence)
    const int* table;        // [sequences][table_width] block ids
    int table_width, pool_blocks;
    int q_cols, kv_cols, kv_heads;
    float attention_scaling;
};

struct Args {
    const float* bias;       // float32 [features] or null
    void* out;               // float32 partial sums, or bfloat16 activations (SWIGLU)
    long long ld_out;        // elements between token rows of out
    long long split_stride;  // elements between k-slices of out
    int tokens, features, k;
    int k_blocks_per_split;
    int up_row_offset;       // SWIGLU: row of w where the up projection starts (= features of the output)
    int accumulate;          // persistent and pair kernels, plain form: out += product instead of out = product
    int bulk_out;            // persistent and pair kernels, plain form: the tile leaves through shared memory and tiled copies (map_out is valid)
    float* shares;           // pair kernel, plain form: where CTA pairs leave their shares of tiles that several pairs work on (null: every tile has one pair)
    QkvRope rope;            // qkv form only
    int rope_head_dim;       // 64 or 128
    int undelivered_bytes;   // 0 in every real call; tests: the first stage's barrier expects this many bytes that no copy brings
    unsigned* status;
};

// GROUP: k-blocks that share one round of the full / empty barriers (STAGES is a multiple of it).  With few tokens
// a k-block is four short products; waiting, fencing and committing once per k-block cost the issuing thread more
// than the products themselves (520 cycles a k-block of which the products are 234, measured with a one-CTA probe),
// so the form for up to 16 tokens takes two k-blocks per round.  Measured on a B200, decode step of the 1B shape:
// batch 16 0.923 -> 0.908 ms, batch 1 and 8 unchanged within noise (there the tiles' arrival paces the loop).
template <int FORM, int BN, int STAGES, int GROUP = 1>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Args args) {
    using S = Shape<FORM, BN>;
    static_assert(STAGES % GROUP == 0, "whole groups of stages");
    constexpr int RING = STAGES / GROUP;                       // barrier rounds the ring holds
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle groups need 1024-byte alignment
    __shared__ uint64_t full_bar[RING], empty_bar[RING], acc_bar;
    __shared__ uint32_t tmem_base_shared;

    tt_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_m = blockIdx.y, tile_n = blockIdx.x, split = blockIdx.z;
    const int k_blocks_total = (args.k + BK - 1) / BK;
    const int kb_begin = split * args.k_blocks_per_split;
    const int kb_end = min(k_blocks_total, kb_begin + args.k_blocks_per_split);
    const int n_kb = max(0, kb_end - kb_begin);
    const int n_groups = (n_kb + GROUP - 1) / GROUP;
    auto blocks_of = [&](int group) { return min(GROUP, n_kb - group * GROUP); };      // k-blocks of a barrier round (the last may be short)

    if (threadIdx.x == 0) {
        for (int s = 0; s < RING; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        mbar_init(smem_u32(&acc_bar), 1);
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_shared), S::tmem_cols);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_shared;

    // rows of the two operands this tile reads
    constexpr bool weights_are_a = FORM == FEATURES_ON_M || FORM == FEATURES_ON_M_SWIGLU;
    constexpr bool paired_rows = FORM == FEATURES_ON_M_SWIGLU;     // 64 gate rows over the 64 up rows of the same features
    const int a_row = tile_m * (paired_rows ? BM / 2 : BM);       // tokens (TOKENS_ON_M*) or features (FEATURES_ON_M*)
    const int b_row = tile_n * BN;
    auto load_a = [&](uint8_t* stage, int kx, uint32_t bar) {
        if (paired_rows) {
            tma_load_2d(smem_u32(stage), &map_a, kx, a_row, bar);
            tma_load_2d(smem_u32(stage + S::a_bytes / 2), &map_a, kx, args.up_row_offset + a_row, bar);
        } else {
            tma_load_2d(smem_u32(stage), &map_a, kx, a_row, bar);
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // The weight operand is written by no kernel of the step, so the first ring of
        // weight tiles is fetched before waiting for the kernel that produces the
        // activations; under programmatic dependent launch that fetch overlaps the
        // tail of the previous kernel.
        if (lane == 0) {
            auto load_weights = [&](uint8_t* stage, int kx, uint32_t bar) {
                if (weights_are_a) {
                    load_a(stage, kx, bar);
                } else {
                    tma_load_2d(smem_u32(stage + S::a_bytes), &map_b, kx, b_row, bar);
                    if (S::dual) tma_load_2d(smem_u32(stage + S::a_bytes + BN * BK * 2), &map_b, kx, args.up_row_offset + b_row, bar);
                }
            };
            auto load_activations = [&](uint8_t* stage, int kx, uint32_t bar) {
                if (weights_are_a) tma_load_2d(smem_u32(stage + S::a_bytes), &map_b, kx, b_row, bar);
                else load_a(stage, kx, bar);
            };
            const int first = min(n_groups, RING);
            for (int g = 0; g < first; ++g) {               // the ring is empty: nothing to wait for
                const uint32_t bar = smem_u32(&full_bar[g]);
                mbar_expect_tx(bar, blocks_of(g) * S::stage_bytes + (g == 0 ? args.undelivered_bytes : 0));
                for (int q = 0; q < blocks_of(g); ++q)
                    load_weights(smem + (size_t)(g * GROUP + q) * S::stage_bytes, (kb_begin + g * GROUP + q) * BK, bar);
            }
            tt_pdl_wait();
            for (int g = 0; g < first; ++g)
                for (int q = 0; q < blocks_of(g); ++q)
                    load_activations(smem + (size_t)(g * GROUP + q) * S::stage_bytes, (kb_begin + g * GROUP + q) * BK, smem_u32(&full_bar[g]));
            int issued = first;
            for (int g = first; g < n_groups; ++g) {
                const int s = g % RING;
                const uint32_t parity = ((g / RING) & 1) ^ 1;
                if (!mbar_wait(smem_u32(&empty_bar[s]), parity)) { atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); break; }
                const uint32_t bar = smem_u32(&full_bar[s]);
                mbar_expect_tx(bar, blocks_of(g) * S::stage_bytes);
                for (int q = 0; q < blocks_of(g); ++q) {
                    uint8_t* stage = smem + (size_t)(s * GROUP + q) * S::stage_bytes;
                    const int kx = (kb_begin + g * GROUP + q) * BK;
                    load_weights(stage, kx, bar);
                    load_activations(stage, kx, bar);
                }
                ++issued;
            }
            // drain: every copy issued must have landed before shared memory is given up
            for (int g = max(0, issued - RING); g < issued; ++g)
                if (!mbar_wait(smem_u32(&full_bar[g % RING]), (g / RING) & 1)) { atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); break; }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BM, S::dual ? 2 * BN : BN);   // gate and up tiles lie like one tile of 2 BN rows
            bool ok = true;
            for (int g = 0; g < n_groups && ok; ++g) {
                const int s = g % RING;
                if (!mbar_wait(smem_u32(&full_bar[s]), (g / RING) & 1)) { atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; break; }
                fence_after_sync();
                for (int q = 0; q < blocks_of(g); ++q) {
                    const uint32_t a_addr = smem_u32(smem + (size_t)(s * GROUP + q) * S::stage_bytes);
                    const uint32_t b_addr = a_addr + S::a_bytes;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint32_t acc = (g > 0 || q > 0 || kk > 0) ? 1u : 0u;
                        const uint64_t da = smem_desc(a_addr + kk * UMMA_K * 2);
                        umma_bf16(tmem_base, da, smem_desc(b_addr + kk * UMMA_K * 2), idesc, acc);
                    }
                }
                umma_commit(smem_u32(&empty_bar[s]));     // the round's stages are free once these products have read them
            }
            if (ok) umma_commit(smem_u32(&acc_bar));      // the accumulator is complete once all products are done
        }
    } else {
        // ------------------------------------------------------------ epilogue
        tt_pdl_wait();                                      // nothing is stored before every earlier kernel is done
        const int quarter = warp & 3;                      // the 32 tensor-memory lanes this warp may read
        const int row = quarter * 32 + lane;               // accumulator row owned by this thread
        bool ok = n_kb == 0 ? true : mbar_wait(smem_u32(&acc_bar), 0);
        if (!ok && lane == 0) { atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); }
        fence_after_sync();
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        if (FORM == FEATURES_ON_M_SWIGLU) {
            // Accumulator rows 0..63 are the gate, rows 64..127 the up projection of features
            // a_row .. a_row + 63.  The up half goes through shared memory to the threads of the
            // gate half (the ring is free: every product has read it), which store
            // silu(gate) * up in bfloat16.  Both halves meet at named barrier 1.
            constexpr int PITCH = BN + 1;
            float* exchange = reinterpret_cast<float*>(smem);
            const bool is_up = quarter >= 2;
            const int r = row & 63;
            if (ok && is_up) {
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    tmem_load16(lane_addr + c, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) exchange[r * PITCH + c + j] = v[j];
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int feature = a_row + r;
            if (ok && !is_up) {
                __nv_bfloat16* out = (__nv_bfloat16*)args.out;
                for (int c = 0; c < BN; c += 16) {
                    float g[16];
                    tmem_load16(lane_addr + c, g);
                    if (feature < args.features) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int token = b_row + c + j;
                            if (token < args.tokens)
                                out[(size_t)token * args.ld_out + feature] = __float2bfloat16_rn(g[j] / (1.0f + __expf(-g[j])) * exchange[r * PITCH + c + j]);
                        }
                    }
                }
            }
        } else if (ok) {
            if (FORM == TOKENS_ON_M) {
                const int token = a_row + row;
                float* out = (float*)args.out + (size_t)split * args.split_stride + (size_t)token * args.ld_out;
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    if (n_kb > 0) tmem_load16(lane_addr + c, v);
                    else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    }
                    const int f0 = b_row + c;
                    if (token < args.tokens) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int f = f0 + j;
                            if (f < args.features) out[f] = v[j] + ((args.bias && split == 0) ? args.bias[f] : 0.0f);
                        }
                    }
                }
            } else if (FORM == TOKENS_ON_M_SWIGLU) {
                const int token = a_row + row;
                __nv_bfloat16* out = (__nv_bfloat16*)args.out + (size_t)token * args.ld_out;
                for (int c = 0; c < BN; c += 16) {
                    float g[16], u[16];
                    tmem_load16(lane_addr + c, g);
                    tmem_load16(lane_addr + BN + c, u);
                    const int f0 = b_row + c;
                    if (token < args.tokens) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int f = f0 + j;
                            if (f < args.features) out[f] = __float2bfloat16_rn(g[j] / (1.0f + __expf(-g[j])) * u[j]);
                        }
                    }
                }
            } else {
                const int feature = a_row + row;
                float* out = (float*)args.out + (size_t)split * args.split_stride;
                const float bias = (args.bias && split == 0 && feature < args.features) ? args.bias[feature] : 0.0f;
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    if (n_kb > 0) tmem_load16(lane_addr + c, v);
                    else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    }
                    if (feature < args.features) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int token = b_row + c + j;
                            if (token < args.tokens) out[(size_t)token * args.ld_out + feature] = v[j] + bias;
                        }
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, S::tmem_cols);
}


// An epilogue thread asks for its row of the output tile into the L2 while the products still run
// (accumulate form: the row is read before it is written).
__device__ __forceinline__ void prefetch_output_row(int token, int f_base, const Args& args) {
    if (!args.accumulate || token >= args.tokens) return;
    const float* row = (const float*)args.out + (size_t)token * args.ld_out;
    for (int c = 0; c < 256 && f_base + c < args.features; c += 32)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(row + f_base + c));
}

// What an epilogue thread does with its row of a 128 x 256 accumulator (lane_addr: the row's
// first column): plain form, 256 features from f_base as float32 (+ bias); SwiGLU form, columns
// 0..127 the gate and 128..255 the up projection of 128 features from f_base, stored as bfloat16.
// The tensor-memory loads are warp-collective: every lane runs them, valid row or not.
template <bool dual, int WIDE = 256>
__device__ __forceinline__ void store_accumulator(uint32_t lane_addr, int token, int f_base, const Args& args) {
    if (dual) {
        // A tile's epilogue has to fit under the next tile's products (16,400 cycles for k = 2,048): with one round trip to
        // tensor memory per half chunk and 4-byte stores (every lane its own row: 32 sectors an instruction for 128 bytes)
        // it took 19,200 cycles and bounded the kernel (clock stamps on a B200).  So the next chunk's gate and up are on
        // their way while this one is worked on, and eight results go out as one 16-byte store.
        __nv_bfloat16* out = (__nv_bfloat16*)args.out + (size_t)token * args.ld_out;
        const bool vec = (args.ld_out & 7) == 0 && (((uintptr_t)args.out) & 15) == 0 && (f_base & 7) == 0;
        uint32_t gate[2][32], up[2][32];
        tmem_load32_issue(lane_addr, gate[0]);
        tmem_load32_issue(lane_addr + 128, up[0]);
#pragma unroll
        for (int ci = 0; ci < 4; ++ci) {
            const int c = 32 * ci, cur = ci & 1;
            tmem_load_wait();
            if (ci + 1 < 4) {
                tmem_load32_issue(lane_addr + c + 32, gate[cur ^ 1]);
                tmem_load32_issue(lane_addr + 128 + c + 32, up[cur ^ 1]);
            }
            if (token < args.tokens) {
#pragma unroll
                for (int e0 = 0; e0 < 32; e0 += 8) {
                    const int f = f_base + c + e0;
                    float y[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float g = tmem_loaded(gate[cur][e0 + e]), u = tmem_loaded(up[cur][e0 + e]);
                        y[e] = __fdividef(g, 1.0f + __expf(-g)) * u;
                    }
                    if (vec && f + 8 <= args.features) {
                        const __nv_bfloat162 p0 = __floats2bfloat162_rn(y[0], y[1]), p1 = __floats2bfloat162_rn(y[2], y[3]);
                        const __nv_bfloat162 p2 = __floats2bfloat162_rn(y[4], y[5]), p3 = __floats2bfloat162_rn(y[6], y[7]);
                        *reinterpret_cast<uint4*>(out + f) = make_uint4(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1),
                                                                        *reinterpret_cast<const uint32_t*>(&p2), *reinterpret_cast<const uint32_t*>(&p3));
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (f + e < args.features) out[f + e] = __float2bfloat16_rn(y[e]);
                    }
                }
            }
        }
    } else {
        float* out = (float*)args.out + (size_t)token * args.ld_out;
        const bool vec = (args.ld_out & 3) == 0 && (((uintptr_t)args.out) & 15) == 0;
        for (int c = 0; c < WIDE; c += 32) {
            float v[32];
            const int f0 = f_base + c;
            float4 old[8];
            const bool add_vec = args.accumulate && token < args.tokens && vec && f0 + 32 <= args.features;
            if (add_vec) {                                  // on their way while the accumulator is read
#pragma unroll
                for (int e = 0; e < 8; ++e) old[e] = *reinterpret_cast<const float4*>(out + f0 + 4 * e);
            }
            tmem_load32(lane_addr + c, v);
            if (token < args.tokens) {
                if (args.bias) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) if (f0 + e < args.features) v[e] += args.bias[f0 + e];
                }
                if (add_vec) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) { v[4 * e] += old[e].x; v[4 * e + 1] += old[e].y; v[4 * e + 2] += old[e].z; v[4 * e + 3] += old[e].w; }
                } else if (args.accumulate) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) if (f0 + e < args.features) v[e] += out[f0 + e];
                }
                if (vec && f0 + 32 <= args.features) {
#pragma unroll
                    for (int e = 0; e < 32; e += 4) *reinterpret_cast<float4*>(out + f0 + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) if (f0 + e < args.features) out[f0 + e] = v[e];
                }
            }
        }
    }
}

// The plain form's epilogue through shared memory: a warp's 32 rows x 32 columns of the accumulator go into a 4 KB
// slab (swizzled as the map says, so that the lanes, each with a row of its own, spread over all banks) and leave it
// as one tiled copy, which stores them, or adds them to what the output holds, in whole lines.  With stores from
// registers every lane wrote 16 bytes of another row: 32 sectors an instruction, 10,200 cycles for a tile of
// 128 x 256, and the accumulate form had to read the old values first.  The warp alternates between two slabs;
// `round` counts its copies so far (the slab a copy two rounds back read from is free once all but the latest
// group have read).  The copies clip what hangs over the matrix's edges.  Warp-collective.
template <int WIDE>
__device__ __forceinline__ void store_accumulator_bulk(uint32_t lane_addr, int first_token, int f_base, int slice, const Args& args,
                                                       const CUtensorMap* map_out, uint8_t* slabs, int lane, int& round,
                                                       const float* share_a = nullptr, const float* share_b = nullptr) {
    const float* bias = slice == 0 ? args.bias : nullptr;                      // a later k-slice: its own plane of the output, no bias
#pragma unroll 1
    for (int c = 0; c < WIDE; c += 32) {
        float v[32];
        tmem_load32(lane_addr + c, v);
        const int f0 = f_base + c;
        if (first_token >= args.tokens || f0 >= args.features) continue;       // the same for the whole warp
        // other pairs' shares of this tile's k (see store_share): added in a fixed order, first the one next in k
        if (share_a) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
                const float4 other = __ldcg(reinterpret_cast<const float4*>(share_a) + ((c + e) >> 2) * 32 + lane);
                v[e] += other.x; v[e + 1] += other.y; v[e + 2] += other.z; v[e + 3] += other.w;
            }
        }
        if (share_b) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
                const float4 other = __ldcg(reinterpret_cast<const float4*>(share_b) + ((c + e) >> 2) * 32 + lane);
                v[e] += other.x; v[e + 1] += other.y; v[e + 2] += other.z; v[e + 3] += other.w;
            }
        }
        if (bias) {
#pragma unroll
            for (int e = 0; e < 32; ++e) if (f0 + e < args.features) v[e] += bias[f0 + e];
        }
        uint8_t* slab = slabs + (round & 1) * 4096;
        ++round;
        if (lane == 0) bulk_wait_group_read<1>();
        __syncwarp();
#pragma unroll
        for (int piece = 0; piece < 8; ++piece)
            *reinterpret_cast<float4*>(slab + lane * 128 + ((piece ^ (lane & 7)) << 4)) =
                make_float4(v[4 * piece], v[4 * piece + 1], v[4 * piece + 2], v[4 * piece + 3]);
        fence_async_shared();
        __syncwarp();
        if (lane == 0) {
            if (args.accumulate) tma_reduce_add_3d(map_out, smem_u32(slab), f0, first_token, slice);
            else tma_store_3d(map_out, smem_u32(slab), f0, first_token, slice);
            bulk_commit_group();
        }
    }
}

// The SwiGLU form's tile through shared memory: columns 0..127 of the accumulator are the gate and 128..255 the up
// projection of 128 features from f_base; silu(gate) * up as bfloat16, 64 features (128 bytes) x 32 rows to a slab,
// one tiled copy a slab.  The next chunk's gate and up are on their way while one is worked on, as in the register form.
__device__ __forceinline__ void store_swiglu_bulk(uint32_t lane_addr, int first_token, int f_base, const Args& args, const CUtensorMap* map_out,
                                                  uint8_t* slabs, int lane, int& round) {
    uint32_t gate[2][32], up[2][32];
    tmem_load32_issue(lane_addr, gate[0]);
    tmem_load32_issue(lane_addr + 128, up[0]);
    const bool wanted = first_token < args.tokens;                             // the same for the whole warp
#pragma unroll
    for (int ci = 0; ci < 4; ++ci) {
        const int cur = ci & 1;
        tmem_load_wait();
        if (ci + 1 < 4) {
            tmem_load32_issue(lane_addr + 32 * ci + 32, gate[cur ^ 1]);
            tmem_load32_issue(lane_addr + 128 + 32 * ci + 32, up[cur ^ 1]);
        }
        const int f0 = f_base + 64 * (ci >> 1);                                // first feature of this chunk's slab
        if (!wanted || f0 >= args.features) continue;
        uint8_t* slab = slabs + (round & 1) * 4096;
        if ((ci & 1) == 0) {
            if (lane == 0) bulk_wait_group_read<1>();
            __syncwarp();
        }
#pragma unroll
        for (int e0 = 0; e0 < 32; e0 += 8) {
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float g = tmem_loaded(gate[cur][e0 + e]), u = tmem_loaded(up[cur][e0 + e]);
                y[e] = __fdividef(g, 1.0f + __expf(-g)) * u;
            }
            const __nv_bfloat162 p0 = __floats2bfloat162_rn(y[0], y[1]), p1 = __floats2bfloat162_rn(y[2], y[3]);
            const __nv_bfloat162 p2 = __floats2bfloat162_rn(y[4], y[5]), p3 = __floats2bfloat162_rn(y[6], y[7]);
            const int piece = (ci & 1) * 4 + (e0 >> 3);
            *reinterpret_cast<uint4*>(slab + lane * 128 + ((piece ^ (lane & 7)) << 4)) =
                make_uint4(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1),
                           *reinterpret_cast<const uint32_t*>(&p2), *reinterpret_cast<const uint32_t*>(&p3));
        }
        if (ci & 1) {
            fence_async_shared();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(map_out, smem_u32(slab), f0, first_token);
                bulk_commit_group();
            }
            ++round;
        }
    }
}

// A warp's 32 rows of an accumulator that holds only a share of the tile's k: four columns at a time into the warp's own
// 32 KB of scratch memory, the 32 lanes' 16-byte pieces side by side (whole lines a store; the layout is nobody
// else's business).  The pair that holds the tile's first k-blocks adds it to its own share (store_accumulator_bulk).
template <int WIDE>
__device__ __forceinline__ void store_share(uint32_t lane_addr, float* share, int lane) {
#pragma unroll 1
    for (int c = 0; c < WIDE; c += 32) {
        float v[32];
        tmem_load32(lane_addr + c, v);
#pragma unroll
        for (int e = 0; e < 32; e += 4)
            __stcg(reinterpret_cast<float4*>(share) + ((c + e) >> 2) * 32 + lane, make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]));
    }
}

// The work of CTA pair `pair` of `n_pairs` when the tiles' k-blocks are dealt out evenly (units = tiles * k-blocks in
// tile order, every pair a contiguous run of them): item j of the pair is k-blocks kb0 .. kb1 - 1 of tile `tile`.
// Only a pair's first item can start inside a tile (kb0 > 0: a share that the tile's first pair will add to its
// own), only its last can end inside one (kb0 == 0, kb1 < all: this pair writes the tile, after the shares of the
// pairs behind it have arrived).
struct KRun {
    long long begin, end;       // units
    int k_blocks;               // per tile
    __device__ int items() const { return end > begin ? (int)((end - 1) / k_blocks - begin / k_blocks) + 1 : 0; }
    __device__ void item(int j, int& tile, int& kb0, int& kb1) const {
        const long long t = begin / k_blocks + j;
        tile = (int)t;
        kb0 = j == 0 ? (int)(begin - t * k_blocks) : 0;
        kb1 = end < (t + 1) * k_blocks ? (int)(end - t * k_blocks) : k_blocks;
    }
};
__device__ __forceinline__ KRun k_run_of(int pair, int n_pairs, int tiles_total, int k_blocks) {
    const long long units = (long long)tiles_total * k_blocks;
    return KRun{units * pair / n_pairs, units * (pair + 1) / n_pairs, k_blocks};
}
constexpr int SHARE_FLOATS = 32 * 256;                   // one epilogue warp's share of a 256-wide tile
// scratch memory of pair p, CTA r, epilogue warp w: its share, and behind all shares one flag word each
__device__ __forceinline__ float* share_of(float* shares, int pair, int rank, int quarter) {
    return shares + ((size_t)(pair * 2 + rank) * 4 + quarter) * SHARE_FLOATS;
}
__device__ __forceinline__ unsigned* share_flag_of(float* shares, int n_pairs, int pair, int rank, int quarter) {
    return reinterpret_cast<unsigned*>(shares + (size_t)n_pairs * 8 * SHARE_FLOATS) + (pair * 2 + rank) * 4 + quarter;
}

// The qkv form's epilogue for one thread = one token's row of a 128 x WIDE accumulator, whose WIDE / HD
// heads each lie inside the tile (HD = 64 or 128).  A head's rotation pairs dimension d with d + HD / 2:
// the two come from tensor-memory chunks j and j + HD / 64 of the head, so a thread holds both.  The
// arithmetic is that of rope_append_vec_kernel (elementwise.cu).  Tensor-memory loads are
// warp-collective: every lane runs them, valid row or not.
//
// What the row needs besides the accumulator depends on the token only: where it goes in the cache (position,
// sequence, table entry: two dependent loads) and its cosines and sines (HD / 2 pairs, 256 or 512 bytes that every
// head of the tile would otherwise fetch again, past an L1 that the stages leave a few KB).  QkvRow holds them in
// registers; a thread fills it BEFORE it waits for the accumulator, so all of that is in flight while the tile's
// products still run (measured on a B200, tiles of 256 x 192: 12,000 to 15,000 cycles per tile's epilogue with the
// loads inside it, against 12,300 for the tile's products, so the epilogues bounded the kernel).
template <int HD> struct QkvRow {
    int block, slot;
    bool live;
    float4 cs[HD / 4];          // (cos, sin) of two neighbouring pairs each
};

template <int HD>
__device__ __forceinline__ void prepare_qkv_row(QkvRow<HD>& row, int token, const Args& args) {
    const QkvRope& r = args.rope;
    row.live = token < args.tokens;
    row.block = -1;
    row.slot = 0;
    if (row.live) {
        const int2 w = __ldg(r.where + token);
        const float4* cs = reinterpret_cast<const float4*>(r.cos_sin + (size_t)token * (HD / 2));
#pragma unroll
        for (int i = 0; i < HD / 4; ++i) row.cs[i] = __ldg(cs + i);
        const int entry = __ldg(r.table + (size_t)w.y * r.table_width + w.x / TT_BLOCK_TOKENS);
        if (entry < 0 || entry >= r.pool_blocks) atomicOr(args.status, TT_STATUS_BAD_BLOCK);
        else row.block = entry;
        row.slot = w.x % TT_BLOCK_TOKENS;
    } else {
#pragma unroll
        for (int i = 0; i < HD / 4; ++i) row.cs[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
}

template <int HD, int WIDE = 256>
__device__ __forceinline__ void store_qkv_rope(const QkvRow<HD>& row, uint32_t lane_addr, int token, int f_base, const Args& args) {
    static_assert(WIDE % HD == 0, "a tile holds whole heads");
    constexpr int CH = HD / 32, HALF = HD / 2;
    const QkvRope& r = args.rope;
    const bool live = row.live;
    const int block = row.block, slot = row.slot;
    const float k = r.attention_scaling;
    for (int h = 0; h < WIDE / HD; ++h) {
        const int col0 = f_base + h * HD;                       // the head's first column: the same for the whole CTA
        if (col0 >= args.features) break;
        const uint32_t head_addr = lane_addr + h * HD;
        if (col0 < r.q_cols + r.kv_cols) {
            // a query head or a key head: rotate, narrow, store 64 contiguous bytes per chunk
            __nv_bfloat16* dst = nullptr;
            if (live) {
                if (col0 < r.q_cols) dst = r.q_out + (size_t)token * r.q_cols + col0;
                else if (block >= 0) dst = r.k_pool + (((size_t)block * r.kv_heads + (col0 - r.q_cols) / HD) * TT_BLOCK_TOKENS + slot) * HD;
            }
#pragma unroll
            for (int j = 0; j < CH / 2; ++j) {
                float a[32], b[32];
                {
                    uint32_t ra[32], rb[32];
                    tmem_load32_issue(head_addr + j * 32, ra);
                    tmem_load32_issue(head_addr + HALF + j * 32, rb);
                    tmem_load_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) { a[e] = tmem_loaded(ra[e]); b[e] = tmem_loaded(rb[e]); }
                }
                if (!dst) continue;
                if (args.bias) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) { a[e] += args.bias[col0 + j * 32 + e]; b[e] += args.bias[col0 + HALF + j * 32 + e]; }
                }
#pragma unroll
                for (int e0 = 0; e0 < 32; e0 += 8) {                // eight pairs at a time: one 16-byte store for each half
                    uint32_t lo[4], hi[4];
#pragma unroll
                    for (int e = e0; e < e0 + 8; e += 2) {
                        const float4 t = row.cs[(j * 32 + e) / 2];                                     // (cos, sin) of two neighbouring pairs
                        const float ra0 = (a[e] * t.x - b[e] * t.y) * k, rb0 = (b[e] * t.x + a[e] * t.y) * k;
                        const float ra1 = (a[e + 1] * t.z - b[e + 1] * t.w) * k, rb1 = (b[e + 1] * t.z + a[e + 1] * t.w) * k;
                        const __nv_bfloat162 pa = __floats2bfloat162_rn(ra0, ra1), pb = __floats2bfloat162_rn(rb0, rb1);
                        lo[(e - e0) / 2] = *reinterpret_cast<const uint32_t*>(&pa);
                        hi[(e - e0) / 2] = *reinterpret_cast<const uint32_t*>(&pb);
                    }
                    *reinterpret_cast<uint4*>(dst + j * 32 + e0) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    *reinterpret_cast<uint4*>(dst + HALF + j * 32 + e0) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                }
            }
        } else {
            // a value head: one number per 64-token row of the transposed block; the warp's lanes are
            // neighbouring tokens, so each of these stores covers neighbouring positions of a row
            __nv_bfloat16* dst = nullptr;
            if (live && block >= 0)
                dst = r.v_pool + ((size_t)block * r.kv_heads + (col0 - r.q_cols - r.kv_cols) / HD) * HD * TT_BLOCK_TOKENS + slot;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                float v[32];
                tmem_load32(head_addr + c * 32, v);
                if (!dst) continue;
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float x = v[e] + (args.bias ? args.bias[col0 + c * 32 + e] : 0.0f);
                    dst[(size_t)(c * 32 + e) * TT_BLOCK_TOKENS] = __float2bfloat16_rn(x);
                }
            }
        }
    }
}

// One row's epilogue of the qkv form: ask for what the row needs, wait for the tile's accumulator, rotate and store.
// False if the wait ran out.
template <int HD, int WIDE>
__device__ __forceinline__ bool qkv_row_epilogue(uint32_t acc_bar, uint32_t parity, uint32_t lane_addr, int token, int f_base, const Args& args) {
    QkvRow<HD> row;
    prepare_qkv_row<HD>(row, token, args);
    if (!mbar_wait(acc_bar, parity)) return false;
    fence_after_sync();
    store_qkv_rope<HD, WIDE>(row, lane_addr, token, f_base, args);
    return true;
}

// ------------------------------------------------------------------ persistent kernel
// Tokens on M, for prompts.  One CTA per SM takes tiles blockIdx.x, blockIdx.x + gridDim.x,
// ...; tile id -> (token tile = id % tiles_m, feature tile = id / tiles_m), so the CTAs that
// run together share weight tiles in L2.  A tile is 128 tokens x 256 features (plain) or
// 128 x 128 gate and 128 x 128 up (SwiGLU): 256 accumulator columns, and tensor memory holds
// two such accumulators.  When the tiles are fewer than the SMs (prompts of a few hundred tokens) k is cut
// into slices and a CTA's unit of work is one tile's share of one slice, stored into the slice's own
// plane of the output (measured on a B200, a 512-token prompt of the 1B shape: 2.84 -> 2.21 ms).
// The producer and the issuing thread run ahead over tile
// boundaries; the epilogue warps drain accumulator (j & 1) of the CTA's j-th tile while the
// products of tile j + 1 fill the other one.
constexpr int P_STAGES = 4;
constexpr int OUT_SLAB_BYTES = 4 * 2 * 4096;     // plain and SwiGLU forms of the persistent and pair kernels: two slabs of 4 KB (32 rows of 128 bytes) for each epilogue warp
constexpr int P_STAGE_BYTES = BM * BK * 2 + 256 * BK * 2;       // A tile + 256 rows of B

template <int FORM, int WIDE = 256>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               const __grid_constant__ CUtensorMap map_out, const Args args, int tiles_m, int tiles_total, int splits) {
    constexpr bool dual = FORM == TOKENS_ON_M_SWIGLU;
    static_assert(WIDE == 256 || (!dual && WIDE == 128), "the SwiGLU form has no narrower tile");
    constexpr int TILE_N = dual ? 128 : WIDE;                   // output features per tile
    constexpr int STAGE_TX = BM * BK * 2 + (dual ? 256 : WIDE) * BK * 2;       // bytes a stage's copies bring
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[P_STAGES], empty_bar[P_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_shared;

    tt_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks_total = (args.k + BK - 1) / BK;
    // a work item is a tile's share of one k-slice: item -> (tile = item % tiles_total, slice = item / tiles_total);
    // the launcher makes sure that no slice is empty
    const int items_total = tiles_total * splits;
    const int my_tiles = (int)blockIdx.x < items_total ? (items_total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    auto k_blocks_of = [&](int item, int& kb_begin) {
        kb_begin = (item / tiles_total) * args.k_blocks_per_split;
        return min(k_blocks_total, kb_begin + args.k_blocks_per_split) - kb_begin;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&acc_full[b]), 1); mbar_init(smem_u32(&acc_empty[b]), 4); }
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_shared), 512);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_shared;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tt_pdl_wait();
            long long it = 0;                                  // k-blocks issued so far, over all tiles
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const int item = (int)blockIdx.x + j * (int)gridDim.x, tile = item % tiles_total;
                const int a_row = (tile % tiles_m) * BM, b_row = (tile / tiles_m) * TILE_N;
                int kb_begin;
                const int n_kb = k_blocks_of(item, kb_begin);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = (int)(it % P_STAGES);
                    if (!mbar_wait(smem_u32(&empty_bar[s]), (uint32_t)(((it / P_STAGES) & 1) ^ 1))) {
                        atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; break;
                    }
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    mbar_expect_tx(bar, STAGE_TX);
                    uint8_t* stage = smem + (size_t)s * P_STAGE_BYTES;
                    const int kx = (kb_begin + i) * BK;
                    tma_load_2d(smem_u32(stage), &map_a, kx, a_row, bar);
                    if (dual) {
                        tma_load_2d(smem_u32(stage + BM * BK * 2), &map_b, kx, b_row, bar);
                        tma_load_2d(smem_u32(stage + BM * BK * 2 + 128 * BK * 2), &map_b, kx, args.up_row_offset + b_row, bar);
                    } else {
                        tma_load_2d(smem_u32(stage + BM * BK * 2), &map_b, kx, b_row, bar);       // one box of WIDE rows
                    }
                }
            }
            // drain: every copy issued must have landed before shared memory is given up
            for (long long i = it > P_STAGES ? it - P_STAGES : 0; i < it; ++i)
                if (!mbar_wait(smem_u32(&full_bar[i % P_STAGES]), (uint32_t)((i / P_STAGES) & 1))) { atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); break; }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // The gate rows and the up rows of a SwiGLU stage lie next to each other in shared memory
            // exactly like one box of 256 rows, so both forms issue one product of N = 256 per k step
            // (gate in accumulator columns 0..127, up in 128..255); two of N = 128 would cost twice the
            // issue time, which is what bounds this kernel.
            constexpr uint32_t idesc = instr_desc(BM, dual ? 256 : WIDE);
            long long it = 0;
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const int buf = j & 1;
                // the epilogue must have drained this accumulator (tiles j - 2, j - 4, ...)
                if (j >= 2 && !mbar_wait(smem_u32(&acc_empty[buf]), (uint32_t)(((j >> 1) & 1) ^ 1))) {
                    atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; break;
                }
                fence_after_sync();
                const uint32_t acc_addr = tmem_base + buf * 256;
                int kb_begin;
                const int n_kb = k_blocks_of((int)blockIdx.x + j * (int)gridDim.x, kb_begin);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = (int)(it % P_STAGES);
                    if (!mbar_wait(smem_u32(&full_bar[s]), (uint32_t)((it / P_STAGES) & 1))) {
                        atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; break;
                    }
                    fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * P_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + BM * BK * 2;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint32_t accumulate = (i > 0 || kk > 0) ? 1u : 0u;
                        const uint64_t da = smem_desc(a_addr + kk * UMMA_K * 2);
                        umma_bf16(acc_addr, da, smem_desc(b_addr + kk * UMMA_K * 2), idesc, accumulate);
                    }
                    umma_commit(smem_u32(&empty_bar[s]));
                }
                if (ok) umma_commit(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        tt_pdl_wait();
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const bool bulk_out = (FORM == TOKENS_ON_M || dual) && args.bulk_out;
        uint8_t* slabs = smem + (size_t)P_STAGES * P_STAGE_BYTES + quarter * OUT_SLAB_BYTES / 4;     // plain and SwiGLU forms
        int round = 0;
        for (int j = 0; j < my_tiles; ++j) {
            const int buf = j & 1;
            const int item = (int)blockIdx.x + j * (int)gridDim.x, tile = item % tiles_total, slice = item / tiles_total;
            const int token = (tile % tiles_m) * BM + row, f_base = (tile / tiles_m) * TILE_N;
            if (!dual && !bulk_out) prefetch_output_row(token, f_base, args);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256;
            const uint32_t acc_bar = smem_u32(&acc_full[buf]), acc_parity = (uint32_t)((j >> 1) & 1);
            bool ok;
            if constexpr (FORM == TOKENS_ON_M_QKV) {            // never sliced along k
                ok = args.rope_head_dim == 64 ? qkv_row_epilogue<64, WIDE>(acc_bar, acc_parity, lane_addr, token, f_base, args)
                                              : qkv_row_epilogue<128, WIDE>(acc_bar, acc_parity, lane_addr, token, f_base, args);
            } else {
                ok = mbar_wait(acc_bar, acc_parity);
                fence_after_sync();
            }
            if (!ok) {
                if (lane == 0) atomicOr(args.status, TT_STATUS_WAIT_EXPIRED);
                break;
            }
            if constexpr (FORM == TOKENS_ON_M_QKV) {
                // stored by qkv_row_epilogue
            } else if (bulk_out) {
                if constexpr (FORM == TOKENS_ON_M) store_accumulator_bulk<WIDE>(lane_addr, token - lane, f_base, slice, args, &map_out, slabs, lane, round);
                else if constexpr (dual) store_swiglu_bulk(lane_addr, token - lane, f_base, args, &map_out, slabs, lane, round);
            } else if (dual || slice == 0) {
                store_accumulator<dual, WIDE>(lane_addr, token, f_base, args);
            } else {                                            // a later k-slice: its own plane of the output, no bias
                Args mine = args;
                mine.out = (float*)args.out + (size_t)slice * args.split_stride;
                mine.bias = nullptr;
                store_accumulator<dual, WIDE>(lane_addr, token, f_base, mine);
            }
            // this warp is done with the accumulator: tell the issuer
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
        }
        if (bulk_out && lane == 0) bulk_wait_group_read<0>();   // the slabs stay until the last copies have read them
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ------------------------------------------------------------------ CTA pairs
// The persistent kernel with products of CTA pairs (tcgen05.mma.cta_group::2): two CTAs on
// neighbouring SMs share tiles of 256 tokens.  Each loads its own 128 token rows of A and half of
// the tile's 256 weight rows (plain form: features 0..127 or 128..255 of the tile; SwiGLU form: the
// even CTA the 128 gate rows, the odd CTA the 128 up rows), so a k-block costs each SM 32 KB of
// shared-memory fill instead of 48 KB for the same 128 x 256 x 64 multiply-adds.  The even CTA's
// thread issues the products for both; every CTA keeps and drains its own 128 rows of the
// accumulator.  Barriers: full (the even CTA's, counting both CTAs' bytes), empty and acc_full
// (one in each CTA, signalled together by a multicast commit), acc_empty (the even CTA's,
// eight arrivals: four epilogue warps of each CTA).
// Measured on a B200 against the single-CTA persistent kernel (same shapes, 512 to 16,384 tokens):
// 5 to 20 % faster from 2,048 tokens on (up to 1.46 PFLOP/s), a few per cent slower below, except
// the SwiGLU form, which gains from 512 tokens on.
constexpr int PAIR_MIN_TOKENS = 2048, PAIR_MIN_TOKENS_SWIGLU = 512;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = BM * BK * 2 + 128 * BK * 2;    // 128 rows of A + 128 rows of B

// WIDE: the features of a plain tile, 256, or (qkv form, head size 64) 192 where that leaves the last round of the
// CTA pairs fuller: 2,048 tokens x 3,072 features are 96 tiles of 256 for 74 pairs, two rounds of which the second
// is a third full, or 128 tiles of 192, two rounds of three quarters the length.
template <int FORM, int WIDE = 256>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_out, const Args args, int tiles_m, int tiles_total) {
    constexpr bool dual = FORM == TOKENS_ON_M_SWIGLU;
    static_assert(WIDE == 256 || (FORM == TOKENS_ON_M_QKV && WIDE == 192), "only the qkv form has a narrower tile");
    constexpr int TILE_N = dual ? 128 : WIDE;                   // output features per tile
    constexpr int B_ROWS = dual ? 128 : WIDE / 2;               // weight rows each CTA of the pair fetches per k-block
    constexpr int STAGE_TX = BM * BK * 2 + B_ROWS * BK * 2;     // bytes one CTA's copies bring per stage
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[PAIR_STAGES], empty_bar[PAIR_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_shared;

    tt_pdl_launch_dependents();
    cg::cluster_group cluster = cg::this_cluster();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster.block_rank();                 // 0: the CTA that issues
    const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
    const int n_kb = (args.k + BK - 1) / BK;
    // A pair's items: whole tiles pair, pair + n_pairs, ... or, where the launcher gave scratch memory for shares (plain
    // form, fewer whole rounds of tiles than would fill the pairs), its run of the tiles' k-blocks dealt out evenly.
    const bool dealt = FORM == TOKENS_ON_M && args.shares != nullptr;
    const KRun run = k_run_of(pair, n_pairs, tiles_total, n_kb);
    const int my_tiles = dealt ? run.items() : (pair < tiles_total ? (tiles_total - pair + n_pairs - 1) / n_pairs : 0);
    auto item = [&](int j, int& tile, int& kb0, int& kb1) {
        if (dealt) run.item(j, tile, kb0, kb1);
        else { tile = pair + j * n_pairs; kb0 = 0; kb1 = n_kb; }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&acc_full[b]), 1); mbar_init(smem_u32(&acc_empty[b]), 8); }
        fence_barrier_init();
    }
    cluster.sync();                                             // both CTAs' barriers exist before anything arrives from the other side
    if (warp == 1) tmem_alloc_pair(smem_u32(&tmem_base_shared), 512);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_shared;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one in each CTA)
        if (lane == 0) {
            tt_pdl_wait();
            long long it = 0;
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; ++j) {
                int tile, kb0, kb1;
                item(j, tile, kb0, kb1);
                const int a_row = (tile % tiles_m) * 2 * BM + rank * BM;
                const int b_row = dual ? (rank == 0 ? 0 : args.up_row_offset) + (tile / tiles_m) * TILE_N
                                       : (tile / tiles_m) * TILE_N + rank * B_ROWS;
                for (int i = kb0; i < kb1; ++i, ++it) {
                    const int s = (int)(it % PAIR_STAGES);
                    if (!mbar_wait(smem_u32(&empty_bar[s]), (uint32_t)(((it / PAIR_STAGES) & 1) ^ 1))) {
                        atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; break;
                    }
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    if (rank == 0) mbar_expect_tx(bar, 2 * STAGE_TX);                // both CTAs' copies
                    uint8_t* stage = smem + (size_t)s * PAIR_STAGE_BYTES;
                    const int kx = i * BK;
                    tma_load_2d_pair(smem_u32(stage), &map_a, kx, a_row, bar);
                    tma_load_2d_pair(smem_u32(stage + BM * BK * 2), &map_b, kx, b_row, bar);
                }
            }
            // Every copy issued has landed once the products that read it are done, and the epilogue
            // warps wait for the last of those before the CTAs meet at the end.
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (the even CTA's)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instr_desc(2 * BM, dual ? 256 : WIDE);
            long long it = 0;
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const int buf = j & 1;
                // both CTAs' epilogues must have drained this accumulator (tiles j - 2, j - 4, ...)
                if (j >= 2 && !mbar_wait(smem_u32(&acc_empty[buf]), (uint32_t)(((j >> 1) & 1) ^ 1))) {
                    atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; break;
                }
                fence_after_sync();
                const uint32_t acc_addr = tmem_base + buf * 256;
                int tile, kb0, kb1;
                item(j, tile, kb0, kb1);
                for (int i = kb0; i < kb1; ++i, ++it) {
                    const int s = (int)(it % PAIR_STAGES);
                    if (!mbar_wait(smem_u32(&full_bar[s]), (uint32_t)((it / PAIR_STAGES) & 1))) {
                        atomicOr(args.status, TT_STATUS_WAIT_EXPIRED); ok = false; break;
                    }
                    fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * PAIR_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + BM * BK * 2;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk)
                        umma_bf16_pair(acc_addr, smem_desc(a_addr + kk * UMMA_K * 2), smem_desc(b_addr + kk * UMMA_K * 2), idesc,
                                       (i > kb0 || kk > 0) ? 1u : 0u);
                    umma_commit_pair(smem_u32(&empty_bar[s]), 3);          // the stage is free in both CTAs
                }
                if (ok) umma_commit_pair(smem_u32(&acc_full[buf]), 3);     // both CTAs' halves of the accumulator are complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (each CTA its own 128 rows)
        tt_pdl_wait();
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const bool bulk_out = (FORM == TOKENS_ON_M || dual) && args.bulk_out;
        uint8_t* slabs = smem + (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + quarter * OUT_SLAB_BYTES / 4;   // plain and SwiGLU forms
        int round = 0;
        for (int j = 0; j < my_tiles; ++j) {
            const int buf = j & 1;
            int tile, kb0, kb1;
            item(j, tile, kb0, kb1);
            const int token = (tile % tiles_m) * 2 * BM + rank * BM + row, f_base = (tile / tiles_m) * TILE_N;
            if (!dual && !bulk_out) prefetch_output_row(token, f_base, args);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256;
            const uint32_t acc_bar = smem_u32(&acc_full[buf]), acc_parity = (uint32_t)((j >> 1) & 1);
            bool ok;
            if constexpr (FORM == TOKENS_ON_M_QKV) {
                if constexpr (WIDE == 192) ok = qkv_row_epilogue<64, 192>(acc_bar, acc_parity, lane_addr, token, f_base, args);
                else ok = args.rope_head_dim == 64 ? qkv_row_epilogue<64, WIDE>(acc_bar, acc_parity, lane_addr, token, f_base, args)
                                                   : qkv_row_epilogue<128, WIDE>(acc_bar, acc_parity, lane_addr, token, f_base, args);
            } else {
                ok = mbar_wait(acc_bar, acc_parity);
                fence_after_sync();
            }
            if (!ok) {
                if (lane == 0) atomicOr(args.status, TT_STATUS_WAIT_EXPIRED);
                break;
            }
            if constexpr (FORM == TOKENS_ON_M) {
                if (dealt && kb0 > 0) {
                    // a share of a tile whose first k-blocks another pair has: into scratch memory, then the flag
                    store_share<WIDE>(lane_addr, share_of(args.shares, pair, rank, quarter), lane);
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) flag_release(share_flag_of(args.shares, n_pairs, pair, rank, quarter), 1u);
                } else if (dealt && kb1 < n_kb) {
                    // this pair writes the tile; the pairs behind it hold the rest of its k (at most two of them: the launcher
                    // deals k out only where a pair's run is at least half a tile long)
                    const long long tile_end = (long long)(tile + 1) * n_kb;
                    const float* share[2] = {nullptr, nullptr};
                    bool arrived = true;
                    for (int q = pair + 1, n = 0; q < n_pairs && k_run_of(q, n_pairs, tiles_total, n_kb).begin < tile_end; ++q, ++n) {
                        if (n == 2) { if (lane == 0) atomicOr(args.status, TT_STATUS_BAD_SHAPE); break; }
                        if (lane == 0) arrived = flag_wait(share_flag_of(args.shares, n_pairs, q, rank, quarter), 1u) && arrived;
                        share[n] = share_of(args.shares, q, rank, quarter);
                    }
                    arrived = __shfl_sync(0xffffffffu, arrived ? 1 : 0, 0) != 0;
                    __threadfence();
                    if (!arrived) {
                        if (lane == 0) atomicOr(args.status, TT_STATUS_WAIT_EXPIRED);
                        share[0] = share[1] = nullptr;
                    }
                    store_accumulator_bulk<WIDE>(lane_addr, token - lane, f_base, 0, args, &map_out, slabs, lane, round, share[0], share[1]);
                    __syncwarp();
                    if (lane == 0 && arrived) {                       // the flags as they were found, for the next launch
                        for (int q = pair + 1; q < n_pairs && k_run_of(q, n_pairs, tiles_total, n_kb).begin < tile_end; ++q)
                            *share_flag_of(args.shares, n_pairs, q, rank, quarter) = 0u;
                    }
                } else if (bulk_out) {
                    store_accumulator_bulk<WIDE>(lane_addr, token - lane, f_base, 0, args, &map_out, slabs, lane, round);
                } else {
                    store_accumulator<dual>(lane_addr, token, f_base, args);
                }
            } else if constexpr (dual) {
                if (bulk_out) store_swiglu_bulk(lane_addr, token - lane, f_base, args, &map_out, slabs, lane, round);
                else store_accumulator<dual>(lane_addr, token, f_base, args);
            }                                                                // the qkv form has stored its row
            // this warp is done with the accumulator: tell the issuer, who sits in the even CTA
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_even_cta(smem_u32(&acc_empty[buf]));
        }
        if (bulk_out && lane == 0) bulk_wait_group_read<0>();   // the slabs stay until the last copies have read them
    }
    fence_before_sync();
    __syncthreads();
    cluster.sync();                                             // nobody's shared or tensor memory goes while the other CTA may touch it
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// ------------------------------------------------------------------------- host side
// A [rows, k] bfloat16 matrix with `ld` elements between rows, read in boxes of box_rows x 64.
bool make_map(CUtensorMap* map, const void* base, long long rows, long long k, long long ld, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    return tc::make_map(map, base, 2, dims, strides, box);
}

template <int FORM, int BN, int STAGES, int GROUP = 1>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const Args& args, dim3 grid, cudaStream_t stream) {
    constexpr int shared = Shape<FORM, BN>::stage_bytes * STAGES + 1024;
    static bool configured = false;
    auto kernel = gemm_tcgen05_kernel<FORM, BN, STAGES, GROUP>;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
        if (err != cudaSuccess) return (int)err;
        configured = true;
    }
    tt_launch_pdl(kernel, grid, dim3(THREADS), shared, stream, map_a, map_b, args);
    return (int)cudaGetLastError();
}

template <int FORM, int WIDE = 256>
int launch_persistent(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_out, const Args& args, int tiles_m, int tiles_total,
                      int splits, cudaStream_t stream) {
    constexpr int shared = P_STAGE_BYTES * P_STAGES + 1024 + (FORM == TOKENS_ON_M || FORM == TOKENS_ON_M_SWIGLU ? OUT_SLAB_BYTES : 0);
    static bool configured = false;
    static int sm_count = 0;
    auto kernel = gemm_tcgen05_persistent_kernel<FORM, WIDE>;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
        if (err != cudaSuccess) return (int)err;
        int device = 0;
        if ((err = cudaGetDevice(&device)) != cudaSuccess) return (int)err;
        if ((err = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return (int)err;
        configured = true;
    }
    const int items = tiles_total * splits;
    const int ctas = items < sm_count ? items : sm_count;
    tt_launch_pdl(kernel, dim3(ctas), dim3(THREADS), shared, stream, map_a, map_b, map_out, args, tiles_m, tiles_total, splits);
    return (int)cudaGetLastError();
}

template <int FORM, int WIDE = 256>
int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_out, const Args& args, int tiles_m, int tiles_total,
                cudaStream_t stream) {
    constexpr int shared = PAIR_STAGE_BYTES * PAIR_STAGES + 1024 + (FORM == TOKENS_ON_M || FORM == TOKENS_ON_M_SWIGLU ? OUT_SLAB_BYTES : 0);
    static bool configured = false;
    static int sm_count = 0;
    auto kernel = gemm_tcgen05_pair_kernel<FORM, WIDE>;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
        if (err != cudaSuccess) return (int)err;
        int device = 0;
        if ((err = cudaGetDevice(&device)) != cudaSuccess) return (int)err;
        if ((err = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return (int)err;
        configured = true;
    }
    // with the tiles' k-blocks dealt out (args.shares) every pair has work even where the tiles are fewer than the pairs
    const int pairs = (tiles_total < sm_count / 2 && !args.shares) ? tiles_total : sm_count / 2;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * pairs);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = 2;
    attribute[1].val.clusterDim.y = 1;
    attribute[1].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 2;
    const cudaError_t err = cudaLaunchKernelEx(&config, kernel, map_a, map_b, map_out, args, tiles_m, tiles_total);
    return err != cudaSuccess ? (int)err : (int)cudaGetLastError();
}

int undelivered_bytes_for_tests = 0;

}  // namespace

// For tests of the failure path only.  The limit of every bounded wait in this library, in
// nanoseconds (0: back to the default of two seconds).
extern "C" int tt_gemm_tcgen05_set_wait_limit_ns(unsigned long long ns) { return tc::set_wait_limit_ns(ns); }
// From now on the first stage of every CTA of the few-token and small-prompt kernel expects `bytes`
// more than its copies deliver (0: back to normal): its barrier never completes, every wait on
// it runs out, and the kernel has to raise TT_STATUS_WAIT_EXPIRED, free its tensor memory and return.
extern "C" void tt_gemm_tcgen05_expect_undelivered_bytes(int bytes) { undelivered_bytes_for_tests = bytes < 0 ? 0 : bytes; }

// The qkv projection of a prompt with rotation, narrowing and the cache append in the epilogue:
// x [tokens, k] @ w[q_cols + 2 kv_cols, k]^T (+ bias); q rotated to q_out (bfloat16 [tokens, q_cols]), k rotated and
// v as they are into the block pools at each token's position.  cos_sin and where come from tt_rope_table
// (elementwise.cu).  Only for the shapes the persistent and CTA-pair kernels run without slicing k (the caller asks
// tt_gemm_tcgen05_qkv_rope_takes first) and head sizes 64 and 128 rotated whole.  Returns a cudaError_t value, -1
// if a tensor map could not be made, -2 if the shape is not taken.
// Tile width of the qkv form below the pairs' range, 0 where the form is not taken.  The form does not slice k, so it is
// taken where the plain product would not slice either: with more tiles of 256 features than half the SMs, or, failing
// that, with more tiles of 128 features than half the SMs.  Slices and a rotation kernel of its own are faster only where
// even those are few (measured on a B200, 1B shape, whole prefill: 1,024 tokens = 96 tiles of 256: 2.91 -> 2.77 ms with
// this form; 768 and 512 tokens with tiles of 256: 2.43 -> 2.46 and 2.00 -> 2.07 ms, one SM per tile for all of k).
static int qkv_rope_tile_width(int tokens, int features) {
    int device = 0, sm_count = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    const int tiles_m = (tokens + BM - 1) / BM;
    if (tiles_m * ((features + 255) / 256) * 2 > sm_count) return 256;
    if (tiles_m * ((features + 127) / 128) * 2 > sm_count) return 128;
    return 0;
}

extern "C" int tt_gemm_tcgen05_qkv_rope_takes(int tokens, int features, int k, int head_dim) {
    if (head_dim != 64 && head_dim != 128) return 0;
    if (tokens <= 128 || features % head_dim) return 0;
    const int tiles = ((tokens + BM - 1) / BM) * ((features + 255) / 256);
    if (tiles < 8) return 0;
    if (tokens >= PAIR_MIN_TOKENS) return 1;
    return qkv_rope_tile_width(tokens, features) ? 1 : 0;
}

extern "C" int tt_gemm_tcgen05_qkv_rope(const void* x, long long ldx, const void* w, long long ldw, const float* bias, int tokens, int k,
                                        void* q_out, void* k_pool, void* v_pool, const void* cos_sin, const void* where, const int* table,
                                        int table_width, int pool_blocks, int heads, int kv_heads, int head_dim, float attention_scaling,
                                        unsigned* status, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int q_cols = heads * head_dim, kv_cols = kv_heads * head_dim, features = q_cols + 2 * kv_cols;
    if (k <= 0 || (k % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)q_out & 15) ||
        ((uintptr_t)k_pool & 15) || ((uintptr_t)cos_sin & 15))
        return (int)cudaErrorInvalidValue;
    if (!tt_gemm_tcgen05_qkv_rope_takes(tokens, features, k, head_dim)) return -2;
    Args args = {};
    args.bias = bias; args.tokens = tokens; args.features = features; args.k = k;
    args.k_blocks_per_split = (k + BK - 1) / BK;
    args.status = status;
    args.rope_head_dim = head_dim;
    args.rope.q_out = (__nv_bfloat16*)q_out; args.rope.k_pool = (__nv_bfloat16*)k_pool; args.rope.v_pool = (__nv_bfloat16*)v_pool;
    args.rope.cos_sin = (const float2*)cos_sin; args.rope.where = (const int2*)where; args.rope.table = table;
    args.rope.table_width = table_width; args.rope.pool_blocks = pool_blocks; args.rope.q_cols = q_cols; args.rope.kv_cols = kv_cols;
    args.rope.kv_heads = kv_heads; args.rope.attention_scaling = attention_scaling;
    CUtensorMap map_a, map_b;
    const int tiles_m = (tokens + BM - 1) / BM;
    if (tokens < PAIR_MIN_TOKENS) {
        if (qkv_rope_tile_width(tokens, features) == 128) {
            if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, features, k, ldw, 128)) return -1;
            return launch_persistent<TOKENS_ON_M_QKV, 128>(map_a, map_b, map_a, args, tiles_m, tiles_m * ((features + 127) / 128), 1, stream);
        }
        if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, features, k, ldw, 256)) return -1;
        return launch_persistent<TOKENS_ON_M_QKV>(map_a, map_b, map_a, args, tiles_m, tiles_m * ((features + 255) / 256), 1, stream);
    }
    const int pair_tiles_m = (tokens + 2 * BM - 1) / (2 * BM);
    if (head_dim == 64) {
        // tiles of 192 features where the pairs' rounds times the tile's width come out shorter than with 256
        int device = 0, sm_count = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
        const long long pairs = sm_count / 2 > 0 ? sm_count / 2 : 1;
        auto cost = [&](int wide) { return ((long long)pair_tiles_m * ((features + wide - 1) / wide) + pairs - 1) / pairs * wide; };
        if (cost(192) < cost(256)) {
            if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, features, k, ldw, 96)) return -1;
            return launch_pair<TOKENS_ON_M_QKV, 192>(map_a, map_b, map_a, args, pair_tiles_m, pair_tiles_m * ((features + 191) / 192), stream);
        }
    }
    if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, features, k, ldw, 128)) return -1;
    return launch_pair<TOKENS_ON_M_QKV>(map_a, map_b, map_a, args, pair_tiles_m, pair_tiles_m * ((features + 255) / 256), stream);
}

// How many tokens the features-on-m form takes at most.
extern "C" int tt_gemm_tcgen05_max_skinny_tokens() { return 128; }

// Operands must be 16-byte aligned with row strides that are multiples of 8 elements.
// form: 0 float32 partial sums out[splits][tokens][features]; 1 SwiGLU, out bfloat16
// [tokens][features] with w holding `features` gate rows then `features` up rows; 2 the product
// (+ bias) is added to float32 out[tokens][features]: prompts that run the persistent or the
// CTA-pair kernel with one k-slice only (every tile has one writer), anything else is refused.
// Returns a cudaError_t value, or -1 if the driver's tensor-map encoder is unavailable
// or refused the operands.
// shares, shares_bytes: scratch memory of at least tt_gemm_tcgen05_shares_bytes() whose flag words (its tail) are zero,
// or null.  With it, the CTA pairs' plain form deals the tiles' k-blocks out evenly where whole tiles would leave
// pairs idle (see deals_k_out); the flags are zero again when the kernel ends.
extern "C" long long tt_gemm_tcgen05_shares_bytes() {
    int device = 0, sm_count = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    return (long long)(sm_count / 2) * 8 * (SHARE_FLOATS * 4 + 4);
}

// Whether dealing k out pays: with whole tiles the pairs would work `rounds` rounds of which the last is part empty.
// A tile's k may be shared by three pairs at most (its first pair adds two shares), so a pair's run must be at least
// half a tile long; and a run needs a few k-blocks to be worth a share's trip through scratch memory.  While all
// pairs are busy the products are bound by what the L2 delivers to the SMs together (64 KB per k-block and pair,
// about 11 TB/s), not by the number of busy pairs, so only a last round that is mostly empty is worth filling.
// Measured on a B200, whole prefill of the 1B shape (o and down dealt out / whole tiles, share of the pairs' rounds
// that tiles fill): 2,560 tokens 5.17 / 5.54 ms (0.54), 3,000 tokens 6.20 / 6.32 (0.65), 4,864 tokens 10.91 / 11.01
// (0.68), but 3,584 tokens 7.61 / 7.39 (0.76), 5,632 tokens 13.56 / 13.12 (0.79), 2,048 tokens 4.44 / 3.97 (0.86).
static bool deals_k_out(int tiles, int pairs, int k_blocks) {
    if (pairs < 2 || tiles * 2 <= pairs + 1 || k_blocks < 16) return false;
    const int rounds = (tiles + pairs - 1) / pairs;
    return (long long)tiles * 100 < (long long)rounds * pairs * 70;
}

extern "C" int tt_gemm_tcgen05(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* out,
                               long long ld_out, long long split_stride, int tokens, int features, int k, int splits,
                               int form, unsigned* status, cudaStream_t stream, void* shares, long long shares_bytes) {
    if (tokens <= 0 || features <= 0) return 0;
    if (k <= 0 || (k % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || splits < 1)
        return (int)cudaErrorInvalidValue;
    const int k_blocks = (k + BK - 1) / BK;
    if (splits > k_blocks) splits = k_blocks;
    Args args;
    args.bias = bias; args.out = out; args.ld_out = ld_out; args.split_stride = split_stride;
    args.tokens = tokens; args.features = features; args.k = k;
    args.k_blocks_per_split = (k_blocks + splits - 1) / splits;
    args.up_row_offset = features; args.status = status;
    args.accumulate = form == 2 ? 1 : 0;
    args.undelivered_bytes = undelivered_bytes_for_tests;
    args.bulk_out = 0;
    args.shares = nullptr;
    CUtensorMap map_a, map_b;
    const int tiles_m = (tokens + BM - 1) / BM;
    if (form == 2 && !(tokens > 128 && tiles_m * ((features + 255) / 256) >= 8 && splits == 1)) return (int)cudaErrorInvalidValue;
    if (form == 1) {
        if (splits != 1 || bias) return (int)cudaErrorInvalidValue;
        if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, 2LL * features, k, ldw, 128)) return -1;
        if (tokens <= 128) {
            // few tokens: features on the 128-row side, 64 gate rows paired with their 64 up rows
            const int bn = tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : 128;
            if (!make_map(&map_a, w, 2LL * features, k, ldw, BM / 2) || !make_map(&map_b, x, tokens, k, ldx, bn)) return -1;
            const dim3 grid(1, (features + BM / 2 - 1) / (BM / 2), 1);
            switch (bn) {
                case 16: return launch<FEATURES_ON_M_SWIGLU, 16, 6>(map_a, map_b, args, grid, stream);
                case 32: return launch<FEATURES_ON_M_SWIGLU, 32, 5>(map_a, map_b, args, grid, stream);
                case 64: return launch<FEATURES_ON_M_SWIGLU, 64, 4>(map_a, map_b, args, grid, stream);
                default: return launch<FEATURES_ON_M_SWIGLU, 128, 3>(map_a, map_b, args, grid, stream);
            }
        }
        const int tiles = tiles_m * ((features + 127) / 128);
        // the activations leave through shared memory and tiled copies where those can write their rows (16-byte aligned,
        // a multiple of 16 bytes apart): boxes of 64 features x 32 tokens
        CUtensorMap map_out = map_a;
        if (tiles >= 8 && (ld_out % 8) == 0 && (((uintptr_t)out) & 15) == 0) {
            const cuuint64_t dims[2] = {(cuuint64_t)features, (cuuint64_t)tokens};
            const cuuint64_t strides[1] = {(cuuint64_t)ld_out * 2};
            const cuuint32_t box[2] = {64, 32};
            args.bulk_out = tc::make_map(&map_out, out, 2, dims, strides, box) ? 1 : 0;
        }
        if (tiles >= 8 && tokens < PAIR_MIN_TOKENS_SWIGLU) return launch_persistent<TOKENS_ON_M_SWIGLU>(map_a, map_b, map_out, args, tiles_m, tiles, 1, stream);
        if (tiles >= 8) {
            const int pair_tiles_m = (tokens + 2 * BM - 1) / (2 * BM);
            return launch_pair<TOKENS_ON_M_SWIGLU>(map_a, map_b, map_out, args, pair_tiles_m, pair_tiles_m * ((features + 127) / 128), stream);
        }
        const dim3 grid((features + 127) / 128, tiles_m, 1);
        return launch<TOKENS_ON_M_SWIGLU, 128, 4>(map_a, map_b, args, grid, stream);
    }
    // no slice may be empty in the persistent kernel (the generic kernel below writes zeros for one)
    const bool slices_full = (long long)(splits - 1) * args.k_blocks_per_split < k_blocks;
    if (tokens > 128 && tiles_m * ((features + 255) / 256) >= 8 && (splits == 1 || (tokens < PAIR_MIN_TOKENS && slices_full))) {
        // The tiles leave through shared memory and tiled copies where those can write the output's rows: 16-byte aligned
        // and a multiple of 16 bytes apart (the k-slices' planes too).
        CUtensorMap map_out = {};
        args.bulk_out = (ld_out % 4) == 0 && (splits == 1 || (split_stride % 4) == 0) && (((uintptr_t)out) & 15) == 0 &&
                        make_map_f32_out(&map_out, out, splits, tokens, features, ld_out, split_stride) ? 1 : 0;
        // from 8 tiles of 128 x 256 on the persistent kernel wins (measured); fewer tiles than SMs are cut along k
        if (tokens < PAIR_MIN_TOKENS) {
            // Where tiles of 256 features would fill at most an eighth of the SMs (prompts of up to 256 tokens at the 1B
            // shape), tiles of 128 features are taken and k is sliced half as often: an item's epilogue (10,200 cycles for
            // 128 x 256 numbers) then weighs half as much against its few products.  Measured on a B200, 1B shape, whole
            // prefill: 200 tokens 1.54 -> 1.43 ms, 256 tokens 1.60 -> 1.44; at 320 and 384 tokens nothing either way, and
            // from 512 tokens on the narrow tiles lose (512: 1.76 -> 1.83, 768: 2.16 -> 2.50: a k-block then brings 32 KB
            // into shared memory for half the products).  gemm_tcgen05_splits (kernels/api.py) counts the tiles the same way.
            int device = 0, sm_count = 0;
            if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
            if (form == 0 && tiles_m * ((features + 255) / 256) * 8 <= sm_count) {
                if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, features, k, ldw, 128)) return -1;
                return launch_persistent<TOKENS_ON_M, 128>(map_a, map_b, map_out, args, tiles_m, tiles_m * ((features + 127) / 128), splits, stream);
            }
            if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, features, k, ldw, 256)) return -1;
            return launch_persistent<TOKENS_ON_M>(map_a, map_b, map_out, args, tiles_m, tiles_m * ((features + 255) / 256), splits, stream);
        }
        if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, features, k, ldw, 128)) return -1;
        const int pair_tiles_m = (tokens + 2 * BM - 1) / (2 * BM);
        const int pair_tiles = pair_tiles_m * ((features + 255) / 256);
        if (args.bulk_out && shares && (((uintptr_t)shares) & 15) == 0 && shares_bytes >= tt_gemm_tcgen05_shares_bytes()) {
            int device = 0, sm_count = 0;
            if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
            if (deals_k_out(pair_tiles, sm_count / 2, k_blocks)) args.shares = (float*)shares;
        }
        return launch_pair<TOKENS_ON_M>(map_a, map_b, map_out, args, pair_tiles_m, pair_tiles, stream);
    }
    if (tokens > 128) {
        if (!make_map(&map_a, x, tokens, k, ldx, BM) || !make_map(&map_b, w, features, k, ldw, 128)) return -1;
        const dim3 grid((features + 127) / 128, (tokens + BM - 1) / BM, splits);
        return launch<TOKENS_ON_M, 128, 3>(map_a, map_b, args, grid, stream);
    }
    const int bn = tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : 128;
    if (!make_map(&map_a, w, features, k, ldw, BM) || !make_map(&map_b, x, tokens, k, ldx, bn)) return -1;
    const dim3 grid(1, (features + BM - 1) / BM, splits);
    switch (bn) {
        case 16: return launch<FEATURES_ON_M, 16, 6, 2>(map_a, map_b, args, grid, stream);
        case 32: return launch<FEATURES_ON_M, 32, 5>(map_a, map_b, args, grid, stream);
        case 64: return launch<FEATURES_ON_M, 64, 4>(map_a, map_b, args, grid, stream);
        default: return launch<FEATURES_ON_M, 128, 3>(map_a, map_b, args, grid, stream);
    }
}

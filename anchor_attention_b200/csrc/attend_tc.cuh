// Steps 1 and 3 on the Blackwell tensor cores (tcgen05 + tensor memory + TMA).
//
// One CTA owns 256 query rows of one head (two 128-row tiles A and B that lie
// in the same big block and therefore share their key/value tiles) and walks a
// list of 128-row key/value tiles:
//
//   kWindow  (step 1)  contiguous tiles of [0, min(G, end)) U [max(b*G, that), end),
//            end = last query row + 1; additive -1e6 causal mask on diagonal tiles;
//            query scaled with dtype-rounded constants; writes M, L, Acc (Acc in 128-row
//            chunk-major tiles, see acc_tile()).
//            Reference: anchor_attn/src/ops/anchor_step_1_2_v2.py:8-161.
//   kStripe  (step 3)  tiles of 128 ids from the big block's id list; state starts
//            from step 1's (M, L, Acc); slots past the count masked to -inf;
//            writes bf16(acc / l).  Reference: anchor_attn/src/ops/anchor_attn_v4.py:7-105.
//   kBlock   (block-granular comparator)  whole 128-row key blocks from the merged block list
//            of the CTA's two query tiles; an entry says which of the two tiles attends it (the
//            other one gets no products for it); -inf causal mask on a tile's own block;
//            state starts empty; writes bf16(acc / l).
//            Reference: anchor_attn/src/ops/block_sparse_flash_attention_v2.py:10-110.
//            Its dense causal variant (the last q rows of a longer sequence attend every key up
//            to their own position; lists made up on the fly, mask placed by position) serves
//            the tail of a prefill and later prefill chunks
//            (anchor_attn/src/modules/llama/anchor_attention.py:76-88, 101-113).
//
// Warp roles (384 threads):
//   warps 0-3   softmax of tile A: thread r owns query row r = tensor-memory lane r
//   warps 4-7   softmax of tile B
//   warp  8     MMA issuer (one elected lane): S = Q K^T and O += P V with tcgen05.mma
//   warps 9-11  loaders, into a 5-slot ring of 32 KB tiles: one TMA box load for a run of 128
//               consecutive rows; one bulk copy for a tile the gather pass (gather.cuh) put
//               into scratch; discrete rows without a scratch slot are split between TMA row
//               gathers (tile::gather4, four rows per instruction, warp 9) and 16-byte
//               cp.async copies (warps 10-11; all three warps for stride patterns no 2-D
//               tensor map covers)
//
// Tensor memory (512 columns): S_A | S_B | O_A | O_B, 128 fp32 columns each.  P (bf16)
// overwrites the first 64 columns of its S and is consumed from tensor memory as
// the A operand of the P V product.
//
// The running maximum used as the exponent reference is only moved when the
// true maximum has grown by more than 8 (a factor 256), and the accumulator in
// tensor memory is rescaled only then; the final scaling makes the result equal
// to the eager recurrence up to rounding.
//
// Every wait is bounded (tc_ptx.cuh); a wait that gives up sets the status word
// and the CTA drains and frees its tensor memory.
#pragma once
#include "common.cuh"
#include "tc_ptx.cuh"

namespace aa {
namespace tc {

constexpr int kLoaderWarps = 3;                        // warps 9 .. 11
constexpr int kThreads = (9 + kLoaderWarps) * 32;
constexpr int kSoftmaxRegs = 208;                      // registers per thread after setmaxnreg: softmax warps
constexpr int kOtherRegs = 88;                         //                                        MMA and loader warps
// setmaxnreg only moves registers between the warps of the CTA: what the CTA gets at launch
// (64 K registers / threads, rounded down to a multiple of 8, per thread) must cover the
// re-allocated sizes, or the growing warps wait for ever.  Warps re-allocate in groups of four.
static_assert(kThreads * (65536 / kThreads / 8 * 8) >= 256 * kSoftmaxRegs + (kThreads - 256) * kOtherRegs,
              "register re-allocation exceeds the CTA's registers");
constexpr int kStages = 5;
constexpr int kTile = 128;                        // rows per query tile and per key tile
constexpr int kTileBytes = kTile * kRowBytes;     // 32 KB
constexpr int kSlabBytes = kTileBytes / 2;        // 64 columns x 128 rows, one swizzle slab
constexpr int kSmemQ = 2 * kTileBytes;
constexpr int kSmemRing = kStages * kTileBytes;
constexpr int kSmemBars = 256;
constexpr int kSmemTotal = kSmemQ + kSmemRing + kSmemBars + 1024;   // + slack to align to 1024
constexpr float kRescaleThreshold = 8.0f;
constexpr uint32_t kTmemCols = 512;

constexpr int kMaxPeers = 8;

struct TcArgs {
    AttendArgs a;
    int kpos_n, kpos_h, kpos_b;      // which tensor-map coordinate (1..3 -> 0..2) carries n / head / batch
    int vpos_n, vpos_h, vpos_b;
    int k_gather, v_gather;          // 1: the 2-D row-gather tensor map of K / V is usable
    int list_stride;                 // kBlock only: entries reserved per query-tile pair in a.ids
    // kBlock, dense causal variant (the tail of a prefill, a later prefill chunk): no lists; the query
    // rows are the LAST q_rows positions of a kv_rows-long sequence (a.N = the rows rounded up to
    // 256), row i attends every key up to position q_off + i, q_off = kv_rows - q_rows
    int dense, q_rows, q_off, kv_blocks;
    const int32_t* tile_slot;        // step 3 only: gather slot of every id tile ([B*H, ids_per_head/128]) or NULL
    const uint8_t* gather;           // step 3 only: the 64 KB slots (K image, V image) the gather pass filled
    int n_slots;                     // step 3 only: slots in `gather`; a table entry beyond it is ignored
    int n_peers;                     // step 3 only: > 0 -> write the output to peers[0 .. n_peers) instead of a.out
    int rows_per_peer;               // with n_peers > 0: 0 -> every row goes to every peer; > 0 -> row n goes only to
                                     // peer n / rows_per_peer, at row n % rows_per_peer of that peer's buffer
    __nv_bfloat16* peers[kMaxPeers]; // same element offsets and strides as a.out; may be other GPUs' memory
    int32_t* status;
};

constexpr int kTmaRows = 32;                // rows of a gathered tile fetched by TMA row gathers (multiple of 4)
constexpr int kPParts = 2;                  // P is handed to the MMA warp in two halves

// byte offset of (row, 16-byte chunk) inside a 32 KB tile made of two 128B-swizzled slabs
__device__ __forceinline__ uint32_t sw_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * kSlabBytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// The un-normalised fp32 output of step 1 (the reference's Acc_buffer, anchor_step_1_2_v2.py:176)
// is private to steps 1 and 3, and both touch it with one thread per row.  It is therefore kept in
// tiles of 128 rows (64 KB, tile t = rows 128t .. 128t+127 of a (batch, head)), each tile
// chunk-major: the 16-byte chunk k (columns 4k .. 4k+3) of all 128 rows is one 2 KB run, row r at
// offset 16 r.  A warp whose lane r reads or writes chunk k of row r then touches 512 contiguous
// bytes, instead of 32 lines 512 bytes apart as it would with row-major rows.
__device__ __forceinline__ float* acc_tile(float* acc, int64_t hz, int N, int qb) {
    return acc + ((int64_t)hz * N + (int64_t)qb * kTile) * kD;
}
__device__ __forceinline__ int acc_chunk_off(int k, int r) { return k * (kTile * 4) + r * 4; }      // in floats

__device__ __forceinline__ void tma_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, int pos_n, int pos_h,
                                         int pos_b, int row, int head, int z) {
    const int c0 = pos_n == 0 ? row : (pos_h == 0 ? head : z);
    const int c1 = pos_n == 1 ? row : (pos_h == 1 ? head : z);
    const int c2 = pos_n == 2 ? row : (pos_h == 2 ? head : z);
    tma_load_4d(dst, map, bar, 0, c0, c1, c2);
    tma_load_4d(dst + kSlabBytes, map, bar, 64, c0, c1, c2);
}

// Entry t of a block-mode CTA's tile list: read from the merged list, or, in the dense causal
// variant, made up on the spot -- key block t, attended by both query tiles up to the first
// tile's last block and by the second tile alone beyond it.
__device__ __forceinline__ uint32_t block_entry(const TcArgs& ta, const int32_t* list, int t, int dense_last0) {
    if (ta.dense) return (uint32_t)t | ((t <= dense_last0 ? 3u : 2u) << kBlockFlagShift);
    return (uint32_t)list[t];
}

// What the softmax warps need to know about their CTA: where the tiles and barriers are.
// q_full / p_part are arrived on, s_full / o_done are waited on.
struct SoftmaxCtx {
    uint8_t* smem;
    uint32_t tmem_base;
    volatile int* abort_flag;
    uint32_t q_full[2], s_full[2], o_done[2], p_part[2][4];
    int pair, z, h, hz, ntiles, n_init, local_start, count;
    const int32_t* list;             // kBlock only: the pair's tile list
    int dense_last0;                 // kBlock, dense variant: last key block of the pair's first query tile
};

// The softmax role of warps 0-7 (see the file header): thread r of tile j owns query row r.
template <int MODE>
__device__ __forceinline__ void softmax_role(const TcArgs& ta, const SoftmaxCtx& cx, int tid) {
    const AttendArgs& a = ta.a;
    const int warp = tid >> 5;
    uint8_t* smem = cx.smem;
    const uint32_t tmem_base = cx.tmem_base;
    volatile int* abort_flag = cx.abort_flag;
    const int pair = cx.pair, z = cx.z, h = cx.h, hz = cx.hz;
    const int ntiles = cx.ntiles, n_init = cx.n_init, local_start = cx.local_start, count = cx.count;
    (void)n_init; (void)local_start; (void)count;
    const int j = warp >> 2;
    const uint32_t q_full_j = cx.q_full[j], s_full_j = cx.s_full[j], o_done_j = cx.o_done[j];
    uint32_t p_part_j[kPParts];
#pragma unroll
    for (int q = 0; q < kPParts; ++q) p_part_j[q] = cx.p_part[j][q];
    const int r = tid & 127;
    const int qb = 2 * pair + j;
    const int row_g = qb * kTile + r;
    const int64_t srow = (int64_t)hz * a.N + row_g;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + (uint32_t)j * 128u;
    const uint32_t tO = tmem_base + lane_base + 256u + (uint32_t)j * 128u;

    // Q tile: load, scale, round, store in the K-major 128B-swizzled layout the MMA reads
    // (not needed when there is no key tile to multiply it with)
    if (ntiles > 0) {
        const __nv_bfloat16* qbase = a.q.ptr + z * a.q.sb + h * a.q.sh + (int64_t)qb * kTile * a.q.sn;
        const __nv_bfloat162 c1b = __float2bfloat162_rn(a.sm_scale), c2b = __float2bfloat162_rn(kLog2e);
        uint8_t* qs = smem + j * kTileBytes;
        // all sixteen loads of the thread are issued before the first one is used
        uint4 raws[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int id = r + 128 * i;
            if (MODE == kBlock && qb * kTile + (id >> 4) >= ta.q_rows)
                raws[i] = make_uint4(0u, 0u, 0u, 0u);          // padding rows of the dense variant
            else
                raws[i] = *reinterpret_cast<const uint4*>(qbase + (int64_t)(id >> 4) * a.q.sn + (id & 15) * 8);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int id = r + 128 * i;
            const int rr = id >> 4, ch = id & 15;
            uint4 raw = raws[i];
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (MODE == kWindow) {
                    // bf16(bf16(q * c1) * c2) with bf16 constants: a product of two bf16 values is exact
                    // in fp32, so the packed bf16 multiply (one rounding) gives the same bits
                    p2[e] = __hmul2(__hmul2(p2[e], c1b), c2b);
                } else if (MODE == kBlock) {
                    // bf16(q * (sm_scale * log2e)): the constants are multiplied first
                    const float qk = __fmul_rn(a.sm_scale, kLog2e);
                    float2 f = __bfloat1622float2(p2[e]);
                    p2[e] = __floats2bfloat162_rn(__fmul_rn(f.x, qk), __fmul_rn(f.y, qk));
                } else {
                    float2 f = __bfloat1622float2(p2[e]);
                    f.x = __fmul_rn(__fmul_rn(f.x, a.sm_scale), kLog2e);
                    f.y = __fmul_rn(__fmul_rn(f.y, a.sm_scale), kLog2e);
                    p2[e] = __floats2bfloat162_rn(f.x, f.y);
                }
            }
            *reinterpret_cast<uint4*>(qs + sw_off(rr, ch)) = raw;
        }
        fence_proxy_async();
        mbar_arrive(q_full_j);
    }

    float m_true, m_ref, l;
    if (MODE == kStripe) {
        m_true = m_ref = a.M[srow];
        l = a.L[srow];
        if (ntiles > 0) {
            const float* tile_acc = acc_tile(a.Acc, hz, a.N, qb);
            // all 32 loads of the row are issued before the first tensor-memory store (the stores
            // are ordered against memory operations, so loads behind one would wait for it)
            uint32_t v[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 x = *reinterpret_cast<const float4*>(tile_acc + acc_chunk_off(c * 8 + i, r));
                    v[c][4 * i] = __float_as_uint(x.x);
                    v[c][4 * i + 1] = __float_as_uint(x.y);
                    v[c][4 * i + 2] = __float_as_uint(x.z);
                    v[c][4 * i + 3] = __float_as_uint(x.w);
                }
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_st32(tO + c * 32, v[c]);
            tmem_wait_st();
        }
    } else {
        m_true = m_ref = -INFINITY;
        l = 0.f;
    }

    auto signal = [&](uint32_t bar) {
        tmem_wait_st();
        tcgen05_fence_before();
        // one arrival per warp: 128 arrivals on one barrier would queue up behind each other
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar);
    };
    uint32_t entry_next = (MODE == kBlock && ntiles > 0) ? block_entry(ta, cx.list, 0, cx.dense_last0) : 0u;
    int mine = 0;        // kBlock: tiles of this query tile so far (the MMA warp counts the same way)
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
        const uint32_t entry = entry_next;
        if (MODE == kBlock) {
            if (t + 1 < ntiles) entry_next = block_entry(ta, cx.list, t + 1, cx.dense_last0);
            // a block of the other query tile only: no S is produced for this one, nothing to do
            if (!((entry >> (kBlockFlagShift + j)) & 1u)) continue;
        }
        const int seq = (MODE == kBlock) ? mine : t;      // which of this tile's score tiles
        ++mine;
        ok = mbar_wait(s_full_j, seq & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        uint32_t sv[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sv[c]);
        tmem_wait_ld();

        if (MODE == kWindow) {
            const int col0 = (t < n_init) ? t * kTile : local_start + (t - n_init) * kTile;
            if (col0 + kTile - 1 > qb * kTile) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + c * 32 + i > row_g)
                            sv[c][i] = __float_as_uint(__uint_as_float(sv[c][i]) + -1e6f);
            }
        } else if (MODE == kBlock) {
            // keys after the query row: d = position of the tile's first query row minus the block's
            // first key (0 on the tile's own block of the comparator; any value in the dense variant)
            const int d = ta.q_off + (qb - (int)(entry & kBlockIdMask)) * kTile;
            if (d < kTile - 1) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i > r + d) sv[c][i] = __float_as_uint(-INFINITY);
            }
        } else {
            const int valid = count - t * kTile;
            if (valid < kTile) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i >= valid) sv[c][i] = __float_as_uint(-INFINITY);
            }
        }
        {   // row maximum: four independent chains of three-input max
            float mx[4] = {m_true, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                    mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
            m_true = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        }
        // move the exponent reference only when some row of the warp needs it
        if (__any_sync(0xffffffffu, m_true > m_ref + kRescaleThreshold)) {
            const float alpha = fast_exp2(m_ref - m_true);
            if (!(MODE != kStripe && seq == 0)) {     // nothing accumulated yet when the state starts empty
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tO + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st32(tO + c * 32, v);
                }
            }
            l *= alpha;
            m_ref = m_true;
        }
        float2 rs[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        const float2 neg_ref = make_float2(-m_ref, -m_ref);
        // P goes to the MMA warp in two halves of 64 key columns (32 packed tensor-memory columns),
        // each enough for four k-steps of P V, so that P V starts while the second half is computed.
        // (Four parts, or signalling the first half later so that its store completes in the shadow of
        // the second half's arithmetic, measured slower or equal.)
        auto exp_pairs = [&](uint32_t (&pk)[32], int c, int i_begin, int i_end) {
#pragma unroll
            for (int i = i_begin; i < i_end; ++i) {
                const int e = c * 64 + 2 * i;
                const float2 d = __fadd2_rn(make_float2(__uint_as_float(sv[e >> 5][e & 31]),
                                                        __uint_as_float(sv[(e + 1) >> 5][(e + 1) & 31])), neg_ref);
                const float2 p = make_float2(fast_exp2(d.x), fast_exp2(d.y));
                rs[i & 3] = __fadd2_rn(rs[i & 3], p);
                pk[i] = pack_bf16x2(p.x, p.y);
            }
        };
        uint32_t pk0[32], pk1[32];
        exp_pairs(pk0, 0, 0, 32);
        tmem_st32(tS, pk0);
        signal(p_part_j[0]);
        exp_pairs(pk1, 1, 0, 32);
        tmem_st32(tS + 32, pk1);
        signal(p_part_j[1]);
        const float2 rsum = __fadd2_rn(__fadd2_rn(rs[0], rs[1]), __fadd2_rn(rs[2], rs[3]));
        l += rsum.x + rsum.y;
    }

    // ---- epilogue ----
    if (ok && ntiles > 0) {
        ok = mbar_wait(o_done_j, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tcgen05_fence_after();
    }
    if (MODE == kWindow) {
        // All 128 threads of the tile get here; they first agree that none of them gave up.  The fp32
        // accumulator goes out in the tile layout of acc_tile(): thread r stores the 16-byte chunks
        // of its row, a warp 512 contiguous bytes per instruction, straight from registers.
        const bool all_ok = bar_and(1 + j, 128, ok);
        if (all_ok) {
            const float sc = fast_exp2(m_ref - m_true);
            a.M[srow] = m_true;
            a.L[srow] = l * sc;
            float* tile_acc = acc_tile(a.Acc, hz, a.N, qb);
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(tO + c * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 x = make_float4(__uint_as_float(v[4 * i]) * sc, __uint_as_float(v[4 * i + 1]) * sc,
                                                 __uint_as_float(v[4 * i + 2]) * sc, __uint_as_float(v[4 * i + 3]) * sc);
                    *reinterpret_cast<float4*>(tile_acc + acc_chunk_off(c * 8 + i, r)) = x;
                }
            }
        }
    } else {
        // The 128 rows of the tile are staged in shared memory (the tile's query buffer, which
        // no MMA reads any more) and then written out as whole 256-byte rows by consecutive
        // threads: coalesced stores, which matters most when the destination is another GPU.
        // All 128 threads of the tile get here; they first agree that none of them gave up.
        const bool all_ok = bar_and(1 + j, 128, ok);
        if (all_ok) {
            uint8_t* stage = smem + j * kTileBytes;
            // acc / l, correctly rounded: one IEEE reciprocal of l per row, then the quotient estimate
            // acc * (1/l) corrected once with the exact remainder (two fused multiply-adds).  Equals the
            // IEEE quotient for normal operands, at a third of the instructions of a division.
            if (MODE == kBlock && ntiles == 0) l = 1.f;          // an empty list: zeros (the lists are never empty)
            const float rl = __frcp_rn(l);
            auto div_l = [&](float x) {
                const float q0 = __fmul_rn(x, rl);
                const float rem = __fmaf_rn(-q0, l, x);
                return __fmaf_rn(rem, rl, q0);
            };
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                if (ntiles > 0) {
                    tmem_ld32(tO + c * 32, v);
                    tmem_wait_ld();
                } else {                 // block mode with an empty list (step 3 never gets here without tiles)
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 o4;
                    o4.x = pack_bf16x2(div_l(__uint_as_float(v[8 * i])), div_l(__uint_as_float(v[8 * i + 1])));
                    o4.y = pack_bf16x2(div_l(__uint_as_float(v[8 * i + 2])), div_l(__uint_as_float(v[8 * i + 3])));
                    o4.z = pack_bf16x2(div_l(__uint_as_float(v[8 * i + 4])), div_l(__uint_as_float(v[8 * i + 5])));
                    o4.w = pack_bf16x2(div_l(__uint_as_float(v[8 * i + 6])), div_l(__uint_as_float(v[8 * i + 7])));
                    // row r, 16-byte chunk c*4+i, stored at chunk slot (chunk ^ (r & 7)): conflict-free
                    *reinterpret_cast<uint4*>(stage + r * kRowBytes + (((c * 4 + i) ^ (r & 7)) << 4)) = o4;
                }
            }
            bar_sync(1 + j, 128);
            int64_t tile_off = z * a.osb + h * a.osh + (int64_t)qb * kTile * a.osn;
            // token-sharded destination: the whole tile belongs to one rank (rows_per_peer is a
            // multiple of the tile height), whose buffer starts at that rank's first row
            const int owner = ta.rows_per_peer > 0 ? (qb * kTile) / ta.rows_per_peer : 0;
            if (ta.rows_per_peer > 0) tile_off -= (int64_t)owner * ta.rows_per_peer * a.osn;
            const int ch = r & 15;
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
                const int row = it * 8 + (r >> 4);
                const uint4 val = *reinterpret_cast<const uint4*>(stage + row * kRowBytes + ((ch ^ (row & 7)) << 4));
                const int64_t off = tile_off + (int64_t)row * a.osn + ch * 8;
                if (MODE == kBlock && qb * kTile + row >= ta.q_rows) continue;      // padding rows of the dense variant
                if (ta.n_peers == 0) {
                    *reinterpret_cast<uint4*>(a.out + off) = val;
                } else if (ta.rows_per_peer > 0) {
                    *reinterpret_cast<uint4*>(ta.peers[owner] + off) = val;
                } else {
                    // head-parallel runs: the rows go straight into every rank's copy of the
                    // assembled output (16-byte stores, a row per 16 threads, over NVLink);
                    // no collective follows
                    for (int pr = 0; pr < ta.n_peers; ++pr) *reinterpret_cast<uint4*>(ta.peers[pr] + off) = val;
                }
            }
        }
    }
}

// Which (batch, head, pair of query tiles) CTA `bid` works on.  CTAs that run at the same time
// share one KV head: its K and V (2 x 256 B x N) stay in L2 while the query heads of the group
// and their query-tile pairs (heaviest first) walk them.
struct WorkItem {
    int pair, z, h, kvh, hz;
};
__device__ __forceinline__ WorkItem work_item(const AttendArgs& a, int bid) {
    const int npairs = a.N / (2 * kTile);
    const int Hg = a.H / a.Hkv;
    const int per_kv = Hg * npairs;
    const int kvz = bid / per_kv, rem = bid % per_kv;
    WorkItem w;
    w.pair = npairs - 1 - rem / Hg;
    w.z = kvz / a.Hkv;
    w.kvh = kvz % a.Hkv;
    w.h = w.kvh * Hg + rem % Hg;
    w.hz = w.z * a.H + w.h;
    return w;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
attend_tc_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                 const __grid_constant__ CUtensorMap kgmap, const __grid_constant__ CUtensorMap vgmap, TcArgs ta) {
    extern __shared__ uint8_t smem_raw[];
    const AttendArgs& a = ta.a;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const uint32_t raw_u = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_u & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t s_u = raw_u + pad;
    const uint32_t ring_u = s_u + kSmemQ;
    const uint32_t bars = ring_u + kSmemRing;
    auto kv_full = [&](int i) { return bars + 8u * i; };
    auto kv_empty = [&](int i) { return bars + 40u + 8u * i; };
    auto q_full = [&](int j) { return bars + 80u + 8u * j; };
    auto s_full = [&](int j) { return bars + 96u + 8u * j; };
    auto o_done = [&](int j) { return bars + 112u + 8u * j; };
    auto p_part = [&](int j, int q) { return bars + 128u + 8u * (4 * j + q); };
    const uint32_t tmem_slot_u = bars + 192u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kSmemQ + kSmemRing + 192);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kSmemQ + kSmemRing + 196);

    // ---- which work item ----
    const int npairs = a.N / (2 * kTile);
    const WorkItem wi = work_item(a, (int)blockIdx.x);
    const int pair = wi.pair, z = wi.z, kvh = wi.kvh, h = wi.h, hz = wi.hz;
    const int G = a.block * a.step;
    const int b = (pair * 2 * kTile) / G;
    const int NB = a.N / G;

    int ntiles, n_init = 0, local_start = 0, count = 0, dense_last0 = 0;
    const int32_t* idp = nullptr;
    const int32_t* slotp = nullptr;      // step 3: gather slots of this list's tiles
    if (MODE == kWindow) {
        const int end = (2 * pair + 2) * kTile;
        const int init_end = min(G, end);
        local_start = max(b * G, init_end);
        n_init = init_end / kTile;
        ntiles = n_init + (end - local_start) / kTile;
    } else if (MODE == kBlock && ta.dense) {
        // key blocks 0 .. the one that holds the last position a row of the tile may attend
        dense_last0 = min((ta.q_off + (2 * pair) * kTile + kTile - 1) / kTile, ta.kv_blocks - 1);
        ntiles = min((ta.q_off + (2 * pair + 1) * kTile + kTile - 1) / kTile, ta.kv_blocks - 1) + 1;
    } else if (MODE == kBlock) {
        count = a.counts[(int64_t)hz * npairs + pair];          // entries of the pair's merged tile list
        ntiles = count;
        idp = a.ids + (int64_t)hz * a.ids_per_head + (int64_t)pair * ta.list_stride;
    } else {
        // never beyond the capacity of the big block's list, whatever the workspace holds
        count = min(max(a.counts[(int64_t)hz * NB + b], 0), max(b * G - 2 * a.block, 0));
        ntiles = (count + kTile - 1) / kTile;
        const int64_t row_off = (b == 0) ? 0 : ((int64_t)G * b * (b - 1) / 2 - 2 * (int64_t)a.block * (b - 1));
        idp = a.ids + (int64_t)hz * a.ids_per_head + row_off;
        if (ta.tile_slot) slotp = ta.tile_slot + (int64_t)hz * (a.ids_per_head / kTile) + row_off / kTile;
    }

    if (MODE == kStripe && ntiles == 0) {
        // Nothing selected for these rows (always so in the first big block): the output is step 1's
        // state normalised, acc / l, with the arithmetic of the epilogue.  No tensor memory, no
        // barriers.  A warp takes 32 rows x 32 columns at a time: lane r reads the eight 16-byte
        // chunks of its row (512 contiguous bytes per instruction in the tile layout), divides,
        // and the warp turns its 32 x 64 bytes of bf16 through shared memory so that the rows go
        // out as 64-byte pieces from four consecutive lanes.
        constexpr int kWarps = kThreads / 32;
        uint8_t* wbuf = smem + warp * 2048;
        for (int u = warp; u < 32; u += kWarps) {
            const int row = (u >> 2) * 32 + lane, quarter = u & 3;          // row inside the pair's 256 rows
            const int64_t srow = (int64_t)hz * a.N + pair * 2 * kTile + row;
            const float* tile_acc = acc_tile(a.Acc, hz, a.N, 2 * pair + (row >> 7));
            const float li = a.L[srow];
            float4 x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                x[i] = *reinterpret_cast<const float4*>(tile_acc + acc_chunk_off(quarter * 8 + i, row & 127));
            const float rl = __frcp_rn(li);
            auto div_l = [&](float v) {
                const float q0 = __fmul_rn(v, rl);
                const float rem = __fmaf_rn(-q0, li, v);
                return __fmaf_rn(rem, rl, q0);
            };
            __syncwarp();                                                   // the previous unit's rows have been read
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 o4;
                o4.x = pack_bf16x2(div_l(x[2 * i].x), div_l(x[2 * i].y));
                o4.y = pack_bf16x2(div_l(x[2 * i].z), div_l(x[2 * i].w));
                o4.z = pack_bf16x2(div_l(x[2 * i + 1].x), div_l(x[2 * i + 1].y));
                o4.w = pack_bf16x2(div_l(x[2 * i + 1].z), div_l(x[2 * i + 1].w));
                *reinterpret_cast<uint4*>(wbuf + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4)) = o4;
            }
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int rr = it * 8 + (lane >> 2), cc = lane & 3;
                const uint4 val = *reinterpret_cast<const uint4*>(wbuf + rr * 64 + ((cc ^ ((rr >> 1) & 3)) << 4));
                const int grow = pair * 2 * kTile + (u >> 2) * 32 + rr;      // row inside the head
                int64_t off = z * a.osb + h * a.osh + (int64_t)grow * a.osn + quarter * 32 + cc * 8;
                if (ta.n_peers == 0) {
                    *reinterpret_cast<uint4*>(a.out + off) = val;
                } else if (ta.rows_per_peer > 0) {
                    const int owner = grow / ta.rows_per_peer;
                    off -= (int64_t)owner * ta.rows_per_peer * a.osn;
                    *reinterpret_cast<uint4*>(ta.peers[owner] + off) = val;
                } else {
                    for (int pr = 0; pr < ta.n_peers; ++pr) *reinterpret_cast<uint4*>(ta.peers[pr] + off) = val;
                }
            }
        }
        return;
    }

    // ---- set-up ----
    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(kv_full(i), 32 * kLoaderWarps);
            mbar_init(kv_empty(i), 1);
        }
        for (int j = 0; j < 2; ++j) {
            mbar_init(q_full(j), 128);
            mbar_init(s_full(j), 1);
            for (int q = 0; q < kPParts; ++q) mbar_init(p_part(j, q), 4);       // one arrival per softmax warp
            mbar_init(o_done(j), 1);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot_u, kTmemCols);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // =================================================== softmax warps
        setmaxnreg_inc<kSoftmaxRegs>();
        SoftmaxCtx sc;
        sc.smem = smem;
        sc.tmem_base = tmem_base;
        sc.abort_flag = abort_flag;
        for (int jj = 0; jj < 2; ++jj) {
            sc.q_full[jj] = q_full(jj);
            sc.s_full[jj] = s_full(jj);
            for (int q = 0; q < 4; ++q) sc.p_part[jj][q] = p_part(jj, q);
            sc.o_done[jj] = o_done(jj);
        }
        sc.pair = pair; sc.z = z; sc.h = h; sc.hz = hz;
        sc.ntiles = ntiles; sc.n_init = n_init; sc.local_start = local_start; sc.count = count;
        sc.list = idp;
        sc.dense_last0 = dense_last0;
        softmax_role<MODE>(ta, sc, tid);
    } else {
        setmaxnreg_dec<kOtherRegs>();
        if (warp == 8 && ntiles > 0) {
            const bool issuer = elect_one();
            // =================================================== MMA issuer
            constexpr uint32_t kIdescQK = idesc_bf16_128x128(0);
            constexpr uint32_t kIdescPV = idesc_bf16_128x128(1);
            // descriptors: high word constant (8-row group stride 1024 B, version 1, 128B swizzle);
            // low word = start address / 16 | leading offset / 16 << 16; advancing inside a
            // tile only adds to the start-address field
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            auto desc = [&](uint32_t lo) { return ((uint64_t)kDescHi << 32) | lo; };
            auto lo_kmajor = [&](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1u << 16); };
            auto lo_mnmajor = [&](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | ((uint32_t)(kSlabBytes >> 4) << 16); };
            const uint32_t q_lo[2] = {lo_kmajor(s_u), lo_kmajor(s_u + (uint32_t)kTileBytes)};
            auto slot_addr = [&](int n) { return ring_u + (uint32_t)(n % kStages) * kTileBytes; };
            auto issue_qk = [&](int j, uint32_t kaddr) {
                const uint32_t k_lo = lo_kmajor(kaddr);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (uint32_t)(((ks >> 2) * kSlabBytes + (ks & 3) * 32) >> 4);
                    if (issuer)
                        mma_ss(tmem_base + (uint32_t)j * 128u, desc(q_lo[j] + off), desc(k_lo + off), kIdescQK, ks > 0);
                }
            };
            auto issue_pv = [&](int j, uint32_t vaddr, bool acc, int ks0) {
                const uint32_t v_lo = lo_mnmajor(vaddr);
#pragma unroll
                for (int ks = ks0; ks < ks0 + 8 / kPParts; ++ks)
                    if (issuer)
                        mma_ts(tmem_base + 256u + (uint32_t)j * 128u, tmem_base + (uint32_t)j * 128u + (uint32_t)ks * 8u,
                               desc(v_lo + (uint32_t)ks * (2048u >> 4)), kIdescPV, (ks > 0) || acc);
            };
            auto wait_all = [&](uint32_t bar, uint32_t parity) {
                return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
            };
            // kBlock: an entry of the tile list names the query tiles that attend the block; the
            // other tile gets no Q K^T and no P V for it, and its barriers count its own tiles only.
            // The list entries are read two tiles ahead.
            uint32_t e_cur = 0xC0000000u, e_next = 0xC0000000u;
            if (MODE == kBlock) {
                e_cur = block_entry(ta, idp, 0, dense_last0);
                e_next = ntiles > 1 ? block_entry(ta, idp, 1, dense_last0) : 0u;
            }
            auto attends = [&](uint32_t e, int j) { return MODE != kBlock || ((e >> (kBlockFlagShift + j)) & 1u) != 0u; };
            int done[2] = {0, 0};          // P V products issued per query tile
            bool ok = wait_all(q_full(0), 0) && wait_all(q_full(1), 0) && wait_all(kv_full(0), 0);
            if (ok) {
                fence_proxy_async();
                tcgen05_fence_after();
                if (attends(e_cur, 0)) {
                    issue_qk(0, slot_addr(0));
                    commit_if(issuer, s_full(0));
                }
                if (attends(e_cur, 1)) {
                    issue_qk(1, slot_addr(0));
                    commit_if(issuer, s_full(1));
                }
                commit_if(issuer, kv_empty(0));
            }
            for (int t = 0; t < ntiles && ok; ++t) {
                const int nv = 2 * t + 1, nk = 2 * t + 2;
                uint32_t e_after = 0u;
                if (MODE == kBlock && t + 2 < ntiles) e_after = block_entry(ta, idp, t + 2, dense_last0);
                ok = wait_all(kv_full(nv % kStages), (nv / kStages) & 1);
                if (!ok) break;
                fence_proxy_async();
                for (int j = 0; j < 2 && ok; ++j) {
                    if (attends(e_cur, j)) {
                        const int seq = (MODE == kBlock) ? done[j] : t;
                        for (int q = 0; q < kPParts && ok; ++q) {
                            ok = wait_all(p_part(j, q), seq & 1);
                            if (!ok) break;
                            tcgen05_fence_after();
                            issue_pv(j, slot_addr(nv), (seq > 0) || (MODE == kStripe) || q > 0, q * (8 / kPParts));
                        }
                        if (!ok) break;
                        ++done[j];
                    }
                    if (j == 1) commit_if(issuer, kv_empty(nv % kStages));
                    if (t + 1 < ntiles) {
                        if (j == 0) {
                            ok = wait_all(kv_full(nk % kStages), (nk / kStages) & 1);
                            if (!ok) break;
                            fence_proxy_async();
                            tcgen05_fence_after();
                        }
                        if (attends(e_next, j)) {
                            issue_qk(j, slot_addr(nk));
                            commit_if(issuer, s_full(j));
                        }
                        if (j == 1) commit_if(issuer, kv_empty(nk % kStages));
                    } else {
                        commit_if(issuer, o_done(j));
                    }
                }
                e_cur = e_next;
                e_next = e_after;
            }
        } else if (warp >= 9 && ntiles > 0) {
            // =================================================== loaders (three warps)
            const int lw = warp - 9;
            const __nv_bfloat16* kbase = a.k.ptr + z * a.k.sb + kvh * a.k.sh;
            const __nv_bfloat16* vbase = a.v.ptr + z * a.v.sb + kvh * a.v.sh;
            // row-gather maps see the tensor as rows of `sn` elements: this head's rows start at
            // row (offset / sn), column (offset % sn)
            const int64_t koff = z * a.k.sb + kvh * a.k.sh, voff = z * a.v.sb + kvh * a.v.sh;
            const int k_row0 = (int)(koff / a.k.sn), k_col0 = (int)(koff % a.k.sn);
            const int v_row0 = (int)(voff / a.v.sn), v_col0 = (int)(voff % a.v.sn);
            bool ok = true;
            int row0 = 0, gslot = -1;
            bool run = true;         // 128 consecutive rows -> one TMA tile
            for (int n = 0; n < 2 * ntiles && ok; ++n) {
                const int slot = n % kStages, it = n / kStages;
                const int t = n >> 1;
                const bool is_v = n & 1;
                // where the tile comes from is decided once, for its K half (before the wait for a
                // free slot, so that the loads of the list entries overlap it)
                if (!is_v) {
                    if (MODE == kWindow) {
                        row0 = (t < n_init) ? t * kTile : local_start + (t - n_init) * kTile;
                    } else if (MODE == kBlock) {
                        row0 = (int)(block_entry(ta, idp, t, dense_last0) & kBlockIdMask) * kTile;
                    } else {
                        const int s0 = t * kTile;
                        run = false;
                        gslot = slotp ? slotp[t] : -1;     // only meaningful when the tile is not a run
                        if (gslot >= ta.n_slots) gslot = -1;
                        if (s0 + kTile <= count) {
                            row0 = idp[s0];
                            run = (idp[s0 + kTile - 1] - row0) == kTile - 1;
                        }
                    }
                }
                if (it > 0) {
                    ok = mbar_wait(kv_empty(slot), (it - 1) & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                const uint32_t dst = ring_u + (uint32_t)slot * kTileBytes;
                if (run || gslot >= 0) {
                    // a run of 128 rows of K / V itself (two box loads), or the tile's image in the
                    // gather scratch (one bulk copy)
                    if (lw == 0 && lane == 0) {
                        mbar_arrive_expect_tx(kv_full(slot), kTileBytes);
                        if (!run)
                            bulk_load(dst, ta.gather + (int64_t)gslot * (2 * kTileBytes) + (is_v ? kTileBytes : 0),
                                      kTileBytes, kv_full(slot));
                        else if (is_v)
                            tma_tile(dst, &vmap, kv_full(slot), ta.vpos_n, ta.vpos_h, ta.vpos_b, row0, kvh, z);
                        else
                            tma_tile(dst, &kmap, kv_full(slot), ta.kpos_n, ta.kpos_h, ta.kpos_b, row0, kvh, z);
                    } else {
                        mbar_arrive(kv_full(slot));
                    }
                    continue;
                }
                // Discrete rows.  The TMA unit and the load/store unit each sustain only about one
                // 128-byte row segment per 17-24 cycles on gathers, so the tile is split between
                // them: rows [0, tma_rows) by TMA row gathers from the first loader warp
                // (tile::gather4, lane i takes rows 4i .. 4i+3, two 64-column halves each), the rest
                // by 16-byte cp.async copies from the other loader warps (a warp sustains only a few
                // copies in flight, so the rate grows with the warp count).  Without a usable 2-D
                // map all loader warps copy.
                // Slots past the count read row 0 / zero-fill; the softmax masks them.
                const bool g4 = MODE == kStripe && (is_v ? ta.v_gather : ta.k_gather);
                const int tma_rows = g4 ? kTmaRows : 0;
                // this warp's cp.async rows [ra, rb): the non-TMA rows in even-sized shares
                int ra, rb;
                {
                    const int first = g4 ? 1 : 0, nw = kLoaderWarps - first;
                    const int pairs = (kTile - tma_rows) / 2;              // two rows per copy instruction
                    const int w = lw - first;
                    ra = tma_rows + 2 * ((pairs * w) / nw);
                    rb = tma_rows + 2 * ((pairs * (w + 1)) / nw);
                    if (w < 0) ra = rb = 0;
                }
                if (g4 && lw == 0) {
                    if (lane == 0)
                        mbar_arrive_expect_tx(kv_full(slot), (uint32_t)tma_rows * kRowBytes);
                    else
                        mbar_arrive(kv_full(slot));
                    if (4 * lane < tma_rows) {
                        const int s0 = t * kTile + 4 * lane;
                        int4 id4 = make_int4(0, 0, 0, 0);
                        if (s0 + 4 <= count) {
                            id4 = *reinterpret_cast<const int4*>(idp + s0);
                        } else {
                            if (s0 < count) id4.x = idp[s0];
                            if (s0 + 1 < count) id4.y = idp[s0 + 1];
                            if (s0 + 2 < count) id4.z = idp[s0 + 2];
                        }
                        // ids are addresses from here on: keep them inside the tensor
                        id4.x = min(max(id4.x, 0), a.N - 1);
                        id4.y = min(max(id4.y, 0), a.N - 1);
                        id4.z = min(max(id4.z, 0), a.N - 1);
                        id4.w = min(max(id4.w, 0), a.N - 1);
                        const CUtensorMap* gm = is_v ? &vgmap : &kgmap;
                        const int r0 = is_v ? v_row0 : k_row0, c0 = is_v ? v_col0 : k_col0;
                        const uint32_t d = dst + (uint32_t)lane * 512u;
                        tma_gather4(d, gm, kv_full(slot), c0, r0 + id4.x, r0 + id4.y, r0 + id4.z, r0 + id4.w);
                        tma_gather4(d + kSlabBytes, gm, kv_full(slot), c0 + 64, r0 + id4.x, r0 + id4.y, r0 + id4.z,
                                    r0 + id4.w);
                    }
                } else {
                    const __nv_bfloat16* base = is_v ? vbase : kbase;
                    const int64_t sn = is_v ? a.v.sn : a.k.sn;
                    const int s0 = t * kTile + ra;
                    // this warp's ids (at most 64): two coalesced loads, handed round by shuffle
                    const int id_lo = (ra + lane < rb && s0 + lane < count) ? idp[s0 + lane] : -1;
                    const int id_hi = (ra + 32 + lane < rb && s0 + 32 + lane < count) ? idp[s0 + 32 + lane] : -1;
                    const int ch = lane & 15;
                    const int npairs_rows = (rb - ra) >> 1;
#pragma unroll 4
                    for (int i = 0; i < npairs_rows; ++i) {
                        const int rel = 2 * i + (lane >> 4);
                        const int v0 = __shfl_sync(0xffffffffu, id_lo, rel & 31);
                        const int v1 = __shfl_sync(0xffffffffu, id_hi, rel & 31);
                        const int row = rel < 32 ? v0 : v1;
                        const bool valid = row >= 0;
                        cp_async16(dst + sw_off(ra + rel, ch), base + (int64_t)(valid ? min(row, a.N - 1) : 0) * sn + ch * 8,
                                   valid ? 16 : 0);
                    }
                    cp_async_mbar_arrive_noinc(kv_full(slot));
                }
            }
            cp_async_wait<0>();
        }
    }

    // ---- teardown ----
    tcgen05_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicMax(ta.status, 1);
    if (warp == 8) tmem_dealloc(tmem_base, kTmemCols);
}

// Self-test of the bounded-wait path: one warp waits on a barrier that nothing ever arrives
// on; the wait gives up after its poll limit, raises the abort flag and the status word is
// set exactly as the attention kernels set it.  Nothing faults, the context stays usable.
__global__ void __launch_bounds__(32, 1) wait_timeout_selftest_kernel(int32_t* status) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;
    const uint32_t bar_u = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(bar_u, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncwarp();
    const bool ok = mbar_wait(bar_u, 0, abort_flag);
    __syncwarp();
    if (threadIdx.x == 0 && (!ok || *abort_flag)) atomicMax(status, 1);
}

}  // namespace tc
}  // namespace aa

// Attention on the Blackwell tensor cores (tcgen05 + tensor memory + TMA): what the three passes
// share, and the block-granular pass.  Steps 1 and 3 of the operator run the same tile loop as
// persistent CTAs (attend_persist.cuh).
//
// One CTA owns 256 query rows of one head (two 128-row tiles A and B that share their key/value
// tiles) and walks a list of 128-row key/value tiles.  The pass here:
//
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
//   warps 9-11  loaders, into a 5-slot ring of 32 KB tiles: one TMA box load per 128-row block
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
    int pair, z, h, ntiles;
    const int32_t* list;             // the pair's tile list
    int dense_last0;                 // dense variant: last key block of the pair's first query tile
};

// The softmax role of warps 0-7 (see the file header): thread r of tile j owns query row r.
__device__ __forceinline__ void softmax_role(const TcArgs& ta, const SoftmaxCtx& cx, int tid) {
    const AttendArgs& a = ta.a;
    const int warp = tid >> 5;
    uint8_t* smem = cx.smem;
    const uint32_t tmem_base = cx.tmem_base;
    volatile int* abort_flag = cx.abort_flag;
    const int pair = cx.pair, z = cx.z, h = cx.h;
    const int ntiles = cx.ntiles;
    const int j = warp >> 2;
    const uint32_t q_full_j = cx.q_full[j], s_full_j = cx.s_full[j], o_done_j = cx.o_done[j];
    uint32_t p_part_j[kPParts];
#pragma unroll
    for (int q = 0; q < kPParts; ++q) p_part_j[q] = cx.p_part[j][q];
    const int r = tid & 127;
    const int qb = 2 * pair + j;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + (uint32_t)j * 128u;
    const uint32_t tO = tmem_base + lane_base + 256u + (uint32_t)j * 128u;

    // Q tile: load, scale, round, store in the K-major 128B-swizzled layout the MMA reads
    // (not needed when there is no key tile to multiply it with)
    if (ntiles > 0) {
        const __nv_bfloat16* qbase = a.q.ptr + z * a.q.sb + h * a.q.sh + (int64_t)qb * kTile * a.q.sn;
        uint8_t* qs = smem + j * kTileBytes;
        // all sixteen loads of the thread are issued before the first one is used
        uint4 raws[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int id = r + 128 * i;
            if (qb * kTile + (id >> 4) >= ta.q_rows)
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
                // bf16(q * (sm_scale * log2e)): the constants are multiplied first
                const float qk = __fmul_rn(a.sm_scale, kLog2e);
                float2 f = __bfloat1622float2(p2[e]);
                p2[e] = __floats2bfloat162_rn(__fmul_rn(f.x, qk), __fmul_rn(f.y, qk));
            }
            *reinterpret_cast<uint4*>(qs + sw_off(rr, ch)) = raw;
        }
        fence_proxy_async();
        mbar_arrive(q_full_j);
    }

    float m_true = -INFINITY, m_ref = -INFINITY, l = 0.f;

    auto signal = [&](uint32_t bar) {
        tmem_wait_st();
        tcgen05_fence_before();
        // one arrival per warp: 128 arrivals on one barrier would queue up behind each other
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar);
    };
    uint32_t entry_next = ntiles > 0 ? block_entry(ta, cx.list, 0, cx.dense_last0) : 0u;
    int mine = 0;        // tiles of this query tile so far (the MMA warp counts the same way)
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
        const uint32_t entry = entry_next;
        if (t + 1 < ntiles) entry_next = block_entry(ta, cx.list, t + 1, cx.dense_last0);
        // a block of the other query tile only: no S is produced for this one, nothing to do
        if (!((entry >> (kBlockFlagShift + j)) & 1u)) continue;
        const int seq = mine;                             // which of this tile's score tiles
        ++mine;
        ok = mbar_wait(s_full_j, seq & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        uint32_t sv[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sv[c]);
        tmem_wait_ld();

        {
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
            if (seq != 0) {                           // nothing accumulated yet on the first tile
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
    {
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
            if (ntiles == 0) l = 1.f;                            // an empty list: zeros (the lists are never empty)
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
                } else {                 // an empty list
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
            const int64_t tile_off = z * a.osb + h * a.osh + (int64_t)qb * kTile * a.osn;
            const int ch = r & 15;
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
                const int row = it * 8 + (r >> 4);
                const uint4 val = *reinterpret_cast<const uint4*>(stage + row * kRowBytes + ((ch ^ (row & 7)) << 4));
                const int64_t off = tile_off + (int64_t)row * a.osn + ch * 8;
                if (qb * kTile + row >= ta.q_rows) continue;      // padding rows of the dense variant
                *reinterpret_cast<uint4*>(a.out + off) = val;
            }
        }
    }
}

// Which (batch, head, pair of query tiles) work item `bid` is.  CTAs that run at the same time
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

__global__ void __launch_bounds__(kThreads, 1)
attend_block_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, TcArgs ta) {
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

    int ntiles, dense_last0 = 0;
    const int32_t* idp = nullptr;
    if (ta.dense) {
        // key blocks 0 .. the one that holds the last position a row of the tile may attend
        dense_last0 = min((ta.q_off + (2 * pair) * kTile + kTile - 1) / kTile, ta.kv_blocks - 1);
        ntiles = min((ta.q_off + (2 * pair + 1) * kTile + kTile - 1) / kTile, ta.kv_blocks - 1) + 1;
    } else {
        ntiles = a.counts[(int64_t)hz * npairs + pair];          // entries of the pair's merged tile list
        idp = a.ids + (int64_t)hz * a.ids_per_head + (int64_t)pair * ta.list_stride;
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
        sc.pair = pair; sc.z = z; sc.h = h;
        sc.ntiles = ntiles;
        sc.list = idp;
        sc.dense_last0 = dense_last0;
        softmax_role(ta, sc, tid);
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
            // An entry of the tile list names the query tiles that attend the block; the other tile
            // gets no Q K^T and no P V for it, and its barriers count its own tiles only.  The list
            // entries are read two tiles ahead.
            uint32_t e_cur = block_entry(ta, idp, 0, dense_last0);
            uint32_t e_next = ntiles > 1 ? block_entry(ta, idp, 1, dense_last0) : 0u;
            auto attends = [&](uint32_t e, int j) { return ((e >> (kBlockFlagShift + j)) & 1u) != 0u; };
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
                if (t + 2 < ntiles) e_after = block_entry(ta, idp, t + 2, dense_last0);
                ok = wait_all(kv_full(nv % kStages), (nv / kStages) & 1);
                if (!ok) break;
                fence_proxy_async();
                for (int j = 0; j < 2 && ok; ++j) {
                    if (attends(e_cur, j)) {
                        const int seq = done[j];
                        for (int q = 0; q < kPParts && ok; ++q) {
                            ok = wait_all(p_part(j, q), seq & 1);
                            if (!ok) break;
                            tcgen05_fence_after();
                            issue_pv(j, slot_addr(nv), (seq > 0) || q > 0, q * (8 / kPParts));
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
            // every tile is a whole 128-row block of K or V: one TMA box load (two slabs) from one
            // lane; the other lanes only arrive
            const int lw = warp - 9;
            bool ok = true;
            int row0 = 0;
            for (int n = 0; n < 2 * ntiles && ok; ++n) {
                const int slot = n % kStages, it = n / kStages;
                const bool is_v = n & 1;
                if (!is_v) row0 = (int)(block_entry(ta, idp, n >> 1, dense_last0) & kBlockIdMask) * kTile;
                if (it > 0) {
                    ok = mbar_wait(kv_empty(slot), (it - 1) & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                const uint32_t dst = ring_u + (uint32_t)slot * kTileBytes;
                if (lw == 0 && lane == 0) {
                    mbar_arrive_expect_tx(kv_full(slot), kTileBytes);
                    if (is_v)
                        tma_tile(dst, &vmap, kv_full(slot), ta.vpos_n, ta.vpos_h, ta.vpos_b, row0, kvh, z);
                    else
                        tma_tile(dst, &kmap, kv_full(slot), ta.kpos_n, ta.kpos_h, ta.kpos_b, row0, kvh, z);
                } else {
                    mbar_arrive(kv_full(slot));
                }
            }
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

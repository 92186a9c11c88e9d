// Steps 1 and 3 of the operator on the Blackwell tensor cores, as PERSISTENT CTAs: one CTA per SM
// walks work items of 256 query rows of one head (two 128-row tiles A and B that lie in the same
// big block and therefore share their key/value tiles), heaviest first, and for each item a list
// of 128-row key/value tiles:
//
//   kWindow  (step 1)  contiguous tiles of [0, min(G, end)) U [max(b*G, that), end),
//            end = last query row + 1; additive -1e6 causal mask on diagonal tiles;
//            query scaled with dtype-rounded constants; writes M, L, Acc (Acc in 128-row
//            chunk-major tiles, see acc_tile()).
//            Reference: anchor_attn/src/ops/anchor_step_1_2_v2.py:8-161.
//   kStripe  (step 3)  tiles of 128 ids from the big block's id list; state starts
//            from step 1's (M, L, Acc); slots past the count masked to -inf;
//            writes bf16(acc / l).  Reference: anchor_attn/src/ops/anchor_attn_v4.py:7-105.
//
// Warp roles, tensor-memory layout and the lazily moved exponent reference are those of
// attend_tc.cuh.  The loaders (warps 9-11) fill the 5-slot ring of 32 KB tiles with: one TMA box
// load for a run of 128 consecutive rows; one bulk copy for a tile the gather pass (gather.cuh)
// put into scratch; discrete rows without a scratch slot split between TMA row gathers
// (tile::gather4, four rows per instruction, warp 9) and 16-byte cp.async copies (warps 10-11; all
// three warps for stride patterns no 2-D tensor map covers).
//
// Why persistent: a kernel that allocates tensor memory gets one resident CTA per SM, so with one
// CTA per item nothing overlaps an item's start-up (launch, barrier and tensor-memory set-up, the
// query tile and, in step 3, the 128 KB of step-1 state arriving from DRAM) or its tail (the
// output leaving).  With short key lists -- step 1 always, step 3 at low density -- those two
// are a large part of an item.  Here
//   * tensor memory, barriers and register re-allocation are set up once per SM;
//   * an item's query tiles and (step 3) its accumulator tiles are fetched by the loader warps
//     through the same ring as the key/value tiles, as asynchronous bulk copies that run
//     while the previous item is still being computed and written out;
//   * items are handed out by an atomic counter, each shortly before the previous one ends, through
//     a two-entry queue in shared memory, so that items start in order on whichever SM is free, as
//     CTAs of a grid would.
//
// Ring entries of one item, in order (each 32 KB):
//   step 1:                Q_A Q_B                      K_0 V_0 K_1 V_1 ...
//   step 3, list not empty: Q_A Q_B AccA_lo AccA_hi AccB_lo AccB_hi   K_0 V_0 K_1 V_1 ...
//   step 3, empty list:             AccA_lo AccA_hi AccB_lo AccB_hi
// (Putting K_0 among the first five entries, so that it is on its way before any entry has to be
// released, measured slower on most lists: V_0 then waits for K_0's slot.)
// Q_x is the raw query tile (a TMA box load, 128-byte swizzle): the tile's softmax warps scale and
// round it into the CTA's query buffer, at the same offsets.  Acc?_lo / _hi are the two halves of
// an accumulator tile in its chunk-major layout (acc_tile()): thread r reads the 16-byte chunk k
// of its row at k * 2048 + 16 r, conflict-free.  Entries consumed by softmax warps are released
// by them (one arrival after a named barrier over the tile's 128 threads); K/V entries by the MMA
// warp's tcgen05.commit.
//
// Barrier phases run on across items: ring entries by a running entry number, score and
// probability barriers by a running tile number, per-item barriers by the number of items with
// tiles.  Every wait is bounded; a warp whose wait gave up still walks to the next named
// barrier of its tile, which is where the tile's four warps agree to stop.
#pragma once
#include "attend_tc.cuh"

namespace aa {
namespace tc {

struct PersistArgs {
    int qpos_n, qpos_h, qpos_b;      // query tensor map: which coordinate carries n / head / batch
    int32_t* item_counter;           // before the launch: the first item the launch is to take (0 when it takes all)
    int n_items;                     // one past the last item the launch is to take
};

// what every role needs to know about one item
struct Item {
    int pair, z, h, kvh, hz, b;
    int ntiles, n_init, local_start, count;
    const int32_t* idp;
    const int32_t* slotp;
};

template <int MODE>
__device__ __forceinline__ int item_count(const TcArgs& ta, int bid) {
    if (MODE != kStripe) return 0;
    const AttendArgs& a = ta.a;
    const WorkItem w = work_item(a, bid);
    const int G = a.block * a.step, NB = a.N / G;
    const int b = (w.pair * 2 * kTile) / G;
    return min(max(a.counts[(int64_t)w.hz * NB + b], 0), max(b * G - 2 * a.block, 0));
}

template <int MODE>
__device__ __forceinline__ Item make_item(const TcArgs& ta, int bid, int count) {
    const AttendArgs& a = ta.a;
    const WorkItem w = work_item(a, bid);
    Item it;
    it.pair = w.pair; it.z = w.z; it.h = w.h; it.kvh = w.kvh; it.hz = w.hz;
    const int G = a.block * a.step;
    it.b = (w.pair * 2 * kTile) / G;
    it.n_init = 0; it.local_start = 0; it.count = count;
    it.idp = nullptr; it.slotp = nullptr;
    if (MODE == kWindow) {
        const int end = (2 * w.pair + 2) * kTile;
        const int init_end = min(G, end);
        it.local_start = max(it.b * G, init_end);
        it.n_init = init_end / kTile;
        it.ntiles = it.n_init + (end - it.local_start) / kTile;
    } else {
        it.ntiles = (count + kTile - 1) / kTile;
        const int b = it.b;
        const int64_t row_off = (b == 0) ? 0 : ((int64_t)G * b * (b - 1) / 2 - 2 * (int64_t)a.block * (b - 1));
        it.idp = a.ids + (int64_t)w.hz * a.ids_per_head + row_off;
        if (ta.tile_slot) it.slotp = ta.tile_slot + (int64_t)w.hz * (a.ids_per_head / kTile) + row_off / kTile;
    }
    return it;
}

// ring entries before the first key tile of an item
template <int MODE>
__device__ __forceinline__ int header_entries(int ntiles) {
    if (MODE == kWindow) return 2;
    return ntiles > 0 ? 6 : 4;
}

// ring entry, counted from the item's first, of key tile t / value tile t / the first accumulator half
template <int MODE>
__device__ __forceinline__ int k_entry(int t) { return (MODE == kWindow ? 2 : 6) + 2 * t; }
template <int MODE>
__device__ __forceinline__ int v_entry(int t) { return (MODE == kWindow ? 3 : 7) + 2 * t; }
__device__ __forceinline__ int acc_entry(int ntiles) { return ntiles > 0 ? 2 : 0; }

struct PersistBars {
    uint32_t bars;
    __device__ __forceinline__ uint32_t kv_full(int i) const { return bars + 8u * i; }
    __device__ __forceinline__ uint32_t kv_empty(int i) const { return bars + 40u + 8u * i; }
    __device__ __forceinline__ uint32_t q_full(int j) const { return bars + 80u + 8u * j; }
    __device__ __forceinline__ uint32_t s_full(int j) const { return bars + 96u + 8u * j; }
    __device__ __forceinline__ uint32_t o_done(int j) const { return bars + 112u + 8u * j; }
    __device__ __forceinline__ uint32_t p_part(int j, int q) const { return bars + 128u + 8u * (4 * j + q); }
    __device__ __forceinline__ uint32_t item_full(int k) const { return bars + 200u + 8u * k; }
    __device__ __forceinline__ uint32_t item_empty(int k) const { return bars + 216u + 8u * k; }
};
constexpr int kQueueOff = 232;               // four ints: {item, count} x 2, behind the barriers
constexpr int kItemConsumers = 11;           // warps that read the queue: 8 softmax, the MMA warp, loader warps 10 and 11

// A consumer warp takes item number k (0, 1, ...) from the queue.  False: a wait gave up.
__device__ __forceinline__ bool take_item(const PersistBars& B, volatile int* queue, volatile int* abort_flag, int k,
                                          int lane, int& bid, int& count) {
    bool ok = mbar_wait(B.item_full(k & 1), (k >> 1) & 1, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return false;
    bid = queue[2 * (k & 1)];
    count = queue[2 * (k & 1) + 1];
    __syncwarp();
    if (lane == 0) mbar_arrive(B.item_empty(k & 1));
    return true;
}

// --------------------------------------------------------------------------------------------
// softmax warps 0-7: thread r of tile j owns query row r of the item's tile j
// --------------------------------------------------------------------------------------------
template <int MODE>
__device__ __forceinline__ void persist_softmax(const TcArgs& ta, const PersistBars& B, uint8_t* smem, uint32_t tmem_base,
                                                volatile int* queue, volatile int* abort_flag, int tid) {
    const AttendArgs& a = ta.a;
    const int warp = tid >> 5, lane = tid & 31;
    const int j = warp >> 2;
    const int r = tid & 127;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + (uint32_t)j * 128u;
    const uint32_t tO = tmem_base + lane_base + 256u + (uint32_t)j * 128u;
    uint8_t* const qs = smem + j * kTileBytes;                     // the tile's query buffer; output stage later
    uint8_t* const ring = smem + kSmemQ;
    const __nv_bfloat162 c1b = __float2bfloat162_rn(a.sm_scale), c2b = __float2bfloat162_rn(kLog2e);

    int n0 = 0;          // ring entry number of the item's first entry
    int T = 0;           // score tiles of this query tile before the item
    int I = 0;           // items with tiles before the item
    bool ok = true;

    auto wait_entry = [&](int n) {
        if (ok) ok = mbar_wait(B.kv_full(n % kStages), (n / kStages) & 1, abort_flag);
    };
    auto signal = [&](uint32_t bar) {
        tmem_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };

    for (int k = 0;; ++k) {
        int bid = -1, count = 0;
        const bool got = take_item(B, queue, abort_flag, k, lane, bid, count);
        if (!bar_and(1 + j, 128, got)) break;                     // the tile's four warps go on or stop together
        if (bid < 0) break;
        const Item it = make_item<MODE>(ta, bid, count);
        const int ntiles = it.ntiles;
        const int qb = 2 * it.pair + j;
        const int row_g = qb * kTile + r;
        const int64_t srow = (int64_t)it.hz * a.N + row_g;
        const int hdr = header_entries<MODE>(ntiles);

        float m_true = -INFINITY, m_ref = -INFINITY, l = 0.f;
        if (MODE == kStripe) {
            m_true = m_ref = a.M[srow];
            l = a.L[srow];
        }

        // ---- query tile: raw rows from the ring, scaled and rounded into the query buffer
        if (ntiles > 0) {
            const int n = n0 + j;
            wait_entry(n);
            if (ok) {
                const uint8_t* src = ring + (n % kStages) * kTileBytes;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int id = r + 128 * i;
                    const uint32_t off = sw_off(id >> 4, id & 15);
                    uint4 raw = *reinterpret_cast<const uint4*>(src + off);
                    __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (MODE == kWindow) {
                            p2[e] = __hmul2(__hmul2(p2[e], c1b), c2b);
                        } else {
                            float2 f = __bfloat1622float2(p2[e]);
                            f.x = __fmul_rn(__fmul_rn(f.x, a.sm_scale), kLog2e);
                            f.y = __fmul_rn(__fmul_rn(f.y, a.sm_scale), kLog2e);
                            p2[e] = __floats2bfloat162_rn(f.x, f.y);
                        }
                    }
                    *reinterpret_cast<uint4*>(qs + off) = raw;
                }
                fence_proxy_async();
                mbar_arrive(B.q_full(j));
            }
            const bool all_ok = bar_and(1 + j, 128, ok);           // every thread has read the raw tile
            if (!all_ok) break;
            if (r == 0) mbar_arrive(B.kv_empty(n % kStages));
        }

        // ---- step 3: the accumulator tile, two ring entries
        const int n_acc = n0 + acc_entry(ntiles) + 2 * j;
        if (MODE == kStripe && ntiles > 0) {
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                wait_entry(n_acc + half);
                if (ok) {
                    const uint8_t* src = ring + ((n_acc + half) % kStages) * kTileBytes + r * 16;
                    uint32_t v[2][32];
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const uint4 x = *reinterpret_cast<const uint4*>(src + (c * 8 + i) * (kTile * 16));
                            v[c][4 * i] = x.x; v[c][4 * i + 1] = x.y; v[c][4 * i + 2] = x.z; v[c][4 * i + 3] = x.w;
                        }
                    tmem_st32(tO + (2 * half) * 32, v[0]);
                    tmem_st32(tO + (2 * half + 1) * 32, v[1]);
                }
            }
            if (ok) tmem_wait_st();
            const bool all_ok = bar_and(1 + j, 128, ok);
            if (!all_ok) break;
            if (r == 0) {
                mbar_arrive(B.kv_empty(n_acc % kStages));
                mbar_arrive(B.kv_empty((n_acc + 1) % kStages));
            }
        }

        // ---- the tile loop
        for (int t = 0; t < ntiles && ok; ++t) {
            ok = mbar_wait(B.s_full(j), (T + t) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            uint32_t sv[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sv[c]);
            tmem_wait_ld();

            if (MODE == kWindow) {
                const int col0 = (t < it.n_init) ? t * kTile : it.local_start + (t - it.n_init) * kTile;
                if (col0 + kTile - 1 > qb * kTile) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + c * 32 + i > row_g)
                                sv[c][i] = __float_as_uint(__uint_as_float(sv[c][i]) + -1e6f);
                }
            } else {
                const int valid = it.count - t * kTile;
                if (valid < kTile) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i >= valid) sv[c][i] = __float_as_uint(-INFINITY);
                }
            }
            {
                float mx[4] = {m_true, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
                m_true = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            }
            if (__any_sync(0xffffffffu, m_true > m_ref + kRescaleThreshold)) {
                const float alpha = fast_exp2(m_ref - m_true);
                if (!(MODE != kStripe && t == 0)) {
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
            auto exp_pairs = [&](uint32_t (&pk)[32], int c) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int e = c * 64 + 2 * i;
                    const float2 d = __fadd2_rn(make_float2(__uint_as_float(sv[e >> 5][e & 31]),
                                                            __uint_as_float(sv[(e + 1) >> 5][(e + 1) & 31])), neg_ref);
                    const float2 p = make_float2(fast_exp2(d.x), fast_exp2(d.y));
                    rs[i & 3] = __fadd2_rn(rs[i & 3], p);
                    pk[i] = pack_bf16x2(p.x, p.y);
                }
            };
            uint32_t pk0[32], pk1[32];
            exp_pairs(pk0, 0);
            tmem_st32(tS, pk0);
            signal(B.p_part(j, 0));
            exp_pairs(pk1, 1);
            tmem_st32(tS + 32, pk1);
            signal(B.p_part(j, 1));
            const float2 rsum = __fadd2_rn(__fadd2_rn(rs[0], rs[1]), __fadd2_rn(rs[2], rs[3]));
            l += rsum.x + rsum.y;
        }

        // ---- the item's result
        if (ntiles > 0) {
            if (ok) ok = mbar_wait(B.o_done(j), I & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            tcgen05_fence_after();
        }
        if (MODE == kWindow) {
            const bool all_ok = bar_and(1 + j, 128, ok);
            if (!all_ok) break;
            const float sc = fast_exp2(m_ref - m_true);
            a.M[srow] = m_true;
            a.L[srow] = l * sc;
            float* tile_acc = acc_tile(a.Acc, it.hz, a.N, qb);
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
            // the next item's first P V overwrites this accumulator: order the reads before the
            // arrivals that let the MMA warp issue it
            tcgen05_fence_before();
        } else {
            // acc / l, rounded to bf16, staged in the tile's query buffer (no MMA reads it any more) and
            // written out as whole rows; with an empty list the accumulator comes from the ring entries
            if (ntiles == 0) {
                wait_entry(n_acc);
                wait_entry(n_acc + 1);
            }
            const bool all_ok = bar_and(1 + j, 128, ok);
            if (!all_ok) break;
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
                } else {
                    const uint8_t* src = ring + ((n_acc + (c >> 1)) % kStages) * kTileBytes + r * 16;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint4 x = *reinterpret_cast<const uint4*>(src + ((c & 1) * 8 + i) * (kTile * 16));
                        v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 o4;
                    o4.x = pack_bf16x2(div_l(__uint_as_float(v[8 * i])), div_l(__uint_as_float(v[8 * i + 1])));
                    o4.y = pack_bf16x2(div_l(__uint_as_float(v[8 * i + 2])), div_l(__uint_as_float(v[8 * i + 3])));
                    o4.z = pack_bf16x2(div_l(__uint_as_float(v[8 * i + 4])), div_l(__uint_as_float(v[8 * i + 5])));
                    o4.w = pack_bf16x2(div_l(__uint_as_float(v[8 * i + 6])), div_l(__uint_as_float(v[8 * i + 7])));
                    *reinterpret_cast<uint4*>(qs + r * kRowBytes + (((c * 4 + i) ^ (r & 7)) << 4)) = o4;
                }
            }
            bar_sync(1 + j, 128);                                   // the stage is complete, the ring entries are read
            if (ntiles == 0 && r == 0) {
                mbar_arrive(B.kv_empty(n_acc % kStages));
                mbar_arrive(B.kv_empty((n_acc + 1) % kStages));
            }
            int64_t tile_off = it.z * a.osb + it.h * a.osh + (int64_t)qb * kTile * a.osn;
            const int owner = ta.rows_per_peer > 0 ? (qb * kTile) / ta.rows_per_peer : 0;
            if (ta.rows_per_peer > 0) tile_off -= (int64_t)owner * ta.rows_per_peer * a.osn;
            const int ch = r & 15;
#pragma unroll 4
            for (int s = 0; s < 16; ++s) {
                const int row = s * 8 + (r >> 4);
                const uint4 val = *reinterpret_cast<const uint4*>(qs + row * kRowBytes + ((ch ^ (row & 7)) << 4));
                const int64_t off = tile_off + (int64_t)row * a.osn + ch * 8;
                if (ta.n_peers == 0) {
                    *reinterpret_cast<uint4*>(a.out + off) = val;
                } else if (ta.rows_per_peer > 0) {
                    *reinterpret_cast<uint4*>(ta.peers[owner] + off) = val;
                } else {
                    for (int pr = 0; pr < ta.n_peers; ++pr) *reinterpret_cast<uint4*>(ta.peers[pr] + off) = val;
                }
            }
            bar_sync(1 + j, 128);                                   // the stage has been read: the buffer may take the next query tile
        }

        n0 += hdr + 2 * ntiles;
        T += ntiles;
        if (ntiles > 0) ++I;
    }
}

// --------------------------------------------------------------------------------------------
// warp 8: the MMA issuer
// --------------------------------------------------------------------------------------------
template <int MODE>
__device__ __forceinline__ void persist_mma(const TcArgs& ta, const PersistBars& B, uint32_t s_u, uint32_t ring_u,
                                            uint32_t tmem_base, volatile int* queue, volatile int* abort_flag, int lane) {
    const bool issuer = elect_one();
    constexpr uint32_t kIdescQK = idesc_bf16_128x128(0);
    constexpr uint32_t kIdescPV = idesc_bf16_128x128(1);
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
            if (issuer) mma_ss(tmem_base + (uint32_t)j * 128u, desc(q_lo[j] + off), desc(k_lo + off), kIdescQK, ks > 0);
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
    auto wait_entry = [&](int n) { return wait_all(B.kv_full(n % kStages), (n / kStages) & 1); };

    int n0 = 0, T = 0, I = 0;
    for (int k = 0;; ++k) {
        int bid, count;
        if (!take_item(B, queue, abort_flag, k, lane, bid, count)) break;
        if (bid < 0) break;
        const Item it = make_item<MODE>(ta, bid, count);
        const int ntiles = it.ntiles;
        const int hdr = header_entries<MODE>(ntiles);
        if (ntiles == 0) {
            n0 += hdr;
            continue;
        }
        const int nkv = n0 + k_entry<MODE>(0);                     // ring entry of K_0
        bool ok = wait_all(B.q_full(0), I & 1) && wait_all(B.q_full(1), I & 1) && wait_entry(nkv);
        if (!ok) break;
        fence_proxy_async();
        tcgen05_fence_after();
        issue_qk(0, slot_addr(nkv));
        commit_if(issuer, B.s_full(0));
        issue_qk(1, slot_addr(nkv));
        commit_if(issuer, B.s_full(1));
        commit_if(issuer, B.kv_empty(nkv % kStages));
        for (int t = 0; t < ntiles && ok; ++t) {
            const int nv = n0 + v_entry<MODE>(t), nk = n0 + k_entry<MODE>(t + 1);
            ok = wait_entry(nv);
            if (!ok) break;
            fence_proxy_async();
            for (int j = 0; j < 2 && ok; ++j) {
                for (int q = 0; q < kPParts && ok; ++q) {
                    ok = wait_all(B.p_part(j, q), (T + t) & 1);
                    if (!ok) break;
                    tcgen05_fence_after();
                    issue_pv(j, slot_addr(nv), (t > 0) || (MODE == kStripe) || q > 0, q * (8 / kPParts));
                }
                if (!ok) break;
                if (j == 1) commit_if(issuer, B.kv_empty(nv % kStages));
                if (t + 1 < ntiles) {
                    if (j == 0) {
                        ok = wait_entry(nk);
                        if (!ok) break;
                        fence_proxy_async();
                        tcgen05_fence_after();
                    }
                    issue_qk(j, slot_addr(nk));
                    commit_if(issuer, B.s_full(j));
                    if (j == 1) commit_if(issuer, B.kv_empty(nk % kStages));
                } else {
                    commit_if(issuer, B.o_done(j));
                }
            }
        }
        if (!ok) break;
        n0 += hdr + 2 * ntiles;
        T += ntiles;
        ++I;
    }
}

// --------------------------------------------------------------------------------------------
// warps 9-11: loaders.  Warp 9 also draws the items and publishes them.
// --------------------------------------------------------------------------------------------
template <int MODE>
__device__ __forceinline__ void persist_loader(const CUtensorMap* kmap, const CUtensorMap* vmap, const CUtensorMap* kgmap,
                                               const CUtensorMap* vgmap, const CUtensorMap* qmap, const TcArgs& ta,
                                               const PersistArgs& pa, const PersistBars& B, uint32_t ring_u,
                                               volatile int* queue, volatile int* abort_flag, int lw, int lane) {
    const AttendArgs& a = ta.a;
    bool ok = true;
    int n = 0;                                                     // running ring entry number

    // wait until the slot of entry n is free again
    auto acquire = [&](int e) {
        const int use = e / kStages;
        if (use > 0) {
            ok = mbar_wait(B.kv_empty(e % kStages), (use - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        return ok;
    };
    // The leader draws the next item shortly before the current one's last entries go out: the draw
    // (an atomic) sixteen entries before the end, its answer and the item's count (a load) eight
    // before, so that neither is waited for.  Not earlier: CTAs that work on the same big block of a
    // head read the same key/value tiles (step 3: the same 64 KB slots of the gather scratch, far more
    // than L2 holds in total) and should start together, as consecutive items do when each is drawn
    // just before it starts.  Drawing an item a whole item ahead let them drift apart by the length
    // of the items in between; it cost 4 % of the SM clock under the power cap (the slots then come
    // from DRAM more than once).  An item of fewer than sixteen entries draws at its start.
    auto clamp_bid = [&](int v) { return v < pa.n_items ? v : -1; };
    int bid0 = -1, count0 = 0, bid1 = -1, count1 = 0, drawn = 0;
    if (lw == 0) {
        if (lane == 0) drawn = atomicAdd(pa.item_counter, 1);
        bid0 = clamp_bid(__shfl_sync(0xffffffffu, drawn, 0));
        count0 = bid0 >= 0 ? item_count<MODE>(ta, bid0) : 0;
    }
    for (int k = 0;; ++k) {
        int bid, count;
        if (lw == 0) {
            bid = bid0;
            count = count0;
            if (k >= 2) {
                ok = mbar_wait(B.item_empty(k & 1), ((k >> 1) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            if (lane == 0) {
                queue[2 * (k & 1)] = bid;
                queue[2 * (k & 1) + 1] = count;
                mbar_arrive(B.item_full(k & 1));
            }
            if (bid < 0) break;
        } else {
            if (!take_item(B, queue, abort_flag, k, lane, bid, count)) break;
            if (bid < 0) break;
        }
        const Item it = make_item<MODE>(ta, bid, count);
        const int ntiles = it.ntiles;
        const int hdr = header_entries<MODE>(ntiles);
        const int a0 = acc_entry(ntiles);

        const __nv_bfloat16* kbase = a.k.ptr + it.z * a.k.sb + it.kvh * a.k.sh;
        const __nv_bfloat16* vbase = a.v.ptr + it.z * a.v.sb + it.kvh * a.v.sh;
        const int64_t koff = it.z * a.k.sb + it.kvh * a.k.sh, voff = it.z * a.v.sb + it.kvh * a.v.sh;
        const int k_row0 = (int)(koff / a.k.sn), k_col0 = (int)(koff % a.k.sn);
        const int v_row0 = (int)(voff / a.v.sn), v_col0 = (int)(voff % a.v.sn);
        const int32_t* idp = it.idp;
        int row0 = 0, gslot = -1;
        bool run = true;
        const int entries = hdr + 2 * ntiles;
        const int e_draw = max(0, entries - 16), e_answer = max(0, entries - 8);
        for (int e = 0; e < entries && ok; ++e, ++n) {
            if (lw == 0) {
                if (e == e_draw && lane == 0) drawn = atomicAdd(pa.item_counter, 1);
                if (e == e_answer) {
                    bid1 = clamp_bid(__shfl_sync(0xffffffffu, drawn, 0));
                    count1 = bid1 >= 0 ? item_count<MODE>(ta, bid1) : 0;
                }
            }
            // what entry e is: a query tile (e < 2 when the item has tiles), an accumulator half
            // (ea = 0 .. 3), or half m of the key/value stream (m = 2 t + is_v)
            int m = -1, ea = -1;
            if (e >= hdr) m = e - hdr;
            else if (e >= a0) ea = e - a0;
            const int slot = n % kStages;
            const uint32_t dst = ring_u + (uint32_t)slot * kTileBytes;
            if (m < 0) {
                if (!acquire(n)) break;
                if (lw == 0 && lane == 0) {
                    mbar_arrive_expect_tx(B.kv_full(slot), kTileBytes);
                    if (ea < 0) {
                        tma_tile(dst, qmap, B.kv_full(slot), pa.qpos_n, pa.qpos_h, pa.qpos_b, (2 * it.pair + e) * kTile, it.h,
                                 it.z);
                    } else {
                        const float* src = acc_tile(a.Acc, it.hz, a.N, 2 * it.pair + (ea >> 1)) + (ea & 1) * (kTileBytes / 4);
                        bulk_load(dst, src, kTileBytes, B.kv_full(slot));
                    }
                } else {
                    mbar_arrive(B.kv_full(slot));
                }
                continue;
            }
            const int t = m >> 1;
            const bool is_v = m & 1;
            if (!is_v) {
                if (MODE == kWindow) {
                    row0 = (t < it.n_init) ? t * kTile : it.local_start + (t - it.n_init) * kTile;
                } else {
                    const int s0 = t * kTile;
                    run = false;
                    gslot = it.slotp ? it.slotp[t] : -1;
                    if (gslot >= ta.n_slots) gslot = -1;
                    if (s0 + kTile <= count) {
                        row0 = idp[s0];
                        run = (idp[s0 + kTile - 1] - row0) == kTile - 1;
                    }
                }
            }
            if (!acquire(n)) break;
            if (run || gslot >= 0) {
                if (lw == 0 && lane == 0) {
                    mbar_arrive_expect_tx(B.kv_full(slot), kTileBytes);
                    if (!run)
                        bulk_load(dst, ta.gather + (int64_t)gslot * (2 * kTileBytes) + (is_v ? kTileBytes : 0), kTileBytes,
                                  B.kv_full(slot));
                    else if (is_v)
                        tma_tile(dst, vmap, B.kv_full(slot), ta.vpos_n, ta.vpos_h, ta.vpos_b, row0, it.kvh, it.z);
                    else
                        tma_tile(dst, kmap, B.kv_full(slot), ta.kpos_n, ta.kpos_h, ta.kpos_b, row0, it.kvh, it.z);
                } else {
                    mbar_arrive(B.kv_full(slot));
                }
                continue;
            }
            // Discrete rows without a scratch slot.  The TMA unit and the load/store unit each sustain
            // only about one 128-byte row segment per 17-24 cycles on gathers, so the tile is split
            // between them: rows [0, tma_rows) by TMA row gathers from the first loader warp (lane i takes
            // rows 4i .. 4i+3, two 64-column halves each), the rest by 16-byte cp.async copies from the
            // other loader warps; without a usable 2-D map all loader warps copy.  Slots past the count
            // read row 0 / zero-fill; the softmax masks them.
            const bool g4 = is_v ? ta.v_gather : ta.k_gather;
            const int tma_rows = g4 ? kTmaRows : 0;
            int ra, rb;
            {
                const int first = g4 ? 1 : 0, nw = kLoaderWarps - first;
                const int pairs = (kTile - tma_rows) / 2;
                const int w = lw - first;
                ra = tma_rows + 2 * ((pairs * w) / nw);
                rb = tma_rows + 2 * ((pairs * (w + 1)) / nw);
                if (w < 0) ra = rb = 0;
            }
            if (g4 && lw == 0) {
                if (lane == 0)
                    mbar_arrive_expect_tx(B.kv_full(slot), (uint32_t)tma_rows * kRowBytes);
                else
                    mbar_arrive(B.kv_full(slot));
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
                    id4.x = min(max(id4.x, 0), a.N - 1);
                    id4.y = min(max(id4.y, 0), a.N - 1);
                    id4.z = min(max(id4.z, 0), a.N - 1);
                    id4.w = min(max(id4.w, 0), a.N - 1);
                    const CUtensorMap* gm = is_v ? vgmap : kgmap;
                    const int r0 = is_v ? v_row0 : k_row0, c0 = is_v ? v_col0 : k_col0;
                    const uint32_t d = dst + (uint32_t)lane * 512u;
                    tma_gather4(d, gm, B.kv_full(slot), c0, r0 + id4.x, r0 + id4.y, r0 + id4.z, r0 + id4.w);
                    tma_gather4(d + kSlabBytes, gm, B.kv_full(slot), c0 + 64, r0 + id4.x, r0 + id4.y, r0 + id4.z,
                                r0 + id4.w);
                }
            } else {
                const __nv_bfloat16* base = is_v ? vbase : kbase;
                const int64_t sn = is_v ? a.v.sn : a.k.sn;
                const int s0 = t * kTile + ra;
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
                cp_async_mbar_arrive_noinc(B.kv_full(slot));
            }
        }
        if (!ok) break;
        bid0 = bid1;
        count0 = count1;
    }
    cp_async_wait<0>();
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
attend_persist_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                      const __grid_constant__ CUtensorMap kgmap, const __grid_constant__ CUtensorMap vgmap,
                      const __grid_constant__ CUtensorMap qmap, TcArgs ta, PersistArgs pa) {
    static_assert(MODE == kWindow || MODE == kStripe, "the persistent kernel runs steps 1 and 3");
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const uint32_t raw_u = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_u & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t s_u = raw_u + pad;
    const uint32_t ring_u = s_u + kSmemQ;
    PersistBars B;
    B.bars = ring_u + kSmemRing;
    uint8_t* bar_mem = smem + kSmemQ + kSmemRing;
    const uint32_t tmem_slot_u = B.bars + 192u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_mem + 192);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 196);
    volatile int* queue = reinterpret_cast<volatile int*>(bar_mem + kQueueOff);

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(B.kv_full(i), 32 * kLoaderWarps);
            mbar_init(B.kv_empty(i), 1);
        }
        for (int j = 0; j < 2; ++j) {
            mbar_init(B.q_full(j), 128);
            mbar_init(B.s_full(j), 1);
            for (int q = 0; q < kPParts; ++q) mbar_init(B.p_part(j, q), 4);
            mbar_init(B.o_done(j), 1);
            mbar_init(B.item_full(j), 1);
            mbar_init(B.item_empty(j), kItemConsumers);
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
        setmaxnreg_inc<kSoftmaxRegs>();
        persist_softmax<MODE>(ta, B, smem, tmem_base, queue, abort_flag, tid);
    } else {
        setmaxnreg_dec<kOtherRegs>();
        if (warp == 8)
            persist_mma<MODE>(ta, B, s_u, ring_u, tmem_base, queue, abort_flag, lane);
        else
            persist_loader<MODE>(&kmap, &vmap, &kgmap, &vgmap, &qmap, ta, pa, B, ring_u, queue, abort_flag, warp - 9, lane);
    }

    tcgen05_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicMax(ta.status, 1);
    if (warp == 8) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tc
}  // namespace aa

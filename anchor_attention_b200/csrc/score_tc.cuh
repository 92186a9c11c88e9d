// Step 2, scoring pass on the Blackwell tensor cores (tcgen05 + tensor memory + TMA).
//
// Replaces the key-column loop of get_q_mask_triton (reference:
// anchor_attn/src/ops/get_mask_test.py:93-121): for every big block b >= 1 and every
// 128-column key tile that holds candidate columns [block, b*G - block), G = block*step
// (for block = 128: tiles 1 .. b*step - 2), the `step` block-pooled query rows of each
// query head are multiplied with the 128 keys; a column is hit for (head, b) when
//     fp32(bf16(dot * qk_scale)) + diff >= anchor(row)          for some pooled row.
// Output: one bit per (query head, big block, column) in the hit bitmap.
//
// A "unit" is the `step` pooled rows of one (query head of the KV group, big block);
// units are ordered big block first.  One CTA owns up to 2 * (128 / step) consecutive
// units of one KV head -- two 128-row A tiles that stay in shared memory -- and a chunk
// of kTilesPerCta key tiles that it streams once through a 4-slot TMA ring:
//   S_i = A_i K^T  (tcgen05.mma, M = N = K-extent 128, accumulators double-buffered in
//   tensor memory), then one thread per pooled row turns its 128 scores into hit bits.
// The key stream is therefore shared by all query heads of the KV group and by up to
// four big blocks.
//
// The per-element test is a single comparison: the chain dot -> *qk_scale (fp32, rn) ->
// bf16 (rn) -> +diff (fp32, rn) -> >= anchor is monotone in dot, so each row first finds
// by bisection over the ordered float encodings the smallest dot that passes (evaluating
// exactly that chain), and then compares accumulators against it.  The result equals the
// chain applied to every element, bit for bit.
//
// Warp roles (320 threads): warps 0-3 / 4-7 = epilogue of A tile 0 / 1 (thread r owns
// pooled row r = tensor-memory lane r), warp 8 = TMA producer, warp 9 = MMA issuer.
// Every wait is bounded (tc_ptx.cuh).
#pragma once
#include "attend_tc.cuh"

namespace aa {
namespace sc {

using namespace aa::tc;

constexpr int kScThreads = 320;
constexpr int kScStages = 4;
constexpr int kTilesPerCta = 16;
constexpr int kScSmemA = 2 * kTileBytes;
constexpr int kScSmemRing = kScStages * kTileBytes;
constexpr int kScSmemTotal = kScSmemA + kScSmemRing + 256 + 1024;

struct ScoreArgs {
    const float* apool;        // [B, H, N/128] block-mean anchors (already rounded to bf16 values)
    uint32_t* bitmap;          // [B, H, NB, N/32]
    int B, H, Hkv, N, step, block;      // block = pooling block size; candidates of big block b: [block, b*G - block)
    float qk_scale, diff;
    int kpos_n, kpos_h, kpos_b;
    int32_t* status;
};

// ordered encoding of floats: key(a) < key(b)  <=>  a < b  (for non-NaN a, b)
__device__ __forceinline__ float key_to_float(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

__device__ __forceinline__ bool passes(float dot, float qk_scale, float diff, float anchor) {
    const float sc = bf16_round(__fmul_rn(dot, qk_scale));
    return __fadd_rn(sc, diff) >= anchor;
}

// smallest float `dot` with passes(dot); NaN if none does
__device__ __forceinline__ float pass_threshold(float qk_scale, float diff, float anchor) {
    uint32_t lo = 0x007FFFFFu, hi = 0xFF800000u;          // keys of -inf and +inf
    if (!passes(key_to_float(hi), qk_scale, diff, anchor)) return __uint_as_float(0x7FC00000u);
#pragma unroll 1
    while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (passes(key_to_float(mid), qk_scale, diff, anchor)) hi = mid; else lo = mid + 1;
    }
    return key_to_float(lo);
}

__global__ void __launch_bounds__(kScThreads, 1)
score_tc_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap qmap, ScoreArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- which work item (uniform for the CTA; empty items leave before any set-up) ----
    const int step = a.step;
    const int Hg = a.H / a.Hkv;
    const int G = a.block * step;
    const int NB = a.N / G;
    const int t_first = a.block / 128;               // first 128-column tile that holds candidates
    auto t_last = [&](int b) { return (b * G - a.block - 1) >> 7; };   // last one of big block b
    const int upt = 128 / step;                      // units per A tile
    const int units_kv = (NB - 1) * Hg;
    const int u0 = blockIdx.y * 2 * upt;
    if (u0 >= units_kv) return;
    const int u_end = min(u0 + 2 * upt, units_kv);   // exclusive
    const int nA = (u_end - u0 + upt - 1) / upt;
    const int t_begin = t_first + blockIdx.x * kTilesPerCta;
    // tiles each A tile needs from this chunk: candidates of its last big block
    int nt[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int ul = min(u0 + (i + 1) * upt, u_end) - 1;            // last unit of tile i
        const int bmax = 1 + ul / Hg;
        nt[i] = (i < nA) ? max(0, min(kTilesPerCta, t_last(bmax) - t_begin + 1)) : 0;
    }
    const int ntiles = max(nt[0], nt[1]);
    if (ntiles <= 0) return;
    const int z = blockIdx.z / a.Hkv, kvh = blockIdx.z % a.Hkv;

    const uint32_t raw_u = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_u & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t s_u = raw_u + pad;
    const uint32_t ring_u = s_u + kScSmemA;
    const uint32_t bars = ring_u + kScSmemRing;
    auto k_full = [&](int i) { return bars + 8u * i; };
    auto k_empty = [&](int i) { return bars + 32u + 8u * i; };
    auto d_full = [&](int i, int buf) { return bars + 64u + 8u * (2 * i + buf); };
    auto d_empty = [&](int i, int buf) { return bars + 96u + 8u * (2 * i + buf); };
    const uint32_t a_full = bars + 128u;
    const uint32_t tmem_slot_u = bars + 136u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kScSmemA + kScSmemRing + 136);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kScSmemA + kScSmemRing + 140);

    if (tid == 0) {
        for (int i = 0; i < kScStages; ++i) {
            mbar_init(k_full(i), 1);
            mbar_init(k_empty(i), 1);
        }
        for (int i = 0; i < 2; ++i)
            for (int buf = 0; buf < 2; ++buf) {
                mbar_init(d_full(i, buf), 1);
                mbar_init(d_empty(i, buf), 128);
            }
        mbar_init(a_full, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot_u, kTmemCols);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // =================================================== epilogue warps
        const int i = warp >> 2;                     // A tile
        const int r = tid & 127;                     // pooled row inside the A tile = TMEM lane
        const int u = u0 + i * upt + r / step;
        const bool valid = (i < nA) && (u < u_end);
        const int b = 1 + (valid ? u : u0) / Hg;
        const int h = kvh * Hg + (valid ? u : u0) % Hg;
        const int words_per_row = a.N / 32;
        float thr = __uint_as_float(0x7FC00000u);
        if (valid) {
            const float anchor = a.apool[(int64_t)(z * a.H + h) * (a.N / a.block) + b * step + r % step];
            thr = pass_threshold(a.qk_scale, a.diff, anchor);
        }
        uint32_t* brow = a.bitmap + ((int64_t)(z * a.H + h) * NB + b) * words_per_row;
        const int last_tile = t_last(b);             // last candidate tile of this row's big block
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        bool ok = true;
        for (int tt = 0; tt < nt[i] && ok; ++tt) {
            const int buf = tt & 1;
            ok = mbar_wait(d_full(i, buf), (tt >> 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t tD = tmem_base + lane_base + (uint32_t)(2 * i + buf) * 128u;
            uint32_t word[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(tD + c * 32, v);
                tmem_wait_ld();
                uint32_t w = 0;
#pragma unroll
                for (int e = 0; e < 32; ++e)
                    if (__uint_as_float(v[e]) >= thr) w |= 1u << e;
                word[c] = w;
            }
            tcgen05_fence_before();
            mbar_arrive(d_empty(i, buf));
            // OR over the `step` rows of the unit (16 or 32 consecutive lanes)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int off = 1; off < 16; off <<= 1) word[c] |= __shfl_xor_sync(0xffffffffu, word[c], off);
                if (step == 32) word[c] |= __shfl_xor_sync(0xffffffffu, word[c], 16);
            }
            const int tg = t_begin + tt;
            const int j = lane & 3;
            const uint32_t mine = j == 0 ? word[0] : (j == 1 ? word[1] : (j == 2 ? word[2] : word[3]));
            if (valid && tg <= last_tile && (lane & (step - 1)) < 4) brow[tg * 4 + j] = mine;
        }
    } else if (warp == 8) {
        // =================================================== TMA producer
        bool ok = true;
        if (lane == 0) {
            const int nunits = u_end - u0;
            mbar_arrive_expect_tx(a_full, (uint32_t)(nunits * step * kRowBytes));
            for (int k = 0; k < nunits; ++k) {
                const int u = u0 + k;
                const int b = 1 + u / Hg, h = kvh * Hg + u % Hg;
                // unit k occupies rows (k % upt) * step .. of A tile k / upt
                const uint32_t dst = s_u + (uint32_t)(k / upt) * kTileBytes + (uint32_t)((k % upt) * step) * 128u;
                tma_load_3d(dst, &qmap, a_full, 0, b * step, z * a.H + h);
                tma_load_3d(dst + kSlabBytes, &qmap, a_full, 64, b * step, z * a.H + h);
            }
        }
        for (int tt = 0; tt < ntiles && ok; ++tt) {
            const int slot = tt % kScStages, it = tt / kScStages;
            if (it > 0) {
                ok = mbar_wait(k_empty(slot), (it - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(k_full(slot), kTileBytes);
                tma_tile(ring_u + (uint32_t)slot * kTileBytes, &kmap, k_full(slot), a.kpos_n, a.kpos_h, a.kpos_b,
                         (t_begin + tt) * kTile, kvh, z);
            }
        }
    } else {
        // =================================================== MMA issuer (warp 9)
        const bool issuer = elect_one();
        constexpr uint32_t kIdesc = idesc_bf16_128x128(0);
        constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
        auto desc = [&](uint32_t lo) { return ((uint64_t)kDescHi << 32) | lo; };
        auto lo_kmajor = [&](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1u << 16); };
        auto wait_all = [&](uint32_t bar, uint32_t parity) {
            return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
        };
        bool ok = wait_all(a_full, 0);
        for (int tt = 0; tt < ntiles && ok; ++tt) {
            const int slot = tt % kScStages, buf = tt & 1;
            ok = wait_all(k_full(slot), (tt / kScStages) & 1);
            if (!ok) break;
            const uint32_t k_lo = lo_kmajor(ring_u + (uint32_t)slot * kTileBytes);
            for (int i = 0; i < 2 && ok; ++i) {
                if (tt >= nt[i]) continue;
                if (tt >= 2) {
                    ok = wait_all(d_empty(i, buf), ((tt >> 1) - 1) & 1);
                    if (!ok) break;
                }
                tcgen05_fence_after();
                const uint32_t a_lo = lo_kmajor(s_u + (uint32_t)i * kTileBytes);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (uint32_t)(((ks >> 2) * kSlabBytes + (ks & 3) * 32) >> 4);
                    if (issuer)
                        mma_ss(tmem_base + (uint32_t)(2 * i + buf) * 128u, desc(a_lo + off), desc(k_lo + off), kIdesc,
                               ks > 0);
                }
                commit_if(issuer, d_full(i, buf));
            }
            if (ok) commit_if(issuer, k_empty(slot));
        }
    }

    // ---- teardown ----
    tcgen05_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicMax(a.status, 1);
    if (warp == 9) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace sc
}  // namespace aa

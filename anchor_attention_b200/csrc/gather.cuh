// Step 3, first pass: the selected key/value rows of every id tile that is not a run of
// consecutive rows are copied ONCE into contiguous scratch, already in the shared-memory
// image the tensor cores read, and the id lists can be validated without gathering anything.
//
// Why: the 2048 query rows of a big block are served by eight CTAs of the attention kernel
// (256 rows each) that all walk the same id list (reference: anchor_attn/src/ops/
// anchor_attn_v4.py:72-101, where every 128-row program gathers its rows through pointer
// loads).  Gathering 128 discrete 256-byte rows costs an SM about twice as long as the
// products on them take, and eight SMs would each pay it for the same rows.  After this pass
// a tile is one contiguous 64 KB slot (K image, then V image) that each of the eight CTAs
// fetches with two bulk copies at the full L2 -> shared-memory rate.
//
// Slot layout (kTileBytes = 32 KB per image): the image of a tile is what the attention
// kernel's ring slot holds -- two slabs of 64 columns, 128 rows of 128 bytes each, the
// 16-byte chunk c of row r stored at chunk position (c & 7) ^ (r & 7) of its slab row
// (the 128-byte swizzle of the TMA box loads and MMA descriptors).  Rows past the list's
// count are zero.
//
// Slots come from a bump counter (one atomicAdd per tile); the per-tile table says where a
// tile went, or -1 when it is a run (the attention kernel box-loads those from K/V directly)
// or when the scratch is full (the attention kernel then gathers the rows itself, as it
// does when no scratch is given).  Slot numbers depend on scheduling, slot contents do not,
// so results are bit-identical from run to run.
#pragma once
#include "common.cuh"

namespace aa {

constexpr int kGatherThreads = 256;
constexpr int kGatherSplit = 8;          // CTAs that share the tiles of one (head, big block)

struct GatherArgs {
    TensorView k, v;
    const int32_t* counts;               // [B, H, NB]
    const int32_t* ids;                  // [B, H, ids_per_head]
    int64_t ids_per_head;
    int32_t* tile_slot;                  // [B, H, ids_per_head / 128]
    uint8_t* scratch;                    // n_slots x 64 KB, 1024-byte aligned
    int32_t* slot_counter;               // zero before the launch
    int n_slots;
    int hz0;                             // first (batch, head) of this launch: blockIdx.z counts from it
    const int32_t* plan;                 // NULL, or: the launch only runs when *plan == run_if (plan_step3_kernel)
    int run_if;
    int H, Hkv, N, step, block;
};

// first id slot of big block b inside a head's list (aa_id_row_offset)
__device__ __forceinline__ int64_t id_row_offset(int G, int block, int b) {
    return (b == 0) ? 0 : ((int64_t)G * b * (b - 1) / 2 - 2 * (int64_t)block * (b - 1));
}

// grid (kGatherSplit, NB - 1, heads of the launch); big block b = blockIdx.y + 1
__global__ void __launch_bounds__(kGatherThreads) gather_tiles_kernel(GatherArgs a) {
    constexpr int kTileRows = 128, kImage = kTileRows * kRowBytes, kSlab = kImage / 2;
    if (a.plan && *a.plan != a.run_if) return;
    const int b = blockIdx.y + 1, hz = a.hz0 + blockIdx.z;
    const int z = hz / a.H, h = hz % a.H, kvh = h / (a.H / a.Hkv);
    const int G = a.block * a.step, NB = a.N / G;
    const int cap = b * G - 2 * a.block;
    const int count = min(max(a.counts[(int64_t)hz * NB + b], 0), cap);
    const int ntiles = (count + kTileRows - 1) / kTileRows;
    if ((int)blockIdx.x >= ntiles) return;
    const int64_t row_off = id_row_offset(G, a.block, b);
    const int32_t* idp = a.ids + (int64_t)hz * a.ids_per_head + row_off;
    // a full list holds every candidate column in order: all of its tiles are runs (the attention
    // kernel finds that out by itself and never looks at their slots)
    if (count == cap && idp[0] == a.block && idp[cap - 1] == b * G - a.block - 1) return;
    int32_t* slots = a.tile_slot + (int64_t)hz * (a.ids_per_head / kTileRows) + row_off / kTileRows;
    const __nv_bfloat16* kbase = a.k.ptr + z * a.k.sb + kvh * a.k.sh;
    const __nv_bfloat16* vbase = a.v.ptr + z * a.v.sb + kvh * a.v.sh;

    __shared__ int32_t id_s[kTileRows];
    __shared__ int slot_s;
    const int tid = threadIdx.x;
    const int ch = tid & 15, rg = tid >> 4;          // 16-byte chunk of the row, row inside a group of 16
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int s0 = t * kTileRows;
        __syncthreads();                             // id_s / slot_s of the previous tile are no longer read
        if (tid < kTileRows) id_s[tid] = (s0 + tid < count) ? idp[s0 + tid] : -1;
        __syncthreads();
        if (tid == 0) {
            const bool run = s0 + kTileRows <= count && id_s[kTileRows - 1] - id_s[0] == kTileRows - 1;
            int slot = -1;
            if (!run && a.n_slots > 0) {
                slot = atomicAdd(a.slot_counter, 1);
                if (slot >= a.n_slots) slot = -1;
            }
            slots[t] = slot;
            slot_s = slot;
        }
        __syncthreads();
        const int slot = slot_s;
        if (slot < 0) continue;
        uint8_t* dst = a.scratch + (int64_t)slot * (2 * kImage);
        // 8 K rows and 8 V rows per thread: all sixteen loads are issued before the first store
        uint4 kx[8], vx[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int id = id_s[i * 16 + rg];
            const int row = min(max(id, 0), a.N - 1);
            kx[i] = make_uint4(0u, 0u, 0u, 0u);
            vx[i] = make_uint4(0u, 0u, 0u, 0u);
            if (id >= 0) {
                kx[i] = __ldg(reinterpret_cast<const uint4*>(kbase + (int64_t)row * a.k.sn) + ch);
                vx[i] = __ldg(reinterpret_cast<const uint4*>(vbase + (int64_t)row * a.v.sn) + ch);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = i * 16 + rg;
            const int off = (ch >> 3) * kSlab + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
            *reinterpret_cast<uint4*>(dst + off) = kx[i];
            *reinterpret_cast<uint4*>(dst + kImage + off) = vx[i];
        }
    }
}

// ---------------------------------------------------------------------------
// How step 3 runs when the scratch cannot hold a slot for every tile that any list COULD have:
// *plan = 0 -> the lists at hand need no more than n_slots slots (tiles of the lists that are not
// full; a full list is all runs), everything goes in one gather pass and one attention launch;
// *plan = 1 -> KV head by KV head, the scratch reused.  Both sequences are launched; the kernels of
// the one that was not chosen leave at once (the gather pass reads *plan, the attention kernel
// finds its item counter exhausted: arm_step3_kernel).  One block of 256 threads.
// ---------------------------------------------------------------------------
// Sets the two counters of one part of step 3 (the status words at `counters`).  A part that is to run
// (no plan, or *plan == run_if): slot counter 0, item counter at the part's first item.  A part that is
// not: item counter beyond any item, so that the attention kernel's CTAs find nothing to draw and leave;
// the slot counter keeps what the sequence that did run left in it.
__global__ void arm_step3_kernel(int32_t* counters, const int32_t* plan, int run_if, int first_item) {
    if (threadIdx.x == 0) {
        if (!plan || *plan == run_if) {
            counters[0] = 0;
            counters[1] = first_item;
        } else {
            counters[1] = 0x7F000000;
        }
    }
}

__global__ void __launch_bounds__(256) plan_step3_kernel(const int32_t* __restrict__ counts, int n_lists, int NB, int G,
                                                         int block, int n_slots, int32_t* plan) {
    __shared__ unsigned long long part[256];
    unsigned long long tiles = 0;
    for (int i = threadIdx.x; i < n_lists; i += blockDim.x) {
        const int b = i % NB;
        const int cap = max(b * G - 2 * block, 0);
        const int count = min(max(counts[i], 0), cap);
        if (count < cap) tiles += (unsigned long long)((count + 127) / 128);
    }
    part[threadIdx.x] = tiles;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) *plan = part[0] > (unsigned long long)n_slots ? 1 : 0;
}

// ---------------------------------------------------------------------------
// List validation (reads counts and ids only, gathers nothing): every count within the
// capacity of its big block, every list ascending and inside the candidate range
// [block, b*G - block).  A violation sets *flag to 1.  grid (NB, B * H), 256 threads.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) validate_lists_kernel(const int32_t* __restrict__ counts,
                                                             const int32_t* __restrict__ ids, int64_t ids_per_head,
                                                             int N, int step, int block, int32_t* flag) {
    const int b = blockIdx.x, hz = blockIdx.y;
    const int G = block * step, NB = N / G;
    const int cap = (b == 0) ? 0 : b * G - 2 * block;
    const int count = counts[(int64_t)hz * NB + b];
    bool bad = count < 0 || count > cap;
    if (!bad) {
        const int32_t* idp = ids + (int64_t)hz * ids_per_head + id_row_offset(G, block, b);
        const int lo = block, hi = b * G - block;
        for (int i = threadIdx.x; i < count; i += blockDim.x) {
            const int v = idp[i];
            if (v < lo || v >= hi) bad = true;
            if (i > 0 && idp[i - 1] >= v) bad = true;
        }
    }
    if (bad) atomicMax(flag, 1);
}

}  // namespace aa

// Block-granular comparator: turning the per-query-block key-block lists into the
// per-CTA tile lists the attention kernel walks.
//
// The comparator's attention kernel (anchor_attn/src/ops/block_sparse_flash_attention_v2.py:10-110)
// gives every 128-row query block m its own list and reads the first
// min(m + 1, max_blocks) entries of it (:66).  Here one CTA owns two consecutive query
// blocks that share the key tiles in shared memory, so their two lists are merged into
// one ascending list; each entry carries, next to the key block index, which of the two
// query tiles attends it.  An index that occurs c0 times in one list and c1 times in the
// other occurs max(c0, c1) times in the merged list, the first c0 (c1) copies flagged for
// the first (second) tile, so every tile still sees exactly its own sequence, duplicates
// included (the reference's index builders pad short rows with zeros, which sort to the
// front and make key block 0 count several times).
#pragma once
#include <limits.h>

#include "common.cuh"

namespace aa {

// One thread per (batch*head, pair of query blocks).  Entries beyond a tile's own block are
// causally masked for all of its rows and change nothing in the reference; they are dropped.
// *unsorted is set to 1 when a list is not ascending (the merge needs sorted lists, which is
// what every index builder of the reference produces).
__global__ void __launch_bounds__(128)
merge_block_lists_kernel(const int32_t* __restrict__ block_index, int BH, int num_rows, int max_blocks,
                         int32_t* __restrict__ lists, int32_t* __restrict__ counts, int list_stride,
                         int32_t* __restrict__ unsorted) {
    const int npairs = num_rows / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= BH * npairs) return;
    const int hz = idx / npairs, pair = idx % npairs;
    const int m0 = 2 * pair, m1 = m0 + 1;
    const int32_t* l0 = block_index + ((int64_t)hz * num_rows + m0) * max_blocks;
    const int32_t* l1 = l0 + max_blocks;
    const int n0 = min(m0 + 1, max_blocks), n1 = min(m1 + 1, max_blocks);
    int32_t* out = lists + (int64_t)idx * list_stride;
    int i = 0, j = 0, n = 0;
    int prev0 = -1, prev1 = -1;
    bool sorted = true;
    // the whole of both rows must ascend, also behind the entry at which the merge stops reading
    for (int k = 1; k < n0; ++k) sorted = sorted && l0[k] >= l0[k - 1];
    for (int k = 1; k < n1; ++k) sorted = sorted && l1[k] >= l1[k - 1];
    // a value above the tile's own block ends that tile's list (ascending order)
    int a = (i < n0) ? l0[i] : INT_MAX, b = (j < n1) ? l1[j] : INT_MAX;
    while (true) {
        if (a < 0 || a > m0) a = INT_MAX;
        if (b < 0 || b > m1) b = INT_MAX;
        if (a == INT_MAX && b == INT_MAX) break;
        uint32_t e;
        if (a == b) {
            e = (uint32_t)a | (3u << kBlockFlagShift);
        } else if (a < b) {
            e = (uint32_t)a | (1u << kBlockFlagShift);
        } else {
            e = (uint32_t)b | (2u << kBlockFlagShift);
        }
        if (n < list_stride) out[n] = (int32_t)e;
        ++n;
        if (e & (1u << kBlockFlagShift)) {
            sorted = sorted && a >= prev0;
            prev0 = a;
            ++i;
            a = (i < n0) ? l0[i] : INT_MAX;
        }
        if (e & (2u << kBlockFlagShift)) {
            sorted = sorted && b >= prev1;
            prev1 = b;
            ++j;
            b = (j < n1) ? l1[j] : INT_MAX;
        }
    }
    counts[idx] = min(n, list_stride);
    if (!sorted) atomicMax(unsorted, 1);
}

}  // namespace aa

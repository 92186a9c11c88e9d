// Step 2: difference-aware stripe identification.
//
// Replaces get_q_mask_triton (reference: anchor_attn/src/ops/get_mask_test.py:7-124).
// Three kernels:
//   pool_kernel     block-mean queries (bf16 running sum in the reference's add
//                   order) and block-mean anchors                       (this file)
//   score_tc_kernel pooled rows against the key columns on the tensor cores; emits
//                   one hit bit per (query head, big block, column)     (score_tc.cuh)
//   compact_kernel  ordered compaction of the hit bitmap into ascending id lists
//                                                                       (this file)
#pragma once
#include "common.cuh"

namespace aa {

// ---------------------------------------------------------------------------
// pool_kernel: grid (N/BS, H, B), 64 threads; thread t owns columns 2t, 2t+1.  BS = pooling
// block size (64, 128 or 256 rows).
// The rows are summed in bf16 in this order (for BS = 128 the one the reference's compiled
// reduction uses): rows 32w..32w+31 form group w and are reduced by halving
// (i + 16, i + 8, i + 4, i + 2, i + 1); the BS/32 group sums are combined by halving as well
// (for four groups: (W0 + W2) + (W1 + W3)).  Division by BS is exact.
// Warp 0 also reduces the BS anchors of the block (fp32, same tree).
// ---------------------------------------------------------------------------
template <int BS>
__global__ void __launch_bounds__(64) pool_kernel(TensorView q, const float* __restrict__ M,
                                                  __nv_bfloat16* __restrict__ qpool, float* __restrict__ apool,
                                                  int H, int N) {
    constexpr int NG = BS / 32;
    const int blk = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int t = threadIdx.x;
    const __nv_bfloat16* src = q.ptr + z * q.sb + h * q.sh + (int64_t)blk * BS * q.sn + 2 * t;
    __nv_bfloat162 w[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
        __nv_bfloat162 x[32];
#pragma unroll
        for (int r = 0; r < 32; ++r)
            x[r] = *reinterpret_cast<const __nv_bfloat162*>(src + (int64_t)(g * 32 + r) * q.sn);
#pragma unroll
        for (int half = 16; half >= 1; half >>= 1)
#pragma unroll
            for (int i = 0; i < half; ++i) x[i] = __hadd2(x[i], x[i + half]);
        w[g] = x[0];
    }
#pragma unroll
    for (int half = NG / 2; half >= 1; half >>= 1)
#pragma unroll
        for (int i = 0; i < half; ++i) w[i] = __hadd2(w[i], w[i + half]);
    float2 f = __bfloat1622float2(w[0]);
    __nv_bfloat162 mean = __floats2bfloat162_rn(f.x / (float)BS, f.y / (float)BS);
    const int64_t prow = ((int64_t)(z * H + h) * (N / BS) + blk);
    *reinterpret_cast<__nv_bfloat162*>(qpool + prow * kD + 2 * t) = mean;

    if (t < 32) {
        const float* m = M + (int64_t)(z * H + h) * N + (int64_t)blk * BS;
        float v[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) v[g] = m[g * 32 + t];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
            for (int g = 0; g < NG; ++g) v[g] = __fadd_rn(v[g], __shfl_xor_sync(0xffffffffu, v[g], off));
#pragma unroll
        for (int half = NG / 2; half >= 1; half >>= 1)
#pragma unroll
            for (int i = 0; i < half; ++i) v[i] = __fadd_rn(v[i], v[i + half]);
        if (t == 0) apool[prow] = bf16_round(v[0] / (float)BS);
    }
}

// ---------------------------------------------------------------------------
// compact_kernel: grid (NB, H, B), 256 threads.  Turns the bitmap row of one
// (head, big block) into an ascending id list and its count.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) compact_kernel(const uint32_t* __restrict__ bitmap, int32_t* __restrict__ ids,
                                                      int32_t* __restrict__ counts, int H, int N, int step,
                                                      int block, int64_t ids_per_head) {
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int NB = N / (block * step);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t hz = (int64_t)z * H + h;
    if (b == 0) {
        if (tid == 0) counts[hz * NB] = 0;
        return;
    }
    const int G = block * step;
    const int nwords = (b * G - 2 * block) / 32;  // candidate columns [block, b*G - block) / 32
    const int w0 = block / 32;                    // first candidate word
    const uint32_t* row = bitmap + (hz * NB + b) * (int64_t)(N / 32);
    const int64_t row_off = (int64_t)G * b * (b - 1) / 2 - 2 * (int64_t)block * (b - 1);
    int32_t* dst = ids + hz * ids_per_head + row_off;
    __shared__ int warp_sums[8];
    __shared__ int base_s;
    if (tid == 0) base_s = 0;
    __syncthreads();
    for (int c0 = 0; c0 < nwords; c0 += 256) {
        const int wi = c0 + tid;
        const uint32_t w = (wi < nwords) ? row[w0 + wi] : 0u;
        const int cnt = __popc(w);
        int incl = cnt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += v;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        int wbase = 0, total = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int s = warp_sums[i];
            if (i < warp) wbase += s;
            total += s;
        }
        // the warp writes its 32 words one after the other: lane i stores bit i of the word,
        // so the ids of a word go out as one contiguous segment
        const int excl = base_s + wbase + incl - cnt;
        const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll 4
        for (int k = 0; k < 32; ++k) {
            const uint32_t wk = __shfl_sync(0xffffffffu, w, k);
            const int ok_ = __shfl_sync(0xffffffffu, excl, k);
            if (wk == 0u) continue;
            if ((wk >> lane) & 1u) dst[ok_ + __popc(wk & lt_mask)] = (w0 + c0 + warp * 32 + k) * 32 + lane;
        }
        __syncthreads();
        if (tid == 0) base_s += total;
        __syncthreads();
    }
    if (tid == 0) counts[hz * NB + b] = base_s;
}

}  // namespace aa

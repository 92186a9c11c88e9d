// Step 2: difference-aware stripe identification.
//
// Replaces get_q_mask_triton (reference: anchor_attn/src/ops/get_mask_test.py:7-124).
// Three kernels:
//   pool_kernel     block-mean queries (bf16 running sum in the reference's add
//                   order) and block-mean anchors
//   score_kernel    streams the key columns once per (KV head, big block); the
//                   pooled rows of all query heads of the KV group are compared
//                   against each key tile, so the key stream is shared by the
//                   group.  Emits one hit bit per (query head, big block, column).
//   compact_kernel  ordered compaction of the hit bitmap into ascending id lists.
#pragma once
#include "common.cuh"

namespace aa {

// ---------------------------------------------------------------------------
// pool_kernel: grid (N/128, H, B), 64 threads; thread t owns columns 2t, 2t+1.
// The 128 rows are summed in bf16 in this order (the one the reference's compiled
// reduction uses): rows 32w..32w+31 form group w and are reduced by halving
// (i + 16, i + 8, i + 4, i + 2, i + 1); the four group sums are combined as
// (W0 + W2) + (W1 + W3).  Division by 128 is exact.
// Warp 0 also reduces the 128 anchors of the block (fp32, same tree).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(64) pool_kernel(TensorView q, const float* __restrict__ M,
                                                  __nv_bfloat16* __restrict__ qpool, float* __restrict__ apool,
                                                  int H, int N) {
    const int blk = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int t = threadIdx.x;
    const __nv_bfloat16* src = q.ptr + z * q.sb + h * q.sh + (int64_t)blk * 128 * q.sn + 2 * t;
    __nv_bfloat162 w[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
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
    __nv_bfloat162 s = __hadd2(__hadd2(w[0], w[2]), __hadd2(w[1], w[3]));
    float2 f = __bfloat1622float2(s);
    __nv_bfloat162 mean = __floats2bfloat162_rn(f.x / 128.0f, f.y / 128.0f);
    const int64_t prow = ((int64_t)(z * H + h) * (N / 128) + blk);
    *reinterpret_cast<__nv_bfloat162*>(qpool + prow * kD + 2 * t) = mean;

    if (t < 32) {
        const float* m = M + (int64_t)(z * H + h) * N + (int64_t)blk * 128;
        float v[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) v[g] = m[g * 32 + t];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
            for (int g = 0; g < 4; ++g) v[g] = __fadd_rn(v[g], __shfl_xor_sync(0xffffffffu, v[g], off));
        float a = __fadd_rn(__fadd_rn(v[0], v[2]), __fadd_rn(v[1], v[3]));
        if (t == 0) apool[prow] = bf16_round(a / 128.0f);
    }
}

// ---------------------------------------------------------------------------
// score_kernel
//   grid  (ceil(max_tiles / kTilesPerCta), NB - 1, B * Hkv), 128 threads.
//   CTA (c, b-1, z*Hkv+kvh) handles key tiles t = 1 + c*kTilesPerCta ... of big
//   block b (tile t = columns [128 t, 128 t + 128)); candidates of big block b
//   are tiles 1 .. b*step - 2  (get_mask_test.py:93-94).
//   Warp w owns columns 32 w .. 32 w + 31 of each tile and all pooled rows.
//   score = bf16(dot * fp32(sm_scale * log2e)); hit = fp32(score) + diff >= anchor.
//   bitmap[(z,h,b)][col / 32] bit (col % 32).
// Dynamic shared memory: pooled queries of the group (Hg * step rows) then two
// key tiles of 32 KB.
// ---------------------------------------------------------------------------
constexpr int kTilesPerCta = 8;

__global__ void __launch_bounds__(128) score_kernel(TensorView k, const __nv_bfloat16* __restrict__ qpool,
                                                    const float* __restrict__ apool, uint32_t* __restrict__ bitmap,
                                                    int H, int Hkv, int N, int step, float qk_scale, float diff) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int b = blockIdx.y + 1;
    const int z = blockIdx.z / Hkv, kvh = blockIdx.z % Hkv;
    const int Hg = H / Hkv;
    const int ntiles = b * step - 2;
    const int t_begin = 1 + blockIdx.x * kTilesPerCta;
    if (t_begin > ntiles) return;
    const int t_end = min(t_begin + kTilesPerCta, ntiles + 1);   // exclusive
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NB = N / (128 * step);
    const int prow_per_head = N / 128;

    uint8_t* sq = smem;                                  // [Hg*step][128] bf16, swizzled
    const int qrows = Hg * step;
    uint8_t* sk = smem + (size_t)qrows * kRowBytes;      // 2 x [128][128] bf16, swizzled
    const uint32_t sq_u = smem_u32(sq), sk_u = smem_u32(sk);

    // pooled queries of the group -> shared
    for (int c = tid; c < qrows * 16; c += 128) {
        const int r = c >> 4, ch = c & 15;
        const int g = r / step, j = r % step;
        const int64_t prow = (int64_t)(z * H + kvh * Hg + g) * prow_per_head + b * step + j;
        cp_async16(sq_u + tile_off(r, ch), qpool + prow * kD + ch * 8, 16);
    }
    const __nv_bfloat16* kbase = k.ptr + z * k.sb + kvh * k.sh;
    auto load_tile = [&](int t, int buf) {
        const uint32_t dst = sk_u + buf * (128 * kRowBytes);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int c = tid + i * 128;
            const int r = c >> 4, ch = c & 15;
            cp_async16(dst + tile_off(r, ch), kbase + (int64_t)(t * 128 + r) * k.sn + ch * 8, 16);
        }
    };
    load_tile(t_begin, 0);
    cp_async_commit();

    const int words_per_row = N / 32;
    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) & 1;
        if (t + 1 < t_end) {
            load_tile(t + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        // B fragments of this warp's 32 columns: [kstep][ntile][2]
        uint32_t bfr[8][4][2];
        const uint32_t kt = sk_u + buf * (128 * kRowBytes);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                const int row = warp * 32 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int ch = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(kt + tile_off(row, ch), bfr[ks][np * 2][0], bfr[ks][np * 2][1], bfr[ks][np * 2 + 1][0],
                            bfr[ks][np * 2 + 1][1]);
            }

        for (int g = 0; g < Hg; ++g) {
            uint32_t word = 0;
            const int h = kvh * Hg + g;
            for (int mt = 0; mt < step / 16; ++mt) {
                float acc[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
                const int arow0 = g * step + mt * 16;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    uint32_t a[4];
                    const int row = arow0 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    const int ch = ks * 2 + (lane >> 4);
                    ldmatrix_x4(sq_u + tile_off(row, ch), a[0], a[1], a[2], a[3]);
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) mma_bf16_16816(acc[nt], a, bfr[ks][nt][0], bfr[ks][nt][1]);
                }
                const int64_t prow = (int64_t)(z * H + h) * prow_per_head + b * step + mt * 16 + (lane >> 2);
                const float a0 = apool[prow], a1 = apool[prow + 8];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float sc = bf16_round(__fmul_rn(acc[nt][j], qk_scale));
                        const bool hit = __fadd_rn(sc, diff) >= ((j < 2) ? a0 : a1);
                        if (hit) word |= 1u << (nt * 8 + (lane & 3) * 2 + (j & 1));
                    }
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) word |= __shfl_xor_sync(0xffffffffu, word, off);
            if (lane == 0)
                bitmap[((int64_t)(z * H + h) * NB + b) * words_per_row + t * 4 + warp] = word;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// compact_kernel: grid (NB, H, B), 256 threads.  Turns the bitmap row of one
// (head, big block) into an ascending id list and its count.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) compact_kernel(const uint32_t* __restrict__ bitmap, int32_t* __restrict__ ids,
                                                      int32_t* __restrict__ counts, int H, int N, int step,
                                                      int64_t ids_per_head) {
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int NB = N / (128 * step);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t hz = (int64_t)z * H + h;
    if (b == 0) {
        if (tid == 0) counts[hz * NB] = 0;
        return;
    }
    const int nwords = (b * step - 2) * 4;        // candidate columns / 32
    const int w0 = 4;                             // first candidate word (column 128)
    const uint32_t* row = bitmap + (hz * NB + b) * (int64_t)(N / 32);
    const int G = 128 * step;
    const int64_t row_off = (int64_t)G * b * (b - 1) / 2 - 256 * (int64_t)(b - 1);
    int32_t* dst = ids + hz * ids_per_head + row_off;
    __shared__ int warp_sums[8];
    __shared__ int base_s;
    if (tid == 0) base_s = 0;
    __syncthreads();
    for (int c0 = 0; c0 < nwords; c0 += 256) {
        const int wi = c0 + tid;
        uint32_t w = (wi < nwords) ? row[w0 + wi] : 0u;
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
        int pos = base_s + wbase + incl - cnt;
        const int col0 = (w0 + wi) * 32;
        while (w) {
            const int bit = __ffs(w) - 1;
            dst[pos++] = col0 + bit;
            w &= w - 1;
        }
        __syncthreads();
        if (tid == 0) base_s += total;
        __syncthreads();
    }
    if (tid == 0) counts[hz * NB + b] = base_s;
}

}  // namespace aa

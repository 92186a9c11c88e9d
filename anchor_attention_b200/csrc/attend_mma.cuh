// Steps 1 and 3 as one flash-attention kernel over a list of key rows.
//
//   kWindow  (step 1) rows come from contiguous 64-row tiles of the window
//            [0, min(G, (qb+1)*128)) U [max(b*G, that), (qb+1)*128), causal mask as an
//            additive -1e6, query scaled with dtype-rounded constants; writes
//            M, L and the un-normalised accumulator.
//            Reference: anchor_attn/src/ops/anchor_step_1_2_v2.py:8-161.
//   kStripe  (step 3) rows are gathered through the big block's id list, the
//            running state starts from step 1's (M, L, Acc), slots past the count are
//            masked to -inf; writes bf16(acc / l).
//            Reference: anchor_attn/src/ops/anchor_attn_v4.py:7-105.
//
// One CTA = 128 query rows, 8 warps of 16 rows, key tiles of 64 rows moved with
// 16-byte cp.async (a row is 256 contiguous bytes whether gathered or not),
// double buffered.  Tensor-core work uses mma.sync m16n8k16.
#pragma once
#include "common.cuh"

namespace aa {

enum AttendMode { kWindow = 0, kStripe = 1 };

constexpr int kQRows = 128;      // query rows per CTA
constexpr int kKvTile = 64;      // key rows per pipeline stage
constexpr int kAttendThreads = 256;
constexpr int kAttendSmem = kQRows * kRowBytes + 2 * 2 * kKvTile * kRowBytes;   // Q + 2 stages x (K, V)

struct AttendArgs {
    TensorView q, k, v;
    __nv_bfloat16* out;
    int64_t osb, osh, osn;
    float* M;
    float* L;
    float* Acc;
    const int32_t* counts;
    const int32_t* ids;
    int64_t ids_per_head;
    int B, H, Hkv, N, step;
    float sm_scale;
};

template <int MODE>
__global__ void __launch_bounds__(kAttendThreads, 1) attend_mma_kernel(AttendArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int BH = a.B * a.H;
    const int nqb = a.N / kQRows;
    // heaviest query blocks first
    const int qb = nqb - 1 - (int)(blockIdx.x / BH);
    const int hz = blockIdx.x % BH;
    const int z = hz / a.H, h = hz % a.H;
    const int kvh = h / (a.H / a.Hkv);
    const int G = 128 * a.step;
    const int b = (qb * kQRows) / G;
    const int NB = a.N / G;

    const uint32_t sq_u = smem_u32(smem);
    const uint32_t skv_u = sq_u + kQRows * kRowBytes;   // stage s holds a K tile then a V tile
    auto k_stage = [&](int s) { return skv_u + s * (2 * kKvTile * kRowBytes); };
    auto v_stage = [&](int s) { return skv_u + s * (2 * kKvTile * kRowBytes) + kKvTile * kRowBytes; };

    // ---- tile list ----
    int ntiles, n_init = 0, local_start = 0, count = 0;
    const int32_t* idp = nullptr;
    if (MODE == kWindow) {
        const int init_end = min(G, (qb + 1) * kQRows);
        local_start = max(b * G, init_end);
        n_init = init_end / kKvTile;
        ntiles = n_init + ((qb + 1) * kQRows - local_start) / kKvTile;
    } else {
        count = a.counts[(int64_t)hz * NB + b];
        ntiles = (count + kKvTile - 1) / kKvTile;
        const int64_t row_off = (b == 0) ? 0 : ((int64_t)G * b * (b - 1) / 2 - 256 * (int64_t)(b - 1));
        idp = a.ids + (int64_t)hz * a.ids_per_head + row_off;
    }

    const __nv_bfloat16* kbase = a.k.ptr + z * a.k.sb + kvh * a.k.sh;
    const __nv_bfloat16* vbase = a.v.ptr + z * a.v.sb + kvh * a.v.sh;
    auto load_tile = [&](int t, int s) {
        const uint32_t kd = k_stage(s), vd = v_stage(s);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = tid + i * kAttendThreads;
            const int r = c >> 4, ch = c & 15;
            int64_t row;
            int bytes = 16;
            if (MODE == kWindow) {
                row = (t < n_init) ? (t * kKvTile + r) : (local_start + (t - n_init) * kKvTile + r);
            } else {
                const int slot = t * kKvTile + r;
                if (slot < count) {
                    row = idp[slot];
                } else {
                    row = 0;
                    bytes = 0;
                }
            }
            cp_async16(kd + tile_off(r, ch), kbase + row * a.k.sn + ch * 8, bytes);
            cp_async16(vd + tile_off(r, ch), vbase + row * a.v.sn + ch * 8, bytes);
        }
    };

    if (ntiles > 0) load_tile(0, 0);
    cp_async_commit();

    // ---- Q tile: load, scale, round, park in shared, then keep A fragments in registers ----
    {
        const __nv_bfloat16* qbase = a.q.ptr + z * a.q.sb + h * a.q.sh + (int64_t)qb * kQRows * a.q.sn;
        const float c1 = bf16_round(a.sm_scale), c2 = bf16_round(kLog2e);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = tid + i * kAttendThreads;
            const int r = c >> 4, ch = c & 15;
            uint4 raw = *reinterpret_cast<const uint4*>(qbase + (int64_t)r * a.q.sn + ch * 8);
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __bfloat1622float2(p2[j]);
                if (MODE == kWindow) {
                    f.x = bf16_round(__fmul_rn(bf16_round(__fmul_rn(f.x, c1)), c2));
                    f.y = bf16_round(__fmul_rn(bf16_round(__fmul_rn(f.y, c1)), c2));
                } else {
                    f.x = __fmul_rn(__fmul_rn(f.x, a.sm_scale), kLog2e);
                    f.y = __fmul_rn(__fmul_rn(f.y, a.sm_scale), kLog2e);
                }
                p2[j] = __floats2bfloat162_rn(f.x, f.y);
            }
            *reinterpret_cast<uint4*>(smem + tile_off(r, ch)) = raw;
        }
    }
    __syncthreads();
    uint32_t qf[8][4];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int ch = ks * 2 + (lane >> 4);
        ldmatrix_x4(sq_u + tile_off(row, ch), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    // ---- running state; this thread owns rows r0 and r0 + 8 of its warp's 16 ----
    const int r0 = qb * kQRows + warp * 16 + (lane >> 2);
    const int64_t srow = (int64_t)hz * a.N + r0;
    float o[16][4];
    float m_i[2], l_i[2];
    if (MODE == kWindow) {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        m_i[0] = m_i[1] = -INFINITY;
        l_i[0] = l_i[1] = 0.f;
    } else {
        m_i[0] = a.M[srow];
        m_i[1] = a.M[srow + 8];
        // the row sum is accumulated per thread and reduced over the quad at the end
        l_i[0] = ((lane & 3) == 0) ? a.L[srow] : 0.f;
        l_i[1] = ((lane & 3) == 0) ? a.L[srow + 8] : 0.f;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            const float2 x = *reinterpret_cast<const float2*>(a.Acc + srow * kD + nt * 8 + (lane & 3) * 2);
            const float2 y = *reinterpret_cast<const float2*>(a.Acc + (srow + 8) * kD + nt * 8 + (lane & 3) * 2);
            o[nt][0] = x.x; o[nt][1] = x.y; o[nt][2] = y.x; o[nt][3] = y.y;
        }
    }

    for (int t = 0; t < ntiles; ++t) {
        const int s = t & 1;
        if (t + 1 < ntiles) {
            load_tile(t + 1, s ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        // S = Q K^T for 16 rows x 64 key rows
        float sc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
        const uint32_t kt = k_stage(s);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b0, b1, b2, b3;
                const int row = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int ch = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(kt + tile_off(row, ch), b0, b1, b2, b3);
                mma_bf16_16816(sc[np * 2], qf[ks], b0, b1);
                mma_bf16_16816(sc[np * 2 + 1], qf[ks], b2, b3);
            }

        // masks
        if (MODE == kWindow) {
            const int col0 = (t < n_init) ? t * kKvTile : local_start + (t - n_init) * kKvTile;
            if (col0 + kKvTile - 1 > qb * kQRows + warp * 16) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int col = col0 + nt * 8 + (lane & 3) * 2 + (j & 1);
                        const int row = r0 + ((j >> 1) << 3);
                        if (col > row) sc[nt][j] += -1e6f;
                    }
            }
        } else {
            const int valid = count - t * kKvTile;
            if (valid < kKvTile) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (nt * 8 + (lane & 3) * 2 + (j & 1) >= valid) sc[nt][j] = -INFINITY;
            }
        }

        // online softmax
        float mx[2] = {m_i[0], m_i[1]};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            mx[0] = fmaxf(mx[0], fmaxf(sc[nt][0], sc[nt][1]));
            mx[1] = fmaxf(mx[1], fmaxf(sc[nt][2], sc[nt][3]));
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        }
        const float alpha0 = fast_exp2(m_i[0] - mx[0]), alpha1 = fast_exp2(m_i[1] - mx[1]);
        m_i[0] = mx[0];
        m_i[1] = mx[1];
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t pf[4][4];   // P as A fragments for the four 16-row k-steps
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float p0 = fast_exp2(sc[nt][0] - mx[0]), p1 = fast_exp2(sc[nt][1] - mx[0]);
            const float p2 = fast_exp2(sc[nt][2] - mx[1]), p3 = fast_exp2(sc[nt][3] - mx[1]);
            rs0 += p0 + p1;
            rs1 += p2 + p3;
            pf[nt >> 1][(nt & 1) * 2] = pack_bf16x2(p0, p1);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
        }
        l_i[0] = l_i[0] * alpha0 + rs0;
        l_i[1] = l_i[1] * alpha1 + rs1;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            o[nt][0] *= alpha0; o[nt][1] *= alpha0;
            o[nt][2] *= alpha1; o[nt][3] *= alpha1;
        }

        // O += P V
        const uint32_t vt = v_stage(s);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {
                uint32_t b0, b1, b2, b3;
                const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                const int ch = dp * 2 + (lane >> 4);
                ldmatrix_x4_trans(vt + tile_off(row, ch), b0, b1, b2, b3);
                mma_bf16_16816(o[dp * 2], pf[kk], b0, b1);
                mma_bf16_16816(o[dp * 2 + 1], pf[kk], b2, b3);
            }
        __syncthreads();
    }

    // ---- epilogue ----
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_i[i] += __shfl_xor_sync(0xffffffffu, l_i[i], 1);
        l_i[i] += __shfl_xor_sync(0xffffffffu, l_i[i], 2);
    }
    if (MODE == kWindow) {
        if ((lane & 3) == 0) {
            a.M[srow] = m_i[0];
            a.M[srow + 8] = m_i[1];
            a.L[srow] = l_i[0];
            a.L[srow + 8] = l_i[1];
        }
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            *reinterpret_cast<float2*>(a.Acc + srow * kD + nt * 8 + (lane & 3) * 2) = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(a.Acc + (srow + 8) * kD + nt * 8 + (lane & 3) * 2) =
                make_float2(o[nt][2], o[nt][3]);
        }
    } else {
        __nv_bfloat16* ob = a.out + z * a.osb + h * a.osh;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            const int col = nt * 8 + (lane & 3) * 2;
            *reinterpret_cast<uint32_t*>(ob + (int64_t)r0 * a.osn + col) =
                pack_bf16x2(__fdiv_rn(o[nt][0], l_i[0]), __fdiv_rn(o[nt][1], l_i[0]));
            *reinterpret_cast<uint32_t*>(ob + (int64_t)(r0 + 8) * a.osn + col) =
                pack_bf16x2(__fdiv_rn(o[nt][2], l_i[1]), __fdiv_rn(o[nt][3], l_i[1]));
        }
    }
}

}  // namespace aa

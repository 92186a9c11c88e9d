// Tokens -> heads exchange of a sequence-parallel prefill, fused with the rotary embedding.
//
// A rank holds the q/k/v projections of ITS tokens for ALL heads; attention needs, on every rank,
// the rotated q/k and v of ALL tokens for ITS heads.  The reference applies the rotary embedding
// and reorders on one GPU (anchor_attn/src/modules/llama/anchor_attention.py:38-48, 89-91:
// apply_rotary_pos_emb, then transposes and copies).  Here one kernel reads each projection row
// once, rotates q and k, and stores the row straight into the buffer of the rank that owns its
// head -- plain 8-byte stores, coalesced to 128-byte segments, over NVLink for remote owners -- so
// no separate rotary kernels, no packing copy and no all-to-all collective run.  A flag barrier
// (peer_barrier.cuh) follows.
//
// Arithmetic is that of the rotate-half formulation on bf16 tensors, rounding included:
//   out = bf16( bf16(x * cos) + bf16(rotate_half(x) * sin) ),  rotate_half(x) = [-x[64:], x[:64]].
//
// Destination layout on every rank: [N tokens, h + 2*hkv heads, 128] bf16, token-major: the rank's
// h query heads, then its hkv key heads, then its hkv value heads (what an all-to-all of packed
// rows would deliver); the attention kernels read q, k and v out of it through their strides.
#pragma once
#include "common.cuh"

namespace aa {

constexpr int kRopeMaxPeers = 8;

struct RopeDispatchArgs {
    const __nv_bfloat16 *q, *k, *v;      // [n, H, 128], [n, Hkv, 128], [n, Hkv, 128]: this rank's tokens
    int64_t q_sn, k_sn, v_sn;            // row (token) strides in elements; heads are 128 apart
    const __nv_bfloat16 *cos, *sin;      // [n, 128]
    __nv_bfloat16* dst[kRopeMaxPeers];   // rank d's [N, h + 2 hkv, 128] buffer
    int n, H, Hkv, n_peers;
    int token0;                          // global position of this rank's first token
};

// grid ceil(n / 16), 256 threads: 16 threads per token, looping over the token's heads; thread c
// owns elements 4c..4c+3 and 64+4c..64+4c+3 of every head row.
__global__ void __launch_bounds__(256) rope_dispatch_kernel(RopeDispatchArgs a) {
    const int c = threadIdx.x & 15;
    const int tok = blockIdx.x * 16 + (threadIdx.x >> 4);
    if (tok >= a.n) return;
    const int h = a.H / a.n_peers, hkv = a.Hkv / a.n_peers, width = h + 2 * hkv;
    const uint2 cs_lo = *reinterpret_cast<const uint2*>(a.cos + (int64_t)tok * kD + 4 * c);
    const uint2 cs_hi = *reinterpret_cast<const uint2*>(a.cos + (int64_t)tok * kD + 64 + 4 * c);
    const uint2 sn_lo = *reinterpret_cast<const uint2*>(a.sin + (int64_t)tok * kD + 4 * c);
    const uint2 sn_hi = *reinterpret_cast<const uint2*>(a.sin + (int64_t)tok * kD + 64 + 4 * c);
    auto rot = [&](uint2 lo, uint2 hi, uint2& out_lo, uint2& out_hi) {
        const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi);
        const __nv_bfloat162* cl = reinterpret_cast<const __nv_bfloat162*>(&cs_lo);
        const __nv_bfloat162* ch = reinterpret_cast<const __nv_bfloat162*>(&cs_hi);
        const __nv_bfloat162* sl = reinterpret_cast<const __nv_bfloat162*>(&sn_lo);
        const __nv_bfloat162* sh = reinterpret_cast<const __nv_bfloat162*>(&sn_hi);
        __nv_bfloat162* ol = reinterpret_cast<__nv_bfloat162*>(&out_lo);
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out_hi);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            // each bf16 product and sum is rounded on its own: the _rn forms are never contracted
            // into a fused multiply-add, which would skip the rounding of the product
            ol[e] = __hadd2_rn(__hmul2_rn(l2[e], cl[e]), __hmul2_rn(__hneg2(h2[e]), sl[e]));
            oh[e] = __hadd2_rn(__hmul2_rn(h2[e], ch[e]), __hmul2_rn(l2[e], sh[e]));
        }
    };
    const int64_t drow = (int64_t)(a.token0 + tok) * width * kD;
#pragma unroll 4
    for (int hd = 0; hd < a.H; ++hd) {
        const __nv_bfloat16* src = a.q + (int64_t)tok * a.q_sn + hd * kD;
        uint2 lo = *reinterpret_cast<const uint2*>(src + 4 * c), hi = *reinterpret_cast<const uint2*>(src + 64 + 4 * c);
        uint2 ol, oh;
        rot(lo, hi, ol, oh);
        __nv_bfloat16* d = a.dst[hd / h] + drow + (hd % h) * kD;
        *reinterpret_cast<uint2*>(d + 4 * c) = ol;
        *reinterpret_cast<uint2*>(d + 64 + 4 * c) = oh;
    }
    for (int hd = 0; hd < a.Hkv; ++hd) {
        const __nv_bfloat16* src = a.k + (int64_t)tok * a.k_sn + hd * kD;
        uint2 lo = *reinterpret_cast<const uint2*>(src + 4 * c), hi = *reinterpret_cast<const uint2*>(src + 64 + 4 * c);
        uint2 ol, oh;
        rot(lo, hi, ol, oh);
        __nv_bfloat16* d = a.dst[hd / hkv] + drow + (h + hd % hkv) * kD;
        *reinterpret_cast<uint2*>(d + 4 * c) = ol;
        *reinterpret_cast<uint2*>(d + 64 + 4 * c) = oh;
        const __nv_bfloat16* vs = a.v + (int64_t)tok * a.v_sn + hd * kD;
        __nv_bfloat16* dv = a.dst[hd / hkv] + drow + (h + hkv + hd % hkv) * kD;
        *reinterpret_cast<uint2*>(dv + 4 * c) = *reinterpret_cast<const uint2*>(vs + 4 * c);
        *reinterpret_cast<uint2*>(dv + 64 + 4 * c) = *reinterpret_cast<const uint2*>(vs + 64 + 4 * c);
    }
}

}  // namespace aa

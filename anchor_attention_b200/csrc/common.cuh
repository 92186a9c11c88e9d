// Shared device helpers: bf16 rounding, cp.async, fast exp2, the argument structs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace aa {

constexpr float kLog2e = 1.44269504f;   // the literal the reference kernels use
constexpr int kD = 128;                  // head dimension the kernels are written for
constexpr int kRowBytes = kD * 2;        // one bf16 K/V/Q row

struct TensorView {          // one [B, heads, N, 128] bf16 tensor, strides in elements
    const __nv_bfloat16* ptr;
    int64_t sb, sh, sn;
};

// Which attention pass a kernel instance runs: the operator's two passes, or the
// block-granular comparator (whole 128-row key blocks from a per-query-block list).
enum AttendMode { kWindow = 0, kStripe = 1, kBlock = 2 };

// kBlock tile-list entries: key block index in the low bits, one flag per query tile of the pair.
constexpr uint32_t kBlockIdMask = 0x00FFFFFFu;
constexpr int kBlockFlagShift = 30;       // bit 30: first query tile attends the block, bit 31: second

// Arguments shared by both passes: the tensors, the inter-kernel state in the
// workspace and the problem sizes.
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
    int B, H, Hkv, N, step, block;      // block = pooling block size (64, 128 or 256); big block G = block * step
    float sm_scale;
};

__device__ __forceinline__ float bf16_round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous copy global -> shared; src_bytes == 0 zero-fills.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

}  // namespace aa

// C ABI of the anchor-attention operator: argument checks, workspace layout and
// kernel launches.  Declarations and the reference functions each entry point
// replaces are in include/anchor_attn_b200.h.
#include "../../include/anchor_attn_b200.h"

#include <stdio.h>
#include <math.h>
#include <mutex>
#include <stdlib.h>
#include <string.h>

#include "attend_tc.cuh"
#include "attend_persist.cuh"
#include "block_list.cuh"
#include "common.cuh"
#include "gather.cuh"
#include "peer_barrier.cuh"
#include "rope_dispatch.cuh"
#include "score_tc.cuh"
#include "stripe.cuh"

namespace {

thread_local char g_cuda_err[256] = "";

int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
    return AA_ERR_CUDA;
}

size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

int check_shape(const aa_params_t* p) {
    if (!p) return AA_ERR_NULL;
    if (p->B <= 0 || p->H <= 0 || p->Hkv <= 0 || p->N <= 0 || p->H % p->Hkv != 0) return AA_ERR_SHAPE;
    if (p->D != 128) return AA_ERR_HEAD_DIM;
    if (p->step != 16 && p->step != 32) return AA_ERR_STEP;
    if (p->block_size != 64 && p->block_size != 128 && p->block_size != 256) return AA_ERR_BLOCK;
    if (p->N % (p->block_size * p->step) != 0) return AA_ERR_SEQ;
    if (p->dtype != AA_BF16) return AA_ERR_DTYPE;
    if ((int64_t)p->N * p->H * p->B > (int64_t)1 << 40) return AA_ERR_TOO_LARGE;
    return AA_OK;
}

bool stride_ok(int64_t s) { return s % 8 == 0; }

int check_full(const aa_params_t* p, aa_workspace_layout_t* lay) {
    int rc = check_shape(p);
    if (rc) return rc;
    if (!p->q || !p->k || !p->v || !p->out) return AA_ERR_NULL;
    const int64_t st[] = {p->q_stride_b, p->q_stride_h, p->q_stride_n, p->k_stride_b, p->k_stride_h, p->k_stride_n,
                          p->v_stride_b, p->v_stride_h, p->v_stride_n, p->o_stride_b, p->o_stride_h, p->o_stride_n};
    for (int64_t s : st)
        if (!stride_ok(s)) return AA_ERR_STRIDE;
    if (((uintptr_t)p->q | (uintptr_t)p->k | (uintptr_t)p->v | (uintptr_t)p->out) & 15) return AA_ERR_STRIDE;
    rc = aa_workspace_layout(p, lay);
    if (rc) return rc;
    if (!p->workspace || ((uintptr_t)p->workspace & 255) || p->workspace_bytes < lay->min_bytes)
        return AA_ERR_WORKSPACE;
    return AA_OK;
}

// How step 3 is laid out for a problem and workspace: whether there is a gather pass at all, whether
// the scratch may be too small for the lists (then the device decides between one go and parts), and how
// many KV heads one part takes.
struct Step3Layout {
    int n_slots, kv_total, kv_per_part;
    bool gather, may_overflow;
};
int gather_slots(const aa_params_t* p, const aa_workspace_layout_t& lay);
Step3Layout step3_layout(const aa_params_t* p, const aa_workspace_layout_t& lay) {
    Step3Layout s;
    s.n_slots = gather_slots(p, lay);
    const int NB = p->N / (p->block_size * p->step);
    const int64_t tiles_per_kv = (int64_t)(p->H / p->Hkv) * (lay.ids_per_head / aa::tc::kTile);
    s.kv_total = p->B * p->Hkv;
    s.gather = s.n_slots > 0 && NB > 1;
    s.may_overflow = s.gather && s.kv_total > 1 && (int64_t)s.n_slots < tiles_per_kv * s.kv_total;
    s.kv_per_part = s.kv_total;
    if (s.may_overflow) {
        s.kv_per_part = (int)(s.n_slots / tiles_per_kv);
        if (s.kv_per_part < 1) s.kv_per_part = 1;
    }
    return s;
}

// 64 KB gather slots the caller's workspace holds beyond the mandatory sections
int gather_slots(const aa_params_t* p, const aa_workspace_layout_t& lay) {
    const size_t have = (p->workspace_bytes - lay.gather_off) / (2 * (size_t)aa::tc::kTileBytes);
    const size_t all = (size_t)p->B * p->H * (size_t)(lay.ids_per_head / aa::tc::kTile);
    const size_t n = have < all ? have : all;
    return (int)(n < (size_t)0x7FFFFFFF ? n : (size_t)0x7FFFFFFF);
}

aa::TensorView view(const void* ptr, int64_t sb, int64_t sh, int64_t sn) {
    return aa::TensorView{static_cast<const __nv_bfloat16*>(ptr), sb, sh, sn};
}

double scale_of(const aa_params_t* p) { return p->sm_scale != 0.0 ? p->sm_scale : 1.0 / sqrt((double)p->D); }

template <typename T>
T* ws_ptr(const aa_params_t* p, size_t off) {
    return reinterpret_cast<T*>(static_cast<uint8_t*>(p->workspace) + off);
}

aa::AttendArgs attend_args(const aa_params_t* p, const aa_workspace_layout_t& lay) {
    aa::AttendArgs a;
    a.q = view(p->q, p->q_stride_b, p->q_stride_h, p->q_stride_n);
    a.k = view(p->k, p->k_stride_b, p->k_stride_h, p->k_stride_n);
    a.v = view(p->v, p->v_stride_b, p->v_stride_h, p->v_stride_n);
    a.out = static_cast<__nv_bfloat16*>(p->out);
    a.osb = p->o_stride_b;
    a.osh = p->o_stride_h;
    a.osn = p->o_stride_n;
    a.M = ws_ptr<float>(p, lay.m_off);
    a.L = ws_ptr<float>(p, lay.l_off);
    a.Acc = ws_ptr<float>(p, lay.acc_off);
    a.counts = ws_ptr<int32_t>(p, lay.counts_off);
    a.ids = ws_ptr<int32_t>(p, lay.ids_off);
    a.ids_per_head = lay.ids_per_head;
    a.B = p->B;
    a.H = p->H;
    a.Hkv = p->Hkv;
    a.N = p->N;
    a.step = p->step;
    a.block = p->block_size;
    a.sm_scale = (float)scale_of(p);
    return a;
}

int clear_status(const aa_params_t* p, const aa_workspace_layout_t& lay, cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(ws_ptr<int32_t>(p, lay.status_off), 0, 4 * sizeof(int32_t), st);
    return e == cudaSuccess ? AA_OK : cuda_fail(e, "cudaMemsetAsync(status)");
}

// ---- tensor maps for the TMA tile loads of K and V ----------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// A [B, heads, N, 128] bf16 tensor with arbitrary (16-byte multiple) strides as a 4-D
// tensor map: dimension 0 is the head dimension, the other three are ordered by
// increasing stride; pos_* tell the kernel which coordinate carries n / head / batch.
// Box: 64 elements x 128 rows, 128-byte swizzle.
int make_kv_map(CUtensorMap* map, const void* ptr, int64_t sb, int64_t sh, int64_t sn, int B, int heads, int N,
                int* pos_n, int* pos_h, int* pos_b) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) {
        snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled entry point not found");
        return AA_ERR_CUDA;
    }
    struct Dim { int64_t stride; uint64_t size; int which; };   // which: 0 = n, 1 = head, 2 = batch
    Dim d[3] = {{sn, (uint64_t)N, 0}, {sh, (uint64_t)heads, 1}, {sb, (uint64_t)B, 2}};
    // size-1 dimensions go last (their stride is irrelevant); otherwise sort by stride
    for (int i = 0; i < 3; ++i)
        for (int j = i + 1; j < 3; ++j) {
            const bool swap = (d[i].size == 1 && d[j].size != 1) ||
                              (!(d[j].size == 1 && d[i].size != 1) && d[j].stride < d[i].stride);
            if (swap) { Dim t = d[i]; d[i] = d[j]; d[j] = t; }
        }
    cuuint64_t gdim[4] = {128, d[0].size, d[1].size, d[2].size};
    cuuint64_t gstr[3];
    for (int i = 0; i < 3; ++i) {
        int64_t st = d[i].stride;
        if (d[i].size == 1) st = (i == 0) ? 128 : (int64_t)(gstr[i - 1] / 2 * gdim[i]);   // any legal value
        gstr[i] = (cuuint64_t)st * 2;
    }
    cuuint32_t box[4] = {64, 128, 1, 1};
    if (d[0].which != 0) {
        // the row dimension is not the innermost of the three: boxes still span 128 rows
        box[1] = 1;
        for (int i = 0; i < 3; ++i)
            if (d[i].which == 0) box[1 + i] = 128;
    }
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return AA_ERR_CUDA;
    }
    for (int i = 0; i < 3; ++i) {
        if (d[i].which == 0) *pos_n = i;
        if (d[i].which == 1) *pos_h = i;
        if (d[i].which == 2) *pos_b = i;
    }
    return AA_OK;
}

// The same tensor seen as a 2-D matrix of rows of `sn` elements, for TMA row gathers
// (tile::gather4): box = 64 elements of one row, 128-byte swizzle.  Row id n of (batch z,
// head g) is matrix row (z*sb + g*sh) / sn + n, starting at column (z*sb + g*sh) % sn.
// Possible when every head's 128 columns lie inside one matrix row; *usable says so.
int make_gather_map(CUtensorMap* map, const void* ptr, int64_t sb, int64_t sh, int64_t sn, int B, int heads, int N,
                    int* usable) {
    *usable = 0;
    memset(map, 0, sizeof(*map));
    if (sn < 128 || sb < 0 || sh < 0) return AA_OK;
    int64_t max_row0 = 0;
    for (int z = 0; z < B; ++z)
        for (int g = 0; g < heads; ++g) {
            const int64_t off = (int64_t)z * sb + (int64_t)g * sh;
            if (off % sn + 128 > sn) return AA_OK;
            if (off / sn > max_row0) max_row0 = off / sn;
        }
    const int64_t rows = max_row0 + N;
    if (rows >= ((int64_t)1 << 31) || sn >= ((int64_t)1 << 31)) return AA_OK;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return AA_OK;
    cuuint64_t gdim[2] = {(cuuint64_t)sn, (cuuint64_t)rows};
    cuuint64_t gstr[1] = {(cuuint64_t)sn * 2};
    cuuint32_t box[2] = {64, 1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) *usable = 1;
    return AA_OK;
}

// Dense causal variant of the block mode: the query tensor holds the last q_rows positions of a
// kv_rows-long sequence (p->N is q_rows rounded up to 256 and only sizes the grid).
struct DenseTail {
    int q_rows, kv_rows;
};

template <int MODE>
int launch_attend_tc(const aa_params_t* p, const aa_workspace_layout_t& lay, cudaStream_t st,
                     const aa_push_t* push = nullptr, int list_stride = 0, const DenseTail* dense = nullptr) {
    // per thread and kernel: the device the kernel's shared-memory size was last raised on, and its SM count
    static thread_local int configured_dev = -1;
    static thread_local int sm_count = 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (configured_dev != dev) {
        if (MODE == aa::kBlock) {
            e = cudaFuncSetAttribute(aa::tc::attend_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     aa::tc::kSmemTotal);
        } else {
            constexpr int PM = MODE == aa::kWindow ? aa::kWindow : aa::kStripe;
            e = cudaFuncSetAttribute(aa::tc::attend_persist_kernel<PM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     aa::tc::kSmemTotal);
        }
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(attention kernel)");
        e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(SM count)");
        configured_dev = dev;
    }
    aa::tc::TcArgs ta;
    ta.a = attend_args(p, lay);
    ta.status = ws_ptr<int32_t>(p, lay.status_off);
    ta.n_peers = 0;
    ta.rows_per_peer = 0;
    ta.dense = 0;
    ta.q_rows = p->N;
    ta.q_off = 0;
    ta.kv_blocks = p->N / aa::tc::kTile;
    const int kv_rows = dense ? dense->kv_rows : p->N;
    if (dense) {
        ta.dense = 1;
        ta.q_rows = dense->q_rows;
        ta.q_off = dense->kv_rows - dense->q_rows;
        ta.kv_blocks = (dense->kv_rows + aa::tc::kTile - 1) / aa::tc::kTile;
    }
    ta.tile_slot = nullptr;
    ta.gather = nullptr;
    ta.n_slots = 0;
    ta.list_stride = list_stride;
    for (int i = 0; i < aa::tc::kMaxPeers; ++i) ta.peers[i] = nullptr;
    if (push) {
        ta.n_peers = push->n_peers;
        ta.rows_per_peer = push->rows_per_peer;
        for (int i = 0; i < push->n_peers; ++i) ta.peers[i] = static_cast<__nv_bfloat16*>(push->out[i]);
    }
    CUtensorMap kmap, vmap;
    int rc = make_kv_map(&kmap, p->k, p->k_stride_b, p->k_stride_h, p->k_stride_n, p->B, p->Hkv, kv_rows, &ta.kpos_n,
                         &ta.kpos_h, &ta.kpos_b);
    if (rc) return rc;
    rc = make_kv_map(&vmap, p->v, p->v_stride_b, p->v_stride_h, p->v_stride_n, p->B, p->Hkv, kv_rows, &ta.vpos_n,
                     &ta.vpos_h, &ta.vpos_b);
    if (rc) return rc;
    CUtensorMap kgmap, vgmap;
    ta.k_gather = ta.v_gather = 0;
    if (MODE == aa::kStripe) {
        make_gather_map(&kgmap, p->k, p->k_stride_b, p->k_stride_h, p->k_stride_n, p->B, p->Hkv, p->N, &ta.k_gather);
        make_gather_map(&vgmap, p->v, p->v_stride_b, p->v_stride_h, p->v_stride_n, p->B, p->Hkv, p->N, &ta.v_gather);
    } else {
        memset(&kgmap, 0, sizeof(kgmap));
        memset(&vgmap, 0, sizeof(vgmap));
    }
    const unsigned grid = (unsigned)((int64_t)p->B * p->H * (p->N / (2 * aa::tc::kTile)));
    if (MODE == aa::kBlock) {
        aa::tc::attend_block_kernel<<<grid, aa::tc::kThreads, aa::tc::kSmemTotal, st>>>(kmap, vmap, ta);
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "launch block-sparse (tc)");
        return AA_OK;
    }
    // Steps 1 and 3: one persistent CTA per SM; the query tiles arrive through the ring, so the query
    // tensor needs a tensor map like K and V.  The item counter (status word 3) is zero here: step 1's
    // entry point has just cleared the status words, step 3 cleared it above.
    constexpr int PM = MODE == aa::kWindow ? aa::kWindow : aa::kStripe;
    aa::tc::PersistArgs pa;
    CUtensorMap qmap;
    rc = make_kv_map(&qmap, p->q, p->q_stride_b, p->q_stride_h, p->q_stride_n, p->B, p->H, p->N, &pa.qpos_n, &pa.qpos_h,
                     &pa.qpos_b);
    if (rc) return rc;
    pa.item_counter = ws_ptr<int32_t>(p, lay.status_off) + 3;
    if (MODE == aa::kWindow) {
        pa.n_items = (int)grid;
        const unsigned ctas = grid < (unsigned)sm_count ? grid : (unsigned)sm_count;
        aa::tc::attend_persist_kernel<PM><<<ctas, aa::tc::kThreads, aa::tc::kSmemTotal, st>>>(kmap, vmap, kgmap, vgmap, qmap,
                                                                                            ta, pa);
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "launch step1 (tc)");
        return AA_OK;
    }

    // Step 3 = gather pass (the tiles that are not runs go to the gather scratch once) + attention.
    // When the scratch has a slot for every tile any list COULD have, that is one pass and one launch.
    // Otherwise whether the slots suffice is only known on the device (a tile without a slot is gathered
    // by each of the eight CTAs that read it, at a third of the speed): plan_step3_kernel decides, from the
    // counts, between that same sequence and one that goes KV head by KV head (or several at a time) with
    // the scratch reused; both sequences are launched and the kernels of the other one leave at once.
    // Status words 2 and 3 (slot counter, item counter) are set before each part, word 4 is the plan.
    const Step3Layout s3 = step3_layout(p, lay);
    const int n_slots = s3.n_slots, kv_total = s3.kv_total;
    const bool gather = s3.gather, may_overflow = s3.may_overflow;
    const int NB = p->N / (p->block_size * p->step);
    const int Hg = p->H / p->Hkv;
    const int per_kv = Hg * (p->N / (2 * aa::tc::kTile));
    int32_t* counter = ws_ptr<int32_t>(p, lay.status_off) + 2;
    int32_t* plan = ws_ptr<int32_t>(p, lay.status_off) + 4;
    if (gather) {
        ta.tile_slot = ws_ptr<int32_t>(p, lay.tile_slot_off);
        ta.gather = ws_ptr<uint8_t>(p, lay.gather_off);
        ta.n_slots = n_slots;
    }
    if (may_overflow) {
        aa::plan_step3_kernel<<<1, 256, 0, st>>>(ta.a.counts, p->B * p->H * NB, NB, p->block_size * p->step, p->block_size,
                                                 n_slots, plan);
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "launch step 3 plan");
    }
    // one part: KV heads k0 .. k1 - 1
    auto run_part = [&](int k0, int k1, const int32_t* plan_word, int run_if) -> int {
        // the item counter starts at the part's first item; the kernel draws until it reaches the last
        cudaError_t err = cudaSuccess;
        if (!plan_word && k0 == 0) {
            err = cudaMemsetAsync(counter, 0, 2 * sizeof(int32_t), st);
            if (err != cudaSuccess) return cuda_fail(err, "cudaMemsetAsync(step 3 counters)");
        } else {
            aa::arm_step3_kernel<<<1, 32, 0, st>>>(counter, plan_word, run_if, k0 * per_kv);
            err = cudaGetLastError();
            if (err != cudaSuccess) return cuda_fail(err, "launch step 3 arm");
        }
        if (gather) {
            aa::GatherArgs ga;
            ga.k = ta.a.k;
            ga.v = ta.a.v;
            ga.counts = ta.a.counts;
            ga.ids = ta.a.ids;
            ga.ids_per_head = lay.ids_per_head;
            ga.tile_slot = ws_ptr<int32_t>(p, lay.tile_slot_off);
            ga.scratch = ws_ptr<uint8_t>(p, lay.gather_off);
            ga.slot_counter = counter;
            ga.n_slots = n_slots;
            ga.hz0 = k0 * Hg;
            ga.plan = plan_word;
            ga.run_if = run_if;
            ga.H = p->H; ga.Hkv = p->Hkv; ga.N = p->N; ga.step = p->step; ga.block = p->block_size;
            aa::gather_tiles_kernel<<<dim3(aa::kGatherSplit, NB - 1, (k1 - k0) * Hg), aa::kGatherThreads, 0, st>>>(ga);
            err = cudaGetLastError();
            if (err != cudaSuccess) return cuda_fail(err, "launch gather pass");
        }
        pa.n_items = k1 * per_kv;
        const int part_items = (k1 - k0) * per_kv;
        const unsigned ctas = part_items < sm_count ? (unsigned)part_items : (unsigned)sm_count;
        aa::tc::attend_persist_kernel<PM><<<ctas, aa::tc::kThreads, aa::tc::kSmemTotal, st>>>(kmap, vmap, kgmap, vgmap, qmap,
                                                                                            ta, pa);
        err = cudaGetLastError();
        if (err != cudaSuccess) return cuda_fail(err, "launch step3 (tc)");
        return AA_OK;
    };
    rc = run_part(0, kv_total, may_overflow ? plan : nullptr, 0);
    if (rc) return rc;
    if (may_overflow) {
        const int kv_per_part = s3.kv_per_part;
        for (int k0 = 0; k0 < kv_total; k0 += kv_per_part) {
            rc = run_part(k0, k0 + kv_per_part < kv_total ? k0 + kv_per_part : kv_total, plan, 1);
            if (rc) return rc;
        }
    }
    return AA_OK;
}

// Pooled queries [B*H, N/block, 128] bf16 (contiguous) as a 3-D tensor map; box = 64 elements x
// `step` rows (the pooled rows of one query head and big block), 128-byte swizzle.
int make_qpool_map(CUtensorMap* map, const void* qpool, int BH, int N, int step, int block) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) {
        snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled entry point not found");
        return AA_ERR_CUDA;
    }
    const cuuint64_t rows = (cuuint64_t)(N / block);
    cuuint64_t gdim[3] = {128, rows, (cuuint64_t)BH};
    cuuint64_t gstr[2] = {256, rows * 256};
    cuuint32_t box[3] = {64, (cuuint32_t)step, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(qpool), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled(qpool) failed with CUresult %d", (int)r);
        return AA_ERR_CUDA;
    }
    return AA_OK;
}

// Block-mean queries and anchors for pooling block size `block` (64, 128 or 256).
int launch_pool(aa::TensorView q, const float* M, __nv_bfloat16* qpool, float* apool, int B, int H, int N, int block,
                cudaStream_t st) {
    const dim3 grid(N / block, H, B);
    if (block == 64)
        aa::pool_kernel<64><<<grid, 64, 0, st>>>(q, M, qpool, apool, H, N);
    else if (block == 128)
        aa::pool_kernel<128><<<grid, 64, 0, st>>>(q, M, qpool, apool, H, N);
    else
        aa::pool_kernel<256><<<grid, 64, 0, st>>>(q, M, qpool, apool, H, N);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AA_OK : cuda_fail(e, "launch pool");
}

// The scoring pass of step 2 (csrc/score_tc.cuh) for NB > 1.
int launch_score(const void* k, int64_t ksb, int64_t ksh, int64_t ksn, const __nv_bfloat16* qpool, const float* apool,
                 uint32_t* bitmap, int32_t* status, int B, int H, int Hkv, int N, int step, int block, float qk_scale,
                 float diff, cudaStream_t st) {
    if (!(qk_scale > 0.f)) return AA_ERR_SHAPE;      // the kernel relies on scores growing with the dot product
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (configured_dev != dev) {
        e = cudaFuncSetAttribute(aa::sc::score_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 aa::sc::kScSmemTotal);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(score_tc)");
        configured_dev = dev;
    }
    aa::sc::ScoreArgs sa;
    sa.apool = apool; sa.bitmap = bitmap; sa.B = B; sa.H = H; sa.Hkv = Hkv; sa.N = N; sa.step = step;
    sa.block = block;
    sa.qk_scale = qk_scale; sa.diff = diff; sa.status = status;
    CUtensorMap kmap, qmap;
    int rc = make_kv_map(&kmap, k, ksb, ksh, ksn, B, Hkv, N, &sa.kpos_n, &sa.kpos_h, &sa.kpos_b);
    if (rc) return rc;
    rc = make_qpool_map(&qmap, qpool, B * H, N, step, block);
    if (rc) return rc;
    const int G = block * step, NB = N / G, Hg = H / Hkv;
    const int max_tiles = (((NB - 1) * G - block - 1) >> 7) - block / 128 + 1;      // candidate tiles of the last big block
    const int units_per_cta = 2 * (128 / step);
    dim3 grid((max_tiles + aa::sc::kTilesPerCta - 1) / aa::sc::kTilesPerCta,
              ((NB - 1) * Hg + units_per_cta - 1) / units_per_cta, B * Hkv);
    aa::sc::score_tc_kernel<<<grid, aa::sc::kScThreads, aa::sc::kScSmemTotal, st>>>(kmap, qmap, sa);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch score");
    return AA_OK;
}

template <int MODE>
int launch_attend(const aa_params_t* p, const aa_workspace_layout_t& lay, cudaStream_t st) {
    return launch_attend_tc<MODE>(p, lay, st);
}

}  // namespace

extern "C" {

int64_t aa_id_row_offset(int32_t block_size, int32_t step, int32_t b) {
    if (b <= 0) return 0;
    const int64_t G = (int64_t)block_size * step;
    return G * b * (b - 1) / 2 - 2 * (int64_t)block_size * (b - 1);
}

int aa_workspace_layout(const aa_params_t* p, aa_workspace_layout_t* lay) {
    if (!lay) return AA_ERR_NULL;
    int rc = check_shape(p);
    if (rc) return rc;
    const size_t B = p->B, H = p->H, N = p->N, D = p->D;
    const size_t NB = N / ((size_t)p->block_size * p->step);
    const size_t BH = B * H;
    lay->ids_per_head = aa_id_row_offset(p->block_size, p->step, (int32_t)NB);
    size_t off = 0;
    lay->m_off = off;       off = align_up(off + BH * N * sizeof(float));
    lay->l_off = off;       off = align_up(off + BH * N * sizeof(float));
    lay->acc_off = off;     off = align_up(off + BH * N * D * sizeof(float));
    lay->qpool_off = off;   off = align_up(off + BH * (N / p->block_size) * D * 2);
    lay->apool_off = off;   off = align_up(off + BH * (N / p->block_size) * sizeof(float));
    lay->bitmap_off = off;  off = align_up(off + BH * NB * (N / 32) * sizeof(uint32_t));
    lay->counts_off = off;  off = align_up(off + BH * NB * sizeof(int32_t));
    lay->ids_off = off;     off = align_up(off + BH * (size_t)lay->ids_per_head * sizeof(int32_t) + 256);
    lay->status_off = off;  off = align_up(off + 8 * sizeof(int32_t));
    const size_t tiles = BH * (size_t)(lay->ids_per_head / aa::tc::kTile);
    lay->tile_slot_off = off;  off = align_up(off + tiles * sizeof(int32_t) + 256);
    lay->gather_off = off;
    lay->min_bytes = off;
    const size_t all = tiles * 2 * (size_t)aa::tc::kTileBytes;
    lay->gather_bytes = all < AA_GATHER_SCRATCH_CAP ? all : AA_GATHER_SCRATCH_CAP;
    lay->total_bytes = off + lay->gather_bytes;
    return AA_OK;
}

int aa_workspace_bytes(const aa_params_t* p, size_t* bytes) {
    if (!bytes) return AA_ERR_NULL;
    aa_workspace_layout_t lay;
    int rc = aa_workspace_layout(p, &lay);
    if (rc) return rc;
    *bytes = lay.total_bytes;
    return AA_OK;
}

int aa_step1_anchor(const aa_params_t* p, void* stream) {
    aa_workspace_layout_t lay;
    int rc = check_full(p, &lay);
    if (rc) return rc;
    rc = clear_status(p, lay, static_cast<cudaStream_t>(stream));
    if (rc) return rc;
    return launch_attend<aa::kWindow>(p, lay, static_cast<cudaStream_t>(stream));
}

int aa_step2_stripes(const aa_params_t* p, void* stream) {
    aa_workspace_layout_t lay;
    int rc = check_full(p, &lay);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int NB = p->N / (p->block_size * p->step);
    const double sm = scale_of(p);
    // the reference forms both constants in double precision on the host and passes
    // them to the kernel as fp32 (anchor_attn_v4.py:298, get_mask_test.py:86)
    const float qk_scale = (float)(sm * 1.44269504);
    const float diff = (float)(p->theta * 1.44269504);

    __nv_bfloat16* qpool = ws_ptr<__nv_bfloat16>(p, lay.qpool_off);
    float* apool = ws_ptr<float>(p, lay.apool_off);
    uint32_t* bitmap = ws_ptr<uint32_t>(p, lay.bitmap_off);
    int32_t* counts = ws_ptr<int32_t>(p, lay.counts_off);
    int32_t* ids = ws_ptr<int32_t>(p, lay.ids_off);

    int rcp = launch_pool(view(p->q, p->q_stride_b, p->q_stride_h, p->q_stride_n), ws_ptr<float>(p, lay.m_off), qpool, apool,
                          p->B, p->H, p->N, p->block_size, st);
    if (rcp) return rcp;
    cudaError_t e = cudaSuccess;

    if (NB > 1) {
        int rc2 = launch_score(p->k, p->k_stride_b, p->k_stride_h, p->k_stride_n, qpool, apool, bitmap,
                               ws_ptr<int32_t>(p, lay.status_off), p->B, p->H, p->Hkv, p->N, p->step, p->block_size, qk_scale,
                               diff, st);
        if (rc2) return rc2;
    }
    aa::compact_kernel<<<dim3(NB, p->H, p->B), 256, 0, st>>>(bitmap, ids, counts, p->H, p->N, p->step,
                                                            p->block_size, lay.ids_per_head);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch compact");
    return AA_OK;
}

int aa_step3_sparse(const aa_params_t* p, void* stream) {
    aa_workspace_layout_t lay;
    int rc = check_full(p, &lay);
    if (rc) return rc;
    return launch_attend<aa::kStripe>(p, lay, static_cast<cudaStream_t>(stream));
}

int aa_step3_sparse_push(const aa_params_t* p, const aa_push_t* push, void* stream) {
    if (!p || !push) return AA_ERR_NULL;
    if (push->n_peers < 1 || push->n_peers > AA_MAX_PEERS) return AA_ERR_SHAPE;
    if (push->rows_per_peer < 0 || push->rows_per_peer % aa::tc::kTile != 0 ||
        (push->rows_per_peer > 0 && (int64_t)push->rows_per_peer * push->n_peers < p->N))
        return AA_ERR_SHAPE;
    for (int i = 0; i < push->n_peers; ++i) {
        if (!push->out[i]) return AA_ERR_NULL;
        if ((uintptr_t)push->out[i] & 15) return AA_ERR_STRIDE;
    }
    aa_params_t q = *p;
    q.out = push->out[0];                      // the argument checks want a non-NULL output
    aa_workspace_layout_t lay;
    int rc = check_full(&q, &lay);
    if (rc) return rc;
    return launch_attend_tc<aa::kStripe>(&q, lay, static_cast<cudaStream_t>(stream), push);
}

int aa_peer_barrier(const aa_peer_barrier_t* b, void* stream) {
    if (!b || !b->status) return AA_ERR_NULL;
    if (b->n_peers < 1 || b->n_peers > AA_MAX_PEERS || b->rank < 0 || b->rank >= b->n_peers) return AA_ERR_SHAPE;
    aa::PeerBarrierArgs a;
    for (int i = 0; i < aa::kBarrierMaxPeers; ++i) a.flags[i] = nullptr;
    for (int i = 0; i < b->n_peers; ++i) {
        if (!b->flags[i]) return AA_ERR_NULL;
        if ((uintptr_t)b->flags[i] & 3) return AA_ERR_STRIDE;
        a.flags[i] = static_cast<int32_t*>(b->flags[i]);
    }
    a.n_peers = b->n_peers;
    a.rank = b->rank;
    a.epoch = b->epoch;
    a.timeout_ns = (unsigned long long)(b->timeout_ms ? b->timeout_ms : 10000u) * 1000000ull;
    a.status = b->status;
    aa::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AA_OK : cuda_fail(e, "launch peer barrier");
}

int aa_rope_dispatch(const aa_rope_dispatch_t* r, void* stream) {
    if (!r) return AA_ERR_NULL;
    if (r->n <= 0 || r->H <= 0 || r->Hkv <= 0 || r->n_peers < 1 || r->n_peers > AA_MAX_PEERS || r->token0 < 0 ||
        r->H % r->n_peers != 0 || r->Hkv % r->n_peers != 0)
        return AA_ERR_SHAPE;
    if (r->D != 128) return AA_ERR_HEAD_DIM;
    if (r->dtype != AA_BF16) return AA_ERR_DTYPE;
    if (!r->q || !r->k || !r->v || !r->cos || !r->sin) return AA_ERR_NULL;
    if (!stride_ok(r->q_stride_n) || !stride_ok(r->k_stride_n) || !stride_ok(r->v_stride_n)) return AA_ERR_STRIDE;
    if (((uintptr_t)r->q | (uintptr_t)r->k | (uintptr_t)r->v | (uintptr_t)r->cos | (uintptr_t)r->sin) & 15)
        return AA_ERR_STRIDE;
    aa::RopeDispatchArgs a;
    for (int i = 0; i < aa::kRopeMaxPeers; ++i) a.dst[i] = nullptr;
    for (int i = 0; i < r->n_peers; ++i) {
        if (!r->dst[i]) return AA_ERR_NULL;
        if ((uintptr_t)r->dst[i] & 15) return AA_ERR_STRIDE;
        a.dst[i] = static_cast<__nv_bfloat16*>(r->dst[i]);
    }
    a.q = static_cast<const __nv_bfloat16*>(r->q);
    a.k = static_cast<const __nv_bfloat16*>(r->k);
    a.v = static_cast<const __nv_bfloat16*>(r->v);
    a.q_sn = r->q_stride_n; a.k_sn = r->k_stride_n; a.v_sn = r->v_stride_n;
    a.cos = static_cast<const __nv_bfloat16*>(r->cos);
    a.sin = static_cast<const __nv_bfloat16*>(r->sin);
    a.n = r->n; a.H = r->H; a.Hkv = r->Hkv; a.n_peers = r->n_peers; a.token0 = r->token0;
    aa::rope_dispatch_kernel<<<(r->n + 15) / 16, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AA_OK : cuda_fail(e, "launch rope dispatch");
}

int aa_forward(const aa_params_t* p, void* stream) {
    int rc = aa_step1_anchor(p, stream);
    if (rc) return rc;
    rc = aa_step2_stripes(p, stream);
    if (rc) return rc;
    return aa_step3_sparse(p, stream);
}

int aa_check_status(const aa_params_t* p, void* stream) {
    aa_workspace_layout_t lay;
    int rc = check_full(p, &lay);
    if (rc) return rc;
    int32_t status[4] = {0, 0, 0, 0};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(status, ws_ptr<int32_t>(p, lay.status_off), sizeof(status),
                                    cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(status)");
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    if (status[0] != 0) return AA_ERR_DEVICE_TIMEOUT;
    return status[1] == 0 ? AA_OK : AA_ERR_BAD_LIST;
}

int aa_validate_lists(const aa_params_t* p, void* stream) {
    aa_workspace_layout_t lay;
    int rc = check_full(p, &lay);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t* flag = ws_ptr<int32_t>(p, lay.status_off) + 1;
    cudaError_t e = cudaMemsetAsync(flag, 0, sizeof(int32_t), st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(list flag)");
    const int NB = p->N / (p->block_size * p->step);
    aa::validate_lists_kernel<<<dim3(NB, p->B * p->H), 256, 0, st>>>(
        ws_ptr<int32_t>(p, lay.counts_off), ws_ptr<int32_t>(p, lay.ids_off), lay.ids_per_head, p->N, p->step,
        p->block_size, flag);
    e = cudaGetLastError();
    return e == cudaSuccess ? AA_OK : cuda_fail(e, "launch list validation");
}

int aa_selftest_wait_timeout(const aa_params_t* p, void* stream) {
    aa_workspace_layout_t lay;
    int rc = check_full(p, &lay);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = clear_status(p, lay, st);
    if (rc) return rc;
    aa::tc::wait_timeout_selftest_kernel<<<1, 32, 0, st>>>(ws_ptr<int32_t>(p, lay.status_off));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch wait self-test");
    return AA_OK;
}

int aa_total_selected(const aa_params_t* p, void* stream, int64_t* total) {
    if (!total) return AA_ERR_NULL;
    aa_workspace_layout_t lay;
    int rc = check_full(p, &lay);
    if (rc) return rc;
    const size_t n = (size_t)p->B * p->H * (p->N / (p->block_size * p->step));
    int32_t* host = (int32_t*)malloc(n * sizeof(int32_t));
    if (!host) return AA_ERR_TOO_LARGE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(host, ws_ptr<int32_t>(p, lay.counts_off), n * sizeof(int32_t),
                                    cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        free(host);
        return cuda_fail(e, "read counts");
    }
    int64_t s = 0;
    for (size_t i = 0; i < n; ++i) s += host[i];
    free(host);
    *total = s;
    return AA_OK;
}

// ---------------------------------------------------------------------------
// aa_step2_stripes_static: stripe identification with its intermediates in a
// fixed array inside the library image, for hosts that may not allocate device
// memory when they call us (see the header).  Same three kernels as
// aa_step2_stripes, so counts and ids come out bit-identical.
// ---------------------------------------------------------------------------
}  // extern "C"

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime's
// symbol table, never a device pointer; kernels get the address that
// cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char g_static_scratch[AA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};
std::mutex g_static_mutex;

// Device address of the scratch array on the current device, looked up once per device.
int static_scratch_for_current_device(void** addr, int* dev_out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return AA_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        if (!p) return AA_ERR_CUDA;
        g_static_scratch_addr[dev] = p;
    }
    *addr = g_static_scratch_addr[dev];
    *dev_out = dev;
    return AA_OK;
}

}  // namespace

extern "C" {

int aa_step2_stripes_static(const aa_stripes_static_args_t* a, void* stream) {
    if (!a) return AA_ERR_NULL;
    aa_params_t shape;
    memset(&shape, 0, sizeof(shape));
    shape.B = a->B; shape.H = a->H; shape.Hkv = a->Hkv; shape.N = a->N; shape.D = a->D;
    shape.block_size = a->block_size; shape.step = a->step; shape.dtype = a->dtype;
    int rc = check_shape(&shape);
    if (rc) return rc;
    if (!a->q || !a->k || !a->anchors || !a->counts || !a->ids) return AA_ERR_NULL;
    const int64_t st[] = {a->q_stride_b, a->q_stride_h, a->q_stride_n, a->k_stride_b, a->k_stride_h, a->k_stride_n};
    for (int64_t x : st)
        if (!stride_ok(x)) return AA_ERR_STRIDE;
    if (((uintptr_t)a->q | (uintptr_t)a->k) & 15) return AA_ERR_STRIDE;

    // carve the three intermediates out of the fixed array; refuse what does not fit
    const size_t BH = (size_t)a->B * a->H, nblk = (size_t)a->N / a->block_size;
    const int NB = a->N / (a->block_size * a->step);
    const size_t qpool_off = 0;
    const size_t apool_off = align_up(qpool_off + BH * nblk * aa::kRowBytes);
    const size_t bitmap_off = align_up(apool_off + BH * nblk * sizeof(float));
    const size_t need = align_up(bitmap_off + BH * (size_t)NB * ((size_t)a->N / 32) * sizeof(uint32_t));
    if (need + 256 > AA_STATIC_SCRATCH_BYTES) return AA_ERR_TOO_LARGE;      // + the status word at the end

    void* base = nullptr;
    int dev = 0;
    rc = static_scratch_for_current_device(&base, &dev);
    if (rc) return rc;
    unsigned char* sc = static_cast<unsigned char*>(base);
    __nv_bfloat16* qpool = reinterpret_cast<__nv_bfloat16*>(sc + qpool_off);
    float* apool = reinterpret_cast<float*>(sc + apool_off);
    uint32_t* bitmap = reinterpret_cast<uint32_t*>(sc + bitmap_off);

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const double sm = a->sm_scale != 0.0 ? a->sm_scale : 1.0 / sqrt((double)a->D);
    const float qk_scale = (float)(sm * 1.44269504);
    const float diff = (float)(a->theta * 1.44269504);
    const int64_t ids_per_head = aa_id_row_offset(a->block_size, a->step, NB);

    int rcp = launch_pool(view(a->q, a->q_stride_b, a->q_stride_h, a->q_stride_n), a->anchors, qpool, apool, a->B, a->H,
                          a->N, a->block_size, s);
    if (rcp) return rcp;
    cudaError_t e = cudaSuccess;
    // the status word of the bounded device-side waits lives at the end of the fixed array
    // (aa_step2_stripes_static_check_status reads it back)
    int32_t* status = reinterpret_cast<int32_t*>(sc + AA_STATIC_SCRATCH_BYTES - 256);
    cudaError_t em = cudaMemsetAsync(status, 0, sizeof(int32_t), s);
    if (em != cudaSuccess) return cuda_fail(em, "cudaMemsetAsync(static status)");
    if (NB > 1) {
        int rc2 = launch_score(a->k, a->k_stride_b, a->k_stride_h, a->k_stride_n, qpool, apool, bitmap, status, a->B,
                               a->H, a->Hkv, a->N, a->step, a->block_size, qk_scale, diff, s);
        if (rc2) return rc2;
    }
    aa::compact_kernel<<<dim3(NB, a->H, a->B), 256, 0, s>>>(bitmap, a->ids, a->counts, a->H, a->N, a->step,
                                                           a->block_size, ids_per_head);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch compact (static)");
    return AA_OK;
}

int aa_step2_stripes_static_check_status(void* stream) {
    void* base = nullptr;
    int dev = 0;
    int rc = static_scratch_for_current_device(&base, &dev);
    if (rc) return rc;
    int32_t status = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(&status, static_cast<unsigned char*>(base) + AA_STATIC_SCRATCH_BYTES - 256,
                                    sizeof(status), cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(static status)");
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    return status == 0 ? AA_OK : AA_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// The block-granular comparator (see the header): merged tile lists in the caller's
// workspace, then the attention kernel in its block mode.
// ---------------------------------------------------------------------------
namespace {

struct BlockSparseLayout {
    size_t lists_off, counts_off, status_off, total_bytes;
    int npairs, list_stride;
};

int block_sparse_layout(const aa_block_sparse_t* a, BlockSparseLayout* lay) {
    if (!a) return AA_ERR_NULL;
    if (a->B <= 0 || a->H <= 0 || a->Hkv <= 0 || a->N <= 0 || a->H % a->Hkv != 0 || a->max_blocks <= 0)
        return AA_ERR_SHAPE;
    if (a->D != 128) return AA_ERR_HEAD_DIM;
    if (a->N % (2 * aa::tc::kTile) != 0) return AA_ERR_SEQ;
    if (a->dtype != AA_BF16) return AA_ERR_DTYPE;
    if ((int64_t)a->N * a->H * a->B > (int64_t)1 << 40 || a->N / aa::tc::kTile > (int)aa::kBlockIdMask)
        return AA_ERR_TOO_LARGE;
    const size_t BH = (size_t)a->B * a->H;
    lay->npairs = a->N / (2 * aa::tc::kTile);
    // a pair's merged list holds at most the entries both query blocks read
    const int64_t stride = 2 * (int64_t)(a->max_blocks < a->N / aa::tc::kTile ? a->max_blocks : a->N / aa::tc::kTile);
    lay->list_stride = (int)stride;
    size_t off = 0;
    lay->lists_off = off;   off = align_up(off + BH * lay->npairs * (size_t)stride * sizeof(int32_t));
    lay->counts_off = off;  off = align_up(off + BH * lay->npairs * sizeof(int32_t));
    lay->status_off = off;  off = align_up(off + 4 * sizeof(int32_t));
    lay->total_bytes = off;
    return AA_OK;
}

int block_sparse_check(const aa_block_sparse_t* a, BlockSparseLayout* lay) {
    int rc = block_sparse_layout(a, lay);
    if (rc) return rc;
    if (!a->q || !a->k || !a->v || !a->out || !a->block_index) return AA_ERR_NULL;
    const int64_t st[] = {a->q_stride_b, a->q_stride_h, a->q_stride_n, a->k_stride_b, a->k_stride_h, a->k_stride_n,
                          a->v_stride_b, a->v_stride_h, a->v_stride_n, a->o_stride_b, a->o_stride_h, a->o_stride_n};
    for (int64_t s : st)
        if (!stride_ok(s)) return AA_ERR_STRIDE;
    if (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->out) & 15) return AA_ERR_STRIDE;
    if (!a->workspace || ((uintptr_t)a->workspace & 255) || a->workspace_bytes < lay->total_bytes)
        return AA_ERR_WORKSPACE;
    return AA_OK;
}

}  // namespace

extern "C" {

int aa_block_sparse_workspace_bytes(const aa_block_sparse_t* a, size_t* bytes) {
    if (!bytes) return AA_ERR_NULL;
    BlockSparseLayout lay;
    int rc = block_sparse_layout(a, &lay);
    if (rc) return rc;
    *bytes = lay.total_bytes;
    return AA_OK;
}

int aa_block_sparse_attend(const aa_block_sparse_t* a, void* stream) {
    BlockSparseLayout bl;
    int rc = block_sparse_check(a, &bl);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    int32_t* status = reinterpret_cast<int32_t*>(ws + bl.status_off);
    cudaError_t e = cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");
    const int BH = a->B * a->H, items = BH * bl.npairs;
    aa::merge_block_lists_kernel<<<(items + 127) / 128, 128, 0, st>>>(
        a->block_index, BH, a->N / aa::tc::kTile, a->max_blocks, reinterpret_cast<int32_t*>(ws + bl.lists_off),
        reinterpret_cast<int32_t*>(ws + bl.counts_off), bl.list_stride, status + 1);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch merge_block_lists");

    // the attention kernel takes the operator's argument block: fill in what the block mode reads
    aa_params_t p;
    memset(&p, 0, sizeof(p));
    p.B = a->B; p.H = a->H; p.Hkv = a->Hkv; p.N = a->N; p.D = a->D;
    p.block_size = 128; p.step = 16; p.dtype = a->dtype;
    p.sm_scale = a->sm_scale;
    p.q = a->q; p.k = a->k; p.v = a->v; p.out = a->out;
    p.q_stride_b = a->q_stride_b; p.q_stride_h = a->q_stride_h; p.q_stride_n = a->q_stride_n;
    p.k_stride_b = a->k_stride_b; p.k_stride_h = a->k_stride_h; p.k_stride_n = a->k_stride_n;
    p.v_stride_b = a->v_stride_b; p.v_stride_h = a->v_stride_h; p.v_stride_n = a->v_stride_n;
    p.o_stride_b = a->o_stride_b; p.o_stride_h = a->o_stride_h; p.o_stride_n = a->o_stride_n;
    p.workspace = a->workspace;
    p.workspace_bytes = a->workspace_bytes;
    aa_workspace_layout_t lay;
    memset(&lay, 0, sizeof(lay));
    lay.counts_off = bl.counts_off;
    lay.ids_off = bl.lists_off;
    lay.status_off = bl.status_off;
    lay.ids_per_head = (int64_t)bl.npairs * bl.list_stride;
    lay.total_bytes = bl.total_bytes;
    return launch_attend_tc<aa::kBlock>(&p, lay, st, nullptr, bl.list_stride);
}

int aa_dense_causal_attend(const aa_dense_causal_t* a, void* stream) {
    if (!a) return AA_ERR_NULL;
    if (a->B <= 0 || a->H <= 0 || a->Hkv <= 0 || a->Nq <= 0 || a->Nkv < a->Nq || a->H % a->Hkv != 0) return AA_ERR_SHAPE;
    if (a->D != 128) return AA_ERR_HEAD_DIM;
    if (a->dtype != AA_BF16) return AA_ERR_DTYPE;
    if ((int64_t)a->Nkv * a->H * a->B > (int64_t)1 << 40 || a->Nkv / aa::tc::kTile >= (int)aa::kBlockIdMask)
        return AA_ERR_TOO_LARGE;
    if (!a->q || !a->k || !a->v || !a->out || !a->status) return AA_ERR_NULL;
    const int64_t strides[] = {a->q_stride_b, a->q_stride_h, a->q_stride_n, a->k_stride_b, a->k_stride_h, a->k_stride_n,
                               a->v_stride_b, a->v_stride_h, a->v_stride_n, a->o_stride_b, a->o_stride_h, a->o_stride_n};
    for (int64_t s : strides)
        if (!stride_ok(s)) return AA_ERR_STRIDE;
    if (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->out) & 15) return AA_ERR_STRIDE;
    if ((uintptr_t)a->status & 15) return AA_ERR_STRIDE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(a->status, 0, 4 * sizeof(int32_t), st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");
    // the attention kernel takes the operator's argument block: fill in what the dense variant reads
    aa_params_t p;
    memset(&p, 0, sizeof(p));
    p.B = a->B; p.H = a->H; p.Hkv = a->Hkv; p.D = a->D;
    p.N = (a->Nq + 2 * aa::tc::kTile - 1) / (2 * aa::tc::kTile) * (2 * aa::tc::kTile);      // grid: pairs of query tiles
    p.block_size = 128; p.step = 16; p.dtype = a->dtype;
    p.sm_scale = a->sm_scale;
    p.q = a->q; p.k = a->k; p.v = a->v; p.out = a->out;
    p.q_stride_b = a->q_stride_b; p.q_stride_h = a->q_stride_h; p.q_stride_n = a->q_stride_n;
    p.k_stride_b = a->k_stride_b; p.k_stride_h = a->k_stride_h; p.k_stride_n = a->k_stride_n;
    p.v_stride_b = a->v_stride_b; p.v_stride_h = a->v_stride_h; p.v_stride_n = a->v_stride_n;
    p.o_stride_b = a->o_stride_b; p.o_stride_h = a->o_stride_h; p.o_stride_n = a->o_stride_n;
    p.workspace = a->status;                     // only the status words are used
    p.workspace_bytes = 4 * sizeof(int32_t);
    aa_workspace_layout_t lay;
    memset(&lay, 0, sizeof(lay));
    DenseTail dt{a->Nq, a->Nkv};
    return launch_attend_tc<aa::kBlock>(&p, lay, st, nullptr, 0, &dt);
}

int aa_block_sparse_check_status(const aa_block_sparse_t* a, void* stream) {
    BlockSparseLayout bl;
    int rc = block_sparse_check(a, &bl);
    if (rc) return rc;
    int32_t status[4] = {0, 0, 0, 0};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(status, static_cast<uint8_t*>(a->workspace) + bl.status_off, sizeof(status),
                                    cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(status)");
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    if (status[0] != 0) return AA_ERR_DEVICE_TIMEOUT;
    if (status[1] != 0) return AA_ERR_UNSORTED;
    return AA_OK;
}

}  // extern "C"

extern "C" {

const char* aa_strerror(int code) {
    switch (code) {
        case AA_OK: return "ok";
        case AA_ERR_NULL: return "a required pointer is NULL";
        case AA_ERR_SHAPE: return "bad shape: B, H, Hkv, N must be positive and Hkv must divide H";
        case AA_ERR_HEAD_DIM: return "head dimension must be 128";
        case AA_ERR_STEP: return "Invalid step size. Only step sizes 16 or 32 are supported.";
        case AA_ERR_BLOCK: return "block_size must be 64, 128 or 256";
        case AA_ERR_SEQ: return "Sequence length must be divisible by (block_size * step)";
        case AA_ERR_WORKSPACE: return "workspace missing, not 256-byte aligned, or too small";
        case AA_ERR_STRIDE: return "pointers must be 16-byte aligned and strides multiples of 8 elements";
        case AA_ERR_DTYPE: return "only bf16 is supported";
        case AA_ERR_CUDA: return "CUDA call failed";
        case AA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
        case AA_ERR_TOO_LARGE: return "problem too large for this entry point";
        case AA_ERR_UNSORTED: return "a block list is not in ascending order";
        case AA_ERR_BAD_LIST: return "an id list in the workspace is malformed (count or id out of range, or not ascending)";
        default: return "unknown error";
    }
}

const char* aa_last_cuda_error(void) { return g_cuda_err; }
int aa_version(void) { return 2; }
int aa_launches_per_forward(void) { return 6; }
int aa_forward_launches(const aa_params_t* p) {
    aa_workspace_layout_t lay;
    int rc = check_full(p, &lay);
    if (rc) return rc < 0 ? rc : -rc;
    const Step3Layout s3 = step3_layout(p, lay);
    const int NB = p->N / (p->block_size * p->step);
    int n = 1 + 2 + (NB > 1 ? 1 : 0);                       // step 1; pool, compact and (with candidates) the score kernel
    if (!s3.gather) return n + 1;                           // step 3: the attention kernel alone
    if (!s3.may_overflow) return n + 2;                     // gather pass + attention kernel
    const int parts = (s3.kv_total + s3.kv_per_part - 1) / s3.kv_per_part;
    return n + 1 + 3 * (1 + parts);                         // plan; counters, gather pass, attention kernel per sequence part
}

}  // extern "C"

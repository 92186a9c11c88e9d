/*
 * C ABI of the B200 anchor-attention prefill operator.
 *
 * One shared library (libanchor_attn_b200.so), plain C symbols, raw device
 * pointers and sizes.  Nothing here allocates or synchronises unless stated:
 * every entry point enqueues kernels on the caller's CUDA stream and returns.
 * The caller owns every buffer.  Two calls may run concurrently on different
 * streams as long as they use different workspaces.
 *
 * Citations are paths inside the reference project (yuzhouzhang9/Anchor-Attention).
 * The reference has no FFI of its own: its operator is a Python function that
 * launches three Triton kernels.  Each entry point below names the Python
 * function whose work it replaces.
 */
#ifndef ANCHOR_ATTN_B200_H
#define ANCHOR_ATTN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error codes (0 = success).  aa_strerror() gives the text. */
enum {
    AA_OK = 0,
    AA_ERR_NULL = -1,          /* a required pointer is NULL                         */
    AA_ERR_SHAPE = -2,         /* B/H/Hkv/N non-positive, H % Hkv != 0               */
    AA_ERR_HEAD_DIM = -3,      /* D != 128                                           */
    AA_ERR_STEP = -4,          /* step not in {16, 32}  (anchor_attn_v4.py:305)      */
    AA_ERR_BLOCK = -5,         /* block_size not in {64, 128, 256}                   */
    AA_ERR_SEQ = -6,           /* N % (block_size*step) != 0 (anchor_attn_v4.py:308) */
    AA_ERR_WORKSPACE = -7,     /* workspace missing, misaligned or too small         */
    AA_ERR_STRIDE = -8,        /* a stride is not a multiple of 8 elements (16 B)    */
    AA_ERR_DTYPE = -9,         /* dtype is not AA_BF16                               */
    AA_ERR_CUDA = -10,         /* a CUDA runtime/driver call failed (see aa_last_cuda_error) */
    AA_ERR_DEVICE_TIMEOUT = -11,/* a bounded device-side wait gave up (status word)  */
    AA_ERR_TOO_LARGE = -12,    /* size beyond what an entry point supports           */
    AA_ERR_UNSORTED = -13,     /* a key-block list of the comparator is not ascending */
    AA_ERR_BAD_LIST = -14      /* aa_validate_lists found a count or an id out of range  */
};

enum { AA_BF16 = 0 };

/*
 * Problem description.  Logical tensor shapes:
 *   q, out : [B, H,   N, D]      k, v : [B, Hkv, N, D]
 * Query head h reads KV head h / (H / Hkv), the order repeat_kv produces
 * (my_utils/ops_util.py:6-24); pass Hkv == H for pre-expanded K/V, which is
 * what the reference's caller does (modules/llama/anchor_attention.py:89-91).
 * Strides are in ELEMENTS; the D axis must be contiguous (stride 1) and every
 * other stride a multiple of 8 elements.  Any of [B,H,N,D] and [B,N,H,D]
 * memory orders is therefore accepted without a copy.
 */
typedef struct aa_params {
    int32_t B, H, Hkv, N, D;
    int32_t block_size;        /* pooling block of step 2: 64, 128 or 256; the default of every
                                  harness is 128 (patch.py:36-40 "block_size_M").  The big block is
                                  block_size*step rows; steps 1 and 3 always work on 128-row tiles,
                                  as the reference's do (anchor_attn_v4.py:232)              */
    int32_t step;              /* 16 or 32 (patch.py:36-40 "step")                       */
    int32_t dtype;             /* AA_BF16                                                */
    double  theta;             /* "difference"/theta in natural-log units, default 12;
                                  the library multiplies by log2(e) as anchor_attn_v4.py:298 does */
    double  sm_scale;          /* 0 => D^-0.5 (anchor_attn_v4.py:312); a double because the
                                  reference derives its fp32/bf16 constants from a Python float */
    const void *q, *k, *v;     /* device pointers, bf16                                  */
    void       *out;           /* device pointer, bf16, same logical shape as q          */
    int64_t q_stride_b, q_stride_h, q_stride_n;
    int64_t k_stride_b, k_stride_h, k_stride_n;
    int64_t v_stride_b, v_stride_h, v_stride_n;
    int64_t o_stride_b, o_stride_h, o_stride_n;
    void   *workspace;         /* device scratch, 256-byte aligned; aa_workspace_bytes() is the
                                  recommended size, aa_workspace_layout().min_bytes the least   */
    size_t  workspace_bytes;
} aa_params_t;

/* Where the inter-kernel state lives inside the workspace (byte offsets).
 * Replaces the tensors the reference allocates per call: L_buffer, M_buffer,
 * Acc_buffer (anchor_step_1_2_v2.py:174-176), true_coords, true_counts
 * (get_mask_test.py:138-145).  The id lists are stored CSR-style with a static
 * capacity: big block b of a head owns ids[id_row_offset(b) .. +counts[b]),
 * id_row_offset(b) = sum_{b'<b} max(0, b'*G - 2*block_size), G = block_size*step,
 * ids_per_head = id_row_offset(NB). */
typedef struct aa_workspace_layout {
    size_t m_off;        /* float   [B,H,N]          row maxima of step 1 (log2 domain)        */
    size_t l_off;        /* float   [B,H,N]          softmax denominators of step 1             */
    size_t acc_off;      /* float   [B,H,N/128,D/4,128,4]  un-normalised outputs of step 1, in tiles of
                                                     128 rows, each tile chunk-major: the 16-byte chunk k
                                                     (columns 4k..4k+3) of row r is at float offset
                                                     512 k + 4 r of the tile (steps 1 and 3 touch it with
                                                     one thread per row; this makes their accesses contiguous) */
    size_t qpool_off;    /* bf16    [B,H,N/bs,D]     block-mean queries                         */
    size_t apool_off;    /* float   [B,H,N/bs]       block-mean anchors (bf16-valued)           */
    size_t bitmap_off;   /* uint32  [B,H,NB,N/32]    hit bitmap of step 2                       */
    size_t counts_off;   /* int32   [B,H,NB]         selected columns per big block             */
    size_t ids_off;      /* int32   [B,H,ids_per_head] ascending selected column ids            */
    size_t status_off;   /* int32   [8]              [0] a bounded device-side wait gave up,
                                                     [1] aa_validate_lists found a bad list,
                                                     [2] gather slots handed out by step 3,
                                                     [3] item counter of the step-1 or step-3
                                                         kernel that ran last,
                                                     [4] step 3 ran KV head by KV head (1) or in
                                                         one go (0); only written when the gather
                                                         scratch has no slot for every possible tile */
    size_t total_bytes;  /* recommended workspace size: min_bytes + gather_bytes                 */
    int64_t ids_per_head;
    size_t tile_slot_off;/* int32   [B,H,ids_per_head/128] gather slot of every 128-id tile, or -1 */
    size_t gather_off;   /* gather scratch of step 3: 64 KB slots (K image, V image) for the id
                            tiles that are not runs of consecutive rows; the LAST section        */
    size_t gather_bytes; /* recommended size of it: every tile of every list, but at most
                            AA_GATHER_SCRATCH_CAP bytes                                          */
    size_t min_bytes;    /* smallest workspace the entry points accept (= gather_off).  Step 3
                            uses as many 64 KB slots as workspace_bytes - gather_off holds;
                            tiles without a slot are gathered inside the attention kernel       */
} aa_workspace_layout_t;

#define AA_GATHER_SCRATCH_CAP ((size_t)8 << 30)

/* Size and layout of the workspace for a problem (only the shape fields of p
 * are read).  Host-only, no CUDA calls. */
int aa_workspace_bytes(const aa_params_t *p, size_t *bytes);
int aa_workspace_layout(const aa_params_t *p, aa_workspace_layout_t *layout);

/* First id slot of big block b inside a head's id list (see above). */
int64_t aa_id_row_offset(int32_t block_size, int32_t step, int32_t b);

/* The whole operator: steps 1, 2, 3 back to back on `stream` (a cudaStream_t).
 * Replaces anchor_attn -> _anchor_attn (anchor_attn_v4.py:291-324, 226-273). */
int aa_forward(const aa_params_t *p, void *stream);

/* Step 1, anchor / window attention: fills M, L, Acc in the workspace.
 * Replaces anchor_attn_step_1 (anchor_step_1_2_v2.py:164-196). */
int aa_step1_anchor(const aa_params_t *p, void *stream);

/* Step 2, difference-aware stripe identification: reads q, k and M, fills
 * qpool, apool, bitmap, counts and ids.  Replaces anchor_attn_step_2 ->
 * get_q_mask (anchor_step_1_2_v2.py:199-210, get_mask_test.py:127-159). */
int aa_step2_stripes(const aa_params_t *p, void *stream);

/* Step 3, gathered sparse flash attention merged with the step-1 state:
 * reads M, L, Acc, counts, ids; writes out.  Replaces the launch of
 * _triton_stripe_sparse_attn_fwd_kernel_step3 (anchor_attn_v4.py:246-268).
 * Two kernels: a gather pass that copies the selected K/V rows of every id tile that is
 * not a run of consecutive rows into the workspace's gather scratch once (the eight CTAs
 * that serve the 2048 query rows of a big block then fetch it with bulk copies instead
 * of gathering the same rows eight times), and the attention kernel.  Counts are clamped
 * to the capacity of their big block and ids to [0, N) before they are used as
 * addresses, so a stale or foreign workspace cannot make the kernels read outside K/V
 * (aa_validate_lists tells whether the lists are well formed). */
int aa_step3_sparse(const aa_params_t *p, void *stream);

/* Checks the id lists in the workspace without gathering anything: every count within
 * [0, b*G - 2*block_size], every list ascending and inside [block_size, b*G - block_size)
 * (the shape get_mask_test.py:111-124 produces).  Enqueues one small kernel; a following
 * aa_check_status returns AA_ERR_BAD_LIST if a list is malformed.  For callers that fill
 * or keep the lists themselves before aa_step3_sparse.  (No counterpart in the
 * reference, whose step 3 trusts its lists.) */
int aa_validate_lists(const aa_params_t *p, void *stream);

/* Step 3 for head-parallel runs: identical to aa_step3_sparse, except that every output
 * row is stored to push->out[0 .. n_peers) instead of p->out -- same element offsets and
 * strides (p->o_stride_*) in each.  The pointers may be peer-mapped memory of other GPUs
 * of the node (symmetric or IPC-opened buffers): each rank then writes its heads into every
 * rank's copy of the assembled [B,N,H,D] output while it computes, and no all-gather
 * follows; the ranks only need a barrier before they read their copy.  p->out is ignored.
 * (No counterpart in the reference, which is single-GPU: test_hf.py:126.) */
#define AA_MAX_PEERS 8
typedef struct aa_push {
    int32_t n_peers;
    int32_t rows_per_peer;     /* 0: every row goes to every peer (replicated output).
                                  > 0 (a multiple of 128, n_peers * rows_per_peer >= N): token-sharded
                                  output -- row n goes only to out[n / rows_per_peer], at row
                                  n % rows_per_peer of that buffer (whose o_stride_* are p's)      */
    void   *out[AA_MAX_PEERS];
} aa_push_t;
int aa_step3_sparse_push(const aa_params_t *p, const aa_push_t *push, void *stream);

/* Barrier between the ranks of a head-parallel layer, to follow aa_step3_sparse_push: the
 * rank announces epoch `epoch` in every peer's flag array (flags[p] + rank) and waits until
 * every peer has announced it in this rank's own array (flags[rank] + p).  Plain peer
 * stores and loads, release / acquire at system scope.  flags[p] is rank p's array of at
 * least n_peers int32 in device memory every rank can address (symmetric or IPC-opened),
 * zero before the first use; `epoch` must grow by one with every call and be the same on
 * all ranks.  The wait is bounded: after timeout_ms (0 = 10 s) without a peer's
 * announcement the kernel sets *status (a device int32 of this rank, which the caller
 * zeroes once) to 1 and returns, so a rank that left between steps cannot hang the
 * others' GPUs; read *status on the host before using the assembled output.  One launch,
 * no synchronisation.  (No counterpart in the reference, which is single-GPU.) */
typedef struct aa_peer_barrier {
    int32_t n_peers, rank;
    int32_t epoch;
    uint32_t timeout_ms;
    void   *flags[AA_MAX_PEERS];
    int32_t *status;
} aa_peer_barrier_t;
int aa_peer_barrier(const aa_peer_barrier_t *b, void *stream);

/* Tokens -> heads exchange of a sequence-parallel prefill, fused with the rotary embedding: reads
 * the q/k/v projections of this rank's n tokens (q [n,H,128], k/v [n,Hkv,128] bf16, row strides
 * in elements, heads 128 apart), rotates q and k with the rotate-half formulation on bf16 values,
 * rounding included (what apply_rotary_pos_emb computes in the reference's forward,
 * modules/llama/anchor_attention.py:38-48; cos/sin are [n,128] bf16), and stores every head row
 * into dst[d] of the rank d that owns the head: a [N, h + 2*hkv, 128] token-major buffer
 * (h = H / n_peers query heads, then hkv = Hkv / n_peers key heads, then the value heads), at
 * token row token0 + i.  Plain coalesced stores, to peer memory for d != this rank; replaces the
 * rotary kernels, the packing copies (anchor_attention.py:89-91) and an all-to-all.  Follow it
 * with aa_peer_barrier before any rank reads its buffer.  One launch, no synchronisation. */
typedef struct aa_rope_dispatch {
    int32_t n, H, Hkv, D, dtype;
    int32_t n_peers, token0;
    const void *q, *k, *v;
    int64_t q_stride_n, k_stride_n, v_stride_n;
    const void *cos, *sin;
    void   *dst[AA_MAX_PEERS];
} aa_rope_dispatch_t;
int aa_rope_dispatch(const aa_rope_dispatch_t *r, void *stream);

/* Reads the device status words (synchronises the stream first).  Returns AA_OK,
 * AA_ERR_DEVICE_TIMEOUT, AA_ERR_BAD_LIST or AA_ERR_CUDA. */
int aa_check_status(const aa_params_t *p, void *stream);

/* Self-test of the failure path: enqueues a one-warp kernel that waits on a barrier nothing
 * arrives on.  Its bounded wait gives up (about half a second), sets the workspace's status
 * word and returns; a following aa_check_status reports AA_ERR_DEVICE_TIMEOUT.  No fault, no
 * trap: the CUDA context stays usable.  (No counterpart in the reference.) */
int aa_selftest_wait_timeout(const aa_params_t *p, void *stream);

/* Sum of all counts as computed by the last aa_step2_stripes on this
 * workspace, written to *total (synchronises the stream).  The numerator of the
 * reference's sparsity ratio (anchor_attn_v4.py:271). */
int aa_total_selected(const aa_params_t *p, void *stream, int64_t *total);

/*
 * Stripe identification for callers that must not allocate device memory.
 * (No counterpart in the reference: its step 2 allocates fresh tensors on every
 * call, get_mask_test.py:138-145.)
 *
 * Some hosts of this library are not allowed to obtain scratch memory at call
 * time: an inference-runtime plug-in whose enqueue hook is forbidden from
 * allocating, or a process whose whole device memory has already been handed to
 * a framework's arena, where a raw allocation would fail.  For them this entry
 * point does the same work as aa_step2_stripes -- same kernels, same bits in
 * `counts` and `ids` -- but keeps its intermediates (pooled queries, pooled
 * anchors, hit bitmap) in a fixed AA_STATIC_SCRATCH_BYTES array that is part of
 * the library image.  Every GPU that loads the library carries that array until
 * the process exits.
 *
 * The caller passes q, k, the step-1 row maxima `anchors` (fp32 [B,H,N], log2
 * domain) and the two output buffers: counts int32 [B,H,NB] and ids int32
 * [B,H,ids_per_head] (ids_per_head = aa_id_row_offset(block_size, step, NB)).
 *
 * - Problems whose intermediates exceed the array are refused with
 *   AA_ERR_TOO_LARGE; nothing is launched.  The need is
 *   B*H*(N/block_size)*(256+4) + B*H*NB*(N/32)*4 + 256 bytes plus alignment padding
 *   (NB = N / (block_size*step)), e.g. 4.1 MiB for B*H = 32, N = 32768, block_size 128.
 * - It calls no cudaMalloc / cudaFree and no allocating library routine.
 * - The first call on a device looks up the array's device address (once per
 *   device, with that device current); make that first call before starting
 *   any stream capture.
 * - All calls share the one array and it keeps whatever the last call left in
 *   it.  Nothing in it has to start at zero (every word a kernel reads is
 *   written earlier in the same call), but two calls that overlap on the GPU --
 *   different streams, or different host threads -- race on it: serialise them.
 */
#define AA_STATIC_SCRATCH_BYTES (8u << 20)

typedef struct aa_stripes_static_args {
    int32_t B, H, Hkv, N, D;
    int32_t block_size, step, dtype;          /* as in aa_params_t                 */
    double  theta, sm_scale;                  /* as in aa_params_t                 */
    const void *q, *k;                        /* bf16 device pointers              */
    int64_t q_stride_b, q_stride_h, q_stride_n;
    int64_t k_stride_b, k_stride_h, k_stride_n;
    const float *anchors;                     /* in:  [B,H,N] step-1 row maxima    */
    int32_t *counts;                          /* out: [B,H,NB]                     */
    int32_t *ids;                             /* out: [B,H,ids_per_head]           */
} aa_stripes_static_args_t;

int aa_step2_stripes_static(const aa_stripes_static_args_t *args, void *stream);

/* Status of the bounded device-side waits of the aa_step2_stripes_static calls made so
 * far on the current device (the word lives at the end of the fixed array and is
 * cleared by every call): synchronises `stream`, returns AA_OK or
 * AA_ERR_DEVICE_TIMEOUT.  After a timeout the counts and ids of that call are incomplete. */
int aa_step2_stripes_static_check_status(void *stream);

/*
 * The block-granular comparator the reference measures anchor attention against:
 * block-sparse flash attention in which every 128-row query block attends a list of whole
 * 128-row key blocks.  Replaces _triton_block_sparse_attention and its kernel
 * (block_sparse_flash_attention_v2.py:113-144, 10-110); the lists come from the
 * reference's index builders (:150-309) or the host-side mirrors of them.
 *
 * block_index is int32 [B, H, N/128, max_blocks] (device memory), each row ascending, exactly
 * what the reference's builders hand to its kernel.  As there, query block m reads the first
 * min(m + 1, max_blocks) entries of its row (:66), an index that occurs several times is
 * attended several times (short rows are zero-padded and sorted, so key block 0 repeats), the
 * row's own block gets a -inf causal mask (:76-77) and the softmax state starts empty (:52-54).
 * Entries above the query block's own index are masked for every row there and are skipped
 * here.  Logical shapes, strides and the GQA mapping are those of aa_params_t; N must be a
 * multiple of 256 (the caller pads, as the reference's wrapper pads to 128, :334-339).
 * The workspace holds the per-CTA tile lists (at most 2*max_blocks entries per pair of query
 * blocks), their lengths and the status words.
 */
typedef struct aa_block_sparse {
    int32_t B, H, Hkv, N, D;
    int32_t dtype;                 /* AA_BF16                                              */
    int32_t max_blocks;            /* last dimension of block_index (MAX_BLOCKS_PRE_ROW)   */
    double  sm_scale;              /* 0 => D^-0.5 (block_sparse_flash_attention_v2.py:341) */
    const void *q, *k, *v;
    void       *out;
    int64_t q_stride_b, q_stride_h, q_stride_n;
    int64_t k_stride_b, k_stride_h, k_stride_n;
    int64_t v_stride_b, v_stride_h, v_stride_n;
    int64_t o_stride_b, o_stride_h, o_stride_n;
    const int32_t *block_index;
    void   *workspace;             /* 256-byte aligned, >= aa_block_sparse_workspace_bytes() */
    size_t  workspace_bytes;
} aa_block_sparse_t;

int aa_block_sparse_workspace_bytes(const aa_block_sparse_t *a, size_t *bytes);
/* Two launches on `stream`: the list merge and the attention kernel. */
int aa_block_sparse_attend(const aa_block_sparse_t *a, void *stream);
/* Synchronises the stream; AA_OK, AA_ERR_DEVICE_TIMEOUT (a bounded wait gave up) or
 * AA_ERR_UNSORTED (a row of block_index was not ascending; the output is then undefined). */
int aa_block_sparse_check_status(const aa_block_sparse_t *a, void *stream);

/*
 * Dense causal attention of the last Nq positions of an Nkv-long sequence: query row i (position
 * Nkv - Nq + i) attends keys 0 .. Nkv - Nq + i.  The path of the reference's dense calls
 * (modules/llama/anchor_attention.py:76-88 for the last q_len % (block_size*step) queries of a
 * prefill, :101-113 for later chunks), which go to flash-attn there.  It is the comparator's
 * attention kernel with the key-block lists made up on the fly (every block up to the diagonal)
 * and the causal mask placed by the row's position; softmax state from empty, bf16, D = 128.
 * q, out: [B, H, Nq, D]; k, v: [B, Hkv, Nkv, D]; strides as in aa_params_t; any Nq >= 1, Nkv >= Nq
 * (rows are padded to 256 inside the kernel and never written).  `status` is a 16-byte aligned
 * device array of 4 int32 the call clears; [0] != 0 afterwards means a bounded wait gave up.
 * One launch.  A 128-row tile per row group makes it a prefill kernel: for single-token decode a
 * split-KV kernel is the right tool and the host side keeps calling the library one.
 */
typedef struct aa_dense_causal {
    int32_t B, H, Hkv, Nq, Nkv, D;
    int32_t dtype;                 /* AA_BF16 */
    double  sm_scale;              /* 0 => D^-0.5 */
    const void *q, *k, *v;
    void       *out;
    int64_t q_stride_b, q_stride_h, q_stride_n;
    int64_t k_stride_b, k_stride_h, k_stride_n;
    int64_t v_stride_b, v_stride_h, v_stride_n;
    int64_t o_stride_b, o_stride_h, o_stride_n;
    int32_t *status;
} aa_dense_causal_t;
int aa_dense_causal_attend(const aa_dense_causal_t *a, void *stream);

const char *aa_strerror(int code);
/* Text of the last CUDA error this library saw on the calling thread. */
const char *aa_last_cuda_error(void);
/* Library version, and how many of the library's kernels one aa_forward enqueues: the least (a
 * workspace whose gather scratch has a slot for every possible tile), and the number for a given
 * problem and workspace (step 3 then also enqueues its plan kernel and both of its sequences, of
 * which the kernels of one leave at once; < 0: an error code).  No counterpart in the reference. */
int aa_version(void);
int aa_launches_per_forward(void);
int aa_forward_launches(const aa_params_t *p);

#ifdef __cplusplus
}
#endif
#endif /* ANCHOR_ATTN_B200_H */

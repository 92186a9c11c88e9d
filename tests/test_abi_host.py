"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, and its host-only entry points (layout, validation, error text) behave."""
import ctypes
import os
import re

import pytest

from anchor_attention_b200 import _lib

HEADER = os.path.join(os.path.dirname(__file__), "..", "include", "anchor_attn_b200.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aa_[a-z0-9_]+)\s*\(", text)))


def _params(N=8192, H=4, Hkv=1, step=16, block=128, D=128):
    p = _lib.AAParams()
    p.B, p.H, p.Hkv, p.N, p.D = 1, H, Hkv, N, D
    p.block_size, p.step, p.dtype = block, step, _lib.AA_BF16
    p.theta = 12.0
    return p


def test_exports_every_declared_symbol(lib):
    declared = _declared_symbols()
    assert len(declared) >= 13
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.EXPORTS) == sorted(n for n in declared if n not in ("aa_params_t",))


def test_id_row_offsets(lib):
    # capacity of big block b is b*G - 256
    off = 0
    for b in range(0, 70):
        assert lib.aa_id_row_offset(128, 16, b) == off
        off += max(0, b * 2048 - 256)
    off = 0
    for b in range(0, 20):
        assert lib.aa_id_row_offset(128, 32, b) == off
        off += max(0, b * 4096 - 256)


def test_workspace_layout(lib):
    p = _params(N=131072, H=32, Hkv=8)
    lay = _lib.AALayout()
    assert lib.aa_workspace_layout(ctypes.byref(p), ctypes.byref(lay)) == 0
    n = ctypes.c_size_t()
    assert lib.aa_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == 0
    assert n.value == lay.total_bytes == lay.min_bytes + lay.gather_bytes
    offs = [lay.m_off, lay.l_off, lay.acc_off, lay.qpool_off, lay.apool_off, lay.bitmap_off, lay.counts_off,
            lay.ids_off, lay.status_off, lay.tile_slot_off, lay.gather_off, lay.total_bytes]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs)
    assert lay.l_off - lay.m_off >= 32 * 131072 * 4
    assert lay.qpool_off - lay.acc_off >= 32 * 131072 * 128 * 4
    assert lay.ids_per_head == sum(b * 2048 - 256 for b in range(1, 64))
    assert lay.status_off - lay.ids_off >= 32 * lay.ids_per_head * 4
    assert lay.min_bytes == lay.gather_off < 4 * 2 ** 30       # a few GB at the largest benchmark shape
    tiles = 32 * lay.ids_per_head // 128
    assert lay.gather_off - lay.tile_slot_off >= 4 * tiles
    assert lay.gather_bytes == min(tiles * 65536, 8 << 30)      # one 64 KB slot per id tile, capped
    small = _params(N=8192, H=4, Hkv=1)
    assert lib.aa_workspace_layout(ctypes.byref(small), ctypes.byref(lay)) == 0
    assert lay.gather_bytes == 4 * (lay.ids_per_head // 128) * 65536


@pytest.mark.parametrize("change,code", [
    (dict(D=64), -3), (dict(step=8), -4), (dict(block=32), -5), (dict(N=3000), -6),
    (dict(H=3, Hkv=2), -2), (dict(N=0), -2),
])
def test_shape_validation(lib, change, code):
    p = _params(**change)
    n = ctypes.c_size_t()
    assert lib.aa_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == code
    assert len(lib.aa_strerror(code)) > 3


def test_forward_rejects_null_and_misaligned_before_touching_cuda(lib):
    p = _params()
    assert lib.aa_forward(ctypes.byref(p), None) == -1                 # NULL q/k/v/out
    p.q = p.k = p.v = p.out = 4096
    p.q_stride_n = 130                                                 # not a multiple of 8 elements
    assert lib.aa_forward(ctypes.byref(p), None) == -8
    p.q_stride_n = 128
    assert lib.aa_forward(ctypes.byref(p), None) == -7                 # no workspace
    assert lib.aa_forward(None, None) == -1


def test_error_text_mirrors_reference_messages(lib):
    assert b"Only step sizes 16 or 32 are supported" in lib.aa_strerror(-4)
    assert b"divisible by (block_size * step)" in lib.aa_strerror(-6)
    assert lib.aa_version() >= 1 and lib.aa_launches_per_forward() >= 3


def test_python_entry_point_refuses_cpu_tensors(lib):
    import torch
    from anchor_attention_b200 import anchor_attn
    q = torch.zeros(1, 1, 2048, 128, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="no CPU path"):
        anchor_attn(q, q, q)


def test_push_entry_point_validates_its_arguments(lib):
    p = _params()
    p.q = p.k = p.v = p.out = 4096
    for name in ("q", "k", "v", "o"):
        setattr(p, f"{name}_stride_n", 128)
    push = _lib.AAPush()
    assert lib.aa_step3_sparse_push(ctypes.byref(p), None, None) == -1          # no push block
    push.n_peers = 0
    assert lib.aa_step3_sparse_push(ctypes.byref(p), ctypes.byref(push), None) == -2
    push.n_peers = _lib.MAX_PEERS + 1
    assert lib.aa_step3_sparse_push(ctypes.byref(p), ctypes.byref(push), None) == -2
    push.n_peers = 2
    push.out[0] = 4096
    assert lib.aa_step3_sparse_push(ctypes.byref(p), ctypes.byref(push), None) == -1          # out[1] is NULL
    push.out[1] = 4100
    assert lib.aa_step3_sparse_push(ctypes.byref(p), ctypes.byref(push), None) == -8          # not 16-byte aligned
    push.out[1] = 8192
    assert lib.aa_step3_sparse_push(ctypes.byref(p), ctypes.byref(push), None) == -7          # no workspace


def test_without_anchor_alias_exists():
    from anchor_attention_b200 import anchor_attn_without_anchor
    import inspect
    sig = inspect.signature(anchor_attn_without_anchor)
    assert list(sig.parameters) == ["Q", "K", "V", "sm_scale", "block_size", "step", "difference"]
    assert sig.parameters["difference"].default == 12 and sig.parameters["block_size"].default == 128


def test_ctypes_mirrors_match_the_header(tmp_path):
    """Sizes and field offsets of the ctypes structures equal what a C compiler makes of the
    header (a drifted mirror would pass wrong pointers silently)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    checks = {
        "aa_params_t": (_lib.AAParams, ["B", "D", "theta", "sm_scale", "q", "out", "q_stride_b", "o_stride_n",
                                        "workspace", "workspace_bytes"]),
        "aa_workspace_layout_t": (_lib.AALayout, ["m_off", "ids_off", "status_off", "total_bytes", "ids_per_head",
                                                  "tile_slot_off", "gather_off", "gather_bytes", "min_bytes"]),
        "aa_stripes_static_args_t": (_lib.AAStripesStaticArgs, ["B", "theta", "q", "k_stride_n", "anchors", "ids"]),
        "aa_push_t": (_lib.AAPush, ["n_peers", "rows_per_peer", "out"]),
        "aa_peer_barrier_t": (_lib.AAPeerBarrier, ["n_peers", "epoch", "timeout_ms", "flags", "status"]),
        "aa_dense_causal_t": (_lib.AADenseCausal, ["B", "Nkv", "dtype", "sm_scale", "q", "o_stride_n", "status"]),
        "aa_rope_dispatch_t": (_lib.AARopeDispatch, ["n", "dtype", "token0", "q", "v_stride_n", "cos", "dst"]),
        "aa_block_sparse_t": (_lib.AABlockSparse, ["B", "max_blocks", "sm_scale", "q", "o_stride_n", "block_index",
                                                   "workspace_bytes"]),
    }
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{os.path.abspath(HEADER)}"', "int main(void) {"]
    for cname, (_, fields) in checks.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for f in fields:
            lines.append(f'  printf("{cname} {f} %zu\\n", offsetof({cname}, {f}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    seen = 0
    for line in out.splitlines():
        cname, field, value = line.split()
        ct = checks[cname][0]
        want = ctypes.sizeof(ct) if field == "size" else getattr(ct, field).offset
        assert int(value) == want, f"{cname}.{field}: header {value}, ctypes {want}"
        seen += 1
    assert seen == sum(len(f) + 1 for _, f in checks.values())
    assert _lib.MAX_PEERS == 8 and _lib.STATIC_SCRATCH_BYTES == 8 << 20


def _block_args(**kw):
    a = _lib.AABlockSparse()
    a.B, a.H, a.Hkv, a.N, a.D = 1, 4, 2, 1024, 128
    a.dtype, a.max_blocks = _lib.AA_BF16, 5
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_block_sparse_workspace_and_validation(lib):
    """Host-only part of the comparator's entry points: workspace size and argument checks."""
    need = ctypes.c_size_t(0)
    a = _block_args()
    assert lib.aa_block_sparse_workspace_bytes(ctypes.byref(a), ctypes.byref(need)) == 0
    npairs, stride = 1024 // 256, 2 * 5
    lists = 4 * npairs * stride * 4
    assert need.value >= lists + 4 * npairs * 4 + 16 and need.value % 256 == 0
    # max_blocks beyond the block count does not grow the lists further
    big = ctypes.c_size_t(0)
    assert lib.aa_block_sparse_workspace_bytes(ctypes.byref(_block_args(max_blocks=1000)), ctypes.byref(big)) == 0
    assert big.value < 4 * npairs * 2 * 8 * 4 + 1024
    for change, code in [(dict(D=64), -3), (dict(N=1024 + 128), -6), (dict(max_blocks=0), -2), (dict(Hkv=3), -2),
                         (dict(dtype=1), -9)]:
        assert lib.aa_block_sparse_workspace_bytes(ctypes.byref(_block_args(**change)), ctypes.byref(need)) == code
    # NULL tensors and a missing workspace are refused before any CUDA call
    assert lib.aa_block_sparse_attend(ctypes.byref(_block_args()), None) == -1
    assert lib.aa_block_sparse_attend(None, None) == -1
    assert b"ascending" in lib.aa_strerror(-13)


def test_block_sparse_python_entry_refuses_cpu_tensors():
    import torch
    from anchor_attention_b200.block_sparse import block_sparse_attend
    q = torch.zeros(1, 1, 256, 128, dtype=torch.bfloat16)
    idx = torch.zeros(1, 1, 2, 1, dtype=torch.int32)
    with pytest.raises(AssertionError, match="CUDA"):
        block_sparse_attend(q, q, q, idx)


def test_new_entry_points_validate_before_touching_cuda(lib):
    """The barrier, the rotary dispatch, the dense causal variant and the list validator refuse
    bad arguments on the host, before any CUDA call."""
    assert lib.aa_peer_barrier(None, None) == -1
    b = _lib.AAPeerBarrier()
    b.n_peers, b.rank = 2, 0
    assert lib.aa_peer_barrier(ctypes.byref(b), None) == -1            # no status word
    b.status = 4096
    b.n_peers = _lib.MAX_PEERS + 1
    assert lib.aa_peer_barrier(ctypes.byref(b), None) == -2
    b.n_peers, b.rank = 2, 5
    assert lib.aa_peer_barrier(ctypes.byref(b), None) == -2
    b.rank = 1
    assert lib.aa_peer_barrier(ctypes.byref(b), None) == -1            # NULL flag arrays

    assert lib.aa_rope_dispatch(None, None) == -1
    r = _lib.AARopeDispatch()
    r.n, r.H, r.Hkv, r.D, r.n_peers = 16, 8, 4, 128, 3                 # 3 ranks do not divide the heads
    assert lib.aa_rope_dispatch(ctypes.byref(r), None) == -2
    r.n_peers, r.D = 2, 64
    assert lib.aa_rope_dispatch(ctypes.byref(r), None) == -3
    r.D = 128
    assert lib.aa_rope_dispatch(ctypes.byref(r), None) == -1           # NULL tensors

    assert lib.aa_dense_causal_attend(None, None) == -1
    d = _lib.AADenseCausal()
    d.B, d.H, d.Hkv, d.Nq, d.Nkv, d.D = 1, 4, 2, 300, 200, 128         # more queries than keys
    assert lib.aa_dense_causal_attend(ctypes.byref(d), None) == -2
    d.Nkv, d.D = 4000, 64
    assert lib.aa_dense_causal_attend(ctypes.byref(d), None) == -3
    d.D = 128
    assert lib.aa_dense_causal_attend(ctypes.byref(d), None) == -1     # NULL tensors / status

    assert lib.aa_validate_lists(None, None) == -1
    assert lib.aa_validate_lists(ctypes.byref(_params()), None) == -1  # NULL q/k/v/out
    assert b"malformed" in lib.aa_strerror(-14)

    push = _lib.AAPush()
    p = _params()
    p.q = p.k = p.v = p.out = 4096
    for name in ("q", "k", "v", "o"):
        setattr(p, f"{name}_stride_n", 128)
    push.n_peers, push.rows_per_peer = 2, 100                           # not a multiple of the tile height
    push.out[0] = push.out[1] = 4096
    assert lib.aa_step3_sparse_push(ctypes.byref(p), ctypes.byref(push), None) == -2
    push.rows_per_peer = 2048                                           # 2 x 2048 rows do not cover N = 8192
    assert lib.aa_step3_sparse_push(ctypes.byref(p), ctypes.byref(push), None) == -2


def test_forward_launch_count_follows_the_step3_layout(lib):
    """aa_forward_launches only looks at sizes: with a slot for every possible tile step 3 is a gather
    pass and one attention launch (6 kernels in all); without any scratch the attention kernel alone;
    with a scratch that the lists may outgrow, the plan kernel plus both sequences."""
    import ctypes

    def count(N, H, Hkv, scratch):
        p = _params(N=N, H=H, Hkv=Hkv)
        lay = _lib.AALayout()
        assert lib.aa_workspace_layout(ctypes.byref(p), ctypes.byref(lay)) == 0
        for name in "qkv":
            setattr(p, name, 0x10000)
        p.out = 0x10000
        for t in "qkvo":
            setattr(p, f"{t}_stride_b", H * N * 128)
            setattr(p, f"{t}_stride_h", N * 128)
            setattr(p, f"{t}_stride_n", 128)
        p.workspace = 0x100000
        p.workspace_bytes = lay.min_bytes + (lay.gather_bytes if scratch is None else scratch)
        return lib.aa_forward_launches(ctypes.byref(p)), lay

    assert count(32768, 32, 8, None)[0] == 6
    assert count(32768, 32, 8, 0)[0] == 5
    assert count(2048, 2, 1, None)[0] == 4                      # one big block: no candidates, no score kernel
    n, lay = count(131072, 32, 8, None)                         # capped scratch: 8 parts of one KV head
    assert lay.gather_bytes < 32 * (lay.ids_per_head // 128) * 65536
    assert n == 4 + 1 + 3 * (1 + 8)
    assert lib.aa_forward_launches(None) < 0

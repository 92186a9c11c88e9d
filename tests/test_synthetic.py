"""The package's synthetic-input generator equals the oracle's (same seed, same bits)."""
import torch

from anchor_attention_b200.synthetic import make_inputs as make_pkg
from oracle.anchor_oracle import make_inputs as make_oracle


def test_generators_agree():
    for kw in (dict(seed=0, rope=True), dict(seed=3, rope=False, q_shift=0.5)):
        a = make_pkg(4096, 4, 2, **kw)
        b = make_oracle(4096, 4, 2, **kw)
        assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_head_slice_is_a_slice_of_the_full_draw():
    full = make_pkg(2048, 8, 4, seed=0)
    part = make_pkg(2048, 8, 4, seed=0, heads=(2, 4, 1, 2))
    assert torch.equal(part[0], full[0][:, 2:4]) and torch.equal(part[1], full[1][:, 1:2])
    assert torch.equal(part[2], full[2][:, 1:2])

"""Host logic of the module hook, on CPU: configuration handling and the routing of
tokens between the sparse operator and the dense tail.  The operator itself is
replaced by the CPU oracle here (the product path has no CPU implementation)."""
import types

import pytest
import torch

from anchor_attention_b200 import patch
from oracle.anchor_oracle import anchor_attn_oracle, dense_causal_attention, make_inputs


def test_defaults_match_reference():
    assert patch.get_config_example("anchor_attn") == {"block_size_M": 128, "theta": 12, "step": 16}
    assert patch.get_config_example("anchor_attn_lite") == patch.get_config_example("anchor_attn")


def test_config_merging_and_json():
    assert patch.resolve_config("anchor_attn", {"theta": 10}) == {"block_size_M": 128, "theta": 10, "step": 16}
    assert patch.resolve_config("anchor_attn", '{"step": 32}')["step"] == 32
    with pytest.raises(ValueError, match="not valid JSON"):
        patch.resolve_config("anchor_attn", "{theta: 1")
    with pytest.raises(ValueError, match="Unsupported attention pattern"):
        patch.resolve_config("flex_prefill", None)


def test_patch_model_config_writes_attributes():
    model = types.SimpleNamespace(config=types.SimpleNamespace())
    patch.patch_model_config(model, "anchor_attn", {"theta": 9})
    assert (model.config.block_size_M, model.config.theta, model.config.step) == (128, 9, 16)


def test_patch_model_rejects_non_hf_objects():
    with pytest.raises(ValueError, match="Only Hugging Face"):
        patch.patch_model(object(), "anchor_attn")


def _oracle_op(Q, K, V, sm_scale, block, step, theta, ratio):
    return anchor_attn_oracle(Q, K, V, sm_scale, block, step, theta, mode="bf16", keep_state=False).out.to(Q.dtype)


def _module(theta=10.0):
    return types.SimpleNamespace(config=types.SimpleNamespace(block_size_M=128, step=16, theta=theta))


@pytest.mark.parametrize("q_len", [4096, 4096 + 77, 1000])
def test_prefill_routing(q_len):
    """pad == 0: everything sparse (the reference's empty-slice bug is not
    reproduced); pad > 0: sparse head + dense causal tail; q_len < 2048: all dense."""
    H, Hkv = 2, 1
    Q, K, V = make_inputs(4096 + 2048, H, Hkv, seed=11, rope=True, q_shift=0.5)
    Q, K, V = Q[:, :, :q_len], K[:, :, :q_len], V[:, :, :q_len]
    out, w = patch.anchor_attention_forward(_module(), Q, K, V, None, scaling=128 ** -0.5, anchor_attn_fn=_oracle_op)
    assert w is None and out.shape == (1, q_len, H, 128)
    n_sparse = q_len - q_len % 2048
    if n_sparse:
        want = _oracle_op(Q[:, :, :n_sparse], K[:, :, :n_sparse], V[:, :, :n_sparse], None, 128, 16, 10.0, False)
        assert torch.equal(out[:, :n_sparse].transpose(1, 2), want)
    if n_sparse < q_len:
        dense = dense_causal_attention(Q, K, V)[:, :, n_sparse:]
        got = out[:, n_sparse:].transpose(1, 2).float()
        assert (got - dense).abs().max() < 2e-2


def test_decode_and_chunked_prefill_are_dense():
    H, Hkv = 2, 1
    Q, K, V = make_inputs(4096, H, Hkv, seed=12, rope=False)
    called = []

    def never(*a):
        called.append(1)
        raise AssertionError("sparse operator must not run")

    out, _ = patch.anchor_attention_forward(_module(), Q[:, :, -1:], K, V, None, scaling=128 ** -0.5,
                                            anchor_attn_fn=never)
    dense = dense_causal_attention(Q, K, V)[:, :, -1:]
    assert (out.transpose(1, 2).float() - dense).abs().max() < 2e-2 and not called
    out, _ = patch.anchor_attention_forward(_module(), Q[:, :, -2048:], K, V, None, scaling=128 ** -0.5,
                                            anchor_attn_fn=never)
    assert (out.transpose(1, 2).float() - dense_causal_attention(Q, K, V)[:, :, -2048:]).abs().max() < 2e-2


def test_dense_path_is_chunked_and_equal(monkeypatch):
    """The dense path runs in query chunks (bounded mask); the chunks together equal one call."""
    H, Hkv = 2, 1
    Q, K, V = make_inputs(2048, H, Hkv, seed=13, rope=False)
    whole = patch._dense_causal(Q[:, :, -700:], K, V, 128 ** -0.5, 2048 - 700)
    monkeypatch.setattr(patch, "DENSE_CHUNK", 256)
    parts = patch._dense_causal(Q[:, :, -700:], K, V, 128 ** -0.5, 2048 - 700)
    assert parts.shape == whole.shape and (parts.float() - whole.float()).abs().max() < 1e-2
    dense = dense_causal_attention(Q, K, V)[:, :, -700:]
    assert (parts.float() - dense).abs().max() < 2e-2


def test_sliding_window_models_are_refused():
    from transformers import MistralConfig, MistralForCausalLM
    cfg = MistralConfig(vocab_size=64, hidden_size=64, intermediate_size=64, num_hidden_layers=1,
                        num_attention_heads=2, num_key_value_heads=1, head_dim=32, sliding_window=128)
    model = MistralForCausalLM(cfg)
    with pytest.raises(ValueError, match="sliding attention window"):
        patch.patch_model(model, "anchor_attn")

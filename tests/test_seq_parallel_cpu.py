"""Sequence-parallel prefill host logic on two CPU ranks (gloo): token-sharded dense layers,
the tokens->heads and heads->tokens exchanges, last-token logits on every rank.  The CUDA
operator is replaced by the CPU oracle (``attn_fn``), so this tests the partitioning and the
exchanges, not the kernels; the result must equal the same model run in one process."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

N_TOKENS = 4096


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tiny_model():
    from transformers import LlamaConfig, LlamaForCausalLM
    from anchor_attention_b200 import patch
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=128, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=8192,
                      rope_theta=500000.0)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    patch.patch_model_config(model, "anchor_attn", {"theta": 10})
    return model


def _oracle_heads(Q, K, V, theta=10.0):
    """[1,h,N,D] heads -> [1,N,h,D] through the CPU restatement."""
    from oracle.anchor_oracle import anchor_attn_oracle
    out = anchor_attn_oracle(Q, K, V, None, 128, 16, theta, mode="bf16", keep_state=False).out
    return out.to(Q.dtype).transpose(1, 2).contiguous()


def _single_process_logits(model, ids):
    """The same model in one process: HF's own forward with the oracle as attention function."""
    from transformers import AttentionInterface

    def attn(module, query, key, value, attention_mask=None, scaling=None, dropout=0.0, **kw):
        return _oracle_heads(query, key, value), None

    AttentionInterface.register("anchor_attn_cpu_check", attn)
    model.config._attn_implementation = "anchor_attn_cpu_check"
    with torch.no_grad():
        return model(input_ids=ids, use_cache=False, logits_to_keep=1).logits.float()


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from anchor_attention_b200.seq_parallel import SequenceParallelPrefill
        model = _tiny_model()
        g = torch.Generator().manual_seed(5)
        ids = torch.randint(0, 128, (1, N_TOKENS), generator=g)
        sp = SequenceParallelPrefill(model, attn_fn=_oracle_heads)
        logits = sp(ids)
        ret[rank] = logits
    finally:
        dist.destroy_process_group()


def test_two_ranks_equal_one_process():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        got0, got1 = ret[0], ret[1]
    assert torch.equal(got0, got1)                     # every rank ends with the same logits
    model = _tiny_model()
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 128, (1, N_TOKENS), generator=g)
    want = _single_process_logits(model, ids)
    assert got0.shape == want.shape == (1, 1, 128)
    # GEMMs over half the rows may round differently in bf16; the logits are of order one
    assert (got0 - want).abs().max() < 5e-2


def test_rejects_lengths_that_do_not_shard():
    import pytest

    class FakeGroup:
        pass
    from anchor_attention_b200 import seq_parallel
    model = _tiny_model()
    sp = seq_parallel.SequenceParallelPrefill.__new__(seq_parallel.SequenceParallelPrefill)
    sp.model, sp.W, sp.rank, sp.block, sp.step = model, 2, 0, 128, 16
    with pytest.raises(ValueError, match="multiple of"):
        sp(torch.zeros((1, 3000), dtype=torch.long))

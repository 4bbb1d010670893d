"""Checkpoint round trips on CPU: our SafeTensors layout loads back bit-exactly, loads with
``transformers.from_pretrained`` and reproduces our logits there; interrupted saves stay invisible."""

import os

import numpy as np
import pytest
import torch

from halo_b200.checkpoint.atomic import atomic_write_json, staged_path
from halo_b200.checkpoint.load import from_pretrained, load_model_weights
from halo_b200.checkpoint.save import is_complete, mark_complete, save_model
from halo_b200.data.packing import pack_documents
from halo_b200.models.config import ModelConfig, tiny_moe_config
from halo_b200.models.qwen3 import build_model


def test_round_trip_is_exact_and_sharded(tmp_path):
    cfg = tiny_moe_config()
    model = build_model(cfg, device="cpu", seed=3)
    d = str(tmp_path / "ckpt")
    save_model(model, d, save_dtype=None, max_shard_bytes=4 * 1024 * 1024)
    assert os.path.exists(os.path.join(d, "model.safetensors.index.json"))
    assert not is_complete(d)
    mark_complete(d, {"global_step": 7})
    assert is_complete(d)
    back = from_pretrained(d, device="cpu", dtype=torch.float32)
    for (n, a), (_, b) in zip(model.named_parameters(), back.named_parameters()):
        assert torch.equal(a, b), n


def test_missing_tensor_is_refused(tmp_path):
    cfg = tiny_moe_config()
    model = build_model(cfg, device="cpu", seed=3)
    d = str(tmp_path / "ckpt")
    save_model(model, d, save_dtype=None)
    cfg2 = ModelConfig.from_hf_dict(cfg.to_hf_dict())
    cfg2.num_hidden_layers = 5
    bigger = build_model(cfg2, device="cpu", seed=0)
    with pytest.raises(KeyError):
        load_model_weights(bigger, d)


def test_interrupted_write_leaves_no_file(tmp_path):
    target = str(tmp_path / "x.json")
    atomic_write_json(target, {"a": 1})
    with pytest.raises(RuntimeError):
        with staged_path(target) as tmp:
            open(tmp, "w").write("partial")
            raise RuntimeError("crash")
    assert open(target).read().strip().startswith("{")
    assert [f for f in os.listdir(tmp_path) if f.startswith(".staged-")] == []


@pytest.mark.parametrize("moe", [True, False])
def test_transformers_loads_our_checkpoint_and_agrees(tmp_path, moe):
    transformers = pytest.importorskip("transformers")
    if moe:
        cfg = tiny_moe_config()
    else:
        cfg = ModelConfig(vocab_size=1024, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=32, intermediate_size=256, num_experts=0, model_type="qwen3")
    model = build_model(cfg, device="cpu", seed=1, gradient_checkpointing=False)
    d = str(tmp_path / "hf")
    save_model(model, d, save_dtype=None)
    hf = transformers.AutoModelForCausalLM.from_pretrained(d, torch_dtype=torch.float32, attn_implementation="eager")
    hf.eval()
    ids = np.random.default_rng(0).integers(0, cfg.vocab_size, size=48)
    b = pack_documents([ids])
    with torch.no_grad():
        ours = model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens) @ model.head_weight().t()
        theirs = hf(input_ids=b.input_ids[None]).logits[0]
    assert (ours - theirs).abs().max().item() < 5e-2 * theirs.abs().max().item()


def test_reward_model_saves_as_sequence_classification(tmp_path):
    """A model with a sequence-level head is saved as the family's sequence-classification architecture; ``transformers``
    loads it and scores a document as we do; the trainer can resume from it."""
    transformers = pytest.importorskip("transformers")
    from halo_b200.trainers.reward import SequenceHead, _WithHead

    cfg = ModelConfig(vocab_size=1024, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=32, intermediate_size=256, moe_intermediate_size=0, num_experts=0, model_type="qwen3")
    model = build_model(cfg, device="cpu", seed=1, gradient_checkpointing=False)
    head = SequenceHead(cfg.hidden_size, 3)
    wrapped = _WithHead(model, head)
    d = str(tmp_path / "rm")
    save_model(wrapped, d, save_dtype=None)
    hf = transformers.AutoModelForSequenceClassification.from_pretrained(d, dtype=torch.float32, attn_implementation="eager").eval()
    assert type(hf).__name__ == "Qwen3ForSequenceClassification" and hf.config.num_labels == 3
    ids = np.random.default_rng(0).integers(1, cfg.vocab_size, size=40)          # no pad token inside
    b = pack_documents([ids])
    with torch.no_grad():
        ours = head(model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens), b.cu_seqlens)[0]
        theirs = hf(input_ids=b.input_ids[None]).logits[0]
    assert torch.allclose(ours, theirs, atol=1e-4)
    again = _WithHead(build_model(cfg, device="cpu", seed=9, gradient_checkpointing=False), SequenceHead(cfg.hidden_size, 3))
    load_model_weights(again, d)
    assert torch.equal(again.head.score.weight, head.score.weight)

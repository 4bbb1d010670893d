"""The transformers-facing surface on CPU: the decoder as a ``PreTrainedModel`` (padded batches in, ``CausalLMOutput``
out, hub-layout ``save_pretrained`` / ``from_pretrained``) against the packed-row model underneath and against
``transformers``' own implementation of the same family."""

import dataclasses

import numpy as np
import pytest
import torch

from halo_b200.data.packing import pack_documents
from halo_b200.models.config import PRESETS
from halo_b200.models.hf import HaloConfig, HaloForCausalLM, pack_padded_batch


def _tiny():
    return dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=2, vocab_size=512)


def test_padded_batch_equals_packed_rows():
    cfg = _tiny()
    m = HaloForCausalLM(HaloConfig(cfg), device="cpu", dtype=torch.float32, seed=0)
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 512, size=n) for n in (9, 17, 5)]
    S = max(len(d) for d in docs)
    ids = torch.zeros(3, S, dtype=torch.long)
    mask = torch.zeros(3, S, dtype=torch.long)
    for i, d in enumerate(docs):                       # one row left-padded, the others right-padded
        if i == 1:
            ids[i, :len(d)] = torch.from_numpy(d)
            mask[i, :len(d)] = 1
        else:
            ids[i, S - len(d):] = torch.from_numpy(d)
            mask[i, S - len(d):] = 1
    labels = torch.where(mask.bool(), ids, torch.full_like(ids, -100))
    out = m(input_ids=ids, attention_mask=mask, labels=labels, return_logits=True)
    packed = pack_documents(docs)
    want = m.model(packed.input_ids, packed.position_ids, packed.cu_seqlens, packed.labels)
    assert torch.allclose(out.loss, want, atol=1e-5)
    assert out.logits.shape == (3, S, 512)
    # logits of the padded positions are zero, the others equal the packed model's
    h = m.model.hidden_states(packed.input_ids, packed.position_ids, packed.cu_seqlens)
    flat = h.float() @ m.model.head_weight().float().t()
    assert torch.allclose(out.logits[mask.bool()], flat, atol=1e-5)
    assert out.logits[~mask.bool()].abs().max() == 0
    # the trainer's global item count as the normaliser: the loss becomes a share of that count
    n = int((pack_padded_batch(ids, mask, labels)[3] != -100).sum())
    share = m(input_ids=ids, attention_mask=mask, labels=labels, num_items_in_batch=2 * n).loss
    assert torch.allclose(share * 2, out.loss, atol=1e-5)
    out.loss.backward()
    assert all(p.grad is not None for _, p in m.named_parameters())


def test_save_pretrained_round_trip_and_transformers_parity(tmp_path):
    cfg = _tiny()
    m = HaloForCausalLM(HaloConfig(cfg), device="cpu", dtype=torch.float32, seed=3)
    m.save_pretrained(str(tmp_path / "ckpt"))
    again = HaloForCausalLM.from_pretrained(str(tmp_path / "ckpt"), device="cpu", dtype=torch.float32)
    for (n, a), (_, b) in zip(m.named_parameters(), again.named_parameters()):
        assert torch.equal(a, b), n
    assert again.config.to_dict()["model_type"] == "qwen3_moe"
    ids = torch.randint(0, 512, (2, 12))
    mine = again(input_ids=ids, labels=ids, return_logits=True)
    transformers = pytest.importorskip("transformers")
    try:
        theirs_model = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ckpt"), torch_dtype=torch.float32)
    except Exception as exc:  # noqa: BLE001 - a transformers build without this family
        pytest.skip(f"transformers cannot load the family here: {type(exc).__name__}")
    theirs = theirs_model(input_ids=ids, labels=ids)
    assert torch.allclose(mine.logits, theirs.logits, atol=2e-4), (mine.logits - theirs.logits).abs().max()
    assert torch.allclose(mine.loss, theirs.loss, atol=1e-4)


class _StockLoop:
    """The seams of ``transformers.Trainer``'s inner loop, reduced to what a subclass can rely on: the model and the
    arguments are attributes, ``create_optimizer`` runs before the first step, every micro-batch goes through
    ``training_step(model, inputs, num_items_in_batch)``, then ``optimizer.step()``, the scheduler and ``zero_grad``.
    (``transformers.Trainer`` itself cannot be constructed where ``accelerate`` is not installed.)"""

    def __init__(self, model=None, args=None, train_batches=None, **kw):
        self.model, self.args, self.train_batches = model, args, train_batches
        self.optimizer = None
        self.lr_scheduler = None
        self.log = []

    def train(self):
        self.create_optimizer()
        for inputs in self.train_batches:
            n = int((inputs["labels"][:, 1:] != -100).sum())
            loss = self.training_step(self.model, inputs, num_items_in_batch=n)
            self.optimizer.step()
            self.optimizer.zero_grad()
            self.log.append(float(loss))
        return self.log


def test_mixin_drives_the_engine_through_the_stock_loop_seams(tmp_path):
    """The loop above with the mixin in front of it follows the loss curve of the framework's own trainer on the same
    rows, and ``save_model`` writes a checkpoint the loaders read back."""
    from types import SimpleNamespace

    from halo_b200.configs.arguments import TrainingArguments
    from halo_b200.trainers.hf_trainer import EngineOptimizer, hf_trainer_class
    from halo_b200.trainers.sft import SFTTrainer

    cfg = _tiny()
    rng = np.random.default_rng(4)
    rows = [[rng.integers(0, 512, size=n) for n in (11, 7, 14)] for _ in range(4)]

    def padded(docs):
        S = max(len(d) for d in docs)
        ids = torch.zeros(len(docs), S, dtype=torch.long)
        mask = torch.zeros(len(docs), S, dtype=torch.long)
        for i, d in enumerate(docs):
            ids[i, :len(d)] = torch.from_numpy(d)
            mask[i, :len(d)] = 1
        return {"input_ids": ids, "attention_mask": mask, "labels": torch.where(mask.bool(), ids, torch.full_like(ids, -100))}

    cls = hf_trainer_class(_StockLoop, "DistributedStockLoop")
    hf_model = HaloForCausalLM(HaloConfig(cfg), device="cpu", dtype=torch.float32, seed=0)
    args = SimpleNamespace(learning_rate=1e-3, weight_decay=0.0, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8,
                           max_grad_norm=0.5, output_dir=str(tmp_path / "out"))
    t = cls(model=hf_model, args=args, train_batches=[padded(r) for r in rows], halo_optim="adamw_torch")
    got = t.train()
    assert isinstance(t.optimizer, EngineOptimizer) and args.max_grad_norm == 0.0 and t.engine.max_grad_norm == 0.5

    own_model = HaloForCausalLM(HaloConfig(cfg), device="cpu", dtype=torch.float32, seed=0).model
    own = SFTTrainer(own_model, TrainingArguments(output_dir="unused", learning_rate=1e-3, weight_decay=0.0, max_grad_norm=0.5,
                                                  optim="adamw_torch", lr_scheduler_type="constant", logging_steps=1),
                     [pack_documents(r) for r in rows], device="cpu")
    want = [l["loss"] for l in own.train()["log_history"]]
    assert np.allclose(got, want, atol=1e-5), (got, want)
    for (n, a), (_, b) in zip(hf_model.named_parameters(), own_model.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6), n
    t.save_model()
    again = HaloForCausalLM.from_pretrained(args.output_dir, device="cpu", dtype=torch.float32)
    for (n, a), (_, b) in zip(hf_model.named_parameters(), again.named_parameters()):
        assert torch.allclose(a.bfloat16().float(), b, atol=1e-6), n

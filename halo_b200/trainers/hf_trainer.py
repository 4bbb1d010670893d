"""The ``transformers`` / TRL trainer surface over the framework's training engine.

``DistributedTrainerMixin`` goes in front of ``transformers.Trainer`` (or a TRL trainer) in a class's bases and
overrides exactly the seams the stock loop calls - ``create_optimizer``, ``compute_loss``, ``training_step``,
``save_model`` and the optimizer-state checkpoint hooks - so that the stock loop (data loaders, callbacks, logging,
schedules, ``TrainerState``) drives :class:`halo_b200.trainers.engine.TrainEngine`:

* ``create_optimizer`` builds the framework's optimizer (AdamWBF16 by default) over the inner model's named
  parameters and hands the loop an :class:`EngineOptimizer`: its ``step()`` is the engine's gradient synchronisation,
  device-side global-norm clip, non-finite guard and optimizer step in one; the loop's own clipping is switched off.
* ``training_step`` packs the collator's padded batch into one token stream, normalises the loss by the token count
  summed over the data-parallel ranks (the loop's ``num_items_in_batch`` when it supplies one), runs backward and
  returns the detached loss; gradients accumulate across micro-batches exactly as the stock loop expects.
* ``save_model`` writes the hub layout through the gathered writers (collective when experts are sharded), and the
  optimizer shards / RNG sidecars are written per rank beside it.

``hf_trainer_class(base)`` assembles such a class for any base; ``DistributedSFTTrainer`` is that for
``transformers.Trainer`` (TRL's ``SFTTrainer`` when it is importable). ``transformers.Trainer`` itself refuses to
construct without ``accelerate``; the mixin imports without it, so everything below is usable (and tested) with any
loop that keeps the same seams.

Counterpart of halo/trainers/distributed_trainer.py:175-301 (``DistributedTrainerMixin``) and halo/trainers/sft.py:92-148
(``DistributedSFTTrainer(DistributedTrainerMixin, SFTTrainer)``).
"""

from __future__ import annotations

import os

import torch

from halo_b200.data.packing import PackedBatch
from halo_b200.optim.factory import build_optimizer
from halo_b200.trainers.engine import TrainEngine


class EngineOptimizer(torch.optim.Optimizer):
    """What the stock loop sees as "the optimizer": ``step()`` runs the engine's synchronise / clip / guard / update,
    ``zero_grad()`` is a no-op after a step (the engine already dropped the gradients), ``param_groups`` and
    ``state_dict`` are the real optimizer's, so schedulers and checkpoints work on it unchanged."""

    def __init__(self, engine: TrainEngine):
        self.engine = engine
        self.inner = engine.optimizer
        self.defaults = self.inner.defaults
        self.state = self.inner.state
        self.param_groups = self.inner.param_groups
        self._optimizer_step_pre_hooks, self._optimizer_step_post_hooks = {}, {}

    def step(self, closure=None):
        self.engine.clip_and_step()
        self.engine.step_count += 1

    def zero_grad(self, set_to_none: bool = True):
        self.inner.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return self.inner.state_dict()

    def load_state_dict(self, sd):
        return self.inner.load_state_dict(sd)


def _inner(model):
    """The packed-row model behind a ``HaloForCausalLM`` (or the model itself)."""
    return getattr(model, "model", model) if hasattr(getattr(model, "model", None), "cfg") else model


class DistributedTrainerMixin:
    """See the module docstring. Extra constructor keywords: ``parallel`` (a ``ParallelRuntime``), ``halo_optim`` (optimizer
    name of :mod:`halo_b200.optim.factory`), ``max_grad_norm`` is read from ``args``."""

    def __init__(self, *args, parallel=None, halo_optim: str | None = None, **kw):
        self.parallel = parallel
        self.halo_optim = halo_optim
        self.engine: TrainEngine | None = None
        super().__init__(*args, **kw)
        targs = getattr(self, "args", None)
        if targs is not None and getattr(targs, "max_grad_norm", None):
            # the engine clips by the global norm over every parallel axis; the loop's own (local) clip must not run too
            self._engine_max_grad_norm = float(targs.max_grad_norm)
            try:
                targs.max_grad_norm = 0.0
            except Exception:  # noqa: BLE001 - frozen argument objects keep their value; the engine's clip is idempotent
                pass
        else:
            self._engine_max_grad_norm = 0.0

    # ---- construction ----------------------------------------------------------------------------
    def _device(self):
        return next(_inner(self.model).parameters()).device

    def create_optimizer(self, *a, **kw):
        if getattr(self, "optimizer", None) is not None and isinstance(self.optimizer, EngineOptimizer):
            return self.optimizer
        targs = self.args
        inner = _inner(self.model)
        dev = self._device()
        name = self.halo_optim or ("adamw_bf16" if next(inner.parameters()).dtype == torch.bfloat16 else "adamw_torch")
        opt = build_optimizer(inner, name, lr=targs.learning_rate, weight_decay=getattr(targs, "weight_decay", 0.0),
                              betas=(getattr(targs, "adam_beta1", 0.9), getattr(targs, "adam_beta2", 0.999)),
                              eps=getattr(targs, "adam_epsilon", 1e-8))
        self.engine = TrainEngine(inner, opt, dev, max_grad_norm=self._engine_max_grad_norm, parallel=self.parallel)
        self.optimizer = EngineOptimizer(self.engine)
        return self.optimizer

    # ---- one micro-batch -------------------------------------------------------------------------
    def _packed(self, inputs) -> PackedBatch:
        """The collator's output as a packed row: padded ``[B, S]`` tensors are packed here; a ``PackedBatch`` (the
        framework's own collators) passes through."""
        if isinstance(inputs, PackedBatch):
            return inputs
        from halo_b200.models.hf import pack_padded_batch

        ids, pos, cu, labels, _ = pack_padded_batch(inputs["input_ids"], inputs.get("attention_mask"), inputs.get("labels"))
        n_scored = int((labels != -100).sum()) if labels is not None else 0
        return PackedBatch(ids, pos, labels, cu, n_scored)

    def compute_loss(self, model, inputs, return_outputs: bool = False, num_items_in_batch=None):
        batch = self._packed(inputs)
        dbatch = self.engine.to_device(batch)
        if num_items_in_batch is not None:
            normalizer = num_items_in_batch if torch.is_tensor(num_items_in_batch) else float(num_items_in_batch)
        else:
            normalizer = self.engine.global_scored_tokens(batch)
        loss = self.engine.compute_loss(dbatch, normalizer)
        return (loss, None) if return_outputs else loss

    def training_step(self, model, inputs, num_items_in_batch=None):
        if self.engine is None:
            self.create_optimizer()
        _inner(model).train()
        loss = self.compute_loss(model, inputs, num_items_in_batch=num_items_in_batch)
        loss.backward()
        return loss.detach()

    # ---- saving ------------------------------------------------------------------------------------
    def save_model(self, output_dir: str | None = None, _internal_call: bool = False):
        from halo_b200.checkpoint.save import save_model

        output_dir = output_dir or self.args.output_dir
        os.makedirs(output_dir, exist_ok=True)
        group = self.parallel.dp_group if self.parallel is not None else None
        save_model(_inner(self.model), output_dir, group=group)

    def _save_optimizer_and_scheduler(self, output_dir: str):
        from halo_b200.checkpoint import optimizer_state as opt_io

        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        opt_io.save_optimizer_shard(self.engine.optimizer, output_dir, rank, {"world_size": world}, write_meta=rank == 0)
        if rank == 0 and getattr(self, "lr_scheduler", None) is not None:
            torch.save(self.lr_scheduler.state_dict(), os.path.join(output_dir, "scheduler.pt"))

    def _load_optimizer_and_scheduler(self, checkpoint: str | None):
        if not checkpoint:
            return
        from halo_b200.checkpoint import optimizer_state as opt_io

        if self.engine is None:
            self.create_optimizer()
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        opt_io.load_optimizer_shard(self.engine.optimizer, checkpoint, rank, {"world_size": world}, False)
        sched = os.path.join(checkpoint, "scheduler.pt")
        if os.path.isfile(sched) and getattr(self, "lr_scheduler", None) is not None:
            self.lr_scheduler.load_state_dict(torch.load(sched, weights_only=False))


def hf_trainer_class(base: type, name: str | None = None) -> type:
    """``class <name>(DistributedTrainerMixin, base)``: the mixin in front of any trainer that keeps the
    ``transformers.Trainer`` seams (a TRL trainer, ``transformers.Trainer`` itself)."""
    return type(name or f"Distributed{base.__name__}", (DistributedTrainerMixin, base), {"__doc__": DistributedTrainerMixin.__doc__})


def _default_base():
    try:
        from trl import SFTTrainer as base          # the TRL base when it is installed
    except Exception:  # noqa: BLE001
        from transformers import Trainer as base
    return base


def __getattr__(attr):
    # built on first use: importing this module must not import the trainer stack of transformers
    if attr == "DistributedSFTTrainer":
        cls = hf_trainer_class(_default_base(), "DistributedSFTTrainer")
        globals()[attr] = cls
        return cls
    raise AttributeError(attr)

"""The framework's decoder behind the ``transformers`` model interface.

``HaloForCausalLM`` is a ``PreTrainedModel``: it is constructed from a ``PretrainedConfig``, takes the padded
``input_ids`` / ``attention_mask`` / ``labels`` batches every ``transformers`` / TRL trainer produces and returns a
``CausalLMOutput``, while the computation underneath is the packed-row model of :mod:`halo_b200.models.qwen3` on the
sm_100a kernels: the padded batch is packed into one token stream with document boundaries (no padding token is ever
multiplied), and the loss comes from the fused linear + cross-entropy, so no ``[tokens, vocab]`` logits exist unless the
caller asks for them. ``from_pretrained`` / ``save_pretrained`` read and write the standard hub layout through the
lazy per-rank loaders and the gathered writers of :mod:`halo_b200.checkpoint`, so a directory written here loads with
``transformers.AutoModelForCausalLM`` of the same family and the other way round.

The reference reaches the same seam from the other side: it keeps the ``transformers`` model classes and patches their
attention, MoE block and loss (halo/model_loading/loaders.py:106-165, halo/models/attention/selection.py:383-462,
halo/distributed/expert_parallel/moe_layer/layer.py:301-342).
"""

from __future__ import annotations

import os

import torch
from transformers import PretrainedConfig, PreTrainedModel
from transformers.modeling_outputs import CausalLMOutput

from halo_b200.models.config import ModelConfig
from halo_b200.models.qwen3 import build_model


class HaloConfig(PretrainedConfig):
    """``PretrainedConfig`` view of a :class:`ModelConfig`. ``to_dict`` is the hub ``config.json`` of the model's own
    family (``qwen3_moe``, ``qwen3`` ...), so what ``save_pretrained`` writes is what ``transformers`` expects."""

    model_type = "halo_b200"

    def __init__(self, model_config: ModelConfig | dict | None = None, **kw):
        if isinstance(model_config, dict):
            model_config = ModelConfig.from_hf_dict(model_config)
        if model_config is None and "hidden_size" in kw:
            model_config = ModelConfig.from_hf_dict(kw)
        self.model_config = model_config
        hf = model_config.to_hf_dict() if model_config is not None else {}
        passthrough = {k: v for k, v in kw.items() if k not in hf}
        super().__init__(**passthrough)
        for k, v in hf.items():
            if k not in ("model_type", "architectures"):
                setattr(self, k, v)
        self.family = hf.get("model_type", "")

    def to_dict(self) -> dict:
        if self.model_config is None:
            return super().to_dict()
        return dict(self.model_config.to_hf_dict())

    @classmethod
    def from_pretrained(cls, directory, **kw):
        return cls(ModelConfig.load(directory))

    def save_pretrained(self, directory, **kw):
        self.model_config.save(directory)


def pack_padded_batch(input_ids: torch.Tensor, attention_mask: torch.Tensor | None, labels: torch.Tensor | None,
                      shift_labels: bool = True):
    """A right- or left-padded ``[B, S]`` batch as one packed stream: ``(ids [T], position_ids [T], cu_seqlens (host
    int64 [B+1]), labels [T] or None, gather index [T] into the flattened batch)``. ``labels`` follow the
    ``transformers`` convention (aligned with ``input_ids``; the model shifts them) unless ``shift_labels`` is False."""
    import numpy as np

    B, S = input_ids.shape
    if attention_mask is None:
        attention_mask = torch.ones_like(input_ids)
    keep = attention_mask.reshape(-1).bool()
    index = torch.nonzero(keep, as_tuple=False).reshape(-1)
    lengths = attention_mask.sum(-1).to("cpu", torch.int64).numpy()
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
    ids = input_ids.reshape(-1)[index]
    pos = (attention_mask.cumsum(-1) - 1).reshape(-1)[index].to(torch.int32)
    packed_labels = None
    if labels is not None:
        if shift_labels:
            # the target of position t is token t+1 of the same row; a row's last position scores nothing
            nxt = torch.full_like(labels, -100)
            nxt[:, :-1] = labels[:, 1:]
            valid_next = torch.zeros_like(attention_mask)
            valid_next[:, :-1] = attention_mask[:, 1:]
            nxt = torch.where(valid_next.bool(), nxt, torch.full_like(nxt, -100))
            labels = nxt
        packed_labels = labels.reshape(-1)[index]
    return ids, pos, cu, packed_labels, index


class HaloForCausalLM(PreTrainedModel):
    config_class = HaloConfig
    base_model_prefix = "model"
    supports_gradient_checkpointing = True
    _no_split_modules = ["DecoderLayer"]

    def __init__(self, config: HaloConfig, device=None, dtype=None, transport=None, seed: int = 0, init: bool = True, **kw):
        super().__init__(config)
        dev = torch.device(device or "cpu")
        self.model = build_model(config.model_config, device=dev, dtype=dtype, transport=transport, seed=seed, init=init, **kw)

    # ---- transformers plumbing -----------------------------------------------------------------
    def _init_weights(self, module):          # weights come from build_model / the checkpoint, never from the base class
        return

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None):
        self.model.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.model.gradient_checkpointing = False

    @property
    def is_gradient_checkpointing(self) -> bool:
        return bool(self.model.gradient_checkpointing)

    @property
    def cfg(self) -> ModelConfig:
        return self.model.cfg

    def named_parameters(self, *a, **kw):
        """Parameter names are the inner model's own (what checkpoints, optimizers and the parallel layout key on)."""
        yield from self.model.named_parameters(*a, **kw)

    # ---- forward -------------------------------------------------------------------------------
    def forward(self, input_ids=None, attention_mask=None, labels=None, position_ids=None, cu_seqlens=None,
                num_items_in_batch=None, return_logits: bool | None = None, return_dict: bool = True, **unused):
        """``input_ids`` either ``[B, S]`` with an ``attention_mask`` (packed here) or already packed ``[T]`` with
        ``position_ids`` and ``cu_seqlens``. With ``labels`` the loss is the mean cross-entropy over the scored tokens
        (or their sum over ``num_items_in_batch`` when the trainer passes its global count). Logits are materialised
        only without labels or when ``return_logits`` is set."""
        index = None
        shape = None
        if input_ids.dim() == 2:
            shape = tuple(input_ids.shape)
            input_ids, position_ids, cu_seqlens, labels, index = pack_padded_batch(input_ids, attention_mask, labels)
        elif cu_seqlens is None:
            raise ValueError("a packed [T] stream needs cu_seqlens (and position_ids)")
        loss = None
        if labels is not None:
            normalizer = None
            if num_items_in_batch is not None:
                normalizer = num_items_in_batch if torch.is_tensor(num_items_in_batch) else float(num_items_in_batch)
            loss = self.model(input_ids, position_ids, cu_seqlens, labels, normalizer)
        logits = None
        if labels is None or return_logits:
            h = self.model.hidden_states(input_ids, position_ids, cu_seqlens)
            flat = self.model.capped_logits(h) if self.cfg.final_logit_softcapping else h.float() @ self.model.head_weight().float().t()
            if index is not None:
                logits = flat.new_zeros((shape[0] * shape[1], flat.shape[-1]))
                logits[index] = flat
                logits = logits.view(shape[0], shape[1], -1)
            else:
                logits = flat
        if not return_dict:
            return tuple(v for v in (loss, logits) if v is not None)
        return CausalLMOutput(loss=loss, logits=logits)

    # ---- hub layout in and out -------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, *args, device="cpu", dtype=None, torch_dtype=None, transport=None,
                        **kw):
        """Build the model ``config.json`` describes and fill it from the SafeTensors files under the directory: every rank
        reads only what it owns (its experts, its tensor-parallel slices), and a checkpoint that leaves any parameter
        untouched is refused."""
        from halo_b200.checkpoint.load import load_model_weights

        directory = os.fspath(pretrained_model_name_or_path)
        if not os.path.isdir(directory):
            raise FileNotFoundError(f"{directory!r} is not a local checkpoint directory (there is no hub download here)")
        config = HaloConfig(ModelConfig.load(directory))
        model = cls(config, device=device, dtype=dtype or torch_dtype, transport=transport, init=False,
                    **{k: v for k, v in kw.items() if k in ("gradient_checkpointing", "tensor_parallel", "layer_range")})
        for p in model.model.parameters():
            if p.dim() == 1:
                p.data.fill_(1.0)
        load_model_weights(model.model, directory)
        return model

    def save_pretrained(self, save_directory, is_main_process: bool | None = None, safe_serialization: bool = True,
                        max_shard_size: int | str = 5 * 1024**3, **kw):
        """Write ``config.json`` and SafeTensors shards in the hub layout (experts gathered from their owners). Collective
        when experts are sharded over ranks."""
        from halo_b200.checkpoint.save import save_model

        if not safe_serialization:
            raise ValueError("only SafeTensors checkpoints are written")
        if isinstance(max_shard_size, str):
            unit = {"KB": 1 << 10, "MB": 1 << 20, "GB": 1 << 30}
            max_shard_size = int(float(max_shard_size[:-2]) * unit[max_shard_size[-2:].upper()])
        save_model(self.model, os.fspath(save_directory), is_writer=is_main_process, max_shard_bytes=int(max_shard_size),
                   save_dtype=None)      # as transformers does: the parameters' own dtype

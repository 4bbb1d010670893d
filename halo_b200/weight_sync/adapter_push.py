"""Pushing low-rank adapters instead of full weights to a generation server: the adapters are written in the PEFT layout
to a directory both sides see, the server loads them under a versioned name, and rollouts ask for that name. An adapter is
megabytes where the merged model is tens of gigabytes, so a push costs a file write and two HTTP calls.

One version is live at a time: version ``n`` is loaded before version ``n - 1`` is unloaded, so a request that arrives in
between still finds a model. The first push also checks that the server serves the same base model the adapters were
trained on.

Counterpart of halo/weight_sync/adapter_versions.py, adapter_routes.py, adapter_payload.py and adapter_servers.py.
"""

from __future__ import annotations

import os
import shutil

import torch.distributed as dist


class AdapterPusher:
    """The weight pusher a GRPO trainer calls (``push(model)`` / ``close()``) when the policy trains adapters."""

    def __init__(self, client, directory: str, name: str = "policy", keep_versions: int = 2, trainer_group=None, src_rank: int = 0):
        self.client, self.directory, self.name = client, directory, name
        self.keep_versions = max(keep_versions, 1)
        self.trainer_group, self.src_rank = trainer_group, src_rank
        live = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(trainer_group) if live else 0
        self.version = 0
        self.pushes = 0
        self._loaded: list[str] = []

    @property
    def current_model_id(self) -> str:
        """What rollouts must ask for: the newest loaded adapter, or the base model before the first push."""
        return self._loaded[-1] if self._loaded else (getattr(self.client, "model_id", "") or "")

    def _versioned(self, n: int) -> str:
        return f"{self.name}-v{n}"

    def push(self, model) -> None:
        from halo_b200.peft.lora import save_adapters

        if getattr(model, "lora_spec", None) is None:
            raise ValueError("the model carries no adapters: push its weights with EngineWeightPusher")
        self.version += 1
        name = self._versioned(self.version)
        path = os.path.join(self.directory, name)
        sender = self.rank == self.src_rank
        # collective when adapter slices are sharded; the sender writes
        save_adapters(model, path, base_model=getattr(model, "base_model_path", ""), is_writer=sender)
        error = None
        if sender:
            try:
                self.client.load_adapter(name, path)
                self._loaded.append(name)
                while len(self._loaded) > 1:
                    old = self._loaded.pop(0)
                    self.client.unload_adapter(old)
                stale = self._versioned(self.version - self.keep_versions)
                if self.version > self.keep_versions:
                    shutil.rmtree(os.path.join(self.directory, stale), ignore_errors=True)
            except Exception as exc:  # noqa: BLE001 - agreed on below
                error = exc
        if dist.is_available() and dist.is_initialized():
            import torch

            flag = torch.tensor([0 if error is None else 1])
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.trainer_group)
            names = [self.current_model_id]
            dist.broadcast_object_list(names, src=dist.get_global_rank(self.trainer_group, self.src_rank) if self.trainer_group is not None
                                       else self.src_rank, group=self.trainer_group)
            if not sender:
                self._loaded = [names[0]] if names[0] else []
            if int(flag.item()):
                raise RuntimeError(f"pushing adapters to the generation server failed: {error}")
        elif error is not None:
            raise RuntimeError(f"pushing adapters to the generation server failed: {error}")
        self.pushes += 1

    def close(self) -> None:
        if self.rank == self.src_rank and self.client is not None:
            for name in self._loaded:
                try:
                    self.client.unload_adapter(name)
                except Exception:  # noqa: BLE001 - the server may be gone
                    pass
            self.client.close()

"""Weight sync into an SGLang server through its distributed weight-update routes (``/init_weights_update_group``,
``/update_weights_from_distributed``, ``/pause_generation``, ``/continue_generation``, ``/flush_cache``,
``/get_server_info``, ``/destroy_weights_update_group``).

Two data planes:

* ``data_plane="torch"`` (default): the group the server's workers form - a ``torch.distributed`` process group built
  beside the default one from a ``tcp://`` rendezvous and a store prefixed with the group's name - and one
  ``broadcast`` per tensor from rank 0, which is what a stock server expects;
* ``data_plane="packed"``: the framework's own transfer group and packed chunk layout (:mod:`.transport`), for engines
  that load it on their side.

Counterpart of halo/weight_sync/clients/sglang.py:68-591.
"""

from __future__ import annotations

from datetime import timedelta

import torch
import torch.distributed as dist

from .base import SESSION_TIMEOUT_S, AsyncCall, EngineWeightSyncClient, ServerInfo
from .transport import free_port, routable_address


def init_custom_process_group(backend: str, init_method: str, world_size: int, rank: int, group_name: str, timeout_s: float = 120.0):
    """A process group that exists beside the default one (the trainer keeps its job's groups): the rendezvous of
    ``init_method``, a store prefixed with ``group_name``, and the backend's group object built on it. The server's workers
    build theirs the same way, so the two sides meet."""
    from torch.distributed.distributed_c10d import PrefixStore, _new_process_group_helper, _world, rendezvous

    timeout = timedelta(seconds=timeout_s)
    store, rank, world_size = next(iter(rendezvous(init_method, rank, world_size, timeout=timeout)))
    store.set_timeout(timeout)
    store = PrefixStore(group_name, store)
    pg, _ = _new_process_group_helper(world_size, rank, [], backend, store, group_name=group_name, timeout=timeout)
    _world.pg_group_ranks[pg] = {i: i for i in range(world_size)}
    return pg


class SGLangWeightSyncClient(EngineWeightSyncClient):
    BACKEND = "sglang"
    MIN_VERSION = (0, 4, 6)
    INFO_ROUTE = "/get_server_info"
    PAUSE_ROUTE = "/pause_generation"
    RESUME_ROUTE = "/continue_generation"
    SESSION_OPEN_ROUTE = ""                          # no session object: the update that ends a push flushes the cache
    SESSION_CLOSE_ROUTE = ""
    INIT_GROUP_ROUTE = "/init_weights_update_group"
    DESTROY_GROUP_ROUTE = "/destroy_weights_update_group"
    UPDATE_ROUTE = "/update_weights_from_distributed"
    FLUSH_ROUTE = "/flush_cache"
    LOAD_ADAPTER_ROUTE = "/load_lora_adapter"
    UNLOAD_ADAPTER_ROUTE = "/unload_lora_adapter"

    def __init__(self, url: str, *args, data_plane: str = "torch", backend: str | None = None, **kw):
        super().__init__(url, *args, **kw)
        if data_plane not in ("torch", "packed"):
            raise ValueError(f"data_plane must be torch or packed, got {data_plane!r}")
        self.data_plane = data_plane
        self.torch_backend = backend                  # default: nccl on a GPU, gloo on CPU
        self._pg = None

    def parse_info(self, raw: dict) -> ServerInfo:
        return ServerInfo(version=str(raw.get("version", "")), model_id=str(raw.get("served_model_name") or raw.get("model_path") or ""),
                          max_model_len=int(raw.get("context_length") or raw.get("max_total_num_tokens") or 0),
                          tensor_parallel_size=int(raw.get("tp_size") or 1), data_parallel_size=int(raw.get("dp_size") or 1),
                          pipeline_parallel_size=int(raw.get("pp_size") or 1),
                          flags={k: raw[k] for k in ("attention_backend", "disable_cuda_graph", "enable_ep_moe", "tool_call_parser",
                                                     "reasoning_parser", "quantization") if k in raw})

    def init_group_payload(self, master: str, port: int, world_size: int) -> dict:
        return {"master_address": master, "master_port": port, "rank_offset": 1, "world_size": world_size,
                "group_name": self.GROUP_NAME, "backend": self.torch_backend or "nccl"}

    def init_transfer_group(self, device=None, timeout_s: float = 120.0) -> None:
        if self.data_plane != "torch":
            return super().init_transfer_group(device, timeout_s)
        if self._pg is not None:
            return
        info = self.info or self.read_server_info()
        world = info.world_size + 1
        dev = torch.device(device) if device is not None else torch.device("cpu")
        backend = self.torch_backend or ("nccl" if dev.type == "cuda" else "gloo")
        self.torch_backend = backend
        host = self.group_host or routable_address(self.url.split("//", 1)[-1].split(":")[0].split("/")[0])
        port = free_port()
        payload = self.init_group_payload(host, port, world)
        joining = AsyncCall(lambda: self.request("POST", self.INIT_GROUP_ROUTE, json=payload, timeout=timeout_s, retry=False),
                            "transfer-group formation", timeout_s + 5)
        try:
            self._pg = init_custom_process_group(backend, f"tcp://{host}:{port}", world, 0, self.GROUP_NAME, timeout_s)
            joining.result()
        except Exception as exc:
            self._pg = None
            raise RuntimeError(f"could not form the weight-update group with the SGLang server at {self.url} (advertised "
                               f"{host}:{port}); pass group_host= an interface the server can route to. Cause: {exc}") from exc
        self.group = _TorchGroupHandle(dev)

    def chunk_payload(self, slots, nbytes: int, final: bool) -> dict:
        return {"names": [s.name for s in slots], "dtypes": [str(s.dtype).replace("torch.", "") for s in slots],
                "shapes": [list(s.shape) for s in slots], "group_name": self.GROUP_NAME, "flush_cache": bool(final),
                "packed_offsets": [s.offset for s in slots], "packed_bytes": nbytes}

    def send_tensors(self, named_tensors: dict, final: bool = False) -> None:
        if self._pg is None:
            return super().send_tensors(named_tensors, final)
        if not named_tensors:
            return
        payload = {"names": list(named_tensors), "dtypes": [str(t.dtype).replace("torch.", "") for t in named_tensors.values()],
                   "shapes": [list(t.shape) for t in named_tensors.values()], "group_name": self.GROUP_NAME,
                   "flush_cache": bool(final)}
        try:
            announced = AsyncCall(lambda: self.request("POST", self.UPDATE_ROUTE, json=payload, timeout=SESSION_TIMEOUT_S, retry=False),
                                  f"update of {len(named_tensors)} tensors", SESSION_TIMEOUT_S + 5)
            works = [dist.broadcast(t.detach().contiguous(), src=0, group=self._pg, async_op=True) for t in named_tensors.values()]
            for w in works:
                w.wait()
            announced.result()
            self._chunks_sent += 1
        except Exception as exc:
            self._fail(self._chunks_sent, exc)
            raise

    def close(self, remote: bool = True) -> None:
        super().close(remote)
        if self._pg is not None:
            try:
                dist.destroy_process_group(self._pg)
            except Exception:  # noqa: BLE001 - the peer may be gone already
                pass
            self._pg = None


class _TorchGroupHandle:
    def __init__(self, device):
        self.device = device

    def close(self) -> None:
        pass

"""Weight sync into a vLLM server through its own weight-transfer routes (vLLM 0.10+: ``/pause``, ``/resume``,
``/init_weight_transfer_engine``, ``/start_weight_update``, ``/update_weights``, ``/finish_weight_update``,
``/get_world_size``, ``/server_info``).

Two data planes:

* ``data_plane="vllm"`` (default on a GPU when the ``vllm`` package is importable on the trainer): the trainer joins the
  server's transfer group with vLLM's own trainer-side helpers (``NCCLWeightTransferEngine.trainer_init`` /
  ``trainer_send_weights``: a stateless group and an NCCL communicator the workers understand) and streams the tensors
  in its packed-buffer protocol. This is the form that talks to a stock server.
* ``data_plane="packed"``: the framework's own transfer group (:mod:`.transport`) and chunk layout with explicit
  offsets - for engines that load :mod:`halo_b200.weight_sync.clients.transport` on their side, and for the CPU tests.

Counterpart of halo/weight_sync/clients/vllm.py:45-342 (which vendors an NCCL bootstrap instead of importing vllm).
"""

from __future__ import annotations

import torch

from .base import SESSION_TIMEOUT_S, AsyncCall, EngineWeightSyncClient, ServerInfo
from .transport import free_port, routable_address


class VLLMWeightSyncClient(EngineWeightSyncClient):
    BACKEND = "vllm"
    MIN_VERSION = (0, 10, 0)
    INFO_ROUTE = "/server_info"
    PAUSE_ROUTE = "/pause"
    PAUSE_PARAMS = {"mode": "keep"}                  # in-flight generations are frozen and continue under the new weights
    RESUME_ROUTE = "/resume"
    SESSION_OPEN_ROUTE = "/start_weight_update"
    SESSION_CLOSE_ROUTE = "/finish_weight_update"
    INIT_GROUP_ROUTE = "/init_weight_transfer_engine"
    DESTROY_GROUP_ROUTE = ""
    UPDATE_ROUTE = "/update_weights"
    LOAD_ADAPTER_ROUTE = "/v1/load_lora_adapter"
    UNLOAD_ADAPTER_ROUTE = "/v1/unload_lora_adapter"
    PACKED_NUM_BUFFERS = 2

    def __init__(self, url: str, *args, data_plane: str = "auto", **kw):
        super().__init__(url, *args, **kw)
        if data_plane not in ("auto", "vllm", "packed"):
            raise ValueError(f"data_plane must be auto, vllm or packed, got {data_plane!r}")
        self.data_plane = data_plane
        self._native_group = None

    def _plane(self, device) -> str:
        if self.data_plane != "auto":
            return self.data_plane
        if device is not None and torch.device(device).type == "cuda":
            try:
                import vllm.distributed.weight_transfer.nccl_engine  # noqa: F401

                return "vllm"
            except Exception:  # noqa: BLE001 - not installed (or not importable without a GPU build)
                pass
        return "packed"

    # ---- server facts -------------------------------------------------------------------------------
    def parse_info(self, raw: dict) -> ServerInfo:
        cfg = raw.get("vllm_config") or {}
        par = cfg.get("parallel_config") or {}
        model = cfg.get("model_config") or {}
        return ServerInfo(version=str(raw.get("version", "")), model_id=str(model.get("served_model_name") or model.get("model") or ""),
                          max_model_len=int(model.get("max_model_len") or 0),
                          tensor_parallel_size=int(par.get("tensor_parallel_size") or 1),
                          data_parallel_size=int(par.get("data_parallel_size") or 1),
                          pipeline_parallel_size=int(par.get("pipeline_parallel_size") or 1),
                          flags={k: v for k, v in (raw.get("vllm_env") or {}).items()})

    def pause(self) -> None:
        if not self.paused:
            self.request("POST", self.PAUSE_ROUTE, params=self.PAUSE_PARAMS, timeout=SESSION_TIMEOUT_S)
        self.paused = True

    def open_session(self) -> None:
        # tensors travel under their checkpoint names (q_proj / k_proj / v_proj ...): the server's loader fuses them
        self.request("POST", self.SESSION_OPEN_ROUTE, json={"is_checkpoint_format": True}, timeout=SESSION_TIMEOUT_S)
        self.session_open = True

    def close_session(self, flushed: bool = True) -> None:
        if self.session_open:
            self.request("POST", self.SESSION_CLOSE_ROUTE, timeout=SESSION_TIMEOUT_S)
        self.session_open = False

    # ---- the transfer group -------------------------------------------------------------------------
    def init_group_payload(self, master: str, port: int, world_size: int) -> dict:
        return {"init_info": {"master_address": master, "master_port": port, "rank_offset": 1, "world_size": world_size}}

    def init_transfer_group(self, device=None, timeout_s: float = 120.0) -> None:
        if self._plane(device) != "vllm":
            return super().init_transfer_group(device, timeout_s)
        if self._native_group is not None:
            return
        from vllm.distributed.weight_transfer.nccl_engine import NCCLWeightTransferEngine

        info = self.info or self.read_server_info()
        world = info.world_size + 1
        host = self.group_host or routable_address(self.url.split("//", 1)[-1].split(":")[0].split("/")[0])
        port = free_port()
        payload = self.init_group_payload(host, port, world)
        joining = AsyncCall(lambda: self.request("POST", self.INIT_GROUP_ROUTE, json=payload, timeout=timeout_s, retry=False),
                            "transfer-group formation", timeout_s + 5)
        try:
            if device is not None:
                torch.cuda.set_device(torch.device(device))
            self._native_group = NCCLWeightTransferEngine.trainer_init(
                {"master_address": host, "master_port": port, "world_size": world})
            joining.result()
        except Exception as exc:
            self._native_group = None
            raise RuntimeError(f"could not form the weight-transfer group with the vLLM server at {self.url} (advertised "
                               f"{host}:{port}); pass group_host= an interface the server can route to. Cause: {exc}") from exc
        self.group = _NativeGroupHandle(device)

    # ---- chunks -----------------------------------------------------------------------------------------
    def chunk_payload(self, slots, nbytes: int, final: bool) -> dict:
        return {"update_info": {"names": [s.name for s in slots], "dtype_names": [str(s.dtype).replace("torch.", "") for s in slots],
                                "shapes": [list(s.shape) for s in slots], "offsets": [s.offset for s in slots],
                                "packed": True, "packed_bytes": nbytes, "is_last": bool(final)}}

    def send_tensors(self, named_tensors: dict, final: bool = False) -> None:
        if self._native_group is None:
            return super().send_tensors(named_tensors, final)
        if not named_tensors:
            return
        from vllm.distributed.weight_transfer.nccl_engine import NCCLTrainerSendWeightsArgs, NCCLWeightTransferEngine

        update = {"update_info": {"names": list(named_tensors), "dtype_names": [str(t.dtype).replace("torch.", "") for t in named_tensors.values()],
                                  "shapes": [list(t.shape) for t in named_tensors.values()], "packed": True,
                                  "packed_buffer_size_bytes": int(self.chunk_bytes), "packed_num_buffers": self.PACKED_NUM_BUFFERS}}
        try:
            announced = AsyncCall(lambda: self.request("POST", self.UPDATE_ROUTE, json=update, timeout=SESSION_TIMEOUT_S, retry=False),
                                  f"update of {len(named_tensors)} tensors", SESSION_TIMEOUT_S + 5)
            args = NCCLTrainerSendWeightsArgs(group=self._native_group, packed=True, packed_buffer_size_bytes=int(self.chunk_bytes),
                                              packed_num_buffers=self.PACKED_NUM_BUFFERS)
            NCCLWeightTransferEngine.trainer_send_weights(iter(named_tensors.items()), args)
            announced.result()
            self._chunks_sent += 1
        except Exception as exc:
            self._fail(self._chunks_sent, exc)
            raise

    def close(self, remote: bool = True) -> None:
        self._native_group = None
        if isinstance(self.group, _NativeGroupHandle):
            self.group = None
        super().close(remote)


class _NativeGroupHandle:
    """What the base class needs to know about a group vLLM's helpers own: the device, and that it exists."""

    def __init__(self, device):
        self.device = torch.device(device) if device is not None else torch.device("cuda")

    def close(self) -> None:
        pass

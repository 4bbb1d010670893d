"""Routes and payloads of a vLLM server's weight-update interface (pause / layerwise reload session / packed chunks
over a transfer group). Counterpart of halo/weight_sync/clients/vllm.py:45-342."""

from __future__ import annotations

from .base import EngineWeightSyncClient, ServerInfo


class VLLMWeightSyncClient(EngineWeightSyncClient):
    BACKEND = "vllm"
    MIN_VERSION = (0, 10, 0)
    INFO_ROUTE = "/server_info"
    PAUSE_ROUTE = "/pause"
    PAUSE_PAYLOAD = {"params": {"mode": "keep"}}     # in-flight generations continue under the new weights
    RESUME_ROUTE = "/resume"
    SESSION_OPEN_ROUTE = "/start_weight_update"
    SESSION_CLOSE_ROUTE = "/finish_weight_update"
    INIT_GROUP_ROUTE = "/init_weight_transfer_engine"
    DESTROY_GROUP_ROUTE = "/destroy_weight_transfer_engine"
    UPDATE_ROUTE = "/update_weights"
    LOAD_ADAPTER_ROUTE = "/v1/load_lora_adapter"
    UNLOAD_ADAPTER_ROUTE = "/v1/unload_lora_adapter"

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

    def init_group_payload(self, master: str, port: int, world_size: int) -> dict:
        return {"init_info": {"master_address": master, "master_port": port, "rank_offset": 1, "world_size": world_size,
                              "backend": "packed_broadcast", "packed_buffer_bytes": self.chunk_bytes}}

    def chunk_payload(self, slots, nbytes: int, final: bool) -> dict:
        return {"update_info": {"names": [s.name for s in slots], "dtype_names": [str(s.dtype).replace("torch.", "") for s in slots],
                                "shapes": [list(s.shape) for s in slots], "offsets": [s.offset for s in slots],
                                "packed": True, "packed_bytes": nbytes, "is_last": bool(final)}}

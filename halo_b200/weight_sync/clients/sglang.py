"""Routes and payloads of an SGLang server's distributed weight update (``init_weights_update_group`` /
``update_weights_from_distributed``). Counterpart of halo/weight_sync/clients/sglang.py:68-591."""

from __future__ import annotations

from .base import EngineWeightSyncClient, ServerInfo


class SGLangWeightSyncClient(EngineWeightSyncClient):
    BACKEND = "sglang"
    MIN_VERSION = (0, 4, 6)
    INFO_ROUTE = "/get_server_info"
    PAUSE_ROUTE = "/pause_generation"
    RESUME_ROUTE = "/continue_generation"
    SESSION_OPEN_ROUTE = ""                          # no session object: the last chunk carries flush_cache
    SESSION_CLOSE_ROUTE = ""
    INIT_GROUP_ROUTE = "/init_weights_update_group"
    DESTROY_GROUP_ROUTE = "/destroy_weights_update_group"
    UPDATE_ROUTE = "/update_weights_from_distributed"
    FLUSH_ROUTE = "/flush_cache"
    LOAD_ADAPTER_ROUTE = "/load_lora_adapter"
    UNLOAD_ADAPTER_ROUTE = "/unload_lora_adapter"

    def parse_info(self, raw: dict) -> ServerInfo:
        return ServerInfo(version=str(raw.get("version", "")), model_id=str(raw.get("served_model_name") or raw.get("model_path") or ""),
                          max_model_len=int(raw.get("context_length") or raw.get("max_total_num_tokens") or 0),
                          tensor_parallel_size=int(raw.get("tp_size") or 1), data_parallel_size=int(raw.get("dp_size") or 1),
                          pipeline_parallel_size=int(raw.get("pp_size") or 1),
                          flags={k: raw[k] for k in ("attention_backend", "disable_cuda_graph", "enable_ep_moe", "tool_call_parser",
                                                     "reasoning_parser") if k in raw})

    def init_group_payload(self, master: str, port: int, world_size: int) -> dict:
        return {"master_address": master, "master_port": port, "rank_offset": 1, "world_size": world_size,
                "group_name": self.GROUP_NAME, "backend": "nccl"}

    def chunk_payload(self, slots, nbytes: int, final: bool) -> dict:
        return {"names": [s.name for s in slots], "dtypes": [str(s.dtype).replace("torch.", "") for s in slots],
                "shapes": [list(s.shape) for s in slots], "group_name": self.GROUP_NAME, "flush_cache": bool(final),
                "packed_offsets": [s.offset for s in slots], "packed_bytes": nbytes}

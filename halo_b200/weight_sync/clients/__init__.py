"""Weight-sync clients for generation servers (vLLM, SGLang) that run outside the training job."""

from .base import EngineUnusable, EngineWeightSyncClient, ServerInfo
from .sglang import SGLangWeightSyncClient
from .vllm import VLLMWeightSyncClient

CLIENTS = {"vllm": VLLMWeightSyncClient, "sglang": SGLangWeightSyncClient}


def make_client(backend: str, url: str, **kw) -> EngineWeightSyncClient:
    if backend not in CLIENTS:
        raise ValueError(f"no weight-sync client for rollout_backend {backend!r}; choose from {sorted(CLIENTS)}")
    return CLIENTS[backend](url, **kw)

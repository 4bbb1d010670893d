"""Pushing a policy's weights into a generation server that runs outside the training job.

One trainer rank (the forwarding rank, which holds or gathers the full tensors) drives the update:

    pause generation -> open an update session -> for every packed chunk: announce its tensors over HTTP while the
    chunk itself travels over the trainer-to-server process group -> close the session (the server flushes its caches)
    -> resume generation

The HTTP call that announces a chunk blocks on the server until its workers have received the chunk, so it is sent
from a helper thread while the calling thread runs the broadcast (both sides of one rendezvous). A failure after the
first chunk leaves the server with a model that is part old and part new: the client then aborts the session, marks
itself unusable and raises, and refuses further pushes until the server has been restarted and the client re-created.

Subclasses name the routes and payloads of one server (:mod:`.vllm`, :mod:`.sglang`). The server packages are never
imported.

Counterpart of halo/weight_sync/clients/base.py:126-827 (``WeightSyncClientBase``) and
halo/weight_sync/update_stream.py.
"""

from __future__ import annotations

import logging
import threading
import time
from dataclasses import dataclass, field

import torch

from halo_b200.weight_sync.chunking import pack_chunk, plan_chunks

from .transport import EngineGroup, free_port, routable_address

log = logging.getLogger(__name__)

HTTP_PROBE_TIMEOUT_S = 10.0
SESSION_TIMEOUT_S = 120.0
CLEANUP_TIMEOUT_S = 30.0


class EngineUnusable(RuntimeError):
    """The server holds a partly updated model (or lost its transfer group) and must be restarted."""


@dataclass
class ServerInfo:
    version: str = ""
    model_id: str = ""
    max_model_len: int = 0
    tensor_parallel_size: int = 1
    data_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    flags: dict = field(default_factory=dict)

    @property
    def world_size(self) -> int:
        """GPU workers that must each receive every chunk."""
        return self.tensor_parallel_size * self.data_parallel_size * self.pipeline_parallel_size


class AsyncCall:
    """An HTTP call running on a helper thread; ``result()`` joins it (bounded) and re-raises its error."""

    def __init__(self, fn, what: str, timeout_s: float):
        self.what, self.timeout_s = what, timeout_s
        self._out, self._err = None, None

        def run():
            try:
                self._out = fn()
            except BaseException as exc:  # noqa: BLE001 - carried to the caller
                self._err = exc

        self._thread = threading.Thread(target=run, name=f"engine-call:{what}", daemon=True)
        self._thread.start()

    def result(self):
        self._thread.join(self.timeout_s)
        if self._thread.is_alive():
            raise TimeoutError(f"the server did not answer {self.what} within {self.timeout_s:.0f} s")
        if self._err is not None:
            raise self._err
        return self._out


class EngineWeightSyncClient:
    BACKEND = ""
    MIN_VERSION: tuple[int, ...] = ()
    HEALTH_ROUTE = "/health"
    INFO_ROUTE = ""
    PAUSE_ROUTE = ""
    PAUSE_PAYLOAD: dict = {}
    PAUSE_PARAMS: dict = {}
    RESUME_ROUTE = ""
    SESSION_OPEN_ROUTE = ""
    SESSION_CLOSE_ROUTE = ""
    INIT_GROUP_ROUTE = ""
    DESTROY_GROUP_ROUTE = ""
    UPDATE_ROUTE = ""
    FLUSH_ROUTE = ""
    LOAD_ADAPTER_ROUTE = ""
    UNLOAD_ADAPTER_ROUTE = ""
    GROUP_NAME = "halo_b200_weight_sync"

    def __init__(self, url: str, model_id: str = "", chunk_bytes: int = 1 << 30, group_host: str = "", session=None,
                 http_retries: int = 3):
        self.url = url.rstrip("/")
        self.model_id = model_id
        self.chunk_bytes = chunk_bytes
        self.group_host = group_host
        self.http_retries = http_retries
        self._session = session              # an object with .request(method, url, json=, params=, timeout=); tests inject a fake
        self.group: EngineGroup | None = None
        self.info: ServerInfo | None = None
        self.unusable_reason = ""
        self.paused = False
        self.session_open = False
        self.pushes = 0
        self._staging: torch.Tensor | None = None
        self._chunks_sent = 0

    # ---- HTTP ---------------------------------------------------------------------------------------
    def _http(self):
        if self._session is None:
            import requests

            self._session = requests.Session()
        return self._session

    def request(self, method: str, route: str, json=None, params=None, timeout: float = HTTP_PROBE_TIMEOUT_S, retry: bool = True):
        """One call; connection errors and 5xx answers are retried with backoff (idempotent routes only: pass
        ``retry=False`` for a call that blocks on a rendezvous)."""
        attempts = self.http_retries if retry else 1
        delay, last = 0.25, None
        for attempt in range(attempts):
            try:
                resp = self._http().request(method, self.url + route, json=json, params=params, timeout=timeout)
                if resp.status_code >= 500 and attempt + 1 < attempts:
                    last = RuntimeError(f"{route}: HTTP {resp.status_code}")
                elif resp.status_code >= 400:
                    raise RuntimeError(f"{self.BACKEND} server refused {method} {route}: HTTP {resp.status_code} {resp.text[:500]}")
                else:
                    return resp
            except (ConnectionError, OSError, TimeoutError) as exc:
                last = exc
            except Exception as exc:  # noqa: BLE001 - requests' own exception classes
                if type(exc).__module__.startswith("requests") and attempt + 1 < attempts:
                    last = exc
                else:
                    raise
            time.sleep(delay)
            delay = min(delay * 2, 4.0)
        raise ConnectionError(f"{self.BACKEND} server at {self.url} did not answer {method} {route}: {last}")

    def check_server(self, total_timeout: float = 0.0) -> None:
        """Wait (up to ``total_timeout``) until the health route answers."""
        deadline = time.monotonic() + total_timeout
        while True:
            try:
                self.request("GET", self.HEALTH_ROUTE, retry=False)
                return
            except Exception as exc:  # noqa: BLE001
                if time.monotonic() >= deadline:
                    raise ConnectionError(f"{self.BACKEND} server at {self.url} is not healthy: {exc}") from exc
                time.sleep(1.0)

    # ---- server facts -------------------------------------------------------------------------------
    def parse_info(self, raw: dict) -> ServerInfo:
        raise NotImplementedError

    def read_server_info(self) -> ServerInfo:
        raw = self.request("GET", self.INFO_ROUTE, timeout=60.0).json()
        self.info = self.parse_info(raw)
        if self.MIN_VERSION and self.info.version:
            have = tuple(int(p) for p in self.info.version.split("+")[0].split(".")[:3] if p.isdigit())
            if have and have < self.MIN_VERSION:
                raise RuntimeError(f"{self.BACKEND} {self.info.version} is older than {'.'.join(map(str, self.MIN_VERSION))}, "
                                   "the first release with the weight-update routes this client speaks")
        if self.model_id and self.info.model_id and self.info.model_id != self.model_id:
            log.warning("the server serves %r, the trainer trains %r: pushes will overwrite the served weights",
                        self.info.model_id, self.model_id)
        return self.info

    # ---- the transfer group -------------------------------------------------------------------------
    def init_group_payload(self, master: str, port: int, world_size: int) -> dict:
        raise NotImplementedError

    def init_transfer_group(self, device=None, timeout_s: float = 120.0) -> None:
        """Form the trainer-to-server group: this process is rank 0, the server's workers are ranks 1..W."""
        if self.group is not None:
            return
        info = self.info or self.read_server_info()
        world = info.world_size + 1
        host = self.group_host or routable_address(self.url.split("//", 1)[-1].split(":")[0].split("/")[0])
        port = free_port()
        payload = self.init_group_payload(host, port, world)
        joining = AsyncCall(lambda: self.request("POST", self.INIT_GROUP_ROUTE, json=payload, timeout=timeout_s, retry=False),
                            "transfer-group formation", timeout_s + 5)
        try:
            self.group = EngineGroup(host, port, 0, world, device, timeout_s)
            joining.result()
            self.group.barrier(timeout_s)
        except Exception as exc:
            self.group = None
            raise RuntimeError(
                f"could not form the weight-transfer group with the {self.BACKEND} server at {self.url} (advertised "
                f"{host}:{port}). If the server cannot reach that address, pass group_host= an interface it can route to "
                f"(and set NCCL_SOCKET_IFNAME on multi-homed hosts). Cause: {exc}") from exc

    # ---- one update ---------------------------------------------------------------------------------
    def pause(self) -> None:
        if self.PAUSE_ROUTE and not self.paused:
            self.request("POST", self.PAUSE_ROUTE, json=self.PAUSE_PAYLOAD or None, timeout=SESSION_TIMEOUT_S)
        self.paused = True

    def resume(self) -> None:
        if self.RESUME_ROUTE and self.paused:
            self.request("POST", self.RESUME_ROUTE, timeout=SESSION_TIMEOUT_S)
        self.paused = False

    def open_session(self) -> None:
        if self.SESSION_OPEN_ROUTE:
            self.request("POST", self.SESSION_OPEN_ROUTE, timeout=SESSION_TIMEOUT_S)
        self.session_open = True

    def close_session(self, flushed: bool = True) -> None:
        if self.SESSION_CLOSE_ROUTE and self.session_open:
            self.request("POST", self.SESSION_CLOSE_ROUTE, json={"flush_cache": bool(flushed)}, timeout=SESSION_TIMEOUT_S)
        self.session_open = False

    def chunk_payload(self, slots, nbytes: int, final: bool) -> dict:
        raise NotImplementedError

    def begin_update(self, device=None) -> None:
        """Pause the server and open an update session; ``send_tensors`` may then be called any number of times."""
        if self.unusable_reason:
            raise EngineUnusable(self.unusable_reason)
        if self.group is None:
            self.init_transfer_group(device)
        self._chunks_sent = 0
        try:
            self.pause()
            self.open_session()
        except Exception as exc:
            self._fail(0, exc)
            raise

    def send_tensors(self, named_tensors: dict, final: bool = False) -> None:
        """Pack ``named_tensors`` (hub names) into chunks and send each: the announcement over HTTP from a helper thread,
        the bytes over the transfer group from this one."""
        if not named_tensors:
            return
        manifest = [(n, tuple(t.shape), t.dtype) for n, t in named_tensors.items()]
        slots, sizes = plan_chunks(manifest, self.chunk_bytes)
        device = self.group.device
        if self._staging is None or self._staging.numel() < max(sizes):
            self._staging = torch.empty(max(sizes), dtype=torch.uint8, device=device)
        try:
            for chunk, nbytes in enumerate(sizes):
                mine = [s for s in slots if s.chunk == chunk]
                buf = self._staging[:nbytes]
                pack_chunk(slots, chunk, named_tensors, buf)
                payload = self.chunk_payload(mine, nbytes, final=final and chunk == len(sizes) - 1)
                announced = AsyncCall(lambda p=payload: self.request("POST", self.UPDATE_ROUTE, json=p, timeout=SESSION_TIMEOUT_S,
                                                                     retry=False), f"chunk {self._chunks_sent}", SESSION_TIMEOUT_S + 5)
                self.group.broadcast(buf, src=0)
                announced.result()
                self._chunks_sent += 1
        except Exception as exc:
            self._fail(self._chunks_sent, exc)
            raise

    def end_update(self, flushed_by_last_chunk: bool = False) -> None:
        try:
            if self.SESSION_CLOSE_ROUTE:
                self.close_session(flushed=True)
            elif self.FLUSH_ROUTE and not flushed_by_last_chunk:
                self.request("POST", self.FLUSH_ROUTE, timeout=SESSION_TIMEOUT_S)
            self.session_open = False
            self.resume()
            self.pushes += 1
        except Exception as exc:
            self._fail(self._chunks_sent, exc)
            raise

    def push(self, named_tensors: dict) -> None:
        """Send every tensor of ``named_tensors`` (hub names) to the server as one update. Called on the forwarding rank."""
        self.begin_update(next(iter(named_tensors.values())).device)
        self.send_tensors(named_tensors, final=True)
        self.end_update(flushed_by_last_chunk=True)

    def _fail(self, chunks_sent: int, exc: Exception) -> None:
        """After a failed update: close what can be closed; with chunks already applied the server's model is mixed."""
        if chunks_sent > 0 or self.session_open:
            self.unusable_reason = (f"a weight update to the {self.BACKEND} server at {self.url} failed after {chunks_sent} chunk(s) "
                                    f"({type(exc).__name__}: {exc}); the served model is part old and part new. Restart the server.")
        for step in (lambda: self.close_session(flushed=False), self.resume):
            try:
                step()
            except Exception as cleanup_exc:  # noqa: BLE001 - the first error is the one to report
                log.warning("cleanup after a failed weight update: %s", cleanup_exc)
        if self.unusable_reason:
            self.close(remote=False)

    def close(self, remote: bool = True) -> None:
        if remote and self.group is not None and self.DESTROY_GROUP_ROUTE:
            try:
                self.request("POST", self.DESTROY_GROUP_ROUTE, json={"group_name": self.GROUP_NAME}, timeout=CLEANUP_TIMEOUT_S)
            except Exception as exc:  # noqa: BLE001
                log.warning("the server did not release the transfer group: %s", exc)
        if self.group is not None:
            self.group.close()
            self.group = None
        self._staging = None

    # ---- adapters -----------------------------------------------------------------------------------
    def load_adapter(self, name: str, path: str) -> None:
        if not self.LOAD_ADAPTER_ROUTE:
            raise NotImplementedError(f"the {self.BACKEND} client pushes merged weights only")
        self.request("POST", self.LOAD_ADAPTER_ROUTE, json={"lora_name": name, "lora_path": path}, timeout=SESSION_TIMEOUT_S)

    def unload_adapter(self, name: str) -> None:
        if self.UNLOAD_ADAPTER_ROUTE:
            self.request("POST", self.UNLOAD_ADAPTER_ROUTE, json={"lora_name": name}, timeout=SESSION_TIMEOUT_S)

    # ---- scoring (push parity) ------------------------------------------------------------------------
    def score_completion_logprobs(self, prompt_ids: list[int], completion_ids: list[int]) -> list[float]:
        """The server's log-probabilities of ``completion_ids`` after ``prompt_ids`` (teacher-forced, one request):
        after a push they must agree with the trainer's own scores of the same row."""
        ids = list(prompt_ids) + list(completion_ids)
        payload = {"model": self.model_id or (self.info.model_id if self.info else ""), "prompt": ids, "max_tokens": 1,
                   "temperature": 0.0, "echo": True, "logprobs": 1, "prompt_logprobs": 1}
        raw = self.request("POST", "/v1/completions", json=payload, timeout=SESSION_TIMEOUT_S).json()
        choice = raw["choices"][0]
        if choice.get("prompt_logprobs") is not None:       # vLLM: one {token_id: {"logprob": x}} dict per prompt position
            out = []
            for pos, tok in zip(choice["prompt_logprobs"][len(prompt_ids):len(ids)], completion_ids):
                entry = pos.get(str(tok), pos.get(tok)) if isinstance(pos, dict) else None
                out.append(float(entry["logprob"]) if entry is not None else float("nan"))
            return out
        lp = choice["logprobs"]["token_logprobs"]           # OpenAI echo layout
        return [float(x) for x in lp[len(prompt_ids):len(ids)]]

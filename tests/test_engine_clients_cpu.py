"""Weight-sync clients against a fake generation server: an HTTP server in a child process whose "worker" joins the
trainer-to-server group (gloo), receives the packed chunks and applies them to its own tensors."""

import json
import multiprocessing as mp
import socket
import time

import pytest
import torch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_server(port, backend, log_path, fail_on_chunk):
    """Runs in a child: serves the routes of ``backend`` and plays one GPU worker (rank 1 of the transfer group)."""
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer

    import torch

    from halo_b200.weight_sync.clients.transport import EngineGroup

    state = {"group": None, "weights": {}, "calls": [], "chunks": 0, "paused": False}
    routes = {"vllm": {"info": "/server_info", "init": "/init_weight_transfer_engine", "update": "/update_weights"},
              "sglang": {"info": "/get_server_info", "init": "/init_weights_update_group", "update": "/update_weights_from_distributed"}}[backend]

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _answer(self, code, body):
            data = json.dumps(body).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def do_GET(self):
            path = self.path.split("?")[0]
            state["calls"].append(path)
            if path == "/health":
                return self._answer(200, {})
            if path == routes["info"]:
                if backend == "vllm":
                    return self._answer(200, {"version": "0.11.0", "vllm_config": {"parallel_config": {"tensor_parallel_size": 1},
                                                                                 "model_config": {"model": "tiny", "max_model_len": 4096}}})
                return self._answer(200, {"version": "0.5.0", "model_path": "tiny", "tp_size": 1, "context_length": 4096})
            if path == "/dump":
                with open(log_path, "w") as f:
                    json.dump({"calls": state["calls"], "chunks": state["chunks"],
                               "weights": {k: v.tolist() for k, v in state["weights"].items()}}, f)
                return self._answer(200, {})
            return self._answer(404, {})

        def do_POST(self):
            path = self.path
            n = int(self.headers.get("Content-Length") or 0)
            body = json.loads(self.rfile.read(n) or b"{}") if n else {}
            state["calls"].append(path)
            if path == routes["init"]:
                info = body.get("init_info", body)
                if body.get("backend") == "gloo":
                    # a stock SGLang worker: a torch process group beside its default one, one broadcast per tensor
                    from halo_b200.weight_sync.clients.sglang import init_custom_process_group

                    state["pg"] = init_custom_process_group("gloo", f"tcp://{info['master_address']}:{info['master_port']}",
                                                            info["world_size"], info["rank_offset"], info["group_name"], 30.0)
                    return self._answer(200, {"success": True})
                state["group"] = EngineGroup(info["master_address"], info["master_port"], info["rank_offset"], info["world_size"],
                                             "cpu", 30.0)
                threading.Thread(target=lambda: state["group"].barrier(30.0), daemon=True).start()
                return self._answer(200, {"success": True})
            if path == routes["update"] and state.get("pg") is not None:
                import torch.distributed as dist

                for name, dt, shape in zip(body["names"], body["dtypes"], body["shapes"]):
                    t = torch.empty(shape, dtype=getattr(torch, dt))
                    dist.broadcast(t, src=0, group=state["pg"])
                    state["weights"][name] = t.float()
                state["chunks"] += 1
                state["flushed"] = state.get("flushed", 0) + int(bool(body.get("flush_cache")))
                return self._answer(200, {"success": True})
            if path == routes["update"]:
                info = body.get("update_info", body)
                if state["chunks"] == fail_on_chunk:
                    # the worker still takes its side of the broadcast so that the trainer is not left waiting
                    buf = torch.empty(info["packed_bytes"], dtype=torch.uint8)
                    state["group"].broadcast(buf, src=0, timeout_s=30.0)
                    state["chunks"] += 1
                    return self._answer(400, {"error": "shape mismatch"})
                buf = torch.empty(info["packed_bytes"], dtype=torch.uint8)
                state["group"].broadcast(buf, src=0, timeout_s=30.0)
                names = info["names"]
                dtypes = info.get("dtype_names") or info.get("dtypes")
                offsets = info.get("offsets") or info.get("packed_offsets")
                for name, dt, shape, off in zip(names, dtypes, info["shapes"], offsets):
                    dtype = getattr(torch, dt)
                    nbytes = int(torch.tensor(shape).prod()) * torch.empty((), dtype=dtype).element_size()
                    state["weights"][name] = buf[off:off + nbytes].clone().view(dtype).view(shape).float()
                state["chunks"] += 1
                return self._answer(200, {"success": True})
            return self._answer(200, {"success": True})

    HTTPServer(("127.0.0.1", port), Handler).serve_forever()


def test_sglang_torch_plane_meets_a_worker_that_builds_its_group_the_stock_way(tmp_path):
    """The default SGLang data plane: a process group beside the default one on each side (rendezvous + prefixed store),
    one broadcast per tensor, the cache flushed by the update that ends the push."""
    import requests

    from halo_b200.weight_sync.clients import make_client

    port = _free_port()
    dump = str(tmp_path / "dump.json")
    proc = mp.get_context("spawn").Process(target=_fake_server, args=(port, "sglang", dump, -1), daemon=True)
    proc.start()
    try:
        client = make_client("sglang", f"http://127.0.0.1:{port}", model_id="tiny", group_host="127.0.0.1")     # data_plane="torch"
        client.check_server(total_timeout=30.0)
        g = torch.Generator().manual_seed(1)
        weights = {f"model.layers.{i}.mlp.down_proj.weight": torch.randn(12, 20, generator=g).bfloat16() for i in range(3)}
        weights["model.norm.weight"] = torch.randn(20, generator=g)
        client.push(weights)
        client.close()
        requests.get(f"http://127.0.0.1:{port}/dump", timeout=10)
        got = json.load(open(dump))
        for name, t in weights.items():
            assert torch.equal(torch.tensor(got["weights"][name]), t.float()), name
        calls = [c for c in got["calls"] if c not in ("/health", "/dump")]
        assert calls == ["/get_server_info", "/init_weights_update_group", "/pause_generation", "/update_weights_from_distributed",
                         "/continue_generation", "/destroy_weights_update_group"]
    finally:
        proc.terminate()
        proc.join(10)


@pytest.mark.parametrize("backend", ["vllm", "sglang"])
def test_push_reaches_the_fake_server_bit_for_bit(backend, tmp_path):
    import requests

    from halo_b200.weight_sync.clients import make_client

    port = _free_port()
    dump = str(tmp_path / "dump.json")
    proc = mp.get_context("spawn").Process(target=_fake_server, args=(port, backend, dump, -1), daemon=True)
    proc.start()
    try:
        extra = {"data_plane": "packed"} if backend == "sglang" else {}
        client = make_client(backend, f"http://127.0.0.1:{port}", model_id="tiny", chunk_bytes=4096, group_host="127.0.0.1", **extra)
        if backend == "vllm":
            assert client._plane("cpu") == "packed"        # vLLM's own trainer helpers need a GPU: the CPU test uses the packed plane
        client.check_server(total_timeout=30.0)
        info = client.read_server_info()
        assert info.world_size == 1 and info.max_model_len == 4096
        g = torch.Generator().manual_seed(0)
        weights = {f"layers.{i}.w": torch.randn(24, 40, generator=g).bfloat16() for i in range(5)}
        weights["norm"] = torch.randn(40, generator=g)
        client.push(weights)
        client.push(weights)              # a second update reuses the group and the staging buffer
        client.close()
        requests.get(f"http://127.0.0.1:{port}/dump", timeout=10)
        got = json.load(open(dump))
        for name, t in weights.items():
            assert torch.equal(torch.tensor(got["weights"][name]), t.float()), name
        calls = [c for c in got["calls"] if c not in ("/health", "/dump")]
        if backend == "vllm":
            first = calls[:calls.index("/update_weights")]
            assert first == ["/server_info", "/init_weight_transfer_engine", "/pause?mode=keep", "/start_weight_update"]
            assert calls[-2:] == ["/finish_weight_update", "/resume"]
        else:
            assert calls[:3] == ["/get_server_info", "/init_weights_update_group", "/pause_generation"]
            assert calls[-2:] == ["/continue_generation", "/destroy_weights_update_group"]
        assert got["chunks"] >= 4          # 4 KiB chunks: the tensors did not travel in one piece
    finally:
        proc.terminate()
        proc.join(10)


def test_a_failed_chunk_marks_the_server_unusable(tmp_path):
    from halo_b200.weight_sync.clients import EngineUnusable, make_client

    port = _free_port()
    proc = mp.get_context("spawn").Process(target=_fake_server, args=(port, "vllm", str(tmp_path / "d.json"), 1), daemon=True)
    proc.start()
    try:
        client = make_client("vllm", f"http://127.0.0.1:{port}", chunk_bytes=4096, group_host="127.0.0.1")
        client.check_server(total_timeout=30.0)
        weights = {f"w{i}": torch.full((32, 40), float(i)).bfloat16() for i in range(4)}
        with pytest.raises(RuntimeError, match="refused"):
            client.push(weights)
        assert "part old and part new" in client.unusable_reason
        assert not client.paused and not client.session_open and client.group is None
        with pytest.raises(EngineUnusable):
            client.push(weights)
    finally:
        proc.terminate()
        proc.join(10)


def test_completion_scores_are_read_from_both_answer_layouts():
    from halo_b200.weight_sync.clients.vllm import VLLMWeightSyncClient

    class Resp:
        status_code = 200
        text = ""

        def __init__(self, body):
            self._b = body

        def json(self):
            return self._b

    class Session:
        def __init__(self, body):
            self.body = body

        def request(self, method, url, json=None, params=None, timeout=None):
            self.sent = json
            return Resp(self.body)

    vllm_body = {"choices": [{"prompt_logprobs": [None, {"5": {"logprob": -0.1}}, {"7": {"logprob": -0.5}, "9": {"logprob": -2.0}},
                                                  {"8": {"logprob": -0.25}}]}]}
    c = VLLMWeightSyncClient("http://x", session=Session(vllm_body))
    assert c.score_completion_logprobs([1, 5], [7, 8]) == [-0.5, -0.25]
    openai_body = {"choices": [{"logprobs": {"token_logprobs": [None, -0.1, -0.5, -0.25]}}]}
    c = VLLMWeightSyncClient("http://x", session=Session(openai_body))
    assert c.score_completion_logprobs([1, 5], [7, 8]) == [-0.5, -0.25]


class _ScriptedClient:
    """A client whose completion route is a function of the request (no HTTP)."""

    def __init__(self, answer, info):
        from halo_b200.weight_sync.clients.base import ServerInfo

        self.model_id, self.info = "tiny", ServerInfo(**info)
        self._answer = answer
        self.began = self.ended = 0
        self.pushes = 0

    def check_server(self, total_timeout=0.0):
        pass

    def read_server_info(self):
        return self.info

    def request(self, method, route, json=None, timeout=None, retry=True, params=None):
        out = self._answer(json)
        if isinstance(out, Exception):
            raise out

        class R:
            def json(self_inner):
                return out

        return R()

    def begin_update(self, device=None):
        self.began += 1

    def end_update(self):
        self.ended += 1


def _good_answer(body):
    n = body.get("max_tokens", 1)
    temp = body.get("temperature", 1.0) or 1.0
    return {"choices": [{"logprobs": {"tokens": [f"token_id:{7 + i}" for i in range(n)],
                                      "token_logprobs": [-0.5 / max(temp, 0.1)] * n}}],
            "usage": {"completion_tokens": n}}


def test_preflight_accepts_a_well_configured_server_and_names_every_fault():
    from types import SimpleNamespace

    from halo_b200.trainers.grpo import engine_preflight as pf

    cfg = SimpleNamespace(vocab_size=1000)
    args = SimpleNamespace(max_prompt_length=512, max_completion_length=1024, temperature=0.7)
    good = _ScriptedClient(_good_answer, {"version": "0.11.0", "model_id": "tiny", "max_model_len": 4096})
    report = pf.run_preflight(good, cfg, args)
    assert not report.refusals and good.began == 1 and good.ended == 1
    assert report.facts["idle_tokens_per_s"] > 0

    def bad_answer(body):
        n = body.get("max_tokens", 1)
        if body.get("prompt") == [999]:
            return RuntimeError("token id out of range")
        return {"choices": [{"logprobs": {"tokens": ["hello"] * n, "token_logprobs": [-0.5] * n}}], "usage": {"completion_tokens": n}}

    bad = _ScriptedClient(bad_answer, {"version": "0.11.0", "model_id": "tiny", "max_model_len": 1024,
                                       "flags": {"quantization": "fp8"}})
    with pytest.raises(ValueError) as err:
        pf.run_preflight(bad, cfg, args)
    text = str(err.value)
    for needle in ("context window (1024)", "quantised weights (fp8)", "rejects token id 999", "sampled token ids",
                   "untempered distribution"):
        assert needle in text, needle
    assert bad.began == 0                      # no push is tried against a refused server


def test_server_rollout_source_builds_rollouts_with_sampler_logprobs():
    import numpy as np

    from halo_b200.weight_sync.engine_push import ServerRolloutSource

    class Resp:
        status_code = 200
        text = ""

        def __init__(self, body):
            self._b = body

        def json(self):
            return self._b

    class Session:
        def request(self, method, url, json=None, timeout=None):
            first = json["prompt"][0]
            return Resp({"choices": [{"logprobs": {"tokens": [f"token_id:{first}", f"token_id:{g}"], "token_logprobs": [-0.1, -0.2 * (g + 1)]}}
                                     for g in range(json["n"])]})

    src = ServerRolloutSource("http://x", "tiny", [np.array([3, 4]), np.array([5])], lambda p, c, t: float(c[-1]), num_generations=3,
                              max_new_tokens=2, prompts_per_round=2, session=Session())
    rollouts = src(0)
    assert len(rollouts) == 6
    assert [int(r.completion_ids[0]) for r in rollouts] == [3, 3, 3, 5, 5, 5]
    assert [r.reward for r in rollouts] == [0.0, 1.0, 2.0, 0.0, 1.0, 2.0]
    assert np.allclose(rollouts[4].sampler_logprobs, [-0.1, -0.4])
    assert src.mean_reward == 1.0


def test_adapter_pusher_loads_the_new_version_before_it_unloads_the_old(tmp_path):
    import os

    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.peft.lora import LoraSpec, apply_lora
    from halo_b200.weight_sync.adapter_push import AdapterPusher

    class Client:
        model_id = "base"

        def __init__(self):
            self.calls = []

        def load_adapter(self, name, path):
            assert os.path.isfile(os.path.join(path, "adapter_config.json")), "the adapter must be on disk before it is announced"
            self.calls.append(("load", name))

        def unload_adapter(self, name):
            self.calls.append(("unload", name))

        def close(self):
            self.calls.append(("close", ""))

    model = build_model(PRESETS["tiny-moe"](), device="cpu", dtype=torch.float32)
    apply_lora(model, LoraSpec(r=4, alpha=8.0, target_modules=["q_proj", "v_proj"]))
    client = Client()
    pusher = AdapterPusher(client, str(tmp_path), name="policy", keep_versions=2)
    assert pusher.current_model_id == "base"
    for _ in range(3):
        pusher.push(model)
    assert pusher.current_model_id == "policy-v3"
    assert client.calls == [("load", "policy-v1"), ("load", "policy-v2"), ("unload", "policy-v1"), ("load", "policy-v3"),
                            ("unload", "policy-v2")]
    assert sorted(os.listdir(tmp_path)) == ["policy-v2", "policy-v3"]        # older directories are removed
    pusher.close()
    assert client.calls[-2:] == [("unload", "policy-v3"), ("close", "")]

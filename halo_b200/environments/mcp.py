"""Model Context Protocol client and the ``mcp`` environment: tools served by MCP servers (child processes speaking
JSON-RPC 2.0 over stdin / stdout, one JSON object per line) appear to the policy as ordinary function tools.

The client is synchronous and small on purpose: an episode runs on a worker thread of the rollout loop, every request
has a deadline (a hung server costs the episode one tool error, not its whole time budget), and ``close()`` never waits
longer than a few seconds for a server to leave. The protocol subset is what tool use needs: ``initialize`` ->
``notifications/initialized`` -> ``tools/list`` -> ``tools/call``.

Known servers are listed by name (``MCP_SERVERS``) with the environment variables they need; a server that needs a
directory gets a scratch directory of its own that dies with the episode. Any other server is given as
``{"command": ..., "args": [...], "env": {...}}``.

Counterpart of halo/environments/protocols/mcp.py:1-434 (which drives the ``mcp`` SDK's asyncio sessions).
"""

from __future__ import annotations

import json
import os
import queue
import shutil
import subprocess
import tempfile
import threading

from .protocols import ToolCall, ToolRegistry
from .registry import register_environment
from .tasks import ToolQAEnvironment

PROTOCOL_VERSION = "2024-11-05"
REQUEST_TIMEOUT_S = 120.0
DISCONNECT_TIMEOUT_S = 5.0

MCP_SERVERS = {
    "filesystem": {"command": "npx", "args": ["-y", "@modelcontextprotocol/server-filesystem"], "env": [], "scratch_arg": True},
    "fetch": {"command": "uvx", "args": ["mcp-server-fetch"], "env": []},
    "memory": {"command": "npx", "args": ["-y", "@modelcontextprotocol/server-memory"], "env": [],
               "scratch_env": {"MEMORY_FILE_PATH": "memory.jsonl"}},
    "brave_search": {"command": "npx", "args": ["-y", "@modelcontextprotocol/server-brave-search"], "env": ["BRAVE_API_KEY"]},
    "github": {"command": "npx", "args": ["-y", "@modelcontextprotocol/server-github"], "env": ["GITHUB_PERSONAL_ACCESS_TOKEN"]},
}


class McpError(RuntimeError):
    pass


class McpStdioClient:
    """One server process. ``request`` is safe to call from one thread at a time."""

    def __init__(self, command: str, args: list[str] | None = None, env: dict | None = None, cwd: str | None = None,
                 request_timeout_s: float = REQUEST_TIMEOUT_S):
        if shutil.which(command) is None and not os.path.isfile(command):
            raise McpError(f"MCP server command {command!r} is not on PATH")
        self.request_timeout_s = request_timeout_s
        full_env = {k: v for k, v in os.environ.items() if k in ("PATH", "HOME", "LANG", "LC_ALL", "TMPDIR", "PYTHONPATH")}
        full_env.update(env or {})
        self.proc = subprocess.Popen([command, *(args or [])], stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                     env=full_env, cwd=cwd, text=True, bufsize=1)
        self._answers: queue.Queue = queue.Queue()
        self._next_id = 0
        self._reader = threading.Thread(target=self._read, name="mcp-reader", daemon=True)
        self._reader.start()
        self.server_info: dict = {}

    def _read(self) -> None:
        for line in self.proc.stdout:
            line = line.strip()
            if not line:
                continue
            try:
                msg = json.loads(line)
            except json.JSONDecodeError:
                continue                         # servers may log to stdout; only JSON-RPC objects count
            if isinstance(msg, dict) and "id" in msg and ("result" in msg or "error" in msg):
                self._answers.put(msg)
        self._answers.put(None)                  # the server closed its stdout

    def _send(self, obj: dict) -> None:
        try:
            self.proc.stdin.write(json.dumps(obj) + "\n")
            self.proc.stdin.flush()
        except (BrokenPipeError, OSError) as exc:
            raise McpError(f"the MCP server is gone: {exc}") from exc

    def notify(self, method: str, params: dict | None = None) -> None:
        self._send({"jsonrpc": "2.0", "method": method, **({"params": params} if params else {})})

    def request(self, method: str, params: dict | None = None, timeout_s: float | None = None) -> dict:
        self._next_id += 1
        rid = self._next_id
        self._send({"jsonrpc": "2.0", "id": rid, "method": method, "params": params or {}})
        deadline = timeout_s if timeout_s is not None else self.request_timeout_s
        while True:
            try:
                msg = self._answers.get(timeout=deadline)
            except queue.Empty:
                raise McpError(f"the MCP server did not answer {method} within {deadline:g} s") from None
            if msg is None:
                raise McpError(f"the MCP server exited before answering {method}")
            if msg.get("id") != rid:
                continue                         # the answer to a request that timed out earlier
            if "error" in msg:
                err = msg["error"]
                raise McpError(f"{method}: {err.get('message', err)} (code {err.get('code')})")
            return msg["result"]

    def initialize(self, client_name: str = "halo_b200") -> dict:
        result = self.request("initialize", {"protocolVersion": PROTOCOL_VERSION, "capabilities": {},
                                             "clientInfo": {"name": client_name, "version": "1"}})
        self.server_info = result.get("serverInfo", {})
        self.notify("notifications/initialized")
        return result

    def list_tools(self) -> list[dict]:
        tools, cursor = [], None
        while True:
            result = self.request("tools/list", {"cursor": cursor} if cursor else {})
            tools += result.get("tools", [])
            cursor = result.get("nextCursor")
            if not cursor:
                return tools

    def call_tool(self, name: str, arguments: dict) -> str:
        result = self.request("tools/call", {"name": name, "arguments": arguments})
        parts = [c.get("text", "") for c in result.get("content", []) if c.get("type") == "text"]
        text = "\n".join(p for p in parts if p)
        return ("error: " + text) if result.get("isError") else text

    def close(self) -> None:
        try:
            if self.proc.stdin:
                self.proc.stdin.close()
            self.proc.wait(DISCONNECT_TIMEOUT_S)
        except Exception:  # noqa: BLE001
            self.proc.kill()
            try:
                self.proc.wait(DISCONNECT_TIMEOUT_S)
            except Exception:  # noqa: BLE001
                pass


def resolve_server(spec) -> tuple[dict, str | None]:
    """``spec``: a name of ``MCP_SERVERS`` or a ``{"command", "args", "env"}`` mapping. Returns the launch mapping and the
    scratch directory created for it (or None)."""
    if isinstance(spec, dict):
        if "command" not in spec:
            raise ValueError("an MCP server mapping needs a 'command'")
        return {"command": spec["command"], "args": list(spec.get("args", [])), "env": dict(spec.get("env", {}))}, None
    if spec not in MCP_SERVERS:
        raise KeyError(f"unknown MCP server {spec!r}; known: {sorted(MCP_SERVERS)} (or give a command mapping)")
    known = MCP_SERVERS[spec]
    missing = [k for k in known["env"] if not os.environ.get(k)]
    if missing:
        raise McpError(f"MCP server {spec!r} needs the environment variable(s) {missing}")
    env = {k: os.environ[k] for k in known["env"]}
    args = list(known["args"])
    scratch = None
    if known.get("scratch_arg") or known.get("scratch_env"):
        scratch = tempfile.mkdtemp(prefix=f"mcp_{spec}_")
        if known.get("scratch_arg"):
            args.append(scratch)                 # the directory is the server's whole access allowlist
        for k, rel in (known.get("scratch_env") or {}).items():
            env[k] = os.path.join(scratch, rel)
    return {"command": known["command"], "args": args, "env": env}, scratch


def bridge_tools(client: McpStdioClient, registry: ToolRegistry, prefix: str = "") -> list[str]:
    """Register every tool the server lists as a function tool of ``registry``."""
    names = []
    for tool in client.list_tools():
        schema = tool.get("inputSchema") or {}
        required = set(schema.get("required", []))
        params = {}
        for pname, p in (schema.get("properties") or {}).items():
            entry = {k: v for k, v in p.items() if k in ("type", "description", "enum", "items")}
            entry.setdefault("type", "string")
            if pname not in required:
                entry["optional"] = True
            params[pname] = entry
        name = prefix + tool["name"]

        def call(_tool=tool["name"], **arguments):
            return client.call_tool(_tool, arguments)

        registry.register(name, tool.get("description", ""), params, call)
        names.append(name)
    return names


@register_environment("mcp")
class McpEnvironment(ToolQAEnvironment):
    """``tool_qa`` whose tools come from MCP servers (option ``servers``: names or command mappings). Tool names are
    prefixed with the server's name when several servers are connected."""

    env_type = "mcp"

    def __init__(self, task, **options):
        servers = options.get("servers") or task.get("servers") or []
        if not servers:
            raise ValueError("the mcp environment needs servers: [name or {command, args, env}, ...]")
        registry = ToolRegistry()
        self.clients, self.scratch = [], []
        try:
            for spec in servers:
                launch, scratch = resolve_server(spec)
                if scratch:
                    self.scratch.append(scratch)
                client = McpStdioClient(launch["command"], launch["args"], launch["env"],
                                        request_timeout_s=float(options.get("request_timeout_s", REQUEST_TIMEOUT_S)))
                self.clients.append(client)
                client.initialize()
                label = spec if isinstance(spec, str) else client.server_info.get("name", f"server{len(self.clients)}")
                bridge_tools(client, registry, prefix=f"{label}__" if len(servers) > 1 else "")
        except Exception:
            self._shutdown()
            raise
        super().__init__(task, **{**options, "tools": registry})

    def _shutdown(self) -> None:
        for c in self.clients:
            c.close()
        for d in self.scratch:
            shutil.rmtree(d, ignore_errors=True)
        self.clients, self.scratch = [], []

    def close(self):
        self._shutdown()
        super().close()


__all__ = ["McpStdioClient", "McpEnvironment", "McpError", "bridge_tools", "resolve_server", "MCP_SERVERS", "ToolCall"]

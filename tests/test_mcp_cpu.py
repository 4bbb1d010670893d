"""The MCP client and environment against a fake server process (tests/common/fake_mcp_server.py)."""

import os
import sys

import pytest

SERVER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "common", "fake_mcp_server.py")


def test_client_lists_pages_of_tools_and_calls_them():
    from halo_b200.environments.mcp import McpError, McpStdioClient

    client = McpStdioClient(sys.executable, [SERVER], request_timeout_s=20.0)
    try:
        client.initialize()
        assert client.server_info["name"] == "fake"
        assert [t["name"] for t in client.list_tools()] == ["add", "lookup", "hang"]
        assert client.call_tool("add", {"a": 2, "b": 40}) == "42"
        assert client.call_tool("lookup", {"key": "nothing"}).startswith("error: no entry")
        with pytest.raises(McpError, match="no tool"):
            client.call_tool("absent", {})
        with pytest.raises(McpError, match="did not answer"):
            client.request("tools/call", {"name": "hang", "arguments": {}}, timeout_s=0.5)
    finally:
        client.close()
    assert client.proc.poll() is not None          # close() does not leave the server behind


def test_mcp_environment_plays_an_episode_with_bridged_tools():
    from halo_b200.environments.base import Turn
    from halo_b200.environments.registry import make_environment

    env = make_environment("mcp", {"question": "What is the capital of France?", "answer": "Paris"},
                           servers=[{"command": sys.executable, "args": [SERVER]}], request_timeout_s=20.0)
    try:
        names = [d["function"]["name"] for d in env.tools()]
        assert names == ["add", "lookup", "hang"]
        lookup = next(d for d in env.tools() if d["function"]["name"] == "lookup")
        assert lookup["function"]["parameters"]["required"] == ["key"]
        env.reset()
        call = Turn("assistant", "", tool_calls=[{"id": "c1", "type": "function",
                                         "function": {"name": "lookup", "arguments": '{"key": "capital_of_france"}'}}])
        messages, done = env.step(call)
        assert not done and messages[0]["role"] == "tool" and messages[0]["content"] == "Paris"
        bad = Turn("assistant", "", tool_calls=[{"id": "c2", "type": "function", "function": {"name": "lookup", "arguments": "{}"}}])
        messages, done = env.step(bad)
        assert "missing ['key']" in messages[0]["content"]
        _, done = env.step(Turn("assistant", "Paris"))
        assert done and env.score() == 1.0
    finally:
        env.close()


def test_known_servers_refuse_without_their_credentials(monkeypatch):
    from halo_b200.environments.mcp import McpError, resolve_server

    monkeypatch.delenv("BRAVE_API_KEY", raising=False)
    with pytest.raises(McpError, match="BRAVE_API_KEY"):
        resolve_server("brave_search")
    launch, scratch = resolve_server("memory")
    try:
        assert scratch and launch["env"]["MEMORY_FILE_PATH"].startswith(scratch)
    finally:
        os.rmdir(scratch)
    with pytest.raises(KeyError):
        resolve_server("nope")

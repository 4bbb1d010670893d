"""A minimal MCP server over stdin / stdout for tests: tools ``add`` and ``lookup`` (and ``hang`` that never answers)."""

import json
import sys
import time

TOOLS = [
    {"name": "add", "description": "Add two numbers.", "inputSchema": {"type": "object", "properties": {
        "a": {"type": "number"}, "b": {"type": "number"}}, "required": ["a", "b"]}},
    {"name": "lookup", "description": "Look a key up.", "inputSchema": {"type": "object", "properties": {
        "key": {"type": "string"}, "default": {"type": "string"}}, "required": ["key"]}},
    {"name": "hang", "description": "Never answers.", "inputSchema": {"type": "object", "properties": {}}},
]
FACTS = {"capital_of_france": "Paris"}

print("starting fake server (a log line on stdout that is not JSON-RPC)", flush=True)
for line in sys.stdin:
    msg = json.loads(line)
    if "id" not in msg:
        continue
    method, params = msg["method"], msg.get("params", {})
    if method == "initialize":
        result = {"protocolVersion": params["protocolVersion"], "capabilities": {"tools": {}}, "serverInfo": {"name": "fake", "version": "0"}}
    elif method == "tools/list":
        cursor = params.get("cursor")
        result = {"tools": TOOLS[:2], "nextCursor": "page2"} if not cursor else {"tools": TOOLS[2:]}
    elif method == "tools/call":
        name, args = params["name"], params.get("arguments", {})
        if name == "add":
            result = {"content": [{"type": "text", "text": str(args["a"] + args["b"])}]}
        elif name == "lookup":
            hit = FACTS.get(args["key"], args.get("default"))
            result = ({"content": [{"type": "text", "text": hit}]} if hit is not None
                      else {"content": [{"type": "text", "text": f"no entry {args['key']!r}"}], "isError": True})
        elif name == "hang":
            time.sleep(3600)
        else:
            print(json.dumps({"jsonrpc": "2.0", "id": msg["id"], "error": {"code": -32601, "message": f"no tool {name}"}}), flush=True)
            continue
    else:
        print(json.dumps({"jsonrpc": "2.0", "id": msg["id"], "error": {"code": -32601, "message": "method not found"}}), flush=True)
        continue
    print(json.dumps({"jsonrpc": "2.0", "id": msg["id"], "result": result}), flush=True)

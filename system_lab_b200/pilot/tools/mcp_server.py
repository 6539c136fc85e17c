"""Minimal JSON-RPC 2.0 tool server over stdio (the MCP subset an agent host needs: ``initialize``,
``tools/list``, ``tools/call``) exposing the Pilot worker tools with their real handlers.

The reference's integration config points at ``python -m pilot.tools.mcp_server`` but does not ship the
module (``pilot/integrations/cursor/mcp.json.example:1-20``); this is that server for this framework.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from ..agent.state import StateStore
from ..agent.worker_tools import ALL_TOOLS, ToolContext, handle_tool_call
from ..runner import JobRunner


def serve(ctx: ToolContext, stdin=sys.stdin, stdout=sys.stdout) -> None:
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        try:
            req = json.loads(line)
        except json.JSONDecodeError:
            continue
        rid, method, params = req.get("id"), req.get("method"), req.get("params") or {}
        try:
            if method == "initialize":
                result = {"protocolVersion": "2024-11-05", "serverInfo": {"name": "pilot-tools", "version": "0.1"},
                          "capabilities": {"tools": {}}}
            elif method == "tools/list":
                result = {"tools": [{"name": t["name"], "description": t["description"],
                                     "inputSchema": t["input_schema"]} for t in ALL_TOOLS
                                    if t["name"] != "return_subagent_result"]}
            elif method == "tools/call":
                out = handle_tool_call(params["name"], params.get("arguments") or {}, ctx)
                result = {"content": [{"type": "text", "text": json.dumps(out, default=str)}]}
            elif method and method.startswith("notifications/"):
                continue
            else:
                raise ValueError(f"unknown method {method}")
            resp = {"jsonrpc": "2.0", "id": rid, "result": result}
        except Exception as e:
            resp = {"jsonrpc": "2.0", "id": rid, "error": {"code": -32000, "message": f"{type(e).__name__}: {e}"}}
        stdout.write(json.dumps(resp) + "\n")
        stdout.flush()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("pilot-mcp")
    ap.add_argument("--state-dir", default="pilot/state", type=Path)
    ap.add_argument("--session", default="mcp")
    ap.add_argument("--preset", default="simplemoe-tiny")
    ap.add_argument("--nproc", type=int, default=1)
    args = ap.parse_args(argv)
    store = StateStore(args.state_dir / args.session)
    runner = JobRunner(store.jobs_dir, args.preset, (), args.nproc)
    serve(ToolContext(store, runner, args.preset, (), world=max(args.nproc, 1)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

"""Cluster dashboard: every rank writes a small status file while it trains; ``idrak cluster ui`` reads the folder and
shows one row per rank (step, loss, tokens/s, memory, network bytes, seconds since the last beat), as text in the
terminal or as a page served over HTTP that refreshes itself.

    writer = StatusWriter(folder, rank, world)            # in the training loop
    writer.update(step=s, loss=l, tokens_per_s=t, memory_bytes=m, network=comm.network_summary())

Files are written to a temporary name and renamed, so a reader never sees half a file. A rank whose file is older than
``stale_after`` seconds is shown as silent - the same signal the heartbeat uses (``cluster.heartbeat``).

Reference: the cluster dashboard of the command line (src/Idrak.Cli.Commands/Commands/Cluster/ClusterUiCommand.cs).
"""
from __future__ import annotations

import html
import json
import os
import time
from typing import Any, Dict, List, Optional

FORMAT = "idrak-rank-status/1"


class StatusWriter:
    def __init__(self, folder: str, rank: int, world: int, name: str = ""):
        self.folder, self.rank, self.world, self.name = folder, rank, world, name
        os.makedirs(folder, exist_ok=True)
        self.path = os.path.join(folder, f"rank-{rank:04d}.json")
        self.started = time.time()
        self.fields: Dict[str, Any] = {}

    def update(self, **fields) -> None:
        self.fields.update(fields)
        doc = {"format": FORMAT, "rank": self.rank, "world": self.world, "name": self.name, "time": time.time(),
               "started": self.started, **self.fields}
        tmp = self.path + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            json.dump(doc, f)
        os.replace(tmp, self.path)

    def finish(self, reason: str = "finished") -> None:
        self.update(state=reason)


def read_status(folder: str, stale_after: float = 10.0, now: Optional[float] = None) -> List[Dict[str, Any]]:
    """One dict per rank file, in rank order, with ``age`` (seconds since its last update) and ``state``: what the rank
    wrote (``finished``, ``stopped`` ...), else ``running`` or - past ``stale_after`` - ``silent``."""
    now = time.time() if now is None else now
    rows = []
    for name in sorted(os.listdir(folder)) if os.path.isdir(folder) else []:
        if not (name.startswith("rank-") and name.endswith(".json")):
            continue
        try:
            with open(os.path.join(folder, name), "r", encoding="utf-8") as f:
                d = json.load(f)
        except (OSError, ValueError):
            continue                      # being replaced right now: next refresh has it
        if d.get("format") != FORMAT:
            continue
        d["age"] = max(0.0, now - float(d.get("time", now)))
        if "state" not in d:
            d["state"] = "silent" if d["age"] > stale_after else "running"
        rows.append(d)
    rows.sort(key=lambda d: d["rank"])
    return rows


def _bytes(n) -> str:
    n = float(n or 0)
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if n < 1024 or unit == "TiB":
            return f"{n:.0f} {unit}" if unit == "B" else f"{n:.1f} {unit}"
        n /= 1024
    return ""


COLUMNS = [("rank", "rank"), ("state", "state"), ("step", "step"), ("loss", "loss"), ("tokens_per_s", "tokens/s"),
           ("memory_bytes", "memory"), ("sent", "sent"), ("read", "read"), ("age", "last beat")]


def _cells(d: Dict[str, Any]) -> List[str]:
    net = d.get("network") or {}
    return [str(d["rank"]), str(d["state"]), str(d.get("step", "")),
            f"{d['loss']:.4f}" if isinstance(d.get("loss"), (int, float)) else "",
            f"{d['tokens_per_s']:,.0f}" if isinstance(d.get("tokens_per_s"), (int, float)) else "",
            _bytes(d["memory_bytes"]) if d.get("memory_bytes") is not None else "",
            _bytes(net.get("bytes_sent")) if net else "", _bytes(net.get("bytes_read")) if net else "",
            f"{d['age']:.1f} s"]


def summary(rows: List[Dict[str, Any]]) -> Dict[str, Any]:
    rates = [d["tokens_per_s"] for d in rows if isinstance(d.get("tokens_per_s"), (int, float)) and d["state"] == "running"]
    steps = [d["step"] for d in rows if isinstance(d.get("step"), int)]
    return {"ranks": len(rows), "world": rows[0]["world"] if rows else 0,
            "running": sum(d["state"] == "running" for d in rows), "silent": [d["rank"] for d in rows if d["state"] == "silent"],
            "tokens_per_s": sum(rates), "step_min": min(steps) if steps else None, "step_max": max(steps) if steps else None}


def render_text(rows: List[Dict[str, Any]]) -> str:
    table = [[h for _, h in COLUMNS]] + [_cells(d) for d in rows]
    widths = [max(len(r[i]) for r in table) for i in range(len(COLUMNS))]
    lines = ["  ".join(c.rjust(w) for c, w in zip(r, widths)) for r in table]
    s = summary(rows)
    missing = s["world"] - s["ranks"] if s["world"] else 0
    tail = (f"{s['running']} of {s['world'] or s['ranks']} ranks running, {s['tokens_per_s']:,.0f} tokens/s in all"
            + (f", steps {s['step_min']}..{s['step_max']}" if s["step_min"] is not None else "")
            + (f", silent: {s['silent']}" if s["silent"] else "") + (f", {missing} never reported" if missing > 0 else ""))
    return "\n".join(lines + [tail])


def render_html(rows: List[Dict[str, Any]], refresh: float = 2.0) -> str:
    head = "".join(f"<th>{html.escape(h)}</th>" for _, h in COLUMNS)
    body = "".join("<tr class='{}'>{}</tr>".format(html.escape(str(d["state"])),
                                                   "".join(f"<td>{html.escape(c)}</td>" for c in _cells(d))) for d in rows)
    s = summary(rows)
    return (f"<!doctype html><html><head><meta charset='utf-8'><meta http-equiv='refresh' content='{refresh:g}'>"
            "<title>idrak cluster</title><style>body{font-family:monospace}td,th{padding:2px 10px;text-align:right}"
            "tr.silent{background:#fdd}tr.finished{color:#777}</style></head><body>"
            f"<p>{s['running']} of {s['world'] or s['ranks']} ranks running &middot; {s['tokens_per_s']:,.0f} tokens/s</p>"
            f"<table><tr>{head}</tr>{body}</table></body></html>")


def serve(folder: str, host: str = "127.0.0.1", port: int = 0, stale_after: float = 10.0):
    """``GET /`` the page, ``GET /status.json`` the rows. Returns the running server (``.shutdown()`` stops it)."""
    import threading
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_GET(self):
            rows = read_status(folder, stale_after)
            if self.path.startswith("/status.json"):
                body, kind = json.dumps({"summary": summary(rows), "ranks": rows}).encode(), "application/json"
            elif self.path in ("/", "/index.html"):
                body, kind = render_html(rows).encode(), "text/html; charset=utf-8"
            else:
                self.send_response(404)
                self.end_headers()
                return
            self.send_response(200)
            self.send_header("Content-Type", kind)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)
    httpd = ThreadingHTTPServer((host, port), Handler)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    return httpd


def local_rank_commands(topology, node: str, script: List[str], master_port: int = 29500) -> List[Dict[str, Any]]:
    """What ``cluster start`` runs on ``node``: one process per GPU of that node with the rendezvous variables set
    (RANK, LOCAL_RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT), the first node's address as the master."""
    ranks = [r for r in topology.ranks() if r["node"] == node]
    if not ranks:
        raise KeyError(f"node '{node}' is not in the topology; known: {', '.join(n.name for n in topology.nodes)}")
    master = topology.ranks()[0]["address"]
    out = []
    for local, r in enumerate(ranks):
        env = {"RANK": str(r["rank"]), "LOCAL_RANK": str(local), "WORLD_SIZE": str(topology.world),
               "LOCAL_WORLD_SIZE": str(len(ranks)), "MASTER_ADDR": master, "MASTER_PORT": str(master_port)}
        out.append({"rank": r["rank"], "device": r["device"], "env": env, "command": list(script)})
    return out

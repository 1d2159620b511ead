"""More commands: `train` / `predict` for networks described as JSON over CSV data, `runs`, `cluster` (init, inspect,
sim, replay), `transports`, `env`, `completion`, `alias`, `verify`, `list`, `bench-compare` and `train-tokenizer`.

Reference: the command groups of src/Idrak.Cli.Commands (Train, Cluster, Config, Models, Health), README.md:277-289.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import time
from typing import List


def _home() -> str:
    from .. import config
    return os.path.expanduser(config.get("IDRAK_HOME") or "~/.idrak")


# ------------------------------------------------------------------------------------------- train / predict
def _read_table(path: str, target: str):
    import csv

    import torch
    with open(path, newline="", encoding="utf-8") as f:
        rows = list(csv.DictReader(f))
    if not rows:
        raise SystemExit(f"{path}: no rows")
    if target and target not in rows[0]:
        raise SystemExit(f"{path}: no column named '{target}' (columns: {', '.join(rows[0])})")
    features = [c for c in rows[0] if c != target]
    x = torch.tensor([[float(r[c]) for c in features] for r in rows])
    y = torch.tensor([[float(r[target])] for r in rows]) if target else None
    return features, x, y


def cmd_train(a) -> int:
    """Fit a network (JSON description, or a default two-layer one) to a CSV table and write a run folder."""
    import torch

    from ..formats import ikw
    from ..nn.builder import Network
    from ..training.trainer import CsvLogger, Trainer
    features, x, y = _read_table(a.data, a.target)
    torch.manual_seed(a.seed)
    if a.network:
        with open(a.network, "r", encoding="utf-8") as f:
            builder = Network.from_json(json.load(f))
    else:
        builder = Network.input(len(features)).linear(a.hidden).relu().linear(a.hidden).relu().linear(1)
    net = builder.build()
    n_val = int(len(x) * a.validation)
    perm = torch.randperm(len(x), generator=torch.Generator().manual_seed(a.seed))
    xv, yv, xt, yt = x[perm[:n_val]], y[perm[:n_val]], x[perm[n_val:]], y[perm[n_val:]]
    xm, xs, ym, ys = xt.mean(0), xt.std(0).clamp_min(1e-6), yt.mean(0), yt.std(0).clamp_min(1e-6)
    if a.task == "classification":
        ym, ys = torch.zeros(1), torch.ones(1)
        loss = torch.nn.functional.binary_cross_entropy_with_logits
    else:
        loss = torch.nn.functional.mse_loss
    def batches(xs_, ys_):
        return [((xs_[i: i + a.batch] - xm) / xs, (ys_[i: i + a.batch] - ym) / ys) for i in range(0, len(xs_), a.batch)]
    os.makedirs(a.output, exist_ok=True)
    trainer = Trainer(net, torch.optim.AdamW(net.parameters(), lr=a.lr), loss,
                      callbacks=[CsvLogger(os.path.join(a.output, "log.csv"))])
    t0 = time.time()
    trainer.fit(batches(xt, yt), epochs=a.epochs, validation=batches(xv, yv) if n_val else None)
    ikw.save_module(net, os.path.join(a.output, "model.ikw"))
    result = trainer.evaluate(batches(xv, yv) if n_val else batches(xt, yt))
    with open(os.path.join(a.output, "run.json"), "w", encoding="utf-8") as f:
        json.dump({"format": "idrak-run/1", "task": a.task, "features": features, "target": a.target,
                   "network": builder.to_json(), "x_mean": xm.tolist(), "x_std": xs.tolist(), "y_mean": ym.tolist(),
                   "y_std": ys.tolist(), "epochs": a.epochs, "rows": len(x), "loss": result.loss, "seconds": round(time.time() - t0, 2),
                   "finished": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}, f, indent=1)
    print(f"{len(xt)} rows, {a.epochs} epochs: {'validation' if n_val else 'training'} loss {result.loss:.5f}; run written to {a.output}")
    return 0


def _load_run(folder: str):
    import torch

    from ..formats import ikw
    from ..nn.builder import Network
    with open(os.path.join(folder, "run.json"), "r", encoding="utf-8") as f:
        run = json.load(f)
    net = Network.from_json(run["network"]).build()
    ikw.load_module(net, os.path.join(folder, "model.ikw"))
    return run, net.eval(), {k: torch.tensor(run[k]) for k in ("x_mean", "x_std", "y_mean", "y_std")}


def cmd_predict(a) -> int:
    import torch
    run, net, s = _load_run(a.run)
    if a.data:
        _, x, _ = _read_table(a.data, run["target"] if a.has_target else "")
        x = x[:, : len(run["features"])]
    else:
        x = torch.tensor([[float(v) for v in a.values]])
    if x.shape[1] != len(run["features"]):
        raise SystemExit(f"expected {len(run['features'])} values ({', '.join(run['features'])}), got {x.shape[1]}")
    with torch.no_grad():
        y = net((x - s["x_mean"]) / s["x_std"]) * s["y_std"] + s["y_mean"]
        if run["task"] == "classification":
            y = torch.sigmoid(y)
    for row in y.tolist():
        print(" ".join(f"{v:.6g}" for v in row))
    return 0


def cmd_runs(a) -> int:
    """List the run folders under a directory, newest first."""
    rows = []
    for name in sorted(os.listdir(a.folder)) if os.path.isdir(a.folder) else []:
        for meta in ("run.json", "train-state.json"):
            p = os.path.join(a.folder, name, meta)
            if os.path.isfile(p):
                with open(p, "r", encoding="utf-8") as f:
                    d = json.load(f)
                rows.append((os.path.getmtime(p), name, d))
                break
    rows.sort(reverse=True)
    if a.json:
        print(json.dumps([{"name": n, **d} for _, n, d in rows]))
        return 0
    for _, name, d in rows:
        loss = d.get("loss", d.get("best_loss"))
        print(f"{name:30s} {d.get('finished', ''):22s} epochs {d.get('epochs', d.get('epoch', '?'))}  "
              f"loss {loss if loss is None else round(float(loss), 5)}")
    if not rows:
        print(f"no runs under {a.folder}")
    return 0


# ------------------------------------------------------------------------------------------- cluster
def cmd_cluster(a) -> int:
    from ..cluster import sim
    from ..cluster.topology import load_topology
    if a.action == "init":
        nodes = [{"name": f"node{i}", "address": "127.0.0.1" if a.nodes == 1 else f"10.0.0.{i + 1}",
                  "gpus": [{"device": g, "memory": a.memory} for g in range(a.gpus)]} for i in range(a.nodes)]
        doc = {"format": "idrak-topology/1", "nodes": nodes, "links": {"intra-node": "nvlink", "inter-node": a.inter_node}}
        text = json.dumps(doc, indent=2)
        if a.path:
            with open(a.path, "w", encoding="utf-8") as f:
                f.write(text + "\n")
            print(f"wrote {a.path}: {a.nodes} node(s) x {a.gpus} GPU(s)")
        else:
            print(text)
        return 0
    if a.action == "inspect":
        topo = load_topology(a.path)
        for r in topo.ranks():
            print(f"rank {r['rank']:3d}  {r['node']:10s} {r['address']:15s} cuda:{r['device']:<3d} {r['memory']}")
        names = [n.name for n in topo.nodes]
        print(f"world {topo.world}; inside a node: {topo.link_type(names[0], names[0])}"
              + (f"; between nodes: {topo.link_type(names[0], names[1])}" if len(names) > 1 else ""))
        if a.bytes:
            from ..cluster.links import ClusterCache, predict_all_reduce
            measured = ClusterCache(os.path.join(_home(), "cluster.json")).load()
            for algorithm in ("naive", "ring", "hierarchical"):
                t = predict_all_reduce(topo, a.bytes, algorithm, measured)
                print(f"predicted {algorithm:12s} all-reduce of {a.bytes} bytes: {t * 1e3:.3f} ms")
        return 0
    if a.action == "ui":
        # path: the folder the ranks write their status files to
        from ..cluster import dashboard
        if a.serve is not None:
            httpd = dashboard.serve(a.path, port=a.serve)
            print(f"http://127.0.0.1:{httpd.server_address[1]}/  (Ctrl-C stops)")
            try:
                while True:
                    time.sleep(1.0)
            except KeyboardInterrupt:
                httpd.shutdown()
            return 0
        while True:
            rows = dashboard.read_status(a.path)
            print(dashboard.render_text(rows))
            if a.once or not rows or all(r["state"] not in ("running",) for r in rows):
                return 0 if not any(r["state"] == "silent" for r in rows) else 1
            time.sleep(a.refresh)
            print()
    if a.action == "start":
        # path: topology file; everything after "--" is the program every rank runs
        import subprocess
        from ..cluster import dashboard
        topo = load_topology(a.path)
        node = a.node or topo.nodes[0].name
        jobs = dashboard.local_rank_commands(topo, node, a.program or [sys.executable, "-c", "print('rank up')"], a.master_port)
        if a.dry_run:
            for j in jobs:
                print(f"rank {j['rank']} cuda:{j['device']}: " + " ".join(f"{k}={v}" for k, v in j["env"].items()) + "  " + " ".join(j["command"]))
            return 0
        procs = [subprocess.Popen(j["command"], env={**os.environ, **j["env"]}) for j in jobs]
        codes = [p.wait() for p in procs]
        bad = [(j["rank"], c) for j, c in zip(jobs, codes) if c != 0]
        for r, c in bad:
            print(f"rank {r} exited with {c}")
        return 1 if bad else 0
    if a.action == "calibrate":
        # path: CSV of "bytes,seconds" rows measured on the link (the link bench prints them); stored under --link
        from ..cluster.links import ClusterCache, LinkCalibration
        with open(a.path, "r", encoding="utf-8") as f:
            rows = [line.strip().split(",") for line in f if line.strip() and line[0].isdigit()]
        cal = LinkCalibration.fit([(float(r[0]), float(r[1])) for r in rows])
        ClusterCache(os.path.join(_home(), "cluster.json")).store(a.link, cal)
        print(f"{a.link}: latency {cal.link.latency * 1e6:.2f} us, bandwidth {cal.link.bandwidth / 1e9:.2f} GB/s, "
              f"r2 {cal.r2:.5f} over {cal.samples} samples")
        return 0
    if a.action in ("sim", "replay"):
        import numpy as np
        if a.action == "replay":
            failures = sim.ClusterReplay(sim.EventLog.load(a.path))
        else:
            failures = sim.FaultInjector(seed=a.seed, model=a.failures, rate=a.rate)
        link = sim.LinkModel(latency=a.latency, bandwidth=a.bandwidth, jitter=a.jitter)
        cluster = sim.InProcessCluster(a.world, link, failures, seed=a.seed, timeout=a.timeout, wall_timeout=a.wall_timeout)
        n = a.values

        def step(ctx, s):
            ctx.compute(a.compute)
            g = np.full(n, float(ctx.rank + 1 + s), dtype=np.float32)
            return float(ctx.all_reduce(g)[0])
        result = cluster.run(step, steps=a.steps)
        faults = cluster.log.of("fault")
        print(f"world {a.world}, {a.steps} steps, failure model {a.failures if a.action == 'sim' else 'replay'}: "
              f"{len(faults)} fault(s)")
        for f in faults:
            print(f"  {f['key']}")
        errors = getattr(result, "errors", {})
        for r, e in sorted(errors.items()):
            print(f"  rank {r}: {type(e).__name__}: {e}")
        clock = getattr(result, "virtual_seconds", None)
        if clock is not None:
            print(f"virtual time {clock:.6f} s")
        if a.log:
            cluster.log.save(a.log)
            print(f"event log written to {a.log}")
        return 0
    raise SystemExit(f"unknown action {a.action}")


def cmd_transports(a) -> int:
    """What carries bytes between ranks here, fastest first, and whether it is usable on this machine."""
    import torch
    import torch.distributed as dist
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    peer = n > 1 and all(torch.cuda.can_device_access_peer(0, j) for j in range(1, n))
    rows = [("nvlink peer memory (kernels load / store the peers' buffers)", peer, f"{n} GPU(s)" + ("" if peer else "; needs 2+ GPUs with peer access")),
            ("nvswitch multicast (multimem stores / reducing loads)", peer, "bound through symmetric memory when the driver offers it"),
            ("nccl", dist.is_nccl_available() and n > 0, "torch.distributed backend"),
            ("gloo (tcp / shared memory, host tensors)", dist.is_gloo_available(), "torch.distributed backend; the CPU tests run on it"),
            ("sim (in-process cluster with a virtual clock)", True, "idrak_b200.cluster.sim")]
    for name, ok, note in rows:
        print(f"{'yes' if ok else 'no ':3s}  {name:62s} {note}")
    return 0


# ------------------------------------------------------------------------------------------- config-side helpers
def cmd_env(a) -> int:
    from .. import config
    for s in config.TABLE:
        v = os.environ.get(s.name)
        if a.all or v is not None:
            print(f"{'export ' if a.export else ''}{s.name}={v if v is not None else s.default}")
    return 0


def cmd_completion(a) -> int:
    from .__main__ import build_parser
    sub = next(x for x in build_parser()._actions if isinstance(x, argparse._SubParsersAction))
    names = " ".join(sorted(sub.choices))
    if a.shell == "bash":
        print(f'_idrak() {{ COMPREPLY=( $(compgen -W "{names}" -- "${{COMP_WORDS[COMP_CWORD]}}") ); }}\ncomplete -F _idrak idrak')
    elif a.shell == "zsh":
        print(f"#compdef idrak\n_arguments '1: :({names})'")
    else:
        print(f"complete -c idrak -f -a '{names}'")
    return 0


def _aliases_path() -> str:
    return os.path.join(_home(), "aliases.json")


def read_aliases() -> dict:
    try:
        with open(_aliases_path(), "r", encoding="utf-8") as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


def cmd_alias(a) -> int:
    table = read_aliases()
    if a.name is None:
        for k, v in sorted(table.items()):
            print(f"{k} -> {v}")
        return 0
    if a.remove:
        if table.pop(a.name, None) is None:
            raise SystemExit(f"no alias named '{a.name}'")
    elif a.target is None:
        if a.name not in table:
            raise SystemExit(f"no alias named '{a.name}'")
        print(table[a.name])
        return 0
    else:
        table[a.name] = a.target
    os.makedirs(_home(), exist_ok=True)
    with open(_aliases_path(), "w", encoding="utf-8") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    return 0


def cmd_list(a) -> int:
    """Model folders under the models directory (anything holding a config.json, a .gguf or an .ikm)."""
    root = a.folder or os.path.join(_home(), "models")
    found = []
    for base, dirs, files in os.walk(root) if os.path.isdir(root) else []:
        hit = [f for f in files if f == "config.json" or f.endswith((".gguf", ".ikm"))]
        if hit:
            size = sum(os.path.getsize(os.path.join(base, f)) for f in files)
            found.append((os.path.relpath(base, root), size, hit[0]))
            dirs[:] = []
    for name, size, kind in sorted(found):
        print(f"{name:50s} {size / 2 ** 20:10.1f} MiB  {kind}")
    if not found:
        print(f"no models under {root}")
    return 0


def cmd_verify(a) -> int:
    """Read every tensor of a weights file or folder (headers, offsets, sizes) and print a SHA-256 per file."""
    from ..formats.safetensors import SafeTensorsReader
    paths = [a.path] if os.path.isfile(a.path) else sorted(os.path.join(a.path, f) for f in os.listdir(a.path)
                                                            if f.endswith((".safetensors", ".ikw", ".gguf", ".ikm")))
    if not paths:
        raise SystemExit(f"{a.path}: nothing to verify")
    bad = 0
    for p in paths:
        h = hashlib.sha256()
        with open(p, "rb") as f:
            for block in iter(lambda: f.read(1 << 22), b""):
                h.update(block)
        note = ""
        try:
            if p.endswith(".safetensors"):
                r = SafeTensorsReader(p)
                names = list(r.keys())
                for n in names:
                    r.get(n)
                note = f"{len(names)} tensors"
            elif p.endswith(".gguf"):
                from ..formats.gguf import GgufFile
                g = GgufFile(p)
                note = f"{len(g.tensors)} tensors"
            elif p.endswith(".ikm"):
                from ..formats import ikm
                note = f"{len(ikm.open_package(p).entries)} entries"
            elif p.endswith(".ikw"):
                from ..formats import ikw
                note = f"{len(ikw.read(p).tensors)} tensors"
        except Exception as e:                                      # a damaged file is the finding, not a crash
            note, bad = f"DAMAGED: {type(e).__name__}: {e}", bad + 1
        print(f"{h.hexdigest()}  {os.path.basename(p)}  {note}")
    return 1 if bad else 0


def cmd_bench_compare(a) -> int:
    """Compare two files of JSON lines (one result per line, keyed by `case` + `args` or by `metric`)."""
    def read(path):
        out = {}
        with open(path, "r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if not line.startswith("{"):
                    continue
                d = json.loads(line)
                key = d.get("case") or d.get("metric") or d.get("op") or "?"
                args = d.get("args") or d.get("config") or {}
                if isinstance(args, dict):
                    args = {k: v for k, v in args.items() if k not in ("warmup", "iters", "graph", "flush_l2")}
                out[f"{key} {json.dumps(args, sort_keys=True)}"] = d
        return out
    before, after = read(a.before), read(a.after)
    worse = 0
    for key in sorted(set(before) & set(after)):
        b, c = before[key], after[key]
        field = "ms" if "ms" in b and "ms" in c else "ms_per_step" if "ms_per_step" in b else "value"
        x, y = float(b[field]), float(c[field])
        lower_better = field != "value" or b.get("higher_is_better") is False
        change = (y / x - 1.0) * 100 if x else 0.0
        regress = change > a.threshold if lower_better else change < -a.threshold
        worse += regress
        print(f"{'WORSE ' if regress else '      '}{key[:90]:90s} {field} {x:.4g} -> {y:.4g} ({change:+.1f} %)")
    for key in sorted(set(before) ^ set(after)):
        print(f"only in {'before' if key in before else 'after'}: {key[:100]}")
    return 1 if worse else 0


def cmd_train_tokenizer(a) -> int:
    from ..data.sources import read_records
    from ..text.tokenizers_native import train_bpe

    def lines():
        for p in a.inputs:
            if p.endswith((".jsonl", ".json", ".csv", ".tsv", ".parquet")):
                for r in read_records(p):
                    t = r.get(a.field)
                    if isinstance(t, str):
                        yield t
            else:
                with open(p, "r", encoding="utf-8", errors="replace") as f:
                    yield from f
    os.makedirs(a.output, exist_ok=True)
    if getattr(a, "kind", "bpe") == "unigram":
        from ..text.sentencepiece_model import write_model
        from ..text.unigram_trainer import train_unigram
        specials = a.special if a.special != ["<|endoftext|>"] else ["<unk>", "<s>", "</s>"]
        tok = train_unigram(lines(), a.vocab, special_tokens=specials, byte_fallback=a.byte_fallback)
        write_model(tok.model, os.path.join(a.output, "tokenizer.model"))       # the SentencePiece form beside the json
    else:
        tok = train_bpe(lines(), a.vocab, special_tokens=a.special, min_frequency=a.min_frequency)
    tok.save(os.path.join(a.output, "tokenizer.json"))
    cfg = {}
    if tok.eos_token_ids:
        cfg["eos_token"] = tok.id_to_token[tok.eos_token_ids[0]]
    with open(os.path.join(a.output, "tokenizer_config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    print(f"vocabulary {tok.vocab_size} written to {a.output}")
    return 0


def register(add) -> None:
    p = add("train", cmd_train, "fit a network to a CSV table and write a run folder")
    p.add_argument("data")
    p.add_argument("--target", required=True)
    p.add_argument("--output", "-o", required=True)
    p.add_argument("--network", help="JSON description of the network (default: two hidden layers)")
    p.add_argument("--task", choices=["regression", "classification"], default="regression")
    p.add_argument("--hidden", type=int, default=32)
    p.add_argument("--epochs", type=int, default=50)
    p.add_argument("--batch", type=int, default=256)
    p.add_argument("--lr", type=float, default=1e-2)
    p.add_argument("--validation", type=float, default=0.1)
    p.add_argument("--seed", type=int, default=0)
    p = add("predict", cmd_predict, "run a trained run folder on values or a CSV table")
    p.add_argument("run")
    p.add_argument("values", nargs="*")
    p.add_argument("--data")
    p.add_argument("--has-target", action="store_true")
    p = add("runs", cmd_runs, "list run folders")
    p.add_argument("folder", nargs="?", default=".")
    p.add_argument("--json", action="store_true")
    p = add("cluster", cmd_cluster, "topology files, the in-process simulator, local rank launch and the dashboard: init / inspect / sim / replay / calibrate / start / ui")
    p.add_argument("action", choices=["init", "inspect", "sim", "replay", "calibrate", "start", "ui"])
    p.add_argument("path", nargs="?")
    p.add_argument("program", nargs="*", help="start: the program every rank runs (after --)")
    p.add_argument("--node", help="start: which node of the topology this machine is (default: the first)")
    p.add_argument("--master-port", type=int, default=29500)
    p.add_argument("--dry-run", action="store_true", help="start: print what would run")
    p.add_argument("--serve", type=int, nargs="?", const=0, default=None, metavar="PORT", help="ui: serve the page over HTTP")
    p.add_argument("--once", action="store_true", help="ui: print the table once")
    p.add_argument("--refresh", type=float, default=2.0)
    p.add_argument("--nodes", type=int, default=1)
    p.add_argument("--gpus", type=int, default=8)
    p.add_argument("--memory", default="180GiB")
    p.add_argument("--inter-node", default="tcp")
    p.add_argument("--link", default="tcp", help="calibrate: the link type the measurements belong to")
    p.add_argument("--bytes", type=int, default=0)
    p.add_argument("--world", type=int, default=4)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--failures", default="none")
    p.add_argument("--rate", type=float, default=0.2)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--latency", type=float, default=5e-6)
    p.add_argument("--bandwidth", type=float, default=50e9)
    p.add_argument("--jitter", type=float, default=0.0)
    p.add_argument("--compute", type=float, default=0.01)
    p.add_argument("--values", type=int, default=1 << 20)
    p.add_argument("--timeout", type=float, default=120.0)
    p.add_argument("--wall-timeout", type=float, default=20.0)
    p.add_argument("--log")
    add("transports", cmd_transports, "what carries bytes between ranks on this machine")
    p = add("env", cmd_env, "settings as environment lines")
    p.add_argument("--all", action="store_true")
    p.add_argument("--export", action="store_true")
    add("completion", cmd_completion, "print a shell completion script").add_argument("shell", choices=["bash", "zsh", "fish"])
    p = add("alias", cmd_alias, "short names for model paths")
    p.add_argument("name", nargs="?")
    p.add_argument("target", nargs="?")
    p.add_argument("--remove", action="store_true")
    add("list", cmd_list, "model folders under the models directory").add_argument("folder", nargs="?")
    add("verify", cmd_verify, "read every tensor of a weights file / folder and print checksums").add_argument("path")
    p = add("bench-compare", cmd_bench_compare, "compare two files of benchmark JSON lines")
    p.add_argument("before")
    p.add_argument("after")
    p.add_argument("--threshold", type=float, default=3.0, help="per cent change that counts as worse")
    p = add("train-tokenizer", cmd_train_tokenizer, "train a byte-level BPE tokenizer on text / record files")
    p.add_argument("inputs", nargs="+")
    p.add_argument("--output", "-o", required=True)
    p.add_argument("--vocab", type=int, default=8192)
    p.add_argument("--special", nargs="*", default=["<|endoftext|>"])
    p.add_argument("--min-frequency", type=int, default=2)
    p.add_argument("--kind", choices=["bpe", "unigram"], default="bpe")
    p.add_argument("--byte-fallback", action="store_true", help="unigram: add the 256 byte pieces")
    p.add_argument("--field", default="text")

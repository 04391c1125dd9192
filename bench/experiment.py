"""Experiment runner: template TOML -> instance runs -> client.jsonl + SLO summary, with resume.

The counterpart of the reference's batch job runner (scripts/batch/main.py:62-252, parser.py:24-114,
runner.py:124-790): a *template* lists models, datasets, feature sets and router options; every list-valued
`[router]` key fans out, the cartesian product over models x datasets x features x router options gives the
*instances*; each instance writes `config-server.json` (cluster layout), `config-router.json`,
`config-stubs.json`, starts workers (GPU workers under torch.distributed.run, or GPU-less stub workers),
the router and the trace client, waits, tears down, summarises (`summary.json`) and appends its path to
`checkpoint.txt` so `--checkpoint` skips finished instances.  `--dry-run` only writes the configs and the
command lines.  `<out>/provenance/` records the commit, the uncommitted diff and small untracked files of the
source tree the run used; the exit status is non-zero when an instance failed (see `<out>/error.log`).

    python bench/experiment.py --template bench/templates/cpu_plumbing.toml --out runs/ [--dry-run] [--force]
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import shlex
import shutil
import signal
import subprocess
import sys
import time
import tomllib
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def expand(template: dict) -> list:
    """Cartesian product over models, datasets, feature sets and list-valued router keys."""
    router = template.get("router", {})
    fan_keys = [k for k, v in router.items() if isinstance(v, list)]
    fan_vals = [router[k] for k in fan_keys]
    models = template.get("models", {"default": {}})
    datasets = template.get("datasets", {"default": {}})
    features = template.get("features", {}).get("sets", ["impl_blitz,impl_fast_pro,impl_live_pro"])
    out = []
    for (mname, m), (dname, d), feat in itertools.product(models.items(), datasets.items(), features):
        for combo in itertools.product(*fan_vals) if fan_vals else [()]:
            r = dict(router)
            r.update(dict(zip(fan_keys, combo)))
            tag = "-".join([mname, dname, feat.replace(",", "+")] + [f"{k}={v}" for k, v in zip(fan_keys, combo)])
            out.append({"tag": tag, "model": dict(m, name=mname), "dataset": dict(d, name=dname), "features": feat,
                        "router": r, "global": template.get("global", {}), "server": template.get("server", {}),
                        "envs": template.get("extra-envs", {})})
    return out


def cluster_json(inst: dict) -> dict:
    g = inst["global"]
    n, tp = int(g.get("num_gpus", 2)), int(inst["model"].get("tp", 1))
    states = list(g.get("init_states", ["Prefill", "Decode"] + ["Inactive"] * (n // tp - 2)))
    per_rank = [s for s in states for _ in range(tp)]
    return {"init_states": per_rank, "replicas": [list(range(r * tp, (r + 1) * tp)) for r in range(n // tp)],
            "machines": [0] * n}


def commands(inst: dict, d: Path) -> dict:
    g, m, r, ds = inst["global"], inst["model"], inst["router"], inst["dataset"]
    n, tp = int(g.get("num_gpus", 2)), int(m.get("tp", 1))
    base = int(g.get("worker_port", 50051))
    urls = [f"127.0.0.1:{base + i}" for i in range(n)]
    (d / "config-stubs.json").write_text(json.dumps(urls))
    py = sys.executable
    if g.get("stub_workers", False):
        workers = [f"{py} -m blitz_scale_b200.sim.stub_worker --rank {i} --world {n} --port {base + i} "
                   f"--config {d / 'config-server.json'} --seed {g.get('seed', 0)} --layers {m.get('layers', 2)}" for i in range(n)]
    else:
        workers = [f"{py} -m torch.distributed.run --nnodes=1 --nproc-per-node {n} --master-addr 127.0.0.1 "
                   f"--master-port {g.get('master_port', 29600)} -m blitz_scale_b200.worker.launcher --model-name {m['name']} "
                   f"--config {d / 'config-server.json'} --port {base} -TP {tp} "
                   f"--num-total-blocks {m.get('num_available_blocks', 4096)} --page-size {m.get('page_size', 64)} "
                   f"--log-dir {d / 'worker-logs'}"]
    router_args = {
        "--port": r.get("port", 3000), "--client-config": str(d / "config-stubs.json"),
        "--deployment-config-path": str(d / "config-server.json"), "--features": inst["features"],
        "--tensor-parallel-size": tp, "--model-name": m["name"],
        "--max-blocks-per-replica": m.get("num_available_blocks", 4096),
        "--tokens-prefilled-per-sec": m.get("tokens_prefilled_per_sec", 15000),
        "--tokens-transferred-per-sec": m.get("tokens_transferred_per_sec", 96000),
        "--block-size": m.get("page_size", 64),
    }
    for k in ("prefill-lower-bound", "prefill-upper-bound", "decode-lower-bound", "decode-upper-bound",
              "migration-lower-bound", "migration-upper-bound", "min-prefill-num", "max-prefill-num", "min-decode-num",
              "max-decode-num", "scale-down-threshold-millis", "mock-load-millis", "max-input-length", "max-total-tokens",
              "decode-steps-per-call", "max-incoming-migrations", "health-interval-ms", "health-misses", "rpc-timeout-ms",
              "quarantine-ms", "planner-horizon-ms", "otlp-endpoint", "max-batch-size"):
        kk = k.replace("-", "_")
        if kk in r:
            router_args["--" + k] = r[kk]
    (d / "config-router.json").write_text(json.dumps(router_args, indent=1))
    router = f"{py} -m blitz_scale_b200.router.server " + " ".join(f"{k} {shlex.quote(str(v))}" for k, v in router_args.items())
    client = (f"{py} -m blitz_scale_b200.sim.request_sim --endpoint http://127.0.0.1:{r.get('port', 3000)}/generate --protocol st "
              f"--replay-mode --scale-factor {ds.get('scale_factor', 1.0)} --output-path {d / 'client.jsonl'} "
              f"--vocab {m.get('vocab', 32000)} ")
    if ds.get("path"):
        client += f"--dataset-type csv --dataset-path {ds['path']} --time-in-secs {ds.get('time_in_secs', 60)}"
    else:
        client += (f"--dataset-type mock --rate {ds.get('rate', 4.0)} --cv {ds.get('cv', 1.0)} --duration {ds.get('duration', 50)} "
                   f"--num-requests {ds.get('num_requests', 200)} --seed {ds.get('seed', 0)}")
    return {"workers": workers, "router": router, "client": client}


def wait_for(path: Path, needle: str, count: int, timeout: float, also_glob: str = "", procs=()) -> bool:
    """Wait until `needle` occurs `count` times in `path` plus the files matching `also_glob` (workers started with
    --log-dir write one file per rank instead of their stdout).  Gives up at once when one of `procs` has exited:
    a worker that could not bind its port will never print the line."""
    t0 = time.time()
    while time.time() - t0 < timeout:
        files = [path] + (sorted(path.parent.glob(also_glob)) if also_glob else [])
        if sum(f.read_text(errors="ignore").count(needle) for f in files if f.exists()) >= count:
            return True
        if any(p.poll() is not None for p in procs):
            return False
        time.sleep(0.2)
    return False


def run_instance(inst: dict, d: Path, dry: bool) -> dict:
    d.mkdir(parents=True, exist_ok=True)
    (d / "config-server.json").write_text(json.dumps(cluster_json(inst)))
    cmds = commands(inst, d)
    (d / "commands.json").write_text(json.dumps(cmds, indent=1))
    if dry:
        return {"tag": inst["tag"], "dry_run": True}
    env = dict(os.environ, PYTHONPATH=str(ROOT), **{k: str(v) for k, v in inst["envs"].items()})
    procs, logs = [], []
    try:
        wl = open(d / "workers.log", "w")
        logs.append(wl)
        for c in cmds["workers"]:
            procs.append(subprocess.Popen(shlex.split(c), stdout=wl, stderr=subprocess.STDOUT, env=env, start_new_session=True))
        n = int(inst["global"].get("num_gpus", 2))
        if not wait_for(d / "workers.log", "Start gRPC server", n, float(inst["global"].get("boot_timeout", 600)),
                        also_glob="worker-logs/*.log", procs=procs):
            raise RuntimeError("workers did not start (see workers.log)")
        rl = open(d / "router.log", "w")
        logs.append(rl)
        procs.append(subprocess.Popen(shlex.split(cmds["router"]), stdout=rl, stderr=subprocess.STDOUT, env=env, start_new_session=True))
        if not wait_for(d / "router.log", "Router listening", 1, 60, procs=procs[-1:]):
            raise RuntimeError("router did not start")
        # scripted manual scaling: [[global.manual_scale]] at_s = 20, replica = 2, state = "Prefill"  (needs the
        # manually_scale feature; entries with the same at_s reach the router before its next step and therefore
        # share one parameter multicast)
        events = sorted(inst["global"].get("manual_scale", []), key=lambda e: float(e["at_s"]))
        if events:
            import threading
            import urllib.request
            url = f"http://127.0.0.1:{inst['router'].get('port', 3000)}/modify_cluster_state"
            t_begin = time.time()

            def fire():
                for e in events:
                    time.sleep(max(0.0, float(e["at_s"]) - (time.time() - t_begin)))
                    body = json.dumps({"replica": int(e["replica"]), "state": str(e["state"])}).encode()
                    try:
                        urllib.request.urlopen(urllib.request.Request(url, data=body, headers={"Content-Type": "application/json"}),
                                               timeout=10).read()
                    except Exception as ex:  # noqa: BLE001 - recorded, the run goes on
                        print(f"manual_scale {e} failed: {ex}", flush=True)
            threading.Thread(target=fire, daemon=True).start()
        cl = open(d / "client.log", "w")
        logs.append(cl)
        rc = subprocess.call(shlex.split(cmds["client"]), stdout=cl, stderr=subprocess.STDOUT, env=env,
                             timeout=float(inst["global"].get("client_timeout", 3600)))
        if rc != 0:
            raise RuntimeError(f"client exited with {rc}")
    finally:
        for p in reversed(procs):
            try:
                os.killpg(p.pid, signal.SIGTERM)   # the exact process groups started above
            except ProcessLookupError:
                pass
        for p in procs:
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
        for f in logs:
            f.close()
        if not inst["global"].get("stub_workers", False):
            wait_gpus_released(int(inst["global"].get("num_gpus", 2)))
    from blitz_scale_b200.utils import analysis
    recs = analysis.load_jsonl(str(d / "client.jsonl"))
    log = analysis.parse_router_log(open(d / "router.log", errors="ignore"))
    summary = {"tag": inst["tag"], "slo": analysis.slo_table(recs), "scale_out": analysis.scale_out_latencies(log["transitions"]),
               "transitions": len(log["transitions"])}
    (d / "summary.json").write_text(json.dumps(summary, indent=1))
    try:      # figures of the run (TTFT / TBT against the SLO lines, replica states, token rates)
        from blitz_scale_b200.utils import plots
        (d / "report.html").write_text(plots.report(open(d / "router.log", errors="ignore"), recs, inst["tag"]))
    except Exception as e:  # noqa: BLE001 - a figure must not fail a finished run
        print(f"report for {inst['tag']} not written: {e}", flush=True)
    return summary


def _terminate(signum, frame):
    raise KeyboardInterrupt      # run the `finally` blocks: the worker / router process groups must not outlive us


def wait_gpus_released(num_gpus: int, timeout: float = 60.0, query=None) -> bool:
    """After tearing a GPU instance down, wait until no compute process is left on the first `num_gpus` devices, so
    that the next instance finds its memory free (the reference's runner polls the same before it goes on,
    scripts/batch/runner.py:563-790).  Read-only NVML queries; `query(i)` -> number of compute processes on device
    i can be injected for tests.  True when the devices are free (or cannot be inspected)."""
    if query is None:
        try:
            import pynvml
            pynvml.nvmlInit()
        except Exception:  # noqa: BLE001 - no driver here: nothing to wait for
            return True

        def query(i):
            return len(pynvml.nvmlDeviceGetComputeRunningProcesses(pynvml.nvmlDeviceGetHandleByIndex(i)))
    t0 = time.time()
    while True:
        try:
            busy = [i for i in range(num_gpus) if query(i) > 0]
        except Exception:  # noqa: BLE001
            return True
        if not busy:
            return True
        if time.time() - t0 > timeout:
            print(f"GPUs {busy} still hold compute processes after {timeout:.0f} s", flush=True)
            return False
        time.sleep(0.5)


def record_provenance(dest: Path, max_file_bytes: int = 1 << 20) -> None:
    """What exactly ran: commit, branch and status, the uncommitted diff, and copies of small untracked files, so
    that a result directory can be traced back to its source (the reference's harness archives the same,
    scripts/batch/runner.py:60-121).  Best effort: outside a git checkout it only notes that."""
    dest.mkdir(parents=True, exist_ok=True)

    def git(*args):
        r = subprocess.run(["git", "-C", str(ROOT), *args], capture_output=True, text=True, timeout=60)
        if r.returncode != 0:
            raise RuntimeError(r.stderr.strip() or "git failed")
        return r.stdout
    try:
        info = "commit " + git("rev-parse", "HEAD").strip() + "\nbranch " + git("rev-parse", "--abbrev-ref", "HEAD").strip()
        info += "\n\n" + git("status", "--short")
        (dest / "git-info.txt").write_text(info)
        (dest / "git-diff.patch").write_text(git("diff", "HEAD"))
        for rel in git("ls-files", "--others", "--exclude-standard").splitlines():
            src = ROOT / rel
            if src.is_file() and src.stat().st_size <= max_file_bytes:
                tgt = dest / "untracked" / rel
                tgt.parent.mkdir(parents=True, exist_ok=True)
                shutil.copy2(src, tgt)
    except Exception as e:  # noqa: BLE001
        (dest / "git-info.txt").write_text(f"no source provenance: {e}\n")


def main():
    signal.signal(signal.SIGTERM, _terminate)
    ap = argparse.ArgumentParser()
    ap.add_argument("--template", "--templates", required=True)
    ap.add_argument("--out", default="runs")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--checkpoint", default="")
    a = ap.parse_args()
    tpl = tomllib.load(open(a.template, "rb"))
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    ck = Path(a.checkpoint) if a.checkpoint else out / "checkpoint.txt"
    if a.force and ck.exists():
        ck.unlink()
    done = set(ck.read_text().split()) if ck.exists() else set()
    if not a.dry_run:
        record_provenance(out / "provenance")
    results = []
    for inst in expand(tpl):
        d = out / inst["tag"]
        if str(d) in done:
            continue
        try:
            results.append(run_instance(inst, d, a.dry_run))
            if not a.dry_run:
                with open(ck, "a") as f:
                    f.write(str(d) + "\n")
        except Exception as e:  # noqa: BLE001
            with open(out / "error.log", "a") as f:
                f.write(f"{inst['tag']}: {e}\n")
            results.append({"tag": inst["tag"], "error": str(e)})
    print(json.dumps(results, indent=1))
    if any("error" in r for r in results):
        sys.exit(1)


if __name__ == "__main__":
    main()

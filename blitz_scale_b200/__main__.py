"""`python -m blitz_scale_b200 <command> [args...]`: one entry point for the programs of the framework.

    worker        GPU worker (one process per GPU; start under torch.distributed.run)   -> worker.launcher
    stub-worker   GPU-less worker for plumbing tests                                    -> sim.stub_worker
    router        router / autoscaler with the HTTP API                                 -> router.server
    client        trace-replay client (writes client.jsonl)                             -> sim.request_sim
    convert       Hugging Face safetensors -> weight-segment files                      -> models.convert
    repl          interactive gRPC client / load-latency / broadcast benchmark          -> utils.worker_client
    logs          log debuggers (merge, grep, zigzag, usage, migrations)                -> utils.logtools
    trace         trace-file tools (slice, scale, concat, stats, compare)               -> sim.trace_tools
    report        figures of a run (TTFT / TBT vs SLO, replica states, token rates) as HTML -> utils.plots
    chrome-trace  router log (+ client.jsonl) as a Chrome / Perfetto trace                  -> utils.tracing
    build         compile the kernel library and the native core                        -> build
    proto         print the gRPC contract as a .proto file                              -> pb.schema
"""
import importlib
import sys

COMMANDS = {
    "worker": "blitz_scale_b200.worker.launcher", "stub-worker": "blitz_scale_b200.sim.stub_worker",
    "router": "blitz_scale_b200.router.server", "client": "blitz_scale_b200.sim.request_sim",
    "convert": "blitz_scale_b200.models.convert", "repl": "blitz_scale_b200.utils.worker_client",
    "logs": "blitz_scale_b200.utils.logtools", "trace": "blitz_scale_b200.sim.trace_tools",
    "report": "blitz_scale_b200.utils.plots", "chrome-trace": "blitz_scale_b200.utils.tracing",
    "build": "blitz_scale_b200.build", "proto": "blitz_scale_b200.pb.schema",
}


def main() -> int:
    if len(sys.argv) < 2 or sys.argv[1] in ("-h", "--help") or sys.argv[1] not in COMMANDS:
        print(__doc__)
        return 0 if len(sys.argv) >= 2 and sys.argv[1] in ("-h", "--help") else 2
    mod = importlib.import_module(COMMANDS[sys.argv[1]])
    sys.argv = [f"blitz_scale_b200 {sys.argv[1]}"] + sys.argv[2:]
    try:
        rc = getattr(mod, "cli", mod.main)()      # `cli` where a module keeps a command-line wrapper around `main`
    except (FileNotFoundError, IsADirectoryError, PermissionError) as e:
        print(f"{sys.argv[0]}: {e}", file=sys.stderr)   # a path that cannot be read or written: one line is enough
        return 1
    return int(rc or 0)


if __name__ == "__main__":
    sys.exit(main())

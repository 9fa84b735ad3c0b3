"""Secondary benchmark workloads (fan-out, reshard, digest); see bench.py."""


def run(args):
    raise SystemExit(f"workload {args.workload!r} is not wired up yet")

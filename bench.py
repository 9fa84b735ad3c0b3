#!/usr/bin/env python
"""Benchmark of the weight-placement hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload place|moe|fanout|reshard|digest|vllm|convert]

Default workload (the headline): a Llama-3-8B-shaped bf16 synthetic checkpoint
(4 safetensors files, ~16 GB, seed 1) placed into tensor-parallel TP=8 shards.
One step = one GPU places one rank's shard (2,008,031,232 bytes); with N GPUs
rank r places TP rank r (weak scaling, no data-path collective).

  value, e2e   memory -> HBM through the public call (place_checkpoint): the
               checkpoint files are mapped and page-locked in host memory, the
               copy engine gathers the rank's slices over PCIe into device
               staging, the scatter kernel writes the shards, a status word
               comes back per step.
  file_to_hbm  the same bytes from the same files as ordinary pageable memory:
               gather threads -> pinned ring -> PCIe -> staging -> scatter; also
               the one-shot call as a fresh process pays for it.
  roofline     the scatter kernel alone (checkpoint image resident in HBM).
  parity       every placed tensor of every rank, each path, against the
               reference's CPU loop: both reference digests and memcmp.
  multi_gpu    with more than one GPU: fan-out and refit reshard over NVLink.

Rank 0 prints one JSON line.  ``--impl reference`` times the reference's
host-staged CPU load-and-shard (full ``get_tensor`` + ``narrow`` + ``copy_`` per
tensor) on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import threading
import time
import warnings

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TP = 8
FALLBACK_HBM_GBS = 6650.0


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while a timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        try:
            self.proc = subprocess.Popen(
                [exe, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def checkpoint_dir(cfg_name: str, layers: int) -> str:
    base = os.environ.get("MXB_BENCH_DIR")
    if not base:
        shm = "/dev/shm"
        ok = os.path.isdir(shm) and shutil.disk_usage(shm).free > (24 << 30)
        base = shm if ok else "/tmp"
    return os.path.join(base, f"mxb200_{cfg_name}_L{layers}")


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, copy read+write)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s; MEASURED_PEAKS.json was not found)"


# DRAM bytes moved per byte placed, from ncu captures (--set full) of the 4-layer case: read +
# written bytes of one resident-table launch divided by the 480,845,824 bytes it places.  Every
# byte is read once and written once, so the traffic of a larger launch is this ratio times its
# bytes placed.
NCU_DRAM_BYTES_PER_BYTE_PLACED = {
    "scatter_bulk_kernel": (480.93e6 + 430.71e6) / 480845824,
    "scatter_vec_kernel": (480.94e6 + 432.56e6) / 480845824,
}


def ncu_traffic(kernel: str, bytes_placed: int):
    ratio = NCU_DRAM_BYTES_PER_BYTE_PLACED.get(kernel)
    if ratio is None:
        return None
    return {"bytes_per_launch": int(ratio * bytes_placed),
            "how": "dram__bytes_read.sum + dram__bytes_write.sum of one launch in the ncu capture of "
                   "the 4-layer case, scaled by bytes placed (about 50 MB of written lines were still "
                   "in L2 when the captured kernel ended, hence slightly under 2.0 per byte)"}


def dist_setup(n_gpus: int):
    import torch

    rank = env_int("RANK", 0)
    world = env_int("WORLD_SIZE", 1)
    local = env_int("LOCAL_RANK", 0)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(local)
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def make_checkpoint(rank: int, world: int, layers: int, moe: bool = False):
    from dataclasses import replace

    from modelexpress_b200 import synth

    if moe:
        cfg = replace(synth.DEEPSEEK_V3_SLICE, layers=layers)
        tensors = synth.moe_tensors(cfg)
    else:
        cfg = synth.scaled(synth.LLAMA3_8B, layers=layers)
        tensors = synth.dense_tensors(cfg)
    d = checkpoint_dir(cfg.name, layers)
    if rank == 0:
        t0 = time.perf_counter()
        import torch

        synth.ensure_checkpoint(d, tensors, cfg.seed, cfg.files,
                                device="cuda" if torch.cuda.is_available() else "cpu")
        log(f"[bench] checkpoint at {d} ready in {time.perf_counter() - t0:.1f}s")
    barrier(world)
    return cfg, d


# ---------------------------------------------------------------------------
# ours: placement
# ---------------------------------------------------------------------------

WORKLOAD_DENSE = ("configs[1]: Llama-3-8B-shaped bf16 checkpoint (seed 1, 4 safetensors files), "
                  "one TP=8 rank shard per GPU per step")
WORKLOAD_MOE = ("configs[4]: DeepSeek-V3-style FP8 MoE slice (256 routed + 1 shared expert per layer, seed 3), "
                "experts expert-parallel 32 per GPU, attention TP=8, scales co-placed; one rank per GPU per step")
METRIC_DENSE = "GB/s placed into HBM (Llama-3-8B bf16, TP=8 shards)"
METRIC_MOE = "GB/s placed into HBM (DeepSeek-V3-style FP8 slice, EP=8/TP=8)"


def _digests(ctx, params, names):
    """(safe_checksum string, tensor_digest scalar list) per parameter: the reference's two
    digests (tensor_utils.py:27-44, refit/reshard/verify.py:113-150) from one kernel launch."""
    from modelexpress_b200.digest import scalars_from_record
    from modelexpress_b200.runtime import DIGEST_ROWS, DIGEST_SAFE32

    spans = [(params[n].data_ptr(), params[n].numel() * params[n].element_size()) for n in names]
    recs = ctx.digest(spans, DIGEST_SAFE32 | DIGEST_ROWS)
    return [(format(int(r.safe_checksum) & 0xFFFFFFFF, "08x"), scalars_from_record(r)) for r in recs]


def oracle_digests(ckpt: str, tp_rank: int, names, moe: bool):
    """The same tuples from the CPU: the reference's host-staged loop for this rank
    (oracle port), digested by the oracle's C restatement.  Returns (digests, host params)."""
    import numpy as np
    import torch

    from oracle import c_port, cpu_loader, ref_port  # the checker; never on the product path

    if moe:
        tensors = {}
        for fn in sorted(f for f in os.listdir(ckpt) if f.endswith(".safetensors")):
            path = os.path.join(ckpt, fn)
            raw = np.memmap(path, dtype=np.uint8, mode="r")
            for n, info in ref_port.parse_safetensors_header(path).items():
                dt = {"F8_E4M3": np.uint8, "F32": np.float32, "BF16": np.uint16}[info["dtype"]]
                tensors[n] = raw[info["file_offset"]: info["file_offset"] + info["size"]].view(dt).reshape(info["shape"])
        host = {n: np.ascontiguousarray(a) for n, a in ref_port.load_and_shard_moe(tensors, tp_rank, TP).items()}
        as_bytes = {n: a.view(np.uint8).reshape(-1) for n, a in host.items()}
    else:
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(1, env_int("LOCAL_WORLD_SIZE", 1))))
        host, _placed, _s = cpu_loader.load_and_shard_torch(ckpt, tp_rank, TP)
        as_bytes = {n: t.contiguous().view(torch.uint8).reshape(-1).numpy() for n, t in host.items()}
    out = []
    for n in names:
        a = as_bytes[n]
        out.append((c_port.safe_checksum(a, mt=True), c_port.digest_scalars(a, mt=True)))
    return out, as_bytes


def bench_place(args):
    import numpy as np
    import torch

    from modelexpress_b200 import loader
    from modelexpress_b200.runtime import (PLACE_COPY_ENGINE, PLACE_ZERO_COPY, SCATTER_VECTOR,
                                           SCATTER_DEFAULT, Context)

    rank, world, local = dist_setup(args.gpus)
    moe = args.workload == "moe"
    layers = env_int("MXB_BENCH_LAYERS", 4 if moe else 32)
    cfg, ckpt = make_checkpoint(rank, world, layers, moe)
    tp_rank = rank % TP
    dev = f"cuda:{local}"
    ctx = Context([local])
    prep = loader.Prepared.build(ckpt, tp_rank, TP, "auto")
    idx, plan = prep.index, prep.plan
    params = loader.allocate_params(plan, dev)
    names = list(plan.params)
    torch.cuda.synchronize()
    bytes_placed = plan.bytes_placed
    total_bytes = bytes_placed * world  # every rank places one shard of equal size
    local_world = max(1, env_int("LOCAL_WORLD_SIZE", world))
    # gather threads for pageable sources: three quarters of the cores, shared by the ranks of the box
    threads = env_int("MXB_HOST_THREADS", max(2, min(32, (os.cpu_count() or 8) * 3 // 4 // local_world)))
    slots = env_int("MXB_RING_SLOTS", 4)
    mode = PLACE_ZERO_COPY if os.environ.get("MXB_PLACE_MODE", "ce") == "zc" else PLACE_COPY_ENGINE
    ring_bytes = env_int("MXB_RING_BYTES", 128 << 20)
    ring = ctx.ring(ring_bytes, slots, local)
    skip_e2e = os.environ.get("MXB_BENCH_SKIP_E2E") == "1"  # profiling runs that only want the table launches

    def zero_params():
        for v in params.values():
            v.zero_()
        torch.cuda.synchronize()

    def timed(fn, steps, everyone=True):
        """Wall time of ``steps`` calls bracketed by barrier + synchronize; max over ranks."""
        if everyone:
            barrier(world)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = [fn() for _ in range(steps)]
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if everyone:
            barrier(world)
            dt = max_over_ranks(dt, world)
        return dt, out

    # ---- memory -> HBM: this rank's bytes are kept page-locked in host memory, packed as they
    # cross PCIe (made by the first load).  Every step is the public call: one contiguous
    # copy-engine transfer per chunk into device staging, the scatter kernel writes the shards --
    images = loader.HostImages()

    def load_pinned():
        return loader.place_checkpoint(ckpt, tp_rank, TP, dev, params=params, ring=ring, ctx=ctx,
                                       host_threads=threads, mode=mode, pin="keep", images=images)

    sampler = ClockSampler(local)
    mem = {}
    if not skip_e2e:
        first_s, first = timed(load_pinned, 1)      # gathers into the page-locked image that is kept
        pinned_bytes = images.packed_bytes
        for _ in range(args.warmup):
            load_pinned()
        launches0 = ctx.launch_count
        sampler.start()
        mem_s, mem_stats = timed(load_pinned, args.steps)
        mem_launches = ctx.launch_count - launches0
        if any(p.stats.bytes_direct != bytes_placed or p.stats.seconds_gather for p in mem_stats):
            raise SystemExit("bench: a load from the kept image went through the gather threads")
        d_mem = _digests(ctx, params, names)
        single_s = None
        if world > 1:   # the same load with the other ranks idle: what one GPU gets from the box alone
            barrier(world)
            if rank == 0:
                single_s, _ = timed(load_pinned, min(3, args.steps), everyone=False)
                single_s /= min(3, args.steps)
            barrier(world)
            single_s = max_over_ranks(single_s or 0.0, world)
        mem = {"first_s": first_s, "first_timings": first[0].timings, "pinned_bytes": pinned_bytes,
               "s": mem_s, "stats": mem_stats, "launches": mem_launches, "single_s": single_s}

    # ---- for comparison, one GPU only (pinning 6 GB of page cache per rank takes seconds): the
    # files' own pages page-locked and read in place by the copy engine (2-D gathers) -----------
    pages = None
    if not skip_e2e and (world == 1 or os.environ.get("MXB_BENCH_PAGES") == "1") and \
            os.environ.get("MXB_BENCH_PAGES") != "0":
        zero_params()
        pg_images = loader.HostImages()

        def load_pages():
            return loader.place_checkpoint(ckpt, tp_rank, TP, dev, params=params, ring=ring, ctx=ctx,
                                           host_threads=threads, mode=mode, pin="pages", images=pg_images)

        pg_first_s, pg_first = timed(load_pages, 1)
        load_pages()
        pg_s, pg_stats = timed(load_pages, min(5, args.steps))
        if _digests(ctx, params, names) != d_mem:
            raise SystemExit("bench: the page-locked file path placed different bytes")
        pages = {"value": round(total_bytes * min(5, args.steps) / pg_s / 1e9, 2), "unit": "GB/s",
                 "first_load_s": round(pg_first_s, 4), "pin_s": pg_first[0].timings["pin"],
                 "pinned_bytes_per_rank": int(pg_images.pinned_bytes),
                 "mapping": "+".join(sorted({"shared" if pg_images.open(p).shared else "private"
                                             for p in prep.files})),
                 "what": "place_checkpoint(pin='pages'): the checkpoint files' own page-cache pages are "
                         "page-locked (whole row-parallel tensors, since a rank's slice touches every "
                         "page of them) and the copy engine gathers the slices from there"}
        pg_images.close()

    # ---- file -> HBM: the same files as ordinary pageable memory (page cache / tmpfs): gather
    # threads copy the rank's bytes into the pinned ring, their own streams carry them over PCIe -
    fil = {}
    if not skip_e2e:
        zero_params()
        plain = {p: loader.FileImage(p) for p in prep.files}
        items = prep.items({p: im.address for p, im in plain.items()}, params)
        for _ in range(max(1, args.warmup)):
            ring.place(items, threads, mode)
        file_s, file_stats = timed(lambda: ring.place(items, threads, mode), args.steps)
        if any(s.bytes_direct for s in file_stats):
            raise SystemExit("bench: the pageable mapping was treated as pinned")
        d_file = _digests(ctx, params, names)
        # one load as a fresh process pays for it: the public one-shot call maps the files,
        # pins its own ring, places, and leaves the teardown to a background thread
        one_shot = []
        for _ in range(2):
            zero_params()
            s, res = timed(lambda: loader.place_checkpoint(ckpt, tp_rank, TP, dev, params=params, ctx=ctx,
                                                           host_threads=threads, mode=mode), 1)
            one_shot.append({"s": round(s, 4), "timings": res[0].timings})
            time.sleep(0.3)  # that call's ring and mappings are released in the background
        fil = {"s": file_s, "stats": file_stats, "one_shot": one_shot}
        for im in plain.values():
            im.close()

    # the binding roofline of host -> HBM: pinned -> device copies, all ranks at once
    pin = torch.empty(1 << 30, dtype=torch.uint8).pin_memory()
    dev_buf = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    dev_buf.copy_(pin, non_blocking=True)
    torch.cuda.synchronize()
    barrier(world)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(3):
        dev_buf.copy_(pin, non_blocking=True)
    ev1.record()
    torch.cuda.synchronize()
    copy_ms = ev0.elapsed_time(ev1)
    pcie_gbs = sum_over_ranks(3 * (1 << 30) / (copy_ms * 1e-3) / 1e9, world)
    # the same copies on the basis `value` is measured on: all bytes over the slowest rank's time
    # (ranks whose links get a smaller share finish later; the sum of rates does not show that)
    pcie_all_done_gbs = world * 3 * (1 << 30) / (max_over_ranks(copy_ms, world) * 1e-3) / 1e9
    pcie_single = None
    if world > 1:
        barrier(world)
        if rank == 0:
            ev0.record()
            for _ in range(3):
                dev_buf.copy_(pin, non_blocking=True)
            ev1.record()
            torch.cuda.synchronize()
            pcie_single = 3 * (1 << 30) / (ev0.elapsed_time(ev1) * 1e-3) / 1e9
        barrier(world)
        pcie_single = max_over_ranks(pcie_single or 0.0, world)
    del pin, dev_buf

    # ---- the scatter kernel alone: checkpoint image resident in HBM, one launch per step -------
    file_dev, file_base = {}, {}
    for p in prep.files:
        im = images.open(p) if not skip_e2e else loader.FileImage(p)
        # place the image so that the safetensors data section (which starts 8 + header
        # bytes into the file, only 8-byte aligned) begins on a 256-byte boundary
        first_off = min(i["file_offset"] for i in idx.values() if i["file"] == p)
        lead = (-first_off) % 256 + (8 if os.environ.get("MXB_BENCH_MISALIGN") == "1" else 0)
        t = torch.empty(im.size + lead, dtype=torch.uint8, device=dev)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t[lead:].copy_(torch.from_numpy(np.frombuffer(im._mm, dtype=np.uint8)))
        file_dev[p], file_base[p] = t, t.data_ptr() + lead
        if skip_e2e:
            im.close()
    torch.cuda.synchronize()
    dev_items = prep.items(file_base, params)
    zero_params()
    table = ctx.table(dev_items, local)
    flags = SCATTER_VECTOR if os.environ.get("MXB_SCATTER", "auto") == "vec" else SCATTER_DEFAULT
    for _ in range(max(3, args.warmup)):
        table.launch(flags)
    ctx.sync(local)
    launches1 = ctx.launch_count
    barrier(world)
    torch.cuda.synchronize()
    ctx.event_record(0, local)
    for _ in range(args.steps):
        table.launch(flags)
    ctx.event_record(1, local)
    kern_ms = ctx.event_elapsed_ms(0, 1, local)
    ctx.sync(local)
    barrier(world)
    clocks = sampler.stop() if not skip_e2e else {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    kern_ms = max_over_ranks(kern_ms, world) / args.steps
    kern_launches = ctx.launch_count - launches1
    d_res = _digests(ctx, params, names)
    del file_dev

    # ---- parity at full size: every placed tensor of every rank, each of the three paths, against
    # the reference's CPU loop for the same rank: both reference digests, then memcmp -------------
    parity = None
    if os.environ.get("MXB_BENCH_SKIP_PARITY") != "1":
        want, host = oracle_digests(ckpt, tp_rank, names, moe)
        bad = []
        paths = {"kernel_resident": d_res}
        if not skip_e2e:
            paths.update({"memory_to_hbm": d_mem, "file_to_hbm": d_file})
        for label, got in paths.items():
            bad += [f"{label}:{n}" for n, g, w in zip(names, got, want) if g != w]
        for n in names:   # params hold the resident path's result, digest-equal to the other two
            got = params[n].detach().contiguous().view(torch.uint8).reshape(-1).cpu().numpy()
            if got.shape != host[n].shape or not np.array_equal(got, host[n]):
                bad.append(f"memcmp:{n}")
        nbad = int(sum_over_ranks(float(len(bad)), world))
        if bad:
            log(f"[bench] rank {rank}: parity FAILED for {bad[:8]}")
        if nbad:
            raise SystemExit(f"bench: {nbad} placed tensors differ from the CPU reference loop")
        parity = {"ok": True, "ranks": world, "tensors_per_rank": len(names), "paths": sorted(paths),
                  "checks": "safe_checksum + tensor_digest scalars of every placed tensor per path, then "
                            "memcmp of every tensor, against the reference's CPU loop (oracle port) for "
                            "the same rank"}
        del host

    peak, peak_src = measured_peak()
    achieved = 2.0 * bytes_placed / (kern_ms * 1e-3) / 1e9  # read + write per GPU
    kernel = "scatter_vec_kernel" if table.engine(flags) == "vector" else "scatter_bulk_kernel"
    table.close()

    def gbs(seconds, steps=args.steps):
        return total_bytes * steps / seconds / 1e9

    out = {
        "metric": METRIC_MOE if moe else METRIC_DENSE,
        "value": None, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {
            "workload": WORKLOAD_MOE if moe else WORKLOAD_DENSE,
            "layers": layers, "bytes_placed_per_gpu_per_step": bytes_placed,
            "tensors": len(idx), "records_per_step": len(plan.placements),
            "source_for_value": "this rank's checkpoint bytes kept page-locked in host memory, packed as they "
                                "cross PCIe (made by the first load, whose cost is config.pinning); every "
                                "step is one place_checkpoint(pin='keep') call: copy engine -> device "
                                "staging -> scatter kernel",
            "l2": "inputs larger than L2 (every step reads and writes bytes_placed, far above 126 MB)",
            "ring": {"bytes": ring_bytes, "slots": slots, "host_threads": threads,
                     "mode": "zero_copy" if mode == PLACE_ZERO_COPY else "copy_engine"},
        },
        "clocks": clocks,
    }
    pcie = {"bound": "pcie_h2d", "peak": round(pcie_gbs, 1), "unit": "GB/s",
            "how": "pinned->device cudaMemcpyAsync of 1 GiB x3 on every rank at once, summed over ranks, "
                   "measured in this run"}
    if not skip_e2e:
        value = gbs(mem["s"])
        out["value"] = round(value, 2)
        out["ms_per_step"] = round(mem["s"] / args.steps * 1e3, 4)
        out["config"]["seconds_to_loaded"] = round(mem["s"] / args.steps, 4)
        out["config"]["pinning"] = {
            "first_load_s": round(mem["first_s"], 4), "first_load_timings": mem["first_timings"],
            "pinned_bytes_per_rank": int(mem["pinned_bytes"]),
            "what": "first place_checkpoint(pin='keep') of the process: allocates the page-locked image, "
                    "gathers this rank's bytes into it through the gather threads and places them from "
                    "there; max over ranks"}
        out["e2e"] = {"value": round(value, 2), "unit": "GB/s",
                      "h2d_bytes_per_step": int(bytes_placed), "d2h_bytes_per_step": 4,
                      "source": "memory -> HBM: page-locked packed image of the rank's bytes, public "
                                "place_checkpoint() per step",
                      "device_s_per_step": round(sum(p.stats.seconds_device for p in mem["stats"]) / args.steps, 4),
                      "host_copy_bytes_per_step": 0,
                      "chunks_per_step": int(mem["stats"][0].stats.chunks),
                      "binding_roofline": dict(pcie, frac=round(value / pcie_gbs, 4),
                                               peak_until_the_slowest_rank_is_done=round(pcie_all_done_gbs, 1),
                                               frac_until_the_slowest_rank_is_done=round(value / pcie_all_done_gbs, 4))}
        if world > 1 and mem["single_s"]:
            single = bytes_placed / mem["single_s"] / 1e9
            out["e2e"]["one_rank_alone_gbs"] = round(single, 2)
            out["e2e"]["efficiency_vs_one_rank_alone"] = round(value / world / single, 4)
            out["e2e"]["binding_roofline"]["one_rank_alone_peak"] = round(pcie_single, 1)
        fvalue = gbs(fil["s"])
        out["file_to_hbm"] = {
            "value": round(fvalue, 2), "unit": "GB/s", "ms_per_step": round(fil["s"] / args.steps * 1e3, 4),
            "source": "file -> HBM: the same files as pageable memory (tmpfs / page cache mapping): gather "
                      "threads -> pinned ring sub-slots -> PCIe on their own streams -> staging -> scatter",
            "host_threads": threads,
            "host_gather_s_per_step": round(sum(s.seconds_gather for s in fil["stats"]) / args.steps, 4),
            "device_s_per_step": round(sum(s.seconds_device for s in fil["stats"]) / args.steps, 4),
            "chunks_per_step": int(fil["stats"][0].chunks),
            "frac_of_pcie": round(fvalue / pcie_gbs, 4),
            "bound": "host memory: every byte is read and written by a core and read again by the DMA; "
                     "pinning the pages instead costs more than one load (config.pinning)",
            "seconds_to_loaded_one_shot": fil["one_shot"]}
        if pages is not None:
            out["pinned_file_pages"] = pages
        out["gpu_launches"] = int(mem["launches"])
    else:
        out["value"] = round(total_bytes / (kern_ms * 1e-3) / 1e9, 2)
        out["ms_per_step"] = round(kern_ms, 4)
        out["profiling_only"] = ("host->HBM regions skipped (MXB_BENCH_SKIP_E2E=1): value is the resident-table "
                                 "kernel rate, not a measurement of the path")
        out["gpu_launches"] = int(kern_launches)
    out["gpu_launches_kernel_region"] = int(kern_launches)
    out["roofline"] = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                       "frac": round(achieved / peak, 4), "traffic": ncu_traffic(kernel, bytes_placed),
                       "kernel": kernel, "kernel_ms": round(kern_ms, 4), "peak_source": peak_src,
                       "algorithmic_bytes_per_launch": int(2 * bytes_placed),
                       "how": "the scatter kernel timed alone with CUDA events on its stream: checkpoint image "
                              "resident in HBM, one persistent launch per step over the same records; in the "
                              "host->HBM steps the same kernel runs once per staging chunk, hidden behind PCIe"}
    if parity is not None:
        out["parity"] = parity
    if world == 1 and rank == 0 and os.environ.get("MXB_BENCH_SKIP_CPU") != "1" and not moe:
        out["cpu_baseline"] = cpu_baseline(ckpt, tp_rank)
    ring.close()
    images.close()
    if world > 1 and not moe and os.environ.get("MXB_BENCH_SKIP_MULTI") != "1":
        import bench_workloads

        del params
        torch.cuda.empty_cache()
        out["multi_gpu"] = bench_workloads.multi_gpu_section(args, ctx, rank, world, local)
    if rank == 0:
        print(json.dumps(out), flush=True)
    ctx.close()
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def cpu_baseline(ckpt: str, tp_rank: int) -> dict:
    """The oracle's port of the reference's host-staged loop on ONE host core, a
    bounded sample (its results were checked against the GPU's in ``parity``)."""
    import torch

    from oracle import cpu_loader  # the one place bench.py may run oracle/

    torch.set_num_threads(1)
    params, placed, _sec = cpu_loader.load_and_shard_torch(ckpt, tp_rank, TP)  # warm page cache
    n, tot_b, tot_s = 0, 0, 0.0
    while tot_s < 12.0 and n < 6:
        _p, b, s = cpu_loader.load_and_shard_torch(ckpt, tp_rank, TP, params)
        n, tot_b, tot_s = n + 1, tot_b + b, tot_s + s
    return {"value": round(tot_b / tot_s / 1e9, 3), "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": f"{n} pass(es) over one TP=8 rank shard ({placed} B placed per pass; get_tensor maps "
                      "the file, narrow + copy_ touch only the bytes the rank keeps), page cache warm"}


# ---------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------

_REF_WORKER = r"""
import sys, time, os
sys.path.insert(0, sys.argv[1])
import torch
from oracle import cpu_loader
ckpt, tp_rank, threads, warm, steps = sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]), int(sys.argv[6])
torch.set_num_threads(threads)
params, placed, _ = cpu_loader.load_and_shard_torch(ckpt, tp_rank, 8)
for _ in range(warm):
    cpu_loader.load_and_shard_torch(ckpt, tp_rank, 8, params)
print("ready", flush=True)
sys.stdin.readline()
t0 = time.perf_counter()
for _ in range(steps):
    cpu_loader.load_and_shard_torch(ckpt, tp_rank, 8, params)
print("done", placed, time.perf_counter() - t0, flush=True)
"""


def bench_reference(args):
    """The reference's CPU host-staged load-and-shard on the box's host cores: one
    worker process per rank of the compared run, the cores split between them,
    every worker placing one TP=8 rank shard per step into host tensors."""
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    import torch

    from modelexpress_b200 import synth

    layers = env_int("MXB_BENCH_LAYERS", 32)
    cfg = synth.scaled(synth.LLAMA3_8B, layers=layers)
    d = checkpoint_dir(cfg.name, layers)
    synth.ensure_checkpoint(d, synth.dense_tensors(cfg), cfg.seed, cfg.files,
                            device="cuda" if torch.cuda.is_available() else "cpu")
    n = max(1, args.gpus)
    cores = os.cpu_count() or 1
    per = max(1, cores // n)
    workers = [subprocess.Popen([sys.executable, "-c", _REF_WORKER, ROOT, d, str(r % TP), str(per),
                                 str(max(0, args.warmup - 1)), str(args.steps)],
                                stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True) for r in range(n)]
    for w in workers:
        if w.stdout.readline().strip() != "ready":
            raise SystemExit("reference arm: a worker failed to start")
    t0 = time.perf_counter()
    for w in workers:
        w.stdin.write("go\n")
        w.stdin.flush()
    placed, slowest = 0, 0.0
    for w in workers:
        f = w.stdout.readline().split()
        placed += int(f[1])
        slowest = max(slowest, float(f[2]))
        w.wait()
    wall = time.perf_counter() - t0
    v = placed * args.steps / slowest / 1e9
    base = {"value": round(v, 3), "unit": "GB/s", "cores": per * n, "kind": "port",
            "sample": f"{n} worker process(es) x {per} torch threads, one TP=8 rank shard per worker per step "
                      f"({placed // n} B placed each), page cache warm; slowest worker {slowest:.3f} s, "
                      f"wall {wall:.3f} s"}
    out = {
        "impl": "reference",
        "metric": METRIC_DENSE,
        "value": round(v, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(slowest / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic",
        "config": {"workload": WORKLOAD_DENSE, "layers": layers,
                   "bytes_placed_per_gpu_per_step": placed // n,
                   "arm": "the reference's host-staged CPU loop (get_tensor + narrow + copy_) into host "
                          "tensors: no PCIe copy, so an upper bound on what it can feed a GPU"},
        "cpu_baseline": base,
        "e2e": {"value": round(v, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="place", choices=["place", "moe", "fanout", "reshard", "digest", "vllm", "convert"])
    args = ap.parse_args()
    if args.impl == "reference":
        return bench_reference(args)
    if args.workload in ("place", "moe"):
        return bench_place(args)
    import bench_workloads

    return bench_workloads.run(args)


if __name__ == "__main__":
    main()

"""Secondary benchmark workloads, run through ``bench.py --workload ...``.

digest   integrity digests of a Llama-3-8B-sized byte image resident in HBM
fanout   serving-peer fan-out of the 8B weights from GPU 0 to the other GPUs
reshard  FSDP-8 -> TP-8 refit reshard of a Qwen2.5-32B-shaped model
vllm     a whole Llama-3-8B-shaped model loaded through vLLM's model-loader seam
         (needs vLLM; one GPU), next to vLLM's own default loader on the same files

Each prints one JSON line on rank 0 in the same shape as the headline bench.
Multi-GPU workloads run one process per GPU (torchrun); peers' memory is mapped
with CUDA IPC and the data path uses no collective library.
"""

from __future__ import annotations

import json
import os
import sys
import time

import numpy as np


def _env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def _dist():
    import torch

    rank, world, local = _env_int("RANK", 0), _env_int("WORLD_SIZE", 1), _env_int("LOCAL_RANK", 0)
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def _barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def _gather_objects(obj, world):
    if world == 1:
        return [obj]
    import torch.distributed as dist

    out = [None] * world
    dist.all_gather_object(out, obj)
    return out


def _max(x, world):
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _peaks():
    root = os.path.dirname(os.path.abspath(__file__))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s)"


NVLINK_NOMINAL_GBS = 900.0  # NVLink 5, per direction per GPU


class _Holder:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


def as_tensor(ptr: int, nbytes: int, device: int):
    """uint8 tensor over a raw device range (to fill and inspect library-owned arenas)."""
    import torch

    return torch.as_tensor(_Holder(int(ptr), int(nbytes)), device=f"cuda:{device}")


def nvlink_peaks(ctx, rank, world, local, nbytes=1 << 30, reps=3) -> dict:
    """What the links give a plain copy in this run, per direction: a 16-byte
    store kernel and the copy engine, one pair alone and every GPU sending to its
    neighbour at once."""
    import torch

    base = ctx.alloc(2 * nbytes, local)
    peers = _open_peers(ctx, base, world)
    mine = as_tensor(base, 2 * nbytes, local)
    mine.zero_()
    torch.cuda.synchronize()
    nxt = (rank + 1) % world
    out = {}
    # one pair alone: rank 0 stores into rank 1
    _barrier(world)
    ms = ctx.copy_probe(base, peers[1] + nbytes, nbytes, reps, local) if rank == 0 else 0.0
    _barrier(world)
    out["store_kernel_one_pair_gbs"] = round(nbytes / (_max(ms, world) * 1e-3) / 1e9, 1)
    # every GPU stores into its neighbour at once (each link direction carries one stream)
    _barrier(world)
    ms = ctx.copy_probe(base, peers[nxt] + nbytes, nbytes, reps, local)
    _barrier(world)
    out["store_kernel_all_pairs_gbs"] = round(nbytes / (_max(ms, world) * 1e-3) / 1e9, 1)
    # the same with 32-byte stores
    os.environ["MXB_PROBE_WIDTH"] = "32"
    try:
        _barrier(world)
        ms = ctx.copy_probe(base, peers[nxt] + nbytes, nbytes, reps, local)
        _barrier(world)
    finally:
        os.environ.pop("MXB_PROBE_WIDTH", None)
    out["store_kernel_32B_all_pairs_gbs"] = round(nbytes / (_max(ms, world) * 1e-3) / 1e9, 1)
    # the copy engine over the same mapping
    dst = as_tensor(peers[nxt] + nbytes, nbytes, local)
    src = mine[:nbytes]
    dst.copy_(src)
    torch.cuda.synchronize()
    _barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        dst.copy_(src)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    _barrier(world)
    out["copy_engine_all_pairs_gbs"] = round(nbytes / (_max(ms, world) * 1e-3) / 1e9, 1)
    # local HBM copy with the same kernel, for scale
    ms = ctx.copy_probe(base, base + nbytes, nbytes, reps, local)
    out["store_kernel_local_hbm_gbs_read_plus_write"] = round(2 * nbytes / (_max(ms, world) * 1e-3) / 1e9, 1)
    out["how"] = (f"{nbytes >> 20} MiB, {reps} launches each, CUDA events, slowest rank; store kernel = the "
                  "library's plain 16-byte copy kernel writing into the peer's memory; copy engine = "
                  "cudaMemcpyAsync to the peer mapping")
    out["peak_gbs"] = max(out["store_kernel_one_pair_gbs"], out["store_kernel_all_pairs_gbs"],
                          out["store_kernel_32B_all_pairs_gbs"], out["copy_engine_all_pairs_gbs"])
    del dst, src, mine
    _barrier(world)
    ctx.free(base, local)
    return out


def _base(metric, value, unit, world, args, ms_per_step, config, dtype="u8", scaling="weak"):
    return {"metric": metric, "value": round(value, 6 if unit == "s" else 2), "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": dtype,
            "data": "synthetic", "config": config}


def _open_peers(ctx, local_ptr, world):
    """Exchange CUDA IPC handles of one device allocation per rank; returns the
    address of every rank's allocation as mapped into this process."""
    from modelexpress_b200.runtime import ipc_export, ipc_open

    rank = _env_int("RANK", 0)
    handle, off = ipc_export(local_ptr)
    allh = _gather_objects((handle, off), world)
    ptrs = []
    for r, (h, o) in enumerate(allh):
        ptrs.append(local_ptr if r == rank else ipc_open(h, o))
    return ptrs


# ---------------------------------------------------------------------------
# digest
# ---------------------------------------------------------------------------


def run_digest(args):
    import torch

    from modelexpress_b200 import synth
    from modelexpress_b200.runtime import DIGEST_BLOCK64, DIGEST_ROWS, DIGEST_SAFE32, Context

    rank, world, local = _dist()
    ctx = Context([local])
    cfg = synth.scaled(synth.LLAMA3_8B, layers=_env_int("MXB_BENCH_LAYERS", 32))
    sizes = [synth.tensor_nbytes(s, d) for _n, s, d, _k in synth.dense_tensors(cfg)]
    total = sum(sizes)
    g = torch.Generator(device="cuda")
    g.manual_seed(1 + rank)
    arena = torch.randint(0, 256, (total,), dtype=torch.uint8, device="cuda", generator=g)
    spans, pos = [], 0
    for n in sizes:
        spans.append((arena.data_ptr() + pos, n))
        pos += n
    torch.cuda.synchronize()
    results = {}
    for label, modes in (("all", DIGEST_SAFE32 | DIGEST_ROWS | DIGEST_BLOCK64),
                         ("safe32", DIGEST_SAFE32), ("rows", DIGEST_ROWS), ("block64", DIGEST_BLOCK64)):
        for _ in range(max(3, args.warmup)):
            recs = ctx.digest(spans, modes, local)
        _barrier(world)
        torch.cuda.synchronize()
        ctx.event_record(0, local)
        for _ in range(args.steps):
            recs = ctx.digest(spans, modes, local)
        ctx.event_record(1, local)
        ms = _max(ctx.event_elapsed_ms(0, 1, local), world)
        results[label] = (ms / args.steps, recs)
    ms_all = results["all"][0]
    peak, src = _peaks()
    achieved = total / (ms_all * 1e-3) / 1e9
    out = _base("GB/s digested (safe_checksum + tensor_digest scalars + block hash, one pass)",
                achieved * world, "GB/s", world, args, ms_all,
                {"workload": "Llama-3-8B-sized byte image resident in HBM, 291 ranges, one launch",
                 "bytes_per_gpu_per_step": total, "l2": "input larger than L2",
                 "per_mode_ms": {k: round(v[0], 4) for k, v in results.items()},
                 "per_mode_gbs": {k: round(total / (v[0] * 1e-3) / 1e9, 1) for k, v in results.items()}})
    out["gpu_launches"] = args.steps
    out["roofline"] = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                       "frac": round(achieved / peak, 4), "traffic": None, "kernel": "digest_kernel",
                       "peak_source": src + "; read-only kernel against a read+write copy figure",
                       "algorithmic_bytes_per_launch": total}
    if rank == 0 and world == 1 and os.environ.get("MXB_BENCH_SKIP_CPU") != "1":
        from oracle import c_port  # cpu_baseline leg: the checker and the timed CPU port

        n = 1 << 30
        host = arena[:n].cpu().numpy()
        rec = ctx.digest([(arena.data_ptr(), n)], 7, local)[0]
        sc = c_port.digest_scalars(host, mt=True)
        if (format(rec.safe_checksum, "08x") != c_port.safe_checksum(host, mt=True)
                or int(rec.row_sum) != sc[1] or int(rec.row_sum_w) != sc[2]
                or int(rec.block_hash) != c_port.block_hash64(host)):
            raise SystemExit("digest bench: kernel disagrees with the oracle")
        t0 = time.perf_counter()
        c_port.safe_checksum(host, mt=True)
        c_port.digest_scalars(host, mt=True)
        c_port.block_hash64(host)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": round(n / dt / 1e9, 3), "unit": "GB/s", "cores": os.cpu_count(),
                               "kind": "port", "sample": "first 1 GiB of the image, three digests, OpenMP"}
    if rank == 0:
        print(json.dumps(out), flush=True)
    ctx.close()


# ---------------------------------------------------------------------------
# fan-out
# ---------------------------------------------------------------------------


def _layout_ranges(sizes, align=256):
    offs, pos = [], 0
    for n in sizes:
        offs.append(pos)
        pos = (pos + n + align - 1) // align * align
    return offs, pos


def fanout_measure(args, ctx, rank, world, local, nv=None) -> dict:
    """Broadcast the 8B weights (TP=1 copy on GPU 0) to every other GPU, sweeping
    the chunk size; with an even GPU count also the rank-matched pair copy (first
    half of the GPUs -> second half, two TP=8 shards each at 8 GPUs).  Comparison
    line: ncclBroadcast of the same bytes.  Every destination is checked."""
    import torch

    from modelexpress_b200 import synth
    from modelexpress_b200.fanout import topology
    from modelexpress_b200.runtime import DIGEST_BLOCK64, DIGEST_SAFE32

    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 3))
    cfg = synth.scaled(synth.LLAMA3_8B, layers=_env_int("MXB_BENCH_LAYERS", 32))
    sizes = [synth.tensor_nbytes(s, d) for _n, s, d, _k in synth.dense_tensors(cfg)]
    offs, total = _layout_ranges(sizes)
    payload = sum(sizes)
    base = ctx.alloc(total, local)
    arena = as_tensor(base, total, local)   # only to fill / check the library-owned arena
    if rank == 0:
        g = torch.Generator(device="cuda")
        g.manual_seed(1)
        arena.copy_(torch.randint(0, 256, (total,), dtype=torch.uint8, device="cuda", generator=g))
    else:
        arena.zero_()
    torch.cuda.synchronize()
    peers = _open_peers(ctx, base, world)
    spans = [(base + o, n) for o, n in zip(offs, sizes)]
    topologies = {}
    kinds = os.environ.get("MXB_FANOUT_TOPOLOGY", "chain").split(",")
    # the sweep the benchmark configuration names (1, 4, 16, 64 MiB) plus two finer points (a chunk
    # of one 64 KiB piece is the finest the counters resolve)
    chunks_mib = {"vector": [float(x) for x in os.environ.get("MXB_FANOUT_CHUNKS", "0.0625,0.25,1,4,16,64").split(",")],
                  "dma": [64.0]}
    # the copy-engine push announces everything at the end: it is measured where the broadcast is
    # one hop (two GPUs); on a longer chain every hop would wait for the whole payload
    engines = os.environ.get("MXB_FANOUT_ENGINES", "vector,dma" if world == 2 else "vector").split(",")
    launches = 0
    for kind in kinds:
        children = topology(kind, world, 0)
        by_engine = {}
        for engine in engines:
            sweep = {}
            for mib in chunks_mib.get(engine, chunks_mib["vector"]):
                node = ctx.fanout(spans, int(mib * (1 << 20)) // 4096 * 4096, local)
                node.set_engine(engine)
                ctrs = _open_peers(ctx, node.counters, world)
                for c in children[rank]:
                    node.add_child([(peers[c] + o, n) for o, n in zip(offs, sizes)], ctrs[c])
                _barrier(world)
                times = []
                for it in range(warmup + steps):
                    if rank != 0:
                        arena.zero_()
                        torch.cuda.synchronize()
                    _barrier(world)
                    t0 = time.perf_counter()
                    before = ctx.launch_count
                    node.run(rank == 0, 20000)
                    ms = node.wait()
                    wall = (time.perf_counter() - t0) * 1e3
                    ms = _max(ms, world)
                    wall = _max(wall, world)
                    launches += ctx.launch_count - before
                    if it >= warmup:
                        times.append((ms, wall))
                dev_ms = sum(t[0] for t in times) / len(times)
                wall_ms = sum(t[1] for t in times) / len(times)
                sweep[f"{mib:g}"] = {"device_ms": round(dev_ms, 3), "wall_ms": round(wall_ms, 3),
                                   "gbs_per_target": round(payload / (dev_ms * 1e-3) / 1e9, 1),
                                   "gbs_aggregate": round(payload * (world - 1) / (dev_ms * 1e-3) / 1e9, 1)}
                # every destination range must digest like the source's
                recs = ctx.digest(spans, DIGEST_SAFE32 | DIGEST_BLOCK64, local)
                mine = [(int(r.safe_checksum), int(r.block_hash)) for r in recs]
                alld = _gather_objects(mine, world)
                for r in range(1, world):
                    if alld[r] != alld[0]:
                        raise SystemExit(f"fan-out ({kind}, {engine}): rank {r} digests differ from the source "
                                         f"(chunk {mib:g} MiB)")
                _barrier(world)
                node.close()
            best = max(sweep, key=lambda k: sweep[k]["gbs_per_target"])
            by_engine[engine] = {"chunk_sweep_mib": sweep, "best_chunk_mib": float(best),
                                 "gbs_per_target": sweep[best]["gbs_per_target"],
                                 "device_ms": sweep[best]["device_ms"]}
        top = max(by_engine, key=lambda e: by_engine[e]["gbs_per_target"])
        topologies[kind] = dict(by_engine[top], engine=top, engines=by_engine)
    # comparison line: ncclBroadcast of the same arena
    import torch.distributed as dist

    nccl = None
    if world > 1:
        for _ in range(2):
            dist.broadcast(arena, src=0)
        torch.cuda.synchronize()
        _barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            dist.broadcast(arena, src=0)
        e1.record()
        torch.cuda.synchronize()
        ms = _max(e0.elapsed_time(e1) / steps, world)
        nccl = {"device_ms": round(ms, 3), "gbs_per_target": round(total / (ms * 1e-3) / 1e9, 1),
                "what": "torch.distributed.broadcast (ncclBroadcast) of the same arena, CUDA events, slowest rank"}
    # rank-matched pair copy: the first half of the GPUs each hold two TP=8 shards and
    # replicate them to the matching GPU of the second half (independent 1-hop copies)
    pairs = None
    if world % 2 == 0:
        half = world // 2
        shard = 2008031232
        pay = 2 * shard if total >= 2 * shard else (total // 512) * 256
        pspans = [(base, pay)]
        if rank < half:
            g = torch.Generator(device="cuda")
            g.manual_seed(100 + rank)
            arena[:pay].copy_(torch.randint(0, 256, (pay,), dtype=torch.uint8, device="cuda", generator=g))
        torch.cuda.synchronize()
        # one hop: 256 KiB pieces (fewer system-scope fences per byte than the chain's 64 KiB) for the
        # store kernel; the copy-engine push beside it (every range one peer copy, one announcement)
        pairs = {"pairs": half, "bytes_per_pair": pay, "piece_bytes": 256 << 10}
        for engine in ("vector", "dma"):
            node = ctx.fanout(pspans, 16 << 20, local, 256 << 10)
            node.set_engine(engine)
            ctrs = _open_peers(ctx, node.counters, world)
            if rank < half:
                node.add_child([(peers[rank + half], pay)], ctrs[rank + half])
            _barrier(world)
            times = []
            for it in range(warmup + steps):
                if rank >= half:
                    arena[:pay].zero_()
                    torch.cuda.synchronize()
                _barrier(world)
                node.run(rank < half, 20000)
                ms = _max(node.wait(), world)
                launches += 1
                if it >= warmup:
                    times.append(ms)
            recs = ctx.digest(pspans, DIGEST_SAFE32 | DIGEST_BLOCK64, local)
            alld = _gather_objects((int(recs[0].safe_checksum), int(recs[0].block_hash)), world)
            for r in range(half):
                if alld[r] != alld[r + half]:
                    raise SystemExit(f"pair copy ({engine}): GPU {r + half} differs from GPU {r}")
            pms = sum(times) / len(times)
            res_e = {"device_ms": round(pms, 3), "gbs_per_pair": round(pay / (pms * 1e-3) / 1e9, 1),
                     "gbs_aggregate": round(pay * half / (pms * 1e-3) / 1e9, 1)}
            pairs[engine] = res_e
            _barrier(world)
            node.close()
        best = max(("vector", "dma"), key=lambda e: pairs[e]["gbs_per_pair"])
        pairs.update(pairs[best], engine=best)
    first = topologies[kinds[0]]
    peak = (nv or {}).get("peak_gbs")
    res = {"workload": "configs[2]: 16.06 GB TP=1 copy on GPU 0 broadcast over NVLink P2P stores",
           "payload_bytes": payload, "ranges": len(sizes), "topology": kinds[0],
           "gbs_per_target": first["gbs_per_target"], "device_ms": first["device_ms"],
           "best_chunk_mib": first["best_chunk_mib"], "engine": first["engine"],
           "topologies": topologies,
           "rank_matched_pairs": pairs, "nccl_broadcast": nccl, "gpu_launches": launches,
           "frac_of_nominal_900": round(first["gbs_per_target"] / NVLINK_NOMINAL_GBS, 4),
           "frac_of_measured_peak": round(first["gbs_per_target"] / peak, 4) if peak else None,
           "check": "ok: safe_checksum and 64-bit block hash of every destination range equal the source, "
                    "every topology and chunk size; pair copies equal their sources"}
    del arena
    ctx.free(base, local)
    return res


def _fanout_loopback(args, local):
    """One GPU: the root's kernel pushes into a second buffer of the same device, then the leaf's
    kernel finds every chunk arrived (kernels that wait on one another never share a GPU).  The
    same ``fanout_kernel`` as between GPUs with HBM in place of the link: what a profiler can be
    pointed at, since a multi-rank command cannot be profiled."""
    import torch

    from modelexpress_b200.runtime import DIGEST_BLOCK64, DIGEST_SAFE32, Context

    ctx = Context([local])
    mib = _env_int("MXB_FANOUT_LOOPBACK_MIB", 2048)
    sizes = [(mib << 20) // 40 // 256 * 256] * 40
    offs, total = _layout_ranges(sizes)
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    src = torch.randint(0, 256, (total,), dtype=torch.uint8, device="cuda", generator=g)
    dst = torch.zeros(total, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    s_spans = [(src.data_ptr() + o, n) for o, n in zip(offs, sizes)]
    d_spans = [(dst.data_ptr() + o, n) for o, n in zip(offs, sizes)]
    root, leaf = ctx.fanout(s_spans, 64 << 10, local), ctx.fanout(d_spans, 64 << 10, local)
    root.add_child(d_spans, leaf.counters)
    times = []
    for it in range(max(3, args.warmup) + args.steps):
        root.run(True, 5000)
        ms = root.wait()
        leaf.run(False, 5000)
        leaf.wait()
        if it >= max(3, args.warmup):
            times.append(ms)
    a = [(int(r.safe_checksum), int(r.block_hash)) for r in ctx.digest(s_spans, DIGEST_SAFE32 | DIGEST_BLOCK64, local)]
    b = [(int(r.safe_checksum), int(r.block_hash)) for r in ctx.digest(d_spans, DIGEST_SAFE32 | DIGEST_BLOCK64, local)]
    if a != b:
        raise SystemExit("fan-out loopback: destination digests differ from the source")
    ms = sum(times) / len(times)
    payload = sum(sizes)
    peak, peak_src = _peaks()
    gbs = 2 * payload / (ms * 1e-3) / 1e9
    out = _base("fan-out loopback GB/s read+write (root kernel into a buffer of the same GPU)", gbs, "GB/s", 1, args, ms,
                {"workload": f"{payload} B in 40 ranges, 64 KiB chunks of one piece, same-device child",
                 "l2": "input larger than L2", "check": "digests of every destination range equal the source"})
    out["gpu_launches"] = 2 * (max(3, args.warmup) + args.steps)
    out["roofline"] = {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                       "frac": round(gbs / peak, 4), "traffic": None, "kernel": "fanout_kernel",
                       "peak_source": peak_src, "algorithmic_bytes_per_launch": 2 * payload}
    print(json.dumps(out), flush=True)
    root.close()
    leaf.close()
    ctx.close()


def run_fanout(args):
    import torch.distributed as dist

    from modelexpress_b200.runtime import Context

    rank, world, local = _dist()
    if world < 2:
        return _fanout_loopback(args, local)
    ctx = Context([local])
    nv = nvlink_peaks(ctx, rank, world, local)
    res = fanout_measure(args, ctx, rank, world, local, nv)
    out = _base("fan-out GB/s delivered per target (8B bf16 weights, GPU 0 -> all others)",
                res["gbs_per_target"], "GB/s", world, args, res["device_ms"],
                {k: v for k, v in res.items() if k not in ("gpu_launches",)}, scaling="strong")
    out["config"]["nvlink_measured"] = nv
    out["gpu_launches"] = res["gpu_launches"]
    out["roofline"] = {"bound": "nvlink", "achieved": res["gbs_per_target"], "peak": nv["peak_gbs"],
                       "unit": "GB/s", "frac": res["frac_of_measured_peak"], "traffic": None,
                       "kernel": "fanout_kernel",
                       "peak_source": "best plain peer copy measured in this run, per direction per GPU "
                                      "(900 GB/s nominal)"}
    if rank == 0:
        print(json.dumps(out), flush=True)
    ctx.close()
    dist.destroy_process_group()


# ---------------------------------------------------------------------------
# reshard
# ---------------------------------------------------------------------------

_PAT_A, _PAT_B = 2654435761, 40503


def _pattern_words(torch, param_id: int, w0: int, n: int, device):
    """int32 words of parameter ``param_id`` at word indices [w0, w0+n): a value
    that depends on where the word sits in the FULL tensor, so a misplaced slice
    cannot pass."""
    idx = torch.arange(w0, w0 + n, dtype=torch.int64, device=device)
    return ((idx * _PAT_A + param_id * _PAT_B) & 0xFFFFFFFF).to(torch.int32)


def reshard_measure(args, ctx, rank, world, local, nv=None) -> dict:
    """FSDP-8 flat shards -> TP-8 parameters with fused qkv_proj / gate_up_proj.
    The 8 trainer ranks and 8 inference ranks are spread round-robin over the
    available GPUs (8 GPUs: one each); every source rank pushes its records with
    one scatter launch, stores to other GPUs crossing NVLink.  Comparison line:
    an all_to_all_single (NCCL grouped send/recv) of the bytes that cross."""
    import torch

    from modelexpress_b200 import layout, reshard, synth
    from modelexpress_b200.runtime import SCATTER_VECTOR

    steps, warmup = max(1, min(args.steps, 10)), max(1, min(args.warmup, 3))
    R = 8
    if R % world:
        raise SystemExit("reshard bench: the GPU count must divide 8")
    cfg = synth.scaled(synth.QWEN25_32B, layers=_env_int("MXB_RESHARD_LAYERS", 64))
    tensors = synth.dense_tensors(cfg)
    index = {n: {"shape": list(s), "dtype": d} for n, s, d, _k in tensors}
    pid = {n: i for i, (n, _s, _d, _k) in enumerate(tensors)}
    sa = reshard.shard_arena(index, R)
    plans = [layout.plan_checkpoint(index, t, R, "dense") for t in range(R)]
    pa = reshard.param_arena(plans[0])
    mine = [r for r in range(R) if r % world == rank]  # logical ranks hosted on this GPU
    per = len(mine)
    shard_base = ctx.alloc(sa.total * per, local)
    param_base = ctx.alloc(pa.total * per, local)
    shards_t = as_tensor(shard_base, sa.total * per, local)
    params_t = as_tensor(param_base, pa.total * per, local)
    # fill this GPU's flat shards with the position pattern
    for j, r in enumerate(mine):
        for name, off in sa.offsets.items():
            nb = sa.sizes[name]
            words = _pattern_words(torch, pid[name], r * nb // 4, nb // 4, "cuda")
            shards_t[j * sa.total + off: j * sa.total + off + nb].view(torch.int32).copy_(words)
    params_t.zero_()
    torch.cuda.synchronize()
    peer_params = _open_peers(ctx, param_base, world)
    param_bases = [peer_params[t % world] + (t // world) * pa.total for t in range(R)]
    t0 = time.perf_counter()
    nbytes, remote, nrecs = 0, 0, 0
    all_recs = []
    for j, r in enumerate(mine):
        recs = reshard.plan_reshard(index, R, R, r, shard_base + j * sa.total, param_bases, "dense",
                                    shards=sa, params=pa)
        nbytes += reshard.reshard_bytes(recs)
        nrecs += len(recs)
        lo, hi = param_base, param_base + pa.total * per
        far = (recs[:, 1] < lo) | (recs[:, 1] >= hi)
        remote += int((recs[far, 2] * recs[far, 3]).sum())
        all_recs.append(recs)
    # one resident table (one launch) per GPU for all the logical ranks it hosts
    table = ctx.table(np.concatenate(all_recs), local)
    plan_s = time.perf_counter() - t0
    from modelexpress_b200.runtime import SCATTER_OVERLAP

    schedules = {"two kernels side by side": SCATTER_OVERLAP, "one kernel after the other": 0}
    if os.environ.get("MXB_SCATTER", "auto") == "vec":
        schedules = {"vector engine only": SCATTER_VECTOR}
    parts = {}
    if os.environ.get("MXB_RESHARD_PARTS") == "1":   # each engine's share of the table alone
        parts = {"bulk-engine part alone (local copies)": 8, "vector-engine part alone (peer stores)": 16}
    per_schedule = {}
    for label, flags in {**parts, **schedules}.items():
        times = []
        for it in range(warmup + steps):
            _barrier(world)
            torch.cuda.synchronize()
            ctx.event_record(0, local)
            table.launch(flags)
            ctx.event_record(1, local)
            ms = ctx.event_elapsed_ms(0, 1, local)
            ctx.sync(local)
            _barrier(world)
            ms = _max(ms, world)
            if it >= warmup:
                times.append(ms)
        per_schedule[label] = round(sum(times) / len(times), 4)
    best_label = min(schedules, key=per_schedule.get)
    ms, flags = per_schedule[best_label], schedules[best_label]
    # the pattern check below reads what the last launch wrote; make that the reported schedule
    params_t.zero_()
    torch.cuda.synchronize()
    _barrier(world)
    table.launch(flags)
    ctx.sync(local)
    _barrier(world)
    # check every destination parameter hosted here against the pattern
    bad = 0
    for j, t in enumerate(mine):
        plan = plans[t]
        for pl in plan.placements:
            so, do, rows, rb, sp, dp = pl.geometry()
            dst0 = j * pa.total + pa.offsets[pl.dst_name] + do
            # compare row by row in bulk: build expected words for the strided source region
            r_idx = torch.arange(rows, dtype=torch.int64, device="cuda").unsqueeze(1)
            c_idx = torch.arange(rb // 4, dtype=torch.int64, device="cuda").unsqueeze(0)
            widx = (so // 4) + r_idx * (sp // 4) + c_idx
            exp = ((widx * _PAT_A + pid[pl.src_name] * _PAT_B) & 0xFFFFFFFF).to(torch.int32)
            if rows == 1:
                got = params_t[dst0: dst0 + rb].view(torch.int32).unsqueeze(0)
            else:
                got = torch.as_strided(params_t[dst0:].view(torch.int32), (rows, rb // 4), (dp // 4, 1))
            if not torch.equal(got, exp):
                bad += 1
            del exp, widx
    bad = int(_max(float(bad), world))
    if bad:
        raise SystemExit(f"reshard bench: {bad} placements differ from the expected pattern")
    engine = table.engine(flags)
    table.close()
    # comparison line: the bytes that cross NVLink as one all_to_all_single (the local HBM
    # copies and the fused concat would come on top of it)
    nccl = None
    if world > 1:
        import torch.distributed as dist

        per_peer = (remote // max(1, world - 1)) // 256 * 256
        send = params_t[: per_peer * world]
        recv = shards_t[: per_peer * world]
        for _ in range(2):
            dist.all_to_all_single(recv, send)
        torch.cuda.synchronize()
        _barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            dist.all_to_all_single(recv, send)
        e1.record()
        torch.cuda.synchronize()
        a2a = _max(e0.elapsed_time(e1) / steps, world)
        nccl = {"device_ms": round(a2a, 3), "bytes_per_peer": per_peer,
                "gbs_received_per_gpu": round(per_peer * (world - 1) / (a2a * 1e-3) / 1e9, 1),
                "what": "torch.distributed.all_to_all_single (NCCL grouped send/recv) of the cross-GPU bytes "
                        "only; the reshard's local copies and concatenation are not in it"}
    total_bytes = sum(p.bytes_placed for p in plans)
    peak_hbm, src = _peaks()
    link = (nv or {}).get("peak_gbs") or NVLINK_NOMINAL_GBS
    # per GPU: local records are read and written here; remote ones are read here, and as many
    # bytes arrive from the peers and are written here
    hbm_time = 2.0 * nbytes / (peak_hbm * 1e9)
    bound_meas = max(hbm_time, remote / (link * 1e9))
    bound_nom = max(hbm_time, remote / (NVLINK_NOMINAL_GBS * 1e9))
    res = {"workload": "configs[3]: Qwen2.5-32B shapes, 771 parameters, 65.5 GB, flat 8-way FSDP shards -> "
                       "vLLM TP=8 layout with fused qkv_proj / gate_up_proj",
           "layers": cfg.layers, "seconds": round(ms * 1e-3, 6), "device_ms": round(ms, 4),
           "bytes_written_total": total_bytes, "bytes_pushed_per_gpu": nbytes,
           "bytes_crossing_nvlink_per_gpu": remote, "records_per_gpu": nrecs,
           "plan_seconds": round(plan_s, 3),
           "gbs_written_aggregate": round(total_bytes / (ms * 1e-3) / 1e9, 1),
           "nvlink_gbs_per_gpu": round(remote / (ms * 1e-3) / 1e9, 1),
           "engine": engine, "schedule": best_label, "device_ms_per_schedule": per_schedule,
           "gpu_launches": (warmup + steps) * len(schedules) + 1,
           "bound_seconds_measured_peaks": round(bound_meas, 6),
           "bound_seconds_nominal_900": round(bound_nom, 6),
           "frac_of_measured_bound": round(bound_meas / (ms * 1e-3), 4),
           "frac_of_nominal_bound": round(bound_nom / (ms * 1e-3), 4),
           "bound_how": f"max(HBM: 2 x bytes pushed per GPU / {peak_hbm} GB/s {src}; NVLink: bytes "
                        f"crossing per GPU / link rate ({link} GB/s measured in this run, 900 nominal))",
           "nccl_all_to_all": nccl,
           "check": "ok: every destination word equals the position pattern of its source element"}
    del shards_t, params_t
    ctx.free(shard_base, local)
    ctx.free(param_base, local)
    return res, cfg, R


def run_reshard(args):
    from modelexpress_b200.runtime import Context

    rank, world, local = _dist()
    ctx = Context([local])
    nv = nvlink_peaks(ctx, rank, world, local) if world > 1 else None
    res, cfg, R = reshard_measure(args, ctx, rank, world, local, nv)
    out = _base("refit reshard seconds (Qwen2.5-32B bf16, FSDP-8 -> TP-8, fused qkv/gate_up)",
                res["seconds"], "s", world, args, res["device_ms"],
                {k: v for k, v in res.items() if k != "gpu_launches"}, scaling="strong")
    out["config"]["nvlink_measured"] = nv
    out["higher_is_better"] = False
    out["gpu_launches"] = res["gpu_launches"]
    out["roofline"] = {"bound": "nvlink" if world > 1 else "hbm", "achieved": res["seconds"],
                       "peak": res["bound_seconds_measured_peaks"], "unit": "s",
                       "frac": res["frac_of_measured_bound"], "traffic": None,
                       "kernel": "scatter_bulk_kernel + scatter_vec_kernel" if res["engine"] != "vector"
                       else "scatter_vec_kernel", "peak_source": res["bound_how"]}
    if rank == 0 and world == 1 and os.environ.get("MXB_BENCH_SKIP_CPU") != "1":
        out["cpu_baseline"] = _reshard_cpu_baseline(cfg, R)
    if rank == 0:
        print(json.dumps(out), flush=True)
    ctx.close()
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def multi_gpu_section(args, ctx, rank, world, local) -> dict:
    """Fan-out and refit reshard on the GPUs of this run, with the link rates a plain
    copy reaches measured first; attached to the placement line when N > 1."""
    out = {"gpus": world}
    nv = nvlink_peaks(ctx, rank, world, local)
    out["nvlink_measured"] = nv
    out["fanout"] = fanout_measure(args, ctx, rank, world, local, nv)
    if 8 % world == 0:
        out["reshard"] = reshard_measure(args, ctx, rank, world, local, nv)[0]
    return out


def _reshard_cpu_baseline(cfg, R):
    """The reference's CPU regather-and-reslice (its memmove transport loop,
    refit/reshard/transport/base.py:56-62, here the oracle's C port on all host
    threads) over a 2-layer model of the same shapes: the same plan, host buffers."""
    from modelexpress_b200 import layout, reshard, synth
    from oracle import c_port  # cpu_baseline leg: the timed CPU port

    small = synth.scaled(cfg, layers=2)
    tensors = synth.dense_tensors(small)
    index = {n: {"shape": list(s), "dtype": d} for n, s, d, _k in tensors}
    sa = reshard.shard_arena(index, R)
    pa = reshard.param_arena(layout.plan_checkpoint(index, 0, R, "dense"))
    shards = [np.full(sa.total, 7, dtype=np.uint8) for _ in range(R)]  # memmove speed is data-independent
    params = [np.full(pa.total, 1, dtype=np.uint8) for _ in range(R)]  # touched, so no page faults are timed
    recs = [reshard.plan_reshard(index, R, R, s, shards[s].ctypes.data, [p.ctypes.data for p in params],
                                 "dense", shards=sa, params=pa) for s in range(R)]
    moved = sum(reshard.reshard_bytes(r) for r in recs)
    c_port.scatter2d(recs[0].tolist(), mt=True)  # warm
    t0 = time.perf_counter()
    for r in recs:
        c_port.scatter2d(r.tolist(), mt=True)
    dt = time.perf_counter() - t0
    return {"value": round(moved / dt / 1e9, 3), "unit": "GB/s written", "cores": os.cpu_count(),
            "kind": "port", "sample": f"2 of {cfg.layers} layers plus embed/lm_head ({moved} B), "
                                      "all 8 source ranks, OpenMP memmove loop over the same records"}


# ---------------------------------------------------------------------------
# vLLM seam
# ---------------------------------------------------------------------------


def run_vllm(args):
    """Time to loaded weights at the seam the reference plugs into: vLLM's
    model-loader interface (engines/vllm/loader.py:62-183 in the reference).
    One real ``LlamaForCausalLM`` is built on the GPU; each step loads every
    parameter from safetensors files in the page cache, once per arm:
    ``MxModelLoader.load_weights`` (capture of vLLM's own load_weights -> pinned
    ring -> PCIe -> scatter kernel) and vLLM's ``DefaultModelLoader.load_weights``
    (what the reference's chain ends in).  Both must leave identical parameters."""
    import torch

    from modelexpress_b200 import synth
    from modelexpress_b200.digest import digest_many
    from modelexpress_b200.engines.vllm.loader import MxModelLoader

    rank, world, local = _dist()
    if world != 1:
        raise SystemExit("the vllm workload runs on one GPU")
    try:
        from vllm.config import (DeviceConfig, LoadConfig, ModelConfig, VllmConfig,
                                 set_current_vllm_config)
        from vllm.distributed import parallel_state as ps
        from vllm.model_executor.model_loader.default_loader import DefaultModelLoader
        from vllm.model_executor.model_loader.utils import initialize_model
        from vllm.utils.torch_utils import set_default_torch_dtype
    except Exception as e:
        raise SystemExit(f"the vllm workload needs vLLM: {type(e).__name__}: {e}")

    cfg = synth.scaled(synth.LLAMA3_8B, layers=_env_int("MXB_BENCH_LAYERS", 32))
    tensors = synth.dense_tensors(cfg)
    total = sum(synth.tensor_nbytes(s, d) for _n, s, d, _k in tensors)
    root = os.environ.get("MXB_BENCH_DIR", "/tmp/mxb_bench")
    d = synth.ensure_checkpoint(os.path.join(root, f"vllm_{cfg.name}_{cfg.layers}"), tensors, 1, 4,
                                device="cuda")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({"architectures": ["LlamaForCausalLM"], "model_type": "llama",
                   "hidden_size": cfg.hidden, "intermediate_size": cfg.intermediate,
                   "num_hidden_layers": cfg.layers, "num_attention_heads": cfg.q_heads,
                   "num_key_value_heads": cfg.kv_heads, "head_dim": cfg.head_dim,
                   "vocab_size": cfg.vocab, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5,
                   "rope_theta": 500000.0, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
                   "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2}, f)
    mc = ModelConfig(model=d, skip_tokenizer_init=True, dtype="bfloat16", enforce_eager=True)
    vc = VllmConfig(model_config=mc, device_config=DeviceConfig(device="cuda"),
                    load_config=LoadConfig(load_format="dummy"))
    with set_current_vllm_config(vc):
        ps.init_distributed_environment(world_size=1, rank=0, local_rank=0, backend="nccl",
                                        distributed_init_method=f"tcp://127.0.0.1:{29600 + os.getpid() % 300}")
        ps.initialize_model_parallel(1, 1)
        with set_default_torch_dtype(torch.bfloat16), torch.device("cuda"):
            model = initialize_model(vllm_config=vc)
        params = [p.data for _n, p in model.named_parameters()]
        loaded_bytes = sum(p.numel() * p.element_size() for p in params)

        def digests():
            return [(r["safe_checksum"], r["block_hash64"]) for r in digest_many(params)]

        def timed(fn, steps, warmup):
            for _ in range(warmup):
                fn()
            times = []
            for _ in range(steps):
                for p in params:
                    p.zero_()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                fn()
                torch.cuda.synchronize()
                times.append(time.perf_counter() - t0)
            return times

        ours = MxModelLoader(LoadConfig(load_format="auto"))
        t_ours = timed(lambda: ours.load_weights(model, mc), args.steps, max(1, args.warmup))
        if ours.last_strategy != "b200_captured" or (ours.last_metadata or {}).get("engine_loaded", 1) != 0:
            raise SystemExit(f"vllm bench: weights were placed by {ours.last_strategy!r} with "
                             f"{(ours.last_metadata or {}).get('engine_loaded')} tensors left to the "
                             "engine's own loader (expected: b200_captured, none)")
        mine = digests()
        # the same seam when the engine reloads weights it has loaded before (MXB_PIN=keep): the
        # first load keeps page-locked images, later ones skip the dry run and the gather
        os.environ["MXB_PIN"] = "keep"
        try:
            kept = MxModelLoader(LoadConfig(load_format="auto"))
            t_first = timed(lambda: kept.load_weights(model, mc), 1, 0)
            t_kept = timed(lambda: kept.load_weights(model, mc), max(2, min(args.steps, 5)), 1)
        finally:
            os.environ.pop("MXB_PIN", None)
        if digests() != mine:
            raise SystemExit("vllm bench: a reload from kept images changed the parameters")
        from modelexpress_b200.loader import host_images

        kept_bytes = host_images.packed_bytes
        host_images.close()
        native = DefaultModelLoader(LoadConfig(load_format="auto"))
        native_steps = max(1, min(args.steps, _env_int("MXB_BENCH_NATIVE_STEPS", 3)))
        t_native = timed(lambda: native.load_weights(model, mc), native_steps, 1)
        if digests() != mine:
            raise SystemExit("vllm bench: parameters differ between the two loaders")
    s_ours, s_native = sum(t_ours) / len(t_ours), sum(t_native) / len(t_native)
    out = _base("GB/s of parameters loaded through vLLM's model-loader seam (files in page cache -> HBM)",
                loaded_bytes / s_ours / 1e9, "GB/s", 1, args, s_ours * 1e3,
                {"workload": f"vLLM LlamaForCausalLM, Llama-3-8B shapes, {cfg.layers} layers, TP=1, bf16, "
                             f"4 safetensors files ({total} B), every parameter loaded per step",
                 "parameter_bytes": loaded_bytes, "l2": "input larger than L2",
                 "seconds_per_load": round(s_ours, 4), "best_seconds": round(min(t_ours), 4),
                 "seconds_each": [round(t, 4) for t in t_ours], "last_load": ours.last_metadata})
    out["e2e"] = {"value": out["value"], "unit": "GB/s", "h2d_bytes_per_step": loaded_bytes,
                  "d2h_bytes_per_step": 0}
    s_kept = sum(t_kept) / len(t_kept)
    out["reload_from_kept_images"] = {
        "value": round(loaded_bytes / s_kept / 1e9, 2), "unit": "GB/s", "seconds_per_load": round(s_kept, 4),
        "first_load_s": round(t_first[0], 4), "page_locked_bytes": int(kept_bytes),
        "what": "MXB_PIN=keep: MxModelLoader.load_weights again on the same model; no dry run, no gather, "
                "one copy-engine transfer and one scatter launch per chunk", "parameters_identical": True}
    out["engine_default_loader"] = {
        "value": round(loaded_bytes / s_native / 1e9, 2), "unit": "GB/s", "steps": native_steps,
        "seconds_per_load": round(s_native, 4), "best_seconds": round(min(t_native), 4),
        "what": "vllm DefaultModelLoader.load_weights on the same model and files",
        "parameters_identical": True}
    out["gpu_launches"] = None
    print(json.dumps(out), flush=True)


def _refit_cast_step(torch, local) -> dict:
    """One refit step whose trainer publishes fp32 and whose engine holds bf16: eight 8192 x 8192
    parameters, each source in eight row shards on this GPU, through ``ReshardReceiver``.  Fused:
    the convert kernel reads the shards in place.  Staged: the reference's order (pull the served
    dtype into a staging buffer, cast afterwards; transfer_plan.py:49-60, receiver.py:964-971)."""
    from modelexpress_b200.planner import ShardSpec, SourceSpec
    from modelexpress_b200.refit import ReshardReceiver

    rows, cols, layers = 8192, 8192, 8

    class Engine(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.ParameterList(
                [torch.nn.Parameter(torch.zeros(rows, cols, dtype=torch.bfloat16)) for _ in range(layers)])

        def load_weights(self, weights):
            for name, w in weights:
                self.w[int(name[1:])].data.copy_(w)

    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    srcs = [torch.randn(rows, cols, device="cuda", generator=g) for _ in range(layers)]
    per = rows // 8
    sources = {f"w{i}": SourceSpec((rows, cols), torch.float32, 4,
                                   [ShardSpec((s * per, 0), (per, cols), "t0", t.data_ptr() + s * per * cols * 4, 4)
                                    for s in range(8)]) for i, t in enumerate(srcs)}
    out = {"elements": rows * cols * layers, "bytes_read_plus_written": rows * cols * layers * 6}
    saved = os.environ.get("MXB_RESHARD_FUSED_CASTS")
    try:
        for label, fused in (("fused", "1"), ("staged", "0")):
            os.environ["MXB_RESHARD_FUSED_CASTS"] = fused
            model = Engine().to(f"cuda:{local}")
            rx = ReshardReceiver(model, device=f"cuda:{local}")
            rx.prepare(sources)
            staging = int(rx._staging.numel())
            steps = [rx.update_weights(k) for k in range(6)]
            for i, t in enumerate(srcs):
                if not torch.equal(model.w[i].data, t.to(torch.bfloat16)):
                    raise SystemExit(f"refit cast step ({label}): parameter {i} differs from torch's cast")
            best = min(steps[2:], key=lambda st: st["total_s"])
            out[label] = {"ms_per_step": round(best["total_s"] * 1e3, 3), "read_ms": round(best["read_s"] * 1e3, 3),
                          "install_ms": round(best["install_s"] * 1e3, 3), "staging_bytes": staging if staging > 1 else 0,
                          "gbs": round(out["bytes_read_plus_written"] / best["total_s"] / 1e9, 1)}
            rx.close()
            del model, rx
            torch.cuda.empty_cache()
    finally:
        if saved is None:
            os.environ.pop("MXB_RESHARD_FUSED_CASTS", None)
        else:
            os.environ["MXB_RESHARD_FUSED_CASTS"] = saved
    out["check"] = "every parameter bit-identical to torch's cast, both ways"
    return out


def run_convert(args):
    """The box-convert kernel on the parameter list of a Llama-3-8B-shaped model (every 2-D
    weight and the norms): cast fp32 -> bf16 (a trainer that serves fp32 masters), transposed
    bf16 (weights stored transposed) and both at once, one launch per case (every case holds one
    pair of dtypes); beside each the
    per-tensor ``dst.copy_(src)`` loop the reference leaves to torch (receiver.py:964-971).
    Every case is compared bit for bit with torch's result before it is timed."""
    import torch

    from modelexpress_b200 import synth
    from modelexpress_b200.runtime import Context

    rank, world, local = _dist()
    ctx = Context([local])
    layers = _env_int("MXB_CONVERT_LAYERS", 8)
    cfg = synth.scaled(synth.LLAMA3_8B, layers=layers, vocab=_env_int("MXB_CONVERT_VOCAB", synth.LLAMA3_8B.vocab))
    shapes = [tuple(s) for _n, s, _d, _k in synth.dense_tensors(cfg)]
    elems = sum(int(torch.Size(s).numel()) for s in shapes)
    g = torch.Generator(device="cuda")
    g.manual_seed(5 + rank)
    src32 = torch.randn(elems, dtype=torch.float32, device="cuda", generator=g)
    src16 = src32.to(torch.bfloat16)
    dst16 = torch.zeros(elems, dtype=torch.bfloat16, device="cuda")
    want = torch.zeros(elems, dtype=torch.bfloat16, device="cuda")
    peak, peak_src = _peaks()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    cases = {}
    for label, src, transposed in (("cast fp32 -> bf16", src32, False), ("transpose bf16", src16, True),
                                   ("transpose + cast fp32 -> bf16", src32, True)):
        boxes, views, pos = [], [], 0
        for shp in shapes:
            n = int(torch.Size(shp).numel())
            two_d = transposed and len(shp) == 2
            strides = [1, shp[0]] if two_d else [int(torch.Size(shp[k + 1:]).numel()) for k in range(len(shp))]
            kinds = ("f32", "bf16") if src.dtype == torch.float32 else ("raw", "raw")
            boxes.append((src.data_ptr() + pos * src.element_size(), dst16.data_ptr() + pos * 2, list(shp), strides,
                          kinds[0], kinds[1], src.element_size()))
            s_view = src[pos: pos + n].view(shp)
            views.append((s_view, torch.as_strided(want, shp, strides, pos)))
            pos += n
        # torch's loop: the check and the comparison line
        def torch_loop():
            for s_view, d_view in views:
                d_view.copy_(s_view)
        for _ in range(warmup):
            torch_loop()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            torch_loop()
        e1.record()
        torch.cuda.synchronize()
        torch_ms = _max(e0.elapsed_time(e1) / steps, world)
        dst16.zero_()
        torch.cuda.synchronize()
        moved = ctx.convert_boxes(boxes, local)
        if not torch.equal(dst16.view(torch.int16), want.view(torch.int16)):
            raise SystemExit(f"convert bench ({label}): kernel result differs from torch's copy")
        prepared = ctx.convert_array(boxes)
        for _ in range(warmup):
            ctx.convert_boxes(prepared, local)
        _barrier(world)
        total_ms = 0.0
        for _ in range(steps):   # table upload + kernel of each call, on the library's stream
            ctx.event_record(0, local)
            ctx.convert_boxes(prepared, local)
            ctx.event_record(1, local)
            total_ms += ctx.event_elapsed_ms(0, 1, local)
        ms = _max(total_ms / steps, world)
        cases[label] = {"ms": round(ms, 4), "gbs": round(moved / (ms * 1e-3) / 1e9, 1),
                        "frac_of_hbm_peak": round(moved / (ms * 1e-3) / 1e9 / peak, 4),
                        "bytes_read_plus_written": moved, "launches_per_step": 1,
                        "torch_copy_loop_ms": round(torch_ms, 4), "torch_launches_per_step": len(views),
                        "torch_gbs": round(moved / (torch_ms * 1e-3) / 1e9, 1), "check": "bit-identical to torch"}
    del src32, src16, dst16, want
    torch.cuda.empty_cache()
    refit = _refit_cast_step(torch, local)
    head = cases["cast fp32 -> bf16"]
    out = _base("GB/s converted (bytes read + written, box-convert kernel, one launch)", head["gbs"] * world,
                "GB/s", world, args, head["ms"],
                {"workload": f"Llama-3-8B parameter list, {layers} layers, {len(shapes)} tensors, "
                             f"{elems} elements resident in HBM", "l2": "input larger than L2", "cases": cases,
                 "refit_step_fp32_shards_to_bf16_params": refit},
                dtype="f32->bf16")
    out["gpu_launches"] = steps * len(cases)
    out["roofline"] = {"bound": "hbm", "achieved": head["gbs"], "peak": peak, "unit": "GB/s",
                       "frac": head["frac_of_hbm_peak"], "traffic": None, "kernel": "convert_kernel",
                       "peak_source": peak_src, "algorithmic_bytes_per_launch": head["bytes_read_plus_written"]}
    if rank == 0:
        print(json.dumps(out), flush=True)
    ctx.close()


def run(args):
    fn = {"digest": run_digest, "fanout": run_fanout, "reshard": run_reshard,
          "vllm": run_vllm, "convert": run_convert}.get(args.workload)
    if fn is None:
        raise SystemExit(f"unknown workload {args.workload!r}")
    return fn(args)

#!/usr/bin/env python
"""Benchmark of the token-sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one reuse-step attention call of the bf16 video-DiT configuration
(B=1, H=24, L=32,760, D=128, 256 query groups x top-k 2048 selected KV tokens, cached
residual added in the epilogue) on seeded synthetic clustered Q/K/V.  With N > 1 ranks the
same call runs as the attention core of a Ulysses context-parallel layer: each rank holds a
sequence shard, an all-to-all reshards to a head shard, the sparse attention runs on H/N
heads, an all-to-all returns to the sequence shard (strong scaling: total work fixed).

Prints ONE JSON line on rank 0.  ``value`` is effective TFLOP/s over the algorithmic FLOPs
4*L*K_sel*D*H with inputs resident in HBM; ``e2e`` is the same metric through the public
Python entry point with host buffers (pinned host -> device copy of q, k, v and device ->
host copy of the output inside the timed region).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "gather_kv_sparse_attn_effective_tflops"
UNIT = "TFLOP/s"
# DRAM traffic of one attention-kernel launch per head, from ncu captures of 4-head launches
# (dram__bytes_read.sum + dram__bytes_write.sum; summaries under profiles/)
NCU_DRAM_BYTES_PER_HEAD = {"c2": 0.94e9 / 24}


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16_tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples under load are the upper half of what was seen (idle samples bracket the region)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


def _config(shape, world: int, args, q_bytes_per_gpu: float, indices: str = ""):
    """The ``config`` object of the JSON line; both arms build it from the same arguments."""
    if world > 1:
        par = f"ulysses{world}-{args.ulysses}-chunks{args.chunks}" + (f"-scatter_{args.scatter}" if args.ulysses == "fused" else "") + \
              ("-graph" if args.graph and args.ulysses == "fused" else "")
    else:
        par = "single"
    return {"workload": shape.name, "B": 1, "H": shape.heads, "L": shape.seq_len, "D": shape.head_dim, "groups": shape.n_groups,
            "topk": shape.topk, "residual": "fused",
            "indices": indices or f"4 sinks + top-{shape.topk - 4} by exact fp32 group mass, ascending", "parallelism": par,
            "l2": f"inputs ({q_bytes_per_gpu / 1e9:.2f} GB per call and GPU) larger than L2; no explicit flush"}


def _input_bytes_per_gpu(shape, world: int) -> float:
    hl = shape.heads // world
    return 4.0 * shape.seq_len * hl * shape.head_dim * 2 + hl * shape.n_groups * shape.topk * 4.0


def _cpu_topmass_indices(q, k, shape, rows_per_chunk: int = 2048):
    """The configuration's index definition evaluated on the host for one head (oracle arithmetic, fp32,
    query groups a few at a time): 4 sinks + the top tokens by group mass, ascending."""
    import math
    import torch
    from oracle.select import select_topk_ref
    L, D = shape.seq_len, shape.head_dim
    qf, kf = q[0, :, 0].float(), k[0, :, 0].float()
    scale = 1.0 / math.sqrt(D)
    mass = torch.empty(shape.n_groups, L)
    for r0 in range(0, L, rows_per_chunk):
        r1 = min(L, r0 + rows_per_chunk)
        s = (qf[r0:r1] @ kf.T) * scale
        pr = torch.exp(s - torch.logsumexp(s, -1, keepdim=True))
        for g0 in range(r0, r1, shape.group_rows):
            mass[g0 // shape.group_rows] = pr[g0 - r0:min(g0 - r0 + shape.group_rows, r1 - r0)].sum(0)
    return select_topk_ref(mass, shape.topk, range(synth_n_sink())).view(1, 1, shape.n_groups, shape.topk)


def synth_n_sink() -> int:
    from mcsparse_b200 import synth
    return synth.N_SINK


def _cpu_oracle_sample(shape, budget_s: float, threads: int):
    """Times the CPU oracle (port of the reference math) on whole heads of the workload until
    ``budget_s`` is used.  Returns (tflops, heads_done, seconds)."""
    import torch
    from mcsparse_b200 import synth
    from oracle.gather_attn import gather_attn_ref
    torch.set_num_threads(threads)
    done, elapsed = 0, 0.0
    while done < shape.heads and (done == 0 or elapsed < budget_s):
        q, k, v = synth.clustered_qkv(shape, heads=1, head_offset=done)
        res = synth.residual_like(shape, heads=1, head_offset=done)
        gi = synth.random_sorted_indices(1, 1, shape.n_groups, shape.topk, shape.seq_len, seed=done)
        t0 = time.perf_counter()
        gather_attn_ref(q, k, v, gi, residual=res)
        elapsed += time.perf_counter() - t0
        done += 1
    return shape.attn_flops(done) / elapsed / 1e12, done, elapsed


def run_reference(args):
    """Reference arm: the reference ships no CPU (or sm_100) implementation of gather-KV attention,
    so the arm times the oracle port of its math on the host cores, same metric and config."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from mcsparse_b200 import synth
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    which = args.shape if args.shape != "auto" else ("c2" if world == 1 else "c5")
    shape = synth.C2 if which == "c2" else synth.C5          # the workload of the other arm at this GPU count
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    from oracle.gather_attn import gather_attn_ref
    heads_per_step = 1
    q, k, v = synth.clustered_qkv(shape, heads=heads_per_step)
    res = synth.residual_like(shape, heads=heads_per_step)
    gi = _cpu_topmass_indices(q, k, shape)          # same index definition as the other arm, built outside the timed steps
    for _ in range(args.warmup):
        gather_attn_ref(q, k, v, gi, residual=res)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        gather_attn_ref(q, k, v, gi, residual=res)
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    val = shape.attn_flops(heads_per_step) / (ms * 1e-3) / 1e12
    sample = f"{heads_per_step} of {shape.heads} heads per step (all {shape.n_groups} groups), torch fp32 on host"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": _config(shape, world, args, _input_bytes_per_gpu(shape, world)),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def _oracle_check(q, k, v, gi, residual, out, head: int, fp8=None):
    """Compares one head of a finished attention call with the CPU oracle (outside any timed region).
    q, k, v, out: (1, L, H, D) device tensors, residual (1, H, L, D), gi (1, H, M, K).  Returns the error figures
    and whether they are inside the tolerance stated for the path."""
    import torch
    from oracle.gather_attn import error_metrics, gather_attn_fp8_ref, gather_attn_ref
    sl = slice(head, head + 1)
    c = lambda t: t.cpu()
    if fp8 is None:
        ref, _ = gather_attn_ref(c(q[:, :, sl]), c(k[:, :, sl]), c(v[:, :, sl]), c(gi[:, sl]), residual=c(residual[:, sl]))
        tol = (2e-2, 1e-2)
    else:
        scale_qk, scale_v = fp8
        ref, _ = gather_attn_fp8_ref(c(q[:, :, sl]), c(k[:, :, sl]), c(v[:, :, sl]), c(gi[:, sl]), c(scale_qk[:, sl]),
                                     c(scale_v[:, sl]), residual=c(residual[:, sl]))
        tol = (6e-2, 3e-2)
    mx, mr = error_metrics(c(out[:, :, sl]).float(), ref)
    return {"against": "cpu oracle, fp32", "head": head, "max_abs": mx, "mean_rel": mr, "tol_max_abs": tol[0],
            "tol_mean_rel": tol[1], "ok": bool(mx < tol[0] and mr < tol[1])}


def _sequence_shards(shape, rank: int, world: int, dev, hc: int = 8):
    """This rank's (1, L/N, H, D) sequence shards of the SAME clustered q, k, v whose head shards the indices
    are built from (heads generated a few at a time to bound memory)."""
    import torch
    from mcsparse_b200 import synth
    H, L, D = shape.heads, shape.seq_len, shape.head_dim
    Ls = L // world
    outs = [torch.empty(1, Ls, H, D, dtype=torch.bfloat16, device=dev) for _ in range(3)]
    for h0 in range(0, H, hc):
        n = min(hc, H - h0)
        full = synth.clustered_qkv(shape, heads=n, head_offset=h0, device=dev)
        for o, t in zip(outs, full):
            o[:, :, h0:h0 + n] = t[:, rank * Ls:(rank + 1) * Ls]
        del full
    return outs


def _single_gpu_same_workload(shape, dev, attn_fn, steps: int = 3, compare_rows=None, compare_to=None):
    """All heads of `shape` on one GPU, in head chunks launched back to back (device-resident, CUDA events).
    With ``compare_to`` (a (1, rows, H, D) sequence shard produced by the multi-GPU step) the single-GPU outputs
    of rows ``compare_rows`` are compared with it, and head 0 is compared with the CPU oracle."""
    import torch
    from mcsparse_b200 import synth
    hc = 8 if shape.heads % 8 == 0 else shape.heads
    parts = []
    for h0 in range(0, shape.heads, hc):
        q, k, v = synth.clustered_qkv(shape, heads=hc, head_offset=h0, device=dev)
        res = synth.residual_like(shape, heads=hc, head_offset=h0, device=dev)
        parts.append((q, k, v, res, synth.topmass_indices(q, k, shape), torch.empty_like(q)))

    def run():
        for q, k, v, res, gi, out in parts:
            attn_fn(q, k, v, gi, out=out, residual=res)

    for _ in range(2):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    res = {"n_gpus": 1, "ms_per_step": ms, "value": shape.attn_flops() / (ms * 1e-3) / 1e12, "unit": UNIT,
           "steps": steps, "launches_per_step": shape.heads // hc}
    check = None
    if compare_to is not None:
        r0, r1 = compare_rows
        diff = 0.0
        for i, (q, k, v, r, gi, out) in enumerate(parts):
            d = (out[:, r0:r1].float() - compare_to[:, :, i * hc:(i + 1) * hc].float()).abs().max()
            diff = max(diff, float(d))
        q, k, v, r, gi, out = parts[0]
        check = _oracle_check(q, k, v, gi, r, out, head=0)
        check["multi_gpu_shard_vs_single_gpu_max_abs"] = diff
        check["ok"] = bool(check["ok"] and diff == 0.0)
    del parts
    torch.cuda.empty_cache()
    return res, check


def _layer_bench(args, shape, world: int, rank: int, dev, steps: int):
    """The Ulysses layer of the multi-GPU configuration (hidden 5120, 40 heads x 128, QKV and output projections,
    RMSNorm on q/k, 3-D RoPE, exchange, token-sparse attention with reused metadata and cached residual, exchange
    back): time per call on N ranks (device time, max over ranks), the same layer on rank 0's GPU alone in the same
    run, and a comparison of the two results.  Returns the ``layer`` record (rank 0) or None."""
    import torch
    import torch.distributed as dist
    from mcsparse_b200 import synth
    from mcsparse_b200.h3.ulysses_layer import UlyssesDiTAttentionLayer, layer_weights
    H, L, D, hidden = shape.heads, shape.seq_len, shape.head_dim, shape.heads * shape.head_dim
    Ls, Hl = L // world, H // world
    chunks = 5 if Hl % 5 == 0 else 1
    w = layer_weights(hidden, H, D, seed=0, device=dev)
    g = torch.Generator(device=dev).manual_seed(1234)
    x_full = torch.randn(L, hidden, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)     # same on every rank
    x = x_full[rank * Ls:(rank + 1) * Ls].contiguous()
    if rank != 0:
        del x_full
    layer = UlyssesDiTAttentionLayer(dist.group.WORLD if world > 1 else None, hidden, H, D, shape.grid, w, dev,
                                     heads_per_chunk=Hl // chunks)
    # metadata of the local heads from the layer's own q and k (anchor-step kernels), once, outside the timed region
    for e in layer.project_and_scatter(x):
        torch.cuda.current_stream().wait_event(e)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    gi = torch.cat([synth.topmass_indices(layer.local_qkv(c)[0], layer.local_qkv(c)[1], shape) for c in range(layer.chunks)], dim=1)
    residual = synth.residual_like(shape, heads=Hl, head_offset=rank * Hl, device=dev)
    layer.set_metadata(gi, residual)
    for _ in range(3):
        out = layer.forward(x)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = layer.forward(x)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    fl = layer.flops(shape.topk)
    # one more forward with timing events around every phase (rank 0's two streams), outside the timed region
    _, spans = layer.traced_forward(x)
    if world > 1:
        dist.barrier()
    rec = {"workload": f"ulysses_layer_hidden{hidden}_H{H}_D{D}_L{L}_topk{shape.topk}", "n_gpus": world, "ms": ms,
           "tflops": fl["total"] / (ms * 1e-3) / 1e12, "gemm_flops": fl["gemm"], "attention_flops": fl["attention"],
           "head_chunks": layer.chunks, "steps": steps,
           "timeline_ms_rank0": [[n, round(a, 3), round(b, 3)] for n, a, b in spans],
           "what": "QKV projection by head chunk (library GEMM) -> RMSNorm + RoPE-3D + peer-store exchange in one kernel per "
                   "chunk under the next chunk's GEMM -> sparse attention, rows stored into the owners' shards -> output projection"}
    if world == 1:
        return rec
    # all ranks' indices to rank 0, which then runs the whole layer alone
    gis = [torch.empty_like(gi) for _ in range(world)] if rank == 0 else None
    dist.gather(gi, gis, dst=0)
    out_multi = out.clone()
    del layer
    torch.cuda.empty_cache()
    single = None
    if rank == 0:
        lay1 = UlyssesDiTAttentionLayer(None, hidden, H, D, shape.grid, w, dev, heads_per_chunk=H // 5 if H % 5 == 0 else 1)
        lay1.set_metadata(torch.cat(gis, dim=1), synth.residual_like(shape, heads=H, device=dev))
        for _ in range(2):
            o1 = lay1.forward(x_full)
        torch.cuda.synchronize()
        e0.record()
        n1 = max(2, min(steps, 3))
        for _ in range(n1):
            o1 = lay1.forward(x_full)
        e1.record()
        torch.cuda.synchronize()
        single = e0.elapsed_time(e1) / n1
        d = (o1[:Ls].float() - out_multi.float()).abs()
        rec.update({"single_gpu_ms": single, "speedup": single / ms, "efficiency": single / ms / world,
                    "check": {"against": "the same layer on one GPU, rows of rank 0", "max_abs": float(d.max()),
                              "mean_rel": float(d.mean() / o1[:Ls].float().abs().mean()),
                              "ok": bool(float(d.mean() / o1[:Ls].float().abs().mean()) < 1e-2)}})
        del lay1
    dist.barrier()
    return rec if rank == 0 else None


def run_ours(args):
    import torch
    import torch.distributed as dist
    from mcsparse_b200 import _lib, synth
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func

    os.environ["MCSPARSE_B200_CHECK"] = "0"   # no per-call synchronisation inside timed regions
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback for the kernels")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _lib.lib()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # one GPU: the bf16 video-DiT shape the headline metric is quoted on; several GPUs: the attention of the
    # Ulysses context-parallel layer (long-video grid, 40 heads), the configuration named for 2/4/8 GPUs
    which = args.shape if args.shape != "auto" else ("c2" if world == 1 else "c5")
    shape = synth.C2 if which == "c2" else synth.C5
    if args.heads:
        # reduced head count: a small case of the same kernel for profiler captures, not a bench line
        import dataclasses
        shape = dataclasses.replace(shape, heads=args.heads, name=shape.name + f"_heads{args.heads}")
    wide = bool(args.head_dim) and args.head_dim not in (64, 128)
    if args.head_dim:
        # another head dimension on the same grid: not a bench line of the headline metric; the sizes other than 64 and
        # 128 run on the kernel that pads rows on their way into shared memory
        import dataclasses
        if world > 1:
            raise RuntimeError("--head-dim is a one-GPU option")
        shape = dataclasses.replace(shape, head_dim=args.head_dim, name=shape.name + f"_D{args.head_dim}")
    H, L, D = shape.heads, shape.seq_len, shape.head_dim
    if H % world or L % world:
        raise RuntimeError(f"heads ({H}) and sequence ({L}) must divide by the number of ranks ({world})")
    Hl = H // world
    # head shard of this rank (what the attention kernel sees after the all-to-all)
    q, k, v = synth.clustered_qkv(shape, heads=Hl, head_offset=rank * Hl, device=dev)
    residual = synth.residual_like(shape, heads=Hl, head_offset=rank * Hl, device=dev)
    # indices as the configuration defines them: 4 sinks + top-(topk-4) tokens by exact fp32 group mass,
    # built once with this package's own anchor-step kernels (group mass + top-k), outside the timed region
    if wide:
        # (the group-mass kernel exists for head dimensions 64 and 128 only)
        gi = synth.random_sorted_indices(1, Hl, shape.n_groups, shape.topk, L, seed=3, device=dev)
    else:
        gi = synth.topmass_indices(q, k, shape)
    torch.cuda.synchronize()
    out = torch.empty_like(q)

    if world > 1:
        from mcsparse_b200.h3.context_parallel import UlyssesFusedAttention, UlyssesSparseAttention
        Ls = L // world
        # sequence shards of the very tensors the indices were built from
        q_s, k_s, v_s = _sequence_shards(shape, rank, world, dev)
        if args.ulysses == "fused":
            # peer-store scatter in front, attention epilogue storing into the owners' sequence shards
            dma_from = {"sm": None, "mixed": 1, "dma": 0}[args.scatter]
            ul = UlyssesFusedAttention(dist.group.WORLD, L, H, D, torch.bfloat16, dev, chunks=args.chunks, dma_from_chunk=dma_from)

            def attn(qh, kh, vh, h0, h1, out_peers):
                flash_attn_gather_kv_func(qh, kh, vh, gi[:, h0:h1], residual=residual[:, h0:h1], out_peers=out_peers)
            # one attention kernel per head chunk + three scatter kernels per chunk that is not moved by the copy engines
            launches_per_step = ul.chunks + 3 * (ul.chunks if dma_from is None else min(dma_from, ul.chunks))
        else:
            # library all-to-alls around the attention (comparison arm)
            ul = UlyssesSparseAttention(dist.group.WORLD, L, H, D, torch.bfloat16, dev, chunks=args.chunks)
            o_chunks = [torch.empty(1, L, ul.hc, D, device=dev, dtype=torch.bfloat16) for _ in range(ul.chunks)]

            def attn(qh, kh, vh, h0, h1):
                o = o_chunks[h0 // ul.hc]
                flash_attn_gather_kv_func(qh, kh, vh, gi[:, h0:h1], out=o, residual=residual[:, h0:h1])
                return o
            launches_per_step = ul.chunks

        def eager_step():
            return ul.forward(q_s, k_s, v_s, attn)

        if args.ulysses == "fused" and args.graph:
            graph, _ = ul.capture(q_s, k_s, v_s, attn)

            def step():
                graph.replay()
        else:
            step = eager_step
    else:
        def step():
            flash_attn_gather_kv_func(q, k, v, gi, out=out, residual=residual)
            return out
        launches_per_step = 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    _lib.check_status(dev, "bench warm-up")

    # ---- correctness of what is being timed, outside the timed region
    check, single = None, None
    if world == 1:
        if not args.no_check:
            check = _oracle_check(q, k, v, gi, residual, out, head=0)
    else:
        shard_out = eager_step().clone()          # this rank's (1, L/N, H, D) output shard of one full step
        barrier()
        # the same workload (all heads) on rank 0's GPU alone: the single-GPU time of this very shape measured in the
        # same run, and the reference the multi-GPU result is compared with (same kernels, same inputs: bit-equal)
        if rank == 0 and not args.no_single:
            single, check = _single_gpu_same_workload(shape, dev, flash_attn_gather_kv_func, compare_rows=(0, Ls),
                                                      compare_to=None if args.no_check else shard_out)
        del shard_out
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    # the attention kernel reports the cycles and nanoseconds of its own tile loop (first CTA): the SM clock
    # under the timed load itself
    import ctypes
    kclk = torch.zeros(3, dtype=torch.int64, device=dev)
    _lib.lib().mcs_set_clock_buffer(ctypes.c_void_p(kclk.data_ptr()))
    # ---- device-resident timing: whole region + per-launch kernel time on the launching stream
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    # SM clock right behind the timed region (the GPU is still under that load's power state): one CTA
    # counting SM cycles against the nanosecond timer; nvidia-smi's poll cannot resolve a region of a
    # few milliseconds
    probe = torch.zeros(2, dtype=torch.int64, device=dev)
    _lib.lib().mcs_sm_clock_probe(ctypes.c_void_p(probe.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    per = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        pc, pn = int(probe[0]), int(probe[1])
        clocks["sm_mhz_probe_after_timed_region"] = round(pc * 1000.0 / pn, 1) if pn > 0 else None
        kc, kn = int(kclk[0]), int(kclk[1])
        clocks["sm_mhz_in_kernel_last_timed_launch"] = round(kc * 1000.0 / kn, 1) if kn > 0 else None
    _lib.lib().mcs_set_clock_buffer(None)
    _lib.check_status(dev, "bench timed region")

    # ---- the floor under the kernel that is not the tensor pipe: the launch's K/V row gather alone (same grid, item walk
    # and copy routine as the attention kernel's producer warps, nothing else running), timed the same way
    gather_ms = None
    if world == 1 and not wide:
        from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute.interface import gather_rate_probe
        for _ in range(3):
            gather_rate_probe(q, k, v, gi)
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            gather_rate_probe(q, k, v, gi)
        g1.record()
        torch.cuda.synchronize()
        gather_ms = g0.elapsed_time(g1) / 5

    # ---- end to end through the public entry point with host buffers
    e2e_steps = max(2, min(args.steps, 10))
    if world == 1:
        # Host tensors in (B, H, L, D) storage (the entry point takes them as strided (B, L, H, D) views), so that
        # a head chunk is one contiguous block.  Three streams: inbound copies of chunk c+1, the kernel on chunk c
        # and the outbound copy of chunk c-1 overlap, one async copy per chunk and tensor; PCIe runs both
        # directions at once and the step is bounded by the inbound bytes.
        hcn = args.e2e_chunk if H % args.e2e_chunk == 0 else H
        hq, hk, hv = (t.permute(0, 2, 1, 3).contiguous().cpu().pin_memory() for t in (q, k, v))
        hout = torch.empty(1, H, L, D, dtype=out.dtype).pin_memory()
        dq, dk, dv, do = (torch.empty(1, H, L, D, dtype=q.dtype, device=dev) for _ in range(4))
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        n_ch = H // hcn
        e2e_launches = n_ch

        prev = {"k": None, "o": None}      # the previous step's per-chunk events: kernel done, outbound copy done

        def e2e_step():
            # Steps follow each other as a stream of requests would: the inbound copy of chunk c of the next step may start
            # as soon as this step's kernel on chunk c has read its inputs, and a kernel may overwrite its output chunk as
            # soon as the previous step's outbound copy of that chunk is done.  Every step still moves all of its inputs
            # in and all of its output out.
            main = torch.cuda.current_stream()
            ev_in = [torch.cuda.Event() for _ in range(n_ch)]
            ev_k = [torch.cuda.Event() for _ in range(n_ch)]
            ev_o = [torch.cuda.Event() for _ in range(n_ch)]
            if prev["k"] is None:
                start = torch.cuda.Event()
                start.record(main)
                s_in.wait_event(start)
                s_out.wait_event(start)
            with torch.cuda.stream(s_in):
                for c in range(n_ch):
                    sl = slice(c * hcn, (c + 1) * hcn)
                    if prev["k"] is not None:
                        s_in.wait_event(prev["k"][c])
                    dq[:, sl].copy_(hq[:, sl], non_blocking=True)
                    dk[:, sl].copy_(hk[:, sl], non_blocking=True)
                    dv[:, sl].copy_(hv[:, sl], non_blocking=True)
                    ev_in[c].record(s_in)
            for c in range(n_ch):
                sl = slice(c * hcn, (c + 1) * hcn)
                main.wait_event(ev_in[c])
                if prev["o"] is not None:
                    main.wait_event(prev["o"][c])
                flash_attn_gather_kv_func(dq[:, sl].transpose(1, 2), dk[:, sl].transpose(1, 2), dv[:, sl].transpose(1, 2),
                                          gi[:, sl], out=do[:, sl].transpose(1, 2), residual=residual[:, sl])
                ev_k[c].record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_k[c])
                    hout[:, sl].copy_(do[:, sl], non_blocking=True)
                    ev_o[c].record(s_out)
            prev["k"], prev["o"] = ev_k, ev_o

        def e2e_drain():
            # the timed region ends when the last outbound copy has landed
            if prev["o"] is not None:
                torch.cuda.current_stream().wait_event(prev["o"][-1])
        h2d = 3 * q.numel() * q.element_size()
        d2h = out.numel() * out.element_size()
        e2e_desc = (f"pinned host q,k,v in / out, {n_ch} head chunks of {hcn}; inbound copies, kernels and outbound copies on three "
                    "streams, consecutive steps overlap chunk by chunk")
    else:
        # host sequence shard -> device -> scatter to the peers -> attention -> rows stored into the owners' shards
        # -> host: the exchange in both directions is inside the step
        hq, hk, hv = (t.cpu().pin_memory() for t in (q_s, k_s, v_s))
        hout = torch.empty(1, Ls, H, D, dtype=torch.bfloat16).pin_memory()
        e2e_launches = launches_per_step
        # Two sets of device input shards and two copy streams: the inbound copy of step i+1 runs while step i computes
        # and while the output shard of step i-1 goes back (the two directions of the host link run at once); every
        # step still moves all of its inputs in and its output out.
        sets = [(q_s, k_s, v_s), tuple(torch.empty_like(t) for t in (q_s, k_s, v_s))]
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        st = {"i": 0, "computed": [None, None], "out_done": None}

        def e2e_step():
            main = torch.cuda.current_stream()
            i = st["i"]
            cur = sets[i & 1]
            ev_in = torch.cuda.Event()
            with torch.cuda.stream(s_in):
                if st["computed"][i & 1] is not None:
                    s_in.wait_event(st["computed"][i & 1])     # the step that last read this set has finished
                else:
                    s_in.wait_stream(main)
                for d, h in zip(cur, (hq, hk, hv)):
                    d.copy_(h, non_blocking=True)
                ev_in.record(s_in)
            main.wait_event(ev_in)
            if st["out_done"] is not None:
                main.wait_event(st["out_done"])                # the output shard is overwritten by this step
            o = ul.forward(*cur, attn)
            ev_c = torch.cuda.Event()
            ev_c.record(main)
            st["computed"][i & 1] = ev_c
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c)
                hout.copy_(o, non_blocking=True)
                ev_o = torch.cuda.Event()
                ev_o.record(s_out)
            st["out_done"] = ev_o
            st["i"] = i + 1

        def e2e_drain():
            if st["out_done"] is not None:
                torch.cuda.current_stream().wait_event(st["out_done"])
        h2d = 3 * q_s.numel() * q_s.element_size()
        d2h = hout.numel() * hout.element_size()
        e2e_desc = ("pinned host sequence shards in, Ulysses step (exchange both ways inside), output shard to pinned host; inbound "
                    "copy of the next step and outbound copy of the previous one overlap the step")

    e2e_step()
    e2e_drain()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_drain()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    e2e_check = None
    if world == 1 and not args.no_check:
        # the bytes that came back to the host are the bytes of the device-resident call
        e2e_check = bool(torch.equal(hout.permute(0, 2, 1, 3), out.cpu()))

    t = torch.tensor([total_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(t[0]), float(t[1])
    layer_rec = None
    if (world > 1 or args.layer) and not args.no_layer and which == "c5" and not args.heads:
        # free what the attention-core measurement held, then measure the whole layer
        if world > 1:
            del ul, q_s, k_s, v_s, sets
        del hq, hk, hv, hout
        torch.cuda.empty_cache()
        layer_rec = _layer_bench(args, shape, world, rank, dev, steps=max(3, min(args.steps, 10)))
    ms_per_step = total_ms / args.steps
    flops = shape.attn_flops()                      # whole job (all heads, all ranks)
    value = flops / (ms_per_step * 1e-3) / 1e12
    e2e_value = flops / (e2e_ms * 1e-3) / 1e12

    rc = 0
    if rank == 0:
        peaks = _peaks()
        kern_ms = statistics.mean(per) if world == 1 else None
        # dominant kernel: the attention kernel; algorithmic FLOPs per launch = this rank's heads
        achieved = shape.attn_flops(Hl) / ((kern_ms if kern_ms else ms_per_step) * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops"],
                    # DRAM bytes per launch from an ncu capture of a 4-head launch of this kernel and workload
                    # (dram__bytes_read.sum + dram__bytes_write.sum), scaled by heads: traffic grows with the heads
                    "traffic": (0 if args.head_dim else NCU_DRAM_BYTES_PER_HEAD.get(which, 0)) * Hl or None,
                    "traffic_source": "ncu, 4-head capture scaled by heads (profiles/)",
                    "algorithmic_bytes_per_launch": 5 * q.numel() * 2 + gi.numel() * 4,
                    "peak_source": peaks["source"] + " cuBLAS bf16 burst",
                    "kernel": f"gather_attn_wide_kernel<{(D + 63) // 64},bf16>" if wide else f"gather_attn_kernel<{D},bf16>",
                    "algorithmic_flops_per_launch": shape.attn_flops(Hl)}
        if gather_ms is not None and kern_ms:
            gbytes = 2.0 * gi.numel() * D * q.element_size()       # every selected K row and V row once per query group
            roofline["l2_gather"] = {
                "what": "second bound of the same kernel: every query group pulls its selected K/V rows out of L2 into shared "
                        "memory; gather_only = the launch's row gather alone (mcs_gather_rate_probe), same grid and copy routine",
                "bytes_per_launch": gbytes, "gather_only_ms": gather_ms, "gather_only_gbs": gbytes / gather_ms / 1e6,
                "in_kernel_gbs": gbytes / kern_ms / 1e6, "frac": gather_ms / kern_ms}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": _config(shape, world, args, _input_bytes_per_gpu(shape, world),
                              indices=f"4 sinks + {shape.topk - 4} random tokens, ascending" if wide else ""),
            "clocks": clocks, "gpu_launches": launches_per_step * args.steps,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps, "gpu_launches_per_step": e2e_launches, "how": e2e_desc},
            "roofline": roofline,
        }
        if e2e_check is not None:
            line["e2e"]["host_output_equals_device_output"] = e2e_check
        if check is not None:
            line["check"] = check
            if not check["ok"] or e2e_check is False:
                rc = 3
        if layer_rec is not None:
            line["layer"] = layer_rec
            if "check" in layer_rec and not layer_rec["check"]["ok"]:
                rc = 3
        if single is not None:
            line["single_gpu_same_workload"] = single
            sp = single["ms_per_step"] / ms_per_step
            line["scaling_same_workload"] = {"workload": shape.name, "single_ms": single["ms_per_step"], "multi_ms": ms_per_step,
                                             "speedup": sp, "efficiency": sp / world,
                                             "note": "the one-GPU line of this bench is quoted on another workload; this is "
                                                     "the same workload on one GPU of this box, measured in this run"}
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            cv, heads_done, secs = _cpu_oracle_sample(shape, args.cpu_budget, threads)
            line["cpu_baseline"] = {"value": cv, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"{heads_done} of {H} heads, all {shape.n_groups} groups each, {secs:.1f} s, torch fp32"}
        print(json.dumps(line))
        if rc:
            print("bench.py: the result check failed (see \"check\" in the line above)", file=sys.stderr)
    if world > 1:
        # Leave without running destructors: symmetric-memory handles, a captured graph that contains
        # collectives and the communicators have no defined teardown order between them, and a rank that
        # blocks in one of them keeps the launcher (and the box) waiting after the result is out.
        sys.stdout.flush()
        sys.stderr.flush()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(rc)
    if rc:
        sys.exit(rc)


def run_anchor(args):
    """Secondary measurement: the anchor-step (metadata build) kernels at the same shape, each timed alone
    with CUDA events on resident inputs: dense attention + LSE, group mass, top-k selection, Fast PDDP,
    permutation apply/invert."""
    import math
    import torch
    from mcsparse_b200 import _lib, synth
    from mcsparse_b200.kernels.flash_mcsa.pca_group import apply_perm, invert_perm, pca_group_perm, pddp_start_vectors
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import dense_attention_with_lse, group_mass, select_topk_with_sinks
    os.environ["MCSPARSE_B200_CHECK"] = "0"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shape = synth.C2
    if args.head_dim:
        # the same grid at another head dimension (those other than 64 / 128 run on the padded-layout kernels)
        import dataclasses
        shape = dataclasses.replace(shape, head_dim=args.head_dim, name=shape.name + f"_D{args.head_dim}")
    H = args.heads or shape.heads
    L, D = shape.seq_len, shape.head_dim
    q, k, _ = synth.clustered_qkv(shape, heads=H, device=dev)
    qh, kh = q.transpose(1, 2), k.transpose(1, 2)
    scale = 1.0 / math.sqrt(D)
    # dense pass (q, k, k): the library's own attention kernel in dense mode, strided views, one launch
    _, lse = dense_attention_with_lse(qh, kh, kh, scale)

    def timeit(fn):
        for _ in range(max(1, args.warmup)):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b in ev:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in ev)

    peaks = _peaks()
    mass = torch.empty(1, H, shape.n_groups, L, dtype=torch.float32, device=dev)
    gi = torch.empty(1, H, shape.n_groups, shape.topk, dtype=torch.int32, device=dev)
    x = q[0].transpose(0, 1)
    sv = pddp_start_vectors(H, L, 128, D, 0).to(dev)
    t_dense = timeit(lambda: dense_attention_with_lse(qh, kh, kh, scale))
    t_mass = timeit(lambda: group_mass(qh, kh, lse, out=mass))
    t_topk = timeit(lambda: select_topk_with_sinks(mass, shape.topk, [(0, 4)], out=gi))
    t_pddp = timeit(lambda: pca_group_perm(x, C=128, pow_iters=8, start_vectors=sv))
    perm = pca_group_perm(x, C=128, pow_iters=8, start_vectors=sv)
    xc = x.contiguous()
    t_app = timeit(lambda: apply_perm(xc, perm))
    t_inv = timeit(lambda: invert_perm(xc, perm))
    _lib.check_status(dev, "anchor bench")
    levels = 8
    rows = {
        "dense_attn_lse": {"ms": t_dense, "tflops": 4.0 * L * L * D * H / t_dense / 1e9, "bound": "tensor",
                           "frac": 4.0 * L * L * D * H / t_dense / 1e9 / peaks["bf16_tflops"]},
        "group_mass": {"ms": t_mass, "tflops": 2.0 * L * L * D * H / t_mass / 1e9, "gexp_per_s": L * L * H / t_mass / 1e6,
                       "bound": "sfu ex2 (16/clk/SM) and tensor"},
        "topk_select": {"ms": t_topk, "gbs": (mass.numel() * 4 + gi.numel() * 4) / t_topk / 1e6, "bound": "hbm",
                        "frac": (mass.numel() * 4 + gi.numel() * 4) / t_topk / 1e6 / peaks["hbm_gbs"]},
        "pddp_perm": {"ms": t_pddp, "gbs": levels * 2 * x.numel() * 2 / t_pddp / 1e6, "bound": "hbm",
                      "frac": levels * 2 * x.numel() * 2 / t_pddp / 1e6 / peaks["hbm_gbs"]},
        "perm_apply": {"ms": t_app, "gbs": 2 * xc.numel() * 2 / t_app / 1e6, "frac": 2 * xc.numel() * 2 / t_app / 1e6 / peaks["hbm_gbs"]},
        "perm_invert": {"ms": t_inv, "gbs": 2 * xc.numel() * 2 / t_inv / 1e6, "frac": 2 * xc.numel() * 2 / t_inv / 1e6 / peaks["hbm_gbs"]},
    }
    total = t_mass + t_topk + t_pddp          # metadata build; the dense pass is listed separately
    print(json.dumps({"metric": "anchor_metadata_build_ms", "value": total, "unit": "ms", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(1, args.warmup), "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": f"anchor_L{L}_H{H}_D{D}_topk{shape.topk}_pddp8"}, "kernels": rows,
                      "peak_source": peaks["source"]}))


def _fp8_dense_peak(dev, n: int = 8192, reps: int = 10, sustain_s: float = 2.0):
    """Dense e4m3 GEMM rate of this GPU through the library (torch._scaled_mm, n^3, fp32 scales, bf16 out): best of
    ``reps`` single launches (burst) and back-to-back launches for ``sustain_s`` seconds (sustained).  The
    denominator of the FP8 roofline; measured live because no stored figure exists for this pool."""
    import torch
    a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()            # column-major second operand
    one = torch.ones((), device=dev)
    f = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    for _ in range(3):
        f()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        f()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    flops = 2.0 * n ** 3
    # sustained: as many launches as fit the time budget by the burst rate
    iters = max(10, int(sustain_s * 1e3 / best))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        f()
    e1.record()
    torch.cuda.synchronize()
    sus = e0.elapsed_time(e1) / iters
    return {"fp8_tflops": flops / best / 1e9, "fp8_tflops_sustained": flops / sus / 1e9,
            "how": f"torch._scaled_mm e4m3 {n}^3, bf16 out: best of {reps} (burst), {iters} launches back to back (sustained)"}


def run_fp8(args):
    """The FP8 (e4m3) variant of the attention kernel at the long-video shape (H=40, L=98,280, 768 groups x top-k
    4096, per-head scales amax/448, bf16 residual and output): device-resident timing, roofline against a
    dense e4m3 GEMM rate measured in the same run, result check on one head, CPU baseline, end-to-end step."""
    import math
    import torch
    from mcsparse_b200 import _lib, synth
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_fp8_func
    os.environ["MCSPARSE_B200_CHECK"] = "0"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shape = synth.C3
    if args.heads:
        import dataclasses
        shape = dataclasses.replace(shape, heads=args.heads, name=shape.name + f"_heads{args.heads}")
    wide = bool(args.head_dim) and args.head_dim != 128
    if args.head_dim:
        import dataclasses
        shape = dataclasses.replace(shape, head_dim=args.head_dim, name=shape.name + f"_D{args.head_dim}")
    H, L, D = shape.heads, shape.seq_len, shape.head_dim
    M = shape.n_groups
    # clustered bf16 tensors -> top-mass indices (bf16 anchor-step kernels) -> per-head e4m3 quantisation
    hc = 8 if H % 8 == 0 else H
    q8 = torch.empty(1, L, H, D, dtype=torch.float8_e4m3fn, device=dev)
    k8, v8 = torch.empty_like(q8), torch.empty_like(q8)
    sq, sk, sv = (torch.empty(1, H, dtype=torch.float32, device=dev) for _ in range(3))
    gi = torch.empty(1, H, M, shape.topk, dtype=torch.int32, device=dev)
    for h0 in range(0, H, hc):
        q, k, v = synth.clustered_qkv(shape, heads=hc, head_offset=h0, device=dev)
        if wide:     # (the group-mass kernel exists for head dimensions 64 and 128 only)
            gi[:, h0:h0 + hc] = synth.random_sorted_indices(1, hc, M, shape.topk, L, seed=3 + h0, device=dev)
        else:
            gi[:, h0:h0 + hc] = synth.topmass_indices(q, k, shape)
        for dst, sc, t in ((q8, sq, q), (k8, sk, k), (v8, sv, v)):
            t8, s_ = synth.quantize_e4m3_per_head(t)
            dst[:, :, h0:h0 + hc] = t8
            sc[:, h0:h0 + hc] = s_
        del q, k, v
    scale_qk = (sq * sk * (D ** -0.5) * math.log2(math.e)).view(1, H, 1).expand(1, H, M).contiguous().float()
    residual = synth.residual_like(shape, heads=H, device=dev)
    out = torch.empty(1, L, H, D, device=dev, dtype=torch.bfloat16)
    step = lambda: flash_attn_gather_kv_fp8_func(q8, k8, v8, gi, scale_qk, sv, out=out, residual=residual)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    _lib.check_status(dev, "fp8 warm-up")
    check = None if args.no_check else _oracle_check(q8, k8, v8, gi, residual, out, head=0, fp8=(scale_qk, sv))
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.2)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    _lib.check_status(dev, "fp8 timed region")
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * L * shape.topk * D * H
    # end to end: e4m3 q, k, v from pinned host memory, bf16 output back to the host, every step
    hq, hk, hv = (t.view(torch.uint8).cpu().pin_memory() for t in (q8, k8, v8))
    hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    dq, dk, dv = (torch.empty_like(q8) for _ in range(3))

    def e2e_step():
        dq.view(torch.uint8).copy_(hq, non_blocking=True)
        dk.view(torch.uint8).copy_(hk, non_blocking=True)
        dv.view(torch.uint8).copy_(hv, non_blocking=True)
        flash_attn_gather_kv_fp8_func(dq, dk, dv, gi, scale_qk, sv, out=out, residual=residual)
        hout.copy_(out, non_blocking=True)
    e2e_step()
    torch.cuda.synchronize()
    n_e2e = max(2, min(args.steps, 3))
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    peak = _fp8_dense_peak(dev, sustain_s=0.2 if args.heads else 2.0)      # (a head subset is a profiling run: keep it short)
    bf16 = _peaks()
    achieved = flops / (ms * 1e-3) / 1e12
    line = {
        "metric": "gather_kv_sparse_attn_fp8_effective_tflops", "value": achieved, "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "e4m3", "data": "synthetic",
        "config": {"workload": shape.name, "B": 1, "H": H, "L": L, "D": D, "groups": M, "topk": shape.topk,
                   "residual": "fused",
                   "indices": (f"4 sinks + {shape.topk - 4} random tokens, ascending" if wide else
                               f"4 sinks + top-{shape.topk - 4} by exact fp32 group mass (bf16 anchor pass), ascending"),
                   "quantisation": "per head, scale = amax / 448",
                   "l2": f"inputs ({(3 * q8.numel() + 2 * out.numel() * 2 + gi.numel() * 4) / 1e9:.2f} GB per call) larger than L2; no explicit flush"},
        "clocks": clocks, "gpu_launches": args.steps,
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 3 * q8.numel(), "d2h_bytes_per_step": out.numel() * 2},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak["fp8_tflops"], "unit": "TFLOP/s",
                     "frac": achieved / peak["fp8_tflops"], "frac_of_sustained": achieved / peak["fp8_tflops_sustained"],
                     "frac_of_2x_bf16_burst": achieved / (2 * bf16["bf16_tflops"]), "traffic": None,
                     "peak_source": "measured in this run: " + peak["how"], "peak_sustained": peak["fp8_tflops_sustained"],
                     "kernel": f"gather_attn_wide_kernel<{(D + 127) // 128},e4m3>" if wide else "gather_attn_kernel<128,e4m3>",
                     "algorithmic_flops_per_launch": flops,
                     "algorithmic_bytes_per_launch": 3 * q8.numel() + 2 * out.numel() * 2 + gi.numel() * 4},
    }
    if check is not None:
        line["check"] = check
    if not args.no_cpu_baseline:
        from oracle.gather_attn import gather_attn_fp8_ref
        threads = os.cpu_count() or 1
        torch.set_num_threads(threads)
        c = lambda t: t.cpu()
        a = (c(q8[:, :, :1]), c(k8[:, :, :1]), c(v8[:, :, :1]), c(gi[:, :1]), c(scale_qk[:, :1]), c(sv[:, :1]))
        r = c(residual[:, :1])
        t0 = time.perf_counter()
        n = 0
        while n == 0 or time.perf_counter() - t0 < args.cpu_budget:
            gather_attn_fp8_ref(*a, residual=r)
            n += 1
        secs = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 4.0 * L * shape.topk * D * n / secs / 1e12, "unit": "TFLOP/s", "cores": threads,
                                "kind": "port", "sample": f"head 0 of {H}, all {M} groups, {n} passes, {secs:.1f} s, torch fp32 on dequantised inputs"}
    print(json.dumps(line))
    if check is not None and not check["ok"]:
        sys.exit(3)


def run_layer(args):
    """Secondary measurement on one GPU: the whole Ulysses DiT attention layer of the multi-GPU configuration
    (``--heads N`` shrinks heads and hidden size together: the small case used for profiler captures)."""
    import dataclasses
    import torch
    from mcsparse_b200 import _lib, synth
    os.environ["MCSPARSE_B200_CHECK"] = "0"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shape = synth.C5
    if args.heads:
        shape = dataclasses.replace(shape, heads=args.heads, name=shape.name + f"_heads{args.heads}")
    rec = _layer_bench(args, shape, 1, 0, dev, steps=max(2, args.steps))
    _lib.check_status(dev, "layer bench")
    print(json.dumps({"metric": "ulysses_layer_ms", "value": rec["ms"], "unit": "ms", "n_gpus": 1, "steps": rec["steps"],
                      "warmup": 3, "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": rec["workload"]}, "layer": rec}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU oracle work for cpu_baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--chunks", type=int, default=2,
                    help="head chunks of the Ulysses pipeline (N > 1); lowered to a divisor of the local head count")
    ap.add_argument("--graph", action="store_true", help="N > 1, fused: replay one captured CUDA graph per step instead of launching eagerly")
    ap.add_argument("--ulysses", default="fused", choices=["fused", "nccl"],
                    help="N > 1: peer-store reshard fused with the attention kernel, or library all-to-alls around it")
    ap.add_argument("--scatter", default="mixed", choices=["sm", "mixed", "dma"],
                    help="N > 1, fused: reshard by the scatter kernel, by the copy engines, or (mixed) kernel for the first "
                         "head chunk and copy engines for the chunks that move under an attention kernel")
    ap.add_argument("--shape", default="auto", choices=["auto", "c2", "c5"],
                    help="attn workload: c2 = L=32,760 H=24 top-k 2048 (default on one GPU); c5 = attention of the Ulysses "
                         "layer, L=98,280 H=40 top-k 4096 in bf16 (default on several GPUs)")
    ap.add_argument("--no-single", action="store_true", help="N > 1: skip rank 0's single-GPU run of the same workload")
    ap.add_argument("--heads", type=int, default=0, help="profiling aid: run a head subset of the workload")
    ap.add_argument("--layer", action="store_true", help="one GPU with --shape c5: also time the whole Ulysses layer")
    ap.add_argument("--no-layer", action="store_true", help="N > 1: skip the measurement of the whole layer")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of the result with the CPU oracle / the single-GPU run")
    ap.add_argument("--head-dim", type=int, default=0,
                    help="one GPU: the same grid with another head dimension (a multiple of 8 up to 256); random sorted indices "
                         "when it is not 64 or 128")
    ap.add_argument("--e2e-chunk", type=int, default=8, help="heads per chunk of the pipelined end-to-end step (one GPU)")
    ap.add_argument("--workload", default="attn", choices=["attn", "anchor", "attn_fp8", "layer"],
                    help="attn: the headline reuse-step attention; anchor: times the anchor-step kernels (1 GPU); "
                         "attn_fp8: the e4m3 variant at the long-video shape (1 GPU); layer: the whole Ulysses DiT attention layer (1 GPU)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "anchor":
        run_anchor(args)
    elif args.workload == "attn_fp8":
        run_fp8(args)
    elif args.workload == "layer":
        run_layer(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the fused PE-attention forward on B200.

Workload: the combined FoPE+PoPE causal attention forward of the benchmark
configuration list -- bf16, batch 2, 16 heads, sequence 16384, content dim 128, position
dim 64 (d_qk = 256), value dim 128; Q, K, V ~ N(0, 1) seeded, key phase bias ~ U(-pi, pi),
16 Fourier terms (sigma 0.3), floor 2 pi / 16384.  Heads are sharded over the N GPUs of one
box (16 / N heads each, both batch items), no collective on the data path.

A step is one forward over the whole workload.  ``value`` is algorithmic TFLOP/s,
B H S^2 (d_qk + d_v) per step (3.2985 TFLOP), over the slowest rank's device time with the
inputs resident in HBM; ``e2e`` is the same through ``pe_attention`` with pinned host
buffers, host-to-device copies of all five inputs and a device-to-host copy of the output
inside the timed region.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
  python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

``--impl reference`` times the reference's eager data flow on the host cores (the reference's
own modules when oracle/_ref holds them, else the CPU port under oracle/), on a bounded slice
of the same workload: always one (batch, head) slice at the full sequence length.

The default line also carries compact summaries of the secondary workloads (every variant's
forward beside the reference's live GPU data flow -- ATen positional ops + SDPA -- on the same
GPU, one decode step, one training step) and a ``parity`` figure against the CPU oracle.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

B, H, S, D_C, D_R, D_V = 2, 16, 16384, 128, 64, 128
N_FOURIER, SIGMA = 16, 0.3
FLOPS_PER_STEP = float(B) * H * S * S * (D_C + 2 * D_R + D_V)
METRIC = "fused PE-attention TFLOP/s (FoPE+PoPE causal forward, bf16, B2 H16 S16384 d_qk256 d_v128)"
WORKLOAD = "config 4: FoPE+PoPE causal attention forward, bf16, B2 H16 S16384 d_c128 d_r64 d_v128"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of pe_attn_tc2_kernel on this
# workload (ncu --set full capture of the CTA-pair kernel: 546.7 MB read + 121.0 MB written)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 667_700_000
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        return FALLBACK_BF16_TFLOPS, "fallback (1.59 PFLOP/s)"


def measured_sustained_peak():
    """cuBLAS bf16 throughput of a seconds-long loop under the power cap, or None."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the idle samples before and after the kernels would drag the median down
        busy = [x for x in sm if x >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def bench_config(world: int) -> dict:
    """The ``config`` object of the JSON line; both arms print the same one."""
    return {"workload": WORKLOAD, "parallelism": f"heads sharded over {world} GPU(s), {H // world} heads each",
            "l2": "flushed between steps by writing a 256 MiB buffer",
            "flops_per_step": FLOPS_PER_STEP, "flops_convention": "B*H*S^2*(d_qk+d_v), causal"}


def bind_host_memory_near_gpu(torch, local_rank: int) -> dict:
    """Best effort: run this process on the CPUs of the GPU's NUMA node before its pinned buffers
    are allocated and first touched, so that host<->device copies do not cross the socket link.
    Only affinity is used (no memory-policy call); a failure leaves everything as it was."""
    info = {"gpu_numa_node": None, "bound": False}
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        info["gpu_numa_node"] = node
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["bound"], info["cpus"] = True, len(allowed)
    except Exception as e:   # no sysfs entry, no permission, a cpuset without local CPUs ...
        info["note"] = f"{type(e).__name__}"
    return info


def make_inputs(torch, heads: int, seed: int, pinned: bool):
    """Seeded N(0,1) inputs for ``heads`` heads of the workload, on the host (bf16)."""
    g = torch.Generator().manual_seed(seed)

    def mk(d):
        t = torch.randn(B, S, heads, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
        return t.pin_memory() if pinned else t

    host = dict(q=mk(D_C), k=mk(D_C), q_r=mk(D_R), k_r=mk(D_R), v=mk(D_V))
    gp = torch.Generator().manual_seed(12345)  # positional parameters are replicated, not sharded
    params = dict(
        delta=(torch.rand(D_R, generator=gp) * 2 - 1) * math.pi,
        fourier_coeffs=torch.randn(D_R, N_FOURIER, generator=gp) * SIGMA,
        freqs=10000.0 ** (-(torch.arange(0, D_R, dtype=torch.float32) / D_R)),
        floor_freq=2 * math.pi / S,
    )
    return host, params


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    import pe_ablations_b200 as P
    from pe_ablations_b200 import _lib  # noqa: F401  fails loudly here if the CUDA library is missing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if H % world != 0:
        raise SystemExit(f"{H} heads do not shard over {world} GPUs")
    heads = H // world
    numa = bind_host_memory_near_gpu(torch, local_rank)

    host, params = make_inputs(torch, heads, seed=1000 + rank, pinned=True)
    dparams = {k: (v.to(dev) if hasattr(v, "to") else v) for k, v in params.items()}
    dten = {k: v.to(dev) for k, v in host.items()}
    out = torch.empty(B, S, heads, D_V, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB of L2

    def step(t):
        P.pe_attention("pope", t["q"], t["k"], t["v"], q_r=t["q_r"], k_r=t["k_r"], out=out, **dparams)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing -------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step(dten)
    barrier()
    P.check_device_status()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for e0, e1 in ev:
        flush.zero_()          # evict the previous step's tensors from L2
        e0.record()
        step(dten)
        e1.record()
    barrier()
    P.check_device_status()
    step_ms = [e0.elapsed_time(e1) for e0, e1 in ev]
    local_ms = sum(step_ms)
    total_ms = max_over_ranks(local_ms)
    # keep the GPU busy a little longer so that nvidia-smi gets samples under load
    t_end = time.time() + 1.0
    while time.time() < t_end:
        step(dten)
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = total_ms / args.steps
    value = FLOPS_PER_STEP / (ms_per_step * 1e-3) / 1e12
    kernel_ms = statistics.mean(step_ms)            # one kernel launch per step on this rank
    kernel_tflops = (FLOPS_PER_STEP / world) / (kernel_ms * 1e-3) / 1e12

    # ---- end-to-end: host buffers in, host buffer out -----------------------------------
    # the library's host-buffer call: sequence blocks are copied in, attended and copied
    # back on three streams, so the step costs about what its host->device bytes cost
    in_bytes = sum(v.numel() * v.element_size() for v in host.values())
    # at least four row blocks per rank at every N, so that copy-in, kernels and copy-out
    # overlap; eight where a rank holds enough for 32 MiB blocks
    chunks = args.e2e_chunks or (8 if in_bytes >= (256 << 20) else 4)
    streamed = P.HostStreamedAttention("pope", B=B, S=S, H=heads, Hkv=heads, d_c=D_C, d_r=D_R, d_v=D_V,
                                       dtype=torch.bfloat16, device=dev, chunks=chunks, **dparams)
    out_host = torch.empty(B, S, heads, D_V, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        streamed(host, out_host)

    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = min(args.steps, 10)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    streamed.synchronize()      # raises if a kernel reported an expired wait
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_host.numel() * out_host.element_size()

    peak, peak_src = measured_peak()
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": bench_config(world),
        "e2e": {"value": round(FLOPS_PER_STEP / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "ms_per_step": round(e2e_ms, 3), "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                "chunks": chunks, "host_gbs_per_gpu": round((h2d + d2h) / (e2e_ms * 1e-3) / 1e9, 1),
                "host_numa": numa,
                "call": "HostStreamedAttention (copy-in / attend / copy-out pipelined over sequence blocks)"},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "pe_attn_tc2_kernel<128,64,POPE> (CTA pair, cta_group::2)",
                     "achieved": round(kernel_tflops, 2), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(kernel_tflops / peak, 4), "peak_source": peak_src,
                     "frac_of_nominal_2250": round(kernel_tflops / 2250.0, 4),
                     # context only: what cuBLAS sustains under the same 1 kW cap (the kernel, too,
                     # runs power-capped for the whole timed region)
                     "frac_of_sustained_cublas": (round(kernel_tflops / measured_sustained_peak(), 4)
                                                  if measured_sustained_peak() else None),
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH // world,   # compulsory-traffic kernel: scales with the heads per rank
                     "launch_ms": round(kernel_ms, 4),
                     # CTA pairs of 512 query rows per launch over the GPU's pair slots (1 CTA/SM)
                     "waves": round(B * heads * (S // 512) / (torch.cuda.get_device_properties(dev).multi_processor_count // 2), 2)},
    }
    if not args.no_eval:
        ev_line = run_eval(torch, dist, dev, rank, world, args.eval_sequences, not args.eval_graph)
        if ev_line is not None:
            line["eval_1b_16k"] = ev_line
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(budget_s=20.0)
        line["parity"] = parity_vs_oracle(torch, dten, dparams, out)
    if rank == 0 and world == 1 and not args.no_secondary:
        del dten, out, streamed
        torch.cuda.empty_cache()
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = min(args.steps, 10), 3
        v = run_variants(sub)
        line["variants"] = {"peak": v["peak"], "rows": v["variants"], "gpu_eager": v["gpu_eager"]}
        d = run_decode(sub)
        line["decode"] = {"workload": d["config"]["workload"], "tokens_per_s": d["value"], "ms_per_step": d["ms_per_step"],
                          "roofline": d["roofline"], "query_tiled_kernel": d["query_tiled_kernel"],
                          "other_variants": d["other_variants"]}
        t = run_training(sub)
        line["training"] = {"workload": t["config"]["workload"], "tflops": t["value"], "ms_per_step": t["ms_per_step"],
                            "backward_kernel": t["backward_kernel"]}
        line["fused_gemms"] = run_gemm(sub)["rows"]
    if world > 1:
        dist.destroy_process_group()
    return line if rank == 0 else None


def run_eval(torch, dist, dev, rank: int, world: int, n_sequences: int, no_graph: bool = True):
    """Second headline: 1B-shape forward + perplexity, 16k context, sequences sharded over ranks.

    Random-init bf16 weights (seeded), ``n_sequences`` x 16384 uniform-random token ids; each
    rank runs its shard through the fused attention and the loss-sum kernel, one NCCL
    all-reduce of (sum NLL, count).  Timed once over the whole evaluation after one warm-up
    sequence, device time, max over ranks.
    """
    from pe_ablations_b200 import eval as E

    seq = E.MODEL_1B["max_seq_len"]
    model = E.build_1b_model(dev, seed=0)
    g = torch.Generator().manual_seed(4242)
    ids = torch.randint(0, E.MODEL_1B["vocab_size"], (n_sequences, seq), generator=g)
    mine = E.shard_range(n_sequences, world, rank)
    my_ids = ids[mine.start:mine.stop].to(dev)
    # warm-up (cuBLAS heuristics, allocator) and capture of one sequence's forward into a CUDA graph
    graphed = None if no_graph else E.GraphedLossSums(model, my_ids[:1])
    E.evaluate_shard(model, my_ids[:1], graphed=graphed)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    nll, cnt = E.evaluate_shard(model, my_ids, graphed=graphed)
    tot_nll, tot_cnt = E.reduce_loss_sums(nll, cnt)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    del model
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {"metric": "1B-shape forward+perplexity tokens/s at 16k context", "value": round(n_sequences * seq / (ms * 1e-3), 1),
            "unit": "tokens/s", "sequences": n_sequences, "seq_len": seq, "ms_total": round(ms, 2),
            "perplexity": round(E.perplexity(tot_nll, tot_cnt), 3), "scaling": "strong",
            "parallelism": f"sequences sharded over {world} GPU(s); one all-reduce of 2 scalars",
            "launch": "eager" if no_graph else "one CUDA graph per sequence",
            "flops_per_token": 3.52e9}


def cpu_baseline(budget_s: float) -> dict:
    """The reference's eager data flow on the host cores, on a bounded slice of the workload:
    one of the 32 (batch, head) slices at the full sequence length."""
    from oracle.cpu_baseline import time_cfg4_sample

    r = time_cfg4_sample(S, 1)
    return {"value": round(r["flops"] / r["seconds"] / 1e12, 5), "unit": "TFLOP/s", "cores": r["threads"],
            "kind": r["kind"], "seconds": round(r["seconds"], 3),
            "sample": f"1 of the {B * H} (batch, head) slices at sequence {S} (eager fp32 transform + bf16 SDPA on CPU)"}


def parity_vs_oracle(torch, dten, dparams, out) -> dict:
    """Max abs error of the timed launch's output against the CPU oracle on rows that the oracle
    can afford: the first and the last 512 query rows (the last ones against all 16384 keys) of
    four (batch, head) slices.  Runs outside every timed region; the oracle is only the checker."""
    from oracle import pe_attention_oracle as O

    tol, rows = 2e-2, 512
    eff = O.fope_effective_freqs(dparams["freqs"].cpu(), dparams["fourier_coeffs"].cpu(), training_length=S)
    delta = dparams["delta"].cpu()
    heads = dten["q"].shape[2]
    worst = {"prefix": 0.0, "tail": 0.0}
    for b, h in ((0, 0), (0, heads - 1), (1, 0), (1, heads - 1)):
        f = lambda name, lo, hi: dten[name][b:b + 1, lo:hi, h:h + 1].float().cpu()
        for part, (q0, k1) in (("prefix", (0, rows)), ("tail", (S - rows, S))):
            want = O.attention_core("pope", f("q", q0, q0 + rows), f("k", 0, k1), f("v", 0, k1), dtype=torch.bfloat16,
                                    q_r=f("q_r", q0, q0 + rows), k_r=f("k_r", 0, k1), freqs=eff, delta=delta,
                                    pos0=q0, k_pos0=0)
            got = out[b:b + 1, q0:q0 + rows, h:h + 1].float().cpu()
            worst[part] = max(worst[part], (got - want.float()).abs().max().item())
    err = max(worst.values())
    return {"max_abs_err": round(err, 6), "max_abs_err_prefix": round(worst["prefix"], 6),
            "max_abs_err_tail": round(worst["tail"], 6), "tolerance": tol, "ok": bool(err <= tol),
            "rows": f"query rows 0..{rows - 1} and {S - rows}..{S - 1} of 4 (batch, head) slices vs the CPU oracle"}


def run_reference(args) -> dict | None:
    """The reference arm: always one (batch, head) slice of the workload at the FULL sequence
    length per step.  A host too slow for ``--steps`` such passes in a few minutes runs fewer
    passes (and says so), never a shorter sequence."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    from oracle.cpu_baseline import time_cfg4_sample

    budget_s = 200.0
    first = time_cfg4_sample(S, 1)
    fit = max(1, int(budget_s / max(first["seconds"], 1e-3)))
    warm = max(0, min(args.warmup - 1, fit // 4))
    steps = max(1, min(args.steps, fit - warm))
    for _ in range(warm):
        time_cfg4_sample(S, 1)
    t = [time_cfg4_sample(S, 1) for _ in range(steps)]
    sec = sum(x["seconds"] for x in t) / len(t)
    val = t[0]["flops"] / sec / 1e12
    kind = t[0]["kind"]
    sample = (f"per step: 1 of the {B * H} (batch, head) slices at sequence {S}, the reference's eager data flow on CPU "
              f"({'its own modules from oracle/_ref' if kind == 'reference' else 'CPU port of it'})")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(val, 5), "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm + 1, "ms_per_step": round(sec * 1e3, 2), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": bench_config(max(1, args.gpus)),
        "cpu_baseline": {"value": round(val, 5), "unit": "TFLOP/s", "cores": t[0]["threads"], "kind": kind,
                         "sample": sample},
        "e2e": {"value": round(val, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if steps != args.steps or warm + 1 != args.warmup:
        line["steps_requested"], line["warmup_requested"] = args.steps, args.warmup
    return line


def run_training(args) -> dict:
    """Secondary workload (``--workload training``): one forward + backward of the fused
    attention op at the reference's training shape (configs/fpope.yaml: 8 heads, 4 KV heads,
    head_dim 64, d_rope 32, sequence 512; bf16 autocast precision), through the same autograd
    path ``loss.backward()`` takes, and the backward kernel alone on prepared operands."""
    import torch

    import pe_ablations_b200 as P
    from pe_ablations_b200.ops import attention_backward

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Bt, Ht, Hkv, St, dc, dr, dv = args.train_batch, 8, 4, args.train_seq, 64, 32, 64
    d_qk = dc + 2 * dr
    g = torch.Generator().manual_seed(7)
    mk = lambda h, d: torch.randn(Bt, St, h, d, generator=g).to(torch.bfloat16).to(dev).requires_grad_(True)
    q, k, q_r, k_r, v = mk(Ht, dc), mk(Hkv, dc), mk(Ht, dr), mk(Hkv, dr), mk(Hkv, dv)
    freqs = (10000.0 ** (-(torch.arange(0, dr, dtype=torch.float32) / dr))).to(dev)
    coeffs = (torch.randn(dr, 64, generator=g) * 0.4).to(dev).requires_grad_(True)
    delta = (-torch.rand(dr, generator=g) * 3).to(dev).requires_grad_(True)
    dout = torch.randn(Bt, St, Ht, dv, generator=g).to(torch.bfloat16).to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    leaves = (q, k, q_r, k_r, v, coeffs, delta)

    def step():
        # gradients start out absent, as after optimizer.zero_grad(): in a model these tensors are
        # projection outputs, nothing accumulates into them from one step to the next
        for t in leaves:
            t.grad = None
        out = P.pe_attention("pope", q, k, v, q_r=q_r, k_r=k_r, freqs=freqs, fourier_coeffs=coeffs, delta=delta,
                             floor_freq=2 * math.pi / 512)
        out.backward(dout)

    def timed(fn, n):
        for _ in range(max(args.warmup, 3)):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for e0, e1 in ev:
            flush.zero_()
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        return statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)

    step_ms = timed(step, args.steps)
    # the backward kernel alone, on operands prepared once
    from pe_ablations_b200.autograd import transformed_operands

    with torch.no_grad():
        lse = torch.empty(Bt, Ht, St, dtype=torch.float32, device=dev)
        o = P.pe_attention("pope", q, k, v, q_r=q_r, k_r=k_r, freqs=freqs, fourier_coeffs=coeffs, delta=delta,
                           floor_freq=2 * math.pi / 512, lse=lse)
        opts = dict(start_pos=0, k_start_pos=0, normalize_coeffs=True, floor_freq=2 * math.pi / 512, ceil_freq=None)
        qt, kt = (t.to(torch.bfloat16) for t in transformed_operands("pope", q, k, q_r, k_r, opts, freqs, delta, coeffs))
        vv = v.detach()
    bwd_ms = timed(lambda: attention_backward(qt, kt, vv, o, dout, lse, scale=d_qk ** -0.5), args.steps)
    P.check_device_status()
    fwd_flops = Bt * Ht * St * St * (d_qk + dv)
    bwd_flops = Bt * Ht * St * St * (3 * d_qk + 2 * dv)
    peak, peak_src = measured_peak()
    return {
        "metric": "fused PE-attention forward+backward TFLOP/s (FoPE+PoPE, bf16, reference training shape)",
        "value": round((fwd_flops + bwd_flops) / (step_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(step_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"training step of the attention op: B{Bt} H{Ht} Hkv{Hkv} S{St} d_c{dc} d_r{dr} d_v{dv}, "
                               "fused forward + autograd transform + tensor-core backward",
                   "l2": "flushed between steps by writing a 256 MiB buffer",
                   "flops_convention": "B*H*S^2*(d_qk+d_v) forward + B*H*S^2*(3 d_qk + 2 d_v) backward, causal"},
        "backward_kernel": {"ms": round(bwd_ms, 4), "tflops": round(bwd_flops / (bwd_ms * 1e-3) / 1e12, 2),
                            "frac_of_peak": round(bwd_flops / (bwd_ms * 1e-3) / 1e12 / peak, 4), "peak": peak,
                            "peak_source": peak_src, "launches_per_step": 2},
    }


def measured_hbm_peak():
    """Measured copy bandwidth in GB/s, or the fallback figure."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s)"


def run_decode(args) -> dict:
    """Secondary workload (``--workload decode``): one generated token of the 1B shape's attention
    (16 heads, d_c 128 / d_r 64 / d_v 128, FoPE+PoPE, bf16) against a cache of ``--decode-cache``
    keys, batch ``--decode-batch``: the split-KV kernel and, beside it, the query-tiled kernel
    on the same call.  HBM-bound: the algorithmic bytes are the raw cached K halves and V, read
    once (B * Hkv * Sk * (d_c + d_r + d_v) * 2)."""
    import torch

    import pe_ablations_b200 as P
    from pe_ablations_b200 import pe as PE

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Bd, Hd, Sk = args.decode_batch, H, args.decode_cache
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator().manual_seed(11)
    mk = lambda Sv, d: torch.randn(Bd, Sv, Hd, d, generator=g).to(torch.bfloat16).to(dev)
    q, q_r = mk(1, D_C), mk(1, D_R)
    k, k_r, v = mk(Sk, D_C), mk(Sk, D_R), mk(Sk, D_V)
    fp4 = PE.FoPEPoPEEmbedding(dim=D_R, max_seq_len=Sk, num_fourier_terms=N_FOURIER, fourier_sigma=SIGMA,
                               training_length=Sk, delta_init="uniform").to(dev)
    kw = dict(q_r=q_r, k_r=k_r, start_pos=Sk - 1, k_start_pos=0, **fp4.kernel_args())

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for e0, e1 in ev:
            flush.zero_()
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        return statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)

    with torch.no_grad():
        split_ms = timed(lambda: P.pe_attention("pope", q, k, v, split_kv=True, **kw))
        tiled_ms = timed(lambda: P.pe_attention("pope", q, k, v, split_kv=False, **kw))
        a = P.pe_attention("pope", q, k, v, split_kv=True, **kw)
        b = P.pe_attention("pope", q, k, v, split_kv=False, **kw)
    torch.cuda.synchronize()
    P.check_device_status()
    nbytes = Bd * Hd * Sk * (D_C + D_R + D_V) * 2
    peak, peak_src = measured_hbm_peak()

    # the other variants' decode steps (one token, same cache length), split-KV kernel only
    others = []

    def other(name, variant, Hq, Hk, d_c, d_r, d_v, **okw):
        mk2 = lambda Sv, h, d: None if d == 0 else torch.randn(Bd, Sv, h, d, generator=g).to(torch.bfloat16).to(dev)
        oq, ok_, ov = mk2(1, Hq, d_c), mk2(Sk, Hk, d_c), mk2(Sk, Hk, d_v)
        oqr, okr = mk2(1, Hq, d_r), mk2(Sk, Hk, d_r)
        with torch.no_grad():
            ms = timed(lambda: P.pe_attention(variant, oq, ok_, ov, q_r=oqr, k_r=okr, start_pos=Sk - 1, k_start_pos=0,
                                              split_kv=True, **okw))
        nb = Bd * Hk * Sk * (d_c + d_r + d_v) * 2
        others.append({"variant": name, "shape": f"B{Bd} H{Hq} Hkv{Hk} Sk{Sk} d_c{d_c} d_r{d_r} d_v{d_v}",
                       "ms": round(ms, 4), "GB/s": round(nb / (ms * 1e-3) / 1e9, 1),
                       "frac": round(nb / (ms * 1e-3) / 1e9 / peak, 4)})

    rope = PE.RotaryEmbedding(64, Sk, 10000.0).to(dev)
    other("rope, head_dim 64", "rotary", 12, 12, 64, 0, 64, rotary_table=rope.freqs_cis, table_geometric=True)
    other("rope + QKNorm, head_dim 64", "rotary", 12, 12, 64, 0, 64, rotary_table=rope.freqs_cis, table_geometric=True,
          qk_norm=True)
    other("rope, head_dim 64, every table row read", "rotary", 12, 12, 64, 0, 64, rotary_table=rope.freqs_cis)
    other("nope, head_dim 128", "nope", 16, 16, 128, 0, 128)
    other("alibi, head_dim 128, 4:1 GQA", "alibi", 16, 4, 128, 0, 128, alibi_slopes=PE.alibi_slopes(16).to(dev))
    fp2 = PE.FoPEPoPEEmbedding(dim=32, max_seq_len=Sk, num_fourier_terms=64, fourier_sigma=0.4, training_length=512,
                               delta_init="uniform").to(dev)
    other("fope+pope, head_dim 64 / d_rope 32, 2:1 GQA", "pope", 8, 4, 64, 32, 64, **fp2.kernel_args())
    P.check_device_status()
    gbs = nbytes / (split_ms * 1e-3) / 1e9
    return {
        "metric": "cached-decode attention tokens/s (FoPE+PoPE, bf16, one new token per sequence)",
        "value": round(Bd / (split_ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(split_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"decode step of one attention layer: B{Bd} H{Hd} Sq1 Sk{Sk} d_c{D_C} d_r{D_R} d_v{D_V}",
                   "l2": "flushed between steps by writing a 256 MiB buffer"},
        "roofline": {"bound": "hbm", "kernel": "pe_attn_decode_kernel<128,64,128,POPE,1> + decode_merge_kernel",
                     "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                     "peak_source": peak_src, "algorithmic_bytes": nbytes, "traffic": None},
        "query_tiled_kernel": {"ms": round(tiled_ms, 4), "speedup_of_split_kv": round(tiled_ms / split_ms, 2)},
        "max_abs_diff_between_kernels": round((a.float() - b.float()).abs().max().item(), 5),
        "other_variants": others,
        "gpu_launches": 2 * args.steps,
    }


def run_gemm(args) -> dict:
    """Secondary workload (``--workload gemm``): the two fused GEMMs of the 1B-shape evaluation,
    16 384 tokens, against the library GEMM + stand-alone kernel they replace, and the plain-store
    form of the same kernel against the library GEMM.  One GPU, CUDA events, L2 flushed."""
    import torch

    import pe_ablations_b200 as P
    from pe_ablations_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peak, peak_src = measured_peak()
    g = torch.Generator().manual_seed(0)
    M, K, FFN, V = 16384, 2048, 5632, 32000
    mk = lambda r, c, s: (torch.randn(r, c, generator=g) * s).to(torch.bfloat16).to(dev)
    x, wg, wu, wv = mk(M, K, 1.0), mk(FFN, K, 0.02), mk(FFN, K, 0.02), mk(V, K, 0.02)
    tgt = torch.randint(0, V, (M,), generator=g).to(dev)
    sums = torch.zeros(2, dtype=torch.float64, device=dev)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for e0, e1 in ev:
            flush.zero_()
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        return statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)

    def library_head():
        for i in range(0, M, 8192):
            ops.ce_loss_sums(x[i:i + 8192] @ wv.T, tgt[i:i + 8192], out=sums)

    rows = []
    with torch.no_grad():
        for name, flops, fused, library, what in (
                ("lm head + cross-entropy", 2.0 * M * V * K, lambda: ops.lm_head_ce_loss_sums(x, wv, tgt, out=sums),
                 library_head, "library GEMM (8192-token chunks) + pe_ce_loss_sums"),
                ("w3 | w1 projections + SwiGLU", 4.0 * M * FFN * K, lambda: ops.swiglu_gemm(x, wg, wu),
                 lambda: ops.swiglu(x @ wg.T, x @ wu.T), "two library GEMMs + pe_swiglu_forward"),
                ("plain store, N = 2048", 2.0 * M * 2048 * K, lambda: ops.gemm_nt(x, wv[:2048]),
                 lambda: x @ wv[:2048].T, "library GEMM")):
            ms, ms_lib = timed(fused), timed(library)
            tf = flops / (ms * 1e-3) / 1e12
            rows.append({"op": name, "shape": f"M{M} K{K}", "ms": round(ms, 4), "tflops": round(tf, 1),
                         "frac_of_peak": round(tf / peak, 4), "replaces": what, "replaced_ms": round(ms_lib, 4),
                         "speedup": round(ms_lib / ms, 3)})
    P.check_device_status()
    trace = None
    from pe_ablations_b200 import _lib

    if hasattr(_lib.lib, "pe_gemm_trace_read"):
        # a library built with -DPE_GEMM_TRACE: clocks per CTA each role spent waiting / issuing
        import ctypes

        import numpy as np

        buf = np.zeros(148 * 16, dtype=np.int64)
        _lib.lib.pe_gemm_trace_read(buf.ctypes.data_as(ctypes.c_void_p), 1)
        with torch.no_grad():
            ops.gemm_nt(x, wv)
        _lib.lib.pe_gemm_trace_read(buf.ctypes.data_as(ctypes.c_void_p), 1)
        t = buf.reshape(148, 16)
        names = ("producer_total", "producer_wait_free_stage", "producer_issue", "mma_total", "mma_wait_full_stage",
                 "mma_wait_free_accumulator", "epilogue_total", "epilogue_wait_full_accumulator")
        trace = {"launch": f"plain store, M{M} N{V} K{K}",
                 "leader_ctas": {n: int(t[0::2, i].mean()) for i, n in enumerate(names)},
                 "peer_ctas": {n: int(t[1::2, i].mean()) for i, n in enumerate(names)}}
    return {"metric": "fused GEMMs of the 1B-shape evaluation (16 384 tokens)", "trace_clocks": trace, "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "dtype": "bf16", "data": "synthetic",
            "peak": {"tflops": peak, "source": peak_src}, "rows": rows,
            "config": {"workload": "pe_gemm_pair_kernel: head + cross-entropy, SwiGLU feed-forward input, plain store",
                       "l2": "flushed between steps by writing a 256 MiB buffer"}}


def run_variants(args) -> dict:
    """Secondary workload (``--workload variants``): the fused forward of every positional-encoding
    variant at the configuration the benchmark list gives it (configurations 1-4; NoPE and ALiBi
    at configuration 2's shape), one GPU, CUDA events, L2 flushed between launches."""
    import torch

    import pe_ablations_b200 as P
    from pe_ablations_b200 import pe as PE

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peak, peak_src = measured_peak()
    g = torch.Generator().manual_seed(0)

    def tensors(Bv, Sv, Hv, dims, dtype):
        return [None if d == 0 else torch.randn(Bv, Sv, Hv, d, generator=g).to(dtype).to(dev) for d in dims]

    def timed(fn, steps=None, warmup=None):
        for _ in range(max(args.warmup, 3) if warmup is None else warmup):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(steps or args.steps)]
        for e0, e1 in ev:
            flush.zero_()
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        return statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)

    rows = []

    def add(name, Bv, Hv, Sv, d_c, d_r, d_v, dtype, variant, eager=None, **kw):
        q, k, v, q_r, k_r = tensors(Bv, Sv, Hv, (d_c, d_c, d_v, d_r, d_r), dtype)
        call = lambda: P.pe_attention(variant, q, k, v, q_r=q_r, k_r=k_r, **kw)
        with torch.no_grad():
            ms = timed(call)
        flops = Bv * Hv * Sv * Sv * (d_c + 2 * d_r + d_v)
        tf = flops / (ms * 1e-3) / 1e12
        row = {"variant": name, "shape": f"B{Bv} H{Hv} S{Sv} d_qk{d_c + 2 * d_r} d_v{d_v}",
               "dtype": "bf16" if dtype == torch.bfloat16 else "fp32", "ms": round(ms, 4), "tflops": round(tf, 2),
               "frac_of_peak": round(tf / peak, 4) if dtype == torch.bfloat16 else None}
        if eager is not None:
            # the reference's live GPU data flow on the same tensors, same timing protocol
            try:
                with torch.no_grad():
                    ref_out = eager(q, k, v, q_r, k_r)
                    got = call()
                    row["max_abs_diff_vs_gpu_eager"] = round((got.float() - ref_out.float()).abs().max().item(), 5)
                    del ref_out, got
                    ems = timed(lambda: eager(q, k, v, q_r, k_r), steps=min(args.steps, 5), warmup=2)
                row["gpu_eager_ms"] = round(ems, 4)
                row["gpu_eager_tflops"] = round(flops / (ems * 1e-3) / 1e12, 2)
                row["speedup_vs_gpu_eager"] = round(ems / ms, 2)
            except Exception as e:      # e.g. out of memory in the S x S path of the comparator
                row["gpu_eager_unavailable"] = f"{type(e).__name__}: {str(e)[:120]}"
                torch.cuda.empty_cache()
        rows.append(row)

    # ---- the comparator: what the reference itself runs on a GPU (no kernels of this library) ----
    import torch.nn.functional as F

    def eager_rotate(x, cis):
        # src/model/rope.py:35-57: complex multiply of interleaved pairs in fp32, type_as
        xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
        return torch.view_as_real(xc * cis.view(1, x.shape[1], 1, -1)).flatten(3).type_as(x)

    def eager_qknorm(t, eps=1e-6):
        # src/model/normalization.py:44-56
        return t / (t.norm(dim=-1, keepdim=True) + eps)

    def eager_rotary(cis=None, mscale=1.0, qk_norm=False):
        # src/model/attention.py:77-96
        def run(q, k, v, q_r, k_r):
            if cis is not None:
                q, k = eager_rotate(q, cis[: q.shape[1]]), eager_rotate(k, cis[: k.shape[1]])
                if mscale != 1.0:
                    q, k = q * mscale, k * mscale
            q, k, vv = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
            if qk_norm:
                q, k = eager_qknorm(q), eager_qknorm(k)
            return F.scaled_dot_product_attention(q, k, vv, attn_mask=None, is_causal=True,
                                                  scale=1.0 / (q.shape[-1] ** 0.5)).transpose(1, 2)
        return run

    def eager_alibi(slopes, qk_norm=True):
        # src/model/alibi.py:86-109,137-160: S x S bias and scores in memory, explicit softmax
        def run(q, k, v, q_r, k_r):
            q, k, vv = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
            if qk_norm:
                q, k = eager_qknorm(q), eager_qknorm(k)
            Sv = q.shape[2]
            pos = torch.arange(Sv, device=q.device)
            rel = (pos.unsqueeze(0) - pos.unsqueeze(1)).abs().float()
            bias = -slopes.view(1, -1, 1, 1) * rel.view(1, 1, Sv, Sv)
            scores = torch.matmul(q, k.transpose(-2, -1)) * (q.shape[-1] ** -0.5) + bias.to(q.dtype)
            mask = torch.triu(torch.ones(Sv, Sv, dtype=torch.bool, device=q.device), diagonal=1)
            scores = scores.masked_fill(mask, float("-inf"))
            return torch.matmul(torch.softmax(scores, dim=-1), vv).transpose(1, 2)
        return run

    def eager_pope(freqs, delta):
        # src/model/fpope.py:266-338 + src/model/fpope_attention.py:145-177 under bf16 autocast:
        # fp32 transform, cat with the content halves, operands cast to bf16 for SDPA
        def run(q, k, v, q_r, k_r):
            Sv = q_r.shape[1]
            pos = torch.arange(Sv, dtype=torch.float32, device=q_r.device)
            ph_q = (pos[:, None] * freqs[None, :]).view(1, Sv, 1, -1)
            ph_k = (pos[:, None] * freqs[None, :] + delta.clamp(-2 * math.pi, 0.0)[None, :]).view(1, Sv, 1, -1)
            mu_q, mu_k = F.softplus(q_r.float()), F.softplus(k_r.float())
            qr = torch.cat([mu_q * ph_q.cos(), mu_q * ph_q.sin()], dim=-1).transpose(1, 2)
            kr = torch.cat([mu_k * ph_k.cos(), mu_k * ph_k.sin()], dim=-1).transpose(1, 2)
            dt = v.dtype
            qq = torch.cat([q.transpose(1, 2), qr], dim=-1).to(dt)
            kk = torch.cat([k.transpose(1, 2), kr], dim=-1).to(dt)
            return F.scaled_dot_product_attention(qq, kk, v.transpose(1, 2), attn_mask=None, dropout_p=0.0,
                                                  is_causal=True, scale=qq.shape[-1] ** -0.5).transpose(1, 2)
        return run

    bf, f32 = torch.bfloat16, torch.float32
    with torch.no_grad():
        # configuration 1: PoPE, fp32 (FFMA kernel: no tensor-core roofline applies)
        pope = PE.PoPEEmbedding(dim=32, max_seq_len=512).to(dev)
        pope.phase_bias.uniform_(-math.pi, math.pi)
        add("pope (configuration 1)", 1, 8, 512, 64, 32, 64, f32, "pope", scale=128 ** -0.5,
            eager=eager_pope(pope.effective_freqs.float(), pope.phase_bias.float()), **pope.kernel_args())
        # configuration 2: RoPE / NTK (scale 4) / YaRN (scale 4), plus NoPE and ALiBi at the same shape
        for name, rope in (("rope (configuration 2)", PE.RotaryEmbedding(64, 2048, 10000.0)),
                           ("rope-ntk (configuration 2)", PE.NTKAwareRotaryEmbedding(64, 2048, 10000.0, 4.0)),
                           ("rope-yarn", PE.YaRNRotaryEmbedding(64, 2048, 10000.0, 4.0, original_max_seq_len=512))):
            rope = rope.to(dev)
            ms_ = float(getattr(rope, "mscale", 1.0))
            add(name, 8, 12, 2048, 64, 0, 64, bf, "rotary", rotary_table=rope.freqs_cis, mscale=ms_,
                eager=eager_rotary(rope.freqs_cis, ms_))
        rope = PE.RotaryEmbedding(64, 2048, 10000.0).to(dev)
        add("rope + QKNorm", 8, 12, 2048, 64, 0, 64, bf, "rotary", qk_norm=True, rotary_table=rope.freqs_cis,
            eager=eager_rotary(rope.freqs_cis, qk_norm=True))
        add("nope", 8, 12, 2048, 64, 0, 64, bf, "nope", eager=eager_rotary())
        sl = PE.alibi_slopes(12).to(dev)
        add("alibi + QKNorm", 8, 12, 2048, 64, 0, 64, bf, "alibi", qk_norm=True, alibi_slopes=sl, eager=eager_alibi(sl))
        # the reference's own training shape (configs/*.yaml: 8 heads, 4 K/V heads, head_dim 64, sequence 512)
        rope512 = PE.RotaryEmbedding(64, 512, 10000.0).to(dev)
        add("rope + QKNorm, reference training shape", 64, 8, 512, 64, 0, 64, bf, "rotary", qk_norm=True,
            rotary_table=rope512.freqs_cis, eager=eager_rotary(rope512.freqs_cis, qk_norm=True))
        # configuration 3: FoPE frequencies driving a rotary table, head_dim 128
        fope = PE.FoPEPoPEEmbedding(dim=64, max_seq_len=4096, num_fourier_terms=16, fourier_sigma=0.3,
                                    training_length=4096)
        ang = torch.outer(torch.arange(4096, dtype=torch.float32), fope.effective_freqs().float().cpu())
        cis = torch.polar(torch.ones_like(ang), ang).to(dev)
        add("fope-rotary (configuration 3)", 4, 16, 4096, 128, 0, 128, bf, "rotary", rotary_table=cis,
            eager=eager_rotary(cis))
        # the reference's own attention shape (head_dim 64, d_rope 32) at a long context
        fp = PE.FoPEPoPEEmbedding(dim=32, max_seq_len=4096, num_fourier_terms=64, fourier_sigma=0.4,
                                  training_length=512, delta_init="uniform").to(dev)
        add("fope+pope, head_dim 64 / d_rope 32", 8, 8, 4096, 64, 32, 64, bf, "pope",
            eager=eager_pope(fp.effective_freqs().float(), fp.phase_bias.float()), **fp.kernel_args())
        # configuration 4
        fp4 = PE.FoPEPoPEEmbedding(dim=64, max_seq_len=S, num_fourier_terms=N_FOURIER, fourier_sigma=SIGMA,
                                   training_length=S, delta_init="uniform").to(dev)
        add("fope+pope (configuration 4)", B, H, S, D_C, D_R, D_V, bf, "pope",
            eager=eager_pope(fp4.effective_freqs().float(), fp4.phase_bias.float()), **fp4.kernel_args())
    P.check_device_status()
    return {"metric": "fused PE-attention forward TFLOP/s per variant", "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True, "data": "synthetic",
            "config": {"workload": "every variant at its benchmark configuration, one launch per step",
                       "l2": "flushed between steps by writing a 256 MiB buffer",
                       "flops_convention": "B*H*S^2*(d_qk+d_v), causal"},
            "peak": peak, "peak_source": peak_src, "variants": rows,
            "gpu_eager": "the reference's live GPU data flow on the same tensors and GPU: ATen positional ops "
                         "(fp32 rotation / softplus-cos-sin expansion, QKNorm, cat, transposes) + "
                         "F.scaled_dot_product_attention(is_causal=True), or the explicit S x S scores for ALiBi"}


PROFILE_CASES = {
    # name: (variant, B, H, Hkv, S, d_c, d_r, d_v, qk_norm) -- each a few hundred MB at most, inputs larger than L2
    "pair_fpope": ("pope", 1, 4, 4, 16384, 128, 64, 128, False),      # pe_attn_tc2_kernel, the headline loop
    "pair_fope_rotary": ("rotary", 4, 16, 16, 4096, 128, 0, 128, False),
    "tile4_nope": ("nope", 4, 16, 16, 8192, 64, 0, 64, False),        # pe_attn_tc4_kernel (2 tiles, 2 CTAs/SM)
    "tile4_rope_qknorm": ("rotary", 4, 16, 16, 8192, 64, 0, 64, True),
    "tile4_fpope_gqa": ("pope", 8, 8, 4, 4096, 64, 32, 64, False),
}


def run_profile_case(args) -> dict:
    """``--workload profile --case NAME``: a few launches of one small case, for ``ncu -k ... -c 1``."""
    import torch

    import pe_ablations_b200 as P
    from pe_ablations_b200 import pe as PE

    variant, Bp, Hp, Hkv, Sp, d_c, d_r, d_v, qk_norm = PROFILE_CASES[args.case]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(0)
    mk = lambda h, d: None if d == 0 else torch.randn(Bp, Sp, h, d, generator=g).to(torch.bfloat16).to(dev)
    q, k, v, q_r, k_r = mk(Hp, d_c), mk(Hkv, d_c), mk(Hkv, d_v), mk(Hp, d_r), mk(Hkv, d_r)
    kw = {}
    if variant == "pope":
        kw = PE.FoPEPoPEEmbedding(dim=d_r, max_seq_len=Sp, num_fourier_terms=N_FOURIER, fourier_sigma=SIGMA,
                                  training_length=Sp, delta_init="uniform").to(dev).kernel_args()
    elif variant == "rotary":
        kw = dict(rotary_table=PE.RotaryEmbedding(d_c, Sp, 10000.0).to(dev).freqs_cis)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.no_grad():
        for i in range(3):
            if i == 2:
                ev0.record()
            out = P.pe_attention(variant, q, k, v, q_r=q_r, k_r=k_r, qk_norm=qk_norm, **kw)
        ev1.record()
    torch.cuda.synchronize()
    P.check_device_status()
    ms = ev0.elapsed_time(ev1)
    flops = Bp * Hp * Sp * Sp * (d_c + 2 * d_r + d_v)
    return {"workload": "profile", "case": args.case, "shape": f"B{Bp} H{Hp}/{Hkv} S{Sp} d_qk{d_c + 2 * d_r} d_v{d_v}",
            "ms": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 1), "mean_abs_out": float(out.float().abs().mean())}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-eval", action="store_true", help="skip the 1B-shape 16k perplexity evaluation")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the compact variants / decode / training summaries of the default line (1 GPU)")
    ap.add_argument("--eval-sequences", type=int, default=64)
    ap.add_argument("--eval-graph", action="store_true",
                    help="replay the evaluation forward from a CUDA graph (measured: no gain, the eager path is "
                         "already GPU-bound)")
    ap.add_argument("--e2e-chunks", type=int, default=0,
                    help="sequence blocks of the pipelined host-buffer call (0: about 32 MiB of input per block, 2 to 8)")
    ap.add_argument("--decode-batch", type=int, default=8, help="sequences in the decode workload")
    ap.add_argument("--decode-cache", type=int, default=16384, help="cached keys per sequence in the decode workload")
    ap.add_argument("--case", default="pair_fpope", choices=sorted(PROFILE_CASES),
                    help="--workload profile: which small case to launch (for an ncu capture of one kernel)")
    ap.add_argument("--workload", default="forward", choices=["forward", "training", "variants", "decode", "profile", "gemm"],
                    help="forward: the headline benchmark; training: forward+backward of the attention op (1 GPU); "
                         "variants: the forward of every variant at its benchmark configuration (1 GPU); "
                         "decode: one generated token against a long cache, split-KV kernel (1 GPU); "
                         "gemm: the evaluation's fused GEMMs against the library path they replace (1 GPU)")
    ap.add_argument("--train-batch", type=int, default=64)
    ap.add_argument("--train-seq", type=int, default=512)
    args = ap.parse_args()
    if args.workload == "profile" and args.impl == "ours":
        line = run_profile_case(args)
    elif args.workload == "training" and args.impl == "ours":
        line = run_training(args)
    elif args.workload == "variants" and args.impl == "ours":
        line = run_variants(args)
    elif args.workload == "decode" and args.impl == "ours":
        line = run_decode(args)
    elif args.workload == "gemm" and args.impl == "ours":
        line = run_gemm(args)
    else:
        line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line is not None:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()

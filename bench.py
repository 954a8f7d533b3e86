"""Benchmark of the MoE layer (router -> permute -> grouped expert GEMMs -> combine), forward and
backward, on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward + backward pass of the layer over one batch of synthetic tokens
(x ~ N(0,1), weights ~ N(0,0.02), upstream gradient ~ N(0,1), random-init weights).
N = 1: T=16384, d_model=2048, E=64, d_ff=1408, top-6, bf16 (the headline configuration).
N > 1: one process per GPU (torchrun); see `_workload` for the per-N workload.
Prints ONE JSON line on rank 0.  `value` = tokens/s of the whole job with inputs resident in HBM;
`e2e` = the same through the public nn.Module with host buffers (H2D of x and the upstream
gradient, D2H of the output and grad_x inside the timed region).

`--impl reference` times the reference's eager algorithm (the CPU oracle port) on the host cores
on a bounded token sample of the same configuration.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

PKG = "triton-kernel-fused_b200"
HEADLINE = dict(T=16384, H=2048, E=64, I=1408, k=6)
# small case for profiler captures: weights (277 MB) exceed L2, about 1.5 GB held on the device
PROFILE = dict(T=4096, H=2048, E=16, I=1408, k=6)
# expert-parallel configuration: 65536 global tokens, 256 experts sharded over the ranks
EP5 = dict(T=65536, H=7168, E=256, I=2048, k=8)
# MXFP8 configuration (e4m3 + E8M0 block-32 scales), one GPU
MXFP8 = dict(T=32768, H=4096, E=8, I=14336, k=2)
# small MXFP8 case for profiler captures: expert weights 403 MB (above L2), about 2 GB held on the device
MXFP8_PROFILE = dict(T=8192, H=2048, E=8, I=4096, k=2)
# skewed routing: per-expert selection bias from Zipf(1.1) frequencies, some experts receive no token
ZIPF = dict(T=32768, H=2048, E=128, I=768, k=8)
METRIC = "moe_layer_fwd_bwd_tokens_per_s"
# DRAM bytes (read + written) per launch measured with ncu on the profile workload (24 576 routed rows,
# H=2048, I=1408, 1536 rows per expert; the capture is summarised under profiles/).  Traffic grows in
# proportion to the routed rows when H, I and the rows per expert stay the same (the headline workload).
NCU_TRAFFIC = {"rows": 24576, "H": 2048, "I": 1408, "rows_per_expert": 1536,
               "bytes": {"expert_gate_up_swiglu": 479.2e6, "expert_down": 243.0e6, "expert_down_dgrad_glu": 482.0e6,
                         "expert_gate_up_dgrad": 422.8e6, "expert_wgrad": (394.8e6 + 237.9e6) / 2}}


def _peaks(precision="bf16"):
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        d = dict(hbm_gbs=p["hbm_gbs"], tflops=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                 source="measured (MEASURED_PEAKS.json, sustained bf16)")
    else:
        d = dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback (6.65 TB/s, 1.4 PFLOP/s sustained)")
    if precision == "mxfp8":   # no fp8 measurement exists: the fp8 tensor rate is twice the bf16 rate
        d["tflops"] *= 2.0
        d["source"] = "2 x " + d["source"] + " (fp8 dense rate = 2 x bf16; no fp8 peak was measured)"
    return d


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 4), ("hw_thermal_slowdown", 5), ("sw_thermal_slowdown", 6),
                              ("sw_power_cap", 7)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    samples=len(sm), reasons=sorted(reasons))


def _workload(n_gpus, which="headline"):
    """Per-rank workload.  N=1: the headline layer on one GPU.  N>1: the same layer expert-parallel:
    every rank keeps T tokens (weak scaling in tokens) and owns E/N of the experts; rows travel by NCCL
    all-to-all.  `ep5` is the expert-parallel configuration with 65536 global tokens."""
    if which == "ep5":
        w = dict(EP5)
        w["T"] = EP5["T"] // n_gpus
    elif which in ("mxfp8", "mxfp8_profile"):
        w = dict(MXFP8 if which == "mxfp8" else MXFP8_PROFILE)
    elif which == "zipf":
        w = dict(ZIPF)
    else:
        w = dict(HEADLINE if which == "headline" else PROFILE)
    w["precision"] = "mxfp8" if which.startswith("mxfp8") else "bf16"
    w["name"] = (w["precision"] + " MoE layer T={T}/GPU H={H} E={E} I={I} top{k} fwd+bwd").format(**w)
    w["parallelism"] = "single GPU" if n_gpus == 1 else f"expert parallel ep{n_gpus} (E/{n_gpus} experts per GPU, NCCL all-to-all)"
    return w


def _make_layer(pkg, w, device, seed, world):
    torch.manual_seed(seed)
    with torch.device(device):      # build the (large) expert stacks directly on the GPU
        if world > 1:
            layer = pkg.ExpertParallelMoELayer(w["H"], w["I"], w["E"], top_k=w["k"],
                                               overlap_chunks=int(os.environ.get("B200MOE_EP_CHUNKS", "1")),
                                               reserved_sms=int(os.environ.get("B200MOE_EP_RESERVED_SMS", "12")),
                                               transport=os.environ.get("B200MOE_EP_TRANSPORT", "p2p"),
                                               exchange=os.environ.get("B200MOE_EP_EXCHANGE", "push"))
        else:
            layer = pkg.MoELayer(w["H"], w["I"], w["E"], top_k=w["k"], precision=w["precision"])
    return layer.to(torch.bfloat16)


def run_ours(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    pkg = importlib.import_module(PKG)
    pkg.lib()
    ops = pkg.ops
    w = _workload(world, args.workload)
    T, H, E, I, k = w["T"], w["H"], w["E"], w["I"], w["k"]
    layer = _make_layer(pkg, w, dev, seed=0, world=world)
    params = [layer.gate.weight, layer.gate_up_proj, layer.down_proj]
    if args.workload == "zipf":   # selection bias = 0.15 x log of Zipf(1.1) frequencies over a seeded expert order
        gz = torch.Generator().manual_seed(7)
        ranks = (torch.randperm(E, generator=gz) + 1).float()
        pz = ranks.pow(-1.1)
        layer.bias.copy_((0.15 * torch.log(pz / pz.sum())).to(dev))
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    x_dev = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    go_dev = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    x_host = x_dev.cpu().pin_memory()
    go_host = go_dev.cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    gx_host = torch.empty_like(x_host).pin_memory()

    def step_resident():
        for p in params:
            p.grad = None
        x = x_dev.detach().requires_grad_(True)
        out = layer(x)
        out.backward(go_dev)
        return out, x.grad

    # e2e: every step copies its inputs from pinned host memory and its results back.  The copies run
    # on two copy streams with double-buffered device tensors, so step i+1's H2D and step i-1's D2H
    # overlap step i's kernels (a user's input pipeline does the same); nothing is skipped.
    h2d, d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    in_bufs = [(torch.empty_like(x_dev), torch.empty_like(go_dev)) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    e2e_state = {"i": 0, "primed": False}

    def _upload(slot):
        with torch.cuda.stream(h2d):
            h2d.wait_event(in_free[slot])
            in_bufs[slot][0].copy_(x_host, non_blocking=True)
            in_bufs[slot][1].copy_(go_host, non_blocking=True)
            in_ready[slot].record(h2d)

    def step_e2e():
        cur = torch.cuda.current_stream(dev)
        i = e2e_state["i"]
        slot = i & 1
        if not e2e_state["primed"]:
            for ev in in_free + out_done:
                ev.record(cur)
            _upload(slot)
            e2e_state["primed"] = True
        _upload(slot ^ 1)                      # next step's inputs travel while this step computes
        for p in params:
            p.grad = None
        cur.wait_event(in_ready[slot])
        x = in_bufs[slot][0].detach().requires_grad_(True)
        out = layer(x)
        out.backward(in_bufs[slot][1])
        in_free[slot].record(cur)
        done = torch.cuda.Event()
        done.record(cur)
        with torch.cuda.stream(d2h):
            d2h.wait_event(done)
            out_host.copy_(out.detach(), non_blocking=True)
            gx_host.copy_(x.grad, non_blocking=True)
            out.record_stream(d2h)
            x.grad.record_stream(d2h)
            out_done[slot].record(d2h)
        cur.wait_event(out_done[slot ^ 1])     # at most one result copy in flight behind the compute
        e2e_state["i"] = i + 1

    def drain_e2e():
        torch.cuda.current_stream(dev).wait_stream(d2h)
        torch.cuda.current_stream(dev).wait_stream(h2d)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, after=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if after is not None:
            after()                       # the last copies finish inside the timed region
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    n_warm = args.warmup if args.workload.endswith("profile") else max(args.warmup, 3)
    for _ in range(n_warm):
        step_resident()
    pkg.check_status()

    # ---- timed region 1: inputs resident in HBM; per-op CUDA events on the launching stream
    records = []
    ops.set_hook(lambda name, launches, a, b: records.append((name, launches, a, b)))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_total = timed(step_resident, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ops.set_hook(None)
    pkg.check_status()
    per_op = {}
    launches = 0
    for name, n, a, b in records:
        d = per_op.setdefault(name, [0.0, 0])
        d[0] += a.elapsed_time(b)
        d[1] += 1
        launches += n
    ms_step = ms_total / args.steps

    # ---- timed region 2: through the module with host buffers
    for _ in range(min(2, n_warm)):
        step_e2e()
    ms_e2e = timed(lambda: step_e2e(), args.steps, after=drain_e2e) / args.steps
    pkg.check_status()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peaks = _peaks(w["precision"])
    M = T * k
    flops = {  # algorithmic FLOPs per launch (padding rows not counted)
        "expert_gate_up_swiglu": 2.0 * M * H * 2 * I, "expert_down": 2.0 * M * I * H,
        "expert_down_dgrad_glu": 2.0 * M * H * I, "expert_gate_up_dgrad": 2.0 * M * 2 * I * H,
        "expert_wgrad": (2.0 * M * H * I + 2.0 * M * 2 * I * H) / 2.0,   # two launches per step, averaged
        "mxfp8_expert_gemm": 12.0 * M * H * I / 4.0,                     # four launches per step, averaged
        "mxfp8_expert_wgrad": 6.0 * M * H * I / 2.0,
    }
    kernels = {}
    for name, (ms, n) in sorted(per_op.items(), key=lambda kv: -kv[1][0]):
        avg = ms / n
        entry = dict(launches_per_step=n / args.steps, avg_ms=round(avg, 4), share=round(ms / ms_total, 4))
        if name in flops:
            entry["tflops"] = round(flops[name] / (avg * 1e-3) / 1e12, 1)
        kernels[name] = entry
    gemm_ms = sum(per_op[n][0] for n in flops if n in per_op) / args.steps
    top = max((n for n in flops if n in per_op), key=lambda n: per_op[n][0])
    top_avg_ms = per_op[top][0] / per_op[top][1]
    achieved = flops[top] / (top_avg_ms * 1e-3) / 1e12
    traffic = None
    if (H, I, M // E) == (NCU_TRAFFIC["H"], NCU_TRAFFIC["I"], NCU_TRAFFIC["rows_per_expert"]) and top in NCU_TRAFFIC["bytes"] \
            and w["precision"] == "bf16" and world == 1:
        traffic = round(NCU_TRAFFIC["bytes"][top] * M / NCU_TRAFFIC["rows"])
    layer_flops = 18.0 * H * I * T * k
    line = {
        "metric": METRIC, "value": round(T * world / (ms_step * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": n_warm, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["precision"], "data": "synthetic",
        "config": {"workload": w["name"], "tokens_per_gpu": T, "d_model": H, "experts": E, "d_ff": I, "top_k": k,
                   "parallelism": w["parallelism"],
                   "l2": "no flush: the working set (expert weights + activations, several GB) exceeds the 126 MB L2"},
        "tokens_per_expert": ({"min": int(layer.last_counts.min()), "max": int(layer.last_counts.max()),
                               "experts_without_tokens": int((layer.last_counts == 0).sum())}
                              if getattr(layer, "last_counts", None) is not None else None),
        "layer_tflops_per_gpu": round(layer_flops / (ms_step * 1e-3) / 1e12, 1),
        "layer_frac_of_peak": round(layer_flops / (ms_step * 1e-3) / 1e12 / peaks["tflops"], 4),
        "gemm_ms_per_step": round(gemm_ms, 4),
        "roofline": {"bound": "tensor", "kernel": f"gemm_kernel via {top}", "achieved": round(achieved, 1),
                     "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": round(achieved / peaks["tflops"], 4),
                     "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read+write, scaled from the "
                     "profile workload by routed rows)" if traffic else None, "peak_source": peaks["source"]},
        "kernels": kernels,
        "e2e": {"value": round(T * world / (ms_e2e * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 4),
                "h2d_bytes_per_step": 2 * T * H * 2, "d2h_bytes_per_step": 2 * T * H * 2},
        "gpu_launches": launches,
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(w, steps=1, warmup=0)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_muon(args):
    """--workload muon: one optimizer step (FusedMuon, the reference's default scale mode) over the two expert stacks of
    the headline layer, (E,2I,H) and (E,H,I) in bf16 with bf16 gradients.  Not the headline metric: a line of its own
    for the optimizer row, same timing rules (CUDA events on the launching stream, warm-up, working set above L2)."""
    if int(os.environ.get("WORLD_SIZE", 1)) > 1:
        if int(os.environ.get("RANK", 0)) == 0:
            print(json.dumps({"workload": "muon", "unavailable": "single-GPU workload (stacks are not sharded)"}), flush=True)
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pkg = importlib.import_module(PKG)
    pkg.lib()
    ops = pkg.ops
    H, E, I = HEADLINE["H"], HEADLINE["E"], HEADLINE["I"]
    if args.workload == "muon_profile":     # small case for profiler captures: 8 experts, under 1 GB on the device
        E = 8
    shapes = [(E, 2 * I, H), (E, H, I)]
    g = torch.Generator(device=dev).manual_seed(3)
    params = [torch.nn.Parameter((torch.randn(*sh, device=dev, generator=g) * 0.02).to(torch.bfloat16)) for sh in shapes]
    grads_host = [torch.randn(*sh, generator=torch.Generator().manual_seed(4 + i)).to(torch.bfloat16).pin_memory()
                  for i, sh in enumerate(shapes)]
    grads_dev = [t.to(dev) for t in grads_host]
    params_host = [torch.empty_like(t).pin_memory() for t in grads_host]
    opt = pkg.FusedMuon(params, lr=3e-4, weight_decay=0.1)

    def step_resident():
        for p, gr in zip(params, grads_dev):
            p.grad = gr
        opt.step()

    def step_e2e():
        for p, gh in zip(params, grads_host):
            p.grad = gh.to(dev, non_blocking=True)
        opt.step()
        for p, ph in zip(params, params_host):
            ph.copy_(p.detach(), non_blocking=True)

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    n_warm = args.warmup if args.workload.endswith("profile") else max(args.warmup, 3)
    for _ in range(n_warm):
        step_resident()
    pkg.check_status()
    records = []
    ops.set_hook(lambda name, launches, a, b: records.append((name, launches, a, b)))
    sampler = ClockSampler(0)
    sampler.start()
    ms_total = timed(step_resident, args.steps)
    clocks = sampler.stop()
    ops.set_hook(None)
    pkg.check_status()
    ms_e2e = timed(step_e2e, args.steps) / args.steps
    per_op, launches = {}, 0
    for name, n, a, b in records:
        d = per_op.setdefault(name, [0.0, 0])
        d[0] += a.elapsed_time(b)
        d[1] += 1
        launches += n
    ms_step = ms_total / args.steps
    iters = len(pkg.muon.DSV4_COEFFS)
    # algorithmic FLOPs per matrix and iteration (s = smaller, w = larger dimension; padding not counted).
    # As the reference evaluates it: 2 s^2 w (X X^T) + 2 s^3 (A A) + 2 s^2 w (B X).  X X^T and A A are symmetric and
    # computed over their upper triangle here: s^2 w + s^3 + 2 s^2 w, the count the roofline figure uses.
    flops = flops_ref = 0.0
    for (n, r, c) in shapes:
        s_, w_ = min(r, c), max(r, c)
        flops += n * iters * (3.0 * s_ * s_ * w_ + 1.0 * s_ ** 3)
        flops_ref += n * iters * (4.0 * s_ * s_ * w_ + 2.0 * s_ ** 3)
    gemm_names = [n for n in ("expert_gram", "expert_linear", "expert_linear_axpby", "expert_linear_t") if n in per_op]
    gemm_ms = sum(per_op[n][0] for n in gemm_names) / args.steps
    peaks = _peaks("bf16")
    kernels = {name: dict(launches_per_step=n / args.steps, avg_ms=round(ms / n, 4), share=round(ms / ms_total, 4))
               for name, (ms, n) in sorted(per_op.items(), key=lambda kv: -kv[1][0])}
    achieved = flops / (gemm_ms * 1e-3) / 1e12
    nbytes = sum(2 * n * r * c for n, r, c in shapes)
    line = {
        "metric": "expert_stack_muon_step_ms", "value": round(ms_step, 3), "unit": "ms", "n_gpus": 1, "steps": args.steps,
        "warmup": n_warm, "ms_per_step": round(ms_step, 3), "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"FusedMuon step (aurora, {iters} Newton-Schulz iterations) over expert stacks "
                               f"{shapes[0]} and {shapes[1]}, bf16 parameters and gradients",
                   "l2": "no flush: every stack (0.4-0.7 GB) exceeds the 126 MB L2"},
        "step_tflops": round(flops / (ms_step * 1e-3) / 1e12, 1),
        "step_tflops_reference_count": round(flops_ref / (ms_step * 1e-3) / 1e12, 1),
        "gemm_ms_per_step": round(gemm_ms, 3),
        "roofline": {"bound": "tensor", "kernel": "gemm_kernel via expert_gram / expert_linear_axpby / expert_linear_t (Newton-Schulz products)",
                     "achieved": round(achieved, 1), "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": round(achieved / peaks["tflops"], 4), "traffic": None, "peak_source": peaks["source"]},
        "kernels": kernels,
        "e2e": {"value": round(ms_e2e, 3), "unit": "ms", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes},
        "gpu_launches": launches, "clocks": clocks,
    }
    if not args.no_cpu_baseline:
        from oracle import muon_oracle as MO
        t0 = time.perf_counter()
        for (n, r, c) in shapes:       # one matrix of each stack, fp32, the oracle's step
            p1 = torch.randn(1, r, c) * 0.02
            MO.muon_step(p1, torch.randn(1, r, c), torch.zeros(1, r, c), 3e-4, weight_decay=0.1)
        sec = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": round(sec * 1e3 * E, 1), "unit": "ms", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"1 of {E} matrices of each stack, fp32, oracle/muon_oracle.py muon_step "
                                          f"({round(sec, 2)} s), scaled by {E}; host cpu_count={os.cpu_count()}"}
    print(json.dumps(line), flush=True)


def cpu_baseline(w, steps, warmup, sample_tokens=512):
    """The oracle port (plain PyTorch fp32 on the host cores) on a bounded sample: `sample_tokens`
    tokens through the full-size layer (all E experts, full d_model and d_ff), forward + backward."""
    from oracle import moe_oracle as O
    T, H, E, I, k = sample_tokens, w["H"], w["E"], w["I"], w["k"]
    inp = O.make_inputs(T, H, E, I, k, seed=0)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.layer_fwd_bwd(inp["x"], inp["gate_weight"], None, inp["gate_up"], inp["down"], k, inp["grad_out"])
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return {"value": round(T / sec, 1), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "ms_per_step": round(sec * 1e3, 2),
            "sample": f"{T} of {w['T']} tokens through the full-size layer (E={E}, H={H}, I={I}, top{k}), fp32, "
                      f"oracle/moe_oracle.py layer_fwd_bwd, host cpu_count={os.cpu_count()}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if rank != 0:
        return
    w = _workload(world, args.workload)
    cb = cpu_baseline(w, steps=max(1, min(args.steps, 3)), warmup=min(args.warmup, 1))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tokens/s", "n_gpus": world,
            "steps": max(1, min(args.steps, 3)), "warmup": min(args.warmup, 1), "ms_per_step": cb["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "d_model": w["H"], "experts": w["E"], "d_ff": w["I"], "top_k": w["k"],
                       "parallelism": "host cores, one process"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="headline", choices=["headline", "profile", "ep5", "mxfp8", "mxfp8_profile", "zipf", "muon", "muon_profile"],
                    help="profile = small case for profiler captures (not a benchmark number)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload.startswith("muon"):
        run_muon(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

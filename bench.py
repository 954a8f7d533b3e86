"""Benchmark of the MoE layer (router -> permute -> grouped expert GEMMs -> combine), forward and
backward, on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|torch_grouped]

One step = one forward + backward pass of the layer over one batch of synthetic tokens
(x ~ N(0,1), weights ~ N(0,0.02), upstream gradient ~ N(0,1), random-init weights).
N = 1: T=16384, d_model=2048, E=64, d_ff=1408, top-6, bf16 (the headline configuration).
N > 1: one process per GPU (torchrun); see `_workload` for the per-N workload.
Prints ONE JSON line on rank 0.  `value` = tokens/s of the whole job with inputs resident in HBM;
`e2e` = the same through the public nn.Module with host buffers (H2D of x and the upstream
gradient, D2H of the output and grad_x inside the timed region).

`--impl reference` times the reference's eager algorithm (the CPU oracle port) on the host cores
on a bounded token sample of the same configuration (rank 0, all host threads).
`--impl torch_grouped` times a plain-PyTorch composition of the reference's library path (sort ->
torch._grouped_mm x2 with SiLU-GLU between -> index_add_, autograd backward) on the same GPU: a same-box
library yardstick reported beside the number, not a target and not part of this package.

Beside the headline, the line carries `secondary` (the skewed-routing and the MXFP8 configurations at N = 1,
the 65536-token expert-parallel configuration at N > 1, a few steps each) and, at N > 1, `ep_parity`: one
forward + backward of a small expert-parallel layer checked against the single-GPU layer on the concatenated
batch; the process exits non-zero when that check fails.
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
               "bytes": {"expert_gate_up_swiglu": 482.7e6, "expert_down": 244.4e6, "expert_down_dgrad_glu": 487.1e6,
                         "expert_gate_up_dgrad": 423.9e6, "expert_wgrad": (398.0e6 + 240.6e6) / 2}}


def _peaks(precision="bf16"):
    """Measured denominators (MEASURED_PEAKS.json): the cuBLAS bf16 rate as a burst and sustained under the
    power cap.  Which of the two a measurement is divided by follows the SM clock sampled during it
    (`_pick_peak`)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        d = dict(hbm_gbs=p["hbm_gbs"], burst=p["bf16_tflops"], sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                 source="measured (MEASURED_PEAKS.json)")
    else:
        d = dict(hbm_gbs=6650.0, burst=1590.0, sustained=1400.0, source="fallback (6.65 TB/s, 1.59 / 1.4 PFLOP/s)")
    if precision == "mxfp8":   # no fp8 measurement exists: the fp8 tensor rate is twice the bf16 rate
        d["burst"] *= 2.0
        d["sustained"] *= 2.0
        d["source"] = "2 x " + d["source"] + " (fp8 dense rate = 2 x bf16; no fp8 peak was measured)"
    return d


def _pick_peak(peaks, clocks):
    """Like for like: a timed region whose median SM clock stayed at >= 90 % of the maximum ran in the regime the
    burst figure was taken in; below that (power cap) it is compared with the sustained figure."""
    sm, mx = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
    if sm and mx and sm >= 0.9 * mx:
        return "burst", peaks["burst"]
    if sm and mx:
        return "sustained", peaks["sustained"]
    return "sustained (no clock sample)", peaks["sustained"]


def _fractions(tflops, peaks, clocks):
    rule, peak = _pick_peak(peaks, clocks)
    return dict(frac=round(tflops / peak, 4), peak=peak, rule=rule,
                frac_of_burst=round(tflops / peaks["burst"], 4), frac_of_sustained=round(tflops / peaks["sustained"], 4))


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


def _ep_settings():
    """Transport and exchange of the expert-parallel layer in this run (environment overrides for A/B runs)."""
    return dict(transport=os.environ.get("B200MOE_EP_TRANSPORT", "p2p"), exchange=os.environ.get("B200MOE_EP_EXCHANGE", "push"),
                overlap_chunks=int(os.environ.get("B200MOE_EP_CHUNKS", "1")),
                reserved_sms=int(os.environ.get("B200MOE_EP_RESERVED_SMS", "16")),
                expert_groups=int(os.environ.get("B200MOE_EP_GROUPS", "1")),
                capacity_factor=float(os.environ.get("B200MOE_EP_CAPACITY", "1.5")) or None)


def _parallelism_label(n_gpus):
    if n_gpus == 1:
        return "single GPU"
    ep = _ep_settings()
    if ep["transport"] == "nccl":
        plane = "rows by NCCL all_to_all_single, four payload exchanges per step"
    elif ep["exchange"] == "push":
        plane = ("peer memory over NVLink: token rows pulled by the experts' owners, result rows pushed home by the "
                 "GEMM epilogues; NCCL carries only the count all-gather")
    else:
        plane = "peer memory over NVLink: rows pulled in both directions; NCCL carries only the count all-gather"
    cap = ""
    if ep["transport"] == "p2p" and ep["exchange"] == "push" and ep.get("capacity_factor"):
        cap = (f"; local buffers of a fixed capacity, {ep['capacity_factor']} x a rank's own routed rows, no host wait "
               "(a step that does not fit raises an error, nothing is dropped)")
    return f"expert parallel ep{n_gpus} (E/{n_gpus} experts per GPU; transport={ep['transport']}, exchange={ep['exchange']}: {plane}{cap})"


def _workload(n_gpus, which="headline"):
    """Per-rank workload.  N=1: the headline layer on one GPU.  N>1: the same layer expert-parallel:
    every rank keeps T tokens (weak scaling in tokens) and owns E/N of the experts.  `ep5` is the
    expert-parallel configuration with 65536 global tokens."""
    if which == "ep5":
        w = dict(EP5)
        w["T"] = EP5["T"] // n_gpus
    elif which in ("mxfp8", "mxfp8_profile"):
        w = dict(MXFP8 if which == "mxfp8" else MXFP8_PROFILE)
    elif which == "zipf":
        w = dict(ZIPF)
    elif which == "polyglu":          # the headline layer with experts of activation codes 0 / 1 / 5 in turn
        w = dict(HEADLINE)
    else:
        w = dict(HEADLINE if which == "headline" else PROFILE)
    w["which"] = which
    w["precision"] = "mxfp8" if which.startswith("mxfp8") else "bf16"
    w["name"] = (w["precision"] + " MoE layer T={T}/GPU H={H} E={E} I={I} top{k} fwd+bwd").format(**w)
    w["parallelism"] = _parallelism_label(n_gpus)
    return w


def _make_layer(pkg, w, device, seed, world):
    torch.manual_seed(seed)
    with torch.device(device):      # build the (large) expert stacks directly on the GPU
        if world > 1:
            layer = pkg.ExpertParallelMoELayer(w["H"], w["I"], w["E"], top_k=w["k"], **_ep_settings())
        else:
            codes = [(0, 1, 5)[e % 3] for e in range(w["E"])] if w["which"] == "polyglu" else None
            layer = pkg.MoELayer(w["H"], w["I"], w["E"], top_k=w["k"], precision=w["precision"], act_codes=codes)
    layer = layer.to(torch.bfloat16)
    if w["which"] == "zipf":   # selection bias = 0.15 x log of Zipf(1.1) frequencies over a seeded expert order
        gz = torch.Generator().manual_seed(7)
        ranks = (torch.randperm(w["E"], generator=gz) + 1).float()
        pz = ranks.pow(-1.1)
        layer.bias.copy_((0.15 * torch.log(pz / pz.sum())).to(device))
    return layer


GEMM_OPS = ("expert_gate_up_swiglu", "expert_down", "expert_down_dgrad_glu", "expert_gate_up_dgrad", "expert_wgrad",
            "expert_linear_push", "mxfp8_expert_gemm", "mxfp8_expert_wgrad")


def _gemm_flops(w):
    """Algorithmic FLOPs per launch of each expert GEMM op (padding rows not counted)."""
    M, H, I = w["T"] * w["k"], w["H"], w["I"]
    return {"expert_gate_up_swiglu": 2.0 * M * H * 2 * I, "expert_down": 2.0 * M * I * H,
            "expert_down_dgrad_glu": 2.0 * M * H * I, "expert_gate_up_dgrad": 2.0 * M * 2 * I * H,
            "expert_wgrad": (2.0 * M * H * I + 2.0 * M * 2 * I * H) / 2.0,   # two launches per step, averaged
            "expert_linear_push": (2.0 * M * I * H + 2.0 * M * 2 * I * H) / 2.0,   # down + gate/up dgrad, averaged
            "mxfp8_expert_gemm": 12.0 * M * H * I / 4.0,                     # four launches per step, averaged
            "mxfp8_expert_wgrad": 6.0 * M * H * I / 2.0}


class Ctx:
    """Process-wide pieces of one benchmark run."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.pkg = importlib.import_module(PKG)
        self.pkg.lib()

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps, after=None):
        """CUDA events on the launching stream around exactly `steps` calls, barrier + synchronize on both
        sides, maximum over the ranks."""
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if after is not None:
            after()                       # the last copies finish inside the timed region
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1)
        if self.dist is not None:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms


def measure_layer(cx, w, steps, n_warm, e2e=True):
    """Build the layer of workload `w`, warm up, time `steps` steps with inputs resident in HBM (per-op CUDA
    events on the launching stream) and, if asked, the same through host buffers.  Returns a dict of raw figures."""
    pkg, dev, rank, world = cx.pkg, cx.dev, cx.rank, cx.world
    ops = pkg.ops
    T, H = w["T"], w["H"]
    layer = _make_layer(pkg, w, dev, seed=0, world=world)
    if w["precision"] == "mxfp8":
        # no optimizer step runs between the timed steps, so the stacks never change: with the cache of quantised
        # weights on, every step after the first would skip the weight quantisation that a training step pays
        importlib.import_module(PKG + ".mxfp8").WEIGHT_CACHE = False
    params = [layer.gate.weight, layer.gate_up_proj, layer.down_proj]
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    x_dev = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    go_dev = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)

    def step_resident():
        for p in params:
            p.grad = None
        x = x_dev.detach().requires_grad_(True)
        out = layer(x)
        out.backward(go_dev)
        return out, x.grad

    for _ in range(n_warm):
        step_resident()
    pkg.check_status()

    # ---- timed region 1: inputs resident in HBM; per-op CUDA events on the launching stream
    records = []
    ops.set_hook(lambda name, launches, a, b: records.append((name, launches, a, b)))
    sampler = ClockSampler(cx.local)
    if rank == 0:
        sampler.start()
    ms_total = cx.timed(step_resident, steps)
    clocks = sampler.stop() if rank == 0 else None
    ops.set_hook(None)
    pkg.check_status()
    per_op, launches = {}, 0
    for name, n, a, b in records:
        d = per_op.setdefault(name, [0.0, 0])
        d[0] += a.elapsed_time(b)
        d[1] += 1
        launches += n
    res = dict(ms_step=ms_total / steps, ms_total=ms_total, per_op=per_op, launches=launches, clocks=clocks,
               counts=getattr(layer, "last_counts", None))
    if not e2e:
        return res

    # ---- timed region 2: through the module with host buffers.  Every step copies its inputs from pinned host
    # memory and its results back.  The copies run on two copy streams with double-buffered device tensors, so step
    # i+1's H2D and step i-1's D2H overlap step i's kernels (a user's input pipeline does the same); nothing is skipped.
    x_host = x_dev.cpu().pin_memory()
    go_host = go_dev.cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    gx_host = torch.empty_like(x_host).pin_memory()
    h2d, d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    in_bufs = [(torch.empty_like(x_dev), torch.empty_like(go_dev)) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    state = {"i": 0, "primed": False}

    def _upload(slot):
        with torch.cuda.stream(h2d):
            h2d.wait_event(in_free[slot])
            in_bufs[slot][0].copy_(x_host, non_blocking=True)
            in_bufs[slot][1].copy_(go_host, non_blocking=True)
            in_ready[slot].record(h2d)

    def step_e2e(compute=True):
        cur = torch.cuda.current_stream(dev)
        i = state["i"]
        slot = i & 1
        if not state["primed"]:
            for ev in in_free + out_done:
                ev.record(cur)
            _upload(slot)
            state["primed"] = True
        _upload(slot ^ 1)                      # next step's inputs travel while this step computes
        cur.wait_event(in_ready[slot])
        if compute:
            for p in params:
                p.grad = None
            x = in_bufs[slot][0].detach().requires_grad_(True)
            out = layer(x)
            out.backward(in_bufs[slot][1])
            out_t, gx_t = out.detach(), x.grad
        else:                                  # copies only: the device tensors stand in for the results
            out_t, gx_t = in_bufs[slot][0], in_bufs[slot][1]
        done = torch.cuda.Event()
        done.record(cur)
        in_free[slot].record(cur)
        with torch.cuda.stream(d2h):
            d2h.wait_event(done)
            out_host.copy_(out_t, non_blocking=True)
            gx_host.copy_(gx_t, non_blocking=True)
            out_t.record_stream(d2h)
            gx_t.record_stream(d2h)
            out_done[slot].record(d2h)
        cur.wait_event(out_done[slot ^ 1])     # at most one result copy in flight behind the compute
        state["i"] = i + 1

    def drain():
        torch.cuda.current_stream(dev).wait_stream(d2h)
        torch.cuda.current_stream(dev).wait_stream(h2d)

    for _ in range(min(2, n_warm)):
        step_e2e()
    res["ms_e2e"] = cx.timed(step_e2e, steps, after=drain) / steps
    pkg.check_status()
    # what the host side alone allows: the same copies (2 x T x H bf16 each way per step and rank) with no kernels
    # between them, all ranks at once; an e2e step cannot be faster than this on this host
    for _ in range(2):
        step_e2e(False)
    res["ms_copy_only"] = cx.timed(lambda: step_e2e(False), steps, after=drain) / steps
    return res


def _kernel_table(res, w, steps):
    flops = _gemm_flops(w)
    kernels = {}
    for name, (ms, n) in sorted(res["per_op"].items(), key=lambda kv: -kv[1][0]):
        avg = ms / n
        entry = dict(launches_per_step=n / steps, avg_ms=round(avg, 4), share=round(ms / res["ms_total"], 4))
        if name in flops:
            entry["tflops"] = round(flops[name] / (avg * 1e-3) / 1e12, 1)
        kernels[name] = entry
    return kernels


def _secondary(cx, which, steps, n_warm):
    """A few steps of another configuration after the headline, resident inputs only."""
    torch.cuda.empty_cache()
    w = _workload(cx.world, which)
    res = measure_layer(cx, w, steps, n_warm, e2e=False)
    if cx.rank != 0:
        return None
    peaks = _peaks(w["precision"])
    tf = 18.0 * w["H"] * w["I"] * w["T"] * w["k"] / (res["ms_step"] * 1e-3) / 1e12
    fr = _fractions(tf, peaks, res["clocks"])
    out = {"workload": w["name"], "steps": steps, "warmup": n_warm, "ms_per_step": round(res["ms_step"], 4),
           "tokens_per_s": round(w["T"] * cx.world / (res["ms_step"] * 1e-3), 1), "layer_tflops_per_gpu": round(tf, 1),
           "layer_frac": fr["frac"], "layer_frac_rule": fr["rule"], "layer_frac_of_burst": fr["frac_of_burst"],
           "layer_frac_of_sustained": fr["frac_of_sustained"], "peak_source": peaks["source"], "clocks": res["clocks"],
           "kernels": _kernel_table(res, w, steps)}
    if res["counts"] is not None:
        c = res["counts"]
        out["tokens_per_expert"] = {"min": int(c.min()), "max": int(c.max()), "experts_without_tokens": int((c == 0).sum())}
    return out


def _library_mxfp8_tflops(dev):
    """cuBLAS's own MXFP8 GEMM (torch._scaled_mm with E8M0 block-32 scales) on this GPU in this run: the library
    yardstick for the block-scaled kernels.  Returns TFLOP/s or the error text."""
    try:
        M, N, K = 16384, 8192, 8192
        a = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(N, K, device=dev).to(torch.float8_e4m3fn)
        blocks = lambda r, k: ((r + 127) // 128) * ((k // 32 + 3) // 4) * 512
        sa = torch.full((blocks(M, K),), 127, dtype=torch.uint8, device=dev).view(torch.float8_e8m0fnu)
        sb = torch.full((blocks(N, K),), 127, dtype=torch.uint8, device=dev).view(torch.float8_e8m0fnu)
        fn = lambda: torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return round(2.0 * M * N * K * 20 / (e0.elapsed_time(e1) * 1e-3) / 1e12, 1)
    except Exception as exc:   # the box's torch may not expose MX scales
        return f"unavailable: {repr(exc)[:160]}"


EP_PARITY_TOL = 1e-2


def ep_parity(cx):
    """One forward + backward of a small expert-parallel layer (the transport and exchange of this run) against
    the single-GPU layer holding all experts on the concatenated batch, plus one load-balance step.  Every rank
    takes part; rank 0 compares.  Returns the report (rank 0) or None."""
    pkg, dist, dev, rank, W = cx.pkg, cx.dist, cx.dev, cx.rank, cx.world
    T, H, I, k = 1024, 512, 256, 4
    E = 8 * W
    El = E // W
    gen = torch.Generator().manual_seed(1234)                       # the same full model on every rank
    gate_w = (torch.randn(E, H, generator=gen) * 0.02).to(torch.bfloat16)
    gu = (torch.randn(E, 2 * I, H, generator=gen) * 0.02).to(torch.bfloat16)
    dn = (torch.randn(E, H, I, generator=gen) * 0.02).to(torch.bfloat16)
    bias = torch.randn(E, generator=gen) * 0.01
    x_all = torch.randn(W * T, H, generator=gen).to(torch.bfloat16)
    go_all = torch.randn(W * T, H, generator=gen).to(torch.bfloat16)
    ep = _ep_settings()
    with torch.device(dev):
        layer = pkg.ExpertParallelMoELayer(H, I, E, top_k=k, **ep).to(torch.bfloat16)
    with torch.no_grad():
        layer.gate.weight.copy_(gate_w)
        layer.gate_up_proj.copy_(gu[rank * El:(rank + 1) * El])
        layer.down_proj.copy_(dn[rank * El:(rank + 1) * El])
        layer.bias.copy_(bias)
    x = x_all[rank * T:(rank + 1) * T].to(dev).requires_grad_(True)
    out = layer(x)
    out.backward(go_all[rank * T:(rank + 1) * T].to(dev))
    idx, _ = pkg.fused_mlp_router(x.detach(), layer.gate.weight, layer.bias, k, E)
    layer.update_bias(0.001)
    torch.cuda.synchronize()
    pkg.check_status()

    def gather(t):          # equal shapes on every rank -> list on every rank
        parts = [torch.empty_like(t) for _ in range(W)]
        dist.all_gather(parts, t.contiguous())
        return parts

    outs, gxs, idxs = gather(out.detach()), gather(x.grad), gather(idx)
    ggu, gdn = gather(layer.gate_up_proj.grad), gather(layer.down_proj.grad)
    biases = gather(layer.bias)
    grw = layer.gate.weight.grad.float()
    dist.all_reduce(grw)                                            # the replicated router weight holds local sums
    if rank != 0:
        return None
    with torch.device(dev):
        ref = pkg.MoELayer(H, I, E, top_k=k).to(torch.bfloat16)
    with torch.no_grad():
        ref.gate.weight.copy_(gate_w)
        ref.gate_up_proj.copy_(gu)
        ref.down_proj.copy_(dn)
        ref.bias.copy_(bias)
    xr = x_all.to(dev).requires_grad_(True)
    out_r = ref(xr)
    out_r.backward(go_all.to(dev))
    idx_r, _ = pkg.fused_mlp_router(xr.detach(), ref.gate.weight, ref.bias, k, E)
    ref.update_bias(0.001)
    torch.cuda.synchronize()
    pkg.check_status()

    def rel(a, b):
        a, b = a.double().flatten(), b.double().flatten()
        return float((a - b).norm() / b.norm().clamp_min(1e-30))

    errs = {"out": rel(torch.cat(outs), out_r.detach()), "grad_x": rel(torch.cat(gxs), xr.grad),
            "grad_gate_up": rel(torch.cat(ggu), ref.gate_up_proj.grad), "grad_down": rel(torch.cat(gdn), ref.down_proj.grad),
            "grad_router_w": rel(grw, ref.gate.weight.grad.float())}
    routing_equal = bool(torch.equal(torch.cat(idxs), idx_r))
    bias_same_on_all_ranks = all(bool(torch.equal(b, biases[0])) for b in biases)
    bias_equals_single = bool(torch.equal(biases[0], ref.bias))
    ok = routing_equal and bias_same_on_all_ranks and bias_equals_single and all(e < EP_PARITY_TOL for e in errs.values())
    return {"passed": ok, "routing_equal": routing_equal, "rel_l2": {n: float(f"{e:.3e}") for n, e in errs.items()},
            "tol": EP_PARITY_TOL, "bias_update": {"identical_on_all_ranks": bias_same_on_all_ranks,
                                                  "equals_single_gpu": bias_equals_single},
            "case": f"T={T}/rank H={H} E={E} I={I} top{k}, transport={ep['transport']}, exchange={ep['exchange']}, "
                    f"against MoELayer with all {E} experts on the concatenated {W * T} tokens"}


def _nvlink_bytes(index):
    """Cumulative NVLink payload counters of one GPU (NVML field values, a read-only query): (tx, rx) bytes, or the
    reason why the counters cannot be read."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        # scope 0xFFFFFFFF = the sum over all links of the GPU
        ids = [(pynvml.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX, 0xFFFFFFFF), (pynvml.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX, 0xFFFFFFFF)]
        vals = pynvml.nvmlDeviceGetFieldValues(h, ids)
        out = []
        for v in vals:
            if v.nvmlReturn != 0:
                return f"NVML field {v.fieldId} (NVLink data throughput) returned code {v.nvmlReturn} (3 = not supported on this GPU / driver)"
            out.append(int(v.value.ullVal) * 1024)     # the counters are in KiB
        return tuple(out)
    except Exception as exc:
        return f"NVML query failed: {repr(exc)[:120]}"


def run_ours(args):
    cx = Ctx()
    rank, world, dev, dist, pkg = cx.rank, cx.world, cx.dev, cx.dist, cx.pkg
    parity = ep_parity(cx) if (world > 1 and not args.no_parity) else None
    torch.cuda.empty_cache()
    w = _workload(world, args.workload)
    T, H, E, I, k = w["T"], w["H"], w["E"], w["I"], w["k"]
    n_warm = args.warmup if args.workload.endswith("profile") else max(args.warmup, 3)
    nv0 = _nvlink_bytes(cx.local) if (rank == 0 and world > 1) else None
    res = measure_layer(cx, w, args.steps, n_warm, e2e=True)
    nv1 = _nvlink_bytes(cx.local) if (rank == 0 and world > 1) else None
    ms_step = res["ms_step"]

    secondary = {}
    if args.workload == "polyglu" and world == 1:
        # the same stack through the generic path (plain GEMM -> row kernel -> GEMM): what the fused epilogues save
        moe_mod = importlib.import_module(PKG + ".moe")
        fused_codes, moe_mod.FUSED_CODES = moe_mod.FUSED_CODES, ()
        try:
            torch.cuda.empty_cache()
            r2 = measure_layer(cx, w, max(3, min(args.steps, 10)), 3, e2e=False)
            secondary["row_kernel_path"] = {"ms_per_step": round(r2["ms_step"], 4), "clocks": r2["clocks"],
                                            "kernels": _kernel_table(r2, w, max(3, min(args.steps, 10)))}
        finally:
            moe_mod.FUSED_CODES = fused_codes
    if not args.no_secondary and args.workload == "headline":
        sec_steps, sec_warm = max(3, min(args.steps, 10)), 3
        names = ("zipf", "mxfp8") if world == 1 else ("ep5",)
        for name in names:
            try:
                secondary[name] = _secondary(cx, name, sec_steps if name != "ep5" else max(3, min(args.steps, 5)), sec_warm)
            except Exception as exc:            # the headline line is still printed
                secondary[name] = {"failed": repr(exc)[:300]}
        if world == 1:
            torch.cuda.empty_cache()
            lib = _library_mxfp8_tflops(dev)
            if isinstance(secondary.get("mxfp8"), dict):
                secondary["mxfp8"]["library_mxfp8_tflops"] = lib
                secondary["mxfp8"]["library_mxfp8_what"] = ("torch._scaled_mm, e4m3 x e4m3 with E8M0 block-32 scales, "
                                                             "16384 x 8192 x 8192, 20 calls, same GPU and run")

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peaks = _peaks(w["precision"])
    clocks = res["clocks"]
    M = T * k
    flops = _gemm_flops(w)
    per_op = res["per_op"]
    kernels = _kernel_table(res, w, args.steps)
    gemm_ms = sum(per_op[n][0] for n in GEMM_OPS if n in per_op) / args.steps
    top = max((n for n in GEMM_OPS if n in per_op), key=lambda n: per_op[n][0])
    top_avg_ms = per_op[top][0] / per_op[top][1]
    achieved = flops[top] / (top_avg_ms * 1e-3) / 1e12
    traffic = None
    if (H, I, M // E) == (NCU_TRAFFIC["H"], NCU_TRAFFIC["I"], NCU_TRAFFIC["rows_per_expert"]) and top in NCU_TRAFFIC["bytes"] \
            and w["precision"] == "bf16" and world == 1:
        traffic = round(NCU_TRAFFIC["bytes"][top] * M / NCU_TRAFFIC["rows"])
    layer_tf = 18.0 * H * I * T * k / (ms_step * 1e-3) / 1e12
    lf, kf = _fractions(layer_tf, peaks, clocks), _fractions(achieved, peaks, clocks)
    counts = res["counts"]
    line = {
        "metric": METRIC, "value": round(T * world / (ms_step * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": n_warm, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["precision"], "data": "synthetic",
        "config": {"workload": w["name"], "tokens_per_gpu": T, "d_model": H, "experts": E, "d_ff": I, "top_k": k,
                   "parallelism": w["parallelism"],
                   "l2": "no flush: the working set (expert weights + activations, several GB) exceeds the 126 MB L2"},
        "tokens_per_expert": ({"min": int(counts.min()), "max": int(counts.max()),
                               "experts_without_tokens": int((counts == 0).sum())} if counts is not None else None),
        "layer_tflops_per_gpu": round(layer_tf, 1),
        "layer_frac_of_peak": lf["frac"], "layer_frac_of_burst": lf["frac_of_burst"],
        "layer_frac_of_sustained": lf["frac_of_sustained"],
        "gemm_ms_per_step": round(gemm_ms, 4),
        "roofline": {"bound": "tensor", "kernel": f"gemm_kernel via {top}", "achieved": round(achieved, 1),
                     "peak": kf["peak"], "unit": "TFLOP/s", "frac": kf["frac"],
                     "peak_rule": f"{kf['rule']}: median SM clock {clocks.get('sm_mhz')} of {clocks.get('sm_max_mhz')} MHz "
                                  "(>= 90 % of max -> burst cuBLAS figure, else the sustained one)",
                     "frac_of_burst": kf["frac_of_burst"], "frac_of_sustained": kf["frac_of_sustained"],
                     "peaks": {"bf16_tflops_burst": peaks["burst"], "bf16_tflops_sustained": peaks["sustained"]},
                     "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read+write, scaled from the "
                     "profile workload by routed rows)" if traffic else None, "peak_source": peaks["source"]},
        "kernels": kernels,
        "e2e": {"value": round(T * world / (res["ms_e2e"] * 1e-3), 1), "unit": "tokens/s",
                "ms_per_step": round(res["ms_e2e"], 4),
                "h2d_bytes_per_step": 2 * T * H * 2, "d2h_bytes_per_step": 2 * T * H * 2,
                "host_copy_ceiling_ms": round(res["ms_copy_only"], 4),
                "host_copy_ceiling_what": "the same pinned-memory copies on all ranks at once with no kernels between "
                                          "them: the floor the host side sets for an e2e step"},
        "gpu_launches": res["launches"],
        "clocks": clocks,
    }
    if secondary:
        line["secondary"] = secondary
    if parity is not None:
        line["ep_parity"] = parity
    if world > 1:
        # what the push exchange sends per step and GPU: a result row leaves once per routed row whose token lives on
        # another GPU, forward (down projection) and backward (gate/up dgrad)
        nvl = {"result_rows_bytes_per_step_algorithmic": round(2.0 * M * H * 2 * (world - 1) / world)}
        if isinstance(nv0, tuple) and isinstance(nv1, tuple):
            steps_all = n_warm + args.steps + min(2, n_warm) + args.steps          # resident + host-buffer steps
            nvl.update(tx_bytes_per_step_counted=round((nv1[0] - nv0[0]) / steps_all),
                       rx_bytes_per_step_counted=round((nv1[1] - nv0[1]) / steps_all),
                       source="NVML NVLINK_THROUGHPUT_DATA_TX/RX of GPU 0 before and after the timed regions (a query), "
                              f"divided by the {steps_all} layer steps between the two reads (copy-only steps move "
                              "nothing over NVLink)")
        else:
            nvl["counted"] = None
            nvl["counters_unavailable"] = nv0 if isinstance(nv0, str) else nv1
        line["nvlink"] = nvl
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(w, steps=1, warmup=0)
    print(json.dumps(line), flush=True)
    failed = parity is not None and not parity["passed"]
    if dist is not None:
        dist.destroy_process_group()
    if failed:
        sys.exit(3)


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
    fr = _fractions(achieved, peaks, clocks)
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
                     "achieved": round(achieved, 1), "peak": fr["peak"], "unit": "TFLOP/s", "frac": fr["frac"],
                     "peak_rule": fr["rule"], "frac_of_burst": fr["frac_of_burst"],
                     "frac_of_sustained": fr["frac_of_sustained"], "traffic": None, "peak_source": peaks["source"]},
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


def run_conv_router(args):
    """--workload conv_router: forward + backward of `fused_router` (causal K-tap conv router) on the token count and
    width of the headline layer, once with the GEMMs that read x in place through shifted TMA boxes and once over
    the unfolded (B*S, K*H) copy.  A line of its own for the conv-router row, not the headline metric."""
    if int(os.environ.get("WORLD_SIZE", 1)) > 1:
        if int(os.environ.get("RANK", 0)) == 0:
            print(json.dumps({"workload": "conv_router", "unavailable": "single-GPU workload"}), flush=True)
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pkg = importlib.import_module(PKG)
    pkg.lib()
    ops = pkg.ops
    B, S, H, E, K, k = 16, 1024, HEADLINE["H"], HEADLINE["E"], 4, HEADLINE["k"]
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(B, S, H, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(E, H, K, device=dev, generator=g) * 0.02).to(torch.bfloat16).requires_grad_(True)
    bias = torch.randn(E, device=dev, generator=g) * 0.01
    G = torch.randn(B, S, k, device=dev, generator=g)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)     # larger than the 126 MB L2

    def step():
        x.grad = w.grad = None
        _, wt = pkg.fused_router(x, w, bias, k, E)
        (wt * G).sum().backward()

    def measure(steps, warm):
        for _ in range(warm):
            step()
        pkg.check_status()
        records = []
        ops.set_hook(lambda name, launches, a, b: records.append((name, launches, a, b)))
        total = 0.0
        sampler = ClockSampler(0)
        sampler.start()
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        clocks = sampler.stop()
        ops.set_hook(None)
        pkg.check_status()
        per_op, launches = {}, 0
        for name, n, a, b in records:
            d = per_op.setdefault(name, [0.0, 0])
            d[0] += a.elapsed_time(b)
            d[1] += 1
            launches += n
        kernels = {name: dict(launches_per_step=n / steps, avg_ms=round(ms / n, 4))
                   for name, (ms, n) in sorted(per_op.items(), key=lambda kv: -kv[1][0])}
        return total / steps, kernels, launches, clocks

    n_warm = max(args.warmup, 3)
    steps = max(3, min(args.steps, 50))
    ms, kernels, launches, clocks = measure(steps, n_warm)
    direct_ok = ops.conv_direct_ok
    ops.conv_direct_ok = lambda S_, H_: False
    try:
        ms_u, kernels_u, _, clocks_u = measure(steps, n_warm)
    finally:
        ops.conv_direct_ok = direct_ok
    flops = 6.0 * B * S * K * H * E          # logits, dX and dW GEMMs
    line = {
        "metric": "conv_router_fwd_bwd_ms", "value": round(ms, 4), "unit": "ms", "n_gpus": 1, "steps": steps, "warmup": n_warm,
        "ms_per_step": round(ms, 4), "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"fused_router fwd+bwd, x ({B},{S},{H}) bf16, conv weight ({E},{H},{K}), top-{k}",
                   "l2": "flushed between steps (256 MB write)"},
        "gemm_tflops": round(flops / (ms * 1e-3) / 1e12, 1),
        "kernels": kernels, "gpu_launches": launches, "clocks": clocks,
        "unfolded_copy_path": {"ms_per_step": round(ms_u, 4), "kernels": kernels_u, "clocks": clocks_u},
    }
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
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm runs on rank 0 alone and uses every host core
    torch.set_num_threads(os.cpu_count() or 1)
    w = _workload(world, args.workload)
    cb = cpu_baseline(w, steps=max(1, min(args.steps, 3)), warmup=min(args.warmup, 1))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tokens/s", "n_gpus": world,
            "steps": max(1, min(args.steps, 3)), "warmup": min(args.warmup, 1), "ms_per_step": cb["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "d_model": w["H"], "experts": w["E"], "d_ff": w["I"], "top_k": w["k"],
                       "parallelism": f"host cores, one process, {torch.get_num_threads()} threads"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_torch_grouped(args):
    """Same-box library yardstick: the reference's library-GEMM formulation of the expert pipeline written out in
    plain PyTorch (sort by expert -> torch._grouped_mm -> SiLU-GLU -> torch._grouped_mm -> weighted index_add_,
    backward by autograd; the formulation of kernels/sm120/moe_grouped.py:93-121), fed by this package's router so
    that only the expert pipeline differs.  Not part of the product; printed with "impl": "torch_grouped"."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pkg = importlib.import_module(PKG)
    w = _workload(1, args.workload)
    T, H, E, I, k = w["T"], w["H"], w["E"], w["I"], w["k"]
    line = {"impl": "torch_grouped", "metric": METRIC, "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
            "dtype": "bf16", "data": "synthetic", "config": {"workload": w["name"], "parallelism": "single GPU",
                                                             "what": "torch.sort + torch._grouped_mm x2 + index_add_, autograd backward"}}
    if not hasattr(torch, "_grouped_mm"):
        line["unavailable"] = "this torch has no torch._grouped_mm"
        print(json.dumps(line), flush=True)
        return
    layer = _make_layer(pkg, w, dev, seed=0, world=1)
    g = torch.Generator(device=dev).manual_seed(1)
    x_dev = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    go_dev = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    params = [layer.gate.weight, layer.gate_up_proj, layer.down_proj]

    def experts(flat, idx, wt):
        order = torch.sort(idx.flatten(), stable=True).indices
        tok = order // k
        offs = torch.cumsum(torch.bincount(idx.flatten(), minlength=E), 0).to(torch.int32)
        xs = flat[tok]
        gu = torch._grouped_mm(xs, layer.gate_up_proj.transpose(-2, -1), offs=offs)
        inter = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        eo = torch._grouped_mm(inter, layer.down_proj.transpose(-2, -1), offs=offs)
        out = torch.zeros(T, H, dtype=torch.float32, device=dev)
        out.index_add_(0, tok, eo.float() * wt.flatten()[order].unsqueeze(-1))
        return out.to(flat.dtype)

    def step():
        for p in params:
            p.grad = None
        x = x_dev.detach().requires_grad_(True)
        idx, wt = pkg.fused_mlp_router(x, layer.gate.weight, layer.bias, k, E)
        experts(x, idx, wt).backward(go_dev)

    try:
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1) / args.steps
        line.update(value=round(T / (ms * 1e-3), 1), steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=round(ms, 4),
                    layer_tflops_per_gpu=round(18.0 * H * I * T * k / (ms * 1e-3) / 1e12, 1), clocks=clocks,
                    peak_memory_gb=round(torch.cuda.max_memory_allocated() / 1e9, 2))
    except Exception as exc:
        line["unavailable"] = repr(exc)[:300]
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch_grouped"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary configurations after the headline")
    ap.add_argument("--no-parity", action="store_true", help="N > 1: skip the expert-parallel parity check")
    ap.add_argument("--workload", default="headline", choices=["headline", "profile", "ep5", "mxfp8", "mxfp8_profile", "zipf", "polyglu", "muon", "muon_profile",
                             "conv_router"],
                    help="profile = small case for profiler captures (not a benchmark number)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "torch_grouped":
        run_torch_grouped(args)
    elif args.workload.startswith("muon"):
        run_muon(args)
    elif args.workload == "conv_router":
        run_conv_router(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

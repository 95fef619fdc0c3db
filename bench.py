#!/usr/bin/env python
"""Benchmark of the SRU hot path on B200: forward+backward tokens/s of a batch-sharded
training step (projection GEMMs + light-recurrence scans + per-layer gradient all-reduce).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 5] [--impl ours|reference]

One process per GPU (torchrun for N > 1).  Rank 0 prints ONE JSON line.  `value` is measured
with inputs resident in HBM; `e2e` is the same step through the public module API with the
step's input copied from pinned host memory and the loss read back inside the timed region.
`roofline` describes the kernel class that takes the most time (CUDA events around every
C-ABI launch in a separate instrumented pass); `kernels` lists every class.  `cpu_baseline`
(N = 1 only) times the CPU implementation on a bounded sample of the same workload (1 warm-up
+ 3 timed steps, median): for forward-only workloads the reference's own compiled CPU operator
(kind "reference", when its library was built beside the oracle), else the C restatement of the
reference's CPU path (kind "port").  `--impl reference` times that CPU implementation instead,
with all host threads, and imports nothing of the shipped package.  `check` carries the loss and
a float64 checksum of one layer's reduced weight gradient, equal at every N up to summation order.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The five workloads (shapes and distributions of the benchmark definition; synthetic data).
CONFIGS = {
    1: dict(name="config1: 2-layer uni SRU 128->128, fp32, L=20 B=32", L=20, B=32, amp=None,
            kwargs=dict(input_size=128, hidden_size=128, num_layers=2, dropout=0.0, highway_bias=-2.0,
                        layer_norm=False), x_std=1.0, lens=None, loss="sum", train=True),
    2: dict(name="config2: 4-layer bi SRU 512->512/dir, layer_norm, rescale, bf16 autocast, L=256 B=64, mask_pad",
            L=256, B=64, amp=torch.bfloat16,
            kwargs=dict(input_size=512, hidden_size=512, num_layers=4, bidirectional=True, layer_norm=True,
                        rescale=True), x_std=1.0, lens=(128, 256), loss="sum", train=True),
    3: dict(name="config3: 6-layer uni SRU 2048, projection 512, highway_bias -3, fp16 autocast, L=512 B=32",
            L=512, B=32, amp=torch.float16,
            kwargs=dict(input_size=2048, hidden_size=2048, num_layers=6, projection_size=512,
                        highway_bias=-3.0), x_std=0.5, lens=None, loss="meansq", train=True, c0=True,
            loss_scale=65536.0),   # static loss scale, as a GradScaler would hold (fp16 gradients underflow without)
    4: dict(name="config4: 1-layer uni SRU 1024, bf16, L=8192 B=16, inference", L=8192, B=16, amp=None,
            kwargs=dict(input_size=1024, hidden_size=1024, num_layers=1), x_std=1.0, lens=None, loss=None,
            train=False, param_dtype=torch.bfloat16),
    5: dict(name="config5: 12-layer bi SRU 120->1024/dir, dropout 0.1, bf16 autocast, L=1000 B=256, mask_pad",
            L=1000, B=256, amp=torch.bfloat16,
            kwargs=dict(input_size=120, hidden_size=1024, num_layers=12, bidirectional=True, dropout=0.1),
            x_std=1.0, lens=(600, 1000), loss="meansq", train=True),
}


def make_inputs(cfg, cfg_id, B, batch_offset=0):
    """Seeded synthetic inputs on the CPU: x ~ N(0, x_std), tail padding from uniform lengths."""
    g = torch.Generator().manual_seed(1000 + cfg_id)
    L, Bfull = cfg["L"], cfg["B"]
    x = torch.randn(L, Bfull, cfg["kwargs"]["input_size"], generator=g) * cfg["x_std"]
    mask = None
    if cfg["lens"] is not None:
        lo, hi = cfg["lens"]
        lens = torch.randint(lo, hi + 1, (Bfull,), generator=g)
        mask = torch.arange(L).view(L, 1) >= lens.view(1, Bfull)
    x = x[:, batch_offset:batch_offset + B].contiguous()
    if mask is not None:
        mask = mask[:, batch_offset:batch_offset + B].contiguous()
    return x, mask


def layer_shapes(kwargs):
    """[(in, D, k, dirs, proj)] per layer, as sru/modules.py:126-133,551-568 derive them."""
    dirs = 2 if kwargs.get("bidirectional") else 1
    D = kwargs["hidden_size"] * dirs
    out = []
    for i in range(kwargs.get("num_layers", 2)):
        n_in = kwargs["input_size"] if i == 0 else D
        k = 4 if (kwargs.get("has_skip_term", True) and n_in != D) else 3
        p = kwargs.get("projection_size", 0)
        p = p if 0 < p < min(n_in, D) else 0
        out.append((n_in, D, k, dirs, p))
    return out


def algorithmic_work(cfg, B, s_bytes, c_bytes):
    """Bytes of the scans and flops of the GEMMs for one step on B sequences.

    Per column-step: forward (training) reads U[k] (+x when k=3) and writes h and c:
    (k + e3 + 1)*s + c_bytes; inference (no c history) (k + e3 + 1)*s; backward reads U[k], x,
    c, grad_h and writes grad_U[k], grad_x: (2k + 2*e3 + 1)*s + c_bytes.  GEMM flops:
    2*M*K*N per product, backward = dgrad + wgrad (no dgrad for the first layer's input).
    """
    L = cfg["L"]
    fwd = bwd = 0
    flops_f = flops_b = 0
    gemm_bytes = 0
    ln_f = ln_b = 0
    for li, (n_in, D, k, dirs, p) in enumerate(layer_shapes(cfg["kwargs"])):
        cols = L * B * D
        e3 = 1 if k == 3 else 0
        if cfg["train"]:
            fwd += cols * ((k + e3 + 1) * s_bytes + c_bytes)
            bwd += cols * ((2 * k + 2 * e3 + 1) * s_bytes + c_bytes)
        else:
            fwd += cols * (k + e3 + 1) * s_bytes
        M = L * B
        f = 2 * M * (n_in * p + p * D * k) if p else 2 * M * n_in * D * k
        flops_f += f
        # operand + result bytes of this layer's products (16-bit), each matrix counted once per product
        prods = [(M, n_in, p), (M, p, D * k)] if p else [(M, n_in, D * k)]
        for (m_, k_, n_) in prods:
            once = 2 * (m_ * k_ + k_ * n_ + m_ * n_)
            gemm_bytes += once * (3 if (cfg["train"] and (li > 0 or (m_, k_, n_) != prods[0])) else (2 if cfg["train"] else 1))
        if cfg["train"]:
            flops_b += 2 * f if li > 0 else (2 * f - (2 * M * n_in * (p if p else D * k)))
        if cfg["kwargs"].get("layer_norm"):
            # layer normalisation: forward reads x, writes y; backward reads dy and x, writes dx
            after = cfg["kwargs"].get("normalize_after", False)
            n_ln = D if after else n_in
            sx = s_bytes if (after or li > 0) else 4          # the first layer's input is the fp32 batch
            sy = s_bytes
            ln_f += M * n_ln * (sx + sy)
            ln_b += M * n_ln * (sy + 2 * sx)
    return dict(scan_fwd_bytes=fwd, scan_bwd_bytes=bwd, gemm_fwd_flops=flops_f, gemm_bwd_flops=flops_b,
                gemm_bytes=gemm_bytes, ln_fwd_bytes=ln_f, ln_bwd_bytes=ln_b)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], 0, set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                mhz.append(float(r[0])); mx = max(mx, float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not mhz:
            return None
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], tflops_burst=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


def build_model(cfg, device):
    from sru_b200.modules import SRU
    torch.manual_seed(0)
    model = SRU(**cfg["kwargs"])
    if cfg.get("param_dtype") is not None:
        model = model.to(cfg["param_dtype"])
    model = model.to(device)
    model.train(cfg["train"])
    return model


def run_step(model, cfg, x, mask, c0, tokens_global, reducer=None):
    """One step on device-resident inputs.  Returns the loss tensor (or h for inference)."""
    if not cfg["train"]:
        with torch.no_grad():
            h, c = model(x, c0, mask_pad=mask)
        return c
    if reducer is not None:
        reducer.zero_grad()
    else:
        model.zero_grad(set_to_none=True)
    amp = cfg["amp"]
    with torch.autocast("cuda", dtype=amp, enabled=amp is not None):
        h, c = model(x, c0, mask_pad=mask)
    D = h.size(-1)
    if cfg["loss"] == "sum":
        loss = h.float().sum()
    else:
        loss = (h.float() ** 2).sum() / float(tokens_global * D)
    scale = cfg.get("loss_scale", 1.0)
    (loss * scale if scale != 1.0 else loss).backward()
    if reducer is not None:
        reducer.finish()
    return loss.detach()


def _reference_cpu_op():
    """The reference's own compiled CPU scan (forward only), if its library was built beside the oracle."""
    so = os.path.join(ROOT, "oracle", "_ref", "libsru_cpu_ref.so")
    if not os.path.exists(so):
        return None
    try:
        torch.ops.load_library(so)
        return torch.ops.sru_cpu
    except (OSError, RuntimeError):
        return None


def cpu_baseline(cfg, cfg_id, threads, sample_B, steps=3, warmup=1):
    """Times the CPU implementation of the path on sample_B sequences.  Returns (tokens per step, step times, kind).

    Training workloads: the oracle model (C restatement of the reference's CPU training path, whose own form is a
    Python loop over time steps, sru/ops.py:205-248): kind "port".  Forward-only workloads: the same layer stack
    with the recurrence done by the reference's own compiled operator sru_cpu::cpu_forward / cpu_bi_forward
    (sru/csrc/sru_cpu_impl.cpp:56-226): kind "reference"; "port" if that library is absent.
    Nothing of the shipped package is imported here.
    """
    from oracle import sru_oracle
    from oracle.ref_model import OracleSRU
    torch.set_num_threads(threads)
    sru_oracle.set_threads(threads)
    torch.manual_seed(0)
    kw = dict(cfg["kwargs"])
    model = OracleSRU(kw.pop("input_size"), kw.pop("hidden_size"), **kw)
    model.train(cfg["train"])
    kind = "port"
    if not cfg["train"]:
        ops = _reference_cpu_op()
        if ops is not None:
            kind = "reference"

            def recurrence(U, x, V, bias, c0, act, d, bi, skip, scale, mask_c, mask_pad):
                L_, B_ = x.size(0), x.size(1)
                k = U.size(-1) // d // (2 if bi else 1)
                fn = ops.cpu_bi_forward if bi else ops.cpu_forward
                h, c = fn(U.contiguous(), x.contiguous(), V.contiguous(), bias.contiguous(), c0.contiguous(),
                          None if mask_pad is None else mask_pad.bool().contiguous(), L_, B_, d, k, act, skip,
                          1.0 if scale is None else float(scale), False)
                return h, c
            model.recurrence = recurrence
    x, mask = make_inputs(cfg, cfg_id, sample_B)
    tokens = cfg["L"] * sample_B
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        if cfg["train"]:
            model.zero_grad(set_to_none=True)
            h, c = model(x, mask_pad=mask)
            loss = h.sum() if cfg["loss"] == "sum" else (h ** 2).sum() / float(tokens * h.size(-1))
            loss.backward()
        else:
            with torch.no_grad():
                model(x, mask_pad=mask)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return tokens, times, kind


def traffic_ratios():
    """DRAM bytes / algorithmic bytes per kernel class, from the ncu captures summarised beside the profiles."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", type=int, default=5, choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="capture the step in one CUDA graph and time its replays (1 GPU; for launch-bound configs)")
    ap.add_argument("--cpu-sample-batch", type=int, default=0)
    ap.add_argument("--reduce-dtype", default="fp32", choices=["fp32", "bf16"],
                    help="N > 1: type the layer gradient buckets are all-reduced in")
    ap.add_argument("--no-defer", action="store_true",
                    help="N > 1: start a layer's all-reduce as soon as its bucket is complete instead of behind the "
                         "next backward scan")
    ap.add_argument("--nccl-max-ctas", type=int, default=0,
                    help="N > 1: cap on the CTAs NCCL uses per collective (NCCL_MAX_CTAS), 0 = NCCL's default")
    ap.add_argument("--no-bias-fold", action="store_true",
                    help="leave the gate bias to the scan instead of the GEMM epilogue (A/B measurement)")
    ap.add_argument("--sustain-seconds", type=float, default=3.0,
                    help="N > 1: after the timed steps, keep stepping for about this long and report that step time too")
    ap.add_argument("--c-hist", default="float32", choices=["float32", "storage"],
                    help="type of the saved state history: float32 (default) or the 16-bit storage type (2 bytes less "
                         "per column-step in both scans; backward then feeds a 16-bit-rounded c[t-1] into the sigmoid)")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the global batch (profiling on a small case; the workload name says so)")
    ap.add_argument("--length", type=int, default=0,
                    help="override the sequence length (profiling on a small case; the workload name says so)")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.length:
        cfg["name"] = cfg["name"] + " [length reduced to %d]" % args.length
        if cfg["lens"] is not None:
            cfg["lens"] = (max(1, cfg["lens"][0] * args.length // cfg["L"]), args.length)
        cfg["L"] = args.length
    if args.batch:
        cfg["name"] = cfg["name"] + " [batch reduced to %d]" % args.batch
        cfg["B"] = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    metric = "sru_fwd_bwd_tokens_per_sec" if cfg["train"] else "sru_fwd_tokens_per_sec"
    host_cores = os.cpu_count() or 1
    sample_B = args.cpu_sample_batch or {1: 32, 2: 8, 3: 2, 4: 2, 5: 4}[args.config]
    sample_desc = "%s at batch %d of %d (all layers, full length, fp32 on CPU)" % (
        cfg["name"].split(":")[0], sample_B, cfg["B"])

    if args.impl == "reference":
        if rank != 0:
            return
        threads = host_cores
        tokens, times, kind = cpu_baseline(cfg, args.config, threads, sample_B, steps=max(1, args.steps),
                                           warmup=min(args.warmup, 1))
        ms = 1e3 * sum(times) / len(times)
        val = tokens / (ms / 1e3)
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg["name"], "sample": sample_desc},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": kind,
                             "sample": sample_desc},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    import torch.distributed as dist
    from sru_b200 import _lib, ops
    from sru_b200.distributed import LayerGradAllReducer, shard_batch, use_global_dropout_masks
    from sru_b200.projection import gemm_backend
    _lib.lib()  # fail loudly here if the native library is missing
    if args.no_bias_fold:
        from sru_b200 import projection
        projection.set_bias_fold_enabled(False)
    ops.set_c_hist_dtype(args.c_hist)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        if args.nccl_max_ctas > 0:
            os.environ["NCCL_MAX_CTAS"] = str(args.nccl_max_ctas)     # this script is the launcher of its ranks
        dist.init_process_group("nccl", device_id=device)
    if world != args.gpus and rank == 0:
        sys.stderr.write("warning: --gpus %d but WORLD_SIZE %d\n" % (args.gpus, world))

    model = build_model(cfg, device)
    if cfg["train"] and cfg["kwargs"].get("dropout", 0) > 0:
        # every rank draws the masks of the global batch and keeps its rows: the step computes the same numbers at every N
        use_global_dropout_masks(model, cfg["B"], rank, world, seed=1234)
    x_cpu, mask_cpu = make_inputs(cfg, args.config, cfg["B"])
    x_cpu = shard_batch(x_cpu, rank, world)
    mask_cpu = shard_batch(mask_cpu, rank, world)
    if cfg.get("param_dtype") is not None:
        x_cpu = x_cpu.to(cfg["param_dtype"])
    B_local = x_cpu.size(1)
    tokens_global = cfg["L"] * cfg["B"]
    x_pin = x_cpu.pin_memory()
    mask_pin = None if mask_cpu is None else mask_cpu.pin_memory()
    x_dev = x_pin.to(device)
    mask_dev = None if mask_pin is None else mask_pin.to(device)
    c0 = None
    if cfg.get("c0"):
        dirs = 2 if cfg["kwargs"].get("bidirectional") else 1
        c0 = torch.zeros(cfg["kwargs"]["num_layers"], B_local, cfg["kwargs"]["hidden_size"] * dirs, device=device)
    reducer = None
    if cfg["train"] and world > 1:
        reducer = LayerGradAllReducer(model, reduce_dtype=torch.bfloat16 if args.reduce_dtype == "bf16" else None,
                                      defer_to_scan_end=not args.no_defer)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up ----
    for _ in range(max(args.warmup, 3)):
        run_step(model, cfg, x_dev, mask_dev, c0, tokens_global, reducer)
    barrier()

    # ---- optional: the whole step as one CUDA graph (the launchers are capture-safe) ----
    graph = None
    graph_out = None
    graph_launches = 0
    if args.cuda_graph and world == 1:
        n0 = _lib.launch_count
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = run_step(model, cfg, x_dev, mask_dev, c0, tokens_global, None)
        graph_launches = _lib.launch_count - n0
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()

    def step_resident():
        if graph is not None:
            graph.replay()
            return graph_out
        return run_step(model, cfg, x_dev, mask_dev, c0, tokens_global, reducer)

    # ---- timed: device-resident inputs ----
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = _lib.launch_count
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    launches = _lib.launch_count - launches0          # this rank's own kernels inside the timed region
    if graph is not None:
        launches = graph_launches * args.steps        # kernel nodes of the graph, replayed
    clocks = sampler.stop() if sampler else None
    ms_per_step = ms_total / args.steps
    value = tokens_global / (ms_per_step / 1e3)

    # ---- timed: end to end (pinned host input -> device, loss -> host) ----
    result_bytes = 0
    if graph is not None:
        barrier()
        e0.record()
        for _ in range(args.steps):
            x_dev.copy_(x_pin, non_blocking=True)         # the graph reads its inputs from these buffers
            if mask_pin is not None:
                mask_dev.copy_(mask_pin, non_blocking=True)
            out = step_resident()
            host = out.float().cpu()
            result_bytes = host.numel() * host.element_size()
    else:
        # Every step's input comes from pinned host memory through the package's input pipeline: the copy of step i + 1
        # runs on a side stream while step i computes.  One untimed step fills the pipeline (buffers, first copy);
        # during each of the timed steps exactly one input copy runs (that of the following step), so the timed region
        # holds as many host-to-device copies as steps.
        from sru_b200.data import DevicePrefetcher
        feed = iter(DevicePrefetcher(((x_pin, mask_pin) for _ in range(args.steps + 2)), device))
        xd, md = next(feed)
        run_step(model, cfg, xd, md, c0, tokens_global, reducer).float().cpu()
        barrier()
        e0.record()
        for _ in range(args.steps):
            xd, md = next(feed)
            out = run_step(model, cfg, xd, md, c0, tokens_global, reducer)
            host = out.float().cpu()
            result_bytes = host.numel() * host.element_size()
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    h2d = x_pin.numel() * x_pin.element_size() + (0 if mask_pin is None else mask_pin.numel())

    # ---- what the step computed: the loss and a checksum of one layer's (reduced) weight gradient ----
    check = None
    if cfg["train"]:
        # the check step always uses the first draw of the global dropout masks, whatever --steps / --warmup were, so
        # that its numbers compare across runs and world sizes
        use_global_dropout_masks(model, cfg["B"], rank, world, seed=1234)
        out_loss = run_step(model, cfg, x_dev, mask_dev, c0, tokens_global, reducer)
        loss_t = out_loss.double().clone()
        if world > 1:
            dist.all_reduce(loss_t)          # each rank holds the loss of its shard, normalised by the global count
        wlast = model.rnn_lst[-1].weight.grad.double() / cfg.get("loss_scale", 1.0)
        check = {"loss": float(loss_t), "grad_weight_last_layer_sum": float(wlast.sum()),
                 "grad_weight_last_layer_abs_sum": float(wlast.abs().sum())}

    # ---- N > 1: the same step over a longer stretch (power-limited steady state), reported beside the timed steps ----
    sustained = None
    if world > 1 and args.sustain_seconds > 0:
        n_more = max(args.steps, int(math.ceil(args.sustain_seconds * 1e3 / max(ms_per_step, 1e-3))))
        barrier()
        e0.record()
        for _ in range(n_more):
            step_resident()
        e1.record()
        barrier()
        ms_more = max_over_ranks(e0.elapsed_time(e1)) / n_more
        sustained = {"steps": n_more, "ms_per_step": ms_more, "value": tokens_global / (ms_more / 1e3),
                     "unit": "tokens/s"}

    # ---- instrumented pass: CUDA events around every C-ABI launch ----
    _lib.timer = _lib.KernelTimer()
    for _ in range(2):
        run_step(model, cfg, x_dev, mask_dev, c0, tokens_global, reducer)
    ksum = _lib.timer.summary()
    _lib.timer = None
    nprof = 2

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    s_bytes = 4 if (cfg["amp"] is None and cfg.get("param_dtype") is None) else 2
    c_bytes = 4 if (s_bytes == 4 or ops._c_hist_dtype == "float32") else s_bytes
    work = algorithmic_work(cfg, B_local, s_bytes, c_bytes)
    kernels = {}
    for name, (calls, ms) in ksum.items():
        per_step_ms = ms / nprof
        ent = {"launches_per_step": calls // nprof, "ms_per_step": per_step_ms}
        if name in ("scan_fwd", "scan_fwd_infer"):
            ent.update(bound="hbm", achieved=work["scan_fwd_bytes"] / (per_step_ms * 1e6), unit="GB/s",
                       peak=peaks["hbm_gbs"])
        elif name == "scan_bwd":
            ent.update(bound="hbm", achieved=work["scan_bwd_bytes"] / (per_step_ms * 1e6), unit="GB/s",
                       peak=peaks["hbm_gbs"])
        elif name == "layer_norm_fwd" and work["ln_fwd_bytes"]:
            ent.update(bound="hbm", achieved=work["ln_fwd_bytes"] / (per_step_ms * 1e6), unit="GB/s",
                       peak=peaks["hbm_gbs"])
        elif name == "layer_norm_bwd" and work["ln_bwd_bytes"]:
            ent.update(bound="hbm", achieved=work["ln_bwd_bytes"] / (per_step_ms * 1e6), unit="GB/s",
                       peak=peaks["hbm_gbs"])
        ent["frac"] = ent["achieved"] / ent["peak"] if "achieved" in ent else None
        kernels[name] = ent
    gemm_ms = sum(v["ms_per_step"] for k, v in kernels.items() if k.startswith("gemm"))
    if gemm_ms > 0:
        fl = work["gemm_fwd_flops"] + work["gemm_bwd_flops"]
        kernels["gemm_all"] = {"ms_per_step": gemm_ms, "bound": "tensor", "achieved": fl / (gemm_ms * 1e9),
                               "unit": "TFLOP/s", "peak": peaks["tflops_sustained"],
                               "frac": fl / (gemm_ms * 1e9) / peaks["tflops_sustained"]}
    cands = {k: v for k, v in kernels.items() if v.get("frac") is not None and not (k.startswith("gemm_") and k != "gemm_all")}
    roofline = None
    if cands:
        top = max(cands, key=lambda k: cands[k]["ms_per_step"])
        t = cands[top]
        # DRAM traffic per launch: ratio of measured dram bytes to algorithmic bytes from the ncu captures
        # (small case of the same kernels; the capture's summary writes the ratios to a file), applied to this
        # run's units.
        ratio = traffic_ratios().get(top, {}).get("dram_over_algorithmic")
        alg = {"scan_fwd": work["scan_fwd_bytes"], "scan_fwd_infer": work["scan_fwd_bytes"],
               "scan_bwd": work["scan_bwd_bytes"], "gemm_all": work["gemm_bytes"]}.get(top)
        if top == "gemm_all":
            n_launch = sum(v["launches_per_step"] for k2, v in kernels.items()
                           if k2.startswith("gemm_") and k2 != "gemm_all")
        else:
            n_launch = kernels[top]["launches_per_step"]
        traffic = (ratio * alg / max(1, n_launch)) if (ratio and alg) else None
        roofline = {"kernel": top, "bound": t["bound"], "achieved": t["achieved"], "peak": t["peak"],
                    "unit": t["unit"], "frac": t["frac"], "traffic": traffic,
                    "traffic_note": "bytes per launch; ncu dram bytes / algorithmic bytes of a small case, scaled by units",
                    "peak_source": peaks["source"]}

    out = {
        "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "f32" if s_bytes == 4 else ("bf16" if (cfg["amp"] or cfg.get("param_dtype")) == torch.bfloat16 else "f16"),
        "data": "synthetic",
        "config": {"workload": cfg["name"], "global_batch": cfg["B"], "seq_len": cfg["L"],
                   "parallelism": "batch-sharded dp%d" % world, "l2": "inputs larger than L2",
                   "gemm": gemm_backend(), "c_hist": ops._c_hist_dtype, "amp_mode": ops.get_amp_mode(),
                   "cuda_graph": graph is not None, "bias_in_gemm_epilogue": not args.no_bias_fold,
                   "inference_path": None if cfg["train"] else
                   "layer loop as one native call; the 16-bit copy of the weights and the bias layout are kept between calls",
                   "all_reduce": None if reducer is None else {
                       "dtype": args.reduce_dtype, "bytes_per_step": reducer.bytes_per_step(),
                       "start": "at bucket completion" if args.no_defer else "behind the next backward scan",
                       "nccl_max_ctas": args.nccl_max_ctas or None}},
        "e2e": {"value": tokens_global / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": result_bytes},
        "gpu_launches": launches,
        "gpu_launches_per_step": launches // max(1, args.steps),
        "check": check,
        "sustained": sustained,
        "clocks": clocks,
        "roofline": roofline,
        "kernels": kernels,
    }
    if world == 1 and not args.no_cpu_baseline:
        tokens, times, kind = cpu_baseline(cfg, args.config, host_cores, sample_B, steps=3, warmup=1)
        med = sorted(times)[len(times) // 2]
        out["cpu_baseline"] = {"value": tokens / med, "unit": "tokens/s", "cores": host_cores, "kind": kind,
                               "sample": sample_desc + "; 1 warm-up + 3 timed steps, median"}
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the quantized MoE block (BASELINE.json metric: MoE layer tokens/s, 4-bit
Qwen3-30B-A3B shape; % of roofline).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]

One step = one forward of the block over one batch of T synthetic tokens (seeded random
weights quantized with the library's own quantize kernel; there are no checkpoints here).
Prints ONE JSON line.  `value` is timed with the inputs resident in HBM, `e2e` through the
public API with host buffers (H2D of x and D2H of the output inside the timed region).
L2 is flushed between timed iterations (a 512 MB buffer is overwritten), and every iteration is
timed with its own pair of CUDA events on the launching stream.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
SWEEP = (1, 4, 16, 64, 512, 2048, 8192)  # BASELINE.json configs[1]

# BASELINE.json configs: 1 = Qwen3-30B-A3B layer (the metric's configuration; its sweep is attached to the
# default run), 2 = 48-layer stack of config 1 (--workload stack), 3 = Qwen3-235B-A22B layer, 4 = Mixtral
# layer (top-k on the logits then softmax over the selected; Zipf(1.2)-skewed routing; 4- or 8-bit).
CONFIGS = {
    1: dict(shape=dict(hidden=2048, inter=768, n_experts=128, top_k=8, bits=4, group_size=64), tokens=8192,
            router_mode=0, norm_topk_prob=True, zipf=False,
            name="configs[1] point T={T}: Qwen3-30B-A3B MoE layer (H2048 E128 top-8 I768, {bits}-bit g64), bf16 N(0,1) tokens"),
    3: dict(shape=dict(hidden=4096, inter=1536, n_experts=128, top_k=8, bits=4, group_size=64), tokens=8192,
            router_mode=0, norm_topk_prob=True, zipf=False,
            name="configs[3] T={T}: Qwen3-235B-A22B MoE layer (H4096 E128 top-8 I1536, {bits}-bit g64), bf16 N(0,1) tokens"),
    4: dict(shape=dict(hidden=4096, inter=14336, n_experts=8, top_k=2, bits=4, group_size=64), tokens=16384,
            router_mode=1, norm_topk_prob=False, zipf=True,
            name="configs[4] T={T}: Mixtral MoE layer (H4096 E8 top-2 I14336, {bits}-bit g64, softmax over the selected, "
                 "Zipf(1.2) logit bias), bf16 N(0,1) tokens"),
}
CONFIGS[2] = dict(CONFIGS[1])
SHAPE = dict(CONFIGS[1]["shape"])   # replaced by main() according to --config / --bits
CFG = CONFIGS[1]


def zipf_bias(E):
    """Per-expert router logit bias 2*ln(p_e), p_e ~ rank^-1.2 (constant offset dropped)."""
    import math
    return [-2.4 * math.log(r) for r in range(1, E + 1)]


def traffic_table():
    """profiles/traffic.json: DRAM bytes per launch of the dominant kernel from the committed ncu
    summaries, keyed by (config, tokens, bits); written next to each summary, never typed in here."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(p):
        return {}
    out = {}
    for e in json.load(open(p)).get("entries", []):
        out[(int(e["config"]), int(e["tokens"]), int(e["bits"]), e["kernel"])] = e
    return out


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=float(d["hbm_gbs"]), tensor=float(d["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, tensor=1590.0, source="fallback")


def expert_bytes(H, I, bits, gs=64):
    """Packed weight + scale + bias bytes of one expert's three matrices."""
    return 3 * (H * I * bits // 8 + 2 * (H * I // gs) * 2)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) in a thread while the timed
    region runs; falls back to `nvidia-smi -lms` when NVML is not importable."""
    NAMES = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device, period_s=0.01):
        self.device, self.period = device, period_s
        self.sm, self.reasons, self.max_mhz = [], set(), None
        self._stop, self._thr, self.proc = None, None, None

    def _run(self, nv, h):
        while not self._stop.is_set():
            try:
                self.sm.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in self.NAMES.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            # NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            idx = self.device
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                idx = int(vis.split(",")[self.device])
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            self._stop = threading.Event()
            self._thr = threading.Thread(target=self._run, args=(nv, h), daemon=True)
            self._thr.start()
        except Exception:
            self._thr = None
        return self

    def __exit__(self, *a):
        if self._thr is not None:
            self._stop.set()
            self._thr.join(timeout=2)

    def summary(self):
        if not self.sm:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=["unsampled"])
        hi = [s for s in self.sm if s >= 0.5 * max(self.sm)]   # idle samples bracket the region
        return dict(sm_mhz=statistics.median(hi), sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons),
                    samples=len(self.sm))


def build_block(pkg, torch, seed, shape, device, cfg=None):
    """Seeded random-init weights of the named architecture, quantized on the GPU by the library."""
    cfg = cfg or CFG
    H, I, E = shape["hidden"], shape["inter"], shape["n_experts"]
    g = torch.Generator(device=device).manual_seed(seed)
    lin = []
    for r, c in ((I, H), (I, H), (H, I)):
        parts = []
        for e0 in range(0, E, 16):       # sixteen experts at a time bounds the float32 staging memory
            w = (torch.randn(min(16, E - e0), r, c, generator=g, device=device, dtype=torch.float32) * 0.02).bfloat16()
            parts.append(pkg.ops.quantize(w, shape["group_size"], shape["bits"]))
            del w
        wq, sc, bi = (torch.cat([p_[i] for p_ in parts]) for i in range(3))
        lin.append(pkg.nn.QuantizedSwitchLinear(wq, sc, bi, shape["group_size"], shape["bits"]))
    wr = (torch.randn(E, H, generator=g, device=device, dtype=torch.float32) * 0.02).bfloat16()
    bias = torch.tensor(zipf_bias(E), dtype=torch.float32, device=device) if cfg["zipf"] else None
    return pkg.nn.MoeBlock(wr, pkg.nn.SwitchGlu(*lin), shape["top_k"], cfg["norm_topk_prob"], cfg["router_mode"], bias)


def time_steps(torch, fn, steps, warmup, flush):
    """-> list of per-step milliseconds (CUDA events on the current stream, L2 flushed in between)."""
    for _ in range(warmup):
        flush()
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        flush()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


def cpu_block_inputs(T_sample, shape, cfg, seed):
    """Seeded CPU-side inputs of the oracle block: every expert distinct, drawn and quantized one expert
    at a time so that only the packed weights stay in memory."""
    import numpy as np
    import torch
    from oracle import oracle as O
    H, I, E = shape["hidden"], shape["inter"], shape["n_experts"]
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T_sample, H, generator=g).bfloat16().float().numpy()
    wr = (torch.randn(E, H, generator=g) * 0.02).bfloat16().float().numpy()
    q = []
    for r, c in ((I, H), (I, H), (H, I)):
        parts = [O.quantize((torch.randn(1, r, c, generator=g) * 0.02).bfloat16().float().numpy(), shape["group_size"],
                            shape["bits"]) for _ in range(E)]
        q.append(tuple(np.concatenate([p_[i] for p_ in parts]) for i in range(3)))
    bias = np.asarray(zipf_bias(E), dtype=np.float32) if cfg["zipf"] else None
    return x, wr, q, bias


def cpu_sample_tokens(T, shape):
    """Tokens of the bounded CPU sample: about 4e10 flop per forward (a fraction of a second to a few
    seconds on the host cores), at most 512 tokens."""
    per_token = shape["top_k"] * 3 * 2 * shape["hidden"] * shape["inter"]
    return int(max(8, min(T, 512, 4e10 // per_token)))


def cpu_forward_timer(T_sample, shape, cfg, seed):
    """-> (callable running one oracle forward of the sample and returning its seconds, thread count)."""
    from oracle import oracle as O
    O.set_num_threads(0)   # all host cores, also when a launcher exported OMP_NUM_THREADS=1
    x, wr, q, bias = cpu_block_inputs(T_sample, shape, cfg, seed)
    k = shape["top_k"]

    def once():
        t0 = time.perf_counter()
        O.moe_block(x, wr, q[0], q[1], q[2], k, cfg["router_mode"], cfg["norm_topk_prob"], bias, shape["group_size"],
                    shape["bits"])
        return time.perf_counter() - t0
    return once, O.num_threads()


def cpu_baseline(T, shape, cfg, seed, reps_budget_s=15.0):
    """Times the CPU oracle (a port: the reference's MLX CPU path cannot be built here) on the host
    cores on a bounded sample of the workload: forwards of a `cpu_sample_tokens`-token block."""
    Ts = cpu_sample_tokens(T, shape)
    once, cores = cpu_forward_timer(Ts, shape, cfg, seed)
    once()  # warm-up
    t, n = 0.0, 0
    while t < reps_budget_s and n < 50:
        t += once()
        n += 1
    return dict(value=Ts * n / t, unit=UNIT, cores=cores, kind="port",
                sample=f"{n} forwards of a {Ts}-token block of the same layer (all {shape['n_experts']} experts distinct), "
                       f"{t:.1f} s, OpenMP on all host threads")


def layer_config(T, shape, **extra):
    """The `config` object of the JSON line: the same keys for both arms."""
    d = dict(workload=workload_name(T), tokens=T)
    d.update(extra)
    d.update(shape)
    d.update(router_mode=CFG["router_mode"], norm_topk_prob=CFG["norm_topk_prob"], zipf_skew=CFG["zipf"])
    return d


def run_reference(args):
    """Reference arm: the CPU oracle (port of the reference semantics; the reference itself is a
    Rust binding over an absent MLX and cannot be built) on all host threads, same config.  One
    step = one forward of a bounded sample of the workload (`sample_tokens` tokens of the same
    layer); `ms_per_step` is what that sample forward took, `value` the tokens/s it achieved, and
    `extrapolated` says what a full step would take at that rate (linear in the token count)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.tokens
    Ts = cpu_sample_tokens(T, SHAPE)
    once, cores = cpu_forward_timer(Ts, SHAPE, CFG, args.seed)
    for _ in range(args.warmup):
        once()
    secs = [once() for _ in range(args.steps)]
    ms = 1e3 * statistics.mean(secs)
    v = Ts / (ms * 1e-3)
    sample = (f"{args.steps} forwards of a {Ts}-token block of the same layer (all {SHAPE['n_experts']} experts distinct), "
              f"{sum(secs):.1f} s, OpenMP on all host threads")
    line = dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32",
                data="synthetic", impl="reference",
                config=layer_config(T, SHAPE, l2="not applicable (host cores)", parallelism=f"{cores} host threads",
                                    cuda_graph=False),
                sample_tokens=Ts, sample_ms=ms,
                extrapolated=dict(is_extrapolated=Ts != T, full_step_tokens=T, full_step_ms=ms * T / Ts,
                                  rule="linear in the token count"),
                cpu_baseline=dict(value=v, unit=UNIT, cores=cores, kind="port", sample=sample),
                e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def workload_name(T):
    return CFG["name"].format(T=T, bits=SHAPE["bits"])


def run_stack(args, pkg, torch, dev, peaks):
    """BASELINE.json configs[2]: 48 pre-RMSNorm MoE blocks with residuals, a 2048-token prefill followed
    by 256 single-token decode steps (each step feeds the previous output row back in).  One bench
    step = the whole sequence.  The decode step (48 layers, ~390 kernels) is replayed from a CUDA graph."""
    import statistics as st
    n_layers, t_prefill, n_decode = args.layers, 2048, 256
    H = SHAPE["hidden"]
    ctx = pkg.default_context()
    blocks = [build_block(pkg, torch, args.seed + l, SHAPE, dev) for l in range(n_layers)]
    stack = pkg.nn.MoeStack(blocks, eps=1e-6)
    ctx.reserve(blocks[0].config, t_prefill)
    g = torch.Generator(device=dev).manual_seed(args.seed + 99)
    xp = torch.randn(t_prefill, H, generator=g, device=dev, dtype=torch.float32).bfloat16()
    xd = torch.zeros(1, H, dtype=torch.bfloat16, device=dev)
    holder = {}

    def decode_step():
        holder["o"] = stack.forward(xd)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        decode_step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        decode_step()

    def sequence():
        out = stack.forward(xp)
        xd.copy_(out[-1:])
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(n_decode):
            graph.replay()
            xd.copy_(holder["o"])
        ev1.record()
        return ev0, ev1
    for _ in range(max(1, args.warmup // 3)):
        sequence()
    torch.cuda.synchronize()
    tot, dec = [], []
    l0 = ctx.launch_count()
    with ClockSampler(dev.index or 0) as clk:
        for _ in range(args.steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            e0, e1 = sequence()
            b.record()
            torch.cuda.synchronize()
            tot.append(a.elapsed_time(b))
            dec.append(e0.elapsed_time(e1))
    ms, dms = st.mean(tot), st.mean(dec)
    we = expert_bytes(H, SHAPE["inter"], SHAPE["bits"])
    dec_bytes = n_layers * (SHAPE["top_k"] * we + SHAPE["n_experts"] * H * 2)
    line = dict(metric=METRIC, value=(t_prefill + n_decode) / (ms * 1e-3), unit=UNIT, n_gpus=1, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                data="synthetic",
                config=dict(workload=f"configs[2]: {n_layers} x (RMSNorm eps 1e-6 + MoE block + residual), 2048-token prefill "
                                     "then 256 decode steps", l2="working set 16 GB per pass, far larger than L2",
                            parallelism="single GPU", cuda_graph="decode steps", **SHAPE),
                prefill=dict(tokens=t_prefill, ms=ms - dms, tokens_per_s=t_prefill / ((ms - dms) * 1e-3)),
                decode=dict(steps=n_decode, ms_per_token=dms / n_decode, tokens_per_s=n_decode / (dms * 1e-3),
                            hbm_gbs=dec_bytes / (dms / n_decode * 1e-3) / 1e9,
                            frac_hbm=dec_bytes / (dms / n_decode * 1e-3) / 1e9 / peaks["hbm"]),
                roofline=dict(bound="hbm", achieved=dec_bytes / (dms / n_decode * 1e-3) / 1e9, peak=peaks["hbm"], unit="GB/s",
                              frac=dec_bytes / (dms / n_decode * 1e-3) / 1e9 / peaks["hbm"], traffic=None,
                              peak_source=peaks["source"], kernel="whole 48-layer decode step (all kernels)"),
                cpu_baseline=None, e2e=None, gpu_launches=ctx.launch_count() - l0, clocks=clk.summary())
    print(json.dumps(line))


def run_gather_mm(args, pkg, torch, dev, peaks):
    """ops.gather_mm (mlx-rs/src/ops/arithmetic.rs:1568-1632) on un-quantised bf16 experts of the config's gate shape:
    a [T*k, 1, H], b [E, H, I], uniformly random rhs indices -> [T*k, 1, I].  Side measurement (row f1 of the
    scope table), not the headline metric: one JSON line with the whole-call time (index expansion, sort, row
    gather, grouped tcgen05 product) against the measured dense bf16 peak."""
    H, I, E, k = (SHAPE[n] for n in ("hidden", "inter", "n_experts", "top_k"))
    rows = args.tokens * k
    g = torch.Generator(device=dev).manual_seed(args.seed)
    a = (torch.randn(rows, 1, H, generator=g, device=dev) / 8).bfloat16()
    b = (torch.randn(E, H, I, generator=g, device=dev) / 8).bfloat16()
    rhs = torch.randint(0, E, (rows,), generator=g, device=dev, dtype=torch.int32)
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    ctx = pkg.default_context()
    l0 = ctx.launch_count()
    with ClockSampler(dev.index or 0) as clk:
        times = time_steps(torch, lambda: pkg.ops.gather_mm(a, b, None, rhs), args.steps, args.warmup,
                           lambda: flush_buf.fill_(1))
    ctx.check()
    out = pkg.ops.gather_mm(a, b, None, rhs)
    idx = torch.randint(0, rows, (256,), generator=g, device=dev)
    ref = torch.einsum("rk,rkn->rn", a[idx, 0].float(), b[rhs[idx].long()].float())
    err = float((out[idx, 0].float() - ref).abs().max() / ref.abs().max())
    ms = statistics.mean(times)
    flops = 2.0 * rows * H * I
    print(json.dumps(dict(metric="gather_mm_tflops", value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s", n_gpus=1, steps=args.steps,
                          warmup=args.warmup, ms_per_step=ms, higher_is_better=True, dtype="bf16", data="synthetic",
                          config=dict(workload=f"gather_mm a[{rows},1,{H}] x b[{E},{H},{I}], random rhs indices",
                                      l2="flushed between iterations (512 MB overwrite)"),
                          roofline=dict(bound="tensor", achieved=flops / (ms * 1e-3) / 1e12, peak=peaks["tensor"], unit="TFLOP/s",
                                        frac=flops / (ms * 1e-3) / 1e12 / peaks["tensor"], traffic=None,
                                        peak_source=peaks["source"], kernel="whole gather_mm call"),
                          check=dict(rows_sampled=256, max_rel_err_vs_float32=err),
                          gpu_launches=(ctx.launch_count() - l0) // (args.steps + args.warmup + 1) * args.steps,
                          clocks=clk.summary())))


def main():
    global SHAPE, CFG
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=1, choices=[1, 2, 3, 4],
                    help="BASELINE.json configs index: 1 = Qwen3-30B-A3B layer (default, the metric's configuration), "
                         "2 = its 48-layer stack, 3 = Qwen3-235B-A22B layer, 4 = Mixtral layer with skewed routing")
    ap.add_argument("--bits", type=int, default=None, choices=[4, 8], help="weight bits (configs[4] asks for both)")
    ap.add_argument("--workload", default=None, choices=["layer", "stack", "gather_mm"],
                    help="layer: one MoE layer; stack: configs[2] (implied by --config 2); gather_mm: the un-quantised "
                         "gathered product (the op behind a bf16 SwitchLinear) at the config's gate shape, tokens x top_k rows")
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=None, help="tokens per step per GPU (default: the config's)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the step from a CUDA graph (auto: for steps of at most 1024 tokens)")
    ap.add_argument("--ep-transport", default="device", choices=["device", "peer", "peer_push", "nccl"],
                    help="N > 1: device = the one-call block (dispatch and combine kernels over peer memory, phases ordered "
                         "on the device, no host synchronisation); peer = the same kernels ordered by NCCL collectives with "
                         "one host synchronisation per step; peer_push = dispatch kernel + down projection whose epilogue "
                         "stores the rows back into the source GPU; nccl = torch.distributed all-to-all-v (the baseline)")
    ap.add_argument("--ep-chunks", type=int, default=0, choices=[0, 1, 2],
                    help="N > 1: halves of a rank's tokens whose exchange overlaps the other half's products "
                         "(0 = default: one)")
    ap.add_argument("--qmm-path", default="auto", choices=["auto", "small", "tensor_core"],
                    help="pin the grouped-product kernel (default: the library chooses)")
    args = ap.parse_args()
    CFG = CONFIGS[args.config]
    SHAPE = dict(CFG["shape"])
    if args.bits:
        SHAPE["bits"] = args.bits
    if args.tokens is None:
        args.tokens = CFG["tokens"]
    if args.workload is None:
        args.workload = "stack" if args.config == 2 else "layer"
    args.config_id = args.config
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import __graft_entry__ as ge
    pkg = ge.load_package()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    T = args.tokens
    H, I, E, k, bits = (SHAPE[n] for n in ("hidden", "inter", "n_experts", "top_k", "bits"))

    if world > 1:
        from importlib import import_module
        ep = import_module("mlx_rs_b200.ep")
        if args.workload == "stack":
            return ep.bench_stack(args, pkg, SHAPE, CFG, peaks, METRIC, UNIT, ClockSampler)
        return ep.bench_main(args, pkg, SHAPE, CFG, peaks, METRIC, UNIT, workload_name, ClockSampler, zipf_bias)

    if args.workload == "stack":
        return run_stack(args, pkg, torch, dev, peaks)
    if args.workload == "gather_mm":
        return run_gather_mm(args, pkg, torch, dev, peaks)
    ctx = pkg.default_context()
    ctx.set_qmm_path(dict(auto=ctx.QMM_AUTO, small=ctx.QMM_SMALL, tensor_core=ctx.QMM_TENSOR_CORE)[args.qmm_path])
    block = build_block(pkg, torch, args.seed, SHAPE, dev)
    do_sweep = args.config == 1 and bits == 4 and not args.no_sweep
    ctx.reserve(block.config, max(T, max(SWEEP)) if do_sweep else T)
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def flush():
        flush_buf.fill_(1)

    g = torch.Generator(device=dev).manual_seed(args.seed + 1)
    decode_below = 1024      # steps below this many tokens are reported against the HBM roofline

    def point(Tp, steps, warmup, profile):
        x = torch.randn(Tp, H, generator=g, device=dev, dtype=torch.float32).bfloat16()
        out_holder = {}

        def eager_step():
            out_holder["o"] = block.forward(x)
        l0 = ctx.launch_count()
        eager_step()
        launches = ctx.launch_count() - l0
        # Decode-sized steps are launch-bound when driven call by call from Python; like a serving
        # loop would, the timed step replays a CUDA graph of the same library call (same kernels,
        # same inputs resident in HBM).  Prefill-sized steps run eagerly.
        use_graph = args.graph == "on" or (args.graph == "auto" and Tp <= 1024)
        step = eager_step
        if use_graph:
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for _ in range(2):
                    eager_step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                eager_step()
            step = graph.replay
        ms = time_steps(torch, step, steps, warmup, flush)
        res = dict(tokens=Tp, ms_per_step=statistics.mean(ms), ms_min=min(ms), launches_per_step=launches,
                   cuda_graph=use_graph)
        res["tokens_per_s"] = Tp / (res["ms_per_step"] * 1e-3)
        # routing actually taken -> algorithmic bytes of this batch
        _, aux = block.forward(x, return_aux=True)
        counts = aux["counts"].cpu()
        n_act = int((counts > 0).sum())
        res["active_experts"] = n_act
        res["max_expert_share"] = float(counts.max()) / max(1, int(counts.sum()))
        we = expert_bytes(H, I, bits)
        res["block_bytes"] = n_act * we + E * H * 2 + 2 * Tp * H * 2
        res["block_flops"] = Tp * (k * 3 * 2 * H * I + 2 * H * E)
        res["block_gbs"] = res["block_bytes"] / (res["ms_per_step"] * 1e-3) / 1e9
        res["block_tflops"] = res["block_flops"] / (res["ms_per_step"] * 1e-3) / 1e12
        if profile:
            ctx.set_profiling(True)
            stage = {n: [] for n in ctx.STAGES}
            for _ in range(max(3, steps)):
                flush()
                block.forward(x)
                for n, v in ctx.stage_ms().items():
                    stage[n].append(v)
            ctx.set_profiling(False)
            res["stage_ms"] = {n: statistics.mean(v) for n, v in stage.items()}
            gu_ms = res["stage_ms"]["gate_up"]
            gu_bytes = n_act * (we * 2 // 3) + Tp * k * H * 2 + Tp * k * I * 2
            gu_flops = Tp * k * 2 * 2 * H * I
            res["gate_up"] = dict(ms=gu_ms, bytes=gu_bytes, flops=gu_flops, gbs=gu_bytes / (gu_ms * 1e-3) / 1e9,
                                  tflops=gu_flops / (gu_ms * 1e-3) / 1e12)
            dn_ms = res["stage_ms"]["down"]
            dn_flops = Tp * k * 2 * H * I
            res["down"] = dict(ms=dn_ms, flops=dn_flops, tflops=dn_flops / (dn_ms * 1e-3) / 1e12)
        return res, x

    with ClockSampler(local) as clk:
        main_res, x_main = point(T, args.steps, args.warmup, True)
    clocks = clk.summary()

    # end to end through the public API with host buffers
    xh = x_main.cpu().pin_memory()
    oh = torch.empty_like(xh).pin_memory()
    xd = torch.empty_like(x_main)

    def e2e_step():
        xd.copy_(xh, non_blocking=True)
        o = block.forward(xd)
        oh.copy_(o, non_blocking=True)
    serial_ms = time_steps(torch, e2e_step, max(3, args.steps // 4), 3, flush)
    # The serving form of the same call: HostPipeline overlaps step i+1's upload and step i-1's
    # download with step i's kernels.  Every step's upload and download is inside the timed
    # region; all K steps are timed as one region (they overlap, so per-step events mean nothing).
    # L2: each step streams the layer's weights and its intermediates, far more than the 126 MB L2.
    pipe = pkg.nn.HostPipeline(block, T, H, dev, depth=2)
    xhs = [xh, xh.clone().pin_memory()]
    ohs = [oh, torch.empty_like(oh).pin_memory()]
    for i in range(max(3, args.warmup)):
        pipe.submit(xhs[i % 2], ohs[i % 2])
    pipe.drain()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        pipe.submit(xhs[i % 2], ohs[i % 2])
    pipe.drain()
    ev1.record()
    torch.cuda.synchronize()
    ctx.check()
    e2e_step_ms = ev0.elapsed_time(ev1) / args.steps
    e2e = dict(value=T / (e2e_step_ms * 1e-3), unit=UNIT, h2d_bytes_per_step=xh.numel() * 2,
               d2h_bytes_per_step=oh.numel() * 2, ms_per_step=e2e_step_ms, pipeline="HostPipeline depth 2",
               unpipelined_value=T / (statistics.mean(serial_ms) * 1e-3))

    sweep = []
    if do_sweep:
        for Tp in SWEEP:
            if Tp == T:
                r = main_res
            else:
                r, _ = point(Tp, max(5, min(args.steps, 10)), 3, True)
            gu = r["gate_up"]
            decode = Tp < decode_below
            fused = r["launches_per_step"] == 1      # a whole block in one launch would have no per-stage split
            sweep.append(dict(tokens=Tp, tokens_per_s=r["tokens_per_s"], ms=r["ms_per_step"], cuda_graph=r["cuda_graph"],
                              active_experts=r["active_experts"], launches=r["launches_per_step"], single_launch=fused,
                              block_frac_hbm=r["block_gbs"] / peaks["hbm"], block_frac_tensor=r["block_tflops"] / peaks["tensor"],
                              gate_up_ms=None if fused else gu["ms"],
                              gate_up_frac=None if fused else ((gu["gbs"] / peaks["hbm"]) if decode else (gu["tflops"] / peaks["tensor"])),
                              bound="hbm" if decode else "tensor", stage_ms=None if fused else r["stage_ms"]))

    gu = main_res["gate_up"]
    if main_res["launches_per_step"] == 1:     # single-launch block: the dominant kernel is the whole step
        roof = dict(bound="hbm", achieved=main_res["block_gbs"], peak=peaks["hbm"], unit="GB/s",
                    frac=main_res["block_gbs"] / peaks["hbm"], block_frac=main_res["block_gbs"] / peaks["hbm"])
        gu = dict(ms=main_res["ms_per_step"], bytes=main_res["block_bytes"], flops=main_res["block_flops"])
    elif T < decode_below:
        roof = dict(bound="hbm", achieved=gu["gbs"], peak=peaks["hbm"], unit="GB/s", frac=gu["gbs"] / peaks["hbm"],
                    block_frac=main_res["block_gbs"] / peaks["hbm"])
    else:
        roof = dict(bound="tensor", achieved=gu["tflops"], peak=peaks["tensor"], unit="TFLOP/s",
                    frac=gu["tflops"] / peaks["tensor"], block_frac=main_res["block_tflops"] / peaks["tensor"],
                    down_frac=main_res["down"]["tflops"] / peaks["tensor"])
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this size, from the ncu
    # capture summarised under profiles/ (a profiler cannot run inside the timed bench)
    tr = traffic_table().get((args.config_id, T, bits, "gate_up"))
    roof.update(kernel="whole block, one launch" if main_res["launches_per_step"] == 1 else "gate+up grouped quantized GEMM (dominant)",
                peak_source=peaks["source"],
                traffic=(tr["dram_bytes_per_launch"] if tr else None), traffic_source=(tr["profile"] if tr else None),
                kernel_ms=gu["ms"], algorithmic_bytes=gu["bytes"], algorithmic_flops=gu["flops"])

    base = None if args.no_cpu_baseline else cpu_baseline(T, SHAPE, CFG, args.seed)
    line = dict(metric=METRIC, value=main_res["tokens_per_s"], unit=UNIT, n_gpus=1, steps=args.steps, warmup=args.warmup,
                ms_per_step=main_res["ms_per_step"], higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                data="synthetic",
                config=layer_config(T, SHAPE, l2="flushed between iterations (512 MB overwrite)", parallelism="single GPU",
                                    cuda_graph=main_res["cuda_graph"]),
                roofline=roof, cpu_baseline=base, e2e=e2e, gpu_launches=main_res["launches_per_step"] * args.steps,
                clocks=clocks, block=dict(active_experts=main_res["active_experts"],
                                          max_expert_share=main_res["max_expert_share"], gbs=main_res["block_gbs"],
                                          tflops=main_res["block_tflops"], stage_ms=main_res["stage_ms"]),
                sweep=sweep)
    print(json.dumps(line))


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the quantised MoE FFN block (decode), one JSON line on rank 0.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (synthetic, seeded): the Qwen3-Next MoE block with Q4_K_M-style mixed quantisation --
hidden 2048, 512 routed experts (gate/up Q4_K [512x2048], down Q6_K [2048x512]), top-10, one
Q8_0 shared expert with a sigmoid gate, f32 router -- at decode batch 64 per GPU, bf16 inputs
~N(0,1), uniform random routing.  A step is one forward of one block; consecutive steps use
different, independently seeded layers so that the weights of a step are never in L2.

N = 1: the whole block on one GPU.  N > 1: expert parallelism, 512/N experts per GPU, every
rank home to 64 tokens (weak scaling), dispatch/combine over NCCL.

`value` is tokens/s with the inputs resident in HBM; `e2e` is the same metric through the
host-buffer entry point (host->device copy of x and device->host copy of the result inside
the timed region).  `--impl reference` times the CPU restatement of the reference's own CPU
path (oracle/) on the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Q4_K MoE layer tokens/s (decode)"
UNIT = "tokens/s"
H, F, E, TOPK = 2048, 512, 512, 10
PRESET = "q4k_m"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="pmoe", choices=["pmoe", "reference"])
    ap.add_argument("--batch", type=int, default=64, help="decode tokens per GPU per step")
    ap.add_argument("--layers", type=int, default=4, help="distinct layers cycled through")
    ap.add_argument("--no-sweep", action="store_true", help="skip the batch 1/4/16 sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--no-graph", action="store_true", help="do not try CUDA-graph replay of the block")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--ep-mode", default="all_gather", choices=["all_to_all", "all_gather"])
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill"],
                    help="decode: the headline workload; prefill: 4096 tokens, Zipf-skewed routing, one GPU")
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per step in prefill mode")
    ap.add_argument("--preset", default="q4k_q6k_all",
                    help="prefill mode: dtype mix of the layer (paramecia_b200.synth.PRESETS), e.g. q4k_m for a Q8_0 shared expert")
    return ap.parse_args()


def workload_name(batch, n_gpus):
    s = (f"qwen3next-moe-block q4k_m (gate/up Q4_K, down Q6_K, shared Q8_0) H{H} F{F} E{E} top{TOPK}, "
         f"decode batch {batch}/GPU, bf16 x, uniform routing")
    if n_gpus > 1:
        s += f", expert-parallel {E // n_gpus} experts/GPU"
    return s


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.path = None
        self.skip = 0

    def mark(self):
        """Samples taken so far (while the layers were being built, the GPU idle) do not count."""
        try:
            self.skip = sum(1 for _ in open(self.path))
        except Exception:
            self.skip = 0

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.idx)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            lines = open(self.path).read().splitlines()
            window = lines[self.skip:]
            if not any(len(l.split(",")) >= 9 for l in window):
                window = lines   # a run shorter than the sampling period: fall back to every sample of the process
                out["window"] = "whole process (the marked region held no sample)"
            for line in window:
                p = [c.strip() for c in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1])); mx.append(float(p[2]))
                except ValueError:
                    continue
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                                  ("sw_power_cap", 8)):
                    if p[col].lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_cpu_baseline(layer_host, batch, seconds, seed=1234):
    """Times the oracle (the port of the reference's CPU path) on whole-block forwards of `batch` tokens."""
    import torch
    from oracle import pmoe_oracle as po
    from tests.common import oracle_layer
    ol = oracle_layer(layer_host)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((batch, H), generator=g).to(torch.bfloat16).float().numpy()
    ol.forward(x)  # warm-up (page in the weights)
    t0 = time.perf_counter()
    reps = 0
    while True:
        ol.forward(x)
        reps += 1
        el = time.perf_counter() - t0
        if el >= seconds or reps >= 50:
            break
    return dict(value=batch * reps / el, unit=UNIT, cores=po.max_threads(), kind="port",
                sample=f"{reps} whole-block forwards of batch {batch} on one layer, {el:.1f} s; "
                       f"C restatement of the reference CPU path ({po.simd_kind()}), OpenMP over experts and rows",
                ms_per_step=1e3 * el / reps)


def reference_arm(args, rank):
    """--impl reference: the CPU restatement of the reference's own CPU path on the host cores."""
    if rank != 0:
        return
    import torch
    from paramecia_b200 import synth
    layer = synth.make_layer(H, F, E, TOPK, PRESET, seed=0, device="cpu", layer=0)
    from oracle import pmoe_oracle as po
    from tests.common import oracle_layer
    ol = oracle_layer(layer)
    batch = args.batch * args.gpus
    g = torch.Generator().manual_seed(99)
    x = torch.randn((batch, H), generator=g).to(torch.bfloat16).float().numpy()
    steps = max(1, min(args.steps, 20))
    warm = max(1, min(args.warmup, 2))
    for _ in range(warm):
        ol.forward(x)
    t0 = time.perf_counter()
    for _ in range(steps):
        ol.forward(x)
    el = time.perf_counter() - t0
    val = batch * steps / el
    line = dict(metric=METRIC, value=val, unit=UNIT, n_gpus=args.gpus, steps=steps, warmup=warm,
                ms_per_step=1e3 * el / steps, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="int8 x int4/6/8 block dots, f32 accumulate", data="synthetic", impl="reference",
                config=dict(workload=workload_name(args.batch, args.gpus), global_batch=batch,
                            note="the Rust reference cannot be built here (no cargo, candle fork not vendored); "
                                 "this is the C restatement of its CPU path in oracle/"),
                cpu_baseline=dict(value=val, unit=UNIT, cores=po.max_threads(), kind="port",
                                  sample=f"{steps} whole-block forwards of batch {batch}, one layer, all host threads"),
                e2e=dict(value=val, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 439.356672 / 429.555712   # gate/up launch, batch 64 (see profiles/)


def prefill_main(args):
    """Benchmark configuration 3 (prefill) on one GPU: 4096 bf16 tokens through one Q4_K / Q6_K block whose router carries the
    bias 2*ln(1/rank_e) (rank = seeded permutation), so a dozen experts take most tokens.  Reports tokens/s and the
    tensor-core roofline of the gate/up grouped GEMM (tcgen05 kind::i8, two digit MMAs per algorithmic MMA)."""
    import torch
    import paramecia_b200 as pm
    from paramecia_b200 import synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    tpeak = float(peaks.get("bf16_tflops", 1590.0))
    n = args.tokens
    nl = max(1, min(args.layers, 2))
    blocks = [synth.make_block(synth.make_layer(H, F, E, TOPK, args.preset, seed=0, device=dev, layer=li, zipf=True),
                               dev, max_tokens=n) for li in range(nl)]
    g = torch.Generator(device=dev).manual_seed(11)
    xs = [torch.randn((n, H), generator=g, device=dev).to(torch.bfloat16) for _ in range(2)]
    out = torch.empty((n, H), dtype=torch.bfloat16, device=dev)
    W = max(args.warmup, 3)
    steps = min(args.steps, 50)
    sampler = ClockSampler(0)
    sampler.start()
    for i in range(2):   # (first touches; nvidia-smi comes up meanwhile)
        blocks[i % nl].forward_into(xs[i % 2], out)
    torch.cuda.synchronize()
    sampler.mark()       # window: warm-up and timed steps, the same load
    for i in range(W):
        blocks[i % nl].forward_into(xs[i % 2], out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = pm.launch_count()
    e0.record()
    for i in range(steps):
        blocks[i % nl].forward_into(xs[i % 2], out)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    launches = pm.launch_count() - before
    for b in blocks:
        b.status()
    phase = {}
    reps = min(steps, 10)
    blocks[0].trace(True)
    for i in range(reps):
        blocks[0].forward_into(xs[0], out)
        for k_, v in blocks[0].trace_read().items():
            phase[k_] = phase.get(k_, 0.0) + v / reps
    blocks[0].trace(False)
    _, _, idx = blocks[0].route(xs[0])
    counts = torch.bincount(idx.flatten().long(), minlength=E)
    rows = n * TOPK + n
    gu_flops = rows * 2 * 2 * H * F
    ach = gu_flops / (phase["gate_up"] * 1e-3) / 1e12
    xh = xs[0].cpu().pin_memory()
    oh = torch.empty((n, H), dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        blocks[0].forward_host(xh, oh)
    t0 = time.perf_counter()
    for i in range(steps):
        blocks[i % nl].forward_host(xh, oh)
    el = (time.perf_counter() - t0) / steps
    line = dict(metric="Q4_K MoE layer tokens/s (prefill)", value=n / (ms * 1e-3), unit=UNIT, n_gpus=1, steps=steps,
                warmup=W, ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="int8 digit MMAs (gate/up, exact) + fp16 MMAs (down), f32 accumulate", data="synthetic",
                config=dict(workload=f"qwen3next-moe-block preset {args.preset} (gate/up Q4_K, down Q6_K) H{H} F{F} E{E} "
                                     f"top{TOPK}, prefill {n} bf16 tokens, Zipf-biased router",
                            active_experts=int((counts > 0).sum()), max_tokens_per_expert=int(counts.max()),
                            layers_cycled=nl, block_tflops=n * 71303168 / (ms * 1e-3) / 1e12),
                roofline=dict(bound="tensor", kernel="k_gu_prefill", achieved=ach, peak=tpeak, unit="TFLOP/s",
                              frac=ach / tpeak, traffic=None, peak_kind="measured bf16 burst (MEASURED_PEAKS.json)",
                              algorithmic_flops_per_launch=gu_flops, us_per_launch=phase["gate_up"] * 1e3,
                              phases_us={k_: round(v * 1e3, 1) for k_, v in phase.items()}),
                cpu_baseline=None,
                e2e=dict(value=n / el, unit=UNIT, h2d_bytes_per_step=n * H * 2, d2h_bytes_per_step=n * H * 2,
                         ms_per_step=el * 1e3),
                gpu_launches=launches, clocks=clocks)
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    if args.mode == "prefill" and args.impl != "reference":
        prefill_main(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    import torch
    import torch.distributed as dist
    import paramecia_b200 as pm
    from paramecia_b200 import synth

    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()   # early: nvidia-smi takes a moment to come up; idle samples are dropped by mark()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    N = world
    batch = args.batch
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"

    # ---- layers: every rank builds the same seeded layers and keeps its slice of the experts
    E_local = E // N
    max_tok = batch * N if N > 1 else max(batch, 64)
    blocks, host_layer0 = [], None
    for li in range(args.layers):
        t = synth.make_layer(H, F, E, TOPK, PRESET, seed=0, device=dev, layer=li)
        if li == 0 and rank == 0 and not args.no_cpu:
            host_layer0 = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in t.items()}
            host_layer0["shared"] = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in t["shared"].items()}
        blocks.append(synth.make_block(t, dev, max_tokens=max_tok, expert_base=rank * E_local, E_local=E_local))
        del t
    torch.cuda.synchronize()

    if N > 1:
        from paramecia_b200.ep import ExpertParallelMoe
        eps = [ExpertParallelMoe(b, mode=args.ep_mode) for b in blocks]

    def make_x(n, seed):
        g = torch.Generator(device=dev).manual_seed(seed + 7919 * rank)
        return torch.randn((n, H), generator=g, device=dev).to(torch.bfloat16)

    def barrier():
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def time_steps(n_tok, steps, warmup):
        """Device time (ms) of `steps` forwards of n_tok tokens per GPU, layers cycled; max over ranks."""
        xs = [make_x(n_tok, 100 + i) for i in range(4)]
        out = torch.empty((n_tok, H), dtype=torch.bfloat16, device=dev)

        def step(i):
            b = i % len(blocks)
            if N > 1:
                eps[b].forward_into(xs[i % 4], out)
            else:
                blocks[b].forward_into(xs[i % 4], out)
        for i in range(warmup):
            step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = pm.launch_count()
        e0.record()
        for i in range(steps):
            step(warmup + i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        launches = pm.launch_count() - before
        if N > 1:
            tms = torch.tensor([ms], device=dev)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            ms = float(tms.item())
        return ms, launches

    def time_steps_graph(n_tok, steps, warmup):
        """Same steps replayed from one CUDA graph that holds one forward per layer (single GPU)."""
        nb = len(blocks)
        xs = [make_x(n_tok, 100 + i) for i in range(nb)]
        out = torch.empty((n_tok, H), dtype=torch.bfloat16, device=dev)
        fwd = [(eps[i].forward_into if N > 1 else blocks[i].forward_into) for i in range(nb)]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for i in range(nb):
                fwd[i](xs[i], out)
        torch.cuda.current_stream(dev).wait_stream(side)
        barrier()
        g = torch.cuda.CUDAGraph()
        before_cap = pm.launch_count()
        with torch.cuda.graph(g):
            for i in range(nb):
                fwd[i](xs[i], out)
        per_replay = pm.launch_count() - before_cap
        # exactly `steps` forwards are timed: whole replays plus, for the remainder, a second graph
        reps, rem = steps // nb, steps % nb
        g_rem = None
        if rem:
            g_rem = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_rem):
                for i in range(rem):
                    fwd[i](xs[i], out)
        for _ in range(max(1, -(-warmup // nb))):
            g.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        if g_rem is not None:
            g_rem.replay()
        e1.record()
        barrier()
        g_ms = e0.elapsed_time(e1)
        if N > 1:
            t_ = torch.tensor([g_ms], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            g_ms = float(t_.item())
        return g_ms, steps, per_replay * reps + (per_replay // nb) * rem

    def distinct_experts(n_tok):
        """Average number of distinct local experts a step touches (for the algorithmic bytes)."""
        tot = 0
        for i in range(4):
            x = make_x(n_tok, 100 + i)
            if N > 1:
                x = eps[0].gather_tokens(x)
            _, _, idx = blocks[i % len(blocks)].route(x)
            idx = idx.to(torch.int64)
            loc = idx[(idx >= rank * E_local) & (idx < (rank + 1) * E_local)]
            tot += int(torch.unique(loc).numel())
        return tot / 4.0

    W = max(args.warmup, 3)
    if rank == 0:
        sampler.mark()   # window: warm-up, the timed steps and their graph replay (all the same load)
    ms, launches = time_steps(batch, args.steps, W)
    ms_per_step = ms / args.steps
    value = batch * N * args.steps / (ms * 1e-3)
    launch_mode = "direct C-ABI calls"
    direct = dict(tokens_per_s=value, ms_per_step=ms_per_step)
    steps_done = args.steps
    if not args.no_graph:
        g_ms, g_steps, g_launches = time_steps_graph(batch, args.steps, W)
        if g_ms / g_steps < ms_per_step:
            ms, ms_per_step, steps_done, launches = g_ms, g_ms / g_steps, g_steps, g_launches
            value = batch * N * g_steps / (g_ms * 1e-3)
            launch_mode = f"CUDA graph holding one forward per layer ({len(blocks)}), replayed"
    clocks = sampler.stop() if rank == 0 else {}

    # ---- roofline of the dominant kernel (gate/up GEMV): traced pass, events around each kernel
    D = distinct_experts(batch)
    blk0 = blocks[0]
    d = blk0._desc
    gu_bytes = D * F * (pm.row_bytes(d.gate_dtype, H) + pm.row_bytes(d.up_dtype, H))
    gu_bytes += F * (pm.row_bytes(d.sh_gate_dtype, H) + pm.row_bytes(d.sh_up_dtype, H))
    step_bytes = blk0.weight_bytes(int(round(D))) + batch * H * 4  # weights + x in + out (bf16 each)
    phase_ms = {}
    reps = min(args.steps, 50)
    if N == 1:
        x = make_x(batch, 5)
        out = torch.empty((batch, H), dtype=torch.bfloat16, device=dev)
        for b in blocks:
            b.trace(True)
        for i in range(reps + 3):
            b = blocks[i % len(blocks)]
            b.forward_into(x, out)
            t = b.trace_read()
            if i >= 3:
                for k_, v in t.items():
                    phase_ms[k_] = phase_ms.get(k_, 0.0) + v / reps
        for b in blocks:
            b.trace(False)
    else:
        # expert-parallel: time this rank's expert kernels on the rows the dispatch delivered
        out = torch.empty((batch, H), dtype=torch.bfloat16, device=dev)
        for i, e in enumerate(eps):
            e.forward_into(make_x(batch, 5 + i), out)
        for b in blocks:
            b.trace(True)
        for i in range(reps + 3):
            e = eps[i % len(eps)]
            e.block.experts_forward_batched(e.recv_x, e.recv_idx, e.recv_w, TOPK, shared_rows=(rank * batch, batch),
                                            out=e.part)
            t = e.block.trace_read()
            if i >= 3:
                for k_, v in t.items():
                    phase_ms[k_] = phase_ms.get(k_, 0.0) + v / reps
        for b in blocks:
            b.trace(False)
    roofline = None
    if phase_ms.get("gate_up"):
        ach = gu_bytes / (phase_ms["gate_up"] * 1e-3) / 1e9
        # DRAM traffic of this launch: the ncu capture of the same workload (profiles/
        # k_expert_gemv_decode_batch64_ncu_full.md: 439.4 MB read + written against 429.6 MB algorithmic,
        # growing in proportion to the experts hit) scaled to this run's algorithmic bytes
        roofline = dict(bound="hbm", kernel="k_expert_gemv<gate+up>", achieved=ach, peak=hbm_peak, unit="GB/s",
                        frac=ach / hbm_peak, peak_kind=peak_kind, traffic=gu_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE,
                        traffic_kind="ncu dram__bytes_read+write of a captured launch, scaled by algorithmic bytes",
                        algorithmic_bytes_per_launch=gu_bytes, us_per_launch=phase_ms["gate_up"] * 1e3,
                        phases_us={k_: round(v * 1e3, 2) for k_, v in phase_ms.items()},
                        layer_gbs=step_bytes / (ms_per_step * 1e-3) / 1e9,
                        layer_frac=step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
                        layer_bytes_per_step=step_bytes, distinct_experts=D)

    # ---- batch sweep 1/4/16 (tokens/s and whole-layer GB/s)
    sweep = {}
    if N == 1 and not args.no_sweep:
        for nb in (1, 4, 16):
            s_ms, _ = time_steps(nb, args.steps, W)
            us = 1e3 * s_ms / args.steps
            direct_us = us
            if not args.no_graph:
                g_ms, g_steps, _ = time_steps_graph(nb, args.steps, W)
                us = min(us, 1e3 * g_ms / g_steps)
            Dn = distinct_experts(nb)
            byt = blk0.weight_bytes(int(round(Dn))) + nb * H * 4
            gbs = byt / (us * 1e-6) / 1e9
            sweep[str(nb)] = dict(tokens_per_s=nb / (us * 1e-6), us_per_step=us, us_per_step_direct=direct_us,
                                  layer_gbs=gbs, layer_frac=gbs / hbm_peak, distinct_experts=Dn)
        sweep[str(batch)] = dict(tokens_per_s=value, us_per_step=1e3 * ms_per_step,
                                 layer_gbs=roofline["layer_gbs"] if roofline else None,
                                 layer_frac=roofline["layer_frac"] if roofline else None, distinct_experts=D)

    # ---- end to end: host buffers through the public host entry point
    e2e = None
    if N == 1:
        xh = [make_x(batch, 300 + i).cpu().pin_memory() for i in range(4)]
        oh = torch.empty((batch, H), dtype=torch.bfloat16).pin_memory()
        for i in range(W):
            blocks[i % len(blocks)].forward_host(xh[i % 4], oh)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(args.steps):
            blocks[i % len(blocks)].forward_host(xh[i % 4], oh)
        torch.cuda.synchronize()
        el = time.perf_counter() - t0
        e2e = dict(value=batch * args.steps / el, unit=UNIT, h2d_bytes_per_step=batch * H * 2,
                   d2h_bytes_per_step=batch * H * 2, ms_per_step=1e3 * el / args.steps)
    else:
        xh = [make_x(batch, 300 + i).cpu().pin_memory() for i in range(4)]
        oh = torch.empty((batch, H), dtype=torch.bfloat16).pin_memory()
        xd = torch.empty((batch, H), dtype=torch.bfloat16, device=dev)
        od = torch.empty((batch, H), dtype=torch.bfloat16, device=dev)

        def e2e_step(i):
            xd.copy_(xh[i % 4], non_blocking=True)
            eps[i % len(blocks)].forward_into(xd, od)
            oh.copy_(od, non_blocking=True)
            torch.cuda.synchronize()
        for i in range(W):
            e2e_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        barrier()
        el = torch.tensor([time.perf_counter() - t0], device=dev)
        dist.all_reduce(el, op=dist.ReduceOp.MAX)
        el = float(el.item())
        e2e = dict(value=batch * N * args.steps / el, unit=UNIT, h2d_bytes_per_step=batch * H * 2,
                   d2h_bytes_per_step=batch * H * 2, ms_per_step=1e3 * el / args.steps)

    cpu = None
    if rank == 0 and N == 1 and not args.no_cpu and host_layer0 is not None:
        cpu = run_cpu_baseline(host_layer0, batch, args.cpu_seconds)

    if rank == 0:
        line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=N, steps=steps_done, warmup=W,
                    ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="int8 x int4/6/8 block dots, f32 accumulate", data="synthetic",
                    config=dict(workload=workload_name(batch, N), global_batch=batch * N, layers_cycled=len(blocks),
                                l2="each step reads a layer not touched for layers-1 steps; per-step weight "
                                   "traffic exceeds the 126 MB L2", parallelism=f"ep{N}" if N > 1 else "single", launch=launch_mode, direct_calls=direct,
                                ep_mode=args.ep_mode if N > 1 else None),
                    roofline=roofline, cpu_baseline=cpu, e2e=e2e, gpu_launches=launches, clocks=clocks,
                    sweep=sweep or None)
        print(json.dumps(line), flush=True)
    if N > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

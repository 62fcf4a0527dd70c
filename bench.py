#!/usr/bin/env python
"""Benchmark of the quantised MoE FFN block, one JSON line on rank 0.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline workload (synthetic, seeded): the Qwen3-Next MoE block with Q4_K_M-style mixed
quantisation -- hidden 2048, 512 routed experts (gate/up Q4_K [512x2048], down Q6_K [2048x512]),
top-10, one Q8_0 shared expert with a sigmoid gate, f32 router -- at decode batch 64 per GPU, bf16
inputs ~N(0,1), uniform random routing.  A step is one forward of one block.  Consecutive steps
use different, independently seeded layers and a rotating set of inputs, so a step's weights are
never in L2 (every step of the small batches also meets experts it has not met before).

N = 1: the whole block on one GPU.  N > 1: expert parallelism, 512/N experts per GPU, every rank
home to 64 tokens (weak scaling), dispatch/combine over NCCL.

`value` is tokens/s with the inputs resident in HBM: the median over `repeats` timed blocks of
exactly K steps each (`spread` gives min and max).  `e2e` is the same metric through the
host-buffer entry point (host->device copy of x and device->host copy of the result inside the
timed region).  Extra keys carry the other benchmark configurations: `sweep` (decode batch 1/4/16,
cold and L2-hot), `prefill` (4096 tokens, Zipf-biased router, tensor-core roofline), `stack48`
(48 stacked blocks with RMSNorm and residual, global batch 256, strong scaling) and, for N > 1,
`ep_prefill` (16384 tokens through 4 all-Q8_0 blocks) and `ep_check` (the expert-parallel result
against the whole block on one GPU).

`--impl reference` times the CPU restatement of the reference's own CPU path (oracle/) on the
host cores instead, on the same workload and with all host threads.
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
L2_BYTES = 126e6
FLOPS_PER_TOKEN = (TOPK + 1) * 3 * 2 * H * F + 2 * H * E   # experts + shared + router


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="pmoe", choices=["pmoe", "reference"])
    ap.add_argument("--batch", type=int, default=64, help="decode tokens per GPU per step")
    ap.add_argument("--layers", type=int, default=8, help="distinct layers cycled through")
    ap.add_argument("--repeats", type=int, default=9, help="timed blocks of --steps steps; the median is reported")
    ap.add_argument("--no-sweep", action="store_true", help="skip the batch 1/4/16 sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baselines")
    ap.add_argument("--no-graph", action="store_true", help="do not try CUDA-graph replay of the block")
    ap.add_argument("--no-extra", action="store_true", help="skip the prefill / stack48 / ep_prefill records")
    ap.add_argument("--only", default="", help="comma list of extra records to run (prefill,stack48,ep_prefill)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--ep-mode", default="auto", choices=["auto", "native", "all_to_all", "all_gather"])
    ap.add_argument("--placement", default="contiguous", choices=["contiguous", "round_robin"])
    ap.add_argument("--ep-prefill-placement", default="round_robin", choices=["contiguous", "round_robin"],
                    help="expert -> rank table of the ep_prefill record (its router is Zipf-skewed: neighbouring hot "
                         "experts would pile up on one rank of a contiguous split)")
    ap.add_argument("--stack-layers", type=int, default=48)
    ap.add_argument("--stack-batch", type=int, default=256, help="global decode batch of the stack48 record")
    ap.add_argument("--prefill-tokens", type=int, default=4096)
    ap.add_argument("--ep-prefill-tokens", type=int, default=16384, help="global tokens of the ep_prefill record")
    ap.add_argument("--ep-prefill-layers", type=int, default=4)
    return ap.parse_args()


def workload_name(batch, n_gpus):
    s = (f"qwen3next-moe-block q4k_m (gate/up Q4_K, down Q6_K, shared Q8_0) H{H} F{F} E{E} top{TOPK}, "
         f"decode batch {batch}/GPU, bf16 x, uniform routing")
    if n_gpus > 1:
        s += f", expert-parallel {E // n_gpus} experts/GPU"
    return s


def workload_config(batch, n_gpus):
    """What defines the workload; identical in the library's arm and the reference arm."""
    return dict(workload=workload_name(batch, n_gpus), global_batch=batch * n_gpus, tokens_per_gpu=batch,
                parallelism=f"ep{n_gpus}" if n_gpus > 1 else "single")


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


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


# ------------------------------------------------------------------------------------------------ CPU legs
def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def use_all_host_threads():
    """The launcher of multi-rank runs exports OMP_NUM_THREADS=1; the CPU legs set their own count."""
    from oracle import pmoe_oracle as po
    found = os.environ.get("OMP_NUM_THREADS")
    po.set_threads(cpu_threads())
    return dict(threads=po.max_threads(), omp_num_threads_env=found, simd=po.simd_kind())


def run_cpu_baseline(layer_host, batch, seconds, seed=1234, what="whole-block forwards"):
    """Times the oracle (the port of the reference's CPU path) on whole-block forwards of `batch` tokens."""
    import torch
    from tests.common import oracle_layer
    th = use_all_host_threads()
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
        if el >= seconds or reps >= 2000:
            break
    return dict(value=batch * reps / el, unit=UNIT, cores=th["threads"], kind="port",
                sample=f"{reps} {what} of {batch} tokens on one layer, {el:.1f} s; C restatement of the reference "
                       f"CPU path ({th['simd']}), OpenMP over experts and rows",
                ms_per_step=1e3 * el / reps, omp_num_threads_env=th["omp_num_threads_env"])


def reference_arm(args, rank):
    """--impl reference: the CPU restatement of the reference's own CPU path on the host cores.  Same workload,
    steps and warm-up as the library's arm; a step is one whole-block forward of the global batch."""
    if rank != 0:
        return
    import torch
    from paramecia_b200 import synth
    from tests.common import oracle_layer
    th = use_all_host_threads()
    layer = synth.make_layer(H, F, E, TOPK, PRESET, seed=0, device="cpu", layer=0)
    ol = oracle_layer(layer)
    batch = args.batch * args.gpus
    g = torch.Generator().manual_seed(99)
    x = torch.randn((batch, H), generator=g).to(torch.bfloat16).float().numpy()
    steps, warm = args.steps, max(args.warmup, 3)
    ol.forward(x)
    t0 = time.perf_counter()
    ol.forward(x)
    one = time.perf_counter() - t0
    # bounded: the run must end within a few minutes whatever K the caller asks for
    budget = 120.0
    timed = max(1, min(steps, int(budget / max(one, 1e-6))))
    for _ in range(min(warm, 3)):
        ol.forward(x)
    t0 = time.perf_counter()
    for _ in range(timed):
        ol.forward(x)
    el = time.perf_counter() - t0
    val = batch * timed / el
    sample = (f"{timed} whole-block forwards of the global batch {batch} on one layer, {th['threads']} host threads "
              f"({th['simd']}); OMP_NUM_THREADS found: {th['omp_num_threads_env']}")
    line = dict(metric=METRIC, value=val, unit=UNIT, n_gpus=args.gpus, steps=steps, warmup=warm,
                ms_per_step=1e3 * el / timed, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="int8 x int4/6/8 block dots, f32 accumulate", data="synthetic", impl="reference",
                config=workload_config(args.batch, args.gpus),
                note="the Rust reference cannot be built here (no cargo, candle fork not vendored); this is the C "
                     "restatement of its CPU path in oracle/" + ("" if timed == steps else f"; {timed} of {steps} steps timed"),
                cpu_baseline=dict(value=val, unit=UNIT, cores=th["threads"], kind="port", sample=sample),
                e2e=dict(value=val, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ helpers
class Ctx:
    """What every part of the library's arm needs: ranks, device, peaks, barriers."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.args = args
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.N = int(os.environ.get("WORLD_SIZE", "1"))
        if self.N != args.gpus and self.N == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.torch, self.dist = torch, dist
        if self.N > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        pk = load_peaks()
        self.hbm_peak = float(pk.get("hbm_gbs", 6650.0))
        self.hbm_kind = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in pk else "fallback 6650 GB/s"
        self.tensor_peak = float(pk.get("bf16_tflops", 1590.0))
        self.tensor_kind = ("measured bf16 burst (MEASURED_PEAKS.json bf16_tflops)" if "bf16_tflops" in pk
                            else "fallback 1590 TFLOP/s")

    def barrier(self):
        if self.N > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.N == 1:
            return float(v)
        t = self.torch.tensor([float(v)], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def x(self, n, seed):
        g = self.torch.Generator(device=self.dev).manual_seed(seed + 7919 * self.rank)
        return self.torch.randn((n, H), generator=g, device=self.dev).to(self.torch.bfloat16)

    def free(self):
        import gc
        gc.collect()
        self.torch.cuda.empty_cache()


def median(v):
    s = sorted(v)
    return s[len(s) // 2]


def timed_blocks(ctx, step, steps, warmup, repeats):
    """`repeats` timed blocks of exactly `steps` calls of step(i), CUDA events on the launching stream, a barrier and a
    synchronize on both sides of every block; returns the per-block milliseconds (max over ranks)."""
    torch = ctx.torch
    for i in range(warmup):
        step(i)
    out, i0 = [], warmup
    for _ in range(repeats):
        ctx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step(i0 + i)
        e1.record()
        ctx.barrier()
        out.append(ctx.max_over_ranks(e0.elapsed_time(e1)))
        i0 += steps
    return out


def make_graph_step(ctx, fwd, n_slots):
    """One CUDA graph that holds fwd(i) for i in [0, n_slots); returns (replay callable, launches per replay)."""
    import paramecia_b200 as pm
    torch = ctx.torch
    side = torch.cuda.Stream(device=ctx.dev)
    side.wait_stream(torch.cuda.current_stream(ctx.dev))
    with torch.cuda.stream(side):
        for i in range(n_slots):
            fwd(i)
    torch.cuda.current_stream(ctx.dev).wait_stream(side)
    ctx.barrier()
    g = torch.cuda.CUDAGraph()
    before = pm.launch_count()
    with torch.cuda.graph(g):
        for i in range(n_slots):
            fwd(i)
    return g, pm.launch_count() - before


def decode_timing(ctx, fwd_of, n_tok, n_layers, steps, warmup, repeats, use_graph, n_inputs=5):
    """Times steps of n_tok tokens per GPU.  fwd_of(layer, x, out) runs one block forward.  Layers cycle with period
    n_layers and inputs with period n_inputs (coprime), so a layer meets a different input on every visit.  Returns
    the direct-call and (optionally) graph-replay timings; a graph holds n_layers * n_inputs forwards and the timed
    block replays it whole, so graph blocks time a multiple of that many steps and are scaled per step."""
    import paramecia_b200 as pm
    torch = ctx.torch
    xs = [ctx.x(n_tok, 100 + i) for i in range(n_inputs)]
    out = torch.empty((n_tok, H), dtype=torch.bfloat16, device=ctx.dev)

    def step(i):
        fwd_of(i % n_layers, xs[i % n_inputs], out)
    before = pm.launch_count()
    ms = timed_blocks(ctx, step, steps, warmup, repeats)
    launches = (pm.launch_count() - before) * steps // (warmup + repeats * steps)
    res = dict(direct_ms_per_step=[m / steps for m in ms], launches=launches)
    if use_graph:
        period = n_layers * n_inputs
        g, per_replay = make_graph_step(ctx, step, period)
        reps = max(1, round(steps / period))
        g_ms = timed_blocks(ctx, lambda i: g.replay(), reps, max(1, -(-warmup // period)), repeats)
        res.update(graph_ms_per_step=[m / (reps * period) for m in g_ms], graph_steps_per_block=reps * period,
                   graph_launches_per_step=per_replay / period)
        del g
    return res


# ------------------------------------------------------------------------------------------------ extra records
def prefill_record(ctx, preset="q4k_q6k_all"):
    """Configuration 3 on one GPU: 4096 bf16 tokens through one Q4_K / Q6_K block whose router carries the bias
    2*ln(1/rank_e) (rank = seeded permutation), so a dozen experts take most tokens.  Tokens/s of the block, the
    tensor-core roofline of the two grouped GEMMs and a CPU baseline on a 256-token sample."""
    import paramecia_b200 as pm
    from paramecia_b200 import synth
    torch, dev, args = ctx.torch, ctx.dev, ctx.args
    n = args.prefill_tokens
    nl = 2
    layers = [synth.make_layer(H, F, E, TOPK, preset, seed=0, device=dev, layer=li, zipf=True) for li in range(nl)]
    blocks = [synth.make_block(t, dev, max_tokens=n) for t in layers]
    xs = [ctx.x(n, 11 + i) for i in range(3)]
    out = torch.empty((n, H), dtype=torch.bfloat16, device=dev)
    steps, W, R = min(args.steps, 20), 3, min(args.repeats, 5)
    before = pm.launch_count()
    ms = timed_blocks(ctx, lambda i: blocks[i % nl].forward_into(xs[i % 3], out), steps, W, R)
    launches = (pm.launch_count() - before) * steps // (W + R * steps)
    for b in blocks:
        b.status()
    ms_step = median(ms) / steps
    phase = {}
    reps = 6
    blocks[0].trace(True)
    for i in range(reps + 2):
        blocks[0].forward_into(xs[i % 3], out)
        if i >= 2:
            for k_, v in blocks[0].trace_read().items():
                phase[k_] = phase.get(k_, 0.0) + v / reps
    blocks[0].trace(False)
    _, _, idx = blocks[0].route(xs[0])
    counts = torch.bincount(idx.flatten().long(), minlength=E)
    rows = n * TOPK + n
    gu_flops = rows * 2 * 2 * H * F
    dn_flops = rows * 2 * H * F
    rec = dict(metric="Q4_K MoE layer tokens/s (prefill)", value=n / (ms_step * 1e-3), unit=UNIT, ms_per_step=ms_step,
               steps=steps, repeats=R, spread_ms_per_step=[min(ms) / steps, max(ms) / steps],
               config=dict(workload=f"qwen3next-moe-block preset {preset} H{H} F{F} E{E} top{TOPK}, prefill {n} bf16 "
                                    f"tokens, Zipf-biased router (b_e = 2 ln(1/rank_e), seeded permutation)",
                           active_experts=int((counts > 0).sum()), max_tokens_per_expert=int(counts.max()),
                           layers_cycled=nl),
               block_tflops=n * FLOPS_PER_TOKEN / (ms_step * 1e-3) / 1e12,
               block_frac_of_tensor_peak=n * FLOPS_PER_TOKEN / (ms_step * 1e-3) / 1e12 / ctx.tensor_peak,
               phases_us={k_: round(v * 1e3, 1) for k_, v in phase.items()}, gpu_launches=launches)
    if phase.get("gate_up"):
        ach = gu_flops / (phase["gate_up"] * 1e-3) / 1e12
        rec["roofline"] = dict(bound="tensor", kernel="gate/up grouped GEMM", achieved=ach, peak=ctx.tensor_peak,
                               unit="TFLOP/s", frac=ach / ctx.tensor_peak, traffic=None, peak_kind=ctx.tensor_kind,
                               algorithmic_flops_per_launch=gu_flops, us_per_launch=phase["gate_up"] * 1e3)
    if phase.get("down"):
        ach = dn_flops / (phase["down"] * 1e-3) / 1e12
        rec["roofline_down"] = dict(bound="tensor", kernel="down grouped GEMM", achieved=ach, peak=ctx.tensor_peak,
                                    unit="TFLOP/s", frac=ach / ctx.tensor_peak,
                                    algorithmic_flops_per_launch=dn_flops, us_per_launch=phase["down"] * 1e3)
    xh = xs[0].cpu().pin_memory()
    oh = torch.empty((n, H), dtype=torch.bfloat16).pin_memory()
    for _ in range(3):
        blocks[0].forward_host(xh, oh)
    t0 = time.perf_counter()
    for i in range(steps):
        blocks[i % nl].forward_host(xh, oh)
    el = (time.perf_counter() - t0) / steps
    rec["e2e"] = dict(value=n / el, unit=UNIT, h2d_bytes_per_step=n * H * 2, d2h_bytes_per_step=n * H * 2,
                      ms_per_step=el * 1e3)
    if not args.no_cpu:
        host = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in layers[0].items()}
        host["shared"] = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in layers[0]["shared"].items()}
        rec["cpu_baseline"] = run_cpu_baseline(host, 256, min(args.cpu_seconds, 8.0), what="whole-block forwards (Zipf router)")
    del blocks, layers
    ctx.free()
    return rec


def make_ep(ctx, block):
    from paramecia_b200.ep import ExpertParallelMoe
    mode = ctx.args.ep_mode
    if mode == "auto":
        mode = ExpertParallelMoe.default_mode()
    return ExpertParallelMoe(block, mode=mode)


def build_rank_blocks(ctx, n_layers, preset, max_tokens, zipf=False, seed=0, layer0=0, placement=None):
    """Every rank builds the same seeded layers and keeps its slice of the experts."""
    from paramecia_b200 import synth
    N, rank = ctx.N, ctx.rank
    blocks = []
    for li in range(n_layers):
        t = synth.make_layer(H, F, E, TOPK, preset, seed=seed, device=ctx.dev, layer=layer0 + li, zipf=zipf)
        blocks.append(synth.make_rank_block(t, ctx.dev, max_tokens, rank, N, placement or ctx.args.placement))
        del t
    ctx.torch.cuda.synchronize()
    return blocks


def stack_record(ctx):
    """Configuration 4: `stack_layers` MoE blocks in a row, h <- h + moe(rms_norm(h)) (eps 1e-6, weight 1), global
    decode batch 256 split over the ranks (strong scaling), experts sharded E/N per rank."""
    import paramecia_b200 as pm
    torch, args, N = ctx.torch, ctx.args, ctx.N
    nl, gb = args.stack_layers, args.stack_batch
    n_home = gb // N
    blocks = build_rank_blocks(ctx, nl, "q4k_q6k_all", max_tokens=gb if N > 1 else max(gb, 64), seed=3)
    eps = [make_ep(ctx, b) for b in blocks] if N > 1 else None
    h0 = ctx.x(n_home, 500).float()
    resid = torch.empty_like(h0)
    y = torch.empty_like(h0)
    delta = torch.empty_like(h0)

    def step(_i):
        resid.copy_(h0)
        pm.add_rms_norm_into(resid, None, None, 1e-6, resid, y)
        for li in range(nl):
            if N > 1:
                eps[li].forward_into(y, delta)
            else:
                blocks[li].forward_into(y, delta)
            pm.add_rms_norm_into(resid, delta, None, 1e-6, resid, y)
    steps, W, R = max(3, min(args.steps, 10)), 3, min(args.repeats, 5)
    before = pm.launch_count()
    ms = timed_blocks(ctx, step, steps, W, R)
    launches = (pm.launch_count() - before) * steps // (W + R * steps)
    mode = "direct C-ABI calls"
    if N == 1 and not args.no_graph:
        g, per = make_graph_step(ctx, step, 1)
        g_ms = timed_blocks(ctx, lambda i: g.replay(), steps, W, R)
        if median(g_ms) < median(ms):
            ms, mode, launches = g_ms, "one CUDA graph of the whole stack, replayed", per * steps
        del g
    for b in blocks:
        b.status()
    ms_step = median(ms) / steps
    d = blocks[0]._desc
    per_expert = F * (pm.row_bytes(d.gate_dtype, H) + pm.row_bytes(d.up_dtype, H)) + H * pm.row_bytes(d.down_dtype, F)
    # distinct local experts a layer's batch hits, from the first layer's routing of the first input
    xg = y if N == 1 else eps[0].gather_tokens(y)
    _, _, idx = blocks[0].route(xg.to(torch.bfloat16))
    D = int(torch.unique(idx[blocks[0].local_mask(idx)]).numel())
    layer_bytes = blocks[0].weight_bytes(D) + n_home * H * 8
    rec = dict(metric="48-layer MoE FFN stack tokens/s (decode)", value=gb / (ms_step * 1e-3), unit=UNIT,
               ms_per_step=ms_step, us_per_layer=1e3 * ms_step / nl, steps=steps, repeats=R,
               spread_ms_per_step=[min(ms) / steps, max(ms) / steps], scaling="strong",
               config=dict(workload=f"{nl} stacked qwen3next-moe blocks (gate/up Q4_K, down Q6_K, shared expert quantised like the "
                                    f"routed ones), residual add + RMSNorm(eps 1e-6, weight 1) between layers, global decode "
                                    f"batch {gb}, f32 residual stream", global_batch=gb, tokens_per_gpu=n_home,
                           parallelism=f"ep{N}" if N > 1 else "single", launch=mode,
                           weights_gb_per_gpu=round(sum(b.resident_bytes() for b in blocks) / 1e9, 2)),
               layer_gbs_per_gpu=layer_bytes / (1e-3 * ms_step / nl) / 1e9,
               layer_frac_of_hbm_peak=layer_bytes / (1e-3 * ms_step / nl) / 1e9 / ctx.hbm_peak,
               distinct_local_experts=D, per_expert_bytes=per_expert, gpu_launches=launches)
    if N > 1:
        rec["exposed_collective_us_per_layer"] = ep_exposed_us(ctx, eps[:4], y, delta)
        rec["ep_mode"] = eps[0].mode
    del blocks, eps
    ctx.free()
    return rec


def ep_exposed_us(ctx, eps, x, out, reps=8):
    """Per-layer time the collectives add to a rank's step: CUDA events around the dispatch and the combine on the
    launching stream (everything on that stream waits for them, so what they take is exposed), max over ranks."""
    acc = dict(dispatch=0.0, combine=0.0, total=0.0)
    for i in range(reps + 2):
        t = eps[i % len(eps)].forward_into(x, out, profile=True)
        if i >= 2:
            for k_ in acc:
                acc[k_] += t[k_] / reps
    return {k_: round(1e3 * ctx.max_over_ranks(v), 2) for k_, v in acc.items()}


def ep_prefill_record(ctx):
    """Configuration 5: expert-parallel prefill of 16384 tokens (global) through 4 stacked all-Q8_0 blocks, Zipf-biased
    routing, hidden state carried through residual + RMSNorm like the stack."""
    import paramecia_b200 as pm
    torch, args, N = ctx.torch, ctx.args, ctx.N
    nl, gt = args.ep_prefill_layers, args.ep_prefill_tokens
    n_home = gt // N
    blocks = build_rank_blocks(ctx, nl, "q8_0", max_tokens=gt, zipf=True, seed=5, placement=args.ep_prefill_placement)
    eps = [make_ep(ctx, b) for b in blocks]
    h0 = ctx.x(n_home, 900).float()
    resid, y, delta = torch.empty_like(h0), torch.empty_like(h0), torch.empty_like(h0)

    def step(_i):
        resid.copy_(h0)
        pm.add_rms_norm_into(resid, None, None, 1e-6, resid, y)
        for li in range(nl):
            eps[li].forward_into(y, delta)
            pm.add_rms_norm_into(resid, delta, None, 1e-6, resid, y)
    steps, W, R = max(2, min(args.steps, 5)), 3, min(args.repeats, 3)
    ms = timed_blocks(ctx, step, steps, W, R)
    for b in blocks:
        b.status()
    ms_step = median(ms) / steps
    _, _, idx = blocks[0].route(eps[0].gather_tokens(y).to(torch.bfloat16))
    pairs = blocks[0].local_mask(idx).sum().float()
    load = [torch.zeros(1, device=ctx.dev) for _ in range(N)]
    ctx.dist.all_gather(load, pairs.reshape(1))
    rec = dict(metric="expert-parallel Q8_0 prefill tokens/s", value=gt / (ms_step * 1e-3), unit=UNIT, ms_per_step=ms_step,
               ms_per_layer=ms_step / nl, steps=steps, repeats=R, spread_ms_per_step=[min(ms) / steps, max(ms) / steps],
               config=dict(workload=f"{nl} stacked all-Q8_0 qwen3next-moe blocks, {gt} bf16-valued tokens (global), Zipf-biased "
                                    f"router, residual + RMSNorm between blocks", global_tokens=gt, tokens_per_gpu=n_home,
                           parallelism=f"ep{N}", placement=args.ep_prefill_placement),
               block_tflops=gt * FLOPS_PER_TOKEN / (1e-3 * ms_step / nl) / 1e12,
               exposed_collective_us_per_layer=ep_exposed_us(ctx, eps, y, delta, reps=3),
               pairs_per_gpu=[int(v.item()) for v in load], ep_mode=eps[0].mode)
    del blocks, eps
    ctx.free()
    return rec


def ep_check(ctx, ep, whole_layer):
    """The expert-parallel forward against the whole block evaluated on this rank's GPU, on the rank's own rows."""
    from paramecia_b200 import synth
    torch, N, rank = ctx.torch, ctx.N, ctx.rank
    n = ctx.args.batch
    whole = synth.make_block(whole_layer, ctx.dev, max_tokens=N * n)
    g = torch.Generator(device=ctx.dev).manual_seed(4242)   # the same rows on every rank
    x_all = torch.randn((N * n, H), generator=g, device=ctx.dev).to(torch.bfloat16)
    x = x_all[rank * n:(rank + 1) * n].contiguous()
    out = torch.empty((n, H), dtype=torch.float32, device=ctx.dev)
    stats = {}
    ep.forward_into(x, out, stats)
    want, (_, want_idx) = whole.forward_with_stats(x_all, out_dtype=torch.float32)
    want = want[rank * n:(rank + 1) * n]
    torch.cuda.synchronize()
    err = float((out - want).abs().max() / want.abs().max())
    same = 1.0 if torch.equal(stats["top_indices"], want_idx[rank * n:(rank + 1) * n]) else 0.0
    worst = ctx.max_over_ranks(err)
    all_same = -ctx.max_over_ranks(-same)
    whole.close()
    del whole
    ctx.free()
    return dict(max_rel_err=worst, idx_equal=bool(all_same == 1.0), world=N, rows_per_rank=n,
                against="whole block on one GPU (libpmoe), same seeded rows")


# ------------------------------------------------------------------------------------------------ the library's arm
def pmoe_arm(args):
    import paramecia_b200 as pm
    from paramecia_b200 import synth
    ctx = Ctx(args)
    torch, dist, dev, N, rank = ctx.torch, ctx.dist, ctx.dev, ctx.N, ctx.rank
    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()   # early: nvidia-smi takes a moment to come up; idle samples are dropped by mark()
    batch = args.batch
    only = [s for s in args.only.split(",") if s]

    # ---- layers: every rank builds the same seeded layers and keeps its slice of the experts
    max_tok = batch * N if N > 1 else max(batch, 64)
    blocks, host_layer0, layer0_dev = [], None, None
    for li in range(args.layers):
        t = synth.make_layer(H, F, E, TOPK, PRESET, seed=0, device=dev, layer=li)
        if li == 0 and rank == 0 and not args.no_cpu and N == 1:
            host_layer0 = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in t.items()}
            host_layer0["shared"] = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in t["shared"].items()}
        if li == 0 and N > 1:
            layer0_dev = t
        blocks.append(synth.make_rank_block(t, dev, max_tok, rank, N, args.placement))
        del t
    torch.cuda.synchronize()
    eps = [make_ep(ctx, b) for b in blocks] if N > 1 else None

    def fwd_of(layer, x, out):
        if N > 1:
            eps[layer].forward_into(x, out)
        else:
            blocks[layer].forward_into(x, out)

    check = ep_check(ctx, eps[0], layer0_dev) if N > 1 else None
    layer0_dev = None
    ctx.free()

    # ---- headline: decode batch per GPU, layers cycled, inputs rotated
    W = max(args.warmup, 3)
    if rank == 0:
        sampler.mark()   # window: warm-up, the timed blocks and their graph replay (all the same load)
    tim = decode_timing(ctx, fwd_of, batch, len(blocks), args.steps, W, args.repeats,
                        use_graph=not args.no_graph and N == 1)
    d_med = median(tim["direct_ms_per_step"])
    ms_per_step, launch_mode, spread = d_med, "direct C-ABI calls", tim["direct_ms_per_step"]
    launches = tim["launches"]
    if "graph_ms_per_step" in tim and median(tim["graph_ms_per_step"]) < d_med:
        ms_per_step, spread = median(tim["graph_ms_per_step"]), tim["graph_ms_per_step"]
        launch_mode = (f"CUDA graph holding {tim['graph_steps_per_block']} forwards ({len(blocks)} layers x 5 inputs), "
                       f"replayed; per-step time = replay time / forwards held")
        launches = int(round(tim["graph_launches_per_step"] * args.steps))
    value = batch * N / (ms_per_step * 1e-3)
    clocks = sampler.stop() if rank == 0 else {}

    # ---- roofline of the dominant kernel (gate/up GEMV): traced pass, events around each kernel
    def distinct_experts(n_tok):
        tot = 0
        for i in range(4):
            x = ctx.x(n_tok, 100 + i)
            if N > 1:
                x = eps[0].gather_tokens(x)
            b = blocks[i % len(blocks)]
            _, _, idx = b.route(x)
            tot += int(torch.unique(idx[b.local_mask(idx)]).numel())
        return tot / 4.0

    D = distinct_experts(batch)
    blk0 = blocks[0]
    d = blk0._desc
    gu_bytes = D * F * (pm.row_bytes(d.gate_dtype, H) + pm.row_bytes(d.up_dtype, H))
    gu_bytes += F * (pm.row_bytes(d.sh_gate_dtype, H) + pm.row_bytes(d.sh_up_dtype, H))
    dn_bytes = D * H * pm.row_bytes(d.down_dtype, F) + H * pm.row_bytes(d.sh_down_dtype, F)
    step_bytes = blk0.weight_bytes(int(round(D))) + batch * H * 4  # weights + x in + out (bf16 each)
    phase_ms = {}
    reps = min(max(args.steps, 10), 50)
    if N == 1:
        out = torch.empty((batch, H), dtype=torch.bfloat16, device=dev)
        xs = [ctx.x(batch, 5 + i) for i in range(5)]
        for b in blocks:
            b.trace(True)
        for i in range(reps + 3):
            b = blocks[i % len(blocks)]
            b.forward_into(xs[i % 5], out)
            t = b.trace_read()
            if i >= 3:
                for k_, v in t.items():
                    phase_ms[k_] = phase_ms.get(k_, 0.0) + v / reps
        for b in blocks:
            b.trace(False)
    else:
        phase_ms = eps[0].trace_experts(ctx.x(batch, 5), reps)
    roofline = None
    if phase_ms.get("gate_up"):
        ach = gu_bytes / (phase_ms["gate_up"] * 1e-3) / 1e9
        roofline = dict(bound="hbm", kernel="k_gate_up_q4k_mma (gate + up + SiLU, Q4_K experts)", achieved=ach, peak=ctx.hbm_peak, unit="GB/s",
                        frac=ach / ctx.hbm_peak, peak_kind=ctx.hbm_kind,
                        # DRAM bytes of one captured launch of this kernel on this workload (ncu dram__bytes_read.sum +
                        # dram__bytes_write.sum) divided by that launch's algorithmic bytes; regenerate the constant
                        # whenever the kernel changes
                        traffic=gu_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE,
                        traffic_kind="ncu dram__bytes_read+write of a captured launch, scaled by algorithmic bytes",
                        algorithmic_bytes_per_launch=gu_bytes, us_per_launch=phase_ms["gate_up"] * 1e3,
                        phases_us={k_: round(v * 1e3, 2) for k_, v in phase_ms.items()},
                        layer_gbs=step_bytes / (ms_per_step * 1e-3) / 1e9,
                        layer_frac=step_bytes / (ms_per_step * 1e-3) / 1e9 / ctx.hbm_peak,
                        layer_bytes_per_step=step_bytes, distinct_experts=D)
        if phase_ms.get("down"):
            a2 = dn_bytes / (phase_ms["down"] * 1e-3) / 1e9
            roofline["down"] = dict(kernel="k_down_q6k_mma (down x routing weight, Q6_K experts)", achieved=a2, frac=a2 / ctx.hbm_peak,
                                    algorithmic_bytes_per_launch=dn_bytes, us_per_launch=phase_ms["down"] * 1e3)

    # ---- batch sweep 1/4/16: cold (layers and inputs rotate) and L2-hot (one layer, one input)
    sweep = {}
    if N == 1 and not args.no_sweep:
        for nb in (1, 4, 16):
            Dn = distinct_experts(nb)
            byt = blk0.weight_bytes(int(round(Dn))) + nb * H * 4
            t_c = decode_timing(ctx, fwd_of, nb, len(blocks), args.steps, W, min(args.repeats, 5), not args.no_graph)
            us = 1e3 * min(median(t_c["direct_ms_per_step"]), median(t_c.get("graph_ms_per_step", [1e9])))
            t_h = decode_timing(ctx, lambda l, x, o: blocks[0].forward_into(x, o), nb, 1, args.steps, W, 3,
                                not args.no_graph, n_inputs=1)
            us_hot = 1e3 * min(median(t_h["direct_ms_per_step"]), median(t_h.get("graph_ms_per_step", [1e9])))
            gbs = byt / (us * 1e-6) / 1e9
            sweep[str(nb)] = dict(tokens_per_s=nb / (us * 1e-6), us_per_step=us,
                                  us_per_step_direct=1e3 * median(t_c["direct_ms_per_step"]),
                                  us_per_step_hot_l2=us_hot, layer_gbs=gbs, layer_frac=gbs / ctx.hbm_peak,
                                  distinct_experts=Dn, bytes_per_step=byt,
                                  bytes_between_visits_of_a_layer=byt * len(blocks),
                                  cold=bool(byt * len(blocks) > 1.5 * L2_BYTES))
        sweep[str(batch)] = dict(tokens_per_s=value, us_per_step=1e3 * ms_per_step,
                                 layer_gbs=roofline["layer_gbs"] if roofline else None,
                                 layer_frac=roofline["layer_frac"] if roofline else None, distinct_experts=D,
                                 bytes_per_step=step_bytes, cold=True)

    # ---- end to end: host buffers through the public host entry point
    xh = [ctx.x(batch, 300 + i).cpu().pin_memory() for i in range(5)]
    oh = torch.empty((batch, H), dtype=torch.bfloat16).pin_memory()
    if N == 1:
        def e2e_step(i):
            blocks[i % len(blocks)].forward_host(xh[i % 5], oh)
    else:
        xd = torch.empty((batch, H), dtype=torch.bfloat16, device=dev)
        od = torch.empty((batch, H), dtype=torch.bfloat16, device=dev)

        def e2e_step(i):
            xd.copy_(xh[i % 5], non_blocking=True)
            eps[i % len(blocks)].forward_into(xd, od)
            oh.copy_(od, non_blocking=True)
            torch.cuda.synchronize()
    for i in range(W):
        e2e_step(i)
    els = []
    for r in range(min(args.repeats, 5)):
        ctx.barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(W + r * args.steps + i)
        ctx.barrier()
        els.append(ctx.max_over_ranks(time.perf_counter() - t0))
    el = median(els)
    e2e = dict(value=batch * N * args.steps / el, unit=UNIT, h2d_bytes_per_step=batch * H * 2,
               d2h_bytes_per_step=batch * H * 2, ms_per_step=1e3 * el / args.steps,
               api="MoeBlock.forward_host (pmoe_forward_host)" if N == 1 else
                   "pinned host -> device copy, ExpertParallelMoe.forward_into, device -> pinned host copy, synchronize")

    cpu = None
    if rank == 0 and N == 1 and not args.no_cpu and host_layer0 is not None:
        cpu = run_cpu_baseline(host_layer0, batch, args.cpu_seconds)
    for b in blocks:
        b.status()
    ep_mode = eps[0].mode if N > 1 else None
    n_layers = len(blocks)
    del blocks, eps
    ctx.free()

    # ---- the other benchmark configurations
    extra = {}
    if not args.no_extra:
        want = lambda name: (not only) or name in only
        if N == 1 and want("prefill"):
            extra["prefill"] = prefill_record(ctx)
            keep = ("value", "ms_per_step", "phases_us", "config", "block_tflops", "roofline", "roofline_down")
            extra["prefill_q8_0_shared"] = {k_: v for k_, v in prefill_record(ctx, "q4k_m").items() if k_ in keep}
            extra["prefill_q8_0"] = {k_: v for k_, v in prefill_record(ctx, "q8_0").items() if k_ in keep}
        if want("stack48"):
            extra["stack48"] = stack_record(ctx)
        if N > 1 and want("ep_prefill"):
            extra["ep_prefill"] = ep_prefill_record(ctx)

    if rank == 0:
        cfg = workload_config(batch, N)
        line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=N, steps=args.steps, warmup=W,
                    ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="int8 x int4/6/8 block dots, f32 accumulate", data="synthetic", config=cfg,
                    run=dict(layers_cycled=n_layers, inputs_rotated=5, repeats=args.repeats,
                             value_is="median over repeats of K-step blocks",
                             spread_ms_per_step=[min(spread), max(spread)],
                             l2="a step reads a layer not touched for layers-1 steps, with an input that layer has not met "
                                "in the last 4 visits; per-step weight traffic exceeds the 126 MB L2 at batch 64 (see "
                                "sweep[...].cold for the small batches)",
                             launch=launch_mode, direct_calls_ms_per_step=d_med, ep_mode=ep_mode,
                             placement=args.placement if N > 1 else None),
                    roofline=roofline, cpu_baseline=cpu, e2e=e2e, gpu_launches=launches, clocks=clocks,
                    sweep=sweep or None, ep_check=check, **extra)
        print(json.dumps(line), flush=True)
    if N > 1:
        dist.destroy_process_group()


NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = (435.556352 + 8.189952) / 429.555712   # gate/up launch at batch 64, 362 experts hit


def main():
    args = parse()
    if args.impl == "reference":
        reference_arm(args, int(os.environ.get("RANK", "0")))
        return
    pmoe_arm(args)


if __name__ == "__main__":
    main()

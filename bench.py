"""Benchmark of the triangle-attention hot path (starting node, ending node, pair transition) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg5|cfg2|cfg3|n768|block768|cfg4pair|cfg4] [--blocks M]
                    [--exchange all_to_all|peer_stores] [--no-also] [--no-cpu-baseline]

One "step" is one pass of the hot path over one batch of synthetic pair tensors: the starting-node and the
ending-node TriangleAttention (LayerNorm, q/k/v/gate + triangle-bias projections, masked biased attention, sigmoid
gate, output projection, residual) applied in sequence; workloads with a transition also run the fused pair
transition.

Default workload ("cfg5", the same at every N): 4 pair-track blocks (start node, transpose, end node, transition) on
ONE pair tensor z[1, 4096, 4096, 128] bf16 with 3900 valid tokens, its pair rows sharded over the N ranks: strong
scaling, `value` = total TFLOP/s of the job, so value_N / (N * value_1) is the parallel efficiency.  With N > 1 the
run first checks the sharded block against the single-GPU modules on a small tensor (`sharded_check`) and exits
non-zero when they disagree.  With N = 1 the same JSON line carries, under `also`, the single-GPU figures of
"cfg2" (z[1, 512, 512, 128], 475 valid tokens, start + end node) and "n768" (z[1, 768, 768, 128], start + end node
+ transition), each with its own roofline.

Metric: tri-attn TFLOP/s = algorithmic flops of the step (valid positions only) / time.  Rank 0 prints one JSON
line.  `value` is timed with CUDA events with inputs resident in HBM (inputs far larger than L2, or L2 flushed
between steps); `e2e` runs the same step through the module API from pinned host memory and back.

Other workloads: "block768" adds the two triangle multiplications (the pair track of one Pairformer block),
"cfg4pair" / "cfg4" replay a 48-block trunk without / with the single track from one CUDA graph (`--blocks`
overrides the depth); with N > 1 these non-sharded workloads run one independent batch per rank (weak scaling).

--impl reference times the CPU implementation of the reference's eager path on the host cores, on a bounded row
sample of the same workload: the reference's own modules when they have been staged next to the oracle, else the
restatement in oracle/.
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
import types
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (batch, tokens, valid-length spec, transition?)
    "cfg2": dict(B=1, N=512, valid="475", transition=False,
                 desc="start+end TriangleAttention, z[1,512,512,128] bf16, 475 valid tokens (BASELINE config 2)"),
    "cfg3": dict(B=64, N=256, valid="U160-256", transition=True,
                 desc="start+end TriangleAttention + transition, z[64,256,256,128] bf16, valid ~U{160..256} (BASELINE config 3)"),
    "n768": dict(B=1, N=768, valid="768", transition=True,
                 desc="start+end TriangleAttention + transition, z[1,768,768,128] bf16, all valid (pair track of BASELINE config 4)"),
    "block768": dict(B=1, N=768, valid="768", transition=True, trimul=True,
                     desc="pair track of one Pairformer block: triangle multiplication outgoing + incoming, "
                          "start+end TriangleAttention, transition, z[1,768,768,128] bf16, all valid (BASELINE config 4)"),
    "cfg4pair": dict(B=1, N=768, valid="768", transition=True, trimul=True, blocks=48,
                     desc="pair track of a 48-block Pairformer trunk (PairformerNoSeqModule: per block triangle "
                          "multiplication out + in, start+end TriangleAttention, transition), z[1,768,768,128] bf16, "
                          "all valid (pair track of BASELINE config 4), replayed from one CUDA graph"),
    "cfg4": dict(B=1, N=768, valid="768", transition=True, trimul=True, blocks=48, single=True,
                 desc="48-block Pairformer trunk (PairformerModule: per block triangle multiplication out + in, "
                      "start+end TriangleAttention, pair transition, single-track attention with pair bias (c_s=384, "
                      "16 heads), single transition), z[1,768,768,128] and s[1,768,384] bf16, all valid (BASELINE "
                      "config 4), replayed from one CUDA graph"),
    "cfg5": dict(B=1, N=4096, valid="3900", transition=True, sharded=True, blocks=4,
                 desc="4 x (start node, all-to-all, end node, transition), z[1,4096,4096,128] bf16 row-sharded over the "
                      "GPUs, 3900 valid tokens (BASELINE config 5)"),
}
DEFAULT_STEPS = {"cfg2": 100, "cfg3": 20, "n768": 50, "block768": 50, "cfg4pair": 5, "cfg4": 5, "cfg5": 5}
ALSO_STEPS = 20  # timed steps of each extra single-GPU workload reported under "also"


def valid_lengths(spec: str, B: int, N: int, gen: torch.Generator) -> list[int]:
    if spec.startswith("U"):
        lo, hi = map(int, spec[1:].split("-"))
        return torch.randint(lo, hi + 1, (B,), generator=gen).tolist()
    return [int(spec)] * B


def node_flops(L: int) -> float:
    """Algorithmic flops of one node for an item with L valid tokens: L² positions x (projections + 512·L)."""
    return float(L) * L * (164864.0 + 512.0 * L)


def attention_core_flops(L: int) -> float:
    return float(L) * L * 512.0 * L


def transition_flops(L: int) -> float:
    return float(L) * L * 393216.0


def trimul_flops(L: int, N: int) -> float:
    """One triangle-multiplication node: projections (128 -> 2x256, 2x 128 -> 128) on the L² valid positions plus the
    contraction, 2·L flops per valid position and channel (128 channels)."""
    return float(L) * L * (131072.0 + 65536.0 + 256.0 * L)


def single_track_flops(L: int) -> float:
    """Single track of one block for L valid tokens: in-projection (384 -> 4x384), pair-bias projection (128 -> 16 on
    L² positions), q·k and p·v (16 heads of 24), output projection, and the transition (384 -> 2x1536 -> 384)."""
    return float(L) * (2.0 * 384 * 1536 + 2.0 * 384 * 384 + 2.0 * 384 * 3072 + 2.0 * 1536 * 384) \
        + float(L) * L * (2.0 * 128 * 16 + 4.0 * 16 * 24)


def measured_peaks() -> tuple[float, float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


def sustained_bf16_peak() -> float:
    """cuBLAS bf16 throughput of a seconds-long loop under the power cap (the denominator for a kernel timed inside a
    long power-capped step; the burst figure is for a kernel timed alone)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        if d.get("bf16_tflops_sustained"):
            return float(d["bf16_tflops_sustained"])
    return 1400.0


def peak_for_step(burst_tf: float, clk: dict, step_ms: float) -> tuple[float, str]:
    """Burst peak unless the timed step is long (>= 100 ms) and ran power-capped below 95 % of the maximum SM clock."""
    capped = ("sw_power_cap" in clk.get("reasons", []) and clk.get("sm_mhz") and clk.get("sm_max_mhz")
              and clk["sm_mhz"] < 0.95 * clk["sm_max_mhz"])
    if capped and step_ms >= 100.0:
        return sustained_bf16_peak(), (f"bf16 sustained (kernel timed inside a {step_ms:.0f} ms step under sw_power_cap at "
                                       f"{clk['sm_mhz']:.0f} of {clk['sm_max_mhz']:.0f} MHz)")
    return burst_tf, "bf16 burst"


class ClockSampler:
    """Samples SM clock and throttle reasons (NVML, else nvidia-smi) while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples: list[tuple[float, float, str]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run_nvml(self) -> bool:
        """Reads the same fields through NVML in-process (a sample takes well under a millisecond)."""
        try:
            import pynvml as nv

            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            h = nv.nvmlDeviceGetHandleByIndex(index)
            max_sm = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = (("hw_slowdown", nv.nvmlClocksThrottleReasonHwSlowdown),
                     ("hw_thermal_slowdown", nv.nvmlClocksThrottleReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", nv.nvmlClocksThrottleReasonSwThermalSlowdown),
                     ("sw_power_cap", nv.nvmlClocksThrottleReasonSwPowerCap))
        except Exception:
            return False
        while not self._stop.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((sm, max_sm, ",".join(n for n, bit in names if mask & bit)))
            except Exception:
                pass
            self._stop.wait(0.005)
        return True

    def _run(self):
        if self._run_nvml():
            return
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                f = [x.strip() for x in out.split(",")]
                reasons = [n for n, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                              "sw_power_cap"), f[2:6]) if v == "Active"]
                self.samples.append((float(f[0]), float(f[1]), ",".join(reasons)))
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = sorted({r for s in self.samples for r in s[2].split(",") if r})
        return {"sm_mhz": statistics.median(s[0] for s in self.samples), "sm_max_mhz": self.samples[0][1],
                "reasons": reasons, "samples": len(self.samples)}


# Seeded random weights of the benchmark's modules (matrices ~N(0, 0.02²), LayerNorm at identity, as BASELINE's
# configs describe them), under the attribute names the module builders below read.
def node_weights(seed: int) -> types.SimpleNamespace:
    g = torch.Generator().manual_seed(seed)
    return types.SimpleNamespace(w_bias=torch.randn(4, 128, generator=g) * 0.02, w_in=torch.randn(512, 128, generator=g) * 0.02,
                                 w_out=torch.randn(128, 128, generator=g) * 0.02, ln_w=torch.ones(128),
                                 ln_b=torch.zeros(128), b_in=None, b_out=None)


def transition_weights(seed: int) -> types.SimpleNamespace:
    g = torch.Generator().manual_seed(seed)
    return types.SimpleNamespace(w1=torch.randn(1024, 128, generator=g) * 0.02, w2=torch.randn(128, 512, generator=g) * 0.02,
                                 ln_w=torch.ones(128), ln_b=torch.zeros(128))


def trimul_weights(seed: int) -> types.SimpleNamespace:
    g = torch.Generator().manual_seed(seed)
    return types.SimpleNamespace(w_p_in=torch.randn(256, 128, generator=g) * 0.02, w_g_in=torch.randn(256, 128, generator=g) * 0.02,
                                 w_p_out=torch.randn(128, 128, generator=g) * 0.02, w_g_out=torch.randn(128, 128, generator=g) * 0.02,
                                 ln_in_w=torch.ones(128), ln_in_b=torch.zeros(128), ln_out_w=torch.ones(128),
                                 ln_out_b=torch.zeros(128))


def make_inputs(cfg: dict, seed: int, device):
    gen = torch.Generator().manual_seed(seed)
    B, N = cfg["B"], cfg["N"]
    z = torch.randn(B, N, N, 128, generator=gen).to(torch.bfloat16)
    lens = valid_lengths(cfg["valid"], B, N, gen)
    m = torch.zeros(B, N)
    for b, L in enumerate(lens):
        m[b, :L] = 1
    mask = m[:, :, None] * m[:, None, :]
    return z, mask, lens, node_weights(seed + 1), node_weights(seed + 2), transition_weights(seed + 3)


def build_modules(w_start, w_end, w_tr, device):
    import bionemo_inference_runtime_b200 as b200

    def node(cls, w):
        n = cls(128, 32, 4, dtype=torch.bfloat16, attn_backend="Heuristic")
        n.load_state_dict({"layer_norm.weight": w.ln_w, "layer_norm.bias": w.ln_b, "pair_bias_proj.weight": w.w_bias,
                           "mha.in_proj.weight": w.w_in, "mha.o_proj.weight": w.w_out}, strict=True)
        return n.to(device)

    start = node(b200.TriangleAttentionStartingNode, w_start)
    end = node(b200.TriangleAttentionEndingNode, w_end)
    tr = b200.Transition(128, 512, dtype=torch.bfloat16)
    tr.load_state_dict({"norm.weight": w_tr.ln_w, "norm.bias": w_tr.ln_b, "fused_fc2_fc1.weight": w_tr.w1,
                        "fc3.weight": w_tr.w2}, strict=True)
    return start, end, tr.to(device)


def build_trimul(seed: int, device):
    import bionemo_inference_runtime_b200 as b200

    nodes = []
    for k, kind in enumerate((b200.TriangleMultiplicationNodeType.OUTGOING, b200.TriangleMultiplicationNodeType.INCOMING)):
        w = trimul_weights(seed + 10 + k)
        n = b200.TriangleMultiplicationNode(multiplication_type=kind, dtype=torch.bfloat16, high_precision=False)
        n.load_state_dict({"norm_in.weight": w.ln_in_w, "norm_in.bias": w.ln_in_b, "p_in.weight": w.w_p_in,
                           "g_in.weight": w.w_g_in, "norm_out.weight": w.ln_out_w, "norm_out.bias": w.ln_out_b,
                           "p_out.weight": w.w_p_out, "g_out.weight": w.w_g_out}, strict=True)
        nodes.append(n.to(device))
    return nodes


def run_ours(args, brief: bool = False) -> dict:
    """Non-sharded workloads: one independent batch per rank.  ``brief`` (used for the extra workloads reported
    beside the default one) skips the CPU baseline and the one-step-at-a-time latency loop."""
    import torch.distributed as dist

    from bionemo_inference_runtime_b200 import _lib, ops
    import bionemo_inference_runtime_b200 as b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    numa_cores = b200.bind_to_gpu_numa_node(device) if world > 1 else None  # pinned buffers next to this rank's GPU
    cfg = dict(WORKLOADS[args.workload])
    if args.blocks is not None and cfg.get("blocks") and not cfg.get("sharded"):
        cfg["blocks"] = args.blocks
        cfg["desc"] += f" [--blocks {args.blocks}]"
    z_host, mask_host, lens, w_start, w_end, w_tr = make_inputs(cfg, 1000 + rank, device)
    start, end, trans = build_modules(w_start, w_end, w_tr, device)
    pre = b200.precompute_pair_masks("Heuristic", mask_host.to(device))
    z_dev = z_host.to(device)
    bufs: dict = {}
    trimul = build_trimul(1000 + rank, device) if cfg.get("trimul") else []
    mask_dev = mask_host.to(device)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    stack = None
    if cfg.get("blocks") and not cfg.get("sharded"):
        # a whole trunk: the package's stack module with random weights per block, one CUDA graph for all blocks
        cls = b200.PairformerModule if cfg.get("single") else b200.PairformerNoSeqModule
        extra = dict(attention_initial_norm=True) if cfg.get("single") else {}
        stack = cls(num_blocks=cfg["blocks"], dtype=torch.bfloat16, triangle_attn_backend="Heuristic",
                    trimul_high_precision=False, use_cuda_graph=True, **extra).to(device)
        gen = torch.Generator(device=device).manual_seed(2000 + rank)
        for name, prm in stack.named_parameters():
            if prm.dim() == 2:
                prm.data.copy_(torch.randn(prm.shape, generator=gen, device=device) * 0.02)
            else:
                prm.data.fill_(0.0 if name.endswith("bias") else 1.0)

    single = bool(cfg.get("single"))
    if single:
        s_pin = torch.randn(cfg["B"], cfg["N"], 384, generator=torch.Generator().manual_seed(3000 + rank)).bfloat16().pin_memory()
        s_out_pin = torch.empty_like(s_pin).pin_memory()
        s_dev = s_pin.to(device)
        token_mask = torch.stack([(torch.arange(cfg["N"]) < L).float() for L in lens]).to(device)
    last_s = [None]

    def step(z, b=None, s=None):
        if stack is not None and single:
            last_s[0], z_new = stack(s_dev if s is None else s, z, token_mask, mask_dev)
            return z_new
        if stack is not None:
            return stack(z, mask_dev)
        b = bufs if b is None else b
        for tm in trimul:  # Pairformer order: triangle multiplication out, in, then the attention nodes
            z = tm(z, mask_dev, residual=True, buffers=b)
        z1 = start(z, mask_bias=pre.mask_bias, buffers=b, residual=True)
        z2 = end(z1, mask_bias=pre.mask_bias_transposed, buffers=b, residual=True, inplace_residual=True)
        if cfg["transition"]:
            z2 = trans(z2, residual=True, inplace=True)
        return z2

    launches_per_step = 6 + (1 if cfg["transition"] else 0) + 3 * len(trimul) + (8 if single else 0)
    flops_step = sum(2 * node_flops(L) + (transition_flops(L) if cfg["transition"] else 0.0)
                     + len(trimul) * trimul_flops(L, cfg["N"]) + (single_track_flops(L) if single else 0.0) for L in lens)
    if stack is not None:
        launches_per_step *= cfg["blocks"]
        flops_step *= cfg["blocks"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ---------------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step(z_dev)
    barrier()
    times = []
    with ClockSampler(local_rank) as clocks:
        barrier()
        for _ in range(args.steps):
            flush.fill_(1)  # evict L2 (126 MB) between timed steps
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step(z_dev)
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
        barrier()
    ms = sum(times) / len(times)
    ms_median, ms_min = sorted(times)[len(times) // 2], min(times)
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait during the benchmark")

    # ---- the same step replayed from a CUDA graph (launch overhead removed; L2 not flushed) ------------------
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(z_dev)
        with torch.cuda.graph(graph, stream=side):
            step(z_dev)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    reps = max(10, min(args.steps, 50))
    graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    e1.synchronize()
    graph_ms = e0.elapsed_time(e1) / reps
    del graph

    # ---- end to end: pinned host -> device -> step -> pinned host ----------------------------------------
    # Through the package's HostPipeline: every step copies its 64 MiB input in and its result out; the copies
    # of neighbouring steps overlap the compute on separate streams (two device slots, two buffer sets).
    z_pin = z_host.pin_memory()
    outs_pin = [torch.empty_like(z_pin).pin_memory() for _ in range(2)]
    slot_bufs: list[dict] = [{}, {}]

    def slot_step(zd, slot):
        if single:  # the single representation travels with its pair tensor: in before the step, out after it
            z_out = step(zd, slot_bufs[slot], s=s_pin.to(device, non_blocking=True))
            s_out_pin.copy_(last_s[0], non_blocking=True)
            return z_out
        return step(zd, slot_bufs[slot])

    pipe = b200.HostPipeline(slot_step, z_pin, device, depth=2)
    pipe.run([z_pin] * 4, [outs_pin[i & 1] for i in range(4)])  # warm-up
    barrier()
    t0 = time.perf_counter()
    pipe.run([z_pin] * args.steps, [outs_pin[i & 1] for i in range(args.steps)])
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    # the same path one step at a time (latency of a single pair tensor: copy in, compute, copy out)
    serial = []
    for i in range(3 + (3 if brief else min(args.steps, 20))):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        pipe.run([z_pin], [outs_pin[0]])
        if i >= 3:
            serial.append((time.perf_counter() - t0) * 1e3)
    e2e_serial_ms = sum(serial) / len(serial)
    if not torch.equal(outs_pin[0], outs_pin[1]):
        raise RuntimeError("pipelined end-to-end outputs differ between slots")

    # ---- per-kernel timing of the dominant kernel (attention core), live, with CUDA events ------------------
    B, N = cfg["B"], cfg["N"]
    packed = start._packed(device)
    qkvg, bias = ops.prologue(z_dev, packed)
    og = torch.empty(B, N, N, 128, dtype=torch.bfloat16, device=device)
    ktimes = []
    for i in range(3 + args.steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.attention(qkvg, bias, pre.mask_bias, B, N, N, out=og)
        e1.record()
        e1.synchronize()
        if i >= 3:
            ktimes.append(e0.elapsed_time(e1))
    attn_ms = sum(ktimes) / len(ktimes)
    attn_flops = sum(attention_core_flops(L) for L in lens)
    peak_tf, peak_gbs, peak_kind = measured_peaks()

    # ---- the single track's kernels one by one (CUDA events, L2 flushed before each launch) -----------------------
    single_kernels = None
    if single:
        import math

        layer = stack.layers[0]
        att, tr_s = layer.attention, layer.transition_s
        wts = att._weights(device)
        stats = ops.row_stats(s_dev)
        planes = ops.linear(s_dev, wts["w_in"], wts["sc_in"], ops.LINEAR_PLANES, B=B, rows=N, stats=stats)
        pbias = att.project_pair_bias(z_dev)
        len4 = torch.tensor(lens, dtype=torch.int32, device=device).repeat_interleave(4)
        q4, b4 = planes.view(4, 4 * B, 4, N, 32), pbias.view(4 * B, 4, N, pbias.shape[-1])
        o4 = ops.attention(q4, b4, len4, 4 * B, 1, N, scale=1 / math.sqrt(24))

        def event_us(fn):
            ts = []
            for i in range(13):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                e1.synchronize()
                if i >= 3:
                    ts.append(e0.elapsed_time(e1) * 1e3)
            return sorted(ts)[len(ts) // 2]

        pair_bias_us = event_us(lambda: att.project_pair_bias(z_dev, bias=pbias))
        pair_bias_bytes = z_dev.numel() * 2 + pbias.numel() * 2
        single_kernels = {
            "unit": "us per launch, median of 10",
            "row_stats": event_us(lambda: ops.row_stats(s_dev, stats=stats)),
            "linear_in_proj": event_us(lambda: ops.linear(s_dev, wts["w_in"], wts["sc_in"], ops.LINEAR_PLANES, B=B, rows=N,
                                                          stats=stats, out=planes)),
            "pair_bias": pair_bias_us,
            "pair_bias_roofline": {"bound": "hbm", "achieved": pair_bias_bytes / pair_bias_us / 1e3, "peak": peak_gbs,
                                   "unit": "GB/s", "frac": pair_bias_bytes / pair_bias_us / 1e3 / peak_gbs,
                                   "algorithmic_bytes": pair_bias_bytes},
            "attention_16_heads": event_us(lambda: ops.attention(q4, b4, len4, 4 * B, 1, N, out=o4, scale=1 / math.sqrt(24))),
            "linear_out_proj": event_us(lambda: ops.linear(o4, wts["w_o"], wts["sc_o"], ops.LINEAR_ROWS, B=B, rows=N,
                                                           a_strides=(4 * N * 128, 128, N * 128), residual=s_dev)),
            "transition_s_3_launches": event_us(lambda: tr_s(s_dev, residual=True)),
        }

    # ---- aggregate over ranks ------------------------------------------------------------------------------
    stats = torch.tensor([ms, e2e_ms, attn_ms], dtype=torch.float64, device=device)
    total_flops = torch.tensor([flops_step], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_flops, op=dist.ReduceOp.SUM)
    ms, e2e_ms, attn_ms = stats.tolist()
    flops_all = total_flops.item()
    bytes_io = z_host.numel() * 2 + (s_pin.numel() * 2 if single else 0)

    result = {
        "metric": "tri_attn_tflops", "value": flops_all / ms / 1e9, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "ms_per_step_median": ms_median,
        "ms_per_step_min": ms_min, "ms_per_step_cuda_graph_warm_l2": graph_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg['desc']}", "per_gpu_batch": cfg["B"], "tokens": cfg["N"],
                   "valid_lengths": cfg["valid"], "l2": "flushed between timed steps (256 MiB write)",
                   "empty_row_mode": "uniform", "parallelism": f"independent batches x{world}"},
        "e2e": {"value": flops_all / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": bytes_io, "d2h_bytes_per_step": bytes_io,
                "mode": "HostPipeline depth 2: copies of neighbouring steps overlap the compute",
                "single_step_latency_ms": e2e_serial_ms,
                "host_cores_per_rank": None if numa_cores is None else len(numa_cores)},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"kernel": "attention_kernel", "bound": "tensor", "achieved": attn_flops / attn_ms / 1e9,
                     "peak": peak_tf, "unit": "TFLOP/s", "frac": attn_flops / attn_ms / 1e9 / peak_tf,
                     "peak_source": f"{peak_kind} bf16 burst", "ms_per_launch": attn_ms, "traffic": TRAFFIC.get(args.workload)},
        "clocks": clocks.summary(),
    }
    if single_kernels is not None:
        result["single_track_kernels"] = single_kernels
    if rank == 0 and world == 1 and not brief and not args.no_cpu_baseline and not cfg.get("trimul"):
        result["cpu_baseline"] = cpu_baseline(cfg, args.workload)  # rows of the attention nodes and the transition only
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result if rank == 0 else {}


NVLINK_GBS = 900.0  # per direction per GPU, the figure the config-5 roofline is defined on


def sharded_check(args, world: int, rank: int, device) -> dict:
    """The sharded block against the same modules on one GPU, on a tensor small enough to hold whole on rank 0:
    z[1, 512, 512, 128] (1024 tokens on 8 ranks), the last 37 tokens padded, one block, the exchange form the
    benchmark uses.  Every rank takes part;
    rank 0 compares.  The block runs twice when the transposes are fused (the second call reuses the
    symmetric-memory shards, as consecutive blocks of the benchmark do)."""
    import torch.distributed as dist

    from bionemo_inference_runtime_b200 import sharded

    N = max(512, 128 * world)  # at least 128 pair rows per rank
    valid = N - 37
    n = N // world
    z = torch.randn(1, N, N, 128, generator=torch.Generator().manual_seed(77)).bfloat16().to(device)
    start, end, trans = build_modules(node_weights(7001), node_weights(7002), transition_weights(7003), device)
    idx = torch.arange(rank * n, (rank + 1) * n, device=device)
    lengths = torch.where(idx < valid, valid, 0).to(torch.int32).reshape(1, n)
    fused = args.exchange == "peer_stores"
    block = sharded.ShardedPairBlock(start, end, trans, fused_transpose=fused)
    out_rows = block(sharded.shard(z, rank, world), lengths, lengths)
    if fused:
        out_rows = block(sharded.shard(z, rank, world), lengths, lengths)
    gathered = [torch.empty_like(out_rows) for _ in range(world)]
    dist.all_gather(gathered, out_rows)
    verdict = torch.zeros(3, dtype=torch.float64, device=device)
    if rank == 0:
        full = torch.where(torch.arange(N, device=device) < valid, valid, 0).to(torch.int32).reshape(1, N)
        want = start(z, mask_bias=full, residual=True)
        want = end(want, mask_bias=full, residual=True)
        want = trans(want, residual=True)
        got = torch.cat(gathered, dim=1)
        diff = (got.float() - want.float()).abs()
        within = bool((diff <= 2e-2 + 2e-2 * want.float().abs()).all())
        verdict[0], verdict[1], verdict[2] = float(torch.equal(got, want)), float(diff.max()), float(within)
    dist.broadcast(verdict, src=0)
    torch.cuda.synchronize()
    del block
    return {"equal": bool(verdict[0].item()), "max_abs_diff": verdict[1].item(), "within_bf16_tolerance": bool(verdict[2].item()),
            "tolerance": "rtol = atol = 2e-2", "exchange": args.exchange, "tokens": N, "valid": valid, "blocks": 1,
            "against": "the same modules on rank 0 alone"}


def run_sharded(args) -> dict:
    """Benchmark config 5: one pair tensor z[1, 4096, 4096, 128] (3900 valid tokens) row-sharded over the ranks,
    4 pair-track blocks of start node -> transpose -> end node -> transition (-> transpose back).  The total work
    is fixed (strong scaling); with one rank the same blocks run on the whole tensor without any exchange."""
    import torch.distributed as dist

    import bionemo_inference_runtime_b200 as b200
    from bionemo_inference_runtime_b200 import _lib, ops, sharded
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cfg = WORKLOADS[args.workload]
    N, valid, nblocks = cfg["N"], int(cfg["valid"]), cfg["blocks"]
    if N % world:
        raise SystemExit(f"{N} pair rows do not divide over {world} ranks")
    check = None
    if world > 1:
        check = sharded_check(args, world, rank, device)
        if not check["within_bf16_tolerance"]:
            if rank == 0:
                print(json.dumps({"sharded_check": check, "error": "sharded block differs from the single-GPU modules"}),
                      flush=True)
            dist.barrier()
            dist.destroy_process_group()
            raise SystemExit(3)
    n = N // world
    gen = torch.Generator(device=device).manual_seed(2000 + rank)
    z_rows = torch.empty(1, n, N, 128, dtype=torch.bfloat16, device=device)
    for r0 in range(0, n, 256):  # generate in slabs: keeps the fp32 temporary small
        z_rows[:, r0:r0 + 256] = torch.randn(1, min(256, n - r0), N, 128, generator=gen, device=device).bfloat16()
    idx = torch.arange(rank * n, (rank + 1) * n, device=device)
    lengths_local = torch.where(idx < valid, valid, 0).to(torch.int32).reshape(1, n)  # m (x) m mask, rows == cols

    blocks = []
    for k in range(nblocks):
        start, end, trans = build_modules(node_weights(3000 + 3 * k), node_weights(3001 + 3 * k),
                                          transition_weights(3002 + 3 * k), device)
        blocks.append((start, end, trans))
    if world > 1:
        fused = args.exchange == "peer_stores"
        drivers = [sharded.ShardedPairBlock(s, e, t, fused_transpose=fused) for s, e, t in blocks]

        def step(z):
            for d in drivers:
                z = d(z, lengths_local, lengths_local)
            return z
    else:
        full_lengths = lengths_local

        def step(z):
            for s, e, t in blocks:
                z = s(z, mask_bias=full_lengths, residual=True, inplace_residual=True)
                z = e(z, mask_bias=full_lengths, residual=True, inplace_residual=True)
                z = t(z, residual=True, inplace=True)
            return z

    flops_block = 2 * node_flops(valid) + transition_flops(valid)
    flops_total = nblocks * flops_block
    launches = nblocks * 7

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    work = z_rows.clone()
    for _ in range(max(args.warmup, 3)):
        work.copy_(z_rows)
        step(work)
    barrier()
    times = []
    with ClockSampler(local_rank) as clocks:
        barrier()
        for _ in range(args.steps):
            work.copy_(z_rows)  # fresh input (the blocks work in place); the 4.3 GB / G copy also evicts L2
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step(work)
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
        barrier()
    ms = sum(times) / len(times)
    ms_median, ms_min = sorted(times)[len(times) // 2], min(times)
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait during the benchmark")

    # End to end: every step copies its shard in from pinned host memory, runs the blocks and copies the result back
    # to pinned host memory.  Two device buffers and two copy streams: the copy-in of step k + 1 and the copy-out of
    # step k - 1 run beside the compute of step k (the same pipelining as HostPipeline for the node workloads); the
    # timed region runs from the first copy-in to the last copy-out, fill and drain included.
    z_pin = z_rows.cpu().pin_memory()
    outs_pin = [torch.empty_like(z_pin).pin_memory() for _ in range(2)]
    bufs = [torch.empty_like(z_rows) for _ in range(2)]
    s_in, s_out, cur = torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.current_stream(device)
    e2e_steps = max(2, min(args.steps, 8))

    def e2e_run(count: int) -> float:
        ev_out: list = []
        barrier()
        t0 = time.perf_counter()
        for k in range(count):
            b = k % 2
            ev_in = torch.cuda.Event()
            with torch.cuda.stream(s_in):
                if k >= 2:
                    s_in.wait_event(ev_out[k - 2])  # the buffer's previous result has left the device
                bufs[b].copy_(z_pin, non_blocking=True)
                ev_in.record(s_in)
            cur.wait_event(ev_in)
            res = step(bufs[b])
            if res.data_ptr() != bufs[b].data_ptr():
                bufs[b].copy_(res)
            ev_done = torch.cuda.Event()
            ev_done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done)
                outs_pin[b].copy_(bufs[b], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_out)
                ev_out.append(ev)
        barrier()
        return (time.perf_counter() - t0) * 1e3 / count

    e2e_run(1)
    e2e_ms = e2e_run(e2e_steps)
    del bufs

    # dominant kernel on this rank's shard of the first block's starting node
    start = blocks[0][0]
    packed = start._packed(device)
    bias_loc = torch.empty((1, 4, n, ops.pad8(N)), dtype=torch.bfloat16, device=device)
    qkvg, bias_loc = ops.prologue(z_rows, packed, bias=bias_loc)
    bias_full = sharded.gather_bias(bias_loc) if world > 1 else bias_loc
    og = torch.empty(1, n, N, 128, dtype=torch.bfloat16, device=device)
    ktimes = []
    for i in range(4):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.attention(qkvg, bias_full, lengths_local, 1, n, N, out=og)
        e1.record()
        e1.synchronize()
        if i >= 1:
            ktimes.append(e0.elapsed_time(e1))
    attn_ms = sum(ktimes) / len(ktimes)
    attn_flops = float((lengths_local > 0).sum().item()) * valid * 512.0 * valid
    del qkvg, og, bias_full, bias_loc
    peak_tf, peak_gbs, peak_kind = measured_peaks()

    stats = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms, e2e_ms = stats.tolist()
    shard_bytes = z_rows.numel() * 2
    a2a_bytes = 0 if world == 1 else int(shard_bytes * (world - 1) / world)
    # roofline of one block as the configuration defines it: the slower of (flops at the bf16 peak, compulsory bytes
    # at the copy bandwidth) per GPU, plus the bytes of the two transposes at the link bandwidth
    block_ms = ms / nblocks
    t_flops = flops_block / world / (peak_tf * 1e12) * 1e3
    t_bytes = 3 * 512.0 * N * N / world / (peak_gbs * 1e9) * 1e3  # three modules, 512 B per position each
    t_links = 2 * a2a_bytes / (NVLINK_GBS * 1e9) * 1e3
    t_roof = max(t_flops, t_bytes) + t_links
    if world > 1:
        transposes = ("rows->columns by peer stores from the starting node's output kernel, columns->rows by peer TMA "
                      "stores from the transition kernel" if args.exchange == "peer_stores" else "2 NCCL all-to-all")
        collectives = (f"per block: 2 all-gathers of the triangle bias ({N * ops.pad8(N) * 4 * 2} B in total each)"
                       + (" and 2 one-element all-reduces that order the peer stores" if args.exchange == "peer_stores"
                          else " and 2 all-to-all of the shard"))
        parallelism = f"pair rows sharded x{world}; {transposes}; {a2a_bytes} B per rank and transpose cross the links"
    else:
        collectives, parallelism = "none", "pair rows sharded x1 (single GPU, no exchange)"
    clk = clocks.summary()
    attn_peak, attn_peak_name = peak_for_step(peak_tf, clk, ms)
    result = {
        "metric": "tri_attn_tflops", "value": flops_total / ms / 1e9, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "ms_per_step_median": ms_median,
        "ms_per_step_min": ms_min, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg['desc']}", "tokens": N, "valid_lengths": cfg["valid"],
                   "blocks": nblocks, "block_ms": block_ms, "l2": "inputs far larger than L2 (4.3 GB pair tensor)",
                   "empty_row_mode": "uniform", "parallelism": parallelism, "collectives": collectives},
        "e2e": {"value": flops_total / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": shard_bytes, "d2h_bytes_per_step": shard_bytes,
                "mode": f"each rank copies its row shard in from pinned host memory, runs the 4 blocks, copies it back; "
                        f"two device buffers, the copies of neighbouring steps overlap the compute; {e2e_steps} steps "
                        "timed from the first copy-in to the last copy-out"},
        "gpu_launches": launches * args.steps,
        "roofline": {"kernel": "attention_kernel", "bound": "tensor", "achieved": attn_flops / attn_ms / 1e9,
                     "peak": attn_peak, "unit": "TFLOP/s", "frac": attn_flops / attn_ms / 1e9 / attn_peak,
                     "frac_of_burst": attn_flops / attn_ms / 1e9 / peak_tf,
                     "peak_source": f"{peak_kind} {attn_peak_name}", "ms_per_launch": attn_ms,
                     "traffic": TRAFFIC[args.workload] / world,
                     "note": "rank 0's shard of one starting node; algorithmic flops = 512 x valid keys per valid position; "
                             "traffic scaled by pair positions from the ncu capture of the 512-token launch"},
        "roofline_block": {"definition": "max(flops / bf16 peak, 3 x 512 B per position / HBM) per GPU + bytes of the two "
                                         "transposes / 900 GB/s", "flops_ms": t_flops, "hbm_ms": t_bytes,
                           "links_ms": t_links, "roofline_ms": t_roof, "block_ms": block_ms, "frac": t_roof / block_ms,
                           "peaks": f"{peak_kind}: {peak_tf} TFLOP/s bf16 burst, {peak_gbs} GB/s copy; NVLink nominal"},
        "clocks": clk,
    }
    if check is not None:
        result["sharded_check"] = check
    del work, z_rows, z_pin, outs_pin, blocks
    torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return {}
    if world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline_rows_scaled(cfg, args.workload)
    if world == 1 and not args.no_also:
        result["also"] = {}
        for name in ("cfg2", "n768"):
            sub = argparse.Namespace(**{**vars(args), "workload": name, "steps": ALSO_STEPS, "blocks": None})
            r = run_ours(sub, brief=True)
            result["also"][name] = {k: r[k] for k in ("value", "unit", "steps", "ms_per_step", "ms_per_step_median",
                                                      "ms_per_step_cuda_graph_warm_l2", "config", "e2e", "gpu_launches",
                                                      "roofline", "clocks")}
            torch.cuda.empty_cache()
    return result


# dram__bytes_read.sum + dram__bytes_write.sum per attention launch, from the committed ncu summary of the cfg2
# capture (profiles/attention_kernel_cfg2.md: 270.6 MB read + 53.4 MB written for 512 x 512 positions).  The traffic is
# the q / k / v / gate planes read once and the output written once, i.e. proportional to the pair positions of the
# launch, so the larger workloads scale that capture by their positions (cfg5: one rank's shard of a node).
TRAFFIC_PER_POSITION = 324.0e6 / (512 * 512)
TRAFFIC: dict[str, float | None] = {"cfg2": 324.0e6, "cfg3": None, "n768": TRAFFIC_PER_POSITION * 768 * 768,
                                    "cfg5": TRAFFIC_PER_POSITION * 4096 * 4096}


def cpu_sample(cfg: dict, rows: int, threads: int):
    """Times the oracle (CPU restatement of the reference's eager path, fp32) on a row sample of the workload."""
    from oracle import triangle_oracle as orc

    torch.set_num_threads(threads)
    z, mask, lens, w_start, w_end, w_tr = make_inputs(cfg, 1000, "cpu")
    w_start, w_end = (orc.NodeWeights(w.ln_w, w.ln_b, w.w_bias, w.w_in, w.b_in, w.w_out, w.b_out) for w in (w_start, w_end))
    w_tr = orc.TransitionWeights(w_tr.ln_w, w_tr.ln_b, w_tr.w1, w_tr.w2)
    B, N = cfg["B"], cfg["N"]
    items = min(B, 2)
    z, mask = z[:items].float(), mask[:items]
    rows = min(rows, N)
    sel = torch.linspace(0, max(lens[0] - 1, 0), rows).long().unique()  # valid rows of the first item, spread out

    t0 = time.perf_counter()
    orc.node_forward_rows(z, mask, w_start, orc.STARTING, sel, residual=True)
    orc.node_forward_rows(z, mask, w_end, orc.ENDING, sel, residual=True)
    if cfg["transition"]:
        orc.transition_forward(z[:, sel], None, w_tr, residual=True)
    dt = time.perf_counter() - t0
    # flops of the sample: rows x valid columns of each sampled item (LayerNorm/bias of unsampled rows earn nothing)
    fl = 0.0
    for b in range(items):
        L = lens[b]
        r = int((sel < L).sum())
        fl += 2 * r * L * (164864.0 + 512.0 * L) + (r * L * 393216.0 if cfg["transition"] else 0.0)
    return fl, dt, len(sel), items


def cpu_baseline(cfg: dict, name: str, rows: int = 128, budget_s: float = 12.0) -> dict:
    """Repeats the row sample until about ``budget_s`` seconds of CPU work have been timed."""
    threads = os.cpu_count() or 1
    cpu_sample(cfg, 16, threads)  # warm the thread pool and the allocator
    fl = dt = 0.0
    nrows = items = reps = 0
    while dt < budget_s and reps < 64:
        f, d, nrows, items = cpu_sample(cfg, rows, threads)
        fl, dt, reps = fl + f, dt + d, reps + 1
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "seconds": dt,
            "sample": f"{name}: {reps} x ({nrows} of {cfg['N']} pair rows of {items} item(s)), both nodes"
                      f"{' + transition' if cfg['transition'] else ''}, fp32 eager restatement (oracle/), torch CPU"}


class CpuRowSampler:
    """The CPU restatement on a row sample of a workload too large to run whole on the host (config 5: the eager
    path's logits alone would need 1.1 TB).  The triangle bias of ALL pair rows is computed once per node (that is
    whole-node work and is timed as such); a step then runs ``rows`` sampled pair rows of both nodes and of the
    transition, in chunks of 16 rows, and the node time is extrapolated as bias + rows-time x N / rows (the eager
    path computes every row, padded ones included; rows are independent given the bias)."""

    def __init__(self, cfg: dict, threads: int):
        from oracle import triangle_oracle as orc

        self.orc, self.cfg = orc, cfg
        torch.set_num_threads(threads)
        N, valid = cfg["N"], int(cfg["valid"])
        self.N, self.valid = N, valid
        slab = torch.randn(1, 256, N, 128, generator=torch.Generator().manual_seed(1000)).bfloat16()
        self.z = slab.repeat(1, N // 256, 1, 1)  # z ~ N(0,1), a seeded 256-row slab tiled to N rows (4.3 GB in bf16)
        ws, we, wt = node_weights(3000), node_weights(3001), transition_weights(3002)
        self.w = [orc.NodeWeights(w.ln_w, w.ln_b, w.w_bias, w.w_in, w.b_in, w.w_out, w.b_out) for w in (ws, we)]
        self.wt = orc.TransitionWeights(wt.ln_w, wt.ln_b, wt.w1, wt.w2)
        self.m = (torch.arange(N) < valid).float()
        t0 = time.perf_counter()
        self.tb = [orc.triangle_bias(self.z, self.w[k], k) for k in (orc.STARTING, orc.ENDING)]
        self.bias_s = time.perf_counter() - t0  # both nodes, all rows
        self.cursor = 0

    def step(self, rows: int) -> float:
        orc, N = self.orc, self.N
        sel = (torch.arange(rows) * (N // rows) + self.cursor) % N  # spread over valid and padded rows alike
        self.cursor += 1
        t0 = time.perf_counter()
        for c0 in range(0, rows, 16):
            r = sel[c0:c0 + 16]
            mk = (self.m[r, None] * self.m[None, :])[None]  # m (x) m restricted to the sampled rows
            for k in (orc.STARTING, orc.ENDING):
                orc.node_forward_rows(self.z, mk, self.w[k], k, r, residual=True, tri_bias=self.tb[k])
            orc.transition_forward(self.z[:, r].float(), None, self.wt, residual=True)
        return time.perf_counter() - t0

    def flops_per_block(self) -> float:
        return 2 * node_flops(self.valid) + transition_flops(self.valid)

    def block_seconds(self, step_s: float, rows: int) -> float:
        return self.bias_s + step_s * self.N / rows

    def describe(self, rows: int, reps: int) -> str:
        return (f"{reps} x ({rows} of {self.N} pair rows in chunks of 16, both nodes + transition) + the triangle bias "
                f"of all rows once ({self.bias_s:.1f} s), extrapolated to one block as bias + rows-time x {self.N}/{rows}; "
                "fp32 eager restatement (oracle/), torch CPU")


def cpu_baseline_rows_scaled(cfg: dict, name: str, rows: int = 16, budget_s: float = 12.0) -> dict:
    threads = os.cpu_count() or 1
    sampler = CpuRowSampler(cfg, threads)
    sampler.step(16)  # warm the thread pool and the allocator
    dt, reps = 0.0, 0
    while dt < budget_s and reps < 16:
        dt += sampler.step(rows)
        reps += 1
    block_s = sampler.block_seconds(dt / reps, rows)
    return {"value": sampler.flops_per_block() / block_s / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "seconds": dt + sampler.bias_s, "extrapolated_block_seconds": block_s,
            "sample": f"{name}: " + sampler.describe(rows, reps)}


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    cfg = WORKLOADS[args.workload]
    threads = os.cpu_count() or 1
    world = int(os.environ.get("WORLD_SIZE", "1"))
    warmup = max(args.warmup, 0)
    if cfg.get("sharded"):
        rows = 8
        sampler = CpuRowSampler(cfg, threads)
        for _ in range(warmup):
            sampler.step(rows)
        dt = sum(sampler.step(rows) for _ in range(args.steps))
        block_s = sampler.block_seconds(dt / args.steps, rows)
        value = sampler.flops_per_block() / block_s / 1e12
        sample = f"{args.workload}: " + sampler.describe(rows, args.steps)
        ms_step = dt / args.steps * 1e3
    else:
        for _ in range(warmup):
            cpu_sample(cfg, 48, threads)
        fl = dt = 0.0
        nrows = items = 0
        for _ in range(args.steps):
            f, d, nrows, items = cpu_sample(cfg, 48, threads)
            fl += f
            dt += d
        value = fl / dt / 1e12
        sample = (f"{args.workload}: {nrows} of {cfg['N']} pair rows of {items} item(s) per step, both nodes"
                  f"{' + transition' if cfg['transition'] else ''}, fp32 eager restatement (oracle/), torch CPU")
        ms_step = dt / args.steps * 1e3
    return {"impl": "reference", "metric": "tri_attn_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong" if cfg.get("sharded") else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {cfg['desc']}", "sampled": sample},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default depends on the workload)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="cfg5")
    ap.add_argument("--blocks", type=int, default=None,
                    help="override the number of blocks of a stack workload (cfg4, cfg4pair), e.g. 1 for a profile")
    ap.add_argument("--exchange", choices=["all_to_all", "peer_stores"], default="peer_stores",
                    help="sharded workloads: how the rows->columns transpose crosses the links (NCCL all-to-all, or "
                         "stores from the starting node's output kernel into the peers' column shards)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true",
                    help="single-GPU run of the default workload: leave out the extra cfg2 / n768 figures")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = DEFAULT_STEPS[args.workload] if args.impl == "ours" else 5
    if args.impl == "reference":
        result = run_reference(args)
    elif WORKLOADS[args.workload].get("sharded"):
        result = run_sharded(args)
    else:
        result = run_ours(args)
    if result:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()

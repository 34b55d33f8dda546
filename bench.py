#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

One "step" = one pass of a dense decoder MLP block over one batch of M tokens:
  BF16 activations -> dynamic MXFP8 quantisation -> gate_up GEMM with fused SwiGLU + MXFP8
  requant -> down GEMM -> (row-parallel all-reduce +) residual add + RMSNorm.
Workload: the benchmark configuration "MXFP8 dense decoder MLP block" (hidden 2560, intermediate 9728),
headline batch M = 4096; with --gpus N the MLP is tensor-parallel over N GPUs (gate_up
column-parallel, down row-parallel, total work fixed => strong scaling).

Prints ONE JSON line (rank 0). `value` is device-resident throughput (CUDA events, max over
ranks); `e2e` is the same step driven through the public Python API with pinned host buffers,
host->device and device->host copies inside the timed region.

`--impl reference` times the reference's own CPU statement of the path (quantise ->
dequantise -> FP32 matmul -> BF16, tests/native_mxfp6/test_mxfp8_sm120.py:53-57 of the
reference, restated in oracle/mx_oracle.py) on the host cores, at the GPU arm's batch size.
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
sys.path.insert(0, str(ROOT / "vllm-mach_b200"))

import torch  # noqa: E402

HIDDEN, INTER = 2560, 9728
HEADLINE_M = 4096
SWEEP_M = (1, 8, 16, 64, 256, 1024, 4096)
EPS = 1e-6
NUM_WEIGHT_SETS = 4       # 4 x 77 MB > 126 MB L2: weights always come from HBM
CPU_SAMPLE_TOKENS = HEADLINE_M   # the CPU arm runs the GPU arm's configuration
SOAK_SECONDS = 1.0
STEP_VARIANTS = 4         # step i uses input i % 4 and weight set i % NUM_WEIGHT_SETS
KERNEL_TIMING_LAUNCHES = 200     # launches of the dominant kernel timed one by one
OWNER_MIN_BYTES = 1 << 20        # tensor-parallel payloads above this take the owner form


def owner_min_bytes(world: int) -> int:
    """Payload from which the owner form is faster than the push form. Measured on B200s
    (fused reduce alone, hidden 2560, microseconds push / owner): two GPUs 10.9 / 14.8 at 64
    tokens and 15.9 / 15.7 at 256; four GPUs 15.7 / 15.8 and 18.6 / 16.9; eight GPUs 19.0 / 16.9
    and 21.4 / 18.3."""
    return OWNER_MIN_BYTES if world <= 2 else OWNER_MIN_BYTES // 4
TRAFFIC_FILE = ROOT / "profiles" / "ncu_traffic.json"


def ncu_traffic(kernel: str, tokens: int):
    """DRAM bytes (read + write) per launch from the committed profiler capture of
    `bench.py --kernel-only <kernel> --tokens <tokens>`, with where it came from."""
    try:
        entry = json.loads(TRAFFIC_FILE.read_text())[kernel][str(tokens)]
        return entry["dram_read_bytes"] + entry["dram_write_bytes"], entry["source"]
    except (OSError, KeyError, ValueError):
        return None, None


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def shard_blocks(inter: int, world: int, rank: int) -> tuple[int, int]:
    """Intermediate dimension split in whole 32-feature blocks (one MX scale block of the down
    projection, one gate/up row group of the fused gate_up). Returns (first feature, count)."""
    blocks = inter // 32
    base, extra = divmod(blocks, world)
    counts = [base + (1 if r < extra else 0) for r in range(world)]
    start = sum(counts[:rank])
    return start * 32, counts[rank] * 32


# ------------------------------------------------------------------ clocks sampler
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); sm_max.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ GPU arm
def make_weights(device, world, rank, seed, hidden=HIDDEN, inter=INTER, fmt="e4m3", sigma=0.02,
                 logical=False):
    """Synthetic weights with the checkpoint's shapes: BF16 ~N(0, sigma) quantised on the
    device (E4M3 codes + E8M0 per 1x32; for the 6-bit formats the E4M3 codes are replaced by
    seeded random 6-bit codes, timing only). Returns MxMlpWeights of this rank's shard; with
    `logical` also the shard's checkpoint-layout tensors (codes, scales) of both matrices."""
    from mach_b200 import native
    from mach_b200.mlp import MxMlpWeights
    start, count = shard_blocks(inter, world, rank)
    g = torch.Generator(device=device).manual_seed(seed)
    w_gu = (torch.randn(2 * inter, hidden, generator=g, device=device) * sigma).to(torch.bfloat16)
    w_d = (torch.randn(hidden, inter, generator=g, device=device) * sigma).to(torch.bfloat16)
    gate = w_gu[start:start + count]
    up = w_gu[inter + start:inter + start + count]
    shard_gu = torch.cat([gate, up], 0).contiguous()
    shard_d = w_d[:, start:start + count].contiguous()
    del w_gu, w_d
    c_gu, s_gu = native.quantize_mxfp8(shard_gu)
    c_d, s_d = native.quantize_mxfp8(shard_d)
    l_gu = native.unpack_scales(s_gu, shard_gu.shape[0], hidden)
    l_d = native.unpack_scales(s_d, hidden, count)
    if fmt != "e4m3":
        c_gu = torch.randint(0, 256, (2 * count, hidden * 3 // 4), dtype=torch.uint8, device=device,
                             generator=g)
        c_d = torch.randint(0, 256, (hidden, count * 3 // 4), dtype=torch.uint8, device=device,
                            generator=g)
    weights = MxMlpWeights.from_logical(c_gu, l_gu, c_d, l_d, hidden, fmt=fmt)
    if logical:
        return weights, (c_gu, l_gu, c_d, l_d)
    return weights


def gemm_flops(m, inter_local, hidden=HIDDEN):
    return 2.0 * m * (2 * inter_local) * hidden + 2.0 * m * hidden * inter_local


def mlp_bytes(m, inter_local, hidden=HIDDEN, weight_bytes=1.0):
    """Algorithmic HBM bytes of one MLP pass: weights + scales once, activations in,
    FP8 intermediate written and read once, BF16 output."""
    w = 3 * inter_local * hidden * (weight_bytes + 1 / 32)
    return w + m * hidden * 2 + 2 * m * inter_local * (1 + 1 / 32) + m * hidden * 2


def bf16_ulps(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance between two BF16 tensors in units in the last place."""
    def key(t):
        bits = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        return torch.where(bits >= 0x8000, 0x8000 - bits, bits)
    return int((key(a) - key(b)).abs().max()) if a.numel() else 0


def tp_step(x, residual, residual_rows, gamma, w, group, owner):
    """One MLP block. Tensor-parallel payloads above OWNER_MIN_BYTES keep the residual stream
    and the BF16 norm row-owned and replicate the MXFP8 codes (owner form); smaller ones, and
    one GPU, return norm and residual for all rows."""
    from mach_b200.mlp import mlp_block, mlp_block_owner
    if owner or group is None:
        codes, scales, res_rows, norm_rows = mlp_block_owner(x, residual_rows, gamma, EPS, w, group,
                                                             codes_in_workspace=True)
        return norm_rows, (codes, scales, res_rows)
    norm, res = mlp_block(x, residual, gamma, EPS, w, group)
    return norm, (res,)


def tp_parity(group, world, rank, device, tokens):
    """Checker leg, outside every timed region: the tensor-parallel block on `tokens` seeded
    rows against the CPU oracle. (1) the fused reduce vs the oracle's rank-order sum +
    residual + norm over the ranks' gathered partial sums: residual_out bit-equal, norm within
    one BF16 ulp, codes and scales equal to the oracle quantiser applied to the kernel's own
    norm; (2) relative Frobenius error of the normalised output against the oracle's UNSHARDED
    MLP (quantise -> dequantise -> FP32 matmul path) on a row sample."""
    import torch.distributed as dist
    from mach_b200 import collective, native
    from mach_b200.mlp import mlp_forward
    from oracle import mx_oracle as ora   # checker only
    g = torch.Generator().manual_seed(4242 + tokens)
    x = torch.randn(tokens, HIDDEN, generator=g).to(torch.bfloat16).to(device)
    residual = torch.randn(tokens, HIDDEN, generator=g).to(torch.bfloat16).to(device)
    gamma = (0.1 * torch.randn(HIDDEN, generator=g)).to(torch.bfloat16).to(device)
    w, (c_gu, l_gu, c_d, l_d) = make_weights(device, world, rank, 1000, logical=True)
    partial = mlp_forward(x, w)
    owner = tokens * HIDDEN * 2 > owner_min_bytes(world)
    first, count = collective.owner_rows(tokens, group)
    if owner:
        norm_rows, (codes, scales, res_rows) = tp_step(
            x, residual, residual[first:first + count].contiguous(), gamma, w, group, True)
        norm = collective.gather_owned_rows(norm_rows, tokens, group)
        res = collective.gather_owned_rows(res_rows, tokens, group)
    else:
        norm, res, codes, scales = collective.allreduce_add_rmsnorm(
            partial, residual, gamma, EPS, group, want_quant=True)
    torch.cuda.synchronize()
    status = native.device_status()
    parts = [torch.empty_like(partial) for _ in range(world)] if rank == 0 else None
    dist.gather(partial, parts, dst=0, group=group)
    # full checkpoint-layout weights on rank 0: gate rows | up rows, down columns by shard
    half = c_gu.shape[0] // 2
    mine = [t.contiguous().view(torch.uint8).cpu().numpy()
            for t in (c_gu[:half], c_gu[half:], l_gu[:half], l_gu[half:], c_d, l_d)]
    shards = [None] * world if rank == 0 else None
    dist.gather_object(mine, shards, dst=0, group=group)
    if rank != 0:
        return None
    ref_norm, ref_res = ora.allreduce_rmsnorm([p.cpu() for p in parts], residual.cpu(),
                                              gamma.cpu(), EPS)
    ref_codes, ref_scales = ora.quantize_mxfp8(norm.cpu())
    gate_c, up_c, gate_s, up_s = (torch.cat([torch.from_numpy(sh[i]) for sh in shards], 0)
                                  for i in range(4))
    down_c, down_s = (torch.cat([torch.from_numpy(sh[i]) for sh in shards], 1) for i in (4, 5))
    rows = torch.randperm(tokens, generator=g)[:32]
    a_c, a_s = ora.quantize_mxfp8(x.cpu()[rows])
    w_gu = ora.dequantize_mx(torch.cat([gate_c, up_c], 0).view(torch.uint8),
                             torch.cat([gate_s, up_s], 0))
    h_c, h_s = ora.swiglu_quantize(ora.mx_gemm(a_c, a_s, w_gu))
    y = ora.mx_gemm(h_c, h_s, ora.dequantize_mx(down_c.view(torch.uint8), down_s))
    full_norm, _ = ora.allreduce_rmsnorm([y], residual.cpu()[rows], gamma.cpu(), EPS)
    got = norm.cpu()[rows].float()
    return {
        "n": world, "tokens": tokens, "form": "owner" if owner else "push",
        "residual_equal": bool(torch.equal(res.cpu().view(torch.int16), ref_res.view(torch.int16))),
        "norm_max_ulp": bf16_ulps(norm.cpu(), ref_norm),
        "codes_equal": bool(torch.equal(codes.view(torch.uint8).cpu(), ref_codes)
                            and torch.equal(ora.unswizzle_scales(scales.cpu(), tokens, HIDDEN),
                                            ref_scales)),
        "rel_fro_vs_unsharded_oracle": float((got - full_norm.float()).norm()
                                             / full_norm.float().norm()),
        "device_status": status,
    }


def fp8_library_peak(device):
    """cuBLASLt through torch on this box: per-tensor-scaled E4M3 8192^3 (burst = best of 10,
    sustained = back to back for ~1.5 s) and, where the installed torch accepts it, the MXFP8
    block-scaled form at the two shapes of the benchmarked MLP."""
    import torch.nn.functional as F
    out = {}

    def time_fn(fn, flops, seconds):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(seconds * 1e3 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return flops / (best * 1e-3) / 1e12, flops * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12

    try:
        n = 8192
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=device)
        burst, sustained = time_fn(lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one,
                                                            out_dtype=torch.bfloat16),
                                   2.0 * n ** 3, 1.5)
        out["e4m3_tensorwise_8192"] = {"burst": round(burst, 1), "sustained": round(sustained, 1)}
    except Exception as error:  # noqa: BLE001
        out["e4m3_tensorwise_8192"] = {"error": str(error)[:160]}
    for name, (m, n, k) in (("mxfp8_gate_up_4096x19456x2560", (HEADLINE_M, 2 * INTER, HIDDEN)),
                            ("mxfp8_down_4096x2560x9728", (HEADLINE_M, HIDDEN, INTER))):
        try:
            a = torch.randn(m, k, device=device).to(torch.float8_e4m3fn)
            b = torch.randn(n, k, device=device).to(torch.float8_e4m3fn).t()
            sa = torch.full((((m + 127) // 128) * 128 * ((k // 32 + 3) // 4) * 4,), 1.0,
                            device=device).to(torch.float8_e8m0fnu)
            sb = torch.full((((n + 127) // 128) * 128 * ((k // 32 + 3) // 4) * 4,), 1.0,
                            device=device).to(torch.float8_e8m0fnu)
            fn = lambda: F.scaled_mm(a, b, sa, F.ScalingType.BlockWise1x32, sb,  # noqa: E731
                                     F.ScalingType.BlockWise1x32,
                                     swizzle_a=F.SwizzleType.SWIZZLE_32_4_4,
                                     swizzle_b=F.SwizzleType.SWIZZLE_32_4_4,
                                     output_dtype=torch.bfloat16)
            burst, sustained = time_fn(fn, 2.0 * m * n * k, 0.5)
            out[name] = {"burst": round(burst, 1), "sustained": round(sustained, 1)}
        except Exception as error:  # noqa: BLE001
            out[name] = {"error": str(error)[:160]}
    return out


def run_gpu(args):
    import torch.distributed as dist
    from mach_b200 import collective, native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    native.lib()
    peaks = measured_peaks()
    m = args.tokens
    _, inter_local = shard_blocks(INTER, world, rank)
    owner = world > 1 and not args.no_owner and m * HIDDEN * 2 > owner_min_bytes(world)

    sets = [make_weights(device, world, rank, 1000 + i) for i in range(NUM_WEIGHT_SETS)]
    g = torch.Generator(device=device).manual_seed(7)
    xs = [torch.randn(m, HIDDEN, generator=g, device=device).to(torch.bfloat16) for _ in range(4)]
    residual = torch.randn(m, HIDDEN, generator=g, device=device).to(torch.bfloat16)
    gamma = (0.1 * torch.randn(HIDDEN, generator=g, device=device)).to(torch.bfloat16)
    first, count = collective.owner_rows(m, group)
    residual_rows = residual[first:first + count].contiguous()

    def step(i):
        return tp_step(xs[i % 4], residual, residual_rows, gamma, sets[i % NUM_WEIGHT_SETS], group,
                       owner)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.kernel_only:
        run_kernel_only(args, xs, sets, device)
        return

    # ---- device-resident timing
    barrier()   # the ranks built their weights at different speeds; start the first step together
    for i in range(args.warmup):
        step(i)
    barrier()
    # Safety net: if a device-side wait of the owner form gave up during warm-up on any rank
    # (status 401 / 402 / 403), say so in the line and measure the push form instead of
    # publishing numbers computed on poisoned activations.
    reduce_note = None

    def status_over_ranks():
        code = torch.tensor([float(native.device_status())], device=device)
        if world > 1:
            dist.all_reduce(code, op=dist.ReduceOp.MAX)
        return int(code.item())

    def fall_back(where, code):
        nonlocal owner, reduce_note
        reduce_note = f"owner form gave up during {where} (device status {code})"
        collective.poll_status()
        for ws in list(collective._workspaces.values()):
            ws.reset()
        owner = False
        for i in range(args.warmup):
            step(i)
        barrier()

    if world > 1:
        code = status_over_ranks()
        if code != 0:
            fall_back("warm-up", code)

    # The steps of the loop are captured once per (input, weight set) pair and replayed, as a
    # serving engine does: with N ranks a step lasts little longer than the Python and ctypes
    # calls that launch its kernels one by one, and a host thread that is descheduled for a
    # moment would stall every rank through the reduce.
    def capture_steps():
        """([single-step graphs], chain graph of STEP_VARIANTS consecutive steps) or ([], None)."""
        graphs, chain, fine = [], None, True
        # No collective call sits inside a try block: a rank whose capture fails still takes
        # part in every barrier, and the vote below puts all ranks on the same route.
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for j in range(STEP_VARIANTS):
                    step(j)
            torch.cuda.current_stream().wait_stream(side)
        except RuntimeError:
            fine = False
        barrier()
        if fine:
            try:
                for j in range(STEP_VARIANTS):
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        result = step(j)
                    graphs.append((graph, result))
                # Consecutive blocks of one graph keep the programmatic-dependent-launch chain
                # across the block boundary, as the layers of a captured forward pass do.
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for j in range(STEP_VARIANTS):
                        result = step(j)
                chain = (graph, result)
            except RuntimeError:
                graphs, chain = [], None
        barrier()
        ok = torch.tensor([1.0 if graphs else 0.0], device=device)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)   # every rank takes the same route
        return (graphs, chain) if ok.item() != 0.0 else ([], None)

    step_graphs, step_chain = ([], None) if args.no_step_graphs else capture_steps()

    def run_steps(first, count, marks=None, marked=None):
        """Steps first .. first + count - 1 (first a multiple of STEP_VARIANTS): whole chains of
        STEP_VARIANTS steps, then single steps. Records marks[i] after step i where it can (after
        every step, or at the end of a chain). Returns the last step's result."""
        result, i = None, first
        while i < first + count:
            if step_chain is not None and i % STEP_VARIANTS == 0 and i + STEP_VARIANTS <= first + count:
                step_chain[0].replay()
                result = step_chain[1]
                i += STEP_VARIANTS
            elif step_graphs:
                graph, result = step_graphs[i % STEP_VARIANTS]
                graph.replay()
                i += 1
            else:
                result = step(i)
                i += 1
            if marks is not None:
                marks[i - first - 1].record()
                marked.append(i - first - 1)
        return result

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # Untimed soak (extra warm-up): nvidia-smi samples every 50 ms, a 50-step timed region lasts
    # ~20 ms, so the same steps run for about a second first; the sampler then covers the soak,
    # the timed region, the per-kernel timing and the end-to-end region.
    soak_steps = 0
    soak_until = time.perf_counter() + args.soak
    while args.soak > 0:
        run_steps(soak_steps, 16)
        soak_steps += 16
        torch.cuda.synchronize()
        flag = torch.tensor([1.0 if time.perf_counter() < soak_until else 0.0], device=device)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if flag.item() == 0.0:
            break
    if world > 1 and owner:
        code = status_over_ranks()
        if code != 0:
            fall_back("the soak", code)
            step_graphs, step_chain = ([], None) if args.no_step_graphs else capture_steps()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    if world > 1:
        # A rank whose host thread leaves the barrier late would be waited for inside the first
        # step's reduce of every other rank. This all-reduce is only ENQUEUED here: the device
        # passes it once every rank has enqueued it, and each host follows it at once with the
        # start event and the steps, so the timed region starts on all ranks together.
        gate = torch.zeros(1, device=device)
        dist.all_reduce(gate)
    start.record()
    marked = []
    out = run_steps(0, args.steps, marks, marked)
    end.record()
    barrier()
    ms = start.elapsed_time(end)
    ms_rank = ms
    # longest stretch between two recorded marks, per step (diagnostic: a stalled rank shows up
    # here); marks inside a chain of steps are not recorded
    step_ms, last, last_i = [0.0] * args.steps, start, -1
    for i in marked:
        span = last.elapsed_time(marks[i]) / (i - last_i)
        for j in range(last_i + 1, i + 1):
            step_ms[j] = span
        last, last_i = marks[i], i
    worst_step = max(range(args.steps), key=lambda i: step_ms[i])
    status_timed = status_over_ranks() if world > 1 else native.device_status()
    assert torch.isfinite(out[0].float()).all()

    # ---- dominant kernel (gate_up GEMM with the SwiGLU epilogue): every launch timed with its
    # own pair of CUDA events on its stream; median and spread over KERNEL_TIMING_LAUNCHES
    codes, scales = native.quantize_mxfp8(xs[0])
    evs = []
    for i in range(args.warmup):
        native.mx_gemm_swiglu(codes, scales, sets[i % NUM_WEIGHT_SETS].w_gate_up,
                              sets[i % NUM_WEIGHT_SETS].s_gate_up, layout=native.LAYOUT_GATE_UP_32)
    torch.cuda.synchronize()
    for i in range(KERNEL_TIMING_LAUNCHES):
        w = sets[i % NUM_WEIGHT_SETS]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        native.mx_gemm_swiglu(codes, scales, w.w_gate_up, w.s_gate_up,
                              layout=native.LAYOUT_GATE_UP_32)
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    k_all = sorted(a.elapsed_time(b) for a, b in evs)
    k_ms = statistics.median(k_all)
    k_mean = statistics.mean(k_all)
    k_p10, k_p90 = k_all[len(k_all) // 10], k_all[(len(k_all) * 9) // 10]

    # ---- end to end through the public API with host buffers. Every step copies its input
    # from pinned host memory and its result back; the three legs run on their own streams
    # (double-buffered), so step i+1's upload and step i-1's download overlap step i's kernels,
    # as a serving engine would pipeline them. PCIe is full duplex. With N ranks each rank
    # uploads the token rows it owns and the ranks all-gather them over NVLink (the activations
    # of a tensor-parallel layer are replicated), and each rank downloads the rows of the
    # result it owns, so the bytes crossing PCIe per step do not grow with N.
    rows_lo, rows_hi = first, first + count
    host_in = [torch.randn(m, HIDDEN).to(torch.bfloat16).pin_memory() for _ in range(2)]
    host_out = [torch.empty((m, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dev_in = [torch.empty((m, HIDDEN), dtype=torch.bfloat16, device=device) for _ in range(2)]
    even_split = world > 1 and m % world == 0
    main = torch.cuda.current_stream()
    s_in, s_run, s_out = (torch.cuda.Stream(device) for _ in range(3))
    ev_in = [torch.cuda.Event() for _ in range(2)]       # upload of buffer b finished
    ev_free = [torch.cuda.Event() for _ in range(2)]     # kernels that read buffer b finished
    ev_done = [torch.cuda.Event() for _ in range(2)]     # result b computed
    ev_out = [torch.cuda.Event() for _ in range(2)]      # download into host buffer b finished
    keep = [None, None]

    # The device part of a step is captured once per (input buffer, weight set) in a CUDA graph
    # and replayed, as a serving engine does: at N >= 4 the kernels of a step take less time
    # than the Python and ctypes calls that launch them one by one.
    graphs = {}
    if not args.no_e2e_graphs:
        fine = True
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                for b in range(2):
                    for w in range(NUM_WEIGHT_SETS):
                        tp_step(dev_in[b], residual, residual_rows, gamma, sets[w], group, owner)
            main.wait_stream(side)
        except RuntimeError:
            fine = False
        barrier()
        if fine:
            try:
                for b in range(2):
                    for w in range(NUM_WEIGHT_SETS):
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph):
                            result = tp_step(dev_in[b], residual, residual_rows, gamma, sets[w],
                                             group, owner)
                        graphs[(b, w)] = (graph, result)
            except RuntimeError:
                graphs = {}
        barrier()
    flag = torch.tensor([1.0 if graphs else 0.0], device=device)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)   # every rank takes the same route
    if flag.item() == 0.0:
        graphs = {}

    def e2e_steps(count_steps):
        for st in (s_in, s_run, s_out):
            st.wait_stream(main)
        for i in range(count_steps):
            b = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_free[b])
                if even_split:
                    dev_in[b][rows_lo:rows_hi].copy_(host_in[b][rows_lo:rows_hi], non_blocking=True)
                else:
                    dev_in[b].copy_(host_in[b], non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[b])
                if even_split:
                    # On the compute stream, not beside it: the all-gather and the fused reduce
                    # both wait for their peers on the device, and two such kernels of one GPU
                    # in two streams can each hold the SMs the other one needs on another rank.
                    dist.all_gather_into_tensor(dev_in[b], dev_in[b][rows_lo:rows_hi], group=group)
                if graphs:
                    # the graph's output buffer is reused by its next replay: wait for the
                    # download that still reads it
                    if i >= 2:
                        s_run.wait_event(ev_out[b])
                    graph, result = graphs[(b, i % NUM_WEIGHT_SETS)]
                    graph.replay()
                else:
                    result = tp_step(dev_in[b], residual, residual_rows, gamma,
                                     sets[i % NUM_WEIGHT_SETS], group, owner)
                norm = result[0]
                ev_free[b].record(s_run)
                ev_done[b].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                if i >= 2:
                    s_out.wait_event(ev_out[b])
                if not graphs:
                    norm.record_stream(s_out)
                if owner:
                    host_out[b][rows_lo:rows_hi].copy_(norm, non_blocking=True)
                elif even_split:
                    host_out[b][rows_lo:rows_hi].copy_(norm[rows_lo:rows_hi], non_blocking=True)
                else:
                    host_out[b].copy_(norm, non_blocking=True)
                ev_out[b].record(s_out)
                keep[b] = result
        for st in (s_in, s_run, s_out):
            main.wait_stream(st)

    e2e_steps(args.warmup)
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    host_t0 = time.perf_counter()
    e2e_steps(args.steps)
    e2e_host_ms = (time.perf_counter() - host_t0) * 1e3   # time to enqueue the steps
    e2.record()
    barrier()
    e2e_ms = s2.elapsed_time(e2)
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([ms, e2e_ms, k_ms], dtype=torch.float64, device=device)
    ms_all = [ms_rank]
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        gathered = [torch.zeros(3, dtype=torch.float64, device=device) for _ in range(world)]
        dist.all_gather(gathered, torch.tensor([ms_rank, step_ms[worst_step], float(worst_step)],
                                               dtype=torch.float64, device=device))
        ms_all = [float(t[0].item()) for t in gathered]
        if rank == 0:
            print("timed steps by rank (ms total, longest step ms, its index): " +
                  ", ".join(f"{t[0].item():.3f}/{t[1].item():.3f}/{int(t[2].item())}"
                            for t in gathered), file=sys.stderr)
    ms, e2e_ms, k_ms = times.tolist()
    status = native.device_status()

    # ---- checker leg (N >= 2): the tensor-parallel block against the CPU oracle
    parity = None
    if world > 1 and not args.no_parity:
        parity = [tp_parity(group, world, rank, device, t) for t in (32, 512, HEADLINE_M)]

    # ---- the other tensor-parallel configurations (MXFP6 MLP, expert-parallel MoE)
    tp_suite = None
    if not args.no_tp_suite:
        tp_suite = run_tp_suite(group, world, rank, device, peaks)

    # ---- batch sweep under CUDA graphs (decode sizes are launch-bound otherwise), 1 GPU only
    sweep = None
    if world == 1 and not args.no_sweep:
        sweep = run_sweep(device, sets, gamma, peaks, args)

    library = None
    if world == 1 and rank == 0 and not args.no_library:
        library = fp8_library_peak(device)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu_baseline = run_cpu_baseline(steps=20, warmup=1)

    if rank == 0:
        flops = 2.0 * m * (2 * inter_local) * HIDDEN
        achieved = flops / (k_ms * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        traffic, traffic_source = ncu_traffic("gate_up_swiglu", m) if world == 1 else (None, None)
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_source,
                    "kernel": "mx_gemm_pair_kernel<SwiGLU> (gate_up + SwiGLU + MXFP8 "
                              "requant, cta_group::2, 256 x 192 tiles)",
                    "kernel_ms": k_ms,
                    "kernel_ms_stats": {"launches": KERNEL_TIMING_LAUNCHES, "median": k_ms,
                                        "mean": k_mean, "p10": k_p10, "p90": k_p90},
                    "frac_of_burst_peak": achieved / (2.0 * peaks["bf16_tflops"]),
                    "peak_note": f"2 x bf16_tflops_sustained ({peaks['source']}): FP8 issues "
                                 "at twice the BF16 rate; frac_of_burst_peak uses 2 x bf16_tflops"}
        if library is not None:
            roofline["fp8_library_tflops"] = library
            ref = library.get("mxfp8_gate_up_4096x19456x2560", {})
            if "sustained" in ref:
                roofline["vs_library_mxfp8_gate_up"] = achieved / ref["sustained"]
        outputs = ("MXFP8 codes + scales replicated (read in the communication buffer, where "
                   "the rows' owners store them); BF16 norm and residual stream row-owned "
                   "(1/N of the rows per rank)") if owner else \
                  "BF16 norm + residual (all rows)" if world > 1 else \
                  "BF16 norm + residual + MXFP8 codes + scales"
        line = {
            "metric": "mlp_layer_tokens_per_s", "value": m * args.steps / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (ue8m0 block scales, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": "MXFP8 dense decoder MLP block, hidden 2560, intermediate 9728",
                       "tokens": m, "parallelism": f"tp{world}", "soak_steps": soak_steps,
                       "reduce": "owner form" if owner else ("push form" if world > 1 else "none"),
                       "reduce_note": reduce_note,
                       "launch": (f"CUDA graph replay, {STEP_VARIANTS} consecutive steps per graph "
                                  "(single-step graphs for the remainder)"
                                  if step_chain is not None else
                                  "CUDA graph replay, one graph per step" if step_graphs
                                  else "kernels launched one by one"),
                       "step_outputs": outputs,
                       "l2": f"rotates {NUM_WEIGHT_SETS} weight sets "
                             f"({NUM_WEIGHT_SETS * sets[0].nbytes() * world / 1e6:.0f} MB > 126 MB L2)"},
            "e2e": {"value": m * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": m * HIDDEN * 2, "d2h_bytes_per_step": m * HIDDEN * 2,
                    "host_enqueue_ms_per_step": e2e_host_ms / args.steps,
                    "note": ("bytes over all ranks; each rank moves the rows it owns and the "
                             "ranks all-gather the input over NVLink" if world > 1 else
                             "upload, kernels and download on three streams, double-buffered")
                            + ("; device part of the step replayed from a CUDA graph" if graphs
                               else "; kernels launched one by one")},
            "gpu_launches": 4 * args.steps,
            "roofline": roofline,
            "clocks": clocks, "device_status": status,
            "device_status_after_timed_steps": status_timed,
            "ms_per_step_by_rank": [t / args.steps for t in ms_all],
        }
        if parity is not None:
            line["parity"] = parity
        if tp_suite is not None:
            line["tp_suite"] = tp_suite
        if sweep is not None:
            line["sweep"] = sweep
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line))
    if world > 1:
        graphs.clear()
        step_graphs.clear()
        step_chain = None
        torch.cuda.synchronize()
        collective.close_all()
        dist.destroy_process_group()


def run_tp_suite(group, world, rank, device, peaks):
    """The other configurations that shard over N GPUs, per batch: the MXFP6 (E2M3) MLP, hidden
    5120 / intermediate 17408, gate_up column- and down row-parallel with the fused reduce, and
    the 256-expert top-8 MoE (hidden 2048, intermediate 512, E2M3) with the experts split N
    ways and the same fused reduce over the combined output. CUDA-graph replays, CUDA events,
    max over ranks. Random 6-bit codes with oracle-like scales (timing only)."""
    import torch.distributed as dist
    from mach_b200 import collective, native
    from mach_b200 import moe as moe_mod
    from mach_b200.mlp import mlp_block, mlp_block_owner
    out = []
    g = torch.Generator(device=device).manual_seed(21)

    def timed(fn, variants, calls):
        try:
            us = graph_time_us(fn, variants, calls=calls, reps=5)
        except RuntimeError:
            # a launch that cannot be captured: time the same calls eagerly
            torch.cuda.synchronize()
            for i in range(3):
                fn(i)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for i in range(calls * 3):
                fn(i)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (calls * 3)
        t = torch.tensor([us], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    # ---- MXFP6 dense MLP, tensor parallel
    hid, inter = 5120, 17408
    _, inter_local = shard_blocks(inter, world, rank)
    n_sets = 2 if world == 1 else max(2, min(8, (2 * world)))   # > L2 in total on every rank
    sets = [make_weights(device, world, rank, 3000 + i, hid, inter, "e2m3", 0.015)
            for i in range(n_sets)]
    gamma = (0.1 * torch.randn(hid, generator=g, device=device)).to(torch.bfloat16)
    for m in (1, 32, 512, 4096):
        x = torch.randn(m, hid, generator=g, device=device).to(torch.bfloat16)
        residual = torch.randn(m, hid, generator=g, device=device).to(torch.bfloat16)
        owner = world > 1 and m * hid * 2 > owner_min_bytes(world)
        first, count = collective.owner_rows(m, group)
        rows = residual[first:first + count].contiguous()
        if owner:
            fn = lambda i: mlp_block_owner(x, rows, gamma, EPS, sets[i % n_sets], group,  # noqa: E731
                                           codes_in_workspace=True)
        else:
            fn = lambda i: mlp_block(x, residual, gamma, EPS, sets[i % n_sets], group)  # noqa: E731
        us = timed(fn, n_sets, 10)
        flops = 2.0 * m * 3 * hid * inter              # whole job, all ranks
        nbytes = mlp_bytes(m, inter_local, hid, 0.75)   # per rank
        out.append({"config": "mxfp6_e2m3_mlp_h5120_i17408", "tp": world, "tokens": m,
                    "reduce": "owner" if owner else ("push" if world > 1 else "none"),
                    "us": round(us, 2), "tokens_per_s": m / (us * 1e-6),
                    "tflops_per_gpu": round(flops / world / (us * 1e-6) / 1e12, 1),
                    "hbm_gbs_per_gpu": round(nbytes / (us * 1e-6) / 1e9, 1),
                    "frac_hbm_measured": round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 3),
                    "frac_fp8_measured": round(flops / world / (us * 1e-6) / 1e12
                                               / (2 * peaks["bf16_tflops_sustained"]), 3)})
    del sets
    torch.cuda.empty_cache()

    # ---- MoE, expert parallel
    e, hid, inter, top_k = 256, 2048, 512, 8
    per = e // world
    w13 = torch.randint(0, 256, (per, 2 * inter, hid * 3 // 4), dtype=torch.uint8, device=device,
                        generator=g)
    s13 = torch.randint(116, 120, (per, 2 * inter, hid // 32), dtype=torch.uint8, device=device,
                        generator=g)
    w2 = torch.randint(0, 256, (per, hid, inter * 3 // 4), dtype=torch.uint8, device=device,
                       generator=g)
    s2 = torch.randint(116, 120, (per, hid, inter // 32), dtype=torch.uint8, device=device,
                       generator=g)
    weights = moe_mod.MoeWeights.from_logical(w13, s13, w2, s2, fmt="e2m3")
    del w13, s13, w2, s2
    expert_map = None
    if world > 1:
        expert_map = torch.full((e,), -1, dtype=torch.int32, device=device)
        expert_map[rank * per:(rank + 1) * per] = torch.arange(per, dtype=torch.int32, device=device)
    gamma = (0.1 * torch.randn(hid, generator=g, device=device)).to(torch.bfloat16)
    per_expert = 3 * hid * inter * (0.75 + 1 / 32)
    for m in (1, 64, 1024, 4096):
        gen = torch.Generator(device=device).manual_seed(77 + m)   # same tokens on every rank
        x = torch.randn(m, hid, generator=gen, device=device).to(torch.bfloat16)
        logits = torch.randn(m, e, generator=gen, device=device).to(torch.bfloat16)
        residual = torch.randn(m, hid, generator=gen, device=device).to(torch.bfloat16)
        _, ids = moe_mod.router_topk(logits, top_k)
        local_ids = ids[(ids // per) == rank] if world > 1 else ids
        distinct = int(torch.unique(local_ids).numel())
        owner = world > 1 and m * hid * 2 > owner_min_bytes(world)
        first, count = collective.owner_rows(m, group)
        rows = residual[first:first + count].contiguous()

        def fn(i):
            tw, ti = moe_mod.router_topk(logits, top_k)
            partial = moe_mod.experts_forward(x, weights, tw, ti, expert_map)
            if world == 1:
                return native.add_rmsnorm_mxfp8(partial, residual, gamma, EPS)
            if owner:
                return collective.allreduce_owner_add_rmsnorm(partial, rows, gamma, EPS, group, m)
            return collective.allreduce_add_rmsnorm(partial, residual, gamma, EPS, group,
                                                    want_quant=True)
        us = timed(fn, 1, 10)
        nbytes = distinct * per_expert + m * hid * 4
        flops = 2.0 * m * top_k * 3 * hid * inter
        out.append({"config": "moe_e256_top8_h2048_i512_e2m3", "ep": world, "tokens": m,
                    "reduce": "owner" if owner else ("push" if world > 1 else "none"),
                    "distinct_local_experts": distinct, "us": round(us, 2),
                    "tokens_per_s": m / (us * 1e-6),
                    "tflops_per_gpu": round(flops / world / (us * 1e-6) / 1e12, 1),
                    "hbm_gbs_per_gpu": round(nbytes / (us * 1e-6) / 1e9, 1),
                    "frac_hbm_measured": round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 3)})
    return out


def run_ar_local(args, device):
    """The owner-form reduce with all ranks of a 4-way group on ONE device (a single cooperative
    grid, "peer" pointers local): the kernel a profiler can capture without a multi-rank run."""
    import ctypes
    from mach_b200 import native
    lib, world, h, m = native.lib(), 4, HIDDEN, args.tokens
    nbytes = lib.mach_ar_buffer_bytes(world, m, h)
    buffers = []
    for _ in range(world):
        ptr = ctypes.c_void_p()
        native._check(lib.mach_ar_buffer_alloc(nbytes, ctypes.byref(ptr)), "ar_buffer_alloc")
        buffers.append(ptr.value)
    arr = (ctypes.c_void_p * world)(*buffers)
    handles = []
    for r in range(world):
        ws = ctypes.c_void_p()
        native._check(lib.mach_ar_create(world, r, m, h, arr, ctypes.byref(ws)), "ar_create")
        handles.append(ws.value)
    g = torch.Generator(device=device).manual_seed(3)
    rpo = (m + world - 1) // world
    partials = [torch.randn(m, h, generator=g, device=device).to(torch.bfloat16) for _ in range(world)]
    residual = torch.randn(m, h, generator=g, device=device).to(torch.bfloat16)
    gamma = (0.1 * torch.randn(h, generator=g, device=device)).to(torch.bfloat16)
    rows = [residual[r * rpo:min(m, (r + 1) * rpo)].contiguous() for r in range(world)]
    norms = [torch.empty_like(t) for t in rows]
    ress = [torch.empty_like(t) for t in rows]
    codes = [torch.empty((m, h), dtype=torch.uint8, device=device) for _ in range(world)]
    scales = [torch.empty(native.sf_bytes(m, h), dtype=torch.uint8, device=device) for _ in range(world)]

    def ptrs(ts):
        return (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def launch():
        native._check(lib.mach_allreduce_local_ranks(
            world, (ctypes.c_void_p * world)(*handles), ptrs(partials), ptrs(rows), gamma.data_ptr(),
            EPS, 1.0, ptrs(norms), ptrs(ress), ptrs(codes), ptrs(scales), m, h, 0, 1, stream),
            "allreduce_local_ranks")
    for _ in range(args.warmup):
        launch()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        launch()
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"kernel_only": "ar_owner_local", "ranks_on_one_device": world, "tokens": m,
                      "hidden": h, "us_per_launch": e0.elapsed_time(e1) * 1e3 / args.steps,
                      "device_status": native.device_status()}))
    for hnd in handles:
        lib.mach_ar_destroy(hnd)
    for b in buffers:
        lib.mach_ar_buffer_free(b)


def run_kernel_only(args, xs, sets, device):
    """One kernel of the step alone (for profiler captures and tile sweeps): `warmup` + `steps`
    launches cycling the weight sets, CUDA-event time of the `steps` launches on one JSON line."""
    from mach_b200 import native
    if args.kernel_only == "ar_owner_local":
        run_ar_local(args, device)
        return
    m = args.tokens
    codes, scales = native.quantize_mxfp8(xs[0])
    inter_local = sets[0].w_down.shape[1]
    h = torch.randn(m, inter_local, device=device).to(torch.bfloat16)
    h_codes, h_scales = native.quantize_mxfp8(h)

    def launch(i):
        w = sets[i % NUM_WEIGHT_SETS]
        if args.kernel_only == "gate_up_swiglu":
            return native.mx_gemm_swiglu(codes, scales, w.w_gate_up, w.s_gate_up,
                                         layout=native.LAYOUT_GATE_UP_32)
        if args.kernel_only == "down":
            return native.mx_gemm(h_codes, h_scales, w.w_down, w.s_down)
        return native.quantize_mxfp8(xs[i % 4])

    for i in range(args.warmup):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        launch(i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    flops = {"gate_up_swiglu": 2.0 * m * 2 * inter_local * HIDDEN,
             "down": 2.0 * m * HIDDEN * inter_local, "quantize": 0.0}[args.kernel_only]
    print(json.dumps({"kernel_only": args.kernel_only, "tokens": m, "us_per_launch": us,
                      "tflops": flops / (us * 1e-6) / 1e12, "steps": args.steps,
                      "device_status": native.device_status()}))


def run_sweep(device, sets, gamma, peaks, args):
    """Per-batch MLP time under CUDA-graph replay: 8 passes per graph cycling the weight sets."""
    from mach_b200.mlp import mlp_block
    out = []
    g = torch.Generator(device=device).manual_seed(11)
    for m in SWEEP_M:
        x = torch.randn(m, HIDDEN, generator=g, device=device).to(torch.bfloat16)
        res = torch.randn(m, HIDDEN, generator=g, device=device).to(torch.bfloat16)
        passes = 8
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(3):
                mlp_block(x, res, gamma, EPS, sets[i % NUM_WEIGHT_SETS], None)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(passes):
                mlp_block(x, res, gamma, EPS, sets[i % NUM_WEIGHT_SETS], None)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        reps = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * passes)
        tf = gemm_flops(m, INTER) / (us * 1e-6) / 1e12
        gbs = mlp_bytes(m, INTER) / (us * 1e-6) / 1e9
        out.append({"tokens": m, "us_per_mlp": round(us, 2), "tokens_per_s": m / (us * 1e-6),
                    "gemm_tflops": round(tf, 1), "hbm_gbs": round(gbs, 1),
                    "frac_hbm_measured": round(gbs / peaks["hbm_gbs"], 3),
                    "frac_fp8_measured": round(tf / (2 * peaks["bf16_tflops_sustained"]), 3)})
    return out



# ------------------------------------------------------------------ per-config suite
def graph_time_us(fn, variants: int, calls: int = 20, reps: int = 10):
    """CUDA-event time per call of `fn(i)` replayed from a CUDA graph of `calls` back-to-back
    invocations cycling `variants` operand sets (weights larger than L2 in total)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(max(3, variants)):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(calls):
            fn(i)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * calls)


def run_suite(args):
    """Every benchmark configuration that fits one GPU, one JSON line per case: microseconds per
    call (CUDA graph of 20 calls cycling weight copies), algorithmic GB/s and TFLOP/s and their
    fractions of the measured peaks. Synthetic operands: random codes with plausible scales
    (timing only; parity is the test suite's job)."""
    from mach_b200 import native
    from mach_b200.mlp import MxMlpWeights, mlp_forward
    from mach_b200 import moe as moe_mod
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    native.lib()
    peaks = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(5)
    only = set(args.suite.split(",")) if args.suite != "all" else None

    def emit(config, case, m, us, nbytes, flops, tensor_peak_scale=2.0):
        gbs = nbytes / (us * 1e-6) / 1e9
        tf = flops / (us * 1e-6) / 1e12
        print(json.dumps({"suite": config, "case": case, "tokens": m, "us": round(us, 2),
                          "gbs": round(gbs, 1), "tflops": round(tf, 1),
                          "frac_hbm_measured": round(gbs / peaks["hbm_gbs"], 3),
                          "frac_tensor_measured": round(
                              tf / (tensor_peak_scale * peaks["bf16_tflops_sustained"]), 3),
                          "device_status": native.device_status()}), flush=True)

    def rand_codes(rows, cols):
        return torch.randint(0, 256, (rows, cols), dtype=torch.uint8, device=dev, generator=g)

    def fp8_weight(n, k, sigma=0.02):
        w = (torch.randn(n, k, generator=g, device=dev) * sigma).to(torch.bfloat16)
        codes, sw = native.quantize_mxfp8(w)
        return codes, sw

    def want(name):
        return only is None or name in only

    # ---- C1: one MXFP8 linear, M 16, K 2048, N 6144 (quantise + GEMM)
    if want("c1"):
        m, k, n = 16, 2048, 6144
        ws = [fp8_weight(n, k) for _ in range(12)]       # 12 x 12.6 MB > L2
        x = torch.randn(m, k, generator=g, device=dev).to(torch.bfloat16)

        def c1(i):
            c, s = native.quantize_mxfp8(x)
            return native.mx_gemm(c, s, ws[i % 12][0], ws[i % 12][1])
        us = graph_time_us(c1, 12)
        emit("c1", "mxfp8 linear 16x6144x2048 (quantise + GEMM)", m, us,
             n * k * (1 + 1 / 32) + m * k * 2 + m * n * 2, 2.0 * m * n * k)

    # ---- C2: the two GEMMs of the dense MLP alone, per batch
    if want("c2"):
        sets = [make_weights(dev, 1, 0, 1000 + i) for i in range(NUM_WEIGHT_SETS)]
        for m in SWEEP_M:
            x = torch.randn(m, HIDDEN, generator=g, device=dev).to(torch.bfloat16)
            xc, xs = native.quantize_mxfp8(x)
            h = torch.randn(m, INTER, generator=g, device=dev).to(torch.bfloat16)
            hc, hs = native.quantize_mxfp8(h)
            us = graph_time_us(lambda i: native.mx_gemm_swiglu(
                xc, xs, sets[i % 4].w_gate_up, sets[i % 4].s_gate_up,
                layout=native.LAYOUT_GATE_UP_32), 4)
            emit("c2", "gate_up + SwiGLU + requant", m, us,
                 2 * INTER * HIDDEN * (1 + 1 / 32) + m * HIDDEN * (1 + 1 / 32)
                 + m * INTER * (1 + 1 / 32), 2.0 * m * 2 * INTER * HIDDEN)
            us = graph_time_us(lambda i: native.mx_gemm(hc, hs, sets[i % 4].w_down,
                                                        sets[i % 4].s_down), 4)
            emit("c2", "down", m, us, HIDDEN * INTER * (1 + 1 / 32) + m * INTER * (1 + 1 / 32)
                 + m * HIDDEN * 2, 2.0 * m * HIDDEN * INTER)
        del sets

    # ---- C3: block-FP8 linear (group quantise + GEMM), both orientations
    if want("c3"):
        for (k, n) in ((2560, 9728), (9728, 2560)):
            bs = []
            for _ in range(6):                              # 6 x 24.9 MB > L2
                b = rand_codes(n, k) & 0x77                  # finite E4M3 codes
                sb = torch.rand((n + 127) // 128, k // 128, generator=g, device=dev) * 1e-3 + 1e-4
                bs.append((b.view(torch.float8_e4m3fn), sb))
            for m in (1, 32, 512, 8192):
                x = torch.randn(m, k, generator=g, device=dev).to(torch.bfloat16)

                def c3(i):
                    q, sa = native.fp8_group_quantize(x)
                    return native.block_fp8_gemm(q, sa, bs[i % 6][0], bs[i % 6][1])
                us = graph_time_us(c3, 6)
                emit("c3", f"block-FP8 linear K{k} N{n} (quantise + GEMM)", m, us,
                     n * k + (n // 128) * (k // 128) * 4 + m * k * 2 + m * n * 2, 2.0 * m * n * k)

    # ---- C4: MXFP6 (E2M3) dense MLP, hidden 5120, intermediate 17408, one GPU
    if want("c4"):
        hid, inter = 5120, 17408
        sets = []
        for _ in range(2):                                   # 2 x 209 MB > L2
            w_gu = rand_codes(2 * inter, hid * 3 // 4)
            s_gu = torch.full((2 * inter, hid // 32), 118, dtype=torch.uint8, device=dev)
            w_d = rand_codes(hid, inter * 3 // 4)
            s_d = torch.full((hid, inter // 32), 118, dtype=torch.uint8, device=dev)
            sets.append(MxMlpWeights.from_logical(w_gu, s_gu, w_d, s_d, hid, fmt="e2m3"))
        for m in (1, 32, 512, 4096):
            x = torch.randn(m, hid, generator=g, device=dev).to(torch.bfloat16)
            us = graph_time_us(lambda i: mlp_forward(x, sets[i % 2]), 2, calls=10)
            wbytes = 3 * hid * inter * (0.75 + 1 / 32)
            emit("c4", "MXFP6 E2M3 MLP (quantise, gate_up+SwiGLU, down)", m, us,
                 wbytes + m * hid * 2 + 2 * m * inter * (1 + 1 / 32) + m * hid * 2,
                 2.0 * m * 3 * hid * inter)
        del sets

    # ---- C5: MoE, 256 experts, top-8, hidden 2048, intermediate 512, MXFP6 E2M3 weights
    if want("c5"):
        e, hid, inter, top_k = 256, 2048, 512, 8
        w13 = rand_codes(e * 2 * inter, hid * 3 // 4).view(e, 2 * inter, -1)
        s13 = torch.full((e, 2 * inter, hid // 32), 118, dtype=torch.uint8, device=dev)
        w2 = rand_codes(e * hid, inter * 3 // 4).view(e, hid, -1)
        s2 = torch.full((e, hid, inter // 32), 118, dtype=torch.uint8, device=dev)
        weights = moe_mod.MoeWeights.from_logical(w13, s13, w2, s2, fmt="e2m3")
        del w13, s13, w2, s2
        per_expert = 3 * hid * inter * (0.75 + 1 / 32)
        for m in (1, 64, 1024, 4096):
            x = torch.randn(m, hid, generator=g, device=dev).to(torch.bfloat16)
            logits = torch.randn(m, e, generator=g, device=dev).to(torch.bfloat16)
            tw, ids = moe_mod.router_topk(logits, top_k)
            distinct = int(torch.unique(ids).numel())

            def c5(i):
                tw_i, ids_i = moe_mod.router_topk(logits, top_k)
                return moe_mod.experts_forward(x, weights, tw_i, ids_i)
            us = graph_time_us(c5, 1, calls=10)
            emit("c5", f"MoE router + experts ({distinct} distinct experts)", m, us,
                 distinct * per_expert + m * hid * 4, 2.0 * m * top_k * 3 * hid * inter)


# ------------------------------------------------------------------ CPU arm
def run_cpu_baseline(steps: int, warmup: int, tokens: int = CPU_SAMPLE_TOKENS):
    """The reference's CPU-expressible path on the host cores (torch CPU, all threads):
    quantise -> dequantise -> FP32 matmul -> BF16 for gate_up and down, SwiGLU requant and
    residual + RMSNorm between/after. Weights are dequantised once (they are static)."""
    from oracle import mx_oracle as ora
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(3)
    w_gu = (torch.randn(2 * INTER, HIDDEN, generator=g) * 0.02).to(torch.bfloat16)
    w_d = (torch.randn(HIDDEN, INTER, generator=g) * 0.02).to(torch.bfloat16)
    wgu = ora.dequantize_mx(*ora.quantize_weight_mxfp8(w_gu))
    wd = ora.dequantize_mx(*ora.quantize_weight_mxfp8(w_d))
    x = torch.randn(tokens, HIDDEN, generator=g).to(torch.bfloat16)
    res = torch.randn(tokens, HIDDEN, generator=g).to(torch.bfloat16)
    gamma = (0.1 * torch.randn(HIDDEN, generator=g)).to(torch.bfloat16)

    def step():
        a_c, a_s = ora.quantize_mxfp8(x)
        gate_up = ora.mx_gemm(a_c, a_s, wgu)
        h_c, h_s = ora.swiglu_quantize(gate_up)
        y = ora.mx_gemm(h_c, h_s, wd)
        return ora.gemma_rmsnorm(y, res, gamma, EPS)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return {"value": tokens * steps / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{tokens} tokens per step x {steps} steps of the same MLP block "
                      f"({dt / steps:.2f} s/step), weights dequantised once outside the timing",
            "ms_per_step": dt / steps * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = run_cpu_baseline(steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": "mlp_layer_tokens_per_s", "value": base["value"],
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3 (ue8m0 block scales, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": "MXFP8 dense decoder MLP block, hidden 2560, intermediate 9728",
                   "tokens": CPU_SAMPLE_TOKENS, "parallelism": "cpu"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--tokens", type=int, default=HEADLINE_M)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check at N >= 2")
    ap.add_argument("--no-tp-suite", action="store_true",
                    help="skip the MXFP6 MLP / MoE tensor-parallel timings")
    ap.add_argument("--no-library", action="store_true", help="skip the cuBLASLt FP8 peak")
    ap.add_argument("--no-step-graphs", action="store_true",
                    help="launch the kernels of the timed steps one by one instead of replaying graphs")
    ap.add_argument("--no-e2e-graphs", action="store_true",
                    help="end-to-end leg: launch the kernels one by one instead of replaying graphs")
    ap.add_argument("--no-owner", action="store_true",
                    help="N >= 2: push-form reduce with all rows on every rank")
    ap.add_argument("--suite", default=None,
                    help="'all' or a comma list of c1,c2,c3,c4,c5: per-config timings, one JSON "
                         "line per case, instead of the headline step")
    ap.add_argument("--soak", type=float, default=SOAK_SECONDS,
                    help="seconds of untimed steps before the timed region (clock samples)")
    ap.add_argument("--kernel-only", choices=["gate_up_swiglu", "down", "quantize", "ar_owner_local"],
                    default=None,
                    help="run one kernel of the step alone (profiler captures)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.suite:
        run_suite(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()

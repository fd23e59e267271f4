#!/usr/bin/env python
"""Benchmark of the W8A8 expert-parallel MoE layer: int8 MoE-layer tokens/s on 1/2/4/8 B200.

    python bench.py --gpus 1 --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W     # the CPU formulas of the path on the host cores
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass of the layer (dispatch with per-token int8 quantisation -> gate_up grouped GEMM with the
dequant+SwiGLU+requant epilogue -> down grouped GEMM -> combine) over one batch of seeded synthetic tokens.
N = 1 runs the decode shape with all 256 experts local (256 tokens, hidden 7168, top-8, intermediate 2048);
N > 1 runs the expert-parallel decode shape (128 tokens per rank, 256/N experts per rank).
Prints ONE JSON line on rank 0.

A timed block is exactly --steps steps between two barrier + synchronize pairs, timed with CUDA events, maximum over
ranks; blocks are repeated until about a second has been measured and the median block is reported (`repeats`), so
that the clock sampler sees the GPU under load.  At N = 1 the line also carries, under roofline.others, the kernels
that the decode shape cannot show at a meaningful size: both grouped GEMMs on two tensor-bound shapes and the row
kernels at 65536 x 7168, each timed inside a CUDA graph in the same process.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "int8_moe_layer_tokens_per_s"
UNIT = "tokens/s"
SCALING = "strong"
SCALING_NOTE = ("the bytes that bound a step -- this rank's int8 expert weights -- are sharded, 1/N per rank (strong); tokens "
                "per rank are fixed, so the token count grows with N; N=1 runs the all-experts-local shape (256 tokens). "
                "stream_frac = per-rank weight bytes / step time / HBM peak is comparable across N")

# single-GPU study cases: name -> (description, T, H, E, K, I, zipf exponent)
EXTRA_WORKLOADS = {
    "cfg1_small": ("cfg1_small: decode shape at 1/8 scale (32 tokens, 32 experts; 1.4 GB of weights)", 32, 7168, 32, 8, 2048, 0.0),
    "cfg2_rank": ("cfg2_rank: one rank's expert work of the 8-GPU decode (1024 rows over 32 local experts)", 128, 7168, 32, 8, 2048, 0.0),
    "cfg3_rank": ("cfg3_rank: one rank's share of the skewed 8-GPU prefill (65536 rows over 32 local experts, Zipf 1.2)",
                  8192, 7168, 32, 8, 2048, 1.2),
    "prefill_small": ("prefill_small: 2048 tokens top-8 over 8 experts of the DeepSeek-V3 expert shape (16384 rows, 2048 per expert)",
                      2048, 7168, 8, 8, 2048, 0.0),
    "cfg4": ("cfg4: Qwen3-235B-A22B shape, 4096 tokens, 128 experts local", 4096, 4096, 128, 8, 1536, 0.0),
}

# expert-parallel prefill cases (tokens per rank, total experts): usable at N > 1
EP_WORKLOADS = {
    "cfg3": ("cfg3: expert-parallel prefill with Zipf(1.2) routing skew, DeepSeek-V3 shape, 8192 tokens/rank", 8192, 7168, 256, 8, 2048, 1.2),
    "cfg4": ("cfg4: Qwen3-235B-A22B shape, 4096 tokens/rank", 4096, 4096, 128, 8, 1536, 0.0),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (N=1)")
    ap.add_argument("--no-others", action="store_true",
                    help="N=1: skip the tensor-bound GEMM shapes and the row kernels under roofline.others")
    ap.add_argument("--ep-transport", default="peer", choices=["peer", "nccl"],
                    help="N > 1: rows move by this library's peer-memory kernels (default) or by NCCL all-to-all")
    ap.add_argument("--kernels", action="store_true",
                    help="also write the per-kernel table of this workload to stderr (study aid, N=1)")
    ap.add_argument("--workload", default="auto", choices=["auto", "cfg3"] + sorted(EXTRA_WORKLOADS),
                    help="auto = the headline configuration for this GPU count; the others are single-GPU study cases")
    return ap.parse_args()


def workload(n_gpus, name="auto"):
    """(name, T per rank, H, E total, K, I, zipf) of the configuration benchmarked at this GPU count."""
    if name in EP_WORKLOADS and (n_gpus > 1 or name not in EXTRA_WORKLOADS):
        desc, T, H, E, K, I, z = EP_WORKLOADS[name]
        return f"{desc}, {n_gpus}xB200, {E // n_gpus} experts/rank", T, H, E, K, I, z
    if name != "auto":
        if n_gpus != 1:
            raise RuntimeError("this study workload runs on one GPU")
        return EXTRA_WORKLOADS[name]
    if n_gpus == 1:
        return "cfg1: 1xB200 decode MoE layer, DeepSeek-V3 shape, 256 tokens, all 256 experts local", 256, 7168, 256, 8, 2048, 0.0
    return (f"cfg2: {n_gpus}xB200 expert-parallel decode, DeepSeek-V3 shape, 128 tokens/rank, {256 // n_gpus} experts/rank",
            128, 7168, 256, 8, 2048, 0.0)


def synthetic_tokens(torch, T, H, E, K, zipf, seed, rank=0):
    """Seeded synthetic inputs of the benchmark's shapes and distributions: tokens bf16 ~ N(0, 1); router logits fp32 ~ N(0, 1),
    plus a Zipf(zipf) bias over a permutation of the experts when zipf > 0; the K most probable experts of a token (ties to
    the lower id) and their probabilities renormalised to sum 1.  Returns (x [T, H], expert ids int32 [T, K], weights fp32)."""
    g = torch.Generator().manual_seed(seed * 1000 + rank)
    x = torch.randn(T, H, generator=g, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, dtype=torch.float32)
    if zipf > 0:
        perm = torch.randperm(E, generator=torch.Generator().manual_seed(seed))
        p = (torch.arange(E, dtype=torch.float64) + 1.0) ** (-zipf)
        logits = logits + torch.log(p / p.sum())[perm].float()
    order = torch.sort(torch.softmax(logits, dim=-1), dim=-1, descending=True, stable=True)
    w = order.values[:, :K]
    return x, order.indices[:, :K].to(torch.int32).contiguous(), (w / w.sum(dim=-1, keepdim=True)).contiguous()


def config_dict(name, T, H, E, K, I, world):
    return {"workload": name, "tokens_per_rank": T, "hidden": H, "experts": E, "experts_per_rank": E // world, "top_k": K,
            "intermediate": I, "parallelism": f"ep{world}"}


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle's formulas on the host cores
# ---------------------------------------------------------------------------------------------------
def _host_weights(cfg, seed):
    """Weights for the CPU arm.  Eight experts are drawn from the seeded generator; the others are rolled copies of
    them (same value distribution; drawing 11 GB from a serial generator would take a minute and times nothing)."""
    import torch
    from oracle import moe_oracle as O
    base = O.make_weights(cfg, seed, experts=range(min(8, cfg.E)))
    if cfg.E <= 8:
        return base
    w1 = torch.empty((cfg.E, cfg.H, 2 * cfg.I), dtype=torch.int8)
    w2 = torch.empty((cfg.E, cfg.I, cfg.H), dtype=torch.int8)
    s1 = torch.empty((cfg.E, 2 * cfg.I))
    s2 = torch.empty((cfg.E, cfg.H))
    for e in range(cfg.E):
        b, sh = e % 8, e // 8
        w1[e] = torch.roll(base.w1[b], sh, 0)
        w2[e] = torch.roll(base.w2[b], sh, 0)
        s1[e] = torch.roll(base.s1[b], sh, 0)
        s2[e] = torch.roll(base.s2[b], sh, 0)
    return O.MoeWeights(w1, s1, w2, s2)


def _host_ram_available():
    try:
        import psutil
        return int(psutil.virtual_memory().available)
    except Exception:
        return 0


def run_cpu(steps, warmup, seed, n_gpus=1, budget_s=150.0):
    """Times the oracle on the full configuration of this GPU count (all ranks simulated in one process) when the host
    holds its weights and the run fits the time budget; else on a sample with the same rows per expert."""
    import torch
    from oracle import moe_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    saved = O.SILU_IMPL
    O.SILU_IMPL = "libm"                 # the literal eager-torch formula (F.silu); parity tests use the deterministic restatement
    try:
        return _run_cpu(torch, O, steps, warmup, seed, n_gpus, budget_s)
    finally:
        O.SILU_IMPL = saved


def _run_cpu(torch, O, steps, warmup, seed, n_gpus, budget_s):
    name, T, H, E, K, I, zipf = workload(n_gpus)
    full = O.MoeConfig("full", T, H, E, K, I, zipf_s=zipf)
    weight_bytes = E * 3 * H * I
    ranks = n_gpus
    what = f"the full configuration ({T * ranks} tokens over {E} experts, {weight_bytes / 1e9:.2f} GB of int8 weights on the host)"
    cfg = full
    if _host_ram_available() < 2.3 * weight_bytes:
        cfg = None
    if cfg is not None:
        w = _host_weights(cfg, seed)
        toks = [O.make_tokens(cfg, seed, r) for r in range(ranks)]
        xs, ids, wts = zip(*toks)
        t0 = time.perf_counter()
        O.moe_layer(xs, ids, wts, w)
        first = time.perf_counter() - t0
        if first * (steps + warmup) > budget_s:
            cfg = None
            del w
    if cfg is None:
        e_s = 32
        t_s = max(8, T * ranks * e_s // E)
        cfg = O.MoeConfig("sample", t_s, H, e_s, K, I)
        ranks = 1
        what = (f"a sample: {t_s} tokens over {e_s} of the {E} experts (the same rows per expert), because the full configuration "
                "does not fit the host's memory or the time budget")
        w = _host_weights(cfg, seed)
        xs, ids, wts = zip(*[O.make_tokens(cfg, seed, 0)])
    for _ in range(warmup):
        O.moe_layer(xs, ids, wts, w)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.moe_layer(xs, ids, wts, w)
    dt = time.perf_counter() - t0
    tokens = cfg.T * ranks
    return {"value": tokens * steps / dt, "ms_per_step": dt / steps * 1e3, "cores": torch.get_num_threads(),
            "full_config": cfg is full,
            "sample": f"{what}; {steps} passes after {warmup} warm-up; eager torch on CPU (int8 matmul, F.silu)",
            "cpu_model": _cpu_model(), "torch": torch.__version__}


def _cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = run_cpu(args.steps, args.warmup, args.seed, args.gpus)
    name, T, H, E, K, I, _ = workload(args.gpus)
    cfg = config_dict(name, T, H, E, K, I, args.gpus)
    cfg["sample"] = r["sample"]
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": SCALING,
            "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"],
                             "full_config": r["full_config"], "cpu_model": r["cpu_model"], "torch": r["torch"]},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "the reference's arithmetic for this path is closed vendor code; this arm times its op formulas "
                    "(eager torch on CPU) on the host cores"}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# clock sampling during the measured sections
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.samples = []
        self.proc = None
        self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                try:
                    self.samples.append((time.time(), float(parts[0]), float(parts[1]), parts[2], parts[3:7]))
                except ValueError:
                    pass

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in windows)]
        used = inside if len(inside) >= 3 else self.samples
        if not used:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in used for n, v in zip(names, s[4]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(s[1] for s in used), "sm_max_mhz": max(s[2] for s in used), "reasons": reasons,
                "samples": len(used), "window": "timed regions" if used is inside else "whole run (timed regions too short to sample)"}


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
class Timer:
    """Device timing with CUDA events on the current stream."""

    def __init__(self, torch, windows):
        self.torch = torch
        self.windows = windows

    def each(self, fn, reps):
        torch = self.torch
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        t_a = time.time()
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
        self.windows.append((t_a, time.time()))
        return statistics.median(times)

    def launches(self, fn, reps, inner=5):
        """Device time of one call of fn: `inner` calls are captured into one CUDA graph and the replays are timed with
        events, so that the host's per-call work (allocation, ctypes, launch latency) is not counted as kernel time."""
        torch = self.torch
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g_ = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_):
            for _ in range(inner):
                fn()
        g_.replay()
        torch.cuda.synchronize()
        times = []
        t_a = time.time()
        for _ in range(max(5, reps // inner)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g_.replay()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b) / inner)
        self.windows.append((t_a, time.time()))
        del g_
        return statistics.median(times)


def gemm_pair(torch, timer, dev, spec, seed, reps, peak_tops, peak_gbs, row_kernels):
    """Both grouped GEMMs of the layer (gate_up with its fused epilogue, down) on one single-GPU shape, each timed inside
    a CUDA graph; optionally the row kernels of the path on the same rows."""
    import torchair_b200
    npu = torch.ops.npu
    desc, T, H, E, K, I, zipf = spec
    g = torch.Generator(device=dev).manual_seed(seed * 100003 + 17)
    w1 = torch.randint(-127, 128, (E, H, 2 * I), generator=g, dtype=torch.int8, device=dev)
    w2 = torch.randint(-127, 128, (E, I, H), generator=g, dtype=torch.int8, device=dev)
    s1 = torch.rand(E, 2 * I, generator=g, device=dev) * 9e-3 + 1e-3
    s2 = torch.rand(E, H, generator=g, device=dev) * 9e-3 + 1e-3
    x, ids, wt = (t.to(dev) for t in synthetic_tokens(torch, T, H, E, K, zipf, seed))
    ex, xs, expand_idx, nums, ep_recv, _, _ = npu.npu_moe_distribute_dispatch(x, ids, "", 1, 0, E, quant_mode=2)
    M = ex.shape[0]
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1)
    hit = int((nums > 0).sum().item())
    ops_up, ops_down = 2.0 * M * H * 2 * I, 2.0 * M * I * H
    bytes_up = hit * H * 2 * I + M * H + 2 * M * I * 4 + M * I + hit * 2 * I * 4 + M * 8      # weights, rows, fp32 h out and back, int8 out
    bytes_down = hit * I * H + M * I + M * H * 2 + hit * H * 4 + M * 4
    ms_up = timer.launches(lambda: npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1), reps)
    down = lambda: npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2,
                                          group_type=0, group_list_type=1, output_dtype=15)
    ms_down = timer.launches(down, reps)

    def tensor_entry(ms, ops, nbytes):
        # "frac" is of the tensor peak; which roof is the nearer one for this launch (its bytes at the measured copy bandwidth
        # against its operations at the tensor peak) is said beside it, with the fraction of that roof
        tops = ops / (ms * 1e-3) / 1e12
        gbs = nbytes / (ms * 1e-3) / 1e9
        t_hbm, t_tc = nbytes / (peak_gbs * 1e9), ops / (peak_tops * 1e12)
        return {"ms": ms, "int8_tops": tops, "frac": tops / peak_tops, "frac_of_nominal_4500": tops / 4500.0,
                "GB/s": gbs, "frac_of_hbm": gbs / peak_gbs, "nearer_roof": "hbm" if t_hbm >= t_tc else "tensor",
                "frac_of_nearer_roof": max(t_hbm, t_tc) / (ms * 1e-3), "ops": ops, "bytes": nbytes}
    out = {"workload": desc, "rows": M, "experts_hit": hit, "bound": "tensor", "unit": "TOP/s", "peak": peak_tops,
           "gate_up_fused(gemm+swiglu+requant)": tensor_entry(ms_up, ops_up, bytes_up), "down": tensor_entry(ms_down, ops_down, bytes_down)}
    if row_kernels:
        y = down()[0]
        row_idx = torch.arange(T * K, dtype=torch.int32, device=dev).view(K, T).t().contiguous()
        exb = x[torch.arange(M, device=dev) % T].contiguous()                  # [M, H] 16-bit rows for the quantiser
        h32 = npu.npu_grouped_matmul([ex], [w1], group_list=nums, split_item=2, group_type=0, group_list_type=1, output_dtype=3)[0]
        hb = (h32.float() * (xs[:, None] * 5.5e-3)).to(torch.bfloat16)         # [M, 2I] gate|up values as the layer's dequantisation spreads them
        table = {
            "init_routing(sort+gather)": (lambda: npu.npu_moe_init_routing(x, row_idx, ids, T), 2 * T * H + 2 * M * H + 24 * M),
            "dynamic_quant": (lambda: npu.npu_dynamic_quant(exb), 2 * M * H + M * H + 4 * M),
            "dispatch_pack(sort+quant+scatter)": (lambda: npu.npu_moe_distribute_dispatch(x, ids, "", 1, 0, E, quant_mode=2),
                                                  2 * T * H + M * H + 4 * M),
            "swiglu": (lambda: npu.npu_swiglu(hb), 2 * M * 2 * I + 2 * M * I),
            "dequant_swiglu_quant": (lambda: npu.npu_dequant_swiglu_quant(h32, weight_scale=s1, activation_scale=xs, group_index=nums,
                                                                         activate_left=True, quant_mode=1), M * (8 * I + I + 8)),
            "combine": (lambda: npu.npu_moe_distribute_combine(y, ids, expand_idx, ep_recv, wt, "", 1, 0, E), 2 * M * H + 4 * M + 2 * T * H),
        }
        rows = {}
        for k, (fn, nbytes) in table.items():
            ms = timer.launches(fn, reps)
            gbs = nbytes / (ms * 1e-3) / 1e9
            rows[k] = {"ms": ms, "GB/s": gbs, "frac": gbs / peak_gbs, "bytes": nbytes}
        out["row_kernels"] = {"rows": M, "cols": H, "bound": "hbm", "unit": "GB/s", "peak": peak_gbs, "kernels": rows}
    torchair_b200.check_status(dev)
    del w1, w2, ex, hq
    torch.cuda.empty_cache()
    return out


def check_layer(torch, dist, world, rank, dev, layer, x_d, ids_d, wt_d, w1, s1, w2, s2, E, tune):
    """Before anything is timed: the fused and the unfused layer must agree bit for bit on every rank, and the rows of
    two of this rank's experts (gate_up int8 + scales, down output) must equal the CPU formulas evaluated on the same
    received rows."""
    from oracle import moe_oracle as O
    npu = torch.ops.npu
    out_f = layer(x_d, ids_d, wt_d, fused=True)
    out_u = layer(x_d, ids_d, wt_d, fused=False)
    same = bool(torch.equal(out_f, out_u))
    ex, xs, expand_idx, nums, ep_recv, _, _ = npu.npu_moe_distribute_dispatch(x_d, ids_d, "ep", world, rank, E, quant_mode=2)
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1, tuning_config=tune)
    y = npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2, group_type=0,
                               group_list_type=1, output_dtype=15, tuning_config=tune)[0]
    out_c = npu.npu_moe_distribute_combine(y, ids_d, expand_idx, ep_recv, wt_d, "ep", world, rank, E)
    same = same and bool(torch.equal(out_c, out_u))
    nums_h = nums.cpu()
    starts = torch.cumsum(nums_h, 0) - nums_h
    hit = [int(e) for e in torch.nonzero(nums_h > 0).reshape(-1)]
    picked = sorted({hit[0], hit[-1]}) if hit else []
    rows_checked, oracle_ok = 0, True
    for e in picked:
        s0, c = int(starts[e]), int(nums_h[e])
        c = min(c, 64)
        we = O.MoeWeights(w1[e:e + 1].cpu(), s1[e:e + 1].cpu(), w2[e:e + 1].cpu(), s2[e:e + 1].cpu())
        col = {}
        yref = O.expert_ffn(ex[s0:s0 + c].cpu(), xs[s0:s0 + c].cpu(), torch.tensor([c]), we, col)
        oracle_ok = oracle_ok and torch.equal(hq[s0:s0 + c].cpu(), col["hq"][:c]) and torch.equal(hs[s0:s0 + c].cpu(), col["hs"][:c]) \
            and torch.equal(y[s0:s0 + c].cpu(), yref[:c])
        rows_checked += c
    flags = torch.tensor([int(same), int(oracle_ok)], device=dev)
    if world > 1:
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    ok_same, ok_oracle = bool(flags[0].item()), bool(flags[1].item())
    if not (ok_same and ok_oracle):
        raise RuntimeError(f"rank {rank}: output check failed before timing (fused == unfused on all ranks: {ok_same}; "
                           f"sampled experts equal the CPU formulas on all ranks: {ok_oracle})")
    return {"fused_equals_unfused_bit_for_bit": True, "ranks": world, "experts_vs_cpu_formulas": picked, "rows_vs_cpu_formulas": rows_checked,
            "compared": "int8 gate_up output, its scales and the 16-bit down output of the sampled experts: equal"}


def gpu_arm(args):
    import torch
    import torch.distributed as dist
    import torchair_b200
    from torchair_b200 import _lib, ep
    from torchair_b200.layer import moe_layer

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the CUDA path has no CPU fallback (use --impl reference for the CPU arm)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch N>1 with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        ep.register_ep_group("ep", dist.group.WORLD, transport=args.ep_transport)
    name, T, H, E, K, I, zipf = workload(world, args.workload)
    E_l = E // world

    # weights of this rank's experts, generated on the device; tokens generated on the host (seeded)
    g = torch.Generator(device=dev).manual_seed(args.seed * 100003 + rank)
    w1 = torch.randint(-127, 128, (E_l, H, 2 * I), generator=g, dtype=torch.int8, device=dev)
    w2 = torch.randint(-127, 128, (E_l, I, H), generator=g, dtype=torch.int8, device=dev)
    s1 = torch.rand(E_l, 2 * I, generator=g, device=dev) * 9e-3 + 1e-3
    s2 = torch.rand(E_l, H, generator=g, device=dev) * 9e-3 + 1e-3
    x_src, ids_src, wt_src = synthetic_tokens(torch, T, H, E, K, zipf, args.seed, rank)

    # the step's inputs live in ONE pinned host buffer and one device buffer per set, so that a step's host-to-device
    # transfer is a single copy: [x bf16 | expert ids int32 | routing weights fp32], each part 256-byte aligned
    al = lambda n: (n + 255) // 256 * 256
    nx, ni, nw = x_src.numel() * 2, ids_src.numel() * 4, wt_src.numel() * 4
    off_i, off_w, in_bytes = al(nx), al(nx) + al(ni), al(nx) + al(ni) + al(nw)
    in_h = torch.empty(in_bytes, dtype=torch.uint8).pin_memory()

    def views(buf):
        return (buf[:nx].view(torch.bfloat16).view(T, H), buf[off_i:off_i + ni].view(torch.int32).view(T, K),
                buf[off_w:off_w + nw].view(torch.float32).view(T, K))
    for dst, src in zip(views(in_h), (x_src, ids_src, wt_src)):
        dst.copy_(src)
    NSETS = 3                # buffer sets of the end-to-end pipeline: previous step's result, this step, next step's inputs
    LAG = 2                  # the host reads a result two steps after issuing it
    in_d = [in_h.to(dev) for _ in range(NSETS)]
    x_d, ids_d, wt_d = views(in_d[0])
    out_h = [torch.empty((T, H), dtype=torch.bfloat16).pin_memory() for _ in range(NSETS)]

    def layer(x, ids, wt, fused=True, after_dispatch=None):
        return moe_layer(x, ids, wt, w1, s1, w2, s2, group_ep="ep", ep_world_size=world, ep_rank_id=rank, moe_expert_num=E, fused=fused,
                         after_dispatch=after_dispatch)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    windows = []
    timer = Timer(torch, windows)

    # warm-up (also fills the packed-weight cache), then the output check, then capture
    for _ in range(3):
        layer(x_d, ids_d, wt_d)
    torch.cuda.synchronize()
    tune = [max(1, -(-T * K * world // E))]       # rows an expert is expected to receive: the grouped matmuls' tiling hint
    checked = check_layer(torch, dist, world, rank, dev, layer, x_d, ids_d, wt_d, w1, s1, w2, s2, E, tune)
    torchair_b200.check_status(dev)

    use_graph = world == 1 or args.ep_transport == "peer"     # the peer-memory exchange has no host read: one graph per rank
    graphs, outs = [], []
    launches_per_step = None
    for b in range(NSETS if use_graph else 0):
        gr = torch.cuda.CUDAGraph()
        c0 = _lib.launch_count()
        with torch.cuda.graph(gr):
            o = layer(*views(in_d[b]))
        if launches_per_step is None:
            launches_per_step = _lib.launch_count() - c0      # this library's kernels recorded into one step's graph
        graphs.append(gr)
        outs.append(o)
    if not use_graph:
        torch.cuda.synchronize()
        c0 = _lib.launch_count()
        layer(x_d, ids_d, wt_d)
        launches_per_step = _lib.launch_count() - c0
    for gr in graphs:
        gr.replay()
    torch.cuda.synchronize()

    def step_resident():
        if use_graph:
            graphs[0].replay()
        else:
            layer(x_d, ids_d, wt_d)

    def timed(fn, steps, finish=None):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_a = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()                 # the timed stream waits for the last results to reach the host buffers
        e1.record()
        torch.cuda.synchronize()
        t_b = time.time()
        if world > 1:
            dist.barrier()
        windows.append((t_a, t_b))
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def timed_blocks(fn, steps, finish=None, target_ms=1000.0):
        """Blocks of exactly `steps` steps; their number follows from the first block (a maximum over ranks, so every rank
        computes the same count) so that about a second is measured in all; the median block is the result."""
        first = timed(fn, steps, finish)
        repeats = int(max(3, min(400, math.ceil(target_ms / max(first, 1e-3)))))
        blocks = [first] + [timed(fn, steps, finish) for _ in range(repeats - 1)]
        return statistics.median(blocks), blocks

    # (1) device-resident inputs
    for _ in range(max(args.warmup, 3)):
        step_resident()
    total_ms, blocks = timed_blocks(step_resident, args.steps)
    ms_per_step = total_ms / args.steps
    value = T * world * args.steps / (total_ms * 1e-3)

    # (2) end to end through the public ops with host buffers: every step copies its inputs from pinned host memory and its
    # result back into pinned host memory.  With a captured layer the step's graph has three branches: the layer on set b
    # and, forked off after its dispatch, the host-to-device copy of the NEXT step's inputs into set b + 1 and the
    # device-to-host copy of the PREVIOUS step's result (set b - 1).  A step is then one graph launch; the host waits for the result of the
    # step issued two steps earlier, so the device queue never runs dry, and no cross-stream event sits between two steps
    # (with expert parallelism the ranks move in lock step, so a late start on one rank delays all of them).
    finish_e2e = None
    if use_graph:
        side_in, side_out = torch.cuda.Stream(), torch.cuda.Stream()
        stage = [torch.empty((T, H), dtype=torch.bfloat16, device=dev) for _ in range(NSETS)]    # a step's result on the device
        e2e_graphs = []
        for b_ in range(NSETS):
            nxt, prv = (b_ + 1) % NSETS, (b_ - 1) % NSETS
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                main = torch.cuda.current_stream()

                def fork_copies():
                    # Called by the layer once its dispatch is enqueued: the transfers then run beside the expert GEMMs.
                    # Forked at the start of the step they ran beside the latency-bound exchange and cost the step 31 us
                    # on 2 GPUs; here 12 us.
                    side_in.wait_stream(main)
                    side_out.wait_stream(main)
                    with torch.cuda.stream(side_in):
                        in_d[nxt].copy_(in_h, non_blocking=True)
                    with torch.cuda.stream(side_out):
                        out_h[prv].copy_(stage[prv], non_blocking=True)
                stage[b_].copy_(layer(*views(in_d[b_]), after_dispatch=fork_copies))
                main.wait_stream(side_in)
                main.wait_stream(side_out)
            e2e_graphs.append(gr)
        ev_step = [torch.cuda.Event() for _ in range(NSETS)]
        state = {"s": 0}
        in_d[0].copy_(in_h, non_blocking=True)          # the first step's inputs (every later copy-in rides in a step's graph)

        def step_e2e():
            s_ = state["s"]
            b = s_ % NSETS
            e2e_graphs[b].replay()
            ev_step[b].record()
            if s_ >= LAG:
                ev_step[(s_ - LAG + 1) % NSETS].synchronize()   # that graph carried the copy-out of step s - LAG: the caller reads it
            state["s"] = s_ + 1

        def finish_e2e():
            # the result of the block's last step leaves with the next step's graph; at the end of a block it is copied here
            last = (state["s"] - 1) % NSETS
            out_h[last].copy_(stage[last], non_blocking=True)
    else:
        def step_e2e():
            in_d[0].copy_(in_h, non_blocking=True)
            out_h[0].copy_(layer(x_d, ids_d, wt_d), non_blocking=True)
            torch.cuda.current_stream().synchronize()     # the caller reads the result every step

    for _ in range(max(args.warmup, 3)):
        step_e2e()
    e2e_ms, e2e_blocks = timed_blocks(step_e2e, args.steps, finish_e2e)
    e2e_value = T * world * args.steps / (e2e_ms * 1e-3)
    h2d = nx + ni + nw
    d2h = out_h[0].numel() * 2
    if use_graph:                      # the pipelined result must be the layer's result
        torch.cuda.synchronize()
        if not torch.equal(out_h[(state["s"] - 1) % NSETS], outs[0].cpu()):
            raise RuntimeError("the end-to-end pipeline returned a result that differs from the resident run")

    # (3) the dominant kernel alone: gate_up grouped GEMM (+ its two helper launches) and the down GEMM
    npu = torch.ops.npu
    ex, xs, expand_idx, nums, ep_recv, _, _ = npu.npu_moe_distribute_dispatch(x_d, ids_d, "ep", world, rank, E, quant_mode=2)
    M = ex.shape[0]
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1, tuning_config=tune)
    rows = int(nums.sum().item())
    experts_hit = int((nums > 0).sum().item())
    reps = max(20, min(args.steps * 2, 100))
    ms_up = timer.launches(lambda: npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1,
                                                                          tuning_config=tune), reps)
    ms_down = timer.launches(lambda: npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2,
                                                            group_type=0, group_list_type=1, output_dtype=15, tuning_config=tune), reps)
    ms_disp = timer.launches(lambda: npu.npu_moe_distribute_dispatch(x_d, ids_d, "", 1, 0, E, quant_mode=2), reps) if world == 1 else None
    bytes_up = experts_hit * H * 2 * I + rows * H + rows * I * 4 + experts_hit * 2 * I * 4 + rows * 4   # weights + A + fp32 h + scales
    bytes_down = experts_hit * I * H + rows * I + rows * H * 2 + experts_hit * H * 4 + rows * 4
    torchair_b200.check_status(dev)

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    # int8 dense tensor peak: twice the bf16 rate; the measured bf16 GEMM burst figure when the pod wrote one
    peak_tops = 2.0 * float(peaks.get("bf16_tflops", 1590.0))
    measured = "hbm_gbs" in peaks
    ops_up = 2.0 * rows * H * 2 * I
    ops_down = 2.0 * rows * I * H
    t_hbm, t_tc = bytes_up / (peak_gbs * 1e9), ops_up / (peak_tops * 1e12)
    gbs_up = bytes_up / (ms_up * 1e-3) / 1e9
    tops_up = ops_up / (ms_up * 1e-3) / 1e12
    hbm_source = "measured copy bandwidth (MEASURED_PEAKS.json)" if measured else "fallback 6650 GB/s"
    tc_source = ("2 x measured bf16 GEMM burst (MEASURED_PEAKS.json); nominal int8 dense is 4500"
                 if measured else "2 x fallback bf16 1590; nominal int8 dense is 4500")
    if t_hbm >= t_tc:
        main = {"bound": "hbm", "achieved": gbs_up, "peak": peak_gbs, "unit": "GB/s", "frac": gbs_up / peak_gbs, "peak_source": hbm_source}
    else:
        main = {"bound": "tensor", "achieved": tops_up, "peak": peak_tops, "unit": "TOP/s", "frac": tops_up / peak_tops,
                "peak_source": tc_source, "frac_of_nominal_4500": tops_up / 4500.0}
    # DRAM bytes per launch, from an ncu capture of this kernel on the 1/8-scale decode case: 948.42 MB for 32 experts hit; the
    # traffic is one pass over each hit expert's weights, so it is scaled by the experts hit
    traffic = 948.417e6 / 32 * experts_hit if (H, I) == (7168, 2048) and rows <= 16 * experts_hit else None
    roofline = dict(main)
    roofline.update({"kernel": "gmm_i8_kernel<NT,fused> gate_up (timed with its memset and requantise helper launches)",
                     "timing": "CUDA events around replays of a CUDA graph that holds five launches of the operator; median",
                     "algorithmic_bytes": bytes_up, "algorithmic_ops": ops_up, "ms_per_launch": ms_up, "traffic": traffic,
                     "traffic_source": None if traffic is None else "ncu dram__bytes of the 1/8-scale decode case, scaled by experts hit",
                     "GB/s": gbs_up, "int8_tops": tops_up, "rows": rows, "experts_hit": experts_hit,
                     "others": {"down_gemm": {"ms": ms_down, "GB/s": bytes_down / (ms_down * 1e-3) / 1e9,
                                              "frac": bytes_down / (ms_down * 1e-3) / 1e9 / peak_gbs,
                                              "int8_tops": ops_down / (ms_down * 1e-3) / 1e12},
                                "dispatch_sort_quant_scatter": None if ms_disp is None else
                                {"ms": ms_disp, "GB/s": (2 * T * H + M * H + 4 * M) / (ms_disp * 1e-3) / 1e9,
                                 "note": "latency-bound at this size; the bandwidth-bound size is under row_kernels"}}})

    others_on = world == 1 and not args.no_others and args.workload == "auto"
    if others_on:
        # the parts of the metric that the decode shape cannot show: tensor-bound grouped GEMMs and bandwidth-bound row kernels
        oth = roofline["others"]
        oth["peak_sources"] = {"tensor": tc_source, "hbm": hbm_source}
        r3 = gemm_pair(torch, timer, dev, EXTRA_WORKLOADS["cfg3_rank"], args.seed, reps, peak_tops, peak_gbs, row_kernels=True)
        oth["row_kernels_65536x7168"] = r3.pop("row_kernels")
        oth["prefill_gemm_cfg3_rank"] = r3
        oth["prefill_gemm_cfg4"] = gemm_pair(torch, timer, dev, EXTRA_WORKLOADS["cfg4"], args.seed, reps, peak_tops, peak_gbs, row_kernels=False)
    if args.kernels and world == 1 and args.workload != "auto":
        rep = gemm_pair(torch, timer, dev, EXTRA_WORKLOADS[args.workload], args.seed, reps, peak_tops, peak_gbs, row_kernels=True)
        print("KERNELS " + json.dumps(rep), file=sys.stderr, flush=True)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.workload == "auto":
        r = run_cpu(steps=10, warmup=2, seed=args.seed, n_gpus=1, budget_s=60.0)
        cpu = {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"],
               "full_config": r["full_config"], "cpu_model": r["cpu_model"], "torch": r["torch"]}

    if sampler is not None:
        sampler.stop()
    if rank == 0:
        weight_bytes = w1.numel() + w2.numel()
        conf = config_dict(name, T, H, E, K, I, world)
        conf.update({"cuda_graph": use_graph, "ep_transport": None if world == 1 else args.ep_transport,
                     "exchange": None if world == 1 else ("this library's kernels store rows into the owners' buffers over NVLink peer "
                                                          "memory; NCCL only carries the rendezvous" if args.ep_transport == "peer"
                                                          else "NCCL all_to_all_single"),
                     "l2": "inputs larger than L2: every step streams this rank's int8 expert weights "
                           f"({weight_bytes / 1e9:.2f} GB) from HBM"})
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": SCALING, "scaling_note": SCALING_NOTE,
                "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": conf,
                "repeats": len(blocks), "block_ms": {"median": total_ms, "min": min(blocks), "max": max(blocks)},
                "stream_frac": weight_bytes / (ms_per_step * 1e-3) / 1e9 / peak_gbs,
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms / args.steps, "repeats": len(e2e_blocks),
                        "pipelining": ("a step is one CUDA-graph launch with three branches: the layer and, beside its expert GEMMs, the "
                                       "copy-in of the next step's inputs and the copy-out of the previous step's result (three buffer "
                                       "sets); the host reads a result two steps after issuing it") if use_graph else "none"},
                "gpu_launches": launches_per_step * args.steps, "gpu_launches_per_step": launches_per_step,
                "gpu_launches_counted": "kernels this library enqueued while one step was recorded (tab_launch_count)",
                "checked": checked, "roofline": roofline, "cpu_baseline": cpu,
                "clocks": sampler.summary(windows) if sampler is not None else None}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()

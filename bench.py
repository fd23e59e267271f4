#!/usr/bin/env python
"""Benchmark of the W8A8 expert-parallel MoE layer: int8 MoE-layer tokens/s on 1/2/4/8 B200.

    python bench.py --gpus 1 --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W     # the CPU formulas of the path on the host cores
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass of the layer (dispatch with per-token int8 quantisation -> gate_up grouped GEMM with the
dequant+SwiGLU+requant epilogue -> down grouped GEMM -> combine) over one batch of seeded synthetic tokens.
N = 1 runs the decode shape with all 256 experts local (256 tokens, hidden 7168, top-8, intermediate 2048);
N > 1 runs the expert-parallel decode shape (128 tokens per rank, 256/N experts per rank, NCCL all-to-all).
Prints ONE JSON line on rank 0.
"""
import argparse
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

METRIC = "int8_moe_layer_tokens_per_s"
UNIT = "tokens/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (N=1)")
    ap.add_argument("--ep-transport", default="peer", choices=["peer", "nccl"],
                    help="N > 1: rows move by this library's peer-memory kernels (default) or by NCCL all-to-all")
    ap.add_argument("--kernels", action="store_true",
                    help="also time every kernel of the path alone and write the table to stderr (study aid, N=1)")
    ap.add_argument("--workload", default="auto", choices=["auto", "cfg3"] + sorted(EXTRA_WORKLOADS),
                    help="auto = the headline configuration for this GPU count; the others are single-GPU study cases")
    return ap.parse_args()


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


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle on the host cores, on a bounded sample of the workload
# ---------------------------------------------------------------------------------------------------
def cpu_sample_config(n_gpus=1):
    """A bounded sample with the workload's rows per expert and expert shape.  N = 1: 32 tokens routed top-8 over 32
    experts (1/8 of the 256-token / 256-expert layer).  N > 1: a 32-expert slice of one rank's experts with the tokens
    scaled alike (128 tokens per rank spread over 256/N local experts)."""
    from oracle import moe_oracle as O
    if n_gpus == 1:
        return O.MoeConfig("cfg1_sample", 32, 7168, 32, 8, 2048), "1/8 of the 256-token/256-expert layer at the same rows per expert"
    e_l = 256 // n_gpus
    e_s = min(e_l, 32)
    t_s = max(8, 128 * e_s // e_l)
    return (O.MoeConfig("cfg2_sample", t_s, 7168, e_s, 8, 2048),
            f"{e_s} of the {e_l} experts of one rank with {t_s} of its 128 tokens (same rows per expert)")


def run_cpu(steps, warmup, seed, n_gpus=1):
    import torch
    from oracle import moe_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    cfg, what = cpu_sample_config(n_gpus)
    w = O.make_weights(cfg, seed)
    x, ids, wt = O.make_tokens(cfg, seed)
    for _ in range(warmup):
        O.moe_layer([x], [ids], [wt], w)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.moe_layer([x], [ids], [wt], w)
    dt = time.perf_counter() - t0
    return {"value": cfg.T * steps / dt, "ms_per_step": dt / steps * 1e3, "cores": torch.get_num_threads(),
            "sample": f"{cfg.T} tokens top-{cfg.K} over {cfg.E} experts (hidden {cfg.H}, intermediate {cfg.I}): {what}; "
                      f"{steps} passes after {warmup} warm-up",
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
    steps = max(1, min(args.steps, 100))         # a pass is ~0.2 s of CPU work: the whole run stays well under a minute
    warmup = max(1, min(args.warmup, 3))
    r = run_cpu(steps, warmup, args.seed, args.gpus)
    name = workload(args.gpus)[0]
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": name, "sample": r["sample"]},
            "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"],
                             "cpu_model": r["cpu_model"], "torch": r["torch"]},
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
def gpu_arm(args):
    import torch
    import torch.distributed as dist
    import torchair_b200
    from torchair_b200 import ep
    from torchair_b200.layer import moe_layer
    from oracle import moe_oracle as O

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
    cfg = O.MoeConfig("bench", T, H, E, K, I, zipf_s=zipf)

    # weights of this rank's experts, generated on the device; tokens generated on the host (seeded)
    g = torch.Generator(device=dev).manual_seed(args.seed * 100003 + rank)
    w1 = torch.randint(-127, 128, (E_l, H, 2 * I), generator=g, dtype=torch.int8, device=dev)
    w2 = torch.randint(-127, 128, (E_l, I, H), generator=g, dtype=torch.int8, device=dev)
    s1 = torch.rand(E_l, 2 * I, generator=g, device=dev) * 9e-3 + 1e-3
    s2 = torch.rand(E_l, H, generator=g, device=dev) * 9e-3 + 1e-3
    x_h, ids_h, wt_h = O.make_tokens(cfg, args.seed, rank)
    x_h, ids_h, wt_h = x_h.pin_memory(), ids_h.pin_memory(), wt_h.pin_memory()
    out_h = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    x_d, ids_d, wt_d = x_h.to(dev), ids_h.to(dev), wt_h.to(dev)

    def layer(x, ids, wt):
        return moe_layer(x, ids, wt, w1, s1, w2, s2, group_ep="ep", ep_world_size=world, ep_rank_id=rank, moe_expert_num=E)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    windows = []

    # warm-up (also fills the packed-weight cache); single rank: capture the layer into one CUDA graph
    for _ in range(max(args.warmup, 3)):
        out = layer(x_d, ids_d, wt_d)
    torch.cuda.synchronize()
    graph = None
    if world == 1 or args.ep_transport == "peer":     # the peer-memory exchange has no host read: one graph per rank
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = layer(x_d, ids_d, wt_d)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()

    def step_resident():
        if graph is not None:
            graph.replay()
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
            finish()                 # the timed stream waits for the last result to reach the host buffer
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

    # (1) device-resident inputs
    for _ in range(args.warmup):
        step_resident()
    total_ms = timed(step_resident, args.steps)
    ms_per_step = total_ms / args.steps
    value = T * world * args.steps / (total_ms * 1e-3)

    # (2) end to end through the public ops with host buffers: H2D of the step's inputs, layer, D2H of the result.
    # With a captured layer the three stages of consecutive steps overlap on three streams over two buffer sets (copy in
    # step s+1 while step s computes and step s-1 copies out); the caller reads a result one step after it was issued.
    finish_e2e = None
    if graph is not None:
        x_d2, ids_d2, wt_d2 = x_d.clone(), ids_d.clone(), wt_d.clone()
        out_h2 = torch.empty_like(out_h).pin_memory()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2):
            out2 = layer(x_d2, ids_d2, wt_d2)
        sets = [(x_d, ids_d, wt_d, graph, out, out_h), (x_d2, ids_d2, wt_d2, graph2, out2, out_h2)]
        copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event(), torch.cuda.Event()]
        ev_comp = [torch.cuda.Event(), torch.cuda.Event()]
        ev_out = [torch.cuda.Event(), torch.cuda.Event()]
        state = {"s": 0}

        def step_e2e():
            s_ = state["s"]
            b = s_ & 1
            xd, idd, wtd, g, o, oh = sets[b]
            main = torch.cuda.current_stream()
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(ev_comp[b])          # this set's previous compute has consumed its inputs
                xd.copy_(x_h, non_blocking=True)
                idd.copy_(ids_h, non_blocking=True)
                wtd.copy_(wt_h, non_blocking=True)
                ev_in[b].record(copy_in)
            main.wait_event(ev_in[b])
            main.wait_event(ev_out[b])                  # this set's previous result has left the device
            g.replay()
            ev_comp[b].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(ev_comp[b])
                oh.copy_(o, non_blocking=True)
                ev_out[b].record(copy_out)
            if s_ >= 1:
                ev_out[b ^ 1].synchronize()             # the caller reads the previous step's result
            state["s"] = s_ + 1

        def finish_e2e():
            last = (state["s"] - 1) & 1
            torch.cuda.current_stream().wait_event(ev_out[last])
    else:
        def step_e2e():
            x_d.copy_(x_h, non_blocking=True)
            ids_d.copy_(ids_h, non_blocking=True)
            wt_d.copy_(wt_h, non_blocking=True)
            out_h.copy_(layer(x_d, ids_d, wt_d), non_blocking=True)
            torch.cuda.current_stream().synchronize()     # the caller reads the result every step

    for _ in range(args.warmup):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps, finish_e2e)
    e2e_value = T * world * args.steps / (e2e_ms * 1e-3)
    h2d = x_h.numel() * 2 + ids_h.numel() * 4 + wt_h.numel() * 4
    d2h = out_h.numel() * 2

    # (3) the dominant kernel alone: gate_up grouped GEMM (+ its two helper launches) and the down GEMM
    npu = torch.ops.npu
    ex, xs, expand_idx, nums, ep_recv, _, _ = npu.npu_moe_distribute_dispatch(x_d, ids_d, "ep", world, rank, E, quant_mode=2)
    M = ex.shape[0]
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1)
    rows = int(nums.sum().item())
    experts_hit = int((nums > 0).sum().item())

    def time_each(fn, reps):
        times = []
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        t_a = time.time()
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
        windows.append((t_a, time.time()))
        return sum(times) / len(times)

    def time_launches(fn, reps, inner=5):
        """Average device time of one call of fn: `inner` calls are captured into one CUDA graph and the replays are timed
        with events, so that the host's per-call work (allocation, ctypes, launch latency) is not counted as kernel time."""
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
        for _ in range(max(3, reps // inner)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g_.replay()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b) / inner)
        windows.append((t_a, time.time()))
        del g_
        return sum(times) / len(times)

    reps = max(10, min(args.steps, 100))
    ms_up = time_launches(lambda: npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1), reps)
    ms_down = time_launches(lambda: npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2,
                                                           group_type=0, group_list_type=1, output_dtype=15), reps)
    ms_disp = time_each(lambda: npu.npu_moe_distribute_dispatch(x_d, ids_d, "", 1, 0, E, quant_mode=2), reps) if world == 1 else None
    bytes_up = experts_hit * H * 2 * I + rows * H + rows * I * 4 + experts_hit * 2 * I * 4 + rows * 4   # weights + A + fp32 h + scales
    bytes_down = experts_hit * I * H + rows * I + rows * H * 2 + experts_hit * H * 4 + rows * 4
    status = torchair_b200.gmm_status(dev)
    if status != 0:
        raise RuntimeError(f"grouped GEMM reported a timed-out wait (code {status})")
    if ep.peer_status() != 0:
        raise RuntimeError(f"a peer-memory flag wait ran out of time (code {ep.peer_status()})")

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
    if t_hbm >= t_tc:
        main = {"bound": "hbm", "achieved": gbs_up, "peak": peak_gbs, "unit": "GB/s", "frac": gbs_up / peak_gbs,
                "peak_source": "measured copy bandwidth (MEASURED_PEAKS.json)" if measured else "fallback 6650 GB/s"}
    else:
        main = {"bound": "tensor", "achieved": tops_up, "peak": peak_tops, "unit": "TOP/s", "frac": tops_up / peak_tops,
                "peak_source": ("2 x measured bf16 GEMM burst (MEASURED_PEAKS.json); nominal int8 dense is 4500"
                                if measured else "2 x fallback bf16 1590; nominal int8 dense is 4500"),
                "frac_of_nominal_4500": tops_up / 4500.0}
    # DRAM bytes per launch from the ncu capture of the 1/8-scale decode case (profiles/gmm_i8_kernel_decode_small.md):
    # 948.42 MB for 32 experts; traffic is one pass over each hit expert's weights, so it scales with experts_hit.
    traffic = 948.417e6 / 32 * experts_hit if (H, I) == (7168, 2048) and rows <= 16 * experts_hit else None
    roofline = dict(main)
    roofline.update({"kernel": "gmm_i8_kernel<NT,fused> gate_up (timed with its memset and requantise helper launches)",
                     "timing": "CUDA events around replays of a CUDA graph that holds five launches of the operator",
                     "algorithmic_bytes": bytes_up, "algorithmic_ops": ops_up, "ms_per_launch": ms_up, "traffic": traffic,
                     "GB/s": gbs_up, "int8_tops": tops_up, "rows": rows, "experts_hit": experts_hit,
                     "others": {"down_gemm": {"ms": ms_down, "GB/s": bytes_down / (ms_down * 1e-3) / 1e9,
                                              "int8_tops": ops_down / (ms_down * 1e-3) / 1e12},
                                "dispatch_sort_quant_scatter": None if ms_disp is None else
                                {"ms": ms_disp, "GB/s": (2 * T * H + M * H + 4 * M) / (ms_disp * 1e-3) / 1e9}}})

    if args.kernels and world == 1:
        def gbs(nbytes, ms):
            return round(nbytes / (ms * 1e-3) / 1e9, 1)
        row_idx = torch.arange(T * K, dtype=torch.int32, device=dev).view(K, T).t().contiguous()
        y_bf16 = npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2,
                                        group_type=0, group_list_type=1, output_dtype=15)[0]
        exb = x_d[torch.arange(M, device=dev) % T].contiguous()          # [M, H] bf16 rows for the quantiser
        h32 = torch.randint(-2000000, 2000000, (min(M, 16384), 2 * I), dtype=torch.int32, device=dev)
        hb = torch.randn((M, 2 * I), dtype=torch.float32, device=dev).to(torch.bfloat16)
        m32 = h32.shape[0]
        ones = torch.ones(m32, dtype=torch.float32, device=dev)
        table = {
            "init_routing": (time_launches(lambda: npu.npu_moe_init_routing(x_d, row_idx, ids_d, T), reps), 2 * T * H + 2 * M * H + 24 * M),
            "dynamic_quant": (time_launches(lambda: npu.npu_dynamic_quant(exb), reps), 2 * M * H + M * H + 4 * M),
            "dispatch_pack(sort+quant+scatter)": (time_launches(lambda: npu.npu_moe_distribute_dispatch(x_d, ids_d, "", 1, 0, E, quant_mode=2), reps),
                                                  2 * T * H + M * H + 4 * M),
            "swiglu_bf16": (time_launches(lambda: npu.npu_swiglu(hb), reps), 2 * M * 2 * I + 2 * M * I),
            "dequant_swiglu_quant": (time_launches(lambda: npu.npu_dequant_swiglu_quant(h32, weight_scale=s1[:1], activation_scale=ones,
                                                                                   activate_left=True, quant_mode=1), reps),
                                     m32 * (8 * I + I + 8)),
            "combine": (time_launches(lambda: npu.npu_moe_distribute_combine(y_bf16, ids_d, expand_idx, ep_recv, wt_d, "", 1, 0, E), reps),
                        2 * M * H + 4 * M + 2 * T * H),
            "gmm_gate_up_fused": (ms_up, bytes_up), "gmm_down": (ms_down, bytes_down),
        }
        # down GEMM + logit-weighted scatter-add as one operator (int32 accumulators round-trip through the workspace)
        tok_of_row = torch.arange(M, device=dev) % T          # K rows per token; which ones does not matter for the timing
        lg = torch.rand(M, device=dev)
        table["gmm_down+finalize_routing"] = (
            time_launches(lambda: npu.npu_grouped_matmul_finalize_routing(hq, w2, nums, scale=s2, pertoken_scale=hs, logit=lg,
                                                                      row_index=tok_of_row, output_bs=T, group_list_type=1), reps),
            experts_hit * I * H + rows * I + 2 * rows * H * 4 + T * H * 4 + experts_hit * H * 4 + rows * 16)
        # context: what plain torch kernels reach on this GPU for write-only and copy traffic of 1 GiB
        probe = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
        probe2 = torch.empty_like(probe)
        # (single eager calls: inside a graph a device-to-device copy_ becomes a copy-engine node, not the kernel)
        table["context: torch fill (write only)"] = (time_each(lambda: probe.fill_(1), reps), probe.numel())
        table["context: torch copy (read + write)"] = (time_each(lambda: probe2.copy_(probe), reps), 2 * probe.numel())
        report = {k: {"ms": round(ms, 4), "GB/s": gbs(b, ms), "frac_hbm": round(gbs(b, ms) / peak_gbs, 3)} for k, (ms, b) in table.items()}
        report["gmm_gate_up_fused"]["int8_tops"] = round(tops_up, 1)
        report["gmm_down"]["int8_tops"] = round(ops_down / (ms_down * 1e-3) / 1e12, 1)
        print("KERNELS " + json.dumps({"workload": name, "kernels": report}), file=sys.stderr, flush=True)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = run_cpu(steps=50, warmup=2, seed=args.seed)     # ~10-20 s of CPU work
        cpu = {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"],
               "cpu_model": r["cpu_model"], "torch": r["torch"]}

    if sampler is not None:
        sampler.stop()
    if rank == 0:
        # sort x3, pack, gemm, requant, gemm, combine; nccl adds plan + permute each way; peer adds send, unpack, two plans,
        # the return-address table (the down GEMM stores into the peers itself) and eight flag kernels
        launches_per_step = 8 if world == 1 else (21 if args.ep_transport == "peer" else 12)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
                "data": "synthetic",
                "config": {"workload": name, "tokens_per_rank": T, "hidden": H, "experts": E, "experts_per_rank": E_l, "top_k": K,
                           "intermediate": I, "parallelism": f"ep{world}", "cuda_graph": graph is not None,
                           "ep_transport": None if world == 1 else args.ep_transport,
                           "l2": "inputs larger than L2: every step streams this rank's int8 expert weights "
                                 f"({(w1.numel() + w2.numel()) / 1e9:.2f} GB) from HBM"},
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms / args.steps,
                        "pipelining": "copy-in, compute and copy-out of consecutive steps overlap (two buffer sets)"
                        if graph is not None else "none"},
                "gpu_launches": launches_per_step * args.steps,
                "roofline": roofline, "cpu_baseline": cpu,
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

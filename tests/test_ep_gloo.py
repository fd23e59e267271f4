"""Expert-parallel host logic over real torch.distributed ranks on CPU (gloo, world size 2 and 4).

The exchange code of torchair_b200.ep is the shipped one; only the four device steps are replaced by the CPU
stand-ins of oracle/ep_standins.py.  Results must equal the oracle's simulated-ranks layer bit for bit.
"""
import os
import socket
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O
from oracle.ep_standins import OracleKernels
from torchair_b200 import ep


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, cfg_name, nums_type, q, outdir):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ep.register_ep_group("ep_test", dist.group.WORLD)
        cfg = O.CONFIGS[cfg_name]
        E_l = cfg.E // world
        w = O.make_weights(cfg, seed=0, experts=range(rank * E_l, (rank + 1) * E_l))
        x, ids, wt = O.make_tokens(cfg, 0, rank)
        outs = ep.dispatch(OracleKernels, x, ids, "ep_test", world, rank, cfg.E, 2, nums_type)
        ex, ds, expand_idx, nums, ep_recv = outs[:5]
        counts = nums if nums_type == 1 else torch.diff(nums, prepend=torch.zeros(1, dtype=torch.int64))
        y = O.expert_ffn(ex, ds, counts, w)
        # once through the remembered split sizes, once with copied handshake tensors (sizes rebuilt from them)
        out_a = ep.combine(OracleKernels, y, ids, expand_idx, ep_recv, wt, "ep_test", world, rank, cfg.E)
        out_b = ep.combine(OracleKernels, y, ids, expand_idx.clone(), ep_recv.clone(), wt, "ep_test", world, rank, cfg.E)
        torch.save((out_a, out_b, ex, ds, nums, ep_recv), os.path.join(outdir, f"rank{rank}.pt"))
        q.put((rank, "ok"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.parametrize("world,nums_type", [(2, 1), (2, 0), (4, 1), (8, 1)])
def test_expert_parallel_layer_over_gloo_matches_oracle(world, nums_type, tmp_path):
    cfg = O.CONFIGS["cfg0"]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, "cfg0", nums_type, q, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        item = q.get(timeout=180)
        assert item[1] == "ok", item[2]
    for p in procs:
        p.join(timeout=60)
    results = {r: torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)}
    w = O.make_weights(cfg, seed=0)
    xs, idl, wl = zip(*[O.make_tokens(cfg, 0, r) for r in range(world)])
    collect = []
    ref = O.moe_layer(xs, idl, wl, w, collect)
    for r in range(world):
        out_a, out_b, ex, ds, nums, ep_recv = results[r]
        d = collect[r]["disp"]
        n_rows = int(d.expert_token_nums.sum())             # rows past the received total are not written
        assert torch.equal(ex[:n_rows], d.expand_x[:n_rows]) and torch.equal(ds[:n_rows], d.dynamic_scales[:n_rows])
        assert torch.equal(ep_recv, d.ep_recv_count)
        want_nums = d.expert_token_nums if nums_type == 1 else torch.cumsum(d.expert_token_nums, 0)
        assert torch.equal(nums, want_nums)
        assert torch.equal(out_a, ref[r]) and torch.equal(out_b, ref[r])


def _failing_worker(rank, world, port, q):
    """Rank 1 raises before the exchange; rank 0 must get an error from its collective instead of hanging."""
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import datetime
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
        ep.register_ep_group("ep_fail", dist.group.WORLD)
        cfg = O.CONFIGS["cfg0"]
        x, ids, _ = O.make_tokens(cfg, 0, rank)
        if rank == 1:
            raise RuntimeError("injected host-side failure before dispatch")
        ep.dispatch(OracleKernels, x, ids, "ep_fail", world, rank, cfg.E, 2, 1)
        q.put((rank, "finished"))
    except Exception as e:
        q.put((rank, "raised", type(e).__name__, str(e)[:200]))


def test_peer_failure_surfaces_as_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        item = q.get(timeout=120)
        got[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert got[1][0] == "raised" and "injected" in got[1][2]
    assert got[0][0] == "raised", f"rank 0 should see a collective error, got {got[0]}"


def test_group_registry_and_argument_mismatch():
    with pytest.raises(RuntimeError, match="not registered"):
        ep.get_ep_group("nobody")
    with pytest.raises(ValueError):
        ep.register_ep_group("", None)
    x = torch.zeros(4, 32, dtype=torch.bfloat16)
    ids = torch.zeros(4, 2, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="inconsistent"):
        ep.check_dispatch_args(x, ids, 3, 0, 8, None, None, 0, 0, 0, 2, 0, 1)
    with pytest.raises(RuntimeError, match="inconsistent"):
        ep.check_dispatch_args(x, ids, 2, 2, 8, None, None, 0, 0, 0, 2, 0, 1)
    assert ep.dispatch_rows(128, 8, 256, 8) == 8192
    assert ep.dispatch_rows(8192, 8, 256, 8) == 524288


def test_single_rank_dispatch_needs_no_group():
    cfg = O.CONFIGS["cfg0"]
    x, ids, wt = O.make_tokens(cfg, 0, 0)
    outs = ep.dispatch(OracleKernels, x, ids, "", 1, 0, cfg.E, 2, 0)
    d = O.moe_distribute_dispatch([x], [ids], cfg.E, expert_token_nums_type=0)[0]
    assert torch.equal(outs[0], d.expand_x) and torch.equal(outs[3], d.expert_token_nums)
    assert torch.equal(outs[2], d.expand_idx) and torch.equal(outs[4], d.ep_recv_count)


def _options_inputs(world):
    """Ranks with different numbers of tokens (global_bs), a token mask each, and special experts among the ids."""
    E, K, H, special = 8, 3, 64, 3
    toks, g = [], torch.Generator().manual_seed(99)
    for r in range(world):
        T = 12 + 5 * r
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        ids = torch.stack([torch.randperm(E + special, generator=g)[:K] for _ in range(T)]).to(torch.int32)
        wt = torch.rand(T, K, generator=g)
        mask = torch.rand(T, generator=g) < 0.8
        toks.append((x, ids, wt, mask))
    consts = [torch.randn(1, H, generator=g).to(torch.bfloat16) for _ in range(3)]
    return E, K, H, special, toks, consts


def _options_worker(rank, world, port, q, outdir):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ep.register_ep_group("ep_opt", dist.group.WORLD)
        E, K, H, special, toks, consts = _options_inputs(world)
        x, ids, wt, mask = toks[rank]
        gbs = world * max(t[0].shape[0] for t in toks)
        outs = ep.dispatch(OracleKernels, x, ids, "ep_opt", world, rank, E, 0, 1, mask=mask, special=special, global_bs=gbs)
        ex, ds, expand_idx, nums, ep_recv = outs[:5]
        y = (ex.float() * 2).to(torch.bfloat16)                      # a stand-in for the experts: every row doubled
        sp = {"expert_ids": ids, "E": E, "zero": 1, "copy": 1, "const": 1, "ori_x": x, "alpha_1": consts[0], "alpha_2": consts[1],
              "const_v": consts[2]}
        out = ep.combine(OracleKernels, y, ids, expand_idx, ep_recv, wt, "ep_opt", world, rank, E, mask=mask, special=sp)
        torch.save((out, ex, nums, ep_recv, expand_idx), os.path.join(outdir, f"rank{rank}.pt"))
        q.put((rank, "ok"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.parametrize("world", [2, 4])
def test_mask_special_experts_and_uneven_batches_over_gloo(world, tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_options_worker, args=(r, world, port, q, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for _ in range(world):
        item = q.get(timeout=180)
        assert item[1] == "ok", item[2]
    for p in procs:
        p.join(timeout=60)
    E, K, H, special, toks, consts = _options_inputs(world)
    xs, idl, wl, masks = zip(*toks)
    gbs = world * max(x.shape[0] for x in xs)
    disp = O.moe_distribute_dispatch(xs, idl, E, quant_mode=0, x_active_mask=masks, special_experts=special, global_bs=gbs)
    ys = [(d.expand_x.float() * 2).to(torch.bfloat16) for d in disp]
    sps = [{"ori_x": xs[r], "zero": 1, "copy": 1, "alpha_1": consts[0], "alpha_2": consts[1], "const_v": consts[2]} for r in range(world)]
    ref = O.moe_distribute_combine(ys, idl, disp, wl, E, None, masks, sps)
    for r in range(world):
        out, ex, nums, ep_recv, expand_idx = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        n_rows = int(disp[r].expert_token_nums.sum())
        assert ex.shape == disp[r].expand_x.shape and torch.equal(ex[:n_rows], disp[r].expand_x[:n_rows])
        assert torch.equal(nums, disp[r].expert_token_nums) and torch.equal(ep_recv, disp[r].ep_recv_count)
        assert torch.equal(expand_idx, disp[r].expand_idx)
        assert torch.equal(out, ref[r])

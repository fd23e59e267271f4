"""Expert parallelism on real GPUs: R ranks (one process per GPU, NCCL) against the oracle's simulated ranks.

Needs at least two visible GPUs; skipped otherwise.  No failure is injected here (host-side failure handling is
covered by the gloo tests on CPU).
"""
import os
import socket
import traceback

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, outdir, transport):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import torch.distributed as dist
        import torchair_b200
        from torchair_b200.layer import moe_layer
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        torchair_b200.register_ep_group("ep", dist.group.WORLD, transport=transport)
        results = {}
        for cfg_name, cfg in (("cfg0", O.CONFIGS["cfg0"]), ("skew", O.MoeConfig("skew", 96, 512, 16, 4, 256, zipf_s=1.2))):
            E_l = cfg.E // world
            w = O.make_weights(cfg, 0, experts=range(rank * E_l, (rank + 1) * E_l))
            x, ids, wt = O.make_tokens(cfg, 0, rank)
            xd, idd, wtd = x.to(dev), ids.to(dev), wt.to(dev)
            disp = torch.ops.npu.npu_moe_distribute_dispatch(xd, idd, "ep", world, rank, cfg.E, quant_mode=2)
            for fused in (True, False):
                out = moe_layer(xd, idd, wtd, w.w1.to(dev), w.s1.to(dev), w.w2.to(dev), w.s2.to(dev), group_ep="ep",
                                ep_world_size=world, ep_rank_id=rank, moe_expert_num=cfg.E, fused=fused)
                results[(cfg_name, fused)] = out.cpu()
            results[(cfg_name, "disp")] = [t.cpu() for t in disp]
        # the same layer through torch.compile: with the peer transport the whole expert-parallel layer is one CUDA graph
        from torchair_b200 import backend as _backend
        cfg = O.CONFIGS["cfg0"]
        E_l = cfg.E // world
        w = O.make_weights(cfg, 0, experts=range(rank * E_l, (rank + 1) * E_l))
        gw = [t.to(dev) for t in (w.w1, w.s1, w.w2, w.s2)]
        x, ids, wt = O.make_tokens(cfg, 0, rank)

        def fn(x, ids, wt, w1, s1, w2, s2):
            return moe_layer(x, ids, wt, w1, s1, w2, s2, group_ep="ep", ep_world_size=world, ep_rank_id=rank,
                             moe_expert_num=cfg.E, fused=False)
        config = torchair_b200.CompilerConfig()
        config.mode = "reduce-overhead"
        compiled = torch.compile(fn, backend=torchair_b200.get_npu_backend(compiler_config=config), fullgraph=True, dynamic=False)
        caps = _backend.counters["captures"]
        fdc = _backend.counters["fused_down_combine"]
        with torch.no_grad():
            for _ in range(3):
                out_c = compiled(x.to(dev), ids.to(dev), wt.to(dev), *gw)
        torch.cuda.synchronize(dev)
        results["compiled"] = out_c.cpu()
        results["captures"] = _backend.counters["captures"] - caps
        results["fused_down_combine"] = _backend.counters["fused_down_combine"] - fdc
        results["status"] = torchair_b200.gmm_status(dev)
        from torchair_b200 import ep as _ep
        results["peer_status"] = _ep.peer_status()
        if transport == "peer":
            # one exchange, two streams: the second stream's call arrives while the first one's work is still pending
            # (behind a 0.2 s device-side delay) and must be refused on the host, before anything is launched
            xd, idd = x.to(dev), ids.to(dev)
            side = torch.cuda.Stream(dev)
            torch.cuda.synchronize(dev)
            torch.cuda._sleep(400_000_000)
            torch.ops.npu.npu_moe_distribute_dispatch(xd, idd, "ep", world, rank, cfg.E, quant_mode=2)
            try:
                with torch.cuda.stream(side):
                    torch.ops.npu.npu_moe_distribute_dispatch(xd, idd, "ep", world, rank, cfg.E, quant_mode=2)
                results["two_streams"] = "accepted"
            except RuntimeError as exc:
                results["two_streams"] = str(exc)
            torch.cuda.synchronize(dev)
            results["peer_status_after"] = _ep.peer_status()
        torch.save(results, os.path.join(outdir, f"rank{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
        open(os.path.join(outdir, f"ok{rank}"), "w").write("ok")
    except Exception:
        open(os.path.join(outdir, f"err{rank}"), "w").write(traceback.format_exc())


@pytest.mark.parametrize("transport", ["peer", "nccl"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_layer_on_gpus_matches_oracle(world, transport, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path), transport)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
        if p.is_alive():
            p.kill()
    for r in range(world):
        err = os.path.join(str(tmp_path), f"err{r}")
        assert not os.path.exists(err), open(err).read()
        assert os.path.exists(os.path.join(str(tmp_path), f"ok{r}")), f"rank {r} did not finish"
    got = [torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)]
    for cfg_name, cfg in (("cfg0", O.CONFIGS["cfg0"]), ("skew", O.MoeConfig("skew", 96, 512, 16, 4, 256, zipf_s=1.2))):
        w = O.make_weights(cfg, 0)
        xs, idl, wl = zip(*[O.make_tokens(cfg, 0, r) for r in range(world)])
        collect = []
        ref = O.moe_layer(xs, idl, wl, w, collect)
        for r in range(world):
            assert got[r]["status"] == 0
            d = collect[r]["disp"]
            g = got[r][(cfg_name, "disp")]
            assert got[r]["peer_status"] == 0, "a peer-memory flag wait ran out of time"
            want_idx = d.expand_idx
            if transport == "peer":
                # the peer transport hands combine the slot position: owner rank * C + offset inside that owner's rows
                E_l = cfg.E // world
                C = cfg.T * min(E_l, cfg.K)
                sent = torch.bincount(idl[r].reshape(-1).long() // E_l, minlength=world)
                base = torch.cumsum(sent, 0) - sent
                owner = torch.bucketize(d.expand_idx.long(), torch.cumsum(sent, 0), right=True)
                want_idx = (owner * C + d.expand_idx.long() - base[owner]).to(torch.int32)
            n_rows = int(d.expert_token_nums.sum())         # rows past the received total are not written
            want = (d.expand_x[:n_rows], d.dynamic_scales[:n_rows], want_idx, d.expert_token_nums, d.ep_recv_count)
            have = (g[0][:n_rows], g[1][:n_rows], g[2], g[3], g[4])
            for a, b in zip(want, have):
                assert torch.equal(a, b), "dispatch outputs (int8 rows, scales, indices, counts) must be bit-exact"
            for fused in (True, False):
                assert torch.equal(got[r][(cfg_name, fused)], ref[r]), "the expert-parallel layer must equal the oracle bit for bit"
            # fused gate_up and (over peer memory) the down GEMM storing into the senders' buffers change no bit
            assert torch.equal(got[r][(cfg_name, True)], got[r][(cfg_name, False)])
            assert torch.equal(got[r][(cfg_name, True)], got[r][(cfg_name, False)])
            if transport == "peer":
                assert "two group names" in got[r]["two_streams"], got[r]["two_streams"]
                assert got[r]["peer_status_after"] == 0
            if cfg_name == "cfg0":
                assert torch.equal(got[r]["compiled"], got[r][(cfg_name, False)]), "compiled and eager layers must agree"
                assert got[r]["captures"] == (1 if transport == "peer" else 0)
                assert got[r]["fused_down_combine"] == (1 if transport == "peer" else 0)


def test_static_scratch_routing_on_a_second_device():
    """tab_moe_init_routing_static keeps one scratch array per GPU and looks its address up per device: the same call on
    cuda:1 (after cuda:0) must use that device's array and give the workspace entry point's results."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from tests.test_zz_no_alloc import _route
    g = torch.Generator().manual_seed(43)
    T, K, E, H = 1000, 4, 128, 128
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    row = torch.arange(T * K, dtype=torch.int32).view(K, T).t().contiguous()
    for index in (0, 1, 0):
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            want = _route("workspace", x.to(dev), row.to(dev), ids.to(dev), T, E)
            got = _route("static", x.to(dev), row.to(dev), ids.to(dev), T, E)
        for a, b in zip(want, got):
            assert torch.equal(a, b)


DECODE = O.MoeConfig("decode64", 128, 7168, 64, 8, 2048)     # the 8-GPU decode architecture at a quarter of its experts


def _decode_worker(rank, world, port, outdir, transport):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import torch.distributed as dist
        import torchair_b200
        from torchair_b200.layer import moe_layer
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        torchair_b200.register_ep_group("ep", dist.group.WORLD, transport=transport)
        cfg = DECODE
        E_l = cfg.E // world
        w = O.make_weights(cfg, 0, experts=range(rank * E_l, (rank + 1) * E_l))
        gw = [t.to(dev) for t in (w.w1, w.s1, w.w2, w.s2)]
        x, ids, wt = O.make_tokens(cfg, 0, rank)
        xd, idd, wtd = x.to(dev), ids.to(dev), wt.to(dev)
        results = {}
        for fused in (True, False):
            for rep in range(2):          # twice: flags, counters and buffers of the exchange are reused
                out = moe_layer(xd, idd, wtd, *gw, group_ep="ep", ep_world_size=world, ep_rank_id=rank, moe_expert_num=cfg.E,
                                fused=fused)
            results[fused] = out.cpu()
        torchair_b200.check_status(dev)
        torch.save(results, os.path.join(outdir, f"rank{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
        open(os.path.join(outdir, f"ok{rank}"), "w").write("ok")
    except Exception:
        open(os.path.join(outdir, f"err{rank}"), "w").write(traceback.format_exc())


@pytest.mark.parametrize("transport", ["peer", "nccl"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_decode_architecture_matches_oracle(world, transport, tmp_path):
    """Hidden 7168, intermediate 2048, top-8, 128 tokens per rank over 64 experts: the decode-orientation GEMM at its
    real K and channel counts with 32 / 16 / 8 experts per rank, and (peer transport, fused) its epilogue storing rows
    into the other GPUs' buffers -- against the oracle's simulated ranks, bit for bit."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_decode_worker, args=(r, world, port, str(tmp_path), transport)) for r in range(world)]
    for p in procs:
        p.start()
    cfg = DECODE
    w = O.make_weights(cfg, 0)                      # the oracle's side runs while the ranks work
    xs, idl, wl = zip(*[O.make_tokens(cfg, 0, r) for r in range(world)])
    ref = O.moe_layer(xs, idl, wl, w)
    for p in procs:
        p.join(timeout=900)
        if p.is_alive():
            p.kill()
    for r in range(world):
        err = os.path.join(str(tmp_path), f"err{r}")
        assert not os.path.exists(err), open(err).read()
        assert os.path.exists(os.path.join(str(tmp_path), f"ok{r}")), f"rank {r} did not finish"
    for r in range(world):
        got = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        assert torch.equal(got[True], got[False]), "fused and unfused layers must agree"
        assert torch.equal(got[True], ref[r]), f"rank {r}: layer output differs from the oracle"

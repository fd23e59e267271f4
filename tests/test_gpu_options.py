"""GPU parity tests of the optional arguments around the path: token masks, smooth scales, special experts of the
second-generation dispatch / combine, an expert range and a row limit in npu_moe_init_routing_v2, the `finished` flag of
the gating operators, the int32 bias and the 16-bit scale of npu_grouped_matmul.  Everything is compared bit for bit
with the oracle (whose choices are marked "decision" there: the reference names these arguments without defining them).
"""
import pytest
import torch

import torchair_b200
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
npu = torch.ops.npu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _tokens(T, H, E, K, seed, extra_ids=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E + extra_ids, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    wt = torch.rand(T, K, generator=g)
    return x, ids, wt, g


@pytest.mark.parametrize("T,H,E,K", [(64, 1024, 8, 2), (700, 512, 32, 4)])      # sort inside the pack kernel / three sort kernels
@pytest.mark.parametrize("quant_mode", [2, 0])
def test_dispatch_with_token_mask(dev, T, H, E, K, quant_mode):
    x, ids, wt, g = _tokens(T, H, E, K, 5)
    mask = torch.rand(T, generator=g) < 0.7
    mask[0] = False
    d = O.moe_distribute_dispatch([x], [ids], E, quant_mode=quant_mode, x_active_mask=[mask])[0]
    got = npu.npu_moe_distribute_dispatch(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=quant_mode, x_active_mask=mask.to(dev))
    kept = int(d.expert_token_nums.sum())
    assert kept == int(mask.sum()) * K
    assert torch.equal(got[0].cpu()[:kept], d.expand_x[:kept]) and torch.equal(got[1].cpu()[:kept], d.dynamic_scales[:kept])
    assert torch.equal(got[2].cpu(), d.expand_idx) and torch.equal(got[3].cpu(), d.expert_token_nums)
    assert torch.equal(got[4].cpu(), d.ep_recv_count)
    # combine: rows of masked tokens are zero, the others the usual weighted sum
    y = torch.randn(T * K, H, generator=g).to(torch.bfloat16)
    ref = O.combine_rows(y, d.expand_idx.view(T, K), wt, ids, E, None, mask, None)
    out = npu.npu_moe_distribute_combine(y.to(dev), ids.to(dev), got[2], got[4], wt.to(dev), "", 1, 0, E, x_active_mask=mask.to(dev))
    assert torch.equal(out.cpu(), ref) and not out.cpu()[~mask].any()
    assert torchair_b200.routing_status(dev) == 0


@pytest.mark.parametrize("T,H,E,K,rows", [(64, 1024, 8, 2, 8), (600, 512, 16, 4, 1), (300, 20480, 8, 2, 8)])
def test_dispatch_with_smooth_scales(dev, T, H, E, K, rows):
    """`scales`: every copy is quantised on its own after the fp32 product with the smooth-scale row of its expert."""
    x, ids, wt, g = _tokens(T, H, E, K, 9)
    scales = torch.rand(rows, H, generator=g) + 0.5
    d = O.moe_distribute_dispatch([x], [ids], E, quant_mode=2, scales=scales if rows > 1 else scales.expand(E, H))[0]
    got = npu.npu_moe_distribute_dispatch(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=2, scales=scales.to(dev))
    assert torch.equal(got[0].cpu(), d.expand_x) and torch.equal(got[1].cpu(), d.dynamic_scales)
    assert torch.equal(got[2].cpu(), d.expand_idx) and torch.equal(got[3].cpu(), d.expert_token_nums)
    with pytest.raises(RuntimeError, match="quant_mode 2"):
        npu.npu_moe_distribute_dispatch(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=0, scales=scales.to(dev))


def test_global_bs_sizes_the_outputs_for_the_largest_rank(dev):
    T, H, E, K = 40, 256, 8, 2
    x, ids, wt, g = _tokens(T, H, E, K, 2)
    d = O.moe_distribute_dispatch([x], [ids], E, quant_mode=2, global_bs=64)[0]
    got = npu.npu_moe_distribute_dispatch(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=2, global_bs=64)
    assert got[0].shape == (64 * K, H) and d.expand_x.shape == (64 * K, H)
    assert torch.equal(got[0].cpu()[:T * K], d.expand_x[:T * K]) and torch.equal(got[3].cpu(), d.expert_token_nums)


@pytest.mark.parametrize("T,H,E,K", [(64, 1024, 8, 3), (900, 256, 16, 4)])
def test_special_experts_of_the_second_generation_ops(dev, T, H, E, K):
    """ids >= moe_expert_num name zero, copy and constant experts: dispatch_v2 does not send those pairs, combine_v2 forms
    their rows from ori_x and the constants; the whole single-rank layer then equals the oracle."""
    zero, copy, const = 1, 2, 2
    special = zero + copy + const
    x, ids, wt, g = _tokens(T, H, E, K, 21, extra_ids=special)
    a1 = torch.randn(const, H, generator=g).to(torch.bfloat16)
    a2 = torch.randn(const, H, generator=g).to(torch.bfloat16)
    cv = torch.randn(const, H, generator=g).to(torch.bfloat16)
    d = O.moe_distribute_dispatch([x], [ids], E, quant_mode=2, special_experts=special)[0]
    got = npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=2, zero_expert_num=zero,
                                             copy_expert_num=copy, const_expert_num=const)
    kept = int(d.expert_token_nums.sum())
    assert 0 < kept < T * K
    assert torch.equal(got[0].cpu()[:kept], d.expand_x[:kept]) and torch.equal(got[2].cpu(), d.expand_idx)
    assert torch.equal(got[3].cpu(), d.expert_token_nums)
    assert torchair_b200.routing_status(dev) == 0, "special expert ids are expected, not out of range"
    y = torch.randn(T * K, H, generator=g).to(torch.bfloat16)
    sp = {"ori_x": x, "zero": zero, "copy": copy, "alpha_1": a1, "alpha_2": a2, "const_v": cv}
    ref = O.combine_rows(y, d.expand_idx.view(T, K), wt, ids, E, None, None, sp)
    out = npu.npu_moe_distribute_combine_v2(y.to(dev), ids.to(dev), got[2], got[4], wt.to(dev), "", 1, 0, E, ori_x=x.to(dev),
                                            const_expert_alpha_1=a1.to(dev), const_expert_alpha_2=a2.to(dev),
                                            const_expert_v=cv.to(dev), zero_expert_num=zero, copy_expert_num=copy,
                                            const_expert_num=const)
    assert torch.equal(out.cpu(), ref)
    with pytest.raises(RuntimeError, match="ori_x"):
        npu.npu_moe_distribute_combine_v2(y.to(dev), ids.to(dev), got[2], got[4], wt.to(dev), "", 1, 0, E, copy_expert_num=1)
    # without special experts an id >= moe_expert_num is an error that the status word reports
    npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=2)
    assert torchair_b200.routing_status(dev) == 1


def test_elastic_and_performance_info_are_accepted_for_the_full_group(dev):
    T, H, E, K = 32, 256, 8, 2
    x, ids, wt, g = _tokens(T, H, E, K, 4)
    base = npu.npu_moe_distribute_dispatch(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=2)
    info = torch.zeros(4 + 2, dtype=torch.int32, device=dev)
    perf = torch.zeros(1, dtype=torch.int64, device=dev)
    got = npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=2, elastic_info=info, performance_info=perf)
    for a, b in zip(base, got):
        assert torch.equal(a, b)
    info[0] = 1
    with pytest.raises(NotImplementedError, match="elastic"):
        npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=2, elastic_info=info)
    with pytest.raises(RuntimeError, match="elastic_info"):
        npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, E, quant_mode=2, elastic_info=info[:3])


@pytest.mark.parametrize("T,K,E,H", [(300, 6, 64, 1024), (40, 4, 16, 256), (2000, 4, 64, 256)])
@pytest.mark.parametrize("quant_mode,row_type,active", [(-1, 1, 0), (1, 0, 0), (1, 1, 500), (-1, 0, 77)])
def test_init_routing_v2_expert_range_and_row_limit(dev, T, K, E, H, quant_mode, row_type, active):
    cfg = O.MoeConfig("v2", T, H, E, K, 128)
    x, ids, _ = O.make_tokens(cfg, seed=4)
    lo, hi = E // 4, E - E // 8
    ref = O.moe_init_routing_v2(x, ids, E, quant_mode, 1, row_type, active_expert_range=[lo, hi], active_num=active)
    got = npu.npu_moe_init_routing_v2(x.to(dev), ids.to(dev), expert_num=E, quant_mode=quant_mode, expert_tokens_num_type=1,
                                      expert_tokens_num_flag=True, row_idx_type=row_type, active_expert_range=[lo, hi],
                                      active_num=active)
    kept = int(ref[2].sum())
    rows = kept if active <= 0 else min(kept, active)
    assert got[2].shape == (hi - lo,) and torch.equal(got[2].cpu(), ref[2])
    assert got[0].shape[0] == (active if 0 < active < T * K else T * K)
    assert torch.equal(got[0].cpu()[:rows], ref[0][:rows]) and torch.equal(got[3].cpu()[:rows], ref[3][:rows])
    assert torch.equal(got[1].cpu(), ref[1])
    assert torchair_b200.routing_status(dev) == 0


@pytest.mark.parametrize("quant_mode", [-1, 1])
def test_init_routing_v2_scale_input(dev, quant_mode):
    T, K, E, H = 200, 4, 32, 512
    cfg = O.MoeConfig("v2", T, H, E, K, 128)
    x, ids, _ = O.make_tokens(cfg, seed=6)
    g = torch.Generator().manual_seed(8)
    scale = torch.rand(T, generator=g) if quant_mode == -1 else torch.rand(E, H, generator=g) + 0.5
    ref = O.moe_init_routing_v2(x, ids, E, quant_mode, 0, 1, scale=scale)
    got = npu.npu_moe_init_routing_v2(x.to(dev), ids.to(dev), scale=scale.to(dev), expert_num=E, quant_mode=quant_mode,
                                      expert_tokens_num_type=0, expert_tokens_num_flag=True, row_idx_type=1)
    for a, b in zip(ref, got):
        assert a.dtype == b.dtype and torch.equal(a, b.cpu())
    if quant_mode == 1:       # one smooth row for every expert
        ref1 = O.moe_init_routing_v2(x, ids, E, 1, 0, 1, scale=scale[:1])
        got1 = npu.npu_moe_init_routing_v2(x.to(dev), ids.to(dev), scale=scale[:1].to(dev), expert_num=E, quant_mode=1,
                                           expert_tokens_num_type=0, expert_tokens_num_flag=True, row_idx_type=1)
        assert torch.equal(ref1[0], got1[0].cpu()) and torch.equal(ref1[3], got1[3].cpu())


def test_gating_finished_rows_point_past_the_experts(dev):
    g = torch.Generator().manual_seed(12)
    T, E, k = 257, 64, 6
    x = torch.randn(T, E, generator=g)
    fin = torch.rand(T, generator=g) < 0.3
    y, ei, ri = O.moe_gating_top_k_softmax(x, k, fin)
    yg, eg, rg = npu.npu_moe_gating_top_k_softmax(x.to(dev), fin.to(dev), k)
    assert torch.equal(ei, eg.cpu()) and torch.equal(ri, rg.cpu()) and bool((eg.cpu()[fin] == E).all())
    torch.testing.assert_close(yg.cpu(), y, rtol=1e-5, atol=1e-7)
    y2, e2, _ = O.moe_gating_top_k_softmax_v2(x, k, 1, False, fin)
    yg2, eg2, _ = npu.npu_moe_gating_top_k_softmax_v2(x.to(dev), k=k, finished=fin.to(dev), renorm=1)
    assert torch.equal(e2, eg2.cpu())
    torch.testing.assert_close(yg2.cpu(), y2, rtol=1e-5, atol=1e-7)
    with pytest.raises(RuntimeError, match="finished"):
        npu.npu_moe_gating_top_k_softmax(x.to(dev), fin[:5].to(dev), k)


@pytest.mark.parametrize("M,Kd,N,E", [(96, 512, 384, 8), (1500, 256, 520, 3)])      # decode / prefill orientation
@pytest.mark.parametrize("out_dtype", [3, 15])
def test_grouped_matmul_int32_bias_and_16_bit_scale(dev, M, Kd, N, E, out_dtype):
    g = torch.Generator().manual_seed(M + N)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    bias = torch.randint(-100000, 100000, (E, N), generator=g, dtype=torch.int32)
    sc = (torch.rand(E, N, generator=g) * 9e-3 + 1e-3).to(torch.bfloat16)
    pts = torch.rand(M, generator=g) * 1e-2
    covered = M - M // 12
    cnt = torch.bincount(torch.randint(0, E, (covered,), generator=g), minlength=E)
    ref = O.grouped_matmul_w8a8(x, w, sc.float(), pts, cnt, 1, out_dtype, bias=bias)
    got = npu.npu_grouped_matmul([x.to(dev)], [w.to(dev)], bias=[bias.to(dev)], scale=[sc.to(dev)], per_token_scale=[pts.to(dev)],
                                 group_list=cnt.to(dev), split_item=2, group_type=0, group_list_type=1, output_dtype=out_dtype)[0]
    assert torchair_b200.gmm_status(dev) == 0
    assert torch.equal(ref[:covered], got.cpu()[:covered])
    with pytest.raises(NotImplementedError, match="int32"):
        npu.npu_grouped_matmul([x.to(dev)], [w.to(dev)], bias=[bias.float().to(dev)], group_list=cnt.to(dev), split_item=2,
                               group_type=0, group_list_type=1, output_dtype=3)

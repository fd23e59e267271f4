"""GPU parity tests: every CUDA path, called through torch.ops.npu.* -> ctypes -> C ABI, against the CPU oracle.

Bars: integer, byte and index outputs bit-exact, including the int8 values quantised after SwiGLU (the exp inside
SwiGLU is a fixed sequence of correctly rounded fp32 operations that the oracle restates, so CPU and GPU agree bit for
bit); fp32 scales within 1 ulp (they are in fact equal); bf16 layer outputs within rtol 1e-2 / atol 1e-2.
"""
import os

import pytest
import torch

import torchair_b200
from oracle import moe_oracle as O
from oracle.ep_standins import OracleKernels
from torchair_b200 import ep, ops
from torchair_b200.layer import moe_layer

pytestmark = pytest.mark.gpu
npu = torch.ops.npu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "cfg0_golden.pt")


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _ulp_equal(a, b, ulps=1):
    a, b = a.float().cpu(), b.float().cpu()
    return bool(((a.view(torch.int32) - b.view(torch.int32)).abs() <= ulps).all())


def _gmm_ok(dev):
    assert torchair_b200.gmm_status(dev) == 0, "a bounded wait inside the grouped GEMM gave up"


# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(64, 1024), (2048, 7168), (3, 16), (5, 24576), (2, 3, 512), (0, 64)])
def test_dynamic_quant_bit_exact(dev, dtype, shape):
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(*shape, generator=g) * 2).to(dtype)
    if x.numel():
        x.view(-1, shape[-1])[0] = 0            # an all-zero row: scale 0, q 0
    q, s = O.dynamic_quant(x)
    qg, sg = npu.npu_dynamic_quant(x.to(dev))
    assert qg.dtype == torch.int8 and sg.dtype == torch.float32 and sg.shape == x.shape[:-1]
    assert torch.equal(q, qg.cpu())
    assert _ulp_equal(s, sg) and torch.equal(s, sg.cpu())


def test_dynamic_quant_smooth_scales_and_unsupported_modes(dev):
    g = torch.Generator().manual_seed(12)
    x = torch.randn(130, 2048, generator=g).to(torch.bfloat16)
    sm = (torch.rand(2048, generator=g) + 0.5).to(torch.bfloat16)
    q, s = O.dynamic_quant(x, sm)
    qg, sg = npu.npu_dynamic_quant(x.to(dev), smooth_scales=sm.to(dev))
    assert torch.equal(q, qg.cpu()) and torch.equal(s, sg.cpu())
    with pytest.raises(NotImplementedError):
        npu.npu_dynamic_quant(x.to(dev), dst_type=16)
    with pytest.raises(NotImplementedError):
        npu.npu_dynamic_quant(x.to(dev), quant_mode="pergroup")
    with pytest.raises(RuntimeError, match="multiple of 16"):
        npu.npu_dynamic_quant(x[:, :24].to(dev))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_swiglu_bit_exact(dev, dtype):
    g = torch.Generator().manual_seed(13)
    x = (torch.randn(257, 4096, generator=g) * 3).to(dtype)
    x[0, :64] = torch.linspace(-100, 100, 64).to(dtype)          # through the cap of the exponent on both sides
    x[1, :4] = torch.tensor([0.0, -0.0, 80.0, -80.0]).to(dtype)
    ref = O.swiglu(x)
    got = npu.npu_swiglu(x.to(dev)).cpu()
    assert got.shape == (257, 2048) and got.dtype == dtype
    assert torch.equal(got.view(torch.int32 if dtype == torch.float32 else torch.int16),
                       ref.view(torch.int32 if dtype == torch.float32 else torch.int16))
    # and the deterministic form stays within rounding distance of the libm formula
    torch.testing.assert_close(got.float(), O.silu_mul(*torch.chunk(x.float(), 2, dim=-1), impl="libm").to(dtype).float(),
                               rtol=1e-2 if dtype != torch.float32 else 2e-6, atol=1e-6)


@pytest.mark.parametrize("T,K,E,H,active", [(3, 2, 4, 8, 3), (64, 2, 8, 1024, 64), (256, 8, 256, 7168, 256),
                                            (3000, 8, 256, 64, 3000), (100, 4, 1000, 32, 7), (1, 1, 1, 16, 1)])
def test_init_routing_bit_exact(dev, T, K, E, H, active):
    g = torch.Generator().manual_seed(T * 31 + K)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    row = torch.arange(T * K, dtype=torch.int32).view(K, T).t().contiguous()
    a = O.moe_init_routing(x, row, ids, active)
    b = npu.npu_moe_init_routing(x.to(dev), row.to(dev), ids.to(dev), active)
    for u, v in zip(a, b):
        assert u.shape == v.shape and torch.equal(u, v.cpu())
    xf = x.float()
    bf = npu.npu_moe_init_routing(xf.to(dev), row.to(dev), ids.to(dev), active)
    assert torch.equal(O.moe_init_routing(xf, row, ids, active)[0], bf[0].cpu())


@pytest.mark.parametrize("cfg_name,quant_mode,nums_type", [("cfg0", 2, 1), ("cfg0", 0, 0), ("cfg1", 2, 1)])
def test_single_rank_dispatch_bit_exact(dev, cfg_name, quant_mode, nums_type):
    cfg = O.CONFIGS[cfg_name]
    x, ids, wt = O.make_tokens(cfg, seed=3)
    d = O.moe_distribute_dispatch([x], [ids], cfg.E, quant_mode=quant_mode, expert_token_nums_type=nums_type)[0]
    g = npu.npu_moe_distribute_dispatch(x.to(dev), ids.to(dev), "", 1, 0, cfg.E, quant_mode=quant_mode,
                                        expert_token_nums_type=nums_type)
    want = (d.expand_x, d.dynamic_scales, d.expand_idx, d.expert_token_nums, d.ep_recv_count, d.tp_recv_count, d.expand_scales)
    for u, v in zip(want, g):
        assert u.dtype == v.dtype and torch.equal(u, v.cpu())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,K,H,shared", [(64, 2, 1024, False), (256, 8, 7168, True), (7, 3, 64, False)])
def test_single_rank_combine_bit_exact(dev, dtype, T, K, H, shared):
    g = torch.Generator().manual_seed(17)
    y = torch.randn(T * K, H, generator=g).to(dtype)
    pos = torch.randperm(T * K, generator=g).to(torch.int32).view(T, K)
    wt = torch.rand(T, K, generator=g)
    sh = torch.randn(T, H, generator=g).to(dtype) if shared else None
    ref = O.weighted_gather_sum(y, pos, wt, sh)
    ids = torch.zeros(T, K, dtype=torch.int32)
    got = npu.npu_moe_distribute_combine(y.to(dev), ids.to(dev), pos.reshape(-1).to(dev),
                                         torch.zeros(1, dtype=torch.int32, device=dev), wt.to(dev), "", 1, 0, 1,
                                         shared_expert_x=None if sh is None else sh.to(dev))
    assert torch.equal(ref, got.cpu())


@pytest.mark.parametrize("R,E_l,slot", [(2, 4, 0), (8, 32, 0), (4, 3, 0), (2, 4, 40), (1, 8, 0)])
def test_exchange_plan_and_rows_bit_exact(dev, R, E_l, slot):
    g = torch.Generator().manual_seed(R * 100 + E_l)
    counts = torch.randint(0, 6, (R, E_l), generator=g, dtype=torch.int32)
    counts[0, 0] = 0
    H = 64
    for nums_type in (0, 1):
        pc, nc, ec = OracleKernels.exchange_plan(counts, R, E_l, slot, nums_type)
        pg, ng, eg = ep.CudaKernels.exchange_plan(counts.to(dev), R, E_l, slot, nums_type)
        assert torch.equal(pc, pg.cpu()) and torch.equal(nc, ng.cpu()) and torch.equal(ec, eg.cpu())
    total = int(counts.sum())
    wire_rows = R * slot if slot else total
    wire = torch.randint(-127, 128, (wire_rows, H), generator=g, dtype=torch.int8)
    wsc = torch.rand(wire_rows, generator=g)
    A = total + 5
    dc, sc = OracleKernels.exchange_rows(wire, wsc, pc, R, E_l, slot, 0, A, True)
    dg, sg = ep.CudaKernels.exchange_rows(wire.to(dev), wsc.to(dev), pg, R, E_l, slot, 0, A, True)
    assert torch.equal(dc, dg.cpu()) and torch.equal(sc, sg.cpu())
    y = torch.randn(A, H, generator=g).to(torch.bfloat16)
    bc, _ = OracleKernels.exchange_rows(y, None, pc, R, E_l, slot, 1, wire_rows, True)
    bg, _ = ep.CudaKernels.exchange_rows(y.to(dev), None, pg, R, E_l, slot, 1, wire_rows, True)
    assert torch.equal(bc, bg.cpu())


# ---------------------------------------------------------------------------------------------------
GMM_SHAPES = [  # M, Kd, N, E
    (128, 1024, 1024, 8), (64, 512, 256, 4), (700, 1024, 384, 3), (2048, 2048, 512, 64), (5, 64, 128, 2),
    (1000, 1536, 640, 2), (33, 7168, 256, 16), (4096, 256, 128, 1),
    (40, 144, 72, 3), (300, 80, 200, 2),      # K ends inside a 128-byte block (zero-filled by TMA), channels not a multiple of 8
]


@pytest.mark.parametrize("M,Kd,N,E", GMM_SHAPES)
def test_grouped_matmul_int32_bit_exact(dev, M, Kd, N, E):
    g = torch.Generator().manual_seed(M + Kd + N + E)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    cnt = torch.bincount(torch.randint(0, E, (M,), generator=g), minlength=E)
    ref = O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)
    got = npu.npu_grouped_matmul([x.to(dev)], [w.to(dev)], group_list=cnt.to(dev), split_item=2, group_type=0,
                                 group_list_type=1, output_dtype=3)[0]
    _gmm_ok(dev)
    assert torch.equal(ref, got.cpu())
    got0 = npu.npu_grouped_matmul([x.to(dev)], [w.to(dev)], group_list=torch.cumsum(cnt, 0).to(dev), split_item=3,
                                  group_type=0, group_list_type=0, output_dtype=3)[0]
    assert torch.equal(ref, got0.cpu())


@pytest.mark.parametrize("out_dtype", [15, 5])
@pytest.mark.parametrize("M,Kd,N,E", [(300, 1024, 1024, 8), (2048, 2048, 7168, 32), (17, 512, 136, 3)])
def test_grouped_matmul_scaled_output(dev, out_dtype, M, Kd, N, E):
    g = torch.Generator().manual_seed(M + N)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    sc = torch.rand(E, N, generator=g) * 9e-3 + 1e-3
    pts = torch.rand(M, generator=g) * 1e-2
    covered = M - M // 10                         # the tail rows belong to no group: they are left unwritten
    cnt = torch.bincount(torch.randint(0, E, (covered,), generator=g), minlength=E)
    ref = O.grouped_matmul_w8a8(x, w, sc, pts, cnt, 1, out_dtype)
    got = npu.npu_grouped_matmul([x.to(dev)], [w.to(dev)], scale=[sc.to(dev)], per_token_scale=[pts.to(dev)],
                                 group_list=cnt.to(dev), split_item=2, group_type=0, group_list_type=1,
                                 output_dtype=out_dtype)[0]
    _gmm_ok(dev)
    assert got.dtype == O.SCALAR_TYPE[out_dtype]
    assert torch.equal(ref[:covered], got.cpu()[:covered]), "same fp32 operation order must give identical 16-bit results"


def test_grouped_matmul_skewed_and_empty_groups(dev):
    g = torch.Generator().manual_seed(99)
    M, Kd, N, E = 3000, 512, 256, 16
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    cnt = torch.tensor([0, 2500, 0, 1, 0, 0, 300, 17, 0, 0, 0, 100, 0, 0, 0, 82])
    ref = O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)
    got = npu.npu_grouped_matmul([x.to(dev)], [w.to(dev)], group_list=cnt.to(dev), split_item=2, group_type=0,
                                 group_list_type=1, output_dtype=3)[0]
    _gmm_ok(dev)
    assert torch.equal(ref, got.cpu())
    zero = npu.npu_grouped_matmul([x.to(dev)], [w.to(dev)], group_list=torch.zeros(E, dtype=torch.int64, device=dev),
                                  split_item=2, group_type=0, group_list_type=1, output_dtype=3)[0]
    _gmm_ok(dev)                 # all groups empty: no tile exists, nothing is written, nothing may wait forever
    assert zero.shape == (M, N)


def test_use_internal_format_weight_packs_expert_weights_ahead_of_the_first_run(dev):
    from torchair_b200 import ops
    ops.clear_weight_cache()
    m = torch.nn.Module()
    m.register_buffer("w1", torch.randint(-127, 128, (2, 64, 128), dtype=torch.int8, device=dev))
    m.register_buffer("other", torch.zeros(3, 3, device=dev))
    before = len(ops._packed_cache)
    torchair_b200.use_internal_format_weight(m)
    assert len(ops._packed_cache) == before + 1
    x = torch.randint(-127, 128, (16, 64), dtype=torch.int8, device=dev)
    cnt = torch.tensor([10, 6], device=dev)
    y = npu.npu_grouped_matmul([x], [m.w1], group_list=cnt, split_item=2, group_type=0, group_list_type=1, output_dtype=3)[0]
    assert len(ops._packed_cache) == before + 1                  # the GEMM found the packed form
    assert torch.equal(y.cpu(), O.grouped_matmul_w8a8(x.cpu(), m.w1.cpu(), None, None, cnt.cpu(), 1, 3))


def test_packed_weight_cache_follows_storage_lifetime_and_version(dev):
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-127, 128, (64, 256), generator=g, dtype=torch.int8).to(dev)
    cnt = torch.tensor([64], device=dev)

    def run(w):
        return npu.npu_grouped_matmul([x], [w], group_list=cnt, split_item=2, group_type=0, group_list_type=1, output_dtype=3)[0]
    for i in range(3):      # fresh weights that are likely to reuse the freed address must not hit a stale entry
        w = torch.randint(-127, 128, (1, 256, 128), generator=g, dtype=torch.int8).to(dev)
        assert torch.equal(run(w).cpu(), (x.cpu().int() @ w[0].cpu().int()))
        del w
    w = torch.randint(-127, 128, (1, 256, 128), generator=g, dtype=torch.int8).to(dev)
    run(w)
    w.neg_()                # in-place update bumps the version counter
    assert torch.equal(run(w).cpu(), (x.cpu().int() @ w[0].cpu().int()))


def _swiglu_quant_equal(q_gpu, s_gpu, q_ref, s_ref):
    assert torch.equal(q_gpu.cpu(), q_ref), "int8 values quantised after SwiGLU must be bit-exact"
    assert _ulp_equal(s_gpu, s_ref, ulps=1) and torch.equal(s_gpu.cpu(), s_ref)


@pytest.mark.parametrize("activate_left", [True, False])
def test_dequant_swiglu_quant_standalone(dev, activate_left):
    g = torch.Generator().manual_seed(23)
    M, N2, E = 300, 1024, 6
    acc = torch.randint(-2_000_000, 2_000_000, (M, N2), generator=g, dtype=torch.int32)
    ws = torch.rand(E, N2, generator=g) * 9e-3 + 1e-3
    a = torch.rand(M, generator=g) * 1e-3
    cnt = torch.tensor([50, 0, 100, 70, 30, 20])          # 270 of 300 rows
    q, s = O.dequant_swiglu_quant(acc, ws, a, cnt, activate_left, 1)
    qg, sg = npu.npu_dequant_swiglu_quant(acc.to(dev), weight_scale=ws.to(dev), activation_scale=a.to(dev),
                                          group_index=cnt.to(dev), activate_left=activate_left, quant_mode=1)
    _swiglu_quant_equal(qg, sg, q, s)
    assert int(qg[270:].abs().sum()) == 0 and float(sg[270:].abs().sum()) == 0
    # one weight-scale row for all rows, no groups
    q1, s1 = O.dequant_swiglu_quant(acc, ws[:1], a, None, activate_left, 1)
    qg1, sg1 = npu.npu_dequant_swiglu_quant(acc.to(dev), weight_scale=ws[:1].to(dev), activation_scale=a.view(-1, 1).to(dev),
                                            activate_left=activate_left, quant_mode=1)
    _swiglu_quant_equal(qg1, sg1, q1, s1)


@pytest.mark.parametrize("cfg_name", ["cfg0"])
def test_fused_gate_up_matches_unfused_and_oracle(dev, cfg_name):
    cfg = O.CONFIGS[cfg_name]
    w = O.make_weights(cfg, 0)
    x, ids, wt = O.make_tokens(cfg, 0)
    collect = []
    O.moe_layer([x], [ids], [wt], w, collect)
    c = collect[0]
    d = c["disp"]
    args = (d.expand_x.to(dev), [w.w1.to(dev)], [w.s1.to(dev)], d.dynamic_scales.to(dev), d.expert_token_nums.to(dev))
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(*args, group_list_type=1)
    _gmm_ok(dev)
    _swiglu_quant_equal(hq, hs, c["hq"], c["hs"])
    h32 = npu.npu_grouped_matmul([args[0]], args[1], group_list=args[4], split_item=2, group_type=0, group_list_type=1,
                                 output_dtype=3)[0]
    assert torch.equal(h32.cpu(), c["h32"])
    q2, s2 = npu.npu_dequant_swiglu_quant(h32, weight_scale=args[2][0], activation_scale=args[3], group_index=args[4],
                                          activate_left=True, quant_mode=1)
    assert torch.equal(q2, hq) and torch.equal(s2, hs), "fused and unfused GPU paths must agree bit for bit"


@pytest.mark.parametrize("M,Kd,I,E", [(128, 1024, 512, 8), (3000, 512, 256, 4), (700, 256, 136, 2)])
def test_fused_gate_up_fp32_values_and_quantiser_through_the_c_abi(dev, M, Kd, I, E):
    """tab_grouped_matmul_swiglu_quant with a caller workspace, so that the fp32 SwiGLU values and row maxima the
    kernel leaves there can be read back: (1) they equal the oracle's fp32 values bit for bit, (2) the oracle's
    quantiser applied to the GPU's own fp32 values reproduces the int8 output and the scales exactly.  Both GEMM
    orientations (a handful of rows per expert, hundreds of rows per expert)."""
    import ctypes
    from torchair_b200 import _lib
    g = torch.Generator().manual_seed(M + I)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, 2 * I), generator=g, dtype=torch.int8)
    ws = torch.rand(E, 2 * I, generator=g) * 9e-3 + 1e-3
    xs = torch.rand(M, generator=g) * 1e-2
    covered = M - M // 16
    cnt = torch.bincount(torch.randint(0, E, (covered,), generator=g), minlength=E)
    xd, wd, wsd, xsd, cd = x.to(dev), w.to(dev), ws.to(dev), xs.to(dev), cnt.to(dev)
    wp = ops.packed_weight(wd)
    nbytes = _lib.workspace_bytes("tab_grouped_matmul_swiglu_quant_workspace_bytes", M, I)
    wsp = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    yq = torch.zeros((M, I), dtype=torch.int8, device=dev)
    ys = torch.zeros((M,), dtype=torch.float32, device=dev)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.call("tab_grouped_matmul_swiglu_quant", P(xd), P(wp), P(wsd), P(xsd), P(cd), 1, M, Kd, I, E, 1, P(yq), P(ys), P(wsp), nbytes, 0,
              ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _gmm_ok(dev)
    amax_bytes = (M * 4 + 255) // 256 * 256
    amax_gpu = wsp[:M * 4].view(torch.float32).cpu()
    h_gpu = wsp[amax_bytes:amax_bytes + M * I * 4].view(torch.float32).view(M, I).cpu()
    h32 = O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)
    h_ref = O.dequant_swiglu_f32(h32, ws, xs, cnt, True)
    assert torch.equal(h_gpu[:covered].view(torch.int32), h_ref[:covered].view(torch.int32)), "fp32 SwiGLU values must be bit-exact"
    assert torch.equal(amax_gpu[:covered], h_ref[:covered].abs().amax(dim=1))
    q_own, s_own = O.quantize_rows_f32(h_gpu[:covered])
    assert torch.equal(q_own, yq.cpu()[:covered]) and torch.equal(s_own, ys.cpu()[:covered]), \
        "the quantiser is bit-exact given the GPU's own fp32 inputs"
    q_ref, s_ref = O.dequant_swiglu_quant(h32, ws, xs, cnt, True, 1)
    _swiglu_quant_equal(yq[:covered], ys[:covered], q_ref[:covered], s_ref[:covered])


def test_layer_cfg0_against_oracle_and_golden(dev):
    cfg = O.CONFIGS["cfg0"]
    gold = torch.load(GOLDEN)
    w = O.make_weights(cfg, 0)
    x, ids, wt = O.make_tokens(cfg, 0)
    assert torch.equal(ids, gold["expert_ids"]) and torch.equal(wt, gold["expert_scales"])
    gw = [t.to(dev) for t in (w.w1, w.s1, w.w2, w.s2)]
    for fused in (True, False):
        out = moe_layer(x.to(dev), ids.to(dev), wt.to(dev), *gw, fused=fused).cpu()
        _gmm_ok(dev)
        assert torch.equal(out, gold["out"])
    d = npu.npu_moe_distribute_dispatch(x.to(dev), ids.to(dev), "", 1, 0, cfg.E, quant_mode=2)
    assert torch.equal(d[0].cpu(), gold["expand_x"]) and torch.equal(d[1].cpu(), gold["dynamic_scales"])
    assert torch.equal(d[2].cpu(), gold["expand_idx"]) and torch.equal(d[3].cpu(), gold["expert_token_nums"])
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(d[0], [gw[0]], [gw[1]], d[1], d[3], group_list_type=1)
    assert torch.equal(hq.cpu(), gold["hq"]) and torch.equal(hs.cpu(), gold["hs"])
    y = npu.npu_grouped_matmul([hq], [gw[2]], scale=[gw[3]], per_token_scale=[hs], group_list=d[3], split_item=2, group_type=0,
                               group_list_type=1, output_dtype=15)[0]
    out = npu.npu_moe_distribute_combine(y, ids.to(dev), d[2], d[4], wt.to(dev), "", 1, 0, cfg.E)
    assert torch.equal(out.cpu(), gold["out"]), "with bit-exact int8 activations the whole layer is bit-exact"


def test_layer_decode_shape_sampled_experts(dev):
    """Config-1 architecture at a reduced expert count (32 experts, 32 tokens: the same ~8 rows per expert)."""
    cfg = O.MoeConfig("cfg1_small", 32, 7168, 32, 8, 2048)
    w = O.make_weights(cfg, 1)
    x, ids, wt = O.make_tokens(cfg, 1)
    ref = O.moe_layer([x], [ids], [wt], w)[0]
    out = moe_layer(x.to(dev), ids.to(dev), wt.to(dev), w.w1.to(dev), w.s1.to(dev), w.w2.to(dev), w.s2.to(dev)).cpu()
    _gmm_ok(dev)
    assert torch.equal(out, ref)


def test_layer_prefill_shape_with_skew(dev):
    """Qwen3-shaped experts (H 4096 -> 512 here, I 1536) with Zipf routing: large, uneven groups, 256-token tiles."""
    cfg = O.MoeConfig("skew", 2048, 512, 16, 4, 1536, zipf_s=1.2)
    w = O.make_weights(cfg, 2)
    x, ids, wt = O.make_tokens(cfg, 2)
    ref = O.moe_layer([x], [ids], [wt], w)[0]
    out = moe_layer(x.to(dev), ids.to(dev), wt.to(dev), w.w1.to(dev), w.s1.to(dev), w.w2.to(dev), w.s2.to(dev)).cpu()
    _gmm_ok(dev)
    assert torch.equal(out, ref)


def test_full_size_decode_layer_properties(dev):
    """Config 1 at full size (256 experts, 11 GB of int8 weights generated on the device): checked through
    properties instead of a full CPU run -- sampled experts against the oracle, linearity in the routing weights,
    and zero output for zero weights."""
    cfg = O.CONFIGS["cfg1"]
    g = torch.Generator(device=dev).manual_seed(7)
    w1 = torch.randint(-127, 128, (cfg.E, cfg.H, 2 * cfg.I), generator=g, dtype=torch.int8, device=dev)
    w2 = torch.randint(-127, 128, (cfg.E, cfg.I, cfg.H), generator=g, dtype=torch.int8, device=dev)
    s1 = torch.rand(cfg.E, 2 * cfg.I, generator=g, device=dev) * 9e-3 + 1e-3
    s2 = torch.rand(cfg.E, cfg.H, generator=g, device=dev) * 9e-3 + 1e-3
    x, ids, wt = O.make_tokens(cfg, 0)
    xd, idd, wtd = x.to(dev), ids.to(dev), wt.to(dev)
    ex, xs, expand_idx, nums, ep_recv, _, _ = npu.npu_moe_distribute_dispatch(xd, idd, "", 1, 0, cfg.E, quant_mode=2)
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1)
    y = npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2, group_type=0,
                               group_list_type=1, output_dtype=15)[0]
    _gmm_ok(dev)
    starts = (torch.cumsum(nums, 0) - nums).cpu()
    for e in (0, 101, 255):
        s0, c = int(starts[e]), int(nums[e])
        if c == 0:
            continue
        we = O.MoeWeights(w1[e:e + 1].cpu(), s1[e:e + 1].cpu(), w2[e:e + 1].cpu(), s2[e:e + 1].cpu())
        col = {}
        yref = O.expert_ffn(ex[s0:s0 + c].cpu(), xs[s0:s0 + c].cpu(), torch.tensor([c]), we, col)
        _swiglu_quant_equal(hq[s0:s0 + c], hs[s0:s0 + c], col["hq"], col["hs"])
        assert torch.equal(y[s0:s0 + c].cpu(), yref)
    out = npu.npu_moe_distribute_combine(y, idd, expand_idx, ep_recv, wtd, "", 1, 0, cfg.E)
    out2 = npu.npu_moe_distribute_combine(y, idd, expand_idx, ep_recv, wtd * 2, "", 1, 0, cfg.E)
    torch.testing.assert_close(out2.float(), out.float() * 2, rtol=1e-2, atol=1e-2)
    out0 = npu.npu_moe_distribute_combine(y, idd, expand_idx, ep_recv, torch.zeros_like(wtd), "", 1, 0, cfg.E)
    assert float(out0.float().abs().sum()) == 0
    del w1, w2
    torchair_b200.clear_weight_cache()
    torch.cuda.empty_cache()


def test_torch_compile_backend_runs_the_ops_and_captures_a_cuda_graph(dev):
    from torchair_b200 import backend
    cfg = O.CONFIGS["cfg0"]
    w = O.make_weights(cfg, 0)
    x, ids, wt = O.make_tokens(cfg, 0)
    ref = O.moe_layer([x], [ids], [wt], w)[0]

    class Layer(torch.nn.Module):
        def __init__(self):
            super().__init__()
            for n, t in (("w1", w.w1), ("s1", w.s1), ("w2", w.w2), ("s2", w.s2)):
                self.register_buffer(n, t.to(dev))

        def forward(self, x, ids, wt):
            return moe_layer(x, ids, wt, self.w1, self.s1, self.w2, self.s2, fused=False)

    config = torchair_b200.CompilerConfig()
    config.mode = "reduce-overhead"
    fused_before, cap_before = backend.counters["fused_gate_up"], backend.counters["captures"]
    model = torch.compile(Layer(), backend=torchair_b200.get_npu_backend(compiler_config=config), fullgraph=True, dynamic=False)
    with torch.no_grad():
        for i in range(3):
            out = model(x.to(dev), ids.to(dev), wt.to(dev))
    _gmm_ok(dev)
    assert torch.equal(out.cpu(), ref)
    assert backend.counters["fused_gate_up"] == fused_before + 1, "the FX pass should fuse gate_up with its epilogue"
    assert backend.counters["captures"] == cap_before + 1 and backend.counters["replays"] >= 3


def test_shared_expert_on_a_second_stream_inside_one_cuda_graph(dev):
    """The documented use of npu_stream_switch: the shared expert's dense MLP on its own stream while the routed experts
    run on the main one, joined by npu_wait_tensor.  The compiled graph must give exactly the result of the same ops run
    one after the other, and must still be captured as one CUDA graph."""
    from torchair_b200 import backend, scope
    cfg = O.CONFIGS["cfg0"]
    w = O.make_weights(cfg, 0)
    x, ids, wt = O.make_tokens(cfg, 0)
    w1, s1, w2, s2 = (t.to(dev) for t in (w.w1, w.s1, w.w2, w.s2))

    def shared_expert(x):      # stands for the dense MLP; built from this library's deterministic kernels so that == holds
        q, s = torch.ops.npu.npu_dynamic_quant(torch.cat([x, x * 0.5], dim=-1))
        return torch.ops.npu.npu_swiglu((q.float() * s[:, None]).to(torch.bfloat16))

    def block(x, ids, wt, streams):
        if streams:
            with scope.npu_stream_switch("shared_expert", 1):
                shared = shared_expert(x)
        else:
            shared = shared_expert(x)
        routed = moe_layer(x, ids, wt, w1, s1, w2, s2)
        if streams:
            routed = scope.npu_wait_tensor(routed, shared)
        return routed + shared

    xd, idd, wtd = x.to(dev), ids.to(dev), wt.to(dev)
    want = block(xd, idd, wtd, False)
    config = torchair_b200.CompilerConfig()
    config.mode = "reduce-overhead"
    cap_before = backend.counters["captures"]
    model = torch.compile(lambda a, b, c: block(a, b, c, True), backend=torchair_b200.get_npu_backend(compiler_config=config),
                          fullgraph=True, dynamic=False)
    with torch.no_grad():
        for _ in range(3):
            out = model(xd, idd, wtd)
    torch.cuda.synchronize()
    _gmm_ok(dev)
    assert torch.equal(out, want)
    assert backend.counters["captures"] == cap_before + 1
    # eager replay of the same graph (no capture) takes the same streams
    config2 = torchair_b200.CompilerConfig()
    model2 = torch.compile(lambda a, b, c: block(a, b, c, True), backend=torchair_b200.get_npu_backend(compiler_config=config2),
                           fullgraph=True, dynamic=False)
    with torch.no_grad():
        out2 = model2(xd, idd, wtd)
    torch.cuda.synchronize()
    assert torch.equal(out2, want)


def test_quantiser_fast_path_is_exact_at_ties_and_extreme_scales(dev):
    """The quantiser approximates v/scale by v*(1/scale) and redoes the division only near rounding ties: rows built
    from exact ties (k + 0.5) * scale, denormal-scale rows and huge rows must still match IEEE division bit for bit."""
    g = torch.Generator().manual_seed(77)
    rows = []
    for s in (1.0, 3.0, 0.1, 1.0 / 3.0, 7e-3, 1e-38, 3e38 / 127):
        k = torch.arange(-127, 127, dtype=torch.float32) + 0.5
        r = torch.cat([k * s, torch.tensor([127.0 * s, -127.0 * s])])
        rows.append(r)
        rows.append(r * (1 + 2.0 ** -23))
        rows.append(r * (1 - 2.0 ** -23))
    x = torch.stack(rows)
    x = torch.cat([x, torch.randn(64, x.shape[1], generator=g) * 1e-3])
    q, s = O.dynamic_quant(x)
    qg, sg = npu.npu_dynamic_quant(x.to(dev))
    assert torch.equal(s, sg.cpu()) and torch.equal(q, qg.cpu())


def test_compute_expert_tokens_bit_exact(dev):
    g = torch.Generator().manual_seed(3)
    se = torch.sort(torch.randint(0, 300, (5000,), generator=g, dtype=torch.int32)).values
    for E in (256, 300, 400):
        assert torch.equal(O.moe_compute_expert_tokens(se.clamp(max=E - 1), E), npu.npu_moe_compute_expert_tokens(se.clamp(max=E - 1).to(dev), E).cpu())
    assert npu.npu_moe_compute_expert_tokens(torch.empty(0, dtype=torch.int32, device=dev), 4).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,k", [(256, 256, 8), (1000, 128, 8), (3, 4, 1), (17, 1000, 6)])
def test_gating_top_k_softmax(dev, dtype, T, E, k):
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, E, generator=g).to(dtype)
    y, ei, ri = O.moe_gating_top_k_softmax(x, k)
    yg, eg, rg = npu.npu_moe_gating_top_k_softmax(x.to(dev), None, k)
    assert torch.equal(ri, rg.cpu())
    # 16-bit logits repeat values, so ties are common there: equal probabilities may swap only if both are ties
    same = ei == eg.cpu()
    if dtype == torch.float32:
        assert bool(same.all()), "expert ids are index work: exact"
    else:
        assert float(same.float().mean()) > 0.999
    torch.testing.assert_close(yg.cpu().float(), y.float(), rtol=2e-2 if dtype != torch.float32 else 1e-5, atol=1e-7)
    y0, e0, r0 = npu.npu_moe_gating_top_k_softmax(x.to(dev), torch.zeros(T, dtype=torch.bool, device=dev), k)
    assert torch.equal(e0, eg) and torch.equal(y0, yg) and torch.equal(r0, rg)      # nothing finished: same outputs


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("with_extras", [False, True])
def test_finalize_routing_bit_exact(dev, dtype, with_extras):
    g = torch.Generator().manual_seed(9)
    T, K, H, E = 96, 4, 512, 16
    rows = torch.randn(T * K, H, generator=g).to(dtype)
    s2d = torch.randperm(T * K, generator=g).to(torch.int32)
    sc = torch.rand(T, K, generator=g)
    efr = torch.randint(0, E, (T, K), generator=g, dtype=torch.int32)
    skip1 = torch.randn(T, H, generator=g).to(dtype) if with_extras else None
    skip2 = torch.randn(T, H, generator=g).to(dtype) if with_extras else None
    bias = torch.randn(E, H, generator=g).to(dtype) if with_extras else None
    ref = O.moe_finalize_routing(rows, skip1, skip2, bias, sc, s2d, efr)
    d = lambda t: None if t is None else t.to(dev)
    got = npu.npu_moe_finalize_routing(d(rows), d(skip1), d(skip2), d(bias), d(sc), d(s2d), d(efr), 0)
    assert torch.equal(ref, got.cpu())


@pytest.mark.parametrize("quant_mode,tok_type,row_type", [(-1, 0, 0), (1, 1, 1), (1, 0, 0), (-1, 1, 1)])
def test_init_routing_v2_bit_exact(dev, quant_mode, tok_type, row_type):
    cfg = O.MoeConfig("v2", 300, 1024, 64, 6, 128)
    x, ids, _ = O.make_tokens(cfg, seed=4)
    ref = O.moe_init_routing_v2(x, ids, cfg.E, quant_mode, tok_type, row_type)
    got = npu.npu_moe_init_routing_v2(x.to(dev), ids.to(dev), expert_num=cfg.E, quant_mode=quant_mode,
                                      expert_tokens_num_type=tok_type, expert_tokens_num_flag=True, row_idx_type=row_type,
                                      active_expert_range=[0, cfg.E])
    for a, b in zip(ref, got):
        assert a.dtype == b.dtype and torch.equal(a, b.cpu())
    with pytest.raises(NotImplementedError):
        npu.npu_moe_init_routing_v2(x.to(dev), ids.to(dev), expert_num=cfg.E, drop_pad_mode=1)


@pytest.mark.parametrize("M,Kd,N,E,idx_dtype,extras,gl_type", [
    (256, 512, 1024, 8, torch.int64, True, 1),      # decode orientation, every optional input
    (2000, 256, 516, 4, torch.int32, False, 0),     # prefill orientation, cumulative group list, N % 8 != 0
    (640, 2048, 7168, 16, torch.int64, True, 1),    # the down projection's shape
])
def test_grouped_matmul_finalize_routing(dev, M, Kd, N, E, idx_dtype, extras, gl_type):
    """Down GEMM + logit-weighted scatter-add (+ shared rows): every term is exact fp32 of exact int32 accumulators, the
    only freedom is the order in which the K rows of a token are added, hence the fp32-ulp-sized tolerance."""
    g = torch.Generator().manual_seed(M + N)
    K = 4
    T = M // K
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    cuts = torch.sort(torch.randint(0, M - 7, (E - 1,), generator=g)).values      # the last 7 rows belong to no group
    ends = torch.cat([cuts, torch.tensor([M - 7])])
    counts = torch.diff(ends, prepend=torch.tensor([0]))
    group_list = (ends if gl_type == 0 else counts).to(torch.int64)
    scale = torch.rand(E, N, generator=g) * 1e-3 + 1e-4
    pts = torch.rand(M, generator=g) * 1e-2 + 1e-3
    row_index = (torch.randperm(M, generator=g) % T).to(idx_dtype)               # K rows per token
    kw = dict(scale=scale, pertoken_scale=pts, row_index=row_index, group_list_type=gl_type)
    out_bs = T
    if extras:
        out_bs = T + 5
        kw.update(bias=torch.randn(E, N, generator=g).to(torch.bfloat16), logit=torch.rand(M, generator=g),
                  shared_input=torch.randn(T // 2, N, generator=g).to(torch.bfloat16), shared_input_weight=0.75,
                  shared_input_offset=3)
        row_index[5] = -1            # out-of-range rows add nothing
        row_index[6] = out_bs
    ref = O.grouped_matmul_finalize_routing(x, w, group_list, output_bs=out_bs, **kw)
    d = lambda v: v.to(dev) if isinstance(v, torch.Tensor) else v
    got = npu.npu_grouped_matmul_finalize_routing(x.to(dev), w.to(dev), group_list.to(dev), output_bs=out_bs,
                                                  **{k: d(v) for k, v in kw.items()})
    _gmm_ok(dev)
    assert got.dtype == torch.float32 and got.shape == ref.shape
    torch.testing.assert_close(got.cpu(), ref, rtol=2e-6, atol=2e-6 * float(ref.abs().max()))
    if extras:     # rows no token points at and no shared row covers stay exactly zero
        untouched = torch.ones(out_bs, dtype=torch.bool)
        untouched[row_index[(row_index >= 0) & (row_index < out_bs)].long()] = False
        untouched[3:3 + T // 2] = False
        assert not got.cpu()[untouched].any()


def test_layer_from_gating_to_finalize_with_neighbour_ops(dev):
    """The single-rank layer written with the neighbouring ops: gating -> init_routing_v2 (quantising) ->
    fused gate_up -> down -> finalize_routing."""
    cfg = O.CONFIGS["cfg0"]
    w = O.make_weights(cfg, 0)
    x, _, _ = O.make_tokens(cfg, 0)
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(cfg.T, cfg.E, generator=g)
    probs, ids, _ = O.moe_gating_top_k_softmax(logits, cfg.K)
    ref = O.moe_layer([x], [ids], [probs], w)[0]
    pg, idg, _ = npu.npu_moe_gating_top_k_softmax(logits.to(dev), None, cfg.K)
    assert torch.equal(idg.cpu(), ids)
    ex, scatter_idx, counts, xs = npu.npu_moe_init_routing_v2(x.to(dev), idg, expert_num=cfg.E, quant_mode=1,
                                                             expert_tokens_num_type=1, expert_tokens_num_flag=True, row_idx_type=1)
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w.w1.to(dev)], [w.s1.to(dev)], xs, counts, group_list_type=1)
    y = npu.npu_grouped_matmul([hq], [w.w2.to(dev)], scale=[w.s2.to(dev)], per_token_scale=[hs], group_list=counts, split_item=2,
                               group_type=0, group_list_type=1, output_dtype=15)[0]
    # finalize wants src_to_dst indexed k*T + t; the scatter index is indexed t*K + k
    s2d = scatter_idx.view(cfg.T, cfg.K).t().contiguous().view(-1)
    out = npu.npu_moe_finalize_routing(y, None, None, None, pg, s2d, idg, 0)
    _gmm_ok(dev)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)


def test_quantiser_equals_ieee_division_on_a_large_sample(dev):
    """470 M values, bf16 and fp32 inputs: the branch-free quotient correction must reproduce rint(x / scale) of IEEE
    division everywhere (checked on the GPU against torch's own division)."""
    g = torch.Generator(device=dev).manual_seed(5)
    for dtype, rows in ((torch.bfloat16, 65536), (torch.float32, 16384)):
        x = (torch.randn(rows, 7168, generator=g, device=dev) * 3).to(dtype)
        q, s = npu.npu_dynamic_quant(x)
        xf = x.float()
        amax = xf.abs().amax(dim=1)
        want_s = amax / torch.full_like(amax, 127.0)     # tensor / tensor: IEEE division (a scalar divisor becomes a multiply)
        assert torch.equal(s, want_s)
        bad = 0
        for lo in range(0, rows, 8192):
            want_q = torch.round(xf[lo:lo + 8192] / want_s[lo:lo + 8192, None]).clamp_(-127, 127).to(torch.int8)
            bad += int((want_q != q[lo:lo + 8192]).sum())
        assert bad == 0


@pytest.mark.parametrize("M,Kd,I,E", [(3000, 512, 256, 4), (8192, 1024, 1536, 8), (700, 256, 136, 2)])
def test_fused_gate_up_prefill_orientation_equals_unfused(dev, M, Kd, I, E):
    """Experts with hundreds of rows take the prefill-orientation kernel (fp32 SwiGLU values + row amax, then the
    requantise pass): results must equal int32 GEMM + npu_dequant_swiglu_quant bit for bit."""
    g = torch.Generator().manual_seed(M + I)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8).to(dev)
    w = torch.randint(-127, 128, (E, Kd, 2 * I), generator=g, dtype=torch.int8).to(dev)
    ws = (torch.rand(E, 2 * I, generator=g) * 9e-3 + 1e-3).to(dev)
    xs = (torch.rand(M, generator=g) * 1e-2).to(dev)
    covered = M - 37
    cnt = torch.bincount(torch.randint(0, E, (covered,), generator=g), minlength=E).to(dev)
    for _ in range(2):      # twice: the row-amax scratch in the workspace must be reset by every call
        hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(x, [w], [ws], xs, cnt, group_list_type=1)
    _gmm_ok(dev)
    h32 = npu.npu_grouped_matmul([x], [w], group_list=cnt, split_item=2, group_type=0, group_list_type=1, output_dtype=3)[0]
    q2, s2 = npu.npu_dequant_swiglu_quant(h32, weight_scale=ws, activation_scale=xs, group_index=cnt, activate_left=True, quant_mode=1)
    assert torch.equal(hq[:covered], q2[:covered]) and torch.equal(hs[:covered], s2[:covered])
    ref32 = O.grouped_matmul_w8a8(x.cpu(), w.cpu(), None, None, cnt.cpu(), 1, 3)
    assert torch.equal(ref32[:covered], h32.cpu()[:covered])


@pytest.mark.parametrize("Kd,I", [(512, 256), (384, 200)])
def test_prefill_narrow_tail_tiles_are_bit_exact(dev, Kd, I):
    """Token tiles with at most 64 valid rows are computed with swapped operands (channels on the lanes, tokens on the
    columns).  Experts sized around every boundary of that path (1, 15..17, 47..49, 63..65 rows, the same as tails behind
    one and two full tiles, and an empty expert) must give the results of the wide tiles: raw int32, scaled bf16, and
    the fused SwiGLU + requantise epilogue."""
    counts = [1, 15, 16, 17, 47, 48, 49, 63, 64, 65, 0, 128 + 1, 128 + 33, 128 + 64, 128 + 65, 256 + 9, 256 + 127, 300]
    E = len(counts)
    M = sum(counts) + 11                       # 11 rows past the last group
    assert M > 64 * E                          # the prefill orientation is taken by itself
    g = torch.Generator().manual_seed(Kd + I)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, 2 * I), generator=g, dtype=torch.int8)
    ws = torch.rand(E, 2 * I, generator=g) * 9e-3 + 1e-3
    xs = torch.rand(M, generator=g) * 1e-2
    cnt = torch.tensor(counts, dtype=torch.int64)
    covered = sum(counts)
    xd, wd, wsd, xsd, cd = x.to(dev), w.to(dev), ws.to(dev), xs.to(dev), cnt.to(dev)
    h32 = npu.npu_grouped_matmul([xd], [wd], group_list=cd, split_item=2, group_type=0, group_list_type=1, output_dtype=3)[0]
    ref32 = O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)
    assert torch.equal(ref32[:covered], h32.cpu()[:covered])
    y16 = npu.npu_grouped_matmul([xd], [wd], scale=[wsd], per_token_scale=[xsd], group_list=cd, split_item=2, group_type=0,
                                 group_list_type=1, output_dtype=15)[0]
    ref16 = O.grouped_matmul_w8a8(x, w, ws, xs, cnt, 1, 15)
    assert torch.equal(ref16[:covered], y16.cpu()[:covered])
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(xd, [wd], [wsd], xsd, cd, group_list_type=1)
    q2, s2 = npu.npu_dequant_swiglu_quant(h32, weight_scale=wsd, activation_scale=xsd, group_index=cd, activate_left=True, quant_mode=1)
    _gmm_ok(dev)
    assert torch.equal(hq[:covered], q2[:covered]) and torch.equal(hs[:covered], s2[:covered])


def test_peer_flag_wait_runs_out_and_reports_instead_of_hanging(dev):
    """Failure detection on the GPU without faulting it: a flag that nobody sets makes the bounded wait of the
    peer-memory exchange give up (about 2 s), write its code into the status word and let the stream continue."""
    import ctypes
    import time
    from torchair_b200 import _lib
    R = 2
    flags = torch.zeros(R, dtype=torch.int64, device=dev)        # arrival counters that no peer will ever advance
    counter = torch.zeros(1, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    after = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    t0 = time.time()
    _lib.call("tab_ep_wait", P(flags), P(counter), R, 1, P(status), 123, stream)
    after.fill_(7)                                                # work queued behind the wait still runs
    torch.cuda.synchronize(dev)
    dt = time.time() - t0
    assert int(status.item()) == 123 and int(counter.item()) == 1 and int(after.item()) == 7
    assert 0.5 < dt < 30.0
    # an acknowledgement wait whose flags already hold the expected value returns at once
    status.zero_()
    flags.fill_(1)
    _lib.call("tab_ep_wait", P(flags), P(counter), R, 0, P(status), 124, stream)
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0 and int(counter.item()) == 2


@pytest.mark.parametrize("E,groups,k_group,k,mode,norm", [(256, 8, 4, 8, 1, 1), (256, 1, 1, 8, 0, 0), (128, 4, 2, 6, 0, 1),
                                                          (64, 8, 3, 4, 1, 0)])
def test_gating_top_k_group_limited(dev, E, groups, k_group, k, mode, norm):
    g = torch.Generator().manual_seed(E + k)
    T = 333
    x = torch.randn(T, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.1
    y, idx, sc = O.moe_gating_top_k(x, k, bias, k_group, groups, mode, norm, 2.5, 1e-20)
    yg, ig, sg = npu.npu_moe_gating_top_k(x.to(dev), k, bias=bias.to(dev), k_group=k_group, group_count=groups,
                                          group_select_mode=mode, norm_type=norm, out_flag=True, routed_scaling_factor=2.5)
    assert torch.equal(idx, ig.cpu()), "selected experts are index work: exact"
    torch.testing.assert_close(sg.cpu(), sc, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(yg.cpu(), y, rtol=1e-5, atol=1e-7)
    with pytest.raises(NotImplementedError):
        npu.npu_moe_gating_top_k(x.to(dev), k, renorm=1, norm_type=1)
    with pytest.raises(RuntimeError):
        npu.npu_moe_gating_top_k(x.to(dev), k, k_group=groups + 1, group_count=groups)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("renorm,full", [(0, True), (0, False), (1, False), (1, True)])
def test_gating_top_k_softmax_v2(dev, dtype, renorm, full):
    g = torch.Generator().manual_seed(17 + renorm)
    T, E, k = 515, 256, 8
    x = torch.randn(T, E, generator=g).to(dtype)
    y, ei, sm = O.moe_gating_top_k_softmax_v2(x, k, renorm, full)
    yg, eg, sg = npu.npu_moe_gating_top_k_softmax_v2(x.to(dev), k=k, renorm=renorm, output_softmax=full)
    same = ei == eg.cpu()
    if dtype == torch.float32:
        assert bool(same.all()), "expert ids are index work: exact"
    else:
        assert float(same.float().mean()) > 0.999     # 16-bit logits repeat values: equal probabilities may swap
    torch.testing.assert_close(yg.cpu().float(), y.float(), rtol=2e-2 if dtype != torch.float32 else 1e-5, atol=1e-7)
    assert sg.shape == sm.shape and sg.dtype == torch.float32
    if sm.numel():
        torch.testing.assert_close(sg.cpu(), sm, rtol=1e-5, atol=1e-7)
    if renorm:
        torch.testing.assert_close(yg.float().sum(-1).cpu(), torch.ones(T), rtol=0, atol=2e-2 if dtype != torch.float32 else 1e-5)
        # the renormalised form of the general gating operator is the same kernel path
        y2, e2, _ = npu.npu_moe_gating_top_k(x.to(dev), k, renorm=1, norm_type=0, eps=0.0)
        assert torch.equal(y2, yg) and torch.equal(e2, eg)


def test_second_generation_dispatch_combine_names(dev):
    cfg = O.CONFIGS["cfg0"]
    x, ids, wt = O.make_tokens(cfg, 0)
    a = npu.npu_moe_distribute_dispatch(x.to(dev), ids.to(dev), "", 1, 0, cfg.E, quant_mode=2)
    b = npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, cfg.E, quant_mode=2)
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    # y_dtype may restate the output type, comm_alg is a hint without effect
    c = npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, cfg.E, quant_mode=2, y_dtype=1, comm_alg="fullmesh")
    assert torch.equal(c[0], a[0])
    with pytest.raises(NotImplementedError):
        npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, cfg.E, quant_mode=2, y_dtype=15)
    # special experts declared but not used by any id: nothing changes
    z = npu.npu_moe_distribute_dispatch_v2(x.to(dev), ids.to(dev), "", 1, 0, cfg.E, quant_mode=2, zero_expert_num=1)
    for u, v in zip(a, z):
        assert torch.equal(u, v)
    y = torch.randn(cfg.T * cfg.K, cfg.H, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(dev)
    o1 = npu.npu_moe_distribute_combine(y, ids.to(dev), a[2], a[4], wt.to(dev), "", 1, 0, cfg.E)
    o2 = npu.npu_moe_distribute_combine_v2(y, ids.to(dev), b[2], b[4], wt.to(dev), "", 1, 0, cfg.E)
    assert torch.equal(o1, o2)
    o3 = npu.npu_moe_distribute_combine_v2(y, ids.to(dev), b[2], b[4], wt.to(dev), "", 1, 0, cfg.E, comm_alg="fullmesh")
    assert torch.equal(o1, o3)
    with pytest.raises(RuntimeError, match="ori_x"):      # copy experts need the tokens themselves
        npu.npu_moe_distribute_combine_v2(y, ids.to(dev), b[2], b[4], wt.to(dev), "", 1, 0, cfg.E, copy_expert_num=1)


def test_full_size_prefill_layer_properties(dev):
    """Config 4 at full size (4096 tokens, 128 experts, hidden 4096, intermediate 1536; 32768 rows through the
    prefill-orientation GEMM): sampled experts against the oracle, every row of a sampled expert, plus the permutation
    and count properties of the dispatch."""
    cfg = O.CONFIGS["cfg4"]
    g = torch.Generator(device=dev).manual_seed(11)
    w1 = torch.randint(-127, 128, (cfg.E, cfg.H, 2 * cfg.I), generator=g, dtype=torch.int8, device=dev)
    w2 = torch.randint(-127, 128, (cfg.E, cfg.I, cfg.H), generator=g, dtype=torch.int8, device=dev)
    s1 = torch.rand(cfg.E, 2 * cfg.I, generator=g, device=dev) * 9e-3 + 1e-3
    s2 = torch.rand(cfg.E, cfg.H, generator=g, device=dev) * 9e-3 + 1e-3
    x, ids, wt = O.make_tokens(cfg, 0)
    xd, idd, wtd = x.to(dev), ids.to(dev), wt.to(dev)
    ex, xs, expand_idx, nums, ep_recv, _, _ = npu.npu_moe_distribute_dispatch(xd, idd, "", 1, 0, cfg.E, quant_mode=2)
    M = cfg.T * cfg.K
    assert int(nums.sum()) == M and torch.equal(torch.sort(expand_idx).values.cpu(), torch.arange(M, dtype=torch.int32))
    assert torch.equal(nums.cpu(), torch.bincount(ids.reshape(-1).long(), minlength=cfg.E))
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1)
    y = npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2, group_type=0,
                               group_list_type=1, output_dtype=15)[0]
    _gmm_ok(dev)
    starts = (torch.cumsum(nums, 0) - nums).cpu()
    for e in (0, 63, 127):
        s0, c = int(starts[e]), int(nums[e])
        we = O.MoeWeights(w1[e:e + 1].cpu(), s1[e:e + 1].cpu(), w2[e:e + 1].cpu(), s2[e:e + 1].cpu())
        col = {}
        yref = O.expert_ffn(ex[s0:s0 + c].cpu(), xs[s0:s0 + c].cpu(), torch.tensor([c]), we, col)
        _swiglu_quant_equal(hq[s0:s0 + c], hs[s0:s0 + c], col["hq"], col["hs"])
        # the down GEMM on the GPU's own int8 activations must be exact
        yexact = O.grouped_matmul_w8a8(hq[s0:s0 + c].cpu(), we.w2, we.s2, hs[s0:s0 + c].cpu(), torch.tensor([c]), 1, 15)
        assert torch.equal(y[s0:s0 + c].cpu(), yexact)
        assert torch.equal(y[s0:s0 + c].cpu(), yref)
    out = npu.npu_moe_distribute_combine(y, idd, expand_idx, ep_recv, wtd, "", 1, 0, cfg.E)
    pos = expand_idx.view(cfg.T, cfg.K).cpu()
    ref_out = O.weighted_gather_sum(y.cpu(), pos, wt)
    assert torch.equal(out.cpu(), ref_out)
    del w1, w2
    torchair_b200.clear_weight_cache()
    torch.cuda.empty_cache()


def test_out_of_range_indices_are_reported_not_silently_clamped(dev):
    """An expert id equal to the number of experts, and a row_idx value past T*K: every access stays in range (ids are
    clamped, the bad row_idx is skipped), and the routing status word says so until it is read."""
    T, K, E, H = 64, 2, 8, 64
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    row = torch.arange(T * K, dtype=torch.int32).view(K, T).t().contiguous()
    assert torchair_b200.routing_status(dev) == 0
    npu.npu_moe_distribute_dispatch(x, ids.to(dev), "", 1, 0, E, quant_mode=2)
    assert torchair_b200.routing_status(dev) == 0
    bad = ids.clone()
    bad[5, 1] = E
    out = npu.npu_moe_distribute_dispatch(x, bad.to(dev), "", 1, 0, E, quant_mode=2)
    assert int(out[3].sum()) == T * K                      # the clamped pair still has a row (expert E-1)
    assert torchair_b200.routing_status(dev) == 1
    assert torchair_b200.routing_status(dev) == 0          # reading clears the word
    bad_row = row.clone()
    bad_row[7, 0] = T * K + 3
    npu.npu_moe_init_routing(x, bad_row.to(dev), ids.to(dev), T)
    with pytest.raises(RuntimeError, match="out of range"):
        torchair_b200.check_status(dev)
    assert torchair_b200.routing_status(dev) == 0


def test_scatter_gemm_skips_rows_without_a_destination(dev):
    """Row table of the scatter epilogue with null entries (rows the exchange plan does not cover): those rows are
    not stored, every other row lands at its address, nothing faults.  Both GEMM orientations and the CTA-pair kernel
    (its wide and narrow tiles)."""
    import ctypes
    from torchair_b200 import _lib
    for M, Kd, N, E, hint in ((96, 256, 512, 8, 0), (1200, 256, 264, 3, 0), (2600, 256, 264, 2, 2000)):
        g = torch.Generator().manual_seed(M)
        x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
        w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
        sc = torch.rand(E, N, generator=g) * 9e-3 + 1e-3
        pts = torch.rand(M, generator=g) * 1e-2
        cnt = torch.bincount(torch.randint(0, E, (M,), generator=g), minlength=E)
        ref = O.grouped_matmul_w8a8(x, w, sc, pts, cnt, 1, 15)
        out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=dev)
        perm = torch.randperm(M, generator=g)
        dst = out.data_ptr() + perm.to(torch.int64) * (N * 2)
        skipped = torch.zeros(M, dtype=torch.bool)
        skipped[::5] = True
        skipped[-40:] = True                               # e.g. a group list that covers more rows than the plan
        dst[skipped] = 0
        xd, sd, pd, cd, dd = x.to(dev), sc.to(dev), pts.to(dev), cnt.to(dev), dst.to(dev)
        wp = ops.packed_weight(w.to(dev))
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        _lib.call("tab_grouped_matmul_w8a8_scatter", P(xd), P(wp), P(sd), P(pd), P(cd), 1, M, Kd, N, E, 15, P(dd), hint,
                  ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        _gmm_ok(dev)
        got = out.cpu()
        keep = ~skipped
        assert torch.equal(got[perm[keep]], ref[keep])
        assert bool((got[perm[skipped]] == 7.0).all()), "rows with a null destination must stay untouched"


def test_swiglu_reciprocal_is_the_ieee_reciprocal_for_every_significand(dev):
    """SwiGLU divides through a reciprocal built from the hardware seed and one Newton step.  Its results are reproducible
    on a CPU only if that reciprocal is the correctly rounded one: checked exhaustively, all 2^23 significands, at the
    exponents that 1 + exp(-a) takes between its bounds (2^0 .. 2^115) and below."""
    import ctypes
    from torchair_b200 import _lib
    bad = torch.zeros(1, dtype=torch.int64, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for exponent in (0, 1, 2, 23, 24, 57, 100, 115, -3):
        _lib.call("tab_selftest_reciprocal", exponent, ctypes.c_void_p(bad.data_ptr()), stream)
    torch.cuda.synchronize(dev)
    assert int(bad.item()) == 0


@pytest.mark.parametrize("counts,Kd,N", [([3000, 1096], 256, 512), ([0, 2500, 3407], 384, 264), ([1025, 1, 2300], 144, 1024)])
def test_cta_pair_gemm_plain_outputs_are_bit_exact(dev, counts, Kd, N):
    """Experts that hold many rows run on CTA pairs (256-token x 256-channel tiles, tcgen05.mma.cta_group::2, each CTA
    loading half of the weight tile): raw int32, scaled bf16 with an int32 bias, and rows past the last group untouched.
    Counts are chosen to leave last tiles with one row, with 129 rows (one row in the second CTA) and an empty expert."""
    E, covered = len(counts), sum(counts)
    M = covered + 13
    g = torch.Generator().manual_seed(Kd + N)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    sc = torch.rand(E, N, generator=g) * 9e-3 + 1e-3
    pts = torch.rand(M, generator=g) * 1e-2
    bias = torch.randint(-50000, 50000, (E, N), generator=g, dtype=torch.int32)
    cnt = torch.tensor(counts, dtype=torch.int64)
    hint = [max(counts)]                      # the tiling hint that selects the pair kernel (>= 1024 rows per group at this K)
    xd, wd, cd = x.to(dev), w.to(dev), cnt.to(dev)
    h32 = npu.npu_grouped_matmul([xd], [wd], group_list=cd, split_item=2, group_type=0, group_list_type=1, output_dtype=3,
                                 tuning_config=hint)[0]
    _gmm_ok(dev)
    assert torch.equal(O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)[:covered], h32.cpu()[:covered])
    y = torch.full((M, N), 3.0, dtype=torch.bfloat16, device=dev)
    got = npu.npu_grouped_matmul([xd], [wd], bias=[bias.to(dev)], scale=[sc.to(dev)], per_token_scale=[pts.to(dev)], group_list=cd,
                                 split_item=2, group_type=0, group_list_type=1, output_dtype=15, tuning_config=hint)[0]
    _gmm_ok(dev)
    ref = O.grouped_matmul_w8a8(x, w, sc, pts, cnt, 1, 15, bias=bias)
    assert torch.equal(ref[:covered], got.cpu()[:covered])
    # the same through the kernel that takes one CTA per tile: the choice of kernel changes no bit
    one = npu.npu_grouped_matmul([xd], [wd], bias=[bias.to(dev)], scale=[sc.to(dev)], per_token_scale=[pts.to(dev)], group_list=cd,
                                 split_item=2, group_type=0, group_list_type=1, output_dtype=15, tuning_config=[300])[0]
    assert torch.equal(one[:covered], got[:covered])


@pytest.mark.parametrize("counts,Kd,I", [([3000, 1096], 512, 256), ([2049, 0, 2900], 256, 136), ([4096], 1024, 1536)])
def test_cta_pair_gemm_fused_gate_up_is_bit_exact(dev, counts, Kd, I):
    """gate_up + SwiGLU + requantise on CTA pairs (each CTA loads 64 gate and the matching 64 up channels of a tile)
    against the oracle and against the unfused pair of operators."""
    E, covered = len(counts), sum(counts)
    M = covered + 5
    g = torch.Generator().manual_seed(Kd + I)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, 2 * I), generator=g, dtype=torch.int8)
    ws = torch.rand(E, 2 * I, generator=g) * 9e-3 + 1e-3
    xs = torch.rand(M, generator=g) * 1e-2
    cnt = torch.tensor(counts, dtype=torch.int64)
    xd, wd, wsd, xsd, cd = x.to(dev), w.to(dev), ws.to(dev), xs.to(dev), cnt.to(dev)
    for _ in range(2):
        hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(xd, [wd], [wsd], xsd, cd, group_list_type=1, tuning_config=[max(counts)])
    _gmm_ok(dev)
    h32 = O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)
    q_ref, s_ref = O.dequant_swiglu_quant(h32, ws, xs, cnt, True, 1)
    _swiglu_quant_equal(hq[:covered], hs[:covered], q_ref[:covered], s_ref[:covered])
    hq1, hs1 = npu.npu_grouped_matmul_swiglu_quant_v2(xd, [wd], [wsd], xsd, cd, group_list_type=1, tuning_config=[300])
    assert torch.equal(hq1[:covered], hq[:covered]) and torch.equal(hs1[:covered], hs[:covered])


def test_weights_can_be_held_once_in_the_packed_layout(dev):
    """use_internal_format_weight(model, release_original=True) turns every int8 [E, K, N] expert weight into an [E, K, N]
    view of its K-major relayout: same values element for element, the grouped GEMM uses the buffer underneath without
    another relayout or a cache entry, and its results do not change by a bit."""
    import torchair_b200
    E, Kd, N, M = 4, 256, 384, 96
    g = torch.Generator().manual_seed(5)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    cnt = torch.tensor([20, 0, 50, 26], dtype=torch.int64)

    class Experts(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(w.to(dev), requires_grad=False)

    m = Experts()
    before = npu.npu_grouped_matmul([x.to(dev)], [m.w], group_list=cnt.to(dev), split_item=2, group_type=0, group_list_type=1,
                                    output_dtype=3)[0].cpu()
    old_ptr = m.w.data_ptr()
    torchair_b200.use_internal_format_weight(m, release_original=True)
    assert m.w.shape == (E, Kd, N) and m.w.stride() == (Kd * N, 1, Kd) and m.w.data_ptr() != old_ptr
    assert torch.equal(m.w.cpu(), w)                                         # the same tensor, element for element
    assert ops.packed_weight(m.w).data_ptr() == m.w.data_ptr() and len(ops._packed_cache) == 0
    after = npu.npu_grouped_matmul([x.to(dev)], [m.w], group_list=cnt.to(dev), split_item=2, group_type=0, group_list_type=1,
                                   output_dtype=3)[0].cpu()
    covered = int(cnt.sum())
    assert torch.equal(before[:covered], after[:covered])
    assert torch.equal(after[:covered], O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)[:covered])


_PAIR_TAILS = [256 + 16, 512 + 17, 256 + 33, 48, 64, 65 + 256, 256 + 63, 0, 9]


@pytest.mark.parametrize("Kd,N", [(256, 512), (144, 264)])
def test_cta_pair_narrow_tail_tiles_plain_are_bit_exact(dev, Kd, N):
    """On CTA pairs an expert's last tile with at most 64 rows is computed with the operands swapped (weights as the 256-row
    operand, 16..64 tokens as N, each CTA loading half of them).  Tails of 9, 16, 17, 33, 48, 63 and 64 rows take that form,
    65 rows the wide one; raw int32, scaled bf16 with bias, against the oracle and against the one-CTA kernel."""
    counts = _PAIR_TAILS
    E, covered = len(counts), sum(counts)
    M = covered + 11
    g = torch.Generator().manual_seed(Kd * 5 + N)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    sc = torch.rand(E, N, generator=g) * 9e-3 + 1e-3
    pts = torch.rand(M, generator=g) * 1e-2
    bias = torch.randint(-50000, 50000, (E, N), generator=g, dtype=torch.int32)
    cnt = torch.tensor(counts, dtype=torch.int64)
    xd, wd, cd = x.to(dev), w.to(dev), cnt.to(dev)
    hint = [2000]
    h32 = npu.npu_grouped_matmul([xd], [wd], group_list=cd, split_item=2, group_type=0, group_list_type=1, output_dtype=3,
                                 tuning_config=hint)[0]
    _gmm_ok(dev)
    assert torch.equal(O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)[:covered], h32.cpu()[:covered])
    for dt, code in ((torch.bfloat16, 15), (torch.float16, 5)):
        got = npu.npu_grouped_matmul([xd], [wd], bias=[bias.to(dev)], scale=[sc.to(dev)], per_token_scale=[pts.to(dev)], group_list=cd,
                                     split_item=2, group_type=0, group_list_type=1, output_dtype=code, tuning_config=hint)[0]
        _gmm_ok(dev)
        ref = O.grouped_matmul_w8a8(x, w, sc, pts, cnt, 1, code, bias=bias)
        assert torch.equal(ref[:covered], got.cpu()[:covered])
        one = npu.npu_grouped_matmul([xd], [wd], bias=[bias.to(dev)], scale=[sc.to(dev)], per_token_scale=[pts.to(dev)], group_list=cd,
                                     split_item=2, group_type=0, group_list_type=1, output_dtype=code, tuning_config=[100])[0]
        assert torch.equal(one[:covered], got[:covered])


@pytest.mark.parametrize("Kd,I,left", [(512, 256, True), (256, 136, True), (256, 192, False)])
def test_cta_pair_narrow_tail_tiles_fused_are_bit_exact(dev, Kd, I, left):
    """The fused gate_up on narrow pair tiles: a CTA's accumulator lanes hold 64 gate channels and the 64 matching up channels,
    the up warps hand their values to the gate warps through shared memory.  Against the oracle (both activation orders)
    and against the one-CTA kernel."""
    counts = _PAIR_TAILS
    E, covered = len(counts), sum(counts)
    M = covered + 5
    g = torch.Generator().manual_seed(Kd + 11 * I)
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, 2 * I), generator=g, dtype=torch.int8)
    ws = torch.rand(E, 2 * I, generator=g) * 9e-3 + 1e-3
    xs = torch.rand(M, generator=g) * 1e-2
    cnt = torch.tensor(counts, dtype=torch.int64)
    xd, wd, wsd, xsd, cd = x.to(dev), w.to(dev), ws.to(dev), xs.to(dev), cnt.to(dev)
    h32 = O.grouped_matmul_w8a8(x, w, None, None, cnt, 1, 3)
    if left:
        for _ in range(2):
            hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(xd, [wd], [wsd], xsd, cd, group_list_type=1, tuning_config=[2000])
        _gmm_ok(dev)
        q_ref, s_ref = O.dequant_swiglu_quant(h32, ws, xs, cnt, True, 1)
        _swiglu_quant_equal(hq[:covered], hs[:covered], q_ref[:covered], s_ref[:covered])
        hq1, hs1 = npu.npu_grouped_matmul_swiglu_quant_v2(xd, [wd], [wsd], xsd, cd, group_list_type=1, tuning_config=[100])
        assert torch.equal(hq1[:covered], hq[:covered]) and torch.equal(hs1[:covered], hs[:covered])
    else:
        # activate_left=False through the C entry point (the fused operator of the reference has no such argument)
        import ctypes
        from torchair_b200 import _lib
        wp = ops.packed_weight(wd)
        nbytes = _lib.workspace_bytes("tab_grouped_matmul_swiglu_quant_workspace_bytes", M, I)
        wsp = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        outs = []
        for hint in (2000, 100):
            yq = torch.zeros((M, I), dtype=torch.int8, device=dev)
            ys = torch.zeros((M,), dtype=torch.float32, device=dev)
            _lib.call("tab_grouped_matmul_swiglu_quant", P(xd), P(wp), P(wsd), P(xsd), P(cd), 1, M, Kd, I, E, 0, P(yq), P(ys), P(wsp),
                      nbytes, hint, ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
            _gmm_ok(dev)
            outs.append((yq.cpu(), ys.cpu()))
        q_ref, s_ref = O.dequant_swiglu_quant(h32, ws, xs, cnt, False, 1)
        _swiglu_quant_equal(outs[0][0][:covered], outs[0][1][:covered], q_ref[:covered], s_ref[:covered])
        assert torch.equal(outs[0][0][:covered], outs[1][0][:covered]) and torch.equal(outs[0][1][:covered], outs[1][1][:covered])


def test_combine_that_acknowledges_from_its_last_cta(dev):
    """tab_moe_combine_ack = the weighted sum of tab_moe_combine plus, once every CTA has read its rows, one release store of
    the next sequence number into each peer's flag slot.  One GPU stands for three peers here (three local flag words):
    same output, flags = counter + 1, the signal counter advanced, the arrival counter back at zero; twice in a row."""
    import ctypes
    from torchair_b200 import _lib
    T, K, H, M = 96, 4, 512, 400
    g = torch.Generator().manual_seed(3)
    rows = torch.randn(M, H, generator=g).to(torch.bfloat16).to(dev)
    idx = torch.randint(0, M, (T * K,), generator=g, dtype=torch.int32).to(dev)
    wts = torch.rand(T, K, generator=g).to(dev)
    want = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    _lib.call("tab_moe_combine", P(rows), 15, P(idx), P(wts), None, T, K, H, P(want), st)
    flags = torch.zeros(3, dtype=torch.int64, device=dev)
    table = torch.tensor([flags.data_ptr() + 8 * i for i in range(3)], dtype=torch.int64, device=dev)
    counters_ = torch.tensor([41, 0], dtype=torch.int64, device=dev)       # [signal counter, arrival counter (low 32 bits)]
    for step in (1, 2):
        got = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)
        _lib.call("tab_moe_combine_ack", P(rows), 15, P(idx), P(wts), None, T, K, H, P(got), None, None, 0, 0, 0, 0, None, None, None,
                  None, P(table), ctypes.c_void_p(counters_.data_ptr()), ctypes.c_void_p(counters_.data_ptr() + 8), 3, st)
        torch.cuda.synchronize(dev)
        assert torch.equal(got, want)
        assert flags.tolist() == [41 + step] * 3 and counters_.tolist() == [41 + step, 0]
    with pytest.raises(RuntimeError):       # no tokens: nothing would acknowledge
        _lib.call("tab_moe_combine_ack", P(rows), 15, P(idx), P(wts), None, 0, K, H, P(got), None, None, 0, 0, 0, 0, None, None, None,
                  None, P(table), ctypes.c_void_p(counters_.data_ptr()), ctypes.c_void_p(counters_.data_ptr() + 8), 3, st)


def test_combine_on_many_tokens_with_some_pairs_that_have_no_row(dev):
    """From 2048 tokens on, tab_moe_combine runs a lean kernel for the tokens whose pairs all have rows and a second pass for
    the others (a negative index contributes an exact zero).  Both kinds of token against the oracle, bit for bit, with
    and without the shared-expert rows."""
    import ctypes
    from torchair_b200 import _lib
    T, K, H, M = 2304, 4, 256, 5000
    g = torch.Generator().manual_seed(17)
    rows = torch.randn(M, H, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, M, (T, K), generator=g, dtype=torch.int32)
    drop = torch.rand(T, K, generator=g) < 0.02
    drop[5] = True                                    # one token without any row
    pos[drop] = -1
    wts = torch.rand(T, K, generator=g)
    shared = torch.randn(T, H, generator=g).to(torch.bfloat16)
    ids = torch.zeros(T, K, dtype=torch.int32)
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rd, pd, wd, sd = rows.to(dev), pos.to(dev), wts.to(dev), shared.to(dev)
    for sh_cpu, sh_dev in ((None, None), (shared, sd)):
        out = torch.full((T, H), 9.0, dtype=torch.bfloat16, device=dev)
        _lib.call("tab_moe_combine", P(rd), 15, P(pd), P(wd), P(sh_dev), T, K, H, P(out), st)
        want = O.combine_rows(rows, pos, wts, ids, 1, shared=sh_cpu)
        assert torch.equal(out.cpu(), want)
    assert int((drop.any(dim=1)).sum()) > 20 and int((~drop.any(dim=1)).sum()) > 1000


def test_full_size_skewed_prefill_share_on_cta_pairs(dev):
    """One rank's share of the skewed expert-parallel prefill at full size (8192 tokens top-8 over 32 experts with Zipf(1.2)
    routing, hidden 7168, intermediate 2048: 65536 rows, hundreds to thousands per expert) runs on CTA pairs.  The
    least-loaded expert in full and the first and last rows of the most-loaded one (its narrow or partial last tile
    included) against the oracle, bit for bit; dispatch permutation and counts; the combine over all rows."""
    cfg = O.MoeConfig("cfg3_rank", 8192, 7168, 32, 8, 2048, zipf_s=1.2)
    g = torch.Generator(device=dev).manual_seed(13)
    w1 = torch.randint(-127, 128, (cfg.E, cfg.H, 2 * cfg.I), generator=g, dtype=torch.int8, device=dev)
    w2 = torch.randint(-127, 128, (cfg.E, cfg.I, cfg.H), generator=g, dtype=torch.int8, device=dev)
    s1 = torch.rand(cfg.E, 2 * cfg.I, generator=g, device=dev) * 9e-3 + 1e-3
    s2 = torch.rand(cfg.E, cfg.H, generator=g, device=dev) * 9e-3 + 1e-3
    x, ids, wt = O.make_tokens(cfg, 0)
    xd, idd, wtd = x.to(dev), ids.to(dev), wt.to(dev)
    ex, xs, expand_idx, nums, ep_recv, _, _ = npu.npu_moe_distribute_dispatch(xd, idd, "", 1, 0, cfg.E, quant_mode=2)
    M = cfg.T * cfg.K
    assert int(nums.sum()) == M and torch.equal(torch.sort(expand_idx).values.cpu(), torch.arange(M, dtype=torch.int32))
    assert torch.equal(nums.cpu(), torch.bincount(ids.reshape(-1).long(), minlength=cfg.E))
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1)     # 2048 rows per expert on average
    y = npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2, group_type=0,
                               group_list_type=1, output_dtype=15)[0]
    _gmm_ok(dev)
    counts = nums.cpu()
    starts = torch.cumsum(counts, 0) - counts
    small, big = int(torch.argmin(counts)), int(torch.argmax(counts))
    assert int(counts[big]) > 4 * int(counts[small]) > 0            # the skew is there
    picks = [(small, torch.arange(int(counts[small])))]
    cb = int(counts[big])
    picks.append((big, torch.cat([torch.arange(48), torch.arange(cb - 80, cb)])))
    for e, rel in picks:
        rows_ = (int(starts[e]) + rel).to(dev)
        c = rel.numel()
        we = O.MoeWeights(w1[e:e + 1].cpu(), s1[e:e + 1].cpu(), w2[e:e + 1].cpu(), s2[e:e + 1].cpu())
        col = {}
        yref = O.expert_ffn(ex[rows_].cpu(), xs[rows_].cpu(), torch.tensor([c]), we, col)
        _swiglu_quant_equal(hq[rows_], hs[rows_], col["hq"], col["hs"])
        assert torch.equal(y[rows_].cpu(), yref)
    out = npu.npu_moe_distribute_combine(y, idd, expand_idx, ep_recv, wtd, "", 1, 0, cfg.E)
    ref_out = O.weighted_gather_sum(y.cpu(), expand_idx.view(cfg.T, cfg.K).cpu(), wt)
    assert torch.equal(out.cpu(), ref_out)
    del w1, w2
    torchair_b200.clear_weight_cache()
    torch.cuda.empty_cache()

"""CPU tests of the oracle: golden vectors, known answers and the properties the domain offers."""
import os

import pytest
import torch

from oracle import moe_oracle as O
from tests.golden.make_golden import build as build_golden, checksum

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "cfg0_golden.pt")


def _eq(a, b):
    if isinstance(a, dict):
        return set(a) == set(b) and all(_eq(a[k], b[k]) for k in a)
    if isinstance(a, (list, tuple)):
        return len(a) == len(b) and all(_eq(x, y) for x, y in zip(a, b))
    if isinstance(a, torch.Tensor):
        return a.dtype == b.dtype and torch.equal(a, b)
    return a == b


def test_oracle_matches_committed_golden_vectors():
    gold = torch.load(GOLDEN)
    now = build_golden()
    assert now["input_checksums"] == gold["input_checksums"], "seeded input stream changed"
    for k in gold:
        assert _eq(now[k], gold[k]), f"oracle output {k} differs from the committed golden vector"


def test_init_routing_known_answer():
    # shape of the reference's only declared case: x F32(3,4), row_idx/expert_idx I32(3,2), active_num=3
    # (python/torchair/_ge_concrete_graph/ge_converter/custom/moe_init_routing.py:4-8)
    x = torch.arange(12, dtype=torch.float32).view(3, 4)
    expert = torch.tensor([[1, 0], [0, 2], [1, 2]], dtype=torch.int32)
    row = torch.arange(6, dtype=torch.int32).view(2, 3).t().contiguous()      # value k*T + t
    ex, eri, eei = O.moe_init_routing(x, row, expert, 3)
    assert eei.tolist() == [0, 0, 1, 1, 2, 2]
    # sorted pairs (flat t*K+k): (0,1)->e0, (1,0)->e0, (0,0)->e1, (2,0)->e1, (1,1)->e2, (2,1)->e2
    assert torch.equal(ex, x[[0, 1, 0, 2, 1, 2]])
    # row_idx values of those pairs: 3, 1, 0, 2, 4, 5 -> inverse
    assert eri.tolist() == [2, 1, 3, 0, 4, 5]
    ex2, _, _ = O.moe_init_routing(x, row, expert, 2)
    assert ex2.shape == (4, 4) and torch.equal(ex2, ex[:4])


def test_dynamic_quant_known_answers_half_even_and_clamp():
    x = torch.tensor([[127.0, 63.5, 62.5, -0.5, -1.5, 2.5, 0.0, -127.0]])
    q, s = O.dynamic_quant(x)
    assert float(s) == 1.0
    assert q.tolist() == [[127, 64, 62, 0, -2, 2, 0, -127]]
    q0, s0 = O.dynamic_quant(torch.zeros(2, 16))
    assert float(s0.abs().sum()) == 0 and int(q0.abs().sum()) == 0
    x3 = torch.randn(2, 3, 32, dtype=torch.float32).to(torch.bfloat16)
    q3, s3 = O.dynamic_quant(x3)
    assert q3.shape == (2, 3, 32) and s3.shape == (2, 3) and q3.dtype == torch.int8 and s3.dtype == torch.float32


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_dynamic_quant_properties(dtype):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(257, 512, generator=g) * 3).to(dtype)
    q, s = O.dynamic_quant(x)
    assert int(q.abs().max()) <= 127
    assert bool((q.abs().amax(dim=1) == 127).all()), "the row maximum must map to +-127"
    err = (x.float() - q.float() * s[:, None]).abs()
    assert bool((err <= s[:, None] * 0.5 * (1 + 1e-5) + 1e-12).all())
    sm = torch.rand(512, generator=g).to(dtype)
    q2, s2 = O.dynamic_quant(x, sm)
    qa, sa = O.quantize_rows_f32(x.float() * sm.float())
    assert torch.equal(q2, qa) and torch.equal(s2, sa)


def test_swiglu_and_dequant_swiglu_quant_halves():
    x = torch.tensor([[1.0, -2.0, 3.0, 0.5]])
    y = O.swiglu(x)
    ref = torch.nn.functional.silu(torch.tensor([1.0, -2.0])) * torch.tensor([3.0, 0.5])
    assert torch.allclose(y, ref.view(1, 2))
    acc = torch.tensor([[100, -200, 300, 50]], dtype=torch.int32)
    ws = torch.tensor([0.01, 0.02, 0.03, 0.04])
    a = torch.tensor([0.5])
    left = O.dequant_swiglu_f32(acc, ws, a, None, True)
    right = O.dequant_swiglu_f32(acc, ws, a, None, False)
    v = acc.float() * 0.5 * ws
    assert torch.allclose(left, torch.nn.functional.silu(v[:, :2]) * v[:, 2:])
    assert torch.allclose(right, torch.nn.functional.silu(v[:, 2:]) * v[:, :2])
    q, s = O.dequant_swiglu_quant(acc, ws, a, None, True, 1)
    assert q.dtype == torch.int8 and q.shape == (1, 2) and s.shape == (1,)
    with pytest.raises(NotImplementedError):
        O.dequant_swiglu_quant(acc, ws, a, None, True, 0)


def test_grouped_matmul_group_list_types_and_uncovered_rows():
    g = torch.Generator().manual_seed(5)
    M, Kd, N, E = 37, 64, 48, 5
    x = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    counts = torch.tensor([5, 0, 12, 9, 4])                  # 30 of 37 rows covered
    y1 = O.grouped_matmul_w8a8(x, w, None, None, counts, 1, 3)
    y0 = O.grouped_matmul_w8a8(x, w, None, None, torch.cumsum(counts, 0), 0, 3)
    assert torch.equal(y0, y1)
    assert int(y1[30:].abs().sum()) == 0
    ref = (x[5:17].double() @ w[2].double()).to(torch.int32)
    assert torch.equal(y1[5:17], ref)
    sc, pts = torch.rand(E, N, generator=g), torch.rand(M, generator=g)
    yb = O.grouped_matmul_w8a8(x, w, sc, pts, counts, 1, 15)
    want = ((y1[17:26].float() * pts[17:26, None]) * sc[3][None]).to(torch.bfloat16)
    assert torch.equal(yb[17:26], want)


def test_dispatch_is_a_valid_permutation_and_counts_add_up():
    cfg = O.CONFIGS["cfg0"]
    x, ids, wt = O.make_tokens(cfg, seed=1)
    d = O.moe_distribute_dispatch([x], [ids], cfg.E)[0]
    M = cfg.T * cfg.K
    assert sorted(d.expand_idx.tolist()) == list(range(M))
    assert int(d.expert_token_nums.sum()) == M
    q, s = O.dynamic_quant(x)
    pos = d.expand_idx.view(cfg.T, cfg.K).long()
    for k in range(cfg.K):
        assert torch.equal(d.expand_x[pos[:, k]], q) and torch.equal(d.dynamic_scales[pos[:, k]], s)
    # rows are grouped by expert in ascending order
    sorted_e = torch.repeat_interleave(torch.arange(cfg.E), d.expert_token_nums)
    assert torch.equal(sorted_e[pos.reshape(-1)].to(torch.int32), ids.reshape(-1))


def test_dispatch_then_combine_with_identity_experts_is_weighted_sum():
    cfg = O.CONFIGS["cfg0"]
    for R in (1, 2, 4):
        xs, idl, wl = zip(*[O.make_tokens(cfg, 2, r) for r in range(R)])
        disp = O.moe_distribute_dispatch(xs, idl, cfg.E, quant_mode=0)
        ys = [d.expand_x for d in disp]
        outs = O.moe_distribute_combine(ys, idl, disp, wl, cfg.E)
        for r in range(R):
            acc = None
            for k in range(cfg.K):
                term = wl[r][:, k:k + 1] * xs[r].float()
                acc = term if acc is None else acc + term
            assert torch.equal(outs[r], acc.to(torch.bfloat16))


@pytest.mark.parametrize("R", [2, 4, 8])
def test_r_rank_layer_equals_one_rank_layer(R):
    cfg = O.CONFIGS["cfg0"]
    w = O.make_weights(cfg, seed=0)
    xs, idl, wl = zip(*[O.make_tokens(cfg, 0, r) for r in range(R)])
    multi = O.moe_layer(xs, idl, wl, w)
    for r in range(R):
        single = O.moe_layer([xs[r]], [idl[r]], [wl[r]], w)[0]
        assert torch.equal(single, multi[r])


def test_zipf_routing_is_skewed_and_gating_is_normalised():
    cfg = O.MoeConfig("skew", 512, 64, 64, 8, 32, zipf_s=1.2)
    _, ids, wt = O.make_tokens(cfg, seed=0)
    assert torch.allclose(wt.sum(1), torch.ones(cfg.T), atol=1e-5)
    assert all(len(set(r)) == cfg.K for r in ids.tolist()), "top-k experts of a token are distinct"
    hist = torch.bincount(ids.reshape(-1).long(), minlength=cfg.E).float()
    assert hist.max() / hist.mean() > 3.0
    _, ids_u, _ = O.make_tokens(O.MoeConfig("flat", 512, 64, 64, 8, 32), seed=0)
    hist_u = torch.bincount(ids_u.reshape(-1).long(), minlength=64).float()
    assert hist_u.max() / hist_u.mean() < 2.0


def test_checksum_is_order_sensitive():
    a = torch.arange(16, dtype=torch.int32)
    assert checksum(a) != checksum(a.flip(0))


def test_neighbour_ops_known_answers():
    se = torch.tensor([0, 0, 2, 2, 2, 5], dtype=torch.int32)
    assert O.moe_compute_expert_tokens(se, 6).tolist() == [2, 2, 5, 5, 5, 6]
    x = torch.tensor([[1.0, 3.0, 2.0, 3.0], [0.0, 0.0, 0.0, 0.0]])
    y, ei, ri = O.moe_gating_top_k_softmax(x, 2)
    assert ei.tolist() == [[1, 3], [0, 1]] and ri.tolist() == [[0, 2], [1, 3]]
    assert torch.allclose(y[1], torch.tensor([0.25, 0.25]))
    # finalize: T=2, K=2, rows indexed by src_to_dst[k*T+t]
    rows = torch.tensor([[1.0, 1.0], [2.0, 2.0], [3.0, 3.0], [4.0, 4.0]])
    s2d = torch.tensor([3, 0, 1, 2], dtype=torch.int32)       # (k=0: t0->3, t1->0), (k=1: t0->1, t1->2)
    sc = torch.tensor([[0.5, 2.0], [1.0, 1.0]])
    out = O.moe_finalize_routing(rows, None, None, None, sc, s2d, None)
    assert out.tolist() == [[0.5 * 4 + 2 * 2, 0.5 * 4 + 2 * 2], [1 + 3, 1 + 3]]
    bias = torch.tensor([[10.0, 10.0], [20.0, 20.0]])
    efr = torch.tensor([[0, 1], [1, 1]], dtype=torch.int32)
    skip = torch.ones(2, 2)
    out2 = O.moe_finalize_routing(rows, skip, None, bias, sc, s2d, efr)
    assert out2.tolist() == [[0.5 * 14 + 2 * 22 + 1] * 2, [21 + 23 + 1] * 2]
    xx = torch.arange(8, dtype=torch.float32).view(4, 2).to(torch.bfloat16)
    ids = torch.tensor([[1, 0], [0, 2], [2, 1], [0, 1]], dtype=torch.int32)
    ex, ridx, tok, es = O.moe_init_routing_v2(xx, ids, 3, -1, 1, 0)
    assert ridx.tolist() == [1, 2, 6, 0, 5, 7, 3, 4] and tok.tolist() == [3, 3, 2]
    assert torch.equal(ex, xx[[0, 1, 3, 0, 2, 3, 1, 2]])
    _, ridx1, tok0, _ = O.moe_init_routing_v2(xx, ids, 3, -1, 0, 1)
    assert tok0.tolist() == [3, 6, 8] and ridx1[ridx.long()].tolist() == list(range(8))


def test_gating_top_k_group_limited_known_answer():
    # 8 experts in 4 groups of 2; group scores (max): g0=.9 g1=.8 g2=.7 g3=.1 -> keep g0,g1; top-3 of {0,1,2,3}
    x = torch.logit(torch.tensor([[0.9, 0.2, 0.8, 0.5, 0.7, 0.6, 0.1, 0.05]]))
    y, idx, sc = O.moe_gating_top_k(x, 3, None, k_group=2, group_count=4, group_select_mode=0, norm_type=1)
    assert idx.tolist() == [[0, 2, 3]]
    assert torch.allclose(sc, torch.tensor([[0.9, 0.2, 0.8, 0.5, 0.7, 0.6, 0.1, 0.05]]), atol=1e-6)
    assert torch.allclose(y, torch.tensor([[0.9, 0.8, 0.5]]) / 2.2, atol=1e-6)
    # top-2 sums: g0=1.1 g1=1.3 g2=1.3 g3=.15 -> keep g1, g2 (tie keeps the lower group first; both kept)
    _, idx2, _ = O.moe_gating_top_k(x, 2, None, k_group=2, group_count=4, group_select_mode=1, norm_type=1)
    assert idx2.tolist() == [[2, 4]]
    # the bias steers the selection but not the returned score
    b = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 5.0, 0.0])
    y3, idx3, _ = O.moe_gating_top_k(x, 1, b, norm_type=1, routed_scaling_factor=2.0)
    assert idx3.tolist() == [[6]] and torch.allclose(y3, torch.tensor([[2.0]]), atol=1e-5)


def test_grouped_matmul_finalize_routing_known_answer_and_composition():
    """A hand-checkable case, then: with logit = routing weight and row_index = token, the op equals the fp32 down GEMM
    followed by the weighted sum over a token's rows."""
    x = torch.tensor([[1, 2], [3, 4], [5, 6], [7, 8]], dtype=torch.int8)
    w = torch.tensor([[[1, 0, 2, 0], [0, 1, 0, 2]], [[-1, 0, 1, 0], [0, -1, 0, 1]]], dtype=torch.int8)      # [2, 2, 4]
    y = O.grouped_matmul_finalize_routing(x, w, torch.tensor([1, 2]), scale=torch.full((2, 4), 0.5),
                                          pertoken_scale=torch.tensor([1.0, 2.0, 1.0, 9.0]), logit=torch.tensor([2.0, 1.0, 1.0, 1.0]),
                                          row_index=torch.tensor([1, 0, 0, 1]), shared_input=torch.ones(1, 4, dtype=torch.bfloat16),
                                          shared_input_weight=3.0, shared_input_offset=2, output_bs=3)
    # row 0 -> expert 0 -> out 1: 2 * 0.5 * [1, 2, 2, 4]; rows 1, 2 -> expert 1 -> out 0; row 3 is in no group
    assert torch.equal(y[1], torch.tensor([1.0, 2.0, 2.0, 4.0]))
    assert torch.equal(y[0], torch.tensor([-3.0, -4.0, 3.0, 4.0]) + 0.5 * torch.tensor([-5.0, -6.0, 5.0, 6.0]))
    assert torch.equal(y[2], torch.full((4,), 3.0))
    g = torch.Generator().manual_seed(2)
    M, Kd, N, E, K = 48, 32, 16, 3, 4
    xq = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    wq = torch.randint(-127, 128, (E, Kd, N), generator=g, dtype=torch.int8)
    counts = torch.tensor([20, 0, 28])
    sc, pts, lg = torch.rand(E, N, generator=g), torch.rand(M, generator=g), torch.rand(M, generator=g)
    tok = torch.randperm(M, generator=g) % (M // K)
    got = O.grouped_matmul_finalize_routing(xq, wq, counts, scale=sc, pertoken_scale=pts, logit=lg, row_index=tok, output_bs=M // K)
    starts, cnt = O.group_bounds(counts, 1)
    full = torch.zeros(M, N)
    for e in range(E):
        s, c = int(starts[e]), int(cnt[e])
        full[s:s + c] = (O.int8_matmul(xq[s:s + c], wq[e]).float() * pts[s:s + c, None]) * sc[e][None]
    want = torch.zeros(M // K, N).index_add_(0, tok, full * lg[:, None])
    torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-6)


# ---------------------------------------------------------------------------------------------------
# deterministic SwiGLU arithmetic
# ---------------------------------------------------------------------------------------------------
def _silu_inputs():
    g = torch.Generator().manual_seed(5)
    a = torch.cat([torch.randn(300_000, generator=g) * 5, torch.randn(50_000, generator=g) * 40, torch.linspace(-90, 90, 20001),
                   torch.tensor([0.0, -0.0, 80.0, -80.0, 81.0, -81.0, 1e4, -1e4, 1e-30, -1e-30, 0.34657359, -0.34657359])])
    b = torch.randn(a.numel(), generator=g)
    return a, b


def test_fma_emulation_is_correctly_rounded_on_hard_cases():
    """RN32(a*b + c) through fp64 with round-to-odd, checked against exact rational arithmetic; the first case is one
    where plain fp64 arithmetic double-rounds (the fp64 sum lands exactly on an fp32 tie that the true sum misses)."""
    import fractions
    u = 2.0 ** -23
    a = torch.tensor([2.0 ** -24 * (1 + u), 1.0 + u, 1.0 + u, 3.0, 1.0, -5.5], dtype=torch.float32)
    b = torch.tensor([1.0 - u, 1.0 + u, 1.0 - u, 1.0 / 3.0, 2.0 ** -24, 1.4426950216293335], dtype=torch.float32)
    c = torch.tensor([1.0 + u, 2.0 ** -70, -(2.0 ** -60), 2.0 ** -80, 1.0, 12582912.0], dtype=torch.float32)
    got = O._fma32(a, b, c)
    for i in range(a.numel()):
        exact = fractions.Fraction(float(a[i])) * fractions.Fraction(float(b[i])) + fractions.Fraction(float(c[i]))
        lo = torch.nextafter(got[i], torch.tensor(-float("inf")))
        hi = torch.nextafter(got[i], torch.tensor(float("inf")))
        d = abs(fractions.Fraction(float(got[i])) - exact)
        assert d <= abs(fractions.Fraction(float(lo)) - exact) and d <= abs(fractions.Fraction(float(hi)) - exact)
    assert float(got[0]) == 1.0 + u
    naive = (a[:1].double() * b[:1].double() + c[:1].double()).float()
    assert float(naive[0]) == 1.0 + 2 * u, "the first case is meant to be one that plain fp64 arithmetic gets wrong"
    assert float(got[4]) == 1.0                      # an exact tie rounds to even


def test_c_and_torch_restatements_of_the_swiglu_arithmetic_agree_bit_for_bit():
    if not O.build_c_oracle():
        pytest.skip("gcc is not available to build oracle/silu_exact.c")
    a, b = _silu_inputs()
    c = O.silu_mul(a, b, "exact")
    t = O.silu_mul(a, b, "exact_torch")
    assert torch.equal(c.view(torch.int32), t.view(torch.int32))


def test_deterministic_swiglu_stays_within_a_few_ulp_of_the_libm_formula():
    a, b = _silu_inputs()
    exact = O.silu_mul(a, b, "exact_torch")
    ref = a.double() / (1 + torch.exp(-a.double())) * b.double()
    near = a.abs() <= 20
    rel = (exact.double() - ref).abs() / ref.abs().clamp_min(1e-300)
    assert float(rel[near & (ref.abs() > 1e-30)].max()) < 6e-7
    libm = O.silu_mul(a, b, "libm")
    ulps = (exact.view(torch.int32) - libm.view(torch.int32)).abs()
    assert int(ulps[near].max()) <= 8 and float((ulps[near] > 2).float().mean()) < 0.03
    # far out the cap takes over: results are exactly a*b (1 + e == 1) or below 1e-30 in magnitude
    big = a >= 81
    assert torch.equal(exact[big], (a * b)[big])
    assert float(exact[a <= -81].abs().max()) < 1e-30 * float(b.abs().max()) * 1e4


def test_quantised_layer_barely_moves_between_the_two_swiglu_forms():
    cfg = O.CONFIGS["cfg0"]
    w = O.make_weights(cfg, 0)
    x, ids, wt = O.make_tokens(cfg, 0)
    a, b = [], []
    O.moe_layer([x], [ids], [wt], w, a)
    try:
        O.SILU_IMPL = "libm"
        O.moe_layer([x], [ids], [wt], w, b)
    finally:
        O.SILU_IMPL = "exact"
    dq = (a[0]["hq"].int() - b[0]["hq"].int()).abs()
    assert int(dq.max()) <= 1 and float((dq > 0).float().mean()) < 2e-3
    assert bool(((a[0]["hs"].view(torch.int32) - b[0]["hs"].view(torch.int32)).abs() <= 8).all())

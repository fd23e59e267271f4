"""Writes tests/golden/cfg0_golden.pt: outputs of the CPU oracle on the seeded config-0 inputs.

    python tests/golden/make_golden.py

The reference holds no golden vectors for this path (its kernels are closed binaries), so these fixtures pin the
oracle against accidental change and let the GPU tests run where the oracle's inputs are regenerated from seeds.
A checksum of the regenerated inputs is stored so that a drift in the random-number stream is detected.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import moe_oracle as O  # noqa: E402


def checksum(t: torch.Tensor) -> int:
    v = t.contiguous().view(torch.uint8).to(torch.int64)
    idx = torch.arange(v.numel(), dtype=torch.int64) % 65521 + 1
    return int((v.reshape(-1) * idx).sum() % (2 ** 61 - 1))


def build():
    cfg = O.CONFIGS["cfg0"]
    w = O.make_weights(cfg, seed=0)
    x, ids, wt = O.make_tokens(cfg, seed=0)
    collect = []
    out = O.moe_layer([x], [ids], [wt], w, collect)[0]
    c = collect[0]
    row_idx = torch.arange(cfg.T * cfg.K, dtype=torch.int32).view(cfg.K, cfg.T).t().contiguous()
    ex, eri, eei = O.moe_init_routing(x, row_idx, ids, cfg.T)
    # two simulated ranks on the same weights
    xs, idl, wl = [], [], []
    for r in range(2):
        a, b, c2 = O.make_tokens(cfg, 0, r)
        xs.append(a); idl.append(b); wl.append(c2)
    out2 = O.moe_layer(xs, idl, wl, w)
    return {
        "input_checksums": {"x": checksum(x), "ids": checksum(ids), "wt": checksum(wt), "w1": checksum(w.w1),
                            "s1": checksum(w.s1), "w2": checksum(w.w2), "s2": checksum(w.s2)},
        "expert_ids": ids, "expert_scales": wt,
        "expand_x": c["disp"].expand_x, "dynamic_scales": c["disp"].dynamic_scales, "expand_idx": c["disp"].expand_idx,
        "expert_token_nums": c["disp"].expert_token_nums,
        "h32_checksum": checksum(c["h32"]), "hq": c["hq"], "hs": c["hs"], "y_checksum": checksum(c["y"]), "out": out,
        "init_routing": {"expanded_x_checksum": checksum(ex), "expanded_row_idx": eri, "expanded_expert_idx": eei},
        "two_rank_out_checksums": [checksum(o) for o in out2],
    }


if __name__ == "__main__":
    torch.save(build(), os.path.join(HERE, "cfg0_golden.pt"))
    print("wrote cfg0_golden.pt", os.path.getsize(os.path.join(HERE, "cfg0_golden.pt")), "bytes")

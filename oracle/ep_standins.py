"""CPU stand-ins for the four device steps of expert-parallel dispatch/combine (TEST INFRASTRUCTURE).

Same call shapes as torchair_b200.ep.CudaKernels, written with the CPU oracle and plain loops.  Tests use them
(a) to drive the host-side exchange logic over gloo ranks on CPU and (b) as the checker for the CUDA pack /
permute / reduce kernels.  The shipped package never imports this module.
"""
import torch

from . import moe_oracle as O


class OracleKernels:
    @staticmethod
    def dispatch_pack(x, expert_ids, E, quant_mode, nums_type=None, mask=None, scales=None, special=0):
        T, K = expert_ids.shape
        flat = expert_ids.reshape(-1).to(torch.int64)
        keep = flat < E if special > 0 else torch.ones_like(flat, dtype=torch.bool)
        if mask is not None:
            keep = keep & mask.to(torch.bool).repeat_interleave(K)
        keys = torch.where(keep, flat.clamp(0, E - 1), torch.full_like(flat, E))
        order = torch.sort(keys, stable=True)
        kept = int(keep.sum())
        tok = (order.indices // K)[:kept]
        rows = torch.zeros(T * K, x.shape[1], dtype=torch.int8 if quant_mode == 2 else x.dtype)
        out_scales = torch.zeros(T * K, dtype=torch.float32)
        if quant_mode == 2 and scales is not None:
            sm = scales.float()
            srow = sm[order.values[:kept]] if sm.shape[0] > 1 else sm[:1].expand(kept, -1)
            rows[:kept], out_scales[:kept] = O.quantize_rows_f32(x[tok].float() * srow)
        elif quant_mode == 2:
            q, s = O.dynamic_quant(x)
            rows[:kept], out_scales[:kept] = q[tok], s[tok]
        else:
            rows[:kept] = x[tok]
        expand_idx = torch.full((T * K,), -1, dtype=torch.int32)
        expand_idx[order.indices[:kept]] = torch.arange(kept, dtype=torch.int32)
        counts = torch.bincount(keys, minlength=E + 1)[:E].to(torch.int32)
        nums = None
        if nums_type is not None:
            nums = counts.to(torch.int64) if nums_type == 1 else torch.cumsum(counts.to(torch.int64), 0)
        return rows, out_scales, expand_idx, counts, nums

    @staticmethod
    def exchange_plan(recv_counts, R, E_l, slot_rows, nums_type):
        c = recv_counts.reshape(R, E_l).to(torch.int64).clamp(min=0)
        wire = torch.zeros(R * E_l, dtype=torch.int64)
        run = 0
        for s in range(R):
            base = s * slot_rows if slot_rows > 0 else run
            off = 0
            for e in range(E_l):
                wire[s * E_l + e] = base + off
                off += int(c[s, e])
            run += off
        exp = torch.zeros(R * E_l + 1, dtype=torch.int64)
        run = 0
        for e in range(E_l):
            for s in range(R):
                exp[e * R + s] = run
                run += int(c[s, e])
        exp[R * E_l] = run
        plan = torch.cat([wire, exp]).to(torch.int32)
        per_e = c.sum(0)
        nums = per_e if nums_type == 1 else torch.cumsum(per_e, 0)
        ep_recv = c.t().contiguous().reshape(-1).to(torch.int32)
        return plan, nums.to(torch.int64), ep_recv

    @staticmethod
    def exchange_rows(src, src_scales, plan, R, E_l, slot_rows, direction, dst_rows, zero_fill):
        n = R * E_l
        wire, exp = plan[:n].tolist(), plan[n:].tolist()
        dst = torch.zeros(dst_rows, src.shape[1], dtype=src.dtype) if zero_fill else torch.empty(dst_rows, src.shape[1], dtype=src.dtype)
        dsc = None
        if src_scales is not None:
            dsc = torch.zeros(dst_rows, dtype=torch.float32)
        for e in range(E_l):
            for s in range(R):
                cnt = exp[e * R + s + 1] - exp[e * R + s]
                a, b = exp[e * R + s], wire[s * E_l + e]
                if direction == 0:
                    dst[a:a + cnt] = src[b:b + cnt]
                    if dsc is not None:
                        dsc[a:a + cnt] = src_scales[b:b + cnt]
                else:
                    dst[b:b + cnt] = src[a:a + cnt]
        return dst, dsc

    @staticmethod
    def combine(rows, expand_idx, expert_scales, shared, T, K, mask=None, special=None):
        if mask is None and special is None:
            return O.weighted_gather_sum(rows, expand_idx.reshape(T, K), expert_scales, shared)
        sp = None
        ids = torch.zeros(T, K, dtype=torch.int32)
        E = 1 << 30
        if special is not None:
            ids, E = special["expert_ids"], special["E"]
            sp = {"ori_x": special.get("ori_x"), "zero": special.get("zero", 0), "copy": special.get("copy", 0),
                  "alpha_1": special.get("alpha_1"), "alpha_2": special.get("alpha_2"), "const_v": special.get("const_v")}
        return O.combine_rows(rows, expand_idx.reshape(T, K), expert_scales, ids, E, shared, mask, sp)

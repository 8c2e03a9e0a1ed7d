"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run in a container that has the reference checked out (it is imported, never copied):

    PYTHONPATH=<reference root> PYTHONDONTWRITEBYTECODE=1 TORCHDYNAMO_DISABLE=1 \
        python tests/golden/make_golden.py

The reference has no tests or fixtures of its own, so these files pin the oracle
(oracle/dax_oracle.py) and, through it, the CUDA kernels to what the reference computes:
  quant_*.pt      dax.quant.nn.dynamic.functional.dynamic_quantize_to_{int8,fp8}
  weight_*.pt     dax.quant.nn.dynamic.Linear.from_float (observer + weight quantisation)
  linear_int8.pt  dax.quant.nn.dynamic.Linear.forward, INT8 branch, end to end on the CPU
  swap.pt         dax.quant.quantization.quantize_dynamic on a small module tree
  microbatch.pt   dax.parallel.patches.wanx2_1_t2v_opt.micro_batch_project_O_strategy
  layout.pt       the reshape/permute pairs around all_to_all_single in
                  dax.parallel.patches.wanx2_1_t2v_opt.layer (exchange emulated in-process)
  teacache.pt     dax.cache.teacache: skip decisions and accumulators over a synthetic schedule
Tensors are small (a few hundred KB in total).
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    import dax.quant.nn.dynamic.functional as dqf
    from dax.quant.nn.dynamic import Linear as RefLinear
    from dax.quant.qscheme import per_token_symmetric
    from dax.quant.quantization import quantize_dynamic
    from dax.quant.quantization.qconfig import (
        get_dynamic_fp8_per_token_act_per_channel_weight_qconfig as fp8_cfg,
        get_dynamic_int8_per_token_act_per_channel_weight_qconfig as int8_cfg,
    )

    torch.manual_seed(1234)
    g = torch.Generator().manual_seed(1234)

    # ---- activations: a mix of magnitudes, an all-zero row, a row whose bf16-rounded scale
    # rounds down (so that -128 is reachable), exact ties ----
    def acts(dtype):
        x = torch.randn(48, 256, generator=g) * torch.logspace(-3, 2, 48).unsqueeze(1)
        x[5] = 0.0
        x[6, :] = 0.5
        x[7, 0] = -300.0
        x[8] = torch.arange(256) - 128.0
        return x.to(dtype)

    for name, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        x = acts(dt)
        q, s = dqf.dynamic_quantize_to_int8(x, qscheme=per_token_symmetric)
        out = {"x": x, "q_int8": q, "s_int8": s}
        for fname, fdt in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
            qf, sf = dqf.dynamic_quantize_to_fp8(x, qscheme=per_token_symmetric, target_dtype=fdt)
            out["q_" + fname] = qf.view(torch.uint8)
            out["s_" + fname] = sf
        torch.save(out, os.path.join(HERE, f"quant_{name}.pt"))

    # ---- weights + INT8 linear forward ----
    lin = torch.nn.Linear(256, 192, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(192, 256, generator=g) * 0.02)
        lin.bias.copy_(torch.randn(192, generator=g) * 0.1)
    for name, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        m = torch.nn.Linear(256, 192, bias=True).to(dt)
        m.load_state_dict({k: v.to(dt) for k, v in lin.state_dict().items()})
        w = m.weight.detach().clone()
        b = m.bias.detach().clone()
        m.qconfig = int8_cfg()
        ql = RefLinear.from_float(m, reserve_float_weight=True)
        m2 = torch.nn.Linear(256, 192, bias=True).to(dt)
        m2.load_state_dict({k: v.to(dt) for k, v in lin.state_dict().items()})
        m2.qconfig = fp8_cfg(activation_dtype=torch.float8_e4m3fn)
        qf = RefLinear.from_float(m2, reserve_float_weight=True)
        torch.save({"w": w, "b": b, "qweight_int8": ql.qweight, "wscale_int8": ql.weight_scale,
                    "qweight_e4m3": qf.qweight.view(torch.uint8), "wscale_e4m3": qf.weight_scale,
                    "fp8_bias_dtype": str(qf.bias.dtype)},
                   os.path.join(HERE, f"weight_{name}.pt"))
        if name == "bf16":
            x = (torch.randn(2, 40, 256, generator=g) * 1.5).to(dt)
            with torch.no_grad():
                y = ql(x)
            torch.save({"x": x, "y": y}, os.path.join(HERE, "linear_int8.pt"))

    # ---- module swap ----
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.to_q = torch.nn.Linear(32, 32)
            self.proj_out = torch.nn.Linear(32, 8)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = torch.nn.ModuleList([Block(), Block()])
            self.condition_embedder = torch.nn.Sequential(torch.nn.Linear(32, 32))
            self.proj_out = torch.nn.Linear(32, 8)

    net = Net()
    quantize_dynamic(net, {"": int8_cfg(), "condition_embedder": None, "proj_out": None})
    torch.save({n: (type(m).__name__, hasattr(m, "qweight")) for n, m in net.named_modules()},
               os.path.join(HERE, "swap.pt"))

    # ---- micro-batch strategy + exchange layouts (P ranks emulated in-process) ----
    from dax.parallel.patches.wanx2_1_t2v_opt.layer import _generate_layout_params, post_all2all, pre_all2all_fun
    from dax.parallel.patches.wanx2_1_t2v_opt.micro_batch_layer import micro_batch_project_O_strategy

    t = torch.arange(1 * 48 * 2 * 4, dtype=torch.float32).reshape(1, 48, 2, 4)
    mbs = micro_batch_project_O_strategy(t, 2, 4)
    torch.save({"t": t, "mb": mbs}, os.path.join(HERE, "microbatch.pt"))

    P, s, H, d = 4, 6, 8, 4
    shards = [torch.randn(1, s, H, d, generator=g) for _ in range(P)]

    def exchange(inputs):  # all_to_all_single with equal splits over dim 0
        return [torch.cat([inputs[src][dst:dst + 1] for src in range(P)], dim=0) for dst in range(P)]

    pre = []
    for r in range(P):
        pi, ish, po, rsh = _generate_layout_params(2, 0, P, shards[r])
        pre.append(pre_all2all_fun(pi, ish, shards[r]))
    got = [post_all2all(po, rsh)(o) for o in exchange(pre)]            # [1, S, h, d] per rank
    pre2 = []
    for r in range(P):
        pi, ish, po2, rsh2 = _generate_layout_params(1, 0, P, got[r])
        pre2.append(pre_all2all_fun(pi, ish, got[r]))
    back = [post_all2all(po2, rsh2)(o) for o in exchange(pre2)]        # [1, s, H, d] per rank
    torch.save({"shards": shards, "tokens": got, "heads": back}, os.path.join(HERE, "layout.pt"))

    # ---- TeaCache: skip decisions over a synthetic 20-step CFG schedule (40 calls) ----
    import dax.cache.teacache as ref_tc

    class Dummy:
        enable_teacache = True
        cnt = 0
        teacache_thresh = 0.2
        use_ref_steps = True
        coefficients = [-3.03318725e05, 4.90537029e04, -2.65530556e03, 5.87365115e01, -3.15583525e-01]
        ret_steps = 5 * 2
        cutoff_steps = 20 * 2
        accumulated_rel_l1_distance_even = 0
        accumulated_rel_l1_distance_odd = 0
        previous_e0_even = None
        previous_e0_odd = None
        previous_residual_even = None
        previous_residual_odd = None

    d = Dummy()
    base = torch.randn(1, 6, 64, generator=g)
    drift = torch.randn(1, 6, 64, generator=g)
    inputs, skips, accs = [], [], []
    for step in range(20):
        for branch in range(2):
            tp = base + drift * (0.02 * step + 0.005 * branch) * (1.0 + 0.3 * torch.sin(torch.tensor(float(step))))
            inputs.append(tp)
            skips.append(bool(ref_tc.should_skip_forward_for_cached_states(d, timestep_proj=tp, temb=tp[:, 0])))
            accs.append((float(d.accumulated_rel_l1_distance_even), float(d.accumulated_rel_l1_distance_odd)))
    hs, orig = torch.randn(1, 5, 8, generator=g), torch.randn(5, 8, generator=g)
    d.is_even = True
    ref_tc.maybe_cache_states(d, hs, orig)
    torch.save({"inputs": inputs, "skips": skips, "accs": accs, "hs": hs, "orig": orig,
                "residual": d.previous_residual_even, "retrieved": ref_tc.retrieve_cached_states(d, orig)},
               os.path.join(HERE, "teacache.pt"))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    sys.exit(main())

"""TeaCache host logic against decisions recorded from the reference's own implementation
(tests/golden/teacache.pt, made by tests/golden/make_golden.py).  CPU only."""
import os

import torch

from dax_b200.cache import teacache


class Holder:
    pass


def fresh():
    class T(Holder):
        pass
    t = T()
    teacache.configure(t, teacache_thresh=0.2, num_inference_steps=20, use_ref_steps=True)
    return t


def test_skip_decisions_match_reference(golden_dir):
    g = torch.load(os.path.join(golden_dir, "teacache.pt"))
    t = fresh()
    assert t.ret_steps == 10 and t.cutoff_steps == 40
    for i, tp in enumerate(g["inputs"]):
        skip = teacache.should_skip_forward_for_cached_states(t, timestep_proj=tp, temb=tp[:, 0])
        assert skip == g["skips"][i], f"call {i}"
        acc = (float(t.accumulated_rel_l1_distance_even), float(t.accumulated_rel_l1_distance_odd))
        assert abs(acc[0] - g["accs"][i][0]) < 1e-9 and abs(acc[1] - g["accs"][i][1]) < 1e-9
    assert t.cnt == 40 and any(g["skips"]) and not all(g["skips"])


def test_residual_cache_and_reset(golden_dir):
    g = torch.load(os.path.join(golden_dir, "teacache.pt"))
    t = fresh()
    t.is_even = True
    teacache.maybe_cache_states(t, g["hs"], g["orig"])
    assert torch.equal(t.previous_residual_even, g["residual"])
    assert torch.equal(teacache.retrieve_cached_states(t, g["orig"]), g["retrieved"])
    t.cnt = 7
    holder = Holder()
    holder.transformer = t
    teacache.reset_cache(holder)
    assert t.cnt == 0 and t.previous_residual_even is None and t.previous_e0_odd is None


def test_disabled_never_skips():
    t = Holder()
    t.enable_teacache = False
    assert teacache.should_skip_forward_for_cached_states(t, timestep_proj=None, temb=None) is False


def test_temb_variant_windows():
    class T(Holder):
        pass
    t = T()
    teacache.configure(t, teacache_thresh=0.1, num_inference_steps=50, use_ref_steps=False)
    assert t.ret_steps == 2 and t.cutoff_steps == 98 and len(t.coefficients) == 5


# ---- the denoising loop that drives the cached forward (dax_b200/adapters/wan/sampling.py) ----------------
def test_flow_match_sigmas():
    from dax_b200.adapters.wan.sampling import flow_match_sigmas
    s = flow_match_sigmas(50, flow_shift=5.0)
    assert s.shape == (51,) and float(s[0]) == 1.0 and float(s[-1]) == 0.0
    assert torch.all(s[1:] < s[:-1])
    # the shift keeps more steps at high noise: the midpoint of the schedule sits well above 0.5
    assert float(s[25]) > 0.8
    plain = flow_match_sigmas(50, flow_shift=1.0)
    assert abs(float(plain[25]) - (1.0 - 25 * (1.0 - 1e-3) / 49)) < 1e-6


def test_denoise_loop_integrates_and_drives_the_cache():
    from dax_b200.adapters.wan.sampling import denoise

    class Stub(torch.nn.Module):
        """velocity = c for the prompt, c / 2 for the negative prompt; counts its calls like the cached DiT"""
        def __init__(self):
            super().__init__()
            self.calls = []

        def forward(self, x, t, ctx, return_dict=False):
            self.calls.append((float(t[0]), float(ctx.flatten()[0])))
            self.cnt += 1
            return (torch.full_like(x, 2.0 * float(ctx.flatten()[0])),)

    class Pipe:
        pass

    pipe = Pipe()
    pipe.transformer = Stub()
    pipe.transformer.cnt = 7  # stale counter of an earlier trajectory: the loop must reset it
    x0 = torch.zeros(1, 2, 1, 4, 4)
    pos, neg = torch.ones(1, 3, 8), torch.full((1, 3, 8), 0.5)
    seen = []
    out = denoise(pipe, x0, pos, neg, num_inference_steps=10, guidance_scale=5.0, flow_shift=3.0,
                  on_step=lambda i, x: seen.append(i))
    # v = v_u + g (v_c - v_u) = 1 + 5 * (2 - 1) = 6, integrated from sigma = 1 to 0: x = x0 - 6
    assert torch.allclose(out, torch.full_like(x0, -6.0), atol=1e-5)
    assert seen == list(range(10)) and pipe.transformer.cnt == 20
    # conditional first, then unconditional, at the same timestep; timesteps run from 1000 downwards
    assert [c[1] for c in pipe.transformer.calls[:4]] == [1.0, 0.5, 1.0, 0.5]
    assert pipe.transformer.calls[0][0] == 1000.0 and pipe.transformer.calls[0][0] == pipe.transformer.calls[1][0]
    ts = [c[0] for c in pipe.transformer.calls[::2]]
    assert all(a > b for a, b in zip(ts, ts[1:]))
    # without guidance: one forward per step
    pipe.transformer.calls.clear()
    denoise(pipe, x0, pos, None, num_inference_steps=4)
    assert len(pipe.transformer.calls) == 4


def test_planned_trajectory_gives_the_same_decisions(golden_dir):
    """The distances of a whole trajectory read back once (plan_trajectory) lead to the decisions and
    accumulators the per-forward host read produces, call for call (both guidance branches see the same
    timestep embedding, as in the denoising loop)."""
    g = torch.load(os.path.join(golden_dir, "teacache.pt"))
    per_step = g["inputs"][::2]
    calls = [tp for tp in per_step for _ in range(2)]
    lazy, planned = fresh(), fresh()
    it = iter(per_step)
    teacache.plan_trajectory(planned, range(len(per_step)), lambda _t: next(it), calls_per_step=2)
    skips = []
    for i, tp in enumerate(calls):
        a = teacache.should_skip_forward_for_cached_states(lazy, timestep_proj=tp, temb=tp[:, 0])
        b = teacache.should_skip_forward_for_cached_states(planned, timestep_proj=tp, temb=tp[:, 0])
        assert a == b, f"call {i}"
        skips.append(a)
        for name in ("accumulated_rel_l1_distance_even", "accumulated_rel_l1_distance_odd"):
            assert abs(float(getattr(lazy, name)) - float(getattr(planned, name))) < 1e-6
    assert any(skips) and not all(skips)
    holder = Holder()
    holder.transformer = planned
    teacache.reset_cache(holder)
    assert not hasattr(planned, "_rel_l1_plan")

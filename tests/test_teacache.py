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

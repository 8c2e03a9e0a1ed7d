"""TeaCache step skipping (counterpart of ``dax/cache/teacache.py``).

Host-side control around the DiT forward: successive denoising steps whose timestep embedding barely
moved reuse the residual (output minus input of the block stack) of the last computed step.  Calls
alternate between the conditional (even) and unconditional (odd) branch of classifier-free guidance,
each with its own accumulator and cached residual.  The accumulated quantity is a fixed polynomial of
the relative L1 change of the modulation input; a forward is skipped while it stays below the threshold,
never during the first ``ret_steps`` or from ``cutoff_steps`` on.

State lives on the transformer object under the reference's attribute names (``cnt``,
``accumulated_rel_l1_distance_even`` …) so that ``reset_cache`` and external tooling keep working."""
from __future__ import annotations

import numpy as np
import torch

_BRANCHES = ("even", "odd")


def _branch(self) -> str:
    return "even" if self.is_even else "odd"


def retrieve_cached_states(self, hidden_states: torch.Tensor) -> torch.Tensor:
    """Skipped step: input plus the cached residual of this branch."""
    return hidden_states + getattr(self, f"previous_residual_{_branch(self)}")


def maybe_cache_states(self, hidden_states: torch.Tensor, original_hidden_states: torch.Tensor) -> None:
    """Computed step: remember output minus input for this branch."""
    setattr(self, f"previous_residual_{_branch(self)}", hidden_states.squeeze(0) - original_hidden_states)


def should_skip_forward_for_cached_states(self, **kwargs) -> bool:
    if not getattr(self, "enable_teacache", False):
        return False
    inp = kwargs["timestep_proj"] if self.use_ref_steps else kwargs["temb"]
    self.is_even = self.cnt % 2 == 0
    b = _branch(self)
    acc_name, prev_name, calc_name = (f"accumulated_rel_l1_distance_{b}", f"previous_e0_{b}", f"should_calc_{b}")
    if self.cnt < self.ret_steps or self.cnt >= self.cutoff_steps:
        calc = True
        setattr(self, acc_name, 0)
    else:
        plan = getattr(self, "_rel_l1_plan", None)
        if plan is not None and self.cnt // plan["calls_per_step"] < len(plan["rel"]):
            # distances of the whole trajectory were read back once, before the loop: no device
            # synchronisation per forward
            rel = plan["rel"][self.cnt // plan["calls_per_step"]]
        else:
            prev = getattr(self, prev_name)
            assert prev is not None, f"{prev_name} is not initialized"
            # one host read per forward, as in the reference (the decision steers Python control flow)
            rel = float(((inp - prev).abs().mean() / prev.abs().mean()).cpu().item())
        acc = getattr(self, acc_name) + float(np.poly1d(self.coefficients)(rel))
        calc = acc >= self.teacache_thresh
        setattr(self, acc_name, 0 if calc else acc)
    setattr(self, calc_name, calc)
    setattr(self, prev_name, inp.clone())
    self.cnt += 1
    return not calc


@torch.no_grad()
def plan_trajectory(transformer, timesteps, embed, calls_per_step: int = 2) -> None:
    """Read the relative L1 distances of a whole denoising trajectory back in ONE device->host copy.

    The quantity the cache accumulates depends on the timestep embedding alone (never on the latents), so
    when the loop knows its timesteps in advance every decision can be prepared before the first forward.
    ``embed(t)`` returns the modulation input the decision looks at (``timestep_proj`` with ``use_ref_steps``,
    else ``temb``) for one timestep tensor; ``calls_per_step`` is 2 under classifier-free guidance (both
    branches see the same timestep).  ``should_skip_forward_for_cached_states`` then takes its distance from the
    plan instead of synchronising with the device at every forward; the per-forward read of the reference
    (``dax/cache/teacache.py:58-65``) stays as the path for callers that do not plan."""
    inps = torch.stack([embed(t).float() for t in timesteps], 0)
    flat = inps.flatten(1)
    rel = (flat[1:] - flat[:-1]).abs().mean(1) / flat[:-1].abs().mean(1)
    transformer._rel_l1_plan = {"rel": [0.0] + [float(v) for v in rel.cpu()], "calls_per_step": calls_per_step}


def reset_cache(pipe) -> None:
    t = pipe.transformer
    if hasattr(t, "_rel_l1_plan"):
        del t._rel_l1_plan
    if hasattr(t, "cnt"):
        t.cnt = 0
        for b in _BRANCHES:
            setattr(t, f"accumulated_rel_l1_distance_{b}", 0)
            setattr(t, f"previous_e0_{b}", None)
            setattr(t, f"previous_residual_{b}", None)


# polynomial coefficients and windows of the two variants the reference ships for Wan2.1-14B
# (dax/adapters/wan/transformer_adapter.py:196-219)
REF_STEPS_COEFFICIENTS = [-3.03318725e05, 4.90537029e04, -2.65530556e03, 5.87365115e01, -3.15583525e-01]
TEMB_COEFFICIENTS = [-5784.54975374, 5449.50911966, -1811.16591783, 256.27178429, -13.02252404]


def configure(transformer, teacache_thresh: float = 0.1, num_inference_steps: int = 50, use_ref_steps: bool = True) -> None:
    """Install the TeaCache state on the transformer's class, as the reference does."""
    cls = transformer.__class__
    cls.enable_teacache = True
    cls.cnt = 0
    cls.teacache_thresh = teacache_thresh
    cls.use_ref_steps = use_ref_steps
    for b in _BRANCHES:
        setattr(cls, f"accumulated_rel_l1_distance_{b}", 0)
        setattr(cls, f"previous_e0_{b}", None)
        setattr(cls, f"previous_residual_{b}", None)
    if use_ref_steps:
        cls.coefficients = list(REF_STEPS_COEFFICIENTS)
        cls.ret_steps = 5 * 2
        cls.cutoff_steps = num_inference_steps * 2
    else:
        cls.coefficients = list(TEMB_COEFFICIENTS)
        cls.ret_steps = 1 * 2
        cls.cutoff_steps = num_inference_steps * 2 - 2

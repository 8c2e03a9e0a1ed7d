"""A denoising loop around the optimised DiT forward.

The reference drives the transformer from the diffusers ``WanPipeline`` with a flow-prediction scheduler
(``examples/wan_t2v_example.py:107-118``: flow sigmas, ``flow_shift`` 5.0 for 720p and 3.0 for 480p) and with
classifier-free guidance, i.e. two transformer forwards per step, which is what the even/odd counters of the
step cache are for (``dax/cache/teacache.py:41-47``).  diffusers is not a dependency of this package, so the
loop here is the plain first-order (Euler) flow-matching update on the same sigma schedule: enough to run the
transformer, the sequence-parallel split/gather and the step cache through a whole trajectory on synthetic
inputs.  It is not a replacement for the pipeline's multistep solver.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ...cache import teacache


def flow_match_sigmas(num_steps: int, flow_shift: float = 5.0, num_train_timesteps: int = 1000) -> torch.Tensor:
    """``num_steps + 1`` noise levels from 1 to 0 with the resolution-dependent shift
    ``sigma' = shift * sigma / (1 + (shift - 1) * sigma)`` of flow-matching schedulers."""
    if num_steps < 1:
        raise ValueError("num_steps must be positive")
    sigma = torch.linspace(1.0, 1.0 / num_train_timesteps, num_steps, dtype=torch.float64)
    sigma = flow_shift * sigma / (1.0 + (flow_shift - 1.0) * sigma)
    return torch.cat([sigma, sigma.new_zeros(1)]).float()


@torch.no_grad()
def denoise(pipe, latents: torch.Tensor, prompt_embeds: torch.Tensor,
            negative_prompt_embeds: Optional[torch.Tensor] = None, num_inference_steps: int = 50,
            guidance_scale: float = 5.0, flow_shift: float = 5.0, num_train_timesteps: int = 1000,
            on_step: Optional[Callable[[int, torch.Tensor], None]] = None) -> torch.Tensor:
    """Integrate ``dx/dsigma = v(x, sigma)`` from pure noise to the sample with ``num_inference_steps`` Euler
    steps.  With ``negative_prompt_embeds`` and ``guidance_scale > 1`` every step runs the conditional and the
    unconditional forward (in that order, as the pipeline does) and combines them
    ``v = v_uncond + g * (v_cond - v_uncond)``.  The step cache installed by ``optimize_pipe(...,
    cache_strategy="teacache")`` is reset first and then decides per forward whether the block stack runs."""
    transformer = pipe.transformer
    teacache.reset_cache(pipe)
    sigmas = flow_match_sigmas(num_inference_steps, flow_shift, num_train_timesteps).to(latents.device)
    use_cfg = negative_prompt_embeds is not None and guidance_scale > 1.0
    x = latents
    steps = [(sigmas[i] * num_train_timesteps).reshape(1).expand(x.shape[0]) for i in range(num_inference_steps)]
    if getattr(transformer, "enable_teacache", False) and hasattr(transformer, "condition_embedder"):
        # the cache's decisions depend on the timestep embedding only: prepare them all with one host read
        def embed(t):
            temb, timestep_proj = transformer.condition_embedder(t, prompt_embeds, None)[:2]
            return timestep_proj.unflatten(1, (6, -1)) if transformer.use_ref_steps else temb
        teacache.plan_trajectory(transformer, steps, embed, calls_per_step=2 if use_cfg else 1)
    for i in range(num_inference_steps):
        t = steps[i]
        v = transformer(x, t, prompt_embeds, return_dict=False)[0]
        if use_cfg:
            v_u = transformer(x, t, negative_prompt_embeds, return_dict=False)[0]
            v = v_u + guidance_scale * (v - v_u)
        x = (x.float() + (sigmas[i + 1] - sigmas[i]) * v.float()).to(latents.dtype)
        if on_step is not None:
            on_step(i, x)
    return x

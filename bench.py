#!/usr/bin/env python
"""Benchmark of one Wan2.1-14B-shaped DiT denoising step at 720p / 81 frames (latents 16x21x90x160 ->
75,600 tokens on a 21x45x80 grid; 40 blocks, hidden 5120, 40 heads of 128, FFN 13,824, 512 text tokens;
FP8-e4m3 dynamic linears, INT8-QK / FP8-PV attention), Ulysses sequence parallel over N GPUs.

    --workload dit       (default) the whole DiT forward: patch embedding, condition embedder, 40 x
                         (self-attention block, cross-attention, FFN), output head
    --workload hotpath   only the 40 self-attention blocks (the hot path proper)

    python bench.py [--gpus N] [--steps K] [--warmup W]            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                            CPU arm: the reference's algorithm
                                                                    (oracle port) on the host cores

One "step" = one pass of all 40 blocks over the token sequence (weights differ per block, activations
are synthetic N(0,1), weights N(0,0.02) seeded).  The work is fixed and the tokens are sharded over
the ranks, so scaling is "strong".  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

GRID = (21, 45, 80)
TOKENS = GRID[0] * GRID[1] * GRID[2]  # 75,600
DIM, HEADS, HEAD_DIM, LAYERS = 5120, 40, 128, 40
FFN, TEXT_TOKENS, TEXT_DIM = 13824, 512, 4096
LATENT = (1, 16, 21, 90, 160)
METRICS = {"dit": "wan2.1-14b_dit_step_ms_720p", "hotpath": "wan2.1-14b_dit_step_self_attention_hot_path_ms_720p"}


def flops_per_step(tokens: int = TOKENS, workload: str = "hotpath") -> float:
    attn = 4.0 * HEADS * tokens * tokens * HEAD_DIM
    lin = 4 * 2.0 * tokens * DIM * DIM
    if workload == "dit":  # + cross-attention (q, o on tokens; k, v on the text; attention) + FFN
        lin += 2 * 2.0 * tokens * DIM * DIM + 2 * 2.0 * TEXT_TOKENS * DIM * DIM + 2 * 2.0 * tokens * DIM * FFN
        attn += 4.0 * HEADS * tokens * TEXT_TOKENS * HEAD_DIM
    return LAYERS * (attn + lin)


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs: ONE long-lived `nvidia-smi -lms`
    process (spawning a query per sample stalls kernel launches of short steps)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        samples = []
        if self.proc is not None:
            self.proc.terminate()  # the exact process started above
            try:
                out, _ = self.proc.communicate(timeout=5)
                samples = [[f.strip() for f in ln.split(",")] for ln in out.splitlines() if ln.strip()]
            except Exception:
                self.proc.kill()
        sm = [int(s[0]) for s in samples if s[0].isdigit()]
        mx = [int(s[1]) for s in samples if len(s) > 1 and s[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(s) > 2 + i and s[2 + i].lower() == "active" for s in samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's algorithm (oracle port) on the host cores, bounded sample
# ----------------------------------------------------------------------------------------------
def cpu_hot_path_ms(sample_rows: int = 2048, sample_queries: int = 1024, repeats: int = 2, workload: str = "hotpath"):
    """Time the reference's CPU-runnable path (its dynamic quantised linear + fp32 SDPA,
    dax/quant/nn/dynamic/linear.py:145-228 and dax/adapters/wan/attn_adapter.py:222-229, as restated in
    oracle/) on a bounded sample and scale it to one full step.  Linears are timed on `sample_rows` of
    the 75,600 token rows (cost is linear in rows); attention on `sample_queries` query rows of one head
    against all 75,600 keys (cost is linear in query rows and heads)."""
    from oracle import dax_oracle as O
    torch.manual_seed(0)
    threads = torch.get_num_threads()
    x = torch.randn(sample_rows, DIM).bfloat16()
    w = (torch.randn(DIM, DIM) * 0.02).bfloat16()
    qw, sw = O.quantize_weight(w, torch.float8_e4m3fn)
    t0 = time.perf_counter()
    for _ in range(repeats):
        O.linear_fp8(x, qw, sw, None, torch.bfloat16, torch.float8_e4m3fn)
    t_lin = (time.perf_counter() - t0) / repeats * (TOKENS / sample_rows)
    q = torch.randn(1, 1, sample_queries, HEAD_DIM)
    k = torch.randn(1, 1, TOKENS, HEAD_DIM)
    v = torch.randn(1, 1, TOKENS, HEAD_DIM)
    t0 = time.perf_counter()
    for _ in range(repeats):
        O.sdpa_fp32(q, k, v)
    t_att = (time.perf_counter() - t0) / repeats * (TOKENS / sample_queries) * HEADS
    lin_units = 4.0  # in units of one 5120 -> 5120 linear over all tokens
    if workload == "dit":  # cross-attention q/o, FFN up/down (cost proportional to K x N); text-side terms negligible
        lin_units += 2.0 + 2.0 * FFN / DIM
        t_att *= 1.0 + TEXT_TOKENS / TOKENS
    step_ms = LAYERS * (lin_units * t_lin + t_att) * 1e3
    sample = (f"1 layer: FP8 linear 5120->5120 on {sample_rows} of {TOKENS} rows (x{lin_units:.1f} by K x N), fp32 SDPA on "
              f"{sample_queries} query rows of 1 head x all keys; scaled linearly to {LAYERS} layers, {TOKENS} rows, {HEADS} heads")
    return step_ms, threads, sample


def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    steps = max(1, args.steps)
    vals = []
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_hot_path_ms(256, 64)
    threads = sample = None
    for _ in range(min(steps, 3)):
        ms, threads, sample = cpu_hot_path_ms(workload=args.workload)
        vals.append(ms)
    ms = statistics.mean(vals)
    line = {"impl": "reference", "metric": METRICS[args.workload], "value": ms, "unit": "ms", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp32 SDPA + fp8 linears (CPU)", "data": "synthetic",
            "config": workload_config(args.gpus, args.workload),
            "cpu_baseline": {"value": ms, "unit": "ms", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(n: int, workload: str = "hotpath"):
    what = ("one full DiT forward (patch embedding, condition embedder, 40 x [self-attention, cross-attention over 512 text "
            "tokens, FFN 13,824], output head) of a Wan2.1-14B-shaped model" if workload == "dit"
            else "hot path only: the 40 self-attention blocks of a Wan2.1-14B-shaped DiT step")
    return {"workload": f"cfg5 step: {what}, 720p/81 frames, "
                        "75,600 tokens (21x45x80), dim 5120, 40 heads x 128, FP8-e4m3 dynamic linears, "
                        "INT8-QK/FP8-PV attention, RMSNorm + 3-D RoPE",
            "tokens": TOKENS, "layers": LAYERS, "parallelism": f"ulysses_sp{n}", "overlap_comm": n > 1,
            "l2": "inputs_larger_than_L2 (774 MB of activations per tensor per step)"}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="dax_b200", choices=["dax_b200", "reference"])
    ap.add_argument("--workload", default="dit", choices=["dit", "hotpath"])
    ap.add_argument("--qkv-chunks", type=int, default=0,
                    help="sequence parallel only: row chunks of the Q/K/V projections whose exchange overlaps the "
                         "next chunk (0 = the processor's default)")
    ap.add_argument("--loop", type=int, default=0,
                    help="dit workload only: after the timed steps, also run one flow-matching loop of this many "
                         "denoising steps (classifier-free guidance 5.0, TeaCache threshold 0.2) and report it")
    ap.add_argument("--layers", type=int, default=LAYERS, help=argparse.SUPPRESS)  # profiling captures only
    ap.add_argument("--tokens", type=int, default=TOKENS, help=argparse.SUPPRESS)  # profiling captures only
    ap.add_argument("--no-cpu-baseline", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--attention-mode", default="sage", help=argparse.SUPPRESS)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch.distributed as dist

    from dax_b200 import _lib, ops
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import WanSelfAttentionStack, _Pipe, wan_rope_table

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (use --impl reference for the CPU arm)"
    assert args.warmup >= 3 or args.layers != LAYERS or args.tokens != TOKENS, "timing rules: at least 3 warm-up steps"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sp = world > 1
    if sp:
        os.environ.setdefault("LOCAL_WORLD_SIZE", str(world))
    full = args.layers == LAYERS and args.tokens == TOKENS
    tokens, layers = args.tokens, args.layers
    assert tokens % world == 0 and HEADS % world == 0
    s = tokens // world

    # ---- model: random-init weights N(0, 0.02), zero bias, created directly on the device ----
    from dax_b200.adapters.wan.modules import WanDiT
    torch.manual_seed(1234)
    dit = args.workload == "dit"
    with torch.device("meta"):
        model = (WanDiT(layers=layers, dim=DIM, ffn_dim=FFN, heads=HEADS, text_dim=TEXT_DIM) if dit
                 else WanSelfAttentionStack(layers, DIM, HEADS))
    model = model.to_empty(device=dev).to(torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(1234)  # same stream on every rank: identical replicas
    with torch.no_grad():
        for p_name, p in model.named_parameters():
            if p_name.endswith(("norm_q.weight", "norm_k.weight", "norm2.weight")):
                p.fill_(1.0)
            elif p_name.endswith("bias"):
                p.zero_()
            elif "scale_shift_table" in p_name:
                p.copy_((torch.randn(p.shape, generator=g, device=dev) / DIM ** 0.5).to(p.dtype))
            else:
                p.copy_((torch.randn(p.shape, generator=g, device=dev) * 0.02).to(p.dtype))
    pipe = _Pipe(model)
    optimize_pipe(pipe, sequence_parallel=sp, compile=False, overlap_comm=sp, fp8_linear=True,
                  attention_mode=args.attention_mode)
    if args.qkv_chunks > 0:
        for mod in model.modules():
            proc = getattr(mod, "processor", None)
            if proc is not None and hasattr(proc, "qkv_chunks"):
                proc.qkv_chunks = args.qkv_chunks
    torch.cuda.empty_cache()

    gx = torch.Generator().manual_seed(99)
    if dit:
        latent = LATENT
        if tokens != TOKENS:  # reduced case for profiler captures: 4 frames of a square latent
            side = int(round((tokens // 4) ** 0.5))
            assert 4 * side * side == tokens, "--tokens for the dit workload must be 4 * n^2"
            latent = (1, 16, 4, 2 * side, 2 * side)
        x_host = torch.randn(latent, generator=gx).to(torch.bfloat16).pin_memory()  # replicated latent, split inside
        text = torch.randn(1, TEXT_TOKENS, TEXT_DIM, generator=gx).to(torch.bfloat16).to(dev)
        timestep = torch.randint(0, 1000, (1,), generator=gx).to(dev)
        y_host = torch.empty(latent, dtype=torch.bfloat16).pin_memory()
        h2d_bytes = d2h_bytes = x_host.numel() * 2 * world
    else:
        rope = wan_rope_table(GRID if tokens == TOKENS else (1, 1, tokens), device=dev)
        x_full = torch.randn(1, tokens, DIM, generator=gx).to(torch.bfloat16)
        x_host = x_full[:, rank * s:(rank + 1) * s].contiguous().pin_memory()
        y_host = torch.empty_like(x_host).pin_memory()
        h2d_bytes = d2h_bytes = x_host.numel() * 2 * world
    x_dev = x_host.to(dev)

    def barrier():
        if sp:
            dist.barrier()
        torch.cuda.synchronize()

    def step(x):
        with torch.no_grad():
            if dit:
                return pipe.transformer(x, timestep, text, return_dict=False)[0]
            return pipe.transformer(x, rotary_emb=rope)

    for _ in range(args.warmup):
        step(x_dev)
    barrier()

    # ---- timed region: K steps, inputs resident in HBM ----
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ops.TRACE.reset(timing=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        y = step(x_dev)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = ops.TRACE.launches
    trace = ops.TRACE.summary()
    ops.TRACE.reset(timing=False)
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms_total], device=dev)
    if sp:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps

    # ---- end to end through the public API with host buffers (H2D + D2H inside the timed region) ----
    e2e_steps = max(1, min(args.steps, 2))
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        x_dev.copy_(x_host, non_blocking=True)
        y = step(x_dev)
        y_host.copy_(y, non_blocking=True)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if sp:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    status = _lib.device_status()
    assert status == 0, f"device status {status}: a kernel wait timed out"
    assert torch.isfinite(y_host.float()).all(), "non-finite output"

    # ---- optional: BASELINE config 5's loop (50 steps, guidance => two forwards per step, TeaCache 0.2) ----
    loop = None
    if dit and args.loop > 0:
        from dax_b200.adapters.wan.sampling import denoise
        from dax_b200.cache import teacache
        teacache.configure(pipe.transformer, teacache_thresh=0.2, num_inference_steps=args.loop)
        neg = torch.randn(1, TEXT_TOKENS, TEXT_DIM, generator=gx).to(torch.bfloat16).to(dev)
        computed = [0]

        def count(i, _x):
            computed[0] += int(bool(pipe.transformer.should_calc_even)) + int(bool(pipe.transformer.should_calc_odd))

        barrier()
        e0.record()
        out = denoise(pipe, x_dev, text, neg, num_inference_steps=args.loop, guidance_scale=5.0, flow_shift=5.0,
                      on_step=count)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if sp:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pipe.transformer.__class__.enable_teacache = False
        assert torch.isfinite(out.float()).all(), "non-finite sample"
        loop = {"denoising_steps": args.loop, "forwards": 2 * args.loop, "forwards_computed": computed[0],
                "forwards_skipped": 2 * args.loop - computed[0], "ms_total": float(t.item()),
                "ms_per_denoising_step": float(t.item()) / args.loop, "guidance_scale": 5.0, "teacache_thresh": 0.2,
                "solver": "first-order flow matching (Euler), flow_shift 5.0"}

    if rank != 0:
        if sp:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (attention forward), from the live CUDA-event trace ----
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    bf16_peak = peaks.get("bf16_tflops_sustained")
    peak_src = "2 x measured sustained bf16 (8-bit tensor pipe)"
    if bf16_peak is None:
        bf16_peak, peak_src = 1400.0, "2 x fallback sustained bf16 (8-bit tensor pipe)"
    peak8 = 2.0 * bf16_peak
    calls, att_ms, metas = trace.get("attn_forward", (0, 0.0, []))
    att_flops = sum(4.0 * m[0] * m[1] * m[2] * m[3] * HEAD_DIM for m in metas)
    achieved = att_flops / (att_ms * 1e-3) / 1e12 if att_ms > 0 else None
    # DRAM traffic per launch: ncu measured 392 MB for a 40-head, 16,384-token launch (profiles/), 0.936 of the
    # compulsory operand bytes (INT8 Q 128 B + bf16 O 256 B per query row, INT8 K + FP8 V 256 B per key row, per head);
    # it grows in proportion to rows x heads, so the same factor is applied to the launches timed here
    traffic = (sum(0.936 * m[0] * m[1] * (384.0 * m[2] + 256.0 * m[3]) for m in metas) / calls) if calls else None
    roofline = {"bound": "tensor", "kernel": "attn_fwd_kernel", "achieved": achieved, "peak": peak8, "unit": "TFLOP/s",
                "frac": achieved / peak8 if achieved else None, "traffic": traffic, "peak_source": peak_src,
                "launches": calls, "avg_launch_ms": att_ms / calls if calls else None,
                "share_of_step": att_ms / (ms_step * args.steps) if calls else None}
    breakdown = {k: {"calls": c, "ms_per_step": tms / args.steps} for k, (c, tms, _) in trace.items()}

    cpu = None
    if not args.no_cpu_baseline:
        ms, threads, sample = cpu_hot_path_ms(workload=args.workload)
        cpu = {"value": ms, "unit": "ms", "cores": threads, "kind": "port", "sample": sample}

    line = {"metric": METRICS[args.workload], "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8/fp8 (fp32 accumulate)", "data": "synthetic",
            "config": workload_config(world, args.workload) if full else
            {"workload": f"REDUCED profiling case ({args.workload}): {layers} layers, {tokens} tokens"},
            "tflops": flops_per_step(tokens, args.workload) * layers / LAYERS / (ms_step * 1e-3) / 1e12,
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "kernel_ms_per_step": breakdown}
    if loop is not None:
        line["denoise_loop"] = loop
    print(json.dumps(line), flush=True)
    if sp:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

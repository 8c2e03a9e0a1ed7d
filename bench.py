#!/usr/bin/env python
"""Benchmark of one Wan2.1-14B-shaped DiT denoising step, Ulysses sequence parallel over N GPUs.

Default workload: 720p / 81 frames (latents 16x21x90x160 -> 75,600 tokens on a 21x45x80 grid; 40 blocks, hidden
5120, 40 heads of 128, FFN 13,824, 512 text tokens), FP8-e4m3 dynamic linears, quantised attention.

    --workload dit       (default) the whole DiT forward: patch embedding, condition embedder, 40 x
                         (self-attention block, cross-attention, FFN), output head
    --workload hotpath   only the 40 self-attention blocks (the hot path proper)
    --grid FxHxW         token grid (default 21x45x80; 21x30x52 = 480p, 32,760 tokens)
    --linear fp8|int8    dynamic linear arithmetic (default fp8)
    --attention-mode M   auto (default) | sage | int8_bf16 | bf16.  "auto" measures every mode of the attention
                         kernel against fp32 SDPA on a slice at the benchmark's sequence length and times the
                         FASTEST MODE THAT MEETS rel-L2 <= 1e-2 and cosine >= 0.999; the other modes' step times
                         and parity figures are reported beside it under "attention_modes".

    python bench.py [--gpus N] [--steps K] [--warmup W]            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                            CPU arm: the reference's algorithm
                                                                    (oracle port) on all host cores

One "step" = one pass of all 40 blocks over the token sequence (weights differ per block, activations are
synthetic N(0,1), weights N(0,0.02), seeded).  The work is fixed and the tokens are sharded over the ranks, so
scaling is "strong".  Prints ONE JSON line on rank 0.  Besides the timed step the line carries: the parity of
every attention mode, a sequence-parallel parity check (N > 1), the measured exchange overlap (N > 1), and at
N = 1 the standalone attention (40 heads x 32,760 tokens) and the dynamic-linear sweep at 75,600 rows.
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

DIM, HEADS, HEAD_DIM, LAYERS = 5120, 40, 128, 40
FFN, TEXT_TOKENS, TEXT_DIM = 13824, 512, 4096
GRID_720P, GRID_480P = (21, 45, 80), (21, 30, 52)
MODES = ("sage", "int8_bf16", "bf16")
MODE_NAMES = {"sage": "INT8-QK/FP8-PV", "int8_bf16": "INT8-QK/bf16-PV", "bf16": "bf16-QK/bf16-PV"}
PARITY_BOUND = {"rel_l2": 1e-2, "cosine": 0.999}
LINEAR_SWEEP = ((5120, 5120), (5120, 13824), (13824, 5120), (4096, 5120))  # (K, N) at M = 75,600


def metric_name(workload: str, grid) -> str:
    res = {GRID_720P: "720p", GRID_480P: "480p"}.get(tuple(grid), "x".join(map(str, grid)))
    base = "wan2.1-14b_dit_step_ms_" if workload == "dit" else "wan2.1-14b_dit_step_self_attention_hot_path_ms_"
    return base + res


def flops_per_step(tokens: int, workload: str) -> float:
    attn = 4.0 * HEADS * tokens * tokens * HEAD_DIM
    lin = 4 * 2.0 * tokens * DIM * DIM
    if workload == "dit":  # + cross-attention (q, o on tokens; k, v on the text; attention) + FFN
        lin += 2 * 2.0 * tokens * DIM * DIM + 2 * 2.0 * TEXT_TOKENS * DIM * DIM + 2 * 2.0 * tokens * DIM * FFN
        attn += 4.0 * HEADS * tokens * TEXT_TOKENS * HEAD_DIM
    return LAYERS * (attn + lin)


def load_peaks():
    """Measured denominators (bf16 tensor TFLOP/s sustained, HBM GB/s) or the stated fallback."""
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(pk["bf16_tflops_sustained"]), float(pk["hbm_gbs"]), "measured"
    except Exception:
        return 1400.0, 6650.0, "fallback"


def mode_peak(mode: str, peak16: float) -> float:
    """Tensor roofline of an attention mode: both contractions have the same FLOPs; 8-bit operands run at twice
    the 16-bit rate, so a mixed mode is bounded by the harmonic combination."""
    peak8 = 2.0 * peak16
    return {"sage": peak8, "bf16": peak16, "int8_bf16": 2.0 / (1.0 / peak8 + 1.0 / peak16)}[mode]


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
def use_all_host_cores() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core at every N."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0)) or n
    except Exception:
        pass
    torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_step_ms(tokens: int, workload: str, linear: str, sample_rows: int = 4096, sample_queries: int = 2048,
                repeats: int = 2):
    """Time the reference's CPU-runnable path (its dynamic quantised linear + fp32 SDPA,
    dax/quant/nn/dynamic/linear.py:145-228 and dax/adapters/wan/attn_adapter.py:222-229, as restated in
    oracle/) on a bounded sample and scale it to one full step.  Linears are timed on `sample_rows` of
    the token rows (cost is linear in rows); attention on `sample_queries` query rows of one head
    against all keys (cost is linear in query rows and heads)."""
    from oracle import dax_oracle as O
    threads = use_all_host_cores()
    torch.manual_seed(0)
    x = torch.randn(sample_rows, DIM).bfloat16()
    w = (torch.randn(DIM, DIM) * 0.02).bfloat16()
    wdt = torch.int8 if linear == "int8" else torch.float8_e4m3fn
    qw, sw = O.quantize_weight(w, wdt)
    t0 = time.perf_counter()
    for _ in range(repeats):
        if linear == "int8":
            O.linear_int8(x, qw, sw, None, torch.bfloat16)
        else:
            O.linear_fp8(x, qw, sw, None, torch.bfloat16, torch.float8_e4m3fn)
    t_lin = (time.perf_counter() - t0) / repeats * (tokens / sample_rows)
    q = torch.randn(1, 1, sample_queries, HEAD_DIM)
    k = torch.randn(1, 1, tokens, HEAD_DIM)
    v = torch.randn(1, 1, tokens, HEAD_DIM)
    t0 = time.perf_counter()
    for _ in range(repeats):
        O.sdpa_fp32(q, k, v)
    t_att = (time.perf_counter() - t0) / repeats * (tokens / sample_queries) * HEADS
    lin_units = 4.0  # in units of one 5120 -> 5120 linear over all tokens
    if workload == "dit":  # cross-attention q/o, FFN up/down (cost proportional to K x N); text-side terms negligible
        lin_units += 2.0 + 2.0 * FFN / DIM
        t_att *= 1.0 + TEXT_TOKENS / tokens
    step_ms = LAYERS * (lin_units * t_lin + t_att) * 1e3
    sample = (f"1 layer: {linear.upper()} linear 5120->5120 on {sample_rows} of {tokens} rows (x{lin_units:.1f} by K x N), "
              f"fp32 SDPA on {sample_queries} query rows of 1 head x all keys; scaled linearly to {LAYERS} layers, "
              f"{tokens} rows, {HEADS} heads")
    return step_ms, threads, sample


def run_reference_arm(args, rank: int, grid, tokens: int):
    if rank != 0:
        return
    vals = []
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_step_ms(tokens, args.workload, args.linear, 256, 64)
    threads = sample = None
    for _ in range(min(max(1, args.steps), 3)):
        ms, threads, sample = cpu_step_ms(tokens, args.workload, args.linear)
        vals.append(ms)
    ms = statistics.mean(vals)
    line = {"impl": "reference", "metric": metric_name(args.workload, grid), "value": ms, "unit": "ms", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": f"fp32 SDPA + {args.linear} linears (CPU)", "data": "synthetic",
            "config": workload_config(args.gpus, args.workload, grid, tokens, args.linear, None),
            "cpu_baseline": {"value": ms, "unit": "ms", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(n: int, workload: str, grid, tokens: int, linear: str, mode):
    what = ("one full DiT forward (patch embedding, condition embedder, 40 x [self-attention, cross-attention over 512 text "
            "tokens, FFN 13,824], output head) of a Wan2.1-14B-shaped model" if workload == "dit"
            else "hot path only: the 40 self-attention blocks of a Wan2.1-14B-shaped DiT step")
    res = {GRID_720P: "720p/81 frames", GRID_480P: "480p/81 frames"}.get(tuple(grid), "custom grid")
    lin = "FP8-e4m3" if linear == "fp8" else "INT8"
    att = f"{MODE_NAMES[mode]} attention" if mode else "quantised attention"
    return {"workload": f"{what}, {res}, {tokens:,} tokens ({grid[0]}x{grid[1]}x{grid[2]}), dim 5120, 40 heads x 128, "
                        f"{lin} dynamic linears, {att}, RMSNorm + 3-D RoPE",
            "tokens": tokens, "layers": LAYERS, "parallelism": f"ulysses_sp{n}", "overlap_comm": n > 1,
            "l2": f"inputs_larger_than_L2 ({tokens * DIM * 2 / 1e6:.0f} MB of activations per tensor per step)"}


# ----------------------------------------------------------------------------------------------
# GPU arm helpers
# ----------------------------------------------------------------------------------------------
def cfg2_qkv(heads: int, S: int, seed: int, device=None):
    """Standalone-attention inputs: Q, V ~ N(0,1), K ~ N(0,1) + a per-channel offset ~ N(0, std 2) broadcast
    over the tokens (the case K mean-smoothing exists for), bf16."""
    g = torch.Generator(device=device).manual_seed(seed) if device is not None else torch.Generator().manual_seed(seed)
    kw = dict(generator=g, device=device) if device is not None else dict(generator=g)
    q = torch.randn(1, heads, S, HEAD_DIM, **kw).bfloat16()
    k = (torch.randn(1, heads, S, HEAD_DIM, **kw) + 2.0 * torch.randn(1, heads, 1, HEAD_DIM, **kw)).bfloat16()
    v = torch.randn(1, heads, S, HEAD_DIM, **kw).bfloat16()
    return q, k, v


def attention_parity(ops, S: int, dev, rows: int = 256, heads: int = 2):
    """rel-L2 and cosine of every attention mode against fp32 SDPA (the reference's TORCH_SDPA branch,
    dax/adapters/wan/attn_adapter.py:222-229) on two slices of `rows` query rows x `heads` heads x ALL keys at the
    benchmark's sequence length: the first rows and the last rows (the ragged last tile).  Outside any timed region."""
    from oracle import dax_oracle as O
    use_all_host_cores()
    q, k, v = cfg2_qkv(heads, S, seed=7)
    idx = torch.cat([torch.arange(0, min(rows, S)), torch.arange(max(0, S - rows), S)]).unique()
    ref = O.sdpa_fp32(q[:, :, idx], k, v)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out = {}
    for mode in MODES:
        o = ops.attention(qd, kd, vd, mode=mode)[:, :, idx.to(dev)].float().cpu()
        rel, cos = O.rel_l2(o, ref), O.cosine(o, ref)
        out[mode] = {"rel_l2": rel, "cosine": cos, "bound": PARITY_BOUND["rel_l2"], "cosine_bound": PARITY_BOUND["cosine"],
                     "pass": bool(rel <= PARITY_BOUND["rel_l2"] and cos >= PARITY_BOUND["cosine"])}
    return out, {"against": "fp32 SDPA (oracle)", "heads": heads, "query_rows": int(idx.numel()), "keys": S,
                 "k_offset_std": 2.0}


def time_events(fn, repeats: int, warm: int = 2):
    """Average milliseconds of fn() over `repeats` calls, CUDA events on the current stream."""
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(repeats):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / repeats


def attention_kernel_ms(ops, heads: int, S: int, dev, repeats: int = 5):
    """Forward-kernel time of every mode on one (heads x S) problem; also the prepare step's."""
    q, k, v = cfg2_qkv(heads, S, seed=11, device=dev)
    out = torch.empty((1, S, heads, HEAD_DIM), dtype=torch.bfloat16, device=dev).transpose(1, 2)
    res = {}
    for mode in MODES:
        if mode == "bf16":  # reads Q, K, V in place: one kernel, nothing to prepare
            res[mode] = {"forward_ms": time_events(lambda: ops.attention_direct(q, k, v, out), repeats, 2), "prepare_ms": 0.0}
            continue
        prep = time_events(lambda: ops.attn_prepare(q, k, v, mode), 3, 1)
        plan = ops.attn_prepare(q, k, v, mode)
        fwd = time_events(lambda: ops.attn_forward(plan, out), repeats, 2)
        res[mode] = {"forward_ms": fwd, "prepare_ms": prep}
    return res


def linear_sweep(ops, M: int, dev, peak8: float, hbm: float, repeats: int = 10):
    """Dynamic-linear sweep at M rows: per (K -> N) and arithmetic the quantiser's GB/s and the GEMM's TOP/s
    (dax/quant/nn/dynamic/linear.py:145-228)."""
    rows = []
    g = torch.Generator(device=dev).manual_seed(5)
    for K, N in LINEAR_SWEEP:
        x = torch.randn(M, K, generator=g, device=dev).bfloat16()
        w = torch.randn(N, K, generator=g, device=dev) * 0.02
        bias = torch.zeros(N, device=dev, dtype=torch.bfloat16)
        for name, qd, qmax in (("int8", torch.int8, 127.0), ("fp8_e4m3", torch.float8_e4m3fn, 448.0)):
            sw = (w.abs().amax(1) / qmax).clamp_min(1e-12).float().contiguous()
            qw = (w / sw[:, None]).round().clamp(-127, 127).to(torch.int8) if qd == torch.int8 else (w / sw[:, None]).to(qd)
            qw = qw.contiguous()
            t_q = time_events(lambda: ops.quant_rowwise(x, qd), repeats, 2)
            qx, sx = ops.quant_rowwise(x, qd)
            out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            t_g = time_events(lambda: ops.gemm_dequant(qx, sx, qw, sw, bias, torch.bfloat16, out=out, ldo=N), repeats, 2)
            tops = 2.0 * M * N * K / (t_g * 1e-3) / 1e12
            gbs = (M * K * 3.0 + 4.0 * M) / (t_q * 1e-3) / 1e9
            rows.append({"K": K, "N": N, "arith": name, "gemm_ms": t_g, "gemm_tops": tops, "gemm_frac_of_8bit_peak": tops / peak8,
                         "quant_ms": t_q, "quant_gbs": gbs, "quant_frac_of_hbm": gbs / hbm})
            del qx, sx, out, qw
        del x, w
        torch.cuda.empty_cache()
    return rows


def sequence_parallel_parity(mode: str, world: int, rank: int, dev):
    """One INT8-linear self-attention layer at 32,760 tokens (21x30x52: at 8 ranks the local length 4,095 is odd,
    so the Q/K/V chunks and both O micro-batches are ragged) run sequence-parallel with the overlapped exchange, in
    both O-path splits, against the SAME layer run un-sharded on this rank's own GPU; every rank checks its own rows."""
    import torch.distributed as dist

    from dax_b200.adapters.wan.attn_adapter import DAXWanAttnProcessor2_0
    from dax_b200.adapters.wan.modules import Attention, wan_rope_table
    from dax_b200.adapters.wan.transformer_adapter import quantize_transformer
    grid = GRID_480P
    S = grid[0] * grid[1] * grid[2]
    assert S % world == 0
    s = S // world
    torch.manual_seed(4321)
    holder = torch.nn.Module()
    with torch.device("meta"):
        holder.attn = Attention(DIM, HEADS)
    holder = holder.to_empty(device=dev).to(torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(4321)
    with torch.no_grad():
        for name, p in holder.named_parameters():
            if name.endswith(("norm_q.weight", "norm_k.weight")):
                p.copy_((1 + 0.1 * torch.randn(p.shape, generator=g, device=dev)).to(p.dtype))
            elif name.endswith("bias"):
                p.copy_((0.05 * torch.randn(p.shape, generator=g, device=dev)).to(p.dtype))
            else:
                p.copy_((torch.randn(p.shape, generator=g, device=dev) * 0.02).to(p.dtype))
    quantize_transformer(holder, "int8")
    x = torch.randn(1, S, DIM, generator=g, device=dev).bfloat16()
    rope = wan_rope_table(grid, device=dev)
    with torch.no_grad():
        holder.attn.set_processor(DAXWanAttnProcessor2_0(sequence_parallel=False, attention_mode=mode))
        want = holder.attn(x, rotary_emb=rope)[:, rank * s:(rank + 1) * s].float()
        rels = {}
        info = {}
        variants = (("peer_stores", dict(exchange="auto")), ("nccl_o_split_rows", dict(exchange="nccl", o_split="rows")),
                    ("nccl_o_split_ranks", dict(exchange="nccl", o_split="ranks")))
        for name, kw in variants:
            proc = DAXWanAttnProcessor2_0(sp_size=world, overlap_comm=True, attention_mode=mode, **kw)
            holder.attn.set_processor(proc)
            got = holder.attn(x[:, rank * s:(rank + 1) * s].contiguous(), rotary_emb=rope).float()
            rels[name] = float((got - want).norm() / want.norm())
            info = {"qkv_chunks": proc.qkv_chunks, "o_micro_batches": proc.o_micro_batches}
    t = torch.tensor([rels[n] for n, _ in variants], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    worst = float(t.max())
    del holder, x, want, got
    torch.cuda.empty_cache()
    return {"rel_l2": worst, **{"rel_l2_" + n: float(t[i]) for i, (n, _) in enumerate(variants)},
            "bound": 2e-3, "pass": worst <= 2e-3, "tokens": S, "s_local": s, "linear": "int8", "attention_mode": mode,
            "against": "the same layer un-sharded on each rank's own GPU (max over ranks)", **info}


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
    ap.add_argument("--grid", default="21x45x80", help="token grid FxHxW (21x45x80 = 720p, 21x30x52 = 480p)")
    ap.add_argument("--linear", default="fp8", choices=["fp8", "int8"])
    ap.add_argument("--attention-mode", default="auto", choices=["auto"] + list(MODES))
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="sequence parallel only: how the sequence<->head exchanges travel (peer = stores into the other "
                         "GPUs' buffers by the producing kernels; nccl = chunked point-to-point groups; auto = peer if available)")
    ap.add_argument("--qkv-chunks", type=int, default=0,
                    help="sequence parallel only: row chunks of the Q/K/V projections whose exchange overlaps the "
                         "next chunk (0 = the processor's default)")
    ap.add_argument("--loop", type=int, default=0,
                    help="dit workload only: after the timed steps, also run one flow-matching loop of this many "
                         "denoising steps (classifier-free guidance 5.0, TeaCache threshold 0.2) and report it")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the per-mode step times, the standalone attention, the linear sweep and the overlap legs")
    ap.add_argument("--layers", type=int, default=LAYERS, help=argparse.SUPPRESS)  # profiling captures only
    ap.add_argument("--tokens", type=int, default=0, help=argparse.SUPPRESS)       # profiling captures only: 4 * n^2
    ap.add_argument("--no-cpu-baseline", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    grid = tuple(int(v) for v in args.grid.lower().split("x"))
    assert len(grid) == 3, "--grid wants FxHxW"
    if args.tokens:  # reduced case for profiler captures: 4 frames of a square latent
        side = int(round((args.tokens // 4) ** 0.5))
        assert 4 * side * side == args.tokens, "--tokens must be 4 * n^2"
        grid = (4, side, side)
    tokens = grid[0] * grid[1] * grid[2]

    if args.impl == "reference":
        run_reference_arm(args, rank, grid, tokens)
        return

    import torch.distributed as dist

    from dax_b200 import _lib, ops
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import WanDiT, WanSelfAttentionStack, _Pipe, wan_rope_table

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (use --impl reference for the CPU arm)"
    full = args.layers == LAYERS and not args.tokens
    assert args.warmup >= 3 or not full, "timing rules: at least 3 warm-up steps"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sp = world > 1
    if sp:
        os.environ.setdefault("LOCAL_WORLD_SIZE", str(world))
    layers = args.layers
    assert tokens % world == 0 and HEADS % world == 0
    s = tokens // world
    peak16, hbm, peak_kind = load_peaks()
    peak8 = 2.0 * peak16

    # ---- model: random-init weights N(0, 0.02), zero bias, created directly on the device ----
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
    optimize_pipe(pipe, sequence_parallel=sp, compile=False, overlap_comm=sp, fp8_linear=args.linear == "fp8",
                  int8_linear=args.linear == "int8", attention_mode="sage")
    procs = [m.processor for m in model.modules() if hasattr(getattr(m, "processor", None), "attention_mode")]
    for proc in procs:
        proc.exchange = args.exchange
        if args.qkv_chunks > 0:
            proc.qkv_chunks = args.qkv_chunks
    torch.cuda.empty_cache()

    def set_mode(mode):
        for proc in procs:
            proc.attention_mode = mode

    def barrier():
        if sp:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        if sp:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- parity of every attention mode at this sequence length, and the choice of the timed mode ----
    parity, parity_info = (attention_parity(ops, tokens, dev) if rank == 0 else ({}, {}))
    kernel_ms = attention_kernel_ms(ops, HEADS // world, tokens, dev, repeats=3) if rank == 0 else {}
    choice = [None]
    if rank == 0:
        if args.attention_mode != "auto":
            choice[0] = args.attention_mode
        else:
            ok = [m for m in MODES if parity[m]["pass"]]
            assert ok, f"no attention mode meets the parity bound: {parity}"
            choice[0] = min(ok, key=lambda m: kernel_ms[m]["forward_ms"])
    if sp:
        dist.broadcast_object_list(choice, src=0)
    mode = choice[0]
    set_mode(mode)
    torch.cuda.empty_cache()

    parity_sp = sequence_parallel_parity(mode, world, rank, dev) if sp else None
    if parity_sp is not None:
        assert parity_sp["pass"], f"sequence-parallel result differs from the un-sharded layer: {parity_sp}"

    # ---- inputs ----
    gx = torch.Generator().manual_seed(99)
    if dit:
        latent = (1, 16, grid[0], 2 * grid[1], 2 * grid[2])
        x_host = torch.randn(latent, generator=gx).to(torch.bfloat16).pin_memory()  # replicated latent, split inside
        text = torch.randn(1, TEXT_TOKENS, TEXT_DIM, generator=gx).to(torch.bfloat16).to(dev)
        timestep = torch.randint(0, 1000, (1,), generator=gx).to(dev)
        y_host = torch.empty(latent, dtype=torch.bfloat16).pin_memory()
        h2d_bytes = d2h_bytes = x_host.numel() * 2 * world
    else:
        rope = wan_rope_table(grid, device=dev)
        x_full = torch.randn(1, tokens, DIM, generator=gx).to(torch.bfloat16)
        x_host = x_full[:, rank * s:(rank + 1) * s].contiguous().pin_memory()
        y_host = torch.empty_like(x_host).pin_memory()
        h2d_bytes = d2h_bytes = x_host.numel() * 2 * world
    x_dev = x_host.to(dev)

    def step(x):
        with torch.no_grad():
            if dit:
                return pipe.transformer(x, timestep, text, return_dict=False)[0]
            return pipe.transformer(x, rotary_emb=rope)

    def timed_steps(n: int) -> float:
        """Milliseconds per step over n steps: barrier + synchronise on both sides, CUDA events, max over ranks."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            step(x_dev)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / n

    for _ in range(args.warmup):
        step(x_dev)
    barrier()

    # ---- timed region: K steps, inputs resident in HBM ----
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ops.TRACE.reset(timing=True)
    ms_step = timed_steps(args.steps)
    launches = ops.TRACE.launches
    trace = ops.TRACE.summary()
    ops.TRACE.reset(timing=False)
    clocks = sampler.stop() if sampler else None

    # ---- end to end through the public API with host buffers (H2D + D2H inside the timed region) ----
    e2e_steps = max(1, min(args.steps, 2))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        x_dev.copy_(x_host, non_blocking=True)
        y = step(x_dev)
        y_host.copy_(y, non_blocking=True)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    status = _lib.device_status()
    assert status == 0, f"device status {status}: a kernel wait timed out"
    assert torch.isfinite(y_host.float()).all(), "non-finite output"

    # ---- the other attention modes through the same step (>= 3 steps each after one warm-up step) ----
    mode_steps = {mode: ms_step}
    if not args.no_extras:
        for m in MODES:
            if m != mode:
                set_mode(m)
                step(x_dev)
                mode_steps[m] = timed_steps(3)
        set_mode(mode)
        step(x_dev)

    # ---- exchange overlap (N > 1): all exchanges of a step alone; the step with the exchanges left out ----
    overlap = None
    if sp and not args.no_extras:
        from dax_b200.adapters.wan.attn_adapter import shared_exchange
        from dax_b200.parallel.peer import shared_peer_buffers
        xchg = shared_exchange()
        peers = shared_peer_buffers(xchg.group, world, rank) if args.exchange != "nccl" else None
        hd = DIM // world
        if peers is not None:
            # peer stores: the bytes of one step's exchanges moved ALONE by this library's own scatter kernel (a plain
            # copy: no norm, no rotation) into the other ranks' buffers; then the step with every "peer" pointer
            # redirected to this rank's own buffer (same kernels and barriers, no NVLink traffic)
            recv, recv_ptrs = peers.get("qkv_recv", (3, tokens, hd), torch.bfloat16, dev)
            o_recv, o_ptrs = peers.get("o_recv", (world, s, hd), torch.bfloat16, dev)
            src = torch.zeros((world, s, hd), dtype=torch.bfloat16, device=dev)
            src_o = torch.zeros((tokens, hd), dtype=torch.bfloat16, device=dev)

            def exchanges_alone():
                for _ in range(layers):
                    for i in range(3):  # Q, K, V slabs: copy engines
                        for dp in range(1, world):
                            p = (rank + dp) % world
                            ops.peer_copy(recv_ptrs[p] + ((i * tokens + rank * s) * hd) * 2, src[p])
                    for dp in range(1, world):  # attention rows: this library's scatter kernel (a plain copy here)
                        d = (rank + dp) % world
                        ops.rmsnorm_rope_pack(src_o[d * s:(d + 1) * s], norm_weight=None, do_norm=False, ldo=hd, col_group=hd,
                                              group_ptrs=[o_ptrs[d] + rank * s * hd * 2])
                peers.barrier(0)
            n_groups = 0
            how_total = ("total = the Q/K/V slabs (copy engines) and the attention rows (this library's scatter kernel) of one "
                         "step moved into the other ranks' buffers with nothing else running")
        else:
            xchg.recorded = []
            step(x_dev)
            replay, xchg.recorded = xchg.recorded, None
            n_groups = len(replay)

            def exchanges_alone():
                works = [c() for c in replay]
                for w in works:
                    w.wait()
            how_total = "total = every tokens<->heads exchange group of one step issued alone (nothing else running)"
        barrier()
        exchanges_alone()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(3):
            exchanges_alone()
        e1.record()
        barrier()
        total_ms = max_over_ranks(e0.elapsed_time(e1)) / 3
        def set_left_out(flag: bool):
            if peers is not None:
                peers.local_only = flag
            else:
                xchg.skip_comm = flag

        def leg(left_out: bool):
            """One warm-up step and three timed steps with the inter-GPU transfers on or left out; also the kernel
            times and the SM clock during the leg (the step is power-capped, so the clock is part of the result)."""
            set_left_out(left_out)
            step(x_dev)
            clock = ClockSampler(local_rank) if rank == 0 else None
            if clock:
                clock.start()
            ops.TRACE.reset(timing=True)
            ms = timed_steps(3)
            mhz = clock.stop()["sm_mhz"] if clock else None
            kernels = {k: tms / 3 for k, (c, tms, _) in ops.TRACE.summary().items()}
            ops.TRACE.reset(timing=False)
            set_left_out(False)
            return ms, mhz, kernels

        # with / left out / with: the first and the last leg bracket the diagnostic one, so that a drift of the
        # power-capped clock over the legs shows up instead of being booked as exchange time
        with_a, mhz_a, with_kernels = leg(False)
        nocomm_ms, nocomm_mhz, nocomm_kernels = leg(True)
        with_b, mhz_b, _ = leg(False)
        with_ms = 0.5 * (with_a + with_b)
        exposed = max(0.0, with_ms - nocomm_ms)
        bytes_out = layers * 4 * s * DIM * 2 * (world - 1) / world
        overlap = {"exchange": "peer_stores" if peers is not None else "nccl_p2p", "total_ms": total_ms, "exposed_ms": exposed,
                   "frac": 1.0 - exposed / total_ms if total_ms > 0 else None,
                   "step_ms_with_exchanges": with_ms, "step_ms_exchanges_left_out": nocomm_ms,
                   "bytes_out_per_gpu_per_step": bytes_out, "alone_gbs_per_gpu": bytes_out / (total_ms * 1e-3) / 1e9,
                   "exchange_groups_per_step": n_groups,
                   "kernel_ms_with_exchanges": with_kernels, "kernel_ms_exchanges_left_out": nocomm_kernels,
                   "step_ms_with_exchanges_before_and_after": [with_a, with_b],
                   "sm_mhz_with_exchanges_before_and_after": [mhz_a, mhz_b], "sm_mhz_exchanges_left_out": nocomm_mhz,
                   "how": how_total + "; exposed = step time minus the time of the same schedule with the inter-GPU "
                          "transfers left out (diagnostic leg, its outputs are not used); 3 steps each, max over ranks"}
        assert _lib.device_status() == 0

    # ---- optional: the 50-step loop (guidance => two forwards per step, TeaCache 0.2) ----
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
        loop_ms = max_over_ranks(e0.elapsed_time(e1))
        pipe.transformer.__class__.enable_teacache = False
        assert torch.isfinite(out.float()).all(), "non-finite sample"
        loop = {"denoising_steps": args.loop, "forwards": 2 * args.loop, "forwards_computed": computed[0],
                "forwards_skipped": 2 * args.loop - computed[0], "ms_total": loop_ms,
                "ms_per_denoising_step": loop_ms / args.loop, "guidance_scale": 5.0, "teacache_thresh": 0.2,
                "solver": "first-order flow matching (Euler), flow_shift 5.0",
                "cache_decisions": "planned before the loop from the timestep embeddings (one host read)"}

    if rank != 0:
        if sp:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- rank 0, others waiting at the final barrier: single-GPU extras, roofline, CPU baseline ----
    del model, pipe
    torch.cuda.empty_cache()
    cfg2 = sweep = None
    if not args.no_extras and not sp and full:
        k2 = attention_kernel_ms(ops, HEADS, GRID_480P[0] * GRID_480P[1] * GRID_480P[2], dev, repeats=10)
        fl2 = 4.0 * HEADS * (GRID_480P[0] * GRID_480P[1] * GRID_480P[2]) ** 2 * HEAD_DIM
        cfg2 = {"shape": "B=1, 40 heads x 128, S=32,760 (21x30x52), K with per-channel offset std 2", "flops": fl2,
                "modes": {m: {"forward_ms": r["forward_ms"], "prepare_ms": r["prepare_ms"],
                              "tflops": fl2 / (r["forward_ms"] * 1e-3) / 1e12,
                              "frac_of_mode_peak": fl2 / (r["forward_ms"] * 1e-3) / 1e12 / mode_peak(m, peak16)} for m, r in k2.items()}}
        sweep = {"M": GRID_720P[0] * GRID_720P[1] * GRID_720P[2],
                 "rows": linear_sweep(ops, GRID_720P[0] * GRID_720P[1] * GRID_720P[2], dev, peak8, hbm)}

    # roofline of the dominant kernel (attention forward), from the live CUDA-event trace
    calls, att_ms, metas = trace.get("attn_forward", (0, 0.0, []))
    att_flops = sum(4.0 * m[0] * m[1] * m[2] * m[3] * HEAD_DIM for m in metas)
    achieved = att_flops / (att_ms * 1e-3) / 1e12 if att_ms > 0 else None
    peak = mode_peak(mode, peak16)
    # DRAM traffic per launch = compulsory operand bytes (Q and O per query row, K and V per key row, per head) times
    # the factor an ncu capture of a 40-head, 16,384-token launch measured for this mode (K/V re-reads by the other
    # query tiles hit L2; traffic grows in proportion to rows x heads)
    q_b, kv_b = {"sage": (384.0, 256.0), "int8_bf16": (384.0, 384.0), "bf16": (512.0, 512.0)}[mode]
    ncu_factor = {"sage": 0.936, "bf16": 0.975}.get(mode)
    traffic = (sum(ncu_factor * m[0] * m[1] * (q_b * m[2] + kv_b * m[3]) for m in metas) / calls) if calls and ncu_factor else None
    src = {"sage": "2 x", "bf16": "1 x", "int8_bf16": "4/3 x"}[mode]
    roofline = {"bound": "tensor", "kernel": f"attn_fwd_kernel<{mode}>", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak if achieved else None, "traffic": traffic,
                "peak_source": f"{src} {peak_kind} sustained bf16 tensor rate ({MODE_NAMES[mode]} operands)",
                "frac_of_8bit_peak": achieved / peak8 if achieved else None,
                "launches": calls, "avg_launch_ms": att_ms / calls if calls else None,
                "share_of_step": att_ms / (ms_step * args.steps) if calls else None}
    breakdown = {k: {"calls": c, "ms_per_step": tms / args.steps} for k, (c, tms, _) in trace.items()}

    cpu = None
    if not args.no_cpu_baseline:
        ms, threads, sample = cpu_step_ms(tokens, args.workload, args.linear)
        cpu = {"value": ms, "unit": "ms", "cores": threads, "kind": "port", "sample": sample}

    att_modes = {m: {"ms_per_step": mode_steps.get(m), "attention_kernel_ms_one_layer": kernel_ms[m]["forward_ms"],
                     **parity[m]} for m in MODES}
    lin_name = "fp8" if args.linear == "fp8" else "int8"
    line = {"metric": metric_name(args.workload, grid), "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": f"{MODE_NAMES[mode]} attention + {lin_name} linears (fp32 accumulate)", "data": "synthetic",
            "config": workload_config(world, args.workload, grid, tokens, args.linear, mode) if full else
            {"workload": f"REDUCED profiling case ({args.workload}): {layers} layers, {tokens} tokens, {mode} attention"},
            "tflops": flops_per_step(tokens, args.workload) * layers / LAYERS / (ms_step * 1e-3) / 1e12,
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "parity": {"mode": mode, **parity[mode], **parity_info},
            "attention_mode_choice": ("fastest mode whose parity passes" if args.attention_mode == "auto" else "given on the command line"),
            "attention_modes": att_modes, "kernel_ms_per_step": breakdown}
    if parity_sp is not None:
        line["parity_sp"] = parity_sp
    if overlap is not None:
        line["overlap"] = overlap
    if cfg2 is not None:
        line["standalone_attention"] = cfg2
    if sweep is not None:
        line["linear_sweep"] = sweep
    if loop is not None:
        line["denoise_loop"] = loop
    print(json.dumps(line), flush=True)
    if sp:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

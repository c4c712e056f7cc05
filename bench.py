#!/usr/bin/env python
"""Benchmark of the decode hot paths on B200: one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (benchmark configuration 1, the configuration the metric is quoted on): the fused Mamba2
MX8 state update at batch 8 per GPU, 128 heads x 64 x 128 state, 8 B/C groups, stochastic
rounding, for the 24 Mamba2 layers of one Nemotron-H-8B decode step.  One "step" = those 24
per-layer launches over 24 distinct layer states (453 MB of packed state per step, larger than
the 126 MB L2, so no launch finds its state cached from the previous step).

  value     algorithmic GB/s over all ranks, operands resident in HBM (18 B per 16-value block,
            read + written)
  e2e       the same metric through the public Python API with the step's x / dt / B / C copied
            from pinned host memory and y copied back, all inside the timed region: prepared
            launches (MxUpdatePlan) and the copies, in four pieces of six layers on their own
            streams, replayed as one CUDA graph per step (`e2e.per_call` is the plain
            mx_state_selective_update call per layer)
  roofline  the MX8 update kernel against the measured HBM copy bandwidth
  sweep     larger shapes of the same kernels (MX8 / MX4 at batch 256, INT4-KV decode attention
            cells), each as algorithmic GB/s and fraction of the measured peak

Ranks shard the batch (weak scaling: batch 8 per GPU) and exchange nothing on the hot path;
torch.distributed carries only the barrier and the max-over-ranks of the timings.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
# The JSON line is the LAST line of stdout.  NCCL's log level is left as the environment sets it (a
# launcher that asks for NCCL_DEBUG=INFO gets its rank / transport lines, on stdout or in NCCL_DEBUG_FILE);
# only when nothing is set is the banner a system-wide nccl.conf might ask for kept quiet.
os.environ.setdefault("NCCL_DEBUG", "WARN")

HEADS, DIM, DSTATE, GROUPS, LAYERS = 128, 64, 128, 8, 24
MX8_BYTES_PER_SEQ_LAYER = HEADS * DIM * (DSTATE // 16) * 18 * 2  # 2,359,296
MX4_BYTES_PER_SEQ_LAYER = HEADS * DIM * (DSTATE // 16) * 10 * 2  # 1,310,720
BF16_BYTES_PER_SEQ_LAYER = HEADS * DIM * DSTATE * 2 * 2  # 4,194,304
FALLBACK_HBM_GBS = 6650.0


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def attn_bytes(batch: int, ctx: int, gs: int = 32, hkv: int = 8, hq: int = 32, d: int = 128) -> int:
    row = d // 2 * 2 + 2 * 4 * (d // gs)  # K + V codes and scales of one token of one kv head
    return batch * (hkv * ctx * row + hkv * row + 2 * hkv * d * 2 + 2 * hq * d * 2)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled every 200 ms while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            sm.sort()
            self.result = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


REFERENCE_ARM_MAX_STEPS = 30


def reference_arm(args, rank: int, world: int) -> int:
    """The CPU arm: the hot path of this workload on the box's host cores.  The reference has no CPU
    code for the fused update (its Triton kernels need a GPU; the interpreter is an oracle, not a
    timing baseline), so what runs here is the oracle's numpy restatement of its kernel: kind "port".
    One timed step = ONE of the step's 24 layers (`layers_timed`); `ms_per_step` is the time of that
    one-layer sample, `value` its algorithmic GB/s."""
    if rank != 0:
        return 0
    import oracle.timing as ot
    cores = os.cpu_count() or 1
    batch = args.batch_per_gpu
    steps = max(1, min(args.steps, REFERENCE_ARM_MAX_STEPS))
    warmup = max(0, min(args.warmup, 3))
    for _ in range(warmup):
        ot.time_mx_update(batch, 8, threads=cores)
    times, draws = [], []
    for _ in range(steps):
        sec, used, nbytes, draw = ot.time_mx_update(batch, 8, threads=cores)
        times.append(sec)
        draws.append(draw)
    sec = sum(times) / len(times)
    value = nbytes / sec / 1e9
    sample = (f"one of the step's 24 layers per timed step (batch {batch}, {nbytes} algorithmic bytes), numpy port of the "
              f"reference kernel, {used} threads over (sequence, group) pieces")
    line = {
        "impl": "reference", "metric": "mx8_state_update_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "layers_timed": 1, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus, batch, "reference"),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": used, "kind": "port", "sample": sample,
                         "philox_draw_share": sum(draws) / sum(times)},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "max_steps": REFERENCE_ARM_MAX_STEPS,
        "note": "kind=port: a numpy restatement, NOT the reference's own code (which is Triton and needs a GPU; its kernels are "
                "timed on the GPU in the sweep's triton_ref_* cells of the default arm).  A timed step is one layer, not the "
                "24-layer step; the port always draws the reference's Philox stream (one block per value), and "
                "philox_draw_share of its time goes into that draw.",
    }
    print(json.dumps(line), flush=True)
    return 0


def triton_reference_cells(dev, peak: float) -> dict:
    """The reference's own Triton kernels (unmodified, from baseline/_ref) compiled for and timed on this GPU,
    with the same algorithmic byte counts as the library's cells.  A missing copy, a missing Triton or a
    failure of the reference's code is reported in place of the numbers, never raised."""
    try:
        from baseline import reference, triton_cells as tc
        if not reference.available():
            return {"triton_ref": {"unavailable": "baseline/_ref is empty (python baseline/reference.py --from <Layer_Quant checkout>)"}}
        import triton
        ria, rmk = reference.load()
    except Exception as exc:
        return {"triton_ref": {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}}
    import torch
    out = {"triton_ref": {"triton": triton.__version__, "source": "baseline/_ref (unmodified phcool/Layer_Quant hybrid_quant/)",
                          "note": "cache.step held fixed so the per-step recompile of the MX kernels is excluded (mx8_rejit_ms)"}}

    def cell(name, fn):
        try:
            r = fn()
            if "GBps" in r:
                r["frac_of_hbm_peak"] = round(r["GBps"] / peak, 5)
            out[name] = r
        except Exception as exc:
            out[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        torch.cuda.empty_cache()

    cell("triton_ref_int4_attn_b1_ctx1024_gs32", lambda: tc.decode_attention_cell(ria, 1, 1024, 32, dev))        # configuration 0
    cell("triton_ref_int4_attn_b8_ctx2048_gs64", lambda: tc.decode_attention_cell(ria, 8, 2048, 64, dev))        # the published shape
    cell("triton_ref_int4_attn_b16_ctx8192_gs32", lambda: tc.decode_attention_cell(ria, 16, 8192, 32, dev))
    cell("triton_ref_int4_attn_b64_ctx32768_gs32", lambda: tc.decode_attention_cell(ria, 64, 32768, 32, dev, iters=2))
    cell("triton_ref_mx8_update_b8", lambda: tc.mx8_update_cell(rmk, 8, LAYERS, dev, rejit=True))                # configuration 1
    cell("triton_ref_mx8_update_b256", lambda: tc.mx8_update_cell(rmk, 256, 4, dev))
    cell("triton_ref_mx4_update_b64", lambda: tc.mx4_update_cell(rmk, 64, 4, dev))                               # configuration 3
    cell("triton_ref_mx4_update_b256", lambda: tc.mx4_update_cell(rmk, 256, 2, dev))
    return out


def workload_config(n_gpus: int, batch_per_gpu: int, rng: str = "reference") -> dict:
    return {
        "workload": "benchmark configuration 1: Mamba2 MX8 state update, one Nemotron-H-8B decode step = 24 layers",
        "batch_per_gpu": batch_per_gpu, "global_batch": batch_per_gpu * n_gpus, "heads": HEADS, "head_dim": DIM, "d_state": DSTATE,
        "bc_groups": GROUPS, "layers_per_step": LAYERS, "state_format": "MX8 packed (18 B / 16-value block)",
        "rounding": f"stochastic, Philox4x32-10, {rng} stream, seed 0", "parallelism": f"batch-sharded dp{n_gpus}, no collective",
        "l2": "24 distinct layer states per step (453 MB per GPU) exceed the 126 MB L2; no flush needed",
    }


def model_case(args, dev, rank, world, quiet=False):
    """benchmark configuration 4 in this repository's terms: a random-init Nemotron-H-8B-shaped model (the stand-in of
    tests/models/nemotron_h_shim; projections, norms and MLP are torch library calls) reads a ``--model-prompt``-token
    random prompt and decodes ``--model-steps`` teacher-forced random tokens, ``--case-batch`` sequences per rank:
    first unpatched (bf16 KV cache, bf16 SSM state through the library's dense-state kernel), then with INT4 KV
    (group 32) + MX8 state on every Mamba2 layer.  BOTH arms replay their decode step from one CUDA graph (the bf16
    arm on pre-sized K / V buffers), so the two differ only in the cache / state formats and their kernels.
    Returns (and prints unless ``quiet``) tokens/s of both arms and the KL divergence of the logits at the checkpoints."""
    import torch
    import torch.distributed as dist
    from layer_quant_b200 import _lib, int4_8b_attention as ia, mamba_state_8b_kernel as mk, sharding
    from tests.models.nemotron_h_shim import modeling_nemotron_h_shim as shim
    cfg = shim.nemotron_h_8b_config() if args.model_shape == "8b" else shim.tiny_config()
    bm, prompt, steps = args.model_batch, args.model_prompt, args.model_steps
    checkpoints = [c for c in (128, 256, 512, 1024, 2048) if c <= steps] or [steps]
    torch.manual_seed(0)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = shim.NemotronHShimForCausalLM(cfg)
    torch.set_default_dtype(old)
    with torch.no_grad():
        for prm in model.parameters():
            if prm.dim() > 1:
                prm.normal_(0.0, 0.02)
    model.eval()
    nparams = sum(prm.numel() for prm in model.parameters())
    ids = torch.randint(0, cfg.vocab_size, (bm, prompt + steps + 1), generator=torch.Generator().manual_seed(100 + rank)).to(dev)
    mamba_layers = [i for i, kind in enumerate(cfg.hybrid_override_pattern) if kind == "M"]

    def timed_region(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sharding.barrier()
        torch.cuda.synchronize(dev)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(dev)
        sharding.barrier()
        return sharding.all_reduce_max(e0.elapsed_time(e1) / 1e3, dev)

    def decode(quantised):
        shim._mamba_decode_state_kernel_caches = {}
        cache = shim.HybridMambaAttentionDynamicCache(cfg, bm, torch.bfloat16, device=dev)
        kept = {}
        token = torch.zeros((bm, 1), dtype=ids.dtype, device=dev)
        position = torch.zeros((1,), dtype=torch.long, device=dev)
        with torch.inference_mode():
            model(ids[:, :prompt], cache_params=cache, cache_position=torch.arange(prompt, device=dev), logits_to_keep=1)
            if quantised:
                mk.register_mamba_state_kernel_caches(model, cache, {i: "mx8" for i in mamba_layers})
                ia.prepare_graph_decode(cache, prompt + steps)
                mk.prepare_graph_decode(model)
                step_model = lambda: model(token, cache_params=cache)
            else:
                cache.presize_kv(prompt + steps)
                step_model = lambda: model(token, cache_params=cache, cache_position=position)
            token.copy_(ids[:, prompt:prompt + 1])
            position.fill_(prompt)
            first = step_model().logits[:, -1].float()  # step 1, eager (also warms every library up)
            if 1 in checkpoints:
                kept[1] = first
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_logits = step_model().logits

            def run():
                for st in range(1, steps):
                    token.copy_(ids[:, prompt + st:prompt + st + 1])
                    position.fill_(prompt + st)
                    graph.replay()
                    if st + 1 in checkpoints:
                        kept[st + 1] = static_logits[:, -1].float().clone()
            sec = timed_region(run)
        del graph
        return sec, steps - 1, kept

    sec_base, n_base, logits_base = decode(False)
    ia.patch_nemotron_h_attention_int4_kv(model, group_size=32)
    mk.patch_nemotron_h_mamba_decode_state_kernel(model, 16, stochastic=True, seed=0, rng_stream=args.rng)
    sec_q, n_q, logits_q = decode(True)
    status = _lib.device_status()
    kl = {}
    for c in checkpoints:
        lp, lq = torch.log_softmax(logits_base[c], -1), torch.log_softmax(logits_q[c], -1)
        v = (lp.exp() * (lp - lq)).sum(-1).mean()
        if world > 1:
            dist.all_reduce(v)
            v = v / world
        kl[str(c)] = float(v)
    result = {
        "case": "model", "shape": args.model_shape, "params": nparams, "n_gpus": world, "batch_per_gpu": bm,
        "global_batch": bm * world, "prompt": prompt, "decode_steps": steps,
        "tokens_per_s": bm * world * n_q / sec_q, "ms_per_step": sec_q / n_q * 1e3,
        "tokens_per_s_bf16": bm * world * n_base / sec_base, "ms_per_step_bf16": sec_base / n_base * 1e3,
        "kl_bf16_vs_quantised_at_step": kl, "device_status": status, "rng_stream": args.rng,
        "note": "INT4 KV (group 32) + MX8 state on all 24 Mamba2 layers against the same model with bf16 KV and bf16 state; both "
                "arms replay one CUDA graph per decode step; random-init weights ~N(0, 0.02), teacher-forced random tokens; "
                "projections / norms / MLP are torch library kernels"}
    del model
    torch.cuda.empty_cache()
    if rank == 0 and not quiet:
        print(json.dumps(result), flush=True)
    return result


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch-per-gpu", type=int, default=8)
    ap.add_argument("--rng", default="layered", choices=["reference", "layered", "layered4"],
                    help="random stream of the headline number (both are always reported)")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--model-prompt", type=int, default=1024, help="--case model: prompt length")
    ap.add_argument("--model-steps", type=int, default=0, help="model case: decode steps (default 2048 with --case model, 256 inside the default line)")
    ap.add_argument("--model-shape", default="8b", choices=["8b", "tiny"], help="--case model: Nemotron-H-8B shape or the test shape")
    ap.add_argument("--case", default="", choices=["", "mx8", "mx4", "attn", "bf16", "model"],
                    help="run only one small kernel case (for ncu captures): plain launches, no graph, no sweep")
    ap.add_argument("--case-batch", type=int, default=64)
    ap.add_argument("--model-batch", type=int, default=32, help="model case: sequences per GPU")
    ap.add_argument("--no-model", action="store_true", help="leave the model case (benchmark configuration 4) out of the default line")
    ap.add_argument("--case-ctx", type=int, default=8192)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-triton-ref", action="store_true", help="skip the sweep's triton_ref_* cells (the reference's kernels on this GPU)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return reference_arm(args, rank, world)

    import numpy as np
    import torch
    from layer_quant_b200 import int4_8b_attention as ia
    from layer_quant_b200 import mamba_state_8b_kernel as mk
    from layer_quant_b200 import sharding

    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl ours needs a CUDA device (there is no CPU path)")
    rank, local_rank, world = sharding.init_from_env()
    dev = torch.device("cuda", local_rank)
    B = args.batch_per_gpu
    peak, peak_src = hbm_peak()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def randn(*shape, dtype=torch.bfloat16):
        return torch.randn(shape, generator=gen, device=dev, dtype=torch.float32).to(dtype)

    # ---- per-layer states and operands (config 1 distributions) -------------------------------------
    def make_layers(batch, n_layers, bits):
        layers = []
        for li in range(n_layers):
            cache = mk.allocate_state_kernel_cache(randn(batch, HEADS, DIM, DSTATE, dtype=torch.float32) * 0.5, 16, bits)
            cache.layer = li
            ops = dict(
                x=randn(batch, HEADS, DIM), dt=randn(batch, HEADS)[:, :, None].expand(batch, HEADS, DIM),
                A=(-torch.exp(torch.rand(HEADS, generator=gen, device=dev) * float(np.log(16.0))))[:, None, None].expand(HEADS, DIM, DSTATE),
                B=randn(batch, GROUPS, DSTATE), C=randn(batch, GROUPS, DSTATE),
                D=torch.rand(HEADS, generator=gen, device=dev)[:, None].expand(HEADS, DIM),
                dt_bias=(torch.rand(HEADS, generator=gen, device=dev) * 2.0 - 4.0)[:, None].expand(HEADS, DIM),
                out=torch.empty((batch, HEADS, DIM), device=dev, dtype=torch.bfloat16))
            layers.append((cache, ops))
        return layers

    counter = torch.zeros(1, dtype=torch.int64, device=dev)  # device-side decode-step counter read by the kernels

    def make_step(layers, stream_name, graph=True):
        """The decode step's state updates as one replayable unit: 24 prepared launches plus the
        one-thread counter bump, captured in a CUDA graph (as a serving loop would replay it)."""
        plans = [mk.MxUpdatePlan(cache, o["x"], o["dt"], o["A"], o["B"], o["C"], D=o["D"], dt_bias=o["dt_bias"], dt_softplus=True,
                                 stochastic=True, seed=0, rng_stream=stream_name, out=o["out"], step_counter=counter)
                 for cache, o in layers]

        def eager():
            for p in plans:
                p.run()
            mk.advance_step_counter(counter)

        if not graph:
            return eager
        eager()
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            eager()
        g._plans = plans
        return g.replay

    def timed(fn, steps, warmup):
        """Max-over-ranks seconds for `steps` calls of fn, CUDA events on the launching stream."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize(dev)
        sharding.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        sharding.barrier()
        return sharding.all_reduce_max(e0.elapsed_time(e1) / 1e3, dev)

    if args.case == "model":
        args.model_steps = args.model_steps or 2048
        model_case(args, dev, rank, world)
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return 0
    if args.case:
        # one kernel, a few plain launches on a working set larger than L2 and at most a few GB
        cb = args.case_batch
        if args.case == "attn":
            ctx = args.case_ctx
            c = ia._allocate_layer_cache(cb, 8, ctx, 128, 4, dev)
            for tns in (c.k_packed, c.v_packed):
                tns.copy_(torch.randint(0, 256, tns.shape, generator=gen, device=dev, dtype=torch.int16).to(torch.uint8))
            for tns in (c.k_scale, c.v_scale):
                tns.copy_(torch.rand(tns.shape, generator=gen, device=dev) * 0.4 + 0.1)
            q, kn, vn = randn(cb, 32, 1, 128), randn(cb, 8, 1, 128), randn(cb, 8, 1, 128)
            plan = ia.Int4DecodePlan(q, c, ctx, 32, k_new=kn, v_new=vn)
            fn = plan.launch
            nbytes = attn_bytes(cb, ctx)
        elif args.case == "bf16":
            from layer_quant_b200 import dense_state
            st = torch.randn(cb, HEADS, DIM, DSTATE, generator=gen, device=dev).mul_(0.5).to(torch.bfloat16)
            o = make_layers(cb, 1, 8)[0][1]
            fn = lambda: dense_state.selective_state_update(st, o["x"], o["dt"], o["A"], o["B"], o["C"], D=o["D"], dt_bias=o["dt_bias"],
                                                            dt_softplus=True, out=o["out"])
            nbytes = BF16_BYTES_PER_SEQ_LAYER * cb
        else:
            bits = 8 if args.case == "mx8" else 4
            lay = make_layers(cb, 1, bits)
            fn = make_step(lay, args.rng, graph=False)
            nbytes = (MX8_BYTES_PER_SEQ_LAYER if bits == 8 else MX4_BYTES_PER_SEQ_LAYER) * cb
        sec = timed(fn, args.steps, args.warmup)
        print(json.dumps({"case": args.case, "batch": cb, "ctx": args.case_ctx if args.case == "attn" else None, "rng": args.rng,
                          "us_per_launch": sec / args.steps * 1e6, "GBps": nbytes * args.steps / sec / 1e9,
                          "frac_of_hbm_peak": nbytes * args.steps / sec / 1e9 / peak}), flush=True)
        return 0

    layers8 = make_layers(B, LAYERS, 8)
    bytes_step = MX8_BYTES_PER_SEQ_LAYER * B * LAYERS

    results = {}
    head_step = make_step(layers8, args.rng)
    other = "reference" if args.rng == "layered" else "layered"
    with ClockSampler(local_rank) as clocks:
        results[args.rng] = timed(head_step, args.steps, args.warmup)  # the headline: exactly --steps steps
        # The same step repeated for about a second (SUSTAINED_STEPS is fixed from the short run's rate), so that the
        # 200 ms clock samples fall inside a timed region and an issue-bound kernel's clock is on record.
        sustained_steps = int(min(20000, max(args.steps, 1.0 / max(results[args.rng] / args.steps, 1e-6))))
        sustained_sec = timed(head_step, sustained_steps, 0)
    results[other] = timed(make_step(layers8, other), args.steps, args.warmup)
    results["layered4"] = timed(make_step(layers8, "layered4"), args.steps, args.warmup)
    eager_sec = timed(make_step(layers8, args.rng, graph=False), args.steps, args.warmup)
    sec = results[args.rng]
    value = bytes_step * world * args.steps / sec / 1e9
    ms_per_step = sec / args.steps * 1e3
    per_launch_s = sec / (args.steps * LAYERS)
    achieved = MX8_BYTES_PER_SEQ_LAYER * B / per_launch_s / 1e9

    # ---- end to end: host buffers in, host buffer out, through the reference's own call signature ----------
    # Every variant calls mx_state_selective_update(cache, x, dt, A, B, C, D=, dt_bias=, dt_softplus=) once per layer, as
    # the reference's decode loop does.  The step's x / dt / B / C of all layers sit in ONE pinned host buffer.
    #   e2e           the 24 calls and the copies recorded once in a CUDA graph (the caches in graph mode: their step lives
    #                 in a device counter, prepare_graph_decode's mechanism) and replayed per step: copies in four pieces of
    #                 six layers on a copy stream, each piece's outputs copied back on a third stream
    #   e2e.per_call  the same calls launched eagerly every step (one host-to-device copy per layer in, one out)
    #   e2e.prepared  the graph built from prepared launches (MxUpdatePlan) that share one step counter: what the call
    #                 itself costs beyond the kernel is the difference
    shapes = (("x", (B, HEADS, DIM)), ("dt", (B, HEADS)), ("B", (B, GROUPS, DSTATE)), ("C", (B, GROUPS, DSTATE)))
    per_layer = sum(int(np.prod(sh)) for _, sh in shapes)
    host_all = torch.randn(LAYERS * per_layer).to(torch.bfloat16).pin_memory()
    dev_all = torch.empty(LAYERS * per_layer, dtype=torch.bfloat16, device=dev)
    out_all = torch.empty((LAYERS, B, HEADS, DIM), dtype=torch.bfloat16, device=dev)
    host_out_all = torch.empty((LAYERS, B, HEADS, DIM), dtype=torch.bfloat16).pin_memory()

    def views(flat, li):
        off, d = li * per_layer, {}
        for k, sh in shapes:
            n = int(np.prod(sh))
            d[k] = flat[off:off + n].view(sh)
            off += n
        return d

    h2d = host_all.numel() * host_all.element_size()
    d2h = host_out_all.numel() * host_out_all.element_size()
    e2e_layers = []
    for li, (cache, o) in enumerate(layers8):
        di = views(dev_all, li)
        e2e_layers.append((cache, dict(o, x=di["x"], dt=di["dt"][:, :, None].expand(B, HEADS, DIM), B=di["B"], C=di["C"], out=out_all[li])))

    def call_layer(cache, o):
        return mk.mx_state_selective_update(cache, o["x"], o["dt"], o["A"], o["B"], o["C"], D=o["D"], dt_bias=o["dt_bias"],
                                            dt_softplus=True, stochastic=True, seed=0, rng_stream=args.rng, out=o["out"])

    # The step's operands travel in E2E_CHUNKS pieces, and each piece's outputs leave as soon as its launches are done (in
    # the recorded forms on a copy stream and a third stream, overlapping the compute).
    E2E_CHUNKS = int(os.environ.get("LQ_BENCH_E2E_CHUNKS", "4"))  # tuning aid; must divide the 24 layers
    lpc = LAYERS // E2E_CHUNKS

    def e2e_per_call_step():
        for c in range(E2E_CHUNKS):
            lo, hi = c * lpc * per_layer, (c + 1) * lpc * per_layer
            dev_all[lo:hi].copy_(host_all[lo:hi], non_blocking=True)
            for li in range(c * lpc, (c + 1) * lpc):
                call_layer(*e2e_layers[li])
            host_out_all[c * lpc:(c + 1) * lpc].copy_(out_all[c * lpc:(c + 1) * lpc], non_blocking=True)

    sec_e2e_call = timed(e2e_per_call_step, args.steps, args.warmup)

    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_graph_of(launch_layer, after_step):
        def body():
            main = torch.cuda.current_stream(dev)
            s_in.wait_stream(main)
            s_out.wait_stream(main)
            for c in range(E2E_CHUNKS):
                lo, hi = c * lpc * per_layer, (c + 1) * lpc * per_layer
                with torch.cuda.stream(s_in):
                    dev_all[lo:hi].copy_(host_all[lo:hi], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(s_in)
                main.wait_event(ev)
                for li in range(c * lpc, (c + 1) * lpc):
                    launch_layer(li)
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    host_out_all[c * lpc:(c + 1) * lpc].copy_(out_all[c * lpc:(c + 1) * lpc], non_blocking=True)
            after_step()
            main.wait_stream(s_in)
            main.wait_stream(s_out)

        body()
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            body()
        return g

    e2e_plans = [mk.MxUpdatePlan(cache, o["x"], o["dt"], o["A"], o["B"], o["C"], D=o["D"], dt_bias=o["dt_bias"], dt_softplus=True,
                                 stochastic=True, seed=0, rng_stream=args.rng, out=o["out"], step_counter=counter)
                 for cache, o in e2e_layers]
    g_prepared = e2e_graph_of(lambda li: e2e_plans[li].run(), lambda: mk.advance_step_counter(counter))
    sec_e2e_prepared = timed(g_prepared.replay, args.steps, args.warmup)
    del g_prepared
    # graph mode of the public call, set up as for a model: the caches share one device counter, which the last layer's
    # call advances on the stream
    from types import SimpleNamespace
    mk.prepare_graph_decode(SimpleNamespace(_mamba_decode_state_kernel_caches={id(c): c for c, _ in e2e_layers}))
    g_calls = e2e_graph_of(lambda li: call_layer(*e2e_layers[li]), lambda: None)
    e2e_step = g_calls.replay
    sec_e2e = timed(e2e_step, args.steps, args.warmup)
    e2e_value = bytes_step * world * args.steps / sec_e2e / 1e9

    # ---- sweep: the larger shapes of the same kernels -----------------------------------------------------
    sweep = {}
    if not args.no_sweep:
        del layers8
        torch.cuda.empty_cache()
        for bits, per_seq in ((8, MX8_BYTES_PER_SEQ_LAYER), (4, MX4_BYTES_PER_SEQ_LAYER)):
            big = make_layers(256, 4, bits)
            for name in ("reference", "layered4", "layered"):
                s = timed(make_step(big, name), 5, 3)
                gbs = per_seq * 256 * 4 * 5 / s / 1e9
                sweep[f"mx{bits}_update_b256_{name}_stream"] = {"GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4),
                                                               "us_per_launch": round(s / 20 * 1e6, 1)}
            del big
            torch.cuda.empty_cache()
        # benchmark configuration 3: the MX4 update at batch 64 / 256 / 1024 x the step's 24 layers (library stream), and the
        # BF16 state it is compared with (24 layers where they fit beside everything else, 4 at batch 1024: 8.6 GB,
        # still far larger than L2)
        for bb in (64, 256, 1024):
            big = make_layers(bb, LAYERS, 4)
            s = timed(make_step(big, "layered"), 3, 3)
            gbs = MX4_BYTES_PER_SEQ_LAYER * bb * LAYERS * 3 / s / 1e9
            sweep[f"mx4_update_b{bb}_x24_layered_stream"] = {"GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4),
                                                             "us_per_launch": round(s / (3 * LAYERS) * 1e6, 1),
                                                             "ms_per_24_layer_step": round(s / 3 * 1e3, 3)}
            del big
            torch.cuda.empty_cache()
        from layer_quant_b200 import dense_state
        for bb in (64, 256, 1024):
            nlay = LAYERS if bb < 1024 else 4
            states = [torch.randn(bb, 128, 64, 128, generator=gen, device=dev).mul_(0.5).to(torch.bfloat16) for _ in range(nlay)]
            ops = make_layers(bb, 1, 8)[0][1]
            def dense_step():
                for st in states:
                    dense_state.selective_state_update(st, ops["x"], ops["dt"], ops["A"], ops["B"], ops["C"], D=ops["D"],
                                                       dt_bias=ops["dt_bias"], dt_softplus=True, out=ops["out"])
            s = timed(dense_step, 3, 3)
            gbs = BF16_BYTES_PER_SEQ_LAYER * bb * nlay * 3 / s / 1e9
            sweep[f"bf16_state_update_b{bb}"] = {"GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4),
                                                 "us_per_launch": round(s / (3 * nlay) * 1e6, 1), "layers": nlay}
            del states, ops
            torch.cuda.empty_cache()
        # benchmark configuration 2: batch {1, 16, 64, 256} x context {1k, 8k, 32k, 128k} (the largest cell holds 42.9 GB
        # of cache), plus (8, 32k)
        cells = [(bb, ctx) for bb in (1, 16, 64, 256) for ctx in (1024, 8192, 32768, 131072)] + [(8, 32768)]
        for (bb, ctx) in cells:
            cap = ctx
            reps = max(1, int(np.ceil(4 * 126e6 / attn_bytes(bb, ctx))))  # distinct caches: >= 4x L2 in rotation
            reps = min(reps, 64)
            caches = []
            for _ in range(reps):
                c = ia._allocate_layer_cache(bb, 8, cap, 128, 4, dev)
                c.k_packed.random_(0, 256, generator=gen)  # in place: the largest cell has no room for temporaries
                c.v_packed.random_(0, 256, generator=gen)
                c.k_scale.uniform_(0.1, 0.5, generator=gen)
                c.v_scale.uniform_(0.1, 0.5, generator=gen)
                caches.append(c)
            q = randn(bb, 32, 1, 128)
            kn, vn = randn(bb, 8, 1, 128), randn(bb, 8, 1, 128)

            # prepared launches, one per cache of the rotation, replayed from a CUDA graph: small cells are
            # otherwise bound by the host's call overhead, not by the kernel
            plans = [ia.Int4DecodePlan(q, c, ctx, 32, k_new=kn, v_new=vn) for c in caches]
            plans[0].launch()
            torch.cuda.synchronize(dev)
            attn_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(attn_graph):
                for pl in plans:
                    pl.launch()
            s = timed(attn_graph.replay, 5, 3)
            del attn_graph, plans
            gbs = attn_bytes(bb, ctx) * reps * 5 / s / 1e9
            sweep[f"int4_attn_b{bb}_ctx{ctx}"] = {"GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4),
                                                  "us_per_launch": round(s / (5 * reps) * 1e6, 1)}
            del caches
            torch.cuda.empty_cache()
        # Yardstick for short launches: a plain device-to-device copy (library code, not the product) moving the same
        # number of bytes (read + written) as one launch of the cells above, replayed from a CUDA graph over buffers
        # that rotate through more than 4x L2.  The HBM peak in the roofline is a long copy; a launch of 19 MB or 151 MB
        # does not reach it whatever the kernel, and these cells say how far such a launch can get.
        for label, total in (("19MB_config1_launch", MX8_BYTES_PER_SEQ_LAYER * 8), ("151MB", attn_bytes(16, 8192)),
                             ("302MB", attn_bytes(8, 32768)), ("1208MB", attn_bytes(64, 16384))):
            words = (total // 2 + 15) // 16 * 4  # int32 words per buffer; one launch reads and writes this much
            reps = min(64, max(2, int(np.ceil(4 * 126e6 / total))))
            srcs = [torch.empty(words, dtype=torch.int32, device=dev).random_(0, 1 << 20, generator=gen) for _ in range(reps)]
            dsts = [torch.empty(words, dtype=torch.int32, device=dev) for _ in range(reps)]
            entry = {"bytes_read_plus_written": 8 * words}
            # "memcpy": cudaMemcpyAsync between device buffers; "elementwise": torch's vectorised add-one kernel on the SMs
            for kind, op in (("memcpy", lambda d_, s_: d_.copy_(s_)), ("elementwise", lambda d_, s_: torch.add(s_, 1, out=d_))):
                op(dsts[0], srcs[0])
                torch.cuda.synchronize(dev)
                copy_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(copy_graph):
                    for s_, d_ in zip(srcs, dsts):
                        op(d_, s_)
                s = timed(copy_graph.replay, 5, 3)
                gbs = 8 * words * reps * 5 / s / 1e9
                entry[kind] = {"GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4), "us_per_launch": round(s / (5 * reps) * 1e6, 1)}
                del copy_graph
            sweep[f"copy_yardstick_{label}"] = entry
            del srcs, dsts
            torch.cuda.empty_cache()
        # prefill over the quantised cache (the step before decode): a 1024-token prompt, 8 sequences, one layer,
        # beside torch's fused attention over the un-quantised bf16 K / V (what the forward uses by default)
        import torch.nn.functional as F
        bb, tq = 8, 1024
        c = ia._allocate_layer_cache(bb, 8, tq, 128, 4, dev)
        kk, vv = randn(bb, 8, tq, 128), randn(bb, 8, tq, 128)
        ia._pack_kv_into_cache(c, kk, vv, torch.arange(tq, device=dev), 32)
        qq = randn(bb, 32, tq, 128)
        pre_out = torch.empty_like(qq)
        s = timed(lambda: ia._prefill_attention(qq, c, 4, 32, out=pre_out), 5, 3)
        kf, vf = kk.repeat_interleave(4, dim=1), vv.repeat_interleave(4, dim=1)
        s2 = timed(lambda: F.scaled_dot_product_attention(qq, kf, vf, is_causal=True), 5, 3)
        sweep["int4_prefill_b8_q1024"] = {"us_per_launch": round(s / 5 * 1e6, 1), "torch_sdpa_bf16_us": round(s2 / 5 * 1e6, 1),
                                          "cache_bytes_read": int(bb * 8 * 160 * sum(min(i + 8, tq) for i in range(0, tq, 8)))}
        del c, kk, vv, qq, kf, vf, pre_out
        torch.cuda.empty_cache()
        if rank == 0 and world == 1 and not args.no_triton_ref:
            sweep.update(triton_reference_cells(dev, peak))
        if rank == 0 and not args.no_cpu_baseline:
            # benchmark configuration 0 on the host cores, the reference's own CPU-runnable path: torch fake-quant of K / V
            # (int4_quant_dequant, group 32) + scaled_dot_product_attention, batch 1, 1024 tokens; beside it the
            # (1, 1024) cell above is the same problem on the GPU.
            import time
            gq = torch.Generator().manual_seed(0)
            q0 = torch.randn(1, 32, 1, 128, generator=gq).to(torch.bfloat16)
            k0, v0 = (torch.randn(1, 8, 1024, 128, generator=gq).to(torch.bfloat16) for _ in range(2))

            def cpu_config0():
                kq = ia.int4_quant_dequant(k0, 32).repeat_interleave(4, dim=1)
                vq = ia.int4_quant_dequant(v0, 32).repeat_interleave(4, dim=1)
                return F.scaled_dot_product_attention(q0, kq, vq)

            for _ in range(3):
                cpu_config0()
            t0 = time.perf_counter()
            for _ in range(20):
                cpu_config0()
            cpu_ms = (time.perf_counter() - t0) / 20 * 1e3
            sweep["config0_int4_attn_b1_ctx1024_cpu_torch"] = {"ms_per_call": round(cpu_ms, 3), "threads": torch.get_num_threads(),
                                                               "gpu_us_per_launch": sweep["int4_attn_b1_ctx1024"]["us_per_launch"]}

    # ---- CPU baseline (rank 0, bounded sample) ----------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle.timing as ot
        csec, cores, nbytes, cdraw = ot.time_mx_update(B, 8, threads=os.cpu_count() or 1, repeats=3, layers=LAYERS)
        cpu = {"value": nbytes / csec / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
               "sample": f"the whole 24-layer step (batch {B}, {nbytes / 1e6:.1f} MB algorithmic), numpy restatement of the reference "
                         f"kernel (NOT the reference's own code), best of 3 runs, {cores} threads over (sequence, group) pieces",
               "seconds_per_step": csec,
               "philox_draw_share": cdraw / csec}

    # ---- benchmark configuration 4 at every N: the full decode step of the 8B-shaped model ---------------------------
    model = None
    if not args.no_model:
        args.model_steps = args.model_steps or 256
        try:
            model = model_case(args, dev, rank, world, quiet=True)
        except Exception as exc:  # the kernel-level line must survive a failure of the model-level case
            model = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    # DRAM bytes of one launch of the headline kernel: from the ncu capture summarised under profiles/ (a smaller
    # batch, scaled by the batch: the kernel's traffic is proportional to it)
    traffic, traffic_src = None, None
    tj = ROOT / "profiles" / "mx8_state_update_traffic.json"
    if tj.exists():
        t = json.loads(tj.read_text())
        traffic = (t["dram_bytes_read"] + t["dram_bytes_written"]) * B / t["batch"]
        traffic_src = f"profiles/{tj.name}: ncu capture at batch {t['batch']}, scaled to batch {B}"

    if rank == 0:
        line = {
            "metric": "mx8_state_update_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(world, B, args.rng),
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": sec_e2e / args.steps * 1e3,
                    "mode": "mx_state_selective_update (the reference's call signature) once per layer, caches in graph mode (one shared "
                            f"device step counter); pinned-host -> device copies of the step's x/dt/B/C in {E2E_CHUNKS} pieces of {lpc} layers on a "
                            "copy stream, device -> pinned-host copies of each piece's y on a third stream; calls and copies recorded once "
                            "in a CUDA graph, replayed per step",
                    "per_call": {"value": bytes_step * world * args.steps / sec_e2e_call / 1e9,
                                 "ms_per_step": sec_e2e_call / args.steps * 1e3,
                                 "mode": f"the same 24 calls launched eagerly every step (no graph), copies in {E2E_CHUNKS} pieces on the launching stream"},
                    "prepared": {"value": bytes_step * world * args.steps / sec_e2e_prepared / 1e9,
                                 "ms_per_step": sec_e2e_prepared / args.steps * 1e3,
                                 "mode": "the graph built from prepared launches (MxUpdatePlan) sharing one step counter"}},
            "gpu_launches": args.steps * (LAYERS + 1),  # the device-resident timed region: 24 updates + 1 counter bump per step
            "launch_mode": "24 update launches + 1 counter bump per step, replayed from a CUDA graph",
            "eager_launch": {"GBps": bytes_step * world * args.steps / eager_sec / 1e9, "ms_per_step": eager_sec / args.steps * 1e3},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_source": traffic_src, "peak_source": peak_src,
                         "kernel": f"mx_state_update_fast_kernel<8, packed, {'PHILOX_LAYERED' if args.rng == 'layered' else 'PHILOX_REF'}, 128>",
                         "algorithmic_bytes_per_launch": MX8_BYTES_PER_SEQ_LAYER * B, "us_per_launch": per_launch_s * 1e6},
            "cpu_baseline": cpu,
            "clocks": clocks.result,
            "sustained": {"steps": sustained_steps, "seconds": sustained_sec, "GBps": bytes_step * world * sustained_steps / sustained_sec / 1e9,
                          "note": "the headline step repeated for about a second inside the clock-sampled region"},
            "streams": {k: {"GBps": bytes_step * world * args.steps / v / 1e9, "ms_per_step": v / args.steps * 1e3} for k, v in results.items()},
            "sweep": sweep,
            "model": model,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

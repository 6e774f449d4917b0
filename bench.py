#!/usr/bin/env python
"""Benchmark of the MoE feed-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--rows fresh|chained] [--layers L]
                    [--launch fused|layers] [--impl ours|reference]

One step = one pass of the 40-layer Qwen3.6-A3B-shaped MoE FFN stack (hidden 2048, 256 experts top-8 + 1 shared,
intermediate 512, 4-bit group-64 affine weights, bf16 activations, RMSNorm in front of every layer) over one decode
batch of B token rows.  Weights are seeded synthetic (generated on the device) and fully resident in HBM.

--rows chained  the residual stream h <- h + MoE(RMSNorm(h)) runs through all layers (mfb_moe_stack).  With the
                configuration's all-positive synthetic weights every expert's output is close to a multiple of the
                all-ones vector, so after the first layer all rows route alike and a batch touches far fewer distinct
                experts than independent rows would.
--rows fresh    (default for B > 1) every layer gets its own N(0,1) bf16 batch, layers still run strictly one after
                the other on one stream; rows route independently as the configuration intends (about 57 distinct
                experts per layer at B = 8, 222 at B = 64).  For B = 1 both modes touch 8 experts per layer; the
                default there is chained, which keeps the true layer-to-layer dependency.

Prints ONE JSON line.  `value` is whole-job tokens/s with inputs resident in HBM; `e2e` is the same through the
C ABI with host buffers (pinned host -> device copy of the step's rows and device -> host read of the result inside
the timed region); `roofline` relates the step to the measured HBM copy bandwidth; `cpu_baseline` is the CPU port of
the reference's scalar path timed on this box's host cores (a baseline, not a target).

With --gpus N > 1 (under torchrun) every rank serves its own batch from its own full replica of the pool (decode
does not shard: replicas only), so scaling is weak and `value` sums the ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, F, E, K, LAYERS = 2048, 512, 256, 8, 40
ROOT_SEED = 0xB2000001
N_INPUTS = 4          # distinct input sets cycled through the steps
# DRAM bytes (read + write) per layer of one stack_mega_kernel launch, from ncu captures of 2-layer cases of this build
# (profiles/), keyed by (batch, rows); scaled by the layer count since every layer reads its own weights once
TRAFFIC_PER_LAYER: dict = {(64, "fresh"): 400.2e6, (8, "fresh"): 107.0e6, (1, "chained"): 17.37e6}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def layer_bytes(unique_experts: int, n_tokens: int, blob: int) -> int:
    """Algorithmic bytes of one decode layer: each distinct routed expert once, the shared expert, the bf16 gate,
    and the activation rows in and out."""
    return unique_experts * blob + blob + E * D * 2 + n_tokens * D * 2 * 2


# ----------------------------------------------------------------------------------------------- CPU arm

def cpu_port_tokens_per_s(batch: int, budget_s: float, layers: int = LAYERS):
    """Times the CPU port of the reference's scalar decode path (oracle/mfb_oracle.c: mfbo_ref_moe_layer_f32 plus the
    router) on this box's host cores, on ONE layer of the stack over the whole batch, and scales by the layer count."""
    from oracle import oracle as O
    rows = batch
    W0 = O.LayerWeights(D, F, E, K, root=ROOT_SEED, layer=0, experts=[])
    x = O.fill_normal(O.seed_for_label(ROOT_SEED, "x"), rows * D, dtype=O.DT_BF16).reshape(rows, D)
    lg = O.router_logits(x, O.DT_BF16, W0.router)
    idx, w = O.topk_softmax(lg, K)
    W = O.LayerWeights(D, F, E, K, root=ROOT_SEED, layer=0, experts=sorted(set(idx.reshape(-1).tolist())))
    xf = O.bf16_to_f32(x)
    O.ref_moe_layer_f32(W, xf, idx, w)   # warm-up
    reps, t0 = 0, time.perf_counter()
    while True:
        lg = O.router_logits(x, O.DT_BF16, W.router)
        idx2, w2 = O.topk_softmax(lg, K)
        O.ref_moe_layer_f32(W, xf, idx2, w2)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or reps >= 2000:
            break
    per_layer = dt / reps
    tok_s = rows / (per_layer * layers)
    return tok_s, O.num_threads(), f"1 of {layers} layers x {rows} token rows x {reps} repeats, scaled x{layers}"


def cpu_port_prefill_tokens_per_s(sample_rows: int, budget_s: float, zipf: bool, shape=None):
    """CPU port of the reference's scalar prefill path on a sample of the batch's rows: router, grouping by expert,
    the per-pair scalar int4 loop (oracle mfbo_pair_partials, the restatement of the reference's test-local loop) and
    the token-major weighted reduce.  Tokens/s of the sample; the cost per token row does not depend on the batch."""
    import numpy as np
    from oracle import oracle as O
    T = sample_rows
    D, F, E, K, bits, sbits = shape or (2048, 512, 256, 8, 4, 4)   # layer shape (default: the Q layer)
    W0 = O.LayerWeights(D, F, E, K, bits=bits, shared_bits=sbits, root=ROOT_SEED, layer=0, experts=[])
    x = O.fill_normal(O.seed_for_label(ROOT_SEED, "x.prefill.cpu"), T * D, dtype=O.DT_BF16).reshape(T, D)
    bias = zipf_logit_bias(E) if zipf else None
    lg = O.router_logits(x, O.DT_BF16, W0.router, logit_bias=bias)
    idx, w = O.topk_softmax(lg, K)
    W = O.LayerWeights(D, F, E, K, bits=bits, shared_bits=sbits, root=ROOT_SEED, layer=0, experts=sorted(set(idx.reshape(-1).tolist())))
    pairs = np.zeros(T * K, dtype=O.PAIR_DTYPE)
    pairs["token"] = np.repeat(np.arange(T), K)
    pairs["expert"] = idx.reshape(-1)
    pairs["rank"] = np.tile(np.arange(K), T)
    reps, t0 = 0, time.perf_counter()
    while True:
        lg = O.router_logits(x, O.DT_BF16, W.router, logit_bias=bias)
        idx2, w2 = O.topk_softmax(lg, K)
        g = O.group_pairs(pairs, T, K, E)
        part = O.pair_partials(W, x, O.DT_BF16, g["sorted_pairs"])
        full = np.empty((T * K, D), dtype=np.float32)
        sp = g["sorted_pairs"]
        full[sp["token"] * K + sp["rank"]] = part
        O.reduce_token_major(full.reshape(T, K, D), w2, T, K, D)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or reps >= 200:
            break
    return T * reps / dt, O.num_threads(), f"{T} token rows ({T * K} pairs) of one layer x {reps} repeats; tokens/s of the sample"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # under torchrun every rank is given OMP_NUM_THREADS=1; this arm is rank 0 alone and uses every host core
    try:
        from oracle import oracle as O
        O.set_num_threads(os.cpu_count() or 1)
    except Exception:
        pass
    steps, warm = max(args.steps, 1), args.warmup
    budget = max(1.0, min(15.0, 90.0 / (steps + warm)))
    vals = []
    cores, sample = 1, ""
    for i in range(steps + warm):
        tok_s, cores, sample = cpu_port_tokens_per_s(args.batch, budget, args.layers)
        if i >= warm:
            vals.append(tok_s)
    v = statistics.mean(vals)
    rows = args.batch
    print(json.dumps({
        "impl": "reference", "metric": "moe_decode_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": 1e3 * rows / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"configs[1]: {args.layers}-layer Qwen3.6-A3B MoE FFN stack, decode batch {rows}, {args.rows} rows",
                   "hidden": D, "intermediate": F, "experts": E, "top_k": K, "shared_experts": 1, "bits": 4,
                   "group_size": 64, "layers": args.layers, "batch_per_gpu": rows,
                   "note": "the reference is Swift + Metal and cannot be built here; this arm is the C port of its scalar "
                           "path (oracle/mfb_oracle.c) on the host cores, one layer timed per step and scaled by the "
                           "layer count; its tokens/s does not depend on how rows are chained between layers"},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------------------------- GPU arm

class DecodeBench:
    """The resident 40-layer pool and the decode measurements over it (configs[1])."""

    def __init__(self, args, world, rank, local):
        from mference_b200 import _lib as L
        from mference_b200.moe import expert_layout, synth_layer
        self.args, self.world, self.rank, self.local = args, world, rank, local
        self.L, self.lib = L, L.load()
        self.NL = args.layers
        _, self.blob = expert_layout(4, D, F)
        self.layers = [synth_layer(ROOT_SEED, l, D, F, E) for l in range(self.NL)]

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(self, B, rows, steps, warmup, *, launch="fused", trace=False, cpu_budget=10.0, sampler=None):
        """One decode configuration: batch B, rows 'fresh' | 'chained'.  Returns the record of the measurement."""
        import torch
        import torch.distributed as dist
        from mference_b200.moe import MoE, synth_normal
        L, lib, NL, layers, world, rank = self.L, self.lib, self.NL, self.layers, self.world, self.rank
        fresh = rows == "fresh"
        moe = MoE(D, F, E, K, max_tokens=B, max_layers=max(NL, 1))
        if launch == "layers":
            moe.set_generic(2)
        stack = moe.make_stack(layers)
        n_sets = N_INPUTS
        shape = (NL, B, D) if fresh else (B, D)
        inputs = [synth_normal(ROOT_SEED + rank, f"x.{B}.{i}", (NL if fresh else 1) * B * D, dtype=L.DT_BF16).view(*shape)
                  for i in range(n_sets)]
        torch.cuda.synchronize()

        # distinct experts per layer for each input set (untimed; same kernels, layer by layer)
        step_bytes = []
        idx = torch.empty((B, K), dtype=torch.int32, device="cuda")
        w = torch.empty((B, K), dtype=torch.float16, device="cuda")
        for h0 in inputs:
            total = 0
            h = None if fresh else h0.clone()
            for l, lw in enumerate(layers):
                src = h0[l] if fresh else h
                xn = torch.empty_like(src)
                moe.encode_rmsnorm(src, xn, lw.norm_w)
                moe.encode_router(xn, lw, idx, w)
                total += layer_bytes(int(torch.unique(idx).numel()), B, self.blob)
                if not fresh:
                    nxt = torch.empty_like(h)
                    moe.encode_decode(lw, xn, idx, w, nxt, residual=h)
                    h = nxt
            step_bytes.append(total)
        torch.cuda.synchronize()
        work = [torch.empty_like(t) for t in inputs]
        kev = []   # (start, end) events around the stack call alone

        def step(i, src=None, timed=False):
            buf = work[i % n_sets]
            if src is None:
                buf.copy_(inputs[i % n_sets])
            if timed:
                kev.append((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
                kev[-1][0].record()
            if fresh:
                moe.encode_stack_rows(stack, buf)    # layer l on rows buf[l]; strictly one layer after the other
            else:
                moe.encode_stack(stack, buf)
            if timed:
                kev[-1][1].record()
            return buf

        for i in range(warmup):
            step(i)
        self.barrier()
        if sampler is not None:
            sampler.start()
        launches0 = lib.mfb_launch_count()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        self.barrier()
        ev[0].record()
        for i in range(steps):
            step(i, timed=True)
            ev[i + 1].record()
        self.barrier()
        launches = lib.mfb_launch_count() - launches0
        total_ms = ev[0].elapsed_time(ev[-1])
        stack_ms = [a.elapsed_time(b) for a, b in kev]   # the pass alone, without the refresh of its input rows

        # end to end through the C ABI with host buffers
        host_in = [t.cpu().pin_memory() for t in inputs]
        host_out = torch.empty_like(host_in[0]).pin_memory()
        for i in range(3):
            work[i % n_sets].copy_(host_in[i % n_sets], non_blocking=True)
            host_out.copy_(step(i, src="host"), non_blocking=True)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            work[i % n_sets].copy_(host_in[i % n_sets], non_blocking=True)
            host_out.copy_(step(i, src="host"), non_blocking=True)
            torch.cuda.current_stream().synchronize()   # the caller reads the result before the next step
        e1.record()
        self.barrier()
        clocks = sampler.stop() if sampler is not None else None
        e2e_ms = e0.elapsed_time(e1)
        status = moe.device_status()   # a bounded wait that ran out would have unwound the launch early: not a valid timing

        # untimed check of one step's result against the layer-by-layer launches of the same layers (bit for bit)
        check = inputs[0].clone()
        if fresh:
            moe.encode_stack_rows(stack, check)
        else:
            moe.encode_stack(stack, check)
        ref = inputs[0].clone()
        for l, lw in enumerate(layers):
            if fresh:
                moe.encode_layer(lw, ref[l], ref[l])
            else:
                moe.encode_layer(lw, ref, ref)
        output_ok = bool(torch.equal(check.view(torch.int16), ref.view(torch.int16))) and bool(torch.isfinite(check.float()).all())
        status |= moe.device_status()

        phase_us = None
        if trace and launch == "fused":
            tr = torch.zeros((NL + 17, 8), dtype=torch.int64, device="cuda")
            moe.set_trace(tr)
            step(0)
            moe.set_trace(None)
            torch.cuda.synchronize()
            st = tr[:NL].cpu().numpy().astype("float64")
            names = ["norm", "logits", "select", "sort", "phase1", "barrier", "phase2"]
            phase_us = {n: round(float((st[:, i + 1] - st[:, i]).mean() / 1e3), 2) for i, n in enumerate(names)}
            if NL > 1:
                phase_us["combine_to_next_layer"] = round(float((st[1:, 0] - st[:-1, 7]).mean() / 1e3), 2)
                phase_us["layer_period"] = round(float((st[1:, 0] - st[:-1, 0]).mean() / 1e3), 2)
            # SM-cycle counters of one CTA (number 1), per layer: a computing warp's wait for a stage and its work on it, per FFN
            # phase; the copy-issuing warp's time spent issuing (mostly waiting for a free stage)
            cyc = tr[NL:NL + 17].cpu().numpy().astype("float64") / NL
            cw = [r for r in range(16) if cyc[r, 1] > 0 or cyc[r, 3] > 0]     # the computing warps (8 or 16)
            cp = 16 if len(cw) == 16 else 8                                     # the copy-issuing warp follows them
            phase_us["cta_kcycles_per_layer"] = {
                "computing_warps": len(cw),
                "phase1_wait": round(float(cyc[cw, 0].mean() / 1e3), 2), "phase1_compute": round(float(cyc[cw, 1].mean() / 1e3), 2),
                "phase2_wait": round(float(cyc[cw, 2].mean() / 1e3), 2), "phase2_compute": round(float(cyc[cw, 3].mean() / 1e3), 2),
                "phase1_total": round(float(cyc[cw, 5].mean() / 1e3), 2), "phase2_total": round(float(cyc[cw, 7].mean() / 1e3), 2),
                "phase1_copy_issue": round(float(cyc[cp, 0] / 1e3), 2), "phase2_copy_issue": round(float(cyc[cp, 2] / 1e3), 2)}

        times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = float(times[0]), float(times[1])
        hbm_peak, _, peak_kind = measured_peaks()
        bytes_per_step = statistics.mean(step_bytes[i % n_sets] for i in range(steps))
        launch_ms = statistics.mean(stack_ms)
        achieved = bytes_per_step / (launch_ms * 1e-3) / 1e9
        fused = launch == "fused"
        traffic = None
        if fused and (B, rows) in TRAFFIC_PER_LAYER:   # ncu capture of a 2-layer case of this build, scaled by the layer count
            traffic = TRAFFIC_PER_LAYER[(B, rows)] * NL
        rec = {
            "value": world * B * steps / (total_ms * 1e-3), "unit": "tokens/s", "ms_per_step": total_ms / steps,
            "batch_per_gpu": B, "rows": rows,
            "distinct_experts_per_layer": round((bytes_per_step / NL - self.blob - E * D * 2 - B * D * 4) / self.blob, 1),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "peak_kind": peak_kind, "traffic": traffic,
                         "kernel": "stack_mega_kernel (one cooperative launch = the whole pass)" if fused
                                   else "all kernels of the pass, launched layer by layer",
                         "launch_ms": launch_ms, "algorithmic_bytes_per_launch": bytes_per_step},
            "e2e": {"value": world * B * steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": inputs[0].numel() * 2, "d2h_bytes_per_step": inputs[0].numel() * 2},
            "gpu_launches": int(launches), "device_status": int(status), "output_matches_layer_by_layer": output_ok,
            "clocks": clocks, "l2": f"inputs larger than L2: {bytes_per_step / 1e6:.0f} MB of distinct weight bytes per step, "
                                    f"{n_sets} input sets cycled",
        }
        if phase_us is not None:
            rec["phase_us"] = phase_us
        if cpu_budget and rank == 0:
            tok_s, cores, sample = cpu_port_tokens_per_s(B, cpu_budget, NL)
            rec["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        else:
            rec["cpu_baseline"] = None
        moe.close()
        return rec


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    bench = DecodeBench(args, world, rank, local)
    B, NL = args.batch, args.layers
    head = bench.run(B, args.rows, args.steps, args.warmup, launch=args.launch, trace=args.trace, cpu_budget=10.0,
                     sampler=ClockSampler(local))
    bad = head["device_status"] != 0 or not head["output_matches_layer_by_layer"]
    out = {
        "metric": "moe_decode_tokens_per_s", "value": head["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"configs[1]: {NL}-layer Qwen3.6-A3B MoE FFN stack, decode batch {B}, {args.rows} rows",
                   "hidden": D, "intermediate": F, "experts": E, "top_k": K, "shared_experts": 1, "bits": 4,
                   "group_size": 64, "layers": NL, "batch_per_gpu": B, "rows": args.rows, "activation_dtype": "bf16",
                   "accumulate": "f32", "parallelism": "replicas" if world > 1 else "single",
                   "distinct_experts_per_layer": head["distinct_experts_per_layer"], "l2": head["l2"]},
        "roofline": head["roofline"], "cpu_baseline": head["cpu_baseline"], "e2e": head["e2e"],
        "gpu_launches": head["gpu_launches"], "device_status": head["device_status"],
        "output_matches_layer_by_layer": head["output_matches_layer_by_layer"], "clocks": head["clocks"],
    }
    if "phase_us" in head:
        out["phase_us"] = head["phase_us"]

    if args.extras and args.launch == "fused":
        extras = {}
        if world == 1:
            # the rest of the metric in the same run: the other decode batches of configs[1], configs[2] and configs[4]
            for name, (b, rows, steps) in {"decode_b1": (1, "chained", 50), "decode_b8": (8, "fresh", 30),
                                           "decode_b64_chained": (64, "chained", 30)}.items():
                if (b, rows) == (B, args.rows):
                    continue
                rec = bench.run(b, rows, steps, 3, trace=args.trace, cpu_budget=4.0)
                rec["metric"], rec["workload"] = "moe_decode_tokens_per_s", f"configs[1]: decode batch {b}, {rows} rows"
                bad |= rec["device_status"] != 0 or not rec["output_matches_layer_by_layer"]
                extras[name] = rec
            layer0 = bench.layers[0]
            del bench.layers[1:]          # the prefill workloads use one layer: release the rest of the pool
            torch.cuda.empty_cache()
            extras["prefill"] = prefill_case("prefill", 4096, 20, 3, layer0, cpu_budget=5.0)
            extras["ragged"] = prefill_case("ragged", 0, 5, 3, layer0, cpu_budget=0.0)
            extras["ragged"]["cpu_baseline"] = dict(extras["prefill"]["cpu_baseline"] or {}) or None
            if extras["ragged"]["cpu_baseline"]:
                extras["ragged"]["cpu_baseline"]["sample"] += " (the sample of the prefill workload: same layer, same cost per token row)"
            bad |= any(extras[k]["device_status"] != 0 for k in ("prefill", "ragged"))
        else:
            del bench.layers[:]
            torch.cuda.empty_cache()
            extras["ep"] = ep_case(world, rank, local, 10, 3)
        out["extras"] = extras
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    if bad:
        sys.exit("bench: a device status word was set or an output check failed")


def zipf_logit_bias(num_experts: int, exponent: float = 1.1):
    """log p_e with p_e proportional to rank_e ** -exponent under a seeded permutation of the experts (configs[2])."""
    import numpy as np
    rng = np.random.Generator(np.random.PCG64(ROOT_SEED))
    rank = rng.permutation(num_experts) + 1
    p = rank.astype(np.float64) ** -exponent
    return np.log(p / p.sum()).astype(np.float32)


RAGGED_SEQUENCES, RAGGED_PARTS = 48, (1, 256, 512, 1024)


def ragged_mix_offsets():
    """configs[4]: row offsets of the segments of the packed batch (sequence-major: decode row, then the three chunks)."""
    import numpy as np
    sizes = np.tile(np.asarray(RAGGED_PARTS, dtype=np.int64), RAGGED_SEQUENCES)
    return np.concatenate([[0], np.cumsum(sizes)])


def prefill_case(workload, tokens, steps, warmup, layer=None, cpu_budget=5.0, sampler=None):
    """configs[2] ('prefill': `tokens` rows, Zipf(1.1) logit bias) or configs[4] ('ragged': the 86,064-row mix, unbiased
    router) through one Q layer - RMSNorm, router, sort by expert, the ragged grouped GEMM on the tensor cores (routed
    experts + the shared expert), weighted reduce + residual.  Returns the record of the measurement."""
    import copy
    import torch
    from mference_b200 import _lib as L
    from mference_b200.moe import MoE, synth_layer, synth_normal

    lib = L.load()
    ragged = workload == "ragged"
    offsets = ragged_mix_offsets() if ragged else None
    T = int(offsets[-1]) if ragged else tokens
    layer = copy.copy(layer) if layer is not None else synth_layer(ROOT_SEED, 0, D, F, E)
    layer.logit_bias = None if ragged else torch.from_numpy(zipf_logit_bias(E)).cuda()
    moe = MoE(D, F, E, K, max_tokens=T, tensor_core_prefill=True)
    n_sets = N_INPUTS
    inputs = [synth_normal(ROOT_SEED, f"x.{workload}.{i}", T * D, dtype=L.DT_BF16).view(T, D) for i in range(n_sets)]
    out = torch.empty_like(inputs[0])
    # group sizes of the first input set (untimed)
    idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w = torch.empty((T, K), dtype=torch.float16, device="cuda")
    xn = torch.empty_like(inputs[0])
    moe.encode_rmsnorm(inputs[0], xn, layer.norm_w)
    moe.encode_router(xn, layer, idx, w)
    counts = torch.bincount(idx.view(-1).long(), minlength=E)
    torch.cuda.synchronize()

    def step(i):
        moe.encode_layer_prefill(layer, inputs[i % n_sets], out)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    launches0 = lib.mfb_launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        step(i)
        ev[i + 1].record()
    torch.cuda.synchronize()
    launches = lib.mfb_launch_count() - launches0
    total_ms = ev[0].elapsed_time(ev[-1])
    # end to end: pinned host rows in, result out
    host_in = [t.cpu().pin_memory() for t in inputs]
    host_out = torch.empty_like(host_in[0]).pin_memory()
    dev_in = torch.empty_like(inputs[0])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(steps):
        dev_in.copy_(host_in[i % n_sets], non_blocking=True)
        moe.encode_layer_prefill(layer, dev_in, out)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    e2e_ms = e0.elapsed_time(e1)
    status = moe.device_status()

    ms = total_ms / steps
    flops = 2 * 3 * D * F * (T * K + T) + 2 * T * D * E      # routed pairs + shared rows, plus the gate GEMV
    _, tf_peak, peak_kind = measured_peaks()
    achieved = flops / (ms * 1e-3) / 1e12
    io_bytes = T * D * 2
    cpu = None
    if cpu_budget:
        tok_s, cores, sample = cpu_port_prefill_tokens_per_s(64, cpu_budget, zipf=not ragged)
        cpu = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    rec = {
        "metric": "moe_prefill_tokens_per_s", "value": T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
        "workload": (f"configs[4]: ragged continuous-batch mix, 48 sequences x (1 decode row + prefill chunks of 256/512/1024) "
                     f"= {T} rows in {len(offsets) - 1} segments packed into one batch, one Qwen3.6-A3B MoE layer, unbiased router"
                     if ragged else
                     f"configs[2]: prefill gather-QMM, {T} tokens, one Qwen3.6-A3B MoE layer, Zipf(1.1) router bias"),
        "pairs": T * K, "largest_group": int(counts.max()), "smallest_group": int(counts.min()),
        "experts_used": int((counts > 0).sum()),
        "l2": f"{n_sets} input sets cycled; 453 MB of expert weights per step exceed L2",
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s", "frac": achieved / tf_peak,
                     "peak_kind": peak_kind, "traffic": None, "kernel": "whole layer (tc_ffn_kernel<1>, <2> dominate)",
                     "algorithmic_flops_per_step": flops},
        "cpu_baseline": cpu,
        "e2e": {"value": T / (e2e_ms / steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": io_bytes,
                "d2h_bytes_per_step": io_bytes},
        "gpu_launches": int(launches), "device_status": int(status), "clocks": clocks,
    }
    moe.close()
    return rec


def run_prefill(args):
    import torch
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    rec = prefill_case(args.workload, args.tokens, args.steps, args.warmup, cpu_budget=8.0,
                       sampler=ClockSampler(torch.cuda.current_device()))
    line = {"metric": rec["metric"], "value": rec["value"], "unit": rec["unit"], "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
            "config": {"workload": rec["workload"], "hidden": D, "intermediate": F, "experts": E, "top_k": K,
                       "shared_experts": 1, "bits": 4, "group_size": 64, "pairs": rec["pairs"],
                       "largest_group": rec["largest_group"], "smallest_group": rec["smallest_group"],
                       "experts_used": rec["experts_used"], "l2": rec["l2"]}}
    for k in ("roofline", "cpu_baseline", "e2e", "gpu_launches", "device_status", "clocks"):
        line[k] = rec[k]
    print(json.dumps(line))
    if rec["device_status"]:
        sys.exit("bench: device status word set")


VD, VF, VE, VK, VT = 4096, 2048, 256, 6, 2048      # configs[3]: DeepSeek-V4-Flash-shaped layer, 2-bit experts + 4-bit shared


def v_layer(first_expert, n_experts):
    """Seeded V-shape layer holding experts [first_expert, first_expert + n_experts) of the pool, the router and the
    shared expert (the same bytes on every rank for the same expert)."""
    import torch
    from mference_b200 import _lib as L
    from mference_b200.moe import MoELayerWeights, _ptr, _stream, expert_layout, synth_normal
    lib = L.load()
    off, blob = expert_layout(2, VD, VF)
    stride = (blob + 255) // 256 * 256
    pool = torch.empty(n_experts * stride, dtype=torch.uint8, device="cuda")
    # the generator places expert e at base + e * stride: hand it the base of the (virtual) full pool, of which this
    # tensor is the slice starting at first_expert
    import ctypes
    base = ctypes.c_void_p(pool.data_ptr() - first_expert * stride)
    L.check(lib.mfb_synth_expert_pool(_stream(), ROOT_SEED, 0, first_expert, n_experts, 0, 2, L.DT_F16, VD, VF, base, stride))
    soff, sblob = expert_layout(4, VD, VF)
    shared = torch.empty(sblob, dtype=torch.uint8, device="cuda")
    L.check(lib.mfb_synth_expert_pool(_stream(), ROOT_SEED, 0, 0, 1, 1, 4, L.DT_F16, VD, VF, _ptr(shared), 0))
    router = synth_normal(ROOT_SEED, "L0.router", VE * VD, std=0.02, dtype=L.DT_BF16).view(VE, VD)
    return MoELayerWeights(router_w=router, pool=pool, slot_stride=stride, routed_off=off, shared_blob=shared, shared_off=soff,
                           norm_w=torch.ones(VD, dtype=torch.bfloat16, device="cuda"))


def ep_case(world, rank, local, steps, warmup):
    """configs[3]: the V-shape layer (hidden 4096, intermediate 2048, 256 experts top-6, 2-bit experts + 4-bit shared) over
    2048 tokens, experts block-sharded over the ranks, tokens split evenly (strong scaling), dispatch and combine as
    one-sided peer stores over NVLink.  Returns the record (on rank 0; None elsewhere)."""
    import copy
    import torch
    import torch.distributed as dist
    from mference_b200 import _lib as L
    from mference_b200.ep import DeviceOps, PeerExpertParallelLayer
    from mference_b200.moe import MoE, synth_normal

    lib = L.load()
    T = VT // world
    local_E = VE // world
    mine = v_layer(rank * local_E, local_E)          # this rank's slice of the pool + the replicated parts
    replicated = copy.copy(mine)                     # router, norm (the pool field is not used on the home side)
    local_w = copy.copy(mine)
    local_w.shared_blob = None
    shared_w = copy.copy(mine)
    shared_w.pool, shared_w.slot_stride, shared_w.routed_off = mine.shared_blob, mine.shared_blob.numel(), mine.shared_off
    shared_w.shared_blob = None
    ops = DeviceOps(VD, VF, VE, VK, world, max_tokens=T, max_recv_rows=world * T * VK, bits=2, shared_bits=4)
    layer = PeerExpertParallelLayer(ops, rank, world, T)
    xs = [synth_normal(ROOT_SEED, f"x.ep.{i}", VT * VD, dtype=L.DT_BF16).view(VT, VD)[rank * T:(rank + 1) * T].contiguous()
          for i in range(N_INPUTS)]
    y = torch.empty_like(xs[0])

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        layer.forward(replicated, local_w, shared_w, xs[i % N_INPUTS], y)
    barrier()
    # the layer as a CUDA graph over one input buffer that every step refreshes (a device copy inside the timed region)
    x_static = torch.empty_like(xs[0])
    launches0 = lib.mfb_launch_count()
    layer.capture(replicated, local_w, shared_w, x_static, y)
    launches_per_step = lib.mfb_launch_count() - launches0
    barrier()
    for i in range(2):
        x_static.copy_(xs[i % N_INPUTS])
        layer.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(steps):
        x_static.copy_(xs[i % N_INPUTS])
        layer.replay()
    e1.record()
    barrier()
    launches = launches_per_step * steps
    ms_dev = e0.elapsed_time(e1)
    # stage breakdown of one more call
    marks = []
    layer.forward(replicated, local_w, shared_w, xs[0], y, marks=marks)
    barrier()
    stage_us = {b[0]: round(a[1].elapsed_time(b[1]) * 1e3, 1) for a, b in zip(marks[:-1], marks[1:])}
    y0 = y.clone()
    status, recv_counts = layer.ex.status(with_counts=True)
    status |= ops.expert.device_status() | ops.shared.device_status() | ops.home.device_status()
    # end to end with host rows
    host_in = [t.cpu().pin_memory() for t in xs]
    host_out = torch.empty_like(host_in[0]).pin_memory()
    barrier()
    e0.record()
    for i in range(steps):
        x_static.copy_(host_in[i % N_INPUTS], non_blocking=True)
        layer.replay()
        host_out.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    barrier()
    t = torch.tensor([ms_dev, e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    recv_all = [torch.zeros(1, dtype=torch.float64, device="cuda") for _ in range(world)]
    dist.all_gather(recv_all, torch.tensor([float(sum(recv_counts))], dtype=torch.float64, device="cuda"))
    rec = None
    if rank == 0:
        # one GPU, the whole batch and the whole pool: the time strong scaling is measured against, and the check
        full = v_layer(0, VE)
        one = MoE(VD, VF, VE, VK, bits=2, shared_bits=4, max_tokens=VT, tensor_core_prefill=True)
        x_all = synth_normal(ROOT_SEED, "x.ep.0", VT * VD, dtype=L.DT_BF16).view(VT, VD)
        y_all = torch.empty_like(x_all)
        for _ in range(3):
            one.encode_layer_prefill(full, x_all, y_all)
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(steps):
            one.encode_layer_prefill(full, x_all, y_all)
        s1.record()
        torch.cuda.synchronize()
        ms_one = s0.elapsed_time(s1) / steps
        matches = bool(torch.equal(y0, y_all[:T]))
        status |= one.device_status()
        ms = float(t[0]) / steps
        flops = 2 * 3 * VD * VF * (VT * VK + VT) + 2 * VT * VD * VE
        _, tf_peak, peak_kind = measured_peaks()
        achieved = flops / (ms * 1e-3) / 1e12
        pairs_remote = VT * VK * (world - 1) / world
        try:
            from oracle import oracle as O
            O.set_num_threads(os.cpu_count() or 1)     # torchrun exports OMP_NUM_THREADS=1 to its ranks
        except Exception:
            pass
        tok_s, cores, sample = cpu_port_prefill_tokens_per_s(16, 5.0, zipf=False, shape=(VD, VF, VE, VK, 2, 4))
        cpu = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        rec = {
            "metric": "moe_prefill_tokens_per_s", "value": VT / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "n_gpus": world,
            "scaling": "strong",
            "workload": f"configs[3]: DeepSeek-V4-Flash-shaped layer (hidden {VD}, intermediate {VF}, {VE} experts top-{VK} + 1 shared, 2-bit "
                        f"experts, 4-bit shared), {VT} tokens over {world} ranks, {local_E} experts per rank, dispatch and combine as "
                        f"one-sided peer stores over NVLink; the layer replayed as a CUDA graph",
            "one_gpu_ms_per_step": ms_one, "speedup_vs_one_gpu": ms_one / ms, "strong_scaling_efficiency": ms_one / ms / world,
            "pairs_received_per_rank": [int(r.item()) for r in recv_all],
            "dispatch_bytes_per_step": int(pairs_remote * VD * 2), "combine_bytes_per_step": int(pairs_remote * VD * 4),
            "stage_us_rank0": stage_us,
            "output_matches_single_gpu_layer": matches,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf_peak * world, "unit": "TFLOP/s",
                         "frac": achieved / (tf_peak * world), "peak_kind": peak_kind, "traffic": None,
                         "kernel": "whole layer incl. both exchanges", "algorithmic_flops_per_step": flops},
            "cpu_baseline": cpu,
            "e2e": {"value": VT / (float(t[1]) / steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": VT * VD * 2,
                    "d2h_bytes_per_step": VT * VD * 2},
            "gpu_launches": int(launches), "device_status": int(status),
        }
    barrier()
    return rec


def run_ep(args):
    """--workload ep: configs[3] alone (under torchrun with --gpus N ranks; also runs with one rank)."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29577", rank=0, world_size=1, device_id=torch.device("cuda", local))
    sampler = ClockSampler(local)
    sampler.start()
    rec = ep_case(world, rank, local, args.steps, args.warmup)
    clocks = sampler.stop()
    if rank == 0:
        line = {"metric": rec["metric"], "value": rec["value"], "unit": rec["unit"], "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
                "config": {k: rec[k] for k in ("workload", "one_gpu_ms_per_step", "speedup_vs_one_gpu", "strong_scaling_efficiency",
                                               "pairs_received_per_rank", "dispatch_bytes_per_step", "combine_bytes_per_step",
                                               "stage_us_rank0", "output_matches_single_gpu_layer")}}
        line["config"]["parallelism"] = f"ep{world}"
        line["config"]["l2"] = f"{N_INPUTS} input sets cycled; 2 GB of expert weights"
        for k in ("roofline", "cpu_baseline", "e2e", "gpu_launches", "device_status"):
            line[k] = rec[k]
        line["clocks"] = clocks
        print(json.dumps(line))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=64, help="decode batch (token rows per step per GPU): 1, 8 or 64")
    ap.add_argument("--rows", default=None, choices=["fresh", "chained"])
    ap.add_argument("--layers", type=int, default=LAYERS, help="fewer layers only for profiling a small case")
    ap.add_argument("--launch", default="fused", choices=["fused", "layers"],
                    help="layers: per-layer, per-phase launches of the same kernels (for profiling one phase alone)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "ragged", "ep"],
                    help="decode: configs[1] (the headline); prefill: configs[2], 4096 tokens through one layer's gather-QMM; "
                         "ragged: configs[4], the 86,064-row continuous-batch mix through the same layer; "
                         "ep: the same prefill layer with experts sharded over --gpus ranks (NCCL all-to-all)")
    ap.add_argument("--tokens", type=int, default=4096, help="prefill token rows")
    ap.add_argument("--trace", action="store_true", help="decode: add the fused kernel's per-phase times (one untimed step) as phase_us")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="decode: only the headline measurement (default: also decode batch 1 / 8 / 64 chained, configs[2] and "
                         "configs[4] at 1 GPU, the expert-parallel layer of configs[3] at N > 1, under the line's `extras` key)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.rows is None:
        args.rows = "chained" if args.batch == 1 else "fresh"
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("prefill", "ragged"):
        run_prefill(args)
    elif args.workload == "ep":
        run_ep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the fused forward+backward thunks on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case <name> [--launches N] [--batch B] [--tune KNOB=VALUE]   # one small workload, for profilers

Headline workload (N = 1): benchmark config 2 -- causal row softmax forward+backward on scores
[1, 32, 2048, 2048] fp16 (fp32 accumulation), one fused launch per step.  `value` is the HBM GB/s of that launch
with inputs resident in HBM, counted on the bytes a causal forward+backward has to move (the unmasked prefixes of
S and dP read, P and dS written: 805 MB); the figure on the dense accounting (all four tensors whole, 1074 MB, of
which the masked half of the inputs is never read) is reported beside it under `dense_accounting`.  `e2e` is the same
quantity measured through the C-ABI call with HOST buffers (pinned H2D of scores and dP, D2H of P and dScores inside
the timed region, pipelined per (batch, head) block).  Under torchrun (N > 1) every rank runs its own config-2 sized
batch (weak scaling, no data-path collective: softmax rows are independent).

`--impl reference` times the CPU restatement of the reference chain (oracle/ref_chain.c: one OpenMP loop per
primitive thunk over materialised intermediates, all host threads) on a bounded sample of the same workload, in the
same unit; the reference itself (Rust + patched Futhark) cannot be built on this image.

`train_step` in the line is benchmark config 5 (see train_step_leg); `thunks` the other kernels at their shapes.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADS, SEQ = 32, 2048                       # config 2: [1, 32, 2048, 2048]
ROWS, COLS = HEADS * SEQ, SEQ
ELEMS = ROWS * COLS
DENSE_BYTES = 4 * ELEMS * 2                 # S, dP, P, dS whole
# what a causal kernel must move: row r reads r + 1 elements of S and of dP and writes whole rows of P and dS
MOVED_BYTES = HEADS * (2 * (SEQ * (SEQ + 1) // 2) + 2 * SEQ * SEQ) * 2
METRIC = "fused fwd+bwd thunk HBM GB/s (causal softmax, config 2)"
CONFIG = {"workload": "causal softmax fwd+bwd, scores [1,32,2048,2048] f16 (benchmark config 2)", "rows": ROWS, "cols": COLS,
          "bytes_per_step": MOVED_BYTES}
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one softmax_rows_kernel launch on config 2, from an ncu capture of
# `bench.py --case softmax_full` (277.0 MB read + 474.0 MB written); not re-measured by a bench run
NCU_TRAFFIC_BYTES = 750946560


def measured_tensor_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid, self.rows, self.proc = uuid, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def physical_cores():
    """Unique (core, socket) pairs, which is what the reference counts (src/pctx/smp.rs:158-181)."""
    try:
        out = subprocess.run(["lscpu", "-p=CORE,SOCKET"], capture_output=True, text=True).stdout
        cores = {l for l in out.splitlines() if l and not l.startswith("#")}
        n = len(cores)
        avail = len(os.sched_getaffinity(0))
        return max(1, min(n, avail)) if n else avail
    except Exception:
        return os.cpu_count() or 1


def cpu_reference_time(sample_heads, reps, threads):
    """Seconds per pass of the C restatement over `sample_heads` (batch, head) blocks of config 2."""
    import numpy as np
    from oracle import c_oracle as CO
    from oracle import ref_chain as R
    CO.set_num_threads(threads)
    rows = sample_heads * SEQ
    s = R.normal(0, (rows, COLS), np.float16, 0.1)
    dp = R.normal(1, (rows, COLS), np.float16)
    CO.softmax_fwd_bwd(s[:SEQ], dp[:SEQ], (1, SEQ, 0))            # warm-up (page in, spin up the team)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        CO.softmax_fwd_bwd(s, dp, (1, SEQ, 0))
        times.append(time.perf_counter() - t0)
    return statistics.median(times), rows


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = physical_cores()
    sample_heads = 4
    t0 = time.time()
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_reference_time(1, 1, threads)
    sec, rows = cpu_reference_time(sample_heads, max(1, args.steps), threads)
    gbs = MOVED_BYTES * (rows / ROWS) / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3 * (ROWS / rows), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 storage / f32 accumulate", "data": "synthetic", "config": dict(CONFIG),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{sample_heads} of 32 (batch, head) blocks = {rows} rows per step; "
                                   "ms_per_step is scaled to the full 65536 rows"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.time() - t0,
    }
    print(json.dumps(line), flush=True)


def time_thunk(fn, launches, warmup, torch):
    """Average device time per call of fn over `launches` back-to-back calls (CUDA events on the launch stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches * 1e-3


def other_thunks(torch, ops, peak):
    """Device-resident GB/s of the other fused thunks at their benchmark shapes (explanatory, not the headline)."""
    out = {}
    gen = torch.Generator(device="cuda").manual_seed(1)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=gen) * scale).half()

    def report(name, sec, nbytes, launches):
        out[name] = {"GB/s": round(nbytes / sec / 1e9, 1), "frac_of_peak": round(nbytes / sec / 1e9 / peak, 3),
                     "us": round(sec * 1e6, 1), "algorithmic_bytes": nbytes, "launches_per_step": launches}

    # K1 RMSNorm fwd+bwd at the config-5 activation shape [16384, 3200] f16
    x, dy, g = rnd(16384, 3200), rnd(16384, 3200), rnd(3200)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    dg = torch.empty(3200, dtype=torch.float16, device="cuda")
    ws = ops.rmsnorm_workspace(16384, 3200, x.device)
    sec = time_thunk(lambda: ops.rmsnorm_fwd_bwd(x, g, dy, 1e-6, y=y, dx=dx, dgamma=dg, workspace=ws), 20, 5, torch)
    report("rmsnorm_fwd_bwd[16384x3200,f16]", sec, 4 * 16384 * 3200 * 2 + 2 * 3200 * 2, 2)
    del x, dy, y, dx
    # K5 softmax-NLL config 3
    lg = rnd(8192, 32000, scale=2.0)
    tg = torch.randint(0, 32000, (8192,), device="cuda", dtype=torch.int32, generator=gen)
    dl = torch.empty_like(lg)
    sec = time_thunk(lambda: ops.softmax_nll_fwd_bwd(lg, tg, w_scalar=1.0 / 8192, dlogits=dl), 20, 5, torch)
    report("softmax_nll_fwd_bwd[8192x32000,f16]", sec, 2 * 8192 * 32000 * 2 + 8192 * 4 + 4, 2)
    del lg, dl
    # K3 RoPE config 4 (one of Q / K per launch)
    cos, sin = ops.rope_tables(2048, 100)
    q, dq = rnd(16384, 32, 100), rnd(16384, 32, 100)
    yq, dxq = torch.empty_like(q), torch.empty_like(q)
    sec = time_thunk(lambda: ops.rope_fwd_bwd(q, dq, cos, sin, y=yq, dx=dxq), 20, 5, torch)
    report("rope_fwd_bwd[16384x32x100,f16]", sec, 4 * 16384 * 3200 * 2, 1)
    del q, dq, yq, dxq
    # K4 SwiGLU config 4
    ga, up, dh = rnd(16384, 8640), rnd(16384, 8640), rnd(16384, 8640)
    h, dga, dup = torch.empty_like(ga), torch.empty_like(ga), torch.empty_like(ga)
    sec = time_thunk(lambda: ops.swiglu_fwd_bwd(ga, up, dh, h=h, dgate=dga, dup=dup), 20, 5, torch)
    report("swiglu_fwd_bwd[16384x8640,f16]", sec, 6 * 16384 * 8640 * 2, 1)
    del ga, up, dh, h, dga, dup
    # K8 AdamW32 update of one gate-projection-sized parameter block x4 (f32 master/m/v, f16 gradient and copy)
    n = 4 * 8640 * 3200
    wm = torch.randn(n, device="cuda", generator=gen)
    m1, m2 = torch.zeros_like(wm), torch.zeros_like(wm)
    gg = rnd(n)
    pc = torch.empty_like(gg)
    sec = time_thunk(lambda: ops.adamw32_step(wm, m1, m2, gg, 5, param_out=pc), 10, 3, torch)
    report("adamw32_step[110.6M params]", sec, 28 * n, 1)
    del wm, m1, m2, gg, pc
    # G1 dense matmul: gate projection x[16384,3200] W[8640,3200]^T and its two adjoints (tensor roofline)
    tpeak = measured_tensor_peak()
    x, w, dyp = rnd(16384, 3200), rnd(8640, 3200, scale=0.02), rnd(16384, 8640)
    c = torch.empty(16384, 8640, dtype=torch.float16, device="cuda")
    dxp = torch.empty(16384, 3200, dtype=torch.float16, device="cuda")
    dw = torch.empty(8640, 3200, dtype=torch.float16, device="cuda")
    flops = 2 * 16384 * 8640 * 3200
    for name, fn in (("gemm_nt y=xW^T", lambda: ops.gemm(x, w, False, True, c=c)),
                     ("gemm_nn dx=dyW", lambda: ops.gemm(dyp, w, False, False, c=dxp)),
                     ("gemm_tn dW=dy^Tx", lambda: ops.gemm(dyp, x, True, False, c=dw))):
        sec = time_thunk(fn, 10, 3, torch)
        out[name + "[16384x8640x3200,f16]"] = {"TFLOP/s": round(flops / sec / 1e12, 1), "frac_of_measured_burst_peak": round(flops / sec / 1e12 / tpeak, 3),
                                              "frac_of_nominal_2250": round(flops / sec / 1e12 / 2250.0, 3), "us": round(sec * 1e6, 1), "launches_per_step": 1}
    del x, w, dyp, c, dxp, dw
    # G2 block matmul at config 5 (B = 8): HBM-bound by the 2.1 GB score tensor
    B, S, H, hd = 8, 2048, 32, 100
    q, k = rnd(B, S, H, hd), rnd(B, S, H, hd)
    sc = torch.empty(B, S, H, S, dtype=torch.float16, device="cuda")
    ws = torch.empty(ops.lib().cacti_b200_gemm_workspace_bytes(S, S, hd, B, H), dtype=torch.uint8, device="cuda")
    sec = time_thunk(lambda: ops.block_gemm(q, k, False, True, alpha=0.1, c=sc, workspace=ws), 5, 3, torch)
    nbytes = B * H * S * S * 2 + 2 * B * S * H * hd * 2
    out["block_gemm QK^T[8x2048x32x100]"] = {"TFLOP/s": round(2 * B * H * S * S * hd / sec / 1e12, 1), "GB/s": round(nbytes / sec / 1e9, 1),
                                             "frac_of_peak": round(nbytes / sec / 1e9 / peak, 3), "us": round(sec * 1e6, 1), "launches_per_step": 3}
    v = rnd(B, S, H, hd)
    ctx = torch.empty(B, S, H, hd, dtype=torch.float16, device="cuda")
    sec = time_thunk(lambda: ops.block_gemm(sc, v, False, False, c=ctx, workspace=ws), 5, 3, torch)
    out["block_gemm PV[8x2048x32x100]"] = {"TFLOP/s": round(2 * B * H * S * S * hd / sec / 1e12, 1), "GB/s": round(nbytes / sec / 1e9, 1),
                                           "frac_of_peak": round(nbytes / sec / 1e9 / peak, 3), "us": round(sec * 1e6, 1), "launches_per_step": 2}
    # the same two block matmuls with the causal-structure hints the training step passes
    from cacti_b200 import capi
    sec = time_thunk(lambda: ops.block_gemm(q, k, False, True, alpha=0.1, c=sc, workspace=ws, tri=capi.TRI_C_LOWER), 5, 3, torch)
    out["block_gemm QK^T, C_LOWER hint[8x2048x32x100]"] = {"us": round(sec * 1e6, 1), "launches_per_step": 3}
    pz = torch.tril(torch.ones(S, S, device="cuda", dtype=torch.float16))[None, :, None, :].expand(B, S, H, S).contiguous()
    sec = time_thunk(lambda: ops.block_gemm(pz, v, False, False, c=ctx, workspace=ws, tri=capi.TRI_A_LOWER), 5, 3, torch)
    out["block_gemm PV, A_LOWER hint[8x2048x32x100]"] = {"us": round(sec * 1e6, 1), "launches_per_step": 2}
    del sc, pz
    # A1 fused attention (what the training step runs by default): q, k, v padded to 128 columns; HBM traffic is
    # q, k, v, ctx and the row statistics; "TFLOP/s" counts the 2 * 2 * S^2/2 * hd useful flops per (batch, head)
    qp, kp, vp = (ops.block_pad(t, 128) for t in (q, k, v))
    st = torch.empty(B, H, S, 4, device="cuda")
    sec = time_thunk(lambda: ops.attention_fwd(qp, kp, vp, hd, 0.1, ctx=ctx, stats=st), 10, 3, torch)
    useful = 2 * 2 * B * H * (S * S / 2) * hd
    out["attention_fwd[8x2048x32x100]"] = {"us": round(sec * 1e6, 1), "TFLOP/s_useful": round(useful / sec / 1e12, 1), "launches_per_step": 1}
    do = rnd(B, S, H, hd)
    dop = ops.block_pad(do, 128)
    pp = torch.empty(B, S, H, S, dtype=torch.float16, device="cuda")
    dss = torch.empty_like(pp)
    sec = time_thunk(lambda: ops.attention_bwd_prep(qp, kp, vp, dop, ctx, st, 0.1, p=pp, ds=dss), 5, 3, torch)
    wbytes = 2 * B * H * (S * S // 2) * 2                       # P and dS, lower triangles
    out["attention_bwd_prep[8x2048x32x100]"] = {"us": round(sec * 1e6, 1), "GB/s_written": round(wbytes / sec / 1e9, 1), "launches_per_step": 1}
    sec = time_thunk(lambda: ops.block_pad(q, 128, out=qp), 10, 3, torch)
    report("block_pad[8x2048x32x100->128]", sec, B * S * H * (100 + 128) * 2, 1)
    del pp, dss
    # residual add fused into the norm (one pass over [16384, 3200] saved per norm)
    a_, b_, g_ = rnd(16384, 3200), rnd(16384, 3200), rnd(3200)
    y_, t_ = torch.empty_like(a_), torch.empty_like(a_)
    sec = time_thunk(lambda: ops.add_rmsnorm_fwd(a_, b_, g_, 1e-6, y=y_, total=t_), 20, 5, torch)
    report("add_rmsnorm_fwd[16384x3200,f16]", sec, 4 * 16384 * 3200 * 2, 1)
    return out


def host_max(dist, ctl, value):
    """Maximum of a host float over the ranks, through the CPU (gloo) control group: the timing scalars stay off NCCL,
    so NCCL's algorithm for the gradient buckets can be pinned from the environment without touching them."""
    if ctl is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctl)
    return float(t.item())


def train_step_leg(torch, dist, ctl, rank, world, dev, steps):
    """benchmark config 5: one OpenLLaMA-3B-shaped forward+backward over 8 sequences of 2048 tokens, the sequences
    split across the ranks (strong scaling), weight gradients summed with bucketed NCCL all-reduces that overlap
    the backward pass.  Random-init weights, synthetic token ids.  Reported beside the step time: the same step
    replayed with the exchange left out (`compute_ms`; `exposed_comm_ms` is the difference), and the sum and sum of
    magnitudes of three gradient tensors after the exchange, which must agree between 1, 2, 4 and 8 GPUs up to
    summation order."""
    from cacti_b200 import dp, llama_step as LS, ops
    cfg = LS.LlamaShape.open_llama_3b()
    n_seq = 8
    first, count = dp.shard_sequences(n_seq, world, rank)
    P = LS.init_weights(cfg, dev, seed=0)
    grads, buckets = dp.alloc_bucketed_grads(P)
    red = dp.GradReducer(buckets)
    step = LS.TrainStep(cfg, P, count, loss_tokens=n_seq * cfg.seq)
    # SMs left to the all-reduce kernels that run beside the backward pass (0: none)
    margin = int(os.environ.get("CACTI_B200_GEMM_SM_MARGIN", "0")) if world > 1 else 0
    if margin:
        ops.lib().cacti_b200_tune(b"gemm_sms", 148 - margin)
    fixed_walk = os.environ.get("CACTI_B200_FIXED_WALK", "0") == "1"     # A/B: the matmuls' fixed-stride tile walk
    if fixed_walk:
        ops.lib().cacti_b200_tune(b"gemm_dynamic", 0)
    g = torch.Generator(device=dev).manual_seed(1)
    tok_all = torch.randint(0, cfg.vocab, (n_seq * cfg.seq,), device=dev, dtype=torch.int32, generator=g)
    tgt_all = torch.randint(0, cfg.vocab, (n_seq * cfg.seq,), device=dev, dtype=torch.int32, generator=g)
    sl = slice(first * cfg.seq, (first + count) * cfg.seq)
    h_tok, h_tgt = tok_all[sl].cpu().pin_memory(), tgt_all[sl].cpu().pin_memory()
    tok, tgt = torch.empty_like(tok_all[sl]), torch.empty_like(tgt_all[sl])
    nl = cfg.layers

    def make_body(exchange):
        def body():
            # end to end: token ids come from pinned host memory, the loss goes back to the host
            tok.copy_(h_tok, non_blocking=True); tgt.copy_(h_tgt, non_blocking=True)
            loss = step.forward_backward(tok, tgt, grads, on_layer_done=red.reduce_bucket if exchange else None)
            if exchange:
                red.reduce_bucket(nl + 1)                  # the embedding gradient, complete last
                red.finish()
                if world > 1:
                    dist.all_reduce(loss)
            return loss
        return body

    # the step is replayed from a CUDA graph (kernels, pinned-memory token copies and the bucketed all-reduces are all
    # captured); CACTI_B200_STEP_GRAPH=0 launches it eagerly instead
    use_graph = os.environ.get("CACTI_B200_STEP_GRAPH", "1") != "0"

    def timed(exchange, reps):
        body = make_body(exchange)
        launch, graphed = "eager", None
        if use_graph:
            try:
                graphed = LS.GraphedStep(body)
                launch = "cuda graph"
            except Exception as e:                     # same kernels either way; the line says which launch it timed
                graphed = None
                launch = "eager (graph capture failed: %s)" % (str(e).splitlines()[0][:120] if str(e) else type(e).__name__)
                torch.cuda.synchronize()

        def one():
            return (graphed.replay() if graphed is not None else body()).cpu()

        for _ in range(3):
            one()
        if world > 1:
            dist.barrier(group=ctl)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            loss = one()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=ctl)
        ms = host_max(dist, ctl if world > 1 else None, e0.elapsed_time(e1) / reps)
        del graphed
        torch.cuda.empty_cache()
        return ms, float(loss.item()), launch

    reps = max(10, min(steps, 20))
    compute_ms = None
    if world > 1:
        compute_ms, _, _ = timed(False, reps)          # before the real step, so that the gradients left behind are the reduced ones
    ms, loss, launch = timed(True, reps)
    if margin:
        ops.lib().cacti_b200_tune(b"gemm_sms", 0)
    if fixed_walk:
        ops.lib().cacti_b200_tune(b"gemm_dynamic", 1)
    # f64 sum and sum of magnitudes of three gradients after the exchange (torch reductions: verification, not the path)
    checks = {}
    for name, t in (("lm_head", grads["lm_head"]), ("layers.0.q", grads["layers"][0]["q"]), ("embed", grads["embed"])):
        d = t.double()
        checks[name] = {"sum": float(d.sum().item()), "abs_sum": float(d.abs().sum().item())}
    out = {"workload": "OpenLLaMA-3B-shaped fwd+bwd, 8 x 2048 tokens, 26 layers, f16 / f32 accumulate (benchmark config 5)",
           "tokens_per_s": n_seq * cfg.seq / (ms * 1e-3), "ms_per_step": ms, "scaling": "strong", "n_gpus": world,
           "timed_replays": reps, "sequences_per_gpu": count, "loss": loss, "gpu_launches_per_step": step.launches,
           "launch": launch, "peak_mem_gib": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
           "h2d_bytes_per_step": 2 * count * cfg.seq * 4, "d2h_bytes_per_step": 4, "grad_checksums": checks,
           "note": "no optimizer step (the optimizer thunks are outside this path); gradients of all parameters are produced and all-reduced"}
    if compute_ms is not None:
        out.update({"compute_ms": compute_ms, "exposed_comm_ms": ms - compute_ms, "gemm_sm_margin": margin, "matmul_tile_walk": "fixed stride" if fixed_walk else "dynamic",
                    "exchange": {"collective": "ncclAllReduce(sum) per bucket via torch.distributed", "buckets": len(buckets),
                                 "bytes_per_rank": sum(b.numel() * b.element_size() for b in buckets),
                                 "env": {k: v for k, v in os.environ.items() if k.startswith("NCCL_")}}})
    return out


def train_step_spill_leg(torch, dev, steps):
    """benchmark config 5 on one GPU the way the reference would run it: every tensor a cell of one arena, every op a
    thunk, the arena's soft limit (CACTI_VMEM_SOFT_LIMIT, default 40GiB here) below the step's resident peak of about
    63 GiB, so that the soft-OOM policy spills cells to page-locked host memory during the forward pass and the
    backward pass copies them back (cacti_b200/cell_step.py over the C++ shim in cacti_b200/host/).  Same weights,
    tokens and kernels as `train_step`: the loss must be the same number."""
    import numpy as np
    from cacti_b200 import llama_step as LS
    from cacti_b200.cell_step import CellTrainStep
    from cacti_b200.host import binding as H
    cfg = LS.LlamaShape.open_llama_3b()
    n_seq = 8
    P = LS.init_weights(cfg, dev, seed=0)
    W = {k: v.cpu().numpy() for k, v in P.items() if k != "layers"}
    W["layers"] = [{k: v.cpu().numpy() for k, v in Lw.items()} for Lw in P["layers"]]
    del P
    g = torch.Generator(device=dev).manual_seed(1)
    tok = torch.randint(0, cfg.vocab, (n_seq * cfg.seq,), device=dev, dtype=torch.int32, generator=g).cpu().numpy()
    tgt = torch.randint(0, cfg.vocab, (n_seq * cfg.seq,), device=dev, dtype=torch.int32, generator=g).cpu().numpy()
    torch.cuda.empty_cache()
    free_b, total_b = torch.cuda.mem_get_info(dev)
    text = os.environ.get("CACTI_VMEM_SOFT_LIMIT", "40GiB")
    limit = H.lib().cbh_parse_vmem_soft_limit(text.encode(), total_b, free_b)
    if not limit:
        return {"skipped": f"CACTI_VMEM_SOFT_LIMIT={text!r} is neither a fraction nor a byte size"}
    ctx = H.Ctx(cuda=True, arena_bytes=min(limit + (4 << 30), free_b - (2 << 30)), soft_limit=limit)
    try:
        step = CellTrainStep(ctx, cfg, W, n_seq, loss_tokens=n_seq * cfg.seq)
        stream = torch.cuda.ExternalStream(H.lib().cbh_stream(ctx.h), device=dev)
        step.forward_backward(tok, tgt)                       # warm-up: page-locked buffers get allocated here
        before = ctx.stats()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            loss = step.forward_backward(tok, tgt)
        e1.record(stream)
        e1.synchronize()
        ms = e0.elapsed_time(e1) / steps
        after = ctx.stats()
        per = {k: (after[k] - before[k]) / steps for k in ("spills", "reloads", "spill_bytes", "reload_bytes", "oom_retries")}
        return {"workload": "the train_step workload on one GPU, tensors as cells of an arena under the soft-OOM spill policy",
                "tokens_per_s": n_seq * cfg.seq / (ms * 1e-3), "ms_per_step": ms, "timed_steps": steps, "loss": loss,
                "soft_limit_bytes": int(limit), "soft_limit_text": text, "arena_peak_bytes": int(after["peak_in_use"]),
                "per_step": per, "hard_oom": after["hard_oom"], "thunks_per_step": step.launches,
                "note": "spill and reload copies run on the thunks' own stream, as the reference's do (it synchronises around each); "
                        "the policy evicts in creation order, so parameters are spilled and reloaded as well as activations"}
    finally:
        ctx.close()


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from cacti_b200 import capi, ops
    capi.lib()                                   # raises when the CUDA library is missing: no fallback
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the CPU arm is --impl reference")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ctl = None
    if world > 1:
        # a rank that dies or never joins ends the others' next collective with an error after this long, not a hang
        limit = datetime.timedelta(seconds=int(os.environ.get("CACTI_B200_PG_TIMEOUT_S", "300")))
        dist.init_process_group("nccl", device_id=dev, timeout=limit)
        ctl = dist.new_group(backend="gloo", timeout=limit)      # host-side control plane: barriers and timing scalars
    peak, peak_kind = measured_peak()
    gen = torch.Generator(device=dev).manual_seed(rank)
    s = (torch.randn(ROWS, COLS, device=dev, generator=gen) * 0.1).half()
    dp = torch.randn(ROWS, COLS, device=dev, generator=gen).half()
    p, ds = torch.empty_like(s), torch.empty_like(s)
    mask = (1, SEQ, 0)

    def step():
        ops.softmax_fwd_bwd(s, dp, mask, p=p, ds=ds)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=ctl)

    for _ in range(max(args.warmup, 3)):
        step()
    uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid).replace("GPU-", "")
    with ClockSampler(uuid) as clocks:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        dev_ms = e0.elapsed_time(e1)
        # keep the sampler alive long enough to see the load on short runs
        if dev_ms < 400:
            t_end = time.time() + 0.6
            while time.time() < t_end:
                step()
            torch.cuda.synchronize()
    ms_step = host_max(dist, ctl, dev_ms) / args.steps
    value = world * MOVED_BYTES / (ms_step * 1e-3) / 1e9

    if args.train_only:                          # sweeps of the multi-GPU step: only the train_step entry is printed
        del s, dp, p, ds
        torch.cuda.empty_cache()
        train = train_step_leg(torch, dist, ctl, rank, world, dev, args.steps)
        if rank == 0:
            print(json.dumps({"n_gpus": world, "train_step": train}), flush=True)
        if world > 1:
            dist.barrier(group=ctl)
            dist.destroy_process_group()
        return

    # ---- end to end: host buffers through the same call, pipelined per (batch, head) block -------------
    hs, hdp = s.cpu().pin_memory(), dp.cpu().pin_memory()
    hp, hds = torch.empty_like(hs).pin_memory(), torch.empty_like(hs).pin_memory()
    nblk, brow = HEADS, SEQ
    NBUF = 4
    bufs = [tuple(torch.empty(brow, COLS, dtype=torch.float16, device=dev) for _ in range(4)) for _ in range(NBUF)]
    st_in, st_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream()

    def e2e_step():
        ev_in = [torch.cuda.Event() for _ in range(nblk)]
        ev_k = [torch.cuda.Event() for _ in range(nblk)]
        ev_out = [torch.cuda.Event() for _ in range(nblk)]
        for b in range(nblk):
            bs, bdp, bp, bds = bufs[b % NBUF]
            r = slice(b * brow, (b + 1) * brow)
            with torch.cuda.stream(st_in):
                if b >= NBUF:
                    st_in.wait_event(ev_k[b - NBUF])          # inputs of the block that used this slot are consumed
                bs.copy_(hs[r], non_blocking=True)
                bdp.copy_(hdp[r], non_blocking=True)
                ev_in[b].record(st_in)
            main.wait_event(ev_in[b])
            if b >= NBUF:
                main.wait_event(ev_out[b - NBUF])             # outputs of that slot are on the host
            ops.softmax_fwd_bwd(bs, bdp, mask, p=bp, ds=bds)
            ev_k[b].record(main)
            with torch.cuda.stream(st_out):
                st_out.wait_event(ev_k[b])
                hp[r].copy_(bp, non_blocking=True)
                hds[r].copy_(bds, non_blocking=True)
                ev_out[b].record(st_out)
        main.wait_stream(st_out)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = host_max(dist, ctl, e0.elapsed_time(e1)) / e2e_steps
    e2e_ok = bool(torch.equal(hp[:SEQ], p[:SEQ].cpu()) and torch.equal(hds[-SEQ:], ds[-SEQ:].cpu()))
    del hs, hdp, hp, hds, bufs
    unmasked_ms = None
    if rank == 0 and not args.no_extra:             # the same kernel without the mask: every byte of the four tensors moves
        unmasked_ms = time_thunk(lambda: ops.softmax_fwd_bwd(s, dp, None, p=p, ds=ds), 10, 3, torch) * 1e3

    train = None
    if not args.no_train:
        torch.cuda.empty_cache()
        train = train_step_leg(torch, dist, ctl, rank, world, dev, args.steps)
        torch.cuda.empty_cache()
    spill = None
    if world == 1 and not args.no_train and not args.no_spill:
        spill = train_step_spill_leg(torch, dev, 2)
        torch.cuda.empty_cache()
    line = None
    if rank == 0:
        thunks = other_thunks(torch, ops, peak) if not args.no_extra else {}
        if unmasked_ms is not None:
            thunks["softmax_fwd_bwd, no mask[65536x2048,f16]"] = {
                "GB/s": round(DENSE_BYTES / unmasked_ms / 1e6, 1), "frac_of_peak": round(DENSE_BYTES / unmasked_ms / 1e6 / peak, 3),
                "us": round(unmasked_ms * 1e3, 1), "algorithmic_bytes": DENSE_BYTES, "launches_per_step": 1}
        cpu = None
        if world == 1 and not args.no_cpu:
            threads = physical_cores()
            sec, rows = cpu_reference_time(4, 3, threads)
            cpu = {"value": MOVED_BYTES * (rows / ROWS) / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                   "sample": f"4 of 32 (batch, head) blocks ({rows} rows), median of 3 passes of oracle/ref_chain.c"}
        achieved = MOVED_BYTES / (ms_step * 1e-3) / 1e9
        dense = DENSE_BYTES / (ms_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 storage / f32 accumulate", "data": "synthetic", "config": dict(CONFIG),
            "notes": {"per_gpu": "every rank runs the config's workload (weak scaling)", "mask": "causal, applied in-kernel",
                      "l2": "working set 0.8 GB per step, far larger than the 126 MB L2; no flush needed",
                      "bytes": "value, roofline and e2e count the bytes a causal kernel must move (masked inputs are never read); "
                               "dense_accounting counts all four tensors whole"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8TBs": achieved / 8000.0, "peak_kind": peak_kind + " copy bandwidth",
                         "traffic": NCU_TRAFFIC_BYTES, "traffic_source": "ncu capture of `bench.py --case softmax_full`, one launch",
                         "algorithmic_bytes": MOVED_BYTES, "kernel": "softmax_rows_kernel<half,8,fwd,bwd>",
                         "dense_accounting": {"bytes": DENSE_BYTES, "achieved": dense, "frac": dense / peak}},
            "cpu_baseline": cpu,
            "e2e": {"value": world * MOVED_BYTES / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 2 * ELEMS * 2, "d2h_bytes_per_step": 2 * ELEMS * 2, "verified": e2e_ok},
            "gpu_launches": args.steps, "clocks": clocks.summary(), "thunks": thunks, "train_step": train, "train_step_spill": spill,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier(group=ctl)
        dist.destroy_process_group()


def run_case(a):
    """One small single-kernel workload, a few launches, for a profiler (a few GB at most; inputs larger than the
    126 MB L2 so that DRAM counters mean something).  Cases: softmax (causal fwd+bwd, 8 heads x 2048 x 2048 f16),
    softmax_full (config 2), nll (2048 x 32000), rmsnorm / rmsnorm_bwd_acc (16384 x 3200), rope (16384 x 32 x 100),
    rope_pitched (the same rows written 128 wide), block_pad (the same shape), swiglu (4096 x 8640),
    gemm_nt / gemm_nn / gemm_tn / gemm_nn_acc (4096 x 3200 x 3200), qk / pv / ds_k / dst_q (block matmuls of the
    unfused step and of the attention adjoint), attn_fwd / attn_bwd (P and dS for the block matmuls) / attn_bwd_fused
    (--batch sequences of config 5), train_step (one config-5 forward+backward over --batch sequences; only for a
    single-pass launch list)."""
    import torch
    from cacti_b200 import ops
    for kv in a.tune:
        k, v = kv.split("=")
        if ops.lib().cacti_b200_tune(k.encode(), int(v)) != 0:
            raise SystemExit(f"tune {kv} rejected")
    gen = torch.Generator(device="cuda").manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=gen) * scale).half()

    def empty(*shape):
        return torch.empty(*shape, dtype=torch.float16, device="cuda")

    case = a.case
    if case in ("softmax", "softmax_full"):
        heads = 32 if case == "softmax_full" else 8
        s, dp = rnd(heads * 2048, 2048, scale=0.1), rnd(heads * 2048, 2048)
        p, ds = torch.empty_like(s), torch.empty_like(s)
        fn = lambda: ops.softmax_fwd_bwd(s, dp, (1, 2048, 0), p=p, ds=ds)
    elif case == "nll":
        lg = rnd(2048, 32000, scale=2.0)
        tg = torch.randint(0, 32000, (2048,), device="cuda", dtype=torch.int32, generator=gen)
        dl = torch.empty_like(lg)
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        fn = lambda: ops.softmax_nll_fwd_bwd(lg, tg, w_scalar=1.0 / 2048, dlogits=dl, status=st)
    elif case == "rmsnorm":
        x, dy, g = rnd(16384, 3200), rnd(16384, 3200), rnd(3200)
        y, dx, dg = torch.empty_like(x), torch.empty_like(x), empty(3200)
        ws = ops.rmsnorm_workspace(16384, 3200, x.device)
        fn = lambda: ops.rmsnorm_fwd_bwd(x, g, dy, 1e-6, y=y, dx=dx, dgamma=dg, workspace=ws)
    elif case == "rope":
        cos, sin = ops.rope_tables(2048, 100)
        q, dq = rnd(16384, 32, 100), rnd(16384, 32, 100)
        yq, dxq = torch.empty_like(q), torch.empty_like(q)
        fn = lambda: ops.rope_fwd_bwd(q, dq, cos, sin, y=yq, dx=dxq)
    elif case in ("rope_pitched", "block_pad"):
        q, out = rnd(16384, 32, 100), empty(16384, 32, 128)
        if case == "rope_pitched":
            cos, sin = ops.rope_tables(2048, 100)
            fn = lambda: ops.rope_fwd_pitched(q, cos, sin, 128, y=out)
        else:
            q4, out4 = q.view(8, 2048, 32, 100), out.view(8, 2048, 32, 128)
            fn = lambda: ops.block_pad(q4, 128, out=out4)
    elif case == "swiglu":
        ga, up, dh = rnd(4096, 8640), rnd(4096, 8640), rnd(4096, 8640)
        h, dga, dup = torch.empty_like(ga), torch.empty_like(ga), torch.empty_like(ga)
        fn = lambda: ops.swiglu_fwd_bwd(ga, up, dh, h=h, dgate=dga, dup=dup)
    elif case == "train_step":
        from cacti_b200 import dp as DP, llama_step as LS
        cfg = LS.LlamaShape.open_llama_3b()
        P = LS.init_weights(cfg, torch.device("cuda"))
        grads, _ = DP.alloc_bucketed_grads(P)
        step = LS.TrainStep(cfg, P, a.batch)
        tok = torch.randint(0, cfg.vocab, (a.batch * cfg.seq,), device="cuda", dtype=torch.int32, generator=gen)
        tgt = torch.randint(0, cfg.vocab, (a.batch * cfg.seq,), device="cuda", dtype=torch.int32, generator=gen)
        fn = lambda: step.forward_backward(tok, tgt, grads)
    elif case == "rmsnorm_bwd_acc":        # the adjoint in Accumulate mode (dX += ...), as every norm of the step runs it
        x, dy, g = rnd(16384, 3200), rnd(16384, 3200), rnd(3200)
        dx, dg = rnd(16384, 3200), empty(3200)
        ws = ops.rmsnorm_workspace(16384, 3200, x.device)
        fn = lambda: ops.rmsnorm_bwd(x, g, dy, 1e-6, dx=dx, dgamma=dg, beta_dx=1, workspace=ws)
    elif case == "gemm_nn_acc":            # dx += dy W (beta = 1): old C comes in by TMA
        m, n, k = 4096, 3200, 3200
        x, w, c = rnd(m, n), rnd(n, k, scale=0.02), rnd(m, k)
        fn = lambda: ops.gemm(x, w, False, False, beta=1.0, c=c)
    elif case in ("gemm_nt", "gemm_nn", "gemm_tn"):
        m, n, k = 4096, 3200, 3200
        if case == "gemm_nt":          # y = x W^T (forward projection)
            x, w, c = rnd(m, k), rnd(n, k, scale=0.02), empty(m, n)
            fn = lambda: ops.gemm(x, w, False, True, c=c)
        elif case == "gemm_nn":        # dx = dy W
            x, w, c = rnd(m, n), rnd(n, k, scale=0.02), empty(m, k)
            fn = lambda: ops.gemm(x, w, False, False, c=c)
        else:                          # dW = dy^T x
            x, w, c = rnd(m, n), rnd(m, k), empty(n, k)
            fn = lambda: ops.gemm(x, w, True, False, c=c)
    elif case in ("qk", "pv", "ds_k", "dst_q", "attn_fwd", "attn_bwd", "attn_bwd_fused"):
        bsz, sq, h, hd = a.batch, 2048, 32, 100
        if case == "qk":
            q, kk, c = rnd(bsz, sq, h, hd), rnd(bsz, sq, h, hd), empty(bsz, sq, h, sq)
            ws = torch.empty(ops.lib().cacti_b200_gemm_workspace_bytes(sq, sq, hd, bsz, h), dtype=torch.uint8, device="cuda")
            fn = lambda: ops.block_gemm(q, kk, False, True, alpha=0.1, c=c, workspace=ws)
        elif case == "pv":
            pr, v, c = rnd(bsz, sq, h, sq, scale=0.02), rnd(bsz, sq, h, hd), empty(bsz, sq, h, hd)
            ws = torch.empty(ops.lib().cacti_b200_gemm_workspace_bytes(sq, hd, sq, bsz, h), dtype=torch.uint8, device="cuda")
            fn = lambda: ops.block_gemm(pr, v, False, False, c=c, workspace=ws)
        elif case in ("ds_k", "dst_q"):   # dq = dS K and dk = dS^T Q of the attention adjoint: hinted, operand padded to 128
            from cacti_b200 import capi
            dsm = torch.tril(rnd(bsz, sq, h, sq, scale=0.02).permute(0, 2, 1, 3)).permute(0, 2, 1, 3).contiguous()
            kp, c = ops.block_pad(rnd(bsz, sq, h, hd), 128), empty(bsz, sq, h, hd)
            if case == "ds_k":
                fn = lambda: ops.block_gemm(dsm, kp, False, False, alpha=0.1, c=c, tri=capi.TRI_A_LOWER, b_valid=hd)
            else:
                fn = lambda: ops.block_gemm(dsm, kp, True, False, alpha=0.1, c=c, tri=capi.TRI_A_UPPER, b_valid=hd)
        else:
            alpha = hd ** -0.5
            q, kk, v, do = (ops.block_pad(rnd(bsz, sq, h, hd), 128) for _ in range(4))
            ctx, st = ops.attention_fwd(q, kk, v, hd, alpha)
            if case == "attn_fwd":
                fn = lambda: ops.attention_fwd(q, kk, v, hd, alpha, ctx=ctx, stats=st)
            elif case == "attn_bwd":
                pp, dss = empty(bsz, sq, h, sq), empty(bsz, sq, h, sq)
                fn = lambda: ops.attention_bwd_prep(q, kk, v, do, ctx, st, alpha, p=pp, ds=dss)
            else:
                dq, dk, dv = empty(bsz, sq, h, hd), empty(bsz, sq, h, hd), empty(bsz, sq, h, hd)
                fn = lambda: ops.attention_bwd(q, kk, v, do, ctx, st, alpha, dq=dq, dk=dk, dv=dv)
    else:
        raise SystemExit(f"unknown case {case}")
    for _ in range(a.launches):
        fn()
    torch.cuda.synchronize()
    print("done", case)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the per-thunk table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-train", action="store_true", help="skip the config-5 training-step leg")
    ap.add_argument("--train-only", action="store_true", help="print only the config-5 train_step entry (for sweeps; not a bench line)")
    ap.add_argument("--no-spill", action="store_true", help="skip the config-5 leg under the spill policy (N = 1 only)")
    ap.add_argument("--case", default=None, help="run one small single-kernel workload (see run_case) and exit")
    ap.add_argument("--launches", type=int, default=3, help="launches of the --case workload")
    ap.add_argument("--batch", type=int, default=2, help="sequences for the attention / train_step cases")
    ap.add_argument("--tune", action="append", default=[], metavar="KNOB=VALUE",
                    help="set a cacti_b200_tune knob before a --case run (repeatable), e.g. gemm_pair=1")
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()

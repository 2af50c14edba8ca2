#!/usr/bin/env python
"""Benchmark of the Zoph_RNN inference forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2]

One "step" = one pass of the hot path over one synthetic minibatch of the workload (teacher-forced
scoring: gather -> LSTM stack -> attention -> softmax log-probs; for c4: one batched beam decode).
Prints ONE JSON line (rank 0).  `value` is whole-job throughput with inputs resident in HBM; `e2e` is the
same metric through the host-buffer C-ABI call (H2D of the ids and D2H of the results inside the timed
region).  The line also carries `parity` (the GPU results of the timed model against the CPU oracle on a
sample of the same batch), `cpu_baseline`, and - for the default workload - `configs`: the other four
benchmark configurations, a few steps each.  With --gpus N >= 2 sentences shard by rank (weak scaling, no
collective) and the line adds `c5_sharded`: configuration 5 with its softmax sharded by vocabulary rows over
the N ranks (strong scaling, NCCL all-gathers), split by stage.
`--impl reference` times the CPU restatement of the reference's math (the oracle) on the host cores on a
bounded sample of the same workload: the full minibatch width, fewer time steps.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from zoph_rnn_b200 import synth  # noqa: E402

WORKLOADS = {
    # BASELINE.json configs[0..4]
    "c1": dict(desc="LM 1x100 V=10k B=8 T=35 fp32", kind="lm", L=1, H=100, Vs=0, Vt=10000, B=8, S=0, T=35,
               att=0, feed=0, scale=0.08, dist="uniform", zipf=None),
    "c2": dict(desc="seq2seq 4x1000 V=50k/50k B=128 S=50 T=50 global-dot attention + feed-input fp32", kind="s2s",
               L=4, H=1000, Vs=50000, Vt=50000, B=128, S=(50, 50), T=(50, 50), att=2, feed=1, scale=0.1,
               dist="uniform", zipf=1.1),
    # small stand-in with config 2's layer shapes (H=1000, B=128, feed-input, global attention) for profiler captures
    "c2s": dict(desc="profiling stand-in: 1x1000 V=8k/8k B=128 S=4 T=4 global-dot attention + feed-input fp32", kind="s2s",
                L=1, H=1000, Vs=8000, Vt=8000, B=128, S=(4, 4), T=(4, 4), att=2, feed=1, scale=0.1,
                dist="uniform", zipf=1.1),
    "c3": dict(desc="seq2seq 2x1000 V=40k/40k B=64 S~U[10,80] T=60 local-p D=10 + feed-input fp32", kind="s2s",
               L=2, H=1000, Vs=40000, Vt=40000, B=64, S=(10, 80), T=(60, 60), att=1, feed=1, scale=0.1,
               dist="uniform", zipf=1.1),
    # small stand-in with config 3's layer shapes (H=1000, B=64, local-p D=10, feed-input, ragged sources)
    "c3s": dict(desc="profiling stand-in: 1x1000 V=8k/8k B=64 S~U[10,24] T=4 local-p D=10 + feed-input fp32", kind="s2s",
                L=1, H=1000, Vs=8000, Vt=8000, B=64, S=(10, 24), T=(4, 4), att=1, feed=1, scale=0.1,
                dist="uniform", zipf=1.1),
    "c4": dict(desc="beam decode 2x1000 V=50k global-dot attention beam 12, 64 sentences S~U[10,50]", kind="decode",
               L=2, H=1000, Vs=50000, Vt=50000, B=64, S=(10, 50), T=None, att=2, feed=1, scale=0.1,
               dist="uniform", zipf=1.1, beam=12, max_ratio=2.0, min_ratio=0.5, longest_sent=100),
    # short-sentence stand-in with config 4's shapes (768 hypothesis columns, V=50k) for profiler captures
    "c4s": dict(desc="profiling stand-in: beam decode 2x1000 V=50k global-dot attention beam 12, 64 sentences S~U[4,6]",
                kind="decode", L=2, H=1000, Vs=50000, Vt=50000, B=64, S=(4, 6), T=None, att=2, feed=1, scale=0.1,
                dist="uniform", zipf=1.1, beam=12, max_ratio=2.0, min_ratio=0.5, longest_sent=100),
    "c5": dict(desc="LM 2x2048 V=200k B=256 T=64, bf16 weights", kind="lm", L=2, H=2048, Vs=0, Vt=200000, B=256, S=0,
               T=64, att=0, feed=0, scale=0.02, dist="normal", zipf=1.05, bf16_weights=True),
}


ARITH = {
    "f32": "fp32-accurate: tcgen05 on split operands (fp16 hi + scaled fp16 lo: 3 MMAs per product, fp32 accumulate) "
           "when H >= 64, else fp32 FMA",
    "f32_3xtf32": "fp32-accurate: tcgen05 3xTF32 (hi/lo split operands, fp32 accumulate)",
    "f32_f16x2": "fp32-accurate: tcgen05 on fp16 hi + scaled fp16 lo operands (3 MMAs per product, fp32 accumulate)",
    "f32_simt": "exact fp32 FMA kernels",
    "bf16": "tcgen05 bf16 operands, fp32 accumulate and state",
    "tf32": "tcgen05 tf32 operands, fp32 accumulate and state",
}


def make_cfg(w):
    return synth.make_cfg(w["L"], w["H"], w["Vs"], w["Vt"], lm=int(w["kind"] == "lm"), attention=w["att"],
                          feed_input=w["feed"], D=10)


def make_inputs(w, seed, B=None):
    B = B or w["B"]
    if w["kind"] == "lm":
        tin, tout = synth.make_lm_batch(w["Vt"], B, w["T"], seed=seed, zipf_s=w["zipf"])
        return dict(src=None, tin=tin, tout=tout, tokens=int((tout != -1).sum()))
    if w["kind"] == "s2s":
        src, tin, tout = synth.make_s2s_batch(w["Vs"], w["Vt"], B, w["S"][0], w["S"][1], w["T"][0], w["T"][1],
                                              seed=seed, zipf_s=w["zipf"])
        return dict(src=src, tin=tin, tout=tout, tokens=int((tout != -1).sum()))
    srcs = synth.make_decode_sources(w["Vs"], B, w["S"][0], w["S"][1], seed=seed, zipf_s=w["zipf"])
    return dict(srcs=srcs)


def sample_clocks_start(path):
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    try:
        f = open(path, "w")
        return subprocess.Popen(["nvidia-smi", "--query-gpu=" + q, "--format=csv,noheader,nounits", "-lms", "50"],
                                stdout=f, stderr=subprocess.DEVNULL), f
    except OSError:
        return None, None


def sample_clocks_stop(proc, f, path, gpu_index):
    out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
    if proc is None:
        return out
    proc.terminate()
    try:
        proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
        proc.kill()
    f.close()
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in open(path):
        p = [x.strip() for x in line.split(",")]
        if len(p) < 9 or not p[0].isdigit() or int(p[0]) != gpu_index:
            continue
        try:
            sm.append(float(p[1])); mx.append(float(p[2]))
        except ValueError:
            continue
        for nm, v in zip(names, p[5:9]):
            if v.lower().startswith("active"):
                reasons.add(nm)
    if sm:
        out = dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
    return out


def host_cores():
    """Host threads this process may use."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def reference_sample(w):
    """The bounded CPU sample of a scoring workload: the FULL minibatch width (so that every weight byte the CPU
    streams is used for as many columns as on the GPU) and only the first few source / target steps."""
    inp = make_inputs(w, 1234)
    Tn = 2 if w["H"] >= 2048 else 4
    src = inp["src"]
    if src is not None:
        src = np.ascontiguousarray(src[-Tn:])  # the reversed source is left-padded: its last rows are the words
    tin, tout = np.ascontiguousarray(inp["tin"][:Tn]), np.ascontiguousarray(inp["tout"][:Tn])
    S_full = inp["src"].shape[0] if inp["src"] is not None else 0
    sample = (f"all {w['B']} sentences x first {Tn} of {inp['tin'].shape[0]} target steps"
              + (f" and {Tn} of {S_full} source steps" if src is not None else "") + ", full model")
    return src, tin, tout, sample


def run_reference(args, w, rank, emit):
    """CPU arm: the oracle (a port of the reference's kernel math; the reference itself cannot be built
    for this machine) on a bounded sample of the workload, all host threads."""
    if rank != 0:
        return
    from oracle import oracle_lib as ol
    ol.build()
    cfg = make_cfg(w)
    weights = synth.make_weights(cfg, seed=1234, dist=w["dist"], scale=w["scale"], round_bf16=bool(w.get("bf16_weights")))
    om = ol.OracleModel(cfg, weights)
    ol.set_acc_float(True)  # float accumulation = the reference's SGEMM arithmetic
    ol.set_num_threads(host_cores())  # launchers such as torchrun export OMP_NUM_THREADS=1
    cores = ol.num_threads()
    if w["kind"] == "decode":
        Bs = 1
        inp = make_inputs(w, 1234, B=Bs)
        sample = f"{Bs} of {w['B']} sentences, full beam {w['beam']} (the reference decodes one sentence at a time)"

        def step():
            ids, ln, sc = om.beam_decode(inp["srcs"], w["beam"], 1, w["min_ratio"], w["max_ratio"], 0.0, w["longest_sent"])
            return int(np.maximum(ln[:, 0] - 1, 0).sum())
    else:
        src, tin, tout, sample = reference_sample(w)

        def step():
            om.score_batch(src, tin, tout)
            return int((tout != -1).sum())
    for _ in range(min(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    toks = 0
    for _ in range(args.steps):
        toks += step()
    dt = time.perf_counter() - t0
    val = toks / dt
    unit = "tokens/s"
    line = dict(impl="reference", metric=metric_name(w), value=val, unit=unit, n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 * dt / args.steps, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=args.workload + ": " + w["desc"], sample=sample),
                cpu_baseline=dict(value=val, unit=unit, cores=cores, kind="port", sample=sample),
                e2e=dict(value=val, unit=unit, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    emit(line)


def metric_name(w):
    return "beam-decode tokens/sec" if w["kind"] == "decode" else "scored tokens/sec"


def cpu_baseline(w):
    """Bounded CPU sample (rank 0, N=1 only), reported next to the GPU number."""
    from oracle import oracle_lib as ol
    ol.build()
    cfg = make_cfg(w)
    weights = synth.make_weights(cfg, seed=1234, dist=w["dist"], scale=w["scale"], round_bf16=bool(w.get("bf16_weights")))
    om = ol.OracleModel(cfg, weights)
    ol.set_acc_float(True)
    ol.set_num_threads(host_cores())
    if w["kind"] == "decode":
        inp = make_inputs(w, 1234, B=1)
        t0 = time.perf_counter()
        ids, ln, sc = om.beam_decode(inp["srcs"], w["beam"], 1, w["min_ratio"], w["max_ratio"], 0.0, w["longest_sent"])
        dt = time.perf_counter() - t0
        toks = int(np.maximum(ln[:, 0] - 1, 0).sum())
        sample = f"1 of {w['B']} sentences, full beam {w['beam']}"
    else:
        src, tin, tout, sample = reference_sample(w)
        t0 = time.perf_counter()
        om.score_batch(src, tin, tout)
        dt = time.perf_counter() - t0
        toks = int((tout != -1).sum())
        sample += ", 1 pass"
    ol.set_acc_float(False)
    return dict(value=toks / dt, unit="tokens/s", cores=ol.num_threads(), kind="port", sample=sample)


PARITY_SENTENCES = 8


def parity_check(w, cfg, weights, model, dtype, inp):
    """The timed model's results against the CPU oracle (double accumulation) on a sample of the SAME batch: the first
    PARITY_SENTENCES sentences over all their steps (a sentence scores the same alone as inside the batch).  fp32-
    accurate modes: largest relative log-prob error against 1e-5, plus the fp32 noise floor of this input (how far
    the oracle itself moves when its GEMMs accumulate in fp32 like the reference's SGEMM, in three summation orders,
    instead of in double);
    bf16 / tf32: perplexity within 0.5 %.  Decoding: the hypotheses of the first sentences, token for token."""
    from oracle import oracle_lib as ol
    ol.build()
    ol.set_num_threads(host_cores())
    om = ol.OracleModel(cfg, weights)
    exact = dtype in ("f32", "f32_simt", "f32_3xtf32", "f32_f16x2")
    if w["kind"] == "decode":
        n = 2
        srcs = inp["srcs"][:n]
        kw = dict(beam=w["beam"], k_best=1, min_ratio=w["min_ratio"], max_ratio=w["max_ratio"], penalty=0.0,
                  longest_sent=w["longest_sent"])
        ids, ln, sc = om.beam_decode(srcs, **kw)
        gi, gl, gs = model.decode(srcs, **kw)
        same = bool(np.array_equal(ln, gl) and np.array_equal(ids, gi))
        out = dict(sample=f"first {n} sentences, beam {w['beam']}", hypotheses_identical=same,
                   max_score_diff=float(np.abs(sc - gs).max()))
        out["ok"] = same if exact else None
        return out
    ns = min(PARITY_SENTENCES, w["B"])
    Tn = 16 if w["H"] >= 2048 else inp["tin"].shape[0]
    src = None
    if inp["src"] is not None:
        src = np.ascontiguousarray(inp["src"][:, :ns])
        keep = (src != -1).any(axis=1)  # rows that are padding for all of these sentences
        src = np.ascontiguousarray(src[keep])
    tin, tout = np.ascontiguousarray(inp["tin"][:Tn, :ns]), np.ascontiguousarray(inp["tout"][:Tn, :ns])
    want = om.score_batch(src, tin, tout)
    got, _ = model.get_error(src, tin, tout)
    msk = tout != -1
    out = dict(sample=f"first {ns} sentences x {Tn} target steps of the timed batch, full model")
    if exact:
        floor, _ = ol.fp32_noise_floor(lambda: om.score_batch(src, tin, tout)[msk], want[msk])
        use = msk
        if cfg["attention"] == 1:
            # local-p cuts its window at int(p_t): where p_t sits within fp32 rounding of an integer the window may
            # shift by one position, and feed-input carries that to the end of the sentence; those tokens are set aside
            clear, margin = ol.localp_clear_tokens(om, src, tin, tout)
            use = msk & clear
            out.update(window_margin_min=margin, tokens_after_near_integer_window=int((msk & ~clear).sum()))
        err = np.abs(got - want)[use] / np.abs(want[use])
        out.update(tokens=int(use.sum()), max_rel_err=float(err.max()), mean_rel_err=float(err.mean()), tol=1e-5,
                   fp32_noise_floor=floor, ok=bool(err.max() <= 1e-5 + floor), ok_without_floor=bool(err.max() <= 1e-5))
    else:
        n = msk.sum()
        pg, pw = float(np.exp(-got[msk].sum() / n)), float(np.exp(-want[msk].sum() / n))
        out.update(ppl=pg, ppl_oracle=pw, ppl_rel_err=abs(pg - pw) / pw, tol=5e-3, ok=bool(abs(pg - pw) / pw <= 5e-3),
                   max_abs_logp_err=float(np.abs(got - want)[msk].max()))
    return out


def measure(args, w, cfg, dtype, rank, world, steps=None, parity=False):
    """Builds the model in `dtype`, times K steps on the device (value), K steps through the host-buffer entry
    point (e2e) and an instrumented pass for per-kernel durations.  Returns a dict of raw measurements."""
    import tempfile
    import torch
    import torch.distributed as dist
    from zoph_rnn_b200 import api

    steps = steps or args.steps
    weights = synth.make_weights(cfg, seed=1234, dist=w["dist"], scale=w["scale"], round_bf16=bool(w.get("bf16_weights")))
    dtype_id = dict(f32=0, bf16=1, tf32=2, f32_simt=3, f32_3xtf32=4, f32_f16x2=5)[dtype]
    model = api.neuralMT_model(cfg, dtype=dtype_id)
    model.load_weights(weights)
    # sentences are sharded by rank (weak scaling: every rank scores/decodes its own minibatch, no collective)
    inp = make_inputs(w, 1234 + rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    if w["kind"] == "decode":
        srcs = inp["srcs"]
        lens = np.array([len(s) for s in srcs], dtype=np.int32)
        S_max, n = int(lens.max()), len(srcs)
        padded = np.full((S_max, n), -1, dtype=np.int32)
        for i, s in enumerate(srcs):
            padded[S_max - len(s):, i] = s
        d_src = torch.as_tensor(padded).cuda()
        Lmax = w["longest_sent"] + 4
        d_ids = torch.empty(n * Lmax, dtype=torch.int32, device="cuda")
        d_len = torch.empty(n, dtype=torch.int32, device="cuda")
        d_sc = torch.empty(n, dtype=torch.float32, device="cuda")

        def step_device():
            model.decode_device(d_src, lens, S_max, w["beam"], 1, w["min_ratio"], w["max_ratio"], 0.0,
                                w["longest_sent"], d_ids, d_len, d_sc)

        def step_host():
            model.decode(srcs, w["beam"], 1, w["min_ratio"], w["max_ratio"], 0.0, w["longest_sent"])
        h2d = int(lens.sum()) * 4
        d2h = n * (Lmax + 2) * 4
        step_device()
        torch.cuda.synchronize()
        tokens_per_step = int(np.maximum(d_len.cpu().numpy() - 1, 0).sum())  # emitted 1-best tokens incl. <EOF>
        ncols = n * synth.beam_cap(w["beam"], w["Vt"])
    else:
        src, tin, tout = inp["src"], inp["tin"], inp["tout"]
        T, B = tin.shape
        S = src.shape[0] if src is not None else 0
        d_src = torch.as_tensor(src).cuda() if src is not None else None
        d_tin, d_tout = torch.as_tensor(tin).cuda(), torch.as_tensor(tout).cuda()
        d_lp = torch.empty(T * B, dtype=torch.float32, device="cuda")
        p_src = torch.as_tensor(src).pin_memory() if src is not None else None
        p_tin, p_tout = torch.as_tensor(tin).pin_memory(), torch.as_tensor(tout).pin_memory()

        def step_device():
            model.get_error_device(d_src, S, d_tin, d_tout, T, B, d_lp)

        def step_host():
            model.get_error(p_src, p_tin, p_tout)
        h2d = (S * B + 2 * T * B) * 4
        d2h = T * B * 4
        tokens_per_step = inp["tokens"]
        ncols = T * B

    for _ in range(max(args.warmup, 3)):
        step_device()
    barrier()
    clk_dir = tempfile.mkdtemp(prefix="zrnn_bench_")
    clk_path = os.path.join(clk_dir, f"clocks_{dtype}_rank{rank}.csv")
    proc, f = sample_clocks_start(clk_path)
    api.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(steps):
        step_device()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = api.launch_count()
    # Per-kernel durations for the roofline: the same K steps again with a CUDA-event pair around every launch
    # group.  This pass launches eagerly (event pairs cannot be read back out of a replayed graph), so the
    # durations include any launch gap: they are upper bounds on kernel time, lower bounds on achieved bandwidth.
    api.lib().zrnn_kernel_timing(1)
    api.reset_launch_count()
    for _ in range(steps):
        step_device()
    torch.cuda.synchronize()
    eager_launches = api.launch_count()
    ktime = api.kernel_timing_report()
    api.lib().zrnn_kernel_timing(0)
    if launches == 0:
        launches = eager_launches  # the timed region replayed a CUDA graph holding this many kernel nodes per K steps
    # end-to-end through the host-buffer entry point (warmed up like the device path: its second call captures the
    # CUDA graph of the pass on the library's own stream)
    for _ in range(3):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step_host()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sample_clocks_stop(proc, f, clk_path, torch.cuda.current_device())
    try:
        os.remove(clk_path)
        os.rmdir(clk_dir)
    except OSError:
        pass
    par = parity_check(w, cfg, weights, model, dtype, inp) if (parity and rank == 0) else None
    del weights
    if world > 1:
        t = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1]) / 1e3
        tk = torch.tensor([tokens_per_step], dtype=torch.int64, device="cuda")
        dist.all_reduce(tk, op=dist.ReduceOp.SUM)
        tokens_all = int(tk[0])
    else:
        tokens_all = tokens_per_step
    del model
    torch.cuda.empty_cache()
    return dict(ms=ms, e2e_s=e2e_s, tokens_all=tokens_all, launches=int(launches), ktime=ktime, clocks=clocks,
                h2d=h2d, d2h=d2h, ncols=ncols, steps=steps, parity=par)


def run_c5_sharded(args, rank, world, steps):
    """Config 5 on N GPUs: ONE minibatch scored by all ranks (strong scaling) through zrnn_score_batch_sharded.
    Sentences are sharded for the recurrent stack, the softmax matrix by vocabulary rows; two NCCL all-gathers per
    batch (top-layer vectors in operand form, then 3 floats per token), issued by the library behind the C ABI.
    Timed end to end from host id arrays to host log-probs, max over ranks; the stage split is rank 0's device time."""
    import torch
    import torch.distributed as dist
    from zoph_rnn_b200 import api, sharded
    w = WORKLOADS["c5"]
    cfg = make_cfg(w)
    dtype = "bf16"
    weights = synth.make_weights(cfg, seed=1234, dist=w["dist"], scale=w["scale"], round_bf16=True)
    comm = api.Communicator.from_torch_distributed()
    model = sharded.ShardedModel(cfg, weights, comm, dtype=1)
    inp = make_inputs(w, 1234)  # the same minibatch on every rank
    for _ in range(3):
        model.score(None, inp["tin"], inp["tout"])
    torch.cuda.synchronize()
    dist.barrier()
    stages = {k: 0.0 for k in api.Communicator.STAGES}
    t0 = time.perf_counter()
    for _ in range(steps):
        lp, _ = model.score(None, inp["tin"], inp["tout"])
        for k, v in comm.last_stage_ms().items():
            stages[k] += v / steps
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t[0])
    out = None
    if rank == 0:
        T, B = inp["tin"].shape
        H, V = cfg["H"], cfg["V_tgt"]
        Bp = -(-B // world)
        par = None
        if not args.no_parity:
            from oracle import oracle_lib as ol
            ol.build()
            ol.set_num_threads(host_cores())
            ns, Tn = PARITY_SENTENCES, 16
            tin, tout = np.ascontiguousarray(inp["tin"][:Tn, :ns]), np.ascontiguousarray(inp["tout"][:Tn, :ns])
            want = ol.OracleModel(cfg, weights).score_batch(None, tin, tout)
            got = lp[:Tn, :ns]
            msk = tout != -1
            n = msk.sum()
            pg, pw = float(np.exp(-got[msk].sum() / n)), float(np.exp(-want[msk].sum() / n))
            par = dict(sample=f"first {ns} sentences x {Tn} target steps of the sharded batch against the CPU oracle",
                       ppl=pg, ppl_oracle=pw, ppl_rel_err=abs(pg - pw) / pw, tol=5e-3, ok=bool(abs(pg - pw) / pw <= 5e-3),
                       max_abs_logp_err=float(np.abs(got - want)[msk].max()))
        out = dict(workload="c5: " + w["desc"], metric=metric_name(w), value=inp["tokens"] * steps / dt, unit="tokens/s",
                   n_gpus=world, steps=steps, warmup=3, ms_per_step=1e3 * dt / steps, scaling="strong", dtype=dtype,
                   timing="host clock around the host-buffer C-ABI call (ids in, log-probs out), max over ranks",
                   sharding="sentences by rank for the LSTM stack + vocabulary rows of D by rank; NCCL all-gather of the "
                            "top-layer vectors (bf16 operand form) and of (max, sum, target) per token, inside the library",
                   stages_ms_rank0={k: round(v, 4) for k, v in stages.items()},
                   nvlink_bytes_per_step_per_rank=int((world - 1) * (T * Bp * (-(-H // 64) * 64) * 2 + 3 * 4 * T * Bp * world)),
                   e2e=dict(value=inp["tokens"] * steps / dt, unit="tokens/s", h2d_bytes_per_step=(T * Bp + T * Bp * world) * 4,
                            d2h_bytes_per_step=T * Bp * world * 4),
                   parity=par)
    del model, weights
    comm.close()
    torch.cuda.empty_cache()
    return out


def cell_phases(w, dtype_name):
    """Runs one hidden-to-hidden LSTM cell (H x B of the workload) with the kernel's phase stamps on and returns, per
    phase, the min / mean / max over the launch's CTAs in microseconds since the first CTA started."""
    import ctypes
    import torch
    from zoph_rnn_b200 import api
    H, B = w["H"], w["B"] * (w.get("beam", 1) if w["kind"] == "decode" else 1)
    rng = np.random.default_rng(0)
    mats = [(rng.standard_normal(H * H) * 0.02).astype(np.float32) for _ in range(8)]
    tensors = []
    for g in range(4):
        tensors += [mats[g], np.zeros(H, np.float32)]
    tensors += mats[4:]
    layer = api.Hidden_To_Hidden_Layer(H, dtype=dict(f32=0, bf16=1, tf32=2, f32_simt=3, f32_3xtf32=4, f32_f16x2=5)[dtype_name])
    layer.load_weights(tensors)
    x, h0, c0 = (torch.randn(H * B, device="cuda") for _ in range(3))
    mask = torch.ones(B, dtype=torch.int32, device="cuda")
    for _ in range(3):
        layer.forward_prop(x, mask, h0, c0)
    torch.cuda.synchronize()
    buf = torch.zeros(8 * 4096, dtype=torch.int64, device="cuda")
    api.check(api.lib().zrnn_debug_tc_profile(ctypes.c_void_p(buf.data_ptr())))
    layer.forward_prop(x, mask, h0, c0)
    torch.cuda.synchronize()
    api.check(api.lib().zrnn_debug_tc_profile(None))
    t = buf.cpu().numpy().reshape(-1, 8)
    t = t[t[:, 0] > 0]
    if len(t) == 0:
        return dict(error="no stamps: this shape does not run the split-K tensor-core cell")
    rel = (t - t[:, 0].min()) / 1e3
    names = ["start", "setup_done", "accumulators_complete", "partial_tile_pushed", "cluster_barrier_passed",
             "slots_read", "gate_math_done", "stores_issued"]
    return dict(kernel="lstm_cell", H=H, B=B, dtype=dtype_name, ctas=int(len(t)), unit="us",
                phases={n: dict(min=round(float(rel[:, i].min()), 2), mean=round(float(rel[:, i].mean()), 2),
                                max=round(float(rel[:, i].max()), 2)) for i, n in enumerate(names)})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16", "tf32", "f32_simt", "f32_3xtf32", "f32_f16x2"],
                    help="arithmetic of the GEMM-shaped work (f32 = fp32-accurate: split-operand tensor cores when H >= 64)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-bf16", action="store_true", help="skip the additional bf16 measurement of an f32 run")
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the `configs` block (configurations 1, 3, 4, 5 on one GPU) and the `c5_sharded` block")
    ap.add_argument("--no-parity", action="store_true", help="skip the comparison with the CPU oracle")
    ap.add_argument("--cell-phases", action="store_true",
                    help="diagnostic: device-side phase times of one LSTM cell launch of the workload's layer shape "
                         "(per-CTA %%globaltimer stamps written by the kernel), printed as one JSON line")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    # stdout carries the ONE JSON line and nothing else: whatever a library prints to file descriptor 1 meanwhile (NCCL's
    # version banner, for one) goes to stderr
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        os.write(json_fd, (json.dumps(obj) + "\n").encode())

    if args.impl == "reference":
        run_reference(args, w, rank, emit)
        return

    import torch
    import torch.distributed as dist

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    if args.cell_phases:
        if rank == 0:
            emit(cell_phases(w, args.dtype))
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    cfg = make_cfg(w)
    if args.workload == "c5" and args.dtype == "f32":
        args.dtype = "bf16"  # config 5 is specified with bf16 weights
    peaks, peak_src = {}, "fallback"
    pk_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk_path):
        peaks, peak_src = json.load(open(pk_path)), "measured"
    parity = not args.no_parity
    r = measure(args, w, cfg, args.dtype, rank, world, parity=parity)
    extra = None
    if args.dtype == "f32" and not args.no_bf16 and cfg["H"] % 8 == 0:
        extra = measure(args, w, cfg, "bf16", rank, world, parity=parity)
    line = None
    if rank == 0:
        line = summary(args.workload, w, cfg, r, args.dtype, peaks, peak_src, full=True)
        line.update(n_gpus=world, warmup=max(args.warmup, 3), higher_is_better=True, scaling="weak", vs_baseline=None,
                    data="synthetic")
        line["config"].update(sharding="sentences by rank, no collective",
                              l2="weights and embeddings (>1 GB) exceed the 126 MB L2 every step")
        if extra:
            line["bf16"] = summary(args.workload, w, cfg, extra, "bf16", peaks, peak_src, full=True)
    # the other benchmark configurations, a few steps each (single GPU: they are parity + throughput records, not
    # scaling lines)
    if args.workload == "c2" and world == 1 and not args.no_configs:
        others = {}
        for name, dt_name, k in (("c1", "f32", 5), ("c3", "f32", 3), ("c4", "f32", 2), ("c5", "bf16", 2)):
            wo = WORKLOADS[name]
            co = make_cfg(wo)
            ro = measure(args, wo, co, dt_name, rank, world, steps=k, parity=parity)
            others[name] = summary(name, wo, co, ro, dt_name, peaks, peak_src, full=False)
        line["configs"] = others
    # configuration 5 with its softmax sharded by vocabulary rows over the N ranks
    if world > 1 and args.workload in ("c2", "c5") and not args.no_configs:
        c5 = run_c5_sharded(args, rank, world, steps=3)
        if rank == 0:
            line["c5_sharded"] = c5
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def summary(name, w, cfg, r, dtype, peaks, peak_src, full):
    """One measured configuration as a JSON object (the headline line when full, else the short form of `configs`)."""
    k = r["steps"]
    out = dict(metric=metric_name(w), value=r["tokens_all"] * k / (r["ms"] / 1e3), unit="tokens/s", steps=k,
               ms_per_step=r["ms"] / k, dtype=dtype,
               config=dict(workload=name + ": " + w["desc"], arithmetic=ARITH[dtype]),
               clocks=r["clocks"], gpu_launches=r["launches"],
               launch_mode="CUDA graph replay of the scoring pass" if w["kind"] != "decode" else "eager launches",
               e2e=dict(value=r["tokens_all"] * k / r["e2e_s"], unit="tokens/s", h2d_bytes_per_step=r["h2d"],
                        d2h_bytes_per_step=r["d2h"]),
               roofline=roofline(w, cfg, r["ktime"], peaks, peak_src, r["ncols"], dtype))
    if full:
        out["kernels"] = r["ktime"]
    else:
        out["kernel_ms"] = {n: round(v["ms"], 3) for n, v in (r["ktime"] or {}).items()}
    out["parity"] = r["parity"]
    return out


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the LSTM cell kernel on an 8-matrix
# layer (no feed-input operand) from an ncu capture, keyed by (kernel class, dtype, H, B): a figure applies only to the
# shape it was captured on; every other shape reports null.  The capture ran the c2s workload, whose layer shapes are
# configuration 2's.
NCU_TRAFFIC = {("lstm_cell", "f32", 1000, 128): 35.2e6, ("lstm_cell", "f32_f16x2", 1000, 128): 35.2e6,
               ("lstm_cell", "f32_3xtf32", 1000, 128): 71.6e6, ("lstm_cell", "bf16", 1000, 128): 17.9e6}


def roofline(w, cfg, ktime, peaks, peak_src, softmax_cols, dtype):
    """Roofline of the dominant kernel class.  Durations are CUDA-event pairs around every launch of the class in
    the instrumented pass (one pair per encoder layer sweep).  Algorithmic bytes per LSTM cell launch: the layer's
    H x H weight matrices as stored (4 or 2 bytes each) plus 5 H x B fp32 activations; flops of the softmax GEMM:
    2 V H N."""
    if not ktime:
        return None
    top = max(ktime, key=lambda k: ktime[k]["ms"])
    H = cfg["H"]
    B = w["B"] * (w.get("beam", 1) if w["kind"] == "decode" else 1)
    n = ktime[top]["launches"]
    avg_s = ktime[top]["ms"] / 1e3 / max(n, 1)
    wbytes = 2 if dtype == "bf16" else 4   # bytes per weight as the reference stores them (fp32) or bf16
    out = dict(kernel=top, launches=n, avg_launch_us=avg_s * 1e6, peak_source=peak_src, traffic=None)
    sm_flops = 2.0 * cfg["V_tgt"] * H * softmax_cols
    sm_bytes = cfg["V_tgt"] * H * wbytes + (H * softmax_cols + 2 * softmax_cols) * 4
    # the vocabulary GEMM is bound by whichever lower bound is larger: its flops at the tensor peak or its
    # algorithmic bytes at the copy peak
    sm_tensor_bound = (sm_flops / (float(peaks.get("bf16_tflops_sustained", 1400.0)) * 1e12)
                       > sm_bytes / (float(peaks.get("hbm_gbs", 6650.0)) * 1e9))
    if top == "softmax_gemm" and sm_tensor_bound:
        flops = sm_flops
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        out.update(bound="tensor", unit="TFLOP/s", peak=peak, achieved=flops / avg_s / 1e12,
                   algorithmic_flops_per_launch=flops,
                   note="2*V*H*N flops; peak = measured sustained bf16 cuBLAS (also the denominator for the "
                        "fp32-accurate modes, which spend 3 tensor-core passes per product)")
    elif top == "lstm_cell":
        L = cfg["num_layers"]
        mats = 8.0
        if cfg["feed_input"] and not cfg["lm"]:
            mats = (8.0 * (2 * L - 1) + 12.0) / (2 * L) if w["kind"] != "decode" else (8.0 * (L - 1) + 12.0) / L
        alg = mats * H * H * wbytes + (4 * H + 5.0 * H * B) * 4
        cap = NCU_TRAFFIC.get((top, dtype, H, B))
        if cap:  # captured on an 8-matrix launch; the average launch of this workload holds `mats` matrices
            alg8 = 8.0 * H * H * wbytes + (4 * H + 5.0 * H * B) * 4
            out["traffic"] = cap * alg / alg8
            out["traffic_note"] = ("ncu capture of an 8-matrix cell launch of this shape, scaled by the algorithmic "
                                   "bytes of the workload's average launch")
        out.update(bound="hbm", unit="GB/s", peak=float(peaks.get("hbm_gbs", 6650.0)), achieved=alg / avg_s / 1e9,
                   algorithmic_bytes_per_launch=alg,
                   note=f"avg {mats:.2f} HxH matrices of {wbytes}-byte weights + 5 HxB fp32 activations per launch")
    elif top == "softmax_gemm":
        alg = sm_bytes
        out.update(bound="hbm", unit="GB/s", peak=float(peaks.get("hbm_gbs", 6650.0)), achieved=alg / avg_s / 1e9,
                   algorithmic_bytes_per_launch=alg, note="D once + h columns + 2 floats per column")
    else:
        out.update(bound="hbm", unit="GB/s", peak=float(peaks.get("hbm_gbs", 6650.0)), achieved=None,
                   note="no algorithmic-bytes model for this class")
    if out.get("achieved"):
        out["frac"] = out["achieved"] / out["peak"]
    return out


if __name__ == "__main__":
    main()

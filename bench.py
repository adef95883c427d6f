"""Benchmark of the decode hot path: Llama-3-8B-architecture, int8 per-channel weights, bf16 activations,
batch 32, 2048-token context, greedy decode — tokens per second of the whole job.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --case {gemv|gemm|attention|prefill_gemm|prefill_attention|prefill_model|w8a8|suite} [...]

Default case ("step").  A step is one decode step of the whole batch (32 new tokens).  Weights are random-init (N(0, 0.02),
quantised with the engine's quantizer), the 2048-token context is synthetic KV (N(0,1) * 0.5, one seed for the whole cache,
each tensor-parallel rank keeps its heads): there is no dataset or checkpoint on this path.  Tensor parallel over N GPUs of
one node (one process per GPU, NCCL): total work is fixed, so scaling is "strong".  The working set (7.5 GB of weights +
8.6 GB of KV per step) is far larger than L2, so no flush is needed between iterations.

Printed JSON (rank 0): value = device-resident throughput (token ids fed back on the device, CUDA events around exactly K
steps, max over ranks; the block of K steps is repeated and the median block is reported, with min and max beside it);
e2e = the same through model(state, outputs, inputs) with HOST buffers (pinned ids in, token ids out every step);
e2e_logits = the same with the engine's real graph output, full logits to the host every step; roofline = the largest
launch of the dominant kernel (the tcgen05 int8 DequantMatMul, gate/up shape) timed live over the model's own weights;
gemm_kernel / attention_kernel = every DequantMatMul launch of one step, and the decode-attention launches of one step,
each timed in one graph; cpu_baseline = the CPU oracle on a bounded slice of the same workload.
`--impl reference` times the CPU restatement of the engine's CPU backend instead (the engine itself, Rust + LLVM 18,
cannot be built here) with all host threads.

The other cases time single kernels of the path the way the step's kernels are fed: every launch reads a different copy of
its weights / KV (copies x size > L2), the launches are replayed from one CUDA graph, CUDA events on the launching stream.
Algorithmic bytes: GEMM  N*K + N*sizeof(scale) + M*K*sizeof(act) + M*N*sizeof(out);  attention  2*B*Hkv*L*D*2 + Q + out.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
import zlib

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA3_8B = dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                 intermediate_size=14336, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)
TINYLLAMA = dict(hidden_size=2048, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                 intermediate_size=5632, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)
BATCH, CONTEXT = 32, 2048
METRIC, UNIT = "decode_tokens_per_second", "tok/s"


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s, 'measured' | 'fallback'): the driver-written measurement of this pool's B200s."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def workload_name(cfg):
    return (f"llama3-8b-arch int8-W bf16 decode, batch {BATCH}, context {CONTEXT}, "
            f"{cfg['num_hidden_layers']} layers, vocab {cfg['vocab_size']}")


# --------------------------------------------------------------------------------------------------------
# CPU arm: the oracle (a restatement of the engine's CPU backend) on a bounded slice of the workload
# --------------------------------------------------------------------------------------------------------
class CpuSample:
    """A bounded slice of one decode step on the host, extrapolated to the whole step.

    Per call: the seven DequantMatMuls, norms, RoPE, SwiGLU and residual adds of ONE layer at batch 32 in full; its
    attention over `att_batch` of the 32 sequences (scaled by 32/att_batch; the reference's attention kernel is scalar
    and single-threaded, sequences are independent); the lm_head over vocab/`head_div` rows (scaled by head_div).
    Layer time is multiplied by the depth.  Data are generated once, outside the timed region."""

    def __init__(self, cfg, context=CONTEXT, att_batch=4, head_div=8, seed=0):
        import numpy as np

        from oracle import c_oracle
        from oracle import ref_ops as R
        self.np, self.R, self.c = np, R, c_oracle
        self.cfg, self.context, self.att_batch, self.head_div = cfg, context, att_batch, head_div
        rng = np.random.default_rng(seed)
        h, f, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
        hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

        def w(n, k):
            return rng.integers(-127, 128, size=(n, k), dtype=np.int8), rng.uniform(0.002, 0.02, n).astype(np.float32)

        self.layer = dict(q=w(hq * d, h), k=w(hkv * d, h), v=w(hkv * d, h), o=w(h, hq * d), g=w(f, h), u=w(f, h), dn=w(h, f))
        self.head = w(v // head_div, h)
        self.kc = (rng.standard_normal((att_batch, hkv, context + 1, d)) * 0.5).astype(np.float32)
        self.vc = (rng.standard_normal((att_batch, hkv, context + 1, d)) * 0.5).astype(np.float32)
        self.x = rng.standard_normal((BATCH, h)).astype(np.float32)
        self.ones = np.ones(h, np.float32)
        self.cos, self.sin = R.rope_table(context + 1, d, cfg["rope_theta"], "bf16")
        self.desc = (f"1 of {cfg['num_hidden_layers']} layers (attention on {att_batch} of {BATCH} sequences) + lm_head on "
                     f"1/{head_div} of the vocabulary of one batch-{BATCH} decode step at context {context}, extrapolated")

    def step(self):
        np, R, c_oracle, cfg = self.np, self.R, self.c, self.cfg
        hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        ctx, L, ab = self.context, self.layer, self.att_batch
        cr, sr = self.cos[ctx:ctx + 1], self.sin[ctx:ctx + 1]

        def mm(a, wq_s):  # M > 1: dequantise to an f32 workspace, then sgemm (all BLAS threads)
            return R.round_bf16(R.dequant_matmul_variant_c(a, wq_s[0], wq_s[1]))

        t0 = time.perf_counter()
        x = self.x
        n1 = R.round_bf16(R.rms_norm(x, self.ones, cfg["rms_norm_eps"]))
        q = mm(n1, L["q"]).reshape(BATCH, 1, hq, d).transpose(0, 2, 1, 3)
        k = mm(n1, L["k"]).reshape(BATCH, 1, hkv, d).transpose(0, 2, 1, 3)
        vv = mm(n1, L["v"]).reshape(BATCH, 1, hkv, d).transpose(0, 2, 1, 3)
        q = R.round_bf16(R.rope(q, cr, sr))
        k = R.round_bf16(R.rope(k, cr, sr))
        t_a0 = time.perf_counter()
        R.kv_cache_update(self.kc, k[:ab], ctx)
        R.kv_cache_update(self.vc, vv[:ab], ctx)
        a_sub = c_oracle.attention(np.ascontiguousarray(q[:ab]), self.kc, self.vc, 1.0 / np.sqrt(d), ctx + 1)
        t_att = time.perf_counter() - t_a0
        a = np.tile(R.round_bf16(a_sub), (BATCH // ab, 1, 1, 1)).transpose(0, 2, 1, 3).reshape(BATCH, hq * d)
        x = R.round_bf16(x + mm(a, L["o"]))
        n2 = R.round_bf16(R.rms_norm(x, self.ones, cfg["rms_norm_eps"]))
        hh = R.round_bf16(R.swish_mul(mm(n2, L["g"]), mm(n2, L["u"])))
        x = R.round_bf16(x + mm(hh, L["dn"]))
        t_layer = time.perf_counter() - t0 - t_att + t_att * (BATCH / ab)
        t0 = time.perf_counter()
        logits = mm(R.round_bf16(R.rms_norm(x, self.ones, cfg["rms_norm_eps"])), self.head)
        _ = [R.argmax_last(r) for r in logits]
        t_head = (time.perf_counter() - t0) * self.head_div
        return t_layer * cfg["num_hidden_layers"] + t_head


def run_reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample = CpuSample(cfg)
    desc = sample.desc
    times = []
    for i in range(args.warmup + args.steps):
        t = sample.step()
        if i >= args.warmup:
            times.append(t)
    sec = sum(times) / len(times)
    val = BATCH / sec
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(cfg), "l2": "inputs larger than L2"},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) == 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(float(s[0])) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(float(self.samples[0][1])), "reasons": reasons,
                "samples": len(mhz)}


def fill_synthetic_context(model, cfg, rank, world, dev):
    """The 2048-row context of every layer from ONE seed for the whole (unsharded) cache; a tensor-parallel rank keeps its
    own kv heads, so the model sees the same context at every N."""
    import torch
    hkv, d = cfg["num_key_value_heads"], cfg["head_dim"]
    per = hkv // world
    g = torch.Generator(device=dev).manual_seed(1)
    for t in model.k_cache + model.v_cache:
        full = torch.randn((BATCH, hkv, CONTEXT, d), generator=g, device=dev, dtype=torch.float32) * 0.5
        mine = full[:, rank * per:(rank + 1) * per]
        t[:, :, :CONTEXT].copy_((mine * 40).clamp(-127, 127).round() if model.kv_int8 else mine)
        del full
    for t in model.k_scale + model.v_scale:
        t[:, :, :CONTEXT].fill_(1.0 / 80)


def run_gpu_arm(args, cfg):
    import torch
    import torch.distributed as dist

    from my_nn_engine_b200 import collective, ffi
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    collective.set_communicator(rank, world)
    lib = ffi.lib()

    steps, warm, blocks = args.steps, max(args.warmup, 8), max(args.blocks, 1)  # the first 8 steps are always run (their ids are reported)
    max_seq = CONTEXT + warm + steps + 16
    state = random_llama_state(cfg, seed=0, device=str(dev))  # identical on every rank (same seed)
    def build_model(output, fused):
        m = DecoderModel(cfg, state, dtype="bf16", max_seq_len=max_seq, batch=BATCH, tp_rank=rank, tp_world=world,
                         output=output, use_graph=True, kv_int8=args.kv == "int8", tp_fused=fused)
        fill_synthetic_context(m, cfg, rank, world, dev)
        return m

    model = build_model("ids", True)
    ids0 = torch.randint(0, cfg["vocab_size"], (BATCH,), device=dev, dtype=torch.int64,
                         generator=torch.Generator(device=dev).manual_seed(7))
    stream = torch.cuda.Stream(device=dev)  # a real stream handle: the library treats NULL as the model's own stream
    torch.cuda.set_stream(stream)
    # Several GPUs: one step through the host entry first, which reads the status words of the bounded waits.  If the
    # peer-memory reduction reports a wait that ran out (a width this build could not be tried on), every rank switches to
    # the NCCL all-reduce together, and the line says so, instead of spending the whole run in timed-out waits.
    tp_note = None
    if world > 1 and model.tp_fused:
        ok = 1
        ffi.set_option(ffi.OPT_WAIT_BUDGET_US, 300000)
        try:
            model.step(ids0.cpu(), CONTEXT)
        except ffi.MynnError as exc:
            ok, tp_note = 0, str(exc)
        ffi.set_option(ffi.OPT_WAIT_BUDGET_US, 2000000)
        agreed = torch.tensor([ok], device=dev, dtype=torch.int32)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            dist.barrier()
            torch.cuda.synchronize()
            model.close()
            model = build_model("ids", False)
            tp_note = "nccl all-reduce: the peer-memory reduction reported a timed-out wait at this width (%s)" % (tp_note or "on another rank")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput ----
    past = CONTEXT
    l0 = lib.mynn_b200_launch_count()
    tok_dev = torch.zeros(BATCH, dtype=torch.int32, device=dev)
    model.step_device(ids0, past, tok_dev)  # first call captures the graph
    launches_per_step = lib.mynn_b200_launch_count() - l0
    past += 1
    first_ids = [tok_dev.cpu().numpy().copy()]
    for _ in range(7):  # the greedy ids of the first 8 steps: the same at every N unless a near-tie flips
        model.step_device(None, past, tok_dev)
        past += 1
        first_ids.append(tok_dev.cpu().numpy().copy())
    for _ in range(max(warm - 8, 0)):
        model.step_device(None, past)
        past += 1
    barrier()
    block_ms, past0 = [], past  # every block decodes the same rows [past0, past0 + steps): equal work per block
    with ClockSampler(local) as clocks:
        torch.cuda.cudart().cudaProfilerStart()  # lets `ncu --profile-from-start off` see only the timed steps
        for _ in range(blocks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            past = past0
            e0.record(stream)
            for _ in range(steps):
                model.step_device(None, past)
                past += 1
            e1.record(stream)
            barrier()
            block_ms.append(max_over_ranks(e0.elapsed_time(e1)) / steps)
        torch.cuda.cudart().cudaProfilerStop()
    srt = sorted(block_ms)
    ms_dev = srt[len(srt) // 2]

    # ---- end to end through model(state, outputs, inputs) with host buffers ----
    def time_e2e(m, past):
        tok = ids0.cpu()
        for i in range(3):
            out = m.step(tok, past + steps - 3 + i)  # warm-up on rows the timed steps overwrite later
            tok = out.clone() if m.output == "ids" else ids0.cpu()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            out = m.step(tok, past)  # pinned ids -> device, graph replay, result -> pinned host, stream sync
            if m.output == "ids":
                tok = out
            past += 1
        barrier()
        return max_over_ranks((time.perf_counter() - t0) * 1e3) / steps, past

    ms_e2e, _ = time_e2e(model, past0)

    # ---- roofline figures, timed live over this model's own layers ----
    roof = kernel_roofline(model, cfg, world, dev)
    gemm_all = gemm_kernel_wide(model, cfg, world, dev)
    attn_all = attention_kernel_figure(model, cfg, world, dev)
    weight_bytes = model.weight_bytes()
    h2d, d2h = model.h2d_bytes_per_step, model.d2h_bytes_per_step
    kv_int8 = model.kv_int8
    tp_fused = model.tp_fused
    model.close()
    del model
    torch.cuda.empty_cache()

    # ---- the engine's own output mode: full logits to the host every step, argmax there ----
    e2e_logits = None
    if not args.no_logits:
        lm = build_model("logits", tp_fused or world == 1)
        ms_lg, _ = time_e2e(lm, past0)
        e2e_logits = {"value": BATCH * 1e3 / ms_lg, "unit": UNIT, "ms_per_step": ms_lg, "h2d_bytes_per_step": lm.h2d_bytes_per_step,
                      "d2h_bytes_per_step": lm.d2h_bytes_per_step,
                      "what": "model(state, outputs, inputs) returning the logits [batch, vocab] to pinned host memory every step "
                              "(the engine's graph output; the host-side argmax of its loop is not part of the timed call)"}
        lm.close()
        del lm
    del state

    if rank == 0:
        peak, _, peak_kind = measured_peaks()
        ids = __import__("numpy").stack(first_ids)
        line = {"metric": METRIC, "value": BATCH * 1e3 / ms_dev, "unit": UNIT, "n_gpus": world, "steps": steps,
                "warmup": warm, "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": workload_name(cfg), "parallelism": f"tp{world}", "l2": "inputs larger than L2",
                           "kv_cache": "int8 + per-token scale (quant_kv_cache option; not the headline configuration)" if kv_int8 else "bf16",
                           "tp_reduce": ("nvlink peer memory, fused with add + rmsnorm" if tp_fused else ((tp_note or "nccl") if world > 1 else "none"))},
                "timed_blocks": {"blocks": blocks, "steps_per_block": steps, "ms_per_step_median": ms_dev,
                                 "ms_per_step_min": srt[0], "ms_per_step_max": srt[-1]},
                "clocks": clocks.summary(),
                "e2e": {"value": BATCH * 1e3 / ms_e2e, "unit": UNIT, "ms_per_step": ms_e2e,
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "gpu_launches": int(launches_per_step * steps),
                "launches_per_step": int(launches_per_step),
                "token_ids_first_8_steps_crc32": zlib.crc32(ids.astype("<i4").tobytes()),
                "token_ids_first_step_crc32": zlib.crc32(ids[0].astype("<i4").tobytes()),
                # the ids themselves, so that runs at different N can be compared pick by pick: the logits of a random-init model
                # are nearly uniform, and a top-2 gap below the bf16 resolution may fall either way when the f32 summation order
                # changes with the number of ranks
                "token_ids_first_step": [int(t) for t in ids[0]]}
        if e2e_logits:
            line["e2e_logits"] = e2e_logits
        for key, fig in (("roofline", roof), ("gemm_kernel", gemm_all), ("attention_kernel", attn_all)):
            if fig:
                fig["peak"], fig["peak_kind"] = peak, peak_kind
                fig["frac"] = fig["achieved"] / peak
                line[key] = fig
        # algorithmic bytes of a whole step on this rank: weights once + KV once (per KV head) over HBM
        kv_row_bytes = cfg["head_dim"] + 2 if kv_int8 else cfg["head_dim"] * 2
        kv_bytes = 2 * cfg["num_hidden_layers"] * BATCH * (cfg["num_key_value_heads"] // world) * (CONTEXT + warm + steps // 2) * kv_row_bytes
        step_bytes = weight_bytes - cfg["vocab_size"] * cfg["hidden_size"] + kv_bytes
        line["step_hbm"] = {"algorithmic_bytes_per_gpu": int(step_bytes), "achieved_gbs": step_bytes / ms_dev / 1e6,
                            "frac_of_peak": step_bytes / ms_dev / 1e6 / peak}
        if world == 1 and not args.no_cpu:
            try:
                sample = CpuSample(cfg)
                secs = [sample.step() for _ in range(4)][1:]
                sec = sum(secs) / len(secs)
                line["cpu_baseline"] = {"value": BATCH / sec, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                                        "sample": sample.desc + " (mean of 3 samples after 1 warm-up)"}
            except Exception as e:  # the CPU leg must never hide the GPU number
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                                        "sample": f"failed: {e}"}
        print(json.dumps(line), flush=True)
    collective.destroy_communicator()
    if world > 1:
        dist.destroy_process_group()


def _graph_us(launch_all, n_launches, reps=3):
    """Capture `launch_all()` (which enqueues n_launches kernels on the current stream) in one CUDA graph and return the best
    of `reps` replays in microseconds (CUDA events on the launching stream)."""
    import torch
    stream = torch.cuda.current_stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        launch_all()
    g.replay()
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3)
    return best


def kernel_roofline(model, cfg, world, dev):
    """The gate/up DequantMatMul kernel at M = batch over every layer's own weight block, back to back (each block is read
    once, 3.7 GB in total, so the bytes come from HBM); CUDA events on the launching stream.  Only the GEMM kernel is
    timed, as it runs in the decode step: there the activation limbs are written by the preceding RMSNorm kernel, here
    they are converted once before the timed region."""
    import torch

    from my_nn_engine_b200 import ops
    h, f = cfg["hidden_size"], cfg["intermediate_size"] // world
    blocks = [(w, s) for w, s in zip(model._keep, model._keep[1:]) if w.dtype == torch.int8 and tuple(w.shape) == (2 * f, h)]
    act = torch.randn(BATCH, h, device=dev).bfloat16()
    out = torch.empty(BATCH, 2 * f, device=dev, dtype=torch.bfloat16)
    for w, s in blocks[:3]:
        ops.dequant_matmul(act, w, s, out=out)  # leaves the limbs of `act` in the workspace
    torch.cuda.synchronize()

    def launch_all():
        for w, s in blocks:
            ops.dequant_matmul_same_act(act, w, s, out=out)

    us = _graph_us(launch_all, len(blocks)) / len(blocks)
    n, k, m = 2 * f, h, BATCH
    alg = n * k + n * 2 + m * k * 2 + m * n * 2
    # DRAM traffic of one launch: dram__bytes_read.sum + dram__bytes_write.sum of a separate ncu capture of this kernel at
    # this shape on one GPU (117,945,856 + 3,616,256 bytes); not measured by this run, and not available for a shard
    traffic = 117945856 + 3616256 if world == 1 else None
    return {"kernel": "i8_stream_gemm_kernel (gate/up DequantMatMul, M=32, N=%d, K=%d; limbs written by the preceding kernel as in the step)" % (n, k),
            "bound": "hbm", "achieved": alg / us / 1e3, "unit": "GB/s", "us_per_launch": us, "algorithmic_bytes": alg,
            "traffic": traffic,
            "traffic_source": "separate ncu capture of one launch of this kernel at this shape (tensor parallel 1)" if traffic else None}


def gemm_kernel_wide(model, cfg, world, dev):
    """EVERY DequantMatMul launch of one decode step (per layer qkv, o, gate/up, down; then lm_head) over the model's own
    weights, in step order, in one graph: weight bytes of the step / time.  The limbs of one random activation tensor per
    reduction length are prepared before the timed region, as the step's producers do it outside these kernels."""
    import torch

    from my_nn_engine_b200 import ffi, ops
    weights = [(w, s) for w, s in zip(model._keep, model._keep[1:]) if w.dtype == torch.int8 and w.dim() == 2][1:]  # [0] is the embedding
    spaces, outs = {}, {}
    for w, s in weights:
        n, k = w.shape
        if k not in spaces:
            act = torch.randn(BATCH, k, device=dev).bfloat16()
            ws = torch.zeros(ffi.lib().mynn_b200_dequant_matmul_workspace_bytes(BATCH, n, k), dtype=torch.uint8, device=dev)
            ops.dequant_matmul(act, w, s, workspace=ws)
            spaces[k] = (act, ws)
        if (n, s.dtype) not in outs:
            outs[(n, s.dtype)] = torch.empty(BATCH, n, device=dev, dtype=s.dtype)
    torch.cuda.synchronize()

    def launch_all():
        for w, s in weights:
            act, ws = spaces[w.shape[1]]
            ops.dequant_matmul_same_act(act, w, s, out=outs[(w.shape[0], s.dtype)], workspace=ws)

    us = _graph_us(launch_all, len(weights))
    wbytes = sum(w.numel() for w, _ in weights)
    alg = wbytes + sum(s.numel() * s.element_size() + BATCH * w.shape[1] * 2 + BATCH * w.shape[0] * s.element_size() for w, s in weights)
    return {"kernel": "i8_stream_gemm_kernel, all %d launches of one step" % len(weights), "bound": "hbm", "achieved": alg / us / 1e3,
            "unit": "GB/s", "us_per_step": us, "weight_bytes": wbytes, "algorithmic_bytes": alg, "traffic": None}


def attention_kernel_figure(model, cfg, world, dev):
    """The decode-attention kernel at the bench geometry over every layer's own KV cache (distinct memory per launch),
    one graph."""
    import torch

    from my_nn_engine_b200 import ops
    if model.kv_int8:
        return None
    hq, hkv, d = cfg["num_attention_heads"] // world, cfg["num_key_value_heads"] // world, cfg["head_dim"]
    q = torch.randn(BATCH, hq, 1, d, device=dev).bfloat16()
    out = torch.empty_like(q)
    active = CONTEXT
    ws = ops.attention_workspace(BATCH, hq, hkv, d, model.max_seq_len, dev)
    ops.attention(q, model.k_cache[0], model.v_cache[0], d ** -0.5, active, out=out, workspace=ws)
    torch.cuda.synchronize()

    def launch_all():
        for k, v in zip(model.k_cache, model.v_cache):
            ops.attention(q, k, v, d ** -0.5, active, out=out, workspace=ws)

    n = len(model.k_cache)
    us = _graph_us(launch_all, n) / n
    alg = 2 * BATCH * hkv * active * d * 2 + 2 * q.numel() * 2
    return {"kernel": "attention_decode_kernel (batch %d, %d q / %d kv heads, head_dim %d, %d kv rows)" % (BATCH, hq, hkv, d, active),
            "bound": "hbm", "achieved": alg / us / 1e3, "unit": "GB/s", "us_per_launch": us, "algorithmic_bytes": alg, "traffic": None}


# --------------------------------------------------------------------------------------------------------
# single-kernel cases
# --------------------------------------------------------------------------------------------------------
def _time_launches(fns, reps=3):
    """fns: callables launching one kernel each; microseconds per launch, replayed from one graph on a side stream."""
    import torch
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for f in fns[:2]:
            f()
        torch.cuda.synchronize()
        return _graph_us(lambda: [f() for f in fns], len(fns), reps) / len(fns)


def _torch_dt(name):
    import torch
    return {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[name]


def case_gemm(m, n, k, dtype="bf16", ksplit=0, copies=None, kernel="tcgen05_i8", layout="nk", resident=False):
    """One DequantMatMul shape.  resident=True replays over ONE weight copy (an L2-resident figure when it fits)."""
    import torch

    from my_nn_engine_b200 import ffi, ops
    td = _torch_dt(dtype)
    copies = 1 if resident else (copies or max(3, int(600e6 // (n * k)) + 1))
    shape = (n, k) if layout == "nk" else (k, n)
    ws = [torch.randint(-127, 128, shape, dtype=torch.int8, device="cuda") for _ in range(copies)]
    sc = (torch.rand(n, device="cuda") * 0.018 + 0.002).to(td)
    act = torch.randn(m, k, device="cuda").to(td)
    out = torch.empty(m, n, device="cuda", dtype=td)
    ffi.set_option(ffi.OPT_KSPLIT, ksplit)
    wsp = ops.dequant_matmul_workspace(m, n, k, act.device) if kernel == "tcgen05_i8" and layout == "nk" else None
    fns = [(lambda w=w: ops.dequant_matmul(act, w, sc, axis=0 if layout == "nk" else 1, out=out, workspace=wsp)) for w in ws]
    if resident:
        fns = fns * 16
    us = _time_launches(fns)
    ffi.set_option(ffi.OPT_KSPLIT, 0)
    esz = act.element_size()
    alg = n * k + n * esz + m * k * esz + m * n * esz
    hbm, tf, kind = measured_peaks()
    if m > 32:  # a dense contraction: tensor throughput (bf16-equivalent flops 2 M N K)
        return {"kernel": "dequant_matmul/prefill_" + kernel, "m": m, "n": n, "k": k, "dtype": dtype, "us": us,
                "TFLOPs_bf16_equivalent": 2.0 * m * n * k / us / 1e6, "frac_of_%s_bf16_peak" % kind: 2.0 * m * n * k / us / 1e6 / tf}
    return {"kernel": "dequant_matmul/" + kernel, "layout": layout, "m": m, "n": n, "k": k, "dtype": dtype, "ksplit": ksplit,
            "weights": "one copy replayed (L2-resident if it fits)" if resident else f"{copies} distinct copies (> L2)", "us": us,
            "GBps": alg / us / 1e3, "frac_of_%s_hbm_peak" % kind: alg / us / 1e3 / hbm, "algorithmic_bytes": alg}


def case_attention(b, hq, hkv, d, length, dtype="bf16", copies=None, kv="16bit"):
    """Decode attention; kv="int8" times the kernel for the int8 cache (bytes: int8 rows + one scale per row)."""
    import numpy as np
    import torch

    from my_nn_engine_b200 import ops
    td = _torch_dt(dtype)
    q8 = kv == "int8"
    kv_bytes = 2 * b * hkv * length * (d + 2) if q8 else 2 * b * hkv * length * d * 2
    copies = copies or max(3, int(600e6 // kv_bytes) + 1)
    q = torch.randn(b, hq, 1, d, device="cuda").to(td)
    out = torch.empty_like(q)
    ws = ops.attention_workspace(b, hq, hkv, d, length, q.device)
    if q8:
        ks = [torch.randint(-127, 128, (b, hkv, length, d), device="cuda", dtype=torch.int8) for _ in range(copies)]
        vs = [torch.randint(-127, 128, (b, hkv, length, d), device="cuda", dtype=torch.int8) for _ in range(copies)]
        sc = [(torch.rand(b, hkv, length, device="cuda") * 0.02 + 0.005).to(td) for _ in range(copies)]
        us = _time_launches([(lambda k=k, v=v, s=s: ops.attention_q8(q, k, v, s, s, 1 / np.sqrt(d), length, out=out, workspace=ws))
                             for k, v, s in zip(ks, vs, sc)])
    else:
        ks = [torch.randn(b, hkv, length, d, device="cuda").to(td) for _ in range(copies)]
        vs = [torch.randn(b, hkv, length, d, device="cuda").to(td) for _ in range(copies)]
        us = _time_launches([(lambda k=k, v=v: ops.attention(q, k, v, 1 / np.sqrt(d), length, out=out, workspace=ws))
                             for k, v in zip(ks, vs)])
    alg = kv_bytes + 2 * q.numel() * 2
    hbm, _, kind = measured_peaks()
    return {"kernel": "attention_decode_q8" if q8 else "attention_decode", "b": b, "hq": hq, "hkv": hkv, "d": d, "len": length,
            "dtype": dtype, "us": us, "GBps": alg / us / 1e3, "frac_of_%s_hbm_peak" % kind: alg / us / 1e3 / hbm, "algorithmic_bytes": alg}


def case_prefill_attention(b, hq, hkv, d, length, dtype="bf16"):
    """Causal self-attention of a whole prompt (Sq = kv length): 4 * Sq^2 / 2 * D * Hq * B flops."""
    import numpy as np
    import torch

    from my_nn_engine_b200 import ops
    td = _torch_dt(dtype)
    q = torch.randn(b, hq, length, d, device="cuda").to(td)
    ks = [torch.randn(b, hkv, length, d, device="cuda").to(td) for _ in range(2)]
    vs = [torch.randn(b, hkv, length, d, device="cuda").to(td) for _ in range(2)]
    out = torch.empty_like(q)
    us = _time_launches([(lambda k=k, v=v: ops.attention(q, k, v, 1 / np.sqrt(d), length, True, out=out)) for k, v in zip(ks, vs)])
    ops.attention_check()
    flops = 4.0 * length * (length + 1) / 2 * d * hq * b
    _, tf, kind = measured_peaks()
    return {"kernel": "attention_prefill", "b": b, "hq": hq, "hkv": hkv, "d": d, "len": length, "dtype": dtype, "us": us,
            "TFLOPs": flops / us / 1e6, "frac_of_%s_bf16_peak" % kind: flops / us / 1e6 / tf}


def case_prefill_model(arch="llama3-8b", batch=1, length=2048, chunk=None, layers=None, dtype="bf16", reps=3, kv_int8=False):
    """Whole-model prefill of ``length`` prompt tokens per sequence (random int8 weights of the named architecture) in
    chunks of ``chunk`` tokens.  Wall-clock per prompt, host call to host result (the last token's id)."""
    import numpy as np
    import torch

    from my_nn_engine_b200 import ops
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    cfg = dict(LLAMA3_8B if arch == "llama3-8b" else TINYLLAMA)
    if layers:
        cfg["num_hidden_layers"] = layers
    chunk = chunk or length
    state = random_llama_state(cfg, seed=0, device="cuda")
    model = DecoderModel(cfg, state, dtype=dtype, max_seq_len=length + 8, batch=batch, output="ids", max_prefill=chunk, kv_int8=kv_int8)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg["vocab_size"], size=(batch, length))
    times = []
    for _ in range(reps + 1):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for p0 in range(0, length, chunk):
            model.prefill(prompt[:, p0:p0 + chunk], p0)
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    ops.attention_check()
    best = min(times[1:])
    model.close()
    return {"kernel": "model_prefill", "arch": arch, "layers": cfg["num_hidden_layers"], "batch": batch, "len": length, "chunk": chunk,
            "dtype": dtype, "kv_cache": "int8" if kv_int8 else dtype, "ms": best * 1e3, "first_call_ms": times[0] * 1e3,
            "prompt_tok_per_s": batch * length / best}


def case_decode_model(arch="tinyllama", batch=1, context=128, steps=128, dtype="f16"):
    """Greedy decode of a small-batch model end to end through model(state, outputs, inputs): tokens per second after a
    prefilled prompt (the TinyLlama-1.1B-architecture configuration: batch 1, 128-token prompt, 128 greedy steps)."""
    import numpy as np
    import torch

    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    cfg = dict(LLAMA3_8B if arch == "llama3-8b" else TINYLLAMA)
    state = random_llama_state(cfg, seed=0, device="cuda")
    model = DecoderModel(cfg, state, dtype=dtype, max_seq_len=context + steps + 8, batch=batch, output="ids", max_prefill=context)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg["vocab_size"], size=(batch, context))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tok = model.prefill(prompt, 0).clone()
    t_prefill = time.perf_counter() - t0
    ids = [tok.numpy().copy()]
    for i in range(3):
        tok = model.step(tok, context + i).clone()
        ids.append(tok.numpy().copy())
    t0 = time.perf_counter()
    for i in range(3, steps):
        tok = model.step(tok, context + i)
        ids.append(tok.numpy().copy())
    sec = time.perf_counter() - t0
    model.close()
    wbytes = sum(v.numel() for k, v in state.items() if v.dtype == torch.int8 and "embed" not in k)
    hbm, _, kind = measured_peaks()
    ms = sec * 1e3 / (steps - 3)
    return {"kernel": "model_decode", "arch": arch, "batch": batch, "context": context, "steps": steps, "dtype": dtype,
            "ms_per_token": ms, "tok_per_s": batch * 1e3 / ms, "prefill_ms_first_call": t_prefill * 1e3,
            "weight_GBps": wbytes / ms / 1e6, "frac_of_%s_hbm_peak" % kind: wbytes / ms / 1e6 / hbm,
            "token_ids_crc32": zlib.crc32(np.stack(ids).astype("<i4").tobytes())}


def case_w8a8(m, n, k, dtype="bf16", copies=None):
    """QuantizedMatMul (int8 x int8) on the tcgen05 kernel; TOP/s counts 2 M N K integer operations."""
    import torch

    from my_nn_engine_b200 import ops
    td = _torch_dt(dtype)
    copies = copies or max(3, int(300e6 // (n * k)) + 1)
    ws = [torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8) for _ in range(copies)]
    lhs = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    ls = (torch.rand(m, device="cuda") * 0.05 + 0.005).to(td)
    rs = (torch.rand(n, device="cuda") * 0.018 + 0.002).to(td)
    out = torch.empty(m, n, device="cuda", dtype=td)
    wsp = ops.dequant_matmul_workspace(1, n, k, "cuda")
    us = _time_launches([(lambda w=w: ops.quantized_matmul(lhs, ls, w, rs, out=out, workspace=wsp)) for w in ws])
    ops.check_workspace(wsp)
    alg = n * k + m * k + 2 * (m + n) + 2 * m * n
    hbm, tf, kind = measured_peaks()
    return {"kernel": "quantized_matmul/tcgen05_i8", "m": m, "n": n, "k": k, "dtype": dtype, "us": us, "TOPs": 2.0 * m * n * k / us / 1e6,
            "frac_of_%s_bf16_peak" % kind: 2.0 * m * n * k / us / 1e6 / tf, "GBps": alg / us / 1e3,
            "frac_of_%s_hbm_peak" % kind: alg / us / 1e3 / hbm, "algorithmic_bytes": alg}


def run_case(args):
    def emit(res):
        print(json.dumps(res), flush=True)

    c = args.case
    prefill = c in ("prefill_gemm", "w8a8")
    args.m = args.m or (2048 if prefill else 32)
    args.n = args.n or (14336 if prefill else 28672)
    args.k = args.k or 4096
    args.b = args.b or (16 if c == "attention" else 1)
    args.len = args.len or (4096 if c == "attention" else 2048)
    if c == "gemv":  # the single-op GEMV configuration: f32 activation [1, 2048], W [2048, 5632] in both layouts
        for layout in ("nk", "kn"):
            for resident in (False, True):
                emit(case_gemm(1, 5632, 2048, "f32", layout=layout, resident=resident))
        emit(case_gemm(1, 5632, 2048, "bf16"))
    elif c == "gemm":
        emit(case_gemm(args.m, args.n, args.k, args.dtype, args.ksplit, args.copies, args.kernel, args.layout))
    elif c == "attention":
        emit(case_attention(args.b, args.hq, args.hkv, args.d, args.len, args.dtype, args.copies, args.kv))
    elif c == "prefill_gemm":
        emit(case_gemm(args.m, args.n, args.k, args.dtype, copies=args.copies or 3))
    elif c == "prefill_attention":
        emit(case_prefill_attention(args.b, args.hq, args.hkv, args.d, args.len, args.dtype))
    elif c == "prefill_model":
        emit(case_prefill_model(args.arch, args.b, args.len, args.chunk, args.layers, args.dtype, kv_int8=args.kv == "int8"))
    elif c == "decode_model":
        emit(case_decode_model(args.arch, args.b, dtype=args.dtype))
    elif c == "w8a8":
        emit(case_w8a8(args.m, args.n, args.k, args.dtype, args.copies))
    elif c == "suite":
        # the projections of both architectures at batch 1 and 32, the single-op GEMV, the attention shapes
        for m in (1, 32):
            for n, k in [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096)]:
                emit(case_gemm(m, n, k))
        for n, k in [(5632, 2048), (2560, 2048), (2048, 2048), (11264, 2048), (2048, 5632), (32000, 2048)]:
            emit(case_gemm(1, n, k))
        emit(case_attention(16, 32, 8, 128, 4096))
        emit(case_attention(32, 32, 8, 128, 2048))
        emit(case_attention(1, 32, 4, 64, 256))
    else:
        raise SystemExit(f"unknown case {c}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--blocks", type=int, default=10, help="how often the block of --steps timed steps is repeated (median reported)")
    ap.add_argument("--impl", default="mynn_b200", choices=["mynn_b200", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="override the depth (testing only; the default is the full model)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-logits", action="store_true", help="skip the e2e_logits leg (a second model instance)")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "16bit", "int8"],
                    help="KV cache storage; the headline configuration is bf16, int8 is the engine's quant_kv_cache option")
    ap.add_argument("--case", default="step", help="step (default) or a single-kernel case, see the module docstring")
    for name in ("m", "n", "k", "b", "len"):  # shape of a single-kernel case; the default depends on the case
        ap.add_argument("--" + name, type=int, default=None)
    for name, default in (("hq", 32), ("hkv", 8), ("d", 128), ("ksplit", 0)):
        ap.add_argument("--" + name, type=int, default=default)
    ap.add_argument("--copies", type=int, default=None)
    ap.add_argument("--chunk", type=int, default=None)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--kernel", default="tcgen05_i8", choices=["tcgen05_i8", "mma_sync"])
    ap.add_argument("--layout", default="nk", choices=["nk", "kn"])
    ap.add_argument("--arch", default="llama3-8b", choices=["llama3-8b", "tinyllama"])
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="library option set before the run (mynn_b200_set_option), e.g. decode_ring=0, fuse_rope=0, ksplit=4")
    args = ap.parse_args()
    if args.kv == "16bit":
        args.kv = "bf16"
    if args.option and args.impl != "reference":
        from my_nn_engine_b200 import ffi
        for item in args.option:
            name, _, value = item.partition("=")
            ffi.set_option(getattr(ffi, "OPT_" + name.upper()), int(value))
    if args.case != "step":
        return run_case(args)
    cfg = dict(LLAMA3_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        run_gpu_arm(args, cfg)


if __name__ == "__main__":
    main()

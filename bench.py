"""Benchmark of the decode hot path: Llama-3-8B-architecture, int8 per-channel weights, bf16 activations,
batch 32, 2048-token context, greedy decode — tokens per second of the whole job.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one decode step of the whole batch (32 new tokens).  Weights are random-init (N(0, 0.02), quantised with
the engine's quantizer), the 2048-token context is synthetic KV (N(0,1) * 0.5): there is no dataset or checkpoint
on this path.  Tensor parallel over N GPUs of one node (one process per GPU, NCCL): total work is fixed, so scaling
is "strong".  The working set (7.5 GB of weights + 8.6 GB of KV per step) is far larger than L2, so no flush is
needed between iterations.

Printed JSON (rank 0): value = device-resident throughput (token ids fed back on the device, CUDA events around
exactly K steps, max over ranks); e2e = the same through model(state, outputs, inputs) with HOST buffers (pinned
ids in, token ids out every step); roofline = the dominant kernel (the tcgen05 int8 DequantMatMul, gate/up shape at M=32) timed live over
the model's own per-layer weights; cpu_baseline = the CPU oracle on a bounded slice of the same workload.
`--impl reference` times the CPU restatement of the engine's CPU backend instead (the engine itself, Rust + LLVM 18,
cannot be built here) with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA3_8B = dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                 intermediate_size=14336, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)
BATCH, CONTEXT = 32, 2048
METRIC, UNIT = "decode_tokens_per_second", "tok/s"


def measured_peak_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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
            self._stop.wait(0.2)

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

    steps, warm = args.steps, max(args.warmup, 3)
    max_seq = CONTEXT + 2 * (steps + warm) + 64
    state = random_llama_state(cfg, seed=0, device=str(dev))  # identical on every rank (same seed)
    model = DecoderModel(cfg, state, dtype="bf16", max_seq_len=max_seq, batch=BATCH, tp_rank=rank, tp_world=world,
                         output="ids", use_graph=True, kv_int8=args.kv == "int8")
    del state
    torch.cuda.empty_cache()
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    for t in model.k_cache + model.v_cache:  # synthetic 2048-token context
        r = torch.randn(t[:, :, :CONTEXT].shape, generator=g, device=dev, dtype=torch.float32) * 0.5
        t[:, :, :CONTEXT].copy_((r * 40).clamp(-127, 127).round() if model.kv_int8 else r)
    for t in model.k_scale + model.v_scale:
        t[:, :, :CONTEXT].fill_(1.0 / 80)
    ids0 = torch.randint(0, cfg["vocab_size"], (BATCH,), device=dev, dtype=torch.int64,
                         generator=torch.Generator(device=dev).manual_seed(7))
    stream = torch.cuda.Stream(device=dev)  # a real stream handle: the library treats NULL as the model's own stream
    torch.cuda.set_stream(stream)

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
    model.step_device(ids0, past)  # first call captures the graph
    launches_per_step = lib.mynn_b200_launch_count() - l0
    past += 1
    for _ in range(warm - 1):
        model.step_device(None, past)
        past += 1
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        torch.cuda.cudart().cudaProfilerStart()  # lets `ncu --profile-from-start off` see only the timed steps
        e0.record(stream)
        for _ in range(steps):
            model.step_device(None, past)
            past += 1
        e1.record(stream)
        barrier()
        torch.cuda.cudart().cudaProfilerStop()
    ms_dev = max_over_ranks(e0.elapsed_time(e1)) / steps

    # ---- end to end through model(state, outputs, inputs) with host buffers ----
    tok = model.step(ids0.cpu(), past).clone()
    past += 1
    for _ in range(2):
        tok = model.step(tok, past).clone()
        past += 1
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = model.step(tok, past)  # pinned ids -> device, graph replay, token ids -> pinned host, stream sync
        past += 1
    barrier()
    ms_e2e = max_over_ranks((time.perf_counter() - t0) * 1e3) / steps

    # ---- roofline of the dominant kernel, timed live over this model's own layers ----
    roof = kernel_roofline(model, cfg, world, dev) if rank == 0 or world > 1 else None

    if rank == 0:
        peak, peak_kind = measured_peak_hbm()
        line = {"metric": METRIC, "value": BATCH * 1e3 / ms_dev, "unit": UNIT, "n_gpus": world, "steps": steps,
                "warmup": warm, "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": workload_name(cfg), "parallelism": f"tp{world}", "l2": "inputs larger than L2",
                           "kv_cache": "int8 + per-token scale (quant_kv_cache option; not the headline configuration)" if model.kv_int8 else "bf16",
                           "tp_reduce": ("nvlink peer loads fused into add+rmsnorm" if model.tp_fused else ("nccl" if world > 1 else "none"))},
                "clocks": clocks.summary(),
                "e2e": {"value": BATCH * 1e3 / ms_e2e, "unit": UNIT, "ms_per_step": ms_e2e,
                        "h2d_bytes_per_step": model.h2d_bytes_per_step, "d2h_bytes_per_step": model.d2h_bytes_per_step},
                "gpu_launches": int(launches_per_step * steps),
                "launches_per_step": int(launches_per_step)}
        if roof:
            roof["peak"], roof["peak_kind"] = peak, peak_kind
            roof["frac"] = roof["achieved"] / peak
            line["roofline"] = roof
        # algorithmic bytes of a whole step on this rank: weights once + KV once (per KV head) over HBM
        kv_row_bytes = cfg["head_dim"] + 2 if model.kv_int8 else cfg["head_dim"] * 2
        kv_bytes = 2 * cfg["num_hidden_layers"] * BATCH * (cfg["num_key_value_heads"] // world) * (CONTEXT + warm + steps // 2) * kv_row_bytes
        step_bytes = model.weight_bytes() - cfg["vocab_size"] * cfg["hidden_size"] + kv_bytes
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
    model.close()
    collective.destroy_communicator()
    if world > 1:
        dist.destroy_process_group()


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
    stream = torch.cuda.current_stream()
    for w, s in blocks[:3]:
        ops.dequant_matmul(act, w, s, out=out)  # leaves the limbs of `act` in the workspace
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):  # one graph of all launches: removes host launch gaps from the measurement
        for w, s in blocks:
            ops.dequant_matmul_same_act(act, w, s, out=out)
    g.replay()
    torch.cuda.synchronize()
    e0.record(stream)
    g.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / len(blocks)
    n, k, m = 2 * f, h, BATCH
    alg = n * k + n * 2 + m * k * 2 + m * n * 2
    # DRAM traffic of one launch from the ncu capture summarised in profiles/i8_stream_gemm_gateup_m32.md
    # (dram__bytes_read.sum + dram__bytes_write.sum at TP1: 117,935,616 + 4,291,328 bytes); the weight stream is
    # proportional to the shard, so it is scaled by 1/world for a tensor-parallel rank.
    traffic = (117935616 + 4291328) // world
    return {"kernel": "i8_stream_gemm_kernel (gate/up DequantMatMul, M=32, N=%d, K=%d; limbs written by the preceding kernel as in the step)" % (n, k),
            "bound": "hbm", "achieved": alg / us / 1e3, "unit": "GB/s", "us_per_launch": us, "algorithmic_bytes": alg,
            "traffic": traffic}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="mynn_b200", choices=["mynn_b200", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="override the depth (testing only; the default is the full model)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "int8"],
                    help="KV cache storage; the headline configuration is bf16, int8 is the engine's quant_kv_cache option")
    args = ap.parse_args()
    cfg = dict(LLAMA3_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        run_gpu_arm(args, cfg)


if __name__ == "__main__":
    main()

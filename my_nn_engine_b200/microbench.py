"""Per-kernel timing of the decode path against the HBM roofline.

    python -m my_nn_engine_b200.microbench gemm --m 32 --n 28672 --k 4096 [--dtype bf16] [--ksplit 0] [--copies 8]
    python -m my_nn_engine_b200.microbench attn --b 16 --hq 32 --hkv 8 --d 128 --len 4096
    python -m my_nn_engine_b200.microbench prefill_attn --len 8192
    python -m my_nn_engine_b200.microbench prefill_model --arch llama3-8b --len 2048
    python -m my_nn_engine_b200.microbench suite

Every launch reads a different copy of its weights / KV (copies x size > L2) and the launches are replayed from one
CUDA graph, so the time is device time of HBM-fed kernels without host launch gaps.  Algorithmic bytes:
GEMM  N*K + N*sizeof(scale) + M*K*sizeof(act) + M*N*sizeof(out);  attention  2*B*Hkv*L*D*2 + Q + out.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import ffi, ops

_DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _peak():
    try:
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        return float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        return 6650.0


def _peak_tflops():
    try:
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        return float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        return 1590.0


def _time_graph(fns, reps=3):
    """fns: list of callables launching one kernel each; returns microseconds per launch."""
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for f in fns[:2]:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        best = 1e30
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            g.replay()
            e1.record(s)
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e3 / len(fns))
    return best


def gemm(m, n, k, dtype="bf16", ksplit=0, copies=None, quiet=False, kernel="tcgen05_i8"):
    td = _DT[dtype]
    copies = copies or max(3, int(600e6 // (n * k)) + 1)
    ws = [torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda") for _ in range(copies)]
    sc = (torch.rand(n, device="cuda") * 0.018 + 0.002).to(td)
    act = torch.randn(m, k, device="cuda").to(td)
    out = torch.empty(m, n, device="cuda", dtype=td)
    ffi.check(ffi.lib().mynn_b200_debug_set_ksplit(ksplit))
    wsp = ops.dequant_matmul_workspace(m, n, k, act.device) if kernel == "tcgen05_i8" else None
    us = _time_graph([(lambda w=w: ops.dequant_matmul(act, w, sc, out=out, workspace=wsp)) for w in ws])
    ffi.lib().mynn_b200_debug_set_ksplit(0)
    esz = act.element_size()
    alg = n * k + n * esz + m * k * esz + m * n * esz
    if m > 32:  # a dense contraction: report tensor throughput (bf16-equivalent flops 2 M N K)
        peak = _peak_tflops()
        res = {"kernel": "dequant_matmul/prefill_" + kernel, "m": m, "n": n, "k": k, "dtype": dtype, "us": us,
               "TFLOPs_bf16_equivalent": 2.0 * m * n * k / us / 1e6, "frac_of_measured_bf16_peak": 2.0 * m * n * k / us / 1e6 / peak}
        if not quiet:
            print(json.dumps(res), flush=True)
        return res
    res = {"kernel": "dequant_matmul/" + kernel, "m": m, "n": n, "k": k, "dtype": dtype, "ksplit": ksplit, "us": us,
           "GBps": alg / us / 1e3, "frac_of_measured_peak": alg / us / 1e3 / _peak(), "algorithmic_bytes": alg}
    if not quiet:
        print(json.dumps(res), flush=True)
    return res


def attn(b, hq, hkv, d, length, dtype="bf16", copies=None, quiet=False, kv="16bit"):
    """Decode attention; kv="int8" times the kernel for the int8 cache (bytes: int8 rows + one scale per row)."""
    td = _DT[dtype]
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
        us = _time_graph([(lambda k=k, v=v, s=s: ops.attention_q8(q, k, v, s, s, 1 / np.sqrt(d), length, out=out, workspace=ws))
                          for k, v, s in zip(ks, vs, sc)])
    else:
        ks = [torch.randn(b, hkv, length, d, device="cuda").to(td) for _ in range(copies)]
        vs = [torch.randn(b, hkv, length, d, device="cuda").to(td) for _ in range(copies)]
        us = _time_graph([(lambda k=k, v=v: ops.attention(q, k, v, 1 / np.sqrt(d), length, out=out, workspace=ws))
                          for k, v in zip(ks, vs)])
    alg = kv_bytes + 2 * q.numel() * 2
    res = {"kernel": "attention_decode_q8" if q8 else "attention_decode", "b": b, "hq": hq, "hkv": hkv, "d": d, "len": length, "dtype": dtype, "us": us,
           "GBps": alg / us / 1e3, "frac_of_measured_peak": alg / us / 1e3 / _peak(), "algorithmic_bytes": alg}
    if not quiet:
        print(json.dumps(res), flush=True)
    return res


def prefill_attn(b, hq, hkv, d, length, dtype="bf16", quiet=False):
    """Causal self-attention of a whole prompt (Sq = kv length): 4 * Sq^2 / 2 * D * Hq * B flops."""
    td = _DT[dtype]
    q = torch.randn(b, hq, length, d, device="cuda").to(td)
    ks = [torch.randn(b, hkv, length, d, device="cuda").to(td) for _ in range(2)]
    vs = [torch.randn(b, hkv, length, d, device="cuda").to(td) for _ in range(2)]
    out = torch.empty_like(q)
    us = _time_graph([(lambda k=k, v=v: ops.attention(q, k, v, 1 / np.sqrt(d), length, True, out=out)) for k, v in zip(ks, vs)])
    flops = 4.0 * length * (length + 1) / 2 * d * hq * b
    res = {"kernel": "attention_prefill", "b": b, "hq": hq, "hkv": hkv, "d": d, "len": length, "dtype": dtype, "us": us,
           "TFLOPs": flops / us / 1e6, "frac_of_measured_bf16_peak": flops / us / 1e6 / _peak_tflops()}
    if not quiet:
        print(json.dumps(res), flush=True)
    return res


LLAMA3_8B = dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                 intermediate_size=14336, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)
TINYLLAMA = dict(hidden_size=2048, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                 intermediate_size=5632, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)


def prefill_model(arch="llama3-8b", batch=1, length=2048, chunk=None, layers=None, dtype="bf16", reps=3, quiet=False, kv_int8=False):
    """Whole-model prefill of ``length`` prompt tokens per sequence (random int8 weights of the named architecture) in
    chunks of ``chunk`` tokens: the prefill DequantMatMul and the prefill attention kernels in context.  Wall-clock per
    prompt, host call to host result (the last token's id)."""
    import time

    from .decoder import DecoderModel
    from .quantize import random_llama_state
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
    res = {"kernel": "model_prefill", "arch": arch, "layers": cfg["num_hidden_layers"], "batch": batch, "len": length, "chunk": chunk,
           "dtype": dtype, "kv_cache": "int8" if kv_int8 else dtype, "ms": best * 1e3, "first_call_ms": times[0] * 1e3, "prompt_tok_per_s": batch * length / best}
    model.close()
    if not quiet:
        print(json.dumps(res), flush=True)
    return res


def w8a8(m, n, k, dtype="bf16", copies=None, quiet=False):
    """QuantizedMatMul (int8 x int8) on the tcgen05 kernel; TFLOP/s counts 2 M N K integer operations."""
    td = _DT[dtype]
    copies = copies or max(3, int(300e6 // (n * k)) + 1)
    ws = [torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8) for _ in range(copies)]
    lhs = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    ls = (torch.rand(m, device="cuda") * 0.05 + 0.005).to(td)
    rs = (torch.rand(n, device="cuda") * 0.018 + 0.002).to(td)
    out = torch.empty(m, n, device="cuda", dtype=td)
    wsp = ops.dequant_matmul_workspace(1, n, k, "cuda")
    us = _time_graph([(lambda w=w: ops.quantized_matmul(lhs, ls, w, rs, out=out, workspace=wsp)) for w in ws])
    ops.check_workspace(wsp)
    alg = n * k + m * k + 2 * (m + n) + 2 * m * n
    res = {"kernel": "quantized_matmul/tcgen05_i8", "m": m, "n": n, "k": k, "dtype": dtype, "us": us, "TOPs": 2.0 * m * n * k / us / 1e6,
           "frac_of_measured_bf16_peak": 2.0 * m * n * k / us / 1e6 / _peak_tflops(), "GBps": alg / us / 1e3,
           "frac_of_measured_hbm_peak": alg / us / 1e3 / _peak(), "algorithmic_bytes": alg}
    if not quiet:
        print(json.dumps(res), flush=True)
    return res


def suite():
    """The shapes of the benchmark configurations: Llama-3-8B and TinyLlama projections at batch 1 and 32, the
    config-1 GEMV, and the decode-attention microbenchmark."""
    for m in (1, 32):
        for n, k in [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096)]:
            gemm(m, n, k)
    for n, k in [(5632, 2048), (2560, 2048), (2048, 2048), (11264, 2048), (2048, 5632), (32000, 2048)]:
        gemm(1, n, k)
    attn(16, 32, 8, 128, 4096)
    attn(32, 32, 8, 128, 2048)
    attn(1, 32, 4, 64, 256)


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=32)
    g.add_argument("--n", type=int, default=28672)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--dtype", default="bf16")
    g.add_argument("--ksplit", type=int, default=0)
    g.add_argument("--copies", type=int, default=None)
    g.add_argument("--kernel", default="tcgen05_i8", choices=["tcgen05_i8", "mma_sync"])
    a = sub.add_parser("attn")
    a.add_argument("--b", type=int, default=16)
    a.add_argument("--hq", type=int, default=32)
    a.add_argument("--hkv", type=int, default=8)
    a.add_argument("--d", type=int, default=128)
    a.add_argument("--len", type=int, default=4096)
    a.add_argument("--dtype", default="bf16")
    a.add_argument("--copies", type=int, default=None)
    a.add_argument("--kv", default="16bit", choices=["16bit", "int8"])
    pa = sub.add_parser("prefill_attn")
    pa.add_argument("--b", type=int, default=1)
    pa.add_argument("--hq", type=int, default=32)
    pa.add_argument("--hkv", type=int, default=8)
    pa.add_argument("--d", type=int, default=128)
    pa.add_argument("--len", type=int, default=2048)
    pa.add_argument("--dtype", default="bf16")
    pm = sub.add_parser("prefill_model")
    pm.add_argument("--arch", default="llama3-8b", choices=["llama3-8b", "tinyllama"])
    pm.add_argument("--b", type=int, default=1)
    pm.add_argument("--len", type=int, default=2048)
    pm.add_argument("--chunk", type=int, default=None)
    pm.add_argument("--layers", type=int, default=None)
    pm.add_argument("--dtype", default="bf16")
    pm.add_argument("--kv", default="16bit", choices=["16bit", "int8"])
    q = sub.add_parser("w8a8")
    q.add_argument("--m", type=int, default=2048)
    q.add_argument("--n", type=int, default=14336)
    q.add_argument("--k", type=int, default=4096)
    q.add_argument("--dtype", default="bf16")
    q.add_argument("--copies", type=int, default=None)
    sub.add_parser("suite")
    args = ap.parse_args()
    if args.cmd == "gemm":
        gemm(args.m, args.n, args.k, args.dtype, args.ksplit, args.copies, kernel=args.kernel)
    elif args.cmd == "prefill_attn":
        prefill_attn(args.b, args.hq, args.hkv, args.d, args.len, args.dtype)
    elif args.cmd == "prefill_model":
        prefill_model(args.arch, args.b, args.len, args.chunk, args.layers, args.dtype, kv_int8=args.kv == "int8")
    elif args.cmd == "w8a8":
        w8a8(args.m, args.n, args.k, args.dtype, args.copies)
    elif args.cmd == "attn":
        attn(args.b, args.hq, args.hkv, args.d, args.len, args.dtype, args.copies, kv=args.kv)
    else:
        suite()


if __name__ == "__main__":
    main()

"""Per-kernel timing of the library's CUDA kernels on synthetic inputs.

    python -m sam_quantization_b200.kernel_bench gemm  --M 32768 --N 5120 --K 1280 --gelu
    python -m sam_quantization_b200.kernel_bench quant --M 65536 --K 1280 [--ln] [--gather] [--hadamard full]
    python -m sam_quantization_b200.kernel_bench attn  --windows 200 --H 14 --W 14 --heads 16 --head-dim 80
    python -m sam_quantization_b200.kernel_bench attn-global --images 8 --H 64 --heads 16 --head-dim 80
    python -m sam_quantization_b200.kernel_bench attn-window14 --windows 200 --heads 16 --head-dim 80
    python -m sam_quantization_b200.kernel_bench sweep            # the W8A8 GEMM sweep: M x (K, N) x granularity
    python -m sam_quantization_b200.kernel_bench library --M 32768 --N 5120 --K 1280   # cuBLASLt int8 / fp16 bars

Each line of output is JSON: the shape, the mean CUDA-event time over ``--iters`` launches after
``--warmup`` launches, and the achieved rate against the roofline that bounds the kernel
(int8 TOP/s for the GEMM: 2*M*N*K per launch; GB/s for the quantization kernels: the
algorithmic M*(in_bytes*K + K + 4) per launch).  Buffers are rotated between launches so that
inputs do not stay in L2 when the working set is small.  The same commands, with small
``--iters``, are what the ncu summaries under profiles/ were captured from.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops

SWEEP_M = (196, 4096, 32768, 262144)
SWEEP_KN = ((768, 2304), (768, 3072), (3072, 768), (1024, 4096), (4096, 1024), (1280, 3840), (1280, 5120), (5120, 1280))


def _time(fn, iters, warmup, head_start_ms=20.0):
    """Mean CUDA-event time of ``fn`` over ``iters`` back-to-back launches.  The loop is enqueued behind a spin
    kernel of ``head_start_ms`` so that the host (tens of microseconds of Python per call) stays ahead of the
    GPU: otherwise a kernel shorter than the host's per-call cost would be timed at the host's pace."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if head_start_ms > 0:
        khz = getattr(torch.cuda.get_device_properties(torch.cuda.current_device()), "clock_rate", 1_900_000)
        torch.cuda._sleep(int(head_start_ms * khz))
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def synthetic_activation(M, K, dtype, device, seed=5):
    """~N(0,1) with 1 % of the channels scaled x20 (the outlier channels of the W8A8 configs)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    idx = torch.randperm(K, generator=g)[:max(1, K // 100)].to(device)
    x = torch.randn((M, K), device=device, dtype=torch.float32)
    x[:, idx] *= 20
    return x.to(dtype)


def bench_gemm(M, N, K, gelu=False, residual=False, w_gran="per_channel", out_dtype=torch.float16, iters=50, warmup=10,
               group_size=128, nbuf=None):
    dev = torch.device("cuda")
    w = (torch.randn((N, K), device=dev) * 0.02).half()
    wq = ops.quantize_weight(w, ops.WEIGHT_GRANULARITY[w_gran], group_size if w_gran == "per_group" else None)
    # enough distinct A / C buffers that consecutive launches do not find their operands in the 126 MB L2
    per = M * K + M * N * 2
    nbuf = nbuf or max(1, min(8, (256 << 20) // max(per, 1) + 1))
    acts = [ops.quantize(synthetic_activation(M, K, torch.float16, dev, seed=5 + i), ops.GRAN_ROW) for i in range(nbuf)]
    outs = [torch.empty((M, N), dtype=out_dtype, device=dev) for _ in range(nbuf)]
    bias = (torch.randn(N, device=dev) * 0.01).half()
    res = torch.randn((M, N), device=dev, dtype=out_dtype) if residual else None

    def run(i):
        a = acts[i % nbuf]
        ops.gemm_i8(a["q"], wq["q"], a["scale"], wq["scale"], ops.GRAN_ROW, ops.WEIGHT_GRANULARITY[w_gran],
                    group_size if w_gran == "per_group" else 0, bias=bias, residual=res,
                    activation=ops.ACT_GELU if gelu else ops.ACT_NONE, out_dtype=out_dtype, out=outs[i % nbuf])

    ms = _time(run, iters, warmup)
    ops.check_status()
    return {"kernel": "gemm_i8", "M": M, "N": N, "K": K, "w_gran": w_gran, "gelu": gelu, "residual": residual,
            "ms": round(ms, 5), "int8_tops": round(2.0 * M * N * K / ms / 1e9, 1), "buffers": nbuf}


def bench_library(M, N, K, iters=50, warmup=10, nbuf=None):
    """Comparison bars on the same shape, never on the product path: the vendor library's int8
    GEMM with int32 accumulation (``torch._int_mm`` -> cuBLASLt CUBLAS_COMPUTE_32I, the call
    quant/qgemm/kernels/matmul_int8.cu:81-137 demonstrates; raw int32 out, no epilogue) and the
    fp16 ``F.linear`` the reference's model path runs (RTN_quantization/per_tensor_channel_group.py:159)."""
    dev = torch.device("cuda")
    per = M * K + M * N * 4
    nbuf = nbuf or max(1, min(8, (256 << 20) // max(per, 1) + 1))
    out = {"kernel": "library", "M": M, "N": N, "K": K}
    w8 = torch.randint(-127, 128, (N, K), device=dev, dtype=torch.int8)
    if M > 16 and K % 8 == 0 and N % 8 == 0:
        a8 = [torch.randint(-127, 128, (M, K), device=dev, dtype=torch.int8) for _ in range(nbuf)]
        try:
            ms = _time(lambda i: torch._int_mm(a8[i % nbuf], w8.t()), iters, warmup)
            out["int_mm_ms"], out["int_mm_tops"] = round(ms, 5), round(2.0 * M * N * K / ms / 1e9, 1)
        except RuntimeError as e:                                  # shape not supported by the library call
            out["int_mm_error"] = str(e).splitlines()[0][:120]
        del a8
    w16 = (torch.randn((N, K), device=dev) * 0.02).half()
    b16 = (torch.randn(N, device=dev) * 0.01).half()
    a16 = [torch.randn((M, K), device=dev, dtype=torch.float16) for _ in range(nbuf)]
    ms = _time(lambda i: torch.nn.functional.linear(a16[i % nbuf], w16, b16), iters, warmup)
    out["f16_linear_ms"], out["f16_linear_tflops"] = round(ms, 5), round(2.0 * M * N * K / ms / 1e9, 1)
    return out


def library_int8_peak(seconds=1.5):
    """Measured dense int8 tensor bar of this GPU through the vendor library: ``torch._int_mm`` on
    8192^3, best single launch of ten (burst) and the mean over ``seconds`` of back-to-back launches
    (sustained, under the power cap).  Returns (burst TOP/s, sustained TOP/s)."""
    dev = torch.device("cuda")
    n = 8192
    a = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
    b = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8).t()
    for _ in range(3):
        torch._int_mm(a, b)
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    reps = max(10, int(seconds * 1000.0 / best))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        torch._int_mm(a, b)
    e1.record()
    torch.cuda.synchronize()
    ops_per = 2.0 * n ** 3
    return ops_per / best / 1e9, ops_per * reps / e0.elapsed_time(e1) / 1e9


def bench_quant(M, K, dtype=torch.float16, ln=False, gather=False, hadamard=None, granularity="per_token", group_size=128,
                iters=50, warmup=10):
    dev = torch.device("cuda")
    esz = torch.empty((), dtype=dtype).element_size()
    nbuf = max(1, min(8, (256 << 20) // (M * K * esz) + 1))
    xs = [synthetic_activation(M, K, dtype, dev, seed=9 + i) for i in range(nbuf)]
    kw = {}
    if ln:
        kw["layer_norm"] = (torch.ones(K, device=dev, dtype=dtype), torch.zeros(K, device=dev, dtype=dtype), 1e-6)
    if gather:
        kw["row_map"] = torch.randperm(M, device=dev).to(torch.int32)
    if hadamard:
        from .quarot.hadamard_utils import get_hadK
        heads = 12 if K % 768 == 0 and hadamard == "partial" else 16
        hadk, had_k = get_hadK(heads if hadamard == "partial" else K)
        kw["hadamard"] = ops.Hadamard(hadamard, had_k=had_k, hadk=None if hadk is None else hadk.to(dev),
                                      had_dim=K // heads if hadamard == "partial" else 0)
    gran = ops.ACT_GRANULARITY[granularity]

    def run(i):
        ops.quantize(xs[i % nbuf], gran, group_size if granularity == "per_group_token" else None, **kw)

    ms = _time(run, iters, warmup)
    nbytes = M * (esz * K + K + 4)
    return {"kernel": "act_quant", "M": M, "K": K, "dtype": str(dtype).split(".")[-1], "ln": ln, "gather": gather,
            "hadamard": hadamard, "granularity": granularity, "ms": round(ms, 5), "gbs": round(nbytes / ms / 1e6, 1)}


def bench_window_attention(windows, H, W, heads, head_dim, dtype=torch.bfloat16, iters=50, warmup=10):
    dev = torch.device("cuda")
    L, C = H * W, heads * head_dim
    qkv = [torch.randn((windows * L, 3 * C), device=dev, dtype=dtype) for _ in range(2)]
    rh = (torch.randn((2 * H - 1, head_dim), device=dev) * 0.02).to(dtype)
    rw = (torch.randn((2 * W - 1, head_dim), device=dev) * 0.02).to(dtype)

    def run(i):
        ops.attn_windowed(qkv[i % 2], windows, H, W, heads, rh, rw, head_dim ** -0.5)

    ms = _time(run, iters, warmup)
    nbytes = windows * L * 4 * C * qkv[0].element_size()
    flops = 4.0 * windows * heads * L * L * head_dim
    return {"kernel": "attn_window", "windows": windows, "H": H, "W": W, "heads": heads, "head_dim": head_dim,
            "ms": round(ms, 5), "gbs": round(nbytes / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 1)}


def bench_window14(windows, heads, head_dim, dtype=torch.bfloat16, iters=50, warmup=10):
    """samq_attn_window14 on [windows*196, 3C]; GB/s over the algorithmic bytes (q, k, v read, out written)."""
    dev = torch.device("cuda")
    C = heads * head_dim
    nbuf = 3
    qkv = [torch.randn((windows * 196, 3 * C), device=dev, dtype=dtype) for _ in range(nbuf)]
    rh = (torch.randn((27, head_dim), device=dev) * 0.02).to(dtype)
    rw = (torch.randn((27, head_dim), device=dev) * 0.02).to(dtype)
    table = ops.rel_pos_table(rh, rw, dtype, dev)

    def run(i):
        ops.attn_window14(qkv[i % nbuf], windows, heads, rh, rw, head_dim ** -0.5, table=table)

    ms = _time(run, iters, warmup)
    ops.check_status()
    nbytes = windows * 196 * 4 * C * qkv[0].element_size()
    flops = 4.0 * windows * heads * 196 * 196 * head_dim
    return {"kernel": "attn_window14", "windows": windows, "heads": heads, "head_dim": head_dim, "ms": round(ms, 5),
            "gbs": round(nbytes / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 1)}


def bench_global_attention(images, H, heads, head_dim, dtype=torch.bfloat16, iters=20, warmup=5, W=64):
    dev = torch.device("cuda")
    L, C = H * W, heads * head_dim
    qkv = [torch.randn((images * L, 3 * C), device=dev, dtype=dtype) for _ in range(2)]
    rh = (torch.randn((2 * H - 1, head_dim), device=dev) * 0.02).to(dtype)
    rw = (torch.randn((2 * W - 1, head_dim), device=dev) * 0.02).to(dtype)
    table = ops.rel_pos_table(rh, rw, dtype, dev)

    def run(i):
        ops.attn_global(qkv[i % 2], images, H, W, heads, rh, rw, head_dim ** -0.5, table=table)

    ms = _time(run, iters, warmup)
    ops.check_status()
    flops = 4.0 * images * heads * L * L * head_dim
    return {"kernel": "attn_global (+ rel products)", "images": images, "H": H, "W": W, "heads": heads,
            "head_dim": head_dim, "ms": round(ms, 5), "tflops": round(flops / ms / 1e9, 1)}


def _measured_int8_peak():
    """(dense int8 TOP/s used as the denominator, where it came from): twice the measured dense
    bf16 burst rate when the pool's peak file is next to the package, else twice 1590."""
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return 2.0 * float(json.load(f)["bf16_tflops"]), "2 x measured bf16 burst"
    return 2.0 * 1590.0, "2 x 1590 (fallback)"


def run_sweep(args):
    """The W8A8 GEMM sweep: every (K, N) x M x weight granularity, int8 TOP/s and fraction of the
    dense int8 peak, next to the vendor library's int8 GEMM and fp16 linear on the same shape."""
    peak, peak_src = (args.peak, "given") if args.peak else _measured_int8_peak()
    grans = args.granularities.split(",")
    rows = {}
    lib_rows = {}
    for K, N in SWEEP_KN:
        for M in SWEEP_M:
            it = args.iters if M <= 32768 else max(10, args.iters // 5)
            for gran in grans:
                r = bench_gemm(M, N, K, w_gran=gran, iters=it, warmup=args.warmup)
                r["frac_of_peak"] = round(r["int8_tops"] / peak, 3)
                rows[(K, N, M, gran)] = r
                print(json.dumps(r), flush=True)
            if not args.no_library:
                r = bench_library(M, N, K, iters=it, warmup=args.warmup)
                lib_rows[(K, N, M)] = r
                print(json.dumps(r), flush=True)
    if args.markdown:
        lines = [f"Dense int8 peak used for the fraction: {peak:.0f} TOP/s ({peak_src}).  Each cell: M = "
                 + " / ".join(str(m) for m in SWEEP_M) + " tokens.", ""]
        head = "| K -> N | " + " | ".join(f"{g} TOP/s | {g} frac" for g in grans)
        if lib_rows:
            head += " | cuBLASLt int8 (int32 out) TOP/s | fp16 F.linear TFLOP/s"
        lines += [head + " |", "|" + "---|" * (head.count("|"))]
        for K, N in SWEEP_KN:
            cells = [f"{K} -> {N}"]
            for g in grans:
                cells.append(" / ".join(f"{rows[(K, N, M, g)]['int8_tops']:.0f}" for M in SWEEP_M))
                cells.append(" / ".join(f"{rows[(K, N, M, g)]['frac_of_peak']:.2f}" for M in SWEEP_M))
            if lib_rows:
                cells.append(" / ".join(f"{lib_rows[(K, N, M)].get('int_mm_tops', float('nan')):.0f}" for M in SWEEP_M))
                cells.append(" / ".join(f"{lib_rows[(K, N, M)]['f16_linear_tflops']:.0f}" for M in SWEEP_M))
            lines.append("| " + " | ".join(cells) + " |")
        with open(args.markdown, "w") as f:
            f.write("\n".join(lines) + "\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pair-mode", dest="pair_mode", type=int, default=None, choices=[0, 1, 2],
                    help="K2 implementation: 0 single CTAs, 1 by size, 2 CTA pairs (default: the library's)")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--M", type=int, default=32768)
    g.add_argument("--N", type=int, default=5120)
    g.add_argument("--K", type=int, default=1280)
    g.add_argument("--gelu", action="store_true")
    g.add_argument("--residual", action="store_true")
    g.add_argument("--w-gran", dest="w_gran", default="per_channel", choices=list(ops.WEIGHT_GRANULARITY))
    g.add_argument("--iters", type=int, default=50)
    g.add_argument("--warmup", type=int, default=10)
    q = sub.add_parser("quant")
    q.add_argument("--M", type=int, default=65536)
    q.add_argument("--K", type=int, default=1280)
    q.add_argument("--dtype", default="float16", choices=["float16", "bfloat16", "float32"])
    q.add_argument("--ln", action="store_true")
    q.add_argument("--gather", action="store_true")
    q.add_argument("--hadamard", default=None, choices=["full", "partial"])
    q.add_argument("--granularity", default="per_token", choices=list(ops.ACT_GRANULARITY))
    q.add_argument("--iters", type=int, default=50)
    q.add_argument("--warmup", type=int, default=10)
    a = sub.add_parser("attn")
    a.add_argument("--windows", type=int, default=200)
    a.add_argument("--H", type=int, default=14)
    a.add_argument("--W", type=int, default=14)
    a.add_argument("--heads", type=int, default=16)
    a.add_argument("--head-dim", dest="head_dim", type=int, default=80)
    a.add_argument("--iters", type=int, default=50)
    a.add_argument("--warmup", type=int, default=10)
    aw = sub.add_parser("attn-window14")
    aw.add_argument("--windows", type=int, default=200)
    aw.add_argument("--heads", type=int, default=16)
    aw.add_argument("--head-dim", dest="head_dim", type=int, default=80)
    aw.add_argument("--iters", type=int, default=50)
    aw.add_argument("--warmup", type=int, default=10)
    ag = sub.add_parser("attn-global")
    ag.add_argument("--images", type=int, default=8)
    ag.add_argument("--H", type=int, default=64)
    ag.add_argument("--W", type=int, default=64, help="64 for whole images; up to 16 (with H <= 16) for windows, --images is then the window count")
    ag.add_argument("--heads", type=int, default=16)
    ag.add_argument("--head-dim", dest="head_dim", type=int, default=80)
    ag.add_argument("--iters", type=int, default=20)
    ag.add_argument("--warmup", type=int, default=5)
    s = sub.add_parser("sweep")
    s.add_argument("--iters", type=int, default=100)
    s.add_argument("--warmup", type=int, default=20)
    s.add_argument("--granularities", default="per_tensor,per_channel,per_group")
    s.add_argument("--no-library", dest="no_library", action="store_true", help="skip the cuBLASLt int8 / fp16 comparison bars")
    s.add_argument("--peak", type=float, default=None, help="dense int8 TOP/s the fraction column divides by (default: "
                   "twice the measured bf16 burst figure of MEASURED_PEAKS.json, else 2 x 1590)")
    s.add_argument("--markdown", default=None, help="also write the sweep as a markdown table to this path")
    lb = sub.add_parser("library")
    lb.add_argument("--M", type=int, default=32768)
    lb.add_argument("--N", type=int, default=5120)
    lb.add_argument("--K", type=int, default=1280)
    lb.add_argument("--iters", type=int, default=50)
    lb.add_argument("--warmup", type=int, default=10)
    args = ap.parse_args()
    if args.pair_mode is not None:
        ops.set_gemm_pair_mode(args.pair_mode)
    if args.cmd == "gemm":
        print(json.dumps(bench_gemm(args.M, args.N, args.K, args.gelu, args.residual, args.w_gran, iters=args.iters, warmup=args.warmup)))
    elif args.cmd == "attn":
        print(json.dumps(bench_window_attention(args.windows, args.H, args.W, args.heads, args.head_dim, iters=args.iters, warmup=args.warmup)))
    elif args.cmd == "attn-window14":
        print(json.dumps(bench_window14(args.windows, args.heads, args.head_dim, iters=args.iters, warmup=args.warmup)))
    elif args.cmd == "attn-global":
        print(json.dumps(bench_global_attention(args.images, args.H, args.heads, args.head_dim, iters=args.iters, warmup=args.warmup, W=args.W)))
    elif args.cmd == "quant":
        print(json.dumps(bench_quant(args.M, args.K, getattr(torch, args.dtype), args.ln, args.gather, args.hadamard,
                                     args.granularity, iters=args.iters, warmup=args.warmup)))
    elif args.cmd == "library":
        print(json.dumps(bench_library(args.M, args.N, args.K, iters=args.iters, warmup=args.warmup)))
    else:
        run_sweep(args)


if __name__ == "__main__":
    main()

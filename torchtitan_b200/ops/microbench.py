"""Kernel micro-benchmarks: ``python -m torchtitan_b200.ops.microbench <kernel> [--case small|8b]``.

Times one hand-written kernel against the library operator that the reference would call
for the same shape (cuBLAS ``torch.mm``, ATen ``rms_norm``...), with CUDA events on the
launching stream, three warm-up launches, and a write larger than the L2 between timed
launches.  Prints one line per shape with achieved TFLOP/s or GB/s.  ``--once`` runs each
shape a single time without the library arm, which is the form to put under a profiler.
"""

from __future__ import annotations

import argparse
import sys

import torch

T = 8192  # tokens per step in the Llama-3 8B headline configuration

# (name, mode, M, N, K) : mode 0 = NT (forward), 1 = NN (input gradient), 2 = TN (weight gradient)
GEMM_8B = [
    ("qkv fwd", 0, T, 6144, 4096), ("wo fwd", 0, T, 4096, 4096), ("w13 fwd", 0, T, 28672, 4096),
    ("w2 fwd", 0, T, 4096, 14336), ("w13 dgrad", 1, T, 4096, 28672), ("w2 dgrad", 1, T, 14336, 4096),
    ("qkv dgrad", 1, T, 4096, 6144), ("w13 wgrad", 2, 28672, 4096, T), ("w2 wgrad", 2, 4096, 14336, T),
    ("qkv wgrad", 2, 6144, 4096, T), ("wo wgrad", 2, 4096, 4096, T), ("lmhead fwd", 0, 1024, 128256, 4096),
    ("lmhead dgrad", 1, 1024, 4096, 128256), ("lmhead wgrad+", 2, 128256, 4096, 1024), ("square", 0, 8192, 8192, 8192),
]
GEMM_SMALL = [("square", 0, 8192, 8192, 8192)]


class Timer:
    def __init__(self):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn, n: int = 10) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]


def bench_gemm(args) -> None:
    ops = torch.ops.tb200
    timer = Timer()
    for name, mode, M, N, K in (GEMM_SMALL if args.case == "small" else GEMM_8B):
        a = torch.randn((K, M) if mode == 2 else (M, K), device="cuda").bfloat16()
        b = torch.randn((N, K) if mode == 0 else (K, N), device="cuda").bfloat16()
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        acc = name.endswith("+")  # accumulate into C (chunked lm_head weight gradient)
        ours = lambda: ops.gemm_bf16(a, b, c, mode, acc)  # noqa: E731
        ops.gemm_set_variant(args.variant)
        if args.once:
            ours()
            torch.cuda.synchronize()
            continue
        lib = {0: lambda: torch.mm(a, b.t(), out=c), 1: lambda: torch.mm(a, b, out=c),
               2: (lambda: c.addmm_(a.t(), b)) if acc else (lambda: torch.mm(a.t(), b, out=c))}[mode]
        t1, t2 = timer(ours), timer(lib)
        fl = 2 * M * N * K
        extra = ""
        if args.mn_boxes and mode != 0:
            # the same MN-major operands through one 2-D load per 64-column box instead of one 3-D load per stage
            ops.gemm_set_mn3d(0)
            t0 = timer(ours)
            ops.gemm_set_mn3d(1)
            extra = f" | 2-D boxes {t0:.3f} ms {fl / t0 / 1e9:.0f} TFLOPS"
        print(f"gemm {name:10s} mode{mode} M{M} N{N} K{K}: tcgen05 {t1:.3f} ms {fl / t1 / 1e9:.0f} TFLOPS | "
              f"cuBLAS {t2:.3f} ms {fl / t2 / 1e9:.0f} TFLOPS | speedup {t2 / t1:.2f}{extra}", flush=True)
    print("gemm status word", ops.gemm_status(True))


def bench_attention(args) -> None:
    import math

    import torch.nn.functional as F

    ops = torch.ops.tb200
    timer = Timer()
    cases = [(8192, 32, 8, 128)] if args.case != "small" else [(4096, 32, 8, 128)]
    for Tn, H, Hkv, D in cases:
        qkv = torch.randn(Tn, (H + 2 * Hkv) * D, device="cuda").bfloat16()
        v3 = qkv.view(Tn, H + 2 * Hkv, D)
        q, k, v = v3[:, :H], v3[:, H:H + Hkv], v3[:, H + Hkv:]
        do = torch.randn(Tn, H, D, device="cuda").bfloat16()
        scale = 1.0 / math.sqrt(D)
        fl_f = 4 * Tn * Tn * H * D / 2
        has_bwd = hasattr(ops, "flash_bwd")
        if args.once:
            o, lse = ops.flash_fwd(q, k, v, scale, True, 0, None)
            if has_bwd:
                ops.flash_bwd(do, q, k, v, o, lse, scale, True, 0, None, None, None, None)
            torch.cuda.synchronize()
            continue
        for variant in (1, 2, 3, 4, 0):   # every forward kernel; the last one (the default) stays selected
            ops.flash_set_fwd_variant(variant)
            tf = timer(lambda: ops.flash_fwd(q, k, v, scale, True, 0, None))
            print(f"attention tcgen05 T{Tn} H{H}/{Hkv} D{D} forward kernel {variant}: {tf:.3f} ms {fl_f / tf / 1e9:.0f} TFLOPS",
                  flush=True)
        line = f"attention tcgen05 T{Tn} H{H}/{Hkv} D{D}: fwd {tf:.3f} ms {fl_f / tf / 1e9:.0f} TFLOPS"
        if has_bwd:
            o, lse = ops.flash_fwd(q, k, v, scale, True, 0, None)
            tb = timer(lambda: ops.flash_bwd(do, q, k, v, o, lse, scale, True, 0, None, None, None, None))
            line += f" | bwd {tb:.3f} ms {2.5 * fl_f / tb / 1e9:.0f} TFLOPS"
        print(line, flush=True)
        # library arm: cuDNN / flash SDPA on [1, H, T, D]
        from torch.nn.attention import SDPBackend, sdpa_kernel

        qh, kh, vh = (t.transpose(0, 1).unsqueeze(0).detach().requires_grad_() for t in (q, k, v))
        with sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION], set_priority=True):
            fwd = lambda: F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=scale, enable_gqa=True)  # noqa: E731
            tf = timer(lambda: fwd())
            out = fwd()
            doh = do.transpose(0, 1).unsqueeze(0)
            tb = timer(lambda: torch.autograd.grad(out, (qh, kh, vh), doh, retain_graph=True))
        print(f"attention sdpa    T{Tn} H{H}/{Hkv} D{D}: fwd {tf:.3f} ms {fl_f / tf / 1e9:.0f} TFLOPS | "
              f"bwd {tb:.3f} ms {2.5 * fl_f / tb / 1e9:.0f} TFLOPS", flush=True)
    print("flash status word", ops.flash_status(True))


def bench_elementwise(args) -> None:
    ops = torch.ops.tb200
    timer = Timer()
    rows, D, F_ = T, 4096, 14336
    x = torch.randn(rows, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    gu = torch.randn(rows, 2 * F_, device="cuda").bfloat16()
    dy = torch.randn(rows, F_, device="cuda").bfloat16()

    def gbs(nbytes, ms):
        return nbytes / ms / 1e6

    y, rstd = ops.rmsnorm_fwd(x, w, 1e-5)
    rows_ = [
        ("rmsnorm_fwd", lambda: ops.rmsnorm_fwd(x, w, 1e-5), 2 * x.numel() * 2),
        ("rmsnorm_bwd", lambda: ops.rmsnorm_bwd(x, x, w, rstd), 3 * x.numel() * 2),
        ("swiglu_fwd", lambda: ops.swiglu_fwd(gu), gu.numel() * 2 + dy.numel() * 2),
        ("swiglu_bwd", lambda: ops.swiglu_bwd(gu, dy), 2 * gu.numel() * 2 + dy.numel() * 2),
    ]
    n = 64 << 20
    master = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").bfloat16()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    lowp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    one = torch.ones(1, device="cuda")
    rows_.append(("adamw", lambda: ops.adamw_(master, g, m, v, lowp, one, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05),
                  n * (4 + 2 + 4 + 4 + 4 + 4 + 4 + 2)))
    for name, fn, nbytes in rows_:
        if args.once:
            fn()
            torch.cuda.synchronize()
            continue
        t = timer(fn)
        print(f"{name:12s}: {t:.3f} ms, {gbs(nbytes, t):.0f} GB/s algorithmic", flush=True)


def bench_gemm_mx(args) -> None:
    """MXFP8 block-scaled GEMM (tcgen05 kind::mxf8f6f4) vs the bf16 tcgen05 GEMM and cuBLAS MXFP8."""
    ops = torch.ops.tb200
    timer = Timer()
    shapes = [s for s in GEMM_8B if s[1] == 0]
    for name, _, M, N, K in (shapes if args.case != "small" else [("square", 0, 8192, 8192, 8192)]):
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = torch.randn(N, K, device="cuda").bfloat16()
        xa, xs = ops.mxfp8_quantize_tiled(x)
        wa, ws = ops.mxfp8_quantize_tiled(w)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        if args.once:
            ops.gemm_mxfp8(xa, xs, wa, ws)
            torch.cuda.synchronize()
            continue
        t_mx = timer(lambda: ops.gemm_mxfp8(xa, xs, wa, ws))
        t_bf = timer(lambda: ops.gemm_bf16(x, w, c, 0, False))
        t_q = timer(lambda: ops.mxfp8_quantize_tiled(x))
        lib = ""
        try:
            a8, b8 = xa.view(torch.float8_e4m3fn), wa.view(torch.float8_e4m3fn)
            sa, sb = xs.view(torch.float8_e8m0fnu), ws.view(torch.float8_e8m0fnu)
            f = lambda: torch._scaled_mm(a8, b8.t(), sa, sb, out_dtype=torch.bfloat16)  # noqa: E731
            ref = f()
            ok = torch.allclose(ref.float(), ops.gemm_mxfp8(xa, xs, wa, ws).float(), atol=1.0, rtol=2e-2)
            t_lib = timer(f)
            lib = f" | cuBLAS mxfp8 {t_lib:.3f} ms {2 * M * N * K / t_lib / 1e9:.0f} TFLOPS (same result: {ok})"
        except Exception as e:  # the library arm is optional
            lib = f" | cuBLAS mxfp8 unavailable ({type(e).__name__})"
        fl = 2 * M * N * K
        print(f"gemm_mx {name:10s} M{M} N{N} K{K}: mxfp8 {t_mx:.3f} ms {fl / t_mx / 1e9:.0f} TFLOPS | bf16 tcgen05 {t_bf:.3f} ms "
              f"{fl / t_bf / 1e9:.0f} | quantize x {t_q:.3f} ms{lib}", flush=True)


def bench_gemm_mx_grouped(args) -> None:
    """Grouped (expert) GEMMs: MXFP8 block-scaled kernel vs the bf16 grouped kernel, Qwen3-30B-A3B expert shapes
    (128 experts, dim 2048, hidden 768, 8192 tokens x top-8 -> 512 rows per expert, padded layout)."""
    ops = torch.ops.tb200
    timer = Timer()
    E, rows = (8, 512) if args.case == "small" else (128, 512)
    R = E * rows
    offs = torch.arange(0, R + 1, rows, dtype=torch.int32, device="cuda")
    for name, K, N in (("w1/w3", 2048, 768), ("w2", 768, 2048)):
        x = torch.randn(R, K, device="cuda").bfloat16()
        w = (torch.randn(E, N, K, device="cuda") * 0.05).bfloat16()
        y = torch.empty(R, N, device="cuda", dtype=torch.bfloat16)
        xq, xs = ops.mxfp8_quantize_tiled(x)
        wq, ws = ops.mxfp8_quantize_tiled(w.view(E * N, K))
        if args.once:
            ops.gemm_mxfp8_grouped(xq, xs, wq, ws, offs, 1)
            torch.cuda.synchronize()
            continue
        t_mx = timer(lambda: ops.gemm_mxfp8_grouped(xq, xs, wq, ws, offs, 1))
        t_bf = timer(lambda: ops.gemm_grouped_bf16(x, w, y, offs, 0, 128, False))
        t_q = timer(lambda: ops.mxfp8_quantize_tiled(x))
        fl = 2 * R * N * K
        print(f"grouped {name:6s} E{E} rows/expert {rows} K{K} N{N}: mxfp8 {t_mx:.3f} ms {fl / t_mx / 1e9:.0f} TFLOPS | "
              f"bf16 {t_bf:.3f} ms {fl / t_bf / 1e9:.0f} | quantize x {t_q:.3f} ms", flush=True)


def bench_tp(args) -> None:
    """Fused tensor-parallel GEMMs vs NCCL collective + cuBLAS; run under torchrun with >= 2 ranks:
    ``python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m torchtitan_b200.ops.microbench tp``."""
    import os

    import torch.distributed as dist

    from torchtitan_b200.parallel.tp_fused import FusedTP

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    ftp = FusedTP(dist.group.WORLD, dev, nbytes=3 << 30)
    timer = Timer()
    Tn = T
    S = Tn // world
    shapes = [("wqkv  ag->gemm", "ag", 4096, 6144 // world), ("w13   ag->gemm", "ag", 4096, 28672 // world),
              ("wo    gemm->rs", "rs", 4096 // world, 4096), ("w2    gemm->rs", "rs", 14336 // world, 4096)]
    for name, kind, K, N in shapes:
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        if kind == "ag":
            x = torch.randn(S, K, device=dev).bfloat16()
            full = torch.empty(Tn, K, device=dev, dtype=torch.bfloat16)
            out = torch.empty(Tn, N, device=dev, dtype=torch.bfloat16)
            fused = lambda: ftp.ag_gemm(x, w, 0)  # noqa: E731

            def lib():
                dist.all_gather_into_tensor(full, x)
                torch.mm(full, w.t(), out=out)
            nv_bytes = (world - 1) * S * K * 2
        else:
            x = torch.randn(Tn, K, device=dev).bfloat16()
            part = torch.empty(Tn, N, device=dev, dtype=torch.bfloat16)
            outs = torch.empty(S, N, device=dev, dtype=torch.bfloat16)
            fused = lambda: ftp.gemm_rs(x, w, 0)  # noqa: E731

            def lib():
                torch.mm(x, w.t(), out=part)
                dist.reduce_scatter_tensor(outs, part)
            nv_bytes = (world - 1) * S * N * 2
        t = torch.tensor([timer(fused), timer(lib)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        fl = 2 * Tn * N * K
        roof = max(fl / 1654.7e12, nv_bytes / 770e9) * 1e3
        if rank == 0:
            print(f"tp{world} {name} T{Tn} K{K} N{N}: fused {t[0]:.3f} ms | NCCL+cuBLAS {t[1]:.3f} ms | speedup "
                  f"{t[1] / t[0]:.2f} | roofline {roof:.3f} ms ({roof / t[0]:.2f} of it)", flush=True)
    torch.cuda.synchronize()
    st = int(ftp.arena.status.item()) | int(torch.ops.tb200.gemm_status(True))
    if rank == 0:
        print("status words", st)
    dist.barrier()
    dist.destroy_process_group()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm_mx", "gemm_mx_grouped", "attention", "elementwise", "tp"])
    ap.add_argument("--case", default="8b", choices=["small", "8b"])
    ap.add_argument("--variant", type=int, default=0, help="GEMM tiling: 0 auto, 1 single CTA, 2 CTA pair")
    ap.add_argument("--once", action="store_true", help="one launch per shape, no library arm (profiler form)")
    ap.add_argument("--mn-boxes", action="store_true",
                    help="gemm: also time MN-major operands staged with one 2-D load per 64-column box")
    args = ap.parse_args(argv)
    from . import ext

    assert torch.cuda.is_available(), "microbench needs a GPU"
    ext.require()
    {"gemm": bench_gemm, "attention": bench_attention, "elementwise": bench_elementwise, "tp": bench_tp, "gemm_mx": bench_gemm_mx, "gemm_mx_grouped": bench_gemm_mx_grouped}[args.kernel](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Small, bounded runs of single kernels and of the whole pipeline, meant to be run under a profiler.

    python -m turbopi_b200.profile_cases gemm --M 712 --N 32768 --K 2048 --pieces 3 --iters 3
    python -m turbopi_b200.profile_cases gemv_tc --iters 3
    python -m turbopi_b200.profile_cases pi05 --steps 1 --iters 2

Only the iterations between cudaProfilerStart / cudaProfilerStop are meant to be captured
(`ncu --profile-from-start off`); weight preparation and warm-up stay outside.  Each case prints its
CUDA-event time per iteration so that the same command line doubles as the plain run.
"""
import argparse

import torch

from . import _lib, ops


def _timed(fn, iters, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return a.elapsed_time(b) / iters


def case_gemm(args):
    """One model-shaped linear: activation-piece quantiser + tensor-core GEMM on the tiled images."""
    from .pi05 import TcLinear
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(args.M, args.K, device=dev, generator=g).to(torch.bfloat16)
    lin = TcLinear.from_weight(torch.randn(args.N, args.K, device=dev, generator=g) * 0.02)
    lin.ws = ops.gemm_workspace(dev)
    q = ops.QuantBuf(args.M, args.K, args.pieces, dev)
    out = torch.empty((args.M, args.N), dtype=torch.bfloat16, device=dev)

    def step():
        ops.rowop(_lib.ROW_NONE, x, args.K, q)
        lin(q, out, activation=args.activation)
    ms = _timed(step, args.iters)
    flops = 2.0 * args.M * args.N * args.K
    print(f"gemm M={args.M} N={args.N} K={args.K} pieces={args.pieces}: {ms * 1e3:.1f} us per quantise+GEMM, "
          f"{flops / (ms * 1e-3) / 1e12:.0f} TFLOP/s effective (weight-only semantics)")


def case_gemv_tc(args):
    """The bench's 54-matrix decode step on the tensor-core GEMV (2 quantiser launches + 1 GEMV launch)."""
    import bench
    dev = torch.device("cuda:0")
    x = {K: torch.randn(1, K, device=dev).to(torch.bfloat16) for K in (bench.HIDDEN, bench.INTER)}
    mats = bench.make_weight_set(100, dev)
    outs = [torch.empty((1, N), dtype=torch.bfloat16, device=dev) for (_, _, _, N, _) in mats]
    tc = ops.TcGemv([dict(x=x[K], weight_packed=p, weight_scales=sc, global_scale=gs, out=o)
                     for (p, sc, gs, N, K), o in zip(mats, outs)], pieces=3)
    ms = _timed(tc.launch, args.iters)
    print(f"gemv_tc 54 matrices: {ms * 1e3:.1f} us per step, {bench.STEP_BYTES / (ms * 1e-3) / 1e9:.0f} GB/s")


def case_pi05(args):
    """Whole Pi0.5-shaped inference (vision tower, prefix pass, `steps` denoise steps), eager launches."""
    from .pi05 import Pi05, Pi05Config
    dev = torch.device("cuda:0")
    cfg = Pi05Config()
    model = Pi05(cfg, dev, seed=0)
    gen = torch.Generator().manual_seed(1)
    images = torch.randint(0, 256, (cfg.num_images, cfg.image_size, cfg.image_size, 3), generator=gen, dtype=torch.uint8)
    tokens = torch.randint(0, cfg.vocab, (cfg.text_len,), generator=gen)
    noise = torch.randn(cfg.action_horizon, cfg.action_dim, generator=gen)
    with torch.no_grad():
        ms = _timed(lambda: model.infer(images, tokens, noise, args.steps, use_graph=False), args.iters, warm=1)
    print(f"pi05 {args.steps} denoise step(s), eager launches: {ms:.2f} ms per inference; "
          f"device_error={_lib.load().tpb200_device_error(0)}")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="case", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--M", type=int, default=712)
    g.add_argument("--N", type=int, default=32768)
    g.add_argument("--K", type=int, default=2048)
    g.add_argument("--pieces", type=int, default=3)
    g.add_argument("--activation", type=int, default=0)
    g.add_argument("--iters", type=int, default=3)
    t = sub.add_parser("gemv_tc")
    t.add_argument("--iters", type=int, default=3)
    p = sub.add_parser("pi05")
    p.add_argument("--steps", type=int, default=1)
    p.add_argument("--iters", type=int, default=2)
    args = ap.parse_args()
    _lib.load()
    {"gemm": case_gemm, "gemv_tc": case_gemv_tc, "pi05": case_pi05}[args.case](args)


if __name__ == "__main__":
    main()

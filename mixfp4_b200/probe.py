"""Single-kernel timing probe (also the command the profiler summaries were captured with).

    python -m mixfp4_b200.probe gemv     N K M [--buffers B] [--iters I]
    python -m mixfp4_b200.probe gemm     N K M [--rotate]
    python -m mixfp4_b200.probe quantize N K

Weights are seeded N(0, 0.02^2) bf16 tensors quantized on the device; the GEMV cycles over
enough distinct packed weights to exceed the L2, all timings are CUDA events after warm-up.
Prints one line per run with the algorithmic bytes / flops of that kernel.
"""

from __future__ import annotations

import argparse

import torch

import mixfp4_b200 as mx


def _time(fn, iters: int, warm: int = 3) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def _weight(n: int, k: int, seed: int) -> torch.Tensor:
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)


def gemv(n: int, k: int, m: int, buffers: int | None, iters: int) -> None:
    per = mx.packed_nbytes(n, k)
    buffers = buffers or max(2, int(600e6 // per))
    packs = [mx.quantize_packed(_weight(n, k, i))[0].to_kernel_layout() for i in range(buffers)]
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)

    def run():
        for p in packs:
            mx.mixfp4_linear(x, p, overlap_previous=True)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        run()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            run()
    t = _time(graph.replay, iters) / buffers
    algo = per + 2 * m * k + 2 * m * n
    print(f"gemv N={n} K={k} M={m}: {t * 1e6:.2f} us/launch, {algo / t / 1e9:.0f} GB/s algorithmic "
          f"({buffers} distinct weights, graph replay)")


def gemm(n: int, k: int, m: int, rotate: bool, iters: int) -> None:
    w = _weight(n, k, 0)
    if rotate:
        packed = mx.quantize_packed(mx.apply_transform(w, "H128"), rotation="H128")[0].to_kernel_layout()
    else:
        packed = mx.quantize_packed(w)[0].to_kernel_layout()
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    t = _time(lambda: mx.mixfp4_linear(x, packed), iters)
    print(f"gemm M={m} N={n} K={k}{' +H128' if rotate else ''}: {t * 1e6:.1f} us, "
          f"{2.0 * m * n * k / t / 1e12:.0f} TFLOP/s")


def quantize(n: int, k: int, iters: int) -> None:
    ws = [_weight(n, k, i) for i in range(max(2, int(400e6 // (2 * n * k))))]
    state = {"i": 0}

    def run():
        state["i"] = (state["i"] + 1) % len(ws)
        mx.quantize_packed(ws[state["i"]])

    t = _time(run, iters)
    algo = 2 * n * k + mx.packed_nbytes(n, k)
    print(f"quantize N={n} K={k}: {t * 1e6:.1f} us (amax + quantize), {algo / t / 1e9:.0f} GB/s algorithmic")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemv", "gemm", "quantize"])
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("m", type=int, nargs="?", default=1)
    ap.add_argument("--buffers", type=int, default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--rotate", action="store_true")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    if args.kernel == "gemv":
        gemv(args.n, args.k, args.m, args.buffers, args.iters)
    elif args.kernel == "gemm":
        gemm(args.n, args.k, args.m, args.rotate, args.iters)
    else:
        quantize(args.n, args.k, args.iters)


if __name__ == "__main__":
    main()

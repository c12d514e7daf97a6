"""Benchmark of the mixed-FP4 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the linear layers of a Llama-3-8B decode step at M=1 --
32 layers x (q 4096x4096, k/v 1024x4096, o 4096x4096, gate/up 14336x4096, down
4096x14336) = 224 mixed-FP4 linears over 3.98 GB of packed weights (every weight is a
distinct buffer, so the working set is ~30x the L2).  One step = one pass over all 224
linears in 128 launches: the projections that share an input (q/k/v, gate/up) go out as one
grouped launch each, as a decoder would issue them.  Weights are seeded synthetic Student-t(4) x 0.02 tensors quantized by the CUDA
quantizer; activations are seeded N(0,1) bf16.

Metric: GEMV HBM GB/s at M=1 = algorithmic bytes (packed weight 0.5703 B/element + bf16
x + bf16 y) / device time.  `value` is timed with CUDA events around K graph replays with
all inputs resident; `e2e` is the same pass driven through the public Python API from
pinned HOST activations (h2d + chained layers + d2h inside the timed region).

With --gpus N > 1 (launched by torch.distributed.run) the same model is tensor-parallel:
q/k/v/gate/up split along N, o/down along K with an NCCL all-reduce; `value` is the
whole-job rate (total algorithmic bytes of the full model / max-over-ranks time).

--impl reference times the reference's CPU path (PyTorch eager port of its quantizer +
fp32 F.linear on the dequantized weight, all host threads) on a bounded sample of the same
workload (one of the 32 layers per step).
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "mixed-FP4 linear: GEMV HBM GB/s @M=1 (Llama-3-8B decode linears)"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
# DRAM traffic of one launch of the dominant kernel from an ncu capture of the gate/up layer
# (14336 x 4096, M = 1): dram__bytes_read.sum + dram__bytes_write.sum = 33.11 MB against 33.52 MB
# algorithmic (the stream layout has no separate format array), i.e. 0.988 x the
# algorithmic bytes; scaled here to the average launch of the step (traffic grows with N*K).
TRAFFIC_OVER_ALGORITHMIC = 0.988
TRAFFIC_BYTES_PER_LAUNCH = None   # set in run_ours once the step's bytes are known
LAUNCHES_PER_LAYER = 4            # q/k/v grouped, o, gate/up grouped, down


def layer_list():
    from mixfp4_b200 import synth
    out = []
    for name, n, k, count in synth.LLAMA3_8B_LAYERS:
        for i in range(count):
            out.append((f"{name}{i}" if count > 1 else name, n, k))
    return out, synth.LLAMA3_8B_NUM_LAYERS


def algorithmic_bytes(n: int, k: int, m: int, out_bytes: int = 2) -> int:
    from mixfp4_b200.quant import packed_nbytes
    return packed_nbytes(n, k) + 2 * m * k + out_bytes * m * n


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int = 0):
        self.index = index
        self.rows: list[str] = []
        self.proc = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in self.rows:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- GPU arm
def to_layout(packed, layout: str):
    return packed.to_stream_layout() if layout == "stream" else packed.to_kernel_layout()


def build_model(device, rank: int, world: int, m: int, layout: str = "stream"):
    """Quantize the (sharded) synthetic 8B linear stack on the device.  Returns a list of
    layers, each a dict name -> (PackedWeight, kind)."""
    import mixfp4_b200 as mx
    layers, nlayers = layer_list()
    gen = torch.Generator(device=device)
    model = []
    for li in range(nlayers):
        entry = {}
        for idx, (name, n, k) in enumerate(layers):
            gen.manual_seed(1000 * li + idx)
            # Student-t(4) = z / sqrt(chi2_4 / 4), drawn on the device (7e9 elements in total)
            z = torch.randn((n, k), generator=gen, device=device)
            chi = torch.zeros((n, k), device=device)
            for _ in range(4):
                d = torch.randn((n, k), generator=gen, device=device)
                chi.addcmul_(d, d)
            w = (z / torch.sqrt(chi / 4) * 0.02).to(torch.bfloat16)
            del z, chi
            row_parallel = name in ("o", "down")
            amax = mx.tensor_amax(w)
            full = w
            if world > 1:
                if row_parallel:       # split K
                    step = k // world
                    w = w[:, rank * step:(rank + 1) * step].contiguous()
                else:                  # split N
                    step = n // world
                    w = w[rank * step:(rank + 1) * step].contiguous()
            if li == 0 and name in ("o", "down"):
                # the unsharded weight of layer 0, dequantized by the (bit-exact) dequant kernel: the
                # reference of the correctness check printed with the result
                entry["full_" + name] = mx.dequantize(mx.quantize_packed(full, amax=amax)[0]) if world > 1 else None
            packed, _, _ = mx.quantize_packed(w, amax=amax)
            entry[name] = to_layout(packed, layout)
            if li == 0 and name in ("o", "down") and world == 1:
                entry["full_" + name] = mx.dequantize(packed)
            del w
        model.append(entry)
    torch.cuda.synchronize(device)
    return model


def decode_pass(model, h, world: int, out_dtype=torch.bfloat16, comm=None):
    """One token through all linears, chained the way a decoder layer chains them
    (attention, norms and activation functions are not part of this path and are skipped)."""
    import torch.distributed as dist
    import mixfp4_b200 as mx
    x, out = h, None
    lin = lambda t, p: mx.mixfp4_linear(t, p, overlap_previous=True)   # weights are never written here
    grp = lambda t, ps: mx.mixfp4_linear_grouped(t, ps, overlap_previous=True)
    for layer in model:
        # every layer starts from the same input so that 32 chained layers of random weights
        # stay finite; inside a layer the seven linears keep their data dependencies; the
        # projections that share an input (q/k/v, gate/up) go out as one launch each
        q, _, _ = grp(x, [layer["q"], layer["kv0"], layer["kv1"]])
        # row-parallel o and down: the all-reduce runs inside the GEMV kernel (peer-memory packets);
        # --nccl-allreduce switches to GEMV + NCCL all-reduce for comparison
        if comm is not None:
            o = comm.linear(q, layer["o"], overlap_previous=True)
            g, _ = grp(o, [layer["gate_up0"], layer["gate_up1"]])
            out = comm.linear(g, layer["down"], overlap_previous=True)
        else:
            o = lin(q, layer["o"])
            if world > 1:
                dist.all_reduce(o)
            g, _ = grp(o, [layer["gate_up0"], layer["gate_up1"]])
            out = lin(g, layer["down"])
            if world > 1:
                dist.all_reduce(out)
    return out


def rel_err(y: torch.Tensor, ref: torch.Tensor) -> float:
    y, ref = y.double(), ref.double()
    return float((y - ref).norm() / ref.norm().clamp_min(1e-300))


def correctness_check(model, world: int, rank: int, m: int, comm, dev) -> dict:
    """Layer 0's o and down projections, outside the timed region, against a float64 matmul on the
    dequantized UNSHARDED weight (mixfp4_dequant: bit-equal to the reference's dequantized weight).
    One GPU: the decode kernel alone.  Several GPUs: the fused GEMV + all-reduce and the GEMV followed
    by an NCCL all-reduce of fp32 partial sums; also whether all ranks hold the same bits."""
    import torch.distributed as dist
    import mixfp4_b200 as mx
    out = {"tolerance": 1e-3}
    worst, same_bits, fused_vs_nccl = 0.0, True, 0.0
    for name in ("o", "down"):
        shard = model[0][name]
        wfull = model[0]["full_" + name]
        kfull = wfull.shape[1]
        x = torch.randn((m, kfull), generator=torch.Generator().manual_seed(11)).to(torch.bfloat16).to(dev)
        ref = x.double() @ wfull.double().T
        step = kfull // world
        xs = x[:, rank * step:(rank + 1) * step].contiguous() if world > 1 else x
        y_plain = mx.mixfp4_linear(xs, shard, out_dtype=torch.float32)
        if world > 1:
            dist.all_reduce(y_plain)
            if comm is not None:
                y_fused = comm.linear(xs, shard, out_dtype=torch.float32)
                worst = max(worst, rel_err(y_fused, ref))
                fused_vs_nccl = max(fused_vs_nccl, rel_err(y_fused, y_plain))
                gathered = [torch.empty_like(y_fused) for _ in range(world)]
                dist.all_gather(gathered, y_fused)
                same_bits = same_bits and all(torch.equal(g, gathered[0]) for g in gathered)
        worst = max(worst, rel_err(y_plain, ref))
        out[name + "_rel"] = round(rel_err(y_plain, ref), 9)
    flag = torch.tensor([worst, fused_vs_nccl, 0.0 if same_bits else 1.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    worst, fused_vs_nccl, differ = flag.tolist()
    out.update({"vs_dequantized_fp64_rel": round(worst, 9), "ok": bool(worst <= 1e-3 and differ == 0.0)})
    if world > 1:
        out.update({"fused_vs_nccl_rel": round(fused_vs_nccl, 9), "all_ranks_same_bits": differ == 0.0,
                    "fused_path": comm is not None})
    return out


def run_ours(args):
    import torch.distributed as dist
    import mixfp4_b200 as mx

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # stdout carries the one result line and nothing else: libraries that write to file descriptor 1
        # (NCCL prints its version banner there) get standard error instead, the result line goes to the
        # original descriptor
        sys.stdout.flush()
        result_fd = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        result_fd = None

    def emit(text: str) -> None:
        if result_fd is None:
            print(text, flush=True)
        else:
            sys.stdout.flush()
            os.write(result_fd, (text + "\n").encode())

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    m = args.m
    layers, nlayers = layer_list()
    total_bytes = nlayers * sum(algorithmic_bytes(n, k, m) for _, n, k in layers)
    launches_per_step = nlayers * LAUNCHES_PER_LAYER
    global TRAFFIC_BYTES_PER_LAUNCH
    TRAFFIC_BYTES_PER_LAUNCH = int(TRAFFIC_OVER_ALGORITHMIC * total_bytes / launches_per_step / world)

    model = build_model(dev, rank, world, m, args.layout)
    x_host = torch.randn((m, 4096), generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    out_host = torch.empty((m, 4096), dtype=torch.bfloat16).pin_memory()

    comm = None
    if world > 1 and not args.nccl_allreduce and m <= 8:
        from mixfp4_b200.parallel import PeerCommunicator
        comm = PeerCommunicator(slot_floats=m * 4096, device=dev)

    check = correctness_check(model, world, rank, m, comm, dev)
    if not check["ok"]:
        if rank == 0:
            emit(json.dumps({"metric": METRIC, "error": "correctness check failed", "check": check}))
        os._exit(3)

    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        static_out = decode_pass(model, x_dev, world, comm=comm)          # warm-up outside capture
        torch.cuda.synchronize(dev)
        with torch.cuda.graph(graph, stream=side):
            static_out = decode_pass(model, x_dev, world, comm=comm)
    torch.cuda.synchronize(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident timing: K graph replays
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1) / args.steps

    # ---- end to end: pinned host x -> device, replay, device -> pinned host, every step
    for _ in range(3):
        x_dev.copy_(x_host, non_blocking=True); graph.replay(); out_host.copy_(static_out, non_blocking=True)
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.steps):
        x_dev.copy_(x_host, non_blocking=True)
        graph.replay()
        out_host.copy_(static_out, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
    e3.record()
    barrier()
    e2e_ms = e2.elapsed_time(e3) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()

    finite = bool(torch.isfinite(static_out.float()).all().item())
    fused = comm is not None
    peer_status = int(comm.status.item()) if comm is not None else None
    decode_status = mx.decode_status(dev)
    extra = {}
    if not args.no_extra:
        del model, graph, static_out
        if comm is not None:
            comm.close()
            comm = None
        torch.cuda.empty_cache()
        from mixfp4_b200 import llama_decode
        if world == 1:
            # short kernels first: the sections after them keep the GPU under its power cap for seconds
            extra.update(secondary_numbers(dev))
            extra["decode_tokens_per_s_linears_only"] = round(1e3 / dev_ms * m, 1)
            extra["prefill_h128"] = prefill_sweep(dev)
            torch.cuda.empty_cache()
        extra["tp70b"] = tp70b(dev, rank, world, args.layout)
        torch.cuda.empty_cache()
        # whole decoder (norms, RoPE, attention over a bf16 KV cache, bf16 head as stock PyTorch operators
        # around the packed linears): tokens/s and the linears' share of a step; head-parallel over the ranks
        keep = {}
        for batch, prompt in ((1, 2048), (8, 2048), (16, 2048), (32, 2048)) if world == 1 else ((1, 2048), (8, 2048)):
            r = llama_decode.run(layers=nlayers, batch=batch, prompt=prompt, tokens=8, device=dev, tp=world,
                                 weights=keep.get("weights"), keep=keep)
            extra["decode_full_model_b%d" % batch] = {k: r[k] for k in (
                "decode_tokens_per_s", "decode_ms_per_step", "mixfp4_linear_time_fraction", "prefill_tokens_per_s", "tp")}

    if rank == 0:
        peak, peak_kind = measured_peak()
        value = total_bytes / (dev_ms * 1e-3) / 1e9
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(dev_ms, 4), "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "ours",
            "config": {"workload": "llama3-8b decode linears, M=%d, 32 layers x 7 linears in 4 launches (q/k/v and gate/up grouped), mixed E2M1/E0M3 K16 blocks" % m,
                       "parallelism": ("tp%d, all-reduce %s" % (world, "fused into the row-parallel GEMV" if fused else "NCCL")) if world > 1 else "single",
                       "l2": "working set 3.98 GB of distinct weights >> 126 MB L2 (no flush needed)",
                       "timing": "cuda events around graph replays, max over ranks"},
            "clocks": clocks,
            "e2e": {"value": round(total_bytes / (e2e_ms * 1e-3) / 1e9, 1), "unit": UNIT,
                    "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(per_gpu / peak, 4), "peak_kind": peak_kind, "kernel": "gemv_stream_kernel" if args.layout == "stream" else "gemv_sm_kernel",
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH,
                         "note": "achieved = algorithmic bytes of the %d GEMV launches of a step / CUDA-event time" % launches_per_step},
            "check": check, "tp_check": check if world > 1 else None, "output_finite": finite, "decode_status": decode_status,
            "peer_wait_status": peer_status,
            "cpu_baseline": cpu_baseline(m, budget_s=12.0) if world == 1 and not args.no_cpu else None,
            "extra": extra,
        }
        emit(json.dumps(line))
    if world > 1:
        # Leave without tearing NCCL down: destroying a process group while a CUDA graph that
        # captured its collectives is alive can block forever.  All ranks are past their last
        # collective (the MAX all-reduce above), so a hard exit is safe.
        torch.cuda.synchronize(dev)
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


def graph_time(fn, dev, iters: int, world: int = 1) -> float:
    """Seconds per call of fn, captured once as a CUDA graph and replayed (max over ranks)."""
    import torch.distributed as dist
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize(dev)
        with torch.cuda.graph(g, stream=side):
            fn()
    for _ in range(3):
        g.replay()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        g.replay()
    b.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([a.elapsed_time(b) / iters * 1e-3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    del g
    return float(t.item())


def tp70b(dev, rank: int, world: int, layout: str) -> dict:
    """BASELINE config 4: Llama-3-70B-shaped linears (hidden 8192, kv 1024, FFN 28672) tensor-parallel
    over the ranks -- q/k/v/gate/up split along N, o/down along K.  Four distinct layers are cycled
    (a layer is 488 MB packed, so four exceed the L2 many times over).
      decode  M = 1: the seven linears of each layer in four launches, the row-parallel ones with the
              all-reduce fused into the GEMV (NCCL-free) when there is more than one rank;
      prefill M = 4096: gate, up (column-parallel) and down (row-parallel) through the tcgen05 GEMM,
              the [4096, 8192] bf16 partial sums of down all-reduced by NCCL, once in stream order and
              once on a side stream under the next layer's GEMMs;
      quantize: the 80-layer weight quantization sharded by layer (layer l on rank l mod N), timed on
              one layer's set of unsharded weights per owned layer.
    Values are whole-job figures (all ranks), times the maximum over ranks."""
    import torch.distributed as dist
    import mixfp4_b200 as mx
    from mixfp4_b200 import synth
    from mixfp4_b200.parallel import PeerCommunicator
    hidden, kvd, ffn, cycled = 8192, 1024, 28672, 4
    shapes = {"q": (hidden, hidden), "k": (kvd, hidden), "v": (kvd, hidden), "o": (hidden, hidden),
              "gate": (ffn, hidden), "up": (ffn, hidden), "down": (hidden, ffn)}
    gen = torch.Generator(device=dev)

    def weight(n, k, seed):
        gen.manual_seed(seed)
        return (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)

    # ---- layer-sharded quantization of 80 layers (unsharded shapes), before anything else holds memory
    full = {name: weight(n, k, 7000 + i) for i, (name, (n, k)) in enumerate(shapes.items()) if name not in ("v", "up")}
    full["v"], full["up"] = full["k"], full["gate"]
    owned = len(range(rank, synth.LLAMA3_70B_NUM_LAYERS, world))
    for w in full.values():
        mx.quantize_packed(w)
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for _ in range(owned):
        for name in shapes:
            mx.quantize_packed(full[name])
    torch.cuda.synchronize(dev)
    tq = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tq, op=dist.ReduceOp.MAX)
    elems_layer = sum(n * k for n, k in shapes.values())
    out = {"quantize_80_layers_s": round(float(tq.item()), 4),
           "quantize_gelem_per_s": round(80 * elems_layer / float(tq.item()) / 1e9, 1),
           "layers_per_rank": owned}

    # ---- sharded packed layers
    layers = []
    for li in range(cycled):
        entry = {}
        for i, (name, (n, k)) in enumerate(shapes.items()):
            w = weight(n, k, 100 * li + i)
            amax = mx.tensor_amax(w)
            if world > 1:
                if name in ("o", "down"):
                    step = k // world
                    w = w[:, rank * step:(rank + 1) * step].contiguous()
                else:
                    step = n // world
                    w = w[rank * step:(rank + 1) * step].contiguous()
            entry[name] = to_layout(mx.quantize_packed(w, amax=amax)[0], layout)
            del w
        layers.append(entry)
    del full
    torch.cuda.empty_cache()
    layer_bytes = sum(algorithmic_bytes(n, k, 1) for n, k in shapes.values())
    comm = PeerCommunicator(slot_floats=hidden, device=dev) if world > 1 else None
    x1 = torch.randn((1, hidden), device=dev).to(torch.bfloat16)

    def decode():
        for layer in layers:
            q, _, _ = mx.mixfp4_linear_grouped(x1, [layer["q"], layer["k"], layer["v"]], overlap_previous=True)
            if comm is not None:
                o = comm.linear(q, layer["o"], overlap_previous=True)
            else:
                o = mx.mixfp4_linear(q, layer["o"], overlap_previous=True)
            g, _ = mx.mixfp4_linear_grouped(o, [layer["gate"], layer["up"]], overlap_previous=True)
            if comm is not None:
                comm.linear(g, layer["down"], overlap_previous=True)
            else:
                mx.mixfp4_linear(g, layer["down"], overlap_previous=True)

    t = graph_time(decode, dev, 10, world) / cycled
    peak, _ = measured_peak()
    out["decode_m1"] = {"ms_per_layer": round(t * 1e3, 4), "gbs": round(layer_bytes / t / 1e9, 1),
                        "per_gpu_frac_of_hbm": round(layer_bytes / t / 1e9 / world / peak, 4),
                        "tokens_per_s_80_layers_linears_only": round(1.0 / (80 * t), 1),
                        "all_reduce": "fused into the GEMV" if comm is not None else "none (one GPU)"}
    if comm is not None:
        out["decode_m1"]["peer_wait_status"] = int(comm.status.item())

    # ---- prefill MLP at M = 4096
    mtok = 4096
    xp = torch.randn((mtok, hidden), device=dev).to(torch.bfloat16)
    side = torch.cuda.Stream(dev)
    flops_layer = 2.0 * mtok * 3 * ffn * hidden

    def prefill(overlap: bool):
        pending = None
        for layer in layers:
            g = mx.mixfp4_linear(xp, layer["gate"])
            mx.mixfp4_linear(xp, layer["up"])
            d = mx.mixfp4_linear(g, layer["down"])               # [4096, 8192] bf16 partial sums of this rank's K shard
            if world > 1:
                if overlap:
                    ev = torch.cuda.Event()
                    ev.record()
                    with torch.cuda.stream(side):
                        side.wait_event(ev)
                        dist.all_reduce(d)
                        pending = torch.cuda.Event()
                        pending.record()
                else:
                    dist.all_reduce(d)
        if pending is not None:
            torch.cuda.current_stream(dev).wait_event(pending)

    def timed_prefill(overlap):
        for _ in range(2):
            prefill(overlap)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            prefill(overlap)
        b.record()
        torch.cuda.synchronize(dev)
        tt = torch.tensor([a.elapsed_time(b) / 3 / cycled * 1e-3], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    tp = timed_prefill(False)
    out["prefill_m4096_mlp"] = {"ms_per_layer": round(tp * 1e3, 3), "tflops": round(flops_layer / tp / 1e12, 1),
                                "all_reduce": "NCCL, bf16 [4096, 8192], in stream order" if world > 1 else "none (one GPU)",
                                "gemm_status": mx.gemm_status(dev)}
    if world > 1:
        to = timed_prefill(True)
        out["prefill_m4096_mlp"]["tflops_all_reduce_on_side_stream"] = round(flops_layer / to / 1e12, 1)
    if comm is not None:
        comm.close()
    return out


def prefill_sweep(dev) -> dict:
    """BASELINE config 3: the Llama-3-8B layer shapes at M = 512, 2048 and 8192 through the tcgen05
    GEMM with the H128 rotation of x applied inside the call (weights rotated before quantization),
    activations N(0,1) with 1 % of the channels scaled by 30, bf16 out, replayed as CUDA graphs (device
    time of rotation pass + GEMM).  TFLOP/s and the fraction of the measured dense bf16 peak."""
    import mixfp4_b200 as mx
    from mixfp4_b200 import synth
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak_tf = float(json.load(f)["bf16_tflops"])
    except Exception:
        peak_tf = 1590.0
    out = {}
    shapes = {"q": (4096, 4096), "kv": (1024, 4096), "o": (4096, 4096), "gate_up": (14336, 4096), "down": (4096, 14336)}
    for name, (n, k) in shapes.items():
        w = (torch.randn((n, k), device=dev) * 0.02).to(torch.bfloat16)
        packed = mx.quantize_packed(mx.apply_transform(w, "H128"), rotation="H128")[0].to_stream_layout()
        for m in (512, 2048, 8192):
            x = synth.activations(m, k, seed=m, outlier_fraction=0.01).to(dev)
            # captured as a CUDA graph: at the small shapes a call's host side (argument marshalling, three
            # tensor-map encodings, two or three launches; about 40 us) is longer than its kernels
            reps = 4 if m <= 512 else (2 if m <= 2048 else 1)

            def fn():
                for _ in range(reps):
                    mx.mixfp4_linear(x, packed)

            for _ in range(2):
                fn()
            t = graph_time(fn, dev, 6) / reps
            tf = 2.0 * m * n * k / t / 1e12
            out["%s_%dx%d_m%d" % (name, n, k, m)] = {"tflops": round(tf, 1), "frac_bf16_peak": round(tf / peak_tf, 3)}
        del w, packed
    out["gemm_status"] = mx.gemm_status(dev)
    return out


def secondary_numbers(dev) -> dict:
    """Other kernels and shapes of the path, device-timed (reported beside the headline, not
    part of `value`): the quantizer, the decode GEMV at M = 4 and 16, and the prefill GEMM at
    M = 4096 (tensor-pipe roofline), with and without the on-line H128 rotation."""
    import mixfp4_b200 as mx
    out = {}

    def timeit(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / iters * 1e-3

    n, k = 14336, 4096
    ws = [(torch.randn((n, k), device=dev) * 0.02).to(torch.bfloat16) for _ in range(4)]  # 470 MB > L2
    state = {"i": 0}

    def quant():
        state["i"] = (state["i"] + 1) % len(ws)
        mx.quantize_packed(ws[state["i"]])

    def quant_all():
        for _ in ws:
            quant()

    # device time of amax + quantize per weight: one CUDA graph over the four weights
    t = graph_time(quant_all, dev, 6) / len(ws)
    out["quantize_gbs_14336x4096"] = round((2 * n * k + mx.packed_nbytes(n, k)) / t / 1e9, 1)
    out["quantize_ms_14336x4096"] = round(t * 1e3, 4)

    # decode GEMV at larger batch, gate/up shape, cycling over distinct weights (> L2)
    packs = [mx.quantize_packed(w)[0].to_stream_layout() for w in ws]
    for m in (4, 16):
        x = torch.randn((m, k), device=dev).to(torch.bfloat16)

        def gemv_pass():
            for _ in range(4):           # 16 launches per replay: the replay's own launch cost stays small
                for p in packs:
                    mx.mixfp4_linear(x, p, overlap_previous=True)

        # as a CUDA graph of dependent launches, like the headline (a Python call per launch costs
        # more than the kernel)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            gemv_pass()
            torch.cuda.synchronize(dev)
            with torch.cuda.graph(g, stream=side):
                gemv_pass()
        torch.cuda.synchronize(dev)
        t = timeit(g.replay, 10) / (4 * len(packs))
        out["gemv_gbs_m%d_14336x4096" % m] = round(algorithmic_bytes(n, k, m) / t / 1e9, 1)

    peak_tf = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak_tf = float(json.load(f)["bf16_tflops"])
    except Exception:
        peak_tf = 1590.0
    for name, (gn, gk) in {"q_4096x4096": (4096, 4096), "gate_14336x4096": (14336, 4096), "down_4096x14336": (4096, 14336)}.items():
        w = (torch.randn((gn, gk), device=dev) * 0.02).to(torch.bfloat16)
        packed = mx.quantize_packed(w)[0].to_kernel_layout()
        x = torch.randn((4096, gk), device=dev).to(torch.bfloat16)
        # device time (CUDA graph replays; eager calls leave a few microseconds between the kernels)
        t = graph_time(lambda: mx.mixfp4_linear(x, packed), dev, 8)
        tf = 2.0 * 4096 * gn * gk / t / 1e12
        out["gemm_tflops_m4096_" + name] = round(tf, 1)
        out["gemm_frac_bf16_peak_m4096_" + name] = round(tf / peak_tf, 3)
        if name == "q_4096x4096":
            rot = mx.quantize_packed(mx.apply_transform(w, "H128"), rotation="H128")[0].to_kernel_layout()
            t = graph_time(lambda: mx.mixfp4_linear(x, rot), dev, 8)
            out["gemm_tflops_m4096_q_4096x4096_h128_rotation"] = round(2.0 * 4096 * gn * gk / t / 1e12, 1)
            # W4A4 in the reference's sense: rotation, activation fake-quantization and GEMM in one call
            t = graph_time(lambda: mx.mixfp4_linear(x, rot, activation_mode="oracle16"), dev, 8)
            out["gemm_tflops_m4096_q_4096x4096_h128_w4a4"] = round(2.0 * 4096 * gn * gk / t / 1e12, 1)
            t = graph_time(lambda: mx.fake_quantize_activations(x, "oracle16"), dev, 8)
            out["fake_quantize_gbs_4096x4096"] = round(4.0 * 4096 * gk / t / 1e9, 1)     # bf16 in + bf16 out
        del w, packed, x
    out["bf16_peak_tflops"] = peak_tf
    out["decode_tokens_per_s_linears_only"] = None   # filled by the caller from ms_per_step
    return out


# --------------------------------------------------------------------------- CPU arm
def cpu_layer_sample(m: int):
    """One decoder layer's seven weights (seeded, CPU) quantized by the eager-op port of the
    reference quantizer; returns (fp32 dequantized weights, activations, quantize seconds)."""
    from mixfp4_b200 import synth
    from oracle import torch_port
    layers, _ = layer_list()
    torch.set_num_threads(os.cpu_count() or 1)
    ws, t_quant, elems = [], 0.0, 0
    for idx, (name, n, k) in enumerate(layers):
        w = (torch.randn((n, k), generator=torch.Generator().manual_seed(idx)) * 0.02).to(torch.bfloat16)
        t0 = time.perf_counter()
        dq = torch_port.quantize_dequant(w)
        t_quant += time.perf_counter() - t0
        elems += n * k
        ws.append(dq.float())
    xs = {k: torch.randn((m, k), generator=torch.Generator().manual_seed(99)).to(torch.bfloat16)
          for k in (4096, 14336)}
    return ws, xs, t_quant, elems


def cpu_linear_step(ws, xs):
    from oracle import torch_port
    for w in ws:
        torch_port.linear(xs[w.shape[1]], w)


def cpu_baseline(m: int, budget_s: float = 12.0) -> dict:
    layers, _ = layer_list()
    ws, xs, t_quant, elems = cpu_layer_sample(m)
    cpu_linear_step(ws, xs)
    reps, t0 = 0, time.perf_counter()
    while True:
        cpu_linear_step(ws, xs)
        reps += 1
        if time.perf_counter() - t0 > max(1.0, budget_s - t_quant) or reps >= 200:
            break
    t_lin = (time.perf_counter() - t0) / reps
    layer_bytes = sum(algorithmic_bytes(n, k, m) for _, n, k in layers)
    return {"value": round(layer_bytes / t_lin / 1e9, 2), "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": "1 of 32 layers (7 linears, 218M weights): eager-op port of the reference quantizer once "
                      "(%.2f s, %.1f M elements/s) + %d passes of fp32 F.linear on the dequantized weights"
                      % (t_quant, elems / t_quant / 1e6, reps),
            "quantize_melem_per_s": round(elems / t_quant / 1e6, 1), "linear_ms_per_layer": round(t_lin * 1e3, 3)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    m = args.m
    layers, _ = layer_list()
    ws, xs, t_quant, elems = cpu_layer_sample(m)
    for _ in range(max(args.warmup, 1)):
        cpu_linear_step(ws, xs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_linear_step(ws, xs)
    ms = (time.perf_counter() - t0) / args.steps * 1e3
    layer_bytes = sum(algorithmic_bytes(n, k, m) for _, n, k in layers)
    value = round(layer_bytes / (ms * 1e-3) / 1e9, 2)
    sample = ("each step = 1 of the 32 layers (7 fp32 F.linear calls on dequantized weights, %d host threads); "
              "weights quantized once by the eager-op port of the reference quantizer in %.2f s" % (os.cpu_count(), t_quant))
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
        "config": {"workload": "llama3-8b decode linears, M=%d, CPU sample of 1/32 of the model per step" % m},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": sample,
                         "quantize_melem_per_s": round(elems / t_quant / 1e6, 1)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------ single-kernel timing
def run_kernel(args):
    """One kernel alone on one shape (the command the profiler summaries under profiles/ were
    captured with): prints one line with the kernel's algorithmic bytes or flops per second.
    Weights are seeded N(0, 0.02^2) bf16 tensors quantized on the device; the GEMV cycles over
    enough distinct packed weights to exceed the L2 and runs as a CUDA graph of dependent launches."""
    import mixfp4_b200 as mx
    torch.cuda.set_device(0)
    n, k, m = args.shape

    def timed(fn, iters, warm=3):
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

    def weight(seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        return (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)

    if args.kernel == "gemv":
        per = mx.packed_nbytes(n, k)
        buffers = args.buffers or max(2, int(600e6 // per))
        packs = [to_layout(mx.quantize_packed(weight(i))[0], args.layout) for i in range(buffers)]
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
        t = timed(graph.replay, args.steps) / buffers
        algo = per + 2 * m * k + 2 * m * n
        print(json.dumps({"kernel": "gemv", "layout": args.layout, "n": n, "k": k, "m": m, "us_per_launch": round(t * 1e6, 2),
                          "gbs": round(algo / t / 1e9, 1), "buffers": buffers, "decode_status": mx.decode_status()}))
    elif args.kernel == "gemm":
        w = weight(0)
        if args.rotate:
            packed = to_layout(mx.quantize_packed(mx.apply_transform(w, "H128"), rotation="H128")[0], args.layout)
        else:
            packed = to_layout(mx.quantize_packed(w)[0], args.layout)
        x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
        t_eager = timed(lambda: mx.mixfp4_linear(x, packed), args.steps)
        # device time: the same call replayed as a CUDA graph (a call's host side costs about 40 us, more
        # than the kernels of a small problem)
        reps = 4 if 2.0 * m * n * k < 4e11 else 1
        t = graph_time(lambda: [mx.mixfp4_linear(x, packed) for _ in range(reps)], torch.device("cuda", 0), args.steps) / reps
        print(json.dumps({"kernel": "gemm", "layout": args.layout, "n": n, "k": k, "m": m, "h128": bool(args.rotate),
                          "us": round(t * 1e6, 1), "tflops": round(2.0 * m * n * k / t / 1e12, 1),
                          "us_eager_calls": round(t_eager * 1e6, 1), "gemm_status": mx.gemm_status()}))
    else:
        ws = [weight(i) for i in range(max(2, int(400e6 // (2 * n * k))))]
        state = {"i": 0}

        def run():
            state["i"] = (state["i"] + 1) % len(ws)
            mx.quantize_packed(ws[state["i"]])

        t = timed(run, args.steps)
        algo = 2 * n * k + mx.packed_nbytes(n, k)
        print(json.dumps({"kernel": "quantize", "n": n, "k": k, "us": round(t * 1e6, 1), "gbs": round(algo / t / 1e9, 1)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="decode batch (1..16)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary kernel numbers")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="multi-GPU: GEMV + NCCL all-reduce instead of the fused GEMV + all-reduce kernel")
    ap.add_argument("--layout", default="stream", choices=["stream", "kernel"],
                    help="packed layout of the weights the linears read (stream: 1152-byte chunks; kernel: row-major)")
    ap.add_argument("--kernel", default=None, choices=["gemv", "gemm", "quantize"],
                    help="time one kernel alone on --shape N K M instead of the decode workload")
    ap.add_argument("--shape", type=int, nargs=3, default=[14336, 4096, 1], metavar=("N", "K", "M"))
    ap.add_argument("--buffers", type=int, default=None, help="--kernel gemv: distinct weights to cycle over")
    ap.add_argument("--rotate", action="store_true", help="--kernel gemm: H128 rotation of x inside the call")
    args = ap.parse_args()
    if args.kernel:
        run_kernel(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

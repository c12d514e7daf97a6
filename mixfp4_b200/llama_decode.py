"""End-to-end decode harness: a random-init Llama-3-8B-shaped decoder whose linears are packed
mixed-FP4 layers, to report tokens/s and the share of a decode step spent in the mixed-FP4 GEMVs.

    python -m mixfp4_b200.llama_decode [--layers 32] [--batch 1] [--prompt 2048] [--tokens 32]
    python -m torch.distributed.run --nproc-per-node 8 -m mixfp4_b200.llama_decode --tp 8 ...

Architecture: hidden 4096, 32 query / 8 KV heads of 128, FFN 14336, RMSNorm, RoPE (theta 5e5),
vocab 128256, bf16 KV cache.  Weights are seeded synthetic tensors (no checkpoint is available
offline), quantized on the device layer by layer; the prompt is uniform random token ids.
Everything that is not a linear -- norms, RoPE, attention over the KV cache, SiLU, the bf16
embedding and output head -- runs as stock PyTorch operators: those are not part of the
mixed-FP4 path, they are here so that the linears run in their real data flow (grouped q/k/v and
gate/up launches, chained launches, batch rows = sequences).  The prompt is prefilled through the
tcgen05 GEMM path, the decode steps are captured in one CUDA graph per step shape.

Tensor parallel (--tp N, one process per GPU): attention heads and FFN columns are split over the
ranks -- q/k/v/gate/up along N, o/down along K with the whole tensor's scale -- the KV cache holds
this rank's heads, and the two row-parallel projections of a layer end in an all-reduce: fused into
the decode GEMV (peer-memory packets) for up to 8 rows, NCCL on fp32 partial sums otherwise.
"""

from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist
import torch.nn.functional as F

import mixfp4_b200 as mx

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, FFN, VOCAB = 4096, 32, 8, 128, 14336, 128256
ROPE_THETA, EPS = 500000.0, 1e-5


def _student_t(n: int, k: int, gen: torch.Generator, device) -> torch.Tensor:
    z = torch.randn((n, k), generator=gen, device=device)
    chi = torch.zeros((n, k), device=device)
    for _ in range(4):
        d = torch.randn((n, k), generator=gen, device=device)
        chi.addcmul_(d, d)
    return (z / torch.sqrt(chi / 4) * 0.02).to(torch.bfloat16)


class Layer:
    def __init__(self, index: int, device, gen: torch.Generator, rank: int = 0, world: int = 1):
        def packed(n, k, tag, split=None):
            gen.manual_seed(1000 * index + tag)
            w = _student_t(n, k, gen, device)
            amax = mx.tensor_amax(w)                 # the whole tensor's scale, whatever the shard
            if world > 1 and split == "n":
                w = w[rank * (n // world):(rank + 1) * (n // world)].contiguous()
            elif world > 1 and split == "k":
                w = w[:, rank * (k // world):(rank + 1) * (k // world)].contiguous()
            return mx.quantize_packed(w, amax=amax)[0].to_stream_layout()
        self.q, self.k, self.v = (packed(HIDDEN, HIDDEN, 0, "n"), packed(KV_HEADS * HEAD_DIM, HIDDEN, 1, "n"),
                                  packed(KV_HEADS * HEAD_DIM, HIDDEN, 2, "n"))
        self.o = packed(HIDDEN, HIDDEN, 3, "k")
        self.gate, self.up, self.down = packed(FFN, HIDDEN, 4, "n"), packed(FFN, HIDDEN, 5, "n"), packed(HIDDEN, FFN, 6, "k")
        self.norm1 = torch.ones(HIDDEN, dtype=torch.bfloat16, device=device)
        self.norm2 = torch.ones(HIDDEN, dtype=torch.bfloat16, device=device)


def rms_norm(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],), w, EPS)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x [B, T, H, D]; cos/sin [T, D/2]
    a, b = x.float().chunk(2, dim=-1)
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat((a * c - b * s, a * s + b * c), dim=-1).to(x.dtype)


class Decoder:
    def __init__(self, layers: int, batch: int, max_len: int, device, rank: int = 0, world: int = 1, weights=None):
        """weights: the `.weights` of another Decoder with the same layers and ranks, to share the
        packed tensors between harness runs at different batch sizes."""
        self.device, self.batch, self.max_len, self.rank, self.world = device, batch, max_len, rank, world
        if HEADS % world or KV_HEADS % world:
            raise ValueError("the tensor-parallel degree must divide 8 KV heads")
        self.heads, self.kv_heads = HEADS // world, KV_HEADS // world
        if weights is None:
            gen = torch.Generator(device=device)
            stack = [Layer(i, device, gen, rank, world) for i in range(layers)]
            gen.manual_seed(99)
            embed = (torch.randn((VOCAB, HIDDEN), generator=gen, device=device) * 0.02).to(torch.bfloat16)
            head = (torch.randn((VOCAB, HIDDEN), generator=gen, device=device) * 0.02).to(torch.bfloat16)
            weights = (stack, embed, head)
        self.weights = weights
        self.layers, self.embed, self.head = weights
        self.final_norm = torch.ones(HIDDEN, dtype=torch.bfloat16, device=device)
        self.k_cache = [torch.zeros((batch, self.kv_heads, max_len, HEAD_DIM), dtype=torch.bfloat16, device=device) for _ in self.layers]
        self.v_cache = [torch.zeros_like(c) for c in self.k_cache]
        inv = 1.0 / (ROPE_THETA ** (torch.arange(0, HEAD_DIM, 2, device=device).float() / HEAD_DIM))
        ang = torch.arange(max_len, device=device).float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.linears_only = False        # timing aid: skip everything but the linears
        self.comm = None
        if world > 1:
            from .parallel import PeerCommunicator
            self.comm = PeerCommunicator(slot_floats=8 * HIDDEN, device=device)

    def row_parallel(self, x: torch.Tensor, packed) -> torch.Tensor:
        """sum over ranks of x_shard @ W_shard^T: the fused GEMV + all-reduce for decode shapes, else
        fp32 partial sums through NCCL, rounded afterwards."""
        if self.world == 1:
            return mx.mixfp4_linear(x, packed, overlap_previous=True)
        if x.shape[0] <= 8:
            y = self.comm.linear(x, packed, overlap_previous=True)
            if y is not None:
                return y
        y = mx.mixfp4_linear(x, packed, out_dtype=torch.float32)
        dist.all_reduce(y)
        return y.to(x.dtype)

    def forward(self, tokens: torch.Tensor, pos: torch.Tensor, length: int) -> torch.Tensor:
        """tokens [B, T] at positions pos [T] (T = prompt length at prefill, 1 at decode); the
        cache holds `length` valid positions after this call.  Returns logits [B, vocab] of the
        last position."""
        b, t = tokens.shape
        width = self.heads * HEAD_DIM                                     # this rank's slice of the hidden size
        h = self.embed[tokens]                                            # [B, T, hidden]
        cos, sin = self.cos[pos], self.sin[pos]
        for i, layer in enumerate(self.layers):
            x = h if self.linears_only else rms_norm(h, layer.norm1)
            q, k, v = mx.mixfp4_linear_grouped(x.reshape(b * t, HIDDEN), [layer.q, layer.k, layer.v], overlap_previous=True)
            if self.linears_only:
                attn = q
            else:
                q = rope(q.view(b, t, self.heads, HEAD_DIM), cos, sin).transpose(1, 2)
                k = rope(k.view(b, t, self.kv_heads, HEAD_DIM), cos, sin).transpose(1, 2)
                v = v.view(b, t, self.kv_heads, HEAD_DIM).transpose(1, 2)
                self.k_cache[i][:, :, pos] = k
                self.v_cache[i][:, :, pos] = v
                keys, vals = self.k_cache[i][:, :, :length], self.v_cache[i][:, :, :length]
                attn = F.scaled_dot_product_attention(q, keys, vals, is_causal=t > 1, enable_gqa=True)
                attn = attn.transpose(1, 2).reshape(b * t, width)
            o = self.row_parallel(attn, layer.o)
            if self.linears_only:
                x, h2 = o, h
            else:
                h2 = h + o.view(b, t, HIDDEN)
                x = rms_norm(h2, layer.norm2).reshape(b * t, HIDDEN)
            g, u = mx.mixfp4_linear_grouped(x, [layer.gate, layer.up], overlap_previous=True)
            act = g if self.linears_only else F.silu(g) * u
            d = self.row_parallel(act, layer.down)
            h = d.view(b, t, HIDDEN) if self.linears_only else h2 + d.view(b, t, HIDDEN)
        last = rms_norm(h[:, -1], self.final_norm)
        return last @ self.head.T


def _time_graph(fn, steps: int) -> float:
    """Median-free simple timing: capture fn once, replay `steps` times, ms per replay."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            fn()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


@torch.no_grad()
def run(layers: int = 32, batch: int = 1, prompt: int = 2048, tokens: int = 32, device=None, tp: int = 1,
        weights=None, keep: dict | None = None) -> dict:
    """tp > 1: torch.distributed must be initialised with `tp` ranks (one per GPU); times are the
    maximum over ranks.  weights / keep: pass keep={} to receive the model's packed weights in
    keep["weights"], and hand them back as `weights` to run another batch size without rebuilding."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    rank = dist.get_rank() if tp > 1 else 0
    model = Decoder(layers, batch, prompt + tokens + 1, device, rank, tp, weights)
    if keep is not None:
        keep["weights"] = model.weights
    gen = torch.Generator(device=device).manual_seed(5)
    ids = torch.randint(0, VOCAB, (batch, prompt), generator=gen, device=device)
    # prefill (tcgen05 GEMM path), timed with events
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    model.forward(ids, torch.arange(prompt, device=device), prompt)      # first call: one-time set-up costs
    torch.cuda.synchronize()
    e0.record()
    logits = model.forward(ids, torch.arange(prompt, device=device), prompt)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    assert torch.isfinite(logits).all()
    # decode: one token per sequence at the position after the prompt, cache length prompt + 1
    nxt = logits.argmax(-1, keepdim=True)
    pos = torch.tensor([prompt], device=device)
    step = lambda: model.forward(nxt, pos, prompt + 1)
    full_ms = _time_graph(step, tokens)
    model.linears_only = True
    lin_ms = _time_graph(step, tokens)
    model.linears_only = False
    if tp > 1:
        t = torch.tensor([prefill_ms, full_ms, lin_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_ms, full_ms, lin_ms = t.tolist()
        status = int(model.comm.status.item())
        model.comm.close()
    else:
        status = 0
    return {
        "layers": layers, "batch": batch, "prompt_tokens": prompt, "decode_steps_timed": tokens, "tp": tp,
        "prefill_ms": round(prefill_ms, 2), "prefill_tokens_per_s": round(batch * prompt / prefill_ms * 1e3, 1),
        "decode_ms_per_step": round(full_ms, 4), "decode_tokens_per_s": round(batch / full_ms * 1e3, 1),
        "mixfp4_linears_ms_per_step": round(lin_ms, 4), "mixfp4_linear_time_fraction": round(lin_ms / full_ms, 3),
        "peer_wait_status": status,
    }


def main() -> None:
    import os
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=32)
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree (launch with torch.distributed.run)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if args.tp > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    result = run(args.layers, args.batch, args.prompt, args.tokens, tp=args.tp)
    if args.tp == 1 or dist.get_rank() == 0:
        print(json.dumps(result))
    if args.tp > 1:
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)          # CUDA graphs that captured collectives are still alive: leave without tearing NCCL down


if __name__ == "__main__":
    main()

"""End-to-end decode harness: a random-init Llama-3-8B-shaped decoder whose linears are packed
mixed-FP4 layers, to report tokens/s and the share of a decode step spent in the mixed-FP4 GEMVs.

    python -m mixfp4_b200.llama_decode [--layers 32] [--batch 1] [--prompt 2048] [--tokens 32]

Architecture: hidden 4096, 32 query / 8 KV heads of 128, FFN 14336, RMSNorm, RoPE (theta 5e5),
vocab 128256, bf16 KV cache.  Weights are seeded synthetic tensors (no checkpoint is available
offline), quantized on the device layer by layer; the prompt is uniform random token ids.
Everything that is not a linear -- norms, RoPE, attention over the KV cache, SiLU, the bf16
embedding and output head -- runs as stock PyTorch operators: those are not part of the
mixed-FP4 path, they are here so that the linears run in their real data flow (grouped q/k/v and
gate/up launches, chained launches, batch rows = sequences).  The prompt is prefilled through the
tcgen05 GEMM path, the decode steps are captured in one CUDA graph per step shape.
"""

from __future__ import annotations

import argparse
import json

import torch
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
    def __init__(self, index: int, device, gen: torch.Generator):
        def packed(n, k, tag):
            gen.manual_seed(1000 * index + tag)
            return mx.quantize_packed(_student_t(n, k, gen, device))[0].to_kernel_layout()
        self.q, self.k, self.v = packed(HIDDEN, HIDDEN, 0), packed(KV_HEADS * HEAD_DIM, HIDDEN, 1), packed(KV_HEADS * HEAD_DIM, HIDDEN, 2)
        self.o = packed(HIDDEN, HIDDEN, 3)
        self.gate, self.up, self.down = packed(FFN, HIDDEN, 4), packed(FFN, HIDDEN, 5), packed(HIDDEN, FFN, 6)
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
    def __init__(self, layers: int, batch: int, max_len: int, device):
        self.device, self.batch, self.max_len = device, batch, max_len
        gen = torch.Generator(device=device)
        self.layers = [Layer(i, device, gen) for i in range(layers)]
        gen.manual_seed(99)
        self.embed = (torch.randn((VOCAB, HIDDEN), generator=gen, device=device) * 0.02).to(torch.bfloat16)
        self.head = (torch.randn((VOCAB, HIDDEN), generator=gen, device=device) * 0.02).to(torch.bfloat16)
        self.final_norm = torch.ones(HIDDEN, dtype=torch.bfloat16, device=device)
        self.k_cache = [torch.zeros((batch, KV_HEADS, max_len, HEAD_DIM), dtype=torch.bfloat16, device=device) for _ in self.layers]
        self.v_cache = [torch.zeros_like(c) for c in self.k_cache]
        inv = 1.0 / (ROPE_THETA ** (torch.arange(0, HEAD_DIM, 2, device=device).float() / HEAD_DIM))
        ang = torch.arange(max_len, device=device).float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.linears_only = False        # timing aid: skip everything but the linears

    def forward(self, tokens: torch.Tensor, pos: torch.Tensor, length: int) -> torch.Tensor:
        """tokens [B, T] at positions pos [T] (T = prompt length at prefill, 1 at decode); the
        cache holds `length` valid positions after this call.  Returns logits [B, vocab] of the
        last position."""
        b, t = tokens.shape
        h = self.embed[tokens]                                            # [B, T, hidden]
        cos, sin = self.cos[pos], self.sin[pos]
        for i, layer in enumerate(self.layers):
            x = h if self.linears_only else rms_norm(h, layer.norm1)
            q, k, v = mx.mixfp4_linear_grouped(x.reshape(b * t, HIDDEN), [layer.q, layer.k, layer.v], overlap_previous=True)
            if self.linears_only:
                attn = q
            else:
                q = rope(q.view(b, t, HEADS, HEAD_DIM), cos, sin).transpose(1, 2)
                k = rope(k.view(b, t, KV_HEADS, HEAD_DIM), cos, sin).transpose(1, 2)
                v = v.view(b, t, KV_HEADS, HEAD_DIM).transpose(1, 2)
                self.k_cache[i][:, :, pos] = k
                self.v_cache[i][:, :, pos] = v
                keys, vals = self.k_cache[i][:, :, :length], self.v_cache[i][:, :, :length]
                attn = F.scaled_dot_product_attention(q, keys, vals, is_causal=t > 1, enable_gqa=True)
                attn = attn.transpose(1, 2).reshape(b * t, HIDDEN)
            o = mx.mixfp4_linear(attn, layer.o, overlap_previous=True)
            if self.linears_only:
                x, h2 = o, h
            else:
                h2 = h + o.view(b, t, HIDDEN)
                x = rms_norm(h2, layer.norm2).reshape(b * t, HIDDEN)
            g, u = mx.mixfp4_linear_grouped(x, [layer.gate, layer.up], overlap_previous=True)
            act = g if self.linears_only else F.silu(g) * u
            d = mx.mixfp4_linear(act, layer.down, overlap_previous=True)
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
def run(layers: int = 32, batch: int = 1, prompt: int = 2048, tokens: int = 32, device=None) -> dict:
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    model = Decoder(layers, batch, prompt + tokens + 1, device)
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
    return {
        "layers": layers, "batch": batch, "prompt_tokens": prompt, "decode_steps_timed": tokens,
        "prefill_ms": round(prefill_ms, 2), "prefill_tokens_per_s": round(batch * prompt / prefill_ms * 1e3, 1),
        "decode_ms_per_step": round(full_ms, 4), "decode_tokens_per_s": round(batch / full_ms * 1e3, 1),
        "mixfp4_linears_ms_per_step": round(lin_ms, 4), "mixfp4_linear_time_fraction": round(lin_ms / full_ms, 3),
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=32)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    print(json.dumps(run(args.layers, args.batch, args.prompt, args.tokens)))


if __name__ == "__main__":
    main()

"""Model conversion (the reference's quantize_model_weights / apply_rotations walk,
project_quant/modeling.py:323-344, 604-639) and the packed checkpoint round trip."""

import io

import numpy as np
import pytest
import torch
from torch import nn

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import convert, synth

pytestmark = pytest.mark.gpu


class Block(nn.Module):
    def __init__(self, hidden, ffn):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, ffn, bias=False)
        self.up_proj = nn.Linear(hidden, ffn, bias=False)
        self.down_proj = nn.Linear(ffn, hidden, bias=True)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class Tiny(nn.Module):
    def __init__(self, hidden=256, ffn=384, vocab=100):
        super().__init__()
        self.layers = nn.ModuleList([Block(hidden, ffn) for _ in range(2)])
        self.lm_head = nn.Linear(hidden, vocab, bias=False)

    def forward(self, x):
        for layer in self.layers:
            x = x + layer(x)
        return self.lm_head(x)


def make_model(seed=0):
    torch.manual_seed(seed)
    model = Tiny().to(torch.bfloat16)
    for i, (_, lin) in enumerate(convert.named_linears(model)):
        lin.weight.data = synth.student_t_weight(*lin.weight.shape, seed=20 + i)
    return model.cuda()


def dense_twin(model, mode="oracle16"):
    """The reference's form of the same model: every linear's weight replaced by its
    dequantized tensor (computed by the oracle)."""
    twin = make_model()
    for (name, lin), (_, src) in zip(convert.named_linears(twin), convert.named_linears(model)):
        ref = oracle.quantize(src.weight.detach().float().cpu().numpy(), mode)
        bits = oracle.dequant(ref, "bf16").astype(np.int16)
        lin.weight.data = torch.from_numpy(bits).view(torch.bfloat16).reshape(lin.weight.shape).cuda()
    return twin


@pytest.mark.parametrize("mode", ["oracle16", "n8k64"])
def test_converted_model_matches_the_reference_form(mode):
    model = make_model()
    twin = dense_twin(model, mode)
    rows = convert.quantize_model_weights(model, mode)
    assert [r["module_name"] for r in rows] == [n for n, _ in convert.named_linears(twin)]
    assert isinstance(model.lm_head, nn.Linear)                       # heads stay dense
    assert all(isinstance(m, mx.MixFP4Linear) for l in model.layers for m in l.children())
    assert rows[0]["module_type"] == "gate_proj" and rows[0]["layer_idx"] == 0 and 0.0 < rows[0]["e0_ratio"] < 1.0
    for m in (1, 5, 200):                                             # GEMV and GEMM paths
        x = synth.activations(m, 256, seed=m).cuda()
        y, yt = model(x).float(), twin(x).float()
        assert (y - yt).norm() / yt.norm() <= 2e-2                    # bf16 activations between layers
    # layer by layer the packed linear is the dense linear on the dequantized weight
    x = synth.activations(7, 256, seed=3).cuda()
    got = model.layers[0].gate_proj(x, out_dtype=torch.float32)
    want = x.float() @ twin.layers[0].gate_proj.weight.float().T
    assert (got - want).norm() / want.norm() <= 1e-3


def test_high_precision_modes_leave_the_model_alone():
    model = make_model()
    assert convert.quantize_model_weights(model, "bf16") == []
    assert isinstance(model.layers[0].gate_proj, nn.Linear)


def test_checkpoint_round_trip_is_bit_exact():
    model = make_model()
    convert.quantize_model_weights(model, "oracle16", per_module_rotation={"layers.1.down_proj": "H128"})
    assert model.layers[1].down_proj.rotation == "H128" and model.layers[0].down_proj.rotation is None
    buf = io.BytesIO()
    torch.save(convert.packed_state(model), buf)
    state = torch.load(io.BytesIO(buf.getvalue()), map_location="cpu", weights_only=True)
    fresh = make_model(seed=1)                                        # dense architecture, other weights
    fresh.lm_head.weight.data.copy_(model.lm_head.weight.data)
    names = convert.load_packed(fresh, state)
    assert len(names) == 6
    for a, b in zip(model.modules(), fresh.modules()):
        if isinstance(a, mx.MixFP4Linear):
            assert torch.equal(a.codes, b.codes) and torch.equal(a.scales, b.scales)
            assert torch.equal(a.global_scale, b.global_scale) and torch.equal(a.lut, b.lut)
            assert a.rotation == b.rotation
            assert (a.bias is None) == (b.bias is None) and (a.bias is None or torch.equal(a.bias, b.bias))
    x = synth.activations(3, 256, seed=9).cuda()
    assert torch.equal(model(x), fresh(x))
    # the stored bytes are the canonical layout the oracle produces
    ref = oracle.quantize(make_model().layers[0].gate_proj.weight.detach().float().cpu().numpy())
    entry = state["layers"]["layers.0.gate_proj"]
    assert np.array_equal(entry["codes"].numpy(), ref.codes) and np.array_equal(entry["fmt"].numpy(), ref.fmt)
    with pytest.raises(ValueError):
        convert.load_packed(fresh, {"format": "other", "version": 1, "layers": {}})
    with pytest.raises(KeyError):
        convert.load_packed(Tiny(hidden=256, ffn=384).layers[0], state)


def test_decode_harness_runs_and_reports():
    """Two layers of the Llama-3-8B-shaped decoder: prefill through the GEMM path, graph-captured
    decode steps through the grouped GEMVs; the report is consistent."""
    from mixfp4_b200 import llama_decode
    r = llama_decode.run(layers=2, batch=2, prompt=48, tokens=3)
    assert r["decode_tokens_per_s"] > 0 and r["prefill_tokens_per_s"] > 0
    assert 0.0 < r["mixfp4_linear_time_fraction"] <= 1.0
    assert r["mixfp4_linears_ms_per_step"] <= r["decode_ms_per_step"]

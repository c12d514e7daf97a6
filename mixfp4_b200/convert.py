"""Model conversion and packed checkpoints.

The reference keeps a model's linears dense: `quantize_model_weights`
(project_quant/modeling.py:604-639) overwrites every `nn.Linear.weight` with its dequantized
tensor, `apply_rotations` (modeling.py:323-344) folds a K-side transform into the weight
beforehand and `ActivationHooks` (modeling.py:662-668) applies the matching transform to the
layer input.  Here the same walk replaces each linear by a `MixFP4Linear` that holds the packed
bytes (and rotates its input itself), and the packed bytes can be written to and read from a
checkpoint file, so a model is quantized once.

Checkpoint format (`torch.save` of plain tensors and python scalars, no code objects):
    {"format": "mixfp4_b200.packed", "version": 1, "layers": {module name: {
        "codes": u8 [n, kpad/2], "scales": u8 [n, kpad/16], "fmt": u8 [n, kpad/128],
        "global_scale": f32 [1], "n": int, "k": int, "rotation": str | None, "mode": str,
        "activation_mode": str | None, "bias": tensor | None}}}
The bytes are the canonical layout of include/mixfp4_b200.h (the one the parity tests hash);
the kernel layout and the decode tables are rebuilt at load time.
"""

from __future__ import annotations

import re
from typing import Any, Iterator

import torch
from torch import nn

from .linear import MixFP4Linear
from .quant import PackedWeight

FORMAT_NAME = "mixfp4_b200.packed"
FORMAT_VERSION = 1
LINEAR_TYPES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def named_linears(model: nn.Module) -> Iterator[tuple[str, nn.Linear]]:
    """Every nn.Linear except output heads (project_quant/modeling.py:65-68)."""
    for name, module in model.named_modules():
        if isinstance(module, nn.Linear) and not name.endswith("lm_head") and "head" not in name.rsplit(".", 1)[-1]:
            yield name, module


def module_type(name: str) -> str:
    suffix = name.rsplit(".", 1)[-1]
    return suffix if suffix in LINEAR_TYPES else "other_linear"


def layer_index(name: str) -> int | None:
    match = re.search(r"(?:^|\.)layers\.(\d+)(?:\.|$)", name)
    return int(match.group(1)) if match else None


def _set_submodule(model: nn.Module, name: str, new: nn.Module) -> None:
    parent = model
    parts = name.split(".")
    for part in parts[:-1]:
        parent = getattr(parent, part)
    setattr(parent, parts[-1], new)


@torch.no_grad()
def quantize_model_weights(model: nn.Module, weight_mode: str = "oracle16", *, rotation: str = "identity",
                           per_module_rotation: dict[str, str] | None = None, device=None,
                           activation_mode: str | None = None) -> list[dict[str, Any]]:
    """Replace every linear of ``model`` (heads excluded) by a packed MixFP4Linear, in place.

    weight_mode: a format region of `quant_mixfp4_granularity` ("oracle16", "n8k64", ...);
    "high_precision" / "fp16" / "bf16" leave the model untouched, as in the reference.
    rotation / per_module_rotation: name of a K-side transform ("H128", ...) folded into the
    weight before quantization; the layer then rotates its input with the same transform.
    activation_mode: format region of the activation fake-quantization each converted layer
    applies to its (rotated) input, as the reference's ActivationHooks do (modeling.py:640-705);
    None / "bf16" leaves the activations in bf16.
    Returns one row per converted layer (name, type, layer index, shape, share of E0M3 blocks,
    packed bytes)."""
    if weight_mode in {"high_precision", "fp16", "bf16"}:
        return []
    rows = []
    for name, linear in list(named_linears(model)):
        chosen = per_module_rotation.get(name, rotation) if per_module_rotation else rotation
        chosen = None if chosen in (None, "identity") else chosen
        layer = MixFP4Linear.from_linear(linear, rotation=chosen, mode=weight_mode, device=device,
                                         activation_mode=activation_mode)
        layer.weight_mode = weight_mode
        _set_submodule(model, name, layer)
        packed = layer.packed
        rows.append({
            "module_name": name, "module_type": module_type(name), "layer_idx": layer_index(name),
            "out_features": layer.out_features, "in_features": layer.in_features, "transform": chosen or "identity",
            "format_granularity": weight_mode,
            "e0_ratio": float(packed.format_ids().float().mean().item()),
            "packed_bytes": packed.nbytes(),
        })
    return rows


def packed_state(model: nn.Module) -> dict[str, Any]:
    """The checkpoint dictionary of every MixFP4Linear in ``model`` (canonical bytes, on the CPU)."""
    layers = {}
    for name, module in model.named_modules():
        if isinstance(module, MixFP4Linear):
            p = module.packed.to_canonical()
            layers[name] = {
                "codes": p.codes.cpu(), "scales": p.scales.cpu(), "fmt": p.fmt.cpu(),
                "global_scale": p.global_scale.cpu(), "n": p.n, "k": p.k, "rotation": p.rotation,
                "mode": getattr(module, "weight_mode", "oracle16"),
                "activation_mode": module.activation_mode,
                "bias": None if module.bias is None else module.bias.detach().cpu(),
            }
    return {"format": FORMAT_NAME, "version": FORMAT_VERSION, "layers": layers}


def save_packed(model: nn.Module, path: str) -> None:
    torch.save(packed_state(model), path)


@torch.no_grad()
def load_packed(model: nn.Module, path_or_state, *, device=None, strict: bool = True) -> list[str]:
    """Install the packed layers of a checkpoint into ``model`` (whose corresponding modules may
    still be dense nn.Linear, e.g. a freshly constructed architecture).  Returns the names that
    were installed; with strict=True a checkpoint layer without a module of that name, or a
    shape mismatch, raises."""
    state = torch.load(path_or_state, map_location="cpu", weights_only=True) if isinstance(path_or_state, str) else path_or_state
    if state.get("format") != FORMAT_NAME or state.get("version") != FORMAT_VERSION:
        raise ValueError("not a mixfp4_b200 packed checkpoint of a known version")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    modules = dict(model.named_modules())
    done = []
    for name, entry in state["layers"].items():
        old = modules.get(name)
        if old is None:
            if strict:
                raise KeyError(f"checkpoint layer {name!r} has no module in the model")
            continue
        shape = (old.out_features, old.in_features) if hasattr(old, "out_features") else None
        if strict and shape is not None and shape != (entry["n"], entry["k"]):
            raise ValueError(f"{name}: checkpoint holds {entry['n']}x{entry['k']}, the model {shape[0]}x{shape[1]}")
        packed = PackedWeight(entry["codes"].to(device), entry["scales"].to(device), entry["fmt"].to(device),
                              entry["global_scale"].to(device), entry["n"], entry["k"], entry["rotation"])
        bias = None if entry["bias"] is None else entry["bias"].to(device)
        layer = MixFP4Linear(packed, bias, entry.get("activation_mode"))
        layer.weight_mode = entry.get("mode", "oracle16")
        _set_submodule(model, name, layer)
        done.append(name)
    return done

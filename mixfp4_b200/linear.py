"""Mixed-FP4 dequant-linear: the layer that replaces ``nn.Linear`` on a weight the
reference would have overwritten with its dequantized tensor
(project_quant/modeling.py:603-639 quantize_model_weights, :629 the weight swap, and the
activation rotation pre-hook :662-668).

``mixfp4_linear`` picks the kernel by shape alone: M <= 16 runs the HBM-bound GEMV,
larger M the tcgen05 GEMM.  There is one implementation per shape class and no
fallback.
"""

from __future__ import annotations

import torch
from torch import nn

from . import _native as nat
from . import rotation as _rotation
from .quant import (HIGH_PRECISION_MODES, PackedWeight, _MODE_CODE, fake_quantize_activations, normalize_region,
                    quantize_packed, region_shape)

GEMV_MAX_M = 16
_workspaces: dict[tuple, torch.Tensor] = {}
_status_words: dict[str, torch.Tensor] = {}


def _workspace(device, nbytes: int) -> torch.Tensor | None:
    if nbytes <= 0:
        return None
    key = (str(device), torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _status_word(device) -> torch.Tensor:
    key = str(device)
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


def gemm_status(device=None) -> int:
    """Value of the GEMM's device-side status word (0 = every bounded wait completed).
    Synchronises the device."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(_status_word(device).item())


def decode_status(device=None) -> int:
    """Status word of the decode kernels on `device` (0 = every weight chunk arrived within the
    wait limit).  Synchronises the current stream."""
    import ctypes
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    value = ctypes.c_int(0)
    with torch.cuda.device(device):
        rc = nat.lib().mixfp4_check_status(None, ctypes.byref(value), nat.stream_ptr(device))
    if rc not in (nat.OK, nat.E_DEVICE_WAIT):
        nat.check("mixfp4_check_status", rc)
    return int(value.value)


def mixfp4_linear(x: torch.Tensor, packed: PackedWeight, *, bias: torch.Tensor | None = None,
                  rotate: bool | None = None, out_dtype: torch.dtype | None = None,
                  overlap_previous: bool = False, activation_mode: str | None = None) -> torch.Tensor:
    """y = x @ W^T (+ bias) with W packed; x bf16 [..., K] on the GPU.

    activation_mode: None / "bf16" keeps x as it is (W4A16).  A format region ("oracle16",
    "all_e2m1", "m8k64", ...) makes this the reference's W4A4 forward (ActivationHooks._hook,
    project_quant/modeling.py:662-705): x is rotated with every stage rounded to bf16 (what the
    hook's apply_transform computes on a bf16 tensor), fake-quantized with its own global scale,
    and the dequantized bf16 tensor goes into the same kernels.  Prefill shapes with a per-block
    or whole-tensor mode run as one ``mixfp4_gemm_a4`` call.

    rotate: apply the weight's folded K-transform to x first (default: yes when the packed
    weight records one).  For H128 at prefill shapes ``mixfp4_gemm`` runs the rotation as a pass of
    its own into the workspace and starts the GEMM kernel under that pass's tail; the GEMV path
    and other block sizes call the FWHT kernel here (fp32 stages, one rounding, in both cases).
    out_dtype: torch.float32 or torch.bfloat16 (default: x.dtype).
    overlap_previous: launch the decode kernel as a programmatic dependent of the previous
    kernel in the stream (its weight prefetch overlaps that kernel's tail).  Only valid when
    the previous kernel does not write this layer's packed weight.
    """
    nat.require_cuda(x, "x")
    if x.dtype != torch.bfloat16:
        raise TypeError("x must be bfloat16")
    if x.shape[-1] != packed.k:
        raise ValueError(f"x has K={x.shape[-1]}, the packed weight K={packed.k}")
    out_dtype = x.dtype if out_dtype is None else out_dtype
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("out_dtype must be float32 or bfloat16")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, packed.k)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    m = x2.shape[0]
    spec = None
    if rotate is None:
        rotate = packed.rotation is not None
    if rotate:
        if packed.rotation is None:
            raise ValueError("rotate=True but the packed weight records no rotation")
        spec = _rotation.get_transform(packed.rotation)
        if spec.block_size is None:
            spec = None
    y = torch.empty((m, packed.n), dtype=out_dtype, device=x.device)
    if m == 0:
        return y.reshape(*lead, packed.n)
    lib = nat.lib()
    act = None
    if activation_mode is not None:
        act = normalize_region(activation_mode, "activation_a")
        act = None if act in HIGH_PRECISION_MODES else act
    if act is not None:
        fusable = (m > GEMV_MAX_M and region_shape(act, "activation_a") is None
                   and (spec is None or (spec.block_size == 128 and spec.seed is None)))
        if fusable:
            nbytes = lib.mixfp4_gemm_workspace_bytes(m, packed.n, packed.k)
            ws = _workspace(x.device, nbytes)
            with torch.cuda.device(x.device):
                st = lib.mixfp4_gemm_a4(x2.data_ptr(), m, x2.stride(0), packed.codes.data_ptr(), packed.scales.data_ptr(),
                                        nat.ptr(packed.fmt), packed.global_scale.data_ptr(), packed.n, packed.k,
                                        packed.layout_code, nat.ptr(packed.lut), 128 if spec is not None else 0,
                                        _MODE_CODE[act], y.data_ptr(), nat.DTYPE_CODE[out_dtype], y.stride(0),
                                        nat.ptr(ws), nbytes, _status_word(x.device).data_ptr(), 0,
                                        nat.stream_ptr(x.device))
            nat.check("mixfp4_gemm_a4", st)
            if bias is not None:
                y += bias.to(y.dtype)
            return y.reshape(*lead, packed.n)
        if spec is not None:
            x2 = _rotation.apply_transform(x2, spec, rounding="reference")
            spec = None
        x2 = fake_quantize_activations(x2, act)
    with torch.cuda.device(x.device):
        stream = nat.stream_ptr(x.device)
        if m <= GEMV_MAX_M:
            if spec is not None:
                x2 = _rotation.apply_transform(x2, spec, rounding="once")
            st = lib.mixfp4_gemv(x2.data_ptr(), m, x2.stride(0), packed.codes.data_ptr(), packed.scales.data_ptr(),
                                 nat.ptr(packed.fmt), packed.global_scale.data_ptr(), packed.n, packed.k,
                                 packed.layout_code, nat.ptr(packed.lut), y.data_ptr(), nat.DTYPE_CODE[out_dtype],
                                 y.stride(0), nat.gemv_flags(overlap_previous, packed.lut), stream)
            nat.check("mixfp4_gemv", st)
        else:
            fused = 0
            if spec is not None:
                if spec.block_size == 128 and spec.seed is None:
                    fused = 128
                else:
                    x2 = _rotation.apply_transform(x2, spec, rounding="once")
            nbytes = lib.mixfp4_gemm_workspace_bytes(m, packed.n, packed.k)
            ws = _workspace(x.device, nbytes)
            st = lib.mixfp4_gemm(x2.data_ptr(), m, x2.stride(0), packed.codes.data_ptr(), packed.scales.data_ptr(),
                                 nat.ptr(packed.fmt), packed.global_scale.data_ptr(), packed.n, packed.k,
                                 packed.layout_code, nat.ptr(packed.lut), fused, y.data_ptr(),
                                 nat.DTYPE_CODE[out_dtype], y.stride(0), nat.ptr(ws), nbytes,
                                 _status_word(x.device).data_ptr(), 0, stream)
            nat.check("mixfp4_gemm", st)
    if bias is not None:
        y += bias.to(y.dtype)
    return y.reshape(*lead, packed.n)


def mixfp4_linear_grouped(x: torch.Tensor, packs: list[PackedWeight], *, out_dtype: torch.dtype | None = None,
                          overlap_previous: bool = False) -> list[torch.Tensor]:
    """[x @ W_i^T for W_i in packs] for weights that take the same x (q/k/v, gate/up).

    Decode shapes (at most 16 rows of x), up to three kernel- or stream-layout weights without a folded
    rotation: one launch (``mixfp4_gemv_grouped``).  Anything else: one ``mixfp4_linear`` per
    weight, same results.
    """
    if not packs:
        return []
    k = packs[0].k
    lead = x.shape[:-1]
    m = x.numel() // max(1, x.shape[-1])
    grouped = (1 <= m <= 16 and 1 <= len(packs) <= 3 and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] == k
               and packs[0].layout in ("kernel", "stream")
               and all(p.k == k and p.layout == packs[0].layout and p.rotation is None for p in packs))
    if grouped:
        out_dtype = x.dtype if out_dtype is None else out_dtype
        if out_dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("out_dtype must be float32 or bfloat16")
        x2 = x.reshape(-1, k)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        ys = [torch.empty((m, p.n), dtype=out_dtype, device=x.device) for p in packs]
        segs = (nat.GemvSegment * len(packs))()
        for seg, p, y in zip(segs, packs, ys):
            seg.codes, seg.scales, seg.global_scale = p.codes.data_ptr(), nat.ptr(p.scales), p.global_scale.data_ptr()
            seg.lut, seg.y, seg.ldy, seg.n = nat.ptr(p.lut), y.data_ptr(), y.stride(0), p.n
        with torch.cuda.device(x.device):
            st = nat.lib().mixfp4_gemv_grouped(x2.data_ptr(), m, x2.stride(0), k, segs, len(packs),
                                               packs[0].layout_code, nat.DTYPE_CODE[out_dtype],
                                               nat.gemv_flags(overlap_previous, *[p.lut for p in packs]),
                                               nat.stream_ptr(x.device))
        if st != nat.E_SHAPE:
            nat.check("mixfp4_gemv_grouped", st)
            return [y.reshape(*lead, p.n) for y, p in zip(ys, packs)]
    return [mixfp4_linear(x, p, out_dtype=out_dtype, overlap_previous=overlap_previous and i == 0)
            for i, p in enumerate(packs)]


class MixFP4Linear(nn.Module):
    """nn.Linear whose weight lives in the packed mixed-FP4 layout."""

    def __init__(self, packed: PackedWeight, bias: torch.Tensor | None = None, activation_mode: str | None = None):
        super().__init__()
        self.in_features, self.out_features = packed.k, packed.n
        self.activation_mode = activation_mode      # None: W4A16; a format region: the reference's W4A4 forward
        packed = packed.to_stream_layout()          # the layers keep the layout the kernels stream fastest
        self.rotation = packed.rotation
        self.register_buffer("codes", packed.codes)
        self.register_buffer("scales", packed.scales)
        self.register_buffer("lut", packed.lut)
        self.register_buffer("global_scale", packed.global_scale)
        self.bias = None if bias is None else nn.Parameter(bias.detach().clone(), requires_grad=False)

    @property
    def packed(self) -> PackedWeight:
        return PackedWeight(self.codes, self.scales, None, self.global_scale, self.out_features,
                            self.in_features, self.rotation, "stream", self.lut)

    @classmethod
    @torch.no_grad()
    def from_linear(cls, linear: nn.Linear, *, rotation: str | None = None, mode: str = "oracle16",
                    device=None, activation_mode: str | None = None) -> "MixFP4Linear":
        """Quantize ``linear.weight`` (optionally rotated along K first, as the reference's
        apply_rotations does offline, modeling.py:323-344) and wrap it."""
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        w = linear.weight.detach().to(device)
        if w.dtype not in nat.DTYPE_CODE:
            w = w.to(torch.bfloat16)
        if rotation is not None:
            w = _rotation.apply_transform(w, rotation)
        packed, _, _ = quantize_packed(w, mode=mode, rotation=rotation)
        bias = None if linear.bias is None else linear.bias.detach().to(device)
        return cls(packed, bias, activation_mode)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype | None = None,
                overlap_previous: bool = False) -> torch.Tensor:
        return mixfp4_linear(x, self.packed, bias=self.bias, out_dtype=out_dtype, overlap_previous=overlap_previous,
                             activation_mode=self.activation_mode)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, rotation={self.rotation}, "
                f"activation_mode={self.activation_mode}")

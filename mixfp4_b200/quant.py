"""Python surface of the block quantizer: the reference's ``quant_mixfp4_granularity``
keyword API plus the packed weight type the reference does not have.

Reference interface mirrored here (paths inside the reference project):
  project_quant/core.py:53-67     quant_mixfp4_granularity signature, defaults, return types
  project_quant/core.py:18-29     GranularityResult fields
  project_quant/candidates.py:46-58  validate_layout error types and messages
  project_quant/region.py:22-39   normalize_region aliases
All arithmetic runs in the CUDA kernels behind the C ABI (mixfp4_amax +
mixfp4_quantize); a host tensor is copied to the current CUDA device and the result is
copied back.  Nothing here computes on the CPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from . import _native as nat
from . import rotation as _rotation

SCALE_GROUP_SIZE = 16
E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E0M3_LEVELS = (0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0)
TAIL_POLICY = (
    "right_zero_pad_only_the_final_partial_K16_scale_block_then_unpad; "
    "partial_N_or_M_and_K_format_regions_use_only_real_K16_blocks"
)

_MODE_CODE = {"oracle16": nat.MODE_ORACLE16, "all_e2m1": nat.MODE_ALL_E2M1, "all_e0m3": nat.MODE_ALL_E0M3}
# coarse format regions (project_quant/region.py:42-70): name -> (rows, K16 blocks) of a region
# (rows, 0) stands for "layer": one format for the whole tensor
_WEIGHT_REGIONS = {"k32_row": (1, 2), "k64_row": (1, 4), "n2k64": (2, 4), "n4k64": (4, 4), "n8k64": (8, 4),
                   "n16k64": (16, 4), "n32k64": (32, 4), "n64k64": (64, 4), "n8k16": (8, 1), "layer": (1, 0)}
_ACTIVATION_REGIONS = {"k64_row": (1, 4), "m4k64": (4, 4), "m8k64": (8, 4), "m16k64": (16, 4), "m32k64": (32, 4),
                       "m16k16": (16, 1), "layer": (1, 0)}


def region_shape(mode: str, operand_role: str) -> tuple[int, int] | None:
    """(rows, K16 blocks) of a coarse format region, None for the per-block / whole-tensor modes."""
    if mode in _MODE_CODE:
        return None
    table = _WEIGHT_REGIONS if operand_role == "weight_b" else _ACTIVATION_REGIONS
    if mode in table:
        return table[mode]
    raise ValueError(f"format_region={mode!r} is invalid for {operand_role}")


def padded_k(k: int) -> int:
    return (k + 127) // 128 * 128


def packed_nbytes(n: int, k: int) -> int:
    """Algorithmic bytes of a packed [n, k] weight: 4-bit codes + one E4M3 scale and one
    format bit per 16 elements (+ the 4-byte tensor scale)."""
    return n * k // 2 + n * k // 16 + n * k // 128 + 4


@dataclass
class PackedWeight:
    """A quantized [n, k] matrix in the packed layout of include/mixfp4_b200.h."""

    codes: torch.Tensor          # uint8 [n, kpad/2]
    scales: torch.Tensor         # uint8 [n, kpad/16]  E4M3 bytes
    fmt: torch.Tensor            # uint8 [n, kpad/128] format bits (1 = E0M3)
    global_scale: torch.Tensor   # float32 [1]
    n: int
    k: int
    rotation: str | None = None  # transform folded into the weight along K before quantization
    # "canonical" (parity-hashed), "kernel" (bit-permuted code words, format bit in the scale byte) or
    # "stream" (1152-byte chunks of 16 rows x 128 K: `codes` is the flat chunk buffer, `scales` is empty)
    layout: str = "canonical"
    lut: torch.Tensor | None = None   # optional decode table (uint8 [4096]) from mixfp4_decode_table

    @property
    def kpad(self) -> int:
        return padded_k(self.k)

    @property
    def groups(self) -> int:
        return (self.k + 15) // 16

    @property
    def device(self) -> torch.device:
        return self.codes.device

    def nbytes(self) -> int:
        return packed_nbytes(self.n, self.k)

    @property
    def layout_code(self) -> int:
        return {"canonical": nat.LAYOUT_CANONICAL, "kernel": nat.LAYOUT_KERNEL, "stream": nat.LAYOUT_STREAM}[self.layout]

    def format_ids(self) -> torch.Tensor:
        """uint8 [n, ceil(k/16)], 1 = E0M3 (GranularityResult.format_ids of the reference)."""
        if self.layout == "stream":
            return self.to_canonical().format_ids()
        if self.layout == "kernel":
            return (self.scales[:, : self.groups] >> 7).contiguous()
        shifts = torch.arange(8, device=self.fmt.device, dtype=torch.uint8)
        bits = (self.fmt.unsqueeze(-1) >> shifts) & 1
        return bits.reshape(self.n, -1)[:, : self.groups].contiguous()

    def selected_scales(self) -> torch.Tensor:
        """float32 [n, ceil(k/16)] decoded block scales."""
        if self.layout == "stream":
            return self.to_canonical().selected_scales()
        return (self.scales[:, : self.groups] & 0x7F).contiguous().view(torch.float8_e4m3fn).float()

    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return dequantize(self, dtype)

    def to(self, device) -> "PackedWeight":
        mv = lambda t: None if t is None else t.to(device)
        return PackedWeight(mv(self.codes), mv(self.scales), mv(self.fmt), mv(self.global_scale), self.n, self.k,
                            self.rotation, self.layout, mv(self.lut))

    def state_dict(self) -> dict:
        return {"codes": self.codes, "scales": self.scales, "fmt": self.fmt, "global_scale": self.global_scale,
                "n": self.n, "k": self.k, "rotation": self.rotation, "layout": self.layout}

    @staticmethod
    def from_state_dict(state: dict) -> "PackedWeight":
        return PackedWeight(state["codes"], state["scales"], state["fmt"], state["global_scale"],
                            int(state["n"]), int(state["k"]), state.get("rotation"), state.get("layout", "canonical"))

    def with_decode_table(self) -> "PackedWeight":
        """Attach the (format, scale) -> bf16 magnitudes table so that the linear kernels copy it
        instead of rebuilding it in every launch: 4 KB, followed for the stream layout by the eightfold
        copy the decode kernel keeps in shared memory (36 KB in all, taken with one bulk copy)."""
        wide = self.layout == "stream"
        if self.lut is None or (wide and self.lut.numel() < nat.WIDE_TABLE_BYTES):
            lut = torch.empty(nat.WIDE_TABLE_BYTES if wide else 4096, dtype=torch.uint8, device=self.device)
            fn = nat.lib().mixfp4_decode_table_wide if wide else nat.lib().mixfp4_decode_table
            with torch.cuda.device(self.device):
                st = fn(self.global_scale.data_ptr(), lut.data_ptr(), nat.stream_ptr(self.device))
            nat.check("mixfp4_decode_table", st)
            self.lut = lut
        return self

    def _repack(self, to: str) -> "PackedWeight":
        if self.layout == to:
            return self
        if to == "stream":
            src = self if self.layout == "canonical" else self._repack("canonical")
            lib = nat.lib()
            chunks = torch.empty(lib.mixfp4_stream_bytes(self.n, self.k), dtype=torch.uint8, device=self.device)
            with torch.cuda.device(self.device):
                st = lib.mixfp4_repack_stream(src.codes.data_ptr(), src.scales.data_ptr(), src.fmt.data_ptr(), self.n,
                                              self.k, chunks.data_ptr(), nat.stream_ptr(self.device))
            nat.check("mixfp4_repack_stream", st)
            empty = torch.empty(0, dtype=torch.uint8, device=self.device)
            return PackedWeight(chunks, empty, None, self.global_scale, self.n, self.k, self.rotation, "stream", self.lut)
        if self.layout == "stream":
            codes = torch.empty((self.n, self.kpad // 2), dtype=torch.uint8, device=self.device)
            scales = torch.empty((self.n, self.kpad // 16), dtype=torch.uint8, device=self.device)
            fmt = torch.empty((self.n, self.kpad // 128), dtype=torch.uint8, device=self.device)
            with torch.cuda.device(self.device):
                st = nat.lib().mixfp4_repack_from_stream(self.codes.data_ptr(), self.n, self.k, codes.data_ptr(),
                                                         scales.data_ptr(), fmt.data_ptr(), nat.stream_ptr(self.device))
            nat.check("mixfp4_repack_from_stream", st)
            canon = PackedWeight(codes, scales, fmt, self.global_scale, self.n, self.k, self.rotation, "canonical", self.lut)
            return canon if to == "canonical" else canon._repack(to)
        codes, scales = torch.empty_like(self.codes), torch.empty_like(self.scales)
        fmt = None if to == "kernel" else torch.empty((self.n, self.kpad // 128), dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            st = nat.lib().mixfp4_repack(self.codes.data_ptr(), self.scales.data_ptr(), nat.ptr(self.fmt), self.n, self.k,
                                         nat.LAYOUT_KERNEL if to == "kernel" else nat.LAYOUT_CANONICAL,
                                         codes.data_ptr(), scales.data_ptr(), nat.ptr(fmt), nat.stream_ptr(self.device))
        nat.check("mixfp4_repack", st)
        return PackedWeight(codes, scales, fmt, self.global_scale, self.n, self.k, self.rotation, to, self.lut)

    def to_kernel_layout(self) -> "PackedWeight":
        """Bit-permuted copy for the GEMV/GEMM kernels (signs regrouped inside each 32-bit code
        word, format bit folded into bit 7 of the scale byte; no format array), with its table."""
        return self._repack("kernel").with_decode_table()

    def to_stream_layout(self) -> "PackedWeight":
        """Copy in the stream layout (one contiguous 1152-byte chunk per 16 rows x 128 K elements:
        what the decode kernels stream with one bulk copy per step), with its decode table."""
        return self._repack("stream").with_decode_table()

    def to_canonical(self) -> "PackedWeight":
        return self._repack("canonical")

    def row_shard(self, start: int, stop: int) -> "PackedWeight":
        """Rows [start, stop) -- a column-parallel (split N) shard; shares the tensor scale."""
        if self.layout == "stream":
            return self.to_canonical().row_shard(start, stop)._repack("stream")
        fmt = None if self.fmt is None else self.fmt[start:stop].contiguous()
        return PackedWeight(self.codes[start:stop].contiguous(), self.scales[start:stop].contiguous(), fmt,
                            self.global_scale, stop - start, self.k, self.rotation, self.layout, self.lut)

    def k_shard(self, start: int, stop: int) -> "PackedWeight":
        """Columns [start, stop) along K (multiples of 128) -- a row-parallel (split K) shard."""
        if start % 128 or (stop % 128 and stop != self.k):
            raise ValueError("K shards must start and end on multiples of 128")
        if self.layout == "stream":
            return self.to_canonical().k_shard(start, stop)._repack("stream")
        pstop = padded_k(stop)
        fmt = None if self.fmt is None else self.fmt[:, start // 128: pstop // 128].contiguous()
        return PackedWeight(self.codes[:, start // 2: pstop // 2].contiguous(),
                            self.scales[:, start // 16: pstop // 16].contiguous(), fmt,
                            self.global_scale, self.n, stop - start, self.rotation, self.layout, self.lut)


@dataclass
class GranularityResult:
    """Same fields as the reference's GranularityResult (project_quant/core.py:18-29),
    plus ``packed``."""

    dequant: torch.Tensor
    format_ids: torch.Tensor
    oracle_format_ids: torch.Tensor
    selected_scales: torch.Tensor
    selected_scale_expansion_ids: torch.Tensor
    e2_scales: torch.Tensor
    e0_scales: torch.Tensor
    e2_errors: torch.Tensor
    e0_errors: torch.Tensor
    summary: dict[str, Any]
    regions: list[dict[str, Any]] = field(default_factory=list)
    packed: PackedWeight | None = None


def normalize_region(mode: str, operand_role: str) -> str:
    value = str(mode).lower().replace("-", "_")
    for prefix in ("mixfp4_", "nvfp4_mixfp4_"):
        if value.startswith(prefix):
            value = value[len(prefix):]
    aliases = {"nvfp4": "all_e2m1", "all_e2": "all_e2m1", "e2": "all_e2m1", "all_e0": "all_e0m3",
               "e0": "all_e0m3", "oracle16_a": "oracle16", "k64_row_a": "k64_row"}
    return aliases.get(value, value)


def validate_layout(x: torch.Tensor, *, scale_group_size: int, operand_role: str) -> None:
    if not torch.is_floating_point(x):
        raise TypeError("x must be floating point")
    if x.ndim < 2:
        raise ValueError("x must preserve a row dimension and a final K dimension")
    if operand_role == "weight_b" and x.ndim != 2:
        raise ValueError("weight_b requires the exact [N,K] matrix layout")
    if operand_role not in {"weight_b", "activation_a"}:
        raise ValueError("operand_role must be 'weight_b' or 'activation_a'")
    if scale_group_size != SCALE_GROUP_SIZE:
        raise ValueError("the primary MixFP4 study fixes scale_group_size=16")
    if x.shape[-1] <= 0:
        raise ValueError("K must be positive")


def tensor_amax(x2: torch.Tensor) -> torch.Tensor:
    """max |x| of a 2-D CUDA tensor as a float32 [1] device tensor (no host sync)."""
    out = torch.empty(1, dtype=torch.float32, device=x2.device)
    with torch.cuda.device(x2.device):
        st = nat.lib().mixfp4_amax(x2.data_ptr(), nat.DTYPE_CODE[x2.dtype], x2.shape[0], x2.shape[1],
                                   x2.stride(0), out.data_ptr(), nat.stream_ptr(x2.device))
    nat.check("mixfp4_amax", st)
    return out


def _as_rows(x: torch.Tensor) -> torch.Tensor:
    if x.dtype not in nat.DTYPE_CODE:
        raise TypeError(f"unsupported dtype {x.dtype}; use bfloat16, float16 or float32")
    nat.require_cuda(x, "x")
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


def quantize_packed(x: torch.Tensor, *, mode: str = "oracle16", amax: torch.Tensor | None = None,
                    want_dequant: bool = False, want_stats: bool = False, rotation: str | None = None,
                    region: tuple[int, int] | None = None):
    """Quantize a CUDA tensor [..., K] (leading dims fold into rows) into a PackedWeight.

    amax: optional float32 [1] device tensor holding max|x| of the WHOLE tensor this is a
    shard of (see mixfp4_amax); default: this tensor's own.
    region: (rows, K16 blocks) of a coarse format region (see region_shape): the errors of both
    candidates are computed first, one format is chosen per region, then the tensor is
    quantized with those formats.
    Returns (packed, dequant_or_None, stats_or_None); stats = dict of per-block float32
    [rows, G] tensors e2_errors, e0_errors, e2_scales, e0_scales.
    """
    if region is None:
        region = _WEIGHT_REGIONS.get(mode) or _ACTIVATION_REGIONS.get(mode)
    if region is None and mode not in _MODE_CODE:
        raise ValueError(f"unsupported mode {mode!r}")
    x2 = _as_rows(x)
    rows, k = x2.shape
    kp = padded_k(k)
    groups = (k + 15) // 16
    dev = x2.device
    if amax is None:
        amax = tensor_amax(x2)
    codes = torch.empty((rows, kp // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((rows, kp // 16), dtype=torch.uint8, device=dev)
    fmt = torch.empty((rows, kp // 128), dtype=torch.uint8, device=dev)
    gs = torch.empty(1, dtype=torch.float32, device=dev)
    stats = None
    if want_stats:
        stats = {name: torch.empty((rows, groups), dtype=torch.float32, device=dev)
                 for name in ("e2_errors", "e0_errors", "e2_scales", "e0_scales")}
    dq = torch.empty((rows, k), dtype=x2.dtype, device=dev) if want_dequant else None
    mode_code = _MODE_CODE[mode] if region is None else nat.MODE_GIVEN
    if region is not None:
        if region[1] > 0 and region[0] > 1 and -(-groups // region[1]) == 1:
            raise NotImplementedError("coarse regions over several rows need more than one region along K")
        e2e = stats["e2_errors"] if stats else torch.empty((rows, groups), dtype=torch.float32, device=dev)
        e0e = stats["e0_errors"] if stats else torch.empty((rows, groups), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            st = nat.lib().mixfp4_quantize(
                x2.data_ptr(), nat.DTYPE_CODE[x2.dtype], rows, k, x2.stride(0), nat.MODE_ORACLE16, amax.data_ptr(),
                codes.data_ptr(), scales.data_ptr(), fmt.data_ptr(), gs.data_ptr(), e2e.data_ptr(), e0e.data_ptr(),
                None, None, None, k, nat.stream_ptr(dev))
            nat.check("mixfp4_quantize", st)
            if region[1] == 0:          # "layer": both error sums of the whole tensor, one decision
                sums = torch.empty(2, dtype=torch.float64, device=dev)
                st = nat.lib().mixfp4_select_layer(e2e.data_ptr(), e0e.data_ptr(), rows, k, sums.data_ptr(),
                                                   fmt.data_ptr(), nat.stream_ptr(dev))
                nat.check("mixfp4_select_layer", st)
            else:
                st = nat.lib().mixfp4_select_regions(e2e.data_ptr(), e0e.data_ptr(), rows, k, region[0], region[1],
                                                     fmt.data_ptr(), nat.stream_ptr(dev))
                nat.check("mixfp4_select_regions", st)
    with torch.cuda.device(dev):
        st = nat.lib().mixfp4_quantize(
            x2.data_ptr(), nat.DTYPE_CODE[x2.dtype], rows, k, x2.stride(0), mode_code, amax.data_ptr(),
            codes.data_ptr(), scales.data_ptr(), fmt.data_ptr(), gs.data_ptr(),
            nat.ptr(stats["e2_errors"]) if stats else None, nat.ptr(stats["e0_errors"]) if stats else None,
            nat.ptr(stats["e2_scales"]) if stats else None, nat.ptr(stats["e0_scales"]) if stats else None,
            nat.ptr(dq), k, nat.stream_ptr(dev))
    nat.check("mixfp4_quantize", st)
    return PackedWeight(codes, scales, fmt, gs, rows, k, rotation), dq, stats


def _codebook(x: torch.Tensor, e0m3: bool) -> torch.Tensor:
    if not torch.is_floating_point(x):
        raise TypeError("x must be floating point")
    host_input = not x.is_cuda
    xf = x.detach().to(torch.float32)
    xf = (xf.cuda() if host_input else xf).contiguous()
    out = torch.empty_like(xf)
    if xf.numel():
        with torch.cuda.device(xf.device):
            st = nat.lib().mixfp4_round_codebook(xf.data_ptr(), out.data_ptr(), xf.numel(), int(e0m3),
                                                 nat.stream_ptr(xf.device))
        nat.check("mixfp4_round_codebook", st)
    out = out.to(x.dtype)
    return out.to(x.device) if host_input else out


@torch.no_grad()
def quantize_e2m1(x: torch.Tensor) -> torch.Tensor:
    """E2M1 round-to-nearest of every element, ties away from zero on the private mantissa, saturated
    to +-6 (project_quant/codebook.py:12-25); computed by the CUDA kernel the quantizer shares its
    rounding with."""
    return _codebook(x, False)


@torch.no_grad()
def quantize_e0m3(x: torch.Tensor) -> torch.Tensor:
    """Project E0M3: sign-magnitude integers 0, +-1 ... +-7, round half even
    (project_quant/codebook.py:41-43)."""
    return _codebook(x, True)


@dataclass
class CandidateBlocks:
    """Both independently scaled K16 candidates of a tensor; fields as
    project_quant/candidates.py:22-43 (codes are level values in float32, -0.0 where a negative
    element rounds to zero; everything [rows, groups(, 16)] float32 unless noted)."""

    original_shape: tuple[int, ...]
    source_dtype: torch.dtype
    operand_role: str
    rows: int
    k: int
    groups: int
    padded_k: int
    tail_padding: int
    grouped_original: torch.Tensor
    e2_dequant: torch.Tensor
    e0_dequant: torch.Tensor
    e2_codes: torch.Tensor
    e0_codes: torch.Tensor
    e2_scales: torch.Tensor
    e0_scales: torch.Tensor
    e2_errors: torch.Tensor
    e0_errors: torch.Tensor
    e2_scale_expansion_ids: torch.Tensor    # uint8, all zero under the standard scale rule
    e0_scale_expansion_ids: torch.Tensor
    global_scale: torch.Tensor              # 0-dim float32
    scale_rule: str


def _level_values(codes: torch.Tensor, groups: int, levels: tuple[float, ...]) -> torch.Tensor:
    """Packed nibbles [rows, kpad/2] -> signed level values float32 [rows, groups, 16]."""
    rows = codes.shape[0]
    nib = torch.stack((codes & 15, codes >> 4), dim=-1).reshape(rows, -1)[:, : groups * 16].long()
    mag = torch.tensor(levels, dtype=torch.float32, device=codes.device)[nib & 7]
    return torch.where((nib & 8) != 0, -mag, mag).reshape(rows, groups, 16)


@torch.no_grad()
def build_candidates(x: torch.Tensor, *, scale_group_size: int = SCALE_GROUP_SIZE, operand_role: str = "weight_b",
                     scale_rule: str = "standard") -> CandidateBlocks:
    """The reference's ``build_candidates`` (project_quant/candidates.py:62-106): the tensor up-cast
    to float32, right-zero-padded to whole K16 blocks, and for each block the E2M1 and the E0M3
    candidate with its own E4M3 scale -- level values, dequantized values, scales and squared errors.
    Two launches of the CUDA quantizer (one per forced format) on the float32 tensor produce every
    field; the nibble codes are expanded to level values on the device.  A host tensor is copied to
    the current CUDA device and the fields are copied back."""
    validate_layout(x, scale_group_size=scale_group_size, operand_role=operand_role)
    if scale_rule == "four_over_six":
        raise NotImplementedError("scale_rule='four_over_six' needs the FourOverSix upstream for its E2M1 branch")
    if scale_rule != "standard":
        raise ValueError(f"unknown scale_rule={scale_rule!r}")
    original_shape = tuple(x.shape)
    k = x.shape[-1]
    rows = x.numel() // k
    host_input = not x.is_cuda
    source = x.detach().reshape(rows, k).to(torch.float32)
    source = source.cuda() if host_input else source
    tail = (-k) % scale_group_size
    padded = torch.nn.functional.pad(source, (0, tail)) if tail else source.contiguous()
    groups = padded.shape[1] // scale_group_size
    amax = tensor_amax(padded)
    e2p, e2d, stats = quantize_packed(padded, mode="all_e2m1", amax=amax, want_dequant=True, want_stats=True)
    e0p, e0d, _ = quantize_packed(padded, mode="all_e0m3", amax=amax, want_dequant=True)
    zeros = torch.zeros((rows, groups), dtype=torch.uint8, device=padded.device)
    mv = (lambda t: t.to(x.device)) if host_input else (lambda t: t)
    return CandidateBlocks(
        original_shape=original_shape, source_dtype=x.dtype, operand_role=operand_role, rows=rows, k=k, groups=groups,
        padded_k=padded.shape[1], tail_padding=tail,
        grouped_original=mv(padded.reshape(rows, groups, scale_group_size)),
        e2_dequant=mv(e2d.reshape(rows, groups, scale_group_size)), e0_dequant=mv(e0d.reshape(rows, groups, scale_group_size)),
        e2_codes=mv(_level_values(e2p.codes, groups, E2M1_LEVELS)), e0_codes=mv(_level_values(e0p.codes, groups, E0M3_LEVELS)),
        e2_scales=mv(stats["e2_scales"]), e0_scales=mv(stats["e0_scales"]),
        e2_errors=mv(stats["e2_errors"]), e0_errors=mv(stats["e0_errors"]),
        e2_scale_expansion_ids=mv(zeros), e0_scale_expansion_ids=mv(zeros.clone()),
        global_scale=mv(e2p.global_scale.reshape(())), scale_rule=scale_rule)


@dataclass
class ScaledCandidate:
    """One independently scaled datatype candidate per K16 block (project_quant/scale.py:19-25)."""

    codes: torch.Tensor          # float32 [..., 16] level values with sign
    dequant: torch.Tensor        # float32 [..., 16]
    scales: torch.Tensor         # float32 [...]
    errors: torch.Tensor         # float32 [...]
    expansion_ids: torch.Tensor  # uint8 [...]: 1 where the expanded (x1.5) scale was kept


@torch.no_grad()
def build_scaled_candidate(grouped: torch.Tensor, *, format_name: str, global_scale: torch.Tensor | None = None,
                           scale_rule: str = "standard") -> ScaledCandidate:
    """The reference's ``build_scaled_candidate`` (project_quant/scale.py:165-225) for a grouped float32
    tensor [..., 16]: one candidate (``format_name`` "e2m1" or "e0m3") per block.

    scale_rule "standard": the candidate the quantizer builds (scale.py:43-61); ``global_scale`` is
    recomputed from the tensor as the reference's callers do.  scale_rule "four_over_six": the E0M3
    candidate with the base or the 1.5x expanded scale, whichever has the smaller error
    (scale.py:64-103, 207-225).  Its E2M1 counterpart is delegated by the reference to the FourOverSix
    package, which its tree does not contain: NotImplementedError."""
    if format_name not in ("e2m1", "e0m3"):
        raise ValueError(f"unknown format {format_name!r}")
    if scale_rule not in ("standard", "four_over_six"):
        raise ValueError(f"unknown scale_rule={scale_rule!r}")
    if grouped.shape[-1] != SCALE_GROUP_SIZE:
        raise ValueError("grouped must have 16 elements along its last axis")
    host_input = not grouped.is_cuda
    g = grouped.detach().to(torch.float32)
    g = (g.cuda() if host_input else g).contiguous()
    lead = g.shape[:-1]
    mv = (lambda t: t.to(grouped.device)) if host_input else (lambda t: t)
    if scale_rule == "standard":
        flat = g.reshape(-1, SCALE_GROUP_SIZE) if g.ndim < 3 else g.reshape(-1, g.shape[-2] * SCALE_GROUP_SIZE)
        mode = "all_e2m1" if format_name == "e2m1" else "all_e0m3"
        packed, dq, stats = quantize_packed(flat, mode=mode, want_dequant=True, want_stats=True)
        groups = flat.shape[1] // SCALE_GROUP_SIZE
        levels = E2M1_LEVELS if format_name == "e2m1" else E0M3_LEVELS
        key = "e2" if format_name == "e2m1" else "e0"
        return ScaledCandidate(mv(_level_values(packed.codes, groups, levels).reshape(g.shape)), mv(dq.reshape(g.shape)),
                               mv(stats[key + "_scales"].reshape(lead)), mv(stats[key + "_errors"].reshape(lead)),
                               mv(torch.zeros(lead, dtype=torch.uint8, device=g.device)))
    if format_name == "e2m1":
        raise NotImplementedError("scale_rule='four_over_six' delegates its E2M1 candidate to the FourOverSix package, "
                                  "which the reference tree does not contain")
    nblocks = g.numel() // SCALE_GROUP_SIZE
    codes, deq = torch.empty_like(g), torch.empty_like(g)
    scales = torch.empty(lead, dtype=torch.float32, device=g.device)
    errors = torch.empty(lead, dtype=torch.float32, device=g.device)
    exp = torch.empty(lead, dtype=torch.uint8, device=g.device)
    if nblocks:
        amax = tensor_amax(g.reshape(-1, SCALE_GROUP_SIZE))
        with torch.cuda.device(g.device):
            st = nat.lib().mixfp4_e0_four_over_six(g.data_ptr(), nblocks, amax.data_ptr(), codes.data_ptr(), deq.data_ptr(),
                                                   scales.data_ptr(), errors.data_ptr(), exp.data_ptr(),
                                                   nat.stream_ptr(g.device))
        nat.check("mixfp4_e0_four_over_six", st)
    return ScaledCandidate(mv(codes), mv(deq), mv(scales), mv(errors), mv(exp))


HIGH_PRECISION_MODES = ("high_precision", "fp16", "bf16")


@torch.no_grad()
def fake_quantize_activations(x: torch.Tensor, mode: str = "oracle16", *, in_place: bool = False) -> torch.Tensor:
    """The tensor the reference's forward-pre-hook hands to a linear in its W4A4 modes
    (project_quant/modeling.py:669-705): ``quant_mixfp4_granularity(x, format_region=mode,
    operand_role="activation_a")`` -- x's own global scale, K16 block scales, one format per
    block or per activation region (m4k64 ...), dequantized back to x.dtype.  x: CUDA tensor
    [..., K].  Per-block and whole-tensor modes run as one amax and one quantizer launch with
    no packed outputs (``mixfp4_fake_quantize``); region modes take the three-pass route.
    in_place=True overwrites x (it must then be contiguous along K with a dense row stride)."""
    mode = normalize_region(mode, "activation_a")
    if mode in HIGH_PRECISION_MODES:
        return x
    region = region_shape(mode, "activation_a")
    x2 = _as_rows(x)
    if region is not None:
        dq = quantize_packed(x2, mode=mode, want_dequant=True, region=region)[1]
        if in_place:
            x.copy_(dq.reshape(x.shape))
            return x
        return dq.reshape(x.shape)
    aliases_input = x2.data_ptr() == x.data_ptr() and x2.stride(-1) == 1
    out = x2 if in_place and aliases_input else torch.empty_like(x2, memory_format=torch.contiguous_format)
    amax = torch.empty(1, dtype=torch.float32, device=x2.device)
    with torch.cuda.device(x2.device):
        st = nat.lib().mixfp4_fake_quantize(x2.data_ptr(), nat.DTYPE_CODE[x2.dtype], x2.shape[0], x2.shape[1],
                                            x2.stride(0), _MODE_CODE[mode], amax.data_ptr(), out.data_ptr(),
                                            out.stride(0), nat.stream_ptr(x2.device))
    nat.check("mixfp4_fake_quantize", st)
    if in_place and not aliases_input:
        x.copy_(out.reshape(x.shape))
        return x
    return out.reshape(x.shape)


def dequantize(packed: PackedWeight, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Dense [n, k] tensor with exactly the values the reference's dequantized weight holds."""
    if dtype not in nat.DTYPE_CODE:
        raise TypeError("dtype must be bfloat16, float16 or float32")
    nat.require_cuda(packed.codes, "packed weight")
    out = torch.empty((packed.n, packed.k), dtype=dtype, device=packed.device)
    with torch.cuda.device(packed.device):
        st = nat.lib().mixfp4_dequant(packed.codes.data_ptr(), packed.scales.data_ptr(), nat.ptr(packed.fmt),
                                      packed.global_scale.data_ptr(), packed.n, packed.k, packed.layout_code,
                                      out.data_ptr(), nat.DTYPE_CODE[dtype], packed.k, nat.stream_ptr(packed.device))
    nat.check("mixfp4_dequant", st)
    return out


def _tensor_error_metrics(source: torch.Tensor, dequant: torch.Tensor) -> dict[str, float]:
    # formulas of project_quant/metrics.py:15-34, evaluated on the device
    x = source.detach().float().reshape(-1)
    q = dequant.detach().float().reshape(-1)
    delta = q - x
    err, sx, sq = torch.dot(delta, delta), torch.dot(x, x), torch.dot(q, q)
    tiny = torch.finfo(torch.float32).tiny
    cosine = torch.dot(x, q) / torch.sqrt(sx * sq).clamp_min(tiny)
    mae, mx = delta.abs().mean(), delta.abs().max()
    vals = torch.stack([err / x.numel(), err / sx.clamp_min(tiny), torch.sqrt(err / sx.clamp_min(tiny)),
                        cosine, 1 - cosine, mae, mx]).tolist()
    keys = ("mse", "nmse", "relative_l2", "cosine_similarity", "cosine_error", "mean_absolute_error",
            "max_absolute_error")
    out = dict(zip(keys, vals))
    out["mean_abs_error"] = out["mean_absolute_error"]
    out["max_abs_error"] = out["max_absolute_error"]
    return out


@torch.no_grad()
def quant_mixfp4_granularity(
    x: torch.Tensor,
    *,
    scale_group_size: int = SCALE_GROUP_SIZE,
    format_region: str = "oracle16",
    operand_role: str = "weight_b",
    selector: str = "mse",
    scale_rule: str = "standard",
    calibration_stats: dict[str, Any] | None = None,
    transform: Any = None,
    permutation: torch.Tensor | None = None,
    return_stats: bool = False,
    collect_regions: bool = False,
    region_sample_limit: int | None = None,
) -> torch.Tensor | GranularityResult:
    """Fake-quantize ``x`` with K16 block scales and a per-block E2M1/E0M3 choice.

    Drop-in for the reference function of the same name: returns a new tensor of
    ``x.shape`` / ``x.dtype`` (or a GranularityResult with ``return_stats=True``).
    Supported here: format_region oracle16 / all_e2m1 / all_e0m3 and the coarse regions
    k32_row, k64_row, n2k64 ... n64k64 (weights), m4k64 ... m32k64 (activations) with
    selector "mse" and scale_rule "standard" (n8k16 / m16k16 sum their columns in the order
    PyTorch's CPU kernels use on an AVX-512 host, "layer" decides on double-precision sums); the
    output-aware selector and the four_over_six rule raise NotImplementedError.
    """
    working = x
    if permutation is not None:
        if operand_role != "weight_b" or x.ndim != 2:
            raise ValueError("permutation is defined only for [N,K] weights")
        if permutation.numel() != x.shape[0]:
            raise ValueError("permutation length must equal N")
        working = working.index_select(0, permutation.to(working.device))
    mode = normalize_region(format_region, operand_role)
    validate_layout(working, scale_group_size=scale_group_size, operand_role=operand_role)
    if scale_rule == "four_over_six":
        raise NotImplementedError("scale_rule='four_over_six' is not implemented in the CUDA path")
    if scale_rule != "standard":
        raise ValueError(f"unknown scale_rule={scale_rule!r}")
    if selector in {"output_aware", "activation_aware"}:
        if operand_role != "weight_b" or mode != "n8k64":
            raise ValueError("output-aware selection is defined for N8K64 weights")
        raise NotImplementedError("output-aware selection is not implemented in the CUDA path")
    if selector != "mse":
        raise ValueError(f"unknown selector={selector!r}")
    region = region_shape(mode, operand_role)

    host_input = not working.is_cuda
    if host_input:
        working = working.cuda()
    if transform is not None:
        working = _rotation.apply_transform(working, transform)

    packed, dq, stats = quantize_packed(working, mode=mode, want_dequant=True, want_stats=return_stats, region=region)
    dequant = dq.reshape(working.shape)
    if host_input:
        dequant = dequant.to(x.device)
    if not return_stats:
        return dequant

    e2e, e0e = stats["e2_errors"], stats["e0_errors"]
    ids = packed.format_ids()
    oracle_ids = (e0e < e2e).to(torch.uint8)
    margin = e2e - e0e
    selected_err = torch.where(ids.bool(), e0e, e2e).sum()
    oracle_err = torch.minimum(e2e, e0e).sum()
    numel = working.numel()
    blocks = ids.numel()
    k = working.shape[-1]
    rows = numel // k
    small = torch.stack([ids.float().sum(), oracle_ids.float().sum(), margin.mean(), margin.abs().mean(),
                         margin.median(), oracle_err, selected_err, e2e.sum(), e0e.sum(),
                         packed.global_scale[0]]).tolist()
    e0_count, oracle_e0 = int(small[0]), int(small[1])
    coarse = region is not None and region[1] > 0          # "layer" reports the whole tensor as its region
    summary: dict[str, Any] = {
        **_tensor_error_metrics(working, dq.reshape(working.shape)),
        "scale_group_size": scale_group_size, "scale_rule": scale_rule, "format_granularity": mode,
        "format_region_rows": region[0] if coarse else (1 if mode == "oracle16" else rows),
        "format_region_k16_groups": region[1] if coarse else (1 if mode == "oracle16" else packed.groups),
        "format_region_k_values": 16 * (region[1] if coarse else (1 if mode == "oracle16" else packed.groups)),
        "operand_role": operand_role, "selector": "mse", "tail_policy": TAIL_POLICY,
        "tail_padding_values": (-k) % 16, "rows": rows, "N_or_M": rows, "K": k, "numel": numel,
        "num_scale_blocks": blocks, "e0_count": e0_count, "e2_count": blocks - e0_count,
        "e0_ratio": e0_count / blocks, "e2_ratio": 1.0 - e0_count / blocks,
        "oracle_e0_count": oracle_e0, "oracle_e2_count": blocks - oracle_e0, "oracle_e0_ratio": oracle_e0 / blocks,
        "mean_format_margin": small[2], "mean_signed_format_margin": small[2], "mean_abs_format_margin": small[3],
        "median_format_margin": small[4], "oracle_mse": small[5] / numel, "constrained_mse": small[6] / numel,
        "selected_mse": small[6] / numel, "oracle_error": small[5], "constrained_error": small[6],
        "selected_weight_error": small[6], "granularity_regret": small[6] - small[5],
        "all_e2m1_error": small[7], "all_e0m3_error": small[8], "global_scale": small[9],
        "transform": getattr(transform, "name", transform) if transform is not None else "identity",
        "permutation_applied": permutation is not None,
    }
    mv = lambda t: t.to(x.device) if host_input else t
    return GranularityResult(
        dequant=dequant, format_ids=mv(ids), oracle_format_ids=mv(oracle_ids),
        selected_scales=mv(packed.selected_scales()),
        selected_scale_expansion_ids=mv(torch.zeros_like(ids)),
        e2_scales=mv(stats["e2_scales"]), e0_scales=mv(stats["e0_scales"]),
        e2_errors=mv(e2e), e0_errors=mv(e0e), summary=summary, regions=[], packed=packed)

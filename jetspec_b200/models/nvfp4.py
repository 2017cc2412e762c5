"""NVFP4 quantisation: e2m1 values, one e4m3 scale per 16 elements along K, one fp32 scale above them.

The reference has no low-precision path (its linears are bf16 ``nn.Linear`` / cuBLAS,
``jetspec/fused_gemm.py:1-80``); this module is the weight/activation format of the 4-bit target.

Layout of a quantised ``(rows, K)`` matrix (``K % 64 == 0``):

* ``packed``  ``(rows, K/2) uint8`` — two e2m1 codes per byte, element ``2i`` in the low nibble;
* ``scales``  ``(rows, K/16) float8_e4m3fn`` — block scale, stored divided by the outer scale;
* outer scale — one fp32 per tensor (weights) or one fp32 per row (activations quantised on the fly);
* ``dequant = e2m1 * e4m3 * outer``.

The tensor-core kernel reads the block scales in 512-byte tiles of 128 rows x 4 blocks
(``swizzle_scales``): byte ``(r % 32) * 16 + (r // 32 % 4) * 4 + b`` of tile ``(r // 128, kblock // 4)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

E2M1_MAX = 6.0
E4M3_MAX = 448.0
BLOCK = 16
# magnitudes of the eight e2m1 codes and the midpoints that round a magnitude to the nearest code
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def _e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 values (already divided by their scale) -> 4-bit codes (sign in bit 3); ties go to the even code."""
    mag = x.abs()
    bounds = torch.tensor(_BOUNDS, dtype=torch.float32, device=x.device)
    code = torch.bucketize(mag, bounds, right=False)          # mag == bound -> lower code
    # round-half-to-even on the code's mantissa bit: at a midpoint pick the code whose lsb is 0
    at_mid = (mag.unsqueeze(-1) == bounds).any(-1)
    code = torch.where(at_mid & (code % 2 == 1), code + 1, code).clamp_(max=7)
    return (code | ((x < 0).to(code.dtype) << 3)).to(torch.uint8)


def _e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), dtype=torch.float32, device=code.device)
    return lut[code.long()]


@dataclass
class NVFP4Tensor:
    """A quantised matrix; ``outer`` is a 0-d tensor (per tensor) or ``(rows,)`` (per row).

    Rows are independent given the outer scale, so row slices, row concatenations (of tensors that share
    one outer scale) and row permutations are exact; K can be cut at multiples of 64.
    """
    packed: torch.Tensor
    scales: torch.Tensor
    outer: torch.Tensor
    shape: tuple
    scales_swizzled: Optional[torch.Tensor] = None

    @property
    def device(self):
        return self.packed.device

    @property
    def dtype(self):
        return torch.uint8

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return dequantize_nvfp4(self, dtype)

    def nbytes(self) -> int:
        return self.packed.numel() + self.scales.numel() + 4 * max(1, self.outer.numel())

    def swizzled(self) -> "NVFP4Tensor":
        """Make sure the tile-ordered copy of the block scales exists (the tensor-core kernel reads it)."""
        if self.scales_swizzled is None:
            self.scales_swizzled = swizzle_scales(self.scales)
        return self

    def to(self, device) -> "NVFP4Tensor":
        sw = self.scales_swizzled.to(device) if self.scales_swizzled is not None else None
        return NVFP4Tensor(self.packed.to(device), self.scales.to(device), self.outer.to(device), self.shape, sw)

    def _outer_rows(self, sel):
        return self.outer[sel] if self.outer.dim() == 1 else self.outer

    def rows(self, a: int, b: int) -> "NVFP4Tensor":
        return NVFP4Tensor(self.packed[a:b], self.scales[a:b], self._outer_rows(slice(a, b)), (b - a, self.shape[1]))

    def index_rows(self, idx: torch.Tensor) -> "NVFP4Tensor":
        return NVFP4Tensor(self.packed[idx].contiguous(), self.scales.view(torch.uint8)[idx].contiguous()
                           .view(torch.float8_e4m3fn), self._outer_rows(idx), (int(idx.numel()), self.shape[1]))

    def cols(self, k0: int, k1: int) -> "NVFP4Tensor":
        if k0 % 64 or k1 % 64:
            raise ValueError("NVFP4 matrices can be cut along K at multiples of 64 only")
        return NVFP4Tensor(self.packed[:, k0 // 2:k1 // 2].contiguous(),
                           self.scales.view(torch.uint8)[:, k0 // BLOCK:k1 // BLOCK].contiguous().view(torch.float8_e4m3fn),
                           self.outer, (self.shape[0], k1 - k0))

    @staticmethod
    def cat_rows(parts: list) -> "NVFP4Tensor":
        o = parts[0].outer
        if o.dim() != 0 or any(p.outer.dim() != 0 or float(p.outer) != float(o) for p in parts):
            raise ValueError("only matrices that share one per-tensor scale can be stacked")
        return NVFP4Tensor(torch.cat([p.packed for p in parts], 0).contiguous(),
                           torch.cat([p.scales.view(torch.uint8) for p in parts], 0).contiguous().view(torch.float8_e4m3fn),
                           o, (sum(p.shape[0] for p in parts), parts[0].shape[1]))


def quantize_nvfp4(x: torch.Tensor, per_row: bool = False, swizzle: bool = True) -> NVFP4Tensor:
    """Quantise a ``(rows, K)`` matrix.  ``per_row`` picks one outer scale per row (the on-the-fly
    activation mode) instead of one per tensor (the offline weight mode)."""
    if x.dim() != 2 or x.shape[1] % 64:
        raise ValueError(f"NVFP4 needs a 2-D matrix with K % 64 == 0, got {tuple(x.shape)}")
    rows, K = x.shape
    xf = x.detach().float()
    amax = xf.abs().amax(dim=1) if per_row else xf.abs().amax()
    # divisors are device tensors: dividing a CUDA tensor by a Python number multiplies by the rounded
    # reciprocal instead, which would make the bytes depend on the device
    c_full = torch.tensor(E2M1_MAX * E4M3_MAX, dtype=torch.float32, device=xf.device)
    c_six = torch.tensor(E2M1_MAX, dtype=torch.float32, device=xf.device)
    outer = torch.div(amax, c_full).clamp_min(1e-30)
    blocks = xf.view(rows, K // BLOCK, BLOCK)
    o = outer.view(-1, 1) if per_row else outer
    want = torch.div(torch.div(blocks.abs().amax(dim=2), c_six), o)       # block scale before rounding
    scales = want.clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    sf = scales.float() * o                                                # the scale the decoder will apply
    q = torch.where(sf.unsqueeze(-1) > 0, blocks / sf.unsqueeze(-1).clamp_min(1e-30), torch.zeros_like(blocks))
    code = _e2m1_encode(q.clamp(-E2M1_MAX, E2M1_MAX)).view(rows, K)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    t = NVFP4Tensor(packed, scales.contiguous(), outer.float().contiguous(), (rows, K))
    if swizzle:
        t.scales_swizzled = swizzle_scales(t.scales)
    return t


def dequantize_nvfp4(t: NVFP4Tensor, dtype=torch.float32) -> torch.Tensor:
    rows, K = t.shape
    lo, hi = t.packed & 0xF, t.packed >> 4
    code = torch.stack([lo, hi], dim=-1).view(rows, K)
    vals = _e2m1_decode(code).view(rows, K // BLOCK, BLOCK)
    o = t.outer.view(-1, 1, 1) if t.outer.dim() == 1 else t.outer
    return (vals * t.scales.float().unsqueeze(-1) * o).view(rows, K).to(dtype)


def swizzle_scales(scales: torch.Tensor) -> torch.Tensor:
    """``(rows, K/16)`` block scales -> the tensor-core tile order, rows padded to a multiple of 128."""
    rows, nb = scales.shape
    if nb % 4:
        raise ValueError("K must be a multiple of 64")
    pad = (-rows) % 128
    raw = scales.view(torch.uint8)
    if pad:
        raw = torch.cat([raw, raw.new_zeros(pad, nb)], dim=0)
    t = raw.view(-1, 4, 32, nb // 4, 4)                # (row tile, c = r//32 % 4, l = r % 32, k tile, b)
    return t.permute(0, 3, 2, 1, 4).contiguous().view(-1)


def unswizzle_scales(flat: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """Inverse of :func:`swizzle_scales` (returns ``(rows, K/16) float8_e4m3fn``)."""
    nb = K // BLOCK
    t = flat.view(-1, nb // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1, nb)
    return t[:rows].view(torch.float8_e4m3fn)


def nvfp4_linear_reference(x: torch.Tensor, w: NVFP4Tensor, quantize_input: bool = True) -> torch.Tensor:
    """Oracle of the 4-bit linear: (optionally fake-quantised) ``x`` times the dequantised weight, fp32 math."""
    xf = x.float()
    if quantize_input:
        xf = quantize_nvfp4(xf, per_row=True, swizzle=False).dequantize()
    wd = w.__dict__.get("_deq")
    if wd is None:                      # the oracle keeps the dequantised weight (CPU tests call it every step)
        wd = w.dequantize()
        w.__dict__["_deq"] = wd
    return xf @ wd.t()


class NVFP4Linear(torch.nn.Module):
    """Stand-in for ``nn.Linear(bias=False)`` holding NVFP4 weights; activations are quantised per call
    (one outer scale per row).  ``.weight`` is the :class:`NVFP4Tensor`, which ``ops.linear`` understands, so
    model code written as ``ops.linear(x, proj.weight, proj.bias)`` runs unchanged.

    On a CUDA device the product runs on the block-scaled tensor-core kernel; elsewhere on the oracle.
    """
    bias = None

    def __init__(self, weight):
        super().__init__()
        q = weight if isinstance(weight, NVFP4Tensor) else quantize_nvfp4(weight, per_row=False)
        self.out_features, self.in_features = q.shape
        self.register_buffer("packed", q.packed.contiguous())
        self.register_buffer("scales", q.scales.contiguous().view(torch.uint8))
        self.register_buffer("outer", q.outer.clone())

    @property
    def weight(self) -> NVFP4Tensor:
        q = self.__dict__.get("_q")
        if q is None or q.packed.data_ptr() != self.packed.data_ptr():     # rebuilt after .to(device)
            q = NVFP4Tensor(self.packed, self.scales.view(torch.float8_e4m3fn), self.outer,
                            (self.out_features, self.in_features))
            self.__dict__["_q"] = q
        return q

    qweight = weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .. import ops
        shp = x.shape
        y = ops.linear(x.reshape(-1, shp[-1]), self.weight)
        return y.view(*shp[:-1], self.out_features)


# projections that read the same activations are quantised as ONE matrix, so that the fused
# (QKV, gate|up) weights the kernels use are row stacks of exactly the per-projection weights
_GROUPS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))


def quantize_model_nvfp4(model: torch.nn.Module, skip=("lm_head", "embed_tokens")) -> int:
    """Replace every bias-free ``nn.Linear`` of ``model`` (except names containing ``skip``) in place.
    Returns the number of layers converted."""
    n = 0
    for name, mod in list(model.named_modules()):
        kids = dict(mod.named_children())

        def ok(cname):
            c = kids.get(cname)
            full = f"{name}.{cname}" if name else cname
            return (isinstance(c, torch.nn.Linear) and c.bias is None and c.in_features % 64 == 0
                    and not any(s in full for s in skip))
        done = set()
        for group in _GROUPS:
            if all(ok(c) for c in group):
                q = quantize_nvfp4(torch.cat([kids[c].weight.data for c in group], 0), swizzle=False)
                r0 = 0
                for c in group:
                    r1 = r0 + kids[c].out_features
                    setattr(mod, c, NVFP4Linear(q.rows(r0, r1)))
                    r0 = r1
                    done.add(c)
                    n += 1
        for cname in kids:
            if cname not in done and ok(cname):
                setattr(mod, cname, NVFP4Linear(kids[cname].weight.data))
                n += 1
    return n

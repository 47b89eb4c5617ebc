"""A linear map y = W x without bias, W stored [out, in] as model folders hold it
(reference: kernels/megakernel_ops.hip:168-216).  Several named tensors can be
stacked along `out` at load time (q, k and v; gate and up) so that one product
serves them all; stacking rows changes no output value.

Not a registered part: mixers, feed-forwards and heads are built from it.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .spec import TensorSpec

_SMS = None


def stream_k_pays(rows: int, w_rows: int, k_in: int, sms: Optional[int] = None) -> bool:
    """Whether the product of `rows` tokens with a [w_rows, k_in] weight should be spread evenly over
    all SMs along k as well ("stream-k" partial sums plus a kernel that adds them up) rather than
    cut into whole output tiles: it pays when whole tiles would leave SMs idle and the partial sums
    (rows x w_rows floats a CTA that shares a tile) are small beside the weights (w_rows x k_in).
    Measured on the 7B layer sizes at 1 to 2,048 tokens.  Up to 128 tokens whole tiles are [128 x token
    tile] on single SMs: stream-k when the last round of tiles would be less than 70 % full (80 % for up
    to 48 tokens: at 33 tokens gate+up is 2.6 % of a step faster so, at 64 it is a tie).  Beyond, whole tiles are [256 x 256] on pairs of SMs: stream-k when their last round
    would be less than 70 % full and rows <= min(k_in / 16, 512): at 256 tokens every product of width
    4096 but gate+up, at 512 only down (k_in = 14336), from 513 on none."""
    from ..csrc.api import PAIR_TOKEN_TILE, token_tile
    global _SMS
    if sms is None:
        if _SMS is None:
            _SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        sms = _SMS
    tile = token_tile(rows)
    if tile == PAIR_TOKEN_TILE:
        if rows > min(k_in // 16, 512):
            return False
        units, pairs = -(-w_rows // 256) * -(-rows // tile), max(sms // 2, 1)
        return units / (-(-units // pairs) * pairs) < 0.7
    tiles = -(-w_rows // 128) * -(-rows // tile)
    fill = tiles / (-(-tiles // sms) * sms)
    return fill < (0.8 if rows <= 48 else 0.7)


# Rows up to which a norm may leave its scale to the next product: beyond the token tiles of the
# one-SM kernel the products run on pairs of SMs, which take no row scale.
ROW_SCALE_MAX_ROWS = 128


class Linear:
    def __init__(self, rt, names: Sequence[str], out_features: Sequence[int], in_features: int,
                 gate_up: bool = False) -> None:
        """`gate_up`: the two tensors are the gate and up halves of a SwiGLU; where the
        tensor-core kernel will run them, they are stored interleaved in blocks of 16 rows
        for its epilogue instead of stacked."""
        self.rt = rt
        self.names = list(names)
        self.out_features = list(out_features)
        self.in_features = in_features
        self.weight: Optional[torch.Tensor] = None
        self.gate_up = gate_up
        self.interleaved = False

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {n: TensorSpec((o, self.in_features)) for n, o in zip(self.names, self.out_features)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        parts = [tensors[n] for n in self.names]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.float() for p in parts]
        if (self.gate_up and len(parts) == 2 and parts[0].dtype == torch.bfloat16 and self.rt.gemm_backend == "auto"
                and self.rt.act_dtype == torch.bfloat16 and self.in_features % 8 == 0 and self.rt.kernels is not None):
            from ..csrc.api import interleave_gate_up
            self.weight = interleave_gate_up(parts[0], parts[1])
            self.interleaved = True
            return
        self.weight = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def share(self, weight: torch.Tensor) -> None:
        """Use a tensor that another part owns (a tied output head)."""
        self.weight = weight

    @property
    def total_out(self) -> int:
        return sum(self.out_features)

    def takes_row_scale(self) -> bool:
        """Whether `forward` can apply a row scale that its input still wants (`in_scale`): the
        tensor-core products do, in their epilogues and in the kernels that add up their partial sums."""
        w = self.weight
        return (self.rt.gemm_backend == "auto" and self.rt.act_dtype == torch.bfloat16 and w is not None
                and w.dtype == torch.bfloat16 and self.in_features % 8 == 0 and w.stride(0) % 8 == 0
                and w.data_ptr() % 16 == 0 and (not self.gate_up or self.interleaved))

    def forward(self, x: torch.Tensor, *, out_dtype: Optional[torch.dtype] = None,
                residual: Optional[torch.Tensor] = None, swiglu: bool = False, defer_to=None,
                in_scale=None) -> torch.Tensor:
        """x [rows, in].  Plain: returns [rows, out] in `out_dtype` (default x's type).
        `residual` (float32 [rows, out]): returns residual + product, written in place.
        `swiglu`: the weight holds gate rows then up rows; returns silu(gate) * up.
        `defer_to` (a StepContext): when the product runs in its stream-k form, leave the
        adding-up of its partial sums to whoever reads the result next
        (`StepContext.deferred`); the returned tensor is complete only after that.
        `in_scale` (csrc.api.RowScale): x's rows still want this scale; the product applies it to
        its results (only where `takes_row_scale()`, and not with a residual)."""
        K = self.rt.kernels
        w = self.weight
        rows = x.shape[0]
        w_rows = w.shape[0]
        if in_scale is not None and (residual is not None or not self.takes_row_scale() or x.dtype != torch.bfloat16
                                     or not K.gemm_tc_eligible(x, w)):
            raise RuntimeError("this product cannot apply a row scale (see Linear.takes_row_scale)")
        if w.dtype == torch.float32 and x.dtype != torch.float32:
            # a weight stored in 32-bit stays so: this product runs in float32
            x32 = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            K.cast(x, x32)
            y = self.forward(x32, out_dtype=torch.float32 if residual is None else None,
                             residual=residual, swiglu=swiglu)
            if residual is not None:
                return y
            want = out_dtype or x.dtype
            if want == torch.float32:
                return y
            y2 = torch.empty(y.shape, dtype=want, device=y.device)
            K.cast(y, y2)
            return y2
        use_tc = (self.rt.gemm_backend == "auto" and x.dtype == torch.bfloat16 and K.gemm_tc_eligible(x, w))
        sk = use_tc and stream_k_pays(rows, w_rows, x.shape[1])
        can_defer = (defer_to is not None and sk and not swiglu
                     and self.rt.fuse_reduce and K.pending_partial is None)
        if residual is not None:
            if can_defer:
                defer_to.defer(residual, K.gemm_tc_partial(x, w), "residual")
            elif use_tc:
                K.gemm_tc(x, w, residual, residual=residual, stream_k=sk)
            else:
                K.gemm_simt(x, w, residual, residual=residual)
            return residual
        if swiglu:
            inter = self.out_features[0]
            out = torch.empty((rows, inter), dtype=out_dtype or x.dtype, device=x.device)
            if self.interleaved:
                if not use_tc:
                    raise RuntimeError("interleaved gate/up weights need the tensor-core product; its input rows "
                                       "must be 16-byte aligned bfloat16")
                K.gemm_tc(x, w, out, swiglu=True, stream_k=sk, in_scale=in_scale)
            else:
                gu = torch.empty((rows, w_rows), dtype=x.dtype, device=x.device)
                K.gemm_simt(x, w, gu)
                K.silu_mul(gu, out)
            return out
        out = torch.empty((rows, w_rows), dtype=out_dtype or x.dtype, device=x.device)
        if can_defer:
            defer_to.defer(out, K.gemm_tc_partial(x, w, in_scale=in_scale), "store")
        elif use_tc:
            K.gemm_tc(x, w, out, stream_k=sk, in_scale=in_scale)
        else:
            K.gemm_simt(x, w, out)
        return out

"""RMSNorm, alone or fused with the residual add before it.

Formula of the reference: vllm/kernels/layernorm_kernels.cu:13-68, called from
core/src/model_executor/models/llama/llama.rs:295-317, :333, :461-462.  The residual stream is
float32 here whatever the activation dtype.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple, Union

import torch

from .. import kernels
from .base import Norm, Normed, Prenormed, WeightSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    splittable = True

    def __init__(self, hidden_size: int, eps: float, weight_offset: float = 0.0, layer_scale: bool = False):
        self.hidden_size = int(hidden_size)
        # a second learned vector that multiplies the normed output element by element (a branch's "layer scale");
        # a weight of its own, `scale`, so that the product w * scale is formed in float32 at run time
        self.has_layer_scale = bool(layer_scale)
        self.scale: Optional[torch.Tensor] = None
        self._w32: Optional[torch.Tensor] = None
        self._s32: Optional[torch.Tensor] = None
        self.eps = float(eps)
        # architectures that scale by (1 + w) store w: the offset is folded into the weight when it is set, as the
        # reference's loader does (vllm/src/rms_norm.rs:45-56); 0 for Llama
        self.weight_offset = float(weight_offset)
        self.weight: Optional[torch.Tensor] = None

    def set_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        super().set_weights(tensors)
        if self.weight_offset and "weight" in tensors:
            self.weight = (tensors["weight"].float() + self.weight_offset).to(tensors["weight"].dtype)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"weight": WeightSpec([(self.hidden_size,)], keep_fp32=True)}
        if self.has_layer_scale:
            specs["scale"] = WeightSpec([(self.hidden_size,)], keep_fp32=True)
        return specs

    def weight_f32(self) -> torch.Tensor:
        """The weight as float32 (exact: the stored values are of 16 or 32 bits), for the kernels that take it so."""
        if self._w32 is None or self._w32.device != self.weight.device:
            self._w32 = self.weight.float().contiguous()
        return self._w32

    def scale_f32(self) -> Optional[torch.Tensor]:
        if not self.has_layer_scale:
            return None
        if self._s32 is None or self._s32.device != self.scale.device:
            self._s32 = self.scale.float().contiguous()
        return self._s32

    _act_dtype: Optional[torch.dtype] = None

    def prepare(self, dtype, device) -> None:
        self._act_dtype = dtype
        self._w32 = self._s32 = None
        self.weight_f32()
        self.scale_f32()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = torch.empty_like(x)
        kernels.add_rmsnorm(h, x, None, self.weight, self.eps, 0)
        if self.has_layer_scale:
            h.mul_(self.scale.to(h.dtype))
        return h

    def of_stream(self, res: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """norm(res) * w of a complete float32 stream, in the activation type."""
        h = torch.empty(res.shape, dtype=dtype, device=res.device)
        kernels.stream_norm(res, h=h, w_next=self.weight_f32(), eps_next=self.eps)
        return h

    def forward_residual(self, x: Union[torch.Tensor, Prenormed], res: Optional[torch.Tensor]
                         ) -> Tuple[Union[torch.Tensor, Prenormed], torch.Tensor]:
        if isinstance(x, Prenormed):
            if x.norm is not self or x.res is not res:
                raise ValueError("a Prenormed activation was prepared for another norm or residual stream")
            return x, res
        if isinstance(x, Normed):            # the block before has applied this norm to the complete stream
            if x.norm is not self or x.res is not res:
                raise ValueError("a Normed activation was prepared for another norm or residual stream")
            return x.h, res
        if x is None:                        # nothing pending: the stream is complete
            if self.has_layer_scale:
                raise ValueError("a norm with a layer scale norms a branch, not the stream")
            return self.of_stream(res, self._act_dtype or torch.float32), res
        if self.has_layer_scale:
            raise ValueError("a norm with a layer scale norms a branch, not the stream")
        h = torch.empty_like(x)
        if res is None:
            res = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            kernels.add_rmsnorm(h, x, res, self.weight, self.eps, 1)
        else:
            kernels.add_rmsnorm(h, x, res, self.weight, self.eps, 2)
        return h, res

    def finish(self, p: Prenormed) -> torch.Tensor:
        """The ordinary output of the norm from a `Prenormed`, for a product that cannot take one."""
        h = torch.empty_like(p.x)
        kernels.finish_rmsnorm(h, p.res, p.sumsq, self.weight, self.eps)
        return h

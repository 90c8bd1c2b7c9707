"""Element-wise gated recurrences with one state vector per request.

minGRU: the update gate and the candidate read only the current token,

    z_t = sigmoid(W_z x_t + b_z)        u_t = W_x x_t + b_x
    c_t = u_t + 1/2  where u_t >= 0,    sigmoid(u_t)  elsewhere
    S_t = (1 - z_t) S_(t-1) + z_t c_t   out_t = W_o (S_t * silu(W_g x_t))

The state starts at zero, is 32-bit and lives in the request's slot of the cache manager's state tensor; the three
projections are one stacked product whose result stays 32-bit, so that everything that enters the recurrence is.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateSpec, TensorSpec, register_part

_NAMES = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "gate": "g", "out": "o"}


class MinGRU(Mixer):
    graph_safe = True
    accepts_sink = True

    def __init__(self, hidden_size: int, width: int, bias: bool = True, tensor_names: dict[str, str] | None = None):
        self.hidden_size, self.width, self.bias = int(hidden_size), int(width), bool(bias)
        self.names = {**_NAMES, **(tensor_names or {})}
        self.w_in = self.w_out = self.b_z = self.b_x = None
        self.dtype: torch.dtype | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        n, w, h = self.names, self.width, self.hidden_size
        specs = {n["z"]: TensorSpec((w, h)), n["x"]: TensorSpec((w, h)), n["gate"]: TensorSpec((w, h)), n["out"]: TensorSpec((h, w))}
        if self.bias:
            specs[n["z_bias"]] = TensorSpec((w,))
            specs[n["x_bias"]] = TensorSpec((w,))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n[k]].to(dtype) for k in ("z", "x", "gate")], dim=0).to(device).contiguous()
        self.w_out = tensors[n["out"]].to(device=device, dtype=dtype).contiguous()
        if self.bias:
            self.b_z = tensors[n["z_bias"]].to(device=device, dtype=torch.float32).contiguous()
            self.b_x = tensors[n["x_bias"]].to(device=device, dtype=torch.float32).contiguous()
        self.dtype = dtype

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.width,), torch.float32)

    def forward(self, x, ctx, cache, sink=None):
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [N, z | x | gate], 32-bit
        out = ops.mingru_scan(proj, self.b_z, self.b_x, cache.states, cache.slots, ctx.cu_tokens, ctx.num_requests, self.width, self.dtype, ctx.max_query_len)
        if sink is not None:
            handed_on = sink.linear(out, self.w_out)
            if handed_on is not None:
                return handed_on
        return ops.linear(out, self.w_out, out_dtype=torch.float32)


register_part("mixer", "mingru", MinGRU)

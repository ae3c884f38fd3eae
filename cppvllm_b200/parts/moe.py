"""Feed-forward parts beside the gated dense one (parts/mlp.py):

* ``act_mlp``: y = Wdown act(Wup x [+ b_up]) [+ b_down], no gate; act = "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))))
  or "relu2" (relu(z)^2); ``bias=True`` adds the two bias vectors ``<up>.b`` and ``<down>.b``.
* ``routed_glu``: a mixture of experts.  Router logits z = Wr x + b in float32 (x as the norm rounded it); each token uses
  its ``top`` best-scoring experts C, with weights w_e = exp(z_e) / sum_{c in C} exp(z_c); an expert is
  Wdown (silu(Wgate x) * (Wup x)) without biases; the output is the weighted sum of the chosen experts' outputs.  Expert e's
  tensors are ``<prefix>e<e>.gate|up|down``; they are stacked at load time into [E, 2 ff, D] (gate rows over up rows) and
  [E, D, ff], so that a kernel reaches every expert from one base address.  One or two tokens read only their chosen
  experts' weights pair by pair (two kernels spread over all SMs); more are sorted by expert on the device and go through
  two grouped products on the tcgen05 kernel (csrc/moe.cu, csrc/gemm_tcgen05.cu); nothing travels to the host, so steps
  stay capturable.  Options: ``score = "sigmoid"``: the chosen experts' weights are their own sigmoid(z_e), not renormalised;
  ``weight_on_input``: the weight multiplies the expert's input, y = sum_e expert_e(w_e x); ``router_bias = False``: no bias
  tensor; ``shared_size`` > 0: a shared expert of the same gated form (``<prefix>shared.gate|up|down``) runs for every token
  and is added.
* ``clamped_glu``: dense and gated with clamps: g = min(Wgate x, L), u = clamp(Wup x, -L, L); y = Wdown (g sigmoid(alpha g) (u + 1)).
* ``routed_act``: a mixture of ungated experts Wdown act(Wup x) (act = relu2) whose weights are `scale` times the chosen experts'
  shares of the softmax over ALL experts (not renormalised over the winners); no router bias.  Optionally a shared expert of
  the same form and a size of its own runs for every token and joins through sigmoid(w_sg . x), one number per token; its
  gate's row rides behind the router's rows, so one kernel makes both.  Same kernels as ``routed_glu`` with the activation
  as a parameter (the grouped tcgen05 product takes the squared relu as its epilogue).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, WeightSpec, register_part


@register_part("ffn", "act_mlp")
class ActMLP(FeedForward):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh",
                 up_name: str = "up", down_name: str = "down", bias: bool = False):
        super().__init__(runtime, prefix, names)
        if activation not in ("gelu_tanh", "relu2"):
            raise ValueError(f"activation '{activation}' is not built; built: gelu_tanh, relu2")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.activation, self.bias = activation, bool(bias)
        self.up_name, self.down_name = up_name, down_name
        self.w_up = self.w_down = self.b_up = self.b_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, I = self.hidden_size, self.intermediate_size
        specs = {self.full_name(self.up_name): WeightSpec((I, D)), self.full_name(self.down_name): WeightSpec((D, I))}
        if self.bias:
            specs[self.full_name(self.up_name + ".b")] = WeightSpec((I,), role="vector")
            specs[self.full_name(self.down_name + ".b")] = WeightSpec((D,), role="vector")
        return specs

    def bind(self, tensors) -> None:
        self.w_up, self.w_down = tensors[self.full_name(self.up_name)], tensors[self.full_name(self.down_name)]
        if self.bias:
            self.b_up, self.b_down = tensors[self.full_name(self.up_name + ".b")], tensors[self.full_name(self.down_name + ".b")]

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down))

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def forward_unbiased(self, x, ctx):
        """(Wdown act(Wup x + b_up), b_down): for a caller whose next kernel adds the output bias itself."""
        T = x.shape[0]
        ws = self.rt.workspace
        up = self._project(x, self.w_up, ws.rows("ffn_up", T, self.intermediate_size, x.dtype), T)
        if self.activation == "gelu_tanh" and self.b_up is None:
            ops.gelu_tanh(up, up)
        else:
            ops.bias_act(up, up, self.b_up, self.activation)
        return self._project(up, self.w_down, ws.rows("ffn_out", T, self.hidden_size, x.dtype), T), self.b_down

    def forward(self, x, ctx):
        y, bias = self.forward_unbiased(x, ctx)
        return ops.bias_act(y, y, bias, "none") if bias is not None else y


@register_part("ffn", "routed_glu")
class RoutedGLU(FeedForward):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 router_name: str = "router", router_bias_name: str = "router.b", expert_prefix: str = "e", score: str = "softmax",
                 weight_on_input: bool = False, router_bias: bool = True, shared_size: int = 0, shared_prefix: str = "shared."):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.num_experts, self.top = int(num_experts), int(top)
        if not (0 < self.top <= self.num_experts):
            raise ValueError(f"a token cannot use {self.top} of {self.num_experts} experts")
        if score not in ("softmax", "sigmoid"):
            raise ValueError(f"score is 'softmax' (over the chosen experts) or 'sigmoid', got {score!r}")
        self.router_name, self.router_bias_name, self.expert_prefix = router_name, router_bias_name, expert_prefix
        self.score, self.weight_on_input, self.router_bias = score, bool(weight_on_input), bool(router_bias)
        self.shared_size, self.shared_prefix = int(shared_size), shared_prefix
        self.w_router = self.b_router = self.w_gate_up = self.w_down = self.shared_gate_up = self.shared_down = None

    def _expert(self, e: int, which: str) -> str:
        return self.full_name(f"{self.expert_prefix}{e}.{which}")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, I, E = self.hidden_size, self.intermediate_size, self.num_experts
        specs = {self.full_name(self.router_name): WeightSpec((E, D), role="vector")}
        if self.router_bias:
            specs[self.full_name(self.router_bias_name)] = WeightSpec((E,), role="vector")
        for e in range(E):
            specs[self._expert(e, "gate")] = WeightSpec((I, D))
            specs[self._expert(e, "up")] = WeightSpec((I, D))
            specs[self._expert(e, "down")] = WeightSpec((D, I))
        if self.shared_size:
            sp = self.shared_prefix
            specs[self.full_name(sp + "gate")] = WeightSpec((self.shared_size, D))
            specs[self.full_name(sp + "up")] = WeightSpec((self.shared_size, D))
            specs[self.full_name(sp + "down")] = WeightSpec((D, self.shared_size))
        return specs

    def bind(self, tensors) -> None:
        E = self.num_experts
        self.w_router = tensors[self.full_name(self.router_name)]
        self.b_router = tensors[self.full_name(self.router_bias_name)] if self.router_bias else None
        if self.shared_size:
            sp = self.shared_prefix
            g, u = tensors[self.full_name(sp + "gate")], tensors[self.full_name(sp + "up")]
            if g.dtype != u.dtype:
                g, u = g.float(), u.float()
            self.shared_gate_up = torch.cat([g, u], dim=0).contiguous()
            self.shared_down = tensors[self.full_name(sp + "down")]
        gu = [torch.cat([tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]], dim=0) for e in range(E)]
        self.w_gate_up = torch.stack(gu, dim=0).to(self.rt.dtype).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in range(E)], dim=0).to(self.rt.dtype).contiguous()

    def weight_bytes(self) -> int:
        """What a decoded token reads: the router, `top` of the experts and the shared expert."""
        per_expert = (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size() // self.num_experts
        shared = sum(w.numel() * w.element_size() for w in (self.shared_gate_up, self.shared_down)) if self.shared_size else 0
        return self.w_router.numel() * 4 + (self.b_router.numel() * 4 if self.router_bias else 0) + self.top * per_expert + shared

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def forward(self, x, ctx):
        T = x.shape[0]
        ws = self.rt.workspace
        ids = ws.rows("moe_ids", T, self.top, torch.int32)
        weights = ws.rows("moe_weights", T, self.top, torch.float32)
        ops.route_topk(ids, weights, x, self.w_router, self.b_router, logistic=self.score == "sigmoid")
        y = ws.rows("ffn_out", T, self.hidden_size, x.dtype)
        ops.routed_experts(y, x, ids, weights, self.w_gate_up, self.w_down, workspace=ws,
                           kernel="rows" if self.rt.plain_kernels else "", weight_on_input=self.weight_on_input)
        if self.shared_size:
            gu = self._project(x, self.shared_gate_up, ws.rows("ffn_gate_up", T, 2 * self.shared_size, x.dtype), T)
            act = ops.swiglu(ws.rows("ffn_act", T, self.shared_size, x.dtype), gu)
            s = self._project(act, self.shared_down, ws.rows("ffn_shared", T, self.hidden_size, x.dtype), T)
            if ctx.extras.get("takes_two_outputs"):      # the block adds the two in float when it writes them to its stream
                return y, s
            ops.add_(y, s)
        return y


@register_part("ffn", "clamped_glu")
class ClampedGLU(FeedForward):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702,
                 gate_name: str = "gate", up_name: str = "up", down_name: str = "down"):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.alpha = float(limit), float(alpha)
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, I = self.hidden_size, self.intermediate_size
        return {self.full_name(self.gate_name): WeightSpec((I, D)), self.full_name(self.up_name): WeightSpec((I, D)),
                self.full_name(self.down_name): WeightSpec((D, I))}

    def bind(self, tensors) -> None:
        g, u = tensors[self.full_name(self.gate_name)], tensors[self.full_name(self.up_name)]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[self.full_name(self.down_name)]

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def forward(self, x, ctx):
        T = x.shape[0]
        ws = self.rt.workspace
        gu = self._project(x, self.w_gate_up, ws.rows("ffn_gate_up", T, 2 * self.intermediate_size, x.dtype), T)
        act = ops.glu_clamped(ws.rows("ffn_act", T, self.intermediate_size, x.dtype), gu, self.limit, self.alpha)
        return self._project(act, self.w_down, ws.rows("ffn_out", T, self.hidden_size, x.dtype), T)


@register_part("ffn", "routed_act")
class RoutedAct(FeedForward):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 scale: float = 1.0, activation: str = "relu2", shared_size: int = 0, router_name: str = "router",
                 expert_prefix: str = "e", shared_prefix: str = "shared."):
        super().__init__(runtime, prefix, names)
        if activation != "relu2":
            raise ValueError(f"activation '{activation}' is not built for ungated experts; built: relu2")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.num_experts, self.top, self.scale = int(num_experts), int(top), float(scale)
        if not (0 < self.top <= self.num_experts):
            raise ValueError(f"a token cannot use {self.top} of {self.num_experts} experts")
        self.shared_size = int(shared_size)
        self.router_name, self.expert_prefix, self.shared_prefix = router_name, expert_prefix, shared_prefix
        self.w_router = self.w_up = self.w_down = self.shared_up = self.shared_down = None

    def _expert(self, e: int, which: str) -> str:
        return self.full_name(f"{self.expert_prefix}{e}.{which}")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, I, E = self.hidden_size, self.intermediate_size, self.num_experts
        specs = {self.full_name(self.router_name): WeightSpec((E, D), role="vector")}
        for e in range(E):
            specs[self._expert(e, "up")] = WeightSpec((I, D))
            specs[self._expert(e, "down")] = WeightSpec((D, I))
        if self.shared_size:
            sp = self.shared_prefix
            specs[self.full_name(sp + "up")] = WeightSpec((self.shared_size, D))
            specs[self.full_name(sp + "down")] = WeightSpec((D, self.shared_size))
            specs[self.full_name(sp + "sg")] = WeightSpec((1, D), role="vector")
        return specs

    def bind(self, tensors) -> None:
        E = self.num_experts
        router = tensors[self.full_name(self.router_name)]
        self.w_up = torch.stack([tensors[self._expert(e, "up")] for e in range(E)], dim=0).to(self.rt.dtype).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in range(E)], dim=0).to(self.rt.dtype).contiguous()
        if self.shared_size:
            sp = self.shared_prefix
            router = torch.cat([router, tensors[self.full_name(sp + "sg")].reshape(1, -1)], dim=0)
            self.shared_up, self.shared_down = tensors[self.full_name(sp + "up")], tensors[self.full_name(sp + "down")]
        self.w_router = router.contiguous()

    def weight_bytes(self) -> int:
        """What a decoded token reads: the router, `top` of the experts and the shared expert."""
        per_expert = (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size() // self.num_experts
        shared = sum(w.numel() * w.element_size() for w in (self.shared_up, self.shared_down)) if self.shared_size else 0
        return self.w_router.numel() * 4 + self.top * per_expert + shared

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def forward(self, x, ctx):
        T = x.shape[0]
        ws = self.rt.workspace
        ids = ws.rows("moe_ids", T, self.top, torch.int32)
        weights = ws.rows("moe_weights", T, self.top, torch.float32)
        gate = ws.rows("moe_shared_gate", T, 1, torch.float32) if self.shared_size else None
        ops.route_topk(ids, weights, x, self.w_router, None, over_all=True, scale=self.scale, extra_out=gate)
        y = ws.rows("ffn_out", T, self.hidden_size, x.dtype)
        ops.routed_experts(y, x, ids, weights, self.w_up, self.w_down, workspace=ws, kernel="rows" if self.rt.plain_kernels else "",
                           gated=False)
        if self.shared_size:
            up = self._project(x, self.shared_up, ws.rows("ffn_up", T, self.shared_size, x.dtype), T)
            ops.bias_act(up, up, None, "relu2")
            s = self._project(up, self.shared_down, ws.rows("ffn_shared", T, self.hidden_size, x.dtype), T)
            ops.add_gated_rows(y, s, gate.view(-1))
        return y

"""A feed-forward made of many small gated experts of which every token uses a few, plus an optional expert that every
token uses.

Router: z = W_r x in float; the ``top`` experts with the largest z per token; an expert's weight is sigmoid(z), not
renormalised (``weighting`` = ``sigmoid``), and it multiplies what the expert *reads*, not what it returns
(``weight_on`` = ``input``):  y = shared(x) + sum over the chosen e of expert_e(w_e x), every expert being
down(silu(gate(h)) * up(h)) without biases.  On the device the (token, choice) pairs are sorted by expert into runs padded
to whole tiles, the weighted rows are gathered into that order, two grouped products and the gating run over the runs, and a
last kernel adds a token's rows and the shared expert's; nothing of it needs the host to know how many rows an expert got.
Parameters: ``hidden_size``, ``experts``, ``top``, ``expert_size`` (an expert's inner width), ``shared_size`` (the shared
expert's inner width, None for none), ``weighting``, ``weight_on``.  Tensors: router, e<i>.{gate,up,down}, shared.{gate,up,down}.

``scored_experts`` is the other family of routers: the scores are a softmax over *all* router outputs, s = softmax(W_r x); the choice is
made on s + correction (a stored vector that steers the load, not the weights), only inside the ``groups.keep`` groups of
neighbouring outputs (of ``groups.count`` equal groups) whose best choice score is largest, and the weight of a chosen output is its
plain score times ``scale``, not renormalised; it multiplies what the expert *returns*.  The last ``identity`` router outputs have no
matrices: such an expert returns what it read.  Experts are down(act(up(h))) without a gate and without biases.  A shared expert of
the same form runs for every token and is added times sigmoid(w_sg . x), one number per token.
    y = sigmoid(w_sg . x) shared(x) + sum over the chosen e of s_e * scale * (expert_e(x), or x for an identity expert)
Parameters: ``hidden_size``, ``experts`` (those with matrices), ``identity``, ``top``, ``expert_size``, ``activation``, ``scale``, ``group_count``
(0: no groups), ``group_keep``, ``shared_size`` (None for none).  Tensors: router [experts + identity, hidden], correction
[experts + identity], e<i>.{up,down}, shared.{up,down,sg}.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import moe
from .base import FEED_FORWARDS, BuildContext, FeedForward, WeightSpec, make, register_feed_forward
from .spec import PartSpec


class RoutedExperts(FeedForward):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.experts, self.top, self.inter = int(p["hidden_size"]), int(p["experts"]), int(p["top"]), int(p["expert_size"])
        if not 0 < self.top <= self.experts or self.experts > 1024:
            raise ValueError(f"{self.top} of {self.experts} experts: the router takes up to 1,024 experts and at least one of them per token")
        self.weighting, self.weight_on = str(p.get("weighting", "sigmoid")), str(p.get("weight_on", "input"))
        if self.weighting != "sigmoid" or self.weight_on != "input":
            raise ValueError("the router's weights are sigmoid scores that multiply an expert's input")
        self.shared = None
        if p.get("shared_size") is not None:
            self.shared = make(FEED_FORWARDS, PartSpec("swiglu", "", {"hidden_size": self.hidden, "intermediate_size": int(p["shared_size"]),
                                                                      "names": {"gate": "gate", "up": "up", "down": "down"}}), build)

    def weights(self) -> dict[str, WeightSpec]:
        wanted = {"router": WeightSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            wanted[f"e{e}.gate"] = WeightSpec((self.inter, self.hidden))
            wanted[f"e{e}.up"] = WeightSpec((self.inter, self.hidden))
            wanted[f"e{e}.down"] = WeightSpec((self.hidden, self.inter))
        if self.shared is not None:
            wanted.update({"shared." + name: spec for name, spec in self.shared.weights().items()})
        return wanted

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.router = tensors["router"].to(torch.float32).contiguous()
        # per expert [gate rows | up rows], all experts stacked: [experts, 2 * inter, hidden]; down: [experts, hidden, inter]
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0) for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.load({name: tensors["shared." + name] for name in self.shared.weights()})

    def kernel_modules(self):
        modules = [("moe", {}), ("elementwise", {})]
        if self.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0:
            modules.append(("moe_gemm_tcgen05", {}))
        return modules + (self.shared.kernel_modules() if self.shared is not None else [])

    def forward(self, x, step):
        chosen, weights = moe.route(x, self.router, self.top)
        where = moe.plan(chosen, weights, self.experts)
        rows = moe.gather(x, where)
        act = ops.swiglu(moe.grouped_linear(rows, self.w_gate_up, where))
        y = moe.grouped_linear(act, self.w_down, where)
        base = None
        if self.shared is not None:
            base = self.shared.forward(x, step)
            base = base.tensor() if hasattr(base, "tensor") else base
        return moe.combine(y, where, base, x.shape[0])


register_feed_forward("routed_experts", RoutedExperts)


class ScoredExperts(FeedForward):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.experts, self.identity = int(p["hidden_size"]), int(p["experts"]), int(p.get("identity") or 0)
        self.top, self.inter, self.scale = int(p["top"]), int(p["expert_size"]), float(p.get("scale", 1.0))
        self.activation = str(p.get("activation", "gelu_erf"))
        self.group_count, self.group_keep = int(p.get("group_count") or 0), int(p.get("group_keep") or 0)
        self.outputs = self.experts + self.identity
        if self.experts < 1 or self.outputs > 1024 or not 0 < self.top <= self.outputs:
            raise ValueError(f"{self.top} of {self.outputs} router outputs: the router takes up to 1,024 outputs, at least one expert with matrices and one choice per token")
        if self.group_count and (self.outputs % self.group_count or not 0 < self.group_keep <= self.group_count
                                 or self.top > self.group_keep * (self.outputs // self.group_count)):
            raise ValueError(f"{self.group_count} groups of which {self.group_keep} are kept do not fit {self.outputs} router outputs and {self.top} choices")
        if self.activation not in ("gelu_erf", "gelu_tanh"):
            raise ValueError(f"no activation {self.activation!r} (known: gelu_erf, gelu_tanh)")
        self.shared = None
        if p.get("shared_size") is not None:
            self.shared = make(FEED_FORWARDS, PartSpec("activated_mlp", "", {"hidden_size": self.hidden, "intermediate_size": int(p["shared_size"]),
                                                                             "activation": self.activation, "names": {"up": "up", "down": "down"}}), build)

    def weights(self) -> dict[str, WeightSpec]:
        wanted = {"router": WeightSpec((self.outputs, self.hidden)), "correction": WeightSpec((self.outputs,))}
        for e in range(self.experts):
            wanted[f"e{e}.up"] = WeightSpec((self.inter, self.hidden))
            wanted[f"e{e}.down"] = WeightSpec((self.hidden, self.inter))
        if self.shared is not None:
            wanted.update({"shared." + name: spec for name, spec in self.shared.weights().items()})
            wanted["shared.sg"] = WeightSpec((1, self.hidden))
        return wanted

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.router = tensors["router"].to(torch.float32).contiguous()
        self.correction = tensors["correction"].to(torch.float32).contiguous()
        self.w_up = torch.stack([tensors[f"e{e}.up"] for e in range(self.experts)]).contiguous()  # [experts, inter, hidden]
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).contiguous()  # [experts, hidden, inter]
        if self.shared is not None:
            self.shared.load({name: tensors["shared." + name] for name in self.shared.weights()})
            self.w_shared_gate = tensors["shared.sg"].contiguous()

    def kernel_modules(self):
        modules = [("moe", {}), ("elementwise", {})]
        if self.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0:
            modules.append(("moe_gemm_tcgen05", {}))
        return modules + (self.shared.kernel_modules() if self.shared is not None else [])

    def forward(self, x, step):
        chosen, weights = moe.route_scored(x, self.router, self.correction, self.top, self.group_count, self.group_keep, self.scale)
        where = moe.plan(chosen, None, self.experts)  # the weights multiply what an expert returns, so the rows are gathered as they are
        rows = moe.gather(x, where)
        act = getattr(ops, self.activation)(moe.grouped_linear(rows, self.w_up, where))
        y = moe.grouped_linear(act, self.w_down, where)
        base = gate = None
        if self.shared is not None:
            base = self.shared.forward(x, step)
            base = base.tensor() if hasattr(base, "tensor") else base
            gate = ops.linear(x, self.w_shared_gate, None, torch.float32).reshape(-1)
        return moe.combine_weighted(y, where, weights, x, base, gate)


register_feed_forward("scored_experts", ScoredExperts)

"""Gated feed-forward: f = W_down (act(W_gate x) * (W_up x)).

Reference: ``src/backend/bindless/sh_layer_v1.wgsl:1024-1070`` (gate and up),
``:1079`` (tanh-GELU), ``:1082`` (SiLU), ``:1104-1140`` (down).  The reference
picks the activation by a proxy (softcap > 0); here it is a parameter.

``routed_experts``: a mixture of small feed-forwards of which a token uses a
few.  The router's scores are sigmoids of its logits (32-bit), the ``top``
largest choose the experts, and a chosen expert's score multiplies the expert's
*input*: f = sum over the chosen e of E_e(s_e h), with E(h) = W_down (act(W_gate h,
W_up h)) and act(g, u) = g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit),
u' = clamp(u, -limit, limit).  A shared expert of the same form (own size and limit)
may run for every token; it is added times sigmoid(w_sg . h).  Nothing is read back
by the host: the pairs are sorted by expert on the device and the products walk
tiles of one expert's pairs, so a decode step can be captured.

Other designs' routers and experts are options of the same part.  The router may add
a learned correction to the scores *for the choice only*, may choose among the
experts of the best groups only (``groups`` equal groups of neighbours, a group's
score the sum of its two largest choice scores, the ``keep`` best kept), and may
divide the chosen scores by their sum and multiply them by a constant.  An expert
may be of one matrix and an activation, E(h) = W_down gelu(W_up h) with the exact
(erf) GELU (``expert`` = "gelu_erf"); its weight then multiplies the expert's
*output* (it is applied behind the activation, in front of the linear down product).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import WeightDecl
from .base import FeedForward, register_part
from .linear import PartialSums, WeightedSum, gated_linear, linear_split


@register_part("feed_forward", "gated_mlp")
class GatedMlp(FeedForward):
    """Parameters: ``hidden_size``, ``intermediate_size``, ``activation``
    (``gelu_tanh`` or ``silu``), ``gate_weight``/``up_weight``/``down_weight``; optional
    ``wide_output`` (default false): the down projection's result stays float32 on its way
    into the residual sum."""
    graph_safe = True


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.activation = self.param("activation")
        if self.activation not in kernels.ACTIVATIONS:
            raise ConfigError(f"gated_mlp: unknown activation '{self.activation}' "
                              f"(known: {sorted(kernels.ACTIVATIONS)})")
        self.names = [self.param(k) for k in ("gate_weight", "up_weight", "down_weight")]
        self.w_gu = None
        self.interleaved = False
        self.w_down = None

    def weight_decls(self):
        g, u, d = self.names
        return [WeightDecl(g, (self.inter, self.hidden)), WeightDecl(u, (self.inter, self.hidden)),
                WeightDecl(d, (self.hidden, self.inter))]

    def load(self, weights):
        g, u, d = self.names
        dt = self.ctx.compute_dtype
        wg, wu = weights[g].to(dt), weights[u].to(dt)
        # bfloat16 with a K the tensor-core product takes: gate and up rows interleaved per
        # tile, activation in the product's epilogue; else [gate; up] and a kernel of its own
        self.interleaved = dt == torch.bfloat16 and self.hidden % 8 == 0
        self.w_gu = (kernels.interleave_gate_up(wg, wu) if self.interleaved
                     else torch.cat([wg, wu], dim=0).contiguous())
        self.w_down = weights[d].to(dt).contiguous()

    def decode_bytes(self, lens) -> int:
        return 3 * self.hidden * self.inter * (4 if self.ctx.compute_dtype == torch.float32 else 2)

    def prefill_flops(self, lens) -> int:
        return 2 * sum(lens) * 3 * self.hidden * self.inter

    def forward(self, x, batch):
        h = gated_linear(x, self.w_gu, self.inter, self.activation, self.interleaved)
        return linear_split(h, self.w_down, wide=bool(self.params.get("wide_output", False)))


@register_part("feed_forward", "none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward: a block that knows of it leaves the
    sublayer and its norm out (``prenorm`` does)."""
    graph_safe = True
    present = False

    def forward(self, x, batch):
        raise ConfigError("a layer without a feed-forward was asked to run one (its block does not leave it out)")


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """Parameters: ``hidden_size``, ``intermediate_size``, ``num_experts``, ``top``, ``limit``,
    ``router_weight`` ([experts, hidden]) and ``expert_weights``: a pattern with ``{e}`` for the expert's number
    and ``{role}`` for gate / up / down; optional ``shared``: {``intermediate_size``, ``limit``,
    ``gate_weight``, ``up_weight``, ``down_weight``, ``mix_weight`` ([1, hidden])}.  Optional ``expert``:
    "clamped_glu" (the default, with ``limit``) or "gelu_erf" (up and down only; the weight on the output; no
    ``limit``).  Optional ``router``: {``correction_weight`` (tensor name, [experts]), ``groups``: {``count``,
    ``keep``}, ``normalise`` (bool), ``scale``}.  The result is a sum of 32-bit terms that the residual kernel takes."""
    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.n_experts = int(self.param("num_experts"))
        self.top = int(self.param("top"))
        self.expert = self.params.get("expert", "clamped_glu")
        if self.expert not in ("clamped_glu", "gelu_erf"):
            raise ConfigError(f"routed_experts: unknown expert '{self.expert}' (known: clamped_glu, gelu_erf)")
        self.gated = self.expert == "clamped_glu"
        self.limit = float(self.param("limit")) if self.gated else 0.0
        ro = self.params.get("router") or {}
        self.correction_name = ro.get("correction_weight")
        groups = ro.get("groups") or {}
        self.groups, self.keep = int(groups.get("count", 1)), int(groups.get("keep", 1))
        self.normalise = bool(ro.get("normalise", False))
        self.route_scale = float(ro.get("scale", 1.0))
        if self.groups < 1 or self.n_experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ConfigError(f"routed_experts: {self.n_experts} experts in {self.groups} groups of which {self.keep} are kept")
        if self.keep * (self.n_experts // self.groups) < self.top:
            raise ConfigError(f"routed_experts: the kept groups hold fewer than the {self.top} experts a token uses")
        if not 1 <= self.top <= self.n_experts:
            raise ConfigError(f"routed_experts: {self.top} of {self.n_experts} experts")
        self.router_name = self.param("router_weight")
        self.pattern = self.param("expert_weights")
        self.shared = self.params.get("shared")
        if self.shared is not None:
            missing = [k for k in ("intermediate_size", "limit", "gate_weight", "up_weight", "down_weight", "mix_weight")
                       if k not in self.shared]
            if missing:
                raise ConfigError(f"routed_experts: 'shared' needs {missing}")

    def _name(self, e: int, role: str) -> str:
        return self.pattern.format(e=e, role=role)

    def weight_decls(self):
        h, f = self.hidden, self.inter
        decls = [WeightDecl(self.router_name, (self.n_experts, h))]
        if self.correction_name:
            decls.append(WeightDecl(self.correction_name, (self.n_experts,), "norm"))
        for e in range(self.n_experts):
            if self.gated:
                decls.append(WeightDecl(self._name(e, "gate"), (f, h)))
            decls += [WeightDecl(self._name(e, "up"), (f, h)), WeightDecl(self._name(e, "down"), (h, f))]
        if self.shared is not None:
            sf, sh = int(self.shared["intermediate_size"]), self.shared
            decls += [WeightDecl(sh["gate_weight"], (sf, h)), WeightDecl(sh["up_weight"], (sf, h)),
                      WeightDecl(sh["down_weight"], (h, sf)), WeightDecl(sh["mix_weight"], (1, h))]
        return decls

    def load(self, weights):
        dt = self.ctx.compute_dtype
        E = range(self.n_experts)
        self.w_gate = (torch.stack([weights[self._name(e, "gate")] for e in E]).to(dt).contiguous()
                       if self.gated else None)
        self.correction = (weights[self.correction_name].to(torch.float32).contiguous()
                           if self.correction_name else None)
        self.w_up = torch.stack([weights[self._name(e, "up")] for e in E]).to(dt).contiguous()
        self.w_down = torch.stack([weights[self._name(e, "down")] for e in E]).to(dt).contiguous()
        rows = [weights[self.router_name]]
        if self.shared is not None:
            sh = self.shared
            rows.append(weights[sh["mix_weight"]].reshape(1, self.hidden))       # the shared expert's gate rides with the router
            self.s_gate = weights[sh["gate_weight"]].to(dt).unsqueeze(0).contiguous()
            self.s_up = weights[sh["up_weight"]].to(dt).unsqueeze(0).contiguous()
            self.s_down = weights[sh["down_weight"]].to(dt).unsqueeze(0).contiguous()
        self.router = torch.cat(rows, dim=0).to(torch.float32).contiguous()      # (router logits are 32-bit)

    def _el(self) -> int:
        return 4 if self.ctx.compute_dtype == torch.float32 else 2

    def decode_bytes(self, lens) -> int:
        # the experts whose matrices are read: the expected number under a router that chooses evenly
        used = self.n_experts * (1.0 - (1.0 - self.top / self.n_experts) ** len(lens))
        mats = 3 if self.gated else 2
        total = int(mats * used * self.hidden * self.inter * self._el()) + 4 * self.router.numel()
        if self.shared is not None:
            total += 3 * self.hidden * int(self.shared["intermediate_size"]) * self._el()
        return total

    def prefill_flops(self, lens) -> int:
        per_token = (3 if self.gated else 2) * self.hidden * self.inter * self.top + self.router.numel()
        if self.shared is not None:
            per_token += 3 * self.hidden * int(self.shared["intermediate_size"])
        return 2 * sum(lens) * per_token

    def forward(self, x, batch):
        T, top, dev = x.shape[0], self.top, x.device
        ids = torch.empty(T, top, dtype=torch.int32, device=dev)
        wts = torch.empty(T, top, dtype=torch.float32, device=dev)
        mix = torch.empty(T, dtype=torch.float32, device=dev) if self.shared is not None else None
        kernels.expert_route(ids, wts, mix, x, self.router, self.n_experts, correction=self.correction,
                             groups=self.groups, keep=self.keep, normalise=self.normalise, out_scale=self.route_scale)
        # bfloat16 with sizes the tensor-core products take: the rows in sorted order, then grouped products;
        # else the products on the CUDA cores (32-bit, or odd sizes), which fetch their rows themselves
        fast = (kernels.expert_rows_tc_supported(x, self.w_up) and self.inter % 8 == 0)
        act = None if self.gated else "gelu_erf"
        tile = kernels.expert_tc_tile(T * top, self.n_experts) if fast else kernels.EXPERT_TILE
        perm = torch.empty(T * top, dtype=torch.int32, device=dev)
        plan = torch.empty(1 + 3 * kernels.expert_max_tiles(T * top, self.n_experts, tile), dtype=torch.int32, device=dev)
        kernels.expert_plan(perm, plan, ids, self.n_experts, tile)
        mid = torch.empty(T * top, self.inter, dtype=x.dtype, device=dev)
        out = torch.empty(top, T, self.hidden, dtype=torch.float32, device=dev)
        if fast:
            rows = torch.empty(T * top, self.hidden, dtype=x.dtype, device=dev)
            kernels.expert_gather(rows, x, perm, top)
            if self.gated:
                kernels.expert_rows_tc(mid, rows, self.w_gate, self.w_up, perm=perm, plan=plan, pair_weight=wts,
                                       n_tokens=T, top=top, limit=self.limit, tile=tile)
            else:
                kernels.expert_rows_tc(mid, rows, self.w_up, perm=perm, plan=plan, pair_weight=wts, n_tokens=T, top=top,
                                       tile=tile, act=act)
            kernels.expert_rows_tc(out, mid, self.w_down, perm=perm, plan=plan, n_tokens=T, top=top, tile=tile)
        else:
            if self.gated:
                kernels.expert_rows(mid, x, self.w_gate, self.w_up, perm=perm, plan=plan, pair_weight=wts, n_tokens=T,
                                    top=top, limit=self.limit)
            else:
                kernels.expert_rows(mid, x, self.w_up, perm=perm, plan=plan, pair_weight=wts, n_tokens=T, top=top, act=act)
            kernels.expert_rows(out, mid, self.w_down, perm=perm, plan=plan, n_tokens=T, top=top)
        terms = [(PartialSums(out), 1.0)]
        if self.shared is not None:
            sf = int(self.shared["intermediate_size"])
            smid = torch.empty(T, sf, dtype=x.dtype, device=dev)
            sout = torch.empty(1, T, self.hidden, dtype=torch.float32, device=dev)
            rows_fn = kernels.expert_rows_tc if fast and sf % 8 == 0 else kernels.expert_rows
            rows_fn(smid, x, self.s_gate, self.s_up, scale_out=mix, n_tokens=T, top=1, limit=float(self.shared["limit"]))
            rows_fn(sout, smid, self.s_down, n_tokens=T, top=1)
            terms.append((sout[0], 1.0))
        return WeightedSum(terms)

"""The gated delta rule mixer: a linear recurrence whose state is corrected towards each token's value.

With G query/key heads of size ``dim`` serving H value heads of size ``vdim`` (value head a reads query/key head
a // (H / G)) and S_a [dim, vdim] zero when a request starts:

    q, k, v   = silu(conv(W h))           a short causal convolution over time, one filter per channel
    q <- q / sqrt(sum q^2 + 1e-6) * dim^(-1/2),   k <- k / sqrt(sum k^2 + 1e-6)          per head
    beta_a    = sigmoid(W_b h)_a
    decay_a   = exp(-exp(A_log_a) * softplus(W_a2 (W_a1 h) + dt_bias))_a                 [dim] per head
    S_a <- diag(decay_a) S_a;   u = beta_a (v_a - S_a^T k);   S_a <- S_a + k u^T;   o_a = S_a^T q
    out_a     = out_scale * o_a / sqrt(mean(o_a^2) + eps) * w * sigmoid(W_g2 (W_g1 h))_a  [vdim] per head

and the heads' results go through the output projection.  Per request the mixer keeps the last taps - 1 rows of
the q | k | v projection and the matrices S_a, both float32, in state slots.  One product gives
q | k | v | b | W_a1 h | W_g1 h in float32 (what enters the recurrence stays float from the accumulator on); the
two low-rank expansions, the gates, the norms and the recurrence are float arithmetic in the kernels.  The ranks
of the low-rank pairs are read from the tensors.

``low_rank`` False gives the plainer form of the same mixer: one decay per head and token,
decay_a = exp(-exp(A_log_a) * softplus((W_a h)_a + dt_bias_a)) with W_a [heads, hidden] and dt_bias [heads], and an
output gate from a full projection W_g [heads * vdim, hidden]; ``gate_act`` "silu" makes the gate z * sigmoid(z).
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from .. import ops
from ..weights.spec import GAIN, MATRIX, VECTOR, ParamSpec
from .base import MIXERS, Delta, Mixer, StateSpec


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """names: matrices {"q","k","v","b","a1","a2","g1","g2","o"} ([out, in]; "<q|k|v>.conv" are their filters
    [channels, taps]), vectors {"A_log" [heads], "dt_bias" [heads * dim]}, and "norm" [vdim].  ``rank``: the
    low-rank pairs' inner size when weights are made at random (a checkpoint's own is taken as it is)."""

    def __init__(self, hidden: int, num_heads: int, num_qk_heads: int, dim: int, vdim: int, conv_taps: int, eps: float,
                 names: Dict[str, str], out_scale: float = 1.0, float_out: bool = False, rank: int = 16,
                 low_rank: bool = True, gate_act: str = "sigmoid"):
        if num_heads % num_qk_heads:
            raise ValueError(f"{num_heads} value heads cannot share {num_qk_heads} query/key heads")
        if conv_taps < 1:
            raise ValueError("a convolution needs at least one tap")
        if gate_act not in ("sigmoid", "silu"):
            raise ValueError("the output gate is 'sigmoid' or 'silu'")
        self.low_rank, self.gate_silu = bool(low_rank), gate_act == "silu"
        self.hidden, self.H, self.G, self.dim, self.vdim = hidden, num_heads, num_qk_heads, dim, vdim
        self.taps, self.eps, self.names = int(conv_taps), float(eps), dict(names)
        self.out_scale, self.float_out, self.rank = float(out_scale), bool(float_out), int(rank)
        self.channels = 2 * self.G * dim + self.H * vdim
        self.w_in = self.w_o = self.conv_w = self.w_a2 = self.w_g2 = None
        self.a_log = self.dt_bias = self.norm_w = None
        self.rank_a = self.rank_g = 0

    def param_specs(self) -> List[ParamSpec]:
        n, W, any_rank = self.names, self.hidden, -self.rank
        qk, vw = self.G * self.dim, self.H * self.vdim
        specs = []
        for key, rows in (("q", qk), ("k", qk), ("v", vw)):
            specs.append(ParamSpec(n[key], (rows, W), MATRIX))
            specs.append(ParamSpec(n[key] + ".conv", (rows, self.taps), VECTOR))
        specs.append(ParamSpec(n["b"], (self.H, W), MATRIX))
        if self.low_rank:
            specs += [ParamSpec(n["a1"], (any_rank, W), MATRIX), ParamSpec(n["a2"], (self.H * self.dim, any_rank), MATRIX),
                      ParamSpec(n["g1"], (any_rank, W), MATRIX), ParamSpec(n["g2"], (vw, any_rank), MATRIX),
                      ParamSpec(n["dt_bias"], (self.H * self.dim,), VECTOR)]
        else:
            specs += [ParamSpec(n["a"], (self.H, W), MATRIX), ParamSpec(n["g"], (vw, W), MATRIX),
                      ParamSpec(n["dt_bias"], (self.H,), VECTOR)]
        specs += [ParamSpec(n["A_log"], (self.H,), VECTOR), ParamSpec(n["norm"], (self.vdim,), GAIN),
                  ParamSpec(n["o"], (W, vw), MATRIX)]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        if self.low_rank:
            a1, g1 = tensors.pop(n["a1"]), tensors.pop(n["g1"])
            self.w_a2, self.w_g2 = tensors.pop(n["a2"]).contiguous(), tensors.pop(n["g2"]).contiguous()
            self.rank_a, self.rank_g = a1.shape[0], g1.shape[0]
            if self.w_a2.shape[1] != self.rank_a or self.w_g2.shape[1] != self.rank_g:
                raise ValueError(f"the low-rank pairs of '{n['a1']}' / '{n['g1']}' do not agree in their inner size")
        else:
            # the projection's columns hold the decay logits and the gate logits themselves
            a1, g1 = tensors.pop(n["a"]), tensors.pop(n["g"])
            self.rank_a, self.rank_g = a1.shape[0], g1.shape[0]
        self.w_in = torch.cat([tensors.pop(n["q"]), tensors.pop(n["k"]), tensors.pop(n["v"]), tensors.pop(n["b"]),
                               a1, g1], dim=0).contiguous()
        self.conv_w = torch.cat([tensors.pop(n[k] + ".conv") for k in "qkv"], dim=0).to(torch.float32).contiguous()
        self.w_o = tensors.pop(n["o"])
        self.a_log, self.dt_bias, self.norm_w = tensors[n["A_log"]], tensors[n["dt_bias"]], tensors[n["norm"]]

    def cache_spec(self):
        # the convolution's last inputs (all q | k | v channels), and the state matrices
        return (StateSpec((self.taps - 1, self.channels), torch.float32),
                StateSpec((self.H, self.dim, self.vdim), torch.float32))

    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        tails, mats = cache
        n = h.shape[0]
        proj = ops.linear(h, self.w_in, out_dtype=torch.float32)
        b_off = self.channels
        a_off = b_off + self.H
        g_off = a_off + self.rank_a
        single = bool(getattr(ctx, "single_tokens", False))
        o = torch.empty((n, self.H * self.vdim), dtype=h.dtype, device=h.device)
        scratch = ctx.scratch_f32(ops.delta_rule_scratch(n, self.H, self.G, self.dim, self.vdim))
        ops.delta_rule(proj, b_off, a_off, g_off, self.conv_w, tails.state, self.w_a2, self.a_log, self.dt_bias,
                       self.w_g2, self.norm_w, self.eps, self.out_scale, mats.state, mats.writable, single, scratch, o,
                       ctx.positions, ctx.seq_of_token, ctx.q_start, ctx.slots, ctx.n_seqs, self.H, self.G, self.dim,
                       self.vdim, gate_silu=self.gate_silu)
        if self.taps > 1 and tails.writable and not (single and mats.writable):
            ops.conv_state_update(proj, self.channels, tails.state, ctx.positions, ctx.q_start, ctx.slots, ctx.n_seqs)
        return Delta(ops.linear(o, self.w_o, out_dtype=torch.float32 if self.float_out else None))

    def param_bytes(self) -> int:
        low = (self.w_a2.numel() + self.w_g2.numel()) if self.low_rank else 0
        return (self.w_in.numel() + self.w_o.numel() + low) * self.w_in.element_size()

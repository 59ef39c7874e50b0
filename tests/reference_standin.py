"""A stand-in for the reference's MoE block (my_inkling/model.py:169-374) for machines
without a checkout of the reference: modules with the SAME attribute names, parameter
shapes and forward signatures as MyInklingTopkRouter, MyInklingExperts,
MyInklingSharedExperts and MyInklingMoE, so that `apply_resident_plan` and
`apply_fused_moe_plan` meet what they would meet in the reference's model. Written from
the interface, not copied; tests/test_dropin_names.py checks it against the real classes
wherever the checkout is present. Test infrastructure only."""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class StandInConfig:
    hidden_size: int
    moe_intermediate_size: int
    n_routed_experts: int
    num_experts_per_tok: int
    n_shared_experts: int
    route_scale: float = 8.0


class StandInRouter(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.num_experts, self.n_shared_experts = c.n_routed_experts, c.n_shared_experts
        self.route_scale, self.top_k = c.route_scale, c.num_experts_per_tok
        self.weight = nn.Parameter(torch.empty(self.num_experts + self.n_shared_experts, c.hidden_size))
        self.global_scale = nn.Parameter(torch.ones(1))
        self.e_score_correction_bias = nn.Buffer(torch.zeros(self.num_experts))

    def forward(self, hidden_states):
        logits = F.linear(hidden_states.flatten(0, -2), self.weight)
        ns = self.n_shared_experts
        choice = logits.sigmoid()[..., :-ns] + self.e_score_correction_bias
        indices = torch.topk(choice, self.top_k, dim=-1, sorted=False)[1]
        picked = torch.cat([logits[..., :-ns].gather(-1, indices), logits[..., -ns:]], dim=-1)
        log_p = F.logsigmoid(picked)
        w = torch.exp(log_p - torch.logsumexp(log_p, dim=-1, keepdim=True)) * self.route_scale * self.global_scale
        return logits[..., :-ns], w[..., : self.top_k].contiguous(), indices, w[..., -ns:].contiguous()


class StandInExperts(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.num_experts, self.hidden_dim, self.intermediate_dim = c.n_routed_experts, c.hidden_size, c.moe_intermediate_size
        self.gate_up_proj = nn.Parameter(torch.empty(self.num_experts, 2 * self.intermediate_dim, self.hidden_dim))
        self.down_proj = nn.Parameter(torch.empty(self.num_experts, self.hidden_dim, self.intermediate_dim))

    def forward(self, hidden_states, top_k_index, top_k_weights):
        out = torch.zeros_like(hidden_states)
        for e in torch.unique(top_k_index).tolist():
            tokens, slots = torch.where(top_k_index == e)
            gate, up = F.linear(hidden_states[tokens], self.gate_up_proj[e]).chunk(2, dim=-1)
            y = F.linear(F.silu(gate) * up, self.down_proj[e]) * top_k_weights[tokens, slots, None]
            out.index_add_(0, tokens, y.to(out.dtype))
        return out


class StandInSharedExperts(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.n_shared_experts = c.n_shared_experts
        shape = (c.n_shared_experts, c.moe_intermediate_size, c.hidden_size)
        self.gate_proj, self.up_proj = nn.Parameter(torch.empty(shape)), nn.Parameter(torch.empty(shape))
        self.down_proj = nn.Parameter(torch.empty(c.n_shared_experts, c.hidden_size, c.moe_intermediate_size))

    def forward(self, hidden_states, gammas):
        flat = hidden_states.flatten(0, -2).unsqueeze(0).expand(self.n_shared_experts, -1, -1)
        gate = torch.bmm(flat, self.gate_proj.transpose(1, 2))
        up = torch.bmm(flat, self.up_proj.transpose(1, 2))
        act = F.silu(gate) * up * gammas.T.unsqueeze(-1)
        down = torch.bmm(act, self.down_proj.transpose(1, 2))
        return down.float().sum(0).to(hidden_states.dtype).view(hidden_states.shape)


class StandInMoE(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.gate, self.experts, self.shared_experts = StandInRouter(c), StandInExperts(c), StandInSharedExperts(c)

    def forward(self, hidden_states):
        shape = hidden_states.shape
        _, w, idx, gammas = self.gate(hidden_states)
        routed = self.experts(hidden_states.reshape(-1, shape[-1]), idx, w).view(*shape)
        return routed + self.shared_experts(hidden_states, gammas=gammas)


def reference_root() -> Path | None:
    for candidate in (os.environ.get("INKLING_REFERENCE_ROOT"), Path(__file__).resolve().parents[2] / "reference"):
        if candidate and (Path(candidate) / "my_inkling" / "model.py").exists():
            return Path(candidate)
    return None


def moe_classes():
    """(config factory, MoE class, 'reference' | 'stand-in'): the reference's own classes
    where a checkout is present, the stand-in elsewhere."""
    root = reference_root()
    if root is not None:
        if str(root) not in sys.path:
            sys.path.insert(0, str(root))
        from my_inkling import model as ref

        def config(d, f, experts, top_k, n_shared, route_scale=8.0):
            return ref.InklingTextConfig(hidden_size=d, vocab_size=32, num_hidden_layers=1, pad_token_id=0,
                                         moe_intermediate_size=f, n_routed_experts=experts,
                                         num_experts_per_tok=top_k, n_shared_experts=n_shared, route_scale=route_scale)
        return config, ref.MyInklingMoE, "reference"

    def config(d, f, experts, top_k, n_shared, route_scale=8.0):
        return StandInConfig(d, f, experts, top_k, n_shared, route_scale)
    return config, StandInMoE, "stand-in"

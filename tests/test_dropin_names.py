"""The stand-in MoE block used by the GPU drop-in test has the attribute names, parameter
shapes and results of the reference's own classes (checked wherever a checkout of the
reference is present; the GPU box has none and relies on this check having run)."""
import pytest
import torch

import cases
import reference_standin as rs
from oracle import nvfp4


def _load(moe, p, banks):
    with torch.no_grad():
        moe.gate.e_score_correction_bias = moe.gate.e_score_correction_bias.float()
        moe.gate.weight.copy_(p["router_weight"])
        moe.gate.global_scale.copy_(p["global_scale"])
        moe.gate.e_score_correction_bias.copy_(p["router_bias"])
        moe.shared_experts.gate_proj.copy_(p["shared_gate"])
        moe.shared_experts.up_proj.copy_(p["shared_up"])
        moe.shared_experts.down_proj.copy_(p["shared_down"])
        for e, b in banks.items():
            gu = nvfp4.dequant_bf16(b["gate_up_proj"], b["gate_up_proj_scale"], b["gate_up_proj_scale2"])
            moe.experts.gate_up_proj[e].copy_(torch.cat([gu[0::2], gu[1::2]]))
            moe.experts.down_proj[e].copy_(nvfp4.dequant_bf16(b["down_proj"], b["down_proj_scale"], b["down_proj_scale2"]))
    return moe


def test_stand_in_mirrors_the_reference_block():
    if rs.reference_root() is None:
        pytest.skip("no checkout of the reference on this machine")
    config, real_cls, kind = rs.moe_classes()
    assert kind == "reference"
    c = cases.LAYER_CASES["small"]
    p, banks, x = cases.make_layer(**c)
    real = _load(real_cls(config(c["d"], c["f"], c["experts"], c["top_k"], c["n_shared"])).bfloat16().eval(), p, banks)
    mine = _load(rs.StandInMoE(rs.StandInConfig(c["d"], c["f"], c["experts"], c["top_k"], c["n_shared"])).bfloat16().eval(),
                 p, banks)
    real_state = {k: tuple(v.shape) for k, v in real.state_dict().items()}
    mine_state = {k: tuple(v.shape) for k, v in mine.state_dict().items()}
    assert real_state == mine_state
    for child, attrs in (("gate", ("route_scale", "top_k", "num_experts", "n_shared_experts")),
                         ("experts", ("hidden_dim", "intermediate_dim", "num_experts")),
                         ("shared_experts", ("n_shared_experts",))):
        for attr in attrs:
            assert getattr(getattr(real, child), attr) == getattr(getattr(mine, child), attr), (child, attr)
    with torch.no_grad():
        want, got = real(x.unsqueeze(0)), mine(x.unsqueeze(0))
    assert torch.equal(want, got)

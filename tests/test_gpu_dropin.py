"""The drop-in under the reference's own caller: a model whose decoder layer holds the
reference's MoE block (my_inkling/model.py:353-374; the stand-in of
tests/reference_standin.py where no checkout is present) gets its routed experts replaced by
`apply_resident_plan`, or the whole block by `apply_fused_moe_plan` -- the way
apply_offload_plan does it (my_inkling/offloaded_experts.py:317-340) -- and must return what
the untouched block returns on the same weights, eagerly and under the warm-up + capture
sequence of my_inkling/decode_graph.py:22-41."""
import copy

import pytest
import torch
from torch import nn

import cases
import reference_standin as rs
from helpers import BF16, assert_router_matches, banks_to_device, max_rel
from oracle import moe as oracle_moe
from test_dropin_names import _load

pytestmark = pytest.mark.gpu
TOL = 2e-2
NAME = "layers.0.mlp.experts"


@pytest.fixture(scope="module")
def ib():
    import inkling_b200

    return inkling_b200


@pytest.fixture(scope="module")
def device():
    return torch.device("cuda", 0)


class _Layer(nn.Module):
    def __init__(self, mlp):
        super().__init__()
        self.mlp = mlp


class _Model(nn.Module):
    """Only the nesting matters: `layers.<i>.mlp` is the MoE block, as in the reference's text tower."""

    def __init__(self, mlp):
        super().__init__()
        self.layers = nn.ModuleList([_Layer(mlp)])

    def forward(self, hidden_states):
        return self.layers[0].mlp(hidden_states)


def _build(device, case="mid"):
    c = cases.LAYER_CASES[case]
    p, banks, x = cases.make_layer(**dict(c, tokens=12))
    config, moe_cls, kind = rs.moe_classes()
    moe = _load(moe_cls(config(c["d"], c["f"], c["experts"], c["top_k"], c["n_shared"])).bfloat16().eval(), p, banks)
    return c, p, banks, x, _Model(moe).to(device).eval(), kind


def _capture_like_decode_graph(model, token):
    """my_inkling/decode_graph.py:22-41: three eager steps on a side stream, then capture."""
    static_in = token.clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream), torch.inference_mode():
        for _ in range(3):
            out = model(static_in)
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream), torch.inference_mode():
        out = model(static_in)
    torch.cuda.synchronize()
    return graph, static_in, out


@pytest.mark.parametrize("plan", ["resident", "fused"])
def test_block_with_the_drop_in_matches_the_untouched_block(ib, device, plan):
    c, p, banks, x, model, kind = _build(device)
    state = {NAME: banks_to_device(banks, device)}
    swapped = copy.deepcopy(model)
    if plan == "resident":
        ib.apply_resident_plan(swapped, None, state)
        assert isinstance(swapped.layers[0].mlp.experts, ib.ResidentExperts)
        assert type(swapped.layers[0].mlp) is type(model.layers[0].mlp)          # the reference's block, unchanged
    else:
        ib.apply_fused_moe_plan(swapped, None, state)
        assert isinstance(swapped.layers[0].mlp, ib.FusedMoE)
    with torch.inference_mode():
        for tokens in (1, 5, 12):                                                 # one token, a GEMV batch, the grouped path
            xs = x[:tokens].to(device).unsqueeze(0)
            want = model(xs)
            got = swapped(xs)
            torch.cuda.synchronize()
            assert got.shape == want.shape and got.dtype == want.dtype
            same = torch.ones(tokens, dtype=torch.bool)
            if plan == "fused":
                # the block's own router runs here too: tokens on which it and the untouched block's torch.topk
                # pick different sets (a score tie or a logit on a BF16 rounding boundary) are compared with the
                # oracle only, the others with the untouched block as well
                mlp = swapped.layers[0].mlp
                idx, w, gam = (t[:tokens].cpu() for t in (mlp.topk_indices, mlp.topk_weights, mlp.gammas))
                assert_router_matches(p, x[:tokens], idx, w, gam)
                assert max_rel(got[0].float(), oracle_moe.moe_layer_fp32(x[:tokens], p, banks, idx, w, gam)) <= TOL
                theirs = model.layers[0].mlp.gate(xs)[2].cpu()
                same = (theirs.sort(-1).values == idx.sort(-1).values).all(-1)
                assert int(same.sum()) >= tokens - 2
            # the untouched block multiplies BF16-dequantised weights with torch's BF16 GEMMs: same bar as the oracle
            assert max_rel(got[0][same].float(), want[0][same].float()) <= TOL, (kind, plan, tokens)
    experts = swapped.layers[0].mlp.experts
    experts.check_status()


@pytest.mark.parametrize("plan", ["resident", "fused"])
def test_replay_equals_eager_under_the_reference_capture_sequence(ib, device, plan):
    c, p, banks, x, model, kind = _build(device)
    state = {NAME: banks_to_device(banks, device)}
    (ib.apply_resident_plan if plan == "resident" else ib.apply_fused_moe_plan)(model, None, state)
    token = x[:1].to(device).unsqueeze(0)
    graph, static_in, out = _capture_like_decode_graph(model, token)
    for i in range(1, 4):
        static_in.copy_(x[i:i + 1].to(device).unsqueeze(0))
        graph.replay()
        replayed = out.clone()
        torch.cuda.synchronize()
        with torch.inference_mode():
            eager = model(static_in).clone()
        torch.cuda.synchronize()
        assert torch.equal(replayed, eager)
    model.layers[0].mlp.experts.check_status()


def test_banks_packed_by_the_loader_take_the_block_scaled_kernel(ib, device):
    """The rank's records under the reference's naming -> `pack_resident_experts` -> `apply_resident_plan`: the banks of
    one kind sit in one allocation, so the grouped path gets its TMA descriptors (tcgen05 block-scaled kernel) and the
    block still returns what the untouched block returns."""
    from inkling_b200.loader import pack_resident_experts

    c, p, banks, x, model, kind = _build(device)
    records = {f"{NAME}.{name}/{e}": tensor for e, bank in banks.items() for name, tensor in bank.items()}
    state = pack_resident_experts(records, device)
    swapped = copy.deepcopy(model)
    ib.apply_resident_plan(swapped, None, state)
    experts = swapped.layers[0].mlp.experts
    assert isinstance(experts, ib.ResidentExperts) and experts.bank_maps is not None
    with torch.inference_mode():
        for tokens in (1, 12):
            xs = x[:tokens].to(device).unsqueeze(0)
            want, got = model(xs), swapped(xs)
            torch.cuda.synchronize()
            assert max_rel(got[0].float(), want[0].float()) <= TOL, (kind, tokens)
    experts.check_status()

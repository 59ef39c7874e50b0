"""The resident packer: records under the reference's naming -> one allocation per (layer, bank
kind), per-expert views evenly spaced (what the TMA descriptors of the tensor-core kernels need)."""
import torch

import cases
import inkling_b200 as ib
from inkling_b200.loader import pack_resident_experts, split_record_name


def test_record_names_follow_the_reference():
    assert split_record_name("model.layers.7.mlp.experts.gate_up_proj_scale/12") == (
        "model.layers.7.mlp.experts", "gate_up_proj_scale", 12)


def test_banks_of_one_kind_end_up_evenly_spaced():
    records, originals = {}, {}
    for layer in (3, 4):
        gen = torch.Generator().manual_seed(layer)
        banks = cases.make_expert_banks(gen, 5, 128, 64)
        for e, bank in banks.items():
            for name, tensor in bank.items():
                key = f"model.layers.{layer}.mlp.experts.{name}/{e + 8}"      # this rank's experts start at id 8
                records[key] = tensor.view(torch.float8_e4m3fn) if name.endswith("_scale") else tensor
                originals[key] = tensor
    state = pack_resident_experts(records, "cpu")
    assert sorted(state) == ["model.layers.3.mlp.experts", "model.layers.4.mlp.experts"]
    for module, experts in state.items():
        assert sorted(experts) == list(range(8, 13))
        for e, bank in experts.items():
            assert sorted(bank) == sorted(cases.BANK_NAMES)
            for name, tensor in bank.items():
                want = originals[f"{module}.{name}/{e}"]
                assert torch.equal(tensor.reshape(-1).view(torch.uint8), want.reshape(-1).contiguous().view(torch.uint8))
        kinds = ("gate_up_proj", "gate_up_proj_scale", "down_proj", "down_proj_scale")
        addresses = [[experts[e][n].data_ptr() for e in sorted(experts)] for n in kinds]
        sizes = [experts[8][n].numel() * experts[8][n].element_size() for n in kinds]
        layout = ib.ResidentExperts._even_spacing(addresses, sizes)
        assert layout is not None and all(stride == size for (_, stride), size in zip(layout, sizes))

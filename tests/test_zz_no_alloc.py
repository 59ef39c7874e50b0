"""The router entry point that allocates nothing (ink_router_forward_static), called
through the C ABI, against the ordinary entry point (ink_router_forward) on the same
inputs. Some callers cannot allocate device memory at call time -- they run inside an
allocator hook, under a memory plan frozen at start-up, or on a thread that must not
touch the allocator -- so this variant keeps its scratch in an array inside the library.
Two calls in a row with different inputs check that the second call is not confused by
what the first one left in that shared array. This file is collected last on purpose."""
import ctypes

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _call(lib, fn_name, p, x, device, workspace=None):
    t, k, ns = x.shape[0], p["top_k"], p["n_shared"]
    xd, wd = x.to(device), p["router_weight"].to(device)
    bias, gs = p["router_bias"].to(device), p["global_scale"].to(device)
    logits = torch.empty(t, p["experts"], dtype=BF16, device=device)
    weights = torch.empty(t, k, dtype=BF16, device=device)
    indices = torch.full((t, k), -1, dtype=torch.int64, device=device)
    gammas = torch.empty(t, ns, dtype=BF16, device=device)
    stream = torch.cuda.current_stream().cuda_stream
    args = [xd.data_ptr(), wd.data_ptr(), bias.data_ptr(), gs.data_ptr(), ctypes.c_float(p["route_scale"]), t,
            x.shape[1], p["experts"], ns, k, logits.data_ptr(), weights.data_ptr(), indices.data_ptr(),
            gammas.data_ptr()]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel()]
    rc = getattr(lib, fn_name)(*args, stream)
    assert rc == 0, lib.ink_last_error().decode()
    torch.cuda.synchronize()
    return logits, weights, indices, gammas


def test_static_scratch_router_matches_the_ordinary_one_twice_in_a_row():
    import inkling_b200
    from inkling_b200.kernels import _abi

    lib = _abi.lib()
    device = torch.device("cuda", 0)
    # two different problems back to back: 3 tokens over 16 experts, then 8 tokens over 256 experts
    first = cases.make_layer(**cases.LAYER_CASES["small"])
    gen = torch.Generator().manual_seed(21)
    big = dict(experts=256, n_shared=2, top_k=6, route_scale=8.0)
    big["router_weight"] = (torch.randn(258, 4096, generator=gen) * 0.02).to(BF16)
    big["router_bias"] = torch.randn(256, generator=gen) * 0.05
    big["global_scale"] = torch.full((1,), 1.3).to(BF16)
    big_x = torch.randn(8, 4096, generator=gen).to(BF16)
    for p, x in ((first[0], first[2]), (big, big_x), (first[0], first[2])):
        workspace = inkling_b200.kernels.router_workspace(x.shape[0], p["experts"] + p["n_shared"], device)
        want = _call(lib, "ink_router_forward", p, x, device, workspace)
        got = _call(lib, "ink_router_forward_static", p, x, device)
        for g, w in zip(got, want):
            assert torch.equal(g, w)   # same kernel, same arithmetic: bit-exact


def test_static_scratch_router_refuses_what_does_not_fit():
    from inkling_b200.kernels import _abi

    lib = _abi.lib()
    device = torch.device("cuda", 0)
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["small"])
    x9 = x[:1].repeat(9, 1)
    t, k, ns = 9, p["top_k"], p["n_shared"]
    dummy = torch.empty(t * 256, dtype=BF16, device=device)
    idx = torch.empty(t, k, dtype=torch.int64, device=device)
    rc = lib.ink_router_forward_static(
        x9.to(device).data_ptr(), p["router_weight"].to(device).data_ptr(), p["router_bias"].to(device).data_ptr(),
        p["global_scale"].to(device).data_ptr(), ctypes.c_float(8.0), t, x.shape[1], p["experts"], ns, k, None,
        dummy.data_ptr(), idx.data_ptr(), dummy.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc < 0 and b"at most 8" in lib.ink_last_error()


def test_static_scratch_router_allocates_nothing_and_takes_its_largest_case():
    """Free device memory is the same before and after a warm call (nothing was allocated on the
    way), through the Python mirror of the entry point, at the limits it accepts: 8 tokens,
    no logits output; and a router with more rows than the array holds is refused."""
    import inkling_b200
    from inkling_b200.kernels import _abi

    lib = _abi.lib()
    device = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(22)
    p = dict(experts=256, n_shared=2, top_k=6, route_scale=8.0)
    weight = (torch.randn(258, 4096, generator=gen) * 0.02).to(BF16).to(device)
    bias = (torch.randn(256, generator=gen) * 0.05).to(device)
    scale = torch.ones(1, dtype=BF16, device=device)
    x = torch.randn(8, 4096, generator=gen).to(BF16).to(device)
    outs = [(torch.empty(8, 6, dtype=BF16, device=device), torch.full((8, 6), -1, dtype=torch.int64, device=device),
             torch.empty(8, 2, dtype=BF16, device=device)) for _ in range(2)]
    workspace = inkling_b200.kernels.router_workspace(8, 258, device)
    inkling_b200.kernels.router_forward_static(x, weight, bias, scale, 8.0, 6, 2, *outs[0])   # warm: address looked up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(device)
    inkling_b200.kernels.router_forward_static(x, weight, bias, scale, 8.0, 6, 2, *outs[0])
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(device)
    assert free_after == free_before
    inkling_b200.kernels.router_forward(x, weight, bias, scale, 8.0, 6, 2, *outs[1], workspace)
    torch.cuda.synchronize()
    for got, want in zip(outs[0], outs[1]):
        assert torch.equal(got, want)
    # 545 router rows: more than the array holds
    wide = torch.zeros(545, 64, dtype=BF16, device=device)
    rc = lib.ink_router_forward_static(
        x.data_ptr(), wide.data_ptr(), bias.data_ptr(), scale.data_ptr(), ctypes.c_float(8.0), 1, 64, 543, 2, 6, None,
        outs[0][0].data_ptr(), outs[0][1].data_ptr(), outs[0][2].data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc < 0 and b"at most 544" in lib.ink_last_error()

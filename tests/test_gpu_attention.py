"""Decode attention and the cache update through the C ABI against the oracle and against what the reference's
own modules produced (tests/golden/attention.npz)."""
import pytest
import torch

import attention_cases as ac
from oracle import attention as oa
from test_attention_oracle import CASES, load

pytestmark = pytest.mark.gpu
TOL = 2e-2   # of the largest output magnitude: BF16 results of a softmax-weighted sum, FP32 inside


@pytest.fixture(scope="module")
def ib():
    import inkling_b200

    return inkling_b200


def _run(ib, c, f, device, position=None):
    position = f["position"] if position is None else position
    pos = torch.tensor(position, dtype=torch.int64, device=device)
    pad = torch.tensor(c["pad_counts"], dtype=torch.int64, device=device)
    return ib.kernels.decode_attention(
        f["q"].to(device).unsqueeze(2), f["r"].to(device).unsqueeze(1), f["proj"].to(device), f["k_cache"].to(device),
        f["v_cache"].to(device), pos, pad, window=c["window"], log_scaling_n_floor=c["n_floor"],
        log_scaling_alpha=c["alpha"], scale=ac.SCALE)


@pytest.mark.parametrize("kind,step", CASES)
def test_decode_attention_matches_the_reference_module_and_the_oracle(ib, kind, step):
    device = torch.device("cuda", 0)
    c, f = ac.CASES[kind], load(kind, step)
    got = _run(ib, c, f, device)
    torch.cuda.synchronize()
    assert got.shape == (c["batch"], c["heads"], 1, c["head_dim"]) and got.dtype == torch.bfloat16
    got = got[:, :, 0].float().cpu()
    want = f["out"].float()
    exact = oa.decode_attention(f["q"], f["r"], f["proj"], f["k_cache"], f["v_cache"], f["position"],
                                torch.tensor(c["pad_counts"]), c["window"], c["n_floor"], c["alpha"], ac.SCALE, exact=True).float()
    assert (got - want).abs().max() <= TOL * want.abs().max()
    assert (got - exact).abs().max() <= TOL * exact.abs().max()


@pytest.mark.parametrize("kind,step", CASES[:1] + CASES[-1:])
def test_update_kv_stores_the_token_where_the_reference_does(ib, kind, step):
    device = torch.device("cuda", 0)
    c, f = ac.CASES[kind], load(kind, step)
    slot = f["position"] % c["window"] if c["window"] else f["position"]
    k, v = f["k_cache"].clone(), f["v_cache"].clone()
    k[:, :, slot] = 0
    v[:, :, slot] = 0
    k, v = k.to(device), v.to(device)
    pos = torch.tensor(f["position"], dtype=torch.int64, device=device)
    # the reference passes transposed views [bs, hk, 1, c] of a [bs, 1, hk * c] projection
    key = f["new_k"].to(device).reshape(c["batch"], 1, c["kv_heads"], c["head_dim"]).transpose(1, 2)
    value = f["new_v"].to(device).reshape(c["batch"], 1, c["kv_heads"], c["head_dim"]).transpose(1, 2)
    ib.kernels.update_kv(key, value, k, v, pos, c["window"])
    torch.cuda.synchronize()
    assert torch.equal(k.cpu(), f["k_cache"]) and torch.equal(v.cpu(), f["v_cache"])


@pytest.mark.parametrize("kind,step", CASES)
def test_decode_attention_that_stores_the_token_itself(ib, kind, step):
    """The caches as they were BEFORE the reference's update_kv (the token's slot zeroed) plus the token's key and
    value: same result as with the stored token, and the caches end up as the reference left them."""
    device = torch.device("cuda", 0)
    c, f = ac.CASES[kind], load(kind, step)
    slot = f["position"] % c["window"] if c["window"] else f["position"]
    k, v = f["k_cache"].clone(), f["v_cache"].clone()
    k[:, :, slot] = 0
    v[:, :, slot] = 0
    k, v = k.to(device), v.to(device)
    pos = torch.tensor(f["position"], dtype=torch.int64, device=device)
    pad = torch.tensor(c["pad_counts"], dtype=torch.int64, device=device)
    got = ib.kernels.decode_attention(f["q"].to(device), f["r"].to(device), f["proj"].to(device), k, v, pos, pad, window=c["window"],
                                      log_scaling_n_floor=c["n_floor"], log_scaling_alpha=c["alpha"], scale=ac.SCALE,
                                      new_key=f["new_k"].to(device).unsqueeze(2), new_value=f["new_v"].to(device).unsqueeze(2))
    torch.cuda.synchronize()
    want = f["out"].float()
    assert (got[:, :, 0].float().cpu() - want).abs().max() <= TOL * want.abs().max()
    assert torch.equal(k.cpu(), f["k_cache"]) and torch.equal(v.cpu(), f["v_cache"])


def test_decode_attention_at_the_model_shapes_against_the_oracle(ib):
    """64 heads of 128 channels over 16 key/value heads, a full ring of 512 slots, 16 relative patterns: seeded
    inputs, compared with the float64 oracle; and a full-attention layer of 4 096 slots with the scaling on."""
    device = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(5)
    for window, slots, hk, extent, position, n_floor in ((512, 512, 16, 512, 1300, None), (0, 4096, 8, 1024, 3000, 1024)):
        bs, h, c, d_rel = 2, 64, 128, 16
        q = torch.randn(bs, h, c, generator=gen).bfloat16()
        r = torch.randn(bs, h, d_rel, generator=gen).bfloat16()
        proj = (torch.randn(d_rel, extent, generator=gen) * 0.5).bfloat16()
        k = torch.randn(bs, hk, slots, c, generator=gen).bfloat16()
        v = torch.randn(bs, hk, slots, c, generator=gen).bfloat16()
        pad = torch.tensor([0, 7])
        want = oa.decode_attention(q, r, proj, k, v, position, pad, window, n_floor, 0.1, 1.0 / c, exact=True).float()
        got = ib.kernels.decode_attention(q.to(device), r.to(device), proj.to(device), k.to(device), v.to(device),
                                          torch.tensor(position, dtype=torch.int64, device=device), pad.to(device),
                                          window=window, log_scaling_n_floor=n_floor, log_scaling_alpha=0.1)
        torch.cuda.synchronize()
        got = got[:, :, 0].float().cpu()
        assert (got - want).abs().max() <= TOL * want.abs().max(), (window, float((got - want).abs().max()), float(want.abs().max()))


def test_decode_attention_rejects_what_it_was_not_built_for(ib):
    device = torch.device("cuda", 0)
    pos = torch.tensor(3, dtype=torch.int64, device=device)

    def call(c=64, slots=128, window=0, heads=4, hk=2):
        z = lambda *shape: torch.zeros(*shape, dtype=torch.bfloat16, device=device)
        return ib.kernels.decode_attention(z(1, heads, c), z(1, heads, 16), z(16, 32), z(1, hk, slots, c), z(1, hk, slots, c), pos,
                                           None, window=window)

    call()                                                     # the supported form goes through
    with pytest.raises(RuntimeError, match="head_dim"):
        call(c=96)
    with pytest.raises(RuntimeError, match="window"):
        call(window=256)                                       # a ring longer than the cache
    with pytest.raises(RuntimeError, match="kv_heads"):
        call(heads=5, hk=2)
    torch.cuda.synchronize()


@pytest.mark.parametrize("kind,step", CASES)
def test_the_whole_decode_step_of_the_attention_module(ib, kind, step):
    """Hidden state in, hidden state out, like `MyInklingAttention.forward` with a decoding cache: the module's weights,
    the caches and convolution histories as the reference's step found them, its input and its output are in the
    fixture. (The reference ran its short convolution under the Triton interpreter, which truncates where the GPU
    rounds: the key and value of the current token may differ from the recorded ones in the last BF16 bit.)"""
    from types import SimpleNamespace

    import numpy as np
    from test_attention_oracle import GOLDEN_DIR

    device = torch.device("cuda", 0)
    c, f = ac.CASES[kind], load(kind, step)
    z = np.load(GOLDEN_DIR / "attention.npz")

    def t(name, bf16=True):
        a = torch.from_numpy(z[name].copy())
        return (a.view(torch.bfloat16) if bf16 else a).to(device)

    module = ib.DecodeAttention(
        t(f"{kind}/qkvr_weight"), t(f"{kind}/o_weight"), t(f"{kind}/q_norm_weight"), t(f"{kind}/k_norm_weight"),
        t(f"{kind}/k_taps", False), t(f"{kind}/v_taps", False), f["proj"].to(device), layer_idx=0, heads=c["heads"],
        kv_heads=c["kv_heads"], head_dim=c["head_dim"], d_rel=c["d_rel"], window=c["window"],
        log_scaling_n_floor=c["n_floor"], log_scaling_alpha=c["alpha"])
    slot = f["position"] % c["window"] if c["window"] else f["position"]
    k, v = f["k_cache"].clone(), f["v_cache"].clone()
    k[:, :, slot] = 0
    v[:, :, slot] = 0
    layer = SimpleNamespace(k_cache=k.to(device), v_cache=v.to(device),
                            conv_caches=[SimpleNamespace(cache=t(f"{kind}/{step}/k_history", False)),
                                         SimpleNamespace(cache=t(f"{kind}/{step}/v_history", False))])
    cache = SimpleNamespace(layers=[layer], position=torch.tensor(f["position"], dtype=torch.int64, device=device),
                            pad_counts=torch.tensor(c["pad_counts"], dtype=torch.int64, device=device))
    y = module(t(f"{kind}/{step}/hidden").unsqueeze(1), cache)
    torch.cuda.synchronize()
    want = t(f"{kind}/{step}/y").float().cpu()
    got = y[:, 0].float().cpu()
    assert (got - want).abs().max() <= TOL * want.abs().max()
    # the token landed in its slot, up to the last bit; every other slot is untouched
    stored_k, stored_v = layer.k_cache.cpu(), layer.v_cache.cpu()
    assert (stored_k[:, :, slot].float() - f["new_k"].float()).abs().max() <= 2 ** -6 * f["new_k"].float().abs().max()
    assert (stored_v[:, :, slot].float() - f["new_v"].float()).abs().max() <= 2 ** -6 * f["new_v"].float().abs().max()
    stored_k[:, :, slot] = f["k_cache"][:, :, slot]
    stored_v[:, :, slot] = f["v_cache"][:, :, slot]
    assert torch.equal(stored_k, f["k_cache"]) and torch.equal(stored_v, f["v_cache"])


@pytest.mark.parametrize("step", ac.LAYER["record"])
def test_a_whole_sparse_decoder_layer_at_decode(ib, step):
    """`MyInklingDecoderLayer.forward` for one token per sequence: norm, attention, short convolution + residual, norm,
    MoE block (NVFP4 experts here, their BF16 dequantisation in the reference), short convolution + residual. Input,
    output, caches and the four convolution histories of the step were recorded from the reference's layer."""
    from types import SimpleNamespace

    import numpy as np

    import cases
    from helpers import banks_to_device, layer_on_device
    from test_attention_oracle import GOLDEN_DIR

    device = torch.device("cuda", 0)
    c = ac.LAYER
    z = np.load(GOLDEN_DIR / "attention.npz")

    def t(name, bf16=True):
        a = torch.from_numpy(z[f"layer/{step}/{name}"].copy())
        return (a.view(torch.bfloat16) if bf16 else a).to(device)

    w = {k: v.to(device) for k, v in ac.layer_weights(c).items()}
    attention = ib.DecodeAttention(torch.cat([w["q"], w["k"], w["v"], w["r"]]), w["o"], w["q_norm"], w["k_norm"], w["k_taps"],
                                   w["v_taps"], w["rel_proj"], layer_idx=0, heads=c["heads"], kv_heads=c["kv_heads"],
                                   head_dim=c["head_dim"], d_rel=c["d_rel"], window=c["window"],
                                   log_scaling_n_floor=c["n_floor"], log_scaling_alpha=c["alpha"], eps=c["eps"])
    p, banks, _ = cases.make_layer(**cases.LAYER_CASES[c["moe"]])
    dp = layer_on_device(p, device)
    experts = ib.ResidentExperts(p["d"], p["f"], None, banks_to_device(banks, device))
    moe = ib.FusedMoE(dp["router_weight"], dp["router_bias"], dp["global_scale"], p["route_scale"], p["top_k"],
                      dp["shared_gate"], dp["shared_up"], dp["shared_down"], experts, None)
    layer = ib.DecodeLayer(attention, moe, w["input_norm"], w["post_norm"], w["attn_taps"], w["mlp_taps"], eps=c["eps"])
    position = int(z[f"layer/{step}/position"])
    slot = position % c["window"]
    k, v = t("k_cache").clone(), t("v_cache").clone()
    k[:, :, slot] = 0
    v[:, :, slot] = 0
    state = SimpleNamespace(k_cache=k, v_cache=v, conv_caches=[SimpleNamespace(cache=t(f"history{i}", False)) for i in range(4)])
    cache = SimpleNamespace(layers=[state], position=torch.tensor(position, dtype=torch.int64, device=device),
                            pad_counts=torch.tensor(c["pad_counts"], dtype=torch.int64, device=device))
    y = layer(t("hidden").unsqueeze(1), cache)
    torch.cuda.synchronize()
    experts.check_status()
    got, want = y[:, 0].float().cpu(), t("y").float().cpu()
    assert (got - want).abs().max() <= TOL * want.abs().max(), float((got - want).abs().max() / want.abs().max())
    # the token's key and value are in their slot (up to the last bit, see the test above)
    for stored, recorded in ((k, t("k_cache")), (v, t("v_cache"))):
        a, b = stored[:, :, slot].float(), recorded[:, :, slot].float()
        assert (a - b).abs().max() <= 2 ** -6 * b.abs().max()


def test_the_decoder_layer_replays_in_a_cuda_graph(ib):
    """Warm-up steps on a side stream, capture, replay (the sequence of my_inkling/decode_graph.py:22-41): nothing in
    the layer allocates or synchronises once it is warm, the position counter is read on the device, so a replay with
    the caches put back gives the bits of the eager step."""
    from types import SimpleNamespace

    import cases
    from helpers import banks_to_device, layer_on_device

    device = torch.device("cuda", 0)
    c = ac.LAYER
    w = {k: v.to(device) for k, v in ac.layer_weights(c).items()}
    attention = ib.DecodeAttention(torch.cat([w["q"], w["k"], w["v"], w["r"]]), w["o"], w["q_norm"], w["k_norm"], w["k_taps"],
                                   w["v_taps"], w["rel_proj"], layer_idx=0, heads=c["heads"], kv_heads=c["kv_heads"],
                                   head_dim=c["head_dim"], d_rel=c["d_rel"], window=c["window"],
                                   log_scaling_n_floor=c["n_floor"], log_scaling_alpha=c["alpha"], eps=c["eps"])
    p, banks, _ = cases.make_layer(**cases.LAYER_CASES[c["moe"]])
    dp = layer_on_device(p, device)
    experts = ib.ResidentExperts(p["d"], p["f"], None, banks_to_device(banks, device))
    moe = ib.FusedMoE(dp["router_weight"], dp["router_bias"], dp["global_scale"], p["route_scale"], p["top_k"],
                      dp["shared_gate"], dp["shared_up"], dp["shared_down"], experts, None)
    layer = ib.DecodeLayer(attention, moe, w["input_norm"], w["post_norm"], w["attn_taps"], w["mlp_taps"], eps=c["eps"])
    gen = torch.Generator().manual_seed(9)
    bs, d, hk, hd = c["batch"], c["hidden"], c["kv_heads"], c["head_dim"]
    state = SimpleNamespace(
        k_cache=torch.randn(bs, hk, c["window"], hd, generator=gen).bfloat16().to(device),
        v_cache=torch.randn(bs, hk, c["window"], hd, generator=gen).bfloat16().to(device),
        conv_caches=[SimpleNamespace(cache=torch.randn(bs, n, c["conv_k"], generator=gen).to(device)) for n in (hk * hd, hk * hd, d, d)])
    cache = SimpleNamespace(layers=[state], position=torch.tensor(45, dtype=torch.int64, device=device),
                            pad_counts=torch.zeros(bs, dtype=torch.int64, device=device))
    tensors = [state.k_cache, state.v_cache] + [cc.cache for cc in state.conv_caches]
    saved = [t.clone() for t in tensors]
    token = torch.randn(bs, 1, d, generator=gen).bfloat16().to(device)

    def restore():
        for t, s in zip(tensors, saved):
            t.copy_(s)

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream), torch.inference_mode():
        for _ in range(3):
            eager = layer(token, cache).clone()
            after = [t.clone() for t in tensors]
            restore()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream), torch.inference_mode():
        out = layer(token, cache)
    restore()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    assert all(torch.equal(t, a) for t, a in zip(tensors, after))
    cache.position.add_(1)          # the next token: the replay reads the counter on the device
    graph.replay()
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all() and not torch.equal(out, eager)
    experts.check_status()


@pytest.mark.parametrize("step", ac.MODEL["record"])
def test_a_decode_step_of_the_whole_model(ib, step):
    """Token ids in, logits out: `MyInkling.forward` with a decoding cache for a two-layer model (a dense sliding-window
    layer, a sparse full-attention layer with the log scaling on), against the logits the reference's model produced
    from the same caches and histories; the position counter moves on by one."""
    from types import SimpleNamespace

    import numpy as np

    import cases
    from helpers import banks_to_device, layer_on_device
    from test_attention_oracle import GOLDEN_DIR

    device = torch.device("cuda", 0)
    c = ac.MODEL
    z = np.load(GOLDEN_DIR / "attention.npz")

    def t(name, bf16=True):
        a = torch.from_numpy(z[f"model/{step}/{name}"].copy())
        return (a.view(torch.bfloat16) if bf16 else a).to(device)

    def dev(tree):
        return {k: (dev(v) if isinstance(v, dict) else v.to(device)) for k, v in tree.items()}

    w = ac.model_weights(c)
    p, banks, _ = cases.make_layer(**cases.LAYER_CASES[c["moe"]])
    dp = layer_on_device(p, device)
    experts = ib.ResidentExperts(p["d"], p["f"], None, banks_to_device(banks, device))
    moe = ib.FusedMoE(dp["router_weight"], dp["router_bias"], dp["global_scale"], p["route_scale"], p["top_k"],
                      dp["shared_gate"], dp["shared_up"], dp["shared_down"], experts, None)
    dense = dev(w["dense"])
    blocks = [ib.DenseMLP(dense["gate"], dense["up"], dense["down"], dense["global_scale"]), moe]
    layers = []
    for i, (lw, window) in enumerate(zip(w["layers"], (c["window"], 0))):
        lw = dev(lw)
        attention = ib.DecodeAttention(torch.cat([lw["q"], lw["k"], lw["v"], lw["r"]]), lw["o"], lw["q_norm"], lw["k_norm"],
                                       lw["k_taps"], lw["v_taps"], lw["rel_proj"], layer_idx=i, heads=c["heads"],
                                       kv_heads=c["kv_heads"], head_dim=c["head_dim"], d_rel=c["d_rel"], window=window,
                                       log_scaling_n_floor=c["n_floor"], log_scaling_alpha=c["alpha"], eps=c["eps"])
        layers.append(ib.DecodeLayer(attention, blocks[i], lw["input_norm"], lw["post_norm"], lw["attn_taps"], lw["mlp_taps"], eps=c["eps"]))
    model = ib.DecodeModel(w["embedding"].to(device), w["embed_norm"].to(device), layers, w["final_norm"].to(device),
                           w["lm_head"].to(device), c["mup"], eps=c["eps"])
    position = int(z[f"model/{step}/position"])
    states = []
    for li, window in enumerate((c["window"], 0)):
        slot = position % window if window else position
        k, v = t(f"layer{li}/k_cache").clone(), t(f"layer{li}/v_cache").clone()
        k[:, :, slot] = 0
        v[:, :, slot] = 0
        states.append(SimpleNamespace(k_cache=k, v_cache=v,
                                      conv_caches=[SimpleNamespace(cache=t(f"layer{li}/history{i}", False)) for i in range(4)]))
    cache = SimpleNamespace(layers=states, position=torch.tensor(position, dtype=torch.int64, device=device),
                            pad_counts=torch.tensor(c["pad_counts"], dtype=torch.int64, device=device))
    logits = model(t("input_ids", False), cache)
    torch.cuda.synchronize()
    experts.check_status()
    assert int(cache.position) == position + 1
    got, want = logits[:, 0].float().cpu(), t("logits").float().cpu()
    assert got.shape == want.shape == (c["batch"], c["vocab"])
    # The sparse layer's router sees activations that differ from the reference's in the last bits (two layers of
    # BF16 arithmetic in another order), and a near-tie for the sixth expert can fall the other way: sequences routed
    # like the reference's are held to the usual bar, the others only to being close (one expert of six differs).
    mine = moe.topk_indices[: c["batch"]].cpu().sort(-1).values
    theirs = t("expert_indices", False).cpu().sort(-1).values
    same = (mine == theirs).all(-1)
    swapped = sum(len(set(a.tolist()) - set(b.tolist())) for a, b in zip(mine, theirs))
    assert int(same.sum()) >= 1 and swapped <= 1
    scale = want.abs().max()
    assert (got[same] - want[same]).abs().max() <= TOL * scale, float((got[same] - want[same]).abs().max() / scale)
    assert (got - want).abs().max() <= 0.15 * scale
    assert torch.equal(got.argmax(-1), want.argmax(-1))          # the same next token

"""Fixtures for decode attention, produced by RUNNING the reference's own modules on the CPU.

    python tests/golden/make_attention_golden.py <reference_root>     (or INKLING_REFERENCE_ROOT)

`MyInklingAttention` (my_inkling/model.py:431-622) with a `MyInklingCache` (my_inkling/cache.py) is prefilled
with a short prompt, frozen for decode and stepped token by token, once for a sliding-window layer (the ring
wraps during the run) and once for a full-attention layer with the logarithmic scaling on. Its Triton kernels
(`update_kv`, `short_conv`) run under TRITON_INTERPRET=1. At chosen steps the inputs of the attention core are
recorded with hooks -- the module's input and output, the convolution histories, the normed queries, the relative states, the caches as `scaled_dot_product_attention`
sees them, the position counter -- together with what `scaled_dot_product_attention` returned and what
`update_kv` was given. Writes tests/golden/attention.npz (BF16 tensors as their uint16 bit patterns).
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import attention_cases as ac  # noqa: E402

REFERENCE = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("INKLING_REFERENCE_ROOT")
if not REFERENCE:
    raise SystemExit("usage: make_attention_golden.py <reference_root>")
sys.path.insert(0, REFERENCE)
from my_inkling import model as ref_model  # noqa: E402  (reference)
from my_inkling.cache import MyInklingCache  # noqa: E402  (reference)

out: dict[str, np.ndarray] = {}


def put(key: str, t: torch.Tensor) -> None:
    t = t.detach().cpu().contiguous().clone()
    out[key] = t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def run(kind: str) -> None:
    c = ac.CASES[kind]
    config = ref_model.InklingTextConfig(
        hidden_size=c["hidden"], vocab_size=64, num_hidden_layers=2, pad_token_id=0,
        layer_types=["hybrid_sliding", "hybrid"], num_attention_heads=c["heads"], num_key_value_heads=c["kv_heads"],
        head_dim=c["head_dim"], swa_num_attention_heads=c["heads"], swa_num_key_value_heads=c["kv_heads"],
        swa_head_dim=c["head_dim"], sliding_window_size=c["window"] or 32, d_rel=c["d_rel"], rel_extent=c["rel_extent"],
        log_scaling_n_floor=c["n_floor"], log_scaling_alpha=c["alpha"])
    layer_idx = 0 if c["window"] else 1
    gen = torch.Generator().manual_seed(c["seed"])
    attn = ref_model.MyInklingAttention(config, layer_idx)
    for p in attn.parameters():
        p.data.copy_(torch.randn(p.shape, generator=gen) * c["std"])
    attn = attn.bfloat16().eval()
    attn.k_sconv.conv1d.float()   # the reference keeps the convolution taps in FP32
    attn.v_sconv.conv1d.float()
    attn.fuse_projections()
    put(f"{kind}/proj", attn.rel_logits_proj.proj)
    # the whole module's weights, for the test that runs the decode step end to end
    put(f"{kind}/qkvr_weight", attn.qkvr_proj.weight)
    put(f"{kind}/o_weight", attn.o_proj.weight)
    put(f"{kind}/q_norm_weight", attn.q_norm.weight)
    put(f"{kind}/k_norm_weight", attn.k_norm.weight)
    put(f"{kind}/k_taps", attn.k_sconv.conv1d.weight)      # FP32 [hk * c, 1, K]
    put(f"{kind}/v_taps", attn.v_sconv.conv1d.weight)
    cache = MyInklingCache(config, batch_size=c["batch"], capacity=c["capacity"], pad_counts=torch.tensor(c["pad_counts"]),
                           dtype=torch.bfloat16, device="cpu")
    rec: dict[str, torch.Tensor] = {}
    attn.q_norm.register_forward_hook(lambda m, i, o: rec.__setitem__("q", o.detach().clone()))
    attn.qkvr_proj.register_forward_hook(lambda m, i, o: rec.__setitem__("qkvr", o.detach().clone()))
    original_sdpa, original_update = F.scaled_dot_product_attention, cache.update_attn_cache

    def sdpa(q, k, v, attn_mask=None, **kw):
        result = original_sdpa(q, k, v, attn_mask=attn_mask, **kw)
        rec.update(k=k.detach().clone(), v=v.detach().clone(), out=result.detach().clone())
        return result

    def update(key_states, value_states, layer):
        rec.update(new_k=key_states.detach().clone(), new_v=value_states.detach().clone())
        return original_update(key_states, value_states, layer)

    ref_model.F.scaled_dot_product_attention = sdpa
    cache.update_attn_cache = update
    with torch.no_grad():
        attn(torch.randn(c["batch"], c["prompt"], c["hidden"], generator=gen).bfloat16(), cache=cache)
        cache.advance(c["prompt"])
        cache.prepare_decode()
        for step in range(max(c["record"]) + 1):
            position = int(cache.position)
            hidden = torch.randn(c["batch"], 1, c["hidden"], generator=gen).bfloat16()
            if step in c["record"]:     # the convolutions' histories as the step finds them
                put(f"{kind}/{step}/k_history", cache.layers[layer_idx].conv_caches[0].cache)
                put(f"{kind}/{step}/v_history", cache.layers[layer_idx].conv_caches[1].cache)
            y = attn(hidden, cache=cache)
            if step in c["record"]:
                put(f"{kind}/{step}/hidden", hidden[:, 0])
                put(f"{kind}/{step}/y", y[:, 0])
                r = rec["qkvr"].split(attn.projection_sizes, dim=-1)[3].view(c["batch"], c["heads"], c["d_rel"])
                put(f"{kind}/{step}/position", torch.tensor(position))
                put(f"{kind}/{step}/q", rec["q"][:, :, 0])                 # [bs, h, c] after q_norm
                put(f"{kind}/{step}/r", r)                                  # [bs, h, d_rel]
                put(f"{kind}/{step}/k_cache", rec["k"])                     # [bs, hk, capacity, c], this token stored
                put(f"{kind}/{step}/v_cache", rec["v"])
                put(f"{kind}/{step}/new_k", rec["new_k"][:, :, 0])          # [bs, hk, c] what update_kv stored
                put(f"{kind}/{step}/new_v", rec["new_v"][:, :, 0])
                put(f"{kind}/{step}/out", rec["out"][:, :, 0])              # [bs, h, c]
            cache.advance(1)
    ref_model.F.scaled_dot_product_attention = original_sdpa


def run_layer() -> None:
    """A whole sparse decoder layer (my_inkling/model.py:636-675) stepped in decode mode: input, output, caches and all
    four convolution histories as each recorded step finds them. The MoE block holds the NVFP4 banks of
    cases.LAYER_CASES[...] dequantised to BF16, as the reference's PyTorch path does."""
    import cases
    import make_golden   # (the loaders of the MoE fixtures; takes the reference root from the same command line)

    c = ac.LAYER
    mc = cases.LAYER_CASES[c["moe"]]
    config = ref_model.InklingTextConfig(
        hidden_size=c["hidden"], vocab_size=64, num_hidden_layers=1, pad_token_id=0, layer_types=["hybrid_sliding"],
        moe_intermediate_size=mc["f"], n_routed_experts=mc["experts"], num_experts_per_tok=mc["top_k"],
        n_shared_experts=mc["n_shared"], route_scale=8.0, rms_norm_eps=c["eps"],
        swa_num_attention_heads=c["heads"], swa_num_key_value_heads=c["kv_heads"], swa_head_dim=c["head_dim"],
        sliding_window_size=c["window"], d_rel=c["d_rel"], rel_extent=c["rel_extent"], conv_kernel_size=c["conv_k"],
        log_scaling_n_floor=c["n_floor"], log_scaling_alpha=c["alpha"])
    layer = ref_model.MyInklingDecoderLayer(config, 0).bfloat16().eval()
    w = ac.layer_weights(c)
    p, banks, _ = cases.make_layer(**mc)
    with torch.no_grad():
        a = layer.self_attn
        a.q_proj.weight.copy_(w["q"]); a.k_proj.weight.copy_(w["k"]); a.v_proj.weight.copy_(w["v"]); a.r_proj.weight.copy_(w["r"])
        a.o_proj.weight.copy_(w["o"]); a.q_norm.weight.copy_(w["q_norm"]); a.k_norm.weight.copy_(w["k_norm"])
        a.rel_logits_proj.proj.copy_(w["rel_proj"])
        for conv, taps in ((a.k_sconv, "k_taps"), (a.v_sconv, "v_taps"), (layer.attn_sconv, "attn_taps"), (layer.mlp_sconv, "mlp_taps")):
            conv.conv1d.float()            # the reference keeps the convolution taps in FP32
            conv.conv1d.weight.copy_(w[taps])
        layer.input_layernorm.weight.copy_(w["input_norm"]); layer.post_attention_layernorm.weight.copy_(w["post_norm"])
        a.fuse_projections()
        layer.mlp = make_golden.load_reference_moe(mc, p, banks)
        cache = MyInklingCache(config, batch_size=c["batch"], capacity=c["capacity"], pad_counts=torch.tensor(c["pad_counts"]),
                               dtype=torch.bfloat16, device="cpu")
        gen = torch.Generator().manual_seed(c["seed"] + 1)
        layer(torch.randn(c["batch"], c["prompt"], c["hidden"], generator=gen).bfloat16(), cache=cache)
        cache.advance(c["prompt"])
        cache.prepare_decode()
        for step in range(max(c["record"]) + 1):
            position = int(cache.position)
            hidden = torch.randn(c["batch"], 1, c["hidden"], generator=gen).bfloat16()
            if step in c["record"]:
                for i in range(4):
                    put(f"layer/{step}/history{i}", cache.layers[0].conv_caches[i].cache)
            y = layer(hidden, cache=cache)
            if step in c["record"]:
                put(f"layer/{step}/position", torch.tensor(position))
                put(f"layer/{step}/hidden", hidden[:, 0])
                put(f"layer/{step}/y", y[:, 0])
                put(f"layer/{step}/k_cache", cache.layers[0].k_cache)     # after the step: the token is in its slot
                put(f"layer/{step}/v_cache", cache.layers[0].v_cache)
            cache.advance(1)


def _load_layer(layer, w) -> None:
    """Weights of one decoder layer outside its MLP / MoE block into the reference's modules."""
    a = layer.self_attn
    a.q_proj.weight.copy_(w["q"]); a.k_proj.weight.copy_(w["k"]); a.v_proj.weight.copy_(w["v"]); a.r_proj.weight.copy_(w["r"])
    a.o_proj.weight.copy_(w["o"]); a.q_norm.weight.copy_(w["q_norm"]); a.k_norm.weight.copy_(w["k_norm"])
    a.rel_logits_proj.proj.copy_(w["rel_proj"])
    for conv, taps in ((a.k_sconv, "k_taps"), (a.v_sconv, "v_taps"), (layer.attn_sconv, "attn_taps"), (layer.mlp_sconv, "mlp_taps")):
        conv.conv1d.float()            # the reference keeps the convolution taps in FP32
        conv.conv1d.weight.copy_(w[taps])
    layer.input_layernorm.weight.copy_(w["input_norm"]); layer.post_attention_layernorm.weight.copy_(w["post_norm"])
    a.fuse_projections()


def run_model() -> None:
    """The reference's whole model (`MyInkling`, my_inkling/model.py:729-800) with two layers -- a dense sliding-window
    one and a sparse full-attention one -- prefilled and stepped in decode mode: token ids in, logits out, with every
    cache and convolution history as each recorded step finds them."""
    import cases
    import make_golden

    c = ac.MODEL
    mc = cases.LAYER_CASES[c["moe"]]
    text = ref_model.InklingTextConfig(
        hidden_size=c["hidden"], vocab_size=c["vocab"], num_hidden_layers=2, pad_token_id=0,
        layer_types=["hybrid_sliding", "hybrid"], mlp_layer_types=["dense", "sparse"], intermediate_size=c["dense_intermediate"],
        moe_intermediate_size=mc["f"], n_routed_experts=mc["experts"], num_experts_per_tok=mc["top_k"],
        n_shared_experts=mc["n_shared"], route_scale=8.0, rms_norm_eps=c["eps"],
        num_attention_heads=c["heads"], num_key_value_heads=c["kv_heads"], head_dim=c["head_dim"],
        swa_num_attention_heads=c["heads"], swa_num_key_value_heads=c["kv_heads"], swa_head_dim=c["head_dim"],
        sliding_window_size=c["window"], d_rel=c["d_rel"], rel_extent=c["rel_extent"], conv_kernel_size=c["conv_k"],
        log_scaling_n_floor=c["n_floor"], log_scaling_alpha=c["alpha"], logits_mup_width_multiplier=c["mup"])
    model = ref_model.MyInkling(ref_model.InklingConfig(text_config=text, hidden_size=c["hidden"], vocab_size=c["vocab"])).bfloat16().eval()
    w = ac.model_weights(c)
    p, banks, _ = cases.make_layer(**mc)
    with torch.no_grad():
        tower = model.model.language_model
        tower.embed_tokens.weight.copy_(w["embedding"]); tower.embed_tokens.embed_norm.weight.copy_(w["embed_norm"])
        tower.norm.weight.copy_(w["final_norm"]); model.lm_head.weight.copy_(w["lm_head"])
        for layer, lw in zip(tower.layers, w["layers"]):
            _load_layer(layer, lw)
        dense = tower.layers[0].mlp
        dense.gate_proj.weight.copy_(w["dense"]["gate"]); dense.up_proj.weight.copy_(w["dense"]["up"])
        dense.down_proj.weight.copy_(w["dense"]["down"]); dense.global_scale.copy_(w["dense"]["global_scale"])
        tower.layers[1].mlp = make_golden.load_reference_moe(mc, p, banks)
        routed: dict[str, torch.Tensor] = {}
        tower.layers[1].mlp.gate.register_forward_hook(lambda m, i, o: routed.__setitem__("indices", o[2].detach().clone()))
        cache = MyInklingCache(text, batch_size=c["batch"], capacity=c["capacity"], pad_counts=torch.tensor(c["pad_counts"]),
                               dtype=torch.bfloat16, device="cpu")
        gen = torch.Generator().manual_seed(c["seed"] + 1)
        model(torch.randint(1, c["vocab"], (c["batch"], c["prompt"]), generator=gen), cache=cache)
        cache.prepare_decode()
        for step in range(max(c["record"]) + 1):
            position = int(cache.position)
            ids = torch.randint(1, c["vocab"], (c["batch"], 1), generator=gen)
            if step in c["record"]:
                for li in range(2):
                    for i in range(4):
                        put(f"model/{step}/layer{li}/history{i}", cache.layers[li].conv_caches[i].cache)
            logits = model(ids, cache=cache)
            if step in c["record"]:
                put(f"model/{step}/position", torch.tensor(position))
                put(f"model/{step}/input_ids", ids)
                put(f"model/{step}/logits", logits[:, 0])
                put(f"model/{step}/expert_indices", routed["indices"].reshape(c["batch"], -1))   # the sparse layer's routing
                for li in range(2):
                    put(f"model/{step}/layer{li}/k_cache", cache.layers[li].k_cache)      # after the step
                    put(f"model/{step}/layer{li}/v_cache", cache.layers[li].v_cache)


def main() -> None:
    for kind in ac.CASES:
        run(kind)
    run_layer()
    run_model()
    np.savez_compressed(HERE / "attention.npz", **out)
    print(f"wrote {len(out)} arrays, {sum(a.nbytes for a in out.values()) / 1e6:.2f} MB raw")


if __name__ == "__main__":
    main()

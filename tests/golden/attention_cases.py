"""Shapes and seeds of the decode-attention fixtures (shared by the generator and the tests)."""

CASES = {
    # sliding-window layer: ring of 32 slots, prompt 20, recorded before and after the ring wraps
    "sliding": dict(hidden=256, heads=8, kv_heads=4, head_dim=64, window=32, capacity=96, d_rel=16, rel_extent=32,
                    n_floor=8, alpha=0.1, batch=2, pad_counts=[0, 3], prompt=20, record=(0, 11, 12, 40), seed=11, std=0.08),
    # full-attention layer: capacity 96, log scaling on (position >= n_floor), relative extent shorter than the context
    "full": dict(hidden=256, heads=8, kv_heads=2, head_dim=64, window=0, capacity=96, d_rel=16, rel_extent=48,
                 n_floor=8, alpha=0.1, batch=2, pad_counts=[0, 3], prompt=20, record=(0, 30, 60), seed=12, std=0.08),
}
SCALE = 1.0 / 64   # 1 / head_dim, my_inkling/model.py:448

# One whole sparse decoder layer (attention + MoE block + the norms and short convolutions around them): the MoE
# block is cases.LAYER_CASES["mid"] (hidden 1024), the attention a sliding-window layer whose ring wraps in the run.
LAYER = dict(moe="mid", hidden=1024, heads=8, kv_heads=4, head_dim=64, window=32, capacity=96, d_rel=16, rel_extent=32,
             n_floor=8, alpha=0.1, batch=2, pad_counts=[0, 3], prompt=20, record=(0, 13), seed=21, std=0.04, conv_k=4, eps=1e-6)


def layer_weights(c=LAYER):
    """The layer's weights outside the MoE block, from the seed: the same tensors in the generator (copied into the
    reference's modules) and in the tests."""
    import torch

    gen = torch.Generator().manual_seed(c["seed"])
    d, h, hk, hd = c["hidden"], c["heads"], c["kv_heads"], c["head_dim"]

    def w(*shape, std=c["std"], dtype=torch.bfloat16):
        return (torch.randn(*shape, generator=gen) * std).to(dtype)

    def near_one(n):
        return (1.0 + 0.1 * torch.randn(n, generator=gen)).to(torch.bfloat16)

    return dict(
        q=w(h * hd, d), k=w(hk * hd, d), v=w(hk * hd, d), r=w(h * c["d_rel"], d), o=w(d, h * hd),
        q_norm=near_one(hd), k_norm=near_one(hd), rel_proj=w(c["d_rel"], c["rel_extent"], std=0.5),
        k_taps=w(hk * hd, 1, c["conv_k"], std=0.3, dtype=torch.float32), v_taps=w(hk * hd, 1, c["conv_k"], std=0.3, dtype=torch.float32),
        input_norm=near_one(d), post_norm=near_one(d),
        attn_taps=w(d, 1, c["conv_k"], std=0.3, dtype=torch.float32), mlp_taps=w(d, 1, c["conv_k"], std=0.3, dtype=torch.float32))

# A whole (tiny) model for one decode step: normed embedding, a dense sliding-window layer, a sparse full-attention
# layer (MoE block = cases.LAYER_CASES["mid"]), final norm, LM head.
MODEL = dict(moe="mid", hidden=1024, vocab=64, dense_intermediate=512, heads=8, kv_heads=4, head_dim=64, window=32, capacity=96,
             d_rel=16, rel_extent=48, n_floor=8, alpha=0.1, batch=2, pad_counts=[0, 3], prompt=20, record=(0, 13), seed=31,
             std=0.04, conv_k=4, eps=1e-6, mup=24.0)


def model_weights(c=MODEL):
    """Every weight of the tiny model outside the MoE block, from the seed (generator and tests build the same)."""
    import torch

    gen = torch.Generator().manual_seed(c["seed"])
    d = c["hidden"]

    def w(*shape, std=c["std"], dtype=torch.bfloat16):
        return (torch.randn(*shape, generator=gen) * std).to(dtype)

    def near_one(n):
        return (1.0 + 0.1 * torch.randn(n, generator=gen)).to(torch.bfloat16)

    layers = []
    for i, extent in enumerate((c["window"], c["rel_extent"])):       # layer 0 sliding (extent = window), layer 1 full
        lw = layer_weights(dict(c, seed=c["seed"] + 10 * (i + 1), rel_extent=extent))
        layers.append(lw)
    dense = dict(gate=w(c["dense_intermediate"], d), up=w(c["dense_intermediate"], d), down=w(d, c["dense_intermediate"]),
                 global_scale=torch.ones(1, dtype=torch.bfloat16))
    return dict(embedding=w(c["vocab"], d, std=1.0), embed_norm=near_one(d), final_norm=near_one(d), lm_head=w(c["vocab"], d),
                layers=layers, dense=dense)

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

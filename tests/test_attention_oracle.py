"""The attention oracle against fixtures produced by the reference's own modules."""
from pathlib import Path

import numpy as np
import pytest
import torch

import attention_cases as ac
from oracle import attention as oa

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def load(kind, step):
    z = np.load(GOLDEN_DIR / "attention.npz")
    def t(name, bf16=True):
        a = torch.from_numpy(z[f"{kind}/{step}/{name}"].copy())
        return a.view(torch.bfloat16) if bf16 else a
    proj = torch.from_numpy(z[f"{kind}/proj"].copy()).view(torch.bfloat16)
    return dict(q=t("q"), r=t("r"), k_cache=t("k_cache"), v_cache=t("v_cache"), new_k=t("new_k"), new_v=t("new_v"),
                out=t("out"), position=int(t("position", False)), proj=proj)


CASES = [(kind, step) for kind, c in ac.CASES.items() for step in c["record"]]


@pytest.mark.parametrize("kind,step", CASES)
def test_oracle_matches_the_reference_module(kind, step):
    c, f = ac.CASES[kind], load(kind, step)
    args = (f["q"], f["r"], f["proj"], f["k_cache"], f["v_cache"], f["position"], torch.tensor(c["pad_counts"]),
            c["window"], c["n_floor"], c["alpha"], ac.SCALE)
    got = oa.decode_attention(*args).float()
    want = f["out"].float()
    # the reference's result is whatever torch's scaled_dot_product_attention rounds on the CPU: BF16 ulps
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()
    exact = oa.decode_attention(*args, exact=True).float()
    assert (exact - want).abs().max() <= 2e-2 * want.abs().max()


@pytest.mark.parametrize("kind,step", CASES)
def test_the_recorded_cache_holds_the_new_token_where_update_kv_puts_it(kind, step):
    c, f = ac.CASES[kind], load(kind, step)
    k, v = f["k_cache"].clone(), f["v_cache"].clone()
    slot = f["position"] % c["window"] if c["window"] else f["position"]
    k[:, :, slot] = 0
    v[:, :, slot] = 0
    oa.update_kv(k, v, f["new_k"], f["new_v"], f["position"], c["window"])
    assert torch.equal(k, f["k_cache"]) and torch.equal(v, f["v_cache"])

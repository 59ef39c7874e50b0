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


def _module_inputs(kind, step):
    z = np.load(GOLDEN_DIR / "attention.npz")
    c, f = ac.CASES[kind], load(kind, step)

    def t(name, bf16=True):
        a = torch.from_numpy(z[name].copy())
        return a.view(torch.bfloat16) if bf16 else a

    weights = dict(qkvr=t(f"{kind}/qkvr_weight"), o=t(f"{kind}/o_weight"), q_norm=t(f"{kind}/q_norm_weight"),
                   k_norm=t(f"{kind}/k_norm_weight"), k_taps=t(f"{kind}/k_taps", False), v_taps=t(f"{kind}/v_taps", False),
                   rel_proj=f["proj"])
    slot = f["position"] % c["window"] if c["window"] else f["position"]
    k, v = f["k_cache"].clone(), f["v_cache"].clone()
    k[:, :, slot] = 0
    v[:, :, slot] = 0
    return (c, f, weights, k, v, t(f"{kind}/{step}/k_history", False), t(f"{kind}/{step}/v_history", False),
            t(f"{kind}/{step}/hidden"), t(f"{kind}/{step}/y"))


@pytest.mark.parametrize("kind,step", CASES)
def test_oracle_of_the_whole_attention_module(kind, step):
    """Hidden state in, hidden state out, against what the reference's module returned for the same step."""
    c, f, weights, k, v, kh, vh, hidden, want = _module_inputs(kind, step)
    got = oa.attention_decode_step(hidden, weights, k, v, kh, vh, f["position"], torch.tensor(c["pad_counts"]), heads=c["heads"],
                                   kv_heads=c["kv_heads"], head_dim=c["head_dim"], d_rel=c["d_rel"], window=c["window"],
                                   n_floor=c["n_floor"], alpha=c["alpha"], eps=1e-6)
    assert (got.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max()
    # the token the step stored: the reference's short convolution ran under the Triton interpreter, which truncates
    # to BF16 where this restatement (and the GPU) rounds, hence the last bit
    slot = f["position"] % c["window"] if c["window"] else f["position"]
    assert (k[:, :, slot].float() - f["new_k"].float()).abs().max() <= 2 ** -6 * f["new_k"].float().abs().max()
    assert (v[:, :, slot].float() - f["new_v"].float()).abs().max() <= 2 ** -6 * f["new_v"].float().abs().max()


def test_heads_sliced_over_two_ranks_add_up():
    """Tensor parallelism on the heads (the reference slices q/k/v/r rows and o_proj columns per rank and all-reduces
    the output): two half-modules on the same input, their outputs added in FP32, equal the whole module's."""
    kind, step = CASES[0]
    c, f, weights, k, v, kh, vh, hidden, _ = _module_inputs(kind, step)
    h, hk, hd, dr = c["heads"], c["kv_heads"], c["head_dim"], c["d_rel"]
    args = dict(kv_heads=hk, head_dim=hd, d_rel=dr, window=c["window"], n_floor=c["n_floor"], alpha=c["alpha"], eps=1e-6)
    whole = oa.attention_decode_step(hidden, weights, k.clone(), v.clone(), kh.clone(), vh.clone(), f["position"],
                                     torch.tensor(c["pad_counts"]), heads=h, **args).float()
    q, kk, vv, r = weights["qkvr"].split([h * hd, hk * hd, hk * hd, h * dr])
    total = torch.zeros_like(whole)
    for rank in range(2):
        hs, ks = slice(rank * h // 2 * hd, (rank + 1) * h // 2 * hd), slice(rank * hk // 2 * hd, (rank + 1) * hk // 2 * hd)
        part = dict(qkvr=torch.cat([q[hs], kk[ks], vv[ks], r[rank * h // 2 * dr:(rank + 1) * h // 2 * dr]]), o=weights["o"][:, hs],
                    q_norm=weights["q_norm"], k_norm=weights["k_norm"], k_taps=weights["k_taps"][ks], v_taps=weights["v_taps"][ks],
                    rel_proj=weights["rel_proj"])
        kv = slice(rank * hk // 2, (rank + 1) * hk // 2)
        out = oa.attention_decode_step(hidden, part, k[:, kv].clone(), v[:, kv].clone(), kh[:, ks].clone(), vh[:, ks].clone(),
                                       f["position"], torch.tensor(c["pad_counts"]), heads=h // 2,
                                       **dict(args, kv_heads=hk // 2))
        total += out.float()
    assert (total - whole).abs().max() <= 2e-2 * whole.abs().max()

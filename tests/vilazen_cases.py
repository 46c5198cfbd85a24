"""Small Vilazen configurations for the tests, and how a model with tensors the test controls is built.

The configurations differ from one another in every size and option: groups of 1, 2, 3 and 4 query heads a
key/value head; key sizes above, below and equal to the value size; heads of 64 and 128 and heads that are no multiple
of 8; rotation over the whole head, a part of it and two dimensions; windows of 1, 2, 7, 9, 66, 70 and 130 positions
and none, with 0, 1, 3, 5 and 64 first tokens kept; value mixing over layers whose heads differ; latents that fill
a tensor-core head and latents that do not; more than sixteen latent heads; decays of exactly one; layers without
a feed-forward; every kind of layer first, last and twice.
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, Optional

import torch


def _att(heads, kv, dim, vdim, scale, rot_dims, base, mask=None, v_mix=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]} if len(mask) > 1 else {"size": mask[0]}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return m


def _lat(heads, dim, rot_dim, vdim, rank, scale, base, window=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _par(left, left_scale, heads, dim, vdim, decay, right_scale):
    return {"left": left, "left_scale": left_scale, "right_scale": right_scale,
            "right": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


# sizes that are no multiple of 8, groups of 3, 1 and 4, small windows that every prompt crosses many times
CFG_A = {
    "architecture": "Vilazen", "vocab": 157, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _att(6, 2, 24, 40, 0.3, 16, 100.0, (9, 3), True), "mlp": {"kind": "dense", "ff": 136}},
        {"type": "parallel", "mixer": _par(_att(3, 3, 20, 12, 0.25, 20, 1000.0), 0.7, 3, 12, 20, [0.5, 0.9, 0.99], 1.3),
         "mlp": None},
        {"type": "latent_attention", "mixer": _lat(5, 12, 6, 10, 21, 0.3, 50.0, 7), "mlp": {"kind": "dense", "ff": 60}},
        {"type": "attention", "mixer": _att(4, 1, 16, 80, 0.35, 2, 7.0, (70, 0), True), "mlp": {"kind": "dense", "ff": 50}},
        {"type": "attention", "mixer": _att(2, 2, 8, 8, 0.5, 8, 30.0), "mlp": None},
    ],
}
# the head sizes of the tensor-core kernels (64 and 128), windows around a page's length, eighteen latent heads
CFG_B = {
    "architecture": "Vilazen", "vocab": 300, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": _lat(4, 32, 32, 48, 96, 0.15, 10000.0, 70), "mlp": {"kind": "dense", "ff": 200}},
        {"type": "attention", "mixer": _att(4, 2, 64, 64, 0.12, 32, 10000.0, (66, 5), True), "mlp": {"kind": "dense", "ff": 96}},
        {"type": "parallel", "mixer": _par(_att(4, 1, 128, 128, 0.09, 64, 500.0), 1.25, 2, 64, 64, [1.0, 0.95], 0.8),
         "mlp": {"kind": "dense", "ff": 64}},
        {"type": "attention", "mixer": _att(2, 2, 64, 64, 0.12, 64, 1000.0, (130, 64), True), "mlp": None},
        {"type": "latent_attention", "mixer": _lat(18, 16, 16, 8, 48, 0.2, 100.0), "mlp": {"kind": "dense", "ff": 72}},
    ],
}
# the values that make mechanisms vanish: one head, a window of one position, one kept token, one pair rotated
CFG_C = {
    "architecture": "Vilazen", "vocab": 61, "width": 40, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "parallel", "mixer": _par(_att(1, 1, 6, 4, 0.6, 2, 50.0), 1.0, 1, 5, 3, [1.0], 1.0),
         "mlp": {"kind": "dense", "ff": 8}},
        {"type": "attention", "mixer": _att(1, 1, 4, 6, 0.7, 4, 9.0, (1, 1), False), "mlp": {"kind": "dense", "ff": 24}},
        {"type": "latent_attention", "mixer": _lat(1, 3, 2, 5, 8, 0.5, 20.0, 2), "mlp": None},
        {"type": "parallel", "mixer": _par(_att(2, 1, 10, 10, 0.4, 6, 300.0), -0.5, 2, 33, 35, [0.3, 0.999], 2.0),
         "mlp": {"kind": "dense", "ff": 16}},
    ],
}
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def lively(w: Dict[str, torch.Tensor]) -> None:
    """Biases of the size of the projections' outputs (a lost bias shows), sinks of the size of the scores (a sink
    that is left out, or scaled, shows) and mixing weights well inside (0, 1)."""
    for name, t in w.items():
        if name.endswith(".b"):
            t.copy_((t.float() * 3.0).to(t.dtype))
        if name.endswith(".sink"):
            t.copy_((t.float() * 10.0 + 0.5).to(t.dtype))
        if name.endswith(".vmix"):
            t.fill_(0.375)


def build(cfg: dict, seed: int, dn: str, tweak: Optional[Callable] = lively, std: float = 0.12, **options):
    """(engine, config dictionary, tensors on the CPU) of a model with random weights, changed by ``tweak``."""
    from tikalix_cases import build as build_any
    return build_any(cfg, seed, dn, tweak=tweak, std=std, **options)


def plain(cfg: dict, w: Dict[str, torch.Tensor], dn: str):
    import plain_vilazen
    return plain_vilazen.PlainVilazen(cfg, w, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dn])


def rows_close(got: torch.Tensor, want: torch.Tensor, dn: str, what: str = "") -> None:
    """Row by row: the difference of the logits (mean taken off, root mean square over the vocabulary) relative to the
    root mean square of the row.  float32: every row within 3e-5.  bfloat16: all rows but one in fifteen (or two)
    within 0.04, and those within 0.3."""
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    d = got - want
    d = d - d.mean(dim=1, keepdim=True)
    ref = want - want.mean(dim=1, keepdim=True)
    err = d.pow(2).mean(dim=1).sqrt() / ref.pow(2).mean(dim=1).sqrt().clamp_min(1e-6)
    assert torch.isfinite(err).all(), f"{what}: a row is not finite"
    if dn == "float32":
        assert err.max().item() < 3e-5, f"{what}: row {int(err.argmax())} differs by {err.max().item():.3g}"
    else:
        over = int((err > 0.04).sum())
        assert err.max().item() < 0.3 and over <= max(2, got.shape[0] // 15), \
            f"{what}: {over} of {got.shape[0]} rows differ, the worst (row {int(err.argmax())}) by {err.max().item():.3g}"

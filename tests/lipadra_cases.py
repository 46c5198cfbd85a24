"""Small Lipadra configurations for the tests, and how a model with tensors the test controls is built.

The configurations differ from one another in every size and option: groups of 1, 2, 3 and 5 query heads a key/value
head; key sizes above, below and equal to the value size; heads of 64 and heads that are no multiple of 8; rotation
over the whole head, a part of it and two dimensions; chunks of 1, 7, 48, 64, 100 and 130 positions and none; decays
of exactly one; scans with 3 to 40 states, convolutions of 1 to 5 taps and step-size ranks of 1 to 20; routers with
and without identity experts, groups and a shared expert, one expert a token; layers without a feed-forward; layers
that run with another layer's tensors, before and behind it; every kind of layer first, last and twice.
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, Optional

import torch


def _att(heads, kv, dim, vdim, scale, rot_dims, base, chunk=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def _ret(heads, dim, vdim, decay, rot_dims, base):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"dims": rot_dims, "base": base}}


def _ssm(inner, state, conv, dt_rank):
    return {"inner": inner, "state": state, "conv": conv, "dt_rank": dt_rank}


def _moe(experts, identity, top, scale, ff, groups=None, shared=None):
    r = {"experts": experts, "identity": identity, "top": top, "scale": scale}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r, "shared": None if shared is None else {"ff": shared}}


def _shared(layer: dict, owner: int) -> dict:
    out = copy.deepcopy(layer)
    out["weights_of"] = owner
    return out


def _model(vocab, width, eps, alpha, layers):
    return {"architecture": "Lipadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "layers": layers}


# sizes that are no multiple of 8, groups of 3 and 1, small chunks that every prompt crosses many times
_A = [
    {"type": "attention", "mixer": _att(6, 2, 24, 40, 0.3, 16, 100.0, 7), "mlp": _moe(5, 3, 2, 1.5, 36, (4, 2), 20)},
    {"type": "mamba1", "mixer": _ssm(52, 5, 3, 3), "mlp": None},
    {"type": "retention", "mixer": _ret(3, 12, 20, [0.5, 0.9, 1.0], 6, 50.0), "mlp": _moe(7, 0, 3, 0.7, 28, None, None)},
    {"type": "attention", "mixer": _att(4, 4, 16, 8, 0.35, 2, 7.0), "mlp": _moe(4, 2, 1, 2.0, 44, (3, 1), 12)},
]
CFG_A = _model(157, 72, 1e-5, 2.0, [_A[0], _A[1], _A[2], _shared(_A[0], 0), _A[3], _shared(_A[2], 2), _shared(_A[1], 1)])
# the head sizes of the tensor-core kernels, chunks around a page's length, the state counts the scan is compiled for
_B = [
    {"type": "retention", "mixer": _ret(4, 64, 32, [0.96, 0.99, 0.999, 0.9], 64, 10000.0), "mlp": _moe(8, 4, 3, 1.75, 64, (4, 3), 64)},
    {"type": "attention", "mixer": _att(4, 2, 64, 32, 0.12, 32, 10000.0, 64), "mlp": _moe(6, 0, 2, 1.0, 96, (2, 1), None)},
    {"type": "mamba1", "mixer": _ssm(192, 16, 4, 8), "mlp": _moe(3, 1, 2, 1.0, 48, None, 32)},
    {"type": "attention", "mixer": _att(10, 2, 64, 64, 0.12, 64, 1000.0, 130), "mlp": None},
    {"type": "attention", "mixer": _att(2, 2, 48, 64, 0.14, 16, 500.0, 100), "mlp": _moe(4, 4, 3, 1.2, 40, (2, 2), 24)},
]
CFG_B = _model(300, 128, 1e-6, 3.0, [_shared(_B[1], 1), _B[1], _B[0], _B[2], _B[3], _shared(_B[0], 2), _B[4], _shared(_B[2], 3)])
# the values that make mechanisms vanish: one head, a chunk of one position, one tap, one state rank, alpha one
_C = [
    {"type": "mamba1", "mixer": _ssm(24, 40, 1, 1), "mlp": _moe(2, 1, 1, 1.0, 8, None, None)},
    {"type": "attention", "mixer": _att(1, 1, 4, 6, 0.7, 4, 9.0, 1), "mlp": _moe(1, 0, 1, 3.0, 24, None, 8)},
    {"type": "retention", "mixer": _ret(1, 5, 3, [1.0], 2, 20.0), "mlp": None},
    {"type": "mamba1", "mixer": _ssm(33, 3, 5, 20), "mlp": _moe(3, 3, 2, 0.5, 16, (3, 2), None)},
    {"type": "attention", "mixer": _att(5, 1, 10, 10, 0.4, 6, 300.0, 48), "mlp": _moe(9, 0, 4, 1.0, 12, (3, 2), 10)},
]
CFG_C = _model(61, 40, 1e-6, 1.0, _C)
# no size a multiple of 8: width, vocabulary, heads, channels, states, ranks, experts' widths
_D = [
    {"type": "attention", "mixer": _att(5, 1, 12, 6, 0.3, 6, 50.0, 9), "mlp": _moe(3, 2, 2, 1.3, 20, None, 12)},
    {"type": "retention", "mixer": _ret(3, 10, 14, [0.95, 1.0, 0.7], 10, 300.0), "mlp": _moe(5, 1, 3, 0.9, 18, (3, 2), None)},
    {"type": "mamba1", "mixer": _ssm(50, 6, 2, 5), "mlp": _moe(2, 0, 1, 1.0, 26, None, 10)},
]
CFG_D = _model(97, 52, 1e-5, 2.5, [_D[0], _D[1], _D[2], _shared(_D[1], 1)])
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def lively(w: Dict[str, torch.Tensor]) -> None:
    """Biases of the size of the projections' outputs (a lost bias shows), routers with larger weights (logits well
    apart: a close call of the router is rare), offsets that move choices, decays A of everyday size, and a gate of
    the shared expert away from one half."""
    for name, t in w.items():
        f = t.float()
        if name.endswith(".b") and ".dt." not in name:
            t.copy_((f * 3.0).to(t.dtype))
        elif name.endswith(".mlp.router"):
            t.copy_((f * 4.0).to(t.dtype))
        elif name.endswith(".mlp.correction"):
            t.copy_((f * 0.5).to(t.dtype))
        elif name.endswith(".mlp.shared.sg"):
            t.copy_((f * 6.0).to(t.dtype))
        elif name.endswith(".mix.A_log"):
            t.copy_((f * 4.0 - 0.5).to(t.dtype))
        elif name.endswith(".mix.dt.b"):
            t.copy_((f * 5.0 - 1.0).to(t.dtype))
        elif name.endswith(".mix.dt"):
            t.copy_((f * 3.0).to(t.dtype))
        elif name.endswith(".mix.D"):
            t.copy_((f * 4.0 + 0.5).to(t.dtype))


def build(cfg: dict, seed: int, dn: str, tweak: Optional[Callable] = lively, std: float = 0.12, **options):
    """(engine, config dictionary, tensors on the CPU) of a model with random weights, changed by ``tweak``."""
    from tikalix_cases import build as build_any
    return build_any(cfg, seed, dn, tweak=tweak, std=std, **options)


def plain(cfg: dict, w: Dict[str, torch.Tensor], dn: str):
    import plain_lipadra
    return plain_lipadra.PlainLipadra(cfg, w, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dn])


def rows_close(got: torch.Tensor, want: torch.Tensor, dn: str, what: str = "") -> None:
    """Row by row: the difference of the logits (mean taken off, root mean square over the vocabulary) relative to the
    root mean square of the row.  float32: every row within 5e-5.  bfloat16: all rows but one in ten (or two) within
    0.05 (a router's close call may send a token to another expert), and those within 1."""
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    d = got - want
    d = d - d.mean(dim=1, keepdim=True)
    ref = want - want.mean(dim=1, keepdim=True)
    err = d.pow(2).mean(dim=1).sqrt() / ref.pow(2).mean(dim=1).sqrt().clamp_min(1e-6)
    assert torch.isfinite(err).all(), f"{what}: a row is not finite"
    if dn == "float32":
        assert err.max().item() < 5e-5, f"{what}: row {int(err.argmax())} differs by {err.max().item():.3g}"
    else:
        over = int((err > 0.05).sum())
        assert err.max().item() < 1.0 and over <= max(2, got.shape[0] // 10), \
            f"{what}: {over} of {got.shape[0]} rows differ, the worst (row {int(err.argmax())}) by {err.max().item():.3g}"

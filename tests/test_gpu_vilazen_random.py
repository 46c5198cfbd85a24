"""Vilazen models whose every size, option and order of layers is drawn at random (widths 96 to 320; groups of 1 to 4
query heads a key/value head; heads of 16 to 128 with values of another size; rotations over the whole head, a part and
one pair; windows of 1 to 500 with 0 to 100 kept tokens, also more kept tokens than the window is long; decays from 0.3
to exactly 1; latents that fill a tensor-core head and latents that do not; layers without a feed-forward), through
the engine against the plain implementation."""
import random

import pytest
import torch

import vilazen_cases as VC
from helpers import random_tokens
from test_gpu_model import run_batches

pytestmark = pytest.mark.gpu


def random_config(rng):
    """Three to seven layers of random kinds and sizes; value-mixing layers share the first one's values a token."""
    width = rng.choice([96, 128, 160, 224, 256, 320])
    def att(bias_free=True, mask=True, vmix=None):
        G = rng.choice([1, 2, 4])
        H = G * rng.choice([1, 2, 3, 4])
        dim = rng.choice([32, 64, 128, 48, 96])
        vdim = rng.choice([dim, 32, 64, 128, 16, 72])
        dims = rng.choice([dim, dim // 2, dim // 4, 2])
        dims -= dims % 2
        m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": rng.choice([dim ** -0.5, 0.1, 0.2]),
             "rot": {"dims": max(2, dims), "base": rng.choice([10000.0, 300000.0, 100.0, 1e6])}}
        if mask:
            m["mask"] = {"size": rng.choice([1, 5, 33, 64, 70, 100, 128, 200, 500]), "keep_first": rng.choice([0, 1, 4, 24, 64, 65, 100])}
        if vmix is not None:
            m["v_mix"] = vmix
        return m
    layers = []
    n = rng.randint(3, 7)
    vm = None
    for i in range(n):
        kind = rng.choice(["attention", "parallel", "latent_attention"])
        if kind == "attention":
            use = rng.random() < 0.7
            m = att(vmix=use if rng.random() < 0.8 else None)
            if use and m.get("v_mix"):
                if vm is None:
                    vm = (m["kv_heads"], m["vdim"])
                else:
                    m["kv_heads"], m["vdim"] = vm
                    m["heads"] = vm[0] * rng.choice([1, 2, 3])
        elif kind == "parallel":
            left = att(mask=False)
            H = rng.choice([1, 2, 4, 6])
            m = {"left": left, "left_scale": rng.choice([1.0, 1.2, 0.5]), "right_scale": rng.choice([1.0, 1.1, 0.7]),
                 "right": {"heads": H, "dim": rng.choice([16, 32, 64, 128, 24]), "vdim": rng.choice([16, 32, 64, 128, 40]),
                           "decay": [rng.choice([1.0, 0.999, 0.97, 0.9, 0.6, 0.3]) for _ in range(H)]}}
        else:
            rot = rng.choice([16, 32, 64, 8])
            rank = rng.choice([32, 48, 88, 64, 112, 40, 128])
            m = {"heads": rng.choice([2, 4, 8, 5, 16, 20]), "dim": rng.choice([16, 32, 64, 24]), "rot_dim": rot, "vdim": rng.choice([32, 72, 64, 16]),
                 "kv_rank": rank, "scale": rng.choice([0.125, 0.1, 0.2]), "rot": {"base": rng.choice([300000.0, 10000.0]), "dims": rot}}
            if rng.random() < 0.8:
                m["mask"] = {"size": rng.choice([1, 7, 64, 70, 100, 130, 300])}
        mlp = {"kind": "dense", "ff": rng.choice([64, 200, 320, 136])} if rng.random() < 0.85 else None
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Vilazen", "vocab": rng.choice([300, 512, 1000, 257]), "width": width,
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}


@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(10)))
def test_a_random_model_in_every_schedule(seed, dn):
    """Whole prompts of 1, 37, 150 and 260 tokens, a prompt of 120 then token by token, and two unequal batches in
    slots used again, against the plain implementation."""
    rng = random.Random(seed)
    cfg = random_config(rng)
    eng, cfg, w = VC.build(cfg, seed, dn)
    plain = VC.plain(cfg, w, dn)
    reqs = [random_tokens(n, cfg["vocab"], 900 + n + seed) for n in (1, 37, 150, 260)]
    want = [plain.forward(r) for r in reqs]
    # whole
    for r, wl in zip(reqs, want):
        s = eng.alloc_slot()
        got = eng.step([(s, r)], [list(range(len(r)))]).clone()
        eng.free_slot(s)
        VC.rows_close(got, wl, dn, f"whole {len(r)}")
    # prompt then decode
    r, wl = reqs[3], want[3]
    s = eng.alloc_slot()
    first = 120
    rows = [eng.step([(s, r[:first])], [list(range(first))]).clone()] + [eng.step([(s, [t])]).clone() for t in r[first:]]
    eng.free_slot(s)
    VC.rows_close(torch.cat(rows), wl, dn, "decode")
    # batch
    got = run_batches(eng, reqs, [[3, 0, 2], [1, 2, 3]], [1, 30, 100, 200])
    for i, wl in enumerate(want):
        VC.rows_close(got[i], wl, dn, f"batched {i}")

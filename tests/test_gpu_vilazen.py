"""The Vilazen design through the engine against the plain implementation (tests/plain_vilazen.py): whole prompts,
prompts then token by token, prompts in portions down to two tokens, unequal batches with slots and pages used
again, windows whose edges prompts and decoded tokens cross, kept first tokens and sinks made to show, a state that
must start at zero, long decoding, models of one kind of layer, greedy generation through ``Engine.generate``, and
a replay through ``bin/trace_run``; in float32 and in bfloat16, at three configurations that differ in every size."""
import json
import os

import pytest
import torch

import vilazen_cases as VC
from helpers import random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


class Zoo:
    """Engines and plain logits, made once per (configuration, type)."""

    def __init__(self):
        self.made = {}

    def get(self, name, dn):
        key = (name, dn)
        if key not in self.made:
            eng, cfg, w = VC.build(VC.config(name), 11, dn)
            reqs = [random_tokens(n, cfg["vocab"], 500 + n) for n in (1, 2, 63, 64, 65, 130, 201)]
            plain = VC.plain(cfg, w, dn)
            want = [plain.forward(r) for r in reqs]
            self.made[key] = (eng, cfg, w, reqs, want)
        return self.made[key]


@pytest.fixture(scope="module")
def zoo():
    return Zoo()


CASES = [(n, d) for n in ("A", "B", "C") for d in DTYPES]


@pytest.mark.parametrize("name,dn", CASES)
def test_whole_prompts_and_the_first_tokens(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    for r, wl in zip(reqs, want):          # lengths 1 and 2: the first tokens; 63, 64, 65: around a page border
        s = eng.alloc_slot()
        got = eng.step([(s, r)], [list(range(len(r)))]).clone()
        eng.free_slot(s)
        VC.rows_close(got, wl, dn, f"{name} whole, {len(r)} tokens")
    eng.cache.slots.check()


@pytest.mark.parametrize("name,dn", CASES)
def test_prompt_then_token_by_token(zoo, name, dn):
    """Decoded tokens cross every window's edge and the kept first tokens' edge, and pages behind windows are let go."""
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    for r, wl, first in ((reqs[4], want[4], 1), (reqs[5], want[5], 60), (reqs[6], want[6], 127)):
        s = eng.alloc_slot()
        rows = [eng.step([(s, r[:first])], [list(range(first))]).clone()]
        rows += [eng.step([(s, [t])]).clone() for t in r[first:]]          # the decode graph, across page borders
        eng.free_slot(s)
        VC.rows_close(torch.cat(rows), wl, dn, f"{name} {first} tokens then one by one")
    eng.cache.slots.check()


@pytest.mark.parametrize("name,dn", CASES)
def test_prompts_in_portions(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    for r, wl, cuts in ((reqs[6], want[6], [2, 2, 3, 57, 2, 64, 1, 33, 37]), (reqs[5], want[5], [64, 2, 62, 2]),
                        (reqs[4], want[4], [17, 48])):
        assert sum(cuts) == len(r)
        s = eng.alloc_slot()
        rows, at = [], 0
        for n in cuts:
            rows.append(eng.step([(s, r[at:at + n])], [list(range(n))]).clone())
            at += n
        eng.free_slot(s)
        VC.rows_close(torch.cat(rows), wl, dn, f"{name} in portions {cuts}")


@pytest.mark.parametrize("name,dn", CASES)
def test_unequal_batches_with_slots_and_pages_used_again(zoo, name, dn):
    from test_gpu_model import run_batches
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    # batch after batch in the same few slots: a page's rows and a slot's state are what the last user left
    got = run_batches(eng, reqs, [[6, 0, 3], [5, 1], [2, 4]], [150 if len(r) > 150 else max(1, len(r) - k)
                                                              for r, k in zip(reqs, (0, 1, 3, 0, 32, 30, 0))])
    for i, wl in enumerate(want):
        VC.rows_close(got[i], wl, dn, f"{name} batched, request {i}")
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "bfloat16"), ("C", "float32")])
def test_long_decoding(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    r, wl = reqs[6], want[6]
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:3])], [[0, 1, 2]]).clone()] + [eng.step([(s, [t])]).clone() for t in r[3:]]
    eng.free_slot(s)
    VC.rows_close(torch.cat(rows), wl, dn, f"{name} decoded for {len(r) - 3} tokens")


@pytest.mark.parametrize("name", ["A", "C"])
def test_float32_logits_do_not_depend_on_the_batch(zoo, name):
    eng, cfg, w, reqs, want = zoo.get(name, "float32")
    r = reqs[5]
    s = eng.alloc_slot()
    whole = eng.step([(s, r)], [list(range(len(r)))]).clone()
    eng.free_slot(s)
    s, other = eng.alloc_slot(), eng.alloc_slot()
    a = eng.step([(other, reqs[3]), (s, r[:70])], [[], list(range(70))]).clone()
    b = torch.cat([eng.step([(other, [1]), (s, [t])], [[], [0]]).clone() for t in r[70:]])
    eng.free_slot(s); eng.free_slot(other)
    assert (torch.cat([a, b]) - whole).abs().max().item() <= 5e-5 * whole.abs().max().item()


def _one_layer(layer, vocab=90, width=64):
    return {"architecture": "Vilazen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [layer]}


def _standing_out(dn, keep_first, window):
    """One attention layer whose query and key are made from different halves of the residual stream through the same
    matrix, and an embedding in which token 5's first half is token 7's second half: where token 5 asks, its score at a
    position that holds token 7 stands out (the rotation is kept to two dimensions that carry nothing; the norm of q and
    k has a weight of one)."""
    cfg = _one_layer({"type": "attention", "mixer": VC._att(2, 1, 32, 32, 0.4, 2, 10000.0, (window, keep_first), False),
                      "mlp": None})
    half = cfg["width"] // 2

    def tweak(w):
        p = "l0.mix."
        w[p + "q"][:, half:] = 0
        w[p + "k"][:, :half] = 0
        w[p + "k"][:, half:] = w[p + "q"][:32, :half]
        w[p + "q"][32:, :half] = w[p + "q"][:32, :half]
        for n in ("q", "k"):
            rows = w[p + n].view(-1, 32, w[p + n].shape[1])
            rows[:, 0] = 0
            rows[:, 1] = 0
            w[p + n + ".norm"].fill_(1.0)
        w["embed.norm"].zero_(); w["l0.norm1"].zero_()
        w["embed"][5, :half] = w["embed"][7, half:] * 3.0
        w["embed"][7, half:] *= 3.0
        w["embed"][5, half:] = 0

    return cfg, tweak


@pytest.mark.parametrize("dn", DTYPES)
def test_kept_first_tokens_just_inside_and_just_outside(dn):
    """A key that stands out sits at the last kept position (seen from hundreds of tokens and several pages away, in a
    prompt and by a decoded token) or at the first position that is not kept (seen only while the window covers it)."""
    keep, window = 3, 40
    cfg, tweak = _standing_out(dn, keep, window)
    eng, cfg, w = VC.build(cfg, 3, dn, tweak=tweak, max_seq_len=512)
    plain = VC.plain(cfg, w, dn)
    filler = [t if t not in (5, 7) else 6 for t in random_tokens(300, cfg["vocab"], 9)]
    for at, shows in ((keep - 1, True), (keep, False)):
        toks = list(filler)
        toks[at] = 7
        toks[-1] = 5
        want = plain.forward(toks)
        quiet = list(toks); quiet[at] = 6
        moved = (want[-1] - plain.forward(quiet)[-1]).abs().max() > 0.2 * want[-1].abs().max()
        assert bool(moved) == shows                      # the oracle itself: the key matters exactly where it is kept
        for first in (len(toks) - 1, len(toks)):          # the last token decoded alone, and as the end of the prompt
            s = eng.alloc_slot()
            rows = [eng.step([(s, toks[:first])], [list(range(first))]).clone()]
            rows += [eng.step([(s, [t])]).clone() for t in toks[first:]]
            eng.free_slot(s)
            got = torch.cat(rows)
            VC.rows_close(got[-1:], want[-1:], dn, f"key at {at}, last row")
            if dn == "float32":
                VC.rows_close(got, want, dn, f"key at {at}")


@pytest.mark.parametrize("dn", DTYPES)
def test_window_edges_in_prompts_and_decoding(dn):
    """The same standing-out key, asked for from the last position that sees it through the window and from the next."""
    keep, window = 0, 70
    cfg, tweak = _standing_out(dn, keep, window)
    eng, cfg, w = VC.build(cfg, 4, dn, tweak=tweak, max_seq_len=512)
    plain = VC.plain(cfg, w, dn)
    filler = [t if t not in (5, 7) else 6 for t in random_tokens(200, cfg["vocab"], 19)]
    at = 60                                              # the key; position 129 is the last that sees it
    for ask, shows in ((at + window - 1, True), (at + window, False)):
        toks = list(filler[:ask + 1])
        toks[at], toks[ask] = 7, 5
        want = plain.forward(toks)
        quiet = list(toks); quiet[at] = 6
        moved = (want[-1] - plain.forward(quiet)[-1]).abs().max() > 0.2 * want[-1].abs().max()
        assert bool(moved) == shows
        for first in (ask - 3, ask + 1):
            s = eng.alloc_slot()
            rows = [eng.step([(s, toks[:first])], [list(range(first))]).clone()]
            rows += [eng.step([(s, [t])]).clone() for t in toks[first:]]
            eng.free_slot(s)
            VC.rows_close(torch.cat(rows)[-1:], want[-1:], dn, f"asked from {ask}")


@pytest.mark.parametrize("dn", DTYPES)
def test_a_sink_takes_its_share(dn):
    """Sinks far above the scores: nearly all of the softmax goes to them, and the attention's output nearly vanishes."""
    layer = {"type": "parallel", "mlp": None,
             "mixer": VC._par(VC._att(4, 2, 16, 16, 0.3, 8, 100.0), 1.0, 2, 8, 8, [0.9, 0.5], 1e-6)}
    cfg = _one_layer(layer)

    def big(w):
        VC.lively(w)
        w["l0.mix.left.sink"].copy_(torch.tensor([9.0, -30.0, 9.0, 0.0]).to(w["l0.mix.left.sink"]))

    eng, cfg, w = VC.build(cfg, 6, dn, tweak=big)
    toks = random_tokens(90, cfg["vocab"], 2)
    want = VC.plain(cfg, w, dn).forward(toks)
    flat = {k: v.clone() for k, v in w.items()}
    flat["l0.mix.left.sink"].fill_(-30.0)
    assert (want - VC.plain(cfg, flat, dn).forward(toks)).abs().max() > 0.05 * want.abs().max()
    s = eng.alloc_slot()
    rows = [eng.step([(s, toks[:70])], [list(range(70))]).clone()] + [eng.step([(s, [t])]).clone() for t in toks[70:]]
    eng.free_slot(s)
    VC.rows_close(torch.cat(rows), want, dn, "sinks")


@pytest.mark.parametrize("dn", DTYPES)
def test_a_state_starts_at_zero_in_a_slot_used_before(dn):
    """A model of linear attention alone (the left side scaled away): a second request in the slot of a first one must
    not see its state, and a request cut into steps carries its own."""
    layer = {"type": "parallel", "mlp": None,
             "mixer": VC._par(VC._att(1, 1, 8, 8, 0.3, 2, 100.0), 1e-6, 3, 24, 40, [1.0, 0.97, 0.6], 1.0)}
    cfg = _one_layer(layer, width=48)
    eng, cfg, w = VC.build(cfg, 8, dn, max_batch=1)
    plain = VC.plain(cfg, w, dn)
    a, b = random_tokens(150, cfg["vocab"], 1), random_tokens(77, cfg["vocab"], 2)
    s = eng.alloc_slot()
    eng.step([(s, a)])
    eng.free_slot(s)
    s2 = eng.alloc_slot()
    assert s2 == s
    rows = [eng.step([(s2, b[:33])], [list(range(33))]).clone(), eng.step([(s2, b[33:35])], [[0, 1]]).clone()]
    rows += [eng.step([(s2, [t])]).clone() for t in b[35:]]
    eng.free_slot(s2)
    VC.rows_close(torch.cat(rows), plain.forward(b), dn, "state in a slot used before")


@pytest.mark.parametrize("dn", DTYPES)
@pytest.mark.parametrize("kind", ["latent", "attention"])
def test_models_of_one_kind_of_layer(dn, kind):
    if kind == "latent":
        layers = [{"type": "latent_attention", "mixer": VC._lat(3, 8, 4, 16, 12, 0.4, 77.0, 5), "mlp": {"kind": "dense", "ff": 40}},
                  {"type": "latent_attention", "mixer": VC._lat(2, 16, 8, 8, 56, 0.3, 1000.0), "mlp": None}]
    else:
        layers = [{"type": "attention", "mixer": VC._att(4, 4, 8, 16, 0.4, 4, 77.0, (6,), True), "mlp": None},
                  {"type": "attention", "mixer": VC._att(2, 1, 24, 64, 0.3, 24, 1000.0, (33, 33), True), "mlp": {"kind": "dense", "ff": 24}},
                  {"type": "attention", "mixer": VC._att(8, 8, 16, 8, 0.3, 16, 1000.0, (64, 1), True), "mlp": None}]
    cfg = {"architecture": "Vilazen", "vocab": 120, "width": 56, "norm": {"eps": 1e-5}, "layers": layers}
    eng, cfg, w = VC.build(cfg, 17, dn)
    r = random_tokens(140, cfg["vocab"], 5)
    want = VC.plain(cfg, w, dn).forward(r)
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:90])], [list(range(90))]).clone()] + [eng.step([(s, [t])]).clone() for t in r[90:]]
    eng.free_slot(s)
    VC.rows_close(torch.cat(rows), want, dn, f"{kind} layers only")


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_entry_point(name, dn):
    from ziglm_b200 import GenerationOptions, SamplerParams
    eng, cfg, w = VC.build(VC.config(name), 5, dn, std=0.3)       # large weights: well separated logits
    prompts = [random_tokens(n, cfg["vocab"], 70 + n) for n in (3, 40, 9)]
    results, stats = eng.generate(prompts, GenerationOptions(max_tokens=8, ignore_eos=True,
                                                             sampler=SamplerParams(greedy=True)))
    plain = VC.plain(cfg, w, dn)
    for p, r in zip(prompts, results):
        seq = list(p)
        assert len(r.tokens) == 8
        for tok in r.tokens:
            row = plain.forward(seq)[-1]
            slack = 0.0 if dn == "float32" else 0.05 * row.std().item()
            assert row.max().item() - row[tok].item() <= slack, f"token {tok} after {len(seq)} tokens"
            seq.append(tok)
    assert stats.completion_tokens == 24


def test_replay_from_a_folder(tmp_path):
    """A folder written by the library, loaded by name of the architecture and replayed by ``bin/trace_run``."""
    from safetensors.torch import load_file
    from test_gpu_replay import Replay
    from ziglm_b200 import config_from_dict, write_random_model
    cfg = VC.config("C")
    folder = str(tmp_path / "model")
    write_random_model(folder, config_from_dict(cfg), 8, dtype=torch.bfloat16, std=0.12, norm_jitter=0.1, device="cuda")
    w = load_file(os.path.join(folder, "model.safetensors"))
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Vilazen"
    reqs = [random_tokens(n, cfg["vocab"], 30 + n) for n in (70, 9)]
    for dn in DTYPES:
        plain = VC.plain(cfg, w, dn)
        want = [plain.forward(r) for r in reqs]
        rp = Replay(folder, dn, str(tmp_path / ("logits_" + dn)), max_tokens=256)
        try:
            first = rp.step([{"id": "a", "tokens": reqs[0][:40], "want": list(range(40))},
                             {"id": "b", "tokens": reqs[1][:5], "want": [0, 4]}])
            VC.rows_close(first, torch.cat([want[0][:40], want[1][[0, 4]]]), dn, "replay, first step")
            for i in range(4):
                got = rp.step([{"id": "a", "tokens": [reqs[0][40 + i]], "want": [0]},
                               {"id": "b", "tokens": [reqs[1][5 + i]], "want": [0]}], end=["b"] if i == 3 else [])
                VC.rows_close(got, torch.stack([want[0][40 + i], want[1][5 + i]]), dn, f"replay, step {i + 1}")
            for i in range(44, 70):
                got = rp.step([{"id": "a", "tokens": [reqs[0][i]], "want": [0]}], end=["a"] if i == 69 else [])
                VC.rows_close(got, want[0][i:i + 1], dn, f"replay, token {i}")
        finally:
            rp.close()

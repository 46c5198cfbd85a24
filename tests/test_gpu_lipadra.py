"""The Lipadra design through the engine against the plain implementation (tests/plain_lipadra.py): whole prompts,
prompts then token by token, prompts in portions down to two tokens, unequal batches with slots and pages used
again, chunks whose edges prompts and decoded tokens cross, a key made to stand out just inside and just outside a
chunk and hundreds of tokens away, the one more 1 of the softmax, states that must start at zero, long decoding, models
of one kind of layer, greedy generation through ``Engine.generate``, and a replay through ``bin/trace_run``; in
float32 and in bfloat16, at three configurations that differ in every size."""
import json
import os

import pytest
import torch

import lipadra_cases as LC
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
            eng, cfg, w = LC.build(LC.config(name), 11, dn)
            reqs = [random_tokens(n, cfg["vocab"], 500 + n) for n in (1, 2, 63, 64, 65, 130, 201)]
            plain = LC.plain(cfg, w, dn)
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
        LC.rows_close(got, wl, dn, f"{name} whole, {len(r)} tokens")
    eng.cache.slots.check()


@pytest.mark.parametrize("name,dn", CASES)
def test_prompt_then_token_by_token(zoo, name, dn):
    """Decoded tokens cross every chunk's edge, pages behind the running chunk are let go, states are carried."""
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    for r, wl, first in ((reqs[4], want[4], 1), (reqs[5], want[5], 60), (reqs[6], want[6], 127)):
        s = eng.alloc_slot()
        rows = [eng.step([(s, r[:first])], [list(range(first))]).clone()]
        rows += [eng.step([(s, [t])]).clone() for t in r[first:]]          # the decode graph, across page borders
        eng.free_slot(s)
        LC.rows_close(torch.cat(rows), wl, dn, f"{name} {first} tokens then one by one")
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
        LC.rows_close(torch.cat(rows), wl, dn, f"{name} in portions {cuts}")


@pytest.mark.parametrize("name,dn", CASES)
def test_unequal_batches_with_slots_and_pages_used_again(zoo, name, dn):
    from test_gpu_model import run_batches
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    # batch after batch in the same few slots: a page's rows and a slot's state are what the last user left
    got = run_batches(eng, reqs, [[6, 0, 3], [5, 1], [2, 4]], [150 if len(r) > 150 else max(1, len(r) - k)
                                                              for r, k in zip(reqs, (0, 1, 3, 0, 32, 30, 0))])
    for i, wl in enumerate(want):
        LC.rows_close(got[i], wl, dn, f"{name} batched, request {i}")
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "bfloat16"), ("C", "float32")])
def test_long_decoding(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    r, wl = reqs[6], want[6]
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:3])], [[0, 1, 2]]).clone()] + [eng.step([(s, [t])]).clone() for t in r[3:]]
    eng.free_slot(s)
    LC.rows_close(torch.cat(rows), wl, dn, f"{name} decoded for {len(r) - 3} tokens")


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_float32_logits_do_not_depend_on_the_batch_beyond_rounding(zoo, name):
    eng, cfg, w, reqs, want = zoo.get(name, "float32")
    r = reqs[5]
    s = eng.alloc_slot()
    whole = eng.step([(s, r)], [list(range(len(r)))]).clone()
    eng.free_slot(s)
    s, other = eng.alloc_slot(), eng.alloc_slot()
    a = eng.step([(other, reqs[3]), (s, r[:70])], [[], list(range(70))]).clone()
    b = torch.cat([eng.step([(other, [1]), (s, [t])], [[], [0]]).clone() for t in r[70:]])
    eng.free_slot(s); eng.free_slot(other)
    # the scans compose their chunks' maps, so a prompt and its decoded tokens agree to rounding, not to the bit
    assert (torch.cat([a, b]) - whole).abs().max().item() <= 5e-5 * whole.abs().max().item()


@pytest.mark.parametrize("dn", DTYPES)
def test_sizes_that_are_no_multiple_of_eight(zoo, dn):
    """Width 52, vocabulary 97, heads of 12 and 10 with values of 6 and 14, 50 channels of 6 states: whole prompts, a
    prompt then token by token, and portions."""
    eng, cfg, w, reqs, want = zoo.get("D", dn)
    for r, wl in zip(reqs, want):
        s = eng.alloc_slot()
        got = eng.step([(s, r)], [list(range(len(r)))]).clone()
        eng.free_slot(s)
        LC.rows_close(got, wl, dn, f"D whole, {len(r)} tokens")
    r, wl = reqs[5], want[5]
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:31])], [list(range(31))]).clone(), eng.step([(s, r[31:33])], [[0, 1]]).clone()]
    rows += [eng.step([(s, [t])]).clone() for t in r[33:]]
    eng.free_slot(s)
    LC.rows_close(torch.cat(rows), wl, dn, "D in portions, then one by one")
    eng.cache.slots.check()


def _one_layer(layer, vocab=90, width=64, alpha=1.0):
    return {"architecture": "Lipadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "postln_alpha": alpha,
            "layers": [layer]}


def _standing_out(chunk, heads=2, kv=1, dim=32, vdim=32):
    """One attention layer whose query and key are made from different halves of the residual stream through the same
    matrix, and an embedding in which token 5's first half is token 7's second half: where token 5 asks, its score at a
    position that holds token 7 stands out (the rotation is kept to two dimensions that carry nothing; the norms of q
    and k have a weight of one and no bias moves them)."""
    cfg = _one_layer({"type": "attention", "mixer": LC._att(heads, kv, dim, vdim, 0.5, 2, 10000.0, chunk), "mlp": None})
    half = cfg["width"] // 2

    def tweak(w):
        p = "l0.mix."
        w[p + "q"][:, half:] = 0
        w[p + "k"][:, :half] = 0
        w[p + "k"][:dim, half:] = w[p + "q"][:dim, :half]
        for h in range(1, heads):
            w[p + "q"][h * dim:(h + 1) * dim, :half] = w[p + "q"][:dim, :half]
        for n in ("q", "k"):
            rows = w[p + n].view(-1, dim, w[p + n].shape[1])
            rows[:, 0] = 0
            rows[:, 1] = 0
            w[p + n + ".norm"].fill_(2.0)
            w[p + n + ".b"].zero_()
        w["embed"][5, :half] = w["embed"][7, half:]
        w["embed"][5, half:] = 0

    return cfg, tweak


@pytest.mark.parametrize("dn", DTYPES)
@pytest.mark.parametrize("chunk,dim,vdim", [(70, 32, 32), (64, 64, 32), (128, 24, 40)])
def test_a_key_just_inside_and_just_outside_the_chunk(dn, chunk, dim, vdim):
    """The key that stands out sits at the first position of the asking token's chunk (seen from the chunk's last
    position, in a prompt and by a decoded token) or at the position before it (the chunk before: never seen)."""
    cfg, tweak = _standing_out(chunk, dim=dim, vdim=vdim)
    eng, cfg, w = LC.build(cfg, 3, dn, tweak=tweak, max_seq_len=512)
    plain = LC.plain(cfg, w, dn)
    filler = [t if t not in (5, 7) else 6 for t in random_tokens(3 * chunk, cfg["vocab"], 9)]
    ask = 3 * chunk - 1                                   # the last position of the third chunk
    for at, shows in ((2 * chunk, True), (2 * chunk - 1, False)):
        toks = list(filler)
        toks[at], toks[ask] = 7, 5
        want = plain.forward(toks)
        quiet = list(toks); quiet[at] = 6
        moved = (want[-1] - plain.forward(quiet)[-1]).abs().max() > 0.2 * want[-1].abs().max()
        assert bool(moved) == shows                       # the oracle itself: the key matters exactly inside the chunk
        for first in (ask, ask + 1, 2 * chunk + 1):       # the last token decoded alone, as the end of the prompt,
            s = eng.alloc_slot()                          # and after a chunk of decoded tokens
            rows = [eng.step([(s, toks[:first])], [list(range(first))]).clone()]
            rows += [eng.step([(s, [t])]).clone() for t in toks[first:]]
            eng.free_slot(s)
            got = torch.cat(rows)
            LC.rows_close(got[-1:], want[-1:], dn, f"key at {at}, prompt of {first}, last row")
            if dn == "float32":
                LC.rows_close(got, want, dn, f"key at {at}, prompt of {first}")
    eng.cache.slots.check()


@pytest.mark.parametrize("dn", DTYPES)
def test_a_key_hundreds_of_tokens_away_without_chunks(dn):
    cfg, tweak = _standing_out(None, heads=3, kv=3, dim=64, vdim=64)
    eng, cfg, w = LC.build(cfg, 5, dn, tweak=tweak, max_seq_len=1024)
    plain = LC.plain(cfg, w, dn)
    toks = [t if t not in (5, 7) else 6 for t in random_tokens(700, cfg["vocab"], 4)]
    toks[3], toks[-1] = 7, 5
    want = plain.forward(toks)
    quiet = list(toks); quiet[3] = 6
    assert (want[-1] - plain.forward(quiet)[-1]).abs().max() > 0.2 * want[-1].abs().max()
    for first in (699, 700, 300):
        s = eng.alloc_slot()
        rows = [eng.step([(s, toks[:first])], [[first - 1]]).clone()]
        rows += [eng.step([(s, [t])]).clone() for t in toks[first:]]
        eng.free_slot(s)
        LC.rows_close(torch.cat(rows)[-1:], want[-1:], dn, f"far key, prompt of {first}")


@pytest.mark.parametrize("dn", DTYPES)
def test_the_one_more_one_of_the_softmax_shows(dn):
    """Scores far below zero: nearly all of the softmax goes to the 1 in the denominator and the attention's output
    nearly vanishes; an implementation without it would give the mean of the values."""
    cfg = _one_layer({"type": "attention", "mixer": LC._att(4, 2, 16, 16, 0.3, 8, 100.0, 40), "mlp": None})

    def low(w):
        LC.lively(w)
        w["l0.mix.q"].zero_(); w["l0.mix.k"].zero_()
        w["l0.mix.q.b"].fill_(1.0); w["l0.mix.k.b"].fill_(-1.0)
        w["l0.mix.q.norm"].fill_(4.0); w["l0.mix.k.norm"].fill_(4.0)
        w["l0.mix.v.b"].fill_(2.0)

    eng, cfg, w = LC.build(cfg, 6, dn, tweak=low)
    toks = random_tokens(90, cfg["vocab"], 2)
    want = LC.plain(cfg, w, dn).forward(toks)
    s = eng.alloc_slot()
    rows = [eng.step([(s, toks[:70])], [list(range(70))]).clone()] + [eng.step([(s, [t])]).clone() for t in toks[70:]]
    eng.free_slot(s)
    LC.rows_close(torch.cat(rows), want, dn, "one more 1")


@pytest.mark.parametrize("dn", DTYPES)
@pytest.mark.parametrize("kind", ["retention", "mamba1"])
def test_a_state_starts_at_zero_in_a_slot_used_before(dn, kind):
    """A second request in the slot of a first one must not see its state or the convolution's kept inputs, and a
    request cut into steps carries its own."""
    mixer = LC._ret(3, 24, 40, [1.0, 0.97, 0.6], 8, 100.0) if kind == "retention" else LC._ssm(40, 6, 4, 5)
    cfg = _one_layer({"type": kind, "mixer": mixer, "mlp": None}, width=48, alpha=0.5)
    eng, cfg, w = LC.build(cfg, 8, dn, max_batch=1)
    plain = LC.plain(cfg, w, dn)
    a, b = random_tokens(150, cfg["vocab"], 1), random_tokens(77, cfg["vocab"], 2)
    s = eng.alloc_slot()
    eng.step([(s, a)])
    eng.free_slot(s)
    s2 = eng.alloc_slot()
    assert s2 == s
    rows = [eng.step([(s2, b[:33])], [list(range(33))]).clone(), eng.step([(s2, b[33:35])], [[0, 1]]).clone()]
    rows += [eng.step([(s2, [t])]).clone() for t in b[35:]]
    eng.free_slot(s2)
    LC.rows_close(torch.cat(rows), plain.forward(b), dn, "state in a slot used before")


@pytest.mark.parametrize("dn", DTYPES)
@pytest.mark.parametrize("kind", ["retention", "mamba1", "attention"])
def test_models_of_one_kind_of_layer(dn, kind):
    if kind == "retention":
        layers = [{"type": "retention", "mixer": LC._ret(2, 16, 8, [0.9, 0.999], 16, 77.0), "mlp": LC._moe(4, 0, 2, 1.0, 24)},
                  {"type": "retention", "mixer": LC._ret(5, 8, 24, [1.0, 0.5, 0.8, 0.99, 0.9], 4, 1000.0), "mlp": None}]
    elif kind == "mamba1":
        layers = [{"type": "mamba1", "mixer": LC._ssm(64, 8, 2, 4), "mlp": None},
                  {"type": "mamba1", "mixer": LC._ssm(40, 24, 4, 7), "mlp": LC._moe(2, 2, 2, 1.0, 24, (2, 1), 16)},
                  {"type": "mamba1", "mixer": LC._ssm(96, 32, 3, 2), "mlp": None}]
    else:
        layers = [{"type": "attention", "mixer": LC._att(4, 4, 8, 16, 0.4, 4, 77.0, 6), "mlp": None},
                  {"type": "attention", "mixer": LC._att(2, 1, 24, 64, 0.3, 24, 1000.0, 33), "mlp": LC._moe(3, 0, 1, 2.0, 24)},
                  {"type": "attention", "mixer": LC._att(8, 8, 16, 8, 0.3, 16, 1000.0), "mlp": None}]
    cfg = {"architecture": "Lipadra", "vocab": 120, "width": 56, "norm": {"eps": 1e-5}, "postln_alpha": 1.5, "layers": layers}
    eng, cfg, w = LC.build(cfg, 17, dn)
    r = random_tokens(140, cfg["vocab"], 5)
    want = LC.plain(cfg, w, dn).forward(r)
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:90])], [list(range(90))]).clone()] + [eng.step([(s, [t])]).clone() for t in r[90:]]
    eng.free_slot(s)
    LC.rows_close(torch.cat(rows), want, dn, f"{kind} layers only")


@pytest.mark.parametrize("dn", DTYPES)
def test_a_long_prompt_of_scans_against_token_by_token(dn):
    """A prompt of a thousand tokens (the scans run it in chunks and segments) leaves the states that decoding it token by
    token would: the tokens decoded behind it agree with the plain implementation, which only ever steps."""
    layers = [{"type": "mamba1", "mixer": LC._ssm(64, 16, 4, 4), "mlp": None},
              {"type": "retention", "mixer": LC._ret(2, 32, 32, [0.99, 0.999], 32, 10000.0), "mlp": None}]
    cfg = {"architecture": "Lipadra", "vocab": 80, "width": 48, "norm": {"eps": 1e-5}, "postln_alpha": 2.0, "layers": layers}
    eng, cfg, w = LC.build(cfg, 21, dn, max_tokens=2048, max_seq_len=1100)
    r = random_tokens(1010, cfg["vocab"], 6)
    want = LC.plain(cfg, w, dn).forward(r)
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:1000])], [[0, 500, 999]]).clone()] + [eng.step([(s, [t])]).clone() for t in r[1000:]]
    eng.free_slot(s)
    LC.rows_close(torch.cat(rows), torch.cat([want[[0, 500, 999]], want[1000:]]), dn, "a thousand tokens, then ten")


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_entry_point(name, dn):
    from ziglm_b200 import GenerationOptions, SamplerParams
    eng, cfg, w = LC.build(LC.config(name), 5, dn)
    prompts = [random_tokens(n, cfg["vocab"], 70 + n) for n in (3, 40, 9)]
    results, stats = eng.generate(prompts, GenerationOptions(max_tokens=8, ignore_eos=True,
                                                             sampler=SamplerParams(greedy=True)))
    plain = LC.plain(cfg, w, dn)
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
    cfg = LC.config("C")
    folder = str(tmp_path / "model")
    write_random_model(folder, config_from_dict(cfg), 8, dtype=torch.bfloat16, std=0.12, norm_jitter=0.1, device="cuda")
    w = load_file(os.path.join(folder, "model.safetensors"))
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Lipadra"
    reqs = [random_tokens(n, cfg["vocab"], 30 + n) for n in (70, 9)]
    for dn in DTYPES:
        plain = LC.plain(cfg, w, dn)
        want = [plain.forward(r) for r in reqs]
        rp = Replay(folder, dn, str(tmp_path / ("logits_" + dn)), max_tokens=256)
        try:
            first = rp.step([{"id": "a", "tokens": reqs[0][:40], "want": list(range(40))},
                             {"id": "b", "tokens": reqs[1][:5], "want": [0, 4]}])
            LC.rows_close(first, torch.cat([want[0][:40], want[1][[0, 4]]]), dn, "replay, first step")
            for i in range(4):
                got = rp.step([{"id": "a", "tokens": [reqs[0][40 + i]], "want": [0]},
                               {"id": "b", "tokens": [reqs[1][5 + i]], "want": [0]}], end=["b"] if i == 3 else [])
                LC.rows_close(got, torch.stack([want[0][40 + i], want[1][5 + i]]), dn, f"replay, step {i + 1}")
            for i in range(44, 70):
                got = rp.step([{"id": "a", "tokens": [reqs[0][i]], "want": [0]}], end=["a"] if i == 69 else [])
                LC.rows_close(got, want[0][i:i + 1], dn, f"replay, token {i}")
        finally:
            rp.close()

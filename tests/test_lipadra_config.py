"""Lipadra without a GPU: the configuration reader and its refusals, the layout, the schedule and the tensor names it
produces, what the cache manager lets go behind a chunk, and the plain implementation's own parts on cases whose
answer is known (also: a prompt at once against the same prompt in portions, through the plain implementation)."""
import math

import pytest
import torch

import lipadra_cases as LC
import plain_lipadra as P
from ziglm_b200 import ConfigError, config_from_dict
from ziglm_b200.cache.slots import GroupPages
from ziglm_b200.engine.model import declare_parameters


def test_layout_schedule_and_names():
    conf = config_from_dict(LC.config("A"))
    spec = conf.model_spec()
    assert spec.architecture == "Lipadra" and spec.head_name is None and spec.embed_hook is None
    # four layers have tensors; three more places of the schedule run them again
    assert [l.prefix for l in spec.layers] == ["l0.", "l1.", "l2.", "l4."]
    assert spec.schedule == (0, 1, 2, 0, 3, 2, 1)
    assert [l.block for l in spec.layers] == ["sum_norm"] * 4
    assert [l.mixer.kind for l in spec.layers] == ["capped_attention", "selective_scan", "decayed_linear_attention",
                                                   "capped_attention"]
    assert all(l.options["residual_mult"] == 2.0 and l.mixer_norm is None and l.ffn_norm is None for l in spec.layers)
    names = declare_parameters(spec)
    for n, shape in (("embed", (157, 72)), ("final.norm", (72,)), ("l0.norm1", (72,)), ("l0.norm2", (72,)),
                     ("l0.mix.q", (144, 72)), ("l0.mix.q.b", (144,)), ("l0.mix.k", (48, 72)), ("l0.mix.v", (80, 72)),
                     ("l0.mix.v.b", (80,)), ("l0.mix.q.norm", (24,)), ("l0.mix.k.norm", (24,)), ("l0.mix.o", (72, 240)),
                     ("l0.mlp.router", (8, 72)), ("l0.mlp.correction", (8,)), ("l0.mlp.e4.gate", (36, 72)),
                     ("l0.mlp.e4.down", (72, 36)), ("l0.mlp.shared.up", (20, 72)), ("l0.mlp.shared.sg", (1, 72)),
                     ("l1.mix.in", (104, 72)), ("l1.mix.conv", (52, 3)), ("l1.mix.conv.b", (52,)), ("l1.mix.x", (13, 52)),
                     ("l1.mix.dt", (52, 3)), ("l1.mix.dt.b", (52,)), ("l1.mix.A_log", (52, 5)), ("l1.mix.D", (52,)),
                     ("l1.mix.o", (72, 52)), ("l2.mix.q", (36, 72)), ("l2.mix.v", (60, 72)), ("l2.mix.g", (60, 72)),
                     ("l2.mix.o", (72, 60)), ("l2.mlp.router", (7, 72)), ("l4.mix.q.norm", (16,))):
        assert tuple(names[n].shape) == shape, n
    for absent in ("head", "embed.norm", "l1.norm2", "l1.mlp.router", "l3.norm1", "l5.mix.q", "l6.mix.in", "l0.mlp.e5.gate",
                   "l2.mlp.shared.gate", "l2.mlp.shared.sg", "l2.mix.norm", "l2.mix.q.b", "l0.mix.sink", "l0.mix.g"):
        assert absent not in names, absent
    att, scan, ret, causal = (l.mixer for l in spec.layers)
    assert (att.options["chunk"], att.options["sink"], att.options["qk_norm"]) == (7, "zero", "head_first")
    assert att.window is None and att.bias
    assert causal.options["chunk"] is None and causal.position.rotary_dim == 2
    assert scan.options == {"channels": 52, "states": 5, "taps": 3, "dt_rank": 3}
    assert ret.options["decay"] == (0.5, 0.9, 1.0) and ret.options["key_scale"] == 12 ** -0.5
    assert (ret.options["norm"], ret.options["gate"], ret.position.rotary_dim) == ("head", "silu", 6)
    moe = spec.layers[0].ffn.options
    assert (moe["experts"], moe["identity"], moe["top"], moe["groups"], moe["keep_groups"], moe["group_best"]) == (5, 3, 2, 4, 2, 1)
    assert moe["weight_scale"] == 1.5 and moe["shared_gate"] and moe["score"] == "softmax" and not moe["renormalize"]
    assert spec.layers[2].ffn.options.get("shared") is None and not spec.layers[2].ffn.options.get("shared_gate")
    assert conf.to_dict() == LC.config("A")


def test_a_layer_that_runs_anothers_tensors_with_other_constants_is_a_spec_of_its_own():
    cfg = LC.config("A")
    cfg["layers"][3]["mixer"]["mask"]["size"] = 11
    spec = config_from_dict(cfg).model_spec()
    assert spec.schedule == (0, 1, 2, 4, 3, 2, 1) and spec.layers[4].prefix == "l0."
    assert spec.layers[4].mixer.options["chunk"] == 11 and spec.layers[0].mixer.options["chunk"] == 7
    assert set(declare_parameters(spec)) == set(declare_parameters(config_from_dict(LC.config("A")).model_spec()))


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), 0, "vocab"), (("norm",), 3, "norm"), (("postln_alpha",), "3", "postln_alpha"),
    (("layers", 0, "type"), "mamba2", "type"), (("layers", 0, "mixer", "heads"), 5, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 15, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 26, "rot.dims"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"), (("layers", 0, "mlp", "kind"), "dense", "kind"),
    (("layers", 0, "mlp", "router", "top"), 5, "router"), (("layers", 0, "mlp", "router", "groups", "count"), 3, "router"),
    (("layers", 0, "mlp", "router", "identity"), -1, "identity"), (("layers", 0, "mlp", "router", "scale"), None, "scale"),
    (("layers", 0, "mlp", "shared", "ff"), 0, "ff"), (("layers", 1, "mixer", "state"), 0, "state"),
    (("layers", 1, "mixer", "dt_rank"), 2.5, "dt_rank"), (("layers", 2, "mixer", "decay"), [0.5, 0.9], "decay"),
    (("layers", 2, "mixer", "decay"), [0.5, 0.9, 1.5], "decay"), (("layers", 3, "weights_of"), 3, "weights_of"),
    (("layers", 3, "weights_of"), 5, "weights_of"), (("layers", 3, "weights_of"), 1, "weights_of"),
])
def test_refusals_name_the_key(path, value, word):
    cfg = LC.config("A")
    at = cfg
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_pages_behind_the_running_chunk_are_given_back():
    g = GroupPages(12, 64, None, chunk=100)
    g.grow(0, 330)
    assert g.pages_of[0] == [0, 1, 2, 3, 4, 5]
    g.release_behind_window(0, 199)           # the next token sits at 199, in the chunk from 100 on: page 0 is done with
    assert g.pages_of[0] == [-1, 1, 2, 3, 4, 5]
    g.release_behind_window(0, 200)           # the next token opens the chunk from 200 on, which begins inside page 3
    assert g.pages_of[0] == [-1, -1, -1, 3, 4, 5] and g.pool.n_free == 9
    g.release_behind_window(0, 330)
    assert g.pages_of[0] == [-1, -1, -1, -1, 4, 5]
    g.free(0)
    assert g.pool.n_free == 12
    with pytest.raises(ValueError):
        GroupPages(4, 64, 8, chunk=8)


def test_the_plain_parts_on_known_answers():
    # chunks: position 7 opens a chunk of its own and sees itself only; position 6 sees 0..6
    seen = P.same_chunk(torch.arange(10), torch.arange(10), 7)
    assert seen[6].tolist() == [True] * 7 + [False] * 3 and seen[7].tolist() == [False] * 7 + [True] + [False] * 2
    assert seen[9].tolist() == [False] * 7 + [True] * 3
    assert P.same_chunk(torch.arange(3), torch.arange(3), None).tolist() == [[True, False, False], [True, True, False], [True] * 3]
    # one more 1 in the denominator: a single key of score 0 gets one half; scores of -inf get nothing
    p = P.softmax_one_more(torch.tensor([[0.0, 5.0]]), torch.tensor([[True, False]]))
    assert torch.allclose(p, torch.tensor([[0.5, 0.0]]))
    p = P.softmax_one_more(torch.tensor([[math.log(3.0), math.log(4.0)]]), torch.tensor([[True, True]]))
    assert torch.allclose(p, torch.tensor([[3 / 8, 4 / 8]]))
    # rotation of halves at position 1: the pair (0, 2) turns by one radian, the pair (1, 3) by base^(-1/2); 4.. pass
    x = torch.tensor([[[1.0, 2.0, 0.0, 0.0, 7.0]]])
    r = P.rotate_halves(x, torch.tensor([1]), {"dims": 4, "base": (math.pi / 2) ** -2})
    a1 = math.pi / 2                         # base = (pi/2)^-2, so the second pair's angle is a quarter turn
    assert torch.allclose(r[0, 0, [0, 2, 4]], torch.tensor([math.cos(1.0), math.sin(1.0), 7.0]), atol=1e-6)
    assert torch.allclose(r[0, 0, [1, 3]], torch.tensor([2 * math.cos(a1), 2 * math.sin(a1)]), atol=1e-6)
    # the router: groups are scored by their largest choice score, which may be negative; the weights carry no offset
    z = torch.log(torch.tensor([[0.1, 0.2, 0.3, 0.4]]))
    out = P.route(z, torch.tensor([-5.0, -5.2, -9.0, -9.0]), {"top": 1, "scale": 2.0, "groups": {"count": 2, "keep": 1}})
    assert out["ids"].tolist() == [[0]] and torch.allclose(out["weights"], torch.tensor([[0.2]]))
    out = P.route(z, torch.zeros(4), {"top": 2, "scale": 1.0})
    assert out["ids"].tolist() == [[3, 2]] and torch.allclose(out["weights"], torch.tensor([[0.4, 0.3]]))
    # the convolution: the last tap meets the current token, zeros stand before the start
    p32 = P.Plain()
    y = P.causal_conv(p32, torch.tensor([[1.0], [2.0], [3.0]]), torch.tensor([[10.0, 1.0]]), torch.tensor([0.5]), None)
    assert y.reshape(-1).tolist() == [1.5, 12.5, 23.5]
    # the scan with one channel and one state and constant inputs: S_t = a S_(t-1) + b, a geometric sum
    w = {"in": torch.tensor([[1.0], [0.0]]), "conv": torch.tensor([[1.0]]), "conv.b": torch.zeros(1), "x": torch.tensor([[0.0], [1.0], [1.0]]),
         "dt": torch.zeros(1, 1), "dt.b": torch.tensor([math.log(math.e - 1.0)]), "A_log": torch.zeros(1, 1), "D": torch.zeros(1)}
    h = torch.full((4, 1), 2.0)
    y = P.selective_scan(p32, h, w, {"inner": 1, "state": 1, "dt_rank": 1}, None)
    u = 2.0 / (1.0 + math.exp(-2.0))          # silu(2); dt = softplus(log(e - 1)) = 1, A = -1, B = C = u
    S, want = 0.0, []
    for _ in range(4):
        S = math.exp(-1.0) * S + u * u
        want.append(S * u * 0.0)              # z = 0: silu(0) = 0 closes the gate
    assert torch.allclose(y.reshape(-1), torch.tensor(want))


@pytest.mark.parametrize("name", ["A", "C"])
def test_the_plain_implementation_in_portions(name):
    """States, kept inputs of the convolution and keys are carried: a prompt at once equals the prompt in portions."""
    cfg = LC.config(name)
    conf = config_from_dict(cfg)
    g = torch.Generator().manual_seed(5)
    w = {n: torch.randn(*d.shape, generator=g) * 0.2 if d.init == "normal" else torch.ones(d.shape)
         for n, d in declare_parameters(conf.model_spec()).items()}
    LC.lively(w)
    plain = P.PlainLipadra(cfg, w, wide=True)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=g).tolist()
    whole = plain.forward(toks)
    state, rows, at = plain.new_state(), [], 0
    for n in (9, 1, 2, 17, 1, 10):
        rows.append(plain.forward(toks[at:at + n], state, at))
        at += n
    assert torch.allclose(torch.cat(rows), whole, atol=1e-9, rtol=1e-9)

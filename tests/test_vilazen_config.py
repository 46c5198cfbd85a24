"""Vilazen without a GPU: the configuration reader and its refusals, the layout and the tensor names it produces, the
order in which a rotation of adjacent pairs lays out a head, what the cache manager keeps behind a window with kept
first tokens, and the plain implementation's own parts on cases whose answer is known."""
import math

import pytest
import torch

import plain_vilazen as P
import vilazen_cases as VC
from ziglm_b200 import ConfigError, config_from_dict
from ziglm_b200.cache.slots import GroupPages
from ziglm_b200.config.spec import PositionSpec
from ziglm_b200.engine.model import declare_parameters
from ziglm_b200.parts.rope import Rope


def test_layout_and_names():
    conf = config_from_dict(VC.config("A"))
    spec = conf.model_spec()
    assert spec.architecture == "Vilazen" and spec.head_name == "head" and spec.embed_hook.kind == "rmsnorm"
    assert [l.block for l in spec.layers] == ["shared_norm"] * 5
    assert [l.mixer.kind for l in spec.layers] == ["capped_attention", "side_by_side", "latent_attention",
                                                   "capped_attention", "capped_attention"]
    assert spec.layers[1].ffn is None and spec.layers[4].ffn is None and spec.layers[0].ffn.activation == "gelu"
    names = declare_parameters(spec)
    for n, shape in (("embed", (157, 72)), ("embed.norm", (72,)), ("head", (157, 72)), ("final.norm", (72,)),
                     ("l0.norm1", (72,)), ("l0.mix.q", (144, 72)), ("l0.mix.k", (48, 72)), ("l0.mix.v", (80, 72)),
                     ("l0.mix.q.norm", (144,)), ("l0.mix.k.norm", (48,)), ("l0.mix.g", (6, 72)), ("l0.mix.o", (72, 240)),
                     ("l0.mix.vmix", ()), ("l0.mlp.up", (136, 72)), ("l0.mlp.down", (72, 136)),
                     ("l1.mix.left.q", (60, 72)), ("l1.mix.left.q.b", (60,)), ("l1.mix.left.v.b", (36,)),
                     ("l1.mix.left.sink", (3,)), ("l1.mix.left.g", (3, 72)), ("l1.mix.right.q", (36, 72)),
                     ("l1.mix.right.v", (60, 72)), ("l1.mix.right.norm", (60,)), ("l1.mix.right.g", (60, 72)),
                     ("l1.mix.right.o", (72, 60)), ("l2.mix.q", (90, 72)), ("l2.mix.dkv", (27, 72)),
                     ("l2.mix.dkv.norm", (21,)), ("l2.mix.uk", (60, 21)), ("l2.mix.uv", (50, 21)), ("l2.mix.o", (72, 50)),
                     ("l3.mix.vmix", ())):
        assert tuple(names[n].shape) == shape, n
    for absent in ("l0.norm2", "l1.mlp.up", "l0.mix.q.b", "l0.mix.sink", "l4.mix.vmix", "l2.mix.g", "l1.mix.left.q.norm"):
        assert absent not in names, absent
    first, later, plain_one = spec.layers[0].mixer, spec.layers[3].mixer, spec.layers[4].mixer
    assert (first.window, first.options["keep_first"], first.options["value_mix"]) == (9, 3, "first")
    assert (later.window, later.options["keep_first"], later.options["value_mix"]) == (70, 0, "mix")
    assert plain_one.window is None and plain_one.options.get("value_mix") is None
    left, right = (sub for _, sub in spec.layers[1].mixer.options["parts"])
    assert left.bias and left.options["sink"] and left.options["out_scale"] == 0.7 and left.window is None
    assert right.options["decay"] == (0.5, 0.9, 0.99) and right.options["out_scale"] == 1.3
    lat = spec.layers[2].mixer
    assert (lat.window, lat.options["kv_rank"], lat.options["rot_dim"], lat.options["gate"]) == (7, 21, 6, None)
    assert conf.to_dict() == VC.config("A")


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), 0, "vocab"), (("norm",), 3, "norm"), (("layers", 0, "type"), "mamba", "type"),
    (("layers", 0, "mixer", "heads"), 5, "kv_heads"), (("layers", 0, "mixer", "rot", "dims"), 15, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 26, "rot.dims"), (("layers", 0, "mixer", "v_mix"), "yes", "v_mix"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"), (("layers", 0, "mixer", "mask", "keep_first"), -1, "keep_first"),
    (("layers", 3, "mixer", "vdim"), 8, "v_mix"), (("layers", 0, "mlp", "kind"), "glu", "kind"),
    (("layers", 1, "mixer", "right", "decay"), [0.5, 0.9], "decay"), (("layers", 1, "mixer", "right", "decay"), [0.5, 0.9, 1.5], "decay"),
    (("layers", 1, "mixer", "left_scale"), None, "left_scale"), (("layers", 2, "mixer", "rot_dim"), 5, "rot_dim"),
    (("layers", 2, "mixer", "kv_rank"), None, "kv_rank"),
])
def test_refusals_name_the_key(path, value, word):
    cfg = VC.config("A")
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_adjacent_pairs_become_halves():
    """The order in which a mixer lays out a head: the even dimensions of the rotated part, the odd ones, the rest.
    Turning the halves of the reordered head is turning the adjacent pairs of the head as the file has it."""
    rope = Rope(PositionSpec(kind="rope", rotary_dim=6, theta=50.0, options={"pairs": "adjacent"}), torch.float32,
                torch.device("cpu"))
    order = rope.head_order(10)
    assert order == (0, 2, 4, 1, 3, 5, 6, 7, 8, 9)
    x = torch.arange(20, dtype=torch.float32).view(2, 1, 10) / 7.0
    pos = torch.tensor([3, 11])
    want = P.rotate_pairs(x, pos, {"dims": 6, "base": 50.0})
    y = x[:, :, list(order)].clone()
    f = torch.tensor([50.0 ** (-2 * i / 6) for i in range(3)])
    ang = pos[:, None].float() * f[None, :]
    lo, hi = y[:, 0, :3].clone(), y[:, 0, 3:6].clone()
    y[:, 0, :3] = lo * ang.cos() - hi * ang.sin()
    y[:, 0, 3:6] = hi * ang.cos() + lo * ang.sin()
    torch.testing.assert_close(y, want[:, :, list(order)])
    halves = Rope(PositionSpec(kind="rope", rotary_dim=6, theta=50.0), torch.float32, torch.device("cpu"))
    assert halves.head_order(10) is None


def test_pages_behind_a_window_are_given_back_but_for_the_kept_ones():
    """Pages of 4 positions, a window of 6 that keeps the first 5: the two first pages stay whatever the length."""
    pages = GroupPages(16, 4, 6, 5)
    pages.grow(0, 30)
    assert len(pages.pages_of[0]) == 8
    pages.release_behind_window(0, 30)                            # the next token, at 30, sees 25..30: page 6 onwards
    assert [i for i, p in enumerate(pages.pages_of[0]) if p < 0] == [2, 3, 4, 5]
    assert pages.pool.n_held == 4
    plain = GroupPages(16, 4, 6)
    plain.grow(0, 30)
    plain.release_behind_window(0, 30)
    assert [i for i, p in enumerate(plain.pages_of[0]) if p < 0] == [0, 1, 2, 3, 4, 5]
    pages.free(0)
    assert pages.pool.n_held == 0


def test_the_plain_parts_on_known_answers():
    # a window of 3 that keeps the first 2: position 6 sees 0, 1 and 4, 5, 6
    seen = P.visible(torch.tensor([6]), torch.arange(8), 3, 2)
    assert seen[0].tolist() == [True, True, False, False, True, True, True, False]
    assert P.visible(torch.tensor([2]), torch.arange(4), None)[0].tolist() == [True, True, True, False]
    # two equal scores and a sink of the same size: a third each, and the sink's third is lost
    p = P.softmax_rows(torch.zeros(1, 1, 2), torch.ones(1, 2, dtype=torch.bool), torch.zeros(1))
    torch.testing.assert_close(p, torch.full((1, 1, 2), 1.0 / 3.0))
    # the first pair turns by the position itself (f_0 = 1 whatever the base): (1, 0) at position 1 becomes (cos 1, sin 1)
    x = torch.tensor([[[1.0, 0.0, 5.0, 7.0]]])
    y = P.rotate_pairs(x, torch.tensor([1]), {"dims": 2, "base": 9.0})
    torch.testing.assert_close(y, torch.tensor([[[math.cos(1.0), math.sin(1.0), 5.0, 7.0]]]))
    # norms: eps inside the root; the weight around zero adds one
    v = torch.tensor([[3.0, 4.0]])
    torch.testing.assert_close(P.norm_plain(v, torch.tensor([2.0, 1.0]), 0.5), v / math.sqrt(12.5 + 0.5) * torch.tensor([2.0, 1.0]))
    torch.testing.assert_close(P.norm_around_zero(v, torch.tensor([1.0, 0.0]), 0.5), v / math.sqrt(13.0) * torch.tensor([2.0, 1.0]))
    torch.testing.assert_close(P.gelu_erf(torch.tensor([1.0])), torch.tensor([0.5 * (1.0 + math.erf(1.0 / math.sqrt(2.0)))]))

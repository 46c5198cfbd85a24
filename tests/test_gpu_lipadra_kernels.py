"""Each mechanism of the Lipadra design alone: the kernel, or the part that strings a few kernels together, against the
plain function that states its formula (tests/plain_lipadra.py), at sizes that are no multiple of a tile, with several
sequences in a step, shuffled pages, prompts and decoded tokens, slots used again, and inputs made so that a fault
shows."""
from types import SimpleNamespace

import pytest
import torch

import plain_lipadra as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TYPES = [torch.float32, torch.bfloat16]


def _r(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _tol(dtype, f32=(1e-5, 1e-5), bf16=(2e-2, 2e-2)):
    a, r = f32 if dtype == torch.float32 else bf16
    return dict(atol=a, rtol=r)


def _step(new, past, slots=None):
    """A step in which sequence b brings new[b] tokens behind past[b] ones, as the parts and kernels read it."""
    from ziglm_b200.engine.workspace import Workspace
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    return SimpleNamespace(
        n_tokens=cu[-1], n_seqs=len(new), single_token=all(n == 1 for n in new), max_new=max(new),
        max_total=max(p + n for p, n in zip(past, new)), positions=_i32([p + i for p, n in zip(past, new) for i in range(n)]),
        seq_of_token=_i32([b for b, n in enumerate(new) for _ in range(n)]), cu_seqlens=_i32(cu), past_lens=_i32(past),
        total_lens=_i32([p + n for p, n in zip(past, new)]), slots=_i32(slots if slots is not None else list(range(len(new)))),
        ws=Workspace(torch.device(DEV)))


def _part(family, spec, dtype, seed=0, scale=0.2, tweak=None):
    """A part with random tensors: (part, its tensors on the CPU by the names a model file gives them)."""
    from ziglm_b200 import kernels
    from ziglm_b200.parts import feed_forward_class, mixer_class
    cls = (mixer_class if family == "mixer" else feed_forward_class)(spec.kind)
    w = {}
    for i, (name, decl) in enumerate(cls.declare(spec).items()):
        w[name] = _r(*decl.shape, seed=seed + i, scale=scale, dtype=dtype) if decl.init == "normal" \
            else (torch.ones(decl.shape, dtype=dtype, device=DEV) + _r(*decl.shape, seed=seed + i, scale=0.3, dtype=dtype))
    if tweak is not None:
        tweak(w)
    part = cls(spec, dtype, torch.device(DEV))
    part.bind(w)
    kernels.require(part.kernel_libraries())
    def name(k):
        return k.replace(".weight", "").replace(".bias", ".b").replace("_norm", ".norm").replace("shared_gate", "shared.sg")

    return part, {name(k): v.cpu() for k, v in w.items()}


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("T,d", [(1, 72), (7, 61), (130, 256), (3, 4100)])
def test_the_norm_of_a_sum(dtype, T, d):
    from ziglm_b200 import kernels
    kernels.require(("elementwise",))
    x, branch = _r(T, d, seed=1), _r(T, d, seed=2, scale=3.0)
    w = (_r(d, seed=3) * 0.3 + 1.0).to(dtype)
    want = P.norm_plain(2.5 * x.cpu() + branch.cpu(), w.float().cpu(), 1e-5)
    rows = torch.empty(T, d, dtype=dtype, device=DEV)
    kernels.sum_norm(branch, w, 1e-5, 2.5, x, rows)
    torch.testing.assert_close(x.cpu(), want, atol=2e-6, rtol=2e-6)
    assert torch.equal(rows, x.to(dtype))                                                     # the rows are the stream, rounded once
    y = _r(T, d, seed=4)
    keep = y.clone()
    kernels.sum_norm(branch, w, 1e-5, 0.0, y)                                                  # alpha 0: the norm of the branch
    torch.testing.assert_close(y.cpu(), P.norm_plain(branch.cpu(), w.float().cpu(), 1e-5), atol=2e-6, rtol=2e-6)
    assert not torch.equal(y, keep)


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("H,G,D,V,rot", [(6, 2, 24, 40, 16), (4, 2, 64, 32, 32), (5, 1, 10, 10, 6), (2, 2, 128, 128, 128),
                                         (3, 1, 32, 16, 2), (1, 1, 4, 6, 4)])
def test_weighted_norm_of_every_head_before_the_rotation_and_the_cache_write(dtype, H, G, D, V, rot):
    """Two sequences (a prompt of 70 after 3 cached tokens, one decoded token at position 130) with shuffled pages; heads
    kept with zeros behind them; rows wider than the heads."""
    from ziglm_b200 import kernels
    from ziglm_b200.config.spec import PositionSpec
    from ziglm_b200.parts.rope import Rope
    kernels.require(("attention",))
    eps, page = 1e-5, 64
    hd = -(-max(D, V) // 8) * 8
    positions = list(range(3, 73)) + [130]
    seq = [0] * 70 + [1]
    T = len(positions)
    rope = Rope(PositionSpec(kind="rope", rotary_dim=rot, theta=100.0), dtype, torch.device(DEV))
    q, k, v = _r(T, H, D, seed=1, dtype=dtype), _r(T, G, D, seed=2, dtype=dtype), _r(T, G, V, seed=3, dtype=dtype)
    wq, wk = _r(D, seed=4).abs() + 0.5, _r(D, seed=5).abs() + 0.5
    rotd = {"dims": rot, "base": 100.0}
    qf = P.rotate_halves(P.rms_unit(q.float().cpu(), eps) * wq.cpu(), torch.tensor(positions), rotd)
    kf = P.rotate_halves(P.rms_unit(k.float().cpu(), eps) * wk.cpu(), torch.tensor(positions), rotd)
    rows = torch.zeros(T, (H + 2 * G) * hd + 24, dtype=dtype, device=DEV)
    rows[:, (H + 2 * G) * hd:] = 5.0
    view = rows[:, :(H + 2 * G) * hd].view(T, H + 2 * G, hd)
    view[:, :H, :D], view[:, H:H + G, :D], view[:, H + G:, :V] = q, k, v
    pad = lambda wt: torch.nn.functional.pad(wt, (0, hd - D)).contiguous()
    k_pages = torch.full((5, G, page, hd), 9.0, dtype=dtype, device=DEV)
    v_pages = torch.full((5, G, page, hd), 9.0, dtype=dtype, device=DEV)
    table = _i32([[4, 1, -1], [0, 3, 2]])
    kernels.rope_norm_store(rows, H, G, hd, rot, rope.inv_freq, 1.0, D, eps, _i32(positions), _i32(seq), table, k_pages,
                            v_pages, page, norm_first=True, q_weight=pad(wq), k_weight=pad(wk))
    tol = _tol(dtype, (3e-5, 3e-5), (2e-2, 2e-2))
    got = rows[:, :(H + 2 * G) * hd].float().cpu().view(T, H + 2 * G, hd)
    torch.testing.assert_close(got[:, :H, :D], qf, **tol)
    torch.testing.assert_close(got[:, H:H + G, :D], kf, **tol)
    torch.testing.assert_close(got[:, H + G:, :V], v.float().cpu(), atol=0, rtol=0)
    assert (got[:, :H + G, D:] == 0).all() and (rows[:, (H + 2 * G) * hd:] == 5.0).all()
    for t, (pos, b) in enumerate(zip(positions, seq)):
        pg = table[b, pos // page].item()
        assert torch.equal(k_pages[pg, :, pos % page], view[t, H:H + G])
        assert torch.equal(v_pages[pg, :, pos % page], view[t, H + G:])
    assert (k_pages == 9.0).sum().item() == (5 * page - T) * G * hd


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("H,G,hd,chunk,sink", [(6, 2, 40, 7, True), (4, 1, 64, 70, True), (3, 3, 24, None, True),
                                               (2, 2, 128, 130, False), (8, 2, 64, 1, True), (4, 2, 64, 64, False),
                                               (6, 3, 64, 100, True)])
def test_attention_within_chunks_with_one_more_one_in_the_denominator(dtype, H, G, hd, chunk, sink):
    """Prompts of two sequences, continued prompts and then a decoded token each, against the formula; then the decoded
    token of the long sequence once more with every page that lies wholly before its chunk poisoned."""
    from ziglm_b200 import kernels
    from ziglm_b200.parts.base import LayerIO
    kernels.require(("attention",) + kernels.fast_attention_libraries(dtype, hd, H, G, sinks=sink))
    lens, page, scale = [300, 70], 64, 0.3
    ks = [_r(L + 1, G, hd, seed=i, dtype=dtype) for i, L in enumerate(lens)]
    vs = [_r(L + 1, G, hd, seed=3 + i, dtype=dtype) for i, L in enumerate(lens)]
    qs = [_r(L + 1, H, hd, seed=7 + i, scale=0.6, dtype=dtype) for i, L in enumerate(lens)]
    sinks = torch.zeros(H, device=DEV) if sink else None
    k_pages = torch.zeros(9, G, page, hd, dtype=dtype, device=DEV)
    v_pages = torch.zeros(9, G, page, hd, dtype=dtype, device=DEV)
    table = _i32([[5, 2, 7, 0, 8], [1, 6, -1, -1, -1]])

    def plain(q, k, v):
        n = q.shape[0]
        q, k, v = q.float().cpu(), k.float().cpu(), v.float().cpu()
        seen = P.same_chunk(torch.arange(n), torch.arange(n), chunk)
        out = torch.zeros(n, H, hd)
        for h in range(H):
            g = h // (H // G)
            s = (q[:, h] @ k[:, g].t()) * scale
            out[:, h] = (P.softmax_one_more(s, seen) if sink else torch.softmax(s.masked_fill(~seen, float("-inf")), -1)) @ v[:, g]
        return out.reshape(n, H * hd)

    want = [plain(q, k, v) for q, k, v in zip(qs, ks, vs)]
    for b, (k, v) in enumerate(zip(ks, vs)):
        for pos in range(k.shape[0]):
            pg = table[b, pos // page].item()
            k_pages[pg, :, pos % page] = k[pos]
            v_pages[pg, :, pos % page] = v[pos]
    io = LayerIO(k_pages=k_pages, v_pages=v_pages, block_table=table, page_size=page)
    tol = _tol(dtype, (2e-5, 1e-4), (2e-2, 2e-2))
    for new, past in ((lens, [0, 0]), ([100, 30], [200, 40]), ([2, 2], [298, 68]), ([1, 1], lens)):
        q = torch.cat([x[p:p + n].reshape(n, H * hd) for x, p, n in zip(qs, past, new)]).contiguous()
        out = torch.empty(q.shape[0], H * hd, dtype=dtype, device=DEV)
        kernels.attention(_step(new, past), q, out, H, G, hd, scale, None, io, sinks=sinks, chunk=chunk)
        ref = torch.cat([w[p:p + n] for w, p, n in zip(want, past, new)])
        torch.testing.assert_close(out.float().cpu(), ref, **tol)
    if chunk is not None and chunk + 64 < 300:
        for i in range((300 - 300 % chunk) // page):
            k_pages[table[0, i].item()].fill_(1e4)
            v_pages[table[0, i].item()].fill_(1e4)
        q = qs[0][300:301].reshape(1, H * hd).contiguous()
        out = torch.empty(1, H * hd, dtype=dtype, device=DEV)
        kernels.attention(_step([1], [300]), q, out, H, G, hd, scale, None, io, sinks=sinks, chunk=chunk)
        torch.testing.assert_close(out.float().cpu(), want[0][300:301], **tol)
    q = qs[0][300:301].reshape(1, H * hd).contiguous()
    with pytest.raises(kernels.KernelError):
        kernels.attention(_step([1], [300]), q, torch.empty_like(q), H, G, hd, scale, 5, io, chunk=8)


def _retention_spec(H, D, V, decay, rot, width):
    from ziglm_b200.config.spec import MixerSpec, PositionSpec
    return MixerSpec(kind="decayed_linear_attention", width=width, n_heads=H, head_dim=D,
                     position=PositionSpec(kind="rope", rotary_dim=rot, theta=300.0),
                     options={"value_dim": V, "decay": tuple(decay), "activation": None, "norm": "head", "norm_eps": 1e-5,
                              "gate": "silu", "key_scale": D ** -0.5})


def _run_mixer(part, steps, hs, n_slots, state_shape):
    """The part over steps of several sequences: steps is a list of (new, past, slots); hs[b] the rows of sequence b.
    Returns each sequence's output rows."""
    from ziglm_b200.parts.base import LayerIO
    d = hs[0].shape[1]
    state = _r(n_slots, *state_shape, seed=77)                 # whatever the slots' last users left
    for new, past, slots in steps[:1]:
        for s in slots:
            state[s].zero_()
    got = [[] for _ in hs]
    for new, past, slots in steps:
        live = [b for b, n in enumerate(new) if n > 0]
        st = _step([new[b] for b in live], [past[b] for b in live], [slots[b] for b in live])
        h = torch.cat([hs[b][past[b]:past[b] + new[b]] for b in live]).contiguous()
        out = torch.full((h.shape[0], d), 3.0, device=DEV)
        part.forward(st, LayerIO(state=state), h, out, accumulate=False)
        at = 0
        for b in live:
            got[b].append(out[at:at + new[b]].cpu())
            at += new[b]
    return [torch.cat(g) for g in got], state


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("H,D,V,decay,rot", [(3, 12, 20, [0.5, 0.9, 1.0], 6), (2, 64, 32, [0.99, 0.999], 64),
                                             (1, 5, 3, [1.0], 2), (4, 32, 32, [0.9, 0.95, 0.97, 0.98], 16)])
def test_retention_over_steps_with_slots_used_again(dtype, H, D, V, decay, rot):
    """Three sequences in slots 3, 0, 2, one of them token by token, one with a portion of two tokens: rotated q and k
    by true positions, the factor on k, the state carried, every head normed by itself, the silu gate."""
    d = 48
    spec = _retention_spec(H, D, V, decay, rot, d)
    part, w = _part("mixer", spec, dtype, seed=5)
    lens = [50, 7, 33]
    hs = [_r(L, d, seed=10 + i, dtype=dtype) for i, L in enumerate(lens)]
    portions = [[20, 1, 29, 0, 0, 0, 0], [1] * 7, [2, 30, 1, 0, 0, 0, 0]]
    steps, past = [], [0, 0, 0]
    for i in range(7):
        new = [portions[b][i] for b in range(3)]
        steps.append((new, list(past), [3, 0, 2]))
        past = [p + n for p, n in zip(past, new)]
    got, state = _run_mixer(part, steps, hs, 4, (H, D, V))
    p = P.Plain(dtype)
    m = {"heads": H, "dim": D, "vdim": V, "decay": decay, "rot": {"dims": rot, "base": 300.0}}
    tol = _tol(dtype, (3e-5, 3e-4), (3e-2, 3e-2))
    for b in range(3):
        want = p.linear(P.retention(p, hs[b].float().cpu(), w, m, 1e-5, None, 0), w["o"])
        torch.testing.assert_close(got[b], want, **tol)
    assert torch.equal(state[1], _r(4, H, D, V, seed=77)[1])                 # a slot of no sequence is untouched


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("C,N,K,rank", [(52, 5, 3, 3), (192, 16, 4, 8), (24, 40, 1, 1), (33, 3, 5, 20), (64, 24, 4, 4),
                                        (40, 64, 2, 6)])
def test_selective_scan_over_steps_with_slots_used_again(dtype, C, N, K, rank):
    """The same three sequences through the scan: the convolution's kept inputs and S are carried over the steps; state
    counts the kernel is compiled for and others; decays from nearly none to strong."""
    from ziglm_b200.config.spec import MixerSpec
    d = 40
    spec = MixerSpec(kind="selective_scan", width=d, options={"channels": C, "states": N, "taps": K, "dt_rank": rank})

    def tweak(w):
        w["A_log"].copy_((w["A_log"].float() * 8.0 - 1.0).to(w["A_log"].dtype))
        w["dt.bias"].copy_((w["dt.bias"].float() * 5.0 - 1.0).to(w["dt.bias"].dtype))
        w["dt.weight"].copy_((w["dt.weight"].float() * 3.0).to(w["dt.weight"].dtype))
        w["D"].copy_((w["D"].float() * 4.0 + 0.5).to(w["D"].dtype))

    part, w = _part("mixer", spec, dtype, seed=9, tweak=tweak)
    lens = [50, 7, 33]
    hs = [_r(L, d, seed=20 + i, dtype=dtype) for i, L in enumerate(lens)]
    portions = [[20, 1, 29, 0, 0, 0, 0], [1] * 7, [2, 30, 1, 0, 0, 0, 0]]
    steps, past = [], [0, 0, 0]
    for i in range(7):
        new = [portions[b][i] for b in range(3)]
        steps.append((new, list(past), [3, 0, 2]))
        past = [p + n for p, n in zip(past, new)]
    got, state = _run_mixer(part, steps, hs, 4, (K - 1 + N, C))
    p = P.Plain(dtype)
    m = {"inner": C, "state": N, "dt_rank": rank}
    tol = _tol(dtype, (3e-5, 3e-4), (4e-2, 4e-2))
    for b in range(3):
        want = p.linear(P.selective_scan(p, hs[b].float().cpu(), w, m, None), w["o"])
        torch.testing.assert_close(got[b], want, **tol)
    assert torch.equal(state[1], _r(4, K - 1 + N, C, seed=77)[1])


def test_a_long_scan_in_chunks_equals_token_by_token():
    """1,000 tokens at once (eight chunks whose maps are composed) against the same tokens one by one, in float32."""
    from ziglm_b200.config.spec import MixerSpec
    d, C, N, K = 32, 96, 16, 4
    spec = MixerSpec(kind="selective_scan", width=d, options={"channels": C, "states": N, "taps": K, "dt_rank": 4})
    part, w = _part("mixer", spec, torch.float32, seed=2)
    h = _r(1000, d, seed=1)
    (whole,), s1 = _run_mixer(part, [([1000], [0], [1])], [h], 2, (K - 1 + N, C))
    (single,), s2 = _run_mixer(part, [([1], [t], [1]) for t in range(1000)], [h], 2, (K - 1 + N, C))
    torch.testing.assert_close(whole, single, atol=2e-5, rtol=2e-4)
    torch.testing.assert_close(s1[1], s2[1], atol=2e-5, rtol=2e-4)


@pytest.mark.parametrize("E,identity,top,groups,keep", [(5, 3, 2, 4, 2), (7, 0, 3, 1, 1), (4, 2, 1, 3, 1), (8, 4, 3, 4, 3),
                                                        (1, 0, 1, 1, 1), (9, 0, 4, 3, 2)])
def test_router_over_experts_and_identity_experts(E, identity, top, groups, keep):
    """Softmax scores over all outputs, every choice score negative, groups scored by their largest choice score, the
    weights without the offset and times a factor; the logits in columns of a wider matrix."""
    from ziglm_b200 import kernels
    kernels.require(("moe",))
    T, n = 50, E + identity
    z = _r(T, n + 1, seed=E, scale=2.0)
    corr = _r(n, seed=1, scale=0.3) - 2.0
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    kernels.moe_route(z, corr, top, groups, keep, 1, ids, wts, softmax_scores=1, weight_scale=1.75, n_extra=1)
    want = P.route(z[:, :n].cpu(), corr.cpu(), {"top": top, "scale": 1.75, "groups": {"count": groups, "keep": keep}})
    assert torch.equal(ids.cpu().long(), want["ids"])
    torch.testing.assert_close(wts.cpu(), want["weights"], atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("T", [1, 5, 70, 200])
@pytest.mark.parametrize("E,identity,top,groups,keep,shared", [(5, 3, 2, 4, 2, 20), (6, 0, 2, 2, 1, None), (3, 3, 2, 3, 2, 12)])
def test_mixture_of_experts_with_identity_experts_and_a_gated_shared_expert(dtype, T, E, identity, top, groups, keep, shared):
    """The part as the block calls it: T = 1, 5 stream the experts (the router's product inside the routing kernel),
    70 and 200 run tiles (float32) or the tensor cores (bfloat16).  Identity experts are often chosen."""
    from ziglm_b200.config.spec import FeedForwardSpec
    d, ff = 72, 40
    opts = {"experts": E, "identity": identity, "top": top, "groups": groups, "keep_groups": keep, "group_best": 1,
            "score": "softmax", "correction": True, "weight_scale": 1.5}
    if shared is not None:
        opts["shared"] = FeedForwardSpec("gated_mlp", d, shared, "silu")
        opts["shared_gate"] = True
    spec = FeedForwardSpec("moe", d, ff, "silu", options=opts)

    def tweak(w):
        w["router.weight"].copy_((w["router.weight"].float() * 6.0).to(w["router.weight"].dtype))
        if shared is not None:
            w["shared_gate.weight"].copy_((w["shared_gate.weight"].float() * 8.0).to(dtype))

    part, w = _part("ff", spec, dtype, seed=3, tweak=tweak)
    h = _r(T, d, seed=99, dtype=dtype)
    mlp = {"router": {"experts": E, "identity": identity, "top": top, "scale": 1.5, "groups": {"count": groups, "keep": keep}},
           "shared": None if shared is None else {"ff": shared}}
    p = P.Plain(dtype)
    want = P.mixture(p, h.float().cpu(), w, mlp)
    if identity:
        z = p.linear_wide(h.float().cpu(), w["router"])
        assert (P.route(z, w["correction"].float(), mlp["router"])["ids"] >= E).any() or T == 1
    step = _step([T], [0])
    out = torch.full((T, d), 7.0, device=DEV)
    part.forward(step, h, out, accumulate=False)

    def close(got, ref):
        if dtype == torch.float32:
            torch.testing.assert_close(got, ref, atol=2e-5, rtol=1e-4)
            return
        # bfloat16: a router's close call may send a token to another expert than the plain implementation's sums do
        bad = ((got - ref).abs() > 8e-2 + 5e-2 * ref.abs()).any(dim=1)
        assert int(bad.sum()) <= T // 50, f"{int(bad.sum())} of {T} rows differ"

    close(out.cpu(), want)
    part.forward(step, h, out, accumulate=True)
    close(out.cpu(), 2 * want)

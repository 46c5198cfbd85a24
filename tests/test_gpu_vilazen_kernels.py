"""Each mechanism of the Vilazen design alone: the kernel against the plain function that states its formula
(tests/plain_vilazen.py), at sizes that are no multiple of a tile, with strided rows, several sequences in a step,
shuffled pages, prompts and decoded tokens, slots used again, and inputs made so that a fault shows."""
from types import SimpleNamespace

import pytest
import torch

import plain_vilazen as P

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


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("H,G,D,V,rot,whole,mix", [(6, 2, 24, 40, 16, True, 2), (4, 4, 64, 64, 64, True, 1),
                                                    (5, 1, 16, 8, 2, False, 2), (2, 1, 128, 128, 64, True, 0),
                                                    (3, 1, 32, 16, 16, False, 1), (8, 2, 64, 64, 32, False, 2)])
def test_norm_of_whole_q_and_k_rotation_of_adjacent_pairs_mixed_values_and_cache_write(dtype, H, G, D, V, rot, whole, mix):
    """Two sequences (a prompt of 70 after 3 cached tokens, one decoded token at position 130) with shuffled pages; heads
    kept with zeros behind them; rows wider than the heads.  The plain side turns adjacent pairs of the heads as the
    model lays them out; the kernel's side gets the heads in the order ``Rope.head_order`` gives."""
    from ziglm_b200 import kernels
    from ziglm_b200.config.spec import PositionSpec
    from ziglm_b200.parts.rope import Rope
    kernels.require(("attention",))
    eps, page, lam = 1e-5, 64, 0.375
    hd = -(-max(D, V) // 8) * 8
    positions = list(range(3, 73)) + [130]
    seq = [0] * 70 + [1]
    T = len(positions)
    rope = Rope(PositionSpec(kind="rope", rotary_dim=rot, theta=100.0, options={"pairs": "adjacent"}), dtype, torch.device(DEV))
    order = torch.tensor(rope.head_order(D))
    q, k, v = _r(T, H, D, seed=1, dtype=dtype), _r(T, G, D, seed=2, dtype=dtype), _r(T, G, V, seed=3, dtype=dtype)
    wq, wk = _r(H * D, seed=4).abs() + 0.5, _r(G * D, seed=5).abs() + 0.5
    first = _r(T, G * V, seed=6, dtype=dtype)
    # the plain side
    qf, kf, vf = q.float().cpu(), k.float().cpu(), v.float().cpu()
    if whole:
        qf = P.norm_plain(qf.reshape(T, -1), wq.cpu(), eps).view(T, H, D)
        kf = P.norm_plain(kf.reshape(T, -1), wk.cpu(), eps).view(T, G, D)
    rotd = {"dims": rot, "base": 100.0}
    qf, kf = P.rotate_pairs(qf, torch.tensor(positions), rotd), P.rotate_pairs(kf, torch.tensor(positions), rotd)
    if mix == 2:
        vf = ((1.0 - lam) * vf.reshape(T, -1) + lam * first.float().cpu()).view(T, G, V)
    # the kernel's side: heads in the kernel's order, kept with zeros behind them
    rows = torch.zeros(T, (H + 2 * G) * hd + 24, dtype=dtype, device=DEV)
    rows[:, (H + 2 * G) * hd:] = 5.0
    view = rows[:, :(H + 2 * G) * hd].view(T, H + 2 * G, hd)
    view[:, :H, :D] = q[:, :, order]
    view[:, H:H + G, :D] = k[:, :, order]
    view[:, H + G:, :V] = v
    pad = lambda wt, n: torch.nn.functional.pad(wt.view(n, D)[:, order], (0, hd - D)).reshape(-1).contiguous()
    buf = first.clone() if mix == 2 else torch.zeros(T, G * V, dtype=dtype, device=DEV)
    k_pages = torch.full((5, G, page, hd), 9.0, dtype=dtype, device=DEV)
    v_pages = torch.full((5, G, page, hd), 9.0, dtype=dtype, device=DEV)
    table = _i32([[4, 1, -1], [0, 3, 2]])
    kernels.qk_prep(rows, H, G, hd, rot, rope.inv_freq, pad(wq, H) if whole else None, pad(wk, G) if whole else None,
                    H * D, G * D, eps, mix, lam, buf if mix else None, V, _i32(positions), _i32(seq), table, k_pages,
                    v_pages, page)
    tol = _tol(dtype, (3e-5, 3e-5), (2e-2, 2e-2))
    got = rows[:, :(H + 2 * G) * hd].float().cpu().view(T, H + 2 * G, hd)
    torch.testing.assert_close(got[:, :H, :D], qf[:, :, order], **tol)
    torch.testing.assert_close(got[:, H:H + G, :D], kf[:, :, order], **tol)
    torch.testing.assert_close(got[:, H + G:, :V], vf, **tol)
    assert (got[:, :, max(D, V):] == 0).all() and (rows[:, (H + 2 * G) * hd:] == 5.0).all()
    if mix == 1:
        assert torch.equal(buf.view(T, G, V), v)
    tb = table.cpu()
    for t, (pos, b) in enumerate(zip(positions, seq)):
        pg = tb[b, pos // page].item()
        assert torch.equal(k_pages[pg, :, pos % page], view[t, H:H + G])
        assert torch.equal(v_pages[pg, :, pos % page], view[t, H + G:])
    assert (k_pages == 9.0).sum().item() == (5 * page - T) * G * hd               # nothing else was written


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("H,G,hd,window,keep,sink", [(6, 2, 40, 9, 3, False), (4, 1, 64, 70, 5, True), (3, 3, 24, None, 0, True),
                                                      (2, 2, 128, 130, 64, False), (8, 2, 64, 1, 1, True), (4, 2, 64, 64, 70, False)])
def test_attention_with_a_window_kept_first_tokens_and_sinks(dtype, H, G, hd, window, keep, sink):
    """Prompts of two sequences, continued prompts and then a decoded token each, against the formula.  The pages behind
    the window (but for those of the kept tokens) hold a huge number: a key read from there shows."""
    from ziglm_b200 import kernels
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts.base import LayerIO
    kernels.require(("attention",) + kernels.fast_attention_libraries(dtype, hd, H, G, keep_first=keep if window else 0, sinks=sink))
    lens, page, scale = [300, 70], 64, 0.3
    ks = [_r(L + 1, G, hd, seed=i, dtype=dtype) for i, L in enumerate(lens)]
    vs = [_r(L + 1, G, hd, seed=3 + i, dtype=dtype) for i, L in enumerate(lens)]
    qs = [_r(L + 1, H, hd, seed=7 + i, scale=0.6, dtype=dtype) for i, L in enumerate(lens)]
    sinks = (_r(H, seed=5) * 2.0 + 1.0) if sink else None
    k_pages = torch.zeros(9, G, page, hd, dtype=dtype, device=DEV)
    v_pages = torch.zeros(9, G, page, hd, dtype=dtype, device=DEV)
    table = _i32([[5, 2, 7, 0, 8], [1, 6, -1, -1, -1]])

    def plain(q, k, v):
        n = q.shape[0]
        q, k, v = q.float().cpu(), k.float().cpu(), v.float().cpu()
        seen = P.visible(torch.arange(n), torch.arange(n), window, keep)
        out = torch.zeros(n, H, hd)
        for h in range(H):
            g = h // (H // G)
            s = (q[:, h] @ k[:, g].t()) * scale
            out[:, h] = P.softmax_rows(s, seen, sinks[h].cpu() if sink else None) @ v[:, g]
        return out.reshape(n, H * hd)

    want = [plain(q, k, v) for q, k, v in zip(qs, ks, vs)]
    for b, (k, v) in enumerate(zip(ks, vs)):
        for pos in range(k.shape[0]):
            pg = table[b, pos // page].item()
            k_pages[pg, :, pos % page] = k[pos]
            v_pages[pg, :, pos % page] = v[pos]
    for new, past in ((lens, [0, 0]), ([100, 30], [200, 40]), ([2, 2], [298, 68]), ([1, 1], lens)):
        q = torch.cat([x[p:p + n].reshape(n, H * hd) for x, p, n in zip(qs, past, new)]).contiguous()
        T = q.shape[0]
        step = SimpleNamespace(
            n_tokens=T, n_seqs=2, single_token=new == [1, 1], max_new=max(new), max_total=max(p + n for p, n in zip(past, new)),
            positions=_i32([p + i for p, n in zip(past, new) for i in range(n)]),
            seq_of_token=_i32([b for b, n in enumerate(new) for _ in range(n)]), cu_seqlens=_i32([0, new[0], new[0] + new[1]]),
            past_lens=_i32(past), total_lens=_i32([p + n for p, n in zip(past, new)]), ws=Workspace(torch.device(DEV)))
        io = LayerIO(k_pages=k_pages, v_pages=v_pages, block_table=table, page_size=page)
        out = torch.empty(T, H * hd, dtype=dtype, device=DEV)
        kernels.attention(step, q, out, H, G, hd, scale, window, io, keep_first=keep, sinks=sinks)
        ref = torch.cat([w[p:p + n] for w, p, n in zip(want, past, new)])
        torch.testing.assert_close(out.float().cpu(), ref, **_tol(dtype, (2e-5, 1e-4), (2e-2, 2e-2)))
        # a gate a head, in columns of wider rows: the kernel that says it applied it did, the others left it alone
        gates = _r(T, H + 11, seed=31, scale=2.0, dtype=dtype)[:, 3:3 + H]
        gated = kernels.attention(step, q, out, H, G, hd, scale, window, io, keep_first=keep, sinks=sinks, head_gate=gates,
                                  head_gate_mult=1.3)
        if gated:
            factor = (torch.sigmoid(gates.float().cpu()) * 1.3).repeat_interleave(hd, dim=1)
            torch.testing.assert_close(out.float().cpu(), ref * factor, **_tol(dtype, (2e-5, 1e-4), (2e-2, 2e-2)))
        else:
            torch.testing.assert_close(out.float().cpu(), ref, **_tol(dtype, (2e-5, 1e-4), (2e-2, 2e-2)))
        assert gated == (dtype == torch.bfloat16 and new == [1, 1] and hd in (64, 128) and (keep > 0 and window is not None or sink))
    if window is not None and window + 64 < 300:
        # the decoded token of the long sequence once more, with every page that lies wholly behind its window and
        # holds no kept token poisoned
        first_seen = 300 - window + 1
        for i in range(-(-keep // page), first_seen // page):
            k_pages[table[0, i].item()].fill_(1e4)
            v_pages[table[0, i].item()].fill_(1e4)
        q = qs[0][300:301].reshape(1, H * hd).contiguous()
        step = SimpleNamespace(n_tokens=1, n_seqs=1, single_token=True, max_new=1, max_total=301, positions=_i32([300]),
                               seq_of_token=_i32([0]), cu_seqlens=_i32([0, 1]), past_lens=_i32([300]), total_lens=_i32([301]),
                               ws=Workspace(torch.device(DEV)))
        out = torch.empty(1, H * hd, dtype=dtype, device=DEV)
        kernels.attention(step, q, out, H, G, hd, scale, window, LayerIO(k_pages=k_pages, v_pages=v_pages, block_table=table,
                                                                         page_size=page), keep_first=keep, sinks=sinks)
        torch.testing.assert_close(out.float().cpu(), want[0][300:301], **_tol(dtype, (2e-5, 1e-4), (2e-2, 2e-2)))


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("hd,window,keep,sink", [(64, 100, 130, True), (128, 200, 64, False), (64, 65, 1, False),
                                                 (64, 300, 129, True)])
def test_a_late_portion_of_a_prompt_reads_the_kept_pages_and_its_window_only(dtype, hd, window, keep, sink):
    """The last 100 tokens of a prompt of 700 as a step of their own: the pages between the kept first tokens and the
    step's first window hold a huge number, which a key read from there would show; the kept pages are one, two and
    three (a last step of one page) and the window's first page lies right behind them or far away."""
    from ziglm_b200 import kernels
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts.base import LayerIO
    H, G, page, scale, L, new = 4, 2, 64, 0.25, 700, 100
    kernels.require(("attention",) + kernels.fast_attention_libraries(dtype, hd, H, G, keep_first=keep, sinks=sink))
    k, v = _r(L, G, hd, seed=1, dtype=dtype), _r(L, G, hd, seed=2, dtype=dtype)
    q = _r(L, H, hd, seed=3, scale=0.6, dtype=dtype)
    sinks = (_r(H, seed=5) * 2.0 + 1.0) if sink else None
    n_pages = -(-L // page)
    order = [(7 * i + 3) % n_pages for i in range(n_pages)]
    table = _i32([order])
    k_pages = torch.zeros(n_pages, G, page, hd, dtype=dtype, device=DEV)
    v_pages = torch.zeros(n_pages, G, page, hd, dtype=dtype, device=DEV)
    for pos in range(L):
        k_pages[order[pos // page], :, pos % page] = k[pos]
        v_pages[order[pos // page], :, pos % page] = v[pos]
    past = L - new
    for i in range(-(-keep // page), (past - window + 1) // page):
        k_pages[order[i]].fill_(1e4)
        v_pages[order[i]].fill_(1e4)
    qf, kf, vf = q.float().cpu(), k.float().cpu(), v.float().cpu()
    seen = P.visible(torch.arange(past, L), torch.arange(L), window, keep)
    want = torch.zeros(new, H, hd)
    for h in range(H):
        s_ = (qf[past:, h] @ kf[:, h // (H // G)].t()) * scale
        want[:, h] = P.softmax_rows(s_, seen, sinks[h].cpu() if sink else None) @ vf[:, h // (H // G)]
    step = SimpleNamespace(n_tokens=new, n_seqs=1, single_token=False, max_new=new, max_total=L,
                           positions=_i32(list(range(past, L))), seq_of_token=_i32([0] * new), cu_seqlens=_i32([0, new]),
                           past_lens=_i32([past]), total_lens=_i32([L]), ws=Workspace(torch.device(DEV)))
    out = torch.empty(new, H * hd, dtype=dtype, device=DEV)
    kernels.attention(step, q[past:].reshape(new, H * hd).contiguous(), out, H, G, hd, scale, window,
                      LayerIO(k_pages=k_pages, v_pages=v_pages, block_table=table, page_size=page), keep_first=keep, sinks=sinks)
    torch.testing.assert_close(out.float().cpu(), want.reshape(new, H * hd), **_tol(dtype, (2e-5, 1e-4), (2e-2, 2e-2)))


def _lin_step(slots, new):
    """What the linear attention reads of a step: its sequences' slots and token counts, and scratch."""
    from ziglm_b200.engine.workspace import Workspace
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    return SimpleNamespace(n_seqs=len(new), slots=_i32(slots), cu_seqlens=_i32(cu), single_token=all(n == 1 for n in new),
                           max_new=max(new), ws=Workspace(torch.device(DEV)))


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("H,D,V,decay", [(3, 12, 20, [0.5, 0.9, 1.0]), (2, 64, 64, [0.999, 0.97]), (1, 5, 3, [1.0]),
                                          (2, 33, 35, [0.3, 0.95]), (4, 128, 32, [0.55, 0.8, 0.93, 0.9995]),
                                          (1, 160, 40, [0.9])])
def test_decayed_linear_attention_over_steps_with_slots_used_again(dtype, H, D, V, decay):
    """Three sequences in slots 2, 0, 3 of a state that holds garbage elsewhere: a prompt each (1, 70 and 131 tokens),
    a step of 2, 33 and 1 tokens, then single tokens; against the recurrence token by token.  The rows are wider than
    q, k, v (a gate behind them), and silu is applied as the rows are read."""
    from ziglm_b200 import kernels
    kernels.require(("linear_attention",))
    silu = torch.nn.functional.silu
    lens = [1 + 2 + 4, 70 + 33 + 4, 131 + 1 + 4]
    width = 2 * H * D + H * V + 8
    full = [_r(L, width, seed=10 + i, dtype=dtype) for i, L in enumerate(lens)]
    chunk = kernels.linear_attention_chunk()
    pows = torch.tensor([[a ** n for n in range(chunk + 1)] for a in decay], dtype=torch.float64).float().to(DEV)
    state = torch.full((5, H, D, V), 7.0, device=DEV)
    slots = [2, 0, 3]
    for s in slots:
        state[s].zero_()
    want = []
    for rows in full:
        x = silu(rows.float().cpu())
        q, k, v = x[:, :H * D].view(-1, H, D), x[:, H * D:2 * H * D].view(-1, H, D), x[:, 2 * H * D:2 * H * D + H * V].view(-1, H, V)
        S = torch.zeros(H, D, V, dtype=torch.float64)
        out = []
        for t in range(rows.shape[0]):
            S = torch.tensor(decay, dtype=torch.float64)[:, None, None] * S + k[t, :, :, None].double() * v[t, :, None, :].double()
            out.append(torch.einsum("hdv,hd->hv", S, q[t].double()).reshape(-1))
        want.append(torch.stack(out).float())
    at = [0, 0, 0]
    for new in ([1, 70, 131], [2, 33, 1], [1, 1, 1], [1, 1, 1], [1, 1, 1], [1, 1, 1]):
        proj = torch.cat([f[a:a + n] for f, a, n in zip(full, at, new)]).contiguous()
        T = proj.shape[0]
        step = _lin_step(slots, new)
        out = torch.full((T, H * V), 3.0, device=DEV)
        kernels.decayed_linear_attention(proj, 0, H * D, 2 * H * D, H, D, V, "silu", pows, state, step, out)
        ref = torch.cat([w[a:a + n] for w, a, n in zip(want, at, new)])
        torch.testing.assert_close(out.cpu(), ref, atol=2e-4, rtol=2e-4)
        at = [a + n for a, n in zip(at, new)]
    assert (state[1] == 7.0).all() and (state[4] == 7.0).all()                   # other slots are left alone


@pytest.mark.parametrize("dtype", TYPES)
def test_segments_of_long_prompts_side_by_side(dtype):
    """Five prompts of 1, 128, 129, 600 and 256 tokens in one step (one, one, two, five and two segments), each on top
    of a state that is not zero, against the same prompts one after the other in steps of at most a segment."""
    from ziglm_b200 import kernels
    kernels.require(("linear_attention",))
    H, D, V, decay = 3, 20, 40, [0.99, 0.7, 1.0]
    lens = [1, 128, 129, 600, 256]
    rows = [_r(L, 2 * H * D + H * V, seed=20 + i, scale=0.5, dtype=dtype) for i, L in enumerate(lens)]
    chunk = kernels.linear_attention_chunk()
    pows = torch.tensor([[a ** n for n in range(chunk + 1)] for a in decay], dtype=torch.float64).float().to(DEV)
    start = _r(len(lens), H, D, V, seed=9)
    state = torch.cat([start, start]).contiguous()
    together = torch.empty(sum(lens), H * V, device=DEV)
    kernels.decayed_linear_attention(torch.cat(rows).contiguous(), 0, H * D, 2 * H * D, H, D, V, "silu", pows, state,
                                     _lin_step(list(range(len(lens))), lens), together)
    alone = []
    for i, r in enumerate(rows):
        out = torch.empty(r.shape[0], H * V, device=DEV)
        for t0 in range(0, r.shape[0], 100):
            part = r[t0:t0 + 100].contiguous()
            kernels.decayed_linear_attention(part, 0, H * D, 2 * H * D, H, D, V, "silu", pows, state,
                                             _lin_step([len(lens) + i], [part.shape[0]]), out[t0:t0 + 100])
        alone.append(out)
    torch.testing.assert_close(together, torch.cat(alone), atol=1e-3, rtol=2e-4)
    torch.testing.assert_close(state[:len(lens)], state[len(lens):], atol=1e-3, rtol=2e-4)


@pytest.mark.parametrize("dtype", TYPES)
def test_a_long_prompt_of_linear_attention_against_token_by_token(dtype):
    """1,000 tokens in one step and the same tokens one by one through the same kernel: chunks and single steps agree."""
    from ziglm_b200 import kernels
    kernels.require(("linear_attention",))
    H, D, V, decay = 2, 16, 24, [0.999, 0.9]
    rows = _r(1000, 2 * H * D + H * V, seed=4, scale=0.5, dtype=dtype)
    chunk = kernels.linear_attention_chunk()
    pows = torch.tensor([[a ** n for n in range(chunk + 1)] for a in decay], dtype=torch.float64).float().to(DEV)
    state = torch.zeros(2, H, D, V, device=DEV)
    whole = torch.empty(1000, H * V, device=DEV)
    kernels.decayed_linear_attention(rows, 0, H * D, 2 * H * D, H, D, V, None, pows, state,
                                     _lin_step([0], [1000]), whole)
    single = torch.empty(1000, H * V, device=DEV)
    one = _lin_step([1], [1])
    for t in range(1000):
        kernels.decayed_linear_attention(rows[t:t + 1], 0, H * D, 2 * H * D, H, D, V, None, pows, state,
                                         one, single[t:t + 1])
    torch.testing.assert_close(whole, single, atol=1e-3, rtol=2e-4)
    torch.testing.assert_close(state[0], state[1], atol=1e-3, rtol=2e-4)


@pytest.mark.parametrize("dtype", TYPES)
def test_gates_norm_with_a_gate_exact_gelu_and_the_norm_of_the_embedding(dtype):
    from ziglm_b200 import kernels
    kernels.require(("elementwise",))
    T, H, n = 37, 5, 24
    a = _r(T, H * n + 8, seed=1, dtype=dtype)[:, 8:]
    g = _r(T, H + 3, seed=2, scale=2.0, dtype=dtype)[:, :H]
    out = torch.empty(T, H * n, dtype=dtype, device=DEV)
    kernels.gate_heads(a, g, out, H, 1.3)
    want = (a.float().view(T, H, n) * torch.sigmoid(g.float())[:, :, None] * 1.3).reshape(T, H * n)
    torch.testing.assert_close(out.float(), want, **_tol(dtype))
    x = _r(T, 70, seed=3, scale=3.0)
    w = _r(70, seed=4).abs() + 0.2
    gate = _r(T, 70 + 2, seed=5, dtype=dtype)[:, 2:]
    out = torch.empty(T, 70, dtype=dtype, device=DEV)
    kernels.norm_gate(x, w, gate, out, 1e-5, 0.7)
    want = P.norm_plain(x.cpu(), w.cpu(), 1e-5) * torch.sigmoid(gate.float().cpu()) * 0.7
    torch.testing.assert_close(out.float().cpu(), want, **_tol(dtype))
    kernels.norm_gate(x, w, None, out, 1e-5)
    torch.testing.assert_close(out.float().cpu(), P.norm_plain(x.cpu(), w.cpu(), 1e-5), **_tol(dtype))
    z = _r(T, 96, seed=6, scale=2.0, dtype=dtype)
    act = torch.empty_like(z)
    kernels.unary_act(z, act, "gelu")
    torch.testing.assert_close(act.float().cpu(), P.gelu_erf(z.float().cpu()), **_tol(dtype))
    # the norm of the embedded tokens: float32 rows in place, the weight kept minus one
    rows = _r(T, 72, seed=7, scale=4.0)
    before = rows.cpu().clone()
    wz = _r(72, seed=8, scale=0.3, dtype=dtype)
    kernels.rmsnorm_rows(rows, wz, rows, 1e-5, weight_offset=1.0)
    torch.testing.assert_close(rows.cpu(), P.norm_around_zero(before, wz.float().cpu(), 1e-5), atol=1e-5, rtol=1e-5)
    src = _r(T, 40, seed=9)[:, 3:19]
    dst = torch.zeros(T, 30, dtype=dtype, device=DEV)
    kernels.convert_rows(src, dst[:, 5:21])
    assert torch.equal(dst[:, 5:21], src.to(dtype)) and (dst[:, :5] == 0).all() and (dst[:, 21:] == 0).all()


def test_exact_gelu_in_the_epilogue_of_the_tensor_core_product():
    from ziglm_b200 import kernels
    kernels.require(("gemm_tc", "elementwise"))
    for T in (8, 300):
        x, w = _r(T, 256, seed=1, dtype=torch.bfloat16), _r(384, 256, seed=2, scale=0.1, dtype=torch.bfloat16)
        out = torch.empty(T, 384, dtype=torch.bfloat16, device=DEV)
        assert kernels.gemm_tc_unary(x, w, out, "gelu")
        want = P.gelu_erf(x.float().cpu() @ w.float().cpu().t())
        torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=2e-2)

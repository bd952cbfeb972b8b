"""Each mechanism of the Botuvik decoder alone, its kernels against the plain implementation's function:
the norm behind a sublayer with the residual sum (and the next norm), additions between runs, squared ReLU,
queries / keys / values of the general attention path (biases, neighbour-pair rotation, unit norm, padded heads),
attention with a score cap and a sink (prompts, decoding over several shares, a far key that stands out, keys at
page borders, a sink that takes most of the weight), the matrix memory (gates with a running maximum, state over
steps and slots, chunks side by side), and the routing of experts."""
import math

import pytest
import torch

import plain_botuvik as P
from helpers import check_error

pytestmark = pytest.mark.gpu
PAGE = 64


def rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    return float((got - ref).abs().max() / ref.abs().max())


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# --------------------------------------------------------------------------- small kernels
@pytest.mark.parametrize("rows,d", [(1, 8), (5, 72), (3, 1000), (2, 4100)])
def test_post_norm_add_and_next_norm(rows, d):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(d)
    y, x = (torch.randn(rows, d) * 3).cuda(), torch.randn(rows, d).cuda()
    w, w2 = (1 + 0.3 * torch.randn(d)).cuda(), (1 + 0.3 * torch.randn(d)).cuda()
    ref_x = x.double().cpu() + P.rms_norm(y.double().cpu(), w.double().cpu(), 1e-5)
    ref_h = P.rms_norm(ref_x, w2.double().cpu(), 2e-6)
    alone = x.clone()
    ops.post_norm_add(y, w, 1e-5, alone)
    check_error("post norm + add, float32", f"{rows}x{d}", rel(alone, ref_x), 2e-6)
    for dtype, lim in ((torch.float32, 3e-6), (torch.bfloat16, 5e-3)):
        both, h = x.clone(), torch.empty(rows, d, device="cuda", dtype=dtype)
        ops.post_norm_add(y, w, 1e-5, both, next_weight=w2, next_eps=2e-6, next_out=h)
        assert torch.equal(both, alone)
        check_error(f"post norm + add + next norm, {dtype}", f"{rows}x{d}", rel(h, ref_h), lim)


def test_stream_add_and_squared_relu():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(3)
    x, e, v = torch.randn(5, 24).cuda(), torch.randn(5, 24).cuda(), torch.randn(24).cuda()
    for other, vec in ((e, v), (None, v), (e, None)):
        got = ops.stream_add(x.clone(), other, vec)
        ref = x.double().cpu() + (other.double().cpu() if other is not None else 0) + (vec.double().cpu() if vec is not None else 0)
        assert rel(got, ref) < 1e-6
    wide = (torch.randn(7, 50) * 2).cuda()
    out = torch.empty(7, 33, device="cuda")
    ops.relu2(wide[:, 10:43], out)
    assert rel(out, torch.relu(wide[:, 10:43].double().cpu()) ** 2) < 1e-6


# --------------------------------------------------------------------------- queries, keys, values
@pytest.mark.parametrize("H,G,dk,dv,rd,interleaved", [(4, 2, 24, 40, 16, True), (3, 3, 16, 16, 16, True), (5, 1, 10, 12, 0, True),
                                                      (2, 1, 64, 32, 64, False)])
def test_qkv_prepare(H, G, dk, dv, rd, interleaved):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(H * dk)
    hdp = -(-max(dk, dv) // 16) * 16
    positions = [0, 1, 63, 64, 65, 130, 1000]
    T = len(positions)
    F = (H + G) * dk + G * dv
    qkv, bias = torch.randn(T, F).cuda(), (0.5 * torch.randn(F)).cuda()
    base = 10000.0
    freq = torch.tensor([base ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float64).float().cuda() if rd else None
    rotation = ops.Rotation(freq, rd, interleaved) if rd else ops.NO_ROTATION
    pages = torch.full((20, 2, G, PAGE, hdp), 7.0, device="cuda")
    table = i32([[3, 9, 1] + [0] * 13])                   # positions 0..191 in pages 3, 9, 1; position 1000 in page 0
    q_out = torch.full((T, H * hdp), 7.0, device="cuda")
    ops.qkv_prepare(qkv, bias, rotation, i32(positions), i32([0] * T), table, q_out, pages, num_heads=H, num_kv_heads=G,
                    key_dim=dk, value_dim=dv, unit_norm_eps=1e-5)
    full = qkv.double().cpu() + bias.double().cpu()
    q = full[:, :H * dk].view(T, H, dk)
    k = full[:, H * dk:(H + G) * dk].view(T, G, dk)
    v = full[:, (H + G) * dk:].view(T, G, dv)
    pos = torch.tensor(positions)
    if interleaved:
        q, k = P.rotate_neighbour_pairs(q, pos, base, rd), P.rotate_neighbour_pairs(k, pos, base, rd)
    else:
        import plain_ramupel
        q, k = plain_ramupel.rotate_half_pairs(q, pos, base, rd), plain_ramupel.rotate_half_pairs(k, pos, base, rd)
    q, k = P.unit_rms(q, 1e-5), P.unit_rms(k, 1e-5)
    got_q = q_out.view(T, H, hdp)
    # the angle position * frequency is a float32 product: at position 1000 its rounding alone is worth 1e-5
    check_error("general attention: queries", f"{H}x{dk}", rel(got_q[:, :, :dk], q), 3e-5)
    assert float(got_q[:, :, dk:].abs().max()) == 0.0 if hdp > dk else True
    for t, p in enumerate(positions):
        page = [3, 9, 1][p // PAGE] if p < 192 else 0
        got_k, got_v = pages[page, 0, :, p % PAGE], pages[page, 1, :, p % PAGE]
        assert rel(got_k[:, :dk], k[t]) < 3e-5 and rel(got_v[:, :dv], v[t]) < 1e-6
        assert float(got_k[:, dk:].abs().sum()) == 0.0 and float(got_v[:, dv:].abs().sum()) == 0.0
    assert float((pages[2] - 7.0).abs().max()) == 0.0     # a page of nobody's stays untouched


# --------------------------------------------------------------------------- attention with a cap and a sink
def fill_pages(k, v, table_rows, num_pages, dtype):
    """k, v: [T, G, hd] of ONE sequence -> pages [num_pages, 2, G, 64, hd] laid out through ``table_rows``."""
    T, G, hd = k.shape
    pages = torch.zeros(num_pages, 2, G, PAGE, hd, dtype=dtype, device="cuda")
    for t in range(T):
        page = table_rows[t // PAGE]
        pages[page, 0, :, t % PAGE] = k[t].to(dtype)
        pages[page, 1, :, t % PAGE] = v[t].to(dtype)
    return pages


def plain_attention(q, k, v, scale, cap, sinks, first_query):
    """q [Tq, H, hd] at positions first_query.., k / v [Tk, G, hd]: the plain capped softmax with a sink per head."""
    Tq, H, hd = q.shape
    G = k.shape[1]
    out = torch.zeros(Tq, H, v.shape[2], dtype=torch.float64)
    qpos = torch.arange(first_query, first_query + Tq)
    seen = torch.arange(k.shape[0])[None, :] <= qpos[:, None]
    for h in range(H):
        g = h // (H // G)
        s = P.capped_scores(q[:, h], k[:, g], scale, cap).masked_fill(~seen, -math.inf)
        out[:, h] = P.softmax_with_sink(s, sinks[h]) @ v[:, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,length,new", [(4, 2, 48, 200, 200), (8, 1, 64, 321, 321), (2, 2, 128, 150, 57), (6, 2, 96, 700, 700),
                                               (3, 3, 16, 65, 2)])
def test_prompt_attention_with_cap_and_sink(dtype, H, G, hd, length, new):
    """The last ``new`` tokens of a sequence of ``length`` attend over all of it (pages in a scrambled order): the
    plain kernel in float32, the tensor-core prompt kernel in bfloat16. Scores reach well beyond the cap."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(length + hd)
    scale, cap = 0.9, 2.0
    q = torch.randn(new, H, hd).to(dtype)
    k, v = torch.randn(length, G, hd).to(dtype), torch.randn(length, G, hd).to(dtype)
    sinks = (2.0 * torch.randn(H)).cuda()
    rows = list(torch.randperm(16).tolist())[:-(-length // PAGE)]
    pages = fill_pages(k, v, rows, 16, dtype)
    ref = plain_attention(q.double(), k.double(), v.double(), scale, cap, sinks.double().cpu(), length - new)
    qd = q.reshape(new, H * hd).cuda()
    out = torch.empty_like(qd)
    table = i32([rows + [0] * (16 - len(rows))])
    if dtype == torch.float32:
        ops.attention_plain(qd, out, pages, table, i32([0] * new), i32(list(range(length - new, length))), num_heads=H,
                            num_kv_heads=G, head_dim=hd, scale=scale, window=None, softcap=cap, sinks=sinks)
        lim = 3e-6
    else:
        ops.attention_prefill(qd, out, pages, table, i32([0, new]), i32([length]), new, num_heads=H, num_kv_heads=G,
                              head_dim=hd, scale=scale, window=None, softcap=cap, sinks=sinks)
        lim = 1.5e-2
    check_error(f"capped attention over a prompt, {dtype}", f"{H}/{G} x {hd}, {new} of {length}", rel(out.view(new, H, hd), ref), lim)
    if dtype == torch.bfloat16:
        # the weights at float32 precision (a bfloat16 value plus a bfloat16 rest): what is left is the output's rounding
        fine = torch.empty_like(qd)
        ops.attention_prefill(qd, fine, pages, table, i32([0, new]), i32([length]), new, num_heads=H, num_kv_heads=G,
                              head_dim=hd, scale=scale, window=None, softcap=cap, sinks=sinks, exact_weights=True)
        check_error("capped attention over a prompt, bfloat16, float32 weights", f"{H}/{G} x {hd}, {new} of {length}",
                    rel(fine.view(new, H, hd), ref), 6e-3)
    # without the sink and the cap the result differs visibly: both take part
    for kw in (dict(softcap=cap, sinks=None), dict(softcap=None, sinks=sinks)):
        other = torch.empty_like(qd)
        if dtype == torch.float32:
            ops.attention_plain(qd, other, pages, table, i32([0] * new), i32(list(range(length - new, length))), num_heads=H,
                                num_kv_heads=G, head_dim=hd, scale=scale, window=None, **kw)
        else:
            ops.attention_prefill(qd, other, pages, table, i32([0, new]), i32([length]), new, num_heads=H, num_kv_heads=G,
                                  head_dim=hd, scale=scale, window=None, **kw)
        assert rel(other.view(new, H, hd), ref) > 2e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 3, 63, 64, 127, 128, 500, 698, 699])
def test_decode_attention_finds_a_far_key(dtype, far):
    """One new token over 700 cached keys, two sequences in the batch (the other short): key ``far`` is made to
    stand out for head 1 (its capped score exceeds all others by the cap's width), so its value must come through;
    head 0's sink is large enough to take most of its weight (its output shrinks accordingly)."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(far)
    H, G, hd, length = 4, 2, 64, 700
    scale, cap = 0.5, 6.0
    k, v = 0.3 * torch.randn(length, G, hd), torch.randn(length, G, hd)
    q = 0.3 * torch.randn(1, H, hd)
    direction = torch.randn(hd)
    direction /= direction.norm()
    q[0, 1] = 8.0 * direction
    k[far, 0] = 8.0 * direction                            # raw score 64 * 0.5 = 32, capped to ~6; the others stay near 0
    k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
    sinks = torch.tensor([9.0, -3.0, 0.5, 0.0]).cuda()
    short_len = 5
    ks, vs = torch.randn(short_len, G, hd).to(dtype), torch.randn(short_len, G, hd).to(dtype)
    qs = torch.randn(1, H, hd).to(dtype)
    rows_a, rows_b = [11, 2, 7, 0, 5, 9, 3, 1, 14, 6, 12], [4]
    pages = fill_pages(k, v, rows_a, 16, dtype)
    pages += fill_pages(ks, vs, rows_b, 16, dtype)
    table = i32([rows_a + [0] * 5, rows_b + [0] * 15])
    qd = torch.cat([q, qs]).reshape(2, H * hd).cuda()
    out = torch.empty_like(qd)
    if dtype == torch.float32:
        ops.attention_plain(qd, out, pages, table, i32([0, 1]), i32([length - 1, short_len - 1]), num_heads=H, num_kv_heads=G,
                            head_dim=hd, scale=scale, window=None, softcap=cap, sinks=sinks)
        lim = 3e-6
    else:
        ops.attention_decode(qd, out, pages, table, i32([length, short_len]), lambda n, s, d: torch.empty(s, dtype=d, device="cuda"),
                             num_heads=H, num_kv_heads=G, head_dim=hd, scale=scale, window=None, softcap=cap, sinks=sinks)
        lim = 1.5e-2
    ref_a = plain_attention(q.double(), k.double(), v.double(), scale, cap, sinks.double().cpu(), length - 1)
    ref_b = plain_attention(qs.double(), ks.double(), vs.double(), scale, cap, sinks.double().cpu(), short_len - 1)
    got = out.view(2, H, hd)
    check_error(f"capped decode attention, {dtype}", f"far key {far}", rel(got[0], ref_a[0]), lim)
    check_error(f"capped decode attention, {dtype}", "short neighbour", rel(got[1], ref_b[0]), lim)
    # the far key holds a good share of head 1's weight, and the sink most of head 0's
    weight = math.exp(cap) / (math.exp(cap) + length + math.exp(-3.0))
    assert float((got[0, 1].double().cpu() - weight * v[far, 0].double()).abs().max()) < 0.6
    assert float(got[0, 0].abs().max()) < 0.3 * float(ref_a[0, 2].abs().max()) + 0.02


@pytest.mark.parametrize("shares", [(1, 16), (4, 4), (8, 2)])
def test_decode_attention_in_shares(shares):
    """The same decode step cut into 1, 4 and 8 shares of pages: the sink is counted once, whatever the cut."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(5)
    H, G, hd, length = 6, 2, 96, 1000
    num, per = shares
    k, v = torch.randn(length, G, hd).bfloat16(), torch.randn(length, G, hd).bfloat16()
    q = torch.randn(1, H, hd).bfloat16()
    sinks = torch.tensor([4.0, 2.0, 0.0, -1.0, 6.0, 3.0]).cuda()
    rows = torch.randperm(16).tolist()
    pages = fill_pages(k, v, rows, 16, torch.bfloat16)
    qd = q.reshape(1, H * hd).cuda()
    out = torch.empty_like(qd)
    ops.attention_decode(qd, out, pages, i32([rows]), i32([length]), lambda n, s, d: torch.empty(s, dtype=d, device="cuda"),
                         num_heads=H, num_kv_heads=G, head_dim=hd, scale=0.2, window=None, softcap=10.0, sinks=sinks,
                         pages_per_split=per, num_splits=num)
    ref = plain_attention(q.double(), k.double(), v.double(), 0.2, 10.0, sinks.double().cpu(), length - 1)
    check_error("capped decode attention, bfloat16", f"{num} shares", rel(out.view(1, H, hd), ref), 1.5e-2)
    ops.attention_decode(qd, out, pages, i32([rows]), i32([length]), lambda n, s, d: torch.empty(s, dtype=d, device="cuda"),
                         num_heads=H, num_kv_heads=G, head_dim=hd, scale=0.2, window=None, softcap=10.0, sinks=sinks,
                         pages_per_split=per, num_splits=num, exact_weights=True)
    check_error("capped decode attention, bfloat16, float32 weights", f"{num} shares", rel(out.view(1, H, hd), ref), 6e-3)


# --------------------------------------------------------------------------- matrix memory
def memory_weights(H, dk, dv, d, seed):
    g = torch.Generator().manual_seed(seed)
    w = {n: 0.3 * torch.randn(rows, d, generator=g, dtype=torch.float64)
         for n, rows in (("q", H * dk), ("k", H * dk), ("v", H * dv), ("g", H * dv), ("i", H), ("f", H))}
    w["i.b"] = torch.randn(H, generator=g, dtype=torch.float64)
    w["f.b"] = 2.0 + 2.0 * torch.randn(H, generator=g, dtype=torch.float64)
    w["norm"] = 1 + 0.2 * torch.randn(H * dv, generator=g, dtype=torch.float64)
    w["o"] = 0.3 * torch.randn(d, H * dv, generator=g, dtype=torch.float64)
    return w


def run_memory_kernels(h, w, H, dk, dv, cap, eps, state, maxima, slots, q_start, max_new):
    """The three kernels of the mixer on the float32 projection of ``h`` (formed here in float64, so that only the
    recurrence is under test); returns the normed, gated heads [T, H * dv] before the output projection."""
    from llmplayer_b200.kernels import ops
    T = h.shape[0]
    stacked = torch.cat([w[n] for n in ("q", "k", "v", "g", "i", "f")])
    proj = (h @ stacked.T).float().cuda().contiguous()
    gates = torch.empty(3, T, H, device="cuda")
    i_off = 2 * H * dk + 2 * H * dv
    ops.exp_gates(proj, i_off, i_off + H, w["i.b"].float().cuda(), w["f.b"].float().cuda(), cap, maxima, i32(slots), i32(q_start),
                  gates[0], gates[1], gates[2])
    raw = torch.empty(T, H * (dv + 1), device="cuda")
    ops.gla_scan(proj, 0, H * dk, 2 * H * dk, gates[0], state, i32(slots), i32(q_start), raw, num_heads=H, key_dim=dk,
                 value_dim=dv + 1, q_scale=dk ** -0.5, max_new=max_new, scratch=lambda n, s, d: torch.empty(s, dtype=d, device="cuda"),
                 decay_per_head=True, key_gain=gates[1], ones_column=True)
    out = torch.empty(T, H * dv, device="cuda")
    g_off = 2 * H * dk + H * dv
    ops.gla_finish(raw, w["norm"].float().cuda(), eps, proj[:, g_off:g_off + H * dv], out, num_heads=H, value_dim=dv,
                   gain_per_head=True, gate_sigmoid=True, max_row=gates[2])
    return out


@pytest.mark.parametrize("H,dk,dv,cap", [(3, 10, 28, 6.0), (1, 36, 20, 15.0), (2, 64, 128, 10.0), (2, 6, 70, 4.0)])
def test_matrix_memory_over_steps_and_slots(H, dk, dv, cap):
    """Two sequences in slots 2 and 0 of four: a prompt each (one of 300 tokens: chunks side by side), then portions
    and single tokens; every output against the plain recurrence over the whole sequence; the untouched slots stay
    zero; the state ends as the plain one does."""
    d, eps = 40, 1e-5
    w = memory_weights(H, dk, dv, d, seed=H * dk)
    m = {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}
    wp = {"mix." + n: t for n, t in w.items()}
    torch.manual_seed(dk)
    seq = [torch.randn(420, d, dtype=torch.float64), torch.randn(60, d, dtype=torch.float64)]
    full = [P.matrix_memory(s, wp, "mix.", m, eps) for s in seq]
    state = torch.zeros(4, H, dv + 1, dk, device="cuda")
    maxima = torch.zeros(4, H, device="cuda")
    slots = [2, 0]
    cuts = [(300, 7), (2, 1), (117, 51), (1, 1)]           # new tokens of the two sequences, step by step
    at = [0, 0]
    got = [[], []]
    for a, b in cuts:
        h = torch.cat([seq[0][at[0]:at[0] + a], seq[1][at[1]:at[1] + b]])
        out = run_memory_kernels(h, w, H, dk, dv, cap, eps, state, maxima, slots, [0, a, a + b], max(a, b))
        got[0].append(out[:a])
        got[1].append(out[a:])
        at = [at[0] + a, at[1] + b]
    for s in range(2):
        heads = torch.cat(got[s]).double().cpu() @ w["o"].T
        check_error("matrix memory, float32", f"{H} x {dk} x {dv}, sequence {s}", rel(heads, full[s][0]), 2e-5)
    assert float(state[1].abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0 and float(maxima[[1, 3]].abs().max()) == 0.0
    S, n, big = full[0][1]
    kept = state[2].double().cpu()                          # [H, dv + 1, dk]: value columns, then the normaliser
    assert rel(kept[:, :dv].transpose(1, 2), S) < 2e-5 and rel(kept[:, dv], n) < 2e-5 and rel(maxima[2], big) < 1e-6


def test_matrix_memory_remembers_an_early_token():
    """Forget gates held open (a large positive bias) and a single early token with a large input gate: its value
    must still dominate 400 tokens later, through the chunks of a long prompt; and with m starting at 0, not below,
    the very first outputs are scaled by exp(-m) = 1."""
    H, dk, dv, d, cap, eps = 1, 16, 8, 12, 20.0, 1e-6
    w = memory_weights(H, dk, dv, d, seed=9)
    w["f"] = torch.zeros_like(w["f"])
    w["i"] = torch.zeros_like(w["i"])
    w["f.b"] = torch.full((H,), 12.0, dtype=torch.float64)
    w["i.b"] = torch.full((H,), -6.0, dtype=torch.float64)
    torch.manual_seed(1)
    x = 0.5 * torch.randn(402, d, dtype=torch.float64)
    w["i"][0] = x[2] / (x[2] @ x[2]) * 14.0                 # token 2 alone gets a log input gate of about +8
    m = {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}
    ref, _ = P.matrix_memory(x, {"mix." + n: t for n, t in w.items()}, "mix.", m, eps)
    state, maxima = torch.zeros(1, H, dv + 1, dk, device="cuda"), torch.zeros(1, H, device="cuda")
    out = run_memory_kernels(x, w, H, dk, dv, cap, eps, state, maxima, [0], [0, 402], 402)
    check_error("matrix memory, float32", "an early token through 400 steps", rel(out.double().cpu() @ w["o"].T, ref), 5e-5)
    assert float(maxima[0, 0]) > 5.0


# --------------------------------------------------------------------------- routing
@pytest.mark.parametrize("E,groups,keep,top", [(6, 3, 2, 2), (4, 4, 4, 1), (8, 2, 1, 3), (4, 2, 1, 1), (16, 4, 2, 5), (64, 8, 3, 6), (2, 1, 1, 2)])
def test_routing_against_plain(E, groups, keep, top):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(E + top)
    T = 300
    wide = (2.0 * torch.randn(T, E + 5)).cuda()
    logits = wide[:, 3:3 + E]
    weights = torch.full((T, E), 9.0, device="cuda")
    ops.route(logits, weights, groups=groups, keep=keep, top=top)
    scores = torch.sigmoid(logits.double().cpu())
    chosen, w, gap = P.route(scores, groups, keep, top)
    ref = torch.zeros(T, E, dtype=torch.float64).scatter_(1, chosen, w)
    clear = torch.ones(T, dtype=torch.bool)
    if gap < 1e-6:                                         # leave out the rows where float32 and float64 may order differently
        for t in range(T):
            clear[t] = P.route(scores[t:t + 1], groups, keep, top)[2] > 1e-6
    assert int(clear.sum()) > T - 5
    assert rel(weights[clear.cuda()], ref[clear]) < 2e-6
    assert int((weights > 0).sum(-1).min()) == int((weights > 0).sum(-1).max()) == top
    assert float((weights.sum(-1) - 1).abs().max()) < 1e-5


def test_expert_scale_leaves_the_shared_columns():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(2)
    T, E, ff, shared = 9, 5, 12, 20
    weights = torch.rand(T, E).cuda() * (torch.rand(T, E).cuda() > 0.5)
    for dtype, lim in ((torch.float32, 1e-6), (torch.bfloat16, 8e-3)):
        hidden = torch.randn(T, E * ff + shared).to(dtype).cuda()
        ref = hidden.double().cpu().clone()
        ref[:, :E * ff] *= weights.double().cpu().repeat_interleave(ff, dim=1)
        ops.expert_scale(hidden, weights, ff)
        assert rel(hidden, ref) < lim
        assert torch.equal(hidden[:, E * ff:].double().cpu(), ref[:, E * ff:])

"""Each new mechanism alone, its kernels against the plain implementation's function of the same name:
layer norm, xIELU, the gated residual sum with the weighted sum over depth, latent attention (prompts, decoding
over several shares of keys, a far key that dominates, keys at the borders of pages and key blocks), gated linear
attention (state carried over steps and slots, a slow-decaying channel that remembers an early token)."""
import math

import pytest
import torch

import plain_ramupel as P
from helpers import check_error

pytestmark = pytest.mark.gpu


def rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all()
    return float((got - ref).abs().max() / ref.abs().max())


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# --------------------------------------------------------------------------- small kernels
@pytest.mark.parametrize("rows,d", [(1, 8), (5, 88), (3, 1000), (2, 4100)])
def test_layer_norm(rows, d):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(d)
    x = (torch.randn(rows, d) * 3 + 1.5).cuda()
    gain = (1 + 0.2 * torch.randn(d)).cuda()
    out = torch.empty(rows, d, device="cuda")
    ops.layernorm(x, gain, 1e-5, out)
    check_error("layer norm, float32", f"{rows}x{d}", rel(out, P.layer_norm(x.double().cpu(), gain.double().cpu(), 1e-5)), 2e-6)
    picked = i32([rows - 1, 0])
    out2 = torch.empty(2, d, device="cuda", dtype=torch.bfloat16)
    ops.layernorm(x, gain, 1e-5, out2, rows=picked)
    ref = P.layer_norm(x.double().cpu(), gain.double().cpu(), 1e-5)[[rows - 1, 0]]
    check_error("layer norm, bfloat16 out", f"{rows}x{d}", rel(out2, ref), 5e-3)


def test_xielu_on_a_slice():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(0)
    wide = (torch.randn(7, 50) * 4).cuda()
    wide[0, 10] = 0.0
    pq = torch.tensor([0.3, -1.2], device="cuda")
    out = torch.empty(7, 33, device="cuda")
    ops.xielu(wide[:, 10:43], pq, out)
    ref = P.xielu(wide[:, 10:43].double().cpu(), pq[0].double().cpu(), pq[1].double().cpu())
    check_error("xIELU, float32", "7x33 slice", rel(out, ref), 2e-6)


@pytest.mark.parametrize("with_ffn", [True, False])
def test_gated_sum_and_depth_mix(with_ffn):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(1)
    T, d, total = 6, 40, 5
    streams = torch.zeros(total, T, d, device="cuda")
    x0 = torch.randn(T, d).cuda()
    x = x0.clone()
    kept = [x0.double().cpu()]
    for layer in range(total - 1):
        a, b = torch.randn(T, d).cuda(), torch.randn(T, d).cuda()
        logits = torch.randn(T, 3 * d).cuda()
        ba, bb = torch.randn(d).cuda(), torch.randn(d).cuda()
        mix = torch.randn(layer + 2).cuda()
        before = x.double().cpu()
        ops.gated_sum(x, a, (logits[:, :d], ba), b if with_ffn else None, (logits[:, 2 * d:], bb) if with_ffn else None,
                      streams=streams, mix=mix, count=layer + 2, keep_input=layer == 0)
        y = before + a.double().cpu() * torch.sigmoid(logits[:, :d].double().cpu() + ba.double().cpu())
        if with_ffn:
            y = y + b.double().cpu() * torch.sigmoid(logits[:, 2 * d:].double().cpu() + bb.double().cpu())
        kept.append(y)
        ref = sum(mix[j].double().cpu() * kept[j] for j in range(layer + 2))
        check_error("gated sum + depth mix, float32", f"layer {layer}", rel(x, ref), 3e-6)
    plain = x0.clone()
    ops.gated_sum(plain, a)
    assert rel(plain, x0.double().cpu() + a.double().cpu()) < 1e-6


# --------------------------------------------------------------------------- latent attention
def run_latent(m, w, q, down, gate, lengths_before, new_counts, kv_dtype, pages=None, table=None, shares=None):
    """One step of the kernels for sequences with ``new_counts`` new tokens after ``lengths_before`` cached ones.
    ``q, down, gate``: the projections of the step's tokens, packed sequence after sequence."""
    from llmplayer_b200.kernels import ops
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = sum(new_counts)
    B = len(new_counts)
    proj = torch.cat([q.reshape(T, -1), down, gate], dim=1).float().cuda().contiguous()
    positions, seq_ids, q_start = [], [], [0]
    for b, (have, n) in enumerate(zip(lengths_before, new_counts)):
        positions += list(range(have, have + n))
        seq_ids += [b] * n
        q_start.append(q_start[-1] + n)
    kv_len = [h + n for h, n in zip(lengths_before, new_counts)]
    half = m["rot"]["dims"] // 2
    inv = torch.tensor([m["rot"]["base"] ** (-2.0 * i / m["rot"]["dims"]) for i in range(half)], dtype=torch.float64)
    rotation = ops.Rotation(inv.float().cuda(), m["rot"]["dims"], False) if half else ops.NO_ROTATION
    q_out = torch.empty(T, H, dn + dr, device="cuda")
    ops.latent_prepare(proj, 0, H * (dn + dr), w["dkv.norm"].float().cuda(), 1e-5, rotation, i32(positions), i32(seq_ids),
                       table, q_out, pages, num_heads=H, nope_dim=dn, rope_dim=dr, kv_rank=rank)
    wt = torch.bfloat16 if kv_dtype == torch.bfloat16 else torch.float32
    q_abs = torch.empty(T, H, rank + dr, device="cuda")
    ops.latent_absorb(q_out, w["uk"].to(wt).cuda(), q_abs, nope_dim=dn, rope_dim=dr)
    if shares is None:
        shares = ops.latent_shares(B, max(new_counts), H, table.shape[1], 64)
    part = torch.empty(T, H, shares, rank + 2, device="cuda")
    ops.latent_attend(q_abs, pages, table, i32(q_start), i32(kv_len), part, max_new=max(new_counts), kv_rank=rank,
                      scale=m["scale"])
    out = torch.empty(T, H * dv, device="cuda", dtype=torch.float32)
    g_off = H * (dn + dr) + rank + dr
    ops.latent_expand(part, w["uv"].to(wt).cuda(), proj[:, g_off:g_off + H], out, value_dim=dv)
    return out, shares


def latent_weights(m, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    H, dn, dv, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    w = {"dkv.norm": 1 + 0.2 * torch.randn(rank, generator=g), "uk": 0.3 * torch.randn(H * dn, rank, generator=g),
         "uv": 0.3 * torch.randn(H * dv, rank, generator=g)}
    if dtype == torch.bfloat16:
        w = {k: v.bfloat16().float() for k, v in w.items()}
    return w


LATENT_SHAPES = [
    {"heads": 3, "dim": 24, "rot_dim": 12, "vdim": 20, "kv_rank": 40, "scale": 0.2, "rot": {"base": 10000.0, "dims": 8}},
    {"heads": 1, "dim": 16, "rot_dim": 4, "vdim": 48, "kv_rank": 72, "scale": 0.25, "rot": {"base": 500.0, "dims": 4}},
    {"heads": 40, "dim": 8, "rot_dim": 8, "vdim": 8, "kv_rank": 24, "scale": 0.3, "rot": {"base": 10000.0, "dims": 8}},
    {"heads": 5, "dim": 32, "rot_dim": 16, "vdim": 24, "kv_rank": 300, "scale": 0.15, "rot": {"base": 1e6, "dims": 16}},
]


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", LATENT_SHAPES, ids=lambda m: f"H{m['heads']}r{m['kv_rank']}")
def test_latent_attention_prompts_then_decoding(m, kv_dtype):
    """Two sequences (lengths 150 and 67) as prompts in one step, then both continued by one token, through pages
    in a scrambled order; the decode step cuts its keys into several shares."""
    torch.manual_seed(m["heads"])
    H, dn, dr, rank = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    w = latent_weights(m, 3, kv_dtype)
    lengths = [150, 67]
    qs = [torch.randn(n + 1, H, dn + dr, dtype=torch.float64) for n in lengths]
    downs = [torch.randn(n + 1, rank + dr, dtype=torch.float64) * 2 for n in lengths]
    gates = [torch.randn(n + 1, H, dtype=torch.float64) for n in lengths]
    wd = {"x." + k: v.double() for k, v in w.items()}
    refs = [P.latent_attention_core(q, d, g, wd, "x.", m, 1e-5)[0] for q, d, g in zip(qs, downs, gates)]
    pages = torch.zeros(9, 64, rank + dr, device="cuda", dtype=kv_dtype)
    table = i32([[7, 2, 5, 0, 0, 0, 0, 0], [1, 8, 0, 0, 0, 0, 0, 0]])
    out, _ = run_latent(m, w, torch.cat([q[:-1] for q in qs]), torch.cat([d[:-1] for d in downs]),
                        torch.cat([g[:-1] for g in gates]), [0, 0], lengths, kv_dtype, pages, table)
    tol = 3e-5 if kv_dtype == torch.float32 else 2e-2
    kind = f"latent attention, {'float32' if kv_dtype == torch.float32 else 'bfloat16 cache'}"
    check_error(kind, f"prompts H{H}", rel(out, torch.cat([r[:-1] for r in refs])), tol)
    out, shares = run_latent(m, w, torch.cat([q[-1:] for q in qs]), torch.cat([d[-1:] for d in downs]),
                             torch.cat([g[-1:] for g in gates]), lengths, [1, 1], kv_dtype, pages, table)
    assert shares == 16                      # shares of one block of 32 keys; most of the second sequence's are empty
    check_error(kind, f"decode H{H}", rel(out, torch.cat([r[-1:] for r in refs])), tol)


@pytest.mark.parametrize("target", [3, 31, 32, 63, 64, 127, 128, 500, 699])
def test_latent_attention_finds_one_key_among_hundreds(target):
    """A sequence of 700 positions whose last query is aligned with the rotated key part of ONE position (far back,
    or at the border of a page or of a block of 32 keys): nearly all weight lies there, so a kernel that skipped
    or misplaced that row would miss the whole output. In one step as a prompt, and as a decode step in shares."""
    m = LATENT_SHAPES[0]
    H, dn, dr, rank = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    w = latent_weights(m, 5, torch.float32)
    g = torch.Generator().manual_seed(target)
    n = 700
    q = 0.1 * torch.randn(n, H, dn + dr, generator=g, dtype=torch.float64)
    down = torch.randn(n, rank + dr, generator=g, dtype=torch.float64)
    down[:, rank:] *= 0.1
    gate = torch.randn(n, H, generator=g, dtype=torch.float64)
    # the shared rotated key part is not normed: make the target's large, and turn the last query so that, after
    # both rotations, it points along it
    u = 3.0 * torch.randn(1, dr, generator=g, dtype=torch.float64)
    down[target, rank:] = u[0]
    there = P.rotate_half_pairs(u, torch.tensor([target]), m["rot"]["base"], m["rot"]["dims"])
    back = P.rotate_half_pairs(there, torch.tensor([-(n - 1)]), m["rot"]["base"], m["rot"]["dims"])
    q[-1, :, dn:] = back * (40.0 / (m["scale"] * float((u * u).sum())))
    wd = {"x." + k: v.double() for k, v in w.items()}
    ref, weights = P.latent_attention_core(q, down, gate, wd, "x.", m, 1e-5)
    assert float(weights[:, -1, target].min()) > 0.99
    pages = torch.zeros(16, 64, rank + dr, device="cuda")
    table = i32([[11, 3, 9, 0, 14, 6, 1, 12, 5, 8, 2, 0, 0, 0, 0, 0]])
    out, _ = run_latent(m, w, q, down, gate, [0], [n], torch.float32, pages, table)
    check_error("latent attention, one key stands out", f"prompt, key {target}", rel(out[-1], ref[-1]), 3e-5)
    pages2 = torch.zeros(16, 64, rank + dr, device="cuda")
    run_latent(m, w, q[:-1], down[:-1], gate[:-1], [0], [n - 1], torch.float32, pages2, table)
    out, shares = run_latent(m, w, q[-1:], down[-1:], gate[-1:], [n - 1], [1], torch.float32, pages2, table)
    assert shares == 32
    check_error("latent attention, one key stands out", f"decode, key {target}", rel(out[0], ref[-1]), 3e-5)


# --------------------------------------------------------------------------- gated linear attention
def run_gla(H, dk, dv, q, k, v, z_low, up, bias, gate, gain, tau, state, slots, counts, chunked=False):
    from llmplayer_b200.kernels import ops
    T = q.shape[0]
    R = z_low.shape[1]
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gate, z_low], dim=1).float().cuda().contiguous()
    decay = torch.empty(T, H * dk, device="cuda")
    a_off = 2 * H * dk + 2 * H * dv
    ops.gla_decay(proj[:, a_off:a_off + R], up.float().cuda(), bias.float().cuda(), decay, tau)
    q_start = [0]
    for n in counts:
        q_start.append(q_start[-1] + n)
    raw = torch.empty(T, H * dv, device="cuda")
    kept = {}

    def scratch(name, shape, dtype):
        kept[name] = torch.full(shape, float("nan"), dtype=dtype, device="cuda")      # nothing may be read before it is written
        return kept[name]
    ops.gla_scan(proj, 0, H * dk, 2 * H * dk, decay, state, i32(slots), i32(q_start), raw, num_heads=H, key_dim=dk,
                 value_dim=dv, q_scale=dk ** -0.5, max_new=max(counts) if chunked else 0, scratch=scratch if chunked else None)
    assert bool(kept) == (chunked and max(counts) >= ops.GLA_CHUNKED_FROM)
    out = torch.empty(T, H * dv, device="cuda")
    ops.gla_finish(raw, gain.float().cuda(), 1e-5, proj[:, 2 * H * dk + H * dv:a_off], out, num_heads=H, value_dim=dv)
    return out, decay


@pytest.mark.parametrize("H,dk,dv,R", [(2, 20, 36, 5), (3, 6, 70, 24), (1, 64, 128, 8), (4, 130, 16, 1), (2, 48, 200, 16)])
def test_gated_linear_attention_over_steps_and_slots(H, dk, dv, R):
    """Two sequences (37 and 9 tokens) in one step, then continued by 1 and 20 tokens in a second step, their
    states in rows 4 and 1 of the state area; outputs and final states against the plain recurrence."""
    g = torch.Generator().manual_seed(H * dk + dv)
    tau = 4.0
    first, second = [37, 9], [1, 20]
    total = [a + b for a, b in zip(first, second)]

    def draw(*shape, scale=1.0):
        return scale * torch.randn(*shape, generator=g, dtype=torch.float64)
    seqs = []
    up, bias, gain = draw(H * dk, R, scale=0.6), 2 + 2 * draw(H * dk), 1 + 0.2 * draw(dv)
    for n in total:
        seqs.append({"q": draw(n, H, dk), "k": draw(n, H, dk), "v": draw(n, H, dv), "low": draw(n, R), "gate": draw(n, H * dv)})
    refs = []
    for s in seqs:
        a = (torch.sigmoid(s["low"] @ up.T + bias) ** (1 / tau)).reshape(-1, H, dk)
        refs.append(P.gla_core(s["q"] * dk ** -0.5, s["k"], s["v"], a, s["gate"], gain, 1e-5))
    state = torch.full((6, H, dv, dk), 7.0, device="cuda")         # the kernels keep it [head, value column, key channel]
    state[4].zero_()
    state[1].zero_()

    def step(lo, counts):
        pick = lambda key: torch.cat([s[key][a:a + n] for s, a, n in zip(seqs, lo, counts)])
        return run_gla(H, dk, dv, pick("q"), pick("k"), pick("v"), pick("low"), up, bias, pick("gate"), gain, tau, state,
                       [4, 1], counts)[0]
    out1 = step([0, 0], first)
    out2 = step(first, second)
    want1 = torch.cat([r[0][:n] for r, n in zip(refs, first)])
    want2 = torch.cat([r[0][n:] for r, n in zip(refs, first)])
    check_error("gated linear attention, float32", f"H{H} dk{dk} dv{dv} first step", rel(out1, want1), 3e-5)
    check_error("gated linear attention, float32", f"H{H} dk{dk} dv{dv} second step", rel(out2, want2), 3e-5)
    check_error("gated linear attention, float32", "final state", rel(state[4].transpose(1, 2), refs[0][1]), 3e-5)
    check_error("gated linear attention, float32", "final state", rel(state[1].transpose(1, 2), refs[1][1]), 3e-5)
    assert float((state[0] - 7.0).abs().max()) == 0.0 and float((state[5] - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("H,dk,dv", [(2, 20, 36), (1, 64, 80)])
def test_gated_linear_attention_in_chunks_side_by_side(H, dk, dv):
    """Long prompts (700, 300 and 5 tokens, so sequences with six, three and one chunk in one launch) whose chunks run
    side by side, continuing states that are not zero; outputs and final states against the plain recurrence."""
    g = torch.Generator().manual_seed(dk)
    R, tau, counts = 4, 6.0, [700, 300, 5]

    def draw(*shape, scale=1.0):
        return scale * torch.randn(*shape, generator=g, dtype=torch.float64)
    up, bias, gain = draw(H * dk, R, scale=0.6), 2.5 + 2 * draw(H * dk), 1 + 0.2 * draw(dv)
    start = [draw(H, dk, dv) for _ in counts]
    seqs = [{"q": draw(n, H, dk), "k": draw(n, H, dk), "v": draw(n, H, dv), "low": draw(n, R), "gate": draw(n, H * dv)}
            for n in counts]
    refs = []
    for s0, s in zip(start, seqs):
        a = (torch.sigmoid(s["low"] @ up.T + bias) ** (1 / tau)).reshape(-1, H, dk)
        refs.append(P.gla_core(s["q"] * dk ** -0.5, s["k"], s["v"], a, s["gate"], gain, 1e-5, state=s0))
    state = torch.zeros(4, H, dv, dk, device="cuda")
    slots = [2, 0, 3]
    for slot, s0 in zip(slots, start):
        state[slot] = s0.transpose(1, 2).float().cuda()
    pick = lambda key: torch.cat([s[key] for s in seqs])
    out, _ = run_gla(H, dk, dv, pick("q"), pick("k"), pick("v"), pick("low"), up, bias, pick("gate"), gain, tau, state, slots,
                     counts, chunked=True)
    check_error("gated linear attention, chunks side by side", f"H{H} dk{dk} outputs", rel(out, torch.cat([r[0] for r in refs])), 3e-5)
    for slot, r in zip(slots, refs):
        check_error("gated linear attention, chunks side by side", "final state", rel(state[slot].transpose(1, 2), r[1]), 3e-5)


def test_gated_linear_attention_remembers_an_early_token():
    """One key channel barely decays (a large bias) and carries token 2's value to token 400, whose query reads only
    that channel; every other channel forgets fast. The output at the end is token 2's value, rescaled."""
    H, dk, dv, R, n, tau = 1, 8, 16, 3, 401, 2.0
    g = torch.Generator().manual_seed(9)
    q = torch.zeros(n, H, dk, dtype=torch.float64)
    k = 0.05 * torch.randn(n, H, dk, generator=g, dtype=torch.float64)
    k[:, :, 5] = 0.0
    v = torch.randn(n, H, dv, generator=g, dtype=torch.float64)
    k[2, 0, 5] = 4.0
    q[-1, 0, 5] = 1.0
    low = torch.randn(n, R, generator=g, dtype=torch.float64)
    up = torch.zeros(H * dk, R, dtype=torch.float64)
    bias = torch.full((H * dk,), -3.0, dtype=torch.float64)
    bias[5] = 12.0
    gate, gain = torch.ones(n, H * dv, dtype=torch.float64), torch.ones(dv, dtype=torch.float64)
    a = (torch.sigmoid(low @ up.T + bias) ** (1 / tau)).reshape(n, H, dk)
    ref, _ = P.gla_core(q * dk ** -0.5, k, v, a, gate, gain, 1e-5)
    direction = torch.nn.functional.cosine_similarity(ref[-1], v[2, 0], dim=0)
    assert float(direction) > 0.999
    state = torch.zeros(2, H, dv, dk, device="cuda")
    out, _ = run_gla(H, dk, dv, q, k, v, low, up, bias, gate, gain, tau, state, [1], [n])
    check_error("gated linear attention, float32", "early token remembered", rel(out[-1], ref[-1]), 3e-5)
